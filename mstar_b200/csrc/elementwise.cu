// Memory-bound kernels of the decoder: embedding gather, fused residual-add +
// RMSNorm, rotary position encoding fused with the write of keys and values into
// cache pages, SiLU(gate)*up, row gather, dtype conversion.
//
// Formulas follow the reference model: RMSNorm x*rsqrt(mean(x^2)+eps)*w
// (mstar/model/components/norm.py:45-59, mstar/utils/attention.py:457-474),
// split-half rotary pairs (mstar/utils/attention.py:224-253), down(silu(gate)*up)
// (mstar/model/components/distributed/mlp.py:78-81), plain residual adds
// (mstar/model/components/decoder_layer.py:58-71).  The residual stream is kept in
// float in both dtypes so that the residual sum is a 32-bit sum.
#include <stdlib.h>

#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[t] = float(table[id]) with id = ids[t], or, where `src` is given and src[t] >= 0,
// id = prev[src[t]]: a token that the step before sampled and that is still on the device
// (the engine launches a step before it has read the last one's tokens).
template <typename W>
__global__ void embed_rows_kernel(const W* __restrict__ table, const int* __restrict__ ids,
                                  const int* __restrict__ src, const int* __restrict__ prev,
                                  float* __restrict__ out, int vocab, int hidden, float scale) {
    prev = pdl_after(prev, pdl_wait());       // sampled by the step before
    const int t = blockIdx.x;
    int id = ids[t];
    if (src != nullptr) {
        const int from = src[t];
        if (from >= 0) id = prev[from];
    }
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {  // host validates ids; never read out of the table
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const W* row = table + (size_t)id * hidden;
    if (scale == 1.f)
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
    else
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

// `src` and `prev` are both null or both given (src: [num_tokens] ints, -1 where ids holds
// the token; prev: int tokens on the device).  Rows are multiplied by `scale` in float.
MSTAR_API int mstar_embed_rows(const void* table, int table_dtype, const int* ids, const int* src,
                               const int* prev, float* out, int num_tokens, int vocab, int hidden,
                               float scale, void* stream) {
    if (num_tokens <= 0) return 0;
    if ((src == nullptr) != (prev == nullptr)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == MSTAR_F32)
        mstar_launch((embed_rows_kernel<float>), dim3(num_tokens), dim3(threads), 0, s, (const float*)table, ids,
                     src, prev, out, vocab, hidden, scale);
    else
        mstar_launch((embed_rows_kernel<bf16>), dim3(num_tokens), dim3(threads), 0, s, (const bf16*)table, ids,
                     src, prev, out, vocab, hidden, scale);
    return launch_status();
}

// ------------------------------------------------- residual add + RMSNorm
// resid (float, [rows, hidden]) is updated in place with resid + delta when delta
// is given; out = resid * rsqrt(mean(resid^2) + eps) * (w + w_offset) in type A.
// One block per row.  The sum of squares is accumulated per thread over a fixed
// stride and then reduced in a fixed tree, so a row's result does not depend on
// which other rows are in the batch.  `resid_static`: nonzero promises that the kernel
// before this one on the stream did not write resid (it wrote delta), so resid may be
// read while that kernel is still draining.
template <typename A, typename W, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const A* __restrict__ delta,
                                   const W* __restrict__ weight, A* __restrict__ out, int hidden,
                                   float eps, float w_offset, int resid_static) {
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * hidden;
    float* r = resid + base;
    float ss = 0.f;
    if (VEC) {
        // eight elements per thread and step, 16-byte accesses; the order in which a row's
        // squares are summed depends only on the row's width and the block size
        const int chunks = hidden >> 3;
        if (chunks <= 2 * (int)blockDim.x) {
            // a thread's one or two chunks stay in registers.  The weight is a parameter, and
            // with `resid_static` the kernel before this one wrote the delta only: both are
            // asked for while that kernel is still draining.
            const int c0 = threadIdx.x, c1 = threadIdx.x + blockDim.x;
            const bool h0 = c0 < chunks, h1 = c1 < chunks;
            float v0[8], v1[8], w0[8], w1[8];
            if (h0) load8(weight + 8 * c0, w0);
            if (h1) load8(weight + 8 * c1, w1);
            if (resid_static) {
                if (h0) load8(r + 8 * c0, v0);
                if (h1) load8(r + 8 * c1, v1);
            }
            delta = pdl_after(delta, pdl_wait());
            if (!resid_static) {
                if (h0) load8(r + 8 * c0, v0);
                if (h1) load8(r + 8 * c1, v1);
            }
            if (delta != nullptr) {
                float d[8];
                if (h0) {
                    load8(delta + base + 8 * c0, d);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v0[i] += d[i];
                    store8(r + 8 * c0, v0);
                }
                if (h1) {
                    load8(delta + base + 8 * c1, d);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v1[i] += d[i];
                    store8(r + 8 * c1, v1);
                }
            }
            if (h0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(v0[i], v0[i], ss);
            }
            if (h1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(v1[i], v1[i], ss);
            }
            const float total = block_sum(ss, scratch);
            const float inv = rsqrtf(total / (float)hidden + eps);
            if (h0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v0[i] = v0[i] * inv * (w0[i] + w_offset);
                store8(out + base + 8 * c0, v0);
            }
            if (h1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v1[i] = v1[i] * inv * (w1[i] + w_offset);
                store8(out + base + 8 * c1, v1);
            }
            return;
        }
        delta = pdl_after(delta, pdl_wait());
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            float v[8];
            load8(r + 8 * c, v);
            if (delta != nullptr) {
                float d[8];
                load8(delta + base + 8 * c, d);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += d[i];
                store8(r + 8 * c, v);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
        }
        const float total = block_sum(ss, scratch);
        const float inv = rsqrtf(total / (float)hidden + eps);
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            float v[8], w[8];
            load8(r + 8 * c, v);  // what this thread wrote itself
            load8(weight + 8 * c, w);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * (w[i] + w_offset);
            store8(out + base + 8 * c, v);
        }
        return;
    }
    delta = pdl_after(delta, pdl_wait());
    if (delta != nullptr) {
        const A* d = delta + base;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = r[i] + to_float(d[i]);
            r[i] = v;
            ss = fmaf(v, v, ss);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = r[i];
            ss = fmaf(v, v, ss);
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    A* o = out + base;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        // each thread re-reads only what it wrote itself, so no barrier is needed
        o[i] = from_float<A>(r[i] * inv * (to_float(weight[i]) + w_offset));
    }
}

MSTAR_API int mstar_add_rmsnorm(float* resid, const void* delta, const void* weight,
                                int weight_dtype, void* out, int act_dtype, int rows, int hidden,
                                float eps, float w_offset, int resid_static, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = hidden % 8 == 0 && ((uintptr_t)resid % 32 == 0) && ((uintptr_t)out % 16 == 0) &&
                     ((uintptr_t)weight % 32 == 0) && (delta == nullptr || (uintptr_t)delta % 16 == 0);
    int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (vec) threads = hidden >= 4096 ? 512 : (hidden >= 2048 ? 256 : 128);
    // a thread per 8-element chunk where 512 threads suffice: one load of each kind per thread
    // and a tree that starts at once (a decode step's norm 1.92 -> 1.68 us at width 3072)
    if (vec && hidden / 8 <= 512) threads = ((hidden / 8 + 31) / 32) * 32;
#define LAUNCH(A, W)                                                                             \
    if (vec)                                                                                     \
        mstar_launch((add_rmsnorm_kernel<A, W, true>), dim3(rows), dim3(threads), 0, s,                                  \
            resid, (const A*)delta, (const W*)weight, (A*)out, hidden, eps, w_offset,           \
            resid_static);                                                                       \
    else                                                                                         \
        mstar_launch((add_rmsnorm_kernel<A, W, false>), dim3(rows), dim3(threads), 0, s,                                 \
            resid, (const A*)delta, (const W*)weight, (A*)out, hidden, eps, w_offset, resid_static)
    if (act_dtype == MSTAR_F32) {
        if (weight_dtype == MSTAR_F32) { LAUNCH(float, float); } else { LAUNCH(float, bf16); }
    } else {
        if (weight_dtype == MSTAR_F32) { LAUNCH(bf16, float); } else { LAUNCH(bf16, bf16); }
    }
#undef LAUNCH
    return launch_status();
}

// ------------------------------------------------------ gather (+add) rows
// out[i] = resid[rows[i]] (+ delta[rows[i]]), float.  Used to pick the rows whose
// logits are wanted before the final norm, so norm and LM head run on those only.
template <typename A>
__global__ void gather_add_rows_kernel(const float* __restrict__ resid, const A* __restrict__ delta,
                                       const int* __restrict__ rows, float* __restrict__ out,
                                       int hidden) {
    const unsigned long long waited = pdl_wait();
    resid = pdl_after(resid, waited);
    delta = pdl_after(delta, waited);
    const size_t src = (size_t)rows[blockIdx.x] * hidden;
    const size_t dst = (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = resid[src + i];
        if (delta != nullptr) v += to_float(delta[src + i]);
        out[dst + i] = v;
    }
}

MSTAR_API int mstar_gather_add_rows(const float* resid, const void* delta, int act_dtype,
                                    const int* rows, float* out, int num_rows, int hidden,
                                    void* stream) {
    if (num_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == MSTAR_F32)
        mstar_launch((gather_add_rows_kernel<float>), dim3(num_rows), dim3(256), 0, s, resid, (const float*)delta, rows, out, hidden);
    else
        mstar_launch((gather_add_rows_kernel<bf16>), dim3(num_rows), dim3(256), 0, s, resid, (const bf16*)delta, rows, out, hidden);
    return launch_status();
}

// ------------------------------------------------------------ act(gate)*up
// gate_up: [rows, 2*inter] with gate first (mstar/model/components/distributed/
// mlp.py:78-81); out: [rows, inter].  silu(x) = x / (1 + exp(-x)), or the tanh form of gelu,
// in float.
// kind 0: relu(x)^2, 1: gelu (tanh form), 2: silu.
__device__ __forceinline__ float plain_activation(float v, int kind) {
    if (kind == 0) {
        const float r = fmaxf(v, 0.f);
        return r * r;
    }
    if (kind == 1)
        return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v / (1.f + expf(-v));
}

template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gate_up, A* __restrict__ out, int inter,
                                size_t total, int kind) {
    gate_up = pdl_after(gate_up, pdl_wait());
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t row = idx / inter;
        const int col = (int)(idx - row * inter);
        const A* p = gate_up + row * 2 * (size_t)inter;
        const float g = to_float(p[col]);
        const float u = to_float(p[inter + col]);
        out[idx] = from_float<A>(plain_activation(g, kind) * u);
    }
}

MSTAR_API int mstar_silu_mul(const void* gate_up, void* out, int act_dtype, int rows, int inter,
                             int kind, void* stream) {
    const size_t total = (size_t)rows * inter;
    if (total == 0) return 0;
    if (kind != 1 && kind != 2) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    const size_t most = (size_t)device_sm_count() * 32;   // a grid-stride loop takes the rest
    if (blocks > most) blocks = most;
    if (act_dtype == MSTAR_F32)
        mstar_launch((silu_mul_kernel<float>), dim3((int)blocks), dim3(threads), 0, s, (const float*)gate_up, (float*)out, inter, total, kind);
    else
        mstar_launch((silu_mul_kernel<bf16>), dim3((int)blocks), dim3(threads), 0, s, (const bf16*)gate_up, (bf16*)out, inter, total, kind);
    return launch_status();
}

// out = act(gate + bias_gate) * (up + bias_up) from the float product [rows][2 * inter]
// (gate columns first) and a bias of 2 * inter numbers; float arithmetic, the result in the
// activation type.
template <typename A, typename W>
__global__ void bias_act_mul_kernel(const float* gate_up, const W* __restrict__ bias,
                                    A* __restrict__ out, int inter, size_t total, int kind) {
    gate_up = pdl_after(gate_up, pdl_wait());
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t row = idx / inter;
        const int col = (int)(idx - row * inter);
        const float* p = gate_up + row * 2 * (size_t)inter;
        const float g = p[col] + to_float(bias[col]);
        const float u = p[inter + col] + to_float(bias[inter + col]);
        out[idx] = from_float<A>(plain_activation(g, kind) * u);
    }
}

MSTAR_API int mstar_bias_act_mul(const float* gate_up, const void* bias, int weight_dtype, void* out,
                                 int act_dtype, int rows, int inter, int kind, void* stream) {
    const size_t total = (size_t)rows * inter;
    if (total == 0) return 0;
    if ((kind != 1 && kind != 2) || bias == nullptr) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    const size_t most = (size_t)device_sm_count() * 32;   // a grid-stride loop takes the rest
    if (blocks > most) blocks = most;
#define GO(A, W)                                                                                  \
    mstar_launch((bias_act_mul_kernel<A, W>), dim3((int)blocks), dim3(threads), 0, s, gate_up,   \
                 (const W*)bias, (A*)out, inter, total, kind)
    if (act_dtype == MSTAR_F32) {
        if (weight_dtype == MSTAR_F32) { GO(float, float); } else { GO(float, bf16); }
    } else {
        if (weight_dtype == MSTAR_F32) { GO(bf16, float); } else { GO(bf16, bf16); }
    }
#undef GO
    return launch_status();
}

// ------------------------------------------------- logit scale and soft cap
// x = x * scale, then x = cap * tanh(x / cap) when cap > 0; float, in place.
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t n, float scale, float cap) {
    x = pdl_after(x, pdl_wait());
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v * inv_cap);
        x[i] = v;
    }
}

MSTAR_API int mstar_scale_softcap(float* x, long long n, float scale, float cap, void* stream) {
    if (n <= 0) return 0;
    size_t blocks = ((size_t)n + 255) / 256;
    const size_t most = (size_t)device_sm_count() * 32;
    if (blocks > most) blocks = most;
    mstar_launch(scale_softcap_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, x,
                 (size_t)n, scale, cap);
    return launch_status();
}

// ------------------------------------------------------------- conversion
template <typename S, typename D>
__global__ void convert_kernel(const S* __restrict__ src, D* __restrict__ dst, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = from_float<D>(to_float(src[i]));
}

MSTAR_API int mstar_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long long n,
                            void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    size_t blocks = ((size_t)n + 255) / 256;
    const size_t most = (size_t)device_sm_count() * 32;   // a grid-stride loop takes the rest
    if (blocks > most) blocks = most;
    if (src_dtype == MSTAR_F32 && dst_dtype == MSTAR_BF16)
        convert_kernel<float, bf16><<<(int)blocks, 256, 0, s>>>((const float*)src, (bf16*)dst, (size_t)n);
    else if (src_dtype == MSTAR_BF16 && dst_dtype == MSTAR_F32)
        convert_kernel<bf16, float><<<(int)blocks, 256, 0, s>>>((const bf16*)src, (float*)dst, (size_t)n);
    else if (src_dtype == MSTAR_F32 && dst_dtype == MSTAR_F32)
        convert_kernel<float, float><<<(int)blocks, 256, 0, s>>>((const float*)src, (float*)dst, (size_t)n);
    else
        convert_kernel<bf16, bf16><<<(int)blocks, 256, 0, s>>>((const bf16*)src, (bf16*)dst, (size_t)n);
    return launch_status();
}

// ------------------------------------- rotary encoding + key/value page write
// qkv: [T, (nq + 2*nkv) * hd], rows [q heads | k heads | v heads].  Queries are
// rotated in place; keys are rotated and written, values copied, into the paged
// cache [pages, 2, nkv, page_size, hd] at (page, slot) of the token's cache
// position.  Angle = float(position) * inv_freq[j] in float, sincosf without
// fast-math (full range reduction).  rotary_dim == 0 writes keys unrotated.
// kv_cache == nullptr (a layer that reads another layer's cache): queries only.
struct RopeArgs {
    int nq, nkv, hd, rotary_dim, interleaved;
    int page_size, bt_stride;
};

template <typename A>
__global__ void rope_kv_write_kernel(A* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ cache_pos,
                                     const int* __restrict__ token_req,
                                     const int* __restrict__ block_table,
                                     const float* __restrict__ inv_freq, A* __restrict__ kv_cache,
                                     RopeArgs a) {
    pdl_launch_dependents();   // a short kernel: the long one after it may be scheduled now
    pdl_wait();
    // grid (token, slice): the items of a token (rotated pairs of q and k, unrotated tail
    // of k, values) are spread over all threads of its slices, one or a few each, so that
    // the dependent loads of different items overlap instead of queueing in one thread
    const int t = blockIdx.x;
    const int hd = a.hd, half = a.rotary_dim / 2;
    const int row_elems = (a.nq + 2 * a.nkv) * hd;
    A* row = qkv + (size_t)t * row_elems;
    const bool write = kv_cache != nullptr;
    const int rot_items = (write ? a.nq + a.nkv : a.nq) * half;
    const int tail = hd - a.rotary_dim;
    const int tail_items = write ? a.nkv * tail : 0;
    const int v_items = write ? a.nkv * hd : 0;
    const int total = rot_items + tail_items + v_items;
    const int first = blockIdx.y * blockDim.x + threadIdx.x;
    const int stride = gridDim.y * blockDim.x;
    if (first >= total) return;

    A* kdst = nullptr;
    A* vdst = nullptr;
    if (write) {
        const int cp = cache_pos[t];
        const int page = block_table[(size_t)token_req[t] * a.bt_stride + cp / a.page_size];
        const int slot = cp % a.page_size;
        const size_t page_elems = (size_t)2 * a.nkv * a.page_size * hd;
        kdst = kv_cache + (size_t)page * page_elems + (size_t)slot * hd;
        vdst = kdst + (size_t)a.nkv * a.page_size * hd;
    }
    const float pos = (float)positions[t];
    for (int item = first; item < total; item += stride) {
        if (item < rot_items) {
            const int h = item / half, j = item - h * half;
            const int i0 = a.interleaved ? 2 * j : j;
            const int i1 = a.interleaved ? 2 * j + 1 : j + half;
            float sn, cs;
            sincosf(pos * inv_freq[j], &sn, &cs);
            A* src = row + (size_t)h * hd;
            const float x0 = to_float(src[i0]), x1 = to_float(src[i1]);
            const float y0 = x0 * cs - x1 * sn;
            const float y1 = x1 * cs + x0 * sn;
            A* dst = h < a.nq ? src : kdst + (size_t)(h - a.nq) * a.page_size * hd;
            dst[i0] = from_float<A>(y0);
            dst[i1] = from_float<A>(y1);
        } else if (item < rot_items + tail_items) {
            // features of k beyond rotary_dim are copied unrotated
            const int it = item - rot_items;
            const int h = it / tail, d = a.rotary_dim + (it - h * tail);
            kdst[(size_t)h * a.page_size * hd + d] = row[(size_t)(a.nq + h) * hd + d];
        } else {
            const int it = item - rot_items - tail_items;
            const int h = it / hd, d = it - h * hd;
            vdst[(size_t)h * a.page_size * hd + d] = row[(size_t)(a.nq + a.nkv + h) * hd + d];
        }
    }
}

// Vector form of the kernel above for split-half pairs whose halves are multiples of 8
// features: a thread rotates 8 pairs (two 16-byte loads, two 16-byte stores) or copies
// 8 values; same arithmetic per element.
template <typename A>
__global__ void rope_kv_write_vec_kernel(A* __restrict__ qkv, const int* __restrict__ positions,
                                         const int* __restrict__ cache_pos,
                                         const int* __restrict__ token_req,
                                         const int* __restrict__ block_table,
                                         const float* __restrict__ inv_freq,
                                         A* __restrict__ kv_cache, RopeArgs a) {
    pdl_launch_dependents();   // a short kernel: the long one after it may be scheduled now
    pdl_wait();
    const int t = blockIdx.x;
    const int hd = a.hd, half = a.rotary_dim / 2;
    const int row_elems = (a.nq + 2 * a.nkv) * hd;
    A* row = qkv + (size_t)t * row_elems;
    const bool write = kv_cache != nullptr;
    const int hchunks = half >> 3;                         // 8-pair chunks per head
    const int rot_items = (write ? a.nq + a.nkv : a.nq) * hchunks;
    const int tail = hd - a.rotary_dim;                    // multiple of 8 on this path
    const int tail_items = write ? a.nkv * (tail >> 3) : 0;
    const int v_items = write ? a.nkv * (hd >> 3) : 0;
    const int total = rot_items + tail_items + v_items;
    const int first = blockIdx.y * blockDim.x + threadIdx.x;
    const int stride = gridDim.y * blockDim.x;
    // the token's sines and cosines once per block (every head uses the same); half <= 128
    __shared__ float tab_sn[128], tab_cs[128];
    {
        const float p = (float)positions[t];
        for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(p * inv_freq[j], &tab_sn[j], &tab_cs[j]);
    }
    __syncthreads();
    if (first >= total) return;

    A* kdst = nullptr;
    A* vdst = nullptr;
    if (write) {
        const int cp = cache_pos[t];
        const int page = block_table[(size_t)token_req[t] * a.bt_stride + cp / a.page_size];
        const int slot = cp % a.page_size;
        const size_t page_elems = (size_t)2 * a.nkv * a.page_size * hd;
        kdst = kv_cache + (size_t)page * page_elems + (size_t)slot * hd;
        vdst = kdst + (size_t)a.nkv * a.page_size * hd;
    }
    for (int item = first; item < total; item += stride) {
        if (item < rot_items) {
            const int h = item / hchunks, j0 = (item - h * hchunks) * 8;
            A* src = row + (size_t)h * hd;
            float x0[8], x1[8], y0[8], y1[8];
            load8(src + j0, x0);
            load8(src + j0 + half, x1);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float sn = tab_sn[j0 + i], cs = tab_cs[j0 + i];
                y0[i] = x0[i] * cs - x1[i] * sn;
                y1[i] = x1[i] * cs + x0[i] * sn;
            }
            A* dst = h < a.nq ? src : kdst + (size_t)(h - a.nq) * a.page_size * hd;
            store8(dst + j0, y0);
            store8(dst + j0 + half, y1);
        } else if (item < rot_items + tail_items) {
            const int it = item - rot_items;
            const int per = tail >> 3;
            const int h = it / per, d = a.rotary_dim + (it - h * per) * 8;
            *reinterpret_cast<uint4*>(kdst + (size_t)h * a.page_size * hd + d) =
                *reinterpret_cast<const uint4*>(row + (size_t)(a.nq + h) * hd + d);
        } else {
            const int it = item - rot_items - tail_items;
            const int per = hd >> 3;
            const int h = it / per, d = (it - h * per) * 8;
            float v[8];
            load8(row + (size_t)(a.nq + a.nkv + h) * hd + d, v);
            store8(vdst + (size_t)h * a.page_size * hd + d, v);
        }
    }
}

MSTAR_API int mstar_rope_kv_write(void* qkv, int act_dtype, const int* positions,
                                  const int* cache_pos, const int* token_req,
                                  const int* block_table, int bt_stride, const float* inv_freq,
                                  void* kv_cache, int num_tokens, int nq, int nkv, int hd,
                                  int rotary_dim, int interleaved, int page_size, void* stream) {
    if (num_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    RopeArgs a{nq, nkv, hd, rotary_dim, interleaved, page_size, bt_stride};
    const int threads = 256;
    // split-half pairs, halves and the unrotated tail in whole groups of 8, float angles
    // table aligned: the vector kernel; else one pair per item
    const bool vec = !interleaved && rotary_dim > 0 && rotary_dim <= 256 && (rotary_dim / 2) % 8 == 0 && hd % 8 == 0 &&
                     (hd - rotary_dim) % 8 == 0 && ((uintptr_t)qkv % 32 == 0) &&
                     ((uintptr_t)inv_freq % 32 == 0) && (kv_cache == nullptr || (uintptr_t)kv_cache % 32 == 0) &&
                     act_dtype == MSTAR_BF16;
    if (vec) {
        const int items = (nq + nkv) * (rotary_dim / 16) + nkv * ((hd - rotary_dim) / 8) + nkv * (hd / 8);
        int slices = (items + threads - 1) / threads;
        if (num_tokens >= 256 && slices > 1) slices = 1;
        if (slices < 1) slices = 1;
        dim3 grid(num_tokens, slices);
        mstar_launch((rope_kv_write_vec_kernel<bf16>), dim3(grid), dim3(threads), 0, s, 
            (bf16*)qkv, positions, cache_pos, token_req, block_table, inv_freq, (bf16*)kv_cache, a);
        return launch_status();
    }
    const int items = (nq + nkv) * (rotary_dim / 2) + nkv * (hd - rotary_dim) + nkv * hd;
    // few tokens: one item per thread; many tokens: fewer, longer-running slices
    int slices = (items + threads - 1) / threads;
    if (num_tokens >= 256 && slices > 2) slices = 2;
    if (slices < 1) slices = 1;
    dim3 grid(num_tokens, slices);
    if (act_dtype == MSTAR_F32)
        mstar_launch((rope_kv_write_kernel<float>), dim3(grid), dim3(threads), 0, s, 
            (float*)qkv, positions, cache_pos, token_req, block_table, inv_freq, (float*)kv_cache, a);
    else
        mstar_launch((rope_kv_write_kernel<bf16>), dim3(grid), dim3(threads), 0, s, 
            (bf16*)qkv, positions, cache_pos, token_req, block_table, inv_freq, (bf16*)kv_cache, a);
    return launch_status();
}

// ------------------------------------------- post-norm + residual add + pre-norm
// A sublayer whose output is normalised before it joins the residual:
//   resid += post_scale * rms(delta, post_eps) * (post_w + post_off)   (always)
//   out    = rms(resid, eps) * (weight + w_off)          (when out and weight are given)
//   out    = resid in the activation type                (when out is given without a weight:
//                                                         the next sublayer reads the residual)
// One block per row; the row stays in shared memory between the passes.  Sums, scales and
// the residual are float for both activation types; a row's sums are taken in an order that
// depends only on its width.
template <typename D, typename A, typename W>
__global__ void add_postnorm_rmsnorm_kernel(float* __restrict__ resid, const D* __restrict__ delta,
                                            const float* __restrict__ post_w, float post_eps,
                                            float post_off, float post_scale,
                                            const W* __restrict__ weight, A* __restrict__ out,
                                            int hidden, float eps, float w_off) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * hidden;
    delta = pdl_after(delta, pdl_wait());
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = to_float(delta[base + i]);
        row[i] = d;
        ss = fmaf(d, d, ss);
    }
    const float inv_d = rsqrtf(block_sum(ss, scratch) / (float)hidden + post_eps);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float h = resid[base + i] + post_scale * (row[i] * inv_d * (post_w[i] + post_off));
        resid[base + i] = h;
        row[i] = h;
        ss2 = fmaf(h, h, ss2);
    }
    if (out == nullptr) return;
    if (weight == nullptr) {                 // the new residual itself, in the activation type
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[base + i] = from_float<A>(row[i]);
        return;
    }
    const float inv = rsqrtf(block_sum(ss2, scratch) / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        out[base + i] = from_float<A>(row[i] * inv * (to_float(weight[i]) + w_off));
}

// delta: [rows, hidden] of `delta_dtype`; out: nullptr, or [rows, hidden] of `act_dtype` (the
// pre-normed rows when `weight` is given, the residual itself when it is not).
MSTAR_API int mstar_add_postnorm_rmsnorm(float* resid, const void* delta, int delta_dtype,
                                         const float* post_w, float post_eps, float post_off,
                                         float post_scale, const void* weight, int weight_dtype,
                                         void* out, int act_dtype, int rows, int hidden, float eps,
                                         float w_off, void* stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || hidden > 48 * 1024 / 4) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const size_t smem = sizeof(float) * (size_t)hidden;
#define LAUNCH(D, A, W)                                                                           \
    mstar_launch((add_postnorm_rmsnorm_kernel<D, A, W>), dim3(rows), dim3(threads), smem, s,      \
                 resid, (const D*)delta, post_w, post_eps, post_off, post_scale,                  \
                 (const W*)weight, (A*)out, hidden, eps, w_off)
    if (act_dtype == MSTAR_F32) {
        if (delta_dtype != MSTAR_F32) return -1;
        if (weight_dtype == MSTAR_F32) { LAUNCH(float, float, float); } else { LAUNCH(float, float, bf16); }
    } else if (delta_dtype == MSTAR_F32) {
        if (weight_dtype == MSTAR_F32) { LAUNCH(float, bf16, float); } else { LAUNCH(float, bf16, bf16); }
    } else {
        if (weight_dtype == MSTAR_F32) { LAUNCH(bf16, bf16, float); } else { LAUNCH(bf16, bf16, bf16); }
    }
#undef LAUNCH
    return launch_status();
}

// ------------------------------------------------------------ mean of normed branch outputs
// out[r] = (1/n) sum_b rms(x_b[r]) * w_b, float out; n = 2..4 branches of the same width.
struct BranchPtrs {
    const void* x[4];
    const float* w[4];
};

template <typename A>
__global__ void mean_of_norms_kernel(BranchPtrs p, int n, float* __restrict__ out, int hidden,
                                     float eps) {
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * hidden;
    const unsigned long long waited = pdl_wait();
    float inv[4];
    for (int b = 0; b < n; ++b) {
        const A* x = pdl_after((const A*)p.x[b], waited);
        float ss = 0.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = to_float(x[base + i]);
            ss = fmaf(v, v, ss);
        }
        inv[b] = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    }
    const float share = 1.f / (float)n;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float sum = 0.f;
        for (int b = 0; b < n; ++b) {
            const A* x = pdl_after((const A*)p.x[b], waited);
            sum += to_float(x[base + i]) * inv[b] * p.w[b][i];
        }
        out[base + i] = sum * share;
    }
}

MSTAR_API int mstar_mean_of_norms(const void* x0, const void* x1, const void* x2, const void* x3,
                                  const float* w0, const float* w1, const float* w2,
                                  const float* w3, int n, float* out, int act_dtype, int rows,
                                  int hidden, float eps, void* stream) {
    if (rows <= 0) return 0;
    if (n < 1 || n > 4 || hidden <= 0) return -1;
    BranchPtrs p{{x0, x1, x2, x3}, {w0, w1, w2, w3}};
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == MSTAR_F32)
        mstar_launch((mean_of_norms_kernel<float>), dim3(rows), dim3(threads), 0, s, p, n, out,
                     hidden, eps);
    else
        mstar_launch((mean_of_norms_kernel<bf16>), dim3(rows), dim3(threads), 0, s, p, n, out,
                     hidden, eps);
    return launch_status();
}

// ------------------------------------- mean of two normed branches + post-norm + residual add
//   y      = (rms(x0) * w0 + rms(x1) * w1) / 2
//   resid += post_scale * rms(y, post_eps) * (post_w + post_off)
//   out    = resid in the activation type (when out != nullptr)
// One block per row; y stays in shared memory.  All sums and scales are float.
template <typename A>
__global__ void mean2_postnorm_kernel(float* __restrict__ resid, const A* __restrict__ x0,
                                      const A* __restrict__ x1, const float* __restrict__ w0,
                                      const float* __restrict__ w1, float eps,
                                      const float* __restrict__ post_w, float post_eps,
                                      float post_off, float post_scale, A* __restrict__ out,
                                      int hidden) {
    extern __shared__ float row[];           // [2][hidden]: the branches, then y in the first
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * hidden;
    const unsigned long long waited = pdl_wait();
    x0 = pdl_after(x0, waited);
    x1 = pdl_after(x1, waited);
    float s0 = 0.f, s1 = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float a = to_float(x0[base + i]), b = to_float(x1[base + i]);
        row[i] = a;
        row[hidden + i] = b;
        s0 = fmaf(a, a, s0);
        s1 = fmaf(b, b, s1);
    }
    const float inv0 = rsqrtf(block_sum(s0, scratch) / (float)hidden + eps);
    const float inv1 = rsqrtf(block_sum(s1, scratch) / (float)hidden + eps);
    float sy = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float y = (row[i] * inv0 * w0[i] + row[hidden + i] * inv1 * w1[i]) * 0.5f;
        row[i] = y;
        sy = fmaf(y, y, sy);
    }
    const float invy = rsqrtf(block_sum(sy, scratch) / (float)hidden + post_eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float h = resid[base + i] + post_scale * (row[i] * invy * (post_w[i] + post_off));
        resid[base + i] = h;
        if (out != nullptr) out[base + i] = from_float<A>(h);
    }
}

MSTAR_API int mstar_mean2_postnorm(float* resid, const void* x0, const void* x1, const float* w0,
                                   const float* w1, float eps, const float* post_w, float post_eps,
                                   float post_off, float post_scale, void* out, int act_dtype,
                                   int rows, int hidden, void* stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || hidden > 48 * 1024 / 8) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const size_t smem = sizeof(float) * 2 * (size_t)hidden;
    if (act_dtype == MSTAR_F32)
        mstar_launch((mean2_postnorm_kernel<float>), dim3(rows), dim3(threads), smem, s, resid,
                     (const float*)x0, (const float*)x1, w0, w1, eps, post_w, post_eps, post_off,
                     post_scale, (float*)out, hidden);
    else
        mstar_launch((mean2_postnorm_kernel<bf16>), dim3(rows), dim3(threads), smem, s, resid,
                     (const bf16*)x0, (const bf16*)x1, w0, w1, eps, post_w, post_eps, post_off,
                     post_scale, (bf16*)out, hidden);
    return launch_status();
}

// ------------------------------------------------------------ activations without a gate
// kinds as in plain_activation above.  In place or not.

template <typename A>
__global__ void activation_kernel(const A* __restrict__ x, A* __restrict__ out, size_t total,
                                  int kind) {
    x = pdl_after(x, pdl_wait());
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_float<A>(plain_activation(to_float(x[i]), kind));
}

MSTAR_API int mstar_activation(const void* x, void* out, int act_dtype, long long total, int kind,
                               void* stream) {
    if (total <= 0) return 0;
    if (kind < 0 || kind > 2) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 8192 ? want : 8192);
    if (act_dtype == MSTAR_F32)
        mstar_launch((activation_kernel<float>), dim3(blocks), dim3(threads), 0, s, (const float*)x,
                     (float*)out, (size_t)total, kind);
    else
        mstar_launch((activation_kernel<bf16>), dim3(blocks), dim3(threads), 0, s, (const bf16*)x,
                     (bf16*)out, (size_t)total, kind);
    return launch_status();
}

// ------------------------------------------------------------ y *= sigmoid(gate)
// y: [rows, cols] contiguous; gate: rows of `ldg` elements (a view into a wider product).
template <typename A>
__global__ void sigmoid_gate_mul_kernel(A* __restrict__ y, const A* __restrict__ gate, int cols,
                                        int ldg, size_t total) {
    const unsigned long long waited = pdl_wait();
    y = pdl_after(y, waited);
    gate = pdl_after(gate, waited);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / cols;
        const int c = (int)(idx - r * cols);
        const float g = to_float(gate[r * (size_t)ldg + c]);
        y[idx] = from_float<A>(to_float(y[idx]) / (1.f + expf(-g)));
    }
}

MSTAR_API int mstar_sigmoid_gate_mul(void* y, const void* gate, int act_dtype, int rows, int cols,
                                     int ldg, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)rows * cols;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 4096 ? (total + threads - 1) / threads : 4096);
    if (act_dtype == MSTAR_F32)
        mstar_launch((sigmoid_gate_mul_kernel<float>), dim3(blocks), dim3(threads), 0, s, (float*)y,
                     (const float*)gate, cols, ldg, total);
    else
        mstar_launch((sigmoid_gate_mul_kernel<bf16>), dim3(blocks), dim3(threads), 0, s, (bf16*)y,
                     (const bf16*)gate, cols, ldg, total);
    return launch_status();
}

// ------------------------------------------------------------ out = y * sigmoid(gate of the head)
// y: [rows, heads * dim] contiguous, in In; gate: one number per row and head, rows of `ldg`
// elements (a view into a wider product), in G; out: [rows, heads * dim] in Out (may be y).
template <typename In, typename Out, typename G>
__global__ void head_gate_mul_kernel(const In* y, Out* out, const G* __restrict__ gate, int heads,
                                     int dim, int ldg, size_t total) {
    const unsigned long long waited = pdl_wait();
    y = pdl_after(y, waited);
    gate = pdl_after(gate, waited);
    const int cols = heads * dim;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / cols;
        const int h = (int)(idx - r * cols) / dim;
        const float g = to_float(gate[r * (size_t)ldg + h]);
        out[idx] = from_float<Out>(to_float(y[idx]) / (1.f + expf(-g)));
    }
}

MSTAR_API int mstar_head_gate_mul(const void* y, int in_dtype, void* out, int out_dtype,
                                  const void* gate, int gate_dtype, int ldg, int rows, int heads,
                                  int dim, void* stream) {
    if (rows <= 0 || heads <= 0 || dim <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)rows * heads * dim;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 4096 ? (total + threads - 1) / threads : 4096);
#define GO(I, O, G)                                                                               \
    mstar_launch((head_gate_mul_kernel<I, O, G>), dim3(blocks), dim3(threads), 0, s, (const I*)y, \
                 (O*)out, (const G*)gate, heads, dim, ldg, total)
    const int key = (in_dtype == MSTAR_F32 ? 4 : 0) | (out_dtype == MSTAR_F32 ? 2 : 0) |
                    (gate_dtype == MSTAR_F32 ? 1 : 0);
    switch (key) {
        case 0: GO(bf16, bf16, bf16); break;
        case 1: GO(bf16, bf16, float); break;
        case 2: GO(bf16, float, bf16); break;
        case 3: GO(bf16, float, float); break;
        case 4: GO(float, bf16, bf16); break;
        case 5: GO(float, bf16, float); break;
        case 6: GO(float, float, bf16); break;
        default: GO(float, float, float); break;
    }
#undef GO
    return launch_status();
}
