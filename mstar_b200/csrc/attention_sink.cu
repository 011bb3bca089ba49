// Grouped-query attention with a sliding window that keeps the first keys of a sequence, a
// value size of its own, biased projections and an RMS norm per query and key head.
//
//   prepare   row = [q: nq*hd | k: nkv*hd | v: nkv*vd] (float, the fused projection) + bias;
//             with `taps` > 0 every q and k channel first passes a causal convolution over
//             time, y_t = sum_j w[c][j] u_(t - taps + 1 + j), the rows before a portion's
//             start taken from the request's state slot (advance moves that state on);
//             with `v_from_k` the row has no v part and a key head as it stands here, before
//             its norm, is written as the value head;
//             every q and k head is divided by its root mean square (eps inside the root)
//             and scaled by a weight shared by the heads; the first `rot` features of q and
//             k are rotated (feature i with i + rot/2, or, `interleaved`, feature 2i with
//             2i + 1; angle position * freq[i]); q goes to a dense [tokens, nq*hd] buffer, k
//             and v into the token's cache page.  With `norm_whole` the root mean square is
//             taken over all heads of q (and of k) at once and the weights have a number per
//             feature of the whole projection.  With `temp_every` > 0 the query is multiplied
//             by 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1).
//   attend    the token whose key sits at cache position p sees keys j <= p with
//             p - j < window or j < keep_first (window 0: every j <= p): the keys
//             [0, min(keep_first, lo)) and [lo, p], lo = max(0, p - window + 1).  Softmax over
//             them, scores q.k * scale, float statistics and sums.  With `softcap` > 0 a
//             score becomes softcap * tanh(score / softcap); with `sink` the denominator of
//             head h also holds exp(sink[h]), which has no key and no value; a gate per
//             feature multiplies the output by sigmoid(gate[t][h * vd + d]).
//
// A cache page is [nkv][page_size][hd] keys followed by [nkv][page_size][vd] values.
// Norms, angles, scores, probabilities and output sums are float for both activation types.
#include "common.cuh"

// ------------------------------------------------------------------ prepare
struct PrepArgs {
    int nq, nkv, hd, vd, rot, page_size, bt_stride, q_stride_out;
    float eps;
    int norm;       // 1: q and k heads are normed
    int row_stride; // floats between the rows of two tokens
    int taps;       // 0: no convolution
    int v_from_k;   // 1: the values are the key heads before their norm
    long long state_stride;     // floats between the state of two slots
    int interleaved;            // 1: feature 2i is rotated with 2i + 1
    int norm_whole;             // 1: one root mean square over all q heads, one over all k heads
    float temp_coef;
    int temp_every;             // 0: no query temperature
};

// The convolved value of channel `col` (a column of q or k) of token t, the i-th of its
// portion: taps - 1 earlier rows come from the portion itself or, before its start, from
// the slot, which holds the request's last taps - 1 rows of [q | k] channels in time order.
template <typename W>
__device__ __forceinline__ float conv_feature(const float* __restrict__ row, const W* __restrict__ w,
                                              const float* __restrict__ state, int col, int chan,
                                              int channels, int i, const PrepArgs& a) {
    float y = 0.f;
    const int keep = a.taps - 1;
    if (keep <= i) {                                     // every row is of this portion
        const float* u = row - (ptrdiff_t)keep * a.row_stride + col;
        const W* wc = w + (size_t)chan * a.taps;
#pragma unroll 4
        for (int j = 0; j < a.taps; ++j) y = fmaf(to_float(wc[j]), u[(ptrdiff_t)j * a.row_stride], y);
        return y;
    }
    for (int j = 0; j < a.taps; ++j) {
        const int back = keep - j;                       // rows before this token
        const float u = back <= i ? *(row - (ptrdiff_t)back * a.row_stride + col)
                                  : state[(size_t)(keep + i - back) * channels + col];
        y = fmaf(to_float(w[(size_t)chan * a.taps + j]), u, y);
    }
    return y;
}

// One block per token.  Sines and cosines of the token's angles are made once (double
// precision product) and shared by all heads.
template <typename A, typename W>
__global__ void __launch_bounds__(256)
sink_prepare_kernel(const float* __restrict__ qkv, const W* __restrict__ bias,
                    const W* __restrict__ q_norm, const W* __restrict__ k_norm,
                    const double* __restrict__ freq, const int* __restrict__ positions,
                    const int* __restrict__ cache_pos, const int* __restrict__ token_req,
                    const int* __restrict__ block_table, A* __restrict__ q_out,
                    A* __restrict__ kv_cache, const W* __restrict__ conv_q,
                    const W* __restrict__ conv_k, const int* __restrict__ qo_indptr,
                    const int* __restrict__ slots, const float* state, PrepArgs a) {
    extern __shared__ float sm[];
    const int half = a.rot / 2;
    float* cs = sm;                            // [half] cosines, [half] sines
    float* heads = sm + 2 * half;              // [warps][hd]
    __shared__ float red[32];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const unsigned long long waited = pdl_wait();
    qkv = pdl_after(qkv, waited);
    // the angle in double precision, brought into [-pi, pi] there; sine and cosine of that
    // in float (the argument is then exact to 2e-7 whatever the position)
    const double pos = (double)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double ang = pos * freq[i];
        ang -= 6.283185307179586476925 * rint(ang * 0.15915494309189533577);
        float s, c;
        sincosf((float)ang, &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    __syncthreads();
    const float* row = qkv + (size_t)t * a.row_stride;
    const int channels = (a.nq + a.nkv) * a.hd;          // what the convolution runs over
    int local = 0;                                       // the token's place in its portion
    const float* slot_state = nullptr;
    if (a.taps > 0) {
        const int e = token_req[t];
        local = t - qo_indptr[e];
        slot_state = pdl_after(state, waited) + (size_t)slots[e] * a.state_stride;
    }
    const int key = cache_pos[t];
    const int page = block_table[(size_t)token_req[t] * a.bt_stride + key / a.page_size];
    const int slot = key % a.page_size;
    const size_t page_elems = (size_t)a.nkv * a.page_size * (a.hd + a.vd);
    A* page_base = kv_cache + (size_t)page * page_elems;
    float* mine = heads + warp * a.hd;
    const int nheads = a.v_from_k ? a.nq + a.nkv : a.nq + 2 * a.nkv;
    float inv_whole_q = 1.f, inv_whole_k = 1.f;
    if (a.norm && a.norm_whole) {              // (no convolution in this form)
        float sq = 0.f, sk = 0.f;
        const int nqd = a.nq * a.hd, nkd = a.nkv * a.hd;
        for (int i = threadIdx.x; i < nqd + nkd; i += blockDim.x) {
            float v = row[i];
            if (bias != nullptr) v += to_float(bias[i]);
            if (i < nqd) sq = fmaf(v, v, sq); else sk = fmaf(v, v, sk);
        }
        sq = block_sum(sq, red);
        sk = block_sum(sk, red);
        inv_whole_q = rsqrtf(sq / (float)nqd + a.eps);
        inv_whole_k = rsqrtf(sk / (float)nkd + a.eps);
    }
    float q_mult = 1.f;
    if (a.temp_every > 0)
        q_mult = 1.f + a.temp_coef * logf((float)((positions[t] + 1) / a.temp_every) + 1.f);
    // few tokens (decoding): the heads of a token are dealt out among gridDim.y blocks
    for (int h = blockIdx.y * nwarps + warp; h < nheads; h += nwarps * gridDim.y) {
        if (h >= a.nq + a.nkv) {               // a value head: bias, then the page
            const int g = h - a.nq - a.nkv;
            const int off = (a.nq + a.nkv) * a.hd + g * a.vd;
            A* dst = page_base + (size_t)a.nkv * a.page_size * a.hd +
                     ((size_t)g * a.page_size + slot) * a.vd;
            for (int d = lane; d < a.vd; d += 32) {
                float v = row[off + d];
                if (bias != nullptr) v += to_float(bias[off + d]);
                dst[d] = from_float<A>(v);
            }
            continue;
        }
        const bool is_q = h < a.nq;
        const int off = h * a.hd;
        float ss = 0.f;
        A* as_value = (!is_q && a.v_from_k)
                          ? page_base + (size_t)a.nkv * a.page_size * a.hd +
                                ((size_t)(h - a.nq) * a.page_size + slot) * a.vd
                          : nullptr;
        for (int d = lane; d < a.hd; d += 32) {
            float v;
            if (a.taps > 0) {
                v = is_q ? conv_feature(row, conv_q, slot_state, off + d, off + d, channels, local, a)
                         : conv_feature(row, conv_k, slot_state, off + d, off + d - a.nq * a.hd,
                                        channels, local, a);
            } else {
                v = row[off + d];
                if (bias != nullptr) v += to_float(bias[off + d]);
            }
            if (as_value != nullptr) as_value[d] = from_float<A>(v);
            mine[d] = v;
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        float inv = a.norm ? rsqrtf(ss / (float)a.hd + a.eps) : 1.f;
        const W* nw = is_q ? q_norm : k_norm;
        if (a.norm && a.norm_whole) {
            inv = is_q ? inv_whole_q : inv_whole_k;
            nw += (size_t)(is_q ? h : h - a.nq) * a.hd;
        }
        const float mult = is_q ? q_mult : 1.f;
        __syncwarp();
        if (a.norm)
            for (int d = lane; d < a.hd; d += 32) mine[d] = mine[d] * inv * to_float(nw[d]) * mult;
        else if (mult != 1.f)
            for (int d = lane; d < a.hd; d += 32) mine[d] *= mult;
        __syncwarp();
        A* dst = is_q ? q_out + (size_t)t * a.q_stride_out + (size_t)h * a.hd
                      : page_base + ((size_t)(h - a.nq) * a.page_size + slot) * a.hd;
        for (int d = lane; d < a.hd; d += 32) {
            float v = mine[d];
            if (a.interleaved) {
                if (d < a.rot) {
                    const int i = d >> 1;
                    v = (d & 1) ? mine[d] * cs[i] + mine[d - 1] * cs[half + i]
                                : mine[d] * cs[i] - mine[d + 1] * cs[half + i];
                }
            } else if (d < half) {
                v = mine[d] * cs[d] - mine[d + half] * cs[half + d];
            } else if (d < a.rot) {
                const int i = d - half;
                v = mine[d] * cs[i] + mine[i] * cs[half + i];
            }
            dst[d] = from_float<A>(v);
        }
        __syncwarp();
    }
}

MSTAR_API int mstar_sink_prepare(const float* qkv, const void* bias, const void* q_norm,
                                 const void* k_norm, int weight_dtype, const double* freq,
                                 const int* positions, const int* cache_pos, const int* token_req,
                                 const int* block_table, int bt_stride, void* q_out,
                                 void* kv_cache, int act_dtype, int tokens, int nq, int nkv, int hd,
                                 int vd, int rot, int page_size, float eps, int norm,
                                 int row_stride, const void* conv_q, const void* conv_k, int taps,
                                 int v_from_k, const int* qo_indptr, const int* slots,
                                 const float* state, long long state_stride, int interleaved,
                                 int norm_whole, float temp_coef, int temp_every, void* stream) {
    if (tokens <= 0) return 0;
    if (norm_whole && taps > 0) return -1;
    if (hd <= 0 || vd <= 0 || rot < 0 || rot > hd || (rot & 1) || nq <= 0 || nkv <= 0) return -1;
    if (taps < 0 || (v_from_k && vd != hd)) return -1;
    if (taps > 0 && (bias != nullptr || !conv_q || !conv_k || !qo_indptr)) return -1;
    if (taps > 1 && (!slots || !state)) return -1;
    if (row_stride < (nq + nkv) * hd + (v_from_k ? 0 : nkv * vd)) return -1;
    const int threads = 256;
    const size_t smem = sizeof(float) * ((size_t)rot + (size_t)(threads / 32) * hd);
    if (smem > 48 * 1024) return -1;
    PrepArgs a{nq, nkv, hd, vd, rot, page_size, bt_stride, nq * hd, eps, norm, row_stride, taps,
               v_from_k, state_stride, interleaved, norm_whole, temp_coef, temp_every};
    cudaStream_t s = (cudaStream_t)stream;
    // a block takes 8 heads at a time: with fewer blocks than SMs, a token's heads go to
    // several blocks (each makes the token's sines and cosines for itself)
    const int nheads = v_from_k ? nq + nkv : nq + 2 * nkv;
    int head_blocks = 1;
    if (tokens < device_sm_count()) {
        head_blocks = (nheads + threads / 32 - 1) / (threads / 32);
        const int room = (2 * device_sm_count() + tokens - 1) / tokens;
        if (head_blocks > room) head_blocks = room;
        if (head_blocks < 1) head_blocks = 1;
    }
#define GO(A, W)                                                                                  \
    mstar_launch((sink_prepare_kernel<A, W>), dim3(tokens, head_blocks), dim3(threads), smem, s, qkv, \
                 (const W*)bias, (const W*)q_norm, (const W*)k_norm, freq, positions, cache_pos,  \
                 token_req, block_table, (A*)q_out, (A*)kv_cache, (const W*)conv_q,               \
                 (const W*)conv_k, qo_indptr, slots, state, a)
    if (act_dtype == MSTAR_F32) {
        if (weight_dtype == MSTAR_F32) { GO(float, float); } else { GO(float, bf16); }
    } else {
        if (weight_dtype == MSTAR_F32) { GO(bf16, float); } else { GO(bf16, bf16); }
    }
#undef GO
    return launch_status();
}

// ------------------------------------------------------------------ advance
// After prepare: the slot of every entry keeps the last taps - 1 rows of its sequence's
// projected [q | k] channels (before the convolution).  A portion shorter than that keeps the
// newer part of what the slot held.  A thread per entry and channel, oldest row first: row s
// is read from s + n, which is written later or not at all.
__global__ void conv_state_advance_kernel(const float* __restrict__ qkv, int row_stride, int channels,
                                          int taps, const int* __restrict__ qo_indptr,
                                          const int* __restrict__ slots, float* state,
                                          long long state_stride) {
    const unsigned long long waited = pdl_wait();
    qkv = pdl_after(qkv, waited);
    state = pdl_after(state, waited);
    const int e = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int start = qo_indptr[e], n = qo_indptr[e + 1] - start, keep = taps - 1;
    float* st = state + (size_t)slots[e] * state_stride;
    for (int s = 0; s < keep; ++s) {
        const int src = n - keep + s;                    // place in the portion, or before it
        st[(size_t)s * channels + c] = src >= 0 ? qkv[(size_t)(start + src) * row_stride + c]
                                                : st[(size_t)(s + n) * channels + c];
    }
}

MSTAR_API int mstar_conv_state_advance(const float* qkv, int row_stride, int channels, int taps,
                                       const int* qo_indptr, const int* slots, float* state,
                                       long long state_stride, int entries, void* stream) {
    if (entries <= 0 || taps <= 1 || channels <= 0) return 0;
    if (!qkv || !qo_indptr || !slots || !state) return -1;
    const int threads = 128;
    mstar_launch(conv_state_advance_kernel, dim3((channels + threads - 1) / threads, entries),
                 dim3(threads), 0, (cudaStream_t)stream, qkv, row_stride, channels, taps, qo_indptr,
                 slots, state, state_stride);
    return launch_status();
}

// ------------------------------------------------------------------ attend (CUDA cores)
#define SA_TILE 32
#define SA_THREADS 128
#define SA_MAX_ACC 32

struct SinkArgs {
    int nq, nkv, hd, vd, page_size, bt_stride, window, keep_first, q_stride;
    float scale;
    float softcap;              // 0: none
    const float* sink;          // null, or one number a query head
    const float* gate;          // null, or float rows with a number per (head, feature)
    int gate_stride;
};

// The v-th key a token sees: the kept first keys come before the window's.
__device__ __forceinline__ int visible_key(int v, int kept, int lo) { return v < kept ? v : lo + v - kept; }

// One block per (token, kv head): the group's query heads share the keys and values that
// stream through shared memory in tiles of 32 visible keys, online softmax.  Tiles are
// anchored at the token's own first visible key, so a row's arithmetic does not depend on
// what else is in the batch.
template <typename A>
__global__ void __launch_bounds__(SA_THREADS)
sink_attention_generic_kernel(const A* __restrict__ q, A* __restrict__ out,
                              const A* __restrict__ kv_cache, const int* __restrict__ block_table,
                              const int* __restrict__ token_req, const int* __restrict__ cache_pos,
                              SinkArgs a) {
    extern __shared__ float smem[];
    const int t = blockIdx.x, kvh = blockIdx.y;
    const int hd = a.hd, vd = a.vd, G = a.nq / a.nkv;
    const int wide = hd > vd ? hd : vd;
    const int ldk = wide + 1;
    float* qs = smem;                        // [G][hd]
    float* tile = qs + G * hd;               // [SA_TILE][wide+1]
    float* sc = tile + SA_TILE * ldk;        // [G][SA_TILE]
    float* m_s = sc + G * SA_TILE;           // [G]
    float* l_s = m_s + G;                    // [G]
    float* alpha_s = l_s + G;                // [G]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned long long waited = pdl_wait();
    q = pdl_after(q, waited);
    kv_cache = pdl_after(kv_cache, waited);
    const float* gate = pdl_after(a.gate, waited);
    const int hi = cache_pos[t] + 1;
    const int lo = (a.window > 0 && hi > a.window) ? hi - a.window : 0;
    const int kept = a.keep_first < lo ? a.keep_first : lo;
    const int visible = kept + hi - lo;
    const int* bt = block_table + (size_t)token_req[t] * a.bt_stride;
    const size_t page_elems = (size_t)a.nkv * a.page_size * (hd + vd);
    const size_t k_head = (size_t)kvh * a.page_size * hd;
    const size_t v_head = (size_t)a.nkv * a.page_size * hd + (size_t)kvh * a.page_size * vd;

    const A* qrow = q + (size_t)t * a.q_stride + (size_t)kvh * G * hd;
    for (int i = tid; i < G * hd; i += SA_THREADS) qs[i] = to_float(qrow[i]);
    for (int i = tid; i < G; i += SA_THREADS) {
        m_s[i] = -INFINITY;
        l_s[i] = 0.f;
    }
    float acc[SA_MAX_ACC];
#pragma unroll
    for (int k = 0; k < SA_MAX_ACC; ++k) acc[k] = 0.f;
    const int n_out = G * vd;
    __syncthreads();

    for (int base = 0; base < visible; base += SA_TILE) {
        for (int idx = tid; idx < SA_TILE * hd; idx += SA_THREADS) {
            const int j = idx / hd, d = idx - j * hd;
            float v = 0.f;
            if (base + j < visible) {
                const int key = visible_key(base + j, kept, lo);
                const int page = bt[key / a.page_size];
                v = to_float(kv_cache[(size_t)page * page_elems + k_head +
                                      (size_t)(key % a.page_size) * hd + d]);
            }
            tile[j * ldk + d] = v;
        }
        __syncthreads();
        for (int idx = tid; idx < G * SA_TILE; idx += SA_THREADS) {
            const int g = idx / SA_TILE, j = idx - g * SA_TILE;
            float s = -INFINITY;
            if (base + j < visible) {
                const float* qv = qs + g * hd;
                const float* kv = tile + j * ldk;
                float dot = 0.f;
                for (int d = 0; d < hd; ++d) dot = fmaf(qv[d], kv[d], dot);
                s = dot * a.scale;
                if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
            }
            sc[idx] = s;
        }
        __syncthreads();
        for (int g = warp; g < G; g += SA_THREADS / 32) {
            const float s = sc[g * SA_TILE + lane];
            const float m_old = m_s[g];
            const float m_new = fmaxf(m_old, warp_max(s));  // the tile's first key is visible
            const float p = expf(s - m_new);
            const float psum = warp_sum(p);
            sc[g * SA_TILE + lane] = p;
            if (lane == 0) {
                const float al = expf(m_old - m_new);
                alpha_s[g] = al;
                l_s[g] = l_s[g] * al + psum;
                m_s[g] = m_new;
            }
        }
        __syncthreads();
        for (int idx = tid; idx < SA_TILE * vd; idx += SA_THREADS) {
            const int j = idx / vd, d = idx - j * vd;
            float v = 0.f;
            if (base + j < visible) {
                const int key = visible_key(base + j, kept, lo);
                const int page = bt[key / a.page_size];
                v = to_float(kv_cache[(size_t)page * page_elems + v_head +
                                      (size_t)(key % a.page_size) * vd + d]);
            }
            tile[j * ldk + d] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < SA_MAX_ACC; ++k) {
            const int o = tid + k * SA_THREADS;
            if (o < n_out) {
                const int g = o / vd, d = o - g * vd;
                const float* p = sc + g * SA_TILE;
                float sum = acc[k] * alpha_s[g];
#pragma unroll 8
                for (int j = 0; j < SA_TILE; ++j) sum = fmaf(p[j], tile[j * ldk + d], sum);
                acc[k] = sum;
            }
        }
        __syncthreads();
    }

    if (a.sink != nullptr) {                  // the sink joins the denominator only
        for (int g = tid; g < G; g += SA_THREADS) l_s[g] += expf(a.sink[kvh * G + g] - m_s[g]);
        __syncthreads();
    }
    A* orow = out + (size_t)t * a.nq * vd + (size_t)kvh * G * vd;
#pragma unroll
    for (int k = 0; k < SA_MAX_ACC; ++k) {
        const int o = tid + k * SA_THREADS;
        if (o < n_out) {
            float r = acc[k] / l_s[o / vd];
            if (gate != nullptr)
                r /= 1.f + expf(-gate[(size_t)t * a.gate_stride + (size_t)kvh * G * vd + o]);
            orow[o] = from_float<A>(r);
        }
    }
}

// q: [tokens] rows of q_stride elements (nq*hd used); out: [tokens, nq*vd].  Returns 0, a
// CUDA error code, or -1 when the shape is refused.
MSTAR_API int mstar_sink_attention_generic(const void* q, int q_stride, void* out,
                                           const void* kv_cache, const int* block_table,
                                           int bt_stride, const int* token_req,
                                           const int* cache_pos, int tokens, int nq, int nkv,
                                           int hd, int vd, int page_size, int window,
                                           int keep_first, float scale, int act_dtype,
                                           float softcap, const float* sink, const float* gate,
                                           int gate_stride, void* stream) {
    if (tokens <= 0) return 0;
    if (nkv <= 0 || nq % nkv != 0 || hd <= 0 || vd <= 0) return -1;
    const int G = nq / nkv;
    if (G * vd > SA_MAX_ACC * SA_THREADS) return -1;
    const int wide = hd > vd ? hd : vd;
    const size_t smem = sizeof(float) * ((size_t)G * hd + (size_t)SA_TILE * (wide + 1) +
                                         (size_t)G * SA_TILE + 3 * (size_t)G);
    if (smem > 200 * 1024) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    SinkArgs a{nq, nkv, hd, vd, page_size, bt_stride, window, keep_first, q_stride, scale,
               softcap, sink, gate, gate_stride};
    dim3 grid(tokens, nkv);
    static size_t configured_f32 = 0, configured_bf16 = 0;
    if (act_dtype == MSTAR_F32) {
        if (smem > 48 * 1024 && smem > configured_f32) {
            cudaFuncSetAttribute(sink_attention_generic_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_f32 = smem;
        }
        mstar_launch((sink_attention_generic_kernel<float>), grid, dim3(SA_THREADS), smem, s,
                     (const float*)q, (float*)out, (const float*)kv_cache, block_table, token_req,
                     cache_pos, a);
    } else {
        if (smem > 48 * 1024 && smem > configured_bf16) {
            cudaFuncSetAttribute(sink_attention_generic_kernel<bf16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_bf16 = smem;
        }
        mstar_launch((sink_attention_generic_kernel<bf16>), grid, dim3(SA_THREADS), smem, s,
                     (const bf16*)q, (bf16*)out, (const bf16*)kv_cache, block_table, token_req,
                     cache_pos, a);
    }
    return launch_status();
}
