// Gated delta rule: a matrix memory S [dim][vdim] per head that is decayed row by row,
// corrected towards the token's value along its key, and read with its query.
//
//   prepare  from the float fused projection row [q: G*D | k: G*D | v: H*VD | b: H | ...]:
//            a causal convolution over time on every q, k and v channel (taps weights a
//            channel, the last on the token itself; rows before a portion's start from the
//            request's state slot, which holds the last taps - 1 projected rows) and SiLU;
//            q and k heads to unit length (x / sqrt(sum x^2 + unit_eps)), q times D^-1/2;
//            beta = sigmoid(b);  decay = exp(-exp(A_log_h) * softplus(a + dt_bias)) per head
//            and key channel, a = the low-rank projection's output [H*D].
//   scan     per head, token after token:  S = decay * S (rows);  u = beta (v - S^T k);
//            S += k u^T;  o = S^T q.  Computed as  r = (decay*S)^T k,  p = (decay*S)^T q,
//            u = beta (v - r),  o = p + (q . k) u,  so that one round of shuffles serves a token.
//   finish   o / rms(o per head) * weight * sigmoid(gate), handed on in the activation type.
//
// A slot is [(taps - 1) * (2 G D + H VD) convolution inputs | S^T as [H][VD][D]], float.
// Everything here is float whatever the activation type.
#include "common.cuh"

// ------------------------------------------------------------------ prepare
struct DeltaPrepArgs {
    const float* proj;
    int row_stride;
    const void* conv_w;         // [2 G D + H VD][taps], weight type
    const float* a_proj;        // [tokens][H*D]
    const float* dt_bias;       // [H*D]
    const float* a_exp;         // [H]: exp(A_log)
    const int* token_req;
    const int* qo_indptr;
    const int* slots;
    const float* state;
    long long state_stride;
    float* q;                   // [tokens][G*D]
    float* k;                   // [tokens][G*D]
    float* v;                   // [tokens][H*VD]
    float* beta;                // [tokens][H]
    float* decay;               // [tokens][H*D]
    int H, G, D, VD, taps;
    float unit_eps;
};

__device__ __forceinline__ float gd_softplus(float z) {
    return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
}

template <typename W>
__global__ void __launch_bounds__(256) delta_prepare_kernel(DeltaPrepArgs a) {
    extern __shared__ float ch[];             // [2 G D + H VD] convolved, activated channels
    const int t = blockIdx.x;
    const int qk = a.G * a.D, vv = a.H * a.VD, channels = 2 * qk + vv;
    const W* cw = reinterpret_cast<const W*>(a.conv_w);
    const unsigned long long waited = pdl_wait();
    const float* proj = pdl_after(a.proj, waited);
    const float* a_proj = pdl_after(a.a_proj, waited);
    const float* state = pdl_after(a.state, waited);
    const int e = a.token_req[t];
    const int local = t - a.qo_indptr[e];
    const float* slot = state + (size_t)a.slots[e] * a.state_stride;
    const float* row = proj + (size_t)t * a.row_stride;
    const int keep = a.taps - 1;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float y = 0.f;
        for (int j = 0; j < a.taps; ++j) {
            const int back = keep - j;                   // rows before this token
            const float u = back <= local ? *(row - (ptrdiff_t)back * a.row_stride + c)
                                          : slot[(size_t)(keep + local - back) * channels + c];
            y = fmaf(to_float(cw[(size_t)c * a.taps + j]), u, y);
        }
        y = y / (1.f + expf(-y));
        if (c >= 2 * qk) a.v[(size_t)t * vv + (c - 2 * qk)] = y;
        else ch[c] = y;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const float q_scale = rsqrtf((float)a.D);
    for (int h = warp; h < 2 * a.G; h += nwarps) {        // q heads, then k heads
        const float* src = ch + (size_t)h * a.D;
        float ss = 0.f;
        for (int d = lane; d < a.D; d += 32) ss = fmaf(src[d], src[d], ss);
        ss = warp_sum(ss);
        const bool is_q = h < a.G;
        const float inv = rsqrtf(ss + a.unit_eps) * (is_q ? q_scale : 1.f);
        float* dst = (is_q ? a.q : a.k) + (size_t)t * qk + (size_t)(is_q ? h : h - a.G) * a.D;
        for (int d = lane; d < a.D; d += 32) dst[d] = src[d] * inv;
    }
    for (int h = threadIdx.x; h < a.H; h += blockDim.x)
        a.beta[(size_t)t * a.H + h] = 1.f / (1.f + expf(-row[channels + h]));
    const int hd = a.H * a.D;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        const float step = gd_softplus(a_proj[(size_t)t * hd + i] + a.dt_bias[i]);
        a.decay[(size_t)t * hd + i] = expf(-a.a_exp[i / a.D] * step);
    }
}

MSTAR_API int mstar_delta_prepare(const float* proj, int row_stride, const void* conv_w,
                                  int weight_dtype, const float* a_proj, const float* dt_bias,
                                  const float* a_exp, const int* token_req, const int* qo_indptr,
                                  const int* slots, const float* state, long long state_stride,
                                  float* q, float* k, float* v, float* beta, float* decay,
                                  int tokens, int H, int G, int D, int VD, int taps, float unit_eps,
                                  void* stream) {
    if (tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || VD <= 0 || taps < 1) return -1;
    const int channels = 2 * G * D + H * VD;
    if (row_stride < channels + H) return -1;
    if (taps > 1 && (!slots || !state)) return -1;
    const size_t smem = sizeof(float) * (size_t)(2 * G * D);
    if (smem > 160 * 1024) return -1;
    DeltaPrepArgs a{proj, row_stride, conv_w, a_proj, dt_bias, a_exp, token_req, qo_indptr, slots,
                    state, state_stride, q, k, v, beta, decay, H, G, D, VD, taps, unit_eps};
    cudaStream_t s = (cudaStream_t)stream;
    static size_t configured_f = 0, configured_b = 0;
    if (weight_dtype == MSTAR_F32) {
        if (smem > 48 * 1024 && smem > configured_f) {
            cudaFuncSetAttribute(delta_prepare_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_f = smem;
        }
        mstar_launch((delta_prepare_kernel<float>), dim3(tokens), dim3(256), smem, s, a);
    } else {
        if (smem > 48 * 1024 && smem > configured_b) {
            cudaFuncSetAttribute(delta_prepare_kernel<bf16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_b = smem;
        }
        mstar_launch((delta_prepare_kernel<bf16>), dim3(tokens), dim3(256), smem, s, a);
    }
    return launch_status();
}

// ------------------------------------------------------------------ scan
#define GD_THREADS 128
#define GD_ROWS 16          // most rows of a column that one lane keeps

struct DeltaScanArgs {
    const float* q;
    const float* k;
    const float* v;
    const float* beta;
    const float* decay;
    const int* qo_indptr;
    const int* slots;
    float* state;               // the slot's S^T part starts at state_offset
    long long state_stride;
    long long state_offset;
    float* out;                 // [tokens][H*VD]
    int H, G, D, VD, chunk;
};

// A block owns GD_THREADS / L value columns of one head of one batch entry; the D rows of a
// column lie on L lanes, lane l keeping rows l, l + L, ...  The token's q, k and decay rows
// (shared by the block's columns) are staged in shared memory, `chunk` tokens at a time.
template <int L>
__global__ void __launch_bounds__(GD_THREADS) delta_scan_kernel(DeltaScanArgs a) {
    extern __shared__ float stage[];          // [chunk][3][D]: q, k, decay
    constexpr int COLS = GD_THREADS / L;
    const int e = blockIdx.x, h = blockIdx.y;
    const int g = h / (a.H / a.G);
    const int lane = threadIdx.x % L;
    const int col = blockIdx.z * COLS + threadIdx.x / L;
    const bool live = col < a.VD;
    const int D = a.D;
    const unsigned long long waited = pdl_wait();
    const float* q = pdl_after(a.q, waited);
    const float* k = pdl_after(a.k, waited);
    const float* v = pdl_after(a.v, waited);
    const float* beta = pdl_after(a.beta, waited);
    const float* decay = pdl_after(a.decay, waited);
    float* state = pdl_after(a.state, waited);
    const int start = a.qo_indptr[e], n = a.qo_indptr[e + 1] - start;
    if (n <= 0) return;
    float* s_col = state + (size_t)a.slots[e] * a.state_stride + a.state_offset +
                   ((size_t)h * a.VD + (live ? col : 0)) * D;
    float s[GD_ROWS];
#pragma unroll
    for (int i = 0; i < GD_ROWS; ++i) {
        const int r = lane + L * i;
        s[i] = (live && r < D) ? s_col[r] : 0.f;
    }
    const int qk = a.G * D, hd = a.H * D, vv = a.H * a.VD;
    for (int base = 0; base < n; base += a.chunk) {
        const int here = min(a.chunk, n - base);
        __syncthreads();
        for (int i = threadIdx.x; i < here * D; i += GD_THREADS) {
            const int j = i / D, d = i - j * D;
            const size_t tok = (size_t)(start + base + j);
            float* dst = stage + (size_t)j * 3 * D;
            dst[d] = q[tok * qk + (size_t)g * D + d];
            dst[D + d] = k[tok * qk + (size_t)g * D + d];
            dst[2 * D + d] = decay[tok * hd + (size_t)h * D + d];
        }
        __syncthreads();
        for (int j = 0; j < here; ++j) {
            const size_t tok = (size_t)(start + base + j);
            const float* qs = stage + (size_t)j * 3 * D;
            const float* ks = qs + D;
            const float* gs = ks + D;
            float r = 0.f, p = 0.f, qkdot = 0.f;
#pragma unroll
            for (int i = 0; i < GD_ROWS; ++i) {
                const int row = lane + L * i;
                if (row < D) {
                    s[i] *= gs[row];
                    r = fmaf(ks[row], s[i], r);
                    p = fmaf(qs[row], s[i], p);
                    qkdot = fmaf(qs[row], ks[row], qkdot);
                }
            }
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) {
                r += __shfl_xor_sync(0xffffffffu, r, o);
                p += __shfl_xor_sync(0xffffffffu, p, o);
                qkdot += __shfl_xor_sync(0xffffffffu, qkdot, o);
            }
            const float vt = live ? v[tok * vv + (size_t)h * a.VD + col] : 0.f;
            const float u = beta[tok * a.H + h] * (vt - r);
#pragma unroll
            for (int i = 0; i < GD_ROWS; ++i) {
                const int row = lane + L * i;
                if (row < D) s[i] = fmaf(ks[row], u, s[i]);
            }
            if (live && lane == 0) a.out[tok * vv + (size_t)h * a.VD + col] = fmaf(qkdot, u, p);
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < GD_ROWS; ++i) {
            const int r = lane + L * i;
            if (r < D) s_col[r] = s[i];
        }
    }
}

MSTAR_API int mstar_delta_scan(const float* q, const float* k, const float* v, const float* beta,
                               const float* decay, const int* qo_indptr, const int* slots,
                               float* state, long long state_stride, long long state_offset,
                               float* out, int entries, int H, int G, int D, int VD, void* stream) {
    if (entries <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || VD <= 0 || D > 32 * GD_ROWS) return -1;
    if (entries > 2147483647 / 1 || H > 65535) return -1;
    int L = 4;
    while (L * GD_ROWS < D) L *= 2;
    // few columns a block where the value size is small, so that the lanes are not idle
    int chunk = 16;
    while (chunk > 1 && (size_t)chunk * 3 * D * sizeof(float) > 40 * 1024) chunk /= 2;
    const size_t smem = (size_t)chunk * 3 * D * sizeof(float);
    DeltaScanArgs a{q, k, v, beta, decay, qo_indptr, slots, state, state_stride, state_offset, out,
                    H, G, D, VD, chunk};
    cudaStream_t s = (cudaStream_t)stream;
    const int cols = GD_THREADS / L;
    dim3 grid(entries, H, (VD + cols - 1) / cols);
    if (grid.z > 65535) return -1;
    switch (L) {
        case 4: mstar_launch((delta_scan_kernel<4>), grid, dim3(GD_THREADS), smem, s, a); break;
        case 8: mstar_launch((delta_scan_kernel<8>), grid, dim3(GD_THREADS), smem, s, a); break;
        case 16: mstar_launch((delta_scan_kernel<16>), grid, dim3(GD_THREADS), smem, s, a); break;
        default: mstar_launch((delta_scan_kernel<32>), grid, dim3(GD_THREADS), smem, s, a); break;
    }
    return launch_status();
}

// ------------------------------------------------------------------ finish
// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * weight[:] * sigmoid(gate[t, h, :]) * scale; a
// warp per (token, head).
template <typename A>
__global__ void delta_finish_kernel(const float* o, const A* gate, int gate_stride,
                                    const float* __restrict__ weight, A* __restrict__ out,
                                    int pairs, int heads, int vdim, float eps, float scale) {
    const unsigned long long waited = pdl_wait();
    o = pdl_after(o, waited);
    gate = pdl_after(gate, waited);
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= pairs) return;
    const int t = pair / heads, h = pair - t * heads;
    const float* row = o + (size_t)pair * vdim;
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) ss = fmaf(row[j], row[j], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)vdim + eps) * scale;
    const A* g = gate + (size_t)t * gate_stride + (size_t)h * vdim;
    for (int j = lane; j < vdim; j += 32)
        out[(size_t)pair * vdim + j] =
            from_float<A>(row[j] * inv * weight[j] / (1.f + expf(-to_float(g[j]))));
}

MSTAR_API int mstar_delta_finish(const float* o, const void* gate, int gate_stride,
                                 const float* weight, void* out, int act_dtype, int tokens,
                                 int heads, int vdim, float eps, float scale, void* stream) {
    if (tokens <= 0) return 0;
    const int pairs = tokens * heads, warps = 4;
    dim3 grid((pairs + warps - 1) / warps);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == MSTAR_F32)
        mstar_launch((delta_finish_kernel<float>), grid, dim3(32 * warps), 0, s, o,
                     (const float*)gate, gate_stride, weight, (float*)out, pairs, heads, vdim, eps,
                     scale);
    else
        mstar_launch((delta_finish_kernel<bf16>), grid, dim3(32 * warps), 0, s, o,
                     (const bf16*)gate, gate_stride, weight, (bf16*)out, pairs, heads, vdim, eps,
                     scale);
    return launch_status();
}
