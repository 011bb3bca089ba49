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
//            u = beta (v - r),  o = p + (q . k) u:  the chain from token to token holds one
//            round of shuffles (r); the read-out's round runs beside the next token.
//   finish   o / rms(o per head) * weight * sigmoid(gate), handed on in the activation type.
//
// A slot is [(taps - 1) * (2 G D + H VD) convolution inputs | S^T as [H][VD][D]], float.
// Everything here is float whatever the activation type.
#include "common.cuh"
#include "mma_util.cuh"

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

// The convolved and activated value of channel c of token t (the `local`-th of its portion).
template <typename W>
__device__ __forceinline__ float delta_conv_silu(const float* row, const float* slot, const W* cw,
                                                 int c, int channels, int local,
                                                 const DeltaPrepArgs& a) {
    const int keep = a.taps - 1;
    float y = 0.f;
    for (int j = 0; j < a.taps; ++j) {
        const int back = keep - j;                       // rows before this token
        const float u = back <= local ? *(row - (ptrdiff_t)back * a.row_stride + c)
                                      : slot[(size_t)(keep + local - back) * channels + c];
        y = fmaf(to_float(cw[(size_t)c * a.taps + j]), u, y);
    }
    return y / (1.f + expf(-y));
}

// A block per token, or, with few tokens, several: a token's work comes in units that a warp
// takes whole (a q head or a k head with its unit norm, the values of a head, the decays of a
// head with its write strength), dealt out among the warps of gridDim.y blocks.
template <typename W>
__global__ void __launch_bounds__(256) delta_prepare_kernel(DeltaPrepArgs a) {
    extern __shared__ float ch[];             // [warps][D] a q or k head after its convolution
    const int t = blockIdx.x;
    const int qk = a.G * a.D, vv = a.H * a.VD, channels = 2 * qk + vv;
    const W* cw = reinterpret_cast<const W*>(a.conv_w);
    const unsigned long long waited = pdl_wait();
    const float* proj = pdl_after(a.proj, waited);
    const float* a_proj = pdl_after(a.a_proj, waited);
    const float* state = pdl_after(a.state, waited);
    const int e = a.token_req[t];
    const int local = t - a.qo_indptr[e];
    const float* slot = a.taps > 1 ? state + (size_t)a.slots[e] * a.state_stride : nullptr;
    const float* row = proj + (size_t)t * a.row_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float* mine = ch + (size_t)warp * a.D;
    const float q_scale = rsqrtf((float)a.D);
    const int units = 2 * a.G + 2 * a.H;
    for (int u = blockIdx.y * nwarps + warp; u < units; u += nwarps * gridDim.y) {
        if (u < 2 * a.G) {                                // a q head, then the k heads
            float ss = 0.f;
            for (int d = lane; d < a.D; d += 32) {
                const float y = delta_conv_silu(row, slot, cw, u * a.D + d, channels, local, a);
                mine[d] = y;
                ss = fmaf(y, y, ss);
            }
            ss = warp_sum(ss);
            const bool is_q = u < a.G;
            const float inv = rsqrtf(ss + a.unit_eps) * (is_q ? q_scale : 1.f);
            float* dst = (is_q ? a.q : a.k) + (size_t)t * qk + (size_t)(is_q ? u : u - a.G) * a.D;
            __syncwarp();
            for (int d = lane; d < a.D; d += 32) dst[d] = mine[d] * inv;
            __syncwarp();
        } else if (u < 2 * a.G + a.H) {                   // the values of a head
            const int h = u - 2 * a.G;
            for (int d = lane; d < a.VD; d += 32)
                a.v[(size_t)t * vv + (size_t)h * a.VD + d] =
                    delta_conv_silu(row, slot, cw, 2 * qk + h * a.VD + d, channels, local, a);
        } else {                                          // the decays of a head, its write strength
            const int h = u - 2 * a.G - a.H;
            const float rate = a.a_exp[h];
            for (int d = lane; d < a.D; d += 32) {
                const size_t i = (size_t)h * a.D + d;
                const float step = gd_softplus(a_proj[(size_t)t * a.H * a.D + i] + a.dt_bias[i]);
                a.decay[(size_t)t * a.H * a.D + i] = expf(-rate * step);
            }
            if (lane == 0) a.beta[(size_t)t * a.H + h] = 1.f / (1.f + expf(-row[channels + h]));
        }
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
    const int threads = 256, warps = threads / 32;
    const size_t smem = sizeof(float) * (size_t)warps * D;
    if (smem > 160 * 1024) return -1;
    DeltaPrepArgs a{proj, row_stride, conv_w, a_proj, dt_bias, a_exp, token_req, qo_indptr, slots,
                    state, state_stride, q, k, v, beta, decay, H, G, D, VD, taps, unit_eps};
    cudaStream_t s = (cudaStream_t)stream;
    // with fewer blocks than SMs a token's units go to several blocks
    const int units = 2 * G + 2 * H;
    int parts = 1;
    if (tokens < device_sm_count()) {
        parts = (units + warps - 1) / warps;
        const int room = (2 * device_sm_count() + tokens - 1) / tokens;
        if (parts > room) parts = room;
        if (parts < 1) parts = 1;
    }
    dim3 grid(tokens, parts);
    static size_t configured_f = 0, configured_b = 0;
    if (weight_dtype == MSTAR_F32) {
        if (smem > 48 * 1024 && smem > configured_f) {
            cudaFuncSetAttribute(delta_prepare_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_f = smem;
        }
        mstar_launch((delta_prepare_kernel<float>), grid, dim3(threads), smem, s, a);
    } else {
        if (smem > 48 * 1024 && smem > configured_b) {
            cudaFuncSetAttribute(delta_prepare_kernel<bf16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_b = smem;
        }
        mstar_launch((delta_prepare_kernel<bf16>), grid, dim3(threads), smem, s, a);
    }
    return launch_status();
}

// ------------------------------------------------------------------ scan
#define GD_THREADS 256
#define GD_ROWS 16          // most rows of a column that one lane keeps
#define GD_CHUNK 16         // tokens staged at a time

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

__device__ __forceinline__ void gd_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(
                     (uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void gd_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(
                     (uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

// A block owns GD_THREADS / L value columns of one head of one batch entry; the D rows of a
// column lie on L lanes, lane l keeping rows l, l + L, ...  What the block's columns share of
// a token (its q, k and decay rows, its write strength) and their values are staged in shared
// memory, `chunk` tokens at a time, the next chunk on its way (cp.async) while this one is
// walked.  Along the chain a token costs the decay, four short sums, the shuffles over the L
// lanes and the write; q . k does not depend on the state and runs beside it.
// A warp that waits for its own shuffles has nothing else to issue, so a token's time is the
// length of its instruction chain: the lanes of a column are as many as leave four rows a lane
// (a whole warp a column from 128 rows on), R is the compiled number of rows a lane.
// VEC: rows are whole 16-byte pieces (D a multiple of 4).
template <int L, int R, bool VEC>
__global__ void __launch_bounds__(GD_THREADS) delta_scan_kernel(DeltaScanArgs a) {
    extern __shared__ __align__(16) float stage[];     // [2][chunk][3 D + COLS + 4]
    constexpr int COLS = GD_THREADS / L;
    const int e = blockIdx.x, h = blockIdx.y;
    const int g = h / (a.H / a.G);
    const int lane = threadIdx.x % L;
    const int mycol = threadIdx.x / L;
    const int col0 = blockIdx.z * COLS;
    const int col = col0 + mycol;
    const bool live = col < a.VD;
    const int D = a.D;
    constexpr int DP = L * R;                          // rows as the lanes see them, zeros past D
    const int per_tok = 3 * DP + COLS + 4;             // q, k, decay, values, beta (+ padding)
    const unsigned long long waited = pdl_wait();
    const float* q = pdl_after(a.q, waited);
    const float* k = pdl_after(a.k, waited);
    const float* v = pdl_after(a.v, waited);
    const float* beta = pdl_after(a.beta, waited);
    const float* decay = pdl_after(a.decay, waited);
    float* state = pdl_after(a.state, waited);
    const int start = a.qo_indptr[e], n = a.qo_indptr[e + 1] - start;
    if (n <= 0) return;
    const int qk = a.G * D, hd = a.H * D, vv = a.H * a.VD;
    const int ncols = min(COLS, a.VD - col0);

    auto fetch = [&](int buf, int base) {
        const int here = min(a.chunk, n - base);
        float* dst0 = stage + (size_t)buf * a.chunk * per_tok;
        // copy i of the chunk is piece r of token j; both move on by fixed steps from copy to
        // copy, so the loop divides nothing
        const int unit = VEC ? 4 : 1;
        const int per = 3 * (D / unit);                 // copies a token
        const int dj = GD_THREADS / per, dr = GD_THREADS % per;
        int j = threadIdx.x / per, r = threadIdx.x % per;
        for (; j < here; j += dj, r += dr) {
            if (r >= per) { r -= per; ++j; if (j >= here) break; }
            const int which = r / (D / unit), d = (r - which * (D / unit)) * unit;
            const size_t tok = (size_t)(start + base + j);
            const float* src = which == 0 ? q + tok * qk + (size_t)g * D + d
                             : which == 1 ? k + tok * qk + (size_t)g * D + d
                                          : decay + tok * hd + (size_t)h * D + d;
            float* dst = dst0 + (size_t)j * per_tok + which * DP + d;
            if constexpr (VEC) gd_copy16(dst, src); else gd_copy4(dst, src);
        }
        for (int i = threadIdx.x; i < here * (ncols + 1); i += GD_THREADS) {
            const int j = i / (ncols + 1), c = i - j * (ncols + 1);
            const size_t tok = (size_t)(start + base + j);
            float* dst = dst0 + (size_t)j * per_tok + 3 * DP;
            if (c < ncols) gd_copy4(dst + c, v + tok * vv + (size_t)h * a.VD + col0 + c);
            else gd_copy4(dst + COLS, beta + tok * a.H + h);
        }
    };

    // rows past D read as zeros (q, k) whatever the chunk: no copy ever writes there
    if (DP > D) {
        for (int i = threadIdx.x; i < 2 * a.chunk * 3 * (DP - D); i += GD_THREADS) {
            const int j = i / (3 * (DP - D)), r = i - j * 3 * (DP - D);
            stage[(size_t)j * per_tok + (r / (DP - D)) * DP + D + r % (DP - D)] = 0.f;
        }
    }
    fetch(0, 0);
    cp_async_commit();
    float* s_col = state + (size_t)a.slots[e] * a.state_stride + a.state_offset +
                   ((size_t)h * a.VD + (live ? col : 0)) * D;
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = lane + L * i;
        s[i] = (live && r < D) ? s_col[r] : 0.f;
    }
    int buf = 0;
    float o_prev = 0.f;                        // the last token's read-out, not yet summed
    int prev_tok = -1;
    for (int base = 0; base < n; base += a.chunk, buf ^= 1) {
        if (base + a.chunk < n) fetch(buf ^ 1, base + a.chunk);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int here = min(a.chunk, n - base);
        const float* tokp = stage + (size_t)buf * a.chunk * per_tok;
        // the rows of the token after this one are read from shared memory while this one's
        // sums go round the lanes
        float qn[R], kn[R], gn[R], vn, bn;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            qn[i] = tokp[lane + L * i];
            kn[i] = tokp[DP + lane + L * i];
            gn[i] = tokp[2 * DP + lane + L * i];
        }
        vn = tokp[3 * DP + mycol];
        bn = tokp[3 * DP + COLS];
        for (int j = 0; j < here; ++j) {
            float qr[R], kr[R], gr[R];
#pragma unroll
            for (int i = 0; i < R; ++i) { qr[i] = qn[i]; kr[i] = kn[i]; gr[i] = gn[i]; }
            const float vt = vn, bt = bn;
            tokp += per_tok;
            if (j + 1 < here) {
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    qn[i] = tokp[lane + L * i];
                    kn[i] = tokp[DP + lane + L * i];
                    gn[i] = tokp[2 * DP + lane + L * i];
                }
                vn = tokp[3 * DP + mycol];
                bn = tokp[3 * DP + COLS];
            }
            float r4[4] = {0.f, 0.f, 0.f, 0.f}, p4[4] = {0.f, 0.f, 0.f, 0.f}, qkdot = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                s[i] *= gr[i];
                r4[i & 3] = fmaf(kr[i], s[i], r4[i & 3]);
                p4[i & 3] = fmaf(qr[i], s[i], p4[i & 3]);
                qkdot = fmaf(qr[i], kr[i], qkdot);
            }
            // a warp issues in order, so a round of shuffles costs its latency wherever it
            // stands: the read-out of the token before goes round together with this token's r
            float r = (r4[0] + r4[1]) + (r4[2] + r4[3]);
            float o_red = o_prev;
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) {
                r += __shfl_xor_sync(0xffffffffu, r, o);
                o_red += __shfl_xor_sync(0xffffffffu, o_red, o);
            }
            if (prev_tok >= 0 && live && lane == 0)
                a.out[(size_t)prev_tok * vv + (size_t)h * a.VD + col] = o_red;
            const float u = bt * (vt - r);
#pragma unroll
            for (int i = 0; i < R; ++i) s[i] = fmaf(kr[i], u, s[i]);
            o_prev = fmaf(qkdot, u, (p4[0] + p4[1]) + (p4[2] + p4[3]));
            prev_tok = start + base + j;
        }
        __syncthreads();                       // the buffer is free for the chunk after next
    }
    cp_async_wait<0>();
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) o_prev += __shfl_xor_sync(0xffffffffu, o_prev, o);
    if (live && lane == 0) a.out[(size_t)prev_tok * vv + (size_t)h * a.VD + col] = o_prev;
    if (live) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int r = lane + L * i;
            if (r < D) s_col[r] = s[i];
        }
    }
}

MSTAR_API int mstar_delta_scan(const float* q, const float* k, const float* v, const float* beta,
                               const float* decay, const int* qo_indptr, const int* slots,
                               float* state, long long state_stride, long long state_offset,
                               float* out, int entries, int max_q_len, int H, int G, int D, int VD,
                               void* stream) {
    if (entries <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || VD <= 0 || D > 32 * GD_ROWS) return -1;
    if (H > 65535) return -1;
    // lanes a column: four rows a lane where that fills at most a warp (MSTAR_DELTA_LANES=8
    // or 16: that many from 128 rows on, for measurements)
    int L = 4;
    while (L < 32 && L * 4 < D) L *= 2;
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("MSTAR_DELTA_LANES");
        forced = e != nullptr ? atoi(e) : 0;
    }
    if (L == 32 && (forced == 8 || forced == 16) && D <= forced * 16) L = forced;
    const int R = D <= L * 4 ? 4 : (D <= L * 8 ? 8 : 16);
    const int cols = GD_THREADS / L;
    // (the staged rows are padded to L * R)
    // tokens staged at a time: 16, fewer where a token's rows are wide or the entries short
    int chunk = GD_CHUNK;
    while (chunk > 1 && (chunk / 2 >= max_q_len ||
                         (size_t)2 * chunk * (3 * L * R + cols + 4) * sizeof(float) > 64 * 1024))
        chunk /= 2;
    const size_t smem = (size_t)2 * chunk * (3 * L * R + cols + 4) * sizeof(float);
    DeltaScanArgs a{q, k, v, beta, decay, qo_indptr, slots, state, state_stride, state_offset, out,
                    H, G, D, VD, chunk};
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(entries, H, (VD + cols - 1) / cols);
    if (grid.z > 65535) return -1;
    // 16-byte copies want whole pieces and aligned rows (the buffers are allocations of their own)
    const bool vec = D % 4 == 0 && (state_offset % 4) == 0 &&
                     ((uintptr_t)q % 16 == 0) && ((uintptr_t)k % 16 == 0) && ((uintptr_t)decay % 16 == 0);
#define GO1(LL, RR, VV)                                                                           \
    do {                                                                                          \
        static size_t configured = 0;                                                             \
        if (smem > 48 * 1024 && smem > configured) {                                              \
            cudaFuncSetAttribute(delta_scan_kernel<LL, RR, VV>,                                   \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
            configured = smem;                                                                    \
        }                                                                                         \
        mstar_launch((delta_scan_kernel<LL, RR, VV>), grid, dim3(GD_THREADS), smem, s, a);        \
    } while (0)
#define GO(LL, RR)                                                                                \
    do {                                                                                          \
        if (vec) GO1(LL, RR, true); else GO1(LL, RR, false);                                      \
    } while (0)
    if (L == 4) GO(4, 4);
    else if (L == 8 && R == 4) GO(8, 4);
    else if (L == 8 && R == 8) GO(8, 8);
    else if (L == 8) GO(8, 16);
    else if (L == 16 && R == 4) GO(16, 4);
    else if (L == 16 && R == 8) GO(16, 8);
    else if (L == 16) GO(16, 16);
    else if (R == 4) GO(32, 4);
    else if (R == 8) GO(32, 8);
    else GO(32, 16);
#undef GO
#undef GO1
    return launch_status();
}

// ------------------------------------------------------------------ scan in pieces of 16 tokens
// Within a piece of C tokens that starts from the state S0, with P_t the product of the decays
// from the piece's first token up to t (per key channel):
//   r_t = (P_t k_t) . S0 + sum_{j<t} A_tj u_j,        A_tj = sum_d k_t[d] k_j[d] prod_{i=j+1..t} g_i[d]
//   u_t = beta_t (v_t - r_t)
//   o_t = (P_t q_t) . S0 + sum_{j<=t} B_tj u_j,       B_tj = sum_d q_t[d] k_j[d] prod_{i=j+1..t} g_i[d]
//   S_C = P_C S0 + sum_j (k_j prod_{i>j} g_i) u_j
// A, B and the decayed rows do not depend on the state or on the value column: a first kernel
// makes them for all pieces side by side (products of decays only, never a quotient).  The scan
// then walks a piece with one dot product per token against S0 (a lane a token), a chain of C
// scalar steps for u, and one pass over the rows for the new state.  All float.
#define GC_TOKENS 16
#define GC_MAX_ROWS 8        // rows of a column a lane keeps: D <= 256

struct DeltaPieceArgs {
    const float* q;
    const float* k;
    const float* decay;
    const int* qo_indptr;
    float* kt;                  // [H][tokens][D]  k_t P_t  (a piece's rows of a head lie together)
    float* qt;                  // [H][tokens][D]  q_t P_t
    float* kh;                  // [H][tokens][D]  k_t prod_{i>t} g_i
    float* pc;                  // [entries][pieces][H][D]  P at the piece's last token
    float* A;                   // [H][tokens][C]
    float* B;                   // [H][tokens][C]
    int H, G, D, max_pieces, tokens;
};

__global__ void __launch_bounds__(128) delta_pieces_kernel(DeltaPieceArgs a) {
    extern __shared__ __align__(16) float sm[];          // k, q, g of the piece: [3][C][D]
    const int piece = blockIdx.x, e = blockIdx.y, h = blockIdx.z;
    const int D = a.D, g_head = h / (a.H / a.G);
    const unsigned long long waited = pdl_wait();
    const float* q = pdl_after(a.q, waited);
    const float* k = pdl_after(a.k, waited);
    const float* decay = pdl_after(a.decay, waited);
    const int start = a.qo_indptr[e], n = a.qo_indptr[e + 1] - start;
    const int base = piece * GC_TOKENS;
    if (base >= n) return;
    const int here = min(GC_TOKENS, n - base);
    float* ks = sm;
    float* qs = ks + GC_TOKENS * D;
    float* gs = qs + GC_TOKENS * D;
    const int qk = a.G * D, hd = a.H * D;
    for (int i = threadIdx.x; i < here * D; i += blockDim.x) {
        const int t = i / D, d = i - t * D;
        const size_t tok = (size_t)(start + base + t);
        ks[i] = k[tok * qk + (size_t)g_head * D + d];
        qs[i] = q[tok * qk + (size_t)g_head * D + d];
        gs[i] = decay[tok * hd + (size_t)h * D + d];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float P = 1.f;
        for (int t = 0; t < here; ++t) {
            P *= gs[t * D + d];
            const size_t o = ((size_t)h * a.tokens + start + base + t) * D + d;
            a.kt[o] = ks[t * D + d] * P;
            a.qt[o] = qs[t * D + d] * P;
        }
        a.pc[(((size_t)e * a.max_pieces + piece) * a.H + h) * D + d] = P;
        float S = 1.f;
        for (int t = here - 1; t >= 0; --t) {
            a.kh[((size_t)h * a.tokens + start + base + t) * D + d] = ks[t * D + d] * S;
            S *= gs[t * D + d];
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int j = warp; j < here; j += nwarps) {
        float w[GC_MAX_ROWS];
        float b = 0.f;
#pragma unroll
        for (int i = 0; i < GC_MAX_ROWS; ++i) {
            const int d = lane + 32 * i;
            w[i] = d < D ? ks[j * D + d] : 0.f;
            if (d < D) b = fmaf(qs[j * D + d], w[i], b);
        }
        b = warp_sum(b);
        if (lane == 0) a.B[((size_t)h * a.tokens + start + base + j) * GC_TOKENS + j] = b;
        for (int t = j + 1; t < here; ++t) {
            float av = 0.f, bv = 0.f;
#pragma unroll
            for (int i = 0; i < GC_MAX_ROWS; ++i) {
                const int d = lane + 32 * i;
                if (d < D) {
                    w[i] *= gs[t * D + d];
                    av = fmaf(ks[t * D + d], w[i], av);
                    bv = fmaf(qs[t * D + d], w[i], bv);
                }
            }
            av = warp_sum(av);
            bv = warp_sum(bv);
            if (lane == 0) {
                const size_t o = ((size_t)h * a.tokens + start + base + t) * GC_TOKENS + j;
                a.A[o] = av;
                a.B[o] = bv;
            }
        }
    }
}

struct DeltaChunkArgs {
    const float* kt;
    const float* qt;
    const float* kh;
    const float* pc;
    const float* A;
    const float* B;
    const float* v;
    const float* beta;
    const int* qo_indptr;
    const int* slots;
    float* state;
    long long state_stride;
    long long state_offset;
    float* out;
    int H, VD, max_pieces, tokens;
};

#define GC_THREADS 256
#define GC_COLS (GC_THREADS / 32)

// R consecutive floats as one access.
template <int R> struct GcVec;
template <> struct GcVec<1> { typedef float T; };
template <> struct GcVec<2> { typedef float2 T; };
template <> struct GcVec<4> { typedef float4 T; };
template <int R> __device__ __forceinline__ void gc_load(const float* p, float (&v)[R]) {
    if constexpr (R == 8) {
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else if constexpr (R == 4) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    } else if constexpr (R == 2) {
        const float2 a = *reinterpret_cast<const float2*>(p);
        v[0] = a.x; v[1] = a.y;
    } else {
        v[0] = p[0];
    }
}
template <int R> __device__ __forceinline__ void gc_store(float* p, const float (&v)[R]) {
    if constexpr (R == 8) {
        reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else if constexpr (R == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else if constexpr (R == 2) {
        *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
    } else {
        p[0] = v[0];
    }
}

// A warp owns a value column of one head of one entry; its D = 32 R rows lie on the 32 lanes,
// R consecutive rows a lane.  Per piece: the column goes to shared memory so that lane
// (t, half) can take token t's two dot products over one half of the rows, four rows an
// access (each lane starts its walk at another place, so that the lanes read different
// banks); the scalar chain u_0 .. u_15 goes round by shuffles with every lane's row of A and B
// in registers; then the new column, R rows an access.
template <int R>
__global__ void __launch_bounds__(GC_THREADS) delta_scan_pieces_kernel(DeltaChunkArgs a) {
    extern __shared__ __align__(16) float sm[];
    constexpr int C = GC_TOKENS, D = 32 * R, CP = C + 1;
    constexpr int per_buf = 3 * C * D + 2 * C * CP + C * GC_COLS + C + D;
    static_assert(per_buf % 4 == 0, "the second buffer starts on a 16-byte boundary");
    float* col_sm = sm + 2 * per_buf;                    // [GC_COLS][D] the columns at a piece's start
    const int e = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = blockIdx.z * GC_COLS, col = col0 + warp;
    const bool live = col < a.VD;
    const int ncols = min(GC_COLS, a.VD - col0);
    const unsigned long long waited = pdl_wait();
    const float* kt = pdl_after(a.kt, waited);
    const float* qt = pdl_after(a.qt, waited);
    const float* kh = pdl_after(a.kh, waited);
    const float* pc = pdl_after(a.pc, waited);
    const float* A = pdl_after(a.A, waited);
    const float* B = pdl_after(a.B, waited);
    const float* v = pdl_after(a.v, waited);
    const float* beta = pdl_after(a.beta, waited);
    float* state = pdl_after(a.state, waited);
    const int start = a.qo_indptr[e], n = a.qo_indptr[e + 1] - start;
    if (n <= 0) return;
    const int vv = a.H * a.VD;

    auto fetch = [&](int buf, int piece) {
        const int base = piece * C;
        const int here = min(C, n - base);
        float* dst = sm + buf * per_buf;
        const size_t first = (size_t)h * a.tokens + start + base;      // the piece's first row
        // the decayed rows of the piece's tokens lie together: one run of here * D floats each
        for (int i = threadIdx.x * 4; i < here * D; i += GC_THREADS * 4) {
            gd_copy16(dst + i, kt + first * D + i);
            gd_copy16(dst + C * D + i, qt + first * D + i);
            gd_copy16(dst + 2 * C * D + i, kh + first * D + i);
        }
        for (int i = threadIdx.x; i < here * C; i += GC_THREADS) {
            const int t = i >> 4, j = i & 15;
            gd_copy4(dst + 3 * C * D + t * CP + j, A + first * C + i);
            gd_copy4(dst + 3 * C * D + C * CP + t * CP + j, B + first * C + i);
        }
        float* to = dst + 3 * C * D + 2 * C * CP;
        for (int i = threadIdx.x; i < here * (ncols + 1); i += GC_THREADS) {
            const int t = i / (ncols + 1), c = i - t * (ncols + 1);
            const size_t tok = (size_t)(start + base + t);
            if (c < ncols) gd_copy4(to + t * GC_COLS + c, v + tok * vv + (size_t)h * a.VD + col0 + c);
            else gd_copy4(to + C * GC_COLS + t, beta + tok * a.H + h);
        }
        const float* pcs = pc + (((size_t)e * a.max_pieces + piece) * a.H + h) * D;
        for (int d = threadIdx.x * 4; d < D; d += GC_THREADS * 4)
            gd_copy16(to + C * GC_COLS + C + d, pcs + d);
    };

    const int pieces = (n + C - 1) / C;
    fetch(0, 0);
    cp_async_commit();
    float* s_col = state + (size_t)a.slots[e] * a.state_stride + a.state_offset +
                   ((size_t)h * a.VD + (live ? col : 0)) * D;
    float s[R];
    gc_load<R>(s_col + lane * R, s);
    float* mycol = col_sm + warp * D;
    const int t = lane & 15, half = lane >> 4;
    constexpr int UNITS = D / 8;                         // 16-byte pieces of half a column
    for (int piece = 0; piece < pieces; ++piece) {
        const int buf = piece & 1;
        if (piece + 1 < pieces) fetch(buf ^ 1, piece + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int here = min(C, n - piece * C);
        const float* bufp = sm + buf * per_buf;
        const float* kts = bufp;
        const float* qts = kts + C * D;
        const float* khs = qts + C * D;
        const float* As = khs + C * D;
        const float* Bs = As + C * CP;
        const float* vs = Bs + C * CP;
        const float* betas = vs + C * GC_COLS;
        const float* pcs = betas + C;
        gc_store<R>(mycol + lane * R, s);                // the column as every lane needs it
        __syncwarp();
        float arow[C], brow[C];
#pragma unroll
        for (int j = 0; j < C; ++j) {
            arow[j] = As[t * CP + j];
            brow[j] = Bs[t * CP + j];
        }
        float r0 = 0.f, p0 = 0.f, r1 = 0.f, p1 = 0.f;
        {
            const float4* kr = reinterpret_cast<const float4*>(kts + t * D) + half * UNITS;
            const float4* qr = reinterpret_cast<const float4*>(qts + t * D) + half * UNITS;
            const float4* sr = reinterpret_cast<const float4*>(mycol) + half * UNITS;
#pragma unroll
            for (int i = 0; i < UNITS; ++i) {
                const int unit = (lane + i) & (UNITS - 1);
                const float4 k4 = kr[unit], q4 = qr[unit], s4 = sr[unit];
                r0 = fmaf(k4.x, s4.x, r0); r1 = fmaf(k4.y, s4.y, r1);
                r0 = fmaf(k4.z, s4.z, r0); r1 = fmaf(k4.w, s4.w, r1);
                p0 = fmaf(q4.x, s4.x, p0); p1 = fmaf(q4.y, s4.y, p1);
                p0 = fmaf(q4.z, s4.z, p0); p1 = fmaf(q4.w, s4.w, p1);
            }
        }
        r0 += r1;
        p0 += p1;
        r0 += __shfl_xor_sync(0xffffffffu, r0, 16);
        p0 += __shfl_xor_sync(0xffffffffu, p0, 16);
        float c = vs[t * GC_COLS + warp] - r0;           // v_t - r_t as far as it is known
        float o = p0;
        float u[C];
#pragma unroll
        for (int j = 0; j < C; ++j) {
            // lane j's c is complete here: every earlier u has been taken off it
            const float uj = betas[j] * __shfl_sync(0xffffffffu, c, j);
            u[j] = j < here ? uj : 0.f;
            if (t > j) c = fmaf(-arow[j], u[j], c);
            if (t >= j) o = fmaf(brow[j], u[j], o);
        }
        if (live && half == 0 && t < here)
            a.out[(size_t)(start + piece * C + t) * vv + (size_t)h * a.VD + col] = o;
        float pcv[R];
        gc_load<R>(pcs + lane * R, pcv);
#pragma unroll
        for (int i = 0; i < R; ++i) s[i] *= pcv[i];
#pragma unroll
        for (int j = 0; j < C; ++j)
            if (j < here) {                              // (rows past the piece are not staged)
                float kv[R];
                gc_load<R>(khs + j * D + lane * R, kv);
#pragma unroll
                for (int i = 0; i < R; ++i) s[i] = fmaf(kv[i], u[j], s[i]);
            }
        __syncthreads();                       // the buffer is free for the piece after next
    }
    cp_async_wait<0>();
    if (live) gc_store<R>(s_col + lane * R, s);
}

// The scan in pieces, for key sizes of 32, 64, 128 or 256 (whole accesses a lane): `work` holds
// 3 * tokens * H * D + entries * max_pieces * H * D + 2 * tokens * H * 16 floats.  Returns 0, a CUDA
// error code, or -1 when the shape is refused.
MSTAR_API int mstar_delta_scan_pieces(const float* q, const float* k, const float* v,
                                      const float* beta, const float* decay, const int* qo_indptr,
                                      const int* slots, float* state, long long state_stride,
                                      long long state_offset, float* out, float* work, int tokens,
                                      int entries, int max_q_len, int H, int G, int D, int VD,
                                      void* stream) {
    if (entries <= 0 || tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || VD <= 0) return -1;
    if (D != 32 && D != 64 && D != 128 && D != 256) return -1;
    if (H > 65535 || entries > 65535 || (state_offset % 4) != 0 || (state_stride % 4) != 0) return -1;
    const int max_pieces = (max_q_len + GC_TOKENS - 1) / GC_TOKENS;
    const size_t thd = (size_t)tokens * H * D;
    DeltaPieceArgs p{q, k, decay, qo_indptr, work, work + thd, work + 2 * thd, work + 3 * thd,
                     nullptr, nullptr, H, G, D, max_pieces, tokens};
    p.A = p.pc + (size_t)entries * max_pieces * H * D;
    p.B = p.A + (size_t)tokens * H * GC_TOKENS;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem1 = (size_t)3 * GC_TOKENS * D * sizeof(float);
    mstar_launch(delta_pieces_kernel, dim3(max_pieces, entries, H), dim3(128), smem1, s, p);
    int code = launch_status();
    if (code != 0) return code;
    DeltaChunkArgs c{p.kt, p.qt, p.kh, p.pc, p.A, p.B, v, beta, qo_indptr, slots, state,
                     state_stride, state_offset, out, H, VD, max_pieces, tokens};
    const int per_buf = 3 * GC_TOKENS * D + 2 * GC_TOKENS * (GC_TOKENS + 1) + GC_TOKENS * GC_COLS +
                        GC_TOKENS + D;
    const size_t smem2 = ((size_t)2 * per_buf + (size_t)GC_COLS * D) * sizeof(float);
    dim3 grid(entries, H, (VD + GC_COLS - 1) / GC_COLS);
    if (grid.z > 65535) return -1;
#define GO(RR)                                                                                    \
    do {                                                                                          \
        static size_t configured = 0;                                                             \
        if (smem2 > 48 * 1024 && smem2 > configured) {                                            \
            cudaFuncSetAttribute(delta_scan_pieces_kernel<RR>,                                    \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);        \
            configured = smem2;                                                                   \
        }                                                                                         \
        mstar_launch((delta_scan_pieces_kernel<RR>), grid, dim3(GC_THREADS), smem2, s, c);        \
    } while (0)
    if (D == 32) GO(1);
    else if (D == 64) GO(2);
    else if (D == 128) GO(4);
    else GO(8);
#undef GO
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
