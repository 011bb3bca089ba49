// Hyper-connections: the residual as S copies x_1 .. x_S per token, float [tokens][S][width].
//
// One kernel does what lies between two sublayers:
//   write   (when the sublayer before left an output y):  every copy at once from the old ones,
//           x_t = sum_s mix[s][t] x_s + out[t] * y,   y = a * y1 (+ b * y2) (+ bias);
//   read    (when a sublayer follows):  u = sum_s in[s] x_s,  then the RMS norm of u with a
//           weight, handed on in the activation type;
//   or sum  (at the model's end):  sum_s x_s of the rows asked for, float.
// With `init` the old copies are all the row init[token] (the embedding output) and the
// copies are written for the first time.  S = 1 with in = mix = 1 is the ordinary residual
// x += out * y.  Sums, the norm and the copies are float for both activation types.
#include "common.cuh"

#define HC_MAX_STREAMS 8
#define HC_THREADS 256

struct HyperArgs {
    float* x;                 // [tokens][S][width], updated in place
    const float* init;        // null, or [tokens][width]
    const void* y1;           // null: nothing to write
    const void* y2;           // null, or a second output added to the first
    const void* y_bias;       // null, or [width] in the weight type
    float a, b;
    const float* mix;         // [S][S], from x to
    const float* out;         // [S], the residual multiplier folded in
    const float* in;          // null (sum mode), or [S]
    const void* norm_weight;  // [width] in the weight type (read mode)
    void* normed;             // [tokens][width] in the activation type (read mode)
    const int* rows;          // sum mode: which tokens; the copies are not written back
    float* sum_out;           // sum mode: [len(rows)][width]
    int S, width;
    float eps;
};

// SM: the compiled capacity for copies (1, 2, 4 or 8), the smallest that holds S.
template <typename A, typename W, int SM>
__global__ void __launch_bounds__(HC_THREADS) hyper_step_kernel(HyperArgs a) {
    extern __shared__ float u_row[];          // [width]: what the norm reads (read mode)
    __shared__ float scratch[32];
    __shared__ float tab[HC_MAX_STREAMS * HC_MAX_STREAMS + 2 * HC_MAX_STREAMS];
    const int S = a.S;
    float* mix = tab;
    float* outw = tab + HC_MAX_STREAMS * HC_MAX_STREAMS;
    float* inw = outw + HC_MAX_STREAMS;
    // the tables are parameters: they may be read before the kernel ahead has ended
    for (int i = threadIdx.x; i < S * S; i += HC_THREADS) mix[i] = a.mix[i];
    for (int i = threadIdx.x; i < S; i += HC_THREADS) {
        outw[i] = a.out[i];
        inw[i] = a.in != nullptr ? a.in[i] : 1.f;
    }
    const unsigned long long waited = pdl_wait();
    float* x = pdl_after(a.x, waited);
    const float* init = pdl_after(a.init, waited);
    const A* y1 = pdl_after(reinterpret_cast<const A*>(a.y1), waited);
    const A* y2 = pdl_after(reinterpret_cast<const A*>(a.y2), waited);
    const W* y_bias = reinterpret_cast<const W*>(a.y_bias);
    const bool sum_mode = a.sum_out != nullptr;
    const int t = sum_mode ? pdl_after(a.rows, waited)[blockIdx.x] : blockIdx.x;
    const bool store = !sum_mode && (init != nullptr || y1 != nullptr);
    __syncthreads();
    float* xt = x + (size_t)t * S * a.width;
    float ss = 0.f;
    // four columns a thread at a time (16-byte accesses) where the width allows, else one
    const int V = (a.width % 4 == 0) ? 4 : 1;
    for (int c = threadIdx.x * V; c < a.width; c += HC_THREADS * V) {
        float old[SM][4], y[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
        if (V == 4) {
            if (init != nullptr) {
                const float4 r = *reinterpret_cast<const float4*>(init + (size_t)t * a.width + c);
#pragma unroll
                for (int s = 0; s < SM; ++s)
                    if (s < S) { old[s][0] = r.x; old[s][1] = r.y; old[s][2] = r.z; old[s][3] = r.w; }
            } else {
#pragma unroll
                for (int s = 0; s < SM; ++s)
                    if (s < S) {
                        const float4 r = *reinterpret_cast<const float4*>(xt + (size_t)s * a.width + c);
                        old[s][0] = r.x; old[s][1] = r.y; old[s][2] = r.z; old[s][3] = r.w;
                    }
            }
        } else {
#pragma unroll
            for (int s = 0; s < SM; ++s)
                if (s < S) old[s][0] = init != nullptr ? init[(size_t)t * a.width + c] : xt[(size_t)s * a.width + c];
        }
        if (y1 != nullptr) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (e < V) {
                    y[e] = a.a * to_float(y1[(size_t)t * a.width + c + e]);
                    if (y2 != nullptr) y[e] = fmaf(a.b, to_float(y2[(size_t)t * a.width + c + e]), y[e]);
                    if (y_bias != nullptr) y[e] += to_float(y_bias[c + e]);
                }
        }
#pragma unroll
        for (int to = 0; to < SM; ++to)
            if (to < S) {
                float nv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (e < V) {
                        float v = old[to][e];
                        if (y1 != nullptr) {
                            v = 0.f;
#pragma unroll
                            for (int s = 0; s < SM; ++s)
                                if (s < S) v = fmaf(mix[s * S + to], old[s][e], v);
                            v = fmaf(outw[to], y[e], v);
                        }
                        nv[e] = v;
                        u[e] = fmaf(inw[to], v, u[e]);
                    }
                if (store) {
                    if (V == 4)
                        *reinterpret_cast<float4*>(xt + (size_t)to * a.width + c) =
                            make_float4(nv[0], nv[1], nv[2], nv[3]);
                    else
                        xt[(size_t)to * a.width + c] = nv[0];
                }
            }
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (e < V) {
                if (sum_mode) {
                    a.sum_out[(size_t)blockIdx.x * a.width + c + e] = u[e];
                } else {
                    u_row[c + e] = u[e];
                    ss = fmaf(u[e], u[e], ss);
                }
            }
    }
    if (sum_mode || a.normed == nullptr) return;
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)a.width + a.eps);
    const W* w = reinterpret_cast<const W*>(a.norm_weight);
    A* dst = reinterpret_cast<A*>(a.normed) + (size_t)t * a.width;
    for (int c = threadIdx.x; c < a.width; c += HC_THREADS)
        dst[c] = from_float<A>(u_row[c] * inv * to_float(w[c]));
}

// rows_or_tokens: blocks to launch (tokens, or the number of rows in sum mode).  Returns 0, a
// CUDA error code, or -1 when the shape is refused.
MSTAR_API int mstar_hyper_step(float* x, const float* init, const void* y1, const void* y2,
                               const void* y_bias, float a, float b, const float* mix,
                               const float* out, const float* in, const void* norm_weight,
                               void* normed, const int* rows, float* sum_out, int blocks,
                               int streams, int width, float eps, int act_dtype, int weight_dtype,
                               void* stream) {
    if (blocks <= 0) return 0;
    if (streams < 1 || streams > HC_MAX_STREAMS || width <= 0) return -1;
    if ((sum_out == nullptr) == (in == nullptr)) return -1;      // one of read and sum
    if (in != nullptr && (norm_weight == nullptr || normed == nullptr)) return -1;
    if (sum_out != nullptr && rows == nullptr) return -1;
    const size_t smem = sum_out != nullptr ? 0 : sizeof(float) * (size_t)width;
    if (smem > 160 * 1024) return -1;
    HyperArgs h{x, init, y1, y2, y_bias, a, b, mix, out, in, norm_weight, normed, rows, sum_out,
                streams, width, eps};
    cudaStream_t s = (cudaStream_t)stream;
#define GO1(A, W, SM)                                                                             \
    do {                                                                                          \
        static size_t configured = 0;                                                             \
        if (smem > 48 * 1024 && smem > configured) {                                              \
            cudaFuncSetAttribute(hyper_step_kernel<A, W, SM>,                                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
            configured = smem;                                                                    \
        }                                                                                         \
        mstar_launch((hyper_step_kernel<A, W, SM>), dim3(blocks), dim3(HC_THREADS), smem, s, h);  \
    } while (0)
#define GO(A, W)                                                                                  \
    do {                                                                                          \
        if (streams == 1) GO1(A, W, 1);                                                           \
        else if (streams == 2) GO1(A, W, 2);                                                      \
        else if (streams <= 4) GO1(A, W, 4);                                                      \
        else GO1(A, W, 8);                                                                        \
    } while (0)
    if (act_dtype == MSTAR_F32) {
        if (weight_dtype == MSTAR_F32) GO(float, float); else GO(float, bf16);
    } else {
        if (weight_dtype == MSTAR_F32) GO(bf16, float); else GO(bf16, bf16);
    }
#undef GO1
#undef GO
    return launch_status();
}

// out = a * y1 + b * y2, float sums, for callers that want the weighted sum of two branch
// outputs as a tensor.
template <typename A>
__global__ void weighted_sum2_kernel(const A* y1, const A* y2, A* __restrict__ out, size_t n, float a,
                                     float b) {
    const unsigned long long waited = pdl_wait();
    y1 = pdl_after(y1, waited);
    y2 = pdl_after(y2, waited);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_float<A>(fmaf(b, to_float(y2[i]), a * to_float(y1[i])));
}

MSTAR_API int mstar_weighted_sum2(const void* y1, const void* y2, void* out, long long n, float a,
                                  float b, int act_dtype, void* stream) {
    if (n <= 0) return 0;
    size_t blocks = ((size_t)n + 255) / 256;
    const size_t most = (size_t)device_sm_count() * 32;
    if (blocks > most) blocks = most;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == MSTAR_F32)
        mstar_launch((weighted_sum2_kernel<float>), dim3((int)blocks), dim3(256), 0, s,
                     (const float*)y1, (const float*)y2, (float*)out, (size_t)n, a, b);
    else
        mstar_launch((weighted_sum2_kernel<bf16>), dim3((int)blocks), dim3(256), 0, s,
                     (const bf16*)y1, (const bf16*)y2, (bf16*)out, (size_t)n, a, b);
    return launch_status();
}
