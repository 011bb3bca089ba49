// Attention over a paged cache of latent rows, for any mix of prompt portions and decoded
// tokens, in float arithmetic on CUDA cores.
//
// A token's cache row holds `rank` latent features c (normalised) followed by `rot` rotated
// key features r that all heads share: [pages, 1, 1, page_size, rank + rot].  With the key
// up-projection folded into the query (a = W_uk[h]^T q_plain, float, made by the caller),
// head h scores key j as (a . c_j + q_rot . r_j) * scale, takes a softmax over the keys the
// token sees (lo..p, lo = max(0, p - window + 1), window 0: lo = 0), and returns the
// probability-weighted sum of the latents, sum_j p_j c_j (float, [tokens, heads, rank]); the
// caller applies the value up-projection W_uv[h] to it.  Scores, softmax statistics,
// probabilities and the output sum are float for both activation types.
//
// Every head reads the same rows, so a block takes one token and a group of heads and
// streams the rows through shared memory once, 32 keys at a time, anchored at the token's
// own first visible key.  With few tokens in a step the keys of a token are shared among
// several blocks (tile i of the token goes to block i modulo the number of splits) whose
// partial sums a second kernel merges in the order of the splits.
//
// The first kernel fills the cache: it normalises the latent part of the down-projection
// (RMS, plain weight), rotates the shared key part and the rotated part of every query head
// (pairs (2i, 2i+1) or (i, i + dims/2), angle = position * freq_i in double precision), and
// writes the row; it also norms a query latent where the queries go through one.
#include "common.cuh"
#include "mma_util.cuh"

#define LAT_TILE 32
#define LAT_THREADS 128
#define LAT_MAX_ACC 32

struct LatentArgs {
    int heads, group, rank, rot, page_size, bt_stride, window;
    int ldq;      // elements between tokens of the rotated query part
    int q_head;   // elements between heads of the rotated query part
    int splits;   // blocks that share a token's keys (tile i goes to block i % splits)
    float scale;
    int row_heads = 0;   // rows a token takes in a block of several tokens (a power of two)
    int num_tokens = 0;
    int cols = 0;        // output columns a block of several tokens makes
};

// A row of D cache elements into floats in shared memory; 16-byte loads where the row allows.
__device__ __forceinline__ void latent_row_to_smem(const bf16* src, float* dst, int D, int lane_id,
                                                   int lanes, bool vec) {
    if (vec) {
        for (int c = lane_id; c < (D >> 3); c += lanes) {
            float v[8];
            load8(src + 8 * c, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[8 * c + i] = v[i];
        }
    } else {
        for (int d = lane_id; d < D; d += lanes) dst[d] = to_float(src[d]);
    }
}
__device__ __forceinline__ void latent_row_to_smem(const float* src, float* dst, int D, int lane_id,
                                                   int lanes, bool vec) {
    if (vec) {
        for (int c = lane_id; c < (D >> 2); c += lanes) {
            const float4 v = reinterpret_cast<const float4*>(src)[c];
            dst[4 * c] = v.x; dst[4 * c + 1] = v.y; dst[4 * c + 2] = v.z; dst[4 * c + 3] = v.w;
        }
    } else {
        for (int d = lane_id; d < D; d += lanes) dst[d] = src[d];
    }
}

// out: [tokens, heads, rank] when splits == 1 (normalised), else the partial sums of a split
// go to part_acc [tokens, heads, splits, rank] with part_ml [tokens, heads, splits, 2] =
// (maximum, sum of exponentials), and the merge kernel finishes.
//
// GP heads a block (4, 8 or 16; fewer are padded with zero queries), CPT = 32 / GP output
// columns a thread: a thread keeps GP x CPT sums in registers.  Queries and probabilities lie
// in shared memory with the heads innermost, so that one 16-byte load brings a key's or a
// feature's values for four heads: a score step is 2 loads for 4 multiply-adds, an output
// step GP / 4 + CPT loads for 32.
template <typename A, int GP>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attention_kernel(const float* __restrict__ q_abs, const A* __restrict__ q_rot,
                        float* __restrict__ out, float* __restrict__ part_acc,
                        float* __restrict__ part_ml, const A* __restrict__ cache,
                        const int* __restrict__ block_table, const int* __restrict__ token_req,
                        const int* __restrict__ cache_pos, LatentArgs a) {
    constexpr int CPT = LAT_MAX_ACC / GP;
    extern __shared__ __align__(16) float smem[];
    const int t = blockIdx.x, h0 = blockIdx.y * a.group, split = blockIdx.z;
    const int G = min(a.group, a.heads - h0);
    const int D = a.rank + a.rot, ldk = D + 1;
    float* qs = smem;                         // [D][GP]
    float* sc = qs + D * GP;                  // [TILE][GP]
    float* m_s = sc + LAT_TILE * GP;          // [GP]
    float* l_s = m_s + GP;
    float* alpha_s = l_s + GP;
    float* tile = alpha_s + GP;               // [TILE][D+1]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned long long waited = pdl_wait();
    q_abs = pdl_after(q_abs, waited);
    q_rot = pdl_after(q_rot, waited);
    cache = pdl_after(cache, waited);

    const int hi = cache_pos[t] + 1;
    const int lo = (a.window > 0 && hi > a.window) ? hi - a.window : 0;
    const int* bt = block_table + (size_t)token_req[t] * a.bt_stride;
    // rows start at multiples of D elements: 16-byte loads need D to be a multiple of 8 (4)
    const bool vec = (D % (16 / (int)sizeof(A)) == 0) && (((uintptr_t)cache & 15) == 0);

    for (int i = tid; i < GP * D; i += LAT_THREADS) {
        const int g = i / D, d = i - g * D;
        float v = 0.f;
        if (g < G)
            v = d < a.rank ? q_abs[((size_t)t * a.heads + h0 + g) * a.rank + d]
                           : to_float(q_rot[(size_t)t * a.ldq + (size_t)(h0 + g) * a.q_head + (d - a.rank)]);
        qs[d * GP + g] = v;
    }
    for (int i = tid; i < GP; i += LAT_THREADS) {
        m_s[i] = -INFINITY;
        l_s[i] = 0.f;
    }
    float acc[CPT][GP];
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int g = 0; g < GP; ++g) acc[c][g] = 0.f;
    __syncthreads();

    for (int base = lo + split * LAT_TILE; base < hi; base += a.splits * LAT_TILE) {
        // a quarter warp per row: 8 lanes stream the row with wide loads.  (Bringing the rows by
        // asynchronous copies through a staging buffer was tried: the buffer leaves one block
        // per SM instead of two, and the kernel took 1.7 times as long.)
        for (int j = tid >> 3; j < LAT_TILE; j += LAT_THREADS >> 3) {
            const int key = base + j;
            float* dst = tile + j * ldk;
            if (key < hi) {
                const int page = bt[key / a.page_size];
                const A* src = cache + ((size_t)page * a.page_size + key % a.page_size) * D;
                latent_row_to_smem(src, dst, D, tid & 7, 8, vec);
            } else {
                for (int d = tid & 7; d < D; d += 8) dst[d] = 0.f;
            }
        }
        __syncthreads();
        // scores: a thread takes one key and four heads
        for (int quad = warp; quad < GP / 4; quad += LAT_THREADS / 32) {
            const float* kv = tile + lane * ldk;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 4
            for (int d = 0; d < D; ++d) {
                const float4 q4 = *reinterpret_cast<const float4*>(qs + d * GP + 4 * quad);
                const float k = kv[d];
                s0 = fmaf(q4.x, k, s0);
                s1 = fmaf(q4.y, k, s1);
                s2 = fmaf(q4.z, k, s2);
                s3 = fmaf(q4.w, k, s3);
            }
            const bool seen = base + lane < hi;
            float4 r;
            r.x = seen ? s0 * a.scale : -INFINITY;
            r.y = seen ? s1 * a.scale : -INFINITY;
            r.z = seen ? s2 * a.scale : -INFINITY;
            r.w = seen ? s3 * a.scale : -INFINITY;
            *reinterpret_cast<float4*>(sc + lane * GP + 4 * quad) = r;
        }
        __syncthreads();
        for (int g = warp; g < GP; g += LAT_THREADS / 32) {
            const float s = sc[lane * GP + g];
            const float m_old = m_s[g];
            const float m_new = fmaxf(m_old, warp_max(s));   // key `base` is always valid
            const float p = expf(s - m_new);
            const float psum = warp_sum(p);
            sc[lane * GP + g] = p;
            if (lane == 0) {
                const float al = expf(m_old - m_new);
                alpha_s[g] = al;
                l_s[g] = l_s[g] * al + psum;
                m_s[g] = m_new;
            }
        }
        __syncthreads();
        {
            float al[GP];
#pragma unroll
            for (int g = 0; g < GP; ++g) al[g] = alpha_s[g];
#pragma unroll
            for (int c = 0; c < CPT; ++c)
#pragma unroll
                for (int g = 0; g < GP; ++g) acc[c][g] *= al[g];
        }
        for (int j = 0; j < LAT_TILE; ++j) {
            float p[GP];
#pragma unroll
            for (int q4 = 0; q4 < GP / 4; ++q4) {
                const float4 v = *reinterpret_cast<const float4*>(sc + j * GP + 4 * q4);
                p[4 * q4] = v.x; p[4 * q4 + 1] = v.y; p[4 * q4 + 2] = v.z; p[4 * q4 + 3] = v.w;
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int d = tid + c * LAT_THREADS;
                const float v = d < a.rank ? tile[j * ldk + d] : 0.f;
#pragma unroll
                for (int g = 0; g < GP; ++g) acc[c][g] = fmaf(p[g], v, acc[c][g]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int d = tid + c * LAT_THREADS;
        if (d >= a.rank) continue;
#pragma unroll
        for (int g = 0; g < GP; ++g) {
            if (g >= G) continue;
            const size_t th = (size_t)t * a.heads + h0 + g;
            if (a.splits == 1) {
                out[th * a.rank + d] = acc[c][g] / l_s[g];
            } else {
                part_acc[(th * a.splits + split) * a.rank + d] = acc[c][g];
                if (d == 0) {
                    part_ml[(th * a.splits + split) * 2] = m_s[g];
                    part_ml[(th * a.splits + split) * 2 + 1] = l_s[g];
                }
            }
        }
    }
}

// The same attention for a bfloat16 cache whose rows are whole k-steps (D a multiple of 16):
// the rows stay bfloat16 in shared memory (asynchronous 16-byte copies), and the scores are
// made on the tensor cores (mma.sync m16n8k16, float sums).  The query's folded part is float:
// it is split into a bfloat16 head and a bfloat16 remainder, each multiplied with the keys, so
// that nothing of it is rounded away.  The softmax and the weighted sum of the latents are as in
// the kernel above: float, a thread keeping GP x CPT sums.
template <int GP>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attention_mma_kernel(const float* __restrict__ q_abs, const bf16* __restrict__ q_rot,
                            float* __restrict__ out, float* __restrict__ part_acc,
                            float* __restrict__ part_ml, const bf16* __restrict__ cache,
                            const int* __restrict__ block_table, const int* __restrict__ token_req,
                            const int* __restrict__ cache_pos, LatentArgs a) {
    constexpr int CPT = LAT_MAX_ACC / GP;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int t = blockIdx.x, h0 = blockIdx.y * a.group, split = blockIdx.z;
    const int G = min(a.group, a.heads - h0);
    const int D = a.rank + a.rot, DP = D + 8;          // 16 bytes of padding: no bank conflicts
    bf16* qh = reinterpret_cast<bf16*>(smem_raw);      // [16][DP] head of the query
    bf16* ql = qh + 16 * DP;                           // [16][DP] remainder
    bf16* tile = ql + 16 * DP;                         // [TILE][DP]
    float* sc = reinterpret_cast<float*>(tile + LAT_TILE * DP);   // [TILE][GP]
    float* m_s = sc + LAT_TILE * GP;
    float* l_s = m_s + GP;
    float* alpha_s = l_s + GP;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned long long waited = pdl_wait();
    q_abs = pdl_after(q_abs, waited);
    q_rot = pdl_after(q_rot, waited);
    cache = pdl_after(cache, waited);

    const int hi = cache_pos[t] + 1;
    const int lo = (a.window > 0 && hi > a.window) ? hi - a.window : 0;
    const int* bt = block_table + (size_t)token_req[t] * a.bt_stride;

    for (int i = tid; i < 16 * D; i += LAT_THREADS) {
        const int g = i / D, d = i - g * D;
        float v = 0.f;
        if (g < G)
            v = d < a.rank ? q_abs[((size_t)t * a.heads + h0 + g) * a.rank + d]
                           : to_float(q_rot[(size_t)t * a.ldq + (size_t)(h0 + g) * a.q_head + (d - a.rank)]);
        const bf16 head = __float2bfloat16_rn(v);
        qh[g * DP + d] = head;
        ql[g * DP + d] = __float2bfloat16_rn(v - __bfloat162float(head));
    }
    for (int i = tid; i < GP; i += LAT_THREADS) {
        m_s[i] = -INFINITY;
        l_s[i] = 0.f;
    }
    float acc[CPT][GP];
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int g = 0; g < GP; ++g) acc[c][g] = 0.f;
    const int chunks = D >> 3;

    for (int base = lo + split * LAT_TILE; base < hi; base += a.splits * LAT_TILE) {
        __syncthreads();                               // the tile of the round before is done with
        for (int idx = tid; idx < LAT_TILE * chunks; idx += LAT_THREADS) {
            const int j = idx / chunks, c = idx - j * chunks;
            const int key = base + j;
            const bf16* src = cache;
            if (key < hi)
                src = cache + ((size_t)bt[key / a.page_size] * a.page_size + key % a.page_size) * D + c * 8;
            cp_async_16(smem_u32(tile + j * DP + c * 8), src, key < hi ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        // scores: warp w takes keys 8w .. 8w+7 and all 16 head rows
        {
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
            const int arow = lane & 15, acol = (lane >> 4) * 8;
            const int brow = warp * 8 + (lane & 7), bcol = ((lane >> 3) & 1) * 8;
            for (int k0 = 0; k0 < D; k0 += 16) {
                uint32_t ah[4], al[4], b0, b1;
                ldmatrix_x4(ah, smem_u32(qh + arow * DP + k0 + acol));
                ldmatrix_x4(al, smem_u32(ql + arow * DP + k0 + acol));
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
                             : "=r"(b0), "=r"(b1)
                             : "r"(smem_u32(tile + brow * DP + k0 + bcol)));
                mma_bf16_16816(s4, ah, b0, b1);
                mma_bf16_16816(s4, al, b0, b1);
            }
            const int g = lane >> 2, j0 = warp * 8 + 2 * (lane & 3);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int head = g + 8 * half;
                if (head < GP) {
                    sc[j0 * GP + head] = base + j0 < hi ? s4[2 * half] * a.scale : -INFINITY;
                    sc[(j0 + 1) * GP + head] = base + j0 + 1 < hi ? s4[2 * half + 1] * a.scale : -INFINITY;
                }
            }
        }
        __syncthreads();
        for (int g = warp; g < GP; g += LAT_THREADS / 32) {
            const float s = sc[lane * GP + g];
            const float m_old = m_s[g];
            const float m_new = fmaxf(m_old, warp_max(s));   // key `base` is always valid
            const float p = expf(s - m_new);
            const float psum = warp_sum(p);
            sc[lane * GP + g] = p;
            if (lane == 0) {
                const float al = expf(m_old - m_new);
                alpha_s[g] = al;
                l_s[g] = l_s[g] * al + psum;
                m_s[g] = m_new;
            }
        }
        __syncthreads();
        {
            float al[GP];
#pragma unroll
            for (int g = 0; g < GP; ++g) al[g] = alpha_s[g];
#pragma unroll
            for (int c = 0; c < CPT; ++c)
#pragma unroll
                for (int g = 0; g < GP; ++g) acc[c][g] *= al[g];
        }
#pragma unroll 2
        for (int j = 0; j < LAT_TILE; ++j) {
            float p[GP];
#pragma unroll
            for (int q4 = 0; q4 < GP / 4; ++q4) {
                const float4 v = *reinterpret_cast<const float4*>(sc + j * GP + 4 * q4);
                p[4 * q4] = v.x; p[4 * q4 + 1] = v.y; p[4 * q4 + 2] = v.z; p[4 * q4 + 3] = v.w;
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int d = tid + c * LAT_THREADS;
                const float v = d < a.rank ? __bfloat162float(tile[j * DP + d]) : 0.f;
#pragma unroll
                for (int g = 0; g < GP; ++g) acc[c][g] = fmaf(p[g], v, acc[c][g]);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int d = tid + c * LAT_THREADS;
        if (d >= a.rank) continue;
#pragma unroll
        for (int g = 0; g < GP; ++g) {
            if (g >= G) continue;
            const size_t th = (size_t)t * a.heads + h0 + g;
            if (a.splits == 1) {
                out[th * a.rank + d] = acc[c][g] / l_s[g];
            } else {
                part_acc[(th * a.splits + split) * a.rank + d] = acc[c][g];
                if (d == 0) {
                    part_ml[(th * a.splits + split) * 2] = m_s[g];
                    part_ml[(th * a.splits + split) * 2 + 1] = l_s[g];
                }
            }
        }
    }
}

// Scores and the weighted sum on the tensor cores, for a bfloat16 cache with D a multiple of 16
// and a rank that is a multiple of 32.  A block takes one token and up to 16 heads (the rows of
// the m16n8k16 tiles).  The probabilities are float; for the product with the latents each is
// written as the sum of three bfloat16 numbers (head, middle, tail: 3 x 8 bits hold a float's
// 24-bit mantissa exactly), and the three products are added in the float accumulator, so the
// weighted sum is that of the float probabilities.  Warp w owns the columns
// [w rank/4, (w+1) rank/4) of the output: NB tiles of 8 columns, 4 floats a thread each.
template <int NB>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attention_tc_kernel(const float* __restrict__ q_abs, const bf16* __restrict__ q_rot,
                           float* __restrict__ out, float* __restrict__ part_acc,
                           float* __restrict__ part_ml, const bf16* __restrict__ cache,
                           const int* __restrict__ block_table, const int* __restrict__ token_req,
                           const int* __restrict__ cache_pos, LatentArgs a) {
    constexpr int PK = LAT_TILE + 8;                   // row stride of the probability tiles
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int t = blockIdx.x, h0 = blockIdx.y * a.group, split = blockIdx.z;
    const int G = min(a.group, a.heads - h0);
    const int D = a.rank + a.rot, DP = D + 8;
    bf16* qh = reinterpret_cast<bf16*>(smem_raw);      // [16][DP] head of the query
    bf16* ql = qh + 16 * DP;                           // [16][DP] remainder
    bf16* tile = ql + 16 * DP;                         // [TILE][DP]
    bf16* ph = tile + LAT_TILE * DP;                   // [3][16][PK] probabilities: head, middle, tail
    float* sc = reinterpret_cast<float*>(ph + 3 * 16 * PK);   // [TILE][16]
    float* m_s = sc + LAT_TILE * 16;
    float* l_s = m_s + 16;
    float* alpha_s = l_s + 16;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned long long waited = pdl_wait();
    q_abs = pdl_after(q_abs, waited);
    q_rot = pdl_after(q_rot, waited);
    cache = pdl_after(cache, waited);

    const int hi = cache_pos[t] + 1;
    const int lo = (a.window > 0 && hi > a.window) ? hi - a.window : 0;
    const int* bt = block_table + (size_t)token_req[t] * a.bt_stride;

    for (int i = tid; i < 16 * D; i += LAT_THREADS) {
        const int g = i / D, d = i - g * D;
        float v = 0.f;
        if (g < G)
            v = d < a.rank ? q_abs[((size_t)t * a.heads + h0 + g) * a.rank + d]
                           : to_float(q_rot[(size_t)t * a.ldq + (size_t)(h0 + g) * a.q_head + (d - a.rank)]);
        const bf16 head = __float2bfloat16_rn(v);
        qh[g * DP + d] = head;
        ql[g * DP + d] = __float2bfloat16_rn(v - __bfloat162float(head));
    }
    for (int i = tid; i < 3 * 16 * PK; i += LAT_THREADS) ph[i] = __float2bfloat16_rn(0.f);
    for (int i = tid; i < 16; i += LAT_THREADS) {
        m_s[i] = -INFINITY;
        l_s[i] = 0.f;
        alpha_s[i] = 1.f;
    }
    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;
    const int chunks = D >> 3;
    const int nb_warp = a.rank >> 5;                   // tiles of 8 columns a warp (<= NB)
    const int col_warp = warp * nb_warp * 8;
    const int g = lane >> 2, t4 = lane & 3;

    for (int base = lo + split * LAT_TILE; base < hi; base += a.splits * LAT_TILE) {
        __syncthreads();                               // the tile of the round before is done with
        // a warp per row (the row's address once), lanes over its 16-byte chunks
        for (int j = warp; j < LAT_TILE; j += LAT_THREADS / 32) {
            const int key = base + j;
            const bool seen = key < hi;
            const bf16* src = cache;
            if (seen) src = cache + ((size_t)bt[key / a.page_size] * a.page_size + key % a.page_size) * D;
            for (int c = lane; c < chunks; c += 32)
                cp_async_16(smem_u32(tile + j * DP + c * 8), seen ? src + c * 8 : cache, seen ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        // scores: warp w takes keys 8w .. 8w+7 and all 16 head rows
        {
            // four chains of products (head / remainder of the query, even / odd k-step), so
            // that a product does not wait for the one before it
            float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
            float sc2[4] = {0.f, 0.f, 0.f, 0.f}, sd[4] = {0.f, 0.f, 0.f, 0.f};
            const int arow = lane & 15, acol = (lane >> 4) * 8;
            const int brow = warp * 8 + (lane & 7), bcol = ((lane >> 3) & 1) * 8;
            for (int k0 = 0; k0 < D; k0 += 32) {
                uint32_t ah[4], al[4], b0, b1;
                ldmatrix_x4(ah, smem_u32(qh + arow * DP + k0 + acol));
                ldmatrix_x4(al, smem_u32(ql + arow * DP + k0 + acol));
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
                             : "=r"(b0), "=r"(b1)
                             : "r"(smem_u32(tile + brow * DP + k0 + bcol)));
                mma_bf16_16816(sa, ah, b0, b1);
                mma_bf16_16816(sb, al, b0, b1);
                if (k0 + 16 < D) {
                    ldmatrix_x4(ah, smem_u32(qh + arow * DP + k0 + 16 + acol));
                    ldmatrix_x4(al, smem_u32(ql + arow * DP + k0 + 16 + acol));
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
                                 : "=r"(b0), "=r"(b1)
                                 : "r"(smem_u32(tile + brow * DP + k0 + 16 + bcol)));
                    mma_bf16_16816(sc2, ah, b0, b1);
                    mma_bf16_16816(sd, al, b0, b1);
                }
            }
            float s4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) s4[i] = (sa[i] + sc2[i]) + (sb[i] + sd[i]);
            const int j0 = warp * 8 + 2 * t4;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int head = g + 8 * half;
                sc[j0 * 16 + head] = base + j0 < hi ? s4[2 * half] * a.scale : -INFINITY;
                sc[(j0 + 1) * 16 + head] = base + j0 + 1 < hi ? s4[2 * half + 1] * a.scale : -INFINITY;
            }
        }
        __syncthreads();
        // softmax of the tile, a warp per head; the probabilities in three bfloat16 parts
        for (int hd = warp; hd < G; hd += LAT_THREADS / 32) {
            const float sv = sc[lane * 16 + hd];
            const float m_old = m_s[hd];
            const float m_new = fmaxf(m_old, warp_max(sv));  // key `base` is always valid
            const float p = expf(sv - m_new);
            const float psum = warp_sum(p);
            const bf16 p0 = __float2bfloat16_rn(p);
            const float r1 = p - __bfloat162float(p0);
            const bf16 p1 = __float2bfloat16_rn(r1);
            const bf16 p2 = __float2bfloat16_rn(r1 - __bfloat162float(p1));
            ph[hd * PK + lane] = p0;
            ph[(16 + hd) * PK + lane] = p1;
            ph[(32 + hd) * PK + lane] = p2;
            if (lane == 0) {
                const float al = expf(m_old - m_new);
                alpha_s[hd] = al;
                l_s[hd] = l_s[hd] * al + psum;
                m_s[hd] = m_new;
            }
        }
        __syncthreads();
        // weighted sum: acc = alpha acc + P V, V the first `rank` features of the rows
        {
            const float a_lo = alpha_s[g], a_hi = alpha_s[g + 8];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                acc[nb][0] *= a_lo; acc[nb][1] *= a_lo;
                acc[nb][2] *= a_hi; acc[nb][3] *= a_hi;
            }
            const int arow = lane & 15, acol = (lane >> 4) * 8;
            const int vrow = (lane & 7) + ((lane >> 3) & 1) * 8, vcol = (lane >> 4) * 8;
#pragma unroll
            for (int k0 = 0; k0 < LAT_TILE; k0 += 16) {
                uint32_t p0[4], p1[4], p2[4];
                ldmatrix_x4(p0, smem_u32(ph + arow * PK + k0 + acol));
                ldmatrix_x4(p1, smem_u32(ph + (16 + arow) * PK + k0 + acol));
                ldmatrix_x4(p2, smem_u32(ph + (32 + arow) * PK + k0 + acol));
#pragma unroll
                for (int nb = 0; nb < NB; nb += 2) {
                    if (nb < nb_warp) {
                        uint32_t v[4];
                        ldmatrix_x4_trans(v, smem_u32(tile + (k0 + vrow) * DP + col_warp + nb * 8 + vcol));
                        mma_bf16_16816(acc[nb], p2, v[0], v[1]);
                        mma_bf16_16816(acc[nb], p1, v[0], v[1]);
                        mma_bf16_16816(acc[nb], p0, v[0], v[1]);
                        if (nb + 1 < NB) {
                            mma_bf16_16816(acc[nb + 1 < NB ? nb + 1 : nb], p2, v[2], v[3]);
                            mma_bf16_16816(acc[nb + 1 < NB ? nb + 1 : nb], p1, v[2], v[3]);
                            mma_bf16_16816(acc[nb + 1 < NB ? nb + 1 : nb], p0, v[2], v[3]);
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        if (nb >= nb_warp) continue;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int hd = g + 8 * half;
            if (hd >= G) continue;
            const size_t th = (size_t)t * a.heads + h0 + hd;
            const int d = col_warp + nb * 8 + 2 * t4;
            const float v0 = acc[nb][2 * half], v1 = acc[nb][2 * half + 1];
            if (a.splits == 1) {
                const float inv = 1.f / l_s[hd];
                out[th * a.rank + d] = v0 * inv;
                out[th * a.rank + d + 1] = v1 * inv;
            } else {
                part_acc[(th * a.splits + split) * a.rank + d] = v0;
                part_acc[(th * a.splits + split) * a.rank + d + 1] = v1;
                if (d == 0) {
                    part_ml[(th * a.splits + split) * 2] = m_s[hd];
                    part_ml[(th * a.splits + split) * 2 + 1] = l_s[hd];
                }
            }
        }
    }
}

// The same arithmetic for prompts: a block takes several tokens that follow one another in the
// step, 64 rows of (token, head), a token's heads padded to `row_heads` rows, so that a tile of
// keys is fetched once for all of them and no row of a product tile is empty.  Warp w owns rows
// 16w .. 16w+15 from the scores to the output: its scores of a tile's 32 keys stay in the
// accumulator registers, the softmax runs there (a row's keys lie in the four lanes of a quad),
// and the probabilities go into the second product as its A fragments, again in three bfloat16
// parts, so nothing but the queries and the keys passes through shared memory and a round has
// two barriers (around the tile's copy).  Every row masks by its own token's position
// (lo <= key < hi).  Tokens of one request share a block table; where a block's tokens belong
// to several requests it walks them request by request, the other rows idle.  A block makes
// `cols` of the output's columns (blockIdx.z: a wide latent is shared among two blocks, each
// scoring for itself).  Keys are never shared among blocks here.
__device__ __forceinline__ uint32_t pack_bf16(bf16 lo, bf16 hi) {
    return (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
}

template <int NBT>
__global__ void __launch_bounds__(128, 1)
latent_attention_rows_kernel(const float* __restrict__ q_abs, const bf16* __restrict__ q_rot,
                             float* __restrict__ out, const bf16* __restrict__ cache,
                             const int* __restrict__ block_table, const int* __restrict__ token_req,
                             const int* __restrict__ cache_pos, LatentArgs a) {
    constexpr int ROWS = 64, THREADS = 128;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int GP = a.row_heads, TPB = ROWS / GP;
    const int t0 = blockIdx.x * TPB, h0 = blockIdx.y * a.group;
    const int G = min(a.group, a.heads - h0);
    const int ntok = min(TPB, a.num_tokens - t0);
    const int D = a.rank + a.rot, DP = D + 8;
    const int col0 = blockIdx.z * a.cols;
    const int nb_cols = min(a.cols, a.rank - col0) >> 3;     // tiles of 8 columns, an even count
    bf16* qh = reinterpret_cast<bf16*>(smem_raw);      // [ROWS][DP] head of the query
    bf16* ql = qh + ROWS * DP;                         // [ROWS][DP] remainder
    bf16* tile = ql + ROWS * DP;                       // [TILE][DP]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned long long waited = pdl_wait();
    q_abs = pdl_after(q_abs, waited);
    q_rot = pdl_after(q_rot, waited);
    cache = pdl_after(cache, waited);

    for (int i = tid; i < ROWS * D; i += THREADS) {
        const int r = i / D, d = i - r * D;
        const int tk = r / GP, hd = r - tk * GP;
        float v = 0.f;
        if (tk < ntok && hd < G) {
            const size_t t = (size_t)(t0 + tk);
            v = d < a.rank ? q_abs[(t * a.heads + h0 + hd) * a.rank + d]
                           : to_float(q_rot[t * a.ldq + (size_t)(h0 + hd) * a.q_head + (d - a.rank)]);
        }
        const bf16 head = __float2bfloat16_rn(v);
        qh[r * DP + d] = head;
        ql[r * DP + d] = __float2bfloat16_rn(v - __bfloat162float(head));
    }
    const int chunks = D >> 3;
    const int g = lane >> 2, t4 = lane & 3;
    int row_tk[2], row_hd[2];                          // this thread's rows: 16 warp + g, + 8
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + g + 8 * i;
        row_tk[i] = r / GP;
        row_hd[i] = r - row_tk[i] * GP;
    }
    float acc[NBT][4];

    for (int s0 = 0; s0 < ntok;) {
        // tokens s0 .. s1-1 of the block belong to one request
        const int req = token_req[t0 + s0];
        int s1 = s0 + 1;
        while (s1 < ntok && token_req[t0 + s1] == req) ++s1;
        int lo_min = 0x7fffffff, hi_max = 0;
        for (int tk = s0; tk < s1; ++tk) {
            const int hi = cache_pos[t0 + tk] + 1;
            const int lo = (a.window > 0 && hi > a.window) ? hi - a.window : 0;
            lo_min = min(lo_min, lo);
            hi_max = max(hi_max, hi);
        }
        const int* bt = block_table + (size_t)req * a.bt_stride;
        int lo_r[2], hi_r[2];                          // hi 0: an idle row
        int warp_lo = 0x7fffffff, warp_hi = 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            lo_r[i] = hi_r[i] = 0;
            if (row_tk[i] >= s0 && row_tk[i] < s1 && row_hd[i] < G) {
                hi_r[i] = cache_pos[t0 + row_tk[i]] + 1;
                lo_r[i] = (a.window > 0 && hi_r[i] > a.window) ? hi_r[i] - a.window : 0;
                warp_lo = min(warp_lo, lo_r[i]);
                warp_hi = max(warp_hi, hi_r[i]);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            warp_lo = min(warp_lo, __shfl_xor_sync(0xffffffffu, warp_lo, o));
            warp_hi = max(warp_hi, __shfl_xor_sync(0xffffffffu, warp_hi, o));
        }
        float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
#pragma unroll
        for (int nb = 0; nb < NBT; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;

        for (int base = lo_min; base < hi_max; base += LAT_TILE) {
            __syncthreads();                           // the tile of the round before is done with
            for (int j = warp; j < LAT_TILE; j += THREADS / 32) {
                const int key = base + j;
                const bool seen = key < hi_max;
                const bf16* src = cache;
                if (seen) src = cache + ((size_t)bt[key / a.page_size] * a.page_size + key % a.page_size) * D;
                for (int c = lane; c < chunks; c += 32)
                    cp_async_16(smem_u32(tile + j * DP + c * 8), seen ? src + c * 8 : cache, seen ? 16 : 0);
            }
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
            if (base >= warp_hi || base + LAT_TILE <= warp_lo) continue;   // nothing for these rows
            // scores of the warp's 16 rows and the tile's 32 keys: four tiles of 8 keys
            // (the head and the remainder of the query in chains of their own, so that a
            // product does not wait for the one before it)
            float sc[4][4], sr[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) sc[j][i] = sr[j][i] = 0.f;
            {
                const int arow = warp * 16 + (lane & 15), acol = (lane >> 4) * 8;
                const int krow = (lane & 7) + ((lane >> 4) << 3), kcol = ((lane >> 3) & 1) * 8;
                const uint32_t qh_at = smem_u32(qh + arow * DP + acol), ql_at = smem_u32(ql + arow * DP + acol);
                const uint32_t k_at = smem_u32(tile + krow * DP + kcol);
                for (int k0 = 0; k0 < D; k0 += 16) {
                    uint32_t ah[4], al[4], k01[4], k23[4];
                    ldmatrix_x4(ah, qh_at + 2 * k0);
                    ldmatrix_x4(al, ql_at + 2 * k0);
                    ldmatrix_x4(k01, k_at + 2 * k0);
                    ldmatrix_x4(k23, k_at + 2 * (16 * DP + k0));
                    mma_bf16_16816(sc[0], ah, k01[0], k01[1]);
                    mma_bf16_16816(sc[1], ah, k01[2], k01[3]);
                    mma_bf16_16816(sc[2], ah, k23[0], k23[1]);
                    mma_bf16_16816(sc[3], ah, k23[2], k23[3]);
                    mma_bf16_16816(sr[0], al, k01[0], k01[1]);
                    mma_bf16_16816(sr[1], al, k01[2], k01[3]);
                    mma_bf16_16816(sr[2], al, k23[0], k23[1]);
                    mma_bf16_16816(sr[3], al, k23[2], k23[3]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) sc[j][i] += sr[j][i];
            }
            // mask, softmax of the tile in registers: row i of the thread has its keys in
            // sc[j][2 i], sc[j][2 i + 1] (keys base + 8 j + 2 t4, + 1) of the quad's four lanes
            uint32_t pa[2][3][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int key = base + 8 * j + 2 * t4 + c;
                        const float v = (key >= lo_r[i] && key < hi_r[i]) ? sc[j][2 * i + c] * a.scale
                                                                         : -INFINITY;
                        sc[j][2 * i + c] = v;
                        mx = fmaxf(mx, v);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_r[i], mx);
                const bool none = m_new == -INFINITY;  // the row has seen no key yet
                const float m_use = none ? 0.f : m_new;
                const float alpha = none ? 1.f : expf(m_r[i] - m_new);
                m_r[i] = m_new;
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    bf16 part[3][2];
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const float p = expf(sc[j][2 * i + c] - m_use);
                        sum += p;
                        part[0][c] = __float2bfloat16_rn(p);
                        const float r1 = p - __bfloat162float(part[0][c]);
                        part[1][c] = __float2bfloat16_rn(r1);
                        part[2][c] = __float2bfloat16_rn(r1 - __bfloat162float(part[1][c]));
                    }
                    // A fragment of the k-step j / 2: register i (+ 2 for the upper 8 keys)
#pragma unroll
                    for (int q = 0; q < 3; ++q) pa[j >> 1][q][i + 2 * (j & 1)] = pack_bf16(part[q][0], part[q][1]);
                }
                l_r[i] = l_r[i] * alpha + sum;
#pragma unroll
                for (int nb = 0; nb < NBT; ++nb) {
                    acc[nb][2 * i] *= alpha;
                    acc[nb][2 * i + 1] *= alpha;
                }
            }
            // weighted sum: acc += P V over the block's columns
            {
                const int vrow = (lane & 7) + ((lane >> 3) & 1) * 8, vcol = (lane >> 4) * 8;
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    // two pairs of column tiles at a time: four sums take the three parts in
                    // turn, so that a product does not wait for the one before it
#pragma unroll
                    for (int nb = 0; nb < NBT; nb += 4) {
                        if (nb < nb_cols) {
                            uint32_t v[4], w[4];
                            const bool two = nb + 2 < nb_cols;
                            const uint32_t at = smem_u32(tile + (16 * kk + vrow) * DP + col0 + nb * 8 + vcol);
                            ldmatrix_x4_trans(v, at);
                            ldmatrix_x4_trans(w, two ? at + 32 : at);
#pragma unroll
                            for (int q = 2; q >= 0; --q) {
                                mma_bf16_16816(acc[nb], pa[kk][q], v[0], v[1]);
                                mma_bf16_16816(acc[nb + 1], pa[kk][q], v[2], v[3]);
                                if (two) {
                                    mma_bf16_16816(acc[nb + 2], pa[kk][q], w[0], w[1]);
                                    mma_bf16_16816(acc[nb + 3], pa[kk][q], w[2], w[3]);
                                }
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float l = l_r[i];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            if (hi_r[i] == 0) continue;
            const float inv = 1.f / l;
            const size_t th = (size_t)(t0 + row_tk[i]) * a.heads + h0 + row_hd[i];
            float* dst = out + th * a.rank + col0 + 2 * t4;
#pragma unroll
            for (int nb = 0; nb < NBT; ++nb)
                if (nb < nb_cols)
                    *reinterpret_cast<float2*>(dst + nb * 8) =
                        make_float2(acc[nb][2 * i] * inv, acc[nb][2 * i + 1] * inv);
        }
        s0 = s1;
    }
}

// out[t, h, :] = sum_s exp(m_s - M) acc_s / sum_s exp(m_s - M) l_s, in the order of the splits.
// A split that saw no key has l = 0 and m = -inf and adds nothing.
__global__ void latent_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    float* __restrict__ out, int rank, int splits) {
    __shared__ float w_s[32];                  // exp(m_s - M) of every split (at most 32)
    __shared__ float inv_l;
    const unsigned long long waited = pdl_wait();
    part_acc = pdl_after(part_acc, waited);
    part_ml = pdl_after(part_ml, waited);
    const size_t th = blockIdx.x;
    if (threadIdx.x < 32) {
        const int sp = threadIdx.x;
        const float m = sp < splits ? part_ml[(th * splits + sp) * 2] : -INFINITY;
        const float l = sp < splits ? part_ml[(th * splits + sp) * 2 + 1] : 0.f;
        const float M = warp_max(m);
        const float w = m > -INFINITY ? expf(m - M) : 0.f;
        // the sum over the splits in their order, by one lane
        w_s[sp] = w;
        const float wl = w * l;
        float L = 0.f;
        for (int i = 0; i < splits; ++i) L += __shfl_sync(0xffffffffu, wl, i);
        if (sp == 0) inv_l = 1.f / L;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float sum = 0.f;
        for (int sp = 0; sp < splits; ++sp)
            sum = fmaf(w_s[sp], part_acc[(th * splits + sp) * rank + d], sum);
        out[th * rank + d] = sum * inv_l;
    }
}

template <typename A, int GP>
static int launch_latent(const float* q_abs, const void* q_rot, float* out, float* part_acc,
                         float* part_ml, const void* cache, const int* block_table,
                         const int* token_req, const int* cache_pos, const LatentArgs& a, dim3 grid,
                         size_t smem, cudaStream_t s) {
    static size_t configured = 0;             // largest dynamic shared memory set so far
    if (smem > 48 * 1024 && smem > configured) {
        cudaFuncSetAttribute(latent_attention_kernel<A, GP>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = smem;
    }
    mstar_launch((latent_attention_kernel<A, GP>), grid, dim3(LAT_THREADS), smem, s, q_abs,
                 (const A*)q_rot, out, part_acc, part_ml, (const A*)cache, block_table, token_req,
                 cache_pos, a);
    return 0;
}

// `group` heads a block (0: as many as fit), `splits` > 1 shares a token's keys among that many
// blocks (`scratch`: float [tokens * heads * splits * (rank + 2)]).  Returns 0, a CUDA error
// code, or -1 when the shape is refused (rank > 1024, or a tile of rows that does not fit
// shared memory).
MSTAR_API int mstar_latent_attention(const float* q_abs, const void* q_rot, int ldq, int q_head,
                                     float* out, const void* cache, const int* block_table,
                                     int bt_stride, const int* token_req, const int* cache_pos,
                                     int num_tokens, int heads, int rank, int rot, int page_size,
                                     int window, float scale, int act_dtype, int group, int splits,
                                     float* scratch, int portions, void* stream) {
    if (num_tokens <= 0) return 0;
    if (heads <= 0 || rank <= 0 || rot < 0 || rank > 8 * LAT_THREADS) return -1;
    // heads a block: a thread has 32 sums for GP heads x (rank / 128) columns
    const int most = rank <= 2 * LAT_THREADS ? 16 : (rank <= 4 * LAT_THREADS ? 8 : 4);
    if (group <= 0 || group > most) group = most;
    if (group > heads) group = heads;
    const int gp = group <= 4 ? 4 : (group <= 8 ? 8 : 16);
    if (splits < 1) splits = 1;
    if (splits > 32) return -1;               // the merge kernel takes up to 32
    if (splits > 1 && scratch == nullptr) return -1;
    const int D = rank + rot;
    const size_t smem = sizeof(float) * ((size_t)gp * D + (size_t)LAT_TILE * (D + 1) +
                                   (size_t)gp * LAT_TILE + 3 * (size_t)gp);
    if (smem > 200 * 1024) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    LatentArgs a{heads, group, rank, rot, page_size, bt_stride, window, ldq, q_head, splits, scale};
    dim3 grid(num_tokens, (heads + group - 1) / group, splits);
    float* part_acc = scratch;
    float* part_ml = scratch == nullptr ? nullptr : scratch + (size_t)num_tokens * heads * splits * rank;
    // a bfloat16 cache with rows of whole k-steps: scores on the tensor cores
    // (MSTAR_LATENT_ATTENTION=cores keeps the kernel above)
    static int cores_only = -1;
    if (cores_only < 0) {
        const char* e = getenv("MSTAR_LATENT_ATTENTION");
        cores_only = (e != nullptr && e[0] == 'c') ? 1 : 0;
    }
    // ... and the weighted sum as well where the rank is a multiple of 32 (a block then takes
    // up to 16 heads whatever `group` asks for; MSTAR_LATENT_ATTENTION=scores keeps the sum on
    // the CUDA cores)
    static int scores_only = -1;
    if (scores_only < 0) {
        const char* e = getenv("MSTAR_LATENT_ATTENTION");
        scores_only = (e != nullptr && e[0] == 's') ? 1 : 0;
    }
    // `portions`: the step's tokens come in runs of one request (prompt portions), so a block
    // takes the rows of several tokens (MSTAR_LATENT_ATTENTION=token keeps a token a block)
    static int token_only = -1;
    if (token_only < 0) {
        const char* e = getenv("MSTAR_LATENT_ATTENTION");
        token_only = (e != nullptr && e[0] == 't') ? 1 : 0;
    }
    if (portions && splits == 1 && act_dtype == MSTAR_BF16 && D % 16 == 0 && rank % 32 == 0 &&
        rank <= 256 && ((uintptr_t)cache & 15) == 0 && ((uintptr_t)out & 7) == 0 && !cores_only &&
        !scores_only && !token_only) {
        constexpr int ROWS = 64;
        const int tc_group = heads < 16 ? heads : 16;
        int row_heads = 1;
        while (row_heads < tc_group) row_heads *= 2;
        LatentArgs b = a;
        b.group = tc_group;
        b.row_heads = row_heads;
        b.num_tokens = num_tokens;
        // a block makes all of a row's columns: sharing them among blocks (each scoring for
        // itself) cost more than the warps it added brought, at every rank tried
        const int shares = 1;
        b.cols = rank / shares;                        // a multiple of 16
        const int per_block = ROWS / row_heads;
        dim3 rows_grid((num_tokens + per_block - 1) / per_block, (heads + tc_group - 1) / tc_group,
                       shares);
        const size_t smem_rows = sizeof(bf16) * (size_t)(2 * ROWS + LAT_TILE) * (D + 8);
        if (smem_rows <= 200 * 1024) {
#define GO_ROWS(NBT)                                                                              \
    {                                                                                             \
        static size_t configured = 0;                                                             \
        if (smem_rows > 48 * 1024 && smem_rows > configured) {                                    \
            cudaFuncSetAttribute(latent_attention_rows_kernel<NBT>,                               \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rows);    \
            configured = smem_rows;                                                               \
        }                                                                                         \
        mstar_launch((latent_attention_rows_kernel<NBT>), rows_grid, dim3(128), smem_rows, s,     \
                     q_abs, (const bf16*)q_rot, out, (const bf16*)cache, block_table, token_req,  \
                     cache_pos, b);                                                               \
    }
            if (b.cols <= 64) GO_ROWS(8) else if (b.cols <= 128) GO_ROWS(16) else GO_ROWS(32)
#undef GO_ROWS
            return launch_status();
        }
    }
    const size_t smem_tc = sizeof(bf16) * ((size_t)(32 + LAT_TILE) * (D + 8) + 3 * 16 * (LAT_TILE + 8)) +
                           sizeof(float) * (LAT_TILE * 16 + 3 * 16);
    if (act_dtype == MSTAR_BF16 && D % 16 == 0 && rank % 32 == 0 && ((uintptr_t)cache & 15) == 0 &&
        !cores_only && !scores_only && smem_tc <= 200 * 1024) {
        const int tc_group = heads < 16 ? heads : 16;
        LatentArgs b = a;
        b.group = tc_group;
        dim3 tc_grid(num_tokens, (heads + tc_group - 1) / tc_group, splits);
#define GO_TC(NB)                                                                                 \
    {                                                                                             \
        static size_t configured = 0;                                                             \
        if (smem_tc > 48 * 1024 && smem_tc > configured) {                                        \
            cudaFuncSetAttribute(latent_attention_tc_kernel<NB>,                                  \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_tc);      \
            configured = smem_tc;                                                                 \
        }                                                                                         \
        mstar_launch((latent_attention_tc_kernel<NB>), tc_grid, dim3(LAT_THREADS), smem_tc, s,    \
                     q_abs, (const bf16*)q_rot, out, part_acc, part_ml, (const bf16*)cache,       \
                     block_table, token_req, cache_pos, b);                                       \
    }
        if (rank <= 128) GO_TC(4) else if (rank <= 256) GO_TC(8) else if (rank <= 512) GO_TC(16) else GO_TC(32)
#undef GO_TC
        if (splits > 1)
            mstar_launch(latent_merge_kernel, dim3(num_tokens * heads), dim3(128), 0, s,
                         (const float*)part_acc, (const float*)part_ml, out, rank, splits);
        return launch_status();
    }
    const size_t smem_mma = sizeof(bf16) * (size_t)(32 + LAT_TILE) * (D + 8) +
                            sizeof(float) * ((size_t)gp * LAT_TILE + 3 * (size_t)gp);
    if (act_dtype == MSTAR_BF16 && D % 16 == 0 && ((uintptr_t)cache & 15) == 0 && !cores_only &&
        smem_mma <= 200 * 1024) {
#define GO_MMA(GP)                                                                                \
    {                                                                                             \
        static size_t configured = 0;                                                             \
        if (smem_mma > 48 * 1024 && smem_mma > configured) {                                      \
            cudaFuncSetAttribute(latent_attention_mma_kernel<GP>,                                 \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma);     \
            configured = smem_mma;                                                                \
        }                                                                                         \
        mstar_launch((latent_attention_mma_kernel<GP>), grid, dim3(LAT_THREADS), smem_mma, s,     \
                     q_abs, (const bf16*)q_rot, out, part_acc, part_ml, (const bf16*)cache,       \
                     block_table, token_req, cache_pos, a);                                       \
    }
        if (gp == 4) GO_MMA(4) else if (gp == 8) GO_MMA(8) else GO_MMA(16)
#undef GO_MMA
        if (splits > 1)
            mstar_launch(latent_merge_kernel, dim3(num_tokens * heads), dim3(128), 0, s,
                         (const float*)part_acc, (const float*)part_ml, out, rank, splits);
        return launch_status();
    }
#define GO(A, GP) launch_latent<A, GP>(q_abs, q_rot, out, part_acc, part_ml, cache, block_table, \
                                       token_req, cache_pos, a, grid, smem, s)
    if (act_dtype == MSTAR_F32) {
        if (gp == 4) GO(float, 4); else if (gp == 8) GO(float, 8); else GO(float, 16);
    } else {
        if (gp == 4) GO(bf16, 4); else if (gp == 8) GO(bf16, 8); else GO(bf16, 16);
    }
#undef GO
    if (splits > 1)
        mstar_launch(latent_merge_kernel, dim3(num_tokens * heads), dim3(128), 0, s,
                     (const float*)part_acc, (const float*)part_ml, out, rank, splits);
    return launch_status();
}

// ---------------------------------------------------------------- cache fill + rotation
struct LatentFillArgs {
    int heads, qk_dim, rot, rot_dims, rank, page_size, bt_stride;
    int ldq;        // elements between tokens of the queries
    int ld_dkv;     // elements between tokens of the down-projection
    int interleaved;        // 1: pairs (2i, 2i+1); 0: pairs (i, i + rot_dims/2)
    int q_rank, ld_qlat, ld_qlat_out;   // the query latent: features, strides in and out
    float eps;
};

__device__ __forceinline__ void rotate_pair(float u, float v, int position, double freq, float& x,
                                            float& y) {
    double sn, cs;
    sincos((double)position * freq, &sn, &cs);
    const float c = (float)cs, s = (float)sn;
    x = u * c - v * s;
    y = v * c + u * s;
}

// One block per token; three jobs, each left out when its pointer is null:
//   dkv   [rank latent | rot key] features of the down-projection (type D): the latent is
//         RMS-normed (plain weight), the first rot_dims key features are rotated, and the row
//         goes into the token's cache slot;
//   q     the queries, head by head [qk_dim plain | rot rotated]: the first rot_dims features
//         of every head's rotated part are rotated in place;
//   qlat  q_rank features of a query latent (type D): RMS-normed with a plain weight into
//         qlat_out (type A), the rows the query up-projection reads.
template <typename A, typename D>
__global__ void latent_fill_kernel(A* q, const D* dkv, const float* __restrict__ norm_w,
                                   const double* __restrict__ freq, const int* __restrict__ positions,
                                   const int* __restrict__ cache_pos, const int* __restrict__ token_req,
                                   const int* __restrict__ block_table, A* __restrict__ cache,
                                   const D* qlat, const float* __restrict__ qlat_w, A* qlat_out,
                                   LatentFillArgs a) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const unsigned long long waited = pdl_wait();
    const int pos = positions[t];
    const int half = a.rot_dims / 2;
    const int second = a.interleaved ? 1 : half;          // distance between a pair's features
    const int step = a.interleaved ? 2 : 1;               // distance between two pairs
    if (dkv != nullptr) {
        const D* row = pdl_after(dkv, waited) + (size_t)t * a.ld_dkv;
        const int cp = cache_pos[t];
        const int page = block_table[(size_t)token_req[t] * a.bt_stride + cp / a.page_size];
        A* dst = cache + ((size_t)page * a.page_size + cp % a.page_size) * (a.rank + a.rot);
        float ss = 0.f;
        for (int i = tid; i < a.rank; i += blockDim.x) {
            const float v = to_float(row[i]);
            ss = fmaf(v, v, ss);
        }
        const float inv = rsqrtf(block_sum(ss, scratch) / (float)a.rank + a.eps);
        for (int i = tid; i < a.rank; i += blockDim.x)
            dst[i] = from_float<A>(to_float(row[i]) * inv * norm_w[i]);
        // the shared key part: rotated pairs, then what lies beyond the rotated dimensions
        for (int i = tid; i < half; i += blockDim.x) {
            float x, y;
            rotate_pair(to_float(row[a.rank + step * i]), to_float(row[a.rank + step * i + second]),
                        pos, freq[i], x, y);
            dst[a.rank + step * i] = from_float<A>(x);
            dst[a.rank + step * i + second] = from_float<A>(y);
        }
        for (int i = a.rot_dims + tid; i < a.rot; i += blockDim.x)
            dst[a.rank + i] = from_float<A>(to_float(row[a.rank + i]));
    }
    if (q != nullptr) {
        A* row = pdl_after(q, waited) + (size_t)t * a.ldq;
        for (int idx = tid; idx < a.heads * half; idx += blockDim.x) {
            const int h = idx / half, i = idx - h * half;
            A* qh = row + (size_t)h * (a.qk_dim + a.rot) + a.qk_dim;
            float x, y;
            rotate_pair(to_float(qh[step * i]), to_float(qh[step * i + second]), pos, freq[i], x, y);
            qh[step * i] = from_float<A>(x);
            qh[step * i + second] = from_float<A>(y);
        }
    }
    if (qlat != nullptr) {
        const D* row = pdl_after(qlat, waited) + (size_t)t * a.ld_qlat;
        float ss = 0.f;
        for (int i = tid; i < a.q_rank; i += blockDim.x) {
            const float v = to_float(row[i]);
            ss = fmaf(v, v, ss);
        }
        const float inv = rsqrtf(block_sum(ss, scratch) / (float)a.q_rank + a.eps);
        A* dst = qlat_out + (size_t)t * a.ld_qlat_out;
        for (int i = tid; i < a.q_rank; i += blockDim.x)
            dst[i] = from_float<A>(to_float(row[i]) * inv * qlat_w[i]);
    }
}

// `in_dtype`: the type of dkv and qlat (float, or the activation type).  Returns -1 for a
// rotation over an odd number of features or more than there are, and for float activations
// with inputs that are not float.
MSTAR_API int mstar_latent_fill(void* q, int ldq, const void* dkv, int ld_dkv, int in_dtype,
                                int act_dtype, const float* norm_w, const double* freq,
                                const int* positions, const int* cache_pos, const int* token_req,
                                const int* block_table, int bt_stride, void* cache,
                                const void* qlat, int ld_qlat, const float* qlat_w, void* qlat_out,
                                int ld_qlat_out, int q_rank, int num_tokens, int heads, int qk_dim,
                                int rot, int rot_dims, int rank, int page_size, int interleaved,
                                float eps, void* stream) {
    if (num_tokens <= 0) return 0;
    if (rot_dims % 2 != 0 || rot_dims > rot || rot_dims < 0) return -1;
    if (act_dtype == MSTAR_F32 && in_dtype != MSTAR_F32) return -1;
    if (dkv != nullptr && (!norm_w || !cache || !block_table)) return -1;
    if (qlat != nullptr && (!qlat_w || !qlat_out || q_rank <= 0)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    LatentFillArgs a{heads, qk_dim, rot, rot_dims, rank, page_size, bt_stride, ldq, ld_dkv,
                     interleaved, q_rank, ld_qlat, ld_qlat_out, eps};
    const int threads = rank >= 512 ? 256 : 128;
#define GO(A, D)                                                                                   \
    mstar_launch((latent_fill_kernel<A, D>), dim3(num_tokens), dim3(threads), 0, s, (A*)q,         \
                 (const D*)dkv, norm_w, freq, positions, cache_pos, token_req, block_table,        \
                 (A*)cache, (const D*)qlat, qlat_w, (A*)qlat_out, a)
    if (act_dtype == MSTAR_F32) {
        GO(float, float);
    } else if (in_dtype == MSTAR_F32) {
        GO(bf16, float);
    } else {
        GO(bf16, bf16);
    }
#undef GO
    return launch_status();
}
