// The window attention with kept first keys (attention_sink.cu says what is computed) in
// bfloat16 on the tensor cores, for prompt portions and decoded tokens alike.
//
// The rows of one (entry, kv head) are the pairs (token, query head of the group),
// token-major; a CTA takes 64 consecutive rows (four warps of 16) and streams the keys and
// values its rows can see through shared memory in tiles of 64 (cp.async, two stages).  The
// keys a CTA visits are numbered without the gap: first the kept first keys that lie before
// the window of its first row, then the keys from that window's start to its last row's
// position; each row masks by its own position (j <= p and (p - j < window or j <
// keep_first)).  S = Q K^T is an m16n8k16 MMA with float sums; the softmax is online and
// float; the probabilities enter O += P V as three bfloat16 parts that together hold the
// float exactly, so that the weights stay 32-bit; O is float.  Key and value sizes are
// padded with zeros in shared memory to the next compiled size D.
//
// Options: a soft cap (a score becomes cap * tanh(score / cap) after the scale), a sink a
// query head (exp(sink_h) joins the softmax's denominator where a row's last partial sums
// meet; it has no key and no value), and a gate on the output, one number a head or one a
// feature.
//
// With few rows (decoding) the visited keys are shared among `splits` CTAs, each leaving an
// unnormalised partial (o, running maximum, sum) in scratch, and a second kernel merges.
#include "common.cuh"
#include "mma_util.cuh"

#define ST_THREADS 128
#define ST_ROWS 64
#define ST_TILE 64

struct SinkTcArgs {
    const bf16* q;
    const bf16* kv;
    const int* block_table;
    const int* qo_indptr;
    const int* kv_len;
    bf16* out;
    float* scratch;
    int q_stride, bt_stride, nq, nkv, hd, vd, page_size, window, keep_first, splits;
    float scale_log2e;
    // not null: the output of head h of token t is multiplied by sigmoid(gate[t * gate_stride + h]),
    // or, with gate_features, feature d of it by sigmoid(gate[t * gate_stride + h * vd + d])
    const float* gate;
    int gate_stride;
    int gate_features;
    float scale, softcap;       // softcap 0: none
    float cap_in, cap_log2e;    // 2 log2(e) scale / softcap and softcap log2(e)
    const float* sink;          // null, or one number a query head
};

__device__ __forceinline__ float st_head_gate(const float* gate, int stride, int tok, int head) {
    return gate == nullptr ? 1.f : 1.f / (1.f + expf(-gate[(size_t)tok * stride + head]));
}
// The gate of one output feature: per head (features 0), or per feature.
__device__ __forceinline__ float st_gate(const float* gate, int stride, int features, int vd, int tok,
                                         int head, int d) {
    if (gate == nullptr) return 1.f;
    const size_t i = (size_t)tok * stride + (features ? (size_t)head * vd + d : (size_t)head);
    return 1.f / (1.f + expf(-gate[i]));
}
// What a sink adds to a denominator whose terms are 2^(s - m), m in the base-2 domain.
__device__ __forceinline__ float st_sink_term(const float* sink, int head, float m) {
    return sink == nullptr ? 0.f : exp2f(sink[head] * 1.4426950408889634f - m);
}

template <int D> __device__ __forceinline__ int st_off(int row, int c) { return row * (D + 8) + c * 8; }

// NSTAGE key/value tiles are in flight: two where rows are many (the tensor cores set the
// pace), four where they are few (decoding: the latency of the copies does).
// KEYSPLIT (an entry's rows fit one warp's 16: decoding): the four warps all take those rows
// and each a quarter of every key tile (keys 16 w .. 16 w + 15 of the tile), with a running
// maximum, sum and output of its own; the four are merged through shared memory at the end.
// One warp alone would issue a tile's products one after the other while three wait.
template <int D, int NSTAGE, bool KEYSPLIT>
__global__ void __launch_bounds__(ST_THREADS)
sink_attention_tc_kernel(SinkTcArgs a) {
    constexpr int CPR = D / 8;
    constexpr int LD = D + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* stages = reinterpret_cast<bf16*>(smem_raw);      // [NSTAGE]{K [64][LD], V [64][LD]}
    bf16* Qs = stages + NSTAGE * 2 * ST_TILE * LD;         // [64][LD]

    const int split = blockIdx.x % a.splits;
    const int tile = gridDim.x / a.splits - 1 - blockIdx.x / a.splits;   // long tiles first
    const int kvh = blockIdx.y, e = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.nq / a.nkv;
    const unsigned long long waited = pdl_wait();
    const bf16* q = pdl_after(a.q, waited);
    const bf16* kv = pdl_after(a.kv, waited);
    const float* gate = pdl_after(a.gate, waited);
    const int q_start = a.qo_indptr[e];
    const int q_len = a.qo_indptr[e + 1] - q_start;
    const int rows_total = q_len * G;
    const int row0 = tile * ST_ROWS;
    if (row0 >= rows_total) return;
    const int past = a.kv_len[e] - q_len;      // cache position of the entry's first new token
    const int W = a.window > 0 ? a.window : 0x3fffffff;
    const int last_row = min(rows_total, row0 + ST_ROWS) - 1;
    const int hi = past + last_row / G + 1;
    const int lo = max(0, past + row0 / G - W + 1);
    const int kept = min(a.keep_first, lo);    // kept first keys before the CTA's window
    const int visible = kept + hi - lo;

    const int* bt = a.block_table + (size_t)e * a.bt_stride;
    const size_t page_elems = (size_t)a.nkv * a.page_size * (a.hd + a.vd);
    const size_t k_head = (size_t)kvh * a.page_size * a.hd;
    const size_t v_head = (size_t)a.nkv * a.page_size * a.hd + (size_t)kvh * a.page_size * a.vd;
    const int kc = a.hd / 8, vc = a.vd / 8;    // 16-byte chunks of a real key / value row

    for (int i = tid; i < ST_ROWS * CPR; i += ST_THREADS) {
        const int r = i / CPR, c = i - r * CPR;
        const int row = row0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < rows_total && c < kc) {
            const int tok = q_start + row / G, head = kvh * G + row % G;
            v = *reinterpret_cast<const uint4*>(q + (size_t)tok * a.q_stride + (size_t)head * a.hd + c * 8);
        }
        *reinterpret_cast<uint4*>(Qs + st_off<D>(r, c)) = v;
    }
    auto load_tile = [&](int stage, int base) {
        bf16* Ks = stages + (size_t)stage * 2 * ST_TILE * LD;
        bf16* Vs = Ks + ST_TILE * LD;
        for (int i = tid; i < ST_TILE * CPR; i += ST_THREADS) {
            const int r = i / CPR, c = i - r * CPR;
            const int v = base + r;
            const bool ok = v < visible;
            const bf16* ksrc = kv;
            const bf16* vsrc = kv;
            if (ok) {
                const int key = v < kept ? v : lo + v - kept;
                const int pg = key / a.page_size;
                const bf16* page = kv + (size_t)bt[pg] * page_elems;
                const int slot = key - pg * a.page_size;
                ksrc = page + k_head + (size_t)slot * a.hd + c * 8;
                vsrc = page + v_head + (size_t)slot * a.vd + c * 8;
            }
            const int off = st_off<D>(r, c);
            cp_async_16(smem_u32(Ks + off), ok && c < kc ? ksrc : kv, ok && c < kc ? 16 : 0);
            cp_async_16(smem_u32(Vs + off), ok && c < vc ? vsrc : kv, ok && c < vc ? 16 : 0);
        }
    };

    // this thread's two rows (g and g+8 of the warp's 16) and their positions
    const int wrow = KEYSPLIT ? 0 : warp * 16;         // first of the warp's 16 rows in the tile
    const int rowA = row0 + wrow + (lane >> 2), rowB = rowA + 8;
    const int cpA = past + min(rowA, rows_total - 1) / G;
    const int cpB = past + min(rowB, rows_total - 1) / G;
    // the warp's rows together: newest key any row sees, oldest window key any row sees
    const int warp_hi = past + min(row0 + wrow + 15, rows_total - 1) / G;
    const int warp_lo = max(0, past + min(row0 + wrow, rows_total - 1) / G - W + 1);

    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const int ntiles_all = (visible + ST_TILE - 1) / ST_TILE;
    const int per_split = (ntiles_all + a.splits - 1) / a.splits;
    const int t_first = split * per_split;
    const int ntiles = max(0, min(ntiles_all, t_first + per_split) - t_first);
#pragma unroll
    for (int st = 0; st < NSTAGE - 1; ++st) {
        if (st < ntiles) load_tile(st, (t_first + st) * ST_TILE);
        cp_async_commit();
    }
#pragma unroll 1
    for (int it = 0; it < ntiles; ++it) {
        const int ahead = it + NSTAGE - 1;
        if (ahead < ntiles) load_tile(ahead % NSTAGE, (t_first + ahead) * ST_TILE);
        cp_async_commit();
        cp_async_wait<NSTAGE - 1>();
        __syncthreads();
        const bf16* Ks = stages + (size_t)(it % NSTAGE) * 2 * ST_TILE * LD;
        const bf16* Vs = Ks + ST_TILE * LD;
        const int base = (t_first + it) * ST_TILE;
        // keys of the tile: kept first keys (always of interest), or window keys
        const int key_first = base < kept ? base : lo + base - kept;
        const int key_last = lo + min(base + ST_TILE, visible) - 1 - kept;
        // (a warp whose rows all lie past the entry's last row has nothing to do)
        if (row0 + wrow < rows_total &&
            (base < kept || (key_first <= warp_hi && key_last >= warp_lo))) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t qa[4];
                const int arow = wrow + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(qa, smem_u32(Qs + st_off<D>(arow, 2 * kk + (lane >> 4))));
#pragma unroll
                for (int jp = 0; jp < (KEYSPLIT ? 1 : 4); ++jp) {
                    uint32_t kb[4];
                    const int brow = (KEYSPLIT ? warp : jp) * 16 + (lane & 7) + (lane >> 4) * 8;
                    ldmatrix_x4(kb, smem_u32(Ks + st_off<D>(brow, 2 * kk + ((lane >> 3) & 1))));
                    mma_bf16_16816(s[2 * jp], qa, kb[0], kb[1]);
                    mma_bf16_16816(s[2 * jp + 1], qa, kb[2], kb[3]);
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < (KEYSPLIT ? 2 : 8); ++j)
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int v = base + (KEYSPLIT ? warp * 16 : 0) + j * 8 + (lane & 3) * 2 + (q4 & 1);
                    const int key = v < kept ? v : lo + v - kept;
                    const bool upper = q4 < 2;
                    const int cp = upper ? cpA : cpB;
                    const bool ok = v < visible && key <= cp && (cp - key < W || key < a.keep_first);
                    float sv = -INFINITY;
                    if (ok) {
                        // cap * tanh(x / cap) * log2(e) with tanh(z) = 1 - 2 / (2^(2 z log2 e) + 1):
                        // one exponential and one division, exact at both ends
                        sv = a.softcap > 0.f
                                 ? a.cap_log2e * (1.f - __fdividef(2.f, exp2f(s[j][q4] * a.cap_in) + 1.f))
                                 : s[j][q4] * a.scale_log2e;
                    }
                    s[j][q4] = sv;
                    if (upper) mx0 = fmaxf(mx0, sv); else mx1 = fmaxf(mx1, sv);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float b0 = mn0 == -INFINITY ? 0.f : mn0, b1 = mn1 == -INFINITY ? 0.f : mn1;
            const float al0 = exp2f(m0 - b0), al1 = exp2f(m1 - b1);
            m0 = mn0;
            m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int j = 0; j < (KEYSPLIT ? 2 : 8); ++j) {
                s[j][0] = exp2f(s[j][0] - b0);
                s[j][1] = exp2f(s[j][1] - b0);
                s[j][2] = exp2f(s[j][2] - b1);
                s[j][3] = exp2f(s[j][3] - b1);
                ps0 += s[j][0] + s[j][1];
                ps1 += s[j][2] + s[j][3];
            }
            l0 = l0 * al0 + ps0;
            l1 = l1 * al1 + ps1;
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1;
            }
            // O += P V with P = P1 + P2 + P3, three bfloat16 parts that hold the float exactly.
            // A block of 16 keys at a time: its three parts of P, then every value fragment
            // is fetched once and meets all three.
#pragma unroll
            for (int kk = 0; kk < (KEYSPLIT ? 1 : 4); ++kk) {
                uint32_t pa[3][4];
#pragma unroll
                for (int part = 0; part < 3; ++part) {
                    pa[part][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                    pa[part][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                    pa[part][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                    pa[part][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
                    if (part < 2) {            // what the parts so far leave
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4)
                                s[2 * kk + jj][q4] -= __bfloat162float(__float2bfloat16_rn(s[2 * kk + jj][q4]));
                    }
                }
                const int vrow = (KEYSPLIT ? warp : kk) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                // NG value fragments at a time: 2 NG sums lie between two products into the
                // same one
                constexpr int NG = (D / 16) % 4 == 0 ? 4 : 2;
#pragma unroll
                for (int n2 = 0; n2 < D / 16; n2 += NG) {
                    uint32_t vb[NG][4];
#pragma unroll
                    for (int q = 0; q < NG; ++q)
                        ldmatrix_x4_trans(vb[q], smem_u32(Vs + st_off<D>(vrow, 2 * (n2 + q) + (lane >> 4))));
#pragma unroll
                    for (int part = 0; part < 3; ++part) {
#pragma unroll
                        for (int q = 0; q < NG; ++q) {
                            mma_bf16_16816(o[2 * (n2 + q)], pa[part], vb[q][0], vb[q][1]);
                            mma_bf16_16816(o[2 * (n2 + q) + 1], pa[part], vb[q][2], vb[q][3]);
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if constexpr (KEYSPLIT) {
        // the four warps' partials of rows 0..15 meet in shared memory (the key/value stages are
        // done with): [warp][row][vd + 2] floats, then every thread sums a share of (row, feature)
        float* part = reinterpret_cast<float*>(smem_raw);
        const int pw = a.vd + 2;
        __syncthreads();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = (lane >> 2) + 8 * half;
            float* dst = part + ((size_t)warp * 16 + r) * pw;
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                if (n * 8 < a.vd) {
                    dst[n * 8 + (lane & 3) * 2] = o[n][2 * half];
                    dst[n * 8 + (lane & 3) * 2 + 1] = o[n][2 * half + 1];
                }
            if ((lane & 3) == 0) {
                dst[a.vd] = half ? m1 : m0;
                dst[a.vd + 1] = half ? l1 : l0;
            }
        }
        __syncthreads();
        const int rows_here = min(16, rows_total - row0);
        for (int i = tid; i < rows_here * pw; i += ST_THREADS) {
            const int r = i / pw, d = i - r * pw;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) M = fmaxf(M, part[((size_t)w * 16 + r) * pw + a.vd]);
            float L = 0.f, sum = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float* p = part + ((size_t)w * 16 + r) * pw;
                const float wt = p[a.vd] == -INFINITY ? 0.f : exp2f(p[a.vd] - M);
                L = fmaf(p[a.vd + 1], wt, L);
                sum = fmaf(d < a.vd ? p[d] : 0.f, wt, sum);
            }
            const int row = row0 + r;
            const int tok = q_start + row / G, head = kvh * G + row % G;
            if (a.splits == 1) {
                if (d < a.vd)
                    a.out[((size_t)tok * a.nq + head) * a.vd + d] = __float2bfloat16_rn(
                        sum / (L + st_sink_term(a.sink, head, M)) *
                        st_gate(gate, a.gate_stride, a.gate_features, a.vd, tok, head, d));
            } else {
                float* dst = a.scratch + (((size_t)tok * a.nq + head) * a.splits + split) * pw;
                dst[d] = d < a.vd ? sum : (d == a.vd ? M : L);
            }
        }
    } else {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half ? rowB : rowA;
        if (row >= rows_total) continue;
        const float l = half ? l1 : l0, m = half ? m1 : m0;
        const int tok = q_start + row / G, head = kvh * G + row % G;
        if (a.splits == 1) {
            const float denom = l + st_sink_term(a.sink, head, m);
            const float inv = (a.gate_features ? 1.f : st_head_gate(gate, a.gate_stride, tok, head)) / denom;
            bf16* dst = a.out + ((size_t)tok * a.nq + head) * a.vd + (lane & 3) * 2;
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                if (n * 8 < a.vd) {
                    float g0 = 1.f, g1 = 1.f;
                    if (a.gate_features) {
                        const int d = n * 8 + (lane & 3) * 2;
                        g0 = st_gate(gate, a.gate_stride, 1, a.vd, tok, head, d);
                        g1 = st_gate(gate, a.gate_stride, 1, a.vd, tok, head, d + 1);
                    }
                    *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) =
                        __floats2bfloat162_rn(o[n][2 * half] * inv * g0, o[n][2 * half + 1] * inv * g1);
                }
        } else {
            float* dst = a.scratch + (((size_t)tok * a.nq + head) * a.splits + split) * (a.vd + 2);
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                if (n * 8 < a.vd) {
                    dst[n * 8 + (lane & 3) * 2] = o[n][2 * half];
                    dst[n * 8 + (lane & 3) * 2 + 1] = o[n][2 * half + 1];
                }
            if ((lane & 3) == 0) {
                dst[a.vd] = m;
                dst[a.vd + 1] = l;
            }
        }
    }
    }
}

// One warp per (token, head): the partials of the splits, weighted by 2^(m_s - max m).  Lane s
// fetches the maximum and the sum of split s (at most 64 splits: two a lane), the weights go
// round by shuffles, and every lane sums its features over the splits with the loads of all
// splits in flight together.
__global__ void sink_merge_kernel(const float* __restrict__ scratch, bf16* __restrict__ out,
                                  int rows, int vd, int splits, const float* gate, int gate_stride,
                                  int nq, int gate_features, const float* __restrict__ sink) {
    const unsigned long long waited = pdl_wait();
    scratch = pdl_after(scratch, waited);
    gate = pdl_after(gate, waited);
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* base = scratch + (size_t)row * splits * (vd + 2);
    float m_a = -INFINITY, l_a = 0.f, m_b = -INFINITY, l_b = 0.f;
    if (lane < splits) {
        m_a = base[(size_t)lane * (vd + 2) + vd];
        l_a = base[(size_t)lane * (vd + 2) + vd + 1];
    }
    if (lane + 32 < splits) {
        m_b = base[(size_t)(lane + 32) * (vd + 2) + vd];
        l_b = base[(size_t)(lane + 32) * (vd + 2) + vd + 1];
    }
    const float M = warp_max(fmaxf(m_a, m_b));
    const float w_a = exp2f(m_a - M), w_b = exp2f(m_b - M);   // 0 for a split that saw no key
    const float L = (warp_sum(l_a * w_a + l_b * w_b) + st_sink_term(sink, row % nq, M)) /
                    (gate_features ? 1.f : st_head_gate(gate, gate_stride, row / nq, row % nq));
    // a gate a feature: all of a lane's gate values are asked for before the sums (vd <= 256)
    float gv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = i * 32 + lane;
        gv[i] = (gate_features && d < vd)
                    ? gate[(size_t)(row / nq) * gate_stride + (size_t)(row % nq) * vd + d] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = i * 32 + lane;
        if (i * 32 >= vd) break;
        float sum = 0.f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) {
            const float w = __shfl_sync(0xffffffffu, s < 32 ? w_a : w_b, s & 31);
            if (d < vd) sum = fmaf(base[(size_t)s * (vd + 2) + d], w, sum);
        }
        if (d < vd)
            out[(size_t)row * vd + d] =
                __float2bfloat16_rn(sum / L * (gate_features ? 1.f / (1.f + expf(-gv[i])) : 1.f));
    }
}

template <int D, int NSTAGE, bool KEYSPLIT>
static int launch_sink_tc_stages(const SinkTcArgs& a, int entries, int max_q_len, cudaStream_t s) {
    const size_t smem = (size_t)(2 * NSTAGE + 1) * ST_TILE * (D + 8) * sizeof(bf16);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(sink_attention_tc_kernel<D, NSTAGE, KEYSPLIT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int G = a.nq / a.nkv;
    const long long tiles = ((long long)max_q_len * G + ST_ROWS - 1) / ST_ROWS;
    if (tiles * a.splits > 2147483647LL) return -1;
    dim3 grid((unsigned)(tiles * a.splits), a.nkv, entries);
    mstar_launch((sink_attention_tc_kernel<D, NSTAGE, KEYSPLIT>), grid, dim3(ST_THREADS), smem, s, a);
    return launch_status();
}

template <int D>
static int launch_sink_tc(const SinkTcArgs& a, int entries, int max_q_len, cudaStream_t s) {
    // one row tile per (entry, kv head): few rows, deep prefetch (where shared memory has room)
    const long long rows = (long long)max_q_len * (a.nq / a.nkv);
    if constexpr (D <= 128) {
        if (rows <= 16) return launch_sink_tc_stages<D, 4, true>(a, entries, max_q_len, s);
        if (rows <= ST_ROWS) return launch_sink_tc_stages<D, 4, false>(a, entries, max_q_len, s);
    } else {
        if (rows <= 16) return launch_sink_tc_stages<D, 2, true>(a, entries, max_q_len, s);
    }
    return launch_sink_tc_stages<D, 2, false>(a, entries, max_q_len, s);
}

// Entries [0, entries) of the batch; q: [tokens] rows of q_stride elements; out: [tokens,
// nq * vd]; scratch: float [tokens * nq * splits * (vd + 2)] when splits > 1; gate: null, or
// float rows of gate_stride with one number a head, whose sigmoid scales that head's output.
// Returns 0, a
// CUDA error code, or -1 when the shape is refused (sizes no multiples of 8 or above 256).
MSTAR_API int mstar_sink_attention_tc(const void* q, int q_stride, void* out, const void* kv_cache,
                                      const int* block_table, int bt_stride, const int* qo_indptr,
                                      const int* kv_len, int entries, int tokens, int max_q_len,
                                      int nq, int nkv, int hd, int vd, int page_size, int window,
                                      int keep_first, float scale, int splits, float* scratch,
                                      const float* gate, int gate_stride, int gate_features,
                                      float softcap, const float* sink, void* stream) {
    if (entries <= 0 || max_q_len <= 0) return 0;
    if (nkv <= 0 || nq % nkv != 0 || entries > 65535 || nkv > 65535) return -1;
    if (hd % 8 || vd % 8 || hd <= 0 || vd <= 0 || hd > 256 || vd > 256 || splits < 1 || splits > 64)
        return -1;
    if (splits > 1 && scratch == nullptr) return -1;
    SinkTcArgs a;
    a.q = (const bf16*)q;
    a.kv = (const bf16*)kv_cache;
    a.block_table = block_table;
    a.qo_indptr = qo_indptr;
    a.kv_len = kv_len;
    a.out = (bf16*)out;
    a.scratch = scratch;
    a.q_stride = q_stride;
    a.bt_stride = bt_stride;
    a.nq = nq;
    a.nkv = nkv;
    a.hd = hd;
    a.vd = vd;
    a.page_size = page_size;
    a.window = window;
    a.keep_first = window > 0 ? keep_first : 0;
    a.splits = splits;
    a.scale_log2e = scale * 1.4426950408889634f;
    a.gate = gate;
    a.gate_stride = gate_stride;
    a.gate_features = gate != nullptr && gate_features;
    a.scale = scale;
    a.softcap = softcap;
    a.cap_in = softcap > 0.f ? 2.f * 1.4426950408889634f * scale / softcap : 0.f;
    a.cap_log2e = softcap * 1.4426950408889634f;
    a.sink = sink;
    cudaStream_t s = (cudaStream_t)stream;
    const int wide = hd > vd ? hd : vd;
    int code;
    if (wide <= 32) code = launch_sink_tc<32>(a, entries, max_q_len, s);
    else if (wide <= 64) code = launch_sink_tc<64>(a, entries, max_q_len, s);
    else if (wide <= 96) code = launch_sink_tc<96>(a, entries, max_q_len, s);
    else if (wide <= 128) code = launch_sink_tc<128>(a, entries, max_q_len, s);
    else code = launch_sink_tc<256>(a, entries, max_q_len, s);
    if (code != 0 || splits == 1) return code;
    const int rows = tokens * nq;
    mstar_launch(sink_merge_kernel, dim3((rows + 3) / 4), dim3(128), 0, s, (const float*)scratch,
                 (bf16*)out, rows, vd, splits, gate, gate_stride, nq, a.gate_features, sink);
    return launch_status();
}
