// Backward of the causal per-bucket prefix forward (src/race_baseline.py:45-51), CUDA cores.
// The reference never built a causal backward; the arithmetic is the derivative of its forward:
// with inv_t = 1/(A_t+eps), W_t = pQ_t*inv_t and the forward's prefixes A_t, B_t,
//   X_t[s] = B_t[s,:].dO_t ;  dPQ_t = X_t*inv_t ;  g_t = -X_t*W_t*inv_t        (gradient reaching A_t)
//   SA_j = sum_{t>=j} g_t ;  SB_j = sum_{t>=j} W_t (x) dO_t                     (suffix sums)
//   dPK_j[s] = SA_j[s] + SB_j[s,:].V_j ;  dV_j = sum_s pK_j[s] SB_j[s,:].
// Launches on one stream, over state tiles of `tile_tokens` tokens:
//   tile totals of (pK, V) + exclusive scan           (the forward's kernels: prefix state per tile)
//   bwd_prefix_pass : walks a tile forwards with B on chip; per chunk of 32 tokens
//                       X = dO B^T + tril(dO V^T) pK ;  writes dPQ, and W, g to scratch;
//                       B += pK^T V ;  tile totals of (W (x) dO, g)
//   tile_scan_suffix: exclusive suffix scan of those totals over the tiles of a stream
//   bwd_suffix_pass : walks a tile backwards with SB on chip; per chunk
//                       dPK = SA + V SB^T + triu(V dO^T) W ;  dV = pK SB + triu(pK W^T) dO ;
//                       SB += W^T dO ;  SA += colsum(g)
// S > 64 buckets are split into groups of 64, one CTA each; only dV sums over buckets, and the CTAs of a
// tile (one thread-block cluster) add their shares of it through distributed shared memory in group order.
// Shapes: S <= 64 or a multiple of 64 up to 512, d_k <= 128, fp32 or bf16 tokens; scratch is fp32.
#include <cooperative_groups.h>

#include "common.cuh"
#include "launch.h"

namespace cg = cooperative_groups;

namespace race {
namespace {

constexpr int C = kSimtChunk;

template <int SPT, int DV>
struct BwdLayout {
    static constexpr int SG = 16 * SPT;  // padded buckets
    static constexpr int DP = 64 * DV;   // padded head dim
    static constexpr int LDS = SG + 4;
    static constexpr int LDD = DP + 4;
    static constexpr int LDG = C + 1;
    static constexpr int NSEG = kSimtThreads / SG;  // token segments of the scans along the chunk
    static constexpr int SEGLEN = C / NSEG;
    // offsets in floats
    static constexpr int oQ = 0;                   // pQ -> W (prefix pass) / W (suffix pass)
    static constexpr int oK = oQ + C * LDS;        // pK
    static constexpr int oI = oK + C * LDS;        // inv -> g (prefix pass) / g -> SA_in (suffix pass)
    static constexpr int oV = oI + C * LDS;        // V
    static constexpr int oD = oV + C * LDD;        // dO
    static constexpr int oB = oD + C * LDD;        // B (prefix pass) / SB (suffix pass)
    static constexpr int oG = oB + SG * LDD;       // [2][C][LDG] masked token x token matrices
    static constexpr int oA = oG + 2 * C * LDG;    // [2][SG] running A / SA
    static constexpr int oP = oA + 2 * SG;         // [NSEG][SG]
    static constexpr int floats = oP + NSEG * SG;
};

// acc[i][k] += sum_c X[row0+i][c] * Y[tx+16k][c] over `len` columns (both row-major, 16-byte rows)
template <int NK>
__device__ __forceinline__ void dot_rows(float (&acc)[2][NK], const float* X, int ldx, int row0, const float* Y,
                                         int ldy, int tx, int len) {
#pragma unroll 2
    for (int c = 0; c < len; c += 4) {
        const float4 x0 = *reinterpret_cast<const float4*>(X + row0 * ldx + c);
        const float4 x1 = *reinterpret_cast<const float4*>(X + (row0 + 1) * ldx + c);
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            const float4 y = *reinterpret_cast<const float4*>(Y + (tx + 16 * k) * ldy + c);
            acc[0][k] += x0.x * y.x + x0.y * y.y + x0.z * y.z + x0.w * y.w;
            acc[1][k] += x1.x * y.x + x1.y * y.y + x1.z * y.z + x1.w * y.w;
        }
    }
}

// acc[i][k] += sum_j G[row0+i][j] * Y[j][tx+16k] over the tokens [j0, j1) of a chunk (G is triangular: the
// caller passes the range in which rows row0, row0+1 can be non-zero)
template <int NK>
__device__ __forceinline__ void mix_rows(float (&acc)[2][NK], const float* G, int ldg, int row0, const float* Y,
                                         int ldy, int tx, int j0, int j1) {
#pragma unroll 4
    for (int j = j0; j < j1; ++j) {
        const float g0 = G[row0 * ldg + j], g1 = G[(row0 + 1) * ldg + j];
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            const float y = Y[j * ldy + tx + 16 * k];
            acc[0][k] = fmaf(g0, y, acc[0][k]);
            acc[1][k] = fmaf(g1, y, acc[1][k]);
        }
    }
}

// r[i][..] += sum_t X[t][ty*SPT+i] * Y[t][dv*64 + tx*4 ..+3]   (state update X^T Y, registers)
template <int SPT, int DV>
__device__ __forceinline__ void outer_update(float (&r)[SPT][4 * DV], const float* X, int ldx, const float* Y,
                                             int ldy, int ty, int tx) {
#pragma unroll 4
    for (int t = 0; t < C; ++t) {
        float kk[SPT];
        if constexpr (SPT == 4) {   // the thread's four buckets are one 16-byte word
            const float4 k4 = *reinterpret_cast<const float4*>(X + t * ldx + ty * 4);
            kk[0] = k4.x; kk[1] = k4.y; kk[2] = k4.z; kk[3] = k4.w;
        } else {
#pragma unroll
            for (int i = 0; i < SPT; ++i) kk[i] = X[t * ldx + ty * SPT + i];
        }
#pragma unroll
        for (int dv = 0; dv < DV; ++dv) {
            const float4 vv = *reinterpret_cast<const float4*>(Y + t * ldy + dv * 64 + tx * 4);
#pragma unroll
            for (int i = 0; i < SPT; ++i) {
                r[i][dv * 4 + 0] = fmaf(kk[i], vv.x, r[i][dv * 4 + 0]);
                r[i][dv * 4 + 1] = fmaf(kk[i], vv.y, r[i][dv * 4 + 1]);
                r[i][dv * 4 + 2] = fmaf(kk[i], vv.z, r[i][dv * 4 + 2]);
                r[i][dv * 4 + 3] = fmaf(kk[i], vv.w, r[i][dv * 4 + 3]);
            }
        }
    }
}

template <int SPT, int DV>
__device__ __forceinline__ void publish_state(float* sB, int ldd, const float (&r)[SPT][4 * DV], int ty, int tx) {
#pragma unroll
    for (int i = 0; i < SPT; ++i)
#pragma unroll
        for (int dv = 0; dv < DV; ++dv)
            *reinterpret_cast<float4*>(sB + (ty * SPT + i) * ldd + dv * 64 + tx * 4) =
                make_float4(r[i][dv * 4], r[i][dv * 4 + 1], r[i][dv * 4 + 2], r[i][dv * 4 + 3]);
}

// load the rows [s0, s0+sv) of a state slice ([S][D] then [S]) into registers + shared memory; rows past sv and
// columns past D read 0
template <int SPT, int DV>
__device__ __forceinline__ void load_state(float (&r)[SPT][4 * DV], float* sB, int ldd, float* sA, const float* slice,
                                           int S, int D, int s0, int sv, int tid, int ty, int tx) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int s = ty * SPT + i;
#pragma unroll
        for (int dv = 0; dv < DV; ++dv) {
            const int c = dv * 64 + tx * 4;
            float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
            if (slice && s < sv && c < D) b = load4(slice + (int64_t)(s0 + s) * D + c);
            r[i][dv * 4 + 0] = b.x; r[i][dv * 4 + 1] = b.y; r[i][dv * 4 + 2] = b.z; r[i][dv * 4 + 3] = b.w;
            *reinterpret_cast<float4*>(sB + s * ldd + c) = b;
        }
    }
    if (tid < 16 * SPT) sA[tid] = (slice && tid < sv) ? slice[(int64_t)S * D + s0 + tid] : 0.f;
}

template <int SPT, int DV>
__device__ __forceinline__ void store_state(float* slice, const float (&r)[SPT][4 * DV], float a_sum, int S, int D,
                                            int s0, int sv, int tid, int ty, int tx) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int s = ty * SPT + i;
        if (s < sv) {
#pragma unroll
            for (int dv = 0; dv < DV; ++dv) {
                const int c = dv * 64 + tx * 4;
                if (c < D)
                    *reinterpret_cast<float4*>(slice + (int64_t)(s0 + s) * D + c) =
                        make_float4(r[i][dv * 4], r[i][dv * 4 + 1], r[i][dv * 4 + 2], r[i][dv * 4 + 3]);
            }
        }
    }
    if (tid < sv) slice[(int64_t)S * D + s0 + tid] = a_sum;
}

// ------------------------------------------------------------------------------------------
// prefix pass: dPQ, scratch W and g, tile totals of the suffix quantities
// ------------------------------------------------------------------------------------------
template <typename Tin, int SPT, int DV>
__global__ void __launch_bounds__(kSimtThreads, DV == 1 ? 3 : 2)
bwd_prefix_pass(const Tin* __restrict__ pq, const Tin* __restrict__ pk, const Tin* __restrict__ v,
                const Tin* __restrict__ dout, Tin* __restrict__ dpq, float* __restrict__ w_out,
                float* __restrict__ g_out, const float* __restrict__ ws_prefix, float* __restrict__ ws_suffix,
                Dims dm, int tile_tokens, int groups) {
    using Ly = BwdLayout<SPT, DV>;
    extern __shared__ __align__(16) float smem[];
    float* sQ = smem + Ly::oQ;
    float* sK = smem + Ly::oK;
    float* sI = smem + Ly::oI;
    float* sV = smem + Ly::oV;
    float* sD = smem + Ly::oD;
    float* sB = smem + Ly::oB;
    float* sG = smem + Ly::oG;
    float* sA = smem + Ly::oA;
    float* sP = smem + Ly::oP;

    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int group = blockIdx.x % groups;
    const int64_t tile = blockIdx.x / groups, tiles = gridDim.x / groups, n = blockIdx.y;
    const int S = dm.S, D = dm.D;
    const int s0 = group * kGroupBuckets;          // first bucket of this CTA's group
    const int sv = min(S - s0, Ly::SG);            // buckets it owns
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(dm.T, t_begin + tile_tokens);
    const Tin* pq_n = pq + n * dm.T * S;
    const Tin* pk_n = pk + n * dm.T * S;
    const Tin* v_n = v + n * dm.T * D;
    const Tin* do_n = dout + n * dm.T * D;
    Tin* dpq_n = dpq + n * dm.T * S;
    float* w_n = w_out + n * dm.T * S;
    float* g_n = g_out + n * dm.T * S;
    const int64_t sf = state_floats_per_stream(S, D);

    float rB[SPT][4 * DV], rR[SPT][4 * DV];
    load_state<SPT, DV>(rB, sB, Ly::LDD, sA, ws_prefix + (n * tiles + tile) * sf, S, D, s0, sv, tid, ty, tx);
#pragma unroll
    for (int i = 0; i < SPT; ++i)
#pragma unroll
        for (int j = 0; j < 4 * DV; ++j) rR[i][j] = 0.f;
    float g_sum = 0.f;
    int a_cur = 0;
    const int seg = tid / Ly::SG, scol = tid % Ly::SG;

    for (int64_t c0 = t_begin; c0 < t_end; c0 += C) {
        const int valid = (int)min((int64_t)C, t_end - c0);
        stage_block(sQ, Ly::LDS, pq_n, c0, C, valid, S, s0, Ly::SG, sv, tid, kSimtThreads);
        stage_block(sK, Ly::LDS, pk_n, c0, C, valid, S, s0, Ly::SG, sv, tid, kSimtThreads);
        stage_block(sV, Ly::LDD, v_n, c0, C, valid, D, 0, Ly::DP, D, tid, kSimtThreads);
        stage_block(sD, Ly::LDD, do_n, c0, C, valid, D, 0, Ly::DP, D, tid, kSimtThreads);
        __syncthreads();

        // ---- A_in = A + inclusive cumsum(pK); inv = 1/(A_in+eps); W = pQ*inv (over pQ) --------
        {
            float part = 0.f;
#pragma unroll
            for (int j = 0; j < Ly::SEGLEN; ++j) part += sK[(seg * Ly::SEGLEN + j) * Ly::LDS + scol];
            sP[seg * Ly::SG + scol] = part;
        }
        __syncthreads();
        {
            float a = sA[a_cur * Ly::SG + scol];
            for (int j = 0; j < seg; ++j) a += sP[j * Ly::SG + scol];
#pragma unroll
            for (int j = 0; j < Ly::SEGLEN; ++j) {
                const int t = seg * Ly::SEGLEN + j;
                a += sK[t * Ly::LDS + scol];
                const float inv = (scol < sv) ? 1.f / (a + dm.eps) : 0.f;
                const float wv = sQ[t * Ly::LDS + scol] * inv;
                sI[t * Ly::LDS + scol] = inv;
                sQ[t * Ly::LDS + scol] = wv;
                if (t < valid && scol < sv) w_n[(c0 + t) * S + s0 + scol] = wv;
            }
            if (seg == Ly::NSEG - 1) sA[(a_cur ^ 1) * Ly::SG + scol] = a;
        }
        a_cur ^= 1;

        // ---- P = tril(dO V^T): rows t = ty*2+i, columns j = tx + 16*jj (needs only sD, sV) -----
        {
            float p[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
            dot_rows<2>(p, sD, Ly::LDD, ty * 2, sV, Ly::LDD, tx, Ly::DP);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int t = ty * 2 + i, j = tx + 16 * jj;
                    sG[t * Ly::LDG + j] = (j <= t) ? p[i][jj] : 0.f;
                }
        }
        __syncthreads();

        // ---- X = dO B^T + P pK (rows ty*2+i, buckets tx+16k); dPQ = X*inv; g = -X*W*inv --------
        {
            float x[2][SPT];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int k = 0; k < SPT; ++k) x[i][k] = 0.f;
            dot_rows<SPT>(x, sD, Ly::LDD, ty * 2, sB, Ly::LDD, tx, Ly::DP);
            mix_rows<SPT>(x, sG, Ly::LDG, ty * 2, sK, Ly::LDS, tx, 0, ty * 2 + 2);    // P is lower triangular
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int k = 0; k < SPT; ++k) {
                    const int t = ty * 2 + i, s = tx + 16 * k;
                    const float inv = sI[t * Ly::LDS + s], wv = sQ[t * Ly::LDS + s];
                    const float dq = x[i][k] * inv;
                    const float g = -dq * wv;
                    sI[t * Ly::LDS + s] = g;          // this thread is the only reader of the entry
                    if (t < valid && s < sv) {
                        const int64_t at = (c0 + t) * S + s0 + s;
                        if constexpr (sizeof(Tin) == 4) dpq_n[at] = dq; else dpq_n[at] = __float2bfloat16_rn(dq);
                        g_n[at] = g;
                    }
                }
        }
        __syncthreads();

        // ---- suffix totals: R += W^T dO, sum of g; prefix state: B += pK^T V ---------------------
        outer_update<SPT, DV>(rR, sQ, Ly::LDS, sD, Ly::LDD, ty, tx);
        outer_update<SPT, DV>(rB, sK, Ly::LDS, sV, Ly::LDD, ty, tx);
        if (tid < Ly::SG) {
            float a = 0.f;
#pragma unroll 8
            for (int t = 0; t < C; ++t) a += sI[t * Ly::LDS + tid];
            g_sum += a;
        }
        publish_state<SPT, DV>(sB, Ly::LDD, rB, ty, tx);   // every read of the old B is behind the barrier above
        __syncthreads();                                    // this chunk's tiles may now be overwritten
    }
    store_state<SPT, DV>(ws_suffix + (n * tiles + tile) * sf, rR, g_sum, S, D, s0, sv, tid, ty, tx);
}

// ------------------------------------------------------------------------------------------
// exclusive suffix scan over the tiles of a stream, one thread per state float
// ------------------------------------------------------------------------------------------
// d_state (nullable): gradient reaching the state after the last token, the carry of the last tile;
// d_carry (nullable): receives the sum over all tiles + d_state, the gradient of the carried-in state
__global__ void __launch_bounds__(128)
tile_scan_suffix(float* __restrict__ ws, int64_t tiles, int state_floats, const float* __restrict__ d_state,
                 float* __restrict__ d_carry) {
    constexpr int kInFlight = 16;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= state_floats) return;
    float* p = ws + (int64_t)blockIdx.y * tiles * state_floats + i;
    float run = d_state ? d_state[(int64_t)blockIdx.y * state_floats + i] : 0.f;
    int64_t t = tiles;
    for (; t >= kInFlight; t -= kInFlight) {
        float x[kInFlight];
#pragma unroll
        for (int j = 0; j < kInFlight; ++j) x[j] = p[(t - 1 - j) * state_floats];
#pragma unroll
        for (int j = 0; j < kInFlight; ++j) {
            p[(t - 1 - j) * state_floats] = run;
            run += x[j];
        }
    }
    for (; t > 0; --t) {
        const float x = p[(t - 1) * state_floats];
        p[(t - 1) * state_floats] = run;
        run += x;
    }
    if (d_carry) d_carry[(int64_t)blockIdx.y * state_floats + i] = run;
}

// ------------------------------------------------------------------------------------------
// suffix pass: dPK and dV
// ------------------------------------------------------------------------------------------
template <typename Tin, int SPT, int DV>
__global__ void __launch_bounds__(kSimtThreads)
bwd_suffix_pass(const Tin* __restrict__ pk, const Tin* __restrict__ v, const Tin* __restrict__ dout,
                const float* __restrict__ w_in, const float* __restrict__ g_in, Tin* __restrict__ dpk,
                Tin* __restrict__ dv_out, const float* __restrict__ ws_suffix, Dims dm, int tile_tokens,
                int groups) {
    using Ly = BwdLayout<SPT, DV>;
    extern __shared__ __align__(16) float smem[];
    float* sW = smem + Ly::oQ;
    float* sK = smem + Ly::oK;
    float* sI = smem + Ly::oI;   // g, then SA_in
    float* sV = smem + Ly::oV;
    float* sD = smem + Ly::oD;
    float* sB = smem + Ly::oB;   // SB
    float* sG1 = smem + Ly::oG;               // triu(V dO^T)
    float* sG2 = smem + Ly::oG + C * Ly::LDG;  // triu(pK W^T)
    float* sA = smem + Ly::oA;
    float* sP = smem + Ly::oP;
    float* sO = smem + Ly::floats;   // [C][LDD] partial dV of this bucket group, only with clusters

    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int group = blockIdx.x % groups;
    const int64_t tile = blockIdx.x / groups, tiles = gridDim.x / groups, n = blockIdx.y;
    const int S = dm.S, D = dm.D;
    const int s0 = group * kGroupBuckets;          // first bucket of this CTA's group
    const int sv = min(S - s0, Ly::SG);            // buckets it owns
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(dm.T, t_begin + tile_tokens);
    const Tin* pk_n = pk + n * dm.T * S;
    const Tin* v_n = v + n * dm.T * D;
    const Tin* do_n = dout + n * dm.T * D;
    const float* w_n = w_in + n * dm.T * S;
    const float* g_n = g_in + n * dm.T * S;
    Tin* dpk_n = dpk + n * dm.T * S;
    Tin* dv_n = dv_out + n * dm.T * D;
    const int64_t sf = state_floats_per_stream(S, D);

    float rS[SPT][4 * DV];
    load_state<SPT, DV>(rS, sB, Ly::LDD, sA, ws_suffix + (n * tiles + tile) * sf, S, D, s0, sv, tid, ty, tx);
    int a_cur = 0;
    const int seg = tid / Ly::SG, scol = tid % Ly::SG;
    const int64_t chunks = (t_end - t_begin + C - 1) / C;

    for (int64_t ch = chunks - 1; ch >= 0; --ch) {
        const int64_t c0 = t_begin + ch * C;
        const int valid = (int)min((int64_t)C, t_end - c0);
        stage_block(sW, Ly::LDS, w_n, c0, C, valid, S, s0, Ly::SG, sv, tid, kSimtThreads);
        stage_block(sI, Ly::LDS, g_n, c0, C, valid, S, s0, Ly::SG, sv, tid, kSimtThreads);
        stage_block(sK, Ly::LDS, pk_n, c0, C, valid, S, s0, Ly::SG, sv, tid, kSimtThreads);
        stage_block(sV, Ly::LDD, v_n, c0, C, valid, D, 0, Ly::DP, D, tid, kSimtThreads);
        stage_block(sD, Ly::LDD, do_n, c0, C, valid, D, 0, Ly::DP, D, tid, kSimtThreads);
        __syncthreads();

        // ---- SA_in[j] = SA + sum_{t>=j in chunk} g_t (in place over g) -------------------------
        {
            float part = 0.f;
#pragma unroll
            for (int j = 0; j < Ly::SEGLEN; ++j) part += sI[(seg * Ly::SEGLEN + j) * Ly::LDS + scol];
            sP[seg * Ly::SG + scol] = part;
        }
        // ---- masked token x token matrices: rows j = ty*2+i, columns t = tx + 16*tt, kept for t >= j
        {
            float p1[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, p2[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
            dot_rows<2>(p1, sV, Ly::LDD, ty * 2, sD, Ly::LDD, tx, Ly::DP);
            dot_rows<2>(p2, sK, Ly::LDS, ty * 2, sW, Ly::LDS, tx, Ly::SG);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int tt = 0; tt < 2; ++tt) {
                    const int j = ty * 2 + i, t = tx + 16 * tt;
                    sG1[j * Ly::LDG + t] = (t >= j) ? p1[i][tt] : 0.f;
                    sG2[j * Ly::LDG + t] = (t >= j) ? p2[i][tt] : 0.f;
                }
        }
        __syncthreads();
        {
            float a = sA[a_cur * Ly::SG + scol];
            for (int j = seg + 1; j < Ly::NSEG; ++j) a += sP[j * Ly::SG + scol];
#pragma unroll
            for (int j = Ly::SEGLEN - 1; j >= 0; --j) {
                const int t = seg * Ly::SEGLEN + j;
                a += sI[t * Ly::LDS + scol];
                sI[t * Ly::LDS + scol] = a;
            }
            if (seg == 0) sA[(a_cur ^ 1) * Ly::SG + scol] = a;
        }
        a_cur ^= 1;
        __syncthreads();

        // ---- dPK = SA_in + V SB^T + G1 W (rows ty*2+i, buckets tx+16k) ---------------------------
        {
            float y[2][SPT];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int k = 0; k < SPT; ++k) y[i][k] = sI[(ty * 2 + i) * Ly::LDS + tx + 16 * k];
            dot_rows<SPT>(y, sV, Ly::LDD, ty * 2, sB, Ly::LDD, tx, Ly::DP);
            mix_rows<SPT>(y, sG1, Ly::LDG, ty * 2, sW, Ly::LDS, tx, ty * 2, C);       // G1 is upper triangular
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int k = 0; k < SPT; ++k) {
                    const int j = ty * 2 + i, s = tx + 16 * k;
                    if (j < valid && s < sv) {
                        const int64_t at = (c0 + j) * S + s0 + s;
                        if constexpr (sizeof(Tin) == 4) dpk_n[at] = y[i][k]; else dpk_n[at] = __float2bfloat16_rn(y[i][k]);
                    }
                }
        }
        // ---- dV = pK SB + G2 dO (rows ty*2+i, 4*DV columns) ---------------------------------------
        {
            float o[2][4 * DV];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4 * DV; ++j) o[i][j] = 0.f;
#pragma unroll 2
            for (int s4 = 0; s4 < Ly::SG; s4 += 4) {   // four buckets per 16-byte read of the two pK rows
                const float4 wa = *reinterpret_cast<const float4*>(sK + (ty * 2) * Ly::LDS + s4);
                const float4 wb = *reinterpret_cast<const float4*>(sK + (ty * 2 + 1) * Ly::LDS + s4);
                const float w0s[4] = {wa.x, wa.y, wa.z, wa.w}, w1s[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float w0 = w0s[u], w1 = w1s[u];
#pragma unroll
                    for (int dv = 0; dv < DV; ++dv) {
                        const float4 b = *reinterpret_cast<const float4*>(sB + (s4 + u) * Ly::LDD + dv * 64 + tx * 4);
                        o[0][dv * 4 + 0] = fmaf(w0, b.x, o[0][dv * 4 + 0]); o[1][dv * 4 + 0] = fmaf(w1, b.x, o[1][dv * 4 + 0]);
                        o[0][dv * 4 + 1] = fmaf(w0, b.y, o[0][dv * 4 + 1]); o[1][dv * 4 + 1] = fmaf(w1, b.y, o[1][dv * 4 + 1]);
                        o[0][dv * 4 + 2] = fmaf(w0, b.z, o[0][dv * 4 + 2]); o[1][dv * 4 + 2] = fmaf(w1, b.z, o[1][dv * 4 + 2]);
                        o[0][dv * 4 + 3] = fmaf(w0, b.w, o[0][dv * 4 + 3]); o[1][dv * 4 + 3] = fmaf(w1, b.w, o[1][dv * 4 + 3]);
                    }
                }
            }
#pragma unroll 4
            for (int t = ty * 2; t < C; ++t) {   // G2 is upper triangular
                const float g0 = sG2[(ty * 2) * Ly::LDG + t], g1 = sG2[(ty * 2 + 1) * Ly::LDG + t];
#pragma unroll
                for (int dv = 0; dv < DV; ++dv) {
                    const float4 b = *reinterpret_cast<const float4*>(sD + t * Ly::LDD + dv * 64 + tx * 4);
                    o[0][dv * 4 + 0] = fmaf(g0, b.x, o[0][dv * 4 + 0]); o[1][dv * 4 + 0] = fmaf(g1, b.x, o[1][dv * 4 + 0]);
                    o[0][dv * 4 + 1] = fmaf(g0, b.y, o[0][dv * 4 + 1]); o[1][dv * 4 + 1] = fmaf(g1, b.y, o[1][dv * 4 + 1]);
                    o[0][dv * 4 + 2] = fmaf(g0, b.z, o[0][dv * 4 + 2]); o[1][dv * 4 + 2] = fmaf(g1, b.z, o[1][dv * 4 + 2]);
                    o[0][dv * 4 + 3] = fmaf(g0, b.w, o[0][dv * 4 + 3]); o[1][dv * 4 + 3] = fmaf(g1, b.w, o[1][dv * 4 + 3]);
                }
            }
            if (groups == 1) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int j = ty * 2 + i;
                    if (j < valid) {
#pragma unroll
                        for (int dv = 0; dv < DV; ++dv) {
                            const int c = dv * 64 + tx * 4;
                            if (c < D)
                                store4_stream(dv_n + (c0 + j) * D + c,
                                              make_float4(o[i][dv * 4], o[i][dv * 4 + 1], o[i][dv * 4 + 2], o[i][dv * 4 + 3]));
                        }
                    }
                }
            } else {
                // this group's share of dV -> own shared memory; the cluster adds the shares in group order
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int dv = 0; dv < DV; ++dv)
                        *reinterpret_cast<float4*>(sO + (ty * 2 + i) * Ly::LDD + dv * 64 + tx * 4) =
                            make_float4(o[i][dv * 4], o[i][dv * 4 + 1], o[i][dv * 4 + 2], o[i][dv * 4 + 3]);
            }
        }
        if (groups > 1) {
            cg::cluster_group cluster = cg::this_cluster();
            cluster.sync();
            for (int idx = tid; idx < C * (Ly::DP / 4); idx += kSimtThreads) {   // rows dealt round-robin
                const int j = idx / (Ly::DP / 4);
                const int c = (idx % (Ly::DP / 4)) * 4;
                if ((j % groups) != group || j >= valid || c >= D) continue;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int g = 0; g < groups; ++g) {
                    const float* remote = cluster.map_shared_rank(sO, g);
                    const float4 x = *reinterpret_cast<const float4*>(remote + j * Ly::LDD + c);
                    acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
                }
                store4_stream(dv_n + (c0 + j) * D + c, acc);
            }
            cluster.sync();
        }
        // ---- SB += W^T dO (registers are the master copy) ------------------------------------------
        outer_update<SPT, DV>(rS, sW, Ly::LDS, sD, Ly::LDD, ty, tx);
        __syncthreads();                                    // every read of the old SB is done
        publish_state<SPT, DV>(sB, Ly::LDD, rS, ty, tx);
        // the next iteration's staging barrier covers sB too
    }
}

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

template <typename Tin, int SPT, int DV>
cudaError_t launch_bwd(const Tin* pq, const Tin* pk, const Tin* v, const Tin* dout, Tin* dpq, Tin* dpk, Tin* dv,
                       const float* ws_prefix, float* ws_suffix, float* w_scr, float* g_scr, const float* d_state,
                       float* d_carry, const Dims& dm, int tile_tokens, cudaStream_t stream) {
    using Ly = BwdLayout<SPT, DV>;
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    const int sf = state_floats_per_stream(dm.S, dm.D);
    const int groups = simt_groups(dm.S);
    const size_t smem = (size_t)Ly::floats * sizeof(float);
    const size_t smem3 = smem + (groups > 1 ? (size_t)C * Ly::LDD * sizeof(float) : 0);
    dim3 grid((unsigned)(tiles * groups), (unsigned)dm.N);
    auto k1 = bwd_prefix_pass<Tin, SPT, DV>;
    auto k3 = bwd_suffix_pass<Tin, SPT, DV>;
    cudaError_t err = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
    if (err != cudaSuccess) return err;
    k1<<<grid, kSimtThreads, smem, stream>>>(pq, pk, v, dout, dpq, w_scr, g_scr, ws_prefix, ws_suffix, dm, tile_tokens,
                                             groups);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    dim3 sgrid((unsigned)((sf + 127) / 128), (unsigned)dm.N);
    tile_scan_suffix<<<sgrid, 128, 0, stream>>>(ws_suffix, tiles, sf, d_state, d_carry);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    // the bucket groups of a tile form one thread-block cluster: they add their shares of dV through
    // distributed shared memory
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kSimtThreads);
    cfg.dynamicSmemBytes = smem3;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = groups;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = groups > 1 ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k3, pk, v, dout, (const float*)w_scr, (const float*)g_scr, dpk, dv,
                              (const float*)ws_suffix, dm, tile_tokens, groups);
}

template <typename Tin>
cudaError_t dispatch_bwd(const void* pq, const void* pk, const void* v, const void* dout, void* dpq, void* dpk,
                         void* dv, const float* ws_prefix, float* ws_suffix, float* w_scr, float* g_scr,
                         const float* d_state, float* d_carry, const Dims& dm, int tile_tokens, cudaStream_t stream) {
    const int sg = dm.S > kGroupBuckets ? kGroupBuckets : dm.S;
    const int spt = sg <= 16 ? 1 : (sg <= 32 ? 2 : 4);
    const int dvn = dm.D <= 64 ? 1 : 2;
#define RACE_BWD_CASE(SPT_, DV_)                                                                              \
    if (spt == SPT_ && dvn == DV_)                                                                            \
        return launch_bwd<Tin, SPT_, DV_>((const Tin*)pq, (const Tin*)pk, (const Tin*)v, (const Tin*)dout,    \
                                          (Tin*)dpq, (Tin*)dpk, (Tin*)dv, ws_prefix, ws_suffix, w_scr, g_scr, \
                                          d_state, d_carry, dm, tile_tokens, stream);
    RACE_BWD_CASE(1, 1) RACE_BWD_CASE(2, 1) RACE_BWD_CASE(4, 1)
    RACE_BWD_CASE(1, 2) RACE_BWD_CASE(2, 2) RACE_BWD_CASE(4, 2)
#undef RACE_BWD_CASE
    return cudaErrorInvalidValue;
}

}  // namespace

bool causal_bwd_supported(const Dims& dm) {
    return simt_supported(dm) && dm.H == 1;   // S <= 64, or a multiple of 64 up to 512 (one cluster); d_k <= 128
}

int causal_bwd_tile_tokens(const Dims& dm, int dtype, int sm_count) {
    if (causal_bwd_tensor_supported(dm, dtype)) return causal_bwd_tensor_tile_tokens(dm, sm_count);
    return simt_default_tile_tokens(dm, sm_count);
}

// [prefix tile states | suffix tile states | W | g], each part 256-byte aligned
size_t causal_bwd_workspace_bytes(const Dims& dm, int dtype, int tile_tokens) {
    if (dm.N == 0 || dm.T == 0) return 0;
    if (causal_bwd_tensor_supported(dm, dtype)) return causal_bwd_tensor_workspace_bytes(dm, tile_tokens);
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    const size_t states = align256((size_t)dm.N * tiles * state_floats_per_stream(dm.S, dm.D) * sizeof(float));
    const size_t tokens = align256((size_t)dm.N * dm.T * dm.S * sizeof(float));
    return 2 * states + 2 * tokens;
}

cudaError_t causal_bwd_simt(const void* pq, const void* pk, const void* v, const void* dout, const float* carry_in,
                            const float* d_state, void* dpq, void* dpk, void* dv, float* d_carry, void* ws,
                            const Dims& dm, int dtype, int tile_tokens, cudaStream_t stream, int* status) {
    // fp32, S = 64, d_k = 64: the backward as passes of the tcgen05 forward kernels
    if (causal_bwd_tensor_supported(dm, dtype))
        return causal_bwd_tensor(pq, pk, v, dout, carry_in, d_state, dpq, dpk, dv, d_carry, ws, dm, tile_tokens,
                                 stream, status);
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    const size_t states = align256((size_t)dm.N * tiles * state_floats_per_stream(dm.S, dm.D) * sizeof(float));
    const size_t tokens = align256((size_t)dm.N * dm.T * dm.S * sizeof(float));
    float* ws_prefix = (float*)ws;
    float* ws_suffix = (float*)((char*)ws + states);
    float* w_scr = (float*)((char*)ws + 2 * states);
    float* g_scr = (float*)((char*)ws + 2 * states + tokens);
    // prefix state of every tile: the forward's totals pass (on the tensor cores where that kernel covers the
    // shape) and exclusive scan
    cudaError_t err;
    if (tensor_supported(dm, dtype) && tile_tokens % tensor_chunk_tokens() == 0) {
        err = causal_fwd_tensor(nullptr, pk, v, nullptr, nullptr, nullptr, ws_prefix, false, dm, dtype, tile_tokens, stream,
                                status, kPhaseTotals);
        if (err == cudaSuccess)
            err = causal_scan_tiles(ws_prefix, carry_in, nullptr, dm, tile_tokens, stream, /*write_prefix=*/true);
    } else {
        err = causal_fwd_simt(nullptr, pk, v, nullptr, carry_in, nullptr, ws_prefix, dm, dtype, tile_tokens,
                              /*totals_only=*/false, stream, /*skip_output=*/true, /*skip_totals=*/false);
    }
    if (err != cudaSuccess) return err;
    if (dtype == RACE_DTYPE_F32)
        return dispatch_bwd<float>(pq, pk, v, dout, dpq, dpk, dv, ws_prefix, ws_suffix, w_scr, g_scr, d_state, d_carry,
                                   dm, tile_tokens, stream);
    return dispatch_bwd<__nv_bfloat16>(pq, pk, v, dout, dpq, dpk, dv, ws_prefix, ws_suffix, w_scr, g_scr, d_state,
                                       d_carry, dm, tile_tokens, stream);
}

}  // namespace race
