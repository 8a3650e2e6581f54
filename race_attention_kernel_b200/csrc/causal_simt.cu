// CUDA-core (fp32 FFMA) kernels of the causal per-bucket prefix path.  They accept every
// supported shape and both element types and are the path for shapes the tensor-core kernel
// does not cover; they also provide the tile-totals pass the sequence-sharded driver needs.
//
// Three launches on one stream (reduce-then-scan over state tiles of `tile_tokens` tokens):
//   tile_totals_simt : per (stream, tile, bucket group) sums  A = sum pK, B = sum pK (x) V
//   tile_scan        : in-place exclusive scan over the tiles of a stream (+ carry_in),
//                      inclusive total to state_out
//   causal_out_simt  : per (stream, tile, bucket group): walk the tile in chunks of 32 tokens
//                      with the running state on chip,
//                        A_in = A + incl_cumsum(pK);  W = pQ / (A_in + eps)
//                        G = tril(W pK^T);  O = W B + G V;  B += pK^T V;  A += colsum(pK)
//                      (the chunk identity of docs/causal_v2_design.md:70-77 for the estimator
//                      of src/race_baseline.py:45-51).
// S > 64 buckets are split into groups of 64 owned by the CTAs of one thread-block cluster;
// the groups' partial outputs are summed through distributed shared memory in a fixed order.
#include <cooperative_groups.h>

#include "common.cuh"
#include "launch.h"

namespace cg = cooperative_groups;

namespace race {
namespace {

constexpr int C = kSimtChunk;

template <int SPT, int DV>
struct SimtLayout {
    static constexpr int SG = 16 * SPT;  // padded buckets per group
    static constexpr int DP = 64 * DV;   // padded head dim
    static constexpr int LDS = SG + 4;
    static constexpr int LDD = DP + 4;
    static constexpr int LDG = C + 1;
    static constexpr int NSEG = kSimtThreads / SG;  // token segments of the A scan
    static constexpr int SEGLEN = C / NSEG;
    // offsets in floats
    static constexpr int oQ = 0;
    static constexpr int oK = oQ + C * LDS;
    static constexpr int oV = oK + C * LDS;
    static constexpr int oB = oV + C * LDD;
    static constexpr int oG = oB + SG * LDD;
    static constexpr int oA = oG + C * LDG;        // [2][SG]
    static constexpr int oP = oA + 2 * SG;         // [NSEG][SG]
    static constexpr int oO = oP + NSEG * SG;      // [C][LDD], only with clusters
    static constexpr int floats_single = oO;
    static constexpr int floats_cluster = oO + C * LDD;
};

// ------------------------------------------------------------------------------------------
// K1: tile totals
// ------------------------------------------------------------------------------------------
template <typename Tin, int SPT, int DV>
__global__ void __launch_bounds__(kSimtThreads)
tile_totals_simt(const Tin* __restrict__ pk, const Tin* __restrict__ v, float* __restrict__ ws,
                 Dims dm, int tile_tokens, int groups) {
    using Ly = SimtLayout<SPT, DV>;
    extern __shared__ __align__(16) float smem[];
    float* sK = smem;
    float* sV = smem + C * Ly::LDS;

    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int group = blockIdx.x % groups;
    const int64_t tile = blockIdx.x / groups;
    const int64_t n = blockIdx.y;
    const int s0 = group * kGroupBuckets;
    const int s_valid = min(dm.S - s0, Ly::SG);
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(dm.T, t_begin + tile_tokens);
    const Tin* pk_n = pk + n * dm.T * dm.S;
    const Tin* v_n = v + n * dm.T * dm.D;

    float rB[SPT][4 * DV];
#pragma unroll
    for (int i = 0; i < SPT; ++i)
#pragma unroll
        for (int j = 0; j < 4 * DV; ++j) rB[i][j] = 0.f;
    float a_sum = 0.f;

    for (int64_t c0 = t_begin; c0 < t_end; c0 += C) {
        const int valid = (int)min((int64_t)C, t_end - c0);
        __syncthreads();
        stage_block(sK, Ly::LDS, pk_n, c0, C, valid, dm.S, s0, Ly::SG, s_valid, tid, kSimtThreads);
        stage_block(sV, Ly::LDD, v_n, c0, C, valid, dm.D, 0, Ly::DP, dm.D, tid, kSimtThreads);
        __syncthreads();
#pragma unroll 4
        for (int t = 0; t < C; ++t) {
            float kk[SPT];
#pragma unroll
            for (int i = 0; i < SPT; ++i) kk[i] = sK[t * Ly::LDS + ty * SPT + i];
#pragma unroll
            for (int dv = 0; dv < DV; ++dv) {
                const float4 vv = *reinterpret_cast<const float4*>(sV + t * Ly::LDD + dv * 64 + tx * 4);
#pragma unroll
                for (int i = 0; i < SPT; ++i) {
                    rB[i][dv * 4 + 0] = fmaf(kk[i], vv.x, rB[i][dv * 4 + 0]);
                    rB[i][dv * 4 + 1] = fmaf(kk[i], vv.y, rB[i][dv * 4 + 1]);
                    rB[i][dv * 4 + 2] = fmaf(kk[i], vv.z, rB[i][dv * 4 + 2]);
                    rB[i][dv * 4 + 3] = fmaf(kk[i], vv.w, rB[i][dv * 4 + 3]);
                }
            }
        }
        if (tid < Ly::SG) {
            float a = 0.f;
#pragma unroll 8
            for (int t = 0; t < C; ++t) a += sK[t * Ly::LDS + tid];
            a_sum += a;
        }
    }

    const int64_t tiles = gridDim.x / groups;
    float* slice = ws + (n * tiles + tile) * (int64_t)state_floats_per_stream(dm.S, dm.D);
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int s = ty * SPT + i;
        if (s < s_valid) {
#pragma unroll
            for (int dv = 0; dv < DV; ++dv) {
                const int c = dv * 64 + tx * 4;
                if (c < dm.D)
                    *reinterpret_cast<float4*>(slice + (int64_t)(s0 + s) * dm.D + c) =
                        make_float4(rB[i][dv * 4], rB[i][dv * 4 + 1], rB[i][dv * 4 + 2], rB[i][dv * 4 + 3]);
            }
        }
    }
    if (tid < s_valid) slice[(int64_t)dm.S * dm.D + s0 + tid] = a_sum;
}

// ------------------------------------------------------------------------------------------
// K2: exclusive scan over tiles, one thread per state float, 32 loads in flight
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
tile_scan(float* __restrict__ ws, const float* __restrict__ carry_in, float* __restrict__ state_out,
          int64_t tiles, int state_floats, int write_prefix, int reverse) {
    constexpr int kInFlight = 32;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= state_floats) return;
    const int64_t n = blockIdx.y;
    float run = carry_in ? carry_in[n * state_floats + i] : 0.f;
    float* p = ws + n * tiles * state_floats + i;
    // reverse: exclusive SUFFIX sums -- slot t gets carry + the totals of the tiles after t (last tile first)
    auto at = [&](int64_t t) { return (reverse ? tiles - 1 - t : t) * state_floats; };
    int64_t t = 0;
    for (; t + kInFlight <= tiles; t += kInFlight) {
        float x[kInFlight];
#pragma unroll
        for (int j = 0; j < kInFlight; ++j) x[j] = p[at(t + j)];
#pragma unroll
        for (int j = 0; j < kInFlight; ++j) {
            if (write_prefix) p[at(t + j)] = run;
            run += x[j];
        }
    }
    for (; t < tiles; ++t) {
        const float x = p[at(t)];
        if (write_prefix) p[at(t)] = run;
        run += x;
    }
    if (state_out) state_out[n * state_floats + i] = run;
}

// ------------------------------------------------------------------------------------------
// K3: outputs
// ------------------------------------------------------------------------------------------
// GLOBAL: the global-normalisation estimator (src/causal_v2/reference.py:106-127) on the same states:
// W = pQ, out = (W B + tril(W pK^T) V) / den with den_t = pQ_t . A_t = pQ_t . A_carry + rowsum(tril(W pK^T)),
// and an output row of 0 where den is exactly 0 (:77-81).
template <typename Tin, int SPT, int DV, bool GLOBAL>
__global__ void __launch_bounds__(kSimtThreads)
causal_out_simt(const Tin* __restrict__ pq, const Tin* __restrict__ pk, const Tin* __restrict__ v,
                Tin* __restrict__ out, const float* __restrict__ ws, Dims dm, int tile_tokens,
                int groups) {
    using Ly = SimtLayout<SPT, DV>;
    extern __shared__ __align__(16) float smem[];
    float* sQ = smem + Ly::oQ;  // pQ, overwritten in place by W
    float* sK = smem + Ly::oK;
    float* sV = smem + Ly::oV;
    float* sB = smem + Ly::oB;
    float* sG = smem + Ly::oG;
    float* sA = smem + Ly::oA;
    float* sP = smem + Ly::oP;
    float* sO = smem + Ly::oO;

    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int group = blockIdx.x % groups;
    const int64_t tile = blockIdx.x / groups;
    const int64_t tiles = gridDim.x / groups;
    const int64_t n = blockIdx.y;
    const int s0 = group * kGroupBuckets;
    const int s_valid = min(dm.S - s0, Ly::SG);
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(dm.T, t_begin + tile_tokens);
    const Tin* pq_n = pq + n * dm.T * dm.S;
    const Tin* pk_n = pk + n * dm.T * dm.S;
    const Tin* v_n = v + n * dm.T * dm.D;
    Tin* out_n = out + n * dm.T * dm.D;

    // carry-in: exclusive prefix of this tile (written by tile_scan)
    const float* slice = ws + (n * tiles + tile) * (int64_t)state_floats_per_stream(dm.S, dm.D);
    float rB[SPT][4 * DV];
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int s = ty * SPT + i;
#pragma unroll
        for (int dv = 0; dv < DV; ++dv) {
            const int c = dv * 64 + tx * 4;
            float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s < s_valid && c < dm.D) b = load4(slice + (int64_t)(s0 + s) * dm.D + c);
            rB[i][dv * 4 + 0] = b.x; rB[i][dv * 4 + 1] = b.y;
            rB[i][dv * 4 + 2] = b.z; rB[i][dv * 4 + 3] = b.w;
            *reinterpret_cast<float4*>(sB + s * Ly::LDD + c) = b;
        }
    }
    if (tid < Ly::SG) sA[tid] = (tid < s_valid) ? slice[(int64_t)dm.S * dm.D + s0 + tid] : 0.f;
    int a_cur = 0;

    const int seg = tid / Ly::SG, scol = tid % Ly::SG;

    for (int64_t c0 = t_begin; c0 < t_end; c0 += C) {
        const int valid = (int)min((int64_t)C, t_end - c0);
        stage_block(sQ, Ly::LDS, pq_n, c0, C, valid, dm.S, s0, Ly::SG, s_valid, tid, kSimtThreads);
        stage_block(sK, Ly::LDS, pk_n, c0, C, valid, dm.S, s0, Ly::SG, s_valid, tid, kSimtThreads);
        stage_block(sV, Ly::LDD, v_n, c0, C, valid, dm.D, 0, Ly::DP, dm.D, tid, kSimtThreads);
        __syncthreads();

        // ---- A_in = A + inclusive cumsum(pK); W = pQ/(A_in+eps) (in place over pQ) ----------
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
                const float q = sQ[t * Ly::LDS + scol];
                sQ[t * Ly::LDS + scol] = (scol < s_valid) ? (GLOBAL ? q : q / (a + dm.eps)) : 0.f;
            }
            if (seg == Ly::NSEG - 1) sA[(a_cur ^ 1) * Ly::SG + scol] = a;
        }
        a_cur ^= 1;
        __syncthreads();

        // ---- G = tril(W pK^T), rows t = ty*2+i, columns j = tx + 16*jj -----------------------
        {
            float g[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll 4
            for (int s = 0; s < Ly::SG; s += 4) {
                const float4 w0 = *reinterpret_cast<const float4*>(sQ + (ty * 2) * Ly::LDS + s);
                const float4 w1 = *reinterpret_cast<const float4*>(sQ + (ty * 2 + 1) * Ly::LDS + s);
                const float4 k0 = *reinterpret_cast<const float4*>(sK + tx * Ly::LDS + s);
                const float4 k1 = *reinterpret_cast<const float4*>(sK + (tx + 16) * Ly::LDS + s);
                g[0][0] += w0.x * k0.x + w0.y * k0.y + w0.z * k0.z + w0.w * k0.w;
                g[0][1] += w0.x * k1.x + w0.y * k1.y + w0.z * k1.z + w0.w * k1.w;
                g[1][0] += w1.x * k0.x + w1.y * k0.y + w1.z * k0.z + w1.w * k0.w;
                g[1][1] += w1.x * k1.x + w1.y * k1.y + w1.z * k1.z + w1.w * k1.w;
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int t = ty * 2 + i, j = tx + 16 * jj;
                    sG[t * Ly::LDG + j] = (j <= t) ? g[i][jj] : 0.f;
                }
        }
        __syncthreads();

        // ---- O = W B + G V (rows ty*2+i, 4*DV columns) ----------------------------------------
        float o[2][4 * DV];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4 * DV; ++j) o[i][j] = 0.f;
        float den0 = 0.f, den1 = 0.f;                       // GLOBAL only
        const float* sAc = sA + (a_cur ^ 1) * Ly::SG;       // A before this chunk
#pragma unroll 4
        for (int s = 0; s < Ly::SG; ++s) {
            const float w0 = sQ[(ty * 2) * Ly::LDS + s], w1 = sQ[(ty * 2 + 1) * Ly::LDS + s];
            if (GLOBAL) {
                const float ac = sAc[s];
                den0 = fmaf(w0, ac, den0);
                den1 = fmaf(w1, ac, den1);
            }
#pragma unroll
            for (int dv = 0; dv < DV; ++dv) {
                const float4 b = *reinterpret_cast<const float4*>(sB + s * Ly::LDD + dv * 64 + tx * 4);
                o[0][dv * 4 + 0] = fmaf(w0, b.x, o[0][dv * 4 + 0]); o[1][dv * 4 + 0] = fmaf(w1, b.x, o[1][dv * 4 + 0]);
                o[0][dv * 4 + 1] = fmaf(w0, b.y, o[0][dv * 4 + 1]); o[1][dv * 4 + 1] = fmaf(w1, b.y, o[1][dv * 4 + 1]);
                o[0][dv * 4 + 2] = fmaf(w0, b.z, o[0][dv * 4 + 2]); o[1][dv * 4 + 2] = fmaf(w1, b.z, o[1][dv * 4 + 2]);
                o[0][dv * 4 + 3] = fmaf(w0, b.w, o[0][dv * 4 + 3]); o[1][dv * 4 + 3] = fmaf(w1, b.w, o[1][dv * 4 + 3]);
            }
        }
#pragma unroll 4
        for (int j = 0; j < ty * 2 + 2; ++j) {   // G is lower triangular: rows ty*2, ty*2+1 end at column ty*2+1
            const float g0 = sG[(ty * 2) * Ly::LDG + j], g1 = sG[(ty * 2 + 1) * Ly::LDG + j];
            if (GLOBAL) { den0 += g0; den1 += g1; }
#pragma unroll
            for (int dv = 0; dv < DV; ++dv) {
                const float4 b = *reinterpret_cast<const float4*>(sV + j * Ly::LDD + dv * 64 + tx * 4);
                o[0][dv * 4 + 0] = fmaf(g0, b.x, o[0][dv * 4 + 0]); o[1][dv * 4 + 0] = fmaf(g1, b.x, o[1][dv * 4 + 0]);
                o[0][dv * 4 + 1] = fmaf(g0, b.y, o[0][dv * 4 + 1]); o[1][dv * 4 + 1] = fmaf(g1, b.y, o[1][dv * 4 + 1]);
                o[0][dv * 4 + 2] = fmaf(g0, b.z, o[0][dv * 4 + 2]); o[1][dv * 4 + 2] = fmaf(g1, b.z, o[1][dv * 4 + 2]);
                o[0][dv * 4 + 3] = fmaf(g0, b.w, o[0][dv * 4 + 3]); o[1][dv * 4 + 3] = fmaf(g1, b.w, o[1][dv * 4 + 3]);
            }
        }

        // ---- B += pK^T V (registers are the master copy) ---------------------------------------
#pragma unroll 4
        for (int t = 0; t < C; ++t) {
            float kk[SPT];
#pragma unroll
            for (int i = 0; i < SPT; ++i) kk[i] = sK[t * Ly::LDS + ty * SPT + i];
#pragma unroll
            for (int dv = 0; dv < DV; ++dv) {
                const float4 vv = *reinterpret_cast<const float4*>(sV + t * Ly::LDD + dv * 64 + tx * 4);
#pragma unroll
                for (int i = 0; i < SPT; ++i) {
                    rB[i][dv * 4 + 0] = fmaf(kk[i], vv.x, rB[i][dv * 4 + 0]);
                    rB[i][dv * 4 + 1] = fmaf(kk[i], vv.y, rB[i][dv * 4 + 1]);
                    rB[i][dv * 4 + 2] = fmaf(kk[i], vv.z, rB[i][dv * 4 + 2]);
                    rB[i][dv * 4 + 3] = fmaf(kk[i], vv.w, rB[i][dv * 4 + 3]);
                }
            }
        }

        if (groups == 1) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int t = ty * 2 + i;
                if (GLOBAL) {
                    const float den = i ? den1 : den0;
                    const float r = den == 0.f ? 0.f : 1.f / den;
#pragma unroll
                    for (int j = 0; j < 4 * DV; ++j) o[i][j] *= r;
                }
                if (t < valid) {
#pragma unroll
                    for (int dv = 0; dv < DV; ++dv) {
                        const int c = dv * 64 + tx * 4;
                        if (c < dm.D)
                            store4_stream(out_n + (c0 + t) * dm.D + c,
                                          make_float4(o[i][dv * 4], o[i][dv * 4 + 1], o[i][dv * 4 + 2], o[i][dv * 4 + 3]));
                    }
                }
            }
            __syncthreads();  // every read of sQ/sK/sV/sB/sG of this chunk is done
        } else {
            // partial outputs of this bucket group -> own shared memory; the cluster then sums
            // them in group order (fixed, so results do not depend on timing)
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int dv = 0; dv < DV; ++dv)
                    *reinterpret_cast<float4*>(sO + (ty * 2 + i) * Ly::LDD + dv * 64 + tx * 4) =
                        make_float4(o[i][dv * 4], o[i][dv * 4 + 1], o[i][dv * 4 + 2], o[i][dv * 4 + 3]);
            if (GLOBAL && tx == 0) {   // this group's share of the denominators, in the row padding
                sO[(ty * 2) * Ly::LDD + Ly::DP] = den0;
                sO[(ty * 2 + 1) * Ly::LDD + Ly::DP] = den1;
            }
            cg::cluster_group cluster = cg::this_cluster();
            cluster.sync();
            // rows are dealt round-robin to the CTAs of the cluster
            for (int idx = tid; idx < C * (Ly::DP / 4); idx += kSimtThreads) {
                const int t = idx / (Ly::DP / 4);
                const int c = (idx % (Ly::DP / 4)) * 4;
                if ((t % groups) != group || t >= valid || c >= dm.D) continue;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                float den = 0.f;
                for (int g = 0; g < groups; ++g) {
                    const float* remote = cluster.map_shared_rank(sO, g);
                    const float4 x = *reinterpret_cast<const float4*>(remote + t * Ly::LDD + c);
                    acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
                    if (GLOBAL) den += remote[t * Ly::LDD + Ly::DP];
                }
                if (GLOBAL) {
                    const float r = den == 0.f ? 0.f : 1.f / den;
                    acc.x *= r; acc.y *= r; acc.z *= r; acc.w *= r;
                }
                store4_stream(out_n + (c0 + t) * dm.D + c, acc);
            }
            cluster.sync();
        }

        // publish the updated B for the next chunk's W B product
#pragma unroll
        for (int i = 0; i < SPT; ++i)
#pragma unroll
            for (int dv = 0; dv < DV; ++dv)
                *reinterpret_cast<float4*>(sB + (ty * SPT + i) * Ly::LDD + dv * 64 + tx * 4) =
                    make_float4(rB[i][dv * 4], rB[i][dv * 4 + 1], rB[i][dv * 4 + 2], rB[i][dv * 4 + 3]);
        // the next iteration's stage_block writes sQ/sK/sV, then __syncthreads covers sB too
    }
}

template <typename Tin, int SPT, int DV>
cudaError_t launch_simt(const Tin* pq, const Tin* pk, const Tin* v, Tin* out, const float* carry_in,
                        float* state_out, float* ws, const Dims& dm, int tile_tokens, int groups,
                        bool totals_only, bool skip_output, bool skip_totals, bool global_norm,
                        cudaStream_t stream) {
    using Ly = SimtLayout<SPT, DV>;
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    const int sf = state_floats_per_stream(dm.S, dm.D);
    dim3 grid((unsigned)(tiles * groups), (unsigned)dm.N);

    const size_t smem1 = (size_t)(C * Ly::LDS + C * Ly::LDD) * sizeof(float);
    cudaError_t err = cudaSuccess;
    if (!skip_totals) {
        tile_totals_simt<Tin, SPT, DV><<<grid, kSimtThreads, smem1, stream>>>(pk, v, ws, dm, tile_tokens, groups);
        err = cudaGetLastError();
        if (err != cudaSuccess) return err;
    }

    dim3 sgrid((unsigned)((sf + 127) / 128), (unsigned)dm.N);
    tile_scan<<<sgrid, 128, 0, stream>>>(ws, carry_in, state_out, tiles, sf, totals_only ? 0 : 1, 0);
    err = cudaGetLastError();
    if (err != cudaSuccess || totals_only || skip_output) return err;

    const size_t smem3 = (size_t)(groups > 1 ? Ly::floats_cluster : Ly::floats_single) * sizeof(float);
    auto kern = global_norm ? causal_out_simt<Tin, SPT, DV, true> : causal_out_simt<Tin, SPT, DV, false>;
    err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
    if (err != cudaSuccess) return err;
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
    return cudaLaunchKernelEx(&cfg, kern, pq, pk, v, out, (const float*)ws, dm, tile_tokens, groups);
}

template <typename Tin>
cudaError_t dispatch_simt(const void* pq, const void* pk, const void* v, void* out,
                          const float* carry_in, float* state_out, float* ws, const Dims& dm,
                          int tile_tokens, bool totals_only, bool skip_output, bool skip_totals,
                          bool global_norm, cudaStream_t stream) {
    const int groups = simt_groups(dm.S);
    const int sg = dm.S > kGroupBuckets ? kGroupBuckets : dm.S;
    const int spt = sg <= 16 ? 1 : (sg <= 32 ? 2 : 4);
    const int dv = dm.D <= 64 ? 1 : 2;
#define RACE_SIMT_CASE(SPT_, DV_)                                                                  \
    if (spt == SPT_ && dv == DV_)                                                                  \
        return launch_simt<Tin, SPT_, DV_>((const Tin*)pq, (const Tin*)pk, (const Tin*)v, (Tin*)out, \
                                           carry_in, state_out, ws, dm, tile_tokens, groups,       \
                                           totals_only, skip_output, skip_totals, global_norm, stream);
    RACE_SIMT_CASE(1, 1) RACE_SIMT_CASE(2, 1) RACE_SIMT_CASE(4, 1)
    RACE_SIMT_CASE(1, 2) RACE_SIMT_CASE(2, 2) RACE_SIMT_CASE(4, 2)
#undef RACE_SIMT_CASE
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t causal_scan_tiles(float* ws, const float* carry_in, float* state_out, const Dims& dm,
                              int tile_tokens, cudaStream_t stream, bool write_prefix, bool reverse) {
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    const int sf = state_floats_per_stream(dm.S, dm.D);
    if (tiles == 1 && !carry_in && !write_prefix && state_out)   // one tile per stream: its totals are the state
        return cudaMemcpyAsync(state_out, ws, (size_t)dm.N * sf * sizeof(float), cudaMemcpyDeviceToDevice, stream);
    dim3 sgrid((unsigned)((sf + 127) / 128), (unsigned)dm.N);
    tile_scan<<<sgrid, 128, 0, stream>>>(ws, carry_in, state_out, tiles, sf, write_prefix ? 1 : 0, reverse ? 1 : 0);
    return cudaGetLastError();
}

int simt_groups(int S) { return S <= kGroupBuckets ? 1 : (S + kGroupBuckets - 1) / kGroupBuckets; }

bool simt_supported(const Dims& dm) {
    if (dm.S <= 0 || dm.D <= 0 || dm.D > 128) return false;
    if (dm.S > kGroupBuckets && (dm.S % kGroupBuckets != 0 || dm.S > 8 * kGroupBuckets)) return false;
    return dm.N >= 0 && dm.N <= 65535 && dm.T >= 0;
}

int simt_default_tile_tokens(const Dims& dm, int sm_count) {
    // Largest power-of-two tile <= 2048 tokens (state traffic <= ~5 % of token traffic) that
    // still gives about four CTAs per SM; never below one chunk.
    const int64_t want = (int64_t)sm_count * 4;
    int tile = 2048;
    while (tile > C && dm.N * simt_groups(dm.S) * ((dm.T + tile - 1) / tile) < want) tile >>= 1;
    return tile;
}

cudaError_t causal_fwd_simt(const void* pq, const void* pk, const void* v, void* out,
                            const float* carry_in, float* state_out, float* ws, const Dims& dm,
                            int dtype, int tile_tokens, bool totals_only, cudaStream_t stream,
                            bool skip_output, bool skip_totals, bool global_norm) {
    if (dtype == RACE_DTYPE_F32)
        return dispatch_simt<float>(pq, pk, v, out, carry_in, state_out, ws, dm, tile_tokens,
                                    totals_only, skip_output, skip_totals, global_norm, stream);
    return dispatch_simt<__nv_bfloat16>(pq, pk, v, out, carry_in, state_out, ws, dm, tile_tokens,
                                        totals_only, skip_output, skip_totals, global_norm, stream);
}

}  // namespace race
