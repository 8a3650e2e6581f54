// Non-causal per-bucket forward and backward (CUDA cores, fp32 accumulate).
//
//   forward :  Bs = pK^T V, A = sum_t pK        (tile totals + tile reduction, causal_simt.cu)
//              E  = Bs/(A+eps);  out = pQ E     (nc_query)
//   backward:  dE = pQ^T dO                     (tile totals with (pQ, dO) in place of (pK, V))
//              dBs = dE/(A+eps); dA[s] = -sum_c dE[s,c] E[s,c]/(A[s]+eps)      (nc_state_grads)
//              dPQ = dO E^T; dPK[t,s] = V[t].dBs[s] + dA[s]; dV = pK dBs       (nc_token_grads)
// The forward is the four lines the reference quotes from upstream
// (analysis/hot-path.md:157-162); the gradient formulas are the closed form of that function
// (checked against torch.autograd in the oracle's tests).
#include "common.cuh"
#include "launch.h"

namespace race {
namespace {

constexpr int C = kSimtChunk;

// o[i][:] += sum_s sX[(ty*2+i)][s] * sZ[s][dv*64 + tx*4 ..]   (rows x state)
template <int DV>
__device__ __forceinline__ void mm_rows_state(float (&o)[2][4 * DV], const float* sX, int ldx,
                                              const float* sZ, int ldz, int SG, int ty, int tx) {
#pragma unroll 4
    for (int s = 0; s < SG; ++s) {
        const float w0 = sX[(ty * 2) * ldx + s], w1 = sX[(ty * 2 + 1) * ldx + s];
#pragma unroll
        for (int dv = 0; dv < DV; ++dv) {
            const float4 b = *reinterpret_cast<const float4*>(sZ + s * ldz + dv * 64 + tx * 4);
            o[0][dv * 4 + 0] = fmaf(w0, b.x, o[0][dv * 4 + 0]); o[1][dv * 4 + 0] = fmaf(w1, b.x, o[1][dv * 4 + 0]);
            o[0][dv * 4 + 1] = fmaf(w0, b.y, o[0][dv * 4 + 1]); o[1][dv * 4 + 1] = fmaf(w1, b.y, o[1][dv * 4 + 1]);
            o[0][dv * 4 + 2] = fmaf(w0, b.z, o[0][dv * 4 + 2]); o[1][dv * 4 + 2] = fmaf(w1, b.z, o[1][dv * 4 + 2]);
            o[0][dv * 4 + 3] = fmaf(w0, b.w, o[0][dv * 4 + 3]); o[1][dv * 4 + 3] = fmaf(w1, b.w, o[1][dv * 4 + 3]);
        }
    }
}

// acc[i][j] = sum_c sX[(ty*2+i)][c] * sZ[tx + 16*j][c]   (rows x state^T), c over DP
template <int SPT>
__device__ __forceinline__ void mm_rows_stateT(float (&acc)[2][SPT], const float* sX, const float* sZ,
                                               int ldd, int DP, int ty, int tx) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < SPT; ++j) acc[i][j] = 0.f;
#pragma unroll 2
    for (int c = 0; c < DP; c += 4) {
        const float4 x0 = *reinterpret_cast<const float4*>(sX + (ty * 2) * ldd + c);
        const float4 x1 = *reinterpret_cast<const float4*>(sX + (ty * 2 + 1) * ldd + c);
#pragma unroll
        for (int j = 0; j < SPT; ++j) {
            const float4 z = *reinterpret_cast<const float4*>(sZ + (tx + 16 * j) * ldd + c);
            acc[0][j] += x0.x * z.x + x0.y * z.y + x0.z * z.z + x0.w * z.w;
            acc[1][j] += x1.x * z.x + x1.y * z.y + x1.z * z.z + x1.w * z.w;
        }
    }
}

// Stage one bucket group of a per-stream state into shared memory:
//   mode 0: E = B/(A+eps)        (from the forward totals)
//   mode 1: rows copied as they are (dBs)
template <int SPT, int DV>
__device__ __forceinline__ void stage_state(float* sZ, const float* state, int S, int D, int s0,
                                            int s_valid, float eps, int mode, int tid) {
    constexpr int SG = 16 * SPT, DP = 64 * DV, LDD = DP + 4;
    for (int i = tid; i < SG * (DP / 4); i += kSimtThreads) {
        const int s = i / (DP / 4), c = (i % (DP / 4)) * 4;
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (s < s_valid && c < D) {
            b = load4(state + (int64_t)(s0 + s) * D + c);
            if (mode == 0) {
                const float inv = 1.f / (state[(int64_t)S * D + s0 + s] + eps);
                b.x *= inv; b.y *= inv; b.z *= inv; b.w *= inv;
            }
        }
        *reinterpret_cast<float4*>(sZ + s * LDD + c) = b;
    }
}

// ------------------------------------------------------------------------------------------
// forward: out = pQ E
// ------------------------------------------------------------------------------------------
template <typename Tin, int SPT, int DV>
__global__ void __launch_bounds__(kSimtThreads)
nc_query(const Tin* __restrict__ pq, const float* __restrict__ totals, Tin* __restrict__ out,
         Dims dm, int tile_tokens, int groups) {
    constexpr int SG = 16 * SPT, DP = 64 * DV, LDS = SG + 4, LDD = DP + 4;
    extern __shared__ __align__(16) float smem[];
    float* sQ = smem;
    float* sE = smem + C * LDS;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int64_t n = blockIdx.y;
    const int64_t t_begin = (int64_t)blockIdx.x * tile_tokens;
    const int64_t t_end = min(dm.T, t_begin + tile_tokens);
    const Tin* pq_n = pq + n * dm.T * dm.S;
    Tin* out_n = out + n * dm.T * dm.D;
    const float* st = totals + n * (int64_t)state_floats_per_stream(dm.S, dm.D);

    if (groups == 1) stage_state<SPT, DV>(sE, st, dm.S, dm.D, 0, min(dm.S, SG), dm.eps, 0, tid);
    for (int64_t c0 = t_begin; c0 < t_end; c0 += C) {
        const int valid = (int)min((int64_t)C, t_end - c0);
        float o[2][4 * DV];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4 * DV; ++j) o[i][j] = 0.f;
        for (int g = 0; g < groups; ++g) {
            const int s0 = g * kGroupBuckets;
            const int s_valid = min(dm.S - s0, SG);
            __syncthreads();
            stage_block(sQ, LDS, pq_n, c0, C, valid, dm.S, s0, SG, s_valid, tid, kSimtThreads);
            if (groups > 1) stage_state<SPT, DV>(sE, st, dm.S, dm.D, s0, s_valid, dm.eps, 0, tid);
            __syncthreads();
            mm_rows_state<DV>(o, sQ, LDS, sE, LDD, SG, ty, tx);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int t = ty * 2 + i;
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
    }
}

// ------------------------------------------------------------------------------------------
// backward, state part: grads [N][S*D + S] = (dBs, dA) from totals (Bs, A) and dE
// one warp per (stream, bucket)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
nc_state_grads(const float* __restrict__ totals, const float* __restrict__ dE_state,
               float* __restrict__ grads, int64_t N, int S, int D, float eps) {
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= N * S) return;
    const int64_t n = warp / S;
    const int s = (int)(warp % S);
    const int64_t base = n * (int64_t)state_floats_per_stream(S, D);
    const float inv = 1.f / (totals[base + (int64_t)S * D + s] + eps);
    float dot = 0.f;
    for (int c = lane; c < D; c += 32) {
        const float de = dE_state[base + (int64_t)s * D + c];
        const float e = totals[base + (int64_t)s * D + c] * inv;
        grads[base + (int64_t)s * D + c] = de * inv;
        dot += de * e;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    if (lane == 0) grads[base + (int64_t)S * D + s] = -dot * inv;
}

// ------------------------------------------------------------------------------------------
// backward, token part
// ------------------------------------------------------------------------------------------
template <typename Tin, int SPT, int DV>
__global__ void __launch_bounds__(kSimtThreads)
nc_token_grads(const Tin* __restrict__ pk, const Tin* __restrict__ v, const Tin* __restrict__ dout,
               const float* __restrict__ totals, const float* __restrict__ grads,
               Tin* __restrict__ dpq, Tin* __restrict__ dpk, Tin* __restrict__ dv_out, Dims dm,
               int tile_tokens, int groups) {
    constexpr int SG = 16 * SPT, DP = 64 * DV, LDS = SG + 4, LDD = DP + 4;
    extern __shared__ __align__(16) float smem[];
    float* sdO = smem;
    float* sV = sdO + C * LDD;
    float* sK = sV + C * LDD;
    float* sE = sK + C * LDS;
    float* sdB = sE + SG * LDD;
    float* sdA = sdB + SG * LDD;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int64_t n = blockIdx.y;
    const int64_t t_begin = (int64_t)blockIdx.x * tile_tokens;
    const int64_t t_end = min(dm.T, t_begin + tile_tokens);
    const int64_t sf = state_floats_per_stream(dm.S, dm.D);
    const float* st = totals + n * sf;
    const float* gr = grads + n * sf;
    const Tin* pk_n = pk + n * dm.T * dm.S;
    const Tin* v_n = v + n * dm.T * dm.D;
    const Tin* do_n = dout + n * dm.T * dm.D;
    Tin* dpq_n = dpq + n * dm.T * dm.S;
    Tin* dpk_n = dpk + n * dm.T * dm.S;
    Tin* dv_n = dv_out + n * dm.T * dm.D;

    auto stage_group = [&](int s0, int s_valid) {
        stage_state<SPT, DV>(sE, st, dm.S, dm.D, s0, s_valid, dm.eps, 0, tid);
        stage_state<SPT, DV>(sdB, gr, dm.S, dm.D, s0, s_valid, dm.eps, 1, tid);
        if (tid < SG) sdA[tid] = tid < s_valid ? gr[(int64_t)dm.S * dm.D + s0 + tid] : 0.f;
    };
    if (groups == 1) stage_group(0, min(dm.S, SG));

    for (int64_t c0 = t_begin; c0 < t_end; c0 += C) {
        const int valid = (int)min((int64_t)C, t_end - c0);
        __syncthreads();
        stage_block(sdO, LDD, do_n, c0, C, valid, dm.D, 0, DP, dm.D, tid, kSimtThreads);
        stage_block(sV, LDD, v_n, c0, C, valid, dm.D, 0, DP, dm.D, tid, kSimtThreads);
        float o[2][4 * DV];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4 * DV; ++j) o[i][j] = 0.f;
        for (int g = 0; g < groups; ++g) {
            const int s0 = g * kGroupBuckets;
            const int s_valid = min(dm.S - s0, SG);
            if (g > 0) __syncthreads();
            stage_block(sK, LDS, pk_n, c0, C, valid, dm.S, s0, SG, s_valid, tid, kSimtThreads);
            if (groups > 1) stage_group(s0, s_valid);
            __syncthreads();
            float a[2][SPT];
            mm_rows_stateT<SPT>(a, sdO, sE, LDD, DP, ty, tx);  // dPQ = dO E^T
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int t = ty * 2 + i;
#pragma unroll
                for (int j = 0; j < SPT; ++j) {
                    const int s = tx + 16 * j;
                    if (t < valid && s < s_valid) dpq_n[(c0 + t) * dm.S + s0 + s] = (Tin)a[i][j];
                }
            }
            mm_rows_stateT<SPT>(a, sV, sdB, LDD, DP, ty, tx);  // dPK = V dBs^T + dA
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int t = ty * 2 + i;
#pragma unroll
                for (int j = 0; j < SPT; ++j) {
                    const int s = tx + 16 * j;
                    if (t < valid && s < s_valid)
                        dpk_n[(c0 + t) * dm.S + s0 + s] = (Tin)(a[i][j] + sdA[s]);
                }
            }
            mm_rows_state<DV>(o, sK, LDS, sdB, LDD, SG, ty, tx);  // dV += pK dBs
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int t = ty * 2 + i;
            if (t < valid) {
#pragma unroll
                for (int dv = 0; dv < DV; ++dv) {
                    const int c = dv * 64 + tx * 4;
                    if (c < dm.D)
                        store4_stream(dv_n + (c0 + t) * dm.D + c,
                                      make_float4(o[i][dv * 4], o[i][dv * 4 + 1], o[i][dv * 4 + 2], o[i][dv * 4 + 3]));
                }
            }
        }
    }
}

struct NcPick { int spt, dv, groups; };
NcPick pick(const Dims& dm) {
    const int sg = dm.S > kGroupBuckets ? kGroupBuckets : dm.S;
    return {sg <= 16 ? 1 : (sg <= 32 ? 2 : 4), dm.D <= 64 ? 1 : 2, simt_groups(dm.S)};
}

int token_tile(const Dims& dm, int sm_count) {
    int tile = 1024;
    while (tile > C && dm.N * ((dm.T + tile - 1) / tile) < (int64_t)sm_count * 4) tile >>= 1;
    return tile;
}

template <typename Tin, int SPT, int DV>
cudaError_t launch_query(const void* pq, const float* totals, void* out, const Dims& dm, int groups,
                         int sm_count, cudaStream_t stream) {
    constexpr int SG = 16 * SPT, DP = 64 * DV;
    const int tile = token_tile(dm, sm_count);
    const size_t smem = (size_t)(C * (SG + 4) + SG * (DP + 4)) * sizeof(float);
    auto kern = nc_query<Tin, SPT, DV>;
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    dim3 grid((unsigned)((dm.T + tile - 1) / tile), (unsigned)dm.N);
    kern<<<grid, kSimtThreads, smem, stream>>>((const Tin*)pq, totals, (Tin*)out, dm, tile, groups);
    return cudaGetLastError();
}

template <typename Tin, int SPT, int DV>
cudaError_t launch_token_grads(const void* pk, const void* v, const void* dout, const float* totals,
                               const float* grads, void* dpq, void* dpk, void* dv, const Dims& dm,
                               int groups, int sm_count, cudaStream_t stream) {
    constexpr int SG = 16 * SPT, DP = 64 * DV;
    const int tile = token_tile(dm, sm_count);
    const size_t smem = (size_t)(2 * C * (DP + 4) + C * (SG + 4) + 2 * SG * (DP + 4) + SG) * sizeof(float);
    auto kern = nc_token_grads<Tin, SPT, DV>;
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    dim3 grid((unsigned)((dm.T + tile - 1) / tile), (unsigned)dm.N);
    kern<<<grid, kSimtThreads, smem, stream>>>((const Tin*)pk, (const Tin*)v, (const Tin*)dout, totals,
                                               grads, (Tin*)dpq, (Tin*)dpk, (Tin*)dv, dm, tile, groups);
    return cudaGetLastError();
}

}  // namespace

#define RACE_NC_DISPATCH(FN, ...)                                                      \
    do {                                                                               \
        const NcPick p = pick(dm);                                                     \
        if (dtype == RACE_DTYPE_F32) {                                                 \
            if (p.spt == 1 && p.dv == 1) return FN<float, 1, 1>(__VA_ARGS__);          \
            if (p.spt == 2 && p.dv == 1) return FN<float, 2, 1>(__VA_ARGS__);          \
            if (p.spt == 4 && p.dv == 1) return FN<float, 4, 1>(__VA_ARGS__);          \
            if (p.spt == 1 && p.dv == 2) return FN<float, 1, 2>(__VA_ARGS__);          \
            if (p.spt == 2 && p.dv == 2) return FN<float, 2, 2>(__VA_ARGS__);          \
            if (p.spt == 4 && p.dv == 2) return FN<float, 4, 2>(__VA_ARGS__);          \
        } else {                                                                       \
            if (p.spt == 1 && p.dv == 1) return FN<__nv_bfloat16, 1, 1>(__VA_ARGS__);  \
            if (p.spt == 2 && p.dv == 1) return FN<__nv_bfloat16, 2, 1>(__VA_ARGS__);  \
            if (p.spt == 4 && p.dv == 1) return FN<__nv_bfloat16, 4, 1>(__VA_ARGS__);  \
            if (p.spt == 1 && p.dv == 2) return FN<__nv_bfloat16, 1, 2>(__VA_ARGS__);  \
            if (p.spt == 2 && p.dv == 2) return FN<__nv_bfloat16, 2, 2>(__VA_ARGS__);  \
            if (p.spt == 4 && p.dv == 2) return FN<__nv_bfloat16, 4, 2>(__VA_ARGS__);  \
        }                                                                              \
        return cudaErrorInvalidValue;                                                  \
    } while (0)

cudaError_t noncausal_query(const void* pq, const float* totals, void* out, const Dims& dm, int dtype,
                            int sm_count, cudaStream_t stream) {
    RACE_NC_DISPATCH(launch_query, pq, totals, out, dm, p.groups, sm_count, stream);
}

cudaError_t noncausal_state_grads(const float* totals, const float* dE_state, float* grads,
                                  const Dims& dm, cudaStream_t stream) {
    const int64_t warps = dm.N * dm.S;
    const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
    nc_state_grads<<<blocks, 256, 0, stream>>>(totals, dE_state, grads, dm.N, dm.S, dm.D, dm.eps);
    return cudaGetLastError();
}

cudaError_t noncausal_token_grads(const void* pk, const void* v, const void* dout, const float* totals,
                                  const float* grads, void* dpq, void* dpk, void* dv, const Dims& dm,
                                  int dtype, int sm_count, cudaStream_t stream) {
    RACE_NC_DISPATCH(launch_token_grads, pk, v, dout, totals, grads, dpq, dpk, dv, dm, p.groups,
                     sm_count, stream);
}

}  // namespace race
