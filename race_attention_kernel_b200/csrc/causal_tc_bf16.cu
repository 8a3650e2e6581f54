// tcgen05 / TMEM / TMA causal kernels for bf16 inputs (sm_100a): S = G * 64 buckets, d_k in
// {64, 128}.  Same chunk identity and warp roles as the fp32 kernels (causal_tc.cu); what
// differs:
//   * operands are single bf16 tiles (the inputs already are bf16): every product is one
//     tcgen05.mma pass, and the converter warps only move the TMA-staged (128B-swizzled) tiles
//     into the canonical operand layout;
//   * d_k = 128 runs the state update, W.B and G.V with N = 128 (TMEM: B 128 + 2 x (64 + 128)
//     columns = all 512);
//   * S > 64 (2, 4 or 8 groups of 64 buckets): the tables of this estimator are independent (out = sum
//     over tables), and the sum over groups commutes with the causal mask; causal_out_wide_bf16 (below)
//     walks all groups in one CTA and accumulates their products in tensor memory.  No thread-block
//     clusters, no TMA multicast anywhere.
// Reference semantics: src/race_baseline.py:45-51 (docs/causal_v2_design.md:70-77 for the chunk
// form).  The multi-head configuration N=256 streams, T=262144, d_k=128, L=8, K=6 is G = 8, D = 128.
#include <cudaTypedefs.h>

#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"

namespace race {
namespace {

constexpr int C = 64;   // tokens per chunk
constexpr int SG = 64;  // buckets per CTA
constexpr int kThreads = 15 * 32;
constexpr int kProducerWarp = 12;
constexpr int kMmaWarp = 13;

template <int D>
struct Lay {
    static constexpr int kTileP = C * 64 * 2;   // pK / W / G / tril tile: 64 x 64 bf16
    static constexpr int kTileV = C * D * 2;    // V / B tile: 64 x D bf16
    static constexpr int kStage = kTileP + kTileV;
    static constexpr int oStage = 0;                    // [2] pK | V (D/64 boxes)
    static constexpr int oKt = oStage + 2 * kStage;     // [2]
    static constexpr int oVt = oKt + 2 * kTileP;        // [2]
    static constexpr int oWt = oVt + 2 * kTileV;        // [2] W, then masked G
    static constexpr int oBt = oWt + 2 * kTileP;        // [2]
    static constexpr int oTril = oBt + 2 * kTileV;
    static constexpr int oAcar = oTril + kTileP;        // [2][64] fp32
    static constexpr int oPq = (oAcar + 2 * 64 * 4 + 1023) / 1024 * 1024;   // [2 wg][kTileP] pQ of the group's next chunk
    static constexpr int oBars = oPq + 2 * kTileP;
    static constexpr int kNumBars = 36;
    static constexpr int oMisc = oBars + kNumBars * 8;
    static constexpr int kSmem = oMisc + 16 + 1024;
    // MN-major descriptor words of a [64][D] tile
    static constexpr uint32_t kLboV = (uint32_t)(D / 8) * 128;        // K-direction (row-group) stride
    static constexpr uint32_t kStepV = (2 * kLboV) >> 4;              // lo-word step per 16 K-rows
};

enum BarB {
    bFull = 0, bEmpty = 2, bKReady = 4, bVReady = 6, bXReady = 8, bWReady = 10, bGReady = 12,
    bGtReady = 14, bOReady = 16, bAcar = 18, bAcarFree = 20, bBupdDone = 22, bBaccFree = 23,
    bBtReady = 25, bDrain = 27,
    bPqFull = 29,    // [2] pQ tile of the worker group's next chunk has landed
    bPqEmpty = 31    // [2] ... copied to registers by the four warps
};

__device__ __forceinline__ uint32_t lo_mn_w(uint32_t addr, uint32_t lbo) {
    return ((addr >> 4) & 0x3FFF) | ((lbo >> 4) << 16);
}
__device__ __forceinline__ constexpr uint32_t idesc_n(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((64u >> 4) << 24);
}
// byte offset of (row, col) in a [64][W] bf16 tile of 8x8 core matrices
template <int W>
__device__ __forceinline__ uint32_t off_w(int row, int col) {
    return (uint32_t)((((row >> 3) * (W / 8) + (col >> 3)) << 7) + ((row & 7) << 4) + ((col & 7) << 1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}

// TMA-staged bf16 tile [64 rows][64 values] (128-byte rows, 128B swizzle) -> operand tile
// [64][W] columns [col0, col0 + 64); optionally adds the values into per-thread column sums
template <int W, bool kSum>
__device__ __forceinline__ void copy_tile(const uint8_t* stage, uint8_t* dst, int col0, int tid,
                                          float (*asum)[8]) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 128 + tid;
        const int j = idx >> 6, r = idx & 63;   // 16-byte chunk (8 values), token row
        const uint4 x = *reinterpret_cast<const uint4*>(stage + r * 128 + ((j ^ (r & 7)) << 4));
        if (kSum) {
            const float2 a = unpack_bf16(x.x), b = unpack_bf16(x.y), c = unpack_bf16(x.z), d = unpack_bf16(x.w);
            asum[it][0] += a.x; asum[it][1] += a.y; asum[it][2] += b.x; asum[it][3] += b.y;
            asum[it][4] += c.x; asum[it][5] += c.y; asum[it][6] += d.x; asum[it][7] += d.y;
        }
        *reinterpret_cast<uint4*>(dst + off_w<W>(r, col0 + 8 * j)) = x;
    }
}

// ------------------------------------------------------------------------------------------------
// output pass
// ------------------------------------------------------------------------------------------------
// kGlobal: the global-normalisation estimator (src/causal_v2/reference.py:106-127): W = pQ as given (bf16 inputs
// need no rounding then, so numerator and normaliser see the same values) and each output row divided by
// den_t = pQ_t . A_t (a zero denominator gives a row of zeros).
template <int D, bool kGlobal>
__global__ void __launch_bounds__(kThreads, 1)
causal_out_tc_bf16(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                   const float* __restrict__ ws, int64_t T, int S, int G, int tile_tokens, float eps,
                   int* status) {
    using Ly = Lay<D>;
    constexpr int DH = D / 64;   // 64-column halves of a [64][D] accumulator
    extern __shared__ uint8_t smem_raw[];
    Ctx cx;
    cx.sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    cx.sm_u32 = smem_u32(cx.sm);
    cx.bars = Ly::oBars;
    cx.abort_flag = reinterpret_cast<volatile int*>(cx.sm + Ly::oMisc + 4);
    cx.status = status;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(cx.sm + Ly::oMisc);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = (int)(blockIdx.x % (unsigned)G);          // bucket group = rank in the cluster
    const int64_t tiles = gridDim.x / G;
    const int64_t tile = blockIdx.x / G, n = blockIdx.y;
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(T, t_begin + (int64_t)tile_tokens);
    const int nch = (int)((t_end - t_begin + C - 1) / C);
    const float* slice = ws + (n * tiles + tile) * (int64_t)(S * (D + 1));
    const float* sliceB = slice + (int64_t)g * SG * D;      // this group's rows of B
    const float* sliceA = slice + (int64_t)S * D + g * SG;  // this group's part of A

    if (tid == 0) {
        *cx.abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(cx.bar(bFull + i), 1);
            mbar_init(cx.bar(bEmpty + i), 4);
            mbar_init(cx.bar(bKReady + i), 4);
            mbar_init(cx.bar(bVReady + i), 4);
            mbar_init(cx.bar(bXReady + i), 1);
            mbar_init(cx.bar(bWReady + i), 4);
            mbar_init(cx.bar(bGReady + i), 1);
            mbar_init(cx.bar(bGtReady + i), 4);
            mbar_init(cx.bar(bOReady + i), 1);
            mbar_init(cx.bar(bAcar + i), 1);
            mbar_init(cx.bar(bAcarFree + i), 4);
            mbar_init(cx.bar(bBaccFree + i), 4);
            mbar_init(cx.bar(bBtReady + i), 4);
            mbar_init(cx.bar(bDrain + i), 1);
            mbar_init(cx.bar(bPqFull + i), 1);
            mbar_init(cx.bar(bPqEmpty + i), 4);
        }
        mbar_init(cx.bar(bBupdDone), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(cx.sm_u32 + Ly::oMisc), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < C * 8; i += kThreads) {   // tril[t][j] = (j <= t)
        const int t = i >> 3, jg = i & 7;
        uint32_t w[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int j0 = jg * 8 + 2 * p;
            w[p] = (j0 <= t ? 0x3F80u : 0u) | (j0 + 1 <= t ? 0x3F800000u : 0u);
        }
        *reinterpret_cast<uint4*>(cx.sm + Ly::oTril + off_w<64>(t, jg * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmB = tmem;                                                   // [0, D)
    auto tmAG = [&](int wg) { return tmem + D + wg * (64 + D); };                // A_loc, then G
    auto tmO = [&](int wg) { return tmem + D + wg * (64 + D) + 64; };            // O
    // d_k = 64 leaves 192 columns: W / masked G and the triangular ones matrix are MMA A operands in
    // tensor memory (bf16 pairs, 32 columns each) instead of operand tiles in shared memory
    constexpr bool kTA = (D == 64);
    auto tmW = [&](int wg) { return tmem + 320 + wg * 32; };
    const uint32_t tmTril = tmem + 384;

    if (warp < 8) {
        // =========================== worker warpgroups =========================================
        const int wg = warp >> 2, w = warp & 3;
        const int q = lane & 3, rbase = 16 * w + (lane >> 2);
        const uint32_t lane_base = (uint32_t)(32 * w) << 16;
        uint8_t* wt = cx.sm + Ly::oWt + wg * Ly::kTileP;
        __nv_bfloat16* out_n = out + n * T * D;
        const uint8_t* pq_tile = cx.sm + Ly::oPq + wg * Ly::kTileP;
        float v[32];
        uint32_t ov[16];   // W / masked G pairs on their way to tensor memory (d_k = 64)
        float den[2] = {1.f, 1.f};   // global form: denominators of rows rbase, rbase + 8 of the chunk
        uint32_t ph = 0;
        bool ok = true;
        for (int c = wg; c < nch && ok; c += 2, ph ^= 1) {
            const int64_t tok0 = t_begin + (int64_t)c * C;
            const int valid = (int)min((int64_t)C, t_end - tok0);
            // pQ in the accumulator-fragment layout (pairs of bf16) from the group's TMA-staged tile ([64 tokens][64
            // buckets], 128-byte rows, 128B swizzle: the eight rows a warp instruction reads fall on different banks; rows
            // past the end of the sequence are zero).  The 4-byte global loads this replaces touched eight rows each.
            RACE_TRACE(wg, c >> 1, 0);
            uint32_t pqv[16];
            if (!(ok = wait_bar_warp(cx, bPqFull + wg, ph, 105))) break;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rbase + 8 * h;
#pragma unroll
                for (int x = 0; x < 8; ++x)
                    pqv[2 * x + h] = *reinterpret_cast<const uint32_t*>(pq_tile + row * 128 + ((x ^ (row & 7)) << 4) + 4 * q);
            }
            // generic-proxy reads before the async-proxy write of the next tile: proxy fence, then the slot goes back
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(bPqEmpty + wg));
            // ---- W = pQ / (A + A_loc + eps) --------------------------------------------------------
            if (!(ok = wait_bar_warp(cx, bAcar + wg, ph, 102))) break;
            float acar[16];
            {
                const float* ac = reinterpret_cast<const float*>(cx.sm + Ly::oAcar) + wg * 64;
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    const float2 a2 = *reinterpret_cast<const float2*>(ac + 8 * x + 2 * q);
                    acar[2 * x] = a2.x; acar[2 * x + 1] = a2.y;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(bAcarFree + wg));
            if (w == 3 && c >= 1 && !(ok = wait_bar_warp(cx, bAcarFree + (wg ^ 1), ((c - 1) >> 1) & 1, 107))) break;
            if (!(ok = wait_bar_warp(cx, bXReady + wg, ph, 103))) break;
            tc_fence_after();
            tmem_ld64(lane_base + tmAG(wg), v);
            tc_fence_before();
            if (kGlobal) den[0] = den[1] = 0.f;
#pragma unroll
            for (int x = 0; x < 8; ++x) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = rbase + 8 * h;
                    const float2 pq2 = unpack_bf16(pqv[2 * x + h]);
                    const float a0 = acar[2 * x] + v[4 * x + 2 * h];
                    const float a1 = acar[2 * x + 1] + v[4 * x + 2 * h + 1];
                    uint32_t wp;
                    if (kGlobal) {
                        wp = pqv[2 * x + h];
                        den[h] = fmaf(pq2.x, a0, fmaf(pq2.y, a1, den[h]));
                    } else {
                        wp = pack_bf16(__fdividef(pq2.x, a0 + eps), __fdividef(pq2.y, a1 + eps));
                    }
                    if constexpr (kTA) ov[2 * x + h] = wp;
                    else *reinterpret_cast<uint32_t*>(wt + off_w<64>(row, 8 * x + 2 * q)) = wp;
                    if (h == 1 && w == 3 && (lane >> 2) == 7) {
                        float* an = reinterpret_cast<float*>(cx.sm + Ly::oAcar) + (wg ^ 1) * 64;
                        *reinterpret_cast<float2*>(an + 8 * x + 2 * q) = make_float2(a0, a1);
                    }
                }
            }
            if constexpr (kTA) {
                tmem_st_pairs(lane_base + tmW(wg), ov);
                tmem_wait_st();
                tc_fence_before();
            } else {
                fence_proxy_async();
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(cx.bar(bWReady + wg));
                if (w == 3) mbar_arrive(cx.bar(bAcar + (wg ^ 1)));
            }
            if (kGlobal) {
                // a row's 64 buckets are spread over the four lanes of a quad
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    den[h] += __shfl_xor_sync(0xffffffffu, den[h], 1);
                    den[h] += __shfl_xor_sync(0xffffffffu, den[h], 2);
                }
            }
            // ---- causal mask of G (over W's tile) ----------------------------------------------
            if (!(ok = wait_bar_warp(cx, bGReady + wg, ph, 104))) break;
            tc_fence_after();
            tmem_ld64(lane_base + tmAG(wg), v);
            tc_fence_before();
#pragma unroll
            for (int x = 0; x < 8; ++x) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = rbase + 8 * h, col = 8 * x + 2 * q;
                    const uint32_t gp =
                        pack_bf16(col <= row ? v[4 * x + 2 * h] : 0.f, col + 1 <= row ? v[4 * x + 2 * h + 1] : 0.f);
                    if constexpr (kTA) ov[2 * x + h] = gp;
                    else *reinterpret_cast<uint32_t*>(wt + off_w<64>(row, col)) = gp;
                }
            }
            if constexpr (kTA) {
                tmem_st_pairs(lane_base + tmW(wg), ov);
                tmem_wait_st();
                tc_fence_before();
            } else {
                fence_proxy_async();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(bGtReady + wg));
            // ---- O ---------------------------------------------------------------------------------
            RACE_TRACE(wg, c >> 1, 1);
            if (!(ok = wait_bar_warp(cx, bOReady + wg, ph, 105))) break;
            RACE_TRACE(wg, c >> 1, 2);
#pragma unroll
            for (int dh = 0; dh < DH; ++dh) {
                tc_fence_after();
                tmem_ld64(lane_base + tmO(wg) + dh * 64, v);
                tc_fence_before();
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = rbase + 8 * h;
                    if (row < valid) {
                        __nv_bfloat16* orow = out_n + (tok0 + row) * D + dh * 64 + 2 * q;
                        const float sc = kGlobal ? (den[h] != 0.f ? 1.f / den[h] : 0.f) : 1.f;
#pragma unroll
                        for (int x = 0; x < 8; ++x)
                            *reinterpret_cast<uint32_t*>(orow + 8 * x) =
                                pack_bf16(v[4 * x + 2 * h] * sc, v[4 * x + 2 * h + 1] * sc);
                    }
                }
            }
        }
    } else if (warp < 12) {
        // =========================== converter + carry warpgroup =================================
        const int w = warp & 3, q = lane & 3, rbase = 16 * w + (lane >> 2), wtid = tid & 127;
        const uint32_t lane_base = (uint32_t)(32 * w) << 16;
        float v[32];
        auto write_bt = [&](int buf, int dh) {
            uint8_t* bt = cx.sm + Ly::oBt + buf * Ly::kTileV;
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    *reinterpret_cast<uint32_t*>(bt + off_w<D>(rbase + 8 * h, dh * 64 + 8 * x + 2 * q)) =
                        pack_bf16(v[4 * x + 2 * h], v[4 * x + 2 * h + 1]);
        };
        if constexpr (kTA) {   // tril[t][j] = (j <= t) as an A operand in tensor memory
            uint32_t tr[16];
#pragma unroll
            for (int y = 0; y < 8; ++y)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = rbase + 8 * h, j0 = 8 * y + 2 * q;
                    tr[2 * y + h] = (j0 <= row ? 0x3F80u : 0u) | (j0 + 1 <= row ? 0x3F800000u : 0u);
                }
            tmem_st_pairs(lane_base + tmTril, tr);
        }
        // carry-in: B -> TMEM accumulator and operand buffer 0; A -> the first chunk's running A
#pragma unroll
        for (int dh = 0; dh < DH; ++dh) {
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float2 b2 = *reinterpret_cast<const float2*>(
                        sliceB + (rbase + 8 * h) * D + dh * 64 + 8 * x + 2 * q);
                    v[4 * x + 2 * h] = b2.x; v[4 * x + 2 * h + 1] = b2.y;
                }
            tmem_st64(lane_base + tmB + dh * 64, v);
            write_bt(0, dh);
        }
        tc_fence_before();
        if (warp == 8) {
            float* ac = reinterpret_cast<float*>(cx.sm + Ly::oAcar);
            ac[lane] = sliceA[lane];
            ac[lane + 32] = sliceA[lane + 32];
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(cx.bar(bBaccFree + 0));
            mbar_arrive(cx.bar(bBtReady + 0));
            if (warp == 8) mbar_arrive(cx.bar(bAcar + 0));
        }
        bool ok = true;
        for (int c = 0; c < nch && ok; ++c) {
            const int wg = c & 1;
            const uint32_t ph = (uint32_t)((c >> 1) & 1);
            const uint8_t* stage = cx.sm + Ly::oStage + wg * Ly::kStage;
            // pK tile of the group: last read by the G product of chunk c - 2
            if (c >= 2 && !(ok = wait_bar_warp(cx, bGReady + wg, ph ^ 1, 203))) break;
            if (!(ok = wait_bar_warp(cx, bFull + wg, ph, 201))) break;
            copy_tile<64, false>(stage, cx.sm + Ly::oKt + wg * Ly::kTileP, 0, wtid, nullptr);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(bKReady + wg));
            if (c >= 1) {
                // state after chunk c - 1 -> operand buffer c & 1
                if (!(ok = wait_bar_warp(cx, bBupdDone, (c - 1) & 1, 202))) break;
#pragma unroll
                for (int dh = 0; dh < DH; ++dh) {
                    tc_fence_after();
                    tmem_ld64(lane_base + tmB + dh * 64, v);
                    tc_fence_before();
                    if (dh == DH - 1) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(cx.bar(bBaccFree + wg));   // update of chunk c may start
                    }
                    write_bt(wg, dh);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(cx.bar(bBtReady + wg));
            }
            // V tile of the group: last read by the G.V product of chunk c - 2
            if (c >= 2 && !(ok = wait_bar_warp(cx, bOReady + wg, ph ^ 1, 205))) break;
#pragma unroll
            for (int dh = 0; dh < DH; ++dh)
                copy_tile<D, false>(stage + Ly::kTileP + dh * 8192, cx.sm + Ly::oVt + wg * Ly::kTileV, dh * 64,
                                    wtid, nullptr);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(cx.bar(bVReady + wg)); mbar_arrive(cx.bar(bEmpty + wg)); }
        }
    } else if (warp == kProducerWarp) {
        // =========================== TMA producer ==============================================
        if (lane == 0) {
            int issued = 0, q_issued = 0;
            for (int c = 0; c < nch; ++c) {
                const int st = c & 1;
                if (c >= 2 && !wait_bar(cx, bEmpty + st, ((c >> 1) - 1) & 1, 301)) break;
                const uint32_t dst = cx.sm_u32 + Ly::oStage + st * Ly::kStage;
                const uint32_t bar = cx.bar(bFull + st);
                const int tok = (int)(t_begin + (int64_t)c * C);
                mbar_arrive_expect_tx(bar, Ly::kStage);
                tma_load_4d(dst, &map_k, bar, 0, tok, g, (int)n);
                tma_load_4d(dst + Ly::kTileP, &map_v, bar, 0, tok, 0, (int)n);   // one box: all D / 64 column blocks
                issued = c + 1;
                // pQ of the chunk into the slot of its worker group (c & 1), once the group has taken chunk c - 2
                if (c >= 2 && !wait_bar(cx, bPqEmpty + st, ((c >> 1) - 1) & 1, 302)) break;
                mbar_arrive_expect_tx(cx.bar(bPqFull + st), Ly::kTileP);
                tma_load_4d(cx.sm_u32 + Ly::oPq + st * Ly::kTileP, &map_q, cx.bar(bPqFull + st), 0, tok, g, (int)n);
                q_issued = c + 1;
            }
            if (*cx.abort_flag) {
                for (int c = max(0, issued - 2); c < issued; ++c) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(bFull + (c & 1)), (c >> 1) & 1) && clock64() - t0 < (1ll << 24)) {}
                }
                for (int c = max(0, q_issued - 2); c < q_issued; ++c) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(bPqFull + (c & 1)), (c >> 1) & 1) && clock64() - t0 < (1ll << 24)) {}
                }
            }
        }
    } else {
        // =========================== MMA issuers (one warp per worker group) ====================
        const int wg = __shfl_sync(0xffffffffu, warp, 0) - kMmaWarp;
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
        const uint32_t smb = __shfl_sync(0xffffffffu, cx.sm_u32, 0);
        const uint32_t tril_lo = lo_k(smb + Ly::oTril);
        const uint32_t kt_k = lo_k(smb + Ly::oKt + wg * Ly::kTileP);
        const uint32_t kt_mn = lo_mn(smb + Ly::oKt + wg * Ly::kTileP);
        const uint32_t vt_mn = lo_mn_w(smb + Ly::oVt + wg * Ly::kTileV, Ly::kLboV);
        const uint32_t wt_k = lo_k(smb + Ly::oWt + wg * Ly::kTileP);
        const uint32_t bt_mn = lo_mn_w(smb + Ly::oBt + wg * Ly::kTileV, Ly::kLboV);
        const uint32_t dB = tm, dAG = tm + D + wg * (64 + D), dO = dAG + 64;
        constexpr uint32_t kI64 = idesc_n(64), kID = idesc_n(D);
        if (elect_one()) {
            uint32_t ph = 0;
            bool ok = true;
            for (int c = wg; c < nch && ok; c += 2, ph ^= 1) {
                if (!(ok = wait_bar(cx, bKReady + wg, ph, 401))) break;
                tc_fence_after();
                // A_loc = tril . pK
                if constexpr (D == 64) mma_k64_ta<true, kHiMN, 128>(dAG, tm + 384, kt_mn, kI64 | kBmn);
                else mma_k64<true, kHiK, 16, kHiMN, 128>(dAG, tril_lo, kt_mn, kI64 | kBmn);
                mma_commit(cx.bar(bXReady + wg));
                // B += pK^T . V (N = D)
                if (!(ok = wait_bar(cx, bVReady + wg, ph, 407))) break;
                if (!(ok = wait_bar(cx, bBaccFree + wg, ph, 403))) break;
                tc_fence_after();
                mma_k64<false, kHiMN, 128, kHiMN, Ly::kStepV>(dB, kt_mn, vt_mn, kID | kAmn | kBmn);
                mma_commit(cx.bar(bBupdDone));
                // O = W . B (N = D) and G = W . pK^T
                if (!(ok = wait_bar(cx, bWReady + wg, ph, 404))) break;
                if (!(ok = wait_bar(cx, bBtReady + wg, ph, 405))) break;
                tc_fence_after();
                if constexpr (D == 64) {
                    mma_k64_ta<true, kHiK, 16>(dAG, tm + 320 + wg * 32, kt_k, kI64);
                    mma_k64_ta<true, kHiMN, Ly::kStepV>(dO, tm + 320 + wg * 32, bt_mn, kID | kBmn);
                } else {
                    mma_k64<true, kHiK, 16, kHiK, 16>(dAG, wt_k, kt_k, kI64);
                    mma_k64<true, kHiK, 16, kHiMN, Ly::kStepV>(dO, wt_k, bt_mn, kID | kBmn);
                }
                mma_commit(cx.bar(bGReady + wg));
                // O += G . V
                if (!(ok = wait_bar(cx, bGtReady + wg, ph, 406))) break;
                tc_fence_after();
                if constexpr (D == 64) mma_k64_ta<false, kHiMN, Ly::kStepV>(dO, tm + 320 + wg * 32, vt_mn, kID | kBmn);
                else mma_k64<false, kHiK, 16, kHiMN, Ly::kStepV>(dO, wt_k, vt_mn, kID | kBmn);
                mma_commit(cx.bar(bOReady + wg));
            }
            mma_commit(cx.bar(bDrain + wg));
            const long long t0 = clock64();
            while (!mbar_try_wait(cx.bar(bDrain + wg), 0) && clock64() - t0 < cx.limit) {}
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// tile totals
// ------------------------------------------------------------------------------------------------
constexpr int kT1Threads = 10 * 32;
constexpr int kT1Stages = 4;
// GP bucket groups per CTA: they share the V tile of a chunk, which the CTAs of a (stream, tile) otherwise fetch once
// per group (with GP = 1 and eight groups the kernel moved 3 KB per token-stream from L2 for 1.25 KB of inputs and
// was bound by that)
template <int D, int GP>
struct Lay1 {
    static constexpr int kTileP = C * 64 * 2, kTileV = C * D * 2, kStage = GP * kTileP + kTileV;
    static constexpr int oStage = 0;
    static constexpr int oKt = oStage + kT1Stages * kStage;   // [2][GP]
    static constexpr int oVt = oKt + 2 * GP * kTileP;         // [2]
    static constexpr int oRed = oVt + 2 * kTileV;             // [GP][8 warps][4][8] fp32
    static constexpr int oBars = oRed + GP * 8 * 32 * 4;
    static constexpr int oMisc = oBars + 16 * 8;
    static constexpr int kSmem = oMisc + 16 + 1024;
};
enum Bar1B { b1Full = 0, b1Empty = 4, b1KvReady = 8, b1KvFree = 10, b1Done = 12 };

// heads > 1: V is laid out [N / heads][T][heads][D] and map_v is the 5-D map of that layout
template <int D, int GP>
__global__ void __launch_bounds__(kT1Threads, 1)
tile_totals_tc_bf16(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    float* __restrict__ ws, int64_t T, int S, int G, int tile_tokens, int heads, int* status) {
    using Ly = Lay1<D, GP>;
    constexpr int DH = D / 64;
    static_assert(GP * D <= 512, "one accumulator per group");
    extern __shared__ uint8_t smem_raw[];
    Ctx cx;
    cx.sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    cx.sm_u32 = smem_u32(cx.sm);
    cx.bars = Ly::oBars;
    cx.abort_flag = reinterpret_cast<volatile int*>(cx.sm + Ly::oMisc + 4);
    cx.status = status;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(cx.sm + Ly::oMisc);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int GC = G / GP;                                   // CTAs per (stream, tile)
    const int g = (int)(blockIdx.x % (unsigned)GC) * GP;     // first bucket group of this CTA
    const int64_t tiles = gridDim.x / GC, tile = blockIdx.x / GC, n = blockIdx.y;
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(T, t_begin + (int64_t)tile_tokens);
    const int nch = (int)((t_end - t_begin + C - 1) / C);
    float* slice = ws + (n * tiles + tile) * (int64_t)(S * (D + 1));
    float* sliceB = slice + (int64_t)g * SG * D;            // group g + gp: + gp * SG * D
    float* sliceA = slice + (int64_t)S * D + g * SG;        //               + gp * SG

    if (tid == 0) {
        *cx.abort_flag = 0;
        for (int i = 0; i < kT1Stages; ++i) {
            mbar_init(cx.bar(b1Full + i), 1);
            mbar_init(cx.bar(b1Empty + i), 4);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(cx.bar(b1KvReady + i), 4);
            mbar_init(cx.bar(b1KvFree + i), 1);
        }
        mbar_init(cx.bar(b1Done), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(cx.sm_u32 + Ly::oMisc), "r"((uint32_t)(GP * D)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp < 8) {
        const int wg = warp >> 2, wtid = tid & 127;
        float asum[GP][4][8];
#pragma unroll
        for (int gp = 0; gp < GP; ++gp)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) asum[gp][i][e] = 0.f;
        bool ok = true;
        for (int c = wg; c < nch && ok; c += 2) {
            const int st = c % kT1Stages;
            if (!(ok = wait_bar_warp(cx, b1Full + st, (c / kT1Stages) & 1, 111))) break;
            if (c >= 2 && !(ok = wait_bar_warp(cx, b1KvFree + wg, ((c >> 1) - 1) & 1, 112))) break;
            const uint8_t* stage = cx.sm + Ly::oStage + st * Ly::kStage;
#pragma unroll
            for (int gp = 0; gp < GP; ++gp)
                copy_tile<64, true>(stage + gp * Ly::kTileP, cx.sm + Ly::oKt + (wg * GP + gp) * Ly::kTileP, 0, wtid,
                                    asum[gp]);
#pragma unroll
            for (int dh = 0; dh < DH; ++dh)
                copy_tile<D, false>(stage + GP * Ly::kTileP + dh * 8192, cx.sm + Ly::oVt + wg * Ly::kTileV, dh * 64,
                                    wtid, nullptr);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(cx.bar(b1KvReady + wg)); mbar_arrive(cx.bar(b1Empty + st)); }
        }
        // column sums: item it of a thread covers columns 8 j .. 8 j + 7 with j = 2 it + (wtid >> 6),
        // lanes of a warp hold different token rows of the same columns
#pragma unroll
        for (int gp = 0; gp < GP; ++gp) {
            float* red = reinterpret_cast<float*>(cx.sm + Ly::oRed) + (gp * 8 + warp) * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float x = asum[gp][i][e];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
                    if (lane == 0) red[i * 8 + e] = x;
                }
        }
    } else if (warp == 8) {
        if (lane == 0) {
            int issued = 0;
            for (int c = 0; c < nch; ++c) {
                const int st = c % kT1Stages;
                if (c >= kT1Stages && !wait_bar(cx, b1Empty + st, ((c / kT1Stages) - 1) & 1, 311)) break;
                const uint32_t dst = cx.sm_u32 + Ly::oStage + st * Ly::kStage;
                const uint32_t bar = cx.bar(b1Full + st);
                const int tok = (int)(t_begin + (int64_t)c * C);
                mbar_arrive_expect_tx(bar, Ly::kStage);
                tma_load_4d(dst, &map_k, bar, 0, tok, g, (int)n);                    // one box: GP column blocks
                // one box: all D / 64 blocks
                if (heads > 1) tma_load_5d(dst + GP * Ly::kTileP, &map_v, bar, 0, tok, 0, (int)(n % heads), (int)(n / heads));
                else tma_load_4d(dst + GP * Ly::kTileP, &map_v, bar, 0, tok, 0, (int)n);
                issued = c + 1;
            }
            if (*cx.abort_flag) {
                for (int c = max(0, issued - kT1Stages); c < issued; ++c) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(b1Full + c % kT1Stages), (c / kT1Stages) & 1) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
            }
        }
    } else {
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
        const uint32_t smb = __shfl_sync(0xffffffffu, cx.sm_u32, 0);
        if (elect_one()) {
            bool ok = true;
            for (int c = 0; c < nch && ok; ++c) {
                const int wg = c & 1;
                if (!(ok = wait_bar(cx, b1KvReady + wg, (c >> 1) & 1, 411))) break;
                tc_fence_after();
                const uint32_t vt_mn = lo_mn_w(smb + Ly::oVt + wg * Ly::kTileV, Lay<D>::kLboV);
#pragma unroll
                for (int gp = 0; gp < GP; ++gp) {
                    const uint32_t kt_mn = lo_mn(smb + Ly::oKt + (wg * GP + gp) * Ly::kTileP);
                    if (c == 0) mma_k64<true, kHiMN, 128, kHiMN, Lay<D>::kStepV>(tm + gp * D, kt_mn, vt_mn, idesc_n(D) | kAmn | kBmn);
                    else mma_k64<false, kHiMN, 128, kHiMN, Lay<D>::kStepV>(tm + gp * D, kt_mn, vt_mn, idesc_n(D) | kAmn | kBmn);
                }
                mma_commit(cx.bar(b1KvFree + wg));
            }
            mma_commit(cx.bar(b1Done));
        }
    }
    __syncthreads();   // column-sum partials are in shared memory
    if (warp < 4) {
        if (wait_bar_warp(cx, b1Done, 0, 113)) {
            float v[32];
            const int q = lane & 3, rbase = 16 * warp + (lane >> 2);
#pragma unroll
            for (int gp = 0; gp < GP; ++gp)
#pragma unroll
                for (int dh = 0; dh < DH; ++dh) {
                    tc_fence_after();
                    tmem_ld64(((uint32_t)(32 * warp) << 16) + tmem + gp * D + dh * 64, v);
                    tc_fence_before();
#pragma unroll
                    for (int x = 0; x < 8; ++x)
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            *reinterpret_cast<float2*>(sliceB + ((int64_t)gp * SG + rbase + 8 * h) * D + dh * 64 +
                                                       8 * x + 2 * q) = make_float2(v[4 * x + 2 * h], v[4 * x + 2 * h + 1]);
                }
            if (tid < 64) {
                // column s = 8 j + e, j = 2 item + (warp-in-group >> 1): partials of both converter groups and
                // both row halves in a fixed order
                const int j = tid >> 3, e = tid & 7, it = j >> 1, wh = (j & 1) * 2;
#pragma unroll
                for (int gp = 0; gp < GP; ++gp) {
                    const float* red = reinterpret_cast<const float*>(cx.sm + Ly::oRed) + gp * 8 * 32;
                    float a = 0.f;
#pragma unroll
                    for (int gg = 0; gg < 2; ++gg)
#pragma unroll
                        for (int half = 0; half < 2; ++half) a += red[(gg * 4 + wh + half) * 32 + it * 8 + e];
                    sliceA[gp * SG + tid] = a;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(GP * D)) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// Output pass for S > 64 ("wide"): one CTA owns a (stream, tile, 32-column slice of the head
// dimension) and ALL bucket groups.  Per 64-token chunk it walks the groups one after the other
// ("items"); because out = sum_g [ W_g B_g + tril(W_g pK_g^T) V ] = (sum_g W_g B_g) +
// tril(sum_g W_g pK_g^T) V, the W.B products of all groups accumulate in one TMEM accumulator
// and the W.pK^T products in another, so the causal mask and the G.V product run once per chunk
// and nothing is exchanged between CTAs.  The price: the CTAs of the d_k/32 slices each recompute
// W and G.  TMEM (512 columns): the state B_g of the G <= 8 groups ([64 x 32] each: 256), A_loc /
// W per worker group (2 x 64), G (64; its first 32 columns take the masked operand afterwards) and
// O for even / odd chunks (2 x 32).
// Roles (18 warps): 2 worker warpgroups on alternate items (W of the item -> tensor memory as the
// MMA A operand; the running A of every group stays in shared memory with the group's owner),
// 1 converter warpgroup (TMA-staged pK item tiles and the V slice -> operand layout), 1 auxiliary
// warpgroup (state of a group after its update -> bf16 operand tile; mask of G; output store),
// 1 TMA producer warp, 1 MMA-issuing warp that runs the running-sum product one item ahead.
// ------------------------------------------------------------------------------------------------
constexpr int kWThreads = 18 * 32;
constexpr int kWProducerWarp = 16, kWMmaWarp = 17;
constexpr int kWStages = 4;       // ring of pK item tiles (stage and operand buffers)
constexpr int DS = 32;            // head-dim slice of a CTA
struct LayW {
    static constexpr int kTileP = C * 64 * 2;    // 64 x 64 bf16
    static constexpr int kTileS = C * DS * 2;    // 64 x 32 bf16
    static constexpr int oPq = 0;                             // [2 wg][kTileP] pQ of a worker group's next item (swizzled)
    static constexpr int oStage = oPq + 2 * kTileP;           // [kWStages][kTileP] staged pK
    static constexpr int oVst = oStage + kWStages * kTileP;   // [2][kTileS] staged V slice
    static constexpr int oKt = oVst + 2 * kTileS;             // [kWStages][kTileP]
    static constexpr int oVt = oKt + kWStages * kTileP;       // [2][kTileS]
    static constexpr int oBt = oVt + 2 * kTileS;              // [8][kTileS]
    static constexpr int oTril = oBt + 8 * kTileS;
    static constexpr int oAcar = oTril + kTileP;              // [8][64] fp32
    static constexpr int oBars = oAcar + 8 * 64 * 4;
    static constexpr int kNumBars = 66;
    static constexpr int oMisc = oBars + kNumBars * 8;
    static constexpr int kSmem = oMisc + 16 + 1024;
    static constexpr uint32_t kLboS = (DS / 8) * 128;         // MN-major [64][32] tile: K-direction stride
    static constexpr uint32_t kStepS = (2 * kLboS) >> 4;
};
enum BarW {
    wFull = 0, wEmpty = 4, wVFull = 8, wVEmpty = 10, wKReady = 12, wKFree = 16, wVReady = 20, wVFree = 22,
    wXReady = 24, wWReady = 26, wItemDone = 28, wBtReady = 44, wGtReady = 52, wOReady = 53,
    wOFree = 54, wDrain = 56,
    wAcarReady = 57,   // [2] the group's running A written by the warp that owns row 63
    wAcarRead = 59,    // [2] ... read by the four warps of the worker group
    wPqFull = 61,      // [2] pQ tile of the worker group's next item has landed
    wPqEmpty = 63      // [2] ... copied to registers by the four warps
};

__global__ void __launch_bounds__(kWThreads, 1)
causal_out_wide_bf16(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_vs, __nv_bfloat16* __restrict__ out,
                     const float* __restrict__ ws, int64_t T, int S, int D, int G, int tile_tokens, float eps,
                     int* status) {
    using Ly = LayW;
    extern __shared__ uint8_t smem_raw[];
    Ctx cx;
    cx.sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    cx.sm_u32 = smem_u32(cx.sm);
    cx.bars = Ly::oBars;
    cx.abort_flag = reinterpret_cast<volatile int*>(cx.sm + Ly::oMisc + 4);
    cx.status = status;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(cx.sm + Ly::oMisc);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NS = D / DS;                                   // slices of the head dimension
    const int js = (int)(blockIdx.x % (unsigned)NS);
    const int64_t tiles = gridDim.x / NS;
    const int64_t tile = blockIdx.x / NS, n = blockIdx.y;
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(T, t_begin + (int64_t)tile_tokens);
    const int nch = (int)((t_end - t_begin + C - 1) / C);
    const int nitems = nch * G;
    const float* slice = ws + (n * tiles + tile) * (int64_t)(S * (D + 1));

    if (tid == 0) {
        *cx.abort_flag = 0;
        for (int i = 0; i < kWStages; ++i) {
            mbar_init(cx.bar(wFull + i), 1);
            mbar_init(cx.bar(wEmpty + i), 4);
            mbar_init(cx.bar(wKReady + i), 4);
            mbar_init(cx.bar(wKFree + i), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(cx.bar(wVFull + i), 1);
            mbar_init(cx.bar(wVEmpty + i), 4);
            mbar_init(cx.bar(wVReady + i), 4);
            mbar_init(cx.bar(wVFree + i), 1);
            mbar_init(cx.bar(wXReady + i), 1);
            mbar_init(cx.bar(wWReady + i), 4);
            mbar_init(cx.bar(wOFree + i), 4);
            mbar_init(cx.bar(wAcarReady + i), 1);
            mbar_init(cx.bar(wAcarRead + i), 4);
            mbar_init(cx.bar(wPqFull + i), 1);
            mbar_init(cx.bar(wPqEmpty + i), 4);
        }
        for (int i = 0; i < 8; ++i) {
            mbar_init(cx.bar(wItemDone + i), 1);
            mbar_init(cx.bar(wBtReady + i), 4);
        }
        mbar_init(cx.bar(wGtReady), 4);
        mbar_init(cx.bar(wOReady), 1);
        mbar_init(cx.bar(wDrain), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kWMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(cx.sm_u32 + Ly::oMisc), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < C * 8; i += kWThreads) {   // tril[t][j] = (j <= t)
        const int t = i >> 3, jg = i & 7;
        uint32_t w[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int j0 = jg * 8 + 2 * p;
            w[p] = (j0 <= t ? 0x3F80u : 0u) | (j0 + 1 <= t ? 0x3F800000u : 0u);
        }
        *reinterpret_cast<uint4*>(cx.sm + Ly::oTril + off_w<64>(t, jg * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (int i = tid; i < G * 64; i += kWThreads)   // running A of every group: the carry-in
        reinterpret_cast<float*>(cx.sm + Ly::oAcar)[i] = slice[(int64_t)S * D + i];
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    auto tmBg = [&](int g) { return tmem + g * DS; };                 // [0, 256)
    auto tmX = [&](int wg) { return tmem + 256 + wg * 64; };          // A_loc, then W (32 columns of pairs)
    const uint32_t tmG = tmem + 384;                                  // G, then masked G (32 columns of pairs)
    auto tmO = [&](int c) { return tmem + 448 + (c & 1) * DS; };

    if (warp < 8) {
        // =========================== worker warpgroups: W of every other item ====================
        const int wg = warp >> 2, w = warp & 3;
        const int q = lane & 3, rbase = 16 * w + (lane >> 2);
        const uint32_t lane_base = (uint32_t)(32 * w) << 16;
        float v[32];
        bool ok = true;
        // pQ of the group's next item: a TMA-staged [64 tokens][64 buckets] tile (128-byte rows, 128B swizzle; rows past
        // the end of the sequence are zero) read in the accumulator-fragment layout (pairs of bf16), one item of this
        // worker group ahead; the eight rows a warp instruction reads fall on different banks
        const uint8_t* pq_tile = cx.sm + Ly::oPq + wg * Ly::kTileP;
        auto take_pq = [&](int k, uint32_t (&f)[16]) -> bool {
            if (!wait_bar_warp(cx, wPqFull + wg, (uint32_t)(k & 1), 104)) return false;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rbase + 8 * h;
#pragma unroll
                for (int x = 0; x < 8; ++x)
                    f[2 * x + h] = *reinterpret_cast<const uint32_t*>(pq_tile + row * 128 + ((x ^ (row & 7)) << 4) + 4 * q);
            }
            // generic-proxy reads before the async-proxy write of the next tile: proxy fence, then the slot goes back
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(wPqEmpty + wg));
            return true;
        };
        uint32_t pq_next[16];
        if (wg < nitems) ok = take_pq(0, pq_next);
        for (int i = wg, k = 0; i < nitems && ok; i += 2, ++k) {
            const int c = i / G, g = i - c * G;
            uint32_t pqv[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) pqv[j] = pq_next[j];
            // running A of the group: written at the end of the previous item of this worker group
            // (which is the same bucket group when G = 2)
            if (!(ok = wait_bar_warp(cx, wAcarReady + wg, (uint32_t)((k & 1) ^ 1), 101))) break;
            float* ac = reinterpret_cast<float*>(cx.sm + Ly::oAcar) + g * 64;
            float acar[16];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const float2 a2 = *reinterpret_cast<const float2*>(ac + 8 * x + 2 * q);
                acar[2 * x] = a2.x; acar[2 * x + 1] = a2.y;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(wAcarRead + wg));
            // the warp that owns row 63 overwrites the values below: all four warps must hold them first
            if (w == 3 && !(ok = wait_bar_warp(cx, wAcarRead + wg, (uint32_t)(k & 1), 102))) break;
            if (w == 0) RACE_TRACE(wg, i - 64, 0);
            if (!(ok = wait_bar_warp(cx, wXReady + wg, (uint32_t)(k & 1), 103))) break;
            if (w == 0) RACE_TRACE(wg, i - 64, 1);
            tc_fence_after();
            tmem_ld64(lane_base + tmX(wg), v);
            tc_fence_before();
            if (w == 0) RACE_TRACE(wg, i - 64, 2);
            uint32_t wv[16];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float2 pq2 = unpack_bf16(pqv[2 * x + h]);
                    const float a0 = acar[2 * x] + v[4 * x + 2 * h];
                    const float a1 = acar[2 * x + 1] + v[4 * x + 2 * h + 1];
                    wv[2 * x + h] = pack_bf16(__fdividef(pq2.x, a0 + eps), __fdividef(pq2.y, a1 + eps));
                    if (h == 1 && w == 3 && (lane >> 2) == 7)    // row 63: the running A after this chunk
                        *reinterpret_cast<float2*>(ac + 8 * x + 2 * q) = make_float2(a0, a1);
                }
            }
            tmem_st_pairs(lane_base + tmX(wg), wv);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(cx.bar(wWReady + wg));
                if (w == 3) mbar_arrive(cx.bar(wAcarReady + wg));   // the new running A is in place
            }
            if (w == 0) RACE_TRACE(wg, i - 64, 3);
            if (i + 2 < nitems && !(ok = take_pq(k + 1, pq_next))) break;
        }
    } else if (warp < 12) {
        // =========================== converter warpgroup ==========================================
        const int wtid = tid & 127;
        bool ok = true;
        for (int i = 0; i < nitems && ok; ++i) {
            const int c = i / G, g = i - c * G, st = i % kWStages;
            const uint32_t rp = (uint32_t)((i / kWStages) & 1);
            if (i >= kWStages && !(ok = wait_bar_warp(cx, wKFree + st, rp ^ 1, 203))) break;
            if (!(ok = wait_bar_warp(cx, wFull + st, rp, 201))) break;
            copy_tile<64, false>(cx.sm + Ly::oStage + st * Ly::kTileP, cx.sm + Ly::oKt + st * Ly::kTileP, 0, wtid, nullptr);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(cx.bar(wKReady + st)); mbar_arrive(cx.bar(wEmpty + st)); }
            if (g == 0) {
                // V slice of the chunk: [64 tokens][32 values], staged without swizzle
                const int vb = c & 1;
                const uint32_t vp = (uint32_t)((c >> 1) & 1);
                if (c >= 2 && !(ok = wait_bar_warp(cx, wVFree + vb, vp ^ 1, 205))) break;
                if (!(ok = wait_bar_warp(cx, wVFull + vb, vp, 206))) break;
                const uint8_t* src = cx.sm + Ly::oVst + vb * Ly::kTileS;
                uint8_t* dst = cx.sm + Ly::oVt + vb * Ly::kTileS;
#pragma unroll
                for (int it = 0; it < 2; ++it) {
                    const int idx = it * 128 + wtid;          // 256 items of 16 bytes
                    const int r = idx >> 2, j = idx & 3;
                    *reinterpret_cast<uint4*>(dst + off_w<DS>(r, 8 * j)) =
                        *reinterpret_cast<const uint4*>(src + r * 64 + j * 16);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) { mbar_arrive(cx.bar(wVReady + vb)); mbar_arrive(cx.bar(wVEmpty + vb)); }
            }
        }
    } else if (warp < 16) {
        // =========================== auxiliary warpgroup: state operands, mask, output ============
        const int w = warp & 3, q = lane & 3, rbase = 16 * w + (lane >> 2);
        const uint32_t lane_base = (uint32_t)(32 * w) << 16;
        float b[16];
        auto write_bt = [&](int g) {
            uint8_t* bt = cx.sm + Ly::oBt + g * Ly::kTileS;
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    *reinterpret_cast<uint32_t*>(bt + off_w<DS>(rbase + 8 * h, 8 * x + 2 * q)) =
                        pack_bf16(b[4 * x + 2 * h], b[4 * x + 2 * h + 1]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(wBtReady + g));
        };
        // carry-in of every group: accumulator and operand tile
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float2 b2 = *reinterpret_cast<const float2*>(
                        slice + (int64_t)(g * SG + rbase + 8 * h) * D + js * DS + 8 * x + 2 * q);
                    b[4 * x + 2 * h] = b2.x; b[4 * x + 2 * h + 1] = b2.y;
                }
            tmem_st32(lane_base + tmBg(g), b);
            tc_fence_before();
            write_bt(g);
        }
        bool ok = true;
        for (int c = 0; c < nch && ok; ++c) {
            const uint32_t cp = (uint32_t)(c & 1);
            const int64_t tok0 = t_begin + (int64_t)c * C;
            const int valid = (int)min((int64_t)C, t_end - tok0);
            auto carry = [&](int g) {   // state of group g after this chunk -> operand tile for the next chunk
                tc_fence_after();
                tmem_ld32(lane_base + tmBg(g), b);
                tc_fence_before();
                write_bt(g);   // its arrival also tells the issuer that the accumulator has been read
            };
            for (int g = 0; g < G - 1 && ok; ++g) {
                if (!(ok = wait_bar_warp(cx, wItemDone + g, cp, 501))) break;
                if (c + 1 < nch) carry(g);
            }
            if (!ok) break;
            // all groups have accumulated into G: causal mask -> bf16 pairs over G's first 32 columns
            if (!(ok = wait_bar_warp(cx, wItemDone + G - 1, cp, 502))) break;
            {
                float v[32];
                uint32_t gv[16];
                tc_fence_after();
                tmem_ld64(lane_base + tmG, v);
                tc_fence_before();
#pragma unroll
                for (int x = 0; x < 8; ++x)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int row = rbase + 8 * h, col = 8 * x + 2 * q;
                        gv[2 * x + h] = pack_bf16(col <= row ? v[4 * x + 2 * h] : 0.f,
                                                  col + 1 <= row ? v[4 * x + 2 * h + 1] : 0.f);
                    }
                tmem_st_pairs(lane_base + tmG, gv);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(cx.bar(wGtReady));
            }
            if (c + 1 < nch) carry(G - 1);
            // O of the chunk (this CTA's 32 columns)
            if (!(ok = wait_bar_warp(cx, wOReady, cp, 503))) break;
            tc_fence_after();
            tmem_ld32(lane_base + tmO(c), b);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(wOFree + (c & 1)));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rbase + 8 * h;
                if (row < valid) {
                    __nv_bfloat16* orow = out + (n * T + tok0 + row) * D + js * DS + 2 * q;
#pragma unroll
                    for (int x = 0; x < 4; ++x)
                        *reinterpret_cast<uint32_t*>(orow + 8 * x) = pack_bf16(b[4 * x + 2 * h], b[4 * x + 2 * h + 1]);
                }
            }
        }
    } else if (warp == kWProducerWarp) {
        // =========================== TMA producer ==================================================
        if (lane == 0) {
            int issued = 0, v_issued = 0, q_issued = 0;
            for (int i = 0; i < nitems; ++i) {
                const int c = i / G, g = i - c * G, st = i % kWStages;
                const int tok = (int)(t_begin + (int64_t)c * C);
                if (i >= kWStages && !wait_bar(cx, wEmpty + st, (uint32_t)(((i / kWStages) - 1) & 1), 301)) break;
                mbar_arrive_expect_tx(cx.bar(wFull + st), Ly::kTileP);
                tma_load_4d(cx.sm_u32 + Ly::oStage + st * Ly::kTileP, &map_k, cx.bar(wFull + st), 0, tok, g, (int)n);
                issued = i + 1;
                if (g == 0) {
                    const int vb = c & 1;
                    if (c >= 2 && !wait_bar(cx, wVEmpty + vb, (uint32_t)(((c >> 1) - 1) & 1), 302)) break;
                    mbar_arrive_expect_tx(cx.bar(wVFull + vb), Ly::kTileS);
                    tma_load_4d(cx.sm_u32 + Ly::oVst + vb * Ly::kTileS, &map_vs, cx.bar(wVFull + vb), 0, tok, js, (int)n);
                    v_issued = c + 1;
                }
                {   // pQ of the item into the slot of its worker group, once the group has taken the tile before it
                    const int qs = i & 1, qu = i >> 1;
                    if (qu >= 1 && !wait_bar(cx, wPqEmpty + qs, (uint32_t)((qu - 1) & 1), 303)) break;
                    mbar_arrive_expect_tx(cx.bar(wPqFull + qs), Ly::kTileP);
                    tma_load_4d(cx.sm_u32 + Ly::oPq + qs * Ly::kTileP, &map_q, cx.bar(wPqFull + qs), 0, tok, g, (int)n);
                    q_issued = i + 1;
                }
            }
            if (*cx.abort_flag) {   // copies in flight must land before the CTA may exit
                for (int i = max(0, q_issued - 2); i < q_issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(wPqFull + (i & 1)), (uint32_t)((i >> 1) & 1)) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
                for (int i = max(0, issued - kWStages); i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(wFull + i % kWStages), (uint32_t)((i / kWStages) & 1)) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
                for (int c = max(0, v_issued - 2); c < v_issued; ++c) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(wVFull + (c & 1)), (uint32_t)((c >> 1) & 1)) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
            }
        }
    } else {
        // =========================== MMA issuer ======================================================
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
        const uint32_t smb = __shfl_sync(0xffffffffu, cx.sm_u32, 0);
        const int Gu = __shfl_sync(0xffffffffu, G, 0);
        const uint32_t tril_lo = lo_k(smb + Ly::oTril);
        constexpr uint32_t kI64 = idesc_n(64), kIS = idesc_n(DS);
        if (elect_one()) {
            bool ok = true;
            auto cumsum = [&](int i) -> bool {   // A_loc of item i = tril . pK_g
                const int st = i % kWStages;
                if (!wait_bar(cx, wKReady + st, (uint32_t)((i / kWStages) & 1), 401)) return false;
                tc_fence_after();
                mma_k64<true, kHiK, 16, kHiMN, 128>(tm + 256 + (i & 1) * 64, tril_lo,
                                                    lo_mn(smb + Ly::oKt + st * Ly::kTileP), kI64 | kBmn);
                mma_commit(cx.bar(wXReady + (i & 1)));
                return true;
            };
            auto gv = [&](int c) -> bool {       // O += masked G . V, once per chunk
                if (!wait_bar(cx, wGtReady, (uint32_t)(c & 1), 406)) return false;
                tc_fence_after();
                mma_k64_ta<false, kHiMN, Ly::kStepS>(tm + 448 + (c & 1) * DS, tm + 384,
                                                     lo_mn_w(smb + Ly::oVt + (c & 1) * Ly::kTileS, Ly::kLboS), kIS | kBmn);
                mma_commit(cx.bar(wOReady));
                mma_commit(cx.bar(wVFree + (c & 1)));
                return true;
            };
            if (nitems > 0) ok = cumsum(0);
            for (int i = 0; i < nitems && ok; ++i) {
                const int c = i / Gu, g = i - c * Gu, st = i % kWStages, wg = i & 1;
                if (i + 1 < nitems && !(ok = cumsum(i + 1))) break;      // one item ahead
                if (g == 0 && c >= 1 && !(ok = gv(c - 1))) break;        // frees G for this chunk
                // W of the item in tensor memory; state operand of the group written (which also means that
                // the group's accumulator has been read out after the previous chunk)
                if (!(ok = wait_bar2(cx, wWReady + wg, (uint32_t)((i >> 1) & 1), wBtReady + g, (uint32_t)(c & 1), 404))) break;
                if (g == 0) {
                    if (c >= 2 && !(ok = wait_bar(cx, wOFree + (c & 1), (uint32_t)(((c >> 1) - 1) & 1), 408))) break;
                    if (!(ok = wait_bar(cx, wVReady + (c & 1), (uint32_t)((c >> 1) & 1), 407))) break;
                }
                tc_fence_after();
                const uint32_t a_w = tm + 256 + wg * 64;
                const uint32_t kt = smb + Ly::oKt + st * Ly::kTileP;
                const uint32_t bt_mn = lo_mn_w(smb + Ly::oBt + g * Ly::kTileS, Ly::kLboS);
                const uint32_t vt_mn = lo_mn_w(smb + Ly::oVt + (c & 1) * Ly::kTileS, Ly::kLboS);
                const uint32_t dO = tm + 448 + (c & 1) * DS;
                if (g == 0) {
                    mma_k64_ta<true, kHiK, 16>(tm + 384, a_w, lo_k(kt), kI64);                 // G  = W . pK^T
                    mma_k64_ta<true, kHiMN, Ly::kStepS>(dO, a_w, bt_mn, kIS | kBmn);           // O  = W . B_g
                } else {
                    mma_k64_ta<false, kHiK, 16>(tm + 384, a_w, lo_k(kt), kI64);                // G += ...
                    mma_k64_ta<false, kHiMN, Ly::kStepS>(dO, a_w, bt_mn, kIS | kBmn);          // O += ...
                }
                mma_k64<false, kHiMN, 128, kHiMN, Ly::kStepS>(tm + g * DS, lo_mn(kt), vt_mn, kIS | kAmn | kBmn);   // B_g += pK^T . V
                mma_commit(cx.bar(wItemDone + g));
                mma_commit(cx.bar(wKFree + st));
            }
            if (ok && nch > 0) ok = gv(nch - 1);
            mma_commit(cx.bar(wDrain));
            const long long t0 = clock64();
            while (!mbar_try_wait(cx.bar(wDrain), 0) && clock64() - t0 < cx.limit) {}
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kWMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// Output pass for S > 64 with an even number (>= 4) of bucket groups.  Same decomposition as causal_out_wide_bf16
// (one CTA = stream, tile, DSX-column slice of the head dimension, all groups; items = (chunk, group) in order),
// with the states of two adjacent groups stacked in one M = 128 accumulator (128 buckets x DSX columns on all 128
// lanes of tensor memory); the state update then runs once per pair of groups (M = 128) on a pK tile that is 128
// buckets wide, and the auxiliary group reads a pair's state with the 32-lane TMEM load.  NWG worker groups take
// every NWG-th item, each with its own A_loc / W buffer.
// What runs is DSX = 64, NWG = 2 (TMEM, 512 columns: pair states 4 x 64 | A_loc / W 2 x 64 | G 64 | O 64): the CTAs of
// the d_k / DSX slices each form W and G for themselves, so slices twice as wide halve that repeated work, which
// outweighs having two instead of four W stages in flight (DSX = 32, NWG = 4: pair states 4 x 32 | A_loc / W 4 x 64
// | G 64 | O 2 x 32).  pQ reaches the worker warps through shared memory: one TMA tile per item (full 128-byte
// rows), read in the accumulator-fragment layout with 4-byte loads that the 128B swizzle spreads over all banks;
// the same 4-byte loads straight from global memory touched eight rows per instruction and bound the pass.
// ------------------------------------------------------------------------------------------------
constexpr int kW4MaxStages = 4;
// DSX: columns of the head dimension a CTA owns; NWG: worker groups (A_loc / W buffers in flight); NST: ring of pK
// pair tiles (stage and operand buffers)
template <int DSX, int NWG, int NST>
struct LayW4 {
    static constexpr int kWarps = 4 * NWG + 10;
    static constexpr int kThreads = kWarps * 32;
    static constexpr int kConverterWarp0 = 4 * NWG, kAuxWarp0 = kConverterWarp0 + 4, kProducerWarp = kAuxWarp0 + 4,
                         kMmaWarp = kProducerWarp + 1;
    static constexpr int kOBufs = DSX == 32 ? 2 : 1;
    // tensor memory columns: pair states | A_loc / W per worker group | G | O
    static constexpr int kTmX = 4 * DSX, kTmG = kTmX + NWG * 64, kTmO = kTmG + 64;
    static_assert(kTmO + kOBufs * DSX <= 512, "tensor memory columns");
    static_assert(NST <= kW4MaxStages && NWG <= 4, "barrier array");
    static constexpr int kTileP = C * 64 * 2;     // 64 x 64 bf16
    static constexpr int kTileP2 = 2 * kTileP;    // the pK tiles of two adjacent groups: [64 tokens][128 buckets]
    static constexpr int kTileS = C * DSX * 2;    // 64 x DSX bf16
    static constexpr int oPq = 0;                         // [NWG][kTileP] pQ of a worker group's next item (swizzled)
    static constexpr int oStage = oPq + NWG * kTileP;     // [NST][kTileP2] staged: two boxes of 64 x 64
    static constexpr int oVst = oStage + NST * kTileP2;   // [2][kTileS] staged V slice
    static constexpr int oKt = oVst + 2 * kTileS;         // [NST][kTileP2] operand tile, 128 wide
    static constexpr int oVt = oKt + NST * kTileP2;       // [2][kTileS]
    static constexpr int oBt = oVt + 2 * kTileS;          // [4 pairs][128 x DSX] state operand tiles
    static constexpr int oTril = oBt + 8 * kTileS;
    static constexpr int oAcar = oTril + kTileP;                // [8][64] fp32
    static constexpr int oBars = oAcar + 8 * 64 * 4;
    static constexpr int kNumBars = 64;
    static constexpr int oMisc = oBars + kNumBars * 8;
    static constexpr int kSmem = oMisc + 16 + 1024;
    static constexpr uint32_t kLboS = (DSX / 8) * 128;          // MN-major [.][DSX] tile: stride between 8-row groups
    static constexpr uint32_t kStepS = (2 * kLboS) >> 4;
    static constexpr uint32_t kLboP2 = (128 / 8) * 128;         // MN-major [64][128] tile: stride between 8-token groups
    static constexpr uint32_t kStepP2 = (2 * kLboP2) >> 4;
    static constexpr uint32_t kHiK2 = (kLboP2 >> 4) | (1u << 14);    // K-major use of the 128-wide tile: sbo = 2048
};
static_assert(LayW4<64, 2, 3>::kSmem <= 227 * 1024, "shared memory of the wide kernel");
enum BarW4 {
    w4Full = 0, w4Empty = w4Full + kW4MaxStages, w4KReady = w4Empty + kW4MaxStages, w4KFree = w4KReady + kW4MaxStages,
    w4VFull = w4KFree + kW4MaxStages, w4VEmpty = w4VFull + 2, w4VReady = w4VEmpty + 2, w4VFree = w4VReady + 2,
    w4XReady = w4VFree + 2,          // [4] A_loc of the worker group's item complete
    w4WReady = w4XReady + 4,         // [4] W of the item in tensor memory (four warps)
    w4AcarReady = w4WReady + 4,      // [4] the item's running A written by the warp that owns row 63
    w4AcarRead = w4AcarReady + 4,    // [4] ... read by the four warps of the worker group
    w4PairDone = w4AcarRead + 4,     // [4] every product of a pair of groups of the chunk has run
    w4BtReady = w4PairDone + 4,      // [4] state operand tile of the pair written (four warps)
    w4GtReady = w4BtReady + 4, w4OReady = w4GtReady + 1, w4OFree = w4OReady + 1, w4Drain = w4OFree + 2,
    w4PqFull = w4Drain + 1,          // [4] pQ tile of the worker group's next item has landed
    w4PqEmpty = w4PqFull + 4,        // [4] ... copied to registers by the four warps
    w4NumBars = w4PqEmpty + 4
};
static_assert(w4NumBars <= LayW4<64, 2, 3>::kNumBars, "barrier array of the wide kernel");

__device__ __forceinline__ constexpr uint32_t idesc_mn(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// 32 lanes x 32 columns of fp32: thread t of the warp <-> lane (lane of taddr) + t, register j <-> column + j
__device__ __forceinline__ void tmem_ld_rows32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st_rows32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
        ::"r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31])),
          "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 16 lanes x 16 columns of packed bf16 pairs (half of tmem_st_pairs: 32 K-values per row).  No wait inside.
__device__ __forceinline__ void tmem_st_pairs4(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x128b.x4.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(taddr) : "memory");
}

template <int DSX, int NWG, int NST>
__global__ void __launch_bounds__((LayW4<DSX, NWG, NST>::kThreads), 1)
causal_out_wide4_bf16(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_vs, __nv_bfloat16* __restrict__ out,
                      const float* __restrict__ ws, int64_t T, int S, int D, int G, int tile_tokens, float eps,
                      int heads, int* status) {
    using Ly = LayW4<DSX, NWG, NST>;
    extern __shared__ uint8_t smem_raw[];
    Ctx cx;
    cx.sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    cx.sm_u32 = smem_u32(cx.sm);
    cx.bars = Ly::oBars;
    cx.abort_flag = reinterpret_cast<volatile int*>(cx.sm + Ly::oMisc + 4);
    cx.status = status;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(cx.sm + Ly::oMisc);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NS = D / DSX;                                  // slices of the head dimension
    const int P = G / 2;                                     // pairs of bucket groups
    const int js = (int)(blockIdx.x % (unsigned)NS);
    const int64_t tiles = gridDim.x / NS;
    const int64_t tile = blockIdx.x / NS, n = blockIdx.y;
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(T, t_begin + (int64_t)tile_tokens);
    const int nch = (int)((t_end - t_begin + C - 1) / C);
    const int nitems = nch * G;                              // an item = (chunk, group); a pair item = two of them
    const int npairs = nch * P;
    const float* slice = ws + (n * tiles + tile) * (int64_t)(S * (D + 1));

    if (tid == 0) {
        *cx.abort_flag = 0;
        for (int i = 0; i < NST; ++i) {
            mbar_init(cx.bar(w4Full + i), 1);
            mbar_init(cx.bar(w4Empty + i), 4);
            mbar_init(cx.bar(w4KReady + i), 4);
            mbar_init(cx.bar(w4KFree + i), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(cx.bar(w4VFull + i), 1);
            mbar_init(cx.bar(w4VEmpty + i), 4);
            mbar_init(cx.bar(w4VReady + i), 4);
            mbar_init(cx.bar(w4VFree + i), 1);
            mbar_init(cx.bar(w4OFree + i), 4);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(cx.bar(w4XReady + i), 1);
            mbar_init(cx.bar(w4WReady + i), 4);
            mbar_init(cx.bar(w4AcarReady + i), 1);
            mbar_init(cx.bar(w4AcarRead + i), 4);
            mbar_init(cx.bar(w4PairDone + i), 1);
            mbar_init(cx.bar(w4BtReady + i), 4);
            mbar_init(cx.bar(w4PqFull + i), 1);
            mbar_init(cx.bar(w4PqEmpty + i), 4);
        }
        mbar_init(cx.bar(w4GtReady), 4);
        mbar_init(cx.bar(w4OReady), 1);
        mbar_init(cx.bar(w4Drain), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == Ly::kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(cx.sm_u32 + Ly::oMisc), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < C * 8; i += Ly::kThreads) {   // tril[t][j] = (j <= t)
        const int t = i >> 3, jg = i & 7;
        uint32_t w[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int j0 = jg * 8 + 2 * p;
            w[p] = (j0 <= t ? 0x3F80u : 0u) | (j0 + 1 <= t ? 0x3F800000u : 0u);
        }
        *reinterpret_cast<uint4*>(cx.sm + Ly::oTril + off_w<64>(t, jg * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (int i = tid; i < G * 64; i += Ly::kThreads)   // running A of every group: the carry-in
        reinterpret_cast<float*>(cx.sm + Ly::oAcar)[i] = slice[(int64_t)S * D + i];
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    auto tmBp = [&](int p) { return tmem + p * DSX; };                // pair states, all 128 lanes
    auto tmX = [&](int wg) { return tmem + Ly::kTmX + wg * 64; };          // A_loc of the group's item, then W (32 columns)
    const uint32_t tmG = tmem + Ly::kTmG;                                 // G, then masked G (32 columns of pairs)
    auto tmO = [&](int c) { return tmem + Ly::kTmO + (c % Ly::kOBufs) * DSX; };

    if (warp < 4 * NWG) {
        // =========================== NWG worker groups: W of every NWG-th item ======================
        // G = 4 or 8 is a multiple of NWG: item i belongs to worker group i % NWG, so a bucket group always stays
        // with one worker group (its running A has one owner).
        const int wg = warp >> 2, w = warp & 3;
        const int q = lane & 3, rbase = 16 * w + (lane >> 2);
        const uint32_t lane_base = (uint32_t)(32 * w) << 16;
        bool ok = true;
        // pQ of the group's next item: a TMA-staged [64 tokens][64 buckets] tile (128-byte rows, 128B swizzle; rows past
        // the end of the sequence are zero) read in the accumulator-fragment layout (pairs of bf16), one item of this
        // worker group ahead.  Lanes of a warp instruction read eight rows, whose 16-byte pieces the swizzle spreads
        // over all banks.
        const uint8_t* pq_tile = cx.sm + Ly::oPq + wg * Ly::kTileP;
        auto take_pq = [&](int k, uint32_t (&f)[16]) -> bool {
            if (!wait_bar_warp(cx, w4PqFull + wg, (uint32_t)(k & 1), 104)) return false;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rbase + 8 * h;
#pragma unroll
                for (int x = 0; x < 8; ++x)
                    f[2 * x + h] = *reinterpret_cast<const uint32_t*>(pq_tile + row * 128 + ((x ^ (row & 7)) << 4) + 4 * q);
            }
            // the slot goes back to the TMA thread: these generic-proxy reads are ordered before the async-proxy write
            // of the next tile only through a proxy fence by the reading threads (without it a few 16-byte pieces of the
            // tile were now and then those of the next tile: outputs differed from run to run within the bf16 tolerance)
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(w4PqEmpty + wg));
            return true;
        };
        uint32_t pq_next[16];
        if (wg < nitems) ok = take_pq(0, pq_next);
        for (int i = wg, k = 0; i < nitems && ok; i += NWG, ++k) {
            const int c = i / G, g = i - c * G;
            uint32_t pqv[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) pqv[j] = pq_next[j];
            // running A of the group: written at the end of the previous item of this worker group (which is the
            // same bucket group when G = 4)
            if (!(ok = wait_bar_warp(cx, w4AcarReady + wg, (uint32_t)((k & 1) ^ 1), 101))) break;
            float* ac = reinterpret_cast<float*>(cx.sm + Ly::oAcar) + g * 64;
            float acar[16];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const float2 a2 = *reinterpret_cast<const float2*>(ac + 8 * x + 2 * q);
                acar[2 * x] = a2.x; acar[2 * x + 1] = a2.y;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(w4AcarRead + wg));
            // the warp that owns row 63 overwrites the values below: all four warps must hold them first
            if (w == 3 && !(ok = wait_bar_warp(cx, w4AcarRead + wg, (uint32_t)(k & 1), 102))) break;
            if (!(ok = wait_bar_warp(cx, w4XReady + wg, (uint32_t)(k & 1), 103))) break;
            tc_fence_after();
            // two halves of 32 buckets, to stay inside the registers a thread has: the W pairs of a half
            // go over columns of A_loc this warp has already loaded (half 0: columns 0..15 of its 0..31; half 1:
            // columns 16..31, loaded with half 0)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                float v[16];
                tmem_ld32(lane_base + tmX(wg) + 32 * hf, v);
                uint32_t wv[8];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float2 pq2 = unpack_bf16(pqv[2 * (4 * hf + x) + h]);
                        const float a0 = acar[2 * (4 * hf + x)] + v[4 * x + 2 * h];
                        const float a1 = acar[2 * (4 * hf + x) + 1] + v[4 * x + 2 * h + 1];
                        wv[2 * x + h] = pack_bf16(__fdividef(pq2.x, a0 + eps), __fdividef(pq2.y, a1 + eps));
                        if (h == 1 && w == 3 && (lane >> 2) == 7)    // row 63: the running A after this chunk
                            *reinterpret_cast<float2*>(ac + 8 * (4 * hf + x) + 2 * q) = make_float2(a0, a1);
                    }
                }
                tmem_st_pairs4(lane_base + tmX(wg) + 16 * hf, wv);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(cx.bar(w4WReady + wg));
                if (w == 3) mbar_arrive(cx.bar(w4AcarReady + wg));   // the new running A is in place
            }
            if (i + NWG < nitems && !(ok = take_pq(k + 1, pq_next))) break;
        }
    } else if (warp < Ly::kAuxWarp0) {
        // =========================== converter warpgroup ==========================================
        const int wtid = tid & 127;
        bool ok = true;
        for (int j = 0; j < npairs && ok; ++j) {
            const int c = j / P, p = j - c * P, st = j % NST;
            const uint32_t rp = (uint32_t)((j / NST) & 1);
            if (j >= NST && !(ok = wait_bar_warp(cx, w4KFree + st, rp ^ 1, 203))) break;
            if (!(ok = wait_bar_warp(cx, w4Full + st, rp, 201))) break;
            // two staged 64 x 64 boxes -> one [64 tokens][128 buckets] operand tile
#pragma unroll
            for (int hb = 0; hb < 2; ++hb)
                copy_tile<128, false>(cx.sm + Ly::oStage + st * Ly::kTileP2 + hb * Ly::kTileP,
                                      cx.sm + Ly::oKt + st * Ly::kTileP2, 64 * hb, wtid, nullptr);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(cx.bar(w4KReady + st)); mbar_arrive(cx.bar(w4Empty + st)); }
            if (p == 0) {
                // V slice of the chunk: [64 tokens][32 values], staged without swizzle
                const int vb = c & 1;
                const uint32_t vp = (uint32_t)((c >> 1) & 1);
                if (c >= 2 && !(ok = wait_bar_warp(cx, w4VFree + vb, vp ^ 1, 205))) break;
                if (!(ok = wait_bar_warp(cx, w4VFull + vb, vp, 206))) break;
                const uint8_t* src = cx.sm + Ly::oVst + vb * Ly::kTileS;
                uint8_t* dst = cx.sm + Ly::oVt + vb * Ly::kTileS;
#pragma unroll
                for (int it = 0; it < DSX / 16; ++it) {
                    const int idx = it * 128 + wtid;          // 64 rows of DSX / 8 pieces of 16 bytes
                    const int r = idx / (DSX / 8), jj = idx % (DSX / 8);
                    *reinterpret_cast<uint4*>(dst + off_w<DSX>(r, 8 * jj)) =
                        *reinterpret_cast<const uint4*>(src + r * (DSX * 2) + jj * 16);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) { mbar_arrive(cx.bar(w4VReady + vb)); mbar_arrive(cx.bar(w4VEmpty + vb)); }
            }
        }
    } else if (warp < Ly::kProducerWarp) {
        // =========================== auxiliary warpgroup: state operands, mask, output ============
        const int w = warp & 3, q = lane & 3, rbase = 16 * w + (lane >> 2);
        const uint32_t lane_base = (uint32_t)(32 * w) << 16;
        // a pair's state: thread <-> bucket row 32 w + lane of the pair (128 rows over the four warps), 32 columns
        const int prow = 32 * w + lane;
        float b[DSX];
        auto write_bt = [&](int p) {
            uint8_t* bt = cx.sm + Ly::oBt + p * 2 * Ly::kTileS;   // [128][32] bf16, 8x8 core matrices
#pragma unroll
            for (int j = 0; j < DSX / 8; ++j) {
                uint4 x4;
                x4.x = pack_bf16(b[8 * j], b[8 * j + 1]);
                x4.y = pack_bf16(b[8 * j + 2], b[8 * j + 3]);
                x4.z = pack_bf16(b[8 * j + 4], b[8 * j + 5]);
                x4.w = pack_bf16(b[8 * j + 6], b[8 * j + 7]);
                *reinterpret_cast<uint4*>(bt + off_w<DSX>(prow, 8 * j)) = x4;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(w4BtReady + p));
        };
        // carry-in of every pair: accumulator and operand tile
        for (int p = 0; p < P; ++p) {
            const float* srow = slice + (int64_t)(p * 2 * SG + prow) * D + js * DSX;
#pragma unroll
            for (int j = 0; j < DSX / 4; ++j) {
                const float4 f = *reinterpret_cast<const float4*>(srow + 4 * j);
                b[4 * j] = f.x; b[4 * j + 1] = f.y; b[4 * j + 2] = f.z; b[4 * j + 3] = f.w;
            }
#pragma unroll
            for (int hb = 0; hb < DSX / 32; ++hb)
                tmem_st_rows32(lane_base + tmBp(p) + 32 * hb, *reinterpret_cast<const float(*)[32]>(b + 32 * hb));
            tc_fence_before();
            write_bt(p);
        }
        bool ok = true;
        for (int c = 0; c < nch && ok; ++c) {
            const uint32_t cp = (uint32_t)(c & 1);
            const int64_t tok0 = t_begin + (int64_t)c * C;
            const int valid = (int)min((int64_t)C, t_end - tok0);
            auto carry = [&](int p) {   // state of pair p after this chunk -> operand tile for the next chunk
                tc_fence_after();
#pragma unroll
                for (int hb = 0; hb < DSX / 32; ++hb)
                    tmem_ld_rows32(lane_base + tmBp(p) + 32 * hb, *reinterpret_cast<float(*)[32]>(b + 32 * hb));
                tc_fence_before();
                write_bt(p);   // its arrival also tells the issuer that the accumulator has been read
            };
            for (int p = 0; p < P - 1 && ok; ++p) {
                if (!(ok = wait_bar_warp(cx, w4PairDone + p, cp, 501))) break;
                if (c + 1 < nch) carry(p);
            }
            if (!ok) break;
            // all groups have accumulated into G: causal mask -> bf16 pairs over G's first 32 columns
            if (!(ok = wait_bar_warp(cx, w4PairDone + P - 1, cp, 502))) break;
            {
                float v[32];
                uint32_t gv[16];
                tc_fence_after();
                tmem_ld64(lane_base + tmG, v);
                tc_fence_before();
#pragma unroll
                for (int x = 0; x < 8; ++x)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int row = rbase + 8 * h, col = 8 * x + 2 * q;
                        gv[2 * x + h] = pack_bf16(col <= row ? v[4 * x + 2 * h] : 0.f,
                                                  col + 1 <= row ? v[4 * x + 2 * h + 1] : 0.f);
                    }
                tmem_st_pairs(lane_base + tmG, gv);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(cx.bar(w4GtReady));
            }
            if (c + 1 < nch) carry(P - 1);
            // O of the chunk (this CTA's 32 columns)
            if (!(ok = wait_bar_warp(cx, w4OReady, cp, 503))) break;
            float o[DSX / 32][16];
            tc_fence_after();
#pragma unroll
            for (int hb = 0; hb < DSX / 32; ++hb) tmem_ld32(lane_base + tmO(c) + 32 * hb, o[hb]);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(w4OFree + (c % Ly::kOBufs)));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rbase + 8 * h;
                if (row < valid) {
                    // out in the layout of V: [N][T][D], or [N / heads][T][heads][D]
                    const int64_t orow_idx = heads > 1 ? (((n / heads) * T + tok0 + row) * heads + n % heads) : (n * T + tok0 + row);
                    __nv_bfloat16* orow = out + orow_idx * D + js * DSX + 2 * q;
#pragma unroll
                    for (int hb = 0; hb < DSX / 32; ++hb)
#pragma unroll
                        for (int x = 0; x < 4; ++x)
                            *reinterpret_cast<uint32_t*>(orow + 32 * hb + 8 * x) =
                                pack_bf16(o[hb][4 * x + 2 * h], o[hb][4 * x + 2 * h + 1]);
                }
            }
        }
    } else if (warp == Ly::kProducerWarp) {
        // =========================== TMA producer ==================================================
        if (lane == 0) {
            int issued = 0, v_issued = 0, q_issued = 0;
            bool pok = true;
            for (int j = 0; j < npairs; ++j) {
                const int c = j / P, p = j - c * P, st = j % NST;
                const int tok = (int)(t_begin + (int64_t)c * C);
                if (j >= NST && !wait_bar(cx, w4Empty + st, (uint32_t)(((j / NST) - 1) & 1), 301)) break;
                mbar_arrive_expect_tx(cx.bar(w4Full + st), Ly::kTileP2);
                // one box: the two column blocks of the pair, landing as two consecutive 64 x 64 tiles
                tma_load_4d(cx.sm_u32 + Ly::oStage + st * Ly::kTileP2, &map_k, cx.bar(w4Full + st), 0, tok, 2 * p, (int)n);
                issued = j + 1;
                if (p == 0) {
                    const int vb = c & 1;
                    if (c >= 2 && !wait_bar(cx, w4VEmpty + vb, (uint32_t)(((c >> 1) - 1) & 1), 302)) break;
                    mbar_arrive_expect_tx(cx.bar(w4VFull + vb), Ly::kTileS);
                    // heads > 1: V is [N / heads][T][heads][D] behind a 5-D map
                    if (heads > 1)
                        tma_load_5d(cx.sm_u32 + Ly::oVst + vb * Ly::kTileS, &map_vs, cx.bar(w4VFull + vb), 0, tok, js,
                                    (int)(n % heads), (int)(n / heads));
                    else
                        tma_load_4d(cx.sm_u32 + Ly::oVst + vb * Ly::kTileS, &map_vs, cx.bar(w4VFull + vb), 0, tok, js, (int)n);
                    v_issued = c + 1;
                }
                // pQ of the pair's two items last: their slots free up later than the pK stage does
                for (int i = 2 * j; i < 2 * j + 2 && pok; ++i) {       // pQ of the pair's two items
                    const int qs = i % NWG, qu = i / NWG;
                    if (qu >= 1 && !(pok = wait_bar(cx, w4PqEmpty + qs, (uint32_t)((qu - 1) & 1), 303))) break;
                    mbar_arrive_expect_tx(cx.bar(w4PqFull + qs), Ly::kTileP);
                    tma_load_4d(cx.sm_u32 + Ly::oPq + qs * Ly::kTileP, &map_q, cx.bar(w4PqFull + qs), 0, tok, i - c * G, (int)n);
                    q_issued = i + 1;
                }
                if (!pok) break;
            }
            if (*cx.abort_flag) {   // copies in flight must land before the CTA may exit
                for (int j = max(0, issued - NST); j < issued; ++j) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(w4Full + j % NST), (uint32_t)((j / NST) & 1)) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
                for (int c = max(0, v_issued - 2); c < v_issued; ++c) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(w4VFull + (c & 1)), (uint32_t)((c >> 1) & 1)) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
                for (int i = max(0, q_issued - NWG); i < q_issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(w4PqFull + i % NWG), (uint32_t)((i / NWG) & 1)) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
            }
        }
    } else {
        // =========================== MMA issuer ======================================================
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
        const uint32_t smb = __shfl_sync(0xffffffffu, cx.sm_u32, 0);
        const int Gu = __shfl_sync(0xffffffffu, G, 0);
        const uint32_t tril_lo = lo_k(smb + Ly::oTril);
        constexpr uint32_t kI64 = idesc_n(64), kIS = idesc_n(DSX);
        constexpr uint32_t kIM128S = idesc_mn(128, DSX);
        if (elect_one()) {
            bool ok = true;
            // A_loc of item i = tril . pK_g: the group's 64 buckets are half (i & 1) of its pair's 128-wide tile
            auto cumsum = [&](int i) -> bool {
                const int j = i >> 1, st = j % NST, half = i & 1;
                if (half == 0 && !wait_bar(cx, w4KReady + st, (uint32_t)((j / NST) & 1), 401)) return false;
                tc_fence_after();
                mma_k64<true, kHiK, 16, kHiMN, Ly::kStepP2>(
                    tm + Ly::kTmX + (i % NWG) * 64, tril_lo,
                    lo_mn_w(smb + Ly::oKt + st * Ly::kTileP2 + half * 1024, Ly::kLboP2), kI64 | kBmn);
                mma_commit(cx.bar(w4XReady + (i % NWG)));
                return true;
            };
            auto gv = [&](int c) -> bool {       // O += masked G . V, once per chunk
                if (!wait_bar(cx, w4GtReady, (uint32_t)(c & 1), 406)) return false;
                tc_fence_after();
                mma_k64_ta<false, kHiMN, Ly::kStepS>(tm + Ly::kTmO + (c % Ly::kOBufs) * DSX, tm + Ly::kTmG,
                                                     lo_mn_w(smb + Ly::oVt + (c & 1) * Ly::kTileS, Ly::kLboS), kIS | kBmn);
                mma_commit(cx.bar(w4OReady));
                mma_commit(cx.bar(w4VFree + (c & 1)));
                return true;
            };
            for (int i = 0; i < NWG - 1 && i < nitems && ok; ++i) ok = cumsum(i);
            int c = 0, g = 0;
            for (int i = 0; i < nitems && ok; ++i) {
                const int p = g >> 1, half = g & 1, j = i >> 1, st = j % NST, wg = i % NWG;
                // three items ahead: its buffer held W of item i - 1, whose products were issued in the previous turn
                if (i + NWG - 1 < nitems && !(ok = cumsum(i + NWG - 1))) break;
                if (g == 0 && c >= 1 && !(ok = gv(c - 1))) break;        // frees G for this chunk
                // W of the item in tensor memory; state operand of the pair written (which also means that the
                // pair's accumulator has been read out after the previous chunk)
                if (!(ok = wait_bar2(cx, w4WReady + wg, (uint32_t)((i / NWG) & 1), w4BtReady + p, (uint32_t)(c & 1), 404))) break;
                if (g == 0) {
                    const int ob = c % Ly::kOBufs, ou = c / Ly::kOBufs;    // the chunk's O buffer and its use count
                    if (ou >= 1 && !(ok = wait_bar(cx, w4OFree + ob, (uint32_t)((ou - 1) & 1), 408))) break;
                    if (!(ok = wait_bar(cx, w4VReady + (c & 1), (uint32_t)((c >> 1) & 1), 407))) break;
                }
                tc_fence_after();
                const uint32_t a_w = tm + Ly::kTmX + wg * 64;
                const uint32_t kt = smb + Ly::oKt + st * Ly::kTileP2;
                const uint32_t kt_k = lo_k(kt + half * 1024);       // K-major: the group's buckets start 8 column groups in
                const uint32_t bt_mn = lo_mn_w(smb + Ly::oBt + p * 2 * Ly::kTileS + half * Ly::kTileS, Ly::kLboS);
                const uint32_t dO = tm + Ly::kTmO + (c % Ly::kOBufs) * DSX;
                if (g == 0) {
                    mma_k64_ta<true, Ly::kHiK2, 16>(tm + Ly::kTmG, a_w, kt_k, kI64);               // G  = W . pK^T
                    mma_k64_ta<true, kHiMN, Ly::kStepS>(dO, a_w, bt_mn, kIS | kBmn);          // O  = W . B_g
                } else {
                    mma_k64_ta<false, Ly::kHiK2, 16>(tm + Ly::kTmG, a_w, kt_k, kI64);              // G += ...
                    mma_k64_ta<false, kHiMN, Ly::kStepS>(dO, a_w, bt_mn, kIS | kBmn);         // O += ...
                }
                if (half == 1) {
                    // B_pair += [pK_a | pK_b]^T . V : M = 128, once per pair
                    const uint32_t vt_mn = lo_mn_w(smb + Ly::oVt + (c & 1) * Ly::kTileS, Ly::kLboS);
                    mma_k64<false, kHiMN, Ly::kStepP2, kHiMN, Ly::kStepS>(tm + p * DSX, lo_mn_w(kt, Ly::kLboP2), vt_mn,
                                                                          kIM128S | kAmn | kBmn);
                    mma_commit(cx.bar(w4PairDone + p));
                    mma_commit(cx.bar(w4KFree + st));
                }
                if (++g == Gu) { g = 0; ++c; }
            }
            if (ok && nch > 0) ok = gv(nch - 1);
            mma_commit(cx.bar(w4Drain));
            const long long t0 = clock64();
            while (!mbar_try_wait(cx.bar(w4Drain), 0) && clock64() - t0 < cx.limit) {}
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == Ly::kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// Tile totals for four or eight bucket groups: FOUR groups per CTA (the CTAs of a (stream, tile) then fetch
// the chunk's V tile twice instead of four times: the pass is bound by what the memory system delivers, L2 hits
// included).  The states of two adjacent groups are one M = 128 accumulator, as in the output pass above (A operand:
// the [64 tokens][128 buckets] pair tile, MN-major), and the column sums of pK come out of the same products: the V
// operand tile is 32 columns wider than d_k, column d_k holds ones, so accumulator column d_k is sum_t pK[t][bucket]
// (bf16 values times 1.0, summed in fp32 by the tensor core in a fixed order).
// TMEM: 2 pairs x (D + 32) columns.  Roles as in tile_totals_tc_bf16: two converter groups on alternate chunks
// (a stage always belongs to one group: the ring has two stages), TMA thread, issuing thread.
// ------------------------------------------------------------------------------------------------
constexpr int kT4Stages = 2;
template <int D>
struct Lay4 {
    static constexpr int DX = D + 32;                              // V operand tile: d_k columns, a ones column, padding
    static constexpr int kTileP = C * 64 * 2, kTileP2 = 2 * kTileP, kTileV = C * D * 2, kTileVx = C * DX * 2;
    static constexpr int kStage = 4 * kTileP + kTileV;
    static constexpr int oStage = 0;                               // [kT4Stages][4 pK tiles | V]
    static constexpr int oKt = oStage + kT4Stages * kStage;        // [2 groups][2 pairs][kTileP2]
    static constexpr int oVt = oKt + 2 * 2 * kTileP2;              // [2 groups][kTileVx]
    static constexpr int oBars = oVt + 2 * kTileVx;
    static constexpr int oMisc = oBars + 16 * 8;
    static constexpr int kSmem = oMisc + 16 + 1024;
    static constexpr uint32_t kLboVx = (DX / 8) * 128, kStepVx = (2 * kLboVx) >> 4;
    static constexpr uint32_t kLboP2 = (128 / 8) * 128, kStepP2 = (2 * kLboP2) >> 4;
    static_assert(2 * DX <= 512 && DX % 32 == 0, "tensor memory columns of the four-group totals kernel");
};
static_assert(Lay4<128>::kSmem <= 227 * 1024 && Lay4<64>::kSmem <= 227 * 1024, "shared memory of the four-group totals kernel");

template <int D>
__global__ void __launch_bounds__(kT1Threads, 1)
tile_totals4_tc_bf16(const __grid_constant__ CUtensorMap map_k4, const __grid_constant__ CUtensorMap map_v,
                     float* __restrict__ ws, int64_t T, int S, int G, int tile_tokens, int heads, int* status) {
    using Ly = Lay4<D>;
    constexpr int DX = Ly::DX;
    extern __shared__ uint8_t smem_raw[];
    Ctx cx;
    cx.sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    cx.sm_u32 = smem_u32(cx.sm);
    cx.bars = Ly::oBars;
    cx.abort_flag = reinterpret_cast<volatile int*>(cx.sm + Ly::oMisc + 4);
    cx.status = status;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(cx.sm + Ly::oMisc);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int GC = G / 4;                                    // CTAs per (stream, tile)
    const int g = (int)(blockIdx.x % (unsigned)GC) * 4;      // first bucket group of this CTA
    const int64_t tiles = gridDim.x / GC, tile = blockIdx.x / GC, n = blockIdx.y;
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(T, t_begin + (int64_t)tile_tokens);
    const int nch = (int)((t_end - t_begin + C - 1) / C);
    float* slice = ws + (n * tiles + tile) * (int64_t)(S * (D + 1));
    float* sliceB = slice + (int64_t)g * SG * D;
    float* sliceA = slice + (int64_t)S * D + g * SG;

    if (tid == 0) {
        *cx.abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(cx.bar(b1Full + i), 1);
            mbar_init(cx.bar(b1Empty + i), 4);
            mbar_init(cx.bar(b1KvReady + i), 4);
            mbar_init(cx.bar(b1KvFree + i), 1);
        }
        mbar_init(cx.bar(b1Done), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(cx.sm_u32 + Ly::oMisc), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the constant columns d_k .. d_k + 31 of both V operand tiles: ones in column d_k, zeros after it
    for (int i = tid; i < 2 * C * 4; i += kT1Threads) {
        const int buf = i / (C * 4), r = (i / 4) % C, jj = i % 4;
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (jj == 0) w.x = 0x3F80u;                          // bf16 1.0 in column d_k
        *reinterpret_cast<uint4*>(cx.sm + Ly::oVt + buf * Ly::kTileVx + off_w<DX>(r, D + 8 * jj)) = w;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp < 8) {
        const int wg = warp >> 2, wtid = tid & 127;
        bool ok = true;
        for (int c = wg; c < nch && ok; c += 2) {
            const int st = c % kT4Stages;                    // = wg: a stage always belongs to one group
            if (!(ok = wait_bar_warp(cx, b1Full + st, (c / kT4Stages) & 1, 111))) break;
            if (c >= 2 && !(ok = wait_bar_warp(cx, b1KvFree + wg, ((c >> 1) - 1) & 1, 112))) break;
            const uint8_t* stage = cx.sm + Ly::oStage + st * Ly::kStage;
#pragma unroll
            for (int t4 = 0; t4 < 4; ++t4)    // four staged 64 x 64 boxes -> two [64 tokens][128 buckets] pair tiles
                copy_tile<128, false>(stage + t4 * Ly::kTileP, cx.sm + Ly::oKt + (wg * 2 + (t4 >> 1)) * Ly::kTileP2,
                                      64 * (t4 & 1), wtid, nullptr);
#pragma unroll
            for (int dh = 0; dh < D / 64; ++dh)
                copy_tile<DX, false>(stage + 4 * Ly::kTileP + dh * 8192, cx.sm + Ly::oVt + wg * Ly::kTileVx, dh * 64,
                                     wtid, nullptr);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(cx.bar(b1KvReady + wg)); mbar_arrive(cx.bar(b1Empty + st)); }
        }
    } else if (warp == 8) {
        if (lane == 0) {
            int issued = 0;
            for (int c = 0; c < nch; ++c) {
                const int st = c % kT4Stages;
                if (c >= kT4Stages && !wait_bar(cx, b1Empty + st, ((c / kT4Stages) - 1) & 1, 311)) break;
                const uint32_t dst = cx.sm_u32 + Ly::oStage + st * Ly::kStage;
                const uint32_t bar = cx.bar(b1Full + st);
                const int tok = (int)(t_begin + (int64_t)c * C);
                mbar_arrive_expect_tx(bar, Ly::kStage);
                tma_load_4d(dst, &map_k4, bar, 0, tok, g, (int)n);                     // one box: four column blocks
                if (heads > 1) tma_load_5d(dst + 4 * Ly::kTileP, &map_v, bar, 0, tok, 0, (int)(n % heads), (int)(n / heads));
                else tma_load_4d(dst + 4 * Ly::kTileP, &map_v, bar, 0, tok, 0, (int)n);
                issued = c + 1;
            }
            if (*cx.abort_flag) {
                for (int c = max(0, issued - kT4Stages); c < issued; ++c) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(b1Full + c % kT4Stages), (c / kT4Stages) & 1) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
            }
        }
    } else {
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
        const uint32_t smb = __shfl_sync(0xffffffffu, cx.sm_u32, 0);
        constexpr uint32_t kI = idesc_mn(128, DX) | kAmn | kBmn;
        if (elect_one()) {
            bool ok = true;
            for (int c = 0; c < nch && ok; ++c) {
                const int wg = c & 1;
                if (!(ok = wait_bar(cx, b1KvReady + wg, (c >> 1) & 1, 411))) break;
                tc_fence_after();
                const uint32_t vt_mn = lo_mn_w(smb + Ly::oVt + wg * Ly::kTileVx, Ly::kLboVx);
#pragma unroll
                for (int t2 = 0; t2 < 2; ++t2) {
                    const uint32_t kt_mn = lo_mn_w(smb + Ly::oKt + (wg * 2 + t2) * Ly::kTileP2, Ly::kLboP2);
                    if (c == 0) mma_k64<true, kHiMN, Ly::kStepP2, kHiMN, Ly::kStepVx>(tm + t2 * DX, kt_mn, vt_mn, kI);
                    else mma_k64<false, kHiMN, Ly::kStepP2, kHiMN, Ly::kStepVx>(tm + t2 * DX, kt_mn, vt_mn, kI);
                }
                mma_commit(cx.bar(b1KvFree + wg));
            }
            mma_commit(cx.bar(b1Done));
        }
    }
    __syncthreads();
    if (warp < 4) {
        if (wait_bar_warp(cx, b1Done, 0, 113)) {
            const int q = lane & 3;
            float v[32];
#pragma unroll
            for (int t2 = 0; t2 < 2; ++t2) {
                // rows of the pair's accumulator = its 128 buckets on the 128 lanes; this warp reads lanes 32 w .. 32 w + 31
                // as two 16-lane fragments
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    const int r0 = 32 * warp + 16 * h2 + (lane >> 2);            // bucket row of register half h = 0
#pragma unroll
                    for (int dh = 0; dh < D / 64; ++dh) {
                        tc_fence_after();
                        tmem_ld64(((uint32_t)(32 * warp + 16 * h2) << 16) + tmem + t2 * DX + dh * 64, v);
                        tc_fence_before();
#pragma unroll
                        for (int x = 0; x < 8; ++x)
#pragma unroll
                            for (int h = 0; h < 2; ++h)
                                *reinterpret_cast<float2*>(sliceB + ((int64_t)t2 * 128 + r0 + 8 * h) * D + dh * 64 + 8 * x +
                                                           2 * q) = make_float2(v[4 * x + 2 * h], v[4 * x + 2 * h + 1]);
                    }
                }
                // column d_k of the accumulator: the column sums of pK (thread = bucket row)
                tc_fence_after();
                tmem_ld_rows32(((uint32_t)(32 * warp) << 16) + tmem + t2 * DX + D, v);
                tc_fence_before();
                sliceA[t2 * 128 + 32 * warp + lane] = v[0];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn_bf16() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        p = nullptr;
    if (!p) cudaGetLastError();
    fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
    return fn;
}

// [N][T][width] bf16 viewed as (64 values, T tokens, width/64 column blocks, N streams); one box =
// `blocks` adjacent column blocks of 64 values x 64 tokens (128-byte rows, 128B swizzle), which land as consecutive
// 8 KB tiles: one TMA instruction instead of `blocks` (an elected thread needs about 0.3 k clk for each); tokens past
// T read as zero
bool make_map_bf16(CUtensorMap* map, const void* base, int64_t N, int64_t T, int width, int blocks = 1, int heads = 1) {
    auto fn = encode_fn_bf16();
    if (!fn) return false;
    if (heads > 1) {   // [N / heads][T][heads][width]: (64 values, T tokens, column blocks, heads, outer)
        cuuint64_t dims5[5] = {64, (cuuint64_t)T, (cuuint64_t)(width / 64), (cuuint64_t)heads, (cuuint64_t)(N / heads)};
        cuuint64_t strides5[4] = {(cuuint64_t)heads * width * 2, 128, (cuuint64_t)width * 2,
                                  (cuuint64_t)T * heads * width * 2};
        cuuint32_t box5[5] = {64, (cuuint32_t)C, (cuuint32_t)blocks, 1, 1};
        cuuint32_t estr5[5] = {1, 1, 1, 1, 1};
        return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims5, strides5, box5, estr5,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    cuuint64_t dims[4] = {64, (cuuint64_t)T, (cuuint64_t)(width / 64), (cuuint64_t)N};
    cuuint64_t strides[3] = {(cuuint64_t)width * 2, 128, (cuuint64_t)T * width * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)C, (cuuint32_t)blocks, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// V [N][T][width] bf16 viewed as (ds values, T tokens, width/ds column blocks, N streams); one box =
// ds values x 64 tokens (rows of 2 ds bytes, no swizzle); tokens past T read as zero
bool make_map_bf16_slice(CUtensorMap* map, const void* base, int64_t N, int64_t T, int width, int ds, int heads = 1) {
    auto fn = encode_fn_bf16();
    if (!fn) return false;
    if (heads > 1) {   // [N / heads][T][heads][width]
        cuuint64_t dims5[5] = {(cuuint64_t)ds, (cuuint64_t)T, (cuuint64_t)(width / ds), (cuuint64_t)heads,
                               (cuuint64_t)(N / heads)};
        cuuint64_t strides5[4] = {(cuuint64_t)heads * width * 2, (cuuint64_t)ds * 2, (cuuint64_t)width * 2,
                                  (cuuint64_t)T * heads * width * 2};
        cuuint32_t box5[5] = {(cuuint32_t)ds, (cuuint32_t)C, 1, 1, 1};
        cuuint32_t estr5[5] = {1, 1, 1, 1, 1};
        return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims5, strides5, box5, estr5,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    cuuint64_t dims[4] = {(cuuint64_t)ds, (cuuint64_t)T, (cuuint64_t)(width / ds), (cuuint64_t)N};
    cuuint64_t strides[3] = {(cuuint64_t)width * 2, (cuuint64_t)ds * 2, (cuuint64_t)T * width * 2};
    cuuint32_t box[4] = {(cuuint32_t)ds, (cuuint32_t)C, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
cudaError_t launch_bf16(const void* pq, const void* pk, const void* v, void* out, const float* carry_in,
                        float* state_out, void* ws, const Dims& dm, int tile_tokens, cudaStream_t stream,
                        int* status, int phases, bool global_norm) {
    const int G = dm.S / SG;
    if (global_norm && G > 1) return cudaErrorInvalidValue;   // the one-group kernel has the global form
    if (dm.H > 1 && G < 4) return cudaErrorInvalidValue;      // the heads layout of V / out: the wide kernel below
    // two bucket groups per totals CTA where there are at least two (they share the V tile)
    const int GP = G >= 2 ? 2 : 1;
    auto k1 = GP == 2 ? tile_totals_tc_bf16<D, 2> : tile_totals_tc_bf16<D, 1>;
    const int k1_smem = GP == 2 ? Lay1<D, 2>::kSmem : Lay1<D, 1>::kSmem;
    auto k3 = global_norm ? causal_out_tc_bf16<D, true> : causal_out_tc_bf16<D, false>;
    // runtime call first: binds the primary context to this host thread for the map encoder
    cudaError_t err = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, k1_smem);
    if (err != cudaSuccess) return err;
    // mk: one pK column block per box; mk2: two (a pair of bucket groups); mv: all of V's column blocks in one box
    CUtensorMap mk, mk2, mv;
    if (!make_map_bf16(&mk, pk, dm.N, dm.T, dm.S) || !make_map_bf16(&mk2, pk, dm.N, dm.T, dm.S, GP) ||
        !make_map_bf16(&mv, v, dm.N, dm.T, dm.D, D / 64, dm.H))
        return cudaErrorInvalidValue;
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    dim3 grid((unsigned)(tiles * G), (unsigned)dm.N);
    if ((phases & kPhaseTotals) && G >= 4) {
        // four bucket groups per CTA, pair-stacked accumulators, column sums by the tensor core
        CUtensorMap mk4;
        if (!make_map_bf16(&mk4, pk, dm.N, dm.T, dm.S, 4)) return cudaErrorInvalidValue;
        auto k4 = tile_totals4_tc_bf16<D>;
        err = cudaFuncSetAttribute(k4, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay4<D>::kSmem);
        if (err != cudaSuccess) return err;
        dim3 grid4((unsigned)(tiles * (G / 4)), (unsigned)dm.N);
        k4<<<grid4, kT1Threads, Lay4<D>::kSmem, stream>>>(mk4, mv, (float*)ws, dm.T, dm.S, G, tile_tokens, dm.H, status);
        err = cudaGetLastError();
        if (err != cudaSuccess) return err;
    } else if (phases & kPhaseTotals) {
        dim3 grid1((unsigned)(tiles * (G / GP)), (unsigned)dm.N);
        k1<<<grid1, kT1Threads, k1_smem, stream>>>(mk2, mv, (float*)ws, dm.T, dm.S, G, tile_tokens, dm.H, status);
        err = cudaGetLastError();
        if (err != cudaSuccess) return err;
    }
    if (!(phases & kPhaseOutput)) {
        if (!state_out) return cudaSuccess;   // the caller wants the per-tile totals alone
        return causal_scan_tiles((float*)ws, carry_in, state_out, dm, tile_tokens, stream, false);
    }
    err = causal_scan_tiles((float*)ws, carry_in, state_out, dm, tile_tokens, stream, true);
    if (err != cudaSuccess) return err;
    if (G > 1) {
        // all bucket groups in one CTA, the head dimension in slices
        CUtensorMap mvs;
        if (G >= 4) {
            // 64-column slices, two worker groups: the states of the pairs take 256 columns of tensor memory, which
            // leaves two A_loc / W buffers
            using LyW = LayW4<64, 2, 3>;
            auto kw = causal_out_wide4_bf16<64, 2, 3>;
            constexpr int ds = 64;
            CUtensorMap mq;
            if (!make_map_bf16_slice(&mvs, v, dm.N, dm.T, dm.D, ds, dm.H) || !make_map_bf16(&mq, pq, dm.N, dm.T, dm.S))
                return cudaErrorInvalidValue;
            err = cudaFuncSetAttribute(kw, cudaFuncAttributeMaxDynamicSharedMemorySize, LyW::kSmem);
            if (err != cudaSuccess) return err;
            dim3 wgrid4((unsigned)(tiles * (D / ds)), (unsigned)dm.N);
            kw<<<wgrid4, LyW::kThreads, LyW::kSmem, stream>>>(
                mq, mk2, mvs, (__nv_bfloat16*)out, (const float*)ws, dm.T, dm.S, D, G, tile_tokens,
                dm.eps, dm.H, status);
            return cudaGetLastError();
        }
        if (!make_map_bf16_slice(&mvs, v, dm.N, dm.T, dm.D, DS)) return cudaErrorInvalidValue;
        dim3 wgrid((unsigned)(tiles * (D / DS)), (unsigned)dm.N);
        err = cudaFuncSetAttribute(causal_out_wide_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, LayW::kSmem);
        if (err != cudaSuccess) return err;
        CUtensorMap mq2;
        if (!make_map_bf16(&mq2, pq, dm.N, dm.T, dm.S)) return cudaErrorInvalidValue;
        causal_out_wide_bf16<<<wgrid, kWThreads, LayW::kSmem, stream>>>(
            mq2, mk, mvs, (__nv_bfloat16*)out, (const float*)ws, dm.T, dm.S, D, G, tile_tokens,
            dm.eps, status);
        return cudaGetLastError();
    }
    err = cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay<D>::kSmem);
    if (err != cudaSuccess) return err;
    CUtensorMap mq1;
    if (!make_map_bf16(&mq1, pq, dm.N, dm.T, dm.S)) return cudaErrorInvalidValue;
    k3<<<grid, kThreads, Lay<D>::kSmem, stream>>>(mq1, mk, mv, (__nv_bfloat16*)out,
                                                  (const float*)ws, dm.T, dm.S, G, tile_tokens, dm.eps, status);
    return cudaGetLastError();
}

}  // namespace

bool tensor_bf16_supported(const Dims& dm) {
    const int G = dm.S / SG;
    // the heads layout of V / out ([N / H][T][H][D]) is read by the kernel of four and eight bucket groups
    return dm.S % SG == 0 && (G == 1 || G == 2 || G == 4 || G == 8) && (dm.D == 64 || dm.D == 128) &&
           dm.N >= 0 && dm.N <= 65535 && dm.T < (1ll << 31) && (dm.H == 1 || (G >= 4 && dm.N % dm.H == 0));
}

cudaError_t causal_fwd_tensor_bf16(const void* pq, const void* pk, const void* v, void* out,
                                   const float* carry_in, float* state_out, void* ws, const Dims& dm,
                                   int tile_tokens, cudaStream_t stream, int* status, int phases, bool global_norm) {
    if (dm.D == 64)
        return launch_bf16<64>(pq, pk, v, out, carry_in, state_out, ws, dm, tile_tokens, stream, status, phases,
                               global_norm);
    return launch_bf16<128>(pq, pk, v, out, carry_in, state_out, ws, dm, tile_tokens, stream, status, phases,
                            global_norm);
}

#ifdef RACE_TC_TRACE
extern "C" int race_b200_debug_set_trace_bf16(long long* buf) {
    return (int)cudaMemcpyToSymbol(g_trace_buf, &buf, sizeof(buf));
}
#endif

}  // namespace race
