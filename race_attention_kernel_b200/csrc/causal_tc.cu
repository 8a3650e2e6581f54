// tcgen05 / TMEM / TMA output pass of the causal per-bucket prefix path (sm_100a).
//
// One CTA owns a (stream, state tile) and walks it in chunks of C = 64 tokens.  Per chunk
// (S = 64 buckets, D = 64 head dim, carry (A [S], B [S,D]) from the tiles before it):
//     A_in = A + tril_ones . pK            tcgen05.mma   (inclusive running sum inside the chunk)
//     W    = pQ / (A_in + eps)             CUDA cores, TMEM -> registers -> TMEM (MMA A operand)
//     G    = tril(W . pK^T)                tcgen05.mma, masked on the way TMEM -> registers -> TMEM
//     O    = W . B + G . V                 tcgen05.mma
//     B   += pK^T . V                      tcgen05.mma, accumulator resident in TMEM
// which is the chunk identity of the estimator in src/race_baseline.py:45-51
// (docs/causal_v2_design.md:70-77).  fp32 inputs are split into bf16 hi + lo limbs and every
// product runs as hi*hi + hi*lo + lo*hi with fp32 accumulation, so operand error is ~2^-17.
// pK, V and the state B are limb tiles in shared memory; W, the masked G and the triangular ones
// matrix are A operands in tensor memory and never touch shared memory.
//
// Warp roles (15 warps): two worker warpgroups take alternate chunks (W, mask of G, output
// store); a converter warpgroup turns the TMA-staged fp32 pK and V tiles into limb tiles and
// copies the running B from TMEM to its bf16 operand tile after every update; one warp issues
// TMA loads into a two-stage ring; one warp per worker group issues its tcgen05.mma
// instructions.  All hand-offs are mbarriers; every wait is bounded and a wait that runs out
// raises the status word and makes the CTA drain and exit.
// With heads = H > 1, V is read and out written in the layout [N/H, T, H, D] (stream n =
// outer * H + h): V through a five-dimensional tensor map, out with the head stride.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "launch.h"
#include "probs_frag.cuh"
#include "tc_common.cuh"


namespace race {
namespace {

constexpr int C = 64;           // tokens per chunk
constexpr int S = 64;           // buckets per CTA
constexpr int D = 64;           // head dim
constexpr int kThreads = 15 * 32;
constexpr int kProducerWarp = 12;
constexpr int kMmaWarp = 13;       // warps 13 and 14 issue the MMAs of worker group 0 / 1
constexpr uint32_t kTmemCols = 512;

// ---- shared memory map (bytes from a 1024-aligned base) ---------------------------------------
constexpr int kTileF32 = C * 64 * 4;        // one staged fp32 tile: 64 tokens x 64 values
constexpr int kStageBytes = 2 * kTileF32;   // pK | V  (pQ goes global -> registers)
constexpr int kOpTile = C * 64 * 2;         // one bf16 operand tile (8 KB)
constexpr int oStage = 0;                               // [2][kStageBytes]
constexpr int oKt = oStage + 2 * kStageBytes;           // [2 wg][2 buffers][hi|lo]
constexpr int oVt = oKt + 8 * kOpTile;
constexpr int oBt = oVt + 4 * kOpTile;                  // [2 buffers][hi|lo]
constexpr int oAcar = oBt + 4 * kOpTile;                // [2][64] fp32
constexpr int oBars = oAcar + 2 * 64 * 4;
constexpr int kNumBars = 34;
constexpr int oMisc = oBars + kNumBars * 8;             // tmem base, abort flag
constexpr int oPlaneTab = oMisc + 16;                   // plane fragments (kernels that form the probabilities)
constexpr int kSmemBytes = oPlaneTab + kPlaneTabWords * 4 + 1024;   // + slack for manual alignment

enum Bar {
    kFull = 0,      // [2] stage filled by TMA
    kEmpty = 2,     // [2] stage released by its worker group (4 warp arrivals)
    kKvReady = 4,   // [2] pK operand tile written
    kXReady = 6,    // [2] A_loc accumulator complete
    kWReady = 8,    // [2] W operand tile written
    kGReady = 10,   // [2] W.B and G accumulators complete
    kGtReady = 12,  // [2] masked G operand tile written
    kOReady = 14,   // [2] O accumulator complete
    kAcar = 16,     // [2] running A of the chunk published
    kBupdDone = 18, // B accumulator holds the state after chunk c
    kBaccFree = 19, // [2] B accumulator read out, free for the update of chunk c: barrier c & 1
    kBtReady = 21,  // [2] B operand buffer (c & 1) holds the state before chunk c (count 4)
    kDrain = 23,    // [2]
    kAcarFree = 25, // [2] running-A buffer of group g read by all four of its warps
    kVReady = 27,   // [2] V operand tile written
    kKtFree = 29    // [2 wg][2 buffers] pK operand buffer no longer read by any product
};

// fp32 staged tile (two 128B-swizzled halves of 32 columns) -> bf16 hi/lo operand tiles
__device__ __forceinline__ void convert_tile(const uint8_t* __restrict__ stage, uint8_t* __restrict__ hi,
                                             uint8_t* __restrict__ lo, int tid) {
    // all loads first: the staged tile and the operand tiles are different buffers, but only loads issued
    // ahead of the stores overlap their latencies
    float4 av[4], bv[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 128 + tid;
        const int j = idx >> 6, r = idx & 63;            // 8-column group, token row
        const uint8_t* src = stage + (j >> 2) * 8192 + r * 128;
        const int jj = j & 3;
        av[it] = *reinterpret_cast<const float4*>(src + (((2 * jj) ^ (r & 7)) << 4));
        bv[it] = *reinterpret_cast<const float4*>(src + (((2 * jj + 1) ^ (r & 7)) << 4));
    }
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 128 + tid;
        const int j = idx >> 6, r = idx & 63;
        const float4 a = av[it], b = bv[it];
        uint4 h, l;
        split2(a.x, a.y, h.x, l.x);
        split2(a.z, a.w, h.y, l.y);
        split2(b.x, b.y, h.z, l.z);
        split2(b.z, b.w, h.w, l.w);
        const uint32_t off = (uint32_t)((((r >> 3) * 8 + j) << 7) + ((r & 7) << 4));
        *reinterpret_cast<uint4*>(hi + off) = h;
        *reinterpret_cast<uint4*>(lo + off) = l;
    }
}

// Staged fp32 K tile (64 tokens x 64 features, the same two swizzled halves) -> bucket probabilities -> bf16 hi/lo
// operand tiles, by the four warps of a converter group: warp w takes the tokens 16 w .. 16 w + 15, a lane the rows
// g and g + 8 of them (probs_frag.cuh), and ends up with table t = lane % 4 of both rows, i.e. the 8-column groups
// 2 t and 2 t + 1 of the operand tile.  Rows >= valid (past the end of the sequence) become zero, like the rows the
// TMA unit fills for a probabilities tile.  kSum adds the lane's probabilities into asum[16] (column 16 t + i).
template <bool kSum>
__device__ __forceinline__ void produce_tile(const uint8_t* __restrict__ stage, uint8_t* __restrict__ hi,
                                             uint8_t* __restrict__ lo, const PlaneFrags& pf, int w, int lane,
                                             int valid, float (&asum)[16]) {
    const int g = lane >> 2, t = lane & 3;
    float2 raw[16];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = 16 * w + g + 8 * h;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint8_t* src = stage + (u >> 2) * 8192 + r * 128;
            const int unit = 2 * (u & 3) + (t >> 1);       // 16-byte unit of columns 8 u + 2 t, + 1 within the half
            raw[2 * u + h] = *reinterpret_cast<const float2*>(src + ((unit ^ (r & 7)) << 4) + ((t & 1) << 3));
        }
    }
    float c[2][4];
    project_rows(raw, pf, c);
    float vals[2][16];
    table_probs(c, lane, 0.125f, vals);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = 16 * w + g + 8 * h;
        if (r >= valid) {
#pragma unroll
            for (int i = 0; i < 16; ++i) vals[h][i] = 0.f;
        }
        if (kSum) {
#pragma unroll
            for (int i = 0; i < 16; ++i) asum[i] += vals[h][i];
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            uint4 hv, lv;
            split2(vals[h][8 * half], vals[h][8 * half + 1], hv.x, lv.x);
            split2(vals[h][8 * half + 2], vals[h][8 * half + 3], hv.y, lv.y);
            split2(vals[h][8 * half + 4], vals[h][8 * half + 5], hv.z, lv.z);
            split2(vals[h][8 * half + 6], vals[h][8 * half + 7], hv.w, lv.w);
            const uint32_t off = (uint32_t)((((r >> 3) * 8 + 2 * t + half) << 7) + ((r & 7) << 4));
            *reinterpret_cast<uint4*>(hi + off) = hv;
            *reinterpret_cast<uint4*>(lo + off) = lv;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Barriers of the output phase (one thread; the caller orders this against their use).  With
// `again` the objects held a previous tile's phases and are invalidated first.
// arrival count of output-phase barrier i (the table restates out_phase_init_bars)
__device__ __forceinline__ uint32_t out_bar_count(int i) {
    // bit i set: four arrivals (one per warp of a group), else one
    constexpr uint64_t kFour = (3ull << kEmpty) | (3ull << kKvReady) | (3ull << kWReady) | (3ull << kGtReady) |
                               (3ull << kBaccFree) | (3ull << kBtReady) | (3ull << kAcarFree) | (3ull << kVReady);
    return ((kFour >> i) & 1ull) ? 4u : 1u;
}
// The same from the lanes of one warp (re-initialisation between the tiles of the persistent kernel).
__device__ __forceinline__ void out_phase_reinit_bars_warp(const Ctx& cx, int lane, bool again) {
    for (int i = lane; i < kNumBars; i += 32) {
        if (again) mbar_inval(cx.bar(i));
        mbar_init(cx.bar(i), out_bar_count(i));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// empty_arrivals: warps that release a stage (4: the converter group reads pK and V; 8: the worker group reads its
// K tile itself and the converter group V)
__device__ __forceinline__ void out_phase_init_bars(const Ctx& cx, bool again, uint32_t empty_arrivals = 4) {
    if (again)
        for (int i = 0; i < kNumBars; ++i) mbar_inval(cx.bar(i));
    {
        for (int i = 0; i < 2; ++i) {
            mbar_init(cx.bar(kFull + i), 1);
            mbar_init(cx.bar(kEmpty + i), empty_arrivals);
            mbar_init(cx.bar(kKvReady + i), 4);
            mbar_init(cx.bar(kXReady + i), 1);
            mbar_init(cx.bar(kWReady + i), 4);
            mbar_init(cx.bar(kGReady + i), 1);
            mbar_init(cx.bar(kGtReady + i), 4);
            mbar_init(cx.bar(kOReady + i), 1);
            mbar_init(cx.bar(kAcar + i), 1);
            mbar_init(cx.bar(kAcarFree + i), 4);
            mbar_init(cx.bar(kVReady + i), 4);
            mbar_init(cx.bar(kKtFree + 2 * i), 1);
            mbar_init(cx.bar(kKtFree + 2 * i + 1), 1);
        }
        mbar_init(cx.bar(kBupdDone), 1);
        mbar_init(cx.bar(kBaccFree), 4);
        mbar_init(cx.bar(kBaccFree + 1), 4);
        mbar_init(cx.bar(kBtReady), 4);
        mbar_init(cx.bar(kBtReady + 1), 4);
        mbar_init(cx.bar(kDrain), 1);
        mbar_init(cx.bar(kDrain + 1), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
}

// Output phase of one (stream n, tokens [t_begin, t_end)) tile whose carry (state before its first
// token, state layout) is at `slice`.  Called by all 15 warps with barriers initialised and 512 TMEM
// columns at `tmem`; ends with every issued product retired, before the caller's __syncthreads.
// kMode: kModeBucket is the per-bucket estimator; kModeGlobal the global-normalisation estimator
// (src/causal_v2/reference.py:106-127): W = pQ without the per-bucket divide and every output row divided by
// den_t = pQ_t . A_t (0 -> a row of 0); kModeRaw the plain causal product O = pQ . B + tril(pQ pK^T) . V without any
// normalisation (the building block of the backward passes, where pQ / pK / V stand for other tensors).
// kReverse walks the tile from its last chunk to its first with an upper-triangular mask: out_t sums over
// j >= t, and the carry is the state of everything AFTER the tile (the suffix sums of the backward).
// withhold (self-test of the bounded waits): the TMA producer skips the load of chunk withhold_chunk.
// l2_last_use: this is the second read of the tile's pK and V (single-pass kernel), so their lines are loaded
// with the evict-first priority and leave the L2 to the tiles still waiting for their second read.
// kProj: the kernel forms the bucket probabilities itself (d_k = 64, L = 4 tables of R = 16 buckets;
// src/race_baseline.py:41-44): `pq` is Q and map_k covers K, both in the layout of V ([N/heads, T, heads, 64]); the
// worker warps turn their rows of Q into probabilities in the accumulator-fragment layout, the converter group turns
// the staged K tile into the pK operand tiles; ptab = the plane fragments in shared memory (build_plane_tab).
// kWorkerK: the pK operand tile of a chunk is written by the warps of the chunk's own worker group (at the start of
// their work on the chunk) instead of the converter group, which then only converts V and copies the running B.
// kModeRawX: the plain product with the epilogue of the first backward pass (BwdX in launch.h): after G . V the
// issuer also runs the triangular running-sum product over the chunk's V operand into the accumulator that G has
// left, and the worker warps turn X (the product) into dPQ, W and g where they would store it.
constexpr int kModeBucket = 0, kModeGlobal = 1, kModeRaw = 2, kModeRawX = 3;
template <int kMode, bool kReverse = false, bool kProj = false, bool kWorkerK = kProj>
__device__ __forceinline__ void out_phase(const Ctx& cx, const uint32_t tmem, const float* __restrict__ pq,
                                          const CUtensorMap* map_k, const CUtensorMap* map_v,
                                          float* __restrict__ out, const float* __restrict__ slice, int64_t T,
                                          const int64_t t_begin, const int64_t t_end, const int64_t n, float eps,
                                          int heads, int withhold_chunk, const bool l2_last_use = false,
                                          const uint32_t* ptab = nullptr, const BwdX* bx = nullptr) {
    constexpr bool kGlobal = kMode == kModeGlobal;
    constexpr bool kRaw = kMode == kModeRaw || kMode == kModeRawX;   // no running sum, no normalisation in the W stage
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nch = (int)((t_end - t_begin + C - 1) / C);
    // first token of the chunk that is processed c-th
    auto chunk_tok0 = [&](int c) { return t_begin + (int64_t)(kReverse ? nch - 1 - c : c) * C; };
    const uint32_t tmB = tmem;                               // B accumulator, columns [0, 64)
    auto tmAG = [&](int wg) { return tmem + 64 + wg * 128; };      // A_loc, then G
    auto tmO = [&](int wg) { return tmem + 64 + wg * 128 + 64; };  // O
    // MMA A operands kept in tensor memory (bf16 pairs, 32 columns per limb): W of the chunk, later its
    // masked G, per group [hi | lo]; and the constant lower-triangular ones matrix
    auto tmWG = [&](int wg) { return tmem + 320 + wg * 64; };
    const uint32_t tmTril = tmem + 448;

    if (warp < 8) {
        // =========================== worker warpgroups =========================================
        const int wg = warp >> 2, w = warp & 3;
        const int q = lane & 3, rbase = 16 * w + (lane >> 2);
        const uint32_t lane_base = (uint32_t)(32 * w) << 16;
        // V and out are [N/heads, T, heads, D]: stream n = outer * heads + h (heads = 1: plain [N, T, D])
        const int64_t orow_stride = (int64_t)heads * D;
        float* out_n = out + ((n / heads) * T * heads + (n % heads)) * D;
        // probabilities [N, T, S]; with kProj the rows of Q in the layout of V
        const float* pq_n = kProj ? pq + ((n / heads) * T * heads + (n % heads)) * D : pq + n * T * S;
        const int64_t pq_stride = kProj ? orow_stride : (int64_t)S;
        float v[32];
        uint32_t ohi[16], olo[16];   // operand limbs of W / masked G on their way to tensor memory

        // O of chunk c: TMEM -> global (fragment rows rbase, rbase + 8; 8-byte stores, full sectors)
        float den[2] = {1.f, 1.f};   // global form: denominators of rows rbase, rbase + 8 of the chunk
        auto store_out = [&](int c) {
            const int64_t tok0 = chunk_tok0(c);
            const int valid = (int)min((int64_t)C, t_end - tok0);
            tc_fence_after();
            tmem_ld64(lane_base + tmO(wg), v);
            tc_fence_before();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rbase + 8 * h;
                if (row < valid) {
                    float* orow = out_n + (tok0 + row) * orow_stride + 2 * q;
                    const float sc = kGlobal ? (den[h] != 0.f ? 1.f / den[h] : 0.f) : 1.f;
#pragma unroll
                    for (int x = 0; x < 8; ++x) {
                        float2 o2 = make_float2(v[4 * x + 2 * h], v[4 * x + 2 * h + 1]);
                        if (kGlobal) { o2.x *= sc; o2.y *= sc; }
                        __stcs(reinterpret_cast<float2*>(orow + 8 * x), o2);
                    }
                }
            }
        };

        // pQ (kProj: the rows of Q) of chunk c in the accumulator-fragment layout, straight from global memory
        float2 pqv[16];
        // kModeRawX: X of chunk c (in the O accumulator) and the chunk's running sum of pK (in the accumulator that
        // held G) -> dPQ, W, g; pqv holds the true query probabilities of the chunk (requested after the W stage)
        auto store_bwdx = [&](int c) {
            const int64_t tok0 = chunk_tok0(c);
            const int valid = (int)min((int64_t)C, t_end - tok0);
            const float* ab = bx->ablock + (n * bx->nblk + tok0 / bx->block_tokens) * S;
            const float* ac = bx->achunk + (n * bx->nchunk + tok0 / C) * S;
            float* w_n = bx->w_out + n * T * S;
            float* g_n = bx->g_out + n * T * S;
            tc_fence_after();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float xv[16], av[16];
                tmem_ld32(lane_base + tmO(wg) + 32 * half, xv);
                tmem_ld32(lane_base + tmAG(wg) + 32 * half, av);
#pragma unroll
                for (int xx = 0; xx < 4; ++xx) {
                    const int x = 4 * half + xx, col = 8 * x + 2 * q;
                    const float2 b2 = __ldg(reinterpret_cast<const float2*>(ab + col));
                    const float2 c2 = __ldg(reinterpret_cast<const float2*>(ac + col));
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int row = rbase + 8 * h;
                        if (row < valid) {
                            const float a0 = (b2.x + c2.x) + av[4 * xx + 2 * h];
                            const float a1 = (b2.y + c2.y) + av[4 * xx + 2 * h + 1];
                            const float i0 = __fdividef(1.f, a0 + bx->eps), i1 = __fdividef(1.f, a1 + bx->eps);
                            const float2 pq2 = pqv[2 * x + h];
                            const float2 w2 = make_float2(pq2.x * i0, pq2.y * i1);
                            const float2 d2 = make_float2(xv[4 * xx + 2 * h] * i0, xv[4 * xx + 2 * h + 1] * i1);
                            const int64_t o = (tok0 + row) * S + col;
                            __stcs(reinterpret_cast<float2*>(out_n + o), d2);
                            __stcs(reinterpret_cast<float2*>(w_n + o), w2);
                            __stcs(reinterpret_cast<float2*>(g_n + o), make_float2(-d2.x * w2.x, -d2.y * w2.y));
                        }
                    }
                }
            }
            tc_fence_before();
        };
        auto load_pq_true = [&](int c) {
            const int64_t tok0 = chunk_tok0(c);
            const int valid = (int)min((int64_t)C, t_end - tok0);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rbase + 8 * h;
                const float* prow = bx->pq_true + (n * T + tok0 + row) * S + 2 * q;
#pragma unroll
                for (int x = 0; x < 8; ++x)
                    pqv[2 * x + h] = row < valid ? __ldcs(reinterpret_cast<const float2*>(prow + 8 * x))
                                                 : make_float2(0.f, 0.f);
            }
        };
        auto load_pq = [&](int c) {
            const int64_t tok0 = chunk_tok0(c);
            const int valid = (int)min((int64_t)C, t_end - tok0);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rbase + 8 * h;
                const float* prow = pq_n + (tok0 + row) * pq_stride + 2 * q;
#pragma unroll
                for (int x = 0; x < 8; ++x)
                    pqv[2 * x + h] = row < valid ? __ldcs(reinterpret_cast<const float2*>(prow + 8 * x))
                                                 : make_float2(0.f, 0.f);
            }
        };
        if (kProj && wg < nch) load_pq(wg);
        // kWorkerK: the pK operand tile of chunk c from the group's stage (convert, or with kProj form the
        // probabilities), into buffer (c >> 1) & 1 of the group, last read by the products of the group's chunk c - 4
        auto write_kt = [&](int c, const PlaneFrags& pf) {
            const int kb = (c >> 1) & 1;
            uint8_t* kt_hi = cx.sm + oKt + (wg * 2 + kb) * 2 * kOpTile;
            const uint8_t* stage = cx.sm + oStage + wg * kStageBytes;
            if (kProj) {
                float unused[16];
                produce_tile<false>(stage, kt_hi, kt_hi + kOpTile, pf, w, lane,
                                    (int)min((int64_t)C, t_end - chunk_tok0(c)), unused);
            } else {
                convert_tile(stage, kt_hi, kt_hi + kOpTile, tid & 127);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(cx.bar(kKvReady + wg)); mbar_arrive(cx.bar(kEmpty + wg)); }
        };
        // kProj: the rows of Q in pqv -> the probabilities of chunk c, in place (rows past the end stay zero)
        auto q_to_probs = [&](int c, const PlaneFrags& pf) {
            const int valid = (int)min((int64_t)C, t_end - chunk_tok0(c));
            float cp[2][4];
            project_rows(pqv, pf, cp);
            fragment_probs(cp, lane, 0.125f, pqv);
#pragma unroll
            for (int h = 0; h < 2; ++h)
                if (rbase + 8 * h >= valid) {
#pragma unroll
                    for (int x = 0; x < 8; ++x) pqv[2 * x + h] = make_float2(0.f, 0.f);
                }
        };
        uint32_t ph = 0;   // parity of this group's per-chunk barriers (one use per chunk)
        bool ok = true;
        for (int c = wg; c < nch && ok; c += 2, ph ^= 1) {
            const int64_t tok0 = chunk_tok0(c);
            const int valid = (int)min((int64_t)C, t_end - tok0);
            // probabilities: issued first so that the wait for the running-sum product hides the latency; the
            // rows of Q were requested a chunk ahead (after the W stage of the group's previous chunk), because the
            // projection needs them at once
            if (!kProj) load_pq(c);
            // Both at the start of the chunk, where the group would otherwise idle until the running A of the other
            // group's chunk arrives.  (Done during the waits for this group's own products instead, they delayed the
            // reaction to those products by more than they saved.)
            PlaneFrags pf;   // one read of the plane fragments serves both tiles of the chunk
            if (kProj) load_plane_frags_tab(ptab, lane, pf);
            if (kWorkerK) {
                if (c >= 4 && !(ok = wait_bar_warp(cx, kKtFree + wg * 2 + (int)ph, (uint32_t)(((c >> 2) - 1) & 1), 108))) break;
                if (!(ok = wait_bar_warp(cx, kFull + wg, ph, 109))) break;
                write_kt(c, pf);
            }
            if (kProj) q_to_probs(c, pf);
            RACE_TRACE(wg, c, 0);

            // -- S2: W = pQ / (A + A_loc + eps) ----------------------------------------------------
            // (the plain product needs no running sum: W = pQ goes to the tensor cores as it is)
            float acar[16];
            if (!kRaw) {
            if (!(ok = wait_bar_warp(cx, kAcar + wg, ph, 102))) break;
            {
                const float* ac = reinterpret_cast<const float*>(cx.sm + oAcar) + wg * 64;
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    const float2 a2 = *reinterpret_cast<const float2*>(ac + 8 * x + 2 * q);
                    acar[2 * x] = a2.x; acar[2 * x + 1] = a2.y;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(kAcarFree + wg));
            // the warp that publishes the next running A overwrites the other group's buffer:
            // every warp of that group must have read the values of its previous chunk
            if (w == 3 && c >= 1 && !(ok = wait_bar_warp(cx, kAcarFree + (wg ^ 1), ((c - 1) >> 1) & 1, 107))) break;
            if (!(ok = wait_bar_warp(cx, kXReady + wg, ph, 103))) break;
            RACE_TRACE(wg, c, 5);
            tc_fence_after();
            tmem_ld64(lane_base + tmAG(wg), v);
            tc_fence_before();
            }
            if (kGlobal) den[0] = den[1] = 0.f;
#pragma unroll
            for (int x = 0; x < 8; ++x) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float2 w2;
                    if (kRaw) {
                        w2 = pqv[2 * x + h];
                        split2(w2.x, w2.y, ohi[2 * x + h], olo[2 * x + h]);
                        continue;
                    }
                    // packed fp32x2 arithmetic: (a0, a1) = running A + A_loc; W = pQ / (a + eps)
                    const float2 a2 = __fadd2_rn(make_float2(acar[2 * x], acar[2 * x + 1]),
                                                 make_float2(v[4 * x + 2 * h], v[4 * x + 2 * h + 1]));
                    if (kGlobal) {
                        w2 = pqv[2 * x + h];
                        den[h] = fmaf(w2.x, a2.x, fmaf(w2.y, a2.y, den[h]));
                    } else {
                        const float2 d2 = __fadd2_rn(a2, make_float2(eps, eps));
                        w2 = __fmul2_rn(pqv[2 * x + h], make_float2(__fdividef(1.f, d2.x), __fdividef(1.f, d2.y)));
                    }
                    split2(w2.x, w2.y, ohi[2 * x + h], olo[2 * x + h]);
                    if (h == 1 && w == 3 && (lane >> 2) == 7) {
                        // row 63: the running A after this chunk, for the other group
                        float* an = reinterpret_cast<float*>(cx.sm + oAcar) + (wg ^ 1) * 64;
                        *reinterpret_cast<float2*>(an + 8 * x + 2 * q) = a2;
                    }
                }
            }
            tmem_st_pairs(lane_base + tmWG(wg), ohi);
            tmem_st_pairs(lane_base + tmWG(wg) + 32, olo);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(cx.bar(kWReady + wg));
                if (!kRaw && w == 3) mbar_arrive(cx.bar(kAcar + (wg ^ 1)));
            }
            if (kMode == kModeRawX) load_pq_true(c);   // pqv (the operand of the W stage) is free: for the epilogue
            if (kProj && c + 2 < nch) load_pq(c + 2);
            if (kGlobal) {
                // a row's 64 buckets are spread over the four lanes of a quad, in a fixed order
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    den[h] += __shfl_xor_sync(0xffffffffu, den[h], 1);
                    den[h] += __shfl_xor_sync(0xffffffffu, den[h], 2);
                }
            }

            // -- S3: G -> causal mask -> operand tile (over W's buffer) ----------------------------
            RACE_TRACE(wg, c, 6);
            if (!(ok = wait_bar_warp(cx, kGReady + wg, ph, 104))) break;
            RACE_TRACE(wg, c, 7);
            tc_fence_after();
            tmem_ld64(lane_base + tmAG(wg), v);
            tc_fence_before();
#pragma unroll
            for (int x = 0; x < 8; ++x) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = rbase + 8 * h, col = 8 * x + 2 * q;
                    const float g0 = (kReverse ? col >= row : col <= row) ? v[4 * x + 2 * h] : 0.f;
                    const float g1 = (kReverse ? col + 1 >= row : col + 1 <= row) ? v[4 * x + 2 * h + 1] : 0.f;
                    split2(g0, g1, ohi[2 * x + h], olo[2 * x + h]);
                }
            }
            tmem_st_pairs(lane_base + tmWG(wg), ohi);
            tmem_st_pairs(lane_base + tmWG(wg) + 32, olo);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(kGtReady + wg));
            // -- S4: O -> global --------------------------------------------------------------------
            if (!(ok = wait_bar_warp(cx, kOReady + wg, ph, 105))) break;
            RACE_TRACE(wg, c, 3);
            if (kMode == kModeRawX) store_bwdx(c);
            else store_out(c);
            RACE_TRACE(wg, c, 4);
        }
    } else if (warp < 12) {
        // =========================== converter + carry warpgroup =================================
        // Per chunk: staged fp32 pK, V -> bf16 limb tiles of the chunk's worker group, then the
        // state left by the previous chunk: TMEM accumulator -> bf16 limb tile for the next W.B.
        const int w = warp & 3, q = lane & 3, rbase = 16 * w + (lane >> 2), wtid = tid & 127;
        const uint32_t lane_base = (uint32_t)(32 * w) << 16;
        float v[32];
        auto write_bt = [&](int buf) {
            uint8_t* bt_hi = cx.sm + oBt + buf * 2 * kOpTile;
            uint8_t* bt_lo = bt_hi + kOpTile;
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t hi, lo;
                    split2(v[4 * x + 2 * h], v[4 * x + 2 * h + 1], hi, lo);
                    const uint32_t off = op_off(rbase + 8 * h, 8 * x + 2 * q);
                    *reinterpret_cast<uint32_t*>(bt_hi + off) = hi;
                    *reinterpret_cast<uint32_t*>(bt_lo + off) = lo;
                }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(cx.bar(kBtReady + buf));
        };
        // carry-in: B -> TMEM accumulator and operand buffer 0; A -> the first chunk's running A
#pragma unroll
        for (int x = 0; x < 8; ++x)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float2 b2 = __ldcg(reinterpret_cast<const float2*>(
                    slice + (rbase + 8 * h) * D + 8 * x + 2 * q));
                v[4 * x + 2 * h] = b2.x; v[4 * x + 2 * h + 1] = b2.y;
            }
        {   // tril[t][j] = (j <= t), exact in bf16, as an A operand in tensor memory
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
        tmem_st64(lane_base + tmB, v);   // waits for both stores
        tc_fence_before();
        if (warp == 8) {
            float* ac = reinterpret_cast<float*>(cx.sm + oAcar);
            ac[lane] = __ldcg(slice + S * D + lane);
            ac[lane + 32] = __ldcg(slice + S * D + lane + 32);
        }
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(cx.bar(kBaccFree + 0));
            if (warp == 8) mbar_arrive(cx.bar(kAcar + 0));
        }
        write_bt(0);

        bool ok = true;
        for (int c = 0; c < nch && ok; ++c) {
            const int wg = c & 1;
            const uint32_t ph = (uint32_t)((c >> 1) & 1);
            const uint8_t* stage = cx.sm + oStage + wg * kStageBytes;
            const int kb = (int)ph;   // pK operand buffer of this chunk within its group
            uint8_t* kt_hi = cx.sm + oKt + (wg * 2 + kb) * 2 * kOpTile;
            uint8_t* vt_hi = cx.sm + oVt + wg * 2 * kOpTile;
            // pK buffer: last read by the products of chunk c - 4
            RACE_TRACE(2, c, 0);
            if (!kWorkerK && c >= 4 &&
                !(ok = wait_bar_warp(cx, kKtFree + wg * 2 + kb, (uint32_t)(((c >> 2) - 1) & 1), 203))) break;
            if (!(ok = wait_bar_warp(cx, kFull + wg, ph, 201))) break;
            RACE_TRACE(2, c, 1);
            if (!kWorkerK) {
                if (kProj) {
                    float unused[16];
                    PlaneFrags pf;
                    load_plane_frags_tab(ptab, lane, pf);
                    produce_tile<false>(stage, kt_hi, kt_hi + kOpTile, pf, w, lane,
                                        (int)min((int64_t)C, t_end - chunk_tok0(c)), unused);
                } else {
                    convert_tile(stage, kt_hi, kt_hi + kOpTile, wtid);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(cx.bar(kKvReady + wg));
            }
            RACE_TRACE(2, c, 2);
            if (c >= 1) {
                // state after chunk c - 1 -> operand buffer c & 1 (read by W.B of chunk c; last read
                // by W.B of chunk c - 2)
                if (c >= 2 && !(ok = wait_bar_warp(cx, kGReady + wg, ph ^ 1, 204))) break;
                if (!(ok = wait_bar_warp(cx, kBupdDone, (c - 1) & 1, 202))) break;
                tc_fence_after();
                tmem_ld64(lane_base + tmB, v);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(cx.bar(kBaccFree + wg));   // update of chunk c may start
                write_bt(wg);
            }
            RACE_TRACE(2, c, 3);
            // V tile of the group: last read by the G.V product of chunk c - 2
            if (c >= 2 && !(ok = wait_bar_warp(cx, kOReady + wg, ph ^ 1, 205))) break;
            RACE_TRACE(2, c, 4);
            convert_tile(stage + kTileF32, vt_hi, vt_hi + kOpTile, wtid);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(cx.bar(kVReady + wg)); mbar_arrive(cx.bar(kEmpty + wg)); }
            RACE_TRACE(2, c, 5);
        }
    } else if (warp == kProducerWarp) {
        // =========================== TMA producer ==============================================
        if (lane == 0) {
            int issued = 0;
            const uint64_t pol = l2_policy_evict_first();
            for (int c = 0; c < nch; ++c) {
                const int st = c & 1;
                if (c >= 2 && !wait_bar(cx, kEmpty + st, ((c >> 1) - 1) & 1, 301)) break;
                if (c == withhold_chunk) continue;   // self-test only
                const uint32_t dst = cx.sm_u32 + oStage + st * kStageBytes;
                const uint32_t bar = cx.bar(kFull + st);
                const int tok = (int)chunk_tok0(c);
                mbar_arrive_expect_tx(bar, kStageBytes);
                if (l2_last_use) {
                    tma_load_4d_hint(dst, map_k, bar, 0, tok, 0, (int)n, pol);
                    tma_load_5d_hint(dst + kTileF32, map_v, bar, 0, tok, 0, (int)(n % heads), (int)(n / heads), pol);
                } else {
                    if (kProj) tma_load_5d(dst, map_k, bar, 0, tok, 0, (int)(n % heads), (int)(n / heads));
                    else tma_load_4d(dst, map_k, bar, 0, tok, 0, (int)n);
                    tma_load_5d(dst + kTileF32, map_v, bar, 0, tok, 0, (int)(n % heads), (int)(n / heads));
                }
                issued = c + 1;
            }
            if (*cx.abort_flag) {
                // copies still in flight must land before the CTA may exit
                for (int c = max(0, issued - 2); c < issued; ++c) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(kFull + (c & 1)), (c >> 1) & 1) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
            }
        }
    } else {
        // =========================== MMA issuers (one warp per worker group) ====================
        // Everything the issuing thread feeds to tcgen05.mma is derived from warp-uniform values
        // (the shuffles tell the compiler so), which keeps descriptor arithmetic on the uniform
        // datapath.
        const int wg = __shfl_sync(0xffffffffu, warp, 0) - kMmaWarp;
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
        const uint32_t smb = __shfl_sync(0xffffffffu, cx.sm_u32, 0);
        constexpr uint32_t kLimb = kOpTile >> 4;   // hi -> lo limb tile, in lo-word units
        const uint32_t kt_k0 = lo_k(smb + oKt + wg * 4 * kOpTile);
        const uint32_t kt_mn0 = lo_mn(smb + oKt + wg * 4 * kOpTile);
        const uint32_t vt_mn = lo_mn(smb + oVt + wg * 2 * kOpTile);
        const uint32_t bt_mn = lo_mn(smb + oBt + wg * 2 * kOpTile);
        const uint32_t dB = tm, dAG = tm + 64 + wg * 128, dO = tm + 64 + wg * 128 + 64;
        const uint32_t a_hi = tm + 320 + wg * 64, a_lo = a_hi + 32;   // W / masked G limbs (A operand in TMEM)
        const uint32_t a_tril = tm + 448;
        if (elect_one()) {
            uint32_t ph = 0;
            bool ok = true;
            for (int c = wg; c < nch && ok; c += 2, ph ^= 1) {
                const uint32_t kt_k = kt_k0 + ph * 2 * kLimb, kt_mn = kt_mn0 + ph * 2 * kLimb;   // buffer (c >> 1) & 1
                // A_loc = tril . pK : A = tril (tensor memory), B = pK [token][s] (N-major)
                if (!(ok = wait_bar(cx, kKvReady + wg, ph, 401))) break;
                tc_fence_after();
                RACE_TRACE(4, c, 0);
                if (!kRaw) {
                    mma_k64_ta<true, kHiMN, 128>(dAG, a_tril, kt_mn, kIdescBase | kBmn);
                    mma_k64_ta<false, kHiMN, 128>(dAG, a_tril, kt_mn + kLimb, kIdescBase | kBmn);
                    mma_commit(cx.bar(kXReady + wg));
                }
                RACE_TRACE(4, c, 1);
                // B += pK^T . V, in chunk order: the accumulator is free once the state after
                // chunk c - 1 has been read out
                if (!(ok = wait_bar(cx, kVReady + wg, ph, 407))) break;
                if (!(ok = wait_bar(cx, kBaccFree + wg, ph, 403))) break;
                tc_fence_after();
                RACE_TRACE(4, c, 2);
                mma_k64<false, kHiMN, 128, kHiMN, 128>(dB, kt_mn, vt_mn, kIdescBase | kAmn | kBmn);
                mma_k64<false, kHiMN, 128, kHiMN, 128>(dB, kt_mn, vt_mn + kLimb, kIdescBase | kAmn | kBmn);
                mma_k64<false, kHiMN, 128, kHiMN, 128>(dB, kt_mn + kLimb, vt_mn, kIdescBase | kAmn | kBmn);
                mma_commit(cx.bar(kBupdDone));
                RACE_TRACE(4, c, 3);
                // O = W . B and G = W . pK^T
                if (!(ok = wait_bar(cx, kWReady + wg, ph, 404))) break;
                if (!(ok = wait_bar(cx, kBtReady + wg, ph, 405))) break;
                tc_fence_after();
                RACE_TRACE(4, c, 4);
                mma_k64_ta<true, kHiMN, 128>(dO, a_hi, bt_mn, kIdescBase | kBmn);
                mma_k64_ta<false, kHiMN, 128>(dO, a_hi, bt_mn + kLimb, kIdescBase | kBmn);
                mma_k64_ta<false, kHiMN, 128>(dO, a_lo, bt_mn, kIdescBase | kBmn);
                mma_k64_ta<true, kHiK, 16>(dAG, a_hi, kt_k, kIdescBase);
                mma_k64_ta<false, kHiK, 16>(dAG, a_hi, kt_k + kLimb, kIdescBase);
                mma_k64_ta<false, kHiK, 16>(dAG, a_lo, kt_k, kIdescBase);
                mma_commit(cx.bar(kGReady + wg));
                mma_commit(cx.bar(kKtFree + wg * 2 + (int)ph));   // no later product reads this pK buffer
                RACE_TRACE(4, c, 5);
                // O += G . V : A = masked G (tensor memory), B = V [token][c] (N-major)
                if (!(ok = wait_bar(cx, kGtReady + wg, ph, 406))) break;
                tc_fence_after();
                RACE_TRACE(4, c, 6);
                mma_k64_ta<false, kHiMN, 128>(dO, a_hi, vt_mn, kIdescBase | kBmn);
                mma_k64_ta<false, kHiMN, 128>(dO, a_hi, vt_mn + kLimb, kIdescBase | kBmn);
                mma_k64_ta<false, kHiMN, 128>(dO, a_lo, vt_mn, kIdescBase | kBmn);
                if (kMode == kModeRawX) {
                    // running sum of the chunk's V operand (the pK of the backward) into the accumulator G has left:
                    // the worker warps have read G (their arrival on kGtReady), and the next product into it, G of
                    // the group's next chunk, is issued only after they have read this one
                    mma_k64_ta<true, kHiMN, 128>(dAG, a_tril, vt_mn, kIdescBase | kBmn);
                    mma_k64_ta<false, kHiMN, 128>(dAG, a_tril, vt_mn + kLimb, kIdescBase | kBmn);
                }
                mma_commit(cx.bar(kOReady + wg));
                RACE_TRACE(4, c, 7);
            }
            // everything this thread issued has to retire before TMEM is freed
            mma_commit(cx.bar(kDrain + wg));
            const long long t0 = clock64();
            while (!mbar_try_wait(cx.bar(kDrain + wg), 0) && clock64() - t0 < cx.limit) {}
        }
    }
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_u32, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_u32), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t tmem, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(cols) : "memory");
}

// The output pass as a kernel of its own (second half of a forward whose per-tile prefixes are
// already in the workspace): one CTA per (tile, stream).  wait_cycles > 0 replaces the default limit
// of every wait; withhold_chunk >= 0 makes the producer of CTA (0, 0) skip that chunk's load.
// kProj: pq is Q, map_k covers K and `planes` [16][64] are the hyperplanes (out_phase).
template <int kMode, bool kReverse, bool kProj>
__global__ void __launch_bounds__(kThreads, 1)
causal_out_tc(const float* __restrict__ pq, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, float* __restrict__ out,
              const float* __restrict__ ws, int64_t T, int tile_tokens, float eps, int heads, int* status,
              long long wait_cycles, int withhold_chunk, const float* __restrict__ planes, const BwdX bwdx) {
    extern __shared__ uint8_t smem_raw[];
    Ctx cx;
    cx.sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    cx.sm_u32 = smem_u32(cx.sm);
    cx.bars = oBars;
    cx.abort_flag = reinterpret_cast<volatile int*>(cx.sm + oMisc + 4);
    cx.status = status;
    if (wait_cycles > 0) cx.limit = wait_cycles;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(cx.sm + oMisc);
    const int tid = threadIdx.x, warp = tid >> 5;
    const int64_t tiles = gridDim.x, tile = blockIdx.x, n = blockIdx.y;
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(T, t_begin + (int64_t)tile_tokens);
    const float* slice = ws + (n * tiles + tile) * (int64_t)(S * (D + 1));
    // The worker groups write their own pK tile only where forming the probabilities makes that tile expensive: with
    // probabilities in, leaving it to the converter group measured 3 % faster.
    constexpr bool kWorkerK = kProj;
    if (tid == 0) {
        *cx.abort_flag = 0;
        out_phase_init_bars(cx, false, kWorkerK ? 8u : 4u);
    }
    uint32_t* ptab = reinterpret_cast<uint32_t*>(cx.sm + oPlaneTab);
    if (kProj) build_plane_tab(planes, ptab, tid, kThreads);
    if (warp == kMmaWarp) tmem_alloc(cx.sm_u32 + oMisc, kTmemCols);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    out_phase<kMode, kReverse, kProj, kWorkerK>(cx, tmem, pq, &map_k, &map_v, out, slice, T, t_begin, t_end, n, eps,
                                                heads, (tile == 0 && n == 0) ? withhold_chunk : -1, false, ptab, &bwdx);
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}


#ifdef RACE_FUSED_PROF
// per-CTA cycle counters of the single-pass kernel (profiling builds only): totals phase, wait for
// the look-back flags, prefix sum, output phase, tiles taken
__device__ long long g_fused_prof[160][16];
#define RACE_PROF_ADD(slot, t_from)                                                   \
    do { if (tid == 0) { const long long now_ = clock64(); g_fused_prof[blockIdx.x][slot] += now_ - (t_from); (t_from) = now_; } } while (0)
#else
#define RACE_PROF_ADD(slot, t_from) do {} while (0)
#endif

#ifdef RACE_FUSED_PROF
#define RACE_PROF_T(var) long long var = clock64()
#define RACE_PROF_LANE(slot, t_from) do { const long long now_ = clock64(); g_fused_prof[blockIdx.x][slot] += now_ - (t_from); (t_from) = now_; } while (0)
#else
#define RACE_PROF_T(var) do {} while (0)
#define RACE_PROF_LANE(slot, t_from) do {} while (0)
#endif

// ------------------------------------------------------------------------------------------------
// Tile totals on the tensor cores: B_tile = sum_t pK^T V (tcgen05.mma into one TMEM accumulator),
// A_tile = sum_t pK (fp32 adds while the keys are split into limbs).  A streaming kernel: two
// converter warpgroups take alternate chunks from a four-stage TMA ring; nothing but the
// accumulator is carried from chunk to chunk.
// ------------------------------------------------------------------------------------------------
// kT1Groups converter warpgroups take the chunks c = g (mod kT1Groups), each with its own operand tiles, from a
// TMA ring of kT1Stages stages.  The stage count is a multiple of the group count so that a stage always goes
// to the same group: a group that saw only every other phase of a stage's barrier could not tell a refilled
// stage from the one it read two fills ago by the parity (which made a 3-stage ring with two groups run ahead
// of the copies and overflow its barriers' arrival counts under load).
constexpr int kT1StageBytes = 2 * kTileF32;            // pK | V
template <int kGroupsT, int kStagesT>
struct TotalsLayout {
    static constexpr int kGroups = kGroupsT, kStages = kStagesT;
    static_assert(kStages % kGroups == 0, "a stage must stay with one converter group");
    static constexpr int kProducerWarp = 4 * kGroups, kMmaWarp = 4 * kGroups + 1;
    static constexpr int kThreads = (4 * kGroups + 2) * 32;    // converters, TMA producer, MMA issuer
    static constexpr int oStage = 0;
    static constexpr int oKt = oStage + kStages * kT1StageBytes;   // [group][hi | lo]
    static constexpr int oVt = oKt + kGroups * 2 * kOpTile;        // [group][hi | lo]
    static constexpr int oRed = oVt + kGroups * 2 * kOpTile;       // [converter warps][64] fp32 column-sum partials
    static constexpr int oBars = oRed + 4 * kGroups * 64 * 4;
    static constexpr int oMisc = oBars + 16 * 8;
    static constexpr int oPlaneTab = oMisc + 16;                   // plane fragments (kProj)
    static constexpr int kSmemBytes = oPlaneTab + kPlaneTabWords * 4 + 1024;
    static constexpr int kFull = 0, kEmpty = kStages, kKvReady = 2 * kStages, kKvFree = 2 * kStages + kGroups,
                         kDone = 2 * kStages + 2 * kGroups, kNumBars = kDone + 1;
    static_assert(kNumBars <= 16, "barrier array of the totals phase");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory of the totals phase");
};
// Two groups and four stages: with probabilities in, a streaming, DRAM-bound kernel, which wants many bytes in
// flight; forming the probabilities, the converter groups are the bound, but a third group (with three stages, which
// is what then fits) measured the same.
using T1 = TotalsLayout<2, 4>;
using T1P = TotalsLayout<2, 4>;
static_assert(T1::kThreads <= kThreads, "the single-pass kernel runs the totals phase with its own warps");
// names of the default layout, as the single-pass kernel uses them
constexpr int o1Misc = T1::oMisc, o1Bars = T1::oBars;

// like convert_tile, and adds each thread's 8 values per item into asum[item][8]
__device__ __forceinline__ void convert_tile_sum(const uint8_t* __restrict__ stage, uint8_t* __restrict__ hi,
                                                 uint8_t* __restrict__ lo, int tid, float (&asum)[4][8]) {
    float4 av[4], bv[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 128 + tid;
        const int j = idx >> 6, r = idx & 63;
        const uint8_t* src = stage + (j >> 2) * 8192 + r * 128;
        const int jj = j & 3;
        av[it] = *reinterpret_cast<const float4*>(src + (((2 * jj) ^ (r & 7)) << 4));
        bv[it] = *reinterpret_cast<const float4*>(src + (((2 * jj + 1) ^ (r & 7)) << 4));
    }
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 128 + tid;
        const int j = idx >> 6, r = idx & 63;
        const float4 a = av[it], b = bv[it];
        asum[it][0] += a.x; asum[it][1] += a.y; asum[it][2] += a.z; asum[it][3] += a.w;
        asum[it][4] += b.x; asum[it][5] += b.y; asum[it][6] += b.z; asum[it][7] += b.w;
        uint4 h, l;
        split2(a.x, a.y, h.x, l.x);
        split2(a.z, a.w, h.y, l.y);
        split2(b.x, b.y, h.z, l.z);
        split2(b.z, b.w, h.w, l.w);
        const uint32_t off = (uint32_t)((((r >> 3) * 8 + j) << 7) + ((r & 7) << 4));
        *reinterpret_cast<uint4*>(hi + off) = h;
        *reinterpret_cast<uint4*>(lo + off) = l;
    }
}

template <typename TL = T1>
__device__ __forceinline__ void totals_phase_reinit_bars_warp(const Ctx& cx, int lane, bool again) {
    if (lane < TL::kNumBars) {
        if (again) mbar_inval(cx.bar(lane));
        mbar_init(cx.bar(lane), (lane >= TL::kEmpty && lane < TL::kKvFree) ? 4u : 1u);   // kEmpty, kKvReady: 4 warps
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
template <typename TL = T1>
__device__ __forceinline__ void totals_phase_init_bars(const Ctx& cx, bool again) {
    if (again)
        for (int i = 0; i < TL::kNumBars; ++i) mbar_inval(cx.bar(i));
    {
        for (int i = 0; i < TL::kStages; ++i) {
            mbar_init(cx.bar(TL::kFull + i), 1);
            mbar_init(cx.bar(TL::kEmpty + i), 4);
        }
        for (int i = 0; i < TL::kGroups; ++i) {
            mbar_init(cx.bar(TL::kKvReady + i), 4);
            mbar_init(cx.bar(TL::kKvFree + i), 1);
        }
        mbar_init(cx.bar(TL::kDone), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
}

// Totals phase of one (stream n, tokens [t_begin, t_end)) tile into `slice` (state layout).  Called
// by at least TL::kThreads / 32 warps (the first 4 * TL::kGroups convert, the next issues TMA, the next the products;
// further warps only take part in the block-wide barriers) with barriers initialised and 64 TMEM columns at `tmem`.
// l2_keep: pK and V of the tile are read again soon (single-pass kernel): load them with the evict-last priority.
// kProj: map_k covers K in the layout of V and the converter groups form pK themselves (out_phase); ptab = the
// plane fragments in shared memory.
template <bool kProj = false, typename TL = T1>
__device__ __forceinline__ void totals_phase(const Ctx& cx, const uint32_t tmem, const CUtensorMap* map_k,
                                             const CUtensorMap* map_v, float* __restrict__ slice,
                                             const int64_t t_begin, const int64_t t_end, const int64_t n, int heads,
                                             const bool l2_keep = false, const uint32_t* ptab = nullptr) {
    constexpr int kT1Groups = TL::kGroups, kT1Stages = TL::kStages, kT1ProducerWarp = TL::kProducerWarp,
                  kT1MmaWarp = TL::kMmaWarp, o1Stage = TL::oStage, o1Kt = TL::oKt, o1Vt = TL::oVt, o1Red = TL::oRed,
                  k1Full = TL::kFull, k1Empty = TL::kEmpty, k1KvReady = TL::kKvReady, k1KvFree = TL::kKvFree,
                  k1Done = TL::kDone;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nch = (int)((t_end - t_begin + C - 1) / C);

    if (warp < 4 * kT1Groups) {
        const int wg = warp >> 2, wtid = tid & 127;
        uint8_t* kt_hi = cx.sm + o1Kt + wg * 2 * kOpTile;
        uint8_t* vt_hi = cx.sm + o1Vt + wg * 2 * kOpTile;
        float asum[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) asum[i][e] = 0.f;
        float psum[16];   // kProj: the lane's table (columns 16 (lane % 4) + i), rows lane / 4 and lane / 4 + 8
#pragma unroll
        for (int i = 0; i < 16; ++i) psum[i] = 0.f;
        PlaneFrags pf;    // kProj: the plane fragments stay in registers for the whole tile
        if (kProj) load_plane_frags_tab(ptab, lane, pf);
        bool ok = true;
        int i = 0;   // the group's i-th chunk
        RACE_PROF_T(tq);
        for (int c = wg; c < nch && ok; c += kT1Groups, ++i) {
            const int st = c % kT1Stages;
            const uint8_t* stage = cx.sm + o1Stage + st * kT1StageBytes;
            if (!(ok = wait_bar_warp(cx, k1Full + st, (uint32_t)((c / kT1Stages) & 1), 111))) break;
            if (tid == 0) RACE_PROF_LANE(8, tq);
            if (i >= 1 && !(ok = wait_bar_warp(cx, k1KvFree + wg, (uint32_t)((i - 1) & 1), 112))) break;
            if (tid == 0) RACE_PROF_LANE(9, tq);
            if (kProj)
                produce_tile<true>(stage, kt_hi, kt_hi + kOpTile, pf, warp & 3, lane,
                                   (int)min((int64_t)C, t_end - (t_begin + (int64_t)c * C)), psum);
            else
                convert_tile_sum(stage, kt_hi, kt_hi + kOpTile, wtid, asum);
            convert_tile(stage + kTileF32, vt_hi, vt_hi + kOpTile, wtid);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(cx.bar(k1KvReady + wg)); mbar_arrive(cx.bar(k1Empty + st)); }
            if (tid == 0) RACE_PROF_LANE(10, tq);
        }
        float* red = reinterpret_cast<float*>(cx.sm + o1Red) + warp * 64;
        if (kProj) {
            // column sums: the eight lanes with the same lane % 4 hold different token rows of one table
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float x = psum[i];
#pragma unroll
                for (int off = 16; off >= 4; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
                if (lane < 4) red[16 * lane + i] = x;
            }
        } else {
            // column sums: lanes of a warp hold different token rows of the same 8 columns
#pragma unroll
            for (int it = 0; it < 4; ++it)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float x = asum[it][e];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
                    if (lane == 0) red[it * 8 + e] = x;
                }
        }
    } else if (warp == kT1ProducerWarp) {
        if (lane == 0) {
            int issued = 0;
            const uint64_t pol = l2_policy_evict_last();
            RACE_PROF_T(tq);
            for (int c = 0; c < nch; ++c) {
                const int st = c % kT1Stages, i = c / kT1Stages;
                if (i >= 1 && !wait_bar(cx, k1Empty + st, (uint32_t)((i - 1) & 1), 311)) break;
                RACE_PROF_LANE(11, tq);
                const uint32_t dst = cx.sm_u32 + o1Stage + st * kT1StageBytes;
                const uint32_t bar = cx.bar(k1Full + st);
                const int tok = (int)(t_begin + (int64_t)c * C);
                mbar_arrive_expect_tx(bar, kT1StageBytes);
                if (l2_keep) {
                    tma_load_4d_hint(dst, map_k, bar, 0, tok, 0, (int)n, pol);
                    tma_load_5d_hint(dst + kTileF32, map_v, bar, 0, tok, 0, (int)(n % heads), (int)(n / heads), pol);
                } else {
                    if (kProj) tma_load_5d(dst, map_k, bar, 0, tok, 0, (int)(n % heads), (int)(n / heads));
                    else tma_load_4d(dst, map_k, bar, 0, tok, 0, (int)n);
                    tma_load_5d(dst + kTileF32, map_v, bar, 0, tok, 0, (int)(n % heads), (int)(n / heads));
                }
                issued = c + 1;
                RACE_PROF_LANE(12, tq);
            }
            if (*cx.abort_flag) {
                for (int c = max(0, issued - kT1Stages); c < issued; ++c) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(cx.bar(k1Full + c % kT1Stages), (c / kT1Stages) & 1) &&
                           clock64() - t0 < (1ll << 24)) {}
                }
            }
        }
    } else if (warp == kT1MmaWarp) {
        // every operand of the issuing thread derives from warp-uniform values (cheap descriptor arithmetic)
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
        const uint32_t smb = __shfl_sync(0xffffffffu, cx.sm_u32, 0);
        constexpr uint32_t kLimb = kOpTile >> 4;
        constexpr uint32_t kId = kIdescBase | kAmn | kBmn;
        if (elect_one()) {
            bool ok = true;
            RACE_PROF_T(tq);
            for (int c = 0; c < nch && ok; ++c) {
                const int wg = c % kT1Groups, i = c / kT1Groups;
                if (!(ok = wait_bar(cx, k1KvReady + wg, (uint32_t)(i & 1), 411))) break;
                RACE_PROF_LANE(13, tq);
                tc_fence_after();
                const uint32_t kt = lo_mn(smb + o1Kt + wg * 2 * kOpTile);
                const uint32_t vt = lo_mn(smb + o1Vt + wg * 2 * kOpTile);
                // pK_hi.V_hi + pK_hi.V_lo + pK_lo.V_hi; the first product of the tile starts the accumulator
                if (c == 0) mma_k64<true, kHiMN, 128, kHiMN, 128>(tm, kt, vt, kId);
                else mma_k64<false, kHiMN, 128, kHiMN, 128>(tm, kt, vt, kId);
                mma_k64<false, kHiMN, 128, kHiMN, 128>(tm, kt, vt + kLimb, kId);
                mma_k64<false, kHiMN, 128, kHiMN, 128>(tm, kt + kLimb, vt, kId);
                mma_commit(cx.bar(k1KvFree + wg));
                RACE_PROF_LANE(14, tq);
            }
            mma_commit(cx.bar(k1Done));
        }
    }
    __syncthreads();   // column-sum partials are in shared memory
    if (warp < 4) {
        const bool ok = wait_bar_warp(cx, k1Done, 0, 113);
        if (ok) {
            tc_fence_after();
            float v[32];
            tmem_ld64(((uint32_t)(32 * warp) << 16) + tmem, v);
            tc_fence_before();
            const int q = lane & 3, rbase = 16 * warp + (lane >> 2);
#pragma unroll
            for (int x = 0; x < 8; ++x)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    *reinterpret_cast<float2*>(slice + (rbase + 8 * h) * D + 8 * x + 2 * q) =
                        make_float2(v[4 * x + 2 * h], v[4 * x + 2 * h + 1]);
            if (tid < 64) {
                const float* red = reinterpret_cast<const float*>(cx.sm + o1Red);
                float a = 0.f;
                if (kProj) {
                    // every converter warp holds a partial of every column; added in warp order
#pragma unroll
                    for (int wv = 0; wv < 4 * kT1Groups; ++wv) a += red[wv * 64 + tid];
                } else {
                    // column s = 8 j + e with j = 2 item + (warp_in_group >> 1); partials from both
                    // groups and both row halves, added in a fixed order
                    const int j = tid >> 3, e = tid & 7, it = j >> 1, wh = (j & 1) * 2;
#pragma unroll
                    for (int g = 0; g < kT1Groups; ++g)
#pragma unroll
                        for (int half = 0; half < 2; ++half)
                            a += red[(g * 4 + wh + half) * 64 + it * 8 + e];
                }
                slice[S * D + tid] = a;
            }
        }
    }
}

template <bool kProj> using TotalsLayoutOf = std::conditional_t<kProj, T1P, T1>;
template <bool kProj>
__global__ void __launch_bounds__(TotalsLayoutOf<kProj>::kThreads, 1)
tile_totals_tc(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
               float* __restrict__ ws, int64_t T, int tile_tokens, int heads, int* status,
               const float* __restrict__ planes) {
    extern __shared__ uint8_t smem_raw[];
    Ctx cx;
    cx.sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    cx.sm_u32 = smem_u32(cx.sm);
    using TL = TotalsLayoutOf<kProj>;
    cx.bars = TL::oBars;
    cx.abort_flag = reinterpret_cast<volatile int*>(cx.sm + TL::oMisc + 4);
    cx.status = status;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(cx.sm + TL::oMisc);
    const int tid = threadIdx.x, warp = tid >> 5;
    const int64_t tiles = gridDim.x, tile = blockIdx.x, n = blockIdx.y;
    const int64_t t_begin = tile * tile_tokens;
    const int64_t t_end = min(T, t_begin + (int64_t)tile_tokens);
    float* slice = ws + (n * tiles + tile) * (int64_t)(S * (D + 1));
    if (tid == 0) {
        *cx.abort_flag = 0;
        totals_phase_init_bars<TL>(cx, false);
    }
    uint32_t* ptab = reinterpret_cast<uint32_t*>(cx.sm + TL::oPlaneTab);
    if (kProj) build_plane_tab(planes, ptab, tid, TL::kThreads);
    if (warp == TL::kMmaWarp) tmem_alloc(cx.sm_u32 + TL::oMisc, 64u);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    totals_phase<kProj, TL>(cx, tmem, &map_k, &map_v, slice, t_begin, t_end, n, heads, false, ptab);
    tc_fence_before();
    __syncthreads();
    if (warp == TL::kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, 64u);
    }
}


// ------------------------------------------------------------------------------------------------
// Single-pass forward: one persistent kernel, tiles taken from an atomic ticket.  For its tile a CTA
//   1. reduces the tile to its totals (totals_phase) and publishes them (flag 1);
//   2. looks back over the tiles before it in the stream -- all of them hold smaller tickets, so
//      their CTAs are running or done -- for the nearest one whose inclusive prefix is published
//      (flag 2), adds the totals of the tiles after that one IN TILE ORDER (so the sum is the same
//      left-to-right fp32 sum whichever tile the look-back stopped at, and equal to tile_scan's),
//      publishes its own inclusive prefix (flag 2);
//   3. runs the output phase with that carry; pK and V of the tile are re-read from L2 (the tiles in
//      flight on all SMs are 148 x 1024 tokens x 512 B = 74 MB).
// CTAs drift apart, so the DRAM-bound step 1 of some overlaps the latency-bound step 3 of others.
// Every spin is bounded (cx.limit): a flag that never comes raises the status word and the CTA
// stops taking tickets; nothing is in flight at that point.
// ------------------------------------------------------------------------------------------------
constexpr int kSF = S * (D + 1);                  // floats of one state
constexpr int kFusedMaxGrid = 160;                // per-CTA carry slots in the workspace
constexpr int kLookbackDepth = 24;                // tiles whose totals a look-back adds at most
constexpr int oFusedMisc = (oMisc > o1Misc ? oMisc : o1Misc) + 16;   // tmem base, abort, ticket, j
constexpr int kFusedSmemBytes = oFusedMisc + 32 + 1024;

struct FusedArgs {
    const float* pq;
    float* out;
    float* agg;                   // [N][tiles][kSF] totals of every tile
    float* incl;                  // [N][tiles][kSF] state after every tile
    float* cta_carry;             // [grid][kSF]     state before the tile a CTA is working on
    int* flags;                   // [N * tiles]     0 nothing, 1 totals, 2 inclusive prefix
    unsigned long long* ticket;
    const float* carry_in;        // nullable [N][kSF]
    float* state_out;             // nullable [N][kSF]
    int64_t T, N, tiles;
    int tile_tokens;
    float eps;
    int heads;
    int* status;
    long long wait_cycles;
    int withhold_chunk;
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <bool kGlobal>
__global__ void __launch_bounds__(kThreads, 1)
causal_fused_tc(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                const __grid_constant__ FusedArgs a) {
    extern __shared__ uint8_t smem_raw[];
    Ctx cxA, cxB;   // the two phases keep their barriers at their own offsets
    cxA.sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    cxA.sm_u32 = smem_u32(cxA.sm);
    cxA.bars = o1Bars;
    cxA.abort_flag = reinterpret_cast<volatile int*>(cxA.sm + oFusedMisc + 4);
    cxA.status = a.status;
    if (a.wait_cycles > 0) cxA.limit = a.wait_cycles;
    cxB = cxA;
    cxB.bars = oBars;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(cxA.sm + oFusedMisc);
    volatile unsigned long long* ticket_slot = reinterpret_cast<volatile unsigned long long*>(cxA.sm + oFusedMisc + 8);
    volatile int* j_slot = reinterpret_cast<volatile int*>(cxA.sm + oFusedMisc + 16);
    const int tid = threadIdx.x, warp = tid >> 5;
    const unsigned long long total = (unsigned long long)a.N * (unsigned long long)a.tiles;

    if (tid == 0) {
        *cxA.abort_flag = 0;
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    if (warp == kMmaWarp) tmem_alloc(cxA.sm_u32 + oFusedMisc, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;


    // tiles are drawn one ahead (the ticket of the next tile is taken before the output phase of the current one),
    // which keeps the round trip of the atomic out of the path between two tiles
    if (tid == 0) *ticket_slot = atomicAdd(a.ticket, 1ull);
    __syncthreads();
    unsigned long long t_next = *ticket_slot;
    bool first = true;
    for (;;) {
        const unsigned long long t = t_next;
        if (t >= total) break;
        const int64_t n = (int64_t)(t % (unsigned long long)a.N), tile = (int64_t)(t / (unsigned long long)a.N);
        const int64_t t_begin = tile * a.tile_tokens;
        const int64_t t_end = min(a.T, t_begin + (int64_t)a.tile_tokens);
        float* agg_n = a.agg + n * a.tiles * kSF;
        float* incl_n = a.incl + n * a.tiles * kSF;
        int* flags_n = a.flags + n * a.tiles;

        // ---- 1. totals of the tile ----------------------------------------------------------------
        long long tp = clock64();
        (void)tp;
        if (warp == 0) totals_phase_reinit_bars_warp(cxA, tid, !first);
        __syncthreads();
        totals_phase(cxA, tmem, &map_k, &map_v, agg_n + tile * kSF, t_begin, t_end, n, a.heads, /*l2_keep=*/true);
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        if (*cxA.abort_flag) break;
        // the release store is cumulative over the block's writes that the barrier ordered before it
        if (tid == 0) st_release_gpu(flags_n + tile, 1);
        RACE_PROF_ADD(0, tp);

        // ---- 2. look-back: carry of the tile, inclusive prefix published -----------------------------
        if (tid == 0) {
            int j = -1;                       // -1: the sum starts from carry_in
            if (tile > 0) {
                int64_t m = tile - 1;
                int depth = 0;
                const long long t0 = clock64();
                for (;;) {
                    const int f = ld_acquire_gpu(flags_n + m);
                    if (f == 2) { j = (int)m; break; }
                    if (f == 1 && depth < kLookbackDepth) {
                        if (m == 0) break;    // totals of every earlier tile are there
                        --m; ++depth;
                        continue;
                    }
                    if (clock64() - t0 > cxA.limit) {
                        *cxA.abort_flag = 1;
                        if (a.status) atomicCAS(a.status, 0, 501);
                        break;
                    }
                    __nanosleep(64);
                }
            }
            *j_slot = j;
        }
        __syncthreads();
        RACE_PROF_ADD(1, tp);
        if (*cxA.abort_flag) break;
        {
            const int j = *j_slot;
            float* mine = a.cta_carry + (int64_t)blockIdx.x * kSF;
            constexpr int kPer = (kSF + kThreads - 1) / kThreads;
            float x[kPer], own[kPer];
#pragma unroll
            for (int k = 0; k < kPer; ++k) {
                const int e = tid + k * kThreads;
                own[k] = e < kSF ? __ldcg(agg_n + tile * kSF + e) : 0.f;
            }
#pragma unroll
            for (int k = 0; k < kPer; ++k) {
                const int e = tid + k * kThreads;
                x[k] = 0.f;
                if (e < kSF) {
                    if (j >= 0) x[k] = __ldcg(incl_n + (int64_t)j * kSF + e);
                    else if (a.carry_in) x[k] = a.carry_in[n * kSF + e];
                }
            }
            for (int64_t m = j + 1; m < tile; ++m) {
                float y[kPer];
#pragma unroll
                for (int k = 0; k < kPer; ++k) {
                    const int e = tid + k * kThreads;
                    y[k] = e < kSF ? __ldcg(agg_n + m * kSF + e) : 0.f;
                }
#pragma unroll
                for (int k = 0; k < kPer; ++k) x[k] += y[k];
            }
            const bool last = tile == a.tiles - 1;
#pragma unroll
            for (int k = 0; k < kPer; ++k) {
                const int e = tid + k * kThreads;
                if (e < kSF) {
                    mine[e] = x[k];
                    const float inc = x[k] + own[k];
                    incl_n[tile * kSF + e] = inc;
                    if (last && a.state_out) a.state_out[n * kSF + e] = inc;
                }
            }
        }
        if (warp == 1) out_phase_reinit_bars_warp(cxB, tid & 31, !first);
        if (tid == 0) *ticket_slot = atomicAdd(a.ticket, 1ull);
        fence_proxy_async();
        __syncthreads();
        if (tid == 0) st_release_gpu(flags_n + tile, 2);
        t_next = *ticket_slot;
        RACE_PROF_ADD(2, tp);
#ifdef RACE_FUSED_PROF
        if (tid == 0) { g_fused_prof[blockIdx.x][4] += 1; g_fused_prof[blockIdx.x][5] += tile - 1 - *j_slot; }
#endif

        // ---- 3. outputs of the tile ---------------------------------------------------------------
        out_phase<kGlobal ? kModeGlobal : kModeBucket>(cxB, tmem, a.pq, &map_k, &map_v, a.out, a.cta_carry + (int64_t)blockIdx.x * kSF, a.T,
                           t_begin, t_end, n, a.eps, a.heads, (tile == 0 && n == 0) ? a.withhold_chunk : -1,
                           /*l2_last_use=*/true);
        first = false;
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();                      // nobody still uses this tile's shared memory or tensor memory
        tc_fence_after();
        RACE_PROF_ADD(3, tp);
        // a CTA that gave up a wait stops here (the tile it drew ahead stays undone: the tiles after it in that
        // stream run into their own limits)
        if (*cxA.abort_flag) break;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    int dev_probe = 0;
    cudaGetDevice(&dev_probe);  // make sure the runtime (and with it the driver) is initialised
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) !=
            cudaSuccess || q != cudaDriverEntryPointSuccess)
        p = nullptr;
    if (!p) {
        cudaGetLastError();
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
    }
    if (!p) cudaGetLastError();
    fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
    return fn;
}

// V in the layout [N/heads, T, heads, width] (heads = 1: [N, T, width]) viewed as (32 values, T tokens,
// width/32 column blocks, heads, N/heads); one box = 32 values x 64 tokens x both column blocks (128-byte rows,
// 128B swizzle; the box lands as two consecutive 8 KB tiles, one per column block); tokens past T read as zero
bool make_map_heads(CUtensorMap* map, const void* base, int64_t N, int64_t T, int width, int heads) {
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[5] = {32, (cuuint64_t)T, (cuuint64_t)(width / 32), (cuuint64_t)heads, (cuuint64_t)(N / heads)};
    cuuint64_t strides[4] = {(cuuint64_t)heads * width * 4, 128, (cuuint64_t)width * 4,
                             (cuuint64_t)T * heads * width * 4};
    cuuint32_t box[5] = {32, (cuuint32_t)C, (cuuint32_t)(width / 32), 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [N][T][width] fp32 viewed as (32 values, T tokens, width/32 column blocks, N streams); boxes as above
bool make_map(CUtensorMap* map, const void* base, int64_t N, int64_t T, int width) {
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {32, (cuuint64_t)T, (cuuint64_t)(width / 32), (cuuint64_t)N};
    cuuint64_t strides[3] = {(cuuint64_t)width * 4, 128, (cuuint64_t)T * width * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)C, (cuuint32_t)(width / 32), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool tensor_supported(const Dims& dm, int dtype) {
    // the shape test alone decides: a missing driver entry point surfaces as an error at launch
    if (dtype == RACE_DTYPE_BF16) return tensor_bf16_supported(dm);
    return dtype == RACE_DTYPE_F32 && dm.S == S && dm.D == D && dm.N >= 0 && dm.N <= 65535 &&
           dm.T < (1ll << 31);
}

int tensor_chunk_tokens() { return C; }

int tensor_single_pass_tile_tokens(const Dims& dm, int sm_count) {
    // The persistent kernel hands tiles to the SMs as they become free and reads pK and V of a tile twice:
    // 1024 tokens keep the tiles in flight on all SMs (sm_count x 512 KB) inside the L2.  Short inputs get
    // shorter tiles, about one per SM.
    const int64_t sms = sm_count > 0 ? sm_count : 148;
    const int64_t per_sm = (dm.N * dm.T + sms - 1) / sms;
    const int64_t tile = (per_sm + C - 1) / C * C;
    return (int)(tile < C ? C : (tile > 1024 ? 1024 : tile));
}

int tensor_default_tile_tokens(const Dims& dm, int, int sm_count) {
    // One CTA per SM (and per bucket group) at a time: the CTAs run in waves of sm_count, so the tile
    // length (a multiple of the chunk, at most 2048 tokens) is chosen to fill the last wave:
    // cost = waves x (tokens per tile + the set-up of a CTA, about one and a half chunks).  For long
    // sequences this stays at 2048; for shorter ones it avoids a mostly empty last wave.
    const int64_t groups = dm.S > 64 ? dm.S / 64 : 1;
    const int64_t sms = sm_count > 0 ? sm_count : 148;
    int best = 2048;
    double best_cost = 1e300;
    for (int tile = 2048; tile >= C; tile -= C) {
        const int64_t ctas = dm.N * groups * ((dm.T + tile - 1) / tile);
        const int64_t waves = (ctas + sms - 1) / sms;
        const double cost = (double)waves * (tile + 96.0);
        if (cost < best_cost * 0.999) { best_cost = cost; best = tile; }
        if (ctas > 64 * sms) break;   // many waves already: shorter tiles only add state traffic
    }
    return best;
}

// fp32 single-pass kernel: [totals of every tile | inclusive prefix of every tile | carry slot per CTA | flags, ticket]
struct FusedLayout {
    size_t states, off_incl, off_carry, off_flags, flag_bytes, total;
};
static FusedLayout fused_layout(const Dims& dm, int tile_tokens) {
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    FusedLayout l;
    l.states = (size_t)dm.N * tiles * kSF * sizeof(float);
    l.off_incl = l.states;
    l.off_carry = 2 * l.states;
    l.off_flags = l.off_carry + (size_t)kFusedMaxGrid * kSF * sizeof(float);
    l.flag_bytes = ((size_t)dm.N * tiles * sizeof(int) + 15) / 16 * 16 + 16;   // + the ticket counter
    l.total = l.off_flags + l.flag_bytes;
    return l;
}

size_t tensor_single_pass_workspace_bytes(const Dims& dm, int tile_tokens) { return fused_layout(dm, tile_tokens).total; }

// the three launches (totals, scan, outputs): one state per tile
size_t tensor_workspace_bytes(const Dims& dm, int, int tile_tokens) {
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    return (size_t)dm.N * tiles * state_floats_per_stream(dm.S, dm.D) * sizeof(float);
}

static cudaError_t tensor_f32_launch(const void* pq, const void* pk, const void* v, void* out,
                                     const float* carry_in, float* state_out, void* ws, bool single_pass,
                                     const Dims& dm, int tile_tokens, cudaStream_t stream, int* status, int phases,
                                     int mode, bool reverse, long long wait_cycles, int withhold_chunk,
                                     const float* planes = nullptr, const BwdX* bwdx = nullptr);

cudaError_t causal_fwd_tensor(const void* pq, const void* pk, const void* v, void* out,
                              const float* carry_in, float* state_out, void* ws, bool single_pass, const Dims& dm,
                              int dtype, int tile_tokens, cudaStream_t stream, int* status, int phases,
                              bool global_norm, long long wait_cycles, int withhold_chunk) {
    if (dtype == RACE_DTYPE_BF16)
        return causal_fwd_tensor_bf16(pq, pk, v, out, carry_in, state_out, ws, dm, tile_tokens, stream,
                                      status, phases, global_norm);
    return tensor_f32_launch(pq, pk, v, out, carry_in, state_out, ws, single_pass, dm, tile_tokens, stream, status,
                             phases, global_norm ? kModeGlobal : kModeBucket, false, wait_cycles, withhold_chunk);
}

// The causal forward from Q, K, V and the hyperplanes (fp32, d_k = 64, L = 4, R = 16; Q, K, V and out in the layout
// [N/heads, T, heads, 64]): the kernels form the bucket probabilities of src/race_baseline.py:41-44 in registers and
// shared memory, so the forward moves Q, K, V and out through HBM and nothing else.  The role of the reference's
// race_causal_forward (src/causal_v2/kernels/race_causal_fwd.h:126-130), which also takes q, k, v and planes.
bool tensor_qkv_supported(const Dims& dm, int dtype, int L, int R) {
    return dtype == RACE_DTYPE_F32 && L == 4 && R == 16 && tensor_supported(dm, dtype);
}
cudaError_t causal_fwd_qkv_tensor(const void* q, const void* k, const void* v, const float* planes, void* out,
                                  const float* carry_in, float* state_out, void* ws, const Dims& dm, int tile_tokens,
                                  cudaStream_t stream, int* status, int phases, bool global_norm) {
    if (!planes) return cudaErrorInvalidValue;
    return tensor_f32_launch(q, k, v, out, carry_in, state_out, ws, false, dm, tile_tokens, stream, status, phases,
                             global_norm ? kModeGlobal : kModeBucket, false, 0, -1, planes);
}

// The plain causal (or, with reverse, anti-causal) product out_t = sum_{j <= t} (q_t . k_j) v_j + q_t . carry over
// fp32 [N, T, 64] tensors on the same three launches: what the backward passes are made of.  State layout as
// everywhere: carry[s][c] = sum_j k_j[s] v_j[c] (the A part is carried along and ignored).
cudaError_t causal_raw_tensor(const void* q, const void* k, const void* v, void* out, const float* carry_in,
                              float* state_out, void* ws, const Dims& dm, int tile_tokens, bool reverse,
                              cudaStream_t stream, int* status, int phases, const BwdX* bwdx) {
    if (bwdx && (reverse || dm.H != 1)) return cudaErrorInvalidValue;
    return tensor_f32_launch(q, k, v, out, carry_in, state_out, ws, false, dm, tile_tokens, stream, status, phases,
                             bwdx ? kModeRawX : kModeRaw, reverse, 0, -1, nullptr, bwdx);
}

// planes != nullptr: pq and pk are Q and K in the layout of V and the kernels form the probabilities (the
// three-launch form of the two estimators only).
static cudaError_t tensor_f32_launch(const void* pq, const void* pk, const void* v, void* out,
                                     const float* carry_in, float* state_out, void* ws, bool single_pass,
                                     const Dims& dm, int tile_tokens, cudaStream_t stream, int* status, int phases,
                                     int mode, bool reverse, long long wait_cycles, int withhold_chunk,
                                     const float* planes, const BwdX* bwdx) {
    const bool global_norm = mode == kModeGlobal;
    const bool proj = planes != nullptr;
    const bool raw = mode == kModeRaw || mode == kModeRawX;
    if (proj && (single_pass || reverse || raw)) return cudaErrorInvalidValue;
    if ((mode == kModeRawX) != (bwdx != nullptr)) return cudaErrorInvalidValue;
    // Runtime calls first: they bind the device's primary context to the calling host thread,
    // which the driver-level tensor-map encoder needs (a thread that has made no runtime call
    // yet, e.g. an autograd worker, has no current context).
    auto totals_kern = proj ? tile_totals_tc<true> : tile_totals_tc<false>;
    const int totals_smem = proj ? T1P::kSmemBytes : T1::kSmemBytes, totals_threads = proj ? T1P::kThreads : T1::kThreads;
    cudaError_t err = cudaFuncSetAttribute(totals_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, totals_smem);
    if (err != cudaSuccess) return err;
    CUtensorMap mk, mv;
    if (!(proj ? make_map_heads(&mk, pk, dm.N, dm.T, dm.D, dm.H) : make_map(&mk, pk, dm.N, dm.T, dm.S)) ||
        !make_map_heads(&mv, v, dm.N, dm.T, dm.D, dm.H))
        return cudaErrorInvalidValue;
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    const FusedLayout lay = fused_layout(dm, tile_tokens);
    if (single_pass && phases == kPhaseAll) {
        // the whole forward as one persistent kernel
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const unsigned long long items = (unsigned long long)dm.N * (unsigned long long)tiles;
        const unsigned grid_f = (unsigned)std::min<unsigned long long>(items, (unsigned long long)std::min(sms > 0 ? sms : 148, kFusedMaxGrid));
        char* base = (char*)ws;
        err = cudaMemsetAsync(base + lay.off_flags, 0, lay.flag_bytes, stream);
        if (err != cudaSuccess) return err;
        FusedArgs fa;
        fa.pq = (const float*)pq;
        fa.out = (float*)out;
        fa.agg = (float*)base;
        fa.incl = (float*)(base + lay.off_incl);
        fa.cta_carry = (float*)(base + lay.off_carry);
        fa.flags = (int*)(base + lay.off_flags);
        fa.ticket = (unsigned long long*)(base + lay.off_flags + lay.flag_bytes - 16);
        fa.carry_in = carry_in;
        fa.state_out = state_out;
        fa.T = dm.T; fa.N = dm.N; fa.tiles = tiles;
        fa.tile_tokens = tile_tokens;
        fa.eps = dm.eps;
        fa.heads = dm.H;
        fa.status = status;
        fa.wait_cycles = wait_cycles;
        fa.withhold_chunk = withhold_chunk;
        auto kern = global_norm ? causal_fused_tc<true> : causal_fused_tc<false>;
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kFusedSmemBytes);
        if (err != cudaSuccess) return err;
        kern<<<grid_f, kThreads, kFusedSmemBytes, stream>>>(mk, mv, fa);
        return cudaGetLastError();
    }
    dim3 grid((unsigned)tiles, (unsigned)dm.N);
    // 1. tile totals (tensor cores)  2. exclusive scan over tiles  3. output pass
    if (phases & kPhaseTotals) {
        totals_kern<<<grid, totals_threads, totals_smem, stream>>>(mk, mv, (float*)ws, dm.T, tile_tokens, dm.H, status,
                                                                planes);
        err = cudaGetLastError();
        if (err != cudaSuccess) return err;
    }
    if (!(phases & kPhaseOutput)) {
        // totals only: sum the tiles into state_out, keep the per-tile totals (nothing to do when
        // the caller wants the per-tile totals alone)
        if (!state_out) return cudaSuccess;
        return causal_scan_tiles((float*)ws, carry_in, state_out, dm, tile_tokens, stream, /*write_prefix=*/false);
    }
    err = causal_scan_tiles((float*)ws, carry_in, state_out, dm, tile_tokens, stream, /*write_prefix=*/true, reverse);
    if (err != cudaSuccess) return err;
    auto kern = mode == kModeRawX ? causal_out_tc<kModeRawX, false, false>
                : mode == kModeRaw
                    ? (reverse ? causal_out_tc<kModeRaw, true, false> : causal_out_tc<kModeRaw, false, false>)
                    : proj ? (global_norm ? causal_out_tc<kModeGlobal, false, true> : causal_out_tc<kModeBucket, false, true>)
                           : (global_norm ? causal_out_tc<kModeGlobal, false, false>
                                          : causal_out_tc<kModeBucket, false, false>);
    err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err != cudaSuccess) return err;
    kern<<<grid, kThreads, kSmemBytes, stream>>>((const float*)pq, mk, mv, (float*)out, (const float*)ws, dm.T,
                                                 tile_tokens, dm.eps, dm.H, status, wait_cycles, withhold_chunk, planes,
                                                 bwdx ? *bwdx : BwdX{});
    return cudaGetLastError();
}

#ifdef RACE_FUSED_PROF
extern "C" int race_b200_debug_fused_prof(long long* host_out, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(host_out, g_fused_prof, sizeof(long long) * 160 * 16);
    if (e == cudaSuccess && reset) {
        static long long zeros[160 * 16] = {};
        e = cudaMemcpyToSymbol(g_fused_prof, zeros, sizeof(zeros));
    }
    return (int)e;
}
#endif

#ifdef RACE_TC_TRACE
extern "C" int race_b200_debug_set_trace(long long* buf) {
    return (int)cudaMemcpyToSymbol(g_trace_buf, &buf, sizeof(buf));
}
#endif

}  // namespace race
