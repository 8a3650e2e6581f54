// Causal backward on the tcgen05 kernels (fp32, S = 64, d_k = 64): gradients of
//     out_t = sum_s pQ_t[s] B_t[s,:] / (A_t[s] + eps),   A_t, B_t inclusive prefixes of pK and pK (x) V
// (src/race_baseline.py:45-51; the reference has no causal backward, its design note only outlines one for
// the other estimator, docs/causal_v2_design.md:689-741).  With inv_t = 1/(A_t + eps), W_t = pQ_t inv_t:
//     X_t   = B_t dO_t                         dPQ_t = X_t inv_t          g_t = -X_t W_t inv_t
//     dV_j  = sum_{t >= j} (pK_j . W_t) dO_t
//     dPK_j = sum_{t >= j} g_t + sum_{t >= j} (V_j . dO_t) W_t
// Each sum over tokens with an inner product in it is a plain causal (or anti-causal) product
//     raw(q, k, v)_t = sum_{j <= t} (q_t . k_j) v_j          (reverse: j >= t)
// which is what the forward's tensor kernels compute when they skip the normalisation: same TMA / TMEM /
// tcgen05 pipeline, same bf16 hi/lo limbs, the tile totals / scan / output launches with other tensors in the
// roles of pQ, pK, V.  So the backward is three such passes and a few streaming kernels:
//     1. block sums of pK (with the running sum at every 64-token chunk start) and their scan
//     2. X  = raw(dO, V, pK)                   state of the pass = B^T, so carry_in enters transposed.  X is not
//        stored: the pass takes A_t = block prefix + chunk prefix + running sum inside the chunk (one more
//        triangular product over its V operand, which is pK) and writes dPQ = X inv, W = pQ inv and g = -dPQ W
//        from its epilogue; then the block sums of g
//     3. dV = raw_reverse(pK, W, dO)           state = sum W^T dO: its carry is the gradient of the final B, its
//                                              total the gradient of the carried-in B
//     4. P  = raw_reverse(V, dO, W)            state = the transpose of pass 3's
//     5. reverse scan of the chunk sums of g (carry: gradient of the final A), then dPK = P + running suffix sum
// P is written into the dPK buffer (same shape and type), so the scratch memory is W and g ([N, T, 64] fp32 each)
// plus the block / chunk sums and the tile states of the passes.
#include <algorithm>

#include "common.cuh"
#include "launch.h"

namespace race {
namespace {

constexpr int S = 64, D = 64;
constexpr int kSF = S * (D + 1);
constexpr int kBlk = 512;          // tokens per block of the streaming kernels (one thread per block and column)
constexpr int kPwThreads = 256;    // 4 blocks x 64 columns per CTA

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// sums[n][b][c] = sum over the tokens of block b of x[n][t][c]
__global__ void __launch_bounds__(kPwThreads)
bwd_block_sums(const float* __restrict__ x, float* __restrict__ sums, int64_t T, int64_t nblk, int64_t total_blocks) {
    const int64_t gb = (int64_t)blockIdx.x * (kPwThreads / 64) + (threadIdx.x >> 6);
    if (gb >= total_blocks) return;
    const int c = threadIdx.x & 63;
    const int64_t n = gb / nblk, b = gb - n * nblk;
    const int64_t t0 = b * kBlk, t1 = min(T, t0 + (int64_t)kBlk);
    const float* p = x + (n * T + t0) * 64 + c;
    float acc = 0.f;
    int64_t t = t0;
    for (; t + 8 <= t1; t += 8, p += 8 * 64) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldg(p + u * 64);
#pragma unroll
        for (int u = 0; u < 8; ++u) acc += v[u];
    }
    for (; t < t1; ++t, p += 64) acc += __ldg(p);
    sums[gb * 64 + c] = acc;
}

// in-place exclusive scan over the blocks of a stream (reverse: suffix sums, last block first); carry is the A part
// ([64] floats at offset S*D) of a packed state per stream or null; total (nullable) receives carry + everything
__global__ void __launch_bounds__(64)
bwd_block_scan(float* __restrict__ sums, const float* __restrict__ carry_state, float* __restrict__ total_state,
               int64_t nblk, int reverse) {
    const int c = threadIdx.x;
    const int64_t n = blockIdx.x;
    float run = carry_state ? carry_state[n * kSF + S * D + c] : 0.f;
    float* p = sums + n * nblk * 64 + c;
    auto at = [&](int64_t b) { return (reverse ? nblk - 1 - b : b) * 64; };
    int64_t b = 0;
    for (; b + 16 <= nblk; b += 16) {
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = p[at(b + u)];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            p[at(b + u)] = run;
            run += v[u];
        }
    }
    for (; b < nblk; ++b) {
        const float v = p[at(b)];
        p[at(b)] = run;
        run += v;
    }
    if (total_state) total_state[n * kSF + S * D + c] = run;
}

// sums[n][b][c] as bwd_block_sums, and chunk[n][j][c] = the sum of x over the tokens of chunk j's block that precede
// chunk j (64-token chunks; a block is kBlk / 64 of them)
__global__ void __launch_bounds__(kPwThreads)
bwd_block_chunk_sums(const float* __restrict__ x, float* __restrict__ sums, float* __restrict__ chunk, int64_t T,
                     int64_t nblk, int64_t nchunk, int64_t total_blocks) {
    const int64_t gb = (int64_t)blockIdx.x * (kPwThreads / 64) + (threadIdx.x >> 6);
    if (gb >= total_blocks) return;
    const int c = threadIdx.x & 63;
    const int64_t n = gb / nblk, b = gb - n * nblk;
    const int64_t t0 = b * kBlk, t1 = min(T, t0 + (int64_t)kBlk);
    const float* p = x + (n * T + t0) * 64 + c;
    float* cp = chunk + (n * nchunk + t0 / 64) * 64 + c;
    float acc = 0.f;
    for (int64_t t = t0; t < t1; t += 64, cp += 64) {
        *cp = acc;
        const int cnt = (int)min((int64_t)64, t1 - t);
        if (cnt == 64) {
#pragma unroll
            for (int u8 = 0; u8 < 8; ++u8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = __ldg(p + (u8 * 8 + u) * 64);
#pragma unroll
                for (int u = 0; u < 8; ++u) acc += v[u];
            }
        } else {
            for (int u = 0; u < cnt; ++u) acc += __ldg(p + u * 64);
        }
        p += 64 * 64;
    }
    sums[gb * 64 + c] = acc;
}

// reverse streaming kernel: dPK_j = P_j + suffix[block] + sum_{t >= j, t in block} g_t (P in pdpk on entry)
__global__ void __launch_bounds__(kPwThreads)
bwd_pointwise_rev(const float* __restrict__ g, float* __restrict__ pdpk, const float* __restrict__ gsuffix, int64_t T,
                  int64_t nblk, int64_t total_blocks) {
    const int64_t gb = (int64_t)blockIdx.x * (kPwThreads / 64) + (threadIdx.x >> 6);
    if (gb >= total_blocks) return;
    const int c = threadIdx.x & 63;
    const int64_t n = gb / nblk, b = gb - n * nblk;
    const int64_t t0 = b * kBlk, t1 = min(T, t0 + (int64_t)kBlk);
    float sa = gsuffix[gb * 64 + c];
    for (int64_t t = t1; t > t0; t -= 4) {
        const int cnt = (int)min((int64_t)4, t - t0);
        float g4[4], p4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (u < cnt) {
                const int64_t off = (n * T + (t - 1 - u)) * 64 + c;
                g4[u] = __ldcs(g + off);
                p4[u] = pdpk[off];
            }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (u < cnt) {
                const int64_t off = (n * T + (t - 1 - u)) * 64 + c;
                sa += g4[u];
                pdpk[off] = p4[u] + sa;
            }
    }
}

// dst[n] = the state src[n] with its B part ([64][64]) transposed and its A part zeroed
__global__ void __launch_bounds__(256)
bwd_transpose_state(const float* __restrict__ src, float* __restrict__ dst) {
    __shared__ float tile[64][65];
    const int64_t n = blockIdx.x;
    const float* s = src + n * kSF;
    float* d = dst + n * kSF;
    for (int i = threadIdx.x; i < S * D; i += 256) tile[i >> 6][i & 63] = s[i];
    __syncthreads();
    for (int i = threadIdx.x; i < S * D; i += 256) d[i] = tile[i & 63][i >> 6];
    if (threadIdx.x < S) d[S * D + threadIdx.x] = 0.f;
}

struct BwdLayout {
    size_t tiles, tiles2, w, g, asum, gsum, achunk, st0, st1, total;
};
BwdLayout bwd_layout(const Dims& dm, int tile_tokens) {
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    const int64_t nblk = (dm.T + kBlk - 1) / kBlk;
    const size_t tok = align256((size_t)dm.N * dm.T * 64 * sizeof(float));
    const size_t blk = align256((size_t)dm.N * nblk * 64 * sizeof(float));
    const size_t st = align256((size_t)dm.N * kSF * sizeof(float));
    BwdLayout l;
    const size_t tl = align256((size_t)dm.N * tiles * kSF * sizeof(float));
    l.tiles = 0;
    l.tiles2 = tl;
    l.w = 2 * tl;
    l.g = l.w + tok;
    l.asum = l.g + tok;
    l.gsum = l.asum + blk;
    l.achunk = l.gsum + blk;
    l.st0 = l.achunk + align256((size_t)dm.N * ((dm.T + 63) / 64) * 64 * sizeof(float));
    l.st1 = l.st0 + st;
    l.total = l.st1 + st;
    return l;
}

#define RACE_CK(expr)                                  \
    do {                                               \
        cudaError_t e_ = (expr);                       \
        if (e_ != cudaSuccess) return e_;              \
    } while (0)

}  // namespace

bool causal_bwd_tensor_supported(const Dims& dm, int dtype) {
    return dtype == RACE_DTYPE_F32 && dm.H == 1 && tensor_supported(dm, dtype);
}

int causal_bwd_tensor_tile_tokens(const Dims& dm, int sm_count) {
    return tensor_default_tile_tokens(dm, RACE_DTYPE_F32, sm_count);
}

size_t causal_bwd_tensor_workspace_bytes(const Dims& dm, int tile_tokens) {
    if (dm.N == 0 || dm.T == 0) return 0;
    return bwd_layout(dm, tile_tokens).total;
}

cudaError_t causal_bwd_tensor(const void* pq, const void* pk, const void* v, const void* dout, const float* carry_in,
                              const float* d_state, void* dpq, void* dpk, void* dv, float* d_carry, void* ws,
                              const Dims& dm, int tile_tokens, cudaStream_t stream, int* status) {
    const BwdLayout l = bwd_layout(dm, tile_tokens);
    char* base = (char*)ws;
    float* ws_tiles = (float*)(base + l.tiles);
    float* w = (float*)(base + l.w);
    float* g = (float*)(base + l.g);
    float* asum = (float*)(base + l.asum);
    float* gsum = (float*)(base + l.gsum);
    float* ws_tiles2 = (float*)(base + l.tiles2);
    float* st_t = (float*)(base + l.st0);      // a transposed carry
    float* st_dv = (float*)(base + l.st1);     // final state of pass 3 when the caller does not want it
    const int64_t tiles = (dm.T + tile_tokens - 1) / tile_tokens;
    const int64_t nblk = (dm.T + kBlk - 1) / kBlk, total_blocks = dm.N * nblk;
    const unsigned pw_grid = (unsigned)((total_blocks + kPwThreads / 64 - 1) / (kPwThreads / 64));

    // 1. sums of pK: per block (then scanned, carry included) and inside the block up to every chunk start
    float* achunk = (float*)(base + l.achunk);
    const int64_t nchunk = (dm.T + 63) / 64;
    bwd_block_chunk_sums<<<pw_grid, kPwThreads, 0, stream>>>((const float*)pk, asum, achunk, dm.T, nblk, nchunk,
                                                             total_blocks);
    RACE_CK(cudaGetLastError());
    bwd_block_scan<<<(unsigned)dm.N, 64, 0, stream>>>(asum, carry_in, nullptr, nblk, 0);
    RACE_CK(cudaGetLastError());
    // 2. X = raw(dO, V, pK), the state of the pass is B^T; its epilogue writes dPQ, W and g.  Then the block sums of g.
    if (carry_in) bwd_transpose_state<<<(unsigned)dm.N, 256, 0, stream>>>(carry_in, st_t);
    RACE_CK(cudaGetLastError());
    BwdX bx;
    bx.pq_true = (const float*)pq;
    bx.ablock = asum;
    bx.achunk = achunk;
    bx.w_out = w;
    bx.g_out = g;
    bx.nblk = nblk;
    bx.nchunk = nchunk;
    bx.block_tokens = kBlk;
    bx.eps = dm.eps;
    RACE_CK(causal_raw_tensor(dout, v, pk, dpq, carry_in ? st_t : nullptr, nullptr, ws_tiles, dm, tile_tokens,
                              /*reverse=*/false, stream, status, kPhaseAll, &bx));
    bwd_block_sums<<<pw_grid, kPwThreads, 0, stream>>>(g, gsum, dm.T, nblk, total_blocks);
    RACE_CK(cudaGetLastError());
    // 3. dV = raw_reverse(pK, W, dO); state sum W^T dO: carry = gradient of the final B, total = gradient of carry_in's B.
    //    Pass 4 below has the roles of W and dO swapped, so its tile totals are the transposes of this pass's:
    //    the totals launch runs once and the second tile buffer gets the transposed states.
    RACE_CK(causal_raw_tensor(nullptr, w, dout, nullptr, nullptr, nullptr, ws_tiles, dm, tile_tokens, true, stream, status,
                              kPhaseTotals));
    bwd_transpose_state<<<(unsigned)(dm.N * tiles), 256, 0, stream>>>(ws_tiles, ws_tiles2);
    RACE_CK(cudaGetLastError());
    RACE_CK(causal_raw_tensor(pk, w, dout, dv, d_state, d_carry ? d_carry : st_dv, ws_tiles, dm, tile_tokens,
                              /*reverse=*/true, stream, status, kPhaseOutput));
    // 4. P = raw_reverse(V, dO, W) into the dPK buffer; state = the transpose of pass 3's
    if (d_state) bwd_transpose_state<<<(unsigned)dm.N, 256, 0, stream>>>(d_state, st_t);
    RACE_CK(cudaGetLastError());
    RACE_CK(causal_raw_tensor(v, dout, w, dpk, d_state ? st_t : nullptr, nullptr, ws_tiles2, dm, tile_tokens,
                              /*reverse=*/true, stream, status, kPhaseOutput));
    // 5. dPK = P + suffix sums of g (carry: gradient of the final A; total: gradient of carry_in's A, which
    //    overwrites the A part that pass 3 left in d_carry)
    bwd_block_scan<<<(unsigned)dm.N, 64, 0, stream>>>(gsum, d_state, d_carry, nblk, 1);
    RACE_CK(cudaGetLastError());
    bwd_pointwise_rev<<<pw_grid, kPwThreads, 0, stream>>>(g, (float*)dpk, gsum, dm.T, nblk, total_blocks);
    return cudaGetLastError();
}

}  // namespace race
