// Bucket probabilities of 16 rows at a time with warp-level mma.sync, for the geometry d_k = 64, L = 4 tables,
// K = 4 planes per table (R = 16 buckets, S = L R = 64): shared by the stand-alone producer kernel and by the
// causal kernels that form the probabilities of Q and K themselves (so that they never reach HBM).
//
//   proj[p] = x . planes[p]  (p = 4 l + k)        [16 rows x 64] . [64 x 16] on the tensor cores: bf16 hi/lo limbs
//                                                  of both operands, three products, fp32 accumulation
//   th = tanh(proj) / sqrt(d_k);  p1 = sigmoid(2 th) = 1/2 + tanh(th)/2, p0 = sigmoid(-2 th) = 1 - p1
//   probs[l][8 b0 + 4 b1 + 2 b2 + b3] = p_b0(4l) p_b1(4l+1) p_b2(4l+2) p_b3(4l+3)
// (src/race_baseline.py:41-44; the softmax over the sign corners factorises into this product,
// src/verify_factorization.py:42-57).  All callers run the same instructions in the same order, so the
// probabilities a causal kernel forms are bit-identical to what the stand-alone kernel writes.
//
// Lane roles in a warp (g = lane / 4, t = lane % 4), those of the m16n8k16 fragments: a lane feeds rows g and
// g + 8 and, after the product, holds the projections of those rows on the planes 8 nt + 2 t + e (nt, e in {0,1}).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace race {
namespace {

// tanh(a) = sign(a) (1 - e)/(1 + e), e = exp(-2|a|): absolute error ~1e-7, which is what the logits
// need (they are tanh/sqrt(d_k), and the projections of unit-variance rows mostly saturate)
__device__ __forceinline__ float fast_tanh(float a) {
    const float e = __expf(-2.f * fabsf(a));
    return copysignf(__fdividef(1.f - e, 1.f + e), a);
}

__device__ __forceinline__ void split_pair(float a, float b, uint32_t& hi, uint32_t& lo) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    hi = *reinterpret_cast<uint32_t*>(&h);
    __nv_bfloat162 l = __floats2bfloat162_rn(a - __uint_as_float(hi << 16), b - __uint_as_float(hi & 0xffff0000u));
    lo = *reinterpret_cast<uint32_t*>(&l);
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Plane fragments (B operand, 16 planes x 64 features).  Fragment f = 4 j + 2 nt + half (k-step j, plane block nt)
// of a lane is the pair planes[8 nt + g][16 j + 8 half + 2 t, +1] as a hi and a lo limb word.
struct PlaneFrags {
    uint32_t hi[16], lo[16];
};
__device__ __forceinline__ void plane_frag(const float* __restrict__ planes, int f, int lane, uint32_t& hi,
                                           uint32_t& lo) {
    const int j = f >> 2, nt = (f >> 1) & 1, half = f & 1, g = lane >> 2, t = lane & 3;
    const float2 p = __ldg(reinterpret_cast<const float2*>(planes + (8 * nt + g) * 64 + 16 * j + 8 * half + 2 * t));
    split_pair(p.x, p.y, hi, lo);
}
__device__ __forceinline__ void load_plane_frags(const float* __restrict__ planes, int lane, PlaneFrags& pf) {
#pragma unroll
    for (int f = 0; f < 16; ++f) plane_frag(planes, f, lane, pf.hi[f], pf.lo[f]);
}
// The same table in shared memory for kernels that cannot keep 32 registers for it: word (2 f + limb) * 32 + lane
// (a warp reads 32 consecutive words: no bank conflicts).  Written by nthreads threads; the caller synchronises.
constexpr int kPlaneTabWords = 16 * 2 * 32;
__device__ __forceinline__ void build_plane_tab(const float* __restrict__ planes, uint32_t* tab, int tid,
                                                int nthreads) {
    for (int i = tid; i < 16 * 32; i += nthreads) {
        const int f = i >> 5, lane = i & 31;
        uint32_t hi, lo;
        plane_frag(planes, f, lane, hi, lo);
        tab[(2 * f) * 32 + lane] = hi;
        tab[(2 * f + 1) * 32 + lane] = lo;
    }
}
__device__ __forceinline__ void load_plane_frags_tab(const uint32_t* tab, int lane, PlaneFrags& pf) {
#pragma unroll
    for (int f = 0; f < 16; ++f) {
        pf.hi[f] = tab[(2 * f) * 32 + lane];
        pf.lo[f] = tab[(2 * f + 1) * 32 + lane];
    }
}

// c[nt][2 h + e] = projection of row g + 8 h on plane 8 nt + 2 t + e.  raw[2 u + h] = the lane's pair
// x[row g + 8 h][8 u + 2 t, +1], u = 0..7.  Each of the three limb products has its own accumulator (six
// independent chains of four dependent mma.sync instead of two chains of twelve); they are added at the end.
__device__ __forceinline__ void project_rows(const float2 (&raw)[16], const PlaneFrags& pf, float (&c)[2][4]) {
    float acc[3][2][4];
#pragma unroll
    for (int p = 0; p < 3; ++p)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[p][nt][i] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        // A fragment of k-step j: {row g cols 2t; row g+8 cols 2t; row g cols 8+2t; row g+8 cols 8+2t}
        uint32_t ahi[4], alo[4];
        split_pair(raw[4 * j].x, raw[4 * j].y, ahi[0], alo[0]);
        split_pair(raw[4 * j + 1].x, raw[4 * j + 1].y, ahi[1], alo[1]);
        split_pair(raw[4 * j + 2].x, raw[4 * j + 2].y, ahi[2], alo[2]);
        split_pair(raw[4 * j + 3].x, raw[4 * j + 3].y, ahi[3], alo[3]);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int f = 4 * j + 2 * nt;
            mma_bf16_16816(acc[0][nt], ahi, pf.hi[f], pf.hi[f + 1]);
            mma_bf16_16816(acc[1][nt], ahi, pf.lo[f], pf.lo[f + 1]);
            mma_bf16_16816(acc[2][nt], alo, pf.hi[f], pf.hi[f + 1]);
        }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) c[nt][i] = acc[0][nt][i] + (acc[1][nt][i] + acc[2][nt][i]);
}

// (p0, p1) = (sigmoid(-2 th), sigmoid(2 th)), th = tanh(proj) / sqrt(d_k), of eight projections at once: the
// eight chains are written stage by stage so that they overlap in the pipeline.  sigmoid(2 th) = 1/2 + tanh(th)/2
// and |th| <= 1/sqrt(d_k) <= 1/8, where the odd polynomial of tanh to th^7 is exact to 2e-10; p0 + p1 = 1.
__device__ __forceinline__ void soft_bits8(const float (&proj)[8], float inv_scale, float (&p0)[8], float (&p1)[8]) {
    float e[8], th[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = __expf(-2.f * fabsf(proj[i]));
#pragma unroll
    for (int i = 0; i < 8; ++i) th[i] = copysignf(__fdividef(1.f - e[i], 1.f + e[i]), proj[i]) * inv_scale;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float s = th[i] * th[i];
        const float poly = fmaf(s, fmaf(s, fmaf(s, -17.f / 315.f, 2.f / 15.f), -1.f / 3.f), 1.f);
        const float half = 0.5f * th[i] * poly;
        p1[i] = 0.5f + half;
        p0[i] = 0.5f - half;
    }
}

// Table-per-lane form: lane t gets the 16 probabilities of table t of its rows g (vals[0]) and g + 8 (vals[1]),
// buckets in order.  Table l needs the planes 4l .. 4l+3: they sit in block nt = l >> 1 of the lanes 2 (l & 1)
// and 2 (l & 1) + 1.
__device__ __forceinline__ void table_probs(const float (&c)[2][4], int lane, float inv_scale, float (&vals)[2][16]) {
    const int t = lane & 3;
    const int src_a = (lane & ~3) + 2 * (t & 1), src_b = src_a + 1;
    float th[8];   // [4 h + k]
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float a0 = __shfl_sync(0xffffffffu, c[0][2 * h + e], src_a);
            const float a1 = __shfl_sync(0xffffffffu, c[1][2 * h + e], src_a);
            const float b0 = __shfl_sync(0xffffffffu, c[0][2 * h + e], src_b);
            const float b1 = __shfl_sync(0xffffffffu, c[1][2 * h + e], src_b);
            th[4 * h + e] = (t >> 1) ? a1 : a0;
            th[4 * h + 2 + e] = (t >> 1) ? b1 : b0;
        }
    float p0[8], p1[8];
    soft_bits8(th, inv_scale, p0, p1);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        vals[h][0] = p0[4 * h];
        vals[h][1] = p1[4 * h];
#pragma unroll
        for (int k = 1; k < 4; ++k) {
#pragma unroll
            for (int i = (1 << k) - 1; i >= 0; --i) {
                const float b = vals[h][i];
                vals[h][2 * i] = b * p0[4 * h + k];
                vals[h][2 * i + 1] = b * p1[4 * h + k];
            }
        }
    }
}

// Accumulator-fragment form: out[2 x + h] = probabilities of row g + 8 h at the buckets 8 x + 2 t, + 1 (x = 0..7),
// i.e. of table x >> 1 the buckets with b0 = x & 1, (b1, b2) = the bits of t, b3 = 0 and 1.  Every lane evaluates
// the soft bits of its own four planes and the quad exchanges them; the factors are multiplied in plane order,
// like table_probs does, so both forms give the same bits.
__device__ __forceinline__ void fragment_probs(const float (&c)[2][4], int lane, float inv_scale,
                                               float2 (&out)[16]) {
    const int t = lane & 3, quad = lane & ~3;
    float pr[8], p0[8], p1[8];   // [4 nt + 2 h + e]
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) pr[4 * nt + i] = c[nt][i];
    soft_bits8(pr, inv_scale, p0, p1);
#pragma unroll
    for (int l = 0; l < 4; ++l) {
        const int nt = l >> 1, src_a = quad + 2 * (l & 1), src_b = src_a + 1;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // plane 4l (+1): lane src_a, e = 0 (1); plane 4l+2 (+3): lane src_b, e = 0 (1)
            const int i0 = 4 * nt + 2 * h, i1 = i0 + 1;
            const float a0_0 = __shfl_sync(0xffffffffu, p0[i0], src_a);
            const float a0_1 = __shfl_sync(0xffffffffu, p1[i0], src_a);
            const float a1_0 = __shfl_sync(0xffffffffu, p0[i1], src_a);
            const float a1_1 = __shfl_sync(0xffffffffu, p1[i1], src_a);
            const float a2_0 = __shfl_sync(0xffffffffu, p0[i0], src_b);
            const float a2_1 = __shfl_sync(0xffffffffu, p1[i0], src_b);
            const float a3_0 = __shfl_sync(0xffffffffu, p0[i1], src_b);
            const float a3_1 = __shfl_sync(0xffffffffu, p1[i1], src_b);
            const float s1 = (t >> 1) ? a1_1 : a1_0;
            const float s2 = (t & 1) ? a2_1 : a2_0;
            const float v0 = (a0_0 * s1) * s2, v1 = (a0_1 * s1) * s2;
            out[2 * (2 * l) + h] = make_float2(v0 * a3_0, v0 * a3_1);
            out[2 * (2 * l + 1) + h] = make_float2(v1 * a3_0, v1 * a3_1);
        }
    }
}

}  // namespace
}  // namespace race
