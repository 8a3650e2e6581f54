// Bucket-probability producer: x [rows, d_k] -> probs [rows, L, R], R = 2^K.
//   proj[l,k] = x . planes[l*K+k];  th = tanh(proj)/sqrt(d_k)
//   probs[l,r] = softmax_r( sum_k sign(r,k) th[l,k] ),  sign(r,k) = +1 iff bit (K-1-k) of r
// (src/race_baseline.py:41-44).  The softmax over the 2^K sign corners factorises exactly into
// prod_k sigmoid(+-2 th[l,k]) because sum_r exp(z_r) = prod_k (e^th_k + e^-th_k); the kernel
// evaluates that product (the reference checks the same identity numerically,
// src/verify_factorization.py:42-57).
//
// The stream flattening of the operator ([M,B,T,H,d_k] -> [N,T,d_k], src/race_baseline.py:35-40)
// can be fused into the read: with heads = H the input row of output row (n = mb*H + h, t) is
// ((mb*T + t)*H + h)*d_k; heads = 1 is the plain contiguous case.
//
// A streaming kernel: one row per thread, 128 rows per CTA (several CTAs per SM overlap their phases).  The x tile is read with coalesced
// 16-byte loads into shared memory, each thread then keeps its row in registers (d_k <= 64) and
// runs the L*K dot products against plane values broadcast from shared memory with 16-byte loads
// (4 FMAs per load), the probabilities of a row go back through the same shared-memory tile and
// are written with coalesced 16-byte stores.  Algorithmic bytes per row: d_k*elt in, L*R*elt out.
#include <algorithm>

#include "common.cuh"
#include "launch.h"
#include "probs_frag.cuh"

namespace race {
namespace {

constexpr int RB = 128;  // rows per CTA = threads per CTA

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
    static __device__ __forceinline__ void store(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = __ldcs(reinterpret_cast<const uint2*>(p));
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        __stcs(reinterpret_cast<uint2*>(p), u);
    }
};

// kXReg: d <= 64, the thread's row lives in registers; the tile is then free for the outputs, which go
// through it (stage_out) when a row of L*R values fits, and straight from registers otherwise
template <typename Tx, typename Tp, int K, bool kXReg>
__global__ void __launch_bounds__(RB)
bucket_probs_kernel(const Tx* __restrict__ x, const float* __restrict__ planes, Tp* __restrict__ probs,
                    int64_t rows, int64_t T, int heads, int d, int L, int stage_out) {
    constexpr int R = 1 << K;
    extern __shared__ __align__(16) float smem[];
    const int LK = L * K, LR = L * R;
    const int ldx = d + 4, ldo = LR + 4;                       // row strides, = 4 (mod 32): no bank conflicts
    float* sp = smem;                                          // [LK][d]
    float* sx = sp + LK * d;                                   // [RB][ldx]
    float* so = sx;                                            // [RB][ldo], only with stage_out
    const int tid = threadIdx.x;
    const int64_t row0 = (int64_t)blockIdx.x * RB;
    const int valid = (int)min((int64_t)RB, rows - row0);

    for (int i = tid; i < LK * d / 4; i += RB)
        reinterpret_cast<float4*>(sp)[i] = reinterpret_cast<const float4*>(planes)[i];
    // element offset of every row of the tile in x (the flattening, if any, happens here)
    int64_t* srow = reinterpret_cast<int64_t*>(sx + RB * (kXReg && stage_out && LR > d ? ldo : ldx));
    if (tid < valid) {
        const int64_t g = row0 + tid;                          // output row: stream n, token t
        const int64_t n = g / T, t = g - n * T;
        const int64_t mb = n / heads, h = n - mb * heads;
        srow[tid] = ((mb * T + t) * heads + h) * d;
    }
    __syncthreads();
    {
        // sixteen 16-byte loads in flight per thread; consecutive threads read consecutive 16 bytes of a row
        const int d4 = d >> 2;                                 // 16-byte items per row; divides RB
        const int c = (tid % d4) * 4, r0 = tid / d4, rstep = RB / d4;
        for (int u0 = 0; u0 < d4; u0 += 16) {
            float4 v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int r = r0 + (u0 + u) * rstep;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (u0 + u < d4 && r < valid) v[u] = Vec4<Tx>::load(x + srow[r] + c);
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int r = r0 + (u0 + u) * rstep;
                if (u0 + u < d4) *reinterpret_cast<float4*>(sx + r * ldx + c) = v[u];
            }
        }
    }
    __syncthreads();

    const float* xrow = sx + tid * ldx;
    float xr[kXReg ? 64 : 4];
    if (kXReg) {
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
            const float4 v = c < d ? *reinterpret_cast<const float4*>(xrow + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            xr[c] = v.x; xr[c + 1] = v.y; xr[c + 2] = v.z; xr[c + 3] = v.w;
        }
        __syncthreads();   // every row is in registers: the tile may take the outputs
    }
    const float inv_scale = rsqrtf((float)d);
    float* orow = so + tid * ldo;
    for (int l = 0; l < L; ++l) {
        float acc[K];
#pragma unroll
        for (int k = 0; k < K; ++k) acc[k] = 0.f;
        if (kXReg) {
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
                if (c < d) {
#pragma unroll
                    for (int k = 0; k < K; ++k) {
                        const float4 p = *reinterpret_cast<const float4*>(sp + (l * K + k) * d + c);
                        acc[k] = fmaf(xr[c], p.x, acc[k]);
                        acc[k] = fmaf(xr[c + 1], p.y, acc[k]);
                        acc[k] = fmaf(xr[c + 2], p.z, acc[k]);
                        acc[k] = fmaf(xr[c + 3], p.w, acc[k]);
                    }
                }
            }
        } else {
            for (int c = 0; c < d; c += 4) {
                const float4 xv = *reinterpret_cast<const float4*>(xrow + c);
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    const float4 p = *reinterpret_cast<const float4*>(sp + (l * K + k) * d + c);
                    acc[k] = fmaf(xv.x, p.x, acc[k]);
                    acc[k] = fmaf(xv.y, p.y, acc[k]);
                    acc[k] = fmaf(xv.z, p.z, acc[k]);
                    acc[k] = fmaf(xv.w, p.w, acc[k]);
                }
            }
        }
        float vals[R];
        vals[0] = 1.f;
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const float th = fast_tanh(acc[k]) * inv_scale;
            const float e = __expf(-2.f * th);            // |th| <= 1/sqrt(d): no overflow
            const float p1 = 1.f / (1.f + e);             // sigmoid(+2 th)
            const float p0 = e * p1;                      // sigmoid(-2 th)
#pragma unroll
            for (int i = (1 << k) - 1; i >= 0; --i) {
                const float b = vals[i];
                vals[2 * i] = b * p0;
                vals[2 * i + 1] = b * p1;
            }
        }
        if (stage_out) {
            if (R >= 4) {
#pragma unroll
                for (int i = 0; i < R; i += 4)
                    *reinterpret_cast<float4*>(orow + l * R + i) =
                        make_float4(vals[i], vals[(i + 1) % R], vals[(i + 2) % R], vals[(i + 3) % R]);
            } else {
#pragma unroll
                for (int i = 0; i < R; ++i) orow[l * R + i] = vals[i];
            }
        } else if (tid < valid) {
            Tp* dst = probs + ((row0 + tid) * L + l) * (int64_t)R;
            if (R >= 4) {
#pragma unroll
                for (int i = 0; i < R; i += 4)
                    Vec4<Tp>::store(dst + i, make_float4(vals[i], vals[(i + 1) % R], vals[(i + 2) % R], vals[(i + 3) % R]));
            } else {
#pragma unroll
                for (int i = 0; i < R; ++i) dst[i] = (Tp)vals[i];
            }
        }
    }
    if (!stage_out) return;
    __syncthreads();
    if ((LR & 3) == 0) {
        const int o4 = LR >> 2;
        for (int i = tid; i < RB * o4; i += RB) {
            const int r = i / o4, c = (i - r * o4) * 4;
            if (r < valid)
                Vec4<Tp>::store(probs + (row0 + r) * LR + c, *reinterpret_cast<const float4*>(so + r * ldo + c));
        }
    } else {   // L*R = 2 (one table, one plane) or another count not divisible by 4
        for (int i = tid; i < RB * LR; i += RB) {
            const int r = i / LR, c = i - r * LR;
            if (r < valid) probs[(row0 + r) * LR + c] = (Tp)so[r * ldo + c];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Fast path for the geometry of the causal fp32 configurations (d_k = 64, L = 4, K = 4, fp32 in and out): the
// 16 projections of a row are a [rows x 64] . [64 x 16] product, run on the tensor cores with warp-level
// mma.sync (m16n8k16, bf16 hi/lo limbs of both operands, three passes, fp32 accumulation: operand error
// ~2^-17) straight from registers.  A warp takes 16 rows at a time: each lane loads the 8-byte pieces of its
// two rows that the A fragment needs (a quad reads full 32-byte sectors), the plane fragments stay in
// registers for the whole kernel, and nothing goes through shared memory -- the general kernel above spends
// its time in the shared-memory pipe (one 16-byte broadcast load per four FMAs).  After the product a lane
// holds four projections of each of its two rows; the quad exchanges them by shuffles so that lane t owns
// table t, and writes that table's 16 probabilities with 16-byte stores.
// ------------------------------------------------------------------------------------------------
constexpr int kFastThreads = 128;
__global__ void __launch_bounds__(kFastThreads, 4)
bucket_probs_mma_d64_l4k4(const float* __restrict__ x, const float* __restrict__ planes, float* __restrict__ probs,
                          int64_t rows, int64_t T, int heads) {
    constexpr int D = 64, R = 16, LR = 64;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    PlaneFrags pf;
    load_plane_frags(planes, lane, pf);
    const float inv_scale = rsqrtf((float)D);
    const int64_t blocks = (rows + 15) / 16;
    const int64_t warp_global = (int64_t)blockIdx.x * (kFastThreads / 32) + (threadIdx.x >> 5);
    const int64_t warps_total = (int64_t)gridDim.x * (kFastThreads / 32);
    for (int64_t blk = warp_global; blk < blocks; blk += warps_total) {
        const int64_t r0 = blk * 16;
        // the lane's two rows: r0 + g and r0 + g + 8 (rows past the end read as zero and are not written)
        float2 raw[16];
        bool live[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t row = r0 + g + 8 * h;
            live[h] = row < rows;
            const int64_t rr = live[h] ? row : 0;
            const int64_t n = rr / T, tok = rr - n * T;
            const int64_t mb = n / heads, hd = n - mb * heads;
            const float* src = x + ((mb * T + tok) * heads + hd) * D + 2 * t;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                raw[2 * u + h] = live[h] ? __ldcs(reinterpret_cast<const float2*>(src + 8 * u)) : make_float2(0.f, 0.f);
        }
        float c[2][4];
        project_rows(raw, pf, c);
        float vals[2][R];
        table_probs(c, lane, inv_scale, vals);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (live[h]) {
                float* dst = probs + (r0 + g + 8 * h) * LR + t * R;
#pragma unroll
                for (int i = 0; i < R; i += 4)
                    __stcs(reinterpret_cast<float4*>(dst + i),
                           make_float4(vals[h][i], vals[h][i + 1], vals[h][i + 2], vals[h][i + 3]));
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Tensor-core producer for wider geometries (what the bf16 multi-head configuration uses: d_k = 128, L = 8,
// K = 6): the L K projections of a row are a [rows x D] . [D x L K] product on warp-level mma.sync (m16n8k16).
// A warp takes 16 rows at a time; the plane fragments (hi and lo bf16 limbs) live in shared memory as one 16-byte
// item per (plane block, k-step, lane); bf16 rows are exact A operands (two products: x.hi + x.lo), fp32 rows are
// split into limbs (three products).  Two index permutations keep everything in registers without shuffles:
//   * K side: lane t of a quad loads the 16-byte (bf16) or 32-byte (fp32) piece [32 m + 8 t, +8) of its rows and
//     uses it for the k-steps 2 m and 2 m + 1, i.e. "k index" (j, half, 2 t + e) stands for feature
//     32 (j / 2) + 8 t + 4 (j % 2) + 2 half + e; the plane fragments are built with the same map.
//   * N side: after the product lane t holds the columns 8 nt + 2 t + e of its two rows, 2 NT = L K / 4 of them, and
//     the planes are assigned to columns so that these are exactly the K planes of L / 4 whole tables
//     (column slot s = 2 nt + e of lane t = plane s % K of table (L / 4) t + s / K).
// Each lane then forms the R probabilities of its (row, table) pairs by doubling, in bucket order.  The R values
// of a (row, table) are contiguous in the output but the lanes of a warp hold 32 different such pieces, so they go
// through an 8 KB staging buffer of the warp (16-byte pieces XOR-swizzled inside every 128 bytes: writes and reads
// take the minimum number of shared-memory wavefronts) and leave as 512-byte contiguous warp stores.
// ------------------------------------------------------------------------------------------------
template <int D, int L, int K>
struct WideProbs {
    static constexpr int NT = L * K / 8, NJ = D / 16, R = 1 << K, TPL = L / 4;
    static constexpr int kTabBytes = NT * NJ * 32 * 16;
    static constexpr int kStageBytes = 8192;       // per warp
    static_assert(D % 32 == 0 && L % 4 == 0 && (L * K) % 8 == 0, "geometry of the tensor-core producer");
};
constexpr int kWideThreads = 128;

template <int D, int L, int K, typename Tx, typename Tp>
__global__ void __launch_bounds__(kWideThreads, (sizeof(Tx) == 4 ? 3 : 4))
bucket_probs_mma_wide(const Tx* __restrict__ x, const float* __restrict__ planes, Tp* __restrict__ probs,
                      int64_t rows, int64_t T, int heads) {
    using W = WideProbs<D, L, K>;
    constexpr int NT = W::NT, NJ = W::NJ, R = W::R, TPL = W::TPL;
    constexpr bool kX32 = sizeof(Tx) == 4;
    extern __shared__ __align__(16) uint8_t wide_smem[];
    uint4* tab = reinterpret_cast<uint4*>(wide_smem);          // [(nt NJ + j) 32 + lane] = {b0 hi, b1 hi, b0 lo, b1 lo}
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // staging: PB bytes per (row, table); a flush covers 8 rows x kTPF tables = 8 KB, i.e. kPPF passes over tb
    constexpr int PB = R * (int)sizeof(Tp), kTPF = W::kStageBytes / (8 * PB), kPPF = kTPF / 4;
    static_assert(kPPF >= 1 && TPL % kPPF == 0 && PB % 128 == 0, "staging geometry");
    uint8_t* stage = wide_smem + W::kTabBytes + (threadIdx.x >> 5) * W::kStageBytes;
    auto swz = [](int off) {   // 16-byte piece (off >> 4) & 7 of 128-byte block b = off >> 7, XOR (b / 8 + 2 (b % 8)) % 8
        const int b = off >> 7;
        return (b << 7) | (((((off >> 4) & 7) ^ ((b >> 3) + 2 * (b & 7))) & 7) << 4);
    };
    for (int i = threadIdx.x; i < NT * NJ * 32; i += kWideThreads) {
        const int ln = i & 31, f = i >> 5, j = f % NJ, nt = f / NJ;
        const int fg = ln >> 2, ft = ln & 3;                    // the fragment's lane: column 8 nt + fg, k pairs of ft
        const int slot = 2 * nt + (fg & 1), owner = fg >> 1;   // column 8 nt + 2 owner + e
        const int plane = (TPL * owner + slot / K) * K + slot % K;
        const float* src = planes + (int64_t)plane * D + 32 * (j >> 1) + 8 * ft + 4 * (j & 1);
        const float4 v = __ldg(reinterpret_cast<const float4*>(src));
        uint4 w;
        split_pair(v.x, v.y, w.x, w.z);
        split_pair(v.z, v.w, w.y, w.w);
        tab[i] = w;
    }
    __syncthreads();
    const float inv_scale = rsqrtf((float)D);
    const int64_t blocks = (rows + 15) / 16;
    const int64_t warp_global = (int64_t)blockIdx.x * (kWideThreads / 32) + (threadIdx.x >> 5);
    const int64_t warps_total = (int64_t)gridDim.x * (kWideThreads / 32);
    for (int64_t blk = warp_global; blk < blocks; blk += warps_total) {
        const int64_t r0 = blk * 16;
        bool live[2];
        const Tx* src[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t row = r0 + g + 8 * h;
            live[h] = row < rows;
            const int64_t rr = live[h] ? row : 0;
            const int64_t n = rr / T, tok = rr - n * T;
            const int64_t mb = n / heads, hd = n - mb * heads;
            src[h] = x + ((mb * T + tok) * heads + hd) * D + 8 * t;
        }
        float acc[kX32 ? 3 : 2][NT][4];
#pragma unroll
        for (int p = 0; p < (kX32 ? 3 : 2); ++p)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[p][nt][i] = 0.f;
#pragma unroll
        for (int m = 0; m < D / 32; ++m) {
            // the lane's eight features [32 m + 8 t, +8) of both rows: words {k-step 2m: a0|a2, k-step 2m+1: a0|a2}
            uint32_t hi[2][4], lo[2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (kX32) {
                    float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
                    if (live[h]) {
                        v0 = __ldcs(reinterpret_cast<const float4*>(src[h] + 32 * m));
                        v1 = __ldcs(reinterpret_cast<const float4*>(src[h] + 32 * m) + 1);
                    }
                    split_pair(v0.x, v0.y, hi[h][0], lo[h][0]);
                    split_pair(v0.z, v0.w, hi[h][1], lo[h][1]);
                    split_pair(v1.x, v1.y, hi[h][2], lo[h][2]);
                    split_pair(v1.z, v1.w, hi[h][3], lo[h][3]);
                } else {
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (live[h]) v = __ldcs(reinterpret_cast<const uint4*>(src[h] + 32 * m));
                    hi[h][0] = v.x; hi[h][1] = v.y; hi[h][2] = v.z; hi[h][3] = v.w;
                }
            }
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int j = 2 * m + jj;
                const uint32_t ahi[4] = {hi[0][2 * jj], hi[1][2 * jj], hi[0][2 * jj + 1], hi[1][2 * jj + 1]};
                uint32_t alo[4] = {0u, 0u, 0u, 0u};
                if (kX32) {
                    alo[0] = lo[0][2 * jj]; alo[1] = lo[1][2 * jj]; alo[2] = lo[0][2 * jj + 1]; alo[3] = lo[1][2 * jj + 1];
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint4 b = tab[(nt * NJ + j) * 32 + lane];
                    mma_bf16_16816(acc[0][nt], ahi, b.x, b.y);
                    mma_bf16_16816(acc[1][nt], ahi, b.z, b.w);
                    if (kX32) mma_bf16_16816(acc[2][nt], alo, b.x, b.y);
                }
            }
        }
        // the lane's (row, table) pairs, one at a time
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int tb = 0; tb < TPL; ++tb) {
                float p0[K], p1[K];
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    const int s = tb * K + k, nt = s >> 1, i = 2 * h + (s & 1);
                    float pr = acc[0][nt][i] + acc[1][nt][i];
                    if (kX32) pr = acc[0][nt][i] + (acc[1][nt][i] + acc[2][nt][i]);
                    const float e = __expf(-2.f * fabsf(pr));
                    const float th = copysignf(__fdividef(1.f - e, 1.f + e), pr) * inv_scale;
                    const float sq = th * th;
                    const float poly = fmaf(sq, fmaf(sq, fmaf(sq, -17.f / 315.f, 2.f / 15.f), -1.f / 3.f), 1.f);
                    const float half = 0.5f * th * poly;
                    p1[k] = 0.5f + half;
                    p0[k] = 0.5f - half;
                }
                float vals[R];
                vals[0] = p0[0];
                vals[1] = p1[0];
#pragma unroll
                for (int k = 1; k < K; ++k) {
#pragma unroll
                    for (int i = R / 2 - 1; i >= 0; --i) {     // constant bounds: every index is known at compile time
                        if (i < (1 << k)) {
                            const float b = vals[i];
                            vals[2 * i] = b * p0[k];
                            vals[2 * i + 1] = b * p1[k];
                        }
                    }
                }
                // stage the piece: local table kPPF t + (tb % kPPF) of row g
                const int base = g * (kTPF * PB) + (kPPF * t + tb % kPPF) * PB;
                if (sizeof(Tp) == 4) {
#pragma unroll
                    for (int i = 0; i < R; i += 4)
                        *reinterpret_cast<float4*>(stage + swz(base + 4 * i)) =
                            make_float4(vals[i], vals[i + 1], vals[i + 2], vals[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < R; i += 8) {
                        uint4 w;
                        __nv_bfloat162 a = __floats2bfloat162_rn(vals[i], vals[i + 1]);
                        __nv_bfloat162 b = __floats2bfloat162_rn(vals[i + 2], vals[i + 3]);
                        __nv_bfloat162 c = __floats2bfloat162_rn(vals[i + 4], vals[i + 5]);
                        __nv_bfloat162 d = __floats2bfloat162_rn(vals[i + 6], vals[i + 7]);
                        w.x = *reinterpret_cast<uint32_t*>(&a); w.y = *reinterpret_cast<uint32_t*>(&b);
                        w.z = *reinterpret_cast<uint32_t*>(&c); w.w = *reinterpret_cast<uint32_t*>(&d);
                        *reinterpret_cast<uint4*>(stage + swz(base + 2 * i)) = w;
                    }
                }
                if (tb % kPPF == kPPF - 1) {
                    // flush: 16 warp stores of 512 contiguous staged bytes; PB-byte pieces are contiguous in the output
                    const int tb0 = tb - (kPPF - 1);
                    __syncwarp();
#pragma unroll
                    for (int qq = 0; qq < W::kStageBytes / 512; ++qq) {
                        const int off = qq * 512 + lane * 16;
                        const int gr = off / (kTPF * PB), rem = off % (kTPF * PB), lt = rem / PB, inner = rem % PB;
                        const int table = TPL * (lt / kPPF) + tb0 + lt % kPPF;
                        const int64_t row = r0 + gr + 8 * h;
                        const uint4 w = *reinterpret_cast<const uint4*>(stage + swz(off));
                        if (row < rows)
                            __stcs(reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(probs) +
                                                            (row * L + table) * (int64_t)PB + inner), w);
                    }
                    __syncwarp();
                }
            }
        }
    }
}

template <int D, int L, int K, typename Tx, typename Tp>
cudaError_t launch_probs_wide(const void* x, const float* planes, void* probs, int64_t rows, int64_t T, int heads,
                              cudaStream_t stream) {
    auto kern = bucket_probs_mma_wide<D, L, K, Tx, Tp>;
    constexpr int smem = WideProbs<D, L, K>::kTabBytes + (kWideThreads / 32) * WideProbs<D, L, K>::kStageBytes;
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t want = (rows + 63) / 64;   // 64 rows per CTA and pass
    const unsigned blocks = (unsigned)std::min<int64_t>(want, (int64_t)(sms > 0 ? sms : 148) * 12);
    kern<<<blocks, kWideThreads, smem, stream>>>((const Tx*)x, planes, (Tp*)probs, rows, T, heads);
    return cudaGetLastError();
}

template <typename Tx, typename Tp, int K>
cudaError_t launch_probs_k(const void* x, const float* planes, void* probs, int64_t rows, int64_t T, int heads,
                           int d, int L, cudaStream_t stream) {
    const int LR = L << K;
    const bool xreg = d <= 64;
    const int stage_out = (xreg && LR <= 128) ? 1 : 0;
    const size_t tile = (size_t)RB * (size_t)((stage_out && LR > d ? LR : d) + 4);
    const size_t smem = ((size_t)L * K * d + tile) * sizeof(float) + RB * sizeof(int64_t);
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((rows + RB - 1) / RB);
    cudaError_t err;
    if (xreg) {
        auto kern = bucket_probs_kernel<Tx, Tp, K, true>;
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return err;
        kern<<<blocks, RB, smem, stream>>>((const Tx*)x, planes, (Tp*)probs, rows, T, heads, d, L, stage_out);
    } else {
        auto kern = bucket_probs_kernel<Tx, Tp, K, false>;
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return err;
        kern<<<blocks, RB, smem, stream>>>((const Tx*)x, planes, (Tp*)probs, rows, T, heads, d, L, stage_out);
    }
    return cudaGetLastError();
}

template <typename Tx, typename Tp>
cudaError_t launch_probs(const void* x, const float* planes, void* probs, int64_t rows, int64_t T, int heads,
                         int d, int L, int K, cudaStream_t stream) {
    switch (K) {
        case 1: return launch_probs_k<Tx, Tp, 1>(x, planes, probs, rows, T, heads, d, L, stream);
        case 2: return launch_probs_k<Tx, Tp, 2>(x, planes, probs, rows, T, heads, d, L, stream);
        case 3: return launch_probs_k<Tx, Tp, 3>(x, planes, probs, rows, T, heads, d, L, stream);
        case 4: return launch_probs_k<Tx, Tp, 4>(x, planes, probs, rows, T, heads, d, L, stream);
        case 5: return launch_probs_k<Tx, Tp, 5>(x, planes, probs, rows, T, heads, d, L, stream);
        case 6: return launch_probs_k<Tx, Tp, 6>(x, planes, probs, rows, T, heads, d, L, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t bucket_probs(const void* x, const float* planes, void* probs, int64_t rows, int64_t T, int heads,
                         int d, int L, int K, int dtype_x, int dtype_probs, cudaStream_t stream) {
    if (dtype_x == RACE_DTYPE_F32 && dtype_probs == RACE_DTYPE_F32 && d == 64 && L == 4 && K == 4) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int64_t want = (rows + 63) / 64;   // 64 rows per CTA and pass
        const unsigned blocks = (unsigned)std::min<int64_t>(want, (int64_t)(sms > 0 ? sms : 148) * 16);
        bucket_probs_mma_d64_l4k4<<<blocks, kFastThreads, 0, stream>>>((const float*)x, planes, (float*)probs, rows, T,
                                                                       heads);
        return cudaGetLastError();
    }
    if (d == 128 && L == 8 && K == 6) {
        if (dtype_x == RACE_DTYPE_BF16 && dtype_probs == RACE_DTYPE_BF16)
            return launch_probs_wide<128, 8, 6, __nv_bfloat16, __nv_bfloat16>(x, planes, probs, rows, T, heads, stream);
        if (dtype_x == RACE_DTYPE_F32 && dtype_probs == RACE_DTYPE_F32)
            return launch_probs_wide<128, 8, 6, float, float>(x, planes, probs, rows, T, heads, stream);
        if (dtype_x == RACE_DTYPE_F32 && dtype_probs == RACE_DTYPE_BF16)
            return launch_probs_wide<128, 8, 6, float, __nv_bfloat16>(x, planes, probs, rows, T, heads, stream);
        if (dtype_x == RACE_DTYPE_BF16 && dtype_probs == RACE_DTYPE_F32)
            return launch_probs_wide<128, 8, 6, __nv_bfloat16, float>(x, planes, probs, rows, T, heads, stream);
    }
    if (dtype_x == RACE_DTYPE_F32 && dtype_probs == RACE_DTYPE_F32)
        return launch_probs<float, float>(x, planes, probs, rows, T, heads, d, L, K, stream);
    if (dtype_x == RACE_DTYPE_BF16 && dtype_probs == RACE_DTYPE_BF16)
        return launch_probs<__nv_bfloat16, __nv_bfloat16>(x, planes, probs, rows, T, heads, d, L, K, stream);
    if (dtype_x == RACE_DTYPE_F32 && dtype_probs == RACE_DTYPE_BF16)
        return launch_probs<float, __nv_bfloat16>(x, planes, probs, rows, T, heads, d, L, K, stream);
    if (dtype_x == RACE_DTYPE_BF16 && dtype_probs == RACE_DTYPE_F32)
        return launch_probs<__nv_bfloat16, float>(x, planes, probs, rows, T, heads, d, L, K, stream);
    return cudaErrorInvalidValue;
}

}  // namespace race
