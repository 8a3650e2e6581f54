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
