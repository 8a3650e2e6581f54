// Bucket-probability producer: x [rows, d_k] -> probs [rows, L, R], R = 2^K.
//   proj[l,k] = x . planes[l*K+k];  th = tanh(proj)/sqrt(d_k)
//   probs[l,r] = softmax_r( sum_k sign(r,k) th[l,k] ),  sign(r,k) = +1 iff bit (K-1-k) of r
// (src/race_baseline.py:41-44).  The softmax over the 2^K sign corners factorises exactly into
// prod_k sigmoid(+-2 th[l,k]) because sum_r exp(z_r) = prod_k (e^th_k + e^-th_k); the kernel
// evaluates that product (the reference checks the same identity numerically,
// src/verify_factorization.py:42-57).
#include "common.cuh"
#include "launch.h"

namespace race {
namespace {

constexpr int RB = 64;  // rows per CTA

template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename Tx, typename Tp, int K>
__global__ void __launch_bounds__(256)
bucket_probs_kernel(const Tx* __restrict__ x, const float* __restrict__ planes, Tp* __restrict__ probs,
                    int64_t rows, int d, int L) {
    constexpr int R = 1 << K;
    extern __shared__ __align__(16) float smem[];
    const int LK = L * K;
    float* sx = smem;                     // [RB][d+1]
    float* sp = sx + RB * (d + 1);        // [LK][d]
    float* sth = sp + LK * d;             // [RB][LK+1]
    const int tid = threadIdx.x;
    const int64_t row0 = (int64_t)blockIdx.x * RB;
    const int valid = (int)min((int64_t)RB, rows - row0);

    for (int i = tid; i < LK * d; i += 256) sp[i] = planes[i];
    for (int i = tid; i < RB * d; i += 256) {
        const int r = i / d, c = i - r * d;
        sx[r * (d + 1) + c] = r < valid ? to_float<Tx>(x[(row0 + r) * d + c]) : 0.f;
    }
    __syncthreads();
    {
        const int r = tid & (RB - 1);
        const float inv_scale = rsqrtf((float)d);
        for (int p = tid / RB; p < LK; p += 256 / RB) {
            float acc = 0.f;
            for (int c = 0; c < d; ++c) acc = fmaf(sx[r * (d + 1) + c], sp[p * d + c], acc);
            sth[r * (LK + 1) + p] = tanhf(acc) * inv_scale;
        }
    }
    __syncthreads();
    for (int item = tid; item < RB * L; item += 256) {
        const int r = item / L, l = item - r * L;
        if (r >= valid) continue;
        float vals[R];
        vals[0] = 1.f;
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const float th = sth[r * (LK + 1) + l * K + k];
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
        Tp* dst = probs + ((row0 + r) * L + l) * (int64_t)R;
#pragma unroll
        for (int i = 0; i < R; ++i) dst[i] = (Tp)vals[i];
    }
}

template <typename Tx, typename Tp>
cudaError_t launch_probs(const void* x, const float* planes, void* probs, int64_t rows, int d, int L,
                         int K, cudaStream_t stream) {
    const size_t smem = (size_t)(RB * (d + 1) + L * K * d + RB * (L * K + 1)) * sizeof(float);
    const unsigned blocks = (unsigned)((rows + RB - 1) / RB);
#define RACE_PROBS_CASE(K_)                                                                        \
    case K_: {                                                                                     \
        auto kern = bucket_probs_kernel<Tx, Tp, K_>;                                               \
        cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                               (int)smem);                                         \
        if (err != cudaSuccess) return err;                                                        \
        kern<<<blocks, 256, smem, stream>>>((const Tx*)x, planes, (Tp*)probs, rows, d, L);         \
        return cudaGetLastError();                                                                 \
    }
    switch (K) {
        RACE_PROBS_CASE(1) RACE_PROBS_CASE(2) RACE_PROBS_CASE(3)
        RACE_PROBS_CASE(4) RACE_PROBS_CASE(5) RACE_PROBS_CASE(6)
        default: return cudaErrorInvalidValue;
    }
#undef RACE_PROBS_CASE
}

}  // namespace

cudaError_t bucket_probs(const void* x, const float* planes, void* probs, int64_t rows, int d, int L,
                         int K, int dtype_x, int dtype_probs, cudaStream_t stream) {
    if (dtype_x == RACE_DTYPE_F32 && dtype_probs == RACE_DTYPE_F32)
        return launch_probs<float, float>(x, planes, probs, rows, d, L, K, stream);
    if (dtype_x == RACE_DTYPE_BF16 && dtype_probs == RACE_DTYPE_BF16)
        return launch_probs<__nv_bfloat16, __nv_bfloat16>(x, planes, probs, rows, d, L, K, stream);
    if (dtype_x == RACE_DTYPE_F32 && dtype_probs == RACE_DTYPE_BF16)
        return launch_probs<float, __nv_bfloat16>(x, planes, probs, rows, d, L, K, stream);
    if (dtype_x == RACE_DTYPE_BF16 && dtype_probs == RACE_DTYPE_F32)
        return launch_probs<__nv_bfloat16, float>(x, planes, probs, rows, d, L, K, stream);
    return cudaErrorInvalidValue;
}

}  // namespace race
