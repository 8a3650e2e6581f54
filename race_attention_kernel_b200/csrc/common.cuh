// Shared device/host helpers of the RACE prefix-path kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/race_b200.h"

namespace race {

// Problem sizes every kernel receives by value.
struct Dims {
    int64_t N;  // streams
    int64_t T;  // tokens per stream
    int S;      // L*R bucket features per token
    int D;      // head dim
    float eps;
    int H = 1;  // heads of the V / out layout: [N/H, T, H, D] (1: the plain [N, T, D])
};

constexpr int kSimtThreads = 256;
constexpr int kSimtChunk = 32;    // tokens per chunk of the CUDA-core kernels
constexpr int kGroupBuckets = 64; // buckets one CTA owns; wider S is split over a cluster

__host__ __device__ inline int state_floats_per_stream(int S, int D) { return S * (D + 1); }

// ---- element access: 4 consecutive elements as float4 -------------------------------------
__device__ __forceinline__ float4 load4(const float* p) {
    return *reinterpret_cast<const float4*>(p);
}
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
}
// streaming (read-once) variants
__device__ __forceinline__ float4 load4_stream(const float* p) {
    return __ldcs(reinterpret_cast<const float4*>(p));
}
__device__ __forceinline__ float4 load4_stream(const __nv_bfloat16* p) {
    uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p));
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
}
__device__ __forceinline__ void store4_stream(float* p, float4 x) {
    __stcs(reinterpret_cast<float4*>(p), x);
}
__device__ __forceinline__ void store4_stream(__nv_bfloat16* p, float4 x) {
    __nv_bfloat162 a = __floats2bfloat162_rn(x.x, x.y);
    __nv_bfloat162 b = __floats2bfloat162_rn(x.z, x.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    __stcs(reinterpret_cast<uint2*>(p), raw);
}

// Copy a [rows x cols_pad] block into shared memory (row stride ld floats) from a row-major
// global matrix of row length `width`: rows [row0, row0+rows_valid) and columns
// [col0, col0+cols_valid); everything else is zero-filled (padded tokens must read as pK = 0
// and a finite V so that they add nothing to the running sums).  cols_* are multiples of 4.
template <typename Tin>
__device__ __forceinline__ void stage_block(float* dst, int ld, const Tin* src, int64_t row0,
                                            int rows, int rows_valid, int width, int col0,
                                            int cols_pad, int cols_valid, int tid, int nthreads) {
    const int vec_per_row = cols_pad >> 2;
    const int total = rows * vec_per_row;
    for (int i = tid; i < total; i += nthreads) {
        const int r = i / vec_per_row;
        const int c = (i - r * vec_per_row) << 2;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows_valid && c < cols_valid)
            x = load4_stream(src + (row0 + r) * (int64_t)width + col0 + c);
        *reinterpret_cast<float4*>(dst + r * ld + c) = x;
    }
}

}  // namespace race
