// Incremental (decode) step of the causal per-bucket forward: a few new tokens per stream against a
// running state that stays in device memory between calls.  One step of the reference's chunked
// evaluation (src/race_chunked.py:54-63) with a chunk of 1..kDecodeMaxTokens tokens:
//   A += pK_t ;  B += pK_t (x) v_t ;  out_t = sum_s pQ_t[s] * B[s,:] / (A[s] + eps).
// The work is one read and one write of the state ([S, d_k] + [S] floats per stream): HBM-bound,
// CUDA cores.  A warp owns 32 consecutive columns of B (128-byte rows), the 8 warps of a CTA split
// the buckets, and a CTA owns a 32-column slice of one stream.
#include "launch.h"

namespace race {

namespace {

constexpr int kDecodeThreads = 256;
constexpr int kDecodeWarps = kDecodeThreads / 32;
constexpr int kDecodeCols = 32;

__device__ __forceinline__ float ld1(const float* p) { return *p; }
__device__ __forceinline__ float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st1(float* p, float x) { *p = x; }
__device__ __forceinline__ void st1(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

// grid (column slices or 1, N).  state_in may be null (zeros) and may equal state_out; in that
// in-place case the launcher gives one CTA per stream, because every slice reads all of A and A is
// rewritten at the end.  Shared memory: 3*S + kDecodeWarps*kDecodeCols floats.
template <typename Tin>
__global__ void __launch_bounds__(kDecodeThreads)
decode_step(const Tin* __restrict__ pq, const Tin* __restrict__ pk, const Tin* __restrict__ v, Tin* __restrict__ out,
            const float* state_in, float* state_out, int T, int S, int D, float eps) {
    extern __shared__ float sm[];
    float* a = sm;             // running A
    float* w = sm + S;         // pQ / (A + eps) of the current token
    float* pks = sm + 2 * S;   // pK of the current token
    float* red = sm + 3 * S;   // [warps][32] partial outputs
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t n = blockIdx.y;
    const int64_t sf = (int64_t)state_floats_per_stream(S, D);
    const float* sin = state_in ? state_in + n * sf : nullptr;
    float* sout = state_out + n * sf;
    const Tin* pq_n = pq + n * (int64_t)T * S;
    const Tin* pk_n = pk + n * (int64_t)T * S;
    const Tin* v_n = v + n * (int64_t)T * D;
    Tin* out_n = out + n * (int64_t)T * D;
    const int slices = (D + kDecodeCols - 1) / kDecodeCols;

    for (int slice = blockIdx.x; slice < slices; slice += gridDim.x) {
        const int c = slice * kDecodeCols + lane;
        const bool cv = c < D;
        __syncthreads();  // the previous slice is done with a / w / pks / red
        for (int s = tid; s < S; s += kDecodeThreads) a[s] = sin ? sin[(int64_t)S * D + s] : 0.f;
        for (int t = 0; t < T; ++t) {
            __syncthreads();
            for (int s = tid; s < S; s += kDecodeThreads) {
                const float k = ld1(pk_n + (int64_t)t * S + s);
                const float an = a[s] + k;
                a[s] = an;
                pks[s] = k;
                w[s] = ld1(pq_n + (int64_t)t * S + s) / (an + eps);
            }
            __syncthreads();
            const float vc = cv ? ld1(v_n + (int64_t)t * D + c) : 0.f;
            // the first token reads the incoming state, later tokens what this thread wrote
            const float* bsrc = (t == 0) ? sin : sout;
            float acc = 0.f;
            if (cv) {
#pragma unroll 4
                for (int s = warp; s < S; s += kDecodeWarps) {
                    float b = bsrc ? bsrc[(int64_t)s * D + c] : 0.f;
                    b = fmaf(pks[s], vc, b);
                    sout[(int64_t)s * D + c] = b;
                    acc = fmaf(w[s], b, acc);
                }
            }
            red[warp * kDecodeCols + lane] = acc;
            __syncthreads();
            if (warp == 0 && cv) {
                float o = 0.f;
#pragma unroll
                for (int i = 0; i < kDecodeWarps; ++i) o += red[i * kDecodeCols + lane];
                st1(out_n + (int64_t)t * D + c, o);
            }
        }
    }
    __syncthreads();
    // every CTA of a stream holds the same A; the first one stores it
    if (blockIdx.x == 0)
        for (int s = tid; s < S; s += kDecodeThreads) sout[(int64_t)S * D + s] = a[s];
}

}  // namespace

int decode_max_tokens() { return 64; }

cudaError_t decode_step_launch(const void* pq, const void* pk, const void* v, void* out, const float* state_in,
                               float* state_out, const Dims& dm, int dtype, cudaStream_t stream) {
    const int slices = (dm.D + kDecodeCols - 1) / kDecodeCols;
    const bool in_place = state_in == state_out;
    const int64_t max_y = 65535;
    const size_t smem = (size_t)(3 * dm.S + kDecodeWarps * kDecodeCols) * sizeof(float);
    for (int64_t n0 = 0; n0 < dm.N; n0 += max_y) {
        const int64_t nn = dm.N - n0 < max_y ? dm.N - n0 : max_y;
        dim3 grid(in_place ? 1 : slices, (unsigned)nn);
        const int64_t sf = state_floats_per_stream(dm.S, dm.D);
        const float* sin = state_in ? state_in + n0 * sf : nullptr;
        float* sout = state_out + n0 * sf;
        const int64_t T = dm.T;
        if (dtype == RACE_DTYPE_BF16) {
            auto* q = (const __nv_bfloat16*)pq + n0 * T * dm.S;
            auto* k = (const __nv_bfloat16*)pk + n0 * T * dm.S;
            auto* vv = (const __nv_bfloat16*)v + n0 * T * dm.D;
            auto* o = (__nv_bfloat16*)out + n0 * T * dm.D;
            decode_step<__nv_bfloat16><<<grid, kDecodeThreads, smem, stream>>>(q, k, vv, o, sin, sout, (int)T, dm.S,
                                                                              dm.D, dm.eps);
        } else {
            auto* q = (const float*)pq + n0 * T * dm.S;
            auto* k = (const float*)pk + n0 * T * dm.S;
            auto* vv = (const float*)v + n0 * T * dm.D;
            auto* o = (float*)out + n0 * T * dm.D;
            decode_step<float><<<grid, kDecodeThreads, smem, stream>>>(q, k, vv, o, sin, sout, (int)T, dm.S, dm.D,
                                                                       dm.eps);
        }
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace race
