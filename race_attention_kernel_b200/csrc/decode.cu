// Incremental (decode) step of the causal per-bucket forward: a few new tokens per stream against a
// running state that stays in device memory between calls.  One step of the reference's chunked
// evaluation (src/race_chunked.py:54-63) with a chunk of 1..64 tokens:
//   A += pK_t ;  B += pK_t (x) v_t ;  out_t = sum_s pQ_t[s] * B[s,:] / (A[s] + eps).
// The work is one read and one write of the state ([S, d_k] + [S] floats per stream): HBM-bound,
// CUDA cores.  One CTA owns one stream.  A thread holds four consecutive columns of B (16-byte
// accesses), d_k/4 lanes cover a row, so a warp covers 32/(d_k/4) rows per access and the eight warps
// of the CTA split the buckets.  The rows of B are requested before the token's A / W / pK are
// staged, eight 16-byte loads per thread in flight, so the state read overlaps the prologue.
#include "launch.h"

namespace race {

namespace {

constexpr int kDecodeThreads = 256;
constexpr int kDecodeWarps = kDecodeThreads / 32;
constexpr int kDecodeCols = 128;   // columns one pass over the state covers (32 lanes x 4)
constexpr int kDecodeDepth = 8;    // 16-byte state loads a thread keeps in flight

__device__ __forceinline__ float ld1(const float* p) { return *p; }
__device__ __forceinline__ float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// grid (N).  state_in may be null (zeros) and may equal state_out: a thread only re-reads state it
// wrote itself, and A is stored after the last read of it.  lpr = lanes per row of B (a power of
// two, >= min(d_k, 128)/4).  Shared memory: 3*S + kDecodeWarps*kDecodeCols floats.
template <typename Tin>
__global__ void __launch_bounds__(kDecodeThreads, 4)
decode_step(const Tin* __restrict__ pq, const Tin* __restrict__ pk, const Tin* __restrict__ v, Tin* __restrict__ out,
            const float* state_in, float* state_out, int T, int S, int D, float eps, int lpr_log2) {
    extern __shared__ __align__(16) float sm[];
    float* a = sm;             // running A
    float* w = sm + S;         // pQ / (A + eps) of the current token
    float* pks = sm + 2 * S;   // pK of the current token
    float* red = sm + 3 * S;   // [warps][128] partial outputs
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int lpr = 1 << lpr_log2;
    const int cl = lane & (lpr - 1);              // column quad of this lane
    const int rows_iter = kDecodeWarps * (32 >> lpr_log2);     // rows of B the CTA covers per access
    const int row0 = warp * (32 >> lpr_log2) + (lane >> lpr_log2);
    const int64_t n = blockIdx.x;
    const int64_t sf = (int64_t)state_floats_per_stream(S, D);
    const float* sin = state_in ? state_in + n * sf : nullptr;
    float* sout = state_out + n * sf;
    const Tin* pq_n = pq + n * (int64_t)T * S;
    const Tin* pk_n = pk + n * (int64_t)T * S;
    const Tin* v_n = v + n * (int64_t)T * D;
    Tin* out_n = out + n * (int64_t)T * D;
    const int slices = (D + kDecodeCols - 1) / kDecodeCols;
    // all rows of a thread fit its registers: B stays there across the tokens and is stored once
    const bool fits = S <= kDecodeDepth * rows_iter;

    for (int slice = 0; slice < slices; ++slice) {
        const int c = slice * kDecodeCols + cl * 4;
        const bool cv = c < D;
        __syncthreads();  // the previous slice is done with a
        for (int s = tid; s < S; s += kDecodeThreads) a[s] = sin ? sin[(int64_t)S * D + s] : 0.f;
        float4 b[kDecodeDepth];
        for (int t = 0; t < T; ++t) {
            // the first token reads the incoming state, later tokens what this thread wrote
            const float* bsrc = (t == 0) ? sin : sout;
            if (!(fits && t > 0)) {
#pragma unroll
                for (int i = 0; i < kDecodeDepth; ++i) {
                    const int s = row0 + i * rows_iter;
                    b[i] = (cv && s < S && bsrc) ? *reinterpret_cast<const float4*>(bsrc + (int64_t)s * D + c)
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            __syncthreads();  // readers of w / pks / red of the previous token are done; a is initialised
            for (int s = tid; s < S; s += kDecodeThreads) {
                const float k = ld1(pk_n + (int64_t)t * S + s);
                const float an = a[s] + k;
                a[s] = an;
                pks[s] = k;
                w[s] = ld1(pq_n + (int64_t)t * S + s) / (an + eps);
            }
            const float4 vv = cv ? load4(v_n + (int64_t)t * D + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            __syncthreads();
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int base = 0; base < S; base += kDecodeDepth * rows_iter) {
#pragma unroll
                for (int i = 0; i < kDecodeDepth; ++i) {
                    const int s = base + row0 + i * rows_iter;
                    if (cv && s < S) {
                        const float k = pks[s], ws = w[s];
                        float4 x = b[i];
                        x.x = fmaf(k, vv.x, x.x); x.y = fmaf(k, vv.y, x.y);
                        x.z = fmaf(k, vv.z, x.z); x.w = fmaf(k, vv.w, x.w);
                        if (!fits || t == T - 1) *reinterpret_cast<float4*>(sout + (int64_t)s * D + c) = x;
                        if (fits) b[i] = x;
                        acc.x = fmaf(ws, x.x, acc.x); acc.y = fmaf(ws, x.y, acc.y);
                        acc.z = fmaf(ws, x.z, acc.z); acc.w = fmaf(ws, x.w, acc.w);
                    }
                    if (fits) continue;
                    const int s2 = s + kDecodeDepth * rows_iter;   // the same slot of the next block of rows
                    b[i] = (cv && s2 < S && bsrc) ? *reinterpret_cast<const float4*>(bsrc + (int64_t)s2 * D + c)
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            // lanes that share a column quad hold different rows: add them up, then the warps
            for (int off = lpr; off < 32; off <<= 1) {
                acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
                acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
                acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
                acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
            }
            if (lane < lpr) *reinterpret_cast<float4*>(red + warp * kDecodeCols + cl * 4) = acc;
            __syncthreads();
            if (tid < lpr && cv) {
                float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int i = 0; i < kDecodeWarps; ++i) {
                    const float4 x = *reinterpret_cast<const float4*>(red + i * kDecodeCols + tid * 4);
                    o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w;
                }
                store4_stream(out_n + (int64_t)t * D + c, o);
            }
        }
    }
    __syncthreads();
    for (int s = tid; s < S; s += kDecodeThreads) sout[(int64_t)S * D + s] = a[s];
}

// One token per stream and a state small enough that a thread holds TWO streams' rows (S <= 4 rows per
// thread): a CTA walks `per_cta` consecutive streams and requests the next stream's state, A, pK and pQ
// while it works on the current one, so the chain prologue -> update -> reduction of a stream no longer
// waits on memory.  grid = ceil(N / per_cta); d_k <= 128; shared memory as decode_step.
template <typename Tin>
__global__ void __launch_bounds__(kDecodeThreads, 4)
decode_step_small(const Tin* __restrict__ pq, const Tin* __restrict__ pk, const Tin* __restrict__ v,
                  Tin* __restrict__ out, const float* state_in, float* state_out, int64_t N, int per_cta, int S,
                  int D, float eps, int lpr_log2) {
    constexpr int kHalf = kDecodeDepth / 2;
    extern __shared__ __align__(16) float sm[];
    float* a = sm;
    float* w = sm + S;
    float* pks = sm + 2 * S;
    float* red = sm + 3 * S;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int lpr = 1 << lpr_log2;
    const int cl = lane & (lpr - 1);
    const int rows_iter = kDecodeWarps * (32 >> lpr_log2);
    const int row0 = warp * (32 >> lpr_log2) + (lane >> lpr_log2);
    const int c = cl * 4;
    const bool cv = c < D;
    const int64_t sf = (int64_t)state_floats_per_stream(S, D);
    const int64_t n_first = (int64_t)blockIdx.x * per_cta;
    const int cnt = (int)min((int64_t)per_cta, N - n_first);

    float4 bn[kHalf];
    float an = 0.f, kn = 0.f, qn = 0.f;
    auto request = [&](int64_t n) {   // state rows, A, pK, pQ of stream n -> registers
        const float* sin = state_in ? state_in + n * sf : nullptr;
#pragma unroll
        for (int i = 0; i < kHalf; ++i) {
            const int s = row0 + i * rows_iter;
            bn[i] = (cv && s < S && sin) ? *reinterpret_cast<const float4*>(sin + (int64_t)s * D + c)
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (tid < S) {
            an = sin ? sin[(int64_t)S * D + tid] : 0.f;
            kn = ld1(pk + n * S + tid);
            qn = ld1(pq + n * S + tid);
        }
    };
    request(n_first);
    for (int i = 0; i < cnt; ++i) {
        const int64_t n = n_first + i;
        float4 b[kHalf];
#pragma unroll
        for (int j = 0; j < kHalf; ++j) b[j] = bn[j];
        const float a0 = an, k0 = kn, q0 = qn;
        const float4 vv = cv ? load4(v + n * D + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (i + 1 < cnt) request(n + 1);
        __syncthreads();   // readers of a / w / pks / red of the previous stream are done
        if (tid < S) {
            const float at = a0 + k0;
            a[tid] = at;
            pks[tid] = k0;
            w[tid] = q0 / (at + eps);
        }
        __syncthreads();
        float* sout = state_out + n * sf;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < kHalf; ++j) {
            const int s = row0 + j * rows_iter;
            if (cv && s < S) {
                const float k = pks[s], ws = w[s];
                float4 x = b[j];
                x.x = fmaf(k, vv.x, x.x); x.y = fmaf(k, vv.y, x.y);
                x.z = fmaf(k, vv.z, x.z); x.w = fmaf(k, vv.w, x.w);
                *reinterpret_cast<float4*>(sout + (int64_t)s * D + c) = x;
                acc.x = fmaf(ws, x.x, acc.x); acc.y = fmaf(ws, x.y, acc.y);
                acc.z = fmaf(ws, x.z, acc.z); acc.w = fmaf(ws, x.w, acc.w);
            }
        }
        for (int off = lpr; off < 32; off <<= 1) {
            acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
            acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
            acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
            acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
        }
        if (lane < lpr) *reinterpret_cast<float4*>(red + warp * kDecodeCols + cl * 4) = acc;
        if (tid < S) sout[(int64_t)S * D + tid] = a[tid];   // own entry, written by this thread above
        __syncthreads();
        if (tid < lpr && cv) {
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kDecodeWarps; ++j) {
                const float4 x = *reinterpret_cast<const float4*>(red + j * kDecodeCols + tid * 4);
                o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w;
            }
            store4_stream(out + n * D + c, o);
        }
    }
}

}  // namespace

int decode_max_tokens() { return 64; }

cudaError_t decode_step_launch(const void* pq, const void* pk, const void* v, void* out, const float* state_in,
                               float* state_out, const Dims& dm, int dtype, cudaStream_t stream) {
    const int width = dm.D < kDecodeCols ? dm.D : kDecodeCols;
    int lpr_log2 = 0;
    while ((4 << lpr_log2) < width) ++lpr_log2;
    const size_t smem = (size_t)(3 * dm.S + kDecodeWarps * kDecodeCols) * sizeof(float);
    const unsigned grid = (unsigned)dm.N;
    const int rows_iter = kDecodeWarps * (32 >> lpr_log2);
    if (dm.T == 1 && dm.D <= kDecodeCols && dm.S <= (kDecodeDepth / 2) * rows_iter && dm.S <= kDecodeThreads) {
        // small states: several streams per CTA, the next stream's loads in flight (about 8 CTAs per SM's worth)
        int sms = 148, dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int64_t per_cta = dm.N / ((int64_t)sms * 8);
        per_cta = per_cta < 1 ? 1 : (per_cta > 16 ? 16 : per_cta);
        const unsigned g = (unsigned)((dm.N + per_cta - 1) / per_cta);
        if (dtype == RACE_DTYPE_BF16)
            decode_step_small<__nv_bfloat16><<<g, kDecodeThreads, smem, stream>>>(
                (const __nv_bfloat16*)pq, (const __nv_bfloat16*)pk, (const __nv_bfloat16*)v, (__nv_bfloat16*)out,
                state_in, state_out, dm.N, (int)per_cta, dm.S, dm.D, dm.eps, lpr_log2);
        else
            decode_step_small<float><<<g, kDecodeThreads, smem, stream>>>(
                (const float*)pq, (const float*)pk, (const float*)v, (float*)out, state_in, state_out, dm.N,
                (int)per_cta, dm.S, dm.D, dm.eps, lpr_log2);
        return cudaGetLastError();
    }
    if (dtype == RACE_DTYPE_BF16)
        decode_step<__nv_bfloat16><<<grid, kDecodeThreads, smem, stream>>>(
            (const __nv_bfloat16*)pq, (const __nv_bfloat16*)pk, (const __nv_bfloat16*)v, (__nv_bfloat16*)out, state_in,
            state_out, (int)dm.T, dm.S, dm.D, dm.eps, lpr_log2);
    else
        decode_step<float><<<grid, kDecodeThreads, smem, stream>>>((const float*)pq, (const float*)pk, (const float*)v,
                                                                  (float*)out, state_in, state_out, (int)dm.T, dm.S,
                                                                  dm.D, dm.eps, lpr_log2);
    return cudaGetLastError();
}

}  // namespace race
