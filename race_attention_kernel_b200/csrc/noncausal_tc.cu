// Non-causal per-bucket token kernels on the tensor cores (tcgen05 / TMEM), S = 64 buckets, d_k = 64.
//
// Every token-side product of the non-causal path is "rows of a [T, 64] input times one constant
// 64 x 64 matrix of the stream":
//   forward :  out = pQ . E                         (E = Bs / (A + eps))
//   backward:  dPQ = dO . E^T;  dPK = V . dBs^T + dA;  dV = pK . dBs
// (the forward is the second half of the four lines the reference quotes from upstream,
// analysis/hot-path.md:157-162; the gradients are its closed form).  One kernel runs one or three
// such steps per 64-token chunk.  A CTA is one warpgroup that owns a (stream, token tile):
//   * the constant matrices (E, dBs) are split once into bf16 hi + lo limb tiles in shared memory
//     (no-swizzle canonical layout); the same tile image serves as N-major operand (X) and as
//     K-major operand (X^T);
//   * the input rows go global memory -> registers (accumulator-fragment layout) -> bf16 limbs ->
//     tensor memory with tcgen05.st, where tcgen05.mma reads them as its A operand: the token
//     data never touches shared memory;
//   * fp32 inputs run hi.hi + hi.lo + lo.hi (as the causal kernel), bf16 inputs are exact in one
//     limb and run in . X_hi + in . X_lo;
//   * the next item's rows are loaded while the current product runs; up to four CTAs share an SM
//     (128 of the 512 TMEM columns each), which hides the product latency.
// The one device-side wait (MMA completion) is bounded; a wait that runs out raises the CTA's abort
// flag, is recorded in a device status word, and the CTA leaves without storing.
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"

namespace race {
namespace {

constexpr int kNcThreads = 128;
constexpr uint32_t kNcTmemCols = 128;       // A hi (32) | A lo (32) | O (64)
constexpr int kNcTile = 64 * 64 * 2;        // one bf16 limb tile
constexpr int oNcE = 0;                     // [hi | lo]
constexpr int oNcG = oNcE + 2 * kNcTile;    // dBs [hi | lo]
constexpr int oNcDa = oNcG + 2 * kNcTile;   // dA [64] fp32
constexpr int oNcBar = oNcDa + 64 * 4;
constexpr int oNcMisc = oNcBar + 8;         // tmem base, abort flag
constexpr int kNcSmemUsed = oNcMisc + 16 + 1024;
// requested shared memory: at most four CTAs per SM, so that their TMEM allocations always fit
constexpr int kNcSmemBytes = 56 * 1024;
static_assert(kNcSmemUsed <= kNcSmemBytes, "shared-memory map");

__device__ int g_nc_status = 0;   // first bounded wait that ran out (0: none)

struct NcStep {
    const void* in;   // [N, T, 64]
    void* out;        // [N, T, 64]
    int matrix;       // 0: E, 1: dBs
    int transposed;   // 0: out = in . X, 1: out = in . X^T
    int bias;         // 1: add dA[col] (dPK)
};
struct NcArgs {
    NcStep step[3];
    int nsteps;
};

template <typename Tin> struct NcIo;
template <> struct NcIo<float> {
    static constexpr bool kTwoLimbs = true;
    using Frag = float2;
    static __device__ __forceinline__ Frag load(const float* p) { return __ldcs(reinterpret_cast<const float2*>(p)); }
    static __device__ __forceinline__ Frag zero() { return make_float2(0.f, 0.f); }
    static __device__ __forceinline__ void store(float* p, float a, float b) {
        __stcs(reinterpret_cast<float2*>(p), make_float2(a, b));
    }
};
template <> struct NcIo<__nv_bfloat16> {
    static constexpr bool kTwoLimbs = false;
    using Frag = uint32_t;
    static __device__ __forceinline__ Frag load(const __nv_bfloat16* p) {
        return __ldcs(reinterpret_cast<const unsigned int*>(p));
    }
    static __device__ __forceinline__ Frag zero() { return 0u; }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        __stcs(reinterpret_cast<unsigned int*>(p), *reinterpret_cast<unsigned int*>(&h));
    }
};

template <typename Tin>
__global__ void __launch_bounds__(kNcThreads)
nc_rows_tc(const NcArgs args, const float* __restrict__ totals, const float* __restrict__ grads,
           int64_t T, int tile_tokens, float eps) {
    using Io = NcIo<Tin>;
    using Frag = typename Io::Frag;
    extern __shared__ uint8_t smem_raw[];
    Ctx cx;
    cx.sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    cx.sm_u32 = smem_u32(cx.sm);
    cx.bars = oNcBar;
    cx.abort_flag = reinterpret_cast<volatile int*>(cx.sm + oNcMisc + 4);
    cx.status = &g_nc_status;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(cx.sm + oNcMisc);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t n = blockIdx.y;
    const int64_t t_begin = (int64_t)blockIdx.x * tile_tokens;
    const int64_t t_end = min(T, t_begin + (int64_t)tile_tokens);
    const int nch = (int)((t_end - t_begin + 63) / 64);
    const int64_t sf = state_floats_per_stream(64, 64);

    if (tid == 0) {
        *cx.abort_flag = 0;
        mbar_init(cx.bar(0), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(cx.sm_u32 + oNcMisc), "r"(kNcTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // constant matrices of the stream -> limb tiles, element (s, c) at op_off(s, c)
    {
        const float* st = totals + n * sf;
        for (int i = tid; i < 64 * 32; i += kNcThreads) {
            const int s = i >> 5, c = (i & 31) * 2;
            const float inv = 1.f / (st[64 * 64 + s] + eps);
            const float2 b = *reinterpret_cast<const float2*>(st + s * 64 + c);
            uint32_t hi, lo;
            split2(b.x * inv, b.y * inv, hi, lo);
            *reinterpret_cast<uint32_t*>(cx.sm + oNcE + op_off(s, c)) = hi;
            *reinterpret_cast<uint32_t*>(cx.sm + oNcE + kNcTile + op_off(s, c)) = lo;
        }
        if (grads) {
            const float* gr = grads + n * sf;
            for (int i = tid; i < 64 * 32; i += kNcThreads) {
                const int s = i >> 5, c = (i & 31) * 2;
                const float2 b = *reinterpret_cast<const float2*>(gr + s * 64 + c);
                uint32_t hi, lo;
                split2(b.x, b.y, hi, lo);
                *reinterpret_cast<uint32_t*>(cx.sm + oNcG + op_off(s, c)) = hi;
                *reinterpret_cast<uint32_t*>(cx.sm + oNcG + kNcTile + op_off(s, c)) = lo;
            }
            if (tid < 64) reinterpret_cast<float*>(cx.sm + oNcDa)[tid] = gr[64 * 64 + tid];
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t a_hi = tmem, a_lo = tmem + 32, d_o = tmem + 64;

    const int q = lane & 3, rbase = 16 * warp + (lane >> 2);
    const uint32_t lane_base = (uint32_t)(32 * warp) << 16;
    const int nitems = nch * args.nsteps;

    // rows (rbase, rbase + 8) of the item's input chunk in the accumulator-fragment layout
    auto load_item = [&](int item, Frag (&f)[16]) {
        const int c = item / args.nsteps, i = item - c * args.nsteps;
        const int64_t tok0 = t_begin + (int64_t)c * 64;
        const int valid = (int)min((int64_t)64, t_end - tok0);
        const Tin* in_n = reinterpret_cast<const Tin*>(args.step[i].in) + n * T * 64;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = rbase + 8 * h;
            const Tin* prow = in_n + (tok0 + row) * 64 + 2 * q;
#pragma unroll
            for (int x = 0; x < 8; ++x) f[2 * x + h] = row < valid ? Io::load(prow + 8 * x) : Io::zero();
        }
    };

    Frag nxt[16];
    if (nitems > 0) load_item(0, nxt);
    uint32_t parity = 0;
    bool ok = true;
    for (int item = 0; item < nitems && ok; ++item) {
        const int c = item / args.nsteps, i = item - c * args.nsteps;
        const NcStep stp = args.step[i];
        // ---- input rows -> bf16 limbs -> tensor memory (the A operand) ---------------------------
        {
            uint32_t ohi[16], olo[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                if constexpr (Io::kTwoLimbs) split2(nxt[k].x, nxt[k].y, ohi[k], olo[k]);
                else ohi[k] = nxt[k];
            }
            tmem_st_pairs(lane_base + a_hi, ohi);
            if constexpr (Io::kTwoLimbs) tmem_st_pairs(lane_base + a_lo, olo);
            tmem_wait_st();
        }
        tc_fence_before();
        __syncthreads();   // all rows in place; every warp has read the previous item's O
        if (item + 1 < nitems) load_item(item + 1, nxt);   // in flight while the product runs
        if (warp == 0) {
            const uint32_t tile = __shfl_sync(0xffffffffu, cx.sm_u32 + (stp.matrix ? oNcG : oNcE), 0);
            const int transposed = __shfl_sync(0xffffffffu, stp.transposed, 0);
            constexpr uint32_t kLimb = kNcTile >> 4;
            if (elect_one()) {
                tc_fence_after();
                if (!transposed) {   // X as [K = s][N = c]: N-major
                    const uint32_t b = lo_mn(tile);
                    mma_k64_ta<true, kHiMN, 128>(d_o, a_hi, b, kIdescBase | kBmn);
                    mma_k64_ta<false, kHiMN, 128>(d_o, a_hi, b + kLimb, kIdescBase | kBmn);
                    if constexpr (Io::kTwoLimbs) mma_k64_ta<false, kHiMN, 128>(d_o, a_lo, b, kIdescBase | kBmn);
                } else {             // X^T: rows s of X are the N index, c is K: K-major
                    const uint32_t b = lo_k(tile);
                    mma_k64_ta<true, kHiK, 16>(d_o, a_hi, b, kIdescBase);
                    mma_k64_ta<false, kHiK, 16>(d_o, a_hi, b + kLimb, kIdescBase);
                    if constexpr (Io::kTwoLimbs) mma_k64_ta<false, kHiK, 16>(d_o, a_lo, b, kIdescBase);
                }
                mma_commit(cx.bar(0));
            }
            __syncwarp();
        }
        // ---- O: tensor memory -> (+ bias) -> global memory -------------------------------------------
        if (!(ok = wait_bar_warp(cx, 0, parity, 501))) break;
        parity ^= 1;
        float v[32];
        tc_fence_after();
        tmem_ld64(lane_base + d_o, v);
        tc_fence_before();
        const int64_t tok0 = t_begin + (int64_t)c * 64;
        const int valid = (int)min((int64_t)64, t_end - tok0);
        Tin* out_n = reinterpret_cast<Tin*>(stp.out) + n * T * 64;
        const float* da = reinterpret_cast<const float*>(cx.sm + oNcDa);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = rbase + 8 * h;
            if (row < valid) {
                Tin* orow = out_n + (tok0 + row) * 64 + 2 * q;
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    float o0 = v[4 * x + 2 * h], o1 = v[4 * x + 2 * h + 1];
                    if (stp.bias) { o0 += da[8 * x + 2 * q]; o1 += da[8 * x + 2 * q + 1]; }
                    Io::store(orow + 8 * x, o0, o1);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        if (!ok && lane == 0) {
            // products still in flight have to retire before TMEM is freed (bounded)
            mma_commit(cx.bar(0));
            const long long t0 = clock64();
            while (!mbar_try_wait(cx.bar(0), parity) && clock64() - t0 < cx.limit) {}
        }
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kNcTmemCols) : "memory");
    }
}

// Tokens per CTA: four CTAs share an SM, so the grid runs in waves of 4 x sm_count; pick the multiple
// of 64 that minimises waves x (tokens per CTA + the set-up of a CTA, about three chunks' worth: it splits
// the stream's 64 x 64 matrices into limb tiles).
int nc_tile_tokens(const Dims& dm, int sm_count) {
    const int64_t slots = 4 * (int64_t)(sm_count > 0 ? sm_count : 148);
    int best = 64;
    double best_cost = 1e300;
    for (int tile = 4096; tile >= 64; tile -= 64) {
        const int64_t ctas = dm.N * ((dm.T + tile - 1) / tile);
        const int64_t waves = (ctas + slots - 1) / slots;
        const double cost = (double)waves * (tile + 192.0);
        if (cost < best_cost * 0.999) { best_cost = cost; best = tile; }
        if (ctas > 64 * slots) break;
    }
    return best;
}

cudaError_t launch_nc(const NcArgs& args, const float* totals, const float* grads, const Dims& dm, int dtype,
                      int sm_count, cudaStream_t stream) {
    const int tile = nc_tile_tokens(dm, sm_count);
    dim3 grid((unsigned)((dm.T + tile - 1) / tile), (unsigned)dm.N);
    cudaError_t err;
    if (dtype == RACE_DTYPE_F32) {
        err = cudaFuncSetAttribute(nc_rows_tc<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, kNcSmemBytes);
        if (err != cudaSuccess) return err;
        nc_rows_tc<float><<<grid, kNcThreads, kNcSmemBytes, stream>>>(args, totals, grads, dm.T, tile, dm.eps);
    } else {
        err = cudaFuncSetAttribute(nc_rows_tc<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kNcSmemBytes);
        if (err != cudaSuccess) return err;
        nc_rows_tc<__nv_bfloat16><<<grid, kNcThreads, kNcSmemBytes, stream>>>(args, totals, grads, dm.T, tile,
                                                                              dm.eps);
    }
    return cudaGetLastError();
}

}  // namespace

bool noncausal_tensor_supported(const Dims& dm, int dtype) {
    return (dtype == RACE_DTYPE_F32 || dtype == RACE_DTYPE_BF16) && dm.S == 64 && dm.D == 64 && dm.N <= 65535;
}

cudaError_t noncausal_query_tensor(const void* pq, const float* totals, void* out, const Dims& dm, int dtype,
                                   int sm_count, cudaStream_t stream) {
    NcArgs a{};
    a.nsteps = 1;
    a.step[0] = NcStep{pq, out, 0, 0, 0};
    return launch_nc(a, totals, nullptr, dm, dtype, sm_count, stream);
}

cudaError_t noncausal_token_grads_tensor(const void* pk, const void* v, const void* dout, const float* totals,
                                         const float* grads, void* dpq, void* dpk, void* dv, const Dims& dm,
                                         int dtype, int sm_count, cudaStream_t stream) {
    NcArgs a{};
    a.nsteps = 3;
    a.step[0] = NcStep{dout, dpq, 0, 1, 0};   // dPQ = dO . E^T
    a.step[1] = NcStep{v, dpk, 1, 1, 1};      // dPK = V . dBs^T + dA
    a.step[2] = NcStep{pk, dv, 1, 0, 0};      // dV  = pK . dBs
    return launch_nc(a, totals, grads, dm, dtype, sm_count, stream);
}

}  // namespace race
