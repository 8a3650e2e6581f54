// Shared device helpers of the tcgen05 kernels: PTX wrappers (mbarrier, TMA, tcgen05.mma/ld/st/
// commit, fences), UMMA shared-memory / instruction descriptors for the no-swizzle canonical
// layout, the bounded mbarrier waits and the optional stage tracing.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace race {
namespace {

constexpr long long kWaitCycles = 1ll << 31;   // ~1 s: default bound of every device-side wait

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
// The same loads with an L2 eviction-priority hint (a policy from l2_policy_evict_last / _first)
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_4d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int c0, int c1, int c2, int c3, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy) : "memory");
}
__device__ __forceinline__ void tma_load_5d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int c0, int c1, int c2, int c3, int c4, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4, %5, %6, %7}], [%2], %8;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "l"(policy) : "memory");
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar) : "memory");
}
// 16 lanes x 64 columns of fp32: thread t gets rows (t/4, t/4+8), column pairs 8x + 2(t%4) + {0,1}
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st64(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x256b.x8.b32 [%32], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
        ::"r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31])),
          "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 16 lanes x 32 columns of fp32: thread t gets rows (t/4, t/4+8), column pairs 8x + 2(t%4) + {0,1}, x < 4
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x256b.x4.b32 [%16], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
        ::"r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 16 lanes x 32 columns of packed bf16 pairs (a 16 x 64 slice of an MMA A operand kept in tensor
// memory): register 2y + h of thread t <-> lane t/4 + 8h, column 4y + t%4, i.e. the K-pair
// (8y + 2(t%4), +1) -- the pairs a thread owns in the 16x256b accumulator fragment.  No wait inside.
__device__ __forceinline__ void tmem_st_pairs(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x128b.x8.b32 [%16], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// shared-memory matrix descriptor, no swizzle: 8x(16 B) core matrices of 128 contiguous bytes;
// lbo = byte stride between core matrices along K, sbo = along M/N
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
// The same descriptor split into words so that the issuing thread only adds a constant per
// k-step: hi word is fixed per layout, lo word = (addr >> 4) | (lbo >> 4) << 16.
//   K-major tile  (lbo 128, sbo 1024): 16 K-elements further = +256 B  = +16 in the lo word
//   MN-major tile (lbo 1024, sbo 128): 16 K-elements further = +2048 B = +128 in the lo word
constexpr uint32_t kHiK = (1024u >> 4) | (1u << 14);
constexpr uint32_t kHiMN = (128u >> 4) | (1u << 14);
__device__ __forceinline__ uint32_t lo_k(uint32_t addr) { return ((addr >> 4) & 0x3FFF) | ((128u >> 4) << 16); }
__device__ __forceinline__ uint32_t lo_mn(uint32_t addr) { return ((addr >> 4) & 0x3FFF) | ((1024u >> 4) << 16); }
__device__ __forceinline__ uint64_t desc64(uint32_t hi, uint32_t lo) { return ((uint64_t)hi << 32) | lo; }
template <bool kAccumulate>
__device__ __forceinline__ void mma_issue(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(kAccumulate ? 1u : 0u));
}
// one 64-deep product = 4 k-steps; kAStep / kBStep are the lo-word increments per k-step
template <bool kFirstZero, uint32_t kAHi, uint32_t kAStep, uint32_t kBHi, uint32_t kBStep>
__device__ __forceinline__ void mma_k64(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    if (kFirstZero) mma_issue<false>(d_tmem, desc64(kAHi, a_lo), desc64(kBHi, b_lo), idesc);
    else mma_issue<true>(d_tmem, desc64(kAHi, a_lo), desc64(kBHi, b_lo), idesc);
#pragma unroll
    for (uint32_t k = 1; k < 4; ++k)
        mma_issue<true>(d_tmem, desc64(kAHi, a_lo + k * kAStep), desc64(kBHi, b_lo + k * kBStep), idesc);
}

// The same with the A operand in tensor memory (bf16 pairs, 8 columns per k-step; for M = 64 row r
// lives in lane (r % 16) + 32 (r / 16), like the accumulator).
template <bool kAccumulate>
__device__ __forceinline__ void mma_issue_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(kAccumulate ? 1u : 0u));
}
template <bool kFirstZero, uint32_t kBHi, uint32_t kBStep>
__device__ __forceinline__ void mma_k64_ta(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc) {
    if (kFirstZero) mma_issue_ta<false>(d_tmem, a_tmem, desc64(kBHi, b_lo), idesc);
    else mma_issue_ta<true>(d_tmem, a_tmem, desc64(kBHi, b_lo), idesc);
#pragma unroll
    for (uint32_t k = 1; k < 4; ++k)
        mma_issue_ta<true>(d_tmem, a_tmem + 8 * k, desc64(kBHi, b_lo + k * kBStep), idesc);
}

// instruction descriptor: bf16 x bf16 -> fp32, M = 64, N = 64
constexpr uint32_t kIdescBase = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((64u >> 4) << 24);
constexpr uint32_t kAmn = 1u << 15;  // A operand is M-major
constexpr uint32_t kBmn = 1u << 16;  // B operand is N-major

// byte offset of element (row, col) in a [64][64] bf16 operand tile of 8x8 core matrices
__device__ __forceinline__ uint32_t op_off(int row, int col) {
    return (uint32_t)((((row >> 3) * 8 + (col >> 3)) << 7) + ((row & 7) << 4) + ((col & 7) << 1));
}

__device__ __forceinline__ void split2(float a, float b, uint32_t& hi, uint32_t& lo) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    hi = *reinterpret_cast<uint32_t*>(&h);
    // remainder of both values with one packed fp32x2 add: (a, b) - (hi_a, hi_b)
    const float2 r = __fadd2_rn(make_float2(a, b), make_float2(-__uint_as_float(hi << 16), -__uint_as_float(hi & 0xffff0000u)));
    __nv_bfloat162 l = __floats2bfloat162_rn(r.x, r.y);
    lo = *reinterpret_cast<uint32_t*>(&l);
}

// Optional stage tracing (compiled in with -DRACE_TC_TRACE only): CTA (0,0) records clock64() at
// stage boundaries into a device buffer [role][chunk][stage] for off-line latency analysis.
#ifdef RACE_TC_TRACE
__device__ long long* g_trace_buf = nullptr;
#define RACE_TRACE(role, c, stage)                                                              \
    do {                                                                                        \
        if (g_trace_buf && blockIdx.x == 1 && blockIdx.y == 0 && (threadIdx.x & 31) == 0 && (c) >= 0 && (c) < 32) \
            g_trace_buf[((role) * 32 + (c)) * 8 + (stage)] = clock64();                         \
    } while (0)
#define RACE_TRACE_STUCK(code, bar, parity)                                                     \
    do {                                                                                        \
        if (g_trace_buf && (threadIdx.x & 31) == 0)                                             \
            g_trace_buf[5 * 32 * 8 + (threadIdx.x >> 5)] =                                      \
                (long long)(code) * 10000 + (bar) * 10 + (parity) + 1000000ll * (blockIdx.x + 1); \
    } while (0)
#else
#define RACE_TRACE(role, c, stage) do {} while (0)
#define RACE_TRACE_STUCK(code, bar, parity) do {} while (0)
#endif

struct Ctx {
    uint8_t* sm;        // 1024-aligned shared base (generic pointer)
    uint32_t sm_u32;    // same, shared-window address
    volatile int* abort_flag;
    int* status;
    int bars;           // byte offset of the mbarrier array
    long long limit = kWaitCycles;   // clock cycles after which a wait gives up
    __device__ __forceinline__ uint32_t bar(int i) const { return sm_u32 + bars + i * 8; }
};

// Bounded wait: false if the wait ran out or another role already gave up.
__device__ __forceinline__ bool wait_bar(const Ctx& cx, int bar, uint32_t parity, int code) {
    if (mbar_try_wait(cx.bar(bar), parity)) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try_wait(cx.bar(bar), parity)) {
        if ((++spins & 63) == 0) {
            if (*cx.abort_flag) { RACE_TRACE_STUCK(code, bar, parity); return false; }
            if (clock64() - t0 > cx.limit) {
                *cx.abort_flag = 1;
                if (cx.status) atomicCAS(cx.status, 0, code);
                RACE_TRACE_STUCK(code, bar, parity);
                return false;
            }
        }
    }
    return true;
}

// Two barriers at once (their polls overlap): true when both phases have completed.
__device__ __forceinline__ bool wait_bar2(const Ctx& cx, int bar_a, uint32_t parity_a, int bar_b,
                                          uint32_t parity_b, int code) {
    bool a = mbar_try_wait(cx.bar(bar_a), parity_a), b = mbar_try_wait(cx.bar(bar_b), parity_b);
    if (a && b) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (true) {
        if (!a) a = mbar_try_wait(cx.bar(bar_a), parity_a);
        if (!b) b = mbar_try_wait(cx.bar(bar_b), parity_b);
        if (a && b) return true;
        if ((++spins & 63) == 0) {
            if (*cx.abort_flag) { RACE_TRACE_STUCK(code, a ? bar_b : bar_a, 0); return false; }
            if (clock64() - t0 > cx.limit) {
                *cx.abort_flag = 1;
                if (cx.status) atomicCAS(cx.status, 0, code);
                RACE_TRACE_STUCK(code, a ? bar_b : bar_a, 0);
                return false;
            }
        }
    }
}

// Warp-uniform flavour: every lane gets the same answer, so .aligned instructions that follow
// are never reached by a part of the warp only.
__device__ __forceinline__ bool wait_bar_warp(const Ctx& cx, int bar, uint32_t parity, int code) {
    return __all_sync(0xffffffffu, wait_bar(cx, bar, parity, code));
}

}  // namespace
}  // namespace race
