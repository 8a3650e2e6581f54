// Causal forward for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc when they need the forward: code running
// while a stream is being captured, code inside a memory-pool or allocator callback, real-time
// loops that forbid allocator locks, and embedders whose device memory is handed out once at
// start-up by another component.  race_b200_causal_fwd asks such a caller for a workspace it may
// have no way to provide.  This entry point runs the same kernels with the workspace taken from
// a fixed array that is part of the library image: nothing is allocated or freed, by the
// runtime, by torch or by any other library, on any call.
//
// Price of that: the array is 16 MiB of device memory on every GPU that loads the library, held
// until the process exits, and shapes whose workspace is larger are refused
// (RACE_ERR_SCRATCH).  All calls share the array, so two calls that overlap on the GPU (different
// streams, or different host threads) race on it; the caller has to order them.  The array keeps
// whatever the previous call left in it; nothing in it has to start at zero, because the tile
// totals pass overwrites every slice the later passes read.
//
// Limits that follow from the per-device address cache below: the device that is current when the
// entry point is called must be the device the stream belongs to (the array of the current device
// is the one handed to the kernels); the cached address is not refreshed after cudaDeviceReset, so
// a process that resets a device must not call this entry point on it afterwards.
#include "launch.h"

namespace {

constexpr size_t kScratchBytes = 16u << 20;
constexpr int kMaxDevices = 64;

// The workspace itself.  In host code this name is only a handle for the runtime's symbol
// table, not a device address: the address each device maps it to comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

// Device address of g_scratch per device ordinal, filled on the first call on that device.
void* g_scratch_addr[kMaxDevices] = {};

int scratch_for_current_device(void** ptr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return RACE_ERR_SHAPE;
    void* p = __atomic_load_n(&g_scratch_addr[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        // once per device, with that device current; two host threads racing here store the
        // same value
        e = cudaGetSymbolAddress(&p, g_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return (int)cudaErrorInvalidSymbol;
        __atomic_store_n(&g_scratch_addr[dev], p, __ATOMIC_RELEASE);
    }
    *ptr = p;
    return RACE_OK;
}

}  // namespace

extern "C" {

size_t race_b200_static_scratch_bytes(void) { return kScratchBytes; }

int race_b200_causal_fwd_static(const void* probs_q, const void* probs_k, const void* v, void* out,
                                const float* carry_in, float* state_out, const RaceShape* shape,
                                int tile_tokens, int variant, void* stream, int* status) {
    if (!shape) return RACE_ERR_NULL;
    if (!race_b200_is_supported(shape, variant)) return RACE_ERR_SHAPE;
    // size check first, before any device memory is touched: the caller gets a definite answer (the
    // automatic tile length behind it reads the current device's SM count, 148 if there is none)
    const size_t need = race_b200_causal_workspace_bytes(shape, tile_tokens, variant);
    if (need > kScratchBytes) return RACE_ERR_SCRATCH;
    void* scratch = nullptr;
    if (shape->n_streams > 0 && shape->seq_len > 0) {
        const int rc = scratch_for_current_device(&scratch);
        if (rc != RACE_OK) return rc;
    }
    return race_b200_causal_fwd(probs_q, probs_k, v, out, carry_in, state_out, scratch,
                                scratch ? kScratchBytes : 0, shape, tile_tokens, variant, stream, status);
}

}  // extern "C"
