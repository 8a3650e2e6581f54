// tcgen05 / TMEM / TMA causal kernel (placeholder until the kernel lands: reports unsupported).
#include "launch.h"

namespace race {
bool tensor_supported(const Dims&, int) { return false; }
int tensor_chunk_tokens() { return 64; }
int tensor_default_tile_tokens(const Dims&, int, int) { return 1024; }
size_t tensor_workspace_bytes(const Dims&, int, int) { return 0; }
cudaError_t causal_fwd_tensor(const void*, const void*, const void*, void*, const float*, float*,
                              void*, const Dims&, int, int, cudaStream_t, int*) {
    return cudaErrorNotSupported;
}
}  // namespace race
