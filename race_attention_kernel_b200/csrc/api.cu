// extern "C" entry points: argument validation, workspace bookkeeping and dispatch to the
// kernel families.  Nothing here synchronises or allocates, except the *_host entry point.
#include <cstdio>
#include <cstring>

#include "launch.h"

using namespace race;

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int elt_bytes(int dtype) { return dtype == RACE_DTYPE_BF16 ? 2 : 4; }

// Shape checks shared by every entry point.  Rows of probs ([S] elements) and of V ([d_k]
// elements) must be multiples of 16 bytes: all tile loads are 16-byte vector or TMA loads.
int check_shape(const RaceShape* sh, Dims* dm) {
    if (!sh) return RACE_ERR_NULL;
    if (sh->dtype != RACE_DTYPE_F32 && sh->dtype != RACE_DTYPE_BF16) return RACE_ERR_SHAPE;
    if (sh->heads < 0) return RACE_ERR_SHAPE;
    if (sh->n_streams < 0 || sh->seq_len < 0) return RACE_ERR_SHAPE;
    if (sh->n_tables <= 0 || sh->n_buckets <= 0 || sh->head_dim <= 0) return RACE_ERR_SHAPE;
    if ((int64_t)sh->n_tables * sh->n_buckets > 4096) return RACE_ERR_SHAPE;
    if (!(sh->eps >= 0.f)) return RACE_ERR_SHAPE;
    dm->N = sh->n_streams;
    dm->T = sh->seq_len;
    dm->S = sh->n_tables * sh->n_buckets;
    dm->D = sh->head_dim;
    dm->eps = sh->eps;
    dm->H = sh->heads > 1 ? sh->heads : 1;
    if (dm->N % dm->H != 0) return RACE_ERR_SHAPE;
    const int eb = elt_bytes(sh->dtype);
    if ((dm->S * eb) % 16 != 0 || (dm->D * eb) % 16 != 0) return RACE_ERR_ALIGN;
    return RACE_OK;
}

int sm_count() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms > 0 ? sms : 148;
}

// the single-pass form exists for the fp32 tensor kernels; everything else about it is the TENSOR family
inline bool is_single_pass(int variant) { return variant == RACE_VARIANT_TENSOR_SINGLE_PASS; }
inline int family(int variant) { return is_single_pass(variant) ? RACE_VARIANT_TENSOR : variant; }

int resolve_variant(const Dims& dm, int dtype, int variant) {
    if (variant == RACE_VARIANT_AUTO)
        return tensor_supported(dm, dtype) ? RACE_VARIANT_TENSOR : RACE_VARIANT_SIMT;
    return variant;
}

bool variant_supported(const Dims& dm, int dtype, int variant) {
    // the heads layout of V / out is read by tensor kernels only: fp32 (S = 64, d_k = 64) and bf16 with four or eight
    // bucket groups (tensor_supported says which); the single-pass form is fp32
    if (dm.H > 1 && family(variant) != RACE_VARIANT_TENSOR) return false;
    if (variant == RACE_VARIANT_SIMT) return simt_supported(dm);
    if (variant == RACE_VARIANT_TENSOR) return tensor_supported(dm, dtype);
    if (is_single_pass(variant)) return dtype == RACE_DTYPE_F32 && tensor_supported(dm, dtype);
    return false;
}

int chunk_of(int variant) { return family(variant) == RACE_VARIANT_TENSOR ? tensor_chunk_tokens() : kSimtChunk; }

int pick_tile(const Dims& dm, int dtype, int variant) {
    if (is_single_pass(variant)) return tensor_single_pass_tile_tokens(dm, sm_count());
    if (variant == RACE_VARIANT_TENSOR) return tensor_default_tile_tokens(dm, dtype, sm_count());
    return simt_default_tile_tokens(dm, sm_count());
}

size_t workspace_bytes_for(const Dims& dm, int dtype, int variant, int tile, bool totals_or_resume = false) {
    if (dm.T == 0 || dm.N == 0) return 0;
    if (is_single_pass(variant) && !totals_or_resume) return tensor_single_pass_workspace_bytes(dm, tile);
    if (family(variant) == RACE_VARIANT_TENSOR) return tensor_workspace_bytes(dm, dtype, tile);
    const int64_t tiles = (dm.T + tile - 1) / tile;
    return (size_t)dm.N * tiles * state_floats_per_stream(dm.S, dm.D) * sizeof(float);
}

}  // namespace

extern "C" {

int race_b200_version(void) { return 1008; }

const char* race_b200_error_string(int code) {
    switch (code) {
        case RACE_OK: return "ok";
        case RACE_ERR_NULL: return "a required pointer is NULL";
        case RACE_ERR_SHAPE: return "shape outside the supported range";
        case RACE_ERR_ALIGN: return "pointer or row not 16-byte aligned";
        case RACE_ERR_WORKSPACE: return "workspace too small";
        case RACE_ERR_TILE: return "tile_tokens is not a positive multiple of the chunk length";
        case RACE_ERR_VARIANT: return "kernel variant unknown or unavailable for this shape";
        case RACE_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
        case RACE_ERR_SCRATCH: return "shape needs more workspace than the built-in scratch array holds";
        default: break;
    }
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "unknown error";
}

int race_b200_is_supported(const RaceShape* shape, int variant) {
    Dims dm;
    if (check_shape(shape, &dm) != RACE_OK) return 0;
    const int var = resolve_variant(dm, shape->dtype, variant);
    return variant_supported(dm, shape->dtype, var) ? 1 : 0;
}

size_t race_b200_state_floats(const RaceShape* shape) {
    Dims dm;
    if (check_shape(shape, &dm) != RACE_OK) return 0;
    return (size_t)dm.N * state_floats_per_stream(dm.S, dm.D);
}

int race_b200_select_tile_tokens(const RaceShape* shape, int variant, int* tile_tokens) {
    Dims dm;
    if (!tile_tokens) return RACE_ERR_NULL;
    int rc = check_shape(shape, &dm);
    if (rc != RACE_OK) return rc;
    const int var = resolve_variant(dm, shape->dtype, variant);
    if (!variant_supported(dm, shape->dtype, var)) return RACE_ERR_VARIANT;
    *tile_tokens = pick_tile(dm, shape->dtype, var);
    return RACE_OK;
}

size_t race_b200_causal_workspace_bytes(const RaceShape* shape, int tile_tokens, int variant) {
    Dims dm;
    if (check_shape(shape, &dm) != RACE_OK) return 0;
    const int var = resolve_variant(dm, shape->dtype, variant);
    if (!variant_supported(dm, shape->dtype, var)) return 0;
    const int tile = tile_tokens > 0 ? tile_tokens : pick_tile(dm, shape->dtype, var);
    return workspace_bytes_for(dm, shape->dtype, var, tile);
}

static int causal_entry(const void* probs_q, const void* probs_k, const void* v, void* out,
                        const float* carry_in, float* state_out, void* workspace,
                        size_t workspace_bytes, const RaceShape* shape, int tile_tokens,
                        int variant, void* stream, int* status, int phases, bool global_norm = false,
                        long long wait_cycles = 0, int withhold_chunk = -1) {
    Dims dm;
    int rc = check_shape(shape, &dm);
    if (rc != RACE_OK) return rc;
    const int var = resolve_variant(dm, shape->dtype, variant);
    if (var != RACE_VARIANT_SIMT && var != RACE_VARIANT_TENSOR && !is_single_pass(var)) return RACE_ERR_VARIANT;
    if (!variant_supported(dm, shape->dtype, var)) return var == variant ? RACE_ERR_VARIANT : RACE_ERR_SHAPE;
    // the global-normalisation form runs on the CUDA-core kernels and on the fp32 tensor kernels
    // the global-normalisation form: CUDA-core kernels, fp32 tensor kernels, bf16 tensor kernels with one bucket group
    if (global_norm && family(var) == RACE_VARIANT_TENSOR && shape->dtype != RACE_DTYPE_F32 && dm.S != 64)
        return RACE_ERR_VARIANT;
    if (tile_tokens < 0) return RACE_ERR_TILE;
    const int tile = tile_tokens > 0 ? tile_tokens : pick_tile(dm, shape->dtype, var);
    if (tile % chunk_of(var) != 0) return RACE_ERR_TILE;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sf = (size_t)dm.N * state_floats_per_stream(dm.S, dm.D);
    const bool want_out = (phases & kPhaseOutput) != 0;
    if (!want_out && !state_out) return RACE_ERR_NULL;
    if (dm.N == 0) return RACE_OK;
    if (dm.T == 0) {
        // nothing to launch: the state passes through
        if (state_out) {
            cudaError_t e = carry_in
                ? cudaMemcpyAsync(state_out, carry_in, sf * sizeof(float), cudaMemcpyDeviceToDevice, st)
                : cudaMemsetAsync(state_out, 0, sf * sizeof(float), st);
            return (int)e;
        }
        return RACE_OK;
    }
    if (!probs_k || !v || !workspace || (want_out && (!probs_q || !out))) return RACE_ERR_NULL;
    if (!aligned16(probs_q) || !aligned16(probs_k) || !aligned16(v) || !aligned16(out) ||
        !aligned16(workspace) || !aligned16(carry_in) || !aligned16(state_out))
        return RACE_ERR_ALIGN;
    if (workspace_bytes < workspace_bytes_for(dm, shape->dtype, var, tile, /*totals_or_resume=*/phases != kPhaseAll))
        return RACE_ERR_WORKSPACE;
    if (family(var) == RACE_VARIANT_TENSOR)
        return (int)causal_fwd_tensor(probs_q, probs_k, v, out, carry_in, state_out, workspace,
                                      /*single_pass=*/is_single_pass(var) && phases == kPhaseAll,
                                      dm, shape->dtype, tile, st, status, phases, global_norm, wait_cycles,
                                      withhold_chunk);
    return (int)causal_fwd_simt(probs_q, probs_k, v, out, carry_in, state_out, (float*)workspace,
                                dm, shape->dtype, tile, /*totals_only=*/!want_out, st,
                                /*skip_output=*/false, /*skip_totals=*/!(phases & kPhaseTotals), global_norm);
}

int race_b200_causal_fwd(const void* probs_q, const void* probs_k, const void* v, void* out,
                         const float* carry_in, float* state_out, void* workspace,
                         size_t workspace_bytes, const RaceShape* shape, int tile_tokens,
                         int variant, void* stream, int* status) {
    return causal_entry(probs_q, probs_k, v, out, carry_in, state_out, workspace, workspace_bytes,
                        shape, tile_tokens, variant, stream, status, kPhaseAll);
}

int race_b200_tile_totals(const void* probs_k, const void* v, float* totals, void* workspace,
                          size_t workspace_bytes, const RaceShape* shape, int tile_tokens,
                          int variant, void* stream, int* status) {
    return causal_entry(nullptr, probs_k, v, nullptr, nullptr, totals, workspace, workspace_bytes,
                        shape, tile_tokens, variant, stream, status, kPhaseTotals);
}

int race_b200_causal_fwd_resume(const void* probs_q, const void* probs_k, const void* v, void* out,
                                const float* carry_in, float* state_out, void* workspace,
                                size_t workspace_bytes, const RaceShape* shape, int tile_tokens,
                                int variant, void* stream, int* status) {
    return causal_entry(probs_q, probs_k, v, out, carry_in, state_out, workspace, workspace_bytes,
                        shape, tile_tokens, variant, stream, status, kPhaseOutput);
}

int race_b200_causal_fwd_global(const void* probs_q, const void* probs_k, const void* v, void* out,
                                const float* carry_in, float* state_out, void* workspace,
                                size_t workspace_bytes, const RaceShape* shape, int tile_tokens, int variant,
                                void* stream, int* status) {
    // AUTO: the tensor kernels where they have this form (fp32 S = 64, d_k = 64; bf16 S = 64), else the CUDA cores
    if (variant == RACE_VARIANT_AUTO && shape && shape->dtype != RACE_DTYPE_F32 &&
        shape->n_tables * shape->n_buckets != 64)
        variant = RACE_VARIANT_SIMT;
    return causal_entry(probs_q, probs_k, v, out, carry_in, state_out, workspace, workspace_bytes, shape,
                        tile_tokens, variant, stream, status, kPhaseAll, /*global_norm=*/true);
}

int race_b200_qkv_is_supported(const RaceShape* shape, int n_planes) {
    Dims dm;
    if (check_shape(shape, &dm) != RACE_OK) return 0;
    return (n_planes == 4 && shape->n_buckets == (1 << n_planes) &&
            tensor_qkv_supported(dm, shape->dtype, shape->n_tables, shape->n_buckets)) ? 1 : 0;
}

int race_b200_causal_fwd_qkv(const void* q, const void* k, const void* v, const float* planes, void* out,
                             const float* carry_in, float* state_out, void* workspace, size_t workspace_bytes,
                             const RaceShape* shape, int n_planes, int tile_tokens, int global_norm, void* stream,
                             int* status) {
    Dims dm;
    int rc = check_shape(shape, &dm);
    if (rc != RACE_OK) return rc;
    if (n_planes <= 0 || n_planes > 12 || shape->n_buckets != (1 << n_planes)) return RACE_ERR_SHAPE;
    if (!tensor_qkv_supported(dm, shape->dtype, shape->n_tables, shape->n_buckets)) return RACE_ERR_VARIANT;
    if (tile_tokens < 0) return RACE_ERR_TILE;
    const int tile = tile_tokens > 0 ? tile_tokens : pick_tile(dm, shape->dtype, RACE_VARIANT_TENSOR);
    if (tile % tensor_chunk_tokens() != 0) return RACE_ERR_TILE;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sf = (size_t)dm.N * state_floats_per_stream(dm.S, dm.D);
    if (dm.N == 0) return RACE_OK;
    if (dm.T == 0) {
        if (state_out) {
            cudaError_t e = carry_in
                ? cudaMemcpyAsync(state_out, carry_in, sf * sizeof(float), cudaMemcpyDeviceToDevice, st)
                : cudaMemsetAsync(state_out, 0, sf * sizeof(float), st);
            return (int)e;
        }
        return RACE_OK;
    }
    if (!q || !k || !v || !planes || !out || !workspace) return RACE_ERR_NULL;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(planes) ||
        !aligned16(workspace) || !aligned16(carry_in) || !aligned16(state_out))
        return RACE_ERR_ALIGN;
    if (workspace_bytes < workspace_bytes_for(dm, shape->dtype, RACE_VARIANT_TENSOR, tile)) return RACE_ERR_WORKSPACE;
    return (int)causal_fwd_qkv_tensor(q, k, v, planes, out, carry_in, state_out, workspace, dm, tile, st, status,
                                      kPhaseAll, global_norm != 0);
}

int race_b200_selftest_bounded_wait(const void* probs_q, const void* probs_k, const void* v, void* out,
                                    void* workspace, size_t workspace_bytes, const RaceShape* shape, int variant,
                                    int64_t wait_cycles, int withhold_chunk, void* stream, int* status) {
    if (!status) return RACE_ERR_NULL;
    if (wait_cycles < 1000 || wait_cycles > (1ll << 31) || withhold_chunk < 0) return RACE_ERR_SHAPE;
    if (!shape || shape->dtype != RACE_DTYPE_F32 || family(variant) != RACE_VARIANT_TENSOR) return RACE_ERR_VARIANT;
    return causal_entry(probs_q, probs_k, v, out, nullptr, nullptr, workspace, workspace_bytes, shape, 0,
                        variant, stream, status, kPhaseAll, false, wait_cycles, withhold_chunk);
}

size_t race_b200_causal_bwd_workspace_bytes(const RaceShape* shape) {
    Dims dm;
    if (check_shape(shape, &dm) != RACE_OK || !causal_bwd_supported(dm)) return 0;
    return causal_bwd_workspace_bytes(dm, shape->dtype, causal_bwd_tile_tokens(dm, shape->dtype, sm_count()));
}

int race_b200_causal_bwd(const void* probs_q, const void* probs_k, const void* v, const void* d_out,
                         void* d_probs_q, void* d_probs_k, void* d_v, void* workspace, size_t workspace_bytes,
                         const RaceShape* shape, void* stream, int* status) {
    return race_b200_causal_bwd_carry(probs_q, probs_k, v, d_out, nullptr, nullptr, d_probs_q, d_probs_k, d_v, nullptr,
                                      workspace, workspace_bytes, shape, stream, status);
}

int race_b200_causal_bwd_carry(const void* probs_q, const void* probs_k, const void* v, const void* d_out,
                               const float* carry_in, const float* d_state_out, void* d_probs_q, void* d_probs_k,
                               void* d_v, float* d_carry_in, void* workspace, size_t workspace_bytes,
                               const RaceShape* shape, void* stream, int* status) {
    Dims dm;
    int rc = check_shape(shape, &dm);
    if (rc != RACE_OK) return rc;
    if (!causal_bwd_supported(dm)) return RACE_ERR_SHAPE;
    if (dm.N == 0) return RACE_OK;
    if (dm.T == 0) {   // no tokens: the state passes through, and so does its gradient
        if (!d_carry_in) return RACE_OK;
        const size_t sfb = (size_t)dm.N * state_floats_per_stream(dm.S, dm.D) * sizeof(float);
        return (int)(d_state_out ? cudaMemcpyAsync(d_carry_in, d_state_out, sfb, cudaMemcpyDeviceToDevice, (cudaStream_t)stream)
                                 : cudaMemsetAsync(d_carry_in, 0, sfb, (cudaStream_t)stream));
    }
    if (!probs_q || !probs_k || !v || !d_out || !d_probs_q || !d_probs_k || !d_v || !workspace) return RACE_ERR_NULL;
    if (!aligned16(carry_in) || !aligned16(d_state_out) || !aligned16(d_carry_in)) return RACE_ERR_ALIGN;
    if (!aligned16(probs_q) || !aligned16(probs_k) || !aligned16(v) || !aligned16(d_out) || !aligned16(d_probs_q) ||
        !aligned16(d_probs_k) || !aligned16(d_v) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return RACE_ERR_ALIGN;
    const int tile = causal_bwd_tile_tokens(dm, shape->dtype, sm_count());
    if (workspace_bytes < causal_bwd_workspace_bytes(dm, shape->dtype, tile)) return RACE_ERR_WORKSPACE;
    return (int)causal_bwd_simt(probs_q, probs_k, v, d_out, carry_in, d_state_out, d_probs_q, d_probs_k, d_v,
                                d_carry_in, workspace, dm, shape->dtype, tile, (cudaStream_t)stream, status);
}

int race_b200_decode_step(const void* probs_q, const void* probs_k, const void* v, void* out,
                          const float* state_in, float* state_out, const RaceShape* shape, void* stream) {
    Dims dm;
    int rc = check_shape(shape, &dm);
    if (rc != RACE_OK) return rc;
    if (dm.H > 1 || dm.S > 2048 || dm.T > decode_max_tokens() || dm.N > 0x7fffffff) return RACE_ERR_SHAPE;
    if (!state_out) return RACE_ERR_NULL;
    if (dm.N == 0) return RACE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sf = (size_t)dm.N * state_floats_per_stream(dm.S, dm.D);
    if (dm.T == 0) {
        if (state_in == state_out) return RACE_OK;
        return (int)(state_in ? cudaMemcpyAsync(state_out, state_in, sf * sizeof(float), cudaMemcpyDeviceToDevice, st)
                              : cudaMemsetAsync(state_out, 0, sf * sizeof(float), st));
    }
    if (!probs_q || !probs_k || !v || !out) return RACE_ERR_NULL;
    if (!aligned16(probs_q) || !aligned16(probs_k) || !aligned16(v) || !aligned16(out) || !aligned16(state_in) ||
        !aligned16(state_out))
        return RACE_ERR_ALIGN;
    return (int)decode_step_launch(probs_q, probs_k, v, out, state_in, state_out, dm, shape->dtype, st);
}

namespace {
// tile length of the totals pass of the non-causal path: with many streams one tile per stream (no scan
// over tiles is needed then); never longer than the automatic choice allows the workspace to be
int noncausal_totals_tile(const RaceShape* shape, const Dims& dm) {
    int tile = 0;
    if (race_b200_select_tile_tokens(shape, RACE_VARIANT_AUTO, &tile) != RACE_OK || tile <= 0) return 0;
    const int64_t sms = sm_count();
    while (tile < 16384 && tile < dm.T && dm.N * ((dm.T + 2 * tile - 1) / (2 * tile)) >= 2 * sms) tile *= 2;
    return tile;
}
}  // namespace

int race_b200_noncausal_fwd(const void* probs_q, const void* probs_k, const void* v, void* out,
                            float* totals, void* workspace, size_t workspace_bytes,
                            const RaceShape* shape, void* stream) {
    Dims dm;
    int rc = check_shape(shape, &dm);
    if (rc != RACE_OK) return rc;
    if (!simt_supported(dm) || dm.H > 1) return RACE_ERR_SHAPE;
    if (dm.N == 0) return RACE_OK;
    if (!totals) return RACE_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sf = (size_t)dm.N * state_floats_per_stream(dm.S, dm.D);
    if (dm.T == 0) return (int)cudaMemsetAsync(totals, 0, sf * sizeof(float), st);
    if (!probs_q || !probs_k || !v || !out || !workspace) return RACE_ERR_NULL;
    if (!aligned16(probs_q) || !aligned16(probs_k) || !aligned16(v) || !aligned16(out) ||
        !aligned16(totals) || !aligned16(workspace))
        return RACE_ERR_ALIGN;
    rc = race_b200_tile_totals(probs_k, v, totals, workspace, workspace_bytes, shape,
                               noncausal_totals_tile(shape, dm), RACE_VARIANT_AUTO, stream, nullptr);
    if (rc != RACE_OK) return rc;
    if (noncausal_tensor_supported(dm, shape->dtype))
        return (int)noncausal_query_tensor(probs_q, totals, out, dm, shape->dtype, sm_count(), st);
    return (int)noncausal_query(probs_q, totals, out, dm, shape->dtype, sm_count(), st);
}

size_t race_b200_noncausal_bwd_workspace_bytes(const RaceShape* shape) {
    Dims dm;
    if (check_shape(shape, &dm) != RACE_OK || !simt_supported(dm)) return 0;
    const size_t sf = (size_t)dm.N * state_floats_per_stream(dm.S, dm.D) * sizeof(float);
    const size_t tile_ws = race_b200_causal_workspace_bytes(shape, 0, RACE_VARIANT_AUTO);
    return (tile_ws + 255) / 256 * 256 + 2 * ((sf + 255) / 256 * 256);
}

int race_b200_noncausal_bwd(const void* probs_q, const void* probs_k, const void* v,
                            const float* totals, const void* d_out, void* d_probs_q,
                            void* d_probs_k, void* d_v, void* workspace, size_t workspace_bytes,
                            const RaceShape* shape, void* stream) {
    Dims dm;
    int rc = check_shape(shape, &dm);
    if (rc != RACE_OK) return rc;
    if (!simt_supported(dm) || dm.H > 1) return RACE_ERR_SHAPE;
    if (dm.N == 0 || dm.T == 0) return RACE_OK;
    if (!probs_q || !probs_k || !v || !totals || !d_out || !d_probs_q || !d_probs_k || !d_v ||
        !workspace)
        return RACE_ERR_NULL;
    if (!aligned16(probs_q) || !aligned16(probs_k) || !aligned16(v) || !aligned16(totals) ||
        !aligned16(d_out) || !aligned16(d_probs_q) || !aligned16(d_probs_k) || !aligned16(d_v) ||
        !aligned16(workspace))
        return RACE_ERR_ALIGN;
    if (workspace_bytes < race_b200_noncausal_bwd_workspace_bytes(shape)) return RACE_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sfb = ((size_t)dm.N * state_floats_per_stream(dm.S, dm.D) * sizeof(float) + 255) / 256 * 256;
    const size_t tile_ws = race_b200_causal_workspace_bytes(shape, 0, RACE_VARIANT_AUTO);
    // layout: [tile workspace | dE state | (dBs, dA) state], each part 256-byte aligned
    float* ws_tiles = (float*)workspace;
    float* dE_state = (float*)((char*)workspace + ((tile_ws + 255) / 256 * 256));
    float* grads = (float*)((char*)dE_state + sfb);
    // dE = pQ^T dO : the tile-totals pass with (pQ, dO) in the roles of (pK, V)
    rc = race_b200_tile_totals(probs_q, d_out, dE_state, ws_tiles, tile_ws, shape,
                               noncausal_totals_tile(shape, dm), RACE_VARIANT_AUTO, stream, nullptr);
    if (rc != RACE_OK) return rc;
    cudaError_t e = noncausal_state_grads(totals, dE_state, grads, dm, st);
    if (e != cudaSuccess) return (int)e;
    if (noncausal_tensor_supported(dm, shape->dtype))
        return (int)noncausal_token_grads_tensor(probs_k, v, d_out, totals, grads, d_probs_q, d_probs_k, d_v,
                                                 dm, shape->dtype, sm_count(), st);
    return (int)noncausal_token_grads(probs_k, v, d_out, totals, grads, d_probs_q, d_probs_k, d_v, dm,
                                      shape->dtype, sm_count(), st);
}

namespace {
int probs_entry(const void* x, const float* planes, void* probs, int64_t outer, int64_t seq_len, int32_t heads,
                int32_t d_k, int32_t n_tables, int32_t n_bits, int32_t dtype_x, int32_t dtype_probs,
                void* stream) {
    if (outer < 0 || seq_len < 0 || heads < 1 || d_k < 4 || d_k > 256 || (d_k & (d_k - 1)) || n_tables <= 0 ||
        n_bits < 1 || n_bits > 6 || n_tables * n_bits > 64)
        return RACE_ERR_SHAPE;
    if ((dtype_x != RACE_DTYPE_F32 && dtype_x != RACE_DTYPE_BF16) ||
        (dtype_probs != RACE_DTYPE_F32 && dtype_probs != RACE_DTYPE_BF16))
        return RACE_ERR_SHAPE;
    const int64_t rows = outer * heads * seq_len;
    if (rows == 0) return RACE_OK;
    if (!x || !planes || !probs) return RACE_ERR_NULL;
    if (!aligned16(x) || !aligned16(planes) || !aligned16(probs)) return RACE_ERR_ALIGN;
    return (int)bucket_probs(x, planes, probs, rows, seq_len, heads, d_k, n_tables, n_bits, dtype_x, dtype_probs,
                             (cudaStream_t)stream);
}
}  // namespace

int race_b200_bucket_probs(const void* x, const float* planes, void* probs, int64_t rows,
                           int32_t d_k, int32_t n_tables, int32_t n_bits, int32_t dtype_x,
                           int32_t dtype_probs, void* stream) {
    return probs_entry(x, planes, probs, 1, rows, 1, d_k, n_tables, n_bits, dtype_x, dtype_probs, stream);
}

int race_b200_bucket_probs_streams(const void* x, const float* planes, void* probs, int64_t outer,
                                   int64_t seq_len, int32_t heads, int32_t d_k, int32_t n_tables,
                                   int32_t n_bits, int32_t dtype_x, int32_t dtype_probs, void* stream) {
    return probs_entry(x, planes, probs, outer, seq_len, heads, d_k, n_tables, n_bits, dtype_x, dtype_probs,
                       stream);
}

}  // extern "C"
