/*
 * race_b200.h -- C ABI of the B200 (sm_100a) RACE-attention prefix-path library.
 *
 * Plain pointers and sizes only; no torch types.  Every entry point enqueues work on the
 * caller's stream and returns without synchronising (the *_host entry points are the one
 * exception and say so).  Buffers are caller-owned.  Return value of every int function:
 *   0                      success
 *   < 0                    argument error (RACE_ERR_* below); nothing was launched
 *   > 0                    the first cudaError_t the launcher met
 * The pattern (raw pointers + shape struct + stream, first error returned, unsupported
 * shapes rejected with an error code instead of an exception) follows the reference's
 * plain-C++ launcher layer, src/causal_v2/kernels/race_causal_fwd.h:44-66,126-130.
 *
 * Tensor layouts (row-major, contiguous, 16-byte aligned base pointers):
 *   probsQ, probsK : [N, T, L, R]   bucket probabilities, element type = shape.dtype
 *   V, out         : [N, T, d_k]    element type = shape.dtype
 *   state          : [N, S*(d_k+1)] fp32, S = L*R; for one stream B[s][c] at s*d_k + c and
 *                    A[s] at S*d_k + s  (A = sum of key probabilities, B = sum of pK (x) v)
 * N = M*B*H independent streams (the reference's BatchedACE flattens [M,B,T,H,d_k] to
 * [N,T,d_k], src/race_baseline.py:35-40).
 * With RaceShape.heads = H > 1 the causal entry points read V and write out in the operator's own
 * layout [N/H, T, H, d_k] (stream n = outer*H + h), so that neither the flattened copy of V nor the
 * permuted view of the output (src/race_baseline.py:40,52) is needed; the probabilities stay
 * [N, T, L, R].  Supported by the tensor variant of race_b200_causal_fwd, race_b200_tile_totals and
 * race_b200_causal_fwd_resume for fp32 (S = 64, d_k = 64) and for bf16 with S = 256 or 512 (d_k = 64 or
 * 128); every other entry point, shape and variant rejects heads > 1 with RACE_ERR_SHAPE / reports
 * it as unsupported.
 */
#ifndef RACE_B200_H_
#define RACE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { RACE_DTYPE_F32 = 0, RACE_DTYPE_BF16 = 1 };

/* kernel families: AUTO picks TENSOR when the shape is supported by it, else SIMT.
 * TENSOR_SINGLE_PASS is the fp32 tensor family with the causal forward as ONE persistent kernel
 * (tiles handed out by an atomic ticket; per tile: totals, decoupled look-back over the earlier
 * tiles of the stream, outputs with the tile's pK and V read the second time from L2) instead of
 * the three launches (tile totals, scan over tiles, output pass) of TENSOR.  Same arithmetic in
 * the same order: for equal tile_tokens the two forms give bit-identical results.  It moves
 * about 1.05x the algorithmic bytes through DRAM where the three launches move 1.5x, and wants
 * a larger workspace (race_b200_causal_workspace_bytes with this variant; the launcher zeroes the
 * look-back flags and the tile ticket in it on the caller's stream).  For race_b200_tile_totals
 * and race_b200_causal_fwd_resume it means the same as TENSOR. */
enum { RACE_VARIANT_AUTO = 0, RACE_VARIANT_SIMT = 1, RACE_VARIANT_TENSOR = 2, RACE_VARIANT_TENSOR_SINGLE_PASS = 3 };

enum {
    RACE_OK = 0,
    RACE_ERR_NULL = -1,        /* a required pointer is NULL */
    RACE_ERR_SHAPE = -2,       /* shape outside the supported range */
    RACE_ERR_ALIGN = -3,       /* pointer or row not 16-byte aligned */
    RACE_ERR_WORKSPACE = -4,   /* workspace_bytes smaller than required */
    RACE_ERR_TILE = -5,        /* tile_tokens not a positive multiple of the chunk length */
    RACE_ERR_VARIANT = -6,     /* variant unknown or not available for this shape */
    RACE_ERR_DEVICE_WAIT = -7, /* a bounded device-side wait ran out (read from status word) */
    RACE_ERR_SCRATCH = -8      /* shape needs more workspace than the built-in scratch array holds */
};

typedef struct RaceShape {
    int64_t n_streams; /* N = M*B*H */
    int64_t seq_len;   /* T (may be 0: returns without launching) */
    int32_t n_tables;  /* L */
    int32_t n_buckets; /* R = 2^K buckets per table */
    int32_t head_dim;  /* d_k */
    int32_t dtype;     /* RACE_DTYPE_* of probsQ/probsK/V/out */
    float eps;         /* added to A before the divide; the reference uses 1e-6 */
    int32_t heads;     /* layout of V and out: 0 or 1 = [N, T, d_k]; H > 1 = [N/H, T, H, d_k] (below) */
} RaceShape;

/* Library / ABI version (major*1000 + minor). */
int race_b200_version(void);

/* Static, NUL-terminated description of a return code of this library. */
const char* race_b200_error_string(int code);

/* 1 if the shape can run with the given variant, else 0.
 * Replaces race::causal::is_supported (src/causal_v2/kernels/race_causal_fwd.h:72). */
int race_b200_is_supported(const RaceShape* shape, int variant);

/* Floats in a state / carry buffer: N * L*R * (d_k + 1).
 * Replaces final_state_floats (src/causal_v2/kernels/race_causal_fwd.h:101). */
size_t race_b200_state_floats(const RaceShape* shape);

/* Tokens per state tile the launcher would pick for this shape on the current device.
 * Replaces race_causal_select_tile_tokens (src/causal_v2/kernels/race_causal_fwd.h:89-90). */
int race_b200_select_tile_tokens(const RaceShape* shape, int variant, int* tile_tokens);

/* Bytes of workspace race_b200_causal_fwd / race_b200_tile_totals need for this tile length
 * (tile_tokens = 0: the automatic one of the variant).  Replaces workspace_floats (:99).
 * One state per tile; RACE_VARIANT_TENSOR_SINGLE_PASS: per tile its totals and its inclusive
 * prefix, a carry slot per CTA, the look-back flags and the tile ticket. */
size_t race_b200_causal_workspace_bytes(const RaceShape* shape, int tile_tokens, int variant);

/*
 * Causal per-bucket prefix forward:
 *   out[n,t,:] = sum_s pQ[n,t,s] * B_t[n,s,:] / (A_t[n,s] + eps),
 *   A_t = carry_A + sum_{j<=t} pK[n,j,:],  B_t = carry_B + sum_{j<=t} pK[n,j,:] (x) V[n,j,:].
 * This is BatchedACE.forward's cumsum / divide / bmm (src/race_baseline.py:45-51) and, with
 * carry_in, one chunk step of chunked_forward (src/race_chunked.py:54-63), without ever
 * materialising a T axis.  Replaces race_causal_forward
 * (src/causal_v2/kernels/race_causal_fwd.h:126-130) at the probabilities boundary.
 *   carry_in   nullable; state layout; sums over tokens that precede this call's first token
 *   state_out  nullable; state layout; carry_in + sums over all T tokens of this call
 *   workspace  >= race_b200_causal_workspace_bytes(); contents undefined on entry
 *   status     nullable device int32; set non-zero by a kernel whose bounded wait ran out
 */
int race_b200_causal_fwd(const void* probs_q, const void* probs_k, const void* v, void* out,
                         const float* carry_in, float* state_out, void* workspace,
                         size_t workspace_bytes, const RaceShape* shape, int tile_tokens,
                         int variant, void* stream, int* status);

/*
 * Totals of a token range: totals[n] = (sum_t pK (x) V, sum_t pK) in state layout.  Pass 1 of
 * the sequence-sharded driver and the reduction of the non-causal forward
 * (the `pref[:, -1:]` carry of src/race_chunked.py:62-63 without forming prefixes;
 * role of race_causal_tile_sums + the scan's final_state, race_causal_fwd.h:104-113).
 */
int race_b200_tile_totals(const void* probs_k, const void* v, float* totals, void* workspace,
                          size_t workspace_bytes, const RaceShape* shape, int tile_tokens,
                          int variant, void* stream, int* status);

/*
 * Second half of a causal forward whose first half was race_b200_tile_totals: `workspace` still
 * holds the per-tile totals that call left there (same shape, tile_tokens and variant); this
 * call scans them (adding carry_in) and runs the output pass, so pK and V are not reduced a
 * second time.  The sequence-sharded driver calls race_b200_tile_totals, exchanges the totals
 * between GPUs and then calls this with the received carry.  Arguments as race_b200_causal_fwd.
 */
int race_b200_causal_fwd_resume(const void* probs_q, const void* probs_k, const void* v, void* out,
                                const float* carry_in, float* state_out, void* workspace,
                                size_t workspace_bytes, const RaceShape* shape, int tile_tokens,
                                int variant, void* stream, int* status);

/*
 * Causal forward in the GLOBAL-normalisation form (paper Algorithm 1 made causal, the estimator of
 * the reference's own CUDA kernels and of race_causal_reference, src/causal_v2/reference.py:106-127):
 *   out[n,t,:] = (sum_s pQ[n,t,s] * B_t[n,s,:]) / (sum_s pQ[n,t,s] * A_t[n,s])
 * with the prefixes A_t, B_t of race_b200_causal_fwd; one denominator per token, shape.eps is not
 * used, and a row whose denominator is exactly 0 is written as 0 (:77-81).  carry_in / state_out /
 * workspace / variant / status as in race_b200_causal_fwd (size the workspace with the same variant).
 * RACE_VARIANT_TENSOR (and _SINGLE_PASS) computes this form for fp32, S = 64, d_k = 64 (heads allowed) and for
 * bf16 with S = 64, d_k = 64 or 128 (the geometry of the reference's own tensor-core kernel);
 * RACE_VARIANT_SIMT for every shape the CUDA-core kernels take (heads <= 1); AUTO picks the tensor
 * kernels where they have it.  The wider bf16 tensor kernel (S > 64) does not have it (RACE_ERR_VARIANT).
 * Replaces race_causal_forward (src/causal_v2/kernels/race_causal_fwd.h:126-130) at the
 * probabilities boundary for callers that want the reference kernels' estimator.
 */
int race_b200_causal_fwd_global(const void* probs_q, const void* probs_k, const void* v, void* out,
                                const float* carry_in, float* state_out, void* workspace,
                                size_t workspace_bytes, const RaceShape* shape, int tile_tokens, int variant,
                                void* stream, int* status);

/*
 * Causal forward from Q, K, V and the hyperplanes: the bucket probabilities of BatchedACE.forward
 * (src/race_baseline.py:41-44: projections on the L*K planes, tanh / sqrt(d_k), softmax over the 2^K sign corners)
 * are formed inside the prefix kernels, in registers and shared memory, bit-identical to what
 * race_b200_bucket_probs_streams writes; neither probsQ nor probsK exists in device memory and the forward moves
 * Q, K, V and out through HBM and nothing else.  The counterpart of the reference's race_causal_forward, which
 * also takes q, k, v and planes (src/causal_v2/kernels/race_causal_fwd.h:126-130; its in-kernel feature phases:
 * src/causal_v2/kernels/race_causal_fwd_tc.cu:562-642).
 *   q, k, v, out  [N/H, T, H, d_k] with H = shape.heads (0 or 1: [N, T, d_k]), fp32
 *   planes        [L*K, d_k] fp32, row p = l*K + k (the transpose of BatchedACE.planes_T)
 *   n_planes      K; shape.n_buckets must be 2^K
 *   global_norm   0: the per-bucket estimator of race_b200_causal_fwd; 1: that of race_b200_causal_fwd_global
 * Supported (race_b200_qkv_is_supported): fp32, d_k = 64, L = 4, K = 4 -- the geometry of the tcgen05 fp32
 * kernels; other shapes return RACE_ERR_VARIANT and go through race_b200_bucket_probs_streams +
 * race_b200_causal_fwd.  carry_in / state_out / status as in race_b200_causal_fwd; workspace >=
 * race_b200_causal_workspace_bytes(shape, tile_tokens, RACE_VARIANT_TENSOR).
 */
int race_b200_qkv_is_supported(const RaceShape* shape, int n_planes);
int race_b200_causal_fwd_qkv(const void* q, const void* k, const void* v, const float* planes, void* out,
                             const float* carry_in, float* state_out, void* workspace, size_t workspace_bytes,
                             const RaceShape* shape, int n_planes, int tile_tokens, int global_norm, void* stream,
                             int* status);

/*
 * Backward of race_b200_causal_fwd (carry_in = none): gradients w.r.t. probsQ, probsK and V given
 * d_out [N,T,d_k]; d_probs_q / d_probs_k / d_v have the layouts and dtype of their primals.  The
 * reference has no causal backward (its design note only outlines one for the global form,
 * docs/causal_v2_design.md:689-741); this is the derivative of src/race_baseline.py:45-51:
 *   X_t[s] = B_t[s,:].dO_t, dPQ_t = X_t/(A_t+eps), g_t = -X_t*W_t/(A_t+eps), W_t = pQ_t/(A_t+eps),
 *   dPK_j[s] = sum_{t>=j} g_t[s] + (sum_{t>=j} W_t[s] dO_t).V_j,  dV_j = sum_s pK_j[s] sum_{t>=j} W_t[s] dO_t.
 * Recomputes the forward's prefix states (nothing has to be saved by the forward).  fp32 with L*R = 64, d_k = 64
 * runs as three plain causal / anti-causal passes of the forward's tcgen05 kernels plus two streaming kernels;
 * every other shape (L*R <= 64 or a multiple of 64 up to 512, d_k <= 128, bf16) on CUDA-core kernels; heads <= 1.  workspace: 256-byte aligned, >= race_b200_causal_bwd_workspace_bytes()
 * (two fp32 [N,T,L*R] scratch arrays plus tile states).  status: as in race_b200_causal_fwd (the prefix
 * states come from the forward's tile-totals kernel, whose waits are bounded).
 */
size_t race_b200_causal_bwd_workspace_bytes(const RaceShape* shape);
int race_b200_causal_bwd(const void* probs_q, const void* probs_k, const void* v, const void* d_out,
                         void* d_probs_q, void* d_probs_k, void* d_v, void* workspace, size_t workspace_bytes,
                         const RaceShape* shape, void* stream, int* status);

/*
 * The same backward for one chunk of a longer sequence, i.e. of race_b200_causal_fwd called with carry_in
 * and state_out (the chunk loop of src/race_chunked.py:45-63, differentiated chunk by chunk in reverse):
 *   carry_in     nullable; state layout; the forward's carry_in
 *   d_state_out  nullable; state layout; gradient reaching the forward's state_out (from the chunks after)
 *   d_carry_in   nullable; state layout; receives the gradient of carry_in (for the chunk before)
 */
int race_b200_causal_bwd_carry(const void* probs_q, const void* probs_k, const void* v, const void* d_out,
                               const float* carry_in, const float* d_state_out, void* d_probs_q, void* d_probs_k,
                               void* d_v, float* d_carry_in, void* workspace, size_t workspace_bytes,
                               const RaceShape* shape, void* stream, int* status);

/*
 * Incremental (decode) step: race_b200_causal_fwd for a few NEW tokens per stream (seq_len <= 64,
 * typically 1) against a running state kept in device memory between calls, i.e. chunked_forward's
 * state update (src/race_chunked.py:54-63) with a chunk of seq_len tokens, costing one read and one
 * write of the state.  The reference has no incremental entry point; its launcher only returns the
 * final state of a full forward (src/causal_v2/kernels/race_causal_fwd.h:101,126-130).
 *   state_in   nullable (zeros); state layout; sums over all earlier tokens
 *   state_out  required; receives state_in + sums over the new tokens.  May be the same pointer as
 *              state_in (updated in place); otherwise the two buffers must not overlap.
 * Needs no workspace.  L*R <= 2048, heads <= 1, any d_k whose rows are 16-byte multiples.
 */
int race_b200_decode_step(const void* probs_q, const void* probs_k, const void* v, void* out,
                          const float* state_in, float* state_out, const RaceShape* shape, void* stream);

/*
 * Non-causal per-bucket forward (upstream scaling/benchmark_time.py:155-162 as quoted in the
 * reference's analysis/hot-path.md:157-162):
 *   Bs = pK^T V, A = sum_t pK, E = Bs/(A+eps), out = pQ E.
 * totals (state layout, required) receives (Bs, A); it is what the backward needs saved
 * (the reference saves the same reduced sums, src/noncausal/ops.py:29-33).
 * Replaces race_forward (src/noncausal/kernels/race_fwd.h:66-68) at the probabilities boundary.
 */
int race_b200_noncausal_fwd(const void* probs_q, const void* probs_k, const void* v, void* out,
                            float* totals, void* workspace, size_t workspace_bytes,
                            const RaceShape* shape, void* stream);

/* Bytes of workspace the non-causal backward needs. */
size_t race_b200_noncausal_bwd_workspace_bytes(const RaceShape* shape);

/*
 * Non-causal backward: gradients w.r.t. probsQ, probsK, V given d_out and the forward's
 * totals.  d_probs_q / d_probs_k / d_v have the layouts and dtype of their primals.
 * Replaces race_backward (src/noncausal/kernels/race_bwd.h:81-85) for the per-bucket form.
 */
int race_b200_noncausal_bwd(const void* probs_q, const void* probs_k, const void* v,
                            const float* totals, const void* d_out, void* d_probs_q,
                            void* d_probs_k, void* d_v, void* workspace, size_t workspace_bytes,
                            const RaceShape* shape, void* stream);

/*
 * Bucket-probability producer (src/race_baseline.py:41-44):
 *   probs[row, l, :] = softmax_r( (tanh(x[row] . planes[l,k]) / sqrt(d_k)) . corner_r ),
 * corner r has +1 on plane k iff bit (K-1-k) of r is set.  x [rows, d_k] (dtype_x; d_k a power of two, 4..256),
 * planes [L*K, d_k] fp32 (row-major: planes_T transposed), probs [rows, L, 2^K] (dtype_probs).
 */
int race_b200_bucket_probs(const void* x, const float* planes, void* probs, int64_t rows,
                           int32_t d_k, int32_t n_tables, int32_t n_bits, int32_t dtype_x,
                           int32_t dtype_probs, void* stream);

/*
 * The same producer reading the operator's own layout: x [outer, seq_len, heads, d_k] (outer = M*B of
 * the reference's [M,B,T,H,d_k]) -> probs [outer*heads, seq_len, L, 2^K], i.e. the stream flattening
 * of src/race_baseline.py:35-40 (permute + contiguous) happens inside the read and the flattened
 * copy of x is never written.
 */
int race_b200_bucket_probs_streams(const void* x, const float* planes, void* probs, int64_t outer,
                                   int64_t seq_len, int32_t heads, int32_t d_k, int32_t n_tables,
                                   int32_t n_bits, int32_t dtype_x, int32_t dtype_probs, void* stream);

/*
 * Host-buffer causal forward: same arithmetic as race_b200_causal_fwd with every tensor in
 * HOST memory (pinned for full copy bandwidth).  Allocates device staging buffers, streams
 * the sequence through them in segments (copy-in, kernel and copy-out overlapped on three
 * streams, the carry staying on the device between segments) and SYNCHRONISES before
 * returning.  segment_tokens = 0 picks a default.  device = CUDA ordinal to run on.
 * Returns RACE_ERR_DEVICE_WAIT if a kernel gave up a bounded wait.  The staging buffers (about
 * 2 x 260 MB at the default segment), streams and events of a device are kept for the next call;
 * race_b200_host_release(device) frees them.  Calls on one device are serialised.
 * Role of the reference's chunk loop around its carried state (src/race_chunked.py:41-63).
 */
int race_b200_causal_fwd_host(const void* probs_q, const void* probs_k, const void* v, void* out,
                              const float* carry_in, float* state_out, const RaceShape* shape,
                              int64_t segment_tokens, int variant, int device);
int race_b200_host_release(int device);

/*
 * race_b200_causal_fwd without a caller-provided workspace, for callers that cannot allocate
 * device memory at the point of the call (stream capture in progress, allocator callbacks,
 * allocation-free real-time loops, embedders with a fixed memory plan).  It has no counterpart
 * in the reference, whose binding always allocates its workspace from the torch allocator.
 * Inputs, outputs, carry and state are still the caller's buffers; the workspace is a 16 MiB
 * array inside the library (race_b200_static_scratch_bytes()), resident on every GPU that loads
 * the library until the process exits.  No call allocates or frees anything.
 *   - shapes whose workspace exceeds the array return RACE_ERR_SCRATCH and launch nothing
 *     (at S = 64, d_k = 64 and 2048-token tiles: up to N * ceil(T / 2048) = 1008 tiles,
 *     e.g. 8 streams of 258,048 tokens);
 *   - the first call on a device looks the array's address up (cudaGetSymbolAddress) with that
 *     device current; make that first call before any stream capture begins;
 *   - every call uses the same array: calls that overlap on the GPU race on it, so order them
 *     (one stream, or events).  The array needs no clearing between calls.
 */
size_t race_b200_static_scratch_bytes(void);
int race_b200_causal_fwd_static(const void* probs_q, const void* probs_k, const void* v, void* out,
                                const float* carry_in, float* state_out, const RaceShape* shape,
                                int tile_tokens, int variant, void* stream, int* status);

/*
 * Self-test of the bounded device-side waits (diagnostics; not part of the compute path).  Runs
 * race_b200_causal_fwd with variant RACE_VARIANT_TENSOR or RACE_VARIANT_TENSOR_SINGLE_PASS (fp32,
 * S = 64, d_k = 64) with every device-side wait limited to wait_cycles SM clock cycles
 * (1000 .. 2^31) and with the TMA producer of the CTA that works on the first tile of stream 0
 * skipping the load of chunk withhold_chunk (64-token chunks), so that the consumer of that chunk
 * waits in vain.  Expected behaviour, which a test
 * asserts: the call returns, the kernels end within a few multiples of wait_cycles, *status
 * (required) holds the code of the wait that gave up, the outputs of that CTA are unspecified,
 * and the device stays usable.  Nothing faults and nothing spins without a limit.  The reference
 * has no counterpart: its kernels have no device-side waits on other agents
 * (src/causal_v2/kernels/race_causal_fwd.cu uses __syncthreads only).
 */
int race_b200_selftest_bounded_wait(const void* probs_q, const void* probs_k, const void* v, void* out,
                                    void* workspace, size_t workspace_bytes, const RaceShape* shape, int variant,
                                    int64_t wait_cycles, int withhold_chunk, void* stream, int* status);

#ifdef __cplusplus
}
#endif
#endif /* RACE_B200_H_ */
