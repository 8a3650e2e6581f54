// Internal launcher interfaces shared by the translation units of the library.
#pragma once

#include <cuda_runtime.h>

#include "common.cuh"

namespace race {

// ---- CUDA-core causal path (causal_simt.cu) -------------------------------------------------
int simt_groups(int S);
bool simt_supported(const Dims& dm);
int simt_default_tile_tokens(const Dims& dm, int sm_count);
// tile totals -> scan -> outputs; totals_only stops after the scan and writes only state_out;
// skip_output stops after the scan but leaves the exclusive tile prefixes in ws; global_norm selects
// the global-normalisation estimator (one denominator per token) in the output pass.
cudaError_t causal_fwd_simt(const void* pq, const void* pk, const void* v, void* out,
                            const float* carry_in, float* state_out, float* ws, const Dims& dm,
                            int dtype, int tile_tokens, bool totals_only, cudaStream_t stream,
                            bool skip_output = false, bool skip_totals = false, bool global_norm = false);

// in-place exclusive scan over the per-tile totals in ws (+ carry_in), inclusive total to state_out
// (reverse: exclusive SUFFIX sums, last tile first -- the scans of the backward)
cudaError_t causal_scan_tiles(float* ws, const float* carry_in, float* state_out, const Dims& dm,
                              int tile_tokens, cudaStream_t stream, bool write_prefix = true, bool reverse = false);

// which passes of a causal forward to run: totals (per-tile sums into ws) and/or scan + outputs
constexpr int kPhaseTotals = 1, kPhaseOutput = 2, kPhaseAll = 3;

// ---- causal backward (causal_bwd_simt.cu): S <= 64, d_k <= 128 ---------------------------------
bool causal_bwd_supported(const Dims& dm);
int causal_bwd_tile_tokens(const Dims& dm, int dtype, int sm_count);
size_t causal_bwd_workspace_bytes(const Dims& dm, int dtype, int tile_tokens);
// carry_in: state before the first token (nullable); d_state: gradient reaching the state after the last token
// (nullable); d_carry: receives the gradient of carry_in (nullable)
cudaError_t causal_bwd_simt(const void* pq, const void* pk, const void* v, const void* dout, const float* carry_in,
                            const float* d_state, void* dpq, void* dpk, void* dv, float* d_carry, void* ws,
                            const Dims& dm, int dtype, int tile_tokens, cudaStream_t stream, int* status = nullptr);

// ---- non-causal path (noncausal_simt.cu) ------------------------------------------------------
cudaError_t noncausal_query(const void* pq, const float* totals, void* out, const Dims& dm, int dtype,
                            int sm_count, cudaStream_t stream);
cudaError_t noncausal_state_grads(const float* totals, const float* dE_state, float* grads,
                                  const Dims& dm, cudaStream_t stream);
cudaError_t noncausal_token_grads(const void* pk, const void* v, const void* dout, const float* totals,
                                  const float* grads, void* dpq, void* dpk, void* dv, const Dims& dm,
                                  int dtype, int sm_count, cudaStream_t stream);

// tensor-core token kernels of the non-causal path (noncausal_tc.cu): S = 64, d_k = 64
bool noncausal_tensor_supported(const Dims& dm, int dtype);
cudaError_t noncausal_query_tensor(const void* pq, const float* totals, void* out, const Dims& dm, int dtype,
                                   int sm_count, cudaStream_t stream);
cudaError_t noncausal_token_grads_tensor(const void* pk, const void* v, const void* dout, const float* totals,
                                         const float* grads, void* dpq, void* dpk, void* dv, const Dims& dm,
                                         int dtype, int sm_count, cudaStream_t stream);

// ---- bucket-probability producer (bucket_probs.cu) --------------------------------------------
// x [outer, T, heads, d] -> probs [outer*heads, T, L, 2^K]; rows = outer*heads*T (heads = 1: plain rows)
cudaError_t bucket_probs(const void* x, const float* planes, void* probs, int64_t rows, int64_t T, int heads,
                         int d, int L, int K, int dtype_x, int dtype_probs, cudaStream_t stream);

// ---- incremental step (decode.cu) -------------------------------------------------------------
// a few new tokens per stream (dm.T <= decode_max_tokens()) against a running state; state_in may be
// null (zeros) or equal state_out (in place)
int decode_max_tokens();
cudaError_t decode_step_launch(const void* pq, const void* pk, const void* v, void* out, const float* state_in,
                               float* state_out, const Dims& dm, int dtype, cudaStream_t stream);

// ---- tcgen05 tensor-core causal path (causal_tc.cu) ------------------------------------------
bool tensor_supported(const Dims& dm, int dtype);
int tensor_chunk_tokens();
int tensor_default_tile_tokens(const Dims& dm, int dtype, int sm_count);
size_t tensor_workspace_bytes(const Dims& dm, int dtype, int tile_tokens);
// the single-pass form of the fp32 forward (one persistent kernel): its tile length and its workspace
int tensor_single_pass_tile_tokens(const Dims& dm, int sm_count);
size_t tensor_single_pass_workspace_bytes(const Dims& dm, int tile_tokens);
// single_pass: the fp32 forward as one persistent kernel (needs phases == kPhaseAll and its larger workspace)
cudaError_t causal_fwd_tensor(const void* pq, const void* pk, const void* v, void* out,
                              const float* carry_in, float* state_out, void* ws, bool single_pass, const Dims& dm,
                              int dtype, int tile_tokens, cudaStream_t stream, int* status,
                              int phases = kPhaseAll, bool global_norm = false, long long wait_cycles = 0,
                              int withhold_chunk = -1);

// out_t = sum_{j <= t} (q_t . k_j) v_j + q_t . carry (reverse: j >= t, carry = state of the tokens after the call)
// on fp32 [N, T, 64] tensors with the three launches of the fp32 tensor forward, no normalisation
// The causal forward from Q, K, V and the hyperplanes [16][64] on the fp32 tensor kernels (d_k = 64, L = 4, R = 16);
// Q, K, V, out in the layout [N/heads, T, heads, 64]; workspace as for the three-launch form.
bool tensor_qkv_supported(const Dims& dm, int dtype, int L, int R);
cudaError_t causal_fwd_qkv_tensor(const void* q, const void* k, const void* v, const float* planes, void* out,
                                  const float* carry_in, float* state_out, void* ws, const Dims& dm, int tile_tokens,
                                  cudaStream_t stream, int* status, int phases, bool global_norm);
// Epilogue of the first backward pass, run by the forward-direction plain product X = raw(dO, V, pK) where it stores
// its result: with A_t = ablock[block of t] + achunk[chunk of t] + the running sum of pK inside the chunk (the V
// operand of that pass; taken with the triangular product the forward uses for its running sum), inv = 1/(A_t + eps):
//     out <- dPQ = X inv,   w_out <- W = pq_true inv,   g_out <- g = -dPQ W
struct BwdX {
    const float* pq_true;   // [N, T, 64] the query probabilities
    const float* ablock;    // [N, nblk, 64]  sums of pK over the tokens before each block (carry included)
    const float* achunk;    // [N, nchunk, 64] sums of pK from the start of the block to the start of each chunk
    float* w_out;           // [N, T, 64]
    float* g_out;           // [N, T, 64]
    int64_t nblk, nchunk;
    int block_tokens;       // tokens per block (a multiple of the 64-token chunk)
    float eps;
};
cudaError_t causal_raw_tensor(const void* q, const void* k, const void* v, void* out, const float* carry_in,
                              float* state_out, void* ws, const Dims& dm, int tile_tokens, bool reverse,
                              cudaStream_t stream, int* status, int phases = kPhaseAll, const BwdX* bwdx = nullptr);

// ---- causal backward on the tensor kernels (causal_bwd_tc.cu): fp32, S = 64, d_k = 64 ----------
bool causal_bwd_tensor_supported(const Dims& dm, int dtype);
int causal_bwd_tensor_tile_tokens(const Dims& dm, int sm_count);
size_t causal_bwd_tensor_workspace_bytes(const Dims& dm, int tile_tokens);
cudaError_t causal_bwd_tensor(const void* pq, const void* pk, const void* v, const void* dout, const float* carry_in,
                              const float* d_state, void* dpq, void* dpk, void* dv, float* d_carry, void* ws,
                              const Dims& dm, int tile_tokens, cudaStream_t stream, int* status);

// bf16 tensor path (causal_tc_bf16.cu): S a multiple of 64 (1, 2, 4 or 8 bucket groups), d_k 64 or 128
bool tensor_bf16_supported(const Dims& dm);
cudaError_t causal_fwd_tensor_bf16(const void* pq, const void* pk, const void* v, void* out,
                                   const float* carry_in, float* state_out, void* ws, const Dims& dm,
                                   int tile_tokens, cudaStream_t stream, int* status, int phases,
                                   bool global_norm = false);

}  // namespace race
