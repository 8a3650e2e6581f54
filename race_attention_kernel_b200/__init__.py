"""B200-native (sm_100a) RACE-attention prefix path.

Public surface:
  BatchedACE                      drop-in operator (signature of src/race_baseline.py:21-52)
  race_causal_prefix              probabilities-level causal forward (the hot path)
  race_causal_qkv                 the causal forward from Q, K, V and the planes (probabilities formed in-kernel)
  race_tile_totals                per-stream totals (A, B) of a token range
  race_decode_step                incremental step: a few new tokens against a running state
  DecodeStepper                   the same with shape checks and buffers hoisted out of the serving loop
  race_causal                     the causal forward with autograd (hand-written backward kernels)
  race_causal_chunk               the same for one chunk of a longer sequence (state in, state out)
  race_noncausal                  non-causal forward with autograd
  bucket_probs                    bucket-probability producer
  bucket_probs_streams            the producer reading [M,B,T,H,d_k] directly (flattening fused)
"""
from .operator import BatchedACE  # noqa: F401
from .ops import (DecodeStepper, bucket_probs, bucket_probs_streams, is_supported, pack_state, race_causal_prefix,  # noqa: F401
                  race_causal_prefix_host, race_causal_prefix_static, race_causal, race_causal_qkv, qkv_is_supported, race_causal_backward, race_causal_chunk, race_decode_step, race_noncausal, race_tile_totals, select_tile_tokens,
                  unpack_state)
