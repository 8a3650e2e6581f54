"""Generate ``race_grad_golden.npz``: gradients of the REFERENCE ``BatchedACE`` through K, V and Q.

    python tests/golden/make_golden_grad.py /path/to/reference

The reference module is differentiable by plain autograd over src/race_baseline.py:41-51.  This script
imports it unchanged, runs it in fp64 on seeded inputs (drawn like src/test_equivalence.py:21-29),
back-propagates a seeded output gradient and stores inputs, output and the three input gradients.
The test-suite reads the .npz only.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch


def main(ref_root: str) -> None:
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from race_baseline import BatchedACE  # noqa: E402  (the reference, unmodified)

    out: dict[str, np.ndarray] = {}
    # name, (M,B,H,d_k,K,L), T
    for name, (M, B, H, dk, K, L), T in [("grad_k4l4", (1, 1, 2, 64, 4, 4), 70),
                                         ("grad_k3l2_d32", (2, 1, 3, 32, 3, 2), 33)]:
        torch.manual_seed(1234)
        ace = BatchedACE(dk, K, L, M).double()
        g = torch.Generator().manual_seed(0)
        Kh, Vh, Qh = (torch.randn((M, B, T, H, dk), generator=g, dtype=torch.float64).requires_grad_(True)
                      for _ in range(3))
        dO = torch.randn((M, B, T, H, dk), generator=g, dtype=torch.float64)
        ref = ace(Kh, Vh, Qh)
        ref.backward(dO)
        out[f"{name}/cfg"] = np.array([M, B, H, dk, K, L, T], dtype=np.int64)
        out[f"{name}/planes_T"] = ace.planes_T.contiguous().numpy()
        for key, t in (("K", Kh), ("V", Vh), ("Q", Qh), ("dO", dO), ("out", ref), ("dK", Kh.grad), ("dV", Vh.grad),
                       ("dQ", Qh.grad)):
            out[f"{name}/{key}"] = t.detach().contiguous().numpy()
        print(f"{name}: stored, |dK| {Kh.grad.norm():.4e} |dV| {Vh.grad.norm():.4e} |dQ| {Qh.grad.norm():.4e}")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "race_grad_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden_grad.py /path/to/reference-checkout")
    main(sys.argv[1])
