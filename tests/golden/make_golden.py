"""Generate the golden fixtures in this folder from the REFERENCE implementation itself.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's ``src/race_baseline.py`` (``BatchedACE``) and
``src/race_chunked.py`` (``chunked_forward``) unchanged, feeds them seeded inputs drawn the way
the reference's own tests draw them (src/test_equivalence.py:21-29: data from
``torch.Generator().manual_seed(0)`` in the order K, V, Q; planes from
``torch.manual_seed(1234)``), and writes inputs + outputs to ``race_golden.npz``.
The test-suite never needs the reference checkout: it reads the .npz only.
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
    from race_chunked import chunked_forward  # noqa: E402

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    out: dict[str, np.ndarray] = {}

    def draw(M, B, T, H, dk, dtype, seed=0):
        g = torch.Generator().manual_seed(seed)
        return [torch.randn((M, B, T, H, dk), generator=g, dtype=dtype) for _ in range(3)]

    # name, (M,B,H,d_k,K,L), T, dtype, store inputs?, token stride of the stored output
    cases = [
        ("small_k4l4", (1, 1, 2, 64, 4, 4), 96, torch.float32, True, 1),
        ("small_k2l2", (1, 1, 2, 64, 2, 2), 37, torch.float64, True, 1),
        ("small_k5l1", (1, 2, 1, 64, 5, 1), 37, torch.float64, True, 1),
        ("small_k6l8_d128", (1, 1, 1, 128, 6, 8), 40, torch.float32, True, 1),
        ("mb_k3l2_d32", (2, 2, 3, 32, 3, 2), 50, torch.float32, True, 1),
        ("c1_t4096", (1, 1, 8, 64, 4, 4), 4096, torch.float32, False, 64),
    ]
    for name, (M, B, H, dk, K, L), T, dtype, keep_inputs, stride in cases:
        torch.manual_seed(1234)
        ace = BatchedACE(dk, K, L, M).to(dtype)
        Kh, Vh, Qh = draw(M, B, T, H, dk, dtype)
        with torch.no_grad():
            ref = ace(Kh, Vh, Qh)
        out[f"{name}/cfg"] = np.array([M, B, H, dk, K, L, T, stride], dtype=np.int64)
        out[f"{name}/planes_T"] = ace.planes_T.contiguous().numpy()
        out[f"{name}/protos_T"] = ace.protos_T.contiguous().numpy()
        if keep_inputs:
            out[f"{name}/K"], out[f"{name}/V"], out[f"{name}/Q"] = (
                Kh.numpy(), Vh.numpy(), Qh.numpy())
        out[f"{name}/out"] = ref.contiguous().numpy()[:, :, ::stride]
        print(f"{name}: out {tuple(ref.shape)} stored stride {stride}")

    # chunked_forward pins (src/test_equivalence.py:49-59 uses these (T, chunk) pairs)
    for T, chunk in [(2048, 300), (2048, 512)]:
        M, B, H, dk, K, L = 1, 1, 8, 64, 4, 4
        torch.manual_seed(1234)
        ace = BatchedACE(dk, K, L, M)
        Kh, Vh, Qh = draw(M, B, T, H, dk, torch.float32)
        got = chunked_forward(ace, Kh, Vh, Qh, chunk=chunk)
        name = f"chunked_t{T}_c{chunk}"
        out[f"{name}/cfg"] = np.array([M, B, H, dk, K, L, T, 32], dtype=np.int64)
        out[f"{name}/planes_T"] = ace.planes_T.contiguous().numpy()
        out[f"{name}/out"] = got.contiguous().numpy()[:, :, ::32]
        print(f"{name}: stored")

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "race_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
    main(sys.argv[1])
