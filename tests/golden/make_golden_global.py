"""Generate ``race_global_golden.npz``: golden vectors of the GLOBAL-normalisation causal form
from the REFERENCE implementation itself.

    python tests/golden/make_golden_global.py /path/to/reference

It imports the reference's ``src/causal_v2/reference.py`` unchanged and calls
``race_causal_reference`` (paper Algorithm 1 made causal, :106-127) and
``race_causal_dense_reference`` (:130-141) on seeded inputs drawn the way the reference's own tests
draw them (q, k, v ~ N(0,1) [B,H,T,d], planes W ~ N(0,1) [L,P,d], beta = 1/sqrt(d)).  Stored per case:
the features Phi(q), Phi(k) the reference computed ([B,H,T,S], the probabilities boundary of this
library), v and the reference output.  The test-suite reads the .npz only.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch


def main(ref_root: str) -> None:
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(ref_root, "src", "causal_v2"))
    import reference as ref  # noqa: E402  (the reference, unmodified)

    out: dict[str, np.ndarray] = {}
    # name, (B, H, T, d, L, P), dtype
    cases = [
        ("g_k4l4", (1, 2, 96, 64, 4, 4), torch.float64),
        ("g_k2l2", (1, 2, 37, 64, 2, 2), torch.float64),
        ("g_k6l8_d128", (1, 1, 40, 128, 8, 6), torch.float64),
        ("g_k3l2_d32", (2, 3, 150, 32, 2, 3), torch.float64),
        ("g_k4l4_t700", (1, 2, 700, 64, 4, 4), torch.float32),
    ]
    for name, (B, H, T, d, L, P), dtype in cases:
        g = torch.Generator().manual_seed(len(name) * 1000 + T)
        q, k, v = (torch.randn(B, H, T, d, generator=g, dtype=dtype) for _ in range(3))
        W = torch.randn(L, P, d, generator=g, dtype=dtype)
        beta = torch.tensor(1.0 / d ** 0.5, dtype=dtype)
        with torch.no_grad():
            o = ref.race_causal_reference(q, k, v, W, beta)
            if T <= 200:
                dense = ref.race_causal_dense_reference(q, k, v, W, beta)
                assert torch.allclose(o, dense, rtol=1e-9, atol=1e-11), name
            phi_q, phi_k = ref.features(q, W, beta), ref.features(k, W, beta)
        out[f"{name}/cfg"] = np.array([B, H, T, d, L, 2 ** P], dtype=np.int64)
        out[f"{name}/phi_q"], out[f"{name}/phi_k"] = phi_q.numpy(), phi_k.numpy()
        out[f"{name}/v"], out[f"{name}/out"] = v.numpy(), o.numpy()
        print(f"{name}: out {tuple(o.shape)} {dtype}")

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "race_global_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden_global.py /path/to/reference-checkout")
    main(sys.argv[1])
