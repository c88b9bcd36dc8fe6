"""Generate the golden fixtures in this directory from the REFERENCE implementation.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own naive einsum modules
(``src/flash_trittention/triple_dot_product/trittention_pytorch.py`` and
``src/flash_trittention/dot_product_sum/trittention_pytorch.py``), runs them in fp32 on
the CPU on seeded inputs, back-propagates a seeded upstream gradient through them with
autograd, and stores inputs, output and the five gradients as ``.npz``.  The fixtures
are what pins the CPU oracle (and, through it, the CUDA kernels) to the reference; the
reference checkout itself is not needed at test time.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name, variant, B, N, T, D, causal, softmax_scale, extra, input scale (q,k1,k2,v1,v2)
CASES = [
    ("tdp_T33_causal_full", "tdp", 1, 2, 33, 16, True, 1 / 8, dict(windows=(None, None, None, None)), (1, 1, 1, 1, 1)),
    ("tdp_T64_causal_full", "tdp", 1, 2, 64, 32, True, 1 / 8, dict(windows=(64, 64, 64, 64)), (1, 1, 1, 1, 1)),
    ("tdp_T40_noncausal", "tdp", 1, 2, 40, 16, False, 1 / 8, dict(windows=(40, 40, 40, 40)), (1, 1, 1, 1, 1)),
    ("tdp_T64_narrow_8_8_4_4", "tdp", 1, 2, 64, 16, True, 1 / 8, dict(windows=(8, 8, 4, 4)), (1, 1, 1, 1, 1)),
    ("tdp_T50_asym_16_7_3_9", "tdp", 1, 2, 50, 16, True, 1 / 4, dict(windows=(16, 7, 3, 9)), (1, 1, 1, 1, 1)),
    ("tdp_T48_windows_1_1_1_1", "tdp", 1, 1, 48, 16, True, 1 / 8, dict(windows=(1, 1, 1, 1)), (1, 1, 1, 1, 1)),
    ("tdp_T64_cfg1_alpha_1_over_D", "tdp", 1, 2, 64, 32, True, 1 / 32, dict(windows=(None, None, None, None)), (1, 1, 1, 1, 1)),
    ("dps_T33_causal", "dps", 1, 2, 33, 16, True, 1 / 8, dict(k_diff=33), (1, 1, 1, 1, 1)),
    ("dps_T64_noncausal", "dps", 1, 2, 64, 16, False, 1 / 8, dict(k_diff=64), (1, 1, 1, 1, 1)),
    ("dps_T64_kdiff2", "dps", 1, 2, 64, 16, True, 1 / 8, dict(k_diff=2), (1, 1, 1, 1, 1)),
    ("dps_T64_kdiff8", "dps", 1, 2, 64, 32, True, 1 / 8, dict(k_diff=8), (1, 1, 1, 1, 1)),
    ("dps_T64_large_logits", "dps", 1, 2, 64, 32, True, 1 / 8, dict(k_diff=64), (1, 8, 8, 1, 1)),
]


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from flash_trittention.triple_dot_product.trittention_pytorch import Trittention_pytorch as RefTDP
    from flash_trittention.dot_product_sum.trittention_pytorch import Trittention_pytorch as RefDPS

    for idx, (name, variant, B, N, T, D, causal, scale, extra, in_scale) in enumerate(CASES):
        g = torch.Generator().manual_seed(1000 + idx)
        tensors = [
            (torch.randn(B, N, T, D, generator=g) * s).requires_grad_(True) for s in in_scale
        ]
        dz = torch.randn(B, N, T, D, generator=g)
        if variant == "tdp":
            k1w, k2w, kkl, kkr = extra["windows"]
            mod = RefTDP(causal=causal, softmax_scale=scale, n_ctx=T,
                         k1_window=k1w, k2_window=k2w, kk_left=kkl, kk_right=kkr)
            meta = dict(k1_window=-1 if k1w is None else k1w, k2_window=-1 if k2w is None else k2w,
                        kk_left=-1 if kkl is None else kkl, kk_right=-1 if kkr is None else kkr)
        else:
            mod = RefDPS(causal=causal, softmax_scale=scale, n_ctx=T, k_diff=extra["k_diff"])
            meta = dict(k_diff=extra["k_diff"])
        z = mod(*tensors)[0]
        z.backward(dz)
        out = {n_: t.detach().numpy() for n_, t in zip(("q", "k1", "k2", "v1", "v2"), tensors)}
        out.update({"d" + n_: t.grad.numpy() for n_, t in zip(("q", "k1", "k2", "v1", "v2"), tensors)})
        out.update(dz=dz.numpy(), z=z.detach().numpy(), causal=np.int32(causal),
                   softmax_scale=np.float64(scale), variant=np.array(variant))
        out.update({k: np.int32(v) for k, v in meta.items()})
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(f"wrote {path}  z.abs().max()={float(z.abs().max()):.4f}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
