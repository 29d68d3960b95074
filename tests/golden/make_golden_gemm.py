"""Regenerates tests/golden/gemm_*.npz from the reference's own PyTorch oracle.

Run in a checkout that has the reference project available:

    python tests/golden/make_golden_gemm.py /path/to/reference

It imports scripts/problems/gemm/reference.py UNMODIFIED, feeds it CPU tensors
built from the repository's seeded generator (e4m3fn bytes, |x|<=240, so the
values are representable in e4m3fnuz as well) and stores inputs plus the bf16
output bits.  The fixtures pin the numpy oracle in oracle/fp8_gemm.py.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import fp8_gemm as o  # noqa: E402

# (m, n, k, seed, scale distribution); seeds/shapes echo scripts/problems/gemm/task.yml:53-57
CASES = [
    (64, 64, 128, 6635, "randn"),
    (64, 576, 256, 542, "baseline"),
    (96, 320, 512, 1234, "randn"),
    (128, 192, 384, 624, "baseline"),
]


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "scripts", "problems", "gemm"))
    sys.path.insert(0, os.path.join(ref_root, "scripts"))
    import reference  # the reference's own module

    for (m, n, k, seed, dist) in CASES:
        a, b, a_s, b_s = o.generate_input(m, n, k, seed, dist)
        ta = torch.from_numpy(a).view(torch.float8_e4m3fn)
        tb = torch.from_numpy(b).view(torch.float8_e4m3fn)
        c = torch.zeros((m, n), dtype=torch.bfloat16)
        out = reference.ref_kernel((ta, tb, torch.from_numpy(a_s), torch.from_numpy(b_s), c))
        bits = out.view(torch.uint16).numpy().copy()
        path = os.path.join(HERE, f"gemm_m{m}_n{n}_k{k}_{dist}.npz")
        np.savez_compressed(path, a=a, b=b, a_scale=a_s, b_scale=b_s, c_bits=bits, seed=seed)
        print("wrote", path, bits.shape)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
