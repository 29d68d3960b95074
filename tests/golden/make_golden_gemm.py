"""Regenerates tests/golden/gemm_*.npz from the reference's own PyTorch oracle.

Run in a checkout that has the reference project available:

    python tests/golden/make_golden_gemm.py /path/to/reference

It imports scripts/problems/gemm/reference.py UNMODIFIED, feeds it CPU tensors
built from the repository's seeded generator (e4m3fn bytes, |x|<=240, so the
values are representable in e4m3fnuz as well) and stores inputs plus the bf16
output bits.  The fixtures pin the numpy oracle in oracle/fp8_gemm.py.  The gemm_fnuz_* fixtures are made
the reference's own way (randn cast to float8_e4m3fnuz, transposed views) and pin the e4m3fnuz functions.
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

# (m, n, k, seed) of the e4m3fnuz fixtures (logical [m, k] / [n, k] bytes are stored; seeds from task.yml:54-55)
FNUZ_CASES = [
    (64, 128, 256, 6635),
    (96, 320, 384, 1236),
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

    # The reference's own data path: generate_input's recipe (scripts/problems/gemm/reference.py:28-37) on the
    # CPU - randn in bf16 cast to float8_e4m3fnuz in [k, m] / [k, n], N(0,1) scales in [k/128, m] / [k/128, n/128],
    # everything handed to ref_kernel as .T views - so the fixture pins the e4m3fnuz reading of the oracle.
    for (m, n, k, seed) in FNUZ_CASES:
        gen = torch.Generator()
        gen.manual_seed(seed)
        a = torch.randn((k, m), dtype=torch.bfloat16, generator=gen).to(torch.float8_e4m3fnuz)
        b = torch.randn((k, n), dtype=torch.bfloat16, generator=gen).to(torch.float8_e4m3fnuz)
        a_s = torch.randn((k // 128, m), dtype=torch.float32, generator=gen)
        b_s = torch.randn((k // 128, (n + 127) // 128), dtype=torch.float32, generator=gen)
        c = torch.zeros((m, n), dtype=torch.bfloat16)
        out = reference.ref_kernel((a.T, b.T, a_s.T, b_s.T, c))
        path = os.path.join(HERE, f"gemm_fnuz_m{m}_n{n}_k{k}.npz")
        np.savez_compressed(path, a=a.T.contiguous().view(torch.uint8).numpy(), b=b.T.contiguous().view(torch.uint8).numpy(),
                            a_scale=a_s.T.contiguous().numpy(), b_scale=b_s.T.contiguous().numpy(),
                            c_bits=out.view(torch.uint16).numpy().copy(), seed=seed)
        print("wrote", path, tuple(out.shape))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
