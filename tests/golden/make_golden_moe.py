"""Regenerates tests/golden/moe_*.npz from the reference's own PyTorch MoE oracle.

    python tests/golden/make_golden_moe.py /path/to/reference

Imports scripts/problems/moe/reference.py UNMODIFIED and runs its ref_kernel on CPU fp16 tensors
built by the repository's seeded generator (same tensors, scales and draw order as the reference
generator, which itself only runs on a GPU).  Stored: inputs, weights, the reference output, and
the reference gate's own top-k sets (torch.topk on torch.softmax) for the set-level index check.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import moe as o  # noqa: E402

# (d_hidden, d_expert, n_experts, n_shared, top_k, tokens, seed) - small relatives of
# scripts/problems/moe/task.yml:50-55
CASES = [
    (128, 64, 8, 1, 2, 64, 9371),
    (256, 128, 4, 1, 4, 48, 2291),
    (128, 64, 32, 1, 4, 96, 1212),
    (64, 64, 256, 1, 8, 160, 4242),      # the expert-parallel configuration's routing: 256 experts, top-8
]
# Above this many experts the expert weights are not stored: oracle.moe.generate_input rebuilds them, bit for
# bit, from the seed in `cfg` (numpy's seeded generator), which keeps the fixture at a few tens of KB.
STORE_WEIGHTS_UP_TO = 64


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "scripts", "problems", "moe"))
    sys.path.insert(0, os.path.join(ref_root, "scripts"))
    import reference  # the reference's own module

    for (d, f, e, ns, k, t, seed) in CASES:
        x, w, cfg = o.generate_input(d, f, e, ns, k, t, seed)
        tw = {name: torch.from_numpy(v) for name, v in w.items()}
        tx = torch.from_numpy(x)
        with torch.no_grad():
            out = reference.ref_kernel((tx, tw, cfg)).numpy().copy()
            gate = reference.MoEGate(cfg)
            gate.W_g.weight = torch.nn.Parameter(tw["router.weight"])
            idx, score = gate(tx)
        path = os.path.join(HERE, f"moe_d{d}_f{f}_e{e}_k{k}_t{t}.npz")
        stored = w if e <= STORE_WEIGHTS_UP_TO else {"router.weight": w["router.weight"]}
        np.savez_compressed(path, x=x, ref_out=out, ref_topk_idx=idx.numpy()[0].astype(np.int32),
                            ref_topk_score=score.numpy()[0], cfg=np.array([d, f, e, ns, k, t, seed]),
                            **{"w:" + name: v for name, v in stored.items()})
        print("wrote", path, out.shape, os.path.getsize(path))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
