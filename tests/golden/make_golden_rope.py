"""Generate tests/golden/rope_*.npz by running the REFERENCE's own tensor code for the step in front
of the attention call (tutorial_code/runtime_common.py:540-556 with its apply_rotary_pos_emb,
:174-185) on the CPU, on seeded inputs.  The reference is a Python file here, so it is imported
from its tree; nothing of it is copied.

    python tests/golden/make_golden_rope.py --reference <reference root> [--out tests/golden]
"""
import argparse
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402
from oracle import rope_append as ro  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference tree")
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "tutorial_code"))
    import runtime_common as rc  # the reference

    for name, c in cases.ROPE_CASES.items():
        dt = cases.torch_dtype(c["dtype"])
        q_proj, k_proj, v_proj, kc, vc = cases.make_rope_inputs(c)
        B, H, KVH, D, pos = c["B"], c["H"], c["KVH"], 128, c["pos"]
        position_ids = torch.full((B, 1), pos, dtype=torch.long)
        cos, sin = ro.rope_tables(position_ids[:, 0], D, dt)
        # --- the reference's sequence, runtime_common.py:544-556 -------------------------------
        q = q_proj.view(B, 1, H, D).transpose(1, 2).contiguous()
        k = k_proj.view(B, 1, KVH, D).transpose(1, 2).contiguous()
        v = v_proj.view(B, 1, KVH, D).transpose(1, 2).contiguous()
        q, k = rc.apply_rotary_pos_emb(q, k, cos[:, None, :], sin[:, None, :], unsqueeze_dim=1)
        kc[:, pos].copy_(k[:, :, 0, :])
        vc[:, pos].copy_(v[:, :, 0, :])
        q_bhd = q[:, :, 0, :].contiguous()
        np.savez_compressed(
            os.path.join(args.out, f"rope_{name}.npz"),
            cos=cases.bits(cos), sin=cases.bits(sin), ref_q=cases.bits(q_bhd),
            ref_k_row=cases.bits(kc[:, pos].contiguous()), ref_v_row=cases.bits(vc[:, pos].contiguous()),
            ref_k_cache_sum=np.array(kc.float().abs().sum().item()),
        )
        print("wrote", name)


if __name__ == "__main__":
    main()
