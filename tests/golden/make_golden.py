"""Generate the golden fixtures of tests/golden/ by running the REFERENCE's own
CUDA kernels (oracle/_ref, built unmodified from the reference tree by
`make -C oracle ref`) on a B200, plus the device-only intermediates of this
library's kernel that the reference keeps in shared memory.

Run on a GPU box from the repository root:
    python tests/golden/make_golden.py --out out/golden
then copy the .npz files into tests/golden/.

Each Flash fixture holds, for the seeded inputs of tests/cases.py:
  ref_m_tiles, ref_ell_tiles   fp32 workspaces of the reference kernel
  ref_counts_idx/_val          the reference's sampled row counts (sparse), recovered with a probe V
  ref_out, ref_m_star, ref_vrows  the reference's outputs (out as 16-bit patterns)
  dev_u16, dev_invdel          this library's device values of the two hardware-approximate
                               intermediates (ex2.approx behind __expf, div.approx), which let the
                               CPU oracle be checked bit-for-bit downstream of them
Each Prop fixture holds the reference's m_tiles, ell_tiles, u_stash, S_tiles, invdelta, a0, counts,
out, m_star, vrows.
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
from oracle import ref_gpu  # noqa: E402
from santa_b200 import ops  # noqa: E402


def sparse(c):
    c = c.cpu().numpy()
    idx = np.flatnonzero(c)
    return idx.astype(np.int32), c.reshape(-1)[idx].astype(np.int16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="out/golden")
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    dev = torch.device("cuda:0")
    for name, c in cases.FLASH_CASES.items():
        q, K, V = cases.make_qkv(c["B"], c["Ls"], c["KVH"], c["dtype"], c["gen_seed"], c["kscale"], c["heavy"])
        q, K, V = q.to(dev), K.to(dev), V.to(dev)
        rc, _ = ref_gpu.flash_counts(q, K, c["S"], seed=c["seed"], block_n=c["block_n"], valid_len=c["L"])
        r = ref_gpu.flash_decode(q, K, V, c["S"], seed=c["seed"], block_n=c["block_n"], want_vrows=True,
                                 valid_len=c["L"])
        _, _, _, tr = ops.flash_decode(q, K, V, c["S"], seed=c["seed"], block_n=c["block_n"], want_vrows=True,
                                       valid_len=c["L"], trace=True)
        torch.cuda.synchronize()
        assert (tr.counts.int() == rc).all(), name
        idx, val = sparse(rc)
        np.savez_compressed(
            os.path.join(args.out, f"flash_{name}.npz"),
            ref_m_tiles=r.m_tiles.cpu().numpy(), ref_ell_tiles=r.ell_tiles.cpu().numpy(),
            ref_counts_idx=idx, ref_counts_val=val, ref_out=cases.bits(r.out),
            ref_m_star=r.m_star.cpu().numpy(), ref_vrows=r.vrows.cpu().numpy(),
            dev_u16=tr.u16.cpu().numpy().view(np.uint16), dev_invdel=tr.invdel.cpu().numpy(),
            block_n=np.int32(r.block_n), T_c=np.int32(r.T_c), S_per_tile=np.int32(r.S_per_tile))
        print("flash", name, "counts", int(rc.sum()), "vrows", r.vrows.flatten().tolist())
    for name, c in cases.PROP_CASES.items():
        q, K, V = cases.make_qkv(1, c["L"], c["KVH"], c["dtype"], c["gen_seed"], c["kscale"], c["heavy"], GH=c["GH"])
        q, K, V = q[0].to(dev), K[0].to(dev), V[0].to(dev)
        rc, base = ref_gpu.prop_counts(q, K, c["S"], seed=c["seed"], block_n=c["block_n"])
        r = ref_gpu.prop_decode(q, K, V, c["S"], seed=c["seed"], block_n=c["block_n"], want_vrows=True)
        torch.cuda.synchronize()
        idx, val = sparse(rc)
        np.savez_compressed(
            os.path.join(args.out, f"prop_{name}.npz"),
            ref_m_tiles=r.m_tiles.cpu().numpy(), ref_ell_tiles=r.ell_tiles.cpu().numpy(),
            ref_u_stash=cases.bits(r.u_stash), ref_S_tiles=r.S_tiles.cpu().numpy(),
            ref_invdelta=r.invdelta.cpu().numpy(), ref_a0=r.a0.cpu().numpy(),
            ref_counts_idx=idx, ref_counts_val=val, ref_out=cases.bits(r.out),
            ref_out_fp32=r.out_fp32.cpu().numpy(), ref_m_star=r.m_star.cpu().numpy(),
            ref_vrows=r.vrows.cpu().numpy(), block_n=np.int32(r.block_n), T_c=np.int32(r.T_c))
        print("prop", name, "S_tiles sum", r.S_tiles.sum(1)[:4].tolist(), "counts", int(rc.sum()), "vrows",
              r.vrows.tolist())


if __name__ == "__main__":
    main()
