"""Worker of tests/test_multigpu.py: run as `python -m torch.distributed.run --nproc-per-node G` on G GPUs.
Every rank draws the same sequence, keeps its shard, and decodes it three ways: alone on the whole
sequence (rank-local reference), sharded with the NCCL all-gather, sharded with the peer-memory exchange."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import cases  # noqa: E402
from santa_b200 import ops, sharded  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    B, L, S = 2, 20000, 400
    q, K, V = cases.make_qkv(B, L, 8, "bf16", 123, 1.0, True)
    q, K, V = q.to(dev), K.to(dev), V.to(dev)
    full = ops.flash_decode(q, K, V, S, seed=77)
    bn, T_c, spt, plan = sharded.shard_plan(L, world, S)
    row0, row1, _ = plan[rank]
    Ks, Vs = K[:, row0:row1].contiguous(), V[:, row0:row1].contiguous()
    tol = lambda a, b: (a.float() - b.float()).abs().max().item() <= 2e-2  # noqa: E731
    o_nccl, m_nccl = sharded.seq_sharded_flash_decode(q, Ks, Vs, S, 77, L)
    assert tol(o_nccl, full[0]) and torch.equal(m_nccl, full[1]), "all-gather path differs from the unsharded call"
    # the receiving half inside the decode call (fused) and as a kernel of its own
    for fused in (True, False):
        ex = sharded.PeerExchange(B, 32, dev, fused=fused)
        for step in range(5):                              # several epochs: both buffer halves are reused
            qs = q if step % 2 == 0 else (q * 0.75).to(torch.bfloat16)
            ref = sharded.seq_sharded_flash_decode(qs, Ks, Vs, S, 77, L)
            got = sharded.seq_sharded_flash_decode(qs, Ks, Vs, S, 77, L, exchange=ex)
            ex.check()
            assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1]), \
                f"peer exchange (fused={fused}) differs at step {step}"
            if step == 0:
                assert tol(got[0], full[0]) and torch.equal(got[1], full[1]), "peer exchange differs from the unsharded call"
    # epochs counted on the device: one captured step replayed
    exg = sharded.PeerExchange(B, 32, dev, device_counted=True)
    qs = q.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        sharded.seq_sharded_flash_decode(qs, Ks, Vs, S, 77, L, exchange=exg)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        outg = sharded.seq_sharded_flash_decode(qs, Ks, Vs, S, 77, L, exchange=exg)
    for step in range(3):
        qs.copy_(q if step % 2 == 0 else (q * 0.75).to(torch.bfloat16))
        graph.replay()
        exg.check()
        ref = sharded.seq_sharded_flash_decode(qs, Ks, Vs, S, 77, L)
        assert torch.equal(outg[0], ref[0]) and torch.equal(outg[1], ref[1]), f"graph replay differs at step {step}"
    del graph
    dist.barrier()
    if rank == 0:
        print("MP_SEQ_SHARDED_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
