"""Multi-GPU decode, one process per GPU over torch.distributed.

* ``batch_sharded_flash_decode``: independent sequences, no communication.  The RNG key of the
  Flash sampler contains the batch index (flash_style_fused_santa_fixed_tile_budgets/
  santa_cuda_kernel.cu:281), so each rank passes its first global batch index as ``batch_offset``
  and the union of the ranks' outputs equals the single-GPU call bit for bit.
* ``seq_sharded_flash_decode``: ONE very long sequence (or batch of them) whose KV cache is split
  along the sequence.  Each rank samples inside its own shard with the GLOBAL tile index and the
  GLOBAL per-tile budget, producing an unnormalised partial per head; one all-gather of
  ``[B,H,130]`` fp32 per rank (16.6 KB for 32 heads) follows, then every rank combines locally.
  The reference has no multi-device path; the combine is its finalize step
  (santa_cuda_kernel.cu:386-470) over the union of the shards' tiles.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import capi, ops


def shard_plan(L_total: int, world: int, S: int, block_n: int = 0):
    """Tile-aligned split of a length-``L_total`` sequence over ``world`` ranks.
    Returns (block_n, T_c_global, S_per_tile_global, [(row0, row1, tile0)] per rank)."""
    bn = capi.block_n_rule(L_total, block_n)
    T_c, spt = capi.flash_budget(L_total, bn, S)
    base, extra = divmod(T_c, world)
    plan, t0 = [], 0
    for r in range(world):
        nt = base + (1 if r < extra else 0)
        row0, row1 = t0 * bn, min(L_total, (t0 + nt) * bn)
        plan.append((row0, row1, t0))
        t0 += nt
    return bn, T_c, spt, plan


class PeerExchange:
    """Exchange buffers of a sequence-sharded decode in peer-mapped device memory (NVLink): every rank
    allocates one buffer through torch's symmetric memory, maps all ranks' buffers, and the decode
    kernels store their partials straight into them -- no collective call per step.  One object serves
    one (B, H) problem shape on one stream; the ranks must call in lock-step (as with a collective)."""

    def __init__(self, B: int, H: int, device, group=None, device_counted: bool = False, fused: bool = True):
        # device_counted: the buffers count the steps themselves, so that the call(s) of a step can be
        # captured once in a CUDA graph and replayed (every rank must choose the same mode)
        # fused: the decode call also does the receiving half (one launch sequence per step); otherwise a
        # separate wait-and-combine kernel follows
        self.device_counted = bool(device_counted)
        self.fused = bool(fused)
        self.B, self.H = int(B), int(H)
        self.device = torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        nbytes = int(capi.lib().santa_peer_exchange_bytes(self.world, self.B * self.H))
        if nbytes <= 0:
            raise RuntimeError("santa_b200: a peer exchange takes 1..16 ranks")
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm
            g = group if group is not None else dist.group.WORLD
            self.buf = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
            self.buf.zero_()
            self._handle = symm.rendezvous(self.buf, g.group_name)
            self.ptrs = [int(p) for p in self._handle.buffer_ptrs]
            torch.cuda.synchronize(self.device)
            dist.barrier(group)                      # every buffer is zero before anyone writes
        else:
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            self.ptrs = [self.buf.data_ptr()]
        self.epoch = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # the buffer's own status word (set by either receiving path when a wait ran out)
        self._buf_status = self.buf[136:140].view(torch.int32)

    def check(self) -> None:
        """Synchronise and raise if a wait ran out (a rank never delivered its partial)."""
        code = int(self.status.item()) or int(self._buf_status.item())
        if code != 0:
            raise RuntimeError(f"santa_b200: peer exchange failed with device status {code}")


def seq_sharded_flash_decode(q, K_shard, V_shard, S, seed, L_total, *, block_n=0, group=None,
                             gather_buf: Optional[torch.Tensor] = None, exchange: Optional[PeerExchange] = None):
    """q [B,H,128] (replicated), K_shard/V_shard [B,L_r,KVH,128]: this rank's rows of the cache, as
    given by ``shard_plan``.  Returns (out [B,H,128], m_star [B,H]) on every rank.  With ``exchange`` the
    partials travel through peer-mapped memory (``PeerExchange``) instead of an all-gather."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    bn, T_c, spt, plan = shard_plan(L_total, world, S, block_n)
    row0, row1, tile0 = plan[rank]
    if K_shard.size(1) < row1 - row0:
        raise RuntimeError(f"rank {rank}: shard holds {K_shard.size(1)} rows, plan needs {row1 - row0}")
    B, H = q.size(0), q.size(1)
    mod = _flash_module()   # the compiled module: a few microseconds of host time per call
    if exchange is not None:
        if row1 <= row0:
            raise RuntimeError("the peer exchange needs at least one tile per rank")
        if (exchange.B, exchange.H, exchange.world, exchange.rank) != (B, H, world, rank):
            raise RuntimeError("PeerExchange was built for another problem shape or group")
        exchange.epoch += 1
        epoch = 0 if exchange.device_counted else exchange.epoch
        res = mod.decode_systematic_exchange(q, K_shard, V_shard, S, seed, bn, row1 - row0, 0, tile0, spt,
                                             exchange.ptrs, rank, epoch, exchange.fused)
        if exchange.fused:
            return res
        return mod.lse_combine_wait(exchange.ptrs, rank, epoch, B, H, spt, q.dtype == torch.bfloat16,
                                    exchange.status)
    if row1 > row0:
        part = mod.decode_systematic_partial(q, K_shard, V_shard, S, seed=seed, block_n=bn, valid_len=row1 - row0,
                                             tile_offset=tile0, s_per_tile=spt)
    else:  # more ranks than tiles: an empty shard contributes weight zero
        part = torch.zeros(B, H, 130, device=q.device, dtype=torch.float32)
        part[..., 128] = float("-inf")
    bf16 = q.dtype == torch.bfloat16
    if world == 1:
        return mod.lse_combine(part.unsqueeze(0), spt, bf16)
    if gather_buf is None:
        gather_buf = torch.empty((world,) + tuple(part.shape), device=q.device, dtype=torch.float32)
    # concatenated layout ([world*B,H,130]) is accepted by every backend
    dist.all_gather_into_tensor(gather_buf.view(world * part.size(0), *part.shape[1:]), part, group=group)
    return mod.lse_combine(gather_buf, spt, bf16)


_flash_mod = None


def _flash_module():
    global _flash_mod
    if _flash_mod is None:
        import santa_b200
        santa_b200.enable_dropin()
        import santa_flash_batch_cuda
        _flash_mod = santa_flash_batch_cuda
    return _flash_mod


def batch_sharded_flash_decode(q_local, K_local, V_local, S, seed, batch_offset, **kw):
    """This rank's slice of a batch; ``batch_offset`` is the global index of its first sequence."""
    return ops.flash_decode(q_local, K_local, V_local, S, seed=seed, batch_offset=batch_offset, **kw)


def merge_partials_reference(parts: torch.Tensor, S_per_tile: int):
    """The combine rule in plain torch (any device): used by the CPU/gloo tests of the host logic."""
    A, m, Z = parts[..., :128].double(), parts[..., 128].double(), parts[..., 129].double()
    ms = m.max(0).values
    w = torch.exp(m - ms)
    w = torch.where(torch.isnan(w), torch.zeros_like(w), w)
    Zs = (w * Z).sum(0)
    out = (w[..., None] * A).sum(0) / (Zs * S_per_tile).clamp_min(1e-300)[..., None]
    if S_per_tile <= 0:
        out = out * 0
    return out.float(), ms.float()
