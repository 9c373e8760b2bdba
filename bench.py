#!/usr/bin/env python
"""Decode-attention benchmark of the S2ANTA-Flash hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): santa_flash, B=8 sequences, Hq=32, Hkv=8, head_dim=128, context 32768, S=256,
seed 1690, bf16, K/V ~ N(0,1) with 1% planted heavy hitters, a fresh q every step (pool of 16).
One "step" is one decode call over the whole batch.  N>1 (torchrun, one rank per GPU): every rank
owns its own batch of 8 sequences (batch sharding, no data-path collective, weak scaling).

Timing: W warm-up steps, then blocks of exactly K steps, each block between a barrier +
synchronize on both sides and timed by CUDA events on the launching stream; blocks are repeated
until about a second of device time has passed.  `ms_per_step` is the median block (max over the
ranks' medians), with min / max / repeats and -- at N>1 -- every rank's median beside it.  SM clocks
and throttle reasons are sampled through NVML every few milliseconds during the timed region.

The JSON line carries: `value` = steps/s with inputs resident in HBM (C-ABI path), `e2e` = the same
with host buffers inside the timed region: this step's q / new k,v rows are read from pinned host
memory by the append launch, the output is stored to pinned host memory by the decode call and the
stream is synchronised every step; the result is checked against the reference-facing module
santa_flash_batch_cuda (the KV cache itself is resident device state, as in the reference's runtime), `roofline` for the streaming
kernel against the measured HBM copy peak, `cpu_baseline` (dense SDPA on the host cores, the
reference's only CPU-runnable backend), `vs_reference_cuda_kernels` (the reference's own kernels,
compiled unmodified for sm_100a, timed in the same process on the same inputs) and, as extra
evidence, the ragged santa_prop batch, the sequence-sharded 512k-context case and an end-to-end
Llama-3.1-8B-shaped decode.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

B, H, KVH, D, L, S, SEED = 8, 32, 8, 128, 32768, 256, 1690
QPOOL = 16
WORKLOAD = f"santa_flash B={B} Hq={H} Hkv={KVH} D={D} L={L} S={S} seed={SEED} bf16, 1% heavy hitters"
PROP_WORKLOAD = "santa_prop B=16 ragged L in [8192,65536] (seed-7 draw, sum 562962) S=256"
MIN_TIMED_S = 1.0      # device time to accumulate over the repeated K-step blocks
MAX_BLOCKS = 2000


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def make_inputs(dev, seed, batch=B, length=L, heavy=True):
    """Seeded synthetic q pool / K / V on `dev`: N(0,1) with 1% heavy hitters per (batch, kv-head)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    q0 = torch.randn(batch, H, D, generator=g, device=dev)
    K = torch.randn(batch, length, KVH, D, generator=g, device=dev, dtype=torch.bfloat16)
    V = torch.randn(batch, length, KVH, D, generator=g, device=dev, dtype=torch.bfloat16)
    if heavy:
        nh = length // 100
        for b in range(batch):
            for kv in range(KVH):
                idx = torch.randperm(length, generator=g, device=dev)[:nh]
                qq = q0[b, 4 * kv + (idx % 4)]
                K[b, idx, kv] = (4.0 * qq / qq.norm(dim=-1, keepdim=True)
                                 + 0.1 * torch.randn(nh, D, generator=g, device=dev)).to(torch.bfloat16)
    qpool = [(q0 + 0.5 * torch.randn(batch, H, D, generator=g, device=dev)).to(torch.bfloat16) for _ in range(QPOOL)]
    return qpool, K, V


class ClockSampler:
    """SM clock / throttle-reason samples of one GPU, read through NVML (what nvidia-smi reads) by a
    thread every few milliseconds; `nvidia-smi -lms` is the fallback.  Only reads, never sets."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, cuda_index, period_s=0.004):
        self.samples = []          # (t, sm_mhz, reason mask)
        self.marks = []            # (t0, t1) windows that count
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self._smi = None
        try:
            import pynvml

            pynvml.nvmlInit()
            h = None
            try:
                uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
                h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                vis = os.environ.get("CUDA_VISIBLE_DEVICES")
                idx = cuda_index
                if vis and all(p.strip().isdigit() for p in vis.split(",")):
                    idx = int(vis.split(",")[cuda_index])
                h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def run():
                while not self._stop.is_set():
                    try:
                        mhz = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                        mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                        self.samples.append((time.perf_counter(), float(mhz), int(mask)))
                    except Exception:
                        pass
                    time.sleep(period_s)

            self._thread = threading.Thread(target=run, daemon=True)
            self._thread.start()
        except Exception:
            self._start_smi(cuda_index)

    def _start_smi(self, index):
        self._f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self._smi = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=self._f, stderr=subprocess.DEVNULL)
        except Exception:
            self._smi = None

    def mark(self, t0, t1):
        self.marks.append((t0, t1))

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0, "sm_mhz_min": None}
        sm, reasons = [], set()
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            lo = min((a for a, _ in self.marks), default=0.0)
            hi = max((b for _, b in self.marks), default=float("inf"))
            for t, mhz, mask in self.samples:
                if lo <= t <= hi:
                    sm.append(mhz)
                    for name, bit in self.REASONS:
                        if mask & bit:
                            reasons.add(name)
        elif self._smi is not None:
            self._smi.terminate()
            try:
                self._smi.wait(timeout=5)
            except Exception:
                self._smi.kill()
            self._f.flush()
            self._f.seek(0)
            rows = [r.strip().split(", ") for r in self._f.read().strip().splitlines() if r.strip()]
            self._f.close()
            os.unlink(self._f.name)
            names = [n for n, _ in self.REASONS]
            for r in rows[1:-1] if len(rows) > 3 else rows:
                try:
                    sm.append(float(r[0]))
                    out["sm_max_mhz"] = float(r[1])
                    for n, v in zip(names, r[2:6]):
                        if v.strip() == "Active":
                            reasons.add(n)
                except Exception:
                    pass
        if sm:
            sm.sort()
            out["sm_mhz"] = sm[len(sm) // 2]
            out["sm_mhz_min"] = sm[0]
        out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def dist_setup(n):
    import torch.distributed as dist

    if n > 1 or "RANK" in os.environ:
        rank = int(os.environ.get("RANK", 0))
        local = int(os.environ.get("LOCAL_RANK", rank))
        world = int(os.environ.get("WORLD_SIZE", n))
        torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, local, world
    torch.cuda.set_device(0)
    return 0, 0, 1


def barrier_sync(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x, world, dev):
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_ranks(x, world, dev):
    if world == 1:
        return [x]
    import torch.distributed as dist

    t = torch.tensor([x], device=dev, dtype=torch.float64)
    out = torch.empty(world, device=dev, dtype=torch.float64)
    dist.all_gather_into_tensor(out, t)
    return [float(v) for v in out.tolist()]


def timed_blocks(fn, steps, warmup, world, dev, min_s=None, sampler=None):
    """W warm-up steps, then blocks of exactly K steps; every block sits between barrier + synchronize
    on both sides and is timed by CUDA events on the launching stream.  Blocks repeat until `min_s`
    seconds of device time have passed on the slowest rank.  Returns a dict: `s_per_block` is the
    median block of the slowest rank; `per_rank_ms_per_step` lists every rank's median."""
    min_s = MIN_TIMED_S if min_s is None else min(min_s, MIN_TIMED_S)
    for i in range(warmup):
        fn(i)
    blocks, spent, i0 = [], 0.0, warmup
    while True:
        barrier_sync(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_host0 = time.perf_counter()
        e0.record()
        for i in range(steps):
            fn(i0 + i)
        e1.record()
        barrier_sync(world)
        if sampler is not None:
            sampler.mark(t_host0, time.perf_counter())
        i0 += steps
        dt = e0.elapsed_time(e1) * 1e-3
        blocks.append(dt)
        spent += max_over_ranks(dt, world, dev)   # every rank takes the same decision
        if spent >= min_s or len(blocks) >= MAX_BLOCKS:
            break
    srt = sorted(blocks)
    med = srt[len(srt) // 2]
    per_rank = gather_ranks(med, world, dev)
    return {"s_per_block": max(per_rank), "ms_per_step": max(per_rank) / steps * 1e3,
            "ms_per_step_min": max_over_ranks(srt[0], world, dev) / steps * 1e3,
            "ms_per_step_max": max_over_ranks(srt[-1], world, dev) / steps * 1e3,
            "repeats": len(blocks), "timed_s": spent,
            "per_rank_ms_per_step": [t / steps * 1e3 for t in per_rank]}


def graphed(fn, dev):
    """Capture one call of `fn` in a CUDA graph (after eager warm-up on a side stream) and return a
    function that replays it: both arms of a kernel-to-kernel comparison then run without host time."""
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    g.replay()
    torch.cuda.synchronize(dev)
    return g


def cpu_dense_baseline(budget_s=12.0, length=L, batch=B):
    """Dense SDPA decode (the reference's CPU-runnable backend) on one sequence of the workload's
    shape, fp32, all host threads; scaled to whole-batch steps/s."""
    from oracle.dense_sdpa import sdpa_decode

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(SEED)
    q = torch.randn(1, H, D, generator=g)
    K = torch.randn(1, length, KVH, D, generator=g)
    V = torch.randn(1, length, KVH, D, generator=g)
    sdpa_decode(q, K, V, length)
    times, t_start = [], time.perf_counter()
    while (len(times) < 5 or time.perf_counter() - t_start < budget_s) and len(times) < 200:
        t0 = time.perf_counter()
        sdpa_decode(q, K, V, length)
        times.append(time.perf_counter() - t0)
    times.sort()
    t_seq = times[len(times) // 2]
    return {"value": 1.0 / (t_seq * batch), "unit": "steps/s", "cores": cores, "kind": "port",
            "sample": f"dense fp32 SDPA decode of 1 of the {batch} sequences (L={length}), median of {len(times)} runs, "
                      f"scaled by 1/{batch} to a whole-batch step"}


def reference_arm(args):
    """The reference's own CPU implementation of decode attention for this workload: dense SDPA."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    t0 = time.perf_counter()
    cb = cpu_dense_baseline(budget_s=max(5.0, min(60.0, 2.0 * args.steps)))
    line = {
        "impl": "reference", "metric": "decode_attn_steps_per_sec", "value": cb["value"], "unit": "steps/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / cb["value"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "backend": "reference sdpa backend (dense, exact) on host CPU"},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))


def reference_cuda_flash(dev, qpool, K, V, steps, world):
    """The reference's Flash kernels (compiled unmodified for sm_100a; checker infrastructure) on this
    workload, one captured launch sequence replayed per step."""
    from oracle import ref_gpu

    if not ref_gpu.available():
        return None
    q = qpool[0].clone()
    g = graphed(lambda: ref_gpu.flash_decode(q, K, V, S, seed=SEED), dev)

    def step(i):
        q.copy_(qpool[i % QPOOL])
        g.replay()

    r = timed_blocks(step, steps, 3, world, dev, min_s=0.5)
    del g
    return r


def main():
    global MIN_TIMED_S
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-seq-sharded", action="store_true", help="skip the 512k-context sequence-sharded extra")
    ap.add_argument("--no-prop", action="store_true", help="skip the santa_prop ragged-batch extra")
    ap.add_argument("--no-e2e-model", action="store_true",
                    help="skip the end-to-end Llama-3.1-8B-shaped decode extra (needs ~160 GB of HBM)")
    ap.add_argument("--no-ref-kernels", action="store_true", help="skip timing the reference's CUDA kernels")
    ap.add_argument("--no-b32", action="store_true", help="skip the B=32 variant of the headline workload")
    ap.add_argument("--no-tensor-mode", action="store_true", help="skip the opt-in tensor-core score mode extras")
    ap.add_argument("--min-timed-s", type=float, default=MIN_TIMED_S,
                    help="device seconds to accumulate over the repeated K-step blocks (0: one block; for profiling)")
    ap.add_argument("--score-mode", type=int, default=0, choices=[0, 1],
                    help="score arithmetic of the headline measurement: 0 = the reference's order (default), "
                         "1 = the opt-in tensor-core mode (the line then says so in config.score_mode)")
    ap.add_argument("--e2e-model-batch", type=int, default=32)
    ap.add_argument("--e2e-prefill", action="store_true",
                    help="run the real 512-token-chunk prefill of the end-to-end extra instead of a synthetic cache")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    MIN_TIMED_S = args.min_timed_s

    import santa_b200
    from santa_b200 import ops, sharded

    santa_b200.enable_dropin()
    import santa_flash_batch_cuda as flash_mod  # fails loudly if the extension is missing

    rank, local, world = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    steps, warmup = args.steps, max(3, args.warmup)
    sampler = ClockSampler(local)      # sampling starts before the warm-up
    qpool, K, V = make_inputs(dev, SEED + rank)

    # algorithmic bytes of one step: every valid K row once per kv-head + the distinct sampled V rows
    # + q + out + m_star
    _, _, vrows = ops.flash_decode(qpool[0], K, V, S, seed=SEED, want_vrows=True, batch_offset=rank * B,
                                   score_mode=args.score_mode)
    vrows_total = int(vrows.sum().item())
    alg_bytes = B * L * KVH * D * 2 + vrows_total * D * 2 + 2 * B * H * D * 2 + B * H * 4

    # ---- kernel-resident measurement (C ABI, inputs in HBM) -----------------------------------
    out_dev = torch.empty(B, H, D, device=dev, dtype=torch.bfloat16)
    tm = timed_blocks(lambda i: ops.flash_decode(qpool[i % QPOOL], K, V, S, seed=SEED, batch_offset=rank * B,
                                                 out=out_dev, score_mode=args.score_mode),
                      steps, warmup, world, dev, sampler=sampler)
    clocks = sampler.stop()
    status = ops.workspace_status("flash", dev)

    # ---- end to end through the reference-facing module, host buffers -------------------------
    # This step's inputs -- q and the new token's k / v rows -- sit in pinned host memory.  One launch
    # (the fused RoPE + cache-append + q-pack kernel, here with the identity rotation, so that q and the
    # rows are exactly the given ones) reads them over PCIe, appends the rows to the cache and packs q
    # in device memory; the decode call follows, and its merge kernel stores the result straight into
    # the caller's pinned host buffer.
    q_host = [q.cpu().pin_memory() for q in qpool]
    kv_new_host = torch.randn(2, B, KVH, D, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).pin_memory()
    out_host = torch.empty(B, H, D, dtype=torch.bfloat16).pin_memory()
    q_dev = torch.empty(B, H, D, device=dev, dtype=torch.bfloat16)
    cos1 = torch.ones(B, D, device=dev, dtype=torch.bfloat16)
    sin0 = torch.zeros(B, D, device=dev, dtype=torch.bfloat16)

    def e2e_body(i):
        ops.rope_append(q_host[i], kv_new_host[0], kv_new_host[1], cos1, sin0, K, V, L - 1, q_out=q_dev)
        ops.flash_decode(q_dev, K, V, S, seed=SEED, valid_len=L, out=out_host)

    # first through the reference-facing module + explicit copies in and out (the reference's calling
    # pattern), to have its result; then the timed variant on the same q
    K[:, L - 1].copy_(kv_new_host[0].to(dev))
    V[:, L - 1].copy_(kv_new_host[1].to(dev))
    module_out = flash_mod.decode_systematic_batched(q_host[0].to(dev), K, V, S, seed=SEED, want_vrows=False,
                                                     valid_len=L)[0].cpu()
    out_host.zero_()
    e2e_body(0)
    torch.cuda.synchronize()
    assert torch.equal(module_out, out_host), "host-buffer step differs from the module's output"
    # One CUDA graph per q of the pool (a graph fixes its source address), each holding the whole step;
    # if capture is not possible the step runs eagerly.
    graphs = None
    try:
        graphs = [graphed(lambda i=i: e2e_body(i), dev) for i in range(QPOOL)]
        out_host.zero_()
        graphs[0].replay()
        torch.cuda.synchronize()
        if not torch.equal(module_out, out_host):
            raise RuntimeError("graph replay differs from the eager call")
    except Exception as exc:  # noqa: BLE001
        graphs = None
        e2e_note = f"eager (graph capture failed: {str(exc)[:80]})"
    else:
        e2e_note = ("cuda graph replay per step: one launch reads q and the new k/v rows from pinned host memory "
                    "(append + q pack), decode, result stored by the merge kernel into the pinned host buffer")

    def e2e_step(i):
        if graphs is not None:
            graphs[i % QPOOL].replay()
        else:
            e2e_body(i % QPOOL)
        torch.cuda.current_stream().synchronize()  # the caller consumes the result every step

    te = timed_blocks(e2e_step, steps, 3, world, dev, min_s=0.5)
    h2d = (q_host[0].numel() + kv_new_host.numel()) * 2
    d2h = out_host.numel() * 2

    line = None
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        s_step = tm["s_per_block"] / steps
        ach = alg_bytes / s_step / 1e9
        line = {
            "metric": "decode_attn_steps_per_sec", "value": world / s_step, "unit": "steps/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": tm["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_gpu_batch": B, "parallelism": f"batch-sharded x{world}, no collective",
                       "score_mode": "exact (the reference's fp32 order)" if args.score_mode == 0 else "tensor cores (opt-in)",
                       "l2": "inputs (1 GiB of K+V per GPU) exceed the 126 MB L2", "q": f"pool of {QPOOL} cycled"},
            "timing": {"what": f"median of {tm['repeats']} blocks of {steps} steps (max over ranks of the rank medians)",
                       "ms_per_step_min": tm["ms_per_step_min"], "ms_per_step_max": tm["ms_per_step_max"],
                       "repeats": tm["repeats"], "timed_s": tm["timed_s"],
                       "per_rank_ms_per_step": tm["per_rank_ms_per_step"]},
            "sampled_kv_gbs_per_gpu": ach, "sampled_kv_gbs_total": ach * world,
            "pct_of_measured_hbm_peak": 100.0 * ach / peak, "pct_of_8tbs": 100.0 * ach / 8000.0,
            "algorithmic_bytes_per_step": alg_bytes, "vrows_total": vrows_total,
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "samples": clocks["samples"], "sm_mhz_min": clocks["sm_mhz_min"],
                       "ms_per_step_x_sm_ghz": (tm["ms_per_step"] * clocks["sm_mhz"] / 1e3) if clocks["sm_mhz"] else None},
            "e2e": {"value": world * steps / te["s_per_block"], "unit": "steps/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": steps, "ms_per_step": te["ms_per_step"],
                    "repeats": te["repeats"], "mode": e2e_note},
            "gpu_launches": 2 * steps,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH, "peak_kind": f"of {peak_kind}",
                         "kernel": "stream_kernel<bf16,256,flash> (+ flash_merge_kernel, a few percent of the step)"},
            "device_status_word": status,
        }

    # ---- the reference's own CUDA kernels on the same inputs, same process ----------------------
    if not args.no_ref_kernels:
        rr = None
        try:
            rr = reference_cuda_flash(dev, qpool, K, V, steps, world)
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                line["vs_reference_cuda_kernels"] = {"flash": {"unavailable": str(exc)[:200]}}
        if rank == 0 and rr is not None:
            line["vs_reference_cuda_kernels"] = {"flash": {
                "what": "reference Flash kernels compiled unmodified for sm_100a, launch sequence replayed from a "
                        "CUDA graph, same inputs / steps / timing blocks",
                "reference_ms_per_step": rr["ms_per_step"], "ours_ms_per_step": tm["ms_per_step"],
                "speedup": rr["ms_per_step"] / tm["ms_per_step"], "repeats": rr["repeats"]}}
        elif rank == 0 and "vs_reference_cuda_kernels" not in line:
            line["vs_reference_cuda_kernels"] = {"flash": {"unavailable": "oracle/_ref is not built"}}

    # ---- extra: the opt-in tensor-core score mode on the same workload, beside the exact mode -------
    if not args.no_tensor_mode:
        tt = timed_blocks(lambda i: ops.flash_decode(qpool[i % QPOOL], K, V, S, seed=SEED, batch_offset=rank * B,
                                                     out=out_dev, score_mode=1), steps, 3, world, dev, min_s=0.5)
        r0 = ops.flash_decode(qpool[0], K, V, S, seed=SEED, batch_offset=rank * B, want_vrows=True, trace=True)
        r1 = ops.flash_decode(qpool[0], K, V, S, seed=SEED, batch_offset=rank * B, want_vrows=True, trace=True,
                              score_mode=1)
        c0, c1 = r0[3].counts, r1[3].counts
        sampled, differing = int((c0 > 0).sum().item()), int((c0 != c1).sum().item())
        dd = (r0[0].float() - r1[0].float()).abs()
        if rank == 0:
            peak, _ = measured_peak_gbs()
            bt = alg_bytes - vrows_total * D * 2 + int(r1[2].sum().item()) * D * 2
            line["score_mode_tensor"] = {
                "what": "scores on the tensor cores (mma.sync, split 16-bit query), opt-in; everything else unchanged. "
                        "The exact mode's counts equal the reference's bit for bit, so the mismatch below is the "
                        "distance from the reference",
                "ms_per_step": tt["ms_per_step"], "exact_ms_per_step": tm["ms_per_step"],
                "sampled_kv_gbs_per_gpu": bt / (tt["ms_per_step"] * 1e-3) / 1e9,
                "frac_of_measured_hbm_peak": bt / (tt["ms_per_step"] * 1e-3) / 1e9 / peak,
                "pct_of_8tbs": bt / (tt["ms_per_step"] * 1e-3) / 1e9 / 80.0,
                "count_entries_differing": differing, "count_entries_sampled": sampled,
                "mismatch_rate": differing / max(1, sampled),
                "out_vs_exact_max_abs": dd.max().item(), "out_vs_exact_mean_abs": dd.mean().item(),
                "repeats": tt["repeats"]}
        del r0, r1, c0, c1

    # ---- extra: the same workload at B=32 (the fixed per-call cost amortised over 4x the tiles) --
    if not args.no_b32:
        del K, V, qpool
        torch.cuda.empty_cache()
        qp32, K32, V32 = make_inputs(dev, SEED + 32 + rank, batch=32)
        vr32 = int(ops.flash_decode(qp32[0], K32, V32, S, seed=SEED, want_vrows=True)[2].sum().item())
        o32 = torch.empty(32, H, D, device=dev, dtype=torch.bfloat16)
        t32 = timed_blocks(lambda i: ops.flash_decode(qp32[i % QPOOL], K32, V32, S, seed=SEED, out=o32),
                           max(5, steps // 4), 3, world, dev, min_s=0.5)
        t32t = None
        if not args.no_tensor_mode:
            t32t = timed_blocks(lambda i: ops.flash_decode(qp32[i % QPOOL], K32, V32, S, seed=SEED, out=o32,
                                                           score_mode=1), max(5, steps // 4), 3, world, dev, min_s=0.5)
        if rank == 0:
            b32 = 32 * L * KVH * D * 2 + vr32 * D * 2 + 2 * 32 * H * D * 2 + 32 * H * 4
            peak, _ = measured_peak_gbs()
            line["flash_b32"] = {"workload": WORKLOAD.replace(f"B={B} ", "B=32 "), "ms_per_step": t32["ms_per_step"],
                                 "sampled_kv_gbs_per_gpu": b32 / (t32["ms_per_step"] * 1e-3) / 1e9,
                                 "frac_of_measured_hbm_peak": b32 / (t32["ms_per_step"] * 1e-3) / 1e9 / peak,
                                 "repeats": t32["repeats"]}
            if t32t is not None:
                line["flash_b32"]["tensor_score_mode"] = {
                    "ms_per_step": t32t["ms_per_step"],
                    "sampled_kv_gbs_per_gpu": b32 / (t32t["ms_per_step"] * 1e-3) / 1e9,
                    "frac_of_measured_hbm_peak": b32 / (t32t["ms_per_step"] * 1e-3) / 1e9 / peak,
                    "pct_of_8tbs": b32 / (t32t["ms_per_step"] * 1e-3) / 1e9 / 80.0}
        del K32, V32, qp32
        torch.cuda.empty_cache()
    else:
        del K, V, qpool
        torch.cuda.empty_cache()

    # ---- extra: one 512k-token sequence, KV sharded along the sequence over the N GPUs -----------
    if not args.no_seq_sharded:
        res3 = seq_sharded_extra(dev, rank, world, steps, sharded, ops)
        if rank == 0:
            line["seq_sharded_512k"] = res3

    # ---- extra: santa_prop on the ragged batch, scalar entry point per sequence and one ragged call
    if not args.no_prop:
        res2 = prop_extra(dev, rank, world, steps, args)
        if rank == 0:
            line["prop_ragged_config2"] = res2
            if "reference" in res2:
                line.setdefault("vs_reference_cuda_kernels", {})["prop"] = res2.pop("reference")

    # ---- extra: end-to-end decode of a Llama-3.1-8B-shaped model -----------------------------------
    if not args.no_e2e_model:
        res4 = e2e_model_decode(dev, args.e2e_model_batch, world, prefill=args.e2e_prefill,
                                tensor_mode=not args.no_tensor_mode)
        if rank == 0:
            line["e2e_llama8b_decode"] = res4

    # ---- extra: the reference's CPU-runnable case (B=1, L=4096, S=32) on the GPU: a latency figure ---
    if world == 1:
        line["config0_b1_l4096"] = config0_extra(dev, steps, args)

    if rank == 0:
        if world == 1:
            line["cpu_baseline"] = cpu_dense_baseline()
            c0 = cpu_dense_baseline(budget_s=3.0, length=4096, batch=1)
            c0["sample"] = "dense fp32 SDPA decode, B=1 Hq=32 Hkv=8 D=128 L=4096 (the reference's CPU-runnable case)"
            line["cpu_baseline_b1_l4096"] = c0
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


def config0_extra(dev, steps, args):
    """B=1, L=4096, S=32, seed 1690 (K scaled by 1/sqrt(D)): the case the reference can run on a CPU.  The
    16 MiB of K and V stay in L2, so this is the latency of one call, replayed from a CUDA graph; the
    reference's kernels are timed the same way beside it."""
    from santa_b200 import ops

    g = torch.Generator().manual_seed(SEED)
    q0 = torch.randn(1, H, D, generator=g).to(torch.bfloat16).to(dev)
    K0 = (torch.randn(1, 4096, KVH, D, generator=g) / math.sqrt(D)).to(torch.bfloat16).to(dev)
    V0 = torch.randn(1, 4096, KVH, D, generator=g).to(torch.bfloat16).to(dev)
    o0 = torch.empty(1, H, D, device=dev, dtype=torch.bfloat16)
    n0 = max(50, steps)
    g0 = graphed(lambda: ops.flash_decode(q0, K0, V0, 32, seed=SEED, out=o0), dev)
    t0 = timed_blocks(lambda i: g0.replay(), n0, 5, 1, dev, min_s=0.2)
    res = {"workload": "santa_flash B=1 Hq=32 Hkv=8 D=128 L=4096 S=32 seed=1690 bf16 (L2-resident: a latency figure)",
           "ms_per_step": t0["ms_per_step"], "steps_per_s": 1e3 / t0["ms_per_step"], "how": "cuda graph replay"}
    if not args.no_ref_kernels:
        from oracle import ref_gpu
        if ref_gpu.available():
            r = ref_gpu.flash_decode(q0, K0, V0, 32, seed=SEED)
            res["out_vs_reference_kernels_max_abs"] = (r.out.float() - o0.float()).abs().max().item()
            gr = graphed(lambda: ref_gpu.flash_decode(q0, K0, V0, 32, seed=SEED), dev)
            tr = timed_blocks(lambda i: gr.replay(), n0, 5, 1, dev, min_s=0.2)
            res["reference_cuda_kernels_ms_per_step"] = tr["ms_per_step"]
            del gr
    del g0
    return res


def seq_sharded_extra(dev, rank, world, steps, sharded, ops):
    """B=1, L=524288, S=1024 (Flash rule), the KV cache split along the sequence over the ranks; the
    step includes the exchange of the per-head partials and the combine.  Strong scaling."""
    L3, S3 = 524288, 1024
    bn, T_c, spt, plan = sharded.shard_plan(L3, world, S3)
    row0, row1, _ = plan[rank]
    # every rank draws the same full-length stream and keeps its rows (same data at every N)
    qp3, K3f, V3f = make_inputs(dev, SEED + 3, batch=1, length=L3)
    # the unsharded result, computed by every rank on the whole sequence before it keeps its shard
    whole = [ops.flash_decode(qp3[i], K3f, V3f, S3, seed=SEED)[0].clone() for i in range(2)]
    n3 = max(20, steps // 5)
    # ... and its time on this GPU: the one-GPU reference of the strong-scaling efficiency
    t1 = timed_blocks(lambda i: ops.flash_decode(qp3[i % QPOOL], K3f, V3f, S3, seed=SEED), n3, 5, world, dev, min_s=0.3)
    K3, V3 = K3f[:, row0:row1].contiguous(), V3f[:, row0:row1].contiguous()
    del K3f, V3f
    torch.cuda.empty_cache()
    gbuf = torch.empty(world, 1, H, 130, device=dev, dtype=torch.float32)
    checks = {}
    for i in range(2):
        got = sharded.seq_sharded_flash_decode(qp3[i], K3, V3, S3, SEED, L3, gather_buf=gbuf)[0]
        err = (got.float() - whole[i].float()).abs().max().item()
        checks[f"allgather_vs_unsharded_maxabs_q{i}"] = max_over_ranks(err, world, dev)
    t3 = timed_blocks(lambda i: sharded.seq_sharded_flash_decode(qp3[i % QPOOL], K3, V3, S3, SEED, L3, gather_buf=gbuf),
                      n3, 5, world, dev, min_s=0.3)
    # the same step with the partials exchanged through peer-mapped memory instead of the all-gather
    t3x, x_note, ex, t3g = None, None, None, None
    try:
        if world > 1:
            import importlib
            importlib.import_module("torch.distributed._symmetric_memory")
    except Exception as exc:  # noqa: BLE001
        x_note = f"peer exchange unavailable: {str(exc)[:120]}"
    if max_over_ranks(1.0 if x_note else 0.0, world, dev) != 0.0:
        x_note = x_note or "peer exchange unavailable on another rank"
    try:
        if x_note:
            raise RuntimeError(x_note)
        ex = sharded.PeerExchange(1, H, dev)
        for i in range(2):
            got3 = sharded.seq_sharded_flash_decode(qp3[i], K3, V3, S3, SEED, L3, exchange=ex)[0]
            ex.check()
            err = (got3.float() - whole[i].float()).abs().max().item()
            checks[f"peer_vs_unsharded_maxabs_q{i}"] = err
            if err > 2e-2:
                raise RuntimeError(f"peer exchange result differs from the unsharded result by {err}")
    except Exception as exc:  # noqa: BLE001  (symmetric memory may be unavailable on a box)
        x_note = x_note or f"peer exchange unavailable: {str(exc)[:120]}"
    # every rank must agree before entering a timed loop with barriers
    if max_over_ranks(1.0 if x_note else 0.0, world, dev) == 0.0:
        t3x = timed_blocks(lambda i: sharded.seq_sharded_flash_decode(qp3[i % QPOOL], K3, V3, S3, SEED, L3, exchange=ex),
                           n3, 5, world, dev, min_s=0.3)
        ex.check()
    elif x_note is None:
        x_note = "peer exchange unavailable on another rank"
    # ... and with the calls of a step captured once in a CUDA graph (device-counted epochs)
    if t3x is not None:
        exg = sharded.PeerExchange(1, H, dev, device_counted=True)
        q3 = qp3[0].clone()
        side3 = torch.cuda.Stream()
        side3.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side3):
            for _ in range(2):
                sharded.seq_sharded_flash_decode(q3, K3, V3, S3, SEED, L3, exchange=exg)
        torch.cuda.current_stream().wait_stream(side3)
        torch.cuda.synchronize()
        graph3 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph3, stream=side3):
            out3 = sharded.seq_sharded_flash_decode(q3, K3, V3, S3, SEED, L3, exchange=exg)
        graph3.replay()
        exg.check()
        same = (out3[0].float() - whole[0].float()).abs().max().item() <= 2e-2
        if max_over_ranks(0.0 if same else 1.0, world, dev) == 0.0:
            def graph_step(i):
                q3.copy_(qp3[i % QPOOL])
                graph3.replay()

            t3g = timed_blocks(graph_step, n3, 5, world, dev, min_s=0.3)
            exg.check()
        del graph3
    res = None
    if rank == 0:
        kb = L3 * KVH * D * 2
        res = {
            "workload": f"santa_flash B=1 L={L3} S={S3}, KV sharded over {world} GPU(s); the step includes the "
                        "exchange of (partial, m, Z) and the combine",
            "scaling": "strong", "checks": checks,
            "allgather": {"what": "NCCL all-gather of [1,32,130] fp32 per rank + local combine",
                          "ms_per_step": t3["ms_per_step"], "k_gbs_total": kb / (t3["ms_per_step"] * 1e-3) / 1e9,
                          "per_rank_ms_per_step": t3["per_rank_ms_per_step"]},
            "peer_exchange": ({"what": "partials stored into every rank's peer-mapped buffer by the merge kernel, "
                                       "which then waits (bounded) for the other ranks' rows and combines; no collective call",
                               "ms_per_step": t3x["ms_per_step"], "k_gbs_total": kb / (t3x["ms_per_step"] * 1e-3) / 1e9,
                               "per_rank_ms_per_step": t3x["per_rank_ms_per_step"],
                               "ms_per_step_graph_replay": t3g["ms_per_step"] if t3g else None} if t3x else x_note),
            "ms_per_step": min(t3["ms_per_step"], t3x["ms_per_step"]) if t3x else t3["ms_per_step"]}
        res["unsharded_one_gpu_ms_per_step"] = t1["ms_per_step"]
        res["efficiency_vs_n1"] = t1["ms_per_step"] / (world * res["ms_per_step"])
    del K3, V3, qp3
    torch.cuda.empty_cache()
    return res


def prop_extra(dev, rank, world, steps, args):
    """santa_prop on 16 ragged sequences, S=256: the adapter's loop of 16 scalar calls, one ragged call,
    and -- for a kernel-to-kernel comparison -- the reference's own Prop kernels in the same loop."""
    import santa_prop_batch_cuda as prop_mod

    lengths = torch.randint(8192, 65537, (16,), generator=torch.Generator().manual_seed(7)).tolist()
    qp2, K2, V2 = make_inputs(dev, SEED + 2 + rank, batch=1, length=sum(lengths))
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    Ks = [K2[0, offs[i]:offs[i + 1]] for i in range(16)]   # contiguous [L_b, KVH, D] views, as the adapter passes
    Vs = [V2[0, offs[i]:offs[i + 1]] for i in range(16)]
    vr2 = sum(int(prop_mod.decode_systematic_scalar(qp2[0][0], Ks[i], Vs[i], S, seed=SEED, want_vrows=True)[2]
                  .sum().item()) for i in range(16))

    def prop_step(i):
        q = qp2[i % QPOOL][0]
        for b in range(16):
            prop_mod.decode_systematic_scalar(q, Ks[b], Vs[b], S, seed=SEED, want_vrows=False)

    n2 = max(20, steps // 10)
    t2 = timed_blocks(prop_step, n2, 3, world, dev, min_s=0.4)
    # the same loop replayed from a CUDA graph, and the reference's own kernels likewise
    ref_res = None
    try:
        qg = qp2[0][0].clone()
        g_ours = graphed(lambda: [prop_mod.decode_systematic_scalar(qg, Ks[b], Vs[b], S, seed=SEED) for b in range(16)],
                         dev)

        def ours_graph_step(i):
            qg.copy_(qp2[i % QPOOL][0])
            g_ours.replay()

        t2g = timed_blocks(ours_graph_step, n2, 3, world, dev, min_s=0.4)
        del g_ours
        if not args.no_ref_kernels:
            from oracle import ref_gpu

            if ref_gpu.available():
                g_ref = graphed(lambda: [ref_gpu.prop_decode(qg, Ks[b], Vs[b], S, seed=SEED) for b in range(16)], dev)

                def ref_graph_step(i):
                    qg.copy_(qp2[i % QPOOL][0])
                    g_ref.replay()

                tr = timed_blocks(ref_graph_step, n2, 3, world, dev, min_s=0.4)
                del g_ref
                ref_res = {"what": "reference Prop kernels compiled unmodified for sm_100a, the adapter's loop of 16 "
                                   "per-sequence launch sequences replayed from a CUDA graph; ours likewise",
                           "reference_ms_per_step": tr["ms_per_step"], "ours_loop_ms_per_step": t2g["ms_per_step"]}
    except Exception as exc:  # noqa: BLE001
        ref_res = {"unavailable": str(exc)[:200]}
        t2g = None
    # the same 16 sequences as one padded cache [16, 65536, KVH, D] and ONE ragged call per step
    Lmax = 65536
    Kr = torch.zeros(16, Lmax, KVH, D, device=dev, dtype=torch.bfloat16)
    Vr = torch.zeros(16, Lmax, KVH, D, device=dev, dtype=torch.bfloat16)
    for b in range(16):
        Kr[b, :lengths[b]].copy_(Ks[b])
        Vr[b, :lengths[b]].copy_(Vs[b])
    del K2, V2, Ks, Vs
    torch.cuda.empty_cache()
    lens_dev = torch.tensor(lengths, dtype=torch.int32, device=dev)
    qr = [qp2[i][0].unsqueeze(0).expand(16, H, D).contiguous() for i in range(QPOOL)]
    vr3 = int(prop_mod.decode_systematic_ragged(qr[0], Kr, Vr, lens_dev, S, seed=SEED, want_vrows=True)[2]
              .sum().item())
    t2r = timed_blocks(lambda i: prop_mod.decode_systematic_ragged(qr[i % QPOOL], Kr, Vr, lens_dev, S, seed=SEED),
                       n2, 3, world, dev, min_s=0.4)
    t2rt = None
    if not args.no_tensor_mode:
        t2rt = timed_blocks(lambda i: prop_mod.decode_systematic_ragged(qr[i % QPOOL], Kr, Vr, lens_dev, S, seed=SEED,
                                                                         score_mode=1), n2, 3, world, dev, min_s=0.4)
    res = None
    if rank == 0:
        fixed = 16 * (2 * H * D * 2 + H * 4)
        pb = sum(lengths) * KVH * D * 2 + vr2 * D * 2 + fixed
        pbr = sum(lengths) * KVH * D * 2 + vr3 * D * 2 + fixed
        res = {
            "workload": PROP_WORKLOAD,
            "ragged_call": {
                "what": "one decode_systematic_ragged call per step (4 kernels), lengths in device memory",
                "steps_per_s": world / (t2r["ms_per_step"] * 1e-3), "ms_per_step": t2r["ms_per_step"],
                "sampled_kv_gbs_per_gpu": pbr / (t2r["ms_per_step"] * 1e-3) / 1e9, "algorithmic_bytes_per_step": pbr,
                "repeats": t2r["repeats"],
                "tensor_score_mode_ms_per_step": t2rt["ms_per_step"] if t2rt else None,
                "tensor_score_mode_gbs": (pbr / (t2rt["ms_per_step"] * 1e-3) / 1e9) if t2rt else None},
            "per_sequence_loop": {
                "what": "16 decode_systematic_scalar calls per step (the reference adapter's loop, 4 kernels each)",
                "steps_per_s": world / (t2["ms_per_step"] * 1e-3), "ms_per_step": t2["ms_per_step"],
                "ms_per_step_graph_replay": t2g["ms_per_step"] if t2g else None,
                "sampled_kv_gbs_per_gpu": pb / (t2["ms_per_step"] * 1e-3) / 1e9, "algorithmic_bytes_per_step": pb},
            "scaling": "weak"}
        if ref_res is not None:
            if "reference_ms_per_step" in ref_res:
                ref_res["ours_ragged_ms_per_step"] = t2r["ms_per_step"]
                ref_res["speedup_loop_vs_loop"] = ref_res["reference_ms_per_step"] / ref_res["ours_loop_ms_per_step"]
                ref_res["speedup_ragged_vs_reference_loop"] = ref_res["reference_ms_per_step"] / t2r["ms_per_step"]
            res["reference"] = ref_res
    del qp2, Kr, Vr, qr
    torch.cuda.empty_cache()
    return res


def e2e_model_decode(dev, batch, world, prompt_len=32768, new_tokens=128, prefill=False, tensor_mode=True):
    """Random-init (seed 0) Llama-3.1-8B-shaped decoder, `batch` sequences with `prompt_len` cached tokens
    each, `new_tokens` greedy tokens with santa_flash S=256; one replica per GPU.  By default the caches
    are filled with seeded N(0,1) values instead of running the prefill (random weights: the prefill
    would produce values of no more meaning, and only the decode phase is the metric); `prefill=True`
    runs the real 512-token-chunk prefill of uniform-random token ids first.  Returns per-replica
    numbers; the whole-job token rate is world x the replica's."""
    import torch.distributed as dist
    from santa_b200.runtime import DecodeRuntime, LlamaShape

    torch.cuda.empty_cache()
    out = {"workload": f"Llama-3.1-8B shape, random init seed 0, B={batch} x {prompt_len} cached tokens, "
                       f"{new_tokens} greedy tokens, santa_flash S={S}, CUDA-graph step, 1 replica per GPU",
           "cache": "real chunked prefill (512-token chunks)" if prefill else "synthetic N(0,1) fill (no prefill run)"}
    try:
        rt = DecodeRuntime(LlamaShape(), batch, prompt_len + new_tokens, dev, attention="santa_flash", S=S,
                           attn_seed=SEED, weight_seed=0)
        if prefill:
            ids = torch.randint(0, rt.shape.vocab, (batch, prompt_len), generator=torch.Generator().manual_seed(11))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            first = rt.prefill(ids.to(dev), chunk=512, seqs_per_pass=2)
            e1.record()
            torch.cuda.synchronize(dev)
            out["prefill_s"] = e0.elapsed_time(e1) * 1e-3
            out["prefill_tokens_per_s"] = batch * prompt_len / out["prefill_s"]
        else:
            rt.fill_cache_synthetic(prompt_len, seed=SEED + 4)
            first = torch.zeros(batch, rt.shape.vocab, device=dev)
            first[:, 1] = 1.0
        rt.capture(prompt_len + new_tokens)
        rt.generate(first, prompt_len, 4)                           # warm-up replays
        if world > 1:
            dist.barrier()
        res = rt.generate(first, prompt_len, new_tokens)
        t = torch.tensor([res["decode_time_s"]], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
        steps_fwd = res["steps_sampled"] - 1                         # forward passes inside the timed loop
        # attention share: eager steps with events around every layer's attention call
        rt.attn_events = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        rt.pos.fill_(prompt_len)
        rt._bn = rt._plan_tile(prompt_len + new_tokens)
        for _ in range(2):
            rt._step(prompt_len + new_tokens)
        rt.attn_events = []
        e0.record()
        for _ in range(3):
            rt._step(prompt_len + new_tokens)
        e1.record()
        torch.cuda.synchronize(dev)
        attn_ms = sum(a.elapsed_time(b) for a, b in rt.attn_events) / 3
        eager_ms = e0.elapsed_time(e1) / 3
        kv_bytes = 32 * (batch * prompt_len * KVH * D * 2)           # K rows read per step, all layers
        out.update({
            "tokens_per_s": world * res["timed_generated_tokens"] / dt,
            "ms_per_step_graph": dt / max(1, steps_fwd) * 1e3,
            "ms_per_step_eager": eager_ms, "attention_ms_per_step": attn_ms,
            "attention_share_of_eager_step": attn_ms / eager_ms,
            "attention_k_gbs": kv_bytes / (attn_ms * 1e-3) / 1e9,
            "hbm_gb_allocated": torch.cuda.max_memory_allocated(dev) / 1e9,
            "device_status_word": res["device_status_word"]})
        if tensor_mode:   # the same generation with the opt-in tensor-core scores in every attention call
            rt.score_mode = 1
            rt.capture(prompt_len + new_tokens)
            rt.generate(first, prompt_len, 4)
            if world > 1:
                dist.barrier()
            res1 = rt.generate(first, prompt_len, new_tokens)
            t = torch.tensor([res1["decode_time_s"]], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out["tensor_score_mode"] = {
                "tokens_per_s": world * res1["timed_generated_tokens"] / float(t.item()),
                "ms_per_step_graph": float(t.item()) / max(1, res1["steps_sampled"] - 1) * 1e3,
                "device_status_word": res1["device_status_word"]}
        del rt
    except torch.OutOfMemoryError as exc:
        out["error"] = f"out of device memory: {str(exc)[:120]}"
    torch.cuda.empty_cache()
    return out


# dram__bytes_read.sum + dram__bytes_write.sum of one stream_kernel launch on this workload, from one
# ncu capture of that kernel (read 557.80 MB + write 10.40 MB).
TRAFFIC_BYTES_PER_LAUNCH = 568_195_840

if __name__ == "__main__":
    main()
