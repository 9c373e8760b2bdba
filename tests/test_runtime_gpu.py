"""The decode runtime on a GPU: one decode step equals a prefill of the extended prompt (dense
backend), and the CUDA-graph replay of the sampled-attention step equals its eager run."""
import pytest
import torch

from santa_b200.runtime import DecodeRuntime, LlamaShape

pytestmark = pytest.mark.gpu

SHAPE = LlamaShape(hidden=512, layers=2, heads=4, kv_heads=1, head_dim=128, intermediate=1024, vocab=1000)


def test_decode_steps_equal_prefill_of_the_extended_prompt():
    dev = torch.device("cuda:0")
    B, L, new = 2, 45, 5
    ids = torch.randint(0, 1000, (B, L), generator=torch.Generator().manual_seed(2)).to(dev)
    rt = DecodeRuntime(SHAPE, B, 64, dev, attention="sdpa", init_std=0.05)
    last = rt.prefill(ids, chunk=16)
    res = rt.generate(last, L, new, use_graph=False)
    toks = res["generated_token_ids_all"].to(dev)
    assert toks.shape == (B, new) and res["steps_sampled"] == new and res["timed_generated_tokens"] == B * new
    assert res["device_status_word"] == 0 and rt.pos.tolist() == [L + new - 1] * B
    logits_step = rt.logits.clone()                       # logits after feeding token new-2 at position L+new-2
    k_rows = rt.k_cache[1][:, L:L + new - 1].clone()
    rt2 = DecodeRuntime(SHAPE, B, 64, dev, attention="sdpa", init_std=0.05)
    last2 = rt2.prefill(torch.cat([ids, toks[:, :new - 1]], dim=1), chunk=16)
    assert (logits_step - last2).abs().max().item() < 0.06 * max(1.0, last2.abs().max().item())
    assert (k_rows.float() - rt2.k_cache[1][:, L:L + new - 1].float()).abs().max().item() < 0.06
    assert torch.equal(last.argmax(-1), toks[:, 0])


@pytest.mark.parametrize("backend", ["santa_flash", "santa_prop"])
def test_graph_replay_of_the_sampled_step_equals_eager_and_stops_in_lockstep(backend):
    dev = torch.device("cuda:0")
    B, L, new = 3, 700, 6
    outs = []
    for use_graph in (False, True):
        rt = DecodeRuntime(SHAPE, B, 1024, dev, attention=backend, S=64, init_std=0.05)
        rt.fill_cache_synthetic(L, seed=4)
        first = torch.zeros(B, 1000, device=dev)
        first[:, 7] = 1.0
        res = rt.generate(first, L, new, use_graph=use_graph)
        outs.append((res["generated_token_ids_all"], rt.logits.clone(), rt.k_cache[1][:, L:L + new].clone()))
        assert res["device_status_word"] == 0 and (res["generated_token_ids_all"][:, 0] == 7).all()
        assert rt.pos.tolist() == [L + new - 1] * B
        assert torch.isfinite(rt.logits).all()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert torch.equal(outs[0][2], outs[1][2])
    # stop tokens: a finished sequence keeps emitting the stop token; "all_finished" ends the loop early
    rt = DecodeRuntime(SHAPE, B, 1024, dev, attention=backend, S=64, init_std=0.05)
    rt.fill_cache_synthetic(L, seed=4)
    first = torch.zeros(B, 1000, device=dev)
    first[:, 7] = 1.0
    res = rt.generate(first, L, new, stop_token_ids=[7], lockstep_stop_mode="all_finished")
    assert res["steps_sampled"] == 1 and (res["generated_token_ids_all"] == 7).all()


def test_longctx_harness_writes_the_reference_files(tmp_path):
    import csv
    import json
    from santa_b200 import bench_longctx
    out = tmp_path / "res"
    bench_longctx.main(["--out-dir", str(out), "--batch-size", "2", "--prompt-len", "300", "--max-new-tokens", "5",
                        "--backends", "santa_flash", "sdpa", "--timed-runs", "2", "--warmup-runs", "1",
                        "--layers", "2", "--hidden", "512", "--heads", "4", "--kv-heads", "1",
                        "--intermediate", "1024", "--vocab", "1000", "--prefill-chunk-size", "128"])
    names = {"invocation.json", "config.json", "batch_metrics.jsonl", "run_metrics.jsonl", "generations.jsonl", "aggregates.json",
             "aggregates.csv", "backend_agreement.json"}
    assert names <= {p.name for p in out.iterdir()}
    runs = [json.loads(x) for x in open(out / "run_metrics.jsonl")]
    assert len(runs) == 6 and {r["backend"] for r in runs} == {"santa_flash", "sdpa"}
    assert all(r["timed_generated_tokens"] == 10 and r["output_tokens_per_s"] > 0 for r in runs)
    batches = [json.loads(x) for x in open(out / "batch_metrics.jsonl")]
    assert all(b["steps_sampled"] == 5 and b["prompt_len"] == 300 and b["prefill_time_s"] > 0 for b in batches)
    rows = list(csv.DictReader(open(out / "aggregates.csv")))
    assert [r["backend"] for r in rows] == ["santa_flash", "sdpa"] and rows[0]["runs"] == "2"
    agree = json.load(open(out / "backend_agreement.json"))
    assert agree[0]["backend_a"] == "santa_flash" and agree[0]["comparable_examples"] == 4


def test_backend_objects_follow_the_reference_adapter_contract():
    """decode(q_bhd, k_nhd, v_nhd, valid_len) of the backend objects: Flash equals the module call; Prop's
    single ragged call equals the reference adapter's per-sequence loop in tolerance; dense sdpa is close
    to a large-S sampled estimate; valid_len may be a device tensor."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import cases
    from santa_b200 import backends
    dev = torch.device("cuda:0")
    q, K, V = cases.make_qkv(3, 6000, 8, "bf16", 99, 1.0, True)
    q, K, V = q.to(dev), K.to(dev), V.to(dev)
    L = 5000
    fb = backends.make_backend("santa_flash", santa_s=256, santa_seed=7)
    out = fb.decode(q, K, V, L)
    assert fb.actual_mode == "batch" and out.shape == (3, 32, 128) and fb.info()["module"] == "santa_flash_batch_cuda"
    assert torch.equal(out, fb.module.decode_systematic_batched(q, K, V, 256, seed=7, valid_len=L)[0])
    lens = torch.full((3,), L, dtype=torch.int32, device=dev)
    out_t = fb.decode(q, K, V, lens)
    assert fb.actual_mode == "batch_ragged" and (out_t.float() - out.float()).abs().max().item() <= 2e-2
    pb = backends.make_backend("santa_prop", santa_s=256, santa_seed=7)
    pl = backends.SantaPropBackend(S=256, seed=7, loop=True)
    o_r, o_l = pb.decode(q, K, V, L), pl.decode(q, K, V, L)
    assert (pb.actual_mode, pl.actual_mode) == ("batch_ragged", "single_loop_fallback")
    assert (o_r.float() - o_l.float()).abs().max().item() <= 2e-2
    dense = backends.make_backend("sdpa").decode(q, K, V, L)
    big = backends.SantaFlashBackend(S=L * 8, seed=7).decode(q, K, V, L)
    assert (big.float() - dense.float()).abs().mean().item() < 0.05
    with pytest.raises(backends.BackendError):
        backends.make_backend("fa2")
    # short contexts: the default Prop backend must sample what the reference adapter's loop samples
    # (32-row tiles up to 1536 tokens, 64-row tiles up to 3072), not the ragged call's 256-row tiles
    for Ls in (700, 2500):
        o_d, o_l = pb.decode(q, K, V, Ls), pl.decode(q, K, V, Ls)
        assert pb.actual_mode == "single_loop_fallback" and torch.equal(o_d, o_l)
    p256 = backends.SantaPropBackend(S=256, seed=7, block_n=256)
    p256.decode(q, K, V, 700)
    assert p256.actual_mode == "batch_ragged"
    # the start-up check of the reference (two sequences of 16 cached tokens): 32-row tiles, one tile
    for b in (fb, pb, pl, backends.make_backend("sdpa")):
        rep = b.smoke_test(device=dev, dtype=torch.bfloat16, num_heads=32, num_kv_heads=8, head_dim=128, valid_len=16)
        assert rep["output_shape"] == [2, 32, 128] and rep["backend"] == b.name
