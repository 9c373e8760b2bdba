"""Long-context decode benchmark of this package's runtime, writing the reference harness's files.

    python -m santa_b200.bench_longctx --out-dir results --batch-size 4 --prompt-len 8192 \\
        --max-new-tokens 32 --backends santa_flash sdpa --timed-runs 3

Writes ``config.json``, ``batch_metrics.jsonl``, ``run_metrics.jsonl``, ``generations.jsonl``,
``aggregates.json``, ``aggregates.csv``, ``backend_agreement.json`` and ``invocation.json`` into the output directory, with
the field names of tutorial_code/benchmark_longctx.py (:350-369, :396-425, :486-530, :656-722) of
the reference.  The model is random-initialised from the given shape and the prompts are uniform
random token ids: there are no weights, tokenizer or evaluation prompts to load, so text and
exact-match fields are NaN and agreement is measured on token ids.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch

from . import report
from .runtime import DecodeRuntime, LlamaShape


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out-dir", required=True)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--num-batches", type=int, default=1)
    ap.add_argument("--prompt-len", type=int, default=8192)
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--prefill-chunk-size", type=int, default=512)
    ap.add_argument("--backends", nargs="+", default=["santa_flash"], choices=["santa_flash", "santa_prop", "sdpa"])
    ap.add_argument("--santa-s", type=int, default=256)
    ap.add_argument("--santa-seed", type=int, default=1690)
    ap.add_argument("--santa-block-n", type=int, default=0)
    ap.add_argument("--score-mode", type=int, default=0, choices=[0, 1],
                    help="0: the reference's score arithmetic (default); 1: the opt-in tensor-core scores")
    ap.add_argument("--warmup-runs", type=int, default=1)
    ap.add_argument("--timed-runs", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--synthetic-cache", action="store_true",
                    help="fill the caches with seeded random values instead of running the prefill")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--intermediate", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=128256)
    return ap.parse_args(argv)


def run_batch(rt: DecodeRuntime, args, batch_id: int, prompt_ids: torch.Tensor):
    dev = rt.dev
    torch.cuda.synchronize(dev)
    w0 = time.perf_counter()
    if args.synthetic_cache:
        rt.fill_cache_synthetic(args.prompt_len, seed=args.seed + batch_id)
        last = torch.zeros(rt.B, rt.shape.vocab, device=dev)
        last[:, 1] = 1.0
    else:
        last = rt.prefill(prompt_ids, chunk=args.prefill_chunk_size)
    torch.cuda.synchronize(dev)
    prefill_s = time.perf_counter() - w0
    res = rt.generate(last, args.prompt_len, args.max_new_tokens, use_graph=(rt.attention != "sdpa"))
    torch.cuda.synchronize(dev)
    wall_s = time.perf_counter() - w0
    toks = res["generated_token_ids_all"].tolist()
    row = report.batch_metric(batch_id=batch_id, batch_size=rt.B, prompt_len=args.prompt_len,
                              prefill_time_s=prefill_s, cache_setup_time_s=0.0,  # K/V land in the cache directly
                              decode_time_s=res["decode_time_s"], wall_time_s=wall_s,
                              timed_generated_tokens=res["timed_generated_tokens"],
                              visible_generated_tokens=res["timed_generated_tokens"],
                              example_indices=range(batch_id * rt.B, (batch_id + 1) * rt.B))
    return row, toks


def main(argv=None) -> None:
    args = parse_args(argv)
    os.makedirs(args.out_dir, exist_ok=True)
    dev = torch.device(args.device)
    shape = LlamaShape(hidden=args.hidden, layers=args.layers, heads=args.heads, kv_heads=args.kv_heads,
                       intermediate=args.intermediate, vocab=args.vocab)
    g = torch.Generator().manual_seed(args.seed)
    prompts = [torch.randint(0, args.vocab, (args.batch_size, args.prompt_len), generator=g)
               for _ in range(args.num_batches)]
    batch_rows, run_rows, gen_rows = [], [], []
    for backend in args.backends:
        rt = DecodeRuntime(shape, args.batch_size, args.prompt_len + args.max_new_tokens, dev, attention=backend,
                           S=args.santa_s, attn_seed=args.santa_seed, block_n=args.santa_block_n,
                           weight_seed=args.seed, score_mode=args.score_mode)
        for phase, runs in (("warmup", args.warmup_runs), ("timed", args.timed_runs)):
            for run_idx in range(runs):
                rows = []
                for batch_id, ids in enumerate(prompts):
                    row, toks = run_batch(rt, args, batch_id, ids)
                    row.update({"phase": phase, "run_idx": run_idx, "backend": backend})
                    rows.append(row)
                    for slot, t in enumerate(toks):
                        gen_rows.append({"phase": phase, "run_idx": run_idx, "backend": backend, "batch_id": batch_id,
                                         "batch_slot": slot, "example_index": batch_id * args.batch_size + slot,
                                         "generated_token_ids_all": t, "generated_token_ids_visible": t,
                                         "generated_text": None, "generated_text_normalized": None,
                                         "stop_step": None, "exact_match": None})
                batch_rows.extend(rows)
                summary = report.run_metric(rows)
                summary.update({"phase": phase, "run_idx": run_idx, "backend": backend,
                                "backend_actual_mode": "dense" if backend == "sdpa" else "ragged-device-lengths"})
                run_rows.append(summary)
                print(f"[{phase} run {run_idx}] backend={backend:<12} decode={summary['decode_time_s']:.3f}s "
                      f"output_tok/s={summary['output_tokens_per_s']:.2f} tpot_ms={summary['tpot_ms']:.3f}")
        del rt
        torch.cuda.empty_cache()
    report.write_jsonl(os.path.join(args.out_dir, "batch_metrics.jsonl"), batch_rows)
    report.write_jsonl(os.path.join(args.out_dir, "run_metrics.jsonl"), run_rows)
    report.write_jsonl(os.path.join(args.out_dir, "generations.jsonl"), gen_rows)
    agg = report.aggregates(run_rows)
    report.write_json(os.path.join(args.out_dir, "aggregates.json"), agg)
    report.write_aggregate_csv(os.path.join(args.out_dir, "aggregates.csv"), agg)
    report.write_json(os.path.join(args.out_dir, "backend_agreement.json"),
                      report.token_agreement([r for r in gen_rows if r["phase"] == "timed"]))
    report.write_json(os.path.join(args.out_dir, "invocation.json"),
                      {"argv": list(sys.argv if argv is None else argv), "args": vars(args)})
    report.write_json(os.path.join(args.out_dir, "config.json"), {
        "model_name": f"random-init Llama shape {vars(shape)}", "dataset": "uniform random token ids",
        "batch_size": args.batch_size, "warmup_runs": args.warmup_runs, "timed_runs": args.timed_runs,
        "max_new_tokens": args.max_new_tokens, "target_prompt_token_length": args.prompt_len,
        "dtype": "bf16", "device": str(dev), "prefill_chunk_size": args.prefill_chunk_size,
        "backends": list(args.backends), "santa_s": args.santa_s, "santa_seed": args.santa_seed,
        "santa_block_n": args.santa_block_n, "lockstep_stop_mode": "max_tokens",
        "generation_surface": "manual", "stop_token_ids": [],
        "attention_dims": {"num_attention_heads": args.heads, "num_key_value_heads": args.kv_heads, "head_dim": 128}})


if __name__ == "__main__":
    main()
