"""Benchmark records in the reference harness's formats, so that numbers from this package's own
harness line up column by column with a run of the reference elsewhere.

Field names and formulas follow tutorial_code/benchmark_longctx.py of the reference:
  per-batch record   ``batch_metrics.jsonl``   (:350-369)
  per-run record     ``run_metrics.jsonl``     (:396-425, sums over the run's batches)
  ``aggregates.json`` / ``aggregates.csv``     (:486-530, :664-690) with the statistics of
  tutorial_code/runtime_common.py:449-495 (mean, sample std, interpolated median / p90, 95 % interval)
  ``backend_agreement.json``                   (:429-484; token-id agreement -- text fields need the
  reference's tokenizer and answer files, which synthetic runs do not have, so text / exact-match
  entries are NaN here)
"""
from __future__ import annotations

import csv
import json
import math
from typing import Any, Dict, Iterable, List, Sequence

NAN = float("nan")


def _ratio(num: float, den: float) -> float:
    return (num / den) if den > 0 else NAN


def batch_metric(*, batch_id: int, batch_size: int, prompt_len: int, prefill_time_s: float,
                 cache_setup_time_s: float, decode_time_s: float, wall_time_s: float,
                 timed_generated_tokens: int, visible_generated_tokens: int,
                 example_indices: Sequence[int] = ()) -> Dict[str, Any]:
    """One ``batch_metrics.jsonl`` record."""
    return {
        "batch_id": int(batch_id),
        "batch_size": int(batch_size),
        "example_indices": [int(i) for i in example_indices],
        "prompt_len": int(prompt_len),
        "prefill_time_s": float(prefill_time_s),
        "cache_setup_time_s": float(cache_setup_time_s),
        "decode_time_s": float(decode_time_s),
        "generate_api_wall_time_s": 0.0,
        "hf_generate_wrapper_overhead_s": float(wall_time_s - (prefill_time_s + cache_setup_time_s + decode_time_s)),
        "end_to_end_wall_time_s": float(wall_time_s),
        "timed_generated_tokens": int(timed_generated_tokens),
        "visible_generated_tokens": int(visible_generated_tokens),
        "steps_sampled": int(timed_generated_tokens // batch_size) if batch_size > 0 else 0,
        "tpot_ms": 1000.0 * _ratio(decode_time_s, timed_generated_tokens),
        "output_tokens_per_s": _ratio(timed_generated_tokens, decode_time_s),
        "visible_output_tokens_per_s": _ratio(visible_generated_tokens, decode_time_s),
        "requests_per_s": _ratio(batch_size, wall_time_s),
        "prefill_tokens_per_s": _ratio(batch_size * prompt_len, prefill_time_s),
    }


def run_metric(batch_rows: Sequence[Dict[str, Any]], exact_matches: Sequence[bool] = ()) -> Dict[str, Any]:
    """One run's totals over its batches (a ``run_metrics.jsonl`` record without the labels)."""
    tot = lambda key: sum(float(r[key]) for r in batch_rows)  # noqa: E731
    out: Dict[str, Any] = {
        "num_batches": len(batch_rows),
        "num_requests": int(sum(int(r["batch_size"]) for r in batch_rows)),
        "prefill_time_s": tot("prefill_time_s"),
        "cache_setup_time_s": tot("cache_setup_time_s"),
        "decode_time_s": tot("decode_time_s"),
        "end_to_end_wall_time_s": tot("end_to_end_wall_time_s"),
        "timed_generated_tokens": int(tot("timed_generated_tokens")),
        "visible_generated_tokens": int(tot("visible_generated_tokens")),
        "prompt_tokens_total": int(sum(int(r["batch_size"]) * int(r["prompt_len"]) for r in batch_rows)),
    }
    out["tpot_ms"] = 1000.0 * _ratio(out["decode_time_s"], out["timed_generated_tokens"])
    out["output_tokens_per_s"] = _ratio(out["timed_generated_tokens"], out["decode_time_s"])
    out["visible_output_tokens_per_s"] = _ratio(out["visible_generated_tokens"], out["decode_time_s"])
    out["requests_per_s"] = _ratio(out["num_requests"], out["end_to_end_wall_time_s"])
    out["prefill_tokens_per_s"] = _ratio(out["prompt_tokens_total"], out["prefill_time_s"])
    out["exact_match_rate"] = (sum(1 for m in exact_matches if m) / len(exact_matches)) if exact_matches else NAN
    return out


def quantile(values: Sequence[float], q: float) -> float:
    """Linear interpolation between order statistics at position (n-1)*q."""
    if not values:
        return NAN
    v = sorted(float(x) for x in values)
    pos = (len(v) - 1) * q
    lo, hi = math.floor(pos), math.ceil(pos)
    return v[lo] if lo == hi else v[lo] + (v[hi] - v[lo]) * (pos - lo)


def summarize(values: Iterable[float]) -> Dict[str, float]:
    v = [float(x) for x in values]
    if not v:
        return {k: (0 if k == "count" else NAN) for k in
                ("count", "mean", "std", "median", "p90", "min", "max", "ci95_lo", "ci95_hi")}
    mean = math.fsum(v) / len(v)
    # sample standard deviation, written out so that NaN entries give NaN instead of an exception
    std = math.sqrt(math.fsum((x - mean) ** 2 for x in v) / (len(v) - 1)) if len(v) > 1 else 0.0
    half = 1.96 * std / math.sqrt(len(v)) if len(v) > 1 else 0.0
    return {"count": len(v), "mean": mean, "std": std, "median": quantile(v, 0.5), "p90": quantile(v, 0.9),
            "min": min(v), "max": max(v), "ci95_lo": mean - half, "ci95_hi": mean + half}


SUMMARISED = ("prefill_time_s", "cache_setup_time_s", "decode_time_s", "end_to_end_wall_time_s", "tpot_ms",
              "output_tokens_per_s", "visible_output_tokens_per_s", "requests_per_s", "prefill_tokens_per_s",
              "exact_match_rate")
CSV_METRICS = ("prefill_time_s", "decode_time_s", "end_to_end_wall_time_s", "tpot_ms", "output_tokens_per_s",
               "requests_per_s", "exact_match_rate")


def aggregates(run_rows: Sequence[Dict[str, Any]]) -> Dict[str, Any]:
    """``aggregates.json``: per backend, the statistics of every summarised metric over the timed runs."""
    by_backend: Dict[str, List[Dict[str, Any]]] = {}
    for r in run_rows:
        if r.get("phase", "timed") == "timed":
            by_backend.setdefault(str(r["backend"]), []).append(r)
    return {b: {"num_runs": len(rows),
                "metrics": {m: summarize(float(r[m]) for r in rows) for m in SUMMARISED},
                "last_backend_info": {k: v for k, v in rows[-1].items() if k.startswith("backend_")}}
            for b, rows in by_backend.items()}


def token_agreement(generation_rows: Sequence[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """``backend_agreement.json`` rows: for every pair of backends, on how many (run, example) pairs the
    visible generated token ids are identical."""
    backends = sorted({str(r["backend"]) for r in generation_rows})
    index = {(int(r["run_idx"]), int(r["example_index"]), str(r["backend"])): r for r in generation_rows}
    keys = sorted({(k[0], k[1]) for k in index})
    out = []
    for i, a in enumerate(backends):
        for b in backends[i + 1:]:
            both = [(index[(ri, ei, a)], index[(ri, ei, b)]) for ri, ei in keys
                    if (ri, ei, a) in index and (ri, ei, b) in index]
            if not both:
                continue
            same = sum(1 for ra, rb in both if ra["generated_token_ids_visible"] == rb["generated_token_ids_visible"])
            out.append({"backend_a": a, "backend_b": b, "comparable_examples": len(both),
                        "normalized_text_match_rate": NAN, "visible_token_id_match_rate": same / len(both),
                        "both_exact_match_rate": NAN, "a_only_exact_match_rate": NAN,
                        "b_only_exact_match_rate": NAN})
    return out


def write_jsonl(path: str, rows: Iterable[Dict[str, Any]]) -> None:
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")


def write_json(path: str, payload: Any) -> None:
    with open(path, "w", encoding="utf-8") as f:
        json.dump(payload, f, indent=2)


def write_aggregate_csv(path: str, payload: Dict[str, Any]) -> None:
    """``aggregates.csv``: backend, runs, then <metric>_mean for each CSV metric, then <metric>_median."""
    cols = ["backend", "runs"] + [f"{m}_mean" for m in CSV_METRICS] + [f"{m}_median" for m in CSV_METRICS]
    with open(path, "w", encoding="utf-8", newline="") as f:
        w = csv.DictWriter(f, fieldnames=cols)
        w.writeheader()
        for backend, p in payload.items():
            row = {"backend": backend, "runs": p["num_runs"]}
            for m in CSV_METRICS:
                row[f"{m}_mean"] = p["metrics"][m]["mean"]
                row[f"{m}_median"] = p["metrics"][m]["median"]
            w.writerow(row)
