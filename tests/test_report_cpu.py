"""Benchmark records: field names and formulas of the reference harness
(tutorial_code/benchmark_longctx.py:350-369, :396-425, :486-530; runtime_common.py:449-495)."""
import csv
import json
import math

from santa_b200 import report


def test_batch_and_run_records():
    r = report.batch_metric(batch_id=2, batch_size=4, prompt_len=1000, prefill_time_s=2.0, cache_setup_time_s=0.5,
                            decode_time_s=4.0, wall_time_s=7.0, timed_generated_tokens=128,
                            visible_generated_tokens=100, example_indices=[8, 9, 10, 11])
    assert list(r) == ["batch_id", "batch_size", "example_indices", "prompt_len", "prefill_time_s",
                       "cache_setup_time_s", "decode_time_s", "generate_api_wall_time_s",
                       "hf_generate_wrapper_overhead_s", "end_to_end_wall_time_s", "timed_generated_tokens",
                       "visible_generated_tokens", "steps_sampled", "tpot_ms", "output_tokens_per_s",
                       "visible_output_tokens_per_s", "requests_per_s", "prefill_tokens_per_s"]
    assert r["steps_sampled"] == 32 and r["tpot_ms"] == 1000.0 * 4.0 / 128 and r["output_tokens_per_s"] == 32.0
    assert r["visible_output_tokens_per_s"] == 25.0 and r["requests_per_s"] == 4 / 7.0
    assert r["prefill_tokens_per_s"] == 2000.0 and r["hf_generate_wrapper_overhead_s"] == 0.5
    z = report.batch_metric(batch_id=0, batch_size=0, prompt_len=0, prefill_time_s=0, cache_setup_time_s=0,
                            decode_time_s=0, wall_time_s=0, timed_generated_tokens=0, visible_generated_tokens=0)
    assert math.isnan(z["tpot_ms"]) and math.isnan(z["output_tokens_per_s"]) and z["steps_sampled"] == 0
    run = report.run_metric([r, r], exact_matches=[True, False, True, True])
    assert run["num_requests"] == 8 and run["decode_time_s"] == 8.0 and run["timed_generated_tokens"] == 256
    assert run["output_tokens_per_s"] == 32.0 and run["prompt_tokens_total"] == 8000
    assert run["exact_match_rate"] == 0.75 and math.isnan(report.run_metric([r])["exact_match_rate"])


def test_statistics():
    s = report.summarize([1.0, 2.0, 4.0, 9.0])
    assert s["count"] == 4 and s["mean"] == 4.0 and s["min"] == 1.0 and s["max"] == 9.0
    assert s["median"] == 3.0 and abs(s["p90"] - (4.0 + 0.7 * 5.0)) < 1e-12
    sd = math.sqrt(((3 ** 2) + (2 ** 2) + 0 + (5 ** 2)) / 3)
    assert abs(s["std"] - sd) < 1e-12 and abs(s["ci95_hi"] - (4.0 + 1.96 * sd / 2)) < 1e-12
    one = report.summarize([5.0])
    assert one["std"] == 0.0 and one["ci95_lo"] == 5.0 and one["median"] == 5.0
    assert report.summarize([])["count"] == 0 and math.isnan(report.summarize([])["mean"])


def test_files(tmp_path):
    rows = []
    for backend, tps in (("santa_flash", 100.0), ("sdpa", 50.0)):
        for run_idx in range(3):
            b = report.batch_metric(batch_id=0, batch_size=2, prompt_len=10, prefill_time_s=1.0,
                                    cache_setup_time_s=0.0, decode_time_s=20.0 / tps * (1 + 0.1 * run_idx),
                                    wall_time_s=3.0, timed_generated_tokens=20, visible_generated_tokens=20)
            r = report.run_metric([b])
            r.update({"phase": "timed", "run_idx": run_idx, "backend": backend, "backend_actual_mode": "x"})
            rows.append(r)
    rows.append(dict(rows[0], phase="warmup", decode_time_s=1e9))
    agg = report.aggregates(rows)
    assert set(agg) == {"santa_flash", "sdpa"} and agg["sdpa"]["num_runs"] == 3
    assert agg["santa_flash"]["last_backend_info"] == {"backend_actual_mode": "x"}
    assert abs(agg["santa_flash"]["metrics"]["output_tokens_per_s"]["max"] - 100.0) < 1e-9
    report.write_aggregate_csv(str(tmp_path / "aggregates.csv"), agg)
    report.write_json(str(tmp_path / "aggregates.json"), agg)
    report.write_jsonl(str(tmp_path / "run_metrics.jsonl"), rows)
    with open(tmp_path / "aggregates.csv") as f:
        got = list(csv.DictReader(f))
    assert got[0]["backend"] == "santa_flash" and got[0]["runs"] == "3"
    assert list(got[0])[:4] == ["backend", "runs", "prefill_time_s_mean", "decode_time_s_mean"]
    assert "exact_match_rate_median" in got[0]
    assert len(open(tmp_path / "run_metrics.jsonl").read().splitlines()) == 7
    assert json.load(open(tmp_path / "aggregates.json"))["sdpa"]["num_runs"] == 3
    gen = [{"run_idx": 0, "example_index": i, "backend": b, "generated_token_ids_visible": t}
           for b, toks in (("a", [[1, 2], [3, 4]]), ("b", [[1, 2], [3, 5]])) for i, t in enumerate(toks)]
    pair = report.token_agreement(gen)
    assert pair[0]["comparable_examples"] == 2 and pair[0]["visible_token_id_match_rate"] == 0.5
