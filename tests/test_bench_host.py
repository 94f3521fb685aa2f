"""Host-side pieces of bench.py that need no GPU: the deadline around the collective sections of a multi-rank run (a rank that
fails inside a collective step must not keep rank 0 from printing its line) and the summary of a result line."""
import importlib.util
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_under_test"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_deadline_returns_results_errors_and_marks_what_is_stuck():
    bench = load_bench()
    stuck = []
    assert bench.run_with_deadline("fine", lambda: {"us": 1.0}, 5, stuck) == {"us": 1.0}

    def raises():
        raise RuntimeError("a peer did not arrive")

    out = bench.run_with_deadline("raises", raises, 5, stuck)
    assert out == {"error": "a peer did not arrive"} and stuck == []
    t0 = time.perf_counter()
    out = bench.run_with_deadline("hangs", lambda: time.sleep(30), 0.2, stuck)
    assert time.perf_counter() - t0 < 5 and "did not finish" in out["error"] and stuck == ["hangs"]


def test_summary_takes_the_headline_numbers():
    bench = load_bench()
    line = {"value": 1000.0, "roofline": {"frac": 0.65}, "e2e": {"value": 75.0},
            "extra": {"decode": {"tok_s": 460.0, "frac_of_hbm_peak": 0.35, "multi_token_steps": {"t4": {"ms_per_step": 5.4}}},
                      "prefill_plan": {"t2048": {"tok_s": 55000.0, "e2e_tok_s": 50000.0, "e2e_tflops": 730.0}}}}
    s = bench.summarize(line)
    assert s["gemm_tflops"] == 1000.0 and s["decode_tok_s"] == 460.0 and s["prefill_2048_tok_s"] == 55000.0
    assert s["verify_4_tokens_ms"] == 5.4 and s["prefill_2048_e2e_tflops"] == 730.0
