"""bench.py's host side: the arithmetic of its record and the parts of its contract that need no GPU."""

import importlib.util
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_shape_and_flops_of_the_default_run():
    b = load_bench()
    cfg = b.LLAMA_3_2_1B
    assert (cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
            cfg["intermediate_size"], cfg["vocab_size"]) == (16, 2048, 32, 8, 64, 8192, 128256)
    assert cfg["rope_scaling"]["rope_type"] == "llama3" and cfg["rope_scaling"]["factor"] == 32.0 and cfg["tie_word_embeddings"]
    # per token: q|k|v, o, gate, up, down products; attention over the causal half; the head once
    H, I, d, nh, nkv, V, T, L = 2048, 8192, 64, 32, 8, 128256, 2048, 16
    by_hand = L * (T * 2 * (H * (nh + 2 * nkv) * d + nh * d * H + 3 * H * I) + 2 * T * T * d * nh) + 2 * H * V
    assert b.prefill_flops(cfg, 16, 2048) == by_hand == 4261132894208
    assert b.PROMPT_LEN == 2048 and b.CONTEXT == 4096 and b.PAGE == 16


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    b = load_bench()
    monkeypatch.setattr(b, "ROOT", tmp_path)
    assert b.peaks() == {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 7000, "bf16_tflops": 1500.5, "bf16_tflops_sustained": 1400}))
    assert b.peaks() == {"hbm_gbs": 7000.0, "bf16_tflops": 1500.5, "source": "measured"}
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert b.peaks()["source"] == "fallback"


def test_clock_samples_are_summarised():
    b = load_bench()
    s = b.ClockSampler()
    s.lines = ["1965, 1965, Not Active, Not Active, Not Active, Not Active", "1800, 1965, Not Active, Not Active, Not Active, Active",
               "1700, 1965, Not Active, Not Active, Not Active, Active", "garbage"]
    assert s.summary() == {"sm_mhz": 1800.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    assert b.ClockSampler().summary()["samples"] == 0


def test_more_than_one_gpu_is_refused_with_code_2_and_the_reference_arm_says_why_it_is_absent():
    two = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "2"], capture_output=True, text=True, timeout=120)
    assert two.returncode == 2 and len(two.stdout.strip().splitlines()) == 1 and "one GPU" in two.stdout
    ref = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference"], capture_output=True, text=True, timeout=120)
    rec = json.loads(ref.stdout.strip())
    assert ref.returncode == 0 and rec["impl"] == "reference" and rec["unavailable"]
