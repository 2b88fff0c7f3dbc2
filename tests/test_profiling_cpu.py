"""Profiling switches: CLI flag, window bookkeeping, roofline arithmetic, and the metrics row of a CPU train step."""
import torch

from unirl_b200.config.loader import parse_cli
from unirl_b200.utils.profiling import ProfileWindow, measured_peaks, roofline_metrics


def test_profile_flag_becomes_config_overrides():
    _, _, ov, _ = parse_cli(["--config-name=ar/x", "--profile=5:2", "a=1"])
    assert "+profile.enabled=true" in ov and "+profile.start_step=5" in ov and "+profile.num_steps=2" in ov and "a=1" in ov
    _, _, ov, _ = parse_cli(["--profile"])
    assert ov == ["+profile.enabled=true"]


def test_profile_window_brackets_the_requested_steps(tmp_path):
    w = ProfileWindow(enabled=True, start_step=1, num_steps=2, trace_dir=str(tmp_path), nvtx=False)
    seen = []
    for step in range(4):
        w.step_begin(step)
        seen.append(w._active)
        torch.ones(4).sum()
        w.step_end(step)
    assert seen == [False, True, True, False]
    assert (tmp_path / "trace_steps_1_2.json").exists()


def test_roofline_arithmetic():
    pk = measured_peaks()
    m = roofline_metrics(n_params=4_000_000_000, train_tokens=500_000, train_ms=10_000.0, decode_tokens=0, decode_steps=4096, rollout_ms=40_000.0,
                         kv_bytes_per_token=147456, mean_context=2700, batch=128)
    assert abs(m["kernel/train_tflops"] - 6 * 4e9 * 5e5 / 10 / 1e12) < 1e-6
    assert abs(m["kernel/train_roofline_frac"] - m["kernel/train_tflops"] / pk["tflops_sustained"]) < 1e-9
    want_gbs = 4096 * (8e9 + 147456 * 2700 * 128) / 40 / 1e9
    assert abs(m["kernel/decode_gbs"] - want_gbs) / want_gbs < 1e-6
