"""The profile's arithmetic, without a GPU: the cost table, the limits it is read against, and the
report's sums (the reference tests the same layers: rocml/src/profile/cost.rs:117-216,
profile/report.rs:236-334)."""
import json

import pytest
import torch

from rocml_b200.profile import Peaks, cost, load_peaks
from rocml_b200.profile.profiler import OpRecord, Profiler, StepRecord
from rocml_b200.profile.report import build_report, to_human


def model_of(name, dtype=torch.bfloat16):
    from rocml_b200.config import CATALOG, config_from_dict
    from rocml_b200.engine.model import Model
    from rocml_b200.parts import BuildEnv
    cfg = config_from_dict(CATALOG[name].config)
    return Model(cfg.to_model_spec(), BuildEnv(torch.device("cpu"), dtype)), cfg


def test_cost_of_a_step_at_qwen3_8b_sizes():
    """15.14 GB of weights a decode step reads, 147,456 bytes of keys and values a token, and 29.69
    TFLOP for a prompt of 2,048 tokens (28.45 in the products, 1.24 in the attention)."""
    m, cfg = model_of("qwen3-8b")
    assert abs(m.weight_bytes_per_step() / 1e9 - 15.137) < 0.001
    nbytes, flops = m.step_cost([2048], [2048], 1)
    assert abs(flops / 1e12 - 29.69) < 0.01
    _, attn = cost.attention([2048], [2048], 32, 8, 128, 2)
    assert abs(36 * attn / 1e12 - 1.24) < 0.01
    b8, _ = m.step_cost([1] * 8, [1152] * 8, 8)
    kv = 8 * 1152 * 147456
    assert abs(b8 - (m.weight_bytes_per_step() + kv)) < 8 * 36 * 32 * 128 * 2 * 2 + 1     # + queries in, outputs out
    assert abs(b8 / 1e9 - 16.50) < 0.01
    # the 32-bit path reads twice the bytes
    m32, _ = model_of("qwen3-8b", torch.float32)
    assert m32.weight_bytes_per_step() == 2 * m.weight_bytes_per_step()
    # the same count from the flat formula
    assert cost.decoder_flops(2048, 4096, 4096, 1024, 12288, 36, 151936, 1, 36 * attn) == flops


def test_cost_of_the_other_sizes():
    m4, _ = model_of("qwen3-4b")           # tied: the head reads the embedding table
    assert abs(m4.weight_bytes_per_step() / 1e9 - (8.05 - 0.0)) < 0.75
    m32, _ = model_of("qwen3-32b")
    assert abs(m32.weight_bytes_per_step() / 1e9 - 63.97) < 0.05


def test_attention_cost_counts_what_a_query_can_see():
    # one token over 1,152 keys: keys and values of 8 heads once, 4 operations per (head, key, dimension)
    b, f = cost.attention([1], [1152], 32, 8, 128, 2)
    assert b == 2 * 8 * 1152 * 128 * 2 + 2 * 32 * 128 * 2 and f == 4 * 32 * 128 * 1152
    # a whole prompt: the causal triangle
    _, f = cost.attention([100], [100], 4, 2, 16, 4)
    assert f == 4 * 4 * 16 * (100 * 101 // 2)
    # a continuation sees the earlier keys too
    _, f = cost.attention([10], [50], 4, 2, 16, 4)
    assert f == 4 * 4 * 16 * sum(range(41, 51))
    # a window bounds both the keys read and the pairs
    b, f = cost.attention([10], [50], 4, 2, 16, 4, window=8)
    assert f == 4 * 4 * 16 * 10 * 8 and b == 2 * 2 * (50 - 33) * 16 * 4 + 2 * 10 * 4 * 16 * 4
    _, f = cost.attention([20], [20], 1, 1, 16, 4, window=8)
    assert f == 4 * 16 * (sum(range(1, 8)) + 13 * 8)
    assert cost.attention([0], [7], 4, 2, 16, 4) == (0, 0)


def test_linear_and_small_kernels():
    assert cost.linear(8, 4096, 4096, 2, 2, 4, splits=4) == (4096 * 4096 * 2 + 8 * 4096 * 2 + 4 * 8 * 4096 * 4, 2 * 8 * 4096 * 4096)
    assert cost.linear(8, 64, 32, 2, 2, 4, 1, True)[0] == 64 * 32 * 2 + 8 * 32 * 2 + 2 * 8 * 64 * 4
    assert cost.embedding(8, 4096, 2) == (8 * 4096 * 6, 0)
    assert cost.add_norm(8, 4096, 2, 2, True)[0] == 8 * 4096 * (4 + 4 + 8 + 2) + 4096 * 4
    assert cost.sample(3, 1000)[0] == 12000


def test_peaks_from_a_file_or_the_fallback(tmp_path, monkeypatch):
    path = tmp_path / "peaks.json"
    path.write_text(json.dumps({"hbm_gbs": 6000.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1300.0}))
    p = load_peaks(str(path))
    assert (p.hbm_gbs, p.bf16_tflops, p.bf16_tflops_sustained, p.source) == (6000.0, 1500.0, 1300.0, "measured")
    assert p.flops_per_sec("bfloat16") == 1.5e15 and p.flops_per_sec("bfloat16", sustained=True) == 1.3e15
    assert p.flops_per_sec("float32") < 1e14
    monkeypatch.setenv("ROCML_B200_PEAKS", str(path))
    assert load_peaks().hbm_gbs == 6000.0
    bad = tmp_path / "bad.json"
    bad.write_text("{")
    monkeypatch.setenv("ROCML_B200_PEAKS", str(bad))
    assert load_peaks(str(bad)).source in ("measured", "fallback")     # the checkout's own file, or the fallback


def test_report_sums_and_ranks():
    peaks = Peaks(1000.0, 100.0, 100.0, 10.0, "measured")            # 1 TB/s, 100 TFLOP/s
    prof = Profiler("cpu", peaks, "bfloat16", gate_ms=0)
    gb = 10 ** 9
    prof.ops = [
        OpRecord("gemm", "down_proj", 0, "decode", 2 * gb, 10 ** 9, ms=4.0),     # bound: 2 ms of bandwidth
        OpRecord("gemm", "down_proj", 1, "decode", 2 * gb, 10 ** 9, ms=4.0),
        OpRecord("attention_decode", "attention_decode", 0, "decode", gb, 0, ms=1.5),
        OpRecord("argmax", "sampling", None, "decode", 0, 0, ms=0.5),
        OpRecord("gemm", "down_proj", 0, "prefill", gb, 4 * 10 ** 11, ms=5.0),   # bound: 4 ms of arithmetic
    ]
    prof.steps = [StepRecord("prefill", 100, 1, ms=5.5), StepRecord("decode", 2, 2, ms=6.0), StepRecord("decode", 2, 2, ms=5.0)]
    rep = build_report(prof)
    assert [p["phase"] for p in rep["phases"]] == ["decode", "prefill"]
    dec = rep["phases"][0]
    assert dec["steps"] == 2 and dec["tokens"] == 4 and dec["ops_ms"] == 10.0 and dec["between_kernels_ms"] == 1.0
    down = dec["by_op"][0]
    assert down["label"] == "down_proj" and down["count"] == 2 and down["elapsed_ms"] == 8.0
    assert down["t_min_ms"] == pytest.approx(4.0) and down["efficiency"] == pytest.approx(0.5)
    assert down["wasted_ms"] == pytest.approx(4.0) and down["bound"] == "hbm"
    assert down["gb_per_sec"] == pytest.approx(500.0) and down["frac_of_bandwidth"] == pytest.approx(0.5)
    assert down["pct_of_phase_time"] == pytest.approx(80.0)
    assert [r["label"] for r in dec["by_layer"]] == ["layer 0", "layer 1", "(outside the layers)"]
    pre = rep["phases"][1]["by_op"][0]
    assert pre["bound"] == "flops" and pre["t_min_ms"] == pytest.approx(4.0) and pre["frac_of_flops"] == pytest.approx(0.8)
    assert rep["worklist"][0].startswith("decode down_proj: 4.000 ms above its bound")
    text = to_human(rep, layers=True)
    assert "== decode: 2 steps, 4 tokens" in text and "-- by layer --" in text and "down_proj" in text
    json.dumps(rep)


def test_scopes_cost_nothing_when_no_profiler_is_active():
    from rocml_b200.profile import active, scope
    assert active() is None
    with scope(layer=3):
        pass
    prof = Profiler("cpu", Peaks(1.0, 1.0, 1.0, 1.0, "measured"), gate_ms=0)
    with prof:
        assert active() is prof
        with scope(layer=3), scope(op="x"):
            assert prof._stack == [{"layer": 3}, {"op": "x"}]
        assert prof._stack == []
        with pytest.raises(RuntimeError):
            Profiler("cpu", prof.peaks).__enter__()
    assert active() is None
