"""The plain implementation checked against itself and against hand-made cases (no GPU)."""
import math

import numpy as np
import torch

import plain_qwen3 as P
from plain_sampler import XorShift64Star, sample
from tiny_models import TINY_A, TINY_C, prompt, write_model


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    out = P.rmsnorm(x, w, 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]]))


def test_rope_position_zero_is_identity_and_pairs_are_halves():
    x = torch.randn(3, 2, 8)
    assert torch.allclose(P.rope_neox(x, [0, 0, 0], 1e4), x)
    y = P.rope_neox(x, [0, 1, 2], 1e4)
    # pair (i, i + 4) rotates by pos * theta^(-2i/8): norms of pairs are kept
    assert torch.allclose(x[..., 0] ** 2 + x[..., 4] ** 2, y[..., 0] ** 2 + y[..., 4] ** 2, atol=1e-5)
    a = 2 * 1e4 ** (-2 * 1 / 8)
    assert torch.allclose(y[2, 0, 1], x[2, 0, 1] * math.cos(a) - x[2, 0, 5] * math.sin(a), atol=1e-6)


def test_attention_is_causal_grouped_and_windowed():
    T, nq, nkv, hd = 6, 4, 2, 8
    q, k, v = torch.randn(T, nq, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    out = P.attention(q, k, v)
    assert torch.allclose(out[0, 3], v[0, 1])            # the first token sees itself only; head 3 -> kv head 1
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, 9.0
    assert torch.allclose(P.attention(q, k2, v2)[:4], out[:4])   # later keys do not reach earlier queries
    w = P.attention(q, k, v, window=2)
    s = (q[5, 0] @ k[4:6, 0].t()) / math.sqrt(hd)
    assert torch.allclose(w[5, 0], torch.softmax(s, 0) @ v[4:6, 0], atol=1e-6)


def test_logits_of_a_prefix_do_not_depend_on_what_follows(tmp_path):
    for name, cfg in (("a", TINY_A), ("c", TINY_C)):
        m = P.PlainQwen3(write_model(str(tmp_path / name), cfg, 1, std=0.05))
        ids = prompt(2, 40, cfg["vocab_size"])
        full = m.logits(ids)
        assert torch.allclose(m.logits(ids[:17]), full[:17], atol=1e-5)
        assert full.shape == (40, cfg["vocab_size"]) and torch.isfinite(full).all()


def test_float32_and_float64_agree(tmp_path):
    folder = write_model(str(tmp_path / "m"), TINY_A, 1, std=0.05)
    ids = prompt(3, 30, 256)
    a = P.PlainQwen3(folder, torch.float32).logits(ids)
    b = P.PlainQwen3(folder, torch.float64).logits(ids)
    assert (a.double() - b).abs().max() / b.abs().max() < 1e-5


def test_sampler_basics():
    logits = np.array([0.1, 2.0, -1.0, 2.0, 0.5], dtype=np.float32)
    assert sample(logits, [], 0.0) == 1                                        # first maximum
    assert sample(logits, [], 1.0, top_k=1, rng=XorShift64Star(1)) in (1, 3)
    for seed in range(20):
        assert sample(logits, [], 1.0, top_k=2, rng=XorShift64Star(seed)) in (1, 3)
    peaked = np.array([10.0, 0.0, 0.0], dtype=np.float32)
    assert all(sample(peaked, [], 1.0, top_p=0.5, rng=XorShift64Star(s)) == 0 for s in range(20))
    a = [sample(logits, [], 0.9, top_k=4, top_p=0.9, rng=XorShift64Star(7)) for _ in range(3)]
    b = [sample(logits, [], 0.9, top_k=4, top_p=0.9, rng=XorShift64Star(7)) for _ in range(3)]
    assert a == b
    assert sample(logits, [1, 3], 0.0, repeat_penalty=10.0) == 4               # both 2.0s pushed to 0.2
    r = XorShift64Star(0)
    assert r.s == 0x9E3779B97F4A7C15 and 0.0 <= float(r.next_f32()) < 1.0


def test_library_rng_matches_the_plain_one():
    from rocml_b200.sampling import XorShift64Star as Lib
    for seed in (0, 1, 12345, 2 ** 63 + 5):
        a, b = Lib(seed), XorShift64Star(seed)
        assert [a.next_f32() for _ in range(50)] == [float(b.next_f32()) for _ in range(50)]
