"""Configurations drawn at random, each differing from the others in every size and option: head sizes in
steps of 16 up to 256, any number of heads and groups, widths and vocabularies that are no power of two,
biases, tying, windows on some layers, eps and theta.  For each, in 32-bit and in bfloat16, the engine
against the plain implementation: a batch of unequal prompts cut into pieces of a random size, every
place wanted; then tokens one by one, the shortest sequence ending first.  Whatever kernel the sizes
select (tensor-core or plain), the result must be right."""
import random

import pytest
import torch

from tiny_models import prompt, write_model

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


def draw(seed):
    rng = random.Random(1000 + seed)
    hd = 16 * rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 12, 14, 16]) if seed else 256
    nkv = rng.choice([1, 2, 3, 4])
    group = rng.choice([1, 2, 3, 5, 8, 17]) if hd <= 128 else rng.choice([1, 2, 3])
    layers = rng.choice([1, 2, 3])
    cfg = {
        # every third configuration has a width and an inner width that are multiples of nothing
        "architectures": ["Qwen3ForCausalLM"],
        "hidden_size": rng.choice([37, 50, 77, 101, 130, 203]) if seed % 3 == 2 else 8 * rng.choice([5, 9, 12, 17, 24, 33]),
        "intermediate_size": rng.choice([45, 99, 150, 211]) if seed % 3 == 2 else 16 * rng.choice([3, 7, 10, 13, 20]),
        "num_hidden_layers": layers,
        "num_attention_heads": nkv * group, "num_key_value_heads": nkv, "head_dim": hd,
        "vocab_size": rng.choice([97, 130, 255, 401, 1000, 1031]), "max_position_embeddings": 384,
        "rope_theta": rng.choice([1e4, 5e4, 1e6]), "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-4]),
        "tie_word_embeddings": rng.random() < 0.5, "attention_bias": rng.random() < 0.4, "hidden_act": "silu",
    }
    if rng.random() < 0.5:
        cfg["use_sliding_window"] = True
        cfg["sliding_window"] = rng.choice([7, 40, 64, 100])
        kinds = [rng.choice(["full_attention", "sliding_attention"]) for _ in range(layers)]
        if "sliding_attention" not in kinds:
            kinds[-1] = "sliding_attention"
        cfg["layer_types"] = kinds
    return cfg, rng


def rel_err(got, want):
    want = want.to(torch.float64)
    got = got.to(torch.float64).cpu()
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((got - want).abs() / scale).max())


@pytest.mark.parametrize("seed", range(32))
def test_a_random_configuration(seed, tmp_path):
    from plain_qwen3 import PlainQwen3
    from rocml_b200 import Engine, StepEntry
    cfg, rng = draw(seed)
    folder = str(tmp_path / "m")
    write_model(folder, cfg, seed=seed, std=0.05)
    plain = PlainQwen3(folder, dtype=torch.float64)
    vocab = cfg["vocab_size"]
    lens = [rng.randint(1, 30), rng.randint(60, 200), rng.randint(2, 90)]
    n_dec = [rng.randint(1, 6), rng.randint(1, 6), rng.randint(1, 6)]
    seqs = [prompt(seed * 10 + j, n + d, vocab) for j, (n, d) in enumerate(zip(lens, n_dec))]
    want = [plain.logits(s) for s in seqs]
    piece = rng.choice([32, 50, 64, 128, 4096])
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=3, max_step_tokens=piece)
        slots = [eng.new_sequence() for _ in seqs]
        out = eng.step([StepEntry(sl, s[:n], list(range(n))) for sl, s, n in zip(slots, seqs, lens)])
        err = rel_err(out, torch.cat([w[:n] for w, n in zip(want, lens)]))
        assert err < TOL[dtype], f"seed {seed} {dtype} prompts (pieces of {piece}): {err}; {cfg}"
        for t in range(max(n_dec)):
            live = [j for j in range(3) if t < n_dec[j]]
            out = eng.step([StepEntry(slots[j], [seqs[j][lens[j] + t]], [0]) for j in live])
            ref = torch.stack([want[j][lens[j] + t] for j in live])
            err = rel_err(out, ref)
            assert err < TOL[dtype], f"seed {seed} {dtype} token {t}: {err}; {cfg}"
            for j in live:
                if t == n_dec[j] - 1:
                    eng.release(slots[j])
        eng.cache.check_invariants()
        assert eng.cache.slots.n_held == 0


MEDIUM = [
    # widths from which the products of a long prompt run in the tensor-core kernels for many rows, whose
    # epilogues add into the residual; none a multiple of 256
    dict(hidden_size=320, intermediate_size=544, num_attention_heads=4, num_key_value_heads=2, head_dim=80,
         attention_bias=False, rms_norm_eps=1e-6, tie_word_embeddings=True),
    dict(hidden_size=520, intermediate_size=1040, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
         attention_bias=True, rms_norm_eps=3e-3, tie_word_embeddings=False),
]


@pytest.mark.parametrize("which", range(len(MEDIUM)))
@pytest.mark.parametrize("piece", [4096, 600])
def test_long_prompts_at_medium_widths(which, piece, tmp_path, monkeypatch):
    """Prompts of 700, 300 and 45 tokens in one step (and cut into pieces of 600): more than 256 rows a
    product, so the products add into the residual themselves where the sizes allow and the norms only
    normalise; then a few tokens one by one."""
    from plain_qwen3 import PlainQwen3
    from rocml_b200 import Engine, StepEntry
    cfg = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, vocab_size=777, max_position_embeddings=1024,
               rope_theta=1e6, hidden_act="silu", **MEDIUM[which])
    folder = str(tmp_path / "m")
    write_model(folder, cfg, seed=40 + which, std=0.05)
    plain = PlainQwen3(folder, dtype=torch.float64)
    lens, n_dec = [700, 300, 45], 3
    seqs = [prompt(900 + j, n + n_dec, cfg["vocab_size"]) for j, n in enumerate(lens)]
    want = [plain.logits(s) for s in seqs]
    places = [[0, n // 2, n - 2, n - 1] for n in lens]
    from rocml_b200 import kernels
    norms = []
    real = kernels.add_rmsnorm
    monkeypatch.setattr(kernels, "add_rmsnorm", lambda *a, **k: (norms.append(1), real(*a, **k))[1])
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=2048, max_slots=3, max_step_tokens=piece)
        slots = [eng.new_sequence() for _ in seqs]
        del norms[:]
        out = eng.step([StepEntry(sl, s[:n], w) for sl, s, n, w in zip(slots, seqs, lens, places)])
        err = rel_err(out, torch.cat([w[pl] for w, pl in zip(want, places)]))
        assert err < TOL[dtype], f"{dtype} prompts (pieces of {piece}): {err}"
        if piece == 4096:
            assert len(norms) == 2 * 3 + 1       # two a layer and the final one, in either mode
        for t in range(n_dec):
            out = eng.step([StepEntry(sl, [s[n + t]], [0]) for sl, s, n in zip(slots, seqs, lens)])
            err = rel_err(out, torch.stack([w[n + t] for w, n in zip(want, lens)]))
            assert err < TOL[dtype], f"{dtype} token {t}: {err}"
        for sl in slots:
            eng.release(sl)
        eng.cache.check_invariants()
