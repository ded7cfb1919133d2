"""Acceptance at full layer sizes: Qwen3-8B's sizes (hidden 4096, 32 query and 8 key/value heads of
128, intermediate 12288, vocabulary 151936, untied head, theta 1e6, eps 1e-6) with 2 of its 36
layers, random weights written once to a temporary folder.

The 32-bit engine against the plain implementation in float32, for three prompts of unequal
lengths under every way of cutting the work: each alone and whole, token by token, and batched
then decoded four steps; the same greedy token at every compared place.  Then bfloat16 against
the 32-bit engine, with the reference's rule for near ties (a row whose two best logits lie within
1e-2 of each other, relatively, may pick either: rocml/tests/greedy_parity.rs:30-34).  The
reference pins its numerics the same way, with a 32-bit cache used only by parity tests
(rocml/src/load_opts.rs:20-29, rocml/tests/greedy_parity.rs:108-186).

Sums here are 4,096 and 12,288 terms deep, the tiny models' at most 320: what the 32-bit path
loses to the order of its sums shows at this size or not at all.  Measured on a B200: 32-bit engine
against the plain implementation at most 7e-6 of a row's largest logit in every mode (the test
prints its worst); the bound below leaves a factor of three.
"""
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

N_LAYERS, N_LAYERS_OF = 2, 36
LENS = [40, 17, 5]
N_DECODE = 4
TOL_F32 = 2e-5          # of the row's largest |logit|
TOL_BF16 = 2.5e-2


def rel_err(got, want):
    want = want.to(torch.float64).cpu()
    got = got.to(torch.float64).cpu()
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((got - want).abs() / scale).max())


def near_tie(row, gap=1e-2):
    top = torch.topk(row.double(), 2).values
    return float((top[0] - top[1]) / top[0].abs().clamp_min(1e-30)) < gap


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    from plain_qwen3 import PlainQwen3
    from rocml_b200.config import CATALOG, config_from_dict
    from rocml_b200.weights import write_random_model
    sizes = dict(CATALOG["qwen3-8b"].config)
    assert sizes["num_hidden_layers"] == N_LAYERS_OF and sizes["hidden_size"] == 4096 and sizes["vocab_size"] == 151936
    sizes["num_hidden_layers"] = N_LAYERS
    folder = str(tmp_path_factory.mktemp("qwen3_8b_sizes"))
    write_random_model(folder, config_from_dict(sizes), seed=8)
    g = torch.Generator().manual_seed(80)
    seqs = [torch.randint(0, sizes["vocab_size"], (n + N_DECODE,), generator=g).tolist() for n in LENS]
    plain = PlainQwen3(folder, dtype=torch.float32)
    want = [plain.logits(s) for s in seqs]
    del plain
    return folder, seqs, want


def run_modes(folder, seqs, dtype):
    """Logits at every position of every sequence, three ways."""
    from rocml_b200 import Engine, StepEntry
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=512, max_slots=4)
    whole, single, batched = [], [], []
    for s in seqs:                                   # each alone and whole
        slot = eng.new_sequence()
        whole.append(eng.step([StepEntry(slot, s, list(range(len(s))))]).float().cpu())
        eng.release(slot)
    for s in seqs[1:]:                               # token by token from the first token
        slot = eng.new_sequence()
        single.append(torch.cat([eng.step([StepEntry(slot, [t], [0])]).float().cpu() for t in s]))
        eng.release(slot)
    slots = [eng.new_sequence() for _ in seqs]       # unequal prompts in one step, then one token each
    out = eng.step([StepEntry(sl, s[:n], list(range(n))) for sl, s, n in zip(slots, seqs, LENS)]).float().cpu()
    cuts = [0]
    for n in LENS:
        cuts.append(cuts[-1] + n)
    rows = [[out[cuts[j]:cuts[j + 1]]] for j in range(len(seqs))]
    for k in range(N_DECODE):
        live = [j for j in range(len(seqs)) if k < N_DECODE - j]     # the later sequences end earlier
        out = eng.step([StepEntry(slots[j], [seqs[j][LENS[j] + k]], [0]) for j in live]).float().cpu()
        for r, j in enumerate(live):
            rows[j].append(out[r:r + 1])
    for j in range(len(seqs)):
        batched.append(torch.cat(rows[j]))
    eng.cache.check_invariants()
    return whole, single, batched


@pytest.fixture(scope="module")
def f32(setup):
    folder, seqs, _ = setup
    return run_modes(folder, seqs, "float32")


def test_float32_equals_the_plain_implementation_in_every_mode(setup, f32):
    _, seqs, want = setup
    whole, single, batched = f32
    worst = 0.0
    for j in range(len(seqs)):
        cases = [("whole", whole[j], want[j])]
        if j >= 1:
            cases.append(("token by token", single[j - 1], want[j]))
        cases.append(("batched", batched[j], want[j][:len(batched[j])]))
        for mode, got, ref in cases:
            err = rel_err(got, ref)
            worst = max(worst, err)
            assert err < TOL_F32, f"sequence {j} {mode}: {err}"
            same = got.argmax(-1) == ref.argmax(-1)
            for t in (~same).nonzero().flatten().tolist():
                assert near_tie(ref[t], 1e-4), f"sequence {j} {mode}: another greedy token at place {t}"
    print(f"float32 against the plain implementation: worst {worst:.2e} of the row's largest logit")


def test_float32_does_not_depend_on_the_cut(setup, f32):
    _, seqs, _ = setup
    whole, single, batched = f32
    for j in range(len(seqs)):
        assert rel_err(batched[j], whole[j][:len(batched[j])]) < TOL_F32
        if j >= 1:
            assert rel_err(single[j - 1], whole[j]) < TOL_F32
            assert torch.equal(single[j - 1].argmax(-1), whole[j].argmax(-1))


def test_bfloat16_against_float32_with_the_near_tie_rule(setup, f32):
    folder, seqs, _ = setup
    whole32, single32, batched32 = f32
    whole, single, batched = run_modes(folder, seqs, "bfloat16")
    picked = ties = 0
    for j in range(len(seqs)):
        cases = [(whole[j], whole32[j]), (batched[j], batched32[j])]
        if j >= 1:
            cases.append((single[j - 1], single32[j - 1]))
        for got, ref in cases:
            assert rel_err(got, ref) < TOL_BF16
            for t in range(len(ref)):
                if near_tie(ref[t]):
                    ties += 1
                    continue
                picked += 1
                assert int(got[t].argmax()) == int(ref[t].argmax()), f"sequence {j} place {t}"
    # random weights give flat rows: about a quarter have their two best logits within 1e-2; the
    # rule must still leave most rows to be compared
    assert picked > 2 * ties


def test_a_long_prompt_in_pieces_at_full_sizes(setup):
    """4,200 tokens at the full head counts and widths: the engine cuts the prompt at 4,096 tokens (the first
    piece takes the projection whose epilogue normalises, rotates and caches; the second reads the first's
    keys from the pages), then three tokens one by one.  The last rows of the prompt and the decoded
    rows, 32-bit and bfloat16, against the plain implementation (whose head product is done on those rows
    only)."""
    from plain_qwen3 import PlainQwen3, linear, rmsnorm
    from rocml_b200 import Engine, StepEntry
    folder, _, _ = setup
    n, n_dec = 4200, 3
    g = torch.Generator().manual_seed(81)
    ids = torch.randint(0, 151936, (n + n_dec,), generator=g).tolist()
    plain = PlainQwen3(folder, dtype=torch.float32)
    rows = [4095, 4096, n - 1, n, n + 1, n + 2]
    hidden = plain.hidden_states(ids)[rows]
    want = linear(rmsnorm(hidden, plain.w["model.norm.weight"], plain.eps), plain.w["lm_head.weight"])
    del plain
    got = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=4352, max_slots=1)
        slot = eng.new_sequence()
        before = eng.launches
        out = [eng.step([StepEntry(slot, ids[:n], [4095, 4096, n - 1])]).float().cpu()]
        assert eng.launches - before == 2                       # two pieces
        for t in range(n_dec):
            out.append(eng.step([StepEntry(slot, [ids[n + t]], [0])]).float().cpu())
        got[dtype] = torch.cat(out)
        eng.release(slot)
        del eng
        torch.cuda.empty_cache()
    err32 = rel_err(got["float32"], want)
    assert err32 < TOL_F32, err32                                # measured 7e-6: sums over 4,200 keys in another order
    assert rel_err(got["bfloat16"], got["float32"]) < TOL_BF16
    for t in range(len(rows)):
        assert int(got["float32"][t].argmax()) == int(want[t].argmax()) or near_tie(want[t], 1e-4)
        assert int(got["bfloat16"][t].argmax()) == int(got["float32"][t].argmax()) or near_tie(got["float32"][t])
    print(f"long prompt, float32 against the plain implementation: {err32:.2e}")


@pytest.mark.parametrize("window", [None, 700])
def test_a_batch_of_long_prompts_at_full_sizes(setup, window, tmp_path):
    """Eight prompts of 600 to 1,024 tokens in one step (thousands of attention blocks, every multiprocessor
    busy, two pieces of at most 4,096 tokens), then two tokens each: bfloat16 against the 32-bit engine at the
    prompts' last places and the decoded ones, twice over so that slots and pages are used again.  What depends
    on the order in which a busy GPU runs a kernel's blocks and warps shows here or nowhere; with a sliding
    window in the second layer the warps of an attention block differ most in what they have to do, and a
    token whose row went wrong in the first layer spoils every later token that sees it."""
    from rocml_b200 import Engine, StepEntry
    folder, _, _ = setup
    if window is not None:
        from rocml_b200.config import CATALOG, config_from_dict
        from rocml_b200.weights import write_random_model
        sizes = dict(CATALOG["qwen3-8b"].config)
        sizes.update(num_hidden_layers=N_LAYERS, use_sliding_window=True, sliding_window=window, max_window_layers=0,
                     layer_types=["sliding_attention", "full_attention"])
        folder = str(tmp_path / "windowed")
        write_random_model(folder, config_from_dict(sizes), seed=9)
    g = torch.Generator().manual_seed(82)
    lens = [1024, 600, 777, 1000, 913, 650, 1024, 841]
    prompts = [torch.randint(0, 151936, (n + 2,), generator=g).tolist() for n in lens]
    got = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=8 * 1088, max_slots=8)
        rounds = []
        for _ in range(2):
            slots = [eng.new_sequence() for _ in lens]
            out = [eng.step([StepEntry(s, p[:n], [n - 1]) for s, p, n in zip(slots, prompts, lens)]).float().cpu()]
            for t in range(2):
                out.append(eng.step([StepEntry(s, [p[n + t]], [0]) for s, p, n in zip(slots, prompts, lens)]).float().cpu())
            rounds.append(torch.cat(out))
            for s in slots:
                eng.release(s)
        got[dtype] = rounds
        del eng
        torch.cuda.empty_cache()
    assert torch.equal(got["float32"][0], got["float32"][1])         # the same work gives the same bits
    assert torch.equal(got["bfloat16"][0], got["bfloat16"][1])
    assert not torch.isnan(got["bfloat16"][0]).any()
    err = rel_err(got["bfloat16"][0], got["float32"][0])
    assert err < TOL_BF16, err
    for r in range(got["float32"][0].shape[0]):
        assert int(got["bfloat16"][0][r].argmax()) == int(got["float32"][0][r].argmax()) or near_tie(got["float32"][0][r])
