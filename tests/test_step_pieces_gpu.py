"""Steps larger than the engine's work space: the engine cuts them into pieces that run one after
another against the growing cache, and no logit may depend on where the cuts fall.

The reference feeds every long prompt through chunks of 512 tokens (rocml/src/forward/
chunk_forward.rs:33-53) and compares chunked with serial runs at lengths around the chunk size
(rocml/tests/dense_chunked_prefill_parity.rs:21,128-195).  Here the piece size is set far below
the prompts, so that pieces end in the middle of sequences, a sequence continues beside others,
wanted places fall into different pieces, and layers with a window give pages back between pieces.
"""
import pytest
import torch

from tiny_models import CONFIGS, prompt, write_model

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


def rel_err(got, want):
    want = want.to(torch.float64)
    got = got.to(torch.float64).cpu()
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((got - want).abs() / scale).max())


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E"])
def model_folder(request, tmp_path_factory):
    name = request.param
    folder = tmp_path_factory.mktemp(f"pieces_{name}")
    write_model(str(folder), CONFIGS[name], seed=31 + ord(name), std=0.05)
    return name, str(folder)


@pytest.fixture(scope="module")
def plain(model_folder):
    from plain_qwen3 import PlainQwen3
    return PlainQwen3(model_folder[1], dtype=torch.float64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("piece", [2, 64, 100, 128])
def test_one_long_prompt_in_pieces_then_decoding(model_folder, plain, dtype, piece):
    """A prompt many pieces long (on C and E many times window + piece), every place wanted, then 8
    tokens one by one."""
    from rocml_b200 import Engine, StepEntry
    name, folder = model_folder
    cfg = CONFIGS[name]
    vocab = cfg["vocab_size"]
    total = min(cfg["max_position_embeddings"], 620)
    if piece == 2:
        total = min(total, 90)
    ids = prompt(500 + piece, total, vocab)
    want = plain.logits(ids)
    n = total - 8
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=2, max_step_tokens=piece)
    slot = eng.new_sequence()
    steps_before = eng.launches
    got = [eng.step([StepEntry(slot, ids[:n], list(range(n)))]).clone()]
    assert eng.launches - steps_before == -(-n // piece)
    for t in range(n, total):
        got.append(eng.step([StepEntry(slot, [ids[t]], [0])]).clone())
    eng.cache.check_invariants()
    for g in eng.cache.kv_groups:
        if g.window:     # the window's pages only: the rest went back between the pieces
            assert g.pool.n_held <= (g.window + 63) // 64 + 1
    eng.release(slot)
    err = rel_err(torch.cat(got), want)
    assert err < TOL[dtype], f"{name} {dtype} piece={piece}: {err}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("piece", [64, 128])
def test_unequal_batch_cut_in_mid_sequence(model_folder, plain, dtype, piece):
    """Prompts of 200, 70 and 5 tokens in one step: the cuts fall inside the first and the second
    sequence, a piece holds the end of one sequence and the beginning of the next, and the wanted
    places are spread over the pieces and given out of order, some twice.  Then 8 steps of one token
    each, the shortest sequence ending first.  A second batch follows in the slots of the first."""
    from rocml_b200 import Engine, StepEntry
    name, folder = model_folder
    cfg = CONFIGS[name]
    vocab, maxp = cfg["vocab_size"], cfg["max_position_embeddings"]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=3, max_step_tokens=piece)
    for round_ in range(2):
        lens = [min(200, maxp - 8), 70, 5]
        ndec = [8, 5, 2]
        seqs = [prompt(900 + 10 * round_ + j, n + d, vocab) for j, (n, d) in enumerate(zip(lens, ndec))]
        want = [plain.logits(x) for x in seqs]
        places = [[p % lens[0] for p in (lens[0] - 1, 0, 63, 64, piece - 1, piece, 150, 63)], [69, 3, 3, 0], [4, 0]]
        slots = [eng.new_sequence() for _ in seqs]
        out = eng.step([StepEntry(s, x[:n], w) for s, x, n, w in zip(slots, seqs, lens, places)])
        ref = torch.cat([want[j][places[j]] for j in range(3)])
        assert out.shape == ref.shape
        err = rel_err(out, ref)
        assert err < TOL[dtype], f"{name} {dtype} piece={piece} round {round_} prompts: {err}"
        got = [[] for _ in seqs]
        for t in range(max(ndec)):
            live = [j for j in range(3) if t < ndec[j]]
            out = eng.step([StepEntry(slots[j], [seqs[j][lens[j] + t]], [0]) for j in live])
            for r, j in enumerate(live):
                got[j].append(out[r].clone())
            for j in live:
                if t == ndec[j] - 1:
                    eng.release(slots[j])
        for j in range(3):
            err = rel_err(torch.stack(got[j]), want[j][lens[j]:])
            assert err < TOL[dtype], f"{name} {dtype} piece={piece} round {round_} seq {j}: {err}"
        eng.cache.check_invariants()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pieces_and_whole_prompts_agree(model_folder, dtype):
    """The same batch through an engine whose work space holds it whole and through one that cuts it:
    the two differ by rounding only (float32: sums in another order; bfloat16: other kernels)."""
    from rocml_b200 import Engine, StepEntry
    name, folder = model_folder
    cfg = CONFIGS[name]
    vocab, maxp = cfg["vocab_size"], cfg["max_position_embeddings"]
    lens = [min(maxp, 250), 33, 101]
    seqs = [prompt(40 + j, n, vocab) for j, n in enumerate(lens)]
    outs = []
    for piece in (4096, 96):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=3, max_step_tokens=piece)
        slots = [eng.new_sequence() for _ in seqs]
        outs.append(eng.step([StepEntry(s, x, list(range(len(x)))) for s, x in zip(slots, seqs)]).float().cpu())
    err = rel_err(outs[1], outs[0].double())
    assert err < TOL[dtype], f"{name} {dtype}: {err}"


def test_a_step_that_cannot_fit_takes_nothing(model_folder):
    """The room for all pieces is checked before the first one runs."""
    from rocml_b200 import Engine, StepEntry
    from rocml_b200.errors import CacheFull, ContextOverflow
    name, folder = model_folder
    cfg = CONFIGS[name]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=128, max_slots=2, max_step_tokens=64)
    a, b = eng.new_sequence(), eng.new_sequence()
    ids = prompt(1, 100, cfg["vocab_size"])
    before = eng.launches
    with pytest.raises((CacheFull, ContextOverflow)):
        eng.step([StepEntry(a, ids, [0]), StepEntry(b, ids, [0])])
    assert eng.launches == before and eng.length(a) == 0 and eng.length(b) == 0
    assert all(g.pool.n_held == 0 for g in eng.cache.kv_groups)
    eng.cache.check_invariants()
