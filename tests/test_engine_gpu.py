"""The engine against the plain implementation, in 32-bit and in bfloat16: each request alone
and whole; with the last 32 tokens one by one; in batches of unequal lengths whose shorter
requests end earlier, one batch after another so that slots are used again."""
import pytest
import torch

from tiny_models import CONFIGS, prompt, write_model

pytestmark = pytest.mark.gpu

# Tolerances, as a fraction of the largest |logit| of the row compared.
# float32: sums of a few hundred float32 terms in another order than the plain implementation
# (2^-24 per operation, a few thousand operations deep) stay below 1e-5 of the row's scale.
# bfloat16: activations are rounded to 8 bits of mantissa (2^-9 relative) between kernels,
# a dozen roundings per layer; 2e-2 of the row's scale bounds that for these depths.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


def rel_err(got, want):
    want = want.to(torch.float64)
    got = got.to(torch.float64).cpu()
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((got - want).abs() / scale).max())


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E"])
def model_folder(request, tmp_path_factory):
    name = request.param
    folder = tmp_path_factory.mktemp(f"tiny_{name}")
    write_model(str(folder), CONFIGS[name], seed=11 + ord(name), std=0.05)
    return name, str(folder)


@pytest.fixture(scope="module")
def plain(model_folder):
    from plain_qwen3 import PlainQwen3
    return PlainQwen3(model_folder[1], dtype=torch.float64)


def lengths_for(name):
    maxp = CONFIGS[name]["max_position_embeddings"]
    return [n for n in (1, 7, 33, 64, 65, 100, 129, 200, 256, 300, 500) if n <= maxp]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(model_folder, plain, dtype):
    from rocml_b200 import Engine, StepEntry
    name, folder = model_folder
    vocab = CONFIGS[name]["vocab_size"]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024)
    for n in lengths_for(name):
        ids = prompt(n, n, vocab)
        slot = eng.new_sequence()
        got = eng.step([StepEntry(slot, ids, list(range(n)))])
        eng.release(slot)
        assert got.shape == (n, vocab)
        err = rel_err(got, plain.logits(ids))
        assert err < TOL[dtype], f"{name} {dtype} n={n}: {err}"
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_last_32_one_by_one(model_folder, plain, dtype, graphs):
    from rocml_b200 import Engine, StepEntry
    name, folder = model_folder
    vocab = CONFIGS[name]["vocab_size"]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, use_graphs=graphs)
    for n in [m for m in lengths_for(name) if m > 32][:4]:
        ids = prompt(100 + n, n, vocab)
        want = plain.logits(ids)
        slot = eng.new_sequence()
        head = n - 32
        got = [eng.step([StepEntry(slot, ids[:head], [head - 1])]).clone()]
        for t in range(head, n):
            got.append(eng.step([StepEntry(slot, [ids[t]], [0])]).clone())
        eng.release(slot)
        got = torch.cat(got, dim=0)
        err = rel_err(got, want[head - 1:])
        assert err < TOL[dtype], f"{name} {dtype} n={n} graphs={graphs}: {err}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_and_slot_reuse(model_folder, plain, dtype):
    """Batches of unequal prompts, then one token each; shorter requests end earlier; a second
    and third batch reuse the slots and pages of the first."""
    from rocml_b200 import Engine, StepEntry
    name, folder = model_folder
    vocab = CONFIGS[name]["vocab_size"]
    maxp = CONFIGS[name]["max_position_embeddings"]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024)
    rounds = [[(5, 8), (70, 3), (17, 12), (1, 5)], [(64, 4), (2, 9), (33, 1)], [(90, 6), (90, 2)]]
    for r, batch in enumerate(rounds):
        seqs = []
        for j, (plen, ndec) in enumerate(batch):
            total = min(plen + ndec, maxp)
            ids = prompt(1000 * r + j, total, vocab)
            seqs.append({"ids": ids, "plen": min(plen, total - 1), "slot": eng.new_sequence(),
                         "want": plain.logits(ids), "got": []})
        out = eng.step([StepEntry(s["slot"], s["ids"][:s["plen"]], [s["plen"] - 1]) for s in seqs])
        for i, s in enumerate(seqs):
            s["got"].append(out[i].clone())
            s["pos"] = s["plen"]
        live = list(seqs)
        while live:
            done = [s for s in live if s["pos"] >= len(s["ids"])]
            for s in done:
                eng.release(s["slot"])
            live = [s for s in live if s["pos"] < len(s["ids"])]
            if not live:
                break
            out = eng.step([StepEntry(s["slot"], [s["ids"][s["pos"]]], [0]) for s in live])
            for i, s in enumerate(live):
                s["got"].append(out[i].clone())
                s["pos"] += 1
        for j, s in enumerate(seqs):
            got = torch.stack(s["got"])
            err = rel_err(got, s["want"][s["plen"] - 1:])
            assert err < TOL[dtype], f"{name} {dtype} round {r} seq {j}: {err}"
        eng.cache.check_invariants()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(model_folder, plain, dtype):
    """A sequence grown one token at a time from its very first token, across page boundaries and
    across the context buckets of the captured graphs, next to a second sequence that starts later
    and ends earlier; every logit row is compared."""
    from rocml_b200 import Engine, StepEntry
    name, folder = model_folder
    vocab = CONFIGS[name]["vocab_size"]
    n = min(CONFIGS[name]["max_position_embeddings"], 300)
    ids = prompt(77, n, vocab)
    start, n_other = n // 3, 40          # the second sequence lives for 40 steps from step n / 3
    other = prompt(78, n_other, vocab)
    want, want_other = plain.logits(ids), plain.logits(other)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024)
    a = eng.new_sequence()
    got, got_other, b = [], [], None
    for t in range(n):
        entries = [StepEntry(a, [ids[t]], [0])]
        k = t - start
        if 0 <= k < n_other:
            if k == 0:
                b = eng.new_sequence()
            entries.append(StepEntry(b, [other[k]], [0]))
        out = eng.step(entries)
        got.append(out[0].clone())
        if len(entries) == 2:
            got_other.append(out[1].clone())
            if k == n_other - 1:
                eng.release(b)
    err = rel_err(torch.stack(got), want)
    err_other = rel_err(torch.stack(got_other), want_other)
    assert err < TOL[dtype] and err_other < TOL[dtype], f"{name} {dtype}: {err} {err_other}"


DEFER_CFG = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 3,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 300,
    "max_position_embeddings": 512, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "attention_bias": False, "hidden_act": "silu",
}


@pytest.mark.parametrize("graphs", [False, True])
def test_decode_without_norm_kernels(tmp_path, monkeypatch, graphs):
    """Few tokens per step, head size 128: the products that feed the residual stream add into it
    themselves and prepare the next norm's rows, whose 1/RMS the following product applies, so a layer
    runs no norm kernel.  The library picks this from the weights' sizes; here a small model is made to
    split its sums as a large one would.  Two sequences of unequal lengths, decoded next to each other
    from their first token, against the plain implementation, and against the same engine with the
    offers turned off."""
    from plain_qwen3 import PlainQwen3
    from rocml_b200 import Engine, StepEntry, kernels
    from rocml_b200.parts.linear import Linear
    folder = str(tmp_path / "m")
    write_model(folder, DEFER_CFG, seed=5, std=0.06)
    plain = PlainQwen3(folder, dtype=torch.float32)
    monkeypatch.setattr(Linear, "_splits", lambda self, m: 1 if m > 16 else (2 if self.k == 256 else 8))
    calls = {"residual": 0, "norm": 0}
    real_res, real_norm = kernels.gemm_tcgen05_residual, kernels.add_rmsnorm
    monkeypatch.setattr(kernels, "gemm_tcgen05_residual",
                        lambda *a, **k: calls.__setitem__("residual", calls["residual"] + 1) or real_res(*a, **k))
    monkeypatch.setattr(kernels, "add_rmsnorm",
                        lambda *a, **k: calls.__setitem__("norm", calls["norm"] + 1) or real_norm(*a, **k))
    vocab = DEFER_CFG["vocab_size"]
    ids = [prompt(5, 140, vocab), prompt(6, 90, vocab)]
    want = [plain.logits(x) for x in ids]
    results = {}
    for defer in ("1", "0"):
        monkeypatch.setenv("RB_DEFER", defer)
        calls["residual"] = calls["norm"] = 0
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024, use_graphs=graphs)
        slots = [eng.new_sequence(), eng.new_sequence()]
        got = [[], []]
        for t in range(140):
            live = [j for j in range(2) if t < len(ids[j])]
            out = eng.step([StepEntry(slots[j], [ids[j][t]], [0]) for j in live])
            for r, j in enumerate(live):
                got[j].append(out[r].clone())
        results[defer] = [torch.stack(g) for g in got]
        for j in range(2):
            assert rel_err(results[defer][j], want[j]) < TOL["bfloat16"]
        if defer == "1":
            # two products a layer went into the residual (the last layer's feed-forward has no norm to
            # prepare), and only the first layer's first norm and the final norm ran as kernels
            n_layers = DEFER_CFG["num_hidden_layers"]
            if not graphs:
                assert calls["residual"] == 140 * (2 * n_layers - 1)
                assert calls["norm"] == 140 * 2
        else:
            assert calls["residual"] == 0
    for j in range(2):
        assert rel_err(results["1"][j], results["0"][j].double().cpu()) < TOL["bfloat16"]


@pytest.mark.parametrize("blocks", [1, 2, 5])
@pytest.mark.parametrize("graphs", [False, True])
def test_decode_attention_with_pages_shared_out_equally(tmp_path, monkeypatch, blocks, graphs):
    """Large batches and long contexts make decode attention cut the pages of all sequences into equal
    runs, one per block, a block finishing one sequence and starting the next.  The library picks that
    from the batch and the device; here a small model is made to do it with fewer blocks than
    sequences, as many, and more: three sequences of unequal lengths after prompts of unequal lengths,
    the shortest ending first, against the plain implementation."""
    from plain_qwen3 import PlainQwen3
    from rocml_b200 import Engine, StepEntry, kernels
    folder = str(tmp_path / "m")
    write_model(folder, DEFER_CFG, seed=8, std=0.06)
    plain = PlainQwen3(folder, dtype=torch.float32)
    monkeypatch.setattr(kernels, "decode_split", lambda n_seqs, groups, n_pages, device=0: (blocks, 0))
    vocab = DEFER_CFG["vocab_size"]
    ids = [prompt(11, 300, vocab), prompt(12, 150, vocab), prompt(13, 70, vocab)]
    starts = [250, 70, 3]
    want = [plain.logits(x) for x in ids]
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024, use_graphs=graphs)
    slots = [eng.new_sequence() for _ in ids]
    out = eng.step([StepEntry(s, x[:n], [n - 1]) for s, x, n in zip(slots, ids, starts)])
    got = [[out[j].clone()] for j in range(3)]
    for t in range(80):
        live = [j for j in range(3) if starts[j] + t < len(ids[j])]
        if not live:
            break
        out = eng.step([StepEntry(slots[j], [ids[j][starts[j] + t]], [0]) for j in live])
        for r, j in enumerate(live):
            got[j].append(out[r].clone())
    for j in range(3):
        g = torch.stack(got[j])
        assert rel_err(g, want[j][starts[j] - 1:starts[j] - 1 + len(g)]) < TOL["bfloat16"]
    kernels.check_status("cuda:0")


def test_prompts_add_into_the_residual_inside_the_products(tmp_path, monkeypatch):
    """A prompt of more than 256 tokens: the o- and down-projection add into the residual stream in
    their own epilogue and the norms after them only normalise.  Same logits as the plain
    implementation, and as the same engine with the offers turned off; a second, shorter prompt
    beside the first keeps the plain path for neither."""
    from plain_qwen3 import PlainQwen3
    from rocml_b200 import Engine, StepEntry, kernels
    folder = str(tmp_path / "m")
    write_model(folder, DEFER_CFG, seed=21, std=0.06)
    plain = PlainQwen3(folder, dtype=torch.float32)
    calls = {"add": 0}
    real_add = kernels.gemm_tcgen05_add
    monkeypatch.setattr(kernels, "gemm_tcgen05_add",
                        lambda *a, **k: calls.__setitem__("add", calls["add"] + 1) or real_add(*a, **k))
    vocab = DEFER_CFG["vocab_size"]
    ids = [prompt(31, 400, vocab), prompt(32, 77, vocab)]
    rows = [[0, 255, 256, 399], [0, 76]]
    want = torch.cat([plain.logits(x)[r] for x, r in zip(ids, rows)])
    got = {}
    for defer in ("1", "0"):
        monkeypatch.setenv("RB_DEFER", defer)
        calls["add"] = 0
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024)
        slots = [eng.new_sequence(), eng.new_sequence()]
        got[defer] = eng.step([StepEntry(s, x, r) for s, x, r in zip(slots, ids, rows)]).float().cpu()
        assert rel_err(got[defer], want) < TOL["bfloat16"]
        assert calls["add"] == (2 * DEFER_CFG["num_hidden_layers"] if defer == "1" else 0)
    assert rel_err(got["1"], got["0"].double()) < TOL["bfloat16"]
    kernels.check_status("cuda:0")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_graphs_are_bounded(tmp_path, monkeypatch, dtype):
    """Decode graphs are kept per context bucket; only ``max_graphs`` of them stay, the least recently
    used goes first, and a bucket that was dropped is captured again when a sequence comes back to it.
    Buckets of 32 tokens here, so that a sequence of 290 tokens crosses ten of them with a cap of 3;
    every logit row is compared with the plain implementation."""
    from plain_qwen3 import PlainQwen3
    from rocml_b200 import Engine, StepEntry
    from rocml_b200.engine import engine as engine_module
    folder = str(tmp_path / "m")
    write_model(folder, CONFIGS["D"], seed=61, std=0.05)
    plain = PlainQwen3(folder, dtype=torch.float64)
    monkeypatch.setattr(engine_module, "_ctx_bucket", lambda n: max(32, -(-n // 32) * 32))
    vocab = CONFIGS["D"]["vocab_size"]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=2, max_graphs=3)
    for round_ in range(2):              # the second sequence starts again in the first, dropped, bucket
        ids = prompt(300 + round_, 290, vocab)
        want = plain.logits(ids)
        slot = eng.new_sequence()
        got = []
        for t, tok in enumerate(ids):
            got.append(eng.step([StepEntry(slot, [tok], [0])]).clone())
            assert len(eng._graphs) <= 3
        eng.release(slot)
        assert rel_err(torch.cat(got), want) < TOL[dtype]
    assert eng.graphs_captured == 20 and list(eng._graphs) == [(1, 256), (1, 288), (1, 320)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_three_hundred_short_sequences_at_once(tmp_path, dtype):
    """More live sequences than any kernel's per-batch tables were sized for by habit (256): the cache
    gives every page's worth of budget a slot, the prompts go in one step, then three tokens each."""
    from plain_qwen3 import PlainQwen3
    from rocml_b200 import Engine, StepEntry
    folder = str(tmp_path / "m")
    write_model(folder, CONFIGS["D"], seed=71, std=0.05)
    plain = PlainQwen3(folder, dtype=torch.float64)
    vocab = CONFIGS["D"]["vocab_size"]
    n_seqs = 300
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=64 * n_seqs)
    assert eng.cache.max_slots == n_seqs
    seqs = [prompt(5000 + j, 3 + j % 9 + 3, vocab) for j in range(n_seqs)]
    lens = [len(s) - 3 for s in seqs]
    slots = [eng.new_sequence() for _ in seqs]
    out = eng.step([StepEntry(sl, s[:n], [n - 1]) for sl, s, n in zip(slots, seqs, lens)]).clone()
    got = [[out[j]] for j in range(n_seqs)]
    for t in range(3):
        out = eng.step([StepEntry(sl, [s[n + t]], [0]) for sl, s, n in zip(slots, seqs, lens)]).clone()
        for j in range(n_seqs):
            got[j].append(out[j])
    for j in list(range(0, n_seqs, 23)) + [255, 256, 257, n_seqs - 1]:
        want = plain.logits(seqs[j])[lens[j] - 1:]
        assert rel_err(torch.stack(got[j]), want) < TOL[dtype], (j, dtype)
    for sl in slots:
        eng.release(sl)
    eng.cache.check_invariants()


@pytest.mark.gpu
def test_weights_reach_the_device_through_the_library_reader(tmp_path):
    """File -> pinned staging -> device by the library's own reader: tensors larger than a staging buffer
    (64 MB), of odd sizes, several in a row on one handle, and a conversion on the device afterwards."""
    from rocml_b200.weights import ModelFiles, save_state_dict
    g = torch.Generator().manual_seed(5)
    state = {"big": torch.randn((5000, 4099), generator=g).bfloat16(),          # 41 MB
             "odd": torch.randn((1234567,), generator=g),                       # 4.9 MB float32
             "bigger": torch.randint(-100, 100, (5, 33_000_001), generator=g, dtype=torch.int8),   # 165 MB: three pieces
             "small": torch.randn((3, 5), generator=g).half(), "none": torch.zeros((0, 7))}
    save_state_dict(str(tmp_path / "model.safetensors"), state)
    with ModelFiles(str(tmp_path)) as files:
        got = {}
        for k, v in state.items():
            got[k] = torch.empty(v.shape, dtype=v.dtype, device="cuda")
            files.read_into(k, got[k])
        half = got["small"].to(torch.bfloat16)
    torch.cuda.synchronize()
    for k, v in state.items():
        assert torch.equal(got[k].cpu(), v), k
    assert torch.equal(half.cpu(), state["small"].to(torch.bfloat16))
