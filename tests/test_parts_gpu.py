"""Each part alone against the plain functions; a schedule that names a layer twice and lets a layer
read another's cache; and a toy mixer with state of its own, defined here, registered, built and
stepped without touching the library's files."""
import math

import pytest
import torch

import plain_qwen3 as P
from tiny_models import prompt

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def env(dtype):
    from rocml_b200.parts import BuildEnv
    return BuildEnv(DEV, dtype)


def rnd(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def one_sequence_batch(n, old=0, slot=0, want=()):
    from rocml_b200.engine.batch import BatchBuffers, HostBatch, StepBatch, pack_entries
    packed = pack_entries([slot], [old], [list(range(n))], [list(want)])
    buf = BatchBuffers(max(n, 1), 1, max(n, 1), DEV)
    buf.fill(*packed, [slot], pad_tokens=n, pad_seqs=1, pad_want=len(want))
    return StepBatch(n_tokens=n, n_seqs=1, n_want=len(want), max_q_len=n, max_kv_len=old + n, is_decode=False,
                     token_ids=buf.token_ids, positions=buf.positions, slot_of_token=buf.slot_of_token,
                     seq_slot=buf.seq_slot, cu_q=buf.cu_q, kv_len=buf.kv_len, want_rows=buf.want_rows,
                     host=HostBatch([slot], [n], [old + n], list(want)))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_norm_part(dtype, tol):
    from rocml_b200.config import NormSpec
    from rocml_b200.parts import build_norm
    H, T = 72, 5
    norm = build_norm(NormSpec("rmsnorm", 1e-5), H, env(dtype))
    assert [d.name for d in norm.declare("x.norm")] == ["x.norm.weight"]
    w = (1 + 0.1 * rnd((H,), 1)).to(dtype)
    norm.load({"x.norm.weight": w.to(DEV)}, "x.norm")
    resid, delta = rnd((T, H), 2), rnd((2, T, H), 3)
    r = resid.to(DEV)
    out = norm.forward(r, delta.to(DEV), T)
    total = resid.double() + delta.double().sum(0)
    want = P.rmsnorm(total, w.double(), 1e-5)
    assert (out.cpu().double() - want).abs().max() < tol * want.abs().max()
    assert (r.cpu().double() - total).abs().max() < 1e-5


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_feed_forward_part(dtype, tol):
    from rocml_b200.config import FeedForwardSpec
    from rocml_b200.parts import build_feed_forward
    H, I, T = 96, 208, 7
    ff = build_feed_forward(FeedForwardSpec.make("gated_mlp", intermediate=I, activation="silu"), H, env(dtype))
    ws = {"m.gate_proj.weight": rnd((I, H), 1, 0.1), "m.up_proj.weight": rnd((I, H), 2, 0.1),
          "m.down_proj.weight": rnd((H, I), 3, 0.1)}
    ws = {k: v.to(dtype) for k, v in ws.items()}
    assert sorted(d.name for d in ff.declare("m.")) == sorted(ws)
    ff.load({k: v.to(DEV) for k, v in ws.items()}, "m.")
    x = rnd((T, H), 4).to(dtype)
    delta = ff.forward(x.to(DEV), one_sequence_batch(T))
    xd = x.double()
    want = P.linear(P.silu_mul(P.linear(xd, ws["m.gate_proj.weight"].double()), P.linear(xd, ws["m.up_proj.weight"].double())),
                    ws["m.down_proj.weight"].double())
    got = delta.sum(0).cpu().double()
    assert (got - want).abs().max() < tol * want.abs().max()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("window,bias,rot", [(None, False, None), (9, True, 16)])
def test_attention_part_prompt_then_decode(dtype, tol, window, bias, rot):
    """The mixer alone, with its own cache: a prompt in one step, then tokens one by one, against
    the plain attention block over the whole sequence; once with a window, biases and a partial
    rotation."""
    from rocml_b200.cache import SequenceCache
    from rocml_b200.config import MixerSpec, PositionSpec
    from rocml_b200.parts import build_mixer
    H, nq, nkv, hd, T = 80, 6, 2, 32, 41
    pos_spec = PositionSpec("rope_neox", theta=1e4, rot_dim=rot)
    spec = MixerSpec.make("attention", position=pos_spec, n_heads=nq, n_kv_heads=nkv, head_dim=hd, bias=bias,
                          qk_norm=True, qk_norm_eps=1e-6, window=window, scale=None)
    mixer = build_mixer(spec, H, env(dtype))
    ws = {}
    for d in mixer.declare("a."):
        t = rnd(d.shape, len(ws) + 1, 0.15)
        ws[d.name] = (1 + t if d.role == "norm" else t).to(dtype)
    mixer.load({k: v.to(DEV) for k, v in ws.items()}, "a.")
    cache = SequenceCache([mixer.cache_requirement()], [None], 256, 2, 128, dtype, DEV)
    slot = cache.alloc_slot()
    x = rnd((T, H), 99).to(dtype)

    def run(lo, hi):
        cache.grow(slot, hi - lo)
        cache.flush()
        b = one_sequence_batch(hi - lo, old=lo, slot=slot)
        b.is_decode = hi - lo == 1
        out = mixer.forward(x[lo:hi].to(DEV).contiguous(), b, cache.views[0]).sum(0)
        cache.commit(slot, hi - lo)
        return out.cpu().double()

    got = torch.cat([run(0, 30)] + [run(t, t + 1) for t in range(30, T)])
    # plain: the same block over the whole sequence
    wd = {k: v.double() for k, v in ws.items()}
    xd = x.double()
    bget = (lambda n: wd[f"a.{n}.bias"]) if bias else (lambda n: None)
    q = P.linear(xd, wd["a.q_proj.weight"], bget("q_proj")).view(T, nq, hd)
    k = P.linear(xd, wd["a.k_proj.weight"], bget("k_proj")).view(T, nkv, hd)
    v = P.linear(xd, wd["a.v_proj.weight"], bget("v_proj")).view(T, nkv, hd)
    q, k = P.rmsnorm(q, wd["a.q_norm.weight"], 1e-6), P.rmsnorm(k, wd["a.k_norm.weight"], 1e-6)
    r = rot or hd
    q = torch.cat([P.rope_neox(q[..., :r], range(T), 1e4), q[..., r:]], -1)
    k = torch.cat([P.rope_neox(k[..., :r], range(T), 1e4), k[..., r:]], -1)
    want = P.linear(P.attention(q, k, v, window=window).reshape(T, nq * hd), wd["a.o_proj.weight"], bget("o_proj"))
    assert (got - want).abs().max() < tol * want.abs().max()


def test_position_part_tables():
    from rocml_b200.config import PositionSpec
    from rocml_b200.parts import build_position
    full = build_position(PositionSpec("rope_neox", theta=1e6), 32, env(torch.float32))
    part = build_position(PositionSpec("rope_neox", theta=5e4, rot_dim=8), 32, env(torch.float32))
    none = build_position(PositionSpec("none"), 32, env(torch.float32))
    assert full.rot_dim == 32 and full.inv_freq.shape == (16,) and part.rot_dim == 8 and none.inv_freq is None
    want = torch.pow(torch.tensor(5e4, dtype=torch.float64), -2.0 * torch.arange(4, dtype=torch.float64) / 8).float()
    assert torch.equal(part.inv_freq.cpu(), want)


def test_schedule_with_a_repeated_layer_and_a_shared_cache(tmp_path):
    """The order in which layers run is data: layer 0 runs twice (with a cache for each run), and a
    last layer keeps no cache but reads the one of the first run.  Checked against the plain parts
    composed in the same order."""
    from rocml_b200.config import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                   ScheduleEntry)
    from rocml_b200.engine import Engine, Model, StepEntry
    from rocml_b200.weights.random_init import random_tensor
    H, nq, nkv, hd, I, V = 64, 4, 2, 16, 96, 101
    norm = NormSpec("rmsnorm", 1e-6)
    pos = PositionSpec("rope_neox", theta=1e4)
    att = MixerSpec.make("attention", position=pos, n_heads=nq, n_kv_heads=nkv, head_dim=hd, bias=False,
                         qk_norm=True, qk_norm_eps=1e-6, window=None, scale=None)
    ff = FeedForwardSpec.make("gated_mlp", intermediate=I, activation="silu")
    layers = tuple(LayerSpec(f"model.layers.{i}", att, ff, norm, norm) for i in range(3))
    sched = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2, reads_cache_of=0))
    spec = ModelSpec("ToySchedule", H, V, 256, layers, sched, norm, tie_embeddings=True)
    model = Model(spec, env(torch.float32))
    tensors = {d.name: random_tensor(d, 7).float() * (2.5 if d.role == "matrix" else 1.0) for d in model.declare()}
    assert "model.layers.2.self_attn.k_proj.weight" not in tensors      # the reading layer projects only q
    model.load({k: v.to(DEV) for k, v in tensors.items()})
    eng = Engine(model, max_tokens=256)
    assert len(eng.cache.kv_groups) == 1 and eng.cache.kv_groups[0].n_entries == 3
    ids = prompt(3, 37, V)
    slot = eng.new_sequence()
    got = [eng.step([StepEntry(slot, ids[:20], list(range(20)))]).clone()]
    got += [eng.step([StepEntry(slot, [t], [0])]).clone() for t in ids[20:]]
    got = torch.cat(got).cpu().double()

    w = {k: v.double() for k, v in tensors.items()}
    T = len(ids)
    x = w["model.embed_tokens.weight"][ids]
    k_first = v_first = None
    for run, e in enumerate(sched):
        p = f"model.layers.{e.layer}."
        xn = P.rmsnorm(x, w[p + "input_layernorm.weight"], 1e-6)
        q = P.rope_neox(P.rmsnorm(P.linear(xn, w[p + "self_attn.q_proj.weight"]).view(T, nq, hd),
                                  w[p + "self_attn.q_norm.weight"], 1e-6), range(T), 1e4)
        if e.reads_cache_of is None:
            k = P.rope_neox(P.rmsnorm(P.linear(xn, w[p + "self_attn.k_proj.weight"]).view(T, nkv, hd),
                                      w[p + "self_attn.k_norm.weight"], 1e-6), range(T), 1e4)
            v = P.linear(xn, w[p + "self_attn.v_proj.weight"]).view(T, nkv, hd)
            if run == 0:
                k_first, v_first = k, v
        else:
            k, v = k_first, v_first
        x = x + P.linear(P.attention(q, k, v).reshape(T, nq * hd), w[p + "self_attn.o_proj.weight"])
        xn = P.rmsnorm(x, w[p + "post_attention_layernorm.weight"], 1e-6)
        x = x + P.linear(P.silu_mul(P.linear(xn, w[p + "mlp.gate_proj.weight"]), P.linear(xn, w[p + "mlp.up_proj.weight"])),
                         w[p + "mlp.down_proj.weight"])
    want = P.linear(P.rmsnorm(x, w["model.norm.weight"], 1e-6), w["model.embed_tokens.weight"])
    assert (got - want).abs().max() < 3e-5 * want.abs().max()


def test_a_toy_mixer_with_state_registers_builds_and_steps():
    """A mixer defined HERE, with per-sequence state of fixed size (a running sum of its projected
    inputs), is registered, built from a spec, given its state by the cache, and stepped by the
    engine: whole prompts, single tokens, two sequences at once, a slot used again."""
    from rocml_b200.cache import StateRequirement
    from rocml_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, ScheduleEntry
    from rocml_b200.engine import Engine, Model, StepEntry
    from rocml_b200.parts import Mixer, register_mixer
    from rocml_b200.weights import TensorDecl
    from rocml_b200.weights.random_init import random_tensor

    @register_mixer("toy_running_sum")
    class RunningSum(Mixer):
        graph_safe = False   # it reads the batch on the host: the engine must not capture it

        def __init__(self, spec, hidden, env):
            self.hidden, self.width, self.env = hidden, spec.params["width"], env

        def cache_requirement(self):
            return StateRequirement((self.width,), torch.float32)

        def declare(self, prefix):
            return [TensorDecl(f"{prefix}in.weight", (self.width, self.hidden)),
                    TensorDecl(f"{prefix}out.weight", (self.hidden, self.width))]

        def load(self, tensors, prefix):
            self.w_in, self.w_out = tensors[f"{prefix}in.weight"].float(), tensors[f"{prefix}out.weight"].float()

        def forward(self, xn, batch, view):
            out = torch.zeros((1, batch.n_tokens, self.hidden), dtype=torch.float32, device=xn.device)
            start = 0
            for slot, n in zip(batch.host.seq_slots, batch.host.q_lens):
                u = xn[start:start + n].float() @ self.w_in.t()
                run = view.state[slot] + torch.cumsum(u, 0)          # state: the sum over earlier tokens
                view.state[slot] = run[-1]
                out[0, start:start + n] = run @ self.w_out.t()
                start += n
            return out

    H, V, W = 48, 77, 12
    norm = NormSpec("rmsnorm", 1e-6)
    # the tensors' names come from the spec alone: the parts know no names of their own
    layer = LayerSpec("model.layers.0", MixerSpec.make("toy_running_sum", width=W),
                      FeedForwardSpec.make("gated_mlp", intermediate=64, activation="silu",
                                           names={"gate": "w1", "up": "w3", "down": "w2"}), norm, norm,
                      mixer_norm_name="ln_mix", mixer_name="mix.", ff_norm_name="ln_ff", ff_name="ffn.")
    spec = ModelSpec("ToyState", H, V, 128, (layer,), (ScheduleEntry(0),), norm, tie_embeddings=True)
    model = Model(spec, env(torch.float32))
    assert not model.graph_safe
    tensors = {d.name: random_tensor(d, 5).float() * (3.0 if d.role == "matrix" else 1.0) for d in model.declare()}
    assert sorted(tensors) == sorted(
        ["model.embed_tokens.weight", "model.norm.weight"] + [f"model.layers.0.{n}.weight" for n in (
            "ln_mix", "mix.in", "mix.out", "ln_ff", "ffn.w1", "ffn.w3", "ffn.w2")])
    model.load({k: v.to(DEV) for k, v in tensors.items()})
    eng = Engine(model, max_tokens=256, max_slots=2)
    assert not eng.use_graphs and len(eng.cache.state_groups) == 1 and not eng.cache.kv_groups

    w = {k: v.double() for k, v in tensors.items()}

    def plain(ids):
        x = w["model.embed_tokens.weight"][ids]
        xn = P.rmsnorm(x, w["model.layers.0.ln_mix.weight"], 1e-6)
        u = torch.cumsum(xn @ w["model.layers.0.mix.in.weight"].t(), 0)
        x = x + u @ w["model.layers.0.mix.out.weight"].t()
        xn = P.rmsnorm(x, w["model.layers.0.ln_ff.weight"], 1e-6)
        x = x + P.linear(P.silu_mul(P.linear(xn, w["model.layers.0.ffn.w1.weight"]),
                                    P.linear(xn, w["model.layers.0.ffn.w3.weight"])), w["model.layers.0.ffn.w2.weight"])
        return P.linear(P.rmsnorm(x, w["model.norm.weight"], 1e-6), w["model.embed_tokens.weight"])

    for rnd_i in range(2):   # the second round meets the slots (and their state) of the first again
        a, b = prompt(10 + rnd_i, 9, V), prompt(20 + rnd_i, 15, V)
        sa, sb = eng.new_sequence(), eng.new_sequence()
        out = eng.step([StepEntry(sa, a[:5], [4]), StepEntry(sb, b[:11], [0, 10])]).cpu().double()
        got_a, got_b = [out[0]], [out[2]]
        assert (out[1] - plain(b)[0]).abs().max() < 1e-4
        for t in range(4):
            out = eng.step([StepEntry(sa, [a[5 + t]], [0]), StepEntry(sb, [b[11 + t]], [0])]).cpu().double()
            got_a.append(out[0]); got_b.append(out[1])
        assert (torch.stack(got_a) - plain(a)[4:]).abs().max() < 1e-4
        assert (torch.stack(got_b) - plain(b)[10:]).abs().max() < 1e-4
        eng.release(sa); eng.release(sb)


def test_prompt_projection_fused_and_separate_agree(tmp_path, monkeypatch):
    """Long prompt pieces take the projection whose epilogue normalises, rotates and caches; shorter
    ones the plain product and the rotation kernel.  Same logits either way, and both are the plain
    implementation's."""
    from plain_qwen3 import PlainQwen3
    from rocml_b200 import Engine, StepEntry
    from rocml_b200.parts import attention as A
    from tiny_models import CONFIGS, prompt, write_model
    folder = str(tmp_path / "m")
    write_model(folder, CONFIGS["E"], seed=9, std=0.08)      # head size 128, a window on one layer
    plain = PlainQwen3(folder, dtype=torch.float32)
    ids = prompt(4, 600, CONFIGS["E"]["vocab_size"])
    want = plain.logits(ids)[[0, 299, 599]]
    got = {}
    for name, least in (("fused", 1), ("separate", 10 ** 9)):
        monkeypatch.setattr(A, "PROMPT_FUSED_MIN_TOKENS", least)
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024)
        s = eng.new_sequence()
        got[name] = eng.step([StepEntry(s, ids, [0, 299, 599])]).float().cpu()
        scale = want.abs().amax(-1, keepdim=True)
        assert float(((got[name] - want).abs() / scale).max()) < 2.5e-2
    assert float((got["fused"] - got["separate"]).abs().max() / want.abs().max()) < 2.5e-2


def test_a_toy_position_encoding_and_a_toy_routed_feed_forward_register_build_and_step():
    """Two more parts defined HERE: a position encoding (a stretched rotation of half of every head:
    another table behind the same interface, which the attention part's kernels then use) and a
    feed-forward with routing (a router picks one of three small experts per token).  A model of two
    layers built from them is stepped whole, token by token and two sequences at once, and equals
    the same arithmetic in float64."""
    from rocml_b200 import kernels
    from rocml_b200.config import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                   ScheduleEntry)
    from rocml_b200.engine import Engine, Model, StepEntry
    from rocml_b200.parts import FeedForward, PositionEncoding, register_feed_forward, register_position
    from rocml_b200.weights import TensorDecl
    from rocml_b200.weights.random_init import random_tensor

    @register_position("toy_stretched_rope")
    class StretchedRope(PositionEncoding):
        graph_safe = True

        def __init__(self, spec, head_dim, env):
            self.rot_dim = int(spec.rot_dim)
            self.stretch = float(spec.params["stretch"])
            i = torch.arange(self.rot_dim // 2, dtype=torch.float64)
            self.inv_freq = (torch.pow(torch.tensor(spec.theta, dtype=torch.float64), -2.0 * i / self.rot_dim)
                             / self.stretch).float().to(env.device)

        def cos_sin(self, batch):
            key = ("toy_stretched_rope", self.rot_dim, self.stretch)
            if key not in batch.scratch:
                batch.scratch[key] = kernels.rope_table(batch.positions, self.inv_freq, batch.n_tokens)
            return batch.scratch[key]

    @register_feed_forward("toy_top1_experts")
    class Top1Experts(FeedForward):
        graph_safe = False

        def __init__(self, spec, hidden, env):
            self.hidden, self.n, self.inner = hidden, spec.params["experts"], spec.params["intermediate"]

        def declare(self, prefix):
            out = [TensorDecl(f"{prefix}router.weight", (self.n, self.hidden))]
            for e in range(self.n):
                out += [TensorDecl(f"{prefix}experts.{e}.up.weight", (self.inner, self.hidden)),
                        TensorDecl(f"{prefix}experts.{e}.down.weight", (self.hidden, self.inner))]
            return out

        def load(self, tensors, prefix):
            self.router = tensors[f"{prefix}router.weight"].float()
            self.up = [tensors[f"{prefix}experts.{e}.up.weight"].float() for e in range(self.n)]
            self.down = [tensors[f"{prefix}experts.{e}.down.weight"].float() for e in range(self.n)]

        def forward(self, xn, batch):
            x = xn.float()
            p = torch.softmax(x @ self.router.t(), -1)               # router logits and softmax in 32-bit
            weight, choice = p.max(-1)
            out = torch.zeros((1, batch.n_tokens, self.hidden), dtype=torch.float32, device=x.device)
            for e in range(self.n):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    out[0, rows] = weight[rows, None] * (torch.relu(x[rows] @ self.up[e].t()) @ self.down[e].t())
            return out

    H, nq, nkv, hd, V, E, I, rot, theta, stretch = 40, 6, 2, 16, 83, 3, 24, 8, 1e4, 3.0
    norm = NormSpec("rmsnorm", 1e-5)
    pos = PositionSpec("toy_stretched_rope", theta=theta, rot_dim=rot, params_items=(("stretch", stretch),))
    att = MixerSpec.make("attention", position=pos, n_heads=nq, n_kv_heads=nkv, head_dim=hd, bias=False,
                         qk_norm=False, window=None, scale=None)
    ff = FeedForwardSpec.make("toy_top1_experts", experts=E, intermediate=I)
    layers = tuple(LayerSpec(f"model.layers.{i}", att, ff, norm, norm) for i in range(2))
    spec = ModelSpec("ToyRouted", H, V, 128, layers, (ScheduleEntry(0), ScheduleEntry(1)), norm, tie_embeddings=True)
    model = Model(spec, env(torch.float32))
    assert not model.graph_safe
    tensors = {d.name: random_tensor(d, 3).float() * (4.0 if d.role == "matrix" else 1.0) for d in model.declare()}
    model.load({k: v.to(DEV) for k, v in tensors.items()})
    eng = Engine(model, max_tokens=256, max_slots=2)
    w = {k: v.double() for k, v in tensors.items()}

    def rotate(x, T):
        half = rot // 2
        inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / rot)
        ang = torch.arange(T, dtype=torch.float64)[:, None] * (inv.float() / stretch).double()[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        x0, x1 = x[..., :half], x[..., half:rot]
        return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos, x[..., rot:]], -1)

    def plain(ids):
        T = len(ids)
        x = w["model.embed_tokens.weight"][ids]
        picks = []
        for i in range(2):
            p = f"model.layers.{i}."
            xn = P.rmsnorm(x, w[p + "input_layernorm.weight"], 1e-5)
            q = rotate(P.linear(xn, w[p + "self_attn.q_proj.weight"]).view(T, nq, hd), T)
            k = rotate(P.linear(xn, w[p + "self_attn.k_proj.weight"]).view(T, nkv, hd), T)
            v = P.linear(xn, w[p + "self_attn.v_proj.weight"]).view(T, nkv, hd)
            x = x + P.linear(P.attention(q, k, v).reshape(T, nq * hd), w[p + "self_attn.o_proj.weight"])
            xn = P.rmsnorm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
            pr = torch.softmax(xn @ w[p + "mlp.router.weight"].t(), -1)
            weight, choice = pr.max(-1)
            picks.append(choice)
            y = torch.stack([weight[t] * (torch.relu(xn[t] @ w[p + f"mlp.experts.{int(choice[t])}.up.weight"].t())
                                          @ w[p + f"mlp.experts.{int(choice[t])}.down.weight"].t()) for t in range(T)])
            x = x + y
        return P.linear(P.rmsnorm(x, w["model.norm.weight"], 1e-5), w["model.embed_tokens.weight"]), picks

    a, b = prompt(31, 30, V), prompt(32, 21, V)
    want_a, picks = plain(a)
    want_b, _ = plain(b)
    assert all(len(set(c.tolist())) > 1 for c in picks)            # the router does route
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([StepEntry(sa, a[:17], list(range(17))), StepEntry(sb, b[:9], [8])]).cpu().double()
    got_a, got_b = [out[:17]], [out[17:]]
    for t in range(12):
        out = eng.step([StepEntry(sa, [a[17 + t]], [0]), StepEntry(sb, [b[9 + t]], [0])]).cpu().double()
        got_a.append(out[:1]); got_b.append(out[1:])
    out = eng.step([StepEntry(sa, [a[29]], [0])]).cpu().double()      # the shorter one has ended
    got_a.append(out)
    scale = want_a.abs().max()
    assert (torch.cat(got_a) - want_a).abs().max() < 1e-4 * scale
    assert (torch.cat(got_b) - want_b[8:]).abs().max() < 1e-4 * scale


def test_a_toy_arrangement_and_a_toy_norm_register_build_and_step():
    """Another arrangement of a layer (mixer and feed-forward side by side on ONE norm's output, both added
    to the residual) and another norm (mean-centred, with a bias), both defined HERE, registered, and put
    around the library's own attention and gated feed-forward.  The engine steps them: whole prompts,
    pieces of a prompt, single tokens, two sequences at once.  Nothing in the library's files changes."""
    from rocml_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry
    from rocml_b200.engine import Engine, Model, StepEntry
    from rocml_b200.parts import Norm, build_feed_forward, build_mixer, build_norm, register_arrangement, register_norm
    from rocml_b200.weights import TensorDecl
    from rocml_b200.weights.random_init import random_tensor

    @register_norm("toy_layernorm")
    class ToyLayerNorm(Norm):
        graph_safe = True          # torch kernels on the current stream only

        def __init__(self, spec, size, env):
            self.size, self.eps = size, float(spec.eps)

        def declare(self, prefix):
            return [TensorDecl(f"{prefix}.weight", (self.size,), "norm"), TensorDecl(f"{prefix}.bias", (self.size,), "bias")]

        def load(self, tensors, prefix):
            self.w, self.b = tensors[f"{prefix}.weight"].float(), tensors[f"{prefix}.bias"].float()

        def weight_bytes(self):
            return 8 * self.size

        def forward(self, resid, delta, n_rows=None, rows=None, write_back=True):
            n = resid.shape[0] if n_rows is None else n_rows
            if delta is not None:
                resid[:delta.shape[1]] += delta.sum(0)              # the partial sums of the parts before
            x = resid[:n] if rows is None else resid[rows[:n].long()]
            mu = x.mean(-1, keepdim=True)
            return (x - mu) * torch.rsqrt(((x - mu) ** 2).mean(-1, keepdim=True) + self.eps) * self.w + self.b

    @register_arrangement("toy_parallel")
    class ParallelBlock:
        """x += mixer(norm(x)) + ff(norm(x)): the two results travel on as partial sums of one delta."""

        def __init__(self, spec, hidden, env, mixer_spec=None):
            self.spec = spec
            self.norm = build_norm(spec.mixer_norm, hidden, env)
            self.mixer = build_mixer(mixer_spec or spec.mixer, hidden, env)
            self.ff = build_feed_forward(spec.feed_forward, hidden, env)

        def _names(self):
            p, s = self.spec.prefix, self.spec
            return f"{p}.{s.mixer_norm_name}", f"{p}.{s.mixer_name}", f"{p}.{s.ff_name}"

        def declare(self):
            n, mx, ff = self._names()
            return self.norm.declare(n) + self.mixer.declare(mx) + self.ff.declare(ff)

        def load(self, tensors):
            n, mx, ff = self._names()
            self.norm.load(tensors, n); self.mixer.load(tensors, mx); self.ff.load(tensors, ff)

        graph_safe = property(lambda self: self.norm.graph_safe and self.mixer.graph_safe and self.ff.graph_safe)

        def weight_bytes(self):
            return self.norm.weight_bytes() + self.mixer.weight_bytes() + self.ff.weight_bytes()

        def forward(self, resid, pending, batch, view):
            xn = self.norm.forward(resid, pending, batch.n_tokens)
            return torch.cat([self.mixer.forward(xn, batch, view), self.ff.forward(xn, batch)], dim=0)

    H, V, nq, nkv, hd, inter = 40, 91, 3, 1, 16, 56
    norm = NormSpec("toy_layernorm", 1e-4)
    att = MixerSpec.make("attention", position=PositionSpec("rope_neox", theta=1e4), n_heads=nq, n_kv_heads=nkv, head_dim=hd)
    ff = FeedForwardSpec.make("gated_mlp", intermediate=inter)
    layers = tuple(LayerSpec(f"h.{i}", att, ff, norm, norm, arrangement="toy_parallel", mixer_norm_name="ln",
                             mixer_name="attn.", ff_name="mlp.") for i in range(2))
    spec = ModelSpec("ToyParallel", H, V, 256, layers, (ScheduleEntry(0), ScheduleEntry(1)), norm, tie_embeddings=False,
                     embedding_name="wte.weight", final_norm_name="ln_f.weight", head_name="head.weight")
    model = Model(spec, env(torch.float32))
    tensors = {d.name: random_tensor(d, 9).float() * (3.0 if d.role == "matrix" else 1.0) for d in model.declare()}
    assert "h.1.ln.bias" in tensors and "ln_f.bias" in tensors and "h.0.attn.q_proj.weight" in tensors
    assert not any("post_attention" in k for k in tensors)
    model.load({k: v.to(DEV) for k, v in tensors.items()})
    eng = Engine(model, max_tokens=512, max_slots=2, max_step_tokens=16)
    w = {k: v.double() for k, v in tensors.items()}

    def ln(x, p):
        mu = x.mean(-1, keepdim=True)
        return (x - mu) * torch.rsqrt(((x - mu) ** 2).mean(-1, keepdim=True) + 1e-4) * w[p + ".weight"] + w[p + ".bias"]

    def plain(ids):
        T = len(ids)
        x = w["wte.weight"][ids]
        for i in range(2):
            p = f"h.{i}."
            xn = ln(x, p + "ln")
            q = P.rope_neox(P.linear(xn, w[p + "attn.q_proj.weight"]).view(T, nq, hd), range(T), 1e4)
            k = P.rope_neox(P.linear(xn, w[p + "attn.k_proj.weight"]).view(T, nkv, hd), range(T), 1e4)
            v = P.linear(xn, w[p + "attn.v_proj.weight"]).view(T, nkv, hd)
            a = P.linear(P.attention(q, k, v).reshape(T, nq * hd), w[p + "attn.o_proj.weight"])
            m = P.linear(P.silu_mul(P.linear(xn, w[p + "mlp.gate_proj.weight"]), P.linear(xn, w[p + "mlp.up_proj.weight"])),
                         w[p + "mlp.down_proj.weight"])
            x = x + a + m
        return P.linear(ln(x, "ln_f"), w["head.weight"])

    a, b = prompt(1, 50, V), prompt(2, 23, V)
    wa, wb = plain(a), plain(b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    # prompts of 44 and 20 tokens in one step: four pieces of 16 tokens, the second sequence beside the end of the first
    out = eng.step([StepEntry(sa, a[:44], [0, 15, 16, 43]), StepEntry(sb, b[:20], [19])]).cpu().double()
    scale = wa.abs().max()
    assert (out[:4] - wa[[0, 15, 16, 43]]).abs().max() < 2e-5 * scale
    assert (out[4] - wb[19]).abs().max() < 2e-5 * scale
    for t in range(3):
        out = eng.step([StepEntry(sa, [a[44 + t]], [0]), StepEntry(sb, [b[20 + t]], [0])]).cpu().double()
        assert (out[0] - wa[44 + t]).abs().max() < 2e-5 * scale and (out[1] - wb[20 + t]).abs().max() < 2e-5 * scale
    eng.release(sa); eng.release(sb)
    eng.cache.check_invariants()
