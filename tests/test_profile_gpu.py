"""A profiled run on the GPU: every kernel of a step is timed, the times add up to the step's own,
and profiling changes no result."""
import pytest
import torch

pytestmark = pytest.mark.gpu

# Large enough that kernels, not the events between them, make the step's time; two layers of it.
CFG = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 2048, "intermediate_size": 6144, "num_hidden_layers": 2,
    "num_attention_heads": 16, "num_key_value_heads": 4, "head_dim": 128, "vocab_size": 32000,
    "max_position_embeddings": 4096, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "attention_bias": False, "hidden_act": "silu",
}


def engine(dtype):
    from rocml_b200 import Engine
    from rocml_b200.config import config_from_dict
    from rocml_b200.engine.model import Model
    from rocml_b200.parts import BuildEnv
    dev = torch.device("cuda:0")
    m = Model(config_from_dict(CFG).to_model_spec(), BuildEnv(dev, torch.float32 if dtype == "float32" else torch.bfloat16))
    m.load_random(3)
    return Engine(m, max_tokens=8 * 2048, max_slots=8)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_kernel_times_add_up_to_the_step_and_nothing_changes(dtype):
    from rocml_b200 import StepEntry
    from rocml_b200.profile import Profiler, to_human
    eng = engine(dtype)
    g = torch.Generator().manual_seed(1)
    n_prompt = 1024 if dtype == "bfloat16" else 256
    prompts = [torch.randint(0, CFG["vocab_size"], (n_prompt + 4,), generator=g).tolist() for _ in range(8)]

    def run():
        slots = [eng.new_sequence() for _ in prompts]
        outs = [eng.step([StepEntry(s, p[:n_prompt], [n_prompt - 1]) for s, p in zip(slots, prompts)]).clone()]
        for t in range(4):
            outs.append(eng.step([StepEntry(s, [p[n_prompt + t]], [0]) for s, p in zip(slots, prompts)]).clone())
        for s in slots:
            eng.release(s)
        return torch.cat(outs)

    plain = run()                 # warm: loads every kernel, captures the decode graphs
    with Profiler(eng.device, dtype=dtype) as prof:
        profiled = run()
    again = run()
    rep = prof.report()
    scale = plain.abs().amax(dim=-1, keepdim=True)
    tol = 1e-5 if dtype == "float32" else 2.5e-2    # a profiled decode step runs eagerly, a served one from a graph: the same kernels
    assert float(((profiled - plain).abs() / scale).max()) < tol
    assert torch.equal(plain, again)
    phases = {p["phase"]: p for p in rep["phases"]}
    assert set(phases) == {"prefill", "decode"}
    # the engine's work space holds 4,096 tokens: the bfloat16 run's prompts go in two pieces
    assert phases["prefill"]["steps"] == -(-8 * n_prompt // 4096) and phases["prefill"]["tokens"] == 8 * n_prompt
    assert phases["decode"]["steps"] == 4 and phases["decode"]["tokens"] == 32
    for ph in phases.values():
        assert ph["ops_ms"] <= ph["step_ms"] * 1.001
        assert ph["ops_ms"] >= 0.9 * ph["step_ms"], (ph["phase"], ph["ops_ms"], ph["step_ms"], to_human(rep))
        labels = {r["label"] for r in ph["by_op"]}
        assert {"embedding", "mixer_norm", "o_proj", "down_proj", "lm_head"} <= labels
        assert any("q_proj" in x for x in labels) and any("attention" in x for x in labels)
        assert {r["label"] for r in ph["by_layer"]} == {"layer 0", "layer 1", "(outside the layers)"}
        for r in ph["by_op"]:
            assert r["elapsed_ms"] > 0 and r["bytes"] > 0
            assert r["efficiency"] < 1.3, (r["label"], r)        # nothing beats its bound by more than the limits' own slack
    # the products of the prompt are bound by arithmetic, the decode step's by the weights' bytes
    pre = {r["label"]: r for r in phases["prefill"]["by_op"]}
    dec = {r["label"]: r for r in phases["decode"]["by_op"]}
    assert dec["down_proj"]["bound"] == "hbm" and dec["lm_head"]["bound"] == "hbm"
    if dtype == "bfloat16":
        assert pre["down_proj"]["bound"] == "flops" and pre["down_proj"]["frac_of_flops"] > 0.2
        assert dec["lm_head"]["frac_of_bandwidth"] > 0.3
    # the whole step's bytes are what the model says a step has to read
    want_bytes, _ = eng.model.step_cost([1] * 8, [n_prompt + 2] * 8, 8)
    got = phases["decode"]["total"]["bytes"] / 4
    assert 0.9 * want_bytes < got < 1.6 * want_bytes         # kernels also move activations and partial sums
