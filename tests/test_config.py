"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from rocml_b200.config import (CATALOG, Qwen3Config, config_from_dict, load_config, load_model_spec,
                               register_architecture, registered_architectures, resolve)
from rocml_b200.errors import ConfigError, ModelFileMissing, UnknownModel, UnsupportedArchitecture
from tiny_models import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_the_keys():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (96, 208, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (6, 1, 32)
    assert c.q_dim == 192 and c.kv_dim == 32 and c.kv_group_size == 6
    assert c.vocab_size == 311 and c.max_position_embeddings == 256
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5
    assert c.attention_bias and not c.tie_word_embeddings
    assert c.eos_token_ids == (5, 9)


def test_head_dim_defaults_to_hidden_over_heads():
    d = dict(TINY_A)
    del d["head_dim"]
    assert Qwen3Config.from_dict(d).head_dim == 16


def test_round_trip_through_config_json(tmp_path):
    for d in (TINY_A, TINY_B, TINY_C):
        c = Qwen3Config.from_dict(d)
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        c2, _ = load_config(str(tmp_path))
        assert c2 == c


@pytest.mark.parametrize("key,value,needle", [
    ("num_attention_heads", 5, "multiple"), ("head_dim", 15, "even"), ("hidden_size", 0, "positive"),
    ("hidden_act", "gelu", "hidden_act"), ("rope_scaling", {"rope_type": "yarn", "factor": 4.0}, "rope_scaling"),
    ("rms_norm_eps", 0.0, "rms_norm_eps"), ("vocab_size", "many", "integer"),
])
def test_rejections(key, value, needle):
    d = dict(TINY_A)
    d[key] = value
    with pytest.raises(ConfigError, match=needle):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "rope_theta",
                                 "rms_norm_eps", "vocab_size", "max_position_embeddings"])
def test_missing_keys_are_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


def test_windows_per_layer():
    c = Qwen3Config.from_dict(TINY_C)
    assert c.layer_windows == (None, 24, None, 24)
    d = dict(TINY_A, use_sliding_window=True, sliding_window=8, max_window_layers=1)
    assert Qwen3Config.from_dict(d).layer_windows == (None, 8)
    spec = c.to_model_spec()
    assert [l.mixer.params["window"] for l in spec.layers] == [None, 24, None, 24]


def test_model_spec_is_data():
    spec = Qwen3Config.from_dict(TINY_B).to_model_spec()
    assert spec.hidden == 96 and spec.vocab == 311 and len(spec.layers) == 3
    assert [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[0].mixer
    assert m.kind == "attention" and m.params["n_kv_heads"] == 1 and m.position.theta == 1e6
    assert spec.layers[0].feed_forward.params["intermediate"] == 208
    assert spec.final_norm.eps == 1e-5 and spec.stop_tokens == (5, 9)


def test_registry_by_architecture():
    assert "Qwen3ForCausalLM" in registered_architectures()
    with pytest.raises(UnsupportedArchitecture, match="Qwen3ForCausalLM"):
        config_from_dict({"architectures": ["LlamaForCausalLM"]})
    register_architecture("ToyForTests", Qwen3Config.from_dict)
    d = dict(TINY_A, architectures=["ToyForTests"])
    with pytest.raises(ConfigError):  # the Qwen3 class itself insists on its own name
        config_from_dict(d)


def test_resolve_names_and_paths(tmp_path, monkeypatch):
    with pytest.raises(UnknownModel, match="qwen3-8b"):
        resolve("no-such-model")
    monkeypatch.setenv("ROCML_CHECKPOINT_DIR", str(tmp_path))
    with pytest.raises(ModelFileMissing, match="--random"):
        resolve("qwen3-8b")
    r = resolve("qwen3-8b", must_exist=False)
    assert r.entry.default_ctx == 4096 and r.entry.sampling.top_k == 20 and r.entry.sampling.top_p == 0.95
    os.makedirs(tmp_path / "Qwen3-8B")
    (tmp_path / "Qwen3-8B" / "config.json").write_text(json.dumps(CATALOG["qwen3-8b"].config))
    assert resolve("qwen3-8b").path == str(tmp_path / "Qwen3-8B")
    p = resolve(str(tmp_path / "Qwen3-8B"))
    assert p.entry is None  # a path brings no defaults
    assert load_model_spec(p.path).hidden == 4096


def test_generation_config_adds_stop_tokens(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 11]}))
    assert load_model_spec(str(tmp_path)).stop_tokens == (7, 11)


def test_tensor_names_come_from_the_spec():
    """The parts name their tensors by role; the stems and the four prefixes of a layer are the spec's.
    The defaults are the names of Qwen3's checkpoints; another architecture gives its own."""
    import torch
    from rocml_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry
    from rocml_b200.engine.model import declared_tensors
    from rocml_b200.errors import ConfigError
    norm = NormSpec("rmsnorm", 1e-5)
    att = MixerSpec.make("attention", position=PositionSpec("none"), n_heads=2, n_kv_heads=1, head_dim=16, qk_norm=True,
                         names={"q": "wq", "k": "wk", "v": "wv", "o": "wo", "q_norm": "qn"})
    ff = FeedForwardSpec.make("gated_mlp", intermediate=32, names={"gate": "w1", "up": "w3", "down": "w2"})
    layer = LayerSpec("blk.0", att, ff, norm, norm, mixer_norm_name="attn_norm", mixer_name="attn.",
                      ff_norm_name="ffn_norm", ff_name="ffn.")
    spec = ModelSpec("Other", 24, 50, 64, (layer,), (ScheduleEntry(0),), norm, tie_embeddings=False,
                     embedding_name="tok.weight", final_norm_name="out_norm.weight", head_name="out.weight")
    got = sorted(d.name for d in declared_tensors(spec))
    assert got == sorted([
        "tok.weight", "out_norm.weight", "out.weight", "blk.0.attn_norm.weight", "blk.0.ffn_norm.weight",
        "blk.0.attn.wq.weight", "blk.0.attn.wk.weight", "blk.0.attn.wv.weight", "blk.0.attn.wo.weight",
        "blk.0.attn.qn.weight", "blk.0.attn.k_norm.weight",
        "blk.0.ffn.w1.weight", "blk.0.ffn.w3.weight", "blk.0.ffn.w2.weight"])
    hash(att), hash(layer)        # specs stay hashable with a names map inside
    bad = MixerSpec.make("attention", n_heads=2, n_kv_heads=1, head_dim=16, names={"query": "wq"})
    with pytest.raises(ConfigError, match="query"):
        declared_tensors(ModelSpec("Other", 24, 50, 64, (LayerSpec("blk.0", bad, ff, norm, norm),), (ScheduleEntry(0),),
                                   norm, tie_embeddings=True))
