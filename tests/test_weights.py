"""Safetensors reading and writing, loading by name, the one error that lists everything (no GPU)."""
import json
import os
import struct

import pytest
import torch

from rocml_b200.config import config_from_dict
from rocml_b200.engine import declared_tensors
from rocml_b200.errors import ModelFileMissing, SafetensorsError, WeightsError
from rocml_b200.weights import (ModelFiles, NativeReader, SafetensorsFile, load_tensors, save_state_dict, storage_dtype,
                                write_random_model)
from tiny_models import TINY_A, TINY_B


def test_round_trip_and_interop_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    state = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(2, 2)}
    p = str(tmp_path / "x.safetensors")
    save_state_dict(p, state, {"k": "v"})
    theirs = load_file(p)
    with SafetensorsFile(p) as f:
        assert f.metadata == {"k": "v"}
        for k, v in state.items():
            assert torch.equal(f.tensor(k), v) and torch.equal(theirs[k], v)
    save_file(state, p)
    with SafetensorsFile(p) as f:
        assert all(torch.equal(f.tensor(k), v) for k, v in state.items())


def test_truncated_and_malformed_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    save_state_dict(p, {"a": torch.zeros(100)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-8])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(raw[:4])
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    with pytest.raises(ModelFileMissing):
        ModelFiles(str(tmp_path / "nowhere"))


def test_random_model_is_deterministic_and_distributed_as_stated(tmp_path):
    cfg = config_from_dict(TINY_B)
    a = write_random_model(str(tmp_path / "a"), cfg, seed=5)
    b = write_random_model(str(tmp_path / "b"), cfg, seed=5)
    c = write_random_model(str(tmp_path / "c"), cfg, seed=6)
    fa, fb, fc = (ModelFiles(x) for x in (a, b, c))
    names = sorted(fa.names())
    assert names == sorted(d.name for d in declared_tensors(cfg.to_model_spec()))
    assert all(torch.equal(fa.tensor(n), fb.tensor(n)) for n in names)
    assert not torch.equal(fa.tensor(names[0]), fc.tensor(names[0]))
    w = fa.tensor("model.layers.0.mlp.gate_proj.weight").float()
    assert w.dtype == torch.float32 and abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = fa.tensor("model.norm.weight").float()
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15
    assert fa.tensor("model.layers.1.self_attn.q_proj.bias").shape == (192,)
    assert json.load(open(os.path.join(a, "config.json")))["num_key_value_heads"] == 1


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from safetensors.torch import load_file, save_file
    cfg = config_from_dict(TINY_A)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=1)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    w["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    save_file(w, path)
    decls = declared_tensors(cfg.to_model_spec())
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, decls, "bfloat16", "cpu")
    err = e.value
    assert err.missing == ("model.layers.1.mlp.up_proj.weight", "model.norm.weight")
    assert err.unexpected == ("model.layers.0.self_attn.rotary_emb.inv_freq",)
    assert err.wrong_shape == (("model.layers.0.self_attn.k_proj.weight", (32, 64), (16, 64)),)
    for needle in ("up_proj", "rotary_emb", "expected [32, 64], found [16, 64]"):
        assert needle in str(err)


def test_tied_head_may_be_present_and_is_ignored(tmp_path):
    from safetensors.torch import load_file, save_file
    cfg = config_from_dict(TINY_A)  # tied
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=1)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    save_file(w, path)
    decls = declared_tensors(cfg.to_model_spec())
    with pytest.raises(WeightsError):
        load_tensors(folder, decls, "bfloat16", "cpu", strict=True)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("error")              # ignorable: not even a warning
        out = load_tensors(folder, decls, "bfloat16", "cpu", ignorable=["lm_head.weight"], strict=True)
    assert "lm_head.weight" not in out


def test_extra_tensors_alone_are_a_warning_that_names_them(tmp_path):
    """A checkpoint with tensors the model does not read (a rotary table, say) loads, with one warning;
    strict loading refuses it; and a folder that also lacks a tensor is refused with both listed."""
    from safetensors.torch import load_file, save_file
    from rocml_b200.weights.loader import UnexpectedTensors
    cfg = config_from_dict(TINY_A)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=1)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    save_file(w, path)
    decls = declared_tensors(cfg.to_model_spec())
    with pytest.warns(UnexpectedTensors, match="rotary_emb.inv_freq"):
        out = load_tensors(folder, decls, "bfloat16", "cpu")
    assert "model.layers.0.self_attn.rotary_emb.inv_freq" not in out and len(out) == len(decls)
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, decls, "bfloat16", "cpu", strict=True)
    assert e.value.unexpected == ("model.layers.0.self_attn.rotary_emb.inv_freq",) and not e.value.missing


def test_storage_rule():
    assert storage_dtype(torch.bfloat16, "bfloat16", "matrix") == torch.bfloat16
    assert storage_dtype(torch.float16, "bfloat16", "matrix") == torch.bfloat16
    assert storage_dtype(torch.float32, "bfloat16", "norm") == torch.float32   # stored in 32-bit: stays
    assert storage_dtype(torch.bfloat16, "float32", "matrix") == torch.float32
    assert storage_dtype(torch.int64, "bfloat16", "int_table") == torch.int32


def test_sharded_folder(tmp_path):
    from safetensors.torch import save_file
    a = {"x": torch.ones(2), "y": torch.zeros(3)}
    save_file({"x": a["x"]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({"y": a["y"]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        "x": "model-00001-of-00002.safetensors", "y": "model-00002-of-00002.safetensors"}}))
    with ModelFiles(str(tmp_path)) as f:
        assert sorted(f.names()) == ["x", "y"] and torch.equal(f.tensor("y"), a["y"])


def _needs_library():
    """The reader below is part of the kernel library, which nvcc builds at first use (it needs no GPU)."""
    from rocml_b200.csrc.build import library
    from rocml_b200.errors import ExtensionMissing
    try:
        library()
    except ExtensionMissing as e:
        pytest.skip(f"the kernel library cannot be built here: {str(e)[:80]}")


def test_the_library_reader_agrees_with_the_python_reader(tmp_path):
    """The reader inside the kernel library (C++: header parsed and checked there, bytes copied by it) lists the
    same tensors and hands out the same bytes; names with escapes and other alphabets, metadata, an empty
    tensor and every stored type the loader takes."""
    state = {"a.weight": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int64),
             'émb "q" \\ \n': torch.randn(2, 2, 2), "empty": torch.zeros(0, 4), "h": torch.randn(9).half(),
             "i8": torch.arange(-3, 3, dtype=torch.int8), "flag": torch.tensor([True, False])}
    p = str(tmp_path / "x.safetensors")
    save_state_dict(p, state, {"format": "pt", "note": "two\nlines \u00e9"})
    with SafetensorsFile(p) as f, NativeReader(p) as r:
        assert r.metadata == f.metadata
        assert set(r.entries) == set(f.names())
        for k, v in state.items():
            _, dtype, shape, nbytes = r.entries[k]
            assert shape == tuple(v.shape) and nbytes == v.numel() * v.element_size()
            dst = torch.empty_like(v)
            r.read(k, dst, nbytes)
            assert torch.equal(dst, v) and torch.equal(dst, f.tensor(k))
        with pytest.raises(SafetensorsError, match="bytes"):
            r.read("b", torch.empty(3, dtype=torch.int64), 24)


def test_the_library_reader_refuses_what_the_python_reader_refuses(tmp_path):
    _needs_library()
    p = str(tmp_path / "x.safetensors")
    save_state_dict(p, {"a": torch.zeros(100)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-8])
    with pytest.raises(SafetensorsError, match="truncated"):
        NativeReader(p)
    open(p, "wb").write(raw[:4])
    with pytest.raises(SafetensorsError, match="too short"):
        NativeReader(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="not valid"):
        NativeReader(p)
    with pytest.raises(SafetensorsError, match="cannot open"):
        NativeReader(str(tmp_path / "nowhere.safetensors"))

    def with_header(header, data=b""):
        blob = json.dumps(header).encode()
        open(p, "wb").write(struct.pack("<Q", len(blob)) + blob + data)
    with_header({"a": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 20]}}, b"\0" * 24)
    with pytest.raises(SafetensorsError, match="shape needs 24"):
        NativeReader(p)
    with_header({"a": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 2]}}, b"\0" * 2)
    with pytest.raises(SafetensorsError, match="unknown element type"):
        NativeReader(p)
    with_header({"a": {"dtype": "F32", "shape": [2]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="lacks"):
        NativeReader(p)
    with_header({"a": {"dtype": "F32", "shape": [1.5], "data_offsets": [0, 4]}}, b"\0" * 4)
    with pytest.raises(SafetensorsError, match="integer"):
        NativeReader(p)
    with_header([1, 2, 3])
    with pytest.raises(SafetensorsError, match="not a JSON object"):
        NativeReader(p)
    # keys the format does not know are skipped, whatever their values
    with_header({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4], "extra": {"x": [1, 2.5, None, True, "s"]}}}, b"\0" * 4)
    with NativeReader(p) as r:
        assert r.entries["a"][1:] == ("F32", (1,), 4)
