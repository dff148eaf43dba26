"""Weights: the safetensors reader and writer, the loader's one error, precision policy, random mode."""
import json
import os
import struct

import pytest
import torch

import plain_llama as plain
from llm_infer_engine_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, build_model, compare,
                                           open_model_files, save_file, target_dtype, write_random_model)


def test_round_trip_against_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file as st_save
    g = torch.Generator().manual_seed(0)
    tensors = {"a.weight": torch.randn(5, 7, generator=g), "b": torch.randn(3, generator=g).to(torch.bfloat16),
               "ids": torch.arange(6, dtype=torch.int64).view(2, 3), "empty": torch.zeros(0, 4),
               "h": torch.randn(4, 4, generator=g).to(torch.float16)}
    ours = str(tmp_path / "ours.safetensors")
    save_file(tensors, ours, metadata={"format": "pt"})
    theirs = load_file(ours)                                  # the package reads what we wrote
    for k, v in tensors.items():
        assert theirs[k].dtype == v.dtype and torch.equal(theirs[k], v)
    pkg = str(tmp_path / "pkg.safetensors")
    st_save(tensors, pkg)
    f = SafetensorsFile(pkg)                                  # we read what the package wrote
    assert sorted(f.names()) == sorted(tensors)
    for k, v in tensors.items():
        assert f.entries[k] == (v.dtype, tuple(v.shape)) and torch.equal(f.tensor(k), v)


def _write_raw(path, header: dict, data: bytes):
    raw = json.dumps(header).encode()
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(raw)) + raw + data)


def test_header_errors(tmp_path):
    p = str(tmp_path / "x.safetensors")
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    _write_raw(p, {"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}, b"\0" * 8)   # truncated
    with pytest.raises(SafetensorsError, match="outside the data"):
        SafetensorsFile(p)
    _write_raw(p, {"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}, b"\0" * 16)  # size mismatch
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(p)
    _write_raw(p, {"w": {"dtype": "F8_E4M3", "shape": [2], "data_offsets": [0, 2]}}, b"\0" * 2)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(p)
    raw = b'{"w":{"dtype":"U8","shape":[1],"data_offsets":[0,1]},"w":{"dtype":"U8","shape":[1],"data_offsets":[0,1]}}'
    open(p, "wb").write(struct.pack("<Q", len(raw)) + raw + b"\0")
    with pytest.raises(SafetensorsError, match="duplicate"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        open_model_files(str(tmp_path / "nowhere"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = str(tmp_path / "m")
    write_random_model(plain.TINY_A, folder, seed=0)
    from safetensors.torch import load_file, save_file as st_save
    t = load_file(os.path.join(folder, "model.safetensors"))
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63, dtype=torch.bfloat16)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)          # ignored by the architecture
    t["lm_head.weight"] = torch.zeros(256, 32, dtype=torch.bfloat16)            # tied model, and not the embedding's shape
    t["something.else"] = torch.zeros(1)
    st_save(t, os.path.join(folder, "model.safetensors"))
    with pytest.raises(WeightsError) as info:
        build_model(folder, torch.float32, "cpu")
    e = info.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["lm_head.weight", "something.else"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    text = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (1)", "expected (64, 64), file has (64, 63)"):
        assert needle in text
    compare({"a": (1,)}, {"a": (1,), "skip.me": (2,)}, [r"skip\..*"], "x")        # ignore patterns


def test_tied_checkpoint_that_also_stores_the_head_is_accepted(tmp_path, capsys):
    """Some exporters write lm_head.weight beside a tied embedding. With the embedding's shape it is
    skipped and reported (the reference reports and goes on, src/loader.py:147-151)."""
    folder = str(tmp_path / "m")
    write_random_model(plain.TINY_A, folder, seed=0)
    from safetensors.torch import load_file, save_file as st_save
    t = load_file(os.path.join(folder, "model.safetensors"))
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    st_save(t, os.path.join(folder, "model.safetensors"))
    model, _ = build_model(folder, torch.float32, "cpu")
    assert model.load_report["skipped"] == ["lm_head.weight"]
    assert model.head.weight.data_ptr() == model.embedding.data_ptr()
    assert "lm_head.weight is not read" in capsys.readouterr().err


def test_precision_policy():
    bf, f32 = torch.bfloat16, torch.float32
    assert target_dtype(bf, bf) == bf and target_dtype(torch.float16, bf) == bf
    assert target_dtype(bf, f32) == f32
    assert target_dtype(f32, bf) == f32 and target_dtype(f32, f32) == f32         # stored in 32-bit: stays so
    assert target_dtype(torch.int64, bf) == torch.int32 and target_dtype(torch.uint8, f32) == torch.int32


def test_random_mode_writes_a_loadable_folder(tmp_path):
    a1 = write_random_model(plain.TINY_B, str(tmp_path / "a1"), seed=5, std=0.03, norm_range=(0.8, 1.2))
    a2 = write_random_model(plain.TINY_B, str(tmp_path / "a2"), seed=5, std=0.03, norm_range=(0.8, 1.2))
    b = write_random_model(plain.TINY_B, str(tmp_path / "b"), seed=6, std=0.03, norm_range=(0.8, 1.2))
    f1, f2, fb = (open_model_files(x) for x in (a1, a2, b))
    assert set(f1) == set(plain.tensor_shapes(plain.TINY_B))
    for name, shape in plain.tensor_shapes(plain.TINY_B).items():
        t1 = f1[name].tensor(name)
        assert tuple(t1.shape) == shape and t1.dtype == torch.bfloat16
        assert torch.equal(t1, f2[name].tensor(name))                      # same seed, same values
        assert not torch.equal(t1, fb[name].tensor(name))                  # another seed, other values
    w = f1["model.layers.0.mlp.gate_proj.weight"].tensor("model.layers.0.mlp.gate_proj.weight").float()
    assert 0.025 < float(w.std()) < 0.035
    n = f1["model.norm.weight"].tensor("model.norm.weight").float()
    assert 0.8 <= float(n.min()) and float(n.max()) <= 1.2 and float(n.std()) > 0.05
    assert json.load(open(os.path.join(a1, "config.json")))["torch_dtype"] == "bfloat16"
    # tied model: no separate head is written; float32 storage on request
    c = write_random_model(plain.TINY_A, str(tmp_path / "c"), seed=0, dtype="float32")
    fc = open_model_files(c)
    assert "lm_head.weight" not in fc
    assert fc["model.norm.weight"].tensor("model.norm.weight").dtype == torch.float32
    assert torch.equal(fc["model.norm.weight"].tensor("model.norm.weight"), torch.ones(64))
    # the loader keeps 32-bit tensors 32-bit even for a bfloat16 engine, and shares a tied head
    model, cfg = build_model(c, torch.bfloat16, "cpu")
    assert model.embedding.dtype == torch.float32 and model.head.weight.data_ptr() == model.embedding.data_ptr()
    model, cfg = build_model(a1, torch.bfloat16, "cpu")
    assert model.embedding.dtype == torch.bfloat16 and model.blocks[0].mixer.qkv.weight.shape == (96 + 2 * 32, 96)
    model, cfg = build_model(a1, torch.float32, "cpu")
    assert model.embedding.dtype == torch.float32
    assert model.weight_bytes_per_step() > 0
