"""Safetensors reading and writing, binding by name, weight errors, random weights (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from gemmars_b200.engine.model import DecoderModel
from gemmars_b200.models.qwen3 import Qwen3Config, build_plan, checkpoint_layout
from gemmars_b200.weights import (ModelFiles, WeightError, WeightFileError, check_checkpoint, load_checkpoint,
                                  random_weights, write_random_model, write_safetensors)
from tiny_configs import TINY_A, TINY_B


def _write_by_hand(path, entries):
    """A minimal safetensors file written without the package (cf. src/safetensors.rs:1204-1223)."""
    header, blobs, off = {}, [], 0
    for name, (dtype, shape, raw) in entries.items():
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def test_hand_written_file_reads_back(tmp_path):
    f32 = np.arange(6, dtype="<f4").reshape(2, 3)
    bf = (np.array([1.0, -2.5, 3.0, 0.15625], dtype="<f4").view("<u4") >> 16).astype("<u2")
    f16 = np.array([0.5, 1.5], dtype="<f2")
    i64 = np.array([3, -1, 7], dtype="<i8")
    _write_by_hand(tmp_path / "model.safetensors", {
        "a": ("F32", [2, 3], f32.tobytes()), "b": ("BF16", [4], bf.tobytes()),
        "c": ("F16", [2], f16.tobytes()), "d": ("I64", [3], i64.tobytes())})
    files = ModelFiles(str(tmp_path))
    assert files.names() == {"a", "b", "c", "d"}
    got = load_checkpoint(files, {"a": (2, 3), "b": (4,), "c": (2,), "d": (3,)})
    assert got["a"].dtype == torch.float32 and torch.equal(got["a"], torch.from_numpy(f32.copy()))
    assert got["b"].dtype == torch.bfloat16 and got["b"].float().tolist() == [1.0, -2.5, 3.0, 0.15625]
    assert got["c"].dtype == torch.float32 and got["c"].tolist() == [0.5, 1.5]     # float16 widens exactly
    assert got["d"].dtype == torch.int32 and got["d"].tolist() == [3, -1, 7]      # integer tables: int32


def test_write_then_read_and_shards(tmp_path):
    t = {"x": torch.randn(5, 7).bfloat16(), "y": torch.arange(4, dtype=torch.float32)}
    os.makedirs(tmp_path / "one")
    write_safetensors(str(tmp_path / "one" / "model.safetensors"), t)
    f = ModelFiles(str(tmp_path / "one"))
    assert torch.equal(f.tensor("x"), t["x"]) and torch.equal(f.tensor("y"), t["y"])
    os.makedirs(tmp_path / "two")
    write_safetensors(str(tmp_path / "two" / "s1.safetensors"), {"x": t["x"]})
    write_safetensors(str(tmp_path / "two" / "s2.safetensors"), {"y": t["y"]})
    (tmp_path / "two" / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    f2 = ModelFiles(str(tmp_path / "two"))
    assert f2.info("x") == (torch.bfloat16, (5, 7)) and torch.equal(f2.tensor("y"), t["y"])


def test_file_errors(tmp_path):
    with pytest.raises(WeightFileError, match="no model.safetensors"):
        ModelFiles(str(tmp_path))
    p = tmp_path / "model.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightFileError, match="exceeds file"):
        ModelFiles(str(tmp_path))
    h = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 8)
    with pytest.raises(WeightFileError, match="out of bounds"):
        ModelFiles(str(tmp_path))


def test_one_error_lists_everything():
    cfg = Qwen3Config.from_dict(TINY_B)
    model = DecoderModel(build_plan(cfg), "float32", "cpu")
    expected = model.expected_tensors()
    assert set(expected) == set(checkpoint_layout(cfg))          # the parts want exactly the checkpoint
    have = {n: s for n, s in expected.items()}
    del have["model.layers.1.mlp.up_proj.weight"]
    del have["model.layers.0.self_attn.q_proj.bias"]
    have["model.layers.2.self_attn.k_norm.weight"] = (31,)
    have["model.norm.weight"] = (96, 1)
    have["model.layers.0.self_attn.rotary_emb.inv_freq"] = (16,)     # ignored by the plan
    have["model.layers.0.mlp.extra.weight"] = (3,)
    with pytest.raises(WeightError) as e:
        check_checkpoint(have, expected, model.plan.ignored_tensors)
    err = e.value
    assert err.missing == ["model.layers.0.self_attn.q_proj.bias", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.2.self_attn.k_norm.weight", "model.norm.weight"]
    msg = str(err)
    assert "missing tensor model.layers.1.mlp.up_proj.weight" in msg
    assert "tensor model.norm.weight has shape [96, 1], expected [96]" in msg
    assert "unexpected tensor model.layers.0.mlp.extra.weight" in msg


def test_tied_checkpoint_may_carry_a_head():
    cfg = Qwen3Config.from_dict(TINY_A)
    names = set(checkpoint_layout(cfg)) | {"lm_head.weight"}
    plan = build_plan(cfg, names)
    model = DecoderModel(plan, "float32", "cpu")
    have = {n: s for n, (s, _) in checkpoint_layout(cfg).items()}
    have["lm_head.weight"] = (512, 64)
    check_checkpoint(have, model.expected_tensors(), plan.ignored_tensors)


def test_random_weights_are_seeded_and_load(tmp_path):
    a = random_weights(TINY_A, seed=3)
    b = random_weights(TINY_A, seed=3)
    c = random_weights(TINY_A, seed=4)
    assert all(torch.equal(a[n], b[n]) for n in a) and any(not torch.equal(a[n], c[n]) for n in a)
    # a tensor's values do not depend on which other tensors exist
    bigger = random_weights(dict(TINY_A, num_hidden_layers=3), seed=3)
    assert torch.equal(a["model.layers.1.mlp.down_proj.weight"], bigger["model.layers.1.mlp.down_proj.weight"])
    w = a["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.004 and w.dtype == torch.float32 and a["model.norm.weight"].dtype == torch.bfloat16
    assert abs(a["model.norm.weight"].float().mean().item() - 1.0) < 0.1
    folder = write_random_model(str(tmp_path / "m"), TINY_B, seed=5)
    assert json.load(open(os.path.join(folder, "config.json")))["hidden_size"] == 96
    files = ModelFiles(folder)
    cfg = Qwen3Config.from_dict(TINY_B)
    model = DecoderModel(build_plan(cfg, files.names()), "float32", "cpu")
    got = load_checkpoint(files, model.expected_tensors(), model.plan.ignored_tensors)
    assert all(t.dtype == torch.bfloat16 for t in got.values())      # kept as stored
    f32 = write_random_model(str(tmp_path / "m32"), TINY_A, seed=5, dtype=torch.float32)
    assert ModelFiles(f32).info("model.norm.weight")[0] == torch.float32
