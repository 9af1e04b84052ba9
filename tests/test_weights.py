"""Safetensors reading and writing, binding by name and its one error (no GPU)."""
import json
import struct

import pytest
import torch

from gibbs_b200.config import Lfm2Config
from gibbs_b200.parts.base import Runtime
from gibbs_b200.weights import (Checkpoint, SafetensorsError, SafetensorsFile, TensorDict, WeightBinder, WeightError,
                                expected_tensors, memory_dtype, random_tensors, write_random_model,
                                write_safetensors)
from helpers import TINY_A, TINY_B
import plain_lfm2 as plain


def test_round_trip_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
               "d": torch.randn(2, 2, 2).to(torch.float16), "e": torch.empty(0, 4)}
    write_safetensors(tmp_path / "model.safetensors", tensors.items(), metadata={"k": "v"})
    f = SafetensorsFile(tmp_path / "model.safetensors")
    assert f.metadata == {"k": "v"} and set(f.names()) == set(tensors)
    for n, t in tensors.items():
        assert f.dtype(n) == t.dtype and f.shape(n) == tuple(t.shape)
        assert torch.equal(f.tensor(n), t)
    # the oracle's own reader agrees (it widens to float64)
    again = plain.read_safetensors(tmp_path / "model.safetensors")
    assert torch.equal(again["b"].to(torch.bfloat16), tensors["b"])
    raw = (tmp_path / "model.safetensors").read_bytes()
    assert struct.unpack("<Q", raw[:8])[0] % 8 == 0


def test_truncated_and_corrupt_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="does not fit"):
        SafetensorsFile(p)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(p)


def test_sharded_checkpoint(tmp_path):
    write_safetensors(tmp_path / "s1.safetensors", [("a", torch.ones(2))])
    write_safetensors(tmp_path / "s2.safetensors", [("b", torch.zeros(3))])
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    ck = Checkpoint(tmp_path)
    assert sorted(ck.names()) == ["a", "b"] and ck.shape("b") == (3,)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "zz": "s2.safetensors"}}))
    with pytest.raises(SafetensorsError, match="zz"):
        Checkpoint(tmp_path)
    with pytest.raises(FileNotFoundError):
        Checkpoint(tmp_path / "nowhere")


def _binder(tensors, raw=TINY_A, dtype=torch.float32):
    plan = Lfm2Config.from_dict(raw).plan()
    return WeightBinder(plan, TensorDict(tensors), Runtime(dtype, torch.device("cpu")))


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    plan = Lfm2Config.from_dict(TINY_A).plan()
    tensors = dict(random_tensors(plan, 0))
    _binder(tensors).verify()
    del tensors["model.layers.1.self_attn.k_proj.weight"]
    del tensors["model.layers.2.ffn_norm.weight"]
    tensors["model.layers.0.mystery.weight"] = torch.zeros(3)
    tensors["model.layers.0.feed_forward.w1.weight"] = torch.zeros(100, 64)
    tensors["model.layers.0.conv.conv.weight"] = torch.zeros(64, 3)          # squeezed taps are accepted
    with pytest.raises(WeightError) as e:
        _binder(tensors).verify()
    err = e.value
    assert [n for n, _ in err.missing] == ["model.layers.1.self_attn.k_proj.weight", "model.layers.2.ffn_norm.weight"]
    assert [n for n, _ in err.unexpected] == ["model.layers.0.mystery.weight"]
    assert [n for n, _, _ in err.wrong_shape] == ["model.layers.0.feed_forward.w1.weight"]
    text = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors", "wrong shapes (1)", "[192, 64]", "[100, 64]",
                   "k_proj.weight", "mystery"):
        assert needle in text


def test_config_that_disagrees_with_the_tensors_present():
    plan_b = Lfm2Config.from_dict(TINY_B).plan()
    tensors = dict(random_tensors(plan_b, 1))
    raw = dict(TINY_B, full_attn_idxs=[0, 2])            # says layer 5 is conv; the checkpoint has attention
    with pytest.raises(WeightError) as e:
        _binder(tensors, raw).verify()
    assert any("layers.5.conv.in_proj.weight" in n for n, _ in e.value.missing)
    assert any("layers.5.self_attn.q_proj.weight" in n for n, _ in e.value.unexpected)
    # a checkpoint with an untied head under a tied configuration: lm_head.weight is unexpected
    with pytest.raises(WeightError) as e:
        _binder(tensors, dict(TINY_B, tie_embedding=True)).verify()
    assert [n for n, _ in e.value.unexpected] == ["lm_head.weight"]


def test_memory_dtypes():
    bf, f32 = torch.bfloat16, torch.float32
    assert memory_dtype(bf, "matrix", bf) == bf
    assert memory_dtype(f32, "matrix", bf) == f32          # stored in 32-bit stays so
    assert memory_dtype(torch.float16, "matrix", bf) == f32
    assert memory_dtype(bf, "matrix", f32) == f32
    assert memory_dtype(bf, "vector", bf) == f32
    assert memory_dtype(torch.int64, "int", bf) == torch.int32
    b = _binder(dict(random_tensors(Lfm2Config.from_dict(TINY_A).plan(), 0, torch.bfloat16)), dtype=torch.bfloat16)
    b.verify()
    assert b.fetch("model.embed_tokens.weight").dtype == bf
    assert b.fetch("model.layers.0.operator_norm.weight").dtype == f32
    assert b.fetch("model.layers.0.conv.conv.weight").shape == (64, 3)
    assert b.fetch("model.embed_tokens.weight") is b.fetch("model.embed_tokens.weight")   # tied: one copy


def test_random_weights_folder(tmp_path):
    cfg = Lfm2Config.from_dict(TINY_B)
    folder = write_random_model(tmp_path / "m", cfg, seed=1)
    again = write_random_model(tmp_path / "m2", cfg, seed=1)
    other = write_random_model(tmp_path / "m3", cfg, seed=2)
    a, b, c = (Checkpoint(f) for f in (folder, again, other))
    assert set(a.names()) == set(expected_tensors(cfg.plan()))
    for n in a.names():
        assert torch.equal(a.tensor(n), b.tensor(n))
    assert not torch.equal(a.tensor("lm_head.weight"), c.tensor("lm_head.weight"))
    assert a.shape("model.layers.1.conv.conv.weight") == (96, 1, 4)
    w = a.tensor("model.layers.0.self_attn.q_proj.weight")
    assert abs(float(w.std()) - 0.02) < 0.002 and torch.all(a.tensor("model.embedding_norm.weight") == 1)
    assert Lfm2Config.from_dict(json.loads((folder / "config.json").read_text())) == cfg
    # bfloat16 folder = the float32 values rounded
    bf = Checkpoint(write_random_model(tmp_path / "m4", cfg, seed=1, dtype=torch.bfloat16))
    assert torch.equal(bf.tensor("lm_head.weight"), a.tensor("lm_head.weight").to(torch.bfloat16))
