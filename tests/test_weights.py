import json
import os
import struct

import numpy as np
import pytest
import torch

from conftest import TINY_A, TINY_B
from sglang_c_b200.config import GPT2Config, resolve_architecture
from sglang_c_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_checked,
                                   required_tensors, write_random_model, write_safetensors)


def _plan(d):
    arch = resolve_architecture(d)
    cfg = arch.config_class.from_dict(d)
    return arch, cfg, arch.build_plan(cfg)


def test_safetensors_roundtrip_keeps_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "d": torch.randn(2, 2).to(torch.float16),
         "e": torch.empty(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, metadata={"k": "v"})
    with SafetensorsFile(p) as f:
        assert sorted(f.names()) == sorted(t) and f.metadata == {"k": "v"}
        for k, v in t.items():
            got = f.tensor(k)
            assert got.dtype == v.dtype and tuple(got.shape) == tuple(v.shape)
            assert torch.equal(got, v)


def test_safetensors_readable_by_an_independent_reader(tmp_path):
    import plain_gpt2
    t = {"w": torch.randn(4, 3), "h": torch.randn(5).to(torch.bfloat16)}
    p = str(tmp_path / "y.safetensors")
    write_safetensors(p, t)
    got = plain_gpt2.read_safetensors(p)
    assert np.array_equal(got["w"], t["w"].double().numpy())
    assert np.array_equal(got["h"], t["h"].double().numpy())


def _raw(path, header, data=b""):
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + data)


def test_corrupted_files_are_refused(tmp_path):
    p = str(tmp_path / "z.safetensors")
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    _raw(p, {"t": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}, b"\0" * 16)
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFile(p)
    assert "'t'" in str(e.value)
    _raw(p, {"t": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    _raw(p, {"t": {"dtype": "Q4", "shape": [1], "data_offsets": [0, 1]}}, b"\0")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(tmp_path / "absent.safetensors"))


def test_required_tensors_are_the_architectures_names():
    _, cfg, plan = _plan(TINY_B)
    need = required_tensors(plan)
    assert len(need) == 4 + 12 * cfg.n_layer          # the reference fetches 4 + 12 per layer
    assert need["h.1.attn.c_attn.weight"].shape == (96, 288)      # Conv1D layout [in, out]
    assert need["h.2.mlp.c_fc.weight"].shape == (96, 320)
    assert need["h.2.mlp.c_proj.weight"].shape == (320, 96)
    assert need["wte.weight"].shape == (1000, 96) and need["wpe.weight"].shape == (256, 96)


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    arch, cfg, plan = _plan(TINY_A)
    d = str(tmp_path / "m")
    write_random_model(d, arch, cfg, 3, scheme="varied")
    with SafetensorsFile(os.path.join(d, "model.safetensors")) as f:
        t = {n: f.tensor(n) for n in f.names()}
    del t["h.0.ln_1.bias"]
    del t["h.1.mlp.c_fc.weight"]
    t["h.1.attn.c_proj.weight"] = torch.zeros(64, 63)
    t["surprise.weight"] = torch.zeros(3)
    t["h.0.attn.c_attn.bias"] = torch.zeros(192, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_checked(plan, d)
    msg = str(e.value)
    for s in ("missing tensors (2)", "h.0.ln_1.bias", "h.1.mlp.c_fc.weight", "unexpected tensors (1)",
              "surprise.weight", "h.1.attn.c_proj.weight", "[64, 63]", "[64, 64]", "h.0.attn.c_attn.bias"):
        assert s in msg, s


def test_prefix_and_ignorable_names(tmp_path):
    arch, cfg, plan = _plan(TINY_A)
    d = str(tmp_path / "m")
    write_random_model(d, arch, cfg, 3)
    with SafetensorsFile(os.path.join(d, "model.safetensors")) as f:
        t = {"transformer." + n: f.tensor(n) for n in f.names()}
    t["lm_head.weight"] = t["transformer.wte.weight"].clone()
    t["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    refs = load_checked(plan, d)
    assert refs["wte.weight"].name == "transformer.wte.weight"
    os.remove(os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError):
        load_checked(plan, d)


def test_stored_precision_is_kept(tmp_path):
    arch, cfg, plan = _plan(TINY_B)
    d32 = write_random_model(str(tmp_path / "f"), arch, cfg, 5, scheme="varied", store_dtype="float32")
    d16 = write_random_model(str(tmp_path / "b"), arch, cfg, 5, scheme="varied", store_dtype="bfloat16")
    r32, r16 = load_checked(plan, d32), load_checked(plan, d16)
    assert r32["wte.weight"].tensor.dtype == torch.float32
    assert r16["wte.weight"].tensor.dtype == torch.bfloat16            # kept, not widened
    assert r16["h.0.ln_1.weight"].tensor.dtype == torch.float32        # a vector stored in 32-bit stays so
    assert torch.equal(r16["wte.weight"].tensor, r32["wte.weight"].tensor.to(torch.bfloat16))


def test_random_weights_are_seeded_and_follow_the_scheme(tmp_path):
    arch, cfg, plan = _plan(TINY_B)
    a = load_checked(plan, write_random_model(str(tmp_path / "a"), arch, cfg, 11, scheme="standard"))
    b = load_checked(plan, write_random_model(str(tmp_path / "b"), arch, cfg, 11, scheme="standard"))
    c = load_checked(plan, write_random_model(str(tmp_path / "c"), arch, cfg, 12, scheme="standard"))
    v = load_checked(plan, write_random_model(str(tmp_path / "v"), arch, cfg, 11, scheme="varied"))
    assert all(torch.equal(a[k].tensor, b[k].tensor) for k in a)
    assert not torch.equal(a["wte.weight"].tensor, c["wte.weight"].tensor)
    assert float(a["h.0.mlp.c_fc.bias"].tensor.abs().max()) == 0.0
    assert torch.equal(a["ln_f.weight"].tensor, torch.ones(96))
    assert abs(float(a["wte.weight"].tensor.std()) - 0.02) < 0.001
    want = 0.02 / (2 * cfg.n_layer) ** 0.5
    assert abs(float(a["h.1.mlp.c_proj.weight"].tensor.std()) - want) < 0.001
    assert float(v["h.0.mlp.c_fc.bias"].tensor.abs().max()) > 0.0
    assert abs(float(v["ln_f.weight"].tensor.mean()) - 1.0) < 0.05
    assert os.path.exists(os.path.join(str(tmp_path / "a"), "config.json"))
    # the written config reads back to the same configuration
    from sglang_c_b200.config import load_config
    assert load_config(str(tmp_path / "a"))[1] == cfg


def test_sharded_checkpoint_through_its_index(tmp_path):
    """model.safetensors.index.json -> shards (reference src/safetensors.c:676-843): the same
    tensors load from hand-written shards; a shard or a tensor the index names and the folder
    lacks is one clear error."""
    arch, cfg, plan = _plan(TINY_A)
    whole = write_random_model(str(tmp_path / "whole"), arch, cfg, 3, scheme="varied")
    with SafetensorsFile(os.path.join(whole, "model.safetensors")) as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    names = sorted(tensors)
    d = tmp_path / "sharded"
    d.mkdir()
    parts = [names[0::3], names[1::3], names[2::3]]
    wmap = {}
    for i, part in enumerate(parts):
        shard = f"model-{i + 1:05d}-of-00003.safetensors"
        write_safetensors(str(d / shard), {n: tensors[n] for n in part})
        wmap.update({n: shard for n in part})
    with open(d / "config.json", "w") as f:
        json.dump(cfg.to_dict(), f)
    with open(d / "model.safetensors.index.json", "w") as f:
        json.dump({"metadata": {"total_size": 0}, "weight_map": wmap}, f)
    refs = load_checked(plan, str(d))
    assert sorted(refs) == sorted(required_tensors(plan))
    for n, r in refs.items():
        assert torch.equal(r.tensor, tensors[r.name])
    # a tensor the index sends to the wrong shard
    bad = dict(wmap)
    bad[names[0]] = wmap[names[1]]
    with open(d / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": bad}, f)
    with pytest.raises(WeightError, match="not found in the shard"):
        load_checked(plan, str(d))
    # a shard that is not there
    bad = dict(wmap)
    bad[names[0]] = "model-00009-of-00003.safetensors"
    with open(d / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": bad}, f)
    with pytest.raises(WeightError, match="names shard"):
        load_checked(plan, str(d))
    # a tensor missing from the index is reported like any missing tensor
    less = {n: s for n, s in wmap.items() if n != "ln_f.bias"}
    with open(d / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": less}, f)
    with pytest.raises(WeightError, match=r"missing tensors \(1\): ln_f.bias"):
        load_checked(plan, str(d))
