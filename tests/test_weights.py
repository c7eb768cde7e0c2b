import json
import os
import struct

import pytest
import torch

from forge_b200.engine.model import Model
from forge_b200.parts import Runtime
from forge_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_tensors, random_tensors,
                                write_random_model, write_safetensors)
from helpers import tiny_config
from plain.safetensors_reader import read_safetensors


def _specs(name):
    return Model(tiny_config(name).plan(), Runtime(torch.device("cpu"), torch.bfloat16)).tensor_specs()


def test_random_model_folder_loads_and_is_reproducible(tmp_path):
    cfg = tiny_config("B")
    d1 = write_random_model(cfg, str(tmp_path / "m1"), seed=5, norm_std=0.1)
    d2 = write_random_model(cfg, str(tmp_path / "m2"), seed=5, norm_std=0.1)
    d3 = write_random_model(cfg, str(tmp_path / "m3"), seed=6, norm_std=0.1)
    t1, t2, t3 = (load_tensors(d, _specs("B")) for d in (d1, d2, d3))
    assert set(t1) == {n for n, s in _specs("B").items() if s.required}
    assert all(torch.equal(t1[n], t2[n]) for n in t1)
    assert any(not torch.equal(t1[n], t3[n]) for n in t1)
    # matrices stay bfloat16, a tensor stored in 32-bit stays 32-bit
    assert t1["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert t1["model.norm.weight"].dtype == torch.float32
    assert "lm_head.weight" not in t1                      # tied
    assert json.load(open(os.path.join(d1, "config.json")))["architectures"] == ["LlamaForCausalLM"]
    # the independent reader of the test oracle sees the same numbers
    plain = read_safetensors(os.path.join(d1, "model.safetensors"))
    for n in t1:
        assert torch.equal(torch.from_numpy(plain[n]), t1[n].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = tiny_config("A")
    t = random_tensors(cfg, seed=0)
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    t["lm_head.weight"] = torch.zeros(250, 64, dtype=torch.int32)
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), t)
    with pytest.raises(WeightError) as ei:
        load_tensors(str(tmp_path / "m"), _specs("A"))
    e = ei.value
    assert sorted(e.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(e.wrong) == 2 and "k_proj" in e.wrong[0] + e.wrong[1] and "[16, 64]" in str(e)
    for word in ("missing (2)", "unexpected (1)", "wrong shape or dtype (2)"):
        assert word in str(e)


def test_bias_tensors_must_agree_with_config(tmp_path):
    t = random_tensors(tiny_config("B"), seed=0)
    del t["model.layers.2.self_attn.v_proj.bias"]
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), t)
    with pytest.raises(WeightError, match="v_proj.bias"):
        load_tensors(str(tmp_path / "m"), _specs("B"))


def test_truncated_and_garbled_files(tmp_path):
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, {"a": torch.arange(12, dtype=torch.float32).reshape(3, 4)})
    blob = open(p, "rb").read()
    f = SafetensorsFile(p)
    assert torch.equal(f.tensor("a"), torch.arange(12, dtype=torch.float32).reshape(3, 4))
    f.close()
    open(p, "wb").write(blob[:-5])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(blob[:4])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 7) + b"not js!" + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="neither"):
        load_tensors(str(tmp_path / "empty_dir_does_not_exist"), {})


def test_sharded_index(tmp_path):
    cfg = tiny_config("A")
    t = random_tensors(cfg, seed=3)
    names = list(t)
    half = len(names) // 2
    write_safetensors(str(tmp_path / "s1.safetensors"), {n: t[n] for n in names[:half]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: t[n] for n in names[half:]})
    wm = {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    got = load_tensors(str(tmp_path), _specs("A"))
    assert all(torch.equal(got[n], t[n]) for n in names)
