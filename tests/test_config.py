import json
import os

import pytest

from conftest import TINY_A, TINY_B
from sglang_c_b200.config import (ConfigError, GPT2Config, known_architectures, load_config,
                                  register_architecture, resolve_architecture)


def test_reads_every_key():
    c = GPT2Config.from_dict(TINY_B)
    assert (c.n_layer, c.n_embd, c.n_head, c.n_inner, c.vocab_size, c.n_positions) == (3, 96, 3, 320, 1000, 256)
    assert c.layer_norm_epsilon == 1e-6 and c.activation == "gelu_erf"
    assert c.scale_attn_by_inverse_layer_idx is True and c.scale_attn_weights is True
    assert c.head_dim == 32


def test_defaults_defined_by_the_architecture():
    d = {k: v for k, v in TINY_A.items() if k not in ("n_inner", "activation_function",
                                                      "scale_attn_by_inverse_layer_idx")}
    c = GPT2Config.from_dict(d)
    assert c.n_inner == 4 * c.n_embd and c.activation == "gelu_tanh"
    assert c.scale_attn_by_inverse_layer_idx is False
    d["n_inner"] = None
    assert GPT2Config.from_dict(d).n_inner == 4 * c.n_embd


@pytest.mark.parametrize("key", ["n_layer", "n_embd", "n_head", "vocab_size", "n_positions",
                                 "layer_norm_epsilon"])
def test_sizes_are_required_and_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError) as e:
        GPT2Config.from_dict(d)
    assert key in str(e.value) or (key == "n_positions" and "n_ctx" in str(e.value))


def test_n_ctx_stands_for_n_positions():
    d = dict(TINY_A)
    del d["n_positions"]
    d["n_ctx"] = 77
    assert GPT2Config.from_dict(d).n_positions == 77


@pytest.mark.parametrize("key,val", [("n_embd", 65), ("n_layer", 0), ("n_head", "4"),
                                     ("activation_function", "relu"), ("layer_norm_epsilon", 0),
                                     ("vocab_size", -3), ("scale_attn_weights", "yes"),
                                     ("tie_word_embeddings", False)])
def test_bad_values_name_the_key(key, val):
    d = dict(TINY_A)
    d[key] = val
    with pytest.raises(ConfigError) as e:
        GPT2Config.from_dict(d)
    assert key in str(e.value) or "n_head" in str(e.value)


def test_integral_floats_and_bools_are_integers():
    d = dict(TINY_A)
    d["n_layer"] = 2.0
    assert GPT2Config.from_dict(d).n_layer == 2


def test_registry_by_architectures_then_model_type():
    assert "GPT2LMHeadModel" in known_architectures()
    assert resolve_architecture({"architectures": ["GPT2LMHeadModel"]}).name == "GPT2LMHeadModel"
    assert resolve_architecture({"model_type": "gpt2"}).name == "GPT2LMHeadModel"
    with pytest.raises(ConfigError) as e:
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    assert "GPT2LMHeadModel" in str(e.value) and "LlamaForCausalLM" in str(e.value)


def test_load_config_from_folder_and_roundtrip(tmp_path):
    c = GPT2Config.from_dict(TINY_B)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(c.to_dict(), f)
    arch, c2 = load_config(str(tmp_path))
    assert c2 == c and arch.name == "GPT2LMHeadModel"
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nothing"))
    (tmp_path / "bad").mkdir()
    (tmp_path / "bad" / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "bad"))


def test_plan_has_no_size_of_its_own():
    arch = resolve_architecture(TINY_B)
    plan = arch.build_plan(GPT2Config.from_dict(TINY_B))
    assert plan.hidden_size == 96 and plan.vocab_size == 1000 and plan.max_positions == 256
    assert len(plan.layers) == 3 and [c.layer for c in plan.order] == [0, 1, 2]
    m = plan.layers[2].mixer.params
    assert m["n_heads"] == 3 and m["head_dim"] == 32
    assert abs(m["scale"] - (1.0 / 32 ** 0.5) / 3.0) < 1e-12       # inverse layer index scaling
    assert plan.layers[0].ffn.params["inner_size"] == 320
    assert plan.layers[0].ffn.params["activation"] == "gelu_erf"
    assert plan.layers[1].norm1.params["eps"] == 1e-6
    assert plan.head.weights["weight"] == plan.embedding.weights["table"]    # tied


def test_another_architecture_can_be_registered():
    from sglang_c_b200.models.gpt2 import build_plan
    register_architecture("ToyForTest", GPT2Config, build_plan, model_types=("toy",))
    assert resolve_architecture({"architectures": ["ToyForTest"]}).name == "ToyForTest"
    assert resolve_architecture({"model_type": "toy"}).name == "ToyForTest"


def test_log_lines_have_the_reference_format_and_honour_the_level():
    import re
    from sglang_c_b200 import log
    lines = []
    log.set_sink(lines.append)
    before = log.get_level()
    try:
        log.set_level("WARN")
        log.info("not shown")
        log.warn("pool nearly full")
        log.info("always", always=True)
        log.set_level(log.DEBUG)
        log.debug("now shown")
    finally:
        log.set_level(before)
        log.set_sink(None)
    assert len(lines) == 3
    assert re.match(r"^\d\d:\d\d:\d\d\.\d{3} WARN test_config\.py:\d+\] pool nearly full$", lines[0])
    assert " INFO " in lines[1] and lines[2].endswith("now shown")


def test_walker_structures_match_the_c_side_and_every_launcher_binds():
    """Runs without a GPU: loading the libraries and comparing structure sizes needs none."""
    from sglang_c_b200.engine import host_model
    lib = host_model._walker()
    assert lib is host_model._walker()
