"""The plain implementation against the reference's own CPU code (stored
logits, see tests/golden/make_golden.py) and against itself."""
import hashlib
import json
import os

import numpy as np
import pytest

import plain_gpt2

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(HERE, "golden", "gpt2_tiny_reference.json")) as f:
        return json.load(f)


def _golden_model(tmp_path, golden):
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    arch = resolve_architecture(golden["config"])
    cfg = arch.config_class.from_dict(golden["config"])
    d = str(tmp_path / "golden_model")
    write_random_model(d, arch, cfg, golden["seed"], scheme=golden["scheme"], store_dtype="float32")
    with open(os.path.join(d, "model.safetensors"), "rb") as f:
        assert hashlib.sha256(f.read()).hexdigest() == golden["weights_sha256"], \
            "the random-weight generator changed: regenerate tests/golden"
    return d


def test_plain_matches_reference_cpu_code(tmp_path, golden):
    d = _golden_model(tmp_path, golden)
    logits = plain_gpt2.forward_dir(d, golden["tokens"])
    ref = np.array(golden["logits"], dtype=np.float64)
    got = logits[:, golden["columns"]]
    # the reference computes in float32 (with some double accumulators)
    assert np.abs(got - ref).max() < 2e-6
    assert [int(r.argmax()) for r in logits] == golden["argmax"]


@pytest.mark.parametrize("case", ["inverse_layer_idx", "no_scale"])
def test_plain_options_match_reference_on_changed_weights(tmp_path, case):
    """n_inner other than 4*n_embd, scale_attn_by_inverse_layer_idx and scale_attn_weights=false:
    the reference ran an equal function on changed weights (tests/golden/make_golden_b.py); the
    plain implementation runs the options themselves on the original weights."""
    import math
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    with open(os.path.join(HERE, "golden", "gpt2_options_reference.json")) as f:
        g = json.load(f)
    c = g["cases"][case]
    arch = resolve_architecture(c["config"])
    d = str(tmp_path / case)
    write_random_model(d, arch, arch.config_class.from_dict(c["config"]), g["seed"], scheme=g["scheme"],
                       store_dtype="float32")
    with open(os.path.join(d, "model.safetensors"), "rb") as f:
        assert hashlib.sha256(f.read()).hexdigest() == c["weights_sha256"], \
            "the random-weight generator changed: regenerate tests/golden"
    logits = plain_gpt2.forward_dir(d, c["tokens"])
    for n, row in zip(c["prefix_lengths"], c["logits"]):
        got = logits[n - 1, c["columns"]]
        assert np.abs(got - np.array(row)).max() < 3e-6, (case, n)
    # the exact GELU, which no change of weights expresses, against the C library's erf
    u = np.linspace(-6, 6, 49)
    assert np.abs(plain_gpt2.gelu_erf(u) - np.array([0.5 * x * (1 + math.erf(x / math.sqrt(2))) for x in u])).max() < 1e-15


def test_plain_float32_close_to_float64(tmp_path, golden):
    d = _golden_model(tmp_path, golden)
    a = plain_gpt2.forward_dir(d, golden["tokens"], dtype=np.float64)
    b = plain_gpt2.forward_dir(d, golden["tokens"], dtype=np.float32)
    assert np.abs(a - b).max() < 5e-6


def test_plain_is_causal(model_dirs):
    d = model_dirs("B")
    toks = list(np.random.default_rng(0).integers(0, 1000, size=20))
    full = plain_gpt2.forward_dir(d, toks)
    part = plain_gpt2.forward_dir(d, toks[:11])
    assert np.abs(full[:11] - part).max() < 1e-12


def test_plain_options_change_the_result(model_dirs):
    """n_inner, the erf GELU and inverse layer scaling are really read."""
    d = model_dirs("B")
    cfg, w = plain_gpt2.read_model_dir(d)
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    base = plain_gpt2.forward(cfg, w, toks)
    for key, val in (("activation_function", "gelu_new"), ("scale_attn_by_inverse_layer_idx", False),
                     ("layer_norm_epsilon", 1e-2), ("scale_attn_weights", False)):
        c2 = dict(cfg)
        c2[key] = val
        assert np.abs(plain_gpt2.forward(c2, w, toks) - base).max() > 1e-6, key


def test_parts_by_hand():
    x = np.array([[1.0, 2.0, 3.0, 4.0]])
    y = plain_gpt2.layer_norm(x, np.ones(4), np.zeros(4), 0.0)
    assert abs(y.mean()) < 1e-12 and abs(y.var() - 1.0) < 1e-12
    assert abs(plain_gpt2.gelu_new(np.array([1.0]))[0] - 0.8411919906) < 1e-9
    assert abs(plain_gpt2.gelu_erf(np.array([1.0]))[0] - 0.8413447461) < 1e-9
    assert plain_gpt2.gelu_new(np.array([0.0]))[0] == 0.0
    # attention of one head, two positions: second row mixes both values
    q = np.array([[1.0, 0.0], [1.0, 0.0]])
    k = np.array([[1.0, 0.0], [0.0, 0.0]])
    v = np.array([[1.0, 2.0], [3.0, 4.0]])
    o = plain_gpt2.causal_attention(q, k, v, 1, 1.0)
    assert np.allclose(o[0], v[0])
    w0 = np.exp(1.0) / (np.exp(1.0) + 1.0)
    assert np.allclose(o[1], w0 * v[0] + (1 - w0) * v[1])
    # a window of one key sees only itself
    o1 = plain_gpt2.causal_attention(q, k, v, 1, 1.0, window=1)
    assert np.allclose(o1, v)


def test_sampling_restated():
    s = 88172645463325252
    s, u = plain_gpt2.uniform(s)
    assert 0.0 <= u < 1.0
    p = plain_gpt2.temperature_probs([0.0, 1.0, 2.0], 0.5)
    assert abs(p.sum() - 1.0) < 1e-12 and p[2] > p[1] > p[0]
    assert plain_gpt2.greedy([1.0, 3.0, 3.0]) == 1
