import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=64, n_head=4,
              n_inner=256, vocab_size=512, n_positions=128, layer_norm_epsilon=1e-5,
              activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False)
TINY_B = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=3, n_embd=96, n_head=3,
              n_inner=320, vocab_size=1000, n_positions=256, layer_norm_epsilon=1e-6,
              activation_function="gelu", scale_attn_by_inverse_layer_idx=True)
# a third one with a longer context, for long decoding and far keys
TINY_C = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=128, n_head=2,
              n_inner=192, vocab_size=777, n_positions=1024, layer_norm_epsilon=1e-5,
              activation_function="gelu_new", scale_attn_by_inverse_layer_idx=True)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
PAGE_SIZE = {"A": 16, "B": 8, "C": 16}


def make_model_dir(tmp, name, store_dtype="float32", seed=None, scheme="varied"):
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    d = TINY[name]
    arch = resolve_architecture(d)
    cfg = arch.config_class.from_dict(d)
    out = os.path.join(str(tmp), f"tiny_{name}_{store_dtype}")
    if not os.path.exists(os.path.join(out, "model.safetensors")):
        write_random_model(out, arch, cfg, seed if seed is not None else 100 + ord(name), scheme=scheme,
                           store_dtype=store_dtype)
    return out


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """(name, store_dtype) -> model folder, made on first use in a temporary folder."""
    base = tmp_path_factory.mktemp("models")
    cache = {}

    def get(name, store_dtype="float32"):
        key = (name, store_dtype)
        if key not in cache:
            cache[key] = make_model_dir(base, name, store_dtype)
        return cache[key]

    return get


SHARP = 6.0     # factor on the query and key projections of a "sharp" model


def make_sharp_dir(tmp, name, store_dtype="float32", factor=SHARP):
    """The tiny model `name` with the query and key columns of every c_attn (weights and biases)
    multiplied by `factor`: scores grow by its square, the softmax stops being nearly uniform
    (with N(0, 0.02) weights it is), and every single key carries weight: a key dropped, misplaced
    or read from a stale page moves logits by far more than rounding does."""
    import json
    import numpy as np
    import torch
    import plain_gpt2
    from sglang_c_b200.weights.safetensors_io import write_safetensors
    base = make_model_dir(tmp, name, "float32")
    out = os.path.join(str(tmp), f"sharp_{name}_{store_dtype}")
    if os.path.exists(os.path.join(out, "model.safetensors")):
        return out
    cfg, w = plain_gpt2.read_model_dir(base)
    E = cfg["n_embd"]
    tensors = {}
    for k, v in w.items():
        a = np.array(v, dtype=np.float32)
        if k.endswith("attn.c_attn.weight"):
            a[:, :2 * E] *= factor
        elif k.endswith("attn.c_attn.bias"):
            a[:2 * E] *= factor
        t = torch.from_numpy(a)
        tensors[k] = t.to(torch.bfloat16) if (store_dtype == "bfloat16" and t.dim() >= 2) else t
    os.makedirs(out, exist_ok=True)
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(out, "model.safetensors"), tensors)
    return out


@pytest.fixture(scope="session")
def sharp_dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("sharp")
    cache = {}

    def get(name, store_dtype="float32"):
        key = (name, store_dtype)
        if key not in cache:
            cache[key] = make_sharp_dir(base, name, store_dtype)
        return cache[key]

    return get
