"""Makes tests/golden/gpt2_options_reference.json: an anchor for the configuration options that
the reference's GPT-2 does not have (`n_inner` other than 4*n_embd,
`scale_attn_by_inverse_layer_idx`, `scale_attn_weights=false`), taken from the reference's own
CPU code all the same.

Usage:  python tests/golden/make_golden_b.py REFERENCE_TREE

The reference (integemjack/sglang.c, src/gpt2.c) fixes the feed-forward width at 4*n_embd
(:60) and the score scale at 1/sqrt(head_dim) (:253).  A model with the options set is equal,
as a function, to a model without them whose weights are changed:

  * n_inner < 4*n_embd: c_fc gets zero columns (and zero biases) up to 4*n_embd and c_proj zero
    rows; the added units output gelu(0) = 0 and add nothing;
  * a score scale s instead of 1/sqrt(D): the query columns of c_attn (weights and biases) are
    multiplied by s*sqrt(D), which the reference's 1/sqrt(D) then turns into s.
    s = (1/sqrt(D) if scale_attn_weights else 1) / (layer_idx + 1 if
    scale_attn_by_inverse_layer_idx else 1), layer_idx counted from 0.

So this script writes a random model with the options set (this repository's generator), writes
the changed weights beside it, runs the reference's `sgl_gpt2_prefill` on the changed model and
stores its logits; `tests/test_plain.py` compares the plain implementation, run on the ORIGINAL
weights with the options set, with them.  What this pins is that the plain implementation applies
each option where and how the formulas above say; the exact GELU (`activation_function: gelu`) is
not expressible this way and rests on its formula (checked against math.erf in the tests).
"""
import ctypes
import hashlib
import json
import math
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

BASE = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=3, n_embd=96, n_head=3, n_inner=320,
            n_positions=256, vocab_size=1000, layer_norm_epsilon=1e-6, activation_function="gelu_new")
CASES = {
    "inverse_layer_idx": dict(BASE, scale_attn_by_inverse_layer_idx=True),
    "no_scale": dict(BASE, scale_attn_weights=False),
}
SEED = 31337
N_TOKENS = 20
SOURCES = ["gpt2", "ops", "tensor", "alloc", "log", "json", "safetensors", "gguf", "qweight", "sampling"]


def changed_weights(cfg, w):
    E, H, L, I = cfg["n_embd"], cfg["n_head"], cfg["n_layer"], cfg["n_inner"]
    D = E // H
    out = {k: np.array(v, dtype=np.float32) for k, v in w.items()}
    for l in range(L):
        p = f"h.{l}."
        s = (1.0 / math.sqrt(D)) if cfg.get("scale_attn_weights", True) else 1.0
        if cfg.get("scale_attn_by_inverse_layer_idx", False):
            s /= (l + 1)
        f = np.float32(s * math.sqrt(D))
        out[p + "attn.c_attn.weight"][:, :E] *= f
        out[p + "attn.c_attn.bias"][:E] *= f
        fc_w = np.zeros((E, 4 * E), np.float32)
        fc_w[:, :I] = out[p + "mlp.c_fc.weight"]
        fc_b = np.zeros(4 * E, np.float32)
        fc_b[:I] = out[p + "mlp.c_fc.bias"]
        pr_w = np.zeros((4 * E, E), np.float32)
        pr_w[:I] = out[p + "mlp.c_proj.weight"]
        out[p + "mlp.c_fc.weight"], out[p + "mlp.c_fc.bias"], out[p + "mlp.c_proj.weight"] = fc_w, fc_b, pr_w
    return out


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden_b.py REFERENCE_TREE   (a checkout of integemjack/sglang.c)")
    ref = sys.argv[1]
    import torch
    import plain_gpt2
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    from sglang_c_b200.weights.safetensors_io import write_safetensors
    tmp = tempfile.mkdtemp(prefix="sglc_golden_b_")
    lib = os.path.join(tmp, "libsglref.so")
    cmd = ["gcc", "-std=c11", "-O2", "-fopenmp", "-D_GNU_SOURCE", "-shared", "-fPIC",
           f"-I{ref}/include", f"-I{ref}/third_party/stb", "-o", lib]
    cmd += [f"{ref}/src/{s}.c" for s in SOURCES] + ["-lm", "-ldl"]
    subprocess.run(cmd, check=True, stderr=subprocess.DEVNULL)
    L = ctypes.CDLL(lib)
    L.sgl_gpt2_load.restype = ctypes.c_void_p
    L.sgl_gpt2_load.argtypes = [ctypes.c_char_p]
    L.sgl_gpt2_pages_alloc.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    L.sgl_gpt2_prefill.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int,
                                   ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_float)]
    golden = {"source": "reference src/gpt2.c sgl_gpt2_prefill on changed weights (see make_golden_b.py), float32",
              "seed": SEED, "scheme": "varied", "cases": {}}
    for name, cfg_d in CASES.items():
        arch = resolve_architecture(cfg_d)
        cfg = arch.config_class.from_dict(cfg_d)
        d = os.path.join(tmp, name)
        write_random_model(d, arch, cfg, SEED, scheme="varied", store_dtype="float32")
        with open(os.path.join(d, "model.safetensors"), "rb") as f:
            digest = hashlib.sha256(f.read()).hexdigest()
        _, w = plain_gpt2.read_model_dir(d)
        d2 = os.path.join(tmp, name + "_changed")
        os.makedirs(d2)
        write_safetensors(os.path.join(d2, "model.safetensors"),
                          {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in changed_weights(cfg_d, w).items()})
        with open(os.path.join(d2, "config.json"), "w") as f:
            json.dump({"model_type": "gpt2", "n_layer": cfg_d["n_layer"], "n_head": cfg_d["n_head"],
                       "n_embd": cfg_d["n_embd"], "n_positions": cfg_d["n_positions"], "n_ctx": cfg_d["n_positions"],
                       "vocab_size": cfg_d["vocab_size"], "layer_norm_epsilon": cfg_d["layer_norm_epsilon"]}, f)
        m = L.sgl_gpt2_load(d2.encode())
        assert m, "reference failed to load the changed model"
        V = cfg_d["vocab_size"]
        toks = [int(t) for t in np.random.default_rng(11).integers(0, V, size=N_TOKENS)]
        IntArr = ctypes.c_int * N_TOKENS
        pages = IntArr()
        assert L.sgl_gpt2_pages_alloc(m, pages, N_TOKENS) == 0
        tarr = IntArr(*toks)
        rows = []
        for n in (1, 7, N_TOKENS):
            out = (ctypes.c_float * V)()
            assert L.sgl_gpt2_prefill(m, tarr, n, 0, pages, out) == 0
            rows.append((n, np.frombuffer(out, dtype=np.float32).copy()))
        golden["cases"][name] = {"config": cfg_d, "tokens": toks, "weights_sha256": digest,
                                 "prefix_lengths": [n for n, _ in rows], "columns": list(range(0, V, 5)),
                                 "logits": [[float(f"{v:.9g}") for v in r[::5]] for _, r in rows]}
    with open(os.path.join(HERE, "gpt2_options_reference.json"), "w") as f:
        json.dump(golden, f)
    print("wrote gpt2_options_reference.json")


if __name__ == "__main__":
    main()
