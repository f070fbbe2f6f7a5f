"""Makes tests/golden/gpt2_tiny_reference.json: logits of the reference's own CPU
GPT-2 (integemjack/sglang.c, src/gpt2.c) on a tiny random model.

Usage:  python tests/golden/make_golden.py REFERENCE_TREE

It compiles the reference's C sources, unmodified, with gcc into a shared library
in a temporary folder, writes a tiny random model folder with this repository's
generator (seed and configuration are stored in the output), loads it through
`sgl_gpt2_load`, and for every prefix of a token sequence calls
`sgl_gpt2_prefill` from position 0 to get that prefix's last-row logits.  It also
checks that prefill(n-3) followed by three `sgl_gpt2_decode_batch` steps gives
the same logits as the whole prefill.  The reference can express only
`n_inner = 4*n_embd`, tanh GELU and plain 1/sqrt(D) scaling, so only such a
configuration is anchored this way.  `tests/test_plain.py` compares the plain
implementation with the stored logits and also checks a digest of the weights,
so that a change of the generator cannot go unnoticed.
"""
import ctypes
import hashlib
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

CONFIG = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=64, n_head=4,
              n_positions=128, vocab_size=512, layer_norm_epsilon=1e-5,
              activation_function="gelu_new")
SEED = 20240
TOKENS_SEED = 7
N_TOKENS = 24
SOURCES = ["gpt2", "ops", "tensor", "alloc", "log", "json", "safetensors", "gguf", "qweight", "sampling"]


def weights_digest(model_dir):
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def make_model(out_dir):
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    arch = resolve_architecture(CONFIG)
    cfg = arch.config_class.from_dict(CONFIG)
    write_random_model(out_dir, arch, cfg, SEED, scheme="varied", store_dtype="float32")
    return out_dir


def tokens():
    rng = np.random.default_rng(TOKENS_SEED)
    return [int(t) for t in rng.integers(0, CONFIG["vocab_size"], size=N_TOKENS)]


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py REFERENCE_TREE   (a checkout of integemjack/sglang.c)")
    ref = sys.argv[1]
    tmp = tempfile.mkdtemp(prefix="sglc_golden_")
    lib = os.path.join(tmp, "libsglref.so")
    cmd = ["gcc", "-std=c11", "-O2", "-fopenmp", "-D_GNU_SOURCE", "-shared", "-fPIC",
           f"-I{ref}/include", f"-I{ref}/third_party/stb", "-o", lib]
    cmd += [f"{ref}/src/{s}.c" for s in SOURCES] + ["-lm", "-ldl"]
    subprocess.run(cmd, check=True, stderr=subprocess.DEVNULL)
    model_dir = make_model(os.path.join(tmp, "model"))
    L = ctypes.CDLL(lib)
    L.sgl_gpt2_load.restype = ctypes.c_void_p
    L.sgl_gpt2_load.argtypes = [ctypes.c_char_p]
    m = L.sgl_gpt2_load(model_dir.encode())
    assert m, "reference failed to load the model folder"
    V = CONFIG["vocab_size"]
    toks = tokens()
    IntArr = ctypes.c_int * N_TOKENS
    pages = IntArr()
    L.sgl_gpt2_pages_alloc.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    assert L.sgl_gpt2_pages_alloc(m, pages, N_TOKENS) == 0
    L.sgl_gpt2_prefill.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int,
                                   ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                   ctypes.POINTER(ctypes.c_float)]
    tarr = IntArr(*toks)
    rows = []
    for n in range(1, N_TOKENS + 1):
        out = (ctypes.c_float * V)()
        assert L.sgl_gpt2_prefill(m, tarr, n, 0, pages, out) == 0
        rows.append(np.frombuffer(out, dtype=np.float32).copy())
    logits = np.stack(rows)
    # decode_batch after a shorter prefill must agree with the whole prefill
    n0 = N_TOKENS - 3
    out = (ctypes.c_float * V)()
    assert L.sgl_gpt2_prefill(m, tarr, n0, 0, pages, out) == 0
    L.sgl_gpt2_decode_batch.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int),
                                        ctypes.POINTER(ctypes.POINTER(ctypes.c_int)),
                                        ctypes.POINTER(ctypes.c_int), ctypes.c_int,
                                        ctypes.POINTER(ctypes.c_float)]
    dec_max = 0.0
    for i in range(n0, N_TOKENS):
        tok = (ctypes.c_int * 1)(toks[i])
        lens = (ctypes.c_int * 1)(i)
        ptrs = (ctypes.POINTER(ctypes.c_int) * 1)(ctypes.cast(pages, ctypes.POINTER(ctypes.c_int)))
        assert L.sgl_gpt2_decode_batch(m, tok, ptrs, lens, 1, out) == 0
        dec_max = max(dec_max, float(np.abs(np.frombuffer(out, dtype=np.float32) - logits[i]).max()))
    golden = {
        "source": "reference src/gpt2.c sgl_gpt2_prefill, compiled with gcc -O2 -fopenmp, float32",
        "config": CONFIG, "seed": SEED, "scheme": "varied", "tokens": toks,
        "weights_sha256": weights_digest(model_dir),
        "decode_batch_vs_prefill_max_abs": dec_max,
        # every 8th vocabulary column of every position keeps the file small
        "columns": list(range(0, V, 8)),
        "logits": [[float(f"{v:.9g}") for v in row[::8]] for row in logits],
        "argmax": [int(r.argmax()) for r in logits],
    }
    with open(os.path.join(HERE, "gpt2_tiny_reference.json"), "w") as f:
        json.dump(golden, f)
    print("wrote gpt2_tiny_reference.json; decode_batch vs prefill max abs diff:", dec_max)


if __name__ == "__main__":
    main()
