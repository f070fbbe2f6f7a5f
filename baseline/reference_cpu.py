"""The reference's own CPU code (integemjack/sglang.c: src/gpt2.c sgl_gpt2_prefill and
sgl_gpt2_decode_batch), unmodified, compiled with gcc -O2 -fopenmp and timed on this host's
cores at GPT-2 small's layer sizes with random weights: prefill of 2 x 1,024 tokens, decode
at batch 1 and 8 at a context of 512 (its decode batch holds 32 requests at most).

    python baseline/reference_cpu.py REFERENCE_TREE [--layers N]

Prints one JSON line.  With --layers the model has fewer layers (both numbers are printed);
time per layer is what scales.  Nothing of this repository's engine runs here; only its writer
of random model folders is used (the reference has none)."""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
SOURCES = ["gpt2", "ops", "tensor", "alloc", "log", "json", "safetensors", "gguf", "qweight", "sampling"]
SMALL = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=12, n_embd=768, n_head=12,
             vocab_size=50257, n_positions=1024, n_ctx=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("reference")
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--context", type=int, default=512)
    args = ap.parse_args()
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    tmp = tempfile.mkdtemp(prefix="sglc_cpu_")
    lib = os.path.join(tmp, "libsglref.so")
    ref = args.reference
    cmd = ["gcc", "-std=c11", "-O2", "-fopenmp", "-D_GNU_SOURCE", "-shared", "-fPIC", f"-I{ref}/include",
           f"-I{ref}/third_party/stb", "-o", lib] + [f"{ref}/src/{s}.c" for s in SOURCES] + ["-lm", "-ldl"]
    subprocess.run(cmd, check=True, stderr=subprocess.DEVNULL)
    cfg_d = dict(SMALL, n_layer=args.layers)
    arch = resolve_architecture(cfg_d)
    d = write_random_model(os.path.join(tmp, "model"), arch, arch.config_class.from_dict(cfg_d), 1234,
                           scheme="standard", store_dtype="float32")
    os.environ["SGL_POOL_SLOTS"] = "10240"      # its pool of one-position pages (4,096 by default) for 8 requests
    L = C.CDLL(lib)
    L.sgl_gpt2_load.restype = C.c_void_p
    L.sgl_gpt2_load.argtypes = [C.c_char_p]
    m = L.sgl_gpt2_load(d.encode())
    assert m, "the reference failed to load the model folder"
    P = C.POINTER(C.c_int)
    L.sgl_gpt2_pages_alloc.argtypes = [C.c_void_p, P, C.c_int]
    L.sgl_gpt2_prefill.argtypes = [C.c_void_p, P, C.c_int, C.c_int, P, C.POINTER(C.c_float)]
    L.sgl_gpt2_decode_batch.argtypes = [C.c_void_p, P, C.POINTER(P), P, C.c_int, C.POINTER(C.c_float)]
    V = SMALL["vocab_size"]
    rng = np.random.default_rng(3)
    out = {"impl": "reference CPU code (src/gpt2.c), gcc -O2 -fopenmp", "cores": os.cpu_count(),
           "n_layer": args.layers, "n_layer_full": 12, "context": args.context}
    # prefill: two prompts of 1,024 tokens, one call each (its prefill takes one request)
    n = 1024
    pages = [(C.c_int * n)() for _ in range(2)]
    for p in pages:
        assert L.sgl_gpt2_pages_alloc(m, p, n) == 0
    logits = (C.c_float * V)()
    toks = (C.c_int * n)(*[int(t) for t in rng.integers(0, V, size=n)])
    t0 = time.perf_counter()
    for p in pages:
        assert L.sgl_gpt2_prefill(m, toks, n, 0, p, logits) == 0
    dt = time.perf_counter() - t0
    out["prefill_2x1024_s"] = dt
    out["prefill_tok_s"] = 2 * n / dt
    # decode at a context of args.context: the pages above hold 1,024 positions; lengths say 512
    for B in (1, 8):
        reqs = pages[:1] * 1 if B == 1 else None
        if B > 2:
            more = [(C.c_int * n)() for _ in range(B - 2)]
            for p in more:
                assert L.sgl_gpt2_pages_alloc(m, p, n) == 0
                assert L.sgl_gpt2_prefill(m, toks, args.context, 0, p, logits) == 0
            reqs = pages + more
        reqs = reqs or pages[:B]
        tok = (C.c_int * B)(*[int(t) for t in rng.integers(0, V, size=B)])
        ptrs = (P * B)(*[C.cast(p, P) for p in reqs])
        blog = (C.c_float * (B * V))()
        steps = 5
        lens = (C.c_int * B)(*([args.context] * B))
        assert L.sgl_gpt2_decode_batch(m, tok, ptrs, lens, B, blog) == 0        # warm-up
        t0 = time.perf_counter()
        for s in range(steps):
            lens = (C.c_int * B)(*([args.context + 1 + s] * B))
            assert L.sgl_gpt2_decode_batch(m, tok, ptrs, lens, B, blog) == 0
        dt = (time.perf_counter() - t0) / steps
        out[f"decode_b{B}_ms_per_step"] = dt * 1e3
        out[f"decode_b{B}_tok_s"] = B / dt
    print(json.dumps(out))


if __name__ == "__main__":
    main()
