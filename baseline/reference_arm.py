"""The reference arm of the bench: integemjack/sglang.c's own GPT-2 GPU path, unmodified,
timed on the workload of `bench.py`.

Nothing of this repository's engine, models or kernels is on this path.  The reference is
a C/CUDA project without a Python package, so "installing" it means compiling it: its
`src/cuda_backend.cu` with nvcc and the C files its GPT-2 route needs with gcc, linked
with cuBLAS into `baseline/_ref/libsgl_ref.so` (from an unmodified copy of the sources
kept beside it).  The library is driven through the reference's public C API with ctypes:

    sgl_gpt2_load -> sgl_cuda_from_gpt2 -> sgl_cuda_forward_seg        (include/sgl/cuda.h:30-36)

which is what its own command line does (apps/cuda_cli.c:69-145): one forward of the whole
prompt, then one forward of a single token per generated token, logits copied to the host
every call and the next token chosen on the host (`sgl_sample_greedy`).  The reference has
no batched GPT-2 decode on the GPU (src/cuda_backend.cu:6452-6464 is llama arithmetic), so a
decode step of B requests is B such single-token forwards, each in its own segment of the
contiguous cache (`kv_base`), exactly as its API offers.  The cache is one contiguous array
of `n_ctx` rows for all segments, so the model folder written for this arm has a position
table of B x segment rows (positions inside a segment stay below 1,024; the extra rows are
never read).  Weights are float32 (the reference's default on the GPU); a second run with
its `SGL_CUDA_FP16=1` switch (half-precision weights, float32 cache) is reported beside it.

Times are wall-clock around the API calls: every call ends with the reference's own stream
synchronisation and a copy of the logits to the host, so host time is device time plus its
launch overhead, which is the number a user of that API gets.
"""
import ctypes
import json
import os
import shutil
import struct
import subprocess
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(REF_DIR, "libsgl_ref.so")
C_SOURCES = ["gpt2", "ops", "tensor", "alloc", "log", "json", "safetensors", "gguf", "qweight", "sampling"]
CU_SOURCES = ["cuda_backend"]
SEGMENT = 640           # rows of the contiguous cache per decoding request (context 512 + steps)


class Unavailable(RuntimeError):
    pass


def build(ref_tree="/root/reference", verbose=False):
    """Compile the reference (unmodified) into baseline/_ref/libsgl_ref.so, from a copy of its
    sources under baseline/_ref/src.  Returns the library's path."""
    if os.path.exists(LIB):
        return LIB
    src_copy = os.path.join(REF_DIR, "src")
    if not os.path.isdir(os.path.join(src_copy, "src")):
        if not os.path.isdir(os.path.join(ref_tree, "src")):
            raise Unavailable(f"no reference tree at {ref_tree} and no copy under baseline/_ref/src")
        os.makedirs(src_copy, exist_ok=True)
        for sub in ("include", "third_party/stb"):
            shutil.copytree(os.path.join(ref_tree, sub), os.path.join(src_copy, sub), dirs_exist_ok=True)
        os.makedirs(os.path.join(src_copy, "src"), exist_ok=True)
        for s in C_SOURCES:
            shutil.copy(os.path.join(ref_tree, "src", s + ".c"), os.path.join(src_copy, "src"))
        for s in CU_SOURCES:
            shutil.copy(os.path.join(ref_tree, "src", s + ".cu"), os.path.join(src_copy, "src"))
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise Unavailable("nvcc not found: the reference's CUDA backend cannot be compiled")
    obj = os.path.join(REF_DIR, "obj")
    os.makedirs(obj, exist_ok=True)
    inc = [f"-I{src_copy}/include", f"-I{src_copy}/third_party/stb"]
    quiet = None if verbose else subprocess.DEVNULL
    objs = []
    for s in CU_SOURCES:
        o = os.path.join(obj, s + ".o")
        # the reference's own flags (CMakeLists.txt:297-302) with this GPU's architecture
        subprocess.run([nvcc, "-O2", "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC"]
                       + inc + ["-c", os.path.join(src_copy, "src", s + ".cu"), "-o", o],
                       check=True, stdout=quiet, stderr=quiet)
        objs.append(o)
    for s in C_SOURCES:
        o = os.path.join(obj, s + ".o")
        subprocess.run(["gcc", "-std=c11", "-O2", "-fopenmp", "-D_GNU_SOURCE", "-fPIC"] + inc
                       + ["-c", os.path.join(src_copy, "src", s + ".c"), "-o", o],
                       check=True, stdout=quiet, stderr=quiet)
        objs.append(o)
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
    subprocess.run(["g++", "-shared", "-fopenmp", "-o", LIB] + objs
                   + [f"-L{cuda_lib}", f"-Wl,-rpath,{cuda_lib}", "-lcublas", "-lcudart", "-lm", "-ldl"],
                   check=True, stdout=quiet, stderr=quiet)
    return LIB


# ---------------------------------------------------------------------------
def _write_safetensors(path, tensors):
    header, off = {}, 0
    for name, a in tensors.items():
        header[name] = {"dtype": "F32", "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        off += a.nbytes
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * (-len(hb) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for a in tensors.values():
            f.write(np.ascontiguousarray(a, dtype=np.float32).tobytes())


def write_model(out_dir, cfg, n_ctx, seed=1234):
    """A float32 model folder with the bench's layer sizes and init scheme (matrices N(0, 0.02),
    projections into the residual stream N(0, 0.02/sqrt(2L)), zero biases, gains 1), written
    with numpy alone.  `n_ctx` rows of position table (see the module's header)."""
    rng = np.random.default_rng(seed)
    E, L, V = cfg["n_embd"], cfg["n_layer"], cfg["vocab_size"]
    I = 4 * E                                             # the reference knows no other width
    nrm = lambda shape, std: (rng.standard_normal(shape, dtype=np.float32) * np.float32(std))
    t = {"wte.weight": nrm((V, E), 0.02), "wpe.weight": nrm((n_ctx, E), 0.02),
         "ln_f.weight": np.ones(E, np.float32), "ln_f.bias": np.zeros(E, np.float32)}
    rs = 0.02 / np.sqrt(2.0 * L)
    for l in range(L):
        p = f"h.{l}."
        t[p + "ln_1.weight"] = np.ones(E, np.float32)
        t[p + "ln_1.bias"] = np.zeros(E, np.float32)
        t[p + "attn.c_attn.weight"] = nrm((E, 3 * E), 0.02)
        t[p + "attn.c_attn.bias"] = np.zeros(3 * E, np.float32)
        t[p + "attn.c_proj.weight"] = nrm((E, E), rs)
        t[p + "attn.c_proj.bias"] = np.zeros(E, np.float32)
        t[p + "ln_2.weight"] = np.ones(E, np.float32)
        t[p + "ln_2.bias"] = np.zeros(E, np.float32)
        t[p + "mlp.c_fc.weight"] = nrm((E, I), 0.02)
        t[p + "mlp.c_fc.bias"] = np.zeros(I, np.float32)
        t[p + "mlp.c_proj.weight"] = nrm((I, E), rs)
        t[p + "mlp.c_proj.bias"] = np.zeros(E, np.float32)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump({"model_type": "gpt2", "architectures": ["GPT2LMHeadModel"], "n_layer": L,
                   "n_head": cfg["n_head"], "n_embd": E, "n_ctx": n_ctx, "n_positions": n_ctx,
                   "vocab_size": V, "layer_norm_epsilon": cfg["layer_norm_epsilon"]}, f)
    _write_safetensors(os.path.join(out_dir, "model.safetensors"), t)
    return out_dir


class Reference:
    """ctypes view of the reference's public API (include/sgl/gpt2.h, include/sgl/cuda.h)."""

    def __init__(self, lib_path, model_dir, fp16=False):
        os.environ["SGL_POOL_SLOTS"] = "64"              # its CPU cache pool is not used here
        if fp16:
            os.environ["SGL_CUDA_FP16"] = "1"
        else:
            os.environ.pop("SGL_CUDA_FP16", None)
        L = self.L = ctypes.CDLL(lib_path)
        L.sgl_gpt2_load.restype = ctypes.c_void_p
        L.sgl_gpt2_load.argtypes = [ctypes.c_char_p]
        L.sgl_gpt2_free.argtypes = [ctypes.c_void_p]
        L.sgl_cuda_from_gpt2.restype = ctypes.c_void_p
        L.sgl_cuda_from_gpt2.argtypes = [ctypes.c_void_p]
        L.sgl_cuda_free.argtypes = [ctypes.c_void_p]
        L.sgl_cuda_vocab.argtypes = [ctypes.c_void_p]
        L.sgl_cuda_ctx.argtypes = [ctypes.c_void_p]
        L.sgl_cuda_forward_seg.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int,
                                           ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_float)]
        L.sgl_sample_greedy.argtypes = [ctypes.POINTER(ctypes.c_float), ctypes.c_int]
        self.cpu = L.sgl_gpt2_load(model_dir.encode())
        if not self.cpu:
            raise Unavailable("the reference's sgl_gpt2_load refused the model folder")
        self.gpu = L.sgl_cuda_from_gpt2(self.cpu)
        if not self.gpu:
            raise Unavailable("the reference's sgl_cuda_from_gpt2 failed")
        self.V = L.sgl_cuda_vocab(self.gpu)
        self.ctx = L.sgl_cuda_ctx(self.gpu)
        self.logits = (ctypes.c_float * self.V)()

    def forward(self, tokens, pos0, kv_base, want_logits=True):
        n = len(tokens)
        arr = (ctypes.c_int * n)(*tokens)
        rc = self.L.sgl_cuda_forward_seg(self.gpu, arr, n, pos0, kv_base,
                                         self.logits if want_logits else None)
        if rc != 0:
            raise RuntimeError(f"sgl_cuda_forward_seg returned {rc} (n={n}, pos0={pos0}, kv_base={kv_base})")

    def greedy(self):
        return self.L.sgl_sample_greedy(self.logits, self.V)

    def close(self):
        self.L.sgl_cuda_free(self.gpu)
        self.L.sgl_gpt2_free(self.cpu)
        self.gpu = self.cpu = None


def time_decode(ref, batch, context, steps, warmup, seed=0):
    """tokens/s of `steps` decode steps of `batch` requests at `context` tokens each: every
    step is one single-token forward per request, greedy choice on the host."""
    rng = np.random.default_rng(seed + batch)
    for i in range(batch):
        ref.forward([int(t) for t in rng.integers(0, ref.V, size=context)], 0, i * SEGMENT)
    toks = [ref.greedy()] * batch
    lens = [context] * batch

    def step():
        for i in range(batch):
            ref.forward([toks[i]], lens[i], i * SEGMENT)
            toks[i] = ref.greedy()
            lens[i] += 1

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return batch * steps / dt, dt / steps * 1e3


def time_prefill(ref, n_prompts, prompt_len, reps, warmup, seed=0):
    rng = np.random.default_rng(seed)
    times = []
    for it in range(warmup + reps):
        prompts = [[int(t) for t in rng.integers(0, ref.V, size=prompt_len)] for _ in range(n_prompts)]
        t0 = time.perf_counter()
        for i, p in enumerate(prompts):
            ref.forward(p, 0, i * prompt_len)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt * 1e3)
    return sorted(times)[len(times) // 2]


def run(cfg, batch, context, steps, warmup, prefill_tokens, peaks, prefill_flops, decode_bytes,
        clock_sampler=None, points=(1, 64)):
    """The reference's numbers on the bench's workload, as the dict of the bench's JSON line."""
    import tempfile
    lib = build()
    tmp = tempfile.mkdtemp(prefix="sglc_ref_")
    try:
        n_ctx = max(max(points + (batch,)) * SEGMENT, prefill_tokens)
        model_dir = write_model(os.path.join(tmp, "model"), cfg, n_ctx)
        out = None
        for fp16 in (False, True):
            ref = Reference(lib, model_dir, fp16=fp16)
            time_decode(ref, 1, 32, 2, 2)                         # warm its kernels and workspaces
            if clock_sampler is not None and not fp16:
                clock_sampler.start()
            value, ms = time_decode(ref, batch, context, steps, warmup)
            pms = time_prefill(ref, 2, prefill_tokens // 2, 3, 2)
            pts = {}
            for b in points:
                pts[f"decode_b{b}"], _ = time_decode(ref, b, context, max(2, min(steps, 8)), 2)
            ref.close()
            elem = 2 if fp16 else 4
            nbytes = decode_bytes(elem)
            res = {"value": value, "ms_per_step": ms,
                   "prefill": {"value": prefill_tokens / (pms / 1e3), "tokens": prefill_tokens, "ms": pms,
                               "frac": prefill_flops / (pms / 1e3) / (peaks["bf16_tflops"] * 1e12)},
                   "roofline": {"bound": "hbm", "achieved": nbytes / (ms / 1e3) / 1e9, "peak": peaks["hbm_gbs"],
                                "unit": "GB/s", "frac": nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"]},
                   "points": pts}
            if not fp16:
                out = res
                out["clocks"] = clock_sampler.stop() if clock_sampler is not None else None
            else:
                out["fp16_weights"] = res
        return out
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
