"""The runtime: device, precision, and the choice of kernel for each operation.

"float32": weights, activations and cache in 32-bit, every product by plain
FFMA kernels (no tensor-core mode).  "bfloat16": matrices, activations and
cache in bfloat16 with 32-bit accumulation; the residual stream, norms' and
softmax statistics stay 32-bit in both.
"""
import torch

from ..csrc import ops

_NAMES = {"float32": "float32", "fp32": "float32", "f32": "float32",
          "bfloat16": "bfloat16", "bf16": "bfloat16"}


class Runtime:
    def __init__(self, dtype="bfloat16", device="cuda:0"):
        if dtype not in _NAMES:
            raise ValueError(f"dtype '{dtype}' is not handled; choose float32 or bfloat16")
        self.dtype = _NAMES[dtype]
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("this engine runs on a CUDA device only (no CPU path)")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; this engine has no CPU path")
        if self.device.index is not None and self.device.index >= torch.cuda.device_count():
            raise RuntimeError(f"device {device}: this machine has {torch.cuda.device_count()} CUDA device(s)")
        # the kernels are launched through ctypes on the current device's current stream: make
        # the runtime's device the current one (for this thread), or launches and tensors part ways
        torch.cuda.set_device(self.device)
        t = torch.float32 if self.dtype == "float32" else torch.bfloat16
        self.matrix_dtype = t
        self.act_dtype = t
        self.cache_dtype = t

    @property
    def cache_dtype_name(self):
        return self.dtype

    def make_tensor(self, shape, dtype_name):
        dt = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}[dtype_name]
        return torch.zeros(shape, dtype=dt, device=self.device)

    # -- kernel choice --------------------------------------------------------
    def gemm(self, a, w, bias, out=None, residual=None, act=None, few_ok=False):
        if self.dtype == "bfloat16" and ops.gemm_tc_supported(a, w):
            # one or two tokens, and every matrix of the model's layers small (few_ok: the step
            # context says so for the model it runs): the kernel without any exchange between
            # blocks.  (Its blocks are heavy; beside the lighter kernels that wider matrices need
            # it lengthens the step, so the choice is made for the model, not for the product.)
            if few_ok and a.shape[0] <= ops.FEW_MAX_TOKENS and w.numel() <= ops.FEW_MAX_WEIGHT:
                return ops.gemm_few(a, w, bias, out=out, residual=residual, act=act)
            return ops.gemm_tc(a, w, bias, out=out, residual=residual, act=act, supported=True)
        return ops.gemm_simt(a, w, bias, out=out, residual=residual, act=act)

    def project_qkv(self, ctx, h, linear, qkv, binding, grp, n_heads, n_kv_heads, head_dim):
        """qkv = h·Wᵀ + b for a mixer that owns its cache.  In a step with prompt portions the
        tensor-core product writes the keys and values into the cache from its epilogue (they
        are not needed in `qkv` then: the attention kernels of such a step read the cache);
        returns whether it did, for attend()."""
        if self.dtype == "bfloat16" and binding.write and ctx.max_q_len > 1 \
                and ops.gemm_tc_kv(h, linear.weight, linear.bias, qkv, binding.tensor, grp.slots, n_heads,
                                   n_kv_heads, head_dim):
            return True
        linear.forward(ctx, h, out=qkv)
        return False

    def attend(self, ctx, q, k, v, binding, grp, out, n_heads, n_kv_heads, head_dim, scale, window,
               kv_written=False):
        """Put the step's keys and values into the cache (if this call owns it and project_qkv
        has not done so already) and run causal attention of the step's queries over the cache."""
        cache = binding.tensor
        bf16_ok = self.dtype == "bfloat16" and head_dim % 8 == 0 and q.stride(0) % 8 == 0 \
            and q.data_ptr() % 16 == 0
        if bf16_ok and ctx.max_q_len == 1:
            # every request brings one token: keys split across blocks; the same launch writes
            # the new keys and values when this call owns the cache
            fuse = binding.write and k.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0
            if binding.write and not fuse:
                ops.kv_write(k, v, cache, grp.slots, n_kv_heads, head_dim)
            # (token t is the step's t-th request, so no token -> request table is passed)
            return ops.attention_decode(q, cache, grp.block_table, None, ctx.positions, out,
                                        n_heads, scale, window, ctx.max_keys,
                                        k_new=k if fuse else None, v_new=v if fuse else None,
                                        slots=grp.slots if fuse else None,
                                        token_list=ctx.decode_tokens if ctx.decode_ordered else None,
                                        n_tokens=ctx.T)
        if binding.write and not kv_written:
            ops.kv_write(k, v, cache, grp.slots, n_kv_heads, head_dim)
        if bf16_ok and ops.attention_prefill_tc_supported(q, cache, scale) \
                and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0:
            # prompt portions in 128-query tiles on the tensor cores; single decoded tokens beside
            # them go to the split-key kernel (a tile of one query would waste the other 127 rows)
            split = ctx.n_decode > 0
            ops.attention_prefill_tc(q, cache, grp.block_table, ctx.q_start, ctx.kv_len, out, n_heads,
                                     scale, window, ctx.R, ctx.max_q_len, skip_single=split)
            if split:
                ops.attention_decode(q, cache, grp.block_table, ctx.token_req, ctx.positions, out, n_heads,
                                     scale, window, ctx.max_keys, token_list=ctx.decode_tokens,
                                     n_tokens=ctx.n_decode)
            return
        ops.attention_simt(q, cache, grp.block_table, ctx.token_req, ctx.positions, out, n_heads,
                           scale, window, ctx.max_keys, max_q_len=ctx.max_q_len)
