"""The decode-attention entry point that allocates nothing, called through its exported C
symbol, against the ordinary entry point, on two calls in a row.

Some users of the library cannot call cudaMalloc where they run (a plug-in or real-time loop
that may not allocate after start-up, a fixed memory budget); for them the kernel's merge
scratch is an array built into the library.  This file is collected last on purpose: if it
fails, a run that stops at the first failure has already run every other test."""
import ctypes
import math

import pytest
import torch

from test_kernels_gpu import _attention_reference, _paged_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2          # the tolerance the other bfloat16 attention tests use


def _call(lib, c, out, H, scale, window, max_keys, n_splits):
    n_pages, two, Hkv, ps, D = c["cache"].shape
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    return lib.sglc_attention_decode_noalloc(
        p(c["q"]), c["q"].stride(0), p(c["cache"]), p(c["bt"]), c["bt"].stride(0), p(c["token_req"]),
        p(c["positions"]), p(out), out.stride(0), c["q"].shape[0], H, Hkv, D, ps, ctypes.c_float(scale),
        int(window or 0), int(max_keys), int(n_splits),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from sglang_c_b200.csrc import build, ops
    lib = build.load("attention_decode")
    lib.sglc_attention_decode_noalloc_error.restype = ctypes.c_char_p
    cases = [([700, 33, 130], 6, 2, 64, 16, None, 12), ([300, 512], 4, 4, 128, 16, 200, 5),
             ([64], 3, 3, 16, 8, None, 1)]
    for lens, H, Hkv, D, ps, window, n_splits in cases:
        c = _paged_case(lens, [1] * len(lens), H, Hkv, D, ps, torch.bfloat16, seed=len(lens) + D)
        scale = 1.0 / math.sqrt(D)
        T = c["q"].shape[0]
        want = torch.empty(T, H * D, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], want, H, scale,
                             window, max(lens))
        ref = _attention_reference(c, H, Hkv, D, scale, window)
        outs = [torch.full_like(want, float("nan")) for _ in range(3)]
        # a first call looks the scratch's address up; what the device has free is read after it,
        # from the driver (cudaMemGetInfo: the caching allocator's own counters would not see a
        # cudaMalloc made inside the library)
        rc = _call(lib, c, outs[2], H, scale, window, max(lens), n_splits)
        assert rc == 0, lib.sglc_attention_decode_noalloc_error(rc).decode()
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]
        for out in outs[:2]:                     # two calls in a row share the scratch
            rc = _call(lib, c, out, H, scale, window, max(lens), n_splits)
            assert rc == 0, lib.sglc_attention_decode_noalloc_error(rc).decode()
        assert lib.sglc_attention_decode_noalloc_check(
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
        assert torch.cuda.mem_get_info()[0] == free0, "the device's free memory moved during the calls"
        outs = outs[:2]
        for out in outs:
            assert float((out.float() - want.float()).abs().max()) < TOL
            assert float((out.double().cpu() - ref).abs().max()) < TOL
        assert torch.equal(outs[0], outs[1])


def test_no_alloc_entry_point_flags_a_position_beyond_max_keys():
    """A caller's max_keys smaller than a token's position + 1: that token's rows are zeros and the
    status word says so; the other token is computed as ever."""
    from sglang_c_b200.csrc import build, ops
    lib = build.load("attention_decode")
    H, Hkv, D, ps = 4, 2, 64, 16
    c = _paged_case([200, 40], [1, 1], H, Hkv, D, ps, torch.bfloat16, seed=9)
    scale = 1.0 / math.sqrt(D)
    want = torch.empty(2, H * D, dtype=torch.bfloat16, device=DEV)
    ops.attention_decode(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], want, H, scale, None, 200)
    out = torch.full_like(want, float("nan"))
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert _call(lib, c, out, H, scale, None, 48, 2) == 0          # 48 keys cover the second token only
    assert lib.sglc_attention_decode_noalloc_check(stream) == -12
    assert lib.sglc_attention_decode_noalloc_check(stream) == 0     # cleared by the report
    assert float(out[0].float().abs().max()) == 0.0
    assert float((out[1].float() - want[1].float()).abs().max()) < TOL


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from sglang_c_b200.csrc import build
    lib = build.load("attention_decode")
    lib.sglc_attention_decode_noalloc_error.restype = ctypes.c_char_p
    c = _paged_case([40], [1], 2, 2, 64, 16, torch.bfloat16, seed=1)
    out = torch.zeros(1, 128, dtype=torch.bfloat16, device=DEV)
    # claim far more (token, head) pairs than the built-in scratch holds: nothing is launched
    n_pages, two, Hkv, ps, D = c["cache"].shape
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.sglc_attention_decode_noalloc(
        p(c["q"]), c["q"].stride(0), p(c["cache"]), p(c["bt"]), c["bt"].stride(0), p(c["token_req"]),
        p(c["positions"]), p(out), out.stride(0), 100000, 2, Hkv, D, ps, ctypes.c_float(0.125), 0, 40, 4,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -10
    assert b"built-in scratch" in lib.sglc_attention_decode_noalloc_error(rc)
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
