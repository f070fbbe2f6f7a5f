"""Failure detection on the device, without a fault: a wait that nothing completes runs into its
limit, the kernel leaves in order and the host finds the error word."""
import pytest
import torch

import traces
from conftest import TINY

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_engine_goes_on(model_dirs):
    from sglang_c_b200.csrc import ops
    from sglang_c_b200.engine import Engine, StepEntry
    d = model_dirs("A", "bfloat16")
    eng = Engine.from_dir(d, dtype="bfloat16", page_size=16, n_pages=8, max_requests=2, max_step_tokens=64)
    toks = traces.random_tokens(1, 20, TINY["A"]["vocab_size"])
    eng.add_request("a")
    before = eng.step([StepEntry("a", toks, [19])]).clone()
    eng.check_device_errors()                          # nothing wrong so far
    # the probes: a block whose wait runs out; a cluster whose first block waits for a peer that
    # never signals and leaves only after that peer has gone
    trace = ops.wait_probe(eng.rt.device, polls=300)
    assert trace == [2, 2, 2, 1, 1], trace
    with pytest.raises(RuntimeError, match="bounded wait"):
        eng.check_device_errors()
    eng.check_device_errors()                          # the word was cleared by the report
    # the context is intact: the same step on a fresh request gives the same logits
    eng.add_request("b")
    after = eng.step([StepEntry("b", toks, [19])])
    assert torch.equal(before, after)
    eng.check_device_errors()


def test_bounds_check_build_skips_and_flags_a_bad_page_id(model_dirs):
    """The kernels built with bounds checks give the same logits as the ordinary build, and a page
    id beyond the pool (put into the step's block table behind the engine's back, where only a
    kernel can meet it) is skipped and reported instead of dereferenced."""
    from sglang_c_b200.csrc import build
    from sglang_c_b200.engine import Engine, StepEntry
    toks = traces.random_tokens(2, 40, TINY["A"]["vocab_size"])
    for dtype in ("float32", "bfloat16"):
        d = model_dirs("A", dtype)
        plain = Engine.from_dir(d, dtype=dtype, page_size=16, n_pages=8, max_requests=2, max_step_tokens=64)
        plain.add_request("a")
        want = plain.step([StepEntry("a", toks[:39], [38])]).clone()
        want2 = plain.step([StepEntry("a", toks[39:], [0])]).clone()
        build.set_bounds_check(True)
        try:
            eng = Engine.from_dir(d, dtype=dtype, page_size=16, n_pages=8, max_requests=2, max_step_tokens=64,
                                  use_graphs=False)
            eng.add_request("a")
            assert torch.equal(eng.step([StepEntry("a", toks[:39], [38])]), want)
            assert torch.equal(eng.step([StepEntry("a", toks[39:], [0])]), want2)
            eng.check_device_errors()
            # the next step's block table gets a page id far beyond the pool after the host's checks:
            # the upload is what a kernel reads
            upload = eng.bufs.upload

            def corrupt(*a, **k):
                eng.bufs.npview("bt0").reshape(eng.max_requests, eng.b_cap)[0, 0] = 1 << 20
                return upload(*a, **k)

            eng.bufs.upload = corrupt
            eng.step([StepEntry("a", [toks[0]], [0])])
            eng.bufs.upload = upload
            with pytest.raises(RuntimeError, match="outside its range"):
                eng.check_device_errors()
            eng.check_device_errors()
        finally:
            build.set_bounds_check(False)


def test_a_step_that_fails_half_way_is_rolled_back(model_dirs):
    """A launch that raises in the middle of a step (made to, on the host): the requests had been
    grown for the step's tokens, whose keys and values were never all written; the growth is taken
    back, pages return, and the same step run again gives what an undisturbed engine gives."""
    from sglang_c_b200.csrc import ops
    from sglang_c_b200.engine import Engine, StepEntry
    d = model_dirs("A", "float32")
    toks = traces.random_tokens(2, 40, TINY["A"]["vocab_size"])
    kw = dict(dtype="float32", page_size=16, n_pages=8, max_requests=2, max_step_tokens=64)
    eng = Engine.from_dir(d, use_host_walker=False, use_graphs=False, **kw)
    eng.add_request("a")
    eng.step([StepEntry("a", toks[:20], [])])
    free = eng.cache.n_free_pages()
    real, calls = eng.rt.gemm, [0]

    def failing(*a, **k):
        calls[0] += 1
        if calls[0] == 6:                      # in the second layer: the first has written its cache
            raise ops.KernelError("made to fail")
        return real(*a, **k)

    eng.rt.gemm = failing
    with pytest.raises(ops.KernelError, match="made to fail"):
        eng.step([StepEntry("a", toks[20:], [19])])
    eng.rt.gemm = real
    assert eng.length("a") == 20 and eng.cache.n_free_pages() == free
    eng.cache.check()
    again = eng.step([StepEntry("a", toks[20:], [19])]).clone()
    ref = Engine.from_dir(d, **kw)
    ref.add_request("a")
    assert torch.equal(again, ref.step([StepEntry("a", toks, [39])]))
