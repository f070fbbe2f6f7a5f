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
