"""The C++ walker makes a step's launches for a model of built-in parts; the Python forward pass
makes them for every other model.  Both choose the same kernels with the same arguments, so their
logits are equal bit for bit, in every cut and in both precisions."""
import numpy as np
import pytest
import torch

import traces
from conftest import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu


def _run(d, dtype, name, steps, walker, graphs):
    from sglang_c_b200.engine import Engine, StepEntry
    eng = Engine.from_dir(d, dtype=dtype, page_size=PAGE_SIZE[name], n_pages=traces.peak_tokens(steps) // PAGE_SIZE[name],
                          max_requests=8, max_step_tokens=1024, use_host_walker=walker, use_graphs=graphs)
    outs = []
    for st in steps:
        for e in st["entries"]:
            if not eng.has_request(e["id"]):
                eng.add_request(e["id"])
        lg = eng.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]])
        outs.append(lg.clone())
        for rid in st["end"]:
            eng.end_request(rid)
    eng.check_device_errors()
    return outs, eng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_walker_and_python_forward_give_the_same_bits(model_dirs, name, dtype):
    d = model_dirs(name, dtype)
    V = TINY[name]["vocab_size"]
    lens = {"A": [37, 64, 90, 21, 128], "B": [50, 1, 130, 77, 200, 9], "C": [300, 129, 520, 64, 260]}[name]
    reqs = {f"w{i}": traces.random_tokens(60 + i, n, V) for i, n in enumerate(lens)}
    prompt_len = {rid: max(1, len(t) - 20) for rid, t in reqs.items()}
    for steps in (traces.whole(reqs), traces.tail_decoded(reqs), traces.mixed(reqs, prompt_len, seed=2)):
        a, ea = _run(d, dtype, name, steps, True, False)
        b, eb = _run(d, dtype, name, steps, False, False)
        assert ea._host is not None and eb._host is None
        for x, y in zip(a, b):
            assert torch.equal(x, y)
        # and under graph capture and replay (the walker's launches are captured like any others;
        # a graph is launched for a rounded-up bound of the context, which may pick other key
        # ranges than the eager step, so graph runs are compared with graph runs)
        c, ec = _run(d, dtype, name, steps, True, True)
        e, ee = _run(d, dtype, name, steps, False, True)
        for x, y in zip(c, e):
            assert torch.equal(x, y)


def test_walker_declines_models_it_cannot_describe(model_dirs):
    """A part from outside the package: the engine falls back to the Python forward pass."""
    from sglang_c_b200.engine import Engine
    from sglang_c_b200.engine.host_model import HostModel
    from sglang_c_b200.parts import Part, register_part

    @register_part("norm", "toy_identity_gain_for_walker_test")
    class OddNorm(Part):
        @classmethod
        def declare_weights(cls, params):
            return {}

        def forward(self, ctx, x, out, rows=None):
            src = x if rows is None else x[rows.long()]
            out.copy_(src[:out.shape[0]].to(out.dtype))
            return out

    d = model_dirs("A", "float32")
    eng = Engine.from_dir(d, dtype="float32", page_size=16, n_pages=8, max_requests=2, max_step_tokens=64)
    assert HostModel.build(eng.model, eng.cache, 16) is not None
    eng.model.layers[0].parts["norm1"] = OddNorm({"size": 64}, eng.rt)
    eng.model.layers[0].norm1 = eng.model.layers[0].parts["norm1"]
    assert HostModel.build(eng.model, eng.cache, 16) is None
