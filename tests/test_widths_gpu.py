"""The layer widths of GPT-2 small, medium and XL (two layers deep, a small vocabulary so that
the plain implementation stays quick): widths and head counts that are no power of two (1600
wide, 25 heads, 6400 inner) through the real kernels, whole and cut, in both precisions."""
import numpy as np
import pytest

import plain_gpt2
import traces

pytestmark = pytest.mark.gpu

WIDTHS = {
    "small": dict(n_embd=768, n_head=12, n_inner=3072),
    "medium": dict(n_embd=1024, n_head=16, n_inner=4096),
    "xl": dict(n_embd=1600, n_head=25, n_inner=6400),
}
# logits of these models are a few tenths in size (standard init, vocabulary rows N(0, 0.02))
TOL = {"float32": 5e-5, "bfloat16": 2e-2}


@pytest.fixture(scope="module")
def width_dirs(tmp_path_factory):
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    base = tmp_path_factory.mktemp("widths")
    made = {}

    def get(name, store):
        if (name, store) not in made:
            d = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, vocab_size=1031,
                     n_positions=512, layer_norm_epsilon=1e-5, activation_function="gelu_new", **WIDTHS[name])
            arch = resolve_architecture(d)
            made[(name, store)] = write_random_model(str(base / f"{name}_{store}"), arch,
                                                     arch.config_class.from_dict(d), 9, scheme="varied",
                                                     store_dtype=store)
        return made[(name, store)]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "medium", "xl"])
def test_real_widths_whole_and_cut(width_dirs, tmp_path, name, dtype):
    from sglang_c_b200.engine import Engine
    from sglang_c_b200.engine.replay import replay
    d = width_dirs(name, dtype)
    reqs = {"a": traces.random_tokens(1, 150, 1031), "b": traces.random_tokens(2, 37, 1031),
            "c": traces.random_tokens(3, 260, 1031)}
    ref = {rid: plain_gpt2.forward_dir(d, toks) for rid, toks in reqs.items()}
    prompt_len = {"a": 130, "b": 20, "c": 250}
    for mode, steps in (("whole", traces.whole(reqs)), ("mixed", traces.mixed(reqs, prompt_len, seed=2))):
        eng = Engine.from_dir(d, dtype=dtype, page_size=16, n_pages=traces.peak_tokens(steps) // 16,
                              max_requests=4, max_step_tokens=512)
        out = str(tmp_path / mode)
        replay(eng, traces.to_lines(steps), out)
        got = traces.collect(steps, out, 1031)
        err, where = traces.max_error(got, ref)
        assert err < TOL[dtype], f"{name} {mode}: max error {err} at {where}"
        eng.check_device_errors()


def test_many_single_tokens_of_unequal_contexts(width_dirs, tmp_path):
    """Sixteen requests of 12 heads decode together: enough (token, head) items for the streaming
    decode attention, with contexts from 20 to 330 tokens, so that the step lists its tokens
    longest first and the kernel's blocks take them in that order."""
    from sglang_c_b200.engine import Engine
    from sglang_c_b200.engine.replay import replay
    d = width_dirs("small", "bfloat16")
    rng = np.random.default_rng(5)
    lens = [int(n) for n in rng.permutation(np.linspace(20, 330, 16).astype(int))]
    n_tail = 5
    reqs = {f"r{i}": traces.random_tokens(40 + i, n + n_tail, 1031) for i, n in enumerate(lens)}
    ref = {rid: plain_gpt2.forward_dir(d, toks) for rid, toks in reqs.items()}
    steps = []
    ids = list(reqs)
    for g in range(0, 16, 4):                 # prompts, four requests a step
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": rid, "tokens": reqs[rid][:lens[ids.index(rid)]],
                                   "want": list(range(lens[ids.index(rid)]))} for rid in ids[g:g + 4]]})
    for k in range(n_tail):                   # then all sixteen, one token each
        steps.append({"step": len(steps), "end": ids if k == n_tail - 1 else [],
                      "entries": [{"id": rid, "tokens": [reqs[rid][lens[i] + k]], "want": [0]}
                                  for i, rid in enumerate(ids)]})
    eng = Engine.from_dir(d, dtype="bfloat16", page_size=16, n_pages=traces.peak_tokens(steps) // 16,
                          max_requests=16, max_step_tokens=1024)
    out = str(tmp_path / "out")
    replay(eng, traces.to_lines(steps), out)
    got = traces.collect(steps, out, 1031)
    err, where = traces.max_error(got, ref)
    assert err < TOL["bfloat16"], f"max error {err} at {where}"
    eng.check_device_errors()


def test_scheduler_decodes_unequal_contexts_at_small_width(width_dirs):
    """Greedy generation through the scheduler for sixteen prompts of 20 to 330 tokens at 12
    heads: steady decoding runs ahead of the host, on the streaming decode attention with the
    tokens listed longest context first.  A token other than the plain implementation's is
    accepted only at a near tie of the plain logits."""
    from sglang_c_b200.engine import generate, sched_new
    from sglang_c_b200.sampling import SamplingParams
    d = width_dirs("small", "bfloat16")
    rng = np.random.default_rng(11)
    lens = [int(n) for n in rng.permutation(np.linspace(20, 330, 16).astype(int))]
    prompts = [traces.random_tokens(300 + i, n, 1031) for i, n in enumerate(lens)]
    s = sched_new(d, dtype="bfloat16", page_size=16, max_tokens=16 * 384, max_requests=16,
                  max_step_tokens=1024)
    got = generate(s, prompts, SamplingParams(temperature=0.0), max_new=8)
    cfg, w = plain_gpt2.read_model_dir(d)
    for p, g in zip(prompts, got):
        assert len(g) == 8
        seq = list(p)
        for t in g:
            lg = plain_gpt2.forward(cfg, w, seq)[-1]
            best = int(np.argmax(lg))
            assert t == best or lg[best] - lg[t] < TOL["bfloat16"], (t, best, float(lg[best] - lg[t]))
            seq.append(t)
    st = s.get_stats()
    assert st.n_finished == 16 and st.pool_free == st.pool_pages
    s.engine.check_device_errors()
