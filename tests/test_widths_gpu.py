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
# logits of these models are a few tenths in size (vocabulary rows N(0, 0.02)).  bfloat16 runs are
# compared with the plain implementation rounding where the engine rounds; what is left is values
# falling on the other side of a rounding step (see tests/test_replay_gpu.py), more of them and
# through longer sums at these widths than in the tiny models
TOL = {"float32": 5e-5, "bfloat16": 2e-2}
TIE = 2e-2        # a generated token other than the plain one is accepted at a near tie only


def plain(d, toks, dtype):
    return plain_gpt2.forward_dir(d, toks, rounded=(dtype == "bfloat16"))


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
    ref = {rid: plain(d, toks, dtype) for rid, toks in reqs.items()}
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


def test_xl_widths_two_thousand_tokens_a_step(width_dirs, tmp_path):
    """Four prompts of 500 tokens in one step at XL widths: the products are large enough for the
    kernel on pairs of SMs (all four of a layer), and the queries' 1,600 columns end inside one of
    its tiles, beside which keys and values go into the cache from the same epilogue.  The same
    requests cut into portions of changing size stay on the one-block kernel; both against the
    plain implementation."""
    from sglang_c_b200.csrc import ops
    from sglang_c_b200.engine import Engine
    from sglang_c_b200.engine.replay import replay
    for N, K, act in ((4800, 1600, None), (1600, 1600, None), (6400, 1600, "gelu_tanh"), (1600, 6400, None)):
        assert ops.gemm_tc_form(2000, N, K, act) == "pair"
    d = width_dirs("xl", "bfloat16")
    reqs = {rid: traces.random_tokens(10 + i, 500, 1031) for i, rid in enumerate("abcd")}
    ref = {rid: plain(d, toks, "bfloat16") for rid, toks in reqs.items()}
    together = [{"step": 0, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}
                                        for rid, toks in reqs.items()], "end": list(reqs)}]
    for mode, steps in (("together", together), ("portions", traces.portions(reqs))):
        eng = Engine.from_dir(d, dtype="bfloat16", page_size=16, n_pages=traces.peak_tokens(steps) // 16,
                              max_requests=4, max_step_tokens=2048)
        out = str(tmp_path / mode)
        replay(eng, traces.to_lines(steps), out)
        got = traces.collect(steps, out, 1031)
        err, where = traces.max_error(got, ref)
        assert err < TOL["bfloat16"], f"xl {mode}: max error {err} at {where}"
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
    ref = {rid: plain(d, toks, "bfloat16") for rid, toks in reqs.items()}
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_single_tokens_beside_prompt_portions_at_small_width(width_dirs, tmp_path, dtype):
    """One step holds sixteen single decoded tokens (12 heads of size 64: 192 (token, head) items,
    which in bfloat16 go to the streaming decode attention through a token list) beside portions
    of two prompts (which go to the tensor-core prompt attention), with so few pages that the
    pages of the first wave of requests are used again by the second."""
    from sglang_c_b200.engine import Engine
    from sglang_c_b200.engine.replay import replay
    d = width_dirs("small", dtype)
    V = 1031
    rng = np.random.default_rng(8)
    lens = [int(n) for n in rng.permutation(np.linspace(17, 200, 16).astype(int))]
    n_tail = 4
    dec = {f"d{i}": traces.random_tokens(700 + i, n + n_tail, V) for i, n in enumerate(lens)}
    pro = {"p0": traces.random_tokens(800, 300, V), "p1": traces.random_tokens(801, 170, V)}
    first = {f"f{i}": traces.random_tokens(900 + i, 90, V) for i in range(6)}     # come and go first
    ref = {rid: plain(d, toks, dtype) for rid, toks in {**dec, **pro, **first}.items()}
    steps = [{"step": 0, "end": list(first),
              "entries": [{"id": rid, "tokens": t, "want": [0, 89]} for rid, t in first.items()]}]
    ids = list(dec)
    for g in range(0, 16, 4):
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": rid, "tokens": dec[rid][:lens[ids.index(rid)]], "want": [0]}
                                  for rid in ids[g:g + 4]]})
    cuts = {"p0": [0, 130, 132, 260, 300], "p1": [0, 2, 129, 150, 170]}
    for k in range(n_tail):
        entries = [{"id": rid, "tokens": [dec[rid][lens[i] + k]], "want": [0]} for i, rid in enumerate(ids)]
        for rid in pro:
            a, b = cuts[rid][k], cuts[rid][k + 1]
            entries.append({"id": rid, "tokens": pro[rid][a:b], "want": list(range(b - a))})
        steps.append({"step": len(steps), "end": (ids + list(pro)) if k == n_tail - 1 else [], "entries": entries})
    n_pages = traces.peak_tokens(steps) // 16
    assert n_pages * 16 < sum((len(t) + 63) // 64 * 64 for t in {**dec, **pro, **first}.values())
    eng = Engine.from_dir(d, dtype=dtype, page_size=16, n_pages=n_pages, max_requests=18, max_step_tokens=1024)
    out = str(tmp_path / "out")
    replay(eng, traces.to_lines(steps), out)
    got = traces.collect(steps, out, V)
    err, where = traces.max_error(got, ref, all_positions=False)
    assert err < TOL[dtype], f"max error {err} at {where}"
    eng.check_device_errors()
    eng.cache.check()


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
            assert t == best or lg[best] - lg[t] < TIE, (t, best, float(lg[best] - lg[t]))
            seq.append(t)
    st = s.get_stats()
    assert st.n_finished == 16 and st.pool_free == st.pool_pages
    s.engine.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_depth_and_vocabulary_of_gpt2_small(tmp_path_factory, tmp_path, dtype):
    """GPT-2 small as it is: 12 layers, a vocabulary of 50,257 (no multiple of anything), the
    standard init.  Two requests, whole and then cut and mixed, against the plain implementation."""
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.engine import Engine
    from sglang_c_b200.engine.replay import replay
    from sglang_c_b200.weights import write_random_model
    cfg_d = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=12, n_embd=768, n_head=12,
                 n_inner=3072, vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
                 activation_function="gelu_new")
    arch = resolve_architecture(cfg_d)
    d = write_random_model(str(tmp_path_factory.mktemp("small_full") / "m"), arch, arch.config_class.from_dict(cfg_d),
                           5, scheme="standard", store_dtype=dtype)
    V = 50257
    reqs = {"a": traces.random_tokens(21, 40, V), "b": traces.random_tokens(22, 24, V)}
    ref = {rid: plain(d, toks, dtype) for rid, toks in reqs.items()}
    for mode, steps in (("whole", traces.whole(reqs)), ("mixed", traces.mixed(reqs, {"a": 30, "b": 10}, seed=1))):
        eng = Engine.from_dir(d, dtype=dtype, page_size=16, n_pages=traces.peak_tokens(steps) // 16,
                              max_requests=4, max_step_tokens=128)
        out = str(tmp_path / mode)
        replay(eng, traces.to_lines(steps), out)
        got = traces.collect(steps, out, V)
        err, where = traces.max_error(got, ref)
        assert err < TOL[dtype], f"{mode}: max error {err} at {where}"
        eng.check_device_errors()
        del eng
