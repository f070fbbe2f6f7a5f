"""The framework takes parts and architectures it has never seen, registered from here
without a change to its files: a mixer with per-request state of its own (in slots, not
pages), a running order that names a layer twice, a call that reads the cache another call
wrote, and a layer with a window beside layers without.  Each toy model is compared with a
plain restatement written here from the plain implementation's parts.  These are toys, not
models of anyone's."""
import dataclasses
import math
import os

import numpy as np
import pytest
import torch

import plain_gpt2
import traces
from conftest import TINY

pytestmark = pytest.mark.gpu
TOL = {"float32": 3e-5, "bfloat16": 1.5e-2}
DECAY = 0.75


def _register():
    from sglang_c_b200.cache import CacheNeed
    from sglang_c_b200.config import GPT2Config, register_architecture
    from sglang_c_b200.models.gpt2 import build_plan
    from sglang_c_b200.parts import LayerCall, Part, PartSpec, WeightDecl, register_part

    @register_part("mixer", "toy_running_mean")
    class RunningMeanMixer(Part):
        """state <- decay*state + (1-decay)*h_t, token by token; out_t = state·Wᵀ.  The
        state is one vector per request in a slot that the cache manager hands out."""
        graph_safe = False        # it walks the step's requests on the host

        @classmethod
        def declare_weights(cls, params):
            return {"out_weight": WeightDecl((params["size"], params["size"]), "residual_matrix")}

        def load(self, tensors, store):
            self.w = store.matrix(tensors["out_weight"])

        def cache_need(self):
            return CacheNeed.state((self.params["size"],), "float32")

        def forward(self, ctx, h, residual, cache, position=None):
            assert cache.kind == "state"
            d = float(self.params["decay"])
            y = torch.empty(h.shape, dtype=torch.float32, device=h.device)
            t0 = 0
            for n, slot in zip(ctx.h_q_len, ctx.h_state_slots):
                s = cache.tensor[slot]
                for t in range(t0, t0 + n):
                    s = d * s + (1.0 - d) * h[t].float()
                    y[t] = s
                cache.tensor[slot] = s
                t0 += n
            ctx.rt.gemm(y.to(h.dtype), self.w, None, residual=residual)

    def plan_state(cfg):
        plan = build_plan(cfg)
        for l, layer in enumerate(plan.layers):
            if l % 2 == 1:
                layer.mixer = PartSpec("toy_running_mean", {"size": cfg.n_embd, "decay": DECAY},
                                       {"out_weight": f"h.{l}.toy.out.weight"})
        return plan

    def plan_order(cfg):
        plan = build_plan(cfg)
        plan.order = [LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(0, cache_of=0)]
        return plan

    def plan_window(cfg):
        plan = build_plan(cfg)
        plan.layers[1].mixer.params["window"] = 10
        return plan

    register_architecture("ToyStateForTest", GPT2Config, plan_state)
    register_architecture("ToyOrderForTest", GPT2Config, plan_order)
    register_architecture("ToyWindowForTest", GPT2Config, plan_window)


@pytest.fixture(scope="module")
def toy_dirs(tmp_path_factory):
    _register()
    from sglang_c_b200.config import GPT2Config, resolve_architecture
    from sglang_c_b200.weights import write_random_model
    base = tmp_path_factory.mktemp("toys")
    made = {}

    def get(arch_name, tiny, store):
        key = (arch_name, tiny, store)
        if key not in made:
            cfg = dataclasses.replace(GPT2Config.from_dict(TINY[tiny]), architecture=arch_name)
            arch = resolve_architecture({"architectures": [arch_name]})
            made[key] = write_random_model(str(base / f"{arch_name}_{tiny}_{store}"), arch, cfg, 77,
                                           scheme="varied", store_dtype=store)
        return made[key]

    return get


# ---- plain restatements ---------------------------------------------------------
def _qkv(x, w, l, st):
    p = f"h.{l}."
    h = plain_gpt2.layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], st["eps"])
    qkv = plain_gpt2.conv1d(h, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"])
    E = st["E"]
    return h, qkv[:, :E], qkv[:, E:2 * E], qkv[:, 2 * E:]


def _attn_out(x, a, w, l):
    p = f"h.{l}."
    return x + plain_gpt2.conv1d(a, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])


def _finish(x, w, st):
    hf = plain_gpt2.layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], st["eps"])
    return plain_gpt2.lm_head(hf, w["wte.weight"])


def plain_state(cfg, w, toks):
    st = plain_gpt2.settings(cfg)
    x = plain_gpt2.embedding(toks, w["wte.weight"], w["wpe.weight"])
    for l in range(st["L"]):
        if l % 2 == 1:
            p = f"h.{l}."
            h = plain_gpt2.layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], st["eps"])
            s = np.zeros(st["E"])
            y = np.zeros_like(h)
            for t in range(len(toks)):
                s = DECAY * s + (1 - DECAY) * h[t]
                y[t] = s
            x = x + y @ w[p + "toy.out.weight"].T
        else:
            x = plain_gpt2.attention_block(x, w, l, st)
        x = plain_gpt2.mlp_block(x, w, l, st)
    return _finish(x, w, st)


def plain_order(cfg, w, toks):
    st = plain_gpt2.settings(cfg)
    x = plain_gpt2.embedding(toks, w["wte.weight"], w["wpe.weight"])
    kept = None
    for call, (l, shared) in enumerate([(0, False), (1, False), (1, False), (0, True)]):
        h, q, k, v = _qkv(x, w, l, st)
        if call == 0:
            kept = (k, v)
        if shared:
            k, v = kept          # reads what call 0 cached; its own keys and values are unused
        a = plain_gpt2.causal_attention(q, k, v, st["H"], plain_gpt2.attention_scale(st, l))
        x = _attn_out(x, a, w, l)
        x = plain_gpt2.mlp_block(x, w, l, st)
    return _finish(x, w, st)


def plain_window(cfg, w, toks):
    st = plain_gpt2.settings(cfg)
    x = plain_gpt2.embedding(toks, w["wte.weight"], w["wpe.weight"])
    for l in range(st["L"]):
        h, q, k, v = _qkv(x, w, l, st)
        a = plain_gpt2.causal_attention(q, k, v, st["H"], plain_gpt2.attention_scale(st, l),
                                        window=10 if l == 1 else None)
        x = _attn_out(x, a, w, l)
        x = plain_gpt2.mlp_block(x, w, l, st)
    return _finish(x, w, st)


PLAIN = {"ToyStateForTest": plain_state, "ToyOrderForTest": plain_order, "ToyWindowForTest": plain_window}


def run(model_dir, dtype, steps, tmp_path, n_pages, page_size=8):
    from sglang_c_b200.engine import Engine
    from sglang_c_b200.engine.replay import replay
    eng = Engine.from_dir(model_dir, dtype=dtype, page_size=page_size, n_pages=n_pages, max_requests=4,
                          max_step_tokens=256)
    out = str(tmp_path / "o")
    replay(eng, traces.to_lines(steps), out)
    eng.cache.check()
    return eng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("arch", ["ToyStateForTest", "ToyOrderForTest", "ToyWindowForTest"])
@pytest.mark.parametrize("tiny", ["A", "B"])
def test_toy_models_in_every_cut(toy_dirs, tmp_path, arch, tiny, dtype):
    d = toy_dirs(arch, tiny, dtype)
    cfg, w = plain_gpt2.read_model_dir(d)
    V = TINY[tiny]["vocab_size"]
    reqs = {f"t{i}": traces.random_tokens(300 + i, n, V) for i, n in enumerate([33, 70, 12, 100, 57])}
    ref = {rid: PLAIN[arch](cfg, w, toks) for rid, toks in reqs.items()}
    prompt_len = {rid: max(2, len(t) - 12) for rid, t in reqs.items()}
    for mode, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail_decoded(reqs, 32)),
                        ("portions", traces.portions(reqs)), ("mixed", traces.mixed(reqs, prompt_len, seed=4))):
        n_pages = traces.peak_tokens(steps) // 8
        eng = run(d, dtype, steps, tmp_path / mode, n_pages)
        got = traces.collect(steps, str(tmp_path / mode / "o"), V)
        err, where = traces.max_error(got, ref)
        assert err < TOL[dtype], f"{arch} {mode}: max error {err} at {where}"
        assert eng.cache.n_free_pages() == n_pages and eng.cache.n_free_slots() == 4


def test_toy_state_lives_in_slots_and_groups_are_separate(toy_dirs):
    from sglang_c_b200.engine import Engine
    d = toy_dirs("ToyStateForTest", "B", "float32")       # 3 layers: attention, toy, attention
    eng = Engine.from_dir(d, dtype="float32", page_size=8, n_pages=8, max_requests=3, max_step_tokens=64)
    kinds = sorted(g.need.kind for g in eng.cache.groups)
    assert kinds == ["paged_kv", "state"]
    state = [g for g in eng.cache.groups if g.need.kind == "state"][0]
    assert tuple(state.tensor.shape) == (1, 3, 96)
    assert not eng.model.graph_safe
    d2 = toy_dirs("ToyWindowForTest", "A", "float32")
    eng2 = Engine.from_dir(d2, dtype="float32", page_size=8, n_pages=8, max_requests=3, max_step_tokens=64)
    assert sorted(str(g.need.window) for g in eng2.cache.groups) == ["10", "None"]
    d3 = toy_dirs("ToyOrderForTest", "A", "float32")
    eng3 = Engine.from_dir(d3, dtype="float32", page_size=8, n_pages=8, max_requests=3, max_step_tokens=64)
    assert eng3.cache.groups[0].tensor.shape[0] == 3       # four calls, three caches
    assert eng3.cache.binding(3).write is False


def test_window_layer_runs_in_fewer_pages_than_the_sequence(toy_dirs, tmp_path):
    """Only the windowed group can hold 120 positions in 4 pages of 8; the full group of the
    same model cannot, so the pools are separate and the window's pages are used again."""
    from sglang_c_b200.cache import CacheManager, CacheNeed
    m = CacheManager([CacheNeed.paged_kv(2, 8, window=10)], [None], 8, 4, 2)
    m.add_request("w")
    for n in range(1, 121):
        assert m.extend("w", n)
    m.check()
