"""Stand-ins for the GPU side, for host-only tests of the scheduler: an engine
with the real cache manager (no device tensors) whose "logits" are a
deterministic function of the request's tokens so far, and a sampler that reads
them on the host."""
import hashlib
from types import SimpleNamespace

import numpy as np

from sglang_c_b200.cache import CacheManager, CacheNeed
from sglang_c_b200.engine.engine import OutOfPages, StepError


def fake_logits(tokens, vocab):
    h = hashlib.sha256(np.asarray(tokens, dtype=np.int64).tobytes()).digest()
    rng = np.random.default_rng(int.from_bytes(h[:8], "little"))
    return rng.standard_normal(vocab).astype(np.float32)


class FakeEngine:
    def __init__(self, vocab=50, max_positions=64, page_size=4, n_pages=16, max_requests=4,
                 max_step_tokens=32, eos_token_id=None, n_calls=2):
        self.plan = SimpleNamespace(vocab_size=vocab, max_positions=max_positions, eos_token_id=eos_token_id)
        self.rt = SimpleNamespace(device="cpu")
        self.page_size, self.max_requests, self.max_step_tokens = page_size, max_requests, max_step_tokens
        need = CacheNeed.paged_kv(2, 8)
        self.cache = CacheManager([need] * n_calls, [None] * n_calls, page_size, n_pages, max_requests)
        self.history = {}      # request -> tokens fed so far
        self.steps = []        # [(req, n_tokens, wanted?)] per step

    def add_request(self, req):
        if self.cache.add_request(req) is None:
            raise StepError("no slot")
        self.history[req] = []

    def end_request(self, req):
        self.cache.free_request(req)
        del self.history[req]

    def has_request(self, req):
        return self.cache.has_request(req)

    def step(self, entries):
        wants = [(e.req, self.cache.length(e.req) + len(e.tokens)) for e in entries]
        assert sum(len(e.tokens) for e in entries) <= self.max_step_tokens
        if not self.cache.can_extend_all(wants):
            raise OutOfPages("fake")
        rows = []
        for e, (req, new_len) in zip(entries, wants):
            assert self.cache.extend(req, new_len)
            base = len(self.history[req])
            self.history[req].extend(e.tokens)
            for w in e.want:
                rows.append(fake_logits(self.history[req][:base + w + 1], self.plan.vocab_size))
        self.cache.check()
        self.steps.append([(e.req, len(e.tokens), bool(e.want)) for e in entries])
        return np.stack(rows) if rows else np.zeros((0, self.plan.vocab_size), np.float32)


class FakeSampler:
    """Greedy, or temperature by inverse CDF in index order, on the host."""

    def sample(self, logits, params, uniforms, histories=None, want_logprobs=False):
        out = []
        for row, p, u in zip(logits, params, uniforms):
            if p.temperature <= 0:
                out.append(int(np.argmax(row)))
            else:
                w = np.exp((row.astype(np.float64) - row.max()) / p.temperature)
                c = np.cumsum(w) / w.sum()
                out.append(int(min(np.searchsorted(c, u, side="right"), len(row) - 1)))
        return (out, [0.0] * len(out)) if want_logprobs else out
