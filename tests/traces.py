"""Builders of replay traces for the tests: the same requests cut into steps in
different ways.  A trace is a list of step records as `bin/trace_run` reads
them; every fed position is wanted unless said otherwise, so each way of
cutting can be compared with the plain implementation position by position."""
import io
import json
import os

import numpy as np


def random_tokens(seed, n, vocab):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=n)]


def whole(requests):
    """Each request alone and whole, one step each."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_decoded(requests, n_tail=32):
    """Most of each request in one step, the last n_tail tokens one by one."""
    steps = []
    s = 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - n_tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        s += 1
        for i in range(head, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            s += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes=(7, 2, 13, 3, 2, 31, 5, 2, 64, 9)):
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    s = 0
    for rid, toks in requests.items():
        done, k = 0, 0
        while done < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - done)
            k += 1
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[done:done + n],
                                                  "want": list(range(n))}],
                          "end": [rid] if done + n == len(toks) else []})
            done += n
            s += 1
    return steps


def mixed(requests, prompt_len, seed=0, max_live=4, sizes=(5, 2, 11, 3, 17, 2, 8)):
    """Up to max_live live requests: the first prompt_len[rid] tokens of a request
    come in portions, the rest one token a step, beside the portions of others.
    A request may sit out a step.  Finished requests end and new ones start, so
    that with a small pool pages are given back and used again."""
    rng = np.random.default_rng(seed)
    waiting = list(requests)
    live = {}
    steps = []
    s = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, ends = [], []
        ids = list(live)
        sit_out = ids[int(rng.integers(0, len(ids)))] if len(ids) > 1 and rng.random() < 0.3 else None
        for rid in ids:
            if rid == sit_out:
                continue
            toks, done = requests[rid], live[rid]
            if done < prompt_len[rid]:
                n = min(int(sizes[int(rng.integers(0, len(sizes)))]), prompt_len[rid] - done)
            else:
                n = 1
            n = min(n, len(toks) - done)
            entries.append({"id": rid, "tokens": toks[done:done + n], "want": list(range(n))})
            live[rid] = done + n
            if live[rid] == len(toks):
                ends.append(rid)
        for rid in ends:
            del live[rid]
        steps.append({"step": s, "entries": entries, "end": ends})
        s += 1
    return steps


def peak_tokens(steps, round_to=64):
    """The most tokens live requests hold at any time, each rounded up."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def to_lines(steps):
    return [json.dumps(st) for st in steps]


def collect(steps, out_dir, vocab):
    """{request: {position: logits row}} from the files a replay wrote."""
    got, pos = {}, {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        if n_want == 0:
            for e in st["entries"]:
                pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
            continue
        rows = np.fromfile(os.path.join(out_dir, f"{st['step']}.f32"), dtype="<f4").reshape(n_want, vocab)
        r = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[base + w] = rows[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
    return got


def max_error(got, reference, all_positions=True):
    """Largest absolute difference over all collected rows; also checks that
    every position of every request was produced (all_positions=False: that
    some were, and compares those)."""
    worst, where = 0.0, None
    for rid, ref in reference.items():
        assert rid in got, f"no logits for request {rid}"
        if all_positions:
            assert sorted(got[rid]) == list(range(len(ref))), f"request {rid}: positions missing"
        for p in sorted(got[rid]):
            d = float(np.abs(got[rid][p].astype(np.float64) - ref[p]).max())
            if not np.isfinite(d):
                return float("inf"), (rid, p)
            if d > worst:
                worst, where = d, (rid, p)
    return worst, where
