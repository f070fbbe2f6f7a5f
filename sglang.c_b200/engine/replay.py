"""Trace replay: given token ids go through the engine step by step and the
logits at the wanted places are written out.  Nothing is sampled.  It has no
forward pass, cache or loader of its own: it calls `Engine.step`.

(The reference's nearest relatives are its checks of whole against incremental
prefill, tests/test_gpt2.c:75-97, and its 16-step CPU-against-GPU loop,
tests/cuda_test.c:1233-1252.)
"""
import json
import os

import torch

from .step import StepEntry


def run_step_split(engine, entries):
    """One step of the trace as one engine step, or as several when it brings
    more tokens than the engine takes at once (the result does not depend on
    the cut).  Returns a float32 tensor [wanted, vocab] (a copy) or None."""
    cap = engine.max_step_tokens
    if not entries:
        return None
    if sum(len(e.tokens) for e in entries) <= cap:
        out = engine.step(entries)
        return out.clone() if out.shape[0] else None
    rows_of = {}
    pending = [(i, 0) for i in range(len(entries))]
    while pending:
        batch, room, nxt = [], cap, []
        for i, done in pending:
            e = entries[i]
            take = min(len(e.tokens) - done, room)
            if take > 0:
                want = [w - done for w in e.want if done <= w < done + take]
                batch.append((i, done, StepEntry(e.req, e.tokens[done:done + take], want)))
                room -= take
            if done + take < len(e.tokens):
                nxt.append((i, done + take))
        rows = engine.step([b[2] for b in batch]).clone()
        r = 0
        for i, done, se in batch:
            for w in se.want:
                rows_of[(i, w + done)] = rows[r]
                r += 1
        pending = nxt
    ordered = [rows_of[(i, w)] for i, e in enumerate(entries) for w in e.want]
    return torch.stack(ordered) if ordered else None


def replay(engine, lines, out_dir, emit=None):
    """Run every JSON line of `lines` as one step.  Writes <out_dir>/<step>.f32
    for steps that want logits and calls `emit("done <step>")` after each."""
    os.makedirs(out_dir, exist_ok=True)
    live = set()
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in live:
                engine.add_request(rid)
                live.add(rid)
            entries.append(StepEntry(rid, [int(t) for t in e["tokens"]],
                                     [int(w) for w in e.get("want", [])]))
        rows = run_step_split(engine, entries)
        if rows is not None:
            rows.to("cpu", torch.float32).contiguous().numpy().astype("<f4").tofile(
                os.path.join(out_dir, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        engine.check_device_errors()
        for rid in rec.get("end", []):
            if rid in live:
                engine.end_request(rid)
                live.discard(rid)
        if emit is not None:
            emit(f"done {step}")
