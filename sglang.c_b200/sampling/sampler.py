"""Batch sampling on the device: one kernel launch for all rows of a step."""
import struct

import torch

from ..csrc import ops
from .params import SamplingParams


class Sampler:
    """Holds pinned staging buffers sized for `max_rows` rows."""

    def __init__(self, device, max_rows, max_history=4096):
        self.device = device
        self.max_rows = max_rows
        self.h_params = torch.zeros((max_rows, 10), dtype=torch.int32).pin_memory()
        self.d_params = torch.zeros((max_rows, 10), dtype=torch.int32, device=device)
        self.d_out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.d_logprob = torch.zeros(max_rows, dtype=torch.float32, device=device)
        self.h_out = torch.zeros(max_rows, dtype=torch.int32).pin_memory()
        self.h_logprob = torch.zeros(max_rows, dtype=torch.float32).pin_memory()
        self.d_hist_tok = torch.zeros(max(1, max_history), dtype=torch.int32, device=device)
        self.d_hist_cnt = torch.zeros(max(1, max_history), dtype=torch.int32, device=device)

    @staticmethod
    def _bits(f):
        return struct.unpack("<i", struct.pack("<f", float(f)))[0]

    def sample(self, logits, params, uniforms, histories=None, want_logprobs=False):
        """logits: [n, V] float32 on the device (changed in place when penalties
        are on); params: n SamplingParams; uniforms: n floats in [0,1) (ignored
        for greedy rows); histories: per row the generated tokens so far (for
        penalties).  Returns a list of n token ids (and logprobs if asked)."""
        n = logits.shape[0]
        if n == 0:
            return ([], []) if want_logprobs else []
        if n > self.max_rows:
            raise ValueError(f"{n} rows exceed the sampler's {self.max_rows}")
        hp = self.h_params
        hist_tok, hist_cnt = [], []
        for i, (p, u) in enumerate(zip(params, uniforms)):
            hb = len(hist_tok)
            if histories is not None and p.has_penalties() and histories[i]:
                counts = {}
                for t in histories[i]:
                    counts[t] = counts.get(t, 0) + 1
                hist_tok.extend(counts.keys())
                hist_cnt.extend(counts.values())
            b = self._bits
            hp[i] = torch.tensor([b(p.temperature), b(p.top_p), b(p.min_p), b(u), int(p.top_k),
                                  b(p.repetition_penalty), b(p.frequency_penalty), b(p.presence_penalty),
                                  hb, len(hist_tok)], dtype=torch.int32)
        if len(hist_tok) > self.d_hist_tok.numel():
            self.d_hist_tok = torch.zeros(2 * len(hist_tok), dtype=torch.int32, device=self.device)
            self.d_hist_cnt = torch.zeros(2 * len(hist_tok), dtype=torch.int32, device=self.device)
        if hist_tok:
            self.d_hist_tok[:len(hist_tok)].copy_(torch.tensor(hist_tok, dtype=torch.int32))
            self.d_hist_cnt[:len(hist_cnt)].copy_(torch.tensor(hist_cnt, dtype=torch.int32))
        self.d_params[:n].copy_(hp[:n], non_blocking=True)
        ops.sample(logits, self.d_params[:n], self.d_hist_tok, self.d_hist_cnt, self.d_out[:n],
                   self.d_logprob[:n] if want_logprobs else None)
        self.h_out[:n].copy_(self.d_out[:n], non_blocking=True)
        if want_logprobs:
            self.h_logprob[:n].copy_(self.d_logprob[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        toks = self.h_out[:n].tolist()
        if want_logprobs:
            return toks, self.h_logprob[:n].tolist()
        return toks
