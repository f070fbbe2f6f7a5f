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
        # staged on the host in two buffers taken in turn (as the results below): the copy of
        # one launch's records may still be queued when the next launch's are written
        self.h_params = [torch.zeros((max_rows, 10), dtype=torch.int32).pin_memory() for _ in range(2)]
        self.np_i = [h.numpy() for h in self.h_params]         # the same pinned memory
        self.np_f = [a.view("float32") for a in self.np_i]
        self._all_greedy_rows = 0       # rows of d_params known to hold plain greedy records
        self.d_params = torch.zeros((max_rows, 10), dtype=torch.int32, device=device)
        self.d_out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.d_logprob = torch.zeros(max_rows, dtype=torch.float32, device=device)
        # two host copies taken in turn: a launch may follow before the last one's result is read
        self.h_out = [torch.zeros(max_rows, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.h_logprob = [torch.zeros(max_rows, dtype=torch.float32).pin_memory() for _ in range(2)]
        self.done = [torch.cuda.Event(), torch.cuda.Event()]
        self._turn = 0
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
        return self.fetch(self.launch(logits, params, uniforms, histories, want_logprobs))

    def launch(self, logits, params, uniforms, histories=None, want_logprobs=False):
        """The first half of sample(): the kernel and the copies to the host are queued on the
        stream and a ticket is returned; fetch(ticket) waits for them.  The sampled ids also stay
        in `d_out` on the device, in row order, until the next launch."""
        n = logits.shape[0]
        if n == 0:
            return (0, 0, want_logprobs)
        if n > self.max_rows:
            raise ValueError(f"{n} rows exceed the sampler's {self.max_rows}")
        hist_tok, hist_cnt = [], []
        plain_greedy = all(p.temperature <= 0.0 and not p.has_penalties() for p in params)
        if plain_greedy and self._all_greedy_rows >= n:
            pass                        # the device already holds n greedy records
        else:
            fi, ii = self.np_f[self._turn], self.np_i[self._turn]
            for i, (p, u) in enumerate(zip(params, uniforms)):
                hb = len(hist_tok)
                if histories is not None and p.has_penalties() and histories[i]:
                    counts = {}
                    for t in histories[i]:
                        counts[t] = counts.get(t, 0) + 1
                    hist_tok.extend(counts.keys())
                    hist_cnt.extend(counts.values())
                fi[i, 0] = p.temperature
                fi[i, 1] = p.top_p
                fi[i, 2] = p.min_p
                fi[i, 3] = u
                ii[i, 4] = p.top_k if p.temperature > 0.0 else 0
                fi[i, 5] = p.repetition_penalty
                fi[i, 6] = p.frequency_penalty
                fi[i, 7] = p.presence_penalty
                ii[i, 8] = hb
                ii[i, 9] = len(hist_tok)
            if len(hist_tok) > self.d_hist_tok.numel():
                self.d_hist_tok = torch.zeros(2 * len(hist_tok), dtype=torch.int32, device=self.device)
                self.d_hist_cnt = torch.zeros(2 * len(hist_tok), dtype=torch.int32, device=self.device)
            if hist_tok:
                self.d_hist_tok[:len(hist_tok)].copy_(torch.tensor(hist_tok, dtype=torch.int32))
                self.d_hist_cnt[:len(hist_cnt)].copy_(torch.tensor(hist_cnt, dtype=torch.int32))
            self.d_params[:n].copy_(self.h_params[self._turn][:n], non_blocking=True)
            self._all_greedy_rows = n if plain_greedy else 0
        ops.sample(logits, self.d_params[:n], self.d_hist_tok, self.d_hist_cnt, self.d_out[:n],
                   self.d_logprob[:n] if want_logprobs else None)
        turn = self._turn
        self._turn ^= 1
        self.h_out[turn][:n].copy_(self.d_out[:n], non_blocking=True)
        if want_logprobs:
            self.h_logprob[turn][:n].copy_(self.d_logprob[:n], non_blocking=True)
        self.done[turn].record()
        return (n, turn, want_logprobs)

    def fetch(self, ticket):
        """Wait for a launch's results: a list of token ids (and logprobs if they were asked)."""
        n, turn, want_logprobs = ticket
        if n == 0:
            return ([], []) if want_logprobs else []
        self.done[turn].synchronize()
        toks = self.h_out[turn][:n].tolist()
        if want_logprobs:
            return toks, self.h_logprob[turn][:n].tolist()
        return toks
