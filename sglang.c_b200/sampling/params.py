"""Sampling options, with the reference's names and meanings
(include/sgl/sampling.h:12-24)."""
from dataclasses import dataclass, field
from typing import List


@dataclass
class SamplingParams:
    temperature: float = 0.0          # <= 0: greedy
    top_k: int = 0                    # <= 0: off
    top_p: float = 1.0                # outside (0,1): off
    min_p: float = 0.0                # > 0: drop candidates with p < min_p * p_max
    repetition_penalty: float = 1.0   # > 0 and != 1: positive logits divided, negative multiplied
    frequency_penalty: float = 0.0    # logit -= f * count(token)
    presence_penalty: float = 0.0     # logit -= p if the token was generated before
    ignore_eos: bool = False
    stop_ids: List[int] = field(default_factory=list)   # at most 8, as in the reference
    seed: int = 0

    MAX_STOP_TOKENS = 8

    def __post_init__(self):
        if len(self.stop_ids) > self.MAX_STOP_TOKENS:
            raise ValueError(f"at most {self.MAX_STOP_TOKENS} stop ids")

    @property
    def greedy(self):
        return self.temperature <= 0.0

    def has_penalties(self):
        return (self.repetition_penalty > 0.0 and self.repetition_penalty != 1.0) \
            or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    def is_stop(self, token):
        return token in self.stop_ids
