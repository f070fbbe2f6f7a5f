"""Typed configuration of the GPT-2 architecture (`GPT2LMHeadModel`).

Keys and meanings as in the architecture's own config.json
(models/gpt2/config.json of the reference; read at src/gpt2.c:37-42).  The
reference ignores `n_inner`, `activation_function`, `scale_attn_weights` and
`scale_attn_by_inverse_layer_idx` (src/gpt2.c:60,253; src/ops.c:233-241); they
are honoured here.
"""
from dataclasses import dataclass, asdict
from typing import Optional

from .base import ConfigError, get_bool, get_float, get_int, get_str

# activation_function values → the activation part's name
_ACTIVATIONS = {
    "gelu_new": "gelu_tanh",
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu_fast": "gelu_tanh",
    "gelu": "gelu_erf",
}


@dataclass(frozen=True)
class GPT2Config:
    n_layer: int
    n_embd: int
    n_head: int
    n_inner: int                      # feed-forward width (config null/absent: 4*n_embd)
    vocab_size: int
    n_positions: int                  # rows of the learned position table
    layer_norm_epsilon: float
    activation_function: str
    scale_attn_weights: bool          # scores *= 1/sqrt(head_dim)
    scale_attn_by_inverse_layer_idx: bool   # scores /= (layer_idx+1)
    tie_word_embeddings: bool
    bos_token_id: Optional[int]
    eos_token_id: Optional[int]
    architecture: str = "GPT2LMHeadModel"

    @property
    def head_dim(self):
        return self.n_embd // self.n_head

    @property
    def activation(self):
        return _ACTIVATIONS[self.activation_function]

    @classmethod
    def from_dict(cls, d):
        n_embd = get_int(d, "n_embd", minimum=1)
        n_head = get_int(d, "n_head", minimum=1)
        if n_embd % n_head != 0:
            # the reference's one check (src/gpt2.c:44-48)
            raise ConfigError(f"config.json: n_embd ({n_embd}) is not a multiple of n_head ({n_head})")
        n_inner = get_int(d, "n_inner", default=None, minimum=1)
        eos = get_int(d, "eos_token_id", default=None)
        bos = get_int(d, "bos_token_id", default=None)
        cfg = cls(
            n_layer=get_int(d, "n_layer", minimum=1),
            n_embd=n_embd,
            n_head=n_head,
            n_inner=n_inner if n_inner is not None else 4 * n_embd,
            vocab_size=get_int(d, "vocab_size", minimum=1),
            # the reference prefers n_ctx and falls back to n_positions (src/gpt2.c:40)
            n_positions=get_int(d, ["n_ctx", "n_positions"], minimum=1),
            layer_norm_epsilon=get_float(d, "layer_norm_epsilon", positive=True),
            activation_function=get_str(d, "activation_function", default="gelu_new",
                                        choices=set(_ACTIVATIONS)),
            scale_attn_weights=get_bool(d, "scale_attn_weights", default=True),
            scale_attn_by_inverse_layer_idx=get_bool(d, "scale_attn_by_inverse_layer_idx", default=False),
            tie_word_embeddings=get_bool(d, "tie_word_embeddings", default=True),
            bos_token_id=bos,
            eos_token_id=eos,
        )
        if "n_ctx" in d and "n_positions" in d and d["n_ctx"] is not None \
                and d["n_positions"] is not None and d["n_ctx"] > d["n_positions"]:
            raise ConfigError("config.json: n_ctx exceeds n_positions (rows of the position table)")
        if not cfg.tie_word_embeddings:
            raise ConfigError("config.json: tie_word_embeddings=false is not supported for GPT2LMHeadModel "
                              "(the head is the token table, src/gpt2.c:184-193)")
        if get_bool(d, "reorder_and_upcast_attn", default=False):
            # scores are always computed in 32-bit here, so the switch changes nothing
            pass
        return cfg

    def to_dict(self):
        """The config.json this configuration is written as."""
        d = asdict(self)
        d.pop("architecture")
        d["architectures"] = [self.architecture]
        d["model_type"] = "gpt2"
        d["n_ctx"] = self.n_positions
        return d
