"""GPT-2 (`GPT2LMHeadModel`) as a plan of parts: learned token and position
tables, pre-LayerNorm blocks of causal multi-head attention and a GELU MLP, a
final LayerNorm, and a head tied to the token table (reference src/gpt2.c:210-297;
tensor names :61-96, without a "transformer." prefix, which is tried second).
"""
import math

from ..config.gpt2 import GPT2Config
from ..config.registry import register_architecture
from ..parts.plan import LayerCall, LayerPlan, ModelPlan, PartSpec


def build_plan(cfg: GPT2Config) -> ModelPlan:
    E, H, D = cfg.n_embd, cfg.n_head, cfg.head_dim
    layers = []
    for l in range(cfg.n_layer):
        p = f"h.{l}."
        # 1/sqrt(D) (src/gpt2.c:253) unless scale_attn_weights is off; further
        # divided by layer_idx+1 when scale_attn_by_inverse_layer_idx is on
        scale = (1.0 / math.sqrt(D)) if cfg.scale_attn_weights else 1.0
        if cfg.scale_attn_by_inverse_layer_idx:
            scale /= float(l + 1)
        norm = lambda n: PartSpec("layer_norm", {"size": E, "eps": cfg.layer_norm_epsilon},
                                  {"weight": p + n + ".weight", "bias": p + n + ".bias"})
        layers.append(LayerPlan(
            name=f"h.{l}",
            block=PartSpec("pre_norm"),
            norm1=norm("ln_1"),
            mixer=PartSpec("causal_attention",
                           {"size": E, "n_heads": H, "n_kv_heads": H, "head_dim": D, "scale": scale,
                            "window": None, "bias": True, "weight_layout": "conv1d"},
                           {"qkv_weight": p + "attn.c_attn.weight", "qkv_bias": p + "attn.c_attn.bias",
                            "out_weight": p + "attn.c_proj.weight", "out_bias": p + "attn.c_proj.bias"}),
            norm2=norm("ln_2"),
            ffn=PartSpec("mlp",
                         {"size": E, "inner_size": cfg.n_inner, "activation": cfg.activation,
                          "bias": True, "weight_layout": "conv1d"},
                         {"up_weight": p + "mlp.c_fc.weight", "up_bias": p + "mlp.c_fc.bias",
                          "down_weight": p + "mlp.c_proj.weight", "down_bias": p + "mlp.c_proj.bias"}),
        ))
    return ModelPlan(
        hidden_size=E,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.n_positions,
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab_size, "size": E},
                           {"table": "wte.weight"}),
        position=PartSpec("learned_absolute", {"max_positions": cfg.n_positions, "size": E},
                          {"table": "wpe.weight"}),
        layers=layers,
        order=[LayerCall(l) for l in range(cfg.n_layer)],
        final_norm=PartSpec("layer_norm", {"size": E, "eps": cfg.layer_norm_epsilon},
                            {"weight": "ln_f.weight", "bias": "ln_f.bias"}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab_size, "size": E}, {"weight": "wte.weight"}),
        eos_token_id=cfg.eos_token_id,
        # checkpoints of this architecture may carry the tied head and mask buffers
        ignorable=("lm_head.weight", "h.*.attn.bias", "h.*.attn.masked_bias"),
        name_prefixes=("", "transformer."),
    )


register_architecture("GPT2LMHeadModel", GPT2Config, build_plan, model_types=("gpt2",))
