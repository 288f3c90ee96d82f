"""GPT-2 as data: its tensor names, its random initialisation, and its ModelSpec.

Tensor names and the `[in, out]` (Conv1D) layout of the four matrices per layer are those of
GPT-2 checkpoints (kelpie-models/kelpie_models/models/torch/gpt2.py:157-188): `wte.weight`,
`wpe.weight`, `h.{i}.ln_1`, `h.{i}.attn.c_attn`, `h.{i}.attn.c_proj`, `h.{i}.ln_2`,
`h.{i}.mlp.c_fc`, `h.{i}.mlp.c_proj`, `ln_f`; each may carry a `transformer.` prefix. The
head is the token table (gpt2.py:70,101): a stored `lm_head.weight` is not read but must equal
`wte.weight` (the reference's tripwire is its shape assert, gpt2.py:186-187); the causal-mask
buffers `attn.bias` / `attn.masked_bias` are not read.
"""

from __future__ import annotations

import torch

from ..config.gpt2 import GPT2Config
from ..config.registry import Architecture, register_architecture
from ..parts import LayerSpec, PartSpec, Runtime
from ..weights.loader import TensorSpec, WeightSpec
from .decoder import DecoderModel, ModelSpec

NAME = "GPT2LMHeadModel"


def weight_spec(cfg: GPT2Config) -> WeightSpec:
    d, f = cfg.n_embd, cfg.n_inner
    tensors = [TensorSpec("wte.weight", (cfg.vocab_size, d)), TensorSpec("wpe.weight", (cfg.n_positions, d))]
    for i in range(cfg.n_layer):
        p = f"h.{i}"
        tensors += [
            TensorSpec(f"{p}.ln_1.weight", (d,)), TensorSpec(f"{p}.ln_1.bias", (d,)),
            TensorSpec(f"{p}.attn.c_attn.weight", (d, 3 * d)), TensorSpec(f"{p}.attn.c_attn.bias", (3 * d,)),
            TensorSpec(f"{p}.attn.c_proj.weight", (d, d)), TensorSpec(f"{p}.attn.c_proj.bias", (d,)),
            TensorSpec(f"{p}.ln_2.weight", (d,)), TensorSpec(f"{p}.ln_2.bias", (d,)),
            TensorSpec(f"{p}.mlp.c_fc.weight", (d, f)), TensorSpec(f"{p}.mlp.c_fc.bias", (f,)),
            TensorSpec(f"{p}.mlp.c_proj.weight", (f, d)), TensorSpec(f"{p}.mlp.c_proj.bias", (d,)),
        ]
    tensors += [TensorSpec("ln_f.weight", (d,)), TensorSpec("ln_f.bias", (d,))]
    return WeightSpec(
        tensors=tuple(tensors),
        prefixes=("", "transformer."),
        ignorable=(r"(transformer\.)?h\.\d+\.attn\.(bias|masked_bias)",),
        tied=(("lm_head.weight", "wte.weight"),),
    )


def random_weights(cfg: GPT2Config, seed: int, std: float = 0.02, bias_std: float = 0.01,
                   norm_std: float = 0.02) -> dict[str, torch.Tensor]:
    """Float32 draws from ONE CPU generator, in the order of `weight_spec`: matrices and tables
    N(0, std), biases N(0, bias_std), norm gains 1 + N(0, norm_std), norm shifts N(0, norm_std)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for ts in weight_spec(cfg).tensors:
        draw = torch.randn(ts.shape, generator=gen, dtype=torch.float32)
        is_norm = ".ln_" in ts.name or ts.name.startswith("ln_f")
        if is_norm and ts.name.endswith(".weight"):
            out[ts.name] = 1.0 + norm_std * draw
        elif is_norm:
            out[ts.name] = norm_std * draw
        elif ts.name.endswith(".bias"):
            out[ts.name] = bias_std * draw
        else:
            out[ts.name] = std * draw
    return out


def model_spec(cfg: GPT2Config) -> ModelSpec:
    layers = []
    for i in range(cfg.n_layer):
        p = f"h.{i}"
        layers.append(LayerSpec(
            block="pre_norm",
            norm_1=PartSpec("layer_norm", {"eps": cfg.layer_norm_epsilon},
                            {"gamma": f"{p}.ln_1.weight", "beta": f"{p}.ln_1.bias"}),
            mixer=PartSpec(
                "attention",
                {"n_heads": cfg.n_head, "n_kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
                 "scale": cfg.attention_scale(i), "window": 0},
                {"w_qkv": f"{p}.attn.c_attn.weight", "b_qkv": f"{p}.attn.c_attn.bias",
                 "w_out": f"{p}.attn.c_proj.weight", "b_out": f"{p}.attn.c_proj.bias"}),
            norm_2=PartSpec("layer_norm", {"eps": cfg.layer_norm_epsilon},
                            {"gamma": f"{p}.ln_2.weight", "beta": f"{p}.ln_2.bias"}),
            feed_forward=PartSpec(
                "mlp", {"activation": cfg.activation_function},
                {"w_in": f"{p}.mlp.c_fc.weight", "b_in": f"{p}.mlp.c_fc.bias",
                 "w_out": f"{p}.mlp.c_proj.weight", "b_out": f"{p}.mlp.c_proj.bias"}),
        ))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden=cfg.n_embd, max_seq_len=cfg.n_positions, eos_token=cfg.eos_token_id,
        embedding="wte.weight", head="wte.weight",
        positions=PartSpec("learned", {"n_positions": cfg.n_positions}, {"table": "wpe.weight"}),
        layers=tuple(layers),
        final_norm=PartSpec("layer_norm", {"eps": cfg.layer_norm_epsilon}, {"gamma": "ln_f.weight", "beta": "ln_f.bias"}),
    )


def build(cfg: GPT2Config, tensors: dict[str, torch.Tensor], rt: Runtime) -> DecoderModel:
    return DecoderModel(model_spec(cfg), tensors, rt, config=cfg)


GPT2 = register_architecture(Architecture(
    name=NAME, parse_config=GPT2Config.from_json, weight_spec=weight_spec, random_weights=random_weights,
    build=build, config_to_json=GPT2Config.to_json,
))
