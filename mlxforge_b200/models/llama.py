"""``LlamaForCausalLM``: the dense GQA decoder, described as data.

Block order, tensor names and the head rule follow the reference's
``DecoderModel`` (src/model/decoder_model.cpp:166-168 layer key prefix,
:234-253 projections, :277-282 feed-forward, :288-293 pre-norm block with two
residuals, :346-350 final norm and head; src/model/llama.h:13-17 adds nothing).
Every size below comes from the configuration.
"""
from __future__ import annotations

from typing import Iterator, Tuple

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    rs = cfg.rope_scaling
    position = PartSpec("rope", {
        "head_dim": cfg.head_dim, "rotary_dim": cfg.head_dim, "theta": cfg.rope_theta,
        "scaling": None if rs is None else rs.to_json(),
    })
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            block="prenorm",
            mixer=PartSpec("attention", {
                "hidden_size": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
                "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                "softmax_scale": float(cfg.head_dim) ** -0.5, "window": 0, "position": position,
            }, prefix=p + "self_attn."),
            mixer_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                                prefix=p + "input_layernorm."),
            feed_forward=PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                                             "intermediate_size": cfg.intermediate_size},
                                  prefix=p + "mlp."),
            feed_forward_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                                       prefix=p + "post_attention_layernorm."),
        ))
    return ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size},
                           prefix="model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(ScheduleItem(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix="model.norm."),
        head=PartSpec("linear_head", {
            "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
            # lm_head.weight is used when the file has it, else the embedding table
            # (src/model/decoder_model.cpp:348-349); an untied config must have it.
            "tied_to": "model.embed_tokens.weight", "require_own": not cfg.tie_word_embeddings,
        }, prefix="lm_head."),
        eos_token_ids=tuple(cfg.eos_token_ids),
        max_position_embeddings=cfg.max_position_embeddings,
    )


def llama_random_tensors(cfg: LlamaConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """Names, shapes and kinds (``matrix`` / ``norm``) of a checkpoint of this
    configuration, in file order."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq = cfg.num_attention_heads * cfg.head_dim
    nkv = cfg.num_key_value_heads * cfg.head_dim
    yield "model.embed_tokens.weight", (V, H), "matrix"
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        yield p + "input_layernorm.weight", (H,), "norm"
        yield p + "self_attn.q_proj.weight", (nq, H), "matrix"
        yield p + "self_attn.k_proj.weight", (nkv, H), "matrix"
        yield p + "self_attn.v_proj.weight", (nkv, H), "matrix"
        yield p + "self_attn.o_proj.weight", (H, nq), "matrix"
        yield p + "post_attention_layernorm.weight", (H,), "norm"
        yield p + "mlp.gate_proj.weight", (I, H), "matrix"
        yield p + "mlp.up_proj.weight", (I, H), "matrix"
        yield p + "mlp.down_proj.weight", (H, I), "matrix"
    yield "model.norm.weight", (H,), "norm"
    if not cfg.tie_word_embeddings:
        yield "lm_head.weight", (V, H), "matrix"


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama_spec, llama_random_tensors, replace=True)
