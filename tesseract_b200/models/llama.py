"""Llama (``LlamaForCausalLM``): configuration -> model description.

A dense pre-norm decoder: token embedding, ``num_hidden_layers`` identical blocks of
grouped-query attention with rotary encoding and a SwiGLU feed-forward, RMSNorm
everywhere, a final norm and an output head that may share the embedding matrix.
Tensor names are the checkpoint's own (src/model/llama_3_2.rs:226-266).
"""

from __future__ import annotations

from .llama_config import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec.make("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, {"weight": name})

    position = PartSpec.make("rotary", {
        "head_dim": cfg.head_dim,
        "theta": cfg.rope_theta,
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
    })
    layers = []
    for index in range(cfg.num_hidden_layers):
        prefix = f"model.layers.{index}"
        mixer = PartSpec.make(
            "attention",
            {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
             "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "window": None, "scale": None},
            {"q": f"{prefix}.self_attn.q_proj.weight", "k": f"{prefix}.self_attn.k_proj.weight",
             "v": f"{prefix}.self_attn.v_proj.weight", "o": f"{prefix}.self_attn.o_proj.weight"},
            {"position": position},
        )
        feed_forward = PartSpec.make(
            "swiglu",
            {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size},
            {"gate": f"{prefix}.mlp.gate_proj.weight", "up": f"{prefix}.mlp.up_proj.weight",
             "down": f"{prefix}.mlp.down_proj.weight"},
        )
        layers.append(LayerSpec.make("pre_norm", mixer, feed_forward, {
            "input": norm(f"{prefix}.input_layernorm.weight"),
            "post_mixer": norm(f"{prefix}.post_attention_layernorm.weight"),
        }))
    embedding_name = "model.embed_tokens.weight"
    head_name = embedding_name if cfg.tie_word_embeddings else "lm_head.weight"
    sizes = {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}
    return ModelSpec(
        architecture=LlamaConfig.ARCHITECTURE,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec.make("token_embedding", sizes, {"table": embedding_name}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm("model.norm.weight"),
        head=PartSpec.make("lm_head", sizes, {"weight": head_name}),
        bos_token_id=cfg.bos_token_id,
        eos_token_ids=tuple(cfg.eos_token_id),
    )


def _ignorable(cfg: LlamaConfig):
    patterns = ["*.rotary_emb.inv_freq"]
    if cfg.tie_word_embeddings:
        patterns.append("lm_head.weight")
    return patterns


register_architecture(Architecture(
    name=LlamaConfig.ARCHITECTURE,
    read_config=LlamaConfig.from_dict,
    build_spec=llama_spec,
    ignorable_tensors=_ignorable,
))
