"""The dense Llama decoder as an arrangement of parts.

Layer order and tensors follow hostfog/hfee internal/llm/model.go:115-141 and
internal/llm/forward.go:79-115 (there with GGUF tensor names, here with the names
a ``LlamaForCausalLM`` model folder uses): pre-norm blocks of grouped-query
attention with rotary position encoding and a SwiGLU feed-forward, a final RMS
norm and a linear head that may share the embedding table.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    position = PartSpec("rotary", head_dim=cfg.head_dim, rope_dim=cfg.head_dim, theta=cfg.rope_theta,
                        scaling=cfg.rope_scaling, pairing=cfg.rope_pairing)
    mixer = PartSpec("attention", width=cfg.hidden_size, heads=cfg.num_attention_heads,
                     kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, position=position,
                     window=None, scale=None)
    ffn = PartSpec("swiglu", width=cfg.hidden_size, inner=cfg.intermediate_size)
    norm = PartSpec("rms_norm", width=cfg.hidden_size, eps=cfg.rms_norm_eps)
    block = PartSpec("pre_norm", width=cfg.hidden_size)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec.pre_norm(block, mixer, ffn, norm, norm, names={
            "mixer.q": p + "self_attn.q_proj.weight", "mixer.k": p + "self_attn.k_proj.weight",
            "mixer.v": p + "self_attn.v_proj.weight", "mixer.o": p + "self_attn.o_proj.weight",
            "ffn.gate": p + "mlp.gate_proj.weight", "ffn.up": p + "mlp.up_proj.weight",
            "ffn.down": p + "mlp.down_proj.weight",
            "mixer_norm.weight": p + "input_layernorm.weight",
            "ffn_norm.weight": p + "post_attention_layernorm.weight",
        }))
    names = {"embedding.table": "model.embed_tokens.weight", "final_norm.weight": "model.norm.weight",
             "head.weight": "lm_head.weight"}            # optional in the file when the embeddings are tied
    return ModelSpec(
        width=cfg.hidden_size, vocab=cfg.vocab_size,
        embedding=PartSpec("token", vocab=cfg.vocab_size, width=cfg.hidden_size),
        layers=tuple(layers), schedule=ModelSpec.sequential(cfg.num_hidden_layers),
        final_norm=norm,
        head=PartSpec("linear", vocab=cfg.vocab_size, width=cfg.hidden_size, tied=cfg.tie_word_embeddings),
        names=names, eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id,
        max_positions=cfg.max_position_embeddings,
        ignorable=("*.rotary_emb.inv_freq",),             # a buffer that older exports store beside the weights
    )


def llama_sizes_from_tensors(config_json, shapes):
    """``intermediate_size`` from the rows of the first layer's gate projection when config.json
    leaves it out (hostfog/hfee internal/llm/model.go:146-148 takes the feed-forward's width from the gate
    matrix in the same way)."""
    if "intermediate_size" in config_json:
        return config_json
    gate = shapes.get("model.layers.0.mlp.gate_proj.weight")
    if gate is None or len(gate) != 2:
        return config_json          # the typed configuration will name the missing key
    return {**config_json, "intermediate_size": int(gate[0])}


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_spec, llama_sizes_from_tensors)
