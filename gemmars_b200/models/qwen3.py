"""Qwen3 dense (``model_type: "qwen3"``, ``Qwen3ForCausalLM``): configuration, plan, tensor names.

A pre-norm decoder: grouped-query attention with an RMSNorm per head on q and k before the
rotation, a SiLU-gated MLP, RMSNorm, causal attention, tied or untied output head.

This module is all that knows the architecture: it reads config.json into ``Qwen3Config`` and
turns it into a ``ModelPlan`` of generic parts bound to the checkpoint's tensor names.

Reference: src/config.rs:383-507 (``QwenConfig`` and its dense switches, :462-469),
src/qwen.rs:458-544 (tensor names and shapes), src/qwen.rs:658-794 (forward).
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional

from ..config.base import ModelConfig, key
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

FULL, SLIDING = "full_attention", "sliding_attention"


@dataclasses.dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int = key(int)
    hidden_size: int = key(int)
    intermediate_size: int = key(int)
    num_hidden_layers: int = key(int)
    num_attention_heads: int = key(int)
    num_key_value_heads: int = key(int)
    #: Per-head width; heads * head_dim may differ from hidden_size.  Absent: hidden / heads.
    head_dim: Optional[int] = key("opt_int", None)
    rms_norm_eps: float = key(float, 1e-6)          # src/config.rs:404-405
    #: Rotation base.  Top level for Qwen3, else rope_parameters.rope_theta; the reference's
    #: value when both are absent is 10,000,000 (src/config.rs:490-496).
    rope_theta: float = key(float, 10_000_000.0)
    partial_rotary_factor: float = key(float, 1.0)  # src/config.rs:498-506
    tie_word_embeddings: bool = key(bool, False)    # src/config.rs:425-426
    #: Biases on the q, k, v and o projections (the reference's Qwen path has none).
    attention_bias: bool = key(bool, False)
    #: Longest sequence the model accepts; absent: bounded by the cache alone.
    max_position_embeddings: Optional[int] = key("opt_int", None)
    eos_token_id: List[int] = key("int_list", [])   # src/config.rs:322-347
    #: Windowed layers: only when use_sliding_window is set; layer_types then says which layers
    #: ("sliding_attention") see only the last sliding_window keys.  The reference's dense path
    #: is full attention everywhere (src/config.rs:465-469).
    use_sliding_window: bool = key(bool, False)
    sliding_window: Optional[int] = key("opt_int", None)
    layer_types: Optional[List[str]] = key("str_list", None)
    #: Scaling of the rotation for long contexts (YaRN and the like).  The reference's Qwen path
    #: does not read it (src/config.rs:490-506 takes rope_theta and partial_rotary_factor only)
    #: and no part here implements one, so anything but null or the "default" type is refused:
    #: running such a checkpoint unscaled would give other logits than the model's.
    rope_scaling: Optional[dict] = key("opt_dict", None)
    model_type: str = key(str, "qwen3")

    @classmethod
    def from_dict(cls, raw):
        raw = dict(raw)
        text = raw.get("text_config") if isinstance(raw.get("text_config"), dict) else raw
        rp = text.get("rope_parameters")
        if isinstance(rp, dict):  # src/config.rs:490-506: rope_parameters wins over the top level
            text = dict(text)
            for k in ("rope_theta", "partial_rotary_factor"):
                if rp.get(k) is not None:
                    text[k] = rp[k]
            kind = rp.get("rope_type", rp.get("type"))
            if kind not in (None, "default") and text.get("rope_scaling") is None:
                text["rope_scaling"] = {k: v for k, v in rp.items() if k not in ("rope_theta", "partial_rotary_factor")}
            if "text_config" in raw and isinstance(raw["text_config"], dict):
                raw["text_config"] = text
            else:
                raw = text
        return super().from_dict(raw)

    def validate(self):
        p = []
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads"):
            if getattr(self, name) <= 0:
                p.append(f"{name}: must be positive, got {getattr(self, name)}")
        if p:
            return p
        if self.head_dim is not None and self.head_dim <= 0:
            p.append(f"head_dim: must be positive, got {self.head_dim}")
        if self.head_dim is None and self.hidden_size % self.num_attention_heads:
            p.append("head_dim: absent and hidden_size is not a multiple of num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads:
            p.append(f"num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                     f"num_key_value_heads ({self.num_key_value_heads})")
        if not p and self.rotary_dim % 2:
            p.append(f"partial_rotary_factor: rotates {self.rotary_dim} dimensions, not an even number")
        if not self.rms_norm_eps > 0:
            p.append(f"rms_norm_eps: must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            p.append(f"rope_theta: must be positive, got {self.rope_theta}")
        if self.max_position_embeddings is not None and self.max_position_embeddings <= 0:
            p.append("max_position_embeddings: must be positive")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                p.append("layer_types length mismatch")  # src/config.rs:482-484
            for t in self.layer_types:
                if t not in (FULL, SLIDING):
                    p.append(f"layer_types: unknown layer type {t!r}")
                    break
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            p.append("use_sliding_window is set but sliding_window is not a positive integer")
        if self.use_sliding_window and self.layer_types is None:
            p.append("use_sliding_window is set but layer_types is absent: which layers are windowed is not "
                     "known (max_window_layers is not read); give layer_types or unset use_sliding_window")
        if self.rope_scaling is not None:
            kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type"))
            if kind not in (None, "default"):
                p.append(f"rope_scaling: rotation scaling of type {kind!r} is not implemented "
                         "(only null or \"default\")")
        return p

    @property
    def dim_per_head(self) -> int:
        return self.head_dim if self.head_dim is not None else self.hidden_size // self.num_attention_heads

    @property
    def rotary_dim(self) -> int:
        """Rotated dimensions per head (src/config.rs:498-506)."""
        return int(self.dim_per_head * self.partial_rotary_factor)

    def layer_window(self, layer: int) -> Optional[int]:
        if not self.use_sliding_window or self.layer_types is None:
            return None
        return self.sliding_window if self.layer_types[layer] == SLIDING else None


def tensor_prefix(names) -> str:
    """The checkpoint's name prefix, probed on embed_tokens (src/qwen.rs:461-469)."""
    if names is None:
        return "model."
    for p in ("model.language_model.", "model.", ""):
        if p + "embed_tokens.weight" in names:
            return p
    return "model."  # the loader then reports the embedding as missing


def build_plan(cfg: Qwen3Config, names=None) -> ModelPlan:
    """The plan of a Qwen3 checkpoint whose tensor names are ``names`` (None: the usual ones)."""
    p = tensor_prefix(names)
    h, hd = cfg.hidden_size, cfg.dim_per_head
    nh, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    embed_name = p + "embed_tokens.weight"
    # Tied when the configuration says so or when the checkpoint has no head (src/qwen.rs:472).
    tied = cfg.tie_word_embeddings or (names is not None and "lm_head.weight" not in names)

    def norm(name):
        return PartSpec("rmsnorm", {"size": h, "eps": cfg.rms_norm_eps}, {"weight": name})

    layers = []
    for l in range(cfg.num_hidden_layers):
        lp = f"{p}layers.{l}."
        ap, mp = lp + "self_attn.", lp + "mlp."
        at = {"q": ap + "q_proj.weight", "k": ap + "k_proj.weight", "v": ap + "v_proj.weight",
              "o": ap + "o_proj.weight", "q_norm": ap + "q_norm.weight", "k_norm": ap + "k_norm.weight"}
        if cfg.attention_bias:
            at.update({"q_bias": ap + "q_proj.bias", "k_bias": ap + "k_proj.bias",
                       "v_bias": ap + "v_proj.bias", "o_bias": ap + "o_proj.bias"})
        mixer = PartSpec("attention", {
            "hidden_size": h, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
            "qk_norm": True, "qk_norm_eps": cfg.rms_norm_eps, "bias": cfg.attention_bias,
            "window": cfg.layer_window(l),
            "scale": None,  # head_dim ** -0.5 (src/qwen.rs:737)
            "position": PartSpec("rotary", {"head_dim": hd, "rotary_dim": cfg.rotary_dim,
                                            "theta": cfg.rope_theta}),
        }, at)
        ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": cfg.intermediate_size,
                                     "activation": "silu"},
                       {"gate": mp + "gate_proj.weight", "up": mp + "up_proj.weight",
                        "down": mp + "down_proj.weight"})
        layers.append(LayerSpec.prenorm(mixer, ffn, norm(lp + "input_layernorm.weight"),
                                        norm(lp + "post_attention_layernorm.weight")))
    plan = ModelPlan(
        hidden_size=h, vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab_size, "hidden_size": h, "scale": None},
                           {"weight": embed_name}),
        layers=layers,
        schedule=[ScheduleEntry(l) for l in range(cfg.num_hidden_layers)],
        final_norm=norm(p + "norm.weight"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": h},
                      {"weight": embed_name if tied else "lm_head.weight"}),
        max_positions=cfg.max_position_embeddings or 0,
        stop_ids=list(cfg.eos_token_id),
        # a tied model may still carry a head it does not use (src/qwen.rs:472-485); older
        # checkpoints store the rotation's inverse frequencies, which are recomputed here
        ignored_tensors=(["lm_head.weight"] if tied else []) + ["*.rotary_emb.inv_freq"],
    )
    plan.validate()
    return plan


def checkpoint_layout(cfg: Qwen3Config) -> dict:
    """{tensor name: (shape, kind)} of a complete checkpoint; kind is "matrix", "norm" or
    "bias" (shapes: src/qwen.rs:398-403, 384-386, 474-486, 524-525)."""
    h, hd, i = cfg.hidden_size, cfg.dim_per_head, cfg.intermediate_size
    nh, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    out = {"model.embed_tokens.weight": ((cfg.vocab_size, h), "matrix")}
    for l in range(cfg.num_hidden_layers):
        lp = f"model.layers.{l}."
        ap, mp = lp + "self_attn.", lp + "mlp."
        out[lp + "input_layernorm.weight"] = ((h,), "norm")
        out[ap + "q_proj.weight"] = ((nh * hd, h), "matrix")
        out[ap + "k_proj.weight"] = ((nkv * hd, h), "matrix")
        out[ap + "v_proj.weight"] = ((nkv * hd, h), "matrix")
        out[ap + "o_proj.weight"] = ((h, nh * hd), "matrix")
        if cfg.attention_bias:
            out[ap + "q_proj.bias"] = ((nh * hd,), "bias")
            out[ap + "k_proj.bias"] = ((nkv * hd,), "bias")
            out[ap + "v_proj.bias"] = ((nkv * hd,), "bias")
            out[ap + "o_proj.bias"] = ((h,), "bias")
        out[ap + "q_norm.weight"] = ((hd,), "norm")
        out[ap + "k_norm.weight"] = ((hd,), "norm")
        out[lp + "post_attention_layernorm.weight"] = ((h,), "norm")
        out[mp + "gate_proj.weight"] = ((i, h), "matrix")
        out[mp + "up_proj.weight"] = ((i, h), "matrix")
        out[mp + "down_proj.weight"] = ((h, i), "matrix")
    out["model.norm.weight"] = ((h,), "norm")
    if not cfg.tie_word_embeddings:
        out["lm_head.weight"] = ((cfg.vocab_size, h), "matrix")
    return out


register_architecture(["Qwen3ForCausalLM", "qwen3"], Qwen3Config, build_plan, checkpoint_layout)
