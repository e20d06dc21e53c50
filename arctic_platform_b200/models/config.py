"""Model architecture descriptions.

``DecoderConfig`` covers the Qwen3 dense family and the Qwen3-MoE family (the
architectures named by the benchmark configurations); ``from_hf_dict`` reads a
Hugging Face ``config.json`` so HF safetensors checkpoints load without the
``transformers`` model classes.  The reference resolves models through
``AutoModelForCausalLM`` (arctic_platform/model/loaders/huggingface.py:26-43) and a
Qwen3.5-MoE carve-out (arctic_platform/model/loaders/qwen3_5_moe.py:93-123).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Dict, Optional


@dataclass
class DecoderConfig:
    vocab_size: int = 151936
    hidden_size: int = 2560
    intermediate_size: int = 9728
    num_layers: int = 36
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = True
    qk_norm: bool = True
    max_position_embeddings: int = 40960
    # mixture of experts (0 experts = dense)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    moe_score_func: str = "softmax"              # router scores: softmax over experts, or independent sigmoids
    moe_route_scale: float = 1.0                 # factor on the kept routing weights
    moe_expert_bias: bool = False                # selection bias per expert, nudged toward equal load (no aux loss)
    moe_n_group: int = 1                         # group-limited routing: experts in n groups,
    moe_topk_group: int = 1                      # ... only the best topk_group groups are eligible per token
    shared_expert_intermediate_size: int = 0     # > 0: a dense SwiGLU expert with a sigmoid gate beside the routed ones
    moe_activation: str = "swiglu"               # "relu2": non-gated experts down(relu(up x)^2) (models/latent_moe.py)
    moe_latent_dim: int = 0                      # > 0 (relu2 layer): routed rows are projected to this width for the experts
    # hybrid (Qwen3.5 / Qwen3-Next) features; the defaults describe plain Qwen3
    layer_types: Optional[tuple] = None          # per layer "full_attention" | "linear_attention"
    partial_rotary_factor: float = 1.0           # fraction of head_dim that is rotated
    attn_output_gate: bool = False               # attention output multiplied by sigmoid(gate(x)) before o_proj
    norm_one_plus: bool = False                  # RMSNorm weight stored as (w - 1)
    vlm_layout: bool = False                     # checkpoint is a composite: language model + vision tower
    composite_extra: Optional[Dict[str, Any]] = None   # the composite config's top level (vision_config, token ids)
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    model_type: str = "qwen3"
    name: str = "qwen3"

    def layer_type(self, i: int) -> str:
        return "full_attention" if self.layer_types is None else self.layer_types[i]

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def qkv_size(self) -> int:
        return self.q_size + 2 * self.kv_size

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def num_parameters(self, include_embeddings: bool = True) -> int:
        H, L = self.hidden_size, self.num_layers
        attn = self.qkv_size * H + H * self.q_size + (2 * self.head_dim if self.qk_norm else 0)
        if self.is_moe and self.moe_activation == "relu2":
            W = self.moe_latent_dim or H
            mlp = (self.num_experts * 2 * W * self.moe_intermediate_size + self.num_experts * H
                   + (2 * W * H if self.moe_latent_dim else 0) + 2 * H * self.shared_expert_intermediate_size)
        elif self.is_moe:
            mlp = self.num_experts * 3 * H * self.moe_intermediate_size + self.num_experts * H
        else:
            mlp = 3 * H * self.intermediate_size
        per_layer = attn + mlp + 2 * H
        total = L * per_layer + H
        if include_embeddings:
            total += self.vocab_size * H * (1 if self.tie_word_embeddings else 2)
        return total

    def flops_per_token(self, seq_len: int = 0, backward: bool = True) -> float:
        """Matmul FLOPs per token (2 x active weights) plus causal attention at ``seq_len``; x3 with backward."""
        H, L = self.hidden_size, self.num_layers
        attn_w = self.qkv_size * H + H * self.q_size
        mlp_w = (self.num_experts_per_tok * 3 * H * self.moe_intermediate_size if self.is_moe
                 else 3 * H * self.intermediate_size)
        if self.is_moe and self.moe_activation == "relu2":
            W, k = self.moe_latent_dim or H, self.num_experts_per_tok
            mlp_w = (k * 2 * W * self.moe_intermediate_size + (k * 2 * W * H if self.moe_latent_dim else 0)
                     + 2 * H * self.shared_expert_intermediate_size)
        dense = 2.0 * (L * (attn_w + mlp_w) + self.vocab_size * H)
        attn = 2.0 * 2.0 * L * self.num_heads * self.head_dim * seq_len / 2.0
        return (dense + attn) * (3.0 if backward else 1.0)

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @staticmethod
    def from_hf_dict(d: Dict[str, Any], name: str = "") -> "DecoderConfig":
        from .vlm import text_config_of
        top = d
        d, composite = text_config_of(d)
        mt = d.get("model_type", "qwen3")
        heads = d["num_attention_heads"]
        hybrid = mt in HYBRID_MODEL_TYPES
        return DecoderConfig(
            vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
            intermediate_size=d.get("intermediate_size", 0), num_layers=d["num_hidden_layers"],
            num_heads=heads, num_kv_heads=d.get("num_key_value_heads", heads),
            head_dim=d.get("head_dim", d["hidden_size"] // heads), rms_norm_eps=d.get("rms_norm_eps", 1e-6),
            rope_theta=float(d.get("rope_theta", 1e6)), tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            qk_norm=mt.startswith("qwen3"), max_position_embeddings=d.get("max_position_embeddings", 40960),
            num_experts=d.get("num_experts", 0) or 0, num_experts_per_tok=d.get("num_experts_per_tok", 0) or 0,
            moe_intermediate_size=d.get("moe_intermediate_size", 0) or 0,
            norm_topk_prob=bool(d.get("norm_topk_prob", True)),
            moe_score_func=d.get("scoring_func", d.get("score_func", "softmax")) or "softmax",
            moe_route_scale=float(d.get("routed_scaling_factor", d.get("route_scale", 1.0)) or 1.0),
            moe_expert_bias=bool(d.get("moe_expert_bias", d.get("load_balance_coeff") is not None)),
            moe_n_group=int(d.get("n_group", 1) or 1), moe_topk_group=int(d.get("topk_group", 1) or 1),
            shared_expert_intermediate_size=d.get("shared_expert_intermediate_size",
                                                  d.get("moe_shared_expert_intermediate_size", 0)) or 0,
            moe_activation="relu2" if (d.get("moe_activation") or d.get("mlp_hidden_act")) == "relu2" else "swiglu",
            moe_latent_dim=int(d.get("moe_latent_size", d.get("moe_latent_dim", 0)) or 0),
            layer_types=_hybrid_layer_types(d), partial_rotary_factor=float(d.get("partial_rotary_factor", 1.0)),
            attn_output_gate=hybrid, norm_one_plus=hybrid,
            linear_num_key_heads=d.get("linear_num_key_heads", 0) or 0,
            linear_num_value_heads=d.get("linear_num_value_heads", 0) or 0,
            linear_key_head_dim=d.get("linear_key_head_dim", 0) or 0,
            linear_value_head_dim=d.get("linear_value_head_dim", 0) or 0,
            linear_conv_kernel_dim=d.get("linear_conv_kernel_dim", 4) or 4, model_type=mt, name=name or mt,
            vlm_layout=composite,
            composite_extra={k: v for k, v in top.items() if k != "text_config"} if composite else None)

    def to_hf_dict(self) -> Dict[str, Any]:
        d = {
            "architectures": ["Qwen3MoeForCausalLM" if self.is_moe else "Qwen3ForCausalLM"],
            "model_type": "qwen3_moe" if self.is_moe else "qwen3",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads, "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim, "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings, "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": "silu", "torch_dtype": "bfloat16", "attention_bias": False,
        }
        if self.is_moe:
            d.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob)
            # router variants and the expert layout travel only when they differ from the Qwen3-MoE defaults
            if self.moe_score_func != "softmax":
                d["scoring_func"] = self.moe_score_func
            if self.moe_route_scale != 1.0:
                d["routed_scaling_factor"] = self.moe_route_scale
            if self.moe_n_group > 1:
                d.update(n_group=self.moe_n_group, topk_group=self.moe_topk_group)
            if self.moe_expert_bias:
                d["moe_expert_bias"] = True
            if self.moe_activation != "swiglu":
                d.update(moe_activation=self.moe_activation, moe_latent_size=self.moe_latent_dim,
                         shared_expert_intermediate_size=self.shared_expert_intermediate_size)
        if self.layer_types is not None:
            d.update(model_type=self.model_type, architectures=["Qwen3_5MoeForCausalLM" if self.is_moe else "Qwen3NextForCausalLM"],
                     layer_types=list(self.layer_types), partial_rotary_factor=self.partial_rotary_factor,
                     linear_num_key_heads=self.linear_num_key_heads, linear_num_value_heads=self.linear_num_value_heads,
                     linear_key_head_dim=self.linear_key_head_dim, linear_value_head_dim=self.linear_value_head_dim,
                     linear_conv_kernel_dim=self.linear_conv_kernel_dim,
                     shared_expert_intermediate_size=self.shared_expert_intermediate_size)
        if self.vlm_layout:
            from .vlm import composite_config
            d["model_type"] = self.model_type
            d.pop("architectures", None)
            return composite_config(d, self.composite_extra)
        return d


HYBRID_MODEL_TYPES = ("qwen3_next", "qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text")


def _hybrid_layer_types(d: Dict[str, Any]) -> Optional[tuple]:
    """Hybrid checkpoints list the type of every layer, or give ``full_attention_interval`` (every n-th layer is
    full attention, the others linear attention)."""
    if d.get("model_type") not in HYBRID_MODEL_TYPES:
        return None
    if d.get("layer_types"):
        return tuple(d["layer_types"])
    n = int(d.get("full_attention_interval", 4))
    return tuple("full_attention" if (i + 1) % n == 0 else "linear_attention" for i in range(d["num_hidden_layers"]))


PRESETS: Dict[str, DecoderConfig] = {
    # CPU plumbing model of the first benchmark configuration
    "qwen3-tiny": DecoderConfig(vocab_size=32000, hidden_size=256, intermediate_size=688, num_layers=2, num_heads=4,
                                num_kv_heads=2, head_dim=64, name="qwen3-tiny"),
    # same proportions with head_dim 128 so the GPU attention backward applies
    "qwen3-tiny-d128": DecoderConfig(vocab_size=32000, hidden_size=256, intermediate_size=688, num_layers=2,
                                     num_heads=4, num_kv_heads=2, head_dim=128, name="qwen3-tiny-d128"),
    "qwen3-0.6b": DecoderConfig(hidden_size=1024, intermediate_size=3072, num_layers=28, num_heads=16, num_kv_heads=8,
                                name="qwen3-0.6b"),
    "qwen3-1.7b": DecoderConfig(hidden_size=2048, intermediate_size=6144, num_layers=28, num_heads=16, num_kv_heads=8,
                                name="qwen3-1.7b"),
    "qwen3-4b": DecoderConfig(hidden_size=2560, intermediate_size=9728, num_layers=36, num_heads=32, num_kv_heads=8,
                              name="qwen3-4b"),
    "qwen3-8b": DecoderConfig(hidden_size=4096, intermediate_size=12288, num_layers=36, num_heads=32, num_kv_heads=8,
                              tie_word_embeddings=False, name="qwen3-8b"),
    "qwen3-32b": DecoderConfig(hidden_size=5120, intermediate_size=25600, num_layers=64, num_heads=64, num_kv_heads=8,
                               tie_word_embeddings=False, name="qwen3-32b"),
    "qwen3-30b-a3b": DecoderConfig(hidden_size=2048, intermediate_size=6144, num_layers=48, num_heads=32,
                                   num_kv_heads=4, tie_word_embeddings=False, num_experts=128, num_experts_per_tok=8,
                                   moe_intermediate_size=768, model_type="qwen3_moe", name="qwen3-30b-a3b"),
    # hybrid family at test size: 3 of 4 layers are gated-delta-net linear attention, gated full attention with
    # partial rotary, (1+w) norms, routed experts plus a sigmoid-gated shared expert
    "qwen3.5-moe-tiny": DecoderConfig(vocab_size=32000, hidden_size=128, intermediate_size=256, num_layers=4,
                                      num_heads=4, num_kv_heads=2, head_dim=64, num_experts=4, num_experts_per_tok=2,
                                      moe_intermediate_size=64, shared_expert_intermediate_size=64,
                                      layer_types=("linear_attention", "linear_attention", "linear_attention",
                                                   "full_attention"),
                                      partial_rotary_factor=0.25, attn_output_gate=True, norm_one_plus=True,
                                      linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
                                      linear_value_head_dim=32, model_type="qwen3_5_moe_text", name="qwen3.5-moe-tiny"),
    # hybrid checkpoints at their published sizes (linear attention on 3 of every 4 layers)
    "qwen3-next-80b-a3b": DecoderConfig(vocab_size=151936, hidden_size=2048, intermediate_size=5120, num_layers=48,
                                        num_heads=16, num_kv_heads=2, head_dim=256, tie_word_embeddings=False,
                                        num_experts=512, num_experts_per_tok=10, moe_intermediate_size=512,
                                        shared_expert_intermediate_size=512, rope_theta=1e7,
                                        layer_types=tuple("full_attention" if (i + 1) % 4 == 0 else "linear_attention"
                                                          for i in range(48)),
                                        partial_rotary_factor=0.25, attn_output_gate=True, norm_one_plus=True,
                                        linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128,
                                        linear_value_head_dim=128, max_position_embeddings=262144,
                                        model_type="qwen3_next", name="qwen3-next-80b-a3b"),
    "qwen3.5-moe-35b-a3b": DecoderConfig(vocab_size=248320, hidden_size=2048, intermediate_size=5120, num_layers=40,
                                         num_heads=16, num_kv_heads=2, head_dim=256, tie_word_embeddings=False,
                                         num_experts=256, num_experts_per_tok=8, moe_intermediate_size=512,
                                         shared_expert_intermediate_size=512, rope_theta=1e7,
                                         layer_types=tuple("full_attention" if (i + 1) % 4 == 0 else "linear_attention"
                                                           for i in range(40)),
                                         partial_rotary_factor=0.25, attn_output_gate=True, norm_one_plus=True,
                                         linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128,
                                         linear_value_head_dim=128, max_position_embeddings=262144,
                                         model_type="qwen3_5_moe_text", name="qwen3.5-moe-35b-a3b"),
    "qwen3-moe-tiny": DecoderConfig(vocab_size=32000, hidden_size=256, intermediate_size=688, num_layers=2,
                                    num_heads=4, num_kv_heads=2, head_dim=128, num_experts=8, num_experts_per_tok=2,
                                    moe_intermediate_size=128, model_type="qwen3_moe", name="qwen3-moe-tiny"),
    # latent relu^2 experts behind a group-limited sigmoid router (the Nemotron-H style feed-forward)
    "latent-moe-tiny": DecoderConfig(vocab_size=32000, hidden_size=128, intermediate_size=256, num_layers=2,
                                     num_heads=4, num_kv_heads=2, head_dim=32, num_experts=8, num_experts_per_tok=2,
                                     moe_intermediate_size=64, shared_expert_intermediate_size=96,
                                     moe_activation="relu2", moe_latent_dim=64, moe_score_func="sigmoid",
                                     moe_n_group=4, moe_topk_group=2, moe_route_scale=2.5, moe_expert_bias=True,
                                     model_type="qwen3_moe", name="latent-moe-tiny"),
}


def resolve_config(model_name_or_path: str) -> DecoderConfig:
    """Preset name (case-insensitive, with or without an ``org/`` prefix) or a directory with ``config.json``."""
    p = Path(model_name_or_path)
    if p.is_dir() and (p / "config.json").exists():
        return DecoderConfig.from_hf_dict(json.loads((p / "config.json").read_text()), name=p.name)
    key = model_name_or_path.split("/")[-1].lower()
    if key in PRESETS:
        return PRESETS[key]
    raise ValueError(f"unknown model {model_name_or_path!r}: give a preset ({sorted(PRESETS)}) or a directory "
                     "containing config.json")
