"""The Phi architecture (Hugging Face ``PhiForCausalLM``; Phi-1, Phi-1.5, Phi-2).

The reference runs it as graph label ``phi2`` (arch_detect.go:59): LayerNorm
with bias (model.go:245-252), one norm shared by the attention and the MLP
branch (model.go:2738-2740), parallel residual (model.go:260-267), a plain
ungated MLP (model.go:312-319), split-half partial rotary embedding
(model.go:3084-3092), query scaled by 1/sqrt(head_dim) after the rotation
(model.go:2701-2706), biases on every projection and on the output head
(model.go:1894-1908, 2152-2163).

Every size and constant comes from config.json; nothing is fixed here.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict, fields
from typing import Optional

from .registry import Architecture, register_architecture
from .specs import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec,
                    PositionSpec, default_schedule)

_ACTIVATIONS = ("gelu_new", "gelu", "gelu_pytorch_tanh", "relu")


@dataclass
class PhiConfig:
    """Typed view of a Phi config.json (key names are the file's own)."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    hidden_act: str = "gelu_new"
    max_position_embeddings: int = 2048
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 0.5
    qk_layernorm: bool = False
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    model_type: str = "phi"
    architectures: tuple = ("PhiForCausalLM",)

    @classmethod
    def from_dict(cls, d: dict) -> "PhiConfig":
        required = ("vocab_size", "hidden_size", "intermediate_size",
                    "num_hidden_layers", "num_attention_heads")
        missing = [k for k in required if k not in d]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        if d.get("rope_scaling") not in (None, {}):
            raise ValueError("rope_scaling is not supported for this architecture")
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        if "architectures" in kw and kw["architectures"] is not None:
            kw["architectures"] = tuple(kw["architectures"])
        if "dtype" in d and "torch_dtype" not in d:
            kw["torch_dtype"] = d["dtype"]
        cfg = cls(**kw)
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        return {k: v for k, v in d.items() if v is not None}

    # derived sizes -----------------------------------------------------
    @property
    def kv_heads(self) -> int:
        return self.num_key_value_heads or self.num_attention_heads

    @property
    def head_size(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads

    @property
    def rotary_dim(self) -> int:
        return int(self.partial_rotary_factor * self.head_size)

    def validate(self) -> None:
        """Reject impossible shapes before anything is allocated
        (the reference's check: model.go:1847-1849)."""
        ints = dict(dim=self.hidden_size, layers=self.num_hidden_layers,
                    heads=self.num_attention_heads, kv_heads=self.kv_heads,
                    intermediate=self.intermediate_size, vocab=self.vocab_size,
                    positions=self.max_position_embeddings)
        if any((not isinstance(v, int)) or v <= 0 for v in ints.values()):
            raise ValueError("invalid model configuration: " +
                             " ".join(f"{k}={v}" for k, v in ints.items()))
        if self.head_dim is None and self.hidden_size % self.num_attention_heads:
            raise ValueError(f"hidden_size {self.hidden_size} is not divisible by "
                             f"num_attention_heads {self.num_attention_heads}")
        if self.num_attention_heads % self.kv_heads:
            raise ValueError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                             f"num_key_value_heads {self.kv_heads}")
        if not 0.0 <= self.partial_rotary_factor <= 1.0:
            raise ValueError(f"partial_rotary_factor {self.partial_rotary_factor} outside [0, 1]")
        if self.rotary_dim % 2:
            raise ValueError(f"rotary dimension {self.rotary_dim} "
                             f"(partial_rotary_factor x head_dim) must be even")
        if self.hidden_act not in _ACTIVATIONS:
            raise ValueError(f"hidden_act {self.hidden_act!r} unknown (known: {', '.join(_ACTIVATIONS)})")
        if not (self.layer_norm_eps > 0 and math.isfinite(self.layer_norm_eps)):
            raise ValueError(f"layer_norm_eps {self.layer_norm_eps} must be positive")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ValueError(f"rope_theta {self.rope_theta} must be positive")


def phi_model_spec(cfg: PhiConfig) -> ModelSpec:
    """Layers and schedule of a Phi model: every layer the same parallel block."""
    hd = cfg.head_size
    norm = NormSpec("layernorm", cfg.hidden_size, cfg.layer_norm_eps, bias=True)
    qk_norm = NormSpec("layernorm", hd, cfg.layer_norm_eps, bias=True) if cfg.qk_layernorm else None
    position = (PositionSpec("rope", cfg.rotary_dim, cfg.rope_theta, interleaved=False)
                if cfg.rotary_dim > 0 else PositionSpec("none"))
    mixer = MixerSpec(kind="attention", hidden=cfg.hidden_size,
                      num_heads=cfg.num_attention_heads, num_kv_heads=cfg.kv_heads,
                      head_dim=hd, window=0,
                      # float32(1/sqrt(float64(hd))): model.go:2701-2706
                      q_scale=1.0 / math.sqrt(float(hd)),
                      bias=True, qk_norm=qk_norm, position=position)
    ffn = FeedForwardSpec(kind="dense", hidden=cfg.hidden_size,
                          intermediate=cfg.intermediate_size,
                          activation=cfg.hidden_act, bias=True)
    block = BlockSpec(arrangement="parallel", norm=norm, mixer=mixer, ffn=ffn)
    stops = (cfg.eos_token_id,) if cfg.eos_token_id is not None else ()
    return ModelSpec(hidden=cfg.hidden_size, vocab=cfg.vocab_size,
                     max_positions=cfg.max_position_embeddings,
                     layers=tuple(block for _ in range(cfg.num_hidden_layers)),
                     schedule=default_schedule(cfg.num_hidden_layers),
                     final_norm=norm, tie_embeddings=cfg.tie_word_embeddings,
                     head_bias=True, stop_tokens=stops)


class PhiTensorNames:
    """Names of the tensors in a Phi safetensors file.  The reference loads the
    same roles under llama.cpp names (model.go:1872-1909, 2027-2212):
    token_embd, blk.N.attn_norm, blk.N.attn_{q,k,v}, blk.N.attn_output,
    blk.N.ffn_up, blk.N.ffn_down, output_norm, output."""
    embedding = "model.embed_tokens.weight"
    final_norm = "model.final_layernorm"
    head = "lm_head"
    _layer = {
        "norm": "model.layers.{i}.input_layernorm",
        "mixer.q": "model.layers.{i}.self_attn.q_proj",
        "mixer.k": "model.layers.{i}.self_attn.k_proj",
        "mixer.v": "model.layers.{i}.self_attn.v_proj",
        "mixer.out": "model.layers.{i}.self_attn.dense",
        "mixer.q_norm": "model.layers.{i}.self_attn.q_layernorm",
        "mixer.k_norm": "model.layers.{i}.self_attn.k_layernorm",
        "ffn.up": "model.layers.{i}.mlp.fc1",
        "ffn.down": "model.layers.{i}.mlp.fc2",
    }

    def __init__(self, cfg: PhiConfig):
        self.cfg = cfg

    def layer(self, i: int, slot: str, key: str) -> str:
        """Tensor name of parameter ``key`` (e.g. "q.weight", "weight") of the
        part in ``slot`` ("norm", "mixer", "ffn") of layer i."""
        prefix, _, suffix = key.rpartition(".")
        role = f"{slot}.{prefix}" if prefix else slot
        return self._layer[role].format(i=i) + "." + suffix

    def fused(self) -> dict:
        """Tensors a file may hold fused: the three projections as one matrix (and one bias) with rows
        ordered Q, K, V, as the reference takes blk.N.attn_qkv in place of attn_q/k/v (model.go:2046-2065)."""
        out = {}
        for i in range(self.cfg.num_hidden_layers):
            base = f"model.layers.{i}.self_attn."
            for suffix in ("weight", "bias"):
                out[f"{base}Wqkv.{suffix}"] = [f"{base}{p}_proj.{suffix}" for p in ("q", "k", "v")]
        return out


register_architecture(
    Architecture(name="phi", config_class=PhiConfig, build_spec=phi_model_spec,
                 tensor_names=PhiTensorNames),
    aliases=["phi2", "phi-1", "phi-1_5", "phi1", "phi15"],
)
