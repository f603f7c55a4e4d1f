"""Typed configuration of the Qwen2.5 dense decoder, read from config.json.

Keys and defaults follow what the reference reads
(runtime/backends/cuda/inferflux_cuda_executor.cpp:543-598): hidden_size,
num_hidden_layers, num_attention_heads, num_key_value_heads, head_dim (else
hidden_size / heads), intermediate_size, vocab_size, max_position_embeddings,
rope_theta (default 10000), rms_norm_eps (default 1e-6), model_type, hidden_act,
torch_dtype.  Read in addition, because they change the result:
tie_word_embeddings, and the window keys use_sliding_window / sliding_window /
max_window_layers with Qwen2's own meaning (layers from max_window_layers on see
only the last sliding_window keys).  A missing key that has no default is an error,
not a zero.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

from .plan import ModelPlan, PartSpec, default_schedule, prenorm_layer
from .registry import ConfigError, register_architecture

_REQUIRED = ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size", "vocab_size")


@register_architecture("Qwen2ForCausalLM", "qwen2")
@dataclass
class Qwen2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int = 32768
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    qkv_bias: bool = True          # only used when weights are made up; files decide by tensor presence

    architecture = "Qwen2ForCausalLM"
    model_type = "qwen2"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen2Config":
        missing = [k for k in _REQUIRED if raw.get(k) is None]
        if missing:
            raise ConfigError(f"config.json (Qwen2): missing keys {missing}")

        def integer(key, default=None):
            v = raw.get(key, default)
            if v is None:
                return None
            if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
                raise ConfigError(f"config.json (Qwen2): `{key}` must be an integer, got {v!r}")
            return int(v)

        heads = integer("num_attention_heads")
        hidden = integer("hidden_size")
        head_dim = integer("head_dim")
        if head_dim is None:
            if heads <= 0 or hidden % heads:
                raise ConfigError(f"config.json (Qwen2): hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        scaling = raw.get("rope_scaling")
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                raise ConfigError(f"config.json (Qwen2): rope_scaling {scaling!r} is not supported "
                                  f"(the rotation here is the unscaled one)")
        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=integer("num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=integer("num_key_value_heads", heads),
            head_dim=head_dim,
            intermediate_size=integer("intermediate_size"),
            vocab_size=integer("vocab_size"),
            max_position_embeddings=integer("max_position_embeddings", 32768),
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            use_sliding_window=bool(raw.get("use_sliding_window", False)),
            sliding_window=integer("sliding_window"),
            max_window_layers=integer("max_window_layers", 0),
            hidden_act=str(raw.get("hidden_act", "silu")),
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
            qkv_bias=bool(raw.get("qkv_bias", raw.get("attention_bias", True))),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        def positive(name):
            if getattr(self, name) <= 0:
                raise ConfigError(f"Qwen2 config: {name} must be positive, got {getattr(self, name)}")
        for n in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                  "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings"):
            positive(n)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"Qwen2 config: num_attention_heads {self.num_attention_heads} is not a "
                              f"multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"Qwen2 config: head_dim {self.head_dim} must be even for the rotation")
        from ..parts.attention import Attention          # late: parts read the plan classes of this package
        try:
            Attention.check_head_dim(self.head_dim)
        except ValueError as e:
            raise ConfigError(f"Qwen2 config: {e}") from None
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"Qwen2 config: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"Qwen2 config: rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(f"Qwen2 config: hidden_act {self.hidden_act!r} is not supported (silu only)")
        if self.use_sliding_window and self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError(f"Qwen2 config: sliding_window must be positive, got {self.sliding_window}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = self.model_type
        return d

    # --------------------------------------------------------------------- plan
    def window_of_layer(self, layer: int) -> Optional[int]:
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        return self.sliding_window if layer >= self.max_window_layers else None

    def to_plan(self) -> ModelPlan:
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("rope", {"theta": self.rope_theta, "rotary_dim": self.head_dim,
                                 "pairing": "split_half"})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                  "intermediate_size": self.intermediate_size})
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = PartSpec("attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "window": self.window_of_layer(i),
                "position": rope,
                "qkv_bias": "if_present",            # files decide by tensor presence
                "invent_bias": self.qkv_bias,        # random-weights mode decides by this
                "scale": None,                       # 1 / sqrt(head_dim)
            })
            layers.append(prenorm_layer(f"model.layers.{i}.", mixer, ffn, norm, norm))
        plan = ModelPlan(
            architecture=self.architecture,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            layers=layers,
            schedule=default_schedule(self.num_hidden_layers),
            final_norm=norm,
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                         "tied": self.tie_word_embeddings}),
        )
        plan.validate()
        return plan
