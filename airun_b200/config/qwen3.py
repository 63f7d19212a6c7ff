"""Configuration of the dense Qwen3 decoder, read from its config.json keys.

Keys and defaults follow what the reference reads when it converts a model
folder (crates/airun-cli/src/convert.rs:48-91): ``num_hidden_layers``,
``hidden_size``, ``num_attention_heads`` and ``intermediate_size`` are required;
``num_key_value_heads`` defaults to the head count, ``head_dim`` to
``hidden_size / num_attention_heads``, ``max_position_embeddings`` to 4096,
``rms_norm_eps`` to 1e-6, ``rope_theta`` to 10000 and ``tie_word_embeddings`` to
false.  ``vocab_size`` is required here (the reference takes it from the
tokenizer or the embedding tensor, crates/airun-core/src/config.rs:381-393).
Validation collects every problem before it raises, as the reference's does
(crates/airun-core/src/config.rs:666-701).

Sliding-window keys: ``sliding_window`` (tokens a query sees, itself included;
the reference's rule is "key j is hidden when pos - j >= window",
crates/airun-cuda/kernels/ops.cu:573-576), in force only when
``use_sliding_window`` is true.  Which layers use it is given by ``layer_types``
(a list of "full_attention" / "sliding_attention", one per layer) when present,
else layers with index >= ``max_window_layers`` do.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelConfig

_REQUIRED = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
             "intermediate_size")


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    # One entry per layer: 0 = the layer sees the whole context, w > 0 = the last w tokens.
    layer_windows: Tuple[int, ...] = ()
    architecture: str = "Qwen3ForCausalLM"
    model_type: str = "qwen3"
    torch_dtype: str = "bfloat16"

    # ---- derived sizes (crates/airun-core/src/config.rs:704-734) ----
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def gqa_ratio(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def attn_scale(self) -> float:
        return self.head_dim ** -0.5

    def kv_bytes_per_token(self, element_bytes: int) -> int:
        return 2 * self.kv_dim * element_bytes * self.num_hidden_layers

    def window_of(self, layer: int) -> int:
        return self.layer_windows[layer] if self.layer_windows else 0

    # ---- reading ----
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        problems: List[str] = []
        missing = [k for k in _REQUIRED if d.get(k) is None]
        if missing:
            raise ConfigError("config.json is missing " + ", ".join(missing))

        def integer(key: str, default: Optional[int] = None) -> int:
            v = d.get(key, default)
            if v is None:
                v = default
            if isinstance(v, bool) or not isinstance(v, int):
                problems.append(f"{key} must be an integer, found {v!r}")
                return 1
            return v

        V = integer("vocab_size")
        H = integer("hidden_size")
        L = integer("num_hidden_layers")
        nh = integer("num_attention_heads")
        I = integer("intermediate_size")
        nkv = integer("num_key_value_heads", nh)
        hd_default = H // nh if nh > 0 else 0
        hd = integer("head_dim", hd_default)
        maxpos = integer("max_position_embeddings", 4096)
        # Newer config.json files carry the rotary constants in a dictionary, ``rope_parameters``
        # (or ``rope_scaling``): {"rope_type": "default", "rope_theta": ...}.  The plain type is read
        # like the top-level key; any other type is a scaling rule and is refused below.
        rope_dicts = [v for v in (d.get("rope_parameters"), d.get("rope_scaling")) if isinstance(v, dict) and v]
        raw_theta = d.get("rope_theta")
        for rd in rope_dicts:
            if raw_theta is None and rd.get("rope_theta") is not None:
                raw_theta = rd.get("rope_theta")
        try:
            eps = float(d.get("rms_norm_eps") if d.get("rms_norm_eps") is not None else 1e-6)
            theta = float(raw_theta if raw_theta is not None else 10000.0)
        except (TypeError, ValueError):
            problems.append("rms_norm_eps and rope_theta must be numbers")
            eps, theta = 1e-6, 10000.0
        tied = bool(d.get("tie_word_embeddings", False))

        for name, v in (("vocab_size", V), ("hidden_size", H), ("num_hidden_layers", L),
                        ("num_attention_heads", nh), ("intermediate_size", I),
                        ("num_key_value_heads", nkv), ("head_dim", hd),
                        ("max_position_embeddings", maxpos)):
            if v <= 0:
                problems.append(f"{name} must be positive, found {v}")
        if nh > 0 and nkv > 0 and nh % nkv != 0:
            problems.append(f"num_attention_heads ({nh}) must be a multiple of num_key_value_heads ({nkv})")
        if hd > 0 and hd % 2 != 0:
            problems.append(f"head_dim ({hd}) must be even: rotary pairs dimension i with i + head_dim/2")
        if not eps > 0:
            problems.append(f"rms_norm_eps must be positive, found {eps}")
        if not theta > 0:
            problems.append(f"rope_theta must be positive, found {theta}")
        for key in ("rope_scaling", "rope_parameters"):
            rd = d.get(key)
            if rd in (None, {}):
                continue
            kind = (rd.get("rope_type", rd.get("type", "default")) if isinstance(rd, dict) else rd)
            extra = sorted(set(rd) - {"rope_type", "type", "rope_theta"}) if isinstance(rd, dict) else []
            if kind != "default" or extra:
                problems.append(f"{key} {rd!r} is not supported (only plain rotary positions: "
                                f"rope_type \"default\" with rope_theta)")
        if d.get("attention_bias"):
            problems.append("attention_bias=true is not supported (the dense Qwen3 decoder has no biases)")
        if d.get("hidden_act", "silu") != "silu":
            problems.append(f"hidden_act {d.get('hidden_act')!r} is not supported (only silu)")

        windows: Tuple[int, ...] = ()
        if d.get("use_sliding_window"):
            w = d.get("sliding_window")
            if isinstance(w, bool) or not isinstance(w, int) or w <= 0:
                problems.append(f"use_sliding_window is true but sliding_window is {w!r}")
                w = 0
            types = d.get("layer_types")
            if types is not None:
                if not isinstance(types, list) or len(types) != L:
                    problems.append(f"layer_types must list {L} entries")
                    types = ["full_attention"] * max(L, 0)
                bad = sorted({t for t in types if t not in ("full_attention", "sliding_attention")})
                if bad:
                    problems.append(f"layer_types holds unknown kinds {bad}")
                windows = tuple(w if t == "sliding_attention" else 0 for t in types)
            else:
                first = integer("max_window_layers", L)
                windows = tuple(w if i >= first else 0 for i in range(max(L, 0)))
        if problems:
            raise ConfigError("config.json cannot be used: " + "; ".join(problems))
        if not any(windows):
            windows = ()
        return cls(vocab_size=V, hidden_size=H, num_hidden_layers=L, num_attention_heads=nh,
                   intermediate_size=I, num_key_value_heads=nkv, head_dim=hd,
                   max_position_embeddings=maxpos, rms_norm_eps=eps, rope_theta=theta,
                   tie_word_embeddings=tied, layer_windows=windows,
                   architecture=str(d.get("architectures", ["Qwen3ForCausalLM"])[0]),
                   model_type=str(d.get("model_type", "qwen3")),
                   torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "rope_scaling": None,
            "torch_dtype": self.torch_dtype,
        }
        if any(self.layer_windows):
            d["use_sliding_window"] = True
            d["sliding_window"] = max(self.layer_windows)
            d["layer_types"] = ["sliding_attention" if w else "full_attention"
                                for w in self.layer_windows]
        else:
            d["use_sliding_window"] = False
            d["sliding_window"] = None
        return d

    # ---- what the layers are made of ----
    def layer_specs(self) -> List[LayerSpec]:
        specs = []
        for i in range(self.num_hidden_layers):
            specs.append(LayerSpec(
                mixer="gqa_attention",
                mixer_args=dict(hidden_size=self.hidden_size,
                                num_heads=self.num_attention_heads,
                                num_kv_heads=self.num_key_value_heads,
                                head_dim=self.head_dim,
                                scale=self.attn_scale,
                                window=self.window_of(i),
                                qk_norm=True,
                                qk_norm_eps=self.rms_norm_eps,
                                position="rotary_neox",
                                position_args=dict(rotary_dim=self.head_dim,
                                                   theta=self.rope_theta)),
                feed_forward="swiglu",
                ffn_args=dict(hidden_size=self.hidden_size,
                              intermediate_size=self.intermediate_size),
                norm="rmsnorm",
                norm_args=dict(size=self.hidden_size, eps=self.rms_norm_eps),
            ))
        return specs

    def summary(self) -> str:
        return (f"{self.architecture}: {self.num_hidden_layers} layers, hidden {self.hidden_size}, "
                f"{self.num_attention_heads}/{self.num_key_value_heads} heads x {self.head_dim}, "
                f"ffn {self.intermediate_size}, vocab {self.vocab_size}, "
                f"rope {self.rope_theta:g}, eps {self.rms_norm_eps:g}, "
                f"{'tied' if self.tie_word_embeddings else 'untied'} head"
                + (f", windows {sorted(set(self.layer_windows))}" if self.layer_windows else ""))
