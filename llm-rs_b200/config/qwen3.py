"""Typed configuration of the Qwen3 dense decoder, read from its own config.json keys.

Keys, requirements and defaults follow llm-core/src/model/config.rs:15-43 (required:
vocab_size, hidden_size, num_hidden_layers, num_attention_heads, intermediate_size;
defaults: num_key_value_heads = heads, head_dim = hidden/heads,
max_position_embeddings 2048, rope_theta 10000, rms_norm_eps 1e-5,
tie_word_embeddings false, hidden_act SiLU) and llm-core/src/backends/candle.rs:711-722
(eos_token_id, default 2). Keys the reference leaves unread (attention_bias,
sliding_window, use_sliding_window, max_window_layers, layer_types, rope_scaling) are
read here and either implemented or refused.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .errors import ConfigError

_REQUIRED = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
             "intermediate_size")


def _int(raw, key, default=None, minimum=1):
    v = raw.get(key, default)
    if v is None:
        raise ConfigError(f"{key} missing from config")
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"{key} must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"{key} must be >= {minimum}, got {v}")
    return v


def _float(raw, key, default):
    v = raw.get(key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{key} must be a number, got {v!r}")
    return float(v)


def _bool(raw, key, default):
    v = raw.get(key, default)
    if v is None:
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"{key} must be true or false, got {v!r}")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    # One entry per layer: 0 = attends to every earlier key, w > 0 = to the last w keys.
    layer_windows: Tuple[int, ...] = ()
    # Layers that skip the rotation (llm-core/src/model/config.rs:45-59).
    no_rope_layers: Tuple[bool, ...] = ()
    eos_token_ids: Tuple[int, ...] = (2,)
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    # Window keys as config.json spells them, kept for to_dict().
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen3Config":
        for key in _REQUIRED:
            if key not in raw:
                raise ConfigError(f"{key} missing from config")
        hidden = _int(raw, "hidden_size")
        layers = _int(raw, "num_hidden_layers")
        heads = _int(raw, "num_attention_heads")
        kv_heads = _int(raw, "num_key_value_heads", heads)
        if "head_dim" in raw and raw["head_dim"] is not None:
            head_dim = _int(raw, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(
                    f"head_dim absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(
                f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} must be even for the rotation")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported for Qwen3 (silu only)")
        # The rotation's base and kind: top-level ``rope_theta`` / ``rope_scaling`` (the keys the
        # reference knows, config.rs:25), or the ``rope_parameters`` object in which newer files of the
        # architecture store both ({"rope_theta": ..., "rope_type": "default"}) with no top-level key.
        theta_raw = {k: raw[k] for k in ("rope_theta",) if raw.get(k) is not None}
        for key in ("rope_scaling", "rope_parameters"):
            obj = raw.get(key)
            if obj in (None, {}):
                continue
            if not isinstance(obj, dict):
                raise ConfigError(f"{key} must be an object, got {obj!r}")
            kind = obj.get("rope_type", obj.get("type", "default"))
            if kind not in ("default", None):
                raise ConfigError(f"{key} {obj!r} is not supported (only the default rotation is)")
            if obj.get("rope_theta") is not None:
                inner = obj["rope_theta"]
                if "rope_theta" in theta_raw and float(theta_raw["rope_theta"]) != float(inner):
                    raise ConfigError(f"rope_theta {theta_raw['rope_theta']!r} and {key}.rope_theta {inner!r} disagree")
                theta_raw["rope_theta"] = inner

        use_window = _bool(raw, "use_sliding_window", False)
        window = raw.get("sliding_window")
        if window is not None:
            window = _int(raw, "sliding_window")
        max_window_layers = raw.get("max_window_layers")
        if max_window_layers is not None:
            max_window_layers = _int(raw, "max_window_layers", minimum=0)
        layer_types = raw.get("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, list) or len(layer_types) != layers:
                raise ConfigError(f"layer_types must list {layers} entries")
            windows = []
            for i, t in enumerate(layer_types):
                if t == "full_attention":
                    windows.append(0)
                elif t == "sliding_attention":
                    if window is None:
                        raise ConfigError(f"layer_types[{i}] is sliding_attention but sliding_window is null")
                    windows.append(window)
                else:
                    raise ConfigError(f"layer_types[{i}] = {t!r} is not supported")
            use_window = any(windows)
        elif use_window:
            if window is None:
                raise ConfigError("use_sliding_window is true but sliding_window is null")
            first = layers if max_window_layers is None else max_window_layers
            windows = [window if i >= first else 0 for i in range(layers)]
        else:
            windows = [0] * layers

        no_rope = raw.get("no_rope_layers")
        if no_rope is None:
            no_rope = [False] * layers
        else:
            if not isinstance(no_rope, list) or len(no_rope) != layers:
                raise ConfigError(f"no_rope_layers must list {layers} entries")
            no_rope = [bool(v) for v in no_rope]

        # Absent: the reference's default 2 (candle.rs:711-722). null: the model names no end token,
        # so nothing ends a request but its length.
        eos = raw.get("eos_token_id", 2)
        if eos is None:
            eos = []
        if isinstance(eos, bool) or not isinstance(eos, (int, list)):
            raise ConfigError(f"eos_token_id must be an integer, a list or null, got {eos!r}")
        eos_ids = tuple(eos) if isinstance(eos, list) else (eos,)
        if not all(isinstance(e, int) and not isinstance(e, bool) for e in eos_ids):
            raise ConfigError(f"eos_token_id must hold integers, got {eos!r}")

        dtype = raw.get("torch_dtype", raw.get("dtype", "bfloat16"))
        if dtype not in ("float32", "float16", "bfloat16"):
            raise ConfigError(f"torch_dtype {dtype!r} is not supported")

        theta = _float(theta_raw, "rope_theta", 10000.0)
        eps = _float(raw, "rms_norm_eps", 1e-5)
        if theta <= 0:
            raise ConfigError(f"rope_theta must be positive, got {theta}")
        if eps <= 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {eps}")
        return cls(
            vocab_size=_int(raw, "vocab_size"), hidden_size=hidden, num_hidden_layers=layers,
            num_attention_heads=heads, intermediate_size=_int(raw, "intermediate_size"),
            num_key_value_heads=kv_heads, head_dim=head_dim,
            max_position_embeddings=_int(raw, "max_position_embeddings", 2048),
            rope_theta=theta, rms_norm_eps=eps,
            tie_word_embeddings=_bool(raw, "tie_word_embeddings", False),
            hidden_act=act, attention_bias=_bool(raw, "attention_bias", False),
            layer_windows=tuple(windows), no_rope_layers=tuple(no_rope),
            eos_token_ids=eos_ids, bos_token_id=raw.get("bos_token_id"), torch_dtype=dtype,
            use_sliding_window=use_window, sliding_window=window,
            max_window_layers=max_window_layers)

    def to_dict(self) -> Dict[str, Any]:
        """The config.json form (round-trips through ``from_dict``). Keys without a value are left out
        rather than written as null, which stricter readers of the same file refuse."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture], "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "use_sliding_window": self.use_sliding_window,
            "torch_dtype": self.torch_dtype,
        }
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.max_window_layers is not None:
            d["max_window_layers"] = self.max_window_layers
        if len(self.eos_token_ids) == 1:
            d["eos_token_id"] = self.eos_token_ids[0]
        else:
            d["eos_token_id"] = list(self.eos_token_ids)   # [] = no end token (absent would mean 2)
        if any(self.layer_windows):
            d["layer_types"] = ["sliding_attention" if w else "full_attention" for w in self.layer_windows]
        if any(self.no_rope_layers):
            d["no_rope_layers"] = list(self.no_rope_layers)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d
