"""Typed configuration of the Qwen3 dense decoder, read from its config.json keys.

The reference reads the same keys from a plain dict with no defaults
(model/qwen/qwen_kv_paged.py:135-145, model/qwen/qwen_kv_cont.py:56-59) and
ignores the rest of the file (model/configs/qwen3-4b.json).  Here every key that
changes the arithmetic is either honoured or refused; none is silently ignored.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, Mapping, Optional, Tuple

from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry


class ConfigError(ValueError):
    """config.json is missing a key, or asks for something this engine does not do."""


_REQUIRED = (
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "rope_theta",
)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 40960
    # Per layer: None for full attention, else the number of keys a query sees
    # (itself included): keys at positions p-w+1 .. p.
    layer_windows: Tuple[Optional[int], ...] = ()
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    architecture = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {', '.join(missing)}")
        if d.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported: the projections have no bias")
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act={d['hidden_act']!r} is not supported; only 'silu'")
        if d.get("rope_scaling") is not None:
            raise ConfigError("rope_scaling is not supported; it must be null")
        if d.get("mlp_bias", False):
            raise ConfigError("mlp_bias=true is not supported")

        n_layers = int(d["num_hidden_layers"])
        heads = int(d["num_attention_heads"])
        hidden = int(d["hidden_size"])
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("head_dim is absent and hidden_size is no multiple of num_attention_heads")
            head_dim = hidden // heads

        windows = cls._layer_windows(d, n_layers)

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)

        cfg = cls(
            vocab_size=int(d["vocab_size"]), hidden_size=hidden,
            intermediate_size=int(d["intermediate_size"]), num_hidden_layers=n_layers,
            num_attention_heads=heads, num_key_value_heads=int(d["num_key_value_heads"]),
            head_dim=int(head_dim), rms_norm_eps=float(d["rms_norm_eps"]),
            rope_theta=float(d["rope_theta"]),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=int(d.get("max_position_embeddings", 40960)),
            layer_windows=windows, eos_token_ids=eos_ids,
            bos_token_id=d.get("bos_token_id"),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    @staticmethod
    def _layer_windows(d: Mapping[str, Any], n_layers: int) -> Tuple[Optional[int], ...]:
        """Which layers see only a window of keys.

        `layer_types` (a list of "full_attention" / "sliding_attention") wins when
        present; otherwise `use_sliding_window` with `sliding_window` makes layers
        `max_window_layers` and above windowed.
        """
        window = d.get("sliding_window")
        types = d.get("layer_types")
        if types is not None:
            if len(types) != n_layers:
                raise ConfigError(f"layer_types has {len(types)} entries for {n_layers} layers")
            out = []
            for i, t in enumerate(types):
                if t == "full_attention":
                    out.append(None)
                elif t == "sliding_attention":
                    if not window:
                        raise ConfigError(f"layer {i} is sliding_attention but sliding_window is unset")
                    out.append(int(window))
                else:
                    raise ConfigError(f"layer_types[{i}]={t!r} is not a known attention kind")
            return tuple(out)
        if d.get("use_sliding_window", False):
            if not window:
                raise ConfigError("use_sliding_window=true needs sliding_window")
            first = int(d.get("max_window_layers", n_layers))
            return tuple(int(window) if i >= first else None for i in range(n_layers))
        return tuple(None for _ in range(n_layers))

    @classmethod
    def from_json(cls, path: str | Path) -> "Qwen3Config":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    def validate(self) -> None:
        for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"{f} must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is no multiple of "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even: rotation pairs dim j with j+D/2")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be positive")
        if len(self.layer_windows) != self.num_hidden_layers:
            raise ConfigError("layer_windows must have one entry per layer")
        for w in self.layer_windows:
            if w is not None and w < 1:
                raise ConfigError(f"a window of {w} keys is not possible")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        """config.json content that `from_dict` reads back to an equal object."""
        d = {
            "architectures": [self.architecture], "model_type": "qwen3",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "attention_bias": False, "hidden_act": "silu", "rope_scaling": None,
            "torch_dtype": self.torch_dtype,
        }
        if any(w is not None for w in self.layer_windows):
            window = next(w for w in self.layer_windows if w is not None)
            if any(w not in (None, window) for w in self.layer_windows):
                raise ConfigError("config.json can name only one window size")
            d["sliding_window"] = window
            d["use_sliding_window"] = True
            d["layer_types"] = ["full_attention" if w is None else "sliding_attention"
                                for w in self.layer_windows]
        else:
            d["sliding_window"] = None
            d["use_sliding_window"] = False
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    # --------------------------------------------------------------------- plan
    def plan(self) -> ModelPlan:
        """The model as data: parts by kind, one LayerSpec per layer, run in order.

        Formulas: pre-norm residual blocks (model/qwen/qwen_kv_paged.py:178-189),
        GQA attention with per-head QK-RMSNorm before half-split rotation
        (:130-175), SwiGLU (model/qwen/qwen_kv_cont.py:250-266), final norm and
        tied or untied head (model/qwen/qwen_kv_paged.py:223-224).
        """
        norm_params = {"dim": self.hidden_size, "eps": self.rms_norm_eps}
        position = PartSpec("rotary", {"head_dim": self.head_dim, "rotary_dim": self.head_dim,
                                       "theta": self.rope_theta})
        layers = []
        for i in range(self.num_hidden_layers):
            norms = (PartSpec("rmsnorm", norm_params, "input_layernorm."),
                     PartSpec("rmsnorm", norm_params, "post_attention_layernorm."))
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "scale": float(self.head_dim) ** -0.5,
                "qk_norm_eps": self.rms_norm_eps,
                "position": position,
                "window": self.layer_windows[i],
            }, "self_attn.")
            ff = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                     "intermediate_size": self.intermediate_size}, "mlp.")
            layers.append(LayerSpec("pre_norm", f"model.layers.{i}.", norms, mixer, ff))
        head = PartSpec("lm_head", {
            "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
            "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None,
        }, "lm_head.")
        plan = ModelPlan(
            architecture=self.architecture, hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size,
                                             "hidden_size": self.hidden_size},
                               "model.embed_tokens."),
            layers=tuple(layers),
            order=tuple(RunEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", norm_params, "model.norm."), head=head,
        )
        plan.validate()
        return plan

    def describe(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}
