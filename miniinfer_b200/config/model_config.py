"""Typed model configurations, read from the architecture's own ``config.json`` keys.

The reference keeps every JSON key as an untyped attribute (miniinfer/config/model/base.py:29-31)
and gives defaults in the constructor (miniinfer/config/model/qwen3.py:16-35).  Here every key the
architecture defines is a typed field; keys that change the computation but are not implemented
raise an error that names the key instead of being ignored.
"""

from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
  """A configuration that cannot be run, with the key that is at fault."""


@dataclass
class ModelConfig:
  """What every architecture's configuration gives to the engine."""

  architectures: List[str] = field(default_factory=list)
  model_type: str = ""
  vocab_size: int = 0
  max_position_embeddings: int = 0
  bos_token_id: Optional[int] = None
  eos_token_id: Any = None          # int, list of ints or None
  torch_dtype: Optional[str] = None
  extra: Dict[str, Any] = field(default_factory=dict)

  @classmethod
  def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
    names = {f.name for f in dataclasses.fields(cls)}
    known = {k: v for k, v in d.items() if k in names and k != "extra"}
    cfg = cls(**known)
    cfg.extra = {k: v for k, v in d.items() if k not in names}
    # "dtype" is the newer spelling of "torch_dtype" in config.json files.
    if cfg.torch_dtype is None and "dtype" in cfg.extra:
      cfg.torch_dtype = cfg.extra.pop("dtype")
    cfg.validate()
    return cfg

  @classmethod
  def from_json(cls, path: str) -> "ModelConfig":
    if os.path.isdir(path):
      path = os.path.join(path, "config.json")
    with open(path, encoding="utf-8") as f:
      return cls.from_dict(json.load(f))

  def to_dict(self) -> Dict[str, Any]:
    d = dataclasses.asdict(self)
    extra = d.pop("extra")
    d.update(extra)
    return {k: v for k, v in d.items() if v is not None}

  def eos_ids(self) -> List[int]:
    if self.eos_token_id is None:
      return []
    if isinstance(self.eos_token_id, (list, tuple)):
      return [int(x) for x in self.eos_token_id]
    return [int(self.eos_token_id)]

  def validate(self) -> None:  # pragma: no cover - overridden
    pass


@dataclass
class Qwen3Config(ModelConfig):
  """Qwen3 dense decoder (defaults: miniinfer/config/model/qwen3.py:16-35)."""

  model_type: str = "qwen3"
  vocab_size: int = 151936
  hidden_size: int = 1024
  intermediate_size: int = 3072
  num_hidden_layers: int = 28
  num_attention_heads: int = 16
  num_key_value_heads: Optional[int] = 8
  head_dim: Optional[int] = 128
  hidden_act: str = "silu"
  max_position_embeddings: int = 40960
  initializer_range: float = 0.02
  rms_norm_eps: float = 1e-6
  rope_theta: float = 1000000.0
  rope_scaling: Optional[Dict[str, Any]] = None
  attention_bias: bool = False
  attention_dropout: float = 0.0
  tie_word_embeddings: bool = True
  use_cache: bool = True
  use_sliding_window: bool = False
  sliding_window: Optional[int] = None
  max_window_layers: Optional[int] = None
  layer_types: Optional[List[str]] = None

  def validate(self) -> None:
    if self.num_key_value_heads is None:            # qwen3.py:46-48
      self.num_key_value_heads = self.num_attention_heads
    if self.head_dim is None:                        # qwen3.py:75-79
      if self.hidden_size % self.num_attention_heads:
        raise ConfigError("head_dim is absent and hidden_size is not a multiple of num_attention_heads")
      self.head_dim = self.hidden_size // self.num_attention_heads
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
      v = getattr(self, key)
      if not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{key} must be a positive integer, got {v!r}")
    if self.num_attention_heads % self.num_key_value_heads:
      raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads "
                        f"({self.num_attention_heads} vs {self.num_key_value_heads})")
    if self.head_dim % 2:
      raise ConfigError(f"head_dim must be even for the rotary encoding, got {self.head_dim}")
    if self.hidden_act != "silu":                    # fused_qwen3.py:122-123
      raise ConfigError(f"hidden_act={self.hidden_act!r} is not supported (only 'silu')")
    if self.rope_scaling not in (None, {}):
      kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type"))
      if kind not in (None, "default"):
        raise ConfigError(f"rope_scaling={self.rope_scaling!r} is not supported")
    if self.attention_bias:
      raise ConfigError("attention_bias=true is not supported (the architecture has no QKV bias)")
    if not (self.rms_norm_eps > 0):
      raise ConfigError("rms_norm_eps must be positive")
    if self.use_sliding_window:
      if not self.sliding_window or self.sliding_window <= 0:
        raise ConfigError("use_sliding_window=true needs a positive sliding_window")
    if self.layer_types is not None:
      if len(self.layer_types) != self.num_hidden_layers:
        raise ConfigError("layer_types must have num_hidden_layers entries")
      for t in self.layer_types:
        if t not in ("full_attention", "sliding_attention"):
          raise ConfigError(f"layer_types entry {t!r} is not known")

  def window_of_layer(self, layer: int) -> Optional[int]:
    """The attention window of a layer, or None for all keys.  The reference carries these keys
    without reading them; their meaning here: ``layer_types`` decides if given, else the layers
    from ``max_window_layers`` on are windowed when ``use_sliding_window`` is set."""
    if not self.use_sliding_window or not self.sliding_window:
      return None
    if self.layer_types is not None:
      return int(self.sliding_window) if self.layer_types[layer] == "sliding_attention" else None
    first = self.max_window_layers if self.max_window_layers is not None else 0
    return int(self.sliding_window) if layer >= first else None


@dataclass
class RikanexMixerConfig:
  """The attention of one Rikanex layer (``layers[i].mixer``)."""

  heads: int
  kv_heads: int
  dim: int                      # query / key size of a head
  vdim: int                     # value size of a head
  scale: float                  # the scores' factor
  window: Optional[int]         # ``mask.size``: token i sees j with 0 <= i - j < window; None: every earlier token
  v_mix: bool                   # values mixed with those of the first layer that says so


@dataclass
class RikanexMlpConfig:
  """The feed-forward of one Rikanex layer (``layers[i].mlp``): ``kind`` dense (``ff``) or moe (``ff`` of an expert,
  ``experts``, ``top``)."""

  kind: str
  ff: int
  experts: int = 0
  top: int = 0


@dataclass
class RikanexConfig(ModelConfig):
  """Rikanex: a decoder of parallel layers (one layer norm, attention and feed-forward side by side), windowed
  attention with a sink and an output gate, dense or routed feed-forwards.  ``config.json`` keys: ``architecture``,
  ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers[i].{type, mixer, mlp}``; the layers may differ in
  every size.  The design has no position limit of its own; ``max_position_embeddings`` is only the engine's bound."""

  architecture: str = "Rikanex"
  vocab: int = 0
  width: int = 0
  embedding: Dict[str, Any] = field(default_factory=dict)
  norm: Dict[str, Any] = field(default_factory=dict)
  layers: List[Dict[str, Any]] = field(default_factory=list)
  max_position_embeddings: int = 1 << 30
  initializer_range: float = 0.02

  def validate(self) -> None:
    if not self.architectures:
      self.architectures = [self.architecture]
    self.vocab_size = self.vocab
    for key in ("vocab", "width"):
      v = getattr(self, key)
      if not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{key} must be a positive integer, got {v!r}")
    if not isinstance(self.embedding.get("scale"), (int, float)):
      raise ConfigError("embedding.scale must be a number")
    eps = self.norm.get("eps")
    if not isinstance(eps, (int, float)) or not eps > 0:
      raise ConfigError(f"norm.eps must be a positive number, got {eps!r}")
    if not self.layers:
      raise ConfigError("layers must list at least one layer")
    for i in range(len(self.layers)):
      self.mixer_of(i)
      self.mlp_of(i)

  @property
  def embedding_scale(self) -> float:
    return float(self.embedding["scale"])

  @property
  def norm_eps(self) -> float:
    return float(self.norm["eps"])

  def mixer_of(self, i: int) -> RikanexMixerConfig:
    layer = self.layers[i]
    if layer.get("type") != "attention":
      raise ConfigError(f"layers[{i}].type={layer.get('type')!r} is not a mixer of this design (known: 'attention')")
    m = layer.get("mixer")
    if not isinstance(m, dict):
      raise ConfigError(f"layers[{i}].mixer is missing")
    for key in ("heads", "kv_heads", "dim", "vdim"):
      v = m.get(key)
      if not isinstance(v, int) or v <= 0:
        raise ConfigError(f"layers[{i}].mixer.{key} must be a positive integer, got {v!r}")
    if m["heads"] % m["kv_heads"]:
      raise ConfigError(f"layers[{i}].mixer.heads={m['heads']} must be a multiple of kv_heads={m['kv_heads']}")
    if not isinstance(m.get("scale"), (int, float)):
      raise ConfigError(f"layers[{i}].mixer.scale must be a number")
    mask = m.get("mask")
    window = None
    if mask is not None:
      window = mask.get("size") if isinstance(mask, dict) else None
      if not isinstance(window, int) or window <= 0:
        raise ConfigError(f"layers[{i}].mixer.mask.size must be a positive integer, got {mask!r}")
    return RikanexMixerConfig(m["heads"], m["kv_heads"], m["dim"], m["vdim"], float(m["scale"]), window, bool(m.get("v_mix", False)))

  def mlp_of(self, i: int) -> Optional[RikanexMlpConfig]:
    mlp = self.layers[i].get("mlp")
    if mlp is None:
      return None
    kind = mlp.get("kind")
    if kind == "dense":
      ff = mlp.get("ff")
      if not isinstance(ff, int) or ff <= 0:
        raise ConfigError(f"layers[{i}].mlp.ff must be a positive integer, got {ff!r}")
      return RikanexMlpConfig("dense", ff)
    if kind == "moe":
      ff = (mlp.get("expert") or {}).get("ff")
      router = mlp.get("router") or {}
      experts, top = router.get("experts"), router.get("top")
      for key, v in (("expert.ff", ff), ("router.experts", experts), ("router.top", top)):
        if not isinstance(v, int) or v <= 0:
          raise ConfigError(f"layers[{i}].mlp.{key} must be a positive integer, got {v!r}")
      if top > experts:
        raise ConfigError(f"layers[{i}].mlp.router.top={top} is more than experts={experts}")
      return RikanexMlpConfig("moe", ff, experts, top)
    raise ConfigError(f"layers[{i}].mlp.kind={kind!r} is not known (dense, moe)")

  def to_dict(self) -> Dict[str, Any]:
    d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "embedding": dict(self.embedding),
         "norm": dict(self.norm), "layers": [dict(x) for x in self.layers]}
    d.update(self.extra)
    return d
