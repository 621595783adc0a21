"""Rikanex, put together from parts.

Per layer: one layer norm (weight and bias) whose output both the attention and the feed-forward read, their outputs
added to the residual stream together (``ParallelBlock``); attention without rotation, with unit-norm queries and keys,
a sliding window, a sink per head in the softmax, values mixed with those of the first mixing layer, and an output
gate (``GatedAttentionMixer``); a dense SwiGLU feed-forward, a mixture of small SwiGLU experts chosen by a sigmoid
router with a correction (``RoutedExpertsFeedForward``), or none.  Around the layers: an embedding times a constant,
a final layer norm and an untied head.  Layers may differ in every size; each comes from its own entry of the
configuration.  Tensor names: ``embed``, ``l<i>.norm1`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``
(+ ``.b``), ``head``.
"""

from __future__ import annotations

from ..config.model_config import ConfigError, RikanexConfig
from ..config.registry import register_model
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, LMHead, TokenEmbedding, make
from .spec import ModelSpec

VALUE_MIX_KEY = "rikanex_first_values"


@register_model("Rikanex", RikanexConfig)
def build_rikanex(cfg: RikanexConfig) -> ModelSpec:
  W, eps = cfg.width, cfg.norm_eps
  embedding = TokenEmbedding("embed", cfg.vocab, W, scale=cfg.embedding_scale, tensor="embed")
  blocks = []
  source = None            # the first layer whose values are mixed into the later ones
  for i in range(len(cfg.layers)):
    p = f"l{i}"
    m = cfg.mixer_of(i)
    value_mix = None
    if m.v_mix:
      if source is None:
        source, value_mix = m, "source"
      else:
        if (m.kv_heads, m.vdim) != (source.kv_heads, source.vdim):
          raise ConfigError(f"layers[{i}].mixer mixes its values with those of the first such layer, "
                            f"but has {m.kv_heads} x {m.vdim} values a token against {source.kv_heads} x {source.vdim}")
        value_mix = "mixed"
    mixer = make(MIXERS, "gated_attention", f"{p}.mix", W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, eps, m.window,
                 sinks=True, gated=True, value_mix=value_mix, value_mix_key=VALUE_MIX_KEY)
    mlp = cfg.mlp_of(i)
    if mlp is None:
      ffn = None
    elif mlp.kind == "dense":
      ffn = make(FEED_FORWARDS, "swiglu", f"{p}.mlp", W, mlp.ff, tensors=("gate", "up", "down"))
    else:
      ffn = make(FEED_FORWARDS, "routed_experts", f"{p}.mlp", W, mlp.ff, mlp.experts, mlp.top)
    norm = make(NORMS, "layernorm", f"{p}.norm1", W, eps, weight_name=f"{p}.norm1", bias_name=f"{p}.norm1.b")
    blocks.append(make(BLOCKS, "parallel", p, norm, mixer, ffn))
  final_norm = make(NORMS, "layernorm", "final.norm", W, eps, weight_name="final.norm", bias_name="final.norm.b")
  lm_head = LMHead("head", cfg.vocab, W, tensor="head")
  return ModelSpec(config=cfg, embedding=embedding, blocks=blocks, final_norm=final_norm, lm_head=lm_head,
                   position_encodings=[], aliases={}, init_std=cfg.initializer_range)
