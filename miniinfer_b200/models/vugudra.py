"""Vugudra, put together from parts.

Per layer: a block whose mixer and dense SwiGLU feed-forward stand side by side, each behind an RMS norm of its own on the
same residual rows (weights stored around zero), their outputs added to the stream together (``ParallelBlock`` with two
norms).  The mixer is one of

  * ``latent_attention`` - attention through a latent with a rotated key part shared by all heads, stretched rotary
    frequencies, a sink in the softmax and a gate a head (``LatentAttentionMixer``);
  * ``parallel`` - windowed grouped-query attention whose values are its keys, with normed and interleaved-rotated heads
    and kept first tokens (``GatedAttentionMixer`` with those options), beside a gated delta rule (``GatedDeltaMixer``), the
    two outputs RMS-normed and averaged (``SideBySideMixer``);
  * ``mamba1`` - a selective scan (``SelectiveScanMixer``).

``loop`` runs a stretch of layers several times in a row with the same weights: the run list names those blocks again, and
every run has a cache or state of its own.  Around the layers: an embedding, a final norm (stored around zero as well)
and an untied head.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.model_config import VugudraConfig
from ..config.registry import register_model
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LMHead, TokenEmbedding, make
from .spec import LayerRun, ModelSpec


@register_model("Vugudra", VugudraConfig)
def build_vugudra(cfg: VugudraConfig) -> ModelSpec:
  W, eps = cfg.width, cfg.norm_eps
  embedding = TokenEmbedding("embed", cfg.vocab, W, tensor="embed")
  blocks, encodings = [], []

  def rotary(name, rot):
    pe = make(POSITION_ENCODINGS, "scaled_rotary", name, rot.dims, rot.base, cfg.max_position_embeddings, scaling=rot.scaling)
    encodings.append(pe)
    return pe

  for i in range(len(cfg.layers)):
    p = f"l{i}"
    kind, m = cfg.type_of(i), cfg.mixer_of(i)
    if kind == "latent_attention":
      mixer = make(MIXERS, "latent_attention", f"{p}.mix", W, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, eps,
                   rotary(f"{p}.mix.rot", m.rot), rotary_interleaved=False, sinks=True, gated=True)
    elif kind == "mamba1":
      mixer = make(MIXERS, "selective_scan", f"{p}.mix", W, m.inner, m.state, m.dt_rank, m.conv)
    else:
      lc, rc = m
      left = make(MIXERS, "gated_attention", f"{p}.mix.left", W, lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.scale, eps, lc.window,
                  sinks=False, gated=False, rotary=rotary(f"{p}.mix.left.rot", lc.rot), rotary_interleaved=True, norm_weights=True,
                  values_from_keys=True, keep_first=lc.keep_first if lc.window is not None else 0)
      right = make(MIXERS, "gated_delta", f"{p}.mix.right", W, rc.heads, rc.kv_heads, rc.dim, rc.vdim, rc.conv,
                   cfg.low_rank(i, "decay"), cfg.low_rank(i, "gate"), eps)
      mixer = make(MIXERS, "side_by_side", f"{p}.mix", W, left, right, eps, scale=0.5)
    ff = cfg.ff_of(i)
    ffn = make(FEED_FORWARDS, "swiglu", f"{p}.mlp", W, ff, tensors=("gate", "up", "down")) if ff is not None else None
    norm1 = make(NORMS, "rmsnorm", f"{p}.norm1", W, eps, offset=1.0, weight_name=f"{p}.norm1")
    norm2 = make(NORMS, "rmsnorm", f"{p}.norm2", W, eps, offset=1.0, weight_name=f"{p}.norm2") if ffn is not None else None
    blocks.append(make(BLOCKS, "parallel", p, norm1, mixer, ffn, ffn_norm=norm2))
  final_norm = make(NORMS, "rmsnorm", "final.norm", W, eps, offset=1.0, weight_name="final.norm")
  lm_head = LMHead("head", cfg.vocab, W, tensor="head")
  return ModelSpec(config=cfg, embedding=embedding, blocks=blocks, final_norm=final_norm, lm_head=lm_head,
                   position_encodings=encodings, run_list=[LayerRun(i) for i in cfg.layer_order()], aliases={},
                   init_std=cfg.initializer_range)
