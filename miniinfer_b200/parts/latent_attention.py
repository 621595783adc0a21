"""Attention through a latent, as a mixer part over the paged cache.

For the normalised rows ``h`` of a step, with ``H`` heads, per head ``dim`` unrotated and ``rot_dim`` rotated query/key
values and ``vdim`` value values, a query latent of ``q_rank`` and a key/value latent of ``kv_rank`` values:

  * one fused product gives the query latent, the key/value row and the gate's logits: ``[W_dq h | W_dkv h | W_g h]``;
  * ``c_q = rmsnorm(W_dq h)`` (weight, eps), ``q = W_uq c_q``, laid out head by head as ``[dim unrotated | rot_dim rotated]``;
  * of ``W_dkv h`` the first ``kv_rank`` values, RMS-normed with a weight, are the latent ``c``; the last ``rot_dim`` are one key
    part shared by all heads, rotated by the token's position (as the queries' rotated parts are); only ``c`` and that part
    are cached;
  * per head the unrotated key is ``W_uk c`` and the value ``W_uv c``; the score of query i and key j is
    ``scale * (q_plain . W_uk c_j + q_rot . k_rot_j) = scale * ((W_uk^T q_plain) . c_j + q_rot . k_rot_j)``, so the keys' up-projection
    is applied to the query instead, once per token, and attention runs over ONE key/value head whose key row is
    ``[c | k_rot]`` and whose value row is ``c``: ``H`` query heads of ``kv_rank + rot_dim`` values on it (sink in the softmax's
    denominator if ``sinks``), each giving ``sum_j p_j c_j``, which ``W_uv`` of the head then takes to ``vdim`` values;
  * ``gated``: head h's output is multiplied by ``sigmoid((W_g h)_h)``, one gate a head; then the output projection.

The cache keeps rows of ``kv_rank + rot_dim`` values rounded up to a multiple of 16, zero-filled.  The two per-head
products (``W_uk^T`` on the queries, ``W_uv`` on the outputs) are one batched launch each over the heads of the rows.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.specs import CacheSpec, PagedKVSpec
from ..kernels import ops
from .base import ParamSpec, Piece, PositionEncoding, whole
from .mixer import AttentionMixer


class LatentAttentionMixer(AttentionMixer):
  def __init__(self, name: str, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int,
               scale: float, norm_eps: float, rotary: PositionEncoding, rotary_interleaved: bool = False, sinks: bool = True,
               gated: bool = True, tensors: Optional[Dict[str, str]] = None):
    cache_hd = -(-(kv_rank + rot_dim) // 16) * 16
    super().__init__(name, hidden_size, num_heads, 1, cache_hd, scale, norm_eps, rotary, None)
    for what, v in (("dim", dim), ("rot_dim", rot_dim), ("vdim", vdim), ("q_rank", q_rank), ("kv_rank", kv_rank)):
      if v <= 0:
        raise ValueError(f"{name}: {what} must be positive, got {v}")
    if rot_dim % 2 or getattr(rotary, "rotary_dim", None) != rot_dim:
      raise ValueError(f"{name}: the rotated part has {rot_dim} values; it must be even and the position encoding must cover exactly it")
    self.dim, self.rot_dim, self.vdim, self.q_rank, self.kv_rank = dim, rot_dim, vdim, q_rank, kv_rank
    self.cache_head_dim = cache_hd
    self.rotary_interleaved = bool(rotary_interleaved)
    self.sinks, self.gated = bool(sinks), bool(gated)
    t = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "g": "g",
         "o": "o", "sink": "sink"}
    t.update(tensors or {})
    self.tensors = t
    self.q_off, self.kv_off = 0, q_rank
    self.g_off = q_rank + kv_rank + rot_dim
    self.down_width = self.g_off + (num_heads if gated else 0)

  def cache_spec(self) -> Optional[CacheSpec]:
    return PagedKVSpec(1, self.cache_head_dim, None)

  def param_specs(self) -> Dict[str, ParamSpec]:
    W, H, D, R, Dv, Q, C, n, t = (self.hidden_size, self.num_heads, self.dim, self.rot_dim, self.vdim, self.q_rank, self.kv_rank,
                                  self.name, self.tensors)
    pieces = [Piece(f"{n}.{t['dq']}", self.q_off, (Q, W)), Piece(f"{n}.{t['dkv']}", self.kv_off, (C + R, W))]
    if self.gated:
      pieces.append(Piece(f"{n}.{t['g']}", self.g_off, (H, W)))
    specs = {
      "down": ParamSpec((self.down_width, W), "matrix", [pieces]),
      "dq_norm": ParamSpec((Q,), "vector", [whole(f"{n}.{t['dq_norm']}", (Q,))], init="ones_noise"),
      "dkv_norm": ParamSpec((C,), "vector", [whole(f"{n}.{t['dkv_norm']}", (C,))], init="ones_noise"),
      "uq": ParamSpec((H * (D + R), Q), "matrix", [whole(f"{n}.{t['uq']}", (H * (D + R), Q))]),
      "uk": ParamSpec((H * D, C), "matrix", [whole(f"{n}.{t['uk']}", (H * D, C))]),
      "uv": ParamSpec((H * Dv, C), "matrix", [whole(f"{n}.{t['uv']}", (H * Dv, C))]),
      "o": ParamSpec((W, H * Dv), "matrix", [whole(f"{n}.{t['o']}", (W, H * Dv))]),
    }
    if self.sinks:
      specs["sink"] = ParamSpec((H,), "vector", [whole(f"{n}.{t['sink']}", (H,))])
    return specs

  def bind(self, params) -> None:
    super().bind(params)
    if "uk" in params:
      H, D, C = self.num_heads, self.dim, self.kv_rank
      # the keys' up-projection as it is applied to the queries: per head [kv_rank, dim]
      self.uk_t = params["uk"].view(H, D, C).transpose(1, 2).contiguous()
      self.uv_heads = params["uv"].view(H, self.vdim, C)

  def validate(self, dtype: torch.dtype) -> None:
    if self.cache_head_dim > 256:
      raise ValueError(f"{self.name}: kv_rank + rot_dim = {self.kv_rank + self.rot_dim} is more than the attention kernels' "
                       f"largest head size (256)")

  def takes_residual(self, norm, ctx) -> bool:
    return False

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    T = x.shape[0]
    H, D, R, Dv, Q, C, hdp = self.num_heads, self.dim, self.rot_dim, self.vdim, self.q_rank, self.kv_rank, self.cache_head_dim
    if cache.kind != "paged":
      raise RuntimeError(f"{self.name}: attention needs a paged cache, got {cache.kind!r}")
    table = self.position.rotary_table()
    down = ctx.ws.buffer("latent_down", (T, self.down_width), ctx.dtype)
    ops.linear(down, x, self.down)
    cq = ctx.ws.buffer("latent_cq", (T, Q), ctx.dtype)
    ops.latent_down(down, self.q_off, self.kv_off, Q, C, R, self.dq_norm, self.dkv_norm, self.qk_norm_eps, cq, table, ctx.positions,
                    self.rotary_interleaved, ctx.slot_mapping[cache.group] if cache.writes else None,
                    cache.tensor if cache.writes else None)
    q = ctx.ws.buffer("latent_q", (T, H * (D + R)), ctx.dtype)
    ops.linear(q, cq, self.uq)
    q_heads = ctx.ws.buffer("q_heads", (T, H * hdp), ctx.dtype)
    ops.latent_query(q, q_heads, H, D, R, C, table, ctx.positions, self.rotary_interleaved)
    ops.linear_batched(q_heads.view(T, H, hdp)[:, :, :C], q.view(T, H, D + R)[:, :, :D], self.uk_t)
    attn = ctx.ws.buffer("attn_out", (T, H * C), ctx.dtype)
    ops.attention(attn, q_heads, cache.tensor, ctx.block_tables[cache.group], self._batch(ctx), H, 1, hdp, self.scale, None,
                  sink=self.sink if self.sinks else None, out_hd=C)
    heads = ctx.ws.buffer("latent_heads", (T, H * Dv), ctx.dtype)
    ops.linear_batched(heads.view(T, H, Dv), attn.view(T, H, C), self.uv_heads,
                       row_gate=down[:, self.g_off:self.g_off + H] if self.gated else None)
    out = ctx.ws.buffer(self.out_buffer, (T, self.hidden_size), ctx.dtype)
    ops.linear(out, heads, self.o)
    return out
