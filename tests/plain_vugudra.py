"""Plain implementation of the Vugudra design: whole sequences, no cache, float32 on the CPU, one function per
mechanism, written from the design's equations and sharing nothing with the package.  It also makes the random
weights of the tests (``make_model``), with distributions under which every mechanism moves the logits.

Notation: ``T`` tokens, ``W`` width, ``H`` query heads, ``G`` key/value heads, ``D`` query/key size, ``Dv`` value size,
``R`` rotated size, ``C`` latent size.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------ small mechanisms


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
  return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
  """RMS norm whose weight is stored around zero."""
  return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
  return rms_unit(x, eps) * w


def silu(x: torch.Tensor) -> torch.Tensor:
  return x * torch.sigmoid(x)


def swiglu(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
  return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def rotary_frequencies(rot: dict) -> tuple:
  """-> (frequencies [dims / 2], factor on cos and sin).  ``rot``: dims, base and, optionally, scaling
  {factor, original, fast, slow} (frequencies between the two wavelength bounds are blended towards f / factor)."""
  dims, base = rot["dims"], float(rot["base"])
  i = torch.arange(dims // 2, dtype=torch.float64)
  f = base ** (-2.0 * i / dims)
  s = rot.get("scaling")
  if not s:
    return f, 1.0

  def dim_of(turns):
    return dims * math.log(s["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

  lo = max(math.floor(dim_of(s["fast"])), 0)
  hi = min(math.ceil(dim_of(s["slow"])), dims - 1)
  ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
  f = f / s["factor"] * ramp + f * (1 - ramp)
  return f, 0.1 * math.log(s["factor"]) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict, layout: str) -> torch.Tensor:
  """x [T, heads, size]; the first rot.dims values of each head are rotated, pairs (i, i + dims/2) in the ``half``
  layout and (2i, 2i + 1) in the ``interleaved`` one."""
  dims = rot["dims"]
  f, m = rotary_frequencies(rot)
  a = positions.to(torch.float64)[:, None] * f[None, :]
  cos, sin = (a.cos() * m).float()[:, None, :], (a.sin() * m).float()[:, None, :]
  out = x.clone()
  if layout == "half":
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out[..., :dims // 2] = u * cos - v * sin
    out[..., dims // 2:dims] = v * cos + u * sin
  else:
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
  return out


def visible(T: int, window: Optional[int], keep_first: int = 0) -> torch.Tensor:
  """[T, T] bool: query i sees key j iff j <= i and (i - j < window or j < keep_first); window None: every j <= i."""
  i = torch.arange(T)[:, None]
  j = torch.arange(T)[None, :]
  ok = j <= i
  if window is not None:
    ok = ok & ((i - j < window) | (j < keep_first))
  return ok


def softmax_with_sink(scores: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
  """Softmax over the last axis of [H, T, T] (-inf where masked); with a sink the denominator also holds exp(sink_h)."""
  if sink is None:
    return torch.softmax(scores, dim=-1)
  m = torch.maximum(scores.max(-1, keepdim=True).values, sink.view(-1, 1, 1))
  e = torch.exp(scores - m)
  return e / (e.sum(-1, keepdim=True) + torch.exp(sink.view(-1, 1, 1) - m))


def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
  """x [T, channels], w [channels, taps] (last column: the current token), zeros before the start."""
  T, taps = x.shape[0], w.shape[1]
  padded = torch.cat([torch.zeros(taps - 1, x.shape[1]), x], dim=0)
  out = torch.zeros_like(x)
  for k in range(taps):
    out = out + padded[k:k + T] * w[:, k]
  return out if bias is None else out + bias


# ------------------------------------------------------------------------------------------ mixers


def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
  T = h.shape[0]
  H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
  pos = torch.arange(T)
  cq = norm_plain(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
  q = (cq @ W[p + "uq"].T).view(T, H, D + R)
  q_plain, q_rot = q[..., :D], rotate(q[..., D:], pos, m["rot"], "half")
  kv = h @ W[p + "dkv"].T
  c = norm_plain(kv[:, :C], W[p + "dkv.norm"], eps)
  k_rot = rotate(kv[:, None, C:], pos, m["rot"], "half")[:, 0]
  k_plain = (c @ W[p + "uk"].T).view(T, H, D)
  v = (c @ W[p + "uv"].T).view(T, H, Dv)
  s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
  s = s.masked_fill(~visible(T, None), float("-inf"))
  pr = softmax_with_sink(s, W[p + "sink"])
  o = torch.einsum("hij,jhd->ihd", pr, v)
  o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
  return o.reshape(T, H * Dv) @ W[p + "o"].T


def windowed_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
  """Grouped-query attention whose values are the keys as projected; window with kept first tokens."""
  T = h.shape[0]
  H, G, D = m["heads"], m["kv_heads"], m["dim"]
  pos = torch.arange(T)
  q = (h @ W[p + "q"].T).view(T, H, D)
  k = (h @ W[p + "k"].T).view(T, G, D)
  v = k
  q = rotate(norm_plain(q, W[p + "q.norm"], eps), pos, m["rot"], "interleaved")
  k = rotate(norm_plain(k, W[p + "k.norm"], eps), pos, m["rot"], "interleaved")
  kk, vv = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
  s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
  mask = m.get("mask")
  s = s.masked_fill(~visible(T, mask["size"] if mask else None, mask.get("keep_first", 0) if mask else 0), float("-inf"))
  o = torch.einsum("hij,jhd->ihd", torch.softmax(s, dim=-1), vv)
  return o.reshape(T, -1) @ W[p + "o"].T


def gated_delta(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
  T = h.shape[0]
  H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
  q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, D)
  k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, D)
  v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, Dv)
  q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
  k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
  beta = torch.sigmoid(h @ W[p + "b"].T)                                                    # [T, H]
  a = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
  g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * F.softplus(a).view(T, H, D))     # [T, H, D]
  out = torch.zeros(T, H, Dv)
  for hd in range(H):
    kv = hd // (H // G)
    S = torch.zeros(D, Dv)
    for t in range(T):
      S = g[t, hd][:, None] * S
      u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
      S = S + torch.outer(k[t, kv], u)
      out[t, hd] = S.T @ q[t, kv]
  gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, Dv)
  out = rms_unit(out, eps) * W[p + "norm"] * gate
  return out.reshape(T, H * Dv) @ W[p + "o"].T


def side_by_side(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
  left = windowed_attention(h, W, p + "left.", m["left"], eps)
  right = gated_delta(h, W, p + "right.", m["right"], eps)
  return 0.5 * (norm_plain(left, W[p + "left.out"], eps) + norm_plain(right, W[p + "right.out"], eps))


def selective_scan(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
  T = h.shape[0]
  I, N, Rk = m["inner"], m["state"], m["dt_rank"]
  xz = h @ W[p + "in"].T
  x, z = xz[:, :I], xz[:, I:]
  x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
  dbc = x @ W[p + "x"].T
  dt = F.softplus(dbc[:, :Rk] @ W[p + "dt"].T + W[p + "dt.b"])          # [T, I]
  B, Cm = dbc[:, Rk:Rk + N], dbc[:, Rk + N:Rk + 2 * N]
  A = -torch.exp(W[p + "A_log"])                                        # [I, N]
  S = torch.zeros(I, N)
  y = torch.zeros(T, I)
  for t in range(T):
    S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
    y[t] = S @ Cm[t] + W[p + "D"] * x[t]
  return (y * silu(z)) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ the model


def mixer(h, W, p, layer, eps):
  kind, m = layer["type"], layer["mixer"]
  if kind == "latent_attention":
    return latent_attention(h, W, p, m, eps)
  if kind == "parallel":
    return side_by_side(h, W, p, m, eps)
  if kind == "mamba1":
    return selective_scan(h, W, p, m)
  raise ValueError(kind)


def layer_order(cfg: dict) -> List[int]:
  n = len(cfg["layers"])
  loop = cfg.get("loop")
  if not loop:
    return list(range(n))
  a, b, times = loop["start"], loop["stop"], loop["times"]
  return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(W: Dict[str, torch.Tensor], cfg: dict, tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
  """Logits [T, vocab] of a whole sequence; ``residuals`` (a list) receives the stream after every layer run."""
  eps = cfg["norm"]["eps"]
  x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
  for i in layer_order(cfg):
    layer, p = cfg["layers"][i], f"l{i}."
    y = mixer(norm_one_plus(x, W[p + "norm1"], eps), W, p + "mix.", layer, eps)
    if layer.get("mlp") is not None:
      y = y + swiglu(norm_one_plus(x, W[p + "norm2"], eps), W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"])
    x = x + y
    if residuals is not None:
      residuals.append(x.clone())
  return norm_one_plus(x, W["final.norm"], eps) @ W["head"].T


def generate(W, cfg, prompt: List[int], n: int) -> List[int]:
  ids = list(prompt)
  for _ in range(n):
    ids.append(int(forward(W, cfg, ids)[-1].argmax()))
  return ids[len(prompt):]


# ------------------------------------------------------------------------------------------ files


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
  from safetensors.torch import load_file
  return {k: (v.float() if v.is_floating_point() else v) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def read_config(model_dir: str) -> dict:
  with open(os.path.join(model_dir, "config.json"), encoding="utf-8") as f:
    return json.load(f)


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
  """Random weights (bfloat16) under which every mechanism matters: matrices ~ N(0, 1 / fan-in), some a little larger;
  one-plus norm weights ~ 0.1 N, plain ones ~ 1 + 0.1 N; sinks ~ N(0, 1); decays that neither vanish nor stay at 1."""
  g = torch.Generator().manual_seed(seed)
  W = cfg["width"]

  def mat(o, i, gain=1.0):
    return (torch.randn((o, i), generator=g) * gain / math.sqrt(i)).to(torch.bfloat16)

  def vec(n, mean, std):
    return (mean + std * torch.randn((n,), generator=g)).to(torch.bfloat16)

  def uni(shape, lo, hi):
    return (lo + (hi - lo) * torch.rand(shape, generator=g)).to(torch.bfloat16)

  t: Dict[str, torch.Tensor] = {"embed": torch.randn((cfg["vocab"], W), generator=g).to(torch.bfloat16)}
  for i, layer in enumerate(cfg["layers"]):
    m, p = layer["mixer"], f"l{i}."
    t[p + "norm1"] = vec(W, 0.0, 0.1)
    if layer["type"] == "latent_attention":
      H, D, R, Dv, C, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
      q = p + "mix."
      t[q + "dq"], t[q + "dq.norm"], t[q + "uq"] = mat(Q, W), vec(Q, 1.0, 0.1), mat(H * (D + R), Q, 1.5)
      t[q + "dkv"], t[q + "dkv.norm"] = mat(C + R, W), vec(C, 1.0, 0.1)
      t[q + "uk"], t[q + "uv"] = mat(H * D, C, 1.5), mat(H * Dv, C, 1.5)
      t[q + "sink"], t[q + "g"], t[q + "o"] = vec(H, 0.0, 1.0), mat(H, W, 2.0), mat(W, H * Dv, 1.5)
    elif layer["type"] == "parallel":
      l, r = m["left"], m["right"]
      q = p + "mix.left."
      H, G, D = l["heads"], l["kv_heads"], l["dim"]
      t[q + "q"], t[q + "k"], t[q + "o"] = mat(H * D, W, 1.5), mat(G * D, W, 1.5), mat(W, H * D)
      t[q + "q.norm"], t[q + "k.norm"], t[q + "out"] = vec(D, 1.0, 0.1), vec(D, 1.0, 0.1), vec(W, 1.0, 0.1)
      q = p + "mix.right."
      H, G, D, Dv, taps, low = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"], max(8, W // 8)
      for name, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
        t[q + name], t[q + name + ".conv"] = mat(rows, W, 2.0), mat(rows, taps, 2.0)
      t[q + "b"], t[q + "A_log"], t[q + "norm"] = mat(H, W, 2.0), uni((H,), -1.0, 1.0), vec(Dv, 1.0, 0.1)
      t[q + "a1"], t[q + "a2"], t[q + "dt_bias"] = mat(low, W), mat(H * D, low, 2.0), uni((H * D,), -3.0, 0.0)
      t[q + "g1"], t[q + "g2"] = mat(low, W), mat(H * Dv, low, 2.0)
      t[q + "o"], t[q + "out"] = mat(W, H * Dv), vec(W, 1.0, 0.1)
    elif layer["type"] == "mamba1":
      I, N, Rk, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
      q = p + "mix."
      t[q + "in"], t[q + "conv"], t[q + "conv.b"] = mat(2 * I, W), mat(I, taps, 2.0), vec(I, 0.0, 0.1)
      t[q + "x"], t[q + "dt"], t[q + "dt.b"] = mat(Rk + 2 * N, I), mat(I, Rk, 1.0), uni((I,), -4.0, -1.0)
      t[q + "A_log"] = torch.log(1.0 + (N - 1) * torch.rand((I, N), generator=g)).to(torch.bfloat16)
      t[q + "D"], t[q + "o"] = vec(I, 1.0, 0.2), mat(W, I)
    else:
      raise ValueError(layer["type"])
    mlp = layer.get("mlp")
    if mlp is not None:
      Ff = mlp["ff"]
      t[p + "norm2"] = vec(W, 0.0, 0.1)
      t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(Ff, W), mat(Ff, W), mat(W, Ff)
  t["final.norm"] = vec(W, 0.0, 0.1)
  t["head"] = mat(cfg["vocab"], W)
  return t


def make_model(cfg: dict, out_dir: str, seed: int, weights: Optional[Dict[str, torch.Tensor]] = None) -> str:
  """Writes config.json and model.safetensors (matrices in bfloat16, like a released model)."""
  from safetensors.torch import save_file
  t = weights if weights is not None else make_weights(cfg, seed)
  os.makedirs(out_dir, exist_ok=True)
  with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
    json.dump(cfg, f, indent=1)
  save_file({k: v.contiguous() for k, v in t.items()}, os.path.join(out_dir, "model.safetensors"))
  return out_dir


# ------------------------------------------------------------------------------------------ configurations


def dense(ff) -> dict:
  return {"kind": "dense", "ff": ff}


def mamba(inner, state, dt_rank, conv, mlp) -> dict:
  return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, mlp, base=10000.0, scaling=None, scale=None) -> dict:
  rot = {"base": base, "dims": rot_dim}
  if scaling is not None:
    rot["scaling"] = scaling
  return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                "q_rank": q_rank, "rot": rot,
                                                "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}, "mlp": mlp}


def side(left: dict, right: dict, mlp) -> dict:
  return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def left_of(heads, kv_heads, dim, window, keep_first, rot_dims=None, base=10000.0, scale=None) -> dict:
  return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window, "keep_first": keep_first},
          "rot": {"base": base, "dims": rot_dims if rot_dims is not None else dim}, "scale": scale if scale is not None else dim ** -0.5}


def right_of(heads, kv_heads, dim, vdim, conv) -> dict:
  return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}

# Small configurations that differ from one another, and from any released model, in every size.
# A: every mixer once, a loop over the two middle layers, a window of 20 keeping 3 first tokens, a partly rotated left head.
# B: the attention layers first, no loop, a layer without feed-forward, windows longer than a page of 16, grouped
#    q/k heads in the delta rule, convolutions of 2 and 3 taps, a state size that is no power of two.
# C: head sizes 64, a window of 100 over pages of 64 keeping 70 first tokens (more than a page), a loop run three times.
CONFIGS = {
  "A": {"architecture": "Vugudra", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
    mamba(96, 8, 6, 4, dense(96)),
    latent(2, 16, 8, 24, 32, 40, dense(80), base=5000.0, scaling=YARN),
    side(left_of(4, 2, 24, 20, 3, rot_dims=16), right_of(2, 1, 16, 24, 3), dense(72)),
    mamba(64, 12, 4, 2, None)]},
  "B": {"architecture": "Vugudra", "vocab": 512, "width": 96, "norm": {"eps": 1e-6}, "layers": [
    side(left_of(6, 2, 16, 33, 17, scale=0.3), right_of(4, 2, 24, 16, 2), None),
    latent(3, 24, 16, 16, 48, 24, dense(128), scale=0.11),
    mamba(128, 5, 8, 3, dense(64)),
    side(left_of(2, 2, 32, 7, 1, rot_dims=8, base=300.0), right_of(3, 3, 8, 40, 4), dense(64))]},
  "C": {"architecture": "Vugudra", "vocab": 333, "width": 128, "norm": {"eps": 1e-6}, "loop": {"start": 0, "stop": 1, "times": 3}, "layers": [
    side(left_of(4, 1, 64, 100, 70), right_of(2, 2, 64, 64, 4), dense(192)),
    latent(4, 32, 32, 64, 96, 64, dense(160), scaling={"factor": 2.0, "original": 128, "fast": 8.0, "slow": 1.0}),
    mamba(256, 16, 8, 4, dense(128))]},
}
