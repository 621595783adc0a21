"""Plain implementation of the Rikanex design: whole sequences, no cache, float32 on the CPU, one function per
mechanism, written from the design's equations and sharing nothing with the package.  It also makes the random
weights of the tests (``make_model``), with distributions under which every mechanism moves the logits.

Notation: ``T`` tokens, ``W`` width, ``H`` query heads, ``G`` key/value heads, ``D`` query/key size, ``Dv`` value size.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------ mechanisms


def embed(table: torch.Tensor, tokens: List[int], scale: float) -> torch.Tensor:
  return table[torch.tensor(tokens, dtype=torch.long)] * scale


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
  mean = x.mean(-1, keepdim=True)
  var = ((x - mean) ** 2).mean(-1, keepdim=True)
  return (x - mean) / torch.sqrt(var + eps) * weight + bias


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
  """x divided by its root mean square over the last axis (no weight)."""
  return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def mix_values(v: torch.Tensor, v_first: torch.Tensor, lam: torch.Tensor) -> torch.Tensor:
  return (1 - lam) * v + lam * v_first


def visible(T: int, window: Optional[int]) -> torch.Tensor:
  """[T, T] bool: query i sees key j iff 0 <= i - j < window (window None: every earlier key and itself)."""
  i = torch.arange(T)[:, None]
  j = torch.arange(T)[None, :]
  ok = i - j >= 0
  if window is not None:
    ok = ok & (i - j < window)
  return ok


def sink_softmax(scores: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
  """Softmax over the last axis of [H, T, T] scores (-inf where masked) whose denominator also holds exp(sink_h)."""
  if sink is None:
    return torch.softmax(scores, dim=-1)
  m = torch.maximum(scores.max(-1, keepdim=True).values, sink.view(-1, 1, 1))
  e = torch.exp(scores - m)
  return e / (e.sum(-1, keepdim=True) + torch.exp(sink.view(-1, 1, 1) - m))


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int],
           sink: Optional[torch.Tensor]) -> torch.Tensor:
  """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H * Dv]; query head h reads key/value head h // (H / G)."""
  T, H, _ = q.shape
  G = k.shape[1]
  kk = k.repeat_interleave(H // G, dim=1)
  vv = v.repeat_interleave(H // G, dim=1)
  s = torch.einsum("ihd,jhd->hij", q, kk) * scale
  s = s.masked_fill(~visible(T, window), float("-inf"))
  p = sink_softmax(s, sink)
  return torch.einsum("hij,jhd->ihd", p, vv).reshape(T, -1)


def output_gate(heads: torch.Tensor, gate_logits: torch.Tensor) -> torch.Tensor:
  return heads * torch.sigmoid(gate_logits)


def swiglu(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
  g = h @ gate.T
  return (g * torch.sigmoid(g) * (h @ up.T)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int):
  """-> (chosen experts [T, top], their weights [T, top])."""
  s = torch.sigmoid(h @ router.T)
  chosen = torch.topk(s + correction, top, dim=-1).indices
  w = torch.gather(s, 1, chosen)
  return chosen, w / (w.sum(-1, keepdim=True) + 1e-20)


def experts(h: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, num_experts: int, top: int) -> torch.Tensor:
  chosen, w = route(h, W[prefix + "router"], W[prefix + "correction"], top)
  out = torch.zeros_like(h)
  for t in range(h.shape[0]):
    for k in range(top):
      e = int(chosen[t, k])
      out[t] += w[t, k] * swiglu(h[t:t + 1], W[f"{prefix}e{e}.gate"], W[f"{prefix}e{e}.up"], W[f"{prefix}e{e}.down"])[0]
  return out


# ------------------------------------------------------------------------------------------ the model


def attention_layer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, carry: dict) -> torch.Tensor:
  T = h.shape[0]
  H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
  q = unit_rms((h @ W[p + "q"].T).view(T, H, D), eps)
  k = unit_rms((h @ W[p + "k"].T).view(T, G, D), eps)
  v = (h @ W[p + "v"].T).view(T, G, Dv)
  if m.get("v_mix"):
    if "first" in carry:
      v = mix_values(v, carry["first"], W[p + "vmix"])
    else:
      carry["first"] = v
  window = m["mask"]["size"] if m.get("mask") else None
  heads = attend(q, k, v, m["scale"], window, W[p + "sink"])
  return output_gate(heads, h @ W[p + "g"].T) @ W[p + "o"].T


def feed_forward(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: Optional[dict]) -> torch.Tensor:
  if mlp is None:
    return torch.zeros_like(h)
  if mlp["kind"] == "dense":
    return swiglu(h, W[p + "gate"], W[p + "up"], W[p + "down"])
  return experts(h, W, p, mlp["router"]["experts"], mlp["router"]["top"])


def forward(W: Dict[str, torch.Tensor], cfg: dict, tokens: List[int]) -> torch.Tensor:
  """Logits [T, vocab] of a whole sequence."""
  eps = cfg["norm"]["eps"]
  x = embed(W["embed"], tokens, cfg["embedding"]["scale"])
  carry: dict = {}
  for i, layer in enumerate(cfg["layers"]):
    h = layer_norm(x, W[f"l{i}.norm1"], W[f"l{i}.norm1.b"], eps)
    x = x + (attention_layer(h, W, f"l{i}.mix.", layer["mixer"], eps, carry) + feed_forward(h, W, f"l{i}.mlp.", layer.get("mlp")))
  return layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T


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


def make_model(cfg: dict, out_dir: str, seed: int) -> str:
  """Writes config.json and model.safetensors (matrices in bfloat16, like a released model) with weights under which
  sinks, mixing, gates, routers and biases all matter: matrices ~ N(0, 1 / fan-in) (the head and the value / output
  projections a little larger), norm weights ~ 1 + 0.1 N, biases and corrections ~ 0.1 N, sinks ~ N(0, 1), mixing
  scalars in 0.2 .. 0.8."""
  from safetensors.torch import save_file
  g = torch.Generator().manual_seed(seed)
  W = cfg["width"]

  def mat(o, i, gain=1.0):
    return (torch.randn((o, i), generator=g) * gain / math.sqrt(i)).to(torch.bfloat16)

  def vec(n, mean, std):
    return (mean + std * torch.randn((n,), generator=g)).to(torch.bfloat16)

  t: Dict[str, torch.Tensor] = {"embed": (torch.randn((cfg["vocab"], W), generator=g) / cfg["embedding"]["scale"]).to(torch.bfloat16)}
  for i, layer in enumerate(cfg["layers"]):
    m, p = layer["mixer"], f"l{i}."
    t[p + "norm1"], t[p + "norm1.b"] = vec(W, 1.0, 0.1), vec(W, 0.0, 0.1)
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t[p + "mix.q"], t[p + "mix.k"] = mat(H * D, W), mat(G * D, W)
    t[p + "mix.v"], t[p + "mix.g"], t[p + "mix.o"] = mat(G * Dv, W, 1.5), mat(H * Dv, W, 2.0), mat(W, H * Dv, 1.5)
    t[p + "mix.sink"] = vec(H, 0.0, 1.0)
    if m.get("v_mix"):
      t[p + "mix.vmix"] = (0.2 + 0.6 * torch.rand((), generator=g)).to(torch.bfloat16)
    mlp = layer.get("mlp")
    if mlp is None:
      continue
    if mlp["kind"] == "dense":
      F = mlp["ff"]
      t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(F, W), mat(F, W), mat(W, F)
    else:
      F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
      for e in range(E):
        t[f"{p}mlp.e{e}.gate"], t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = mat(F, W), mat(F, W), mat(W, F, 2.0)
      t[p + "mlp.router"], t[p + "mlp.correction"] = mat(E, W, 2.0), vec(E, 0.0, 0.1)
  t["final.norm"], t["final.norm.b"] = vec(W, 1.0, 0.1), vec(W, 0.0, 0.1)
  t["head"] = mat(cfg["vocab"], W)
  os.makedirs(out_dir, exist_ok=True)
  with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
    json.dump(cfg, f, indent=1)
  save_file({k: v.contiguous() for k, v in t.items()}, os.path.join(out_dir, "model.safetensors"))
  return out_dir


def layer(heads, kv_heads, dim, vdim, window, v_mix, mlp, scale=None) -> dict:
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
       "v_mix": v_mix}
  if window is not None:
    m["mask"] = {"size": window}
  return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff) -> dict:
  return {"kind": "dense", "ff": ff}


def moe(ff, num_experts, top) -> dict:
  return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": num_experts, "top": top}}


# Small configurations that differ from one another in every size.  P: key and value sizes differ, two kv heads, a
# layer without a feed-forward, a layer that does not mix its values before the first that does, windows that differ
# from layer to layer.  Q: three query heads per kv head, head size 24 (cache rows padded to 32), one expert of three
# per token, a layer that sees every earlier token.  S: head size 64 with eight query heads on one kv head, sixteen
# experts of which four, a window of 100 (longer than a page of 64).
CONFIGS = {
  "P": {"architecture": "Rikanex", "vocab": 300, "width": 64, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-5}, "layers": [
    layer(4, 2, 16, 32, 20, False, dense(96)), layer(4, 2, 16, 32, 33, True, moe(40, 5, 2)),
    layer(2, 2, 32, 32, 9, True, None), layer(4, 2, 16, 32, 20, True, moe(24, 6, 3), scale=0.3)]},
  "Q": {"architecture": "Rikanex", "vocab": 512, "width": 96, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6}, "layers": [
    layer(6, 2, 24, 24, 7, True, moe(56, 3, 1)), layer(6, 2, 24, 24, None, True, dense(160)),
    layer(6, 2, 24, 24, 40, True, moe(56, 3, 1))]},
  "S": {"architecture": "Rikanex", "vocab": 333, "width": 128, "embedding": {"scale": 12.0}, "norm": {"eps": 1e-6}, "layers": [
    layer(8, 1, 64, 64, 100, True, dense(192)), layer(8, 1, 64, 64, 100, True, moe(48, 16, 4)),
    layer(8, 1, 64, 64, 65, True, moe(48, 16, 4))]},
}
