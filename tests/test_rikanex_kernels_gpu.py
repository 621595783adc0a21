"""Each mechanism of the Rikanex design alone: the kernel against the plain function of tests/plain_rikanex.py, in
float32 and bfloat16, with inputs made so that a fault shows - a key just inside and one just outside every window
given a score that dominates, in prompt portions and in decoding, across page borders; a far key among hundreds; sinks
that dominate or vanish; key and value sizes that differ; experts whose sizes cut every tile."""
import random

import numpy as np
import pytest
import torch

import plain_rikanex as plain
from gpu_helpers import DEV

pytestmark = pytest.mark.gpu


def ops_module():
  from miniinfer_b200.kernels import ops
  return ops


def tol(dtype):
  return 3e-5 if dtype == torch.float32 else 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_times_a_constant(dtype):
  ops = ops_module()
  g = torch.Generator().manual_seed(0)
  table = torch.randn((50, 24), generator=g).to(dtype)
  ids = [3, 49, 0, 3, 17]
  out = torch.empty((5, 24), dtype=torch.float32, device=DEV)
  ops.embedding(out, table.to(DEV), torch.tensor(ids, dtype=torch.int32, device=DEV), 12.5)
  assert torch.equal(out.cpu(), plain.embed(table.float(), ids, 12.5))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [40, 256, 1000])
def test_layer_norm_with_two_pending_outputs(dtype, H):
  ops = ops_module()
  g = torch.Generator().manual_seed(H)
  T = 7
  resid = torch.randn((T, H), generator=g) * 3 + 1.5          # a mean far from zero: E[x^2] - mean^2 would lose digits
  d1, d2 = torch.randn((T, H), generator=g).to(dtype), torch.randn((T, H), generator=g).to(dtype)
  w, b = 1 + 0.1 * torch.randn(H, generator=g), 0.1 * torch.randn(H, generator=g)
  want_sum = resid + (d1.float() + d2.float())
  want = plain.layer_norm(want_sum, w, b, 1e-5)
  r = resid.clone().to(DEV)
  out = torch.empty((T, H), dtype=dtype, device=DEV)
  ops.add_layernorm(out, r, d1.to(DEV), d2.to(DEV), w.to(DEV), b.to(DEV), 1e-5)
  assert torch.allclose(r.cpu(), want_sum, atol=1e-6), "the sum must go back into the residual stream"
  assert float((out.float().cpu() - want).abs().max()) <= tol(dtype)
  # selected rows, one pending output, the residual left alone
  rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
  r2 = resid.clone().to(DEV)
  out2 = torch.empty((3, H), dtype=dtype, device=DEV)
  ops.add_layernorm(out2, r2, None, d2.to(DEV), w.to(DEV), b.to(DEV), 1e-5, rows, False)
  want2 = plain.layer_norm((resid + d2.float())[[5, 0, 5]], w, b, 1e-5)
  assert torch.equal(r2.cpu(), resid)
  assert float((out2.float().cpu() - want2).abs().max()) <= tol(dtype)
  # nothing pending
  out3 = torch.empty((T, H), dtype=dtype, device=DEV)
  ops.add_layernorm(out3, r2, None, None, w.to(DEV), b.to(DEV), 1e-5)
  assert float((out3.float().cpu() - plain.layer_norm(resid, w, b, 1e-5)).abs().max()) <= tol(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Dv", [(4, 2, 16, 32), (6, 3, 24, 24), (3, 1, 80, 48), (2, 2, 128, 128)])
def test_unit_norm_value_mix_and_store(dtype, H, G, D, Dv):
  """Queries and keys divided by their root mean square (no weight), values mixed with the source layer's, keys and
  values stored zero-padded at their slots, queries packed zero-padded."""
  ops = ops_module()
  g = torch.Generator().manual_seed(D + Dv)
  T, P, pages, eps = 9, 4, 6, 1e-5
  hdp = -(-max(D, Dv) // 16) * 16
  width = H * D + G * D + G * Dv + H * Dv
  proj = (torch.randn((T, width), generator=g) * 2).to(dtype)
  q_off, k_off, v_off = 0, H * D, H * D + G * D
  x = proj.float()
  q = plain.unit_rms(x[:, :k_off].view(T, H, D), eps)
  k = plain.unit_rms(x[:, k_off:v_off].view(T, G, D), eps)
  v = x[:, v_off:v_off + G * Dv].view(T, G, Dv)
  lam = torch.tensor(0.3)
  slots = torch.tensor(random.Random(1).sample(range(P, pages * P), T), dtype=torch.int32)
  for mode in (0, 1, 2):
    kv = torch.full((pages, 2, G, P, hdp), 7.0, dtype=dtype, device=DEV)
    q_out = torch.full((T, H * hdp), 7.0, dtype=dtype, device=DEV)
    src = (torch.randn((T, G * Dv), generator=g)).to(dtype)
    other = src.clone().to(DEV) if mode == 2 else (torch.zeros((T, G * Dv), dtype=dtype, device=DEV) if mode == 1 else None)
    ops.qkv_norm_mix_store(proj.to(DEV), q_off, k_off, v_off, q_out, H, G, D, Dv, eps, True, None, None,
                           lam.to(DEV) if mode == 2 else None, other, mode, slots.to(DEV), kv)
    want_v = plain.mix_values(v, src.float().view(T, G, Dv), lam) if mode == 2 else v
    qo = q_out.float().cpu().view(T, H, hdp)
    assert float((qo[..., :D] - q).abs().max()) <= tol(dtype)
    assert not qo[..., D:].any(), "the tail of a packed query head must be zero"
    page, off = (slots // P).long(), (slots % P).long()
    kc = kv[:, 0].float().cpu()[page, :, off]        # [T, G, hdp]
    vc = kv[:, 1].float().cpu()[page, :, off]
    assert float((kc[..., :D] - k).abs().max()) <= tol(dtype)
    assert float((vc[..., :Dv] - want_v).abs().max()) <= tol(dtype)
    assert not kc[..., D:].any() and not vc[..., Dv:].any(), "the tails of cached rows must be zero"
    if mode == 1:
      assert float((other.float().cpu().view(T, G, Dv) - v).abs().max()) <= tol(dtype), "the source layer's values must be left for the others"
    touched = torch.zeros((pages, P), dtype=torch.bool)
    touched[page, off] = True
    assert bool((kv[:, 0, 0, :, 0].float().cpu()[~touched] == 7.0).all()), "a slot of another token was written"


def paged_case(k, v, hdp, page_size, items, seed, dtype):
  """Keys [T, G, D] and values [T, G, Dv] of ONE sequence put into shuffled pages once for every item; ``items``:
  (context length, new tokens).  -> cache layer, block table, AttentionBatch pieces, the positions of the step's rows."""
  from miniinfer_b200.kernels.ops import AttentionBatch
  rng = random.Random(seed)
  G = k.shape[1]
  per = [-(-c // page_size) for c, _ in items]
  ids = list(range(1, sum(per) + 3))
  rng.shuffle(ids)
  kv = torch.zeros((sum(per) + 3, 2, G, page_size, hdp), dtype=torch.float32)
  bt = np.zeros((len(items) + 1, max(per) + 1), dtype=np.int32)
  slots = list(range(len(items)))
  rng.shuffle(slots)
  positions, token_item, q_start, q_len, ctx_len = [], [], [], [], []
  for b, (c, n) in enumerate(items):
    for i in range(per[b]):
      pg = ids.pop()
      bt[slots[b], i] = pg
      lo, hi = i * page_size, min(c, (i + 1) * page_size)
      kv[pg, 0, :, :hi - lo, :k.shape[2]] = k[lo:hi].transpose(0, 1)
      kv[pg, 1, :, :hi - lo, :v.shape[2]] = v[lo:hi].transpose(0, 1)
    q_start.append(len(positions))
    q_len.append(n)
    ctx_len.append(c)
    positions += list(range(c - n, c))
    token_item += [b] * n

  def dev(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)

  tiles = [(b, o) for b, (c, n) in enumerate(items) if n > 1 for o in range(0, n, 64)]
  dec = [b for b, (c, n) in enumerate(items) if n == 1]
  batch = AttentionBatch(
    token_item=dev(token_item), positions=dev(positions), seq_slot=dev(slots), q_start=dev(q_start), q_len=dev(q_len),
    ctx_len=dev(ctx_len), num_tokens=len(positions), num_items=len(items),
    prefill_tiles=dev(tiles).view(-1, 2) if tiles else torch.zeros((0, 2), dtype=torch.int32, device=DEV),
    num_prefill_tiles=len(tiles), prefill_wide_tiles=None, num_prefill_wide_tiles=0,
    decode_items=dev(dec) if dec else torch.zeros(0, dtype=torch.int32, device=DEV), num_decode=len(dec),
    max_ctx_len=max(c for c, _ in items), scratch=None)
  return kv.to(dtype).to(DEV), torch.from_numpy(bt).to(DEV), batch, positions


def edge_sequence(T, H, G, D, Dv, window, probes, seed):
  """A sequence whose queries at the ``probes`` have one key that dominates just inside their window and another just
  outside it (both with values that stand out), so that a window one token off changes the output by units."""
  g = torch.Generator().manual_seed(seed)
  q = plain.unit_rms(torch.randn((T, H, D), generator=g), 1e-6)
  k = plain.unit_rms(torch.randn((T, G, D), generator=g), 1e-6)
  v = torch.randn((T, G, Dv), generator=g)
  for p in probes:
    direction = q[p].view(G, H // G, D).mean(1)
    direction = direction / direction.norm(dim=-1, keepdim=True) * (D ** 0.5)
    if window is not None:
      if p - window + 1 >= 0:
        k[p - window + 1] = direction          # just inside: seen
        v[p - window + 1] = 5.0
      if p - window >= 0:
        k[p - window] = direction              # just outside: not seen
        v[p - window] = -9.0
    else:
      k[0] = direction                         # the farthest key there is
      v[0] = 5.0
  return q, k, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Dv,window,page", [(4, 2, 16, 32, 20, 16), (6, 2, 24, 24, 7, 8), (8, 1, 64, 64, 100, 64),
                                                   (8, 1, 64, 64, 65, 64), (2, 2, 32, 48, None, 16), (16, 1, 128, 128, 130, 64)])
def test_window_edges_sinks_and_gate(dtype, H, G, D, Dv, window, page):
  """Prompt portions that start and end anywhere and single decoded tokens, all read from pages: every row must be the
  plain function's row of the whole sequence.  Probed positions sit at page borders, at the window's length and beyond;
  the sinks include one that dominates and one that vanishes; the gate multiplies the output."""
  ops = ops_module()
  T = 330
  w = window if window is not None else T
  probes = sorted({p for p in (w - 1, w, w + 1, page - 1, page, page + w - 1, page + w, 2 * page + w, 199, 263, 264, T - 1) if 0 <= p < T})
  q, k, v = edge_sequence(T, H, G, D, Dv, window, probes, seed=H * D + (window or 0))
  g = torch.Generator().manual_seed(5)
  sink = torch.randn(H, generator=g)
  sink[0], sink[-1] = 6.0, -30.0
  gate = torch.randn((T, H * Dv), generator=g) * 2
  scale = 1.7 / D ** 0.5
  q, k, v, gate = (t.to(dtype).float() for t in (q, k, v, gate))       # what the kernels are given, exactly
  want = plain.output_gate(plain.attend(q, k, v, scale, window, sink), gate)
  hdp = -(-max(D, Dv) // 16) * 16
  # items: portions (context, new) cut at odd places and across pages, then the probes as decoded tokens
  items = [(T, T), (200, 71), (264, 2), (150, 150), (page + 3, 5)] + [(p + 1, 1) for p in probes]
  kv, bt, batch, positions = paged_case(k, v, hdp, page, items, seed=3, dtype=dtype)
  qp = torch.zeros((len(positions), H, hdp))
  qp[..., :D] = q[positions]
  width = 8 + H * Dv                                   # the gate's columns start at 8 of a wider row
  gate_rows = torch.zeros((len(positions), width))
  gate_rows[:, 8:] = gate[positions]
  out = torch.full((len(positions), H * Dv), 99.0, dtype=dtype, device=DEV)
  ops.attention(out, qp.view(len(positions), H * hdp).to(dtype).to(DEV), kv, bt, batch, H, G, hdp, scale, window,
                sink=sink.to(DEV), gate=gate_rows.to(dtype).to(DEV), gate_offset=8, out_hd=Dv)
  got = out.float().cpu()
  err = (got - want[positions]).abs().max(-1).values
  bad = [(positions[i], round(float(e), 4)) for i, e in enumerate(err) if e > tol(dtype) * 2]
  assert not bad, f"rows that differ from the plain attention (position, error): {bad[:10]}"
  # the probes do tell: with the key just outside the window taken in, the row would move by units
  if window is not None:
    off_by_one = plain.output_gate(plain.attend(q, k, v, scale, window + 1, sink), gate)
    assert float((off_by_one[probes] - want[probes]).abs().max()) > 0.5
  # and without sink or gate the kernels still give plain attention
  out2 = torch.empty_like(out)
  ops.attention(out2, qp.view(len(positions), H * hdp).to(dtype).to(DEV), kv, bt, batch, H, G, hdp, scale, window, out_hd=Dv)
  err2 = (out2.float().cpu() - plain.attend(q, k, v, scale, window, None)[positions]).abs().max()
  assert float(err2) <= tol(dtype) * 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,F,E,top", [(5, 72, 40, 5, 2), (1, 64, 24, 3, 1), (300, 72, 40, 5, 2), (700, 128, 48, 16, 4), (33, 96, 56, 6, 6),
                                         (900, 128, 64, 4, 2), (1100, 192, 136, 6, 3)])
def test_routed_experts(dtype, T, W, F, E, top):
  """Sigmoid scores, choice by score + correction, weights from the scores alone, the weighted sum of the chosen experts:
  few tokens (row tiles of 16) and many (tiles of 64; the last two cases: stretches of 256 rows through the tcgen05
  product in bfloat16), sizes that cut the tiles of the products in both directions."""
  ops = ops_module()
  from miniinfer_b200.engine.context import Workspace
  g = torch.Generator().manual_seed(T + E)
  h = torch.randn((T, W), generator=g).to(dtype)
  Wt = {"router": (torch.randn((E, W), generator=g) * 2 / W ** 0.5).to(torch.bfloat16).float(), "correction": 0.3 * torch.randn(E, generator=g)}
  for e in range(E):
    Wt[f"e{e}.gate"] = (torch.randn((F, W), generator=g) / W ** 0.5).to(dtype).float()
    Wt[f"e{e}.up"] = (torch.randn((F, W), generator=g) / W ** 0.5).to(dtype).float()
    Wt[f"e{e}.down"] = (torch.randn((W, F), generator=g) / F ** 0.5).to(dtype).float()
  want = plain.experts(h.float(), Wt, "", E, top)
  # tokens whose choice hangs on less than rounding moves a score are left out of the comparison
  s = torch.sigmoid(h.float() @ Wt["router"].T) + Wt["correction"]
  ranked = s.sort(-1, descending=True).values
  clear = (ranked[:, top - 1] - ranked[:, top] > 0.01) if top < E else torch.ones(T, dtype=torch.bool)
  gate_up = torch.stack([torch.cat((Wt[f"e{e}.gate"], Wt[f"e{e}.up"])) for e in range(E)]).to(dtype).to(DEV)
  down = torch.stack([Wt[f"e{e}.down"] for e in range(E)]).to(dtype).to(DEV)
  out = torch.empty((T, W), dtype=dtype, device=DEV)
  ws = Workspace(torch.device(DEV))
  for _ in range(2):                                     # twice: the scratch of the first call is used again
    ops.routed_experts(out, h.to(DEV), Wt["router"].to(dtype).to(DEV), Wt["correction"].to(DEV), gate_up, down, top, ws)
  err = (out.float().cpu() - want).abs().max(-1).values
  assert int(clear.sum()) >= 0.7 * T
  assert float(err[clear].max()) <= (1e-4 if dtype == torch.float32 else 4e-2), f"worst rows: {err.topk(min(5, T))}"
  # the weights of a token add up to one: with every expert the same, the mixture is that expert
  for e in range(1, E):
    gate_up[e], down[e] = gate_up[0], down[0]
  ops.routed_experts(out, h.to(DEV), Wt["router"].to(dtype).to(DEV), Wt["correction"].to(DEV), gate_up, down, top, ws)
  one = plain.swiglu(h.float(), Wt["e0.gate"], Wt["e0.up"], Wt["e0.down"])
  assert float((out.float().cpu() - one).abs().max()) <= (1e-4 if dtype == torch.float32 else 4e-2)
