"""Each mechanism of the Vugudra design alone: the engine's operation, run over a step cut in several ways, against the
plain function of tests/plain_vugudra.py on the whole sequence.  Inputs are made so that a fault shows: one key whose
score stands out just inside or just outside a window, among the kept first tokens or behind them; states that must
survive a cut in the middle of a convolution's taps; sizes that are no powers of two."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_vugudra as plain
from gpu_helpers import DEV, make_attention_case

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype):
  return 3e-5 if dtype == "float32" else 4e-2


def step_ctx(cuts, slots):
  """The description of a step with one item per entry of ``cuts`` (new tokens) sitting in ``slots``."""
  q_len = list(cuts)
  q_start = [sum(q_len[:i]) for i in range(len(q_len))]
  dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
  return SimpleNamespace(q_start=dev(q_start), q_len=dev(q_len), seq_slot=dev(slots), num_items=len(q_len),
                         token_item=dev([b for b, n in enumerate(q_len) for _ in range(n)]))


def cuts_of(T, sizes):
  out, pos, k = [], 0, 0
  while pos < T:
    n = min(sizes[k % len(sizes)], T - pos)
    out.append(n)
    pos += n
    k += 1
  return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,bias", [(4, True), (2, False), (3, True), (1, False)])
def test_convolution_carries_its_last_inputs_across_steps(dtype, taps, bias):
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(taps)
  C, T = 40, 37
  x = torch.randn((T, C + 8), generator=g).to(DT[dtype])
  w = torch.randn((C, taps), generator=g)
  b = torch.randn((C,), generator=g) if bias else None
  want = plain.silu(plain.causal_conv(x[:, 3:3 + C].float(), w, b))
  for sizes in ((T,), (1,), (2, 1, 5), (taps - 1 or 1, 7), (13, 1, 1, 2)):
    state = torch.zeros((3, max(1, (taps - 1) * C) + 5), dtype=torch.float32, device=DEV)
    state[0].fill_(9.0)                       # another request's slot, to be left alone
    got = torch.zeros((T, C), dtype=DT[dtype], device=DEV)
    xd, pos = x.to(DEV), 0
    for n in cuts_of(T, sizes):
      # the item shares its step with a one-token item of another request in slot 0
      rows = torch.cat((xd[pos:pos + n], xd[:1]))
      out = torch.zeros((n + 1, C), dtype=DT[dtype], device=DEV)
      ops.causal_conv(out, rows[:, 3:3 + C], w.to(DEV), b.to(DEV) if bias else None, state, step_ctx([n, 1], [2, 0]), silu=True)
      got[pos:pos + n] = out[:n]
      pos += n
    assert float((got.float().cpu() - want).abs().max()) <= tol(dtype), f"cut into {sizes}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner,N,rank", [(48, 5, 6), (96, 16, 8), (33, 40, 4)])
def test_selective_scan_against_the_plain_recurrence(dtype, inner, N, rank):
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(inner)
  T = 45
  r = lambda *s: torch.randn(s, generator=g)
  u, z, dt_in = r(T, inner).to(DT[dtype]), r(T, inner).to(DT[dtype]), r(T, inner).to(DT[dtype])
  bc = r(T, 2 * N + 3).to(DT[dtype])
  dt_b, A_log, D = r(inner) - 2.0, torch.log(1 + 3 * torch.rand((inner, N), generator=g)), r(inner)
  # the plain recurrence, spelled out
  S = torch.zeros(inner, N)
  want = torch.zeros(T, inner)
  for t in range(T):
    dt = torch.nn.functional.softplus(dt_in[t].float() + dt_b)
    S = torch.exp(dt[:, None] * -torch.exp(A_log)) * S + (dt * u[t].float())[:, None] * bc[t, 1:1 + N].float()[None, :]
    want[t] = (S @ bc[t, 3 + N:3 + 2 * N].float() + D * u[t].float()) * plain.silu(z[t].float())
  for sizes in ((T,), (1,), (3, 2, 11)):
    state = torch.zeros((4, inner * N + 7), dtype=torch.float32, device=DEV)
    got = torch.zeros((T, inner), dtype=DT[dtype], device=DEV)
    pos = 0
    for n in cuts_of(T, sizes):
      sl = slice(pos, pos + n)
      y = torch.zeros((n, inner), dtype=DT[dtype], device=DEV)
      ops.selective_scan(y, u[sl].to(DEV), dt_in[sl].to(DEV), bc[sl].to(DEV), 1, 3 + N, z[sl].to(DEV), dt_b.to(DEV), A_log.to(DEV),
                         D.to(DEV), state, step_ctx([n], [1]))
      got[sl] = y
      pos += n
    scale = float(want.abs().max())
    assert float((got.float().cpu() - want).abs().max()) <= tol(dtype) * max(1.0, scale), f"cut into {sizes}"
    assert float(state[0].abs().max()) == 0 and float(state[2].abs().max()) == 0      # other slots untouched


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_selective_scan_of_long_portions(dtype):
  """Portions of hundreds of tokens: in bfloat16 a request's tokens run in stretches side by side that are chained
  afterwards (the state a stretch starts from is the stored state carried through the stretches before it); the result
  is the recurrence's, and the state left behind lets the request go on token by token."""
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(2)
  inner, N, T = 40, 12, 1500
  r = lambda *s: torch.randn(s, generator=g)
  u, z, dt_in, bc = r(T, inner).to(DT[dtype]), r(T, inner).to(DT[dtype]), r(T, inner).to(DT[dtype]), r(T, 2 * N).to(DT[dtype])
  dt_b, A_log, D = r(inner) - 2.0, torch.log(1 + 3 * torch.rand((inner, N), generator=g)), r(inner)
  S = torch.zeros(inner, N)
  want = torch.zeros(T, inner)
  for t in range(T):
    dt = torch.nn.functional.softplus(dt_in[t].float() + dt_b)
    S = torch.exp(dt[:, None] * -torch.exp(A_log)) * S + (dt * u[t].float())[:, None] * bc[t, :N].float()[None, :]
    want[t] = (S @ bc[t, N:].float() + D * u[t].float()) * plain.silu(z[t].float())
  for cuts in ((700, 3, 790, 1, 1, 1, 1, 1, 1, 1), (1490,) + (1,) * 10, (520, 515, 465)):
    state = torch.zeros((3, inner * N), dtype=torch.float32, device=DEV)
    got = torch.zeros((T, inner), dtype=DT[dtype], device=DEV)
    pos = 0
    for n in cuts:
      sl = slice(pos, pos + n)
      y = torch.zeros((n, inner), dtype=DT[dtype], device=DEV)
      ops.selective_scan(y, u[sl].to(DEV), dt_in[sl].to(DEV), bc[sl].to(DEV), 0, N, z[sl].to(DEV), dt_b.to(DEV), A_log.to(DEV),
                         D.to(DEV), state, step_ctx([n], [1]))
      got[sl] = y
      pos += n
    assert pos == T
    scale = float(want.abs().max())
    assert float((got.float().cpu() - want).abs().max()) <= tol(dtype) * max(1.0, scale), f"cut into {cuts}"
    assert float((state[1].cpu().view(inner, N) - S).abs().max()) <= 1e-3 * max(1.0, float(S.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv", [(2, 1, 16, 24), (4, 4, 32, 48), (3, 3, 8, 40), (2, 2, 64, 64), (1, 1, 128, 128), (2, 1, 40, 8)])
def test_gated_delta_rule_against_the_plain_recurrence(dtype, H, G, D, Dv):
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(H * D + Dv)
  T, eps = 40, 1e-5
  r = lambda *s: torch.randn(s, generator=g)
  q, k, v = r(T, G * D).to(DT[dtype]), r(T, G * D).to(DT[dtype]), r(T, H * Dv).to(DT[dtype])
  a, b, gate = r(T, H * D).to(DT[dtype]), r(T, H).to(DT[dtype]), r(T, H * Dv).to(DT[dtype])
  dt_bias, A_log, norm_w = r(H * D) - 1.0, torch.rand((H,), generator=g) - 0.5, 1 + 0.1 * r(Dv)
  qf = q.float().view(T, G, D)
  kf = k.float().view(T, G, D)
  qf = qf / torch.sqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
  kf = kf / torch.sqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
  decay = torch.exp(-torch.exp(A_log)[None, :, None] * torch.nn.functional.softplus(a.float().view(T, H, D) + dt_bias.view(H, D)))
  beta = torch.sigmoid(b.float())
  want = torch.zeros(T, H, Dv)
  for h in range(H):
    S = torch.zeros(D, Dv)
    for t in range(T):
      S = decay[t, h][:, None] * S
      S = S + torch.outer(kf[t, h // (H // G)], beta[t, h] * (v[t].float().view(H, Dv)[h] - S.T @ kf[t, h // (H // G)]))
      want[t, h] = S.T @ qf[t, h // (H // G)]
  want = plain.rms_unit(want, eps) * norm_w * torch.sigmoid(gate.float().view(T, H, Dv))
  for sizes in ((T,), (1,), (2, 7, 1, 33)):
    state = torch.zeros((3, H * D * Dv + 3), dtype=torch.float32, device=DEV)
    got = torch.zeros((T, H * Dv), dtype=DT[dtype], device=DEV)
    pos = 0
    for n in cuts_of(T, sizes):
      sl = slice(pos, pos + n)
      out = torch.zeros((n, H * Dv), dtype=DT[dtype], device=DEV)
      ops.gated_delta(out, q[sl].to(DEV), k[sl].to(DEV), v[sl].to(DEV), a[sl].to(DEV), b[sl].to(DEV), gate[sl].to(DEV), dt_bias.to(DEV),
                      A_log.to(DEV), norm_w.to(DEV), eps, state, step_ctx([n], [2]), H, G, D, Dv)
      got[sl] = out
      pos += n
    assert float((got.float().cpu() - want.reshape(T, -1)).abs().max()) <= tol(dtype) * 2, f"cut into {sizes}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv", [(2, 1, 24, 40), (1, 1, 128, 64)])
def test_gated_delta_rule_of_long_portions(dtype, H, G, D, Dv):
  """Portions of hundreds of tokens: in bfloat16 a request's tokens run in stretches side by side - each from a zero state
  and, in further columns that start as the identity, as the map of the state it starts from - which are chained
  afterwards; the result is the recurrence's, and the state left behind lets the request go on token by token."""
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(D + Dv)
  T, eps = 1300, 1e-5
  r = lambda *s: torch.randn(s, generator=g)
  q, k, v = r(T, G * D).to(DT[dtype]), r(T, G * D).to(DT[dtype]), r(T, H * Dv).to(DT[dtype])
  a, b, gate = r(T, H * D).to(DT[dtype]), r(T, H).to(DT[dtype]), r(T, H * Dv).to(DT[dtype])
  dt_bias, A_log, norm_w = r(H * D) - 3.0, torch.rand((H,), generator=g) - 0.5, 1 + 0.1 * r(Dv)
  qf, kf = q.float().view(T, G, D), k.float().view(T, G, D)
  qf = qf / torch.sqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
  kf = kf / torch.sqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
  decay = torch.exp(-torch.exp(A_log)[None, :, None] * torch.nn.functional.softplus(a.float().view(T, H, D) + dt_bias.view(H, D)))
  beta = torch.sigmoid(b.float())
  want = torch.zeros(T, H, Dv)
  last = torch.zeros(H, D, Dv)
  for h in range(H):
    S = torch.zeros(D, Dv)
    for t in range(T):
      S = decay[t, h][:, None] * S
      S = S + torch.outer(kf[t, h // (H // G)], beta[t, h] * (v[t].float().view(H, Dv)[h] - S.T @ kf[t, h // (H // G)]))
      want[t, h] = S.T @ qf[t, h // (H // G)]
    last[h] = S
  want = plain.rms_unit(want, eps) * norm_w * torch.sigmoid(gate.float().view(T, H, Dv))
  for cuts in ((600, 2, 690, 1, 1, 1, 1, 1, 1, 1, 1), (1290,) + (1,) * 10, (520, 780)):
    state = torch.zeros((3, H * D * Dv), dtype=torch.float32, device=DEV)
    got = torch.zeros((T, H * Dv), dtype=DT[dtype], device=DEV)
    pos = 0
    for n in cuts:
      sl = slice(pos, pos + n)
      out = torch.zeros((n, H * Dv), dtype=DT[dtype], device=DEV)
      ops.gated_delta(out, q[sl].to(DEV), k[sl].to(DEV), v[sl].to(DEV), a[sl].to(DEV), b[sl].to(DEV), gate[sl].to(DEV), dt_bias.to(DEV),
                      A_log.to(DEV), norm_w.to(DEV), eps, state, step_ctx([n], [2]), H, G, D, Dv)
      got[sl] = out
      pos += n
    assert pos == T
    assert float((got.float().cpu() - want.reshape(T, -1)).abs().max()) <= tol(dtype) * 2, f"cut into {cuts}"
    assert float((state[2].cpu().view(H, D, Dv) - last).abs().max()) <= 2e-3 * max(1.0, float(last.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_norms_of_one_row_and_the_mean_of_two_normed_outputs(dtype):
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(4)
  T, W, eps = 9, 72, 1e-5
  resid, d1, d2 = torch.randn((T, W), generator=g), torch.randn((T, W), generator=g).to(DT[dtype]), torch.randn((T, W), generator=g).to(DT[dtype])
  w1, w2 = torch.randn((W,), generator=g), torch.randn((W,), generator=g)
  s = resid + (d1.float() + d2.float())
  r = resid.clone().to(DEV)
  o1, o2 = (torch.zeros((T, W), dtype=DT[dtype], device=DEV) for _ in range(2))
  ops.add_rmsnorm_pair(o1, o2, r, d1.to(DEV), d2.to(DEV), w1.to(DEV), w2.to(DEV), eps)
  assert float((r.cpu() - s).abs().max()) <= 1e-6
  assert float((o1.float().cpu() - plain.norm_plain(s, w1, eps)).abs().max()) <= tol(dtype)
  assert float((o2.float().cpu() - plain.norm_plain(s, w2, eps)).abs().max()) <= tol(dtype)
  rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
  o3 = torch.zeros((2, W), dtype=DT[dtype], device=DEV)
  r2 = resid.clone().to(DEV)
  ops.add_rmsnorm_pair(o3, None, r2, d1.to(DEV), d2.to(DEV), w1.to(DEV), None, eps, rows, False)
  assert torch.equal(r2.cpu(), resid)
  assert float((o3.float().cpu() - plain.norm_plain(s[[7, 2]], w1, eps)).abs().max()) <= tol(dtype)
  a, b = d1, d2
  out = torch.zeros((T, W), dtype=DT[dtype], device=DEV)
  ops.rms_pair_sum(out, a.to(DEV), b.to(DEV), w1.to(DEV), w2.to(DEV), eps, 0.5)
  want = 0.5 * (plain.norm_plain(a.float(), w1, eps) + plain.norm_plain(b.float(), w2, eps))
  assert float((out.float().cpu() - want).abs().max()) <= tol(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batched_product_over_the_heads_of_a_row(dtype):
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(6)
  for M, B, N, K, pad in ((5, 3, 20, 12, 4), (70, 2, 65, 33, 0), (1, 4, 7, 129, 1)):
    x = torch.randn((M, B * (K + pad)), generator=g).to(DT[dtype])
    w = (torch.randn((B, N, K), generator=g) / math.sqrt(K)).to(DT[dtype])
    gate = torch.randn((M, B + 2), generator=g).to(DT[dtype])
    out = torch.zeros((M, B * N), dtype=DT[dtype], device=DEV)
    xv = x.to(DEV).view(M, B, K + pad)[:, :, pad:]
    ops.linear_batched(out.view(M, B, N), xv, w.to(DEV), row_gate=gate.to(DEV))
    want = torch.einsum("mbk,bnk->mbn", x.view(M, B, K + pad)[:, :, pad:].float(), w.float()) * torch.sigmoid(gate.float()[:, :B, None])
    assert float((out.float().cpu().view(M, B, N) - want).abs().max()) <= tol(dtype)
    # a product whose inner size is no multiple of 8, and one whose input is a column range, through ops.linear
    y = torch.zeros((M, N), dtype=DT[dtype], device=DEV)
    ops.linear(y, xv[:, 0, :], w[0].to(DEV).contiguous())
    assert float((y.float().cpu() - x.view(M, B, K + pad)[:, 0, pad:].float() @ w[0].float().T).abs().max()) <= tol(dtype)


def _paged(keys, values, page, hdp, dtype, seed):
  """Keys / values [n, G, size] of one request into a shuffled paged cache; -> (layer, block table row 2)."""
  n, G = keys.shape[0], keys.shape[1]
  pages = -(-n // page)
  order = list(range(1, pages + 3))
  np.random.RandomState(seed).shuffle(order)
  kv = torch.zeros((pages + 3, 2, G, page, hdp), dtype=dtype)
  bt = torch.zeros((4, pages + 1), dtype=torch.int32)
  for j in range(n):
    p = order[j // page]
    bt[2, j // page] = p
    kv[p, 0, :, j % page, :keys.shape[2]] = keys[j].to(dtype)
    kv[p, 1, :, j % page, :values.shape[2]] = values[j].to(dtype)
  return kv.to(DEV), bt.to(DEV)


def _batch(ctx_len, n_new, slot=2):
  from miniinfer_b200.kernels.ops import AttentionBatch
  dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
  tiles = [(0, o) for o in range(0, n_new, 64)] if n_new > 1 else []
  return AttentionBatch(token_item=dev([0] * n_new), positions=dev(list(range(ctx_len - n_new, ctx_len))), seq_slot=dev([slot]),
                        q_start=dev([0]), q_len=dev([n_new]), ctx_len=dev([ctx_len]), num_tokens=n_new, num_items=1,
                        prefill_tiles=dev(tiles).view(-1, 2) if tiles else torch.zeros((0, 2), dtype=torch.int32, device=DEV),
                        num_prefill_tiles=len(tiles), prefill_wide_tiles=None, num_prefill_wide_tiles=0,
                        decode_items=dev([0]) if n_new == 1 else torch.zeros(0, dtype=torch.int32, device=DEV),
                        num_decode=int(n_new == 1), max_ctx_len=ctx_len, scratch=None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,page,window,keep", [(32, 16, 20, 3), (80, 64, 75, 19), (64, 64, 100, 70), (128, 64, 300, 130), (128, 64, 70, 5), (64, 64, 129, 128), (48, 8, 33, 17), (16, 16, 7, 1), (32, 16, 40, 0)])
def test_window_with_kept_first_tokens_edge_keys_stand_out(dtype, hd, page, window, keep):
  """The query of the last token is aligned with ONE key whose score then dominates; the output must be that key's value
  when it is visible - the window's last key, a kept first token, the last kept one - and must not show it when it is
  just outside the window or just behind the kept tokens.  In a prompt portion and as a decoded token."""
  from miniinfer_b200.kernels import ops
  H, G, n = 4, 2, 3 * window + keep + 70
  g = torch.Generator().manual_seed(hd + window)
  keys = torch.randn((n, G, hd), generator=g)
  keys = keys / keys.norm(dim=-1, keepdim=True)
  values = torch.randn((n, G, hd), generator=g)
  kv, bt = _paged(keys, values, page, hd, DT[dtype], 1)
  p = n - 1
  vis = plain.visible(n, window, keep)[p]
  targets = [p - window + 1, p - window, 0, p]
  if keep:
    targets += [keep - 1, keep]
  for n_new in (1, 5, 70):
    for j in targets:
      q = torch.randn((n_new, H, hd), generator=g) * 0.1
      q[-1] = 30.0 * keys[j].repeat_interleave(H // G, dim=0)           # scale 1: the key's score is 30, the others' below 30
      out = torch.zeros((n_new, H * hd), dtype=DT[dtype], device=DEV)
      ops.attention(out, q.reshape(n_new, -1).to(DT[dtype]).to(DEV), kv, bt, _batch(n, n_new), H, G, hd, 1.0, window, keep_first=keep)
      # plain: softmax over the visible keys
      kk = keys.to(DT[dtype]).float().repeat_interleave(H // G, dim=1)
      vv = values.to(DT[dtype]).float().repeat_interleave(H // G, dim=1)
      rows = plain.visible(n, window, keep)[n - n_new:]                      # every row of the portion, not only the last
      s = torch.einsum("ihd,jhd->hij", q.to(DT[dtype]).float(), kk).masked_fill(~rows[None], float("-inf"))
      want_all = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), vv).reshape(n_new, -1)
      assert float((out.float().cpu() - want_all).abs().max()) <= tol(dtype), f"key {j} (visible: {bool(vis[j])}), {n_new} new tokens"
      got = out[-1].float().cpu()
      near = float((got.view(H, hd) - vv[j]).abs().max()) < 0.05
      assert near == bool(vis[j]), f"key {j}: visible {bool(vis[j])}, but the output {'is' if near else 'is not'} its value"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,R,Dv,C,Q,interleaved", [(2, 16, 8, 24, 32, 40, False), (3, 24, 16, 16, 48, 24, False), (4, 32, 32, 64, 96, 64, True)])
def test_latent_attention_pieces_against_the_plain_formulas(dtype, H, D, R, Dv, C, Q, interleaved):
  """The down-projection rows through norm, rotation and store; the queries' rotated parts; the keys' up-projection moved
  to the queries; attention over the one shared key/value head with a sink; the values' up-projection with a gate a head:
  together they must give what the plain formulas give with per-head keys and values."""
  from miniinfer_b200.kernels import ops
  from miniinfer_b200.parts import ScaledRotaryEncoding
  g = torch.Generator().manual_seed(C + R)
  T, page, eps, scale = 50, 16, 1e-5, 0.2
  hdp = -(-(C + R) // 16) * 16
  rot = {"dims": R, "base": 5000.0, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 2.0}}
  pe = ScaledRotaryEncoding("rot", R, rot["base"], 4096, scaling=rot["scaling"])
  pe.prepare(DEV, 128)
  r = lambda *s: torch.randn(s, generator=g)
  down = r(T, Q + C + R + H).to(DT[dtype])
  qn, kn, sink = 1 + 0.1 * r(Q), 1 + 0.1 * r(C), r(H)
  uq, uk, uv = (r(H * (D + R), Q) / math.sqrt(Q)).to(DT[dtype]), (r(H * D, C) / math.sqrt(C)).to(DT[dtype]), (r(H * Dv, C) / math.sqrt(C)).to(DT[dtype])
  pos = torch.arange(T)
  # plain
  layout = "interleaved" if interleaved else "half"
  df = down.float()
  cq = plain.norm_plain(df[:, :Q], qn, eps)
  q = (cq.to(DT[dtype]).float() @ uq.float().T).to(DT[dtype]).float().view(T, H, D + R)
  c = plain.norm_plain(df[:, Q:Q + C], kn, eps).to(DT[dtype]).float()
  k_rot = plain.rotate(df[:, None, Q + C:Q + C + R], pos, rot, layout)[:, 0]
  q_rot = plain.rotate(q[..., D:], pos, rot, layout)
  k_plain, v = (c @ uk.float().T).view(T, H, D), (c @ uv.float().T).view(T, H, Dv)
  s = (torch.einsum("ihd,jhd->hij", q[..., :D], k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * scale
  s = s.masked_fill(~plain.visible(T, None), float("-inf"))
  o = torch.einsum("hij,jhd->ihd", plain.softmax_with_sink(s, sink), v) * torch.sigmoid(df[:, Q + C + R:])[:, :, None]
  # the engine's pieces, the sequence in two steps (the second reads the first one's cache)
  kv = torch.zeros((8, 2, 1, page, hdp), dtype=DT[dtype], device=DEV)
  bt = torch.zeros((4, 8), dtype=torch.int32, device=DEV)
  bt[2, :4] = torch.tensor([5, 2, 7, 3], dtype=torch.int32)
  got = torch.zeros((T, H * Dv), dtype=DT[dtype], device=DEV)
  dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
  for a, b in ((0, 33), (33, T - 1), (T - 1, T)):
    n = b - a
    rows = down[a:b].to(DEV)
    positions = dev(list(range(a, b)))
    slots = dev([int(bt[2, j // page]) * page + j % page for j in range(a, b)])
    cq_d = torch.zeros((n, Q), dtype=DT[dtype], device=DEV)
    ops.latent_down(rows, 0, Q, Q, C, R, qn.to(DEV), kn.to(DEV), eps, cq_d, pe.rotary_table(), positions, interleaved, slots, kv)
    qd = torch.zeros((n, H * (D + R)), dtype=DT[dtype], device=DEV)
    ops.linear(qd, cq_d, uq.to(DEV))
    qh = torch.full((n, H * hdp), 7.0, dtype=DT[dtype], device=DEV)
    ops.latent_query(qd, qh, H, D, R, C, pe.rotary_table(), positions, interleaved)
    ops.linear_batched(qh.view(n, H, hdp)[:, :, :C], qd.view(n, H, D + R)[:, :, :D], uk.to(DEV).view(H, D, C).transpose(1, 2).contiguous())
    attn = torch.zeros((n, H * C), dtype=DT[dtype], device=DEV)
    ops.attention(attn, qh, kv, bt, _batch(b, n), H, 1, hdp, scale, None, sink=sink.to(DEV), out_hd=C)
    ops.linear_batched(got[a:b].view(n, H, Dv), attn.view(n, H, C), uv.to(DEV).view(H, Dv, C), row_gate=rows[:, Q + C + R:])
  assert float((got.float().cpu() - o.reshape(T, -1)).abs().max()) <= (1e-4 if dtype == "float32" else 6e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rot_dims,interleaved", [(16, True), (24, True), (8, False), (24, False)])
def test_head_norm_rotation_and_values_that_are_the_keys(dtype, rot_dims, interleaved):
  from miniinfer_b200.kernels import ops
  from miniinfer_b200.parts import ScaledRotaryEncoding
  g = torch.Generator().manual_seed(rot_dims)
  T, H, G, D, page, eps = 11, 4, 2, 24, 8, 1e-5
  hdp = 32
  pe = ScaledRotaryEncoding("rot", rot_dims, 300.0, 4096)
  pe.prepare(DEV, 64)
  proj = torch.randn((T, (H + G) * D + 5), generator=g).to(DT[dtype])
  qw, kw = 1 + 0.1 * torch.randn((D,), generator=g), 1 + 0.1 * torch.randn((D,), generator=g)
  pos = torch.arange(20, 20 + T)
  rot = {"dims": rot_dims, "base": 300.0}
  layout = "interleaved" if interleaved else "half"
  q = plain.rotate(plain.norm_plain(proj[:, :H * D].float().view(T, H, D), qw, eps), pos, rot, layout)
  k_raw = proj[:, H * D:(H + G) * D].float().view(T, G, D)
  k = plain.rotate(plain.norm_plain(k_raw, kw, eps), pos, rot, layout)
  kv = torch.zeros((6, 2, G, page, hdp), dtype=DT[dtype], device=DEV)
  slots = torch.tensor([3 * page + 5 - j if j < 6 else 4 * page + j for j in range(T)], dtype=torch.int32, device=DEV)
  q_out = torch.full((T, H * hdp), 3.0, dtype=DT[dtype], device=DEV)
  ops.qkv_norm_mix_store(proj.to(DEV), 0, H * D, H * D, q_out, H, G, D, D, eps, True, qw.to(DEV), kw.to(DEV), None, None, 0, slots, kv,
                         rope=pe.rotary_table(), positions=pos.to(torch.int32).to(DEV), interleaved=interleaved)
  qo = q_out.float().cpu().view(T, H, hdp)
  assert float((qo[..., :D] - q).abs().max()) <= tol(dtype) and float(qo[..., D:].abs().max()) == 0
  for j in range(T):
    s = int(slots[j])
    assert float((kv[s // page, 0, :, s % page, :D].float().cpu() - k[j]).abs().max()) <= tol(dtype)
    assert float((kv[s // page, 1, :, s % page, :D].float().cpu() - k_raw[j]).abs().max()) <= tol(dtype)      # the value: the key as projected


def test_stretched_rotary_frequencies():
  from miniinfer_b200.parts import ScaledRotaryEncoding
  for rot in ({"dims": 16, "base": 5000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}},
              {"dims": 32, "base": 20000.0, "scaling": {"factor": 3.0, "original": 512, "fast": 32.0, "slow": 1.0}},
              {"dims": 8, "base": 100.0}):
    pe = ScaledRotaryEncoding("rot", rot["dims"], rot["base"], 4096, scaling=rot.get("scaling"))
    table = pe.build_table(300)
    f, m = plain.rotary_frequencies(rot)
    a = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert float((table[:, :rot["dims"] // 2].double() - a.cos() * m).abs().max()) < 1e-6
    assert float((table[:, rot["dims"] // 2:].double() - a.sin() * m).abs().max()) < 1e-6
