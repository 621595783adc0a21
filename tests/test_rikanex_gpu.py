"""The Rikanex design in the engine against its plain implementation (tests/plain_rikanex.py): every way of cutting
requests into steps, in float32 and bfloat16, on configurations that differ in every size; long decoding past windows
and page borders; pages and slots used again; greedy generation through the entry point and its scheduler."""
import numpy as np
import pytest
import torch

import plain_rikanex as plain
import replay_cases as rc
from gpu_helpers import DEV

pytestmark = pytest.mark.gpu

LENGTHS = {"P": (5, 17, 33, 100, 64, 128, 41, 65, 1, 2), "Q": (1, 9, 40, 71, 130, 65, 200, 2), "S": (130, 70, 300, 64, 200, 65, 257)}
PAGES = {"P": 16, "Q": 8, "S": 64}
# bfloat16: logits of these models have a root mean square near 1; a wrong window edge, a lost sink or a value that was
# not mixed moves them by tenths.  The bounds are about three times what rounding gave on a B200.
BF16_BOUND = {"P": 0.06, "Q": 0.06, "S": 0.08}


@pytest.fixture(scope="module")
def rikanex_dirs(tmp_path_factory):
  made = {}

  def get(tag):
    if tag not in made:
      made[tag] = plain.make_model(plain.CONFIGS[tag], str(tmp_path_factory.mktemp(f"rikanex_{tag}")), seed=11 + len(made))
    return made[tag]

  return get


_refs = {}


def reference(model_dir, reqs):
  key = (model_dir, tuple(sorted(reqs)))
  if key not in _refs:
    W, cfg = plain.read_weights(model_dir), plain.read_config(model_dir)
    with torch.no_grad():
      _refs[key] = {rid: plain.forward(W, cfg, ids) for rid, ids in reqs.items()}
  return _refs[key]


def runner_for(model_dir, dtype, max_tokens, page, max_requests=4):
  from miniinfer_b200.engine.replay import TraceRunner
  return TraceRunner(model_dir, dtype, max_tokens, device=DEV, page_size=page, max_requests=max_requests)


def bound(dtype, tag):
  return 2e-4 if dtype == "float32" else BF16_BOUND[tag]


def compare(got, ref, dtype, tag, what):
  """float32: every row within the bound, equal arg-max where the margin is clear.  bfloat16: a router's close call
  (with three to six experts, one token in thirty has one) may fall the other way after rounding; that moves the
  token's row, and through the cache the rows of the tokens that see it, by more than rounding does.  So up to 15 % of
  the rows may pass the bound.  A wrong window edge, sink, mix or page shows in most rows and in the float32 runs,
  which take the same path through the engine; the bfloat16 kernels' edges are tested on their own, without a router."""
  b = bound(dtype, tag)
  if dtype == "float32":
    rc.compare(got, ref, b, what, check_argmax_margin=1e-3)
    return
  assert got, "nothing was compared"
  over = []
  for key, row in sorted(got.items()):
    assert np.isfinite(row).all(), f"{what}: request {key[0]} position {key[1]}: logits are not finite"
    d = float(np.abs(row - ref[key[0]][key[1]].numpy()).max())
    if d > b:
      over.append((key, round(d, 4)))
  assert len(over) <= max(1, 0.15 * len(got)), f"{what}: {len(over)} of {len(got)} rows differ by more than {b}: {over[:8]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["P", "Q", "S"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed", "preempted"])
def test_every_cut_gives_the_plain_logits(rikanex_dirs, dtype, tag, cut):
  d = rikanex_dirs(tag)
  page = PAGES[tag]
  reqs = rc.make_requests(plain.CONFIGS[tag]["vocab"], LENGTHS[tag], seed=5)
  ref = reference(d, reqs)
  longest = rc.round_up(max(LENGTHS[tag]), page)
  if cut in ("mixed", "preempted"):
    budget = longest + 2 * rc.round_up(70, page)      # requests wait for pages that others give back
    trace = rc.mixed(reqs, budget, seed=1, granule=page, preempt=cut == "preempted")
    assert max(len(r["entries"]) for r in trace) >= 2
  else:
    budget = longest
    trace = {"whole": rc.whole, "tail": rc.tail_one_by_one, "portions": rc.portions}[cut](reqs)
  runner = runner_for(d, dtype, budget, page)
  got = rc.run_in_process(runner, trace)
  compare(got, ref, dtype, tag, f"rikanex {tag}/{dtype}/{cut}")
  runner.cache.check_invariants()
  assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]
  runner.runner.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_windows_and_pages(rikanex_dirs, dtype):
  """Twelve tokens as a prompt, then 250 tokens one by one: every window of Q (7, none, 40) and of P passes over decoded
  tokens, page borders (pages of 8) are crossed dozens of times, pages behind the windows go back and are taken again
  by a second request that decodes beside the first."""
  for tag in ("Q", "P"):
    d = rikanex_dirs(tag)
    page = 8
    reqs = rc.make_requests(plain.CONFIGS[tag]["vocab"], (262, 150), seed=9)
    ref = reference(d, reqs)
    a, b = reqs["r0"], reqs["r1"]
    trace = [{"step": 0, "entries": [{"id": "r0", "tokens": a[:12], "want": list(range(12))}], "end": []}]
    pos_b = 0
    for j in range(12, len(a)):
      entries = [{"id": "r0", "tokens": [a[j]], "want": [0]}]
      if j >= 100 and pos_b < len(b):
        n = 3 if pos_b < 30 else 1           # the second request: a few portions of three, then one by one beside the first
        entries.append({"id": "r1", "tokens": b[pos_b:pos_b + n], "want": list(range(len(b[pos_b:pos_b + n])))})
        pos_b += n
      trace.append({"step": len(trace), "entries": entries, "end": []})
    trace[-1]["end"] = ["r0", "r1"]
    runner = runner_for(d, dtype, 512, page)
    got = rc.run_in_process(runner, trace)
    got = {k: v for k, v in got.items() if k[0] == "r0" or k[1] < pos_b}
    compare(got, ref, dtype, tag, f"rikanex long decode {tag}/{dtype}")
    runner.cache.check_invariants()


@pytest.mark.skipif(DEV == "cpu", reason="a property of the CUDA kernels' order of sums, not of the CPU statements")
def test_float32_logits_do_not_depend_on_the_cut(rikanex_dirs):
  """In float32 a position's logits come out the same to the last bit however the request was cut and whatever else was
  in the batch: every sum of the 32-bit path runs in an order that depends on the position alone."""
  d = rikanex_dirs("P")
  reqs = rc.make_requests(plain.CONFIGS["P"]["vocab"], (70, 33, 90, 41), seed=3)
  whole = rc.run_in_process(runner_for(d, "float32", 128, 16), rc.whole(reqs))
  for name, trace in (("portions", rc.portions(reqs)), ("mixed", rc.mixed(reqs, 224, seed=4, granule=16))):
    got = rc.run_in_process(runner_for(d, "float32", 224, 16), trace)
    for key, row in got.items():
      assert np.array_equal(row, whole[key[:2]]), f"{name}: request {key[0]} position {key[1]} differs in its bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(rikanex_dirs, dtype):
  """``LLMEngine.generate``: the scheduler admits, cuts the prompts into portions under a small token budget, decodes from
  CUDA graphs; more requests than slots, so slots and pages are used again."""
  from miniinfer_b200 import LLMEngine, SamplingParams
  d = rikanex_dirs("P")
  W, cfg = plain.read_weights(d), plain.read_config(d)
  g = torch.Generator().manual_seed(21)
  prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (3, 45, 18, 70, 9, 31)]
  n_new = 40
  eng = LLMEngine(d, dtype=dtype, device=DEV, page_size=16, num_pages=24, max_num_seqs=3, max_model_len=128,
                  max_num_batched_tokens=32)
  outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
  for prompt, out in zip(prompts, outs):
    ids = out["token_ids"]
    assert len(ids) == n_new
    if dtype == "float32":
      assert ids == plain.generate(W, cfg, prompt, n_new)
    else:
      # every token is the plain implementation's choice for the text so far, or within twice the bound of it
      # (but for a router's close call now and then)
      seq, odd = list(prompt), 0
      for t in ids:
        row = plain.forward(W, cfg, seq)[-1]
        odd += float(row.max() - row[t]) > 2 * BF16_BOUND["P"]
        seq.append(t)
      assert odd <= 0.15 * n_new, f"{odd} of {n_new} bfloat16 tokens are not what the plain logits allow"
  if DEV != "cpu":
    eng.runner.check_status()
    assert eng.runner.num_graphs() > 0


@pytest.mark.skipif(DEV == "cpu", reason="the command line runs on a CUDA device")
def test_command_line_and_trace_program(rikanex_dirs, tmp_path):
  """`main.py` generates from a Rikanex folder, and `bin/trace_run` - a process of its own that picks the model by its
  configuration - replays a mixed trace in both dtypes."""
  import json
  import os
  import subprocess
  import sys
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  d = rikanex_dirs("Q")
  W, cfg = plain.read_weights(d), plain.read_config(d)
  proc = subprocess.run([sys.executable, os.path.join(root, "main.py"), "--model", d, "--prompt-ids", "5,17,3,200", "--max-tokens", "6",
                         "--temperature", "0", "--dtype", "float32", "--max-model-len", "64", "--page-size", "16"],
                        capture_output=True, text=True, timeout=900)
  assert proc.returncode == 0, proc.stderr[-3000:]
  assert str(plain.generate(W, cfg, [5, 17, 3, 200], 6)) in proc.stdout
  reqs = rc.make_requests(cfg["vocab"], (70, 9, 130), seed=2)
  ref = reference(d, reqs)
  trace = rc.mixed(reqs, 256, seed=3)
  for dtype in ("float32", "bfloat16"):
    out = tmp_path / dtype
    proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out), "--max-tokens", "256"],
                          input="\n".join(json.dumps(r) for r in trace) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {r['step']}" for r in trace]
    outputs = {r["step"]: np.fromfile(out / f"{r['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
               for r in trace if sum(len(e["want"]) for e in r["entries"])}
    compare(rc.collect(trace, outputs), ref, dtype, "Q", f"trace program {dtype}")
