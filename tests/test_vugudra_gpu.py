"""The Vugudra design in the engine against its plain implementation (tests/plain_vugudra.py): every way of cutting
requests into steps, in float32 and bfloat16, on configurations that differ in every size and in the order of their
layers; long decoding past windows, kept first tokens and page borders; pages and state slots used again; greedy
generation through the entry point and its scheduler."""
import numpy as np
import pytest
import torch

import plain_vugudra as plain
import replay_cases as rc
from gpu_helpers import DEV

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (5, 17, 33, 100, 64, 128, 41, 65, 1, 2), "B": (1, 9, 40, 71, 130, 65, 200, 2), "C": (130, 70, 300, 64, 200, 65, 257)}
PAGES = {"A": 16, "B": 16, "C": 64}
# bfloat16: logits of these models have a root mean square near 1, and rounding every product to bfloat16 moves a row by
# 0.02 on average and a few rows in a hundred by 0.1 to 0.3 (measured by rounding the plain implementation's products):
# the recurrent states carry the rounding of every earlier token.  A wrong window edge, a lost state or a sink left out
# moves most rows by tenths, and shows in the float32 runs, which take the same path through the engine and allow nothing.
BF16_MEAN, BF16_BOUND, BF16_CAP = 0.05, 0.15, 0.45      # the mean over all rows; what one row in twenty may pass; what none may


@pytest.fixture(scope="module")
def vugudra_dirs(tmp_path_factory):
  made = {}

  def get(tag):
    if tag not in made:
      made[tag] = plain.make_model(plain.CONFIGS[tag], str(tmp_path_factory.mktemp(f"vugudra_{tag}")), seed=31 + len(made))
    return made[tag]

  return get


_refs = {}


def reference(model_dir, reqs):
  key = (model_dir, tuple(sorted(reqs)), tuple(len(v) for v in reqs.values()))
  if key not in _refs:
    W, cfg = plain.read_weights(model_dir), plain.read_config(model_dir)
    with torch.no_grad():
      _refs[key] = {rid: plain.forward(W, cfg, ids) for rid, ids in reqs.items()}
  return _refs[key]


def runner_for(model_dir, dtype, max_tokens, page, max_requests=4):
  from miniinfer_b200.engine.replay import TraceRunner
  return TraceRunner(model_dir, dtype, max_tokens, device=DEV, page_size=page, max_requests=max_requests)


def compare(got, ref, dtype, tag, what):
  if dtype == "float32":
    rc.compare(got, ref, 3e-4, what, check_argmax_margin=2e-3)
    return
  assert got, "nothing was compared"
  errs = []
  for key, row in sorted(got.items()):
    assert np.isfinite(row).all(), f"{what}: request {key[0]} position {key[1]}: logits are not finite"
    d = row - ref[key[0]][key[1]].numpy()
    errs.append(float(np.sqrt(((d - d.mean()) ** 2).mean())))       # root mean square of the centred difference
    assert errs[-1] <= BF16_CAP, f"{what}: request {key[0]} position {key[1]}: the row differs by {errs[-1]:.3f}"
  errs = np.array(errs)
  assert errs.mean() <= BF16_MEAN, f"{what}: rows differ by {errs.mean():.4f} on average"
  assert (errs > BF16_BOUND).sum() <= max(1, 0.05 * len(errs)), f"{what}: {(errs > BF16_BOUND).sum()} of {len(errs)} rows differ by more than {BF16_BOUND}"
  rc.log_worst(what, float(errs.max()), ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed", "preempted"])
def test_every_cut_gives_the_plain_logits(vugudra_dirs, dtype, tag, cut):
  d = vugudra_dirs(tag)
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
  compare(got, ref, dtype, tag, f"vugudra {tag}/{dtype}/{cut}")
  runner.cache.check_invariants()
  assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]
  runner.runner.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_windows_kept_tokens_and_pages(vugudra_dirs, dtype):
  """Twelve tokens as a prompt, then 250 tokens one by one: the windows of A (20, keeping 3) and B (33 keeping 17, 7
  keeping 1) pass over decoded tokens, page borders (pages of 8) are crossed dozens of times, pages behind the windows go
  back - those of the kept first tokens stay - and are taken again by a second request that decodes beside the first; the
  recurrent states run over 260 steps."""
  for tag in ("A", "B"):
    d = vugudra_dirs(tag)
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
    compare(got, ref, dtype, tag, f"vugudra long decode {tag}/{dtype}")
    runner.cache.check_invariants()


def test_pages_of_kept_first_tokens_stay_and_the_others_go_back(vugudra_dirs):
  """C's window of 100 keeps 70 first tokens: with pages of 16 a request of 300 tokens holds, in the windowed group, the
  five pages of its first tokens and the pages of its window, and nothing between."""
  d = vugudra_dirs("C")
  reqs = rc.make_requests(plain.CONFIGS["C"]["vocab"], (300,), seed=4)
  runner = runner_for(d, "float32", 320, 16)
  ids = reqs["r0"]
  for pos in range(0, 300, 50):
    runner.run_step({"step": pos, "entries": [{"id": "r0", "tokens": ids[pos:pos + 50], "want": []}], "end": []})
  windowed = [g for g in runner.cache.paged_groups if g.spec.window is not None]
  assert len(windowed) == 1 and windowed[0].spec.keep_first == 70
  held = runner.cache._requests["r0"].pages[windowed[0].index]
  live = [i for i, p in enumerate(held) if p != 0]
  assert live[:5] == [0, 1, 2, 3, 4] and live[5] == (300 - 100 + 1) // 16 and 5 < len(live) <= 13
  runner.cache.check_invariants()


@pytest.mark.skipif(DEV == "cpu", reason="a property of the CUDA kernels' order of sums, not of the CPU statements")
def test_float32_logits_do_not_depend_on_the_cut(vugudra_dirs):
  """In float32 a position's logits come out the same to the last bit however the request was cut and whatever else was
  in the batch: every sum of the 32-bit path runs in an order that depends on the position alone."""
  d = vugudra_dirs("A")
  reqs = rc.make_requests(plain.CONFIGS["A"]["vocab"], (70, 33, 90, 41), seed=3)
  whole = rc.run_in_process(runner_for(d, "float32", 128, 16), rc.whole(reqs))
  for name, trace in (("portions", rc.portions(reqs)), ("mixed", rc.mixed(reqs, 224, seed=4, granule=16))):
    got = rc.run_in_process(runner_for(d, "float32", 224, 16), trace)
    for key, row in got.items():
      assert np.array_equal(row, whole[key[:2]]), f"{name}: request {key[0]} position {key[1]} differs in its bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(vugudra_dirs, dtype):
  """``LLMEngine.generate``: the scheduler admits, cuts the prompts into portions under a small token budget, decodes from
  CUDA graphs; more requests than slots, so state slots and pages are used again."""
  from miniinfer_b200 import LLMEngine, SamplingParams
  d = vugudra_dirs("A")
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
      # every token is the plain implementation's choice for the text so far, or within the bound of it
      seq, odd = list(prompt), 0
      for t in ids:
        row = plain.forward(W, cfg, seq)[-1]
        odd += float(row.max() - row[t]) > 2 * BF16_BOUND
        seq.append(t)
      assert odd <= 0.05 * n_new, f"{odd} of {n_new} bfloat16 tokens are not what the plain logits allow"
  if DEV != "cpu":
    eng.runner.check_status()
    assert eng.runner.num_graphs() > 0


@pytest.mark.skipif(DEV == "cpu", reason="the command line runs on a CUDA device")
def test_command_line_and_trace_program(vugudra_dirs, tmp_path):
  """`main.py` generates from a Vugudra folder, and `bin/trace_run` - a process of its own that picks the model by its
  configuration - replays a mixed trace in both dtypes."""
  import json
  import os
  import subprocess
  import sys
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  d = vugudra_dirs("B")
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
    compare(rc.collect(trace, outputs), ref, dtype, "B", f"trace program {dtype}")
