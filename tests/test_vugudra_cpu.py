"""Vugudra on the host side, without a GPU: its configuration (every key read, faults named, sizes that only a tensor's
shape gives), its weights, the model as data (run list of a loop, cache needs of a mixer made of two), the cache
manager's handling of kept first tokens and of several needs a layer, and the whole path through cache manager, step
function and replay on the CPU with the kernels replaced by their PyTorch statements."""
import copy
import io
import json

import numpy as np
import pytest
import torch

import plain_vugudra as plain
import replay_cases as rc


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
  return plain.make_model(plain.CONFIGS["A"], str(tmp_path_factory.mktemp("vugudra_A")), seed=3)


def test_configuration_is_read_key_by_key(model_a):
  from miniinfer_b200.config import VugudraConfig, load_model_config
  cfg = load_model_config(model_a)
  assert isinstance(cfg, VugudraConfig)
  assert (cfg.vocab_size, cfg.width, cfg.norm_eps) == (300, 64, 1e-5)
  assert cfg.layer_order() == [0, 1, 2, 1, 2, 3]
  scan, lat, (left, right) = cfg.mixer_of(0), cfg.mixer_of(1), cfg.mixer_of(2)
  assert (scan.inner, scan.state, scan.dt_rank, scan.conv) == (96, 8, 6, 4)
  assert (lat.heads, lat.dim, lat.rot_dim, lat.vdim, lat.kv_rank, lat.q_rank) == (2, 16, 8, 24, 32, 40)
  assert lat.rot.base == 5000.0 and lat.rot.scaling == {"factor": 4.0, "original": 64.0, "fast": 16.0, "slow": 2.0} and lat.scale == 24 ** -0.5
  assert (left.heads, left.kv_heads, left.dim, left.window, left.keep_first, left.rot.dims) == (4, 2, 24, 20, 3, 16)
  assert (right.heads, right.kv_heads, right.dim, right.vdim, right.conv) == (2, 1, 16, 24, 3)
  assert [cfg.ff_of(i) for i in range(4)] == [96, 80, 72, None]
  # the two low ranks of the delta rule stand in no key: they are read from the shapes of the file's tensors
  assert cfg.low_ranks == {"l2.decay": 8, "l2.gate": 8}
  d = cfg.to_dict()
  d.pop("low_ranks")
  assert d == plain.CONFIGS["A"]


@pytest.mark.parametrize("change,key", [
  (lambda c: c["layers"][1].__setitem__("type", "attention"), "layers[1].type"),
  (lambda c: c["layers"][2]["mixer"]["left"].__setitem__("kv_heads", 3), "left.heads"),
  (lambda c: c["layers"][2]["mixer"]["left"]["mask"].__setitem__("size", 0), "mask.size"),
  (lambda c: c["layers"][2]["mixer"]["left"]["mask"].__setitem__("keep_first", -1), "keep_first"),
  (lambda c: c["layers"][2]["mixer"]["left"].__setitem__("vdim", 8), "left.vdim"),
  (lambda c: c["layers"][2]["mixer"]["left"]["rot"].__setitem__("dims", 30), "rot.dims"),
  (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 6), "rot.dims"),
  (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].__setitem__("factor", 0), "scaling.factor"),
  (lambda c: c["layers"][0]["mixer"].__setitem__("state", 0), "mixer.state"),
  (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "mlp.kind"),
  (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
  (lambda c: c["norm"].__setitem__("eps", 0), "norm.eps"),
  (lambda c: c.__setitem__("width", 0), "width"),
])
def test_faulty_configurations_are_refused_with_the_key(change, key):
  from miniinfer_b200.config import ConfigError, VugudraConfig
  c = copy.deepcopy(plain.CONFIGS["A"])
  change(c)
  with pytest.raises(ConfigError, match=key.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
    VugudraConfig.from_dict(c)


def test_the_model_as_data(model_a):
  from miniinfer_b200.cache.specs import CompositeSpec, FixedStateSpec, PagedKVSpec
  from miniinfer_b200.config import build_model_spec, load_model_config
  spec = build_model_spec(load_model_config(model_a))
  assert [type(b.mixer_part()).__name__ for b in spec.blocks] == ["SelectiveScanMixer", "LatentAttentionMixer", "SideBySideMixer", "SelectiveScanMixer"]
  assert [r.block for r in spec.run_list] == [0, 1, 2, 1, 2, 3] and all(r.cache_of is None for r in spec.run_list)
  assert spec.blocks[3].ffn is None and spec.blocks[3].ffn_norm is None and spec.blocks[0].ffn_norm is not None
  needs = spec.cache_layer_specs()
  assert needs[0] == FixedStateSpec((3 * 96 + 96 * 8,), "float32")
  assert needs[1] == needs[3] == PagedKVSpec(1, 48, None)                       # latent 32 + rotated 8, rounded up to 48
  side = CompositeSpec((PagedKVSpec(2, 32, 20, 3), FixedStateSpec((2 * (2 * 16 + 2 * 24) + 2 * 16 * 24,), "float32")))
  assert needs[2] == needs[4] == side
  assert needs[5] == FixedStateSpec((1 * 64 + 64 * 12,), "float32")


def test_weights_are_asked_for_by_name(model_a, tmp_path):
  from safetensors.torch import load_file, save_file
  from miniinfer_b200.config import build_model_spec, load_model_config
  from miniinfer_b200.weights import load_weights
  from miniinfer_b200.weights.loader import WeightLoadError
  spec = build_model_spec(load_model_config(model_a))
  load_weights(spec, model_a, torch.bfloat16, "cpu")
  W = plain.read_weights(model_a)
  norm = spec.blocks[0].norm
  assert norm.weight.dtype == torch.float32 and torch.equal(norm.weight, 1.0 + W["l0.norm1"])       # stored around zero
  lat = spec.blocks[1].mixer_part()
  assert lat.down.shape == (40 + 32 + 8 + 2, 64) and torch.equal(lat.down[lat.g_off:].float(), W["l1.mix.g"])
  assert torch.equal(lat.uk_t[1].float(), W["l1.mix.uk"][16:32].T)
  side = spec.blocks[2].mixer_part()
  left, right = side.left, side.right
  assert left.qkvg.shape == ((4 + 2) * 24, 64) and left.v_off == left.k_off and torch.equal(left.q_norm, W["l2.mix.left.q.norm"])
  assert torch.equal(right.proj[right.conv_off + right.k_off:right.conv_off + right.v_off].float(), W["l2.mix.right.k"])
  assert torch.equal(right.proj[:8].float(), W["l2.mix.right.a1"]) and torch.equal(right.conv[right.v_off:], W["l2.mix.right.v.conv"])
  assert right.A_log.dtype == torch.float32 and torch.equal(side.right_out, W["l2.mix.right.out"])
  t = load_file(f"{model_a}/model.safetensors")
  del t["l1.mix.sink"]
  t["l3.norm2"] = torch.zeros(64)
  t["l0.mix.A_log"] = torch.zeros((96, 7))
  d = tmp_path / "broken"
  d.mkdir()
  save_file(t, str(d / "model.safetensors"))
  (d / "config.json").write_text(json.dumps(plain.CONFIGS["A"]))
  with pytest.raises(WeightLoadError) as e:
    load_weights(build_model_spec(load_model_config(str(d))), str(d), torch.bfloat16, "cpu")
  assert e.value.missing == ["l1.mix.sink"] and e.value.unexpected == ["l3.norm2"] and "l0.mix.A_log" in e.value.wrong_shape[0]


def test_random_weights_mode_writes_a_model_of_the_design(tmp_path):
  from miniinfer_b200.weights import write_random_model
  c = copy.deepcopy(plain.CONFIGS["B"])
  c["low_ranks"] = {"l0.decay": 8, "l0.gate": 16, "l3.decay": 8, "l3.gate": 8}
  d = write_random_model(c, str(tmp_path / "m"), seed=4)
  W, cfg = plain.read_weights(d), plain.read_config(d)
  assert W["l0.mix.right.a1"].shape == (8, 96) and W["l0.mix.right.g2"].shape == (4 * 16, 16) and W["l2.mix.conv"].shape == (128, 3)
  assert torch.isfinite(plain.forward(W, cfg, [1, 2, 3])).all()


def test_kept_first_pages_and_several_needs_a_layer():
  from miniinfer_b200.cache.manager import KVCacheManager
  from miniinfer_b200.cache.specs import CompositeSpec, FixedStateSpec, PagedKVSpec
  needs = [CompositeSpec((PagedKVSpec(2, 16, 10, 6), FixedStateSpec((7,), "float32"))), PagedKVSpec(1, 32, None), FixedStateSpec((7,), "float32")]
  m = KVCacheManager(needs, 4, 40, 3, 160, torch.float32, "cpu")
  assert len(m.paged_groups) == 2 and len(m.state_groups) == 1 and m.state_groups[0].num_layers == 2
  lc = m.layer_cache(0)
  assert lc.kind == "composite" and [c.kind for c in lc.members] == ["paged", "state"] and m.layer_cache(2).kind == "state"
  m.admit("a")
  for _ in range(10):
    m.append("a", 5)
    m.commit("a", 5)
  g = next(g for g in m.paged_groups if g.spec.window)
  held = m._requests["a"].pages[g.index]
  # 50 tokens: the two pages of the six kept tokens stay, the pages wholly behind position 50 - 10 + 1 went back
  assert [i for i, p in enumerate(held) if p] == [0, 1] + list(range(41 // 4, 13))
  m.check_invariants()
  m.state_groups[0].state[:, m.slot_of("a")] = 5.0
  m.release_request("a")
  m.admit("b")
  assert float(m.state_groups[0].state[:, m.slot_of("b")].abs().max()) == 0       # a slot that is used again starts at zero
  assert m.free_pages() == [g.num_pages for g in m.paged_groups]


@pytest.mark.parametrize("tag,page", [("A", 16), ("B", 8)])
def test_every_cut_gives_the_plain_logits_on_the_host_path(cpu_kernels, tmp_path, tag, page):
  from miniinfer_b200.engine.replay import TraceRunner
  d = plain.make_model(plain.CONFIGS[tag], str(tmp_path / tag), seed=8)
  lengths = (5, 17, 33, 100, 64, 41, 2)
  reqs = rc.make_requests(plain.CONFIGS[tag]["vocab"], lengths, seed=5)
  W, cfg = plain.read_weights(d), plain.read_config(d)
  ref = {rid: plain.forward(W, cfg, ids) for rid, ids in reqs.items()}
  budget = 2 * rc.round_up(max(lengths), page)
  for name, trace in (("whole", rc.whole(reqs)), ("tail", rc.tail_one_by_one(reqs)), ("portions", rc.portions(reqs)),
                      ("mixed", rc.mixed(reqs, budget, seed=1, granule=page)),
                      ("preempted", rc.mixed(reqs, budget, seed=2, granule=page, preempt=True))):
    runner = TraceRunner(d, "float32", budget, device="cpu", page_size=page, max_requests=4)
    got = rc.run_in_process(runner, trace)
    rc.compare(got, ref, 3e-4, f"vugudra {tag}/{name}")
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]


def test_trace_program_picks_the_model_by_its_configuration(cpu_kernels, model_a, tmp_path):
  from miniinfer_b200.engine import replay
  reqs = rc.make_requests(300, (20, 9), seed=2)
  trace = rc.mixed(reqs, 128, seed=3)
  out = io.StringIO()
  code = replay.main(["--model", model_a, "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128",
                      "--device", "cpu"], stdin=io.StringIO("\n".join(json.dumps(r) for r in trace) + "\n"), stdout=out)
  assert code == 0 and out.getvalue().split("\n")[:-1] == [f"done {r['step']}" for r in trace]
  outputs = {r["step"]: np.fromfile(tmp_path / "o" / f"{r['step']}.f32", dtype="<f4").reshape(-1, 300)
             for r in trace if sum(len(e["want"]) for e in r["entries"])}
  W, cfg = plain.read_weights(model_a), plain.read_config(model_a)
  rc.compare(rc.collect(trace, outputs), {rid: plain.forward(W, cfg, ids) for rid, ids in reqs.items()}, 3e-4, "trace program")
