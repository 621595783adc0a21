"""Rikanex on the host side, without a GPU: its configuration (every key read, faults named), its weights (every tensor
asked for by name, faults collected), the model as data, and the whole path through cache manager, step function and
replay on the CPU with the kernels replaced by their PyTorch statements."""
import copy
import io
import json

import numpy as np
import pytest
import torch

import plain_rikanex as plain
import replay_cases as rc


@pytest.fixture(scope="module")
def model_p(tmp_path_factory):
  return plain.make_model(plain.CONFIGS["P"], str(tmp_path_factory.mktemp("rikanex_P")), seed=3)


def test_configuration_is_read_key_by_key(model_p):
  from miniinfer_b200.config import RikanexConfig, load_model_config
  cfg = load_model_config(model_p)
  assert isinstance(cfg, RikanexConfig)
  assert (cfg.vocab_size, cfg.width, cfg.embedding_scale, cfg.norm_eps) == (300, 64, 8.0, 1e-5)
  m = [cfg.mixer_of(i) for i in range(4)]
  assert [(x.heads, x.kv_heads, x.dim, x.vdim, x.window, x.v_mix) for x in m] == [
    (4, 2, 16, 32, 20, False), (4, 2, 16, 32, 33, True), (2, 2, 32, 32, 9, True), (4, 2, 16, 32, 20, True)]
  assert m[3].scale == 0.3 and m[0].scale == 16 ** -0.5
  mlp = [cfg.mlp_of(i) for i in range(4)]
  assert mlp[2] is None and mlp[0].kind == "dense" and (mlp[1].experts, mlp[1].top, mlp[1].ff) == (5, 2, 40)
  assert cfg.to_dict() == plain.CONFIGS["P"]            # what the random-weights mode writes back is the design's own file


@pytest.mark.parametrize("change,key", [
  (lambda c: c["layers"][1].__setitem__("type", "recurrent"), "layers[1].type"),
  (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
  (lambda c: c["layers"][0]["mixer"].__setitem__("mask", {"size": 0}), "mask.size"),
  (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "router.top"),
  (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "mlp.kind"),
  (lambda c: c["norm"].__setitem__("eps", 0), "norm.eps"),
  (lambda c: c.__setitem__("width", 0), "width"),
])
def test_faulty_configurations_are_refused_with_the_key(change, key):
  from miniinfer_b200.config import ConfigError, RikanexConfig
  c = copy.deepcopy(plain.CONFIGS["P"])
  change(c)
  with pytest.raises(ConfigError, match=key.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
    RikanexConfig.from_dict(c)


def test_values_can_only_be_mixed_with_values_of_their_shape():
  from miniinfer_b200.config import ConfigError, RikanexConfig, build_model_spec
  c = copy.deepcopy(plain.CONFIGS["P"])
  c["layers"][3]["mixer"]["vdim"] = 16
  with pytest.raises(ConfigError, match=r"layers\[3\]"):
    build_model_spec(RikanexConfig.from_dict(c))


def test_the_model_as_data(model_p):
  from miniinfer_b200.cache.specs import PagedKVSpec
  from miniinfer_b200.config import build_model_spec, load_model_config
  spec = build_model_spec(load_model_config(model_p))
  mixers = [b.mixer_part() for b in spec.blocks]
  assert [m.value_mix for m in mixers] == [None, "source", "mixed", "mixed"]
  assert spec.blocks[2].ffn is None
  # key and value sizes 16 and 32 share cache rows of 32; layers with equal needs share a pool
  assert spec.cache_layer_specs() == [PagedKVSpec(2, 32, 20), PagedKVSpec(2, 32, 33), PagedKVSpec(2, 32, 9), PagedKVSpec(2, 32, 20)]


def test_weights_are_asked_for_by_name(model_p, tmp_path):
  from safetensors.torch import load_file, save_file
  from miniinfer_b200.config import build_model_spec, load_model_config
  from miniinfer_b200.weights import load_weights
  from miniinfer_b200.weights.loader import WeightLoadError
  spec = build_model_spec(load_model_config(model_p))
  load_weights(spec, model_p, torch.bfloat16, "cpu")
  W = plain.read_weights(model_p)
  mixer = spec.blocks[1].mixer_part()
  assert mixer.qkvg.shape == (4 * 16 + 2 * 16 + 2 * 32 + 4 * 32, 64) and mixer.qkvg.dtype == torch.bfloat16
  assert torch.equal(mixer.qkvg[mixer.g_off:].float(), W["l1.mix.g"]) and torch.equal(mixer.qkvg[mixer.k_off:mixer.v_off].float(), W["l1.mix.k"])
  assert mixer.mix.shape == () and mixer.sink.dtype == torch.float32
  ffn = spec.blocks[1].ffn
  assert torch.equal(ffn.router.float(), W["l1.mlp.router"]) and ffn.correction.dtype == torch.float32
  assert torch.equal(ffn.gate_up.view(5, 80, 64)[3, 40:].float(), W["l1.mlp.e3.up"]) and torch.equal(ffn.down.view(5, 64, 40)[4].float(), W["l1.mlp.e4.down"])
  # a file with a tensor missing, one too many and one of a wrong shape: one error names all three
  t = load_file(f"{model_p}/model.safetensors")
  del t["l3.mix.sink"]
  t["l2.mlp.gate"] = torch.zeros((4, 4))
  t["l1.mlp.correction"] = torch.zeros(7)
  d = tmp_path / "broken"
  d.mkdir()
  save_file(t, str(d / "model.safetensors"))
  (d / "config.json").write_text(json.dumps(plain.CONFIGS["P"]))
  with pytest.raises(WeightLoadError) as e:
    load_weights(build_model_spec(load_model_config(str(d))), str(d), torch.bfloat16, "cpu")
  assert e.value.missing == ["l3.mix.sink"] and e.value.unexpected == ["l2.mlp.gate"] and "l1.mlp.correction" in e.value.wrong_shape[0]


def test_random_weights_mode_writes_a_model_of_the_design(tmp_path):
  from miniinfer_b200.weights import write_random_model
  d = write_random_model(copy.deepcopy(plain.CONFIGS["Q"]), str(tmp_path / "m"), seed=4)
  W, cfg = plain.read_weights(d), plain.read_config(d)
  assert cfg == {**plain.CONFIGS["Q"], "torch_dtype": "bfloat16"} or {k: cfg[k] for k in plain.CONFIGS["Q"]} == plain.CONFIGS["Q"]
  assert W["l0.mix.vmix"].shape == () and W["l2.mlp.e2.down"].shape == (96, 56)
  assert torch.isfinite(plain.forward(W, cfg, [1, 2, 3])).all()


@pytest.mark.parametrize("tag,page", [("P", 16), ("Q", 8)])
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
    rc.compare(got, ref, 2e-4, f"rikanex {tag}/{name}")
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]


def test_trace_program_picks_the_model_by_its_configuration(cpu_kernels, model_p, tmp_path):
  from miniinfer_b200.engine import replay
  reqs = rc.make_requests(300, (20, 9), seed=2)
  trace = rc.mixed(reqs, 128, seed=3)
  out = io.StringIO()
  code = replay.main(["--model", model_p, "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128",
                      "--device", "cpu"], stdin=io.StringIO("\n".join(json.dumps(r) for r in trace) + "\n"), stdout=out)
  assert code == 0 and out.getvalue().split("\n")[:-1] == [f"done {r['step']}" for r in trace]
  outputs = {r["step"]: np.fromfile(tmp_path / "o" / f"{r['step']}.f32", dtype="<f4").reshape(-1, 300)
             for r in trace if sum(len(e["want"]) for e in r["entries"])}
  W, cfg = plain.read_weights(model_p), plain.read_config(model_p)
  rc.compare(rc.collect(trace, outputs), {rid: plain.forward(W, cfg, ids) for rid, ids in reqs.items()}, 2e-4, "trace program")
