"""The Generax decoder through the engine against the plain NumPy model.

Each scenario runs on the CPU with the plain PyTorch kernel statements (this checks the parts,
the configuration, the cache manager and the step function) and, marked `gpu`, with the CUDA
kernels in float32 and bfloat16."""

import copy
import json
import os

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, SamplingParams, StepEntry
from simply_b200.config import ConfigError, config_from_dict, load_config
from simply_b200.parts.model import DecoderModel
from simply_b200.weights import write_model_folder
from tests import generax_cases as gx
from tests.plain import generax_plain as plain
from tests.reference_ops import ReferenceOps

CPU = pytest.param(("float32", "cpu"), id="cpu")
GPU32 = pytest.param(("float32", "cuda"), id="gpu-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param(("bfloat16", "cuda"), id="gpu-bf16", marks=pytest.mark.gpu)
WHERE = [CPU, GPU32, GPU16]


def engine_for(cfg_dict, where, seed=0, tensors=None, **kw):
  dtype, device = where
  cfg, t = gx.weights(cfg_dict, seed)
  if tensors is not None:
    t = tensors
  ops = ReferenceOps(torch.float32) if device == "cpu" else None
  return gx.build_engine(cfg, t, dtype, device, ops, **kw), t


def tokens_for(cfg_dict, n, seed):
  return np.random.default_rng(seed).integers(0, cfg_dict["vocab"], n).tolist()


# ---- whole prompts, portions, decoding, batches -------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("which", ["a", "b"])
def test_whole_portions_and_decoding(which, where):
  cfg_dict = gx.CONFIG_A if which == "a" else gx.CONFIG_B
  engine, t = engine_for(cfg_dict, where, seed=3)
  toks = tokens_for(cfg_dict, 61, 1)
  want = plain.forward(cfg_dict, gx.as_numpy(t), toks)
  n = len(toks)
  for what, cuts in [
      ("whole", [n]),
      ("token by token", [1] * n),
      ("prompt then decoding", [n - 40] + [1] * 40),
      ("portions down to two tokens", gx.cuts_of(n, [7, 2, 5, 3, 11, 2, 13, 4, 2, 9])),
      ("portions of two", [2] * (n // 2) + [1]),
      ("one token, then the rest", [1, n - 1]),
  ]:
    gx.check_close(gx.run_cuts(engine, toks, cuts), want, where[0], f"{which}: {what}")
  engine.cache.check_invariants()
  assert engine.cache.all_pages_free()
  engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
def test_unequal_requests_side_by_side_with_pages_and_slots_used_again(where):
  cfg_dict = gx.CONFIG_B
  # room for three live requests of these lengths, not for all six: pages and slots come back
  engine, t = engine_for(cfg_dict, where, seed=5, slots=3, max_cache_tokens=3 * 80, poison=True)
  lengths = [70, 9, 33, 1, 58, 21]
  requests = [tokens_for(cfg_dict, n, 10 + i) for i, n in enumerate(lengths)]
  w = gx.as_numpy(t)
  want = [plain.forward(cfg_dict, w, r) for r in requests]
  got = gx.run_mixed(engine, requests, seed=2)
  for i, (g, x) in enumerate(zip(got, want)):
    gx.check_close(g, x, where[0], f"request {i} in a mixed batch")
  # the same requests once more through the used slots and pages, each alone
  for i in (0, 4):
    gx.check_close(gx.run_cuts(engine, requests[i], [len(requests[i])]), want[i], where[0], f"request {i} again")
  engine.cache.check_invariants()
  assert engine.cache.all_pages_free()
  engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
def test_long_decoding_past_windows_blocks_and_pages(where):
  cfg_dict = gx.CONFIG_A
  engine, t = engine_for(cfg_dict, where, seed=7, page_size=4)
  toks = tokens_for(cfg_dict, 150, 4)
  want = plain.forward(cfg_dict, gx.as_numpy(t), toks)
  gx.check_close(gx.run_cuts(engine, toks, [3] + [1] * 147), want, where[0], "long decoding")
  engine.ops.check_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_more_blocks_than_a_tile_holds_and_pages_of_64(dtype):
  """330 tokens with blocks of 4: more block entries than one tile of 64 keys, windows that pass many
  pages of 64, head sizes 32 and 64, four heads per kv head, a reader with a wider window."""
  cfg_dict = gx.config(
      [gx.attention(heads=8, kv_heads=2, dim=32, vdim=32, window=50, dims=16, base=5000.0, factor=4.0, scale=0.2),
       gx.parallel(heads=8, kv_heads=2, dim=32, vdim=32, window=40, pool=4, scale=0.2, r_heads=4, r_kv_heads=2,
                   r_dim=32, r_vdim=64, conv=3, ranks=(16, 8)),
       gx.attention(heads=8, kv_heads=2, dim=32, vdim=32, window=80, dims=16, base=5000.0, factor=4.0, scale=0.2,
                    kv_from=0),
       gx.parallel(heads=4, kv_heads=4, dim=64, vdim=64, window=33, pool=12, scale=0.15, r_heads=2, r_kv_heads=2,
                   r_dim=128, r_vdim=128, conv=4, ranks=(8, 8))],
      width=128, vocab=300, ff=256)
  cfg, t = gx.weights(cfg_dict, seed=3, matrix_std=0.1)
  engine = gx.build_engine(cfg, t, dtype, "cuda", None, page_size=64, slots=2, max_seq_len=512)
  toks = tokens_for(cfg_dict, 330, 1)
  want = plain.forward(cfg_dict, gx.as_numpy(t), toks)
  for what, cuts in [("whole", [330]), ("portions", gx.cuts_of(330, [100, 2, 37, 64, 3, 129])),
                     ("decoding", [270] + [1] * 60)]:
    gx.check_close(gx.run_cuts(engine, toks, cuts), want, dtype, what)
  engine.ops.check_errors()


# ---- a key that stands out ----------------------------------------------------------------------

def needle_case(kind):
  """A one-layer model whose query of token 1 is answered by the key of token 2 alone."""
  if kind == "window":
    layers = [gx.attention(heads=4, kv_heads=2, dim=16, vdim=16, window=12, dims=8, scale=1.0)]
  elif kind == "window, other value size":
    layers = [gx.attention(heads=2, kv_heads=2, dim=16, vdim=8, window=12, dims=8, scale=1.0)]
  else:
    layers = [gx.parallel(heads=4, kv_heads=2, dim=16, vdim=16, window=12, pool=5, scale=1.0)]
  cfg_dict = gx.config(layers, width=32, vocab=50, ff=32)
  cfg, t = gx.weights(cfg_dict, seed=11)
  gx.plant_needle(cfg_dict, t, 0, needle=2, asker=1, left=kind == "pool")
  return cfg_dict, t


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("kind", ["window", "window, other value size", "pool"])
def test_a_key_that_stands_out_at_every_edge(kind, where):
  cfg_dict, t = needle_case(kind)
  w = gx.as_numpy(t)
  window, pool = 12, 5
  rng = np.random.default_rng(0)
  n = 75
  # distances at which the asker sees the needle last / no longer; with blocks, the needle comes
  # back once its whole block has left the window
  distances = [0, 1, window - 1, window, window + 1, 40, 63]
  if kind == "pool":
    distances += [window + pool - 2, window + pool - 1, window + pool, window + 2 * pool]
  engine, _ = engine_for(cfg_dict, where, tensors=t, page_size=8)
  seen_change = False
  for needle_at in (0, 3, 7, 8):  # the first tokens, and either side of a page's border
    for dist in distances:
      ask_at = needle_at + dist
      if ask_at >= n:
        continue
      toks = rng.integers(3, cfg_dict["vocab"], n).tolist()
      toks[needle_at] = 2
      if dist:
        toks[ask_at] = 1
      want = plain.forward(cfg_dict, w, toks)
      without = list(toks)
      without[needle_at] = 5
      if dist and np.abs(plain.forward(cfg_dict, w, without)[ask_at] - want[ask_at]).max() > 0.5:
        seen_change = True  # the needle decides the asker's logits here
      for cuts in ([n], [ask_at, 1, n], [max(ask_at - 1, 1), 2, n], gx.cuts_of(n, [5, 2, 3]), [needle_at + 1] + [1] * n):
        got = gx.run_cuts(engine, toks, [c for c in cuts if c > 0])
        gx.check_close(got, want, where[0], f"{kind}: needle at {needle_at}, asked at {ask_at}, cuts {cuts[:3]}")
  assert seen_change, "the planted key never decided anything: the test's weights are too weak"
  engine.ops.check_errors()


@pytest.mark.parametrize("where", WHERE)
def test_state_that_remembers_far_back(where):
  """Only the delta rule's state connects the last token with the first ones (every window is
  short, no blocks yet), so a state that is lost, zeroed or mixed up between slots shows."""
  layers = [gx.parallel(window=3, pool=64, r_heads=2, r_kv_heads=1, r_dim=16, r_vdim=16, conv=4)]
  cfg_dict = gx.config(layers, width=32, vocab=60, ff=32)
  engine, t = engine_for(cfg_dict, where, seed=21)
  w = gx.as_numpy(t)
  a, b = tokens_for(cfg_dict, 48, 1), tokens_for(cfg_dict, 48, 2)
  c = list(a)
  c[2] = (c[2] + 1) % cfg_dict["vocab"]
  want_a, want_c = plain.forward(cfg_dict, w, a), plain.forward(cfg_dict, w, c)
  assert np.abs(want_a[-1] - want_c[-1]).max() > 1e-2 * np.abs(want_a).max(), "the state forgets too fast for this test"
  got = gx.run_mixed(engine, [a, b, c], seed=5, max_live=3, portions=(2, 3, 4))
  gx.check_close(got[0], want_a, where[0], "a")
  gx.check_close(got[1], plain.forward(cfg_dict, w, b), where[0], "b")
  gx.check_close(got[2], want_c, where[0], "c")


# ---- generation through the entry point and the scheduler -----------------------------------------

@pytest.mark.parametrize("where", [CPU, GPU32])
def test_greedy_generation_through_the_scheduler(where):
  cfg_dict = gx.CONFIG_B
  engine, t = engine_for(cfg_dict, where, seed=9, slots=2)
  w = gx.as_numpy(t)
  prompts = [tokens_for(cfg_dict, n, 30 + i) for i, n in enumerate((5, 17, 1, 26))]
  results = engine.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=12))
  for prompt, r in zip(prompts, results):
    toks = list(prompt)
    for _ in range(12):
      toks.append(int(np.argmax(plain.forward(cfg_dict, w, toks)[-1])))
    assert r.output_token_ids == toks[len(prompt):], (r.output_token_ids, toks[len(prompt):])
  assert engine.cache.all_pages_free()


@pytest.mark.gpu
@pytest.mark.parametrize("which,burst", [("a", 1), ("b", 5)])
def test_decoding_from_cuda_graphs(which, burst):
  """Three live requests decode from the graph of four rows (the fourth repeats the third and
  must not touch its state a second time), several steps per replay burst."""
  cfg_dict = gx.CONFIG_A if which == "a" else gx.CONFIG_B
  engine, t = engine_for(cfg_dict, ("float32", "cuda"), seed=13, slots=4, graphs=True, burst=burst)
  assert engine._decode_runner is not None, "the model's parts must all allow graph capture"
  w = gx.as_numpy(t)
  prompts = [tokens_for(cfg_dict, n, 40 + i) for i, n in enumerate((9, 3, 14))]
  results = engine.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=17))
  assert engine._decode_runner.bursts > 0
  for prompt, r in zip(prompts, results):
    toks = list(prompt)
    for _ in range(17):
      toks.append(int(np.argmax(plain.forward(cfg_dict, w, toks)[-1])))
    assert r.output_token_ids == toks[len(prompt):], (r.output_token_ids, toks[len(prompt):])
  engine.ops.check_errors()


@pytest.mark.gpu
def test_bfloat16_generation_runs_and_samples():
  engine, _ = engine_for(gx.CONFIG_A, ("bfloat16", "cuda"), seed=2, slots=3)
  prompts = [tokens_for(gx.CONFIG_A, n, i) for i, n in enumerate((4, 30, 11, 2, 19))]
  results = engine.generate(prompts, SamplingParams(temperature=0.8, top_k=20, max_decode_steps=20, seed=4))
  assert all(len(r.output_token_ids) == 20 for r in results)
  again = engine.generate(prompts, SamplingParams(temperature=0.8, top_k=20, max_decode_steps=20, seed=4))
  assert [r.output_token_ids for r in results][0] == [r.output_token_ids for r in again][0]
  engine.ops.check_errors()


@pytest.mark.gpu
def test_bfloat16_single_tokens_replayed_from_cuda_graphs():
  """Three requests side by side, their last 30 tokens one by one as replays of the decode graph of
  four rows; the logits of every replayed step against the plain model."""
  cfg_dict = gx.CONFIG_A
  engine, t = engine_for(cfg_dict, ("bfloat16", "cuda"), seed=6, slots=4, graphs=True)
  assert engine._decode_runner is not None
  engine._decode_runner.keep_logits = True
  w = gx.as_numpy(t)
  requests = [tokens_for(cfg_dict, n, 50 + i) for i, n in enumerate((70, 41, 55))]
  want = [plain.forward(cfg_dict, w, r) for r in requests]
  slots = [engine.open_request() for _ in requests]
  heads = [len(r) - 30 for r in requests]
  engine.step_raw([StepEntry(s, r[:h], ()) for s, r, h in zip(slots, requests, heads)])
  got = [[] for _ in requests]
  for step in range(30):
    entries = [StepEntry(s, [r[h + step]], (0,)) for s, r, h in zip(slots, requests, heads)]
    logits = engine.step_raw(entries, from_graph=True).float().cpu().numpy()
    for i in range(len(requests)):
      got[i].append(logits[i])
  for i, h in enumerate(heads):
    gx.check_close(np.stack(got[i]), want[i][h:], "bfloat16", f"request {i}, replayed steps")
  assert engine._decode_runner.bursts >= 30
  engine.ops.check_errors()


# ---- configuration and model folders --------------------------------------------------------------

def test_a_model_folder_gives_the_ranks_that_no_key_names(tmp_path):
  cfg = config_from_dict(gx.CONFIG_B)
  folder = write_model_folder(cfg, 3, str(tmp_path / "m"), matrix_std=0.2, scale_std=0.1)
  path = os.path.join(folder, "config.json")
  with open(path) as f:
    d = json.load(f)
  for layer in d["layers"]:
    if layer["type"] == "parallel":
      del layer["mixer"]["right"]["decay_rank"], layer["mixer"]["right"]["gate_rank"]
  del d["max_context"]
  with open(path, "w") as f:
    json.dump(d, f)
  loaded = load_config(folder)
  assert type(loaded).__name__ == "GeneraxConfig"
  ec = EngineConfig(activation_dtype="float32", page_size=8, batch_size=2, max_seq_len=64)
  engine = Engine.from_folder(folder, ec, ops=ReferenceOps(torch.float32))
  from simply_b200.weights import safetensors_io as st
  reader = st.TensorReader(st.index_files(st.model_files(folder)))
  w = {k: reader.read(k).float().numpy() for k in reader.entries}
  toks = tokens_for(gx.CONFIG_B, 20, 0)
  slot = engine.open_request()
  got = engine.step_raw([StepEntry(slot, toks, tuple(range(20)))]).numpy()
  gx.check_close(got, plain.forward(d, w, toks), "float32", "from a folder")


def test_layers_name_their_caches_and_tensors():
  spec = config_from_dict(gx.CONFIG_A).model_spec()
  model = DecoderModel(spec)
  assert model.cache_names == ["l0#0", "l1#1", "l1#1", "l3#3"]
  needs = model.cache_needs()
  assert needs["l1#1"].window == 9  # the writer's 9 covers the reader's 7
  assert set(needs["l0#0"]) == {"left", "right"} and set(needs["l0#0"]["left"]) == {"kv", "pool"}
  assert needs["l0#0"]["left"]["pool"].stride == 4 and needs["l0#0"]["left"]["pool"].window is None
  names = {s.name for s in model.tensor_specs()}
  assert {"embed", "head", "final.norm", "l0.norm1", "l0.mix.left.q.norm", "l0.mix.right.A_log", "l0.mix.right.q.conv",
          "l0.mix.left.out", "l1.mix.temp", "l2.mix.q", "l3.mlp.down"} <= names
  assert "l2.mix.k" not in names and "l2.mix.k.norm" not in names and "l0.mix.left.temp" not in names
  # a reader with a wider window than its writer widens what the cache keeps
  spec_b = config_from_dict(gx.CONFIG_B).model_spec()
  assert DecoderModel(spec_b).cache_needs()["l0#0"].window == 11


def test_configurations_that_cannot_run_are_refused():
  def broken(change):
    d = copy.deepcopy(gx.CONFIG_A)
    change(d)
    return d
  cases = [
      lambda d: d["layers"][2]["mixer"].update(kv_from=3),  # a later layer
      lambda d: d["layers"][2]["mixer"].update(kv_from=0),  # not an attention layer
      lambda d: d["layers"][2]["mixer"].update(dim=8),  # another key size than the cache's
      lambda d: d["layers"][0].update(type="other"),
      lambda d: d["layers"][0]["mlp"].update(kind="experts"),
      lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7),
      lambda d: d.pop("norm"),
      lambda d: d["layers"][0]["mixer"]["left"]["mask"].pop("size"),
  ]
  for change in cases:
    with pytest.raises(ConfigError):
      config_from_dict(broken(change))


# ---- the command line -----------------------------------------------------------------------------

def _cli(*args):
  import subprocess
  import sys
  repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  env = dict(os.environ, PYTHONPATH=repo + os.pathsep + os.environ.get("PYTHONPATH", ""))
  p = subprocess.run([sys.executable, "-m", "simply_b200", *args], capture_output=True, text=True, env=env, cwd=repo,
                     timeout=900)
  assert p.returncode == 0, p.stderr[-2000:]
  return [json.loads(line) for line in p.stdout.splitlines() if line.startswith("{")]


def test_the_command_line_writes_a_generax_folder(tmp_path):
  out = str(tmp_path / "m")
  assert _cli("--experiment_config", "generax-tiny", "--write_model_dir", out, "--model_seed", "1",
              "--matrix_std", "0.2", "--scale_std", "0.1") == [{"wrote": out}]
  with open(os.path.join(out, "config.json")) as f:
    d = json.load(f)
  assert d["architecture"] == "Generax" and [l["type"] for l in d["layers"]] == ["parallel", "attention", "attention"]
  cfg = load_config(out)
  assert cfg.to_dict() == d
  engine = Engine.from_folder(out, EngineConfig(activation_dtype="float32", page_size=8, batch_size=2, max_seq_len=64),
                              ops=ReferenceOps(torch.float32))
  r = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_decode_steps=4))
  assert len(r[0].output_token_ids) == 4


@pytest.mark.gpu
def test_the_command_line_generates_from_a_generax_folder(tmp_path):
  out = str(tmp_path / "m")
  _cli("--experiment_config", "generax-tiny", "--write_model_dir", out, "--model_seed", "1", "--matrix_std", "0.2",
       "--scale_std", "0.1")
  lines = _cli("--ckpt_dir", out, "--prompt_ids", "1,2,3;9,8,7,6,5", "--temperature", "0", "--max_decode_steps", "12",
               "--activation_dtype", "float32", "--max_seq_len", "128", "--batch_size", "2")
  assert [len(l["output_token_ids"]) for l in lines] == [12, 12]
  from simply_b200.weights import safetensors_io as st
  reader = st.TensorReader(st.index_files(st.model_files(out)))
  w = {k: reader.read(k).float().numpy() for k in reader.entries}
  with open(os.path.join(out, "config.json")) as f:
    d = json.load(f)
  for line in lines:
    toks = list(line["input_token_ids"])
    for _ in range(12):
      toks.append(int(np.argmax(plain.forward(d, w, toks)[-1])))
    assert line["output_token_ids"] == toks[len(line["input_token_ids"]):]
  lines = _cli("--experiment_config", "generax-tiny", "--random_weights", "--prompt_ids", "4,5,6", "--max_decode_steps", "5",
               "--max_seq_len", "128")
  assert len(lines[0]["output_token_ids"]) == 5


# ---- the replay tool, as a user runs it ---------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_tool_four_ways(tmp_path, dtype):
  """bin/trace_run as a child process on a folder of this design: every request whole, prompt then
  single tokens, changing portions, and several live requests in a pool that holds only what is
  live at once (pages and slots come back), against the plain model."""
  from tests import trace_util
  cfg = config_from_dict(dict(gx.CONFIG_B, max_context=1024))
  folder = write_model_folder(cfg, 4, str(tmp_path / "m"), matrix_std=0.2, scale_std=0.15)
  from simply_b200.weights import safetensors_io as st
  reader = st.TensorReader(st.index_files(st.model_files(folder)))
  w = {k: reader.read(k).float().numpy() for k in reader.entries}
  with open(os.path.join(folder, "config.json")) as f:
    d = json.load(f)
  rng = np.random.default_rng(8)
  requests = {f"q{i}": rng.integers(0, d["vocab"], n).tolist() for i, n in enumerate((150, 70, 1, 97, 40, 131))}
  want = {rid: plain.forward(d, w, toks) for rid, toks in requests.items()}
  ways = {"whole": trace_util.whole(requests), "decode": trace_util.prefill_then_decode(requests, tail=40),
          "portions": trace_util.changing_portions(requests), "mixed": trace_util.mixed(requests, seed=1)}
  for name, steps in ways.items():
    out = str(tmp_path / f"{name}_{dtype}")
    trace_util.run_tool(folder, dtype, steps, out, trace_util.tokens_needed(steps), extra=("--poison-freed-pages",))
    got = trace_util.collect(steps, out, d["vocab"])
    for rid, rows in got.items():
      gx.check_close(np.stack([rows[p] for p in sorted(rows)]), want[rid], dtype, f"{name}: {rid}")
