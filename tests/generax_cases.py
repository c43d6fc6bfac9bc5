"""Small Generax configurations with random (and crafted) weights, and the ways the tests run them.

Every comparison is between the engine (`Engine.step_raw` / `Engine.generate` with a kernel
table: the CUDA one on a GPU, the plain PyTorch statements on the CPU) and the plain NumPy model
of `tests/plain/generax_plain.py`, which sees whole sequences and has no cache.
"""

from __future__ import annotations

import copy

import numpy as np
import torch

from simply_b200 import Engine, EngineConfig, StepEntry
from simply_b200.config import config_from_dict
from simply_b200.parts.model import DecoderModel
from simply_b200.weights import random_tensors
from tests.plain import generax_plain as plain
from tests.tolerances import assert_logits_close


def attention(heads=4, kv_heads=2, dim=16, vdim=16, window=9, dims=8, base=300.0, factor=1.5, scale=0.4,
              kv_from=None):
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
       "mask": {"size": window}, "rot": {"dims": dims, "base": base, "scaling": {"factor": factor}}}
  if kv_from is not None:
    m["kv_from"] = kv_from
  return {"type": "attention", "mixer": m}


def parallel(heads=4, kv_heads=2, dim=16, vdim=16, window=10, pool=4, scale=0.4, r_heads=4, r_kv_heads=2,
             r_dim=16, r_vdim=8, conv=3, ranks=(6, 5)):
  return {"type": "parallel", "mixer": {
      "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
               "mask": {"size": window, "pool": pool}},
      "right": {"heads": r_heads, "kv_heads": r_kv_heads, "dim": r_dim, "vdim": r_vdim, "conv": conv,
                "decay_rank": ranks[0], "gate_rank": ranks[1]}}}


def config(layers, width=48, vocab=97, ff=64, eps=1e-5, softcap=25.0, no_mlp=()):
  out = []
  for i, layer in enumerate(layers):
    layer = copy.deepcopy(layer)
    layer["mlp"] = None if i in no_mlp else {"kind": "dense", "ff": ff}
    out.append(layer)
  d = {"architecture": "Generax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": out,
       "max_context": 512}
  if softcap:
    d["logit_softcap"] = softcap
  return d


# Two models that differ in every size and switch.  A: key and value heads of one size, whole heads
# rotated, blocks that divide a page.  B: value heads of another size, partly rotated heads, blocks
# that do not divide a page and are longer than one, a reader with a wider window than the cache's
# writer, one kv head, a layer without feed-forward, no cap on the logits.
CONFIG_A = config([parallel(), attention(dims=16), attention(dims=16, kv_from=1, window=7), parallel(pool=2, window=5)])
CONFIG_B = config(
    [attention(heads=3, kv_heads=1, dim=16, vdim=24, window=6, dims=8, base=50.0, factor=1.0, scale=0.3),
     parallel(heads=2, kv_heads=2, dim=8, vdim=12, window=7, pool=3, r_heads=2, r_kv_heads=1, r_dim=24, r_vdim=16,
              conv=2, ranks=(4, 8)),
     attention(heads=3, kv_heads=1, dim=16, vdim=24, window=11, dims=8, base=50.0, factor=1.0, scale=0.3, kv_from=0),
     parallel(heads=6, kv_heads=2, dim=8, vdim=8, window=4, pool=9, r_heads=3, r_kv_heads=3, r_dim=40, r_vdim=8,
              conv=5, ranks=(8, 3))],
    width=40, vocab=131, ff=56, eps=1e-6, softcap=0.0, no_mlp=(2,))


def weights(cfg_dict, seed=0, matrix_std=0.25, scale_std=0.2, slow_decay=True):
  """bfloat16-representable random weights by tensor name (CPU, float32 holding bfloat16 values)."""
  cfg = config_from_dict(cfg_dict)
  specs = DecoderModel(cfg.model_spec()).tensor_specs()
  t = random_tensors(specs, seed, matrix_std=matrix_std, scale_std=scale_std, dtype=torch.bfloat16)
  gen = torch.Generator().manual_seed(seed + 1)
  for name in t:
    if name.endswith(".dt_bias") and slow_decay:
      # decays near 1, so that the state still holds tokens from far back
      t[name] = (torch.randn(t[name].shape, generator=gen) * 0.5 - 3.5).to(torch.bfloat16)
    if name.endswith(".embed") or name == "embed":
      t[name] = torch.randn(t[name].shape, generator=gen).to(torch.bfloat16)
  return cfg, t


def plant_needle(cfg_dict, t, layer, needle, asker, strength=6.0, left=False):
  """Makes the key of token `needle` and the query of token `asker` point the same way in layer
  `layer` (in dims that no rotation touches), far longer than any other, and gives the needle a
  value of its own: while the asker sees the needle, its attention is all on it."""
  m = cfg_dict["layers"][layer]["mixer"]
  m = m["left"] if left else m
  p = f"l{layer}.mix.left" if left else f"l{layer}.mix"
  width = cfg_dict["width"]
  gen = torch.Generator().manual_seed(1234 + layer)
  for tok, sign in ((needle, 1.0), (asker, -1.0)):
    row = torch.zeros(width)
    row[(7 * tok + 3) % width] = 6.0 * sign
    row[(5 * tok + 1) % width] = 6.0
    t["embed"][tok] = row.to(torch.bfloat16)
  norm1 = t[f"l{layer}.norm1"].float()
  y_needle = plain.rms_norm(t["embed"][needle].float().numpy()[None], norm1.numpy(), cfg_dict["norm"]["eps"])[0]
  y_asker = plain.rms_norm(t["embed"][asker].float().numpy()[None], norm1.numpy(), cfg_dict["norm"]["eps"])[0]
  d = m["dim"]
  last = d - 1  # the last dim of a head is outside any rotated range smaller than the head
  for name, y, heads in ((f"{p}.k", y_needle, m["kv_heads"]), (f"{p}.q", y_asker, m["heads"])):
    w = t[name].float()
    y = torch.from_numpy(y).float()
    for h in range(heads):
      w[h * d + last] += strength * y / (y @ y)
    t[name] = w.to(torch.bfloat16)
  for name in (f"{p}.q.norm", f"{p}.k.norm"):
    t[name] = torch.ones_like(t[name])
  v = t[f"{p}.v"].float()
  v += 2.0 * torch.randn(v.shape[0], generator=gen)[:, None] * torch.from_numpy(y_needle).float()[None, :] / float(y_needle @ y_needle)
  t[f"{p}.v"] = v.to(torch.bfloat16)
  return t


def as_numpy(t):
  return {k: v.float().numpy() for k, v in t.items()}


def build_engine(cfg, tensors, dtype, device, ops, *, page_size=8, slots=4, max_cache_tokens=0, max_seq_len=256,
                 poison=False, graphs=False, burst=1):
  on_device = {k: v.to(device=device, dtype=getattr(torch, dtype) if v.is_floating_point() else v.dtype)
               for k, v in tensors.items()}
  ec = EngineConfig(activation_dtype=dtype, page_size=page_size, batch_size=slots, max_seq_len=max_seq_len,
                    max_cache_tokens=max_cache_tokens or slots * max_seq_len, max_window_cache_tokens=-1,
                    poison_freed_pages=poison, use_cuda_graphs=graphs, intermediate_steps=burst)
  return Engine(cfg, on_device, ec, ops=ops, device=device)


def run_cuts(engine, tokens, cuts):
  """One request alone, cut into portions of the given sizes; logits at every position."""
  slot = engine.open_request()
  got, pos = [], 0
  for n in cuts:
    n = min(n, len(tokens) - pos)
    if n <= 0:
      break
    got.append(engine.step_raw([StepEntry(slot, tokens[pos:pos + n], tuple(range(n)))]).float().cpu().numpy())
    pos += n
  assert pos == len(tokens)
  engine.close_request(slot)
  return np.concatenate(got)


def cuts_of(total, sizes):
  out, pos, j = [], 0, 0
  while pos < total:
    n = min(sizes[j % len(sizes)], total - pos)
    out.append(n)
    pos, j = pos + n, j + 1
  return out


def run_mixed(engine, requests, seed=0, max_live=3, portions=(2, 3, 5, 8), decode_after=0.5):
  """Several requests side by side: portions of some beside single tokens of others, requests that
  start as others end, a request sometimes left out of a step.  Logits at every position."""
  rng = np.random.default_rng(seed)
  waiting = list(enumerate(requests))
  live, got = {}, {i: [] for i in range(len(requests))}
  while waiting or live:
    while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
      i, toks = waiting.pop(0)
      live[i] = [toks, 0, engine.open_request()]
    entries, who = [], []
    for i, (toks, pos, slot) in list(live.items()):
      if len(live) > 1 and rng.random() < 0.2:
        continue
      n = 1 if pos >= decode_after * len(toks) else min(int(rng.choice(portions)), len(toks) - pos)
      entries.append(StepEntry(slot, toks[pos:pos + n], tuple(range(n))))
      who.append((i, n))
      live[i][1] = pos + n
    if not entries:
      continue
    logits = engine.step_raw(entries).float().cpu().numpy()
    r = 0
    for i, n in who:
      got[i].append(logits[r:r + n])
      r += n
      if live[i][1] == len(live[i][0]):
        engine.close_request(live[i][2])
        del live[i]
  return [np.concatenate(got[i]) for i in range(len(requests))]


def check_close(got, want, dtype, what):
  assert_logits_close(got, want, dtype, what)
