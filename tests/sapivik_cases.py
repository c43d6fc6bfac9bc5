"""Small Sapivik configurations with random (and crafted) weights for the tests.

Every comparison is between the engine (with a kernel table: the CUDA one on a GPU, the plain
PyTorch statements on the CPU) and the plain NumPy model of `tests/plain/sapivik_plain.py`, which
sees whole sequences and has no cache.  The ways of running an engine (one request cut into
portions, several side by side) are those of `tests/generax_cases.py`.
"""

from __future__ import annotations

import copy

import numpy as np
import torch

from simply_b200.config import config_from_dict
from simply_b200.parts.model import DecoderModel
from simply_b200.weights import random_tensors
from tests.generax_cases import as_numpy, build_engine, cuts_of, run_cuts, run_mixed  # noqa: F401
from tests.tolerances import BF16_MAX, BF16_MEAN, assert_logits_close
from tests.plain import sapivik_plain as plain


def attention(heads=4, kv_heads=2, dim=16, dims=8, base=300.0, scale=0.4, softcap=8.0):
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
  if softcap:
    m["softcap"] = softcap
  if dims:
    m["rot"] = {"dims": dims, "base": base}
  return {"type": "attention", "mixer": m}


def hgrn2(heads=2, dim=24, vdim=16):
  return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def dense(ff=64, limit=1.5):
  return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=6, identity=2, top=3, ff=24, scale=1.7, shared=40):
  m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
  if shared:
    m["shared"] = {"ff": shared}
  return m


def config(layers, mlps, width=48, vocab=97, eps=1e-5, mult=0.6, loop=None):
  out = []
  for layer, mlp in zip(layers, mlps):
    layer = copy.deepcopy(layer)
    layer["mlp"] = copy.deepcopy(mlp)
    out.append(layer)
  d = {"architecture": "Sapivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
       "layers": out, "max_context": 512}
  if loop is not None:
    d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
  return d


# Two models that differ in every size and switch.  A: a loop over the first layers, whole heads of
# 16 partly rotated, experts with identity experts and a shared expert.  B: no loop entry for the
# first layer, a loop of one layer run three times in the middle, head sizes that no tensor-core kernel
# takes, heads rotated over all their dims, no cap on the scores, one kv head, value heads larger than
# key heads in the recurrence, a layer without a feed-forward, experts without identity or shared
# experts, a router that takes every expert it has, a residual factor of 1.
CONFIG_A = config(
    [attention(), hgrn2(), hgrn2(heads=3, dim=8, vdim=16), attention(heads=2, kv_heads=2, dim=32, dims=32, scale=0.3)],
    [dense(), moe(), dense(ff=40, limit=0.8), moe(experts=4, identity=3, top=2, ff=16, shared=24)],
    loop=(0, 3, 2))
CONFIG_B = config(
    [hgrn2(heads=3, dim=8, vdim=40), attention(heads=3, kv_heads=1, dim=20, dims=20, base=50.0, scale=0.27, softcap=0.0),
     hgrn2(heads=1, dim=40, vdim=8), attention(heads=6, kv_heads=3, dim=12, dims=4, scale=0.5, softcap=3.0)],
    [moe(experts=5, identity=0, top=2, ff=20, scale=1.0, shared=0), None, moe(experts=3, identity=0, top=3, ff=8, shared=56),
     dense(ff=72, limit=4.0)],
    width=40, vocab=131, eps=1e-6, mult=1.0, loop=(1, 2, 3))
# No attention at all (no pages, only state slots), and no loop entry.
CONFIG_C = config([hgrn2(heads=2, dim=16, vdim=16), hgrn2(heads=4, dim=8, vdim=8)], [dense(ff=32), None], width=32, vocab=60)


# Sizes without whole 16-byte groups anywhere: an odd width's worth of heads, odd recurrent heads.
CONFIG_D = config([attention(heads=2, kv_heads=1, dim=6, dims=2, scale=0.6), hgrn2(heads=3, dim=5, vdim=7)],
                  [moe(experts=3, identity=1, top=2, ff=10, shared=6), dense(ff=14, limit=1.0)], width=36, vocab=50,
                  loop=(0, 2, 2))


def weights(cfg_dict, seed=0, matrix_std=0.25, scale_std=0.2, slow=True):
  """bfloat16-representable random weights by tensor name (CPU, bfloat16)."""
  cfg = config_from_dict(cfg_dict)
  specs = DecoderModel(cfg.model_spec()).tensor_specs()
  t = random_tensors(specs, seed, matrix_std=matrix_std, scale_std=scale_std, dtype=torch.bfloat16)
  gen = torch.Generator().manual_seed(seed + 1)
  for name in t:
    if name.endswith(".lower"):
      # lower bounds between 0 and 1; with `slow` many close to 1, so that the state still holds
      # tokens from far back
      u = torch.rand(t[name].shape, generator=gen)
      t[name] = (1.0 - 0.3 * u ** 4 if slow else u).to(torch.bfloat16)
    if name.endswith(".f.b") or name.endswith(".correction"):
      t[name] = (torch.randn(t[name].shape, generator=gen) * (0.5 if name.endswith(".f.b") else 0.05)).to(torch.bfloat16)
    if name.endswith(".router"):
      t[name] = (torch.randn(t[name].shape, generator=gen) * 0.6).to(torch.bfloat16)
    if name == "embed":
      t[name] = torch.randn(t[name].shape, generator=gen).to(torch.bfloat16)
  return cfg, t


def plant_needle(cfg_dict, t, layer, needle, asker):
  """Makes the key of token `needle` and the query of token `asker` point the same way in layer
  `layer`, in the last dim of every head (outside a rotated range smaller than the head) and far
  longer than their other dims: after the heads are normed, that score is near dim * scale and
  stands out however many other keys there are.  The needle's key (also its value) is its own."""
  m = cfg_dict["layers"][layer]["mixer"]
  p = f"l{layer}.mix"
  width, d = cfg_dict["width"], m["dim"]
  for tok, sign in ((needle, 1.0), (asker, -1.0)):
    row = torch.zeros(width)
    row[(7 * tok + 3) % width] = 6.0 * sign
    row[(5 * tok + 1) % width] = 6.0
    t["embed"][tok] = row.to(torch.bfloat16)
  norm1 = t[f"l{layer}.norm1"].float().numpy()
  eps = cfg_dict["norm"]["eps"]
  for name, tok, heads in ((f"{p}.k", needle, m["kv_heads"]), (f"{p}.q", asker, m["heads"])):
    y = torch.from_numpy(plain.rms_norm(t["embed"][tok].float().numpy()[None], norm1, eps)[0]).float()
    w = t[name].float()
    for h in range(heads):
      w[h * d + d - 1] += 40.0 * y / (y @ y)
    t[name] = w.to(torch.bfloat16)
  return t


def check_close(got, want, dtype, what):
  """float32: every position within the float32 bound.  bfloat16: a router's choice between two
  experts whose scores are a rounding apart may fall the other way, which moves that token's
  logits (and, faintly, those after it); so at most one position in ten may be over the
  bfloat16 bound, none may be far over it, and the others keep the bound on the mean.  A lost
  key, state or page moves most positions and fails either way."""
  if dtype == "float32":
    return assert_logits_close(got, want, dtype, what)
  got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
  assert got.shape == want.shape, (what, got.shape, want.shape)
  assert np.isfinite(got).all(), f"{what}: logits are not finite"
  scale = np.abs(want).max()
  err = np.abs(got - want)
  worst = err.max(axis=-1)
  over = worst > BF16_MAX * scale
  assert over.sum() <= max(1, len(worst) // 10), f"{what}: {int(over.sum())} of {len(worst)} positions over the bound"
  assert worst.max() <= 0.3 * scale, f"{what}: max diff {worst.max():.3e} of scale {scale:.3e}"
  assert err[~over].mean() <= BF16_MEAN * scale, f"{what}: mean diff {err[~over].mean():.3e} of scale {scale:.3e}"
