"""Each mechanism of the Generax mixers alone: one call of the kernel table (the CUDA kernels on a
GPU, their plain PyTorch statements on the CPU) against the function of the plain NumPy model."""

import numpy as np
import pytest
import torch

from simply_b200.cache import CacheManager, PagedKVNeed
from simply_b200.engine.batch import StepEntry, pack_step
from simply_b200.parts.normed_attention import rotation_frequencies
from tests.plain import generax_plain as plain
from tests.reference_ops import ReferenceOps

CPU = pytest.param(("float32", "cpu"), id="cpu")
GPU32 = pytest.param(("float32", "cuda"), id="gpu-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param(("bfloat16", "cuda"), id="gpu-bf16", marks=pytest.mark.gpu)
WHERE = [CPU, GPU32, GPU16]


def table(where):
  dtype, device = where
  if device == "cpu":
    return ReferenceOps(torch.float32), torch.float32
  from simply_b200.kernels.ops import CudaOps
  return CudaOps(getattr(torch, dtype)), getattr(torch, dtype)


def close(got, want, dtype, what, f32=2e-5, bf16=2e-2):
  got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
  bound = (f32 if dtype == torch.float32 else bf16) * max(np.abs(want).max(), 1e-6)
  assert np.isfinite(got).all(), what
  assert np.abs(got - want).max() <= bound, f"{what}: {np.abs(got - want).max():.3e} over {bound:.3e}"


def context(ops, device, lengths_before, new_counts, slots=None, tables=(), page_size=8):
  entries = [StepEntry(slots[i] if slots else i, [0] * n, ()) for i, n in enumerate(new_counts)]
  return pack_step(entries, lengths_before, list(tables), page_size, ops, device)


def rounded(x, dtype):
  """What the kernel table gets: values the storage type holds exactly."""
  return torch.from_numpy(np.asarray(x, np.float32)).to(dtype)


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(2, 1, 12, 8), (3, 3, 16, 24), (4, 2, 40, 5), (2, 2, 128, 64)])
def test_the_scan_carries_its_state_between_steps(sizes, where):
  heads, kv_heads, d, dv = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(0)
  lengths = [23, 9]
  total = sum(lengths)
  q = rng.standard_normal((total, kv_heads, d)) * d ** -0.5
  k = plain.unit(rng.standard_normal((total, kv_heads, d)))
  v = rng.standard_normal((total, heads, dv))
  decay = rng.uniform(0.6, 1.0, (total, heads, d))
  beta = rng.uniform(0.0, 1.0, (total, heads))
  f = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(device)
  state = torch.zeros(4, heads, d, dv, device=device)
  state[1] = 7.0  # another request's slot must stay as it is
  rep = heads // kv_heads
  want, got = [], [[], []]
  start = 0
  for n in lengths:
    sl = slice(start, start + n)
    want.append(plain.gated_delta_rule(np.repeat(q[sl], rep, 1), np.repeat(k[sl], rep, 1), v[sl], beta[sl], decay[sl]))
    start += n
  # three steps: unequal portions of both, then the rest; slots 3 and 0
  cuts = [(10, 2), (1, 6), (12, 1)]
  done = [0, 0]
  for cut in cuts:
    rows = np.concatenate([np.arange(done[i], done[i] + cut[i]) + (0 if i == 0 else lengths[0]) for i in range(2)])
    ctx = context(ops, device, done, list(cut), slots=[3, 0])
    out = ops.gated_delta_scan(f(q[rows]), f(k[rows]), f(v[rows]), f(decay[rows]), f(beta[rows]), state, ctx,
                               num_heads=heads, num_kv_heads=kv_heads, head_dim=d, value_dim=dv)
    out = out.cpu().numpy()
    got[0].append(out[:cut[0]])
    got[1].append(out[cut[0]:])
    done = [done[i] + cut[i] for i in range(2)]
  for i in range(2):
    close(np.concatenate(got[i]), want[i], torch.float32, f"sequence {i}", f32=5e-5)
  assert float(state[1].min()) == 7.0 and float(state[1].max()) == 7.0
  assert float(state[2].abs().max()) == 0.0


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("taps", [1, 2, 4, 6])
def test_short_convolutions_unit_vectors_decays_and_beta(taps, where):
  ops, dtype = table(where)
  device = where[1]
  heads, kv_heads, d, dv = 4, 2, 8, 6
  qk, vv = kv_heads * d, heads * dv
  channels = 2 * qk + vv
  rng = np.random.default_rng(taps)
  n = 15
  pre = rounded(rng.standard_normal((n, channels + heads + 3)), dtype)  # (three columns of padding)
  low = rounded(rng.standard_normal((n, heads * d + vv)), dtype)
  conv_w = rng.standard_normal((channels, taps)).astype(np.float32)
  bias = rng.standard_normal(heads * d).astype(np.float32) - 1.0
  neg_rate = -np.exp(rng.standard_normal(heads).astype(np.float32))
  state = torch.zeros(3, max(taps - 1, 0), channels, device=device)
  x = pre.float().numpy()
  y = plain.silu(plain.short_conv(x[:, :channels].astype(np.float64), conv_w.astype(np.float64)))
  want_q = plain.unit(y[:, :qk].reshape(n, kv_heads, d)) * d ** -0.5
  want_k = plain.unit(y[:, qk:2 * qk].reshape(n, kv_heads, d))
  want_v = y[:, 2 * qk:].reshape(n, heads, dv)
  want_beta = plain.sigmoid(x[:, channels:channels + heads].astype(np.float64))
  a = low.float().numpy()[:, :heads * d].astype(np.float64) + bias
  want_decay = np.exp(neg_rate[None, :, None] * plain.softplus(a).reshape(n, heads, d))
  got = [[] for _ in range(5)]
  done = 0
  for cut in (1, 2, 1, 7, 4):  # the first token alone, portions shorter and longer than the taps
    ctx = context(ops, device, [done], [cut], slots=[2])
    outs = ops.delta_rule_inputs(pre[done:done + cut].to(device), low[done:done + cut].to(device),
                                 torch.from_numpy(conv_w).to(device), state, torch.from_numpy(bias).to(device),
                                 torch.from_numpy(neg_rate).to(device), ctx, conv_taps=taps, num_heads=heads,
                                 num_kv_heads=kv_heads, head_dim=d, value_dim=dv)
    for g, o in zip(got, outs):
      g.append(o.float().cpu().numpy())
    done += cut
  for g, want, what in zip(got, (want_q, want_k, want_v, want_decay, want_beta), ("q", "k", "v", "decay", "beta")):
    close(np.concatenate(g), want, torch.float32, what, f32=5e-5)


@pytest.mark.parametrize("where", WHERE)
def test_head_norm_with_gate_and_mean_of_normed_branches(where):
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(2)
  n, heads, dv, eps = 9, 3, 20, 1e-5
  o = rng.standard_normal((n, heads, dv)).astype(np.float32) * 3
  low = rounded(rng.standard_normal((n, 7 + heads * dv)), dtype)
  w = (1 + 0.3 * rng.standard_normal(dv)).astype(np.float32)
  got = ops.gated_head_norm(torch.from_numpy(o).to(device), low.to(device), 7, torch.from_numpy(w).to(device), eps, heads, dv)
  normed = (o / np.sqrt((o.astype(np.float64) ** 2).mean(-1, keepdims=True) + eps) * w).reshape(n, -1)
  want = normed * plain.sigmoid(low.float().numpy()[:, 7:].astype(np.float64))
  close(got.float().cpu().numpy(), want, dtype, "head norm")
  for width in (48, 50):
    xs = [rounded(rng.standard_normal((n, width)) * s, dtype) for s in (1.0, 5.0, 0.1)]
    ws = [(1 + 0.3 * rng.standard_normal(width)).astype(np.float32) for _ in xs]
    for count in (1, 2, 3):
      got = ops.normed_mean([x.to(device) for x in xs[:count]], [torch.from_numpy(v).to(device) for v in ws[:count]], eps)
      want = sum(plain.rms_norm(x.float().numpy().astype(np.float64), v, eps) for x, v in zip(xs[:count], ws)) / count
      close(got.float().cpu().numpy(), want, dtype, f"mean of {count}, width {width}")


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(4, 2, 16, 16, 8), (3, 1, 16, 24, 16), (2, 2, 12, 6, 0), (16, 4, 128, 128, 64)])
def test_norm_over_whole_projections_rotations_and_the_cache(sizes, where):
  heads, kv_heads, d, dv, dims = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(3)
  page, eps, base, factor = 8, 1e-5, 300.0, 2.0
  need = PagedKVNeed(kv_heads, d, None, value_dim=None if dv == d else dv)
  cache = CacheManager({"c": need}, page_size=page, max_slots=2, max_seq_len=64, max_cache_tokens=128, dtype=dtype,
                       device=device)
  slot = cache.acquire_slot("r")
  start, n = 5, 13  # positions 5 .. 17: across two page borders
  cache.extend([(slot, start)])
  cache.extend([(slot, n)])
  ctx = pack_step([StepEntry(slot, [0] * n, ())], [start], [g.tables for g in cache.groups], page, ops, device)
  nq, nk = heads * d, kv_heads * d
  qkv = rounded(rng.standard_normal((n, nq + nk + kv_heads * dv + 8)), dtype)
  qn = (1 + 0.2 * rng.standard_normal(nq)).astype(np.float32)
  kn = (1 + 0.2 * rng.standard_normal(nk)).astype(np.float32)
  scale = rng.uniform(0.1, 0.5, heads).astype(np.float32)
  rot = torch.from_numpy(rotation_frequencies(dims, base, factor)).to(device) if dims else None
  vf = torch.from_numpy(rotation_frequencies(dv, base)).to(device) if dims else None
  storage = cache.paged["c"].storage
  q = ops.qk_norm_rotate_store(qkv.to(device), torch.from_numpy(qn).to(device), torch.from_numpy(kn).to(device), eps,
                               torch.from_numpy(scale).to(device), rot, vf, heads, kv_heads, d, dv, storage,
                               ctx.block_tables[0], ctx)
  x = qkv.float().numpy().astype(np.float64)
  pos = np.arange(start, start + n)
  want_q = plain.rms_norm(x[:, :nq], qn, eps).reshape(n, heads, d)
  want_k = plain.rms_norm(x[:, nq:nq + nk], kn, eps).reshape(n, kv_heads, d)
  want_v = x[:, nq + nk:nq + nk + kv_heads * dv].reshape(n, kv_heads, dv)
  if dims:
    want_q, want_k = plain.rotary(want_q, pos, dims, base, factor), plain.rotary(want_k, pos, dims, base, factor)
    want_v = plain.rotary(want_v, pos, dv, base)
  close(q.float().cpu().numpy().reshape(n, heads, d), want_q * scale[None, :, None], dtype, "queries")
  keys, values = ReferenceOps._kv_views(storage, kv_heads, page, d, dv)
  table_row = cache.groups[0].tables[slot]
  got_k = np.stack([keys[table_row[p // page], :, p % page].float().cpu().numpy() for p in pos])
  got_v = np.stack([values[table_row[p // page], :, p % page].float().cpu().numpy() for p in pos])
  close(got_k, want_k, dtype, "cached keys")
  close(got_v, want_v, dtype, "cached values")
  if dims:  # a head's result turned back by its own position is what came in
    flat = rounded(rng.standard_normal((n, heads * dv)), dtype).to(device)
    there = ops.rotate_heads(flat, ctx.positions, vf, heads, dv)
    back = ops.rotate_heads(there, ctx.positions, vf, heads, dv, inverse=True)
    close(back.float().cpu().numpy(), flat.float().cpu().numpy(), dtype, "there and back")
    want = plain.rotary(flat.float().cpu().numpy().astype(np.float64).reshape(n, heads, dv), pos, dv, base)
    close(there.float().cpu().numpy().reshape(n, heads, dv), want, dtype, "turned")


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("width", [48, 50, 4096])
def test_two_branches_join_the_stream_in_one_step(width, where):
  """h += first + second, then the next norm: what a block adds whose sublayers share one norm."""
  from simply_b200.parts.norm import RMSNorm
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(width)
  n, eps = 7, 1e-5
  h = rng.standard_normal((n, width)).astype(np.float32)
  first, second = (rounded(rng.standard_normal((n, width)), dtype) for _ in range(2))
  norm = RMSNorm("n", width, eps, plus_one=False)
  norm.weight = torch.from_numpy((1 + 0.2 * rng.standard_normal(width)).astype(np.float32)).to(device)
  want_h = h.astype(np.float64) + first.float().numpy() + second.float().numpy()
  want_y = plain.rms_norm(want_h, norm.weight.float().cpu().numpy().astype(np.float64), eps)
  stream = torch.from_numpy(h.copy()).to(device)
  y = ops.residual_norm(stream, first.to(device), None, norm, None, branch2=second.to(device))
  close(stream.cpu().numpy(), want_h, torch.float32, "stream")
  close(y.float().cpu().numpy(), want_y, dtype, "normed")
  rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=device)
  stream = torch.from_numpy(h.copy()).to(device)
  y = ops.residual_norm(stream, first.to(device), None, norm, rows, branch2=second.to(device))
  close(y.float().cpu().numpy(), want_y[[5, 0, 5]], dtype, "gathered rows")
  close(stream.cpu().numpy(), h, torch.float32, "the stream is left alone when rows are gathered")
