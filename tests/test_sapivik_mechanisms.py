"""Each mechanism of the Sapivik layers alone: one call of the kernel table (the CUDA kernels on a
GPU, their plain PyTorch statements on the CPU) against the function of the plain NumPy model, and
one-layer models through the engine."""

import numpy as np
import pytest
import torch

from simply_b200.cache import CacheManager, PagedKVNeed
from simply_b200.engine.batch import StepEntry, pack_step
from simply_b200.parts.normed_attention import rotation_frequencies
from tests import sapivik_cases as sx
from tests.plain import sapivik_plain as plain
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


def held(x, dtype, device):
  """What the kernel table gets: values the storage type holds exactly; also returned as float64."""
  t = torch.from_numpy(np.asarray(x, np.float32)).to(dtype)
  return t.to(device), t.float().numpy().astype(np.float64)


# ---- the forget-gate recurrence -------------------------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(2, 12, 8), (3, 16, 24), (1, 40, 5), (2, 128, 64), (1, 300, 3), (5, 1, 1)])
def test_the_forget_gate_scan_carries_its_state_between_steps(sizes, where):
  heads, d, dv = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(0)
  lengths = [23, 9, 70]
  total = sum(lengths)
  pre, pre64 = held(rng.standard_normal((total, 2 * heads * d + heads * dv + 3)), dtype, device)  # (+3: columns the scan skips)
  bias = rng.standard_normal(heads * d) * 0.5
  lower = rng.uniform(0.0, 1.0, heads * d)
  f32 = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(device)
  bias_t, lower_t = f32(bias), f32(lower)
  bias, lower = bias_t.cpu().numpy().astype(np.float64), lower_t.cpu().numpy().astype(np.float64)
  n = heads * d
  want, start = [], 0
  for length in lengths:
    x = pre64[start:start + length]
    q = plain.silu(x[:, :n]).reshape(length, heads, d)
    f = (lower + (1.0 - lower) * plain.sigmoid(x[:, n:2 * n] + bias)).reshape(length, heads, d)
    v = x[:, 2 * n:2 * n + heads * dv].reshape(length, heads, dv)
    want.append(plain.forget_gate_scan(q, f, v)[0])
    start += length
  state = torch.full((5, heads, d, dv), float("nan"), device=device)
  slots = [3, 0, 4]  # not in order, one slot between them unused
  for s in slots:
    state[s].zero_()
  done = [0, 0, 0]
  got = [[] for _ in lengths]
  starts = np.concatenate([[0], np.cumsum(lengths)[:-1]])
  for portions in ([5, 9, 64], [1, 0, 2], [17, 0, 4]):  # whole sequences, single tokens, leftovers, a sequence left out
    who = [i for i, p in enumerate(portions) if p]
    rows = np.concatenate([np.arange(starts[i] + done[i], starts[i] + done[i] + portions[i]) for i in who])
    ctx = context(ops, device, [done[i] for i in who], [portions[i] for i in who], slots=[slots[i] for i in who])
    out = ops.forget_gate_scan(pre[torch.from_numpy(rows).to(device)].contiguous(), bias_t, lower_t, state, ctx,
                               num_heads=heads, head_dim=d, value_dim=dv).float().cpu().numpy()
    at = 0
    for i in who:
      got[i].append(out[at:at + portions[i]])
      at += portions[i]
      done[i] += portions[i]
  for i in range(len(lengths)):
    g = np.concatenate(got[i])
    close(g, want[i][:len(g)], torch.float32, f"sequence {i} of sizes {sizes}", f32=2e-5 if dtype == torch.float32 else 2e-5)
  assert torch.isnan(state[1]).all() and torch.isnan(state[2]).all(), "a slot no request holds was written"


@pytest.mark.parametrize("where", WHERE)
def test_head_norm_without_a_gate(where):
  ops, dtype = table(where)
  rng = np.random.default_rng(1)
  o = rng.standard_normal((7, 3, 20))
  w = rng.uniform(0.5, 1.5, 20)
  o_t = torch.from_numpy(o.astype(np.float32)).to(where[1])
  w_t = torch.from_numpy(w.astype(np.float32)).to(where[1])
  got = ops.gated_head_norm(o_t, None, -1, w_t, 1e-5, 3, 20).float().cpu().numpy()
  want = plain.rms_norm(o_t.cpu().numpy().astype(np.float64), w_t.cpu().numpy().astype(np.float64), 1e-5).reshape(7, 60)
  close(got, want, dtype, "head norm")


# ---- attention: rotation of neighbours, norm per head, tied values ------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(4, 2, 16, 8), (3, 1, 20, 20), (2, 2, 64, 0), (6, 3, 12, 4)])
def test_rotation_head_norm_and_the_stores(sizes, where):
  heads, kv_heads, d, dims = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(2)
  page_size, lengths_before, new = 8, [13, 0], [9, 5]
  mgr = CacheManager({"c": PagedKVNeed(kv_heads, d, None)}, page_size=page_size, max_slots=3, max_seq_len=64,
                     max_cache_tokens=128, dtype=dtype, device=device)
  slots = [mgr.acquire_slot(i) for i in range(2)]
  mgr.extend([(slots[0], lengths_before[0])])
  mgr.extend([(s, n) for s, n in zip(slots, new)])
  ctx = context(ops, device, lengths_before, new, slots=slots, tables=[g.tables for g in mgr.groups], page_size=page_size)
  total = sum(new)
  width = (heads + kv_heads) * d + heads * d + 5
  proj, proj64 = held(rng.standard_normal((total, width)), dtype, device)
  freq = torch.from_numpy(rotation_frequencies(dims, 300.0)).to(device) if dims else None
  storage = mgr.paged["c"].storage
  storage.fill_(float("nan"))
  q = ops.rotate_headnorm_store(proj, 1e-5, 0.37, freq, interleaved=True, head_norm=True, tie_values=True,
                                num_heads=heads, num_kv_heads=kv_heads, head_dim=d, storage=storage,
                                block_table=ctx.block_tables[0], ctx=ctx).float().cpu().numpy()
  positions = np.concatenate([np.arange(b, b + n) for b, n in zip(lengths_before, new)])
  q_raw = proj64[:, :heads * d].reshape(total, heads, d)
  k_raw = proj64[:, heads * d:(heads + kv_heads) * d].reshape(total, kv_heads, d)
  want_q = plain.rms_norm(plain.turn_neighbours(q_raw, positions, dims, 300.0), None, 1e-5) * 0.37
  want_k = plain.rms_norm(plain.turn_neighbours(k_raw, positions, dims, 300.0), None, 1e-5)
  close(q.reshape(total, heads, d), want_q, dtype, "queries", bf16=1e-2)
  st = storage.float().cpu().numpy()
  tables = mgr.groups[0].tables
  row = 0
  for s, b, n in zip(slots, lengths_before, new):
    for p in range(b, b + n):
      page = int(tables[s, p // page_size])
      close(st[page, 0, :, p % page_size, :], want_k[row], dtype, f"key at {p}", bf16=1e-2)
      close(st[page, 1, :, p % page_size, :], k_raw[row], dtype, f"value at {p} (the key as projected)", bf16=1e-2)
      row += 1
  gate_at = (heads + kv_heads) * d
  x, x64 = held(rng.standard_normal((total, heads * d)), dtype, device)
  got = ops.sigmoid_gate(x.clone(), proj, gate_at).float().cpu().numpy()
  close(got, x64 * plain.sigmoid(proj64[:, gate_at:gate_at + heads * d]), dtype, "output gate")


# ---- feed-forwards ------------------------------------------------------------------------------------

@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("rows,hidden", [(3, 20), (40, 64), (200, 24)])
def test_the_clamped_activation(rows, hidden, where):
  ops, dtype = table(where)
  rng = np.random.default_rng(3)
  gate_up, gu64 = held(rng.standard_normal((rows, 2 * hidden)) * 3.0, dtype, where[1])
  got = ops.gated_activation(gate_up, 3, 1.25).float().cpu().numpy()
  g = np.minimum(gu64[:, :hidden], 1.25)
  u = np.clip(gu64[:, hidden:], -1.25, 1.25)
  close(got, g * plain.sigmoid(1.702 * g) * (u + 1.0), dtype, "clamped activation")


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("sizes", [(8, 2, 3, 24, 40), (37, 0, 37, 16, 8), (3, 5, 4, 72, 20), (2, 1, 1, 64, 32)])
def test_routing_and_the_experts_products(sizes, where):
  experts, identity, top, width, ff = sizes
  ops, dtype = table(where)
  device = where[1]
  rng = np.random.default_rng(4)
  rows = 200  # with few experts: more rows per expert than a tile holds
  mlp = {"kind": "moe", "expert": {"ff": ff}, "shared": {"ff": 16},
         "router": {"experts": experts, "identity": identity, "top": top, "scale": 1.3}}
  w, w64 = {}, {}
  def put(name, value):
    w[name], w64[name] = held(value, dtype, device)
  for e in range(experts):
    put(f"m.e{e}.gate", rng.standard_normal((ff, width)) * 0.3)
    put(f"m.e{e}.up", rng.standard_normal((ff, width)) * 0.3)
    put(f"m.e{e}.down", rng.standard_normal((width, ff)) * 0.3)
  put("m.router", rng.standard_normal((experts + identity, width)))
  # corrections large enough to change who is chosen, but not the weights
  put("m.correction", rng.standard_normal(experts + identity) * 0.2)
  put("m.shared.sg", rng.standard_normal((1, width)) * 0.3)
  x, x64 = held(rng.standard_normal((rows, width)), dtype, device)
  chosen64, weight64 = plain.route(x64, mlp, w64, "m")
  chosen, weight, gate = ops.route_tokens(x, w["m.router"].float().contiguous(), w["m.correction"].float().contiguous(),
                                          w["m.shared.sg"].float().reshape(-1).contiguous(), top=top, scale=1.3)
  plain_scores = np.exp(x64 @ w64["m.router"].T)
  assert not np.array_equal(np.sort(np.argsort(-plain_scores, axis=-1)[:, :top], axis=-1), np.sort(chosen64, axis=-1)) or top == experts + identity, \
      "the corrections never changed a choice: the test's weights are too weak"
  assert np.array_equal(chosen.cpu().numpy(), chosen64), "the chosen experts differ"
  close(weight.cpu().numpy(), weight64, torch.float32, "weights", f32=1e-4)
  close(gate.cpu().numpy(), plain.sigmoid(x64 @ w64["m.shared.sg"].T)[:, 0], torch.float32, "shared gate", f32=1e-4)
  gate_up = torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(experts)]).contiguous()
  down = torch.stack([w[f"m.e{e}.down"] for e in range(experts)]).contiguous()
  shared, shared64 = held(rng.standard_normal((rows, width)), dtype, device)
  got = ops.mix_experts(x, chosen, weight, gate_up, down, experts, 1, shared, gate).float().cpu().numpy()
  want = np.zeros((rows, width))
  for t in range(rows):
    for e, a in zip(chosen64[t], weight64[t]):
      want[t] += a * (plain.silu_expert(x64[t:t + 1], w64, f"m.e{e}")[0] if e < experts else x64[t])
  want += plain.sigmoid(x64 @ w64["m.shared.sg"].T) * shared64
  close(got, want, dtype, f"experts {sizes}", f32=3e-5, bf16=3e-2)
  if hasattr(ops, "expert_rows_for_dense_products"):
    # both ways of multiplying: expert by expert through the dense products, and the grouped kernel
    for threshold in (0, 1):
      ops.expert_rows_for_dense_products = threshold
      got = ops.mix_experts(x, chosen, weight, gate_up, down, experts, 1, shared, gate).float().cpu().numpy()
      close(got, want, dtype, f"experts {sizes}, threshold {threshold}", f32=3e-5, bf16=3e-2)
    ops.check_errors()
  # a step of one token and of three: tiles that are mostly empty
  for n in (1, 3):
    got = ops.mix_experts(x[:n].contiguous(), chosen[:n].contiguous(), weight[:n].contiguous(), gate_up, down, experts, 1,
                          shared[:n].contiguous(), gate[:n].contiguous()).float().cpu().numpy()
    close(got, want[:n], dtype, f"experts {sizes}, {n} token(s)", f32=3e-5, bf16=3e-2)


# ---- one-layer models through the engine: each mixer and feed-forward alone ------------------------------

def one_layer_cases():
  return {
      "attention alone": sx.config([sx.attention()], [None]),
      "attention, no rotation, no cap": sx.config([sx.attention(dims=0, softcap=0.0)], [None], mult=1.0),
      "recurrence alone": sx.config([sx.hgrn2()], [None]),
      "dense": sx.config([sx.hgrn2(heads=1, dim=8, vdim=8)], [sx.dense()]),
      "experts": sx.config([sx.hgrn2(heads=1, dim=8, vdim=8)], [sx.moe()]),
      "experts, all identity but one": sx.config([sx.hgrn2(heads=1, dim=8, vdim=8)], [sx.moe(experts=1, identity=4, top=2, shared=0)]),
      "one layer five times": sx.config([sx.attention()], [sx.dense(ff=16)], loop=(0, 1, 5)),
  }


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("case", list(one_layer_cases()))
def test_one_layer_models(case, where):
  cfg_dict = one_layer_cases()[case]
  dtype, device = where
  cfg, t = sx.weights(cfg_dict, seed=8)
  ops = ReferenceOps(torch.float32) if device == "cpu" else None
  engine = sx.build_engine(cfg, t, dtype, device, ops)
  toks = np.random.default_rng(5).integers(0, cfg_dict["vocab"], 37).tolist()
  trace = []
  want = plain.forward(cfg_dict, sx.as_numpy(t), toks, trace=trace)
  for cuts in ([37], [20] + [1] * 17, sx.cuts_of(37, [2, 9, 3])):
    sx.check_close(sx.run_cuts(engine, toks, cuts), want, dtype, f"{case}, cuts {cuts[:3]}")
  # the stream after every layer call
  slot = engine.open_request()
  ctx = engine._prepare([StepEntry(slot, toks, ())])
  ctx.memo["layer_outputs"] = outs = []
  engine.model.forward(ctx, engine.caches)
  engine.close_request(slot)
  assert len(outs) == len(trace)
  for i, (g, x) in enumerate(zip(outs, trace)):
    close(g.float().cpu().numpy(), x, torch.float32 if dtype == "float32" else torch.bfloat16, f"{case}: stream after call {i}",
          f32=3e-5, bf16=5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [1, 8, 20, 40, 130, 300])
@pytest.mark.parametrize("hidden,width", [(128, 64), (256, 320), (40, 24)])
def test_the_clamped_gated_product_at_every_batch_size(rows, hidden, width, dtype):
  """The product with the clamped activation on its sums: every kernel that serves some number of
  rows (a handful, a serving batch, a prompt) against the plain statement."""
  ops, dt = table((dtype, "cuda"))
  rng = np.random.default_rng(rows + hidden)
  x, x64 = held(rng.standard_normal((rows, width)), dt, "cuda")
  w, w64 = held(rng.standard_normal((2 * hidden, width)) * 0.5, dt, "cuda")
  got = ops.gated_linear(x, w, 3, limit=1.1).float().cpu().numpy()
  gu = x64 @ w64.T
  if dt == torch.bfloat16:  # the projections are held in the storage type before the activation
    gu = torch.from_numpy(gu).to(torch.bfloat16).double().numpy()
  g, u = np.minimum(gu[:, :hidden], 1.1), np.clip(gu[:, hidden:], -1.1, 1.1)
  close(got, g * plain.sigmoid(1.702 * g) * (u + 1.0), dt, f"{rows} rows")
