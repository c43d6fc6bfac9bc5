"""Plain, slow NumPy statement of the Sapivik decoder: the yardstick of its tests.

Whole sequences, no cache, one function per mechanism, float64 unless told otherwise.  It shares
no code with the engine and takes a config dictionary (config.json's contents) and a dictionary
of NumPy weights by tensor name.

Notation.  x is the residual stream [T, width]; e is x as the embedding leaves it.  A layer is

  x += m * rms(mixer(rms(x) w1)) w1b          m = residual_mult
  x += m * rms(ff(rms(x) w2)) w2b             (only if the layer has a feed-forward)

The layers `loop.start .. loop.stop - 1` run `loop.times` times in a row with the same weights
(a memory of its own per pass); before every pass but the first, x += e.  Mixers:

* `attention`: q = W_q y, k = W_k y, the values are k as projected.  The first `rot.dims` dims of
  every q and k head turn by p f_i, f_i = base^(-2i/dims), dims 2i and 2i+1 forming pair i; then
  every head is divided by its root mean square.  score = cap tanh(q.k scale / cap), causal
  softmax, heads side by side times sigmoid(W_g y), then W_o.
* `hgrn2`: per head a matrix S [dim, vdim], S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,
  o_t = S_t^T q_t with q = silu(W_q y), v = W_v y, f = l + (1 - l) sigmoid(W_f y + b); each o is
  RMS-normed over vdim with one scale, heads side by side, then W_o.

Feed-forwards: `dense` with a clamped gate, and `moe` with a softmax router whose choice (not
its weights) is shifted by a per-expert number, identity experts, and a gated shared expert.
"""

from __future__ import annotations

import numpy as np


def rms_norm(x, w, eps):
  y = x / np.sqrt(np.mean(np.square(x), axis=-1, keepdims=True) + eps)
  return y if w is None else y * w


def sigmoid(z):
  return 1.0 / (1.0 + np.exp(-z))


def silu(z):
  return z * sigmoid(z)


def turn_neighbours(x, positions, dims, base):
  """x [T, heads, n]: dims 2i, 2i+1 (i < dims/2) of every head turn by p * base^(-2i/dims)."""
  out = np.array(x, dtype=np.float64, copy=True)
  if not dims:
    return out
  freq = np.power(float(base), -2.0 * np.arange(dims // 2) / dims)
  angle = np.asarray(positions, np.float64)[:, None, None] * freq[None, None, :]
  c, s = np.cos(angle), np.sin(angle)
  a, b = x[..., 0:dims:2], x[..., 1:dims:2]
  out[..., 0:dims:2] = a * c - b * s
  out[..., 1:dims:2] = b * c + a * s
  return out


def capped_causal_attention(q, k, v, scale, cap):
  """q [T, H, d], k [T, G, d], v [T, G, dv]: every query sees itself and all before it."""
  t, h, _ = q.shape
  group = h // k.shape[1]
  mask = np.arange(t)[None, :] <= np.arange(t)[:, None]
  out = np.zeros((t, h, v.shape[-1]))
  for n in range(h):
    s = q[:, n] @ k[:, n // group].T * scale
    if cap:
      s = cap * np.tanh(s / cap)
    s = np.where(mask, s, -np.inf)
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    out[:, n] = (p / p.sum(axis=-1, keepdims=True)) @ v[:, n // group]
  return out


def attention_mixer(y, positions, m, w, p, eps):
  """m: the mixer's config entry; w: weights by name; p: the tensors' prefix ('l0.mix')."""
  t = y.shape[0]
  heads, kv_heads, dim = m["heads"], m["kv_heads"], m["dim"]
  q = (y @ w[f"{p}.q"].T).reshape(t, heads, dim)
  k = (y @ w[f"{p}.k"].T).reshape(t, kv_heads, dim)
  v = k
  rot = m.get("rot") or {}
  q = turn_neighbours(q, positions, rot.get("dims", 0), rot.get("base", 1.0))
  k = turn_neighbours(k, positions, rot.get("dims", 0), rot.get("base", 1.0))
  q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
  o = capped_causal_attention(q, k, v, m["scale"], m.get("softcap") or 0.0).reshape(t, -1)
  o = o * sigmoid(y @ w[f"{p}.g"].T)
  return o @ w[f"{p}.o"].T


def forget_gate_scan(q, f, v, state=None):
  """q, f [T, H, d], v [T, H, dv]: S = diag(f) S + (1 - f) v^T, o = S^T q.  Returns (o, last S)."""
  t, h, d = q.shape
  s = np.zeros((h, d, v.shape[-1])) if state is None else np.array(state, dtype=np.float64)
  out = np.zeros((t, h, v.shape[-1]))
  for i in range(t):
    s = f[i][:, :, None] * s + (1.0 - f[i])[:, :, None] * v[i][:, None, :]
    out[i] = np.einsum("hdv,hd->hv", s, q[i])
  return out, s


def hgrn2_mixer(y, m, w, p, eps):
  t = y.shape[0]
  heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
  q = silu(y @ w[f"{p}.q"].T).reshape(t, heads, dim)
  v = (y @ w[f"{p}.v"].T).reshape(t, heads, vdim)
  low = w[f"{p}.lower"]
  f = (low + (1.0 - low) * sigmoid(y @ w[f"{p}.f"].T + w[f"{p}.f.b"])).reshape(t, heads, dim)
  o, _ = forget_gate_scan(q, f, v)
  o = rms_norm(o, w[f"{p}.norm"], eps).reshape(t, -1)
  return o @ w[f"{p}.o"].T


def clamped_dense(y, mlp, w, p):
  limit = mlp["limit"]
  g = np.minimum(y @ w[f"{p}.gate"].T, limit)
  u = np.clip(y @ w[f"{p}.up"].T, -limit, limit)
  return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[f"{p}.down"].T


def silu_expert(y, w, p):
  return (silu(y @ w[f"{p}.gate"].T) * (y @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def route(y, mlp, w, p):
  """Chosen experts [T, top] and their weights [T, top]."""
  r = mlp["router"]
  z = y @ w[f"{p}.router"].T
  e = np.exp(z - z.max(axis=-1, keepdims=True))
  s = e / e.sum(axis=-1, keepdims=True)
  choice = s + w[f"{p}.correction"]
  chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :r["top"]]
  return chosen, np.take_along_axis(s, chosen, axis=-1) * r["scale"]


def moe(y, mlp, w, p):
  r = mlp["router"]
  real = r["experts"]
  chosen, weight = route(y, mlp, w, p)
  out = np.zeros((y.shape[0], w[f"{p}.e0.down"].shape[0]) if real else y.shape)
  for t in range(y.shape[0]):
    for e, a in zip(chosen[t], weight[t]):
      row = y[t:t + 1]
      out[t] += a * (silu_expert(row, w, f"{p}.e{e}")[0] if e < real else row[0])
  if mlp.get("shared"):
    out = out + sigmoid(y @ w[f"{p}.shared.sg"].T) * silu_expert(y, w, f"{p}.shared")
  return out


def run_order(cfg):
  """[(layer index, first of a repeated pass)] in the order the layers run."""
  n = len(cfg["layers"])
  loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
  start, stop, times = loop["start"], loop["stop"], loop["times"]
  order = [(i, False) for i in range(start)]
  for rep in range(times):
    order += [(i, rep > 0 and i == start) for i in range(start, stop)]
  return order + [(i, False) for i in range(stop, n)]


def forward(cfg, w, tokens, dtype=np.float64, trace=None):
  """Logits [T, vocab] of one sequence; `trace` (a list) receives x after every layer run."""
  w = {k: np.asarray(v, dtype=dtype) for k, v in w.items()}
  eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
  tokens = np.asarray(tokens)
  positions = np.arange(len(tokens))
  x = w["embed"][tokens]
  first = x.copy()
  for i, again in run_order(cfg):
    layer, p = cfg["layers"][i], f"l{i}"
    if again:
      x = x + first
    y = rms_norm(x, w[f"{p}.norm1"], eps)
    if layer["type"] == "attention":
      z = attention_mixer(y, positions, layer["mixer"], w, f"{p}.mix", eps)
    else:
      z = hgrn2_mixer(y, layer["mixer"], w, f"{p}.mix", eps)
    x = x + mult * rms_norm(z, w[f"{p}.norm1b"], eps)
    mlp = layer.get("mlp")
    if mlp:
      y = rms_norm(x, w[f"{p}.norm2"], eps)
      z = clamped_dense(y, mlp, w, f"{p}.mlp") if mlp["kind"] == "dense" else moe(y, mlp, w, f"{p}.mlp")
      x = x + mult * rms_norm(z, w[f"{p}.norm2b"], eps)
    if trace is not None:
      trace.append(x.copy())
  return rms_norm(x, w["final.norm"], eps) @ w["head"].T
