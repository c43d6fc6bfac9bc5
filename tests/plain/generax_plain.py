"""Plain, slow NumPy statement of the Generax decoder: the yardstick of its tests.

Whole sequences, no cache, one function per mechanism, float64 unless told otherwise.  It shares
no code with the engine and takes a config dictionary (config.json's contents) and a dictionary
of NumPy weights by tensor name.

Notation.  A layer reads y = rms(x) once and adds mixer(y) + feed_forward(y) to x.  Mixers:

* `attention`: q, k, v = W y; q and k are normed over their whole rows (all heads at once);
  the first `rot.dims` dims of every q and k head turn by angle p f_i / factor (pairs i,
  i + dims/2, f_i = base^(-2i/dims)); every value head turns by p base^(-2m/vdim) over all its
  dims before it is kept, and a head's result at position p turns back by the same angle;
  scores are q.k * scale * temp[head]; a query at p sees the keys p - size + 1 .. p.
* `parallel`: half of rms(left) * w_left + rms(right) * w_right, where left is attention
  without rotation whose queries see their window and, in front of it, one mean key/value per
  whole block of `pool` tokens that has left the window, and right is the gated delta rule.
"""

from __future__ import annotations

import numpy as np


def rms_norm(x, w, eps):
  return x / np.sqrt(np.mean(np.square(x), axis=-1, keepdims=True) + eps) * w


def silu(z):
  return z / (1.0 + np.exp(-z))


def sigmoid(z):
  return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
  return np.logaddexp(0.0, z)


def turn_pairs(x, angle):
  """x [..., n], angle [..., n/2]: pair (i, i + n/2) turns by angle i."""
  half = x.shape[-1] // 2
  a, b = x[..., :half], x[..., half:]
  c, s = np.cos(angle), np.sin(angle)
  return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def rotary(x, positions, dims, base, factor=1.0):
  """x [T, heads, n]: the first `dims` dims of every head turn, the rest pass."""
  if dims == 0:
    return x
  freq = np.power(float(base), -2.0 * np.arange(dims // 2) / dims) / factor
  angle = np.asarray(positions, np.float64)[:, None, None] * freq[None, None, :]
  return np.concatenate([turn_pairs(x[..., :dims], angle), x[..., dims:]], axis=-1)


def softmax_rows(s, mask):
  s = np.where(mask, s, -np.inf)
  s = s - s.max(axis=-1, keepdims=True)
  e = np.exp(s)
  return e / e.sum(axis=-1, keepdims=True)


def window_attention(q, k, v, head_scale, size):
  """q [T, H, d], k [T, G, d], v [T, G, dv], head_scale [H]; size None sees everything before."""
  t, h, _ = q.shape
  group = h // k.shape[1]
  i, j = np.arange(t)[:, None], np.arange(t)[None, :]
  mask = (j <= i) if size is None else ((i - j >= 0) & (i - j < size))
  out = np.zeros((t, h, v.shape[-1]))
  for n in range(h):
    s = q[:, n] @ k[:, n // group].T * head_scale[n]
    out[:, n] = softmax_rows(s, mask) @ v[:, n // group]
  return out


def pooled_window_attention(q, k, v, head_scale, size, pool):
  """As `window_attention`, and position i also sees block b (the mean key and value of tokens
  b*pool .. b*pool + pool - 1) when b*pool + pool - 1 <= i - size."""
  t, h, _ = q.shape
  g = k.shape[1]
  group = h // g
  nb = t // pool
  kb = k[:nb * pool].reshape(nb, pool, g, k.shape[-1]).sum(axis=1) / pool
  vb = v[:nb * pool].reshape(nb, pool, g, v.shape[-1]).sum(axis=1) / pool
  i, j = np.arange(t)[:, None], np.arange(t)[None, :]
  mask_tokens = (i - j >= 0) & (i - j < size)
  b = np.arange(nb)[None, :]
  mask_blocks = b * pool + pool - 1 <= i - size
  mask = np.concatenate([mask_blocks, mask_tokens], axis=1)
  out = np.zeros((t, h, v.shape[-1]))
  for n in range(h):
    m = n // group
    s = np.concatenate([q[:, n] @ kb[:, m].T, q[:, n] @ k[:, m].T], axis=1) * head_scale[n]
    out[:, n] = softmax_rows(s, mask) @ np.concatenate([vb[:, m], v[:, m]], axis=0)
  return out


def short_conv(x, w):
  """x [T, C], w [C, taps]: y[t] = sum_j w[:, j] * x[t - (taps - 1) + j], zeros before the start."""
  taps = w.shape[1]
  padded = np.concatenate([np.zeros((taps - 1, x.shape[1])), x], axis=0)
  return sum(padded[j:j + x.shape[0]] * w[:, j][None, :] for j in range(taps))


def gated_delta_rule(q, k, v, beta, decay):
  """q, k [T, H, d] (already per value head), v [T, H, dv], beta [T, H], decay [T, H, d].
  Per head, with S [d, dv] starting at zero: S = decay * S (rows); u = beta (v - S^T k);
  S = S + k u^T; o = S^T q."""
  t, h, d = q.shape
  dv = v.shape[-1]
  out = np.zeros((t, h, dv))
  for n in range(h):
    s = np.zeros((d, dv))
    for i in range(t):
      s = decay[i, n][:, None] * s
      u = beta[i, n] * (v[i, n] - s.T @ k[i, n])
      s = s + np.outer(k[i, n], u)
      out[i, n] = s.T @ q[i, n]
  return out


def unit(x):
  return x / np.sqrt(np.sum(np.square(x), axis=-1, keepdims=True) + 1e-6)


# ----------------------------------------------------------------------------
# Mixers
# ----------------------------------------------------------------------------


def attention_keys_values(y, w, prefix, m, eps, positions):
  """What the layer's cache holds: normed, turned keys [T, G, d] and turned values [T, G, dv]."""
  t = y.shape[0]
  g, d, dv = m["kv_heads"], m["dim"], m["vdim"]
  k = rms_norm(y @ w[f"{prefix}.k"].T, w[f"{prefix}.k.norm"], eps).reshape(t, g, d)
  v = (y @ w[f"{prefix}.v"].T).reshape(t, g, dv)
  rot = m.get("rot")
  if rot:
    k = rotary(k, positions, rot["dims"], rot["base"], (rot.get("scaling") or {}).get("factor", 1.0))
    v = rotary(v, positions, dv, rot["base"])
  return k, v


def attention_mixer(y, w, prefix, m, eps, positions, kv=None):
  t = y.shape[0]
  h, d, dv = m["heads"], m["dim"], m["vdim"]
  q = rms_norm(y @ w[f"{prefix}.q"].T, w[f"{prefix}.q.norm"], eps).reshape(t, h, d)
  rot = m.get("rot")
  if rot:
    q = rotary(q, positions, rot["dims"], rot["base"], (rot.get("scaling") or {}).get("factor", 1.0))
  k, v = kv if kv is not None else attention_keys_values(y, w, prefix, m, eps, positions)
  temp = w[f"{prefix}.temp"] if f"{prefix}.temp" in w else np.ones(h)
  mask = m.get("mask") or {}
  if mask.get("pool"):
    o = pooled_window_attention(q, k, v, m["scale"] * temp, mask["size"], mask["pool"])
  else:
    o = window_attention(q, k, v, m["scale"] * temp, mask.get("size"))
  if rot:
    o = rotary(o, -np.asarray(positions, np.float64), dv, rot["base"])
  return o.reshape(t, h * dv) @ w[f"{prefix}.o"].T, (k, v)


def delta_mixer(y, w, prefix, m, eps):
  t = y.shape[0]
  h, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
  rep = h // g

  def conv_branch(name):
    return silu(short_conv(y @ w[f"{prefix}.{name}"].T, w[f"{prefix}.{name}.conv"]))

  q = unit(conv_branch("q").reshape(t, g, d)) * d ** -0.5
  k = unit(conv_branch("k").reshape(t, g, d))
  v = conv_branch("v").reshape(t, h, dv)
  q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)
  beta = sigmoid(y @ w[f"{prefix}.b"].T)
  a = (y @ w[f"{prefix}.a1"].T) @ w[f"{prefix}.a2"].T + w[f"{prefix}.dt_bias"]
  decay = np.exp(-np.exp(w[f"{prefix}.A_log"])[None, :, None] * softplus(a).reshape(t, h, d))
  o = gated_delta_rule(q, k, v, beta, decay)
  o = o / np.sqrt(np.mean(np.square(o), axis=-1, keepdims=True) + eps) * w[f"{prefix}.norm"]
  gate = sigmoid((y @ w[f"{prefix}.g1"].T) @ w[f"{prefix}.g2"].T).reshape(t, h, dv)
  return (o * gate).reshape(t, h * dv) @ w[f"{prefix}.o"].T


def parallel_mixer(y, w, prefix, m, eps, positions):
  left, _ = attention_mixer(y, w, f"{prefix}.left", m["left"], eps, positions)
  right = delta_mixer(y, w, f"{prefix}.right", m["right"], eps)
  return 0.5 * (rms_norm(left, w[f"{prefix}.left.out"], eps) + rms_norm(right, w[f"{prefix}.right.out"], eps))


def dense_feed_forward(y, w, prefix):
  return (silu(y @ w[f"{prefix}.gate"].T) * (y @ w[f"{prefix}.up"].T)) @ w[f"{prefix}.down"].T


# ----------------------------------------------------------------------------
# The model
# ----------------------------------------------------------------------------


def forward(config, weights, tokens, return_layers=False):
  """Logits [T, vocab] of one whole sequence (and the stream after every layer)."""
  w = {k: np.asarray(v, np.float64) for k, v in weights.items()}
  eps = config["norm"]["eps"]
  positions = np.arange(len(tokens))
  x = w["embed"][np.asarray(tokens, np.int64)]
  kept = {}
  after = []
  for i, layer in enumerate(config["layers"]):
    p = f"l{i}"
    y = rms_norm(x, w[f"{p}.norm1"], eps)
    m = layer["mixer"]
    if layer["type"] == "attention":
      source = m.get("kv_from")
      branch, kept[i] = attention_mixer(y, w, f"{p}.mix", m, eps, positions,
                                        kv=None if source is None else kept[source])
    elif layer["type"] == "parallel":
      branch = parallel_mixer(y, w, f"{p}.mix", m, eps, positions)
    else:
      raise ValueError(f"unknown layer type {layer['type']!r}")
    if layer.get("mlp"):
      branch = branch + dense_feed_forward(y, w, f"{p}.mlp")
    x = x + branch
    after.append(x)
  logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
  cap = config.get("logit_softcap")
  if cap:
    logits = cap * np.tanh(logits / cap)
  return (logits, np.stack(after)) if return_layers else logits
