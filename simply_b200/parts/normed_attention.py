"""Grouped-query attention with normed queries and keys over the paged cache.

Beside `paged_attention` (parts/attention.py) for designs whose attention differs from it in
any of these, each switched by a parameter:

* q and k are RMS-normed over their *whole* projection (all heads at once, one scale per
  channel, applied as it is) before they are split into heads;
* rotary positions on the first `rotary["dims"]` dims of every q and k head (pairs i, i + dims/2;
  angle p * base^(-2i/dims) / factor), or none;
* `rotate_values`: a value head at position j is turned over all its dims by
  j * base^(-2m/value_dim) before it is cached, and a head's result at position i is turned
  back by i's angles, so that what is summed depends on i - j only;
* key and value heads of different sizes (`head_dim`, `value_dim`);
* score = q.k * score_scale, times a learned number per head (`head_temperature`);
* a window of `window` keys (the query's own included), and with `pool` = P also one key and
  value per whole block of P tokens that has left the window: block b (tokens bP .. bP + P - 1) is
  seen from position i when bP + P - 1 <= i - window, as the mean of its keys and of its values
  as the cache holds them; tokens and blocks share one softmax.  The block means live in a
  second paged cache with one entry per P tokens, which keeps every block;
* `project_kv=False`: the layer has no k/v tensors and reads the cache another layer writes.

The cache of a layer with a window keeps `cache_window` tokens (at least the window and a
block's length, so that a block's tokens are still there when its last one arrives; more if
another layer reads the cache through a wider window).
"""

from __future__ import annotations

from typing import Any

import numpy as np
import torch

from simply_b200.cache.needs import PagedKVNeed
from simply_b200.parts.base import Mixer
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.registry import MIXERS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "temp": "temp"}


def rotation_frequencies(dims: int, base: float, factor: float = 1.0) -> np.ndarray:
  """float32 [dims / 2]: base^(-2i/dims) / factor."""
  i = np.arange(dims // 2, dtype=np.float64)
  return (np.power(float(base), -2.0 * i / dims) / float(factor)).astype(np.float32)


@MIXERS.register("qk_norm_attention")
class QKNormAttention(Mixer):

  graph_safe = True

  def __init__(self, prefix: str, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
               score_scale: float, eps: float, value_dim: int | None = None, window: int | None = None,
               pool: int | None = None, rotary: dict | None = None, rotate_values: bool = False,
               head_temperature: bool = False, project_kv: bool = True, cache_window: int | None = None,
               names: dict[str, str] | None = None):
    if num_heads % num_kv_heads:
      raise ValueError(f"{prefix}: num_heads {num_heads} is no multiple of num_kv_heads {num_kv_heads}")
    if pool is not None and (window is None or pool <= 0):
      raise ValueError(f"{prefix}: pooled blocks need a window and a positive block length")
    self.prefix = prefix
    self.width = width
    self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
    self.head_dim = head_dim
    self.value_dim = head_dim if value_dim is None else value_dim
    self.score_scale = float(score_scale)
    self.eps = float(eps)
    self.window, self.pool = window, pool
    self.rotary = dict(rotary) if rotary else None
    self.rotate_values = bool(rotate_values)
    if self.rotary and (self.rotary["dims"] % 2 or self.rotary["dims"] > head_dim):
      raise ValueError(f"{prefix}: {self.rotary['dims']} rotated dims do not fit a head of {head_dim}")
    if self.rotate_values and (not self.rotary or self.value_dim % 2):
      raise ValueError(f"{prefix}: rotated values need a rotation base and an even value size")
    self.head_temperature = bool(head_temperature)
    self.project_kv = project_kv
    keep = None if window is None else max(window, pool or 0, cache_window or 0)
    self.cache_window = keep
    n = {**_NAMES, **(names or {})}
    self.q_proj = Linear(f"{prefix}.{n['q']}", num_heads * head_dim, width)
    self.k_proj = Linear(f"{prefix}.{n['k']}", num_kv_heads * head_dim, width)
    self.v_proj = Linear(f"{prefix}.{n['v']}", num_kv_heads * self.value_dim, width)
    self.o_proj = Linear(f"{prefix}.{n['o']}", width, num_heads * self.value_dim)
    self.q_norm_name, self.k_norm_name = f"{prefix}.{n['q_norm']}", f"{prefix}.{n['k_norm']}"
    self.temp_name = f"{prefix}.{n['temp']}"
    self.qkv_weight = self.q_norm = self.k_norm = self.head_scale = None
    self.rot_freq = self.value_freq = None

  # ---- cache ------------------------------------------------------------------
  def cache_need(self):
    value_dim = None if self.value_dim == self.head_dim else self.value_dim
    kv = PagedKVNeed(self.num_kv_heads, self.head_dim, self.cache_window if self.project_kv else self.window,
                     value_dim=value_dim)
    if self.pool is None:
      return kv
    return {"kv": kv, "pool": PagedKVNeed(self.num_kv_heads, self.head_dim, None, value_dim=value_dim,
                                          stride=self.pool)}

  def graph_plans(self, ops, batch: int, bucket: int, max_burst: int, page_size: int) -> list:
    if self.pool is not None:
      plan = ops.pooled_attention_graph_plan(
          window=self.window, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
          value_dim=self.value_dim, pool=self.pool, batch=batch, page_size=page_size)
      return [plan] if plan is not None else []
    if self.value_dim != self.head_dim:
      return []
    plan = ops.attention_graph_plan(
        window=self.window, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
        batch=batch, bucket=bucket, max_burst=max_burst, page_size=page_size)
    return [plan] if plan is not None else []

  # ---- weights ----------------------------------------------------------------
  def tensor_specs(self) -> list[TensorSpec]:
    specs = [self.q_proj.spec(), TensorSpec(self.q_norm_name, (self.num_heads * self.head_dim,), "gain")]
    if self.project_kv:
      specs += [self.k_proj.spec(), self.v_proj.spec(),
                TensorSpec(self.k_norm_name, (self.num_kv_heads * self.head_dim,), "gain")]
    if self.head_temperature:
      specs.append(TensorSpec(self.temp_name, (self.num_heads,), "gain"))
    return specs + [self.o_proj.spec()]

  def bind(self, tensors, ops) -> None:
    if self.head_dim % 2 == 0:  # (odd head sizes run on the general kernel, which takes any)
      ops.check_attention(self.head_dim, self.num_heads, self.num_kv_heads)
    names = [self.q_proj.name] + ([self.k_proj.name, self.v_proj.name] if self.project_kv else [])
    qkv = fuse_rows([tensors[n] for n in names])
    extra = -qkv.shape[0] % 8  # whole 16-byte groups of output features for the products' stores
    self.qkv_weight = torch.cat([qkv, qkv.new_zeros(extra, qkv.shape[1])]).contiguous() if extra else qkv
    self.o_proj.bind(tensors)
    self.q_norm = tensors[self.q_norm_name].float().contiguous()
    self.k_norm = tensors[self.k_norm_name].float().contiguous() if self.project_kv else None
    device = self.q_norm.device
    scale = torch.full((self.num_heads,), self.score_scale, dtype=torch.float32, device=device)
    if self.head_temperature:
      scale = scale * tensors[self.temp_name].float()
    self.head_scale = scale.contiguous()
    if self.rotary:
      freq = rotation_frequencies(self.rotary["dims"], self.rotary["base"], self.rotary.get("factor", 1.0))
      self.rot_freq = torch.from_numpy(freq).to(device)
      if self.rotate_values:
        self.value_freq = torch.from_numpy(rotation_frequencies(self.value_dim, self.rotary["base"])).to(device)

  # ---- forward ----------------------------------------------------------------
  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    ops = ctx.ops
    if writes_cache and not self.project_kv:
      raise ValueError(f"{self.prefix}: a mixer without k/v projections cannot write a cache")
    kv_cache = cache["kv"] if isinstance(cache, dict) else cache
    pool_cache = cache["pool"] if self.pool is not None else None
    block_table = ctx.block_tables[kv_cache.group]
    qkv = ops.linear(x, self.qkv_weight)
    q = ops.qk_norm_rotate_store(
        qkv, self.q_norm, self.k_norm, self.eps, self.head_scale, self.rot_freq, self.value_freq,
        self.num_heads, self.num_kv_heads if self.project_kv else 0, self.head_dim, self.value_dim,
        kv_cache.storage if writes_cache else None, block_table, ctx)
    pooled = None
    if pool_cache is not None:
      pool_table = ctx.block_tables[pool_cache.group]
      if writes_cache:
        ops.pool_blocks(kv_cache.storage, block_table, pool_cache.storage, pool_table, ctx,
                        self.num_kv_heads, self.head_dim, self.value_dim, self.pool)
      pooled = (pool_cache.storage, pool_table, self.pool)
    o = ops.paged_attention(
        q, kv_cache.storage, block_table, ctx, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
        head_dim=self.head_dim, logit_softcap=0.0, window=self.window, value_dim=self.value_dim, pooled=pooled)
    if self.rotate_values:
      o = ops.rotate_heads(o, ctx.positions, self.value_freq, self.num_heads, self.value_dim, inverse=True)
    return self.o_proj(o, ctx)
