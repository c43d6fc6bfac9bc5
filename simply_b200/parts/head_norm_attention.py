"""Grouped-query attention whose heads are normed one by one, with tied values and an output gate.

Beside `paged_attention` and `qk_norm_attention` for designs whose attention differs from them in
any of these, each switched by a parameter:

* rotary positions on the first `rotary["dims"]` dims of every q and k head, pairing neighbours
  (2i, 2i + 1) (`layout` "neighbours") or halves (i, i + dims/2) (`layout` "halves"), angle
  p * base^(-2i/dims);
* `head_norm`: after the rotation every q and k head is divided by its own root mean square
  (over head_dim, eps inside the root, no scale);
* `tie_values`: there is no value projection: a key head as projected (before rotation and
  norm) is also the value head;
* score = q.k * score_scale, then `score_softcap` * tanh(score / score_softcap) before the softmax;
* causal, optionally over a window of `window` keys;
* `output_gate`: the heads side by side are multiplied by sigmoid(W_g y) before the output
  projection; the gate reads the mixer's input, like q and k.

q, k, (v) and the gate come out of one fused product.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import PagedKVNeed
from simply_b200.parts.base import Mixer
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.parts.normed_attention import rotation_frequencies
from simply_b200.registry import MIXERS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}


@MIXERS.register("head_norm_attention")
class HeadNormAttention(Mixer):

  graph_safe = True

  def __init__(self, prefix: str, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
               score_scale: float, eps: float, score_softcap: float = 0.0, window: int | None = None,
               rotary: dict | None = None, head_norm: bool = True, tie_values: bool = True,
               output_gate: bool = True, names: dict[str, str] | None = None):
    if num_heads % num_kv_heads:
      raise ValueError(f"{prefix}: num_heads {num_heads} is no multiple of num_kv_heads {num_kv_heads}")
    self.prefix, self.width = prefix, width
    self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
    self.score_scale, self.eps = float(score_scale), float(eps)
    self.score_softcap = float(score_softcap or 0.0)
    self.window = window
    self.rotary = dict(rotary) if rotary else None
    if self.rotary:
      if self.rotary["dims"] % 2 or self.rotary["dims"] > head_dim:
        raise ValueError(f"{prefix}: {self.rotary['dims']} rotated dims do not fit a head of {head_dim}")
      if self.rotary.get("layout", "neighbours") not in ("neighbours", "halves"):
        raise ValueError(f"{prefix}: rotary layout must be 'neighbours' or 'halves'")
    self.head_norm, self.tie_values, self.output_gate = bool(head_norm), bool(tie_values), bool(output_gate)
    n = {**_NAMES, **(names or {})}
    self.q_proj = Linear(f"{prefix}.{n['q']}", num_heads * head_dim, width)
    self.k_proj = Linear(f"{prefix}.{n['k']}", num_kv_heads * head_dim, width)
    self.v_proj = None if self.tie_values else Linear(f"{prefix}.{n['v']}", num_kv_heads * head_dim, width)
    self.g_proj = Linear(f"{prefix}.{n['g']}", num_heads * head_dim, width) if self.output_gate else None
    self.o_proj = Linear(f"{prefix}.{n['o']}", width, num_heads * head_dim)
    self.in_weight = self.rot_freq = None
    self.gate_offset = 0

  def _inputs(self) -> list[Linear]:
    return [p for p in (self.q_proj, self.k_proj, self.v_proj, self.g_proj) if p is not None]

  def cache_need(self):
    return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window)

  def graph_plans(self, ops, batch: int, bucket: int, max_burst: int, page_size: int) -> list:
    plan = ops.attention_graph_plan(
        window=self.window, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
        batch=batch, bucket=bucket, max_burst=max_burst, page_size=page_size)
    return [plan] if plan is not None else []

  def tensor_specs(self) -> list[TensorSpec]:
    return [p.spec() for p in self._inputs()] + [self.o_proj.spec()]

  def bind(self, tensors, ops) -> None:
    if self.head_dim % 2 == 0:  # (odd head sizes run on the general kernel, which takes any)
      ops.check_attention(self.head_dim, self.num_heads, self.num_kv_heads)
    w = fuse_rows([tensors[p.name] for p in self._inputs()])
    extra = -w.shape[0] % 8  # whole 16-byte groups of output features for the products' stores
    self.in_weight = torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous() if extra else w
    self.gate_offset = sum(p.out_features for p in self._inputs()[:-1]) if self.output_gate else 0
    self.o_proj.bind(tensors)
    if self.rotary:
      freq = rotation_frequencies(self.rotary["dims"], self.rotary["base"])
      self.rot_freq = torch.from_numpy(freq).to(self.in_weight.device)

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    ops = ctx.ops
    block_table = ctx.block_tables[cache.group]
    proj = ops.linear(x, self.in_weight)  # q | k | (v) | (gate)
    q = ops.rotate_headnorm_store(
        proj, self.eps, self.score_scale, self.rot_freq,
        interleaved=bool(self.rotary) and self.rotary.get("layout", "neighbours") == "neighbours",
        head_norm=self.head_norm, tie_values=self.tie_values, num_heads=self.num_heads,
        num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
        storage=cache.storage if writes_cache else None, block_table=block_table, ctx=ctx)
    o = ops.paged_attention(
        q, cache.storage, block_table, ctx, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
        head_dim=self.head_dim, logit_softcap=self.score_softcap, window=self.window)
    if self.output_gate:
      o = ops.sigmoid_gate(o, proj, self.gate_offset)
    return self.o_proj(o, ctx)
