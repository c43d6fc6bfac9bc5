"""A recurrent mixer whose forget gate also decides what is written (HGRN2).

Per head a matrix S [head_dim, value_dim] (float32, zero at a request's start, one per request
in a state slot) that every token updates and then reads:

  q_t = silu(W_q y_t)                                  [heads, head_dim]
  v_t = W_v y_t                                        [heads, value_dim]
  f_t = l + (1 - l) * sigmoid(W_f y_t + b)             [heads, head_dim], l the learned lower bound
  S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T
  o_t = S_t^T q_t

Each head's o is divided by its root mean square over value_dim and scaled per channel (one scale
for all heads); the heads side by side are projected by W_o.  q, f and v come out of one fused
product; everything between it and the output projection is float32.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import SlotStateNeed
from simply_b200.parts.base import Mixer
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.registry import MIXERS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"q": "q", "f": "f", "v": "v", "o": "o", "bias": "f.b", "lower": "lower", "norm": "norm"}


@MIXERS.register("forget_gate_recurrence")
class ForgetGateRecurrence(Mixer):

  graph_safe = True  # reads the step's device tensors only; rows that repeat a slot do not write its state

  def __init__(self, prefix: str, width: int, num_heads: int, head_dim: int, value_dim: int, eps: float,
               names: dict[str, str] | None = None):
    self.prefix, self.width = prefix, width
    self.num_heads, self.head_dim, self.value_dim = num_heads, head_dim, value_dim
    self.eps = float(eps)
    n = self.names = {**_NAMES, **(names or {})}
    self.q_proj = Linear(f"{prefix}.{n['q']}", num_heads * head_dim, width)
    self.f_proj = Linear(f"{prefix}.{n['f']}", num_heads * head_dim, width)
    self.v_proj = Linear(f"{prefix}.{n['v']}", num_heads * value_dim, width)
    self.o_proj = Linear(f"{prefix}.{n['o']}", width, num_heads * value_dim)
    self.in_weight = self.bias = self.lower = self.norm_weight = None

  def _name(self, role: str) -> str:
    return f"{self.prefix}.{self.names[role]}"

  def cache_need(self):
    return SlotStateNeed((self.num_heads, self.head_dim, self.value_dim), "float32")

  def tensor_specs(self) -> list[TensorSpec]:
    qk = self.num_heads * self.head_dim
    return [self.q_proj.spec(), self.f_proj.spec(), self.v_proj.spec(), self.o_proj.spec(),
            TensorSpec(self._name("bias"), (qk,), "scale", precision="stored"),
            TensorSpec(self._name("lower"), (qk,), "scale", precision="stored"),
            TensorSpec(self._name("norm"), (self.value_dim,), "gain")]

  def bind(self, tensors, ops) -> None:
    w = fuse_rows([tensors[p.name] for p in (self.q_proj, self.f_proj, self.v_proj)])
    extra = -w.shape[0] % 8
    self.in_weight = torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous() if extra else w
    self.o_proj.bind(tensors)
    self.bias = tensors[self._name("bias")].float().contiguous()
    self.lower = tensors[self._name("lower")].float().contiguous()
    self.norm_weight = tensors[self._name("norm")].float().contiguous()

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    ops = ctx.ops
    pre = ops.linear(x, self.in_weight)  # q | f | v, before activations
    o = ops.forget_gate_scan(pre, self.bias, self.lower, cache.storage, ctx, num_heads=self.num_heads,
                             head_dim=self.head_dim, value_dim=self.value_dim)
    y = ops.gated_head_norm(o, None, -1, self.norm_weight, self.eps, self.num_heads, self.value_dim)
    return self.o_proj(y, ctx)
