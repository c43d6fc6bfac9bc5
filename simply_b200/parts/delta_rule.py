"""Recurrent mixers with a state of fixed size per request, and a mixer made of mixers.

`gated_delta_rule`: per value head a matrix S [head_dim, value_dim] (float32, zero at a request's
start) that every token updates and reads:

  S <- diag(g_t) S                      one decay per key channel, g = exp(-exp(A) softplus(a + dt))
  u  = beta_t (v_t - S^T k_t)           beta = sigmoid(W_b y)
  S <- S + k_t u^T
  o_t = S^T q_t                         (after the write)

q, k (num_kv_heads heads of head_dim; value head n uses q/k head n // (heads / kv_heads)) and v
pass a short causal convolution per channel and silu; q and k are then made unit vectors per
head (x / sqrt(sum x^2 + 1e-6)) and q is scaled by head_dim^-1/2.  a = W_a2 (W_a1 y) and the
output gate sigmoid(W_g2 (W_g1 y)) come through low ranks that only the tensors' shapes give.
Each head's o is divided by its root mean square, scaled per channel, gated, and projected.  The
state per request is S and the convolution's last taps - 1 inputs; everything between the
projections and the output projection is float32.

`normed_mean`: several mixers read the same input; the result is the mean of their outputs, each
RMS-normed over the model width with a scale of its own.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import SlotStateNeed
from simply_b200.config.model_spec import PartSpec
from simply_b200.parts.base import Mixer, build_part
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.registry import MIXERS
from simply_b200.weights.loader import TensorSpec

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "beta": "b", "decay_in": "a1", "decay_out": "a2",
          "gate_in": "g1", "gate_out": "g2", "decay_log": "A_log", "decay_bias": "dt_bias", "norm": "norm",
          "conv": "conv"}


def _pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
  extra = -w.shape[0] % multiple
  if not extra:
    return w.contiguous()
  return torch.cat([w, w.new_zeros(extra, w.shape[1])], dim=0).contiguous()


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule(Mixer):

  graph_safe = True  # reads the step's device tensors only; rows that repeat a slot do not write its state

  def __init__(self, prefix: str, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
               value_dim: int, conv_taps: int, eps: float, decay_rank: int = -1, gate_rank: int = -1,
               names: dict[str, str] | None = None):
    if num_heads % num_kv_heads:
      raise ValueError(f"{prefix}: num_heads {num_heads} is no multiple of num_kv_heads {num_kv_heads}")
    if conv_taps < 1:
      raise ValueError(f"{prefix}: a convolution needs at least one tap, got {conv_taps}")
    self.prefix, self.width = prefix, width
    self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
    self.head_dim, self.value_dim = head_dim, value_dim
    self.conv_taps = conv_taps
    self.eps = float(eps)
    self.decay_rank, self.gate_rank = decay_rank, gate_rank  # -1: the tensors' shapes give them
    n = self.names = {**_NAMES, **(names or {})}
    qk, vv = num_kv_heads * head_dim, num_heads * value_dim
    self.channels = 2 * qk + vv
    self.q_proj = Linear(f"{prefix}.{n['q']}", qk, width)
    self.k_proj = Linear(f"{prefix}.{n['k']}", qk, width)
    self.v_proj = Linear(f"{prefix}.{n['v']}", vv, width)
    self.beta_proj = Linear(f"{prefix}.{n['beta']}", num_heads, width)
    self.decay_in = Linear(f"{prefix}.{n['decay_in']}", decay_rank, width)
    self.decay_out = Linear(f"{prefix}.{n['decay_out']}", num_heads * head_dim, decay_rank)
    self.gate_in = Linear(f"{prefix}.{n['gate_in']}", gate_rank, width)
    self.gate_out = Linear(f"{prefix}.{n['gate_out']}", vv, gate_rank)
    self.o_proj = Linear(f"{prefix}.{n['o']}", width, vv)

  def _name(self, role: str) -> str:
    return f"{self.prefix}.{self.names[role]}"

  def cache_need(self):
    return {"conv": SlotStateNeed((self.conv_taps - 1, self.channels), "float32"),
            "state": SlotStateNeed((self.num_heads, self.head_dim, self.value_dim), "float32")}

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [p.spec() for p in (self.q_proj, self.k_proj, self.v_proj, self.beta_proj, self.decay_in,
                                self.decay_out, self.gate_in, self.gate_out, self.o_proj)]
    for p in (self.q_proj, self.k_proj, self.v_proj):
      specs.append(TensorSpec(f"{p.name}.{self.names['conv']}", (p.out_features, self.conv_taps), "matrix"))
    specs += [
        TensorSpec(self._name("decay_log"), (self.num_heads,), "scale", precision="stored"),
        TensorSpec(self._name("decay_bias"), (self.num_heads * self.head_dim,), "scale", precision="stored"),
        TensorSpec(self._name("norm"), (self.value_dim,), "gain"),
    ]
    return specs

  def bind(self, tensors, ops) -> None:
    t = tensors
    projections = [t[p.name] for p in (self.q_proj, self.k_proj, self.v_proj, self.beta_proj)]
    self.in_weight = _pad_rows(fuse_rows(projections))
    a1, g1 = t[self.decay_in.name], t[self.gate_in.name]
    a2, g2 = t[self.decay_out.name], t[self.gate_out.name]
    ra, rg = a1.shape[0], g1.shape[0]
    if a2.shape[1] != ra or g2.shape[1] != rg:
      raise ValueError(f"{self.prefix}: the low-rank pairs do not fit ({tuple(a1.shape)} . {tuple(a2.shape)}, "
                       f"{tuple(g1.shape)} . {tuple(g2.shape)})")
    # Both low-rank inputs as one product, both outputs as one product with a block-diagonal
    # matrix: [a | gate] = [y W_a1^T | y W_g1^T] . [[W_a2^T, 0], [0, W_g2^T]].
    self.rank_weight = _pad_rows(fuse_rows([a1, g1]))
    out = a2.new_zeros(a2.shape[0] + g2.shape[0], self.rank_weight.shape[0])
    out[:a2.shape[0], :ra] = a2
    out[a2.shape[0]:, ra:ra + rg] = g2
    self.out_weight = _pad_rows(out)
    self.o_proj.bind(tensors)
    conv = [t[f"{p.name}.{self.names['conv']}"] for p in (self.q_proj, self.k_proj, self.v_proj)]
    self.conv_weight = torch.cat([c.float() for c in conv], dim=0).contiguous()
    self.neg_rate = (-torch.exp(t[self._name("decay_log")].float())).contiguous()
    self.decay_bias = t[self._name("decay_bias")].float().contiguous()
    self.norm_weight = t[self._name("norm")].float().contiguous()

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    ops = ctx.ops
    sizes = dict(num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                 value_dim=self.value_dim)
    pre = ops.linear(x, self.in_weight)  # q | k | v | beta (before convolution and activations)
    low = ops.linear(ops.linear(x, self.rank_weight), self.out_weight)  # a | gate
    q, k, v, decay, beta = ops.delta_rule_inputs(
        pre, low, self.conv_weight, cache["conv"].storage, self.decay_bias, self.neg_rate, ctx,
        conv_taps=self.conv_taps, **sizes)
    o = ops.gated_delta_scan(q, k, v, decay, beta, cache["state"].storage, ctx, **sizes)
    y = ops.gated_head_norm(o, low, self.num_heads * self.head_dim, self.norm_weight, self.eps,
                            self.num_heads, self.value_dim)
    return self.o_proj(y, ctx)


@MIXERS.register("normed_mean")
class NormedMeanOfMixers(Mixer):
  """`branches`: {key: PartSpec of a mixer}; `scales`: {key: the tensor name (after the prefix) of
  the scale that the branch's output is RMS-normed with}."""

  def __init__(self, prefix: str, width: int, eps: float, branches: dict[str, PartSpec],
               scales: dict[str, str]):
    if not 1 <= len(branches) <= 4:
      raise ValueError(f"{prefix}: the mean takes one to four mixers, got {len(branches)}")
    self.prefix, self.width, self.eps = prefix, width, float(eps)
    self.branches = {key: build_part(MIXERS, spec) for key, spec in branches.items()}
    self.scale_names = {key: f"{prefix}.{scales[key]}" for key in branches}
    self.scales: list[torch.Tensor] = []

  def cache_need(self):
    needs = {key: m.cache_need() for key, m in self.branches.items()}
    return {key: need for key, need in needs.items() if need is not None}

  @property
  def graph_safe(self) -> bool:
    return all(m.graph_safe for m in self.branches.values())

  def graph_plans(self, ops, batch: int, bucket: int, max_burst: int, page_size: int) -> list:
    return [p for m in self.branches.values() for p in m.graph_plans(ops, batch, bucket, max_burst, page_size)]

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [s for m in self.branches.values() for s in m.tensor_specs()]
    return specs + [TensorSpec(name, (self.width,), "gain") for name in self.scale_names.values()]

  def bind(self, tensors, ops) -> None:
    for m in self.branches.values():
      m.bind(tensors, ops)
    self.scales = [tensors[name].float().contiguous() for name in self.scale_names.values()]

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    cache = cache or {}
    outs = [m.forward(x, ctx, cache.get(key), writes_cache) for key, m in self.branches.items()]
    return ctx.ops.normed_mean(outs, self.scales, self.eps)
