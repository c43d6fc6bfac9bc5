"""Configuration of the Generax decoder, read from config.json.

config.json of this design:

  architecture    "Generax"
  vocab, width    sizes of the embedding table and of the residual stream
  norm.eps        eps of every RMS norm of the layers, of the mixers and of the final norm
  logit_softcap   soft cap on the output logits (absent or 0: none)
  layers          one entry per layer: `type` ("attention" or "parallel"), `mixer` (its sizes) and
                  `mlp` ({"kind": "dense", "ff": F} or null)
  max_context     (optional) the longest sequence the engine will serve; the design itself has no limit

A layer is `h += mixer(y) + mlp(y)` with `y = rms_norm(h)` (block `parallel_residual`).  Tensor
names: `embed`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`, `final.norm`, `head`.

mixer of type "attention" (mixer `qk_norm_attention`): heads, kv_heads, dim, vdim, scale,
mask.size (window), rot.{dims, base, scaling.factor}, and optionally kv_from: j, which makes
the layer read layer j's cache instead of having keys and values of its own.  Values are
rotated, and every head has a temperature (`temp`).

mixer of type "parallel" (mixer `normed_mean` of two): `left` is attention without rotation with
mask.size and mask.pool (pooled blocks in front of the window), `right` the gated delta rule
with heads, kv_heads, dim, vdim and conv (taps).  The ranks of the delta rule's low-rank pairs
are in no key: they are read off the tensors (`decay_rank`, `gate_rank` are this engine's own
optional keys, written by the random-weights mode, which has no tensors to read them off).
"""

from __future__ import annotations

import copy
import dataclasses
from typing import Any

from simply_b200.config.gemma2 import ConfigError
from simply_b200.config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from simply_b200.registry import ARCHITECTURES

_DEFAULT_MAX_CONTEXT = 1 << 17


def _need(d: dict, key: str, where: str):
  if not isinstance(d, dict) or key not in d or d[key] is None:
    raise ConfigError(f"config.json: {where} lacks {key!r}")
  return d[key]


@dataclasses.dataclass(frozen=True)
class GeneraxConfig:
  vocab: int
  width: int
  eps: float
  layers: tuple[dict, ...]
  logit_softcap: float = 0.0
  max_context: int = _DEFAULT_MAX_CONTEXT
  bos_token_id: int | None = None
  eos_token_id: int | tuple[int, ...] | None = None

  architecture = "Generax"

  # ---- reading and writing ------------------------------------------------------
  @classmethod
  def from_dict(cls, d: dict[str, Any]) -> "GeneraxConfig":
    eos = d.get("eos_token_id")
    if isinstance(eos, list):
      eos = tuple(int(e) for e in eos)
    cfg = cls(
        vocab=int(_need(d, "vocab", "the model")), width=int(_need(d, "width", "the model")),
        eps=float(_need(_need(d, "norm", "the model"), "eps", "norm")),
        layers=tuple(copy.deepcopy(l) for l in _need(d, "layers", "the model")),
        logit_softcap=float(d.get("logit_softcap") or 0.0),
        max_context=int(d.get("max_context") or _DEFAULT_MAX_CONTEXT),
        bos_token_id=d.get("bos_token_id"), eos_token_id=eos)
    cfg.validate()
    return cfg

  def to_dict(self) -> dict[str, Any]:
    d: dict[str, Any] = {
        "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
        "norm": {"eps": self.eps}, "logit_softcap": self.logit_softcap,
        "layers": [copy.deepcopy(l) for l in self.layers], "max_context": self.max_context}
    if self.bos_token_id is not None:
      d["bos_token_id"] = self.bos_token_id
    if self.eos_token_id is not None:
      d["eos_token_id"] = list(self.eos_token_id) if isinstance(self.eos_token_id, tuple) else self.eos_token_id
    return d

  def replace(self, **changes: Any) -> "GeneraxConfig":
    cfg = dataclasses.replace(self, **changes)
    cfg.validate()
    return cfg

  # ---- checks -------------------------------------------------------------------
  def validate(self) -> None:
    if self.vocab <= 0 or self.width <= 0 or self.max_context <= 0:
      raise ConfigError("vocab, width and max_context must be positive")
    if not self.eps > 0:
      raise ConfigError("norm.eps must be positive")
    if not self.layers:
      raise ConfigError("the model has no layers")
    for i, layer in enumerate(self.layers):
      where = f"layer {i}"
      kind = _need(layer, "type", where)
      mixer = _need(layer, "mixer", where)
      if kind == "attention":
        self._check_attention(mixer, where, i)
      elif kind == "parallel":
        self._check_attention(_need(mixer, "left", where), f"{where} (left)", i)
        right = _need(mixer, "right", where)
        for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
          if int(_need(right, key, f"{where} (right)")) <= 0:
            raise ConfigError(f"{where} (right): {key} must be positive")
        if right["heads"] % right["kv_heads"]:
          raise ConfigError(f"{where} (right): heads must be a multiple of kv_heads")
      else:
        raise ConfigError(f"{where}: unknown type {kind!r} (known: attention, parallel)")
      mlp = layer.get("mlp")
      if mlp is not None:
        if mlp.get("kind") != "dense":
          raise ConfigError(f"{where}: unknown mlp kind {mlp.get('kind')!r} (known: dense)")
        if int(_need(mlp, "ff", f"{where} (mlp)")) <= 0:
          raise ConfigError(f"{where}: ff must be positive")

  def _check_attention(self, m: dict, where: str, index: int) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
      if int(_need(m, key, where)) <= 0:
        raise ConfigError(f"{where}: {key} must be positive")
    _need(m, "scale", where)
    if m["heads"] % m["kv_heads"]:
      raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
    mask = m.get("mask") or {}
    if mask.get("pool") is not None and mask.get("size") is None:
      raise ConfigError(f"{where}: pooled blocks need a window (mask.size)")
    rot = m.get("rot")
    if rot:
      dims = int(_need(rot, "dims", f"{where} (rot)"))
      _need(rot, "base", f"{where} (rot)")
      if dims % 2 or dims > m["dim"] or m["vdim"] % 2:
        raise ConfigError(f"{where}: rot.dims must be even and at most dim, and vdim even")
    source = m.get("kv_from")
    if source is not None:
      if not 0 <= int(source) < index:
        raise ConfigError(f"{where}: kv_from must name an earlier layer, got {source}")
      other = self.layers[int(source)]
      om = other.get("mixer", {})
      if other.get("type") != "attention" or om.get("kv_from") is not None:
        raise ConfigError(f"{where}: kv_from must name an attention layer with keys and values of its own")
      for key in ("kv_heads", "dim", "vdim", "rot"):
        if om.get(key) != m.get(key):
          raise ConfigError(f"{where}: {key} differs from layer {source}, whose cache it reads")

  # ---- derived --------------------------------------------------------------------
  def _attention_spec(self, prefix: str, m: dict, *, rotated: bool, cache_window: int | None = None) -> PartSpec:
    mask = m.get("mask") or {}
    rot = m.get("rot") if rotated else None
    params = {
        "width": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
        "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "score_scale": float(m["scale"]),
        "eps": self.eps, "window": None if mask.get("size") is None else int(mask["size"]),
        "pool": None if mask.get("pool") is None else int(mask["pool"]),
        "rotary": None, "rotate_values": False, "head_temperature": rotated,
        "project_kv": m.get("kv_from") is None, "cache_window": cache_window,
    }
    if rot:
      params["rotary"] = {"dims": int(rot["dims"]), "base": float(rot["base"]),
                          "factor": float((rot.get("scaling") or {}).get("factor", 1.0))}
      params["rotate_values"] = True
    return PartSpec("qk_norm_attention", prefix, params)

  def model_spec(self) -> ModelSpec:
    norm = PartSpec("rms_norm", params={"eps": self.eps, "plus_one": False})
    # A cache that other layers read keeps the widest of their windows.
    readers: dict[int, list] = {}
    for layer in self.layers:
      m = layer["mixer"]
      if layer["type"] == "attention" and m.get("kv_from") is not None:
        readers.setdefault(int(m["kv_from"]), []).append((m.get("mask") or {}).get("size"))
    layers, order = [], []
    for i, layer in enumerate(self.layers):
      p = f"l{i}"
      m = layer["mixer"]
      if layer["type"] == "attention":
        sizes = readers.get(i, [])
        if any(s is None for s in sizes) and (m.get("mask") or {}).get("size") is not None:
          raise ConfigError(f"layer {i}: a layer without a window reads this layer's windowed cache")
        keep = max((int(s) for s in sizes if s is not None), default=None)
        mixer = self._attention_spec(f"{p}.mix", m, rotated=True, cache_window=keep)
      else:
        right = m["right"]
        delta = PartSpec("gated_delta_rule", f"{p}.mix.right", {
            "width": self.width, "num_heads": int(right["heads"]), "num_kv_heads": int(right["kv_heads"]),
            "head_dim": int(right["dim"]), "value_dim": int(right["vdim"]), "conv_taps": int(right["conv"]),
            "eps": self.eps, "decay_rank": int(right.get("decay_rank", -1)),
            "gate_rank": int(right.get("gate_rank", -1))})
        mixer = PartSpec("normed_mean", f"{p}.mix", {
            "width": self.width, "eps": self.eps,
            "branches": {"left": self._attention_spec(f"{p}.mix.left", m["left"], rotated=False), "right": delta},
            "scales": {"left": "left.out", "right": "right.out"}})
      mlp = layer.get("mlp")
      if mlp is None:
        ffn = PartSpec("none", f"{p}.mlp")
      else:
        ffn = PartSpec("gated", f"{p}.mlp", {
            "width": self.width, "hidden": int(mlp["ff"]), "activation": "silu",
            "names": {"gate": "gate", "up": "up", "down": "down"}})
      block = PartSpec("parallel_residual", p, {"width": self.width, "norm": norm, "names": {"norm": "norm1"}})
      layers.append(LayerSpec(p, block, mixer, ffn))
      source = m.get("kv_from") if layer["type"] == "attention" else None
      if source is None:
        order.append(LayerCall(p))
      else:
        order.append(LayerCall(p, cache=f"l{int(source)}#{int(source)}", writes_cache=False))
    spec = ModelSpec(
        architecture=self.architecture, vocab_size=self.vocab, width=self.width, max_context=self.max_context,
        embedding=PartSpec("token_embedding", "embed",
                           {"vocab_size": self.vocab, "width": self.width, "scale": 1.0, "name": "embed"}),
        layers=tuple(layers), run_order=tuple(order),
        final_norm=PartSpec("rms_norm", "final", {"width": self.width, "eps": self.eps, "plus_one": False,
                                                  "name": "final.norm"}),
        head=PartSpec("linear_head", "head", {"logit_softcap": self.logit_softcap, "name": "head"}))
    spec.validate()
    return spec


ARCHITECTURES.register(GeneraxConfig.architecture, GeneraxConfig)
