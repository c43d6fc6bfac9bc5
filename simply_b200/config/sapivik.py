"""Configuration of the Sapivik decoder, read from config.json.

config.json of this design:

  architecture    "Sapivik"
  vocab, width    sizes of the embedding table and of the residual stream
  norm.eps        eps of every RMS norm: the layers', the mixers' and the final one
  residual_mult   m: every branch is added to the stream times m
  layers          one entry per layer: `type` ("attention" or "hgrn2"), `mixer` (its sizes) and
                  `mlp` (a feed-forward, or null)
  loop            (optional) {start, stop, times}: layers start .. stop - 1 run `times` times in a
                  row with the same weights and a cache or state of its own per pass; before every
                  pass but the first the embedding's output is added to the stream
  max_context     (optional) the longest sequence the engine will serve; the design has no limit

A layer is `h += m * norm1b(mixer(norm1(h)))`, then `h += m * norm2b(mlp(norm2(h)))` if it has a
feed-forward (block `sandwich_norm` with a residual scale).  Tensor names: `embed`,
`l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.

mixer of type "attention" (mixer `head_norm_attention`): heads, kv_heads, dim, vdim (= dim: the
values are the keys as projected), scale, softcap (absent or 0: none), rot.{dims, base} (neighbouring
dims pair up).  Tensors q, k, g (output gate), o.

mixer of type "hgrn2" (mixer `forget_gate_recurrence`): heads, dim, vdim.  Tensors q, f, f.b,
lower, v, norm, o.

mlp: {"kind": "dense", "ff", "limit"} (feed-forward `gated` with the clamped activation; tensors
gate, up, down) or {"kind": "moe", "expert": {"ff"}, "router": {"experts", "identity", "top",
"scale"}, "shared": {"ff"} or absent} (feed-forward `routed_experts`; tensors e<j>.{gate,up,down},
router, correction, shared.{gate,up,down,sg}).
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
class SapivikConfig:
  vocab: int
  width: int
  eps: float
  residual_mult: float
  layers: tuple[dict, ...]
  loop: tuple[int, int, int] = (0, 0, 1)  # start, stop, times
  max_context: int = _DEFAULT_MAX_CONTEXT
  bos_token_id: int | None = None
  eos_token_id: int | tuple[int, ...] | None = None

  architecture = "Sapivik"

  # ---- reading and writing ------------------------------------------------------
  @classmethod
  def from_dict(cls, d: dict[str, Any]) -> "SapivikConfig":
    eos = d.get("eos_token_id")
    if isinstance(eos, list):
      eos = tuple(int(e) for e in eos)
    loop = d.get("loop")
    if loop:
      loop = (int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")), int(_need(loop, "times", "loop")))
    cfg = cls(
        vocab=int(_need(d, "vocab", "the model")), width=int(_need(d, "width", "the model")),
        eps=float(_need(_need(d, "norm", "the model"), "eps", "norm")),
        residual_mult=float(d["residual_mult"]) if d.get("residual_mult") is not None else 1.0,
        layers=tuple(copy.deepcopy(l) for l in _need(d, "layers", "the model")),
        loop=loop or (0, 0, 1),
        max_context=int(d.get("max_context") or _DEFAULT_MAX_CONTEXT),
        bos_token_id=d.get("bos_token_id"), eos_token_id=eos)
    cfg.validate()
    return cfg

  def to_dict(self) -> dict[str, Any]:
    d: dict[str, Any] = {
        "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
        "norm": {"eps": self.eps}, "residual_mult": self.residual_mult,
        "layers": [copy.deepcopy(l) for l in self.layers],
        "loop": {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]},
        "max_context": self.max_context}
    if self.bos_token_id is not None:
      d["bos_token_id"] = self.bos_token_id
    if self.eos_token_id is not None:
      d["eos_token_id"] = list(self.eos_token_id) if isinstance(self.eos_token_id, tuple) else self.eos_token_id
    return d

  def replace(self, **changes: Any) -> "SapivikConfig":
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
    start, stop, times = self.loop
    if not (0 <= start <= stop <= len(self.layers)) or times < 1:
      raise ConfigError(f"loop {self.loop} does not fit {len(self.layers)} layers (0 <= start <= stop, times >= 1)")
    for i, layer in enumerate(self.layers):
      where = f"layer {i}"
      kind = _need(layer, "type", where)
      m = _need(layer, "mixer", where)
      if kind == "attention":
        for key in ("heads", "kv_heads", "dim", "vdim"):
          if int(_need(m, key, where)) <= 0:
            raise ConfigError(f"{where}: {key} must be positive")
        _need(m, "scale", where)
        if m["heads"] % m["kv_heads"]:
          raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
        if m["vdim"] != m["dim"]:
          raise ConfigError(f"{where}: the values are the keys, so vdim must equal dim")
        rot = m.get("rot")
        if rot:
          dims = int(_need(rot, "dims", f"{where} (rot)"))
          _need(rot, "base", f"{where} (rot)")
          if dims % 2 or dims < 0 or dims > m["dim"]:
            raise ConfigError(f"{where}: rot.dims must be even and at most dim")
      elif kind == "hgrn2":
        for key in ("heads", "dim", "vdim"):
          if int(_need(m, key, where)) <= 0:
            raise ConfigError(f"{where}: {key} must be positive")
      else:
        raise ConfigError(f"{where}: unknown type {kind!r} (known: attention, hgrn2)")
      mlp = layer.get("mlp")
      if mlp is None:
        continue
      if mlp.get("kind") == "dense":
        if int(_need(mlp, "ff", f"{where} (mlp)")) <= 0:
          raise ConfigError(f"{where}: ff must be positive")
        _need(mlp, "limit", f"{where} (mlp)")
      elif mlp.get("kind") == "moe":
        r = _need(mlp, "router", f"{where} (mlp)")
        experts, identity = int(_need(r, "experts", f"{where} (router)")), int(r.get("identity") or 0)
        top = int(_need(r, "top", f"{where} (router)"))
        if experts < 0 or identity < 0 or not 1 <= top <= experts + identity:
          raise ConfigError(f"{where}: the router must choose between 1 and experts + identity experts")
        if experts and int(_need(_need(mlp, "expert", f"{where} (mlp)"), "ff", f"{where} (expert)")) <= 0:
          raise ConfigError(f"{where}: the experts' ff must be positive")
        if mlp.get("shared") and int(_need(mlp["shared"], "ff", f"{where} (shared)")) <= 0:
          raise ConfigError(f"{where}: the shared expert's ff must be positive")
      else:
        raise ConfigError(f"{where}: unknown mlp kind {mlp.get('kind')!r} (known: dense, moe)")

  # ---- derived --------------------------------------------------------------------
  def _mixer_spec(self, p: str, kind: str, m: dict) -> PartSpec:
    if kind == "attention":
      rot = m.get("rot")
      rotary = None
      if rot and int(rot["dims"]) > 0:
        rotary = {"dims": int(rot["dims"]), "base": float(rot["base"]), "layout": "neighbours"}
      return PartSpec("head_norm_attention", f"{p}.mix", {
          "width": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
          "head_dim": int(m["dim"]), "score_scale": float(m["scale"]), "eps": self.eps,
          "score_softcap": float(m.get("softcap") or 0.0), "rotary": rotary, "head_norm": True,
          "tie_values": True, "output_gate": True})
    return PartSpec("forget_gate_recurrence", f"{p}.mix", {
        "width": self.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]),
        "value_dim": int(m["vdim"]), "eps": self.eps})

  def _mlp_spec(self, p: str, mlp: dict | None) -> PartSpec:
    if mlp is None:
      return PartSpec("none", f"{p}.mlp")
    names = {"gate": "gate", "up": "up", "down": "down"}
    if mlp["kind"] == "dense":
      return PartSpec("gated", f"{p}.mlp", {
          "width": self.width, "hidden": int(mlp["ff"]), "activation": "clamped_swish",
          "limit": float(mlp["limit"]), "names": names})
    r = mlp["router"]
    shared = mlp.get("shared")
    return PartSpec("routed_experts", f"{p}.mlp", {
        "width": self.width, "hidden": int((mlp.get("expert") or {}).get("ff", 0)),
        "num_experts": int(r["experts"]), "num_identity": int(r.get("identity") or 0), "top": int(r["top"]),
        "weight_scale": float(r.get("scale", 1.0)), "activation": "silu", "score": "softmax",
        "correction": True, "renormalize": False,
        "shared_hidden": int(shared["ff"]) if shared else 0, "shared_gate": bool(shared)})

  def model_spec(self) -> ModelSpec:
    norm = PartSpec("rms_norm", params={"eps": self.eps, "plus_one": False})
    names = {"pre_mixer": "norm1", "post_mixer": "norm1b", "pre_feed_forward": "norm2", "post_feed_forward": "norm2b"}
    layers = []
    for i, layer in enumerate(self.layers):
      p = f"l{i}"
      block = PartSpec("sandwich_norm", p, {"width": self.width, "norm": norm, "names": names, "full_names": True,
                                            "residual_scale": self.residual_mult})
      layers.append(LayerSpec(p, block, self._mixer_spec(p, layer["type"], layer["mixer"]),
                              self._mlp_spec(p, layer.get("mlp"))))
    start, stop, times = self.loop
    order = [LayerCall(f"l{i}") for i in range(start)]
    for rep in range(times):
      order += [LayerCall(f"l{i}", add_embedding=rep > 0 and i == start) for i in range(start, stop)]
    order += [LayerCall(f"l{i}") for i in range(stop, len(self.layers))]
    spec = ModelSpec(
        architecture=self.architecture, vocab_size=self.vocab, width=self.width, max_context=self.max_context,
        embedding=PartSpec("token_embedding", "embed",
                           {"vocab_size": self.vocab, "width": self.width, "scale": 1.0, "name": "embed"}),
        layers=tuple(layers), run_order=tuple(order),
        final_norm=PartSpec("rms_norm", "final", {"width": self.width, "eps": self.eps, "plus_one": False,
                                                  "name": "final.norm"}),
        head=PartSpec("linear_head", "head", {"logit_softcap": 0.0, "name": "head"}))
    spec.validate()
    return spec


ARCHITECTURES.register(SapivikConfig.architecture, SapivikConfig)
