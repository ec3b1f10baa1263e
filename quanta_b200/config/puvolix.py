"""Typed configuration of the Puvolix decoder, from config.json.

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``norm.groups`` (every norm of the stream divides each of
that many equal parts of the vector by the part's own root mean square), ``logit_softcap`` and ``layers``, a list in
run order whose entries give the layer's ``type`` (the one mixer, ``parallel``), the mixer's sizes and constants
(``mixer``) and its feed-forward (``mlp``; null for a layer with a mixer only).

* ``mixer.left`` (softmax attention): ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``conv`` (taps of the
  short convolution on the projected q, k, v), ``rot.dims`` / ``rot.base`` and ``rot.scaling`` (``factor``, ``low``,
  ``high``, ``original``: the rescaling of the rotation's frequencies by wavelength).
* ``mixer.right`` (gated delta rule): ``heads``, ``kv_heads`` (groups of q/k heads), ``dim``, ``vdim``, ``conv``.
* ``mlp.kind`` ``dense``: ``ff``.  ``moe``: ``expert.ff`` / ``expert.limit``, ``router.experts`` / ``router.top`` and
  ``shared.ff`` / ``shared.limit`` (or no shared expert).

Every size and constant the layers use is read here; what the layers cannot run is refused.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

from .minimax_m3 import ConfigError

MIXER_TYPES = ("parallel",)
MAX_HEAD_SIZE = 256
MAX_NORM_GROUPS = 64


@dataclass(frozen=True)
class PuvolixLayer:
    type: str
    mixer: dict
    mlp: dict | None


def _check_heads(where: str, m: dict, need: tuple) -> None:
    missing = [k for k in need if k not in m]
    if missing:
        raise ConfigError(f"{where} lacks {missing}")
    if int(m["heads"]) <= 0 or int(m["kv_heads"]) <= 0 or int(m["heads"]) % int(m["kv_heads"]):
        raise ConfigError(f"{where}: {m['heads']} heads are not a positive multiple of {m['kv_heads']} kv heads")
    if not 0 < int(m["dim"]) <= MAX_HEAD_SIZE or not 0 < int(m["vdim"]) <= MAX_HEAD_SIZE:
        raise ConfigError(f"{where}: dim and vdim must lie between 1 and {MAX_HEAD_SIZE}")
    if int(m.get("conv") or 0) < 0:
        raise ConfigError(f"{where}.conv cannot be negative")


@dataclass(frozen=True)
class PuvolixConfig:
    vocab: int
    width: int
    layers: tuple[PuvolixLayer, ...]
    norm_eps: float
    norm_groups: int = 1
    logit_softcap: float = 0.0
    eos_token_ids: tuple = ()
    architecture: str = "Puvolix"
    extra: dict = field(default_factory=dict, compare=False)

    # ---- reading ---------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict, generation: dict | None = None) -> "PuvolixConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"config.json lacks {key!r}")
        if "eps" not in raw["norm"]:
            raise ConfigError("config.json lacks norm.eps")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            if "type" not in entry or "mixer" not in entry:
                raise ConfigError(f"layers[{i}] needs 'type' and 'mixer'")
            mlp = entry.get("mlp")
            layers.append(PuvolixLayer(str(entry["type"]), copy.deepcopy(dict(entry["mixer"])),
                                       None if mlp is None else copy.deepcopy(dict(mlp))))
        eos = (generation or {}).get("eos_token_id", raw.get("eos_token_id"))
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        known = {"architecture", "architectures", "model_type", "vocab", "width", "layers", "norm", "logit_softcap",
                 "eos_token_id"}
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), layers=tuple(layers),
                  norm_eps=float(raw["norm"]["eps"]), norm_groups=int(raw["norm"].get("groups") or 1),
                  logit_softcap=float(raw.get("logit_softcap") or 0.0), eos_token_ids=eos,
                  architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Puvolix"])[0]),
                  extra={k: v for k, v in raw.items() if k not in known})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not 1 <= self.norm_groups <= MAX_NORM_GROUPS or self.width % self.norm_groups:
            raise ConfigError(f"norm.groups {self.norm_groups} must divide the width {self.width} "
                              f"(1 to {MAX_NORM_GROUPS})")
        if self.logit_softcap < 0 or self.norm_eps < 0:
            raise ConfigError("logit_softcap and norm.eps cannot be negative")
        for i, layer in enumerate(self.layers):
            if layer.type not in MIXER_TYPES:
                raise ConfigError(f"layers[{i}].type {layer.type!r} is not one of {MIXER_TYPES}")
            m = layer.mixer
            for half in ("left", "right"):
                if half not in m:
                    raise ConfigError(f"layers[{i}].mixer lacks {half!r}")
            left, right = m["left"], m["right"]
            _check_heads(f"layers[{i}].mixer.left", left, ("heads", "kv_heads", "dim", "vdim", "scale"))
            _check_heads(f"layers[{i}].mixer.right", right, ("heads", "kv_heads", "dim", "vdim"))
            rot = left.get("rot")
            if rot is not None:
                dims = int(rot.get("dims") or 0)
                if dims < 0 or dims % 2 or dims > int(left["dim"]) or (dims and float(rot.get("base", 0)) <= 0):
                    raise ConfigError(f"layers[{i}].mixer.left.rot: dims must be even and at most dim, base positive")
                sc = rot.get("scaling")
                if sc is not None:
                    missing = [k for k in ("factor", "low", "high", "original") if k not in sc]
                    if missing:
                        raise ConfigError(f"layers[{i}].mixer.left.rot.scaling lacks {missing}")
                    if float(sc["factor"]) <= 0 or float(sc["original"]) <= 0 or not 0 < float(sc["low"]) < float(sc["high"]):
                        raise ConfigError(f"layers[{i}].mixer.left.rot.scaling: needs factor, original > 0 and "
                                          f"0 < low < high")
            mlp = layer.mlp
            if mlp is None:
                continue
            kind = mlp.get("kind")
            if kind == "dense":
                if int(mlp.get("ff", 0)) <= 0:
                    raise ConfigError(f"layers[{i}].mlp.ff must be positive")
            elif kind == "moe":
                router, expert = mlp.get("router") or {}, mlp.get("expert") or {}
                E, top = int(router.get("experts", 0)), int(router.get("top", 0))
                if not 0 < top <= E <= 1024:
                    raise ConfigError(f"layers[{i}].mlp.router: needs 0 < top <= experts <= 1024")
                if int(expert.get("ff", 0)) <= 0 or not float(expert.get("limit", 0)) > 0:
                    raise ConfigError(f"layers[{i}].mlp.expert: ff and limit must be positive")
                shared = mlp.get("shared")
                if shared is not None and (int(shared.get("ff", 0)) <= 0 or not float(shared.get("limit", 0)) > 0):
                    raise ConfigError(f"layers[{i}].mlp.shared: ff and limit must be positive")
            else:
                raise ConfigError(f"layers[{i}].mlp.kind {kind!r} is not 'dense' or 'moe'")

    def to_dict(self) -> dict:
        d = dict(self.extra)
        d.update({
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "logit_softcap": self.logit_softcap,
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)} for l in self.layers],
        })
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
