"""Typed configuration of the Tarulix decoder, from config.json.

The file is nested: ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list in run order whose entries give the
layer's ``type`` (which mixer: ``attention`` or ``parallel``), the mixer's sizes and constants (``mixer``) and its
feed-forward (``mlp``: ``kind`` ``moe`` with ``expert.ff``, ``router.experts`` / ``router.top`` /
``router.identity`` and ``shared.ff``; null for a layer with a mixer only).

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (the window), ``bias_max``
  (the distance at which the ladder of the distance bias reaches its last row) and ``v_mix`` (the layer takes part
  in the blending of values).  The number of rows of the distance bias is no key of the file: it is the row count
  of the layer's ``rel`` tensor and is filled in by ``with_tensor_shapes`` when a model folder is opened
  (``mixer.bias_rows``).
* ``parallel``: ``left`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap``, ``mask.size``,
  ``mask.pool``, ``rot.dims`` / ``rot.base``), ``right`` (``inner``, ``state``, ``dt_rank``, ``conv``) and the weights
  of the two halves, ``left_scale`` and ``right_scale``.

Every size and constant the layers use is read here; what the layers cannot run is refused.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

from .minimax_m3 import ConfigError

MIXER_TYPES = ("attention", "parallel")
MAX_HEAD_SIZE = 256
MAX_SCAN_STATE = 256
DEFAULT_BIAS_ROWS = 32            # rows of the distance bias when no checkpoint says otherwise (random models)


@dataclass(frozen=True)
class TarulixLayer:
    type: str
    mixer: dict
    mlp: dict | None


def _check_heads(where: str, m: dict) -> None:
    missing = [k for k in ("heads", "kv_heads", "dim", "vdim", "scale", "mask") if k not in m]
    if missing:
        raise ConfigError(f"{where} lacks {missing}")
    if int(m["heads"]) <= 0 or int(m["kv_heads"]) <= 0 or int(m["heads"]) % int(m["kv_heads"]):
        raise ConfigError(f"{where}: {m['heads']} heads are not a positive multiple of {m['kv_heads']} kv heads")
    if not 0 < int(m["dim"]) <= MAX_HEAD_SIZE or not 0 < int(m["vdim"]) <= MAX_HEAD_SIZE:
        raise ConfigError(f"{where}: dim and vdim must lie between 1 and {MAX_HEAD_SIZE}")
    if int((m["mask"] or {}).get("size", 0)) < 1:
        raise ConfigError(f"{where}.mask.size must be at least 1 (the token itself)")


@dataclass(frozen=True)
class TarulixConfig:
    vocab: int
    width: int
    layers: tuple[TarulixLayer, ...]
    norm_eps: float
    eos_token_ids: tuple = ()
    architecture: str = "Tarulix"
    extra: dict = field(default_factory=dict, compare=False)

    # ---- reading ---------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict, generation: dict | None = None) -> "TarulixConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"config.json lacks {key!r}")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            if "type" not in entry or "mixer" not in entry:
                raise ConfigError(f"layers[{i}] needs 'type' and 'mixer'")
            mlp = entry.get("mlp")
            layers.append(TarulixLayer(str(entry["type"]), copy.deepcopy(dict(entry["mixer"])),
                                       None if mlp is None else copy.deepcopy(dict(mlp))))
        eos = (generation or {}).get("eos_token_id", raw.get("eos_token_id"))
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        known = {"architecture", "architectures", "model_type", "vocab", "width", "layers", "norm", "eos_token_id"}
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), layers=tuple(layers),
                  norm_eps=float(raw["norm"]["eps"]), eos_token_ids=eos,
                  architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Tarulix"])[0]),
                  extra={k: v for k, v in raw.items() if k not in known})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        blend_shape = None
        for i, layer in enumerate(self.layers):
            if layer.type not in MIXER_TYPES:
                raise ConfigError(f"layers[{i}].type {layer.type!r} is not one of {MIXER_TYPES}")
            m = layer.mixer
            if layer.type == "attention":
                _check_heads(f"layers[{i}].mixer", m)
                if "bias_max" not in m:
                    raise ConfigError(f"layers[{i}].mixer lacks 'bias_max'")
                rows = m.get("bias_rows")                     # known once a checkpoint has been opened
                if rows is not None and (int(rows) < 1 or (int(rows) > 1 and float(m["bias_max"]) <= int(rows) // 2)):
                    raise ConfigError(f"layers[{i}].mixer: a bias of {rows} rows needs bias_max beyond {int(rows) // 2}")
                if m.get("v_mix"):
                    shape = (int(m["kv_heads"]), int(m["vdim"]))
                    if blend_shape is not None and shape != blend_shape:
                        raise ConfigError(f"layers[{i}] blends its values with an earlier layer's, whose kv_heads or "
                                          f"vdim differ")
                    blend_shape = shape
            else:
                for half in ("left", "right", "left_scale", "right_scale"):
                    if half not in m:
                        raise ConfigError(f"layers[{i}].mixer lacks {half!r}")
                left, right = m["left"], m["right"]
                _check_heads(f"layers[{i}].mixer.left", left)
                if int(left["mask"].get("pool") or 0) < 0 or float(left.get("softcap") or 0.0) < 0:
                    raise ConfigError(f"layers[{i}].mixer.left: mask.pool and softcap cannot be negative")
                rot = left.get("rot")
                if rot is not None:
                    dims = int(rot.get("dims", 0))
                    if dims < 0 or dims % 2 or dims > int(left["dim"]) or (dims and float(rot.get("base", 0)) <= 0):
                        raise ConfigError(f"layers[{i}].mixer.left.rot: dims must be even and at most dim, base positive")
                missing = [k for k in ("inner", "state", "dt_rank", "conv") if k not in right]
                if missing:
                    raise ConfigError(f"layers[{i}].mixer.right lacks {missing}")
                if int(right["inner"]) <= 0 or int(right["dt_rank"]) <= 0 or int(right["conv"]) < 1 \
                        or not 0 < int(right["state"]) <= MAX_SCAN_STATE:
                    raise ConfigError(f"layers[{i}].mixer.right: inner, dt_rank and conv must be positive and state "
                                      f"between 1 and {MAX_SCAN_STATE}")
            mlp = layer.mlp
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"layers[{i}].mlp.kind {mlp.get('kind')!r} is not 'moe'")
                router, expert = mlp.get("router") or {}, mlp.get("expert") or {}
                E, ident, top = int(router.get("experts", 0)), int(router.get("identity") or 0), int(router.get("top", 0))
                if E < 0 or ident < 0 or not 0 < top <= E + ident or E + ident > 1024:
                    raise ConfigError(f"layers[{i}].mlp.router: needs 0 < top <= experts + identity <= 1024")
                if E and int(expert.get("ff", 0)) <= 0:
                    raise ConfigError(f"layers[{i}].mlp.expert.ff must be positive")
                shared = mlp.get("shared")
                if shared is not None and int(shared.get("ff", 0)) <= 0:
                    raise ConfigError(f"layers[{i}].mlp.shared.ff must be positive")

    # ---- sizes that only the checkpoint knows --------------------------------------------------------
    def with_tensor_shapes(self, shape_of) -> "TarulixConfig":
        """``shape_of(name) -> shape or None``: fill in the sizes that are no keys of the file: the number of rows
        of an attention layer's distance bias (``mixer.bias_rows``, the row count of ``l<i>.mix.rel``)."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = dict(layer.mixer)
            if layer.type == "attention":
                shape = shape_of(f"l{i}.mix.rel")
                if shape is None:
                    raise ConfigError(f"layers[{i}]: the checkpoint has no l{i}.mix.rel to take the bias rows from")
                m["bias_rows"] = int(shape[0])
            layers.append(TarulixLayer(layer.type, m, layer.mlp))
        cfg = TarulixConfig(**{**self.__dict__, "layers": tuple(layers)})
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = dict(self.extra)
        d.update({
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)} for l in self.layers],
        })
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
