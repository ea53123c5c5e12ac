"""Typed configuration of the Tibalorn design, read from a checkpoint's ``config.json``.

The file names the design under ``architecture``, gives the global sizes (``vocab``, ``width``), the norms' ``eps``,
the embedding's multiplier (``embedding.scale``), the cap of the logits (``logit_softcap``) and a list ``layers`` whose
entries each name a mixer ``type`` (``attention`` or ``mamba2``) with its sizes and constants (``mixer``) and a
feed-forward (``mlp``, or null).  No size or constant has a default: a missing key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from torchinferno_b200.config.model_config import ConfigError

MIXERS = ("attention", "mamba2")
# The design names no limit.  Positions are exact in the 32-bit floats the rotary angles are made from up to 2^24; the
# limit given here is what block tables and default pools are sized by when the user names none.
MAX_POSITIONS = 1 << 20


def _need(data: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(data, Mapping) or key not in data:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return data[key]


def _positive(data: Mapping[str, Any], key: str, where: str) -> int:
    value = _need(data, key, where)
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {value!r}")
    return value


def _positive_float(data: Mapping[str, Any], key: str, where: str) -> float:
    value = _need(data, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not float(value) > 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class TibalornLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], index: int) -> "TibalornLayer":
        where = f"layers[{index}]"
        kind = _need(data, "type", where)
        if kind not in MIXERS:
            raise ConfigError(f"config.json: {where}.type={kind!r}; known mixers: {list(MIXERS)}")
        mixer = _need(data, "mixer", where)
        at = where + ".mixer"
        if kind == "mamba2":
            heads, groups = _positive(mixer, "heads", at), _positive(mixer, "groups", at)
            if heads % groups:
                raise ConfigError(f"config.json: {at}.heads must be a multiple of groups")
            vdim, parts = _positive(mixer, "vdim", at), _positive(mixer, "norm_groups", at)
            if (heads * vdim) % parts:
                raise ConfigError(f"config.json: {at}.norm_groups must divide heads * vdim")
            _positive(mixer, "state", at), _positive(mixer, "conv", at)
        else:
            heads, kv_heads = _positive(mixer, "heads", at), _positive(mixer, "kv_heads", at)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {at}.heads must be a multiple of kv_heads")
            dim = _positive(mixer, "dim", at)
            if _positive(mixer, "vdim", at) % 2:
                raise ConfigError(f"config.json: {at}.vdim must be even (values are rotated in pairs)")
            _positive_float(mixer, "scale", at)
            mask = _need(mixer, "mask", at)
            _positive(mask, "size", at + ".mask"), _positive(mask, "pool", at + ".mask")
            rot = _need(mixer, "rot", at)
            _positive_float(rot, "base", at + ".rot")
            dims = _positive(rot, "dims", at + ".rot")
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {at}.rot.dims must be even and at most dim")
            scaling = rot.get("scaling")
            if scaling is not None:
                for key in ("factor", "original", "fast", "slow"):
                    _positive_float(scaling, key, at + ".rot.scaling")
        mlp = data.get("mlp")
        if mlp is not None:
            at = where + ".mlp"
            form = _need(mlp, "kind", at)
            if form != "dense":
                raise ConfigError(f"config.json: {at}.kind={form!r}; known: ['dense']")
            _positive(mlp, "ff", at)
        return cls(kind, dict(mixer), None if mlp is None else dict(mlp))


@dataclass(frozen=True)
class TibalornConfig:
    vocab: int
    width: int
    layers: tuple[TibalornLayer, ...]
    eps: float
    embedding_scale: float
    logit_softcap: float | None
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "TibalornConfig":
        where = "the model"
        layers = _need(data, "layers", where)
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one entry")
        typed = tuple(TibalornLayer.from_dict(entry, i) for i, entry in enumerate(layers))
        cap = _need(data, "logit_softcap", where)
        return cls(vocab=_positive(data, "vocab", where), width=_positive(data, "width", where), layers=typed,
                   eps=_positive_float(_need(data, "norm", where), "eps", "norm"),
                   embedding_scale=float(_need(_need(data, "embedding", where), "scale", "embedding")),
                   logit_softcap=None if cap is None else _positive_float(data, "logit_softcap", where), raw=dict(data))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)
