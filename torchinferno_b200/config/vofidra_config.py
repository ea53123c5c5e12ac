"""Typed configuration of the Vofidra design, read from a checkpoint's ``config.json``.

The file names the design under ``architecture``, gives the global sizes (``vocab``, ``width``), the number of
``streams`` the residual is carried in, the ``eps`` of the RMS norms inside the mixers (``norm.eps``), the cap of the
logits (``logit_softcap``) and a list ``layers`` whose entries each name a mixer ``type`` with its sizes and constants
(``mixer``) and a feed-forward (``mlp``, or null).  No size or constant has a default: a missing key is an error that
names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from torchinferno_b200.config.model_config import ConfigError

MIXERS = ("latent_attention", "attention")
FEED_FORWARDS = ("dense", "moe")
# The design names no limit.  Positions are exact in the 32-bit floats the rotary angles are made from up to 2^24; the
# limit given here is what block tables and default pools are sized by when the user names none
# (EngineConfig.max_model_len).
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


def _number(data: Mapping[str, Any], key: str, where: str) -> float:
    value = _need(data, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class VofidraLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], index: int) -> "VofidraLayer":
        where = f"layers[{index}]"
        kind = _need(data, "type", where)
        if kind not in MIXERS:
            raise ConfigError(f"config.json: {where}.type={kind!r}; known mixers: {list(MIXERS)}")
        mixer = _need(data, "mixer", where)
        at = where + ".mixer"
        _number(mixer, "scale", at)
        if kind == "latent_attention":
            for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
                _positive(mixer, key, at)
            rot = _need(mixer, "rot", at)
            if not _number(rot, "base", at + ".rot") > 0:
                raise ConfigError(f"config.json: {at}.rot.base must be positive")
            dims = _positive(rot, "dims", at + ".rot")
            if dims % 2 or dims > mixer["rot_dim"]:
                raise ConfigError(f"config.json: {at}.rot.dims must be even and at most rot_dim")
        else:
            for key in ("heads", "kv_heads", "dim", "vdim", "bias_max"):
                _positive(mixer, key, at)
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"config.json: {at}.heads must be a multiple of kv_heads")
            temp = _need(mixer, "q_temp", at)
            _number(temp, "coef", at + ".q_temp"), _positive(temp, "every", at + ".q_temp")
        mlp = data.get("mlp")
        if mlp is not None:
            at = where + ".mlp"
            form = _need(mlp, "kind", at)
            if form not in FEED_FORWARDS:
                raise ConfigError(f"config.json: {at}.kind={form!r}; known: {list(FEED_FORWARDS)}")
            if form == "dense":
                _positive(mlp, "ff", at)
            else:
                _positive(_need(mlp, "expert", at), "ff", at + ".expert")
                router = _need(mlp, "router", at)
                at += ".router"
                experts, top = _positive(router, "experts", at), _positive(router, "top", at)
                identity = _need(router, "identity", at)
                if not isinstance(identity, int) or isinstance(identity, bool) or identity < 0:
                    raise ConfigError(f"config.json: {at}.identity must be a count, got {identity!r}")
                groups = _need(router, "groups", at)
                count, keep = _positive(groups, "count", at + ".groups"), _positive(groups, "keep", at + ".groups")
                total = experts + identity
                if total % count or keep > count:
                    raise ConfigError(f"config.json: {at}.groups: {count} groups must divide the {total} router outputs, "
                                      f"and keep at most {count}")
                if top > keep * (total // count):
                    raise ConfigError(f"config.json: {at}.top exceeds what the kept groups hold")
        return cls(kind, dict(mixer), None if mlp is None else dict(mlp))


@dataclass(frozen=True)
class VofidraConfig:
    vocab: int
    width: int
    streams: int
    layers: tuple[VofidraLayer, ...]
    eps: float
    logit_softcap: float | None
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "VofidraConfig":
        where = "the model"
        layers = _need(data, "layers", where)
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one entry")
        typed = tuple(VofidraLayer.from_dict(entry, i) for i, entry in enumerate(layers))
        eps = _number(_need(data, "norm", where), "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        cap = data.get("logit_softcap") or None          # (absent, null or 0: the logits are not capped)
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or not float(cap) > 0):
            raise ConfigError("config.json: logit_softcap must be a positive number when given")
        return cls(vocab=_positive(data, "vocab", where), width=_positive(data, "width", where),
                   streams=_positive(data, "streams", where), layers=typed, eps=eps,
                   logit_softcap=None if cap is None else float(cap), raw=dict(data))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)
