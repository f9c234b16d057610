"""Typed configuration of the Tikizen decoder.

config.json gives every size and every constant that differs between models of the design:

    architecture   "Tikizen"
    vocab, width
    norm           {"eps": ...}: every norm of the model
    postln_alpha   what the stream is multiplied by before a sub-layer's output is added and the sum is normed
    layers         a list; every entry has "type" (which mixer), "mixer" (its sizes and constants) and "mlp"
                   (a dense or a routed feed-forward, or null for a layer without one)
    max_positions  optional: the most positions of a sequence (rotation tables are made for that many)

Mixers: "attention" (heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, original, fast, slow}},
mask {size}, kv_from), "retention" (heads, dim, vdim, decay [per head], rot as above), "mamba2" (heads, vdim,
state, groups, conv, norm_groups).  Feed-forwards: {"kind": "dense", "ff", "limit"} and {"kind": "moe", "expert":
{"ff"}, "router": {"experts", "top"}, "shared": {"ff"}}.

A key that the chosen part needs and that is absent is an error: no size stands in code.  Keys that this reader does
not know inside `norm`, a layer, its mixer or its feed-forward are an error too, so that a variant of the design is
refused instead of being run as this one; an unknown key at the top (a seed, a name) is named on standard error and
ignored.  Whether a layer without a feed-forward still has its second norm is read from the weight files (the tensor
``l<i>.norm2``).
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, RawConfig

DEFAULT_MAX_POSITIONS = 131072

_ROT_KEYS = {"base", "dims", "scaling"}
_SCALING_KEYS = {"factor", "original", "fast", "slow"}
MIXER_KEYS = {
    "attention": ({"heads", "kv_heads", "dim", "vdim", "scale"}, {"rot", "mask", "kv_from"}),
    "retention": ({"heads", "dim", "vdim", "decay"}, {"rot"}),
    "mamba2": ({"heads", "vdim", "state", "groups", "conv", "norm_groups"}, set()),
}


def _freeze(v):
    """Lists and objects of config.json as tuples, so that a configuration can be compared and hashed."""
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    if isinstance(v, list):
        return tuple(_freeze(x) for x in v)
    return v


def _thaw(v):
    if isinstance(v, tuple) and all(isinstance(x, tuple) and len(x) == 2 and isinstance(x[0], str) for x in v) and v:
        return {k: _thaw(x) for k, x in v}
    return v


@dataclass(frozen=True)
class TikizenLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]        # the mixer's sizes and constants, as sorted (key, value) pairs
    mlp: Optional[Tuple[Tuple[str, Any], ...]]    # the feed-forward's; None: the layer has none
    bare_norm2: bool = False                  # no feed-forward, but the second norm is there (from the weight files)

    def get(self, key: str, default=None):
        v = dict(self.mixer).get(key, default)
        return _thaw(v)

    def mlp_get(self, key: str, default=None):
        return None if self.mlp is None else _thaw(dict(self.mlp).get(key, default))


@dataclass(frozen=True)
class TikizenConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    residual_scale: float
    layers: Tuple[TikizenLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "TikizenConfig":
        src = raw.source
        known = {"architecture", "architectures", "model_type", "vocab", "width", "max_positions", "norm",
                 "postln_alpha", "layers", "eos_token_id"}
        extra = sorted(k for k in raw.values if k not in known)
        if extra:
            print(f"[inferrs_b200] {src}: keys {extra} are not part of a Tikizen configuration and are ignored",
                  file=sys.stderr)
        missing = [k for k in ("vocab", "width", "norm", "postln_alpha", "layers") if not raw.has(k)]
        if missing:
            raise ConfigError(f"{src}: Tikizen config lacks the keys {missing}")
        vocab, width = raw.get_int("vocab"), raw.get_int("width")
        max_positions = raw.get_int("max_positions", DEFAULT_MAX_POSITIONS)
        for k, v in (("vocab", vocab), ("width", width), ("max_positions", max_positions)):
            if v <= 0:
                raise ConfigError(f"{src}: key '{k}' must be positive, got {v}")
        norm = raw.values["norm"]
        if not isinstance(norm, dict) or set(norm) != {"eps"}:
            raise ConfigError(f"{src}: key 'norm' must be an object with 'eps', got {norm!r}")
        eps = _number(src, "norm.eps", norm["eps"], float)
        alpha = raw.get_float("postln_alpha")
        if eps <= 0 or not alpha > 0:
            raise ConfigError(f"{src}: norm.eps and postln_alpha must be positive, got {eps}, {alpha}")
        layers_raw = raw.get_list("layers")
        if not layers_raw:
            raise ConfigError(f"{src}: key 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or set(entry) - {"type", "mixer", "mlp"} or "type" not in entry \
                    or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"{src}: {where} must be an object with 'type', 'mixer' and 'mlp', got {entry!r}")
            kind = entry["type"]
            if kind not in MIXER_KEYS:
                raise ConfigError(f"{src}: {where}.type '{kind}' is not one of {sorted(MIXER_KEYS)}")
            mixer = _check_mixer(src, where, kind, entry["mixer"], layers, i)
            mlp = _check_mlp(src, where, entry.get("mlp"))
            layers.append(TikizenLayer(type=kind, mixer=_freeze(mixer), mlp=None if mlp is None else _freeze(mlp)))
        eos = raw.values.get("eos_token_id")
        eos_ids = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        if any(isinstance(t, bool) or not isinstance(t, int) or not 0 <= t < vocab for t in eos_ids):
            raise ConfigError(f"{src}: eos_token_id must be token ids inside the vocabulary, got {eos!r}")
        return cls(vocab=vocab, width=width, max_positions=max_positions, norm_eps=eps, residual_scale=float(alpha),
                   layers=tuple(layers), eos_token_ids=eos_ids)

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "TikizenConfig":
        """The configuration with what only the weight files say: whether a layer without a feed-forward keeps its
        second norm."""
        layers = list(self.layers)
        for i, layer in enumerate(layers):
            if layer.mlp is None and f"l{i}.norm2" in shapes:
                layers[i] = TikizenLayer(type=layer.type, mixer=layer.mixer, mlp=None, bare_norm2=True)
        return TikizenConfig(**{**self.__dict__, "layers": tuple(layers)})


def _check_rot(src: str, where: str, rot, key_dim: int):
    if rot is None:
        return
    if not isinstance(rot, dict) or set(rot) - _ROT_KEYS or not {"base", "dims"} <= set(rot):
        raise ConfigError(f"{src}: {where}.rot must be an object with 'base', 'dims' (and 'scaling'), got {rot!r}")
    dims = _number(src, f"{where}.rot.dims", rot["dims"], int)
    base = _number(src, f"{where}.rot.base", rot["base"], float)
    if dims <= 0 or dims % 2 or dims > key_dim or not base > 1:
        raise ConfigError(f"{src}: {where}.rot.dims must be even, positive and at most dim={key_dim}, and rot.base "
                          f"above 1; got {dims}, {base}")
    sc = rot.get("scaling")
    if sc is not None:
        if not isinstance(sc, dict) or set(sc) != _SCALING_KEYS:
            raise ConfigError(f"{src}: {where}.rot.scaling must be an object with {sorted(_SCALING_KEYS)}, got {sc!r}")
        for k in _SCALING_KEYS:
            if not _number(src, f"{where}.rot.scaling.{k}", sc[k], float) > 0:
                raise ConfigError(f"{src}: {where}.rot.scaling.{k} must be positive, got {sc[k]!r}")


def _check_mixer(src: str, where: str, kind: str, given: Dict[str, Any], layers, i: int) -> Dict[str, Any]:
    need, optional = MIXER_KEYS[kind]
    bad = sorted(set(given) - need - optional) + sorted(k for k in need if given.get(k) is None)
    if bad:
        raise ConfigError(f"{src}: {where}.mixer of type '{kind}' has unknown or missing keys {bad}")
    out = {k: v for k, v in given.items() if v is not None}
    for k in need - {"scale", "decay"}:
        if _number(src, f"{where}.mixer.{k}", out[k], int) <= 0:
            raise ConfigError(f"{src}: {where}.mixer.{k} must be positive, got {out[k]!r}")
    if kind == "attention":
        if not _number(src, f"{where}.mixer.scale", out["scale"], float) > 0:
            raise ConfigError(f"{src}: {where}.mixer.scale must be positive, got {out['scale']!r}")
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"{src}: {where}.mixer: {out['heads']} heads are not a multiple of {out['kv_heads']} "
                              f"kv_heads")
        _check_rot(src, f"{where}.mixer", out.get("rot"), out["dim"])
        mask = out.get("mask")
        if mask is not None and (not isinstance(mask, dict) or set(mask) != {"size"}
                                 or _number(src, f"{where}.mixer.mask.size", mask["size"], int) <= 0):
            raise ConfigError(f"{src}: {where}.mixer.mask must be an object with a positive 'size', got {mask!r}")
        if "kv_from" in out:
            j = _number(src, f"{where}.mixer.kv_from", out["kv_from"], int)
            same = ("kv_heads", "dim", "vdim", "rot")
            if not 0 <= j < i or layers[j].type != "attention" or layers[j].get("kv_from") is not None \
                    or any(layers[j].get(k) != out.get(k) for k in same):
                raise ConfigError(f"{src}: {where}.mixer.kv_from must name an earlier attention layer with keys and "
                                  f"values of its own and the same kv_heads, dim, vdim and rot, got {j}")
    elif kind == "retention":
        decay = out["decay"]
        if not isinstance(decay, list) or len(decay) != out["heads"] \
                or any(not 0 < _number(src, f"{where}.mixer.decay", a, float) <= 1 for a in decay):
            raise ConfigError(f"{src}: {where}.mixer.decay must list one decay in (0, 1] per head, got {decay!r}")
        _check_rot(src, f"{where}.mixer", out.get("rot"), out["dim"])
    else:
        if out["heads"] % out["groups"] or (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise ConfigError(f"{src}: {where}.mixer: heads must divide into groups and heads * vdim into norm_groups")
    return out


def _check_mlp(src: str, where: str, mlp) -> Optional[Dict[str, Any]]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{src}: {where}.mlp must be null or an object of kind 'dense' or 'moe', got {mlp!r}")
    if mlp["kind"] == "dense":
        if set(mlp) != {"kind", "ff", "limit"} or _number(src, f"{where}.mlp.ff", mlp["ff"], int) <= 0 \
                or not _number(src, f"{where}.mlp.limit", mlp["limit"], float) > 0:
            raise ConfigError(f"{src}: {where}.mlp of kind 'dense' has a positive 'ff' and 'limit', got {mlp!r}")
        return dict(mlp)
    if set(mlp) - {"kind", "expert", "router", "shared"} or not {"expert", "router"} <= set(mlp):
        raise ConfigError(f"{src}: {where}.mlp of kind 'moe' has 'expert', 'router' (and 'shared'), got {mlp!r}")
    expert, router, shared = mlp["expert"], mlp["router"], mlp.get("shared")
    if not isinstance(expert, dict) or set(expert) != {"ff"} or _number(src, f"{where}.mlp.expert.ff", expert["ff"], int) <= 0:
        raise ConfigError(f"{src}: {where}.mlp.expert must be an object with a positive 'ff', got {expert!r}")
    if not isinstance(router, dict) or set(router) != {"experts", "top"} \
            or not 0 < _number(src, f"{where}.mlp.router.top", router["top"], int) \
            <= _number(src, f"{where}.mlp.router.experts", router["experts"], int):
        raise ConfigError(f"{src}: {where}.mlp.router must give 'experts' and 'top' with 0 < top <= experts, got "
                          f"{router!r}")
    if shared is not None and (not isinstance(shared, dict) or set(shared) != {"ff"}
                               or _number(src, f"{where}.mlp.shared.ff", shared["ff"], int) <= 0):
        raise ConfigError(f"{src}: {where}.mlp.shared must be an object with a positive 'ff', got {shared!r}")
    return {k: v for k, v in mlp.items() if v is not None}


def _number(src: str, key: str, v, kind):
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and not isinstance(v, int)):
        raise ConfigError(f"{src}: key '{key}' must be {'an integer' if kind is int else 'a number'}, got {v!r}")
    return kind(v)
