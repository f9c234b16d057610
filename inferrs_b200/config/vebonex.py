"""Typed configuration of the Vebonex decoder.

config.json gives every size and every constant that differs between models of the design:

    architecture   "Vebonex"
    vocab, width, max_positions
    norm           {"eps": ..., "groups": ...}: every norm of the model, in that many equal parts of the row
    streams        width of the residual in streams (hyper-connections); absent: the plain residual
    layers         a list; every entry has "type" (which mixer), "mixer" (its sizes and constants) and "mlp"
                   ({"kind": "dense", "ff": ...}, or null for a layer without a feed-forward)

One size is given by a tensor's shape and not by config.json: the inner size of the two small products that make a
gated-linear-attention layer's decay (the rows of ``l<i>.mix.a1``).  :meth:`VebonexConfig.with_tensor_shapes` takes it
from the weight files' headers; a configuration without weight files (random weights) gives it as ``mixer.a_rank``.

A key that the chosen mixer needs and that is absent is an error: no size stands in code.  Keys that this reader
does not know inside `norm`, a layer, its mixer or its feed-forward are an error too, so that a variant of the design
is refused instead of being run as this one; an unknown key at the top (a seed, a name) is named on standard error
and ignored.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, RawConfig

MIXER_KEYS = {
    "gla": {"heads": int, "dim": int, "vdim": int, "tau": float},
    "mlstm": {"heads": int, "dim": int, "vdim": int, "gate_cap": float},
    "latent_attention": {"heads": int, "dim": int, "vdim": int, "q_rank": int, "kv_rank": int, "scale": float},
}
MIXER_OPTIONAL = {"gla": {"a_rank": int}, "mlstm": {}, "latent_attention": {"kv_from": int}}


@dataclass(frozen=True)
class VebonexLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]        # the mixer's sizes and constants, as sorted (key, value) pairs
    ff: Optional[int]                         # inner size of the dense feed-forward; None: the layer has none

    def get(self, key: str, default=None):
        return dict(self.mixer).get(key, default)


@dataclass(frozen=True)
class VebonexConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    norm_groups: int
    streams: Optional[int]
    layers: Tuple[VebonexLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "VebonexConfig":
        src = raw.source
        known = {"architecture", "architectures", "model_type", "vocab", "width", "max_positions", "norm", "streams",
                 "layers", "eos_token_id"}
        extra = sorted(k for k in raw.values if k not in known)
        if extra:
            # a key beside the model's own (a seed, a name, a storage dtype) changes no arithmetic that this reader
            # knows of: it is named and left alone.  Unknown keys inside 'norm', a layer, its mixer or its feed-forward
            # are refused below, since those are where a variant of the design would say what it does differently.
            print(f"[inferrs_b200] {src}: keys {extra} are not part of a Vebonex configuration and are ignored",
                  file=sys.stderr)
        missing = [k for k in ("vocab", "width", "max_positions", "norm", "layers") if not raw.has(k)]
        if missing:
            raise ConfigError(f"{src}: Vebonex config lacks the keys {missing}")
        ints = {k: raw.get_int(k) for k in ("vocab", "width", "max_positions")}
        for k, v in ints.items():
            if v <= 0:
                raise ConfigError(f"{src}: key '{k}' must be positive, got {v}")
        norm = raw.values["norm"]
        if not isinstance(norm, dict) or set(norm) - {"eps", "groups"} or "eps" not in norm:
            raise ConfigError(f"{src}: key 'norm' must be an object with 'eps' and 'groups', got {norm!r}")
        eps, groups = _number(src, "norm.eps", norm["eps"], float), _number(src, "norm.groups", norm.get("groups", 1), int)
        if eps <= 0 or groups <= 0 or ints["width"] % groups:
            raise ConfigError(f"{src}: norm.eps must be positive and norm.groups a divisor of width {ints['width']}")
        streams = raw.get_int("streams")
        if streams is not None and streams <= 0:
            raise ConfigError(f"{src}: key 'streams' must be positive, got {streams}")
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
            need, optional = MIXER_KEYS[kind], MIXER_OPTIONAL[kind]
            given: Dict[str, Any] = entry["mixer"]
            bad = sorted(set(given) - set(need) - set(optional)) + sorted(k for k in need if k not in given)
            if bad:
                raise ConfigError(f"{src}: {where}.mixer of type '{kind}' has unknown or missing keys {bad}")
            values = {}
            for k, v in given.items():
                if v is None and k in optional:
                    continue
                values[k] = _number(src, f"{where}.mixer.{k}", v, {**need, **optional}[k])
                if k != "kv_from" and values[k] <= 0:
                    raise ConfigError(f"{src}: {where}.mixer.{k} must be positive, got {v!r}")
            if "kv_from" in values:
                j = values["kv_from"]
                if not 0 <= j < i or layers[j].type != "latent_attention" or layers[j].get("kv_from") is not None \
                        or layers[j].get("kv_rank") != values["kv_rank"]:
                    raise ConfigError(f"{src}: {where}.mixer.kv_from must name an earlier latent-attention layer with "
                                      f"latents of its own and the same kv_rank, got {j}")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or set(mlp) != {"kind", "ff"} or mlp["kind"] != "dense":
                    raise ConfigError(f"{src}: {where}.mlp must be null or {{'kind': 'dense', 'ff': n}}, got {mlp!r}")
                ff = _number(src, f"{where}.mlp.ff", mlp["ff"], int)
                if ff <= 0:
                    raise ConfigError(f"{src}: {where}.mlp.ff must be positive, got {ff}")
            layers.append(VebonexLayer(type=kind, mixer=tuple(sorted(values.items())), ff=ff))
        eos = raw.values.get("eos_token_id")
        eos_ids = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        if any(isinstance(t, bool) or not isinstance(t, int) or not 0 <= t < ints["vocab"] for t in eos_ids):
            raise ConfigError(f"{src}: eos_token_id must be token ids inside the vocabulary, got {eos!r}")
        return cls(vocab=ints["vocab"], width=ints["width"], max_positions=ints["max_positions"], norm_eps=eps,
                   norm_groups=groups, streams=streams, layers=tuple(layers), eos_token_ids=eos_ids)

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "VebonexConfig":
        """The configuration with the sizes that only the weight files give, read from their tensors' shapes."""
        layers = list(self.layers)
        for i, layer in enumerate(layers):
            shape = shapes.get(f"l{i}.mix.a1")
            if layer.type == "gla" and shape is not None and len(shape) == 2:
                layers[i] = _with_rank(layer, shape[0])
        return VebonexConfig(**{**self.__dict__, "layers": tuple(layers)})


def _with_rank(layer: VebonexLayer, rank: int) -> VebonexLayer:
    values = dict(layer.mixer)
    values["a_rank"] = int(rank)
    return VebonexLayer(type=layer.type, mixer=tuple(sorted(values.items())), ff=layer.ff)


def _number(src: str, key: str, v, kind):
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and not isinstance(v, int)):
        raise ConfigError(f"{src}: key '{key}' must be {'an integer' if kind is int else 'a number'}, got {v!r}")
    return kind(v)
