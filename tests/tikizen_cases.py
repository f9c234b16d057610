"""Small Tikizen configurations and weights for the tests: sizes that differ from one another in every field, among
them values that make mechanisms degenerate (one head, one group, one tap, one expert of one, no shared expert, a
layer without a feed-forward, no chunks, no stretched rotation, a rotation of part of a head, values larger and
smaller than keys)."""
from __future__ import annotations

from typing import Dict

import torch

from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import declared_tensors


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _att(heads, kv_heads, dim, vdim, scale, rot, chunk=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(ff, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


# every mixer; chunks of 40 (no multiple of a page); values smaller than keys; a layer on another's keys and values;
# a rotation of part of a head with stretched slow pairs; both feed-forwards
CASE_P = {
    "architecture": "Tikizen", "vocab": 211, "width": 96, "norm": {"eps": 1e-6}, "postln_alpha": 1.7,
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 24, 20, 0.3, _rot(10000.0, 16, (8.0, 64, 16.0, 2.0)), chunk=40),
         "mlp": _dense(136, 2.0)},
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 12, "state": 20, "groups": 2, "conv": 4, "norm_groups": 3},
         "mlp": _moe(24, 5, 2, shared=40)},
        {"type": "attention", "mixer": _att(4, 2, 24, 20, 0.2, _rot(10000.0, 16, (8.0, 64, 16.0, 2.0)), chunk=24,
                                           kv_from=0), "mlp": None},
        {"type": "retention", "mixer": {"heads": 3, "dim": 40, "vdim": 24, "decay": [0.9, 0.97, 0.995],
                                        "rot": _rot(500.0, 24)}, "mlp": _moe(16, 3, 3)},
    ],
}
# recurrent mixers only (no paged cache at all); one group, one tap, one norm part, one head; top 1
CASE_Q = {
    "architecture": "Tikizen", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 1.0,
    "layers": [
        {"type": "mamba2", "mixer": {"heads": 2, "vdim": 30, "state": 16, "groups": 1, "conv": 1, "norm_groups": 1},
         "mlp": _moe(20, 4, 1)},
        {"type": "retention", "mixer": {"heads": 1, "dim": 16, "vdim": 64, "decay": [0.98]},      # no rotation
         "mlp": _dense(48, 0.7)},
        {"type": "mamba2", "mixer": {"heads": 3, "vdim": 8, "state": 36, "groups": 3, "conv": 2, "norm_groups": 2},
         "mlp": None},
    ],
}
# head sizes that the tensor-core attention kernels of the bfloat16 build take (128 and 64), with chunks; no chunks
# and no stretch in the last layer; values larger than keys
CASE_R = {
    "architecture": "Tikizen", "vocab": 130, "width": 128, "norm": {"eps": 1e-5}, "postln_alpha": 2.5,
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 128, 128, 0.09, _rot(1000000.0, 128, (4.0, 48, 32.0, 1.0)), chunk=56),
         "mlp": _moe(32, 8, 4, shared=48)},
        {"type": "attention", "mixer": _att(6, 1, 64, 64, 0.125, _rot(10000.0, 32), chunk=48), "mlp": _dense(96, 1.5)},
        {"type": "attention", "mixer": _att(2, 2, 32, 48, 0.2, _rot(10000.0, 32)), "mlp": None},
    ],
}
# sizes that no vector load, tensor-core tile or 16-byte copy takes
CASE_S = {
    "architecture": "Tikizen", "vocab": 77, "width": 90, "norm": {"eps": 1e-5}, "postln_alpha": 0.8,
    "layers": [
        {"type": "retention", "mixer": {"heads": 1, "dim": 10, "vdim": 7, "decay": [1.0], "rot": _rot(50.0, 6)},
         "mlp": _moe(9, 2, 1, shared=5)},
        {"type": "attention", "mixer": _att(3, 3, 10, 7, 0.4, None, chunk=7), "mlp": _dense(50, 1.0)},
        {"type": "mamba2", "mixer": {"heads": 1, "vdim": 9, "state": 5, "groups": 1, "conv": 3, "norm_groups": 1},
         "mlp": None},
    ],
}
CASES = {"P": CASE_P, "Q": CASE_Q, "R": CASE_R, "S": CASE_S}


def for_dtype(config: dict, dtype) -> dict:
    """The configuration as the tests of a run dtype use it.  In bfloat16 a router that chooses one expert alone is
    given two: where two logits are closer than bfloat16 tells apart the other expert is chosen, the whole output of
    the feed-forward changes, and a mixer's state carries the difference to every later token, so such a model cannot
    be compared with the plain statement token by token.  float32 runs keep the single choice."""
    if dtype != torch.bfloat16:
        return config
    import copy
    out = copy.deepcopy(config)
    for layer in out["layers"]:
        mlp = layer.get("mlp")
        if mlp and mlp.get("kind") == "moe" and mlp["router"]["top"] == 1 and mlp["router"]["experts"] > 1:
            mlp["router"]["top"] = 2
    return out


def make_weights(config: dict, seed: int, bare_norm2: bool = False) -> Dict[str, torch.Tensor]:
    """Weights of a size that keeps activations near one, so that every mechanism moves the logits: matrices N(0, 1 /
    fan-in), norm weights near one, step sizes and decays that let the states live for tens of tokens, router biases
    that do not decide the choice alone.  Rounded to bfloat16 (returned as float32 on the host), so that both run
    dtypes and the plain statement start from the same numbers.  ``bare_norm2``: layers without a feed-forward get
    their second norm all the same."""
    shapes = None
    if bare_norm2:
        shapes = {f"l{i}.norm2": (config["width"],) for i, l in enumerate(config["layers"]) if l.get("mlp") is None}
    spec, _ = spec_from_config(config, tensor_shapes=shapes)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for d in declared_tensors(spec):
        n = d.name
        r = torch.randn(d.shape, generator=g)
        if n == "embed":
            t = r
        elif n.endswith(".dt_bias"):
            t = -1.5 + 0.7 * r
        elif n.endswith(".A_log"):
            t = -0.5 + 0.7 * r
        elif n.endswith(".mix.D"):
            t = 1.0 + 0.3 * r
        elif n.endswith(".conv"):
            t = r * (1.0 / d.shape[1] ** 0.5)
        elif n.endswith(".conv.b") or n.endswith(".router.b"):
            t = 0.3 * r
        elif len(d.shape) == 1:            # norm weights
            t = 1.0 + 0.2 * r
        elif n.endswith(".router") or n.endswith(".shared.sg"):
            t = r * (3.0 / d.shape[1] ** 0.5)     # choices that move with the input
        else:
            t = r * (1.0 / d.shape[1] ** 0.5)
        out[n] = t.to(torch.bfloat16).to(torch.float32)
    return out
