"""Small Vebonex configurations and weights for the tests: sizes that differ from one another in every field, among
them values that make mechanisms degenerate (one stream, one group, one head, a layer without a feed-forward, a
model without any cache of latents, a model without hyper-connections)."""
from __future__ import annotations

from typing import Dict

import torch

from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import declared_tensors


def _latent(heads, dim, vdim, q_rank, kv_rank, scale, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _ff(n):
    return None if n is None else {"kind": "dense", "ff": n}


# three streams, norms in three parts, every mixer, a layer that reads another's latents, two sizes of latent
CASE_P = {
    "architecture": "Vebonex", "vocab": 211, "width": 96, "max_positions": 320, "streams": 3,
    "norm": {"eps": 1e-6, "groups": 3},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 24, 20, 40, 36, 0.2), "mlp": _ff(136)},
        {"type": "gla", "mixer": {"heads": 3, "dim": 40, "vdim": 20, "tau": 8.0, "a_rank": 8}, "mlp": None},
        {"type": "latent_attention", "mixer": _latent(2, 16, 28, 24, 36, 0.25, kv_from=0), "mlp": _ff(72)},
        {"type": "mlstm", "mixer": {"heads": 1, "dim": 72, "vdim": 36, "gate_cap": 8.0}, "mlp": _ff(136)},
        {"type": "latent_attention", "mixer": _latent(4, 8, 12, 16, 70, 0.35), "mlp": None},
    ],
}
# one stream (the connections are single numbers), one group, recurrent mixers only: no paged cache at all
CASE_Q = {
    "architecture": "Vebonex", "vocab": 97, "width": 64, "max_positions": 256, "streams": 1,
    "norm": {"eps": 1e-5, "groups": 1},
    "layers": [
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 32, "vdim": 30, "gate_cap": 20.0}, "mlp": _ff(80)},
        {"type": "gla", "mixer": {"heads": 1, "dim": 16, "vdim": 64, "tau": 2.0, "a_rank": 4}, "mlp": _ff(48)},
    ],
}
# no hyper-connections (the plain residual), norms in two parts, many heads on one latent whose size the tensor-core
# form of the latent attention takes
CASE_R = {
    "architecture": "Vebonex", "vocab": 130, "width": 128, "max_positions": 512,
    "norm": {"eps": 1e-5, "groups": 2},
    "layers": [
        {"type": "gla", "mixer": {"heads": 2, "dim": 64, "vdim": 64, "tau": 32.0, "a_rank": 16}, "mlp": _ff(192)},
        {"type": "latent_attention", "mixer": _latent(18, 16, 8, 32, 64, 0.25), "mlp": _ff(192)},
    ],
}
# sizes that no vector load, tensor-core tile or 16-byte copy takes: a width of 90 in three parts, one head everywhere,
# inner sizes of 3 and 50
CASE_S = {
    "architecture": "Vebonex", "vocab": 77, "width": 90, "max_positions": 300, "streams": 3,
    "norm": {"eps": 1e-5, "groups": 3},
    "layers": [
        {"type": "mlstm", "mixer": {"heads": 1, "dim": 24, "vdim": 10, "gate_cap": 9.0}, "mlp": _ff(50)},
        {"type": "latent_attention", "mixer": _latent(1, 24, 10, 12, 20, 0.3), "mlp": _ff(50)},
        {"type": "gla", "mixer": {"heads": 1, "dim": 10, "vdim": 7, "tau": 3.0, "a_rank": 3}, "mlp": None},
    ],
}
CASES = {"P": CASE_P, "Q": CASE_Q, "R": CASE_R, "S": CASE_S}


def make_weights(config: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Weights of a size that keeps activations near one, so that every mechanism moves the logits: matrices N(0, 1 /
    fan-in), norm weights near one, gate biases that let the states live for tens of tokens.  Rounded to bfloat16
    (returned as float32 on the host), so that both run dtypes and the plain statement start from the same numbers."""
    spec, _ = spec_from_config(config)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for d in declared_tensors(spec):
        n = d.name
        r = torch.randn(d.shape, generator=g)
        if n in ("embed", "pos"):
            t = r * (1.0 if n == "embed" else 0.5)
        elif n.endswith(".hc1.mix") or n.endswith(".hc2.mix"):
            t = torch.eye(d.shape[0]) + 0.25 * r
        elif n.endswith(".in"):
            t = 1.0 / d.shape[0] + 0.25 * r
        elif n.endswith(".out"):
            t = 1.0 + 0.25 * r
        elif n.endswith(".act"):
            t = 0.6 * r + torch.tensor([0.5, 0.3, 0.2, 0.0])
        elif n.endswith(".a2.b") or n.endswith(".f.b"):
            t = 2.5 + 1.5 * r
        elif n.endswith(".i.b"):
            t = 1.0 * r
        elif len(d.shape) == 1:            # norm weights
            t = 1.0 + 0.2 * r
        elif n.endswith(".mix.i") or n.endswith(".mix.f") or n.endswith(".mix.a2"):
            t = r * (3.0 / d.shape[1] ** 0.5)     # gates that move with the input
        else:
            t = r * (1.0 / d.shape[1] ** 0.5)
        out[n] = t.to(torch.bfloat16).to(torch.float32)
    return out
