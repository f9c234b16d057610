"""Mixers that carry a matrix state per head from token to token instead of a cache of keys and values.

Both keep, per request, a float32 state of fixed size in the cache's state slots (one slot per live request, zeroed
when a request takes it) and walk a request's rows in order inside one kernel, so a prompt may be cut anywhere and
a portion may stand beside single tokens of other requests.

Every size is a field of the description; the parts do not know which model or which layer they are in.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.storage import StateNeed
from ..runtime import Runtime
from .basic import Linear, fuse_rows
from .registry import register_mixer
from .spec import ChannelDecayScanSpec, ScalarGateScanSpec, TensorDecl


class _ScanMixer:
    """What the two scans share: the fused q/k/v/gate projection, the state, the norm-and-gate step, the output."""

    graph_safe = True  # launches depend only on shapes, never on the step's host-side values

    @staticmethod
    def cache_need(spec):
        return None

    def _build(self, spec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec, self.rt = spec, rt
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        self.qkvg = Linear(fuse_rows([weights[spec.q_proj], weights[spec.k_proj], weights[spec.v_proj],
                                      weights[spec.gate_proj]]), rt)
        self.cols = (0, hd, 2 * hd, 2 * hd + he)         # where q, k, v and the gate start in a projected row
        self.o = Linear(weights[spec.o_proj], rt)
        self.out_norm = weights[spec.out_norm]

    def _run(self, ctx, cache_id: int, h, mode: int, gates: torch.Tensor, gate_bias: torch.Tensor, gate_param: float,
             gate_act: int):
        s = self.spec
        n = h.shape[0]
        proj = self.qkvg(h)
        o = torch.empty((n, s.n_heads, s.value_dim), dtype=torch.float32, device=h.device)
        kernels.linear_scan(mode, proj, self.cols[0], self.cols[1], self.cols[2], gates, gate_bias, gate_param,
                            float(s.key_dim) ** -0.5, ctx.storage.state(cache_id), ctx.q_start, ctx.slots,
                            ctx.n_requests, o, s.key_dim, max_rows=ctx.max_q_len)
        gated = torch.empty((n, s.n_heads * s.value_dim), dtype=self.rt.dtype, device=h.device)
        kernels.head_norm_gate(o, proj[:, self.cols[3]:], self.out_norm, True, gate_act, s.eps, gated)
        return self.o(gated)


class ChannelDecayScan(_ScanMixer):
    """Gated linear attention (see :class:`~inferrs_b200.parts.spec.ChannelDecayScanSpec`).  The decay's
    pre-activations come out of their two small products in float32; sigmoid, the root of order tau and the
    recurrence are float32 inside the scan kernel."""

    @staticmethod
    def declare(spec: ChannelDecayScanSpec) -> List[TensorDecl]:
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        return [TensorDecl(spec.q_proj, (hd, spec.width)), TensorDecl(spec.k_proj, (hd, spec.width)),
                TensorDecl(spec.v_proj, (he, spec.width)), TensorDecl(spec.gate_proj, (he, spec.width)),
                TensorDecl(spec.o_proj, (spec.width, he)), TensorDecl(spec.out_norm, (spec.value_dim,), init="norm"),
                TensorDecl(spec.decay_down, (spec.decay_rank, spec.width)),
                TensorDecl(spec.decay_up, (hd, spec.decay_rank)),
                TensorDecl(spec.decay_bias, (hd,), init="uniform:3:2")]

    @staticmethod
    def state_need(spec: ChannelDecayScanSpec) -> Optional[StateNeed]:
        return StateNeed(shape=(spec.n_heads * spec.key_dim * spec.value_dim,))

    def __init__(self, spec: ChannelDecayScanSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.tau <= 0:
            raise ValueError(f"the decay's root must be positive, got tau={spec.tau}")
        self._build(spec, weights, rt)
        self.decay_down = Linear(weights[spec.decay_down], rt)
        self.decay_up = Linear(weights[spec.decay_up], rt)
        self.decay_bias = weights[spec.decay_bias].to(torch.float32).contiguous()

    def forward(self, ctx, cache_id: int, h):
        z = self.decay_up(self.decay_down(h), out_dtype=torch.float32)
        return self._run(ctx, cache_id, h, kernels.SCAN_CHANNEL_DECAY, z, self.decay_bias, self.spec.tau,
                         kernels.GATE_SILU)


class ScalarGateScan(_ScanMixer):
    """The matrix memory of xLSTM (see :class:`~inferrs_b200.parts.spec.ScalarGateScanSpec`).  The two gates'
    pre-activations come out of one small product in float32; the caps, the running maximum and the recurrence are
    float32 inside the scan kernel."""

    @staticmethod
    def declare(spec: ScalarGateScanSpec) -> List[TensorDecl]:
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        return [TensorDecl(spec.q_proj, (hd, spec.width)), TensorDecl(spec.k_proj, (hd, spec.width)),
                TensorDecl(spec.v_proj, (he, spec.width)), TensorDecl(spec.gate_proj, (he, spec.width)),
                TensorDecl(spec.o_proj, (spec.width, he)), TensorDecl(spec.out_norm, (he,), init="norm"),
                TensorDecl(spec.i_proj, (spec.n_heads, spec.width)),
                TensorDecl(spec.i_bias, (spec.n_heads,), init="uniform:0:1"),
                TensorDecl(spec.f_proj, (spec.n_heads, spec.width)),
                TensorDecl(spec.f_bias, (spec.n_heads,), init="uniform:3:2")]

    @staticmethod
    def state_need(spec: ScalarGateScanSpec) -> Optional[StateNeed]:
        h, d, e = spec.n_heads, spec.key_dim, spec.value_dim
        return StateNeed(shape=(h * d * e + h * d + h,))     # the matrices, the vectors n, the maxima m

    def __init__(self, spec: ScalarGateScanSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.gate_cap <= 0:
            raise ValueError(f"the gates' cap must be positive, got {spec.gate_cap}")
        self._build(spec, weights, rt)
        self.gates = Linear(fuse_rows([weights[spec.i_proj], weights[spec.f_proj]]), rt)
        self.gate_bias = torch.cat([weights[spec.i_bias].to(torch.float32),
                                    weights[spec.f_bias].to(torch.float32)]).contiguous()

    def forward(self, ctx, cache_id: int, h):
        pre = self.gates(h, out_dtype=torch.float32)
        return self._run(ctx, cache_id, h, kernels.SCAN_SCALAR_GATES, pre, self.gate_bias, self.spec.gate_cap,
                         kernels.GATE_SIGMOID)


register_mixer("channel_decay_scan", ChannelDecayScan)
register_mixer("scalar_gate_scan", ScalarGateScan)
