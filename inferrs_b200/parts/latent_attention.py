"""Attention over a paged cache of latents: one vector per token from which every head makes its key and value.

The cache holds only the latent c (one plane of pages, ``kv_rank`` numbers per token).  The heads' key and value
matrices are not applied to the cached tokens but to the query and to the result:

    score_h(i, j) = q_h(i) . (K_h c_j) = (K_h^T q_h(i)) . c_j          out_h(i) = V_h sum_j p_h(i, j) c_j

so a step costs two batched products per layer (one per head with the step's rows) and the attention kernel reads
each cached latent once for all heads, as key and as value.  A layer may read the latents that another layer
writes (``own_kv=False``) with key and value matrices of its own.

Every size is a field of the description; the part does not know which model or which layer it is in.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.storage import KVNeed
from ..runtime import Runtime
from .basic import Linear, fuse_rows
from .registry import register_mixer
from .spec import LatentAttentionSpec, TensorDecl


class LatentAttention:
    graph_safe = True  # launches depend only on shapes, never on the step's host-side values

    @staticmethod
    def declare(spec: LatentAttentionSpec) -> List[TensorDecl]:
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        d = [TensorDecl(spec.dq_proj, (spec.q_rank, spec.width)),
             TensorDecl(spec.dq_norm, (spec.q_rank,), init="norm"),
             TensorDecl(spec.uq_proj, (hd, spec.q_rank)),
             TensorDecl(spec.uk_proj, (hd, spec.kv_rank)),
             TensorDecl(spec.uv_proj, (he, spec.kv_rank)),
             TensorDecl(spec.gate_proj, (he, spec.width)),
             TensorDecl(spec.o_proj, (spec.width, he))]
        if spec.own_kv:
            d += [TensorDecl(spec.dkv_proj, (spec.kv_rank, spec.width)),
                  TensorDecl(spec.dkv_norm, (spec.kv_rank,), init="norm")]
        return d

    @staticmethod
    def cache_need(spec: LatentAttentionSpec) -> Optional[KVNeed]:
        # one plane: the latent is key and value at once
        return KVNeed(n_kv_heads=1, head_dim=spec.kv_rank, window=spec.window, planes=1)

    @staticmethod
    def state_need(spec: LatentAttentionSpec):
        return None

    @staticmethod
    def writes_cache(spec: LatentAttentionSpec) -> bool:
        return spec.own_kv

    def __init__(self, spec: LatentAttentionSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.own_kv and (spec.dkv_proj is None or spec.dkv_norm is None):
            raise ValueError("a latent-attention layer with latents of its own needs dkv_proj and dkv_norm")
        self.spec, self.rt = spec, rt
        h, d, e, r = spec.n_heads, spec.key_dim, spec.value_dim, spec.kv_rank
        mats = [weights[spec.dq_proj]] + ([weights[spec.dkv_proj]] if spec.own_kv else []) + [weights[spec.gate_proj]]
        self.down = Linear(fuse_rows(mats), rt)          # query latent, key/value latent, gate: one product
        self.kv_col = spec.q_rank
        self.gate_col = spec.q_rank + (r if spec.own_kv else 0)
        self.q_norm = weights[spec.dq_norm]
        self.kv_norm = weights[spec.dkv_norm] if spec.own_kv else None
        if self.kv_norm is not None and self.kv_norm.dtype != self.q_norm.dtype:
            self.q_norm, self.kv_norm = self.q_norm.float(), self.kv_norm.float()
        self.uq = Linear(weights[spec.uq_proj], rt)
        # per head: K_h^T as the matrix of a product "query times weight transposed" [H, R, D], V_h as it is [H, E, R]
        self.uk_t = weights[spec.uk_proj].reshape(h, d, r).transpose(1, 2).contiguous()
        self.uv = weights[spec.uv_proj].reshape(h, e, r).contiguous()
        self.o = Linear(weights[spec.o_proj], rt)

    def forward(self, ctx, cache_id: int, x):
        s = self.spec
        n, h = x.shape[0], s.n_heads
        dev, act = x.device, self.rt.dtype
        proj = self.down(x)
        k_pages, _v, group = ctx.storage.pages(cache_id)
        plane = k_pages.view(k_pages.shape[0], k_pages.shape[2], k_pages.shape[3])     # [pages, page_size, rank]
        table = ctx.block_tables[group]
        cq = torch.empty((n, s.q_rank), dtype=act, device=dev)
        kernels.latent_norm_store(proj, 0, self.q_norm, cq, self.kv_col, self.kv_norm, plane if s.own_kv else None,
                                  table, ctx.row_request, ctx.positions, s.eps)
        q = self.uq(cq)                                                   # [n, H*D]
        q_lat = torch.empty((h, n, s.kv_rank), dtype=act, device=dev)     # the queries in the latents' space
        kernels.batched_linear(q.view(n, h, s.key_dim).transpose(0, 1), self.uk_t, q_lat, act)
        mixed = torch.empty_like(q_lat)
        rows_for_dispatch = ctx.extra.get("dispatch_rows", ctx.n_rows)
        n_slices = kernels.latent_slices(rows_for_dispatch, h, ctx.max_kv_len)
        tiles = None
        if not ctx.decode_only and n_slices == 1 and act == torch.bfloat16 and s.kv_rank % 32 == 0:
            # prompt portions: two tokens of a request per block (the kernel's tensor-core form)
            tile_req, tile_row0, n_tiles = ctx.attention_tiles(kernels.LATENT_TILE_TOKENS)
            tiles = (tile_req, tile_row0, n_tiles, ctx.q_start)
        kernels.latent_attention(q_lat, plane, table, ctx.row_request, ctx.positions, s.scale, s.window, mixed, n_slices,
                                 tiles)
        heads = torch.empty((h, n, s.value_dim), dtype=act, device=dev)
        kernels.batched_linear(mixed, self.uv, heads, act)
        gated = torch.empty((n, h * s.value_dim), dtype=act, device=dev)
        kernels.head_norm_gate(heads.transpose(0, 1), proj[:, self.gate_col:], None, False, kernels.GATE_SIGMOID, s.eps,
                               gated)
        return self.o(gated)


register_mixer("latent_attention", LatentAttention)
