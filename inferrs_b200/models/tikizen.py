"""The Tikizen decoder, written down as a :class:`ModelSpec`.

This file holds no arithmetic.  It says which parts the design is made of, with which tensor names and which
config.json values:

* the embedding row goes through an RMS norm (``embed.norm``) before the first layer;
* a layer norms after the sum: x <- norm1(alpha x + mixer(x)), then x <- norm2(alpha x + ff(x)); the parts read x
  itself, and alpha is ``postln_alpha``;
* the mixer is one of grouped-query attention (rotation with stretched slow pairs, queries and keys divided by their
  root mean square after the rotation, keys visible chunk by chunk, values of a size of their own, optionally on the
  keys and values of an earlier layer: ``kv_from``), retention (a matrix state with a fixed decay per head), or the
  state-space mixer of Mamba-2 (a short convolution, a matrix state with a decay from dt);
* the feed-forward is a gated dense one with a clamped activation, or routed experts with a shared expert;
* tensors: ``embed``, ``embed.norm``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import ConfigError, register_architecture
from ..config.tikizen import TikizenConfig
from ..parts.spec import (AttentionSpec, FixedDecayScanSpec, GatedDenseSpec, LayerSpec, ModelSpec, NormSpec,
                          PositionSpec, RoutedExpertsSpec, ScheduleEntry, StateSpaceScanSpec, SubLayerSpec)

ARCHITECTURE = "Tikizen"


def _position(cfg: TikizenConfig, rot) -> PositionSpec:
    if not rot:
        return PositionSpec(kind="none")
    sc = rot.get("scaling")
    scaling = None if not sc else (float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
    return PositionSpec(kind="rotary_scaled", rot_dim=int(rot["dims"]), theta=float(rot["base"]),
                        max_positions=cfg.max_positions, scaling=scaling)


def _mixer(cfg: TikizenConfig, i: int):
    layer, p = cfg.layers[i], f"l{i}.mix"
    if layer.type == "attention":
        own = layer.get("kv_from") is None
        unit = NormSpec(size=layer.get("dim"), eps=cfg.norm_eps, weight=None)     # division by the rms, no weight
        mask = layer.get("mask")
        return AttentionSpec(width=cfg.width, n_heads=layer.get("heads"), n_kv_heads=layer.get("kv_heads"),
                             head_dim=layer.get("dim"), value_dim=layer.get("vdim"), scale=float(layer.get("scale")),
                             position=_position(cfg, layer.get("rot")), q_proj=f"{p}.q", o_proj=f"{p}.o",
                             k_proj=f"{p}.k" if own else None, v_proj=f"{p}.v" if own else None,
                             q_norm=unit, k_norm=unit, norm_after_rotation=True,
                             chunk=None if not mask else int(mask["size"]), own_kv=own)
    if layer.type == "retention":
        return FixedDecayScanSpec(width=cfg.width, n_heads=layer.get("heads"), key_dim=layer.get("dim"),
                                  value_dim=layer.get("vdim"), decay=tuple(float(a) for a in layer.get("decay")),
                                  eps=cfg.norm_eps, position=_position(cfg, layer.get("rot")), q_proj=f"{p}.q",
                                  k_proj=f"{p}.k", v_proj=f"{p}.v", gate_proj=f"{p}.g", o_proj=f"{p}.o")
    if layer.type == "mamba2":
        return StateSpaceScanSpec(width=cfg.width, n_heads=layer.get("heads"), value_dim=layer.get("vdim"),
                                  state=layer.get("state"), groups=layer.get("groups"), taps=layer.get("conv"),
                                  norm_groups=layer.get("norm_groups"), eps=cfg.norm_eps, in_proj=f"{p}.in",
                                  conv=f"{p}.conv", conv_bias=f"{p}.conv.b", dt_bias=f"{p}.dt_bias",
                                  a_log=f"{p}.A_log", skip=f"{p}.D", out_norm=f"{p}.norm", o_proj=f"{p}.o")
    raise ConfigError(f"layer {i}: no mixer of type '{layer.type}'")


def _feed_forward(cfg: TikizenConfig, i: int):
    layer, p = cfg.layers[i], f"l{i}.mlp"
    if layer.mlp is None:
        return None
    if layer.mlp_get("kind") == "dense":
        return GatedDenseSpec(width=cfg.width, inner=layer.mlp_get("ff"), gate_proj=f"{p}.gate", up_proj=f"{p}.up",
                              down_proj=f"{p}.down", activation="clamped_swish", limit=float(layer.mlp_get("limit")),
                              slope=1.702)
    router, shared = layer.mlp_get("router"), layer.mlp_get("shared")
    return RoutedExpertsSpec(
        width=cfg.width, inner=layer.mlp_get("expert")["ff"], top=router["top"], router=f"{p}.router",
        router_bias=f"{p}.router.b",
        experts=tuple((f"{p}.e{e}.gate", f"{p}.e{e}.up", f"{p}.e{e}.down") for e in range(router["experts"])),
        shared=None if not shared else (f"{p}.shared.gate", f"{p}.shared.up", f"{p}.shared.down", f"{p}.shared.sg"),
        shared_inner=0 if not shared else shared["ff"])


def build_spec(cfg: TikizenConfig) -> ModelSpec:
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        subs = [SubLayerSpec(part=_mixer(cfg, i), category="mixer",
                             sum_norm=NormSpec(size=cfg.width, eps=cfg.norm_eps, weight=f"l{i}.norm1"))]
        ff = _feed_forward(cfg, i)
        if ff is not None or layer.bare_norm2:
            subs.append(SubLayerSpec(part=ff, category="feed_forward",
                                     sum_norm=NormSpec(size=cfg.width, eps=cfg.norm_eps, weight=f"l{i}.norm2")))
        layers.append(LayerSpec(sublayers=tuple(subs), arrangement="norm_after_sum",
                                residual_scale=cfg.residual_scale))
        # a layer that reads an earlier layer's keys and values runs on that layer's cache
        kv_from = layer.get("kv_from") if layer.type == "attention" else None
        schedule.append(ScheduleEntry(layer=i, cache=i if kv_from is None else kv_from))
    return ModelSpec(
        vocab_size=cfg.vocab,
        width=cfg.width,
        embedding="embed",
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=NormSpec(size=cfg.width, eps=cfg.norm_eps, weight="final.norm"),
        lm_head="head",
        lm_head_optional=False,
        max_positions=cfg.max_positions,
        embedding_norm=NormSpec(size=cfg.width, eps=cfg.norm_eps, weight="embed.norm"),
        eos_token_ids=cfg.eos_token_ids,
        architecture=ARCHITECTURE,
    )


register_architecture(ARCHITECTURE, TikizenConfig, build_spec, model_type="tikizen", replace=True)
