"""The Vebonex decoder, written down as a :class:`ModelSpec`.

This file holds no arithmetic.  It says which parts the design is made of, with which tensor names and which
config.json values:

* the embedding row plus a learned vector per position; a residual that is ``streams`` copies wide
  (hyper-connections: every sub-layer reads a weighted sum of the streams and its output comes back through a
  mixing matrix and a gain per stream) whose sum goes to the last norm;
* every norm is an RMS norm in ``norm.groups`` equal parts of the row;
* a layer is a mixer and, unless config.json says null, a dense feed-forward with the polynomial activation of
  unit-rms terms; the mixer is one of gated linear attention (a decay per key channel), the matrix memory of
  xLSTM (scalar gates with a running maximum), or attention over cached latents without positions, whose layer
  may read the latents of an earlier layer (``kv_from``);
* tensors: ``embed``, ``pos``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.up|down|act``,
  ``l<i>.hc1|hc2.in|out|mix``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import ConfigError, register_architecture
from ..config.vebonex import VebonexConfig
from ..parts.spec import (ChannelDecayScanSpec, LatentAttentionSpec, LayerSpec, ModelSpec, NormSpec, PolyNormDenseSpec,
                          ScalarGateScanSpec, ScheduleEntry, StreamConnectionSpec, SubLayerSpec)

ARCHITECTURE = "Vebonex"


def _mixer(cfg: VebonexConfig, i: int):
    layer, p = cfg.layers[i], f"l{i}.mix"
    common = dict(width=cfg.width, n_heads=layer.get("heads"), key_dim=layer.get("dim"), value_dim=layer.get("vdim"),
                  eps=cfg.norm_eps, gate_proj=f"{p}.g", o_proj=f"{p}.o")
    if layer.type == "gla":
        if layer.get("a_rank") is None:
            raise ConfigError(f"layer {i}: the inner size of the decay's two products is given neither by the tensor "
                              f"'{p}.a1' (no weight files were read) nor by the key 'a_rank' of the layer's mixer")
        return ChannelDecayScanSpec(**common, tau=layer.get("tau"), q_proj=f"{p}.q", k_proj=f"{p}.k", v_proj=f"{p}.v",
                                    decay_rank=layer.get("a_rank"), decay_down=f"{p}.a1", decay_up=f"{p}.a2",
                                    decay_bias=f"{p}.a2.b", out_norm=f"{p}.norm")
    if layer.type == "mlstm":
        return ScalarGateScanSpec(**common, gate_cap=layer.get("gate_cap"), q_proj=f"{p}.q", k_proj=f"{p}.k",
                                  v_proj=f"{p}.v", i_proj=f"{p}.i", i_bias=f"{p}.i.b", f_proj=f"{p}.f",
                                  f_bias=f"{p}.f.b", out_norm=f"{p}.norm")
    if layer.type == "latent_attention":
        own = layer.get("kv_from") is None
        return LatentAttentionSpec(**common, q_rank=layer.get("q_rank"), kv_rank=layer.get("kv_rank"),
                                   scale=layer.get("scale"), dq_proj=f"{p}.dq", dq_norm=f"{p}.dq.norm",
                                   uq_proj=f"{p}.uq", uk_proj=f"{p}.uk", uv_proj=f"{p}.uv",
                                   dkv_proj=f"{p}.dkv" if own else None, dkv_norm=f"{p}.dkv.norm" if own else None,
                                   own_kv=own)
    raise ConfigError(f"layer {i}: no mixer of type '{layer.type}'")


def build_spec(cfg: VebonexConfig) -> ModelSpec:
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        mixer = _mixer(cfg, i)
        parts = [(mixer, "mixer")]
        if layer.ff is not None:
            parts.append((PolyNormDenseSpec(width=cfg.width, inner=layer.ff, up_proj=f"l{i}.mlp.up",
                                            down_proj=f"l{i}.mlp.down", coef=f"l{i}.mlp.act", eps=cfg.norm_eps),
                          "feed_forward"))
        subs = []
        for q, (part, category) in enumerate(parts, start=1):
            connection = None if cfg.streams is None else StreamConnectionSpec(
                streams=cfg.streams, read=f"l{i}.hc{q}.in", gain=f"l{i}.hc{q}.out", mix=f"l{i}.hc{q}.mix")
            subs.append(SubLayerSpec(part=part, category=category, connection=connection,
                                     norm=NormSpec(size=cfg.width, eps=cfg.norm_eps, weight=f"l{i}.norm{q}",
                                                   groups=cfg.norm_groups)))
        layers.append(LayerSpec(sublayers=tuple(subs),
                                arrangement="sequential" if cfg.streams is None else "hyper_connections"))
        # a layer that reads an earlier layer's latents runs on that layer's cache
        kv_from = layer.get("kv_from") if layer.type == "latent_attention" else None
        schedule.append(ScheduleEntry(layer=i, cache=i if kv_from is None else kv_from))
    return ModelSpec(
        vocab_size=cfg.vocab,
        width=cfg.width,
        embedding="embed",
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=NormSpec(size=cfg.width, eps=cfg.norm_eps, weight="final.norm", groups=cfg.norm_groups),
        lm_head="head",
        lm_head_optional=False,
        max_positions=cfg.max_positions,
        position_table="pos",
        streams=cfg.streams,
        eos_token_ids=cfg.eos_token_ids,
        architecture=ARCHITECTURE,
    )


register_architecture(ARCHITECTURE, VebonexConfig, build_spec, model_type="vebonex", replace=True)
