"""The Vebonex configuration reader, its model description and its plain statement (no GPU)."""
import copy

import pytest
import torch

import plain_vebonex as pv
from inferrs_b200.config.base import ConfigError
from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import cache_needs, declared_tensors
from inferrs_b200.cache.storage import KVNeed
from vebonex_cases import CASE_P, CASE_Q, CASE_R, make_weights


def test_description_names_every_tensor_with_its_shape():
    spec, cfg = spec_from_config(CASE_P)
    shapes = {d.name: tuple(d.shape) for d in declared_tensors(spec)}
    assert shapes["embed"] == (211, 96) and shapes["pos"] == (320, 96) and shapes["head"] == (211, 96)
    assert shapes["l0.mix.dkv"] == (36, 96) and shapes["l0.mix.uk"] == (72, 36) and shapes["l0.mix.uv"] == (60, 36)
    assert "l2.mix.dkv" not in shapes and "l2.mix.dkv.norm" not in shapes       # it reads layer 0's latents
    assert shapes["l1.mix.a1"] == (8, 96) and shapes["l1.mix.a2"] == (120, 8) and shapes["l1.mix.norm"] == (20,)
    assert shapes["l3.mix.i"] == (1, 96) and shapes["l3.mix.norm"] == (36,)
    assert shapes["l0.hc2.mix"] == (3, 3) and shapes["l0.hc1.in"] == (3,)
    assert "l1.hc2.in" not in shapes and "l1.norm2" not in shapes and "l1.mlp.up" not in shapes  # no feed-forward
    assert [e.cache for e in spec.schedule] == [0, 1, 0, 3, 4]
    kv, states = cache_needs(spec)
    assert kv == {0: KVNeed(1, 36, None, 1), 4: KVNeed(1, 70, None, 1)}
    assert states[1].shape == (3 * 20 * 40,) and states[3].shape == (36 * 72 + 72 + 1,)


def test_a_model_without_streams_has_the_plain_residual_and_no_connection_tensors():
    spec, _ = spec_from_config(CASE_R)
    assert spec.streams is None and all(l.arrangement == "sequential" for l in spec.layers)
    assert not any(".hc" in d.name for d in declared_tensors(spec))
    assert spec.final_norm.groups == 2


def test_the_decay_rank_comes_from_the_tensor_shapes():
    cfg = copy.deepcopy(CASE_Q)
    del cfg["layers"][1]["mixer"]["a_rank"]
    with pytest.raises(ConfigError, match="a_rank"):
        spec_from_config(cfg)
    spec, _ = spec_from_config(cfg, tensor_shapes={"l1.mix.a1": (6, 64)})
    assert spec.layers[1].mixer.decay_rank == 6


@pytest.mark.parametrize("edit,message", [
    (lambda c: c.pop("norm"), "lacks"),
    (lambda c: c["layers"][0].update(type="conv"), "not one of"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "missing"),
    (lambda c: c["layers"][0]["mixer"].update(window=8), "unknown"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=20), "kv_from"),
    (lambda c: c["norm"].update(groups=5), "divisor"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "mlp"),
])
def test_wrong_configurations_are_refused(edit, message):
    cfg = copy.deepcopy(CASE_P)
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        spec_from_config(cfg)


def test_an_unknown_key_at_the_top_is_named_and_ignored(capsys):
    cfg = copy.deepcopy(CASE_Q)
    cfg["seed"] = 1234
    spec, _ = spec_from_config(cfg)
    assert spec.width == 64 and "seed" in capsys.readouterr().err


def test_plain_scans_carry_their_state_across_a_cut():
    g = torch.Generator().manual_seed(0)
    T, H, D, E = 17, 2, 5, 3
    q, k = torch.randn(T, H, D, generator=g, dtype=torch.float64), torch.randn(T, H, D, generator=g, dtype=torch.float64)
    v = torch.randn(T, H, E, generator=g, dtype=torch.float64)
    a = torch.rand(T, H, D, generator=g, dtype=torch.float64)
    whole, S = pv.gla_scan(q, k, v, a)
    first, S1 = pv.gla_scan(q[:6], k[:6], v[:6], a[:6])
    second, S2 = pv.gla_scan(q[6:], k[6:], v[6:], a[6:], S1)
    assert torch.allclose(torch.cat([first, second]), whole) and torch.allclose(S2, S)
    li, lf = torch.randn(T, H, generator=g, dtype=torch.float64), -torch.rand(T, H, generator=g, dtype=torch.float64)
    whole, st = pv.mlstm_scan(q, k, v, li, lf)
    first, s1 = pv.mlstm_scan(q[:9], k[:9], v[:9], li[:9], lf[:9])
    second, s2 = pv.mlstm_scan(q[9:], k[9:], v[9:], li[9:], lf[9:], s1)
    assert torch.allclose(torch.cat([first, second]), whole)
    # the running maximum starts at zero: a first token with a very negative input gate is weighed by exp(i), not by 1
    o, (S, n, m) = pv.mlstm_scan(q[:1], k[:1], v[:1], torch.full((1, H), -30.0, dtype=torch.float64),
                                 torch.zeros((1, H), dtype=torch.float64))
    assert float(m.abs().max()) == 0.0 and float(S.abs().max()) < 1e-10


def test_plain_model_in_float32_agrees_with_float64():
    for case, seed in ((CASE_P, 1), (CASE_Q, 2), (CASE_R, 3)):
        w = make_weights(case, seed)
        toks = torch.randint(0, case["vocab"], (40,), generator=torch.Generator().manual_seed(seed)).tolist()
        a = pv.forward(case, w, toks, torch.float32)
        b = pv.forward(case, w, toks, torch.float64)
        assert float((a.double() - b).abs().max()) < 2e-4 * float(b.abs().max())
        assert float(b.std()) > 0.3          # the weights are of a size that moves the logits
