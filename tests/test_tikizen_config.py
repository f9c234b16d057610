"""The Tikizen configuration reader, its model description and its plain statement (no GPU)."""
import copy

import pytest
import torch

import plain_tikizen as pt
from inferrs_b200.cache.storage import KVNeed
from inferrs_b200.config.base import ConfigError
from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import cache_needs, declared_tensors
from tikizen_cases import CASE_P, CASE_Q, CASE_R, CASE_S, make_weights


def test_description_names_every_tensor_with_its_shape():
    spec, cfg = spec_from_config(CASE_P)
    shapes = {d.name: tuple(d.shape) for d in declared_tensors(spec)}
    assert shapes["embed"] == (211, 96) and shapes["embed.norm"] == (96,) and shapes["head"] == (211, 96)
    assert shapes["l0.mix.q"] == (96, 96) and shapes["l0.mix.k"] == (48, 96) and shapes["l0.mix.v"] == (40, 96)
    assert shapes["l0.mix.o"] == (96, 80) and shapes["l0.mlp.gate"] == (136, 96)
    assert "l2.mix.k" not in shapes and "l2.mix.v" not in shapes            # it reads layer 0's keys and values
    assert "l2.norm2" not in shapes and "l2.mlp.gate" not in shapes          # no feed-forward
    assert shapes["l1.mix.in"] == (48 + 48 + 2 * 2 * 20 + 4, 96) and shapes["l1.mix.conv"] == (48 + 80, 4)
    assert shapes["l1.mix.conv.b"] == (128,) and shapes["l1.mix.A_log"] == (4,) and shapes["l1.mix.norm"] == (48,)
    assert shapes["l1.mlp.router"] == (5, 96) and shapes["l1.mlp.router.b"] == (5,)
    assert shapes["l1.mlp.e4.down"] == (96, 24) and shapes["l1.mlp.shared.up"] == (40, 96)
    assert shapes["l1.mlp.shared.sg"] == (1, 96) and "l3.mlp.shared.sg" not in shapes
    assert shapes["l3.mix.g"] == (72, 96) and shapes["l3.mix.k"] == (120, 96)
    assert [e.cache for e in spec.schedule] == [0, 1, 0, 3]
    assert all(l.arrangement == "norm_after_sum" and l.residual_scale == 1.7 for l in spec.layers)
    kv, states = cache_needs(spec)
    assert kv == {0: KVNeed(2, 24, None, 2, 20)}
    assert states[1].shape == (4 * 20 * 12 + 3 * 128,) and states[3].shape == (3 * 40 * 24,)
    assert spec.layers[0].mixer.chunk == 40 and spec.layers[2].mixer.chunk == 24
    assert spec.layers[0].mixer.position.scaling == (8.0, 64.0, 16.0, 2.0)
    assert spec.layers[3].mixer.position.scaling is None


def test_a_second_norm_without_a_feed_forward_is_read_from_the_tensor_names():
    spec, _ = spec_from_config(CASE_Q)
    assert len(spec.layers[2].sublayers) == 1
    spec, _ = spec_from_config(CASE_Q, tensor_shapes={"l2.norm2": (64,)})
    assert len(spec.layers[2].sublayers) == 2 and spec.layers[2].sublayers[1].part is None
    assert "l2.norm2" in {d.name for d in declared_tensors(spec)}


@pytest.mark.parametrize("edit,message", [
    (lambda c: c.pop("norm"), "lacks"),
    (lambda c: c.pop("postln_alpha"), "lacks"),
    (lambda c: c["layers"][0].update(type="conv"), "not one of"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "missing"),
    (lambda c: c["layers"][0]["mixer"].update(window=8), "unknown"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(dim=16), "kv_from"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot"),
    (lambda c: c["layers"][3]["mixer"].update(decay=[0.5, 0.5]), "decay"),
    (lambda c: c["layers"][3]["mixer"]["rot"].update(scaling={"factor": 2.0}), "scaling"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(slow=0.0), "scaling"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][0].update(mlp={"kind": "dense", "ff": 8}), "dense"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
])
def test_wrong_configurations_are_refused(edit, message):
    cfg = copy.deepcopy(CASE_P)
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        spec_from_config(cfg)


def test_an_unknown_key_at_the_top_is_named_and_ignored(capsys):
    cfg = dict(copy.deepcopy(CASE_S), seed=5)
    spec, _ = spec_from_config(cfg)
    assert "seed" in capsys.readouterr().err and spec.vocab_size == 77


@pytest.mark.parametrize("case", [CASE_P, CASE_Q, CASE_R, CASE_S])
def test_plain_statement_in_float32_agrees_with_float64(case):
    w = make_weights(case, 3)
    toks = torch.randint(0, case["vocab"], (60,), generator=torch.Generator().manual_seed(1)).tolist()
    a, b = pt.forward(case, w, toks, torch.float32), pt.forward(case, w, toks, torch.float64)
    assert float((a.double() - b).abs().max() / b.abs().max()) < 2e-4


def test_plain_statement_sees_chunks_states_and_the_borrowed_keys():
    """A token's logits depend on the tokens of its own chunk and, through the states, on all tokens before it."""
    w = make_weights(CASE_R, 4)          # attention only, chunks of 56 and 48, the last layer without chunks
    toks = torch.randint(0, 130, (100,), generator=torch.Generator().manual_seed(2)).tolist()
    full = pt.forward(CASE_R, w, toks, torch.float64)
    other = list(toks)
    other[3] = (other[3] + 1) % 130
    moved = pt.forward(CASE_R, w, other, torch.float64)
    assert float((full[99] - moved[99]).abs().max()) > 1e-6      # the last layer sees every key
    only_chunks = copy.deepcopy(CASE_R)
    for layer in only_chunks["layers"]:
        layer["mixer"]["mask"] = {"size": 50}
    a, b = pt.forward(only_chunks, w, toks, torch.float64), pt.forward(only_chunks, w, other, torch.float64)
    # every layer in chunks of 50: nothing from position 50 on can have seen position 3
    assert float((a[50:] - b[50:]).abs().max()) == 0.0 and float((a[3:40] - b[3:40]).abs().max()) > 1e-6
