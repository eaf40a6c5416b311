"""Korurax without a GPU: the config and its refusals, the model spec, tensor names, and the plain statement on
cases whose answer is known by hand."""

import copy
import math

import pytest
import torch

import plain_korurax as plain
from tiny_korurax import TINY_R

F = torch.float64


def test_config_round_trip_and_registry():
    from starter_b200.config import KoruraxConfig, config_from_dict

    for raw in TINY_R.values():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, KoruraxConfig)
        again = config_from_dict(cfg.to_dict())
        assert again == cfg and again.to_dict() == cfg.to_dict()


@pytest.mark.parametrize("change, text", [
    (lambda r: r.pop("residual_mult"), "residual_mult"),
    (lambda r: r.pop("logit_softcap"), "logit_softcap"),
    (lambda r: r.update(logit_softcap=0.0), "logit_softcap"),
    (lambda r: r.update(rope_theta=1.0), "rope_theta"),
    (lambda r: r["layers"][0].update(type="wkv"), "mixers"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "cannot share"),
    (lambda r: r["layers"][0]["mixer"].pop("mask"), "mask"),
    (lambda r: r["layers"][0]["mixer"].update(window=4), "window"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda r: r["layers"][1]["mixer"].update(kv_from=0), "kv_from"),
    (lambda r: r["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda r: r["layers"][0]["mlp"]["router"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mlp"]["expert"].update(limit=1.0), "limit"),
    (lambda r: r["layers"][0]["mlp"].update(kind="glu"), "feed-forwards"),
])
def test_config_refusals(change, text):
    from starter_b200.config import ConfigError, config_from_dict

    raw = copy.deepcopy(TINY_R["RA"])
    change(raw)
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    assert text in str(err.value)


def test_model_spec_names_sizes_and_constants():
    from starter_b200.config import config_from_dict
    from starter_b200.engine.model import expected_tensors

    spec = config_from_dict(TINY_R["RA"]).to_model_spec()
    assert spec.tie_embeddings and spec.logit_softcap == 30.0
    assert [layer.arrangement for layer in spec.layers] == ["depth_prenorm", "depth_prenorm", "depth_mixer_only",
                                                            "depth_prenorm"]
    assert [layer.connection.levels for layer in spec.layers] == [2, 3, 4, 5]
    assert all(layer.connection.multiplier == 0.5 for layer in spec.layers)
    first = spec.layers[0].mixer
    assert (first.kind, first.chunk, first.value_dim, first.num_kv_heads) == ("sink_attention", 10, 32, 2)
    assert first.distance_penalty and first.sink and first.head_gate and first.window is None
    second = spec.layers[1].mixer
    assert (second.kind, second.position.kind, second.position.dims, second.window) == ("latent_attention", "rope_partial",
                                                                                        8, None)
    moe = spec.layers[0].feed_forward
    assert (moe.expert, moe.scoring, moe.weight_scale, moe.router_bias) == ("relu2", "sigmoid_normalised", 2.0, False)
    assert spec.layers[1].feed_forward.kind == "gated_clamped" and spec.layers[1].feed_forward.limit == 1.5
    shapes = {name: tuple(p.shape) for name, p in expected_tensors(spec).items()}
    assert shapes["embed"] == (200, 64) and "head" not in shapes
    assert shapes["l0.mix.q"] == (64, 64) and shapes["l0.mix.k"] == (32, 64) and shapes["l0.mix.v"] == (64, 64)
    assert shapes["l0.mix.g"] == (4, 64) and shapes["l0.mix.o"] == (64, 128)
    assert shapes["l0.mix.r1"] == shapes["l0.mix.r2"] == shapes["l0.mix.sink"] == (4,)
    assert shapes["l0.mlp.router"] == (5, 64) and shapes["l0.mlp.e4.up"] == (24, 64) and "l0.mlp.e0.gate" not in shapes
    assert shapes["l1.mix.dkv"] == (40, 64) and shapes["l1.mix.uq"] == (72, 24) and shapes["l1.mix.dkv.norm"] == (32,)
    assert shapes["l1.mlp.gate"] == (96, 64)
    assert shapes["l2.dwa"] == (4,) and "l2.norm2" not in shapes and "l2.mlp.up" not in shapes
    assert shapes["final.norm"] == (64,)
    assert "l2.norm2" in spec.ignored_tensors


def test_sink_splits_and_layouts_are_host_arithmetic():
    from starter_b200 import ops

    assert ops.sink_splits(1, 1, None, None, 64 * 40) == 16
    assert ops.sink_splits(8, 4, 100, None, 5000) == 3          # a chunk of 100 spans at most three pages
    assert ops.sink_splits(64, 8, None, None, 5000) == 1
    assert ops.LATENT_LAYOUTS == {"interleaved": 0, "half_split": 1}


# ------------------------------------------------------------------------------ the plain statement by hand

def test_layer_norm_by_hand():
    x = torch.tensor([[1.0, 3.0], [5.0, 5.0]], dtype=F)
    got = plain.layer_norm(x, torch.tensor([2.0, 0.5], dtype=F), 0.0 + 1e-12)
    assert torch.allclose(got[0], torch.tensor([-2.0, 0.5], dtype=F), atol=1e-6)
    assert torch.allclose(got[1], torch.zeros(2, dtype=F))          # a constant row has no deviation


def test_rotation_by_hand():
    x = torch.tensor([[1.0, 0.0, 0.0, 7.0, 0.0, 1.0, 9.0]], dtype=F).repeat(2, 1)
    got = plain.rotate_half_split(x, torch.tensor([0, 1]), 100.0, 4)
    assert torch.equal(got[0], x[0])
    # pairs (0, 2) and (1, 3) by angles 1 and 100 ** -0.5; entries 4.. untouched
    assert torch.allclose(got[1, [0, 2]], torch.tensor([math.cos(1.0), math.sin(1.0)], dtype=F))
    assert torch.allclose(got[1, [1, 3]], torch.tensor([-7.0 * math.sin(0.1), 7.0 * math.cos(0.1)], dtype=F))
    assert torch.equal(got[1, 4:], x[1, 4:])


def test_attention_by_hand():
    # one head, one key visible: weight e^s / (e^s + e^sink), penalty zero at distance zero
    q = torch.tensor([[[2.0]]], dtype=F)
    k = torch.tensor([[[3.0]]], dtype=F)
    v = torch.tensor([[[10.0]]], dtype=F)
    sink = torch.tensor([1.0], dtype=F)
    out = plain.attend(q, k, v, 0.5, torch.tensor([0.7], dtype=F), torch.tensor([2.0], dtype=F), sink,
                       torch.tensor([[0.25]], dtype=F))
    assert abs(float(out) - 0.25 * 10.0 * math.exp(3.0) / (math.exp(3.0) + math.e)) < 1e-12
    # two keys at distances 1 and 0 with equal products: the far one is down by (1 + r2) ** -r1
    q = torch.ones(2, 1, 1, dtype=F)
    k = torch.ones(2, 1, 1, dtype=F)
    v = torch.tensor([[[1.0]], [[0.0]]], dtype=F)
    out = plain.attend(q, k, v, 1.0, torch.tensor([2.0], dtype=F), torch.tensor([3.0], dtype=F))
    far = 4.0 ** -2.0
    assert abs(float(out[1]) - far / (1.0 + far)) < 1e-12
    # chunks of 2: position 2 starts a chunk and sees itself alone; the matrix form agrees with the loops
    assert plain.chunk_visible(5, 2).tolist() == [[True, False, False, False, False], [True, True, False, False, False],
                                                  [False, False, True, False, False], [False, False, True, True, False],
                                                  [False, False, False, False, True]]
    out = plain.attend(q.repeat(2, 1, 1)[:3], k.repeat(2, 1, 1)[:3], torch.tensor([[[1.0]], [[2.0]], [[5.0]]], dtype=F),
                       1.0, chunk=2)
    assert abs(float(out[2]) - 5.0) < 1e-12


def test_a_key_that_stands_out_shows_in_the_plain_statement():
    """A key made to stand out takes all the weight when the query may see it, and none when it may not."""
    g = torch.Generator().manual_seed(0)
    n, chunk = 40, 10
    q, k = torch.randn(n, 1, 8, generator=g, dtype=F), torch.randn(n, 1, 8, generator=g, dtype=F)
    v = torch.randn(n, 1, 4, generator=g, dtype=F)
    q[35, 0] = k[30, 0] * 50.0           # the first key of its chunk
    q[34, 0] = k[29, 0] * 50.0           # the last key of the chunk before
    out = plain.attend(q, k, v, 1.0, chunk=chunk)
    assert (out[35, 0] - v[30, 0]).abs().max() < 1e-6
    inside = plain.attend(q[34:35], k[30:35], v[30:35], 1.0, start=4)          # what query 34 may see: keys 30 to 34
    assert (out[34, 0] - inside[0, 0]).abs().max() < 1e-9


def test_matrix_form_of_the_attention_equals_the_loops():
    g = torch.Generator().manual_seed(1)
    m = dict(heads=4, kv_heads=2, dim=6, vdim=5, scale=0.3, mask=dict(size=4))
    h = torch.randn(11, 7, generator=g, dtype=F)
    w = {"q": torch.randn(24, 7, generator=g, dtype=F), "k": torch.randn(12, 7, generator=g, dtype=F),
         "v": torch.randn(10, 7, generator=g, dtype=F), "g": torch.randn(4, 7, generator=g, dtype=F),
         "o": torch.eye(20, dtype=F), "r1": torch.rand(4, generator=g, dtype=F), "r2": torch.rand(4, generator=g, dtype=F),
         "sink": torch.randn(4, generator=g, dtype=F)}
    got = plain.chunk_attention(h, w, "", m)
    loops = plain.attend((h @ w["q"].T).reshape(11, 4, 6), (h @ w["k"].T).reshape(11, 2, 6), (h @ w["v"].T).reshape(11, 2, 5),
                         0.3, w["r1"], w["r2"], w["sink"], torch.sigmoid(h @ w["g"].T), chunk=4)
    assert torch.allclose(got, loops.reshape(11, 20), atol=1e-12)


def test_feed_forwards_by_hand():
    w = {"gate": torch.tensor([[3.0]], dtype=F), "up": torch.tensor([[-5.0]], dtype=F), "down": torch.tensor([[2.0]], dtype=F)}
    got = plain.clamped_gated(torch.tensor([[1.0]], dtype=F), w, "", 1.5)          # g = 1.5, u = -1.5
    assert abs(float(got) - 2.0 * 1.5 / (1.0 + math.exp(-1.702 * 1.5)) * (-0.5)) < 1e-12
    ids, weights = plain.route(torch.tensor([[1.0, 0.0]], dtype=F), torch.tensor([[0.0, 9.0], [2.0, 0.0], [-1.0, 0.0]], dtype=F),
                               2, 3.0)
    s = [0.5, 1.0 / (1.0 + math.exp(-2.0))]
    assert ids.tolist() == [[1, 0]]
    assert torch.allclose(weights, torch.tensor([[s[1], s[0]]], dtype=F) / sum(s) * 3.0)


def test_depth_sum_and_cap_by_hand():
    """A model whose sublayers all give zero (zero output projections): the stream behind layer i is the
    embedding times the sum of that layer's weights, and the logits are capped."""
    from starter_b200.config import config_from_dict
    from starter_b200.engine.model import expected_tensors

    raw = copy.deepcopy(TINY_R["RA"])
    spec = config_from_dict(raw).to_model_spec()
    g = torch.Generator().manual_seed(2)
    w = {name: torch.randn(p.shape, generator=g, dtype=F) for name, p in expected_tensors(spec).items()}
    for name in w:
        if name.endswith((".mix.o", ".down")):
            w[name].zero_()
    w["embed"] *= 3.0
    tokens = [3, 9, 3]
    logits, layers = plain.forward(raw, w, tokens, return_layers=True)
    x = w["embed"][tokens]
    results, stream = [1.0], 1.0          # as multiples of the embedding: X_0, and what enters layer 0
    for i in range(4):
        results.append(stream)             # a layer that adds nothing hands its input on as its result
        stream = sum(float(w[f"l{i}.dwa"][j]) * results[j] for j in range(i + 2))
        assert torch.allclose(layers[i], stream * x, atol=1e-9)
    assert float(logits.abs().max()) <= 30.0
    assert torch.equal(logits[0], logits[2])
