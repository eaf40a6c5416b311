"""Bavedra's configuration on the CPU: what config.json means, what is refused, the run order of layers that run
another layer's weights, tensor names, and the plain statement on cases whose answer is known."""

import copy
import math

import pytest
import torch

import plain_bavedra as plain
from tiny_bavedra import B_A, B_B, B_C, TINY_B

F = torch.float64


def spec_of(raw):
    from starter_b200.config import config_from_dict

    return config_from_dict(raw).to_model_spec()


def test_every_size_and_constant_comes_from_the_config():
    spec = spec_of(B_A)
    assert spec.architecture == "Bavedra" and spec.vocab_size == 200 and spec.hidden_size == 64
    assert spec.embedding_scale == 2.0 and not spec.tie_embeddings and spec.lm_head_name == "head"
    assert len(spec.layers) == 4                       # the fifth layer has no tensors of its own
    first, second, third, fourth = spec.layers
    m = first.mixer
    assert (m.kind, m.width, m.blocks, m.conv, m.decay_scale) == ("gated_linear_recurrence", 96, 3, 3, 8.0)
    assert (first.feed_forward.kind, first.feed_forward.intermediate_size, first.feed_forward.bias) == ("dense_biased", 80, False)
    a, s = second.mixer.left, second.mixer.right
    assert (a.kind, a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.scale, a.window) == ("sink_attention", 4, 2, 16, 16, 0.3, 10)
    assert a.values_from_keys and a.fixed_sink == 0.0 and not (a.sink or a.head_gate or a.distance_penalty)
    assert (a.position.kind, a.position.base, a.position.dims) == ("rope_interleaved", 100.0, 8)
    assert (s.kind, s.num_heads, s.head_dim, s.state, s.groups, s.conv, s.norm_groups) == ("state_space", 3, 8, 12, 1, 2, 3)
    ff = second.feed_forward
    assert (ff.experts, ff.top, ff.intermediate_size, ff.identity_experts, ff.group_count, ff.group_keep, ff.shared_size) == (5, 2, 24, 1, 3, 2, 16)
    assert (ff.expert, ff.scoring, ff.correction, ff.router_bias) == ("gated_silu", "softmax_all", True, False)
    d = third.mixer
    assert (d.kind, d.num_heads, d.num_kv_heads, d.head_dim, d.value_dim, d.conv) == ("gated_delta", 4, 2, 12, 8, 4)
    assert third.arrangement == "prenorm32_mixer_only" and "feed_forward" not in third.parts
    assert fourth.mixer.left.window == 500 and fourth.arrangement == "prenorm32"
    assert all(layer.norm1.gain_32bit and layer.norm1.eps == 1e-5 and not layer.norm1.unit_offset for layer in spec.layers)
    plainer = spec_of(B_B).layers[0].feed_forward
    assert (plainer.identity_experts, plainer.group_count, plainer.group_keep, plainer.shared_size) == (0, 1, 1, 0)
    assert spec_of(B_C).layers[2].mixer.left.position is None


def test_run_order_of_layers_that_run_another_layers_weights():
    order = spec_of(B_A).schedule
    assert [(e.layer, e.cache, e.writes_cache) for e in order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 3, True), (2, 4, True)]
    order = spec_of(B_B).schedule
    assert [(e.layer, e.cache) for e in order] == [(0, 0), (0, 1), (1, 2), (2, 3)]


def test_a_layer_may_run_the_weights_of_a_later_layer_or_of_one_that_borrows_itself():
    from starter_b200.engine.model import expected_tensors

    raw = copy.deepcopy(B_A)
    first = dict(raw["layers"][2], weights_of=3)            # in front of the layer that has the tensors
    raw["layers"] = [first] + raw["layers"]                 # layers 1..5 are B_A's 0..4
    raw["layers"][5]["weights_of"] = 0                      # 5 -> 0 -> 3
    spec = spec_of(raw)
    assert [(e.layer, e.cache) for e in spec.schedule] == [(2, 0), (0, 1), (1, 2), (2, 3), (3, 4), (2, 5)]
    names = expected_tensors(spec)
    assert "l3.mix.q" in names and not any(n.startswith(("l0.", "l5.")) for n in names)


def test_tensor_names():
    from starter_b200.engine.model import expected_tensors

    names = expected_tensors(spec_of(B_A))
    for name, shape in {"embed": (200, 64), "head": (200, 64), "final.norm": (64,), "l0.mix.y.b": (96,), "l0.mix.ra": (3, 32, 32),
                        "l0.mix.ri.b": (3, 32), "l0.mix.conv": (96, 3), "l0.mix.lam": (96,), "l0.mlp.down": (64, 80),
                        "l1.mix.left.k": (32, 64), "l1.mix.left.out": (64,), "l1.mix.right.in": (2 * 24 + 2 * 12 + 3, 64),
                        "l1.mix.right.conv": (48, 2), "l1.mix.right.norm": (24,), "l1.mlp.router": (6, 64),
                        "l1.mlp.correction": (6,), "l1.mlp.e4.gate": (24, 64), "l1.mlp.shared.sg": (1, 64),
                        "l2.mix.q.conv": (24, 4), "l2.mix.v": (32, 64), "l2.mix.norm": (8,), "l2.mix.b": (4, 64),
                        "l3.norm2": (64,)}.items():
        assert tuple(names[name].shape) == shape, name
    assert not any(n.startswith("l4.") for n in names) and "l2.norm2" not in names and "l1.mix.left.v" not in names
    assert "l1.mlp.e5.gate" not in names          # the sixth router output is an identity expert


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="lstm"), "mixers"),
    (lambda c: c["layers"][0]["mixer"].update(extra=1), "extra"),
    (lambda c: c["layers"][0]["mixer"].update(blocks=5), "blocks"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "key/value heads"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(norm_groups=5), "norm groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "feed-forwards"),
    (lambda c: c["layers"][4].update(weights_of=4), "another layer"),
    (lambda c: c["layers"][4].update(weights_of=7), "another layer"),
    (lambda c: c["layers"][4].update(weights_of=1), "differs"),
    (lambda c: c["layers"][2].update(weights_of=4), "leads back to itself"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(window=3), "window"),
])
def test_what_is_refused(change, text):
    from starter_b200.config import ConfigError, config_from_dict

    raw = copy.deepcopy(B_A)
    change(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_more_choices_than_experts_when_identity_experts_make_up_for_it():
    from starter_b200.engine.model import expected_tensors

    raw = copy.deepcopy(B_B)
    raw["layers"][3]["mlp"]["router"] = dict(experts=2, top=3, identity=2)
    names = expected_tensors(spec_of(raw))
    assert tuple(names["l3.mlp.router"].shape) == (4, 96) and "l3.mlp.e1.up" in names and "l3.mlp.e2.up" not in names


def test_config_round_trip():
    from starter_b200.config import config_from_dict

    for raw in TINY_B.values():
        cfg = config_from_dict(raw)
        assert config_from_dict(cfg.to_dict()) == cfg


# ------------------------------------------------------------------------------ the plain statement, by hand

def test_plain_convolution_puts_the_last_tap_on_the_current_token():
    x = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=F)
    y = plain.short_convolution(x, torch.tensor([[3.0, 2.0, 1.0]], dtype=F), torch.tensor([0.5], dtype=F))
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5, 1230.5]


def test_plain_attention_with_a_sink_and_a_window():
    q = torch.zeros((4, 1, 2), dtype=F)
    k = torch.zeros((4, 1, 2), dtype=F)
    v = torch.tensor([[[1.0]], [[2.0]], [[4.0]], [[8.0]]], dtype=F)
    out = plain.window_attention(q, k, v, 1.0, 2)
    # every score is 0: a query's keys weigh 1 / (1 + n) each, the sink takes the rest; the window holds two
    assert out[:, 0, 0].tolist() == pytest.approx([1 / 2, 3 / 3, 6 / 3, 12 / 3])
    q[3, 0, 0], k[2, 0, 0] = 1.0, math.log(3.0)
    out = plain.window_attention(q, k, v, 1.0, 2)
    assert float(out[3, 0, 0]) == pytest.approx((3 * 4 + 8) / (1 + 3 + 1))


def test_plain_rotation_turns_neighbouring_entries_and_leaves_the_rest():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]]], dtype=F).repeat(2, 1, 1)
    y = plain.rotate_pairs(x, torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(y[0], x[0])
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    want = [math.cos(a0), math.sin(a0), -2 * math.sin(a1), 2 * math.cos(a1), 5.0, 6.0]
    assert y[1, 0].tolist() == pytest.approx(want)


def test_plain_recurrent_unit_first_token_and_decay():
    u = torch.tensor([[2.0], [0.0]], dtype=F)
    r = torch.tensor([[0.5], [0.25]], dtype=F)
    i = torch.tensor([[0.75], [1.0]], dtype=F)
    lam = torch.tensor([0.3], dtype=F)
    sp = math.log1p(math.exp(0.3))
    a0, a1 = math.exp(-8 * 0.5 * sp), math.exp(-8 * 0.25 * sp)
    S = plain.gated_linear_recurrence(u, r, i, lam)
    assert float(S[0]) == pytest.approx(math.sqrt(1 - a0 * a0) * 0.75 * 2.0)
    assert float(S[1]) == pytest.approx(a1 * float(S[0]))


def test_plain_delta_rule_reads_its_own_write_and_corrects_a_repeated_key():
    k = torch.tensor([[[1.0, 0.0]], [[1.0, 0.0]]], dtype=F)
    q = k.clone()
    v = torch.tensor([[[3.0]], [[5.0]]], dtype=F)
    beta = torch.tensor([[1.0], [1.0]], dtype=F)
    g = torch.tensor([[1.0], [0.5]], dtype=F)
    o = plain.delta_recurrence(q, k, v, beta, g)
    # with beta 1 the state holds exactly v under the key; the second token first halves what is there, then
    # replaces what the key reads by its own value
    assert o[:, 0, 0].tolist() == pytest.approx([3.0, 5.0])
    beta[1, 0] = 0.5
    assert float(plain.delta_recurrence(q, k, v, beta, g)[1, 0, 0]) == pytest.approx(1.5 + 0.5 * (5.0 - 1.5))


def test_plain_state_space_step():
    x = torch.tensor([[[2.0]], [[0.0]]], dtype=F)
    B = torch.tensor([[[1.0, 1.0]], [[0.0, 0.0]]], dtype=F)
    C = torch.tensor([[[1.0, 0.0]], [[1.0, 1.0]]], dtype=F)
    dt = torch.tensor([[0.5], [2.0]], dtype=F)
    y = plain.state_space_recurrence(x, B, C, dt, torch.tensor([0.0], dtype=F), torch.tensor([10.0], dtype=F))
    assert float(y[0, 0, 0]) == pytest.approx(0.5 * 2.0 + 10.0 * 2.0)
    assert float(y[1, 0, 0]) == pytest.approx(math.exp(-2.0) * 2 * 0.5 * 2.0)


def test_plain_router_keeps_the_best_groups_and_counts_identity_experts():
    w = {"r.router": torch.eye(6, dtype=F) * 1.0, "r.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 0.9, 0.0], dtype=F)}
    h = torch.tensor([[3.0, 2.9, 0.0, 0.0, 0.0, 0.0]], dtype=F)
    router = dict(experts=4, identity=2, top=2, groups=dict(count=3, keep=1))
    index, weight, s = plain.route(h, w, "r.", router)
    # the correction lifts output 4 above all, so its group (4, 5) is the one kept, and both choices come from it
    assert index[0].tolist() == [4, 5]
    assert weight[0].tolist() == pytest.approx([0.5, 0.5])
    router["groups"] = dict(count=3, keep=2)
    index, weight, s = plain.route(h, w, "r.", router)
    assert index[0].tolist() == [4, 0]
    assert float(weight[0, 1]) == pytest.approx(float(s[0, 0] / (s[0, 0] + s[0, 4])))
    # an identity expert hands its input on
    mlp = dict(kind="moe", expert=dict(ff=1), router=dict(experts=4, identity=2, top=1, groups=dict(count=3, keep=1)))
    out = plain.routed_feed_forward(h, w, "r.", mlp)
    assert torch.allclose(out, h)


def test_a_layer_run_twice_has_a_state_of_its_own():
    torch.manual_seed(0)
    cfg = copy.deepcopy(B_B)
    cfg["layers"] = cfg["layers"][:2]
    from starter_b200.config import config_from_dict
    from starter_b200.engine.model import expected_tensors

    w = {n: torch.randn(tuple(p.shape), dtype=F) * 0.3 for n, p in expected_tensors(config_from_dict(cfg).to_model_spec()).items()}
    layers = []
    plain.forward(cfg, w, [1, 2, 3, 4], layers)
    once = copy.deepcopy(cfg)
    once["layers"] = once["layers"][:1]
    first = []
    plain.forward(once, w, [1, 2, 3, 4], first)
    assert torch.equal(layers[0], first[0]) and not torch.allclose(layers[1], layers[0])
