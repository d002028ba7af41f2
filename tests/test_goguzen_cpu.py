"""Goguzen without a GPU: configuration round trip, checkpoint naming, the constants the layer struct carries, registry, and
identities of the oracle's mechanisms (oracle/goguzen_oracle.py) that do not depend on the product path."""
import json
import math

import pytest
import torch

from oracle import goguzen_oracle as O
from pegainfer_b200.goguzen import GoguzenConfig, iter_random_weights, weight_shapes

LEFT = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 6, "scale": 0.35, "q_temp": {"coef": 0.7, "every": 5}}
RIGHT = {"heads": 3, "vdim": 4, "state": 5, "groups": 1, "conv": 3, "norm_groups": 2}
ATT = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 10, "scale": 0.3, "mask": {"size": 7, "keep_first": 3},
       "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 20}}}
MLP = {"kind": "moe", "expert": {"ff": 12, "limit": 0.9}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 8, "limit": 1.4}}
CFG = {"architecture": "Goguzen", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "logit_scale": 0.4,
       "logit_softcap": 9.0, "layers": [
           {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT}, "mlp": MLP},
           {"type": "attention", "mixer": ATT, "mlp": None},
           {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT}, "mlp": MLP, "weights_of": 0}]}


def test_config_round_trip_and_tensor_names():
    c = GoguzenConfig.from_dict(CFG)
    assert GoguzenConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c
    assert c.layers[2].weights_of == 0 and c.layers[1].attention.keep_first == 3 and c.layers[0].attention.temp_every == 5
    s = weight_shapes(c)
    assert s["l0.mix.left.q"] == (24, 24) and s["l0.mix.left.k"] == (12, 24) and s["l0.mix.left.q.norm"] == (6,) and s["l0.mix.left.sink"] == (4,)
    assert s["l0.mix.right.in"] == (2 * 12 + 2 * 5 + 3, 24) and s["l0.mix.right.conv"] == (22, 3) and s["l0.mix.right.conv.b"] == (22,)
    assert s["l0.mix.right.norm"] == (12,) and s["l0.mix.right.o"] == (24, 12) and s["l0.mix.left.out"] == (24,) and s["l0.mix.right.D"] == (3,)
    assert s["l1.mix.q"] == (16, 24) and s["l1.mix.v"] == (10, 24) and s["l1.mix.q.norm"] == (16,) and s["l1.mix.k.norm"] == (8,)
    assert s["l1.mix.o"] == (24, 20) and s["l0.mlp.e4.gate"] == (12, 24) and s["l0.mlp.router.b"] == (5,) and s["l0.mlp.shared.down"] == (24, 8)
    for absent in ("l0.mix.left.v", "l1.norm2", "l1.mlp.router", "l2.norm1", "l2.mix.left.q", "l0.mlp.e5.gate"):
        assert absent not in s
    assert {n for n, _ in iter_random_weights(c)} == set(s)


def test_a_borrowing_layer_must_equal_its_owner():
    bad = json.loads(json.dumps(CFG))
    bad["layers"][2]["mixer"]["right"]["state"] = 6
    with pytest.raises(ValueError):
        GoguzenConfig.from_dict(bad)
    bad = json.loads(json.dumps(CFG))
    bad["layers"][1]["weights_of"] = 2  # layer 2 has no weights of its own
    with pytest.raises(ValueError):
        GoguzenConfig.from_dict(bad)


def test_a_chain_of_borrowers_ends_at_the_owner():
    chain = json.loads(json.dumps(CFG))
    chain["layers"].append(dict(chain["layers"][2], weights_of=2))
    c = GoguzenConfig.from_dict(chain)
    assert [l.weights_of for l in c.layers] == [None, None, 0, 0]
    chain["layers"][0]["weights_of"] = 3  # a ring has no owner
    with pytest.raises(ValueError):
        GoguzenConfig.from_dict(chain)


def test_layer_struct_carries_the_designs_constants():
    from pegainfer_b200.goguzen import GoguzenModel
    from pegainfer_b200.layered import ModelCfg
    c = GoguzenConfig.from_dict(CFG)
    a, b, d = (GoguzenModel.layer_struct(l) for l in c.layers)
    assert (a.mixer_kind, a.qk_norm, a.values_are_keys, a.q_temp_every, a.window, a.rot_dims, a.weights_of) == (4, 1, 1, 5, 0, 0, -1)
    assert (a.ssm_heads, a.ssm_vdim, a.ssm_state, a.ssm_groups, a.ssm_norm_groups, a.conv) == (3, 4, 5, 1, 2, 3)
    assert (a.mlp_kind, a.experts, a.top, a.expert_ff, a.shared_ff, a.expert_act, a.router_kind) == (2, 5, 2, 12, 8, 2, 2)
    assert math.isclose(a.act_limit, 0.9, rel_tol=1e-6) and math.isclose(a.shared_limit, 1.4, rel_tol=1e-6) and math.isclose(a.act_slope, 1.702, rel_tol=1e-6)
    assert (b.mixer_kind, b.qk_norm, b.values_are_keys, b.window, b.keep_first, b.rot_dims, b.rot_interleaved, b.mlp_kind) == (1, 2, 0, 7, 3, 4, 0, 0)
    assert (b.has_scaling, b.scaling_kind) == (1, 1) and (b.s_factor, b.s_slow, b.s_fast, b.s_original) == (4.0, 1.0, 2.0, 20.0)
    assert d.weights_of == 0 and d.mixer_kind == 4
    mc = GoguzenModel.model_struct(c, ModelCfg())
    assert mc.block_kind == 3 and math.isclose(mc.logit_softcap, 9.0) and math.isclose(mc.embed_scale, 3.0)


def test_registry_knows_the_design(tmp_path):
    from pegainfer_b200.registry import FLOAT32_CAPABLE, architecture_of
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert architecture_of(str(tmp_path)) == "Goguzen" and "Goguzen" in FLOAT32_CAPABLE
    from pegainfer_b200 import build
    for f in ("gqa_attention.cu", "recurrent_mixers.cu", "moe.cu", "moe_grouped.cu", "residual32_ops.cu"):
        assert f in build.PARTS_OF["Goguzen"][0]
    assert "layered_host.cpp" in build.PARTS_OF["Goguzen"][1]


def weights(seed=0):
    return {n: t.float() for n, t in iter_random_weights(GoguzenConfig.from_dict(CFG), seed)}


def test_oracle_is_causal_and_shares_weights_not_state():
    w = weights()
    toks = torch.randint(0, 50, (30,), generator=torch.Generator().manual_seed(1)).tolist()
    trail = []
    full = O.forward(CFG, w, toks, trail)
    assert torch.allclose(O.forward(CFG, w, toks[:17]), full[:17], atol=1e-5)
    assert len(trail) == 3 and full.abs().max() < 9.0  # soft cap
    # layers 0 and 2 use the same tensors, but see different inputs
    assert not torch.allclose(trail[0], trail[2] - trail[1], atol=1e-3)


def test_oracle_window_keeps_the_first_positions():
    ok = O.visible(torch.arange(30), torch.arange(30), 7, 3)
    assert ok[20, 14] and not ok[20, 13] and ok[20, 2] and not ok[20, 3] and ok[20, 20] and not ok[20, 21]
    assert ok[5, 0] and ok[9, 3] and not ok[10, 3] and ok[10, 2]
    assert O.visible(torch.arange(9), torch.arange(9)).sum() == 45
    # the attention mixer at position 20 depends on inputs 14 .. 20 and 0 .. 2 and on nothing else
    w = weights()
    h = torch.randn(25, 24, generator=torch.Generator().manual_seed(2))
    run = lambda x: O.windowed_attention(x, w, "l1.mix.", ATT, torch.arange(25), 1e-5)[20]  # noqa: E731
    out = run(h)
    for at, seen in ((13, False), (14, True), (3, False), (2, True), (0, True), (21, False)):
        h2 = h.clone()
        h2[at] += 1.0
        assert torch.allclose(run(h2), out, atol=1e-6) != seen, at


def test_oracle_sink_query_factor_and_frequencies():
    s = torch.zeros(1, 3)
    ok = torch.ones(1, 3, dtype=torch.bool)
    assert torch.allclose(O.softmax_with_sink(s, ok, torch.tensor(0.0)), torch.full((1, 3), 0.25))
    assert O.softmax_with_sink(s - 50.0, ok, torch.tensor(0.0)).sum() < 1e-20
    assert torch.allclose(O.softmax_with_sink(s, ok, torch.tensor(-60.0)).sum(), torch.tensor(1.0))
    f = O.query_stretch(torch.tensor([0, 3, 4, 8, 9, 24]), {"coef": 0.7, "every": 5}, torch.float32)
    want = [1.0, 1.0, 1 + 0.7 * math.log(2), 1 + 0.7 * math.log(2), 1 + 0.7 * math.log(3), 1 + 0.7 * math.log(6)]
    assert torch.allclose(f, torch.tensor(want))
    # wavelengths below original / high keep their frequency, those above original / low are slowed by the factor
    rot = {"dims": 8, "base": 10.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 20}}
    plain = 10.0 ** (-2.0 * torch.arange(4, dtype=torch.float64) / 8)
    got = O.rescaled_frequencies(rot)
    assert torch.allclose(got[0], plain[0]) and torch.allclose(got[3], plain[3] / 4.0)
    for i in (1, 2):
        lam = 2 * math.pi / plain[i]
        assert 10 < lam < 20
        blend = (20 / lam - 1.0) / (2.0 - 1.0)
        assert torch.allclose(got[i], (1 - blend) * plain[i] / 4 + blend * plain[i])


def test_oracle_rotation_turns_halves_and_keeps_relative_angles():
    rot = {"dims": 4, "base": 100.0}
    g = torch.Generator().manual_seed(4)
    q, k = torch.randn(1, 1, 6, generator=g), torch.randn(1, 1, 6, generator=g)
    a = (O.rotate_halves(q, torch.tensor([9]), rot) * O.rotate_halves(k, torch.tensor([5]), rot)).sum()
    b = (O.rotate_halves(q, torch.tensor([14]), rot) * O.rotate_halves(k, torch.tensor([10]), rot)).sum()
    assert torch.allclose(a, b, atol=1e-5)
    r = O.rotate_halves(q, torch.tensor([3]), rot)
    assert torch.allclose(r[..., 4:], q[..., 4:]) and torch.allclose(r[..., [0, 2]].norm(), q[..., [0, 2]].norm(), atol=1e-6)
    one = torch.tensor([[[1.0, 0.0, 0.0, 0.0]]])
    assert math.isclose(float(O.rotate_halves(one, torch.tensor([1]), rot)[0, 0, 2]), math.sin(1.0), abs_tol=1e-6)


def test_oracle_state_space_branch_carries_its_state():
    w = weights()
    h = torch.randn(19, 24, generator=torch.Generator().manual_seed(5))
    whole, _ = O.state_space_branch(h, w, "l0.mix.right.", RIGHT, 1e-5)
    a, st = O.state_space_branch(h[:8], w, "l0.mix.right.", RIGHT, 1e-5)
    b, st = O.state_space_branch(h[8:9], w, "l0.mix.right.", RIGHT, 1e-5, st)
    c, _ = O.state_space_branch(h[9:], w, "l0.mix.right.", RIGHT, 1e-5, st)
    assert torch.allclose(torch.cat([a, b, c]), whole, atol=1e-5)
    assert st[0].shape == (3, 5, 4) and st[1].shape == (2, 22)


def test_oracle_experts_clamp_and_route():
    w = {"gate": torch.eye(3), "up": torch.eye(3), "down": torch.eye(3)}
    y = O.clamped_expert(torch.tensor([[5.0, -5.0, 0.5]]), w, "", 2.0)[0]
    sig = lambda z: 1 / (1 + math.exp(-z))  # noqa: E731
    want = [2.0 * sig(1.702 * 2.0) * 3.0, -5.0 * sig(1.702 * -5.0) * (-2.0 + 1.0), 0.5 * sig(1.702 * 0.5) * 1.5]
    assert torch.allclose(y, torch.tensor(want), atol=1e-6)
    r = {"router": torch.eye(4), "router.b": torch.tensor([0.0, 0.0, 0.0, 10.0])}
    idx, wt = O.route(torch.tensor([[3.0, 1.0, 2.0, -6.0]]), r, "", 2)
    assert idx.tolist() == [[3, 0]] and torch.allclose(wt, torch.softmax(torch.tensor([[4.0, 3.0]]), -1))
