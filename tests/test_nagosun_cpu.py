"""Nagosun without a GPU: configuration round trip, checkpoint naming, registry, and identities of the oracle's mechanisms
(oracle/nagosun_oracle.py) that do not depend on the product path."""
import json
import math

import torch

from oracle import nagosun_oracle as O
from pegainfer_b200.nagosun import NagosunConfig, iter_random_weights, weight_shapes

CFG = {"architecture": "Nagosun", "vocab": 50, "width": 24, "norm": {"eps": 1e-5, "groups": 3}, "residual_mult": 0.8, "logit_scale": 0.4, "layers": [
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "mask": {"size": 7}, "scale": 0.3, "softcap": 12.0},
     "mlp": {"kind": "dense", "ff": 20}},
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 10, "mask": {"size": 5}, "scale": 0.25,
                                           "rot": {"dims": 4, "base": 100.0}}, "mlp": None},
]}


def test_config_round_trip_and_tensor_names():
    c = NagosunConfig.from_dict(CFG)
    assert NagosunConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c
    assert c.groups == 3 and c.layers[0].mixer.window == 7 and c.layers[1].ff == 0
    s = weight_shapes(c)
    assert s["embed.norm"] == (24,) and s["l0.mix.q"] == (32, 24) and s["l0.mix.k.b"] == (16,) and s["l0.mix.v"] == (12, 24)
    assert s["l0.mix.g"] == (24, 24) and s["l0.mix.o"] == (24, 24) and s["l0.mix.o.b"] == (24,) and s["l0.rg2.b"] == (24,)
    assert s["l1.mix.q"] == (20, 24) and s["l1.mix.dkv"] == (14, 24) and s["l1.mix.dkv.norm"] == (10,) and s["l1.mix.uk"] == (12, 10)
    assert s["l1.mix.uv"] == (10, 10) and s["l1.norm1b"] == (24,)
    for absent in ("l1.norm2", "l1.rg2", "l1.mlp.gate", "l1.mix.o.b", "l1.mix.g", "l0.mix.sink"):
        assert absent not in s
    assert {n for n, _ in iter_random_weights(c)} == set(s)


def test_layer_struct_carries_the_designs_constants():
    from pegainfer_b200.nagosun import NagosunModel
    c = NagosunConfig.from_dict(CFG)
    a, b = NagosunModel.layer_struct(c.layers[0]), NagosunModel.layer_struct(c.layers[1])
    assert (a.mixer_kind, a.window, a.value_norm, a.sink_kind, a.out_gate, a.proj_bias, a.rot_dims) == (1, 7, 1, 2, 1, 1, 0)
    assert math.isclose(a.softcap, 12.0) and math.isclose(a.slope_log2, 8.0)
    assert (b.mixer_kind, b.window, b.value_norm, b.sink_kind, b.out_gate, b.proj_bias, b.rot_dims, b.rot_interleaved) == (0, 5, 0, 1, 0, 0, 4, 1)
    assert b.softcap == 0.0 and b.slope_log2 == 0.0 and b.mlp_kind == 0 and a.mlp_kind == 1 and a.ff == 20


def test_registry_knows_the_design(tmp_path):
    from pegainfer_b200.registry import FLOAT32_CAPABLE, architecture_of
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert architecture_of(str(tmp_path)) == "Nagosun" and "Nagosun" in FLOAT32_CAPABLE
    from pegainfer_b200 import build
    assert "gqa_attention.cu" in build.PARTS_OF["Nagosun"][0] and "latent_attention.cu" in build.PARTS_OF["Nagosun"][0]
    assert "layered_host.cpp" in build.PARTS_OF["Nagosun"][1]


def weights(seed=0):
    return {n: t.float() for n, t in iter_random_weights(NagosunConfig.from_dict(CFG), seed)}


def test_oracle_is_causal_and_a_window_forgets():
    w = weights()
    toks = torch.randint(0, 50, (30,), generator=torch.Generator().manual_seed(1)).tolist()
    full = O.forward(CFG, w, toks)
    assert torch.allclose(O.forward(CFG, w, toks[:17]), full[:17], atol=1e-5)
    # attention alone: the output at position 20 depends on inputs 14 .. 20 (window 7) and on nothing older
    mx = CFG["layers"][0]["mixer"]
    h = torch.randn(25, 24, generator=torch.Generator().manual_seed(2))
    out = O.attention_mixer(h, w, "l0.mix.", mx, torch.arange(25), 1e-5)
    h2 = h.clone()
    h2[13] += 1.0
    assert torch.allclose(O.attention_mixer(h2, w, "l0.mix.", mx, torch.arange(25), 1e-5)[20], out[20], atol=1e-6)
    h2[14] += 1.0
    assert not torch.allclose(O.attention_mixer(h2, w, "l0.mix.", mx, torch.arange(25), 1e-5)[20], out[20], atol=1e-4)


def test_oracle_group_norm_and_sink_identities():
    x = torch.randn(5, 24, generator=torch.Generator().manual_seed(3))
    y = O.group_norm(x, torch.ones(24), 3, 0.0)
    assert torch.allclose(y.reshape(5, 3, 8).pow(2).mean(-1), torch.ones(5, 3), atol=1e-5)
    assert torch.allclose(O.group_norm(x, torch.ones(24), 1, 1e-5), O.unit_rms(x, 1e-5))
    # scaling one group leaves the others alone
    x2 = x.clone()
    x2[:, :8] *= 7.0
    assert torch.allclose(O.group_norm(x2, torch.ones(24), 3, 0.0), y, atol=1e-5)
    # a sink of score zero: weights sum to less than one; with very negative scores almost everything goes to the sink
    s = torch.tensor([[0.0, 0.0, 0.0]])
    ok = torch.ones(1, 3, dtype=torch.bool)
    assert torch.allclose(O.softmax_plus_one(s, ok), torch.full((1, 3), 0.25))
    assert O.softmax_plus_one(s - 50.0, ok).sum() < 1e-20
    assert torch.allclose(O.softmax_plus_one(s + 50.0, ok).sum(), torch.tensor(1.0))
    assert torch.allclose(O.distance_slopes(4), torch.tensor([0.25, 0.0625, 0.015625, 0.00390625]))


def test_oracle_rotation_turns_pairs_and_keeps_relative_angles():
    rot = {"dims": 4, "base": 100.0}
    g = torch.Generator().manual_seed(4)
    q, k = torch.randn(1, 6, generator=g), torch.randn(1, 6, generator=g)
    a = O.rotate_pairs(q, torch.tensor([9]), rot) @ O.rotate_pairs(k, torch.tensor([5]), rot).T
    b = O.rotate_pairs(q, torch.tensor([14]), rot) @ O.rotate_pairs(k, torch.tensor([10]), rot).T
    assert torch.allclose(a, b, atol=1e-5)
    r = O.rotate_pairs(q, torch.tensor([3]), rot)
    assert torch.allclose(r[:, 4:], q[:, 4:]) and torch.allclose(r[:, :2].norm(), q[:, :2].norm(), atol=1e-6)
    assert math.isclose(float(O.rotate_pairs(torch.tensor([[1.0, 0.0, 0.0, 0.0]]), torch.tensor([1]), rot)[0, 1]), math.sin(1.0), abs_tol=1e-6)
