"""Risolorn without a GPU: configuration round trip, checkpoint naming, registry, and identities of the oracle's mechanisms
(oracle/risolorn_oracle.py) that do not depend on the product path."""
import json
import math

import torch

from oracle import risolorn_oracle as O
from pegainfer_b200.risolorn import RisolornConfig, iter_random_weights, weight_shapes

CFG = {"architecture": "Risolorn", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5}, "logit_scale": 0.25, "layers": [
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "mask": {"size": 7}, "scale": 0.3,
                                    "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}},
     "mlp": {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}},
    {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "conv": 3}, "mlp": None},
    {"type": "mlstm", "mixer": {"heads": 2, "dim": 5, "vdim": 7, "gate_cap": 9.0},
     "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 4, "top": 1, "groups": {"count": 1, "keep": 1}}}},
]}


def test_config_round_trip_and_tensor_names():
    c = RisolornConfig.from_dict(CFG)
    assert RisolornConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c
    s = weight_shapes(c)
    assert s["l0.mix.q"] == (32, 24) and s["l0.mix.k.b"] == (16,) and s["l0.mix.v"] == (12, 24) and s["l0.mix.sink"] == (4,)
    assert s["l0.norm1.alpha"] == () and s["final.norm.b"] == (24,)
    assert s["l1.mix.q"] == (12, 24) and s["l1.mix.v.conv"] == (20, 3) and s["l1.mix.norm"] == (5,) and s["l1.mix.A_log"] == (4,)
    assert s["l2.mix.norm"] == (14,) and s["l2.mix.i.b"] == (2,) and s["l2.mlp.e3.gate"] == (12, 24) and s["l0.mlp.correction"] == (6,)
    assert "l1.mlp.router" not in s
    assert {n for n, _ in iter_random_weights(c)} == set(s)


def test_registry_knows_the_design(tmp_path):
    from pegainfer_b200.registry import FLOAT32_CAPABLE, architecture_of
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert architecture_of(str(tmp_path)) == "Risolorn" and "Risolorn" in FLOAT32_CAPABLE
    from pegainfer_b200 import build
    assert "recurrent_mixers.cu" in build.PARTS_OF["Risolorn"][0] and "layered_host.cpp" in build.PARTS_OF["Risolorn"][1]


def weights(seed=0):
    return {n: t.float() for n, t in iter_random_weights(RisolornConfig.from_dict(CFG), seed)}


def test_oracle_is_causal_and_chunks_count_from_position_zero():
    w = weights()
    toks = torch.randint(0, 50, (30,), generator=torch.Generator().manual_seed(1)).tolist()
    full = O.forward(CFG, w, toks)
    assert torch.allclose(O.forward(CFG, w, toks[:17]), full[:17], atol=1e-5)
    # attention alone: a query at the first position of a chunk sees only itself -> its output is its own value after the sink's share
    mx = CFG["layers"][0]["mixer"]
    h = torch.randn(15, 24, generator=torch.Generator().manual_seed(2))
    out = O.attention_mixer(h, w, "l0.mix.", mx, torch.arange(15))
    alone = O.attention_mixer(h[7:8], w, "l0.mix.", mx, torch.tensor([7]))
    assert torch.allclose(out[7], alone[0], atol=1e-5) and not torch.allclose(out[8], O.attention_mixer(h[8:9], w, "l0.mix.", mx, torch.tensor([8]))[0], atol=1e-4)


def test_oracle_delta_rule_overwrites_a_repeated_key():
    """with full write strength and no decay, writing (k, v2) after (k, v1) leaves exactly v2 readable at k"""
    D, Dv = 6, 5
    g = torch.Generator().manual_seed(3)
    k = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)
    v1, v2 = torch.randn(Dv, generator=g), torch.randn(Dv, generator=g)
    S = torch.zeros(D, Dv)
    for v in (v1, v2):
        S = S + torch.outer(k, 1.0 * (v - S.T @ k))
    assert torch.allclose(S.T @ k, v2, atol=1e-6)


def test_oracle_router_keeps_closed_groups_out_even_with_negative_scores():
    w = {"router": torch.eye(6), "correction": torch.tensor([-3.0, -3.0, -0.1, -4.0, -5.0, -5.0])}
    z = torch.tensor([[0.0, 0.0, 0.0, 0.0, 4.0, 4.0]])
    ids, wt = O.route(z, w, "", {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}})
    # corrected scores: group 0 = (-2.5, -2.5), group 1 = (0.4, -3.5), group 2 = (-4.02, -4.02): groups 1 and 0 stay
    assert sorted(ids[0].tolist()) == [0, 1, 2]
    assert torch.allclose(wt.sort().values, torch.tensor([0.5, 0.5, 0.5]))
    assert math.isclose(float(torch.sigmoid(torch.tensor(4.0))), 0.982, abs_tol=1e-3)
