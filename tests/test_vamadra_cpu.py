"""Host-side parts of the Vamadra path that need no GPU: configuration parsing, tensor naming, the registry, the engine's
scheduler and the trace replay tool (both over a fake model), and a few identities of the oracle's mechanisms."""
import io
import json
import math
import os
import sys

import pytest
import torch

from oracle import vamadra_oracle as O
from pegainfer_b200.engine import Engine
from pegainfer_b200.vamadra import VamadraConfig, pages_for, weight_shapes

CFG = {"architecture": "Vamadra", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "layers": [
    {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 40},
     "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 10, "kv_rank": 12, "scale": 0.3,
               "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 2.0, "original": 8, "fast": 4.0, "slow": 1.0}}}},
    {"type": "latent_attention", "mlp": {"kind": "moe", "expert": {"ff": 8}, "shared": {"ff": 16},
                                         "router": {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}},
     "mixer": {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 12, "scale": 0.3, "kv_from": 0, "rot": {"dims": 4, "base": 100.0}}},
    {"type": "latent_attention", "mlp": None,
     "mixer": {"heads": 1, "dim": 8, "rot_dim": 2, "vdim": 8, "kv_rank": 7, "scale": 0.5, "rot": {"dims": 2, "base": 50.0}}},
]}


def test_config_round_trip_and_tensor_names():
    c = VamadraConfig.from_dict(CFG)
    assert VamadraConfig.from_dict(c.to_dict()) == c
    assert c.layers[1].mixer.kv_from == 0 and c.layers[0].mixer.kv_from is None and c.layers[2].mlp is None
    assert c.layers[1].mlp.groups == 3 and c.layers[1].mlp.keep == 2 and c.layers[1].mlp.shared_ff == 16
    s = weight_shapes(c)
    assert s["l0.mix.q"] == (2 * 10, 24) and s["l0.mix.dkv"] == (16, 24) and s["l0.mix.dkv.norm"] == (12,)
    assert "l1.mix.dkv" not in s and "l1.mix.dkv.norm" not in s            # a borrowing layer has no down-projection
    assert s["l1.mix.uk"] == (18, 12) and s["l1.mix.uv"] == (15, 12) and s["l1.mix.o"] == (24, 15) and s["l1.mix.g"] == (3, 24)
    assert s["l1.mlp.e5.up"] == (8, 24) and s["l1.mlp.e5.down"] == (24, 8) and s["l1.mlp.shared.sg"] == (1, 24)
    assert "l2.norm2" not in s and "l2.norm1" in s and s["final.norm"] == (24,) and s["head"] == (50, 24)
    with pytest.raises(ValueError):
        VamadraConfig.from_dict(dict(CFG, layers=[dict(CFG["layers"][0], type="something_else")]))
    assert pages_for(1) == 1 and pages_for(16) == 1 and pages_for(17) == 2


def test_registry_picks_the_class_from_config_json(tmp_path):
    from pegainfer_b200.registry import ARCHITECTURES, FLOAT32_CAPABLE, architecture_of
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert architecture_of(str(tmp_path)) == "Vamadra" and "Vamadra" in FLOAT32_CAPABLE
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3"}))
    assert architecture_of(str(tmp_path)) == "Qwen3ForCausalLM"
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["NoSuchModel"]}))
    with pytest.raises(KeyError):
        architecture_of(str(tmp_path))
    assert set(FLOAT32_CAPABLE) <= set(ARCHITECTURES)


class FakeModel:
    """Stands in for a model behind the engine: checks slot discipline, records every step, 'samples' last token + 1."""

    def __init__(self, slots, vocab=100):
        self.free, self.len, self.steps, self.vocab = list(range(slots)), {}, [], vocab

    def alloc_request(self):
        if not self.free:
            raise RuntimeError("every request slot is in use")
        rid = self.free.pop(0)
        self.len[rid] = 0
        return rid

    def drop_request(self, rid):
        del self.len[rid]
        self.free.append(rid)

    def step(self, entries, want=None, sample=False, logits=True):
        assert len({r for r, _ in entries}) == len(entries) and all(r in self.len for r, _ in entries)
        self.steps.append([(r, list(t)) for r, t in entries])
        rows = []
        for i, (r, t) in enumerate(entries):
            assert len(t) > 0
            self.len[r] += len(t)
            for k in ([len(t) - 1] if want is None else want[i]):
                rows.append((t[k] + 1) % self.vocab)
        logits = torch.zeros(len(rows), self.vocab)
        for i, v in enumerate(rows):
            logits[i, v] = 1.0
        return (logits, rows) if sample else logits


def test_scheduler_batches_portions_beside_decoding_requests():
    m = FakeModel(slots=2)
    prompts = [[1, 2, 3, 4, 5, 6, 7], [10], [20, 21, 22]]
    out = Engine(m).generate(prompts, max_new_tokens=3, max_live=2, token_budget=4)
    assert out == [[8, 9, 10], [11, 12, 13], [23, 24, 25]]
    assert all(sum(len(t) for _, t in s) <= 4 for s in m.steps)            # the token budget holds in every step
    assert all(len(s) <= 2 for s in m.steps)                               # never more live requests than slots
    assert any(len(s) == 2 and {len(t) for _, t in s} == {1, 3} for s in m.steps)  # a decoded token beside a prompt portion
    assert sorted(m.free) == [0, 1] and not m.len                          # everything was given back
    fed = [t for s in m.steps for r, t in s if t[0] in (1, 2, 3, 4, 5, 6, 7) and len(t) > 1 or t == [7]]
    assert [x for t in fed for x in t][:7] == [1, 2, 3, 4, 5, 6, 7]       # the long prompt went through in order, in portions


def test_scheduler_stops_on_stop_ids():
    out = Engine(FakeModel(slots=1)).generate([[5], [40]], max_new_tokens=10, max_live=1, stop_ids=(8,))
    assert out == [[6, 7, 8], list(range(41, 51))]


def test_engine_explicit_steps_admit_and_release():
    m = FakeModel(slots=2)
    e = Engine(m)
    lg = e.step([("x", [1, 2, 3], [0, 2]), ("y", [9], [])])
    assert lg.shape == (2, 100) and lg[0].argmax() == 2 and lg[1].argmax() == 4
    e.step([("x", [4], [0])], end=["x"])
    assert "x" not in e.slots and m.len == {e.slots["y"]: 1}
    e.step([("z", [1], [0]), ("y", [2], [0])], end=["y", "z"])             # z reuses the slot x held
    assert not e.slots and sorted(m.free) == [0, 1]
    assert e.step([("w", [], [])]).shape[0] == 0 and "w" in e.slots and len(m.steps) == 3  # admitted, nothing ran
    assert e.step([("w", [], []), ("v", [3, 4], [1])]).shape[0] == 1                       # an empty entry beside a real one
    e.release("w"), e.release("v")


def test_trace_replay_writes_logits_and_done_lines(tmp_path, monkeypatch, capsys):
    from pegainfer_b200 import build, registry, trace
    (tmp_path / "m").mkdir()
    (tmp_path / "m" / "config.json").write_text(json.dumps(CFG))
    made = {}

    def fake_load(path, dtype, max_tokens=0, max_requests=4, **kw):
        made.update(dtype=dtype, max_tokens=max_tokens, max_requests=max_requests)
        made["model"] = FakeModel(slots=max_requests, vocab=50)
        return made["model"]
    monkeypatch.setattr(registry, "load_model", fake_load)
    monkeypatch.setattr(build, "build", lambda **kw: None)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}, {"id": "b", "tokens": [7], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": [8, 9], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]}]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    out = tmp_path / "out"
    assert trace.main(["--model", str(tmp_path / "m"), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"]) == 0
    assert capsys.readouterr().out.split("\n")[:3] == ["done 0", "done 1", "done 2"]
    assert made["dtype"] == "float32" and made["max_tokens"] == 128 and made["max_requests"] == 4
    import numpy as np
    a0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, 50)
    assert a0[0].argmax() == 6 and a0[1].argmax() == 4
    assert not (out / "1.f32").exists() and np.fromfile(out / "2.f32", dtype="<f4").shape == (50,)
    assert not made["model"].len                                            # ended requests were released


def test_trace_refuses_float32_for_a_bf16_only_design(tmp_path, monkeypatch):
    from pegainfer_b200 import trace
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["Qwen3ForCausalLM"]}))
    monkeypatch.setattr(sys, "stdin", io.StringIO(""))
    assert trace.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"]) == 3


# ------------------------------------------------------------------ identities of the oracle's mechanisms
def test_oracle_sink_and_causal_mask():
    g = torch.Generator().manual_seed(0)
    qn, qr, kn, kr, v = (torch.randn(5, d, generator=g) for d in (4, 2, 4, 2, 3))
    pos = torch.arange(5)
    no_sink = O.sink_softmax_attention(qn, qr, kn, kr, v, torch.tensor(-1e30), 0.7, pos, pos)
    s = ((qn @ kn.T + qr @ kr.T) * 0.7).masked_fill(pos[None] > pos[:, None], float("-inf"))
    assert torch.allclose(no_sink, torch.softmax(s, -1) @ v, atol=1e-6)
    with_sink = O.sink_softmax_attention(qn, qr, kn, kr, v, torch.tensor(0.4), 0.7, pos, pos)
    shrink = torch.exp(s).sum(-1) / (torch.exp(s).sum(-1) + math.exp(0.4))
    assert torch.allclose(with_sink, no_sink * shrink[:, None], atol=1e-6)
    assert torch.allclose(with_sink[0], v[0] * shrink[0], atol=1e-6)       # the first token sees itself only


def test_oracle_rotation_and_yarn_table():
    f, mag = O.rotary_frequencies({"dims": 8, "base": 10000.0})
    assert mag == 1.0 and torch.allclose(f, torch.tensor([1.0, 0.1, 0.01, 0.001]))
    rot = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 0.5}}
    fy, my = O.rotary_frequencies(rot)
    assert abs(my - (0.1 * math.log(4.0) + 1)) < 1e-7 and fy[0] == f[0] and abs(fy[3] - f[3] / 4) < 1e-9  # fast pair kept, slow pair / factor
    x = torch.randn(3, 2, 10, generator=torch.Generator().manual_seed(1))
    y = O.rotate(x, torch.tensor([0, 5, 9]), {"dims": 8, "base": 10000.0})
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])               # entries past dims pass; position 0 is identity
    assert torch.allclose(y[..., :8].pow(2).sum(-1), x[..., :8].pow(2).sum(-1), atol=1e-5)  # a rotation keeps the norm


def test_oracle_router_weights():
    z = torch.randn(9, 12, generator=torch.Generator().manual_seed(2))
    ids, w = O.grouped_top_router(z, 3, 4, 2, 1.5)
    assert torch.allclose(w.sum(-1), torch.full((9,), 1.5), atol=1e-6)
    s = torch.softmax(z, -1)
    best_groups = s.reshape(9, 4, 3).max(-1).values.topk(2, -1).indices
    for t in range(9):
        assert {int(e) // 3 for e in ids[t]} <= set(best_groups[t].tolist())
    ids1, _ = O.grouped_top_router(z, 3, 1, 1, 1.0)
    assert torch.equal(ids1.sort(-1).values, s.topk(3, -1).indices.sort(-1).values)        # one group: plain top-k
