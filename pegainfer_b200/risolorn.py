"""The Risolorn design on the layer-list host (``pegainfer_b200/layered.py``, csrc/host/layered_host.cpp).

Risolorn is a decoder whose ``config.json`` lists its layers one by one.  A layer reads ONE Dynamic-Tanh norm of the fp32
residual stream and adds the sum of its mixer and its mixture-of-experts feed-forward, both fed by that norm's output
(``x += mixer(h) + ff(h)``).  Three mixers:

* ``attention`` -- grouped-query softmax attention with projection biases, an interleaved rotary embedding over the first
  ``rot.dims`` entries of each head (optionally YaRN-blended frequencies), a chunk-local causal mask (``mask.size``) and a
  learned per-head sink in the softmax denominator; paged K/V cache.
* ``delta`` -- the gated delta rule behind short causal convolutions; fp32 matrix state per head plus the convolutions' tails
  in a per-request state slot.
* ``mlstm`` -- the matrix memory of xLSTM with soft-capped exponential gates and a running maximum; fp32 state slot.

The feed-forward routes with logistic scores, a per-expert correction for the choice only and group-limited top-k (a group
scores as the sum of its two best corrected scores); experts are gated-SiLU.  Embedding and logits carry multipliers.
All sizes and constants come from the configuration; nothing here depends on one particular checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .layered import LayerCfg, LayeredModel, ModelCfg
from .vamadra import RotaryConfig

MIXER_KINDS = {"attention": 1, "delta": 2, "mlstm": 3}


@dataclass(frozen=True)
class MixerConfig:
    kind: str            # "attention" | "delta" | "mlstm"
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0    # attention: key/value heads; delta: query/key heads; mlstm: = heads
    scale: float = 1.0   # attention
    chunk: int = 0       # attention: mask.size
    rot: RotaryConfig | None = None
    conv: int = 0        # delta: taps
    gate_cap: float = 0.0  # mlstm

    @staticmethod
    def parse(kind: str, d: dict) -> "MixerConfig":
        if kind not in MIXER_KINDS:
            raise ValueError(f"unknown mixer type {kind!r}")
        heads, dim, vdim = int(d["heads"]), int(d["dim"]), int(d["vdim"])
        kv = int(d.get("kv_heads") or heads)
        if kind == "attention":  # no mask block: plain causal; no rot block: nothing rotates
            rot = RotaryConfig.parse(d["rot"]) if d.get("rot") else RotaryConfig(0, 1.0, None)
            return MixerConfig(kind, heads, dim, vdim, kv, float(d["scale"]), int((d.get("mask") or {}).get("size", 0)), rot)
        if kind == "delta":
            return MixerConfig(kind, heads, dim, vdim, kv, conv=int(d["conv"]))
        return MixerConfig(kind, heads, dim, vdim, heads, gate_cap=float(d["gate_cap"]))

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.kind == "attention":
            d.update(kv_heads=self.kv_heads, scale=self.scale)
            if self.chunk:
                d["mask"] = {"size": self.chunk}
            if self.rot.dims:
                d["rot"] = {"dims": self.rot.dims, "base": self.rot.base}
                if self.rot.scaling:
                    d["rot"]["scaling"] = dict(self.rot.scaling)
        elif self.kind == "delta":
            d.update(kv_heads=self.kv_heads, conv=self.conv)
        else:
            d.update(gate_cap=self.gate_cap)
        return d


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    groups: int
    keep: int
    ff: int

    @staticmethod
    def parse(d: dict | None) -> "ExpertsConfig | None":
        if not d:
            return None
        if d.get("kind") != "moe":
            raise ValueError(f"unknown feed-forward kind {d.get('kind')!r}")
        r = d["router"]
        g = r.get("groups") or {"count": 1, "keep": 1}
        return ExpertsConfig(int(r["experts"]), int(r["top"]), int(g["count"]), int(g["keep"]), int(d["expert"]["ff"]))

    def to_dict(self) -> dict:
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top, "groups": {"count": self.groups, "keep": self.keep}}}


@dataclass(frozen=True)
class RisolornLayerConfig:
    mixer: MixerConfig
    mlp: ExpertsConfig | None


@dataclass(frozen=True)
class RisolornConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    logit_scale: float
    layers: tuple = field(default_factory=tuple)
    name: str = "custom"

    @staticmethod
    def from_dict(raw: dict, name: str = "custom") -> "RisolornConfig":
        layers = tuple(RisolornLayerConfig(MixerConfig.parse(l["type"], l["mixer"]), ExpertsConfig.parse(l.get("mlp"))) for l in raw["layers"])
        return RisolornConfig(int(raw["vocab"]), int(raw["width"]), float(raw["norm"]["eps"]), float(raw["embedding"]["scale"]),
                              float(raw["logit_scale"]), layers, name)

    def to_dict(self) -> dict:
        """The ``config.json`` form (round-trips through ``from_dict``)."""
        return {"architecture": "Risolorn", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embed_scale}, "logit_scale": self.logit_scale,
                "layers": [{"type": l.mixer.kind, "mixer": l.mixer.to_dict(), "mlp": l.mlp.to_dict() if l.mlp else None} for l in self.layers]}


def weight_shapes(c: RisolornConfig) -> dict:
    """Checkpoint tensor name -> shape (linear weights are [out, in]; a scalar is ())."""
    W = c.width
    s = {"embed": (c.vocab, W)}

    def norm(name):
        s[name], s[name + ".b"], s[name + ".alpha"] = (W,), (W,), ()

    for i, l in enumerate(c.layers):
        m, p = l.mixer, f"l{i}."
        norm(p + "norm1")
        H, G, D, Dv = m.heads, m.kv_heads, m.dim, m.vdim
        if m.kind == "attention":
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                s[p + "mix." + n], s[p + "mix." + n + ".b"] = (rows, W), (rows,)
            s[p + "mix.sink"] = (H,)
        elif m.kind == "delta":
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                s[p + "mix." + n], s[p + "mix." + n + ".conv"] = (rows, W), (rows, m.conv)
            s[p + "mix.b"], s[p + "mix.a"] = (H, W), (H, W)
            s[p + "mix.A_log"], s[p + "mix.dt_bias"] = (H,), (H,)
            s[p + "mix.norm"] = (Dv,)
            s[p + "mix.g"] = (H * Dv, W)
        else:
            s[p + "mix.q"], s[p + "mix.k"], s[p + "mix.v"], s[p + "mix.g"] = (H * D, W), (H * D, W), (H * Dv, W), (H * Dv, W)
            s[p + "mix.norm"] = (H * Dv,)
            for n in ("i", "f"):
                s[p + "mix." + n], s[p + "mix." + n + ".b"] = (H, W), (H,)
        s[p + "mix.o"] = (W, H * Dv)
        f = l.mlp
        if f is not None:
            for e in range(f.experts):
                s[f"{p}mlp.e{e}.gate"], s[f"{p}mlp.e{e}.up"], s[f"{p}mlp.e{e}.down"] = (f.ff, W), (f.ff, W), (W, f.ff)
            s[p + "mlp.router"], s[p + "mlp.correction"] = (f.experts, W), (f.experts,)
    norm("final.norm")
    s["head"] = (c.vocab, W)
    return s


def iter_random_weights(c: RisolornConfig, seed: int = 0, device: str = "cpu"):
    """Random-init checkpoint (bf16): projections N(0, 1/fan_in) so activations stay O(1); norm weights near one, biases, sinks and
    gate parameters of order one."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def rn(shape, std=1.0):
        return std * torch.randn(shape, generator=g, device=device)

    for name, shape in weight_shapes(c).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "alpha":
            t = torch.tensor(0.7, device=device) + 0.1 * rn(())
        elif name.endswith(("norm1", "final.norm", "mix.norm")):
            t = 1.0 + 0.1 * rn(shape)
        elif leaf == "conv":
            t = rn(shape, 0.5)
        elif leaf == "correction":
            t = rn(shape, 0.3)
        elif leaf == "A_log":
            t = rn(shape, 0.5) - 1.0
        elif len(shape) == 1:
            t = rn(shape, 0.5 if leaf in ("sink", "dt_bias") or name.endswith((".i.b", ".f.b")) else 0.1)
        elif name == "embed":
            t = rn(shape)
        else:
            t = rn(shape) / shape[1] ** 0.5
        yield name, t.to(torch.bfloat16)


# ---------------------------------------------------------------- the model class
def _layer_struct(l: RisolornLayerConfig) -> LayerCfg:
    m, f = l.mixer, l.mlp
    sc = m.rot.scaling if m.rot else None
    return LayerCfg(heads=m.heads, dim=m.dim, rot_dim=0, vdim=m.vdim, kv_rank=0, kv_from=-1, rot_dims=m.rot.dims if m.rot else 0,
                    rot_base=m.rot.base if m.rot else 1.0, scale=m.scale, has_scaling=int(sc is not None),
                    s_factor=sc["factor"] if sc else 1.0, s_original=sc["original"] if sc else 1.0, s_fast=sc["fast"] if sc else 1.0,
                    s_slow=sc["slow"] if sc else 1.0, mlp_kind=2 if f else 0, ff=0, experts=f.experts if f else 0, top=f.top if f else 0,
                    groups=f.groups if f else 1, keep=f.keep if f else 1, route_scale=1.0, expert_ff=f.ff if f else 0, shared_ff=0,
                    mixer_kind=MIXER_KINDS[m.kind], kv_heads=m.kv_heads, chunk=m.chunk, conv=m.conv, rot_interleaved=1, gate_cap=m.gate_cap,
                    router_kind=1, expert_act=1)


def _model_struct(cfg: RisolornConfig, mc: ModelCfg) -> ModelCfg:
    mc.block_kind, mc.embed_scale, mc.logit_scale = 1, cfg.embed_scale, cfg.logit_scale
    return mc


class RisolornModel(LayeredModel):
    architecture = "Risolorn"
    config_class = RisolornConfig
    weight_shapes = staticmethod(weight_shapes)
    layer_struct = staticmethod(_layer_struct)
    model_struct = staticmethod(_model_struct)
