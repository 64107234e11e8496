"""The Vamadra design on the layer-list host (``pegainfer_b200/layered.py``, csrc/host/layered_host.cpp).

Vamadra is a decoder whose ``config.json`` lists its layers one by one.  Every layer has a latent-attention mixer
(compressed paged cache, per-head softmax sink, logistic output gate, optionally reading an earlier layer's cache) and
a dense or mixture-of-experts feed-forward; the residual stream is fp32 and each sublayer's *output* is normed.
All sizes and constants come from the configuration; nothing here depends on one particular checkpoint.

Surface, as for the other models of this package: build from a checkpoint folder or a tensor dict, allocate requests,
run ``step`` over a ragged batch (portions of prompts beside single decoded tokens), greedy ``generate``.  Compute runs
in the sm_100a kernels behind the C ABI; there is no fallback path.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .layered import PAGE_SIZE, LayerCfg, LayeredModel, pages_for  # noqa: F401  (PAGE_SIZE / pages_for: part of this module's surface)


# ---------------------------------------------------------------- configuration
@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    scaling: dict | None = None  # YaRN: factor, original, fast, slow

    @staticmethod
    def parse(d: dict) -> "RotaryConfig":
        sc = d.get("scaling") or None
        if sc is not None:
            sc = {k: float(sc[k]) for k in ("factor", "original", "fast", "slow")}
        return RotaryConfig(int(d["dims"]), float(d["base"]), sc)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int        # unrotated query/key entries per head
    rot_dim: int    # rotated entries per head (the key part of this width is shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    kv_from: int | None = None

    @staticmethod
    def parse(d: dict) -> "LatentAttentionConfig":
        kf = d.get("kv_from")
        return LatentAttentionConfig(int(d["heads"]), int(d["dim"]), int(d["rot_dim"]), int(d["vdim"]), int(d["kv_rank"]), float(d["scale"]),
                                     RotaryConfig.parse(d["rot"]), None if kf is None else int(kf))


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                    # "dense" | "moe"
    ff: int = 0                  # dense hidden size
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    route_scale: float = 1.0
    expert_ff: int = 0
    shared_ff: int = 0           # 0: no shared expert

    @staticmethod
    def parse(d: dict | None) -> "FeedForwardConfig | None":
        if not d:
            return None
        if d["kind"] == "dense":
            return FeedForwardConfig("dense", ff=int(d["ff"]))
        if d["kind"] != "moe":
            raise ValueError(f"unknown feed-forward kind {d['kind']!r}")
        r = d["router"]
        g = r.get("groups") or {"count": 1, "keep": 1}
        sh = d.get("shared") or None
        return FeedForwardConfig("moe", experts=int(r["experts"]), top=int(r["top"]), groups=int(g["count"]), keep=int(g["keep"]),
                                 route_scale=float(r.get("scale", 1.0)), expert_ff=int(d["expert"]["ff"]), shared_ff=int(sh["ff"]) if sh else 0)


@dataclass(frozen=True)
class VamadraLayerConfig:
    mixer: LatentAttentionConfig
    mlp: FeedForwardConfig | None


@dataclass(frozen=True)
class VamadraConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple = field(default_factory=tuple)
    name: str = "custom"

    @staticmethod
    def from_dict(raw: dict, name: str = "custom") -> "VamadraConfig":
        layers = []
        for i, l in enumerate(raw["layers"]):
            if l["type"] != "latent_attention":
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            layers.append(VamadraLayerConfig(LatentAttentionConfig.parse(l["mixer"]), FeedForwardConfig.parse(l.get("mlp"))))
        return VamadraConfig(int(raw["vocab"]), int(raw["width"]), float(raw["norm"]["eps"]), tuple(layers), name)

    def to_dict(self) -> dict:
        """The ``config.json`` form (round-trips through ``from_dict``)."""
        out = []
        for l in self.layers:
            m = l.mixer
            mx = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                  "rot": {"dims": m.rot.dims, "base": m.rot.base}}
            if m.rot.scaling:
                mx["rot"]["scaling"] = dict(m.rot.scaling)
            if m.kv_from is not None:
                mx["kv_from"] = m.kv_from
            f = l.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.expert_ff},
                       "router": {"experts": f.experts, "top": f.top, "scale": f.route_scale, "groups": {"count": f.groups, "keep": f.keep}}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            out.append({"type": "latent_attention", "mixer": mx, "mlp": mlp})
        return {"architecture": "Vamadra", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps}, "layers": out}


def weight_shapes(c: VamadraConfig) -> dict:
    """Checkpoint tensor name -> shape (linear weights are [out, in])."""
    W = c.width
    s = {"embed": (c.vocab, W)}
    for i, l in enumerate(c.layers):
        m, p = l.mixer, f"l{i}."
        s[p + "norm1"] = (W,)
        if l.mlp is not None:
            s[p + "norm2"] = (W,)
        s[p + "mix.q"] = (m.heads * (m.dim + m.rot_dim), W)
        if m.kv_from is None:
            s[p + "mix.dkv"] = (m.kv_rank + m.rot_dim, W)
            s[p + "mix.dkv.norm"] = (m.kv_rank,)
        s[p + "mix.uk"] = (m.heads * m.dim, m.kv_rank)
        s[p + "mix.uv"] = (m.heads * m.vdim, m.kv_rank)
        s[p + "mix.sink"] = (m.heads,)
        s[p + "mix.g"] = (m.heads, W)
        s[p + "mix.o"] = (W, m.heads * m.vdim)
        f = l.mlp
        if f is None:
            continue
        if f.kind == "dense":
            s[p + "mlp.gate"] = (f.ff, W)
            s[p + "mlp.up"] = (f.ff, W)
            s[p + "mlp.down"] = (W, f.ff)
        else:
            for e in range(f.experts):
                s[f"{p}mlp.e{e}.up"] = (f.expert_ff, W)
                s[f"{p}mlp.e{e}.down"] = (W, f.expert_ff)
            s[p + "mlp.router"] = (f.experts, W)
            if f.shared_ff:
                s[p + "mlp.shared.up"] = (f.shared_ff, W)
                s[p + "mlp.shared.down"] = (W, f.shared_ff)
                s[p + "mlp.shared.sg"] = (1, W)
    s["final.norm"] = (W,)
    s["head"] = (c.vocab, W)
    return s


def iter_random_weights(c: VamadraConfig, seed: int = 0, device: str = "cpu"):
    """Random-init checkpoint (bf16): projections N(0, 1/fan_in) so activations stay O(1), norm offsets and sinks near zero."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    for name, shape in weight_shapes(c).items():
        if name.endswith("dkv.norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=device)
        elif name.endswith("sink"):
            t = torch.randn(shape, generator=g, device=device)
        elif len(shape) == 1:
            t = 0.1 * torch.randn(shape, generator=g, device=device)
        elif name == "embed":
            t = torch.randn(shape, generator=g, device=device)
        else:
            t = torch.randn(shape, generator=g, device=device) / shape[1] ** 0.5
        yield name, t.to(torch.bfloat16)


# ---------------------------------------------------------------- the model class
def _layer_struct(l: VamadraLayerConfig) -> LayerCfg:
    m, f, sc = l.mixer, l.mlp, l.mixer.rot.scaling
    return LayerCfg(m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, -1 if m.kv_from is None else m.kv_from, m.rot.dims, m.rot.base, m.scale,
                    int(sc is not None), *([sc["factor"], sc["original"], sc["fast"], sc["slow"]] if sc else [1.0, 1.0, 1.0, 1.0]),
                    0 if f is None else (1 if f.kind == "dense" else 2), f.ff if f else 0, f.experts if f else 0, f.top if f else 0,
                    f.groups if f else 1, f.keep if f else 1, f.route_scale if f else 1.0, f.expert_ff if f else 0,
                    f.shared_ff if f else 0)  # mixer_kind 0 (latent attention), softmax router, relu^2 experts: the remaining fields stay 0


class VamadraModel(LayeredModel):
    architecture = "Vamadra"
    config_class = VamadraConfig
    weight_shapes = staticmethod(weight_shapes)
    layer_struct = staticmethod(_layer_struct)
