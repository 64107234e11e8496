"""Python front end of the Vamadra host (``libpegainfer_qwen3_host.so``, csrc/host/vamadra_host.cpp).

Vamadra is a decoder whose ``config.json`` lists its layers one by one.  Every layer has a latent-attention mixer
(compressed paged cache, per-head softmax sink, logistic output gate, optionally reading an earlier layer's cache) and
a dense or mixture-of-experts feed-forward; the residual stream is fp32 and each sublayer's *output* is normed.
All sizes and constants come from the configuration; nothing here depends on one particular checkpoint.

Surface, as for the other models of this package: build from a checkpoint folder or a tensor dict, allocate requests,
run ``step`` over a ragged batch (portions of prompts beside single decoded tokens), greedy ``generate``.  Compute runs
in the sm_100a kernels behind the C ABI; there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from dataclasses import dataclass, field

import torch

from . import ffi
from .model import host_lib


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


# ---------------------------------------------------------------- host binding
class _LayerCfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "kv_from", "rot_dims")] + \
               [("rot_base", C.c_float), ("scale", C.c_float), ("has_scaling", C.c_int)] + \
               [(n, C.c_float) for n in ("s_factor", "s_original", "s_fast", "s_slow")] + \
               [(n, C.c_int) for n in ("mlp_kind", "ff", "experts", "top", "groups", "keep")] + \
               [("route_scale", C.c_float), ("expert_ff", C.c_int), ("shared_ff", C.c_int)]


class _ModelCfg(C.Structure):
    _fields_ = [("vocab", C.c_int), ("width", C.c_int), ("n_layers", C.c_int), ("eps", C.c_float)] + \
               [(n, C.c_int) for n in ("f32", "page_size", "num_pages", "max_requests", "device", "enable_pdl")]


def _typed_host():
    h = host_lib()
    if getattr(h, "_pv_typed", False):
        return h
    vp, i32 = C.c_void_p, C.c_int
    h.pv_create_error.restype = C.c_char_p
    h.pv_create.restype = vp
    h.pv_create.argtypes = [C.POINTER(_ModelCfg), C.POINTER(_LayerCfg), C.c_char_p]
    h.pv_destroy.argtypes = [vp]
    h.pv_last_error.restype = C.c_char_p
    h.pv_last_error.argtypes = [vp]
    h.pv_load_tensor.argtypes = [vp, C.c_char_p, vp, i32, i32, i32]
    h.pv_finalize.argtypes = [vp]
    h.pv_request_alloc.argtypes = [vp]
    h.pv_request_free.argtypes = [vp, i32]
    h.pv_seq_len.argtypes = [vp, i32]
    h.pv_available_pages.argtypes = [vp]
    h.pv_page_size.argtypes = [vp]
    h.pv_request_pages.argtypes = [vp, i32, vp, i32]
    h.pv_step.argtypes = [vp, i32, vp, vp, vp, i32, vp, i32, vp, vp]
    h.pv_keep_trail.argtypes = [vp, i32]
    h.pv_use_graph.argtypes = [vp, i32]
    h.pv_graph_count.argtypes = [vp]
    h.pv_copy_trail.argtypes = [vp, vp]
    h.pv_launch_count.restype = C.c_int64
    h.pv_launch_count.argtypes = [vp, i32]
    h.pv_generate.argtypes = [vp, vp, i32, i32, vp, vp, vp]
    h._pv_typed = True
    return h


PAGE_SIZE = 16


def pages_for(max_tokens: int, page_size: int = PAGE_SIZE) -> int:
    """Pool pages for ``max_tokens`` live tokens (every request's share already rounded up to whole pages by the caller)."""
    return (int(max_tokens) + page_size - 1) // page_size


class VamadraModel:
    architecture = "Vamadra"

    def __init__(self, cfg: VamadraConfig, weights, dtype: torch.dtype = torch.bfloat16, max_tokens: int = 0, max_requests: int = 4,
                 device_ordinal: int = 0, enable_pdl: bool = True, kernel_lib: str | None = None):
        """``weights``: dict or iterable of (checkpoint name, tensor).  ``dtype``: bfloat16 (serving precision) or float32 (every
        product in true fp32).  ``max_tokens``: cache pool size in tokens, 0 = a share of free memory."""
        if not torch.cuda.is_available():
            raise RuntimeError("pegainfer_b200 needs a CUDA device (there is no CPU path)")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be torch.bfloat16 or torch.float32")
        self.cfg, self.dtype, self._h = cfg, dtype, _typed_host()
        f32 = int(dtype == torch.float32)
        lcs = (_LayerCfg * len(cfg.layers))()
        for i, l in enumerate(cfg.layers):
            m, f, sc = l.mixer, l.mlp, l.mixer.rot.scaling
            lcs[i] = _LayerCfg(m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, -1 if m.kv_from is None else m.kv_from, m.rot.dims, m.rot.base, m.scale,
                               int(sc is not None), *([sc["factor"], sc["original"], sc["fast"], sc["slow"]] if sc else [1.0, 1.0, 1.0, 1.0]),
                               0 if f is None else (1 if f.kind == "dense" else 2), f.ff if f else 0, f.experts if f else 0, f.top if f else 0,
                               f.groups if f else 1, f.keep if f else 1, f.route_scale if f else 1.0, f.expert_ff if f else 0,
                               f.shared_ff if f else 0)
        mc = _ModelCfg(cfg.vocab, cfg.width, len(cfg.layers), cfg.eps, f32, PAGE_SIZE, pages_for(max_tokens) if max_tokens > 0 else 0,
                       max_requests, device_ordinal, int(enable_pdl))
        torch.cuda.set_device(device_ordinal)
        self._m = self._h.pv_create(C.byref(mc), lcs, (kernel_lib or ffi.KERNEL_LIB_PATH).encode())
        if not self._m:
            raise RuntimeError("pv_create: " + self._h.pv_create_error().decode())
        shapes = weight_shapes(cfg)
        seen = set()
        for name, t in (weights.items() if isinstance(weights, dict) else weights):
            if name not in shapes:  # nothing in the configuration uses it: leave it out, loudly
                import warnings
                warnings.warn(f"{name}: not a tensor of this configuration, ignored")
                continue
            if tuple(t.shape) != tuple(shapes[name]):
                raise ValueError(f"{name}: shape {tuple(t.shape)} != {tuple(shapes[name])} from the configuration")
            if t.is_cuda:
                torch.cuda.current_stream().synchronize()
            t = t.to(dtype).contiguous()
            rows, cols = (t.shape[0], t.shape[1]) if t.dim() == 2 else (1, t.shape[0])
            self._ck(self._h.pv_load_tensor(self._m, name.encode(), t.data_ptr(), rows, cols, f32))
            seen.add(name)
        missing = [n for n in shapes if n not in seen]
        if missing:
            raise KeyError(f"checkpoint misses {missing[:4]}{' ...' if len(missing) > 4 else ''}")
        self._ck(self._h.pv_finalize(self._m))

    @classmethod
    def from_pretrained(cls, model_path: str, **kw) -> "VamadraModel":
        """``config.json`` + ``model.safetensors`` (or a sharded index) of a Vamadra checkpoint."""
        from safetensors import safe_open
        from .weights import load_shard_info
        with open(os.path.join(model_path, "config.json")) as f:
            cfg = VamadraConfig.from_dict(json.load(f), os.path.basename(os.path.normpath(model_path)) or "custom")
        files, _ = load_shard_info(model_path)

        def tensors():
            for p in files:
                with safe_open(p, framework="pt", device="cpu") as h:
                    for name in h.keys():
                        yield name, h.get_tensor(name)
        return cls(cfg, tensors(), **kw)

    def _ck(self, rc):
        if rc != 0:
            raise RuntimeError(self._h.pv_last_error(self._m).decode())

    def close(self):
        if getattr(self, "_m", None):
            self._h.pv_destroy(self._m)
            self._m = None

    __del__ = close

    # -- request state
    def alloc_request(self) -> int:
        rid = self._h.pv_request_alloc(self._m)
        if rid < 0:
            raise RuntimeError(self._h.pv_last_error(self._m).decode())
        return rid

    def drop_request(self, rid: int) -> None:
        self._h.pv_request_free(self._m, rid)

    def seq_len(self, rid: int) -> int:
        return self._h.pv_seq_len(self._m, rid)

    def available_pages(self) -> int:
        return self._h.pv_available_pages(self._m)

    def request_pages(self, rid: int) -> list[int]:
        buf = (C.c_int * 65536)()
        n = self._h.pv_request_pages(self._m, rid, buf, 65536)
        return list(buf[:max(n, 0)])

    # -- one engine step
    def step(self, entries, want=None, sample: bool = False, logits: bool = True):
        """``entries``: [(request id, [token, ...]), ...] -- each request's next tokens (a portion of its prompt or one decoded
        token); all entries run as one batch.  ``want``: per entry the offsets inside its tokens whose logits are wanted
        (default: the last one).  Returns fp32 logits [rows, vocab] on the host in entry order (and greedy tokens with ``sample``);
        ``logits=False`` leaves the logits on the device and returns ``None`` in their place (a generation loop needs the tokens only)."""
        n = len(entries)
        flat, lens, rids, rows, base = [], [], [], [], 0
        for i, (rid, toks) in enumerate(entries):
            w = [len(toks) - 1] if want is None else want[i]
            rows += [base + int(k) for k in w]
            flat += [int(t) for t in toks]
            lens.append(len(toks))
            rids.append(int(rid))
            base += len(toks)
        out = torch.empty((len(rows), self.cfg.vocab), dtype=torch.float32) if logits else None
        sampled = (C.c_int * max(len(rows), 1))()
        self._ck(self._h.pv_step(self._m, n, (C.c_int * len(flat))(*flat), (C.c_int * n)(*lens), (C.c_int * n)(*rids), len(rows),
                                 (C.c_int * max(len(rows), 1))(*rows), int(sample), out.data_ptr() if logits and len(rows) else None, sampled))
        return (out, list(sampled)[:len(rows)]) if sample else out

    def generate(self, prompt: list[int], max_tokens: int):
        """Greedy generation of one request: (tokens, ttft_ms, step_ms[])."""
        out = (C.c_int * max_tokens)()
        ttft = C.c_double()
        steps = (C.c_double * max(1, max_tokens - 1))()
        self._ck(self._h.pv_generate(self._m, (C.c_int * len(prompt))(*prompt), len(prompt), max_tokens, out, C.byref(ttft), steps))
        return list(out), ttft.value, list(steps)[:max_tokens - 1]

    # -- bring-up aid: residual stream after every layer of the last step, [layers, tokens, width]
    def keep_trail(self, on: bool = True) -> None:
        self._h.pv_keep_trail(self._m, int(on))

    def trail(self, tokens: int) -> torch.Tensor:
        out = torch.empty((len(self.cfg.layers), tokens, self.cfg.width), dtype=torch.float32)
        self._ck(self._h.pv_copy_trail(self._m, out.data_ptr()))
        return out

    def use_graph(self, on: bool = True) -> None:
        """Decode steps (one token per entry) replay a captured launch sequence from their second occurrence on; off = always eager."""
        self._h.pv_use_graph(self._m, int(on))

    def graph_count(self) -> int:
        return int(self._h.pv_graph_count(self._m))

    def launch_count(self, reset: bool = False) -> int:
        return int(self._h.pv_launch_count(self._m, int(reset)))
