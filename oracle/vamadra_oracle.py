"""Plain, slow restatement of the Vamadra design in fp32 PyTorch on the CPU: one function per mechanism.

Test infrastructure only; it shares no code with the product path (``pegainfer_b200/vamadra.py`` and the
CUDA kernels behind it).  Weights are a dict ``name -> tensor`` with the checkpoint's tensor names, configuration is
the parsed ``config.json`` dict.  Everything is computed in fp32 over the whole sequence at once.

Notation: ``h`` is a [T, width] block of one sequence, positions are 0..T-1 unless given.
"""
from __future__ import annotations

import math

import torch

F32 = torch.float32


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is an offset from one: unit_rms(x) * (1 + w)."""
    return unit_rms(x, eps) * (1.0 + w.to(F32))


def plain_norm(x, w, eps):
    return unit_rms(x, eps) * w.to(F32)


def rotary_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """(angular frequency per rotated pair [dims/2], factor on cos and sin) for a ``rot`` block of the config.

    Without ``scaling``: f_i = base^(-2i/dims), factor 1.  With YaRN scaling the pairs whose wavelength is long against
    the original context are slowed down by ``factor``, short ones are kept, and a linear ramp blends in between."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f.to(F32), 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def pair_index(turns):  # the pair that makes `turns` full turns over the original context
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(pair_index(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    f = f / factor * ramp + f * (1 - ramp)
    return f.to(F32), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, pos: torch.Tensor, rot: dict) -> torch.Tensor:
    """Rotary embedding of the first ``rot['dims']`` entries of the last axis; pair (i, i + dims/2).  x [T, ..., d], pos [T]."""
    dims = int(rot["dims"])
    half = dims // 2
    f, m = rotary_frequencies(rot)
    a = pos.to(F32)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = (torch.cos(a) * m).reshape(shape), (torch.sin(a) * m).reshape(shape)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], dim=-1)


def latent_kv(h, w, pre, mx, eps, pos):
    """What a latent-attention layer stores per token: (normed latent c [T, kv_rank], rotated shared key part [T, rot_dim])."""
    r = int(mx["kv_rank"])
    d = h @ w[pre + "dkv"].to(F32).T
    c = plain_norm(d[:, :r], w[pre + "dkv.norm"], eps)
    kr = rotate(d[:, r:], pos, mx["rot"])
    return c, kr


def sink_softmax_attention(qn, qr, kn, kr, v, sink, scale, q_pos, k_pos):
    """Causal attention of one head with a learned sink in the softmax denominator.

    qn [Tq, dim], qr [Tq, rot], kn [Tk, dim], kr [Tk, rot], v [Tk, vdim]; key j is visible to query i iff k_pos[j] <= q_pos[i].
    The sink adds exp(sink) to the denominator (unscaled, once) and carries no value."""
    s = (qn @ kn.T + qr @ kr.T) * scale
    s = s.masked_fill(k_pos[None, :] > q_pos[:, None], float("-inf"))
    m = torch.maximum(s.max(-1, keepdim=True).values, sink.reshape(1, 1))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True) + torch.exp(sink.reshape(1, 1) - m)
    return (e / den) @ v


def latent_attention(h, w, pre, mx, c, kr, pos, k_pos):
    """The mixer: queries from h, keys/values expanded from the cached latent (c, kr) of this or another layer."""
    H, dim, rd, vd = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"])
    T = h.shape[0]
    q = (h @ w[pre + "q"].to(F32).T).reshape(T, H, dim + rd)
    qn, qr = q[..., :dim], rotate(q[..., dim:], pos, mx["rot"])
    kn = (c @ w[pre + "uk"].to(F32).T).reshape(-1, H, dim)
    v = (c @ w[pre + "uv"].to(F32).T).reshape(-1, H, vd)
    gate = torch.sigmoid(h @ w[pre + "g"].to(F32).T)  # [T, H]
    sink = w[pre + "sink"].to(F32)
    heads = []
    for a in range(H):
        o = sink_softmax_attention(qn[:, a], qr[:, a], kn[:, a], kr, v[:, a], sink[a], float(mx["scale"]), pos, k_pos)
        heads.append(o * gate[:, a:a + 1])
    return torch.cat(heads, dim=-1) @ w[pre + "o"].to(F32).T


def dense_ff(h, w, pre):
    g = h @ w[pre + "gate"].to(F32).T
    u = h @ w[pre + "up"].to(F32).T
    return (torch.nn.functional.silu(g) * u) @ w[pre + "down"].to(F32).T


def relu2_expert(h, up, down):
    return torch.relu(h @ up.to(F32).T).pow(2) @ down.to(F32).T


def grouped_top_router(z, top, group_count, group_keep, scale):
    """Softmax scores; only experts of the ``group_keep`` groups with the largest best score are eligible; the ``top`` best
    eligible experts get weight score / sum(chosen scores) * scale.  Returns (expert ids [T, top], weights [T, top])."""
    T, E = z.shape
    s = torch.softmax(z.to(F32), dim=-1)
    per = E // group_count
    gs = s.reshape(T, group_count, per).max(-1).values
    kept = gs.topk(group_keep, dim=-1).indices
    ok = torch.zeros(T, group_count, dtype=torch.bool)
    ok.scatter_(1, kept, True)
    elig = ok[:, :, None].expand(T, group_count, per).reshape(T, E)
    ids = s.masked_fill(~elig, -1.0).topk(top, dim=-1).indices
    ws = s.gather(1, ids)
    return ids, ws / (ws.sum(-1, keepdim=True) + 1e-20) * scale


def moe_ff(h, w, pre, mlp):
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    ids, ws = grouped_top_router(h @ w[pre + "router"].to(F32).T, int(r["top"]), int(groups["count"]), int(groups["keep"]),
                                 float(r.get("scale", 1.0)))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), ws[t]):
            out[t] += g * relu2_expert(h[t:t + 1], w[f"{pre}e{e}.up"], w[f"{pre}e{e}.down"])[0]
    if mlp.get("shared"):
        sh = relu2_expert(h, w[pre + "shared.up"], w[pre + "shared.down"])
        out = out + sh * torch.sigmoid(h @ w[pre + "shared.sg"].to(F32).T)
    return out


def forward(cfg: dict, w: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (fp32); with ``return_layers`` also the residual after every layer."""
    eps = float(cfg["norm"]["eps"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tok))
    x = w["embed"].to(F32)[tok]
    stored, trail = {}, []
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "latent_attention":
            raise ValueError(f"layer {i}: unknown mixer {layer['type']}")
        mx, pre = layer["mixer"], f"l{i}.mix."
        if mx.get("kv_from") is None:
            stored[i] = latent_kv(x, w, pre, mx, eps, pos)
            c, kr = stored[i]
        else:
            c, kr = stored[int(mx["kv_from"])]
        x = x + offset_norm(latent_attention(x, w, pre, mx, c, kr, pos, pos), w[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp:
            y = dense_ff(x, w, f"l{i}.mlp.") if mlp["kind"] == "dense" else moe_ff(x, w, f"l{i}.mlp.", mlp)
            x = x + offset_norm(y, w[f"l{i}.norm2"], eps)
        trail.append(x.clone())
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].to(F32).T
    return (logits, torch.stack(trail)) if return_layers else logits
