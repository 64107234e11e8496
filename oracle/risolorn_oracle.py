"""Plain, slow restatement of the Risolorn design in fp32 PyTorch on the CPU: one function per mechanism.

Test infrastructure only; it shares no code with the product path (``pegainfer_b200/risolorn.py`` and the CUDA
kernels behind it).  Weights are a dict ``name -> tensor`` with the checkpoint's tensor names, configuration is the
parsed ``config.json`` dict.  Everything is computed in fp32, token by token where the design is a recurrence.

Risolorn: a decoder whose ``config.json`` lists its layers.  A layer reads one Dynamic-Tanh norm of the fp32 residual
and adds the sum of a mixer and a mixture-of-experts feed-forward, both fed by that norm's output.  Mixers: softmax
attention with biases, interleaved (optionally YaRN-blended) rotary embedding, a chunk-local causal mask and a learned
sink; the gated delta rule behind short causal convolutions; the matrix memory of xLSTM with stabilised
exponential gates.
"""
from __future__ import annotations

import math

import torch

F32 = torch.float32


def f32(t):
    return t.to(F32)


def dyt(x, w, pre):
    """Dynamic Tanh: tanh(alpha x) * weight + bias."""
    return torch.tanh(f32(w[pre + ".alpha"]) * x) * f32(w[pre]) + f32(w[pre + ".b"])


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


# ---------------------------------------------------------------- rotary embedding
def rotary_frequencies(rot: dict):
    """(angular frequency per pair [dims / 2], factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, pos, rot):
    """x [T, heads, d]; entries (2i, 2i + 1) of the first ``dims`` form a pair; the rest pass."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    a = (pos.to(torch.float64)[:, None] * f[None, :])
    cos, sin = f32(torch.cos(a) * mag)[:, None, :], f32(torch.sin(a) * mag)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ---------------------------------------------------------------- mixers
def attention_mixer(h, w, pre, mx, pos):
    """Chunk-local causal softmax attention with a sink.  h [T, width] of one sequence at positions ``pos``."""
    H, G, D, Dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    T = h.shape[0]
    q = (h @ f32(w[pre + "q"]).T + f32(w[pre + "q.b"])).view(T, H, D)
    k = (h @ f32(w[pre + "k"]).T + f32(w[pre + "k.b"])).view(T, G, D)
    v = (h @ f32(w[pre + "v"]).T + f32(w[pre + "v.b"])).view(T, G, Dv)
    if mx.get("rot"):
        q, k = rotate_interleaved(q, pos, mx["rot"]), rotate_interleaved(k, pos, mx["rot"])
    see = pos[None, :] <= pos[:, None]
    if mx.get("mask"):  # chunks are counted from position 0 of the sequence
        size = int(mx["mask"]["size"])
        see = see & ((pos[None, :] // size) == (pos[:, None] // size))
    sink = f32(w[pre + "sink"])
    out = torch.zeros(T, H, Dv)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(mx["scale"])
        s = s.masked_fill(~see, float("-inf"))
        m = torch.maximum(s.max(-1).values, sink[hd])
        e = torch.exp(s - m[:, None])
        den = e.sum(-1) + torch.exp(sink[hd] - m)
        out[:, hd] = (e @ v[:, g]) / den[:, None]
    return out.reshape(T, H * Dv) @ f32(w[pre + "o"]).T


def causal_conv_silu(x, cw):
    """x [T, C], cw [C, taps]; the last tap multiplies the current token; zeros before the start."""
    T, C = x.shape
    taps = cw.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C), x], 0)
    y = torch.zeros(T, C)
    for j in range(taps):
        y = y + xp[j:j + T] * f32(cw)[:, j]
    return torch.nn.functional.silu(y)


def delta_mixer(h, w, pre, mx, eps):
    """Gated delta rule, one token after the other from a zero state."""
    H, G, D, Dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    T = h.shape[0]
    q = causal_conv_silu(h @ f32(w[pre + "q"]).T, w[pre + "q.conv"]).view(T, G, D)
    k = causal_conv_silu(h @ f32(w[pre + "k"]).T, w[pre + "k.conv"]).view(T, G, D)
    v = causal_conv_silu(h @ f32(w[pre + "v"]).T, w[pre + "v.conv"]).view(T, H, Dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ f32(w[pre + "b"]).T)
    dec = torch.exp(-torch.exp(f32(w[pre + "A_log"])) * torch.nn.functional.softplus(h @ f32(w[pre + "a"]).T + f32(w[pre + "dt_bias"])))
    gate = torch.nn.functional.silu(h @ f32(w[pre + "g"]).T).view(T, H, Dv)
    o = torch.zeros(T, H, Dv)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(D, Dv)
        for t in range(T):
            S = dec[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    o = unit_rms(o, eps) * f32(w[pre + "norm"]) * gate
    return o.reshape(T, H * Dv) @ f32(w[pre + "o"]).T


def mlstm_mixer(h, w, pre, mx, eps):
    """Matrix memory with exponential input gate, logistic forget gate and a running maximum that starts at zero."""
    H, D, Dv, cap = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"]), float(mx["gate_cap"])
    T = h.shape[0]
    q = (h @ f32(w[pre + "q"]).T).view(T, H, D) * D ** -0.5
    k = (h @ f32(w[pre + "k"]).T).view(T, H, D)
    v = (h @ f32(w[pre + "v"]).T).view(T, H, Dv)
    ig = cap * torch.tanh((h @ f32(w[pre + "i"]).T + f32(w[pre + "i.b"])) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ f32(w[pre + "f"]).T + f32(w[pre + "f.b"])) / cap))
    o = torch.zeros(T, H, Dv)
    for hd in range(H):
        S, n, m = torch.zeros(D, Dv), torch.zeros(D), torch.zeros(())
        for t in range(T):
            m_new = torch.maximum(fg[t, hd] + m, ig[t, hd])
            a, b = torch.exp(fg[t, hd] + m - m_new), torch.exp(ig[t, hd] - m_new)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            m = m_new
            o[t, hd] = (S.T @ q[t, hd]) / (torch.maximum((n @ q[t, hd]).abs(), torch.exp(-m)) + 1e-6)
    o = unit_rms(o, eps).reshape(T, H * Dv) * f32(w[pre + "norm"]) * torch.sigmoid(h @ f32(w[pre + "g"]).T)
    return o @ f32(w[pre + "o"]).T


# ---------------------------------------------------------------- feed-forward
def route(h, w, pre, r):
    """(chosen experts [T, top], their weights [T, top]): logistic scores; the choice adds a per-expert correction and is limited to
    the ``keep`` groups whose two best corrected scores sum highest; the weights are the uncorrected scores."""
    E, top = int(r["experts"]), int(r["top"])
    g = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(g["count"]), int(g["keep"])
    s = torch.sigmoid(h @ f32(w[pre + "router"]).T)
    c = s + f32(w[pre + "correction"])
    per = E // count
    gs = c.view(-1, count, per).topk(min(2, per), dim=-1).values.sum(-1)
    kept = gs.topk(keep, dim=-1).indices
    allow = torch.zeros(h.shape[0], count, dtype=torch.bool).scatter_(1, kept, True)
    c = c.masked_fill(~allow.repeat_interleave(per, dim=1), float("-inf"))
    ids = c.topk(top, dim=-1).indices
    return ids, s.gather(1, ids)


def moe(h, w, pre, mlp):
    ids, wt = route(h, w, pre, mlp["router"])
    y = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0])
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            a = torch.nn.functional.silu(h[t] @ f32(w[f"{pre}e{e}.gate"]).T) * (h[t] @ f32(w[f"{pre}e{e}.up"]).T)
            y[t] += wt[t, j] * (a @ f32(w[f"{pre}e{e}.down"]).T)
    return y


# ---------------------------------------------------------------- the model
def forward(cfg, w, tokens, trail=None):
    """Logits [T, vocab] of one sequence from position 0; ``trail`` (a list) receives the residual after every layer."""
    tok = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tok))
    eps = float(cfg["norm"]["eps"])
    x = f32(w["embed"])[tok] * float(cfg["embedding"]["scale"])
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = dyt(x, w, p + "norm1")
        if l["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", l["mixer"], pos)
        elif l["type"] == "delta":
            y = delta_mixer(h, w, p + "mix.", l["mixer"], eps)
        elif l["type"] == "mlstm":
            y = mlstm_mixer(h, w, p + "mix.", l["mixer"], eps)
        else:
            raise ValueError(l["type"])
        if l.get("mlp"):
            y = y + moe(h, w, p + "mlp.", l["mlp"])
        x = x + y
        if trail is not None:
            trail.append(x.clone())
    return dyt(x, w, "final.norm") @ f32(w["head"]).T * float(cfg["logit_scale"])
