"""Plain, slow restatement of the Tafopel decoder: one function per mechanism, whole sequences, no cache,
no batching.  It shares no code with the product path; the tests compare the engine against it.

Notation (all per sequence, L tokens, positions 0..L-1):
    layer:   h = LN(x) * w,  x <- x + mixer(h) + ff(h)          (one norm, both branches read h)
    LN:      (x - mean) / sqrt(var + eps) * w, var = mean of squared deviations, no bias
    rms(v):  v / sqrt(mean(v^2) + eps)

A "config" here is the parsed config.json dict; "W" a dict name -> tensor (float).
"""
from __future__ import annotations

import math

import torch


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_tables(rot, length, dtype=torch.float64):
    """cos, sin [length, dims/2] with the YaRN-corrected frequencies; both carry the magnitude factor."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def corr(t):
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(corr(float(sc["fast"]))), 0)
        hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(length, dtype=torch.float64)[:, None] * f[None, :]
    return (ang.cos() * mag).to(dtype), (ang.sin() * mag).to(dtype)


def rotate_interleaved(v, cos, sin):
    """v [L, ..., dims]: pairs (2i, 2i+1) turned by the angle of their position."""
    a, b = v[..., 0::2], v[..., 1::2]
    while cos.dim() < a.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    out = torch.empty_like(v)
    out[..., 0::2] = a * cos - b * sin
    out[..., 1::2] = b * cos + a * sin
    return out


def latent_kv(h, W, pre, m, eps):
    """The cached part of a latent-attention layer: (c [L, kv_rank], rotated shared key [L, rot_dim])."""
    L = h.shape[0]
    r, rd = m["kv_rank"], m["rot_dim"]
    dkv = h @ W[pre + "dkv"].T
    c = rms_norm(dkv[:, :r], W[pre + "dkv.norm"], eps)
    cos, sin = rotary_tables(m["rot"], L, h.dtype)
    kr = rotate_interleaved(dkv[:, r:r + rd], cos, sin)
    return c, kr


def latent_attention(h, W, pre, m, eps, kv):
    """kv = (c, kr) of this layer or of the layer it borrows from."""
    L = h.shape[0]
    H, d, rd, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = kv
    cq = rms_norm(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps)
    q = (cq @ W[pre + "uq"].T).view(L, H, d + rd)
    cos, sin = rotary_tables(m["rot"], L, h.dtype)
    qn, qr = q[..., :d], rotate_interleaved(q[..., d:], cos, sin)
    kn = (c @ W[pre + "uk"].T).view(L, H, d)
    v = (c @ W[pre + "uv"].T).view(L, H, vd)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    mask = torch.ones(L, L, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    sink = W[pre + "sink"].view(H, 1, 1)
    top = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - top)
    p = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(L, H * vd)
    return o @ W[pre + "o"].T


def mamba1(h, W, pre, m):
    L = h.shape[0]
    inner, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    xz = h @ W[pre + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    wc, bc = W[pre + "conv"], W[pre + "conv.b"]
    xp = torch.cat([torch.zeros(taps - 1, inner, dtype=h.dtype), x], 0)
    u = torch.stack([(xp[t:t + taps].T * wc).sum(-1) for t in range(L)]) + bc
    u = u * torch.sigmoid(u)
    dbc = u @ W[pre + "x"].T
    dt = torch.nn.functional.softplus(dbc[:, :R] @ W[pre + "dt"].T + W[pre + "dt.b"])
    B, C = dbc[:, R:R + N], dbc[:, R + N:R + 2 * N]
    A = -torch.exp(W[pre + "A_log"])
    S = torch.zeros(inner, N, dtype=h.dtype)
    ys = []
    for t in range(L):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        ys.append(S @ C[t] + W[pre + "D"] * u[t])
    y = torch.stack(ys) * (z * torch.sigmoid(z))
    return y @ W[pre + "o"].T


def dense_ff(h, W, pre):
    return (gelu_tanh(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def relu2_expert(x, up, down):
    return (torch.relu(x @ up.T) ** 2) @ down.T


def moe_ff(h, W, pre, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.sigmoid(h @ W[pre + "router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        best = torch.topk(s[t], top).indices
        for e in best.tolist():
            out[t] += relu2_expert(s[t, e] * h[t], W[f"{pre}e{e}.up"], W[f"{pre}e{e}.down"])
    if mlp.get("shared"):
        g = torch.sigmoid(h @ W[pre + "shared.sg"].T)
        out = out + g * relu2_expert(h, W[pre + "shared.up"], W[pre + "shared.down"])
    return out


def forward(cfg, W, tokens, dtype=torch.float64, return_layers=False):
    """logits [L, vocab] for one sequence (and the residual stream after every layer)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kvs, trace = {}, []
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, W[pre + "norm1"], eps)
        if layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kvs[i] = latent_kv(h, W, pre + "mix.", m, eps)
            mix = latent_attention(h, W, pre + "mix.", m, eps, kvs[m["kv_from"] if m.get("kv_from") is not None else i])
        elif layer["type"] == "mamba1":
            mix = mamba1(h, W, pre + "mix.", m)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        ff = 0.0
        if mlp is not None:
            ff = dense_ff(h, W, pre + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, W, pre + "mlp.", mlp)
        x = x + (mix + ff)
        trace.append(x.clone())
    logits = layer_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, torch.stack(trace)) if return_layers else logits
