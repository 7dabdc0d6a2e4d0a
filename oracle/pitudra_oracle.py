"""Plain implementation of the Pitudra design: float64, one function per mechanism, whole sequences, no cache.

The tests compare the framework's kernels and model (`qspec_b200.pitudra`) with these functions; nothing here is
shared with the product path. A sequence is a list of token ids; every function takes the whole sequence [T, ...] and
loops over time where the mechanism is recurrent.

Layer (x is the residual stream, [T, width]):
    h   = token_shift(x)                        h_t + (h_(t-1) - h_t) * shift, h_(-1) = 0
    x  <- x + layer_norm(mixer(h))
    x  <- x + layer_norm(moe(x))                (if the layer has a feed-forward)
    x  <- x + rms(side_proj(gelu(side_gate x) * side_embed[token, layer part])) * side_norm     (if the model has one)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def _w(sd, name):
    return sd[name].to(F64)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(h, shift):
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * shift


def rotate(v, pos, base, dims):
    """v [T, n, d]: the first `dims` entries of the last axis are rotated, entry i paired with i + dims/2."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    a = pos.to(F64)[:, None] * f[None, :]                       # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, w = v[..., :half], v[..., half:dims]
    return torch.cat([u * c - w * s, w * c + u * s, v[..., dims:]], -1)


def windowed_sink_softmax(scores, sink, window):
    """scores [H, T, T] (already scaled), sink [H]: weights over keys i - window < j <= i; the denominator also has exp(sink)."""
    T = scores.shape[-1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = (j <= i) & (i - j < window)
    s = scores.masked_fill(~vis, float("-inf"))
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def latent_kv(h, sd, p, m, eps):
    """The cached part of a latent-attention layer: latent c [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    r, R = m["kv_rank"], m["rot_dim"]
    d = h @ _w(sd, p + "dkv").T
    c = rms_norm(d[:, :r], _w(sd, p + "dkv.norm"), eps)
    kr = rotate(d[:, None, r:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])[:, 0]
    return c, kr


def latent_attention(h, sd, p, m, eps, kv):
    T = h.shape[0]
    H, D, R, DV = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kv
    cq = rms_norm(h @ _w(sd, p + "dq").T, _w(sd, p + "dq.norm"), eps)
    q = (cq @ _w(sd, p + "uq").T).view(T, H, D + R)
    qn = q[..., :D]
    qr = rotate(q[..., D:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    k = (c @ _w(sd, p + "uk").T).view(T, H, D)
    v = (c @ _w(sd, p + "uv").T).view(T, H, DV)
    s = (torch.einsum("ihd,jhd->hij", qn, k) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    w = windowed_sink_softmax(s, _w(sd, p + "sink"), m["mask"]["size"])
    o = torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * DV)
    return o @ _w(sd, p + "o").T


def gated_attention(h, sd, p, m, eps):
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ _w(sd, p + "q").T + _w(sd, p + "q.b"), _w(sd, p + "q.norm"), eps).view(T, H, D)
    k = rms_norm(h @ _w(sd, p + "k").T + _w(sd, p + "k.b"), _w(sd, p + "k.norm"), eps).view(T, G, D)
    v = (h @ _w(sd, p + "v").T + _w(sd, p + "v.b")).view(T, G, DV)
    rep = H // G
    k = k.repeat_interleave(rep, 1)
    v = v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    w = windowed_sink_softmax(s, _w(sd, p + "sink"), m["mask"]["size"])
    o = torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * DV)
    o = o * torch.sigmoid(h @ _w(sd, p + "g").T)
    return o @ _w(sd, p + "o").T


def hgrn2(h, sd, p, m, eps):
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    q = torch.nn.functional.silu(h @ _w(sd, p + "q").T).view(T, H, D)
    v = (h @ _w(sd, p + "v").T).view(T, H, DV)
    low = _w(sd, p + "lower")
    f = (low + (1.0 - low) * torch.sigmoid(h @ _w(sd, p + "f").T + _w(sd, p + "f.b"))).view(T, H, D)
    S = torch.zeros(H, D, DV, dtype=F64)
    out = []
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    o = rms_norm(torch.stack(out), _w(sd, p + "norm"), eps).reshape(T, H * DV)
    return o @ _w(sd, p + "o").T


def moe(x, sd, p, f):
    E, top = f["router"]["experts"], f["router"]["top"]
    z = x @ _w(sd, p + "router").T
    val, idx = torch.topk(z, top, dim=-1)
    w = torch.softmax(val, -1)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for k in range(top):
            e = int(idx[t, k])
            a = torch.relu(x[t] @ _w(sd, p + f"e{e}.up").T) ** 2
            out[t] += w[t, k] * (a @ _w(sd, p + f"e{e}.down").T)
    return out


def token_side(x, tokens, sd, p, i, dim, eps):
    e = _w(sd, "side.embed")[tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ _w(sd, p + "side.gate").T) * e
    y = g @ _w(sd, p + "side.proj").T
    return rms_norm(y, _w(sd, p + "side.norm"), eps)


def forward(cfg: dict, sd: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence; `layers_out` receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = _w(sd, "embed")[tok]
    side_dim = (cfg.get("token_side") or {}).get("dim")
    latents = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = token_shift(x, _w(sd, p + "shift"))
        if L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_kv(h, sd, p + "mix.", m, eps)
                src = i
            y = latent_attention(h, sd, p + "mix.", m, eps, latents[src])
        elif L["type"] == "attention":
            y = gated_attention(h, sd, p + "mix.", m, eps)
        elif L["type"] == "hgrn2":
            y = hgrn2(h, sd, p + "mix.", m, eps)
        else:
            raise ValueError(L["type"])
        x = x + layer_norm(y, _w(sd, p + "norm1"), _w(sd, p + "norm1.b"), eps)
        if L.get("mlp") is not None:
            x = x + layer_norm(moe(x, sd, p + "mlp.", L["mlp"]), _w(sd, p + "norm2"), _w(sd, p + "norm2.b"), eps)
        if side_dim:
            x = x + token_side(x, tok, sd, p, i, side_dim, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, _w(sd, "final.norm"), _w(sd, "final.norm.b"), eps)
    return x @ _w(sd, "head").T
