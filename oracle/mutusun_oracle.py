"""Plain, slow restatement of the Mutusun decoder design in float64/float32 torch on the CPU: one function per
mechanism, whole sequences only (no cache, no batching), sharing no code with the product path. Tests compare
the framework's kernels, cache and scheduler against these functions.

Notation: x [T, W] residual stream of one sequence, positions 0..T-1; weights are [out, in] and applied as W x.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_zero_centred(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Layer norm of the design: unit RMS, times (1 + w) -- the stored weight is centred on zero."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-head query / key norm: unit RMS times w (no one-plus)."""
    return rms_unit(x, eps) * w


def short_conv_residual(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h + conv(h): causal depthwise convolution over time, w [W, taps]; tap `taps-1` multiplies the current
    row, tap j the row `taps-1-j` steps back; rows before the sequence start are zero."""
    T, W = h.shape
    taps = w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def chunk_visible(i: int, j: int, size: int) -> bool:
    """Query position i sees key position j: causal and in the same block of `size` positions counted from 0."""
    return j <= i and (i // size) == (j // size)


def sigmoid_chunk_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """The 'attention' mixer. p: q, k, v, o, q.norm, k.norm, pb. m: heads, kv_heads, dim, vdim, scale, softcap,
    mask.size. No rotation, no softmax: a visible key weighs sigmoid(capped score + per-head bias)."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = m["mask"]["size"]
    cap = m.get("softcap")
    q = (h @ p["q"].T).view(T, H, D)
    k = (h @ p["k"].T).view(T, G, D)
    v = (h @ p["v"].T).view(T, G, DV)
    q = norm_plain(q, p["q.norm"], eps)
    k = norm_plain(k, p["k.norm"], eps)
    out = torch.zeros(T, H, DV, dtype=h.dtype)
    rep = H // G
    for hd in range(H):
        g = hd // rep
        for i in range(T):
            lo = (i // size) * size
            s = (k[lo:i + 1, g] @ q[i, hd]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            wgt = torch.sigmoid(s + p["pb"][hd])
            out[i, hd] = wgt @ v[lo:i + 1, g]
    return out.reshape(T, H * DV) @ p["o"].T


def dense_ff(h: torch.Tensor, p: Dict[str, torch.Tensor]) -> torch.Tensor:
    """down(relu(up h)^2)."""
    a = torch.relu(h @ p["up"].T)
    return (a * a) @ p["down"].T


def expert_ff(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    """One expert: g = min(gate h, limit), u = clamp(up h, +-limit), y = g sigmoid(1.702 g) (u + 1), down y."""
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int):
    """Scores = softmax over ALL router outputs; the `top` largest (score + correction) are chosen; their weights
    are the plain scores, not renormalised. Returns (indices [T, top], weights [T, top])."""
    s = torch.softmax(h @ router.T, dim=-1)
    idx = torch.topk(s + correction, top, dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def moe_ff(h: torch.Tensor, p: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    """Weighted sum of the chosen experts; the last `identity` router outputs stand for experts that return h."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, wgt = route(h, p["router"], p["correction"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t].tolist(), wgt[t]):
            if e >= E:
                out[t] += w * h[t]
            else:
                out[t] += w * expert_ff(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"],
                                        mlp["expert"]["limit"])[0]
    return out


def layer_tensors(weights: Dict[str, torch.Tensor], cfg: dict, i: int) -> Dict[str, torch.Tensor]:
    """Tensors of layer i with the 'l<j>.' prefix removed; a layer with weights_of = j reads layer j's."""
    j = cfg["layers"][i].get("weights_of", i)
    pre = f"l{j}."
    return {k[len(pre):]: v for k, v in weights.items() if k.startswith(pre)}


def sub(p: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in p.items() if k.startswith(prefix)}


def layer_forward(x: torch.Tensor, p: Dict[str, torch.Tensor], entry: dict, eps: float) -> torch.Tensor:
    """x + post-norm(mixer(conv'd pre-norm(x))), then the same around the feed-forward (if the layer has one)."""
    if entry["type"] != "attention":
        raise ValueError(f"unknown mixer {entry['type']}")
    h = short_conv_residual(norm_zero_centred(x, p["norm1"], eps), p["canon1"])
    x = x + norm_zero_centred(sigmoid_chunk_attention(h, sub(p, "mix."), entry["mixer"], eps), p["norm1b"], eps)
    mlp = entry.get("mlp")
    if mlp is None:
        return x
    h = short_conv_residual(norm_zero_centred(x, p["norm2"], eps), p["canon2"])
    y = dense_ff(h, sub(p, "mlp.")) if mlp["kind"] == "dense" else moe_ff(h, sub(p, "mlp."), mlp)
    return x + norm_zero_centred(y, p["norm2b"], eps)


def forward(weights: Dict[str, torch.Tensor], cfg: dict, tokens, dtype=torch.float64, trace: Optional[list] = None):
    """Logits [T, vocab] of one whole sequence. `trace`, if a list, receives the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, entry in enumerate(cfg["layers"]):
        x = layer_forward(x, layer_tensors(w, cfg, i), entry, eps)
        if trace is not None:
            trace.append(x.clone())
    return norm_zero_centred(x, w["final.norm"], eps) @ w["head"].T
