"""Mutusun: a decoder-only design with chunk-local sigmoid attention, a short causal convolution in front of every
sublayer, norms before and after each sublayer, and dense or mixture-of-experts feed-forward layers.

Per layer, with N(v; w) = v / sqrt(mean(v^2) + eps) * (1 + w) and C(h) = h + causal depthwise convolution of h over time:

    x <- x + N(mixer(C(N(x; norm1))); norm1b)
    x <- x + N(ff(C(N(x; norm2))); norm2b)            (layers may have no feed-forward)

mixer: q, k, v projections; per-head unit-RMS norm of q and k with a plain weight; score = scale * q.k, soft-capped by
cap * tanh(score / cap); a query sees the keys of its own block of `chunk` positions up to itself; every visible key
weighs sigmoid(score + bias[head]) (no normalisation over keys); output projection.
ff: down(relu(up h)^2), or a softmax router over experts + identity experts that picks the `top` largest
(score + correction) and sums score-weighted expert outputs; an expert is down(g sigmoid(1.702 g) (u + 1)) with
g = min(gate h, limit), u = clamp(up h, +-limit); an identity expert returns h.
Layers may share another layer's weights while keeping their own cache and convolution tails.

Wiring follows the framework's other decoder (`model.QSpecLlamaModel`): a flat token batch with per-token slot and
position, caches held by the model and indexed by slot, a scratch arena allocated once, the residual sum fused into the
norm that opens the next sublayer. What differs: activations / weights are bfloat16 or float32 (no int4 path), the
residual stream is float32, dense matrix products go to the vendor library, and the key/value cache holds only one
chunk per slot (`chunk` rows: keys of earlier chunks can never be seen again).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import ops
from .state import BatchMeta


@dataclass
class MixerSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float          # 0: no soft cap
    chunk: int

    @property
    def ld(self) -> int:    # row length of the fused [q | k | v] projection
        return self.heads * self.dim + self.kv_heads * (self.dim + self.vdim)


@dataclass
class FeedForwardSpec:
    kind: str               # "dense" | "moe"
    ff: int                 # hidden size of the dense layer / of one expert
    experts: int = 0
    identity: int = 0
    top: int = 0
    limit: float = 0.0


@dataclass
class LayerSpec:
    mixer: MixerSpec
    mlp: Optional[FeedForwardSpec]
    weights_of: int         # index of the layer whose tensors this layer uses (its own index if it has tensors)


@dataclass
class MutusunConfig:
    vocab: int
    width: int
    eps: float
    taps: int               # 0: no input convolution
    layers: List[LayerSpec] = field(default_factory=list)
    name: str = "mutusun"

    @staticmethod
    def from_dict(d: dict) -> "MutusunConfig":
        layers = []
        for i, e in enumerate(d["layers"]):
            if e.get("type") != "attention":
                raise ValueError(f"layer {i}: unknown mixer type {e.get('type')!r}")
            m = e["mixer"]
            mixer = MixerSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                              vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
                              chunk=int(m["mask"]["size"]))
            if mixer.heads % mixer.kv_heads:
                raise ValueError(f"layer {i}: {mixer.heads} query heads do not divide over {mixer.kv_heads} key/value heads")
            f = e.get("mlp")
            if f is None:
                mlp = None
            elif f["kind"] == "dense":
                mlp = FeedForwardSpec(kind="dense", ff=int(f["ff"]))
            elif f["kind"] == "moe":
                r = f["router"]
                mlp = FeedForwardSpec(kind="moe", ff=int(f["expert"]["ff"]), experts=int(r["experts"]),
                                      identity=int(r.get("identity") or 0), top=int(r["top"]), limit=float(f["expert"]["limit"]))
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {f['kind']!r}")
            layers.append(LayerSpec(mixer=mixer, mlp=mlp, weights_of=int(e.get("weights_of", i))))
        for i, l in enumerate(layers):                     # a borrowed layer may itself borrow: follow to the owner
            j, hops = l.weights_of, 0
            while layers[j].weights_of != j:
                j, hops = layers[j].weights_of, hops + 1
                if hops > len(layers):
                    raise ValueError(f"layer {i}: weights_of forms a cycle")
            l.weights_of = j
        canon = d.get("canon") or {}
        return MutusunConfig(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                             taps=int(canon.get("taps") or 0), layers=layers)

    def to_dict(self) -> dict:
        out = {"architecture": "Mutusun", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "canon": {"taps": self.taps}, "layers": []}
        for i, l in enumerate(self.layers):
            m = l.mixer
            e = {"type": "attention",
                 "mixer": {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                           "softcap": m.softcap, "mask": {"size": m.chunk}}}
            f = l.mlp
            if f is None:
                e["mlp"] = None
            elif f.kind == "dense":
                e["mlp"] = {"kind": "dense", "ff": f.ff}
            else:
                e["mlp"] = {"kind": "moe", "expert": {"ff": f.ff, "limit": f.limit},
                            "router": {"experts": f.experts, "identity": f.identity, "top": f.top}}
            if l.weights_of != i:
                e["weights_of"] = l.weights_of
            out["layers"].append(e)
        return out

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Name -> shape of every tensor of a checkpoint of this configuration."""
        W, out = self.width, {"embed": (self.vocab, self.width)}
        for i, l in enumerate(self.layers):
            if l.weights_of != i:
                continue
            m, f, p = l.mixer, l.mlp, f"l{i}."
            out.update({p + "norm1": (W,), p + "norm1b": (W,), p + "mix.q": (m.heads * m.dim, W), p + "mix.k": (m.kv_heads * m.dim, W),
                        p + "mix.v": (m.kv_heads * m.vdim, W), p + "mix.q.norm": (m.dim,), p + "mix.k.norm": (m.dim,),
                        p + "mix.pb": (m.heads,), p + "mix.o": (W, m.heads * m.vdim)})
            if self.taps:
                out[p + "canon1"] = (W, self.taps)
            if f is None:
                continue
            out.update({p + "norm2": (W,), p + "norm2b": (W,)})
            if self.taps:
                out[p + "canon2"] = (W, self.taps)
            if f.kind == "dense":
                out.update({p + "mlp.up": (f.ff, W), p + "mlp.down": (W, f.ff)})
            else:
                for e in range(f.experts):
                    out.update({p + f"mlp.e{e}.gate": (f.ff, W), p + f"mlp.e{e}.up": (f.ff, W), p + f"mlp.e{e}.down": (W, f.ff)})
                out.update({p + "mlp.router": (f.experts + f.identity, W), p + "mlp.correction": (f.experts + f.identity,)})
        out.update({"final.norm": (W,), "head": (self.vocab, W)})
        return out


def random_weights(cfg: MutusunConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bfloat16 tensors of a configuration (CPU): matrices ~ N(0, 1/fan_in), vectors small."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.tensor_shapes().items():
        if len(shape) == 2 and not name.endswith(("canon1", "canon2")):
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif name.endswith(("q.norm", "k.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            t = 0.2 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


class _LayerWeights:
    """Device tensors of one layer that owns tensors: large matrices in the activation type, the rest float32."""

    def __init__(self, cfg: MutusunConfig, i: int, sd: Dict[str, torch.Tensor], dtype, device):
        spec, p = cfg.layers[i], f"l{i}."

        def big(*names):
            t = torch.cat([sd[p + n] for n in names], 0) if len(names) > 1 else sd[p + names[0]]
            return t.to(device=device, dtype=dtype).contiguous()

        def small(name):
            return sd[p + name].to(device=device, dtype=torch.float32).contiguous()

        self.norm1, self.norm1b = small("norm1"), small("norm1b")
        self.canon1 = small("canon1") if cfg.taps else None
        self.qkv = big("mix.q", "mix.k", "mix.v")                    # rows [q ; k ; v]
        self.q_norm, self.k_norm, self.pb = small("mix.q.norm"), small("mix.k.norm"), small("mix.pb")
        self.o = big("mix.o")
        f = spec.mlp
        if f is None:
            return
        self.norm2, self.norm2b = small("norm2"), small("norm2b")
        self.canon2 = small("canon2") if cfg.taps else None
        if f.kind == "dense":
            self.up, self.down = big("mlp.up"), big("mlp.down")
        else:
            self.router, self.correction = small("mlp.router"), small("mlp.correction")
            if f.experts:
                self.gate_up = torch.stack([torch.cat((sd[p + f"mlp.e{e}.gate"], sd[p + f"mlp.e{e}.up"]), 0)
                                            for e in range(f.experts)]).to(device=device, dtype=dtype).contiguous()
                self.edown = torch.stack([sd[p + f"mlp.e{e}.down"] for e in range(f.experts)]).to(device=device, dtype=dtype).contiguous()
            else:
                self.gate_up = self.edown = None


class MutusunModel(torch.nn.Module):
    """Weights, per-slot state and the forward pass over a flat token batch (`state.BatchMeta`).

    dtype: torch.bfloat16 (serving: bfloat16 matrix products with float32 accumulation) or torch.float32 (everything in
    true float32). n_slots sequences can be live at once; a step carries at most max_step_tokens tokens."""

    architecture = "Mutusun"

    def __init__(self, cfg: MutusunConfig, weights: Dict[str, torch.Tensor], dtype=torch.bfloat16, device="cuda",
                 n_slots: int = 8, max_step_tokens: int = 2048):
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("MutusunModel: dtype must be torch.bfloat16 or torch.float32")
        shapes = cfg.tensor_shapes()
        for name, shape in shapes.items():
            if name not in weights:
                raise KeyError(f"tensor {name} is missing from the checkpoint")
            if tuple(weights[name].shape) != tuple(shape):
                raise ValueError(f"tensor {name}: shape {tuple(weights[name].shape)}, the configuration says {tuple(shape)}")
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.n_slots, self.max_step_tokens = n_slots, max_step_tokens
        # true float32 products in float32 mode; no reduced-precision accumulation of bfloat16 products
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        dev, W, T = self.device, cfg.width, max_step_tokens
        self.embed = weights["embed"].to(device=dev, dtype=dtype).contiguous()
        self.head = weights["head"].to(device=dev, dtype=dtype).contiguous()
        self.final_norm = weights["final.norm"].to(device=dev, dtype=torch.float32).contiguous()
        self.weights = {i: _LayerWeights(cfg, i, weights, dtype, dev) for i, l in enumerate(cfg.layers) if l.weights_of == i}
        # per-slot state, one set per layer RUN (a layer that borrows weights still has its own)
        hist = max(cfg.taps - 1, 0)
        self.cache_k, self.cache_v, self.tail1, self.tail2 = [], [], [], []
        for l in cfg.layers:
            m = l.mixer
            self.cache_k.append(torch.zeros(n_slots, m.chunk, m.kv_heads, m.dim, dtype=dtype, device=dev))
            self.cache_v.append(torch.zeros(n_slots, m.chunk, m.kv_heads, m.vdim, dtype=dtype, device=dev))
            self.tail1.append(torch.zeros(2, n_slots, hist, W, dtype=torch.float32, device=dev) if hist else None)
            self.tail2.append(torch.zeros(2, n_slots, hist, W, dtype=torch.float32, device=dev) if hist and l.mlp else None)
        # scratch arena, allocated once
        f32 = dict(dtype=torch.float32, device=dev)
        act = dict(dtype=dtype, device=dev)
        mx = lambda vals: max(list(vals) + [1])
        self.buf_x = [torch.empty(T * W, **f32), torch.empty(T * W, **f32)]          # residual stream, ping-pong
        self.buf_h = torch.empty(T * W, **act)
        self.buf_n = torch.empty(T * W, **f32)                                        # normalised rows of long prompts (seq_norm_conv)
        self.buf_qkv = torch.empty(T * mx(l.mixer.ld for l in cfg.layers), **act)
        self.buf_att = torch.empty(T * mx(l.mixer.heads * l.mixer.vdim for l in cfg.layers), **act)
        self.buf_y = [torch.empty(T * W, **act), torch.empty(T * W, **act)]          # mixer / feed-forward outputs
        self.buf_up = torch.empty(T * mx(l.mlp.ff for l in cfg.layers if l.mlp and l.mlp.kind == "dense"), **act)
        tops = mx(l.mlp.top for l in cfg.layers if l.mlp and l.mlp.kind == "moe")
        has_moe = any(l.mlp and l.mlp.kind == "moe" for l in cfg.layers)
        self.buf_idx = torch.empty(T * tops, dtype=torch.int32, device=dev)
        self.buf_rw = torch.empty(T * tops, **f32)
        self.buf_pair = torch.empty(T * tops * W if has_moe else 1, **act)
        self.buf_ids = torch.empty(T, dtype=torch.int32, device=dev)
        # Prompt-shaped batches take the tensor-core tile kernels (bfloat16); QSPEC_SEQ_TILES=0 keeps the token-per-CTA forms.
        self.use_tiles = dtype == torch.bfloat16 and os.environ.get("QSPEC_SEQ_TILES", "1") != "0"
        self.tiles_min_tokens = 64           # a step with fewer tokens, or fewer than 16 per sequence, is decode-shaped

    # ------------------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, path: str, dtype=torch.bfloat16, device="cuda", **kw) -> "MutusunModel":
        from .checkpoint import read_safetensors_file
        with open(os.path.join(path, "config.json")) as f:
            cfg = MutusunConfig.from_dict(json.load(f))
        return cls(cfg, read_safetensors_file(os.path.join(path, "model.safetensors")), dtype=dtype, device=device, **kw)

    @property
    def vocab_size(self) -> int:
        return self.cfg.vocab

    def state_bytes_per_slot(self) -> int:
        n = 0
        for t in self.cache_k + self.cache_v + self.tail1 + self.tail2:
            if t is not None:
                n += t.numel() * t.element_size() // self.n_slots
        return n

    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_batch(self, input_ids: torch.Tensor, meta: BatchMeta, trace: Optional[list] = None) -> torch.Tensor:
        """input_ids: int32 [ntok] on the device. Returns the final-norm hidden state [ntok, W] (activation type), a view of
        the arena. `trace`, if a list, receives a copy of the residual stream after every layer (debugging)."""
        cfg, T, W = self.cfg, meta.ntok, self.cfg.width
        if T > self.max_step_tokens or input_ids.numel() != T:
            raise ValueError(f"forward_batch: {T} tokens (at most {self.max_step_tokens})")
        tab, eps = meta.table, cfg.eps
        xa, xb = self.buf_x[0][:T * W].view(T, W), self.buf_x[1][:T * W].view(T, W)
        h = self.buf_h[:T * W].view(T, W)
        ya, yb = self.buf_y[0][:T * W].view(T, W), self.buf_y[1][:T * W].view(T, W)
        ops.seq_embed(self.embed, input_ids, xa)
        prompt_shaped = self.use_tiles and T >= self.tiles_min_tokens and T >= 16 * len(meta.segments)
        max_keys = meta.max_length
        pend = None                                    # (y, part weights, post-norm weight) of the sublayer still to be added

        def enter(pre_w, conv_w, tail, out):
            nonlocal xa, xb, pend
            if pend is None:
                ops.seq_norm_conv(xa, tab, eps, out=out, pre_w=pre_w, conv_w=conv_w, tail=tail, scratch=self.buf_n)
            else:
                ops.seq_norm_conv(xa, tab, eps, out=out, pre_w=pre_w, conv_w=conv_w, tail=tail, y=pend[0], y_w=pend[1],
                                  post_w=pend[2], x_out=xb, scratch=self.buf_n)
                xa, xb = xb, xa
                pend = None

        for i, spec in enumerate(cfg.layers):
            p, m, f = self.weights[spec.weights_of], spec.mixer, spec.mlp
            enter(p.norm1, p.canon1, self.tail1[i], h)
            qkv = self.buf_qkv[:T * m.ld].view(T, m.ld)
            att = self.buf_att[:T * m.heads * m.vdim].view(T, m.heads * m.vdim)
            torch.matmul(h, p.qkv.t(), out=qkv)
            ops.seq_qk_norm(qkv, p.q_norm, p.k_norm, m.heads, m.kv_heads, m.dim, eps)
            ops.seq_chunk_attention(qkv, self.cache_k[i], self.cache_v[i], p.pb, att, tab, m.heads, m.kv_heads, m.dim, m.vdim,
                                    m.chunk, m.scale, m.softcap, max_keys=max_keys,
                                    tiles=prompt_shaped and ops.seq_chunk_attention_tiles_supported(qkv, m.heads, m.kv_heads, m.dim, m.vdim))
            ops.seq_cache_append(qkv, self.cache_k[i], self.cache_v[i], tab, m.heads, m.kv_heads, m.dim, m.vdim, m.chunk)
            torch.matmul(att, p.o.t(), out=ya)
            pend = (ya, None, p.norm1b)
            if f is not None:
                enter(p.norm2, p.canon2, self.tail2[i], h)
                if f.kind == "dense":
                    up = self.buf_up[:T * f.ff].view(T, f.ff)
                    torch.matmul(h, p.up.t(), out=up)
                    ops.seq_relu2(up)
                    torch.matmul(up, p.down.t(), out=yb)
                    pend = (yb, None, p.norm2b)
                else:
                    idx = self.buf_idx[:T * f.top].view(T, f.top)
                    rw = self.buf_rw[:T * f.top].view(T, f.top)
                    pair = self.buf_pair[:T * f.top * W].view(T, f.top, W)
                    ops.moe_route(h, p.router, p.correction, idx, rw)
                    # grouped tiles once an expert sees several rows on average (its weights are then read once per tile,
                    # not once per row); a handful of tokens stay with the row-per-CTA form
                    if self.use_tiles and T * f.top >= 4 * max(f.experts, 1) and ops.moe_expert_grouped_supported(h, f.ff):
                        ops.moe_expert_grouped(h, p.gate_up, p.edown, idx, pair, f.experts, f.ff, f.limit)
                    else:
                        ops.moe_expert_tokens(h, p.gate_up, p.edown, idx, pair, f.experts, f.ff, f.limit)
                    pend = (pair, rw, p.norm2b)
            if trace is not None:
                enter(None, None, None, None)          # residual sum only
                trace.append(xa.clone())
        enter(self.final_norm, None, None, h)
        return h

    @torch.no_grad()
    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [n, vocab] of final-norm hidden rows [n, W]."""
        if self.dtype == torch.float32:
            return torch.matmul(hidden_rows, self.head.t())
        return torch.mm(hidden_rows, self.head.t(), out_dtype=torch.float32)
