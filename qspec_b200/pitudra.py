"""Pitudra: a decoder-only design that mixes three kinds of sequence mixers under one residual stream.

Per layer, with x the float32 residual stream and LN the layer norm with weight and bias:

    h  = x_t + (x_(t-1) - x_t) * shift                      token shift on the mixer's input (x_(-1) = 0)
    x <- x + LN(mixer(h); norm1)                            the norm sits on the sublayer's OUTPUT
    x <- x + LN(moe(x); norm2)                              squared-ReLU experts; softmax over the chosen logits only
    x <- x + rms(P (gelu_tanh(G x) * side_embed[token, layer slice])) * side_norm        per-layer token input

mixers (`layers[i].type`):
    latent_attention  queries through a normed low-rank latent; keys / values from a normed low-rank latent c plus one
                      rotary key part shared by the heads; only [c | rotated part] is cached. Run in the absorbed form:
                      score = (W_uk^T q_nope) . c + q_rot . k_rot, output = W_uv (sum_j w_j c_j). A layer with `kv_from`
                      reads another layer's cache with its own up-projections.
    attention         grouped-query attention with biases, a unit-RMS norm over the WHOLE query / key projection, no
                      positions, and a sigmoid output gate.
    hgrn2             gated linear recurrence S <- diag(f) S + (1 - f) v^T, o = S^T q, lower-bounded forget gate, per-head
                      output norm; the state is float32 per slot.
Both attentions see a sliding window (i - j < mask.size) and their softmax denominator carries a per-head sink.

Wiring follows `mutusun.MutusunModel`: a flat token batch with per-token slot and position (`state.BatchMeta`), state
held by the model and indexed by slot, a scratch arena allocated once, dense products in the vendor library, everything
else in the sequence-mixer kernel library (`ops.seq_*`, `ops.moe_*`). Per-slot state: the previous row of every layer
(token shift, double-buffered by the step's phase), ring caches of `window - 1 + max_step_tokens` rows (a step writes its
own rows before any of them is read, and a row is only ever read at a position its current owner wrote), and the
recurrence state. Nothing is cleared when a slot is released: validity follows from positions alone.
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
class PitudraMixer:
    kind: str                       # "latent_attention" | "attention" | "hgrn2"
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0               # attention
    scale: float = 1.0              # both attentions
    window: int = 0                 # both attentions
    q_rank: int = 0                 # latent attention ...
    kv_rank: int = 0
    rot_dim: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    kv_from: Optional[int] = None


@dataclass
class PitudraMoE:
    experts: int
    top: int
    ff: int


@dataclass
class PitudraLayer:
    mixer: PitudraMixer
    mlp: Optional[PitudraMoE]


@dataclass
class PitudraConfig:
    vocab: int
    width: int
    eps: float
    side_dim: int                   # 0: no per-layer token input
    layers: List[PitudraLayer] = field(default_factory=list)
    name: str = "pitudra"

    @staticmethod
    def from_dict(d: dict) -> "PitudraConfig":
        layers = []
        for i, e in enumerate(d["layers"]):
            kind, m = e.get("type"), e["mixer"]
            if kind == "latent_attention":
                rot = m.get("rot") or {}
                mixer = PitudraMixer(kind=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                                     scale=float(m["scale"]), window=int(m["mask"]["size"]), q_rank=int(m["q_rank"]),
                                     kv_rank=int(m["kv_rank"]), rot_dim=int(m["rot_dim"]), rot_dims=int(rot.get("dims", m["rot_dim"])),
                                     rot_base=float(rot.get("base", 10000.0)),
                                     kv_from=None if m.get("kv_from") is None else int(m["kv_from"]))
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ValueError(f"layer {i}: {mixer.rot_dims} rotated dimensions of {mixer.rot_dim}")
            elif kind == "attention":
                mixer = PitudraMixer(kind=kind, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                     vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), window=int(m["mask"]["size"]))
                if mixer.heads % mixer.kv_heads:
                    raise ValueError(f"layer {i}: {mixer.heads} query heads do not divide over {mixer.kv_heads} key/value heads")
            elif kind == "hgrn2":
                mixer = PitudraMixer(kind=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            f = e.get("mlp")
            if f is None:
                mlp = None
            elif f.get("kind") == "moe":
                mlp = PitudraMoE(experts=int(f["router"]["experts"]), top=int(f["router"]["top"]), ff=int(f["expert"]["ff"]))
                if not 1 <= mlp.top <= mlp.experts:
                    raise ValueError(f"layer {i}: top {mlp.top} of {mlp.experts} experts")
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
            layers.append(PitudraLayer(mixer=mixer, mlp=mlp))
        for i, l in enumerate(layers):
            m = l.mixer
            if m.kv_from is None:
                continue
            if not 0 <= m.kv_from < len(layers):
                raise ValueError(f"layer {i}: kv_from {m.kv_from} is not a layer")
            s = layers[m.kv_from].mixer
            if m.kv_from >= i or s.kind != "latent_attention" or s.kv_from is not None:
                raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer with a cache of its own")
            if (s.kv_rank, s.rot_dim, s.rot_dims, s.rot_base) != (m.kv_rank, m.rot_dim, m.rot_dims, m.rot_base):
                raise ValueError(f"layer {i}: latent sizes and rotation differ from layer {m.kv_from}'s")
        side = d.get("token_side") or {}
        return PitudraConfig(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                             side_dim=int(side.get("dim") or 0), layers=layers)

    def to_dict(self) -> dict:
        out = {"architecture": "Pitudra", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps}, "layers": []}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        for l in self.layers:
            m = l.mixer
            if m.kind == "latent_attention":
                mx = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "rot_dim": m.rot_dim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                      "scale": m.scale, "mask": {"size": m.window}, "rot": {"base": m.rot_base, "dims": m.rot_dims}}
                if m.kv_from is not None:
                    mx["kv_from"] = m.kv_from
            elif m.kind == "attention":
                mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "mask": {"size": m.window}}
            else:
                mx = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim}
            f = l.mlp
            out["layers"].append({"type": m.kind, "mixer": mx,
                                  "mlp": None if f is None else {"kind": "moe", "expert": {"ff": f.ff},
                                                                 "router": {"experts": f.experts, "top": f.top}}})
        return out

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Name -> shape of every tensor a checkpoint of this configuration must hold."""
        W = self.width
        out = {"embed": (self.vocab, W)}
        if self.side_dim:
            out["side.embed"] = (self.vocab, len(self.layers) * self.side_dim)
        for i, l in enumerate(self.layers):
            m, f, p = l.mixer, l.mlp, f"l{i}."
            out.update({p + "shift": (W,), p + "norm1": (W,), p + "norm1.b": (W,)})
            x = p + "mix."
            if m.kind == "latent_attention":
                out.update({x + "dq": (m.q_rank, W), x + "dq.norm": (m.q_rank,), x + "uq": (m.heads * (m.dim + m.rot_dim), m.q_rank),
                            x + "uk": (m.heads * m.dim, m.kv_rank), x + "uv": (m.heads * m.vdim, m.kv_rank), x + "sink": (m.heads,),
                            x + "o": (W, m.heads * m.vdim)})
                if m.kv_from is None:
                    out.update({x + "dkv": (m.kv_rank + m.rot_dim, W), x + "dkv.norm": (m.kv_rank,)})
            elif m.kind == "attention":
                out.update({x + "q": (m.heads * m.dim, W), x + "q.b": (m.heads * m.dim,), x + "k": (m.kv_heads * m.dim, W),
                            x + "k.b": (m.kv_heads * m.dim,), x + "v": (m.kv_heads * m.vdim, W), x + "v.b": (m.kv_heads * m.vdim,),
                            x + "q.norm": (m.heads * m.dim,), x + "k.norm": (m.kv_heads * m.dim,), x + "sink": (m.heads,),
                            x + "g": (m.heads * m.vdim, W), x + "o": (W, m.heads * m.vdim)})
            else:
                out.update({x + "q": (m.heads * m.dim, W), x + "f": (m.heads * m.dim, W), x + "f.b": (m.heads * m.dim,),
                            x + "lower": (m.heads * m.dim,), x + "v": (m.heads * m.vdim, W), x + "norm": (m.vdim,),
                            x + "o": (W, m.heads * m.vdim)})
            if f is not None:
                out.update({p + "norm2": (W,), p + "norm2.b": (W,), p + "mlp.router": (f.experts, W)})
                for e in range(f.experts):
                    out.update({p + f"mlp.e{e}.up": (f.ff, W), p + f"mlp.e{e}.down": (W, f.ff)})
            if self.side_dim:
                out.update({p + "side.gate": (self.side_dim, W), p + "side.proj": (W, self.side_dim), p + "side.norm": (W,)})
        out.update({"final.norm": (W,), "final.norm.b": (W,), "head": (self.vocab, W)})
        return out


def random_weights(cfg: PitudraConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bfloat16 tensors of a configuration (CPU): matrices ~ N(0, 1/fan_in), norm weights near 1, the rest small;
    the recurrence's lower bounds lie in (0, 1)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.tensor_shapes().items():
        if len(shape) == 2:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif name.endswith("lower"):
            t = 0.05 + 0.9 * torch.rand(shape, generator=g)
        elif name.endswith((".norm", "norm1", "norm2")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            t = 0.2 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


class _LayerWeights:
    """Device tensors of one layer: large matrices in the activation type (fused where one product serves several),
    vectors and the router float32."""

    def __init__(self, cfg: PitudraConfig, i: int, sd: Dict[str, torch.Tensor], dtype, device):
        spec, p = cfg.layers[i], f"l{i}."
        m, f = spec.mixer, spec.mlp

        def big(*names):
            t = torch.cat([sd[p + n] for n in names], 0) if len(names) > 1 else sd[p + names[0]]
            return t.to(device=device, dtype=dtype).contiguous()

        def small(name):
            return sd[p + name].to(device=device, dtype=torch.float32).contiguous()

        self.shift, self.norm1, self.norm1_b = small("shift"), small("norm1"), small("norm1.b")
        if m.kind == "latent_attention":
            self.down = big("mix.dq", "mix.dkv") if m.kv_from is None else big("mix.dq")       # rows [dq ; dkv]
            self.dq_norm = small("mix.dq.norm")
            self.dkv_norm = small("mix.dkv.norm") if m.kv_from is None else None
            self.uq = big("mix.uq")
            self.uk_flat, self.uv_flat = big("mix.uk"), big("mix.uv")                            # latent rows -> per-head keys / values
            self.uk = self.uk_flat.view(m.heads, m.dim, m.kv_rank)                               # q_nope[h] @ uk[h] -> latent space
            self.uv_t = self.uv_flat.view(m.heads, m.vdim, m.kv_rank).transpose(1, 2)            # latent[h] @ uv_t[h] -> value space
            self.sink = small("mix.sink")
        elif m.kind == "attention":
            self.qkvg = big("mix.q", "mix.k", "mix.v", "mix.g")                                  # rows [q ; k ; v ; g]
            zeros = torch.zeros(m.heads * m.vdim, dtype=sd[p + "mix.q.b"].dtype)
            self.qkvg_b = torch.cat([sd[p + "mix.q.b"], sd[p + "mix.k.b"], sd[p + "mix.v.b"], zeros]).to(device=device, dtype=dtype)
            self.q_norm, self.k_norm, self.sink = small("mix.q.norm"), small("mix.k.norm"), small("mix.sink")
        else:
            self.qfv = big("mix.q", "mix.f", "mix.v")                                            # rows [q ; f ; v]
            self.f_b, self.lower, self.o_norm = small("mix.f.b"), small("mix.lower"), small("mix.norm")
        self.o = big("mix.o")
        if f is not None:
            self.norm2, self.norm2_b, self.router = small("norm2"), small("norm2.b"), small("mlp.router")
            self.up = torch.stack([sd[p + f"mlp.e{e}.up"] for e in range(f.experts)]).to(device=device, dtype=dtype).contiguous()
            self.edown = torch.stack([sd[p + f"mlp.e{e}.down"] for e in range(f.experts)]).to(device=device, dtype=dtype).contiguous()
        if cfg.side_dim:
            self.side_gate, self.side_proj, self.side_norm = big("side.gate"), big("side.proj"), small("side.norm")


class PitudraModel(torch.nn.Module):
    """Weights, per-slot state and the forward pass over a flat token batch (`state.BatchMeta`).

    dtype: torch.bfloat16 (serving: bfloat16 matrix products with float32 accumulation) or torch.float32 (everything in true
    float32). n_slots sequences can be live at once; a step carries at most max_step_tokens tokens."""

    architecture = "Pitudra"

    RING_ROWS_UNBOUNDED = 32768     # rings longer than this are cut to the sequence limit, if the caller gives one

    def __init__(self, cfg: PitudraConfig, weights: Dict[str, torch.Tensor], dtype=torch.bfloat16, device="cuda",
                 n_slots: int = 8, max_step_tokens: int = 2048, max_seq_tokens: Optional[int] = None):
        """max_seq_tokens: the most tokens a sequence will ever hold, if known. It only matters for windows so long that a
        ring of window - 1 + max_step_tokens rows would be wasteful: such rings get max_seq_tokens rows (positions then never
        wrap) and the model refuses longer sequences (`max_seq_len`, checked by the scheduler)."""
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("PitudraModel: dtype must be torch.bfloat16 or torch.float32")
        for name, shape in cfg.tensor_shapes().items():
            if name not in weights:
                raise KeyError(f"tensor {name} is missing from the checkpoint")
            if tuple(weights[name].shape) != tuple(shape):
                raise ValueError(f"tensor {name}: shape {tuple(weights[name].shape)}, the configuration says {tuple(shape)}")
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.n_slots, self.max_step_tokens = n_slots, max_step_tokens
        # true float32 products in float32 mode; no reduced-precision accumulation of bfloat16 products
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        dev, W, T, L = self.device, cfg.width, max_step_tokens, len(cfg.layers)
        f32 = dict(dtype=torch.float32, device=dev)
        act = dict(dtype=dtype, device=dev)
        self.embed = weights["embed"].to(**act).contiguous()
        self.side_embed = weights["side.embed"].to(**act).contiguous() if cfg.side_dim else None
        self.head = weights["head"].to(**act).contiguous()
        self.final_norm = weights["final.norm"].to(**f32).contiguous()
        self.final_norm_b = weights["final.norm.b"].to(**f32).contiguous()
        self.weights = [_LayerWeights(cfg, i, weights, dtype, dev) for i in range(L)]
        # ---- per-slot state ----
        self.prev = [torch.zeros(2, n_slots, W, **f32) for _ in range(L)]                     # token shift: last row, two phases
        self.latent_cache: Dict[int, torch.Tensor] = {}                                       # owner layer -> [slots, cap, kv_rank + rot_dim]
        self.cache_k: Dict[int, torch.Tensor] = {}
        self.cache_v: Dict[int, torch.Tensor] = {}
        self.rec_state: Dict[int, torch.Tensor] = {}
        self.inv_freq: Dict[int, torch.Tensor] = {}
        self.max_seq_len = None                        # set when a ring is cut to the caller's sequence limit

        def ring_rows(window: int) -> int:
            rows = window - 1 + T
            if rows > self.RING_ROWS_UNBOUNDED and max_seq_tokens:
                rows = min(rows, max(int(max_seq_tokens), T))
                self.max_seq_len = rows if self.max_seq_len is None else min(self.max_seq_len, rows)
            return rows

        for i, l in enumerate(cfg.layers):
            m = l.mixer
            if m.kind == "latent_attention":
                if m.kv_from is None:
                    # the ring must hold the widest window of any layer that reads it
                    win = max([m.window] + [o.mixer.window for o in cfg.layers if o.mixer.kv_from == i])
                    self.latent_cache[i] = torch.zeros(n_slots, ring_rows(win), m.kv_rank + m.rot_dim, **act)
                half = m.rot_dims // 2
                f = torch.tensor(m.rot_base, dtype=torch.float64) ** (-2.0 * torch.arange(half, dtype=torch.float64) / max(m.rot_dims, 1))
                self.inv_freq[i] = f.to(**f32)
            elif m.kind == "attention":
                cap = ring_rows(m.window)
                self.cache_k[i] = torch.zeros(n_slots, cap, m.kv_heads * m.dim, **act)
                self.cache_v[i] = torch.zeros(n_slots, cap, m.kv_heads * m.vdim, **act)
            else:
                self.rec_state[i] = torch.zeros(n_slots, m.heads, m.dim, m.vdim, **f32)
        # ---- scratch arena, allocated once ----
        mx = lambda vals: max(list(vals) + [1])
        mix = [l.mixer for l in cfg.layers]
        lat = [m for m in mix if m.kind == "latent_attention"]
        att = [m for m in mix if m.kind == "attention"]
        rec = [m for m in mix if m.kind == "hgrn2"]
        self.buf_x = torch.empty(T * W, **f32)                                                 # residual stream (updated in place)
        self.buf_h = torch.empty(T * W, **act)                                                 # sublayer input in the activation type
        self.buf_y = torch.empty(T * W, **act)                                                 # sublayer output
        self.buf_proj = torch.empty(T * mx([m.q_rank + m.kv_rank + m.rot_dim for m in lat] +
                                           [m.heads * (m.dim + 2 * m.vdim) + m.kv_heads * (m.dim + m.vdim) for m in att] +
                                           [m.heads * (2 * m.dim + m.vdim) for m in rec]), **act)
        self.buf_cq = torch.empty(T * mx(m.q_rank for m in lat), **act)
        self.buf_q = torch.empty(T * mx(m.heads * (m.dim + m.rot_dim) for m in lat), **act)
        self.buf_qa = torch.empty(T * mx([m.heads * (max(m.kv_rank, m.dim) + m.rot_dim) for m in lat] + [m.heads * m.dim for m in att]), **f32)
        self.buf_att = torch.empty(T * mx([m.heads * m.kv_rank for m in lat] + [m.heads * m.vdim for m in att + rec]), **act)
        self.buf_att2 = torch.empty(T * mx(m.heads * m.vdim for m in lat), **act)
        self.buf_rec = torch.empty(T * mx(m.heads * (m.vdim + 3 * m.dim) for m in rec), **f32)   # un-normalised outputs + gates
        moes = [l.mlp for l in cfg.layers if l.mlp]
        tops = mx(f.top for f in moes)
        self.buf_idx = torch.empty(T * tops, dtype=torch.int32, device=dev)
        self.buf_rw = torch.empty(T * tops, **f32)
        self.buf_pair = torch.empty(T * tops * W if moes else 1, **act)
        self.buf_side = torch.empty(T * max(cfg.side_dim, 1), **act)
        # bfloat16 takes the tensor-core forms where the sizes allow: grouped experts once an expert sees several rows, window
        # attention per 16 tokens (prompts) or per group of query heads (decoding). QSPEC_SEQ_TILES=0 keeps the plain forms.
        self.use_tiles = dtype == torch.bfloat16 and os.environ.get("QSPEC_SEQ_TILES", "1") != "0"
        self.tiles_min_tokens = 64           # a step with fewer tokens, or fewer than 16 per sequence, is decode-shaped
        # A prompt portion of a latent-attention layer runs in the expanded form: per-head keys and values of the slot's ring
        # rows from two products (key = [W_uk c | shared rotary part]), which costs a third of the absorbed form's work per
        # (query, key) pair. Scratch for one slot's ring.
        lat_tiles = [l.mixer for l in cfg.layers if l.mixer.kind == "latent_attention" and self.use_tiles and
                     ops.seq_window_attention_mma_supported(dtype, l.mixer.dim, l.mixer.rot_dim, l.mixer.vdim, l.mixer.heads, l.mixer.heads, True)
                     and l.mixer.kv_rank % 8 == 0 and l.mixer.rot_dim % 8 == 0]
        caps = {i: c.shape[1] for i, c in self.latent_cache.items()}
        need_k = mx(caps[i if l.mixer.kv_from is None else l.mixer.kv_from] * l.mixer.heads * l.mixer.dim
                    for i, l in enumerate(cfg.layers) if l.mixer in lat_tiles)
        need_v = mx(caps[i if l.mixer.kv_from is None else l.mixer.kv_from] * l.mixer.heads * l.mixer.vdim
                    for i, l in enumerate(cfg.layers) if l.mixer in lat_tiles)
        self.buf_kmat = torch.empty(need_k, **act)
        self.buf_vmat = torch.empty(need_v, **act)
        self._lat_tiles = {id(m) for m in lat_tiles}
        self._bmm_f32_out = None                       # whether torch.bmm takes bfloat16 operands with a float32 out (probed once)

    # ------------------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, path: str, dtype=torch.bfloat16, device="cuda", **kw) -> "PitudraModel":
        from .checkpoint import read_safetensors_file
        with open(os.path.join(path, "config.json")) as f:
            cfg = PitudraConfig.from_dict(json.load(f))
        return cls(cfg, read_safetensors_file(os.path.join(path, "model.safetensors")), dtype=dtype, device=device, **kw)

    @property
    def vocab_size(self) -> int:
        return self.cfg.vocab

    def state_bytes_per_slot(self) -> int:
        ts = self.prev + list(self.latent_cache.values()) + list(self.cache_k.values()) + list(self.cache_v.values()) + \
            list(self.rec_state.values())
        return sum(t.numel() * t.element_size() // self.n_slots for t in ts)

    def _bmm_to_f32(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
        """out (float32) = a @ b per batch entry, accumulated in float32 whatever the operands' type."""
        if a.dtype == torch.float32:
            torch.bmm(a, b, out=out)
            return
        if self._bmm_f32_out is None:
            try:
                torch.bmm(a, b, out_dtype=torch.float32, out=out)
                self._bmm_f32_out = True
                return
            except (TypeError, RuntimeError):
                self._bmm_f32_out = False
        if self._bmm_f32_out:
            torch.bmm(a, b, out_dtype=torch.float32, out=out)
        else:
            out.copy_(torch.bmm(a, b))

    # ------------------------------------------------------------------------------------------
    def _latent_attention(self, i, m, p, h, meta, T, prompt_shaped):
        tab = meta.table
        own = m.kv_from is None
        ld = m.q_rank + (m.kv_rank + m.rot_dim if own else 0)
        d = self.buf_proj[:T * ld].view(T, ld)
        torch.matmul(h, p.down.t(), out=d)
        cq = self.buf_cq[:T * m.q_rank].view(T, m.q_rank)
        src = i if own else m.kv_from
        cache = self.latent_cache[src]
        ops.seq_latent_prep(d, m.q_rank, m.kv_rank, m.rot_dim, p.dq_norm, p.dkv_norm, self.inv_freq[i], m.rot_dims, cq,
                            cache if own else None, tab, self.cfg.eps)
        H, DQ = m.heads, m.dim + m.rot_dim
        q = self.buf_q[:T * H * DQ].view(T, H, DQ)
        torch.matmul(cq, p.uq.t(), out=q.view(T, H * DQ))
        if prompt_shaped and len(meta.segments) == 1 and id(m) in self._lat_tiles:
            # expanded form on the tensor cores: keys and values of every ring row of this sequence's slot
            slot, cap = meta.segments[0][1], cache.shape[1]
            ring = cache[slot]
            kmat = self.buf_kmat[:cap * H * m.dim].view(cap, H * m.dim)
            vmat = self.buf_vmat[:cap * H * m.vdim].view(cap, H * m.vdim)
            torch.matmul(ring[:, :m.kv_rank], p.uk_flat.t(), out=kmat)
            torch.matmul(ring[:, :m.kv_rank], p.uv_flat.t(), out=vmat)
            qf = self.buf_qa[:T * H * DQ].view(T, H, DQ)
            qf[:, :, :m.dim].copy_(q[:, :, :m.dim])
            ops.seq_rotary(q, m.dim, qf[:, :, m.dim:], m.rot_dims, self.inv_freq[i], tab)
            att = self.buf_att2[:T * H * m.vdim].view(T, H, m.vdim)
            ops.seq_window_attention_mma(qf, kmat.view(1, cap, H, m.dim).expand(self.n_slots, cap, H, m.dim), cache[:, :, m.kv_rank:],
                                         vmat.view(1, cap, H, m.vdim).expand(self.n_slots, cap, H, m.vdim), att, tab, m.window, m.scale,
                                         True, sink=p.sink)
            return att.view(T, H * m.vdim)
        # absorbed form: the query moves into the latent space (W_uk^T q_nope per head, float32) and the cache rows serve as
        # keys and as values; the up-projection of the values follows the attention
        r, R = m.kv_rank, m.rot_dim
        qf = self.buf_qa[:T * H * (r + R)].view(T, H, r + R)
        self._bmm_to_f32(q[:, :, :m.dim].transpose(0, 1), p.uk, qf[:, :, :r].transpose(0, 1))
        ops.seq_rotary(q, m.dim, qf[:, :, r:], m.rot_dims, self.inv_freq[i], tab)
        olat = self.buf_att[:T * H * r].view(T, H, r)
        groups = 1 if H <= 16 else (H // 16 if H % 16 == 0 else 0)                 # the heads share one key row: 16 of them per CTA
        if self.use_tiles and groups and r % 8 == 0 and R % 8 == 0 and \
                ops.seq_window_attention_mma_supported(self.dtype, r, R, r, H, groups, False):
            ck = cache[:, :, :r].unsqueeze(2).expand(cache.shape[0], cache.shape[1], groups, r)
            ops.seq_window_attention_mma(qf, ck, cache[:, :, r:], ck, olat, tab, m.window, m.scale, False, sink=p.sink)
        else:
            ck = cache.unsqueeze(2)                                                 # one key/value head: [slots, cap, 1, kv_rank + rot_dim]
            ops.seq_window_attention(qf[:, :, :r], qf[:, :, r:], ck, ck[..., :r], olat, tab, m.window, m.scale, sink=p.sink)
        att = self.buf_att2[:T * H * m.vdim].view(T, H, m.vdim)
        torch.bmm(olat.transpose(0, 1), p.uv_t, out=att.transpose(0, 1))
        return att.view(T, H * m.vdim)

    def _attention(self, i, m, p, h, tab, T, prompt_shaped):
        HD, GD, GDV, HDV = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim, m.heads * m.vdim
        ld = HD + GD + GDV + HDV
        proj = self.buf_proj[:T * ld].view(T, ld)
        torch.addmm(p.qkvg_b, h, p.qkvg.t(), out=proj)                             # biases added in the projection
        qf = self.buf_qa[:T * HD].view(T, HD)
        ck, cv = self.cache_k[i], self.cache_v[i]
        ops.seq_qkv_prep(proj, HD, GD, GDV, p.q_norm, p.k_norm, qf, ck, cv, tab, self.cfg.eps)
        att = self.buf_att[:T * HDV].view(T, m.heads, m.vdim)
        cap = ck.shape[1]
        k4, v4 = ck.view(self.n_slots, cap, m.kv_heads, m.dim), cv.view(self.n_slots, cap, m.kv_heads, m.vdim)
        gate = proj[:, HD + GD + GDV:]
        if self.use_tiles and ld % 8 == 0 and ops.seq_window_attention_mma_supported(self.dtype, m.dim, 0, m.vdim, m.heads, m.kv_heads, prompt_shaped):
            ops.seq_window_attention_mma(qf.view(T, m.heads, m.dim), k4, None, v4, att, tab, m.window, m.scale, prompt_shaped, sink=p.sink,
                                         gate=gate)
        else:
            ops.seq_window_attention(qf.view(T, m.heads, m.dim), None, k4, v4, att, tab, m.window, m.scale, sink=p.sink, gate=gate)
        return att.view(T, HDV)

    def _hgrn2(self, i, m, p, h, meta, T):
        tab = meta.table
        ld = m.heads * (2 * m.dim + m.vdim)
        proj = self.buf_proj[:T * ld].view(T, ld)
        torch.matmul(h, p.qfv.t(), out=proj)
        att = self.buf_att[:T * m.heads * m.vdim].view(T, m.heads * m.vdim)
        ops.seq_hgrn2(proj, p.f_b, p.lower, p.o_norm, self.rec_state[i], self.buf_rec, att, tab, m.heads, m.dim, m.vdim, self.cfg.eps,
                      seg_starts=meta.seg_starts)
        return att

    @torch.no_grad()
    def forward_batch(self, input_ids: torch.Tensor, meta: BatchMeta, trace: Optional[list] = None) -> torch.Tensor:
        """input_ids: int32 [ntok] on the device. Returns the final-norm hidden state [ntok, W] (activation type), a view of
        the arena. `trace`, if a list, receives a copy of the residual stream after every layer (debugging)."""
        cfg, T, W = self.cfg, meta.ntok, self.cfg.width
        if T > self.max_step_tokens or input_ids.numel() != T:
            raise ValueError(f"forward_batch: {T} tokens (at most {self.max_step_tokens})")
        tab, eps = meta.table, cfg.eps
        x = self.buf_x[:T * W].view(T, W)
        h = self.buf_h[:T * W].view(T, W)
        y = self.buf_y[:T * W].view(T, W)
        ops.seq_embed(self.embed, input_ids, x)
        prompt_shaped = self.use_tiles and T >= self.tiles_min_tokens and T >= 16 * len(meta.segments)
        for i, spec in enumerate(cfg.layers):
            p, m, f = self.weights[i], spec.mixer, spec.mlp
            ops.seq_token_shift(x, p.shift, self.prev[i], h, tab)
            if m.kind == "latent_attention":
                att = self._latent_attention(i, m, p, h, meta, T, prompt_shaped)
            elif m.kind == "attention":
                att = self._attention(i, m, p, h, tab, T, prompt_shaped)
            else:
                att = self._hgrn2(i, m, p, h, meta, T)
            torch.matmul(att, p.o.t(), out=y)
            more = f is not None or cfg.side_dim > 0                                # a later sublayer of this layer reads x
            ops.seq_add_norm(y, p.norm1, p.norm1_b, eps, x_in=x, x_out=x, out=h if more else None)
            if f is not None:
                idx = self.buf_idx[:T * f.top].view(T, f.top)
                rw = self.buf_rw[:T * f.top].view(T, f.top)
                pair = self.buf_pair[:T * f.top * W].view(T, f.top, W)
                ops.moe_route_chosen(h, p.router, idx, rw)
                # grouped tiles once an expert sees several rows on average; a handful of tokens stay with the row-per-CTA form
                if self.use_tiles and T * f.top >= 4 * f.experts and ops.moe_expert_grouped_supported(h, f.ff):
                    ops.moe_expert_grouped(h, p.up, p.edown, idx, pair, f.experts, f.ff, 0.0, act="relu2")
                else:
                    ops.moe_expert_tokens(h, p.up, p.edown, idx, pair, f.experts, f.ff, 0.0, act="relu2")
                ops.seq_add_norm(pair, p.norm2, p.norm2_b, eps, x_in=x, x_out=x, out=h if cfg.side_dim else None, y_w=rw)
            if cfg.side_dim:
                sd = cfg.side_dim
                g = self.buf_side[:T * sd].view(T, sd)
                torch.matmul(h, p.side_gate.t(), out=g)
                ops.seq_side_gate(g, self.side_embed, input_ids, i * sd)
                torch.matmul(g, p.side_proj.t(), out=y)
                ops.seq_add_norm(y, p.side_norm, None, eps, kind="rms", x_in=x, x_out=x)
            if trace is not None:
                trace.append(x.clone())
        ops.seq_add_norm(x, self.final_norm, self.final_norm_b, eps, out=h)
        return h

    @torch.no_grad()
    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [n, vocab] of final-norm hidden rows [n, W]."""
        if self.dtype == torch.float32:
            return torch.matmul(hidden_rows, self.head.t())
        return torch.mm(hidden_rows, self.head.t(), out_dtype=torch.float32)
