"""Mutusun on the GPU against the plain CPU restatement (oracle/mutusun_oracle.py): every mechanism alone, then whole
models through the scheduler's step function -- whole prompts, token-by-token decoding, portions of every size, mixed
batches, reused slots, chunk and tail edges, other sizes, and greedy generation."""
import math

import pytest
import torch

from oracle import mutusun_oracle as O

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from qspec_b200.build import build_seq_library
    build_seq_library()


def meta_table(segments):
    """segments: (slot, first position, count, phase) -> int32 [5, ntok] on the device."""
    rows = [[], [], [], [], []]
    at = 0
    for slot, p0, n, phase in segments:
        for k in range(n):
            for r, v in zip(rows, (slot, p0 + k, at, at + n, phase)):
                r.append(v)
        at += n
    return torch.tensor(rows, dtype=torch.int32, device="cuda")


def bf16_round(t):
    return t.to(BF16).to(torch.float64)


def tol(dtype):
    return 2e-5 if dtype == F32 else 2.5e-2


def close(got, want, dtype, scale=None):
    want = want.to(torch.float64)
    s = float(want.abs().max()) if scale is None else scale
    err = float((got.detach().cpu().to(torch.float64) - want).abs().max())
    assert err <= tol(dtype) * max(s, 1e-6), f"max error {err:.3g} against scale {s:.3g}"


# ---------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("W,taps", [(96, 3), (40, 1), (257, 4), (64, 2)])
def test_norm_conv_with_tail_over_portions(dtype, W, taps):
    """Residual sum + both norms + convolution; the sequence is cut into portions of 1, 2, 5, ... tokens in two slots so
    that every tail row is carried, overwritten and read at a portion's start."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(W * 10 + taps)
    T, eps = 23, 1e-5
    x = torch.randn(T, W, generator=g, dtype=torch.float64) * 3
    y = bf16_round(torch.randn(T, W, generator=g)) if dtype == BF16 else torch.randn(T, W, generator=g, dtype=torch.float64).float().double()
    post_w, pre_w = [0.3 * torch.randn(W, generator=g, dtype=torch.float64).float().double() for _ in range(2)]
    cw = 0.5 * torch.randn(W, taps, generator=g, dtype=torch.float64).float().double()
    r = x.float().double() + O.norm_zero_centred(y, post_w, eps)
    want = O.short_conv_residual(O.norm_zero_centred(r, pre_w, eps), cw)
    hist = taps - 1
    for slot in (0, 2):
        tail = torch.full((2, 3, hist, W), float("nan"), dtype=F32, device="cuda") if hist else None
        phase, at, cuts = 0, 0, [1, 2, 1, 5, 2, 3, 9]
        got, res = [], []
        for n in cuts:
            tab = meta_table([(slot, at, n, phase)])
            out = torch.empty(n, W, dtype=dtype, device="cuda")
            xo = torch.empty(n, W, dtype=F32, device="cuda")
            ops.seq_norm_conv(x[at:at + n].float().cuda(), tab, eps, out=out, pre_w=pre_w.float().cuda(), conv_w=cw.float().cuda(),
                              tail=tail, y=y[at:at + n].to(dtype).cuda(),
                              post_w=post_w.float().cuda(), x_out=xo)
            got.append(out.float().cpu()); res.append(xo.cpu())
            at += n
            phase ^= 1
        close(torch.cat(res), r, F32)
        close(torch.cat(got), want, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("W,taps,parts", [(96, 3, 1), (257, 4, 1), (1024, 2, 3), (2100, 5, 1)])
def test_norm_conv_of_long_prompts_in_two_passes(dtype, W, taps, parts):
    """256 tokens or more with a scratch buffer take the two-launch form (rows independent, then the convolution): two
    sequences in one batch, each continued from an earlier portion whose tail it reads (the other tail buffer is NaN-filled),
    one of them still in its first taps - 1 positions; against the plain implementation and, bit for bit, the one-launch form."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(W + taps)
    eps, hist = 1e-5, taps - 1
    lens = {0: (1, 150), 2: (7, 130)}                        # slot -> (first portion, second portion)
    seqs = {}
    for slot, (n0, n1) in lens.items():
        T = n0 + n1
        x = (torch.randn(T, W, generator=g) * 3).double()
        yp = torch.randn(T, parts, W, generator=g)
        yp = bf16_round(yp) if dtype == BF16 else yp.double()
        yw = torch.rand(T, parts, generator=g).double() if parts > 1 else torch.ones(T, 1, dtype=torch.float64)
        seqs[slot] = (x, yp, yw)
    post_w, pre_w = [0.3 * torch.randn(W, generator=g).double() for _ in range(2)]
    cw = 0.5 * torch.randn(W, taps, generator=g).double()
    want = {}
    for slot, (x, yp, yw) in seqs.items():
        r = x + O.norm_zero_centred((yp.double() * yw[:, :, None]).sum(1), post_w, eps)
        want[slot] = (r, O.short_conv_residual(O.norm_zero_centred(r, pre_w, eps), cw))
    dev = lambda t: t.float().cuda()
    results = []
    for use_scratch in (True, False):
        tail = torch.full((2, 3, hist, W), float("nan"), dtype=F32, device="cuda")
        scratch = torch.full((300 * W,), float("nan"), dtype=F32, device="cuda") if use_scratch else None
        got = {}
        for step in (0, 1):
            segs, xs, ys, ws = [], [], [], []
            for slot, (n0, n1) in lens.items():
                a, b = (0, n0) if step == 0 else (n0, n0 + n1)
                segs.append((slot, a, b - a, step))
                xs.append(seqs[slot][0][a:b]); ys.append(seqs[slot][1][a:b]); ws.append(seqs[slot][2][a:b])
            tab = meta_table(segs)
            x, y, yw = torch.cat(xs), torch.cat(ys), torch.cat(ws)
            n = x.shape[0]
            out = torch.empty(n, W, dtype=dtype, device="cuda")
            xo = torch.empty(n, W, dtype=F32, device="cuda")
            ops.seq_norm_conv(dev(x), tab, eps, out=out, pre_w=dev(pre_w), conv_w=dev(cw), tail=tail,
                              y=(y if parts > 1 else y[:, 0]).to(dtype).cuda().contiguous(), y_w=dev(yw) if parts > 1 else None,
                              post_w=dev(post_w), x_out=xo, scratch=scratch)
            if step == 1:
                at = 0
                for slot, (n0, n1) in lens.items():
                    got[slot] = (xo[at:at + n1].cpu(), out[at:at + n1].float().cpu())
                    at += n1
        for slot, (n0, n1) in lens.items():
            close(got[slot][0], want[slot][0][n0:], F32)
            close(got[slot][1], want[slot][1][n0:], dtype)
        results.append((got, tail[0][[0, 2]].clone()))        # the second step read tail buffer 1 and wrote buffer 0
    for slot in lens:
        assert torch.equal(results[0][0][slot][0], results[1][0][slot][0]) and torch.equal(results[0][0][slot][1], results[1][0][slot][1])
    assert not torch.isnan(results[0][1]).any() and torch.equal(results[0][1], results[1][1])


def test_norm_conv_partial_sums_and_weights():
    """The pending output given as weighted parts (mixture-of-experts form) equals the weighted sum given whole."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(5)
    T, W, P = 7, 48, 3
    x = torch.randn(T, W, generator=g)
    parts = torch.randn(T, P, W, generator=g)
    pw = torch.rand(T, P, generator=g)
    w1, w2 = 0.2 * torch.randn(W, generator=g), 0.2 * torch.randn(W, generator=g)
    tab = meta_table([(0, 0, T, 0)])
    r = x.double() + O.norm_zero_centred((parts.double() * pw.double()[:, :, None]).sum(1), w1.double(), 1e-5)
    want = O.norm_zero_centred(r, w2.double(), 1e-5)
    out = torch.empty(T, W, dtype=F32, device="cuda")
    xo = torch.empty(T, W, dtype=F32, device="cuda")
    ops.seq_norm_conv(x.cuda(), tab, 1e-5, out=out, pre_w=w2.cuda(), y=parts.cuda(), y_w=pw.cuda(), post_w=w1.cuda(), x_out=xo)
    close(out, want, F32)
    close(xo, r, F32)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_qk_norm(dtype):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(1)
    T, H, G, D, DV = 5, 3, 1, 24, 10
    ld = H * D + G * D + G * DV
    buf = torch.randn(T, ld, generator=g).to(dtype)
    qw, kw = 1 + 0.2 * torch.randn(D, generator=g), 1 + 0.2 * torch.randn(D, generator=g)
    ref = buf.to(torch.float64).clone()
    ref[:, :H * D] = O.norm_plain(ref[:, :H * D].view(T, H, D), qw.double(), 1e-6).reshape(T, H * D)
    ref[:, H * D:(H + G) * D] = O.norm_plain(ref[:, H * D:(H + G) * D].view(T, G, D), kw.double(), 1e-6).reshape(T, G * D)
    d = buf.cuda()
    ops.seq_qk_norm(d, qw.cuda(), kw.cuda(), H, G, D, 1e-6)
    close(d, ref, dtype)
    assert torch.equal(d[:, (H + G) * D:].cpu(), buf[:, (H + G) * D:])          # values untouched


def _attention_reference(q, k, v, bias, H, G, size, scale, cap):
    T = q.shape[0]
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            for j in range(T):
                if O.chunk_visible(i, j, size):
                    s = float(q[i, h] @ k[j, g]) * scale
                    if cap:
                        s = cap * math.tanh(s / cap)
                    out[i, h] += (1.0 / (1.0 + math.exp(-(s + float(bias[h]))))) * v[j, g]
    return out.reshape(T, -1)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,G,D,DV,size,cap", [(4, 2, 16, 8, 7, 5.0), (3, 3, 8, 24, 16, 0.0), (2, 1, 32, 32, 5, 30.0)])
def test_chunk_attention_cache_and_edges(dtype, H, G, D, DV, size, cap):
    """Portions that start and end inside chunks, on their borders and span several of them; single tokens; two slots in
    one batch with a slot that held another sequence before."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + size)
    T = 3 * size + 2
    ld = H * D + G * D + G * DV
    seqs = {}
    for slot in (1, 0):
        qkv = torch.randn(T, ld, generator=g).to(dtype)
        f = qkv.to(torch.float64)
        seqs[slot] = (qkv, _attention_reference(f[:, :H * D].view(T, H, D), f[:, H * D:(H + G) * D].view(T, G, D),
                                                f[:, (H + G) * D:].view(T, G, DV), torch.linspace(-1, 1, H), H, G, size, 0.3, cap))
    bias = torch.linspace(-1, 1, H).cuda()
    ck = torch.full((2, size, G, D), 1e4, dtype=dtype, device="cuda")           # stale rows of an earlier owner: loud if ever read
    cv = torch.full((2, size, G, DV), 1e4, dtype=dtype, device="cuda")
    cuts = [1, 1, size - 2, 2, 1, size + 3, 1]
    cuts = [n for n in cuts + [T - sum(cuts)] if n > 0]
    got = {0: [], 1: []}
    at = 0
    for n in cuts:
        tab = meta_table([(1, at, n, 0), (0, at, n, 0)])
        batch = torch.cat((seqs[1][0][at:at + n], seqs[0][0][at:at + n])).cuda()
        out = torch.empty(2 * n, H * DV, dtype=dtype, device="cuda")
        ops.seq_chunk_attention(batch, ck, cv, bias, out, tab, H, G, D, DV, size, 0.3, cap)
        ops.seq_cache_append(batch, ck, cv, tab, H, G, D, DV, size)
        got[1].append(out[:n].float().cpu()); got[0].append(out[n:].float().cpu())
        at += n
    for slot in (0, 1):
        close(torch.cat(got[slot]), seqs[slot][1], dtype)


def _attention_reference_dense(q, k, v, bias, H, G, size, scale, cap):
    """The same sum written with whole matrices (float64), for chunks of a few hundred keys."""
    T = q.shape[0]
    pos = torch.arange(T)
    seen = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        out[:, h] = (torch.sigmoid(s + bias[h]) * seen) @ v[:, g]
    return out.reshape(T, -1)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,G,D,DV,size", [(4, 2, 16, 8, 70), (8, 2, 32, 64, 300), (3, 1, 64, 32, 129), (2, 2, 128, 128, 257),
                                           (8, 2, 64, 64, 300), (12, 2, 128, 64, 100), (16, 1, 64, 128, 70), (12, 1, 128, 128, 33),
                                           (1, 1, 64, 64, 31)])
def test_decoding_attention_with_the_keys_of_a_token_spread_over_a_cluster(dtype, H, G, D, DV, size):
    """Few tokens, many keys: 2, 4 or 8 CTAs share the key blocks of a token. Two sequences decode across a chunk border
    (from nearly `size` keys down to one), one of them two positions ahead of the other; the key bound is given or left out.
    Head sizes of 64 / 128 in bfloat16 take the tensor-core token form (1 to 16 query heads per key/value head, more
    than 8 included), the others and float32 the element-wise one."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(size)
    T = size + 9
    ld = H * D + G * D + G * DV
    bias = torch.linspace(-3, -1, H)
    seqs = {}
    for slot in (0, 1):
        qkv = (0.5 * torch.randn(T, ld, generator=g)).to(dtype)
        f = qkv.to(torch.float64)
        seqs[slot] = (qkv, _attention_reference_dense(f[:, :H * D].view(T, H, D), f[:, H * D:(H + G) * D].view(T, G, D),
                                                      f[:, (H + G) * D:].view(T, G, DV), bias.double(), H, G, size, 0.3, 4.0))
    ck = torch.full((2, size, G, D), 1e4, dtype=dtype, device="cuda")
    cv = torch.full((2, size, G, DV), 1e4, dtype=dtype, device="cuda")
    first = {0: size - 7, 1: size - 5}                       # prompt lengths; then one token per step
    got = {0: [], 1: []}
    at = dict(first)
    tab = meta_table([(0, 0, first[0], 0), (1, 0, first[1], 0)])
    batch = torch.cat((seqs[0][0][:first[0]], seqs[1][0][:first[1]])).cuda()
    out = torch.empty(batch.shape[0], H * DV, dtype=dtype, device="cuda")
    ops.seq_chunk_attention(batch, ck, cv, bias.cuda(), out, tab, H, G, D, DV, size, 0.3, 4.0, max_keys=max(first.values()))
    ops.seq_cache_append(batch, ck, cv, tab, H, G, D, DV, size)
    got[0].append(out[:first[0]].float().cpu()); got[1].append(out[first[0]:].float().cpu())
    for step in range(12):
        tab = meta_table([(1, at[1], 1, 0), (0, at[0], 1, 0)])
        batch = torch.cat((seqs[1][0][at[1]:at[1] + 1], seqs[0][0][at[0]:at[0] + 1])).cuda()
        out = torch.empty(2, H * DV, dtype=dtype, device="cuda")
        ops.seq_chunk_attention(batch, ck, cv, bias.cuda(), out, tab, H, G, D, DV, size, 0.3, 4.0,
                                max_keys=(at[1] + 1) if step % 2 else 0)
        ops.seq_cache_append(batch, ck, cv, tab, H, G, D, DV, size)
        got[1].append(out[:1].float().cpu()); got[0].append(out[1:].float().cpu())
        at[0] += 1; at[1] += 1
    for slot in (0, 1):
        close(torch.cat(got[slot]), seqs[slot][1][:at[slot]], dtype)


def test_attention_far_key_inside_and_outside_the_chunk():
    """One key is made to dominate (score pushed up, bias keeps all others near zero weight): the output equals that key's
    value exactly when it lies in the query's chunk -- first row of the chunk included -- and not one row further."""
    _cuda()
    from qspec_b200 import ops
    H, G, D, DV, size = 2, 1, 8, 4, 50
    T = 2 * size
    ld = H * D + G * D + G * DV
    tab = meta_table([(0, 0, T - 1, 0)])
    tab1 = meta_table([(0, T - 1, 1, 0)])
    for key_pos, visible in ((size, True), (size - 1, False)):
        qkv = torch.zeros(T, ld)
        qkv[:, H * D:(H + G) * D] = 0.0
        qkv[key_pos, H * D] = 10.0                                   # the marked key
        qkv[:, :H * D] = 0.0
        qkv[:, 0] = 10.0; qkv[:, D] = 10.0                           # every query looks for it
        qkv[:, (H + G) * D:] = torch.arange(T)[:, None] * 1.0 + torch.arange(DV)[None, :] * 0.001
        bias = torch.full((H,), -40.0).cuda()                         # unmarked keys weigh sigmoid(-40)
        ck = torch.zeros(1, size, G, D, device="cuda"); cv = torch.zeros(1, size, G, DV, device="cuda")
        d = qkv.cuda()
        out = torch.empty(T - 1, H * DV, device="cuda")
        ops.seq_chunk_attention(d[:T - 1].contiguous(), ck, cv, bias, out, tab, H, G, D, DV, size, 1.0, 0.0)
        ops.seq_cache_append(d[:T - 1].contiguous(), ck, cv, tab, H, G, D, DV, size)
        out1 = torch.empty(1, H * DV, device="cuda")
        ops.seq_chunk_attention(d[T - 1:].contiguous(), ck, cv, bias, out1, tab1, H, G, D, DV, size, 1.0, 0.0)   # decoded alone
        w = 1.0 / (1.0 + math.exp(-(100.0 - 40.0)))
        for o in (out[T - 2], out1[0]):
            if visible:
                assert abs(float(o[0]) - w * key_pos) < 1e-3
            else:
                assert abs(float(o[0])) < 1e-6


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("R,top,ident", [(12, 4, 4), (5, 1, 0), (40, 6, 1)])
def test_router_and_experts(dtype, R, top, ident):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(R)
    T, W, F, E, limit = 9, 48, 20, R - ident, 1.5
    h = torch.randn(T, W, generator=g).to(dtype)
    rw = torch.randn(R, W, generator=g) * 0.5
    corr = torch.randn(R, generator=g) * 0.3
    idx_ref, w_ref = O.route(h.double(), rw.double(), corr.double(), top)
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wt = torch.empty(T, top, dtype=F32, device="cuda")
    ops.moe_route(h.cuda(), rw.cuda(), corr.cuda(), idx, wt)
    assert torch.equal(idx.cpu().long().sort(1).values, idx_ref.sort(1).values)
    order = idx.cpu().long()
    close(wt, torch.gather(torch.softmax(h.double() @ rw.double().T, -1), 1, order), F32)
    gate_up = (torch.randn(E, 2 * F, W, generator=g) / W ** 0.5).to(dtype)
    down = (torch.randn(E, W, F, generator=g) / F ** 0.5).to(dtype)
    out = torch.empty(T, top, W, dtype=dtype, device="cuda")
    ops.moe_expert_tokens(h.cuda(), gate_up.cuda(), down.cuda(), idx, out, E, F, limit)
    ref = torch.zeros(T, top, W, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(order[t, k])
            ref[t, k] = h[t].double() if e >= E else O.expert_ff(h[t:t + 1].double(), gate_up[e, :F].double(), gate_up[e, F:].double(),
                                                                   down[e].double(), limit)[0]
    close(out, ref, dtype)


def test_relu2_and_argmax():
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(3)
    a = torch.randn(1000, generator=g)
    d = a.cuda()
    ops.seq_relu2(d)
    close(d, torch.relu(a.double()) ** 2, F32)
    lg = torch.randn(5, 777, generator=g)
    lg[2, 5] = lg[2, 700] = 9.0                                       # equal maxima: the lower index wins
    assert ops.argmax_rows(lg.cuda()).tolist() == [int(v) for v in lg.argmax(1)[:2]] + [5] + [int(v) for v in lg.argmax(1)[3:]]
    assert ops.argmax_rows(lg.to(BF16).cuda()).tolist()[2] == 5


# ---------------------------------------------------------------------------------------------------------------------
# whole models through the scheduler
# ---------------------------------------------------------------------------------------------------------------------
def mixer(heads=4, kv=2, dim=16, vdim=16, size=12, scale=0.2, cap=8.0):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "softcap": cap, "mask": {"size": size}}


def moe(ff=24, experts=5, identity=2, top=3, limit=1.25):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}


def config(layers, width=64, vocab=97, taps=3, eps=1e-5):
    return {"architecture": "Mutusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "layers": [dict(type="attention", **l) for l in layers]}


CONFIGS = {
    "mixed": config([dict(mixer=mixer(), mlp={"kind": "dense", "ff": 80}), dict(mixer=mixer(), mlp=moe()),
                     dict(mixer=mixer(), mlp=moe(), weights_of=1), dict(mixer=mixer(heads=2, kv=2, dim=8, vdim=24, size=5, cap=0.0), mlp=None)]),
    "odd": config([dict(mixer=mixer(heads=3, kv=1, dim=24, vdim=8, size=7, scale=0.5, cap=2.0), mlp=moe(ff=10, experts=3, identity=0, top=1)),
                   dict(mixer=mixer(heads=1, kv=1, dim=40, vdim=40, size=31), mlp={"kind": "dense", "ff": 33})],
                  width=72, vocab=50, taps=2, eps=1e-6),
    "taps4": config([dict(mixer=mixer(size=9), mlp=moe(experts=2, identity=3, top=4)), dict(mixer=mixer(size=9), mlp=moe(experts=2, identity=3, top=4), weights_of=0)],
                    width=48, taps=4),
    # nothing divisible by anything: odd head sizes and leading dimension (element-wise kernels), five taps, one kv head
    "ragged": config([dict(mixer=mixer(heads=3, kv=1, dim=9, vdim=5, size=6, scale=0.4, cap=3.0), mlp=moe(ff=7, experts=3, identity=1, top=2)),
                      dict(mixer=mixer(heads=2, kv=2, dim=10, vdim=6, size=11), mlp={"kind": "dense", "ff": 13}),
                      dict(mixer=mixer(heads=2, kv=2, dim=10, vdim=6, size=11), mlp={"kind": "dense", "ff": 13}, weights_of=1)],
                     width=50, vocab=33, taps=5),
    "notaps": config([dict(mixer=mixer(size=4), mlp={"kind": "dense", "ff": 16})], width=32, taps=1),
}


def build(name, dtype, seed=0, n_slots=3, max_step_tokens=64):
    _cuda()
    from qspec_b200.mutusun import MutusunConfig, MutusunModel, random_weights
    from qspec_b200.scheduler import Scheduler
    cfg = MutusunConfig.from_dict(CONFIGS[name])
    w = random_weights(cfg, seed)
    model = MutusunModel(cfg, w, dtype=dtype, device="cuda", n_slots=n_slots, max_step_tokens=max_step_tokens)
    return CONFIGS[name], w, model, Scheduler(model)


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def logits_scale(ref):
    return float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())


def close_logits(got, ref, dtype):
    """Per position: root mean square over the vocabulary of the difference (mean taken off), relative to the spread of
    the logits. float32 must sit at rounding level; bfloat16 within what its 8-bit mantissa leaves after a few layers."""
    d = got.detach().cpu().to(torch.float64) - ref.to(torch.float64)
    d = d - d.mean(-1, keepdim=True)
    rows = d.pow(2).mean(-1).sqrt() / logits_scale(ref.to(torch.float64))
    if dtype == F32:                                       # the sharp test of the logic
        assert float(rows.max()) <= 1e-5, f"worst position: {float(rows.max()):.3g} of the logits' spread"
        return
    # bfloat16: rounding level at the typical position; with random weights a router choice can flip on a near tie of
    # two experts' scores, which moves that position (and faintly its chunk) by far more than rounding
    over = float((rows > 6e-2).float().mean())
    assert float(rows.median()) <= 1.5e-2, f"median position: {float(rows.median()):.3g} of the logits' spread"
    assert over <= 0.05, f"{over:.1%} of the positions are off by more than 6% of the logits' spread"


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_the_plain_implementation(name, dtype):
    cfg, w, model, s = build(name, dtype, max_step_tokens=128)
    toks = tokens(70, cfg["vocab"], 1)
    trace_ref = []
    ref = O.forward(w, cfg, toks, trace=trace_ref)
    got = s.feed([("a", toks, list(range(len(toks))))])
    close_logits(got, ref, dtype)
    if dtype == F32:                                       # residual stream after every layer
        meta = s.table.plan([("b", len(toks))])
        tr = []
        model.forward_batch(torch.tensor(toks, dtype=torch.int32, device="cuda"), meta, trace=tr)
        for a, b in zip(tr, trace_ref):
            close(a, b, F32)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("name", ["mixed", "odd", "taps4", "ragged", "tiles"])
def test_decoding_and_portions_equal_the_whole_prompt(name, dtype):
    """Token by token from the first token on; a prompt then 40 single tokens; portions of 2, 3, 1, 7, ... tokens; a step
    longer than the model's step size (cut inside the step function)."""
    cfg, w, model, s = build(name, dtype, max_step_tokens=32)
    toks = tokens(75, cfg["vocab"], 2)
    ref = O.forward(w, cfg, toks)
    schedules = {"single": [1] * len(toks), "prompt+decode": [35] + [1] * 40, "portions": [2, 3, 1, 7, 2, 2, 13, 5, 2, 30, 8],
                 "one step": [len(toks)]}
    for label, cuts in schedules.items():
        assert sum(cuts) == len(toks)
        at, rows = 0, []
        for n in cuts:
            rows.append(s.feed([(label, toks[at:at + n], list(range(n)))]))
            at += n
        s.release(label)
        close_logits(torch.cat(rows), ref, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_mixed_batches_equal_each_request_alone_and_slots_are_reused(dtype):
    """Five requests of unequal length on three slots: prompts in portions next to decoding requests in the same step,
    finished requests give their slot to the next one."""
    cfg, w, model, s = build("mixed", dtype, n_slots=3, max_step_tokens=48)
    lens = [41, 9, 26, 33, 2]
    reqs = {k: tokens(n, cfg["vocab"], 10 + k) for k, n in enumerate(lens)}
    refs = {k: O.forward(w, cfg, t) for k, t in reqs.items()}
    got = {k: [] for k in reqs}
    fed = {k: 0 for k in reqs}
    live, waiting, step = [], list(reqs), 0
    while live or waiting:
        while waiting and len(live) < 3:
            live.append(waiting.pop(0))
        entries = []
        for k in live:
            left = len(reqs[k]) - fed[k]
            n = 1 if fed[k] >= 0.6 * len(reqs[k]) else min(left, [5, 2, 11, 3][(step + k) % 4])
            entries.append((k, reqs[k][fed[k]:fed[k] + n], list(range(n))))
        out = s.feed(entries)
        at = 0
        for k, t, _ in entries:
            got[k].append(out[at:at + len(t)])
            at += len(t)
            fed[k] += len(t)
        for k in [k for k in live if fed[k] == len(reqs[k])]:
            live.remove(k)
            s.release(k)
        step += 1
    assert s.table.pool.free == 3
    for k in reqs:
        close_logits(torch.cat(got[k]), refs[k], dtype)


def test_batch_composition_changes_nothing_in_float32():
    """The same request alone and next to two others: identical kernels per token, so the logits agree to rounding."""
    cfg, w, model, s = build("mixed", F32, n_slots=3, max_step_tokens=64)
    a, b, c = (tokens(n, cfg["vocab"], 20 + n) for n in (17, 30, 5))
    alone = s.feed([("x", a, list(range(len(a))))])
    s.release("x")
    both = s.feed([("p", b, []), ("q", a, list(range(len(a)))), ("r", c, [])])
    assert float((alone - both).abs().max()) <= 1e-4 * logits_scale(alone.double().cpu())


def test_long_decoding_over_many_chunks():
    cfg, w, model, s = build("odd", F32, max_step_tokens=16)
    toks = tokens(150, cfg["vocab"], 3)
    ref = O.forward(w, cfg, toks)
    rows = [s.feed([("a", toks[:10], list(range(10)))])] + [s.feed([("a", [t], [0])]) for t in toks[10:]]
    close_logits(torch.cat(rows), ref, F32)


def test_greedy_generation_through_the_scheduler():
    """More prompts than slots; the continuation of each equals greedy decoding with the plain implementation."""
    cfg, w, model, s = build("mixed", F32, n_slots=2, max_step_tokens=24)
    from qspec_b200.scheduler import Scheduler
    s = Scheduler(model, prefill_portion=7)
    prompts = [tokens(n, cfg["vocab"], 30 + n) for n in (5, 19, 1, 12)]
    outs = s.generate(prompts, max_new_tokens=6)
    assert s.table.pool.free == 2 and not s.has_work()
    for p, o in zip(prompts, outs):
        seq = list(p)
        for t in o:
            lg = O.forward(w, cfg, seq)[-1]
            top2 = lg.topk(2).values
            if float(top2[0] - top2[1]) > 1e-3:                 # no test rests on a near tie
                assert int(lg.argmax()) == t
            seq.append(t)
        assert len(o) == 6


def test_checkpoint_folder_round_trip_through_the_registry(tmp_path):
    _cuda()
    import json
    from qspec_b200 import registry
    from qspec_b200.checkpoint import write_safetensors_file
    from qspec_b200.mutusun import MutusunConfig, random_weights
    from qspec_b200.scheduler import Scheduler
    cfg = CONFIGS["odd"]
    w = random_weights(MutusunConfig.from_dict(cfg), 4)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors_file(str(tmp_path / "model.safetensors"), w)
    model = registry.load_model(str(tmp_path), dtype="float32", n_slots=1, max_step_tokens=32)
    toks = tokens(20, cfg["vocab"], 5)
    ref = O.forward(w, cfg, toks)
    close_logits(Scheduler(model).feed([("a", toks, list(range(20)))]), ref, F32)


# ---------------------------------------------------------------------------------------------------------------------
# tensor-core tile forms (bfloat16, prompt-shaped batches)
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("H,G,D,DV,size", [(4, 2, 64, 64, 50), (2, 1, 128, 64, 200), (2, 2, 64, 128, 33), (1, 1, 128, 128, 64)])
def test_tile_attention_equals_the_token_form(H, G, D, DV, size):
    """Three sequences in one batch: one continues from a cache that ends inside a chunk, one starts at 0 and spans several
    chunks, one is a single decoded token -- tiles see several segments, chunk borders inside a tile and cache rows."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(D + size)
    ld = H * D + G * (D + DV)
    pre = size + size // 3                                   # tokens slot 0 already holds: its chunk began before the step
    lens = [(0, pre, 150), (1, 0, 2 * size + 70), (2, 3 * size - 1, 1)]
    bias = torch.linspace(-2, 0, H).cuda()
    ck = (torch.randn(3, size, G, D, generator=g) * 0.5).to(BF16).cuda()
    cv = torch.randn(3, size, G, DV, generator=g).to(BF16).cuda()
    tab = meta_table([(s, p0, n, 0) for s, p0, n in lens])
    ntok = sum(n for _, _, n in lens)
    qkv = (torch.randn(ntok, ld, generator=g) * 0.5).to(BF16).cuda()
    a = torch.empty(ntok, H * DV, dtype=BF16, device="cuda")
    b = torch.empty_like(a)
    ops.seq_chunk_attention(qkv, ck, cv, bias, a, tab, H, G, D, DV, size, 0.2, 6.0)
    assert ops.seq_chunk_attention_tiles_supported(qkv, H, G, D, DV)
    ops.seq_chunk_attention(qkv, ck, cv, bias, b, tab, H, G, D, DV, size, 0.2, 6.0, tiles=True)
    scale = float(a.float().abs().max())
    assert float((a.float() - b.float()).abs().max()) <= 1e-2 * scale
    assert float((a.float() - b.float()).abs().mean()) <= 2e-3 * scale


@pytest.mark.parametrize("W,F,E,ident,top", [(64, 24, 5, 2, 3), (256, 72, 16, 0, 2), (128, 64, 3, 3, 4)])
def test_grouped_experts_equal_the_token_form(W, F, E, ident, top):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(W + E)
    T = 333
    h = torch.randn(T, W, generator=g).to(BF16).cuda()
    gate_up = (torch.randn(E, 2 * F, W, generator=g) / W ** 0.5).to(BF16).cuda()
    down = (torch.randn(E, W, F, generator=g) / F ** 0.5).to(BF16).cuda()
    idx = torch.stack([torch.randperm(E + ident, generator=g)[:top] for _ in range(T)]).to(torch.int32).cuda()
    idx[:40] = idx[0]                                        # one expert with a run longer than a tile's worth nearby
    a = torch.empty(T, top, W, dtype=BF16, device="cuda")
    b = torch.full_like(a, float("nan"))
    ops.moe_expert_tokens(h, gate_up, down, idx, a, E, F, 1.5)
    assert ops.moe_expert_grouped_supported(h, F)
    ops.moe_expert_grouped(h, gate_up, down, idx, b, E, F, 1.5)
    assert not torch.isnan(b.float()).any()
    scale = float(a.float().abs().max())
    assert float((a.float() - b.float()).abs().max()) <= 2e-2 * scale
    assert float((a.float() - b.float()).abs().mean()) <= 2e-3 * scale
    assert ops.moe_grouped_status() == 0                    # no CTA gave up a wait of its pipeline


CONFIGS["tiles"] = config([dict(mixer=mixer(heads=2, kv=1, dim=64, vdim=64, size=40), mlp=moe(ff=32, experts=4, identity=2, top=2)),
                           dict(mixer=mixer(heads=2, kv=2, dim=64, vdim=128, size=100), mlp={"kind": "dense", "ff": 96})], width=128)


def test_prompts_through_the_tile_kernels_match_the_plain_implementation():
    """bfloat16 prompts long enough for the tile kernels, cut so that portions start inside chunks, next to a decoding
    request; the same model with the tile kernels switched off gives the same logits to bfloat16 rounding."""
    cfg, w, model, s = build("tiles", BF16, n_slots=2, max_step_tokens=256)
    toks = tokens(330, cfg["vocab"], 7)
    other = tokens(40, cfg["vocab"], 8)
    ref, ref_other = O.forward(w, cfg, toks), O.forward(w, cfg, other)
    assert model.use_tiles
    rows, orow, at = [], [s.feed([("o", other[:8], list(range(8)))])], 0
    for k, n in enumerate([130, 97, 103]):
        out = s.feed([("a", toks[at:at + n], list(range(n))), ("o", [other[8 + k]], [0])])
        rows.append(out[:n]); orow.append(out[n:])
        at += n
    close_logits(torch.cat(rows), ref, BF16)
    close_logits(torch.cat(orow), ref_other[:11], BF16)
    model.use_tiles = False
    s.release("a")
    plain = s.feed([("a", toks, list(range(len(toks))))])
    close_logits(plain, ref, BF16)
