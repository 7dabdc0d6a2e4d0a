"""Pitudra on the GPU against the plain CPU restatement (oracle/pitudra_oracle.py): every mechanism alone, then whole
models through the scheduler's step function -- whole prompts, token-by-token decoding, portions down to two tokens,
mixed batches, reused slots, window and ring edges, other sizes, long decoding and greedy generation."""
import json
import math
import os

import pytest
import torch

from oracle import pitudra_oracle as O

pytestmark = pytest.mark.gpu

F32, BF16, F64 = torch.float32, torch.bfloat16, torch.float64


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


def rnd(g, *shape, dtype=F32, scale=1.0):
    """Random values that the element type represents exactly, as float64."""
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(F64)


def tol(dtype):
    return 2e-5 if dtype == F32 else 2.5e-2


def close(got, want, dtype, scale=None):
    want = want.to(F64)
    s = float(want.abs().max()) if scale is None else scale
    err = float((got.detach().cpu().to(F64) - want).abs().max())
    assert err <= tol(dtype) * max(s, 1e-6), f"max error {err:.3g} against scale {s:.3g}"


# ---------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_token_shift_carries_the_last_row_between_portions(dtype):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(1)
    T, W = 21, 70
    x, shift = rnd(g, T, W, scale=2.0), rnd(g, W, scale=0.5)
    want = O.token_shift(x, shift)
    for slot in (0, 2):
        prev = torch.full((2, 3, W), float("nan"), dtype=F32, device="cuda")
        phase, at, got = 0, 0, []
        for n in [1, 2, 1, 6, 2, 9]:
            out = torch.empty(n, W, dtype=dtype, device="cuda")
            ops.seq_token_shift(x[at:at + n].float().cuda(), shift.float().cuda(), prev, out, meta_table([(slot, at, n, phase)]))
            got.append(out.float().cpu())
            at, phase = at + n, phase ^ 1
        close(torch.cat(got), want, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("kind,W,parts", [("layer", 96, 1), ("layer", 257, 3), ("rms", 40, 1), ("rms", 1030, 2)])
def test_residual_sum_with_output_norm(dtype, kind, W, parts):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(W + parts)
    T, eps = 9, 1e-5
    x = rnd(g, T, W, scale=3.0)
    y = (torch.randn(T, parts, W, generator=g) + 0.7).to(dtype).to(F64)      # a mean far from zero: the variance is taken around it
    yw = rnd(g, T, parts).abs()
    w, b = rnd(g, W) + 1.0, rnd(g, W, scale=0.3)
    v = (y * yw[:, :, None]).sum(1)
    want = x + (O.layer_norm(v, w, b, eps) if kind == "layer" else O.rms_norm(v, w, eps))
    xo = x.float().cuda()
    out = torch.empty(T, W, dtype=dtype, device="cuda")
    ya = y.to(dtype).cuda() if parts > 1 else y[:, 0].to(dtype).cuda().contiguous()
    ops.seq_add_norm(ya, w.float().cuda(), b.float().cuda() if kind == "layer" else None, eps, kind=kind, x_in=xo, x_out=xo, out=out,
                     y_w=yw.float().cuda() if parts > 1 else None)
    if parts == 1:
        want = x + (O.layer_norm(y[:, 0] * 1.0, w, b, eps) if kind == "layer" else O.rms_norm(y[:, 0], w, eps))
    close(xo, want, F32)
    close(out, want, dtype)
    # the norm alone, from float32 rows (the form of the model's last norm)
    o2 = torch.empty(T, W, dtype=dtype, device="cuda")
    ops.seq_add_norm(x.float().cuda(), w.float().cuda(), b.float().cuda(), eps, kind="layer", out=o2)
    close(o2, O.layer_norm(x, w, b, eps), dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,rot_dims", [(24, 16, 8, 8), (7, 10, 6, 2), (300, 130, 4, 4)])
def test_latent_norms_rotary_part_and_ring_rows(dtype, q_rank, kv_rank, rot_dim, rot_dims):
    """Rows land at position % cap, far positions rotate by large angles, entries past rot_dims pass unchanged."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(q_rank)
    T, cap, eps, base, p0 = 11, 13, 1e-6, 1000.0, 290        # rows 4 .. 12, 0, 1 of the ring
    d = rnd(g, T, q_rank + kv_rank + rot_dim, dtype=dtype, scale=2.0)
    qw, kw = rnd(g, q_rank) + 1.0, rnd(g, kv_rank) + 1.0
    inv = (torch.tensor(base, dtype=F64) ** (-2.0 * torch.arange(rot_dims // 2, dtype=F64) / rot_dims)).float().cuda()
    cq = torch.empty(T, q_rank, dtype=dtype, device="cuda")
    cache = torch.zeros(2, cap, kv_rank + rot_dim, dtype=dtype, device="cuda")
    ops.seq_latent_prep(d.to(dtype).cuda(), q_rank, kv_rank, rot_dim, qw.float().cuda(), kw.float().cuda(), inv, rot_dims, cq, cache,
                        meta_table([(1, p0, T, 0)]), eps)
    close(cq, O.rms_norm(d[:, :q_rank], qw, eps), dtype)
    pos = torch.arange(p0, p0 + T)
    c = O.rms_norm(d[:, q_rank:q_rank + kv_rank], kw, eps)
    kr = O.rotate(d[:, None, q_rank + kv_rank:], pos, base, rot_dims)[:, 0]
    for t in range(T):
        row = cache[1, (p0 + t) % cap].float().cpu()
        close(row[:kv_rank], c[t], dtype, scale=float(c.abs().max()))
        close(row[kv_rank:], kr[t], dtype, scale=float(kr.abs().max()))
    assert float(cache[0].abs().max()) == 0.0
    # queries: the rotary slice of every head into a float32 buffer
    H, D = 3, 5
    q = rnd(g, T, H, D + rot_dim, dtype=dtype)
    dst = torch.empty(T, H, rot_dim, dtype=F32, device="cuda")
    ops.seq_rotary(q.to(dtype).cuda(), D, dst, rot_dims, inv, meta_table([(0, p0, T, 0)]))
    close(dst, O.rotate(q[..., D:], pos, base, rot_dims), F32 if dtype == F32 else BF16)


def _plain_window_attention(q, k, v, sink, window, scale, G):
    """q [T, H, DK], k [T, G, DK], v [T, G, DV] of one whole sequence -> [T, H, DV] (float64)."""
    H = q.shape[1]
    kk, vv = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    w = O.windowed_sink_softmax(s, sink, window)
    return torch.einsum("hij,jhd->ihd", w, vv)


def _run_window_attention(q, k, v, sink, window, scale, G, cuts, dtype, step_cap, split=None, gate=None, slot=1, p0=0):
    """Feeds the sequence in portions through a ring of window - 1 + step_cap rows, as the model does; returns [T, H, DV]."""
    from qspec_b200 import ops
    T, H, DK = q.shape
    DV = v.shape[2]
    cap = window - 1 + step_cap
    ck = torch.full((3, cap, G, DK), 1e4, dtype=dtype, device="cuda")          # rows of a previous owner must never be read
    cv = torch.full((3, cap, G, DV), 1e4, dtype=dtype, device="cuda")
    at, outs = 0, []
    for n in cuts:
        assert n <= step_cap
        for t in range(at, at + n):
            ck[slot, (p0 + t) % cap] = k[t].to(dtype).cuda()
            cv[slot, (p0 + t) % cap] = v[t].to(dtype).cuda()
        qq = q[at:at + n].float().cuda()
        out = torch.empty(n, H, DV, dtype=dtype, device="cuda")
        qa, qb = (qq, None) if split is None else (qq[..., :split].contiguous(), qq[..., split:].contiguous())
        ops.seq_window_attention(qa, qb, ck, cv, out, meta_table([(slot, p0 + at, n, 0)]), window, scale,
                                 sink=None if sink is None else sink.float().cuda(),
                                 gate=None if gate is None else gate[at:at + n].to(dtype).cuda())
        outs.append(out.float().cpu())
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,G,DK,DV,window,split", [(4, 2, 16, 8, 7, None), (3, 1, 20, 12, 5, 14), (2, 2, 9, 5, 3, None),
                                                     (6, 3, 64, 128, 40, None), (2, 1, 66, 40, 1, 64), (5, 1, 130, 300, 16, 120), (1, 1, 700, 690, 9, 690)])
def test_window_attention_over_portions_and_ring_wraps(dtype, H, G, DK, DV, window, split):
    """Portions that start, end and span ring wraps and window edges; prompt portions and single tokens; the first tokens of a
    sequence (fewer keys than the window); with and without an output gate."""
    _cuda()
    g = torch.Generator().manual_seed(H * 100 + window)
    T, scale = 60, 0.3
    q, k, v = rnd(g, T, H, DK), rnd(g, T, G, DK, dtype=dtype), rnd(g, T, G, DV, dtype=dtype)
    sink = rnd(g, H)
    gate = rnd(g, T, H * DV, dtype=dtype)
    want = _plain_window_attention(q, k, v, sink, window, scale, G)
    for cuts, gt in (([1] * 9 + [2, 5, 8, 1, 1, 7, 3, 8, 8, 8], None), ([8, 8, 8, 2, 1, 1, 8, 8, 8, 8], gate)):
        got = _run_window_attention(q, k, v, sink, window, scale, G, cuts, dtype, 8, split=split, gate=gt)
        w2 = want if gt is None else want * torch.sigmoid(gt.view(T, H, DV))
        close(got, w2, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_far_key_just_inside_and_just_outside_the_window(dtype):
    """One key is made to dominate (score 40 above the rest) and carries a marked value. The query `window - 1` positions
    later must return that value, the next query must not; in a prompt portion and decoded token by token, with the far key
    on either side of a ring wrap."""
    _cuda()
    g = torch.Generator().manual_seed(5)
    H, G, DK, DV, window, scale = 2, 1, 16, 8, 23, 0.5
    for far in (3, 9, 30):
        T = far + window + 3
        q, k, v = rnd(g, T, H, DK, scale=0.1), rnd(g, T, G, DK, dtype=dtype, scale=0.1), rnd(g, T, G, DV, dtype=dtype)
        k[far, 0] = 0.0
        k[far, 0, 0] = 8.0
        q[:, :, 0] = 10.0                                  # every query scores 40 on the far key
        v[far, 0] = 100.0
        sink = torch.zeros(H, dtype=F64)
        want = _plain_window_attention(q, k, v, sink, window, scale, G)
        inside, outside = far + window - 1, far + window
        assert float(want[inside].min()) > 99 and float(want[outside].abs().max()) < 10
        for cuts in ([far + 2] + [window + 1], [far + 1] + [1] * (window + 2), [T]):
            got = _run_window_attention(q, k, v, sink, window, scale, G, cuts, dtype, T)
            close(got, want, dtype)
            assert float(got[inside].min()) > 99 and float(got[outside].abs().max()) < 10


@pytest.mark.parametrize("token_rows", [False, True])
@pytest.mark.parametrize("H,G,DA,DB,DV,window", [(4, 2, 64, 0, 64, 19), (8, 1, 128, 0, 128, 40), (3, 3, 128, 0, 64, 7), (16, 1, 64, 0, 128, 33),
                                                 (2, 2, 128, 64, 128, 25), (5, 5, 128, 64, 128, 1)])
def test_window_attention_on_the_tensor_cores(token_rows, H, G, DA, DB, DV, window):
    """Both row mappings (query heads of a group; 16 consecutive tokens) on batches that mix two sequences: portions that
    end inside a 16-token block, single tokens, ring wraps, the first tokens. With DB > 0 the last DB entries of every key
    come from a part shared by all heads."""
    _cuda()
    from qspec_b200 import ops
    if not ops.seq_window_attention_mma_supported(BF16, DA, DB, DV, H, G, token_rows):
        pytest.skip("shape not taken by this row mapping")
    g = torch.Generator().manual_seed(H + DA + window)
    lens, scale, step_cap = (61, 45), 0.2, 24
    cap = window - 1 + step_cap
    seqs = []
    for n in lens:
        q, k, v = rnd(g, n, H, DA + DB, dtype=BF16), rnd(g, n, G, DA, dtype=BF16), rnd(g, n, G, DV, dtype=BF16)
        ks = rnd(g, n, DB, dtype=BF16) if DB else None
        kfull = k if not DB else torch.cat([k, ks[:, None, :].expand(n, G, DB)], -1)
        seqs.append((q, k, ks, v, kfull))
    sink = rnd(g, H)
    gate = [rnd(g, n, H * DV, dtype=BF16) for n in lens]
    want = [_plain_window_attention(q, kf, v, sink, window, scale, G) * torch.sigmoid(gt.view(n, H, DV))
            for (q, k, ks, v, kf), gt, n in zip(seqs, gate, lens)]
    ck = torch.full((4, cap, G, DA), 1e4, dtype=BF16, device="cuda")
    cs = torch.full((4, cap, max(DB, 8)), 1e4, dtype=BF16, device="cuda")
    cv = torch.full((4, cap, G, DV), 1e4, dtype=BF16, device="cuda")
    slots, at = (3, 1), [0, 0]
    got = [[], []]
    plan = [(20, 5), (1, 1), (24, 23), (3, 0), (13, 16)]
    for step in plan:
        segs, qs, gs = [], [], []
        for b, n in enumerate(step):
            if not n:
                continue
            q, k, ks, v, _ = seqs[b]
            for t in range(at[b], at[b] + n):
                ck[slots[b], t % cap] = k[t].to(BF16).cuda()
                cv[slots[b], t % cap] = v[t].to(BF16).cuda()
                if DB:
                    cs[slots[b], t % cap, :DB] = ks[t].to(BF16).cuda()
            segs.append((slots[b], at[b], n, 0))
            qs.append(q[at[b]:at[b] + n]); gs.append(gate[b][at[b]:at[b] + n])
        ntok = sum(n for n in step)
        out = torch.empty(ntok, H, DV, dtype=BF16, device="cuda")
        ops.seq_window_attention_mma(torch.cat(qs).float().cuda(), ck, cs[:, :, :DB] if DB else None, cv, out, meta_table(segs), window, scale,
                                     token_rows, sink=sink.float().cuda(), gate=torch.cat(gs).to(BF16).cuda())
        o = 0
        for b, n in enumerate(step):
            got[b].append(out[o:o + n].float().cpu())
            o += n
            at[b] += n
    assert at == list(lens)
    for b in range(2):
        close(torch.cat(got[b]), want[b], BF16)


@pytest.mark.parametrize("H,groups,r,R,window,n", [(16, 1, 256, 64, 37, 90), (32, 2, 512, 64, 20, 90), (5, 1, 256, 64, 1, 90),
                                                   (3, 1, 512, 64, 70, 90), (4, 1, 256, 64, 520, 330), (16, 1, 512, 64, 300, 200)])
def test_absorbed_latent_attention_on_the_tensor_cores(H, groups, r, R, window, n):
    """The cache rows are keys and values at once ([latent | shared rotary part], value = the latent); all heads read the same
    rows, 16 heads per CTA. Decoded token by token and in small portions; with a long window and few tokens the blocks of a
    token's keys are shared by a cluster of 2 or 4 CTAs (some of them without a block while the sequence is short)."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(H + r)
    scale, step_cap = 0.05, 8
    cap = window - 1 + step_cap
    q, c = rnd(g, n, H, r + R, dtype=BF16), rnd(g, n, 1, r + R, dtype=BF16)
    sink = rnd(g, H)
    want = _plain_window_attention(q, c, c[..., :r], sink, window, scale, 1)
    cache = torch.full((3, cap, r + R), 1e4, dtype=BF16, device="cuda")
    at, got = 0, []
    cuts, pattern = [], [1] * 40 + [5, 8, 3, 8, 8, 2, 8, 8]
    while sum(cuts) < n:
        cuts.append(min(pattern[len(cuts) % len(pattern)], n - sum(cuts)))
    for k in cuts:
        cache[2, [(t % cap) for t in range(at, at + k)]] = c[at:at + k, 0].to(BF16).cuda()
        out = torch.empty(k, H, r, dtype=BF16, device="cuda")
        ck = cache[:, :, :r].unsqueeze(2).expand(3, cap, groups, r)
        ops.seq_window_attention_mma(q[at:at + k].float().cuda(), ck, cache[:, :, r:], ck, out, meta_table([(2, at, k, 0)]), window, scale,
                                     False, sink=sink.float().cuda())
        got.append(out.float().cpu())
        at += k
    assert at == n
    close(torch.cat(got), want, BF16)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_the_sink_counts_once_unscaled_and_holds_no_value(dtype):
    """A query whose scores are all zero: with sink s and n visible keys every key weighs 1 / (n + e^s)."""
    _cuda()
    H, G, DK, DV, window = 2, 2, 8, 4, 6
    T = 10
    q = torch.zeros(T, H, DK, dtype=F64)
    k = torch.ones(T, G, DK, dtype=F64)
    v = torch.ones(T, G, DV, dtype=F64)
    sink = torch.tensor([math.log(3.0), -50.0], dtype=F64)
    got = _run_window_attention(q, k, v, sink, window, 7.0, G, [4, 1, 5], dtype, 5)
    for t in range(T):
        n = min(t + 1, window)
        close(got[t, 0], torch.full((DV,), n / (n + 3.0), dtype=F64), dtype, scale=1.0)
        close(got[t, 1], torch.ones(DV, dtype=F64), dtype, scale=1.0)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,D,DV", [(2, 16, 24), (1, 33, 7), (3, 130, 40), (2, 64, 64)])
def test_hgrn2_state_over_portions_and_slots(dtype, H, D, DV):
    """The recurrence cut into portions of 1 to 17 tokens (blocks of eight inside the kernel), in a slot whose state is
    NaN before the first token; a second sequence in the same steps must not disturb it."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(D)
    T, eps = 45, 1e-5
    n_in = H * (2 * D + DV)
    proj = rnd(g, T, n_in, dtype=dtype, scale=1.5)
    eye = torch.eye(n_in, dtype=F64)
    sd = {"q": eye[:H * D], "f": eye[H * D:2 * H * D], "v": eye[2 * H * D:], "f.b": rnd(g, H * D), "lower": torch.rand(H * D, generator=g).to(F64),
          "norm": rnd(g, DV) + 1.0, "o": torch.eye(H * DV, dtype=F64)}
    m = {"heads": H, "dim": D, "vdim": DV}
    want = O.hgrn2(proj, sd, "", m, eps)
    other = rnd(g, T, n_in, dtype=dtype)
    want_other = O.hgrn2(other, sd, "", m, eps)
    state = torch.full((3, H, D, DV), float("nan"), dtype=F32, device="cuda")
    scratch = torch.empty(2 * T * H * (DV + 3 * D), dtype=F32, device="cuda")
    at, got, got_other = 0, [], []
    for n in [1, 2, 8, 1, 9, 17, 7]:
        rows = torch.cat([proj[at:at + n], other[at:at + n]]).to(dtype).cuda()
        out = torch.empty(2 * n, H * DV, dtype=dtype, device="cuda")
        starts = torch.tensor([0, n], dtype=torch.int32, device="cuda") if n % 2 else None      # both grid forms
        ops.seq_hgrn2(rows, sd["f.b"].float().cuda(), sd["lower"].float().cuda(), sd["norm"].float().cuda(), state, scratch, out,
                      meta_table([(2, at, n, 0), (0, at, n, 0)]), H, D, DV, eps, seg_starts=starts)
        got.append(out[:n].float().cpu()); got_other.append(out[n:].float().cpu())
        at += n
    close(torch.cat(got), want, dtype)
    close(torch.cat(got_other), want_other, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("W,F,E,top", [(64, 24, 5, 3), (72, 10, 3, 1), (128, 64, 9, 9)])
def test_router_over_chosen_logits_and_squared_relu_experts(dtype, W, F, E, top):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(W + E)
    T = 50
    x = rnd(g, T, W, dtype=dtype)
    sd = {"router": rnd(g, E, W, scale=0.3)}
    for e in range(E):
        sd[f"e{e}.up"], sd[f"e{e}.down"] = rnd(g, F, W, dtype=dtype, scale=W ** -0.5), rnd(g, W, F, dtype=dtype, scale=F ** -0.5)
    want = O.moe(x, sd, "", {"router": {"experts": E, "top": top}})
    h = x.to(dtype).cuda()
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    rw = torch.empty(T, top, dtype=F32, device="cuda")
    ops.moe_route_chosen(h, sd["router"].float().cuda(), idx, rw)
    z = x @ sd["router"].T
    val, ref_idx = torch.topk(z, top, dim=-1)
    assert torch.equal(idx.cpu().long().sort(-1).values, ref_idx.sort(-1).values)
    close(rw.sum(-1), torch.ones(T, dtype=F64), F32)
    up = torch.stack([sd[f"e{e}.up"] for e in range(E)]).to(dtype).cuda()
    down = torch.stack([sd[f"e{e}.down"] for e in range(E)]).to(dtype).cuda()
    forms = ["tokens"] + (["grouped"] if dtype == BF16 and ops.moe_expert_grouped_supported(h, F) else [])
    for form in forms:
        pair = torch.empty(T, top, W, dtype=dtype, device="cuda")
        (ops.moe_expert_tokens if form == "tokens" else ops.moe_expert_grouped)(h, up, down, idx, pair, E, F, 0.0, act="relu2")
        got = (pair.float() * rw[:, :, None]).sum(1)
        close(got, want, dtype)
    if "grouped" in forms:
        assert ops.moe_grouped_status() == 0


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_token_side_input(dtype):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, W, sd_, L, V, layer, eps = 13, 48, 10, 3, 29, 1, 1e-6
    x = rnd(g, T, W, scale=2.0)
    toks = torch.randint(0, V, (T,), generator=g)
    sd = {"side.embed": rnd(g, V, L * sd_, dtype=dtype), "side.gate": rnd(g, sd_, W, dtype=dtype, scale=0.3), "side.proj": rnd(g, W, sd_, dtype=dtype),
          "side.norm": rnd(g, W) + 1.0}
    want = x + O.token_side(x, toks, sd, "", layer, sd_, eps)
    gate = (x @ sd["side.gate"].T).to(dtype).cuda()
    ops.seq_side_gate(gate, sd["side.embed"].to(dtype).cuda(), toks.to(torch.int32).cuda(), layer * sd_)
    ref_g = O.gelu_tanh(x @ sd["side.gate"].T) * sd["side.embed"][toks][:, layer * sd_:(layer + 1) * sd_]
    close(gate, ref_g, dtype)
    y = (gate.float().cpu().to(F64) @ sd["side.proj"].T).to(dtype).cuda()
    xo = x.float().cuda()
    ops.seq_add_norm(y, sd["side.norm"].float().cuda(), None, eps, kind="rms", x_in=xo, x_out=xo)
    close(xo, want, dtype)


# ---------------------------------------------------------------------------------------------------------------------
# whole models through the scheduler
# ---------------------------------------------------------------------------------------------------------------------
def latent(heads=2, dim=8, vdim=12, rot_dim=4, rot_dims=None, q_rank=20, kv_rank=10, window=9, scale=0.3, base=500.0, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "rot_dim": rot_dim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def attention(heads=4, kv=2, dim=8, vdim=6, window=7, scale=0.35):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}}


def recurrent(heads=2, dim=12, vdim=10):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def moe(ff=24, experts=4, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, width=64, vocab=97, eps=1e-5, side=6):
    out = {"architecture": "Pitudra", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [dict(l, mlp=l.get("mlp")) for l in layers]}
    if side:
        out["token_side"] = {"dim": side}
    return out


CONFIGS = {
    # every mixer; the borrowed cache is read through a wider window than its owner's
    "mixed": config([dict(latent(), mlp=moe()), dict(latent(window=13, kv_from=0, heads=3, dim=6, vdim=5), mlp=moe()),
                     dict(recurrent(), mlp=moe()), dict(attention(), mlp=moe()), dict(latent(window=4, kv_from=0), mlp=None)]),
    # nothing divisible by anything, one head, top 1, a window of one, rotated part smaller than the rotary slice, no side input
    "odd": config([dict(attention(heads=3, kv=1, dim=9, vdim=5, window=1), mlp=moe(ff=10, experts=3, top=1)),
                   dict(recurrent(heads=1, dim=33, vdim=7), mlp=None),
                   dict(latent(heads=1, dim=6, vdim=6, rot_dim=6, rot_dims=2, q_rank=7, kv_rank=9, window=3, base=37.0), mlp=moe(ff=7, experts=2, top=2)),
                   dict(attention(heads=2, kv=2, dim=10, vdim=10, window=40), mlp=None)],
                  width=50, vocab=33, eps=1e-6, side=0),
    # windows longer than anything the tests feed; every expert chosen; sizes that take the grouped experts in bfloat16
    "wide": config([dict(recurrent(heads=4, dim=16, vdim=16), mlp=moe(ff=32, experts=2, top=2)),
                    dict(latent(heads=4, dim=16, vdim=16, rot_dim=8, q_rank=32, kv_rank=24, window=500), mlp=moe(ff=32, experts=2, top=2)),
                    dict(attention(heads=4, kv=4, dim=16, vdim=16, window=300), mlp=moe(ff=32, experts=2, top=2))], width=64, side=3),
    # a latent cache wide enough for the tensor-core absorbed form in bfloat16 decoding; the borrowing layer has other heads
    "latent256": config([dict(latent(heads=2, dim=8, vdim=8, rot_dim=64, q_rank=16, kv_rank=256, window=11, scale=0.1), mlp=moe()),
                         dict(latent(heads=3, dim=16, vdim=4, rot_dim=64, q_rank=8, kv_rank=256, window=30, scale=0.1, kv_from=0), mlp=None)],
                        width=48, side=0),
    # head sizes that the tensor-core attention forms take in bfloat16 (prompts of a latent layer run in the expanded form)
    "tiles": config([dict(latent(heads=2, dim=128, vdim=128, rot_dim=64, q_rank=24, kv_rank=32, window=21, scale=0.08), mlp=moe()),
                     dict(attention(heads=4, kv=2, dim=64, vdim=64, window=30, scale=0.12), mlp=moe()),
                     dict(latent(heads=2, dim=128, vdim=128, rot_dim=64, q_rank=24, kv_rank=32, window=70, scale=0.08, kv_from=0), mlp=None),
                     dict(attention(heads=2, kv=1, dim=128, vdim=128, window=9, scale=0.09), mlp=None)], width=64, side=4),
}


def build(name, dtype, seed=0, n_slots=3, max_step_tokens=64):
    _cuda()
    from qspec_b200.pitudra import PitudraConfig, PitudraModel, random_weights
    from qspec_b200.scheduler import Scheduler
    cfg = PitudraConfig.from_dict(CONFIGS[name])
    w = random_weights(cfg, seed)
    model = PitudraModel(cfg, w, dtype=dtype, device="cuda", n_slots=n_slots, max_step_tokens=max_step_tokens)
    return CONFIGS[name], w, model, Scheduler(model)


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def close_logits(got, ref, dtype):
    """Per position: root mean square over the vocabulary of the difference (mean taken off), relative to the spread of
    the logits. float32 must sit at rounding level; bfloat16 within what its 8-bit mantissa leaves after a few layers."""
    ref = ref.to(F64)
    d = got.detach().cpu().to(F64) - ref
    d = d - d.mean(-1, keepdim=True)
    spread = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    rows = d.pow(2).mean(-1).sqrt() / spread
    if dtype == F32:
        assert float(rows.max()) <= 1e-5, f"worst position: {float(rows.max()):.3g} of the logits' spread"
        return
    # bfloat16: the norms sit on the sublayers' outputs, so rounding of a small output is scaled up with it, and with random
    # weights a router choice can flip on a near tie (with one expert per token that replaces the whole feed-forward
    # output); the typical position must sit at rounding level and few may be far off
    over = float((rows > 0.1).float().mean())
    assert float(rows.median()) <= 2.5e-2, f"median position: {float(rows.median()):.3g} of the logits' spread"
    assert over <= 0.1, f"{over:.1%} of the positions are off by more than 10% of the logits' spread"


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_the_plain_implementation(name, dtype):
    cfg, w, model, s = build(name, dtype, max_step_tokens=128)
    toks = tokens(70, cfg["vocab"], 1)
    lay = []
    ref = O.forward(cfg, w, toks, lay)
    got = s.feed([("a", toks, list(range(len(toks))))])
    close_logits(got, ref, dtype)
    if dtype == F32:                                       # residual stream after every layer
        meta = s.table.plan([("b", len(toks))])
        tr = []
        model.forward_batch(torch.tensor(toks, dtype=torch.int32, device="cuda"), meta, trace=tr)
        for a, b in zip(tr, lay):
            close(a, b, F32)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_decoding_and_portions_equal_the_whole_prompt(name, dtype):
    """Token by token from the first token on; a prompt then 40 single tokens; portions of 2, 3, 1, 7, ... tokens; a step
    longer than the model's step size (cut inside the step function). The ring caches hold window - 1 + 16 rows here, so
    the longer windows wrap several times."""
    cfg, w, model, s = build(name, dtype, max_step_tokens=16)
    toks = tokens(75, cfg["vocab"], 2)
    ref = O.forward(cfg, w, toks)
    schedules = {"single": [1] * len(toks), "prompt+decode": [16, 16, 3] + [1] * 40, "portions": [2, 3, 1, 7, 2, 2, 13, 5, 2, 16, 14, 8],
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
    """Five unequal requests on three slots: prompt portions next to single tokens in one step, requests that end while
    others go on, and slots taken over by later requests without being cleared."""
    cfg, w, model, s = build("mixed", dtype, n_slots=3, max_step_tokens=32)
    lens = {"a": 31, "b": 9, "c": 22, "d": 17, "e": 40}
    toks = {r: tokens(n, cfg["vocab"], 10 + k) for k, (r, n) in enumerate(lens.items())}
    if dtype == F32:
        ref = {r: O.forward(cfg, w, t) for r, t in toks.items()}
    else:
        # bfloat16: a router choice that flips against the float64 reference is carried on by the recurrence and the windows
        # for many positions, alone or in a batch alike; what a batch must not change is the request's own bfloat16 result
        ref = {}
        for r, t in toks.items():
            ref[r] = s.feed([(("alone", r), t, list(range(len(t))))]).float().cpu()
            s.release(("alone", r))
    fed = {r: 0 for r in toks}
    got = {r: [] for r in toks}
    plan = [{"a": 12, "b": 2}, {"a": 1, "b": 7, "c": 5}, {"a": 18, "c": 1}, {"c": 16, "d": 3}, {"d": 14, "e": 2}, {"e": 30, "d": 0}, {"e": 8}]
    live = set()
    for step in plan:
        entries = []
        for r, n in step.items():
            if n:
                entries.append((r, toks[r][fed[r]:fed[r] + n], list(range(n))))
                live.add(r)
        out = s.feed(entries)
        at = 0
        for r, t, _ in entries:
            got[r].append(out[at:at + len(t)])
            at += len(t)
            fed[r] += len(t)
            if fed[r] == lens[r]:
                s.release(r)
                live.discard(r)
    assert fed == lens and not live
    for r in toks:
        close_logits(torch.cat(got[r]), ref[r], dtype)


def test_prompt_and_decode_forms_on_the_tensor_cores_match_the_plain_implementation():
    """bfloat16 steps of 64 tokens and more take the 16-token form (and the expanded latent form), shorter ones the
    head-row form; both against the plain implementation, with a portion that continues a sequence."""
    cfg, w, model, s = build("tiles", BF16, max_step_tokens=128)
    toks = tokens(150, cfg["vocab"], 3)
    ref = O.forward(cfg, w, toks)
    rows = [s.feed([("a", toks[:70], list(range(70)))]), s.feed([("a", toks[70:75], list(range(5)))]),
            s.feed([("a", toks[75:], list(range(75)))])]
    close_logits(torch.cat(rows), ref, BF16)
    s.release("a")
    rows = [s.feed([("b", toks[:40], list(range(40)))])] + [s.feed([("b", [t], [0])]) for t in toks[40:90]]
    close_logits(torch.cat(rows), ref[:90], BF16)


def test_windows_longer_than_any_sequence_take_rings_of_the_sequence_limit():
    """A window of ten million positions: with a sequence limit the rings hold that many rows (positions never wrap) and the
    scheduler refuses a longer sequence; the logits are those of the plain implementation."""
    _cuda()
    from qspec_b200.pitudra import PitudraConfig, PitudraModel, random_weights
    from qspec_b200.scheduler import Scheduler
    cfg = config([dict(latent(window=10 ** 7), mlp=moe()), dict(attention(window=10 ** 7), mlp=None), dict(latent(window=5, kv_from=0), mlp=None)])
    w = random_weights(PitudraConfig.from_dict(cfg), 2)
    model = PitudraModel(PitudraConfig.from_dict(cfg), w, dtype=F32, device="cuda", n_slots=2, max_step_tokens=16, max_seq_tokens=90)
    assert model.latent_cache[0].shape[1] == 90 and model.cache_k[1].shape[1] == 90 and model.max_seq_len == 90
    s = Scheduler(model)
    toks = tokens(90, cfg["vocab"], 4)
    rows = [s.feed([("a", toks[:50], list(range(50)))])] + [s.feed([("a", [t], [0])]) for t in toks[50:]]
    close_logits(torch.cat(rows), O.forward(cfg, w, toks), F32)
    with pytest.raises(RuntimeError):
        s.feed([("a", [1], [0])])


def test_batch_composition_changes_nothing_in_float32():
    cfg, w, model, s = build("mixed", F32, n_slots=3, max_step_tokens=64)
    a, b = tokens(30, cfg["vocab"], 5), tokens(12, cfg["vocab"], 6)
    alone = s.feed([("x", a, list(range(30)))]).clone()
    s.release("x")
    s.feed([("y", b[:5], [])])
    both = s.feed([("y", b[5:], []), ("x", a, list(range(30)))]).clone()
    # identical kernels per token; only the vendor library's products may sum in another order for another row count
    spread = float((alone - alone.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    assert float((alone - both).abs().max()) <= 1e-4 * spread


def test_long_decoding_wraps_the_rings_many_times():
    cfg, w, model, s = build("mixed", F32, max_step_tokens=4)          # rings of window + 3 rows: 16, 12 and 10
    toks = tokens(170, cfg["vocab"], 7)
    ref = O.forward(cfg, w, toks)
    rows = [s.feed([("a", toks[:3], [0, 1, 2])])]
    for t in toks[3:]:
        rows.append(s.feed([("a", [t], [0])]))
    close_logits(torch.cat(rows), ref, F32)


def test_greedy_generation_through_the_scheduler():
    cfg, w, model, s = build("mixed", F32, n_slots=2, max_step_tokens=16)
    prompts = [tokens(n, cfg["vocab"], 20 + n) for n in (5, 19, 2, 11)]
    outs = s.generate(prompts, 6)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for _ in range(6):
            seq.append(int(O.forward(cfg, w, seq)[-1].argmax()))
        assert o == seq[len(p):]


def test_checkpoint_folder_through_the_registry_and_the_trace_replay(tmp_path):
    _cuda()
    from qspec_b200 import registry
    from qspec_b200.checkpoint import write_safetensors_file
    from qspec_b200.pitudra import PitudraConfig, random_weights
    from qspec_b200.scheduler import Scheduler
    cfg = CONFIGS["odd"]
    w = random_weights(PitudraConfig.from_dict(cfg), 4)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors_file(str(tmp_path / "model.safetensors"), w)
    model = registry.load_model(str(tmp_path), dtype="float32", n_slots=2, max_step_tokens=32)
    assert model.architecture == "Pitudra"
    toks = tokens(20, cfg["vocab"], 9)
    close_logits(Scheduler(model).feed([("a", toks, [0, 7, 19])]), O.forward(cfg, w, toks)[[0, 7, 19]], F32)
    # the replay program: two steps of one request, logits of the last token of each
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:13], "want": [12]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": toks[13:], "want": [0, 6]}], "end": ["r"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out)],
                       input="\n".join(json.dumps(x) for x in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1"]
    ref = O.forward(cfg, w, toks)
    close_logits(torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(1, -1)), ref[[12]], F32)
    close_logits(torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1)), ref[[13, 19]], F32)
