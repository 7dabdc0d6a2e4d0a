"""`bench.py --design mutusun` and `--design pitudra` (the second half of this file): prefill and decode throughput of the Mutusun design at sizes that resemble a real model's
layers (random weights), next to the framework's int4 Llama decoder at equal width / heads / feed-forward size, both
through the same scheduler; plus the design's kernels one by one against their roofline and against the like kernel of
the int4 decoder. Prints one JSON line. The default workload of bench.py is untouched by this option.
"""
from __future__ import annotations

import json
import os
import time

SIZES = {
    # width, heads, kv, dim, chunk, dense ff, (experts, expert ff, identity, top)
    "w2048": dict(width=2048, heads=16, kv=4, dim=128, chunk=1024, ff=7168, moe=(16, 1024, 2, 4)),
    "w4096": dict(width=4096, heads=32, kv=8, dim=128, chunk=2048, ff=14336, moe=(8, 2048, 1, 2)),
}
VOCAB = 32000


def mutusun_config(s):
    mixer = {"heads": s["heads"], "kv_heads": s["kv"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5, "softcap": 30.0,
             "mask": {"size": s["chunk"]}}
    E, F, ident, top = s["moe"]
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": F, "limit": 7.0}, "router": {"experts": E, "identity": ident, "top": top}}
    layers = [{"type": "attention", "mixer": mixer, "mlp": dense}, {"type": "attention", "mixer": mixer, "mlp": moe},
              {"type": "attention", "mixer": mixer, "mlp": dense, "weights_of": 0}, {"type": "attention", "mixer": mixer, "mlp": moe, "weights_of": 1}]
    return {"architecture": "Mutusun", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "layers": layers}


def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _throughput(torch, sched, vocab, n_seqs, ctx, prompt, portion, steps, warmup):
    """Prefill: one request of `prompt` tokens in portions. Decode: n_seqs requests with `ctx` tokens each, one token per
    sequence per step through Scheduler.step (greedy sampling, tokens read back every step)."""
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, vocab, (prompt,), generator=g).tolist()
    for rep in range(2):                                   # first pass warms up
        torch.cuda.synchronize()
        a, b = _events(torch)
        a.record()
        at = 0
        while at < prompt:
            n = min(portion, prompt - at)
            sched.feed([("p", toks[at:at + n], [n - 1] if at + n == prompt else [])])
            at += n
        b.record(); b.synchronize()
        sched.release("p")
        prefill_ms = a.elapsed_time(b)
    for k in range(n_seqs):
        # long enough that no request finishes inside the timed steps: the batch stays at n_seqs tokens (a changing token
        # count sends every dense product through the vendor library's heuristics again, which is not the steady state)
        sched.add(("d", k), torch.randint(0, vocab, (ctx,), generator=g).tolist(), max_new_tokens=warmup + steps + 4 * n_seqs)
    while any(r.fed < len(r.prompt) for r in list(sched.waiting) + sched.running):
        sched.step()
    for _ in range(warmup):
        sched.step()
    torch.cuda.synchronize()
    a, b = _events(torch)
    t0 = time.perf_counter()
    a.record()
    n = 0
    for _ in range(steps):
        n += len(sched.step())
    b.record(); b.synchronize()
    wall = time.perf_counter() - t0
    for r in list(sched.running):                          # retire the requests without decoding them to the end
        sched.running.remove(r)
        sched.release(r.rid)
    return {"prefill_tokens_per_s": prompt / (prefill_ms / 1e3), "prefill_ms": prefill_ms, "prefill_tokens": prompt, "portion": portion,
            "decode_tokens_per_s": n / (a.elapsed_time(b) / 1e3), "decode_ms_per_step": a.elapsed_time(b) / steps,
            "decode_e2e_tokens_per_s": n / wall, "decode_seqs": n_seqs, "context": ctx}


def _time_us(torch, fns, reps=20):
    """Mean microseconds per call over `fns` called round robin (callers pass variants on distinct buffers that together
    exceed the L2 where the kernel is meant to stream from HBM)."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    a, b = _events(torch)
    a.record()
    for r in range(reps):
        fns[r % len(fns)]()
    b.record(); b.synchronize()
    return a.elapsed_time(b) * 1e3 / reps


def _kernel_table(torch, s, hbm_gbs, bf16_tflops):
    """Each Mutusun kernel at a prompt shape (T = 2048, one sequence) and a decode shape (64 sequences x 1 token), with the
    like kernel of the int4 decoder at its own operating shapes. frac = achieved / measured peak of the binding resource."""
    from . import ops
    dev = "cuda"
    W, H, G, D, size = s["width"], s["heads"], s["kv"], s["dim"], s["chunk"]
    E, F, ident, top = s["moe"]
    ld = H * D + 2 * G * D
    bf, f32 = torch.bfloat16, torch.float32
    rows = []

    def meta(segs):
        r = [[], [], [], [], []]
        at = 0
        for slot, p0, n in segs:
            r[0] += [slot] * n; r[1] += list(range(p0, p0 + n)); r[2] += [at] * n; r[3] += [at + n] * n; r[4] += [0] * n
            at += n
        return torch.tensor(r, dtype=torch.int32, device=dev)

    def add(name, shape, us, nbytes=None, flops=None, like=None):
        e = {"kernel": name, "shape": shape, "us": round(us, 2)}
        if nbytes is not None:
            e["GBps"] = round(nbytes / us / 1e3, 1); e["frac_hbm"] = round(nbytes / us / 1e3 / hbm_gbs, 3)
        if flops is not None:
            e["TFLOPs"] = round(flops / us / 1e6, 1); e["frac_bf16"] = round(flops / us / 1e6 / bf16_tflops, 3)
        if like:
            e["like"] = like
        rows.append(e)

    shapes = {"prompt": [(0, 0, 2048)], "decode": [(k, size // 2 + k, 1) for k in range(64)]}
    nslots = 64
    copies = 3
    ck = [torch.randn(nslots, size, G, D, device=dev).to(bf) for _ in range(copies)]
    cv = [torch.randn(nslots, size, G, D, device=dev).to(bf) for _ in range(copies)]
    pb = torch.zeros(H, device=dev)
    for label, segs in shapes.items():
        T = sum(n for _, _, n in segs)
        tab = meta(segs)
        nbuf = max(2, min(8, int(200e6 / (T * W * 12)) + 1))
        x = [torch.randn(T, W, device=dev) for _ in range(nbuf)]
        xo = [torch.empty(T, W, device=dev) for _ in range(nbuf)]
        y = [torch.randn(T, W, device=dev).to(bf) for _ in range(nbuf)]
        h = [torch.empty(T, W, device=dev, dtype=bf) for _ in range(nbuf)]
        w1, w2 = torch.zeros(W, device=dev), torch.zeros(W, device=dev)
        cw = torch.randn(W, 4, device=dev) * 0.1
        tail = torch.zeros(2, nslots, 3, W, device=dev)
        scr = torch.empty(T * W, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_norm_conv(x[i], tab, 1e-5, out=h[i], pre_w=w1, conv_w=cw, tail=tail, y=y[i], post_w=w2,
                                                            x_out=xo[i], scratch=scr) for i in range(nbuf)])
        add("seq_norm_conv (residual + 2 norms + conv)", f"{label} T={T} W={W}", us, nbytes=T * W * 12)
        qkv = [(torch.randn(T, ld, device=dev) * 0.3).to(bf) for _ in range(nbuf)]
        qn = torch.ones(D, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_qk_norm(qkv[i], qn, qn, H, G, D, 1e-5) for i in range(nbuf)])
        add("seq_qk_norm", f"{label} T={T}", us, nbytes=T * (H + G) * D * 4)
        us = _time_us(torch, [lambda i=i: ops.seq_cache_append(qkv[i], ck[i % copies], cv[i % copies], tab, H, G, D, D, size) for i in range(nbuf)])
        add("seq_cache_append", f"{label} T={T}", us, nbytes=T * 2 * G * D * 4)
        att = torch.empty(T, H * D, device=dev, dtype=bf)
        if label == "prompt":
            us = _time_us(torch, [lambda i=i: ops.seq_chunk_attention(qkv[i], ck[0], cv[0], pb, att, tab, H, G, D, D, size, D ** -0.5, 30.0,
                                                                      tiles=True) for i in range(nbuf)])
            visible = sum((p % size) + 1 for p in range(T))
            add("seq_chunk_attention (tiles)", f"T={T} chunk={size} H={H} G={G} D={D}", us, flops=2.0 * visible * H * 2 * D)
            rows[-1]["note"] = ("algorithmic flops of the visible (query, key) pairs; the kernel issues the P.V product twice "
                                "(two-term bfloat16 split of the float32 weights) and computes whole 64x64 tiles on the diagonal")
        else:
            us = _time_us(torch, [lambda i=i: ops.seq_chunk_attention(qkv[i % nbuf], ck[i % copies], cv[i % copies], pb, att, tab, H, G, D, D,
                                                                      size, D ** -0.5, 30.0, max_keys=max(p for _, p, _ in segs) + 1)
                                  for i in range(copies)])
            visible = sum((p % size) + 1 for _, p, _ in segs)
            add("seq_chunk_attention (token form)", f"64 seqs x 1, {visible // 64} keys each", us, nbytes=visible * G * 2 * D * 2)
        hb = [torch.randn(T, W, device=dev).to(bf) for _ in range(nbuf)]
        rw = torch.randn(E + ident, W, device=dev) * 0.05
        corr = torch.zeros(E + ident, device=dev)
        idx = torch.empty(T, top, dtype=torch.int32, device=dev)
        wt = torch.empty(T, top, device=dev)
        us = _time_us(torch, [lambda i=i: ops.moe_route(hb[i], rw, corr, idx, wt) for i in range(nbuf)])
        add("moe_route", f"{label} T={T} R={E + ident}", us, nbytes=T * W * 2)
        gu = [(torch.randn(E, 2 * F, W, device=dev) * W ** -0.5).to(bf) for _ in range(2)]
        dn = [(torch.randn(E, W, F, device=dev) * F ** -0.5).to(bf) for _ in range(2)]
        pair = torch.empty(T, top, W, device=dev, dtype=bf)
        real = int((idx < E).sum())
        if label == "prompt":
            us = _time_us(torch, [lambda i=i: ops.moe_expert_grouped(hb[i % nbuf], gu[i % 2], dn[i % 2], idx, pair, E, F, 7.0) for i in range(2)])
            add("moe_expert_grouped (sort + 2 tile GEMMs)", f"T={T} top={top} E={E} F={F}", us, flops=2.0 * real * 3 * W * F)
        else:
            us = _time_us(torch, [lambda i=i: ops.moe_expert_tokens(hb[i % nbuf], gu[i % 2], dn[i % 2], idx, pair, E, F, 7.0) for i in range(2)])
            touched = len(set(idx[idx < E].tolist()))
            add("moe_expert_tokens", f"T={T} top={top}, {touched} of {E} experts touched", us, nbytes=touched * 3 * W * F * 2)
            rows[-1]["note"] = ("bytes = the touched experts' weights once (each (token, choice) CTA re-reads its expert from L2); "
                                "the model takes this form only below 4 rows per expert")
            us = _time_us(torch, [lambda i=i: ops.moe_expert_grouped(hb[i % nbuf], gu[i % 2], dn[i % 2], idx, pair, E, F, 7.0) for i in range(2)])
            add("moe_expert_grouped (sort + 2 tile GEMMs)", f"T={T} top={top}, {touched} of {E} experts touched", us,
                nbytes=touched * 3 * W * F * 2)
        # vendor products, for scale
        wq = (torch.randn(ld, W, device=dev) * 0.02).to(bf)
        o = torch.empty(T, ld, device=dev, dtype=bf)
        us = _time_us(torch, [lambda i=i: torch.matmul(hb[i], wq.t(), out=o) for i in range(nbuf)])
        add("qkv product (vendor library)", f"{label} {T}x{ld}x{W}", us, nbytes=(ld * W + T * W + T * ld) * 2, flops=2.0 * T * ld * W)
        del x, xo, y, h, qkv, hb, gu, dn, pair
    return rows


def _like_kernels(torch, s, hbm_gbs, bf16_tflops):
    """The int4 decoder's kernels of the same roles at its operating shapes (verify pass: 64 sequences x 4 tokens)."""
    from . import ops
    from .model import random_int4_linear
    dev, f16 = "cuda", torch.float16
    W, H, G, D = s["width"], s["heads"], s["kv"], s["dim"]
    rows = []

    def add(name, shape, us, nbytes=None, flops=None):
        e = {"kernel": name, "shape": shape, "us": round(us, 2)}
        if nbytes is not None:
            e["GBps"] = round(nbytes / us / 1e3, 1); e["frac_hbm"] = round(nbytes / us / 1e3 / hbm_gbs, 3)
        if flops is not None:
            e["TFLOPs"] = round(flops / us / 1e6, 1); e["frac_bf16"] = round(flops / us / 1e6 / bf16_tflops, 3)
        rows.append(e)

    for T in (256, 64):
        nbuf = 8
        x = [torch.randn(T, W, device=dev).to(f16) for _ in range(nbuf)]
        dl = [torch.randn(T, W, device=dev).to(f16) for _ in range(nbuf)]
        out = torch.empty(T, W, device=dev, dtype=f16)
        us = _time_us(torch, [lambda i=i: ops.add_rms_norm_fuse_sum_fp16(out, x[i], dl[i], 1e-5) for i in range(nbuf)])
        add("add + norm (f16)", f"T={T} W={W}", us, nbytes=T * W * 8)
    S, B = 1024, 64
    ck = torch.randn(B, S, G, D, device=dev).to(f16)
    cv = torch.randn(B, S, G, D, device=dev).to(f16)
    for per in (4, 1):
        T = B * per
        qkv = (torch.randn(T, (H + 2 * G) * D, device=dev) * 0.3).to(f16)
        pos = (torch.arange(T, device=dev, dtype=torch.int32) % per) + 512
        sid = (torch.arange(T, device=dev, dtype=torch.int32) // per).contiguous()
        att = torch.empty(T, H * D, device=dev, dtype=f16)
        cs = torch.randn(S, D, device=dev).to(f16)
        us = _time_us(torch, [lambda: ops.rope_kvcache(qkv, cs, pos, sid, ck, cv, H, G, D)])
        add("rope + cache append", f"T={T}", us, nbytes=T * ((H + G) * D * 4 + 2 * G * D * 2))
        if ops.seq_attention_supported(T, H, G, D, S):
            us = _time_us(torch, [lambda: ops.seq_attention(qkv, ck, cv, pos, sid, att, H, G, D, D ** -0.5)])
            add("seq_attention", f"64 seqs x {per}, 512 keys", us, nbytes=B * 513 * G * 2 * D * 2)
        us = _time_us(torch, [lambda: ops.decode_attention(qkv, ck, cv, pos, sid, att, H, G, D, D ** -0.5)])
        add("decode_attention", f"64 seqs x {per}, 512 keys", us, nbytes=B * 513 * G * 2 * D * 2)
    ops.reserve_workspaces(256, [(s["ff"] * 2, W)], torch.device(dev))
    lins = [random_int4_linear(2 * s["ff"], W, 100 + i, dev) for i in range(3)]
    for T in (256, 64):
        xin = torch.randn(T, W, device=dev).to(f16)
        o = torch.empty(T, 2 * s["ff"], device=dev, dtype=f16)
        us = _time_us(torch, [lambda l=l: l(xin, o) for l in lins])
        add("W4A16 gate_up product", f"{T}x{2 * s['ff']}x{W}", us, nbytes=s["ff"] * W + T * W * 2 + T * 2 * s["ff"] * 2, flops=2.0 * T * 2 * s["ff"] * W)
    return rows


def run(args, peaks, clock_sampler_cls) -> dict:
    import torch
    from . import ops
    from .build import build_library
    from .model import QSpecLlamaConfig, QSpecLlamaModel
    from .mutusun import MutusunConfig, MutusunModel, random_weights
    from .scheduler import Scheduler
    build_library()
    torch.cuda.set_device(0)
    hbm_gbs, bf16_tflops, peak_src = peaks
    bf16_tflops = bf16_tflops or 1590.0
    names = [n for n in (args.sizes.split(",") if args.sizes else SIZES) if n in SIZES]
    steps, warmup = args.steps, max(3, args.warmup)
    out = {}
    sampler = clock_sampler_cls(0)
    sampler.start()
    l0 = ops.seq_launch_count()
    for name in names:
        s = SIZES[name]
        res = {"layers": 4, "sizes": s}
        cfgd = mutusun_config(s)
        cfg = MutusunConfig.from_dict(cfgd)
        model = MutusunModel(cfg, random_weights(cfg, 0), dtype=torch.bfloat16, device="cuda", n_slots=65, max_step_tokens=2048)
        res["mutusun"] = {p: _throughput(torch, Scheduler(model, prefill_portion=p), VOCAB, 64, 300, 4096, p, steps, warmup) for p in (2048, 256)}
        res["mutusun"]["state_bytes_per_sequence"] = model.state_bytes_per_slot()
        del model
        torch.cuda.empty_cache()
        lc = QSpecLlamaConfig.llama3_8b(hidden_size=s["width"], intermediate_size=s["ff"], num_attention_heads=s["heads"],
                                        num_key_value_heads=s["kv"], head_dim=s["dim"], num_hidden_layers=4, vocab_size=VOCAB,
                                        max_seq_len=4096 + 8, name=f"int4-llama-{name}")
        llama = QSpecLlamaModel(lc, max_batch=65, max_tokens=256, device="cuda")
        res["int4_llama_w4a16"] = {256: _throughput(torch, Scheduler(llama, prefill_portion=256), VOCAB, 64, 300, 4096, 256, steps, warmup)}
        res["int4_llama_w4a16"]["state_bytes_per_sequence"] = int(2 * llama.cache_k[:, 0].numel() * 2)
        del llama
        torch.cuda.empty_cache()
        res["kernels"] = _kernel_table(torch, s, hbm_gbs, bf16_tflops)
        res["like_kernels_int4_decoder"] = _like_kernels(torch, s, hbm_gbs, bf16_tflops)
        out[name] = res
    clocks = sampler.stop()
    head = out[names[-1]]["mutusun"][2048]
    return {"metric": "mutusun_prefill_decode_tokens_per_s", "value": head["decode_tokens_per_s"], "unit": "tokens/s (decode, 64 sequences)",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": head["decode_ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (float32 residual, norms, scores)", "data": "synthetic",
            "config": {"design": "mutusun", "sizes": names, "weights": "random", "layers": 4,
                       "l2": "kernel timings rotate buffers larger than the L2 where the kernel streams from HBM"},
            "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops, "source": peak_src},
            "gpu_launches": ops.seq_launch_count() - l0, "clocks": clocks, "results": out}


# ---------------------------------------------------------------------------------------------------------------------
# `bench.py --design pitudra`: the Pitudra design (latent + grouped-query window attention, HGRN2, squared-ReLU experts)
# next to Mutusun, the framework's closest model, at equal width / heads / expert sizes, both through the scheduler; and
# Pitudra's kernels one by one against their roofline, with Mutusun's kernel table of the same size beside them.
# ---------------------------------------------------------------------------------------------------------------------
PITUDRA_SIZES = {
    # latent attention: (q_rank, kv_rank, rot_dim); window of both attentions; side = width of the per-layer token input
    "w2048": dict(width=2048, heads=16, kv=4, dim=128, window=1024, latent=(768, 512, 64), moe=(16, 1024, 4), side=256),
    "w4096": dict(width=4096, heads=32, kv=8, dim=128, window=2048, latent=(1536, 512, 64), moe=(8, 2048, 2), side=256),
}


def pitudra_config(s):
    H, D, win = s["heads"], s["dim"], s["window"]
    qr, kvr, rot = s["latent"]
    E, F, top = s["moe"]
    moe = {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": top}}
    lat = {"heads": H, "dim": D, "vdim": D, "rot_dim": rot, "q_rank": qr, "kv_rank": kvr, "scale": (D + rot) ** -0.5, "mask": {"size": win},
           "rot": {"base": 10000.0, "dims": rot}}
    layers = [{"type": "latent_attention", "mixer": lat, "mlp": moe},
              {"type": "latent_attention", "mixer": dict(lat, kv_from=0), "mlp": moe},
              {"type": "hgrn2", "mixer": {"heads": H, "dim": D, "vdim": D}, "mlp": moe},
              {"type": "attention", "mixer": {"heads": H, "kv_heads": s["kv"], "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": win}},
               "mlp": moe}]
    return {"architecture": "Pitudra", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5}, "token_side": {"dim": s["side"]},
            "layers": layers}


def _pitudra_kernel_table(torch, s, hbm_gbs, bf16_tflops):
    """Each Pitudra kernel at a prompt shape (2 048 tokens of one sequence) and a decode shape (64 sequences x 1 token with a
    full window behind it). frac = achieved / measured peak of the binding resource."""
    from . import ops
    dev = "cuda"
    W, H, G, D, win = s["width"], s["heads"], s["kv"], s["dim"], s["window"]
    qr, kvr, rot = s["latent"]
    E, F, top = s["moe"]
    bf, f32 = torch.bfloat16, torch.float32
    rows = []

    def meta(segs):
        r = [[], [], [], [], []]
        at = 0
        for slot, p0, n in segs:
            r[0] += [slot] * n; r[1] += list(range(p0, p0 + n)); r[2] += [at] * n; r[3] += [at + n] * n; r[4] += [0] * n
            at += n
        return torch.tensor(r, dtype=torch.int32, device=dev)

    def add(name, shape, us, nbytes=None, flops=None, note=None):
        e = {"kernel": name, "shape": shape, "us": round(us, 2)}
        if nbytes is not None:
            e["GBps"] = round(nbytes / us / 1e3, 1); e["frac_hbm"] = round(nbytes / us / 1e3 / hbm_gbs, 3)
        if flops is not None:
            e["TFLOPs"] = round(flops / us / 1e6, 1); e["frac_bf16"] = round(flops / us / 1e6 / bf16_tflops, 3)
        if note:
            e["note"] = note
        rows.append(e)

    nslots, Tmax = 64, 2048
    cap = win - 1 + Tmax
    shapes = {"prompt": [(0, 0, 2048)], "decode": [(k, win + 3 * k, 1) for k in range(64)]}
    lat_cache = [torch.randn(nslots, cap, kvr + rot, device=dev).to(bf) for _ in range(2)]
    ck = [torch.randn(nslots, cap, G * D, device=dev).to(bf) for _ in range(2)]
    cv = [torch.randn(nslots, cap, G * D, device=dev).to(bf) for _ in range(2)]
    inv = (10000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(dev)
    for label, segs in shapes.items():
        T = sum(n for _, _, n in segs)
        tab = meta(segs)
        nbuf = max(2, min(8, int(200e6 / (T * W * 12)) + 1))
        x = [torch.randn(T, W, device=dev) for _ in range(nbuf)]
        y = [torch.randn(T, W, device=dev).to(bf) for _ in range(nbuf)]
        h = [torch.empty(T, W, device=dev, dtype=bf) for _ in range(nbuf)]
        wv, bv = torch.ones(W, device=dev), torch.zeros(W, device=dev)
        prev = torch.zeros(2, nslots, W, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_token_shift(x[i], bv, prev, h[i], tab) for i in range(nbuf)])
        add("seq_token_shift", f"{label} T={T} W={W}", us, nbytes=T * W * 6)
        us = _time_us(torch, [lambda i=i: ops.seq_add_norm(y[i], wv, bv, 1e-5, x_in=x[i], x_out=x[i], out=h[i]) for i in range(nbuf)])
        add("seq_add_norm (residual + layer norm of the output + cast)", f"{label} T={T} W={W}", us, nbytes=T * W * 12)
        pair = [torch.randn(T, top, W, device=dev).to(bf) for _ in range(2)]
        rw = torch.rand(T, top, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_add_norm(pair[i % 2], wv, bv, 1e-5, x_in=x[i], x_out=x[i], out=h[i], y_w=rw) for i in range(nbuf)])
        add("seq_add_norm (weighted sum of the experts' parts)", f"{label} T={T} top={top}", us, nbytes=T * W * (10 + 2 * top))
        # latent attention
        ld = qr + kvr + rot
        dd = [(torch.randn(T, ld, device=dev)).to(bf) for _ in range(nbuf)]
        cq = torch.empty(T, qr, device=dev, dtype=bf)
        us = _time_us(torch, [lambda i=i: ops.seq_latent_prep(dd[i], qr, kvr, rot, wv[:qr].contiguous(), wv[:kvr].contiguous(), inv, rot, cq,
                                                              lat_cache[i % 2], tab, 1e-5) for i in range(nbuf)])
        add("seq_latent_prep (2 norms + rotary + cache rows)", f"{label} T={T}", us, nbytes=T * (ld * 2 + qr * 2 + (kvr + rot) * 2))
        q = [(torch.randn(T, H, D + rot, device=dev) * 0.3).to(bf) for _ in range(2)]
        qb = torch.empty(T, H, rot, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_rotary(q[i % 2], D, qb, rot, inv, tab) for i in range(2)])
        add("seq_rotary (query part)", f"{label} T={T} H={H}", us, nbytes=T * H * rot * 6)
        qa = [torch.randn(H, T, kvr, device=dev) * 0.05 for _ in range(2)]
        olat = torch.empty(T, H, kvr, device=dev, dtype=bf)
        sink = torch.zeros(H, device=dev)
        visible = sum(min(p + 1, win) for _, p0, n in segs for p in range(p0, p0 + n))

        def lat_attn(i):
            c = lat_cache[i % 2].unsqueeze(2)
            ops.seq_window_attention(qa[i % 2].transpose(0, 1), qb, c, c[..., :kvr], olat, tab, win, 0.07, sink=sink)
        if label == "prompt":
            # prompts run the expanded form: per-head keys / values of one slot's ring rows from two products, then tiles
            wuk = (torch.randn(H * D, kvr, device=dev) * kvr ** -0.5).to(bf)
            wuv = (torch.randn(H * D, kvr, device=dev) * kvr ** -0.5).to(bf)
            kmat = torch.empty(cap, H * D, device=dev, dtype=bf)
            vmat = torch.empty(cap, H * D, device=dev, dtype=bf)

            def expand(i):
                ring = lat_cache[i % 2][0]
                torch.matmul(ring[:, :kvr], wuk.t(), out=kmat)
                torch.matmul(ring[:, :kvr], wuv.t(), out=vmat)
            us = _time_us(torch, [lambda i=i: expand(i) for i in range(2)])
            add("latent keys / values of a slot's ring rows (2 vendor products)", f"{cap}x{H * D}x{kvr} x 2", us, flops=4.0 * cap * H * D * kvr)
            qfull = [torch.randn(T, H, D + rot, device=dev) * 0.3 for _ in range(2)]
            oexp = torch.empty(T, H, D, device=dev, dtype=bf)
            us = _time_us(torch, [lambda i=i: ops.seq_window_attention_mma(
                qfull[i % 2], kmat.view(1, cap, H, D).expand(nslots, cap, H, D), lat_cache[i % 2][:, :, kvr:],
                vmat.view(1, cap, H, D).expand(nslots, cap, H, D), oexp, tab, win, 0.07, True, sink=sink) for i in range(2)])
            add("seq_window_attention_mma, latent expanded form (16 tokens per CTA)", f"T={T} window={win} H={H} key {D}+{rot} value {D}", us,
                flops=2.0 * visible * H * (2 * D + rot))
        else:
            us = _time_us(torch, [lambda i=i: lat_attn(i) for i in range(2)])
            add("seq_window_attention, latent absorbed form (CUDA cores; float32 and odd sizes)", f"64 seqs x 1, {visible // 64} keys each", us,
                nbytes=visible * (kvr + rot) * 2)
            qabs = [torch.randn(T, H, kvr + rot, device=dev) * 0.05 for _ in range(2)]
            groups = 1 if H <= 16 else H // 16

            def lat_mma(i):
                c = lat_cache[i % 2]
                k4 = c[:, :, :kvr].unsqueeze(2).expand(nslots, cap, groups, kvr)
                ops.seq_window_attention_mma(qabs[i % 2], k4, c[:, :, kvr:], k4, olat, tab, win, 0.07, False, sink=sink)
            us = _time_us(torch, [lambda i=i: lat_mma(i) for i in range(2)])
            add("seq_window_attention_mma, latent absorbed form (16 heads per CTA, key blocks shared by a cluster)",
                f"64 seqs x 1, {visible // 64} keys each", us, nbytes=visible * (kvr + rot) * 2)
        # grouped-query attention
        ldq = H * D + 2 * G * D + H * D
        pq = [(torch.randn(T, ldq, device=dev) * 0.3).to(bf) for _ in range(nbuf)]
        qf = [torch.empty(T, H * D, device=dev) for _ in range(2)]
        wq = torch.ones(H * D, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_qkv_prep(pq[i], H * D, G * D, G * D, wq, wq[:G * D].contiguous(), qf[i % 2], ck[i % 2], cv[i % 2],
                                                           tab, 1e-5) for i in range(nbuf)])
        add("seq_qkv_prep (2 norms + cache rows)", f"{label} T={T}", us, nbytes=T * ((H + 2 * G) * D * 2 + H * D * 4 + 2 * G * D * 2))
        att = torch.empty(T, H, D, device=dev, dtype=bf)

        k4 = [c.view(nslots, cap, G, D) for c in ck]
        v4 = [c.view(nslots, cap, G, D) for c in cv]

        def gqa(i):
            ops.seq_window_attention_mma(qf[i % 2].view(T, H, D), k4[i % 2], None, v4[i % 2], att, tab, win, D ** -0.5, label == "prompt",
                                         sink=sink, gate=pq[i % nbuf][:, H * D + 2 * G * D:])
        us = _time_us(torch, [lambda i=i: gqa(i) for i in range(2)])
        if label == "prompt":
            add("seq_window_attention_mma, grouped-query form + gate (16 tokens per CTA)", f"T={T} window={win} H={H} G={G} D={D}", us,
                flops=2.0 * visible * H * 2 * D)
        else:
            add("seq_window_attention_mma, grouped-query form + gate (heads of a group per CTA)", f"64 seqs x 1, {visible // 64} keys each", us,
                nbytes=visible * G * 2 * D * 2)
        # recurrence
        ldr = H * 3 * D
        pr = [(torch.randn(T, ldr, device=dev)).to(bf) for _ in range(nbuf)]
        state = torch.zeros(nslots, H, D, D, device=dev)
        scr = torch.empty(T * H * 4 * D, device=dev)
        orec = torch.empty(T, H * D, device=dev, dtype=bf)
        fb, lo = torch.zeros(H * D, device=dev), torch.full((H * D,), 0.5, device=dev)
        starts = tab[2].unique().to(torch.int32).contiguous()
        us = _time_us(torch, [lambda i=i: ops.seq_hgrn2(pr[i], fb, lo, wv[:D].contiguous(), state, scr, orec, tab, H, D, D, 1e-5, seg_starts=starts)
                              for i in range(nbuf)])
        nseg = len(segs)
        add("seq_hgrn2 (gates + scan + head norm)", f"{label} T={T} H={H} D={D}", us,
            nbytes=T * (ldr * 2 + H * D * 10) + (2 * nseg * H * D * D * 4 if label == "decode" else 0), flops=4.0 * T * H * D * D,
            note="sequential over a sequence's tokens: H x DV/16 CTAs per sequence" if label == "prompt" else None)
        # router and experts
        hb = [torch.randn(T, W, device=dev).to(bf) for _ in range(nbuf)]
        rwt = torch.randn(E, W, device=dev) * 0.05
        idx = torch.empty(T, top, dtype=torch.int32, device=dev)
        wt = torch.empty(T, top, device=dev)
        us = _time_us(torch, [lambda i=i: ops.moe_route_chosen(hb[i], rwt, idx, wt) for i in range(nbuf)])
        add("moe_route_chosen", f"{label} T={T} R={E}", us, nbytes=T * W * 2)
        up = [(torch.randn(E, F, W, device=dev) * W ** -0.5).to(bf) for _ in range(2)]
        dn = [(torch.randn(E, W, F, device=dev) * F ** -0.5).to(bf) for _ in range(2)]
        pr2 = torch.empty(T, top, W, device=dev, dtype=bf)
        us = _time_us(torch, [lambda i=i: ops.moe_expert_grouped(hb[i % nbuf], up[i % 2], dn[i % 2], idx, pr2, E, F, 0.0, act="relu2") for i in range(2)])
        if label == "prompt":
            add("moe_expert_grouped, squared ReLU (sort + 2 tile GEMMs)", f"T={T} top={top} E={E} F={F}", us, flops=2.0 * T * top * 2 * W * F)
        else:
            touched = len(set(idx.flatten().tolist()))
            add("moe_expert_grouped, squared ReLU (sort + 2 tile GEMMs)", f"T={T} top={top}, {touched} of {E} experts touched", us,
                nbytes=touched * 2 * W * F * 2)
        del x, y, h, pair, dd, q, qa, pq, qf, pr, hb, up, dn
    return rows


def run_pitudra(args, peaks, clock_sampler_cls) -> dict:
    import torch
    from . import ops
    from .build import build_seq_library
    from .mutusun import MutusunConfig, MutusunModel, random_weights as mutusun_weights
    from .pitudra import PitudraConfig, PitudraModel, random_weights
    from .scheduler import Scheduler
    build_seq_library()
    torch.cuda.set_device(0)
    hbm_gbs, bf16_tflops, peak_src = peaks
    bf16_tflops = bf16_tflops or 1590.0
    names = [n for n in (args.sizes.split(",") if args.sizes else PITUDRA_SIZES) if n in PITUDRA_SIZES]
    steps, warmup = args.steps, max(3, args.warmup)
    out = {}
    sampler = clock_sampler_cls(0)
    sampler.start()
    l0 = ops.seq_launch_count()
    for name in names:
        s = PITUDRA_SIZES[name]
        res = {"layers": 4, "sizes": s}
        cfg = PitudraConfig.from_dict(pitudra_config(s))
        model = PitudraModel(cfg, random_weights(cfg, 0), dtype=torch.bfloat16, device="cuda", n_slots=65, max_step_tokens=2048)
        res["pitudra"] = {p: _throughput(torch, Scheduler(model, prefill_portion=p), VOCAB, 64, s["window"] + 300, 4096, p, steps, warmup)
                          for p in (2048, 256)}
        res["pitudra"]["state_bytes_per_sequence"] = model.state_bytes_per_slot()
        del model
        torch.cuda.empty_cache()
        mcfg = MutusunConfig.from_dict(mutusun_config(SIZES[name]))
        mut = MutusunModel(mcfg, mutusun_weights(mcfg, 0), dtype=torch.bfloat16, device="cuda", n_slots=65, max_step_tokens=2048)
        res["mutusun"] = {p: _throughput(torch, Scheduler(mut, prefill_portion=p), VOCAB, 64, s["window"] + 300, 4096, p, steps, warmup)
                          for p in (2048, 256)}
        res["mutusun"]["state_bytes_per_sequence"] = mut.state_bytes_per_slot()
        del mut
        torch.cuda.empty_cache()
        res["kernels"] = _pitudra_kernel_table(torch, s, hbm_gbs, bf16_tflops)
        res["like_kernels_mutusun"] = _kernel_table(torch, SIZES[name], hbm_gbs, bf16_tflops)
        out[name] = res
    clocks = sampler.stop()
    head = out[names[-1]]["pitudra"][2048]
    return {"metric": "pitudra_prefill_decode_tokens_per_s", "value": head["decode_tokens_per_s"], "unit": "tokens/s (decode, 64 sequences)",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": head["decode_ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (float32 residual, norms, scores, recurrence)", "data": "synthetic",
            "config": {"design": "pitudra", "sizes": names, "weights": "random", "layers": 4,
                       "l2": "kernel timings rotate buffers larger than the L2 where the kernel streams from HBM"},
            "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops, "source": peak_src},
            "gpu_launches": ops.seq_launch_count() - l0, "clocks": clocks, "results": out}
