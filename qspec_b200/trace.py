"""Trace replay: feeds recorded steps of token ids through a model and writes the logits that each step asks for.

    python -m qspec_b200.trace --model DIR --dtype bfloat16|float32 --out DIR [--max-tokens N]      (or bin/trace_run)

Standard input carries one JSON object per line: {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}.
Every step goes through `scheduler.Scheduler.feed` -- the step function the generation loop uses -- on the model the
registry builds for the folder's config.json. For a step that wants logits, OUT/<n>.f32 receives them as little-endian
float32 [wanted, vocab]; after every step a line "done <n>" is printed. Requests listed under "end" give their slot
back. Exit status 3: the model has no implementation in the requested number format.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="replay recorded steps through a model and write the requested logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, default=0, help="most tokens that live requests hold at any time")
    ap.add_argument("--slots", type=int, default=4, help="requests that can be live at once")
    ap.add_argument("--step-tokens", type=int, default=2048, help="tokens per pass through the model (longer steps are cut)")
    args = ap.parse_args(argv)

    from . import registry
    cfg = registry.read_config(args.model)
    arch = registry.architecture_of(cfg)
    if not registry.supports_dtype(arch, args.dtype):
        print(f"{arch} has no {args.dtype} implementation", file=sys.stderr)
        return 3
    from .build import build_seq_library
    build_seq_library()                      # compiled on first use (seconds); a no-op afterwards
    import torch
    from .scheduler import Scheduler
    if not torch.cuda.is_available():
        print("no CUDA device: this framework has no CPU path", file=sys.stderr)
        return 2
    model = registry.load_model(args.model, dtype=args.dtype, device="cuda", n_slots=args.slots,
                                max_step_tokens=args.step_tokens, max_seq_tokens=args.max_tokens or None)
    sched = Scheduler(model)
    os.makedirs(args.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in step.get("entries", [])]
        logits = sched.feed(entries)
        if logits.shape[0]:
            data = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4")
            tmp = os.path.join(args.out, f".{step['step']}.f32.part")
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(args.out, f"{step['step']}.f32"))
        else:
            torch.cuda.synchronize()
        for rid in step.get("end", []):
            sched.release(rid)
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
