"""Command line of the text-only decoder LMs.

    python -m moshi_b200.cli trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N     (bin/trace_run)
    python -m moshi_b200.cli generate --model DIR --prompt 5,17,3 [--max-new 16] [--temp 0.8 --top-k 250]

``trace`` replays a schedule of steps from standard input through the model's own step function and scheduler and writes the
logits it is asked for; ``generate`` runs prompts through ``TokenScheduler.run`` (greedy unless --temp is given).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def _load(model_dir: str, dtype_name: str):
    import torch

    from . import build
    build.ensure("decoder")                       # a fresh checkout compiles what this model family needs, and only that
    from .models import loaders
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype_name]
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    if loaders.model_class(raw).__name__ != "DecoderLM":
        raise SystemExit("this command line serves text-only decoder LMs")
    torch.cuda.set_device(0)
    return loaders.get_decoder_lm(model_dir, device="cuda:0", dtype=dtype)


def trace_main(argv: list[str]) -> int:
    ap = argparse.ArgumentParser(prog="trace_run")
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, default=4096)
    ap.add_argument("--slots", type=int, default=4)
    ap.add_argument("--max-step-tokens", type=int, default=1024)
    a = ap.parse_args(argv)
    import numpy as np
    import torch

    from .models import DecoderLMGen
    from .serving import TokenScheduler
    model = _load(a.model, a.dtype)
    out_dir = Path(a.out)
    # every live request may hold up to --max-tokens tokens; portions larger than a step's buffers are cut by the scheduler
    gen = DecoderLMGen(model, slots=a.slots, capacity=max(a.max_tokens, 1), max_step_tokens=a.max_step_tokens, max_want=a.max_step_tokens)
    sched = TokenScheduler(gen)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        order = []
        for e in step["entries"]:
            sched.feed(e["id"], e["tokens"], e.get("want", []))
            order.append(e["id"])
        rows: dict[str, list] = {rid: [] for rid in order}
        while True:
            got = sched.run_step()
            if got is None:
                break
            for rid, lg in got.items():
                rows[rid].append(lg)
        parts = [t for rid in order for t in rows[rid]]
        if parts:
            logits = torch.cat(parts, dim=0).float().cpu().numpy().astype("<f4")
            tmp = out_dir / f".{step['step']}.tmp"
            logits.tofile(tmp)
            tmp.rename(out_dir / f"{step['step']}.f32")
        else:
            torch.cuda.synchronize()
        for rid in step.get("end", []):
            sched.end(rid)
        print(f"done {step['step']}", flush=True)
    flags = gen.error_flags()
    gen.close()
    if flags:
        print(f"device error flags {flags}", file=sys.stderr)
        return 1
    return 0


def generate_main(argv: list[str]) -> int:
    ap = argparse.ArgumentParser(prog="generate")
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeat for a batch")
    ap.add_argument("--max-new", type=int, default=16)
    ap.add_argument("--temp", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=250)
    ap.add_argument("--eos", type=int, default=None)
    a = ap.parse_args(argv)
    from .models import DecoderLMGen
    from .serving import TokenScheduler
    model = _load(a.model, a.dtype)
    prompts = [[int(x) for x in p.split(",") if x.strip()] for p in a.prompt]
    cap = max(len(p) for p in prompts) + a.max_new
    gen = DecoderLMGen(model, slots=min(len(prompts), 64), capacity=cap, max_step_tokens=min(2048, max(cap, 16)),
                       use_sampling=a.temp > 0, temp=a.temp, top_k=a.top_k)
    sched = TokenScheduler(gen, eos=a.eos)
    for i, p in enumerate(prompts):
        sched.submit(f"p{i}", p, a.max_new)
    for rid, toks in sched.run().items():
        print(json.dumps({"id": rid, "tokens": toks}))
    gen.close()
    return 0


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] not in ("trace", "generate"):
        print(__doc__, file=sys.stderr)
        return 2
    return trace_main(argv[1:]) if argv[0] == "trace" else generate_main(argv[1:])


if __name__ == "__main__":
    sys.exit(main())
