"""Trace replay: feeds given token ids through the model step by step and writes logits.  It samples nothing
and has no forward pass, cache or loader of its own: it drives the ``ModelRunner`` (model, step function, cache
manager and kernels) that generation uses.  The reference has no such tool.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` hold, per request, its next tokens and the indices among them whose logits are wanted; all entries
of a step run as one batch.  A request is admitted at its first appearance, may skip steps, and gives back
what it holds when it is named in ``end``.  For a step in which something is wanted, ``<out>/<step>.f32``
receives the logits as little-endian float32 [wanted, vocab], in the order of the entries and of ``want``.
After every step the line ``done <step>`` is printed and flushed.  The cache pool holds ``--max-tokens`` tokens
(a multiple of the page size), so pages are used again as requests end.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder that receives <step>.f32")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="tokens the cache pool holds (each live request's count rounded up to a multiple of 64)")
    p.add_argument("--block-size", type=int, default=32, help="tokens per cache page (must divide 64)")
    p.add_argument("--max-num-seqs", type=int, default=16, help="most requests in one step")
    p.add_argument("--enforce-eager", action="store_true", help="never replay CUDA graphs for decode-only steps")
    p.add_argument("--use-ref-kernels", action="store_true", help="plain twin kernels only (general attention, library products)")
    return p


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.max_tokens <= 0:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    if args.block_size <= 0 or 64 % args.block_size:
        print("trace_run: --block-size must divide 64", file=sys.stderr)
        return 2
    from ..config.engine_config import parse_dtype
    from ..cache.manager import OutOfPages
    from .runner import ModelRunner, StepEntry

    os.makedirs(args.out, exist_ok=True)
    ps = args.block_size
    num_pages = (args.max_tokens + ps - 1) // ps
    runner = ModelRunner(args.model, dtype=parse_dtype(args.dtype), device="cuda:0", page_size=ps,
                         num_pages=num_pages, max_step_tokens=max(64, min(args.max_tokens, 32768)),
                         max_seqs=args.max_num_seqs, max_model_len=max(64, args.max_tokens),
                         enforce_eager=args.enforce_eager, use_ref_kernels=args.use_ref_kernels)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            toks = [int(t) for t in e["tokens"]]
            if not toks:
                continue
            if rid not in runner.cache.leases:
                runner.cache.admit(rid)
            start = runner.cache.lease(rid).computed
            try:
                runner.cache.reserve(rid, start + len(toks))
            except OutOfPages as ex:
                print(f"trace_run: step {step}: {ex} (the pool holds {args.max_tokens} tokens)", file=sys.stderr)
                return 3
            entries.append(StepEntry(rid, toks, start, [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                host = logits.to("cpu", torch.float32).contiguous().numpy()
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                host.astype("<f4", copy=False).tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            runner.check_errors()
        for rid in rec.get("end", []):
            if rid in runner.cache.leases:
                runner.cache.release(rid)
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
