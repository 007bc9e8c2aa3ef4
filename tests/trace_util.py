"""Helpers for the replay tests: build traces in different cuttings, run bin/trace_run, collect rows."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def run_trace(model_dir, dtype, steps, max_tokens, out_dir, extra=()):
    """Feed `steps` (list of dicts) to trace_run one at a time, waiting for `done <step>` after each.
    Returns {step: float32 array [wanted, vocab]}."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)] + list(extra)
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        for st in steps:
            p.stdin.write(json.dumps(st) + "\n")
            p.stdin.flush()
            line = p.stdout.readline()
            if line.strip() != f"done {st['step']}":
                p.stdin.close()
                err = p.stderr.read()
                raise AssertionError(f"trace_run answered {line!r} to step {st['step']}; stderr:\n{err[-3000:]}")
        p.stdin.close()
        rc = p.wait(timeout=120)
        err = p.stderr.read()
        assert rc == 0, f"trace_run exited with {rc}:\n{err[-3000:]}"
    finally:
        if p.poll() is None:
            p.kill()
    out = {}
    for st in steps:
        n = sum(len(e["want"]) for e in st["entries"])
        f = os.path.join(out_dir, f"{st['step']}.f32")
        if n:
            a = np.fromfile(f, dtype="<f4")
            out[st["step"]] = a.reshape(n, -1)
        else:
            assert not os.path.exists(f)
    return out


def run_trace_in_process(runner, steps):
    """The same protocol as trace_run's loop, on a ModelRunner that the test holds (one model load for many traces).
    Returns {step: float32 array [wanted, vocab]}."""
    from cppvllm_b200.engine.runner import StepEntry
    out = {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            rid = e["id"]
            if rid not in runner.cache.leases:
                runner.cache.admit(rid)
            start = runner.cache.lease(rid).computed
            runner.cache.reserve(rid, start + len(e["tokens"]))
            entries.append(StepEntry(rid, list(e["tokens"]), start, list(e["want"])))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                out[st["step"]] = logits.float().cpu().numpy().copy()
            runner.check_errors()
        for rid in st.get("end", []):
            if rid in runner.cache.leases:
                runner.cache.release(rid)
    return out


def rows_by_position(steps, outputs, repeats=False):
    """{(request id, absolute position): logits row} from a trace and its outputs.  With `repeats`, a request that
    was ended and fed again from its first token (dropped and recomputed) may produce a position twice: the values are
    lists of rows."""
    fed = {}
    rows = {}
    for st in steps:
        r = 0
        for e in st["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                key = (e["id"], base + w)
                if repeats:
                    rows.setdefault(key, []).append(outputs[st["step"]][r])
                else:
                    assert key not in rows
                    rows[key] = outputs[st["step"]][r]
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
        for rid in st.get("end", []):
            fed.pop(rid, None)
    return rows


class TraceBuilder:
    def __init__(self):
        self.steps = []

    def add(self, entries, end=()):
        self.steps.append({"step": len(self.steps), "entries": [
            {"id": rid, "tokens": list(toks), "want": list(want)} for rid, toks, want in entries], "end": list(end)})
        return self


def whole(tb, rid, toks):
    tb.add([(rid, toks, range(len(toks)))], end=[rid])


def tail_one_by_one(tb, rid, toks, tail=32):
    n = len(toks) - tail
    tb.add([(rid, toks[:n], range(n))])
    for i in range(n, len(toks)):
        tb.add([(rid, toks[i:i + 1], [0])], end=[rid] if i == len(toks) - 1 else [])


def portions(tb, rid, toks, sizes=(7, 2, 13, 3, 2, 29, 2, 5, 17, 2, 11)):
    pos, i = 0, 0
    while pos < len(toks):
        n = min(sizes[i % len(sizes)], len(toks) - pos)
        if len(toks) - pos - n == 1:          # never leave a single token: portions go down to two
            n += 1
        tb.add([(rid, toks[pos:pos + n], range(n))], end=[rid] if pos + n == len(toks) else [])
        pos += n
        i += 1


def needed_max_tokens(steps):
    """The most tokens live requests hold at any time, each request's count rounded up to a multiple of 64."""
    fed, worst = {}, 0
    for st in steps:
        for e in st["entries"]:
            fed[e["id"]] = fed.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum((n + 63) // 64 * 64 for n in fed.values()))
        for rid in st.get("end", []):
            fed.pop(rid, None)
    return worst
