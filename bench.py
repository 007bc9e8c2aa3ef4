#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen3-0.6B shape with random weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  Default run: 28 layers of the Qwen3-0.6B
sizes, batch 8, context 4096 (the last timed step runs at 4096 tokens per request), bf16, synthetic token ids.

    value      decoded tokens per second, timed on the device with CUDA events over K steps that are enqueued
               back to back: every step copies its index arrays from pinned host memory, takes its input tokens
               from the previous step's samples on the device, replays the captured graph and samples.
    e2e        the same through the Python entry point (LLMEngine.add_request / step): host token ids in, sampled
               token ids out, every step; wall clock between device synchronisations.
    prefill    one prompt of 2,048 tokens in one step: tokens per second and the fraction of the bf16 peak
               (flops of the matrix products and of causal attention / time / peak).
    roofline   for the decode step: bytes it has to read (every weight once, the cache of the live requests)
               / time, against the measured copy bandwidth.
    points     decode tokens per second at batch 1 and 64, same context; and the reference's own benchmark (256
               requests with random lengths through the engine, output tokens a second; the reference's README gives
               5156 tok/s for it on an A10G).
Peaks come from MEASURED_PEAKS.json next to this file when the driver wrote it, else from the fallback
(6650 GB/s, 1590 TFLOP/s).  Every timed step reads several GB, far more than the 126 MB L2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=1024, num_hidden_layers=28,
             num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936,
             rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=40960)
FULL_LAYERS = 28
# the next larger shape of the same architecture (Qwen3-8B sizes); --shape 8b with --layers N checks the kernels there
MODEL_8B = dict(MODEL, hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, tie_word_embeddings=False)
CONTEXT = 4096
PREFILL_TOKENS = 2048


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            flat = {}

            def walk(x):
                if isinstance(x, dict):
                    for k, v in x.items():
                        if isinstance(v, (int, float)):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(d)
            if "hbm_gbs" in flat:
                out["hbm_gbs"] = flat["hbm_gbs"]
            if "bf16_tflops" in flat:
                out["bf16_tflops"] = flat["bf16_tflops"]
            out["source"] = "measured"
        except Exception:
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        rows = [r for t, r in self.rows if any(a <= t <= b for a, b in windows)] or [r for _, r in self.rows]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_flops_prefill(cfg, layers, T):
    D, H, KV, hd, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                          cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = 2 * T * (D * (H + 2 * KV) * hd + H * hd * D + 3 * D * I)
    attn = 4 * H * hd * T * (T + 1) // 2
    return layers * (per_layer + attn) + 2 * D * V


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a CMake C++/CUDA project without setup.py or pyproject.toml (pip: 'not installable'); its "
                      "build fetches flash-attention from the network and targets sm_80/86/89 only"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--shape", default="0.6b", choices=["0.6b", "8b"], help="layer sizes: Qwen3-0.6B (default) or Qwen3-8B")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    K, W, B, CTX = args.steps, max(3, args.warmup), args.batch, args.context

    import torch
    from cppvllm_b200 import EngineConfig, SamplingParams
    from cppvllm_b200.csrc import ops
    from cppvllm_b200.engine.llm_engine import LLMEngine
    from cppvllm_b200.engine.runner import StepEntry
    from cppvllm_b200.weights.random_init import write_random_model

    pk = peaks()
    base = MODEL if args.shape == "0.6b" else MODEL_8B
    full_layers = base["num_hidden_layers"]
    if args.shape != "0.6b" and args.layers == FULL_LAYERS:
        args.layers = full_layers
    cfg = dict(base, num_hidden_layers=args.layers)
    tmp = tempfile.mkdtemp(prefix="cppvllm_b200_bench_")
    t_build = time.time()
    model_dir = write_random_model(os.path.join(tmp, "qwen3_0p6b_random"), cfg, seed=0, std=0.02, norm_spread=0.0)
    max_b = B if args.no_points else max(B, 256)                # 256: the reference's throughput workload (bench.cpp)
    max_len = max(CTX + 64, PREFILL_TOKENS)              # the prefill point needs its 2,048 positions at any --context
    page = 32
    llm = LLMEngine(EngineConfig(model_path=model_dir, dtype="bfloat16", max_num_batched_tokens=8192, max_num_seqs=max_b,
                                 max_chunk_tokens=4096, max_model_len=max_len, block_size=page,
                                 num_kv_blocks=max(max(B, 64) * ((max_len + page - 1) // page),
                                                   0 if args.no_points else 256 * (2048 // page)) + 8, seed=0))
    r, sampler = llm.runner, llm.sampler
    vocab = r.vocab_size
    gen = torch.Generator().manual_seed(0)
    print(f"[bench] model written and loaded in {time.time() - t_build:.1f} s; {r.num_pages} pages of {page} tokens",
          file=sys.stderr, flush=True)
    clocks = ClockSampler()
    clocks.start()
    windows = []

    def rand_tokens(n):
        return torch.randint(0, min(10000, vocab), (n,), generator=gen).tolist()

    # ---- prefill: one prompt of 2,048 tokens in one step ------------------------------------------------------
    pre_ms = []
    for it in range(1 + 3):
        toks = rand_tokens(PREFILL_TOKENS)
        r.cache.admit("pf")
        r.cache.reserve("pf", PREFILL_TOKENS)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        r.step([StepEntry("pf", toks, 0, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        if it > 0:
            pre_ms.append(e0.elapsed_time(e1))
            windows.append((t0, time.time()))
        r.cache.release("pf")
    pre = min(pre_ms)
    flops = model_flops_prefill(cfg, args.layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (pre / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre, 3),
               "frac": round(flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode on the device: K steps enqueued back to back ---------------------------------------------------
    def decode_run(batch, steps, warm):
        ctx0 = CTX - steps - warm                               # the last timed step runs at CTX tokens
        ids = [f"d{i}" for i in range(batch)]
        prompts = {i: rand_tokens(ctx0) for i in ids}
        for i in ids:
            r.cache.admit(i)
            r.cache.reserve(i, CTX + 1)
        fed = 0
        per_step = max(1, 8192 // batch)
        last = None
        while fed < ctx0:                                       # fill the context: prompt portions of all requests
            n = min(per_step, ctx0 - fed)
            last = r.step([StepEntry(i, prompts[i][fed:fed + n], fed, [n - 1] if fed + n == ctx0 else []) for i in ids])
            fed += n
        temps, seeds = [0.6] * batch, list(range(1, batch + 1))
        sampled = sampler.sample_async(last, temps, seeds, [0] * batch)
        src = list(range(batch))
        pos = ctx0
        launches0 = 0
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        t0 = 0.0
        for s in range(warm + steps):
            if s == warm:
                torch.cuda.synchronize()
                launches0 = ops.launches()
                t0 = time.time()
                ev[0].record()
            logits = r.step([StepEntry(i, [0], pos, [0]) for i in ids], feed=(sampled, src))
            sampled = sampler.sample_async(logits, temps, seeds, [s + 1] * batch)
            pos += 1
        ev[1].record()
        torch.cuda.synchronize()
        windows.append((t0, time.time()))
        ms = ev[0].elapsed_time(ev[1]) / steps
        n_launch = ops.launches() - launches0
        r.check_errors()
        mean_kv = sum(range(ctx0 + warm + 1, ctx0 + warm + steps + 1)) / steps
        nbytes = r.model.decode_weight_bytes() + batch * mean_kv * r.kv_bytes_per_token()
        for i in ids:
            r.cache.release(i)
        return ms, n_launch, nbytes

    ms8, launches, bytes8 = decode_run(B, K, W)
    value = B / (ms8 / 1e3)
    achieved = bytes8 / (ms8 / 1e3) / 1e9
    points = {}
    if not args.no_points:
        for b in (1, 64):
            ms_b, _, _ = decode_run(b, max(8, K // 4), W)
            points[f"decode_b{b}"] = round(b / (ms_b / 1e3), 1)

    # ---- end to end through the public entry point --------------------------------------------------------------
    ctx0 = CTX - K - W
    sp = SamplingParams(temperature=0.6, max_tokens=K + W + 8, ignore_eos=True)
    for _ in range(B):
        llm.add_request(rand_tokens(ctx0), sp)
    guard = 0
    while llm.num_without_first_token() > 0 and guard < 1000:
        llm.step()                                              # prompt portions until every request has sampled once
        guard += 1
    for _ in range(W - 1):
        llm.step()
    torch.cuda.synchronize()
    gen0 = llm.stats().tokens_generated
    t0 = time.time()
    c0 = time.perf_counter()
    for _ in range(K):
        llm.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - c0
    windows.append((t0, time.time()))
    e2e_tokens = llm.stats().tokens_generated - gen0
    h2d = r.h2d_bytes_last_step + sampler.h2d_bytes_last
    while not llm.is_finished():
        llm.step()
    llm.take_finished()

    # ---- the reference's own benchmark (bench.cpp:10-63): 256 requests, prompt and output lengths uniform in
    # [100, 1024], token ids uniform in [0, 10000], temperature 0.6, ignore_eos; output tokens a second -----------
    if not args.no_points:
        import random
        rng = random.Random(0)
        reqs = [([rng.randint(0, min(10000, vocab - 1)) for _ in range(rng.randint(100, 1024))],
                 SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=rng.randint(100, 1024))) for _ in range(256)]
        llm.generate([[1, 2, 3, 4, 5, 6, 7, 8]], SamplingParams(max_tokens=16))
        torch.cuda.synchronize()
        t0 = time.time()
        c0 = time.perf_counter()
        for pr, sp_i in reqs:
            llm.add_request(pr, sp_i)
        while not llm.is_finished():
            llm.step()
        torch.cuda.synchronize()
        points["throughput_256_requests"] = round(sum(sp_i.max_tokens for _, sp_i in reqs) / (time.perf_counter() - c0), 1)
        windows.append((t0, time.time()))
        llm.take_finished()
    clocks.stop()

    line = {
        "metric": f"decode tok/s at batch {B}, context {CTX} (Qwen3-{args.shape.upper()} shape, random weights)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform random token ids",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": args.layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied": cfg["tie_word_embeddings"],
                   "global_batch": B, "seq_len": CTX, "page_size": page, "parallelism": "single GPU",
                   "l2": "each step reads > L2 (weights + cache)", "peaks": pk["source"],
                   "hbm_peak_gbs": pk["hbm_gbs"], "bf16_peak_tflops": pk["bf16_tflops"]},
        "e2e": {"value": round(e2e_tokens / e2e_s, 1), "unit": "tok/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": 4 * B},
        "gpu_launches": int(launches),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(windows),
    }
    print(json.dumps(line))
    try:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)
    except Exception:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
