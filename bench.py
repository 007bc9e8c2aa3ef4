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
    points     decode tokens per second at batch 1 and 64, same context, each with its fraction of the copy bandwidth;
               the reference's own benchmark (256 requests with random lengths through the engine, output tokens a
               second; the reference's README gives 5156 tok/s for it on an A10G); the same decode and prefill points at
               the Qwen3-8B layer sizes (contexts 4096 and 8192) and a mixed step at the Qwen3-32B layer sizes (64
               decoding requests at context 4096 beside a 1,024-token portion of a 2,048-token prompt), both with fewer
               layers than the models have (the number is named beside them), each with its fraction of the peak.
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
# the larger shapes of the same architecture (Qwen3-8B and Qwen3-32B layer sizes) for the further points
MODEL_8B = dict(MODEL, hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, tie_word_embeddings=False)
MODEL_32B = dict(MODEL, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                 intermediate_size=25600, tie_word_embeddings=False)
LAYERS_8B, LAYERS_32B = 4, 2        # layers that the further points run with (of 36 and 64)
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


class Bench:
    """One model shape on the device: the engine, and the measurements that the points are made of."""

    def __init__(self, cfg, max_b, max_len, pages, page=32, seed=0):
        import torch
        from cppvllm_b200 import EngineConfig
        from cppvllm_b200.engine.llm_engine import LLMEngine
        from cppvllm_b200.weights.random_init import write_random_model
        self.torch, self.cfg, self.page = torch, cfg, page
        self.tmp = tempfile.mkdtemp(prefix="cppvllm_b200_bench_")
        t0 = time.time()
        model_dir = write_random_model(os.path.join(self.tmp, "random_model"), cfg, seed=seed, std=0.02, norm_spread=0.0)
        self.llm = LLMEngine(EngineConfig(model_path=model_dir, dtype="bfloat16", max_num_batched_tokens=8192, max_num_seqs=max_b,
                                          max_chunk_tokens=4096, max_model_len=max_len, block_size=page, num_kv_blocks=pages, seed=0))
        self.r, self.sampler = self.llm.runner, self.llm.sampler
        self.gen = torch.Generator().manual_seed(0)
        self.windows = []
        print(f"[bench] {cfg['hidden_size']}-wide model with {cfg['num_hidden_layers']} layers written and loaded in "
              f"{time.time() - t0:.1f} s; {self.r.num_pages} pages of {page} tokens", file=sys.stderr, flush=True)

    def close(self):
        import gc
        import shutil
        self.llm = self.r = self.sampler = None
        gc.collect()
        self.torch.cuda.empty_cache()
        shutil.rmtree(self.tmp, ignore_errors=True)

    def rand_tokens(self, n):
        return self.torch.randint(0, min(10000, self.r.vocab_size), (n,), generator=self.gen).tolist()

    def prefill(self, tokens, pk):
        """One prompt of `tokens` tokens in one step: (ms, tokens per second, fraction of the bf16 peak)."""
        from cppvllm_b200.engine.runner import StepEntry
        torch, r = self.torch, self.r
        ms = []
        for it in range(1 + 3):
            toks = self.rand_tokens(tokens)
            r.cache.admit("pf")
            r.cache.reserve("pf", tokens)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.time()
            e0.record()
            r.step([StepEntry("pf", toks, 0, [tokens - 1])])
            e1.record()
            torch.cuda.synchronize()
            if it > 0:
                ms.append(e0.elapsed_time(e1))
                self.windows.append((t0, time.time()))
            r.cache.release("pf")
        best = min(ms)
        flops = model_flops_prefill(self.cfg, self.cfg["num_hidden_layers"], tokens)
        return best, tokens / (best / 1e3), flops / (best / 1e3) / (pk["bf16_tflops"] * 1e12)

    def portion(self, cached, tokens, pk):
        """A portion of `tokens` tokens of a prompt whose first `cached` tokens are in the cache already, in one step:
        (ms, tokens per second, fraction of the bf16 peak; the flops are the portion's own)."""
        from cppvllm_b200.engine.runner import StepEntry
        torch, r = self.torch, self.r
        ms = []
        budget = r.max_step_tokens
        for it in range(1 + 3):
            toks = self.rand_tokens(cached + tokens)
            r.cache.admit("pp")
            r.cache.reserve("pp", cached + tokens)
            for a in range(0, cached, budget):
                r.step([StepEntry("pp", toks[a:min(cached, a + budget)], a, [])])
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.time()
            e0.record()
            r.step([StepEntry("pp", toks[cached:], cached, [tokens - 1])])
            e1.record()
            torch.cuda.synchronize()
            if it > 0:
                ms.append(e0.elapsed_time(e1))
                self.windows.append((t0, time.time()))
            r.cache.release("pp")
        best = min(ms)
        c = self.cfg
        D, H, KV, hd, I, V, L = (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                                 c["intermediate_size"], c["vocab_size"], c["num_hidden_layers"])
        per_token = 2 * (D * (H + 2 * KV) * hd + H * hd * D + 3 * D * I)
        flops = L * (tokens * per_token + 4 * H * hd * tokens * (cached + (tokens + 1) / 2.0)) + 2 * D * V
        return best, tokens / (best / 1e3), flops / (best / 1e3) / (pk["bf16_tflops"] * 1e12)

    def decode(self, batch, ctx, steps, warm, repeats=1):
        """`steps` decode steps of `batch` requests enqueued back to back, the last at `ctx` tokens per request, timed
        on the device (`repeats` times; the median counts).  Returns (ms per step, launches, bytes a step must read)."""
        from cppvllm_b200.csrc import ops
        from cppvllm_b200.engine.runner import StepEntry
        torch, r, sampler = self.torch, self.r, self.sampler
        total = warm + steps * repeats
        ctx0 = ctx - total
        ids = [f"d{i}" for i in range(batch)]
        prompts = {i: self.rand_tokens(ctx0) for i in ids}
        for i in ids:
            r.cache.admit(i)
            r.cache.reserve(i, ctx + 1)
        fed, per_step, last = 0, max(1, 8192 // batch), None
        while fed < ctx0:                                       # fill the context: prompt portions of all requests
            n = min(per_step, ctx0 - fed)
            last = r.step([StepEntry(i, prompts[i][fed:fed + n], fed, [n - 1] if fed + n == ctx0 else []) for i in ids])
            fed += n
        temps, seeds = [0.6] * batch, list(range(1, batch + 1))
        sampled = sampler.sample_async(last, temps, seeds, [0] * batch)
        src = list(range(batch))
        pos, timings, launches = ctx0, [], 0
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        t0 = 0.0
        for s in range(total):
            timed = s - warm
            if timed >= 0 and timed % steps == 0:
                torch.cuda.synchronize()
                launches0 = ops.launches()
                t0 = time.time()
                ev[0].record()
            logits = r.step([StepEntry(i, [0], pos, [0]) for i in ids], feed=(sampled, src))
            sampled = sampler.sample_async(logits, temps, seeds, [s + 1] * batch)
            pos += 1
            if timed >= 0 and timed % steps == steps - 1:
                ev[1].record()
                torch.cuda.synchronize()
                self.windows.append((t0, time.time()))
                timings.append(ev[0].elapsed_time(ev[1]) / steps)
                launches = ops.launches() - launches0
        r.check_errors()
        ms = statistics.median(timings)
        mean_kv = ctx - (steps * repeats) / 2.0
        nbytes = r.model.decode_weight_bytes() + batch * mean_kv * r.kv_bytes_per_token()
        for i in ids:
            r.cache.release(i)
        return ms, launches, nbytes

    def mixed(self, decoders, ctx, prompt_len, portion, steps, warm):
        """Steps that hold one decoded token of each of `decoders` requests (at about `ctx` tokens) beside a portion of
        `portion` tokens of a prompt of `prompt_len`, prompts following one another.  Returns (ms per step, bytes the step
        must read, flops of the step)."""
        from cppvllm_b200.engine.runner import StepEntry
        torch, r = self.torch, self.r
        total = warm + steps
        ctx0 = ctx - total
        ids = [f"m{i}" for i in range(decoders)]
        for i in ids:
            r.cache.admit(i)
            r.cache.reserve(i, ctx + 1)
        fed, per_step = 0, max(1, 8192 // decoders)
        toks = {i: self.rand_tokens(ctx0) for i in ids}
        while fed < ctx0:
            n = min(per_step, ctx0 - fed)
            r.step([StepEntry(i, toks[i][fed:fed + n], fed, []) for i in ids])
            fed += n
        pos, p_pos, p_id, prompt = ctx0, 0, 0, self.rand_tokens(prompt_len)
        r.cache.admit("p0")
        r.cache.reserve("p0", prompt_len)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        t0 = 0.0
        for s in range(total):
            if s == warm:
                torch.cuda.synchronize()
                t0 = time.time()
                ev[0].record()
            entries = [StepEntry(i, [1 + (s % 7)], pos, [0]) for i in ids]
            last = p_pos + portion >= prompt_len
            entries.append(StepEntry(f"p{p_id}", prompt[p_pos:p_pos + portion], p_pos, [portion - 1] if last else []))
            r.step(entries)
            pos += 1
            p_pos += portion
            if last:                                            # the next prompt takes its place
                r.cache.release(f"p{p_id}")
                p_id, p_pos = p_id + 1, 0
                r.cache.admit(f"p{p_id}")
                r.cache.reserve(f"p{p_id}", prompt_len)
        ev[1].record()
        torch.cuda.synchronize()
        self.windows.append((t0, time.time()))
        r.check_errors()
        ms = ev[0].elapsed_time(ev[1]) / steps
        r.cache.release(f"p{p_id}")
        for i in ids:
            r.cache.release(i)
        c = self.cfg
        D, H, KV, hd, I, V, L = (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                                 c["intermediate_size"], c["vocab_size"], c["num_hidden_layers"])
        per_token = 2 * (D * (H + 2 * KV) * hd + H * hd * D + 3 * D * I)
        mean_p = prompt_len / 2.0                                # keys a portion's tokens see, on average over the prompt
        flops = L * ((decoders + portion) * per_token + 4 * H * hd * (decoders * ctx + portion * mean_p)) + 2 * D * V * (decoders + 1)
        nbytes = r.model.decode_weight_bytes() + (decoders * (ctx - steps / 2.0) + mean_p) * r.kv_bytes_per_token()
        return ms, nbytes, flops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--no-points", action="store_true", help="the headline numbers only: no further batches, shapes or workloads")
    ap.add_argument("--no-larger-shapes", action="store_true", help="skip the points at the 8B and 32B layer sizes")
    ap.add_argument("--shape", default="0.6b", choices=["0.6b", "8b"], help="layer sizes of the headline run: Qwen3-0.6B (default) or Qwen3-8B")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    K, W, B, CTX = args.steps, max(3, args.warmup), args.batch, args.context
    REPEATS = 5                                                 # the K timed steps are taken this often; the median counts

    import torch
    from cppvllm_b200 import SamplingParams

    pk = peaks()
    base = MODEL if args.shape == "0.6b" else MODEL_8B
    full_layers = base["num_hidden_layers"]
    if args.shape != "0.6b" and args.layers == FULL_LAYERS:
        args.layers = full_layers
    cfg = dict(base, num_hidden_layers=args.layers)
    max_b = B if args.no_points else max(B, 256)                # 256: the reference's throughput workload (bench.cpp)
    max_len = max(CTX + 64, PREFILL_TOKENS)              # the prefill point needs its 2,048 positions at any --context
    page = 32
    pages = max(max(B, 1 if args.no_points else 64) * ((max_len + page - 1) // page), 0 if args.no_points else 256 * (2048 // page)) + 8
    bench = Bench(cfg, max_b, max_len, pages, page)
    llm, r = bench.llm, bench.r
    vocab = r.vocab_size
    clocks = ClockSampler()
    clocks.start()

    pre_ms, pre_tps, pre_frac = bench.prefill(PREFILL_TOKENS, pk)
    prefill = {"value": round(pre_tps, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3), "frac": round(pre_frac, 4)}

    ms8, launches, bytes8 = bench.decode(B, CTX, K, W, REPEATS)
    value = B / (ms8 / 1e3)
    achieved = bytes8 / (ms8 / 1e3) / 1e9
    points = {}
    if not args.no_points:
        for b in (1, 16, 64):
            ms_b, _, nb = bench.decode(b, CTX, max(8, K // 4), W, 3)
            points[f"decode_b{b}"] = round(b / (ms_b / 1e3), 1)
            points[f"decode_b{b}_frac"] = round(nb / (ms_b / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        if CTX >= 1024:
            # a prompt portion behind a long context: few query blocks with many key tiles each
            _, tps_p, frac_p = bench.portion(CTX - 512, 512, pk)
            points[f"portion_512_behind_{CTX - 512}_tok_s"], points[f"portion_512_behind_{CTX - 512}_frac"] = round(tps_p, 1), round(frac_p, 4)

    # ---- end to end through the public entry point --------------------------------------------------------------
    ctx0 = CTX - K - W
    sp = SamplingParams(temperature=0.6, max_tokens=K + W + 8, ignore_eos=True)
    for _ in range(B):
        llm.add_request(bench.rand_tokens(ctx0), sp)
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
    bench.windows.append((t0, time.time()))
    e2e_tokens = llm.stats().tokens_generated - gen0
    h2d = r.h2d_bytes_last_step + bench.sampler.h2d_bytes_last
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
        bench.windows.append((t0, time.time()))
        llm.take_finished()
    windows = list(bench.windows)
    llm = r = None
    bench.close()

    # ---- the larger shapes of the architecture, with fewer layers than the models have ----------------------------
    if not args.no_points and not args.no_larger_shapes and args.shape == "0.6b":
        big = Bench(dict(MODEL_8B, num_hidden_layers=LAYERS_8B), 64, 8192 + 64, 64 * ((8192 + 64 + page - 1) // page) + 8, page, seed=1)
        points["8b_layers"], points["8b_layers_full"] = LAYERS_8B, MODEL_8B["num_hidden_layers"]
        ms_p, tps, frac = big.prefill(PREFILL_TOKENS, pk)
        points["8b_prefill_2048_tok_s"], points["8b_prefill_2048_frac"] = round(tps, 1), round(frac, 4)
        _, tps, frac = big.portion(7680, 512, pk)
        points["8b_portion_512_behind_7680_tok_s"], points["8b_portion_512_behind_7680_frac"] = round(tps, 1), round(frac, 4)
        for ctx in (4096, 8192):
            for b in (1, 8, 64):
                ms_b, _, nb = big.decode(b, ctx, 16, 4, 1)
                points[f"8b_decode_b{b}_ctx{ctx}"] = round(b / (ms_b / 1e3), 1)
                points[f"8b_decode_b{b}_ctx{ctx}_frac"] = round(nb / (ms_b / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        windows += big.windows
        big.close()
        big = Bench(dict(MODEL_32B, num_hidden_layers=LAYERS_32B), 72, 4096 + 64, 66 * ((4096 + 64 + page - 1) // page) + 8, page, seed=2)
        ms_m, nb, fl = big.mixed(64, 4096, 2048, 1024, 16, 4)
        points["32b_layers"], points["32b_layers_full"] = LAYERS_32B, MODEL_32B["num_hidden_layers"]
        points["32b_mixed_step_ms"] = round(ms_m, 3)
        points["32b_mixed_decode_tok_s"] = round(64 / (ms_m / 1e3), 1)
        points["32b_mixed_prefill_tok_s"] = round(1024 / (ms_m / 1e3), 1)
        points["32b_mixed_hbm_frac"] = round(nb / (ms_m / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        points["32b_mixed_flops_frac"] = round(fl / (ms_m / 1e3) / (pk["bf16_tflops"] * 1e12), 4)
        windows += big.windows
        big.close()
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
                   "hbm_peak_gbs": pk["hbm_gbs"], "bf16_peak_tflops": pk["bf16_tflops"],
                   "timed": f"median of {REPEATS} runs of {K} steps"},
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
    return 0


if __name__ == "__main__":
    sys.exit(main())
