"""Command lines in the reference's manner: ``example <model_dir>`` and ``bench <model_dir>``.

The reference's programs take only the model folder and keep everything else in the source (example.cpp:13-48:
two chat prompts, temperature 0.6, 512 new tokens; bench.cpp:10-63: 256 requests, prompt lengths and output
lengths uniform in [100, 1024], token ids uniform in [0, 10000], temperature 0.6, ``ignore_eos``, generator seed 0,
``max_num_batched_tokens`` 4096, ``gpu_memory_utilization`` 0.80, a warm-up request of 8 tokens).  The same defaults
hold here; every engine option is additionally a flag named like the field of ``EngineConfig``.  There is no
tokenizer: ``example`` takes prompts as comma-separated token ids.
"""
from __future__ import annotations

import argparse
import random
import sys
import time


def _engine_flags(p: argparse.ArgumentParser, util: float) -> None:
    p.add_argument("model_dir", help="folder with config.json and *.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--max-num-batched-tokens", type=int, default=4096)
    p.add_argument("--max-num-seqs", type=int, default=256)
    p.add_argument("--max-chunk-tokens", type=int, default=1024)
    p.add_argument("--max-model-len", type=int, default=4096)
    p.add_argument("--gpu-memory-utilization", type=float, default=util)
    p.add_argument("--num-kv-blocks", type=int, default=-1)
    p.add_argument("--block-size", type=int, default=32)
    p.add_argument("--enforce-eager", action="store_true")
    p.add_argument("--enable-prefix-caching", action="store_true")
    p.add_argument("--use-ref-kernels", action="store_true")
    p.add_argument("--python-runtime", action="store_true",
                   help="the cache manager and the scheduler in Python (their plain twins) instead of C++")
    p.add_argument("--seed", type=int, default=0)


def _engine(args):
    from .config.engine_config import EngineConfig
    from .engine.llm_engine import LLMEngine
    return LLMEngine(EngineConfig(
        model_path=args.model_dir, dtype=args.dtype, max_num_batched_tokens=args.max_num_batched_tokens,
        max_num_seqs=args.max_num_seqs, max_chunk_tokens=args.max_chunk_tokens, max_model_len=args.max_model_len,
        gpu_memory_utilization=args.gpu_memory_utilization, num_kv_blocks=args.num_kv_blocks,
        block_size=args.block_size, enforce_eager=args.enforce_eager, enable_prefix_caching=args.enable_prefix_caching,
        use_ref_kernels=args.use_ref_kernels, native_cache_manager=not args.python_runtime,
        native_scheduler=not args.python_runtime, seed=args.seed))


def example_main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="example", description="generate completions for prompts given as token ids")
    _engine_flags(p, 0.90)
    p.add_argument("--prompt", action="append", default=None,
                   help="comma-separated token ids; may be given several times (default: two short prompts)")
    p.add_argument("--temperature", type=float, default=0.6)
    p.add_argument("--max-tokens", type=int, default=512)
    p.add_argument("--ignore-eos", action="store_true")
    if argv is None and len(sys.argv) < 2:
        print("usage: example <model_dir>", file=sys.stderr)
        return 2
    args = p.parse_args(argv)
    from .sampling.params import SamplingParams
    llm = _engine(args)
    vocab = llm.runner.vocab_size
    prompts = ([[int(t) for t in s.split(",") if t.strip()] for s in args.prompt] if args.prompt
               else [[(7 * i + 3) % vocab for i in range(12)], [(11 * i + 5) % vocab for i in range(9)]])
    params = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    outs = llm.generate(prompts, params)
    for prompt, o in zip(prompts, outs):
        print("\n")
        print(f"Prompt: {prompt}")
        print(f"Completion: {o.token_ids}" + ("  (stopped on EOS)" if o.stopped_on_eos else ""))
    return 0


def bench_main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="bench", description="throughput of 256 requests with random lengths")
    _engine_flags(p, 0.80)
    p.add_argument("--num-seqs", type=int, default=256)
    p.add_argument("--max-input-len", type=int, default=1024)
    p.add_argument("--max-output-len", type=int, default=1024)
    p.add_argument("--min-len", type=int, default=100)
    p.add_argument("--temperature", type=float, default=0.6)
    if argv is None and len(sys.argv) < 2:
        print("usage: bench <model_dir>", file=sys.stderr)
        return 2
    args = p.parse_args(argv)
    from .sampling.params import SamplingParams
    import torch
    llm = _engine(args)
    vocab = llm.runner.vocab_size
    gen = random.Random(0)
    prompts = [[gen.randint(0, min(10000, vocab - 1)) for _ in range(gen.randint(args.min_len, args.max_input_len))]
               for _ in range(args.num_seqs)]
    params = [SamplingParams(temperature=args.temperature, ignore_eos=True,
                             max_tokens=gen.randint(args.min_len, args.max_output_len)) for _ in range(args.num_seqs)]
    llm.generate([[1 % vocab, 2 % vocab, 3 % vocab, 4 % vocab, 5 % vocab, 6 % vocab, 7 % vocab, 8 % vocab]],
                 SamplingParams(max_tokens=16))
    before = llm.stats()
    steps0, pre0 = before.steps, before.preemptions
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for pr, sp in zip(prompts, params):
        llm.add_request(pr, sp)
    while not llm.is_finished():
        llm.step()
    torch.cuda.synchronize()
    t = time.perf_counter() - t0
    llm.take_finished()
    total = sum(sp.max_tokens for sp in params)
    print(f"Total: {total}tok, Time: {t:.2f}s, Throughput: {total / t:.2f}tok/s")
    after = llm.stats()
    print(f"steps: {after.steps - steps0}, preemptions: {after.preemptions - pre0}, KV blocks: {llm.num_kv_blocks}")
    return 0
