"""Generation through the public entry point: greedy against the plain implementation, temperature sampling
that does not depend on batching, scheduling under pressure (portions, preemption and recomputation), the
command lines, and a toy mixer with state of its own that is registered from here."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as plain
import tiny_models

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine(model_dir, name, dtype="float32", **kw):
    from cppvllm_b200 import LLM
    args = dict(dtype=dtype, block_size=tiny_models.page_size(name), num_kv_blocks=64, max_num_batched_tokens=64,
                max_num_seqs=8, max_chunk_tokens=24, max_model_len=256)
    args.update(kw)
    return LLM(model_dir, **args)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_matches_the_plain_implementation(model_dirs, name):
    from cppvllm_b200 import SamplingParams
    d = model_dirs[name]
    vocab = tiny_models.config(name)["vocab_size"]
    prompts = [tiny_models.random_tokens(vocab, n, 20 + n) for n in (5, 17, 33)]
    llm = engine(d, name)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.prompt_ids == p and len(o.token_ids) == 8
        assert o.token_ids == plain.greedy_generate(d, p, 8)
    assert llm.stats().tokens_generated == 24 and llm.stats().steps >= 8
    assert llm.runner.cache.num_free_pages() == 64                  # everything was given back
    llm.runner.cache.check_invariants()


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_bfloat16_greedy_tokens_are_near_arg_maxima_of_the_plain_model(model_dirs, name):
    from cppvllm_b200 import SamplingParams
    d = model_dirs[name]
    vocab = tiny_models.config(name)["vocab_size"]
    prompts = [tiny_models.random_tokens(vocab, n, 40 + n) for n in (1, 31, 65)]
    outs = engine(d, name, "bfloat16").generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        seq = p + o.token_ids
        ref = plain.forward(d, seq[:-1], "bfloat16")
        for i, tok in enumerate(o.token_ids):
            row = ref[len(p) - 1 + i]
            assert row[tok] >= row.max() - 0.02 * max(1.0, float(row.abs().max()))


def test_temperature_sampling_is_reproducible_and_independent_of_batching(model_dirs):
    from cppvllm_b200 import SamplingParams
    d = model_dirs["tiny_b"]
    prompts = [tiny_models.random_tokens(320, n, 60 + n) for n in (1, 31, 32, 65, 100)]
    sp = [SamplingParams(temperature=0.7, max_tokens=12, ignore_eos=True, seed=100 + i) for i in range(5)]
    together = engine(d, "tiny_b", seed=5).generate(prompts, sp)
    again = engine(d, "tiny_b", seed=5).generate(prompts, sp)
    assert [o.token_ids for o in together] == [o.token_ids for o in again]
    alone = engine(d, "tiny_b", seed=5, max_chunk_tokens=0, max_num_batched_tokens=256)
    for i in (4, 0, 2):
        assert alone.generate([prompts[i]], sp[i])[0].token_ids == together[i].token_ids
    other = engine(d, "tiny_b", seed=6).generate(prompts, sp)
    assert [o.token_ids for o in other] != [o.token_ids for o in together]
    greedy = engine(d, "tiny_b").generate(prompts[:2], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    assert greedy[1].token_ids != together[1].token_ids            # temperature 0.7 really samples


@pytest.mark.parametrize("prefix_cache", [False, True])
def test_pages_run_out_requests_are_preempted_recomputed_and_still_right(model_dirs, prefix_cache):
    """With the prefix cache a preempted request may find its first pages again and recompute less; the tokens are the same."""
    from cppvllm_b200 import SamplingParams
    d = model_dirs["tiny_a"]
    prompts = [tiny_models.random_tokens(256, n, 80 + n) for n in (30, 31, 29, 12)]
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    llm = engine(d, "tiny_a", num_kv_blocks=7, enable_prefix_caching=prefix_cache)   # 112 tokens for four requests of up to 51
    outs = llm.generate(prompts, sp)
    assert llm.stats().preemptions > 0
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain.greedy_generate(d, p, 20)
    llm.runner.cache.check_invariants()
    with pytest.raises(ValueError, match="cache pages"):
        llm.add_request(list(range(100)), SamplingParams(max_tokens=50))
    with pytest.raises(ValueError, match="outside the vocabulary"):
        llm.add_request([1, 2, 999], sp)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_that_share_a_prefix_read_the_same_pages_and_generate_the_same_tokens(model_dirs, dtype):
    """With the prefix cache, later requests start behind the registered pages of a common prefix (here also behind
    their own pages after a preemption).  Tokens are those of an engine without it, and in float32 those of the plain
    implementation."""
    from cppvllm_b200 import SamplingParams
    name = "tiny_c"
    d = model_dirs[name]
    vocab = tiny_models.config(name)["vocab_size"]
    stem = tiny_models.random_tokens(vocab, 70, 5)
    prompts = [stem + tiny_models.random_tokens(vocab, n, 60 + n) for n in (3, 9, 1)] + [stem[:49], stem[:48]]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    outs = {}
    for on in (False, True):
        llm = engine(d, name, dtype, enable_prefix_caching=on, max_num_seqs=2)      # two at a time: later ones find pages
        outs[on] = [o.token_ids for o in llm.generate(prompts, sp)]
        llm.runner.check_errors()
        llm.runner.cache.check_invariants()
        assert llm.runner.cache.num_free_pages() == 64
        # pages of 16: the third request finds the stem's four full pages, the 49-token one three, the 48-token one two
        assert llm.stats().prefix_hit_pages == (9 if on else 0)
    if dtype == "float32":
        assert outs[True] == outs[False]
        for p, o in zip(prompts, outs[True]):
            assert o == plain.greedy_generate(d, p, 10)
    else:
        for p, o in zip(prompts, outs[True]):
            ref = plain.forward(d, (p + o)[:-1], "bfloat16")
            for i, tok in enumerate(o):
                row = ref[len(p) - 1 + i]
                assert row[tok] >= row.max() - 0.02 * max(1.0, float(row.abs().max()))


def test_plain_twin_kernels_give_the_same_logits_as_the_fast_ones(model_dirs):
    """use_ref_kernels: the general attention kernel and library products with separate norm and activation kernels, in
    place of the tensor-core attention kernels, the weight-streaming products and the fusions.  Same steps (a prompt
    portion, short portions, decoded tokens of two requests), bfloat16: the logits agree to rounding, and both agree
    with the plain implementation."""
    from cppvllm_b200.csrc import ops
    from cppvllm_b200.engine.runner import ModelRunner, StepEntry
    name = "tiny_c"
    d = model_dirs[name]
    vocab = tiny_models.config(name)["vocab_size"]
    a, b = tiny_models.random_tokens(vocab, 100, 3), tiny_models.random_tokens(vocab, 40, 4)
    ref = {"a": plain.forward(d, a, "bfloat16"), "b": plain.forward(d, b, "bfloat16")}
    plan = [[("a", 70)], [("a", 5), ("b", 30)], [("a", 1), ("b", 1)], [("a", 1), ("b", 1)], [("b", 8)], [("a", 23)]]
    rows = {}
    for twin in (False, True):
        r = ModelRunner(d, dtype=torch.bfloat16, page_size=16, num_pages=24, max_step_tokens=128, max_seqs=4,
                        max_model_len=256, use_ref_kernels=twin)
        before = ops.launches()
        pos, seqs, got = {"a": 0, "b": 0}, {"a": a, "b": b}, []
        for rid in pos:
            r.cache.admit(rid)
        for step in plan:
            entries = []
            for rid, n in step:
                r.cache.reserve(rid, pos[rid] + n)
                entries.append(StepEntry(rid, seqs[rid][pos[rid]:pos[rid] + n], pos[rid], list(range(n))))
            out = r.step(entries).float().cpu().clone()
            k = 0
            for rid, n in step:
                for w in range(n):
                    got.append((rid, pos[rid] + w, out[k]))
                    k += 1
                pos[rid] += n
        r.check_errors()
        rows[twin] = got
        assert ops.launches() > before
    for (rid, p_, fast), (_, _, twin) in zip(rows[False], rows[True]):
        want = ref[rid][p_]
        scale = max(1.0, float(want.abs().max()))
        assert (fast - want).abs().max() <= 2e-2 * scale and (twin - want).abs().max() <= 2e-2 * scale
        assert (fast - twin).abs().max() <= 2e-2 * scale


def test_overlapped_and_step_by_step_engines_generate_the_same_tokens(model_dirs):
    """pipeline_depth 2 schedules step n + 1 before the samples of step n are read back (the tokens travel on the
    device); depth 1 waits for every step.  Same tokens, greedy and sampled, also when pages run out."""
    from cppvllm_b200 import SamplingParams
    d = model_dirs["tiny_b"]
    prompts = [tiny_models.random_tokens(320, n, 70 + n) for n in (1, 31, 32, 65, 100, 7)]
    for kw, sp in ((dict(), SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)),
                   (dict(), SamplingParams(temperature=0.8, max_tokens=9, ignore_eos=True, seed=3)),
                   (dict(num_kv_blocks=7), SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True))):
        outs = {}
        for depth in (1, 2):
            llm = engine(d, "tiny_b", pipeline_depth=depth, **kw)
            outs[depth] = [o.token_ids for o in llm.generate(prompts, sp)]
            llm.runner.cache.check_invariants()
            assert llm.runner.cache.num_free_pages() == llm.num_kv_blocks
            if kw:
                assert llm.stats().preemptions > 0
        assert outs[1] == outs[2]
        assert all(len(t) == sp.max_tokens for t in outs[2])


@pytest.mark.parametrize("prefix_cache", [False, True])
def test_cache_manager_in_cpp_and_in_python_run_the_same_engine(model_dirs, prefix_cache):
    """The engine with the cache manager in C++ (the default) and with its plain twin in Python: the same tokens, the
    same preemptions and prefix hits, and the same pages in every request's table after every step."""
    from cppvllm_b200 import SamplingParams
    from cppvllm_b200.cache.native import NativeCacheManager
    d = model_dirs["tiny_b"]
    stem = tiny_models.random_tokens(320, 70, 5)
    prompts = [stem + tiny_models.random_tokens(320, n, 90 + n) for n in (1, 31, 40, 3)] + [tiny_models.random_tokens(320, 50, 8)]
    sp = SamplingParams(temperature=0.7, max_tokens=24, ignore_eos=True, seed=11)
    llms = [engine(d, "tiny_b", num_kv_blocks=11, enable_prefix_caching=prefix_cache, native_cache_manager=native)
            for native in (True, False)]
    assert isinstance(llms[0].runner.cache, NativeCacheManager) and not isinstance(llms[1].runner.cache, NativeCacheManager)
    for llm in llms:
        for pr in prompts:
            llm.add_request(pr, sp)
    steps = 0
    while not llms[0].is_finished():
        for llm in llms:
            llm.step()
        a, b = (llm.runner.cache for llm in llms)
        assert set(a.leases) == set(b.leases) and a.num_free_pages() == b.num_free_pages()
        for rid in a.leases:
            assert a.block_table(rid, 0) == b.block_table(rid, 0) and a.lease(rid).computed == b.lease(rid).computed
        steps += 1
        assert steps < 500
    assert llms[1].is_finished()
    outs = [sorted((o.request_id, tuple(o.token_ids)) for o in llm.take_finished()) for llm in llms]
    assert outs[0] == outs[1] and len(outs[0]) == len(prompts)
    assert llms[0].stats().preemptions == llms[1].stats().preemptions > 0
    assert llms[0].stats().prefix_hit_pages == llms[1].stats().prefix_hit_pages
    assert (llms[0].stats().prefix_hit_pages > 0) == prefix_cache
    for llm in llms:
        llm.runner.cache.check_invariants()
        assert llm.runner.cache.num_free_pages() == llm.num_kv_blocks


def test_end_of_sequence_stops_a_request(model_dirs, tmp_path):
    from cppvllm_b200 import SamplingParams
    d = model_dirs["tiny_a"]
    p = tiny_models.random_tokens(256, 9, 3)
    ref = plain.greedy_generate(d, p, 6)
    eos_dir = str(tmp_path / "eos")
    os.makedirs(eos_dir)
    cfg = dict(tiny_models.TINY_A, eos_token_id=[ref[3]])
    json.dump(cfg, open(os.path.join(eos_dir, "config.json"), "w"))
    os.symlink(os.path.join(d, "model.safetensors"), os.path.join(eos_dir, "model.safetensors"))
    llm = engine(eos_dir, "tiny_a")
    out = llm.generate([p], SamplingParams(temperature=0.0, max_tokens=6))[0]
    first = ref.index(ref[3])
    assert out.stopped_on_eos and out.token_ids == ref[:first]
    out = llm.generate([p], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))[0]
    assert not out.stopped_on_eos and out.token_ids == ref


def test_command_lines(model_dirs):
    d = model_dirs["tiny_a"]
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "example"), d, "--dtype", "float32", "--max-tokens", "5",
                        "--temperature", "0", "--prompt", "1,2,3", "--max-model-len", "64", "--num-kv-blocks", "16",
                        "--max-num-seqs", "4", "--ignore-eos"], capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert f"Completion: {plain.greedy_generate(d, [1, 2, 3], 5)}" in r.stdout
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bench"), d, "--num-seqs", "6", "--min-len", "5",
                        "--max-input-len", "40", "--max-output-len", "20", "--max-model-len", "64", "--num-kv-blocks", "12",
                        "--max-num-seqs", "4", "--max-num-batched-tokens", "64"], capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "Throughput:" in r.stdout and "KV blocks: 12" in r.stdout
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "example"), d, "--dtype", "float32", "--max-tokens", "5",
                        "--temperature", "0", "--prompt", "1,2,3", "--max-model-len", "64", "--num-kv-blocks", "16",
                        "--max-num-seqs", "4", "--ignore-eos", "--python-runtime"], capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert f"Completion: {plain.greedy_generate(d, [1, 2, 3], 5)}" in r.stdout
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "example")], capture_output=True, text=True, env=env)
    assert r.returncode == 2 and "usage: example <model_dir>" in r.stderr


# ---- a toy mixer with state of its own -----------------------------------------------------------------------

def test_a_toy_mixer_with_its_own_state_can_be_registered_built_and_stepped(tmp_path):
    """The mixer keeps, per request, a decaying sum of its inputs: state_t = 0.5 * state_{t-1} + x_t W, y_t = state_t.
    It is defined, registered and given an architecture here; the framework's files stay as they are.  Steps that
    cut the sequence anywhere, with another request in the batch and a slot that is used again, must give what a
    whole-sequence loop gives."""
    from cppvllm_b200.config.registry import register_architecture, unregister_architecture
    from cppvllm_b200.engine.runner import ModelRunner, StepEntry
    from cppvllm_b200.parts.base import Mixer, StateSpec, WeightSpec, register_part, unregister_part
    from cppvllm_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
    from cppvllm_b200.weights.random_init import write_random_model

    class DecayMixer(Mixer):
        capturable = False          # its loop reads lengths on the host

        def __init__(self, runtime, prefix="", names=None, *, hidden_size, decay):
            super().__init__(runtime, prefix, names)
            self.hidden_size, self.decay, self.w = hidden_size, decay, None

        def state_spec(self):
            return StateSpec((self.hidden_size,), torch.float32)

        def weight_specs(self):
            return {self.full_name("mix.weight"): WeightSpec((self.hidden_size, self.hidden_size))}

        def bind(self, tensors):
            self.w = tensors[self.full_name("mix.weight")]

        def forward(self, x, ctx, cache, state):
            u = x.float() @ self.w.float().t()
            out = torch.empty_like(u)
            cu = ctx.cu_seqlens.tolist()
            slots = ctx.state_slots.tolist()
            for s in range(ctx.num_seqs):
                st = state[slots[s]]
                for t in range(cu[s], cu[s + 1]):
                    st = self.decay * st + u[t]
                    out[t] = st
                state[slots[s]] = st
            return out.to(x.dtype)

    def build(cfg):
        D, V = cfg["hidden_size"], cfg["vocab_size"]
        layers = [LayerSpec(
            mixer=PartSpec("decay_sum", dict(hidden_size=D, decay=0.5), prefix=f"toy.layers.{i}."),
            ffn=PartSpec("swiglu", dict(hidden_size=D, intermediate_size=cfg["intermediate_size"]), prefix=f"toy.layers.{i}.mlp."),
            mixer_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-5), prefix=f"toy.layers.{i}.norm1."),
            ffn_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-5), prefix=f"toy.layers.{i}.norm2.")) for i in range(cfg["num_layers"])]
        return ModelSpec("ToyStateForCausalLM", D, V,
                         embedding=PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), prefix="toy.embed."),
                         layers=layers, final_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-5, buffer="head_normed"), prefix="toy.norm."),
                         lm_head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=D), prefix="toy.head."), max_positions=512)

    register_part("mixer", "decay_sum", DecayMixer)
    register_architecture("ToyStateForCausalLM", dict, build)
    try:
        cfg = dict(architectures=["ToyStateForCausalLM"], hidden_size=48, vocab_size=70, intermediate_size=80, num_layers=2)
        d = write_random_model(str(tmp_path / "toy"), cfg, seed=3, std=0.2, store_dtype=torch.float32)
        r = ModelRunner(d, dtype=torch.float32, page_size=16, num_pages=4, max_step_tokens=64, max_seqs=4, max_model_len=128,
                        num_state_slots=2)
        assert r.group_specs == [] and len(r.states) == 2 and r.states[0].shape == (3, 48)
        toks = {"a": tiny_models.random_tokens(70, 40, 1), "b": tiny_models.random_tokens(70, 25, 2), "c": tiny_models.random_tokens(70, 18, 3)}

        def whole(rid):
            rr = ModelRunner(d, dtype=torch.float32, page_size=16, num_pages=4, max_step_tokens=64, max_seqs=4, max_model_len=128)
            rr.cache.admit(rid)
            return rr.step([StepEntry(rid, toks[rid], 0, list(range(len(toks[rid]))))]).cpu().clone()

        ref = {k: whole(k) for k in toks}
        got = {k: [] for k in toks}
        fed = {k: 0 for k in toks}
        plan = [[("a", 7), ("b", 2)], [("a", 1), ("b", 13)], [("a", 20)], [("b", 10), ("a", 1)], [("a", 11)],   # a, b done
                [("c", 5)], [("c", 1)], [("c", 12)]]                                                          # c reuses a slot
        for step in plan:
            entries = []
            for rid, n in step:
                if rid not in r.cache.leases:
                    r.cache.admit(rid)
                entries.append(StepEntry(rid, toks[rid][fed[rid]:fed[rid] + n], fed[rid], list(range(n))))
            out = r.step(entries).cpu()
            o = 0
            for rid, n in step:
                got[rid].append(out[o:o + n].clone())
                o += n
                fed[rid] += n
                if fed[rid] == len(toks[rid]):
                    r.cache.release(rid)
        for k in toks:
            g = torch.cat(got[k])
            assert g.shape == ref[k].shape
            assert (g - ref[k]).abs().max() < 1e-4 * max(1.0, ref[k].abs().max())
        assert not torch.allclose(ref["a"][5], ref["a"][6])
    finally:
        unregister_part("mixer", "decay_sum")
        unregister_architecture("ToyStateForCausalLM")
