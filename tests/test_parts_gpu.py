"""Each part of a layer alone on the GPU against the plain function of the same name, with the tiny models'
weights; and parts composed in ways the architecture itself does not use (a window, a layer run twice, a layer
that reads another layer's cache), to show that the run list and the parameters are data."""
import json
import os

import pytest
import torch

import plain_qwen3 as plain
import tiny_models

pytestmark = pytest.mark.gpu


def make_runner(model_dir, dtype, page, **kw):
    from cppvllm_b200.engine.runner import ModelRunner
    args = dict(dtype=dtype, page_size=page, num_pages=24, max_step_tokens=256, max_seqs=8, max_model_len=256,
                enforce_eager=True)
    args.update(kw)
    return ModelRunner(model_dir, **args)


def one_sequence_context(r, toks, rid="s"):
    from cppvllm_b200.engine.runner import StepEntry
    r.cache.admit(rid)
    r.cache.reserve(rid, len(toks))
    e = [StepEntry(rid, toks, 0, list(range(len(toks))))]
    W = len(r.cache.lease(rid).tables[0])
    lay, T, S, R = r._fill(e, len(toks), 1, len(toks), W)
    return r._context(lay, T, S, R, W, [len(toks)], len(toks))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_parts_alone(model_dirs, name, dtype):
    d = model_dirs[name]
    act = "float32" if dtype == torch.float32 else "bfloat16"
    cfg, w = plain.read_config(d), plain.read_weights(d)
    if act == "bfloat16":
        w = {k: plain.rnd(v, act) for k, v in w.items()}
    r = make_runner(d, dtype, tiny_models.page_size(name))
    T = 45
    toks = tiny_models.random_tokens(cfg["V"], T, 9)
    ctx = one_sequence_context(r, toks)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    m = r.model
    # embedding
    h = m.embedding.forward(ctx.tokens, T)
    ref_h = plain.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    torch.testing.assert_close(h.float().cpu(), ref_h, atol=0, rtol=0)
    # norm, alone and fused with the residual add
    blk = m.blocks[1]
    p = "model.layers.1."
    x = blk.mixer_norm.forward(h).clone()
    ref_x = plain.rms_norm(ref_h, w[p + "input_layernorm.weight"], cfg["eps"], act)
    torch.testing.assert_close(x.float().cpu(), ref_x, **tol)
    delta = (torch.randn(T, cfg["D"]) * 0.1).to(dtype)
    h2 = h.clone()
    x2 = blk.ffn_norm.add_forward(h2, delta.to(r.device)).clone()
    ref_h2 = plain.rnd(ref_h + delta.float(), act)
    torch.testing.assert_close(h2.float().cpu(), ref_h2, atol=0, rtol=0)
    torch.testing.assert_close(x2.float().cpu(), plain.rms_norm(ref_h2, w[p + "post_attention_layernorm.weight"], cfg["eps"], act), **tol)
    # rotary tables
    cos, sin = plain.rope_tables(cfg["hd"], cfg["theta"], cfg["max_pos"])
    rope = m.positions["rope"]
    torch.testing.assert_close(rope.cos.cpu(), cos, atol=0, rtol=0)
    torch.testing.assert_close(rope.sin.cpu(), sin, atol=0, rtol=0)
    # mixer (attention) on the normed input, through the paged cache
    xin = ref_x.to(dtype).to(r.device)
    a = blk.mixer.forward(xin, ctx, r.cache_views[1], None).clone()
    H, KV, hd = cfg["H"], cfg["KV"], cfg["hd"]
    pos = torch.arange(T)
    xin_f = xin.float().cpu()
    q = plain.linear(xin_f, w[p + "self_attn.q_proj.weight"], act).view(T, H, hd)
    k = plain.linear(xin_f, w[p + "self_attn.k_proj.weight"], act).view(T, KV, hd)
    v = plain.linear(xin_f, w[p + "self_attn.v_proj.weight"], act).view(T, KV, hd)
    q = plain.apply_rope(plain.qk_norm(q, w[p + "self_attn.q_norm.weight"], cfg["eps"], act), cos, sin, pos, act)
    k = plain.apply_rope(plain.qk_norm(k, w[p + "self_attn.k_norm.weight"], cfg["eps"], act), cos, sin, pos, act)
    ref_a = plain.linear(plain.attention(q, k, v, act).reshape(T, H * hd), w[p + "self_attn.o_proj.weight"], act)
    torch.testing.assert_close(a.float().cpu(), ref_a, **tol)
    # the keys and values it left in the pages
    lease = r.cache.lease("s")
    pages = r.cache_views[1].pages
    ps = r.page_size
    got_k = torch.stack([pages[lease.tables[0][t // ps], 0, :, t % ps] for t in range(T)]).float().cpu()
    got_v = torch.stack([pages[lease.tables[0][t // ps], 1, :, t % ps] for t in range(T)]).float().cpu()
    torch.testing.assert_close(got_k, k, **tol)
    torch.testing.assert_close(got_v, v, **tol)
    # feed-forward
    f = blk.ffn.forward(xin, ctx)
    g_, u_ = plain.linear(xin_f, w[p + "mlp.gate_proj.weight"], act), plain.linear(xin_f, w[p + "mlp.up_proj.weight"], act)
    torch.testing.assert_close(f.float().cpu(), plain.linear(plain.swiglu(g_, u_, act), w[p + "mlp.down_proj.weight"], act), **tol)
    # head
    y = ref_x[:7].to(dtype).to(r.device).contiguous()
    out = torch.empty(7, cfg["V"], dtype=torch.float32, device=r.device)
    m.head.forward(y, out)
    head_w = w["model.embed_tokens.weight"] if cfg["tie"] else w["lm_head.weight"]
    torch.testing.assert_close(out.cpu(), plain.lm_head(y.float().cpu(), head_w), **tol)
    r.check_errors()


def test_layers_differ_and_the_run_list_is_data(model_dirs):
    """A toy arrangement registered from the test: tiny_b's weights, but layer 0 has a window of 24 positions
    (its pages form a group of their own and are given back as the window passes), layer 1 runs twice (second time
    with a cache unit of its own), and layer 2 computes queries only and reads the cache of the first run of layer 1."""
    from cppvllm_b200.config.model_config import Qwen3Config
    from cppvllm_b200.config.registry import register_architecture, unregister_architecture
    from cppvllm_b200.engine.runner import StepEntry
    from cppvllm_b200.models.qwen3 import build_qwen3_spec
    from cppvllm_b200.parts.spec import RunEntry

    def build(cfg):
        spec = build_qwen3_spec(cfg)
        spec.layers[0].mixer.params["window"] = 24
        spec.run_order = [RunEntry(0), RunEntry(1, cache=7), RunEntry(1), RunEntry(2, cache=7, writes_cache=False)]
        return spec

    register_architecture("ToyWindowedForCausalLM", Qwen3Config.from_dict, build)
    try:
        d = model_dirs["tiny_b"] + "_toy_windowed"
        os.makedirs(d, exist_ok=True)
        cfg = dict(tiny_models.TINY_B, architectures=["ToyWindowedForCausalLM"])
        json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
        if not os.path.exists(os.path.join(d, "model.safetensors")):
            os.symlink(os.path.join(model_dirs["tiny_b"], "model.safetensors"), os.path.join(d, "model.safetensors"))
        r = make_runner(d, torch.float32, 16, num_pages=12)
        assert len(r.group_specs) == 2 and sorted(len(m) for _, m in r.group_specs) == [1, 2]
        win_group = [g for g, (cs, _) in enumerate(r.group_specs) if cs.window == 24][0]
        toks = tiny_models.random_tokens(320, 150, 4)

        ref = _toy_reference(model_dirs["tiny_b"], toks)
        r.cache.admit("a")
        got, pos = [], 0
        for n in (40, 3, 2, 30, 1, 1, 1, 50, 22):
            r.cache.reserve("a", pos + n)
            got.append(r.step([StepEntry("a", toks[pos:pos + n], pos, list(range(n)))]).cpu().clone())
            pos += n
            # the windowed group holds at most what the window and one page's slack need
            held = sum(1 for p in r.cache.lease("a").tables[win_group] if p >= 0)
            assert held <= (24 + 15) // 16 + 1
        r.check_errors()
        got = torch.cat(got)
        assert (got - ref).abs().max() < 1e-5 * max(1.0, ref.abs().max())
        r.cache.release("a")
        r.cache.check_invariants()
    finally:
        unregister_architecture("ToyWindowedForCausalLM")


@pytest.mark.parametrize("prefill_kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("window", [24, 150])
def test_windowed_layers_in_bfloat16_through_the_tensor_core_kernels(model_dirs, window, prefill_kernel):
    """tiny_c's weights (head size 64: the tensor-core attention kernels) with a window on every layer, pages of 16
    tokens, bfloat16.  The prompt comes in portions longer than the window plus a page, so from the second portion on the
    request has given back pages that lie below the window (their table entries are -1) while the kernels' first key tile
    still starts below it; then single tokens are decoded past the window.  Logits against the plain windowed model;
    no kernel may report a missing page."""
    from cppvllm_b200.config.model_config import Qwen3Config
    from cppvllm_b200.config.registry import register_architecture, unregister_architecture
    from cppvllm_b200.engine.runner import StepEntry
    from cppvllm_b200.models.qwen3 import build_qwen3_spec

    def build(cfg):
        spec = build_qwen3_spec(cfg)
        for layer in spec.layers:
            layer.mixer.params["window"] = window
            layer.mixer.params["prefill_kernel"] = prefill_kernel
        return spec

    arch = f"ToyWindowed{window}{prefill_kernel}ForCausalLM"
    register_architecture(arch, Qwen3Config.from_dict, build)
    try:
        d = model_dirs["tiny_c"] + f"_toy_windowed_{window}_{prefill_kernel}"
        os.makedirs(d, exist_ok=True)
        json.dump(dict(tiny_models.TINY_C, architectures=[arch]), open(os.path.join(d, "config.json"), "w"))
        if not os.path.exists(os.path.join(d, "model.safetensors")):
            os.symlink(os.path.join(model_dirs["tiny_c"], "model.safetensors"), os.path.join(d, "model.safetensors"))
        cuts = (60, 45, 70, 2, 41) if window == 24 else (180, 170, 2, 30)
        n_decode = 40
        toks = tiny_models.random_tokens(200, sum(cuts) + n_decode, 8)
        r = make_runner(d, torch.bfloat16, 16, num_pages=40, max_step_tokens=256, max_model_len=512)
        ref = _windowed_reference(model_dirs["tiny_c"], toks, window, "bfloat16")
        r.cache.admit("a")
        got, pos, freed = [], 0, 0
        for n in cuts + (1,) * n_decode:
            r.cache.reserve("a", pos + n)
            got.append(r.step([StepEntry("a", toks[pos:pos + n], pos, list(range(n)))]).float().cpu().clone())
            pos += n
            table = r.cache.lease("a").tables[0]
            freed = max(freed, sum(1 for i, p in enumerate(table) if p < 0 and i * 16 < pos))
            r.check_errors()                                 # after every step: a missing page would show at once
        assert freed >= (pos - window) // 16 - 1             # pages below the window really went back
        got = torch.cat(got)
        assert (got - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))
        r.cache.release("a")
        r.cache.check_invariants()
    finally:
        unregister_architecture(arch)


def test_a_parts_options_are_data(model_dirs, monkeypatch):
    """A part's options travel in the specification (LayerSpec.mixer.params).  tiny_c's layers with the decode steps'
    one-kernel attention switched off and the mma.sync prompt kernel chosen: the engine then runs other kernels (counted),
    and the logits agree with the default choice to rounding, over a prompt cut into portions, decoded tokens and a
    second request beside them."""
    from cppvllm_b200.config.model_config import Qwen3Config
    from cppvllm_b200.config.registry import register_architecture, unregister_architecture
    from cppvllm_b200.csrc import ops
    from cppvllm_b200.engine.runner import StepEntry
    from cppvllm_b200.models.qwen3 import build_qwen3_spec

    def build(cfg):
        spec = build_qwen3_spec(cfg)
        for layer in spec.layers:
            layer.mixer.params["fuse_decode_attention"] = False
            layer.mixer.params["prefill_kernel"] = "mma"
        return spec

    calls = {"fused": 0, "mma": 0, "tcgen05": 0}
    for key, fn_name in (("fused", "attn_decode_fused_bf16"), ("mma", "attn_prefill_bf16"), ("tcgen05", "attn_prefill_tcgen05")):
        fn = getattr(ops, fn_name)
        monkeypatch.setattr(ops, fn_name, lambda *a, _fn=fn, _k=key, **k: (calls.__setitem__(_k, calls[_k] + 1), _fn(*a, **k))[1])
    register_architecture("ToyOptionsForCausalLM", Qwen3Config.from_dict, build)
    try:
        name = "tiny_c"
        d = model_dirs[name] + "_toy_options"
        os.makedirs(d, exist_ok=True)
        cfg = dict(tiny_models.config(name), architectures=["ToyOptionsForCausalLM"])
        json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
        if not os.path.exists(os.path.join(d, "model.safetensors")):
            os.symlink(os.path.join(model_dirs[name], "model.safetensors"), os.path.join(d, "model.safetensors"))
        vocab = cfg["vocab_size"]
        a, b = tiny_models.random_tokens(vocab, 60, 5), tiny_models.random_tokens(vocab, 23, 6)
        plan = [[("a", 40)], [("a", 5)], [("a", 2), ("b", 6)], [("a", 1), ("b", 1)], [("b", 16)], [("a", 8)], [("a", 1)],
                [("a", 3)]]
        results, counted = [], []
        for folder in (model_dirs[name], d):
            for k in calls:
                calls[k] = 0
            r = make_runner(folder, torch.bfloat16, tiny_models.page_size(name), enforce_eager=True)
            pos = {"a": 0, "b": 0}
            seqs = {"a": a, "b": b}
            for rid in pos:
                r.cache.admit(rid)
            got = []
            for step in plan:
                entries = []
                for rid, n in step:
                    r.cache.reserve(rid, pos[rid] + n)
                    entries.append(StepEntry(rid, seqs[rid][pos[rid]:pos[rid] + n], pos[rid], list(range(n))))
                    pos[rid] += n
                got.append(r.step(entries).float().cpu().clone())
            r.check_errors()
            results.append(torch.cat(got))
            counted.append(dict(calls))
        default, toy = counted
        assert default["fused"] > 0 and default["tcgen05"] > 0 and default["mma"] == 0
        assert toy["fused"] == 0 and toy["tcgen05"] == 0 and toy["mma"] > 0
        ref, other = results
        assert (other - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))
    finally:
        unregister_architecture("ToyOptionsForCausalLM")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_steps_of_a_repeated_shape_replay_a_graph_and_stay_right(model_dirs, dtype):
    """The second step of a shape (portion lengths, wanted rows) is captured, later ones replay the capture: a prompt
    cut into equal portions beside a second request, other tokens, positions, pages and wanted rows every time.  Every
    logit row is compared with the plain implementation, and a runner that never captures gives the same rows."""
    name = "tiny_c"
    d = model_dirs[name]
    act = "float32" if dtype == torch.float32 else "bfloat16"
    from cppvllm_b200.engine.runner import StepEntry
    vocab = tiny_models.config(name)["vocab_size"]
    a, b = tiny_models.random_tokens(vocab, 400, 31), tiny_models.random_tokens(vocab, 120, 32)
    ref = {"a": plain.forward(d, a, act), "b": plain.forward(d, b, act)}
    # shapes: (80,), (80,), (80,) [graph from the 2nd on], (64, 16) x 3 mixed, (80,) again, then (70,) once (eager)
    plan = [[("a", 80, [0, 79])], [("a", 80, [5, 79])], [("a", 80, [40, 41])], [("a", 64, [63, 1]), ("b", 16, [15])],
            [("b", 64, [0, 63]), ("a", 16, [3])], [("a", 64, [10, 20]), ("b", 16, [0])], [("b", 24, [23])]]
    got = {}
    for eager in (False, True):
        r = make_runner(d, dtype, tiny_models.page_size(name), num_pages=40, max_model_len=512, enforce_eager=eager)
        pos, seqs, rows = {"a": 0, "b": 0}, {"a": a, "b": b}, []
        for rid in pos:
            r.cache.admit(rid)
        for step in plan:
            entries = []
            for rid, n, want in step:
                r.cache.reserve(rid, pos[rid] + n)
                entries.append(StepEntry(rid, seqs[rid][pos[rid]:pos[rid] + n], pos[rid], want))
            out = r.step(entries).float().cpu().clone()
            k = 0
            for rid, n, want in step:
                for w in want:
                    rows.append((rid, pos[rid] + w, out[k]))
                    k += 1
                pos[rid] += n
        r.check_errors()
        got[eager] = rows
        if not eager:
            assert r.stats["graph_steps"] == 4           # the 2nd and 3rd (80,), the 2nd and 3rd (64, 16)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for (rid, p_, row), (_, _, row_e) in zip(got[False], got[True]):
        want = ref[rid][p_]
        scale = max(1.0, float(want.abs().max()))
        assert (row - want).abs().max() <= tol * scale
        assert (row - row_e).abs().max() <= tol * scale


def _windowed_reference(d, toks, window, act):
    """The plain model (tests/plain_qwen3.py, same rounding places) with every layer's attention limited to the last
    `window` positions."""
    c, w = plain.read_config(d), plain.read_weights(d)
    if act == "bfloat16":
        w = {k: plain.rnd(t, act) for k, t in w.items()}
    T = len(toks)
    cos, sin = plain.rope_tables(c["hd"], c["theta"], c["max_pos"])
    pos = torch.arange(T)
    H, KV, hd, eps = c["H"], c["KV"], c["hd"], c["eps"]
    h = plain.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    far = (pos[:, None] - pos[None, :]) >= window            # [query, key]: the key has left the window
    future = pos[None, :] > pos[:, None]
    for l in range(c["L"]):
        p = f"model.layers.{l}."
        x = plain.rms_norm(h, w[p + "input_layernorm.weight"], eps, act)
        q = plain.apply_rope(plain.qk_norm(plain.linear(x, w[p + "self_attn.q_proj.weight"], act).view(T, H, hd),
                                           w[p + "self_attn.q_norm.weight"], eps, act), cos, sin, pos, act)
        k = plain.apply_rope(plain.qk_norm(plain.linear(x, w[p + "self_attn.k_proj.weight"], act).view(T, KV, hd),
                                           w[p + "self_attn.k_norm.weight"], eps, act), cos, sin, pos, act)
        v = plain.linear(x, w[p + "self_attn.v_proj.weight"], act).view(T, KV, hd)
        att = torch.empty(T, H, hd)
        for hh in range(H):
            g = hh // (H // KV)
            s_ = (q[:, hh] @ k[:, g].t()) / hd ** 0.5
            s_ = s_.masked_fill(far | future, float("-inf"))
            att[:, hh] = torch.softmax(s_, -1) @ v[:, g]
        att = plain.rnd(att, act)
        h = plain.rnd(h + plain.linear(att.reshape(T, -1), w[p + "self_attn.o_proj.weight"], act), act)
        x = plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps, act)
        m = plain.linear(plain.swiglu(plain.linear(x, w[p + "mlp.gate_proj.weight"], act), plain.linear(x, w[p + "mlp.up_proj.weight"], act), act),
                         w[p + "mlp.down_proj.weight"], act)
        h = plain.rnd(h + m, act)
    y = plain.rms_norm(h, w["model.norm.weight"], eps, act)
    return plain.lm_head(y, w["model.embed_tokens.weight"] if c["tie"] else w["lm_head.weight"])


def _toy_reference(d, toks):
    """Plain float32 forward of the toy arrangement above."""
    c, w = plain.read_config(d), plain.read_weights(d)
    T = len(toks)
    cos, sin = plain.rope_tables(c["hd"], c["theta"], c["max_pos"])
    pos = torch.arange(T)
    H, KV, hd, eps = c["H"], c["KV"], c["hd"], c["eps"]
    h = plain.embedding(w["model.embed_tokens.weight"], torch.tensor(toks))
    kept = {}
    for i, (l, window, reads) in enumerate([(0, 24, None), (1, 0, None), (1, 0, None), (2, 0, 1)]):
        p = f"model.layers.{l}."
        x = plain.rms_norm(h, w[p + "input_layernorm.weight"], eps, "float32")
        q = plain.apply_rope(plain.qk_norm((x @ w[p + "self_attn.q_proj.weight"].t()).view(T, H, hd),
                                           w[p + "self_attn.q_norm.weight"], eps, "float32"), cos, sin, pos, "float32")
        if reads is not None:
            k, v = kept[reads]
        else:
            k = plain.apply_rope(plain.qk_norm((x @ w[p + "self_attn.k_proj.weight"].t()).view(T, KV, hd),
                                               w[p + "self_attn.k_norm.weight"], eps, "float32"), cos, sin, pos, "float32")
            v = (x @ w[p + "self_attn.v_proj.weight"].t()).view(T, KV, hd)
            kept[i] = (k, v)
        att = torch.empty(T, H, hd)
        for t in range(T):
            lo = max(0, t - window + 1) if window else 0
            for hh in range(H):
                g = hh // (H // KV)
                s = (k[lo:t + 1, g] @ q[t, hh]) / hd ** 0.5
                att[t, hh] = torch.softmax(s, 0) @ v[lo:t + 1, g]
        h = h + att.reshape(T, -1) @ w[p + "self_attn.o_proj.weight"].t()
        x = plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps, "float32")
        h = h + plain.swiglu(x @ w[p + "mlp.gate_proj.weight"].t(), x @ w[p + "mlp.up_proj.weight"].t(), "float32") @ w[p + "mlp.down_proj.weight"].t()
    y = plain.rms_norm(h, w["model.norm.weight"], eps, "float32")
    return y @ w["lm_head.weight"].t()
