"""Parts that this architecture does not have, defined and registered here, in the test, and run through the
framework's model, cache and step function as they are: a feed-forward that routes every token to one of a few
small experts, and a position encoding with scaled positions.  They stand for what another architecture would bring;
they are toys and no model of anyone's."""
import json
import os

import pytest
import torch

import plain_qwen3 as plain
import tiny_models

pytestmark = pytest.mark.gpu


def test_a_toy_feed_forward_with_routing_can_be_registered_built_and_stepped(tmp_path):
    """Top-1 routing over four experts: router logits and their softmax in float32, the token goes to the expert with
    the largest logit and its output is scaled by that expert's probability.  The part names its tensors per expert,
    the loader checks them, the random-weights writer fills them; the model's other parts are the framework's own.
    Steps that cut the sequence anywhere and put another request beside it must give what one whole step gives, and
    the part alone must give what a loop over tokens gives."""
    from cppvllm_b200.config.registry import register_architecture, unregister_architecture
    from cppvllm_b200.engine.runner import ModelRunner, StepEntry
    from cppvllm_b200.parts.base import FeedForward, WeightSpec, register_part, unregister_part
    from cppvllm_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
    from cppvllm_b200.weights.random_init import write_random_model
    from cppvllm_b200.weights.safetensors_io import SafetensorsFile

    class RoutedFFN(FeedForward):
        def __init__(self, runtime, prefix="", names=None, *, hidden_size, expert_size, num_experts):
            super().__init__(runtime, prefix, names)
            self.D, self.I, self.E = hidden_size, expert_size, num_experts
            self.router = self.w_in = self.w_out = None

        def weight_specs(self):
            specs = {self.full_name("router.weight"): WeightSpec((self.E, self.D))}
            for e in range(self.E):
                specs[self.full_name(f"experts.{e}.in.weight")] = WeightSpec((self.I, self.D))
                specs[self.full_name(f"experts.{e}.out.weight")] = WeightSpec((self.D, self.I))
            return specs

        def bind(self, tensors):
            self.router = tensors[self.full_name("router.weight")].float()
            self.w_in = torch.stack([tensors[self.full_name(f"experts.{e}.in.weight")] for e in range(self.E)]).float()
            self.w_out = torch.stack([tensors[self.full_name(f"experts.{e}.out.weight")] for e in range(self.E)]).float()

        def forward(self, x, ctx):
            xf = x.float()
            prob = torch.softmax(xf @ self.router.t(), dim=-1)                  # router logits and softmax in float32
            gate, expert = prob.max(dim=-1)
            out = torch.zeros_like(xf)
            for e in range(self.E):                                              # tokens of one expert run together
                rows = (expert == e).nonzero().flatten()
                if rows.numel():
                    out[rows] = torch.relu(xf[rows] @ self.w_in[e].t()) @ self.w_out[e].t() * gate[rows, None]
            return out.to(x.dtype)

    def build(cfg):
        D, V, H, KV, hd = cfg["hidden_size"], cfg["vocab_size"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
        layers = [LayerSpec(
            mixer=PartSpec("paged_attention", dict(hidden_size=D, num_heads=H, num_kv_heads=KV, head_dim=hd, qk_norm=True,
                                                   qk_norm_eps=1e-6, position="rope"), prefix=f"toy.layers.{i}.attn."),
            ffn=PartSpec("routed_toy", dict(hidden_size=D, expert_size=cfg["expert_size"], num_experts=cfg["num_experts"]),
                         prefix=f"toy.layers.{i}.moe."),
            mixer_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-6), prefix=f"toy.layers.{i}.norm1."),
            ffn_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-6), prefix=f"toy.layers.{i}.norm2.")) for i in range(cfg["num_layers"])]
        return ModelSpec("ToyRoutedForCausalLM", D, V,
                         embedding=PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), prefix="toy.embed."),
                         layers=layers, final_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-6, buffer="head_normed"), prefix="toy.norm."),
                         lm_head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=D), prefix="toy.head."),
                         positions={"rope": PartSpec("rotary", dict(rotary_dim=hd, theta=10000.0, max_positions=256, pairing="half"))},
                         max_positions=256)

    register_part("ffn", "routed_toy", RoutedFFN)
    register_architecture("ToyRoutedForCausalLM", dict, build)
    try:
        cfg = dict(architectures=["ToyRoutedForCausalLM"], hidden_size=48, vocab_size=90, heads=4, kv_heads=2, head_dim=16,
                   expert_size=40, num_experts=4, num_layers=2)
        d = write_random_model(str(tmp_path / "toy"), cfg, seed=5, std=0.3, store_dtype=torch.float32)
        names = SafetensorsFile(os.path.join(d, "model.safetensors")).names()
        assert "toy.layers.1.moe.experts.3.out.weight" in names and "toy.layers.0.moe.router.weight" in names

        def runner():
            return ModelRunner(d, dtype=torch.float32, page_size=16, num_pages=12, max_step_tokens=64, max_seqs=4, max_model_len=128)

        toks = {"a": tiny_models.random_tokens(90, 50, 1), "b": tiny_models.random_tokens(90, 21, 2)}

        def whole(rid):
            rr = runner()
            rr.cache.admit(rid)
            rr.cache.reserve(rid, len(toks[rid]))
            return rr.step([StepEntry(rid, toks[rid], 0, list(range(len(toks[rid]))))]).cpu().clone()

        ref = {k: whole(k) for k in toks}
        r = runner()
        got, fed = {k: [] for k in toks}, {k: 0 for k in toks}
        for step in ([("a", 9), ("b", 2)], [("a", 1), ("b", 13)], [("a", 30)], [("b", 6), ("a", 2)], [("a", 8)]):
            entries = []
            for rid, n in step:
                if rid not in r.cache.leases:
                    r.cache.admit(rid)
                r.cache.reserve(rid, fed[rid] + n)
                entries.append(StepEntry(rid, toks[rid][fed[rid]:fed[rid] + n], fed[rid], list(range(n))))
            out = r.step(entries).cpu()
            o = 0
            for rid, n in step:
                got[rid].append(out[o:o + n].clone())
                o += n
                fed[rid] += n
        r.check_errors()
        for k in toks:
            g = torch.cat(got[k])
            assert g.shape == ref[k].shape
            assert (g - ref[k]).abs().max() < 1e-4 * max(1.0, ref[k].abs().max())

        # the part alone against a loop over tokens; and the router does send tokens to different experts
        ffn = r.model.blocks[0].ffn
        x = torch.randn(23, 48, device=r.device)
        y = ffn.forward(x, None).cpu()
        used = set()
        for t in range(23):
            xt = x[t].cpu().float()
            prob = torch.softmax(xt @ ffn.router.cpu().t(), dim=-1)
            e = int(prob.argmax())
            used.add(e)
            want = torch.relu(xt @ ffn.w_in[e].cpu().t()) @ ffn.w_out[e].cpu().t() * prob[e]
            assert (y[t] - want).abs().max() < 1e-4 * max(1.0, float(want.abs().max()))
        assert len(used) >= 2
    finally:
        unregister_part("ffn", "routed_toy")
        unregister_architecture("ToyRoutedForCausalLM")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_toy_position_encoding_can_be_registered_and_used(model_dirs, dtype, monkeypatch):
    """Rotary tables whose positions are divided by four (positions 0..3 share an angle), as a part of its own kind:
    tiny_c's weights, the framework's attention reading this part's tables.  The plain implementation with the same
    tables gives the reference; with the architecture's own tables the logits differ."""
    from cppvllm_b200.config.model_config import Qwen3Config
    from cppvllm_b200.config.registry import register_architecture, unregister_architecture
    from cppvllm_b200.engine.runner import ModelRunner, StepEntry
    from cppvllm_b200.models.qwen3 import build_qwen3_spec
    from cppvllm_b200.parts.base import PositionEncoding, register_part, unregister_part
    from cppvllm_b200.parts.spec import PartSpec

    FACTOR = 4.0

    def scaled_tables(hd, theta, max_pos):
        idx = torch.arange(0, hd, 2, dtype=torch.float64)
        inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float64), idx / hd).reciprocal()
        angle = torch.outer(torch.arange(max_pos, dtype=torch.float64) / FACTOR, inv_freq)
        return angle.cos().float(), angle.sin().float()

    class ScaledRotary(PositionEncoding):
        def __init__(self, runtime, prefix="", names=None, *, rotary_dim, theta, max_positions):
            super().__init__(runtime, prefix, names)
            self.rotary_dim, self.interleaved = rotary_dim, False
            cos, sin = scaled_tables(rotary_dim, theta, max_positions)
            self.cos, self.sin = cos.contiguous().to(runtime.device), sin.contiguous().to(runtime.device)

    def build(cfg):
        spec = build_qwen3_spec(cfg)
        spec.positions = {"rope": PartSpec("scaled_rotary_toy", dict(rotary_dim=cfg.head_dim, theta=cfg.rope_theta,
                                                                      max_positions=cfg.max_position_embeddings))}
        return spec

    register_part("position", "scaled_rotary_toy", ScaledRotary)
    register_architecture("ToyScaledRopeForCausalLM", Qwen3Config.from_dict, build)
    try:
        name = "tiny_c"
        d = model_dirs[name] + "_toy_scaled_rope"
        os.makedirs(d, exist_ok=True)
        json.dump(dict(tiny_models.config(name), architectures=["ToyScaledRopeForCausalLM"]), open(os.path.join(d, "config.json"), "w"))
        if not os.path.exists(os.path.join(d, "model.safetensors")):
            os.symlink(os.path.join(model_dirs[name], "model.safetensors"), os.path.join(d, "model.safetensors"))
        act = "float32" if dtype == torch.float32 else "bfloat16"
        toks = tiny_models.random_tokens(tiny_models.config(name)["vocab_size"], 90, 12)
        own = plain.forward(model_dirs[name], toks, act)
        monkeypatch.setattr(plain, "rope_tables", scaled_tables)
        ref = plain.forward(model_dirs[name], toks, act)
        assert (own - ref).abs().max() > 1e-2                      # the encoding matters
        r = ModelRunner(d, dtype=dtype, page_size=16, num_pages=12, max_step_tokens=128, max_seqs=4, max_model_len=256)
        r.cache.admit("a")
        got, pos = [], 0
        for n in (50, 3, 1, 1, 35):                                # a portion, a short one, decoded tokens, the rest
            r.cache.reserve("a", pos + n)
            got.append(r.step([StepEntry("a", toks[pos:pos + n], pos, list(range(n)))]).float().cpu().clone())
            pos += n
        r.check_errors()
        got = torch.cat(got)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert (got - ref).abs().max() <= tol * max(1.0, float(ref.abs().max()))
    finally:
        unregister_part("position", "scaled_rotary_toy")
        unregister_architecture("ToyScaledRopeForCausalLM")


def test_a_toy_mixer_with_a_latent_cache_can_be_registered_built_and_stepped(tmp_path):
    """A mixer that keeps ONE vector per token instead of keys and values: the token's latent z = x Wdown^T goes into
    pages of shape [page, width] (CacheSpec((width,), token_axis=0)), and the output is softmax attention of a query
    over the latents of the positions so far, projected back up.  Layer 0 has this mixer, layer 1 the framework's own
    attention: two groups of pages with different entries side by side, each with its own block tables.  Steps that
    cut the sequences anywhere, put two requests beside one another and reuse the pages of a finished request must give
    what a plain whole-sequence computation gives."""
    from cppvllm_b200.config.registry import register_architecture, unregister_architecture
    from cppvllm_b200.engine.runner import ModelRunner, StepEntry
    from cppvllm_b200.parts.base import CacheSpec, Mixer, WeightSpec, register_part, unregister_part
    from cppvllm_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
    from cppvllm_b200.weights.random_init import write_random_model
    from cppvllm_b200.weights.safetensors_io import SafetensorsFile

    class LatentMixer(Mixer):
        capturable = False                                   # reads the step's positions on the host

        def __init__(self, runtime, prefix="", names=None, *, hidden_size, width):
            super().__init__(runtime, prefix, names)
            self.D, self.C = hidden_size, width

        def cache_spec(self):
            return CacheSpec((self.C,), token_axis=0)

        def weight_specs(self):
            return {self.full_name("down.weight"): WeightSpec((self.C, self.D)), self.full_name("query.weight"): WeightSpec((self.C, self.D)),
                    self.full_name("up.weight"): WeightSpec((self.D, self.C))}

        def bind(self, tensors):
            self.down, self.query, self.up = (tensors[self.full_name(n + ".weight")].float() for n in ("down", "query", "up"))

        def forward(self, x, ctx, cache, state):
            g = ctx.groups[cache.group]
            xf = x.float()
            z, q = xf @ self.down.t(), xf @ self.query.t()
            flat = cache.pages.view(-1, self.C)              # [pages * page_size, width]: slot = page * page_size + offset
            flat[g.slot_mapping[:x.shape[0]].long()] = z.to(flat.dtype)
            pos, seq = ctx.positions[:x.shape[0]].tolist(), ctx.seq_of_token[:x.shape[0]].tolist()
            out = torch.empty_like(z)
            for t in range(x.shape[0]):
                idx = torch.arange(pos[t] + 1, device=x.device)
                slots = g.block_tables[seq[t], idx // g.page_size].long() * g.page_size + idx % g.page_size
                lat = flat[slots].float()
                out[t] = torch.softmax(lat @ q[t] / self.C ** 0.5, 0) @ lat
            return (out @ self.up.t()).to(x.dtype)

    def build(cfg):
        D, V, C = cfg["hidden_size"], cfg["vocab_size"], cfg["latent_width"]
        norms = lambda i: dict(mixer_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-6), prefix=f"toy.layers.{i}.norm1."),
                               ffn_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-6), prefix=f"toy.layers.{i}.norm2."),
                               ffn=PartSpec("swiglu", dict(hidden_size=D, intermediate_size=cfg["inter"]), prefix=f"toy.layers.{i}.mlp."))
        layers = [LayerSpec(mixer=PartSpec("latent_toy", dict(hidden_size=D, width=C), prefix="toy.layers.0.latent."), **norms(0)),
                  LayerSpec(mixer=PartSpec("paged_attention", dict(hidden_size=D, num_heads=4, num_kv_heads=2, head_dim=16, qk_norm=True,
                                                                   qk_norm_eps=1e-6, position="rope"), prefix="toy.layers.1.attn."), **norms(1))]
        return ModelSpec("ToyLatentForCausalLM", D, V,
                         embedding=PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), prefix="toy.embed."),
                         layers=layers, final_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-6, buffer="head_normed"), prefix="toy.norm."),
                         lm_head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=D), prefix="toy.head."),
                         positions={"rope": PartSpec("rotary", dict(rotary_dim=16, theta=10000.0, max_positions=256, pairing="half"))},
                         max_positions=256)

    register_part("mixer", "latent_toy", LatentMixer)
    register_architecture("ToyLatentForCausalLM", dict, build)
    try:
        cfg = dict(architectures=["ToyLatentForCausalLM"], hidden_size=48, vocab_size=90, latent_width=24, inter=64)
        d = write_random_model(str(tmp_path / "toy"), cfg, seed=9, std=0.3, store_dtype=torch.float32)
        assert "toy.layers.0.latent.down.weight" in SafetensorsFile(os.path.join(d, "model.safetensors")).names()

        def runner(pages):
            return ModelRunner(d, dtype=torch.float32, page_size=16, num_pages=pages, max_step_tokens=64, max_seqs=4, max_model_len=128)

        r = runner(8)
        shapes = sorted(tuple(s.shape[2:]) for s in r.storage)
        assert shapes == [(2, 2, 16, 16), (16, 24)]          # attention's keys and values; the latents
        toks = {"a": tiny_models.random_tokens(90, 50, 1), "b": tiny_models.random_tokens(90, 21, 2), "c": tiny_models.random_tokens(90, 40, 3)}

        def whole(rid):
            rr = runner(8)
            rr.cache.admit(rid)
            rr.cache.reserve(rid, len(toks[rid]))
            return rr.step([StepEntry(rid, toks[rid], 0, list(range(len(toks[rid]))))]).cpu().clone()

        ref = {k: whole(k) for k in toks}
        # the latent layer alone against a plain loop on the CPU
        mix = r.model.blocks[0].mixer
        got, fed = {k: [] for k in toks}, {k: 0 for k in toks}
        # 8 pages of 16 tokens: "a" (50) and "b" (21) take 6; "c" (40) fits only once "a" has ended and given back its pages
        plan = ([("a", 9), ("b", 2)], [("a", 1), ("b", 13)], [("a", 30)], [("b", 6), ("a", 2)], [("a", 8)], "end a",
                [("c", 17)], [("c", 2)], [("c", 21)])
        for step in plan:
            if step == "end a":
                r.cache.release("a")
                continue
            entries = []
            for rid, n in step:
                if rid not in r.cache.leases:
                    r.cache.admit(rid)
                r.cache.reserve(rid, fed[rid] + n)
                entries.append(StepEntry(rid, toks[rid][fed[rid]:fed[rid] + n], fed[rid], list(range(n))))
            out = r.step(entries).cpu()
            o = 0
            for rid, n in step:
                got[rid].append(out[o:o + n].clone())
                o += n
                fed[rid] += n
        r.check_errors()
        for k in toks:
            g_ = torch.cat(got[k])
            assert g_.shape == ref[k].shape
            assert (g_ - ref[k]).abs().max() < 1e-4 * max(1.0, ref[k].abs().max())
        # the mixer's arithmetic itself: whole sequence "b" through the plain formula
        x = torch.randn(21, 48)
        z, q = x @ mix.down.cpu().t(), x @ mix.query.cpu().t()
        want = torch.stack([torch.softmax(z[:t + 1] @ q[t] / 24 ** 0.5, 0) @ z[:t + 1] for t in range(21)]) @ mix.up.cpu().t()
        rr = runner(8)
        import test_parts_gpu
        ctx = test_parts_gpu.one_sequence_context(rr, list(range(21)), rid="y")
        view = next(v for v in rr.cache_views.values() if v.spec.entry_shape == (24,))
        y = rr.model.blocks[0].mixer.forward(x.to(rr.device), ctx, view, None).cpu()
        assert (y - want).abs().max() < 1e-4 * max(1.0, float(want.abs().max()))
    finally:
        unregister_part("mixer", "latent_toy")
        unregister_architecture("ToyLatentForCausalLM")


def test_a_toy_norm_and_a_toy_arrangement_can_be_registered_built_and_stepped(tmp_path):
    """Another norm (it subtracts the mean, divides by the standard deviation, scales and shifts: two tensors) and another
    arrangement of a layer (mixer and feed-forward both read the same normed input and are added to the stream together),
    defined here and named in a model specification.  The mixer and the feed-forward are the framework's own.  The
    engine in steps that cut two requests anywhere against one whole step each, and the whole step against a plain
    computation of the same formulas on the CPU."""
    from cppvllm_b200.config.registry import register_architecture, unregister_architecture
    from cppvllm_b200.engine.runner import ModelRunner, StepEntry
    from cppvllm_b200.parts.base import Block, Norm, WeightSpec, register_part, unregister_part
    from cppvllm_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
    from cppvllm_b200.weights.random_init import write_random_model

    class CentredNorm(Norm):
        def __init__(self, runtime, prefix="", names=None, *, size, eps):
            super().__init__(runtime, prefix, names)
            self.size, self.eps = size, eps

        def weight_specs(self):
            return {self.full_name("scale"): WeightSpec((self.size,), role="vector", init="norm"),
                    self.full_name("shift"): WeightSpec((self.size,), role="vector")}

        def bind(self, tensors):
            self.scale, self.shift = tensors[self.full_name("scale")], tensors[self.full_name("shift")]

        def forward(self, x, out=None):
            xf = x.float()
            y = (xf - xf.mean(-1, keepdim=True)) * torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + self.eps) * self.scale + self.shift
            if out is not None:
                out.copy_(y)
                return out
            return y.to(x.dtype)

        def add_forward(self, residual, delta, out=None):
            residual.add_(delta)
            return self.forward(residual, out)

    class ParallelBlock(Block):
        """h <- h + mixer(norm(h)) + ffn(norm(h)): one norm, both branches read it."""
        def __init__(self, runtime, prefix="", names=None, *, mixer, ffn, mixer_norm, ffn_norm):
            super().__init__(runtime, prefix, names)
            self.mixer, self.ffn, self.norm = mixer, ffn, mixer_norm

        def parts(self):
            return (self.norm, self.mixer, self.ffn)

        def forward(self, h, pending, ctx, cache, state):
            x = self.norm.forward(h) if pending is None else self.norm.add_forward(h, pending)
            a = self.mixer.forward(x, ctx, cache, state)
            m = self.ffn.forward(x, ctx)
            return h, a + m

    D, V, H, KV, hd, I = 48, 90, 4, 2, 16, 64

    def build(cfg):
        layers = [LayerSpec(
            mixer=PartSpec("paged_attention", dict(hidden_size=D, num_heads=H, num_kv_heads=KV, head_dim=hd, qk_norm=False, position="rope"),
                           prefix=f"toy.layers.{i}.attn."),
            ffn=PartSpec("swiglu", dict(hidden_size=D, intermediate_size=I), prefix=f"toy.layers.{i}.mlp."),
            mixer_norm=PartSpec("centred_toy", dict(size=D, eps=1e-5), prefix=f"toy.layers.{i}.norm."),
            ffn_norm=PartSpec("centred_toy", dict(size=D, eps=1e-5), prefix=f"toy.layers.{i}.unused_norm."),
            block="parallel_toy") for i in range(2)]
        return ModelSpec("ToyParallelForCausalLM", D, V,
                         embedding=PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), prefix="toy.embed."),
                         layers=layers, final_norm=PartSpec("centred_toy", dict(size=D, eps=1e-5), prefix="toy.norm."),
                         lm_head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=D), prefix="toy.head."),
                         positions={"rope": PartSpec("rotary", dict(rotary_dim=hd, theta=10000.0, max_positions=256, pairing="half"))},
                         max_positions=256)

    register_part("norm", "centred_toy", CentredNorm)
    register_part("block", "parallel_toy", ParallelBlock)
    register_architecture("ToyParallelForCausalLM", dict, build)
    try:
        d = write_random_model(str(tmp_path / "toy"), dict(architectures=["ToyParallelForCausalLM"]), seed=4, std=0.3,
                               store_dtype=torch.float32)

        def runner():
            return ModelRunner(d, dtype=torch.float32, page_size=16, num_pages=12, max_step_tokens=64, max_seqs=4, max_model_len=128)

        toks = {"a": tiny_models.random_tokens(V, 50, 1), "b": tiny_models.random_tokens(V, 21, 2)}

        def whole(rid):
            rr = runner()
            rr.cache.admit(rid)
            rr.cache.reserve(rid, len(toks[rid]))
            return rr.step([StepEntry(rid, toks[rid], 0, list(range(len(toks[rid]))))]).cpu().clone()

        ref = {k: whole(k) for k in toks}
        r = runner()
        got, fed = {k: [] for k in toks}, {k: 0 for k in toks}
        for step in ([("a", 9), ("b", 2)], [("a", 1), ("b", 13)], [("a", 30)], [("b", 6), ("a", 2)], [("a", 8)]):
            entries = []
            for rid, n in step:
                if rid not in r.cache.leases:
                    r.cache.admit(rid)
                r.cache.reserve(rid, fed[rid] + n)
                entries.append(StepEntry(rid, toks[rid][fed[rid]:fed[rid] + n], fed[rid], list(range(n))))
            out = r.step(entries).cpu()
            o = 0
            for rid, n in step:
                got[rid].append(out[o:o + n].clone())
                o += n
                fed[rid] += n
        r.check_errors()
        for k in toks:
            assert (torch.cat(got[k]) - ref[k]).abs().max() < 1e-4 * max(1.0, ref[k].abs().max())

        # the whole step against the same formulas on the CPU
        from cppvllm_b200.weights.safetensors_io import SafetensorsFile
        f = SafetensorsFile(os.path.join(d, "model.safetensors"))
        w = {n: f.tensor(n).float() for n in f.names()}

        def cnorm(x, p):
            return (x - x.mean(-1, keepdim=True)) * torch.rsqrt(x.var(-1, unbiased=False, keepdim=True) + 1e-5) * w[p + "scale"] + w[p + "shift"]

        t = torch.tensor(toks["b"])
        T = len(t)
        cos, sin = plain.rope_tables(hd, 10000.0, 256)
        pos = torch.arange(T)
        h = w["toy.embed.weight"][t]
        for i in range(2):
            p = f"toy.layers.{i}."
            x = cnorm(h, p + "norm.")
            q = plain.apply_rope((x @ w[p + "attn.q_proj.weight"].t()).view(T, H, hd), cos, sin, pos, "float32")
            kk = plain.apply_rope((x @ w[p + "attn.k_proj.weight"].t()).view(T, KV, hd), cos, sin, pos, "float32")
            v = (x @ w[p + "attn.v_proj.weight"].t()).view(T, KV, hd)
            a = plain.attention(q, kk, v, "float32").reshape(T, -1) @ w[p + "attn.o_proj.weight"].t()
            m = plain.swiglu(x @ w[p + "mlp.gate_proj.weight"].t(), x @ w[p + "mlp.up_proj.weight"].t(), "float32") @ w[p + "mlp.down_proj.weight"].t()
            h = h + a + m
        want = cnorm(h, "toy.norm.") @ w["toy.head.weight"].t()
        assert (ref["b"] - want).abs().max() < 1e-4 * max(1.0, float(want.abs().max()))
    finally:
        unregister_part("norm", "centred_toy")
        unregister_part("block", "parallel_toy")
        unregister_architecture("ToyParallelForCausalLM")
