"""Parts that the framework does not have, defined here and registered from outside: a mixer with a
state of its own (a running mean over the sequence, kept in the per-request state slots), a block
arrangement with four norms (one before and one after each of its two parts), a feed-forward that
routes every token over three small experts, a position encoding that rotates neighbouring pairs
(and so takes the attention's general path, outside the fused kernels), an input part that scales
the embeddings and an output part that scales and caps the logits, in a toy architecture
whose run order names a layer twice and lets a layer read another layer's cache.  The model is
built, stepped whole, in portions and mixed with other requests, and compared with a plain float64
computation written in this file.  No file of the framework is changed for it."""

import json
import math

import pytest
import torch

from plain_qwen3 import F64, plain_mlp, plain_rmsnorm
from replay_util import collect, random_tokens, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, HEADS, KV_HEADS, HEAD_DIM, INTER, EPS, THETA, MAX_POS = 48, 101, 4, 2, 16, 80, 1e-5, 10000.0, 128
SCORE_SLOPE = 0.25        # head h of the toy attention adds -SCORE_SLOPE / 2^h per position of distance to its scores
EMBED_SCALE, LOGIT_SCALE, LOGIT_CAP = 3.0, 0.5, 2.0
EXPERTS, EXPERT_INTER, ROUTER_SHARPNESS = 3, 24, 4.0


def toy_classes():
    from zephyr_b200.cache import StateCacheSpec
    from zephyr_b200.config import (FeedForwardSpec, InputSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                                    OutputSpec, PositionSpec)
    from zephyr_b200.kernels import ops
    from zephyr_b200.parts import NORMS, Block, FeedForward, InputPart, Mixer, OutputPart, PositionEncoding, lookup
    from zephyr_b200.weights import WeightDecl
    from zephyr_b200.weights.loader import ROLE_NORM

    class NeighbourPairRope(PositionEncoding):
        """Rotates the pairs (2i, 2i + 1) of every head by position * theta^(-2i / head_dim).  It offers
        no rotation tables, so the attention applies it through ``apply`` and runs its own norm and
        cache-write kernels around it.  It is also a bias on the scores: query head h adds
        -slope / 2^h for every position between the query and the key."""

        def __init__(self, spec, dtype, device):
            self.head_dim = spec.head_dim
            index = torch.arange(0, spec.head_dim, 2, dtype=torch.float32)
            self.inv_freq = (float(spec.params["theta"]) ** (-index / spec.head_dim)).to(device)
            self.slopes = torch.tensor([float(spec.params["slope"]) / 2 ** h for h in range(int(spec.params["heads"]))],
                                       dtype=torch.float32, device=device)

        def as_score_slopes(self):
            return self.slopes

        def apply(self, x, heads, positions, status):
            T = x.shape[0]
            pairs = x.view(T, heads, self.head_dim // 2, 2).float()
            angle = positions.to(torch.float32)[:, None] * self.inv_freq[None, :]
            c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            rotated = torch.stack([pairs[..., 0] * c - pairs[..., 1] * s, pairs[..., 1] * c + pairs[..., 0] * s], dim=-1)
            x.copy_(rotated.view(T, heads * self.head_dim).to(x.dtype))
            return x

    class SoftRoutedExperts(FeedForward):
        """y = sum_e softmax(sharpness * (x R^T))_e * down_e(silu(gate_e x) * up_e x): a router and a
        handful of small experts, every token weighting all of them."""

        def __init__(self, spec, weights, dtype):
            p = spec.params
            self.router, self.sharpness = weights[p["router"]], float(p["sharpness"])
            self.experts = [tuple(weights[f"{p['prefix']}.{e}.{name}.weight"] for name in ("gate_proj", "up_proj", "down_proj"))
                            for e in range(int(p["experts"]))]

        @staticmethod
        def weight_decls(spec):
            p = spec.params
            decls = {p["router"]: WeightDecl((p["experts"], p["hidden_size"]))}
            for e in range(int(p["experts"])):
                decls[f"{p['prefix']}.{e}.gate_proj.weight"] = WeightDecl((p["intermediate_size"], p["hidden_size"]))
                decls[f"{p['prefix']}.{e}.up_proj.weight"] = WeightDecl((p["intermediate_size"], p["hidden_size"]))
                decls[f"{p['prefix']}.{e}.down_proj.weight"] = WeightDecl((p["hidden_size"], p["intermediate_size"]))
            return decls

        def forward(self, x):
            share = torch.softmax(ops.linear(x, self.router, out_dtype=torch.float32) * self.sharpness, dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e, (gate, up, down) in enumerate(self.experts):
                hidden = ops.silu_mul(torch.cat([ops.linear(x, gate), ops.linear(x, up)], dim=1))
                out += share[:, e:e + 1] * ops.linear(hidden, down).float()
            return out.to(x.dtype)

    class SandwichBlock(Block):
        """r = x + post_mixer(mixer(pre_mixer(x))); x' = r + post_ffn(ffn(pre_ffn(r))): four norms."""

        norm_names = ("pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward")

        def __init__(self, mixer, feed_forward, norms):
            self.mixer, self.feed_forward, self.norms = mixer, feed_forward, dict(norms)

        def forward(self, stream, ctx, call):
            x = stream.flush()
            x = x + self.norms["post_mixer"].forward(self.mixer.forward(self.norms["pre_mixer"].forward(x), ctx, call))
            x = x + self.norms["post_feed_forward"].forward(
                self.feed_forward.forward(self.norms["pre_feed_forward"].forward(x)))
            stream.hidden = x
            return stream

    class ScaledEmbedding(InputPart):
        """h = scale * E[id]."""

        def __init__(self, spec, weights, dtype):
            self.table, self.scale = weights[spec.params["weight"]], float(spec.params["scale"])

        @staticmethod
        def weight_decls(spec):
            return {spec.params["weight"]: WeightDecl((spec.params["vocab_size"], spec.params["hidden_size"]), "embedding")}

        def forward(self, ctx):
            return (ops.embedding(self.table, ctx.token_ids, ctx.status).float() * self.scale).to(self.table.dtype)

    class CappedHead(OutputPart):
        """logits = cap * tanh(scale * (norm(h) W^T) / cap)."""

        def __init__(self, spec, weights, dtype):
            p = spec.params
            self.norm = lookup(NORMS, "norm", p["norm"].kind)(p["norm"], weights, dtype)
            self.weight, self.scale, self.cap = weights[p["weight"]], float(p["scale"]), float(p["cap"])

        @staticmethod
        def weight_decls(spec):
            p = spec.params
            return {**lookup(NORMS, "norm", p["norm"].kind).weight_decls(p["norm"]),
                    p["weight"]: WeightDecl((p["vocab_size"], p["hidden_size"]))}

        def forward(self, stream, ctx):
            rows = ops.gather_rows(stream.flush(), ctx.logit_tokens, ctx.status)
            logits = ops.linear(self.norm.forward(rows), self.weight, out_dtype=torch.float32)
            return self.cap * torch.tanh(logits * (self.scale / self.cap))

    class RunningMeanMixer(Mixer):
        """y_t = W * mean(x_0 .. x_t) + b (a projection with a bias, which the one architecture has
        not).  The state is the running sum, one float32 vector per request."""

        def __init__(self, spec, weights, dtype, device):
            self.weight = weights[spec.params["proj"]]
            self.bias = weights[spec.params["proj_bias"]]
            self.hidden = spec.params["hidden_size"]

        @staticmethod
        def weight_decls(spec):
            return {spec.params["proj"]: WeightDecl((spec.params["hidden_size"], spec.params["hidden_size"])),
                    spec.params["proj_bias"]: WeightDecl((spec.params["hidden_size"],), ROLE_NORM)}

        @staticmethod
        def cache_spec(spec):
            return StateCacheSpec(shape=(spec.params["hidden_size"],), dtype="float32")

        def forward(self, x, ctx, call):
            state = ctx.caches[call.cache]
            means = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            start = 0
            for n, before, slot in zip(ctx.host_q_len, ctx.host_ctx, ctx.host_slots):
                sums = state[slot] + torch.cumsum(x[start:start + n].float(), dim=0)
                counts = torch.arange(before + 1, before + n + 1, device=x.device, dtype=torch.float32)
                means[start:start + n] = sums / counts[:, None]
                if call.writes_cache:
                    state[slot] = sums[-1]
                start += n
            return ops.linear(means.to(x.dtype), self.weight, bias=self.bias)

    class ToyConfig:
        model_type, architecture = "toy_mix", "ToyMixForCausalLM"

        @classmethod
        def from_dict(cls, config, where="config.json"):
            assert config["model_type"] == cls.model_type
            return cls()

        def to_dict(self):
            return {"model_type": self.model_type, "architectures": [self.architecture]}

        def to_model_spec(self):
            position = PositionSpec("toy_neighbour_rope", HEAD_DIM, MAX_POS, {"theta": THETA, "slope": SCORE_SLOPE, "heads": HEADS})

            def norm(name):
                return NormSpec("rmsnorm", HIDDEN, EPS, name)

            def ffn(prefix):
                return FeedForwardSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": INTER,
                                                  "gate_proj": f"{prefix}.gate_proj.weight",
                                                  "up_proj": f"{prefix}.up_proj.weight",
                                                  "down_proj": f"{prefix}.down_proj.weight"})

            def attention(prefix):
                return MixerSpec("attention", {
                    "hidden_size": HIDDEN, "num_heads": HEADS, "num_kv_heads": KV_HEADS, "head_dim": HEAD_DIM,
                    "window": 0, "qk_norm_eps": EPS, "q_proj": f"{prefix}.q_proj.weight",
                    "k_proj": f"{prefix}.k_proj.weight", "v_proj": f"{prefix}.v_proj.weight",
                    "o_proj": f"{prefix}.o_proj.weight", "q_norm": f"{prefix}.q_norm.weight",
                    "k_norm": f"{prefix}.k_norm.weight"}, position)

            layers = []
            for index in range(3):
                prefix = f"toy.layers.{index}"
                mixer = (MixerSpec("running_mean", {"hidden_size": HIDDEN, "proj": f"{prefix}.mean.proj.weight",
                                                    "proj_bias": f"{prefix}.mean.proj.bias"})
                         if index == 1 else attention(f"{prefix}.attn"))
                if index == 1:      # the stateful mixer, and the routed feed-forward
                    routed = FeedForwardSpec("toy_soft_experts", {
                        "hidden_size": HIDDEN, "intermediate_size": EXPERT_INTER, "experts": EXPERTS,
                        "sharpness": ROUTER_SHARPNESS, "router": f"{prefix}.router.weight", "prefix": f"{prefix}.experts"})
                    layers.append(LayerSpec("prenorm_residual", mixer, routed,
                                            {"mixer": norm(f"{prefix}.norm1.weight"),
                                             "feed_forward": norm(f"{prefix}.norm2.weight")}))
                    continue
                if index == 2:      # the arrangement with four norms
                    layers.append(LayerSpec("toy_sandwich", mixer, ffn(f"{prefix}.mlp"), {
                        "pre_mixer": norm(f"{prefix}.norm1.weight"), "post_mixer": norm(f"{prefix}.norm1b.weight"),
                        "pre_feed_forward": norm(f"{prefix}.norm2.weight"),
                        "post_feed_forward": norm(f"{prefix}.norm2b.weight")}))
                    continue
                layers.append(LayerSpec("prenorm_residual", mixer, ffn(f"{prefix}.mlp"),
                                        {"mixer": norm(f"{prefix}.norm1.weight"),
                                         "feed_forward": norm(f"{prefix}.norm2.weight")}))
            run_order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2),        # layer 0 runs twice, own caches
                         LayerCall(2, 0, writes_cache=False),                     # layer 2 reads the cache of call 0
                         LayerCall(1, 3))                                         # the stateful layer again, own state
            return ModelSpec(
                "ToyMixForCausalLM", VOCAB, HIDDEN, MAX_POS,
                InputSpec("toy_scaled_embedding", {"weight": "toy.embed.weight", "vocab_size": VOCAB,
                                                   "hidden_size": HIDDEN, "scale": EMBED_SCALE}),
                tuple(layers), run_order,
                OutputSpec("toy_capped_head", {"norm": norm("toy.norm.weight"), "weight": "toy.head.weight",
                                               "vocab_size": VOCAB, "hidden_size": HIDDEN, "scale": LOGIT_SCALE,
                                               "cap": LOGIT_CAP}))

    return RunningMeanMixer, ToyConfig, SandwichBlock, ScaledEmbedding, CappedHead, NeighbourPairRope, SoftRoutedExperts


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from zephyr_b200.config import register_architecture, unregister_architecture
    from zephyr_b200.parts import (BLOCKS, FEED_FORWARDS, INPUTS, MIXERS, OUTPUTS, POSITION_ENCODINGS, register_block,
                                   register_feed_forward, register_input, register_mixer, register_output,
                                   register_position_encoding)
    from zephyr_b200.weights import write_random_model

    mixer, config, block, embedding, head, rope, experts = toy_classes()
    register_mixer("running_mean", mixer)
    register_position_encoding("toy_neighbour_rope", rope)
    register_feed_forward("toy_soft_experts", experts)
    register_block("toy_sandwich", block)
    register_input("toy_scaled_embedding", embedding)
    register_output("toy_capped_head", head)
    register_architecture(config.model_type, config.architecture, config)
    folders = {}
    for dtype in ("float32", "bfloat16"):
        folders[dtype] = write_random_model(config(), 11, tmp_path_factory.mktemp(f"toy_{dtype}"),
                                            dtype=getattr(torch, dtype))
    yield folders
    unregister_architecture(config.architecture)
    MIXERS.pop("running_mean", None)
    BLOCKS.pop("toy_sandwich", None)
    INPUTS.pop("toy_scaled_embedding", None)
    OUTPUTS.pop("toy_capped_head", None)
    POSITION_ENCODINGS.pop("toy_neighbour_rope", None)
    FEED_FORWARDS.pop("toy_soft_experts", None)


# ------------------------------------------------------------- the plain computation
def plain_toy_logits(folder, tokens):
    from safetensors import safe_open

    w = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as handle:
        for name in handle.keys():
            w[name] = handle.get_tensor(name).to(F64)
    T = len(tokens)
    index = torch.arange(0, HEAD_DIM, 2, dtype=torch.float32)
    angle = (torch.arange(T, dtype=torch.float32)[:, None] * (THETA ** (-index / HEAD_DIM))[None, :]).to(F64)
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]

    def rotate(v):          # pairs (2i, 2i + 1) of every head
        pairs = v.view(T, v.shape[1], HEAD_DIM // 2, 2)
        return torch.stack([pairs[..., 0] * cos - pairs[..., 1] * sin, pairs[..., 1] * cos + pairs[..., 0] * sin],
                           dim=-1).view(v.shape)

    x = EMBED_SCALE * w["toy.embed.weight"][torch.tensor(tokens)]

    def qkv(h, prefix):
        q = rotate(plain_rmsnorm((h @ w[f"{prefix}.q_proj.weight"].T).view(T, HEADS, HEAD_DIM),
                                 w[f"{prefix}.q_norm.weight"], EPS))
        k = rotate(plain_rmsnorm((h @ w[f"{prefix}.k_proj.weight"].T).view(T, KV_HEADS, HEAD_DIM),
                                 w[f"{prefix}.k_norm.weight"], EPS))
        v = (h @ w[f"{prefix}.v_proj.weight"].T).view(T, KV_HEADS, HEAD_DIM)
        return q, k, v

    def sloped_attention(q, k, v):       # causal, grouped, with the encoding's bias on the scores
        out = torch.zeros_like(q)
        t, u = torch.arange(T)[:, None], torch.arange(T)[None, :]
        for head in range(HEADS):
            kv_head = head // (HEADS // KV_HEADS)
            scores = (q[:, head, :] @ k[:, kv_head, :].T) / math.sqrt(HEAD_DIM) + (SCORE_SLOPE / 2 ** head) * (u - t).to(F64)
            out[:, head, :] = torch.softmax(scores.masked_fill(u > t, float("-inf")), dim=-1) @ v[:, kv_head, :]
        return out

    def finish(x, mixed, index):
        r = x + mixed
        return r + plain_mlp(plain_rmsnorm(r, w[f"toy.layers.{index}.norm2.weight"], EPS), w, f"toy.layers.{index}.mlp")

    def attention_layer(x, index, kv=None):
        h = plain_rmsnorm(x, w[f"toy.layers.{index}.norm1.weight"], EPS)
        q, k, v = qkv(h, f"toy.layers.{index}.attn")
        if kv is not None:
            k, v = kv
        out = sloped_attention(q, k, v).reshape(T, HEADS * HEAD_DIM) @ w[f"toy.layers.{index}.attn.o_proj.weight"].T
        if index == 2:      # four norms: one more after each part
            prefix = f"toy.layers.{index}"
            r = x + plain_rmsnorm(out, w[f"{prefix}.norm1b.weight"], EPS)
            fed = plain_mlp(plain_rmsnorm(r, w[f"{prefix}.norm2.weight"], EPS), w, f"{prefix}.mlp")
            return r + plain_rmsnorm(fed, w[f"{prefix}.norm2b.weight"], EPS), (k, v)
        return finish(x, out, index), (k, v)

    def mean_layer(x, index):
        prefix = f"toy.layers.{index}"
        h = plain_rmsnorm(x, w[f"{prefix}.norm1.weight"], EPS)
        means = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=F64)[:, None]
        r = x + means @ w[f"{prefix}.mean.proj.weight"].T + w[f"{prefix}.mean.proj.bias"]
        fed = plain_rmsnorm(r, w[f"{prefix}.norm2.weight"], EPS)
        share = torch.softmax(fed @ w[f"{prefix}.router.weight"].T * ROUTER_SHARPNESS, dim=-1)
        out = sum(share[:, e:e + 1] * plain_mlp(fed, w, f"{prefix}.experts.{e}") for e in range(EXPERTS))
        return r + out

    x, kv0 = attention_layer(x, 0)
    x = mean_layer(x, 1)
    x, _ = attention_layer(x, 0)
    x, _ = attention_layer(x, 2, kv=kv0)
    x = mean_layer(x, 1)
    logits = plain_rmsnorm(x, w["toy.norm.weight"], EPS) @ w["toy.head.weight"].T
    return (LOGIT_CAP * torch.tanh(logits * (LOGIT_SCALE / LOGIT_CAP))).numpy()


def test_toy_architecture_is_found_and_built(toy_folder, cuda_device):
    from zephyr_b200.cache import PagedCacheSpec, StateCacheSpec
    from zephyr_b200.config import load_model_spec
    from zephyr_b200.parts import Model
    from zephyr_b200.weights import Checkpoint

    spec = load_model_spec(toy_folder["float32"])
    model = Model.load(spec, Checkpoint(toy_folder["float32"]), torch.float32, cuda_device)
    kinds = [type(s).__name__ for s in model.cache_specs]
    assert kinds == ["PagedCacheSpec", "StateCacheSpec", "PagedCacheSpec", "StateCacheSpec"]
    assert len(model.layers) == 3 and len(spec.run_order) == 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_toy_model_under_every_cutting(toy_folder, cuda_device, dtype, mode):
    from zephyr_b200.engine.replay import TraceReplayer
    from replay_util import peak_tokens

    folder = toy_folder[dtype]
    requests = {f"t{i}": random_tokens(VOCAB, n, seed=50 + i) for i, n in enumerate((40, 75, 9, 128, 33, 60))}
    steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions, "mixed": trace_mixed}[mode](requests)
    replayer = TraceReplayer(folder, dtype, peak_tokens(steps), page_size=8, max_requests=4)
    replayer.runner.poison_freed_pages = True
    outputs = {}
    for step in steps:
        result = replayer.step(step)
        if result is not None:
            outputs[step["step"]] = result
        replayer.runner.manager.check_invariants()
    rows = collect(steps, outputs)
    tolerance = 1e-4 if dtype == "float32" else 0.03
    expected = {rid: plain_toy_logits(folder, tokens) for rid, tokens in requests.items()}
    worst = 0.0
    for (rid, position), got in sorted(rows.items()):
        error = float(abs(got - expected[rid][position]).max())
        worst = max(worst, error)
        assert error <= tolerance, f"{mode} {dtype}: request {rid} position {position}: {error:.3e}"
    assert replayer.runner.manager.slots.num_free == 4          # every state slot came back
