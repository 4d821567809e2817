"""A toy mixer with state of its own, defined here, is registered, built and stepped without a change
to the framework's files: it keeps a decaying sum of its inputs per request in a state slot.  The model
alternates it with the framework's attention, so pages and state slots are used side by side."""
import pytest
import torch

import plain_model
from helpers import assert_close, tokens_for

pytestmark = pytest.mark.gpu
DEVICE = torch.device("cuda:0")
DECAY = 0.7


def register_toy():
    from llmserver_b200.cache import StateNeed
    from llmserver_b200.parts import MIXERS, Mixer
    from llmserver_b200.weights.declare import WeightDecl

    @MIXERS.register("toy_decaying_sum")
    class DecayingSum(Mixer):
        """state <- decay * state + x_t ; out_t = state W^T.  State: one float32 [hidden] row per request."""

        capturable = False        # walks the batch's rows on the host

        @classmethod
        def declare_weights(cls, params):
            return {"mix.weight": WeightDecl((params["hidden"], params["hidden"]))}

        @classmethod
        def cache_need(cls, params):
            return StateNeed((params["hidden"],), "float32")

        def __init__(self, params, weights, runtime):
            super().__init__(params, weights, runtime)
            self.weight, self.decay = weights["mix.weight"].float(), float(params["decay"])

        def forward(self, x, batch, cache):
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            slots, begin = batch.state_slots.tolist(), 0
            for slot, count in zip(slots, batch.q_lens):
                state = cache.state[slot]
                for row in range(begin, begin + count):
                    state.mul_(self.decay).add_(x[row].float())
                    out[row] = state @ self.weight.T
                begin += count
            return out.to(x.dtype)

    return DecayingSum


def toy_spec(hidden=48, vocab=120):
    from llmserver_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    norm = PartSpec.of("rmsnorm", width=hidden, eps=1e-5)
    block = PartSpec.of("pre_norm", mixer_prefix="mixer.", feed_forward_prefix="ffn.", mixer_norm_prefix="norm1.",
                        feed_forward_norm_prefix="norm2.")
    feed_forward = PartSpec.of("swiglu", hidden=hidden, intermediate=80)
    attention = PartSpec.of("gqa_attention", hidden=hidden, heads=3, kv_heads=1, head_dim=16, scale=0.25, qk_norm=True,
                            eps=1e-5, window=None)
    toy = PartSpec.of("toy_decaying_sum", hidden=hidden, decay=DECAY)
    layers = [LayerSpec(f"toy.layers.{i}.", block, mixer, feed_forward, norm, norm, "rotary" if mixer is attention else None)
              for i, mixer in enumerate((attention, toy, attention))]
    return ModelSpec(architecture="ToyForTests", vocab_size=vocab, hidden_size=hidden, layers=layers,
                     schedule=[ScheduleEntry(i) for i in range(3)],
                     positions={"rotary": PartSpec.of("rotary", head_dim=16, theta=10000.0)}, final_norm=norm,
                     embedding_name="toy.embed.weight", final_norm_prefix="toy.norm.", head_name="toy.head.weight")


class MovedSource:
    """Random tensors drawn on the CPU (so the plain side sees the same values), moved to the device."""

    def __init__(self, spec, seed, dtype):
        from llmserver_b200.weights import RandomSource
        self.inner, self.dtype = RandomSource(spec, seed, torch.float32, "cpu"), dtype
        self.seen = {}

    def get(self, name):
        self.seen[name] = self.inner.get(name).to(self.dtype)
        return self.seen[name].to(DEVICE)


def plain_toy_forward(weights, tokens):
    """Whole sequence, no cache: the same model written with the plain functions."""
    w = {name: tensor.double() for name, tensor in weights.items()}
    h = w["toy.embed.weight"][torch.tensor(tokens)]
    cosine, sine = plain_model.rope_tables(torch.arange(len(tokens)), 16, 10000.0, torch.float64)
    for index in range(3):
        p = f"toy.layers.{index}."
        normed = plain_model.rms_norm(h, w[p + "norm1.weight"], 1e-5)
        if index == 1:
            state, rows = torch.zeros(h.shape[1], dtype=torch.float64), []
            for row in normed:
                state = DECAY * state + row
                rows.append(state @ w[p + "mixer.mix.weight"].T)
            mixed = torch.stack(rows)
        else:
            layer = {"self_attn." + k[len(p + "mixer."):]: v for k, v in w.items() if k.startswith(p + "mixer.")}
            q, k, v = plain_model.project_qkv(normed, layer, 3, 1, 16, 1e-5, cosine, sine)
            mixed = plain_model.causal_attention(q, k, v, 0.25) @ layer["self_attn.o_proj.weight"].T
        h = h + mixed
        normed = plain_model.rms_norm(h, w[p + "norm2.weight"], 1e-5)
        h = h + plain_model.swiglu_mlp(normed, {"mlp." + k[len(p + "ffn."):]: v for k, v in w.items() if k.startswith(p + "ffn.")})
    return (plain_model.rms_norm(h, w["toy.norm.weight"], 1e-5) @ w["toy.head.weight"].T).numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    from llmserver_b200.cache import CacheManager, StateNeed
    from llmserver_b200.engine.step import StepFunction
    from llmserver_b200.models import DecoderModel
    from llmserver_b200.parts import Runtime

    register_toy()
    spec = toy_spec()
    source = MovedSource(spec, 5, dtype)
    model = DecoderModel(spec, source, Runtime(dtype, DEVICE))
    needs = model.cache_needs()
    assert isinstance(needs[1], StateNeed) and needs[1].shape == (48,)
    cache = CacheManager(needs, 4, 40, num_slots=2, prefix_sharing=True)
    assert not cache.prefix_sharing           # a mixer with state rules shared prefixes out
    cache.materialize(DEVICE, dtype)
    step = StepFunction(model, cache)
    first, second = tokens_for(120, 37, 1), tokens_for(120, 22, 2)
    want_first, want_second = plain_toy_forward(source.seen, first), plain_toy_forward(source.seen, second)
    name = "float32" if dtype == torch.float32 else "bfloat16"
    # two requests interleaved, cut differently, one of them ended and its slot reused
    step.admit("x")
    step.admit("y")
    got_x = [step.run([("x", first[:20], list(range(20)))])]
    both = step.run([("x", first[20:23], [0, 1, 2]), ("y", second[:9], list(range(9)))])
    got_x.append(both[:3])
    got_y = [both[3:]]
    both = step.run([("y", second[9:10], [0]), ("x", first[23:], list(range(14)))])
    got_y.append(both[:1])
    got_x.append(both[1:])
    step.release("x")
    got_y.append(step.run([("y", second[10:], list(range(12)))]))
    assert_close(torch.cat(got_x).cpu().numpy(), want_first, name, "toy model, request x")
    assert_close(torch.cat(got_y).cpu().numpy(), want_second, name, "toy model, request y")
    step.admit("z")                            # takes x's slot, which must start from zero again
    again = step.run([("z", first, list(range(len(first))))])
    assert_close(again.cpu().numpy(), want_first, name, "toy model, reused slot")
    step.check_errors()
    step.release("y")
    step.release("z")
    cache.check_invariants()


# ---------------------------------------------------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, defined here as well: the model below uses them in
# one layer and the framework's SwiGLU and rotary encoding in the other, through the same registries.

N_EXPERTS = 3


def register_toy_feed_forward_and_position():
    from llmserver_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding
    from llmserver_b200.weights.declare import WeightDecl

    @FEED_FORWARDS.register("toy_top1_experts")
    class Top1Experts(FeedForward):
        """probabilities = softmax(x R^T) in 32-bit; out = p[e] * (x W_e^T) for the likeliest expert e of each token."""

        @classmethod
        def declare_weights(cls, params):
            decls = {"router.weight": WeightDecl((params["experts"], params["hidden"]))}
            for e in range(params["experts"]):
                decls[f"experts.{e}.weight"] = WeightDecl((params["hidden"], params["hidden"]))
            return decls

        def __init__(self, params, weights, runtime):
            super().__init__(params, weights, runtime)
            self.router = weights["router.weight"].float()
            self.experts = [weights[f"experts.{e}.weight"].float() for e in range(params["experts"])]

        def forward(self, x):
            probabilities = torch.softmax(x.float() @ self.router.T, dim=-1)
            weight, chosen = probabilities.max(dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e, expert in enumerate(self.experts):
                rows = (chosen == e).nonzero().flatten()
                if rows.numel():
                    out[rows] = (x[rows].float() @ expert.T) * weight[rows, None]
            return out.to(x.dtype)

    @POSITION_ENCODINGS.register("toy_harmonic_rotary")
    class HarmonicRotary(PositionEncoding):
        """Rotation by position / (1 + i) for pair i: another set of frequencies for the same rotating kernel."""

        def __init__(self, params, weights, runtime):
            super().__init__(params, weights, runtime)
            self.head_dim = int(params["head_dim"])
            self.inv_freq = (1.0 / (1.0 + torch.arange(self.head_dim // 2, dtype=torch.float32))).to(runtime.device)

    return Top1Experts, HarmonicRotary


def routed_spec(hidden=40, vocab=90):
    from llmserver_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    norm = PartSpec.of("rmsnorm", width=hidden, eps=1e-6)
    block = PartSpec.of("pre_norm", mixer_prefix="mixer.", feed_forward_prefix="ffn.", mixer_norm_prefix="norm1.",
                        feed_forward_norm_prefix="norm2.")
    attention = PartSpec.of("gqa_attention", hidden=hidden, heads=2, kv_heads=2, head_dim=16, scale=0.25, qk_norm=True,
                            eps=1e-6, window=None)
    layers = [LayerSpec("toy.layers.0.", block, attention, PartSpec.of("toy_top1_experts", hidden=hidden, experts=N_EXPERTS),
                        norm, norm, "harmonic"),
              LayerSpec("toy.layers.1.", block, attention, PartSpec.of("swiglu", hidden=hidden, intermediate=56), norm, norm, "rotary")]
    return ModelSpec(architecture="ToyRoutedForTests", vocab_size=vocab, hidden_size=hidden, layers=layers,
                     schedule=[ScheduleEntry(0), ScheduleEntry(1)],
                     positions={"rotary": PartSpec.of("rotary", head_dim=16, theta=10000.0),
                                "harmonic": PartSpec.of("toy_harmonic_rotary", head_dim=16)},
                     final_norm=norm, embedding_name="toy.embed.weight", final_norm_prefix="toy.norm.", head_name="toy.head.weight")


def plain_routed_forward(weights, tokens):
    w = {name: tensor.double() for name, tensor in weights.items()}
    h = w["toy.embed.weight"][torch.tensor(tokens)]
    positions = torch.arange(len(tokens), dtype=torch.float64)
    harmonic = positions[:, None] * (1.0 / (1.0 + torch.arange(8, dtype=torch.float32))).double()[None, :]
    tables = [(torch.cos(torch.cat([harmonic, harmonic], dim=-1)), torch.sin(torch.cat([harmonic, harmonic], dim=-1))),
              plain_model.rope_tables(torch.arange(len(tokens)), 16, 10000.0, torch.float64)]
    for index in range(2):
        p = f"toy.layers.{index}."
        normed = plain_model.rms_norm(h, w[p + "norm1.weight"], 1e-6)
        layer = {"self_attn." + k[len(p + "mixer."):]: v for k, v in w.items() if k.startswith(p + "mixer.")}
        q, k, v = plain_model.project_qkv(normed, layer, 2, 2, 16, 1e-6, *tables[index])
        h = h + plain_model.causal_attention(q, k, v, 0.25) @ layer["self_attn.o_proj.weight"].T
        normed = plain_model.rms_norm(h, w[p + "norm2.weight"], 1e-6)
        if index == 0:
            probabilities = torch.softmax(normed @ w[p + "ffn.router.weight"].T, dim=-1)
            weight, chosen = probabilities.max(dim=-1)
            h = h + torch.stack([(row @ w[p + f"ffn.experts.{int(e)}.weight"].T) * g for row, e, g in zip(normed, chosen, weight)])
        else:
            h = h + plain_model.swiglu_mlp(normed, {"mlp." + k[len(p + "ffn."):]: v for k, v in w.items() if k.startswith(p + "ffn.")})
    return (plain_model.rms_norm(h, w["toy.norm.weight"], 1e-6) @ w["toy.head.weight"].T).numpy()


def test_toy_routed_feed_forward_and_position_encoding():
    """A feed-forward that routes each token to one of three experts and a position encoding with other frequencies
    are registered from here, built by the generic decoder beside the framework's own parts, and stepped in pieces."""
    from llmserver_b200.cache import CacheManager
    from llmserver_b200.engine.step import StepFunction
    from llmserver_b200.models import DecoderModel
    from llmserver_b200.parts import Runtime

    register_toy_feed_forward_and_position()
    dtype = torch.float32
    spec = routed_spec()
    source = MovedSource(spec, 9, dtype)
    model = DecoderModel(spec, source, Runtime(dtype, DEVICE))
    cache = CacheManager(model.cache_needs(), 8, 24, num_slots=2)
    cache.materialize(DEVICE, dtype)
    step = StepFunction(model, cache)
    tokens = tokens_for(90, 41, 4)
    want = plain_routed_forward(source.seen, tokens)
    step.admit("r")
    got = [step.run([("r", tokens[:17], list(range(17)))]), step.run([("r", tokens[17:19], [0, 1])])]
    got += [step.run([("r", [token], [0])]) for token in tokens[19:30]]
    got.append(step.run([("r", tokens[30:], list(range(11)))]))
    assert_close(torch.cat(got).cpu().numpy(), want, "float32", "toy routed model")
    step.check_errors()
    step.release("r")
    cache.check_invariants()


# ---------------------------------------------------------------------------------------------------------------------
# A block arrangement with four norms per layer, defined here; the framework's attention with a rotation of only a
# part of each head, paired as halves in one layer and interleaved in the other; two cache groups (the layers differ in
# kv heads and head size) that both keep every key, so prompts' beginnings are shared across requests.

def register_sandwich_block():
    from llmserver_b200.parts import BLOCKS, Block

    @BLOCKS.register("toy_sandwich")
    class SandwichBlock(Block):
        """h += norm_b(mixer(norm_a(h))); h += norm_d(feed_forward(norm_c(h))): the outputs are normalised too."""

        KNOWN_PARAMS = None

        @classmethod
        def roles(cls, params):
            return {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm",
                    "mixer_out_norm": "norm", "feed_forward_out_norm": "norm"}

        def forward(self, residual, delta, batch, cache):
            normed = self.mixer_norm.add_norm(residual, delta)
            mixed = self.mixer_out_norm.norm(self.mixer.forward(normed, batch, cache))
            normed = self.feed_forward_norm.add_norm(residual, mixed)
            return residual, self.feed_forward_out_norm.norm(self.feed_forward.forward(normed))

    return SandwichBlock


SANDWICH_LAYERS = ((4, 2, 16, 8, "halves", 10000.0), (2, 1, 32, 16, "interleaved", 500.0))   # heads, kv, D, rotary, pairing, theta


def sandwich_spec(hidden=48, vocab=131):
    from llmserver_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    norm = PartSpec.of("rmsnorm", width=hidden, eps=1e-5)
    block = PartSpec.of("toy_sandwich", mixer_prefix="attn.", feed_forward_prefix="ffn.", mixer_norm_prefix="norm_a.",
                        mixer_out_norm_prefix="norm_b.", feed_forward_norm_prefix="norm_c.", feed_forward_out_norm_prefix="norm_d.")
    feed_forward = PartSpec.of("swiglu", hidden=hidden, intermediate=72)
    layers, positions = [], {}
    for index, (heads, kv_heads, dim, rotary, pairing, theta) in enumerate(SANDWICH_LAYERS):
        attention = PartSpec.of("gqa_attention", hidden=hidden, heads=heads, kv_heads=kv_heads, head_dim=dim, scale=dim ** -0.5,
                                qk_norm=True, eps=1e-5, window=None)
        positions[f"rope{index}"] = PartSpec.of("rotary", head_dim=dim, theta=theta, rotary_dim=rotary, pairing=pairing)
        layers.append(LayerSpec(f"toy.layers.{index}.", block, attention, feed_forward, norm, norm, f"rope{index}",
                                extra=(("mixer_out_norm", norm), ("feed_forward_out_norm", norm))))
    return ModelSpec(architecture="ToySandwichForTests", vocab_size=vocab, hidden_size=hidden, layers=layers,
                     schedule=[ScheduleEntry(0), ScheduleEntry(1)], positions=positions, final_norm=norm,
                     embedding_name="toy.embed.weight", final_norm_prefix="toy.norm.", head_name="toy.head.weight")


def partly_rotated(x, positions, rotary, pairing, theta):
    """The first ``rotary`` elements of every head rotated by position * theta^(-2i / rotary), as halves or as
    neighbouring pairs; the rest untouched.  x [T, heads, D] float64."""
    inverse = 1.0 / (theta ** (torch.arange(0, rotary, 2, dtype=torch.long).to(torch.float32) / rotary))
    angles = (positions.to(torch.float32).unsqueeze(-1) * inverse.view(1, -1)).double()      # [T, rotary / 2]
    cosine, sine = torch.cos(angles).unsqueeze(1), torch.sin(angles).unsqueeze(1)
    out = x.clone()
    if pairing == "halves":
        first, second = x[..., :rotary // 2], x[..., rotary // 2:rotary]
        out[..., :rotary // 2] = first * cosine - second * sine
        out[..., rotary // 2:rotary] = second * cosine + first * sine
    else:
        first, second = x[..., 0:rotary:2], x[..., 1:rotary:2]
        out[..., 0:rotary:2] = first * cosine - second * sine
        out[..., 1:rotary:2] = second * cosine + first * sine
    return out


def plain_sandwich_forward(weights, tokens, hidden=48):
    w = {name: tensor.double() for name, tensor in weights.items()}
    h = w["toy.embed.weight"][torch.tensor(tokens)]
    positions = torch.arange(len(tokens))
    for index, (heads, kv_heads, dim, rotary, pairing, theta) in enumerate(SANDWICH_LAYERS):
        p = f"toy.layers.{index}."
        x = plain_model.rms_norm(h, w[p + "norm_a.weight"], 1e-5)
        count = len(tokens)
        q = plain_model.rms_norm((x @ w[p + "attn.q_proj.weight"].T).view(count, heads, dim), w[p + "attn.q_norm.weight"], 1e-5)
        k = plain_model.rms_norm((x @ w[p + "attn.k_proj.weight"].T).view(count, kv_heads, dim), w[p + "attn.k_norm.weight"], 1e-5)
        v = (x @ w[p + "attn.v_proj.weight"].T).view(count, kv_heads, dim)
        q, k = partly_rotated(q, positions, rotary, pairing, theta), partly_rotated(k, positions, rotary, pairing, theta)
        mixed = plain_model.causal_attention(q, k, v, dim ** -0.5) @ w[p + "attn.o_proj.weight"].T
        h = h + plain_model.rms_norm(mixed, w[p + "norm_b.weight"], 1e-5)
        x = plain_model.rms_norm(h, w[p + "norm_c.weight"], 1e-5)
        fed = plain_model.swiglu_mlp(x, {"mlp." + name[len(p + "ffn."):]: t for name, t in w.items() if name.startswith(p + "ffn.")})
        h = h + plain_model.rms_norm(fed, w[p + "norm_d.weight"], 1e-5)
    return (plain_model.rms_norm(h, w["toy.norm.weight"], 1e-5) @ w["toy.head.weight"].T).numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_with_more_norms_partial_rotation_and_prefixes_across_two_groups(dtype):
    from llmserver_b200 import Engine
    from llmserver_b200.models import DecoderModel
    from llmserver_b200.parts import Runtime
    from llmserver_b200.weights import declared_weights

    register_sandwich_block()
    spec = sandwich_spec()
    names = declared_weights(spec)
    assert "toy.layers.0.norm_b.weight" in names and "toy.layers.1.norm_d.weight" in names and len(names) == 2 * 13 + 3
    source = MovedSource(spec, 21, dtype)
    model = DecoderModel(spec, source, Runtime(dtype, DEVICE))
    name = "float32" if dtype == torch.float32 else "bfloat16"
    engine = Engine(model, max_new_tokens=6, max_batch_size=3, max_num_batched_tokens=64, prefill_chunk_size=11,
                    kv_cache_num_blocks=24, kv_cache_block_size=8, ignore_eos=True, max_context=128)
    assert len(engine.cache.groups) == 2 and engine.cache.prefix_sharing
    # logits under cuts, through the engine's own step function
    tokens = tokens_for(131, 45, 8)
    want = plain_sandwich_forward(source.seen, tokens)
    step = engine.step_function
    step.admit("s")
    got = [step.run([("s", tokens[:13], list(range(13)))]), step.run([("s", tokens[13:15], [0, 1])])]
    got += [step.run([("s", [token], [0])]) for token in tokens[15:24]]
    got.append(step.run([("s", tokens[24:], list(range(21)))]))
    assert_close(torch.cat(got).cpu().numpy(), want, name, "sandwich model")
    step.check_errors()
    step.release("s")
    # generation: the second request begins like the first and takes its complete pages over in both groups
    common = tokens_for(131, 24, 9)
    prompts = [common + tokens_for(131, 5, 10), common + tokens_for(131, 9, 11)]
    first = engine.generate([prompts[0]])
    assert engine.stats["prefix_tokens"] == 0
    second = engine.generate([prompts[1]])
    assert engine.stats["prefix_tokens"] == 24
    if dtype == torch.float32:
        fresh = Engine(model, max_new_tokens=6, max_batch_size=1, kv_cache_num_blocks=24, kv_cache_block_size=8,
                       ignore_eos=True, prefix_caching=False, cuda_graphs=False, max_context=128)
        assert fresh.generate([prompts[0]]) == first and fresh.generate([prompts[1]]) == second
        for prompt, generated in zip(prompts, first + second):
            sequence = prompt + generated
            logits = plain_sandwich_forward(source.seen, sequence)
            assert generated == [int(logits[len(prompt) - 1 + index].argmax()) for index in range(6)]
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity()


def test_parts_refuse_what_they_cannot_do():
    """A specification that asks a built-in part for something it has no code for is refused by the part itself."""
    from llmserver_b200.config.spec import PartSpec
    from llmserver_b200.parts import FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Runtime
    attention = MIXERS.get("gqa_attention")
    good = dict(hidden=32, heads=2, kv_heads=1, head_dim=16, scale=0.25, qk_norm=False, eps=1e-6, window=None)
    attention.check_params(good)
    for extra in (dict(bias=True), dict(softcap=30.0), dict(rope_scaling="yarn")):
        with pytest.raises(ValueError):
            attention.check_params({**good, **extra})
    with pytest.raises(ValueError):
        FEED_FORWARDS.get("swiglu").check_params(dict(hidden=8, intermediate=16, activation="gelu"))
    with pytest.raises(ValueError):
        NORMS.get("rmsnorm").check_params(dict(width=8, eps=1e-6, unit_offset=True))
    runtime = Runtime(torch.float32, DEVICE)
    weights = {"q_proj.weight": torch.zeros(32, 32, device=DEVICE), "k_proj.weight": torch.zeros(16, 32, device=DEVICE),
               "v_proj.weight": torch.zeros(16, 32, device=DEVICE), "o_proj.weight": torch.zeros(32, 32, device=DEVICE)}
    mixer = attention(good, weights, runtime)
    rotary = POSITION_ENCODINGS.get("rotary")
    with pytest.raises(ValueError):
        mixer.attach(rotary(dict(head_dim=16, theta=1e4, attention_factor=1.2), {}, runtime))
    with pytest.raises(ValueError):
        mixer.attach(rotary(dict(head_dim=32, theta=1e4), {}, runtime))            # rotates more than a head holds
    with pytest.raises(ValueError):
        mixer.attach(rotary(dict(head_dim=16, theta=1e4, pairing="triples"), {}, runtime))
    mixer.attach(rotary(dict(head_dim=16, theta=1e4, rotary_dim=8, pairing="interleaved"), {}, runtime))
    assert mixer.rotary_dim == 8 and mixer.interleaved
