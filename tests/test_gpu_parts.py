"""Each part of a layer alone on the GPU against the plain functions, at sizes of its own, and a model
whose schedule names a layer twice and lets an entry read another entry's cache."""
import pytest
import torch

import plain_model
from helpers import assert_close, plain_folder, tokens_for

pytestmark = pytest.mark.gpu
DEVICE = torch.device("cuda:0")


def runtime(dtype):
    from llmserver_b200.parts import Runtime
    return Runtime(dtype, DEVICE)


def rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def bound(dtype):
    return 3e-6 if dtype == torch.float32 else 2e-2


def close(got, want, dtype, what):
    error = (got.double().cpu() - want.double()).abs().max().item() / want.abs().max().item()
    assert error < bound(dtype), f"{what}: {error:.3e}"


def one_sequence_batch(start, count, pages_per_table, n_groups=1):
    from llmserver_b200.engine.batch import SequenceSlice, build_batch
    return build_batch([SequenceSlice("r", list(range(count)), start, [], [list(range(pages_per_table))] * n_groups, 0)],
                       n_groups, DEVICE)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from llmserver_b200.parts import NORMS
    weight = (rand((200,), 1) * 0.1 + 1).to(dtype)
    part = NORMS.get("rmsnorm")({"width": 200, "eps": 1e-4}, {"weight": weight.to(DEVICE)}, runtime(dtype))
    residual, delta = rand((6, 200), 2), rand((6, 200), 3).to(dtype)
    work = residual.to(DEVICE)
    out = part.add_norm(work, delta.to(DEVICE))
    close(out, plain_model.rms_norm(residual.double() + delta.double(), weight.double(), 1e-4), dtype, "rmsnorm part")
    close(work, residual.double() + delta.double(), torch.float32, "residual stream")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from llmserver_b200.parts import FEED_FORWARDS
    names = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
    shapes = ((176, 72), (176, 72), (72, 176))
    weights = {name: rand(shape, 10 + i, 0.2).to(dtype) for i, (name, shape) in enumerate(zip(names, shapes))}
    part = FEED_FORWARDS.get("swiglu")({"hidden": 72, "intermediate": 176}, {k: v.to(DEVICE) for k, v in weights.items()}, runtime(dtype))
    x = rand((9, 72), 20).to(dtype)
    want = plain_model.swiglu_mlp(x.double(), {"mlp." + k: v.double() for k, v in weights.items()})
    close(part.forward(x.to(DEVICE)), want, dtype, "swiglu part")


def test_rotary_part_builds_the_reference_frequencies():
    from llmserver_b200.parts import POSITION_ENCODINGS
    part = POSITION_ENCODINGS.get("rotary")({"head_dim": 48, "theta": 500000.0}, {}, runtime(torch.float32))
    want = 1.0 / (500000.0 ** (torch.arange(0, 48, 2).float() / 48))
    assert torch.equal(part.inv_freq.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 13])
def test_attention_part_over_two_portions(dtype, window):
    """The mixer alone: a prompt in two portions (29 + 12 tokens) against whole-sequence plain attention."""
    from llmserver_b200.parts import MIXERS, POSITION_ENCODINGS, EntryCache
    hidden, heads, kv_heads, dim, eps, theta = 56, 6, 2, 32, 1e-5, 30000.0
    params = {"hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": dim, "scale": dim ** -0.5,
              "qk_norm": True, "eps": eps, "window": window}
    cls = MIXERS.get("gqa_attention")
    weights = {}
    for index, (name, declaration) in enumerate(cls.declare_weights(params).items()):
        values = rand(declaration.shape, 30 + index, 0.15)
        weights[name] = (values + 1 if "norm" in name else values).to(dtype)
    mixer = cls(params, {k: v.to(DEVICE) for k, v in weights.items()}, runtime(dtype))
    mixer.attach(POSITION_ENCODINGS.get("rotary")({"head_dim": dim, "theta": theta}, {}, runtime(dtype)))
    assert cls.cache_need(params).window == window
    x = rand((41, hidden), 40).to(dtype)
    pages = torch.zeros((2, 8, kv_heads, 8, dim), dtype=dtype, device=DEVICE)
    cache = EntryCache(k_pages=pages[0], v_pages=pages[1], group=0, writes=True)
    outputs = []
    for start, count in ((0, 29), (29, 12)):
        batch = one_sequence_batch(start, count, 6)
        outputs.append(mixer.forward(x[start:start + count].to(DEVICE).contiguous(), batch, cache))
    got = torch.cat(outputs)
    plain = {"self_attn." + k: v.double() for k, v in weights.items()}
    cosine, sine = plain_model.rope_tables(torch.arange(41), dim, theta, torch.float64)
    q, k, v = plain_model.project_qkv(x.double(), plain, heads, kv_heads, dim, eps, cosine, sine)
    want = plain_model.causal_attention(q, k, v, dim ** -0.5, window) @ plain["self_attn.o_proj.weight"].T
    close(got, want, dtype, "attention part")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_with_a_repeated_layer_and_a_shared_cache(tiny_folders, dtype):
    """Layer 1 runs twice; its second run attends over the keys and values its first run cached."""
    from llmserver_b200.cache import CacheManager
    from llmserver_b200.config import ARCHITECTURES, Qwen3Config
    from llmserver_b200.config.spec import ScheduleEntry
    from llmserver_b200.engine.step import StepFunction
    from llmserver_b200.models import DecoderModel
    from llmserver_b200.models.loading import as_dtype
    from llmserver_b200.parts import Runtime
    from llmserver_b200.weights import CheckpointSource
    from tiny_configs import TINY_A

    folder = tiny_folders["a"]
    spec = ARCHITECTURES["Qwen3ForCausalLM"].build_spec(Qwen3Config.from_dict(TINY_A))
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_from=1)]
    run = Runtime(as_dtype(dtype), DEVICE)
    model = DecoderModel(spec, CheckpointSource(folder, spec, run.dtype, run.device), run)
    assert [need is not None for need in model.cache_needs()] == [True, True, True, False]
    cache = CacheManager(model.cache_needs(), 4, 32, num_slots=2, prefix_sharing=False)
    cache.materialize(run.device, run.dtype)
    assert cache.groups[0].entries == [0, 1, 2]
    step = StepFunction(model, cache)
    tokens = tokens_for(256, 45, 77)
    step.admit("r")
    got = torch.cat([step.run([("r", tokens[:31], list(range(31)))]), step.run([("r", tokens[31:33], [0, 1])]),
                     step.run([("r", tokens[33:], list(range(12)))])]).cpu().numpy()
    step.check_errors()
    config, weights = plain_folder(folder)
    want = plain_model.forward(config, weights, tokens, order=[(0, None), (1, None), (0, None), (1, 1)]).numpy()
    assert_close(got, want, dtype, "repeated layer + shared cache")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pre_norm_block_alone(dtype):
    """One block (norm, attention, norm, feed-forward around the 32-bit stream) against the plain decoder layer,
    with the not-yet-added output of a previous block handed in and its own handed out."""
    from llmserver_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, EntryCache
    hidden, heads, kv_heads, dim, inter, eps, theta = 40, 5, 5, 16, 72, 2e-6, 20000.0
    config = {"hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": dim,
              "rms_norm_eps": eps}
    run = runtime(dtype)
    mixer_params = {"hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": dim, "scale": dim ** -0.5,
                    "qk_norm": True, "eps": eps, "window": None}
    plain_weights, parts = {}, {}
    for role, registry, kind, params, prefix in (
            ("mixer", MIXERS, "gqa_attention", mixer_params, "self_attn."),
            ("feed_forward", FEED_FORWARDS, "swiglu", {"hidden": hidden, "intermediate": inter}, "mlp."),
            ("mixer_norm", NORMS, "rmsnorm", {"width": hidden, "eps": eps}, "input_layernorm."),
            ("feed_forward_norm", NORMS, "rmsnorm", {"width": hidden, "eps": eps}, "post_attention_layernorm.")):
        cls = registry.get(kind)
        weights = {}
        for index, (name, declaration) in enumerate(cls.declare_weights(params).items()):
            values = rand(declaration.shape, 300 + 10 * len(plain_weights) + index, 0.2)
            weights[name] = (values + 1 if declaration.kind == "norm" else values).to(dtype)
            plain_weights[prefix + name] = weights[name].double()
        parts[role] = cls(params, {k: v.to(DEVICE) for k, v in weights.items()}, run)
    parts["mixer"].attach(POSITION_ENCODINGS.get("rotary")({"head_dim": dim, "theta": theta}, {}, run))
    block = BLOCKS.get("pre_norm")({}, parts)
    tokens = 23
    stream, pending = rand((tokens, hidden), 70), rand((tokens, hidden), 71).to(dtype)
    pages = torch.zeros((2, 8, kv_heads, 4, dim), dtype=dtype, device=DEVICE)
    cache = EntryCache(k_pages=pages[0], v_pages=pages[1], group=0, writes=True)
    residual = stream.to(DEVICE)
    residual, delta = block.forward(residual, pending.to(DEVICE), one_sequence_batch(0, tokens, 6), cache)
    got = residual.double().cpu() + delta.double().cpu()
    cosine, sine = plain_model.rope_tables(torch.arange(tokens), dim, theta, torch.float64)
    want, _ = plain_model.decoder_layer(stream.double() + pending.double(), plain_weights, config, cosine, sine)
    close(got, want, dtype, "pre-norm block")
