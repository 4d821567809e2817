"""Plain, slow Qwen3-dense implementation used as the oracle of the test-suite.

Whole sequences, no cache, no batching, one function per part, PyTorch on the CPU (or any
device the tensors live on).  It shares no code with ``llmserver_b200``: it reads a model
folder with the ``safetensors`` library directly and takes the configuration as a plain
``dict`` of config.json keys.

Every function is written from the formulas of AshvinSehgal/LLMServer (paths are relative
to that project) and cites the lines it follows.  ``tests/golden/make_golden.py`` compares
it once against that project's own ``utils.model.Model`` on two tiny random models; the
outputs of that run are committed under ``tests/golden/``.

Two generalisations go beyond what that project runs; both are used only by tests of the
engine's parts, never by the golden comparison:
  * ``window``: a query at position i sees keys j with i - window < j <= i;
  * ``order``: the list of (layer, cache_from) pairs that says in which order layers run
    and whether an entry attends over the keys and values another entry produced.
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------------------
# loading
# --------------------------------------------------------------------------------------
def read_model_folder(path, dtype=torch.float64):
    """config.json as a dict and every tensor of model.safetensors, cast to ``dtype``.

    Names are the checkpoint's own (utils/model_loader.py:54-67 strips the prefixes
    ``model.embed_tokens.``, ``model.norm.``, ``lm_head.``, ``model.layers.{i}.``)."""
    from safetensors import safe_open

    with open(os.path.join(path, "config.json")) as handle:
        config = json.load(handle)
    weights = {}
    with safe_open(os.path.join(path, "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            weights[name] = handle.get_tensor(name).to(dtype)
    return config, weights


def head_dim_of(config):
    """utils/architecture.py:88 — explicit ``head_dim`` or hidden_size // heads."""
    return config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]


def rope_theta_of(config):
    """utils/architecture.py:23-30 — ``rope_theta``, else rope_parameters.rope_theta, else 10000."""
    theta = config.get("rope_theta")
    if theta is None:
        parameters = config.get("rope_scaling") or config.get("rope_parameters") or {}
        theta = parameters.get("rope_theta", 10000.0)
    return float(theta)


def layer_windows_of(config):
    """Per-layer window (None = all keys) from ``layer_types`` and ``sliding_window``.

    AshvinSehgal/LLMServer refuses these keys (utils/architecture.py:72-76); the engine
    accepts them, so the oracle has to as well."""
    layers = config["num_hidden_layers"]
    types = config.get("layer_types")
    window = config.get("sliding_window")
    if types is None:
        if config.get("use_sliding_window") and window:
            first = config.get("max_window_layers", 0)
            types = ["sliding_attention" if i >= first else "full_attention" for i in range(layers)]
        else:
            types = ["full_attention"] * layers
    return [int(window) if kind == "sliding_attention" else None for kind in types]


# --------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------
def rms_norm(x, weight, eps):
    """utils/layers.py:133-138 — x / sqrt(mean(x^2) + eps), then times weight (not 1 + weight)."""
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_tables(positions, head_dim, theta, dtype):
    """utils/layers.py:147,155-164 — inv_freq[i] = theta^(-2i/D) in 32-bit, angle = pos * inv_freq,
    both halves carry the same angles; attention factor 1 for the default schedule."""
    dim_indices = torch.arange(0, head_dim, 2, dtype=torch.long)
    inverse = 1.0 / (theta ** (dim_indices.to(torch.float32) / head_dim))  # fp32 as the reference builds it
    frequencies = positions.to(torch.float32).unsqueeze(-1) * inverse.view(1, -1)  # 32-bit angles (layers.py:160)
    angles = torch.cat([frequencies, frequencies], dim=-1).to(dtype)
    return torch.cos(angles), torch.sin(angles)


def rotate_half(x):
    """utils/layers.py:166-170 — cat(-second half, first half)."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rope(x, cosine, sine):
    """utils/layers.py:172-177 — x * cos + rotate_half(x) * sin; x is [T, heads, D], tables [T, D]."""
    return x * cosine.unsqueeze(1) + rotate_half(x) * sine.unsqueeze(1)


def project_qkv(x, layer_weights, n_heads, n_kv_heads, head_dim, eps, cosine, sine):
    """utils/attention.py:114-160 — Q, K, V = x W^T; per-head RMSNorm of Q and K with the
    shared [D] weights (utils/attention.py:38-39,143-150) before the rotation; V untouched."""
    tokens = x.shape[0]
    q = (x @ layer_weights["self_attn.q_proj.weight"].T).view(tokens, n_heads, head_dim)
    k = (x @ layer_weights["self_attn.k_proj.weight"].T).view(tokens, n_kv_heads, head_dim)
    v = (x @ layer_weights["self_attn.v_proj.weight"].T).view(tokens, n_kv_heads, head_dim)
    q = rms_norm(q, layer_weights["self_attn.q_norm.weight"], eps)
    k = rms_norm(k, layer_weights["self_attn.k_norm.weight"], eps)
    return apply_rope(q, cosine, sine), apply_rope(k, cosine, sine), v


def causal_attention(q, k, v, scale, window=None):
    """utils/attention.py:186-198 — S = Q K^T * scale, keys after the query masked, softmax over
    keys, O = P V; query head h reads kv head h // group (utils/attention.py:186-190).

    q [T, Hq, D], k and v [T, Hkv, D] -> [T, Hq * D] (utils/attention.py:299 layout)."""
    tokens, n_heads, head_dim = q.shape
    group = n_heads // k.shape[1]
    keys = k.repeat_interleave(group, dim=1)
    values = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, keys) * scale
    query_pos = torch.arange(tokens).view(-1, 1)
    key_pos = torch.arange(tokens).view(1, -1)
    hidden = key_pos > query_pos
    if window is not None:
        hidden = hidden | (key_pos <= query_pos - window)
    scores = scores.masked_fill(hidden.unsqueeze(0), float("-inf"))
    probabilities = torch.softmax(scores, dim=-1)
    out = torch.einsum("hqk,khd->qhd", probabilities, values)
    return out.reshape(tokens, n_heads * head_dim)


def swiglu_mlp(x, layer_weights):
    """utils/layers.py:210-218 — down(silu(gate(x)) * up(x)), no biases for Qwen3."""
    gate = x @ layer_weights["mlp.gate_proj.weight"].T
    up = x @ layer_weights["mlp.up_proj.weight"].T
    return (torch.nn.functional.silu(gate) * up) @ layer_weights["mlp.down_proj.weight"].T


def layer_weights_of(weights, index):
    prefix = f"model.layers.{index}."
    return {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}


def decoder_layer(h, layer_weights, config, cosine, sine, window=None, shared_kv=None):
    """utils/model.py:16-35 — h += attn(norm(h)); h += mlp(norm(h)).

    Returns the new hidden states and the (k, v) this layer produced, so that a later entry
    of ``order`` can attend over them instead of its own."""
    eps = config["rms_norm_eps"]
    head_dim = head_dim_of(config)
    n_heads, n_kv_heads = config["num_attention_heads"], config["num_key_value_heads"]
    normed = rms_norm(h, layer_weights["input_layernorm.weight"], eps)
    q, k, v = project_qkv(normed, layer_weights, n_heads, n_kv_heads, head_dim, eps, cosine, sine)
    if shared_kv is not None:
        k, v = shared_kv
    scale = head_dim ** -0.5  # utils/architecture.py:105
    attended = causal_attention(q, k, v, scale, window)
    h = h + attended @ layer_weights["self_attn.o_proj.weight"].T
    normed = rms_norm(h, layer_weights["post_attention_layernorm.weight"], eps)
    return h + swiglu_mlp(normed, layer_weights), (k, v)


def forward(config, weights, token_ids, order=None, return_hidden=False):
    """utils/model.py:109-158 — embed, layers in order, final norm, output head; logits [T, V].

    ``order``: list of (layer index, index into ``order`` whose k/v to read or None);
    default is every layer once (utils/model.py:134-146)."""
    dtype = weights["model.embed_tokens.weight"].dtype
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    h = weights["model.embed_tokens.weight"][ids]  # utils/model.py:56-59,110: no scaling
    positions = torch.arange(len(ids))
    cosine, sine = rope_tables(positions, head_dim_of(config), rope_theta_of(config), dtype)
    windows = layer_windows_of(config)
    if order is None:
        order = [(index, None) for index in range(config["num_hidden_layers"])]
    produced = []
    for layer_index, cache_from in order:
        shared = produced[cache_from] if cache_from is not None else None
        h, kv = decoder_layer(h, layer_weights_of(weights, layer_index), config, cosine, sine,
                              windows[layer_index], shared)
        produced.append(shared if shared is not None else kv)
    if return_hidden:
        return h
    h = rms_norm(h, weights["model.norm.weight"], config["rms_norm_eps"])  # utils/model.py:157
    # utils/model_loader.py:56-57 — tied when the config says so or the checkpoint has no head
    head = weights["lm_head.weight"] if "lm_head.weight" in weights and not config.get("tie_word_embeddings") \
        else weights["model.embed_tokens.weight"]
    return h @ head.T  # utils/model.py:158,170 — no bias


# --------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------
def greedy(logits):
    """utils/engine.py:295-297 — argmax over the vocabulary (lowest index on ties, as torch.argmax)."""
    return int(torch.argmax(logits, dim=-1))


_MASK32 = 0xFFFFFFFF


def _mix32(value):
    value &= _MASK32
    value ^= value >> 16
    value = (value * 0x7FEB352D) & _MASK32
    value ^= value >> 15
    value = (value * 0x846CA68B) & _MASK32
    value ^= value >> 16
    return value


def uniform_for(seed, step, index):
    """The engine's counter-based uniform in (0, 1): a function of (seed, step, vocabulary index)
    only, so that batching cannot change a draw.  AshvinSehgal/LLMServer samples greedily only
    (utils/engine.py:295-297; README.md:125); the temperature sampler is this engine's own."""
    word = _mix32((seed & _MASK32) ^ 0x9E3779B9)
    word = _mix32(word ^ ((seed >> 32) & _MASK32))
    word = _mix32(word ^ (step & _MASK32))
    word = _mix32(word ^ (index & _MASK32))
    return ((word >> 9) + 0.5) * (1.0 / 8388608.0)


def gumbel_scores(logits, temperature, seed, step):
    """logits / T + Gumbel noise; the sampled token is the argmax of these scores, which draws
    from softmax(logits / T)."""
    vocab = logits.shape[-1]
    noise = torch.tensor([-math.log(-math.log(uniform_for(seed, step, index))) for index in range(vocab)],
                         dtype=torch.float64)
    return logits.to(torch.float64) / temperature + noise
