"""Grouped-query attention over the paged cache, with optional per-head Q/K RMSNorm, rotary
positions and a sliding window."""
from __future__ import annotations

import functools

import torch

from .. import ops
from ..cache.manager import KVPagesNeed
from ..weights.declare import NORM, WeightDecl
from .base import Mixer
from .registry import MIXERS


@MIXERS.register("gqa_attention")
class GQAttention(Mixer):
    """Q, K, V = x Wq^T, x Wk^T, x Wv^T as one fused product (utils/attention.py:54-66,118-128); each Q
    and K head RMS-normalised with a shared [D] weight before the rotation (utils/attention.py:38-39,
    143-158); K stored after norm and rotation, V raw (utils/attention.py:172-176); softmax(Q K^T *
    scale) V over the request's cached tokens, query head h reading kv head h // group
    (utils/attention.py:186-198); output through Wo (utils/attention.py:299-300).

    Parameters: ``hidden``, ``heads``, ``kv_heads``, ``head_dim``, ``scale``, ``qk_norm`` (bool),
    ``eps`` (of the Q/K norms), ``window`` (None = all keys; else a query at position p reads keys
    p - window + 1 .. p).  ``bias`` and ``softcap`` are known and must be off: the kernels have neither a bias
    epilogue nor score capping, and say so instead of computing without them.

    How positions are encoded comes from the position encoding the layer names (``attach``): its inverse
    frequencies, how many elements of a head rotate (``rotary_dim``, at most head_dim) and how they pair
    ("halves" or "interleaved").  An encoding that scales the rotated values (``attention_factor`` other than 1) is
    refused: the rotation kernel does not scale."""

    KNOWN_PARAMS = ("hidden", "heads", "kv_heads", "head_dim", "scale", "qk_norm", "eps", "window", "bias", "softcap")

    @classmethod
    def check_params(cls, params):
        super().check_params(params)
        if params.get("bias"):
            raise ValueError("gqa_attention has no biases in its projections (bias must be absent or false)")
        if params.get("softcap"):
            raise ValueError("gqa_attention does not cap attention scores (softcap must be absent or 0)")

    @classmethod
    def declare_weights(cls, params):
        hidden, heads, kv_heads, dim = params["hidden"], params["heads"], params["kv_heads"], params["head_dim"]
        wanted = {"q_proj.weight": WeightDecl((heads * dim, hidden)),
                  "k_proj.weight": WeightDecl((kv_heads * dim, hidden)),
                  "v_proj.weight": WeightDecl((kv_heads * dim, hidden)),
                  "o_proj.weight": WeightDecl((hidden, heads * dim))}
        if params.get("qk_norm"):
            wanted["q_norm.weight"] = WeightDecl((dim,), NORM)
            wanted["k_norm.weight"] = WeightDecl((dim,), NORM)
        return wanted

    @classmethod
    def cache_need(cls, params):
        return KVPagesNeed(int(params["kv_heads"]), int(params["head_dim"]), params.get("window"))

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.heads, self.kv_heads, self.head_dim = int(params["heads"]), int(params["kv_heads"]), int(params["head_dim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are no multiple of {self.kv_heads} kv heads")
        self.scale = float(params["scale"])
        self.window = int(params["window"]) if params.get("window") else 0
        self.eps = float(params.get("eps", 0.0))
        self.qkv = torch.cat([weights["q_proj.weight"], weights["k_proj.weight"], weights["v_proj.weight"]], dim=0).contiguous()
        self.out = weights["o_proj.weight"].contiguous()
        self.q_norm = weights["q_norm.weight"].contiguous() if params.get("qk_norm") else None
        self.k_norm = weights["k_norm.weight"].contiguous() if params.get("qk_norm") else None
        self.inv_freq, self.rotary_dim, self.interleaved = None, self.head_dim, False

    def attach(self, position):
        """``position``: None (no rotation) or an encoding with ``inv_freq`` (float32 [rotary_dim / 2] on the device)
        and, optionally, ``rotary_dim``, ``pairing`` ("halves" | "interleaved") and ``attention_factor``."""
        if position is None:
            return
        inv_freq = getattr(position, "inv_freq", None)
        if inv_freq is None:
            raise ValueError(f"gqa_attention rotates queries and keys: the position encoding {type(position).__name__} "
                             "gives no inv_freq (an encoding that acts on the embedding is not named by a layer)")
        rotary_dim = int(getattr(position, "rotary_dim", 2 * inv_freq.numel()))
        if rotary_dim != 2 * inv_freq.numel() or rotary_dim > self.head_dim or rotary_dim % 2:
            raise ValueError(f"the position encoding rotates {rotary_dim} elements with {inv_freq.numel()} frequencies; "
                             f"gqa_attention needs an even rotary_dim of at most head_dim {self.head_dim} and half as many frequencies")
        pairing = getattr(position, "pairing", "halves")
        if pairing not in ("halves", "interleaved"):
            raise ValueError(f"gqa_attention pairs rotated elements as 'halves' or 'interleaved', not {pairing!r}")
        if float(getattr(position, "attention_factor", 1.0)) != 1.0:
            raise ValueError("gqa_attention's rotation kernel does not scale the rotated values: the position encoding's "
                             f"attention_factor is {position.attention_factor}, only 1 is supported")
        self.inv_freq, self.rotary_dim, self.interleaved = inv_freq, rotary_dim, pairing == "interleaved"

    feeds_stream = True

    @functools.cached_property
    def takes_unscaled(self):
        return ops.unscaled_rows_supported(self.qkv)

    def forward(self, x, batch, cache, sink=None):
        tables = batch.block_tables[cache.group]
        qkv = ops.qkv_projection(x, self.qkv, self.q_norm, self.k_norm, self.inv_freq, batch.positions, batch.seq_of_token,
                                 tables, cache.k_pages, cache.v_pages, self.heads, self.kv_heads, self.head_dim, self.eps,
                                 cache.writes, batch.error_flag, self.rotary_dim, self.interleaved)
        attended = ops.attention(qkv, batch, tables, cache.k_pages, cache.v_pages, self.heads, self.kv_heads,
                                 self.head_dim, self.scale, self.window)
        return ops.linear(attended, self.out, sink=sink)
