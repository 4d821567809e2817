"""Grouped-query attention over the paged cache, with optional per-head Q/K RMSNorm, rotary
positions and a sliding window."""
from __future__ import annotations

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
    p - window + 1 .. p)."""

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
        self.inv_freq = None

    def attach(self, position):
        if position is not None:
            if getattr(position, "head_dim", self.head_dim) != self.head_dim:
                raise ValueError("the position encoding was built for another head_dim")
            self.inv_freq = position.inv_freq

    def forward(self, x, batch, cache):
        qkv = ops.linear(x, self.qkv)
        tables = batch.block_tables[cache.group]
        ops.qk_norm_rope_kv_write(qkv, self.q_norm, self.k_norm, self.inv_freq, batch.positions, batch.seq_of_token,
                                  tables, cache.k_pages, cache.v_pages, self.heads, self.kv_heads, self.head_dim,
                                  self.eps, cache.writes, batch.error_flag)
        attended = ops.attention(qkv, batch, tables, cache.k_pages, cache.v_pages, self.heads, self.kv_heads,
                                 self.head_dim, self.scale, self.window)
        return ops.linear(attended, self.out)
