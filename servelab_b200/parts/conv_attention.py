"""Windowed attention with a short convolution on queries and keys, tied values, a
log-distance bias, mixed heads and an output gate (spec: ``ConvTalkAttentionSpec``).

Per step, with h the mixer's input [T, hidden]:

  1. one product for q | k | gate (their matrices are concatenated at load);
  2. one kernel: causal convolution over time on the q and k channels (the rows before a
     portion come from the request's state slot, which is updated), q times its temperature
     1 + coef ln(floor((p + 1) / every) + 1), k into the request's pages -- the values are
     these keys, so nothing else is stored;
  3. attention of every query over its request's visible keys (0 <= i - j < window):
     score = q.k scale - r1_h ln(1 + r2_h (i - j)), softmax in float32;
  4. the heads' weights are mixed after the softmax, w'_h = sum_g talk[h, g] w_g, and head h
     applies w'_h to the values of its own kv head c(h).  Because the mix is linear,
     sum_j w'_h(i, j) v_c(h)(j) = sum_g talk[h, g] O[g, c(h)] with
     O[g, c] = sum_j w_g(i, j) v_c(j): the attention kernels produce O for every (query head,
     kv head) pair with an online softmax and one more kernel mixes them, multiplied by
     sigmoid(gate);
  5. the output projection.

State: ``PagedKVRequest(..., tied_values=True)`` for the keys and a ``FixedStateRequest`` of
(taps - 1) x (q width + kv width) float32 for the rows the convolution looks back on.
"""

from __future__ import annotations

import math

import torch

from ..cache.manager import FixedStateRequest, PagedKVRequest
from ..ops import attention as A
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.source import BIAS, MATRIX, MIXING, POSITIVE, TensorDecl
from .base import Mixer
from .registry import register_mixer


@register_mixer("conv_talk_attention")
class ConvTalkAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not spec.tied_values:
            raise ValueError("conv_talk_attention: only tied values (v = k) are built")
        if spec.conv_taps < 0 or spec.conv_taps > K.CONV_MAX_TAPS:
            raise ValueError(f"conv_talk_attention: 0..{K.CONV_MAX_TAPS} taps, got {spec.conv_taps}")
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        A.check_supported(spec.head_dim, env.dtype)
        A.prepare_talk_attention(spec.head_dim, env.dtype)

    @classmethod
    def _names(cls, spec, prefix):
        sfx = spec.weight_suffix
        return {n: f"{prefix}.{getattr(spec, n + '_name')}{sfx}" for n in ("q", "k", "o", "gate")}

    @classmethod
    def declare(cls, spec, prefix):
        h, q, kv = spec.hidden_size, spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        n = cls._names(spec, prefix)
        out = [TensorDecl(n["q"], (q, h), MATRIX), TensorDecl(n["k"], (kv, h), MATRIX),
               TensorDecl(n["o"], (h, q), MATRIX)]
        if spec.conv_taps >= 1:
            out += [TensorDecl(n["q"] + spec.conv_suffix, (q, spec.conv_taps), BIAS),
                    TensorDecl(n["k"] + spec.conv_suffix, (kv, spec.conv_taps), BIAS)]
        if spec.distance_bias:
            out += [TensorDecl(f"{prefix}.{spec.bias_r1_name}", (spec.num_heads,), POSITIVE),
                    TensorDecl(f"{prefix}.{spec.bias_r2_name}", (spec.num_heads,), POSITIVE)]
        if spec.talking_heads:
            out.append(TensorDecl(f"{prefix}.{spec.talk_name}", (spec.num_heads, spec.num_heads), MIXING))
        if spec.output_gate:
            out.append(TensorDecl(n["gate"], (q, h), MATRIX))
        return out

    @classmethod
    def cache_request(cls, spec):
        pages = PagedKVRequest(spec.num_kv_heads, spec.head_dim, spec.window, tied_values=True)
        if spec.conv_taps <= 1:
            return pages
        width = (spec.num_heads + spec.num_kv_heads) * spec.head_dim
        return (pages, FixedStateRequest((spec.conv_taps - 1, width)))

    def load(self, store):
        s = self.spec
        n = self._names(s, self.prefix)
        self.w_in = store.cat([n["q"], n["k"]] + ([n["gate"]] if s.output_gate else []))
        self.w_o = store.get(n["o"])
        if s.conv_taps >= 1:
            # [taps, channels]: a tap's weights of neighbouring channels are neighbours
            self.taps = store.cat([n["q"] + s.conv_suffix, n["k"] + s.conv_suffix]).t().contiguous()
        else:
            self.taps = torch.ones((1, self.q_size + self.kv_size), dtype=torch.float32,
                                   device=self.env.device)
        self.r1 = store.get(f"{self.prefix}.{s.bias_r1_name}") if s.distance_bias else None
        self.r2 = store.get(f"{self.prefix}.{s.bias_r2_name}") if s.distance_bias else None
        self.talk = store.get(f"{self.prefix}.{s.talk_name}") if s.talking_heads else None

    def forward(self, ctx, x, cache, owns_cache):
        s = self.spec
        T = x.shape[0]
        table = ctx.block_tables[cache.group]
        proj = linear(x, self.w_in)                    # [T, q | k | gate]
        q = torch.empty((T, self.q_size), dtype=x.dtype, device=x.device)
        if not owns_cache:
            raise NotImplementedError("conv_talk_attention: a run that reads another run's cache")
        K.qk_conv_cache(proj, self.taps, cache.state, ctx, table, cache.page_size, s.q_temp_coef or 0.0, s.q_temp_every, q,
                        cache.k, s.num_kv_heads, s.head_dim)
        gate = proj[:, self.q_size + self.kv_size:] if s.output_gate else None
        out = torch.empty_like(q)
        A.talk_attention(ctx, q, cache.k, cache.v, out, table, s.num_heads, s.num_kv_heads, s.head_dim,
                         cache.page_size, self.scale, s.window or 0, self.r1, self.r2, self.talk, gate)
        return linear(out, self.w_o, consumer="norm")
