"""Latent attention (spec: ``LatentAttentionSpec``): the cache holds, per token, one normed latent
vector c of ``kv_rank`` elements and one rotated key part of ``rope_dim`` elements; head h's
unrotated key is W_uk[h] c and its value W_uv[h] c.

Neither is ever expanded.  Because q.(W_uk[h] c) = (W_uk[h]^T q).c, the unrotated part of a query
is multiplied by its head's W_uk once, and the attention runs over the cached rows themselves:

  1. one product for q | dkv | gate;
  2. one kernel: RMS norm of the latent part of dkv, rotation of its last ``rope_dim`` elements
     (neighbouring pairs), the row [c | rotated part] into the request's page; rotation of the last
     ``rope_dim`` elements of every query head, written behind where the absorbed part will go;
  3. per head: q'[h] = W_uk[h]^T q_unrotated[h]   (``kv_rank`` elements);
  4. attention with ONE kv head for all query heads, keys = cached rows (kv_rank + rope_dim
     elements), values = the first kv_rank elements of the same rows, float32 softmax, window;
  5. per head: o[h] = W_uv[h] o'[h], times sigmoid(gate), and the output projection.

The scores and results equal those of the expanded form exactly (up to rounding), for prompts and
single tokens alike, so no per-head key or value is cached or recomputed for earlier tokens.
"""

from __future__ import annotations

import math

import torch

from ..cache.manager import PagedKVRequest
from ..ops import attention as A
from ..ops import kernels as K
from ..ops.linear import batched_head_linear, linear
from ..weights.source import MATRIX, NORM, TensorDecl
from .base import Mixer
from .normed_attention import pad_rows
from .registry import POSITIONS, build_part, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.position = build_part(POSITIONS, spec.position, f"{prefix}.rot", env)
        self.q_head = spec.head_dim + spec.rope_dim
        self.row = spec.kv_rank + spec.rope_dim                    # a cached row; a query row after step 3
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(self.q_head)
        A.check_kv_supported(self.row, spec.kv_rank)
        A.prepare_kv_attention(self.row, spec.kv_rank, env.dtype)

    @classmethod
    def _names(cls, spec, prefix):
        return {n: f"{prefix}.{getattr(spec, n + '_name')}"
                for n in ("q", "down", "latent_norm", "up_k", "up_v", "o", "gate")}

    @classmethod
    def declare(cls, spec, prefix):
        h, H, D, Dr, Dv, R = (spec.hidden_size, spec.num_heads, spec.head_dim, spec.rope_dim,
                              spec.value_dim, spec.kv_rank)
        n = cls._names(spec, prefix)
        out = [TensorDecl(n["q"], (H * (D + Dr), h), MATRIX), TensorDecl(n["down"], (R + Dr, h), MATRIX),
               TensorDecl(n["latent_norm"], (R,), NORM), TensorDecl(n["up_k"], (H * D, R), MATRIX),
               TensorDecl(n["up_v"], (H * Dv, R), MATRIX), TensorDecl(n["o"], (h, H * Dv), MATRIX)]
        if spec.element_gate:
            out.append(TensorDecl(n["gate"], (H * Dv, h), MATRIX))
        return out

    @classmethod
    def cache_request(cls, spec):
        return PagedKVRequest(1, spec.kv_rank + spec.rope_dim, spec.window, tied_values=True)

    def load(self, store):
        s = self.spec
        n = self._names(s, self.prefix)
        self.w_in = pad_rows(store.cat([n["q"], n["down"]] + ([n["gate"]] if s.element_gate else [])))
        self.latent_norm = store.get(n["latent_norm"])
        # [H, kv_rank, head_dim]: q' = q_unrotated . this^T per head
        self.w_uk_t = store.get(n["up_k"]).view(s.num_heads, s.head_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = store.get(n["up_v"]).view(s.num_heads, s.value_dim, s.kv_rank).contiguous()
        self.w_o = store.get(n["o"])

    def forward(self, ctx, x, cache, owns_cache):
        s = self.spec
        T, H, D, Dr, R = x.shape[0], s.num_heads, s.head_dim, s.rope_dim, s.kv_rank
        table = ctx.block_tables[cache.group]
        proj = K.plain_unless(None, linear(x, self.w_in))             # [T, q | dkv | gate]
        q_size = H * self.q_head
        q_abs = torch.empty((T, H * self.row), dtype=x.dtype, device=x.device)
        pairs = getattr(self.position, "pair_table", None)
        freq, rot_dims, mag = pairs() if pairs is not None else (None, 0, 1.0)
        K.head_prep(proj, ctx, table, cache.page_size,
                    q_off=0, num_heads=H, q_dim=self.q_head, q_norm_w=None, q_norm_dims=0, q_rot_off=D,
                    k_off=q_size, num_kv_heads=1, k_dim=self.row, k_norm_w=self.latent_norm,
                    k_norm_dims=R, k_rot_off=R, v_off=-1, v_dim=0,
                    freq=freq, rot_dims=rot_dims, rot_mag=mag, eps=s.latent_norm_eps,
                    q_out=q_abs[:, R:], k_cache=cache.k if owns_cache else None, v_cache=None,
                    q_head_stride=self.row, q_skip=D)
        # q'[:, h, :R] = q[:, h, :D] . W_uk[h]
        batched_head_linear(proj[:, :q_size].view(T, H, self.q_head)[:, :, :D], self.w_uk_t,
                            q_abs.view(T, H, self.row)[:, :, :R])
        o_lat = torch.empty((T, H * R), dtype=x.dtype, device=x.device)
        A.kv_attention(ctx, q_abs, cache.k, cache.k, self.row, o_lat, table, H, 1, self.row, R,
                       cache.page_size, self.scale, s.window or 0, None)
        out = torch.empty((T, H * s.value_dim), dtype=x.dtype, device=x.device)
        batched_head_linear(o_lat.view(T, H, R), self.w_uv, out.view(T, H, s.value_dim))
        if s.element_gate:
            K.sigmoid_gate(out, proj[:, q_size + self.row:q_size + self.row + H * s.value_dim], out)
        return linear(out, self.w_o, consumer="norm")
