"""A plain, slow implementation of the Dezelorn decoder: one function per mechanism, whole
sequences only, torch on the CPU (float64 by default).  It shares no code with the package:
it reads config.json and model.safetensors itself and knows no cache, page, slot or step.

Notation: x [T, width] the residual stream, h a sublayer's input, positions 0..T-1.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch


def read_safetensors(path: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    raw = open(path, "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = raw[8 + n + lo:8 + n + hi]
        if meta["dtype"] == "BF16":
            bits = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype=np.float32).copy())
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(buf, dtype=np.int32).copy())
        else:
            raise ValueError(meta["dtype"])
        out[name] = t.reshape(meta["shape"]).to(dtype if t.is_floating_point() else t.dtype)
    return out


def load_folder(folder: str, dtype=torch.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"), dtype)


# ------------------------------------------------------------- mechanisms
def dynamic_tanh(x, w, b, alpha):
    """tanh(alpha x) w + b, element by element."""
    return torch.tanh(alpha * x) * w + b


def causal_conv(u, taps):
    """u [T, C], taps [C, n]: y_t = sum_j taps[:, j] u_(t - n + 1 + j), zeros before t = 0."""
    T, n = u.shape[0], taps.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(n):
            src = t - n + 1 + j
            if src >= 0:
                y[t] += taps[:, j] * u[src]
    return y


def query_temperature(T, coef, every, dtype):
    p = torch.arange(T, dtype=dtype)
    return 1.0 + coef * torch.log(torch.floor((p + 1) / every) + 1.0)


def attention_weights(q, k, scale, r1, r2, window):
    """q [T, H, D], k [T, G, D] -> softmax weights [H, T, T] with the distance bias and the
    sliding window (query i sees key j iff 0 <= i - j < window)."""
    T, H, _ = q.shape
    G = k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    dist = (i - j)
    visible = (dist >= 0) & (dist < window)
    out = torch.zeros(H, T, T, dtype=q.dtype)
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        s = s - r1[h] * torch.log(1.0 + r2[h] * dist.clamp(min=0).to(q.dtype))
        s = s.masked_fill(~visible, float("-inf"))
        out[h] = torch.softmax(s, dim=-1)
    return out


def mix_heads(weights, talk):
    """w'_h = sum_g talk[h, g] w_g."""
    return torch.einsum("hg,gij->hij", talk, weights)


def apply_weights(weights, v):
    """weights [H, T, T], v [T, G, D] -> [T, H D]; head h reads kv head h // (H / G)."""
    H, G = weights.shape[0], v.shape[1]
    return torch.stack([weights[h] @ v[:, h // (H // G)] for h in range(H)], dim=1).reshape(v.shape[0], -1)


def attention_mixer(h, W, prefix, m):
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = h @ W[prefix + "q"].T
    k = h @ W[prefix + "k"].T
    q = causal_conv(q, W[prefix + "q.conv"])            # (one tap: a factor per channel)
    k = causal_conv(k, W[prefix + "k.conv"])
    q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype)[:, None]
    q, k = q.view(T, H, D), k.view(T, G, D)
    w = attention_weights(q, k, m["scale"], W[prefix + "r1"], W[prefix + "r2"], m["mask"]["size"])
    o = apply_weights(mix_heads(w, W[prefix + "talk"]), k)           # the values are the keys
    return (o * torch.sigmoid(h @ W[prefix + "g"].T)) @ W[prefix + "o"].T


def feed_forward(h, W, prefix):
    gate = h @ W[prefix + "gate"].T
    return ((gate * torch.sigmoid(gate)) * (h @ W[prefix + "up"].T)) @ W[prefix + "down"].T


def norm(x, W, name):
    return dynamic_tanh(x, W[name], W[name + ".b"], W[name + ".alpha"])


def forward_logits(cfg, W, ids: List[int], streams: Optional[list] = None) -> torch.Tensor:
    x = W["embed"][torch.tensor(ids, dtype=torch.long)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + norm(attention_mixer(norm(x, W, p + "norm1"), W, p + "mix.", layer["mixer"]), W, p + "norm1b")
        if layer["mlp"] is not None:
            x = x + norm(feed_forward(norm(x, W, p + "norm2"), W, p + "mlp."), W, p + "norm2b")
        if streams is not None:
            streams.append(x.clone())
    return norm(x, W, "final.norm") @ W["head"].T


def greedy(cfg, W, prompt: List[int], steps: int) -> List[int]:
    ids = list(prompt)
    for _ in range(steps):
        ids.append(int(torch.argmax(forward_logits(cfg, W, ids)[-1])))
    return ids[len(prompt):]
