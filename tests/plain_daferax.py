"""A plain, slow implementation of the Daferax decoder: whole sequences, float64, no cache,
one function per mechanism.  It shares no code with the package; the tests compare the
engine with it.

Notation: x [T, w] is the residual stream of one sequence, p = 0..T-1 the positions.  A layer is
x <- x + LN1(mix(x)); x <- x + LN2(ff(x)): the sublayers read x itself and only their results
are normed (layer norm with weight and bias).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------ norms
def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


# --------------------------------------------------------------- rotation
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency per pair [dims/2], factor on cos and sin)."""
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, pos, dims: int, base: float, scaling: Optional[dict] = None):
    """x [T, heads, D]: the first ``dims`` elements of every head are rotated, element 2i with
    element 2i+1, by the angle pos * f_i; the rest pass."""
    f, mag = rotary_frequencies(dims, base, scaling)
    a = pos.to(F64)[:, None] * f[None, :]                    # [T, dims/2]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---------------------------------------------------------------- scores
def visible(T: int, window: Optional[int]):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window:
        ok &= (i - j) < window
    return ok


def softmax_attention(q, k, v, scale, window):
    """q [T, H, Dk], k [T, H, Dk], v [T, H, Dv] (already one key head per query head)."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~visible(T, window)[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(s, dim=-1), v)


# ---------------------------------------------------------------- mixers
def attention_mixer(h, W: Dict[str, torch.Tensor], pre: str, m: dict, eps: float, pos, shared: dict):
    """Grouped-query attention with normed, rotated queries and keys, values mixed with those of
    the first value-mixing layer, and a gate per head."""
    T = h.shape[0]
    H, G = int(m["heads"]), int(m.get("kv_heads", m["heads"]))
    D, Dv = int(m["dim"]), int(m.get("vdim", m["dim"]))
    q = (h @ W[pre + "q"].T).view(T, H, D)
    k = (h @ W[pre + "k"].T).view(T, G, D)
    v = (h @ W[pre + "v"].T).view(T, G, Dv)
    q = rms_norm(q, W[pre + "q.norm"], eps)
    k = rms_norm(k, W[pre + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, pos, int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        k = rotate_pairs(k, pos, int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = W[pre + "vmix"]
            v = (1 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    rep = H // G
    o = softmax_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1),
                          float(m["scale"]), (m.get("mask") or {}).get("size"))
    gate = torch.sigmoid(h @ W[pre + "g"].T)                 # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * Dv) @ W[pre + "o"].T


def latent_attention_mixer(h, W, pre: str, m: dict, eps: float, pos, shared: dict):
    """Keys and values of all heads are expanded from one normed latent vector per token; a
    rotated key part is shared by the heads; the result is gated element by element."""
    T = h.shape[0]
    H, D, Dr, Dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = m["rot"]
    q = (h @ W[pre + "q"].T).view(T, H, D + Dr)
    down = h @ W[pre + "dkv"].T                              # [T, R + Dr]
    c = rms_norm(down[:, :R], W[pre + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, None, R:], pos, Dr, float(rot["base"]), rot.get("scaling"))
    q_rot = rotate_pairs(q[..., D:], pos, Dr, float(rot["base"]), rot.get("scaling"))
    k_plain = (c @ W[pre + "uk"].T).view(T, H, D)
    v = (c @ W[pre + "uv"].T).view(T, H, Dv)
    qq = torch.cat([q[..., :D], q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, Dr)], dim=-1)
    o = softmax_attention(qq, kk, v, float(m["scale"]), (m.get("mask") or {}).get("size"))
    o = o.reshape(T, H * Dv) * torch.sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


MIXERS = {"attention": attention_mixer, "latent_attention": latent_attention_mixer}


# ---------------------------------------------------------- feed-forward
def gated_ff(h, W, pre: str):
    z = h @ W[pre + "gate"].T
    return (z * torch.sigmoid(z) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def route(h, W, pre: str, r: dict):
    """(chosen experts [T, top], their weights [T, top])."""
    s = torch.softmax(h @ W[pre + "router"].T, dim=-1)
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups")
    allowed = s
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        best = s.view(-1, n, E // n).max(-1).values.topk(keep, dim=-1).indices      # [T, keep]
        ok = torch.zeros(s.shape[0], n, dtype=torch.bool)
        ok.scatter_(1, best, True)
        allowed = s.masked_fill(~ok.repeat_interleave(E // n, 1), -1.0)
    idx = allowed.topk(top, dim=-1).indices
    return idx, s.gather(1, idx) * float(r.get("scale", 1.0))


def moe_ff(h, W, pre: str, mlp: dict):
    idx, wgt = route(h, W, pre, mlp["router"])
    out = torch.zeros(h.shape[0], W[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(idx[t].tolist(), wgt[t]):
            out[t] += g * gated_ff(h[t:t + 1], W, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_ff(h, W, pre + "shared.")
    return out


def feed_forward(h, W, pre: str, mlp: dict):
    return moe_ff(h, W, pre, mlp) if mlp["kind"] == "moe" else gated_ff(h, W, pre)


# ------------------------------------------------------------------ model
def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], streams: Optional[list] = None):
    """Logits [T, vocab] of one sequence; ``streams`` (a list) receives x after every layer."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    pos = torch.arange(len(tokens))
    x = W["embed"][torch.tensor(tokens)]
    shared: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a = MIXERS[layer["type"]](x, W, p + "mix.", layer["mixer"], eps, pos, shared)
        x = x + layer_norm(a, W[p + "norm1"], W[p + "norm1.b"], eps)
        if layer.get("mlp"):
            f = feed_forward(x, W, p + "mlp.", layer["mlp"])
            x = x + layer_norm(f, W[p + "norm2"], W[p + "norm2.b"], eps)
        if streams is not None:
            streams.append(x.clone())
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return x @ W["embed"].T


def greedy(cfg, W, prompt: List[int], steps: int) -> List[int]:
    ids = list(prompt)
    for _ in range(steps):
        ids.append(int(torch.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]


def load_folder(folder: str):
    """(config dict, name -> float64 tensor) of a model folder; reads the safetensors file
    itself: 8 bytes of header length, the JSON header, then the data."""
    import json
    import os
    import struct
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        raw = f.read()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32}
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + a:8 + n + b]), dtype=kinds[meta["dtype"]])
        out[name] = t.to(F64).reshape(meta["shape"])
    return cfg, out
