"""Tiny Daferax configurations for the tests.  Their layers differ in every size, constant and
order and include the values a model could happen to make equal or 1: one kv head, as many kv
heads as heads, values larger and smaller than keys, rotation of a part of a head and of all of
it, a window of one key, a window beyond any request, no window, one group of experts, one
chosen expert, no shared expert, a dense feed-forward, a layer without feed-forward, a model that
starts with either mixer, and sizes that fit no 16-byte access."""

from __future__ import annotations


def attention(heads, kv, dim, vdim, rot_dims, base, scale, v_mix=False, window=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"base": base, "dims": rot_dims}}
    if v_mix:
        m["v_mix"] = True
    if window:
        m["mask"] = {"size": window}
    return "attention", m


def latent(heads, dim, rot_dim, vdim, rank, base, scale, window=None, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if scaling:
        m["rot"]["scaling"] = scaling
    if window:
        m["mask"] = {"size": window}
    return "latent_attention", m


def moe(experts, top, ff, groups=None, scale=1.0, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}
U = {"architecture": "Daferax", "vocab": 211, "width": 48, "norm": {"eps": 1e-6},
     "layers": [layer(attention(4, 2, 16, 8, 8, 10000.0, 0.3, v_mix=True), moe(6, 2, 24, (3, 2), 1.5, 40)),
                layer(latent(3, 8, 4, 12, 20, 5000.0, 0.25, window=9, scaling=YARN), None),
                layer(attention(2, 2, 8, 8, 8, 300.0, 0.4, v_mix=True, window=5), moe(4, 1, 16)),
                layer(latent(2, 16, 8, 8, 24, 100.0, 0.2), {"kind": "dense", "ff": 56})]}
V = {"architecture": "Daferax", "vocab": 300, "width": 80, "norm": {"eps": 1e-5},
     "layers": [layer(latent(4, 16, 16, 16, 32, 20000.0, 0.15, window=1000), moe(8, 3, 32, (4, 3), 2.0, 24)),
                layer(attention(6, 2, 32, 16, 16, 1000000.0, 0.12, v_mix=True), {"kind": "dense", "ff": 96}),
                layer(latent(2, 8, 2, 24, 40, 700.0, 0.3, window=1,
                             scaling={"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}), moe(8, 2, 16, (2, 1), 0.7)),
                layer(attention(2, 2, 24, 16, 24, 50000.0, 0.2, v_mix=True, window=70), moe(5, 5, 8, None, 1.0, 16)),
                layer(attention(4, 1, 64, 64, 32, 10000.0, 0.11), None)]}
# sizes that no 16-byte access fits
W = {"architecture": "Daferax", "vocab": 97, "width": 50, "norm": {"eps": 1e-5},
     "layers": [layer(attention(3, 3, 10, 6, 4, 900.0, 0.3, window=25), moe(3, 2, 10, None, 1.2, 6)),
                layer(latent(2, 6, 2, 10, 14, 2000.0, 0.35, window=13), moe(6, 2, 14, (2, 1), 2.2))]}
# key and value sizes that are multiples of 64 and differ: the tcgen05 attention for two sizes, with the
# values inside the key rows (latent: 64 + 64 against 64) and apart from them (128 against 64)
X = {"architecture": "Daferax", "vocab": 150, "width": 64, "norm": {"eps": 1e-5},
     "layers": [layer(latent(2, 16, 64, 16, 64, 3000.0, 0.1, window=40,
                             scaling={"factor": 2.0, "original": 48, "fast": 6.0, "slow": 1.0}), moe(4, 2, 16, None, 1.3)),
                layer(attention(2, 1, 128, 64, 64, 40000.0, 0.08), {"kind": "dense", "ff": 48})]}
CASES = {"U": (U, 5, 8), "V": (V, 9, 16), "W": (W, 13, 4), "X": (X, 17, 16)}        # config, seed, page size
# projections drawn large enough that the softmax of a tiny model is peaked and the router's
# choice is clear of ties
STD_OF = {"embed": 0.5, ".mix.q": 0.3, ".mix.k": 0.3, ".mix.dkv": 0.3, ".mix.uk": 0.3, ".router": 0.4}


def make_model(folder: str, cfg: dict, seed: int) -> str:
    """The weights are stored in bfloat16, as a served model's are: what the engine's bfloat16 path
    computes then differs from the oracle by the rounding of activations only."""
    import torch
    from servelab_b200.config import config_from_dict
    from servelab_b200.weights import write_random_model
    return write_random_model(folder, config_from_dict(cfg), seed, dtype=torch.bfloat16, std=0.15,
                              norm_std=0.3, std_of=STD_OF)
