"""Tiny Dezelorn configurations for the tests.  They differ in every size and constant and
include the values a model could happen to make equal or 1: one kv head, as many kv heads as
heads, one tap (a factor per channel, no state), a window of one key, a window longer than any
request, a temperature that changes every few tokens, layers without a feed-forward and
layers that differ inside one model, head sizes the tensor-core kernels take (16, 32, 64) and
one they do not (24); a third model has sizes that fit no 16-byte access."""

from __future__ import annotations


def _mixer(heads, kv, dim, conv, window, coef, every, scale):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "conv": conv, "scale": scale,
            "mask": {"size": window}, "q_temp": {"coef": coef, "every": every}}


def _layer(mixer, ff):
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


P = {"architecture": "Dezelorn", "vocab": 211, "width": 48, "embedding": {"scale": 6.0},
     "norm": {"eps": 1e-6},
     "layers": [_layer(_mixer(6, 3, 16, 3, 12, 0.4, 5, 0.3), 72),
                _layer(_mixer(2, 1, 32, 5, 33, 0.2, 16, 0.2), None),
                _layer(_mixer(4, 4, 16, 1, 1000, 0.5, 3, 0.25), 40)]}
Q = {"architecture": "Dezelorn", "vocab": 300, "width": 80, "embedding": {"scale": 9.0},
     "norm": {"eps": 1e-5},
     "layers": [_layer(_mixer(6, 2, 64, 3, 70, 0.35, 32, 0.11), 120),
                _layer(_mixer(3, 1, 24, 2, 1, 0.1, 7, 0.2), 96),
                _layer(_mixer(8, 2, 32, 6, 17, 0.25, 64, 0.15), None),
                _layer(_mixer(2, 2, 64, 2, 130, 0.6, 10, 0.12), 64)]}
# sizes that no 16-byte access fits: odd width, head sizes 20 and 10, 3 kv heads for 3 heads
R = {"architecture": "Dezelorn", "vocab": 97, "width": 50, "embedding": {"scale": 4.0},
     "norm": {"eps": 1e-5},
     "layers": [_layer(_mixer(3, 3, 20, 2, 25, 0.45, 4, 0.22), 30),
                _layer(_mixer(2, 1, 10, 3, 9, 0.15, 11, 0.4), 18)]}
CASES = {"P": (P, 5, 8), "Q": (Q, 9, 16), "R": (R, 13, 4)}        # config, seed, page size
STD_OF = {"embed": 0.12, "head": 0.1, ".mix.q": 0.25, ".mix.k": 0.25, ".conv": 0.5}


def make_model(folder: str, cfg: dict, seed: int) -> str:
    from servelab_b200.config import config_from_dict
    from servelab_b200.weights import write_random_model
    return write_random_model(folder, config_from_dict(cfg), seed, std=0.15, norm_std=0.3, std_of=STD_OF)
