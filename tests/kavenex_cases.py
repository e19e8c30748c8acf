"""Tiny Kavenex configurations of the tests, their model folders and plain logits.

The configurations differ from one another in every size and option: head
counts, widths that are no power of two, the order of dense, routed and absent
feed-forwards, a rotation narrower than the rotated part, with and without a
loop (also a loop that starts at layer 0 and one that runs once), with and
without the token branch or a shared expert, a residual multiplier and an
embedding scale of exactly 1.
"""
from __future__ import annotations

import tempfile

import numpy as np
import torch


def _mixer(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
            "rot": {"base": base, "dims": rot_dim if dims is None else dims}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": shared}


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


KA = {"architecture": "Kavenex", "vocab": 211, "width": 48, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
      "residual_mult": 0.5, "token_side": {"dim": 8},
      "layers": [_layer(_mixer(2, 16, 8, 24, 40, 0.2), _moe(6, 2, 24, 1.5, {"ff": 40, "limit": 0.75})),
                 _layer(_mixer(2, 16, 8, 24, 40, 0.2), _dense(72)),
                 _layer(_mixer(2, 16, 8, 24, 40, 0.2), None)],
      "loop": {"start": 0, "stop": 2, "times": 3}}

# three heads, a rotation that turns only part of the rotated channels, no loop, no token branch, a
# routed layer without a shared expert, every expert chosen (top = experts), multipliers of exactly 1
KB = {"architecture": "Kavenex", "vocab": 97, "width": 40, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
      "residual_mult": 1.0,
      "layers": [_layer(_mixer(3, 8, 12, 10, 20, 0.3, base=500000.0, dims=8), _dense(56)),
                 _layer(_mixer(3, 8, 12, 10, 20, 0.3, base=500000.0, dims=8), _moe(3, 3, 16, 3.0))]}

# layers whose mixers differ in every size, a loop over the last layer alone that runs once, one head
KC = {"architecture": "Kavenex", "vocab": 150, "width": 64, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-5},
      "residual_mult": 0.25, "token_side": {"dim": 4},
      "layers": [_layer(_mixer(1, 32, 16, 32, 48, 0.15), _moe(9, 1, 20, 1.0, {"ff": 12, "limit": 2.0})),
                 _layer(_mixer(4, 8, 4, 12, 16, 0.35, base=100.0), _dense(100))],
      "loop": {"start": 1, "stop": 2, "times": 1}}

# sizes that the tensor-core products take (multiples of 64), four heads, a loop in the middle
KD = {"architecture": "Kavenex", "vocab": 320, "width": 128, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-5},
      "residual_mult": 0.4, "token_side": {"dim": 16},
      "layers": [_layer(_mixer(4, 32, 32, 32, 64, 0.12), _dense(192)),
                 _layer(_mixer(4, 32, 32, 32, 64, 0.12), _moe(8, 2, 64, 2.0, {"ff": 64, "limit": 1.0})),
                 _layer(_mixer(4, 32, 32, 32, 64, 0.12), _dense(256))],
      "loop": {"start": 1, "stop": 3, "times": 2}}

CASES = {"KA": (KA, 11), "KB": (KB, 12), "KC": (KC, 13), "KD": (KD, 14)}

# Random N(0, 0.02) weights give scores so close to zero that every key weighs the same; these
# factors spread the scores (so that a wrong position, rotation or page shows), the router's
# logits (so that no choice is a close call) and the activations (so that the clamps bite).
SHARPEN = {"mix.q": 12.0, "mix.dkv": 10.0, "mix.uk": 8.0, "mix.uv": 4.0, "mix.o": 4.0, ".router": 40.0,
           ".gate": 6.0, ".up": 6.0, ".down": 4.0, "side.proj": 4.0, "head": 4.0, "embed": 20.0, "loop.step": 30.0}

_DIRS, _PLAIN = {}, {}


def model_dir(name: str, store_dtype=torch.float32) -> str:
    from garuda_b200.weights import write_random_model
    key = (name, store_dtype)
    if key not in _DIRS:
        cfg, seed = CASES[name]
        d = tempfile.mkdtemp(prefix=f"garuda_kavenex_{name}_")
        write_random_model(d, cfg, seed, norm_init=("normal_about_one", 0.1), store_dtype=store_dtype, scale=SHARPEN)
        _DIRS[key] = d
    return _DIRS[key]


def weights(name: str, store_dtype=torch.float32) -> dict:
    from tests.helpers import folder_weights
    return folder_weights(model_dir(name, store_dtype))


def plain_logits(name: str, store_dtype, tokens) -> np.ndarray:
    from tests.plain import kavenex_plain
    key = (name, store_dtype, tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = kavenex_plain.forward(CASES[name][0], weights(name, store_dtype), tokens).astype(np.float32)
    return _PLAIN[key]


def random_tokens(name: str, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, CASES[name][0]["vocab"], n).tolist()
