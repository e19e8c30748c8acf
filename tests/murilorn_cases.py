"""Tiny Murilorn configurations of the tests, their model folders and plain logits.

The configurations differ from one another in every size and option: with
streams (3, 2, 1) and without, loops at the start, over one layer, none;
attention with keys and values of unequal widths, windows shorter and longer
than a page, no kept first positions and more than a page of them, no mask at
all, with and without capped scores; delta-rule layers with fewer query/key
heads than heads, two to five taps, key widths that are no multiple of 32;
one, several and all experts per token; layers without a feed-forward.
"""
from __future__ import annotations

import tempfile

import numpy as np
import torch


def _attn(heads, kv_heads, dim, vdim, scale, softcap=None, size=None, keep_first=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep_first or 0}
    return {"type": "attention", "mixer": m}


def _delta(heads, kv_heads, dim, vdim, conv, decay_rank=6, gate_rank=10):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# three streams, a loop in the middle that runs twice, a window shorter than a page of 8 with three kept
# positions, values wider than keys, a delta layer whose heads share query/key heads, a layer without
# a feed-forward
MA = {"architecture": "Murilorn", "vocab": 157, "width": 48, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
      "streams": 3, "logit_scale": 0.25, "logit_softcap": 12.0,
      "layers": [_layer(_delta(4, 2, 12, 20, 3), _moe(5, 2, 24)),
                 _layer(_attn(4, 2, 16, 24, 0.25, softcap=8.0, size=6, keep_first=3), _moe(5, 2, 24)),
                 _layer(_delta(2, 2, 20, 8, 2), None),
                 _layer(_attn(2, 1, 8, 12, 0.35, softcap=20.0, size=21, keep_first=10), _moe(4, 4, 16))],
      "loop": {"start": 1, "stop": 3, "times": 2}}

# one plain residual (no streams), no loop, attention without a mask and without capped scores, as
# many query/key heads as heads everywhere, one expert per token, no cap on the logits
MB = {"architecture": "Murilorn", "vocab": 97, "width": 40, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
      "logit_scale": 1.0,
      "layers": [_layer(_attn(3, 3, 8, 8, 0.3), _moe(3, 1, 20)),
                 _layer(_delta(3, 3, 8, 12, 5, decay_rank=4, gate_rank=4), _moe(6, 1, 12))]}

# a single stream with learned weights, a loop over everything that runs three times, a window of one
# position with one kept, one head
MC = {"architecture": "Murilorn", "vocab": 120, "width": 32, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-5},
      "streams": 1, "logit_scale": 2.0, "logit_softcap": 30.0,
      "layers": [_layer(_attn(1, 1, 24, 16, 0.2, softcap=5.0, size=1, keep_first=1), None),
                 _layer(_delta(1, 1, 40, 36, 4), _moe(2, 2, 16))],
      "loop": {"start": 0, "stop": 2, "times": 3}}

# sizes the tensor-core kernels take (multiples of 64 and 16), two streams, a window of three pages of 16.
# Every expert is chosen (top = experts): this is the configuration that is compared with the plain
# model position by position in bfloat16 over five runs of routed layers, where a choice among random
# routers' scores is a close call (within the rounding of the bfloat16 input) for a few tokens in a
# hundred; the choice itself is tested by the other configurations.
MD = {"architecture": "Murilorn", "vocab": 320, "width": 128, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-5},
      "streams": 2, "logit_scale": 0.5, "logit_softcap": 20.0,
      "layers": [_layer(_attn(4, 2, 64, 64, 0.125, softcap=25.0, size=40, keep_first=2), _moe(4, 4, 64)),
                 _layer(_delta(4, 2, 32, 64, 4, decay_rank=16, gate_rank=16), _moe(3, 3, 64)),
                 _layer(_attn(8, 2, 32, 32, 0.18, softcap=25.0, size=70, keep_first=17), _moe(2, 2, 64))],
      "loop": {"start": 0, "stop": 2, "times": 2}}

# attention alone, one layer, no streams: what a query reads is exactly its mask
ME = {"architecture": "Murilorn", "vocab": 64, "width": 32, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
      "logit_scale": 1.0,
      "layers": [_layer(_attn(2, 1, 16, 8, 0.25, softcap=10.0, size=9, keep_first=2), None)]}

CASES = {"MA": (MA, 21), "MB": (MB, 22), "MC": (MC, 23), "MD": (MD, 24), "ME": (ME, 25)}

# Random N(0, 0.02) weights give scores so close to zero that every key weighs the same; these
# factors spread the scores (so that a wrong key, mask or page shows), the router's logits (so
# that no choice is a close call), the delta rule's writes and the logits. Not sharper than this:
# with scores of the order of ten the softmax, and with decay logits of the order of fifty the
# decay, turn the bfloat16 rounding of their inputs into changes of tens of per cent, which says
# nothing about the kernels.
SHARPEN = {"mix.q": 5.0, "mix.k": 5.0, "mix.v": 6.0, "mix.o": 5.0, "mix.b": 8.0, "mix.a1": 3.0, "mix.a2": 3.0,
           "mix.g1": 4.0, "mix.g2": 4.0, ".router": 20.0, ".gate": 6.0, ".up": 6.0, ".down": 4.0, "head": 6.0,
           "embed": 25.0}

_DIRS, _PLAIN = {}, {}


def model_dir(name: str, store_dtype=torch.float32) -> str:
    from garuda_b200.weights import write_random_model
    key = (name, store_dtype)
    if key not in _DIRS:
        cfg, seed = CASES[name]
        d = tempfile.mkdtemp(prefix=f"garuda_murilorn_{name}_")
        write_random_model(d, cfg, seed, store_dtype=store_dtype, scale=SHARPEN)
        _DIRS[key] = d
    return _DIRS[key]


def weights(name: str, store_dtype=torch.float32) -> dict:
    from tests.helpers import folder_weights
    return folder_weights(model_dir(name, store_dtype))


def plain_logits(name: str, store_dtype, tokens) -> np.ndarray:
    from tests.plain import murilorn_plain
    key = (name, store_dtype, tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = murilorn_plain.forward(CASES[name][0], weights(name, store_dtype), tokens).astype(np.float32)
    return _PLAIN[key]


def random_tokens(name: str, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, CASES[name][0]["vocab"], n).tolist()
