"""Typed configuration of the Murilorn design, read from its config.json.

Keys: ``architecture`` ("Murilorn"), ``vocab``, ``width``, ``embedding.scale``,
``norm.eps``, ``streams`` (optional: the residual is kept as that many streams;
absent: one plain residual), ``logit_scale``, ``logit_softcap`` (optional),
``layers`` (a list; each entry has ``type`` = ``attention`` | ``channel_delta``,
the mixer's sizes under ``mixer`` and its feed-forward under ``mlp`` or null),
``loop`` (``start``, ``stop``, ``times``; optional), ``max_positions`` (optional:
the longest sequence; the design itself has no limit).

``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap``
(optional), ``mask.size`` and ``mask.keep_first`` (optional: no ``mask``, every
earlier position is read). ``channel_delta``: ``heads``, ``kv_heads``, ``dim``,
``vdim``, ``conv`` (taps); the ranks of its two low-rank projections come from the
tensors (``decay_rank`` / ``gate_rank`` may name them for random weights).
``mlp``: ``kind`` = ``moe``, ``router.experts``, ``router.top``, ``expert.ff``.
Every size and constant of a model comes from here; a key that is missing where
the design needs it is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from .kavenex_config import _get
from .model_config import ConfigError

MIXER_TYPES = ("attention", "channel_delta")
DEFAULT_MAX_POSITIONS = 32768


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]        # mask.size: positions a query looks back over, itself included
    keep_first: int              # mask.keep_first


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None


@dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class MurilornLayer:
    type: str
    mixer: object
    mlp: Optional[MoeConfig]


@dataclass(frozen=True)
class MurilornConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: Tuple[MurilornLayer, ...]
    streams: Optional[int] = None
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()
    raw: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "MurilornConfig":
        vocab = _get(d, "vocab", "", int, 1)
        width = _get(d, "width", "", int, 1)
        scale = _get(d.get("embedding"), "scale", "embedding.", float)
        eps = _get(d.get("norm"), "eps", "norm.", float, 0.0)
        entries = _get(d, "layers", "")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            w = f"layers[{i}]."
            kind = _get(e, "type", w)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{w}type' = {kind!r} is not a mixer of this design {MIXER_TYPES}")
            m, wm = _get(e, "mixer", w), w + "mixer."
            heads, kv_heads = _get(m, "heads", wm, int, 1), _get(m, "kv_heads", wm, int, 1)
            if heads % kv_heads:
                raise ConfigError(f"config.json: '{wm}heads' = {heads} is not a multiple of '{wm}kv_heads' = {kv_heads}")
            dim, vdim = _get(m, "dim", wm, int, 1), _get(m, "vdim", wm, int, 1)
            if kind == "attention":
                window, keep = None, 0
                if m.get("mask") is not None:
                    window = _get(m["mask"], "size", wm + "mask.", int, 1)
                    keep = int(m["mask"].get("keep_first") or 0)
                    if keep < 0:
                        raise ConfigError(f"config.json: '{wm}mask.keep_first' must not be negative")
                cap = m.get("softcap")
                mixer = AttentionMixerConfig(heads, kv_heads, dim, vdim, _get(m, "scale", wm, float, 0.0),
                                             float(cap) if cap else None, window, keep)
            else:
                mixer = DeltaMixerConfig(heads, kv_heads, dim, vdim, _get(m, "conv", wm, int, 1),
                                         m.get("decay_rank"), m.get("gate_rank"))
            mlp = None
            if e.get("mlp") is not None:
                f = e["mlp"]
                mk = _get(f, "kind", w + "mlp.")
                if mk != "moe":
                    raise ConfigError(f"config.json: '{w}mlp.kind' = {mk!r}: this design's feed-forward is 'moe'")
                r, x = _get(f, "router", w + "mlp."), _get(f, "expert", w + "mlp.")
                experts, top = _get(r, "experts", w + "mlp.router.", int, 1), _get(r, "top", w + "mlp.router.", int, 1)
                if top > experts:
                    raise ConfigError(f"config.json: '{w}mlp.router.top' = {top} exceeds the {experts} experts")
                mlp = MoeConfig(experts, top, _get(x, "ff", w + "mlp.expert.", int, 1))
            layers.append(MurilornLayer(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            start, stop = _get(lp, "start", "loop.", int, 0), _get(lp, "stop", "loop.", int, 0)
            times = _get(lp, "times", "loop.", int, 1)
            if not start <= stop <= len(layers):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(layers)} layers")
            loop = (start, stop, times)
        streams = d.get("streams")
        if streams is not None:
            streams = _get(d, "streams", "", int, 1)
            if streams > 16:
                raise ConfigError(f"config.json: 'streams' = {streams}: at most 16 are supported")
        cap = d.get("logit_softcap")
        eos = d.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        return cls(architecture=d.get("architecture", "Murilorn"), vocab=vocab, width=width, embedding_scale=scale,
                   eps=eps, layers=tuple(layers), streams=streams,
                   logit_scale=float(d["logit_scale"]) if d.get("logit_scale") is not None else 1.0,
                   logit_softcap=float(cap) if cap else None, loop=loop,
                   max_positions=int(d.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_ids=eos, raw=dict(d))

    def to_dict(self) -> dict:
        return dict(self.raw)
