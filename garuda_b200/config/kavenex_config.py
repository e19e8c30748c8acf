"""Typed configuration of the Kavenex design, read from its config.json.

Keys: ``architecture`` ("Kavenex"), ``vocab``, ``width``, ``embedding.scale``,
``norm.eps``, ``residual_mult``, ``layers`` (a list; each entry has ``type``, the
mixer's sizes under ``mixer`` and its feed-forward under ``mlp`` or null),
``loop`` (``start``, ``stop``, ``times``; optional), ``token_side.dim``
(optional), ``max_positions`` (optional: the longest sequence; the design itself
has no limit). Every size and constant of a model comes from here; a key that
is missing where the design needs it is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from .model_config import ConfigError

MIXER_TYPES = ("latent_attention",)
MLP_KINDS = ("dense", "moe")
DEFAULT_MAX_POSITIONS = 32768


def _get(d, key, where, kind=None, minimum=None):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json is missing '{where}{key}'")
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int) or (minimum is not None and v < minimum):
            raise ConfigError(f"config.json: '{where}{key}' must be an integer >= {minimum}, got {v!r}")
    elif kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{where}{key}' must be a number, got {v!r}")
        v = float(v)
        if minimum is not None and not v > minimum:
            raise ConfigError(f"config.json: '{where}{key}' must be larger than {minimum}, got {v!r}")
    return v


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int            # unrotated query/key channels per head
    rot_dim: int        # rotated query/key channels per head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int       # how many of the rotated part's first channels are turned


@dataclass(frozen=True)
class ExpertConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class MlpConfig:
    kind: str                                   # "dense" | "moe"
    ff: int = 0                                 # dense
    experts: int = 0                            # moe ...
    top: int = 0
    expert: Optional[ExpertConfig] = None
    shared: Optional[ExpertConfig] = None


@dataclass(frozen=True)
class KavenexLayer:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class KavenexConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    residual_mult: float
    layers: Tuple[KavenexLayer, ...]
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times)
    side_dim: Optional[int] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()
    raw: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "KavenexConfig":
        vocab = _get(d, "vocab", "", int, 1)
        width = _get(d, "width", "", int, 1)
        scale = _get(d.get("embedding"), "scale", "embedding.", float)
        eps = _get(d.get("norm"), "eps", "norm.", float, 0.0)
        mult = _get(d, "residual_mult", "", float)
        entries = _get(d, "layers", "")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            w = f"layers[{i}]."
            kind = _get(e, "type", w)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{w}type' = {kind!r} is not a mixer of this design {MIXER_TYPES}")
            m = _get(e, "mixer", w)
            rot = _get(m, "rot", w + "mixer.")
            rot_dim = _get(m, "rot_dim", w + "mixer.", int, 0)
            rot_dims = _get(rot, "dims", w + "mixer.rot.", int, 0)
            if rot_dims % 2 or rot_dims > rot_dim:
                raise ConfigError(f"config.json: '{w}mixer.rot.dims' = {rot_dims} must be even and at most rot_dim = {rot_dim}")
            mixer = LatentMixerConfig(
                heads=_get(m, "heads", w + "mixer.", int, 1), dim=_get(m, "dim", w + "mixer.", int, 1),
                rot_dim=rot_dim, vdim=_get(m, "vdim", w + "mixer.", int, 1),
                kv_rank=_get(m, "kv_rank", w + "mixer.", int, 1), scale=_get(m, "scale", w + "mixer.", float, 0.0),
                rot_base=_get(rot, "base", w + "mixer.rot.", float, 0.0), rot_dims=rot_dims)
            mlp = None
            if e.get("mlp") is not None:
                f = e["mlp"]
                mk = _get(f, "kind", w + "mlp.")
                if mk not in MLP_KINDS:
                    raise ConfigError(f"config.json: '{w}mlp.kind' = {mk!r} is not one of {MLP_KINDS}")
                if mk == "dense":
                    mlp = MlpConfig("dense", ff=_get(f, "ff", w + "mlp.", int, 1))
                else:
                    r, x = _get(f, "router", w + "mlp."), _get(f, "expert", w + "mlp.")
                    experts, top = _get(r, "experts", w + "mlp.router.", int, 1), _get(r, "top", w + "mlp.router.", int, 1)
                    if top > experts:
                        raise ConfigError(f"config.json: '{w}mlp.router.top' = {top} exceeds the {experts} experts")
                    shared = None
                    if f.get("shared") is not None:
                        shared = ExpertConfig(_get(f["shared"], "ff", w + "mlp.shared.", int, 1),
                                              _get(f["shared"], "limit", w + "mlp.shared.", float, 0.0))
                    mlp = MlpConfig("moe", experts=experts, top=top, shared=shared,
                                    expert=ExpertConfig(_get(x, "ff", w + "mlp.expert.", int, 1),
                                                        _get(x, "limit", w + "mlp.expert.", float, 0.0)))
            layers.append(KavenexLayer(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            start, stop = _get(lp, "start", "loop.", int, 0), _get(lp, "stop", "loop.", int, 0)
            times = _get(lp, "times", "loop.", int, 1)
            if not start <= stop <= len(layers):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(layers)} layers")
            loop = (start, stop, times)
        side = None
        if d.get("token_side") is not None:
            side = _get(d["token_side"], "dim", "token_side.", int, 1)
        eos = d.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        return cls(architecture=d.get("architecture", "Kavenex"), vocab=vocab, width=width, embedding_scale=scale,
                   eps=eps, residual_mult=mult, layers=tuple(layers), loop=loop, side_dim=side,
                   max_positions=int(d.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_ids=eos, raw=dict(d))

    def to_dict(self) -> dict:
        return dict(self.raw)
