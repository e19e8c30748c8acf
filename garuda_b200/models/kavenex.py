"""The Kavenex decoder as a ``ModelSpec``.

An embedding times a constant; pre-norm layers (layer norm with weight and
bias) of latent attention and a dense gated feed-forward (tanh-form GELU) or
routed experts with a shared one, every part's output scaled by a residual
multiplier; after each layer's feed-forward a gated per-layer token embedding,
RMS-normed, is added; a stretch of the layers may run several times in a row
with the same weights (each pass with a cache of its own; before every pass but
the first the embedding's output is added to the stream, and before every pass a
row of a learned table); a final layer norm and an output head. Tensor names:
``embed``, ``head``, ``final.norm(.b)``, ``loop.step``, ``side.embed``, and per
layer ``l<i>.norm1|norm2(.b)``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``.
"""
from __future__ import annotations

from ..config.kavenex_config import KavenexConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec, TensorSpec
from ..parts.block import BlockSpec
from .decoder import ModelSpec, LayerCall

STEP_TABLE = "loop.step"
SIDE_TABLE = "side.embed"


def _norm(cfg, prefix, name):
    return PartSpec("layer", dict(width=cfg.width, eps=cfg.eps, weight_name=name, bias_name=name + ".b"), prefix=prefix)


def kavenex_spec(cfg: KavenexConfig) -> ModelSpec:
    layers = []
    n = len(cfg.layers)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        mixer = PartSpec("latent_attention", dict(
            width=cfg.width, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank,
            scale=m.scale, eps=cfg.eps, rot_base=m.rot_base, rot_dims=m.rot_dims), prefix=p + "mix.")
        ff = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            ff = PartSpec("gated", dict(width=cfg.width, inner=layer.mlp.ff, activation="gelu_tanh"), prefix=p + "mlp.")
        elif layer.mlp is not None:
            f = layer.mlp
            ff = PartSpec("routed_experts", dict(
                width=cfg.width, experts=f.experts, top=f.top, inner=f.expert.ff, activation="clamped_swish",
                limit=f.expert.limit, shared_inner=f.shared.ff if f.shared else None,
                shared_limit=f.shared.limit if f.shared else 0.0), prefix=p + "mlp.")
        branches = ()
        if cfg.side_dim:
            branches = (PartSpec("token_side", dict(
                width=cfg.width, dim=cfg.side_dim, vocab=cfg.vocab, table=SIDE_TABLE, table_width=n * cfg.side_dim,
                column=i * cfg.side_dim, eps=cfg.eps), prefix=p + "side."),)
        layers.append(BlockSpec(mixer=mixer, feed_forward=ff, mixer_norm=_norm(cfg, p, "norm1"),
                                feed_forward_norm=_norm(cfg, p, "norm2") if ff is not None else None,
                                residual_mult=cfg.residual_mult, branches=branches))
    order, extra = [LayerCall(i) for i in range(n)], {}
    if cfg.loop is not None:
        start, stop, times = cfg.loop
        order = [LayerCall(i) for i in range(start)]
        for t in range(times):
            for i in range(start, stop):
                first = i == start
                order.append(LayerCall(i, add_embedding=first and t > 0, add_row=(STEP_TABLE, t) if first else None))
        order += [LayerCall(i) for i in range(stop, n)]
        extra[STEP_TABLE] = TensorSpec((times, cfg.width), role="vector", init=("normal", 0.02))
    # what a folder may carry although this model reads nothing from it: tensors of mechanisms
    # that its configuration leaves out
    ignored = [f"l{i}.norm2{b}" for i, layer in enumerate(cfg.layers) if layer.mlp is None for b in ("", ".b")]
    if cfg.loop is None:
        ignored.append(STEP_TABLE)
    if not cfg.side_dim:
        ignored += [SIDE_TABLE] + [f"l{i}.side.{t}" for i in range(n) for t in ("gate", "proj", "norm")]
    return ModelSpec(
        architecture=cfg.architecture, width=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding="embed", layers=layers, order=order, final_norm=_norm(cfg, "", "final.norm"), head="head",
        embedding_scale=cfg.embedding_scale, eos_token_ids=cfg.eos_token_ids, extra_tensors=extra or None, ignored_tensors=tuple(ignored))


register_architecture("Kavenex", KavenexConfig.from_dict, kavenex_spec)
