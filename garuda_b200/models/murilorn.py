"""The Murilorn decoder as a ``ModelSpec``.

An embedding times a constant; pre-norm layers (RMS norm whose weight is stored
about zero) whose mixer is either attention without a position encoding (capped
scores, a sliding window that also keeps a request's first positions, a sink in
the softmax, biases, keys and values of widths of their own) or a gated delta
rule with a decay per key channel, and whose feed-forward is a set of routed
experts (sigmoid scores, the score on the expert's input); the residual kept as
several streams that every sublayer reads a weighted sum of and writes to; a
stretch of the layers may run several times in a row with the same weights, each
pass with a cache or state of its own; a final norm, an output head, and logits
scaled and capped. Tensor names: ``embed``, ``head``, ``final.norm``, and per
layer ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.hc1|hc2.in|out|mix``.
"""
from __future__ import annotations

from ..config.murilorn_config import MurilornConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.block import BlockSpec
from .decoder import ModelSpec, LayerCall


def _norm(cfg, prefix, name):
    return PartSpec("rms", dict(width=cfg.width, eps=cfg.eps, weight_name=name, unit_offset=True), prefix=prefix)


def murilorn_spec(cfg: MurilornConfig) -> ModelSpec:
    layers, ignored = [], []
    n = len(cfg.layers)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "attention":
            mixer = PartSpec("capped_sink_attention", dict(
                width=cfg.width, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale,
                softcap=m.softcap, window=m.window, keep_first=m.keep_first, sink=True, bias=True), prefix=p + "mix.")
        else:
            mixer = PartSpec("channel_delta_rule", dict(
                width=cfg.width, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, taps=m.taps, eps=cfg.eps,
                decay_rank=m.decay_rank, gate_rank=m.gate_rank), prefix=p + "mix.")
        ff = None
        if layer.mlp is not None:
            f = layer.mlp
            ff = PartSpec("routed_experts", dict(
                width=cfg.width, experts=f.experts, top=f.top, inner=f.ff, activation="silu", router_bias=False,
                router_score="sigmoid", scale_input=True), prefix=p + "mlp.")
        else:
            ignored += [p + "norm2"] + [f"{p}hc2.{t}" for t in ("in", "out", "mix")]
        kw = {}
        if cfg.streams is not None:
            kw = dict(arrangement="stream_pre_norm",
                      mixer_connection=PartSpec("stream_mixing", dict(streams=cfg.streams), prefix=p + "hc1."),
                      feed_forward_connection=(PartSpec("stream_mixing", dict(streams=cfg.streams), prefix=p + "hc2.")
                                               if ff is not None else None))
        layers.append(BlockSpec(mixer=mixer, feed_forward=ff, mixer_norm=_norm(cfg, p, "norm1"),
                                feed_forward_norm=_norm(cfg, p, "norm2") if ff is not None else None, **kw))
    order = [LayerCall(i) for i in range(n)]
    if cfg.loop is not None:
        start, stop, times = cfg.loop
        order = ([LayerCall(i) for i in range(start)] + [LayerCall(i) for _ in range(times) for i in range(start, stop)]
                 + [LayerCall(i) for i in range(stop, n)])
    return ModelSpec(
        architecture=cfg.architecture, width=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding="embed", layers=layers, order=order, final_norm=_norm(cfg, "", "final.norm"), head="head",
        embedding_scale=cfg.embedding_scale, streams=cfg.streams, logit_scale=cfg.logit_scale,
        logit_softcap=cfg.logit_softcap, eos_token_ids=cfg.eos_token_ids, ignored_tensors=tuple(ignored))


register_architecture("Murilorn", MurilornConfig.from_dict, murilorn_spec)
