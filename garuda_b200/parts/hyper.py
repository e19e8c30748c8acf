"""A residual kept as several streams, and the layer arrangement that uses it.

In place of one residual ``x`` a model keeps ``S`` streams ``x_1 .. x_S`` (all
equal to the embedding's output at the start; the model's output is their sum).
A sublayer ``f`` with its norm ``n`` reads a weighted sum of the streams and
its output goes to every stream while the streams are mixed among themselves:

    u    = sum_s a_s x_s
    y    = f(n(u))
    x_t' = sum_s M[s, t] x_s + b_t y          (all t at once, from the old streams)

``a`` (``in``, ``[S]``), ``b`` (``out``, ``[S]``) and ``M`` (``mix``, ``[S, S]``,
indexed ``[from, to]``) are learned, per sublayer. The three are held in 32-bit,
as the streams are. With ``S = 1``, ``a = b = M = 1`` this is the ordinary
pre-norm residual.

Two kernels per sublayer: the weighted sum with the norm behind it (one pass
over the streams, the normed row written in the compute dtype), and the update
of all streams from the sublayer's 32-bit output. Where the next sublayer
follows at once, its read is fused into this sublayer's write (one pass over
the streams in place of two).
"""
from __future__ import annotations

from .base import Connection, PartSpec, TensorSpec, build_part, register_block, register_connection
from .block import BlockSpec


@register_connection("stream_mixing")
class StreamMixing(Connection):
    graph_safe = True
    #: the widest row whose weighted sum the fused write keeps in shared memory for the norm; wider
    #: rows are read by a kernel of their own
    FUSED_READ_WIDTH = 10240

    def __init__(self, streams: int, in_name: str = "in", out_name: str = "out", mix_name: str = "mix"):
        if streams < 1:
            raise ValueError(f"a residual has at least one stream, got {streams}")
        self.streams = int(streams)
        self.in_name, self.out_name, self.mix_name = in_name, out_name, mix_name

    def tensors(self):
        S = self.streams
        return {self.in_name: TensorSpec((S,), role="vector", init=("normal_about_one", 0.2)),
                self.out_name: TensorSpec((S,), role="vector", init=("normal_about_one", 0.2)),
                self.mix_name: TensorSpec((S, S), role="vector", init=("normal_about_identity", 0.15))}

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.w_in = tensors[self.in_name].float().contiguous()
        self.w_out = tensors[self.out_name].float().contiguous()
        self.w_mix = tensors[self.mix_name].float().contiguous()

    def read(self, ctx, x, norm):
        return norm.forward(ctx, x, stream_weights=self.w_in)

    def write(self, ctx, x, y, then=None):
        """Updates the streams from the sublayer's output ``y``. ``then = (connection, norm)``: the
        sublayer that follows at once; its normed input is computed in the same pass and returned."""
        if then is None or x.shape[2] > self.FUSED_READ_WIDTH:
            self.ops.streams_update(x, self.w_mix, self.w_out, y)
            return None
        nxt, norm = then
        out = ctx.ws.get("normed", (x.shape[0], norm.width), norm.dtype)
        self.ops.streams_update(x, self.w_mix, self.w_out, y, next_in=nxt.w_in, norm_weight=norm.weight,
                                eps=norm.eps, normed=out)
        return out


@register_block("stream_pre_norm")
class StreamPreNormBlock:
    """A pre-norm layer over a residual of several streams: ``BlockSpec.mixer_connection`` and
    ``BlockSpec.feed_forward_connection`` name the connection parts of its two sublayers. The
    mixer and the feed-forward are run without a residual to add into: they return their output
    (32-bit), which the connection spreads over the streams."""

    def __init__(self, spec: BlockSpec):
        if spec.mixer_connection is None or (spec.feed_forward is not None and spec.feed_forward_connection is None):
            raise ValueError("a layer over streams needs a connection for each of its sublayers")
        if spec.residual_mult != 1.0 or spec.branches:
            raise ValueError("a layer over streams takes no residual multiplier and no branches")
        self.spec = spec
        self.mixer = build_part("mixer", spec.mixer)
        self.mixer_norm = build_part("norm", spec.mixer_norm)
        self.mixer_connection = build_part("connection", spec.mixer_connection)
        self.feed_forward = build_part("feed_forward", spec.feed_forward) if spec.feed_forward else None
        self.feed_forward_norm = build_part("norm", spec.feed_forward_norm) if spec.feed_forward else None
        self.feed_forward_connection = (build_part("connection", spec.feed_forward_connection)
                                        if spec.feed_forward else None)

    def parts(self):
        s = self.spec
        out = [(self.mixer_norm, s.mixer_norm.prefix), (self.mixer_connection, s.mixer_connection.prefix),
               (self.mixer, s.mixer.prefix)]
        if self.feed_forward is not None:
            out += [(self.feed_forward_norm, s.feed_forward_norm.prefix),
                    (self.feed_forward_connection, s.feed_forward_connection.prefix),
                    (self.feed_forward, s.feed_forward.prefix)]
        return out

    @property
    def graph_safe(self):
        return all(part.graph_safe for part, _ in self.parts())

    def first_read(self):
        """(connection, norm) of this layer's first sublayer, for the layer in front to fuse into
        its last write."""
        return self.mixer_connection, self.mixer_norm

    def forward(self, ctx, x, cache, pending=None, next_norm=None, normed=None, then=None):
        """``x``: the streams ``[T, S, d]``. ``normed``: this layer's first normed input, where the
        layer in front has computed it already. ``then``: the next layer's ``first_read()``; its
        normed input is then returned."""
        fuse = hasattr(ctx.ops, "streams_update") and getattr(ctx.ops, "fuses_stream_reads", False)
        h = normed if normed is not None else self.mixer_connection.read(ctx, x, self.mixer_norm)
        y = self.mixer.forward(ctx, h, cache)
        if self.feed_forward is None:
            return self.mixer_connection.write(ctx, x, y, then if fuse else None)
        h2 = self.mixer_connection.write(ctx, x, y, (self.feed_forward_connection, self.feed_forward_norm) if fuse else None)
        if h2 is None:
            h2 = self.feed_forward_connection.read(ctx, x, self.feed_forward_norm)
        y2 = self.feed_forward.forward(ctx, h2)
        return self.feed_forward_connection.write(ctx, x, y2, then if fuse else None)
