"""The arrangement of a layer's parts. ``pre_norm``: h += mixer(norm1(h)); h += feed_forward(norm2(h))
(src/Starlings.Roost.Models.Tiny/RoostTiny.cs:40,49-50,54). The residual stream is carried beside the branch
output so that each residual sum is fused into the norm that follows it; the stream is stored in the
activation dtype and every sum is formed in 32-bit and rounded once."""
from __future__ import annotations

import torch

from ..config.spec import BlockSpec
from .base import CONNECTIONS, FEED_FORWARDS, MIXERS, NORMS, TOKEN_INPUTS, Block, Runtime, register_block


class PreNormBlock(Block):
    def __init__(self, spec: BlockSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.input_norm = NORMS.build(spec.input_norm, runtime)
        self.mixer = MIXERS.build(spec.mixer, runtime)
        self.post_mixer_norm = NORMS.build(spec.post_mixer_norm, runtime)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, runtime)

    def sub_parts(self):
        return {"input_norm": self.input_norm, "mixer": self.mixer, "post_mixer_norm": self.post_mixer_norm,
                "feed_forward": self.feed_forward}

    @classmethod
    def sub_specs(cls, spec: BlockSpec):
        return {"input_norm": (NORMS, spec.input_norm), "mixer": (MIXERS, spec.mixer),
                "post_mixer_norm": (NORMS, spec.post_mixer_norm), "feed_forward": (FEED_FORWARDS, spec.feed_forward)}

    def __call__(self, h, residual, batch, cache, write_cache: bool = True):
        """``h`` is the previous branch output (or the embedding), ``residual`` the stream before it was added
        (None at the first block). Returns the feed-forward's output and the stream it is still to be added to."""
        if residual is None:
            residual = h
            x = self.input_norm(h)
        else:
            x, residual = self.input_norm.add_norm(h, residual)
        a = self.mixer(x, batch, cache, write_cache)
        y, residual = self.post_mixer_norm.add_norm(a, residual)
        return self.feed_forward(y, batch), residual


class PreNormWideBlock(Block):
    """The same arrangement over a stream that is kept and summed in 32-bit whatever the activation dtype is: the
    embedding hands over a float32 stream, every norm reads it (adding the branch output before it first, in 32-bit)
    and writes the activation dtype. The feed-forward and its norm may be absent. With ``token_input`` the layer ends with one
    more sum: what that part makes of the stream's value and the token ids. A run may be handed ``stream_input``, a 32-bit
    tensor that is added to the stream right before the run's first norm (the embedding's output added again)."""

    def __init__(self, spec: BlockSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.input_norm = NORMS.build(spec.input_norm, runtime)
        self.mixer = MIXERS.build(spec.mixer, runtime)
        self.feed_forward = self.post_mixer_norm = None
        if spec.feed_forward is not None:
            if spec.post_mixer_norm is None:
                raise ValueError("pre_norm_wide: a feed-forward needs the norm before it")
            self.post_mixer_norm = NORMS.build(spec.post_mixer_norm, runtime)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, runtime)
        self.token_input = None
        if spec.token_input is not None:
            if not hasattr(self.input_norm, "add_only"):
                raise ValueError(f"pre_norm_wide: a token input needs a norm that hands the stream on without norming it; '{spec.input_norm.kind}' does not")
            self.token_input = TOKEN_INPUTS.build(spec.token_input, runtime)

    def sub_parts(self):
        parts = {"input_norm": self.input_norm, "mixer": self.mixer}
        if self.feed_forward is not None:
            parts.update({"post_mixer_norm": self.post_mixer_norm, "feed_forward": self.feed_forward})
        if self.token_input is not None:
            parts["token_input"] = self.token_input
        return parts

    @classmethod
    def sub_specs(cls, spec: BlockSpec):
        subs = {"input_norm": (NORMS, spec.input_norm), "mixer": (MIXERS, spec.mixer)}
        if spec.feed_forward is not None:
            subs.update({"post_mixer_norm": (NORMS, spec.post_mixer_norm), "feed_forward": (FEED_FORWARDS, spec.feed_forward)})
        if spec.token_input is not None:
            subs["token_input"] = (TOKEN_INPUTS, spec.token_input)
        return subs

    def __call__(self, h, residual, batch, cache, write_cache: bool = True, stream_input=None):
        if residual is None:
            if h.dtype != torch.float32:
                raise ValueError("pre_norm_wide: the embedding must hand over a float32 stream")
            if stream_input is not None:
                raise ValueError("pre_norm_wide: the first run cannot add to a stream that does not exist yet")
            residual = h
            x = self.input_norm(h)
        elif stream_input is not None:
            x, residual = self.input_norm.add_norm(h, residual, extra=stream_input)
        else:
            x, residual = self.input_norm.add_norm(h, residual)
        a = self.mixer(x, batch, cache, write_cache)
        if self.feed_forward is not None:
            y, residual = self.post_mixer_norm.add_norm(a, residual)
            a = self.feed_forward(y, batch)
        if self.token_input is not None:
            # the stream's own value (the last branch output added, not normed) is what the token input reads
            x, residual = self.input_norm.add_only(a, residual)
            a = self.token_input(x, batch.ids)
        return a, residual


class GatedStream:
    """The 32-bit residual between two sublayers of a gated arrangement, and the gate (arguments, bias) that the branch output
    travelling beside it is still to be multiplied by when it is added."""
    __slots__ = ("stream", "gate")

    def __init__(self, stream, gate):
        self.stream, self.gate = stream, gate


class PreNormGatedBlock(Block):
    """x <- x + mixer(n1) sigmoid(W1 n1 + b1); x <- x + ff(n2) sigmoid(W2 n2 + b2), n = norm(x), over a residual kept and summed in
    32-bit: a sublayer's gate is made from the sublayer's own normed input (``connection`` of kind ``sigmoid_gate``) and applied by
    the kernel that adds the sublayer's output to the residual, the next norm's. The block hands on its last branch output and the
    residual with the gate still to be applied; ``close`` does the last gated sum and the final norm of the wanted rows."""

    def __init__(self, spec: BlockSpec, runtime: Runtime):
        if spec.connection is None:
            raise ValueError("pre_norm_gated: the block needs a connection that makes the gates")
        self.spec = spec
        self.rt = runtime
        self.input_norm = NORMS.build(spec.input_norm, runtime)
        self.mixer = MIXERS.build(spec.mixer, runtime)
        self.mixer_connection = CONNECTIONS.build(spec.connection, runtime)
        self.feed_forward = self.post_mixer_norm = self.feed_forward_connection = None
        if spec.feed_forward is not None:
            if spec.post_mixer_norm is None:
                raise ValueError("pre_norm_gated: a feed-forward needs the norm before it")
            self.post_mixer_norm = NORMS.build(spec.post_mixer_norm, runtime)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, runtime)
            self.feed_forward_connection = CONNECTIONS.build(spec.connection, runtime)

    def sub_parts(self):
        parts = {"input_norm": self.input_norm, "mixer": self.mixer, "mixer_connection": self.mixer_connection}
        if self.feed_forward is not None:
            parts.update({"post_mixer_norm": self.post_mixer_norm, "feed_forward": self.feed_forward,
                          "feed_forward_connection": self.feed_forward_connection})
        return parts

    @classmethod
    def sub_specs(cls, spec: BlockSpec):
        subs = {"input_norm": (NORMS, spec.input_norm), "mixer": (MIXERS, spec.mixer), "mixer_connection": (CONNECTIONS, spec.connection)}
        if spec.feed_forward is not None:
            subs.update({"post_mixer_norm": (NORMS, spec.post_mixer_norm), "feed_forward": (FEED_FORWARDS, spec.feed_forward),
                         "feed_forward_connection": (CONNECTIONS, spec.connection)})
        return subs

    def __call__(self, h, residual, batch, cache, write_cache: bool = True):
        if residual is None:
            if h.dtype != torch.float32:
                raise ValueError("pre_norm_gated: the embedding must hand over a float32 stream")
            stream = h
            x = self.input_norm(h)
        else:
            stream = residual.stream
            x, _ = self.input_norm.add_norm(h, stream, gate=residual.gate)
        gate = (self.mixer_connection.arguments(x), self.mixer_connection.bias)
        a = self.mixer(x, batch, cache, write_cache)
        if self.feed_forward is not None:
            y, _ = self.post_mixer_norm.add_norm(a, stream, gate=gate)
            gate = (self.feed_forward_connection.arguments(y), self.feed_forward_connection.bias)
            a = self.feed_forward(y, batch)
        return a, GatedStream(stream, gate)

    def close(self, h, residual, norm, rows):
        """The model's end: the last gated sum of the wanted rows and ``norm`` of it."""
        return norm.add_norm(h, residual.stream, rows=rows, gate=residual.gate)[0]


class StreamState:
    """The residual streams between two sublayers: the 32-bit tensor [tokens, streams, width] and the connection whose
    write-back of the branch output that travels beside it is still to be applied."""
    __slots__ = ("streams", "pending")

    def __init__(self, streams, pending):
        self.streams, self.pending = streams, pending


class PreNormStreamsBlock(Block):
    """h += mixer(norm1(h)); h += ff(norm2(h)) over several 32-bit residual streams: every sum is a connection's read, mix
    and write (``parts/connections.py``). The block hands on its last branch output and the streams it is still to be
    written to; the next block's first kernel applies that write and makes its own read in one pass. ``close`` does the
    same for the model's end: the write, the sum of the streams and the final norm of the wanted rows."""

    def __init__(self, spec: BlockSpec, runtime: Runtime):
        if spec.connection is None:
            raise ValueError("pre_norm_streams: the block needs a connection")
        self.spec = spec
        self.rt = runtime
        self.input_norm = NORMS.build(spec.input_norm, runtime)
        self.mixer = MIXERS.build(spec.mixer, runtime)
        self.mixer_connection = CONNECTIONS.build(spec.connection, runtime)
        self.feed_forward = self.post_mixer_norm = self.feed_forward_connection = None
        if spec.feed_forward is not None:
            if spec.post_mixer_norm is None:
                raise ValueError("pre_norm_streams: a feed-forward needs the norm before it")
            self.post_mixer_norm = NORMS.build(spec.post_mixer_norm, runtime)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, runtime)
            self.feed_forward_connection = CONNECTIONS.build(spec.connection, runtime)

    def sub_parts(self):
        parts = {"input_norm": self.input_norm, "mixer": self.mixer, "mixer_connection": self.mixer_connection}
        if self.feed_forward is not None:
            parts.update({"post_mixer_norm": self.post_mixer_norm, "feed_forward": self.feed_forward,
                          "feed_forward_connection": self.feed_forward_connection})
        return parts

    @classmethod
    def sub_specs(cls, spec: BlockSpec):
        subs = {"input_norm": (NORMS, spec.input_norm), "mixer": (MIXERS, spec.mixer), "mixer_connection": (CONNECTIONS, spec.connection)}
        if spec.feed_forward is not None:
            subs.update({"post_mixer_norm": (NORMS, spec.post_mixer_norm), "feed_forward": (FEED_FORWARDS, spec.feed_forward),
                         "feed_forward_connection": (CONNECTIONS, spec.connection)})
        return subs

    def _read(self, h, state, connection, norm, rows=None):
        """Applies the pending write of ``h`` (if any), then ``connection``'s read (None: the sum of the streams) and ``norm``."""
        k, S = self.rt.kernels, self.spec.connection.streams
        if state is None:       # the embedding: every stream starts as a copy of it
            streams = torch.empty((h.shape[0], S, h.shape[1]), dtype=torch.float32, device=h.device)
            x = k.stream_step(streams, norm.weight, norm.spec.eps, self.rt.dtype, read=connection.read, init_from=h)
            return x, streams
        p = state.pending
        x = k.stream_step(state.streams, norm.weight, norm.spec.eps, self.rt.dtype, read=None if connection is None else connection.read,
                          y=h, mix=p.mix, write=p.write, rows=rows)
        return x, state.streams

    def __call__(self, h, residual, batch, cache, write_cache: bool = True):
        x, streams = self._read(h, residual, self.mixer_connection, self.input_norm)
        a = self.mixer(x, batch, cache, write_cache)
        state = StreamState(streams, self.mixer_connection)
        if self.feed_forward is None:
            return a, state
        y, _ = self._read(a, state, self.feed_forward_connection, self.post_mixer_norm)
        return self.feed_forward(y, batch), StreamState(streams, self.feed_forward_connection)

    def close(self, h, residual, norm, rows):
        """The model's end: the last write, the sum of the streams of the wanted rows and ``norm`` of it."""
        return self._read(h, residual, None, norm, rows=rows)[0]


register_block("pre_norm_streams", PreNormStreamsBlock)
register_block("pre_norm_gated", PreNormGatedBlock)
register_block("pre_norm", PreNormBlock)
register_block("pre_norm_wide", PreNormWideBlock)
