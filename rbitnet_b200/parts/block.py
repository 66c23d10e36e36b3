"""Arrangement of a layer's parts.  "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x))
(crates/bitnet-core/src/llama/model.rs:237-306).  The residual stream x is float32.

A norm between two products.  For a few tokens a norm is a kernel that does a microsecond of work
and costs three in a chain of dependent launches.  Where the operations offer it
(``ops.norm_request``), the norm's own part says what it needs (``deferred``) and the parts on both
sides say that they pass it on (``folds_norms``), the block asks the part before a norm to have its
last product leave the rows times the norm's weights, with their sums of squares, and gives those
to the part after the norm, whose first product multiplies its sums by each row's factor.  Parts
that know nothing of this get the normed rows as before.

An arrangement is a class built from a ``BlockSpec`` with ``parts()`` (name -> part, every part
whose weights are to be bound; the names are those of ``BlockSpec.parts``) and
``run(ctx, x, entry)``.  ``build_parts`` makes every part a spec names, whatever it is called."""
from __future__ import annotations

from .registry import register_part, build_part


def build_parts(spec) -> dict:
    """name -> part for every entry of ``spec.parts``."""
    return {name: build_part(spec.role_of(name), ps) for name, ps in spec.parts.items()}


class PreNormBlock:
    def __init__(self, spec):
        self.spec = spec
        self._parts = build_parts(spec)
        missing = [n for n in ("mixer", "mixer_norm") if n not in self._parts]
        if missing:
            raise ValueError(f"a pre_norm block needs the parts {missing}")
        if ("feed_forward" in self._parts) != ("ffn_norm" in self._parts):
            raise ValueError("a pre_norm block has a feed-forward with its norm, or neither")
        self.mixer, self.feed_forward = self._parts["mixer"], self._parts.get("feed_forward")
        self.mixer_norm, self.ffn_norm = self._parts["mixer_norm"], self._parts.get("ffn_norm")

    def parts(self):
        return self._parts

    #: ``run`` takes the rows of its first norm from the block before and leaves them for the block after
    chains_norms = True

    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _request(ctx, norm, before):
        """A request to the part before ``norm``, if both know how."""
        if norm is None or not getattr(before, "folds_norms", False):
            return None
        deferred = getattr(norm, "deferred", None)
        return deferred(ctx.ops) if deferred is not None else None

    @staticmethod
    def _rows_for(ctx, part, norm, x, pending):
        """The input of ``part``: what the part before left if ``part`` takes it, else the normed rows."""
        if pending is None:
            return norm.forward(ctx, x)
        return pending if getattr(part, "folds_norms", False) else ctx.ops.normed(pending)

    def run(self, ctx, x, entry: int, pending=None, next_norm=None):
        """``pending``: what the block before left for this block's first norm (or None).  Returns what
        it leaves for ``next_norm``, the first norm of the block after (or None)."""
        h = self._rows_for(ctx, self.mixer, self.mixer_norm, x, pending)
        if self.feed_forward is None:
            # a layer of a mixer alone: what the next block's first norm needs is asked of the mixer
            request = self._request(ctx, next_norm, self.mixer)
            if request is None:
                self.mixer.forward(ctx, h, entry, accumulate_into=x)
                return None
            self.mixer.forward(ctx, h, entry, accumulate_into=x, then_norm=request)
            return request.result
        request = self._request(ctx, self.ffn_norm, self.mixer)
        if request is None:
            self.mixer.forward(ctx, h, entry, accumulate_into=x)
        else:
            self.mixer.forward(ctx, h, entry, accumulate_into=x, then_norm=request)
        h = self._rows_for(ctx, self.feed_forward, self.ffn_norm, x, request.result if request is not None else None)
        request = self._request(ctx, next_norm, self.feed_forward)
        if request is None:
            self.feed_forward.forward(ctx, h, accumulate_into=x)
            return None
        self.feed_forward.forward(ctx, h, accumulate_into=x, then_norm=request)
        return request.result


class StreamBlock:
    """Sublayers over a residual state of s rows per token (``x`` is [T, s * E] float32): a mixer and,
    if the layer has one, a feed-forward, each with a norm and a connection (see ``parts/connection.py``):

        h = norm(read(X));  y = sublayer(h);  X <- write(X, y)

    Parts: "mixer", "mixer_norm", "mixer_connection", and none or all of "feed_forward", "ffn_norm",
    "ffn_connection".  What lies between the products of two sublayers (the mean of the normed results of
    mixers that run side by side, the write, the next read and its norm) is one kernel where the
    operations fuse it (``ops.fuse_streams``), else a kernel each; the read of the next block's first
    sublayer is handed on like a pending norm (``chains_reads``)."""

    chains_reads = True

    def __init__(self, spec):
        self.spec = spec
        self._parts = build_parts(spec)
        for n in ("mixer", "mixer_norm", "mixer_connection"):
            if n not in self._parts:
                raise ValueError(f"a multi_stream block needs the part {n!r}")
        ffn = [n for n in ("feed_forward", "ffn_norm", "ffn_connection") if n in self._parts]
        if len(ffn) not in (0, 3):
            raise ValueError("a multi_stream block has a feed-forward with its norm and connection, or none of them")
        self.sublayers = [(self._parts["mixer"], self._parts["mixer_norm"], self._parts["mixer_connection"], True)]
        if ffn:
            self.sublayers.append((self._parts["feed_forward"], self._parts["ffn_norm"], self._parts["ffn_connection"], False))
        self.streams = self._parts["mixer_connection"].streams
        if any(c.streams != self.streams for _, _, c, _ in self.sublayers):
            raise ValueError("a multi_stream block's connections must have the same number of streams")

    def parts(self):
        return self._parts

    @staticmethod
    def _read_of(sub):
        _, norm, conn, _ = sub
        return conn.weights()[0], norm.weight, norm.eps

    def first_read(self):
        return self._read_of(self.sublayers[0])

    def run(self, ctx, x, entry: int, pending=None, next_read=None):
        """``pending``: the normed read of this block's first sublayer, if the block before made it.
        Returns the normed read for ``next_read`` (that of the block after), or None."""
        ops, s = ctx.ops, self.streams
        fuse = bool(getattr(ops, "fuse_streams", False))
        h = pending if pending is not None else ops.stream_step(x, s, read=self.first_read())
        for i, (part, norm, conn, is_mixer) in enumerate(self.sublayers):
            following = self._read_of(self.sublayers[i + 1]) if i + 1 < len(self.sublayers) else next_read
            _, w_out, mix = conn.weights()
            side_by_side = hasattr(part, "results")
            if is_mixer:
                ys, ws = part.results(ctx, h, entry) if side_by_side and fuse else ([part.forward(ctx, h, entry, accumulate_into=None)], None)
            else:
                ys, ws = [part.forward(ctx, h, accumulate_into=None)], None
            eps = norm.eps
            if fuse:
                h = ops.stream_step(x, s, results=ys, result_norms=ws, norm_eps=eps, write=(mix, w_out), read=following)
            else:
                ops.stream_step(x, s, results=ys, write=(mix, w_out))
                h = ops.stream_step(x, s, read=following) if following is not None else None
        return h


class GatedPreNormBlock:
    """Pre-norm sublayers whose inputs may be filtered and whose results may be gated:

        h = norm(x);   x <- x + gate(h) * sublayer(filter(h))

    for the mixer and, if the layer has one, the feed-forward.  Parts: "mixer", "mixer_norm" and optionally
    "mixer_filter" (role "input_filter"), "mixer_gate" (role "result_gate"); "feed_forward" with "ffn_norm" and
    optionally "ffn_filter", "ffn_gate".  Without a gate the sublayer adds its result itself; without a filter it
    reads the normed rows.  A filter's per-sequence state belongs to the run of the layer
    (``ctx.part_state(entry, name)``)."""

    def __init__(self, spec):
        self.spec = spec
        self._parts = build_parts(spec)
        missing = [n for n in ("mixer", "mixer_norm") if n not in self._parts]
        if missing:
            raise ValueError(f"a pre_norm_gated block needs the parts {missing}")
        if ("feed_forward" in self._parts) != ("ffn_norm" in self._parts):
            raise ValueError("a pre_norm_gated block has a feed-forward with its norm, or neither")
        p = self._parts
        self.sublayers = [(p["mixer"], p["mixer_norm"], "mixer_filter", p.get("mixer_filter"), p.get("mixer_gate"), True)]
        if "feed_forward" in p:
            self.sublayers.append((p["feed_forward"], p["ffn_norm"], "ffn_filter", p.get("ffn_filter"), p.get("ffn_gate"), False))
        elif "ffn_filter" in p or "ffn_gate" in p:
            raise ValueError("a pre_norm_gated block without a feed-forward has no filter or gate for one")

    def parts(self):
        return self._parts

    def run(self, ctx, x, entry: int):
        # Where the operations have it, a step of one token per sequence takes what lies between two sublayers (the
        # gated result of the one, the norm and the filter of the next) as one operation; a gated result therefore
        # waits until the next norm, or the block's end, asks for the residual stream.
        rows_between = getattr(ctx.ops, "norm_filter_rows", None)
        waiting = None                                     # (gate, y, logits) not yet added to x

        def settle():
            nonlocal waiting
            if waiting is not None:
                waiting[0].apply(ctx, x, waiting[1], waiting[2])
                waiting = None

        for part, norm, filter_name, filt, gate, is_mixer in self.sublayers:
            h = hf = None
            groups = getattr(norm, "groups", None)
            if rows_between is not None and filt is not None and groups is not None and hasattr(filt, "w"):
                add = None
                if waiting is not None:
                    addend = getattr(waiting[0], "addend", None)
                    if addend is None:
                        settle()
                    else:
                        add = addend(waiting[1], waiting[2])
                got = rows_between(x, norm.weight, groups, norm.eps, filt.w, ctx.part_state(entry, filter_name), ctx.meta,
                                   add=add)
                if got is not None:
                    h, hf = got
                    waiting = None
            if h is None:
                settle()
                h = norm.forward(ctx, x)
                hf = filt.forward(ctx, h, ctx.part_state(entry, filter_name)) if filt is not None else h
            logits = gate.logits(ctx, h) if gate is not None else None
            into = x if gate is None else None
            y = part.forward(ctx, hf, entry, accumulate_into=into) if is_mixer else part.forward(ctx, hf, accumulate_into=into)
            if gate is not None:
                waiting = (gate, y, logits)
        settle()


class PostNormBlock:
    """Sublayers that read the residual stream itself and whose RESULTS are normed:

        x <- x + norm1(mixer(x));   x <- x + norm2(feed_forward(x));   x <- x + token_input(x, token)

    Parts: "mixer" with "mixer_norm"; optionally "feed_forward" with "ffn_norm"; optionally "token_input" (role
    "token_input").  The norms are asked through ``add_to`` (an RMS norm with its weight, layer scale included, as one
    vector).  What a sublayer reads is x rounded to the compute dtype; the kernel that adds a normed result also
    leaves those rows for the next sublayer, so a layer has no kernel that only rounds, but for the very first
    sublayer of a step: the last addition of a block hands its rows to the block after it (``chains_rows``)."""

    chains_rows = True

    def __init__(self, spec):
        self.spec = spec
        self._parts = build_parts(spec)
        missing = [n for n in ("mixer", "mixer_norm") if n not in self._parts]
        if missing:
            raise ValueError(f"a post_norm block needs the parts {missing}")
        if ("feed_forward" in self._parts) != ("ffn_norm" in self._parts):
            raise ValueError("a post_norm block has a feed-forward with its norm, or neither")
        p = self._parts
        self.mixer, self.mixer_norm = p["mixer"], p["mixer_norm"]
        self.feed_forward, self.ffn_norm = p.get("feed_forward"), p.get("ffn_norm")
        self.token_input = p.get("token_input")
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not hasattr(norm, "add_to"):
                raise ValueError("a post_norm block needs norms that can be added to the residual stream (add_to)")

    def parts(self):
        return self._parts

    def run(self, ctx, x, entry: int, rows=None, want_rows: bool = True):
        """``rows``: x in the compute dtype, if the block before left it.  Returns the same for the block after
        (None if ``want_rows`` is false: nobody reads them)."""
        h = rows if rows is not None else ctx.ops.round_rows(x)
        last = "token_input" if self.token_input is not None else ("ffn" if self.feed_forward is not None else "mixer")
        y = self.mixer.forward(ctx, h, entry, accumulate_into=None)
        h = self.mixer_norm.add_to(ctx, x, y, want_rounded=want_rows or last != "mixer")
        if self.feed_forward is not None:
            y = self.feed_forward.forward(ctx, h, accumulate_into=None)
            h = self.ffn_norm.add_to(ctx, x, y, want_rounded=want_rows or last != "ffn")
        if self.token_input is not None:
            h = self.token_input.forward(ctx, x, h, want_rounded=want_rows)
        return h if want_rows else None


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "post_norm", PostNormBlock)
register_part("block", "pre_norm_gated", GatedPreNormBlock)
register_part("block", "multi_stream", StreamBlock)
