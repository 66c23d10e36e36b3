"""Interfaces of the parts a layer is put together from.

A part gets its sizes and constants as constructor parameters, says which
weights it needs (``weight_shapes``), receives them (``bind``) and then runs on
the tokens of a step (``forward``).  Kernels are reached only through
``ctx.ops``; a part never asks which model it is in.

Roles:
  norm              forward(ctx, x[T,E] float32) -> h[T,E] in the compute dtype
  position          describes how positions enter a mixer (``rotary()``)
  mixer             forward(ctx, h, entry, accumulate_into) ; adds its result to the
                    float32 residual stream, or returns it as float32 rows when
                    ``accumulate_into`` is None; may need cache (``cache_need``) and
                    fixed-size per-sequence state (``state_need``: one tensor, or
                    several by name)
  feed_forward      forward(ctx, h, accumulate_into), likewise
  connection        how a sublayer's result enters the residual state (``weights()``)
  input_filter      forward(ctx, h, state) -> what the sublayer reads instead of h (same shape and dtype); may keep
                    fixed-size state per sequence (``state_need``), which the block hands to it
  result_gate       logits(ctx, h) from the sublayer's unfiltered input, and apply(ctx, x, y, logits): how the
                    sublayer's result y enters the residual stream x
  token_input       forward(ctx, x, h): adds to the residual stream x something made from the rows' token ids
                    (``ctx.meta.token_ids``) and from h, the same rows in the compute dtype
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer stores per position.  Layers with equal needs share a cache group
    (one pool of pages per stored tensor); ``window`` None means every earlier position is kept.

    By default two tensors are stored per position, keys and values, each of ``n_kv_heads``
    heads of ``head_dim`` values.  ``streams`` names other contents: a tuple of (heads, width)
    pairs, one per stored tensor, for instance ``((1, 96),)`` for a mixer that keeps one vector
    per position, or keys and values of different widths."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    streams: Optional[Tuple[Tuple[int, int], ...]] = None

    def stream_shapes(self) -> Tuple[Tuple[int, int], ...]:
        if self.streams is not None:
            return tuple((int(h), int(w)) for h, w in self.streams)
        return ((self.n_kv_heads, self.head_dim), (self.n_kv_heads, self.head_dim))


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state per sequence: a tensor of ``shape`` and ``dtype`` per slot,
    zeroed when the slot is handed out."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    role = ""

    def weight_shapes(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        """key -> (shape, "matrix" | "norm")"""
        return {}

    def bind(self, weights: Dict[str, torch.Tensor], ops) -> None:
        """Take the weights (already on the device, as stored in the files)."""


class Norm(Part):
    role = "norm"

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    role = "position"

    def rotary(self):
        """None, or (inv_freq float32 [D/2] device tensor, interleaved: bool, rot_dim)."""
        return None


class Mixer(Part):
    role = "mixer"

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self):
        """None, one ``StateNeed``, or a dict name -> ``StateNeed`` for a mixer that keeps several
        tensors per sequence (``ctx.state_view(entry)`` then gives a dict of the same names)."""
        return None

    def forward(self, ctx, h: torch.Tensor, entry: int, accumulate_into: Optional[torch.Tensor] = None):
        """h[T, E]: the normed input rows of this step's tokens.  ``entry`` is the
        index of this run in the schedule (``ctx.cache_view(entry)``,
        ``ctx.state_view(entry)``); ``ctx.pass_state`` is a dict that lives for one pass over the layers, for what
        a layer leaves for later layers of the same pass.  The result is added to ``accumulate_into``; a mixer that
        can also stand beside another one returns it as float32 [T, E] when that is None."""
        raise NotImplementedError


class FeedForward(Part):
    role = "feed_forward"

    def forward(self, ctx, h: torch.Tensor, accumulate_into: Optional[torch.Tensor] = None):
        raise NotImplementedError


class InputFilter(Part):
    """Replaces what a sublayer reads, h [T, E] in the compute dtype, by a function of h and of the sequence's
    earlier rows.  ``state_need`` as for a mixer; the block keeps the state per run of the layer and hands the
    run's tensor ([n_slots, *shape]) to ``forward``."""
    role = "input_filter"

    def state_need(self):
        return None

    def forward(self, ctx, h: torch.Tensor, state):
        raise NotImplementedError


class ResultGate(Part):
    """Decides how much of a sublayer's result enters the residual stream, from the sublayer's input rows."""
    role = "result_gate"

    def logits(self, ctx, h: torch.Tensor):
        raise NotImplementedError

    def apply(self, ctx, x: torch.Tensor, y: torch.Tensor, logits) -> None:
        """x (float32 [T, E], the residual stream) takes y (float32 [T, E]) in."""
        raise NotImplementedError


class TokenInput(Part):
    """Adds to the residual stream a function of each row's token id and of the row itself."""
    role = "token_input"

    def forward(self, ctx, x: torch.Tensor, h: torch.Tensor, want_rounded: bool = False):
        """x: float32 [T, E], changed in place; h: the same rows in the compute dtype.  With ``want_rounded`` the new
        rows are returned in the compute dtype as well."""
        raise NotImplementedError


class Connection(Part):
    """How a sublayer reads the residual state and how its result enters it.  ``streams`` rows per
    token; ``weights()`` gives float32 device tensors ``w_in`` [s], ``w_out`` [s], ``mix`` [s, s]
    (indexed [from, to])."""
    role = "connection"
    streams = 1

    def weights(self):
        raise NotImplementedError
