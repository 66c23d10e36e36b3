"""The operations a step is made of, on device tensors, each one a launch of this
package's own CUDA kernels.

``CudaOps(dtype)`` is the only implementation on the product path.  With
``torch.float32`` every product is a float32 FFMA sum and every activation,
cache entry and weight is float32 (no tensor-core or reduced-precision mode).
With ``torch.bfloat16`` weights, activations between kernels and the cache are
bfloat16, while the residual stream, norms, rotation angles, softmax and all
accumulation stay float32.
"""
from __future__ import annotations

from ctypes import c_void_p
from dataclasses import dataclass
from typing import List, Optional

import torch

from .lib import load, KernelError

F32, BF16 = 0, 1
_CODE = {torch.float32: F32, torch.bfloat16: BF16}


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


@dataclass
class LinearWeight:
    """A weight matrix [out, in] made ready for ``linear``."""
    w: torch.Tensor
    n_out: int
    n_in: int


@dataclass
class GateUpWeight:
    """Gate and up matrices made ready for ``gated_linear``.

    ``block == 0``: rows [gate | up].  ``block == 16``: for every 16 output features, their 16 gate
    rows followed by their 16 up rows (the last group padded with zero rows), which is how the
    tensor-core product pairs gate and up inside one warp of its epilogue."""
    w: torch.Tensor
    inner: int
    n_in: int
    block: int = 0


@dataclass
class PerHeadWeight:
    """One matrix [n_out, n_in] per head, made ready for ``per_head_linear``: ``w`` is [heads, n_out, n_in]."""
    w: torch.Tensor
    heads: int
    n_out: int
    n_in: int


@dataclass
class ExpertGateUp:
    """The gate and up matrices of gated experts, one expert below the other (``rows`` rows each).
    ``block == 0``: an expert's rows are [gate | up].  ``block == 16``: the interleaved layout of ``GateUpWeight``."""
    w: torch.Tensor
    inner: int
    n_in: int
    rows: int
    block: int = 0

    @property
    def n_out(self):
        return self.w.shape[0]


@dataclass
class NormRequest:
    """Asks the product that adds to the residual stream to leave what the norm after it needs
    (``CudaOps.linear(..., then_norm=request)``).  ``result`` is the ``NormedRows`` if it did."""
    weight: torch.Tensor          # float32 [width]
    eps: float
    result: Optional["NormedRows"] = None


@dataclass
class NormedRows:
    """Rows of the residual stream with an RMS norm pending: a product that takes them multiplies its
    finished sums by each row's 1/sqrt(mean of squares + eps) (``CudaOps.linear``, ``gated_linear`` and
    ``project_rotate_append`` take them in place of the normed rows; ``CudaOps.normed`` gives the normed
    rows themselves).  The norm is the same float32 arithmetic either way; what is rounded to bfloat16
    is row * weight instead of row * factor * weight."""
    x: torch.Tensor               # the rows themselves, float32 [T, width]
    weight: torch.Tensor          # float32 [width]
    eps: float
    scaled: torch.Tensor          # bfloat16 [T, width]: x * weight
    squares: torch.Tensor         # float32 [parts, T]: sums of squares of x over parts of the width

    @property
    def shape(self):
        return self.x.shape


#: per device: the workspace of the tensor-core products (arrival counters, then partial sums of
#: tiles whose inner dimension is shared between teams of CTAs).  One per process and device, never
#: freed: the library keeps its address.
_GEMM_WORKSPACES = {}
_GEMM_WORKSPACE_SET = set()
_GEMM_COUNTER_BYTES = 4 << 16


def _give_gemm_workspace(lib, device: torch.device) -> None:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if (lib.path, index) in _GEMM_WORKSPACE_SET:
        return
    with torch.cuda.device(index):
        ws = _GEMM_WORKSPACES.get(index)
        if ws is None:
            n = int(lib.raw("rb_gemm_tc_workspace_bytes")())
            ws = _GEMM_WORKSPACES[index] = torch.zeros(n, dtype=torch.uint8, device=device)
            torch.cuda.synchronize(index)
        lib.call("rb_gemm_tc_set_workspace", c_void_p(ws.data_ptr()), ws.numel(), launches=0)
    _GEMM_WORKSPACE_SET.add((lib.path, index))


class CudaOps:
    def __init__(self, dtype=torch.bfloat16, device="cuda:0", verbose_build: bool = True):
        if dtype not in _CODE:
            raise ValueError(f"compute dtype must be float32 or bfloat16, found {dtype}")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: rbitnet_b200 runs its kernels on a B200 and has no other path")
        self.dtype = dtype
        self.code = _CODE[dtype]
        self.device = torch.device(device)
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"device {self.device} has compute capability {major}.{minor}; "
                              "the kernels are built for sm_100a only")
        self.lib = load(verbose=verbose_build)
        #: prefill attention of head sizes 64 and 128 runs on tcgen05 (else on the mma.sync kernel)
        self.prefill_on_tcgen05 = True
        #: decode attention of head sizes 64 and 128 gets its keys and values by TMA (else by cp.async)
        self.decode_on_tma = True
        self._flag_ptrs = None
        #: a decode step's norms between two products are folded into them (see ``NormedRows``)
        self.fold_norms = True
        self.fold_norms_up_to = 16
        #: what lies between two sublayers of a block over several residual streams is one kernel
        self.fuse_streams = True
        #: a limited gated activation is applied in the tensor-core product's epilogue (else by a kernel of its own)
        self.fuse_gated_act = True
        #: a decode step's gated linear recurrence (convolution, gates, scan) is one kernel for up to 16 rows
        self.fuse_recurrent_step = True
        #: the delta rule takes runs of several tokens in chunks of 32 (else token by token, as a decode step does)
        self.delta_in_chunks = True
        #: a decode step's gated addition, norm in groups and filter between two sublayers are one kernel
        self.fuse_norm_filter = True
        #: rows from which a scored router's sums are a tensor-core product (where that product gives the same sums)
        self.router_tc_from = 1
        #: so does gated linear attention
        self.gla_in_chunks = True
        #: a decode step's delta rule (convolution to gate) is one kernel while rows x heads fit the SMs
        self.fuse_delta_step = True
        #: tensor-core products of more than 256 tokens may share a weight tile's inner dimension
        #: between teams of CTAs (needs the workspace; tiles are taken in turn without it)
        _give_gemm_workspace(self.lib, self.device)

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _check(self, t: torch.Tensor, dtype, what: str):
        if t.dtype != dtype or not t.is_cuda or not t.is_contiguous():
            raise KernelError(f"{what}: expected a contiguous {dtype} CUDA tensor, found {t.dtype} "
                              f"on {t.device}, contiguous={t.is_contiguous()}")

    def check_errors(self) -> None:
        """Raises if a kernel recorded that one of its bounded waits ran out."""
        import ctypes
        v = ctypes.c_int(0)
        self.lib.call("rb_read_error_flag", ctypes.byref(v), 1, launches=0)
        if v.value:
            ws = _GEMM_WORKSPACES.get(self.device.index if self.device.index is not None else torch.cuda.current_device())
            if ws is not None:
                ws[:_GEMM_COUNTER_BYTES].zero_()      # a product that gave up may have left counts behind
            raise KernelError(f"a kernel gave up waiting (code {v.value}: 1 = loader, 2 = tensor-core issuer, "
                              "3 = epilogue, 4 = the parts of a shared weight tile); its results are not valid")
        if self.lib.raw("rb_is_checked_build")():
            from .lib import CHECKED_FILES
            w = (ctypes.c_int * 4)()
            for tu in CHECKED_FILES:
                self.lib.call(f"rb_check_word_{tu}", w, 1, launches=0)
                if w[0]:
                    raise KernelError(f"checked build ({tu}): a kernel asked for slot {w[1]}, position {w[2]}, kv head "
                                      f"{w[3]}, which lies outside the cache (code {w[0]}); the access was not made")

    def to_compute(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    # ------------------------------------------------------------------ weights
    def prepare_embedding(self, table: torch.Tensor) -> torch.Tensor:
        return self.to_compute(table)

    def prepare_linear(self, weights: List[torch.Tensor]) -> LinearWeight:
        """One matrix from the given ones stacked along the output axis."""
        if len(weights) == 1:
            w = self.to_compute(weights[0])
        else:
            w = torch.cat([self.to_compute(x) for x in weights], dim=0).contiguous()
        return LinearWeight(w, w.shape[0], w.shape[1])

    def rows_of(self, weight: LinearWeight, first: int, count: int) -> LinearWeight:
        """Output rows first .. first+count-1 of a prepared matrix, sharing its memory."""
        return LinearWeight(weight.w[first:first + count], count, weight.n_in)

    def prepare_gate_up(self, gate: torch.Tensor, up: torch.Tensor) -> GateUpWeight:
        gate, up = self.to_compute(gate), self.to_compute(up)
        F, K = gate.shape
        if self.dtype == torch.bfloat16 and K % 8 == 0:
            # the layout of the tensor-core gated product: groups of 16 gate rows and their 16 up rows
            groups = -(-F // 16)
            w = torch.zeros((groups, 2, 16, K), dtype=gate.dtype, device=gate.device)
            for half, m in ((0, gate), (1, up)):
                whole = F // 16
                w[:whole, half] = m[:whole * 16].view(whole, 16, K)
                if F % 16:
                    w[whole, half, :F % 16] = m[whole * 16:]
            return GateUpWeight(w.view(groups * 32, K), F, K, 16)
        return GateUpWeight(torch.cat([gate, up], dim=0).contiguous(), F, K, 0)

    # ------------------------------------------------------------------ ops
    def embed(self, ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """float32 rows table[ids] * scale."""
        T, (V, E) = ids.shape[0], table.shape
        out = torch.empty((T, E), dtype=torch.float32, device=self.device)
        self.lib.call("rb_embed", _ptr(out), _ptr(table), _CODE[table.dtype], _ptr(ids), T, E, V, float(scale),
                      self._stream())
        return out

    def rmsnorm(self, x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype=None) -> torch.Tensor:
        self._check(x, torch.float32, "rmsnorm input")
        T, E = x.shape
        out = torch.empty((T, E), dtype=out_dtype or self.dtype, device=self.device)
        self.lib.call("rb_rmsnorm", _ptr(out), _CODE[out.dtype], _ptr(x), _ptr(w), T, E, float(eps), self._stream())
        return out

    def layernorm(self, x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float, out_dtype=None) -> torch.Tensor:
        """(x - mean) / sqrt(variance + eps) * w + b per row, in float32; the result in the compute dtype."""
        self._check(x, torch.float32, "layernorm input")
        T, E = x.shape
        out = torch.empty((T, E), dtype=out_dtype or self.dtype, device=self.device)
        self.lib.call("rb_layernorm", _ptr(out), _CODE[out.dtype], _ptr(x), _ptr(w), _ptr(b), T, E, float(eps), self._stream())
        return out

    def add_rows(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """x += y, float32 rows of equal shape."""
        self._check(x, torch.float32, "add_rows target")
        self._check(y, torch.float32, "add_rows source")
        if x.shape != y.shape:
            raise KernelError(f"add_rows: shapes {tuple(x.shape)} and {tuple(y.shape)}")
        self.lib.call("rb_add_rows", _ptr(x), _ptr(y), x.numel(), self._stream())
        return x

    def linear(self, x, weight: LinearWeight, out_dtype=None, accumulate_into: Optional[torch.Tensor] = None,
               scale: float = 1.0, then_norm: Optional[NormRequest] = None, act: Optional[str] = None) -> torch.Tensor:
        """scale * x[T, in] * W[out, in]^T (the scale multiplies the finished float32 sums).  With
        ``accumulate_into`` (float32 [T, out]) the product is added to it in float32 and it is returned.
        ``x`` may be ``NormedRows``.  ``then_norm``: see ``NormRequest`` (granted for a few tokens, where
        the product's parts along the inner dimension meet on chip).  ``act`` "relu2": max(v, 0)^2 of the
        finished float32 sums is stored (in the tensor-core product's epilogue, else by a kernel after it)."""
        if act not in (None, "relu2"):
            raise KernelError(f"linear: activation {act!r} is not built (only 'relu2')")
        if act is not None and accumulate_into is not None:
            raise KernelError("linear: an activation goes with a stored product, not an added one")
        pending = x if isinstance(x, NormedRows) else None
        if pending is not None:
            if self._takes_pending(pending, weight.w):
                x = pending.scaled
            else:
                x, pending = self.normed(pending), None
        self._check(x, self.dtype, "linear input")
        T, K = x.shape
        if K != weight.n_in:
            raise KernelError(f"linear: input width {K} does not match the weight's {weight.n_in}")
        N = weight.n_out
        if accumulate_into is not None:
            out, acc = accumulate_into, 1
            self._check(out, torch.float32, "linear accumulate_into")
        else:
            out, acc = torch.empty((T, N), dtype=out_dtype or self.dtype, device=self.device), 0
        if self._tensor_core_ok(x, weight.w):
            # few tokens and few weight tiles: K is cut into parts so that every SM streams a piece
            # of W; the parts of a tile are one thread-block cluster and are summed on chip
            splits = self._k_splits(T, N, K)
            if pending is not None:
                self._pending_norm(pending)
            # (up to 16 tokens: measured at batch 1 and 8 a step gains 2.8 and 1.5 %, at batch 64 it loses 1 %:
            # the norm's kernel also was the time in which the next product's first tiles of W arrived)
            if then_norm is not None and acc and splits >= 2 and T <= self.fold_norms_up_to and out.is_contiguous():
                then_norm.result = self._leave_norm(out, then_norm, T, N)
            if act is not None:
                self.lib.call("rb_gemm_tc_square_relu", launches=0)
            self.lib.call("rb_gemm_tc", _ptr(out), out.stride(0), _CODE[out.dtype], _ptr(x), x.stride(0), T,
                          _ptr(weight.w), weight.w.stride(0), N, N, K, acc, 0, splits,
                          64 if 64 < T <= 256 else 0, float(scale), self._stream())
        else:
            self.lib.call("rb_gemm_simple", _ptr(out), out.stride(0), _CODE[out.dtype], _ptr(x), x.stride(0),
                          _ptr(weight.w), weight.w.stride(0), self.code, T, N, K, acc, float(scale), self._stream())
            if act is not None:
                self.lib.call("rb_square_relu", _ptr(out), _ptr(out), _CODE[out.dtype], out.numel(), self._stream())
        return out

    # ------------------------------------------------------------------ a norm between two products
    def norm_request(self, weight: torch.Tensor, eps: float) -> Optional[NormRequest]:
        """A request for ``linear(..., then_norm=)``, or None where norms are not folded into products
        (the float32 path keeps every norm a kernel of its own)."""
        if self.dtype != torch.bfloat16 or not self.fold_norms:
            return None
        return NormRequest(weight, float(eps))

    def normed(self, rows: NormedRows) -> torch.Tensor:
        """The normed rows themselves, for whoever does not take ``NormedRows``."""
        return self.rmsnorm(rows.x, rows.weight, rows.eps)

    def _takes_pending(self, rows: NormedRows, w: torch.Tensor) -> bool:
        return (self.dtype == torch.bfloat16 and rows.scaled.shape[0] <= 16 and self._tensor_core_ok(rows.scaled, w))

    def _pending_norm(self, rows: NormedRows) -> None:
        """For the next tensor-core product of this thread."""
        self.lib.call("rb_gemm_tc_pending_norm", _ptr(rows.squares), rows.squares.shape[0], float(rows.x.shape[1]),
                      float(rows.eps), launches=0)

    def _leave_norm(self, out: torch.Tensor, request: NormRequest, T: int, N: int) -> NormedRows:
        """For the next tensor-core product of this thread (one that adds into ``out``)."""
        parts = self.lib.raw("rb_gemm_tc_norm_parts")(N)
        scaled = torch.empty((T, N), dtype=torch.bfloat16, device=self.device)
        squares = torch.empty((parts, T), dtype=torch.float32, device=self.device)
        self.lib.call("rb_gemm_tc_leave_norm", _ptr(scaled), scaled.stride(0), _ptr(request.weight), _ptr(squares),
                      launches=0)
        return NormedRows(out, request.weight, request.eps, scaled, squares)

    def _k_splits(self, T: int, N: int, K: int) -> int:
        """Parts to cut the inner dimension into: the library's choice for this device (1 beyond 256
        tokens; else up to 8, so that every SM streams a piece of W)."""
        return self.lib.raw("rb_gemm_tc_splits")(T, N, K)

    def _tensor_core_ok(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        """The tcgen05 product takes bfloat16 operands whose rows TMA can address: inner size and
        row strides multiples of 8 elements, 16-byte aligned bases.  Anything else runs on the
        plain product."""
        return (self.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
                and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and x.stride(1) == 1 and w.stride(1) == 1)

    def gated_linear(self, x: torch.Tensor, weight: GateUpWeight, act=None) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) -> [T, inner] in the compute dtype.  ``act`` = (alpha, limit, shift):
        g' sigmoid(alpha g') (u' + shift) with g' = min(g, limit), u' = clamp(u, -limit, limit) instead."""
        if act is not None and weight.block == 16 and not isinstance(x, NormedRows) and self.fuse_gated_act \
                and self._tensor_core_ok(x, weight.w):
            # the tensor-core gated product with the limited activation in its epilogue
            T, rows = x.shape[0], weight.w.shape[0]
            out = torch.empty((T, weight.inner), dtype=self.dtype, device=self.device)
            self.lib.call("rb_gemm_tc_gated_act", float(act[0]), float(act[1]), float(act[2]), launches=0)
            self.lib.call("rb_gemm_tc", _ptr(out), out.stride(0), self.code, _ptr(x), x.stride(0), T,
                          _ptr(weight.w), weight.w.stride(0), rows, rows, weight.n_in, 3, weight.inner, 1, 0,
                          1.0, self._stream())
            return out
        if act is not None:
            if isinstance(x, NormedRows):
                x = self.normed(x)
            T, rows = x.shape[0], weight.w.shape[0]
            gu = self.linear(x, LinearWeight(weight.w, rows, weight.n_in), out_dtype=torch.float32)
            out = torch.empty((T, weight.inner), dtype=self.dtype, device=self.device)
            alpha, limit, shift = act
            self.lib.call("rb_gated_act", _ptr(out), _ptr(gu), self.code, F32, T, weight.inner, gu.stride(0),
                          weight.block, float(alpha), float(limit), float(shift), self._stream())
            return out
        pending = x if isinstance(x, NormedRows) else None
        if pending is not None:
            if weight.block == 16 and self._takes_pending(pending, weight.w):
                x = pending.scaled
            else:
                x, pending = self.normed(pending), None
        T = x.shape[0]
        out = torch.empty((T, weight.inner), dtype=self.dtype, device=self.device)
        rows = weight.w.shape[0]
        if weight.block == 16 and self._tensor_core_ok(x, weight.w):
            # one accumulator per tile; gate and up of a feature meet in the epilogue, and the
            # activation and the product happen on the way out
            if pending is not None:
                self._pending_norm(pending)
            self.lib.call("rb_gemm_tc", _ptr(out), out.stride(0), self.code, _ptr(x), x.stride(0), T,
                          _ptr(weight.w), weight.w.stride(0), rows, rows, weight.n_in, 3, weight.inner, 1, 0,
                          1.0, self._stream())
            return out
        gu = self.linear(x, LinearWeight(weight.w, rows, weight.n_in))
        self.lib.call("rb_silu_mul", _ptr(out), _ptr(gu), self.code, self.code, T, weight.inner, gu.stride(0),
                      weight.block, self._stream())
        return out

    def rotate_append(self, qkv: torch.Tensor, rotary, meta, view, n_heads: int) -> torch.Tensor:
        """Rotates q (and k) by position, appends k and v to the cache; returns q [T, H, D]."""
        D, Kh = view.head_dim, view.n_kv_heads
        T, width = qkv.shape
        if rotary is None:
            inv_freq, interleaved, rot_dim = self._zeros_freq(D), False, D
        else:
            inv_freq, interleaved, rot_dim = rotary
        want = (n_heads + (2 * Kh if view.writes else 0)) * D
        if width != want:
            raise KernelError(f"rotate_append: rows of {width} values, expected {want}")
        q = torch.empty((T, n_heads, D), dtype=self.dtype, device=self.device)
        self.lib.call("rb_rotate_append", _ptr(q), _ptr(qkv), qkv.stride(0), self.code, _ptr(inv_freq),
                      _ptr(meta.tok_pos), _ptr(meta.tok_slot), _ptr(view.k), _ptr(view.v), _ptr(view.page_table),
                      view.max_pages, view.page_size, T, n_heads, Kh, D, 1 if view.writes else 0, rot_dim,
                      1 if interleaved else 0, self._stream())
        return q

    def project_rotate_append(self, h: torch.Tensor, weight: LinearWeight, rotary, meta, view,
                              n_heads: int) -> torch.Tensor:
        """q/k/v product of the normed rows ``h``, rotation by position and cache append; returns the
        rotated q [T, H, D].  For a few tokens (a decode step) the product's own epilogue rotates and
        appends, from its float32 sums; otherwise the product is stored and ``rotate_append`` follows."""
        pending = h if isinstance(h, NormedRows) else None
        if pending is not None:
            if self._takes_pending(pending, weight.w):
                h = pending.scaled
            else:
                h, pending = self.normed(pending), None
        T, K = h.shape
        D, Kh = view.head_dim, view.n_kv_heads
        splits = self._k_splits(T, weight.n_out, K)
        if rotary is None:
            inv_freq, interleaved, rot_dim = self._zeros_freq(D), False, D
        else:
            inv_freq, interleaved, rot_dim = rotary
        if (self.dtype == torch.bfloat16 and self._tensor_core_ok(h, weight.w)
                and weight.n_out == (n_heads + (2 * Kh if view.writes else 0)) * D
                and self.lib.raw("rb_gemm_tc_qkv_supports")(T, D, splits)):
            q = torch.empty((T, n_heads, D), dtype=self.dtype, device=self.device)
            if pending is not None:
                self._pending_norm(pending)
            self.lib.call("rb_gemm_tc_qkv", _ptr(q), _ptr(h), h.stride(0), T, _ptr(weight.w), weight.w.stride(0), K,
                          splits, _ptr(inv_freq), _ptr(meta.tok_pos), _ptr(meta.tok_slot), _ptr(view.k), _ptr(view.v),
                          _ptr(view.page_table), view.max_pages, view.page_size, n_heads, Kh, D,
                          1 if view.writes else 0, 1 if interleaved else 0, rot_dim, self._stream())
            return q
        return self.rotate_append(self.linear(pending if pending is not None else h, weight), rotary, meta, view, n_heads)

    def _zeros_freq(self, D):
        z = getattr(self, "_zf", None)
        if z is None or z.shape[0] < D // 2:
            self._zf = z = torch.zeros(max(D // 2, 1), dtype=torch.float32, device=self.device)
        return z

    def attention(self, q: torch.Tensor, meta, view, n_heads: int, scale: float,
                  window: Optional[int], sinks: Optional[torch.Tensor] = None, softcap: float = 0.0) -> torch.Tensor:
        """Each new token's queries over its sequence's cached keys up to its own position.  ``sinks`` (float32 [H]):
        head h's softmax denominator also holds exp(sinks[h]); ``softcap`` > 0: score <- softcap * tanh(score /
        softcap).  Every attention kernel of the library takes both."""
        T, H, D = q.shape
        Kh = view.n_kv_heads
        out = torch.empty((T, H * D), dtype=self.dtype, device=self.device)
        win = int(window or 0)
        if sinks is not None or softcap > 0.0:
            if sinks is not None:
                self._check(sinks, torch.float32, "attention sinks")
            self.lib.call("rb_attention_next", _ptr(sinks), float(softcap), launches=0)
        if self.dtype == torch.bfloat16 and meta.single_token and \
                self.lib.raw("rb_attention_tiled_supports")(H, Kh, D, view.page_size, 1):
            on_tma = self.decode_on_tma and self.lib.raw("rb_attention_decode_tma_supports")(H, Kh, D, view.page_size)
            if on_tma:
                n_splits = self.lib.raw("rb_attention_decode_tma_parts")(T * Kh, max(1, -(-meta.max_context // 64)), D)
            else:
                n_splits = self.lib.raw("rb_attention_decode_parts")(T, Kh, meta.max_context)
            part_o = part_ml = None
            # the parts of a small grid are a thread-block cluster and merge on chip
            on_chip = on_tma and bool(self.lib.raw("rb_attention_decode_tma_on_chip")(T * Kh, n_splits, D))
            if n_splits > 1 and not on_chip:
                part_o = torch.empty((T, H, n_splits, D), dtype=torch.float32, device=self.device)
                part_ml = torch.empty((T, H, n_splits, 2), dtype=torch.float32, device=self.device)
            if on_tma:
                # keys and values by TMA (head sizes 64 and 128)
                self.lib.call("rb_attention_decode_tma", _ptr(out), _ptr(q), _ptr(view.k), _ptr(view.v),
                              view.k.shape[0], _ptr(view.page_table), view.max_pages, view.page_size,
                              _ptr(meta.tok_pos), _ptr(meta.tok_slot), T, H, Kh, D, float(scale), win,
                              _ptr(part_o), _ptr(part_ml), n_splits, self._stream(),
                              launches=2 if n_splits > 1 and not on_chip else 1)
            else:
                self.lib.call("rb_attention_decode", _ptr(out), _ptr(q), _ptr(view.k), _ptr(view.v),
                              _ptr(view.page_table), view.max_pages, view.page_size, _ptr(meta.tok_pos),
                              _ptr(meta.tok_slot), T, H, Kh, D, float(scale), win, _ptr(part_o), _ptr(part_ml),
                              n_splits, self._stream(), launches=2 if n_splits > 1 else 1)
        elif self.dtype == torch.bfloat16 and self.prefill_on_tcgen05 and \
                self.lib.raw("rb_attention_prefill_tc_supports")(H, Kh, D, view.page_size):
            tok0, ntok, n_tiles = self._prefill_tiles(meta, 128 // (H // Kh))
            self.lib.call("rb_attention_prefill_tc", _ptr(out), _ptr(q), _ptr(view.k), _ptr(view.v),
                          view.k.shape[0], _ptr(view.page_table), view.max_pages, view.page_size,
                          _ptr(meta.tok_pos), _ptr(meta.tok_slot), _ptr(tok0), _ptr(ntok), n_tiles, H, Kh, D,
                          float(scale), win, self._stream())
        elif self.dtype == torch.bfloat16 and \
                self.lib.raw("rb_attention_tiled_supports")(H, Kh, D, view.page_size, 0):
            tok0, ntok, n_tiles = self._prefill_tiles(meta, 64 // (H // Kh))
            self.lib.call("rb_attention_prefill", _ptr(out), _ptr(q), _ptr(view.k), _ptr(view.v),
                          _ptr(view.page_table), view.max_pages, view.page_size, _ptr(meta.tok_pos),
                          _ptr(meta.tok_slot), _ptr(tok0), _ptr(ntok), n_tiles, H, Kh, D, float(scale), win,
                          self._stream())
        else:
            self.lib.call("rb_attention_simple", _ptr(out), _ptr(q), self.code, _ptr(view.k), _ptr(view.v),
                          _ptr(view.page_table), view.max_pages, view.page_size, _ptr(meta.tok_pos),
                          _ptr(meta.tok_slot), T, H, Kh, D, float(scale), win, self._stream())
        return out

    def _prefill_tiles(self, meta, tokens_per_tile: int):
        """Tiles of at most ``tokens_per_tile`` consecutive tokens of one sequence (device int32 arrays);
        made once per step and kept on the step's meta."""
        import numpy as np
        key = ("attention_tiles", tokens_per_tile)
        if key not in meta.extra and meta.single_token:
            # one token per sequence: a tile per row, made on the device (this also runs while a
            # decode step is being captured, where a copy from the host is not allowed)
            n = meta.n_tokens
            meta.extra[key] = (torch.arange(n, dtype=torch.int32, device=self.device),
                               torch.ones(n, dtype=torch.int32, device=self.device), n)
        if key not in meta.extra:
            tok0, ntok = [], []
            for c in meta.seqs:
                for i in range(0, c.n_new, tokens_per_tile):
                    tok0.append(c.offset + i)
                    ntok.append(min(tokens_per_tile, c.n_new - i))
            dev = torch.from_numpy(np.asarray([tok0, ntok], dtype=np.int32)).to(self.device)
            meta.extra[key] = (dev[0], dev[1], len(tok0))
        return meta.extra[key]

    # ------------------------------------------------------------------ several residual streams
    def streams_expand(self, x: torch.Tensor, s: int) -> torch.Tensor:
        """[T, E] -> [T, s * E]: every stream a copy of the row."""
        T, E = x.shape
        out = torch.empty((T, s * E), dtype=torch.float32, device=self.device)
        self.lib.call("rb_streams_expand", _ptr(out), _ptr(x), T, s, E, self._stream())
        return out

    def streams_sum(self, x: torch.Tensor, s: int) -> torch.Tensor:
        """[R, s * E] -> [R, E]: the streams added up."""
        R, E = x.shape[0], x.shape[1] // s
        out = torch.empty((R, E), dtype=torch.float32, device=self.device)
        self.lib.call("rb_streams_sum", _ptr(out), _ptr(x), R, s, E, self._stream())
        return out

    def stream_step(self, x: torch.Tensor, s: int, results=None, result_norms=None, norm_eps: float = 0.0,
                    write=None, read=None, want_result: bool = False):
        """What lies between two sublayers over a residual state ``x`` [T, s * E] (float32), in one launch:

        ``results`` (float32 [T, E] each) with ``write`` = (mix [s, s], w_out [s]): x_j <- sum_k mix[k, j] x_k +
        w_out[j] * y, where y is the one result, or with ``result_norms`` (a weight [E] per result) the
        mean of the results each under its RMS norm (eps ``norm_eps``);
        ``read`` = (w_in [s], norm weight [E], eps): returns norm(sum_k w_in[k] x_k) in the compute dtype.
        Either part may be left out.  ``want_result``: also returns y."""
        import ctypes
        self._check(x, torch.float32, "stream_step state")
        T, E = x.shape[0], x.shape[1] // s
        n_y = len(results) if results else 0
        ys = (ctypes.c_void_p * max(n_y, 1))(*[r.data_ptr() for r in (results or [])])
        for r in results or []:
            self._check(r, torch.float32, "stream_step result")
        yn = None
        if result_norms:
            yn = (ctypes.c_void_p * n_y)(*[w.data_ptr() for w in result_norms])
        mix, w_out = write if write is not None else (None, None)
        w_in, norm_w, eps = read if read is not None else (None, None, norm_eps)
        if result_norms and read is not None and float(eps) != float(norm_eps):
            raise KernelError("stream_step: the results' norms and the read's norm have different eps")
        h = torch.empty((T, E), dtype=self.dtype, device=self.device) if read is not None else None
        y_out = torch.empty((T, E), dtype=torch.float32, device=self.device) if want_result else None
        self.lib.call("rb_stream_step", _ptr(x), T, s, E, ys, yn, n_y, _ptr(mix), _ptr(w_out), _ptr(w_in), _ptr(norm_w),
                      float(eps if read is not None else norm_eps), _ptr(h), self.code, _ptr(y_out), self._stream())
        return (h, y_out) if want_result else h

    def normed_mean(self, results, weights, eps: float) -> torch.Tensor:
        """float32 [T, E]: the mean of the results, each divided by its root mean square and multiplied by its weight."""
        import ctypes
        T, E = results[0].shape
        n = len(results)
        out = torch.empty((T, E), dtype=torch.float32, device=self.device)
        ys = (ctypes.c_void_p * n)(*[r.data_ptr() for r in results])
        yn = (ctypes.c_void_p * n)(*[w.data_ptr() for w in weights])
        # the combining part of the stream step alone: no state
        self.lib.call("rb_stream_step", c_void_p(0), T, 1, E, ys, yn, n, c_void_p(0), c_void_p(0), c_void_p(0),
                      c_void_p(0), float(eps), c_void_p(0), self.code, _ptr(out), self._stream())
        return out

    # ------------------------------------------------------------------ attention with a projection norm, partial rotation, a gate
    def cache_head_width(self, head_dim: int, value_dim: int) -> int:
        """The width of the cache rows that hold keys of ``head_dim`` and values of ``value_dim`` (both padded
        with zeros to it): the larger of the two, in bfloat16 rounded up to a multiple of 16 so that the
        tensor-core attention kernels take it."""
        w = max(int(head_dim), int(value_dim))
        return -(-w // 16) * 16 if self.dtype == torch.bfloat16 else w

    def norm_rotate_append(self, proj: torch.Tensor, table, meta, view, n_heads: int, head_dim: int, value_dim: int,
                           q_norm_w, k_norm_w, eps: float, head_norm: bool = False) -> torch.Tensor:
        """From rows [q | k | v | ...] of the projections: q and k under an RMS norm over the whole
        projection (if weights are given), the first rot_dim values of every head turned by position, k and v
        appended to the cache (rows ``view.head_dim`` wide, padded with zeros); returns q [T, H, view.head_dim].
        ``head_norm``: instead, every q and k head is divided by its own root mean square AFTER the rotation (no weights)."""
        self._check(proj, self.dtype, "norm_rotate_append projections")
        T, Dc, Kh = proj.shape[0], view.head_dim, view.n_kv_heads
        if table is None:
            freq, magnitude, interleaved, rot_dim = None, 1.0, True, 0
        else:
            freq, magnitude, interleaved, rot_dim = table
        q = torch.empty((T, n_heads, Dc), dtype=self.dtype, device=self.device)
        self.lib.call("rb_norm_rotate_append", _ptr(q), _ptr(proj), proj.stride(0), self.code, _ptr(q_norm_w), _ptr(k_norm_w),
                      float(eps), _ptr(freq), float(magnitude), _ptr(meta.tok_pos), _ptr(meta.tok_slot), _ptr(view.k),
                      _ptr(view.v), _ptr(view.page_table), view.max_pages, view.page_size, T, n_heads, Kh, head_dim,
                      value_dim, Dc, rot_dim, 1 if interleaved else 0, 1, 1 if head_norm else 0, self._stream())
        return q

    def head_gate(self, a: torch.Tensor, proj: torch.Tensor, gate_column, n_heads: int, value_dim: int,
                  cache_width: int, per_value: bool = False) -> torch.Tensor:
        """[T, H * cache_width] -> [T, H * value_dim]: the padding dropped and head h multiplied by
        sigmoid(proj[t, gate_column + h]) (no gate: ``gate_column`` None); ``per_value``: value j of head h by
        sigmoid(proj[t, gate_column + h * value_dim + j])."""
        if gate_column is None and value_dim == cache_width:
            return a
        T = a.shape[0]
        out = torch.empty((T, n_heads * value_dim), dtype=self.dtype, device=self.device)
        gate = c_void_p(proj.data_ptr() + gate_column * proj.element_size()) if gate_column is not None else c_void_p(0)
        self.lib.call("rb_head_gate", _ptr(out), _ptr(a), gate, proj.stride(0) if proj is not None else 0, self.code, T, n_heads, value_dim,
                      cache_width, 1 if per_value else 0, self._stream())
        return out

    # ------------------------------------------------------------------ recurrent mixers
    def _runs(self, meta):
        """The step's runs of consecutive rows, one per sequence (device int32: first row, count; per row: the
        first row of its run); None for a step of one token per sequence, where every row is its own run."""
        if meta.single_token:
            return None, None, None, meta.n_tokens
        key = "runs"
        if key not in meta.extra:
            import numpy as np
            n, T = len(meta.seqs), meta.n_tokens
            packed = np.empty(2 * n + T, dtype=np.int32)
            for i, c in enumerate(meta.seqs):
                packed[i], packed[n + i] = c.offset, c.n_new
                packed[2 * n + c.offset:2 * n + c.offset + c.n_new] = c.offset
            dev = torch.from_numpy(packed).to(self.device)
            meta.extra[key] = (dev[:n], dev[n:2 * n], dev[2 * n:], n)
        return meta.extra[key]

    def gated_recurrence(self, proj: torch.Tensor, p, state, meta) -> torch.Tensor:
        """The gated linear recurrence of ``parts.recurrent.GatedLinearRecurrence`` ``p`` on rows
        [x channels | y channels] (float32): S_t * gelu_tanh(y_t) as [T, inner] in the compute dtype; the
        sequences' state (``state["S"]``, ``state["tail"]``) moves on."""
        self._check(proj, torch.float32, "gated_recurrence projections")
        T, W, B, K = proj.shape[0], p.inner, p.blocks, p.taps
        Wb = W // B
        first, count, tok_first, n_seq = self._runs(meta)
        f = p.f32
        tail = state.get("tail")
        out = torch.empty((T, W), dtype=self.dtype, device=self.device)
        if first is None and T <= self.lib.raw("rb_gated_step_max_rows")() and self.fuse_recurrent_step:
            # a decode step: convolution, gates, recurrence and output in one launch
            self.lib.call("rb_gated_step", _ptr(out), self.code, _ptr(proj), proj.stride(0), F32, 0, W, _ptr(f["x.b"]),
                          _ptr(f["y.b"]), _ptr(f["conv"]), _ptr(f["conv.b"]), _ptr(p.w_gates), _ptr(f["ra.b"]), _ptr(f["ri.b"]),
                          _ptr(f["lam"]), float(p.decay_scale), _ptr(state["S"]), _ptr(tail), _ptr(meta.tok_slot),
                          _ptr(meta.tok_pos), T, W, Wb, K, self._stream())
            return out
        u = torch.empty((T, W), dtype=torch.float32, device=self.device)
        self.lib.call("rb_conv_causal", _ptr(u), _ptr(proj), proj.stride(0), 0, F32, _ptr(f["x.b"]), _ptr(f["conv"]),
                      _ptr(f["conv.b"]), _ptr(tail), _ptr(tok_first), _ptr(meta.tok_slot), _ptr(meta.tok_pos), T, W, K, 0,
                      self._stream())
        gates = torch.empty((T, B, 2 * Wb), dtype=torch.float32, device=self.device)
        self.lib.call("rb_gemm_simple_batched", _ptr(gates), gates.stride(0), F32, _ptr(u), u.stride(0), _ptr(p.w_gates), Wb,
                      F32, T, 2 * Wb, Wb, 0, 1.0, B, 2 * Wb, Wb, 2 * Wb * Wb, self._stream())
        self.lib.call("rb_gated_scan", _ptr(out), self.code, _ptr(u), _ptr(gates), _ptr(f["ra.b"]), _ptr(f["ri.b"]),
                      _ptr(f["lam"]), float(p.decay_scale), _ptr(proj), proj.stride(0), F32, 0, W, _ptr(f["x.b"]),
                      _ptr(f["y.b"]), _ptr(state["S"]), _ptr(tail), _ptr(first), _ptr(count), _ptr(meta.tok_slot),
                      _ptr(meta.tok_pos), n_seq, T, W, Wb, K, self._stream(), launches=1 if first is None else 2)
        return out

    def matrix_memory(self, proj: torch.Tensor, p, state, meta) -> torch.Tensor:
        """The matrix memory of ``parts.recurrent.MatrixMemory`` ``p`` on rows [q | k | v | g | i | f] (float32):
        the heads' outputs under their norm, weight and gate as [T, H * value_dim] in the compute dtype; the
        sequences' state (``state["C"]``, ``["n"]``, ``["m"]``) moves on."""
        self._check(proj, torch.float32, "matrix_memory projections")
        T, H, D, Dv = proj.shape[0], p.n_heads, p.head_dim, p.value_dim
        first, count, _, n_seq = self._runs(meta)
        at = p.offsets()
        o = torch.empty((T, H * Dv), dtype=torch.float32, device=self.device)
        self.lib.call("rb_matrix_memory", _ptr(o), _ptr(proj), proj.stride(0), F32, at["q"], at["k"], at["v"], at["i"],
                      at["f"], _ptr(p.i_bias), _ptr(p.f_bias), float(p.gate_cap), float(D) ** -0.5, float(p.floor),
                      _ptr(state["C"]), _ptr(state["n"]), _ptr(state["m"]), _ptr(first), _ptr(count), _ptr(meta.tok_slot),
                      n_seq, H, D, Dv, self._stream())
        out = torch.empty((T, H * Dv), dtype=self.dtype, device=self.device)
        self.lib.call("rb_head_norm_gate", _ptr(out), self.code, _ptr(o), _ptr(p.norm_w), _ptr(proj), proj.stride(0), F32,
                      at["g"], T, H, Dv, float(p.norm_eps), 0, 0, self._stream())
        return out

    def _delta_chunks(self, meta, size: int = 32):
        """The step's runs cut into chunks of ``size`` rows (device int32: per run its first chunk; per chunk its first
        row and its rows), made once per step."""
        key = ("delta_chunks", size)
        if key not in meta.extra:
            import numpy as np
            run0, rows, lens = [], [], []
            for c in meta.seqs:
                run0.append(len(rows))
                for a in range(0, c.n_new, size):
                    rows.append(c.offset + a)
                    lens.append(min(size, c.n_new - a))
            dev = torch.from_numpy(np.asarray(run0 + rows + lens, dtype=np.int32)).to(self.device)
            n, k = len(run0), len(rows)
            meta.extra[key] = (dev[:n], dev[n:n + k], dev[n + k:], k)
        return meta.extra[key]

    def gated_delta(self, proj: torch.Tensor, p, state, meta) -> torch.Tensor:
        """The gated delta rule of ``parts.delta.GatedDeltaRule`` ``p`` on float32 rows [q | k | v | g | b | a] of its
        stacked projection: short convolution and SiLU of q, k, v; unit vectors; gates; the recurrence; the heads'
        outputs under their norm, weight and SiLU gate as [T, H * value_dim] in the compute dtype.  The sequences'
        state (``state["S"]`` kept by value column, ``state["tail"]``) moves on."""
        self._check(proj, torch.float32, "gated_delta projections")
        T, H, G, D, Dv, K = proj.shape[0], p.n_heads, p.n_kv_heads, p.head_dim, p.value_dim, p.taps
        C = 2 * G * D + H * Dv
        at = p.offsets()
        first, count, tok_first, n_runs = self._runs(meta)
        tail = state.get("tail")
        if first is None and self.fuse_delta_step and self.lib.raw("rb_delta_step_lanes")(D, Dv, T) > 0 and \
                T * H <= self.lib.raw("rb_device_sm_count")():
            # a decode step: convolution, unit vectors, gates, the memory's step, norm and gate in one launch, where its
            # blocks (one per row and head, all of a head's columns) are at most one per SM; beyond that the kernels of
            # a prompt, whose blocks are many and small, are faster (measured: 0.667 against 0.642 ms a step at 32 heads)
            out = torch.empty((T, H * Dv), dtype=self.dtype, device=self.device)
            self.lib.call("rb_delta_step", _ptr(out), self.code, _ptr(proj), proj.stride(0), at["g"], at["b"], at["a"],
                          _ptr(p.conv_w), _ptr(p.a_log), _ptr(p.dt_bias), _ptr(p.norm_w), _ptr(state["S"]), _ptr(tail),
                          _ptr(meta.tok_slot), _ptr(meta.tok_pos), T, H, G, D, Dv, K, float(D) ** -0.5, float(p.unit_eps),
                          float(p.norm_eps), self._stream())
            return out
        u = torch.empty((T, C), dtype=torch.float32, device=self.device)
        self.lib.call("rb_conv_causal", _ptr(u), _ptr(proj), proj.stride(0), 0, F32, c_void_p(0), _ptr(p.conv_w), c_void_p(0),
                      _ptr(tail), _ptr(tok_first), _ptr(meta.tok_slot), _ptr(meta.tok_pos), T, C, K, 1, self._stream())
        gates = torch.empty((T * (3 * H + G),), dtype=torch.float32, device=self.device)
        beta, decay, log_decay, kq = gates[:T * H], gates[T * H:2 * T * H], gates[2 * T * H:3 * T * H], gates[3 * T * H:]
        self.lib.call("rb_delta_prepare", _ptr(u), u.stride(0), _ptr(proj), proj.stride(0), at["b"], at["a"], _ptr(p.a_log),
                      _ptr(p.dt_bias), _ptr(beta), _ptr(decay), _ptr(log_decay), _ptr(kq), T, H, G, D, float(D) ** -0.5,
                      float(p.unit_eps), self._stream())
        o = torch.empty((T, H * Dv), dtype=torch.float32, device=self.device)
        if first is not None and self.delta_in_chunks and self.lib.raw("rb_gated_delta_chunked_supports")(D, Dv, u.stride(0), G):
            # runs of several tokens: chunks of 32, the chain in time only from chunk to chunk
            run_chunk0, chunk_row, chunk_len, n_chunks = self._delta_chunks(meta)
            scratch = torch.empty((n_chunks * H * self.lib.raw("rb_gated_delta_chunk_floats")(D, Dv),), dtype=torch.float32,
                                  device=self.device)
            self.lib.call("rb_gated_delta_chunked", _ptr(o), _ptr(u), u.stride(0), _ptr(beta), _ptr(log_decay), _ptr(state["S"]),
                          _ptr(scratch), _ptr(first), _ptr(count), _ptr(run_chunk0), _ptr(chunk_row), _ptr(chunk_len),
                          _ptr(meta.tok_slot), n_runs, n_chunks, H, G, D, Dv, self._stream(), launches=2)
        else:
            self.lib.call("rb_gated_delta", _ptr(o), _ptr(u), u.stride(0), _ptr(beta), _ptr(decay), _ptr(kq), _ptr(state["S"]),
                          _ptr(first), _ptr(count), _ptr(meta.tok_slot), n_runs, H, G, D, Dv, self._stream())
        if K > 1:
            self.lib.call("rb_conv_tail_update", _ptr(tail), _ptr(proj), proj.stride(0), 0, F32, c_void_p(0), _ptr(first),
                          _ptr(count), _ptr(meta.tok_slot), _ptr(meta.tok_pos), n_runs, C, K, self._stream())
        out = torch.empty((T, H * Dv), dtype=self.dtype, device=self.device)
        self.lib.call("rb_head_norm_gate", _ptr(out), self.code, _ptr(o), _ptr(p.norm_w), _ptr(proj), proj.stride(0), F32,
                      at["g"], T, H, Dv, float(p.norm_eps), 1, 1, self._stream())
        return out


    # ------------------------------------------------------------------ around a sublayer
    def rmsnorm_grouped(self, x: torch.Tensor, w: torch.Tensor, groups: int, eps: float, out_dtype=None) -> torch.Tensor:
        """The row cut into ``groups`` equal consecutive parts, each divided by its own root mean square (eps under the
        root), the whole times w; float32 arithmetic, the result in the compute dtype."""
        self._check(x, torch.float32, "rmsnorm_grouped input")
        T, E = x.shape
        out = torch.empty((T, E), dtype=out_dtype or self.dtype, device=self.device)
        self.lib.call("rb_rmsnorm_grouped", _ptr(out), _CODE[out.dtype], _ptr(x), _ptr(w), T, E, int(groups), float(eps),
                      self._stream())
        return out

    def input_filter(self, h: torch.Tensor, taps: torch.Tensor, ring: Optional[torch.Tensor], meta) -> torch.Tensor:
        """h_t + sum_j taps[:, j] h_(t - K + 1 + j) over a sequence's rows (float32 sums, the result in h's dtype).  The
        sequence's last inputs live in ``ring`` (float32 [n_slots, K, width], a row per position modulo K), which moves on."""
        self._check(h, self.dtype, "input_filter rows")
        T, C = h.shape
        K = taps.shape[1]
        first, count, tok_first, n_runs = self._runs(meta)
        out = torch.empty_like(h)
        self.lib.call("rb_input_filter", _ptr(out), _ptr(h), self.code, _ptr(taps), _ptr(ring), _ptr(tok_first),
                      _ptr(meta.tok_slot), _ptr(meta.tok_pos), T, C, K, self._stream())
        if first is not None and K > 1:
            self.lib.call("rb_conv_tail_update", _ptr(ring), _ptr(h), h.stride(0), 0, self.code, c_void_p(0), _ptr(first),
                          _ptr(count), _ptr(meta.tok_slot), _ptr(meta.tok_pos), n_runs, C, K, self._stream())
        return out

    def norm_filter_rows(self, x: torch.Tensor, w: torch.Tensor, groups: int, eps: float, taps: torch.Tensor,
                         ring: Optional[torch.Tensor], meta, add=None):
        """For a step of one token per sequence, in one launch: ``add`` = (y, logits, bias): x += y * sigmoid(logits +
        bias) first; then (h, hf): the norm in groups of x and its filtered rows (``rmsnorm_grouped`` and
        ``input_filter``), the ring moved on.  None where this step or these sizes do not take it."""
        if not (self.fuse_norm_filter and meta.single_token):
            return None
        self._check(x, torch.float32, "norm_filter_rows rows")
        T, E = x.shape
        y = g = b = None
        if add is not None:
            y, g, b = add
            if g.dtype != torch.float32 or y.dtype != torch.float32:
                return None
        if not self.lib.raw("rb_norm_filter_rows_supports")(E, int(groups), g.stride(0) if g is not None else 0):
            return None
        h = torch.empty((T, E), dtype=self.dtype, device=self.device)
        hf = torch.empty((T, E), dtype=self.dtype, device=self.device)
        self.lib.call("rb_norm_filter_rows", _ptr(h), _ptr(hf), self.code, _ptr(x), _ptr(y), _ptr(g),
                      g.stride(0) if g is not None else 0, _ptr(b), _ptr(w), T, E, int(groups), float(eps), _ptr(taps),
                      _ptr(ring), _ptr(meta.tok_slot), _ptr(meta.tok_pos), taps.shape[1], self._stream())
        return h, hf

    def gated_add(self, x: torch.Tensor, y: torch.Tensor, logits: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
        """x += y * sigmoid(logits + bias), value by value, in float32."""
        self._check(x, torch.float32, "gated_add target")
        self._check(y, torch.float32, "gated_add result")
        T, E = x.shape
        self.lib.call("rb_gated_add", _ptr(x), _ptr(y), _ptr(logits), logits.stride(0), _CODE[logits.dtype], _ptr(bias), T, E,
                      self._stream())
        return x

    def add_scaled_rows(self, y: torch.Tensor, z: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        """y += sigmoid(gate[t]) * z, one number per row; float32."""
        self._check(y, torch.float32, "add_scaled_rows target")
        self._check(z, torch.float32, "add_scaled_rows rows")
        T, E = y.shape
        self.lib.call("rb_add_scaled_rows", _ptr(y), _ptr(z), _ptr(gate), gate.stride(0), T, E, self._stream())
        return y

    def softcap(self, v: torch.Tensor, cap: float) -> torch.Tensor:
        """v <- cap * tanh(v / cap), in place (float32)."""
        self._check(v, torch.float32, "softcap values")
        self.lib.call("rb_softcap", _ptr(v), v.numel(), float(cap), self._stream())
        return v

    # ------------------------------------------------------------------ gated linear attention
    def gated_linear_attention(self, proj: torch.Tensor, p, state, meta) -> torch.Tensor:
        """The recurrence of ``parts.gla.GatedLinearAttention`` ``p`` on float32 rows [q | k | v | g | A1 h] of its stacked
        projection: the decays, the memory's steps, the heads' outputs under their norm, weight and SiLU gate as
        [T, H * value_dim] in the compute dtype.  The sequences' memory (``state["S"]``, by value column) moves on."""
        self._check(proj, torch.float32, "gated_linear_attention projections")
        T, H, D, Dv, R = proj.shape[0], p.n_heads, p.head_dim, p.value_dim, p.decay_rank
        if D > self.lib.raw("rb_gla_max_dim")():
            raise KernelError(f"gated linear attention: {D} key channels per head are more than the kernel holds")
        at = p.offsets()
        first, count, _, n_runs = self._runs(meta)
        chunked = first is not None and self.gla_in_chunks and \
            self.lib.raw("rb_gla_chunked_supports")(D, Dv, proj.stride(0), at["q"], at["k"], at["v"])
        alpha = torch.empty((T, H * D), dtype=torch.float32, device=self.device)       # the decays, or their logarithms
        self.lib.call("rb_gla_decay", _ptr(alpha), _ptr(proj), proj.stride(0), at["a"], _ptr(p.a2), _ptr(p.a2_bias), T, H * D, R,
                      float(p.tau), 1 if chunked else 0, self._stream())
        o = torch.empty((T, H * Dv), dtype=torch.float32, device=self.device)
        if chunked:
            # runs of several tokens: chunks of 32, the chain in time only from chunk to chunk
            run_chunk0, chunk_row, chunk_len, n_chunks = self._delta_chunks(meta)
            scratch = torch.empty((n_chunks * H * self.lib.raw("rb_gla_chunk_floats")(D),), dtype=torch.float32,
                                  device=self.device)
            self.lib.call("rb_gla_chunked", _ptr(o), _ptr(proj), proj.stride(0), at["q"], at["k"], at["v"], _ptr(alpha),
                          float(D) ** -0.5, _ptr(state["S"]), _ptr(scratch), _ptr(first), _ptr(count), _ptr(run_chunk0),
                          _ptr(chunk_row), _ptr(chunk_len), _ptr(meta.tok_slot), n_runs, n_chunks, H, D, Dv, self._stream(),
                          launches=2)
        else:
            self.lib.call("rb_gla_scan", _ptr(o), _ptr(proj), proj.stride(0), at["q"], at["k"], at["v"], _ptr(alpha),
                          float(D) ** -0.5, _ptr(state["S"]), _ptr(first), _ptr(count), _ptr(meta.tok_slot), n_runs, H, D, Dv,
                          self._stream())
        out = torch.empty((T, H * Dv), dtype=self.dtype, device=self.device)
        self.lib.call("rb_head_norm_gate", _ptr(out), self.code, _ptr(o), _ptr(p.norm_w), _ptr(proj), proj.stride(0), F32,
                      at["g"], T, H, Dv, float(p.norm_eps), 1, 1, self._stream())
        return out

    # ------------------------------------------------------------------ sublayers that read the residual stream itself
    def round_rows(self, x: torch.Tensor) -> torch.Tensor:
        """The float32 rows in the compute dtype (the rows themselves where that is float32)."""
        self._check(x, torch.float32, "round_rows rows")
        if self.dtype == torch.float32:
            return x
        out = torch.empty(x.shape, dtype=self.dtype, device=self.device)
        self.lib.call("rb_round_rows", _ptr(out), self.code, _ptr(x), x.numel(), self._stream())
        return out

    def norm_add(self, x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, want_rounded: bool = False):
        """x += y / rms(y) * w, row by row in float32 (y: a sublayer's float32 result).  ``want_rounded``: the new rows
        are also returned in the compute dtype, from the same kernel."""
        self._check(x, torch.float32, "norm_add target")
        self._check(y, torch.float32, "norm_add result")
        T, E = x.shape
        if y.shape != x.shape or w.shape[0] != E:
            raise KernelError(f"norm_add: shapes {tuple(x.shape)}, {tuple(y.shape)}, {tuple(w.shape)}")
        rounded = None
        if want_rounded and self.dtype != torch.float32:
            rounded = torch.empty((T, E), dtype=self.dtype, device=self.device)
        self.lib.call("rb_norm_add", _ptr(x), _ptr(y), _ptr(w), float(eps), T, E, _ptr(rounded), self.code, self._stream())
        if not want_rounded:
            return None
        return x if rounded is None else rounded

    def token_gate(self, a: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """gelu_tanh(a[t]) * table[ids[t]] -> [T, dim] in the compute dtype (a: float32 [T, dim])."""
        self._check(a, torch.float32, "token_gate rows")
        self._check(table, self.dtype, "token_gate table")
        T, dim = a.shape
        out = torch.empty((T, dim), dtype=self.dtype, device=self.device)
        self.lib.call("rb_token_gate", _ptr(out), self.code, _ptr(a), a.stride(0), _ptr(table), self.code, _ptr(ids), T, dim,
                      self._stream())
        return out

    def embed_pairs(self, meta, table: torch.Tensor, scale: float, pair_table: torch.Tensor, pair_hash,
                    previous: torch.Tensor) -> torch.Tensor:
        """float32 rows table[id] * scale + pair_table[(previous id * a + id * b) mod n] with (n, a, b) = ``pair_hash``;
        a sequence's first token takes row n.  ``previous`` (int32 [n_slots, 1]) holds every sequence's last token and
        moves on."""
        T, (V, E) = meta.n_tokens, table.shape
        buckets, mul_prev, mul_cur = pair_hash
        out = torch.empty((T, E), dtype=torch.float32, device=self.device)
        self.lib.call("rb_embed_pairs", _ptr(out), _ptr(table), _ptr(pair_table), _CODE[table.dtype], _ptr(meta.token_ids),
                      _ptr(meta.tok_pos), _ptr(meta.tok_slot), _ptr(previous), T, E, V, float(scale), int(buckets),
                      int(mul_prev), int(mul_cur), 1 if meta.single_token else 0, self._stream(),
                      launches=1 if meta.single_token else 2)
        return out

    def qk_prepare(self, proj: torch.Tensor, meta, view, n_heads: int, head_dim: int, value_dim: int, table, norm,
                   q_norm_w, k_norm_w, eps: float, conv=None, tail=None, values_are_keys: bool = False, v_mix=None,
                   gate_heads: bool = False):
        """From float32 rows [q | k | v (unless ``values_are_keys``) | a gate logit per head (if ``gate_heads``)]:
        ``conv`` ([(H + Kh) D, taps] float32): a causal convolution over time on the q and k channels, whose last
        rows per sequence live in ``tail`` (a ring by position); ``norm`` "projection" (weights [H D], [Kh D]) or
        "head_weight" (one [D] for all q heads, one for all k heads): RMS norms before the rotation; the rotation of
        ``table``; k and v into the cache (v: own, or (1 - l) v + l other[:, at:] with ``v_mix`` = (l, other, at), or
        the keys as they leave the convolution).  Returns (q [T, H, cache width], gate logits [T, H] or None), both in
        the compute dtype."""
        self._check(proj, torch.float32, "qk_prepare projections")
        T, Dc, Kh = proj.shape[0], view.head_dim, view.n_kv_heads
        if table is None:
            freq, magnitude, interleaved, rot_dim = None, 1.0, True, 0
        else:
            freq, magnitude, interleaved, rot_dim = table
        mode = {None: 0, "projection": 1, "head_weight": 2}[norm]
        K = conv.shape[1] if conv is not None else 0
        first = count = tok_first = None
        if conv is not None and K > 1:
            first, count, tok_first, n_runs = self._runs(meta)
        q = torch.empty((T, n_heads, Dc), dtype=self.dtype, device=self.device)
        gates = torch.empty((T, n_heads), dtype=self.dtype, device=self.device) if gate_heads else None
        lam, other, at = v_mix if v_mix is not None else (0.0, None, 0)
        mix_ptr = c_void_p(other.data_ptr() + at * 4) if other is not None else c_void_p(0)
        self.lib.call("rb_qk_prepare", _ptr(q), _ptr(gates), self.code, _ptr(proj), proj.stride(0), _ptr(conv), K, _ptr(tail),
                      _ptr(tok_first), mode, _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(freq), float(magnitude),
                      rot_dim, 1 if interleaved else 0, _ptr(meta.tok_pos), _ptr(meta.tok_slot), _ptr(view.k), _ptr(view.v),
                      _ptr(view.page_table), view.max_pages, view.page_size, T, n_heads, Kh, head_dim, value_dim, Dc,
                      1 if values_are_keys else 0, mix_ptr, other.stride(0) if other is not None else 0, float(lam),
                      1 if gate_heads else 0, self._stream())
        if first is not None:
            # runs of several rows: the ring moves on to each run's end after every row has read it
            C = (n_heads + Kh) * head_dim
            self.lib.call("rb_conv_tail_update", _ptr(tail), _ptr(proj), proj.stride(0), 0, F32, c_void_p(0), _ptr(first),
                          _ptr(count), _ptr(meta.tok_slot), _ptr(meta.tok_pos), n_runs, C, K, self._stream())
        return q, gates

    def latent_rotate_append(self, down: torch.Tensor, n_heads: int, head_dim: int, rot_dim: int, kv_rank: int, table,
                             w: torch.Tensor, eps: float, meta, view) -> torch.Tensor:
        """From float32 rows [H query heads of head_dim + rot_dim | latent of kv_rank | key part of rot_dim]: the
        latent under its RMS norm and weight and the key part turned by position go to the sequence's page as
        [c | k_r | zeros]; the queries are returned ([T, H (head_dim + rot_dim)], compute dtype) with their last
        rot_dim values turned."""
        self._check(down, torch.float32, "latent_rotate_append rows")
        T = down.shape[0]
        freq, magnitude, interleaved = None, 1.0, True
        if rot_dim:
            freq, magnitude, interleaved, turned = table
            if turned != rot_dim:
                raise KernelError("latent_rotate_append: the position encoding turns the whole key part")
        q = torch.empty((T, n_heads * (head_dim + rot_dim)), dtype=self.dtype, device=self.device)
        self.lib.call("rb_latent_rotate_append", _ptr(q), self.code, _ptr(down), down.stride(0), _ptr(w), float(eps),
                      _ptr(freq), float(magnitude), 1 if interleaved else 0, _ptr(meta.tok_pos), _ptr(meta.tok_slot),
                      _ptr(view.k), _ptr(view.page_table), view.max_pages, view.page_size, view.head_dim, T, n_heads,
                      head_dim, rot_dim, kv_rank, self._stream())
        return q

    def retention(self, proj: torch.Tensor, p, state, meta) -> torch.Tensor:
        """The recurrence of ``parts.retention.Retention`` ``p`` on float32 rows [q | k | v | g] of its stacked
        projection: q and k turned by position (in place), the memory's steps with the heads' fixed decays (gated
        linear attention's kernels on one shared row of decays), each head's outputs divided by their root mean square
        and multiplied by silu(g), as [T, H * value_dim] in the compute dtype.  ``state["S"]`` moves on."""
        self._check(proj, torch.float32, "retention projections")
        T, H, D, Dv = proj.shape[0], p.n_heads, p.head_dim, p.value_dim
        if D > self.lib.raw("rb_gla_max_dim")():
            raise KernelError(f"retention: {D} key channels per head are more than the kernel holds")
        at = p.offsets()
        table = p.position.table() if hasattr(p.position, "table") else None
        if table is not None:
            freq, magnitude, interleaved, rot_dim = table
            # q heads and k heads are neighbours in a row: 2 H heads of D from column 0
            self.lib.call("rb_rotate_rows", _ptr(proj), proj.stride(0), at["q"], 2 * H, D, _ptr(freq), float(magnitude),
                          rot_dim, 1 if interleaved else 0, _ptr(meta.tok_pos), T, self._stream())
        first, count, _, n_runs = self._runs(meta)
        chunked = first is not None and self.gla_in_chunks and \
            self.lib.raw("rb_gla_chunked_supports")(D, Dv, proj.stride(0), at["q"], at["k"], at["v"])
        o = torch.empty((T, H * Dv), dtype=torch.float32, device=self.device)
        self.lib.call("rb_gla_shared_decays", launches=0)
        if chunked:
            run_chunk0, chunk_row, chunk_len, n_chunks = self._delta_chunks(meta)
            scratch = torch.empty((n_chunks * H * self.lib.raw("rb_gla_chunk_floats")(D),), dtype=torch.float32,
                                  device=self.device)
            self.lib.call("rb_gla_chunked", _ptr(o), _ptr(proj), proj.stride(0), at["q"], at["k"], at["v"], _ptr(p.log_decays),
                          float(D) ** -0.5, _ptr(state["S"]), _ptr(scratch), _ptr(first), _ptr(count), _ptr(run_chunk0),
                          _ptr(chunk_row), _ptr(chunk_len), _ptr(meta.tok_slot), n_runs, n_chunks, H, D, Dv, self._stream(),
                          launches=2)
        else:
            self.lib.call("rb_gla_scan", _ptr(o), _ptr(proj), proj.stride(0), at["q"], at["k"], at["v"], _ptr(p.decays),
                          float(D) ** -0.5, _ptr(state["S"]), _ptr(first), _ptr(count), _ptr(meta.tok_slot), n_runs, H, D, Dv,
                          self._stream())
        out = torch.empty((T, H * Dv), dtype=self.dtype, device=self.device)
        self.lib.call("rb_head_norm_gate", _ptr(out), self.code, _ptr(o), _ptr(p.norm_w), _ptr(proj), proj.stride(0), F32,
                      at["g"], T, H, Dv, float(p.norm_eps), 1, 1, self._stream())
        return out

    # ------------------------------------------------------------------ attention through latents
    def latent_norm_append(self, down: torch.Tensor, q_rank: int, kv_rank: int, wq: torch.Tensor, wkv: torch.Tensor,
                           eps: float, meta, view) -> torch.Tensor:
        """From float32 rows [query latent | key/value latent]: each under its RMS norm and weight; the query latent is
        returned ([T, q_rank], compute dtype), the other goes to the sequence's page (``view.head_dim`` wide, padded
        with zeros)."""
        self._check(down, torch.float32, "latent_norm_append rows")
        T = down.shape[0]
        cq = torch.empty((T, q_rank), dtype=self.dtype, device=self.device)
        self.lib.call("rb_latent_norm_append", _ptr(cq), self.code, _ptr(down), down.stride(0), 0, q_rank, q_rank, kv_rank,
                      _ptr(wq), _ptr(wkv), float(eps), _ptr(view.k), _ptr(view.page_table), view.max_pages, view.page_size,
                      view.head_dim, _ptr(meta.tok_pos), _ptr(meta.tok_slot), T, self._stream())
        return cq

    def prepare_per_head(self, w: torch.Tensor) -> PerHeadWeight:
        """[heads, n_out, n_in] -> ready for ``per_head_linear``."""
        w = self.to_compute(w)
        return PerHeadWeight(w, w.shape[0], w.shape[1], w.shape[2])

    def per_head_linear(self, x: torch.Tensor, weight: PerHeadWeight) -> torch.Tensor:
        """x [T, heads * n_in] -> [T, heads * n_out]: head h's values times its own matrix (float32 sums)."""
        self._check(x, self.dtype, "per_head_linear input")
        T, H, N, K = x.shape[0], weight.heads, weight.n_out, weight.n_in
        if x.shape[1] != H * K:
            raise KernelError(f"per_head_linear: rows of {x.shape[1]} values are not {H} heads of {K}")
        out = torch.empty((T, H * N), dtype=self.dtype, device=self.device)
        if T <= 16:
            # a decode step: a warp per output and head instead of a few tiles
            self.lib.call("rb_per_head_few_rows", _ptr(out), out.stride(0), self.code, _ptr(x), x.stride(0), _ptr(weight.w),
                          self.code, T, H, N, K, self._stream())
            return out
        self.lib.call("rb_gemm_simple_batched", _ptr(out), out.stride(0), self.code, _ptr(x), x.stride(0), _ptr(weight.w), K,
                      self.code, T, N, K, 0, 1.0, H, N, K, N * K, self._stream())
        return out

    # ------------------------------------------------------------------ routed experts, the variants
    def prepare_expert_gate_up(self, gates: List[torch.Tensor], ups: List[torch.Tensor]) -> ExpertGateUp:
        """The gated experts' first matrices, one expert below the other, an expert's rows [gate | up]."""
        inner, K = gates[0].shape
        if self.dtype == torch.bfloat16 and K % 8 == 0:
            # every expert in the layout of the tensor-core gated product (16 gate rows, then their 16 up rows)
            each = [self.prepare_gate_up(g, u) for g, u in zip(gates, ups)]
            return ExpertGateUp(torch.cat([e.w for e in each], dim=0).contiguous(), inner, K, each[0].w.shape[0], 16)
        w = torch.cat([torch.cat([self.to_compute(g), self.to_compute(u)], dim=0) for g, u in zip(gates, ups)], dim=0)
        return ExpertGateUp(w.contiguous(), inner, K, 2 * inner, 0)

    def route_scored(self, h: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int,
                     keep: int, scoring: str = "softmax", extra_rows: int = 0, router_tc: Optional[LinearWeight] = None):
        """``route`` with its variants: ``scoring`` "sigmoid" takes s = sigmoid(z) output by output; the last
        ``extra_rows`` rows of ``router`` are no outputs: their float32 sums are returned as they are ([T, extra_rows],
        None without).  Returns (ids, weights, extra)."""
        self._check(h, self.dtype, "route input")
        T, K = h.shape
        n = router.shape[0] - extra_rows
        ids = torch.empty((T, top), dtype=torch.int32, device=self.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=self.device)
        extra = torch.empty((T, extra_rows), dtype=torch.float32, device=self.device) if extra_rows else None
        if T >= self.router_tc_from and router_tc is not None and self._tensor_core_ok(h, router_tc.w):
            # the sums (outputs and extra rows) on the tensor cores, then the choice: also for a decode step, where the
            # kernel that does both has a block per token (20 us at 8 tokens against 7 for the two)
            z = self.linear(h, router_tc, out_dtype=torch.float32)
            self.lib.call("rb_route_select_scored", _ptr(ids), _ptr(weights), _ptr(z), _ptr(correction), T, n, int(top),
                          int(groups), int(keep), {"softmax": 0, "sigmoid": 1}[scoring], int(extra_rows), _ptr(extra),
                          self._stream())
            return ids, weights, extra
        z = torch.empty((T, n + extra_rows), dtype=torch.float32, device=self.device) if T >= 64 else None
        self.lib.call("rb_route_scored", _ptr(ids), _ptr(weights), _ptr(h), h.stride(0), self.code, _ptr(router),
                      _ptr(correction), T, K, n, int(top), int(groups), int(keep), _ptr(z),
                      {"softmax": 0, "sigmoid": 1}[scoring], int(extra_rows), _ptr(extra), self._stream(),
                      launches=2 if z is not None else 1)
        return ids, weights, extra

    # ------------------------------------------------------------------ routed experts
    def prepare_router(self, router: torch.Tensor) -> Optional[LinearWeight]:
        """The router's matrix for the tensor-core product, if that product gives the float32 sums: in bfloat16 mode, for
        a matrix whose float32 values are bfloat16 values (then every product of an input value and a weight is exact in
        float32 and the sums are float32 sums); else None, and the router's sums are FFMA sums on the float32 matrix."""
        if self.dtype != torch.bfloat16:
            return None
        w = router.to(device=self.device, dtype=torch.float32)
        if not bool(torch.equal(w.to(torch.bfloat16).to(torch.float32), w)):
            return None
        return self.prepare_linear([w])

    def route(self, h: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int,
              keep: int, router_tc: Optional[LinearWeight] = None):
        """(ids int32 [T, top], weights float32 [T, top]): softmax of the float32 router product over all outputs; the
        ``top`` largest scores plus ``correction`` among the outputs of the ``keep`` best of ``groups`` equal groups;
        the weights are the scores themselves.  ``router_tc``: what ``prepare_router`` gave (many tokens then take the
        tensor-core product for the sums)."""
        self._check(h, self.dtype, "route input")
        T, K = h.shape
        n = router.shape[0]
        ids = torch.empty((T, top), dtype=torch.int32, device=self.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=self.device)
        if T >= 64 and router_tc is not None and self._tensor_core_ok(h, router_tc.w):
            z = self.linear(h, router_tc, out_dtype=torch.float32)
            self.lib.call("rb_route_select", _ptr(ids), _ptr(weights), _ptr(z), _ptr(correction), T, n, int(top), int(groups),
                          int(keep), self._stream())
            return ids, weights
        # from 64 tokens on the router's sums are a tiled product of their own, which leaves them in z
        z = torch.empty((T, n), dtype=torch.float32, device=self.device) if T >= 64 else None
        self.lib.call("rb_route", _ptr(ids), _ptr(weights), _ptr(h), h.stride(0), self.code, _ptr(router), _ptr(correction),
                      T, K, n, int(top), int(groups), int(keep), _ptr(z), self._stream(), launches=2 if z is not None else 1)
        return ids, weights

    def routed_tile(self, pairs: int, n_experts: int, inner: int, width: int) -> int:
        """Rows per tile of the buffer that holds a step's (token, choice) pairs sorted by expert."""
        if not self._routed_on_tensor_cores(inner, width):
            return 64            # the plain grouped product's tile
        per = pairs / max(n_experts, 1)
        return 16 if per <= 16 else 32 if per <= 32 else 64 if per <= 64 else 128

    def _routed_on_tensor_cores(self, inner: int, width: int) -> bool:
        return self.dtype == torch.bfloat16 and inner % 8 == 0 and width % 8 == 0

    def routed_experts(self, h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_up, w_down: LinearWeight,
                       n_experts: int, inner: int, accumulate_into: Optional[torch.Tensor] = None, act=None,
                       weight_on_input: bool = False):
        """sum_j weights[t, j] * expert(ids[t, j])(h[t]) with expert e: W_down_e relu2(W_up_e h); ids >= n_experts are
        identity experts (h[t] itself).  ``w_up``: [n_experts * inner, width], ``w_down``: [n_experts * width, inner].
        Added to ``accumulate_into`` (float32), or returned as float32 rows.
        ``act`` = (alpha, limit, shift): gated experts, ``w_up`` an ``ExpertGateUp``, the inner rows
        g' sigmoid(alpha g') (u' + shift) as in ``gated_linear``.  ``weight_on_input``: sum_j expert(weights[t, j] * h[t])
        instead (the weighted row is rounded to the compute dtype before the expert's first product)."""
        T, E = h.shape
        top = ids.shape[1]
        pairs = T * top
        if accumulate_into is not None:
            out, acc = accumulate_into, 1
        else:
            out, acc = torch.empty((T, E), dtype=torch.float32, device=self.device), 0
        y = pos = None
        if n_experts > 0:
            tile = self.routed_tile(pairs, n_experts, inner, E)
            n_tiles = self.lib.raw("rb_routed_tiles")(pairs, n_experts, tile)
            rows = n_tiles * tile
            plan = torch.empty((pairs + rows + n_tiles,), dtype=torch.int32, device=self.device)
            pos, row_token, tile_group = plan[:pairs], plan[pairs:pairs + rows], plan[pairs + rows:]
            self.lib.call("rb_routed_plan", _ptr(pos), _ptr(row_token), _ptr(tile_group), _ptr(ids), pairs, top, n_experts,
                          tile, n_tiles, self._stream())
            xp = torch.empty((rows, E), dtype=self.dtype, device=self.device)
            if weight_on_input:
                self.lib.call("rb_routed_gather_scaled", _ptr(xp), _ptr(h), h.stride(0), self.code, _ptr(row_token), _ptr(pos),
                              _ptr(weights), top, rows, E, self._stream())
            else:
                self.lib.call("rb_routed_gather", _ptr(xp), _ptr(h), h.stride(0), self.code, _ptr(row_token), rows, E, self._stream())
            mid = torch.empty((rows, inner), dtype=self.dtype, device=self.device)
            y = torch.empty((rows, E), dtype=torch.float32, device=self.device)
            if act is not None:
                # gated experts: the grouped product leaves float32 [gate | up] rows, a kernel makes the inner rows
                per = w_up.rows
                tc = self._routed_on_tensor_cores(inner, E)
                fused = tc and w_up.block == 16 and self.fuse_gated_act
                gu = None if fused else torch.empty((rows, per), dtype=torch.float32, device=self.device)
                if fused:
                    # the activation in the grouped product's epilogue: the inner rows leave it in bfloat16
                    self.lib.call("rb_gemm_tc_gated_act", float(act[0]), float(act[1]), float(act[2]), launches=0)
                    self.lib.call("rb_gemm_tc_grouped", _ptr(tile_group), launches=0)
                    self.lib.call("rb_gemm_tc", _ptr(mid), mid.stride(0), self.code, _ptr(xp), xp.stride(0), rows, _ptr(w_up.w),
                                  w_up.w.stride(0), n_experts * per, per, E, 3, inner, 1, tile, 1.0, self._stream())
                elif tc:
                    self.lib.call("rb_gemm_tc_grouped", _ptr(tile_group), launches=0)
                    self.lib.call("rb_gemm_tc", _ptr(gu), gu.stride(0), F32, _ptr(xp), xp.stride(0), rows, _ptr(w_up.w),
                                  w_up.w.stride(0), n_experts * per, per, E, 0, 0, 1, tile, 1.0, self._stream())
                else:
                    self.lib.call("rb_gemm_grouped_simple", _ptr(gu), gu.stride(0), F32, _ptr(xp), xp.stride(0), _ptr(w_up.w),
                                  w_up.w.stride(0), self.code, _ptr(tile_group), rows, per, E, 0, self._stream())
                if not fused:
                    self.lib.call("rb_gated_act", _ptr(mid), _ptr(gu), self.code, F32, rows, inner, gu.stride(0), w_up.block,
                                  float(act[0]), float(act[1]), float(act[2]), self._stream())
                if tc:
                    self.lib.call("rb_gemm_tc_grouped", _ptr(tile_group), launches=0)
                    self.lib.call("rb_gemm_tc", _ptr(y), y.stride(0), F32, _ptr(mid), mid.stride(0), rows, _ptr(w_down.w),
                                  w_down.w.stride(0), n_experts * E, E, inner, 0, 0, 1, tile, 1.0, self._stream())
                else:
                    self.lib.call("rb_gemm_grouped_simple", _ptr(y), y.stride(0), F32, _ptr(mid), mid.stride(0), _ptr(w_down.w),
                                  w_down.w.stride(0), self.code, _ptr(tile_group), rows, E, inner, 0, self._stream())
            elif self._routed_on_tensor_cores(inner, E):
                self.lib.call("rb_gemm_tc_square_relu", launches=0)
                self.lib.call("rb_gemm_tc_grouped", _ptr(tile_group), launches=0)
                self.lib.call("rb_gemm_tc", _ptr(mid), mid.stride(0), self.code, _ptr(xp), xp.stride(0), rows, _ptr(w_up.w),
                              w_up.w.stride(0), n_experts * inner, inner, E, 0, 0, 1, tile, 1.0, self._stream())
                self.lib.call("rb_gemm_tc_grouped", _ptr(tile_group), launches=0)
                self.lib.call("rb_gemm_tc", _ptr(y), y.stride(0), F32, _ptr(mid), mid.stride(0), rows, _ptr(w_down.w),
                              w_down.w.stride(0), n_experts * E, E, inner, 0, 0, 1, tile, 1.0, self._stream())
            else:
                self.lib.call("rb_gemm_grouped_simple", _ptr(mid), mid.stride(0), self.code, _ptr(xp), xp.stride(0), _ptr(w_up.w),
                              w_up.w.stride(0), self.code, _ptr(tile_group), rows, inner, E, 1, self._stream())
                self.lib.call("rb_gemm_grouped_simple", _ptr(y), y.stride(0), F32, _ptr(mid), mid.stride(0), _ptr(w_down.w),
                              w_down.w.stride(0), self.code, _ptr(tile_group), rows, E, inner, 0, self._stream())
        else:
            pos = torch.full((pairs,), -1, dtype=torch.int32, device=self.device)
        self.lib.call("rb_routed_combine", _ptr(out), out.stride(0), _ptr(y), _ptr(h), h.stride(0), self.code, _ptr(pos),
                      _ptr(None if weight_on_input else weights), T, top, E, acc, self._stream())
        return out

    def gather_rows(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        R, E = rows.shape[0], x.shape[1]
        out = torch.empty((R, E), dtype=torch.float32, device=self.device)
        self.lib.call("rb_gather_rows", _ptr(out), _ptr(x), _ptr(rows), R, E, self._stream())
        return out

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token id per row of float32 logits (into ``out`` if given); temperature <= 0 is the arg-max."""
        self._check(logits, torch.float32, "sample logits")
        R, V = logits.shape
        if out is None:
            out = torch.empty((R,), dtype=torch.int32, device=self.device)
        stats = torch.empty((R, self.lib.raw("rb_sample_chunks")(V) * 3), dtype=torch.float32, device=self.device)
        self.lib.call("rb_sample", _ptr(out), _ptr(logits), logits.stride(0), R, V, _ptr(temperature),
                      _ptr(uniform), _ptr(stats), self._stream(), launches=2)
        return out

    def decode_advance(self, token_ids: torch.Tensor, tok_pos: torch.Tensor, sampled: torch.Tensor,
                       flag_out: Optional[torch.Tensor] = None, n_live: Optional[torch.Tensor] = None) -> None:
        """token_ids <- sampled; tok_pos += 1 (the next decode step's inputs, made on the device), for the
        first ``n_live[0]`` rows (a device int32; all rows if None).
        With ``flag_out`` (one int32) the kernels' error word is written there too, so that it comes
        back with the step's results (0: no bounded wait ran out)."""
        if self._flag_ptrs is None:
            import ctypes
            a, b = ctypes.c_void_p(0), ctypes.c_void_p(0)
            self.lib.call("rb_error_flag_addresses", ctypes.byref(a), ctypes.byref(b), launches=0)
            self._flag_ptrs = (a, b)
        a, b = self._flag_ptrs if flag_out is not None else (c_void_p(0), c_void_p(0))
        self.lib.call("rb_decode_advance", _ptr(token_ids), _ptr(tok_pos), _ptr(sampled), token_ids.shape[0],
                      _ptr(n_live), a, b, _ptr(flag_out), self._stream())
