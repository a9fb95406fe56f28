"""ctypes front end of the CUDA kernels: argument checks, output allocation, launches.

Every method checks dtype, device, contiguity and the sizes its kernel supports
and raises :class:`KernelError` with the reason; a size a kernel cannot handle
is refused, never computed wrongly.  Launches go to PyTorch's current stream,
so they order with PyTorch's own work and can be captured into CUDA graphs.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
import functools
from typing import Dict, Optional, Tuple

import torch

from .build import ALL_LIBRARIES, build_libraries, load_library
from .lazy import PendingProduct, RowScaled

_DT = {torch.float32: 0, torch.bfloat16: 1}

_STATUS = {
    -1: "unsupported dtype",
    -2: "unsupported size",
    -3: "misaligned pointer",
    -4: "needs more shared memory or scratch than available",
}


class KernelError(RuntimeError):
    pass


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current stream's handle.  Asked for at every launch, so by the short way where this
    torch has it (the Stream object costs some 15 us to build, more than the launch itself)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{what}: {_STATUS.get(rc, 'error ' + str(rc))}")
    raise KernelError(f"{what}: CUDA error {rc} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no GPU'})")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda_contig(t: torch.Tensor, name: str, dtype=None) -> None:
    _need(t.is_cuda, f"{name} must live on the GPU (there is no CPU implementation)")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    if dtype is not None:
        _need(t.dtype == dtype, f"{name} must be {dtype}, got {t.dtype}")


def _scale_args(rs: Optional[RowScaled], n_rows: int):
    """The four trailing arguments by which a kernel learns of rows whose normalisation was deferred."""
    if rs is None:
        return ctypes.c_void_p(0), 0, ctypes.c_float(0.0), ctypes.c_float(0.0)
    ssq = rs.ssq
    _need(ssq.is_cuda and ssq.dtype == torch.float32 and ssq.dim() == 2 and ssq.is_contiguous() and ssq.shape[0] >= n_rows,
          "row scale: ssq must be a contiguous float32 [rows, parts] tensor on the GPU")
    return _ptr(ssq), int(ssq.shape[1]), ctypes.c_float(1.0 / rs.dim), ctypes.c_float(rs.eps)


def _timed(fn):
    """While a profile is being taken, bracket the call with CUDA events."""
    name = fn.__name__

    @functools.wraps(fn)
    def wrapper(self, *args, **kwargs):
        prof = self._profile
        if prof is None:
            return fn(self, *args, **kwargs)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        depth, self._profile_depth = self._profile_depth, self._profile_depth + 1
        a.record()
        try:
            out = fn(self, *args, **kwargs)
        finally:
            self._profile_depth = depth
        b.record()
        prof.append((name, a, b, depth))      # depth: a call made inside another is taken off the outer one's time
        return out
    return wrapper


class NativeOps:
    """The kernels as methods.  Libraries are compiled and loaded on first use."""

    PREFILL_MIN_Q = 96      # portions at least this long go to the tcgen05 prefill attention kernel
    FUSE_MAX_ROWS = 16      # steps of at most this many tokens let a product add itself to the residual stream and
                            # prepare the norm that follows in its own kernel; with more rows product + norm
                            # kernel are as fast or faster (measured: 16 rows equal, 32 and 64 rows 2 to 7 % slower)

    name = "native-sm100a"

    def __init__(self):
        if not torch.cuda.is_available():
            raise KernelError(
                "torchllms_b200 runs on a CUDA GPU (sm_100a) only: torch.cuda.is_available() is False "
                "and there is no CPU implementation")
        self.launches = 0          # kernels of this library launched so far (a bench counts with it)
        self._workspace: Dict[Tuple[int, str], torch.Tensor] = {}
        self._retired: list = []
        self.use_tcgen05 = True
        # SwiGLU in the epilogue of the gate/up product (TORCHLLMS_B200_NO_GATED=1 keeps the two kernels, for comparisons)
        self.use_gated = os.environ.get("TORCHLLMS_B200_NO_GATED", "") not in ("1", "true")
        # error word of kernels with bounded waits: pinned host memory the device writes to directly
        self._status = torch.zeros(4, dtype=torch.int32).pin_memory()
        self._mm_out_dtype: Optional[bool] = None
        self._profile = None
        self._profile_depth = 0
        # TORCHLLMS_B200_DEBUG=1: the libraries are built with -DTL_DEBUG (see kernels/build.py); kernels
        # range-check the indices they are given and report through a word that check_status() reads
        self.debug = os.environ.get("TORCHLLMS_B200_DEBUG", "") not in ("", "0")
        # the tcgen05 prefill attention multiplies probabilities as one bfloat16 (1: the faster kernel) or as
        # bfloat16 value + bfloat16 remainder (2: a third slower, half the rounding error)
        self.prefill_probability_parts = int(os.environ.get("TORCHLLMS_B200_PREFILL_PARTS", "1"))
        self.use_fused_residual = os.environ.get("TORCHLLMS_B200_NO_FUSED_RESIDUAL", "") not in ("1", "true")
        # attention with options (kept first keys, distance bias, gate, values of their own size) in bfloat16 on the
        # tensor cores; TORCHLLMS_B200_NO_MMA_OPTIONS=1 keeps such calls on the CUDA-core kernel, for comparisons
        self.use_mma_options = os.environ.get("TORCHLLMS_B200_NO_MMA_OPTIONS", "") not in ("1", "true")

    def graph_capturable(self, dtype: torch.dtype) -> bool:
        """Whether this library's launches for ``dtype`` may be recorded into a CUDA graph (not in
        debug mode: the limits its checks compare with are copied in from the host before launches)."""
        return not self.debug

    def _debug_limit(self, lib_name: str, which: int, value: int) -> None:
        """Debug builds: tell a library how many pages (0) or rows (1) the tensors of the next launch have."""
        if self.debug:
            _check(self._lib(lib_name).tl_debug_set_limit(which, ctypes.c_longlong(int(value)), _stream()), "debug limit")

    # ------------------------------------------------------------ libraries
    def prepare(self, dtype: torch.dtype, sampling: bool = True) -> None:
        """Compile, side by side, what a model of this dtype will call."""
        names = ["elementwise", "sublayer", "rope", "attention", "gemm_simt", "recurrent", "moe", "matrix_state", "stream_sum"]
        if dtype == torch.bfloat16:
            names += ["attention_mma", "attention_decode", "gemm_tcgen05"]
        if sampling:
            names.append("sampling")
        build_libraries(names)

    def _lib(self, name: str):
        return load_library(name)

    @contextlib.contextmanager
    def profile(self):
        """Time every call made inside the block; yields a dict name -> [calls, milliseconds]
        that is filled when the block ends (the stream is synchronised then)."""
        result: Dict[str, list] = {}
        self._profile = []
        try:
            yield result
        finally:
            records, self._profile = self._profile, None
            torch.cuda.synchronize()
            inner: Dict[int, float] = {}            # time of finished calls by depth, not yet taken off their caller
            for name, a, b, depth in records:       # (a call made inside another finishes, and is listed, first)
                ms = a.elapsed_time(b)
                entry = result.setdefault(name, [0, 0.0])
                entry[0] += 1
                entry[1] += ms - inner.pop(depth + 1, 0.0)
                inner[depth] = inner.get(depth, 0.0) + ms

    # ------------------------------------------------------------- checks
    def check_attention_sizes(self, n_heads: int, n_kv_heads: int, head_dim: int, dtype: torch.dtype,
                              v_head_dim: Optional[int] = None) -> None:
        """The general kernel takes any head size up to 512 (keys and values separately); the
        tensor-core kernels take their own few sizes and are chosen only where they apply."""
        _need(dtype in _DT, f"attention supports float32 and bfloat16, not {dtype}")
        _need(n_heads > 0 and n_kv_heads > 0 and n_heads % n_kv_heads == 0,
              f"n_heads ({n_heads}) must be a positive multiple of n_kv_heads ({n_kv_heads})")
        _need(1 <= head_dim <= 512, f"head_dim must lie between 1 and 512, got {head_dim}")
        _need(v_head_dim is None or 1 <= v_head_dim <= 512, f"v_head_dim must lie between 1 and 512, got {v_head_dim}")

    # ------------------------------------------------------------ elementwise
    @_timed
    def embed(self, token_ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0,
              positions: Optional[torch.Tensor] = None, position_table: Optional[torch.Tensor] = None,
              rows_dtype: Optional[torch.dtype] = None):
        """``table[ids]`` as the float32 stream; with ``scale`` and a learned ``position_table``:
        ``table[ids] * scale + position_table[positions]``.  With ``rows_dtype`` the result is
        ``(stream, the stream in that dtype)``: a first layer that reads the stream itself gets its
        input from the same kernel (the stream itself for float32)."""
        _cuda_contig(token_ids, "token_ids", torch.int32)
        _cuda_contig(table, "embedding table")
        _need(table.dtype in _DT and table.dim() == 2, "embedding table must be a float32/bfloat16 matrix")
        n, (vocab, dim) = token_ids.numel(), table.shape
        out = torch.empty((n, dim), dtype=torch.float32, device=table.device)
        if position_table is not None or scale != 1.0 or rows_dtype is not None:
            rows = None
            if rows_dtype is not None and rows_dtype != torch.float32:
                _need(rows_dtype == torch.bfloat16, f"embed: rows dtype {rows_dtype} unsupported")
                rows = torch.empty((n, dim), dtype=rows_dtype, device=table.device)
            if position_table is not None:
                _cuda_contig(position_table, "position table", table.dtype)
                _cuda_contig(positions, "positions", torch.int32)
                _need(position_table.dim() == 2 and position_table.shape[1] == dim and positions.numel() == n,
                      "position table must be [positions, width], with one position per token")
            rc = self._lib("sublayer").tl_embed_positions(
                _ptr(token_ids), _ptr(positions if position_table is not None else None), _ptr(table), _ptr(position_table),
                _DT[table.dtype], ctypes.c_float(scale), _ptr(out), _ptr(rows), n, dim, vocab,
                0 if position_table is None else position_table.shape[0], _stream())
            _check(rc, "embed_positions")
            self.launches += 1
            if rows_dtype is not None:
                return out, (out if rows is None else rows)
            return out
        rc = self._lib("elementwise").tl_embed(_ptr(token_ids), _ptr(table), _DT[table.dtype], _ptr(out),
                                              n, dim, vocab, _stream())
        _check(rc, "embed")
        self.launches += 1
        return out

    @_timed
    def rmsnorm(self, h: torch.Tensor, delta, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, deferred: bool = False):
        """``delta`` may be a tensor, float32 partial sums ``[splits, T, dim]``, or a
        :class:`PendingProduct` (taken here the ordinary way).  ``deferred``: return the rows
        weighted but not normalised, as a :class:`RowScaled` (not with ``rows``)."""
        if isinstance(delta, PendingProduct):
            delta = delta.take(self)
        _cuda_contig(h, "residual stream", torch.float32)
        _cuda_contig(weight, "norm weight", torch.float32)
        _need(h.dim() == 2 and weight.numel() == h.shape[1], "norm weight must match the stream's width")
        _need(out_dtype in _DT, f"norm output dtype {out_dtype} unsupported")
        _need(not (deferred and rows is not None), "a deferred norm leaves whole streams, not gathered rows")
        dim = h.shape[1]
        _need(dim * 4 <= 200 * 1024, f"rmsnorm keeps a row in shared memory: width {dim} exceeds 51200")
        splits, plane = 1, 0
        if delta is not None:
            _cuda_contig(delta, "delta")
            _need(delta.dtype in _DT, "delta must be float32 or bfloat16")
            if delta.dim() == 3:          # partial sums of a split-K product, added up by the kernel
                _need(delta.shape[1:] == h.shape and delta.dtype == torch.float32,
                      "partial sums must be float32 [splits, tokens, width]")
                splits, plane = delta.shape[0], delta.stride(0)
            else:
                _need(delta.shape == h.shape, "delta must have the stream's shape")
        if rows is not None:
            _cuda_contig(rows, "rows", torch.int32)
        n_out = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n_out, dim), dtype=out_dtype, device=h.device)
        ssq = torch.empty((n_out, 1), dtype=torch.float32, device=h.device) if deferred else None
        write_back = 1 if (delta is not None and rows is None) else 0
        self._debug_limit("elementwise", 1, h.shape[0])
        rc = self._lib("elementwise").tl_rmsnorm(
            _ptr(h), _ptr(delta), _DT[delta.dtype] if delta is not None else 0, splits, ctypes.c_longlong(plane),
            _ptr(weight), _ptr(out), _DT[out_dtype], _ptr(rows), n_out, dim, ctypes.c_float(eps), write_back,
            _ptr(ssq), _stream())
        _check(rc, "rmsnorm")
        self.launches += 1
        return RowScaled(out, ssq, dim, float(eps)) if deferred else out

    @_timed
    def stream_rows(self, h: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        """The float32 stream as a sublayer's input: itself in 32-bit mode, rounded once otherwise."""
        _cuda_contig(h, "residual stream", torch.float32)
        if dtype == torch.float32:
            return h
        _need(dtype == torch.bfloat16, f"stream_rows: dtype {dtype} unsupported")
        out = torch.empty(h.shape, dtype=dtype, device=h.device)
        _check(self._lib("sublayer").tl_stream_rows(_ptr(h), _ptr(out), ctypes.c_longlong(h.numel()), _stream()), "stream_rows")
        self.launches += 1
        return out

    @_timed
    def norm_add(self, h: torch.Tensor, delta, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                 then_weight: Optional[torch.Tensor] = None, then_eps: float = 0.0) -> torch.Tensor:
        """``h += delta / sqrt(mean(delta^2) + eps) * weight`` in place (float32): the norm of a
        sublayer's output and the residual sum in one kernel.  ``delta`` is a tensor, float32
        partial sums ``[splits, T, dim]`` or a :class:`PendingProduct`.  Returns the new stream in
        ``out_dtype`` (``h`` itself for float32), or, with ``then_weight``, the RMS norm of the new
        stream under that weight and ``then_eps`` (the norm in front of the next sublayer, from
        the same kernel)."""
        bias = None
        if isinstance(delta, PendingProduct):
            # (a product's bias is added where its partial sums are added up: in this kernel)
            bias = delta.bias
            delta = self.linear(delta.x, delta.w, partials_ok=True)
        _cuda_contig(h, "residual stream", torch.float32)
        _cuda_contig(weight, "norm weight", torch.float32)
        _cuda_contig(delta, "delta")
        _need(h.dim() == 2 and weight.numel() == h.shape[1], "norm weight must match the stream's width")
        if bias is not None:
            _cuda_contig(bias, "bias of the product", torch.float32)
            _need(bias.numel() == h.shape[1], "the product's bias must match the stream's width")
        _need(delta.dtype in _DT and out_dtype in _DT, "norm_add: float32 or bfloat16")
        T, dim = h.shape
        _need(dim * 4 <= 200 * 1024, f"norm_add keeps a row in shared memory: width {dim} exceeds 51200")
        splits, plane = 1, 0
        if delta.dim() == 3:
            _need(delta.shape[1:] == h.shape and delta.dtype == torch.float32, "partial sums must be float32 [splits, tokens, width]")
            splits, plane = delta.shape[0], delta.stride(0)
        else:
            _need(delta.shape == h.shape, "delta must have the stream's shape")
        if then_weight is not None:
            _cuda_contig(then_weight, "following norm's weight", torch.float32)
            _need(then_weight.numel() == dim, "the following norm's weight must match the stream's width")
            out = torch.empty((T, dim), dtype=out_dtype, device=h.device)
            rc = self._lib("sublayer").tl_norm_add_norm(
                _ptr(h), _ptr(delta), _DT[delta.dtype], splits, ctypes.c_longlong(plane), _ptr(bias), _ptr(weight), _ptr(then_weight),
                _ptr(out), _DT[out_dtype], T, dim, ctypes.c_float(eps), ctypes.c_float(then_eps), _stream())
            _check(rc, "norm_add_norm")
            self.launches += 1
            return out
        rows = None if out_dtype == torch.float32 else torch.empty((T, dim), dtype=out_dtype, device=h.device)
        rc = self._lib("sublayer").tl_norm_add(_ptr(h), _ptr(delta), _DT[delta.dtype], splits, ctypes.c_longlong(plane), _ptr(bias),
                                              _ptr(weight), _ptr(rows), T, dim, ctypes.c_float(eps), _stream())
        _check(rc, "norm_add")
        self.launches += 1
        return h if rows is None else rows

    @_timed
    def glu(self, gate_up: torch.Tensor, out_dtype: Optional[torch.dtype] = None, *, limit: float, alpha: float,
            up_offset: float) -> torch.Tensor:
        """``g * sigmoid(alpha g) * (u + up_offset)`` with ``g = min(gate, limit)``, ``u = clamp(up, +-limit)``;
        ``gate_up`` is ``[tokens, 2 * hidden]`` or float32 partial sums of it."""
        _cuda_contig(gate_up, "gate_up")
        _need(gate_up.dim() in (2, 3) and gate_up.shape[-1] % 2 == 0 and gate_up.dtype in _DT,
              "glu input must be [tokens, 2 * hidden] in float32/bfloat16")
        splits = gate_up.shape[0] if gate_up.dim() == 3 else 1
        _need(splits == 1 or gate_up.dtype == torch.float32, "partial sums must be float32")
        out_dtype = out_dtype or gate_up.dtype
        _need(out_dtype in _DT and (out_dtype == gate_up.dtype or gate_up.dtype == torch.float32), "glu cannot widen bfloat16 input")
        n, hidden = gate_up.shape[-2], gate_up.shape[-1] // 2
        out = torch.empty((n, hidden), dtype=out_dtype, device=gate_up.device)
        rc = self._lib("sublayer").tl_glu_clamped(
            _ptr(gate_up), _DT[gate_up.dtype], splits, ctypes.c_longlong(gate_up.stride(0) if splits > 1 else 0), _ptr(out),
            _DT[out_dtype], n, hidden, ctypes.c_float(limit), ctypes.c_float(alpha), ctypes.c_float(up_offset), _stream())
        _check(rc, "glu_clamped")
        self.launches += 1
        return out

    def linear_glu(self, x: torch.Tensor, w_gate_up: torch.Tensor, *, limit: float, alpha: float, up_offset: float) -> torch.Tensor:
        """The gate/up product over the stacked weight ``[2 H, K]`` and the clamped gate, in ``x``'s dtype.
        Decode-sized bfloat16 inputs whose product needs no K split run as one kernel (the gate in the
        product's epilogue), everything else as product + gate kernel."""
        _cuda_contig(x, "linear input")
        _cuda_contig(w_gate_up, "linear weight")
        _need(x.dim() == 2 and w_gate_up.dim() == 2 and x.shape[1] == w_gate_up.shape[1] and w_gate_up.shape[0] % 2 == 0,
              "linear_glu: x [M, K] against w [2 H, K]")
        M, K = x.shape
        hidden = w_gate_up.shape[0] // 2
        if (x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and self.use_tcgen05 and self.use_gated
                and M <= 64 and hidden % 64 == 0 and K % 8 == 0 and K >= 8 and x.data_ptr() % 16 == 0
                and w_gate_up.data_ptr() % 16 == 0
                and self._lib("gemm_tcgen05").tl_gemm_tcgen05_gated_supports(M, hidden, K) == 1):
            return self.gemm_gated_clamped(x, w_gate_up, limit, alpha, up_offset)
        return self.glu(self.linear(x, w_gate_up, partials_ok=True), out_dtype=x.dtype, limit=limit, alpha=alpha,
                        up_offset=up_offset)

    @_timed
    def gemm_gated_clamped(self, x: torch.Tensor, w_gate_up: torch.Tensor, limit: float, alpha: float, up_offset: float) -> torch.Tensor:
        """The one-kernel form of :meth:`linear_glu` (its caller has checked the sizes)."""
        M, K = x.shape
        hidden = w_gate_up.shape[0] // 2
        out = torch.empty((M, hidden), dtype=torch.bfloat16, device=x.device)
        rc = self._lib("gemm_tcgen05").tl_gemm_tcgen05_gated_clamped(
            _ptr(x), _ptr(w_gate_up), _ptr(out), M, hidden, K, ctypes.c_float(limit), ctypes.c_float(alpha),
            ctypes.c_float(up_offset), ctypes.c_void_p(self._status.data_ptr()), _stream())
        _check(rc, "gemm_tcgen05_gated_clamped")
        self.launches += 1
        return out

    @_timed
    def project_and_store(self, proj: torch.Tensor, *, n_q: int, n_k: int, n_v: int, n_extra: int,
                          bias: Optional[torch.Tensor], q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                          eps: float, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                          slot_mapping: Optional[torch.Tensor], page_size: int, out_dtype: torch.dtype,
                          norm_head_dim: Optional[int] = None):
        """What follows a mixer's stacked input projection, whose rows are ``[q | k | v | extra]``
        (``proj`` is ``[T, width]`` or float32 partial sums ``[splits, T, width]``): the bias is
        added, q and k are each RMS-normed over their whole width where a weight is given, k and v
        go into their pages at ``slot_mapping`` (``k_pages`` ``[pages, kv_heads, page_size, k_dim]``,
        ``v_pages`` likewise or ``None``), and ``q`` and ``sigmoid(extra)`` come back in ``out_dtype``.
        With ``norm_head_dim`` q and k are normed head by head (heads of that size) and the weights,
        ``norm_head_dim`` numbers each, are shared by all heads."""
        _cuda_contig(proj, "projection")
        width = n_q + n_k + n_v + n_extra
        _need(proj.dim() in (2, 3) and proj.shape[-1] == width and proj.dtype in _DT, "projection rows must be [q | k | v | extra]")
        splits = proj.shape[0] if proj.dim() == 3 else 1
        _need(splits == 1 or proj.dtype == torch.float32, "partial sums must be float32")
        _need(out_dtype in _DT and (out_dtype == proj.dtype or proj.dtype == torch.float32), "project_and_store cannot widen bfloat16 input")
        _need(width * 4 <= 200 * 1024, f"project_and_store keeps a row in shared memory: {width} columns exceed 51200")
        T = proj.shape[-2]
        nh = int(norm_head_dim or 0)
        _need(nh == 0 or (n_q % nh == 0 and n_k % nh == 0), "q and k must be whole heads of norm_head_dim")
        for t, n, name in ((bias, width, "bias"), (q_norm, nh or n_q, "q_norm"), (k_norm, nh or n_k, "k_norm")):
            if t is not None:
                _cuda_contig(t, name, torch.float32)
                _need(t.numel() == n, f"{name} must have {n} elements")
        kvh = kd = vd = 0
        if k_pages is not None and n_k:
            _cuda_contig(k_pages, "k_pages", out_dtype)
            _cuda_contig(slot_mapping, "slot_mapping", torch.int32)
            _need(k_pages.dim() == 4 and k_pages.shape[2] == page_size and k_pages.shape[1] * k_pages.shape[3] == n_k,
                  "k_pages must be [pages, kv_heads, page_size, k_dim] with kv_heads * k_dim key columns")
            _need(slot_mapping.numel() == T, "one cache slot per token")
            kvh, kd = k_pages.shape[1], k_pages.shape[3]
            if v_pages is not None and n_v:
                _cuda_contig(v_pages, "v_pages", out_dtype)
                _need(v_pages.dim() == 4 and v_pages.shape[:3] == k_pages.shape[:3] and kvh * v_pages.shape[3] == n_v,
                      "v_pages must be [pages, kv_heads, page_size, v_dim] with kv_heads * v_dim value columns")
                vd = v_pages.shape[3]
            self._debug_limit("sublayer", 0, k_pages.shape[0])
        else:
            k_pages = v_pages = None
        q = torch.empty((T, n_q), dtype=out_dtype, device=proj.device)
        extra = torch.empty((T, n_extra), dtype=out_dtype, device=proj.device) if n_extra else None
        rc = self._lib("sublayer").tl_project_store(
            _ptr(proj), _DT[proj.dtype], splits, ctypes.c_longlong(proj.stride(0) if splits > 1 else 0), _ptr(bias),
            _ptr(q_norm), _ptr(k_norm), ctypes.c_float(eps), n_q, n_k, n_v, n_extra, _ptr(q), _ptr(extra), _DT[out_dtype],
            _ptr(k_pages), _ptr(v_pages), _ptr(slot_mapping if k_pages is not None else None), page_size, kvh, kd, vd, T,
            nh, _stream())
        _check(rc, "project_store")
        self.launches += 1
        return q, extra

    @_timed
    def head_linear(self, x: torch.Tensor, w: torch.Tensor, gate: Optional[torch.Tensor] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One small product per head: ``x [T, H, K]`` against ``w [H, N, K]`` gives ``[T, H, N]``,
        ``out[t, h] = w[h] @ x[t, h]``: float32 multiply-adds on the CUDA cores (a kernel of its own for
        the few rows of a decode step), except bfloat16 with more than 64 rows, which goes to the library's
        batched product.  ``x`` may be the first ``K`` coordinates of every head of wider rows, and ``out`` (given)
        the first ``N`` of every head of wider rows: views with strides ``(tokens, heads, 1)``.  ``gate``
        (``[T, H * N]``, x's dtype) multiplies the result element by element."""
        _cuda_contig(w, "head_linear weight", x.dtype)
        _need(x.is_cuda and x.dim() == 3 and w.dim() == 3 and x.shape[1] == w.shape[0] and x.shape[2] == w.shape[2] and x.dtype in _DT
              and x.stride(2) == 1, "head_linear: x [T, H, K] against w [H, N, K]")
        T, H, K = x.shape
        N = w.shape[1]
        if out is None:
            out = torch.empty((T, H, N), dtype=x.dtype, device=x.device)
        _need(out.is_cuda and out.shape == (T, H, N) and out.dtype == x.dtype and out.stride(2) == 1, "head_linear: out [T, H, N] of x's dtype")
        if gate is not None:
            _cuda_contig(gate, "head_linear gate", x.dtype)
            _need(gate.numel() == T * H * N, "head_linear: one gate value per element of the result")
        if x.dtype == torch.bfloat16 and T > 64:
            # prompt portions: the library's batched product, as linear() does for so many rows
            # (heads are the batch: inputs and result are read and written in place through their strides)
            torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
            if gate is not None:
                _need(out.is_contiguous(), "head_linear: a gated result is dense")
                _check(self._lib("sublayer").tl_gate_mul(_ptr(out), _ptr(gate), _ptr(out), _DT[x.dtype], ctypes.c_longlong(out.numel()),
                                                        _stream()), "gate_mul")
                self.launches += 1
            return out
        rc = self._lib("gemm_simt").tl_head_linear_ex(
            _ptr(x), _ptr(w), _ptr(out), _ptr(gate), _DT[x.dtype], T, H, N, K, ctypes.c_longlong(x.stride(0)),
            ctypes.c_longlong(x.stride(1)), ctypes.c_longlong(out.stride(0)), ctypes.c_longlong(out.stride(1)), _stream())
        _check(rc, "head_linear")
        self.launches += 1
        return out

    @_timed
    def latent_store(self, proj: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, *, n_q: int, n_latent: int, n_rot: int,
                     n_extra: int, q_norm: torch.Tensor, latent_norm: torch.Tensor, eps: float, interleaved: bool,
                     k_pages: torch.Tensor, slot_mapping: torch.Tensor, page_size: int, out_dtype: torch.dtype):
        """What follows the stacked input projection of a latent-attention mixer with a rotated key part, whose rows
        are ``[q latent | kv latent | key part | extra]`` (``[T, width]`` or float32 partial sums): both latents are
        RMS-normed under their weights (float32), the key part's ``n_rot`` coordinates are rotated by the position
        (``table`` float32 ``[positions, n_rot / 2, 2]``), ``[kv latent | key part]`` goes into ``k_pages`` ``[pages, 1,
        page_size, n_latent + n_rot]`` at ``slot_mapping``, and the normed q latent and ``sigmoid(extra)`` come back."""
        _cuda_contig(proj, "projection")
        _cuda_contig(positions, "positions", torch.int32)
        _cuda_contig(table, "rotary table", torch.float32)
        _cuda_contig(slot_mapping, "slot_mapping", torch.int32)
        _cuda_contig(k_pages, "k_pages", out_dtype)
        _cuda_contig(q_norm, "q_norm", torch.float32)
        _cuda_contig(latent_norm, "latent_norm", torch.float32)
        width = n_q + n_latent + n_rot + n_extra
        _need(proj.dim() in (2, 3) and proj.shape[-1] == width and proj.dtype in _DT, "projection rows must be [q latent | kv latent | key part | extra]")
        splits = proj.shape[0] if proj.dim() == 3 else 1
        _need(splits == 1 or proj.dtype == torch.float32, "partial sums must be float32")
        _need(out_dtype in _DT and (out_dtype == proj.dtype or proj.dtype == torch.float32), "latent_store cannot widen bfloat16 input")
        _need(n_rot % 2 == 0 and table.dim() == 3 and table.shape[2] == 2 and (n_rot == 0 or table.shape[1] == n_rot // 2),
              "rotary table must be [positions, n_rot / 2, 2]")
        _need(q_norm.numel() == n_q and latent_norm.numel() == n_latent, "one norm weight per latent coordinate")
        T = proj.shape[-2]
        _need(positions.numel() == T and slot_mapping.numel() == T, "one position and one cache slot per token")
        _need(k_pages.dim() == 4 and k_pages.shape[1:] == (1, page_size, n_latent + n_rot), "pages must be [pages, 1, page_size, n_latent + n_rot]")
        self._debug_limit("rope", 0, k_pages.shape[0])
        q = torch.empty((T, n_q), dtype=out_dtype, device=proj.device)
        extra = torch.empty((T, n_extra), dtype=out_dtype, device=proj.device) if n_extra else None
        rc = self._lib("rope").tl_latent_store(
            _ptr(proj), _DT[proj.dtype], splits, _ptr(positions), _ptr(table), _ptr(slot_mapping), _ptr(q_norm), _ptr(latent_norm),
            ctypes.c_float(eps), _ptr(q), _ptr(extra), _ptr(k_pages), _DT[out_dtype], T, n_q, n_latent, n_rot, n_extra, page_size,
            table.shape[0], 1 if interleaved else 0, _stream())
        _check(rc, "latent_store")
        self.launches += 1
        return q, extra

    @_timed
    def latent_query(self, q: torch.Tensor, w_uk_t: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, *, rot_dim: int,
                     interleaved: bool) -> torch.Tensor:
        """The queries of absorbed latent attention: ``q [T, H, d + rot_dim]`` and ``w_uk_t [H, rank, d]`` give
        ``[T, H, rank + rot_dim]`` = ``[w_uk_t[h] @ q[t, h, :d] | q[t, h, d:] rotated by the position]``: a per-head
        product written into the wider rows, and a rotation kernel for their tails."""
        _cuda_contig(q, "latent queries")
        _need(q.dim() == 3 and w_uk_t.dim() == 3 and q.shape[1] == w_uk_t.shape[0] and q.shape[2] == w_uk_t.shape[2] + rot_dim,
              "latent_query: q [T, H, d + rot_dim] against w_uk_t [H, rank, d]")
        T, H, qd = q.shape
        d, rank = qd - rot_dim, w_uk_t.shape[1]
        out = torch.empty((T, H, rank + rot_dim), dtype=q.dtype, device=q.device)
        self.head_linear(q[:, :, :d], w_uk_t, out=out[:, :, :rank])
        if rot_dim:
            _cuda_contig(positions, "positions", torch.int32)
            _cuda_contig(table, "rotary table", torch.float32)
            _need(rot_dim % 2 == 0 and table.dim() == 3 and table.shape[1] == rot_dim // 2 and table.shape[2] == 2 and positions.numel() == T,
                  "rotary table must be [positions, rot_dim / 2, 2], one position per token")
            rc = self._lib("rope").tl_rope_segment(
                ctypes.c_void_p(q.data_ptr() + d * q.element_size()), ctypes.c_longlong(q.stride(0)), ctypes.c_longlong(q.stride(1)),
                ctypes.c_void_p(out.data_ptr() + rank * out.element_size()), ctypes.c_longlong(out.stride(0)),
                ctypes.c_longlong(out.stride(1)), _DT[q.dtype], _ptr(positions), _ptr(table), table.shape[0], T, H, rot_dim,
                1 if interleaved else 0, _stream())
            _check(rc, "rope_segment")
            self.launches += 1
        return out

    @_timed
    def stream_inject(self, h: torch.Tensor, rows: Optional[torch.Tensor], row: Optional[torch.Tensor]) -> None:
        """``h += rows + row`` in place (float32): ``rows`` ``[T, dim]`` (another stream, e.g. the embedding output) and
        ``row`` ``[dim]`` (one vector for every token); either may be ``None``."""
        _cuda_contig(h, "residual stream", torch.float32)
        T, dim = h.shape
        if rows is not None:
            _cuda_contig(rows, "added stream", torch.float32)
            _need(rows.shape == h.shape, "the added stream must have the stream's shape")
        if row is not None:
            _cuda_contig(row, "added row", torch.float32)
            _need(row.numel() == dim, "the added row must have the stream's width")
        if rows is None and row is None:
            return
        _check(self._lib("stream_sum").tl_stream_inject(_ptr(h), _ptr(rows), _ptr(row), T, dim, _stream()), "stream_inject")
        self.launches += 1

    @_timed
    def selective_scan(self, x: torch.Tensor, dt: torch.Tensor, B: torch.Tensor, C: torch.Tensor, z: torch.Tensor, A: torch.Tensor,
                       D: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor,
                       fresh: torch.Tensor, *, n_seqs: int, max_q_len: int, out_dtype: torch.dtype) -> torch.Tensor:
        """The selective scan over every request's portion: with ``step = softplus(dt + dt_bias)`` per channel,
        ``S[c, n] <- exp(step_c A[c, n]) S[c, n] + step_c x_c B_n``, ``y_c = sum_n S[c, n] C_n + D_c x_c``, result
        ``y * silu(z)``.  ``x``, ``dt``, ``z``: ``[T, channels]``; ``B``, ``C``: ``[T, n]`` (all of one dtype; column ranges of
        wider rows will do); ``A`` float32 ``[channels, n]``, ``D`` and ``dt_bias`` float32 ``[channels]``; ``state`` float32
        ``[slots, channels, n]``: read (zeros where ``fresh``) and left as the portion's last token leaves it.  All
        arithmetic is float32."""
        ldx, lddt, ldb, ldc, ldz = (self._rows_view(t, name) for t, name in
                                    ((x, "scan input"), (dt, "step sizes"), (B, "B"), (C, "C"), (z, "scan gate")))
        T, ch = x.shape
        n = B.shape[1]
        _need(dt.shape == (T, ch) and z.shape == (T, ch) and B.shape == (T, n) and C.shape == (T, n), "selective_scan: sizes")
        _need(x.dtype == dt.dtype == B.dtype == C.dtype == z.dtype, "selective_scan: inputs of one dtype")
        _need(out_dtype in _DT and (out_dtype == x.dtype or x.dtype == torch.float32), "selective_scan cannot widen bfloat16 input")
        for t, name, shape in ((A, "A", (ch, n)), (D, "D", (ch,)), (dt_bias, "dt_bias", (ch,))):
            _cuda_contig(t, name, torch.float32)
            _need(tuple(t.shape) == shape, f"selective_scan: {name} must be {shape}")
        _need(state.dim() == 3 and state.shape[1:] == (ch, n), "state must be [slots, channels, n]")
        _need(n <= 512, f"selective_scan keeps a channel's state in registers: {n} numbers exceed 512")
        pitch = self._state_view(state, ch * n, "scan state")
        self._seq_index(q_start, state_slot, fresh, n_seqs)
        out = torch.empty((T, ch), dtype=out_dtype, device=x.device)
        rc = self._lib("selective_scan").tl_selective_scan(
            _ptr(x), ldx, _ptr(dt), lddt, _ptr(B), ldb, _ptr(C), ldc, _ptr(z), ldz, _DT[x.dtype], _ptr(A), _ptr(D), _ptr(dt_bias),
            _ptr(state), pitch, _ptr(q_start), _ptr(state_slot), _ptr(fresh), _ptr(out), _DT[out_dtype], T, n_seqs, ch, n, _stream())
        _check(rc, "selective_scan")
        self.launches += 1
        return out

    # ------------------------------------------- activations by name, depth average, map combination
    _ACTS = {"silu": 0, "gelu_tanh": 1, "relu2": 2, "clamped_swish": 3}      # (the last one: gated forms of the experts' kernels only)

    @_timed
    def depth_mix(self, history: torch.Tensor, coef: torch.Tensor, n: int, out: torch.Tensor,
                  then_weight: Optional[torch.Tensor] = None, then_eps: float = 0.0,
                  out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
        """``out = sum_j coef[j] * history[j]`` over the first ``n`` levels of ``history``
        (float32 ``[levels, T, dim]``); ``out`` (``[T, dim]``) may be a later level of it.  With
        ``then_weight`` the same kernel also returns the RMS norm of ``out`` under that weight and
        ``then_eps`` in ``out_dtype`` (the input norm of whoever reads the average next)."""
        _cuda_contig(history, "history", torch.float32)
        _cuda_contig(coef, "depth coefficients", torch.float32)
        _cuda_contig(out, "depth_mix output", torch.float32)
        _need(history.dim() == 3 and 1 <= n <= history.shape[0] and coef.numel() >= n and out.shape == history.shape[1:],
              "depth_mix: history [levels, T, dim], n coefficients, out [T, dim]")
        T, dim = out.shape
        if then_weight is not None and dim * 4 <= 48 * 1024:
            _cuda_contig(then_weight, "following norm's weight", torch.float32)
            _need(then_weight.numel() == dim and out_dtype in _DT, "the following norm's weight must match the stream's width")
            normed = torch.empty((T, dim), dtype=out_dtype, device=out.device)
            rc = self._lib("sublayer").tl_depth_mix_norm(_ptr(history), ctypes.c_longlong(history.stride(0)), _ptr(coef), int(n),
                                                        _ptr(out), _ptr(then_weight), _ptr(normed), _DT[out_dtype], T, dim,
                                                        ctypes.c_float(then_eps), _stream())
            _check(rc, "depth_mix_norm")
            self.launches += 1
            return normed
        rc = self._lib("sublayer").tl_depth_mix(_ptr(history), ctypes.c_longlong(history.stride(0)), _ptr(coef), int(n), _ptr(out),
                                               ctypes.c_longlong(out.numel()), _stream())
        _check(rc, "depth_mix")
        self.launches += 1
        if then_weight is not None:
            return self.rmsnorm(out, None, then_weight, then_eps, out_dtype=out_dtype)
        return None

    def _act(self, x: torch.Tensor, kind: str, out_dtype: Optional[torch.dtype], gated: bool) -> torch.Tensor:
        _need(kind in self._ACTS, f"unknown activation {kind!r}; known: {', '.join(self._ACTS)}")
        _cuda_contig(x, "activation input")
        _need(x.dim() in (2, 3) and x.dtype in _DT and (not gated or x.shape[-1] % 2 == 0),
              "activation input must be [tokens, width] (gated: [tokens, 2 * hidden]) in float32/bfloat16")
        splits = x.shape[0] if x.dim() == 3 else 1
        _need(splits == 1 or x.dtype == torch.float32, "partial sums must be float32")
        out_dtype = out_dtype or x.dtype
        _need(out_dtype in _DT and (out_dtype == x.dtype or x.dtype == torch.float32), "an activation cannot widen bfloat16 input")
        n, hidden = x.shape[-2], x.shape[-1] // (2 if gated else 1)
        out = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
        rc = self._lib("sublayer").tl_act(_ptr(x), _DT[x.dtype], splits, ctypes.c_longlong(x.stride(0) if splits > 1 else 0),
                                         _ptr(out), _DT[out_dtype], n, hidden, self._ACTS[kind], 1 if gated else 0, _stream())
        _check(rc, "activation")
        self.launches += 1
        return out

    @_timed
    def activation(self, x: torch.Tensor, kind: str, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``act(x)`` by name (``silu``, ``gelu_tanh``, ``relu2``: the square of relu), float32 arithmetic;
        ``x`` is ``[tokens, width]`` or float32 partial sums of it."""
        return self._act(x, kind, out_dtype, False)

    @_timed
    def gated_act(self, gate_up: torch.Tensor, activation: str, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``act(gate) * up`` for rows ``[gate | up]`` (or float32 partial sums of them)."""
        return self._act(gate_up, activation, out_dtype, True)

    def linear_gated_act(self, x: torch.Tensor, w_gate_up: torch.Tensor, *, activation: str) -> torch.Tensor:
        """The gate/up product over the stacked weight ``[2 H, K]`` and ``act(gate) * up``, in ``x``'s dtype.
        Decode-sized bfloat16 inputs whose product needs no K split run as one kernel (the gate in the
        product's epilogue, as :meth:`linear_swiglu` does), everything else as product + gate kernel."""
        if activation == "silu":
            return self.linear_swiglu(x, w_gate_up)
        _cuda_contig(x, "linear input")
        _cuda_contig(w_gate_up, "linear weight")
        _need(x.dim() == 2 and w_gate_up.dim() == 2 and x.shape[1] == w_gate_up.shape[1] and w_gate_up.shape[0] % 2 == 0,
              "linear_gated_act: x [M, K] against w [2 H, K]")
        M, K = x.shape
        hidden = w_gate_up.shape[0] // 2
        if (activation == "gelu_tanh" and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and self.use_tcgen05
                and self.use_gated and M <= 64 and hidden % 64 == 0 and K % 8 == 0 and K >= 8 and x.data_ptr() % 16 == 0
                and w_gate_up.data_ptr() % 16 == 0
                and self._lib("gemm_tcgen05").tl_gemm_tcgen05_gated_supports(M, hidden, K) == 1):
            return self.gemm_gated_gelu(x, w_gate_up)
        return self.gated_act(self.linear(x, w_gate_up, partials_ok=True), activation, out_dtype=x.dtype)

    @_timed
    def gemm_gated_gelu(self, x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
        """The one-kernel form of :meth:`linear_gated_act` for ``gelu_tanh`` (its caller has checked the sizes)."""
        M, K = x.shape
        hidden = w_gate_up.shape[0] // 2
        out = torch.empty((M, hidden), dtype=torch.bfloat16, device=x.device)
        rc = self._lib("gemm_tcgen05").tl_gemm_tcgen05_gated_gelu(_ptr(x), _ptr(w_gate_up), _ptr(out), M, hidden, K,
                                                                 ctypes.c_void_p(self._status.data_ptr()), _stream())
        _check(rc, "gemm_tcgen05_gated_gelu")
        self.launches += 1
        return out

    @_timed
    def differential_combine(self, maps: torch.Tensor, lam: float, *, eps: float, out_scale: float,
                             gate: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
        """Two attention maps over the same values into one result: ``maps`` is float32 ``[T, 2 H, dv]``
        with all first maps before all second maps; per (token, head) ``o = a1 - lam * a2``, then
        ``o / sqrt(mean(o^2) + eps) * out_scale * gate[t, h]``.  Returns ``[T, H * dv]``."""
        _cuda_contig(maps, "attention maps", torch.float32)
        _need(maps.dim() == 3 and maps.shape[1] % 2 == 0 and out_dtype in _DT, "maps must be float32 [tokens, 2 * heads, dv]")
        T, H, dv = maps.shape[0], maps.shape[1] // 2, maps.shape[2]
        if gate is not None:
            _cuda_contig(gate, "gate", out_dtype)
            _need(gate.shape == (T, H), "gate must be [tokens, heads]")
        out = torch.empty((T, H * dv), dtype=out_dtype, device=maps.device)
        rc = self._lib("sublayer").tl_differential_combine(_ptr(maps), _ptr(gate), _ptr(out), _DT[out_dtype], T, H, dv,
                                                          ctypes.c_float(lam), ctypes.c_float(eps), ctypes.c_float(out_scale),
                                                          _stream())
        _check(rc, "differential_combine")
        self.launches += 1
        return out

    @_timed
    def rope_store(self, proj: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, *, n_q_heads: int, n_k_heads: int,
                   n_v_heads: int, head_dim: int, v_head_dim: int, rot_dims: int, interleaved: bool, n_extra: int,
                   k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                   page_size: int, out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None):
        """What follows a stacked projection ``[q heads | k heads | v heads | extra]`` (``[T, width]`` or
        float32 partial sums): the first ``rot_dims`` coordinates of every q and k head are rotated by
        the position's angles (``table`` float32 ``[positions, rot_dims / 2, 2]``), k goes to
        ``k_pages`` ``[pages, n_k_heads, page_size, head_dim]`` and v to ``v_pages`` ``[pages,
        n_v_heads, page_size, v_head_dim]`` at ``slot_mapping``, and ``q [T, n_q_heads, head_dim]`` and
        ``sigmoid(extra)`` come back in ``out_dtype``.  ``n_k_heads = n_v_heads = 0``: a run that reads
        another run's cache."""
        _cuda_contig(proj, "projection")
        _cuda_contig(positions, "positions", torch.int32)
        _cuda_contig(table, "rotary table", torch.float32)
        width = (n_q_heads + n_k_heads) * head_dim + n_v_heads * v_head_dim + n_extra
        _need(proj.dim() in (2, 3) and proj.shape[-1] == width and proj.dtype in _DT, "projection rows must be [q | k | v | extra]")
        splits = proj.shape[0] if proj.dim() == 3 else 1
        _need(splits == 1 or proj.dtype == torch.float32, "partial sums must be float32")
        _need(out_dtype in _DT and (out_dtype == proj.dtype or proj.dtype == torch.float32), "rope_store cannot widen bfloat16 input")
        _need(0 <= rot_dims <= head_dim and rot_dims % 2 == 0, "rot_dims must be even and at most head_dim")
        _need(table.dim() == 3 and table.shape[2] == 2 and (rot_dims == 0 or table.shape[1] == rot_dims // 2),
              "rotary table must be [positions, rot_dims / 2, 2]")
        T = proj.shape[-2]
        _need(positions.numel() == T, "one position per token")
        if bias is not None:          # float32 [width], added to the row before anything else
            _cuda_contig(bias, "bias", torch.float32)
            _need(bias.numel() == width, "one bias per column of the projection")
        if n_k_heads:
            _cuda_contig(k_pages, "k_pages", out_dtype)
            _cuda_contig(v_pages, "v_pages", out_dtype)
            _cuda_contig(slot_mapping, "slot_mapping", torch.int32)
            _need(k_pages.shape[1:] == (n_k_heads, page_size, head_dim) and v_pages.shape[1:] == (n_v_heads, page_size, v_head_dim)
                  and v_pages.shape[0] == k_pages.shape[0], "pages must be [pages, heads, page_size, size] for keys and for values")
            _need(slot_mapping.numel() == T, "one cache slot per token")
            self._debug_limit("rope", 0, k_pages.shape[0])
        else:
            _need(n_v_heads == 0, "values are stored with keys")
            k_pages = v_pages = None
        q = torch.empty((T, n_q_heads, head_dim), dtype=out_dtype, device=proj.device)
        extra = torch.empty((T, n_extra), dtype=out_dtype, device=proj.device) if n_extra else None
        rc = self._lib("rope").tl_rope_store(
            _ptr(proj), _DT[proj.dtype], splits, _ptr(bias), _ptr(positions), _ptr(table), _ptr(slot_mapping if k_pages is not None else None),
            _ptr(q), _ptr(extra), _ptr(k_pages), _ptr(v_pages), _DT[out_dtype], T, n_q_heads, n_k_heads, n_v_heads, head_dim,
            v_head_dim, rot_dims, n_extra, page_size, table.shape[0], 1 if interleaved else 0, _stream())
        _check(rc, "rope_store")
        self.launches += 1
        return q, extra

    # -------------------------------------------------------------- recurrence
    @_timed
    def mingru_scan(self, proj: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, q_start: torch.Tensor,
                    state_slot: torch.Tensor, fresh: torch.Tensor, *, n_seqs: int, max_q_len: int,
                    out_dtype: torch.dtype) -> torch.Tensor:
        """The minGRU recurrence over every request's portion.  ``proj`` is ``[T, 3 W]`` = ``[z | u | g]``
        (or float32 partial sums), ``bias`` float32 ``[3 W]``; with ``a = sigmoid(z)`` and ``c = u + 1/2``
        for ``u >= 0``, ``sigmoid(u)`` elsewhere: ``S <- (1 - a) S + a c`` and ``out = S * silu(g)``.
        ``state`` (float32 ``[slots, W]``) holds every request's ``S`` at row ``state_slot[b]``: read
        (as zero where ``fresh[b]``) and left as the portion's last token leaves it."""
        _cuda_contig(proj, "projection")
        _cuda_contig(state, "state", torch.float32)
        for t, name in ((q_start, "q_start"), (state_slot, "state_slot"), (fresh, "fresh")):
            _cuda_contig(t, name, torch.int32)
        _need(proj.dim() in (2, 3) and proj.shape[-1] % 3 == 0 and proj.dtype in _DT, "projection rows must be [z | u | g]")
        splits = proj.shape[0] if proj.dim() == 3 else 1
        _need(splits == 1 or proj.dtype == torch.float32, "partial sums must be float32")
        _need(out_dtype in _DT and (out_dtype == proj.dtype or proj.dtype == torch.float32), "mingru_scan cannot widen bfloat16 input")
        T, W = proj.shape[-2], proj.shape[-1] // 3
        _need(state.dim() == 2 and state.shape[1] == W, "state must be [slots, width]")
        _need(q_start.numel() >= n_seqs + 1 and state_slot.numel() >= n_seqs and fresh.numel() >= n_seqs,
              "q_start, state_slot and fresh must cover every request of the step")
        if bias is not None:
            _cuda_contig(bias, "bias", torch.float32)
            _need(bias.numel() == 3 * W, "bias must have 3 * width elements")
        lib = self._lib("recurrent")
        lib.tl_mingru_scan_scratch.restype = ctypes.c_longlong
        ws = self._scratch(proj.device, lib.tl_mingru_scan_scratch(n_seqs, W, max_q_len), "recurrent")
        out = torch.empty((T, W), dtype=out_dtype, device=proj.device)
        rc = lib.tl_mingru_scan(_ptr(proj), _DT[proj.dtype], splits, ctypes.c_longlong(proj.stride(0) if splits > 1 else 0),
                                _ptr(bias), _ptr(state), _ptr(q_start), _ptr(state_slot), _ptr(fresh), _ptr(out), _DT[out_dtype],
                                T, n_seqs, W, max_q_len, _ptr(ws), _stream())
        _check(rc, "mingru_scan")
        self.launches += 3 if max_q_len > 8 else 1
        return out

    # ------------------------------------------------- matrix states, short convolutions, sums of sublayers
    @staticmethod
    def _rows_view(t: torch.Tensor, name: str):
        """A ``[T, n]`` tensor whose rows may be a column range of a wider row: the pitch in elements."""
        _need(t.is_cuda and t.dim() == 2 and t.dtype in _DT and (t.shape[1] == 0 or t.stride(1) == 1),
              f"{name} must be [tokens, columns] on the GPU with columns side by side, float32 or bfloat16")
        return ctypes.c_longlong(t.stride(0))

    @staticmethod
    def _state_view(state: torch.Tensor, inner: int, name: str):
        """Per-request state ``[slots, ...]`` that may be a field of a wider row: the slots' pitch in elements."""
        _need(state.is_cuda and state.dtype == torch.float32 and state[0].is_contiguous() and state[0].numel() == inner,
              f"{name} must be float32 [slots, ...] on the GPU, every slot's part contiguous")
        return ctypes.c_longlong(state.stride(0))

    def _seq_index(self, q_start, state_slot, fresh, n_seqs):
        for t, name in ((q_start, "q_start"), (state_slot, "state_slot"), (fresh, "fresh")):
            _cuda_contig(t, name, torch.int32)
        _need(q_start.numel() >= n_seqs + 1 and state_slot.numel() >= n_seqs and fresh.numel() >= n_seqs,
              "q_start, state_slot and fresh must cover every request of the step")

    @_timed
    def short_conv(self, x: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor], q_start: torch.Tensor,
                   state_slot: torch.Tensor, fresh: torch.Tensor, *, n_seqs: int, max_q_len: int, activation: Optional[str],
                   residual: bool, out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Causal convolution over time on every channel: ``out_t = sum_j w[:, j] x_(t - taps + 1 + j)`` (plus ``x_t``
        with ``residual``), then ``silu`` if asked for.  ``x`` is ``[T, C]`` (a column range of a wider row will do),
        ``w`` float32 ``[C, taps]``; ``state`` (float32 ``[slots, taps - 1, C]``, ``None`` with one tap) holds every
        request's last inputs: read (zeros where ``fresh``) and left as the portion leaves them."""
        ldx = self._rows_view(x, "convolution input")
        _cuda_contig(w, "convolution taps", torch.float32)
        C, taps = w.shape
        _need(x.shape[1] == C and 1 <= taps <= 8, "short_conv: x [T, C] against w [C, taps], at most 8 taps")
        _need(activation in (None, "silu"), f"short_conv knows no activation {activation!r}")
        if bias is not None:          # float32 [C], added to the sum before the activation
            _cuda_contig(bias, "convolution bias", torch.float32)
            _need(bias.numel() == C, "one bias per channel")
        _need(out_dtype in _DT and (out_dtype == x.dtype or x.dtype == torch.float32), "short_conv cannot widen bfloat16 input")
        self._seq_index(q_start, state_slot, fresh, n_seqs)
        pitch = ctypes.c_longlong(0)
        if taps > 1:
            _need(state is not None, "a convolution of several taps keeps state")
            pitch = self._state_view(state, (taps - 1) * C, "convolution state")
        T = x.shape[0]
        out = torch.empty((T, C), dtype=out_dtype, device=x.device)
        rc = self._lib("matrix_state").tl_short_conv(
            _ptr(x), _DT[x.dtype], ldx, _ptr(w), _ptr(bias), _ptr(state if taps > 1 else None), pitch, _ptr(q_start), _ptr(state_slot),
            _ptr(fresh), _ptr(out), _DT[out_dtype], T, n_seqs, C, taps, max_q_len, 1 if activation == "silu" else 0,
            1 if residual else 0, _stream())
        _check(rc, "short_conv")
        self.launches += 2 if (max_q_len > 8 and taps > 1) else 1
        return out

    @_timed
    def recurrence_prep(self, x: torch.Tensor, *, scale: float, n_heads: int, head_dim: int,
                        positions: Optional[torch.Tensor] = None, table: Optional[torch.Tensor] = None, rot_dims: int = 0,
                        unit_eps: Optional[float] = None) -> torch.Tensor:
        """q or k on their way into a recurrence, as float32 ``[T, n_heads * head_dim]``: with ``unit_eps`` every head
        becomes ``x / sqrt(sum(x^2) + unit_eps)``; with ``table`` (``[positions, rot_dims / 2, 2]`` of cos and sin) the
        first ``rot_dims`` coordinates of every head turn by the token's position, coordinate ``i`` paired with
        ``i + rot_dims / 2``.  The result is multiplied by ``scale``."""
        ldx = self._rows_view(x, "recurrence input")
        _need(x.shape[1] == n_heads * head_dim, "recurrence_prep: x [T, n_heads * head_dim]")
        unit = unit_eps is not None
        rows = 0
        if not unit and rot_dims:
            _cuda_contig(table, "rotation table", torch.float32)
            _cuda_contig(positions, "positions", torch.int32)
            _need(table.dim() == 3 and table.shape[1] == rot_dims // 2 and table.shape[2] == 2 and positions.numel() == x.shape[0],
                  "rotation table must be [positions, rot_dims / 2, 2], one position per token")
            rows = table.shape[0]
        else:
            table = positions = None
            rot_dims = 0
        out = torch.empty((x.shape[0], n_heads * head_dim), dtype=torch.float32, device=x.device)
        rc = self._lib("matrix_state").tl_recurrence_prep(
            _ptr(x), _DT[x.dtype], ldx, _ptr(out), _ptr(positions), _ptr(table), rows, x.shape[0], n_heads, head_dim, rot_dims,
            1 if unit else 0, ctypes.c_float(unit_eps or 0.0), ctypes.c_float(scale), _stream())
        _check(rc, "recurrence_prep")
        self.launches += 1
        return out

    @_timed
    def linear_recurrence(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor,
                          state_slot: torch.Tensor, fresh: torch.Tensor, *, n_seqs: int, max_q_len: int,
                          decay: Optional[torch.Tensor] = None, beta_logits: Optional[torch.Tensor] = None,
                          decay_logits: Optional[torch.Tensor] = None, decay_rate: Optional[torch.Tensor] = None,
                          decay_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """A matrix ``S`` (``dk x dv``, float32) per head and request that every token updates and then reads,
        ``o = S^T q``.  With ``decay`` (float32 ``[H]``): ``S <- decay_h S + k v^T``.  Otherwise the gated delta rule:
        ``S <- g S; u = beta (v - S^T k); S <- S + k u^T`` with ``beta = sigmoid(beta_logits)`` and
        ``g = exp(-decay_rate softplus(decay_logits + decay_bias))`` (logits ``[T, H]``, the rest float32 ``[H]``).
        ``q``, ``k``: float32 ``[T, G * dk]``, ``G`` heads each shared by ``H / G`` value heads; ``v``: ``[T, H * dv]``;
        ``state``: ``[slots, H, dv, dk]`` (a head's matrix with a column's keys side by side), read (zeros where
        ``fresh``) and left updated.  Returns float32 ``[T, H * dv]``."""
        _cuda_contig(q, "q", torch.float32)
        _cuda_contig(k, "k", torch.float32)
        ldv = self._rows_view(v, "v")
        _need(state.dim() == 4, "state must be [slots, heads, dv, dk]")
        H, dv, dk = state.shape[1:]
        pitch = self._state_view(state, H * dk * dv, "recurrence state")
        T = q.shape[0]
        _need(q.dim() == 2 and q.shape == k.shape and q.shape[1] % dk == 0 and v.shape == (T, H * dv), "linear_recurrence: sizes")
        G = q.shape[1] // dk
        _need(G > 0 and H % G == 0, f"{H} value heads cannot share {G} heads of q and k")
        _need(dk <= 256, f"linear_recurrence keeps a head's state in registers: key size {dk} exceeds 256")
        self._seq_index(q_start, state_slot, fresh, n_seqs)
        delta = decay is None
        ldg = ctypes.c_longlong(0)
        if delta:
            for t, name in ((decay_rate, "decay_rate"), (decay_bias, "decay_bias")):
                _cuda_contig(t, name, torch.float32)
                _need(t.numel() == H, f"{name}: one number per head")
            ldg = self._rows_view(beta_logits, "beta_logits")
            _need(self._rows_view(decay_logits, "decay_logits").value == ldg.value and beta_logits.shape == (T, H)
                  and decay_logits.shape == (T, H) and beta_logits.dtype == v.dtype and decay_logits.dtype == v.dtype,
                  "beta_logits and decay_logits must be [T, H] of v's dtype with one row pitch")
        else:
            _cuda_contig(decay, "decay", torch.float32)
            _need(decay.numel() == H, "decay: one number per head")
        out = torch.empty((T, H * dv), dtype=torch.float32, device=q.device)
        rc = self._lib("matrix_state").tl_linear_recurrence(
            _ptr(q), _ptr(k), _ptr(v), _DT[v.dtype], ldv, _ptr(beta_logits), _ptr(decay_logits), ldg,
            _ptr(decay_rate if delta else decay), _ptr(decay_bias), _ptr(state), pitch, _ptr(q_start), _ptr(state_slot), _ptr(fresh),
            _ptr(out), T, n_seqs, H, G, dk, dv, 1 if delta else 0, _stream())
        _check(rc, "linear_recurrence")
        self.launches += 1
        return out

    @_timed
    def head_norm_gate(self, o: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor], eps: float, *, head_dim: int,
                       out_dtype: torch.dtype) -> torch.Tensor:
        """Every head (``head_dim`` numbers) of ``o`` (float32 ``[T, H * head_dim]``) divided by its root mean square,
        times ``weight`` (float32 ``[head_dim]``, shared by the heads; ``None``: no weight), times ``silu(gate)``."""
        _cuda_contig(o, "recurrence output", torch.float32)
        ldg = self._rows_view(gate, "gate")
        _need(o.dim() == 2 and o.shape[1] % head_dim == 0 and gate.shape == o.shape, "head_norm_gate: o and gate [T, H * head_dim]")
        _need(out_dtype in _DT and (out_dtype == gate.dtype or gate.dtype == torch.float32), "head_norm_gate cannot widen a bfloat16 gate")
        if weight is not None:
            _cuda_contig(weight, "head norm weight", torch.float32)
            _need(weight.numel() == head_dim, "the head norm's weight has head_dim numbers")
        out = torch.empty(o.shape, dtype=out_dtype, device=o.device)
        rc = self._lib("matrix_state").tl_head_norm_gate(_ptr(o), _ptr(gate), _DT[gate.dtype], ldg, _ptr(weight), _ptr(out), _DT[out_dtype],
                                                        o.shape[0], o.shape[1] // head_dim, head_dim, ctypes.c_float(eps), _stream())
        _check(rc, "head_norm_gate")
        self.launches += 1
        return out

    @_timed
    def stream_add(self, h: torch.Tensor, *, normed, coef: float, eps: float, plain, out_dtype: torch.dtype) -> torch.Tensor:
        """``h += coef * sum_i t_i / sqrt(mean(t_i^2) + eps) * w_i + sum_j p_j`` in place (float32), one kernel:
        ``normed`` is up to two ``(t_i, w_i)`` (``[T, dim]``, float32 ``[dim]``), ``plain`` up to three ``[T, dim]``
        tensors; any of them may be float32 partial sums ``[splits, T, dim]`` of a split-K product.  Returns the new stream in ``out_dtype`` (``h`` itself for float32)."""
        _cuda_contig(h, "residual stream", torch.float32)
        _need(h.dim() == 2 and len(normed) <= 2 and len(plain) <= 3, "stream_add: at most two normed and three plain terms")
        _need(out_dtype in _DT, f"stream_add: output dtype {out_dtype} unsupported")
        def term(t, name):
            """(plane count, planes' distance): a term is [T, dim] or float32 partial sums [splits, T, dim]"""
            _cuda_contig(t, name)
            _need(t.dtype in _DT and t.shape[-2:] == h.shape and (t.dim() == 2 or (t.dim() == 3 and t.dtype == torch.float32)),
                  f"a {name} has the stream's shape, or is float32 partial sums of it")
            return (t.shape[0], t.stride(0)) if t.dim() == 3 else (1, 0)
        for _t, w in normed:
            _cuda_contig(w, "norm weight", torch.float32)
            _need(w.numel() == h.shape[1], "a norm weight has the stream's width")
        n, m = len(normed), len(plain)
        n_how = [term(t, "normed term") for t, _w in normed]
        p_how = [term(t, "plain term") for t in plain]
        np_ = (ctypes.c_void_p * 2)(*[t.data_ptr() for t, _w in normed])
        nd = (ctypes.c_int * 2)(*[_DT[t.dtype] for t, _w in normed])
        ns = (ctypes.c_int * 2)(*[a for a, _b in n_how])
        npl = (ctypes.c_longlong * 2)(*[b for _a, b in n_how])
        nw = (ctypes.c_void_p * 2)(*[w.data_ptr() for _t, w in normed])
        pp = (ctypes.c_void_p * 3)(*[t.data_ptr() for t in plain])
        pd = (ctypes.c_int * 3)(*[_DT[t.dtype] for t in plain])
        ps = (ctypes.c_int * 3)(*[a for a, _b in p_how])
        ppl = (ctypes.c_longlong * 3)(*[b for _a, b in p_how])
        rows = None if out_dtype == torch.float32 else torch.empty(h.shape, dtype=out_dtype, device=h.device)
        rc = self._lib("stream_sum").tl_stream_add(_ptr(h), np_, nd, ns, npl, nw, n, pp, pd, ps, ppl, m, ctypes.c_float(coef), ctypes.c_float(eps),
                                                  _ptr(rows), h.shape[0], h.shape[1], _stream())
        _check(rc, "stream_add")
        self.launches += 1
        return h if rows is None else rows

    @_timed
    def sum_partials(self, parts: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """Float32 partial sums ``[splits, ...]`` of a split-K product added up and rounded once, for readers that take
        no partial sums."""
        _cuda_contig(parts, "partial sums", torch.float32)
        _need(parts.dim() >= 2 and out_dtype in _DT, "sum_partials: [splits, ...] float32 to float32 or bfloat16")
        out = torch.empty(parts.shape[1:], dtype=out_dtype, device=parts.device)
        rc = self._lib("stream_sum").tl_sum_partials(_ptr(parts), parts.shape[0], ctypes.c_longlong(parts.stride(0)), _ptr(out),
                                                    _DT[out_dtype], ctypes.c_longlong(out.numel()), _stream())
        _check(rc, "sum_partials")
        self.launches += 1
        return out

    @_timed
    def polynorm(self, z: torch.Tensor, coef: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
        """``a N(z) + b N(z^2) + c N(z^3) + e`` over every row, ``N(y) = y / sqrt(mean(y^2) + eps)``, powers element by
        element; ``coef`` is float32 ``(a, b, c, e)``."""
        _cuda_contig(z, "polynorm input")
        _cuda_contig(coef, "polynorm coefficients", torch.float32)
        _need(z.dim() in (2, 3) and z.dtype in _DT and coef.numel() == 4, "polynorm: z [T, width] or partial sums of it, four coefficients")
        splits = z.shape[0] if z.dim() == 3 else 1
        _need(splits == 1 or z.dtype == torch.float32, "partial sums must be float32")
        _need(out_dtype in _DT and (out_dtype == z.dtype or z.dtype == torch.float32), "polynorm cannot widen bfloat16 input")
        out = torch.empty(z.shape[-2:], dtype=out_dtype, device=z.device)
        rc = self._lib("stream_sum").tl_polynorm(_ptr(z), _DT[z.dtype], splits, ctypes.c_longlong(z.stride(0) if splits > 1 else 0),
                                                _ptr(coef), _ptr(out), _DT[out_dtype], z.shape[-2], z.shape[-1], ctypes.c_float(eps),
                                                _stream())
        _check(rc, "polynorm")
        self.launches += 1
        return out

    @_timed
    def side_gate(self, u: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """``gelu_tanh(u) * table[token]``: ``u`` ``[T, s]`` (or float32 partial sums ``[splits, T, s]``), ``table``
        ``[vocab, s]`` of ``out_dtype``."""
        _cuda_contig(u, "side gate input")
        _cuda_contig(table, "side table", out_dtype)
        _cuda_contig(token_ids, "token ids", torch.int32)
        splits = u.shape[0] if u.dim() == 3 else 1
        _need(out_dtype in _DT and u.dim() in (2, 3) and table.dim() == 2 and table.shape[1] == u.shape[-1]
              and token_ids.numel() == u.shape[-2], "side_gate: u [T, s], table [vocab, s], one token per row")
        _need(u.dtype == torch.float32 or (u.dtype == out_dtype and splits == 1), "side_gate: u of the output's dtype, or float32")
        out = torch.empty(u.shape[-2:], dtype=out_dtype, device=u.device)
        rc = self._lib("stream_sum").tl_side_gate(_ptr(u), _DT[u.dtype], splits, ctypes.c_longlong(u.stride(0) if splits > 1 else 0),
                                                 _ptr(token_ids), _ptr(table), _ptr(out), _DT[out_dtype], u.shape[-2], u.shape[-1],
                                                 table.shape[0], _stream())
        _check(rc, "side_gate")
        self.launches += 1
        return out

    # ----------------------------------------------------------------- experts
    @_timed
    def moe_route(self, x: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], *, n_experts: int,
                  top: int, scale: float, renormalize: bool, shared_gate: bool, logit_bias: Optional[torch.Tensor] = None,
                  score: str = "softmax", n_groups: int = 1, keep_groups: int = 1, group_score_top: int = 2,
                  renorm_eps: float = 0.0):
        """Router of a layer of experts: ``s = softmax(w_router[:E] x)`` in float32, the ``top`` experts
        with the largest ``s + correction`` chosen, weights ``s * scale`` (over their sum with
        ``renormalize``); with ``shared_gate`` the row ``w_router[E]`` gives ``sigmoid(.)`` per token.  ``logit_bias``
        (float32 ``[E]``) is added to the logits first.  (With ``renormalize`` and a scale of one the weights are
        the softmax over the chosen logits alone.)  ``score="sigmoid"``: ``s = sigmoid(z)``, each expert by itself.
        ``n_groups > 1``: the experts form so many equal groups of neighbours, a group's score is the sum of its
        ``group_score_top`` largest ``s + correction``, and only experts of the ``keep_groups`` best groups can be chosen.
        ``renorm_eps`` is added to the sum that ``renormalize`` divides by.
        Returns ``(chosen int32 [T, top], weights float32 [T, top], gate float32 [T] or None)``."""
        _cuda_contig(x, "router input")
        _cuda_contig(w_router, "router weight", torch.float32)
        _need(score in ("softmax", "sigmoid"), f"a router's scores are 'softmax' or 'sigmoid', got {score!r}")
        _need(n_groups >= 1 and n_experts % n_groups == 0 and 0 < keep_groups <= n_groups and group_score_top >= 1
              and keep_groups * (n_experts // n_groups) >= top, "the kept groups must hold at least `top` experts")
        _need(x.dim() == 2 and x.dtype in _DT and w_router.dim() == 2 and w_router.shape[1] == x.shape[1]
              and w_router.shape[0] == n_experts + (1 if shared_gate else 0), "router: x [T, dim] against w [E (+ 1), dim]")
        if correction is not None:
            _cuda_contig(correction, "correction", torch.float32)
            _need(correction.numel() == n_experts, "one correction per expert")
        if logit_bias is not None:
            _cuda_contig(logit_bias, "logit_bias", torch.float32)
            _need(logit_bias.numel() == n_experts, "one logit bias per expert")
        T, dim = x.shape
        rows = w_router.shape[0]
        lib = self._lib("moe")
        if T <= 64:
            # few tokens: a warp per (token, router row)
            logits = torch.empty((T, rows), dtype=torch.float32, device=x.device)
            _check(lib.tl_moe_logits(_ptr(x), _DT[x.dtype], _ptr(w_router), _ptr(logits), T, dim, rows, _stream()), "moe_logits")
            self.launches += 1
        elif x.dtype == torch.float32:
            logits = self.gemm_simt(x, w_router, torch.float32)
        elif torch.backends.cuda.matmul.allow_tf32:
            # many tokens, and the library's float32 product would not be one: this library's own
            logits = self.gemm_simt(x.float(), w_router, torch.float32)
        else:
            # many tokens: the library's float32 product of the rows as the rounded stream holds them (true
            # 32-bit arithmetic: the reduced-precision matrix mode is off), as linear() takes the library for so many rows
            logits = torch.mm(x.float(), w_router.t())
        chosen = torch.empty((T, top), dtype=torch.int32, device=x.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=x.device)
        gate = torch.empty((T,), dtype=torch.float32, device=x.device) if shared_gate else None
        rc = lib.tl_moe_select(_ptr(logits), _ptr(correction), _ptr(logit_bias), _ptr(chosen), _ptr(weights), _ptr(gate), T, n_experts, top,
                               ctypes.c_float(scale), 1 if renormalize else 0, 1 if score == "sigmoid" else 0, n_groups, keep_groups,
                               group_score_top, ctypes.c_float(renorm_eps), _stream())
        _check(rc, "moe_select")
        self.launches += 1
        return chosen, weights, gate

    GROUPED_MIN_PAIRS = 257      # (token, choice) pairs from which the experts' products of bfloat16 go to the library

    @_timed
    def moe_experts(self, x: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor, w_up: torch.Tensor,
                    w_down: torch.Tensor, *, activation: str, shared: Optional[torch.Tensor] = None,
                    shared_gate: Optional[torch.Tensor] = None, gated: bool = False, act_params=None) -> torch.Tensor:
        """``out[t] = sum_k weights[t, k] * down_e(act(up_e x[t]))`` with ``e = chosen[t, k]``, plus
        ``shared[t]`` (``[T, dim]`` or float32 partial sums) times ``shared_gate[t]`` where given.
        With ``gated`` an expert is ``down_e(act(gate_e x) * up_e x)`` and ``w_up`` is ``[E, 2 * hidden, dim]``, an expert's
        rows being ``[gate; up]``; ``activation="clamped_swish"`` (gated only) with ``act_params = (limit, alpha, up_offset)``
        is ``g * sigmoid(alpha g) * (u + up_offset)``, ``g = min(gate, limit)``, ``u = clamp(up, +-limit)``.
        ``w_up`` is ``[E, hidden, dim]``; ``w_down`` is ``[dim, >= E * hidden]``, expert ``e``'s matrix being
        the columns ``e * hidden .. (e + 1) * hidden`` (the layout in which all experts are one
        matrix too).  The (token, choice) pairs are sorted by expert on the device and both products
        run grouped over the sorted rows: float32 multiply-adds of this library, or, for many rows of
        bfloat16, the library's grouped product, as ``linear`` does for so many rows."""
        _cuda_contig(x, "experts' input")
        _cuda_contig(chosen, "chosen", torch.int32)
        _cuda_contig(weights, "weights", torch.float32)
        _cuda_contig(w_up, "experts' up weights", x.dtype)
        _cuda_contig(w_down, "experts' down weights", x.dtype)
        _need(activation in self._ACTS, f"unknown activation {activation!r}")
        clamped = activation == "clamped_swish"
        _need(not clamped or (gated and act_params is not None and len(act_params) == 3), "the clamped activation goes with gated experts and (limit, alpha, up_offset)")
        gate_fn = (lambda t: self.glu(t, limit=act_params[0], alpha=act_params[1], up_offset=act_params[2])) if clamped \
            else (lambda t: self.gated_act(t, activation))
        _need(x.dim() == 2 and x.dtype in _DT and chosen.dim() == 2 and chosen.shape == weights.shape and chosen.shape[0] == x.shape[0],
              "experts: x [T, dim], chosen and weights [T, top]")
        T, dim = x.shape
        top = chosen.shape[1]
        _need(top <= 64, f"a token may use at most 64 experts, got {top}")
        E, up_rows = w_up.shape[0], w_up.shape[1]
        _need(not gated or up_rows % 2 == 0, "gated experts: w_up [E, 2 * hidden, dim]")
        hidden = up_rows // 2 if gated else up_rows
        _need(w_up.shape == (E, up_rows, dim) and w_down.dim() == 2 and w_down.shape[0] == dim and w_down.shape[1] >= E * hidden,
              "experts: w_up [E, hidden, dim], w_down [dim, >= E * hidden]")
        ldd = w_down.shape[1]
        lib = self._lib("moe")
        pairs = T * top
        max_tiles = lib.tl_moe_max_tiles(pairs, E)
        index = torch.empty(2 * pairs + E + 1 + 3 * max_tiles, dtype=torch.int32, device=x.device)
        order, place, ends, tiles = index[:pairs], index[pairs:2 * pairs], index[2 * pairs:2 * pairs + E], index[2 * pairs + E:]
        _check(lib.tl_moe_plan(_ptr(chosen), pairs, E, _ptr(order), _ptr(place), _ptr(tiles), _ptr(ends), _stream()), "moe_plan")
        self.launches += 1
        grouped = getattr(torch, "_grouped_mm", None)
        if (x.dtype == torch.bfloat16 and pairs >= self.GROUPED_MIN_PAIRS and grouped is not None
                and dim % 8 == 0 and hidden % 8 == 0 and ldd % 8 == 0):
            xs = torch.empty((pairs, dim), dtype=x.dtype, device=x.device)
            _check(lib.tl_moe_gather(_ptr(x), _DT[x.dtype], _ptr(order), _ptr(xs), pairs, dim, top, _stream()), "moe_gather")
            self.launches += 1
            u = grouped(xs, w_up.transpose(1, 2), offs=ends, out_dtype=x.dtype)
            u = gate_fn(u) if gated else self.activation(u, activation)
            y = grouped(u, w_down.as_strided((E, hidden, dim), (hidden, 1, ldd)), offs=ends, out_dtype=x.dtype)
        else:
            u = torch.empty((pairs, up_rows), dtype=x.dtype, device=x.device)
            _check(lib.tl_moe_gemm(_ptr(x), _ptr(w_up), _ptr(u), _DT[x.dtype], _ptr(tiles), _ptr(order), top, pairs, E, up_rows, dim,
                                   -1 if gated else self._ACTS[activation], ctypes.c_longlong(up_rows * dim), ctypes.c_longlong(dim),
                                   _stream()), "moe_gemm (up)")
            if gated:
                u = gate_fn(u)
            y = torch.empty((pairs, dim), dtype=x.dtype, device=x.device)
            _check(lib.tl_moe_gemm(_ptr(u), _ptr(w_down), _ptr(y), _DT[x.dtype], _ptr(tiles), _ptr(order), 0, pairs, E, dim, hidden,
                                   -1, ctypes.c_longlong(hidden), ctypes.c_longlong(ldd), _stream()), "moe_gemm (down)")
            self.launches += 2
        splits, plane = 1, 0
        if shared is not None:
            _cuda_contig(shared, "shared expert's output")
            _need(shared.dtype in _DT and shared.shape[-2:] == (T, dim), "shared must be [T, dim] or partial sums of it")
            if shared.dim() == 3:
                _need(shared.dtype == torch.float32, "partial sums must be float32")
                splits, plane = shared.shape[0], shared.stride(0)
            _need(shared.dtype == x.dtype or (shared.dtype == torch.float32 and x.dtype == torch.bfloat16), "shared: dtype")
        if shared_gate is not None:
            _cuda_contig(shared_gate, "shared gate", torch.float32)
            _need(shared is not None and shared_gate.numel() == T, "one gate value per token, with a shared expert")
        out = torch.empty((T, dim), dtype=x.dtype, device=x.device)
        rc = lib.tl_moe_combine(_ptr(y), _DT[x.dtype], _ptr(place), _ptr(weights), _ptr(shared),
                                _DT[shared.dtype] if shared is not None else 0, splits, ctypes.c_longlong(plane), _ptr(shared_gate),
                                _ptr(out), T, dim, top, _stream())
        _check(rc, "moe_combine")
        self.launches += 1
        return out

    def moe_prefers_dense(self, n_tokens: int, top: int, n_experts: int, dtype: torch.dtype) -> bool:
        """Whether a step of so many tokens should take all experts as one matrix (:meth:`moe_dense_hidden`):
        few tokens in bfloat16 that between them touch a good part of the experts anyway.  The weights
        are then read once, at the speed of the decode products, and the rows of experts that a token
        did not choose are multiplied by zero."""
        return dtype == torch.bfloat16 and self.use_tcgen05 and n_tokens <= 64 and 3 * n_tokens * top >= n_experts

    @_timed
    def moe_dense_hidden(self, x: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor, gate: Optional[torch.Tensor],
                         w_up_all: torch.Tensor, *, n_experts: int, hidden: int, activation: str, gated: bool = False,
                         act_params=None, extra_act_params=None) -> torch.Tensor:
        """The hidden rows of *all* experts for a few tokens: ``w_up_all`` is every expert's up matrix
        stacked (``[E * hidden + extra, dim]``, the ``extra`` rows a shared expert's); returns
        ``[T, E * hidden + extra]`` with ``act(up_e x[t]) * weight(t, e)`` in expert ``e``'s columns (zero
        where the token did not choose it) and ``act(.) * gate[t]`` in the extra ones.  With ``gated`` an expert's rows
        of ``w_up_all`` are ``[gate; up]`` (``2 * hidden``) and its ``hidden`` columns of the result hold
        ``act(gate_e x) * (up_e x) * weight``; extra rows are then a shared expert's ``[gate; up]`` too.  With
        ``activation="clamped_swish"`` (gated only) ``act_params`` and ``extra_act_params`` are ``(limit, alpha, up_offset)`` of
        the experts and of the shared expert.  The product of
        that with the experts' down matrices side by side (``[dim, E * hidden + extra]``) is the layer's
        output."""
        _cuda_contig(chosen, "chosen", torch.int32)
        _cuda_contig(weights, "weights", torch.float32)
        _need(activation in self._ACTS, f"unknown activation {activation!r}")
        T, top = chosen.shape
        width = w_up_all.shape[0] // (2 if gated else 1)
        extra = width - n_experts * hidden
        clamped = activation == "clamped_swish"
        _need(not clamped or (gated and act_params is not None), "the clamped activation goes with gated experts and (limit, alpha, up_offset)")
        _need((not gated or extra == 0 or clamped) and extra >= 0 and x.shape[0] == T and weights.shape == chosen.shape,
              "moe_dense_hidden: shapes disagree")
        limit, alpha, up_offset = act_params if clamped else (0.0, 0.0, 0.0)
        extra_limit = (extra_act_params or act_params)[0] if clamped else 0.0
        if gate is not None:
            _cuda_contig(gate, "shared gate", torch.float32)
        u = self.linear(x, w_up_all, partials_ok=True)
        splits = u.shape[0] if u.dim() == 3 else 1
        out = torch.empty((T, width), dtype=x.dtype, device=x.device)
        rc = self._lib("moe").tl_moe_scale_act(_ptr(u), _DT[u.dtype], splits, ctypes.c_longlong(u.stride(0) if splits > 1 else 0),
                                              _ptr(chosen), _ptr(weights), _ptr(gate), _ptr(out), _DT[x.dtype], T, n_experts, hidden,
                                              extra, top, self._ACTS[activation], 1 if gated else 0, ctypes.c_float(limit),
                                              ctypes.c_float(alpha), ctypes.c_float(up_offset), ctypes.c_float(extra_limit), _stream())
        _check(rc, "moe_scale_act")
        self.launches += 1
        return out

    def can_fuse_residual(self, pending, h: torch.Tensor) -> bool:
        """Whether :meth:`linear_residual_norm` takes this pending product for this stream."""
        if not (self.use_fused_residual and self.use_tcgen05 and isinstance(pending, PendingProduct)):
            return False
        x, w = pending.x, pending.w
        if not (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2):
            return False
        M, K = x.shape
        N = w.shape[0]
        if not (h.shape == (M, N) and x.is_contiguous() and w.is_contiguous() and x.data_ptr() % 16 == 0
                and w.data_ptr() % 16 == 0 and M <= self.FUSE_MAX_ROWS):
            return False
        return self._lib("gemm_tcgen05").tl_gemm_tcgen05_residual_supports(M, N, K) == 1

    @_timed
    def linear_residual_norm(self, pending: PendingProduct, h: torch.Tensor, weight: torch.Tensor, eps: float) -> RowScaled:
        """``h += bf16(x @ w.T)`` in place (float32; the product rounded as one that passes through
        memory is) and the rows ``bf16(h * weight)`` with the parts of their sums of squares: one kernel in which the K splits of a column slab are one cluster of
        CTAs that add up through each other's shared memory."""
        x, w = pending.x, pending.w
        _cuda_contig(x, "linear input", torch.bfloat16)
        _cuda_contig(w, "linear weight", torch.bfloat16)
        _cuda_contig(h, "residual stream", torch.float32)
        _cuda_contig(weight, "norm weight", torch.float32)
        M, K = x.shape
        N = w.shape[0]
        _need(w.shape[1] == K and h.shape == (M, N) and weight.numel() == N, "linear_residual_norm: shapes disagree")
        lib = self._lib("gemm_tcgen05")
        _need(lib.tl_gemm_tcgen05_residual_supports(M, N, K) == 1,
              "the fused form takes bfloat16, at most 64 rows and K % 8 == 0")
        xw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        ssq = torch.empty((M, lib.tl_gemm_tcgen05_residual_parts(N)), dtype=torch.float32, device=x.device)
        rc = lib.tl_gemm_tcgen05_residual(_ptr(x), _ptr(w), _ptr(h), _ptr(weight), _ptr(xw), _ptr(ssq), M, N, K,
                                          ctypes.c_void_p(self._status.data_ptr()), _stream())
        _check(rc, "gemm_tcgen05_residual")
        self.launches += 1
        return RowScaled(xw, ssq, N, float(eps))

    @_timed
    def swiglu(self, gate_up, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``gate_up`` is ``[tokens, 2 * hidden]``, or float32 partial sums ``[splits, tokens, 2 * hidden]``
        (then ``out_dtype`` says what to produce), or a :class:`RowScaled` of either (the scale is
        applied to gate and up before the activation)."""
        rs = gate_up if isinstance(gate_up, RowScaled) else None
        if rs is not None:
            gate_up = rs.x
        _cuda_contig(gate_up, "gate_up")
        _need(gate_up.dim() in (2, 3) and gate_up.shape[-1] % 2 == 0 and gate_up.dtype in _DT,
              "swiglu input must be [tokens, 2 * hidden] in float32/bfloat16")
        splits = gate_up.shape[0] if gate_up.dim() == 3 else 1
        _need(splits == 1 or gate_up.dtype == torch.float32, "partial sums must be float32")
        out_dtype = out_dtype or gate_up.dtype
        _need(out_dtype in _DT and (out_dtype == gate_up.dtype or gate_up.dtype == torch.float32),
              "swiglu cannot widen bfloat16 input")
        n, hidden = gate_up.shape[-2], gate_up.shape[-1] // 2
        out = torch.empty((n, hidden), dtype=out_dtype, device=gate_up.device)
        rc = self._lib("elementwise").tl_swiglu(_ptr(gate_up), _DT[gate_up.dtype], splits, _ptr(out), _DT[out_dtype],
                                               n, hidden, *_scale_args(rs, n), _stream())
        _check(rc, "swiglu")
        self.launches += 1
        return out

    # ------------------------------------------------------------------ linear
    @_timed
    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
               partials_ok: bool = False) -> torch.Tensor:
        """``x [M, K] @ w[N, K]^T``.  float32 runs on the CUDA cores (true 32-bit).  bfloat16 with
        at most 64 rows (decode steps) runs on the tcgen05 kernel that streams the weight once;
        more rows use the library product, as the reference's ``nn.Linear`` does.

        With ``partials_ok`` the result may be float32 partial sums ``[splits, M, N]`` of a
        split-K product, for callers that hand it to a kernel which adds them up (residual +
        norm, rope, swiglu).  A :class:`RowScaled` input gives a :class:`RowScaled` result: the
        product is taken of the rows as they are and the scale follows it."""
        if isinstance(x, RowScaled):
            return x.follow(self.linear(x.x, w, out_dtype, partials_ok))
        _cuda_contig(x, "linear input")
        _cuda_contig(w, "linear weight")
        _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], "linear: inner sizes differ")
        _need(x.dtype == w.dtype and x.dtype in _DT, f"linear: dtypes {x.dtype} / {w.dtype} unsupported")
        out_dtype = out_dtype or x.dtype
        M, K = x.shape
        N = w.shape[0]
        if x.dtype == torch.float32:
            _need(out_dtype == torch.float32, "a float32 product has float32 output")
            return self.gemm_simt(x, w, torch.float32)
        if self.use_tcgen05 and M <= 64 and K % 8 == 0 and K >= 8 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
            parts = self.gemm_tcgen05(x, w, out_dtype)
            if parts.dim() == 2 or partials_ok:
                return parts
            return self.sum_partials(parts, out_dtype)
        if out_dtype == torch.bfloat16:
            return torch.mm(x, w.t())
        _need(out_dtype == torch.float32, f"linear: output dtype {out_dtype} unsupported")
        if self._mm_out_dtype is None:
            try:
                torch.mm(x[:1], w[:8].t(), out_dtype=torch.float32)
                self._mm_out_dtype = True
            except (TypeError, RuntimeError):
                self._mm_out_dtype = False
        if self._mm_out_dtype and K % 8 == 0:              # (rows the library can address 16 bytes at a time)
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return self.gemm_simt(x, w, torch.float32)

    def linear_swiglu(self, x: torch.Tensor, w13: torch.Tensor, fused: Optional[bool] = None) -> torch.Tensor:
        """``silu(x @ w13[:H]^T) * (x @ w13[H:]^T)`` for a stacked gate/up weight ``[2 H, K]``, in
        ``x``'s dtype.  Decode-sized bfloat16 inputs whose product needs no K split run as one
        kernel (the activation in the product's epilogue); everything else as product + SwiGLU
        kernel, with the same numbers.  ``fused`` forces the choice (tests).  ``x`` may be a
        :class:`RowScaled`: gate and up are scaled before the activation."""
        rs = x if isinstance(x, RowScaled) else None
        if rs is not None:
            x = rs.x
        _cuda_contig(x, "linear input")
        _cuda_contig(w13, "linear weight")
        _need(x.dim() == 2 and w13.dim() == 2 and x.shape[1] == w13.shape[1] and w13.shape[0] % 2 == 0,
              "linear_swiglu: x [M, K] against w13 [2 H, K]")
        M, K = x.shape
        hidden = w13.shape[0] // 2
        can = (x.dtype == torch.bfloat16 and w13.dtype == torch.bfloat16 and self.use_tcgen05 and M <= 64 and hidden % 64 == 0
               and K % 8 == 0 and K >= 8 and x.data_ptr() % 16 == 0 and w13.data_ptr() % 16 == 0)
        if fused is None:
            fused = (can and self.use_gated and
                     self._lib("gemm_tcgen05").tl_gemm_tcgen05_gated_supports(M, hidden, K) == 1)
        _need(can or not fused, "the fused form takes bfloat16, at most 64 rows, hidden % 64 == 0 and K % 8 == 0")
        if not fused:
            gate_up = self.linear(x, w13, partials_ok=True)
            return self.swiglu(gate_up if rs is None else rs.follow(gate_up), out_dtype=x.dtype)
        return self.gemm_gated(x, w13, rs)

    @_timed
    def gemm_gated(self, x: torch.Tensor, w13: torch.Tensor, rs: Optional[RowScaled] = None) -> torch.Tensor:
        """The one-kernel form of :meth:`linear_swiglu` (its caller has checked the sizes)."""
        M, K = x.shape
        hidden = w13.shape[0] // 2
        out = torch.empty((M, hidden), dtype=torch.bfloat16, device=x.device)
        rc = self._lib("gemm_tcgen05").tl_gemm_tcgen05_gated(
            _ptr(x), _ptr(w13), _ptr(out), M, hidden, K, *_scale_args(rs, M),
            ctypes.c_void_p(self._status.data_ptr()), _stream())
        _check(rc, "gemm_tcgen05_gated")
        self.launches += 1
        return out

    def gemm_tcgen05(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """At most 64 rows of bfloat16 against a bfloat16 weight on the tcgen05 kernel.  Returns
        ``[M, N]`` in ``out_dtype`` when the weight's shape needs no K split, else float32 partial
        sums ``[splits, M, N]``."""
        _cuda_contig(x, "gemm input", torch.bfloat16)
        _cuda_contig(w, "gemm weight", torch.bfloat16)
        M, K = x.shape
        N = w.shape[0]
        _need(x.shape[1] == w.shape[1], "gemm_tcgen05: inner sizes differ")
        _need(1 <= M <= 64 and K % 8 == 0 and K >= 8, "gemm_tcgen05 takes 1..64 rows and K a multiple of 8")
        _need(out_dtype in _DT, f"gemm_tcgen05: output dtype {out_dtype} unsupported")
        lib = self._lib("gemm_tcgen05")
        splits = lib.tl_gemm_tcgen05_splits(M, N, K)
        f32 = out_dtype == torch.float32 or splits > 1
        out = torch.empty((splits, M, N), dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
        rc = lib.tl_gemm_tcgen05(_ptr(x), _ptr(w), _ptr(out), 1 if f32 else 0, M, N, K, splits,
                                 ctypes.c_void_p(self._status.data_ptr()), _stream())
        _check(rc, "gemm_tcgen05")
        self.launches += 1
        return out[0] if splits == 1 else out

    def check_status(self) -> None:
        """Raise if a kernel reported that one of its bounded waits ran out (call after a sync)."""
        code = int(self._status[0])
        if code != 0:
            self._status[0] = 0
            raise KernelError(f"a kernel gave up waiting (code {code}); its output is not valid")
        if self.debug:
            from .build import loaded_libraries
            kinds = {901: "a token id outside the vocabulary", 902: "a position outside the rotary table",
                     903: "a negative cache slot", 904: "a page outside the page tensor", 905: "a row outside the stream"}
            for name in loaded_libraries():
                code = self._lib(name).tl_debug_take()
                if code != 0:
                    raise KernelError(f"debug build: a kernel of {name} was given {kinds.get(code, 'a bad index')} "
                                      f"(code {code}); it skipped the access")

    def wait_selftest(self, limit_ms: float = 1.0) -> float:
        """Run a kernel whose only mbarrier wait nothing will ever satisfy, with a limit of
        ``limit_ms``.  It must give up and say so: :meth:`check_status` then raises, and the device
        stays usable.  Returns the milliseconds the wait took."""
        waited = torch.zeros(1, dtype=torch.int64, device="cuda")
        lib = self._lib("gemm_tcgen05")
        rc = lib.tl_wait_selftest(ctypes.c_void_p(self._status.data_ptr()), ctypes.c_ulonglong(int(limit_ms * 1e6)),
                                  _ptr(waited), _stream())
        _check(rc, "wait_selftest")
        torch.cuda.synchronize()
        return float(waited.item()) / 1e6

    def gemm_simt(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        _cuda_contig(x, "gemm input")
        _cuda_contig(w, "gemm weight")
        _need(x.shape[1] == w.shape[1] and x.dtype == w.dtype and x.dtype in _DT, "gemm_simt: operands disagree")
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        rc = self._lib("gemm_simt").tl_gemm_simt(_ptr(x), _ptr(w), _ptr(out), _DT[x.dtype], _DT[out_dtype],
                                                M, N, K, _stream())
        _check(rc, "gemm_simt")
        self.launches += 1
        return out

    # -------------------------------------------------------------------- rope
    @_timed
    def rope_kv_write(self, qkv, positions: torch.Tensor, table: torch.Tensor, *,
                      n_heads: int, n_kv_heads: int, head_dim: int, interleaved: bool,
                      k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                      slot_mapping: Optional[torch.Tensor], page_size: int,
                      out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``qkv`` is ``[tokens, row]``, or float32 partial sums ``[splits, tokens, row]`` (then
        ``out_dtype`` is the dtype of q and of the pages), or a :class:`RowScaled` of either (every
        row is multiplied by its scale before it is rotated and stored)."""
        rs = qkv if isinstance(qkv, RowScaled) else None
        if rs is not None:
            qkv = rs.x
        _cuda_contig(qkv, "qkv")
        _cuda_contig(positions, "positions", torch.int32)
        _cuda_contig(table, "rotary table", torch.float32)
        splits = qkv.shape[0] if qkv.dim() == 3 else 1
        T = qkv.shape[-2]
        out_dtype = out_dtype or qkv.dtype
        _need(qkv.dim() in (2, 3) and qkv.shape[-1] == (n_heads + 2 * n_kv_heads) * head_dim and qkv.dtype in _DT,
              "qkv must be [tokens, (n_heads + 2 n_kv_heads) * head_dim]")
        _need(splits == 1 or qkv.dtype == torch.float32, "partial sums must be float32")
        _need(out_dtype in _DT and (out_dtype == qkv.dtype or qkv.dtype == torch.float32), "rope cannot widen bfloat16 input")
        _need(table.dim() == 3 and table.shape[1] == head_dim // 2 and table.shape[2] == 2,
              "rotary table must be [positions, head_dim / 2, 2]")
        _need(positions.numel() == T, "one position per token")
        if k_pages is not None:
            _cuda_contig(k_pages, "k_pages", out_dtype)
            _cuda_contig(v_pages, "v_pages", out_dtype)
            _cuda_contig(slot_mapping, "slot_mapping", torch.int32)
            _need(k_pages.shape[1:] == (n_kv_heads, page_size, head_dim) and v_pages.shape == k_pages.shape,
                  "pages must be [pages, n_kv_heads, page_size, head_dim]")
            _need(slot_mapping.numel() == T, "one cache slot per token")
        q = torch.empty((T, n_heads, head_dim), dtype=out_dtype, device=qkv.device)
        if k_pages is not None:
            self._debug_limit("rope", 0, k_pages.shape[0])
        rc = self._lib("rope").tl_rope_kv_write(
            _ptr(qkv), _DT[qkv.dtype], splits, _ptr(positions), _ptr(table),
            _ptr(slot_mapping if k_pages is not None else None),
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _DT[out_dtype], T, n_heads, n_kv_heads, head_dim,
            page_size, table.shape[0], 1 if interleaved else 0, *_scale_args(rs, T), _stream())
        _check(rc, "rope_kv_write")
        self.launches += 1
        return q

    # --------------------------------------------------------------- attention
    def _scratch(self, device: torch.device, floats: int, tag: str = "attention") -> Optional[torch.Tensor]:
        if floats <= 0:
            return None
        key = (device.index or 0, tag)
        buf = self._workspace.get(key)
        if buf is None or buf.numel() < floats:
            if buf is not None:
                self._retired.append(buf)      # a captured graph may still point into it
            buf = torch.empty(max(floats, 1 << 22), dtype=torch.float32, device=device)
            self._workspace[key] = buf
        return buf

    @_timed
    def paged_attention(self, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                        block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor, *,
                        n_seqs: int, max_q_len: int, max_kv_len: int, scale: float,
                        window: Optional[int], page_size: int, allow_split: bool = True,
                        impl: str = "auto", n_tokens: Optional[int] = None,
                        out: Optional[torch.Tensor] = None, keep_first: int = 0,
                        distance_bias: Optional[torch.Tensor] = None, distance_buckets: Optional[torch.Tensor] = None,
                        gate: Optional[torch.Tensor] = None, n_v_heads: Optional[int] = None,
                        out_dtype: Optional[torch.dtype] = None, softcap: float = 0.0, sinks: Optional[torch.Tensor] = None,
                        value_dim: Optional[int] = None) -> torch.Tensor:
        """``impl``: ``"general"`` (CUDA cores, any supported size, both dtypes), ``"mma"`` (tensor
        cores, bfloat16, head_dim 16/32/64/128), ``"decode"`` (tensor cores fed by TMA, bfloat16,
        head_dim 64/128, steps whose requests bring one token or very few), ``"prefill"``
        (tcgen05 tensor cores with accumulators in tensor memory, bfloat16, head_dim 64/128, made
        for long portions; ``"prefill2"`` is its variant that multiplies probabilities as value +
        remainder) or ``"auto"`` (the most specialised kernel that applies).

        ``block_table``, ``q_start`` and ``kv_len`` may be slices that cover only some requests of
        the step (``q_start`` keeps counting tokens from the start of ``q``); ``n_tokens`` then
        bounds the rows those requests own (default: all of ``q``), and ``out`` lets several such
        calls fill one tensor.  ``allow_split``: False keeps every request's keys in one CTA, True lets
        the kernel split them as it sees fit; the decode kernel also takes a number of splits (above 1).

        The general kernel alone also takes: values of another size than keys (``v_pages``
        ``[pages, kv_heads, page_size, v_dim]``, possibly the very tensor ``k_pages``; the result is
        ``[T, H, v_dim]``), ``keep_first`` (with a window: the first so many keys of a request stay
        visible), ``distance_bias`` ``[rows, H]`` float32 with ``distance_buckets`` (int32: the
        table's row for every distance), added to the scaled score, and ``gate`` (``[T, H]`` or
        ``[T, H * v_dim]``, in q's dtype), by which the result is multiplied; ``n_v_heads`` (``v_pages`` has
        fewer heads than ``k_pages``: key head ``j`` goes with value head ``j % n_v_heads``, several maps
        with keys of their own over one set of values) and ``out_dtype=torch.float32`` (the result
        leaves unrounded whatever q's dtype); ``softcap = c > 0`` (the scaled score ``s`` becomes ``c * tanh(s / c)``),
        ``sinks`` (float32 ``[H]``: ``exp(sinks[h])`` joins the softmax's denominator, a key without a value that is neither
        scaled nor capped) and ``value_dim`` (``v_pages`` is ``k_pages`` and a value is the first ``value_dim`` coordinates
        of a stored key; the result is ``[T, H, value_dim]``)."""
        if keep_first or distance_bias is not None or gate is not None or v_pages.shape[-1] != q.shape[-1] \
                or q.shape[-1] % 16 != 0 or v_pages.shape[1] != k_pages.shape[1] or out_dtype not in (None, q.dtype) \
                or softcap or sinks is not None or value_dim:
            _need(impl in ("auto", "general", "mma"), "only the general and the mma.sync attention kernels take these options")
            return self._paged_attention_general(q, k_pages, v_pages, block_table, q_start, kv_len, n_seqs, max_q_len,
                                                 max_kv_len, scale, window, page_size, allow_split, n_tokens, out,
                                                 keep_first, distance_bias, distance_buckets, gate, impl, n_v_heads, out_dtype,
                                                 softcap, sinks, value_dim)
        _cuda_contig(q, "q")
        _cuda_contig(k_pages, "k_pages", q.dtype)
        _cuda_contig(v_pages, "v_pages", q.dtype)
        _cuda_contig(q_start, "q_start", torch.int32)
        _cuda_contig(kv_len, "kv_len", torch.int32)
        _need(block_table.is_cuda and block_table.dtype == torch.int32 and block_table.dim() == 2
              and block_table.stride(1) == 1, "block_table must be an int32 matrix with unit column stride")
        T, n_heads, head_dim = q.shape
        if n_tokens is not None:
            _need(0 < n_tokens <= T, "n_tokens must lie within q")
            T = int(n_tokens)
        if out is not None:
            _cuda_contig(out, "out", q.dtype)
            _need(out.shape == q.shape, "out must have q's shape")
        n_kv_heads = k_pages.shape[1]
        self.check_attention_sizes(n_heads, n_kv_heads, head_dim, q.dtype)
        _need(k_pages.shape[2] == page_size and k_pages.shape[3] == head_dim and v_pages.shape == k_pages.shape,
              "pages must be [pages, n_kv_heads, page_size, head_dim]")
        _need(block_table.shape[0] >= n_seqs and q_start.numel() >= n_seqs + 1 and kv_len.numel() >= n_seqs,
              "block_table, q_start and kv_len must cover every request of the step")
        _need(block_table.shape[1] * page_size >= max_kv_len, "block_table is too narrow for max_kv_len")
        _need(impl in ("auto", "general", "mma", "decode", "prefill", "prefill2"), f"unknown attention implementation {impl!r}")
        # "prefill2": the tcgen05 prefill kernel that multiplies probabilities as value + remainder
        parts = 2 if impl == "prefill2" else self.prefill_probability_parts
        if impl == "prefill2":
            impl = "prefill"
        mma_ok = q.dtype == torch.bfloat16 and head_dim in (16, 32, 64, 128)
        _need(impl != "mma" or mma_ok, "the tensor-core attention kernel takes bfloat16 and head_dim 16, 32, 64 or 128")
        use_mma = mma_ok and impl in ("auto", "mma")
        decode_ok = (q.dtype == torch.bfloat16 and impl in ("auto", "decode") and head_dim in (64, 128) and
                     self._lib("attention_decode").tl_attention_decode_supports(n_heads, n_kv_heads, head_dim,
                                                                                 page_size, max_q_len) == 1)
        _need(impl != "decode" or decode_ok, "the decode attention kernel takes bfloat16, head_dim 64 or 128, a "
              "power-of-two page size and requests whose rows fit one 16-row tile")
        n_splits = ctypes.c_int(0)
        floats = ctypes.c_longlong(0)
        if out is None:
            out = torch.empty_like(q)
        prefill_ok = (q.dtype == torch.bfloat16 and impl in ("auto", "prefill") and head_dim in (64, 128) and not decode_ok
                      and (impl == "prefill" or max_q_len >= self.PREFILL_MIN_Q) and
                      self._lib("attention_prefill").tl_attention_prefill_supports(n_heads, n_kv_heads, head_dim, page_size) == 1)
        _need(impl != "prefill" or prefill_ok, "the tcgen05 prefill attention kernel takes bfloat16, head_dim 64 or 128 "
              "and a power-of-two page size")
        if prefill_ok:
            lib = self._lib("attention_prefill")
            self._debug_limit("attention_prefill", 0, k_pages.shape[0])
            rc = lib.tl_paged_attention_prefill(
                _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(q_start), _ptr(kv_len), ctypes.c_void_p(self._status.data_ptr()), ctypes.c_longlong(q.shape[0]),
                T, n_seqs, n_heads, n_kv_heads, head_dim, page_size, ctypes.c_longlong(k_pages.shape[0]), max_q_len,
                int(window or 0), ctypes.c_float(scale), parts, _stream())
            _check(rc, "paged_attention_prefill")
            self.launches += 1
            return out
        if decode_ok:
            lib = self._lib("attention_decode")
            rc = lib.tl_attention_decode_plan(T, n_seqs, n_heads, n_kv_heads, head_dim, max_q_len, max_kv_len,
                                              int(allow_split), ctypes.byref(n_splits), ctypes.byref(floats))
            _check(rc, "attention_decode_plan")
            ws = self._scratch(q.device, floats.value)
            self._debug_limit("attention_decode", 0, k_pages.shape[0])
            rc = lib.tl_paged_attention_decode(
                _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(q_start), _ptr(kv_len), _ptr(ws), ctypes.c_void_p(self._status.data_ptr()), T, n_seqs,
                n_heads, n_kv_heads, head_dim, page_size, ctypes.c_longlong(k_pages.shape[0]), max_q_len, max_kv_len,
                int(window or 0), ctypes.c_float(scale), int(allow_split), _stream())
            _check(rc, "paged_attention_decode")
        elif use_mma:
            lib = self._lib("attention_mma")
            rc = lib.tl_attention_mma_plan(T, n_seqs, n_heads, n_kv_heads, head_dim, max_q_len, max_kv_len,
                                           1 if allow_split else 0, ctypes.byref(n_splits), ctypes.byref(floats))
            _check(rc, "attention_mma_plan")
            ws = self._scratch(q.device, floats.value)
            self._debug_limit("attention_mma", 0, k_pages.shape[0])
            rc = lib.tl_paged_attention_mma(
                _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(q_start), _ptr(kv_len), _ptr(ws), T, n_seqs, n_heads, n_kv_heads, head_dim,
                page_size, max_q_len, max_kv_len, int(window or 0), ctypes.c_float(scale),
                1 if allow_split else 0, _stream())
            _check(rc, "paged_attention_mma")
        else:
            return self._paged_attention_general(q, k_pages, v_pages, block_table, q_start, kv_len, n_seqs, max_q_len,
                                                 max_kv_len, scale, window, page_size, allow_split, n_tokens, out,
                                                 0, None, None, None)
        self.launches += 2 if n_splits.value > 1 else 1
        return out

    class _AttentionOptions(ctypes.Structure):
        _fields_ = [("v_head_dim", ctypes.c_int), ("keep_first", ctypes.c_int), ("rel", ctypes.c_void_p),
                    ("bucket", ctypes.c_void_p), ("n_bucket", ctypes.c_int), ("gate", ctypes.c_void_p),
                    ("gate_mode", ctypes.c_int), ("n_v_heads", ctypes.c_int), ("out_f32", ctypes.c_int),
                    ("softcap", ctypes.c_float), ("sinks", ctypes.c_void_p), ("v_stride", ctypes.c_int)]

    def _paged_attention_general(self, q, k_pages, v_pages, block_table, q_start, kv_len, n_seqs, max_q_len, max_kv_len,
                                 scale, window, page_size, allow_split, n_tokens, out, keep_first, distance_bias,
                                 distance_buckets, gate, impl: str = "general", n_v_heads: Optional[int] = None,
                                 out_dtype: Optional[torch.dtype] = None, softcap: float = 0.0,
                                 sinks: Optional[torch.Tensor] = None, value_dim: Optional[int] = None) -> torch.Tensor:
        """The CUDA-core kernel with everything it can do (see :meth:`paged_attention`), or, with
        ``impl`` "auto" or "mma", in bfloat16 and for sizes it takes (keys and values multiples of 8
        up to 128), the extended form of the mma.sync kernel, which does the same."""
        _cuda_contig(q, "q")
        _cuda_contig(k_pages, "k_pages", q.dtype)
        _cuda_contig(v_pages, "v_pages", q.dtype)
        _cuda_contig(q_start, "q_start", torch.int32)
        _cuda_contig(kv_len, "kv_len", torch.int32)
        _need(block_table.is_cuda and block_table.dtype == torch.int32 and block_table.dim() == 2
              and block_table.stride(1) == 1, "block_table must be an int32 matrix with unit column stride")
        T_all, n_heads, head_dim = q.shape
        T = T_all if n_tokens is None else int(n_tokens)
        _need(0 < T <= T_all, "n_tokens must lie within q")
        n_kv_heads, v_dim = k_pages.shape[1], v_pages.shape[3]
        v_stride = 0
        if value_dim:
            _need(v_pages.data_ptr() == k_pages.data_ptr() and 0 < value_dim <= head_dim,
                  "value_dim: values are the first coordinates of the stored keys (v_pages is k_pages)")
            v_dim, v_stride = int(value_dim), head_dim
        self.check_attention_sizes(n_heads, n_kv_heads, head_dim, q.dtype, v_dim)
        v_heads = v_pages.shape[1]
        _need(n_v_heads in (None, v_heads) and n_kv_heads % v_heads == 0, "n_v_heads must be the heads of v_pages and divide the key heads")
        _need(k_pages.shape[2] == page_size and k_pages.shape[3] == head_dim and v_pages.shape[0] == k_pages.shape[0]
              and v_pages.shape[2] == page_size,
              "pages must be [pages, n_kv_heads, page_size, head_dim] (values: their own head count and last size)")
        out_dtype = out_dtype or q.dtype
        _need(out_dtype in (q.dtype, torch.float32), "attention writes q's dtype or float32")
        _need(block_table.shape[0] >= n_seqs and q_start.numel() >= n_seqs + 1 and kv_len.numel() >= n_seqs,
              "block_table, q_start and kv_len must cover every request of the step")
        _need(block_table.shape[1] * page_size >= max_kv_len, "block_table is too narrow for max_kv_len")
        _need(keep_first >= 0 and (not keep_first or window), "keep_first goes with a window")
        if out is None:
            out = torch.empty((T_all, n_heads, v_dim), dtype=out_dtype, device=q.device)
        else:
            _cuda_contig(out, "out", out_dtype)
            _need(out.shape == (T_all, n_heads, v_dim), "out must be [tokens, heads, v_dim]")
        opt = self._AttentionOptions(v_dim, int(keep_first), None, None, 0, None, 0, v_heads,
                                     1 if (out_dtype == torch.float32 and q.dtype != torch.float32) else 0,
                                     float(softcap or 0.0), None, v_stride)
        _need(opt.softcap >= 0.0, "softcap must not be negative")
        if sinks is not None:
            _cuda_contig(sinks, "sinks", torch.float32)
            _need(sinks.numel() == n_heads, "one sink per query head")
            opt.sinks = sinks.data_ptr()
        if distance_bias is not None:
            _cuda_contig(distance_bias, "distance_bias", torch.float32)
            _cuda_contig(distance_buckets, "distance_buckets", torch.int32)
            _need(distance_bias.dim() == 2 and distance_bias.shape[1] == n_heads, "distance_bias must be [rows, n_heads]")
            _need(distance_buckets.numel() >= min(max_kv_len, block_table.shape[1] * page_size),
                  "distance_buckets must reach as far as the longest context")
            opt.rel, opt.bucket, opt.n_bucket = distance_bias.data_ptr(), distance_buckets.data_ptr(), distance_buckets.numel()
        if gate is not None:
            _cuda_contig(gate, "gate", q.dtype)
            _need(gate.dim() == 2 and gate.shape[0] == T_all and gate.shape[1] in (n_heads, n_heads * v_dim),
                  "gate must be [tokens, heads] or [tokens, heads * v_dim]")
            opt.gate, opt.gate_mode = gate.data_ptr(), (1 if gate.shape[1] == n_heads and v_dim != 1 else 2)
        n_splits, floats = ctypes.c_int(0), ctypes.c_longlong(0)
        mma_ok = (q.dtype == torch.bfloat16 and impl in ("auto", "mma") and self.use_mma_options
                  and self._lib("attention_mma").tl_attention_mma_ex_supports(head_dim, v_dim) == 1
                  and not (softcap and distance_bias is not None))
        _need(impl != "mma" or mma_ok, "the mma.sync kernel takes bfloat16 and keys and values that are multiples of 8 up to 128")
        if mma_ok:
            lib = self._lib("attention_mma")
            rc = lib.tl_attention_mma_plan_ex(T, n_seqs, n_heads, n_kv_heads, head_dim, v_dim, max_q_len, max_kv_len,
                                              int(window or 0), int(keep_first), 1 if allow_split else 0,
                                              ctypes.byref(n_splits), ctypes.byref(floats))
            _check(rc, "attention_mma_plan")
            ws = self._scratch(q.device, floats.value)
            self._debug_limit("attention_mma", 0, k_pages.shape[0])
            rc = lib.tl_paged_attention_mma_ex(
                _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(q_start), _ptr(kv_len), _ptr(ws), T, n_seqs, n_heads, n_kv_heads, head_dim,
                page_size, max_q_len, max_kv_len, int(window or 0), ctypes.c_float(scale),
                1 if allow_split else 0, ctypes.byref(opt), _stream())
            _check(rc, "paged_attention_mma")
            self.launches += 2 if n_splits.value > 1 else 1
            return out
        lib = self._lib("attention")
        rc = lib.tl_attention_plan_ex(T, n_seqs, n_heads, n_kv_heads, head_dim, v_dim, max_q_len, max_kv_len,
                                      int(window or 0), int(keep_first), 1 if allow_split else 0,
                                      ctypes.byref(n_splits), ctypes.byref(floats))
        _check(rc, "attention_plan")
        ws = self._scratch(q.device, floats.value)
        self._debug_limit("attention", 0, k_pages.shape[0])
        rc = lib.tl_paged_attention_ex(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(block_table), block_table.stride(0),
            _ptr(q_start), _ptr(kv_len), _ptr(ws), _DT[q.dtype], T, n_seqs, n_heads, n_kv_heads, head_dim,
            page_size, max_q_len, max_kv_len, int(window or 0), ctypes.c_float(scale),
            1 if allow_split else 0, ctypes.byref(opt), _stream())
        _check(rc, "paged_attention")
        self.launches += 2 if n_splits.value > 1 else 1
        return out

    # ---------------------------------------------------------------- sampling
    @_timed
    def sample(self, logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
               top_k: Optional[torch.Tensor] = None, row_keys: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Next token of every row.  ``temperature`` (float32), ``top_k`` (int32) and
        ``row_keys`` (int64 holding the 64-bit key) are per row; without a temperature
        every row is greedy."""
        _need(logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1,
              "logits must be a float32 matrix on the GPU with unit column stride")
        n, vocab = logits.shape
        if temperature is not None:
            _cuda_contig(temperature, "temperature", torch.float32)
            _need(row_keys is not None, "sampling with a temperature needs row keys")
            _cuda_contig(row_keys, "row_keys", torch.int64)
            _need(temperature.numel() == n and row_keys.numel() == n, "one temperature and key per row")
        if top_k is not None:
            _cuda_contig(top_k, "top_k", torch.int32)
            _need(top_k.numel() == n, "one top_k per row")
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
        lib = self._lib("sampling")
        if top_k is None and vocab > 8192:
            # no rank filter: spread every row over many CTAs, then pick among their candidates
            lib.tl_sample_wide_scratch.restype = ctypes.c_longlong
            ws = self._scratch(logits.device, lib.tl_sample_wide_scratch(n, vocab), "sampling")
            rc = lib.tl_sample_wide(_ptr(logits), ctypes.c_longlong(logits.stride(0)), n, vocab, _ptr(temperature),
                                    _ptr(row_keys), _ptr(ws), _ptr(out), _stream())
            _check(rc, "sample_wide")
            self.launches += 2
            return out
        rc = lib.tl_sample(
            _ptr(logits), ctypes.c_longlong(logits.stride(0)), n, vocab, _ptr(temperature), _ptr(top_k),
            _ptr(row_keys), _ptr(out), _stream())
        _check(rc, "sample")
        self.launches += 1
        return out


def build_all() -> None:
    """Compile every kernel library (what ``__graft_entry__.build`` calls)."""
    build_libraries(ALL_LIBRARIES)
