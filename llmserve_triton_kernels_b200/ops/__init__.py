"""The engine's device operations: thin, checked wrappers over the CUDA library.

Every function here launches hand-written sm_100a kernels from ``csrc/`` on the current CUDA
stream (the bfloat16 matrix products may go to the vendor's library, as the reference's do:
src/llmserve/model/llama.py:80-88, 120, 185 call ``F.linear``).  There is no CPU path: without
a CUDA device, or if the library cannot be built and loaded, the first call raises.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

from . import build as _build

_F32, _BF16 = 0, 1
_lib = None
_lock = threading.Lock()

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_SIGNATURES = {
    "llm_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _vp],
    "llm_rmsnorm": [_vp, _vp, _i, _vp, _f, _vp, _vp, _i, _i, _i, _vp],
    "llm_rope_kv_write": [_vp, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "llm_swiglu": [_vp, _vp, _i, _i, _i, _vp],
    "llm_add_bias": [_vp, _i, _i, _i, _i, _vp, _vp],
    "llm_fetch_words": [_vp, _vp, _vp, _i, _i, _vp],
    "llm_set_error_flag": [_vp],
    "llm_check_step_arrays": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "llm_check_page_group": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "llm_gemm_simt": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "llm_linear_decode": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _i, _f, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "llm_linear_decode_qkv": [_vp, _vp, _vp, _i, _i, _i, _vp, _i, _f, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "llm_gemm_tcgen05": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "llm_gemm_tcgen05_fused": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp],
    "llm_gemm_tcgen05_parts": [_i],
    "llm_attention_generic": [_vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp],
    "llm_attention_mma": [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "llm_attention_mma_routed": [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp],
    "llm_attention_tcgen05": [_vp, _i, _vp, _i, _vp, ctypes.c_longlong, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp],
    "llm_argmax": [_vp, _i, _i, _vp, _vp, _vp],
    "llm_sample": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
}


class KernelError(RuntimeError):
    pass


def library():
    """The loaded CUDA library; built first if it is missing or out of date."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not torch.cuda.is_available():
                raise KernelError(
                    "no CUDA device is visible: this engine has no CPU path (its kernels are sm_100a CUDA)"
                )
            path = _build.build()
            lib = ctypes.CDLL(str(path))
            for name, args in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = args
                fn.restype = ctypes.c_int
            lib.llm_error_string.argtypes = [ctypes.c_int]
            lib.llm_error_string.restype = ctypes.c_char_p
            _lib = lib
            if torch.cuda.is_available():
                lib.llm_set_error_flag(_error_flag_ptr())  # for kernels whose entry points take no flag of their own
    return _lib


_launches = 0
_MMA_HEAD_DIMS = (16, 32, 64, 128)  # head sizes of the tensor-core attention; others take the general kernel
_SMALL_ROWS = 16  # requests with at most this many (token, group member) rows take the split-key shape
_SMALL_TILE_KEYS = 128  # keys one CTA of that shape covers per tile
_SPLIT_SCRATCH_BYTES = 16 << 20  # most scratch memory the split-key attention's partial results may take per call
_TC_ATTENTION_ENABLED = True
_TC_ATTENTION_HEAD_DIMS = (64, 128)
_TC_ATTENTION_PAGE_SIZES = (8, 16, 32, 64)
_TC_ATTENTION_MIN_TOKENS = 128  # a request with at least this many tokens in the step: attention on tcgen05
_TCGEN05_MIN_ROWS = 128  # from this many rows a bfloat16 product runs on tcgen05 with TMA-fed tiles (own kernel)
_DECODE_LINEAR_MAX_ROWS = 16  # up to this many rows a bfloat16 matrix product streams the weights once (own kernel)
_FORCE_GENERIC_ATTENTION = False  # tests switch the tensor-core attention off to reach the general kernel in bfloat16


_sm_counts: dict[int, int] = {}


def _sm_count() -> int:
    """SMs of the current device (asked once per device)."""
    device = torch.cuda.current_device()
    count = _sm_counts.get(device)
    if count is None:
        count = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return count


def launch_count() -> int:
    """How many kernels of the library have been launched by this process (a CUDA graph's replay
    counts the launches it captured)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _launch(name: str, *args) -> int:
    global _launches
    _launches += 1
    return getattr(library(), name)(*args)


def loaded_library_path() -> str | None:
    return None if _lib is None else _lib._name


def _check(code: int, what: str) -> None:
    if code != 0:
        text = _lib.llm_error_string(code).decode() if _lib is not None else ""
        raise KernelError(f"{what}: error {code} ({text})")


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"element type {dtype} is not supported (float32 or bfloat16)")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Asked once per launch, so by the short way where torch has one (the Stream
    object of ``torch.cuda.current_stream()`` costs several microseconds to build)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _i32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.int32 and t.is_contiguous() and t.is_cuda, f"{name} must be a contiguous int32 CUDA tensor")


# ------------------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """``float32(table[ids])``: ids ``[N]`` int32, table ``[vocab, hidden]`` -> ``[N, hidden]`` float32."""
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous(), "the token table must be a contiguous matrix")
    n, (vocab, hidden) = ids.numel(), table.shape
    out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _check(_launch("llm_embed", _ptr(ids), _ptr(table), _code(table.dtype), _ptr(out), n, hidden, vocab, _stream()), "embed")
    return out


def rmsnorm(
    resid: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    delta: torch.Tensor | None = None,
    rows: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """``v = resid (+ delta)``; returns ``v * rsqrt(mean(v^2) + eps) * weight`` in ``out_dtype``.
    Without ``rows`` the sum is written back to ``resid`` (float32, in place); with ``rows``
    (int32) only those rows are produced and ``resid`` is not changed."""
    _need(resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous(), "the residual must be a contiguous float32 matrix")
    _need(weight.dtype == torch.float32 and weight.numel() == resid.shape[1], "the norm weight must be float32 of the row size")
    if delta is not None:
        _need(delta.shape == resid.shape and delta.is_contiguous(), "delta must have the residual's shape")
    if rows is not None:
        _i32(rows, "rows")
    n_out = resid.shape[0] if rows is None else rows.numel()
    out = torch.empty((n_out, resid.shape[1]), dtype=out_dtype, device=resid.device)
    code = _launch("llm_rmsnorm", 
        _ptr(resid), _ptr(delta), _code(delta.dtype) if delta is not None else -1, _ptr(weight), float(eps),
        _ptr(rows), _ptr(out), _code(out_dtype), n_out, resid.shape[1], _stream(),
    )
    _check(code, "rmsnorm")
    return out


_error_flag: torch.Tensor | None = None


def _error_flag_ptr() -> int:
    """Address of a pinned host word that kernels set when one of their bounded waits gives up."""
    global _error_flag
    if _error_flag is None:
        _error_flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _error_flag.data_ptr()


def check_device_errors() -> None:
    """Raise if a kernel reported that a bounded wait gave up, or (checked mode) that a step's arrays held an index out
    of its bounds (call after a synchronisation)."""
    if _error_flag is not None and int(_error_flag[0]) != 0:
        _error_flag[0] = 0
        raise KernelError("a kernel's wait for an asynchronous copy gave up; its results are not valid")
    if _check_status is not None and int(_check_status[0]) != 0:
        code, group, index, value, limit, count = (int(v) for v in _check_status[:6])
        _check_status.zero_()
        what = _CHECK_CODES.get(code, f"violation {code}")
        where = f" of page group {group}" if group >= 0 else ""
        raise KernelError(
            f"checked mode: {what}{where}: entry {index} holds {value} against {limit} ({count} violations in all); the entries were "
            "replaced by harmless ones before any kernel used them, and the step's results are not valid"
        )


# Checked mode (the environment variable LLMSERVE_B200_CHECKED=1, or set_checked): every step starts with kernels that
# look over its integer arrays on the device, where the step's kernels will read them (csrc/step_check.cu).
_checked = bool(os.environ.get("LLMSERVE_B200_CHECKED"))
_check_status: torch.Tensor | None = None
_CHECK_CODES = {
    1: "a token id outside the vocabulary", 2: "a position beyond the model's positions", 3: "a token that names a request it does not belong to",
    4: "token offsets that do not rise or do not end at the number of tokens", 5: "a context length shorter than the request's new tokens or beyond the model's positions",
    6: "a wanted row beyond the step's tokens", 7: "a state slot beyond the slots there are", 8: "a page table entry outside the pool",
    9: "a slot that is outside the pool or disagrees with the page table", 10: "a page table narrower than a request's pages",
}


def checked() -> bool:
    return _checked


def set_checked(on: bool) -> None:
    """Turn checked mode on or off for steps that run, or are captured as graphs, from now on."""
    global _checked
    _checked = bool(on)


def _check_status_ptr() -> int:
    global _check_status
    if _check_status is None:
        _check_status = torch.zeros(8, dtype=torch.int32).pin_memory()
    return _check_status.data_ptr()


def check_step_arrays(ctx, vocab: int, max_positions: int, state_slot_count: int = 0) -> None:
    """Checked mode: compare a step's token ids, positions, request indices, offsets, lengths, wanted rows and state
    slots with their limits on the device; a violation is recorded for :func:`check_device_errors` and repaired."""
    _check(_launch(
        "llm_check_step_arrays", _ptr(ctx.token_ids), _ptr(ctx.positions), _ptr(ctx.token_request), _ptr(ctx.cu_tokens),
        _ptr(ctx.context_lens), _ptr(ctx.logit_rows) if ctx.num_logits else None, _ptr(ctx.state_slots), ctx.num_tokens,
        ctx.num_requests, ctx.num_logits, vocab, max_positions, state_slot_count, _check_status_ptr(), _stream(),
    ), "check_step_arrays")


def check_page_group(ctx, page_table: torch.Tensor, slot_map: torch.Tensor, page_size: int, num_pages: int,
                     window: int | None, group: int) -> None:
    """Checked mode, after :func:`check_step_arrays`: every page table entry that the step may read lies inside the pool
    of ``num_pages`` pages, and every new token's slot is the one its page table gives."""
    _check(_launch(
        "llm_check_page_group", _ptr(page_table), page_table.shape[1], _ptr(slot_map), _ptr(ctx.positions), _ptr(ctx.token_request),
        _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), ctx.num_tokens, ctx.num_requests, page_size, num_pages, window or 0, group,
        _check_status_ptr(), _stream(),
    ), "check_page_group")


class NormedInput:
    """A normalised activation in factored form, as the fused decode kernels hand it on:
    ``xw [M, hidden]`` holds ``v * norm_weight`` (``v`` the residual stream after the last sum) and
    ``ss [parts, M]`` partial sums of ``v^2`` per row, so that
    ``normalised = xw * rsqrt(ss.sum(0) / hidden + eps)``.  ``ops.linear`` and ``ops.linear_swiglu``
    take it in place of a tensor and apply the row scale to their result; anything else calls
    :meth:`materialize`."""

    def __init__(self, xw: torch.Tensor, ss: torch.Tensor, eps: float, norm=None):
        self.xw, self.ss, self.eps, self.norm = xw, ss, float(eps), norm
        self.shape, self.dtype, self.device = xw.shape, xw.dtype, xw.device

    def materialize(self) -> torch.Tensor:
        scale = torch.rsqrt(self.ss.sum(0) / self.xw.shape[1] + self.eps)
        return (self.xw.float() * scale[:, None]).to(self.xw.dtype)


class _Added:
    """What :meth:`ResidualSink.linear` returns when the product has been added to the residual stream and nothing is
    left pending: the next norm normalises the stream as it stands."""

    def __repr__(self) -> str:
        return "ADDED"


ADDED = _Added()


class ResidualSink:
    """Where a part's last matrix product may put its result: added to the 32-bit residual stream ``resid`` in place.
    For few rows the fused decode kernel does it and hands the stream on normalised for ``norm`` (an RMS norm's
    ``weight`` and ``eps``; None: a norm that cannot be folded into a product's end) as a :class:`NormedInput`; for
    more rows the product's own epilogue adds into the stream (the library's product with the stream as its addend,
    accumulated and written in 32-bit), and :data:`ADDED` is returned: no contribution travels through memory to be
    added by the norm's kernel, which then only reads the stream.  Built by a block for bfloat16 steps."""

    def __init__(self, resid: torch.Tensor, weight: torch.Tensor | None, eps: float, norm=None):
        self.resid, self.weight, self.eps, self.norm = resid, weight, float(eps), norm

    @staticmethod
    def usable(num_tokens: int, dtype: torch.dtype) -> bool:
        return dtype == torch.bfloat16

    def linear(self, x: torch.Tensor, w: torch.Tensor) -> "NormedInput | _Added | None":
        """``resid += x @ w^T``; returns the stream normalised for ``norm``, or :data:`ADDED`, or None if no way
        takes the operands (then nothing was changed)."""
        m, k = x.shape
        n = w.shape[0]
        if not (x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.is_contiguous() and self.resid.is_contiguous()):
            return None
        if m <= _DECODE_LINEAR_MAX_ROWS and self.weight is not None:
            parts = -(-n // 16)
            xw = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
            ss = torch.empty((parts, m), dtype=torch.float32, device=x.device)
            code = _launch(
                "llm_linear_decode", _ptr(x), _ptr(w), None, _BF16, m, n, k, x.stride(0), n, None, 0, 0.0, 2, 0,
                _ptr(self.resid), _ptr(self.weight), _ptr(xw), _ptr(ss), _error_flag_ptr(), _stream(),
            )
            if code != 10002:
                _check(code, "linear into the residual stream")
                return NormedInput(xw, ss, self.eps, self.norm)
            add_launches(-1)  # a shape the kernel refuses: the library's way below
        if _GEMM_POLICY == "own" and m >= _TCGEN05_MIN_ROWS:
            return None  # the caller runs the own tcgen05 product and leaves the sum to the norm's kernel
        library()
        torch.addmm(self.resid, x, w.t(), out_dtype=torch.float32, out=self.resid)
        return ADDED

    def linear_tcgen05(self, x: torch.Tensor, w: torch.Tensor) -> "NormedInput | None":
        """The same by the own tcgen05 kernel for 128 rows and more, whose four epilogue warps turn each 32 x 32 piece
        round in shared memory so that the 32-bit stream is read and written 128 bytes at a time.  Correct, and kept
        under test, but four warps per SM do not keep enough of the stream in flight: a prompt of 2,048 tokens on a
        1.1B model took 6.04 ms this way against 5.46 ms with the sum left to the norm's kernel, so no part calls it."""
        m, k = x.shape
        n = w.shape[0]
        if not (x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.is_contiguous() and m >= _TCGEN05_MIN_ROWS and self.weight is not None):
            return None
        parts = library().llm_gemm_tcgen05_parts(n)
        xw = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        ss = torch.empty((parts, m), dtype=torch.float32, device=x.device)
        code = _launch(
            "llm_gemm_tcgen05_fused", _ptr(x), x.stride(0), _ptr(w), None, _BF16, m, n, k, n, 2, 0, None, 0, 0.0,
            _ptr(self.resid), _ptr(self.weight), _ptr(xw), _ptr(ss), _error_flag_ptr(), _stream(),
        )
        if code == 10002:
            add_launches(-1)
            return None
        _check(code, "linear into the residual stream (tcgen05)")
        return NormedInput(xw, ss, self.eps, self.norm)


def _decode_linear(x, w, out_dtype, mode: int, n_out: int, up_offset: int = 0):
    """The weight-streaming product for few rows; None if it refuses the shape."""
    scaled = isinstance(x, NormedInput)
    xt = x.xw if scaled else x
    m, k = xt.shape
    if not (xt.dtype == torch.bfloat16 and m <= _DECODE_LINEAR_MAX_ROWS and xt.stride(1) == 1 and w.is_contiguous()):
        return None
    out = torch.empty((m, n_out), dtype=out_dtype, device=xt.device)
    code = _launch(
        "llm_linear_decode", _ptr(xt), _ptr(w), _ptr(out), _code(out_dtype), m, n_out, k, xt.stride(0), n_out,
        _ptr(x.ss) if scaled else None, x.ss.shape[0] if scaled else 0, x.eps if scaled else 0.0, mode, up_offset,
        None, None, None, None, _error_flag_ptr(), _stream(),
    )
    if code == 10002:  # a shape the kernel refuses
        add_launches(-1)
        return None
    _check(code, "linear (decode)")
    return out


def linear(x, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K]^T -> [M, N]``.  float32 operands run on the CUDA cores in true 32-bit
    (fixed summation order); bfloat16 operands accumulate in 32-bit on the tensor cores: up to 16 rows
    through the weight-streaming kernel, more through the vendor's library (or, where ``_GEMM_POLICY`` says so,
    the own tcgen05 kernel from 128 rows on).  ``x`` may be a :class:`NormedInput`."""
    if isinstance(x, NormedInput):
        if x.shape[0] >= _TCGEN05_MIN_ROWS:
            out = _tcgen05_linear(x, w, out_dtype or x.dtype, 0, w.shape[0])
        else:
            out = _decode_linear(x, w, out_dtype or x.dtype, 0, w.shape[0])
        return out if out is not None else linear(x.materialize(), w, out_dtype)
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], f"linear: shapes {tuple(x.shape)} and {tuple(w.shape)} do not match")
    _need(x.dtype == w.dtype, f"linear: operand types differ ({x.dtype}, {w.dtype})")
    _need(x.stride(1) == 1 and w.is_contiguous(), "linear: operands must have unit inner stride")
    out_dtype = out_dtype or x.dtype
    m, k = x.shape
    n = w.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        code = _launch("llm_gemm_simt", _ptr(x), _F32, _ptr(w), _F32, _ptr(out), _code(out_dtype), m, n, k, x.stride(0), k, n, _stream())
        _check(code, "linear (float32)")
        return out
    _need(x.dtype == torch.bfloat16, f"linear: element type {x.dtype} is not supported")
    if m <= _DECODE_LINEAR_MAX_ROWS:
        out = _decode_linear(x, w, out_dtype, 0, n)
        if out is not None:
            return out
    if m >= _TCGEN05_MIN_ROWS and not _library_is_faster("plain", m):
        out = _tcgen05_linear(x, w, out_dtype, 0, n)
        if out is not None:
            return out
    return _library_linear(x, w, out_dtype)


# Which of two ways a bfloat16 product of many rows takes: the own tcgen05 kernel or the vendor's library (as the
# reference's F.linear).  Measured on a B200 in graphs of back-to-back products of one shape (hidden 2048, feed-forward
# 5632; own / library in microseconds): 128 rows 13.9 / 5.3 (stacked projection), 30.8 / 9.5 (down); 2,048 rows 28.7 /
# 17.6, 17.0 / 14.5 (output), 36.2 / 31.8; 8,192 rows 87.8 / 58.6, 189.6 / 129.9: the library's tiles of 256 rows over
# two SMs need half the operand traffic per SM of the own kernel's 128-row tiles, and it splits small grids along k.
# Gate and up with SwiGLU in the product's end, against the library's product and an activation kernel: 52 / 45 at 1,024
# rows, 55 / 62 at 1,536, 72 / 85 at 2,048, 285 / 315 at 8,192.  So "auto" gives plain products to the library and the
# gated one to the own kernel from _SWIGLU_OWN_MIN_ROWS rows on; "own" and "library" force one way (also through the
# environment variable LLMSERVE_B200_GEMM; the tests run the own kernel at every shape).
_GEMM_POLICY = os.environ.get("LLMSERVE_B200_GEMM", "auto")
_SWIGLU_OWN_MIN_ROWS = 1536


def _library_is_faster(kind: str, m: int) -> bool:
    if _GEMM_POLICY != "auto":
        return _GEMM_POLICY == "library"
    return kind == "plain" or m < _SWIGLU_OWN_MIN_ROWS


def _library_linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    library()  # the engine never runs without its kernels, even where a matrix product is the vendor's
    if out_dtype == torch.float32 and x.dtype == torch.bfloat16:
        return torch.mm(x, w.t(), out_dtype=torch.float32)  # the 32-bit sums as they are, not rounded on the way
    out = torch.matmul(x, w.t())
    return out if out_dtype == out.dtype else out.to(out_dtype)


def _tcgen05_linear(x, w, out_dtype, mode: int, n_out: int, up_offset: int = 0):
    """The tcgen05 + TMA product for many rows (``x`` a tensor or a :class:`NormedInput`); None if
    it refuses the shape."""
    scaled = isinstance(x, NormedInput)
    xt = x.xw if scaled else x
    m, k = xt.shape
    if not (xt.dtype == torch.bfloat16 and xt.stride(1) == 1 and w.is_contiguous()):
        return None
    out = torch.empty((m, n_out), dtype=out_dtype, device=xt.device)
    code = _launch(
        "llm_gemm_tcgen05_fused", _ptr(xt), xt.stride(0), _ptr(w), _ptr(out), _code(out_dtype), m, n_out, k, n_out, mode,
        up_offset, _ptr(x.ss) if scaled else None, x.ss.shape[0] if scaled else 0, x.eps if scaled else 0.0, None, None, None,
        None, _error_flag_ptr(), _stream(),
    )
    if code == 10002:
        add_launches(-1)
        return None
    _check(code, "linear (tcgen05)")
    return out


def linear_qkv_rope(
    x,
    w_in: torch.Tensor,
    positions: torch.Tensor,
    table: torch.Tensor | None,
    slot_map: torch.Tensor | None,
    pool: torch.Tensor | None,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    write_kv: bool = True,
) -> torch.Tensor | None:
    """For few bfloat16 rows, one kernel instead of three: the stacked query/key/value projection,
    the rotary encoding of query and key heads, and the write of keys and values into their
    pages.  Returns the rotated queries ``[M, num_heads * head_dim]``, or None when the shape is
    not taken (the caller then runs the product, the rotation and the write one by one)."""
    scaled = isinstance(x, NormedInput)
    xt = x.xw if scaled else x
    m, k = xt.shape
    if not (xt.dtype == torch.bfloat16 and m <= _DECODE_LINEAR_MAX_ROWS and xt.stride(1) == 1 and w_in.is_contiguous()):
        return None
    if head_dim % 16 or (table is not None and (table.dtype != torch.float32 or table.shape[1] != head_dim)):
        return None
    kv = num_kv_heads if write_kv else 0
    _need(w_in.shape[0] == (num_heads + 2 * kv) * head_dim, "the stacked projection does not match the heads")
    if kv:
        _i32(slot_map, "slot_map")
        _need(pool.dtype == torch.bfloat16 and pool.is_contiguous() and tuple(pool.shape[1:3]) == (2, kv) and pool.shape[4] == head_dim, "the pool plane does not match the heads")
    q = torch.empty((m, num_heads * head_dim), dtype=torch.bfloat16, device=xt.device)
    code = _launch(
        "llm_linear_decode_qkv", _ptr(xt), _ptr(w_in), _ptr(q), m, k, xt.stride(0), _ptr(x.ss) if scaled else None,
        x.ss.shape[0] if scaled else 0, x.eps if scaled else 0.0, _ptr(positions), _ptr(table),
        table.shape[0] if table is not None else 0, _ptr(slot_map) if kv else None, _ptr(pool) if kv else None, num_heads, kv,
        head_dim, pool.shape[3] if kv else 1, _error_flag_ptr(), _stream(),
    )
    if code == 10002:
        add_launches(-1)
        return None
    _check(code, "linear_qkv_rope")
    return q


def linear_swiglu(x, w_gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(x @ gate^T) * (x @ up^T)`` for ``w_gate_up = [gate rows | up rows]``: one kernel for
    few bfloat16 rows, else a product followed by the activation kernel."""
    inter = w_gate_up.shape[0] // 2
    xt = x.xw if isinstance(x, NormedInput) else x
    if xt.dtype == torch.bfloat16 and xt.shape[0] <= _DECODE_LINEAR_MAX_ROWS:
        out = _decode_linear(x, w_gate_up, torch.bfloat16, 1, inter, up_offset=inter)
        if out is not None:
            return out
    if xt.dtype == torch.bfloat16 and xt.shape[0] >= _TCGEN05_MIN_ROWS:
        scaled = isinstance(x, NormedInput)  # the factored form goes the own way: the library knows nothing of it
        if scaled or not _library_is_faster("swiglu", xt.shape[0]):
            out = _tcgen05_linear(x, w_gate_up, torch.bfloat16, 1, inter, up_offset=inter)
            if out is not None:
                return out
        if not scaled:
            return swiglu(_library_linear(x, w_gate_up, torch.bfloat16))
    return swiglu(linear(x, w_gate_up))


def rope_kv_write(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    table: torch.Tensor | None,
    slot_map: torch.Tensor | None,
    pool: torch.Tensor | None,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    write_kv: bool = True,
) -> None:
    """Rotate the query heads of each ``qkv`` row in place by its position's table row, and (with
    ``write_kv``) store the rotated key heads and the value heads at the row's slot of ``pool``
    ``[pages, 2, kv_heads, page_size, head_dim]``.  ``table`` None: no rotation."""
    n = qkv.shape[0]
    width = (num_heads + (2 * num_kv_heads if write_kv else 0)) * head_dim
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= width, f"qkv rows must hold {width} elements")
    _i32(positions, "positions")
    table_rows = 0
    if table is not None:
        _need(table.dtype == torch.float32 and table.is_contiguous() and table.shape[1] == head_dim, "the rotary table must be float32 [positions, head_dim]")
        table_rows = table.shape[0]
    page_size = 1
    if write_kv:
        _i32(slot_map, "slot_map")
        _need(pool.dtype == qkv.dtype and pool.is_contiguous() and pool.dim() == 5, "the pool plane must be contiguous [pages, 2, kv_heads, page_size, head_dim] of the qkv type")
        _need(pool.shape[1] == 2 and pool.shape[2] == num_kv_heads and pool.shape[4] == head_dim, "the pool plane does not match the heads")
        page_size = pool.shape[3]
    code = _launch("llm_rope_kv_write", 
        _ptr(qkv), _code(qkv.dtype), qkv.stride(0), _ptr(positions), _ptr(table), table_rows, _ptr(slot_map),
        _ptr(pool), n, num_heads, num_kv_heads if write_kv else 0, head_dim, page_size, int(write_kv), _stream(),
    )
    _check(code, "rope_kv_write")


def rope_inplace(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> None:
    """Rotate ``x [N, heads, head_dim]`` (a view with unit inner strides per head) in place."""
    if x.shape[1] == 0 or x.shape[0] == 0:
        return
    _need(x.dim() == 3 and x.stride(2) == 1 and x.stride(1) == x.shape[2], "rope_inplace: x must be [N, heads, head_dim] with packed heads")
    flat = x.as_strided((x.shape[0], x.shape[1] * x.shape[2]), (x.stride(0), 1), x.storage_offset())
    rope_kv_write(flat, positions, table, None, None, x.shape[1], 0, x.shape[2], write_kv=False)


def paged_attention(
    qkv: torch.Tensor,
    pool: torch.Tensor,
    page_table: torch.Tensor,
    ctx,
    *,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int | None = None,
) -> torch.Tensor:
    """Attention of every new token over its request's cached keys and values.

    ``qkv`` rows start with the (already rotated) query heads; the new tokens' keys and values are
    already in ``pool``.  ``ctx`` gives ``token_request``, ``cu_tokens`` and ``context_lens``:
    the token at flat row t of request r stands at position
    ``context_lens[r] - (cu_tokens[r+1] - cu_tokens[r]) + (t - cu_tokens[r])`` and sees the keys
    at positions ``max(0, p - window + 1) .. p``.  Returns ``[N, num_heads * head_dim]``."""
    n = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] >= num_heads * head_dim, "qkv rows must start with the query heads")
    _need(pool.dtype == qkv.dtype and pool.is_contiguous() and pool.dim() == 5, "the pool plane must be contiguous and of the query type")
    _need(tuple(pool.shape[1:3]) == (2, num_kv_heads) and pool.shape[4] == head_dim, "the pool plane does not match the heads")
    _need(1 <= head_dim <= 256, f"head_dim {head_dim} is not supported (up to 256)")
    _i32(page_table, "page_table")
    out = torch.empty((n, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if qkv.dtype == torch.bfloat16 and head_dim in _MMA_HEAD_DIMS and not _FORCE_GENERIC_ATTENTION:
        group = num_heads // num_kv_heads
        # requests that bring at least 128 tokens: 128-token tiles of one head on tcgen05 (head sizes 64 and 128, pages
        # of 8 to 64 keys); the others: rows of (token, group member) on mma.sync, 64 rows a tile or the split-key shape
        tc_min = 0
        if head_dim in _TC_ATTENTION_HEAD_DIMS and pool.shape[3] in _TC_ATTENTION_PAGE_SIZES and _TC_ATTENTION_ENABLED:
            tc_min = _TC_ATTENTION_MIN_TOKENS
        num_requests, tc_longest, small, max_rows_large, other_rows = _attention_route(ctx, group, tc_min)
        if tc_longest:
            code = _launch(
                "llm_attention_tcgen05", _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(pool), pool.shape[0],
                _ptr(page_table), page_table.shape[1], _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), num_requests, n, num_heads,
                num_kv_heads, head_dim, pool.shape[3], int(window or 0), float(scale), tc_min, tc_longest, _error_flag_ptr(),
                _stream(),
            )
            if code == 10002:  # the kernel does not take this layout: all requests go the other way
                add_launches(-1)
                tc_min = 0
                num_requests, tc_longest, small, max_rows_large, other_rows = _attention_route(ctx, group, 0)
            else:
                _check(code, "paged_attention (tcgen05)")
        if not other_rows:
            return out
        splits = 1
        if small:
            longest = getattr(ctx, "max_context_len", None) or int(ctx.context_lens.max())
            useful = -(-longest // _SMALL_TILE_KEYS)
            splits = max(1, min(useful, _sm_count() // (small * num_kv_heads), 32))  # one CTA per SM at most: all run at once
            # the partial results are indexed by token over the whole step: beside a long portion of a prompt the
            # decode tokens are not split so finely that the scratch memory grows past a few megabytes
            splits = min(splits, max(1, _SPLIT_SCRATCH_BYTES // (n * num_heads * head_dim * 4)))
        scratch_o = scratch_ml = counters = None
        if splits > 1:
            counters = _split_counters(qkv.device, num_requests * num_kv_heads)
            scratch_o = torch.empty((n * num_heads * splits * head_dim,), dtype=torch.float32, device=qkv.device)
            scratch_ml = torch.empty((n * num_heads * splits * 2,), dtype=torch.float32, device=qkv.device)
        code = _launch(
            "llm_attention_mma_routed", _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(pool), _ptr(page_table),
            page_table.shape[1], _ptr(ctx.token_request), _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), num_requests, n,
            num_heads, num_kv_heads, head_dim, pool.shape[3], int(window or 0), float(scale), max_rows_large,
            int(small > 0), splits, 1, _ptr(scratch_o), _ptr(scratch_ml), _ptr(counters), tc_min if tc_longest else 0, _stream(),
        )
        add_launches((max_rows_large > 0) + (small > 0) - 1)
        _check(code, "paged_attention (tensor cores)")
        return out
    code = _launch(
        "llm_attention_generic", _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(pool), _code(qkv.dtype),
        _ptr(page_table), page_table.shape[1], _ptr(ctx.token_request), _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), n,
        num_heads, num_kv_heads, head_dim, pool.shape[3], int(window or 0), float(scale), _stream(),
    )
    _check(code, "paged_attention")
    return out


def _attention_route(ctx, group: int, tc_min: int) -> tuple[int, int, int, int, bool]:
    """Which kernels a step's requests go to, from how many tokens each brings: (requests, most tokens of a request
    that the tcgen05 kernel takes (0: none), requests of the split-key shape, most rows of a request of the 64-row
    shape (0: none), any request for the mma.sync kernels at all).  The same for every layer of a step, so it is
    worked out once and kept on the step's context."""
    kept = ctx.__dict__.setdefault("_attention_routes", {}) if hasattr(ctx, "__dict__") else {}
    route = kept.get((group, tc_min))
    if route is None:
        cu = getattr(ctx, "host_cu_tokens", None)
        if cu is None:
            cu = ctx.cu_tokens.tolist()
        lens = [b - a for a, b in zip(cu, cu[1:])]
        tc_longest = max((x for x in lens if tc_min and x >= tc_min), default=0)
        rows = [x * group for x in lens if not (tc_longest and x >= tc_min)]
        small = sum(1 for x in rows if x <= _SMALL_ROWS)
        max_rows_large = max((x for x in rows if x > _SMALL_ROWS), default=0)
        route = kept[(group, tc_min)] = (len(lens), tc_longest, small, max_rows_large, bool(rows))
    return route


_counters: dict = {}


def _split_counters(device, n: int) -> torch.Tensor:
    """Zeroed int32 counters that the split-key attention uses and leaves zeroed; one buffer per
    device, made on first use (outside any graph capture: the first step of a shape runs eagerly)."""
    buf = _counters.get(device)
    if buf is None or buf.numel() < n:
        buf = torch.zeros(max(n, 16384), dtype=torch.int32, device=device)
        _counters[device] = buf
    return buf


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate_up[:, :I]) * gate_up[:, I:]`` computed in 32-bit -> ``[N, I]``."""
    _need(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0, "gate_up must be a contiguous [N, 2 I] matrix")
    n, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(_launch("llm_swiglu", _ptr(gate_up), _ptr(out), _code(gate_up.dtype), n, inter, _stream()), "swiglu")
    return out


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``x [N, C] += bias [C]`` in place (summed in 32-bit, rounded once); returns ``x``."""
    _need(x.dim() == 2 and x.stride(1) == 1 and bias.dim() == 1 and bias.numel() == x.shape[1] and bias.is_contiguous(),
          "add_bias: x [N, C] with unit inner stride and bias [C]")
    _need(bias.dtype == x.dtype, f"add_bias: the bias is {bias.dtype}, the rows are {x.dtype}")
    _check(_launch("llm_add_bias", _ptr(x), _code(x.dtype), x.shape[0], x.shape[1], x.stride(0), _ptr(bias), _stream()), "add_bias")
    return x


def fetch_words(host: torch.Tensor, dev: torch.Tensor, head: torch.Tensor | None = None) -> None:
    """``dev[:] = host`` for int32 arrays of one size, ``host`` in pinned host memory: the kernel reads the host's
    memory itself.  Where ``head`` (int32, on the device) is given, the first ``len(head)`` words come from it
    instead.  The host must leave ``host`` alone until the stream has passed this point."""
    _need(host.dtype == torch.int32 and dev.dtype == torch.int32 and host.numel() == dev.numel(), "two int32 arrays of one size")
    _need(host.is_pinned() and dev.is_cuda and host.is_contiguous() and dev.is_contiguous(), "from pinned host memory to the device")
    if head is not None:
        _need(head.dtype == torch.int32 and head.is_cuda and head.is_contiguous() and head.numel() <= dev.numel(), "head: int32 on the device")
    code = _launch("llm_fetch_words", _ptr(host), _ptr(dev), _ptr(head), 0 if head is None else head.numel(), host.numel(), _stream())
    _check(code, "fetch_words")


def _host_out(host_out: torch.Tensor | None, rows: int) -> int | None:
    if host_out is None:
        return None
    _need(host_out.dtype == torch.int32 and host_out.numel() == rows and host_out.is_pinned() and host_out.is_contiguous(),
          "host_out must be int32 [rows] in pinned host memory")
    return host_out.data_ptr()


def argmax(logits: torch.Tensor, host_out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest logit of each row (the lowest index among equals) -> int32 ``[rows]``.  ``host_out``
    (int32 ``[rows]`` in pinned host memory) gets the same from the kernel itself, valid once the stream has
    passed this point."""
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(), "logits must be a contiguous float32 matrix")
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    _check(_launch("llm_argmax", _ptr(logits), logits.shape[0], logits.shape[1], _ptr(out), _host_out(host_out, logits.shape[0]), _stream()), "argmax")
    return out


def sample(
    logits: torch.Tensor,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    seeds: torch.Tensor,
    counters: torch.Tensor,
    host_out: torch.Tensor | None = None,
) -> torch.Tensor:
    """One token per row: argmax where ``temperature <= 0``, else a draw from
    ``softmax(logits / temperature)`` cut by ``top_k`` (0: off) and ``top_p`` (1: off) at the
    uniform number that ``(seed, counter)`` gives.  All parameter tensors are ``[rows]`` on the
    device: float32, int32, float32, int64, int64.  ``host_out``: as for ``argmax``."""
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(), "logits must be a contiguous float32 matrix")
    rows = logits.shape[0]
    for t, dt, name in ((temperature, torch.float32, "temperature"), (top_k, torch.int32, "top_k"), (top_p, torch.float32, "top_p"), (seeds, torch.int64, "seeds"), (counters, torch.int64, "counters")):
        _need(t.dtype == dt and t.numel() == rows and t.is_contiguous() and t.is_cuda, f"{name} must be {dt} [rows] on the device")
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    code = _launch("llm_sample", 
        _ptr(logits), rows, logits.shape[1], _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(seeds), _ptr(counters),
        _ptr(out), _host_out(host_out, rows), _stream(),
    )
    _check(code, "sample")
    return out
