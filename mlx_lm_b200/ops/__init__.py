"""Python face of the CUDA kernels.

Each function checks what the kernel cannot check for itself (device, dtype,
contiguity, matching sizes), passes raw pointers and the CUDA stream to the
``extern "C"`` launcher of the kernel's library and raises on a non-zero
return code with the launcher's own message.  There is no fallback: without
a CUDA device, or if a library cannot be built, these functions raise.

Tensors are torch tensors used as typed device buffers; no torch operator
runs in here.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import build

import os as _os

F32, BF16 = 0, 1


def _read_activations():
    """``{name: code}`` from the one list of epilogue activations, csrc/activations.cuh, which every linear
    kernel includes: lines ``X(IDENTIFIER, code, name)``."""
    import os
    import re

    with open(os.path.join(build.CSRC, "activations.cuh")) as f:
        text = f.read()
    body = text[text.index("#define MLXB_ACTIVATION_LIST"):]
    body = body[:body.index("\n\n")]
    found = {m.group(3): int(m.group(2)) for m in re.finditer(r"X\((\w+),\s*(\d+),\s*(\w+)\)", body)}
    if "none" not in found or sorted(found.values()) != list(range(len(found))):
        raise RuntimeError(f"csrc/activations.cuh: cannot read the list of activations ({found})")
    return found


ACTIVATION_CODES = _read_activations()
EPI_NONE = ACTIVATION_CODES["none"]
EPI_GELU_NEW = ACTIVATION_CODES["gelu_new"]

_DT = {torch.float32: F32, torch.bfloat16: BF16}

# kernel sources that only a bfloat16 run launches from: a float32 run neither compiles nor loads them
BF16_ONLY_LIBS = frozenset({"gemm_smallm", "gemm_smallm_fold", "gemm_tcgen05", "attention_prefill",
                            "attention_prefill_tc", "attention_wide_tc", "moe_tcgen05"})

# status word bits set by kernels (csrc/common.cuh)
ST_TOKEN_RANGE, ST_POSITION_RANGE, ST_PAGE_RANGE, ST_WAIT_TIMEOUT = 1, 2, 4, 8


class KernelError(RuntimeError):
    pass


def describe_status(word: int) -> str:
    """The bits of a status word in words."""
    names = [n for b, n in ((ST_TOKEN_RANGE, "token id out of range"),
                            (ST_POSITION_RANGE, "position without a page or out of range"),
                            (ST_PAGE_RANGE, "page id outside the pool"),
                            (ST_WAIT_TIMEOUT, "a bounded wait in a kernel gave up")) if word & b]
    return "; ".join(names) or f"status {word}"


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError(
            "mlx_lm_b200 runs on a CUDA device (NVIDIA B200, sm_100a) only: no device is visible and "
            "there is no CPU path")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"unsupported dtype {dt}: the engine runs in float32 or bfloat16") from None


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dt, what: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}, not on a CUDA device")
    if dt is not None and t.dtype != dt:
        raise KernelError(f"{what}: dtype {t.dtype}, expected {dt}")


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")
    return t.stride(0)


_fn_cache = {}


def _fn(libname: str, fname: str, argtypes):
    key = (libname, fname)
    hit = _fn_cache.get(key)
    if hit is None:
        lib = build.load(libname)
        f = getattr(lib, fname)
        f.argtypes = argtypes
        f.restype = c_int
        hit = _fn_cache[key] = (f, lib)
    return hit


launch_count = 0   # kernel launches issued through this module (bench.py reads and resets it)
_recording = None  # while a list: every launch is appended as (launcher, library, name, arguments, label)
_label = None      # what the launches that follow are part of: (name, flops, bytes), set by the parts


def label(name: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
    """Name the work the following launches belong to (a part's tensor name, say) with the floating-point
    operations and the bytes it has to move, where the caller knows them.  Recorded launches carry the label;
    the measuring tools group and rate kernels by it.  Costs nothing when nothing is recorded."""
    global _label
    if _recording is not None:
        _label = (name, float(flops), float(nbytes))


def recording() -> bool:
    """Whether launches are being noted (and labels kept) right now."""
    return _recording is not None


def start_recording() -> None:
    """Begin to note every launch with its raw arguments, so that a step of the same shape can be
    re-issued later without going through the checks and the parts again (``replay``)."""
    global _recording, _label
    _recording = []
    _label = None


def stop_recording():
    global _recording
    calls, _recording = _recording, None
    return calls


def replay(calls) -> None:
    """Re-issue recorded launches.  The caller guarantees that every buffer they name is still where it was."""
    global launch_count
    for f, lib, fname, args, _ in calls:
        rc = f(*args)
        if rc != 0:
            msg = lib.mlxb_last_error()
            raise KernelError(f"{fname} failed ({rc}): {msg.decode() if msg else ''}")
    launch_count += len(calls)


def _call(libname: str, fname: str, argtypes, *args) -> None:
    global launch_count
    f, lib = _fn(libname, fname, argtypes)
    launch_count += 1
    rc = f(*args)
    if rc != 0:
        msg = lib.mlxb_last_error()
        raise KernelError(f"{fname} failed ({rc}): {msg.decode() if msg else ''}")
    if _recording is not None:
        _recording.append((f, lib, fname, args, _label))


# --------------------------------------------------------------------------
# embedding + position add

_EMBED_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
               c_void_p, c_int, c_void_p, c_void_p]


def embed_pos(tokens, positions, wte, wpe, out, status, stream, scale: float = 1.0, freq=None) -> None:
    """``out[t] = wte[tokens[t]] * scale + wpe[positions[t]]`` (``wpe`` may be None).  ``out`` has the tables'
    dtype, or is float32 over bfloat16 tables (a residual stream kept in float32).  ``freq`` (float32
    ``[ceil(width / 2)]``): a sinusoid of the position is added, column ``2i`` gets ``sin(p * freq[i])`` and
    column ``2i + 1`` the cosine of the same angle."""
    _need(tokens, torch.int32, "embed_pos tokens")
    out_f32 = int(out.dtype == torch.float32 and wte.dtype == torch.bfloat16)
    if not out_f32:
        _need(wte, out.dtype, "embed_pos wte")
    T, D = out.shape
    if wte.shape[1] != D or not wte.is_contiguous() or not out.is_contiguous():
        raise KernelError(f"embed_pos: table {tuple(wte.shape)} against output {tuple(out.shape)}")
    if wpe is not None:
        _need(positions, torch.int32, "embed_pos positions")
        _need(wpe, wte.dtype, "embed_pos wpe")
        if wpe.shape[1] != D or not wpe.is_contiguous():
            raise KernelError(f"embed_pos: position table {tuple(wpe.shape)} against width {D}")
    if freq is not None:
        _need(positions, torch.int32, "embed_pos positions")
        _need(freq, torch.float32, "embed_pos freq")
        if freq.numel() != (D + 1) // 2 or not freq.is_contiguous():
            raise KernelError(f"embed_pos: {freq.numel()} frequencies for width {D}")
    _call("embed", "mlxb_embed_pos", _EMBED_ARGS, dtype_code(wte.dtype), _p(tokens), _p(positions), _p(wte),
          _p(wpe), _p(out), T, D, wte.shape[0], 0 if wpe is None else wpe.shape[0], scale, _p(status), out_f32,
          _p(freq), stream)


def gather_tokens(src, index, dst, status, stream) -> None:
    """``dst[i] = src[index[i]]`` where ``index[i] >= 0`` (int32 all): tokens a step has just sampled, handed
    to the next step on the device."""
    for t, what in ((src, "src"), (index, "index"), (dst, "dst")):
        _need(t, torch.int32, f"gather_tokens {what}")
    if index.numel() < dst.numel():
        raise KernelError(f"gather_tokens: {index.numel()} indices for {dst.numel()} tokens")
    _call("embed", "mlxb_gather_tokens", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
          _p(src), src.numel(), _p(index), _p(dst), dst.numel(), _p(status), stream)


# --------------------------------------------------------------------------
# norms

_LN_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]


def layernorm(x, gain, bias, out, eps: float, stream, rows=None) -> None:
    """``out[r] = LayerNorm(x[rows[r]] if rows is given else x[r])``; statistics in float32."""
    _need(x, out.dtype, "layernorm x")
    _need(gain, torch.float32, "layernorm gain")
    if bias is not None:
        _need(bias, torch.float32, "layernorm bias")
    R, D = out.shape
    if x.shape[1] != D or gain.numel() != D or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError(f"layernorm: x {tuple(x.shape)}, gain {tuple(gain.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _need(rows, torch.int32, "layernorm rows")
        if rows.numel() != R:
            raise KernelError(f"layernorm: {rows.numel()} row indices for {R} output rows")
    elif x.shape[0] != R:
        raise KernelError(f"layernorm: {x.shape[0]} input rows for {R} output rows")
    _call("norm", "mlxb_layernorm", _LN_ARGS, dtype_code(out.dtype), _p(x), _p(rows), _p(gain), _p(bias), _p(out),
          R, D, eps, stream)


_STATS_ARGS = [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]


def row_stats(x, stats, eps: float, stream) -> None:
    """``stats[r] = (mean, 1/sqrt(var + eps))`` of the bfloat16 rows of ``x`` (float32 ``[R, 2]``): what the
    epilogue of a linear layer with a folded LayerNorm needs of the rows."""
    _need(x, torch.bfloat16, "row_stats x")
    _need(stats, torch.float32, "row_stats stats")
    R, D = x.shape
    if stats.shape != (R, 2) or not stats.is_contiguous():
        raise KernelError(f"row_stats: statistics {tuple(stats.shape)} for {R} rows")
    _call("norm", "mlxb_row_stats", _STATS_ARGS, _p(x), _p(stats), R, D, _rows(x, "row_stats x"), eps, stream)


_GATHER_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]


def gather_rows(x, rows, out, stream) -> None:
    """``out[r] = x[rows[r]]`` (a row index outside ``x`` gives a row of zeros)."""
    _need(x, out.dtype, "gather_rows x")
    _need(rows, torch.int32, "gather_rows rows")
    R, D = out.shape
    if x.dim() != 2 or x.shape[1] != D or rows.numel() != R or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError(f"gather_rows: x {tuple(x.shape)}, {rows.numel()} indices, out {tuple(out.shape)}")
    _call("norm", "mlxb_gather_rows", _GATHER_ARGS, dtype_code(out.dtype), _p(x), _p(rows), _p(out), R, D, x.shape[0],
          stream)


# --------------------------------------------------------------------------
# linear layers

_SIMT_ARGS = [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
              c_int, c_void_p]


def linear_generic(x, w, bias, out, stream, epilogue: int = EPI_NONE, residual=None) -> None:
    """``out = epilogue(x @ w.T + bias) + residual`` on the CUDA cores in float32 arithmetic.

    ``x [M,K]`` and ``w [N,K]`` (rows are output features) share a dtype; ``out [M,N]`` has that dtype or
    float32, and ``residual [M,N]`` has the dtype of ``out``; ``bias`` is float32."""
    _need(x, None, "linear x")
    _need(w, x.dtype, "linear w")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lda, ldc = _rows(x, "linear x"), _rows(out, "linear out")
    out_f32 = 0
    if out.dtype != x.dtype:
        if out.dtype != torch.float32:
            raise KernelError(f"linear: output dtype {out.dtype} for input dtype {x.dtype}")
        out_f32 = 1
    if bias is not None:
        _need(bias, torch.float32, "linear bias")
        if bias.numel() != N:
            raise KernelError(f"linear: bias of {bias.numel()} for {N} outputs")
    if residual is not None:
        _need(residual, out.dtype, "linear residual")
        if residual.shape != out.shape or _rows(residual, "linear residual") != ldc:
            raise KernelError("linear: residual must have the output's shape and row stride")
    _call("gemm_simt", "mlxb_linear_simt", _SIMT_ARGS, dtype_code(x.dtype), out_f32, _p(x), _p(w), _p(bias),
          _p(residual), _p(out), M, N, K, lda, ldc, epilogue, stream)


_SMALLM_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                c_void_p]

SMALL_M = 64

_SMALLM_FOLD_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                     c_void_p, c_float, c_void_p]


def _fold_args(fold, N: int, what: str):
    colsum, eps = fold
    _need(colsum, torch.float32, what + " column sums")
    if colsum.numel() != N or not colsum.is_contiguous():
        raise KernelError(f"{what}: {colsum.numel()} column sums for {N} outputs")
    return colsum, float(eps)


def linear_few_rows(x, w, bias, out, stream, epilogue: int = EPI_NONE, residual=None, fold=None) -> None:
    """``linear_generic``'s contract for bfloat16 and at most 64 rows: the weight is streamed from HBM once
    with 16-byte loads and multiplied on the tensor cores (csrc/gemm_smallm.cuh).  ``K`` and the row stride of
    ``x`` must be multiples of 8.

    ``fold = (colsum, eps)``: ``x`` holds the rows before a LayerNorm that has been folded into ``w`` and ``bias``
    (``parts.linear.Linear.fold_norm``); the kernel computes ``rstd (x w^T - mean colsum) + bias`` with the
    rows' mean and 1/std found on the way."""
    _need(x, torch.bfloat16, "linear x")
    _need(w, torch.bfloat16, "linear w")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lda, ldc = _rows(x, "linear x"), _rows(out, "linear out")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"linear: output dtype {out.dtype}")
    if bias is not None:
        _need(bias, torch.float32, "linear bias")
        if bias.numel() != N:
            raise KernelError(f"linear: bias of {bias.numel()} for {N} outputs")
    if residual is not None:
        _need(residual, out.dtype, "linear residual")
        if residual.shape != out.shape or _rows(residual, "linear residual") != ldc:
            raise KernelError("linear: residual must have the output's shape and row stride")
    if fold is not None:
        colsum, eps = _fold_args(fold, N, "linear")
        _call("gemm_smallm_fold", "mlxb_linear_smallm_fold", _SMALLM_FOLD_ARGS, int(out.dtype == torch.float32), _p(x),
              _p(w), _p(bias), _p(residual), _p(out), M, N, K, lda, ldc, epilogue, _p(colsum), eps, stream)
        return
    _call("gemm_smallm", "mlxb_linear_smallm", _SMALLM_ARGS, int(out.dtype == torch.float32), _p(x), _p(w), _p(bias),
          _p(residual), _p(out), M, N, K, lda, ldc, epilogue, stream)


_TC_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
            c_void_p, c_void_p]


_TC_FOLD_ARGS = _TC_ARGS[:-1] + [c_void_p, c_void_p, c_void_p]


def linear_tensor_cores(x, w, bias, out, status, stream, epilogue: int = EPI_NONE, residual=None, fold=None) -> None:
    """``linear_generic``'s contract for bfloat16 and many rows, on tcgen05 tensor cores with TMA-fed
    shared-memory stages and the accumulator in tensor memory (csrc/gemm_tcgen05.cu).  ``K`` and the row
    stride of ``x`` must be multiples of 8.  ``status`` receives ``ST_WAIT_TIMEOUT`` if a bounded wait gives up.

    ``fold = (colsum, stats)``: a LayerNorm folded into ``w`` and ``bias``; ``x`` holds the rows before the norm
    and ``stats`` their ``(mean, rstd)`` from ``row_stats``."""
    _need(x, torch.bfloat16, "linear x")
    _need(w, torch.bfloat16, "linear w")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lda, ldc = _rows(x, "linear x"), _rows(out, "linear out")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"linear: output dtype {out.dtype}")
    if bias is not None:
        _need(bias, torch.float32, "linear bias")
        if bias.numel() != N:
            raise KernelError(f"linear: bias of {bias.numel()} for {N} outputs")
    if residual is not None:
        _need(residual, out.dtype, "linear residual")
        if residual.shape != out.shape or _rows(residual, "linear residual") != ldc:
            raise KernelError("linear: residual must have the output's shape and row stride")
    if fold is not None:
        colsum, stats = fold
        _need(colsum, torch.float32, "linear column sums")
        _need(stats, torch.float32, "linear row statistics")
        if colsum.numel() != N or stats.shape != (M, 2) or not stats.is_contiguous():
            raise KernelError(f"linear: {colsum.numel()} column sums, statistics {tuple(stats.shape)} for {M} x {N}")
        _call("gemm_tcgen05", "mlxb_linear_tcgen05_fold", _TC_FOLD_ARGS, int(out.dtype == torch.float32), _p(x), _p(w),
              _p(bias), _p(residual), _p(out), M, N, K, lda, ldc, epilogue, _p(status), _p(colsum), _p(stats), stream)
        return
    _call("gemm_tcgen05", "mlxb_linear_tcgen05", _TC_ARGS, int(out.dtype == torch.float32), _p(x), _p(w), _p(bias),
          _p(residual), _p(out), M, N, K, lda, ldc, epilogue, _p(status), stream)


_QKV_ARGS = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]


_QKV_FOLD_ARGS = _QKV_ARGS[:-1] + [c_void_p, c_float, c_void_p]
_QKV_TC_FOLD_ARGS = _QKV_ARGS[:-1] + [c_void_p, c_void_p, c_void_p]


def linear_qkv_to_cache(x, w, bias, out, positions, token_req, block_table, k_pool, v_pool, q_width: int, status,
                        stream, fold=None) -> None:
    """The fused ``[q | k | v]`` projection of bfloat16 rows with the cache write in its epilogue: query columns
    go to ``out[:, :q_width]``, key and value columns straight into the pages ``[n_pages, Hkv, page, Dh]`` (the
    other columns of ``out`` are not written).  Up to 64 rows run in the weight-streaming kernel, more in the
    tcgen05 kernel.  ``fold``: ``(colsum, eps)`` as in ``linear_few_rows`` for up to 64 rows, ``(colsum, stats)`` as
    in ``linear_tensor_cores`` for more."""
    _need(x, torch.bfloat16, "linear x")
    _need(w, torch.bfloat16, "linear w")
    _need(out, torch.bfloat16, "linear out")
    _need(k_pool, torch.bfloat16, "linear k_pool")
    M, K = x.shape
    N = w.shape[0]
    n_pages, Hkv, page, Dh = k_pool.shape
    if w.shape[1] != K or not w.is_contiguous() or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if N != q_width + 2 * Hkv * Dh or not (k_pool.is_contiguous() and v_pool.is_contiguous()):
        raise KernelError(f"linear (q|k|v): {N} outputs for {q_width} query columns and pools {tuple(k_pool.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "linear bias")
    if fold is not None and M > SMALL_M:
        colsum, stats = fold
        _need(colsum, torch.float32, "linear column sums")
        if not torch.is_tensor(stats) or stats.dtype != torch.float32 or stats.shape != (M, 2) or not stats.is_contiguous():
            raise KernelError(f"linear (q|k|v): more than {SMALL_M} rows need float32 row statistics [{M}, 2]")
        _call("gemm_tcgen05", "mlxb_linear_tcgen05_qkv_fold", _QKV_TC_FOLD_ARGS, _p(x), _p(w), _p(bias), _p(out), M, N, K,
              _rows(x, "linear x"), _rows(out, "linear out"), _p(positions), _p(token_req), _p(block_table),
              block_table.shape[1], n_pages, page, Hkv, Dh, q_width, _p(k_pool), _p(v_pool), _p(status), _p(colsum),
              _p(stats), stream)
        return
    if fold is not None:
        colsum, eps = _fold_args(fold, N, "linear (q|k|v)")
        _call("gemm_smallm_fold", "mlxb_linear_smallm_qkv_fold", _QKV_FOLD_ARGS, _p(x), _p(w), _p(bias), _p(out), M, N, K,
              _rows(x, "linear x"), _rows(out, "linear out"), _p(positions), _p(token_req), _p(block_table),
              block_table.shape[1], n_pages, page, Hkv, Dh, q_width, _p(k_pool), _p(v_pool), _p(status), _p(colsum), eps,
              stream)
        return
    lib, fn = ("gemm_smallm", "mlxb_linear_smallm_qkv") if M <= SMALL_M else ("gemm_tcgen05", "mlxb_linear_tcgen05_qkv")
    _call(lib, fn, _QKV_ARGS, _p(x), _p(w), _p(bias), _p(out), M, N, K,
          _rows(x, "linear x"), _rows(out, "linear out"), _p(positions), _p(token_req), _p(block_table),
          block_table.shape[1], n_pages, page, Hkv, Dh, q_width, _p(k_pool), _p(v_pool), _p(status), stream)


# --------------------------------------------------------------------------
# paged key/value cache and attention

_KVW_ARGS = [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_void_p, c_void_p, c_int, c_void_p, c_void_p]


def kv_write(k_src, v_src, positions, token_req, block_table, k_pool, v_pool, status, stream) -> None:
    """Store this step's key and value rows into the pages of one layer.

    ``k_src``/``v_src``: ``[T, Hkv*Dh]`` views (same row stride); pools ``[n_pages, Hkv, page, Dh]``."""
    n_pages, Hkv, page, Dh = k_pool.shape
    _need(k_src, k_pool.dtype, "kv_write k")
    _need(v_src, k_pool.dtype, "kv_write v")
    ld = _rows(k_src, "kv_write k")
    if _rows(v_src, "kv_write v") != ld or k_src.shape[1] != Hkv * Dh or v_src.shape != k_src.shape:
        raise KernelError(f"kv_write: k {tuple(k_src.shape)} v {tuple(v_src.shape)} for pool {tuple(k_pool.shape)}")
    if not (k_pool.is_contiguous() and v_pool.is_contiguous() and block_table.is_contiguous()):
        raise KernelError("kv_write: pools and block table must be contiguous")
    _call("attention", "mlxb_kv_write", _KVW_ARGS, dtype_code(k_pool.dtype), _p(k_src), _p(v_src), ld,
          _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n_pages, page, Hkv, Dh,
          _p(k_pool), _p(v_pool), k_src.shape[0], _p(status), stream)


_ATTN_ARGS = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
              c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p]


def _sinks(sinks, n_heads: int, what: str):
    """``sinks``: float32 ``[n_heads]`` or None.  A head's sink is one more term ``exp(sink)`` in the denominator
    of its softmax: it has no key (it is not scaled) and no value."""
    if sinks is None:
        return None
    _need(sinks, torch.float32, what + " sinks")
    if sinks.numel() != n_heads or not sinks.is_contiguous():
        raise KernelError(f"{what}: {sinks.numel()} sinks for {n_heads} heads")
    return sinks.data_ptr()


def _attn_shapes(q, out, k_pool, n_heads, what):
    n_pages, Hkv, page, Dh = k_pool.shape
    _need(q, k_pool.dtype, what + " q")
    _need(out, k_pool.dtype, what + " out")
    if q.shape[1] != n_heads * Dh or out.shape[0] != q.shape[0] or out.shape[1] != n_heads * Dh:
        raise KernelError(f"{what}: q {tuple(q.shape)} out {tuple(out.shape)} for {n_heads} heads of {Dh}")
    return n_pages, Hkv, page, Dh


def attention_generic(q, positions, token_req, block_table, k_pool, v_pool, out, n_heads: int, scale: float,
                      window: int, status, stream, rows=None, sinks=None) -> None:
    """Causal attention of tokens over their requests' pages (float32 math, one warp per token and head).

    ``q``: ``[T, n_heads*Dh]`` view; ``out``: ``[T, n_heads*Dh]``; ``rows``: int32 token indices to run
    (default all ``T``); ``window <= 0`` means all keys."""
    n_pages, Hkv, page, Dh = _attn_shapes(q, out, k_pool, n_heads, "attention")
    n = q.shape[0] if rows is None else rows.numel()
    _call("attention", "mlxb_attention_generic", _ATTN_ARGS, dtype_code(k_pool.dtype), _p(q), _rows(q, "attention q"),
          _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv, Dh,
          window, scale, _p(k_pool), _p(v_pool), _p(out), _rows(out, "attention out"), _p(rows), n, _p(status),
          _sinks(sinks, n_heads, "attention"), stream)


_PRE_ARGS = [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
             c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]

PREFILL_TILE = int(_os.environ.get("MLXB_PREFILL_TILE", "128"))   # queries per CTA of the attention kernels for portions
PREFILL_TC = _os.environ.get("MLXB_PREFILL_TC", "1") != "0"         # heads of 64 in tiles of 128 on the tcgen05 kernel

_PRE_TC_ARGS = [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int,
                c_int, c_void_p]


def attention_portions_supported(dtype, head_dim: int, scale: float = 1.0) -> bool:
    # the tensor-core kernels take the maximum of the raw scores before they scale it: the scale must be positive
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128 and scale > 0


def attention_portions_tc_supported(q, out, k_pool, v_pool, tile_rows: int = 0) -> bool:
    """Whether portions over these pools run on the tcgen05 kernel (``attention_portions``): bfloat16, key heads of 64,
    value rows of 64 columns or a multiple of it, value heads as many as the key heads or a divisor of them, tiles of
    128 queries, pages that are a power of two from 8 to 128, rows in whole 16 bytes."""
    page, Dh = k_pool.shape[2], k_pool.shape[3]
    return (PREFILL_TC and k_pool.dtype == torch.bfloat16 and Dh == 64 and v_pool is not None and v_pool.shape[3] % 64 == 0
            and v_pool.shape[3] > 0 and v_pool.shape[1] > 0 and k_pool.shape[1] % v_pool.shape[1] == 0
            and (tile_rows or PREFILL_TILE) == 128 and 8 <= page <= 128 and page & (page - 1) == 0
            and _rows(q, "attention q") % 8 == 0 and _rows(out, "attention out") % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def attention_portions(q, tiles, n_tiles: int, block_table, k_pool, v_pool, out, n_heads: int, scale: float,
                       window: int, status, stream, tile_rows: int = 0, sinks=None, first_positions=None,
                       keep_first: int = 0, softcap: float = 0.0, gate=None) -> None:
    """Causal attention of prompt portions on tensor cores (bfloat16, csrc/attention_prefill.cu).
    ``keep_first``, ``softcap``, ``gate`` (bfloat16 ``[T, n_heads * 64]``, a sigmoid gate per output column): options of
    the tcgen05 kernel only (``attention_portions_tc_supported``).  So are a value pool with fewer heads than the key
    pool (key heads ``c * Hkv/Hv ..`` read value head ``c``), value rows of a multiple of 64 columns (``out`` is then
    ``[T, n_heads * value row]``) and a float32 ``out``.

    ``tiles``: int32 device tensor ``[n_tiles, 4]``: first token row of the tile, queries in it (1..64),
    block-table row of its request, position of its first query.  ``first_positions``: int32, per block-table
    row the first position this step brings for that request; with it the kernel fetches keys older than the
    step before it waits for the kernel that wrote this step's."""
    if first_positions is not None:
        _need(first_positions, torch.int32, "attention_portions first_positions")
        if first_positions.numel() < block_table.shape[0]:
            raise KernelError(f"attention_portions: {first_positions.numel()} first positions for "
                              f"{block_table.shape[0]} requests")
    Dv, Hv = v_pool.shape[3], v_pool.shape[1]
    plain = Dv == k_pool.shape[3] and Hv == k_pool.shape[1] and out.dtype == k_pool.dtype
    if plain:
        n_pages, Hkv, page, Dh = _attn_shapes(q, out, k_pool, n_heads, "attention_portions")
    else:
        n_pages, Hkv, page, Dh = k_pool.shape
        _need(q, k_pool.dtype, "attention_portions q")
        if (q.shape[1] != n_heads * Dh or out.shape != (q.shape[0], n_heads * Dv) or out.dtype not in (k_pool.dtype, torch.float32)
                or not attention_portions_tc_supported(q, out, k_pool, v_pool, tile_rows)):
            raise KernelError(f"attention_portions: q {tuple(q.shape)}, out {out.dtype} {tuple(out.shape)}, pools "
                              f"{tuple(k_pool.shape)} and {tuple(v_pool.shape)}: value heads or rows that differ from the "
                              f"keys', and float32 results, are options of the tcgen05 kernel")
    _need(tiles, torch.int32, "attention_portions tiles")
    if tiles.numel() < 4 * n_tiles:
        raise KernelError(f"attention_portions: {tiles.numel()} integers for {n_tiles} tiles")
    tile_rows = tile_rows or PREFILL_TILE
    ldq, ldo = _rows(q, "attention q"), _rows(out, "attention out")
    if gate is not None:
        _need(gate, torch.bfloat16, "attention_portions gate")
        if gate.shape[0] != q.shape[0] or gate.shape[1] != n_heads * Dv:
            raise KernelError(f"attention_portions: gate {tuple(gate.shape)} for {n_heads} heads of {Dh}")
    if attention_portions_tc_supported(q, out, k_pool, v_pool, tile_rows):
        _call("attention_prefill_tc", "mlxb_attention_prefill_tc", _PRE_TC_ARGS, _p(q), ldq, q.shape[0], _p(tiles),
              n_tiles, _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv, Dh, window, scale,
              _p(k_pool), _p(v_pool), _p(out), ldo, _p(status), _sinks(sinks, n_heads, "attention_portions"),
              int(keep_first or 0), float(softcap or 0.0), _p(gate), _rows(gate, "attention gate") if gate is not None else 0,
              Hv, Dv, int(out.dtype == torch.float32), stream)
        return
    if keep_first or softcap or gate is not None:
        raise KernelError("attention_portions: kept first positions, a cap and a gate are options of the tcgen05 kernel")
    _call("attention_prefill", "mlxb_attention_prefill", _PRE_ARGS, _p(q), _rows(q, "attention q"), _p(tiles), n_tiles,
          tile_rows, _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv, Dh, window, scale, _p(k_pool),
          _p(v_pool), _p(out), _rows(out, "attention out"), _p(status),
          _sinks(sinks, n_heads, "attention_portions"), _p(first_positions), stream)


_ROWS_ARGS = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
              c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]


# (row, head) pairs from which single-token rows run on the tensor-core kernel: about seven times the number
# of SMs.  Below that the split-key kernel on the CUDA cores is as fast or faster inside a step (GPT-2 medium
# on a B200, 512-token contexts: 16 rows 0.88 against 0.96 ms a step, 32 rows 1.37 both, 64 rows 2.24 against 2.07).
ROWS_MIN_PAIRS = int(_os.environ.get("MLXB_ROWS_MIN_PAIRS", "1024"))


def attention_rows_supported(dtype, head_dim: int, n_rows: int = 1 << 30, n_heads: int = 1, scale: float = 1.0) -> bool:
    """Whether these single-token rows run on the tensor-core kernel (else: ``attention_decode``)."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128
            and n_rows * n_heads >= ROWS_MIN_PAIRS and scale > 0)


_sm_count = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def attention_rows(q, tiles, n_rows: int, block_table, k_pool, v_pool, out, n_heads: int, scale: float, window: int,
                   status, stream, sinks=None) -> None:
    """Attention of rows with a single query each (decode steps) on tensor cores (bfloat16,
    csrc/attention_prefill.cu): ``tiles`` is an int32 device tensor ``[n_rows, 4]`` = (token row, 1, block-table
    row, position), or (token row, 0, 0, 0) for a padding row."""
    n_pages, Hkv, page, Dh = _attn_shapes(q, out, k_pool, n_heads, "attention_rows")
    _need(tiles, torch.int32, "attention_rows tiles")
    if tiles.numel() < 4 * n_rows:
        raise KernelError(f"attention_rows: {tiles.numel()} integers for {n_rows} rows")
    _call("attention_prefill", "mlxb_attention_rows", _ROWS_ARGS, _p(q), _rows(q, "attention q"), _p(tiles), n_rows,
          _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv, Dh, window, scale, _p(k_pool),
          _p(v_pool), _p(out), _rows(out, "attention out"), _p(status), _sinks(sinks, n_heads, "attention_rows"), stream)


_DEC_ARGS = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
             c_void_p, c_void_p]

DECODE_CHUNK = 1024   # key positions per CTA of the single-token attention kernel: a constant, never a function of the batch


def attention_decode_scratch(n_rows: int, n_heads: int, head_dim: int, max_len: int, chunk: int = DECODE_CHUNK) -> int:
    """Float32 elements of scratch memory ``attention_decode`` needs for ``n_rows`` rows."""
    return n_rows * n_heads * ((max_len + chunk - 1) // chunk) * (head_dim + 2)


def attention_decode(q, positions, token_req, block_table, k_pool, v_pool, out, n_heads: int, scale: float,
                     window: int, scratch, counters, max_len: int, status, stream, rows=None,
                     chunk: int = DECODE_CHUNK, sinks=None) -> None:
    """Attention for rows with a single query each (decode steps): keys are cut into chunks of ``chunk``
    positions, one CTA per (chunk, head, row) writes a partial result to ``scratch`` (float32, at least
    ``attention_decode_scratch(...)`` elements) and the CTA that finishes last for a (row, head) combines
    them.  ``counters``: int32, at least rows x heads, zero before the first call (every call leaves it zero)."""
    n_pages, Hkv, page, Dh = _attn_shapes(q, out, k_pool, n_heads, "attention_decode")
    n = q.shape[0] if rows is None else rows.numel()
    n_chunks = (max_len + chunk - 1) // chunk
    _need(scratch, torch.float32, "attention_decode scratch")
    _need(counters, torch.int32, "attention_decode counters")
    if scratch.numel() < n * n_heads * n_chunks * (Dh + 2) or counters.numel() < n * n_heads:
        raise KernelError(f"attention_decode: scratch of {scratch.numel()} floats, {counters.numel()} counters "
                          f"for {n} rows")
    _call("attention", "mlxb_attention_decode", _DEC_ARGS, dtype_code(k_pool.dtype), _p(q), _rows(q, "attention q"),
          _p(rows), _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv,
          Dh, window, scale, _p(k_pool), _p(v_pool), _p(scratch), _p(counters), n_chunks, chunk, _p(out),
          _rows(out, "attention out"), n, _p(status), _sinks(sinks, n_heads, "attention_decode"), stream)


# --------------------------------------------------------------------------
# sampling and logits processors

SAMPLE_WORDS, PROCESS_WORDS = 16, 8

_SAMPLE_ARGS = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                c_void_p, c_void_p, c_void_p, c_int, c_void_p]
SAMPLE_SCRATCH_WORDS_PER_ROW = 65      # csrc/sampling.cu: mlxb_sample_scratch_words


def sample_scratch(n_rows: int, device) -> torch.Tensor:
    """Scratch memory for ``sample`` over up to ``n_rows`` rows: zero, and left zero by every launch.  One per
    stream on which launches may overlap."""
    return torch.zeros(max(1, n_rows) * SAMPLE_SCRATCH_WORDS_PER_ROW, dtype=torch.int32, device=device)


def sample(logits, params, out_token, out_logprob, stream, xtc_special=None, out_logprobs=None, status=None,
           status_out=None, scratch=None) -> None:
    """One token per row of float32 ``logits [R, V]``.

    ``params``: int32 ``[R, 16]`` holding the bit patterns of csrc/sampling.cu's ``SampleParams``;
    ``out_token`` int32 ``[R]``, ``out_logprob`` float32 ``[R]`` (log-probability of the chosen token
    under the unfiltered distribution); ``out_logprobs`` (optional) float32 ``[R, V]`` receives
    ``logits - logsumexp(logits)``.  ``xtc_special``: int32 list of the rows' XTC special tokens, each
    row's record naming its range.  ``status`` / ``status_out`` (int32, one word each): the kernel copies
    the step's status word next to its results, so that the host reads both with one copy.  ``scratch``
    (from ``sample_scratch``, for at least this many rows): with it the rows of a wide vocabulary are cut into
    slices over several thread blocks; the tokens are the same with and without it."""
    _need(logits, torch.float32, "sample logits")
    _need(params, torch.int32, "sample params")
    _need(out_token, torch.int32, "sample out_token")
    _need(out_logprob, torch.float32, "sample out_logprob")
    R, V = logits.shape
    if params.numel() < R * SAMPLE_WORDS or out_token.numel() < R or out_logprob.numel() < R:
        raise KernelError(f"sample: {R} rows need {R * SAMPLE_WORDS} parameter words and {R} outputs")
    ldo = 0
    if out_logprobs is not None:
        _need(out_logprobs, torch.float32, "sample out_logprobs")
        if out_logprobs.shape != logits.shape:
            raise KernelError("sample: out_logprobs must have the shape of logits")
        ldo = _rows(out_logprobs, "sample out_logprobs")
    n_special = 0
    if xtc_special is not None:
        _need(xtc_special, torch.int32, "sample xtc_special")
        n_special = xtc_special.numel()
    if (status is None) != (status_out is None):
        raise KernelError("sample: status and status_out go together")
    if status is not None:
        _need(status, torch.int32, "sample status")
        _need(status_out, torch.int32, "sample status_out")
    _call("sampling", "mlxb_sample", _SAMPLE_ARGS, _p(logits), _rows(logits, "sample logits"), R, V, _p(params),
          _p(xtc_special), n_special, _p(out_token), _p(out_logprob), _p(out_logprobs), ldo, _p(status),
          _p(status_out), _p(scratch), 0 if scratch is None else scratch.numel(), stream)


_PROCESS_ARGS = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]


def process_logits(logits, params, context, bias_index, bias_value, stream) -> None:
    """In place on float32 ``logits [R, V]``: additive bias, then repetition, presence and frequency
    penalties over each row's recent tokens.  ``params`` int32 ``[R, 8]`` (``ProcessParams`` bit
    patterns); ``context`` int32 ``[R, C]`` left-padded with -1; ``bias_index`` int32 / ``bias_value``
    float32 ``[R, B]``."""
    _need(logits, torch.float32, "process_logits logits")
    _need(params, torch.int32, "process_logits params")
    _need(context, torch.int32, "process_logits context")
    R, V = logits.shape
    C = context.shape[1] if context.dim() == 2 else 0
    B = bias_index.shape[1] if bias_index is not None and bias_index.dim() == 2 else 0
    if B:
        _need(bias_index, torch.int32, "process_logits bias_index")
        _need(bias_value, torch.float32, "process_logits bias_value")
    _call("sampling", "mlxb_process_logits", _PROCESS_ARGS, _p(logits), _rows(logits, "process_logits logits"), R, V,
          _p(params), _p(context), C, _p(bias_index) if B else None, _p(bias_value) if B else None, B, stream)


# --------------------------------------------------------------------------
# root-mean-square norms and a float32 residual stream (csrc/rms.cu)

_RMS_ARGS = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_int,
             c_int, c_int, c_int, c_float, c_void_p]

GATE_NONE, GATE_BEFORE, GATE_AFTER = 0, 1, 2


def rmsnorm(x, weight, out, eps: float, stream, offset: float = 0.0, groups: int = 1, period: Optional[int] = None,
            gate=None, gate_mode: int = GATE_NONE, rows=None) -> None:
    """``out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * (offset + weight)`` over float32 rows, the row cut into
    ``groups`` equal parts that are normed each by itself; ``weight`` (float32) repeats every ``period`` columns
    (default: the width).  ``gate`` (``out``'s dtype, the shape of ``x``): ``GATE_BEFORE`` multiplies ``x`` by
    ``silu(gate)`` before the statistics, ``GATE_AFTER`` multiplies the normed value.  ``rows``: int32 indices of
    the input rows to take."""
    _need(x, torch.float32, "rmsnorm x")
    _need(weight, torch.float32, "rmsnorm weight")
    R, D = out.shape
    period = D if period is None else int(period)
    if x.shape[1] != D or weight.numel() != period or D % groups:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)}, weight of {weight.numel()} every {period}, {groups} parts, "
                          f"out {tuple(out.shape)}")
    if rows is not None:
        _need(rows, torch.int32, "rmsnorm rows")
        if rows.numel() != R:
            raise KernelError(f"rmsnorm: {rows.numel()} row indices for {R} output rows")
    elif x.shape[0] != R:
        raise KernelError(f"rmsnorm: {x.shape[0]} input rows for {R} output rows")
    ldg = 0
    if gate is not None:
        _need(gate, out.dtype, "rmsnorm gate")
        if gate.shape != x.shape or gate_mode not in (GATE_BEFORE, GATE_AFTER):
            raise KernelError(f"rmsnorm: gate {tuple(gate.shape)} in mode {gate_mode} for x {tuple(x.shape)}")
        ldg = _rows(gate, "rmsnorm gate")
    elif gate_mode != GATE_NONE:
        raise KernelError("rmsnorm: a gate mode without a gate")
    _call("rms", "mlxb_rmsnorm", _RMS_ARGS, dtype_code(out.dtype), _p(x), _rows(x, "rmsnorm x"), _p(rows), x.shape[0],
          _p(weight), float(offset), period, _p(gate), ldg, gate_mode, _p(out), _rows(out, "rmsnorm out"), R, D,
          groups, float(eps), stream)


_RESUP_ARGS = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_int,
               c_int, c_int, c_void_p]


def residual_update(x, y1, stream, w1=None, y2=None, w2=None, scale: float = 1.0, eps: float = 0.0, cast_out=None) -> None:
    """``x += scale * (f1(y1) + f2(y2))`` in place on float32 rows; ``f_i`` is the RMS norm over the whole row
    with the plain weight ``w_i`` (float32), or the identity where ``w_i`` is None.  ``cast_out``: a copy of the
    new rows in its own dtype."""
    _need(x, torch.float32, "residual_update x")
    _need(y1, torch.float32, "residual_update y1")
    R, D = x.shape
    if y1.shape != x.shape or (y2 is not None and (y2.shape != x.shape or y2.dtype != torch.float32)):
        raise KernelError(f"residual_update: x {tuple(x.shape)}, y1 {tuple(y1.shape)}")
    ldy = _rows(y1, "residual_update y1")
    if y2 is not None and _rows(y2, "residual_update y2") != ldy:
        raise KernelError("residual_update: the two inputs must share a row stride")
    for w in (w1, w2):
        if w is not None:
            _need(w, torch.float32, "residual_update weight")
            if w.numel() != D:
                raise KernelError(f"residual_update: weight of {w.numel()} for width {D}")
    ldc, code = 0, F32
    if cast_out is not None:
        if cast_out.shape != x.shape:
            raise KernelError("residual_update: cast_out must have the shape of x")
        ldc, code = _rows(cast_out, "residual_update cast_out"), dtype_code(cast_out.dtype)
    _call("rms", "mlxb_residual_update", _RESUP_ARGS, code, _p(x), _rows(x, "residual_update x"), _p(y1), _p(w1), _p(y2),
          _p(w2), ldy, float(scale), float(eps), _p(cast_out), ldc, R, D, stream)


def head_difference(a, rep: int, value_dim: int, lam: float, eps: float, post: float, out, stream, token_req=None) -> None:
    """Two score maps over the same values combined per head: ``o = a1 - lam * a2``, divided by its root mean square
    over the head's ``value_dim`` columns (eps inside the root, no weight), times ``post``.  ``a``: float32
    ``[T, 2 * H * value_dim]`` in which the heads of key/value group ``g`` lie as ``[map 1: rep heads | map 2: rep
    heads]``; ``out``: ``[T, H * value_dim]`` in the run's dtype or float32, heads in their own order."""
    _need(a, torch.float32, "head_difference a")
    T, n = out.shape
    if n % value_dim or a.shape != (T, 2 * n) or (n // value_dim) % rep:
        raise KernelError(f"head_difference: a {tuple(a.shape)}, out {tuple(out.shape)}, heads of {value_dim} in groups of {rep}")
    _call("rms", "mlxb_head_difference", [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float,
                                          c_void_p, c_int, c_int, c_void_p],
          dtype_code(out.dtype), _p(a), _rows(a, "head_difference a"), _p(token_req), n // value_dim, int(rep),
          int(value_dim), float(lam), float(eps), float(post), _p(out), _rows(out, "head_difference out"), T, stream)


# --------------------------------------------------------------------------
# layers with a state of fixed size per request (csrc/recurrent.cu)

_CONV_ARGS = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
              c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]


def conv_silu(x, weight, bias, state, slots, positions, token_req, req_first_token, req_first_position, out,
              stream, weight_by_tap=None, activation: bool = True) -> None:
    """Causal convolution over time per channel, then silu: ``out[t, c] = silu(bias[c] + sum_j weight[c, taps-1-j]
    * x(t - j, c))``.  ``x``: ``[T, C]`` view (contiguous rows); ``weight`` float32 ``[C, taps]`` (last column: the
    current token); ``state`` float32 ``[slots, taps-1, C]``: each request's last inputs, read for the rows that
    reach back before the step and brought up to date afterwards (two launches).  ``weight_by_tap``: the same
    weights as float32 ``[taps, C]`` (a copy the caller keeps); with it, and with sizes that allow 16-byte accesses,
    a thread takes eight (float32: four) neighbouring channels.  ``activation=False``: the sum as it is, without the
    silu.  With one tap there is no state: ``state`` may be any float32 tensor ``[slots, 0, C]``."""
    _need(x, out.dtype, "conv x")
    _need(weight, torch.float32, "conv weight")
    _need(state, torch.float32, "conv state")
    T, C = out.shape
    taps = weight.shape[1]
    if x.shape != out.shape or weight.shape[0] != C or state.shape[1:] != (taps - 1, C) or not state.is_contiguous() \
            or not weight.is_contiguous():
        raise KernelError(f"conv: x {tuple(x.shape)}, weight {tuple(weight.shape)}, state {tuple(state.shape)}, "
                          f"out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "conv bias")
    if weight_by_tap is not None:
        _need(weight_by_tap, torch.float32, "conv weight_by_tap")
        if weight_by_tap.shape != (taps, C) or not weight_by_tap.is_contiguous():
            raise KernelError(f"conv: weights by tap {tuple(weight_by_tap.shape)} for {taps} taps of {C} channels")
    _call("recurrent", "mlxb_conv_silu", _CONV_ARGS, dtype_code(out.dtype), _p(x), _rows(x, "conv x"), _p(weight),
          _p(weight_by_tap), _p(bias), taps, C, _p(state), _p(slots), _p(positions), _p(token_req), _p(req_first_token),
          _p(req_first_position), _p(out), _rows(out, "conv out"), T, slots.numel(), int(bool(activation)), stream)


_M2_ARGS = [c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]


def mamba2_scan(xbc, x_off: int, b_off: int, c_off: int, dt_raw, dt_bias, a_log, d_skip, state, slots, token_req,
                req_first_token, y, n_heads: int, n_groups: int, stream) -> None:
    """The selective state-space recurrence per (request, head): ``S <- exp(-exp(A_log) dt) S + dt B x^T``,
    ``y = S^T C + D x`` with ``dt = softplus(dt_raw + dt_bias)``.  ``xbc [T, .]`` holds x, B, C from the given
    column offsets; ``state`` float32 ``[slots, heads, V, N]`` (a head's ``N x V`` state column by column); ``y``
    float32 ``[T, heads*V]``."""
    _need(xbc, dt_raw.dtype, "mamba2_scan xbc")
    _need(state, torch.float32, "mamba2_scan state")
    _need(y, torch.float32, "mamba2_scan y")
    _, H, V, N = state.shape
    if H != n_heads or y.shape[1] != H * V or not state.is_contiguous():
        raise KernelError(f"mamba2_scan: state {tuple(state.shape)} for {n_heads} heads, y {tuple(y.shape)}")
    for t in (dt_bias, a_log, d_skip):
        _need(t, torch.float32, "mamba2_scan head constants")
    _call("recurrent", "mlxb_mamba2_scan", _M2_ARGS, dtype_code(xbc.dtype), _p(xbc), _rows(xbc, "mamba2_scan xbc"), x_off,
          b_off, c_off, _p(dt_raw), _rows(dt_raw, "mamba2_scan dt"), _p(dt_bias), _p(a_log), _p(d_skip), _p(state),
          _p(slots), _p(token_req), _p(req_first_token), _p(y), _rows(y, "mamba2_scan y"), H, n_groups, N, V,
          slots.numel(), stream)


_GD_ARGS = [c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]


def gated_delta_scan(qkv, q_off: int, k_off: int, v_off: int, b_raw, a_raw, dt_bias, a_log, state, slots, token_req,
                     req_first_token, o, n_heads: int, n_key_heads: int, stream) -> None:
    """The gated delta rule per (request, head): ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` with
    q and k made unit vectors (q also divided by sqrt(dim)), ``beta = sigmoid(b_raw)``,
    ``g = exp(-exp(A_log) softplus(a_raw + dt_bias))``.  ``state`` float32 ``[slots, heads, V, K]`` (a head's
    ``K x V`` state column by column); ``o`` float32."""
    _need(state, torch.float32, "gated_delta_scan state")
    _need(o, torch.float32, "gated_delta_scan o")
    _need(b_raw, qkv.dtype, "gated_delta_scan b")
    _need(a_raw, qkv.dtype, "gated_delta_scan a")
    _, H, V, K = state.shape
    if H != n_heads or o.shape[1] != H * V or not state.is_contiguous():
        raise KernelError(f"gated_delta_scan: state {tuple(state.shape)} for {n_heads} heads, o {tuple(o.shape)}")
    _call("recurrent", "mlxb_gated_delta_scan", _GD_ARGS, dtype_code(qkv.dtype), _p(qkv), _rows(qkv, "gated_delta qkv"),
          q_off, k_off, v_off, _p(b_raw), _rows(b_raw, "gated_delta b"), _p(a_raw), _rows(a_raw, "gated_delta a"),
          _p(dt_bias), _p(a_log), _p(state), _p(slots), _p(token_req), _p(req_first_token), _p(o),
          _rows(o, "gated_delta o"), H, n_key_heads, K, V, slots.numel(), stream)


# --------------------------------------------------------------------------
# queries, keys and values into shape for the attention kernels (csrc/rotary.cu)

_QKVP_ARGS = [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
              c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
              c_void_p, c_int, c_int, c_void_p, c_int, c_float, c_int, c_int, c_int, c_float, c_float, c_void_p]


def qkv_prepare(proj, q_off: int, k_off: int, v_off: int, n_heads: int, n_kv_heads: int, dk: int, dv: int, q_norm,
                k_norm, eps: float, freq, positions, token_req, block_table, k_pool, v_pool, q_out, write: bool, status,
                stream, interleaved: bool = False, v_norm_eps: Optional[float] = None, mscale: float = 1.0,
                head_norm_eps: Optional[float] = None) -> None:
    """From a fused projection ``proj [T, .]``: optional RMS norm over a token's whole q and whole k projection
    (float32 weights ``q_norm``, ``k_norm`` or None), rotation of the first ``2 * len(freq)`` dimensions of every
    head by the token's position (pairs ``(i, i + len(freq))``; ``freq`` float32 or None), q into ``q_out
    [T, n_heads*Dh]``, k and v into the pages ``[n_pages, n_kv_heads, page, Dh]`` (values: their own row width); columns of a head beyond
    ``dk`` / ``dv`` are zeros.  ``interleaved``: the pairs are ``(2i, 2i+1)``.  ``v_norm_eps``: every value head is
    divided by its root mean square (this eps inside the root, no weight) before it enters the page.  ``mscale``: a
    factor on every cosine and sine (what a stretched rotation multiplies them with).  ``head_norm_eps``: every q and k
    head is divided by its root mean square over its ``dk`` columns AFTER the rotation (no weight).  ``v_pool`` may have
    fewer heads than ``k_pool`` (a divisor of them): the projection then holds that many value heads.  ``q_out`` may
    be float32 in a bfloat16 run."""
    n_pages, Hkv, page, Dh = k_pool.shape
    _need(proj, k_pool.dtype, "qkv_prepare proj")
    if q_out.dtype != torch.float32:
        _need(q_out, k_pool.dtype, "qkv_prepare q_out")
    Hv = v_pool.shape[1]
    if (Hkv != n_kv_heads or q_out.shape[1] != n_heads * Dh or not (k_pool.is_contiguous() and v_pool.is_contiguous())
            or v_pool.shape[0] != n_pages or v_pool.shape[2] != page or Hv <= 0 or Hkv % Hv):
        raise KernelError(f"qkv_prepare: pools {tuple(k_pool.shape)} and {tuple(v_pool.shape)}, q_out {tuple(q_out.shape)}")
    half = 0
    if freq is not None:
        _need(freq, torch.float32, "qkv_prepare freq")
        half = freq.numel()
    for w, n in ((q_norm, n_heads * dk), (k_norm, n_kv_heads * dk)):
        if w is not None:
            _need(w, torch.float32, "qkv_prepare norm weight")
            if w.numel() != n:
                raise KernelError(f"qkv_prepare: norm weight of {w.numel()} for {n} columns")
    _call("rotary", "mlxb_qkv_prepare", _QKVP_ARGS, dtype_code(k_pool.dtype), _p(proj), _rows(proj, "qkv_prepare proj"),
          q_off, k_off, v_off, n_heads, n_kv_heads, dk, dv, Dh, _p(q_norm), _p(k_norm), float(eps), _p(freq), half,
          _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n_pages, page, _p(q_out),
          _rows(q_out, "qkv_prepare q_out"), _p(k_pool), _p(v_pool), int(bool(write)), proj.shape[0], _p(status),
          int(bool(interleaved)), -1.0 if v_norm_eps is None else float(v_norm_eps),
          int(q_out.dtype == torch.float32 and k_pool.dtype != torch.float32), v_pool.shape[3], Hv, float(mscale),
          -1.0 if head_norm_eps is None else float(head_norm_eps), stream)


# --------------------------------------------------------------------------
# attention with a whole group of heads per CTA (csrc/attention_wide.cu)

_WIDE_ARGS = [c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
              c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
              c_int, c_void_p, c_int, c_void_p, c_float, c_int, c_int, c_int, c_void_p]


def _pools_fit(k_pool, v_pool) -> bool:
    """Key and value pools over the same pages, the value heads as many as the key heads or a divisor of them."""
    return (v_pool.shape[0] == k_pool.shape[0] and v_pool.shape[2] == k_pool.shape[2] and v_pool.shape[1] > 0
            and k_pool.shape[1] % v_pool.shape[1] == 0 and k_pool.is_contiguous() and v_pool.is_contiguous())


def _wide_gate(gate, dtype, n_heads: int, value_dim: int, what: str):
    """``(row stride, one gate per output column?)`` of a gate ``[T, n_heads]`` or ``[T, n_heads * value_dim]``."""
    if gate is None:
        return 0, 0
    _need(gate, dtype, what + " gate")
    if gate.shape[1] == n_heads * value_dim and value_dim > 1:
        return _rows(gate, what + " gate"), 1
    if gate.shape[1] != n_heads:
        raise KernelError(f"{what}: gate {tuple(gate.shape)} for {n_heads} heads of {value_dim} columns")
    return _rows(gate, what + " gate"), 0


def attention_wide(q, q_head_stride: int, positions, token_req, block_table, k_pool, v_pool, out, out_head_stride: int,
                   n_heads: int, key_dim: int, value_dim: int, scale: float, status, stream, window: int = 0,
                   chunk: int = 0, talk=None, gate=None, rows=None, softcap: float = 0.0, keep_first: int = 0) -> None:
    """Causal attention of float32 queries ``q [T, .]`` (head ``h`` from column ``h * q_head_stride``, ``key_dim``
    values) over pages ``k_pool [n_pages, kv_heads, page, key row]`` and ``v_pool [n_pages, kv_heads, page, value
    row]`` (``v_pool`` may be ``k_pool``: a value is then the first ``value_dim`` columns of the key row).  Position
    ``p`` sees ``j <= p`` with ``p - j < window`` (if ``window``) and ``j // chunk == p // chunk`` (if ``chunk``).
    ``talk``: float32 ``[n_heads, n_heads]``, the heads' scores mixed before the softmax; ``gate``: ``[T, n_heads]``
    in the pools' dtype, head ``h``'s output times ``sigmoid(gate[t, h])``, or ``[T, n_heads * value_dim]``, a gate per
    output column.  ``softcap``: scores become ``softcap * tanh(s / softcap)`` before the softmax (0: as they are).
    ``keep_first``: beside the window, positions ``j < keep_first`` stay visible.  ``out``: the pools' dtype or float32.
    ``v_pool`` may have fewer heads than ``k_pool`` (``Hv`` dividing ``Hkv``): key heads ``c * Hkv/Hv ..`` read value head
    ``c`` (several score maps over the same values)."""
    _need(q, torch.float32, "attention_wide q")
    _need(k_pool, None, "attention_wide k_pool")
    _need(v_pool, k_pool.dtype, "attention_wide v_pool")
    n_pages, Hkv, page, krs = k_pool.shape
    vrs = v_pool.shape[3]
    if not _pools_fit(k_pool, v_pool):
        raise KernelError(f"attention_wide: pools {tuple(k_pool.shape)} and {tuple(v_pool.shape)}")
    if out.dtype not in (k_pool.dtype, torch.float32) or out.shape[0] != q.shape[0]:
        raise KernelError(f"attention_wide: out {out.dtype} {tuple(out.shape)} for q {tuple(q.shape)}")
    if talk is not None:
        _need(talk, torch.float32, "attention_wide talk")
        if talk.shape != (n_heads, n_heads) or not talk.is_contiguous():
            raise KernelError(f"attention_wide: talk {tuple(talk.shape)} for {n_heads} heads")
    ldg, gate_cols = _wide_gate(gate, k_pool.dtype, n_heads, value_dim, "attention_wide")
    n = q.shape[0] if rows is None else rows.numel()
    _call("attention_wide", "mlxb_attention_wide", _WIDE_ARGS, dtype_code(k_pool.dtype), int(out.dtype == torch.float32
          and k_pool.dtype != torch.float32), _p(q), _rows(q, "attention_wide q"), q_head_stride, _p(positions),
          _p(token_req), _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv, key_dim, value_dim, krs, vrs,
          int(window or 0), int(chunk or 0), float(scale), _p(talk), _p(k_pool), _p(v_pool), _p(gate), ldg, _p(out),
          _rows(out, "attention_wide out"), out_head_stride, _p(rows), n, _p(status), float(softcap or 0.0),
          int(keep_first or 0) if window else 0, gate_cols, v_pool.shape[1], stream)


_WIDE_TC_ARGS = [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                 c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                 c_int, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_void_p]

WIDE_TC = _os.environ.get("MLXB_WIDE_TC", "1") != "0"     # 0: the kernel on the CUDA cores for bfloat16 too


def attention_wide_tc_supported(k_pool, v_pool, n_heads: int, key_dim: int, value_dim: int, talk: bool) -> bool:
    """Whether ``attention_wide_tiles`` serves these sizes (bfloat16 pools, widths in whole 16-byte pieces, at most
    512 value columns, a tile that fits the shared memory)."""
    if not WIDE_TC or k_pool.dtype != torch.bfloat16:
        return False
    f, _ = _fn("attention_wide_tc", "mlxb_attention_wide_tc_supported", [c_int] * 8)
    return bool(f(n_heads, k_pool.shape[1], key_dim, value_dim, k_pool.shape[3], v_pool.shape[3], int(talk),
                  int(v_pool.data_ptr() == k_pool.data_ptr())))


def attention_wide_scratch(n_rows: int, n_heads: int, value_dim: int, window: int, chunk: int, max_len: int,
                           keep_first: int = 0) -> int:
    """Floats of scratch memory with which ``attention_wide_tiles`` splits the keys of single rows over several
    CTAs (0: rows that see few keys are not split)."""
    f, _ = _fn("attention_wide_tc", "mlxb_attention_wide_tc_scratch", [c_int] * 7)
    f.restype = ctypes.c_longlong
    return int(f(n_rows, n_heads, value_dim, int(window or 0), int(chunk or 0), max_len, int(keep_first or 0)))


def attention_wide_tiles(q, q_head_stride: int, tiles, n_tiles: int, tile_queries: int, block_table, k_pool, v_pool, out,
                         out_head_stride: int, n_heads: int, key_dim: int, value_dim: int, scale: float, status, stream,
                         window: int = 0, chunk: int = 0, talk=None, gate=None, scratch=None, max_len: int = 0,
                         softcap: float = 0.0, keep_first: int = 0) -> None:
    """``attention_wide`` on tensor cores for bfloat16 pools.  Instead of token rows it takes tiles, int32
    ``[n_tiles, 4]`` = (first token row, queries, block-table row, first position) of at most ``tile_queries``
    consecutive tokens of one request each (tiles of 0 queries are skipped).  With ``scratch`` (float32, at least
    ``attention_wide_scratch`` floats for ``n_tiles`` rows and ``max_len`` positions) and tiles of one query, a row's
    keys are split over CTAs that each take 64 positions, and a second kernel merges their partial results."""
    _need(q, torch.float32, "attention_wide_tiles q")
    _need(k_pool, torch.bfloat16, "attention_wide_tiles k_pool")
    _need(v_pool, torch.bfloat16, "attention_wide_tiles v_pool")
    _need(tiles, torch.int32, "attention_wide_tiles tiles")
    n_pages, Hkv, page, krs = k_pool.shape
    if not _pools_fit(k_pool, v_pool):
        raise KernelError(f"attention_wide_tiles: pools {tuple(k_pool.shape)} and {tuple(v_pool.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32) or out.shape[0] != q.shape[0] or tiles.numel() < 4 * n_tiles:
        raise KernelError(f"attention_wide_tiles: out {out.dtype} {tuple(out.shape)} for q {tuple(q.shape)}")
    if talk is not None:
        _need(talk, torch.float32, "attention_wide_tiles talk")
        if talk.shape != (n_heads, n_heads) or not talk.is_contiguous():
            raise KernelError(f"attention_wide_tiles: talk {tuple(talk.shape)} for {n_heads} heads")
    ldg, gate_cols = _wide_gate(gate, torch.bfloat16, n_heads, value_dim, "attention_wide_tiles")
    _call("attention_wide_tc", "mlxb_attention_wide_tc", _WIDE_TC_ARGS, int(out.dtype == torch.float32), _p(q),
          _rows(q, "attention_wide_tiles q"), q_head_stride, _p(tiles), n_tiles, tile_queries, _p(block_table),
          block_table.shape[1], n_pages, page, n_heads, Hkv, key_dim, value_dim, krs, v_pool.shape[3], int(window or 0),
          int(chunk or 0), float(scale), _p(talk), _p(k_pool), _p(v_pool), _p(gate), ldg, _p(out),
          _rows(out, "attention_wide_tiles out"), out_head_stride, _p(status), _p(scratch), int(max_len),
          float(softcap or 0.0), int(keep_first or 0), gate_cols, v_pool.shape[1], stream)


def attention_wide_step(ctx, q, q_head_stride: int, cache_k, cache_v, block_table, out, out_head_stride: int, n_heads: int,
                        key_dim: int, value_dim: int, scale: float, window: int = 0, chunk: int = 0, talk=None,
                        gate=None, softcap: float = 0.0, keep_first: int = 0, q_rounded=None) -> None:
    """All of a step's rows through ``attention_wide``: on tensor cores where the sizes allow it (the portions' tiles
    and the single-token rows are two launches), else on the CUDA cores (float32 runs, odd sizes).  ``q_rounded``: the
    same queries in the pages' dtype, ``[T, n_heads * key_dim]``; with them the portions of plain heads of 64 (no score
    mix, no runs of positions, a gate per column or none; values of 64 columns or a multiple, on as many heads as the
    keys or a divisor of them) go to the tcgen05 kernel of ``attention_portions``."""
    if attention_wide_tc_supported(cache_k, cache_v, n_heads, key_dim, value_dim, talk is not None):
        if (ctx.n_portion and ctx.portion_tiles is not None and q_rounded is not None and talk is None and not chunk
                and key_dim == 64 and value_dim % 64 == 0 and out_head_stride == value_dim and cache_v.shape[3] == value_dim
                and scale > 0 and (gate is None or gate.shape[1] == n_heads * value_dim)
                and (gate is None or (_rows(gate, "attention gate") % 8 == 0 and gate.data_ptr() % 16 == 0))
                and out.dtype in (cache_k.dtype, torch.float32)
                and attention_portions_tc_supported(q_rounded, out, cache_k, cache_v)):
            attention_portions(q_rounded, ctx.portion_tiles, ctx.n_portion_tiles, block_table, cache_k, cache_v, out,
                               n_heads, scale, window, ctx.status, ctx.stream, keep_first=keep_first, softcap=softcap,
                               gate=gate)
        elif ctx.n_portion and ctx.portion_tiles is not None:
            attention_wide_tiles(q, q_head_stride, ctx.portion_tiles, ctx.n_portion_tiles, PREFILL_TILE, block_table,
                                 cache_k, cache_v, out, out_head_stride, n_heads, key_dim, value_dim, scale, ctx.status,
                                 ctx.stream, window=window, chunk=chunk, talk=talk, gate=gate, softcap=softcap,
                                 keep_first=keep_first)
        if ctx.n_single and ctx.single_tiles is not None:
            need = attention_wide_scratch(ctx.n_single, n_heads, value_dim, window, chunk, ctx.max_len, keep_first)
            scratch = ctx.ws.flat("attn_wide_partial", need, torch.float32) if need else None
            attention_wide_tiles(q, q_head_stride, ctx.single_tiles, ctx.n_single, 1, block_table, cache_k, cache_v, out,
                                 out_head_stride, n_heads, key_dim, value_dim, scale, ctx.status, ctx.stream,
                                 window=window, chunk=chunk, talk=talk, gate=gate, scratch=scratch, max_len=ctx.max_len,
                                 softcap=softcap, keep_first=keep_first)
        return
    attention_wide(q, q_head_stride, ctx.positions, ctx.token_req, block_table, cache_k, cache_v, out, out_head_stride,
                   n_heads, key_dim, value_dim, scale, ctx.status, ctx.stream, window=window, chunk=chunk, talk=talk,
                   gate=gate, softcap=softcap, keep_first=keep_first)


# --------------------------------------------------------------------------
# attention over latent rows: what stands around it (csrc/latent.cu)

_LATP_ARGS = [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p,
              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
              c_float, c_void_p]


def latent_prepare(proj, q_off: int, c_off: int, n_heads: int, dim: int, rot_dim: int, rank: int, norm_weight, eps: float,
                   freq, interleaved: bool, positions, token_req, block_table, pool, write: bool, q_lat,
                   q_head_stride: int, status, stream, mscale: float = 1.0) -> None:
    """From ``proj [T, .]`` holding ``q`` (``n_heads`` heads of ``[dim | rot_dim]`` from ``q_off``) and the down
    projection (``rank + rot_dim`` columns from ``c_off``): the token's latent row ``[rmsnorm(c) * weight | rotated
    key part | 0..]`` into ``pool [n_pages, 1, page, row]``, and every head's rotated query part, float32, into
    columns ``rank ..`` of its ``q_head_stride`` columns of ``q_lat``.  ``mscale``: a factor on every cosine and sine."""
    n_pages, one, page, Dh = pool.shape
    _need(proj, pool.dtype, "latent_prepare proj")
    _need(q_lat, torch.float32, "latent_prepare q_lat")
    _need(norm_weight, torch.float32, "latent_prepare norm weight")
    if one != 1 or not pool.is_contiguous() or norm_weight.numel() != rank or q_lat.shape[1] < n_heads * q_head_stride:
        raise KernelError(f"latent_prepare: pool {tuple(pool.shape)}, q_lat {tuple(q_lat.shape)}, rank {rank}")
    if rot_dim:
        _need(freq, torch.float32, "latent_prepare freq")
        if freq.numel() != rot_dim // 2:
            raise KernelError(f"latent_prepare: {freq.numel()} frequencies for {rot_dim} rotated dimensions")
    _call("latent", "mlxb_latent_prepare", _LATP_ARGS, dtype_code(pool.dtype), _p(proj), _rows(proj, "latent_prepare proj"),
          q_off, c_off, n_heads, dim, rot_dim, rank, _p(norm_weight), float(eps), _p(freq), int(bool(interleaved)),
          _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n_pages, page, Dh, _p(pool),
          int(bool(write)), _p(q_lat), _rows(q_lat, "latent_prepare q_lat"), q_head_stride, proj.shape[0], _p(status),
          float(mscale), stream)


_HEADLIN_ARGS = [c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                 c_void_p, c_void_p]


def head_linear(x, x_head_stride: int, w, out, out_head_stride: int, stream, token_req=None) -> None:
    """``out[t, h, n] = sum_k x[t, h, k] * w[h, n, k]``: head ``h`` of ``x [T, .]`` from column ``h * x_head_stride``,
    of ``out`` from ``h * out_head_stride``; ``w [H, N, K]`` in the run's dtype; ``x`` and ``out`` in that dtype or
    float32.  Rows whose ``token_req`` is negative are not written."""
    _need(w, None, "head_linear w")
    H, N, K = w.shape
    for t, what in ((x, "x"), (out, "out")):
        if t.dtype not in (w.dtype, torch.float32) or not t.is_cuda:
            raise KernelError(f"head_linear: {what} is {t.dtype} on {t.device} for weights in {w.dtype}")
    if not w.is_contiguous() or out.shape[0] != x.shape[0]:
        raise KernelError(f"head_linear: w {tuple(w.shape)}, x {tuple(x.shape)}, out {tuple(out.shape)}")
    _call("latent", "mlxb_head_linear", _HEADLIN_ARGS, dtype_code(w.dtype),
          int(x.dtype == torch.float32 and w.dtype != torch.float32),
          int(out.dtype == torch.float32 and w.dtype != torch.float32), _p(x), _rows(x, "head_linear x"), x_head_stride,
          _p(w), _p(out), _rows(out, "head_linear out"), out_head_stride, x.shape[0], N, K, H, _p(token_req), stream)


# --------------------------------------------------------------------------
# time mixing with a data-dependent decay (csrc/wkv.cu)

_SHIFT_ARGS = [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
               c_int, c_int, c_int, c_int, c_void_p]


def token_shift_mix(x, mu, state, slots, positions, token_req, req_first_token, out, stream) -> None:
    """``out[t, s*sec : s*sec + D] = x[t] + (prev[t] - x[t]) * mu[s]`` for every mix ``s`` (``mu`` float32 ``[n_mix, D]``;
    ``out [T, n_mix*sec]`` with ``sec >= D``),
    ``prev`` the row of the token before ``t`` in its request: a row of this step, or ``state[slot]`` (float32
    ``[slots, D]``, the last row of the step before; zeros at position 0).  A second launch leaves every request's
    last row in the state."""
    _need(x, out.dtype, "token_shift_mix x")
    _need(mu, torch.float32, "token_shift_mix mu")
    _need(state, torch.float32, "token_shift_mix state")
    T, D = x.shape
    n_mix = mu.shape[0]
    if mu.shape != (n_mix, D) or not mu.is_contiguous() or state.shape[1:] != (D,) or not state.is_contiguous() \
            or out.shape[0] != T or out.shape[1] % n_mix or out.shape[1] // n_mix < D:
        raise KernelError(f"token_shift_mix: x {tuple(x.shape)}, mu {tuple(mu.shape)}, state {tuple(state.shape)}, "
                          f"out {tuple(out.shape)}")
    _call("wkv", "mlxb_token_shift_mix", _SHIFT_ARGS, dtype_code(out.dtype), _p(x), _rows(x, "token_shift_mix x"), _p(mu),
          n_mix, D, _p(state), _p(slots), _p(positions), _p(token_req), _p(req_first_token), _p(out),
          _rows(out, "token_shift_mix out"), out.shape[1] // n_mix, T, slots.numel(), stream)


_WKV_ARGS = [c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]


def wkv_scan(rkv, r_off: int, k_off: int, v_off: int, decay_raw, bonus, state, slots, token_req, req_first_token, o,
             n_heads: int, stream) -> None:
    """Per (request, head): ``o_t = (S + diag(u) k_t v_t^T)^T r_t``, then ``S <- diag(w_t) S + k_t v_t^T`` with
    ``w_t = exp(-exp(decay_raw_t))``.  ``rkv [T, .]`` holds r, k, v from the given column offsets; ``decay_raw``
    float32 ``[T, heads*K]``; ``bonus`` (u) float32 ``[heads, K]``; ``state`` float32 ``[slots, heads, V, K]`` (a head's
    ``K x V`` state column by column); ``o`` float32 ``[T, heads*V]``."""
    _need(state, torch.float32, "wkv_scan state")
    _need(o, torch.float32, "wkv_scan o")
    _need(decay_raw, torch.float32, "wkv_scan decay")
    _need(bonus, torch.float32, "wkv_scan bonus")
    _, H, V, K = state.shape
    if H != n_heads or o.shape[1] != H * V or not state.is_contiguous() or bonus.numel() != H * K \
            or not bonus.is_contiguous() or decay_raw.shape[1] != H * K:
        raise KernelError(f"wkv_scan: state {tuple(state.shape)} for {n_heads} heads, o {tuple(o.shape)}, "
                          f"decay {tuple(decay_raw.shape)}, bonus {tuple(bonus.shape)}")
    _call("wkv", "mlxb_wkv_scan", _WKV_ARGS, dtype_code(rkv.dtype), _p(rkv), _rows(rkv, "wkv_scan rkv"), r_off, k_off,
          v_off, _p(decay_raw), _rows(decay_raw, "wkv_scan decay"), _p(bonus), _p(state), _p(slots), _p(token_req),
          _p(req_first_token), _p(o), _rows(o, "wkv_scan o"), H, K, V, slots.numel(), stream)


# --------------------------------------------------------------------------
# Dynamic Tanh norm and the stream update through it (csrc/dyt.cu)

def dyt_norm(x, alpha, weight, bias, out, stream, rows=None, out_scale: float = 1.0) -> None:
    """``out[r] = (tanh(alpha * x[rows[r]]) * weight + bias) * out_scale`` over float32 rows; ``alpha``: one float32
    number on the device; ``out`` in the activation dtype or float32."""
    _need(x, torch.float32, "dyt_norm x")
    for t, what in ((alpha, "alpha"), (weight, "weight")) + (((bias, "bias"),) if bias is not None else ()):
        _need(t, torch.float32, "dyt_norm " + what)
    D = x.shape[1]
    R = x.shape[0] if rows is None else rows.numel()
    if out.shape != (R, D) or weight.numel() != D or alpha.numel() != 1 or (bias is not None and bias.numel() != D):
        raise KernelError(f"dyt_norm: x {tuple(x.shape)}, out {tuple(out.shape)}, weight {tuple(weight.shape)}")
    _call("dyt", "mlxb_dyt_norm", [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float,
                                   c_void_p, c_int, c_int, c_int, c_void_p],
          dtype_code(out.dtype), _p(x), _rows(x, "dyt_norm x"), _p(rows), x.shape[0], _p(alpha), _p(weight), _p(bias),
          float(out_scale), _p(out), _rows(out, "dyt_norm out"), R, D, stream)


def dyt_residual(x, branch, stream, post=None, nxt=None, next_out=None, terms: int = 1, token_req=None) -> None:
    """``x[t] += f(sum_k branch[t * terms + k])`` over float32 rows, with ``f = tanh(alpha * .) * weight + bias`` for
    ``post = (alpha, weight, bias)`` (None: the identity); then, with ``nxt = (alpha, weight, bias)`` and ``next_out``
    (activation dtype or float32 ``[T, D]``), the same kind of norm of the new rows is left in ``next_out``.  Rows
    whose ``token_req`` is negative are skipped."""
    _need(x, torch.float32, "dyt_residual x")
    _need(branch, torch.float32, "dyt_residual branch")
    T, D = x.shape
    if branch.shape != (T * terms, D):
        raise KernelError(f"dyt_residual: branch {tuple(branch.shape)} for {T} rows of {terms} term(s)")
    pa = pw = pb = na = nw = nb = None
    if post is not None:
        pa, pw, pb = post
    if nxt is not None:
        na, nw, nb = nxt
        if next_out is None or next_out.shape != (T, D):
            raise KernelError("dyt_residual: the next norm needs an output of the stream's shape")
    for t in (pa, pw, pb, na, nw, nb):
        if t is not None:
            _need(t, torch.float32, "dyt_residual norm tensor")
    _call("dyt", "mlxb_dyt_residual", [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
          dtype_code(next_out.dtype) if nxt is not None else F32, _p(x), _rows(x, "dyt_residual x"), _p(branch),
          _rows(branch, "dyt_residual branch"), int(terms), _p(token_req), _p(pa), _p(pw), _p(pb), _p(na), _p(nw), _p(nb),
          _p(next_out) if nxt is not None else None, _rows(next_out, "dyt_residual next") if nxt is not None else 0,
          T, D, stream)


# --------------------------------------------------------------------------
# a feed-forward of many small experts (csrc/moe.cu)

MOE_SCORES = {"sigmoid": 0, "softmax": 1}


def moe_tile_rows(tensor_cores: bool) -> int:
    """Slots a tile of the experts' products takes: of the tensor-core kernel, or of the one on the CUDA cores."""
    f, _ = _fn("moe", "mlxb_moe_tile_rows", [c_int])
    return int(f(int(bool(tensor_cores))))


def moe_few_rows() -> int:
    """Slots a tile takes in the experts' products for a step of a few tokens (bfloat16, a warp per output column)."""
    f, _ = _fn("moe", "mlxb_moe_tile_rows", [c_int])
    return int(f(2))


MOE_FEW_MAX_INNER = 6144     # the widest row the kernel for few slots keeps in shared memory


def moe_route(logits, token_req, top: int, sel_expert, sel_weight, stream, score: str = "sigmoid",
              renormalize: bool = False, correction=None, groups: int = 1, keep_groups: int = 1, identity: int = 0,
              renormalize_eps: float = 0.0, weight_scale: float = 1.0) -> None:
    """Per token the ``top`` experts with the largest scores (``sigmoid`` of the float32 router logits ``[T, E]``, or
    their ``softmax``) into ``sel_expert`` int32 ``[T * top]`` and their scores into ``sel_weight`` float32
    ``[T * top]`` (``renormalize``: divided by their sum plus ``renormalize_eps``), times ``weight_scale``.  Rows whose
    ``token_req`` is negative get expert -1.  ``correction``: float32 ``[E]`` added to the scores for the choice only
    (the weights are the scores without it).  ``groups`` > 1: the experts form that many equal groups of neighbours; a
    group's score is its largest choice score and only experts of the ``keep_groups`` best groups can be chosen.
    ``identity``: the last so many of the ``E`` router outputs are experts without tensors; chosen, they get -2 in
    ``sel_expert`` (``moe_plan`` passes over them, ``moe_combine`` adds weight times input for them)."""
    _need(logits, torch.float32, "moe_route logits")
    _need(sel_expert, torch.int32, "moe_route sel_expert")
    _need(sel_weight, torch.float32, "moe_route sel_weight")
    T, E = logits.shape
    if sel_expert.numel() < T * top or sel_weight.numel() < T * top or score not in MOE_SCORES:
        raise KernelError(f"moe_route: {T} tokens, {top} of {E} experts, score {score!r}")
    if correction is not None:
        _need(correction, torch.float32, "moe_route correction")
        if correction.numel() != E:
            raise KernelError(f"moe_route: a correction of {correction.numel()} for {E} experts")
    _call("moe", "mlxb_moe_route", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                    c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p],
          _p(logits), _rows(logits, "moe_route logits"), _p(token_req), T, E, int(top), MOE_SCORES[score],
          int(bool(renormalize)), _p(sel_expert), _p(sel_weight), _p(correction), int(groups), int(keep_groups),
          E - int(identity), float(renormalize_eps), float(weight_scale), stream)


def moe_combine(x, y, sel_expert, sel_weight, h, top: int, stream, token_req=None) -> None:
    """``x[t] += sum_c term(t, c)`` over float32 rows, in the order of the choices: ``y[t * top + c]`` (float32, the
    expert's weighted output) for a choice with tensors, ``sel_weight[t * top + c] * h[t]`` for an identity expert
    (``sel_expert`` -2).  ``h``: the feed-forward's input in the run's dtype.  Rows whose ``token_req`` is negative are
    passed over."""
    _need(x, torch.float32, "moe_combine x")
    _need(y, torch.float32, "moe_combine y")
    _need(sel_expert, torch.int32, "moe_combine sel_expert")
    _need(sel_weight, torch.float32, "moe_combine sel_weight")
    T, D = x.shape
    if y.shape != (T * top, D) or h.shape != (T, D) or sel_expert.numel() < T * top or sel_weight.numel() < T * top:
        raise KernelError(f"moe_combine: x {tuple(x.shape)}, y {tuple(y.shape)}, h {tuple(h.shape)}, {top} choices")
    _call("moe", "mlxb_moe_combine", [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                      c_void_p, c_int, c_int, c_int, c_void_p],
          dtype_code(h.dtype), _p(x), _rows(x, "moe_combine x"), _p(y), _rows(y, "moe_combine y"), _p(sel_expert),
          _p(sel_weight), _p(h), _rows(h, "moe_combine h"), _p(token_req), T, int(top), D, stream)


def moe_max_tiles(n_slots: int, n_experts: int, tile_rows: int) -> int:
    """The most tiles ``n_slots`` (token, choice) pairs can make, however they fall on the experts."""
    return (n_slots + tile_rows - 1) // tile_rows + n_experts


def moe_plan(sel_expert, n_slots: int, n_experts: int, tile_rows: int, sorted_slots, tile_info, n_tiles, stream) -> None:
    """The slots sorted by expert (``sorted_slots`` int32 ``[n_slots]``) and the tiles of at most ``tile_rows`` slots
    of one expert (``tile_info`` int32 ``[moe_max_tiles, 3]`` = expert, first place, slots; ``n_tiles`` int32 ``[1]``)."""
    for t, what in ((sel_expert, "sel_expert"), (sorted_slots, "sorted"), (tile_info, "tile_info"), (n_tiles, "n_tiles")):
        _need(t, torch.int32, "moe_plan " + what)
    max_tiles = moe_max_tiles(n_slots, n_experts, tile_rows)
    if sorted_slots.numel() < n_slots or tile_info.numel() < 3 * max_tiles or sel_expert.numel() < n_slots:
        raise KernelError(f"moe_plan: {n_slots} slots, {n_experts} experts")
    _call("moe", "mlxb_moe_plan", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
          _p(sel_expert), n_slots, n_experts, tile_rows, max_tiles, _p(sorted_slots), _p(tile_info), _p(n_tiles), stream)


GATED_UNITS = {"silu": 0, "bounded": 1}     # csrc/gated_unit.cuh


def moe_gemm(a, a_div: int, w, n_out: int, sorted_slots, tile_info, n_tiles, max_tiles: int, tile_rows: int, out, stream,
             sel_weight=None, gated: bool = False, unit: str = "silu", limit: float = 0.0) -> None:
    """``out[slot] = a[slot // a_div] @ w[expert(slot)].T`` for every slot of the plan; ``w [E, n_out, K]``.  ``gated``:
    ``w [E, 2 n_out, K]`` holds gate rows then up rows and the result is ``silu(s g) * (s u)`` with ``s`` the slot's
    routing weight; with ``unit="bounded"`` it is ``s g' sigmoid(1.702 g') (u' + 1)``, ``g' = min(g, limit)``,
    ``u' = clamp(u, -limit, limit)`` (the weight on the unit's output).  ``out``: ``a``'s dtype or float32,
    ``[n_slots, n_out]``."""
    _need(a, None, "moe_gemm a")
    _need(w, a.dtype, "moe_gemm w")
    E, NW, K = w.shape
    if NW != (2 if gated else 1) * n_out or a.shape[1] != K or out.shape[1] != n_out or not w.is_contiguous():
        raise KernelError(f"moe_gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if out.dtype not in (a.dtype, torch.float32):
        raise KernelError(f"moe_gemm: out {out.dtype} for inputs {a.dtype}")
    if gated:
        _need(sel_weight, torch.float32, "moe_gemm sel_weight")
    _call("moe", "mlxb_moe_gemm", [c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, ctypes.c_longlong, c_int, c_int,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_float,
                                   c_void_p],
          dtype_code(a.dtype), int(out.dtype == torch.float32 and a.dtype != torch.float32), int(bool(gated)), _p(a),
          _rows(a, "moe_gemm a"), int(a_div), _p(w), NW * K, n_out, K, _p(sorted_slots), _p(tile_info), _p(n_tiles),
          int(max_tiles), int(tile_rows), _p(sel_weight), _p(out), _rows(out, "moe_gemm out"), GATED_UNITS[unit],
          float(limit), stream)


def moe_tc05_tile_rows() -> int:
    """Slots a tile of the experts' products on the 5th-generation tensor cores takes (``moe_gemm_tc05``)."""
    f, _ = _fn("moe_tcgen05", "mlxb_moe_tc05_tile_rows", [])
    return int(f())


def moe_gather(src, a_div: int, sorted_slots, tile_info, n_tiles, max_tiles: int, dst, stream) -> None:
    """``dst[i] = src[sorted_slots[i] // a_div]`` for every place of the plan's tiles: the slots' rows in the plan's
    order, so that one expert's rows lie together.  bfloat16, whole 16 bytes a row."""
    _need(src, torch.bfloat16, "moe_gather src")
    _need(dst, torch.bfloat16, "moe_gather dst")
    if src.shape[1] != dst.shape[1]:
        raise KernelError(f"moe_gather: src {tuple(src.shape)}, dst {tuple(dst.shape)}")
    _call("moe_tcgen05", "mlxb_moe_gather", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                             c_int, c_void_p],
          _p(src), _rows(src, "moe_gather src"), int(a_div), _p(sorted_slots), _p(tile_info), _p(n_tiles), int(max_tiles),
          src.shape[1], _p(dst), _rows(dst, "moe_gather dst"), stream)


def moe_gemm_tc05(a, w, n_out: int, sorted_slots, tile_info, n_tiles, max_tiles: int, out, status, stream,
                  sel_weight=None, gated: bool = False, unit: str = "silu", limit: float = 0.0) -> None:
    """The experts' products over a plan of ``moe_tc05_tile_rows()``-slot tiles on the 5th-generation tensor cores.
    ``a``: bfloat16 rows IN THE PLAN'S ORDER (``moe_gather``, or the gated product's own result); ``w [E, n_out, K]``.
    ``gated``: ``w [E, 2 n_out, K]`` holds gate rows then up rows and ``out`` (bfloat16, in the plan's order) is
    ``silu(s g) * (s u)`` with ``s`` the slot's routing weight (``unit``, ``limit``: as in ``moe_gemm``); else ``out`` (float32) gets the product of the row at
    place ``i`` in row ``sorted_slots[i]``.  ``status``: receives a bit if a bounded wait in the kernel gives up."""
    _need(a, torch.bfloat16, "moe_gemm_tc05 a")
    _need(w, torch.bfloat16, "moe_gemm_tc05 w")
    _need(out, torch.bfloat16 if gated else torch.float32, "moe_gemm_tc05 out")
    _need(status, torch.int32, "moe_gemm_tc05 status")
    E, NW, K = w.shape
    if NW != (2 if gated else 1) * n_out or a.shape[1] != K or out.shape[1] != n_out or not w.is_contiguous():
        raise KernelError(f"moe_gemm_tc05: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if gated:
        _need(sel_weight, torch.float32, "moe_gemm_tc05 sel_weight")
    _call("moe_tcgen05", "mlxb_moe_gemm_tc05", [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                                c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_float,
                                                c_void_p],
          int(bool(gated)), _p(a), _rows(a, "moe_gemm_tc05 a"), a.shape[0], _p(w), E, NW, n_out, K, _p(sorted_slots),
          _p(tile_info), _p(n_tiles), int(max_tiles), _p(sel_weight), _p(out), _rows(out, "moe_gemm_tc05 out"), _p(status),
          GATED_UNITS[unit], float(limit), stream)


# --------------------------------------------------------------------------
# small row-wise kernels (csrc/elementwise.cu)

def xielu(x, out, params, stream) -> None:
    """``out = f(x)`` elementwise (``out`` may be ``x``) with the layer's two numbers ``params`` (float32 ``[2]`` on
    the device): ``z > 0: softplus(a) z^2 + z/2``; ``z <= 0: (1/2 + softplus(b)) (exp(z) - 1 - z) + z/2``."""
    _need(x, out.dtype, "xielu x")
    _need(params, torch.float32, "xielu params")
    T, F_ = out.shape
    if x.shape != out.shape or params.numel() != 2:
        raise KernelError(f"xielu: x {tuple(x.shape)}, out {tuple(out.shape)}, {params.numel()} parameters")
    _call("elementwise", "mlxb_xielu", [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
          dtype_code(out.dtype), _p(x), _rows(x, "xielu x"), _p(out), _rows(out, "xielu out"), F_, T, _p(params), stream)


def gated_unit(x, out, stream, unit: str = "silu", limit: float = 0.0) -> None:
    """``out[t, j] = silu(x[t, j]) * x[t, F + j]`` for ``x [T, 2F]``: the halves of a fused [gate | up] projection.
    ``unit="bounded"``: ``g' sigmoid(1.702 g') (u' + 1)`` with ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)``."""
    _need(x, out.dtype, "gated_unit x")
    T, F_ = out.shape
    if x.shape != (T, 2 * F_):
        raise KernelError(f"gated_unit: x {tuple(x.shape)} for out {tuple(out.shape)}")
    _call("elementwise", "mlxb_gated_unit", [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p],
          dtype_code(out.dtype), _p(x), _rows(x, "gated_unit x"), _p(out), _rows(out, "gated_unit out"), F_, T,
          GATED_UNITS[unit], float(limit), stream)


def scale_by_rows(x, index, table, first: int, out, status, stream) -> None:
    """``out[t, j] = x[t, j] * table[index[t], first + j]``."""
    _need(x, out.dtype, "scale_by_rows x")
    _need(table, out.dtype, "scale_by_rows table")
    _need(index, torch.int32, "scale_by_rows index")
    T, F_ = out.shape
    if x.shape != out.shape or table.dim() != 2:
        raise KernelError(f"scale_by_rows: x {tuple(x.shape)}, out {tuple(out.shape)}, table {tuple(table.shape)}")
    _call("elementwise", "mlxb_scale_by_rows",
          [c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
           c_void_p],
          dtype_code(out.dtype), _p(x), _rows(x, "scale_by_rows x"), _p(index), _p(table), _rows(table, "table"),
          table.shape[0], first, _p(out), _rows(out, "scale_by_rows out"), F_, T, _p(status), stream)


def join_rows(a, b, out, stream) -> None:
    """``out[t] = [a[t] | b[t]]`` in ``out``'s dtype from contiguous float32 rows (``b`` None: a cast of ``a``)."""
    _need(a, torch.float32, "join_rows a")
    T, D = a.shape
    if not a.is_contiguous() or (b is not None and (b.shape != a.shape or b.dtype != torch.float32 or not b.is_contiguous())):
        raise KernelError(f"join_rows: a {tuple(a.shape)}")
    if out.shape != (T, D * (2 if b is not None else 1)):
        raise KernelError(f"join_rows: out {tuple(out.shape)} for rows of {D}")
    _call("elementwise", "mlxb_join_rows", [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
          dtype_code(out.dtype), _p(a), _p(b), D, _p(out), _rows(out, "join_rows out"), T, stream)
