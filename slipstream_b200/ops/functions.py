"""Python entry points of the CUDA kernels.

Each function takes torch tensors that live on the CUDA device, checks what the
kernel cannot check cheaply (dtype, contiguity, sizes), and launches on torch's
current stream.  Nothing here computes on the CPU or falls back to a library
implementation; a failed launch raises ``KernelError``.

Kernels record out-of-range token ids, cache slots and block-table entries in a
device error word instead of trapping; ``check_errors`` reads it (one
synchronising copy) and raises.
"""

from __future__ import annotations

import ctypes
import dataclasses
import functools
from ctypes import c_float, c_int, c_int64, c_void_p

import numpy as np
import torch

from .library import KernelBuildError, load_library, require_cuda

SS_F32, SS_BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return SS_F32
    if dtype == torch.bfloat16:
        return SS_BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


_OPS_SIGNATURES = {
    "ss_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "ss_gather_tokens": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "ss_prepare_decode": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64,
                          c_void_p],
    "ss_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                       c_float, c_int, c_void_p],
    "ss_rope_cache": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                      c_int, c_int, c_int64, c_int, c_int, c_void_p, c_void_p],
    "ss_swiglu": [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p],
    "ss_gemm_simt": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int64,
                     c_int64, c_int, c_int, c_void_p],
    "ss_argmax": [c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p],
    "ss_sample": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "ss_mark_seen": [c_void_p, c_void_p, c_int, c_int, c_void_p],
}

_ATTN_SIGNATURES = {
    "ss_attn_simt": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                     c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float,
                     c_int, c_int, c_void_p, c_void_p],
    "ss_attn_prefill_mma": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                            c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float,
                            c_int, c_void_p, c_void_p],
    "ss_attn_prefill_tc5": [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                            c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float, c_int, c_void_p,
                            c_void_p],
    "ss_attn_decode_tma": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float, c_int, c_int,
                           c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ss_attn_decode_mma": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_float, c_int, c_int,
                           c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
}

_GEMM_SIGNATURES = {
    "ss_gemm_tc5_many": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                         c_int, c_int, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5_many_tile_cols": [c_int, c_int, c_int],
    "ss_gemm_tc5_many_to_stream": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5_many_scaled": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int,
                                c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                    c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "ss_gemm_tc5_to_stream": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int, c_int,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "ss_gemm_tc5_scaled": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                           c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
}

_state: dict[str, object] = {}


def _declare(lib: ctypes.CDLL, table: dict[str, list]) -> None:
    for name, argtypes in table.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int


def ops_library() -> ctypes.CDLL:
    lib = _state.get("ops")
    if lib is None:
        require_cuda()
        lib = load_library("slipstream_ops", ["ops.cu", "sampling.cu"])
        _declare(lib, _OPS_SIGNATURES)
        _state["ops"] = lib
    return lib  # type: ignore[return-value]


def gemm_library() -> ctypes.CDLL:
    lib = _state.get("gemm")
    if lib is None:
        require_cuda()
        lib = load_library("slipstream_gemm", ["gemm_tc5.cu"])
        _declare(lib, _GEMM_SIGNATURES)
        _state["gemm"] = lib
    return lib  # type: ignore[return-value]


def attention_library(head_dim: int) -> ctypes.CDLL:
    key = f"attn{head_dim}"
    lib = _state.get(key)
    if lib is None:
        require_cuda()
        if head_dim % 16 != 0 or not (16 <= head_dim <= 256):
            raise KernelError(
                f"attention kernels take head sizes that are multiples of 16 up to 256, not {head_dim}")
        lib = load_library("slipstream_attn", ["attention.cu"], {"HEAD_DIM": head_dim})
        _declare(lib, _ATTN_SIGNATURES)
        _state[key] = lib
    return lib  # type: ignore[return-value]


def error_word(device: torch.device) -> torch.Tensor:
    key = ("err", device)
    word = _state.get(key)
    if word is None:
        with torch.inference_mode(False):  # the word is cleared in place later, from any mode
            word = torch.zeros(1, dtype=torch.int32, device=device)
        _state[key] = word
    return word  # type: ignore[return-value]


_ERR_NAMES = {1: "a token id outside the vocabulary", 2: "a cache slot outside the pool",
              4: "a block-table entry outside the pool", 8: "a bounded wait gave up"}


def raise_for_status(value: int, device: torch.device) -> None:
    """Raise ``KernelError`` for a non-zero value of the error word (already on the host) and clear the word."""
    if value:
        error_word(device).zero_()
        what = "; ".join(text for bit, text in _ERR_NAMES.items() if value & bit) or f"status {value}"
        raise KernelError(f"a kernel reported: {what}")


def check_errors(device: torch.device) -> None:
    raise_for_status(int(error_word(device).item()), device)


@functools.lru_cache(maxsize=None)
def _device_sm_count(index: int) -> int:
    return int(torch.cuda.get_device_properties(index).multi_processor_count)


def sm_count(device: torch.device | int | None = None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current CUDA device), asked from the device once.
    Every rule below that sizes a grid or a split takes this number as ``sms``."""
    if isinstance(device, torch.device):
        device = device.index
    if device is None:
        require_cuda()
        device = torch.cuda.current_device()
    return _device_sm_count(int(device))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current CUDA stream (every wrapper below asks for it, so the short way is taken when
    this torch has it)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_launches = [0]


def launch_count() -> int:
    """Kernels of this package launched so far (each entry point below launches exactly one;
    a replayed CUDA graph adds the kernels it holds, see ``count_launches``)."""
    return _launches[0]


def count_launches(n: int) -> None:
    _launches[0] += n


def _check(code: int, what: str) -> None:
    _launches[0] += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype: torch.dtype | None, what: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


# --------------------------------------------------------------------------- model ops

def embedding(token_ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Rows of ``table`` [vocab, hidden] at ``token_ids`` (int32 [N]) as float32 [N, hidden]."""
    _need(token_ids, torch.int32, "token_ids")
    _need(table, None, "embedding table")
    n, (vocab, hidden) = token_ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _need(out, torch.float32, "embedding output")
    _check(ops_library().ss_embedding(token_ids.data_ptr(), table.data_ptr(), out.data_ptr(), n, hidden,
                                      vocab, _code(table.dtype), error_word(table.device).data_ptr(),
                                      _stream()), "embedding")
    return out


def gather_tokens(token_ids: torch.Tensor, src_rows: torch.Tensor, pending: torch.Tensor) -> None:
    """``token_ids[r] = pending[src_rows[r]]`` where ``src_rows[r] >= 0`` (int32 tensors on the device): token ids
    sampled by the step before that the host has not read yet."""
    for name, t in (("token_ids", token_ids), ("src_rows", src_rows), ("pending", pending)):
        _need(t, torch.int32, name)
    _check(ops_library().ss_gather_tokens(token_ids.data_ptr(), src_rows.data_ptr(), pending.data_ptr(),
                                          src_rows.numel(), _stream()), "gather_tokens")


def prepare_decode(token_ids: torch.Tensor, src_rows: torch.Tensor, pending: torch.Tensor | None,
                   tables: torch.Tensor, patch_idx: torch.Tensor, patch_val: torch.Tensor,
                   n_patches: torch.Tensor) -> None:
    """The launch in front of a replayed decode step: ``gather_tokens`` (when ``pending`` is given) and
    ``tables.view(-1)[patch_idx[i]] = patch_val[i]`` for ``i < n_patches[0]`` (all int32 tensors on the device;
    the number of patches is read on the device, so the launch is the same every step)."""
    for name, t in (("token_ids", token_ids), ("src_rows", src_rows), ("tables", tables), ("patch_idx", patch_idx),
                    ("patch_val", patch_val), ("n_patches", n_patches)):
        _need(t, torch.int32, name)
    if pending is not None:
        _need(pending, torch.int32, "pending")
    _check(ops_library().ss_prepare_decode(token_ids.data_ptr(), src_rows.data_ptr(), _ptr(pending),
                                           src_rows.numel(), tables.data_ptr(), patch_idx.data_ptr(),
                                           patch_val.data_ptr(), n_patches.data_ptr(), patch_idx.numel(),
                                           tables.numel(), _stream()), "prepare_decode")


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """``residual`` (float32 [N, H]) += ``delta`` in place, then RMSNorm times ``weight``.

    With ``rows`` (int32 [M]) only those rows are produced and ``residual`` is not changed.
    ``weight`` is in ``out_dtype`` or float32."""
    _need(residual, torch.float32, "residual")
    hidden = residual.shape[-1]
    n_out = residual.shape[0] if rows is None else rows.numel()
    if delta is not None:
        _need(delta, out_dtype, "delta")
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match residual {tuple(residual.shape)}")
    _need(weight, None, "norm weight")
    if weight.numel() != hidden or weight.dtype not in (out_dtype, torch.float32):
        raise KernelError("norm weight has the wrong size or dtype")
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if out is None:
        out = torch.empty((n_out, hidden), dtype=out_dtype, device=residual.device)
    _need(out, out_dtype, "norm output")
    w_f32 = int(weight.dtype == torch.float32 and out_dtype != torch.float32)
    _check(ops_library().ss_add_rmsnorm(residual.data_ptr(), _ptr(delta), weight.data_ptr(), w_f32,
                                        out.data_ptr(), _ptr(rows), n_out, hidden, float(eps),
                                        _code(out_dtype), _stream()), "add_rmsnorm")
    return out


def rope_and_cache(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor | None,
                   inv_freq: torch.Tensor | None, kv: torch.Tensor | None, n_q: int, n_kv: int,
                   head_dim: int, rotary_dim: int, write_cache: bool = True) -> None:
    """Rotate queries (in place) and keys of ``qkv`` [N, (n_q + 2 n_kv) * D] by their positions and
    write keys and values to their pages: ``kv`` is [pages, 2, n_kv, page_size, D], ``slots`` int32 [N]
    = page * page_size + offset (-1 skips a token).  ``rotary_dim`` 0 copies without rotating."""
    _need(qkv, None, "qkv")
    _need(positions, torch.int32, "positions")
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError("qkv has the wrong width")
    if rotary_dim % 2 or rotary_dim > head_dim:
        raise KernelError("rotary_dim must be even and at most head_dim")
    if rotary_dim:
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("inv_freq must hold rotary_dim / 2 values")
    write = bool(write_cache and kv is not None and slots is not None)
    pages = page_size = 0
    if write:
        _need(kv, qkv.dtype, "kv pages")
        _need(slots, torch.int32, "slots")
        if kv.dim() != 5 or kv.shape[1] != 2 or kv.shape[2] != n_kv or kv.shape[4] != head_dim:
            raise KernelError(f"kv pages have shape {tuple(kv.shape)}, expected [pages, 2, {n_kv}, page, {head_dim}]")
        pages, page_size = kv.shape[0], kv.shape[3]
    _check(ops_library().ss_rope_cache(qkv.data_ptr(), positions.data_ptr(), _ptr(slots) if write else None,
                                       _ptr(inv_freq), _ptr(kv) if write else None, n, n_q, n_kv, head_dim,
                                       rotary_dim, max(page_size, 1), pages, int(write), _code(qkv.dtype),
                                       error_word(qkv.device).data_ptr(), _stream()), "rope_and_cache")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, block: int | None = None) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up`` = [N, 2 * I].  Gate and up features alternate in runs of ``block``
    columns (gate run, up run, gate run, ...); the default, ``block`` = I, is the plain [gate | up]."""
    _need(gate_up, None, "gate_up")
    n, two_i = gate_up.shape
    inter = two_i // 2
    block = inter if block is None else block
    if block < 1 or inter % block:
        raise KernelError(f"block {block} does not divide the {inter} features")
    if out is None:
        out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    _need(out, gate_up.dtype, "swiglu output")
    _check(ops_library().ss_swiglu(gate_up.data_ptr(), out.data_ptr(), n, inter, block, _code(gate_up.dtype),
                                   _stream()), "swiglu")
    return out


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
              out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T + bias`` on CUDA cores with float32 accumulation (no tensor cores):
    x [M, K], weight [N, K].  The float32 path of every projection."""
    _need(x, None, "x")
    _need(weight, x.dtype, "weight")
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"weight {tuple(weight.shape)} does not match x {tuple(x.shape)}")
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _need(out, out_dtype, "gemm output")
    bias_f32 = 0
    if bias is not None:
        _need(bias, None, "bias")
        bias_f32 = int(bias.dtype == torch.float32)
        if bias.numel() != n or (not bias_f32 and bias.dtype != x.dtype):
            raise KernelError("bias has the wrong size or dtype")
    _check(ops_library().ss_gemm_simt(x.data_ptr(), weight.data_ptr(), _ptr(bias), bias_f32, out.data_ptr(),
                                      m, n, k, k, n, _code(x.dtype), _code(out_dtype), _stream()), "gemm_simt")
    return out


def paged_attention_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                         block_tables: torch.Tensor, tile_req: torch.Tensor, tile_q0: torch.Tensor,
                         q_start: torch.Tensor, seq_lens: torch.Tensor, n_q: int, n_kv: int,
                         head_dim: int, scale: float, window: int = 0) -> None:
    """Causal grouped-query attention of the step's query rows over the pages.

    ``q`` points at the first query head of row 0; rows are ``q_stride`` elements apart.
    ``out`` is [N, n_q * D].  ``tile_req`` / ``tile_q0`` list tiles of 16 consecutive query tokens
    of one request (request index, first token within the request's rows of this step)."""
    _need(out, q.dtype, "attention output")
    _need(kv, q.dtype, "kv pages")
    for name, t in (("block_tables", block_tables), ("tile_req", tile_req), ("tile_q0", tile_q0),
                    ("q_start", q_start), ("seq_lens", seq_lens)):
        _need(t, torch.int32, name)
    lib = attention_library(head_dim)
    _check(lib.ss_attn_simt(q.data_ptr(), q_stride, out.data_ptr(), out.shape[1], kv.data_ptr(),
                            block_tables.data_ptr(), block_tables.shape[1], tile_req.data_ptr(),
                            tile_q0.data_ptr(), tile_req.numel(), q_start.data_ptr(), seq_lens.data_ptr(),
                            n_q, n_kv, kv.shape[3], kv.shape[0], float(scale), int(window or 0),
                            _code(q.dtype), error_word(q.device).data_ptr(), _stream()), "paged_attention_simt")


def paged_attention_prefill(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                            block_tables: torch.Tensor, tile_req: torch.Tensor, tile_row0: torch.Tensor,
                            q_start: torch.Tensor, seq_lens: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                            scale: float, window: int = 0) -> None:
    """bfloat16 tensor-core attention for prompt portions and mixed batches.  A tile is 64 consecutive
    rows of one request, a row being a (query token, head of the kv group) pair in token-major order:
    ``tile_req`` / ``tile_row0`` list (request index, first row)."""
    _need(out, torch.bfloat16, "attention output")
    _need(kv, torch.bfloat16, "kv pages")
    if q.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention kernels take bfloat16")
    for name, t in (("block_tables", block_tables), ("tile_req", tile_req), ("tile_row0", tile_row0),
                    ("q_start", q_start), ("seq_lens", seq_lens)):
        _need(t, torch.int32, name)
    lib = attention_library(head_dim)
    _check(lib.ss_attn_prefill_mma(q.data_ptr(), q_stride, out.data_ptr(), out.shape[1], kv.data_ptr(),
                                   block_tables.data_ptr(), block_tables.shape[1], tile_req.data_ptr(),
                                   tile_row0.data_ptr(), tile_req.numel(), q_start.data_ptr(), seq_lens.data_ptr(),
                                   n_q, n_kv, kv.shape[3], kv.shape[0], float(scale), int(window or 0),
                                   error_word(q.device).data_ptr(), _stream()), "paged_attention_prefill")


def tcgen05_attention_fits(head_dim: int, n_q: int, n_kv: int, page_size: int, window: int) -> bool:
    """Whether the tcgen05 prefill attention kernel takes this layer: head size 64 or 128, no window, pages of
    8, 16, 32 or 64 tokens, at most 128 query heads per kv head."""
    return (head_dim in (64, 128) and not window and page_size in (8, 16, 32, 64) and n_q // n_kv <= 128)


def paged_attention_prefill_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                                    block_tables: torch.Tensor, tile_req: torch.Tensor, tile_tok0: torch.Tensor,
                                    q_start: torch.Tensor, seq_lens: torch.Tensor, n_q: int, n_kv: int,
                                    head_dim: int, scale: float, key_parts: int = 1) -> None:
    """bfloat16 causal attention for prompt portions and mixed batches on the tcgen05 tensor cores (Q, K, V
    tiles by TMA, S and O in tensor memory).  A tile is ``128 // (n_q // n_kv)`` consecutive query tokens of
    one request: ``tile_req`` / ``tile_tok0`` list (request index, first token within the request's rows); blocks
    start in list order, so the list should begin with the tiles that see the most keys.
    ``key_parts`` (1, 2, 4 or 8): the keys of every query tile are shared by that many blocks, a thread-block
    cluster whose results are combined through shared memory (see ``prefill_key_parts``)."""
    _need(out, torch.bfloat16, "attention output")
    _need(kv, torch.bfloat16, "kv pages")
    if q.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention kernels take bfloat16")
    if not tcgen05_attention_fits(head_dim, n_q, n_kv, kv.shape[3], 0):
        raise KernelError("the tcgen05 attention kernel does not take this head size or page size")
    for name, t in (("block_tables", block_tables), ("tile_req", tile_req), ("tile_tok0", tile_tok0),
                    ("q_start", q_start), ("seq_lens", seq_lens)):
        _need(t, torch.int32, name)
    lib = attention_library(head_dim)
    _check(lib.ss_attn_prefill_tc5(q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), out.shape[1], kv.data_ptr(),
                                   block_tables.data_ptr(), block_tables.shape[1], tile_req.data_ptr(),
                                   tile_tok0.data_ptr(), tile_req.numel(), q_start.data_ptr(), seq_lens.data_ptr(),
                                   n_q, n_kv, kv.shape[3], kv.shape[0], float(scale), int(key_parts),
                                   error_word(q.device).data_ptr(), _stream()), "paged_attention_prefill_tcgen05")


def prefill_key_parts(q_lens: np.ndarray, seq_lens: np.ndarray, tile_tokens: int, n_kv: int,
                      sms: int | None = None) -> int:
    """Into how many parts the tcgen05 prefill kernel should cut the keys of its query tiles.  A block walks its
    key tiles one after the other, about a microsecond each, so a step with few query tiles lasts as long as its
    longest one while most SMs idle: a portion of 64 tokens behind 4,096 cached ones is 16 blocks of 64 key
    tiles, 47.5 us; with the keys of every query tile shared by 8 blocks 19.3 us; 512 tokens behind 4,096: 52.3
    against 41.5 us with 2.  Parts are only worth it while all blocks still run at once (every block pays for
    its own set-up and for the combination: a whole prompt of 2,048 tokens, 456 blocks, takes 47.5 us in one
    part and 59.3 in two) and while a part keeps 8 key tiles."""
    q_lens = np.asarray(q_lens, dtype=np.int64)
    seq_lens = np.asarray(seq_lens, dtype=np.int64)
    if q_lens.size == 0:
        return 1
    counts = (q_lens + tile_tokens - 1) // tile_tokens
    blocks = int(counts.sum()) * n_kv
    longest = int(seq_lens.max() - 1) // 64 + 1  # key tiles of the last query tile of the longest request
    sms = sms or sm_count()
    parts = 1
    while parts < 8 and blocks * parts * 2 <= 2 * sms and longest >= 16 * parts:
        parts *= 2
    return parts


_DECODE_COUNTERS = 65536


def decode_counters(device: torch.device) -> torch.Tensor:
    """Counters of the split decode kernel (one per request and head block): zero between launches, which
    the kernel itself restores, so one tensor per device serves every call."""
    key = f"decode_counters{device}"
    counters = _state.get(key)
    if counters is None:
        counters = torch.zeros(_DECODE_COUNTERS, dtype=torch.int32, device=device)
        _state[key] = counters
    return counters  # type: ignore[return-value]


def decode_scratch(n_requests: int, n_q: int, n_slices: int, head_dim: int, device: torch.device):
    """Scratch memory of the split decode kernel: partial outputs and their log-sum-exps."""
    return (torch.empty((n_requests, n_q, n_slices, head_dim), dtype=torch.float32, device=device),
            torch.empty((n_requests, n_q, n_slices), dtype=torch.float32, device=device))


def paged_attention_decode(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                           block_tables: torch.Tensor, q_start: torch.Tensor, seq_lens: torch.Tensor,
                           n_requests: int, n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0,
                           n_slices: int = 1, scratch: tuple[torch.Tensor, torch.Tensor] | None = None,
                           rope: tuple[torch.Tensor | None, int] | None = None, tma: bool | None = None,
                           stages: int = 2) -> None:
    """bfloat16 attention for requests that bring ONE token each, the keys of every request cut into
    ``n_slices`` slices that run in parallel.  Up to 8 slices form a thread-block cluster and are combined
    through shared memory; with more, the partial results (of every cluster of 8 in the TMA-fed kernel when the
    count is a multiple of 8, else of every slice) pass through ``scratch`` (see ``decode_scratch``) and the
    block that finishes a head block last combines them.

    ``rope`` = (inverse frequencies, rotary_dim): ``q`` is then the stacked projection output
    [N, (n_q + 2 n_kv) * D] as projected, and the kernel itself rotates queries and the newest key by each
    request's last position and writes the newest key and value to their page (what ``rope_and_cache`` does
    for other steps).

    ``tma``: the kernel whose tiles are moved by TMA (head size 64 or 128, pages of 8, 16, 32 or 64 tokens;
    the default where it fits), or the one that moves them with cp.async (every head and page size).
    ``stages``: 2 or 3 tiles in the ring of the TMA-fed kernel."""
    fits = tcgen05_attention_fits(head_dim, n_q, n_kv, kv.shape[3], 0)
    if tma is None:
        tma = fits
    elif tma and not fits:
        raise KernelError("the TMA decode kernel takes head size 64 or 128 and pages of 8, 16, 32 or 64 tokens")
    _need(out, torch.bfloat16, "attention output")
    _need(kv, torch.bfloat16, "kv pages")
    if q.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention kernels take bfloat16")
    for name, t in (("block_tables", block_tables), ("q_start", q_start), ("seq_lens", seq_lens)):
        _need(t, torch.int32, name)
    part_o = part_lse = counters = None
    if n_slices > 8:
        counters = decode_counters(q.device)
        if n_requests * n_kv * ((n_q // n_kv + 15) // 16) > _DECODE_COUNTERS:
            raise KernelError("too many (request, head block) pairs for the decode counters")
        if scratch is None:
            scratch = decode_scratch(n_requests, n_q, n_slices, head_dim, q.device)
        part_o, part_lse = scratch
        if part_o.numel() < n_requests * n_q * n_slices * head_dim or part_lse.numel() < n_requests * n_q * n_slices:
            raise KernelError("decode scratch is too small")
    inv_freq, rotary_dim = rope if rope is not None else (None, 0)
    if rope is not None:
        if q_stride != (n_q + 2 * n_kv) * head_dim:
            raise KernelError("the fused rotation takes the stacked q/k/v projection")
        if rotary_dim % 2 or rotary_dim > head_dim:
            raise KernelError("rotary_dim must be even and at most head_dim")
        if rotary_dim:
            _need(inv_freq, torch.float32, "inv_freq")
            if inv_freq.numel() != rotary_dim // 2:
                raise KernelError("inv_freq must hold rotary_dim / 2 values")
    lib = attention_library(head_dim)
    args = (q.data_ptr(), q_stride, out.data_ptr(), out.shape[1], kv.data_ptr(), block_tables.data_ptr(),
            block_tables.shape[1], n_requests, q_start.data_ptr(), seq_lens.data_ptr(), n_q, n_kv, kv.shape[3], kv.shape[0],
            float(scale), int(window or 0), n_slices, _ptr(inv_freq) if rotary_dim else None, rotary_dim,
            int(rope is not None), _ptr(part_o), _ptr(part_lse), _ptr(counters))
    tail = (error_word(q.device).data_ptr(), _stream())
    if tma:
        _check(lib.ss_attn_decode_tma(*args, int(stages), *tail), "paged_attention_decode")
    else:
        _check(lib.ss_attn_decode_mma(*args, *tail), "paged_attention_decode")


WIDE_CONTEXT = 8192  # from this many cached tokens a decode step of few requests may use more than 8 slices


def is_long_context(seq_len: int) -> bool:
    return seq_len >= WIDE_CONTEXT


def decode_slices(n_requests: int, n_kv: int, group: int, max_seq_len: int, wide: bool = False,
                  sms: int | None = None) -> int:
    """How many slices to cut the keys into: as many as keep all blocks resident at once (two per SM),
    so that the step is one wave of blocks; at most 8, the size of a thread-block cluster.

    ``wide`` (the TMA-fed kernel, long contexts): few requests leave most SMs idle with 8 slices (one request on
    4 kv heads: 32 blocks), so the slices become 2, 4 or 8 clusters of 8 whose results meet in scratch memory,
    as long as a slice keeps 8 tiles of 64 keys and all blocks still fit one wave.  One request of 32,768 tokens:
    64.7 us with 8 slices, 23.4 us with 64; two of 16,384: 35.8 against 27.7 with 32; with 32 blocks or more
    (8 requests) 8 slices are the fastest at every length."""
    sms = sms or sm_count()
    blocks = n_requests * n_kv * ((group + 15) // 16)
    tiles = max(1, (max_seq_len + 63) // 64)
    most = max(1, min((2 * sms) // blocks, tiles, 8))
    # a power of two: clusters of 3 blocks pack the SMs of a GPC badly (24 requests x 4 kv heads: 24.8 us with 3
    # slices, 17.2 us with 2)
    slices = 1 << (most.bit_length() - 1)
    if wide and slices == 8:
        clusters = max(1, min((2 * sms) // (blocks * 8), tiles // 64, 8))
        slices = 8 * (1 << (clusters.bit_length() - 1))
    return slices


# Tiles of keys and values in the ring of a block of the TMA-fed decode attention.  With two, each pair of warps has
# one buffer and cannot fetch its next tile before it is done with this one: a block that walks many tiles (64
# requests of 1,024 tokens: 16 each) moves a tile per pair in the time of its products plus a trip to memory.  With
# three the third fills while both pairs work: a decode step of 64 requests 3.68 -> 3.62 ms, of 64 at 4,000 tokens
# 5.51 -> 5.27, of 32 at 16,000 7.78 -> 7.31, of 8 at 30,000 4.85 -> 4.65, of 8 at 1,024 2.70 -> 2.69.
DECODE_RING_STAGES = 3


def fuses_rope(qkv: torch.Tensor, ctx, head_dim: int, n_q: int, n_kv: int, page_size: int) -> bool:
    """Whether ``paged_attention`` should do the rotation and the page write of this step itself (``rope=``):
    bfloat16 steps in which every request brings one token.  With the TMA-fed decode kernel always (3.90
    against 3.94 ms a step at 64 requests, 3.01 against 3.08 at 8); with the cp.async one only up to the batch
    at which the projection before it is the tcgen05 kernel, since behind the library product the separate
    rotary kernel is what lets the attention kernel fetch cached keys early (4.18 against 4.28 ms at 64)."""
    if qkv.dtype != torch.bfloat16 or not ctx.is_decode_only:
        return False
    return tcgen05_attention_fits(head_dim, n_q, n_kv, page_size, 0) or qkv.shape[0] <= CLUSTER_BATCH


def paged_attention(qkv: torch.Tensor, out: torch.Tensor, kv: torch.Tensor, block_tables: torch.Tensor,
                    ctx, n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0,
                    rope: tuple[torch.Tensor | None, int] | None = None) -> None:
    """Attention of the step's rows over the pages, choosing the kernel for the batch.

    ``qkv`` is the stacked projection output [N, (n_q + 2 n_kv) * D] whose first n_q heads are the
    rotated queries; ``ctx`` gives the rows of each request (``q_start``), the cached lengths after
    this step (``seq_lens``) and the lists of query tiles.  float32 runs the CUDA-core kernel;
    bfloat16 the tensor-core kernels: the split decode kernel when every request brings one token, else
    the tcgen05 kernel (head size 64 or 128, no window) or the mma.sync tiled kernel.

    ``rope`` (only where ``fuses_rope``): queries and keys of ``qkv`` are not rotated yet and the newest keys
    and values not yet in their pages; the decode kernel does both."""
    if rope is not None and not (qkv.dtype == torch.bfloat16 and ctx.is_decode_only):
        raise KernelError("only bfloat16 decode steps rotate inside the attention kernel")
    if qkv.dtype == torch.float32:
        tile_req, tile_q0 = ctx.query_tiles(16)
        paged_attention_simt(qkv, qkv.shape[1], out, kv, block_tables, tile_req, tile_q0, ctx.q_start,
                             ctx.seq_lens, n_q, n_kv, head_dim, scale, window)
        return
    group = n_q // n_kv
    if ctx.is_decode_only:
        static = ctx.extras.get("static_max_seq_len")  # fixed when the step is captured
        longest = static or ctx.max_seq_len
        wide = ctx.extras.get("decode_wide", False) if static else is_long_context(ctx.max_seq_len)
        wide = bool(wide) and tcgen05_attention_fits(head_dim, n_q, n_kv, kv.shape[3], 0)
        slices = decode_slices(ctx.num_requests, n_kv, group, min(longest, window or longest), wide,
                               sm_count(qkv.device))
        scratch = ctx.extras.get(("decode_scratch", n_q, head_dim))
        paged_attention_decode(qkv, qkv.shape[1], out, kv, block_tables, ctx.q_start, ctx.seq_lens,
                               ctx.num_requests, n_q, n_kv, head_dim, scale, window, slices, scratch, rope,
                               stages=DECODE_RING_STAGES)
        return
    if tcgen05_attention_fits(head_dim, n_q, n_kv, kv.shape[3], window):
        tile_req, tile_tok0 = ctx.query_tiles_longest_first(128 // group)
        key = ("prefill_key_parts", 128 // group, n_kv)
        parts = ctx.extras.get(key)
        if parts is None:  # the same for every layer of the step
            parts = ctx.extras[key] = prefill_key_parts(ctx.q_lens_host, ctx.seq_lens_host, 128 // group, n_kv,
                                                        sm_count(qkv.device))
        paged_attention_prefill_tcgen05(qkv, qkv.shape[1], out, kv, block_tables, tile_req, tile_tok0, ctx.q_start,
                                        ctx.seq_lens, n_q, n_kv, head_dim, scale, parts)
        return
    tile_req, tile_row0 = ctx.query_tiles(64, group)
    paged_attention_prefill(qkv, qkv.shape[1], out, kv, block_tables, tile_req, tile_row0, ctx.q_start,
                            ctx.seq_lens, n_q, n_kv, head_dim, scale, window)


# --------------------------------------------------------------------------- sampling

def argmax(logits: torch.Tensor, with_status: bool = False) -> torch.Tensor:
    """Index of the largest value of each row of float32 ``logits`` [M, V]; the lowest index wins ties.

    ``with_status``: the result has M + 1 elements, the last being the device error word as it stood when the
    kernel ran (``raise_for_status`` reads it on the host), so that the copy that fetches the tokens also tells
    whether a kernel of the step flagged anything."""
    _need(logits, torch.float32, "logits")
    m, v = logits.shape
    out = torch.empty(m + int(with_status), dtype=torch.int32, device=logits.device)
    scratch = torch.empty(m * 32, dtype=torch.int64, device=logits.device)  # one packed word per (row, chunk)
    status = error_word(logits.device).data_ptr() if with_status else None
    _check(ops_library().ss_argmax(logits.data_ptr(), out.data_ptr(), m, v, logits.stride(0), scratch.data_ptr(),
                                   status, _stream()), "argmax")
    _launches[0] += 1  # two kernels
    return out


def sample(logits: torch.Tensor, *, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, penalty: torch.Tensor, seeds: torch.Tensor, draws: torch.Tensor,
           slots: torch.Tensor | None = None, seen: torch.Tensor | None = None,
           with_status: bool = False) -> torch.Tensor:
    """One token per row of float32 ``logits`` [M, V] with per-row parameters (device tensors [M]):
    repetition penalty (needs ``seen`` int32 [slots, ceil(V/32)] and ``slots``), temperature (0 = arg-max),
    top-k (-1 off), top-p, min-p, then a Gumbel-max draw keyed by (seed, draw index).  ``with_status`` as in
    ``argmax``."""
    _need(logits, torch.float32, "logits")
    m, v = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                        ("penalty", penalty, torch.float32), ("seeds", seeds, torch.int64),
                        ("draws", draws, torch.int64)):
        _need(t, dt, name)
        if t.numel() != m:
            raise KernelError(f"{name} must hold one value per row")
    seen_words = 0
    if seen is not None:
        _need(seen, torch.int32, "seen")
        _need(slots, torch.int32, "slots")
        seen_words = seen.shape[1]
        if seen_words * 32 < v:
            raise KernelError("the seen-token mask is narrower than the vocabulary")
    out = torch.empty(m + int(with_status), dtype=torch.int32, device=logits.device)
    status = error_word(logits.device).data_ptr() if with_status else None
    _check(ops_library().ss_sample(logits.data_ptr(), logits.stride(0), out.data_ptr(), temperature.data_ptr(),
                                   top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(), penalty.data_ptr(),
                                   seeds.data_ptr(), draws.data_ptr(), _ptr(seen), seen_words,
                                   _ptr(slots) if seen is not None else None, m, v, status, _stream()), "sample")
    return out


def mark_seen(seen_row: torch.Tensor, token_ids: torch.Tensor, vocab: int) -> None:
    """Set the bits of ``token_ids`` (int32) in one request's row of the seen-token mask."""
    _need(seen_row, torch.int32, "seen row")
    _need(token_ids, torch.int32, "token_ids")
    _check(ops_library().ss_mark_seen(seen_row.data_ptr(), token_ids.data_ptr(), token_ids.numel(), vocab,
                                      _stream()), "mark_seen")


# --------------------------------------------------------------------------- tensor-core matrix product

_GEMM_COUNTERS = 8192
_GEMM_SCRATCH_FLOATS = 8 * 1024 * 1024


def _gemm_workspace(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Split-K scratch (partial tiles) and per-tile counters; the counters are zero between calls."""
    key = f"gemm_ws{device}"
    ws = _state.get(key)
    if ws is None:
        ws = (torch.empty(_GEMM_SCRATCH_FLOATS, dtype=torch.float32, device=device),
              torch.zeros(_GEMM_COUNTERS, dtype=torch.int32, device=device))
        _state[key] = ws
    return ws  # type: ignore[return-value]


@dataclasses.dataclass
class PendingNorm:
    """``weight * round(stream * rsqrt(mean(stream^2) + eps))`` that has not been computed: the stream is complete
    (the branch in front has been added), ``scaled`` holds ``round(weight * stream)`` in bfloat16 and ``squares``
    [tokens, tiles] the sums of the stream's squares per tile of 128 features.  `linear` and `gate_up_swiglu` take it
    in place of the activations: with few bfloat16 tokens the product runs on ``scaled`` and multiplies every
    token's output by its ``rsqrt(...)`` at the end (the scale does not depend on the feature, so it commutes with
    the product; the activations are then rounded once instead of twice).  Everything else calls
    ``materialize()``, the norm kernel on the stream."""
    stream: torch.Tensor
    scaled: torch.Tensor
    squares: torch.Tensor
    weight: torch.Tensor
    eps: float
    dtype: torch.dtype

    @property
    def shape(self) -> torch.Size:
        return self.stream.shape

    @property
    def device(self) -> torch.device:
        return self.stream.device

    def materialize(self) -> torch.Tensor:
        return add_rmsnorm(self.stream, None, self.weight, self.eps, self.dtype)


def takes_pending_norm(x: "torch.Tensor | PendingNorm", features: int, swiglu: bool = False) -> bool:
    """Whether the product of ``x`` with a [features, K] weight applies the norm's scale inside the kernel: the
    streaming kernel of decode steps, or the two-SM kernel of long prompt portions."""
    if not isinstance(x, PendingNorm) or x.dtype != torch.bfloat16:
        return False
    sms = sm_count(x.device)
    if x.shape[0] <= CLUSTER_BATCH and streams_weights(x.shape[0], features, x.shape[1], sms):
        return True
    if swiglu:
        return x.shape[1] % 8 == 0 and many_tokens_swiglu_fits(x.shape[0], features, sms)
    return many_tokens_fits(x.shape[0], features, x.shape[1], sms)


def gemm_plan(tokens: int, features: int, k: int, sms: int | None = None) -> tuple[bool, int, int]:
    """(swapped, tile width, K slices) for ``x[tokens, k] @ w[features, k].T`` on ``sms`` multiprocessors."""
    return _gemm_plan(tokens, features, k, sms or sm_count())


@functools.lru_cache(maxsize=None)
def _gemm_plan(tokens: int, features: int, k: int, sms: int) -> tuple[bool, int, int]:
    k_iters = (k + 63) // 64
    if tokens <= 64:
        bn = 16 if tokens <= 16 else (32 if tokens <= 32 else 64)
        tiles = (features + 127) // 128
        # at most 8 slices: they then form one thread-block cluster and are added through shared memory
        slices = max(1, min(k_iters, (2 * sms + tiles - 1) // tiles if tiles < sms else 1, 8))
        # the widest tile leaves room for two blocks per SM, and clusters do not pack an SM's last slot: stay
        # within one wave of blocks (36 tiles x 8 slices ran as two waves: 18.1 us against 13.2 with 7 slices)
        while bn == 64 and slices > 1 and tiles * slices > sms + (3 * sms) // 4:
            slices -= 1
        return True, bn, slices
    bn = 256 if features >= 256 else (128 if features >= 128 else (64 if features >= 64 else (32 if features >= 32 else 16)))
    return False, bn, 1


def gemm_tcgen05(x: "torch.Tensor | PendingNorm", weight: torch.Tensor, bias: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None, plan: tuple[bool, int, int] | None = None,
                 swiglu: bool = False, to_stream: tuple[torch.Tensor, torch.Tensor] | None = None):
    """``x @ weight.T + bias`` for bfloat16 ``x`` [tokens, K] and ``weight`` [features, K] on the tcgen05 tensor
    cores (TMA-fed, accumulator in tensor memory); output bfloat16 or float32.  K must be a multiple of 8.

    ``swiglu`` (at most 64 tokens, features a multiple of 128): the weight's rows alternate 64 gate and 64 up
    features; the result is ``silu(gate) * up`` with features / 2 columns, formed in the product's epilogue.

    ``to_stream`` = (float32 stream [tokens, features], weights of the norm behind it), where `adds_to_stream`:
    the product, rounded to bfloat16, is added to the stream in place instead of being returned, and the function
    returns (round(norm weights * new stream) in bfloat16, sums of squares [tokens, features / 128]).
    ``x`` may be a `PendingNorm` (at most 16 tokens): the product runs on its ``scaled`` and applies the scale of
    every token in the epilogue."""
    pending = x if isinstance(x, PendingNorm) else None
    if pending is not None:
        if pending.dtype != torch.bfloat16:
            raise KernelError("a pending norm feeds the tensor-core product only in bfloat16")
        x = pending.scaled
    _need(x, torch.bfloat16, "x")
    _need(weight, torch.bfloat16, "weight")
    tokens, k = x.shape
    features = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"weight {tuple(weight.shape)} does not match x {tuple(x.shape)}")
    if k % 8 != 0:
        raise KernelError(f"the tensor-core matrix product needs K to be a multiple of 8, got {k}")
    out_dtype = out_dtype or torch.bfloat16
    if swiglu and (tokens > 64 or features % 128):
        raise KernelError("the fused SwiGLU epilogue takes at most 64 tokens and a multiple of 128 weight rows")
    out_shape = (tokens, features // 2 if swiglu else features)
    out = None if to_stream is not None else torch.empty(out_shape, dtype=out_dtype, device=x.device)
    if tokens == 0:
        return out
    bias_f32 = 0
    if bias is not None:
        _need(bias, None, "bias")
        bias_f32 = int(bias.dtype == torch.float32)
        if bias.numel() != features or bias.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("bias has the wrong size or dtype")
    swapped, bn, slices = plan or gemm_plan(tokens, features, k, sm_count(x.device))
    partial = counters = None
    if slices > 1 and not (swapped and slices <= 8 and tokens <= bn):
        partial, counters = _gemm_workspace(x.device)
        tiles = ((features if swapped else tokens) + 127) // 128 * (((tokens if swapped else features) + bn - 1) // bn)
        if tiles > _GEMM_COUNTERS or tiles * slices * bn * 128 > _GEMM_SCRATCH_FLOATS:
            raise KernelError("split-K workspace too small for this problem")
    a, b = (weight, x) if swapped else (x, weight)
    if to_stream is not None:
        stream, norm_weight = to_stream
        _need(stream, torch.float32, "stream")
        _need(norm_weight, None, "norm weight")
        if (swiglu or pending is not None or out_dtype != torch.bfloat16 or tuple(stream.shape) != out_shape
                or not (swapped and 2 <= slices <= 8 and tokens <= bn) or features % 128
                or norm_weight.numel() != features or norm_weight.dtype not in (torch.float32, torch.bfloat16)):
            raise KernelError("a product into the stream needs its plain bfloat16 output, K slices in a cluster, a "
                              "width in steps of 128 and a stream of its shape")
        scaled = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
        squares = torch.empty((tokens, features // 128), dtype=torch.float32, device=x.device)
        rc = gemm_library().ss_gemm_tc5_to_stream(a.data_ptr(), b.data_ptr(), _ptr(bias), bias_f32, a.shape[0], b.shape[0],
                                                  k, k, k, bn, slices, stream.data_ptr(), squares.data_ptr(),
                                                  scaled.data_ptr(), norm_weight.data_ptr(),
                                                  int(norm_weight.dtype == torch.float32),
                                                  error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05 into the stream")
        return scaled, squares
    if pending is not None:
        if not swapped or bn != 16 or pending.weight.numel() != k or pending.squares.shape[0] != tokens:
            raise KernelError("a pending norm feeds the swapped product of at most 16 tokens, over the stream's whole width")
        rc = gemm_library().ss_gemm_tc5_scaled(a.data_ptr(), b.data_ptr(), pending.squares.data_ptr(),
                                               pending.squares.shape[1], float(pending.eps), _ptr(bias), bias_f32,
                                               out.data_ptr(), a.shape[0], tokens, k, k, k, out.shape[1], bn,
                                               int(out_dtype == torch.float32), slices, int(swiglu), _ptr(partial),
                                               _ptr(counters), error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05 behind a pending norm")
        return out
    rc = gemm_library().ss_gemm_tc5(a.data_ptr(), b.data_ptr(), _ptr(bias), bias_f32, out.data_ptr(), a.shape[0],
                                    b.shape[0], k, k, k, out.shape[1], bn, int(swapped), int(out_dtype == torch.float32),
                                    slices, int(swiglu), _ptr(partial), _ptr(counters),
                                    error_word(x.device).data_ptr(), _stream())
    _check(rc, "gemm_tcgen05")
    return out


def gemm_tcgen05_many(x: "torch.Tensor | PendingNorm", weight: torch.Tensor, bias: torch.Tensor | None = None,
                      out_dtype: torch.dtype | None = None, swiglu: bool = False, tile_cols: int = 0,
                      to_stream: tuple[torch.Tensor, torch.Tensor] | None = None):
    """``x @ weight.T + bias`` for many rows of ``x`` (prompt portions) on the tcgen05 tensor cores: a persistent
    kernel, one block per SM, the blocks in pairs (``tcgen05.mma.cta_group::2``: each block of a pair loads half
    of A and half of B) that compute tiles of 256 rows with the accumulator double-buffered in tensor memory, so
    that the epilogue of a tile overlaps the products of the next.  ``tile_cols``: the tiles' width, a multiple
    of 16 up to 256; 0 lets the launcher take the width whose tiles fill whole rounds of the pairs of SMs best.
    ``swiglu``: the weight's rows alternate 64 gate and 64 up features; the result is ``silu(gate) * up`` with
    features / 2 columns (tiles of 256 columns).  ``to_stream`` and a `PendingNorm` for ``x``: as in
    `gemm_tcgen05` (features a multiple of 16; the sums of squares come per tile of the chosen width)."""
    pending = x if isinstance(x, PendingNorm) else None
    if pending is not None:
        if pending.dtype != torch.bfloat16:
            raise KernelError("a pending norm feeds the tensor-core product only in bfloat16")
        x = pending.scaled
    _need(x, torch.bfloat16, "x")
    _need(weight, torch.bfloat16, "weight")
    tokens, k = x.shape
    features = weight.shape[0]
    if weight.shape[1] != k or k % 8 != 0:
        raise KernelError("the tensor-core matrix product needs matching K, a multiple of 8")
    out_dtype = out_dtype or torch.bfloat16
    if swiglu and (features % 128 or out_dtype != torch.bfloat16 or (features // 2) % 8):
        raise KernelError("the fused SwiGLU epilogue takes a multiple of 128 weight rows and writes bfloat16")
    out_shape = (tokens, features // 2 if swiglu else features)
    out = None if to_stream is not None else torch.empty(out_shape, dtype=out_dtype, device=x.device)
    if tokens == 0:
        return out
    bias_f32 = 0
    if bias is not None:
        _need(bias, None, "bias")
        bias_f32 = int(bias.dtype == torch.float32)
        if bias.numel() != features or bias.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("bias has the wrong size or dtype")
    if to_stream is not None:
        stream, norm_weight = to_stream
        _need(stream, torch.float32, "stream")
        _need(norm_weight, None, "norm weight")
        if (swiglu or pending is not None or out_dtype != torch.bfloat16 or tuple(stream.shape) != out_shape or features % 16
                or norm_weight.numel() != features or norm_weight.dtype not in (torch.float32, torch.bfloat16)):
            raise KernelError("a product into the stream needs its plain bfloat16 output, a width in steps of 16 and a "
                              "stream of its shape")
        width = tile_cols or gemm_library().ss_gemm_tc5_many_tile_cols(tokens, features, 0)
        scaled = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
        squares = torch.empty((tokens, (features + width - 1) // width), dtype=torch.float32, device=x.device)
        rc = gemm_library().ss_gemm_tc5_many_to_stream(x.data_ptr(), weight.data_ptr(), _ptr(bias), bias_f32, tokens,
                                                       features, k, k, k, width, stream.data_ptr(), squares.data_ptr(),
                                                       scaled.data_ptr(), norm_weight.data_ptr(),
                                                       int(norm_weight.dtype == torch.float32),
                                                       error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05_many into the stream")
        return scaled, squares
    if pending is not None:
        if pending.weight.numel() != k or pending.squares.shape[0] != tokens:
            raise KernelError("a pending norm feeds a product over the stream's whole width")
        rc = gemm_library().ss_gemm_tc5_many_scaled(x.data_ptr(), weight.data_ptr(), pending.squares.data_ptr(),
                                                    pending.squares.shape[1], float(pending.eps), _ptr(bias), bias_f32,
                                                    out.data_ptr(), tokens, features, k, k, k, out.shape[1],
                                                    int(out_dtype == torch.float32), int(swiglu), tile_cols,
                                                    error_word(x.device).data_ptr(), _stream())
        _check(rc, "gemm_tcgen05_many behind a pending norm")
        return out
    rc = gemm_library().ss_gemm_tc5_many(x.data_ptr(), weight.data_ptr(), _ptr(bias), bias_f32, out.data_ptr(), tokens,
                                         features, k, k, k, out.shape[1], int(out_dtype == torch.float32), int(swiglu),
                                         tile_cols, error_word(x.device).data_ptr(), _stream())
    _check(rc, "gemm_tcgen05_many")
    return out


# From this many tokens a bfloat16 projection whose 256 x 256 output tiles make at least a round and a half of the
# pairs of SMs, and whose K is deep enough for a tile's first loads and its epilogue to be a small part of it
# (``many_tokens_fits``), runs the persistent two-SM kernel.  Against the library (us, ours / library) at 2,048 tokens: 7B sizes q/k/v 49.6 / 45.1, o 41.6-47.7 /
# 45.4-52.8, down 191.9-198.2 / 191.6-208.7; 14B sizes 109.4 / 114.6, 79.7 / 77.0, 200.3 / 207.2; a whole 2,048-token
# prefill of the 7B shape takes 22.1 to 25.5 ms either way (the GPU sits at its power cap), and its first call 35
# ms instead of 160.  With fewer tokens or smaller weights there are too few 256-row tiles for the pairs of SMs and
# the library, which splits K, wins: 1,024 tokens at 14B sizes by up to 18 %, 0.5B and 1.5B sizes at any number
# of tokens by up to 50 %, 512 tokens and below by 1.3 to 2 times.  (Cutting K into parts inside this kernel,
# with the parts' sums meeting in scratch memory, was tried for those cases and did not beat narrower tiles.)
MANY_TOKENS = 2048
MANY_K_STEPS = 32  # 64-wide K steps a tile must have (2,048 columns)


def many_tokens_fits(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """Where the persistent two-SM tcgen05 kernel is the product of a prompt portion (see the measurements above):
    at the 7B and 14B layer sizes from 2,048 tokens (112 to 224 tiles on 74 pairs), not at the 0.5B and 1.5B sizes
    (40 to 48 tiles, K of 896 and 1,536)."""
    if tokens < MANY_TOKENS or k % 8 != 0 or k < 64 * MANY_K_STEPS:
        return False
    tiles = ((tokens + 255) // 256) * ((features + 255) // 256)
    return 4 * tiles >= 3 * (sms or sm_count())  # a round and a half of the sms / 2 pairs


SMALL_BATCH = 64  # up to this many tokens a projection may stream its weights through the tcgen05 kernel
# ... when its 128-row weight tiles are at least as many as the SMs (no K slices needed)
CLUSTER_BATCH = 16  # ... or, up to this many tokens, whatever its size (K slices added inside a cluster)
DEEP_K = 8192  # ... or when K is at least this deep: every block then streams enough to pay for its set-up


def streams_weights(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """True where the hand-written tcgen05 kernel is the faster way to run a bfloat16 projection.  Measured
    on the 7B shape inside a decode step: with enough weight tiles to give every SM one (gate/up, LM head) it
    wins up to 64 tokens (43 us against the library's 46.5 us at 8 tokens); the smaller products (q/k/v, o,
    down), whose K range is cut into slices that a thread-block cluster adds, win up to 16 tokens (a step of
    8 requests: 3.18 ms against 3.41 ms with the library's split-K kernels); at 32 and 64 tokens only the
    down product still wins (25.6 and 28.0 us against 29.1 and 30.8), q/k/v and o lose by 1 to 9 us."""
    if k % 8 != 0 or tokens > SMALL_BATCH:
        return False
    return tokens <= CLUSTER_BATCH or (features + 127) // 128 >= (sms or sm_count()) or k >= DEEP_K


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """A projection ``x @ weight.T + bias``.

    float32 runs the CUDA-core kernel (no reduced-precision matrix mode).  bfloat16 with few tokens (decode
    steps) and a large weight runs the hand-written tcgen05 kernel, which streams the weights once and
    overlaps its first fetches with the kernel before it; from ``MANY_TOKENS`` tokens (prompt portions) and with
    enough output tiles (``many_tokens_fits``) the persistent two-SM tcgen05 kernel; everything else runs the
    library matrix product, as the reference's
    nn.Linear does (slipstream/models/layers/attention.py:132-135).  ``x`` may be a `PendingNorm`."""
    if isinstance(x, PendingNorm):
        if not takes_pending_norm(x, weight.shape[0]):
            x = x.materialize()
        elif x.shape[0] <= CLUSTER_BATCH:
            return gemm_tcgen05(x, weight, bias, out_dtype)
        else:
            return gemm_tcgen05_many(x, weight, bias, out_dtype)
    if x.dtype == torch.float32:
        return gemm_simt(x, weight, bias, out_dtype)
    sms = sm_count(x.device)
    if streams_weights(x.shape[0], weight.shape[0], x.shape[1], sms):
        return gemm_tcgen05(x, weight, bias, out_dtype)
    if many_tokens_fits(x.shape[0], weight.shape[0], x.shape[1], sms):
        return gemm_tcgen05_many(x, weight, bias, out_dtype)
    if out_dtype is None or out_dtype == x.dtype:
        if bias is not None:
            return torch.addmm(bias, x, weight.t())
        return torch.mm(x, weight.t())
    out = torch.mm(x, weight.t(), out_dtype=out_dtype)
    if bias is not None:
        out += bias
    return out


def adds_to_stream(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """True where a bfloat16 projection can add its output to the float32 stream itself and prepare the norm
    behind it: the streaming tcgen05 kernel with its K slices as a thread-block cluster (decode steps), a width in
    steps of 128."""
    sms = sms or sm_count()
    if not _state.get("norm_rides_along", True):
        return False
    if _state.get("norm_rides_along_long", False) and features % 16 == 0 and many_tokens_fits(tokens, features, k, sms):
        return True  # the two-SM kernel of long prompt portions: every thread of its epilogue has a row
    if features % 128 != 0 or tokens > CLUSTER_BATCH or not streams_weights(tokens, features, k, sms):
        return False
    swapped, bn, slices = gemm_plan(tokens, features, k, sms)
    return swapped and 2 <= slices <= 8 and tokens <= bn


def set_norm_fusion(enabled: bool, long_portions: bool = False) -> None:
    """Whether `linear_add_rmsnorm` may leave the norm to the products around it (on by default; off for
    comparisons).  ``long_portions``: also in the two-SM kernel of prompt portions from 2,048 tokens.  That is off
    unless asked for, by measurement at the 7B sizes: the o and down products with the add inside take 71 and 225
    us, as long as the product followed by the norm kernel (72 and 225: the read-modify-write of the stream from
    an epilogue that holds a row per thread costs what the norm kernel cost), q/k/v and gate/up with the scale
    in their epilogue take what they took, and a whole 2,048-token step 21.67 ms against 21.5 to 21.6."""
    _state["norm_rides_along"] = bool(enabled)
    _state["norm_rides_along_long"] = bool(enabled and long_portions)


def linear_add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor,
                       norm_weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> "torch.Tensor | PendingNorm":
    """``residual += x @ weight.T + bias`` (float32 stream, in place; the branch output rounded to the compute dtype
    first), then the RMS norm of the stream times ``norm_weight``: a branch's last projection with the add and the
    norm that follow it.  With few bfloat16 tokens the projection adds to the stream in its epilogue and the
    norm comes back as a `PendingNorm`, to be finished by the next product (no norm kernel); everything
    else is `linear` followed by `add_rmsnorm`."""
    if x.shape[0] > 0 and x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 \
            and residual.shape == (x.shape[0], weight.shape[0]) \
            and norm_weight.numel() == weight.shape[0] \
            and adds_to_stream(x.shape[0], weight.shape[0], x.shape[1], sm_count(x.device)):
        product = gemm_tcgen05 if x.shape[0] <= SMALL_BATCH else gemm_tcgen05_many
        scaled, squares = product(x, weight, bias, to_stream=(residual, norm_weight))
        return PendingNorm(residual, scaled, squares, norm_weight, eps, out_dtype)
    return add_rmsnorm(residual, linear(x, weight, bias), norm_weight, eps, out_dtype)


def many_tokens_swiglu_fits(tokens: int, features: int, sms: int | None = None) -> bool:
    """Where the persistent tcgen05 kernel with its fused SwiGLU epilogue is at least as fast as the library
    product followed by the SwiGLU kernel: enough 256 x 256 tiles to keep every pair of SMs busy for several
    rounds (2,048 tokens x 37,888 features: 347 us against 348 + 40 us, and no [tokens, 2 I] intermediate; 1,024
    tokens: 205 against 179 + 20; 512 tokens: 108 against 95 + 10, where the library stays).  Without an epilogue
    to fuse, the library product is as fast as ours or up to 10 % faster, and stays."""
    return ((tokens + 255) // 256) * ((features + 255) // 256) >= 4 * (sms or sm_count())


def gate_up_swiglu(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, block: int) -> torch.Tensor:
    """``silu(x @ Wg.T + bg) * (x @ Wu.T + bu)`` where ``weight`` [2 I, K] holds gate and up rows alternating in
    runs of ``block``.  Small bfloat16 batches with runs of 64 do it in one kernel.  ``x`` may be a `PendingNorm`."""
    if isinstance(x, PendingNorm):
        if block == 64 and weight.shape[0] % 128 == 0 and takes_pending_norm(x, weight.shape[0], swiglu=True):
            if x.shape[0] <= CLUSTER_BATCH:
                return gemm_tcgen05(x, weight, bias, swiglu=True)
            return gemm_tcgen05_many(x, weight, bias, swiglu=True)
        x = x.materialize()
    if x.dtype == torch.bfloat16 and block == 64 and weight.shape[0] % 128 == 0 and x.shape[1] % 8 == 0:
        sms = sm_count(x.device)
        if streams_weights(x.shape[0], weight.shape[0], x.shape[1], sms):
            return gemm_tcgen05(x, weight, bias, swiglu=True)
        if many_tokens_swiglu_fits(x.shape[0], weight.shape[0], sms):
            return gemm_tcgen05_many(x, weight, bias, swiglu=True)
    return swiglu(linear(x, weight, bias), block=block)


def set_programmatic_launch(enabled: bool) -> None:
    """Turn programmatic dependent launch of this package's kernels on or off (on by default)."""
    libs = [ops_library(), gemm_library()] + [lib for key, lib in _state.items() if isinstance(key, str) and key.startswith("attn")]
    for lib in libs:
        lib.ss_set_pdl.argtypes = [c_int]
        lib.ss_set_pdl.restype = None
        lib.ss_set_pdl(int(enabled))
    _state["pdl"] = bool(enabled)


__all__ = ["KernelError", "KernelBuildError", "embedding", "add_rmsnorm", "rope_and_cache", "swiglu",
           "gemm_simt", "paged_attention_simt", "paged_attention", "fuses_rope", "paged_attention_prefill", "paged_attention_prefill_tcgen05", "prefill_key_parts", "tcgen05_attention_fits", "paged_attention_decode", "decode_scratch", "decode_slices", "is_long_context", "require_cuda", "argmax", "sample", "mark_seen", "gather_tokens", "prepare_decode", "gemm_tcgen05", "gemm_tcgen05_many", "many_tokens_fits", "many_tokens_swiglu_fits", "gemm_plan", "gemm_library", "gate_up_swiglu", "set_programmatic_launch", "launch_count", "count_launches", "sm_count", "linear", "linear_add_rmsnorm", "adds_to_stream", "takes_pending_norm", "PendingNorm", "set_norm_fusion", "check_errors", "raise_for_status", "error_word", "ops_library",
           "attention_library"]
