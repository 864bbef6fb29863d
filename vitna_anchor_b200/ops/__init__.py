"""Python faces of the engine's CUDA kernels.

The kernels live in one shared library (csrc/, built by ops.build) with a C
interface; this module checks tensors (device, dtype, contiguity, shapes) and
passes raw pointers and the current CUDA stream.  There is no CPU fallback and
no library stand-in: if the library cannot be built or loaded, or a tensor is
not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

_lib = None

class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded kernel library; built at the first call if need be."""
    global _lib
    if _lib is None:
        # VITNA_KERNEL_LIB names a library that was built elsewhere from these sources (a read-only installation, a build
        # with other compiler flags); otherwise the in-tree library, compiled now if it is missing or out of date
        path = os.environ.get("VITNA_KERNEL_LIB") or _build.library_path(build=True)
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"the kernel library {path} could not be loaded: {e}") from None
    return _lib


_launches = 0

# The 32-bit path has two routings.  Exact (the default): every operation has ONE kernel, whatever the batch (the
# tile product, the row-wise norm, attention_rows), and each of them sums an output's terms in an order that
# depends on that output alone, so the logits of a position are the same BITS however the tokens are cut into
# steps, whatever else is in the batch and wherever the pages lie.  Fast (VITNA_FLOAT32_FAST=1 in the environment,
# or set_float32_exact(False)): the float32 twins of the serving kernels (few-rows products with fused norm,
# rotation and SwiGLU, split-key decode attention) are chosen by batch size as in bfloat16; the result then
# differs between ways of cutting by float32 rounding.
_float32_exact = os.environ.get("VITNA_FLOAT32_FAST", "") in ("", "0")


def set_float32_exact(exact: bool) -> bool:
    """Choose the routing of the 32-bit path (see above); returns the setting that was in force."""
    global _float32_exact
    before, _float32_exact = _float32_exact, bool(exact)
    return before


def float32_exact() -> bool:
    return _float32_exact


def launch_count() -> int:
    """Kernels of this library launched so far by this process (a graph replay counts the kernels it holds)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


_timed = None       # while kernel_times() runs: [(name of the launch, event recorded behind it)]


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        if _timed is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            _timed.append((what, ev))
        return
    fn = lib().vk_error_string
    fn.restype = ctypes.c_char_p
    text = fn(status).decode()
    if status < 0:
        raise KernelError(f"{what}: refused, {text}")
    raise KernelError(f"{what}: CUDA error {status}: {text}")


def kernel_times(fn) -> dict:
    """Run fn() with an event behind every launch of this library and return {launch name: (count, milliseconds)}: the time
    from the end of the launch before it to its own end.  Exact where the stream stays busy (a prompt's step, issued eagerly);
    where launches are shorter than the host takes to issue them, the gaps are counted too.  For measurements only."""
    global _timed
    torch.cuda.synchronize()
    _timed = []
    first = torch.cuda.Event(enable_timing=True)
    first.record()
    try:
        fn()
    finally:
        events, _timed = _timed, None
    torch.cuda.synchronize()
    out, before = {}, first
    for name, ev in events:
        n, ms = out.get(name, (0, 0.0))
        out[name] = (n + 1, ms + before.elapsed_time(ev))
        before = ev
    return out


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not one of float32, bfloat16")


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _req(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device; the engine has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} is {t.dtype}, expected {dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} has {t.dim()} dimensions, expected {dims}")


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# ---------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = float32(table[ids[t], :]); table [V, H] (float32 or bfloat16), ids int32 [T], out float32 [T, H]."""
    _req(table, "table", dims=2); _req(ids, "ids", torch.int32, 1); _req(out, "out", torch.float32, 2)
    if out.shape != (ids.shape[0], table.shape[1]):
        raise KernelError("embed_rows: out is not [tokens, hidden]")
    _check(lib().vk_embed_rows(_p(table), _p(ids), _p(out), ids.shape[0], table.shape[1], table.shape[0], _dt(table),
                               _stream()), "embed_rows")
    return out


def rmsnorm_rows(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r, :] = rmsnorm(x[rows[r], :]) * w; x float32 [T, n], w float32 [n], out [R, n] float32 or bfloat16."""
    _req(x, "x", torch.float32, 2); _req(w, "w", torch.float32, 1); _req(out, "out", dims=2)
    n = x.shape[1]
    if w.shape[0] != n or out.shape[1] != n:
        raise KernelError("rmsnorm_rows: widths differ")
    if rows is not None:
        _req(rows, "rows", torch.int32, 1)
        if rows.shape[0] != out.shape[0]:
            raise KernelError("rmsnorm_rows: rows and out differ in length")
    elif out.shape[0] != x.shape[0]:
        raise KernelError("rmsnorm_rows: out and x differ in rows")
    _check(lib().vk_rmsnorm_rows(_p(x), _p(w), _p(rows), _p(out), out.shape[0], n, ctypes.c_float(eps), _dt(out),
                                 _stream()), "rmsnorm_rows")
    return out


LINEAR_SAME, LINEAR_F32, LINEAR_ACC_F32 = 0, 1, 2


def linear_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, few_rows: int = 8) -> torch.Tensor:
    """out = x @ w.T on CUDA cores in float32 arithmetic.  x [M, K] (rows may be strided), w [N, K],
    out [M, N]: mode 0 stores in x's dtype, 1 stores float32, 2 adds into a float32 out."""
    if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("linear: x must be a CUDA matrix with unit column stride")
    _req(w, "w", x.dtype, 2); _req(out, "out", x.dtype if mode == LINEAR_SAME else torch.float32, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    ldx = x.stride(0) if M > 1 else max(K, x.stride(0))
    _check(lib().vk_linear_simt(_p(x), _p(w), _p(out), M, N, K, ldx, _dt(x), mode, few_rows, _stream()), "linear_simt")
    return out


def rope_store(qkv: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
               slot_mapping: Optional[torch.Tensor], q_out: torch.Tensor, cache_layer: Optional[torch.Tensor],
               nh: int, nkv: int, hd: int, rot: int, page_size: int) -> torch.Tensor:
    """Rotate q and k (half-split pairs within the first `rot` dimensions), write q to q_out and k, v into
    the layer's pages at slot_mapping (page * page_size + offset, or -1 for no write)."""
    _req(qkv, "qkv", dims=2); _req(positions, "positions", torch.int32, 1); _req(q_out, "q_out", qkv.dtype, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd or q_out.shape != (T, nh * hd) or positions.shape[0] != T:
        raise KernelError("rope_store: shapes do not fit the head counts")
    if rot > 0:
        _req(cos, "cos", torch.float32, 2); _req(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rot // 2 or sin.shape != cos.shape:
            raise KernelError("rope_store: tables are not [positions, rot/2]")
    if cache_layer is not None:
        _req(cache_layer, "cache_layer", qkv.dtype)
        _req(slot_mapping, "slot_mapping", torch.int32, 1)
        if tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd) or slot_mapping.shape[0] != T:
            raise KernelError("rope_store: the cache layer is not [pages, 2, nkv, page_size, hd]")
    _check(lib().vk_rope_store(_p(qkv), _p(positions), _p(cos if rot > 0 else None), _p(sin if rot > 0 else None),
                               _p(slot_mapping if cache_layer is not None else None), _p(q_out), _p(cache_layer), T, nh,
                               nkv, hd, rot, page_size, _dt(qkv), _stream()), "rope_store")
    return q_out


def attention_rows(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, token_seg: torch.Tensor,
                   positions: torch.Tensor, out: torch.Tensor, nh: int, nkv: int, hd: int, scale: float,
                   window: int = 0, tok_list: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every token (or of those in tok_list) over its request's pages (any sizes,
    float32 arithmetic)."""
    _req(q, "q", dims=2); _req(cache_layer, "cache_layer", q.dtype, 5); _req(block_tables, "block_tables", torch.int32, 2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(positions, "positions", torch.int32, 1); _req(out, "out", q.dtype, 2)
    T = q.shape[0]
    page_size = cache_layer.shape[3]
    if q.shape[1] != nh * hd or out.shape != q.shape or tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd):
        raise KernelError("attention_rows: shapes do not fit the head counts")
    if token_seg.shape[0] != T or positions.shape[0] != T:
        raise KernelError("attention_rows: per-token arrays differ in length")
    n = T
    if tok_list is not None:
        _req(tok_list, "tok_list", torch.int32, 1)
        n = tok_list.shape[0]
    _check(lib().vk_attention_rows(_p(q), _p(cache_layer), _p(block_tables), _p(token_seg), _p(positions), _p(tok_list), _p(out),
                                   n, nh, nkv, hd, page_size, block_tables.shape[1], ctypes.c_float(scale), window, _dt(q),
                                   _stream()), "attention_rows")
    return out


def attention_decode_scratch_bytes(tokens: int, nh: int, nkv: int, hd: int, max_context: int) -> int:
    fn = lib().vk_attention_decode_scratch_bytes
    fn.restype = ctypes.c_size_t
    return int(fn(tokens, nh, nkv, hd, max_context))


def attention_decode_takes(dtype: torch.dtype, hd: int, max_context: int = 0) -> bool:
    """Whether the split-key decode kernel takes this head size and context (else attention_rows does the work)."""
    vec = 4 if dtype == torch.float32 else 8
    return hd % vec == 0 and hd <= 256 and hd // vec <= 32 and max_context <= 128 * 256


def attention_decode(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, token_seg: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, scratch_tokens: int, nh: int, nkv: int,
                     hd: int, scale: float, max_context: int, grid_context: int, window: int = 0,
                     tok_list: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of single decoded tokens, split over the keys in runs of 256 absolute positions.
    scratch: a byte buffer of attention_decode_scratch_bytes(scratch_tokens, ...) that was zero at first use
    and is used by no other shape; max_context fixes its layout, grid_context (<= max_context) bounds the
    positions of this launch."""
    _req(q, "q", dims=2); _req(cache_layer, "cache_layer", q.dtype, 5); _req(block_tables, "block_tables", torch.int32, 2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(positions, "positions", torch.int32, 1); _req(out, "out", q.dtype, 2)
    _req(scratch, "scratch", torch.uint8, 1)
    T = q.shape[0]
    page_size = cache_layer.shape[3]
    if q.shape[1] != nh * hd or out.shape != q.shape or tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd):
        raise KernelError("attention_decode: shapes do not fit the head counts")
    n = T
    if tok_list is not None:
        _req(tok_list, "tok_list", torch.int32, 1)
        n = tok_list.shape[0]
    if scratch.numel() < attention_decode_scratch_bytes(scratch_tokens, nh, nkv, hd, max_context):
        raise KernelError("attention_decode: the scratch is too small")
    _check(lib().vk_attention_decode(_p(q), _p(cache_layer), _p(block_tables), _p(token_seg), _p(positions), _p(tok_list),
                                     _p(out), _p(scratch), scratch_tokens, n, nh, nkv, hd, page_size, cache_layer.shape[0],
                                     block_tables.shape[1], max_context, grid_context, ctypes.c_float(scale), window, _dt(q),
                                     _p(error_word()), _stream()),
           "attention_decode")
    return out


def set_decode_tma(mode: int) -> int:
    """Which decode-attention launches the persistent TMA kernel takes: 0 none, 1 all whose sizes it takes, 2 those its
    size rule gives it (the default).  Returns the mode that was in force."""
    return int(lib().vk_set_decode_tma(int(mode)))


def set_decode_tma_few(mode: int) -> int:
    """Whether the persistent TMA decode attention takes head groups of at most eight with the keys as the rows of its
    products (1, the default; VITNA_DECODE_TMA_FEW=0 sets the other at start) or with the heads as rows (0), as it takes
    larger groups.  Returns what was in force."""
    return int(lib().vk_set_decode_tma_few(int(mode)))


def set_skinny_stream(mode: int) -> int:
    """Which few-rows products the streaming tensor-core kernel takes: 0 none, 1 all whose sizes it takes, 2 those its
    size rule gives it (the default; VITNA_SKINNY_STREAM sets the initial mode).  Returns the mode that was in force."""
    return int(lib().vk_set_skinny_stream(int(mode)))


def silu_mul(gu: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = silu(gu[:, :I]) * gu[:, I:]."""
    _req(gu, "gu", dims=2); _req(out, "out", gu.dtype, 2)
    T, two_i = gu.shape
    if two_i % 2 or out.shape != (T, two_i // 2):
        raise KernelError("silu_mul: out is not [tokens, width/2]")
    _check(lib().vk_silu_mul(_p(gu), _p(out), T, two_i // 2, _dt(gu), _stream()), "silu_mul")
    return out


def add_inplace(y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """y (float32) += x (float32 or bfloat16)."""
    _req(y, "y", torch.float32); _req(x, "x")
    if y.numel() != x.numel():
        raise KernelError("add_inplace: sizes differ")
    _check(lib().vk_add_inplace(_p(y), _p(x), ctypes.c_size_t(y.numel()), _dt(x), _stream()), "add_inplace")
    return y


def take_tokens(tokens: torch.Tensor, ids: torch.Tensor, src: torch.Tensor) -> None:
    """tokens[i] = ids[src[i]] where src[i] >= 0 (all int32, on the device)."""
    _req(tokens, "tokens", torch.int32, 1); _req(ids, "ids", torch.int32, 1); _req(src, "src", torch.int32, 1)
    if src.shape[0] != tokens.shape[0]:
        raise KernelError("take_tokens: tokens and src differ in length")
    _check(lib().vk_take_tokens(_p(tokens), _p(ids), _p(src), tokens.shape[0], _stream()), "take_tokens")


_argmax_scratch = None


def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = the lowest id among the maxima of logits[r, :]."""
    _req(logits, "logits", torch.float32, 2); _req(out, "out", torch.int32, 1)
    if out.shape[0] != logits.shape[0]:
        raise KernelError("argmax_rows: out and logits differ in rows")
    global _argmax_scratch
    rows = logits.shape[0]
    if _argmax_scratch is None or _argmax_scratch.numel() < rows * 12 or _argmax_scratch.device != logits.device:
        _argmax_scratch = torch.zeros(max(rows, 256) * 12, dtype=torch.uint8, device=logits.device)
    _check(lib().vk_argmax_rows(_p(logits), _p(out), _p(_argmax_scratch), rows, logits.shape[1], _stream()), "argmax_rows")
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                uniform: torch.Tensor, probs_scratch: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One token per row: greedy where temperature <= 0, else temperature / top-k / top-p with the row's uniform."""
    _req(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    _req(temperature, "temperature", torch.float32, 1); _req(top_k, "top_k", torch.int32, 1)
    _req(top_p, "top_p", torch.float32, 1); _req(uniform, "uniform", torch.float64, 1)
    _req(probs_scratch, "probs_scratch", torch.float32); _req(out, "out", torch.int32, 1)
    if min(temperature.shape[0], top_k.shape[0], top_p.shape[0], uniform.shape[0], out.shape[0]) < R:
        raise KernelError("sample_rows: a per-row array is shorter than the rows")
    if probs_scratch.numel() < R * V:
        raise KernelError("sample_rows: the scratch is smaller than [rows, vocab]")
    _check(lib().vk_sample_rows(_p(logits), _p(temperature), _p(top_k), _p(top_p), _p(uniform), _p(probs_scratch), _p(out),
                                R, V, _stream()), "sample_rows")
    return out


_error_word = None


def error_word() -> torch.Tensor:
    """A pinned host word that kernels with bounded waits set when a wait runs out (the device writes it
    through the mapped address; the host reads it for free after any synchronisation)."""
    global _error_word
    if _error_word is None:
        _error_word = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _error_word


class KernelGaveUp(KernelError):
    """A kernel's bounded wait ran out; what it and the kernels after it wrote is not valid."""


def device_error_code() -> int:
    """The code the last kernel that gave up a wait left (0: none), without clearing it.  The word is host memory,
    so reading it costs nothing; it is up to date after any synchronisation with the kernels in question."""
    return 0 if _error_word is None else int(_error_word[0])


def check_device_errors() -> None:
    """Raise if a kernel gave up a bounded wait since the last check (call after a synchronisation)."""
    code = device_error_code()
    if code != 0:
        _error_word[0] = 0
        raise KernelGaveUp(f"a kernel gave up waiting on an mbarrier (code {code}); its results are not valid")


def set_wait_limit_ms(ms: float) -> None:
    """The limit of one wait inside the kernels that wait on mbarriers, for every launch from now on, in
    milliseconds at the device's highest clock (0 or less: the default, about a second).  Launches that a CUDA
    graph already holds keep the limit they were captured with."""
    status = lib().vk_set_wait_limit_ms(ctypes.c_double(float(ms)))
    if status != 0:
        raise KernelError(f"set_wait_limit_ms: CUDA error {status}")


WAIT_FAMILIES = {"linear_tcgen05": 1, "linear_tcgen05_wide": 2, "attention_prefill_tcgen05": 3, "attention_decode_tma": 4}


def skip_stage_once(family: str, stage: int) -> None:
    """For tests of the give-up path: the next launch of the named kernel family leaves one pipeline stage of
    every block unarmed and unfilled, so its waits run out, the error word is set and the kernel returns by
    itself.  Nothing faults: no address is out of range and nothing traps."""
    lib().vk_test_skip_stage(WAIT_FAMILIES[family], int(stage))


def tcgen05_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands (bfloat16, K and the row stride multiples of 8, aligned)."""
    return (x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int) -> torch.Tensor:
    """out (=, or += in mode 2) x @ w.T in bfloat16 on the tcgen05 tensor cores, float32 accumulation in tensor memory."""
    if not tcgen05_takes(x, w):
        raise KernelError("linear_tcgen05: operands must be bfloat16, 16-byte aligned, with K and the row stride multiples of 8")
    _req(w, "w", torch.bfloat16, 2); _req(out, "out", torch.bfloat16 if mode == LINEAR_SAME else torch.float32, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    _check(lib().vk_linear_tcgen05(_p(x), _p(w), _p(out), M, N, K, x.stride(0), mode, _p(error_word()), _stream()), "linear_tcgen05")
    return out


def linear_tcgen05_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out [M, I] = silu(x @ gate.T) * (x @ up.T) in one tcgen05 kernel; w_gate_up [2I, K], gate rows then up rows."""
    if not tcgen05_takes(x, w_gate_up):
        raise KernelError("linear_tcgen05_swiglu: operands must be bfloat16, 16-byte aligned, with K and the row stride multiples of 8")
    _req(w_gate_up, "w_gate_up", torch.bfloat16, 2); _req(out, "out", torch.bfloat16, 2)
    M, K = x.shape
    inter = w_gate_up.shape[0] // 2
    if w_gate_up.shape != (2 * inter, K) or out.shape != (M, inter) or inter % 8:
        raise KernelError("linear_tcgen05_swiglu: shapes do not fit")
    _check(lib().vk_linear_tcgen05_swiglu(_p(x), _p(w_gate_up), _p(out), M, inter, K, x.stride(0), _p(error_word()), _stream()),
           "linear_tcgen05_swiglu")
    return out


def linear_tcgen05_rope(x: torch.Tensor, wqkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor,
                        sin: torch.Tensor, slot_mapping: torch.Tensor, cache_layer: torch.Tensor, nh: int, nkv: int,
                        hd: int) -> torch.Tensor:
    """q, k, v projections with the rotation of q and k and the write of k and v into the pages in the product's
    epilogue (head sizes 64 and 128; the whole head is rotated)."""
    if not tcgen05_takes(x, wqkv):
        raise KernelError("linear_tcgen05_rope: operands must be bfloat16, 16-byte aligned, with K and the row stride multiples of 8")
    _req(wqkv, "wqkv", torch.bfloat16, 2); _req(q_out, "q_out", torch.bfloat16, 2); _req(positions, "positions", torch.int32, 1)
    _req(cos, "cos", torch.float32, 2); _req(sin, "sin", torch.float32, 2); _req(slot_mapping, "slot_mapping", torch.int32, 1)
    _req(cache_layer, "cache_layer", torch.bfloat16, 5)
    M, K = x.shape
    ps = cache_layer.shape[3]
    if (wqkv.shape != ((nh + 2 * nkv) * hd, K) or q_out.shape != (M, nh * hd) or cos.shape[1] != hd // 2 or sin.shape != cos.shape
            or tuple(cache_layer.shape[1:]) != (2, nkv, ps, hd) or positions.shape[0] < M or slot_mapping.shape[0] < M):
        raise KernelError("linear_tcgen05_rope: shapes do not fit the head counts")
    _check(lib().vk_linear_tcgen05_rope(_p(x), _p(wqkv), _p(q_out), M, K, x.stride(0), _p(positions), _p(cos), _p(sin),
                                        _p(slot_mapping), _p(cache_layer), nh, nkv, hd, ps, _p(error_word()), _stream()),
           "linear_tcgen05_rope")
    return q_out


EPI_SAME, EPI_F32, EPI_ACC, EPI_SWIGLU, EPI_ROPE = 0, 1, 2, 3, 4
SKINNY_MAX_ROWS = 64
FUSED_NORM_MAX_ROWS = 16     # a block of the few-rows kernel norms every row it stages: beyond this many a norm kernel runs once
NORM_IN_REGISTERS_MAX_K = 640    # the tensor-core few-rows kernel norms rows of up to this many columns without staging them


def _mma_rows_per_block(M: int, N: int, K: int) -> int:
    """Batch rows a block of the tensor-core few-rows kernel stages (its launcher's rule): all of them in groups
    of eight; at most 16 for weights of up to 16 MB; fewer when the weights make too few tiles to fill the machine."""
    tiles = ((N + 1) // 2 + 7) // 8
    mg = 1 if M <= 8 else 2 if M <= 16 else 4 if M <= 32 else 8
    if mg > 2 and N * K * 2 <= (16 << 20):
        mg = 2
    while mg > 1 and tiles * -(-M // (8 * mg)) < 120:
        mg //= 2
    return 8 * mg


def _mma_norm_smem(M: int, K: int, N: int) -> int:
    """Shared memory of the tensor-core few-rows kernel with the fused norm: a block's rows staged whole in float32."""
    rows = _mma_rows_per_block(M, N, K)
    return rows * (4 * K + 64) + 4 * K + 8 * (rows // 8) * 512


def fused_norm_takes(dtype: torch.dtype, M: int, K: int, N: int) -> bool:
    """Whether norm and product should be one launch.  Every block norms the rows it stages, so the rows of a
    block must be few (at most 16) and, in float32, small enough that two blocks share a multiprocessor."""
    if not skinny_takes(dtype, M, K, N):
        return False
    if dtype == torch.float32 or K % 32 != 0:
        return M <= FUSED_NORM_MAX_ROWS
    rows = _mma_rows_per_block(M, N, K)
    # Rows of up to 640 columns are normed in registers, and a block may norm 16 of them; longer rows are staged in
    # float32 first, and beyond eight of them a norm kernel that runs once is faster (measured at K = 960 and 16 / 64
    # decode rows: 1.48 against 1.53 and 2.73 against 2.91 ms a step; at K = 576 the fused form wins: 1.42 against 1.53).
    if rows > (FUSED_NORM_MAX_ROWS if K <= NORM_IN_REGISTERS_MAX_K else min(8, FUSED_NORM_MAX_ROWS)):
        return False
    return _mma_norm_smem(M, K, N) <= 112 * 1024


def skinny_takes(dtype: torch.dtype, M: int, K: int, N: int = 0) -> bool:
    """Whether the few-rows kernel should take this product (else the tile kernels do the work).  Every block
    stages all M rows for itself, so many rows times many blocks (a large N) is left to the tile kernels."""
    if dtype == torch.float32 and _float32_exact:
        return False
    if not (0 < M <= SKINNY_MAX_ROWS and K % (4 if dtype == torch.float32 else 8) == 0):
        return False
    return M <= 8 or N <= 8192 or dtype == torch.float32


def linear_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, *, norm_weight: Optional[torch.Tensor] = None,
                  eps: float = 0.0, rows: Optional[torch.Tensor] = None, rope: Optional[tuple] = None,
                  force_simt: bool = False) -> torch.Tensor:
    """out = epilogue(x' @ w.T) for at most 64 rows, where x' is x, or rmsnorm(x[rows]) * norm_weight when
    norm_weight is given (x float32 then).  epi: EPI_SAME / EPI_F32 / EPI_ACC as LINEAR_*; EPI_SWIGLU: out [M, N/2] =
    silu(first half) * second half; EPI_ROPE: out = rotated q [M, nh*hd], rotated k and v go into the cache;
    rope = (positions, cos, sin, slot_mapping, cache_layer, nh, nkv, hd)."""
    _req(w, "w", dims=2)
    N, K = w.shape
    if norm_weight is not None:
        _req(x, "x", torch.float32, 2); _req(norm_weight, "norm_weight", torch.float32, 1)
        if x.shape[1] != K or norm_weight.shape[0] != K:
            raise KernelError("linear_skinny: widths differ")
        M = x.shape[0]
        if rows is not None:
            _req(rows, "rows", torch.int32, 1)
            M = rows.shape[0]
        ldx = x.stride(0)
    else:
        if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1 or x.dtype != w.dtype:
            raise KernelError("linear_skinny: x must be a CUDA matrix of the weights' dtype with unit column stride")
        if x.shape[1] != K or rows is not None:
            raise KernelError("linear_skinny: widths differ, or rows given without a norm")
        M = x.shape[0]
        ldx = x.stride(0) if M > 1 else max(K, x.stride(0))
    want = {EPI_SAME: ((M, N), w.dtype), EPI_F32: ((M, N), torch.float32), EPI_ACC: ((M, N), torch.float32),
            EPI_SWIGLU: ((M, N // 2), w.dtype)}
    pos = cos = sin = slot = cache = None
    nh = nkv = hd = ps = 0
    if epi == EPI_ROPE:
        pos, cos, sin, slot, cache, nh, nkv, hd = rope
        _req(pos, "positions", torch.int32, 1); _req(cos, "cos", torch.float32, 2); _req(sin, "sin", torch.float32, 2)
        _req(slot, "slot_mapping", torch.int32, 1); _req(cache, "cache_layer", w.dtype, 5)
        ps = cache.shape[3]
        if (cos.shape[1] != hd // 2 or tuple(cache.shape[1:]) != (2, nkv, ps, hd) or pos.shape[0] < M or slot.shape[0] < M
                or N != (nh + 2 * nkv) * hd):
            raise KernelError("linear_skinny: the rotary epilogue's arrays do not fit the head counts")
        want[EPI_ROPE] = ((M, nh * hd), w.dtype)
    _req(out, "out", want[epi][1], 2)
    if tuple(out.shape) != want[epi][0]:
        raise KernelError(f"linear_skinny: out is {tuple(out.shape)}, expected {want[epi][0]}")
    if (w.dtype == torch.bfloat16 and K % 32 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and not force_simt
            and (ldx % 4 == 0 and norm_weight.data_ptr() % 16 == 0 and _mma_norm_smem(M, K, N) <= 220 * 1024
                 if norm_weight is not None else ldx % 8 == 0)):
        # bfloat16: the tensor-core kernel
        _check(lib().vk_linear_skinny_mma(_p(x), _p(rows), _p(norm_weight), ctypes.c_float(eps), _p(w), _p(out), M, N, K, ldx,
                                          epi, _p(pos), _p(cos), _p(sin), _p(slot), _p(cache), nh, nkv, hd, ps, _stream()),
               "linear_skinny_mma")
        return out
    _check(lib().vk_linear_skinny(_p(x), _p(rows), _p(norm_weight), ctypes.c_float(eps), _p(w), _p(out), M, N, K, ldx, epi,
                                  _p(pos), _p(cos), _p(sin), _p(slot), _p(cache), nh, nkv, hd, ps, _dt(w), _stream()),
           "linear_skinny")
    return out


# ---------------------------------------------------------------------------
# Dispatch: which kernel a part's call runs, by dtype and size.
# ---------------------------------------------------------------------------

def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int) -> torch.Tensor:
    """out (=, or += in mode LINEAR_ACC_F32) x @ w.T.  float32 runs on CUDA cores in float32 arithmetic
    (no reduced-precision matrix mode); bfloat16 runs the tensor-core kernel where it takes the sizes."""
    if skinny_takes(x.dtype, x.shape[0], x.shape[1], w.shape[0]) and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        return linear_skinny(x, w, out, mode)
    if tcgen05_takes(x, w) and out.data_ptr() % 16 == 0:
        return linear_tcgen05(x, w, out, mode)
    if x.dtype == torch.float32 and _float32_exact:
        return linear_simt(x, w, out, mode, few_rows=0)        # the tile kernel for every batch: one order of sums
    return linear_simt(x, w, out, mode)


PREFILL_HEAD_SIZES = (16, 32, 64, 96, 128)


def attention_prefill(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor,
                      out: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of prompt portions in bfloat16 on the tensor cores.  tiles int32 [n, 4]: first token,
    rows (1..64), position of the first token, segment."""
    _req(q, "q", torch.bfloat16, 2); _req(cache_layer, "cache_layer", torch.bfloat16, 5)
    _req(block_tables, "block_tables", torch.int32, 2); _req(tiles, "tiles", torch.int32, 2); _req(out, "out", torch.bfloat16, 2)
    page_size = cache_layer.shape[3]
    if q.shape[1] != nh * hd or out.shape != q.shape or tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd) or tiles.shape[1] != 4:
        raise KernelError("attention_prefill: shapes do not fit the head counts")
    if hd not in PREFILL_HEAD_SIZES:
        raise KernelError(f"attention_prefill: head size {hd} is not one of {PREFILL_HEAD_SIZES}")
    _check(lib().vk_attention_prefill(_p(q), _p(cache_layer), _p(block_tables), _p(tiles), _p(out), tiles.shape[0], nh, nkv, hd,
                                      page_size, block_tables.shape[1], ctypes.c_float(scale), window, _stream()),
           "attention_prefill")
    return out


def set_prefill_streams(mode: int) -> int:
    """Which tcgen05 prompt-attention kernel a launch takes: 0 the kernel with two threads a query row, 1 the kernel with
    two streams of key steps, 2 by the size of the launch (the default).  Returns the mode that was in force."""
    return int(lib().vk_set_prefill_streams(int(mode)))


def attention_prefill_tcgen05_takes(q: torch.Tensor, cache_layer: torch.Tensor, hd: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes these operands: bfloat16, head size 64, pages of 8, 16, 32
    or a multiple of 64 slots, q rows dense and 16-byte aligned."""
    ps = cache_layer.shape[3]
    return (q.dtype == torch.bfloat16 and hd == 64 and ps % 8 == 0 and (64 % ps == 0 or ps % 64 == 0) and q.dim() == 2
            and q.stride(1) == 1 and q.stride(0) == q.shape[1] and q.data_ptr() % 16 == 0 and cache_layer.data_ptr() % 16 == 0
            and cache_layer.is_contiguous())


def attention_prefill_tcgen05_scratch_bytes(cap_tiles: int, nh: int, max_context: int) -> int:
    fn = lib().vk_attention_prefill_tcgen05_scratch_bytes
    fn.restype = ctypes.c_size_t
    return int(fn(cap_tiles, nh, max_context))


def attention_prefill_tcgen05(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor,
                              out: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: int = 0, *,
                              scratch: Optional[torch.Tensor] = None, cap_tiles: int = 0, max_context: int = 0,
                              grid_context: int = 0) -> torch.Tensor:
    """Causal attention of prompt portions on the tcgen05 tensor cores (scores and P V in tensor memory, keys and
    values by TMA straight from the pages).  tiles int32 [n, 4]: first token, rows (1..128), position of the first
    token, segment.  A tile whose walk over the keys is long is cut into parts that different blocks take; their
    partial results meet in `scratch`: a byte buffer of attention_prefill_tcgen05_scratch_bytes(cap_tiles, nh,
    max_context) that was zero at first use and is used with no other (cap_tiles, nh, max_context); grid_context
    (<= max_context) bounds the positions of this launch.  Without a scratch one is made for this call."""
    _req(q, "q", torch.bfloat16, 2); _req(cache_layer, "cache_layer", torch.bfloat16, 5)
    _req(block_tables, "block_tables", torch.int32, 2); _req(tiles, "tiles", torch.int32, 2); _req(out, "out", torch.bfloat16, 2)
    page_size = cache_layer.shape[3]
    if (q.shape[1] != nh * hd or out.shape != q.shape or tuple(cache_layer.shape[1:]) != (2, nkv, page_size, hd) or tiles.shape[1] != 4
            or out.stride(0) != out.shape[1]):
        raise KernelError("attention_prefill_tcgen05: shapes do not fit the head counts")
    if not attention_prefill_tcgen05_takes(q, cache_layer, hd):
        raise KernelError("attention_prefill_tcgen05: bfloat16, head size 64 and pages of 8, 16, 32 or a multiple of 64 slots only")
    if scratch is None:
        cap_tiles = tiles.shape[0]
        max_context = grid_context = max_context or block_tables.shape[1] * page_size
        scratch = torch.zeros(attention_prefill_tcgen05_scratch_bytes(cap_tiles, nh, max_context), dtype=torch.uint8, device=q.device)
    _req(scratch, "scratch", torch.uint8, 1)
    if scratch.numel() < attention_prefill_tcgen05_scratch_bytes(cap_tiles, nh, max_context):
        raise KernelError("attention_prefill_tcgen05: the scratch is too small")
    _check(lib().vk_attention_prefill_tcgen05(_p(q), _p(cache_layer), _p(block_tables), _p(tiles), _p(out), q.shape[0], tiles.shape[0],
                                              cache_layer.shape[0], nh, nkv, hd, page_size, block_tables.shape[1],
                                              ctypes.c_float(scale), window, _p(scratch), cap_tiles, max_context,
                                              grid_context or max_context, _p(error_word()), _stream()),
           "attention_prefill_tcgen05")
    return out


def attention(q: torch.Tensor, pages: torch.Tensor, meta, ctx, out: torch.Tensor, nh: int, nkv: int, hd: int,
              scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of a mixed batch over the paged cache; `meta` is the page group's GroupMeta.
    Single decoded tokens take the split-key kernel; tokens of prompt portions take the tensor-core kernel
    (bfloat16, head sizes it is built for); whatever is left takes attention_rows, which takes every size."""
    dec_ok = (bool(ctx.num_dec) and attention_decode_takes(q.dtype, hd, ctx.workspace.max_context)
              and not (q.dtype == torch.float32 and _float32_exact))
    pre_ok = (bool(ctx.num_pre) and q.dtype == torch.bfloat16 and hd in PREFILL_HEAD_SIZES and ctx.pre_tiles is not None
              and q.data_ptr() % 16 == 0)
    if dec_ok:
        ws = ctx.workspace
        cap, layout = ws.max_segments, ws.max_context
        nbytes = attention_decode_scratch_bytes(cap, nh, nkv, hd, layout)
        scratch = ws.flat(f"att.dec/{nh}/{nkv}/{hd}/{layout}", nbytes, torch.uint8, zero=True)
        attention_decode(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, scratch, cap, nh, nkv, hd, scale,
                         layout, min(layout, max(1, ctx.max_context)), window, ctx.dec_tokens)
    if pre_ok:
        if ctx.pre_tiles_big is not None and attention_prefill_tcgen05_takes(q, pages, hd) and out.stride(0) == out.shape[1]:
            ws = ctx.workspace
            cap_tiles, layout = ws.max_tokens // 128 + ws.max_segments, ws.max_context
            nbytes = attention_prefill_tcgen05_scratch_bytes(cap_tiles, nh, layout)
            scratch = ws.flat(f"att.pre/{nh}/{cap_tiles}/{layout}", nbytes, torch.uint8, zero=True)
            attention_prefill_tcgen05(q, pages, meta.block_tables, ctx.pre_tiles_big, out, nh, nkv, hd, scale, window,
                                      scratch=scratch, cap_tiles=cap_tiles, max_context=layout,
                                      grid_context=min(layout, max(1, ctx.max_context)))
        else:
            attention_prefill(q, pages, meta.block_tables, ctx.pre_tiles, out, nh, nkv, hd, scale, window)
    if not dec_ok and not pre_ok:
        return attention_rows(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, nh, nkv, hd, scale, window)
    if ctx.num_pre and not pre_ok:
        attention_rows(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, nh, nkv, hd, scale, window, ctx.pre_tokens)
    if ctx.num_dec and not dec_ok:
        attention_rows(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, nh, nkv, hd, scale, window, ctx.dec_tokens)
    return out


# ---------------------------------------------------------------------------
# Residual streams, scaled embedding with learned positions, activations
# ---------------------------------------------------------------------------

ACTIVATIONS = {"gelu": 0, "gelu_tanh": 1, "silu": 2}


def activation(x: torch.Tensor, kind: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(x) element by element (in place unless out is given); kind: gelu (the erf form), gelu_tanh, silu."""
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation: {kind!r} is not one of {sorted(ACTIVATIONS)}")
    out = x if out is None else out
    _req(x, "x"); _req(out, "out", x.dtype)
    if out.numel() != x.numel():
        raise KernelError("activation: sizes differ")
    _check(lib().vk_activation(_p(x), _p(out), ctypes.c_size_t(x.numel()), ACTIVATIONS[kind], _dt(x), _stream()), "activation")
    return out


def embed_scaled(table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, pos_table: Optional[torch.Tensor], scale: float,
                 out: torch.Tensor, copies: int = 1) -> torch.Tensor:
    """out[t, j, :] = scale * table[ids[t]] + pos_table[positions[t]] for every copy j; out float32 [T, copies * width]."""
    _req(table, "table", dims=2); _req(ids, "ids", torch.int32, 1); _req(positions, "positions", torch.int32, 1)
    _req(out, "out", torch.float32, 2)
    V, W = table.shape
    if pos_table is not None:
        _req(pos_table, "pos_table", torch.float32, 2)
        if pos_table.shape[1] != W:
            raise KernelError("embed_scaled: the position table's width differs")
    if out.shape != (ids.shape[0], copies * W) or positions.shape[0] < ids.shape[0]:
        raise KernelError("embed_scaled: out is not [tokens, copies * width]")
    _check(lib().vk_embed_scaled(_p(table), _p(ids), _p(positions), _p(pos_table), ctypes.c_float(scale), _p(out), ids.shape[0], W, V,
                                 0 if pos_table is None else pos_table.shape[0], copies, _dt(table), _stream()), "embed_scaled")
    return out


def hyper_step(xs: torch.Tensor, y: Optional[torch.Tensor], streams: int, *, mix: Optional[torch.Tensor] = None,
               out_w: Optional[torch.Tensor] = None, in_w: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
               eps: float = 0.0, xn: Optional[torch.Tensor] = None, sum_out: Optional[torch.Tensor] = None) -> None:
    """What lies between two sublayers of a model with `streams` residual rows a token (xs float32 [T, streams * W]):
    with mix [streams, streams] (from, to) and out_w [streams] the rows become  x_j <- sum_i mix[i, j] x_i + out_w[j] y;
    then  u = sum_i in_w[i] x_i  (all ones without in_w), written to sum_out (float32) and, normed with norm_w and eps,
    to xn (compute dtype).  y (float32 [T, W]) is left zeroed."""
    _req(xs, "xs", torch.float32, 2)
    T, W = xs.shape[0], xs.shape[1] // streams
    if xs.shape[1] != streams * W:
        raise KernelError("hyper_step: xs is not [tokens, streams * width]")
    for name, t, shape in (("y", y, (T, W)), ("mix", mix, (streams, streams)), ("out_w", out_w, (streams,)), ("in_w", in_w, (streams,)),
                           ("norm_w", norm_w, (W,)), ("sum_out", sum_out, (T, W))):
        if t is not None:
            _req(t, name, torch.float32)
            if tuple(t.shape) != shape:
                raise KernelError(f"hyper_step: {name} is {tuple(t.shape)}, expected {shape}")
    if xn is not None:
        _req(xn, "xn", dims=2)
        if tuple(xn.shape) != (T, W):
            raise KernelError("hyper_step: xn is not [tokens, width]")
    _check(lib().vk_hyper_step(_p(xs), _p(y), _p(mix), _p(out_w), _p(in_w), _p(norm_w), ctypes.c_float(eps), _p(xn), _p(sum_out), T, streams,
                               W, 0 if xn is None else _dt(xn), _stream()), "hyper_step")


# ---------------------------------------------------------------------------
# Attention without a rotation: unit-RMS q and k, a query factor that grows with the position, a bias by distance
# ---------------------------------------------------------------------------

def kv_page_elems(nkv: int, page_size: int, hd: int, vd: int, v_share: int = 1) -> int:
    """Elements of one page of one layer: [nkv][page_size][hd] keys, then [nkv / v_share][page_size][vd] values
    (v_share neighbouring key heads read one value head)."""
    return page_size * (nkv * hd + nkv // v_share * vd)


def _page_size_of(cache_layer: torch.Tensor, nkv: int, hd: int, vd: int, v_share: int = 1) -> int:
    per_page = cache_layer[0].numel()
    one = nkv * hd + nkv // v_share * vd
    ps = per_page // one
    if ps < 1 or ps * one != per_page or nkv % v_share or not cache_layer.is_contiguous():
        raise KernelError("the cache layer is not [pages][page_size * (nkv * hd + nkv / v_share * vd)]")
    return ps


def qk_norm_store(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor], q_out: torch.Tensor,
                  cache_layer: Optional[torch.Tensor], nh: int, nkv: int, hd: int, vd: int, page_size: int, *, eps: float = -1.0,
                  q_coef: float = 0.0, q_every: int = 1) -> torch.Tensor:
    """q and k heads divided by their root mean square (eps < 0: not), q times 1 + q_coef * ln(floor((pos + 1) / q_every) + 1);
    q to q_out, k and v into the layer's pages at slot_mapping (-1: no write)."""
    _req(qkv, "qkv", dims=2); _req(positions, "positions", torch.int32, 1); _req(q_out, "q_out", qkv.dtype, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + nkv) * hd + nkv * vd or q_out.shape != (T, nh * hd) or positions.shape[0] < T:
        raise KernelError("qk_norm_store: shapes do not fit the head counts")
    if cache_layer is not None:
        _req(cache_layer, "cache_layer", qkv.dtype); _req(slot_mapping, "slot_mapping", torch.int32, 1)
        if _page_size_of(cache_layer, nkv, hd, vd) != page_size or slot_mapping.shape[0] < T:
            raise KernelError("qk_norm_store: the cache layer does not fit the page size")
    _check(lib().vk_qk_norm_store(_p(qkv), _p(positions), _p(slot_mapping if cache_layer is not None else None), _p(q_out), _p(cache_layer),
                                  T, nh, nkv, hd, vd, page_size, ctypes.c_float(eps), ctypes.c_float(q_coef), int(q_every), _dt(qkv),
                                  _stream()), "qk_norm_store")
    return q_out


def attention_rows_biased(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, token_seg: torch.Tensor,
                          positions: torch.Tensor, out: torch.Tensor, nh: int, nkv: int, hd: int, vd: int, page_size: int, scale: float,
                          window: int = 0, dist_bias: Optional[torch.Tensor] = None, tok_list: Optional[torch.Tensor] = None,
                          v_in_key: bool = False, v_share: int = 1) -> torch.Tensor:
    """Causal attention of every token (or of those in tok_list) over its request's pages, any sizes, float32 arithmetic,
    with values of size vd and, if given, dist_bias [distances, nh] (float32) added to the scaled scores by min(distance, last row).
    v_in_key: the cache holds keys alone and a key's first vd values are its value.  v_share > 1: that many neighbouring
    key heads read one value head (two score maps over the same values)."""
    _req(q, "q", dims=2); _req(cache_layer, "cache_layer", q.dtype); _req(block_tables, "block_tables", torch.int32, 2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(positions, "positions", torch.int32, 1); _req(out, "out", q.dtype, 2)
    T = q.shape[0]
    if q.shape[1] != nh * hd or out.shape != (T, nh * vd) or _page_size_of(cache_layer, nkv, hd, 0 if v_in_key else vd, v_share) != page_size:
        raise KernelError("attention_rows_biased: shapes do not fit the head counts")
    if token_seg.shape[0] != T or positions.shape[0] != T:
        raise KernelError("attention_rows_biased: per-token arrays differ in length")
    if dist_bias is not None:
        _req(dist_bias, "dist_bias", torch.float32, 2)
        if dist_bias.shape[1] != nh:
            raise KernelError("attention_rows_biased: the bias table is not [distances, heads]")
    n = T
    if tok_list is not None:
        _req(tok_list, "tok_list", torch.int32, 1)
        n = tok_list.shape[0]
    _check(lib().vk_attention_rows_biased(_p(q), _p(cache_layer), _p(block_tables), _p(token_seg), _p(positions), _p(tok_list), _p(out), n, nh,
                                          nkv, hd, vd, page_size, block_tables.shape[1], ctypes.c_float(scale), window, _p(dist_bias),
                                          0 if dist_bias is None else dist_bias.shape[0], int(v_in_key), int(v_share), _dt(q), _stream()),
           "attention_rows_biased")
    return out


# ---------------------------------------------------------------------------
# The gated delta rule
# ---------------------------------------------------------------------------

def delta_state_floats(G: int, H: int, dk: int, dv: int, taps: int) -> int:
    """Floats of one request's state in one layer: the transposed matrix state of every head, then the last taps-1
    inputs of the short convolution, rounded up to a multiple of four."""
    return (H * dv * dk + max(0, taps - 1) * (2 * G * dk + H * dv) + 3) // 4 * 4


def delta_prep_width(G: int, H: int, dk: int, dv: int) -> int:
    """Floats of a row of the delta rule's scratch between its kernels: q | k | v | log decay | beta, padded to a multiple of four."""
    return (2 * G * dk + H * dv + 2 * H + 3) // 4 * 4


def delta_decode_takes(G: int, H: int, dk: int, dv: int, taps: int) -> bool:
    """Whether the one-kernel delta rule for single decoded tokens takes these sizes (key size a multiple of 4)."""
    return bool(lib().vk_delta_decode_takes(G, H, dk, dv, taps))


def delta_chunked_takes(G: int, H: int, dk: int, dv: int, taps: int) -> bool:
    """Whether the chunked form of the delta rule takes these sizes (key size a multiple of 4 up to 128, value size a multiple of 4
    up to 256)."""
    return bool(lib().vk_delta_chunked_takes(G, H, dk, dv, taps))


def delta_chunked_scratch_floats(tokens: int, segments: int, H: int, dk: int, dv: int) -> int:
    fn = lib().vk_delta_chunked_scratch_bytes
    fn.restype = ctypes.c_size_t
    return int(fn(tokens, segments, H, dk, dv)) // 4


def delta_rule(proj: torch.Tensor, conv_w: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, norm_w: torch.Tensor, eps: float,
               token_seg: torch.Tensor, seg_starts: torch.Tensor, seg_slots: torch.Tensor, state: torch.Tensor, prep: torch.Tensor,
               o: torch.Tensor, out: torch.Tensor, G: int, H: int, dk: int, dv: int, taps: int,
               chunk_scratch: Optional[torch.Tensor] = None, single_tokens: bool = False) -> torch.Tensor:
    """The gated delta rule on a batch of segments, from the projections to the input of the output projection.
    proj float32 [T, 2 G dk + 2 H dv + 2 H] = q | k | v | gate | b | a;  conv_w float32 [2 G dk + H dv, taps];  a_log, dt_bias [H];
    norm_w [dv];  state float32 [slots, delta_state_floats];  prep [T, delta_prep_width] and o [T, H dv] float32 scratch;
    out [T, H dv] in the compute dtype.  Three launches: prepare, recurrence (which also writes the state), gate.  With
    chunk_scratch (float32, delta_chunked_scratch_floats(T, segments, ...)) the recurrence runs in its chunked form, two launches:
    what does not need the state for all chunks side by side, then the chunks of every request in order.  With single_tokens
    (every segment is one token; sizes that delta_decode_takes) everything is ONE launch."""
    C = 2 * G * dk + H * dv
    _req(proj, "proj", torch.float32, 2); _req(conv_w, "conv_w", torch.float32, 2); _req(a_log, "a_log", torch.float32, 1)
    _req(dt_bias, "dt_bias", torch.float32, 1); _req(norm_w, "norm_w", torch.float32, 1); _req(state, "state", torch.float32, 2)
    _req(prep, "prep", torch.float32, 2); _req(o, "o", torch.float32, 2); _req(out, "out", dims=2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(seg_starts, "seg_starts", torch.int32, 1); _req(seg_slots, "seg_slots", torch.int32, 1)
    T, S = proj.shape[0], seg_slots.shape[0]
    if (proj.shape[1] != C + H * dv + 2 * H or conv_w.shape != (C, taps) or a_log.shape[0] != H or dt_bias.shape[0] != H
            or norm_w.shape[0] != dv or prep.shape != (T, delta_prep_width(G, H, dk, dv)) or o.shape != (T, H * dv) or out.shape != (T, H * dv)
            or state.shape[1] != delta_state_floats(G, H, dk, dv, taps) or token_seg.shape[0] != T or seg_starts.shape[0] != S + 1):
        raise KernelError("delta_rule: shapes do not fit the head counts")
    stride = ctypes.c_size_t(state.stride(0))
    if single_tokens and T == S and delta_decode_takes(G, H, dk, dv, taps):
        _check(lib().vk_delta_decode(_p(proj), _p(conv_w), _p(a_log), _p(dt_bias), _p(norm_w), ctypes.c_float(eps), _p(seg_starts), _p(seg_slots),
                                     _p(state), stride, _p(out), S, G, H, dk, dv, taps, _dt(out), _stream()), "delta_decode")
        return out
    _check(lib().vk_delta_prepare(_p(proj), _p(conv_w), _p(a_log), _p(dt_bias), _p(token_seg), _p(seg_starts), _p(seg_slots), _p(state), stride,
                                  _p(prep), T, G, H, dk, dv, taps, _stream()), "delta_prepare")
    if chunk_scratch is not None:
        _req(chunk_scratch, "chunk_scratch", torch.float32, 1)
        if chunk_scratch.numel() < delta_chunked_scratch_floats(T, S, H, dk, dv):
            raise KernelError("delta_rule: the scratch of the chunked form is too small")
        _check(lib().vk_delta_chunked(_p(prep), prep.shape[1], _p(proj), _p(seg_starts), _p(seg_slots), _p(state), stride, _p(o),
                                      _p(chunk_scratch), S, T, G, H, dk, dv, taps, _stream()), "delta_chunked")
        global _launches
        _launches += 1                              # two kernels
    else:
        _check(lib().vk_delta_recurrence(_p(prep), _p(proj), _p(seg_starts), _p(seg_slots), _p(state), stride, _p(o), S, T, G, H, dk, dv, taps,
                                         _stream()), "delta_recurrence")
    _check(lib().vk_delta_gate(_p(o), _p(proj), _p(norm_w), ctypes.c_float(eps), _p(out), T, G, H, dk, dv, _dt(out), _stream()), "delta_gate")
    return out


def attention_decode_biased(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, token_seg: torch.Tensor,
                            positions: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, scratch_tokens: int, nh: int, nkv: int, hd: int,
                            vd: int, page_size: int, scale: float, max_context: int, grid_context: int, window: int = 0,
                            dist_bias: Optional[torch.Tensor] = None, tok_list: Optional[torch.Tensor] = None,
                            v_in_key: bool = False, v_share: int = 1) -> torch.Tensor:
    """The split-key attention of single decoded tokens in the unrotated form: values of size vd, an optional bias by distance.
    scratch: attention_decode_scratch_bytes(scratch_tokens, nh, nkv, max(hd, vd), max_context) bytes, zero at first use."""
    _req(q, "q", dims=2); _req(cache_layer, "cache_layer", q.dtype); _req(block_tables, "block_tables", torch.int32, 2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(positions, "positions", torch.int32, 1); _req(out, "out", q.dtype, 2)
    _req(scratch, "scratch", torch.uint8, 1)
    T = q.shape[0]
    if q.shape[1] != nh * hd or out.shape != (T, nh * vd) or _page_size_of(cache_layer, nkv, hd, 0 if v_in_key else vd, v_share) != page_size:
        raise KernelError("attention_decode_biased: shapes do not fit the head counts")
    if dist_bias is not None:
        _req(dist_bias, "dist_bias", torch.float32, 2)
        if dist_bias.shape[1] != nh:
            raise KernelError("attention_decode_biased: the bias table is not [distances, heads]")
    n = T
    if tok_list is not None:
        _req(tok_list, "tok_list", torch.int32, 1)
        n = tok_list.shape[0]
    if scratch.numel() < attention_decode_scratch_bytes(scratch_tokens, nh, nkv, max(hd, vd), max_context):
        raise KernelError("attention_decode_biased: the scratch is too small")
    _check(lib().vk_attention_decode_biased(_p(q), _p(cache_layer), _p(block_tables), _p(token_seg), _p(positions), _p(tok_list), _p(out),
                                            _p(scratch), scratch_tokens, n, nh, nkv, hd, vd, page_size, block_tables.shape[1], max_context,
                                            grid_context, ctypes.c_float(scale), window, _p(dist_bias),
                                            0 if dist_bias is None else dist_bias.shape[0], int(v_in_key), int(v_share), _dt(q), _stream()),
           "attention_decode_biased")
    return out


BIASED_PREFILL_HEAD_SIZES = (32, 64, 96, 128)


def attention_prefill_biased(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor, out: torch.Tensor,
                             nh: int, nkv: int, hd: int, vd: int, page_size: int, scale: float, window: int = 0,
                             dist_bias: Optional[torch.Tensor] = None, v_in_key: bool = False, v_share: int = 1) -> torch.Tensor:
    """Causal attention of prompt portions in bfloat16 on the tensor cores, in the unrotated form.  tiles int32 [n, 4]: first
    token, rows (1..64), position of the first token, segment."""
    _req(q, "q", torch.bfloat16, 2); _req(cache_layer, "cache_layer", torch.bfloat16)
    _req(block_tables, "block_tables", torch.int32, 2); _req(tiles, "tiles", torch.int32, 2); _req(out, "out", torch.bfloat16, 2)
    if (q.shape[1] != nh * hd or out.shape != (q.shape[0], nh * vd) or _page_size_of(cache_layer, nkv, hd, 0 if v_in_key else vd, v_share) != page_size
            or tiles.shape[1] != 4):
        raise KernelError("attention_prefill_biased: shapes do not fit the head counts")
    if hd not in BIASED_PREFILL_HEAD_SIZES or vd not in BIASED_PREFILL_HEAD_SIZES:
        raise KernelError(f"attention_prefill_biased: head sizes {hd}, {vd} are not among {BIASED_PREFILL_HEAD_SIZES}")
    if dist_bias is not None:
        _req(dist_bias, "dist_bias", torch.float32, 2)
        if dist_bias.shape[1] != nh:
            raise KernelError("attention_prefill_biased: the bias table is not [distances, heads]")
    _check(lib().vk_attention_prefill_biased(_p(q), _p(cache_layer), _p(block_tables), _p(tiles), _p(out), tiles.shape[0], nh, nkv, hd, vd,
                                             page_size, block_tables.shape[1], ctypes.c_float(scale), window, _p(dist_bias),
                                             0 if dist_bias is None else dist_bias.shape[0], int(v_in_key), int(v_share), _stream()), "attention_prefill_biased")
    return out


def attention_biased(q: torch.Tensor, pages: torch.Tensor, meta, ctx, out: torch.Tensor, nh: int, nkv: int, hd: int, vd: int,
                     page_size: int, scale: float, window: int = 0, dist_bias: Optional[torch.Tensor] = None,
                     v_in_key: bool = False, v_share: int = 1) -> torch.Tensor:
    """Causal attention of a mixed batch over the paged cache in the unrotated form (values of their own size, or the
    first vd values of the keys with v_in_key; v_share neighbouring key heads reading one value head; a bias by distance); `meta` is the page group's GroupMeta.  Single decoded tokens take the split-key kernel, tokens of prompt
    portions the tensor-core kernel (bfloat16, head sizes it is built for); whatever is left, and the whole exact 32-bit
    routing, takes attention_rows_biased, which takes every size."""
    vec = 4 if q.dtype == torch.float32 else 8
    exact = q.dtype == torch.float32 and _float32_exact
    dec_ok = (bool(ctx.num_dec) and not exact and hd % vec == 0 and vd % vec == 0 and max(hd, vd) <= 256 and vd // vec <= 32
              and ctx.workspace.max_context <= 128 * 256)
    pre_ok = (bool(ctx.num_pre) and q.dtype == torch.bfloat16 and hd in BIASED_PREFILL_HEAD_SIZES and vd in BIASED_PREFILL_HEAD_SIZES
              and ctx.pre_tiles is not None and q.data_ptr() % 16 == 0 and pages.data_ptr() % 16 == 0)
    rows = lambda toks: attention_rows_biased(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, nh, nkv, hd, vd, page_size,
                                              scale, window, dist_bias, toks, v_in_key, v_share)
    if dec_ok:
        ws = ctx.workspace
        cap, layout = ws.max_segments, ws.max_context
        nbytes = attention_decode_scratch_bytes(cap, nh, nkv, max(hd, vd), layout)
        scratch = ws.flat(f"att.decb/{nh}/{nkv}/{hd}/{vd}/{layout}", nbytes, torch.uint8, zero=True)
        attention_decode_biased(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, scratch, cap, nh, nkv, hd, vd, page_size,
                                scale, layout, min(layout, max(1, ctx.max_context)), window, dist_bias, ctx.dec_tokens, v_in_key, v_share)
    if pre_ok:
        attention_prefill_biased(q, pages, meta.block_tables, ctx.pre_tiles, out, nh, nkv, hd, vd, page_size, scale, window, dist_bias, v_in_key, v_share)
    if not dec_ok and not pre_ok:
        return rows(None)
    if ctx.num_pre and not pre_ok:
        rows(ctx.pre_tokens)
    if ctx.num_dec and not dec_ok:
        rows(ctx.dec_tokens)
    return out


def linear_act(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """out = act(x @ w.T) in x's dtype; kind one of ACTIVATIONS.  In bfloat16 the activation is the epilogue of the few-rows
    tensor-core product (up to 64 rows) or of the tcgen05 product, on the float32 sums; elsewhere it is a launch of its own."""
    if kind not in ACTIVATIONS:
        raise KernelError(f"linear_act: {kind!r} is not one of {sorted(ACTIVATIONS)}")
    M, K = x.shape
    N = w.shape[0]
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K and tuple(out.shape) == (M, N) and out.dtype == x.dtype:
        _req(w, "w", torch.bfloat16, 2); _req(out, "out", torch.bfloat16, 2)
        act = ACTIVATIONS[kind] + 1
        if (skinny_takes(x.dtype, M, K, N) and K % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
                and w.data_ptr() % 16 == 0):
            ldx = x.stride(0) if M > 1 else max(K, x.stride(0))
            _check(lib().vk_linear_skinny_mma_act(_p(x), _p(None), _p(None), ctypes.c_float(0.0), _p(w), _p(out), M, N, K, ldx, act,
                                                  _stream()), "linear_skinny_mma_act")
            return out
        if M > SKINNY_MAX_ROWS and tcgen05_takes(x, w) and out.data_ptr() % 16 == 0:
            _check(lib().vk_linear_tcgen05_act(_p(x), _p(w), _p(out), M, N, K, x.stride(0), act, _p(error_word()), _stream()),
                   "linear_tcgen05_act")
            return out
    return activation(linear(x, w, out, LINEAR_SAME), kind)


# ---------------------------------------------------------------------------
# Layer norm, the logits' soft cap, gated feed-forwards with any activation
# ---------------------------------------------------------------------------

def layernorm_rows(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float, out: torch.Tensor,
                   rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r, :] = (x[rows[r], :] - mean) / sqrt(var + eps) * w + b; x float32 [T, n], out [R, n] float32 or bfloat16.
    A float32 out may be x itself (rows not given)."""
    _req(x, "x", torch.float32, 2); _req(w, "w", torch.float32, 1); _req(b, "b", torch.float32, 1); _req(out, "out", dims=2)
    n = x.shape[1]
    if w.shape[0] != n or b.shape[0] != n or out.shape[1] != n:
        raise KernelError("layernorm_rows: widths differ")
    if rows is not None:
        _req(rows, "rows", torch.int32, 1)
        if rows.shape[0] != out.shape[0]:
            raise KernelError("layernorm_rows: rows and out differ in length")
    elif out.shape[0] != x.shape[0]:
        raise KernelError("layernorm_rows: out and x differ in rows")
    _check(lib().vk_layernorm_rows(_p(x), _p(w), _p(b), _p(rows), _p(out), out.shape[0], n, ctypes.c_float(eps), _dt(out), _stream()),
           "layernorm_rows")
    return out


def softcap(z: torch.Tensor, cap: float) -> torch.Tensor:
    """z <- cap * tanh(z / cap), float32, in place."""
    _req(z, "z", torch.float32)
    _check(lib().vk_softcap(_p(z), ctypes.c_size_t(z.numel()), ctypes.c_float(cap), _stream()), "softcap")
    return z


def act_mul(gu: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """out = act(gu[:, :I]) * gu[:, I:]; gu [T, 2I], out [T, I], same dtype; kind one of ACTIVATIONS."""
    if kind not in ACTIVATIONS:
        raise KernelError(f"act_mul: {kind!r} is not one of {sorted(ACTIVATIONS)}")
    _req(gu, "gu", dims=2); _req(out, "out", gu.dtype, 2)
    if gu.shape[1] != 2 * out.shape[1] or gu.shape[0] != out.shape[0]:
        raise KernelError("act_mul: gu is not [tokens, 2 * intermediate]")
    _check(lib().vk_act_mul(_p(gu), _p(out), out.shape[0], out.shape[1], ACTIVATIONS[kind], _dt(gu), _stream()), "act_mul")
    return out


# ---------------------------------------------------------------------------
# Latent attention: what lies around its products and the attention itself
# ---------------------------------------------------------------------------

def latent_prepare(proj: torch.Tensor, q_rank: int, q_norm_w: torch.Tensor, cq: torch.Tensor, eps: float, positions: torch.Tensor,
                   freq: torch.Tensor, mag: float, dims: int, interleaved: bool, *, kv_off: int = -1, kv_rank: int = 0, rot_dim: int = 0,
                   kv_norm_w: Optional[torch.Tensor] = None, slot_mapping: Optional[torch.Tensor] = None,
                   cache_layer: Optional[torch.Tensor] = None, page_size: int = 0) -> torch.Tensor:
    """From the float32 rows of the first product: the normed query latent to cq (compute dtype) and, with kv_off >= 0 and a
    cache layer, the normed key-value latent and the rotated shared key part into the tokens' cache slots
    (a page: [page_size][kv_rank + rot_dim]; the row's first kv_rank values are read as the value too)."""
    _req(proj, "proj", torch.float32, 2); _req(q_norm_w, "q_norm_w", torch.float32, 1); _req(cq, "cq", dims=2)
    _req(positions, "positions", torch.int32, 1); _req(freq, "freq", torch.float32, 1)
    T, N = proj.shape
    if cq.shape != (T, q_rank) or q_norm_w.shape[0] != q_rank or positions.shape[0] < T or freq.shape[0] * 2 != dims:
        raise KernelError("latent_prepare: shapes do not fit")
    write = kv_off >= 0 and cache_layer is not None
    if write:
        _req(kv_norm_w, "kv_norm_w", torch.float32, 1); _req(slot_mapping, "slot_mapping", torch.int32, 1)
        _req(cache_layer, "cache_layer", cq.dtype)
        if (kv_norm_w.shape[0] != kv_rank or slot_mapping.shape[0] < T
                or _page_size_of(cache_layer, 1, kv_rank + rot_dim, 0) != page_size):
            raise KernelError("latent_prepare: the cache layer does not fit the latent's sizes")
    _check(lib().vk_latent_prepare(_p(proj), N, q_rank, _p(q_norm_w), _p(cq), kv_off if write else -1, kv_rank, rot_dim,
                                   _p(kv_norm_w if write else None), ctypes.c_float(eps), _p(positions), _p(freq), ctypes.c_float(mag), dims,
                                   int(bool(interleaved)), _p(slot_mapping if write else None), _p(cache_layer if write else None),
                                   page_size, T, _dt(cq), _stream()), "latent_prepare")
    return cq


def latent_rotate_q(q: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, mag: float, heads: int, lat: int, rot_dim: int, dims: int,
                    interleaved: bool) -> torch.Tensor:
    """Rotates the first `dims` of the last rot_dim values of every head of q [T, heads * (lat + rot_dim)], in place."""
    _req(q, "q", dims=2); _req(positions, "positions", torch.int32, 1); _req(freq, "freq", torch.float32, 1)
    if q.shape[1] != heads * (lat + rot_dim) or positions.shape[0] < q.shape[0] or freq.shape[0] * 2 != dims:
        raise KernelError("latent_rotate_q: shapes do not fit")
    _check(lib().vk_latent_rotate_q(_p(q), _p(positions), _p(freq), ctypes.c_float(mag), q.shape[0], heads, lat, rot_dim, dims,
                                    int(bool(interleaved)), _dt(q), _stream()), "latent_rotate_q")
    return q


def head_gate(x: torch.Tensor, gates: torch.Tensor, off: int, heads: int) -> torch.Tensor:
    """x [T, heads * d] in place: head h of token t times sigmoid(gates[t, off + h]); gates float32 [T, N]."""
    _req(x, "x", dims=2); _req(gates, "gates", torch.float32, 2)
    if x.shape[1] % heads or gates.shape[0] != x.shape[0] or off + heads > gates.shape[1]:
        raise KernelError("head_gate: shapes do not fit")
    _check(lib().vk_head_gate(_p(x), _p(gates), gates.shape[1], off, x.shape[0], heads, x.shape[1] // heads, _dt(x), _stream()), "head_gate")
    return x


# ---------------------------------------------------------------------------
# The gated delta rule with a decay per head and key channel
# ---------------------------------------------------------------------------

def channel_delta_prep_width(G: int, H: int, dk: int, dv: int) -> int:
    """Floats of a row of scratch between the kernels: q | k | v | log decay [H dk] | beta [H] | gate [H dv], padded to four."""
    return (2 * G * dk + 2 * H * dv + H * dk + H + 3) // 4 * 4


def channel_delta_group_floats(tokens: int, H: int, dk: int) -> int:
    """Floats of the scratch that holds, for every token and head, what its group of tokens needs besides the state."""
    return tokens * H * (4 * ((dk + 3) // 4 * 4) + 8)


def channel_delta_chunked_scratch_floats(tokens: int, segments: int, H: int, dk: int, dv: int) -> int:
    fn = lib().vk_cdelta_chunked_scratch_bytes
    fn.restype = ctypes.c_size_t
    return int(fn(tokens, segments, H, dk, dv)) // 4


def channel_delta_decode_takes(G: int, H: int, dk: int, dv: int, taps: int, ra: int, rg: int) -> bool:
    """Whether the one-kernel form for single decoded tokens takes these sizes (key size a multiple of 4 up to 512)."""
    return bool(lib().vk_cdelta_decode_takes(G, H, dk, dv, taps, ra, rg))


def channel_delta_rule(proj: torch.Tensor, conv_w: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, a2t: torch.Tensor,
                       g2t: torch.Tensor, norm_w: torch.Tensor, eps: float, token_seg: torch.Tensor, seg_starts: torch.Tensor,
                       seg_slots: torch.Tensor, state: torch.Tensor, prep: torch.Tensor, groups: torch.Tensor, o: torch.Tensor, out: torch.Tensor,
                       G: int, H: int, dk: int, dv: int, taps: int, single_tokens: bool = False,
                       chunk_scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The delta rule whose decay differs by head and key channel, from the projections to the input of the output projection.
    proj float32 [T, 2 G dk + H dv + H + ra + rg] = q | k | v | b | a1 | g1;  a2t float32 [ra, H dk] and g2t [rg, H dv], the wide
    halves of the two low-rank projections, transposed;  dt_bias [H dk];  a_log [H];  norm_w [dv];  state float32
    [slots, delta_state_floats];  prep [T, channel_delta_prep_width], groups (flat, channel_delta_group_floats(T, H, dk)) and o [T, H dv]
    float32 scratch;  out [T, H dv] in the compute dtype.  Four launches: prepare, what the groups of tokens need besides the state
    (all groups side by side), the recurrence (which also writes the state), gate.  With chunk_scratch (float32,
    channel_delta_chunked_scratch_floats(T, segments, ...); sizes that delta_chunked_takes) the recurrence runs in its chunked form
    instead: what does not need the state for all chunks side by side, then the chunks of every request in order.  With
    single_tokens (every segment is one token; sizes that channel_delta_decode_takes) everything is ONE launch."""
    C = 2 * G * dk + H * dv
    for name, t, d in (("proj", proj, 2), ("conv_w", conv_w, 2), ("a_log", a_log, 1), ("dt_bias", dt_bias, 1), ("a2t", a2t, 2), ("g2t", g2t, 2),
                       ("norm_w", norm_w, 1), ("state", state, 2), ("prep", prep, 2), ("o", o, 2), ("groups", groups, 1)):
        _req(t, name, torch.float32, d)
    _req(out, "out", dims=2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(seg_starts, "seg_starts", torch.int32, 1); _req(seg_slots, "seg_slots", torch.int32, 1)
    T, S = proj.shape[0], seg_slots.shape[0]
    ra, rg = a2t.shape[0], g2t.shape[0]
    if (proj.shape[1] != C + H + ra + rg or conv_w.shape != (C, taps) or a_log.shape[0] != H or dt_bias.shape[0] != H * dk
            or a2t.shape[1] != H * dk or g2t.shape[1] != H * dv or norm_w.shape[0] != dv
            or prep.shape != (T, channel_delta_prep_width(G, H, dk, dv)) or o.shape != (T, H * dv) or out.shape != (T, H * dv)
            or state.shape[1] != delta_state_floats(G, H, dk, dv, taps) or token_seg.shape[0] != T or seg_starts.shape[0] != S + 1
            or groups.numel() < channel_delta_group_floats(T, H, dk)):
        raise KernelError("channel_delta_rule: shapes do not fit the head counts")
    stride = ctypes.c_size_t(state.stride(0))
    if single_tokens and T == S and channel_delta_decode_takes(G, H, dk, dv, taps, ra, rg):
        _check(lib().vk_cdelta_decode(_p(proj), _p(conv_w), _p(a_log), _p(dt_bias), _p(a2t), _p(g2t), _p(norm_w), ctypes.c_float(eps),
                                      _p(seg_starts), _p(seg_slots), _p(state), stride, _p(out), S, G, H, dk, dv, taps, ra, rg, _dt(out),
                                      _stream()), "cdelta_decode")
        return out
    _check(lib().vk_cdelta_prepare(_p(proj), _p(conv_w), _p(a_log), _p(dt_bias), _p(a2t), _p(g2t), _p(token_seg), _p(seg_starts), _p(seg_slots),
                                   _p(state), stride, _p(prep), T, G, H, dk, dv, taps, ra, rg, _stream()), "cdelta_prepare")
    global _launches
    if chunk_scratch is not None:
        _req(chunk_scratch, "chunk_scratch", torch.float32, 1)
        if chunk_scratch.numel() < channel_delta_chunked_scratch_floats(T, S, H, dk, dv):
            raise KernelError("channel_delta_rule: the scratch of the chunked form is too small")
        _check(lib().vk_cdelta_chunked(_p(prep), prep.shape[1], _p(proj), proj.shape[1], _p(seg_starts), _p(seg_slots), _p(state), stride, _p(o),
                                       _p(chunk_scratch), S, T, G, H, dk, dv, taps, _stream()), "cdelta_chunked")
    else:
        _check(lib().vk_cdelta_recurrence(_p(prep), _p(proj), proj.shape[1], _p(token_seg), _p(seg_starts), _p(seg_slots), _p(state), stride,
                                          _p(groups), _p(o), S, T, G, H, dk, dv, taps, _stream()), "cdelta_recurrence")
    _launches += 1                                  # two kernels either way
    _check(lib().vk_cdelta_gate(_p(o), _p(prep), _p(norm_w), ctypes.c_float(eps), _p(out), T, G, H, dk, dv, _dt(out), _stream()), "cdelta_gate")
    return out


def linear_gated(x: torch.Tensor, w_gate_up: torch.Tensor, gu: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """out = act(x @ w_gate.T) * (x @ w_up.T) for the two matrices stacked by rows; kind one of ACTIVATIONS.  In bfloat16 the gate's
    function and the product with the other half are the epilogue of the few-rows tensor-core product (up to 64 rows) or of the
    tcgen05 product; elsewhere (float32, sizes those refuse) the product writes gu [T, 2I] (scratch in x's dtype) and a launch of its
    own follows."""
    if kind not in ACTIVATIONS:
        raise KernelError(f"linear_gated: {kind!r} is not one of {sorted(ACTIVATIONS)}")
    M, K = x.shape
    inter = w_gate_up.shape[0] // 2
    if (x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_gate_up.shape == (2 * inter, K) and tuple(out.shape) == (M, inter)
            and out.dtype == x.dtype and out.is_contiguous() and w_gate_up.is_contiguous()):
        act = ACTIVATIONS[kind] + 1
        if (skinny_takes(x.dtype, M, K, 2 * inter) and K % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
                and w_gate_up.data_ptr() % 16 == 0):
            ldx = x.stride(0) if M > 1 else max(K, x.stride(0))
            _check(lib().vk_linear_skinny_mma_gated(_p(x), _p(None), _p(None), ctypes.c_float(0.0), _p(w_gate_up), _p(out), M, 2 * inter, K, ldx,
                                                    act, _stream()), "linear_skinny_mma_gated")
            return out
        if M > SKINNY_MAX_ROWS and inter % 8 == 0 and tcgen05_takes(x, w_gate_up) and out.data_ptr() % 16 == 0:
            _check(lib().vk_linear_tcgen05_gated(_p(x), _p(w_gate_up), _p(out), M, inter, K, x.stride(0), act, _p(error_word()), _stream()),
                   "linear_tcgen05_gated")
            return out
    return act_mul(linear(x, w_gate_up, gu, LINEAR_SAME), out, kind)


# ---------------------------------------------------------------------------
# A decoder whose norm sits on a sublayer's output; an embedding with a second, hashed row; a clamped gated activation
# ---------------------------------------------------------------------------

def embed_hashed(table: torch.Tensor, second: Optional[torch.Tensor], ids: torch.Tensor, positions: torch.Tensor, token_seg: torch.Tensor,
                 seg_starts: torch.Tensor, seg_slots: torch.Tensor, last_token: Optional[torch.Tensor], x: torch.Tensor,
                 xc: Optional[torch.Tensor], buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0) -> torch.Tensor:
    """x[t] = table[id_t] + second[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets] (row `buckets` at position 0), float32; xc the same in
    the tables' dtype.  last_token int32 [slots]: the token before a step's first one, read and moved on by the kernel."""
    _req(table, "table", dims=2); _req(ids, "ids", torch.int32, 1); _req(x, "x", torch.float32, 2)
    T, W = x.shape
    if table.shape[1] != W or ids.shape[0] < T or positions.shape[0] < T or token_seg.shape[0] < T:
        raise KernelError("embed_hashed: shapes do not fit")
    if second is not None:
        _req(second, "second", table.dtype, 2); _req(last_token, "last_token", torch.int32)
        if second.shape != (buckets + 1, W) or buckets < 1:
            raise KernelError("embed_hashed: the second table is not [buckets + 1, width]")
    if xc is not None:
        _req(xc, "xc", table.dtype, 2)
        if xc.shape != (T, W):
            raise KernelError("embed_hashed: xc is not [tokens, width]")
    _check(lib().vk_embed_hashed(_p(table), _p(second), _p(ids), _p(positions), _p(token_seg), _p(seg_starts), _p(seg_slots), _p(last_token),
                                 _p(x), _p(xc), T, W, table.shape[0], buckets, mul_prev, mul_cur, _dt(table), _stream()), "embed_hashed")
    return x


def residual_norm_step(x: torch.Tensor, y: Optional[torch.Tensor], w: Optional[torch.Tensor], xc: Optional[torch.Tensor], eps: float = 0.0,
                       mult: float = 1.0) -> torch.Tensor:
    """x += mult * (y / sqrt(mean(y^2) + eps)) * w, y <- 0, xc <- x in xc's dtype; all float32 [T, W] but xc.  With w None nothing is
    added (y is only zeroed and xc written): the form that starts a pass."""
    _req(x, "x", torch.float32, 2)
    T, W = x.shape
    if y is not None:
        _req(y, "y", torch.float32, 2)
        if y.shape != (T, W):
            raise KernelError("residual_norm_step: y is not x's shape")
    if w is not None:
        _req(w, "w", torch.float32, 1)
        if w.shape[0] != W or y is None:
            raise KernelError("residual_norm_step: the weight does not fit the rows")
    if xc is not None:
        _req(xc, "xc", dims=2)
        if xc.shape != (T, W):
            raise KernelError("residual_norm_step: xc is not x's shape")
    _check(lib().vk_residual_norm_step(_p(x), _p(y), _p(w), _p(xc), T, W, ctypes.c_float(eps), ctypes.c_float(mult),
                                       0 if xc is None else _dt(xc), _stream()), "residual_norm_step")
    return x


def linear_glu_clamped(x: torch.Tensor, w_gate_up: torch.Tensor, gu: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """out = g sigmoid(alpha g) (u + 1) with g = min(x @ w_gate.T, limit), u = clamp(x @ w_up.T, -limit, limit) for the two matrices
    stacked by rows: the product writes gu [T, 2I] and glu_clamped follows.  (As one more case of the gated epilogue shared by the
    tcgen05 products it slowed that epilogue's silu case, which the Llama models' prompts run, by three quarters; it stays a launch.)"""
    return glu_clamped(linear(x, w_gate_up, gu, LINEAR_SAME), out, limit, alpha)


def glu_clamped(gu: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """out = g' sigmoid(alpha g') (u' + 1), g' = min(gu[:, :I], limit), u' = clamp(gu[:, I:], -limit, limit)."""
    _req(gu, "gu", dims=2); _req(out, "out", gu.dtype, 2)
    if gu.shape[1] != 2 * out.shape[1] or gu.shape[0] != out.shape[0]:
        raise KernelError("glu_clamped: gu is not [tokens, 2 * intermediate]")
    _check(lib().vk_glu_clamped(_p(gu), _p(out), out.shape[0], out.shape[1], ctypes.c_float(limit), ctypes.c_float(alpha), _dt(gu), _stream()),
           "glu_clamped")
    return out


# ---------------------------------------------------------------------------
# Differential attention: what lies around its products and the attention itself
# ---------------------------------------------------------------------------

def diff_attn_channels(H: int, G: int, dim: int, vdim: int, own_kv: bool) -> int:
    """Channels that pass the short convolution: q, and k and v where the layer has its own."""
    return H * 2 * dim + (G * 2 * dim + G * vdim if own_kv else 0)


def diff_attn_prepare(proj: torch.Tensor, bias: Optional[torch.Tensor], conv_w: Optional[torch.Tensor], taps: int, tail: Optional[torch.Tensor],
                      ctx, qn_w: torch.Tensor, kn_w: Optional[torch.Tensor], eps: float, freq: Optional[torch.Tensor], mag: float, dims: int,
                      H: int, G: int, dim: int, vdim: int, own_kv: bool, slot_mapping: Optional[torch.Tensor], cache_layer: Optional[torch.Tensor],
                      page_size: int, qout: torch.Tensor, out_bias: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None) -> torch.Tensor:
    """From the float32 rows of the first product [q | k | v | ...]: bias, short convolution (memory in `tail` [slots, taps-1, C]), norm per
    head and map, rotation; q to qout [T, 2H * dim] (order [key head][map][query head of the group]), k and v into the cache slots.
    `ctx` gives token_seg, seg_starts, seg_slots and positions.  out_bias (float32 [width]) is added into y's rows."""
    _req(proj, "proj", torch.float32, 2); _req(qn_w, "qn_w", torch.float32, 1); _req(qout, "qout", dims=2)
    T, N = proj.shape
    C = diff_attn_channels(H, G, dim, vdim, own_kv)
    if qout.shape != (T, 2 * H * dim) or qn_w.shape[0] != dim or N < C or (dims and (freq is None or freq.shape[0] * 2 != dims)):
        raise KernelError("diff_attn_prepare: shapes do not fit")
    if bias is not None:
        _req(bias, "bias", torch.float32, 1)
        if bias.shape[0] < C:
            raise KernelError("diff_attn_prepare: the bias is shorter than the channels")
    if conv_w is not None:
        _req(conv_w, "conv_w", torch.float32, 2)
        if conv_w.shape != (C, taps):
            raise KernelError("diff_attn_prepare: the convolution's weights are not [channels, taps]")
        if taps > 1:
            _req(tail, "tail", torch.float32)
            if tail[0].numel() != (taps - 1) * C:
                raise KernelError("diff_attn_prepare: the convolution's memory is not [slots, taps - 1, channels]")
    if own_kv:
        _req(kn_w, "kn_w", torch.float32, 1); _req(slot_mapping, "slot_mapping", torch.int32, 1); _req(cache_layer, "cache_layer", qout.dtype)
        if kn_w.shape[0] != dim or slot_mapping.shape[0] < T or _page_size_of(cache_layer, 2 * G, dim, vdim, 2) != page_size:
            raise KernelError("diff_attn_prepare: the cache layer does not fit the head counts")
    if out_bias is not None:
        _req(out_bias, "out_bias", torch.float32, 1); _req(y, "y", torch.float32, 2)
        if y.shape != (T, out_bias.shape[0]):
            raise KernelError("diff_attn_prepare: the output bias does not fit y")
    _check(lib().vk_diff_attn_prepare(_p(proj), N, _p(bias), _p(conv_w), taps, _p(tail if conv_w is not None and taps > 1 else None),
                                      _p(ctx.token_seg), _p(ctx.seg_starts), _p(ctx.seg_slots), _p(ctx.positions), _p(qn_w),
                                      _p(kn_w if own_kv else None), ctypes.c_float(eps), _p(freq), ctypes.c_float(mag), dims, H, G, dim, vdim,
                                      int(own_kv), _p(slot_mapping if own_kv else None), _p(cache_layer if own_kv else None), page_size, _p(qout),
                                      _p(out_bias), _p(y if out_bias is not None else None), 0 if out_bias is None else out_bias.shape[0], T,
                                      _dt(qout), _stream()), "diff_attn_prepare")
    return qout


def diff_attn_combine(att: torch.Tensor, proj: torch.Tensor, gate_off: int, lam: float, diff: float, eps: float, H: int, G: int, vdim: int,
                      out: torch.Tensor, bias: Optional[torch.Tensor], taps: int, channels: int, tail: Optional[torch.Tensor], ctx) -> torch.Tensor:
    """out [T, H * vdim] = rms-normed (a1 - lam * a2) * (1 - diff) * sigmoid(gate) per head, from att [T, 2H * vdim] in the order
    diff_attn_prepare wrote the queries; moves the convolution's memory on for every segment."""
    _req(att, "att", dims=2); _req(proj, "proj", torch.float32, 2); _req(out, "out", att.dtype, 2)
    T, N = proj.shape
    if att.shape != (T, 2 * H * vdim) or out.shape != (T, H * vdim) or gate_off + H * vdim > N:
        raise KernelError("diff_attn_combine: shapes do not fit")
    use_tail = tail is not None and taps > 1
    _check(lib().vk_diff_attn_combine(_p(att), _p(proj), N, gate_off, ctypes.c_float(lam), ctypes.c_float(diff), ctypes.c_float(eps), H, G, vdim,
                                      _p(out), _p(bias), taps, channels, _p(tail if use_tail else None), _p(ctx.token_seg), _p(ctx.seg_starts),
                                      _p(ctx.seg_slots), T, _dt(att), _stream()), "diff_attn_combine")
    return out


# ---------------------------------------------------------------------------
# The matrix memory with exponential gates
# ---------------------------------------------------------------------------

def mlstm_state_floats(H: int, dim: int, vdim: int) -> int:
    """A slot's state: S [H, dim, vdim], n [H, dim], m [H]."""
    return H * dim * vdim + H * dim + H


def mlstm_max_dim() -> int:
    return int(lib().vk_mlstm_max_dim())


def mlstm(proj: torch.Tensor, gate_bias: torch.Tensor, cap: float, norm_w: torch.Tensor, eps: float, ctx, state: torch.Tensor,
          o: torch.Tensor, out: torch.Tensor, H: int, dim: int, vdim: int) -> torch.Tensor:
    """proj float32 [T, N] = q | k | v | gate | a | b; the recurrence token after token per segment from and into `state`
    [slots, mlstm_state_floats]; o float32 [T, H * (vdim + 2)] receives each head's numerators, n . q and m;
    out [T, H * vdim] = o / rms(o) * norm_w * sigmoid(gate) in out's dtype."""
    _req(proj, "proj", torch.float32, 2); _req(gate_bias, "gate_bias", torch.float32, 1); _req(norm_w, "norm_w", torch.float32, 1)
    _req(state, "state", torch.float32); _req(o, "o", torch.float32, 2); _req(out, "out", dims=2)
    T, N = proj.shape
    if (N < 2 * H * dim + 2 * H * vdim + 2 * H or gate_bias.shape[0] != 2 * H or norm_w.shape[0] != H * vdim or o.shape != (T, H * (vdim + 2))
            or out.shape != (T, H * vdim) or state[0].numel() != mlstm_state_floats(H, dim, vdim)):
        raise KernelError("mlstm: shapes do not fit the head counts")
    _check(lib().vk_mlstm_recurrence(_p(proj), N, H, dim, vdim, _p(gate_bias), ctypes.c_float(cap), _p(ctx.seg_starts), _p(ctx.seg_slots),
                                     _p(state), _p(o), ctx.num_segments, _stream()), "mlstm_recurrence")
    _check(lib().vk_mlstm_gate(_p(o), _p(proj), N, 2 * H * dim + H * vdim, _p(norm_w), ctypes.c_float(eps), H, dim, vdim, _p(out), T,
                               _p(ctx.seg_starts), _p(ctx.seg_slots), _p(state), ctx.num_segments, _dt(out), _stream()), "mlstm_gate")
    return out


# ---------------------------------------------------------------------------
# A routed feed-forward
# ---------------------------------------------------------------------------

_EPILOGUE_ACT = {"gelu": 1, "gelu_tanh": 2, "silu": 3}


def experts_route(x: torch.Tensor, w_router: torch.Tensor, b_router: Optional[torch.Tensor], top: int, ids: torch.Tensor,
                  wts: torch.Tensor) -> None:
    """ids [T, top], wts [T, top]: the `top` largest of the float32 logits w_router x + b and the softmax over them alone."""
    _req(x, "x", dims=2); _req(w_router, "w_router", torch.float32, 2); _req(ids, "ids", torch.int32, 2); _req(wts, "wts", torch.float32, 2)
    T, W = x.shape
    if w_router.shape[1] != W or ids.shape != (T, top) or wts.shape != (T, top) or (b_router is not None and b_router.shape != (w_router.shape[0],)):
        raise KernelError("experts_route: shapes do not fit")
    if b_router is not None:
        _req(b_router, "b_router", torch.float32, 1)
    _check(lib().vk_experts_route(_p(x), W, _p(w_router), _p(b_router), w_router.shape[0], top, _p(ids), _p(wts), T, _dt(x), _stream()), "experts_route")


def experts_route_table(tokens: torch.Tensor, table: torch.Tensor, E: int, top: int, ids: torch.Tensor, wts: torch.Tensor) -> None:
    """ids [T, top] = table[token id, :top] (int32 [vocab, >= top]); every weight 1 / top."""
    _req(tokens, "tokens", torch.int32, 1); _req(table, "table", torch.int32, 2); _req(ids, "ids", torch.int32, 2); _req(wts, "wts", torch.float32, 2)
    T = tokens.shape[0]
    if table.shape[1] < top or ids.shape != (T, top) or wts.shape != (T, top):
        raise KernelError("experts_route_table: shapes do not fit")
    _check(lib().vk_experts_route_table(_p(tokens), _p(table), table.shape[0], table.shape[1], E, top, _p(ids), _p(wts), T, _stream()),
           "experts_route_table")


def _expert_act(activation: str, what: str) -> int:
    if activation == "clamped":
        return 4
    if activation not in _EPILOGUE_ACT:
        raise KernelError(f"{what}: {activation!r} is not one of {sorted(_EPILOGUE_ACT) + ['clamped']}")
    return _EPILOGUE_ACT[activation]


def experts_apply(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, act_buf: torch.Tensor,
                  y: torch.Tensor, activation: str = "silu", limit: float = 0.0, alpha: float = 1.702) -> torch.Tensor:
    """y [T, W] (float32) += sum_k wts[t, k] W_down,e (act(W_gate,e x) * W_up,e x), e = ids[t, k]; w_gate_up [E, 2 ff, W], w_down [E, W, ff]
    in x's dtype; act_buf [T * top, ff] in x's dtype.  activation "clamped": min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u) + 1)."""
    _req(x, "x", dims=2); _req(w_gate_up, "w_gate_up", x.dtype, 3); _req(w_down, "w_down", x.dtype, 3); _req(y, "y", torch.float32, 2)
    _req(act_buf, "act_buf", x.dtype, 2)
    T, W = x.shape
    E, two_ff, _ = w_gate_up.shape
    ff, top = two_ff // 2, ids.shape[1]
    if w_gate_up.shape != (E, 2 * ff, W) or w_down.shape != (E, W, ff) or y.shape != (T, W) or act_buf.shape != (T * top, ff):
        raise KernelError("experts_apply: shapes do not fit")
    act = _expert_act(activation, "experts_apply")
    _check(lib().vk_experts_gate_up(_p(x), W, _p(w_gate_up), ff, top, _p(ids), act, ctypes.c_float(limit), ctypes.c_float(alpha), _p(act_buf), T,
                                    _dt(x), _stream()), "experts_gate_up")
    _check(lib().vk_experts_down(_p(act_buf), ff, _p(w_down), W, top, _p(ids), _p(wts), _p(y), T, _dt(x), _stream()), "experts_down")
    return y


def experts_grouped_rows(tokens: int, top: int, E: int) -> int:
    """Rows of the grouped matrix for up to `tokens` tokens: every copy, and every expert's rows filled up to whole tiles."""
    rows = int(lib().vk_experts_grouped_rows(tokens, top, E))
    if rows < 0:
        raise KernelError("experts_grouped_rows: too many rows")
    return rows


def experts_grouped_takes(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    """Whether the tensor-core form takes these operands: bfloat16, 16-byte aligned, sizes that are multiples of 8."""
    ff, W = w_gate_up.shape[1] // 2, x.shape[1]
    return (x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16 and W % 8 == 0 and ff % 8 == 0
            and x.stride(0) == W and x.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0 and w_down.data_ptr() % 16 == 0)


def experts_apply_grouped(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, pos: torch.Tensor,
                          row_token: torch.Tensor, tile_group: torch.Tensor, xs: torch.Tensor, act_buf: torch.Tensor, o: torch.Tensor,
                          y: torch.Tensor, activation: str = "silu", limit: float = 0.0, alpha: float = 1.702,
                          gu_buf: Optional[torch.Tensor] = None) -> torch.Tensor:
    """experts_apply on the tensor cores: the tokens' copies are put expert by expert into xs [rows, W] (rows =
    experts_grouped_rows(T, top, E); pos [T, top], row_token [rows], tile_group [rows / 128] int32), two products of row groups give
    act_buf [rows, ff] (bfloat16) and o [rows, W] (float32), and y [T, W] (float32) += the weighted rows of each token.
    activation "clamped" (with gu_buf [rows, 2 ff] bfloat16): the first product leaves gate and up, and glu_clamped follows."""
    _req(x, "x", torch.bfloat16, 2); _req(y, "y", torch.float32, 2); _req(o, "o", torch.float32, 2); _req(xs, "xs", torch.bfloat16, 2)
    _req(act_buf, "act_buf", torch.bfloat16, 2); _req(pos, "pos", torch.int32, 2); _req(row_token, "row_token", torch.int32, 1)
    _req(tile_group, "tile_group", torch.int32, 1)
    T, W = x.shape
    E, two_ff, _ = w_gate_up.shape
    ff, top = two_ff // 2, ids.shape[1]
    rows = experts_grouped_rows(T, top, E)
    if (not experts_grouped_takes(x, w_gate_up, w_down) or w_gate_up.shape != (E, 2 * ff, W) or w_down.shape != (E, W, ff) or y.shape != (T, W)
            or xs.shape != (rows, W) or act_buf.shape != (rows, ff) or o.shape != (rows, W) or pos.shape != (T, top) or row_token.shape != (rows,)
            or tile_group.shape != (rows // 128,)):
        raise KernelError("experts_apply_grouped: shapes do not fit")
    act = _expert_act(activation, "experts_apply_grouped")
    act = 0 if activation == "silu" else act
    if act == 4:
        if gu_buf is None or gu_buf.shape != (rows, 2 * ff):
            raise KernelError("experts_apply_grouped: the clamped form needs gu_buf [rows, 2 ff]")
        _req(gu_buf, "gu_buf", torch.bfloat16, 2)
    _check(lib().vk_experts_sort(_p(ids), T, top, E, rows, _p(pos), _p(row_token), _p(tile_group), _stream()), "experts_sort")
    _check(lib().vk_experts_gather(_p(x), W, _p(row_token), _p(xs), rows, _dt(x), _stream()), "experts_gather")
    if act == 4:
        _check(lib().vk_linear_tcgen05_grouped(_p(xs), _p(w_gate_up), _p(gu_buf), rows, 2 * ff, W, W, E, _p(tile_group), 0, 0, 0, _p(error_word()),
                                               _stream()), "linear_tcgen05_grouped")
        glu_clamped(gu_buf, act_buf, limit, alpha)
    else:
        _check(lib().vk_linear_tcgen05_grouped(_p(xs), _p(w_gate_up), _p(act_buf), rows, ff, W, W, E, _p(tile_group), 0, 1, act, _p(error_word()),
                                               _stream()), "linear_tcgen05_grouped")
    _check(lib().vk_linear_tcgen05_grouped(_p(act_buf), _p(w_down), _p(o), rows, W, ff, ff, E, _p(tile_group), 1, 0, 0, _p(error_word()),
                                           _stream()), "linear_tcgen05_grouped")
    _check(lib().vk_experts_combine(_p(o), W, top, _p(pos), _p(wts), _p(y), T, _stream()), "experts_combine")
    return y


# ---------------------------------------------------------------------------
# A norm before and behind each sublayer; an activation with two numbers of its own
# ---------------------------------------------------------------------------

def sandwich_step(x: torch.Tensor, y: Optional[torch.Tensor], post: Optional[tuple], nxt: Optional[tuple], xn: Optional[torch.Tensor],
                  eps: float) -> Optional[torch.Tensor]:
    """x += LN(y; post = (w, b)) and y = 0 (post None: y is only zeroed), then xn = LN(x; nxt = (w, b)) in xn's dtype (nxt None: none).
    x, y float32 [T, n]; the weights float32 [n]."""
    _req(x, "x", torch.float32, 2)
    T, n = x.shape
    if y is not None:
        _req(y, "y", torch.float32, 2)
        if y.shape != x.shape:
            raise KernelError("sandwich_step: x and y differ in shape")
    for pair in (post, nxt):
        if pair is not None:
            for v in pair:
                _req(v, "a norm's weight", torch.float32, 1)
                if v.shape[0] != n:
                    raise KernelError("sandwich_step: a norm's weight does not fit the width")
    if nxt is not None:
        _req(xn, "xn", dims=2)
        if xn.shape != x.shape:
            raise KernelError("sandwich_step: xn does not fit x")
    wp, bp = post if post is not None else (None, None)
    wn, bn = nxt if nxt is not None else (None, None)
    _check(lib().vk_sandwich_step(_p(x), _p(y), _p(wp), _p(bp), _p(wn), _p(bn), _p(xn if nxt is not None else None), T, n, ctypes.c_float(eps),
                                  _dt(xn) if nxt is not None else 0, _stream()), "sandwich_step")
    return xn if nxt is not None else None


def linear_xielu(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, a_pos: float, a_neg: float) -> torch.Tensor:
    """out = xielu(x @ w.T) in x's dtype: the product, then the activation in place."""
    return xielu(linear(x, w, out, LINEAR_SAME), a_pos, a_neg)


def xielu(x: torch.Tensor, a_pos: float, a_neg: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = a_pos x^2 + x / 2 where x > 0, a_neg (exp(x) - 1 - x) + x / 2 elsewhere (in place unless out is given)."""
    out = x if out is None else out
    _req(x, "x"); _req(out, "out", x.dtype)
    if out.numel() != x.numel():
        raise KernelError("xielu: sizes differ")
    _check(lib().vk_xielu(_p(x), _p(out), ctypes.c_size_t(x.numel()), ctypes.c_float(a_pos), ctypes.c_float(a_neg), _dt(x), _stream()), "xielu")
    return out


# ---------------------------------------------------------------------------
# Gated linear attention
# ---------------------------------------------------------------------------

def gla_state_floats(H: int, dim: int, vdim: int) -> int:
    return H * dim * vdim


def gla_max_dim() -> int:
    return int(lib().vk_gla_max_dim())


def gla(proj: torch.Tensor, a_off: int, a2t: torch.Tensor, bias: torch.Tensor, tau: float, norm_w: torch.Tensor, eps: float, ctx,
        state: torch.Tensor, decay: torch.Tensor, o: torch.Tensor, out: torch.Tensor, H: int, dim: int, vdim: int, gate_off: int) -> torch.Tensor:
    """proj float32 [T, N] = q | k | v | ... with the gate's H vdim columns at gate_off and the decays' narrow half (rank = a2t.shape[0]
    columns) at a_off; a2t float32 [rank, H dim], bias [H dim]; the recurrence S <- diag(a) S + k v^T, o = S^T q dim^-1/2 token after token
    per segment from and into state [slots, H dim vdim]; decay float32 [T, H dim] and o float32 [T, H vdim] are scratch; out [T, H vdim] =
    o / rms(o) per head * norm_w [vdim] * silu(gate) in out's dtype.  A batch of single tokens takes one launch for decays and step."""
    _req(proj, "proj", torch.float32, 2); _req(a2t, "a2t", torch.float32, 2); _req(bias, "bias", torch.float32, 1); _req(norm_w, "norm_w", torch.float32, 1)
    _req(state, "state", torch.float32); _req(decay, "decay", torch.float32, 2); _req(o, "o", torch.float32, 2); _req(out, "out", dims=2)
    T, N = proj.shape
    rank, C = a2t.shape
    if (C != H * dim or bias.shape[0] != C or norm_w.shape[0] != vdim or N < max(2 * H * dim + H * vdim, a_off + rank, gate_off + H * vdim)
            or decay.shape != (T, C) or o.shape != (T, H * vdim) or out.shape != (T, H * vdim) or state[0].numel() != gla_state_floats(H, dim, vdim)):
        raise KernelError("gla: shapes do not fit the head counts")
    L = lib()
    if ctx.decode_only and not (proj.dtype == torch.float32 and out.dtype == torch.float32 and _float32_exact):
        _check(L.vk_gla_decode(_p(proj), N, H, dim, vdim, a_off, rank, _p(a2t), _p(bias), ctypes.c_float(tau), _p(ctx.seg_starts), _p(ctx.seg_slots),
                               _p(state), _p(o), ctx.num_segments, _stream()), "gla_decode")
    else:
        _check(L.vk_gla_prepare(_p(proj), N, a_off, rank, _p(a2t), _p(bias), ctypes.c_float(tau), C, _p(decay), T, _stream()), "gla_prepare")
        _check(L.vk_gla_recurrence(_p(proj), N, H, dim, vdim, _p(decay), _p(ctx.seg_starts), _p(ctx.seg_slots), _p(state), _p(o), ctx.num_segments,
                                   _stream()), "gla_recurrence")
    _check(L.vk_gla_gate(_p(o), _p(proj), N, gate_off, _p(norm_w), ctypes.c_float(eps), H, vdim, _p(out), T, _dt(out), _stream()), "gla_gate")
    return out


# ---------------------------------------------------------------------------
# Attention with capped, mixed scores and rotated values
# ---------------------------------------------------------------------------

def mixed_attn_prepare(proj: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor], q_norm: Optional[torch.Tensor],
                       k_norm: Optional[torch.Tensor], eps: float, freq: Optional[torch.Tensor], dims: int, vfreq: Optional[torch.Tensor],
                       q_out: torch.Tensor, cache_layer: Optional[torch.Tensor], nh: int, nkv: int, hd: int, vd: int, page_size: int) -> torch.Tensor:
    """From the float32 row [q | k | v] of the first product: q and k heads / rms * weight (eps < 0: no norm), the first `dims` values turned
    in pairs (i, i + dims / 2) by position * freq[i]; v turned over all its pairs by position * vfreq[m] (None: not); q to q_out, k and v
    into the layer's pages at slot_mapping (-1: no write)."""
    _req(proj, "proj", torch.float32, 2); _req(positions, "positions", torch.int32, 1); _req(q_out, "q_out", dims=2)
    T, N = proj.shape
    if N < (nh + nkv) * hd + nkv * vd or q_out.shape != (T, nh * hd) or positions.shape[0] < T:
        raise KernelError("mixed_attn_prepare: shapes do not fit the head counts")
    for v, n, name in ((q_norm, hd, "q_norm"), (k_norm, hd, "k_norm"), (freq, dims // 2, "freq"), (vfreq, vd // 2, "vfreq")):
        if v is not None:
            _req(v, name, torch.float32, 1)
            if v.shape[0] != n:
                raise KernelError(f"mixed_attn_prepare: {name} has {v.shape[0]} values, expected {n}")
    if dims and freq is None:
        raise KernelError("mixed_attn_prepare: a rotation needs its frequencies")
    if cache_layer is not None:
        _req(cache_layer, "cache_layer", q_out.dtype); _req(slot_mapping, "slot_mapping", torch.int32, 1)
        if _page_size_of(cache_layer, nkv, hd, vd) != page_size or slot_mapping.shape[0] < T:
            raise KernelError("mixed_attn_prepare: the cache layer does not fit the page size")
    _check(lib().vk_mixed_attn_prepare(_p(proj), N, _p(positions), _p(slot_mapping if cache_layer is not None else None), _p(q_norm), _p(k_norm),
                                       ctypes.c_float(eps), _p(freq if dims else None), dims, _p(vfreq), _p(q_out), _p(cache_layer), T, nh, nkv, hd, vd,
                                       page_size, _dt(q_out), _stream()), "mixed_attn_prepare")
    return q_out


def attention_mixed_rows(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, token_seg: torch.Tensor, positions: torch.Tensor,
                         out: torch.Tensor, nh: int, nkv: int, hd: int, vd: int, page_size: int, scale: float, cap: float = 0.0,
                         mix: Optional[torch.Tensor] = None, vfreq: Optional[torch.Tensor] = None, window: int = 0,
                         tok_list: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every token (or of those in tok_list) over its request's pages with all heads of a token in one block:
    scores scale * q.k, capped by cap * tanh(. / cap) (cap <= 0: not), mixed over the heads by mix [nh, nh] (None: not), softmax,
    the weighted sum of the values, turned back by the query's position with vfreq (None: not).  Any sizes, float32 arithmetic."""
    _req(q, "q", dims=2); _req(cache_layer, "cache_layer", q.dtype); _req(block_tables, "block_tables", torch.int32, 2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(positions, "positions", torch.int32, 1); _req(out, "out", q.dtype, 2)
    T = q.shape[0]
    if q.shape[1] != nh * hd or out.shape != (T, nh * vd) or _page_size_of(cache_layer, nkv, hd, vd) != page_size:
        raise KernelError("attention_mixed_rows: shapes do not fit the head counts")
    if mix is not None:
        _req(mix, "mix", torch.float32, 2)
        if mix.shape != (nh, nh):
            raise KernelError("attention_mixed_rows: the mixing matrix is not [heads, heads]")
    if vfreq is not None:
        _req(vfreq, "vfreq", torch.float32, 1)
        if vfreq.shape[0] != vd // 2:
            raise KernelError("attention_mixed_rows: the values' frequencies do not fit their size")
    n = T
    if tok_list is not None:
        _req(tok_list, "tok_list", torch.int32, 1)
        n = tok_list.shape[0]
    _check(lib().vk_attention_mixed_rows(_p(q), _p(cache_layer), _p(block_tables), _p(token_seg), _p(positions), _p(tok_list), _p(out), n, nh, nkv, hd, vd,
                                         page_size, block_tables.shape[1], ctypes.c_float(scale), ctypes.c_float(cap), _p(mix), _p(vfreq), window,
                                         _dt(q), _stream()), "attention_mixed_rows")
    return out


MIXED_PREFILL_SIZES = (64, 128)
MIXED_SPLIT_MAX = 64            # most splits of a decoded token's keys


def attention_mixed_split_plan(max_context: int):
    """(splits, runs of 128 keys a split) for contexts of up to max_context positions: as many splits as there are runs, up to
    MIXED_SPLIT_MAX.  It depends on the engine's limit alone, so a captured graph holds for every batch."""
    runs = max(1, -(-max_context // 128))
    per = -(-runs // MIXED_SPLIT_MAX)
    return -(-runs // per), per


def attention_mixed_split(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, token_seg: torch.Tensor, positions: torch.Tensor,
                          out: torch.Tensor, part: torch.Tensor, nsplit: int, runs_per_split: int, nh: int, nkv: int, hd: int, vd: int,
                          page_size: int, scale: float, cap: float = 0.0, mix: Optional[torch.Tensor] = None, vfreq: Optional[torch.Tensor] = None,
                          window: int = 0, tok_list: Optional[torch.Tensor] = None) -> torch.Tensor:
    """attention_mixed_rows for single decoded tokens, a block a (token, split of the keys) and a launch that adds the splits up;
    part: float32 scratch of tokens * nsplit * nh * (vd + 2) values."""
    _req(q, "q", dims=2); _req(cache_layer, "cache_layer", q.dtype); _req(block_tables, "block_tables", torch.int32, 2)
    _req(token_seg, "token_seg", torch.int32, 1); _req(positions, "positions", torch.int32, 1); _req(out, "out", q.dtype, 2)
    _req(part, "part", torch.float32, 1)
    T = q.shape[0]
    n = T if tok_list is None else tok_list.shape[0]
    if q.shape[1] != nh * hd or out.shape != (T, nh * vd) or _page_size_of(cache_layer, nkv, hd, vd) != page_size:
        raise KernelError("attention_mixed_split: shapes do not fit the head counts")
    if part.numel() < n * nsplit * nh * (vd + 2):
        raise KernelError("attention_mixed_split: the scratch is too small")
    if (mix is not None and mix.shape != (nh, nh)) or (vfreq is not None and vfreq.shape[0] != vd // 2):
        raise KernelError("attention_mixed_split: the mixing matrix or the values' frequencies do not fit")
    if tok_list is not None:
        _req(tok_list, "tok_list", torch.int32, 1)
    _check(lib().vk_attention_mixed_split(_p(q), _p(cache_layer), _p(block_tables), _p(token_seg), _p(positions), _p(tok_list), _p(out), _p(part), n,
                                          nsplit, runs_per_split, nh, nkv, hd, vd, page_size, block_tables.shape[1], ctypes.c_float(scale),
                                          ctypes.c_float(cap), _p(mix), _p(vfreq), window, _dt(q), _stream()), "attention_mixed_split")
    add_launches(1)
    return out


def attention_mixed_prefill(q: torch.Tensor, cache_layer: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor, out: torch.Tensor, nh: int,
                            nkv: int, hd: int, vd: int, page_size: int, scale: float, cap: float = 0.0, mix: Optional[torch.Tensor] = None,
                            vfreq: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same attention for the tokens of prompt portions on the tensor cores (bfloat16): tiles int32 [n, 4] = first token, rows (up to
    64), position of the first token, segment.  Up to 16 heads; key and value sizes of MIXED_PREFILL_SIZES; no window."""
    _req(q, "q", torch.bfloat16, 2); _req(cache_layer, "cache_layer", torch.bfloat16); _req(block_tables, "block_tables", torch.int32, 2)
    _req(tiles, "tiles", torch.int32, 2); _req(out, "out", torch.bfloat16, 2)
    T = q.shape[0]
    if q.shape[1] != nh * hd or out.shape != (T, nh * vd) or tiles.shape[1] != 4 or _page_size_of(cache_layer, nkv, hd, vd) != page_size:
        raise KernelError("attention_mixed_prefill: shapes do not fit the head counts")
    if (mix is not None and mix.shape != (nh, nh)) or (vfreq is not None and vfreq.shape[0] != vd // 2):
        raise KernelError("attention_mixed_prefill: the mixing matrix or the values' frequencies do not fit")
    _check(lib().vk_attention_mixed_prefill(_p(q), _p(cache_layer), _p(block_tables), _p(tiles), _p(out), tiles.shape[0], nh, nkv, hd, vd, page_size,
                                            block_tables.shape[1], ctypes.c_float(scale), ctypes.c_float(cap), _p(mix), _p(vfreq), _stream()),
           "attention_mixed_prefill")
    return out


def attention_mixed(q: torch.Tensor, pages: torch.Tensor, meta, ctx, out: torch.Tensor, nh: int, nkv: int, hd: int, vd: int, page_size: int,
                    scale: float, cap: float = 0.0, mix: Optional[torch.Tensor] = None, vfreq: Optional[torch.Tensor] = None,
                    window: int = 0) -> torch.Tensor:
    """The attention with capped, mixed scores of a mixed batch over the paged cache; `meta` is the page group's GroupMeta.  Single
    decoded tokens take the split-key form, tokens of prompt portions the tensor-core kernel (bfloat16, sizes it is built for);
    whatever is left, and the whole exact 32-bit routing, takes attention_mixed_rows, which takes every size."""
    exact = q.dtype == torch.float32 and _float32_exact
    ws = ctx.workspace
    dec_ok = bool(ctx.num_dec) and not exact and nh * vd <= 4096
    pre_ok = (bool(ctx.num_pre) and q.dtype == torch.bfloat16 and hd in MIXED_PREFILL_SIZES and vd in MIXED_PREFILL_SIZES and nh <= 16
              and window == 0 and ctx.pre_tiles is not None and q.data_ptr() % 16 == 0 and pages.data_ptr() % 16 == 0)
    rows = lambda toks: attention_mixed_rows(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, nh, nkv, hd, vd, page_size, scale, cap,
                                             mix, vfreq, window, toks)
    if dec_ok:
        nsplit, per = attention_mixed_split_plan(ws.max_context)
        part = ws.flat(f"matt.part/{nh}/{vd}/{nsplit}", ws.max_segments * nsplit * nh * (vd + 2), torch.float32)
        attention_mixed_split(q, pages, meta.block_tables, ctx.token_seg, ctx.positions, out, part, nsplit, per, nh, nkv, hd, vd, page_size, scale,
                              cap, mix, vfreq, window, ctx.dec_tokens)
    if pre_ok:
        attention_mixed_prefill(q, pages, meta.block_tables, ctx.pre_tiles, out, nh, nkv, hd, vd, page_size, scale, cap, mix, vfreq)
    if not dec_ok and not pre_ok:
        return rows(None)
    if ctx.num_pre and not pre_ok:
        rows(ctx.pre_tokens)
    if ctx.num_dec and not dec_ok:
        rows(ctx.dec_tokens)
    return out


def latent_expand_gate(lat: torch.Tensor, w: torch.Tensor, gates: Optional[torch.Tensor], gate_off: int, H: int, rank: int, vd: int,
                       out: torch.Tensor) -> torch.Tensor:
    """out[t, h, :] = (w[h]^T lat[t, h, :]) * sigmoid(gates[t, gate_off + h vd : ...]); lat [T, H rank], w [H, rank, vd] and out [T, H vd] in one
    dtype, gates float32 [T, N] (None: no gate)."""
    _req(lat, "lat", dims=2); _req(w, "w", lat.dtype, 3); _req(out, "out", lat.dtype, 2)
    T = lat.shape[0]
    if lat.shape[1] != H * rank or w.shape != (H, rank, vd) or out.shape != (T, H * vd):
        raise KernelError("latent_expand_gate: shapes do not fit the head counts")
    N = 0
    if gates is not None:
        _req(gates, "gates", torch.float32, 2)
        N = gates.shape[1]
        if gates.shape[0] != T:
            raise KernelError("latent_expand_gate: the gates do not fit the tokens")
    _check(lib().vk_latent_expand_gate(_p(lat), _p(w), _p(gates), N, gate_off, H, rank, vd, _p(out), T, _dt(lat), _stream()), "latent_expand_gate")
    return out
