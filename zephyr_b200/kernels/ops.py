"""Python faces of the hand-written kernels.

Each function checks what the kernel cannot check for itself (device, types, contiguity, sizes),
launches on the current CUDA stream and returns without synchronising.  There is no fallback of
any kind: if the library cannot be built or loaded, or a kernel refuses a shape, the call raises.
"""

from __future__ import annotations

import contextlib
import ctypes
import gc
import math
import os
import struct
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass
from typing import Sequence

import torch

from ..config.errors import InvalidArgumentError, ZephyrError
from .build import BuildError, build_library

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
DECODE_SPLIT_SIZE = 256     # the shortest context a captured decode graph is sized for

_RC_TEXT = {1: "an argument outside the kernel's contract", 2: "the CUDA launch failed",
            3: "a configuration this kernel does not support"}
STATUS_TEXT = {
    1: "a token id outside the vocabulary",
    2: "a position outside the position table",
    3: "a page id outside the cache pool (or the null page) where a real page was expected",
    4: "a request row or block index outside the step's tables",
    5: "NaN or +inf among the logits",
    6: "an asynchronous copy into shared memory that did not complete within the wait limit",
    7: "an address or size that failed a kernel's own check (a bug in this package)",
    8: "a barrier across the grid that did not complete within the wait limit",
}


class KernelError(ZephyrError):
    pass


_lock = threading.Lock()
_lib: ctypes.CDLL | None = None

_SIGNATURES = {
    "zb_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_gather_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_longlong, c_longlong, c_int,
                   c_void_p],
    "zb_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_void_p],
    "zb_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "zb_add_bias": [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "zb_qk_norm_rope_cache": [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p,
                              c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_rope": [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                c_void_p],
    "zb_kv_write": [c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_attention_simt_tile_tokens": [c_int],
    "zb_paged_attention_simt": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_float, c_void_p, c_int, c_void_p, c_void_p],
    "zb_paged_decode_supported": [c_int, c_int, c_int, c_int],
    "zb_paged_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
                        c_void_p, c_void_p],
    "zb_paged_decode_fused": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_longlong, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p],
    "zb_paged_decode_set_trace": [c_void_p],
    "zb_paged_prefill_tile_tokens": [],
    "zb_paged_prefill_supported": [c_int, c_int, c_int, c_int],
    "zb_paged_prefill": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "zb_paged_prefill_tc_supported": [c_int, c_int, c_int, c_int, c_int],
    "zb_paged_prefill_tc_set_trace": [c_void_p],
    "zb_paged_prefill_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "zb_gemm_small_supported": [c_int, c_int, c_int],
    "zb_gemm_small": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                      c_int, c_void_p],
    "zb_fill_normal": [c_void_p, c_longlong, ctypes.c_ulonglong, c_float, c_float, c_int, c_void_p],
    "zb_gemm_tc_supported": [c_int, c_int, c_int, c_longlong, c_int, c_int],
    "zb_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_gemm_nt_simt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                        c_int, c_int, c_void_p],
    "zb_fused_chain_stage_supported": [c_int, c_int, c_int, c_int, c_int],
    "zb_fused_chain_max_stages": [],
    "zb_fused_chain_grid": [],
    "zb_set_sm_share": [c_int],
    "zb_fused_chain_set_flip_bytes": [c_longlong],
    "zb_set_dependent_launch": [c_int],
    "zb_fused_chain": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "zb_sample_chunks": [c_int],
    "zb_sample": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                  c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_void_p],
}


def library() -> ctypes.CDLL:
    """The compiled kernels, built at the first call.  Raises if they cannot be had."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            try:
                path = build_library()
            except BuildError as error:
                raise KernelError(f"the CUDA kernels of zephyr_b200 are unavailable: {error}") from error
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as error:
                raise KernelError(f"cannot load {path}: {error}") from error
            for name, argtypes in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = c_int
            lib.zb_last_cuda_error.argtypes = []
            lib.zb_last_cuda_error.restype = ctypes.c_char_p
            lib.zb_paged_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
            lib.zb_paged_decode_scratch_floats.restype = c_longlong
            lib.zb_paged_decode_balanced_scratch_floats.argtypes = [c_int, c_int, c_int]
            lib.zb_paged_decode_balanced_scratch_floats.restype = c_longlong
            if os.environ.get("ZEPHYR_B200_DEPENDENT_LAUNCH", "1") == "0":
                lib.zb_set_dependent_launch(0)
            _lib = lib
    return _lib


def library_path() -> str:
    return library()._name


LAUNCHES = 0      # kernels of this package launched so far (the bench reports the count of a timed region)
LAUNCH_COUNTS: dict[str, int] = {}      # the same by entry point


def _check(rc: int, name: str, kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += kernels
    LAUNCH_COUNTS[name] = LAUNCH_COUNTS.get(name, 0) + kernels
    if rc != 0:
        detail = ""
        if rc == 2:
            said = library().zb_last_cuda_error()
            detail = (f": {said.decode() if said else 'unknown'} ({torch.cuda.get_device_name()}; "
                      "the library holds sm_100a code only)")
        raise KernelError(f"{name}: {_RC_TEXT.get(rc, f'error {rc}')}{detail}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require(cond: bool, message: str) -> None:
    if not cond:
        raise InvalidArgumentError(message)


def _cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("zephyr_b200 kernels run on CUDA tensors only; there is no CPU path")


def _i32(*tensors: torch.Tensor) -> None:
    for t in tensors:
        _require(t.dtype == torch.int32 and t.is_contiguous(), "index tensors must be contiguous int32")


@contextlib.contextmanager
def capture(graph: "torch.cuda.CUDAGraph", **kwargs):
    """``torch.cuda.graph`` with the garbage collector held still.  A collection that happens to run
    inside a capture may destroy an older CUDA graph (one of a runner that was dropped, kept alive
    until then by a reference cycle); the runtime forbids that while any stream captures and the
    capture is lost ("operation failed due to a previous error during capture").  Such objects wait
    for the first collection after the capture."""
    enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, **kwargs):
            yield
    finally:
        if enabled:
            gc.enable()


def new_status(device: torch.device | str = "cuda") -> torch.Tensor:
    """The device status word kernels report into: [code, detail, index, unused]."""
    return torch.zeros(4, dtype=torch.int32, device=device)


_device_status: dict = {}


def device_status(device: torch.device | str) -> torch.Tensor:
    """The one status word of a device: kernels that are called without a status word report into it,
    and a model runner takes it as its own, so that what a product deep inside a part reports
    (a wait that ran out) is seen by the check after the step."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device(device.type, torch.cuda.current_device())
    word = _device_status.get(device)
    if word is None:
        word = _device_status[device] = new_status(device)
    return word


def check_status(status: torch.Tensor, where: str = "step") -> None:
    """Read the status word (this synchronises) and raise if a kernel reported an error."""
    code, detail, index, _ = status.tolist()
    if code != 0:
        status.zero_()
        for pool in _decode_buffers.values():       # a kernel that gave up may have left counters behind
            for _, count in pool:
                count.zero_()
        for buffer in list(_chain_sync.values()) + [b for (_, name), b in _sample_buffers.items() if name == "counters"]:
            buffer.zero_()
        raise KernelError(f"{where}: a kernel reported {STATUS_TEXT.get(code, f'error {code}')} "
                          f"(value {detail}, at element {index})")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float) -> torch.Tensor:
    """Fills a contiguous bfloat16 or float32 tensor with mean + std * z, z standard normal: element i
    is a function of (key, i) alone (a counter-based generator; see random_fill.cu)."""
    _cuda(out)
    _require(out.is_contiguous() and out.dtype in DTYPE_CODE, "a contiguous bfloat16 or float32 tensor")
    _check(library().zb_fill_normal(_ptr(out), out.numel(), int(key) & (2**64 - 1), float(mean), float(std),
                                    DTYPE_CODE[out.dtype], _stream()), "fill_normal")
    return out


# --------------------------------------------------------------------------- elementwise
def embedding(table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor, out: torch.Tensor | None = None):
    _cuda(table, ids, status)
    _i32(ids)
    _require(table.dim() == 2 and table.is_contiguous() and table.dtype in DTYPE_CODE, "table must be [V, H]")
    V, H = table.shape
    T = ids.numel()
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    _require(out.shape == (T, H) and out.dtype == table.dtype and out.is_contiguous(), "out must be [T, H]")
    _check(library().zb_embedding(_ptr(out), _ptr(table), _ptr(ids), T, H, V, DTYPE_CODE[table.dtype],
                                  _ptr(status), _stream()), "embedding")
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    _cuda(x, rows, status)
    _i32(rows)
    _require(x.dim() == 2 and x.is_contiguous() and x.dtype in DTYPE_CODE, "x must be a contiguous [T, H]")
    out = torch.empty((rows.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _check(library().zb_gather_rows(_ptr(out), _ptr(x), _ptr(rows), rows.numel(), x.shape[1], x.shape[0],
                                    DTYPE_CODE[x.dtype], _ptr(status), _stream()), "gather_rows")
    return out


def _scale_code(w: torch.Tensor, size: int) -> int:
    _require(w.dim() == 1 and w.numel() == size and w.is_contiguous() and w.dtype in DTYPE_CODE,
             f"a norm scale must be a contiguous vector of {size} float32 or bfloat16 values")
    return DTYPE_CODE[w.dtype]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm over the last dimension of a contiguous tensor (any leading shape)."""
    _cuda(x, w)
    _require(x.is_contiguous() and x.dtype in DTYPE_CODE, "x must be contiguous float32 or bfloat16")
    H = x.shape[-1]
    rows = x.numel() // H if H else 0
    if out is None:
        out = torch.empty_like(x)
    _require(out.shape == x.shape and out.dtype == x.dtype and out.is_contiguous(), "out must match x")
    _check(library().zb_rmsnorm(_ptr(out), _ptr(x), _ptr(w), _scale_code(w, H), float(eps), rows, H, H, H,
                                DTYPE_CODE[x.dtype], _stream()), "rmsnorm")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """residual += delta (in place), then return rmsnorm(residual) * w."""
    _cuda(residual, delta, w)
    _require(residual.dim() == 2 and residual.is_contiguous() and residual.dtype in DTYPE_CODE
             and delta.shape == residual.shape and delta.dtype == residual.dtype and delta.is_contiguous(),
             "residual and delta must be matching contiguous [T, H] tensors")
    rows, H = residual.shape
    if out is None:
        out = torch.empty_like(residual)
    _require(out.shape == residual.shape and out.dtype == residual.dtype and out.is_contiguous(), "out must match")
    _check(library().zb_add_rmsnorm(_ptr(out), _ptr(residual), _ptr(delta), _ptr(w), _scale_code(w, H), float(eps),
                                    rows, H, DTYPE_CODE[residual.dtype], _stream()), "add_rmsnorm")
    return out


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y [T, N] += bias [N] in place (rows of y may be strided; the bias bfloat16 or float32)."""
    _cuda(y, bias)
    _require(y.dim() == 2 and y.stride(1) == 1 and y.dtype in DTYPE_CODE, "y must be [T, N] with unit inner stride")
    _require(bias.dim() == 1 and bias.numel() == y.shape[1] and bias.is_contiguous() and bias.dtype in DTYPE_CODE,
             "one bias value per column")
    _check(library().zb_add_bias(_ptr(y), y.stride(0), _ptr(bias), DTYPE_CODE[bias.dtype], y.shape[0], y.shape[1],
                                 DTYPE_CODE[y.dtype], _stream()), "add_bias")
    return y


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None, blocked: bool = False) -> torch.Tensor:
    """silu(gate_up[:, :I]) * gate_up[:, I:] for a contiguous [T, 2I] tensor.  With ``blocked`` the gate
    and up columns alternate in blocks of 8 (the layout ``gemm_small(..., swiglu=True)`` reads)."""
    _cuda(gate_up)
    _require(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.dtype in DTYPE_CODE
             and gate_up.shape[1] % 2 == 0, "gate_up must be a contiguous [T, 2I] tensor")
    T, two_i = gate_up.shape
    if out is None:
        out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _require(out.shape == (T, two_i // 2) and out.dtype == gate_up.dtype and out.is_contiguous(), "out must be [T, I]")
    _require(not blocked or (two_i // 2) % 8 == 0, "the blocked layout needs I to be a multiple of 8")
    _check(library().zb_silu_mul(_ptr(out), _ptr(gate_up), T, two_i // 2, DTYPE_CODE[gate_up.dtype], int(blocked),
                                 _stream()), "silu_mul")
    return out


# ------------------------------------------------------------------ position and cache
def kv_swizzle(pos: int, chunks: int) -> int:
    """By how much the 16-byte chunks of the cache row at position ``pos`` are permuted: logical chunk
    c lives at chunk ``c ^ kv_swizzle(pos, chunks)``, with ``chunks`` = row bytes / 16.  (The same
    function as in csrc/common.cuh; tools and tests that read or fill a cache by hand need it.)"""
    step = chunks & 7
    if step == 0:
        return pos & 7
    if step == 4:
        return (pos >> 1) & 3
    if step in (2, 6):
        return (pos >> 2) & 1
    return 0


def kv_row_permutation(pos: int, head_dim: int, dtype: torch.dtype) -> torch.Tensor:
    """``perm`` with ``stored_row[perm[i]] == logical_row[i]`` for the cache row at position ``pos``."""
    size = torch.empty((), dtype=dtype).element_size()
    per_chunk = 16 // size
    chunks = head_dim * size // 16
    index = torch.arange(head_dim)
    return ((index // per_chunk) ^ kv_swizzle(pos, chunks)) * per_chunk + index % per_chunk



def _check_cache(kv_cache: torch.Tensor, nkv: int, hd: int, dtype: torch.dtype) -> tuple[int, int]:
    _require(kv_cache.dim() == 5 and kv_cache.is_contiguous() and kv_cache.shape[1] == 2
             and kv_cache.shape[2] == nkv and kv_cache.shape[4] == hd and kv_cache.dtype == dtype,
             "a cache must be a contiguous [pages, 2, kv_heads, page_size, head_dim] tensor of the model's type")
    return kv_cache.shape[0], kv_cache.shape[3]


def qk_norm_rope_cache(qkv: torch.Tensor, nh: int, nkv: int, hd: int, q_norm_w: torch.Tensor | None,
                       k_norm_w: torch.Tensor | None, eps: float, cos: torch.Tensor | None,
                       sin: torch.Tensor | None, positions: torch.Tensor, token_row: torch.Tensor,
                       kv_cache: torch.Tensor | None, block_table: torch.Tensor, status: torch.Tensor,
                       q_out: torch.Tensor | None = None) -> torch.Tensor:
    """Fused per-head norm of q and k, rotation, and the cache write; returns q as [T, nh*hd]."""
    _cuda(qkv, positions, token_row, block_table, status, kv_cache)
    _i32(positions, token_row, block_table)
    T = qkv.shape[0]
    width = (nh + 2 * nkv) * hd if kv_cache is not None else nh * hd
    _require(qkv.dim() == 2 and qkv.shape[1] >= width and qkv.stride(1) == 1 and qkv.dtype in DTYPE_CODE,
             "qkv must be [T, (heads + 2*kv_heads)*head_dim] with unit inner stride")
    _require(hd % 2 == 0 and positions.numel() == T and token_row.numel() == T, "one position and row per token")
    _require(block_table.dim() == 2, "block_table must be [rows, blocks]")
    w_code = 0
    if q_norm_w is not None or k_norm_w is not None:
        _require(q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype == k_norm_w.dtype,
                 "q and k norm scales come together and share a type")
        w_code = _scale_code(q_norm_w, hd)
        _scale_code(k_norm_w, hd)
    max_positions = 0
    if cos is not None:
        _require(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32
                 and cos.shape == sin.shape and cos.dim() == 2 and cos.shape[1] == hd // 2
                 and cos.is_contiguous() and sin.is_contiguous(), "cos/sin must be float32 [positions, head_dim/2]")
        max_positions = cos.shape[0]
    pages, page_size = (0, 1)
    if kv_cache is not None:
        pages, page_size = _check_cache(kv_cache, nkv, hd, qkv.dtype)
    if q_out is None:
        q_out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    _require(q_out.shape == (T, nh * hd) and q_out.is_contiguous() and q_out.dtype == qkv.dtype, "q_out shape")
    _check(library().zb_qk_norm_rope_cache(
        _ptr(q_out), _ptr(qkv), qkv.stride(0), _ptr(q_norm_w), _ptr(k_norm_w), w_code, float(eps), _ptr(cos),
        _ptr(sin), max_positions, _ptr(positions), _ptr(token_row), _ptr(kv_cache), _ptr(block_table),
        block_table.shape[1], page_size, pages, block_table.shape[0], T, nh, nkv, hd, DTYPE_CODE[qkv.dtype],
        _ptr(status), _stream()), "qk_norm_rope_cache")
    return q_out


def rope(x: torch.Tensor, heads: int, hd: int, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
         status: torch.Tensor) -> torch.Tensor:
    """Rotate x [T, >= heads*hd] in place (rows may be strided)."""
    _cuda(x, cos, sin, positions, status)
    _i32(positions)
    _require(x.dim() == 2 and x.stride(1) == 1 and x.shape[1] >= heads * hd and x.dtype in DTYPE_CODE, "x shape")
    _require(cos.dtype == torch.float32 and cos.shape == sin.shape and cos.shape[1] == hd // 2
             and cos.is_contiguous() and sin.is_contiguous(), "cos/sin must be float32 [positions, head_dim/2]")
    _check(library().zb_rope(_ptr(x), x.stride(0), x.shape[0], heads, hd, _ptr(cos), _ptr(sin), cos.shape[0],
                             _ptr(positions), DTYPE_CODE[x.dtype], _ptr(status), _stream()), "rope")
    return x


def kv_write(k: torch.Tensor, v: torch.Tensor, nkv: int, hd: int, positions: torch.Tensor, token_row: torch.Tensor,
             kv_cache: torch.Tensor, block_table: torch.Tensor, status: torch.Tensor) -> None:
    _cuda(k, v, positions, token_row, kv_cache, block_table, status)
    _i32(positions, token_row, block_table)
    _require(k.dim() == 2 and v.dim() == 2 and k.stride(1) == 1 and v.stride(1) == 1 and k.dtype == v.dtype
             and k.shape[0] == v.shape[0] and k.shape[1] >= nkv * hd and v.shape[1] >= nkv * hd, "k/v shapes")
    pages, page_size = _check_cache(kv_cache, nkv, hd, k.dtype)
    _check(library().zb_kv_write(_ptr(k), _ptr(v), k.stride(0), v.stride(0), _ptr(positions), _ptr(token_row),
                                 _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages,
                                 block_table.shape[0], k.shape[0], nkv, hd, DTYPE_CODE[k.dtype], _ptr(status),
                                 _stream()), "kv_write")


# ----------------------------------------------------------------------------- attention
def attention_tile_tokens(group: int) -> int:
    """New tokens of one request per tile of the general attention kernel, for this group size."""
    return library().zb_attention_simt_tile_tokens(int(group))


def paged_attention(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, tile_row: torch.Tensor,
                    tile_q0: torch.Tensor, tile_tokens: int, row_q_start: torch.Tensor, row_q_len: torch.Tensor,
                    row_ctx: torch.Tensor, nh: int, nkv: int, hd: int, window: int, scale: float,
                    status: torch.Tensor, out: torch.Tensor | None = None,
                    head_slopes: torch.Tensor | None = None) -> torch.Tensor:
    """The general kernel: causal attention of every new token over its request's pages.
    ``head_slopes`` (float32 [nh]): query head h adds head_slopes[h] * (key position - query position)
    to its scores, a position encoding that is a bias on the scores."""
    _cuda(q, kv_cache, block_table, tile_row, tile_q0, row_q_start, row_q_len, row_ctx, status, head_slopes)
    _require(head_slopes is None or (head_slopes.dtype == torch.float32 and head_slopes.is_contiguous()
                                     and head_slopes.numel() == nh), "one float32 slope per query head")
    _i32(block_table, tile_row, tile_q0, row_q_start, row_q_len, row_ctx)
    _require(q.dim() == 2 and q.is_contiguous() and q.shape[1] == nh * hd and q.dtype in DTYPE_CODE, "q shape")
    pages, page_size = _check_cache(kv_cache, nkv, hd, q.dtype)
    if out is None:
        out = torch.empty_like(q)
    _require(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    _check(library().zb_paged_attention_simt(
        _ptr(out), _ptr(q), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages,
        block_table.shape[0], _ptr(tile_row), _ptr(tile_q0), tile_row.numel(), int(tile_tokens), _ptr(row_q_start),
        _ptr(row_q_len), _ptr(row_ctx), nh, nkv, hd, int(window), float(scale), _ptr(head_slopes), DTYPE_CODE[q.dtype],
        _ptr(status), _stream()), "paged_attention")
    return out


def paged_decode_supported(nh: int, nkv: int, hd: int, dtype: torch.dtype) -> bool:
    return dtype in DTYPE_CODE and bool(library().zb_paged_decode_supported(nh, nkv, hd, DTYPE_CODE[dtype]))


def paged_decode_scratch_floats(n_rows: int, nh: int, hd: int, max_splits: int) -> int:
    return int(library().zb_paged_decode_scratch_floats(n_rows, nh, hd, max_splits))


# Buffers of the decode kernel, kept for the life of the process: the partial results of the splits
# (contents irrelevant between calls) and the arrival counters (zero between calls: the kernel
# leaves them as it found them).  Buffers are only ever added, never freed or moved, because
# captured graphs hold their addresses.
_decode_buffers: dict[tuple[torch.device, int], list[tuple[torch.Tensor, torch.Tensor]]] = {}

# Two halves of a batch may run side by side on two streams (``parts.Model``): each is a lane with
# workspaces of its own (the decode kernel's partial results and counters, the chain's barrier
# counters), and the persistent kernels take half the SMs each.
LANE = 0


class lane:
    """``with ops.lane(1, ctas): ...``: launches inside use lane 1's workspaces and at most ``ctas``
    CTAs per persistent kernel (0: one per SM)."""

    def __init__(self, index: int, ctas: int = 0):
        self.index, self.ctas = index, ctas

    def __enter__(self):
        global LANE
        self.before = (LANE, int(library().zb_set_sm_share(int(self.ctas))))
        LANE = self.index
        return self

    def __exit__(self, *exc):
        global LANE
        LANE = self.before[0]
        library().zb_set_sm_share(self.before[1])
        return False


def _decode_workspace(device: torch.device, floats: int, counters: int) -> tuple[torch.Tensor, torch.Tensor]:
    pool = _decode_buffers.setdefault((device, LANE), [])
    for scratch, count in pool:
        if scratch.numel() >= floats and count.numel() >= counters:
            return scratch, count
    scratch = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
    count = torch.zeros(max(counters, 1 << 12), dtype=torch.int32, device=device)
    pool.append((scratch, count))
    return scratch, count


def decode_split_size(n_rows: int, nkv: int, max_context: int) -> int:
    """A size for fixed splits (``paged_decode(..., split_size=...)``): as many splits of a row's
    context as give every SM one item and none two (a second round of items would leave most SMs
    idle), and no split shorter than 128 positions.  ``paged_decode`` takes fixed splits for a
    handful of rows (4 * rows * key/value heads <= SMs); for more, the kernel spreads the tiles of
    all rows evenly over its CTAs.  Either way, where a row's context is cut, and with that the last
    bits of its result, depends on how many rows are decoded beside it."""
    per_pair = max(1, _sm_count() // max(1, n_rows * nkv))     # splits of a (row, key/value head) pair: one item per SM
    split = -(-max_context // per_pair)
    return max(128, -(-split // 32) * 32)


_SM_COUNT: dict[int, int] = {}


def _sm_count() -> int:
    """SMs a persistent kernel launched now may take (all, or the current lane's share)."""
    device = torch.cuda.current_device()
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    share = int(library().zb_set_sm_share(0))
    library().zb_set_sm_share(share)
    return min(_SM_COUNT[device], share) if share > 0 else _SM_COUNT[device]


def paged_decode(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, rows: torch.Tensor,
                 row_q_start: torch.Tensor, row_ctx: torch.Tensor, max_context: int, nh: int, nkv: int, hd: int,
                 window: int, scale: float, status: torch.Tensor, out: torch.Tensor,
                 scratch: torch.Tensor | None = None, split_size: int | None = None,
                 counters: torch.Tensor | None = None) -> torch.Tensor:
    """Split-context attention for rows with one new token each; writes those tokens' rows of ``out``.

    ``max_context`` is at least the longest context of the rows, the new token included.  ``scratch``
    (float32, any contents) and ``counters`` (int32, zero) come from a process-wide workspace unless
    given.  ``split_size`` None or 0: balanced work items; a multiple of 32: fixed splits of that size."""
    _cuda(q, kv_cache, block_table, rows, row_q_start, row_ctx, status, out)
    _i32(block_table, rows, row_q_start, row_ctx)
    _require(q.dim() == 2 and q.is_contiguous() and q.shape[1] == nh * hd and q.dtype == torch.bfloat16, "q shape")
    _require(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    pages, page_size = _check_cache(kv_cache, nkv, hd, q.dtype)
    n_rows = rows.numel()
    if split_size is None and n_rows * nkv * 4 <= _sm_count():
        # A handful of long rows: fixed splits keep every item inside one row (a CTA whose share
        # straddles two rows pays for two merges, which shows when the shares are a few tiles).
        split_size = decode_split_size(n_rows, nkv, max_context)
    if split_size is None or split_size == 0:
        # Balanced items: the tiles of all rows spread evenly over the CTAs (see attention_decode.cu).
        split_size, max_splits = 0, max(1, math.ceil(max_context / 32))
        need = int(library().zb_paged_decode_balanced_scratch_floats(nh, nkv, hd))
    else:
        max_splits = max(1, math.ceil(max_context / split_size))
        need = paged_decode_scratch_floats(n_rows, nh, hd, max_splits)
    if scratch is None or counters is None:
        scratch, counters = _decode_workspace(q.device, need, n_rows * nkv)
    _require(scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need,
             f"scratch must hold {need} floats")
    _require(counters.dtype == torch.int32 and counters.is_contiguous() and counters.numel() >= n_rows * nkv,
             f"counters must hold {n_rows * nkv} zeroed int32 values")
    _check(library().zb_paged_decode(
        _ptr(out), _ptr(q), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages,
        block_table.shape[0], _ptr(rows), n_rows, _ptr(row_q_start), _ptr(row_ctx), nh, nkv, hd, int(window),
        float(scale), int(split_size), max_splits, _ptr(scratch), _ptr(counters), _ptr(status), _stream()),
        "paged_decode")
    return out


def paged_decode_fused(qkv: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, rows: torch.Tensor,
                       row_q_start: torch.Tensor, row_ctx: torch.Tensor, max_context: int, nh: int, nkv: int, hd: int,
                       window: int, scale: float, q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None, eps: float,
                       cos: torch.Tensor | None, sin: torch.Tensor | None, status: torch.Tensor, out: torch.Tensor,
                       split_size: int | None = None) -> torch.Tensor:
    """``qk_norm_rope_cache`` and ``paged_decode`` in one kernel, for steps in which every request
    has exactly one new token: ``qkv`` [T, >= (nh + 2 nkv) hd] holds the new tokens raw; the per-head
    norms, the rotation and the cache write of the new keys and values happen inside the attention
    kernel (a row's new position is its ``row_ctx``), and ``out`` [T, nh hd] gets the attention's
    result.  No kernel stands between the projection and the attention then."""
    _cuda(qkv, kv_cache, block_table, rows, row_q_start, row_ctx, status, out, q_norm_w, k_norm_w, cos, sin)
    _i32(block_table, rows, row_q_start, row_ctx)
    T = qkv.shape[0]
    _require(qkv.dim() == 2 and qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] >= (nh + 2 * nkv) * hd
             and qkv.stride(0) % 2 == 0, "qkv must be bfloat16 [T, (heads + 2*kv_heads)*head_dim] with unit inner stride")
    _require(out.shape == (T, nh * hd) and out.dtype == torch.bfloat16 and out.is_contiguous(), "out must be [T, heads*head_dim]")
    pages, page_size = _check_cache(kv_cache, nkv, hd, qkv.dtype)
    w_code = 0
    if q_norm_w is not None or k_norm_w is not None:
        _require(q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype == k_norm_w.dtype,
                 "q and k norm scales come together and share a type")
        w_code = _scale_code(q_norm_w, hd)
        _scale_code(k_norm_w, hd)
    max_positions = 0
    if cos is not None:
        _require(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32
                 and cos.shape == sin.shape and cos.dim() == 2 and cos.shape[1] == hd // 2
                 and cos.is_contiguous() and sin.is_contiguous(), "cos/sin must be float32 [positions, head_dim/2]")
        max_positions = cos.shape[0]
    n_rows = rows.numel()
    if split_size is None and n_rows * nkv * 4 <= _sm_count():
        split_size = decode_split_size(n_rows, nkv, max_context)
    if split_size is None or split_size == 0:
        split_size, max_splits = 0, max(1, math.ceil(max_context / 32))
        need = int(library().zb_paged_decode_balanced_scratch_floats(nh, nkv, hd))
    else:
        max_splits = max(1, math.ceil(max_context / split_size))
        need = paged_decode_scratch_floats(n_rows, nh, hd, max_splits)
    scratch, counters = _decode_workspace(qkv.device, need, n_rows * nkv)
    _check(library().zb_paged_decode_fused(
        _ptr(out), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages, block_table.shape[0],
        _ptr(rows), n_rows, _ptr(row_q_start), _ptr(row_ctx), nh, nkv, hd, int(window), float(scale), int(split_size),
        max_splits, _ptr(scratch), _ptr(counters), _ptr(status), _ptr(qkv), qkv.stride(0), _ptr(q_norm_w), _ptr(k_norm_w),
        w_code, float(eps), _ptr(cos), _ptr(sin), max_positions, _stream()), "paged_decode_fused")
    return out


USE_TCGEN05_PREFILL = True      # off: the mma.sync kernel for every head size (for comparisons)


def paged_decode_trace(buffer: torch.Tensor | None) -> None:
    """Later ``paged_decode`` launches write every CTA's timeline into ``buffer`` (int32 [1024, 8] on the
    device: the global timer in ns at the CTA's start, after the wait for earlier kernels, when its
    first tile had landed, after its last tile, at its end; then its items and tiles); None turns it off."""
    if buffer is not None:
        _cuda(buffer)
        _require(buffer.dtype == torch.int32 and buffer.is_contiguous() and buffer.numel() >= 8 * 1024, "int32 [1024, 8]")
    _check(library().zb_paged_decode_set_trace(_ptr(buffer)), "paged_decode_trace", kernels=0)


def paged_prefill_trace(buffer: torch.Tensor | None) -> None:
    """Later tcgen05 prompt-attention launches write the timeline of their first CTA (the longest
    work of the launch) into ``buffer`` (int32 [2, 64, 4] on the device; per tile of keys, [0]: the
    global timer in ns when S was issued, when its softmax began, when its probabilities were written,
    when O += P V was issued; [1]: when the first loader thread began to issue its keys, its values,
    and when it had issued them); None turns it off."""
    if buffer is not None:
        _cuda(buffer)
        _require(buffer.dtype == torch.int32 and buffer.is_contiguous() and buffer.numel() >= 512, "int32 [2, 64, 4]")
    _check(library().zb_paged_prefill_tc_set_trace(_ptr(buffer)), "paged_prefill_trace", kernels=0)


def paged_prefill_tile_tokens() -> int:
    """New tokens of one request per tile of the tensor-core prompt attention kernel."""
    return library().zb_paged_prefill_tile_tokens()


def paged_prefill_supported(nh: int, nkv: int, hd: int, dtype: torch.dtype) -> bool:
    return dtype in DTYPE_CODE and bool(library().zb_paged_prefill_supported(nh, nkv, hd, DTYPE_CODE[dtype]))


def paged_prefill(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, tile_row: torch.Tensor,
                  tile_q0: torch.Tensor, row_q_start: torch.Tensor, row_q_len: torch.Tensor, row_ctx: torch.Tensor,
                  nh: int, nkv: int, hd: int, window: int, scale: float, status: torch.Tensor,
                  out: torch.Tensor) -> torch.Tensor:
    """Tensor-core attention for rows with several new tokens, cut into tiles of
    ``paged_prefill_tile_tokens()``; writes those tokens' rows of ``out``."""
    _cuda(q, kv_cache, block_table, tile_row, tile_q0, row_q_start, row_q_len, row_ctx, status, out)
    _i32(block_table, tile_row, tile_q0, row_q_start, row_q_len, row_ctx)
    _require(q.dim() == 2 and q.is_contiguous() and q.shape[1] == nh * hd and q.dtype == torch.bfloat16, "q shape")
    _require(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    pages, page_size = _check_cache(kv_cache, nkv, hd, q.dtype)
    # Head size 128 runs on tcgen05 with the accumulators in tensor memory; other sizes on mma.sync.
    tensor_memory = USE_TCGEN05_PREFILL and bool(library().zb_paged_prefill_tc_supported(nh, nkv, hd, DTYPE_CODE[q.dtype],
                                                                                     page_size))
    kernel = library().zb_paged_prefill_tc if tensor_memory else library().zb_paged_prefill
    _check(kernel(
        _ptr(out), _ptr(q), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages,
        block_table.shape[0], _ptr(tile_row), _ptr(tile_q0), tile_row.numel(), _ptr(row_q_start), _ptr(row_q_len),
        _ptr(row_ctx), nh, nkv, hd, int(window), float(scale), _ptr(status), _stream()), "paged_prefill")
    return out


# ------------------------------------------------------------------------ matrix products
def gemm_nt_simt(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] times w [N, K] transposed, float32 multiply-adds on CUDA cores."""
    _cuda(x, w)
    _require(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.dtype == w.dtype
             and x.dtype in DTYPE_CODE and x.stride(1) == 1 and w.stride(1) == 1, "x [M, K] and w [N, K] of one type")
    out_dtype = out_dtype or x.dtype
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _require(out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1, "out must be [M, N]")
    _check(library().zb_gemm_nt_simt(_ptr(out), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                                     DTYPE_CODE[x.dtype], DTYPE_CODE[out_dtype], _stream()), "gemm_nt_simt")
    return out


SMALL_GEMM_MAX_ROWS = 64      # what the kernel takes
SMALL_GEMM_ROWS = 16          # up to here it beats the library product; beyond, activations are re-read too often


def gemm_small_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True if the weight-streaming kernel for few rows takes x [M, K] times w [N, K] transposed."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.shape[0] <= SMALL_GEMM_MAX_ROWS and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(library().zb_gemm_small_supported(x.shape[0], w.shape[0], x.shape[1])))


def gemm_small(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
               swiglu: bool = False) -> torch.Tensor:
    """x [M <= 64, K] times w [N, K] transposed, bfloat16, float32 accumulation, weights read once.
    With ``swiglu`` the rows of w are blocks of 8 gate rows each followed by its 8 up rows, and the
    result is silu(gate) * up, [M, N / 2]."""
    _cuda(x, w)
    _require(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], "x [M, K] and w [N, K]")
    _require(gemm_small_supported(x, w), "gemm_small takes bfloat16, M <= 64, K a multiple of 8, 16-byte aligned rows")
    out_dtype = out_dtype or x.dtype
    M, K = x.shape
    N = w.shape[0]
    _require(not swiglu or N % 16 == 0, "swiglu needs a multiple of 16 rows")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    _check(library().zb_gemm_small(_ptr(out), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                                   DTYPE_CODE[out_dtype], int(swiglu), _stream()), "gemm_small")
    return out


GEMM_TC_MIN_ROWS = 512        # from here on the product with the activation in its epilogue beats the library's
                              # product followed by the activation kernel (measured at widths 1024 to 5120)


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> bool:
    """True if the tcgen05 product takes x [M, K] times w [N, K] transposed (bfloat16, K a multiple of 8)."""
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.shape[1] == w.shape[1] and x.stride(1) == 1 and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return False
    M, K = x.shape
    N = w.shape[0]
    ldy = (N // 2 if swiglu else N + 7) // 8 * 8
    return bool(library().zb_gemm_tc_supported(M, N, K, x.stride(0), ldy, int(swiglu)))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, swiglu: bool = False, block_n: int = 0,
            status: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [M, K] times w [N, K] transposed on tcgen05 tensor cores, bfloat16 with float32 sums in
    tensor memory; the result in bfloat16, or with ``out_dtype=torch.float32`` the sums as they are.
    With ``swiglu`` the rows of w are blocks of 8 gate rows each followed by its 8 up
    rows, and the result is silu(gate) * up, [M, N / 2], taken from the float32 sums and rounded once.
    ``block_n`` is the width of an output tile (256, 128; 2: tiles of 256 x 256 on pairs of SMs; 0: chosen).  ``status`` (default: the
    device's status word) receives a report if a wait inside the kernel ran out."""
    _cuda(x, w)
    _require(gemm_tc_supported(x, w, swiglu), "gemm_tc takes bfloat16 x [M, K] and contiguous w [N, K], K a multiple of 8, "
             "16-byte aligned; with swiglu N a multiple of 16")
    wide = out_dtype == torch.float32
    _require(out_dtype in (None, torch.bfloat16, torch.float32) and not (wide and swiglu), "bfloat16 out, or float32 without the activation")
    M, K = x.shape
    N = w.shape[0]
    width = N // 2 if swiglu else N
    ldy = (width + 3) // 4 * 4 if wide else (width + 7) // 8 * 8
    out = torch.empty((M, ldy), dtype=torch.float32 if wide else torch.bfloat16, device=x.device)
    if status is None:
        status = device_status(x.device)
    _check(library().zb_gemm_tc(_ptr(out), _ptr(x), _ptr(w), M, N, K, x.stride(0), ldy, 2 if wide else int(swiglu),
                                int(block_n), _ptr(status), _stream()), "gemm_tc")
    return out if ldy == width else out[:, :width].contiguous()


# ------------------------------------------------------------------ chains of small products
PROLOGUE_NONE, PROLOGUE_NORM, PROLOGUE_ADD_NORM = 0, 1, 2
EPILOGUE_NONE, EPILOGUE_SWIGLU = 0, 1
FUSED_CHAIN_MAX_TOKENS = 16


class _ChainStage(ctypes.Structure):
    _fields_ = [("w", c_void_p), ("ldw", c_longlong), ("N", c_int), ("K", c_int), ("prologue", c_int),
                ("epilogue", c_int), ("x", c_void_p), ("ldx", c_longlong), ("residual_in", c_void_p),
                ("residual_out", c_void_p), ("delta", c_void_p), ("ldd", c_longlong), ("norm_w", c_void_p),
                ("norm_w_dtype", c_int), ("eps", c_float), ("y", c_void_p), ("ldy", c_longlong)]


@dataclass
class ChainStage:
    """One stage of ``fused_chain``: y = epilogue(prologue(...) w^T), bfloat16.

    The input is ``x`` [M, K] as given, or, with ``norm_w``, the RMS norm of ``residual_in`` [M, K]
    (after ``delta`` [M, K] has been added to it, if given; the sum goes to ``residual_out``).  With
    ``swiglu`` the rows of ``w`` are blocks of 8 gate rows and their 8 up rows and y is [M, N / 2]."""

    w: torch.Tensor
    y: torch.Tensor
    x: torch.Tensor | None = None
    residual_in: torch.Tensor | None = None
    residual_out: torch.Tensor | None = None
    delta: torch.Tensor | None = None
    norm_w: torch.Tensor | None = None
    eps: float = 0.0
    swiglu: bool = False

    @property
    def prologue(self) -> int:
        if self.norm_w is None:
            return PROLOGUE_NONE
        return PROLOGUE_ADD_NORM if self.delta is not None else PROLOGUE_NORM


def fused_chain_stage_supported(tokens: int, w: torch.Tensor, normed_input: bool, swiglu: bool) -> bool:
    """True if a product with ``w`` [N, K] can be a stage of a chain for this many tokens."""
    return (w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1 and w.stride(0) % 8 == 0
            and w.data_ptr() % 16 == 0
            and bool(library().zb_fused_chain_stage_supported(int(tokens), w.shape[0], w.shape[1],
                                                              PROLOGUE_NORM if normed_input else PROLOGUE_NONE,
                                                              EPILOGUE_SWIGLU if swiglu else EPILOGUE_NONE)))


def fused_chain_max_stages() -> int:
    return int(library().zb_fused_chain_max_stages())


# The arrival counters of the chain kernel's barrier, per device: zero between launches.
_chain_sync: dict[tuple[torch.device, int], torch.Tensor] = {}
_chain_rows: dict[tuple[torch.device, int], torch.Tensor] = {}


def set_dependent_launch(enabled: bool) -> bool:
    """Launch the kernels of a decode step (position encoding with cache write, decode attention,
    chain) as programmatic dependents of the kernel before them: a kernel's CTAs then set themselves
    up while the one before is still finishing.  On by default; returns the previous setting."""
    return bool(library().zb_set_dependent_launch(int(bool(enabled))))


def fused_chain_grid() -> int:
    """CTAs of a chain launch (one per SM)."""
    return int(library().zb_fused_chain_grid())


def fused_chain(stages: Sequence[ChainStage], tokens: int, status: torch.Tensor,
                trace: torch.Tensor | None = None) -> None:
    """Run the stages one after the other in one cooperative launch (see csrc/fused_chain.cu).
    Every tensor is bfloat16 on the device (a norm weight may be float32); rows are contiguous.
    ``trace`` (int32 [fused_chain_grid(), stages, 4]) receives every CTA's timeline, nanoseconds of
    the device's global timer (low 32 bits): the stage's start, its input in place, its products
    done, the barrier passed."""
    _require(1 <= len(stages) <= fused_chain_max_stages(), "a chain has 1 to 8 stages")
    _require(1 <= tokens <= FUSED_CHAIN_MAX_TOKENS, "a chain takes 1 to 16 tokens")
    packed = (_ChainStage * len(stages))()
    for slot, st in zip(packed, stages):
        N, K = st.w.shape
        _cuda(st.w, st.y, st.x, st.residual_in, st.residual_out, st.delta, st.norm_w)
        for t in (st.w, st.y, st.x, st.residual_in, st.residual_out, st.delta):
            _require(t is None or (t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1), "bfloat16 matrices")
        _require(st.y.shape == (tokens, N // 2 if st.swiglu else N), "y must be [tokens, N] ([tokens, N / 2] with swiglu)")
        slot.w, slot.ldw, slot.N, slot.K = st.w.data_ptr(), st.w.stride(0), N, K
        slot.prologue, slot.epilogue = st.prologue, EPILOGUE_SWIGLU if st.swiglu else EPILOGUE_NONE
        slot.y, slot.ldy = st.y.data_ptr(), st.y.stride(0)
        if st.norm_w is None:
            _require(st.x is not None and st.x.shape == (tokens, K), "x must be [tokens, K]")
            slot.x, slot.ldx = st.x.data_ptr(), st.x.stride(0)
        else:
            _require(st.residual_in is not None and st.residual_in.shape == (tokens, K) and st.residual_in.is_contiguous(),
                     "residual_in must be contiguous [tokens, K]")
            _require(st.norm_w.numel() == K and st.norm_w.dtype in DTYPE_CODE and st.norm_w.is_contiguous(), "norm weight [K]")
            slot.residual_in, slot.norm_w = st.residual_in.data_ptr(), st.norm_w.data_ptr()
            slot.norm_w_dtype, slot.eps = DTYPE_CODE[st.norm_w.dtype], float(st.eps)
            if st.delta is not None:
                _require(st.delta.shape == (tokens, K), "delta must be [tokens, K]")
                _require(st.residual_out is not None and st.residual_out.shape == (tokens, K)
                         and st.residual_out.is_contiguous() and st.residual_out.data_ptr() != st.residual_in.data_ptr(),
                         "residual_out must be a second contiguous [tokens, K] buffer")
                slot.delta, slot.ldd, slot.residual_out = st.delta.data_ptr(), st.delta.stride(0), st.residual_out.data_ptr()
    device = (stages[0].w.device, LANE)
    sync = _chain_sync.get(device)
    if sync is None:
        sync = _chain_sync[device] = torch.zeros(2, dtype=torch.int32, device=stages[0].w.device)
    if trace is not None:
        _cuda(trace)
        _require(trace.dtype == torch.int32 and trace.is_contiguous()
                 and trace.numel() >= 4 * len(stages) * fused_chain_grid(), "trace must be int32 [fused_chain_grid(), stages, 4]")
    # Room for the rows of a long normalised input, which the kernel normalises once for all CTAs.
    longest = max((st.w.shape[1] for st in stages if st.norm_w is not None), default=0)
    scratch = _chain_rows.get(device)
    if longest and (scratch is None or scratch.numel() < FUSED_CHAIN_MAX_TOKENS * longest):
        scratch = _chain_rows[device] = torch.empty(FUSED_CHAIN_MAX_TOKENS * longest, dtype=torch.bfloat16,
                                                    device=stages[0].w.device)
    _check(library().zb_fused_chain(ctypes.addressof(packed), len(stages), int(tokens), _ptr(sync), _ptr(status),
                                    _ptr(trace), _ptr(scratch) if longest else None, _stream()), "fused_chain")


USE_LIBRARY_PRODUCTS = True     # off: every bfloat16 product of more than a few rows runs on this package's tcgen05 kernel


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
           bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x w^T.  float32 runs on this package's CUDA-core kernel (no TF32 anywhere).  bfloat16
    with up to 64 rows (a decode step) runs on this package's weight-streaming kernel; larger
    bfloat16 products run on the vendor library's tensor-core product, as the reference's linear
    layers do (src/layer/linear.cpp:22-24 -> cuBLASLt), where that is the faster one; with
    ``USE_LIBRARY_PRODUCTS`` off they run on this package's tcgen05 kernel (``gemm_tc``), so that no
    library kernel is left on the path.  Accumulation is float32 everywhere.  A ``bias`` [N] is
    added to the product's (rounded) output by a kernel of its own."""
    if bias is not None:
        return add_bias(linear(x, w, out_dtype), bias)
    _cuda(x, w)
    if x.dtype == torch.float32:
        return gemm_nt_simt(x, w, out_dtype)
    if x.shape[0] <= SMALL_GEMM_ROWS and gemm_small_supported(x, w):
        return gemm_small(x, w, out_dtype)
    if not USE_LIBRARY_PRODUCTS and gemm_tc_supported(x, w):
        return gemm_tc(x, w, out_dtype=out_dtype)
    if out_dtype is None or out_dtype == x.dtype:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


# ------------------------------------------------------------------------------ sampling
@dataclass(frozen=True)
class SampleRow:
    """How one row of logits is turned into a token (the kernel's record of a row).

    ``temperature`` below 1e-7 means greedy.  ``top_k`` 0, ``top_p`` 0 and ``min_p`` 0 switch those
    filters off.  ``num_logprobs`` -1 asks for no report; n >= 0 for the chosen token's
    log-probability and the n most probable tokens."""

    temperature: float = 0.0
    uniform: float = 0.0
    top_k: int = 0
    top_p: float = 0.0
    min_p: float = 0.0
    num_logprobs: int = -1
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-7

    @property
    def ranked(self) -> bool:
        return not self.greedy and (self.top_k > 0 or self.top_p > 0.0)


@dataclass(frozen=True)
class TokenAdjustment:
    """What a row's history and biases do to one token's logit."""

    row: int
    token: int
    generated_count: int = 0
    seen: bool = False
    bias: float = 0.0


@dataclass
class SampleOutput:
    """Device results of ``sample_rows``: row r's chosen token is ``ids[offsets[r]]``, followed by its
    top tokens if it reports; ``logprobs`` runs parallel to ``ids`` (None if no row reports)."""

    ids: torch.Tensor
    logprobs: torch.Tensor | None
    offsets: list[int]


_ROW_FORMAT = struct.Struct("<dddffffiiiiii")
_ADJUSTMENT_FORMAT = struct.Struct("<iiiif")
_JOB_FORMAT = struct.Struct("<ii")
_PHASE_WEIGHTS, _PHASE_DRAW_INDEXED, _PHASE_DRAW_RANKED, _PHASE_REPORT = 1, 2, 4, 8

# Work buffers of the sampling kernels, kept per device and only ever grown.  The counters are zero
# between calls: the kernel leaves them as it found them.
_sample_buffers: dict[tuple[torch.device, str], torch.Tensor] = {}


def _sample_buffer(device: torch.device, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
    have = _sample_buffers.get((device, name))
    if have is None or have.numel() < numel:
        size = max(numel, 1024)
        have = (torch.zeros if zero else torch.empty)(size, dtype=dtype, device=device)
        _sample_buffers[(device, name)] = have
    return have


def sample_chunks(vocab: int) -> int:
    return int(library().zb_sample_chunks(int(vocab)))


def sample_rows(logits: torch.Tensor, rows: Sequence[SampleRow] | None, status: torch.Tensor,
                adjustments: Sequence[TokenAdjustment] = ()) -> SampleOutput:
    """One token per row of float32 logits [rows, V], chosen as each row's ``SampleRow`` says
    (``rows`` None: argmax everywhere).  Adjustments are applied to ``logits`` in place first."""
    _cuda(logits, status)
    _require(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1,
             "logits must be float32 [rows, V]")
    R, V = logits.shape
    device = logits.device
    chunks = sample_chunks(V)
    part_f = _sample_buffer(device, "part_f", 3 * R * chunks, torch.float32)
    part_i = _sample_buffer(device, "part_i", R * chunks, torch.int32)
    counters = _sample_buffer(device, "counters", R, torch.int32, zero=True)
    row_max = _sample_buffer(device, "row_max", R, torch.float32)
    row_arg = _sample_buffer(device, "row_arg", R, torch.int32)
    if rows is None:
        _require(not adjustments, "adjustments need row parameters")
        ids = torch.empty(R, dtype=torch.int32, device=device)
        _check(library().zb_sample(_ptr(ids), None, _ptr(logits), logits.stride(0), R, V, None, None, 0, None, 0, 0,
                                   _ptr(part_f), _ptr(part_i), _ptr(counters), _ptr(row_max), _ptr(row_arg), None,
                                   None, None, None, _ptr(status), _stream()), "sample")
        return SampleOutput(ids, None, list(range(R)))
    _require(len(rows) == R, "one SampleRow per row of logits")

    # Pack the rows, the sort jobs they need and the adjustments into one upload.
    jobs: list[tuple[int, int]] = []
    offsets: list[int] = []
    packed_rows = bytearray()
    results, phases = 0, 0
    for r, row in enumerate(rows):
        sort_slot = report_slot = -1
        if not row.greedy or row.num_logprobs >= 0:
            phases |= _PHASE_WEIGHTS
        if row.ranked:
            sort_slot = len(jobs)
            jobs.append((r, 0))
            phases |= _PHASE_DRAW_RANKED
        elif not row.greedy:
            phases |= _PHASE_DRAW_INDEXED
        num_logprobs = min(int(row.num_logprobs), V)
        if num_logprobs >= 0:
            phases |= _PHASE_REPORT
            if num_logprobs > 0:
                report_slot = len(jobs)
                jobs.append((r, 1))
        offsets.append(results)
        packed_rows += _ROW_FORMAT.pack(row.temperature, row.top_p, row.min_p, row.uniform, row.frequency_penalty,
                                        row.presence_penalty, row.repetition_penalty, min(int(row.top_k), V),
                                        num_logprobs, results, sort_slot, report_slot, 0)
        results += 1 + max(num_logprobs, 0)
    for a in adjustments:
        _require(0 <= a.row < R and 0 <= a.token < V, "an adjustment names a row and a token of the logits")
    packed_adjustments = b"".join(_ADJUSTMENT_FORMAT.pack(a.row, a.token, a.generated_count, int(a.seen), a.bias)
                                  for a in adjustments)
    packed_jobs = b"".join(_JOB_FORMAT.pack(*job) for job in jobs)
    at_adjustments = len(packed_rows)
    at_jobs = (at_adjustments + len(packed_adjustments) + 15) // 16 * 16
    blob = bytes(packed_rows) + packed_adjustments + bytes(at_jobs - at_adjustments - len(packed_adjustments)) + packed_jobs
    host = torch.frombuffer(bytearray(blob), dtype=torch.uint8).pin_memory()
    uploaded = host.to(device, non_blocking=True)
    base = uploaded.data_ptr()

    ids = torch.empty(results, dtype=torch.int32, device=device)
    logprobs = torch.zeros(results, dtype=torch.float32, device=device) if phases & _PHASE_REPORT else None
    weights = _sample_buffer(device, "weights", R * V, torch.float32) if phases else None
    sort_keys = _sample_buffer(device, "sort_keys", 2 * len(jobs) * V, torch.int32) if jobs else None
    sort_idx = _sample_buffer(device, "sort_idx", 2 * len(jobs) * V, torch.int32) if jobs else None
    job_state = _sample_buffer(device, "job_state", 4 * len(jobs), torch.int32) if jobs else None
    _check(library().zb_sample(
        _ptr(ids), _ptr(logprobs), _ptr(logits), logits.stride(0), R, V, base,
        base + at_adjustments if adjustments else None, len(adjustments), base + at_jobs if jobs else None, len(jobs),
        phases, _ptr(part_f), _ptr(part_i), _ptr(counters), _ptr(row_max), _ptr(row_arg), _ptr(weights),
        _ptr(sort_keys), _ptr(sort_idx), _ptr(job_state), _ptr(status), _stream()),
        "sample", kernels=1 + bool(adjustments) + 3 * bool(jobs) + bin(phases).count("1"))
    _sample_buffers[(device, "jobs_of_last_call")] = len(jobs)
    return SampleOutput(ids, logprobs, offsets)


def last_sample_job_state(device: torch.device | str | None = None) -> list[tuple[int, bool]]:
    """For every ranking of the last ``sample_rows`` call on ``device``, in the order of the rows (a
    row's draw before its report): how many ranks were sorted, and whether the head of the order was
    enough.  Reads from the device; for tests and timing."""
    device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    count = _sample_buffers.get((device, "jobs_of_last_call"), 0)
    if not count:
        return []
    state = _sample_buffers[(device, "job_state")][:4 * count].cpu().view(count, 4).tolist()
    return [(int(n), bool(done)) for n, done, _, _ in state]


def sample(logits: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """The argmax of every row of float32 logits, the lowest index among equal maxima."""
    return sample_rows(logits, None, status).ids
