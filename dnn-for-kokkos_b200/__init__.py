"""Host-side mirror of the reference's quantized-decode operators on top of the
C ABI of ``libkdnn_b200.so`` (include/kdnn_b200.h).

Names, argument meaning and error behaviour follow the reference's C++ operators
(``KokkosDNN::Gguf::quant_gemv``, ``quant_gemm``, ``quant_moe_decode``,
``make_quant_weight_table``, ``KokkosDNN::moe_route`` ...), with torch CUDA
tensors standing in for ``Kokkos::View`` and ``torch.cuda.current_stream()`` for
the execution-space instance. torch is plumbing only (device memory, streams);
every computation happens in the library's own CUDA kernels. There is no CPU or
library fallback: a missing ``libkdnn_b200.so`` raises at import.

The directory name has a hyphen, so import it through ``__graft_entry__.load_package()``
(which registers it as ``dnn_for_kokkos_b200``).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from . import ggml_pack  # noqa: F401  (re-exported: encoders for synthetic weights)
from .ggml_pack import Q4_K, Q5_K, Q6_K, Q8_0, row_bytes as ggml_row_bytes  # noqa: F401
from . import gguf_io  # noqa: F401
from .gguf_io import GgufFile, GgufTensorInfo, write_gguf  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkdnn_b200.so")

KDNN_OK, KDNN_DECLINED = 0, 1
KDNN_ERR_INVALID, KDNN_ERR_UNSUPPORTED, KDNN_ERR_CUDA, KDNN_ERR_DEVICE_WAIT = -1, -2, -3, -4
F32, BF16 = 0, 1

# every symbol include/kdnn_b200.h declares (checked by the CPU test-suite)
EXPORTS = [
    "kdnn_b200_last_error", "kdnn_b200_device_status", "kdnn_b200_gemv_scratch_bytes",
    "kdnn_b200_gemv_supported", "kdnn_b200_quant_gemv", "kdnn_b200_quant_gemv_ex", "kdnn_b200_quant_gemv_multi", "kdnn_b200_launch_chaining", "kdnn_b200_host_copy_by_kernel", "kdnn_b200_quant_gemv_noalloc",
    "kdnn_b200_quant_gemv_noalloc_ex", "kdnn_b200_quantize_act_q8", "kdnn_b200_quant_gemm_dots", "kdnn_b200_tile_kind",
    "kdnn_b200_weight_table_tma_bytes", "kdnn_b200_weight_table_tma_encode",
    "kdnn_b200_moe_exchange_bytes", "kdnn_b200_moe_block_workspace_bytes", "kdnn_b200_moe_block",
    "kdnn_b200_moe_block_routing", "kdnn_b200_peer_alloc", "kdnn_b200_peer_open", "kdnn_b200_peer_close",
    "kdnn_b200_peer_free", "kdnn_b200_swiglu", "kdnn_b200_moe_expert_weighted_sum", "kdnn_b200_moe_gather_rows",
    "kdnn_b200_moe_scatter_add_weighted", "kdnn_b200_read_probe",
    "kdnn_b200_unit_dots", "kdnn_b200_gemm_workspace_bytes", "kdnn_b200_quant_gemm",
    "kdnn_b200_moe_route", "kdnn_b200_moe_workspace_bytes", "kdnn_b200_moe_ffn",
    "kdnn_b200_residual_rmsnorm", "kdnn_b200_dequant_to_dense", "kdnn_b200_quant_gemv_fp",
    "kdnn_b200_quant_gemv_host",
]


class Declined(RuntimeError):
    """The int8 fast path does not cover this call and launched nothing (the
    reference would now run its own portable kernel)."""


class WeightTableC(C.Structure):
    _fields_ = [("base", C.c_void_p), ("ggml_type", C.c_uint32), ("rows", C.c_size_t),
                ("cols", C.c_size_t), ("row_bytes", C.c_size_t), ("n_experts", C.c_size_t),
                ("tma", C.c_void_p)]


class GemvLayoutC(C.Structure):
    """kdnn_b200_gemv_layout: optional tuning of one GEMV call (all zero = defaults)."""
    _fields_ = [("kernel", C.c_int), ("rows_per_group", C.c_int), ("stages", C.c_int),
                ("early_stages", C.c_int), ("warps", C.c_int), ("no_pdl", C.c_int)]


class MoeExchangeC(C.Structure):
    _fields_ = [("rank", C.c_int), ("world", C.c_int), ("regions", C.POINTER(C.c_void_p)),
                ("wait_ns", C.c_ulonglong)]


KERNEL_AUTO, KERNEL_XREG, KERNEL_SMEM_WINDOW, KERNEL_ITEM_STREAM, KERNEL_PLAIN_LOADS = 0, 1, 2, 3, 4
TILE_DP4A, TILE_MMA_SYNC, TILE_TCGEN05, TILE_AUTO = 0, 1, 2, 3


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
            "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    lib.kdnn_b200_last_error.restype = C.c_char_p
    lib.kdnn_b200_gemv_scratch_bytes.restype = C.c_size_t
    lib.kdnn_b200_gemv_scratch_bytes.argtypes = [C.c_size_t]
    lib.kdnn_b200_gemv_supported.argtypes = [C.c_uint32, C.c_size_t, C.c_int]
    lib.kdnn_b200_quant_gemv.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                         C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.kdnn_b200_quant_gemv_multi.argtypes = [C.c_uint32, C.c_size_t, C.POINTER(C.c_void_p), C.c_size_t, C.c_size_t,
                                               C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_void_p,
                                               C.c_size_t, C.c_void_p, C.c_void_p]
    lib.kdnn_b200_quant_gemv_ex.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                            C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t,
                                            C.POINTER(GemvLayoutC), C.c_void_p]
    lib.kdnn_b200_quant_gemv_noalloc.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                                 C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    lib.kdnn_b200_quant_gemv_noalloc_ex.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                                    C.c_int, C.c_void_p, C.c_int, C.POINTER(GemvLayoutC), C.c_void_p]
    lib.kdnn_b200_quant_gemm_dots.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                              C.c_size_t, C.c_size_t, C.c_int, C.c_void_p, C.c_size_t, C.c_int,
                                              C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.kdnn_b200_tile_kind.argtypes = [C.c_int]
    lib.kdnn_b200_weight_table_tma_bytes.restype = C.c_size_t
    lib.kdnn_b200_weight_table_tma_bytes.argtypes = [C.c_size_t]
    lib.kdnn_b200_weight_table_tma_encode.argtypes = [C.c_void_p, C.c_uint32, C.c_size_t, C.c_size_t, C.c_size_t,
                                                      C.c_void_p]
    lib.kdnn_b200_quant_gemv_host.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_int,
                                              C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                              C.c_void_p]
    lib.kdnn_b200_quantize_act_q8.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p, C.c_size_t,
                                              C.c_void_p]
    lib.kdnn_b200_unit_dots.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                        C.c_void_p, C.c_void_p]
    lib.kdnn_b200_gemm_workspace_bytes.restype = C.c_size_t
    lib.kdnn_b200_gemm_workspace_bytes.argtypes = [C.c_size_t, C.c_size_t]
    lib.kdnn_b200_quant_gemm.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                         C.c_size_t, C.c_size_t, C.c_int, C.c_void_p, C.c_size_t, C.c_int,
                                         C.c_void_p, C.c_size_t, C.c_void_p]
    lib.kdnn_b200_moe_route.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int,
                                        C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p,
                                        C.c_void_p, C.c_void_p]
    lib.kdnn_b200_moe_workspace_bytes.restype = C.c_size_t
    lib.kdnn_b200_moe_workspace_bytes.argtypes = [C.c_size_t] * 5
    lib.kdnn_b200_moe_ffn.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_int,
                                      C.POINTER(WeightTableC), C.POINTER(WeightTableC),
                                      C.POINTER(WeightTableC), C.c_void_p, C.c_void_p, C.c_size_t,
                                      C.c_void_p, C.c_size_t, C.c_int, C.c_size_t, C.c_size_t,
                                      C.c_void_p, C.c_size_t, C.c_void_p]
    lib.kdnn_b200_quant_gemv_fp.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_int,
                                            C.c_void_p, C.c_int, C.c_void_p]
    lib.kdnn_b200_dequant_to_dense.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                               C.c_size_t, C.c_int, C.c_void_p]
    lib.kdnn_b200_moe_exchange_bytes.restype = C.c_size_t
    lib.kdnn_b200_moe_exchange_bytes.argtypes = [C.c_size_t] * 4
    lib.kdnn_b200_moe_block_workspace_bytes.restype = C.c_size_t
    lib.kdnn_b200_moe_block_workspace_bytes.argtypes = [C.c_size_t] * 6 + [C.c_int]
    lib.kdnn_b200_moe_block.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p,
                                        C.c_int, C.c_int, C.c_float, C.c_int, C.POINTER(WeightTableC),
                                        C.POINTER(WeightTableC), C.POINTER(WeightTableC), C.c_size_t, C.c_size_t,
                                        C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t,
                                        C.c_void_p, C.c_size_t, C.c_float, C.POINTER(MoeExchangeC), C.c_void_p,
                                        C.c_size_t, C.c_void_p]
    lib.kdnn_b200_moe_block_routing.argtypes = [C.POINTER(MoeExchangeC), C.c_void_p] + [C.c_size_t] * 6 + \
        [C.c_void_p, C.c_void_p, C.c_void_p]
    lib.kdnn_b200_peer_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]
    lib.kdnn_b200_peer_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    lib.kdnn_b200_peer_close.argtypes = [C.c_void_p]
    lib.kdnn_b200_peer_free.argtypes = [C.c_void_p]
    lib.kdnn_b200_swiglu.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t,
                                     C.c_size_t, C.c_int, C.c_void_p]
    lib.kdnn_b200_moe_expert_weighted_sum.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t,
                                                      C.c_size_t, C.c_size_t, C.c_int, C.c_void_p]
    lib.kdnn_b200_moe_gather_rows.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t,
                                              C.c_size_t, C.c_size_t, C.c_int, C.c_void_p]
    lib.kdnn_b200_moe_scatter_add_weighted.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p,
                                                       C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_void_p]
    lib.kdnn_b200_read_probe.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    lib.kdnn_b200_residual_rmsnorm.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p,
                                               C.c_size_t, C.c_size_t, C.c_size_t, C.c_float, C.c_int, C.c_void_p]
    return lib


lib = _load()


def last_error() -> str:
    return lib.kdnn_b200_last_error().decode()


def device_status() -> int:
    return int(lib.kdnn_b200_device_status())


def _check(rc: int, what: str) -> None:
    if rc == KDNN_OK:
        return
    if rc == KDNN_DECLINED:
        raise Declined(f"{what}: declined by the int8 fast path")
    if rc == KDNN_ERR_INVALID:
        raise ValueError(last_error())          # std::invalid_argument in the reference
    raise RuntimeError(f"{what}: {last_error()} (status {rc})")


def _scalar(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise ValueError(f"Scalar must be float32 or bfloat16, got {t.dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{what} must live on the CUDA device")


# ---------------------------------------------------------------------------
@dataclass
class QuantWeight:
    """Packed rows in ggml block order on the device
    (Gguf::QuantWeight, src/KokkosDNN_GGUF.hpp:851-860)."""
    data: torch.Tensor   # uint8 [rows * row_bytes]
    dtype: int           # ggml type id
    rows: int
    cols: int

    def row_bytes(self) -> int:
        return ggml_row_bytes(self.dtype, self.cols)

    def bytes(self) -> int:
        return self.rows * self.row_bytes()

    @staticmethod
    def from_numpy(packed, dtype: int, rows: int, cols: int, device="cuda") -> "QuantWeight":
        t = torch.from_numpy(packed.reshape(-1)).to(device)
        if t.is_cuda:   # weights are complete before any kernel that may request them ahead of its dependency
            torch.cuda.current_stream(t.device).synchronize()
        return QuantWeight(t, dtype, rows, cols)


def load_quant_weight(file: GgufFile, info: GgufTensorInfo, device="cuda") -> QuantWeight:
    """Gguf::load_quant_weight (src/KokkosDNN_GGUF.hpp:864-885)."""
    import sys
    return gguf_io.load_quant_weight(sys.modules[__name__], file, info, device)


def load_expert_weights(file: GgufFile, info: GgufTensorInfo, device="cuda") -> List[QuantWeight]:
    """Every expert of a stacked {cols, rows, experts} tensor; feed the list to make_quant_weight_table."""
    import sys
    return gguf_io.load_expert_weights(sys.modules[__name__], file, info, device)


def tensor_to_float(file: GgufFile, info: GgufTensorInfo, device="cuda") -> torch.Tensor:
    """Gguf::dequant_tensor_to_float (src/KokkosDNN_GGUF.hpp:778-846): any tensor of the file as fp32."""
    import sys
    return gguf_io.tensor_to_float(sys.modules[__name__], file, info, device)


def _quant_check(w: QuantWeight, what: str) -> None:
    # Impl::quant_check, src/KokkosDNN_GGUF.hpp:1993-2006
    if w.dtype not in (Q8_0, Q4_K, Q5_K, Q6_K):
        raise ValueError(f"{what}: unsupported dtype {w.dtype}")
    want = w.rows * ggml_row_bytes(w.dtype, w.cols)    # raises ValueError on a ragged K
    if w.data.numel() != want:
        raise ValueError(f"{what}: payload size {w.data.numel()} != {want}")


def quant_gemv_int8_scratch_bytes(K: int) -> int:
    return int(lib.kdnn_b200_gemv_scratch_bytes(K))


def quant_gemv_int8_supported(dtype: int, K: int, scalar: torch.dtype = torch.float32) -> bool:
    s = F32 if scalar == torch.float32 else BF16 if scalar == torch.bfloat16 else -1
    return bool(lib.kdnn_b200_gemv_supported(dtype, K, s))


def tile_kind(kind: int = -1) -> int:
    """Selects the kernel of the batched Q4_K calls (TILE_AUTO default = by measured crossover, TILE_TCGEN05,
    TILE_MMA_SYNC, TILE_DP4A); returns the previous selection. A negative kind only queries."""
    return int(lib.kdnn_b200_tile_kind(kind))


def _layout(layout):
    if layout is None:
        return None
    if isinstance(layout, GemvLayoutC):
        return C.byref(layout)
    return C.byref(GemvLayoutC(**layout))


def quant_gemv(x: torch.Tensor, w: QuantWeight, y: torch.Tensor, act_scratch: torch.Tensor, layout=None) -> None:
    """y[N] = W[N,K] x[K] on the int8 path (Gguf::quant_gemv(handle, x, w, y,
    act_scratch), src/KokkosDNN_GGUF.hpp:2531-2551). Raises ValueError where the
    reference throws std::invalid_argument and Declined where its launcher returns
    false. `layout`: optional tuning (a GemvLayoutC or a dict of its fields), the counterpart of
    Impl::GgufMvq::Int8Layout."""
    if x.numel() != w.cols or y.numel() != w.rows:
        raise ValueError("quant_gemv: dimension mismatch")
    _quant_check(w, "quant_gemv")
    if w.rows == 0 or w.cols == 0:
        return
    for t, n in ((x, "x"), (y, "y"), (w.data, "w"), (act_scratch, "act_scratch")):
        _cuda(t, n)
    if x.stride(0) != 1 or y.stride(0) != 1:
        raise Declined("quant_gemv: non-unit stride")
    rc = lib.kdnn_b200_quant_gemv_ex(w.dtype, w.data.data_ptr(), w.rows, w.cols, x.data_ptr(), _scalar(x),
                                     y.data_ptr(), _scalar(y), act_scratch.data_ptr(), act_scratch.numel(),
                                     _layout(layout), _stream())
    _check(rc, "quant_gemv")


def host_copy_by_kernel(on: int = -1) -> int:
    """kdnn_b200_host_copy_by_kernel: 1 = kernels move page-locked host buffers of quant_gemv_host (default),
    0 = the copy engine; returns the previous setting, a negative argument only queries."""
    return int(lib.kdnn_b200_host_copy_by_kernel(int(on)))


def launch_chaining(on: int = -1) -> int:
    """Switches programmatic dependent launch of the library's kernels (kdnn_b200_launch_chaining); returns the
    previous setting, a negative argument only queries."""
    return int(lib.kdnn_b200_launch_chaining(int(on)))


def quant_gemv_multi(x: torch.Tensor, ws: Sequence[QuantWeight], ys: Sequence[torch.Tensor], act_scratch: torch.Tensor,
                     layout=None) -> None:
    """ys[i] = ws[i] . x for matrices of one format and shape that share the activation row
    (kdnn_b200_quant_gemv_multi): what a decoder does for wgate / wup or wk / wv, taken together so that
    Q4_K rows of up to 4096 elements run up to four matrices per launch. Same results as quant_gemv per matrix."""
    if len(ws) != len(ys):
        raise ValueError("quant_gemv_multi: as many outputs as matrices")
    if not ws:
        return
    w0 = ws[0]
    for w, y in zip(ws, ys):
        if (w.dtype, w.rows, w.cols) != (w0.dtype, w0.rows, w0.cols):
            raise ValueError("quant_gemv_multi: matrices of one format and shape")
        if x.numel() != w.cols or y.numel() != w.rows:
            raise ValueError("quant_gemv_multi: dimension mismatch")
        _quant_check(w, "quant_gemv_multi")
        _cuda(y, "y"); _cuda(w.data, "w")
        if y.stride(0) != 1 or _scalar(y) != _scalar(ys[0]):
            raise Declined("quant_gemv_multi: outputs of one scalar type with unit stride")
    _cuda(x, "x"); _cuda(act_scratch, "act_scratch")
    if w0.rows == 0 or w0.cols == 0:
        return
    if x.stride(0) != 1:
        raise Declined("quant_gemv_multi: non-unit stride")
    n = len(ws)
    wp = (C.c_void_p * n)(*[w.data.data_ptr() for w in ws])
    yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    rc = lib.kdnn_b200_quant_gemv_multi(w0.dtype, n, wp, w0.rows, w0.cols, x.data_ptr(), _scalar(x), yp, _scalar(ys[0]),
                                        act_scratch.data_ptr(), act_scratch.numel(), _layout(layout), _stream())
    _check(rc, "quant_gemv_multi")


def quant_gemv_host(x_host: torch.Tensor, w: QuantWeight, y_host: torch.Tensor, x_dev: torch.Tensor,
                    y_dev: torch.Tensor, act_scratch: torch.Tensor) -> None:
    """quant_gemv with the activations and the result in host memory (pinned for the copies to be
    asynchronous): copy in, GEMV, copy out, all enqueued by one call of kdnn_b200_quant_gemv_host on the
    current stream. y_host is valid after the stream has been synchronised."""
    if x_host.numel() != w.cols or y_host.numel() != w.rows or x_dev.numel() != w.cols or y_dev.numel() != w.rows:
        raise ValueError("quant_gemv: dimension mismatch")
    _quant_check(w, "quant_gemv")
    if w.rows == 0 or w.cols == 0:
        return
    if x_host.is_cuda or y_host.is_cuda:
        raise ValueError("quant_gemv_host: x_host / y_host must be host tensors")
    if x_host.dtype != x_dev.dtype or y_host.dtype != y_dev.dtype:
        raise ValueError("quant_gemv_host: host and device buffers must share a dtype")
    for t, n in ((x_dev, "x_dev"), (y_dev, "y_dev"), (w.data, "w"), (act_scratch, "act_scratch")):
        _cuda(t, n)
    if not (x_host.is_contiguous() and y_host.is_contiguous() and x_dev.is_contiguous() and y_dev.is_contiguous()):
        raise Declined("quant_gemv_host: non-unit stride")
    rc = lib.kdnn_b200_quant_gemv_host(w.dtype, w.data.data_ptr(), w.rows, w.cols, x_host.data_ptr(), _scalar(x_dev),
                                       y_host.data_ptr(), _scalar(y_dev), x_dev.data_ptr(), y_dev.data_ptr(),
                                       act_scratch.data_ptr(), act_scratch.numel(), _stream())
    _check(rc, "quant_gemv_host")


NOALLOC_MAX_COLS = 32768


def quant_gemv_noalloc(x: torch.Tensor, w: QuantWeight, y: torch.Tensor, layout=None) -> None:
    """quant_gemv without a caller-owned staging buffer: for hosts that may not allocate device memory
    (see kdnn_b200_quant_gemv_noalloc). K is limited to NOALLOC_MAX_COLS; calls that overlap on the GPU
    race on the shared built-in staging."""
    if x.numel() != w.cols or y.numel() != w.rows:
        raise ValueError("quant_gemv: dimension mismatch")
    _quant_check(w, "quant_gemv")
    if w.rows == 0 or w.cols == 0:
        return
    for t, n in ((x, "x"), (y, "y"), (w.data, "w")):
        _cuda(t, n)
    if x.stride(0) != 1 or y.stride(0) != 1:
        raise Declined("quant_gemv_noalloc: non-unit stride")
    rc = lib.kdnn_b200_quant_gemv_noalloc_ex(w.dtype, w.data.data_ptr(), w.rows, w.cols, x.data_ptr(), _scalar(x),
                                             y.data_ptr(), _scalar(y), _layout(layout), _stream())
    _check(rc, "quant_gemv_noalloc")


def quantize_act_q8(x: torch.Tensor, scratch: torch.Tensor) -> None:
    rc = lib.kdnn_b200_quantize_act_q8(x.data_ptr(), _scalar(x), x.numel(), scratch.data_ptr(),
                                       scratch.numel(), _stream())
    _check(rc, "quantize_act_q8")


def unit_dots(w: QuantWeight, staged_scratch: torch.Tensor) -> torch.Tensor:
    out = torch.empty((w.rows, w.cols // 32, 2), dtype=torch.int32, device=w.data.device)
    rc = lib.kdnn_b200_unit_dots(w.dtype, w.data.data_ptr(), w.rows, w.cols, staged_scratch.data_ptr(),
                                 out.data_ptr(), _stream())
    _check(rc, "unit_dots")
    return out


def quant_gemm_workspace_bytes(M: int, K: int) -> int:
    return int(lib.kdnn_b200_gemm_workspace_bytes(M, K))


def quant_gemm(X: torch.Tensor, w: QuantWeight, Y: torch.Tensor, workspace: torch.Tensor) -> None:
    """Y[M,N] = X[M,K] W[N,K]^T, int8 activations per row
    (Gguf::quant_gemm, src/KokkosDNN_GGUF.hpp:2564-2593)."""
    M, K = X.shape
    if w.cols != K or Y.shape[0] != M or Y.shape[1] != w.rows:
        raise ValueError("quant_gemm: dimension mismatch")
    _quant_check(w, "quant_gemm")
    if X.stride(1) != 1 or Y.stride(1) != 1:
        raise Declined("quant_gemm: non-unit inner stride")
    rc = lib.kdnn_b200_quant_gemm(w.dtype, w.data.data_ptr(), w.rows, K, X.data_ptr(), X.stride(0), M,
                                  _scalar(X), Y.data_ptr(), Y.stride(0), _scalar(Y),
                                  workspace.data_ptr(), workspace.numel(), _stream())
    _check(rc, "quant_gemm")


def quant_gemm_dots(X: torch.Tensor, w: QuantWeight, Y: torch.Tensor, workspace: torch.Tensor) -> torch.Tensor:
    """quant_gemm on the tcgen05 tile kernel, also returning the raw int32 sub-block dots [M, N, K/32] the
    tensor cores produced (parity probe, see kdnn_b200_quant_gemm_dots)."""
    M, K = X.shape
    if w.cols != K or Y.shape[0] != M or Y.shape[1] != w.rows:
        raise ValueError("quant_gemm: dimension mismatch")
    _quant_check(w, "quant_gemm")
    dots = torch.zeros((M, w.rows, K // 32), dtype=torch.int32, device=X.device)
    rc = lib.kdnn_b200_quant_gemm_dots(w.dtype, w.data.data_ptr(), w.rows, K, X.data_ptr(), X.stride(0), M,
                                       _scalar(X), Y.data_ptr(), Y.stride(0), _scalar(Y), dots.data_ptr(),
                                       workspace.data_ptr(), workspace.numel(), _stream())
    _check(rc, "quant_gemm_dots")
    return dots


def quant_gemv_fp(x: torch.Tensor, w: QuantWeight, y: torch.Tensor) -> None:
    """y[N] = W[N,K] x[K] on the fp path, no staging buffer (Gguf::quant_gemv(handle, x, w, y),
    src/KokkosDNN_GGUF.hpp:2394-2493)."""
    if x.numel() != w.cols or y.numel() != w.rows:
        raise ValueError("quant_gemv: dimension mismatch")
    _quant_check(w, "quant_gemv")
    if w.rows == 0 or w.cols == 0:
        return
    if x.stride(0) != 1 or y.stride(0) != 1:
        raise ValueError("quant_gemv: x and y must have unit stride")
    rc = lib.kdnn_b200_quant_gemv_fp(w.dtype, w.data.data_ptr(), w.rows, w.cols, x.data_ptr(), _scalar(x),
                                     y.data_ptr(), _scalar(y), _stream())
    _check(rc, "quant_gemv_fp")


def dequant_to_dense(w: QuantWeight, Y: torch.Tensor) -> None:
    """Y[rows, cols] = Scalar(dequant(W)) (Gguf::dequant_to_dense, src/KokkosDNN_GGUF.hpp:2839-2934)."""
    if tuple(Y.shape) != (w.rows, w.cols):
        raise ValueError("dequant_to_dense: dimension mismatch")
    _quant_check(w, "dequant_to_dense")
    if w.rows == 0 or w.cols == 0:
        return
    if Y.stride(1) != 1:
        raise ValueError("dequant_to_dense: Y must be LayoutRight")
    rc = lib.kdnn_b200_dequant_to_dense(w.dtype, w.data.data_ptr(), w.rows, w.cols, Y.data_ptr(), Y.stride(0),
                                        _scalar(Y), _stream())
    _check(rc, "dequant_to_dense")


def moe_route(logits: torch.Tensor, expert_bias: Optional[torch.Tensor], top_k: int, norm_topk: bool,
              routed_scale: float, top_idx: torch.Tensor, top_w: torch.Tensor,
              sigmoid: bool = False) -> None:
    """KokkosDNN::moe_route / moe_route_sigmoid (src/KokkosDNN_MoE.hpp:240-304)."""
    T, E = logits.shape
    K = max(top_k, 0)
    have_bias = expert_bias is not None and expert_bias.numel() != 0
    name = "moe_route_sigmoid" if sigmoid else "moe_route"
    if have_bias and expert_bias.numel() != E:
        raise ValueError(f"{name}: expert_bias extent must be E")
    if tuple(top_idx.shape) != (T, K) or tuple(top_w.shape) != (T, K):
        raise ValueError(f"{name}: output dimension mismatch")
    if T == 0:
        return
    if top_k <= 0 or K > E:
        raise ValueError(f"{name}: need 1 <= top_k <= E")
    if have_bias and expert_bias.dtype != logits.dtype:
        raise ValueError(f"{name}: bias and logits must share one Scalar")
    rc = lib.kdnn_b200_moe_route(logits.data_ptr(), logits.stride(0), T, E, _scalar(logits),
                                 expert_bias.data_ptr() if have_bias else None, top_k, int(norm_topk),
                                 float(routed_scale), int(sigmoid), top_idx.data_ptr(), top_w.data_ptr(),
                                 _stream())
    _check(rc, name)


@dataclass
class QuantWeightTable:
    """Device array of per-expert payload pointers plus the shared shape
    (Gguf::QuantWeightTable, src/KokkosDNN_GGUF.hpp:2020-2029)."""
    base: torch.Tensor   # int64 [n_experts] device addresses
    dtype: int
    rows: int
    cols: int
    row_bytes: int
    keepalive: Sequence[QuantWeight] = ()
    tma: Optional[torch.Tensor] = None   # uint8 [n_experts * 128] TMA descriptors for the tcgen05 tile kernel

    def __post_init__(self):
        if self.tma is None and self.base.numel() and self.base.is_cuda:
            self.tma = encode_table_tma(self.base, self.dtype, self.rows, self.cols)

    def size(self) -> int:
        return int(self.base.numel())

    def c_struct(self) -> WeightTableC:
        return WeightTableC(self.base.data_ptr(), self.dtype, self.rows, self.cols, self.row_bytes,
                            self.size(), self.tma.data_ptr() if self.tma is not None else None)


def encode_table_tma(base: torch.Tensor, dtype: int, rows: int, cols: int) -> Optional[torch.Tensor]:
    """One TMA descriptor per expert matrix (kdnn_b200_weight_table_tma_encode), uploaded next to the
    pointer table; None when the table's format has no tensor-core kernel."""
    import numpy as np
    host = np.ascontiguousarray(base.cpu().numpy().astype(np.uint64))
    out = np.zeros(host.size * 128, dtype=np.uint8)
    rc = lib.kdnn_b200_weight_table_tma_encode(host.ctypes.data, dtype, rows, cols, host.size, out.ctypes.data)
    if rc == KDNN_DECLINED:
        return None
    _check(rc, "weight_table_tma_encode")
    return torch.from_numpy(out).to(base.device)


def make_quant_weight_table(ws: List[QuantWeight], what: str = "table") -> QuantWeightTable:
    """Gguf::make_quant_weight_table (src/KokkosDNN_GGUF.hpp:2031-2053)."""
    if not ws:
        return QuantWeightTable(torch.empty(0, dtype=torch.int64), 0, 0, 0, 0)
    w0 = ws[0]
    for w in ws:
        if w.dtype != w0.dtype or w.rows != w0.rows or w.cols != w0.cols:
            raise ValueError(f"{what}: entries must share dtype and shape")
        _quant_check(w, what)
    base = torch.tensor([w.data.data_ptr() for w in ws], dtype=torch.int64, device=w0.data.device)
    return QuantWeightTable(base, w0.dtype, w0.rows, w0.cols, w0.row_bytes(), tuple(ws))


def moe_ffn_workspace_bytes(T: int, S: int, H: int, F: int, n_experts: int) -> int:
    return int(lib.kdnn_b200_moe_workspace_bytes(T, S, H, F, n_experts))


def moe_ffn(X: torch.Tensor, gate: QuantWeightTable, up: QuantWeightTable, down: QuantWeightTable,
            idx: torch.Tensor, wts: torch.Tensor, Y: torch.Tensor, workspace: torch.Tensor,
            expert_first: int = 0, expert_count: Optional[int] = None) -> None:
    """Batched expert feed-forward with int8 activations (see kdnn_b200_moe_ffn)."""
    T, H = X.shape
    S = idx.shape[1] if idx.dim() == 2 and idx.shape[0] else 0
    if tuple(Y.shape) != (T, H):
        raise ValueError("moe_ffn: dimension mismatch")
    if idx.shape[0] != T or tuple(wts.shape) != tuple(idx.shape):
        raise ValueError("moe_ffn: routing dimension mismatch")
    if idx.dtype != torch.int32 or wts.dtype != torch.float32:
        raise ValueError("moe_ffn: idx must be int32 and wts float32")
    if X.stride(1) != 1 or Y.stride(1) != 1 or not idx.is_contiguous() or not wts.is_contiguous():
        raise ValueError("moe_ffn: rows must be contiguous")
    g, u, d = gate.c_struct(), up.c_struct(), down.c_struct()
    n = gate.size() if expert_count is None else expert_count
    rc = lib.kdnn_b200_moe_ffn(X.data_ptr(), X.stride(0), T, _scalar(X), C.byref(g), C.byref(u),
                               C.byref(d), idx.data_ptr(), wts.data_ptr(), S, Y.data_ptr(), Y.stride(0),
                               _scalar(Y), expert_first, n, workspace.data_ptr(), workspace.numel(),
                               _stream())
    _check(rc, "moe_ffn")


def quant_moe_decode(X: torch.Tensor, gate: QuantWeightTable, up: QuantWeightTable,
                     down: QuantWeightTable, idx: torch.Tensor, wts: torch.Tensor, act: torch.Tensor,
                     Y: torch.Tensor, workspace: torch.Tensor) -> None:
    """One decoded token (Gguf::quant_moe_decode, src/KokkosDNN_GGUF.hpp:2335-2391):
    same argument checks and messages; `act` is accepted for signature parity (the
    kernels keep the activations in `workspace`)."""
    if X.shape[0] != 1 or Y.shape[0] != 1:
        raise ValueError("quant_moe_decode: expected one row")
    K, MI = X.shape[1], gate.rows
    S = 0 if idx.shape[0] == 0 else idx.shape[1]
    if gate.cols != K or up.cols != K or up.rows != MI or down.rows != K or down.cols != MI \
            or Y.shape[1] != K:
        raise ValueError("quant_moe_decode: dimension mismatch")
    if gate.size() == 0 or gate.size() != up.size() or gate.size() != down.size():
        raise ValueError("quant_moe_decode: expert table mismatch")
    if idx.shape[0] != 1 or wts.shape[0] != 1 or wts.shape[1] != S:
        raise ValueError("quant_moe_decode: routing dimension mismatch")
    if act.shape[0] < S or (S > 0 and act.shape[1] != MI):
        raise ValueError("quant_moe_decode: act scratch too small")
    if S == 0 or K == 0 or MI == 0:
        return
    moe_ffn(X, gate, up, down, idx, wts, Y, workspace)


def residual_rmsnorm(h: torch.Tensor, y: torch.Tensor, out: torch.Tensor, eps: float = 1e-6) -> None:
    """out = Scalar(rmsnorm_noscale(Scalar(h + y))) (see kdnn_b200_residual_rmsnorm)."""
    T, H = h.shape
    if tuple(y.shape) != (T, H) or tuple(out.shape) != (T, H) or y.dtype != torch.float32 or out.dtype != h.dtype:
        raise ValueError("residual_rmsnorm: dimension or dtype mismatch")
    rc = lib.kdnn_b200_residual_rmsnorm(h.data_ptr(), h.stride(0), y.data_ptr(), y.stride(0), out.data_ptr(),
                                        out.stride(0), T, H, float(eps), _scalar(h), _stream())
    _check(rc, "residual_rmsnorm")


# ---------------------------------------------------------------------------
# the reference's small MoE operators (src/KokkosDNN_SwiGLU.hpp, src/KokkosDNN_MoE.hpp:313-381)
def swiglu(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor) -> None:
    """out = Scalar(silu(gate) * up) (KokkosDNN::swiglu, src/KokkosDNN_SwiGLU.hpp:24-38)."""
    T, F = gate.shape
    if tuple(up.shape) != (T, F) or tuple(out.shape) != (T, F) or up.dtype != gate.dtype or out.dtype != gate.dtype:
        raise ValueError("swiglu: dimension mismatch")
    rc = lib.kdnn_b200_swiglu(gate.data_ptr(), gate.stride(0), up.data_ptr(), up.stride(0), out.data_ptr(),
                              out.stride(0), T, F, _scalar(gate), _stream())
    _check(rc, "swiglu")


def moe_expert_weighted_sum(expert_out: torch.Tensor, top_w: torch.Tensor, y: torch.Tensor) -> None:
    """y[t,d] = sum_k top_w[t,k] * expert_out[t,k,d] (KokkosDNN::moe_expert_weighted_sum, src/KokkosDNN_MoE.hpp:313-332)."""
    T, D = y.shape
    K = top_w.shape[1]
    if tuple(expert_out.shape) != (T, K, D) or top_w.shape[0] != T:
        raise ValueError("moe_expert_weighted_sum: dimension mismatch")
    if not expert_out.is_contiguous() or not top_w.is_contiguous() or top_w.dtype != torch.float32:
        raise ValueError("moe_expert_weighted_sum: expert_out / top_w must be contiguous, top_w float32")
    rc = lib.kdnn_b200_moe_expert_weighted_sum(expert_out.data_ptr(), top_w.data_ptr(), y.data_ptr(), y.stride(0), T, K,
                                               D, _scalar(y), _stream())
    _check(rc, "moe_expert_weighted_sum")


def moe_gather_rows(src: torch.Tensor, rows: torch.Tensor, dst: torch.Tensor) -> None:
    """dst[n,:] = src[rows[n],:] (KokkosDNN::moe_gather_rows, src/KokkosDNN_MoE.hpp:337-351)."""
    N = rows.shape[0]
    D = src.shape[1]
    if dst.shape[0] != N or (N > 0 and dst.shape[1] != D):
        raise ValueError("moe_gather_rows: dimension mismatch")
    if rows.dtype != torch.int32 or dst.dtype != src.dtype:
        raise ValueError("moe_gather_rows: rows must be int32, src and dst one Scalar")
    rc = lib.kdnn_b200_moe_gather_rows(src.data_ptr(), src.stride(0), src.shape[0], rows.data_ptr(), dst.data_ptr(),
                                       dst.stride(0) if N else D, N, D, _scalar(src), _stream())
    _check(rc, "moe_gather_rows")


def moe_scatter_add_weighted(src: torch.Tensor, rows: torch.Tensor, weights: torch.Tensor, dst: torch.Tensor) -> None:
    """dst[rows[n],:] += weights[n] * src[n,:], rows unique (KokkosDNN::moe_scatter_add_weighted, src/KokkosDNN_MoE.hpp:360-381)."""
    N = rows.shape[0]
    C_, D = dst.shape
    if src.shape[0] != N or weights.shape[0] != N or (N > 0 and src.shape[1] != D):
        raise ValueError("moe_scatter_add_weighted: dimension mismatch")
    if rows.dtype != torch.int32 or weights.dtype != torch.float32 or dst.dtype != src.dtype:
        raise ValueError("moe_scatter_add_weighted: rows int32, weights float32, src and dst one Scalar")
    rc = lib.kdnn_b200_moe_scatter_add_weighted(src.data_ptr(), src.stride(0) if N else D, rows.data_ptr(),
                                                weights.data_ptr(), dst.data_ptr(), dst.stride(0), C_, N, D,
                                                _scalar(dst), _stream())
    _check(rc, "moe_scatter_add_weighted")


# ---------------------------------------------------------------------------
# the MoE block in four launches, single GPU or expert-parallel over peer memory
class MoeExchange:
    """Exchange regions of an expert-parallel group: this rank's region (peer-visible device memory) and the
    peers' regions opened through IPC handles. ``handles`` is the list of every rank's 64-byte handle in rank
    order (what ``all_gather`` of ``local_handle`` gives); the single-process form (``MoeExchange.local``) maps
    plain device buffers and is what the tests use to stand in for peers that never answer."""

    def __init__(self, rank: int, world: int, regions: Sequence[int], wait_ns: int = 0, owner=None, ipc: bool = False):
        self.rank, self.world, self.regions, self.wait_ns, self._owner = rank, world, list(regions), wait_ns, owner
        self._arr = (C.c_void_p * world)(*self.regions)
        self.c = MoeExchangeC(rank, world, self._arr, wait_ns)
        self._ipc = ipc          # regions came from alloc() / open(): close() gives them back

    def close(self) -> None:
        """Closes the peers' mappings and frees this rank's region (only for regions made by alloc() / open()).
        Call it on every rank after a device synchronisation and a barrier: no peer may still be using them."""
        if not self._ipc:
            return
        self._ipc = False
        for r, ptr in enumerate(self.regions):
            if r == self.rank:
                _check(lib.kdnn_b200_peer_free(ptr), "peer_free")
            else:
                _check(lib.kdnn_b200_peer_close(ptr), "peer_close")

    @staticmethod
    def region_bytes(tokens_local: int, world: int, top_k: int, H: int) -> int:
        return int(lib.kdnn_b200_moe_exchange_bytes(tokens_local, world, top_k, H))

    @staticmethod
    def alloc(nbytes: int):
        """(device pointer, 64-byte IPC handle) of a zeroed peer-visible allocation."""
        ptr, handle = C.c_void_p(), (C.c_ubyte * 64)()
        _check(lib.kdnn_b200_peer_alloc(nbytes, C.byref(ptr), handle), "peer_alloc")
        return int(ptr.value), bytes(handle)

    @staticmethod
    def open(handle: bytes) -> int:
        ptr, buf = C.c_void_p(), (C.c_ubyte * 64).from_buffer_copy(handle)
        _check(lib.kdnn_b200_peer_open(buf, C.byref(ptr)), "peer_open")
        return int(ptr.value)

    @staticmethod
    def local(rank: int, world: int, buffers: Sequence[torch.Tensor], wait_ns: int = 0) -> "MoeExchange":
        return MoeExchange(rank, world, [b.data_ptr() for b in buffers], wait_ns, owner=tuple(buffers))


def moe_block_workspace_bytes(tokens_local: int, world: int, top_k: int, H: int, F: int, n_experts: int,
                              with_region: bool) -> int:
    return int(lib.kdnn_b200_moe_block_workspace_bytes(tokens_local, world, top_k, H, F, n_experts, int(with_region)))


def moe_block(x: torch.Tensor, router_w: torch.Tensor, router_bias: Optional[torch.Tensor], top_k: int, norm_topk: bool,
              routed_scale: float, gate: QuantWeightTable, up: QuantWeightTable, down: QuantWeightTable,
              workspace: torch.Tensor, y: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
              h_out: Optional[torch.Tensor] = None, xn_out: Optional[torch.Tensor] = None, eps: float = 1e-6,
              sigmoid: bool = False, expert_first: int = 0, expert_count: Optional[int] = None,
              exchange: Optional[MoeExchange] = None) -> None:
    """One MoE block for this rank's tokens (see kdnn_b200_moe_block): router logits, routing, expert
    feed-forward on the local experts, combine on the token owner, optional residual add + un-scaled RMS norm."""
    Tl, H = x.shape
    E = gate.size()
    if tuple(router_w.shape) != (E, H) or router_w.dtype != x.dtype:
        raise ValueError("moe_block: router_w must be [E, H] in the Scalar of x")
    have_bias = router_bias is not None and router_bias.numel() != 0
    if have_bias and (router_bias.numel() != E or router_bias.dtype != x.dtype):
        raise ValueError("moe_block: expert_bias extent must be E")
    for t, n in ((y, "y"), (resid, "resid"), (h_out, "h_out"), (xn_out, "xn_out")):
        if t is not None and tuple(t.shape) != (Tl, H):
            raise ValueError(f"moe_block: {n} must be [tokens_local, H]")
    if y is not None and y.dtype != torch.float32:
        raise ValueError("moe_block: y is float32")
    g, u, d = gate.c_struct(), up.c_struct(), down.c_struct()
    n = E if expert_count is None else expert_count
    ptr = lambda t: t.data_ptr() if t is not None else None
    ld = lambda t: t.stride(0) if t is not None else 0
    rc = lib.kdnn_b200_moe_block(x.data_ptr(), x.stride(0), Tl, _scalar(x), router_w.data_ptr(), router_w.stride(0),
                                 router_bias.data_ptr() if have_bias else None, top_k, int(norm_topk),
                                 float(routed_scale), int(sigmoid), C.byref(g), C.byref(u), C.byref(d), expert_first, n,
                                 ptr(y), ld(y), ptr(resid), ld(resid), ptr(h_out), ld(h_out), ptr(xn_out), ld(xn_out),
                                 float(eps), C.byref(exchange.c) if exchange is not None else None,
                                 workspace.data_ptr(), workspace.numel(), _stream())
    _check(rc, "moe_block")


def moe_block_routing(workspace: torch.Tensor, tokens_local: int, world: int, top_k: int, H: int, F: int, n_experts: int,
                      exchange: Optional[MoeExchange] = None):
    """(idx, wts) of ALL tokens from the last moe_block call, as device tensors [T, top_k]."""
    T = tokens_local * world
    idx = torch.empty((T, top_k), dtype=torch.int32, device=workspace.device)
    wts = torch.empty((T, top_k), dtype=torch.float32, device=workspace.device)
    _check(lib.kdnn_b200_moe_block_routing(C.byref(exchange.c) if exchange is not None else None, workspace.data_ptr(),
                                           tokens_local, world, top_k, H, F, n_experts, idx.data_ptr(), wts.data_ptr(),
                                           _stream()), "moe_block_routing")
    return idx, wts


def read_probe(buf: torch.Tensor, sink: torch.Tensor) -> None:
    """Streams `buf` once with read-only 128-bit loads (kdnn_b200_read_probe): the read-only bandwidth ceiling."""
    _check(lib.kdnn_b200_read_probe(buf.data_ptr(), buf.numel() * buf.element_size(), sink.data_ptr(), _stream()),
           "read_probe")
