"""ctypes/numpy front-end for the CPU checkers.

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline legs. The product package never imports it.

Two libraries:

* ``libkdnn_oracle.so``  -- ``kdnn_oracle.c``, the plain-C restatement (class
  :class:`Port`); always available once ``make -C oracle`` has run.
* ``_ref/libkdnn_ref.so`` -- the reference's own operators compiled from its
  header files through ``ref_shim.cpp`` (class :class:`Ref`); present when it
  was built on a machine that has the reference sources.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
Q8_0, Q4_K, Q5_K, Q6_K = 8, 12, 13, 14
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}
# dtype tag of the reference's int8 GEMV (src/KokkosDNN_GGUFGemvInt8.hpp:79)
WD = {Q4_K: 0, Q5_K: 1, Q6_K: 2, Q8_0: 3}


def row_bytes(dtype: int, cols: int) -> int:
    n, b = BLOCK[dtype]
    assert cols % n == 0
    return cols // n * b


def build(quiet: bool = True) -> None:
    """Run the oracle Makefile (compiles the port; compiles _ref when the
    reference sources are present)."""
    subprocess.run(["make", "-C", HERE], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _aligned(nbytes: int, align: int = 64) -> np.ndarray:
    raw = np.zeros(nbytes + align, dtype=np.uint8)
    off = (-raw.ctypes.data) % align
    return raw[off:off + nbytes]


def aligned_copy(a: np.ndarray) -> np.ndarray:
    """Copy of a byte array whose base address is 64-byte aligned."""
    out = _aligned(a.size)
    out[:] = a.reshape(-1).view(np.uint8)
    return out


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


class Port:
    """The plain-C restatement (kdnn_oracle.c)."""

    kind = "port"

    def __init__(self):
        path = os.path.join(HERE, "libkdnn_oracle.so")
        if not os.path.exists(path):
            build()
        self.lib = L = C.CDLL(path)
        L.ko_fp16_to_f32.restype = C.c_float
        L.ko_fp16_to_f32.argtypes = [C.c_uint16]
        L.ko_silu.restype = C.c_float
        L.ko_silu.argtypes = [C.c_float]
        L.ko_dot4.restype = C.c_int32
        L.ko_dot4.argtypes = [C.c_int32] * 3
        L.ko_act_q8_bytes.restype = C.c_size_t
        L.ko_act_q8_bytes.argtypes = [C.c_size_t]
        L.ko_row_bytes.restype = C.c_size_t
        L.ko_row_bytes.argtypes = [C.c_uint32, C.c_size_t]
        L.ko_num_threads.restype = C.c_int

    # -- scalars
    def fp16_to_f32(self, h: int) -> float:
        return float(self.lib.ko_fp16_to_f32(h))

    def scale_min_k4(self, j: int, scales: np.ndarray):
        sc, mn = C.c_uint8(), C.c_uint8()
        s = np.ascontiguousarray(scales, dtype=np.uint8)
        self.lib.ko_scale_min_k4(C.c_int(j), _ptr(s), C.byref(sc), C.byref(mn))
        return sc.value, mn.value

    def dot4(self, a: int, b: int, acc: int) -> int:
        return int(self.lib.ko_dot4(a, b, acc))

    def silu(self, v: float) -> float:
        return float(self.lib.ko_silu(v))

    def set_threads(self, n: int):
        self.lib.ko_set_num_threads(C.c_int(n))

    def threads(self) -> int:
        return int(self.lib.ko_num_threads())

    # -- staging
    def act_bytes(self, K: int) -> int:
        return int(self.lib.ko_act_q8_bytes(K))

    def quantize_act(self, x: np.ndarray) -> np.ndarray:
        """x: fp32 values of the Scalar activations. Returns the staging bytes."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        K = x.size
        s = _aligned(self.act_bytes(K))
        self.lib.ko_quantize_act_q8(_ptr(x), C.c_size_t(K), _ptr(s))
        return s

    def dequant_act(self, scratch: np.ndarray, K: int) -> np.ndarray:
        out = np.empty(K, dtype=np.float32)
        self.lib.ko_dequant_act(_ptr(scratch), C.c_size_t(K), _ptr(out))
        return out

    def unit_window(self, dtype, scratch, K, c):
        w = np.empty(10, dtype=np.int32)
        d = np.empty(2, dtype=np.float32)
        self.lib.ko_unit_window(C.c_uint32(dtype), _ptr(scratch), C.c_size_t(K),
                                C.c_int(c), _ptr(w), _ptr(d))
        return w, d

    def unit_table(self, dtype, w, rows, cols, scratch):
        nu = cols // 32
        ints = np.empty((rows, nu, 2), dtype=np.int32)
        vals = np.empty((rows, nu), dtype=np.float32)
        self.lib.ko_unit_table(C.c_uint32(dtype), _ptr(w), C.c_size_t(rows),
                               C.c_size_t(cols), _ptr(scratch), _ptr(ints), _ptr(vals))
        return ints, vals

    # -- GEMV
    def gemv_int8(self, dtype, w, rows, cols, x):
        """Returns (y fp32 before the Scalar cast, staging bytes)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        s = _aligned(self.act_bytes(cols))
        y = np.empty(rows, dtype=np.float32)
        rc = self.lib.ko_gemv_int8(C.c_uint32(dtype), _ptr(w), C.c_size_t(rows),
                                   C.c_size_t(cols), _ptr(x), _ptr(y), _ptr(s))
        assert rc == 0
        return y, s

    def gemv_int8_staged(self, dtype, w, rows, cols, scratch):
        y = np.empty(rows, dtype=np.float32)
        self.lib.ko_gemv_int8_staged(C.c_uint32(dtype), _ptr(w), C.c_size_t(rows),
                                     C.c_size_t(cols), _ptr(scratch), _ptr(y))
        return y

    def dequant_rows(self, dtype, w, rows, cols):
        rb = row_bytes(dtype, cols)
        out = np.empty((rows, cols), dtype=np.float32)
        for r in range(rows):
            rc = self.lib.ko_dequant_row(C.c_uint32(dtype), C.c_void_p(w.ctypes.data + r * rb),
                                         C.c_size_t(cols), C.c_void_p(out.ctypes.data + r * cols * 4))
            assert rc == 0
        return out

    def gemv_dequant_f64(self, dtype, w, rows, cols, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(rows, dtype=np.float64)
        mag = np.empty(rows, dtype=np.float64)
        rc = self.lib.ko_gemv_dequant_f64(C.c_uint32(dtype), _ptr(w), C.c_size_t(rows),
                                          C.c_size_t(cols), _ptr(x), _ptr(y), _ptr(mag))
        assert rc == 0
        return y, mag

    # -- MoE
    def moe_route(self, logits, bias, top_k, norm_topk, routed_scale=1.0, sigmoid=False):
        lg = np.ascontiguousarray(logits, dtype=np.float32)
        T, E = lg.shape
        b = None if bias is None or len(bias) == 0 else np.ascontiguousarray(bias, dtype=np.float32)
        idx = np.empty((T, top_k), dtype=np.int32)
        w = np.empty((T, top_k), dtype=np.float32)
        rc = self.lib.ko_moe_route(_ptr(lg), C.c_size_t(T), C.c_size_t(E), _ptr(b),
                                   C.c_int(top_k), C.c_int(int(norm_topk)),
                                   C.c_float(routed_scale), C.c_int(int(sigmoid)),
                                   _ptr(idx), _ptr(w))
        if rc != 0:
            raise ValueError("moe_route: need 1 <= top_k <= E")
        return idx, w

    def moe_ffn_int8(self, X, gate, up, down, idx, wts, F, dtypes=(Q4_K, Q4_K, Q4_K),
                     bf16=True, want_act=False):
        """gate/up/down: lists of per-expert packed byte arrays."""
        X = np.ascontiguousarray(X, dtype=np.float32)
        T, H = X.shape
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        wts = np.ascontiguousarray(wts, dtype=np.float32)
        S = idx.shape[1]
        E = len(gate)
        arr = lambda lst: (C.c_void_p * E)(*[a.ctypes.data for a in lst])
        Y = np.empty((T, H), dtype=np.float32)
        act = np.empty((T, S, F), dtype=np.float32) if want_act else None
        rc = self.lib.ko_moe_ffn_int8(_ptr(X), C.c_size_t(T), C.c_size_t(H), C.c_size_t(F),
                                      C.c_size_t(E), C.c_uint32(dtypes[0]), C.c_uint32(dtypes[1]),
                                      C.c_uint32(dtypes[2]), arr(gate), arr(up), arr(down),
                                      _ptr(idx), _ptr(wts), C.c_size_t(S), C.c_int(int(bf16)),
                                      _ptr(Y), _ptr(act))
        assert rc == 0
        return (Y, act) if want_act else Y


class Ref:
    """The reference's own operators (oracle/_ref/libkdnn_ref.so)."""

    kind = "reference"

    @staticmethod
    def available() -> bool:
        return os.path.exists(os.path.join(HERE, "_ref", "libkdnn_ref.so"))

    def __init__(self):
        self.lib = L = C.CDLL(os.path.join(HERE, "_ref", "libkdnn_ref.so"))
        L.kref_last_error.restype = C.c_char_p
        L.kref_int8_scratch_bytes.restype = C.c_size_t
        L.kref_int8_scratch_bytes.argtypes = [C.c_size_t]
        L.kref_row_bytes.restype = C.c_size_t
        L.kref_row_bytes.argtypes = [C.c_uint32, C.c_size_t]
        L.kref_dot4.restype = C.c_int32
        L.kref_dot4.argtypes = [C.c_int32] * 3
        L.kref_silu.restype = C.c_float
        L.kref_silu.argtypes = [C.c_float]
        L.kref_fp16_to_float.restype = C.c_float
        L.kref_fp16_to_float.argtypes = [C.c_uint16]
        L.kref_num_threads.restype = C.c_int

    def _check(self, rc):
        if rc == -1:
            raise ValueError(self.lib.kref_last_error().decode())
        if rc != 0:
            raise RuntimeError(self.lib.kref_last_error().decode())

    # ---- GGUF container: the reference's own writer and reader ------------------------
    def gguf_write(self, path, tensors, strings=None, f32=None, u32=None):
        """tensors: (name, dims in ggml order, ggml type id, uint8 payload). Written by the reference's
        write_synthetic_gguf."""
        n = len(tensors)
        names = (C.c_char_p * n)(*[t[0].encode() for t in tensors])
        dtypes = (C.c_uint32 * n)(*[t[2] for t in tensors])
        ndims = (C.c_uint32 * n)(*[len(t[1]) for t in tensors])
        dims = (C.c_uint64 * (4 * n))()
        raws = [np.ascontiguousarray(t[3]).view(np.uint8).reshape(-1) for t in tensors]
        for i, t in enumerate(tensors):
            for d, v in enumerate(t[1]):
                dims[4 * i + d] = v
        ptrs = (C.c_void_p * n)(*[r.ctypes.data for r in raws])
        sizes = (C.c_size_t * n)(*[r.size for r in raws])

        def kv(m, ctype):
            m = m or {}
            keys = (C.c_char_p * len(m))(*[k.encode() for k in m])
            vals = (ctype * len(m))(*[v.encode() if ctype is C.c_char_p else v for v in m.values()])
            return C.c_size_t(len(m)), keys, vals
        self._check(self.lib.kref_gguf_write(path.encode(), C.c_size_t(n), names, dtypes, ndims, dims, ptrs, sizes,
                                             *kv(strings, C.c_char_p), *kv(f32, C.c_float), *kv(u32, C.c_uint32)))

    def gguf_read_tensor(self, path, name, cap=1 << 24):
        """The reference's GgufFile on `path`: (dtype, dims, offset, nbytes, data_start, payload)."""
        out = (C.c_uint64 * 8)()
        start = C.c_uint64()
        buf = np.zeros(cap, dtype=np.uint8)
        self._check(self.lib.kref_gguf_read_tensor(path.encode(), name.encode(), out, C.byref(start),
                                                   C.c_void_p(buf.ctypes.data), C.c_size_t(cap)))
        nd = int(out[1])
        return int(out[0]), [int(out[2 + d]) for d in range(nd)], int(out[6]), int(out[7]), int(start.value), \
            buf[:min(cap, int(out[7]))]

    def gguf_read_kv(self, path, key, kind):
        buf = C.create_string_buffer(4096)
        f, u = C.c_float(), C.c_uint32()
        k = {"str": 0, "f32": 1, "u32": 2}[kind]
        self._check(self.lib.kref_gguf_read_kv(path.encode(), key.encode(), k, buf, C.c_size_t(4096),
                                               C.byref(f), C.byref(u)))
        return buf.value.decode() if k == 0 else (f.value if k == 1 else u.value)

    def set_threads(self, n: int):
        self.lib.kref_set_num_threads(C.c_int(n))

    def threads(self) -> int:
        return int(self.lib.kref_num_threads())

    def fp16_to_f32(self, h):
        return float(self.lib.kref_fp16_to_float(h))

    def scale_min_k4(self, j, scales):
        sc, mn = C.c_uint8(), C.c_uint8()
        s = np.ascontiguousarray(scales, dtype=np.uint8)
        self.lib.kref_scale_min_k4(C.c_int(j), _ptr(s), C.byref(sc), C.byref(mn))
        return sc.value, mn.value

    def dot4(self, a, b, acc):
        return int(self.lib.kref_dot4(a, b, acc))

    def silu(self, v):
        return float(self.lib.kref_silu(v))

    def act_bytes(self, K):
        return int(self.lib.kref_int8_scratch_bytes(K))

    def int8_supported(self, dtype, K, bf16=False):
        return bool(self.lib.kref_int8_supported(C.c_uint32(dtype), C.c_size_t(K), C.c_int(int(bf16))))

    @staticmethod
    def _scalar(x, bf16):
        """fp32 values -> the array handed to the reference (fp32 or bf16 bits)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        return f32_to_bf16_bits(x) if bf16 else x

    def quantize_act(self, x, bf16=False):
        K = np.asarray(x).size
        xs = self._scalar(x, bf16)
        s = _aligned(self.act_bytes(K))
        self._check(self.lib.kref_quantize_act(_ptr(xs), C.c_int(int(bf16)), C.c_size_t(K), _ptr(s)))
        return s

    def unit_window(self, dtype, scratch, K, c):
        w = np.empty(10, dtype=np.int32)
        d = np.empty(2, dtype=np.float32)
        self._check(self.lib.kref_unit_window(C.c_int(WD[dtype]), _ptr(scratch), C.c_size_t(K),
                                              C.c_int(c), _ptr(w), _ptr(d)))
        return w, d

    def unit_values(self, dtype, w, rows, cols, scratch):
        out = np.empty((rows, cols // 32), dtype=np.float32)
        self._check(self.lib.kref_unit_values(C.c_int(WD[dtype]), _ptr(w), C.c_size_t(rows),
                                              C.c_size_t(cols), C.c_size_t(row_bytes(dtype, cols)),
                                              _ptr(scratch), _ptr(out)))
        return out

    def quant_gemv(self, dtype, w, rows, cols, x, bf16=False, int8=True, scratch_bytes=None):
        """The reference's quant_gemv. Returns (y as fp32 values of Scalar, staging or None)."""
        xs = self._scalar(x, bf16)
        y = np.zeros(rows, dtype=np.uint16 if bf16 else np.float32)
        s = None
        if int8:
            n = self.act_bytes(cols) if scratch_bytes is None else scratch_bytes
            s = _aligned(max(n, 1))[:n]
        self._check(self.lib.kref_quant_gemv(C.c_uint32(dtype), _ptr(w), C.c_size_t(w.size),
                                             C.c_size_t(rows), C.c_size_t(cols), _ptr(xs), _ptr(y),
                                             C.c_int(int(bf16)), _ptr(s),
                                             C.c_size_t(0 if s is None else s.size)))
        return (bf16_bits_to_f32(y) if bf16 else y), s

    def quant_gemm(self, dtype, w, rows, cols, X, bf16=False):
        X = np.ascontiguousarray(X, dtype=np.float32)
        M = X.shape[0]
        xs = self._scalar(X, bf16)
        Y = np.zeros((M, rows), dtype=np.uint16 if bf16 else np.float32)
        self._check(self.lib.kref_quant_gemm(C.c_uint32(dtype), _ptr(w), C.c_size_t(w.size),
                                             C.c_size_t(rows), C.c_size_t(cols), _ptr(xs),
                                             C.c_size_t(M), _ptr(Y), C.c_int(int(bf16))))
        return bf16_bits_to_f32(Y) if bf16 else Y

    def dequant_to_dense(self, dtype, w, rows, cols, bf16=False):
        Y = np.zeros((rows, cols), dtype=np.uint16 if bf16 else np.float32)
        self._check(self.lib.kref_dequant_to_dense(C.c_uint32(dtype), _ptr(w), C.c_size_t(w.size),
                                                   C.c_size_t(rows), C.c_size_t(cols), _ptr(Y),
                                                   C.c_int(int(bf16))))
        return bf16_bits_to_f32(Y) if bf16 else Y

    def dequant_rows(self, dtype, w, rows, cols):
        rb = row_bytes(dtype, cols)
        out = np.empty((rows, cols), dtype=np.float32)
        for r in range(rows):
            self._check(self.lib.kref_dequant_row(C.c_uint32(dtype), C.c_void_p(w.ctypes.data + r * rb),
                                                  C.c_size_t(cols),
                                                  C.c_void_p(out.ctypes.data + r * cols * 4)))
        return out

    def moe_route(self, logits, bias, top_k, norm_topk, routed_scale=1.0, sigmoid=False, bf16=False):
        lg = np.ascontiguousarray(logits, dtype=np.float32)
        T, E = lg.shape
        ls = self._scalar(lg, bf16)
        nb = 0 if bias is None else len(bias)
        bs = None if nb == 0 else self._scalar(np.asarray(bias, dtype=np.float32), bf16)
        k = max(top_k, 0)
        idx = np.full((T, k), -7, dtype=np.int32)
        w = np.zeros((T, k), dtype=np.float32)
        self._check(self.lib.kref_moe_route(_ptr(ls), C.c_int(int(bf16)), C.c_size_t(T), C.c_size_t(E),
                                            _ptr(bs), C.c_size_t(nb), C.c_int(top_k),
                                            C.c_int(int(norm_topk)), C.c_float(routed_scale),
                                            C.c_int(int(sigmoid)), _ptr(idx), _ptr(w)))
        return idx, w

    def quant_moe_decode(self, x, gate, up, down, idx, wts, F, dtypes=(Q4_K, Q4_K, Q4_K), bf16=False):
        """One token through the reference's fused fp-path kernel pair."""
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        K = x.size
        xs = self._scalar(x, bf16)
        idx = np.ascontiguousarray(idx, dtype=np.int32).reshape(-1)
        wts = np.ascontiguousarray(wts, dtype=np.float32).reshape(-1)
        S = idx.size
        E = len(gate)
        arr = lambda lst: (C.c_void_p * E)(*[a.ctypes.data for a in lst])
        st = np.uint16 if bf16 else np.float32
        act = np.zeros((S, F), dtype=st)
        Y = np.zeros(K, dtype=st)
        self._check(self.lib.kref_quant_moe_decode(_ptr(xs), C.c_int(int(bf16)), C.c_size_t(K),
                                                   C.c_size_t(F), C.c_size_t(E), C.c_uint32(dtypes[0]),
                                                   C.c_uint32(dtypes[1]), C.c_uint32(dtypes[2]),
                                                   arr(gate), arr(up), arr(down), _ptr(idx), _ptr(wts),
                                                   C.c_size_t(S), _ptr(act), _ptr(Y)))
        if bf16:
            return bf16_bits_to_f32(Y), bf16_bits_to_f32(act)
        return Y, act

    def rmsnorm_noscale(self, x, eps, bf16=False):
        """KokkosDNN::rmsnorm_noscale (src/KokkosDNN_RMSNorm.hpp:347-361)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        T, D = x.shape
        xs = self._scalar(x, bf16)
        y = np.zeros((T, D), dtype=np.uint16 if bf16 else np.float32)
        self._check(self.lib.kref_rmsnorm_noscale(_ptr(xs), C.c_int(int(bf16)), C.c_size_t(T), C.c_size_t(D),
                                                  C.c_float(eps), _ptr(y)))
        return bf16_bits_to_f32(y) if bf16 else y

    def swiglu(self, gate, up, bf16=False):
        """KokkosDNN::swiglu (src/KokkosDNN_SwiGLU.hpp:24-38)."""
        gate = np.ascontiguousarray(gate, dtype=np.float32)
        up = np.ascontiguousarray(up, dtype=np.float32)
        T, F = gate.shape
        out = np.zeros((T, F), dtype=np.uint16 if bf16 else np.float32)
        self._check(self.lib.kref_swiglu(_ptr(self._scalar(gate, bf16)), _ptr(self._scalar(up, bf16)), C.c_int(int(bf16)),
                                         C.c_size_t(T), C.c_size_t(F), _ptr(out)))
        return bf16_bits_to_f32(out) if bf16 else out

    def moe_weighted_sum(self, expert_out, top_w, bf16=False):
        eo = np.ascontiguousarray(expert_out, dtype=np.float32)
        T, K, D = eo.shape
        es = self._scalar(eo, bf16)
        tw = np.ascontiguousarray(top_w, dtype=np.float32)
        y = np.zeros((T, D), dtype=np.uint16 if bf16 else np.float32)
        self._check(self.lib.kref_moe_weighted_sum(_ptr(es), _ptr(tw), C.c_size_t(T), C.c_size_t(K),
                                                   C.c_size_t(D), _ptr(y), C.c_int(int(bf16))))
        return bf16_bits_to_f32(y) if bf16 else y

    def moe_gather_rows(self, src, rows, bf16=False):
        src = np.ascontiguousarray(src, dtype=np.float32)
        Cn, D = src.shape
        ss = self._scalar(src, bf16)
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        dst = np.zeros((rows.size, D), dtype=np.uint16 if bf16 else np.float32)
        self._check(self.lib.kref_moe_gather_rows(_ptr(ss), C.c_size_t(Cn), C.c_size_t(D), _ptr(rows),
                                                  C.c_size_t(rows.size), _ptr(dst), C.c_int(int(bf16))))
        return bf16_bits_to_f32(dst) if bf16 else dst

    def moe_scatter_add_weighted(self, src, rows, weights, dst, bf16=False):
        src = np.ascontiguousarray(src, dtype=np.float32)
        N, D = src.shape
        ss = self._scalar(src, bf16)
        ds = self._scalar(np.ascontiguousarray(dst, dtype=np.float32), bf16).copy()
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        weights = np.ascontiguousarray(weights, dtype=np.float32)
        self._check(self.lib.kref_moe_scatter_add_weighted(_ptr(ss), C.c_size_t(N), C.c_size_t(D),
                                                           _ptr(rows), _ptr(weights), _ptr(ds),
                                                           C.c_size_t(dst.shape[0]), C.c_int(int(bf16))))
        return bf16_bits_to_f32(ds) if bf16 else ds
