"""Encoders from fp32 matrices to GGUF block-quantized rows (Q8_0, Q4_K, Q6_K).

The reference library has no fp32 -> K-quant quantizer (its tests build blocks by
hand or fill payloads with random bytes), so synthetic benchmark weights need
one. These are simple per-sub-block min/max encoders that emit *valid* blocks in
the unchanged ggml layouts (src/KokkosDNN_GGUF.hpp:242-271 in the reference):
they are not ggml's quantizers and make no claim to match their bit patterns.
Parity is defined on the packed bytes, which the CPU checker and the CUDA
kernels both consume unchanged.

Also provides ``random_payload`` -- random bytes with sanitized fp16 scale fields,
the fixture style of the reference's tests (tests/Test_GGUF.cpp:941-971).
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_K, Q5_K, Q6_K = 8, 12, 13, 14
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}
NAMES = {Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K"}


def row_bytes(dtype: int, cols: int) -> int:
    n, b = BLOCK[dtype]
    if cols % n:
        raise ValueError(f"cols {cols} is not a multiple of {n} for {NAMES[dtype]}")
    return cols // n * b


def _f16(a: np.ndarray) -> np.ndarray:
    """Round to fp16 and return (fp32 value of the fp16, uint16 bits)."""
    h = np.asarray(a, dtype=np.float32).astype(np.float16)
    return h.astype(np.float32), h.view(np.uint16)


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    rows, cols = w.shape
    nb = cols // 32
    x = np.ascontiguousarray(w, dtype=np.float32).reshape(rows, nb, 32)
    amax = np.abs(x).max(axis=2)
    d, dbits = _f16(amax / 127.0)
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1.0), 0.0)
    q = np.clip(np.rint(x * inv[..., None]), -127, 127).astype(np.int8)
    out = np.empty((rows, nb, 34), dtype=np.uint8)
    out[..., 0:2] = dbits.reshape(rows, nb, 1).view(np.uint8)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(rows, nb * 34)


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    rows, cols = w.shape
    nb = cols // 256
    x = np.ascontiguousarray(w, dtype=np.float32).reshape(rows, nb, 8, 32)
    lo = np.minimum(x.min(axis=3), 0.0)           # sub-block offset is subtracted: min >= 0
    hi = np.maximum(x.max(axis=3), lo)
    scale = (hi - lo) / 15.0
    mins = -lo
    d, dbits = _f16(scale.max(axis=2) / 63.0)
    dm, mbits = _f16(mins.max(axis=2) / 63.0)
    sc = np.where(d[..., None] > 0, np.rint(scale / np.where(d > 0, d, 1.0)[..., None]), 0)
    mn = np.where(dm[..., None] > 0, np.rint(mins / np.where(dm > 0, dm, 1.0)[..., None]), 0)
    sc = np.clip(sc, 0, 63).astype(np.uint8)
    mn = np.clip(mn, 0, 63).astype(np.uint8)
    eff = d[..., None] * sc.astype(np.float32)
    off = dm[..., None] * mn.astype(np.float32)
    q = np.where(eff[..., None] > 0,
                 np.rint((x + off[..., None]) / np.where(eff > 0, eff, 1.0)[..., None]), 0)
    q = np.clip(q, 0, 15).astype(np.uint8)
    out = np.zeros((rows, nb, 144), dtype=np.uint8)
    out[..., 0:2] = dbits.reshape(rows, nb, 1).view(np.uint8)
    out[..., 2:4] = mbits.reshape(rows, nb, 1).view(np.uint8)
    s = out[..., 4:16]
    for j in range(4):
        s[..., j] = (sc[..., j] & 63) | ((sc[..., j + 4] >> 4) << 6)
        s[..., j + 4] = (mn[..., j] & 63) | ((mn[..., j + 4] >> 4) << 6)
        s[..., j + 8] = (sc[..., j + 4] & 0xF) | ((mn[..., j + 4] & 0xF) << 4)
    # 64-element group `it`: low nibbles = sub-block 2*it, high nibbles = sub-block 2*it+1
    qq = q.reshape(rows, nb, 4, 2, 32)
    out[..., 16:] = (qq[:, :, :, 0, :] | (qq[:, :, :, 1, :] << 4)).reshape(rows, nb, 128)
    return out.reshape(rows, nb * 144)


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    rows, cols = w.shape
    nb = cols // 256
    x = np.ascontiguousarray(w, dtype=np.float32).reshape(rows, nb, 16, 16)
    s = np.abs(x).max(axis=3) / 31.0
    d, dbits = _f16(s.max(axis=2) / 127.0)
    sc = np.where(d[..., None] > 0, np.rint(s / np.where(d > 0, d, 1.0)[..., None]), 0)
    sc = np.clip(sc, 0, 127).astype(np.int8)
    eff = d[..., None] * sc.astype(np.float32)
    q = np.where(eff[..., None] > 0, np.rint(x / np.where(eff > 0, eff, 1.0)[..., None]), 0)
    q = (np.clip(q, -32, 31) + 32).astype(np.uint8).reshape(rows, nb, 2, 4, 32)  # [chunk, sub, ll]
    out = np.zeros((rows, nb, 210), dtype=np.uint8)
    ql = out[..., 0:128].reshape(rows, nb, 2, 2, 32)     # [chunk, sub&1, ll]
    qh = out[..., 128:192].reshape(rows, nb, 2, 32)      # [chunk, ll]
    lo4, hi2 = q & 0xF, q >> 4
    ql[:, :, :, 0, :] = lo4[:, :, :, 0, :] | (lo4[:, :, :, 2, :] << 4)
    ql[:, :, :, 1, :] = lo4[:, :, :, 1, :] | (lo4[:, :, :, 3, :] << 4)
    qh[...] = hi2[:, :, :, 0, :] | (hi2[:, :, :, 1, :] << 2) | (hi2[:, :, :, 2, :] << 4) | (hi2[:, :, :, 3, :] << 6)
    out[..., 192:208] = sc.view(np.uint8)
    out[..., 208:210] = dbits.reshape(rows, nb, 1).view(np.uint8)
    return out.reshape(rows, nb * 210)


def quantize(dtype: int, w: np.ndarray) -> np.ndarray:
    """fp32 [rows, cols] -> packed uint8 [rows, row_bytes]."""
    if dtype == Q8_0:
        return quantize_q8_0(w)
    if dtype == Q4_K:
        return quantize_q4_k(w)
    if dtype == Q6_K:
        return quantize_q6_k(w)
    raise ValueError(f"no encoder for ggml type {dtype}")


def synth_weight(dtype: int, rows: int, cols: int, seed: int, std: float = 0.02,
                 chunk_rows: int = 2048) -> np.ndarray:
    """Seeded N(0, std) fp32 matrix quantized row-chunk by row-chunk."""
    rng = np.random.default_rng(seed)
    out = np.empty((rows, row_bytes(dtype, cols)), dtype=np.uint8)
    for r0 in range(0, rows, chunk_rows):
        r1 = min(rows, r0 + chunk_rows)
        out[r0:r1] = quantize(dtype, rng.standard_normal((r1 - r0, cols), dtype=np.float32) * std)
    return out


def random_payload(dtype: int, rows: int, cols: int, seed: int, scale_bits: int = 0x2400) -> np.ndarray:
    """Random bytes with every fp16 super-block scale set to `scale_bits`
    (0x2400 = 2^-6 by default) so no block decodes to inf/nan; exercises every 6-bit
    scale/min and every Q6_K int8 scale value."""
    rng = np.random.default_rng(seed)
    nbl, bsz = BLOCK[dtype]
    nb = cols // nbl
    raw = rng.integers(0, 256, size=(rows, nb, bsz), dtype=np.uint8)
    sb = np.array([scale_bits & 0xFF, scale_bits >> 8], dtype=np.uint8)
    if dtype == Q6_K:
        raw[..., 208:210] = sb
    elif dtype == Q8_0:
        raw[..., 0:2] = sb
    else:
        raw[..., 0:2] = sb
        raw[..., 2:4] = sb
    return raw.reshape(rows, nb * bsz)
