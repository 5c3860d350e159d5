"""CPU-only checks of the C ABI: the library loads, exports every symbol the header declares, and the
argument checks that return before any launch behave like the reference's (decline vs invalid_argument)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(kd):
    header = open(os.path.join(ROOT, "include", "kdnn_b200.h")).read()
    declared = set(re.findall(r"\b(kdnn_b200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(kd.EXPORTS)
    for name in declared:
        assert hasattr(kd.lib, name), name


def test_scratch_bytes_and_supported(kd):
    # tests/Test_GGUF.cpp:1121-1137
    assert kd.quant_gemv_int8_scratch_bytes(512) > 512
    assert kd.quant_gemv_int8_scratch_bytes(500) == 0
    assert kd.quant_gemv_int8_scratch_bytes(4096) == 4096 + 16 * 128
    import torch
    assert not kd.quant_gemv_int8_supported(0, 512)             # F32 weights
    assert not kd.quant_gemv_int8_supported(kd.Q4_K, 128)       # K not block aligned
    assert kd.quant_gemv_int8_supported(kd.Q4_K, 512)
    assert kd.quant_gemv_int8_supported(kd.Q6_K, 6656, torch.bfloat16)
    assert kd.quant_gemv_int8_supported(kd.Q8_0, 64)
    assert kd.quant_gemv_int8_supported(kd.Q5_K, 512) and not kd.quant_gemv_int8_supported(kd.Q5_K, 96)
    assert not kd.quant_gemv_int8_supported(kd.Q8_0, 48)
    assert not kd.quant_gemv_int8_supported(kd.Q4_K, 512, torch.float16)


def test_gemv_declines_without_launching(kd):
    """The decline list of src/KokkosDNN_GGUFGemvInt8.hpp:724-745; fake non-null pointers are never touched."""
    f = kd.lib.kdnn_b200_quant_gemv
    W, X, Y, S = 0x10000, 0x20000, 0x30000, 0x40000
    need = kd.quant_gemv_int8_scratch_bytes(512)
    ok = dict(t=kd.Q4_K, w=W, rows=4, cols=512, x=X, y=Y, s=S, sb=need)

    def call(**kw):
        a = dict(ok, **kw)
        return f(a["t"], a["w"], a["rows"], a["cols"], a["x"], 0, a["y"], 0, a["s"], a["sb"], None)

    assert call(w=None) == kd.KDNN_DECLINED
    assert call(s=None) == kd.KDNN_DECLINED
    assert call(cols=128) == kd.KDNN_DECLINED                 # Q4_K needs K % 256 == 0
    assert call(rows=0) == kd.KDNN_DECLINED
    assert call(rows=2 ** 31) == kd.KDNN_DECLINED
    assert call(sb=need // 2) == kd.KDNN_DECLINED             # undersized staging (Test_GGUF.cpp:1039-1042)
    assert call(s=S + 8) == kd.KDNN_DECLINED                  # staging not 16-byte aligned
    assert call(w=W + 1) == kd.KDNN_DECLINED                  # odd payload
    assert call(w=W + 2) == kd.KDNN_DECLINED                  # Q4_K payload not 16-byte aligned
    assert call(t=0) == kd.KDNN_DECLINED                      # F32 weights keep the portable path
    assert call(t=kd.Q5_K, w=W + 2) == kd.KDNN_DECLINED       # Q5_K payload not 16-byte aligned either
    assert call(t=kd.Q5_K, cols=128) == kd.KDNN_DECLINED


def test_host_gemv_declines_before_any_copy(kd):
    """kdnn_b200_quant_gemv_host checks the whole decline list first: a declined call has enqueued no copy
    (the fake pointers would fault one)."""
    f = kd.lib.kdnn_b200_quant_gemv_host
    W, XH, YH, XD, YD, S = 0x10000, 0x20000, 0x30000, 0x40000, 0x50000, 0x60000
    need = kd.quant_gemv_int8_scratch_bytes(512)
    ok = dict(t=kd.Q4_K, w=W, rows=4, cols=512, xh=XH, yh=YH, xd=XD, yd=YD, s=S, sb=need, xs=0)

    def call(**kw):
        a = dict(ok, **kw)
        return f(a["t"], a["w"], a["rows"], a["cols"], a["xh"], a["xs"], a["yh"], 0, a["xd"], a["yd"], a["s"],
                 a["sb"], None)

    for kw in (dict(w=None), dict(s=None), dict(xd=None), dict(yd=None), dict(cols=128), dict(rows=0),
               dict(sb=need // 2), dict(s=S + 8), dict(w=W + 1), dict(w=W + 2), dict(t=0)):
        assert call(**kw) == kd.KDNN_DECLINED, kw
    assert call(xh=None) == kd.KDNN_ERR_INVALID
    assert call(yh=None) == kd.KDNN_ERR_INVALID
    assert call(xs=7) == kd.KDNN_ERR_INVALID


def test_invalid_arguments_raise(kd):
    import torch
    w = kd.QuantWeight(torch.zeros(2 * 34, dtype=torch.uint8), kd.Q8_0, 1, 64)
    x, y, s = torch.zeros(32), torch.zeros(1), torch.zeros(64, dtype=torch.uint8)
    with pytest.raises(ValueError, match="dimension mismatch"):       # tests/Test_GGUF.cpp:1253-1259
        kd.quant_gemv(x, w, y, s)
    with pytest.raises(ValueError):                                   # cols not a whole number of blocks (:1260-1269)
        kd.quant_gemv(torch.zeros(17), kd.QuantWeight(torch.zeros(34, dtype=torch.uint8), kd.Q8_0, 1, 17), y, s)
    with pytest.raises(ValueError, match="unsupported dtype"):        # :1247-1252
        kd.quant_gemv(x, kd.QuantWeight(torch.zeros(18, dtype=torch.uint8), 2, 1, 32), y, s)
    with pytest.raises(ValueError, match="payload size"):
        kd.quant_gemv(torch.zeros(64), kd.QuantWeight(torch.zeros(10, dtype=torch.uint8), kd.Q8_0, 1, 64), y, s)
    # router argument checks (src/KokkosDNN_MoE.hpp:251-258; tests/Test_MoE.cpp:491-518)
    lg = torch.zeros(2, 4)
    with pytest.raises(ValueError, match="top_k"):
        kd.moe_route(lg, None, 5, True, 1.0, torch.zeros(2, 5, dtype=torch.int32), torch.zeros(2, 5))
    with pytest.raises(ValueError, match="output dimension"):
        kd.moe_route(lg, None, 2, True, 1.0, torch.zeros(2, 3, dtype=torch.int32), torch.zeros(2, 2))
    with pytest.raises(ValueError, match="expert_bias"):
        kd.moe_route(lg, torch.zeros(3), 2, True, 1.0, torch.zeros(2, 2, dtype=torch.int32), torch.zeros(2, 2))
    kd.moe_route(torch.zeros(0, 4), None, 2, True, 1.0, torch.zeros(0, 2, dtype=torch.int32), torch.zeros(0, 2))


def test_encoders_round_trip(kd, port):
    import numpy as np
    from oracle import oracle as O
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((32, 1024)) * 0.02).astype(np.float32)
    for dt, tol in ((kd.Q8_0, 0.01), (kd.Q6_K, 0.03), (kd.Q4_K, 0.12)):
        packed = kd.ggml_pack.quantize(dt, w)
        assert packed.shape == (32, kd.ggml_row_bytes(dt, 1024))
        dq = port.dequant_rows(dt, O.aligned_copy(packed), 32, 1024)
        assert np.sqrt(((dq - w) ** 2).mean()) / w.std() < tol
    z = kd.ggml_pack.quantize(kd.Q4_K, np.zeros((1, 256), np.float32))
    assert np.all(port.dequant_rows(kd.Q4_K, O.aligned_copy(z), 1, 256) == 0)
