"""Pins the CPU checker (oracle/kdnn_oracle.c, "port") against
  * the known-answer vectors of the reference's own tests, restated here, and
  * the reference's own operators compiled from its headers (oracle/_ref), and
  * the committed golden fixtures those operators produced.
Runs on CPU only.
"""
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")


# ---- known answers from the reference's tests ---------------------------------
def test_dot4_known_answers(port):
    # tests/Test_IntDot.cpp:112-117
    assert port.dot4(0x01010101, 0x02020202, 100) == 108
    # signed extremes, tests/Test_IntDot.cpp:71-110 construction
    rng = np.random.default_rng(0x1D07)
    menu = np.array([-128, -1, 0, 1, 127], dtype=np.int64)
    for _ in range(2000):
        a = np.where(rng.random(4) < 0.8, rng.choice(menu, 4), rng.integers(-128, 128, 4))
        b = np.where(rng.random(4) < 0.8, rng.choice(menu, 4), rng.integers(-128, 128, 4))
        acc = int(rng.integers(-32768, 32768))
        wa = int(np.sum((a & 0xFF) << (8 * np.arange(4))))
        wb = int(np.sum((b & 0xFF) << (8 * np.arange(4))))
        to_i32 = lambda v: v - (1 << 32) if v >= (1 << 31) else v
        assert port.dot4(to_i32(wa), to_i32(wb), acc) == acc + int(np.dot(a, b))


def test_fp16_known_answers(port):
    # tests/Test_GGUF.cpp:399-410 style spot values, plus subnormals and specials
    for bits, want in [(0x3C00, 1.0), (0x4000, 2.0), (0x3800, 0.5), (0xC000, -2.0), (0x2400, 2.0 ** -6),
                       (0x0001, 2.0 ** -24), (0x03FF, 1023 * 2.0 ** -24), (0x0400, 2.0 ** -14),
                       (0x7BFF, 65504.0), (0x8000, -0.0), (0x7C00, float("inf"))]:
        assert port.fp16_to_f32(bits) == want
    all_bits = np.arange(65536, dtype=np.uint16)
    want = all_bits.view(np.float16).astype(np.float32)
    got = np.array([port.fp16_to_f32(int(b)) for b in all_bits], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])


def test_q4k_hand_computed_block(port):
    # tests/Test_GGUF.cpp:178-233
    b = np.zeros(144, dtype=np.uint8)
    b[0:2] = np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8)
    b[2:4] = np.frombuffer(np.uint16(0x4000).tobytes(), np.uint8)
    b[4:16] = [1, 2, 3, 4, 0, 1, 0, 2, 0x31, 0x02, 0x11, 0x24]
    b[16:] = np.arange(128)
    for j, (sc, mn) in enumerate(zip([1, 2, 3, 4, 1, 2, 1, 4], [0, 1, 0, 2, 3, 0, 1, 2])):
        assert port.scale_min_k4(j, b[4:16]) == (sc, mn)
    out = port.dequant_rows(O.Q4_K, O.aligned_copy(b), 1, 256)[0]
    for i, v in {0: 0.0, 5: 5.0, 32: -2.0, 49: 0.0, 67: 9.0, 103: 4.0, 159: 9.0, 160: 8.0, 202: 8.0,
                 244: 24.0}.items():
        assert out[i] == v


def test_q80_q6k_q5k_spot_blocks(port):
    # tests/Test_GGUF.cpp:238-246
    b = np.zeros(34, dtype=np.uint8)
    b[0:2] = np.frombuffer(np.uint16(0x3800).tobytes(), np.uint8)
    b[2:] = (np.arange(32) * 3 - 20).astype(np.int8).view(np.uint8)
    assert np.array_equal(port.dequant_rows(O.Q8_0, O.aligned_copy(b), 1, 32)[0], 0.5 * (np.arange(32) * 3 - 20))
    # tests/Test_GGUF.cpp:248-283
    b = np.zeros(210, dtype=np.uint8)
    b[208:210] = np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8)
    b[192:208] = 1
    b[5], b[37], b[128 + 5] = 0xA3, 0x7C, 0xE4
    b[64 + 9], b[64 + 41], b[128 + 32 + 9] = 0x51, 0x29, 0x1B
    b[193] = 2
    out = port.dequant_rows(O.Q6_K, O.aligned_copy(b), 1, 256)[0]
    for i, v in {5: -29.0, 37: -4.0, 69: 10.0, 101: 23.0, 137: 17.0, 169: 9.0, 201: -11.0, 233: -30.0,
                 20: -64.0, 0: -32.0, 200: -32.0, 255: -32.0}.items():
        assert out[i] == v
    # tests/Test_GGUF.cpp:285-311
    b = np.zeros(176, dtype=np.uint8)
    b[0:2] = np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8)
    b[2:4] = np.frombuffer(np.uint16(0x4000).tobytes(), np.uint8)
    b[4:16] = [1, 2, 3, 4, 0, 1, 0, 2, 0x31, 0x02, 0x11, 0x24]
    b[16:48] = 0xE4
    b[48:] = np.arange(128)
    out = port.dequant_rows(O.Q5_K, O.aligned_copy(b), 1, 256)[0]
    for i, v in {0: 0.0, 5: 5.0, 32: -2.0, 70: 66.0, 103: 4.0, 128: -6.0, 163: 40.0, 200: 22.0, 235: 84.0}.items():
        assert out[i] == v


def test_router_fixed_logits(port):
    # tests/Test_MoE.cpp:71-75: 3-way tie keeps ids 0, 1 (lower ids first)
    lg = np.array([[0.1, 2.0, -1.0, 0.5, 1.2, -0.3], [1.5, 1.5, 1.5, -2.0, 0.0, 3.0],
                   [-0.5, -0.2, -0.8, -0.1, -1.5, -0.4]], dtype=np.float32)
    idx, w = port.moe_route(lg, None, 2, True)
    assert idx.tolist() == [[1, 4], [5, 0], [3, 1]]
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-5)
    idx3, _ = port.moe_route(lg, None, 4, True)
    assert idx3[1].tolist() == [5, 0, 1, 2]
    with pytest.raises(ValueError):
        port.moe_route(lg, None, 7, True)


def test_int8_gemv_against_double_reference(port):
    """The reference's own check of its int8 GEMV (tests/Test_GGUF.cpp:941-1024): dequantized weights times
    dequantized int8 activations in double, tolerance 1e-4*sum|terms| + 1e-3."""
    import __graft_entry__ as ge
    gp = ge._load_module("_gp_t", os.path.join(ge.PKG_DIR, "ggml_pack.py"))
    for dt in (O.Q4_K, O.Q5_K, O.Q6_K, O.Q8_0):
        for K in (2048, 6656):
            w = O.aligned_copy(gp.random_payload(dt, 7, K, 0xC0FFEE))
            x = (np.random.default_rng(K).integers(-1000, 1001, K) / 1000.0).astype(np.float32)
            y, s = port.gemv_int8(dt, w, 7, K, x)
            acc, mag = port.gemv_dequant_f64(dt, w, 7, K, port.dequant_act(s, K))
            assert np.all(np.abs(y - acc) <= 1e-4 * mag + 1e-3)


# ---- against the reference's own operators (oracle/_ref) ------------------------
def test_port_equals_reference_bit_for_bit(port, ref):
    import __graft_entry__ as ge
    gp = ge._load_module("_gp_t", os.path.join(ge.PKG_DIR, "ggml_pack.py"))
    rng = np.random.default_rng(1)
    for dt in (O.Q4_K, O.Q5_K, O.Q6_K, O.Q8_0):
        for rows, K in ((7, 2048), (3, 512), (2, 6656)):
            w = O.aligned_copy(gp.random_payload(dt, rows, K, rows + K))
            for bf16 in (False, True):
                x = rng.standard_normal(K).astype(np.float32) * rng.choice([1e-3, 1.0, 50.0])
                x[:32] = 0.0
                if bf16:
                    x = O.bf16_round(x)
                sp, sr = port.quantize_act(x), ref.quantize_act(x, bf16=bf16)
                assert np.array_equal(sp, sr)
                for c in (0, 1, 7, K // 32 - 1):
                    wp, dp = port.unit_window(dt, sp, K, c)
                    wr, dr = ref.unit_window(dt, sr, K, c)
                    assert np.array_equal(wp, wr) and np.array_equal(dp, dr)
                _, vals = port.unit_table(dt, w, rows, K, sp)
                assert np.array_equal(vals.view(np.uint32), ref.unit_values(dt, w, rows, K, sr).view(np.uint32))
                yp, _ = port.gemv_int8(dt, w, rows, K, x)
                yr, _ = ref.quant_gemv(dt, w, rows, K, x, bf16=bf16)
                want = O.bf16_round(yp) if bf16 else yp
                assert np.array_equal(want.view(np.uint32), yr.view(np.uint32))
            assert np.array_equal(port.dequant_rows(dt, w, rows, K).view(np.uint32),
                                  ref.dequant_rows(dt, w, rows, K).view(np.uint32))
    for h in (0, 1, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0x8001, 0xFBFF, 0x2400):
        assert port.fp16_to_f32(h) == ref.fp16_to_f32(h)
    for v in (-20.0, -1.0, 0.0, 0.3, 5.0, 30.0):
        assert port.silu(v) == ref.silu(v)


def test_router_equals_reference(port, ref):
    rng = np.random.default_rng(2)
    for T, E, k in ((3, 6, 2), (64, 8, 2), (256, 128, 8), (5, 64, 64)):
        lg = rng.standard_normal((T, E)).astype(np.float32)
        lg[0, : min(E, 4)] = 1.25                      # ties
        bias = (rng.standard_normal(E) * 0.1).astype(np.float32)
        for b in (None, bias):
            for norm in (True, False):
                for sig in (False, True):
                    ip, wp = port.moe_route(lg, b, k, norm, 1.5, sig)
                    ir, wr = ref.moe_route(lg, b, k, norm, 1.5, sig)
                    assert np.array_equal(ip, ir)
                    assert np.array_equal(wp.view(np.uint32), wr.view(np.uint32))


def test_moe_composition_vs_reference_fp_decode(port, ref):
    """The int8 composition stays within the expected ~1% of the reference's fused fp kernel pair
    (activation rounding), and its act rows within bf16 resolution."""
    g = np.load(os.path.join(GOLD, "moe_decode_fp.npz"))
    E, H, F, S = [int(v) for v in g["meta"]]
    al = lambda a: [O.aligned_copy(a[e]) for e in range(E)]
    gate, up, down = al(g["gate"]), al(g["up"]), al(g["down"])
    Yr, actr = ref.quant_moe_decode(g["x"], gate, up, down, g["idx"], g["wts"], F, bf16=True)
    assert np.array_equal(Yr, g["Y"]) and np.array_equal(actr, g["act"])
    Y, act = port.moe_ffn_int8(g["x"][None, :], gate, up, down, g["idx"][None, :], g["wts"][None, :], F,
                               bf16=True, want_act=True)
    assert np.abs(Y[0] - Yr).max() <= 3e-2 * np.abs(Yr).max()
    assert np.abs(act[0] - actr).max() <= 3e-2 * np.abs(actr).max()


# ---- committed fixtures (usable where the reference sources are absent) ---------
def test_port_reproduces_golden_gemv(port):
    g = np.load(os.path.join(GOLD, "gemv_int8.npz"))
    for tag in [t[:-2] for t in g.files if t.endswith("_w")]:
        dt, rows, K = [int(v) for v in g[tag + "_meta"]]
        y, s = port.gemv_int8(dt, O.aligned_copy(g[tag + "_w"]), rows, K, g[tag + "_x"])
        assert np.array_equal(s, g[tag + "_staging"])
        want = O.bf16_round(y) if "bf16" in tag else y
        assert np.array_equal(want.view(np.uint32), g[tag + "_y"].view(np.uint32))


def test_port_reproduces_golden_router(port):
    g = np.load(os.path.join(GOLD, "moe_route.npz"))
    n = len([f for f in g.files if f.endswith("_cfg")])
    for c in range(n):
        k, norm, sig, bf16 = [int(v) for v in g[f"c{c}_cfg"]]
        bias = g[f"c{c}_bias"]
        idx, w = port.moe_route(g[f"c{c}_logits"], bias if bias.size else None, k, bool(norm),
                                float(g[f"c{c}_scale"][0]), bool(sig))
        assert np.array_equal(idx, g[f"c{c}_idx"])
        assert np.array_equal(w.view(np.uint32), g[f"c{c}_w"].view(np.uint32))
