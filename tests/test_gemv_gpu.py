"""Parity of the CUDA int8 GEMV (through the C ABI) against the CPU checker.

Bars: activation staging bytes and per-unit integer dots bit-exact; fp32 row sums
within 1e-3 of max|y| (the north-star tolerance; the reference's own int8 tests use
1e-3 absolute on crafted data and 1e-4*sum|terms|+1e-3 on random payloads,
tests/Test_GGUF.cpp:923, :1021 -- both are asserted where they apply); bf16
outputs within one bf16 ulp of the rounded checker value.
Shapes follow tests/Test_GGUF.cpp:1118-1201.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
DTYPES = [O.Q4_K, O.Q6_K, O.Q8_0]
DTYPES_RANDOM = DTYPES + [O.Q5_K]   # Q5_K has no encoder here: random payloads only


def _run(kd, dtype, packed, rows, K, x_t, y_dtype, layout=None):
    dev = torch.device("cuda:0")
    w = kd.QuantWeight.from_numpy(packed, dtype, rows, K, dev)
    y = torch.full((rows,), float("nan"), dtype=y_dtype, device=dev)
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
    kd.quant_gemv(x_t.to(dev), w, y, scratch, layout)
    torch.cuda.synchronize()
    assert kd.device_status() == 0
    return w, y, scratch


def _check(kd, port, dtype, rows, K, seed, payload, x_dtype=torch.float32, y_dtype=torch.float32,
           probe=True, layout=None):
    if payload == "random":
        packed = kd.ggml_pack.random_payload(dtype, rows, K, seed)
    else:
        packed = kd.ggml_pack.synth_weight(dtype, rows, K, seed)
    g = torch.Generator().manual_seed(seed + 1)
    x_t = torch.randn(K, generator=g).to(x_dtype)
    w, y, scratch = _run(kd, dtype, packed, rows, K, x_t, y_dtype, layout)
    host = O.aligned_copy(packed)
    xf = x_t.float().numpy()
    y_ref, staging = port.gemv_int8(dtype, host, rows, K, xf)
    # 1. staging bytes (int8 row + {d, sum_lo, sum_hi, pad} headers): bit-exact
    assert np.array_equal(scratch.cpu().numpy(), staging)
    # 2. integer dots of every unit: bit-exact
    if probe:
        ints_ref, _ = port.unit_table(dtype, host, rows, K, staging)
        ints = kd.unit_dots(w, scratch).cpu().numpy()
        assert np.array_equal(ints, ints_ref)
    # 3. row sums
    got = y.float().cpu().numpy()
    scale = max(np.abs(y_ref).max(), 1e-30)
    if y_dtype == torch.float32:
        assert np.abs(got - y_ref).max() <= 1e-3 * scale
        # the reference's random-payload bound against double accumulation
        acc, mag = port.gemv_dequant_f64(dtype, host, rows, K, port.dequant_act(staging, K))
        assert np.all(np.abs(got - acc) <= 1e-4 * mag + 1e-3)
    else:
        want = O.bf16_round(y_ref)
        ulp = np.maximum(np.abs(want), 1e-30) * 2.0 ** -7
        assert np.all(np.abs(got - want) <= ulp)
    return got, y_ref


@pytest.mark.parametrize("dtype", DTYPES_RANDOM)
@pytest.mark.parametrize("K", [512, 1024, 2048, 4096, 6656])
def test_random_payload_small_rows(kd, port, dtype, K):
    _check(kd, port, dtype, 7, K, 0xC0FFEE, "random")


@pytest.mark.parametrize("dtype", DTYPES_RANDOM)
@pytest.mark.parametrize("rows", [1, 3, 5, 17, 256, 1023, 1024, 1025, 1102])
def test_row_tails(kd, port, dtype, rows):
    _check(kd, port, dtype, rows, 2048 if dtype != O.Q4_K else 512, 11 + rows, "random")


@pytest.mark.parametrize("dtype", DTYPES)
def test_bf16_activations_and_outputs(kd, port, dtype):
    _check(kd, port, dtype, 256, 4096, 5, "synth", torch.bfloat16, torch.float32)
    _check(kd, port, dtype, 256, 4096, 6, "synth", torch.bfloat16, torch.bfloat16, probe=False)
    _check(kd, port, dtype, 33, 2048, 7, "random", torch.float32, torch.bfloat16, probe=False)


def test_crafted_unit_scale_cases(kd, port):
    """Exact-value packings of tests/Test_GGUF.cpp:616-682 with the 1e-3 absolute bound of :1138-1145."""
    dev = torch.device("cuda:0")
    for dtype, K in [(O.Q4_K, 512), (O.Q4_K, 4096), (O.Q6_K, 2048), (O.Q6_K, 4096), (O.Q8_0, 512)]:
        N = 5
        idx = (np.arange(N * K).reshape(N, K))
        if dtype == O.Q4_K:
            vals = (idx % 16).astype(np.uint8).reshape(N, K // 256, 4, 2, 32)
            blocks = np.zeros((N, K // 256, 144), dtype=np.uint8)
            blocks[..., 0:2] = np.frombuffer(np.uint16(0x3C00).tobytes(), dtype=np.uint8)
            blocks[..., 4:16] = np.array([1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1], dtype=np.uint8)
            blocks[..., 16:] = (vals[:, :, :, 0, :] | (vals[:, :, :, 1, :] << 4)).reshape(N, K // 256, 128)
            dense = (idx % 16).astype(np.float32)
        elif dtype == O.Q6_K:
            v = (idx % 16).astype(np.uint8).reshape(N, K // 256, 2, 4, 32)   # stored nibble = value + 32 - 32
            blocks = np.zeros((N, K // 256, 210), dtype=np.uint8)
            ql = blocks[..., :128].reshape(N, K // 256, 2, 2, 32)
            ql[:, :, :, 0, :] = v[:, :, :, 0, :] | (v[:, :, :, 2, :] << 4)
            ql[:, :, :, 1, :] = v[:, :, :, 1, :] | (v[:, :, :, 3, :] << 4)
            blocks[..., 192:208] = 1
            blocks[..., 208:210] = np.frombuffer(np.uint16(0x3C00).tobytes(), dtype=np.uint8)
            dense = -32.0 + (idx % 16).astype(np.float32)
        else:
            dense = (0.125 * (idx % 5) - 0.25).astype(np.float32)
            blocks = kd.ggml_pack.quantize_q8_0(dense)
        packed = blocks.reshape(N, -1)
        host = O.aligned_copy(packed)
        if dtype != O.Q8_0:
            assert np.array_equal(port.dequant_rows(dtype, host, N, K), dense)
        x = (0.125 * ((np.arange(K) % 7) - 3)).astype(np.float32)
        w, y, scratch = _run(kd, dtype, packed, N, K, torch.from_numpy(x), torch.float32)
        staging = port.quantize_act(x)
        assert np.array_equal(scratch.cpu().numpy(), staging)
        acc, _ = port.gemv_dequant_f64(dtype, host, N, K, port.dequant_act(staging, K))
        assert np.abs(y.cpu().numpy() - acc).max() <= 1e-3


def test_quantizer_edge_values(kd, port):
    """All-zero blocks give d = 0, q = 0; +-amax hit +-127; ties round to even."""
    dev = torch.device("cuda:0")
    K = 256
    x = np.zeros(K, dtype=np.float32)
    x[32:64] = np.linspace(-1, 1, 32)
    x[64:96] = 0.5 * 127.0 / 127.0 * np.where(np.arange(32) % 2, 1.0, -1.0)
    x[96:128] = (np.arange(32) + 0.5) * (1.0 / 127.0) * 4          # .5 ties after scaling by 127/amax
    x[128:160] = 1e-30
    x[160:192] = np.float32(3.0e38)
    for dt in (torch.float32, torch.bfloat16):
        xt = torch.from_numpy(x).to(dt)
        scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
        kd.quantize_act_q8(xt.to(dev), scratch)
        torch.cuda.synchronize()
        assert np.array_equal(scratch.cpu().numpy(), port.quantize_act(xt.float().numpy()))


def test_generic_kernel_matches_for_misaligned_payload(kd, port):
    """A payload base that is only 2-byte aligned (allowed for Q6_K / Q8_0 by the reference's contract,
    src/KokkosDNN_GGUFGemvInt8.hpp:739-743) takes the plain-load kernels."""
    dev = torch.device("cuda:0")
    for dtype in (O.Q6_K, O.Q8_0):
        rows, K = 19, 2048
        packed = kd.ggml_pack.random_payload(dtype, rows, K, 3)
        buf = torch.zeros(packed.size + 16, dtype=torch.uint8, device=dev)
        buf[2:2 + packed.size] = torch.from_numpy(packed.reshape(-1)).to(dev)
        w = kd.QuantWeight(buf[2:2 + packed.size], dtype, rows, K)
        x = torch.randn(K, generator=torch.Generator().manual_seed(9))
        y = torch.empty(rows, dtype=torch.float32, device=dev)
        scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
        kd.quant_gemv(x.to(dev), w, y, scratch)
        torch.cuda.synchronize()
        y_ref, staging = port.gemv_int8(dtype, O.aligned_copy(packed), rows, K, x.numpy())
        assert np.array_equal(scratch.cpu().numpy(), staging)
        assert np.abs(y.cpu().numpy() - y_ref).max() <= 1e-3 * np.abs(y_ref).max()


@pytest.mark.parametrize("dtype,rows,K", [(O.Q4_K, 4096, 4096), (O.Q8_0, 4096, 4096),
                                           (O.Q4_K, 14336, 4096), (O.Q6_K, 4096, 14336)])
def test_baseline_shapes_full_size(kd, port, dtype, rows, K):
    """The benchmark configurations themselves, every row against the checker."""
    _check(kd, port, dtype, rows, K, 1234, "synth", torch.bfloat16, torch.float32, probe=False)


def test_golden_fixture(kd):
    """Outputs of the reference's own int8 quant_gemv, generated by tests/golden/make_golden.py."""
    import os
    path = os.path.join(os.path.dirname(__file__), "golden", "gemv_int8.npz")
    g = np.load(path)
    dev = torch.device("cuda:0")
    for tag in [t[:-2] for t in g.files if t.endswith("_w")]:
        dtype, rows, K = [int(v) for v in g[tag + "_meta"]]
        x = torch.from_numpy(g[tag + "_x"])
        xt = x.to(torch.bfloat16) if "bf16" in tag else x
        w, y, scratch = _run(kd, dtype, g[tag + "_w"], rows, K, xt, torch.float32)
        assert np.array_equal(scratch.cpu().numpy(), g[tag + "_staging"])
        yr = g[tag + "_y"]
        if "bf16" in tag:   # the reference rounded y to bf16
            got = O.bf16_round(y.cpu().numpy())
            assert np.all(np.abs(got - yr) <= np.abs(yr) * 2.0 ** -7 + 1e-30)
        else:
            assert np.abs(y.cpu().numpy() - yr).max() <= 1e-3 * np.abs(yr).max()


@pytest.mark.parametrize("dtype", DTYPES_RANDOM)
def test_graph_replays_recompute_every_row(kd, port, dtype):
    """A captured sequence of GEMVs must do all of its work on every replay: tall matrices
    (more row groups than resident warps, so the in-kernel work distribution is exercised),
    outputs poisoned before each replay, each replay checked against the checker."""
    dev = torch.device("cuda:0")
    rows, K = 9000, 2048
    mats, outs, refs = [], [], []
    g = torch.Generator().manual_seed(77)
    x_t = torch.randn(K, generator=g)
    for i in range(3):
        packed = kd.ggml_pack.random_payload(dtype, rows, K, 500 + i)
        mats.append(kd.QuantWeight.from_numpy(packed, dtype, rows, K, dev))
        outs.append(torch.empty(rows, dtype=torch.float32, device=dev))
        refs.append(port.gemv_int8(dtype, O.aligned_copy(packed), rows, K, x_t.numpy())[0])
    x = x_t.to(dev)
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for w, y in zip(mats, outs):
            kd.quant_gemv(x, w, y, scratch)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for w, y in zip(mats, outs):
                kd.quant_gemv(x, w, y, scratch)
        for _ in range(4):
            for y in outs:
                y.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            for y, ref in zip(outs, refs):
                got = y.cpu().numpy()
                assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()
    assert kd.device_status() == 0


@pytest.mark.parametrize("layout", [{"kernel": 2}, {"kernel": 3}, {"kernel": 3, "rows_per_group": 1}, {"kernel": 4},
                                    {"stages": 2}, {"stages": 4, "early_stages": 1}, {"rows_per_group": 1, "no_pdl": 1}])
@pytest.mark.parametrize("dtype", DTYPES_RANDOM)
def test_alternate_streaming_kernels(kd, port, dtype, layout):
    """The kernels that take over for very long rows (activation window in shared memory, item
    mapping), the plain-load kernels and the other ring depths can be selected per call through the
    layout struct (the counterpart of Int8Layout); they must give the same results as the defaults."""
    _check(kd, port, dtype, 37, 4096, 91, "random", layout=layout)
    _check(kd, port, dtype, 5000, 2048, 92, "random", probe=False, layout=layout)
    _check(kd, port, dtype, 300, 6144 if dtype != O.Q4_K else 6656, 93, "random", probe=False, layout=layout)


def test_q5k_lm_head_like_shape(kd, port):
    """Q4_K_M files keep their largest matrices in Q5_K (src/KokkosDNN_GGUF.hpp:13-19)."""
    _check(kd, port, O.Q5_K, 16000, 4096, 404, "random", torch.bfloat16, torch.float32, probe=False)
    _check(kd, port, O.Q5_K, 64, 4096, 405, "random", torch.bfloat16, torch.bfloat16, probe=False)


@pytest.mark.parametrize("dtype", DTYPES_RANDOM)
@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
def test_host_buffer_call_matches_the_device_call(kd, dtype, x_dtype):
    """kdnn_b200_quant_gemv_host = copy in, the same GEMV, copy out: bit-identical results."""
    dev = torch.device("cuda:0")
    rows, K = 517, 2048
    w = kd.QuantWeight.from_numpy(kd.ggml_pack.random_payload(dtype, rows, K, 77), dtype, rows, K, dev)
    x_host = torch.randn(K, generator=torch.Generator().manual_seed(78)).to(x_dtype).pin_memory()
    y_host = torch.full((rows,), float("nan")).pin_memory()
    x_dev, y_dev = torch.zeros(K, dtype=x_dtype, device=dev), torch.zeros(rows, device=dev)
    y_want = torch.empty(rows, device=dev)
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
    kd.quant_gemv(x_host.to(dev), w, y_want, scratch)
    for _ in range(2):                       # the second call reuses every buffer
        y_host.fill_(float("nan"))
        kd.quant_gemv_host(x_host, w, y_host, x_dev, y_dev, scratch)
        torch.cuda.synchronize()
        assert torch.equal(y_host, y_want.cpu())
    assert kd.device_status() == 0
    with pytest.raises(ValueError, match="host tensors"):
        kd.quant_gemv_host(x_dev, w, y_host, x_dev, y_dev, scratch)


def test_host_buffer_call_with_pageable_memory(kd):
    """Pageable host buffers cannot be touched by a kernel: the call takes the copy engine for them."""
    dev = torch.device("cuda:0")
    rows, K = 129, 1024
    w = kd.QuantWeight.from_numpy(kd.ggml_pack.random_payload(kd.Q4_K, rows, K, 79), kd.Q4_K, rows, K, dev)
    x_host = torch.randn(K, generator=torch.Generator().manual_seed(80))
    y_host = torch.full((rows,), float("nan"))
    x_dev, y_dev = torch.zeros(K, device=dev), torch.zeros(rows, device=dev)
    y_want = torch.empty(rows, device=dev)
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
    kd.quant_gemv(x_host.to(dev), w, y_want, scratch)
    kd.quant_gemv_host(x_host, w, y_host, x_dev, y_dev, scratch)
    torch.cuda.synchronize()
    assert torch.equal(y_host, y_want.cpu())
    assert kd.device_status() == 0


@pytest.mark.parametrize("n,rows,K,dtype_name,x_dtype", [
    (2, 1500, 4096, "Q4_K", torch.bfloat16),     # gate + up: one launch
    (3, 257, 2048, "Q4_K", torch.float32),       # odd row count: the last row group of every matrix is half full
    (4, 64, 256, "Q4_K", torch.bfloat16),        # fewer row groups than CTAs
    (5, 96, 1024, "Q4_K", torch.float32),        # more than four matrices: 4 + 1
    (2, 40, 8192, "Q4_K", torch.float32),        # rows of two chunks: runs as two launches
    (2, 130, 2048, "Q6_K", torch.bfloat16),      # another format: runs as two launches
])
def test_multi_matrix_call_equals_single_calls(kd, n, rows, K, dtype_name, x_dtype):
    """kdnn_b200_quant_gemv_multi against kdnn_b200_quant_gemv per matrix: bit for bit (the same kernel adds
    the same terms in the same order whichever launch a row lands in)."""
    dev = torch.device("cuda:0")
    dtype = getattr(kd, dtype_name)
    ws = [kd.QuantWeight.from_numpy(kd.ggml_pack.random_payload(dtype, rows, K, 900 + i), dtype, rows, K, dev)
          for i in range(n)]
    x = torch.randn(K, generator=torch.Generator().manual_seed(5)).to(x_dtype).to(dev)
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
    singles = []
    for w in ws:
        y = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
        kd.quant_gemv(x, w, y, scratch)
        singles.append(y)
    for rep in range(2):
        ys = [torch.full((rows,), float("nan"), dtype=torch.float32, device=dev) for _ in range(n)]
        kd.quant_gemv_multi(x, ws, ys, scratch)
        torch.cuda.synchronize()
        for a, b in zip(ys, singles):
            assert torch.equal(a, b)
    assert kd.device_status() == 0


def test_multi_matrix_call_rejects_mixed_shapes(kd):
    dev = torch.device("cuda:0")
    mk = lambda r: kd.QuantWeight.from_numpy(kd.ggml_pack.random_payload(kd.Q4_K, r, 256, 1), kd.Q4_K, r, 256, dev)
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(256), dtype=torch.uint8, device=dev)
    with pytest.raises(ValueError):
        kd.quant_gemv_multi(torch.zeros(256, device=dev), [mk(4), mk(6)],
                            [torch.zeros(4, device=dev), torch.zeros(6, device=dev)], scratch)


def test_launch_chaining_switch_does_not_change_results(kd):
    dev = torch.device("cuda:0")
    rows, K = 300, 4096
    w = kd.QuantWeight.from_numpy(kd.ggml_pack.random_payload(kd.Q4_K, rows, K, 77), kd.Q4_K, rows, K, dev)
    x = torch.randn(K, generator=torch.Generator().manual_seed(6)).to(dev)
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
    outs = []
    prev = kd.launch_chaining(-1)
    try:
        for on in (1, 0):
            kd.launch_chaining(on)
            assert kd.launch_chaining(-1) == on
            y = torch.empty(rows, dtype=torch.float32, device=dev)
            for _ in range(3):
                kd.quant_gemv(x, w, y, scratch)
            torch.cuda.synchronize()
            outs.append(y.clone())
    finally:
        kd.launch_chaining(prev)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_second_device_in_the_same_process(kd, port):
    """The per-kernel shared-memory attribute belongs to the (kernel, device) pair: a host thread that moves to a
    second GPU must get it set there too. Kernels with more than 48 KB of dynamic shared memory on both devices."""
    from oracle import oracle as O
    rows, K = 600, 4096
    packed = kd.ggml_pack.random_payload(kd.Q4_K, rows, K, 78)
    xh = torch.randn(K, generator=torch.Generator().manual_seed(7))
    ref, _ = port.gemv_int8(kd.Q4_K, O.aligned_copy(packed), rows, K, xh.numpy())
    for d in (0, 1, 0):
        dev = torch.device("cuda", d)
        with torch.cuda.device(dev):
            w = kd.QuantWeight.from_numpy(packed, kd.Q4_K, rows, K, dev)
            y = torch.empty(rows, dtype=torch.float32, device=dev)
            scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
            kd.quant_gemv(xh.to(dev), w, y, scratch)
            torch.cuda.synchronize(dev)
            assert np.abs(y.cpu().numpy() - ref).max() <= 1e-3 * np.abs(ref).max()
            assert kd.device_status() == 0
