"""The allocation-free GEMV entry point (kdnn_b200_quant_gemv_noalloc) against the regular one.

Some hosts cannot give the library a staging buffer and are not allowed to allocate one: a runtime that
owns all device memory and bans cudaMalloc in plug-ins, or a decode loop that must stay away from the
allocator. For them the staging sits in a fixed array inside the library. This test calls that entry
point through the C ABI twice in a row (different K and different activations, so the second call runs on
top of the first call's left-over staging) and requires the same results as kdnn_b200_quant_gemv, which
is itself checked against the CPU checker elsewhere. Collected last, so a failure here cannot hide other
tests under `pytest -x`; it also passes when run alone in a fresh process.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_matches_regular_entry_point_twice(kd):
    dev = torch.device("cuda:0")
    cases = [(kd.Q4_K, 1500, 4096, 21), (kd.Q6_K, 300, 2048, 22), (kd.Q8_0, 129, 1024, 23)]
    for dtype, rows, K, seed in cases:                      # consecutive calls share the built-in staging
        packed = kd.ggml_pack.random_payload(dtype, rows, K, seed)
        w = kd.QuantWeight.from_numpy(packed, dtype, rows, K, dev)
        for rep in range(2):
            x = torch.randn(K, generator=torch.Generator().manual_seed(seed * 10 + rep)).to(torch.bfloat16).to(dev)
            y_ref = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
            scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
            kd.quant_gemv(x, w, y_ref, scratch)
            y = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
            kd.quant_gemv_noalloc(x, w, y)
            torch.cuda.synchronize()
            a, b = y.cpu().numpy(), y_ref.cpu().numpy()
            assert np.all(np.isfinite(a))
            # tolerance of the GEMV parity tests (1e-3 of max|y|); the two paths run the same kernels
            assert np.abs(a - b).max() <= 1e-3 * np.abs(b).max()
    assert kd.device_status() == 0


@pytest.mark.parametrize("case", ["q6k_ragged_k", "q8_0_ragged_k", "q4k_plain_loads", "q5k_plain_loads"])
def test_noalloc_plain_load_kernels_read_the_builtin_staging(kd, port, case):
    """The plain-load kernels are the ones that really READ the staging (a first kernel writes the quantized
    activation row there, the GEMV kernel loads it back), so here the built-in array is used as scratch in
    earnest: shapes the streaming kernels do not cover (Q6_K with K % 2048 != 0, Q8_0 with K % 256 != 0) and
    the plain-load kernels selected through the layout struct, two calls in a row, against the CPU checker."""
    from oracle import oracle as O
    dev = torch.device("cuda:0")
    dtype, rows, K, layout = {"q6k_ragged_k": (kd.Q6_K, 77, 2304, None), "q8_0_ragged_k": (kd.Q8_0, 130, 1056, None),
                              "q4k_plain_loads": (kd.Q4_K, 65, 1024, {"kernel": kd.KERNEL_PLAIN_LOADS}),
                              "q5k_plain_loads": (kd.Q5_K, 33, 512, {"kernel": kd.KERNEL_PLAIN_LOADS})}[case]
    packed = kd.ggml_pack.random_payload(dtype, rows, K, 31)
    w = kd.QuantWeight.from_numpy(packed, dtype, rows, K, dev)
    host = O.aligned_copy(packed)
    for rep in range(2):
        xh = torch.randn(K, generator=torch.Generator().manual_seed(310 + rep))
        y = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
        kd.quant_gemv_noalloc(xh.to(dev), w, y, layout)
        torch.cuda.synchronize()
        ref, _ = port.gemv_int8(dtype, host, rows, K, xh.numpy())
        assert np.abs(y.cpu().numpy() - ref).max() <= 1e-3 * np.abs(ref).max()
    assert kd.device_status() == 0


@pytest.mark.parametrize("dtype_name", ["Q4_K", "Q6_K", "Q8_0"])
def test_noalloc_at_its_column_limit(kd, port, dtype_name):
    """K = 32768 fills the built-in staging to its last byte (both entry points, against the CPU checker)."""
    from oracle import oracle as O
    dev = torch.device("cuda:0")
    dtype, rows, K = getattr(kd, dtype_name), 6, kd.NOALLOC_MAX_COLS
    packed = kd.ggml_pack.random_payload(dtype, rows, K, 41)
    w = kd.QuantWeight.from_numpy(packed, dtype, rows, K, dev)
    xh = torch.randn(K, generator=torch.Generator().manual_seed(42))
    ref, _ = port.gemv_int8(dtype, O.aligned_copy(packed), rows, K, xh.numpy())
    y = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
    kd.quant_gemv_noalloc(xh.to(dev), w, y)
    y2 = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
    kd.quant_gemv(xh.to(dev), w, y2, scratch)
    torch.cuda.synchronize()
    for got in (y, y2):
        assert np.abs(got.cpu().numpy() - ref).max() <= 1e-3 * np.abs(ref).max()
    assert kd.device_status() == 0


def test_noalloc_declines_strided_views(kd):
    dev = torch.device("cuda:0")
    w = kd.QuantWeight.from_numpy(kd.ggml_pack.random_payload(kd.Q4_K, 4, 256, 1), kd.Q4_K, 4, 256, dev)
    with pytest.raises(kd.Declined):
        kd.quant_gemv_noalloc(torch.zeros(512, device=dev)[::2], w, torch.zeros(4, device=dev))


def test_noalloc_rejects_k_beyond_the_builtin_staging(kd):
    dev = torch.device("cuda:0")
    K = kd.NOALLOC_MAX_COLS + 256
    w = kd.QuantWeight(torch.zeros(kd.ggml_row_bytes(kd.Q4_K, K), dtype=torch.uint8, device=dev), kd.Q4_K, 1, K)
    with pytest.raises(ValueError, match="32768"):
        kd.quant_gemv_noalloc(torch.zeros(K, device=dev), w, torch.zeros(1, device=dev))
