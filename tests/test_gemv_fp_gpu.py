"""Parity of kdnn_b200_quant_gemv_fp against the reference's staging-free quant_gemv (the fp path,
src/KokkosDNN_GGUF.hpp:2394-2493). The weights are dequantized exactly as the reference does; only the
order of the fp32 additions differs, so the bars are the reference's own ones for this path
(tests/Test_GGUF.cpp:744-752: 1e-4 * sum|terms| + 1e-3 against double accumulation) and 1e-3 * max|y|
against the reference's result; bf16 outputs within one bf16 ulp."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
TYPES = [O.Q4_K, O.Q5_K, O.Q6_K, O.Q8_0]


def _fp(kd, port, ref, dtype, rows, cols, seed, x_dtype=torch.float32, y_dtype=torch.float32):
    packed = kd.ggml_pack.random_payload(dtype, rows, cols, seed)
    w = kd.QuantWeight.from_numpy(packed, dtype, rows, cols, "cuda:0")
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(cols, generator=g).to(x_dtype)
    y = torch.full((rows,), float("nan"), dtype=y_dtype, device="cuda:0")
    kd.quant_gemv_fp(x.to("cuda:0"), w, y)
    torch.cuda.synchronize()
    got = y.float().cpu().numpy()
    host = O.aligned_copy(packed)
    xf = x.float().numpy()
    want, _ = ref.quant_gemv(dtype, host, rows, cols, xf, bf16=(x_dtype == torch.bfloat16), int8=False)
    scale = max(np.abs(want).max(), 1e-30)
    if y_dtype == torch.float32 and x_dtype == torch.float32:
        assert np.abs(got - want).max() <= 1e-3 * scale
        acc, mag = port.gemv_dequant_f64(dtype, host, rows, cols, xf)
        assert np.all(np.abs(got - acc) <= 1e-4 * mag + 1e-3)
    else:
        ulp = np.maximum(np.abs(want), 1e-30) * 2.0 ** -7
        assert np.all(np.abs(got - want) <= ulp + 1e-3 * scale * (y_dtype == torch.float32))


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("rows,cols", [(1, 256), (7, 512), (65, 2048), (300, 4096), (33, 14336)])
def test_fp_path_matches_reference(kd, port, ref, dtype, rows, cols):
    _fp(kd, port, ref, dtype, rows, cols, 2000 + rows + cols)


@pytest.mark.parametrize("dtype", TYPES)
def test_fp_path_bf16(kd, port, ref, dtype):
    _fp(kd, port, ref, dtype, 40, 2048, 31, torch.bfloat16, torch.bfloat16)


def test_fp_path_q8_0_ragged_and_large(kd, port, ref):
    _fp(kd, port, ref, O.Q8_0, 9, 32 * 13, 5)
    _fp(kd, port, ref, O.Q4_K, 5000, 1024, 6)


def test_fp_path_argument_errors(kd):
    packed = kd.ggml_pack.random_payload(O.Q4_K, 4, 512, 1)
    w = kd.QuantWeight.from_numpy(packed, O.Q4_K, 4, 512, "cuda:0")
    with pytest.raises(ValueError):
        kd.quant_gemv_fp(torch.zeros(256, device="cuda:0"), w, torch.zeros(4, device="cuda:0"))
    with pytest.raises(ValueError):
        kd.quant_gemv_fp(torch.zeros(512, device="cuda:0"), kd.QuantWeight(w.data, 99, 4, 512), torch.zeros(4, device="cuda:0"))
