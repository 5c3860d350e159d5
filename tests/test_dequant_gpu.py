"""Parity of kdnn_b200_dequant_to_dense against the reference's dequant_to_dense
(src/KokkosDNN_GGUF.hpp:2839-2934) and the checker's per-row dequantizers
(:300-384). Bars: fp32 outputs bit-exact; bf16 outputs equal the reference's bf16
bit pattern. Error behaviour as tests/Test_GGUF.cpp exercises it for this operator
(dimension mismatch, ragged K)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
TYPES = [O.Q4_K, O.Q5_K, O.Q6_K, O.Q8_0]


def _payload(kd, dtype, rows, cols, seed):
    if dtype == O.Q5_K:   # no encoder for Q5_K: random bytes with sane fp16 scales
        rng = np.random.default_rng(seed)
        raw = rng.integers(0, 256, size=(rows * cols // 256, 176), dtype=np.uint8)
        raw[:, 0:2] = np.frombuffer(np.float16(2.0 ** -6).tobytes(), dtype=np.uint8)
        raw[:, 2:4] = np.frombuffer(np.float16(2.0 ** -7).tobytes(), dtype=np.uint8)
        return raw.reshape(-1)
    return kd.ggml_pack.random_payload(dtype, rows, cols, seed)


@pytest.mark.parametrize("dtype", TYPES)
@pytest.mark.parametrize("rows,cols", [(1, 256), (7, 512), (33, 2048), (5, 6656)])
def test_fp32_bit_exact(kd, port, ref, dtype, rows, cols):
    packed = _payload(kd, dtype, rows, cols, 1000 + rows + cols)
    w = kd.QuantWeight.from_numpy(packed, dtype, rows, cols, "cuda:0")
    Y = torch.full((rows, cols), float("nan"), dtype=torch.float32, device="cuda:0")
    kd.dequant_to_dense(w, Y)
    torch.cuda.synchronize()
    got = Y.cpu().numpy()
    host = O.aligned_copy(packed)
    assert np.array_equal(got.view(np.uint32), port.dequant_rows(dtype, host, rows, cols).view(np.uint32))
    assert np.array_equal(got.view(np.uint32), ref.dequant_to_dense(dtype, host, rows, cols).view(np.uint32))


@pytest.mark.parametrize("dtype", TYPES)
def test_bf16_and_pitched_output(kd, ref, dtype):
    rows, cols = 9, 1024
    packed = _payload(kd, dtype, rows, cols, 77)
    w = kd.QuantWeight.from_numpy(packed, dtype, rows, cols, "cuda:0")
    want = ref.dequant_to_dense(dtype, O.aligned_copy(packed), rows, cols, bf16=True)
    big = torch.zeros((rows, cols + 24), dtype=torch.bfloat16, device="cuda:0")
    Y = big[:, 8:8 + cols]            # pitched view, 16-byte aligned rows
    kd.dequant_to_dense(w, Y)
    odd = torch.zeros((rows, cols + 3), dtype=torch.bfloat16, device="cuda:0")
    Z = odd[:, 1:1 + cols]            # rows that are not 16-byte aligned: scalar stores
    kd.dequant_to_dense(w, Z)
    torch.cuda.synchronize()
    assert np.array_equal(Y.float().cpu().numpy(), want)
    assert np.array_equal(Z.float().cpu().numpy(), want)
    assert float(big[:, :8].abs().max()) == 0.0 and float(big[:, 8 + cols:].abs().max()) == 0.0


def test_q8_0_cols_not_multiple_of_256(kd, port):
    rows, cols = 6, 32 * 11
    packed = kd.ggml_pack.random_payload(O.Q8_0, rows, cols, 5)
    w = kd.QuantWeight.from_numpy(packed, O.Q8_0, rows, cols, "cuda:0")
    Y = torch.empty((rows, cols), dtype=torch.float32, device="cuda:0")
    kd.dequant_to_dense(w, Y)
    torch.cuda.synchronize()
    assert np.array_equal(Y.cpu().numpy(), port.dequant_rows(O.Q8_0, O.aligned_copy(packed), rows, cols))


def test_argument_errors(kd):
    packed = kd.ggml_pack.random_payload(O.Q4_K, 4, 512, 1)
    w = kd.QuantWeight.from_numpy(packed, O.Q4_K, 4, 512, "cuda:0")
    with pytest.raises(ValueError):
        kd.dequant_to_dense(w, torch.empty((4, 256), dtype=torch.float32, device="cuda:0"))
    with pytest.raises(ValueError):
        kd.dequant_to_dense(kd.QuantWeight(w.data, 99, 4, 512), torch.empty((4, 512), dtype=torch.float32, device="cuda:0"))
    empty = kd.QuantWeight(torch.empty(0, dtype=torch.uint8, device="cuda:0"), O.Q4_K, 0, 512)
    kd.dequant_to_dense(empty, torch.empty((0, 512), dtype=torch.float32, device="cuda:0"))   # no launch, no error
