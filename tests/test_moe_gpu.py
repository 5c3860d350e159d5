"""Parity of the router, the batched GEMM and the MoE feed-forward (through the C ABI) against the CPU
checker. Router: expert ids exactly equal, weights within 1e-5 (tests/Test_MoE.cpp:117). GEMM / MoE:
fp32 outputs within 1e-3 of max|Y| of the int8-aware checker (the reference's own int8 GEMV applied per
activation row; the reference has no batched int8 kernel)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"
TILE_KINDS = [3, 2, 1, 0]     # by measured crossover (default), tcgen05 + TMEM, mma.sync, CUDA-core dp4a
TILE_NAMES = {3: "auto", 2: "tcgen05", 1: "mma.sync", 0: "dp4a"}


@pytest.fixture(params=TILE_KINDS, ids=lambda k: TILE_NAMES[k])
def tile(kd, request):
    """Runs the test once per Q4_K tile kernel (explicit selection through the C ABI, restored afterwards)."""
    prev = kd.tile_kind(request.param)
    yield request.param
    kd.tile_kind(prev)


@pytest.fixture(params=[3, 2, 1], ids=lambda k: TILE_NAMES[k])
def tensor_tile(kd, request):
    prev = kd.tile_kind(request.param)
    yield request.param
    kd.tile_kind(prev)


def _route(kd, lg_t, bias_t, k, norm, scale, sig):
    T = lg_t.shape[0]
    idx = torch.full((T, k), -9, dtype=torch.int32, device=DEV)
    w = torch.full((T, k), float("nan"), dtype=torch.float32, device=DEV)
    kd.moe_route(lg_t.to(DEV), None if bias_t is None else bias_t.to(DEV), k, norm, scale, idx, w, sigmoid=sig)
    torch.cuda.synchronize()
    return idx.cpu().numpy(), w.cpu().numpy()


def test_router_golden(kd):
    g = np.load(os.path.join(GOLD, "moe_route.npz"))
    n = len([f for f in g.files if f.endswith("_cfg")])
    for c in range(n):
        k, norm, sig, bf16 = [int(v) for v in g[f"c{c}_cfg"]]
        dt = torch.bfloat16 if bf16 else torch.float32
        lg = torch.from_numpy(g[f"c{c}_logits"]).to(dt)
        bias = g[f"c{c}_bias"]
        bt = torch.from_numpy(bias).to(dt) if bias.size else None
        idx, w = _route(kd, lg, bt, k, bool(norm), float(g[f"c{c}_scale"][0]), bool(sig))
        assert np.array_equal(idx, g[f"c{c}_idx"]), c
        assert np.abs(w - g[f"c{c}_w"]).max() <= 1e-5, c


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (3, 6, 6), (64, 8, 2), (256, 128, 8), (7, 64, 4), (5, 1000, 9)])
def test_router_random_and_ties(kd, port, T, E, k):
    rng = np.random.default_rng(T * 1000 + E)
    lg = rng.standard_normal((T, E)).astype(np.float32)
    lg[0, : min(E, 5)] = 0.75            # ties keep the lower ids
    lg[-1, :] = -1.0                     # all equal
    bias = (rng.standard_normal(E) * 0.2).astype(np.float32)
    for dt in (torch.float32, torch.bfloat16):
        lgt = torch.from_numpy(lg).to(dt)
        for b in (None, bias):
            bt = None if b is None else torch.from_numpy(b).to(dt)
            for norm in (True, False):
                for sig in (False, True):
                    idx, w = _route(kd, lgt, bt, k, norm, 1.25, sig)
                    ri, rw = port.moe_route(lgt.float().numpy(), None if bt is None else bt.float().numpy(),
                                            k, norm, 1.25, sig)
                    assert np.array_equal(idx, ri)
                    assert np.abs(w - rw).max() <= 1e-5


def _experts(kd, E, H, F, seed, dtypes, payload="synth"):
    mk = (lambda dt, r, c, s: kd.ggml_pack.synth_weight(dt, r, c, s, std=0.05)) if payload == "synth" else \
        (lambda dt, r, c, s: kd.ggml_pack.random_payload(dt, r, c, s, scale_bits=0x1400))
    gate = [mk(dtypes[0], F, H, seed + e) for e in range(E)]
    up = [mk(dtypes[1], F, H, seed + 1000 + e) for e in range(E)]
    down = [mk(dtypes[2], H, F, seed + 2000 + e) for e in range(E)]
    return gate, up, down


def _tables(kd, gate, up, down, dtypes, H, F):
    mkq = lambda lst, dt, r, c: [kd.QuantWeight.from_numpy(a, dt, r, c, DEV) for a in lst]
    return (kd.make_quant_weight_table(mkq(gate, dtypes[0], F, H), "gate"),
            kd.make_quant_weight_table(mkq(up, dtypes[1], F, H), "up"),
            kd.make_quant_weight_table(mkq(down, dtypes[2], H, F), "down"))


def _ffn(kd, X_t, tabs, idx, wts, y_dtype, e_first=0, e_count=None):
    T, H = X_t.shape
    S = idx.shape[1]
    F, E = tabs[0].rows, tabs[0].size()
    ws = torch.zeros(kd.moe_ffn_workspace_bytes(T, S, H, F, E), dtype=torch.uint8, device=DEV)
    Y = torch.full((T, H), float("nan"), dtype=y_dtype, device=DEV)
    kd.moe_ffn(X_t.to(DEV), *tabs, torch.from_numpy(idx).to(DEV), torch.from_numpy(wts).to(DEV), Y, ws,
               e_first, e_count)
    torch.cuda.synchronize()
    assert kd.device_status() == 0
    return Y.float().cpu().numpy()


@pytest.mark.parametrize("dtypes", [(O.Q4_K, O.Q4_K, O.Q4_K), (O.Q4_K, O.Q4_K, O.Q6_K), (O.Q8_0, O.Q8_0, O.Q8_0),
                                    (O.Q6_K, O.Q6_K, O.Q4_K)])
@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
def test_moe_ffn_small(kd, port, dtypes, x_dtype, tile):
    if dtypes != (O.Q4_K, O.Q4_K, O.Q4_K) and tile != 3:
        pytest.skip("the tile kind only matters for all-Q4_K experts")
    E, H, F, T, S = 6, 512, 256, 21, 3
    gate, up, down = _experts(kd, E, H, F, 40, dtypes)
    tabs = _tables(kd, gate, up, down, dtypes, H, F)
    rng = np.random.default_rng(5)
    X = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(x_dtype)
    idx = np.stack([rng.permutation(E)[:S] for _ in range(T)]).astype(np.int32)
    wts = rng.random((T, S)).astype(np.float32)
    idx[0, 1] = -1          # dead slots contribute nothing (tests/Test_MoeDecode.cpp:368-419)
    idx[1, 0] = E
    wts[2, 2] = 0.0         # zero-weight slot is skipped
    idx[3, :] = -1          # a token with no live slot gets zeros (Y is assigned, not accumulated)
    al = lambda lst: [O.aligned_copy(a) for a in lst]
    ref = port.moe_ffn_int8(X.float().numpy(), al(gate), al(up), al(down), idx, wts, F, dtypes,
                            bf16=(x_dtype == torch.bfloat16))
    got = _ffn(kd, X, tabs, idx, wts, torch.float32)
    assert np.all(got[3] == 0.0)
    assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()
    if x_dtype == torch.bfloat16:       # Scalar output: within one bf16 ulp of the rounded checker value
        gb = _ffn(kd, X, tabs, idx, wts, torch.bfloat16)
        want = O.bf16_round(ref)
        assert np.all(np.abs(gb - want) <= np.abs(want) * 2.0 ** -7 + 1e-3 * np.abs(ref).max())
    # expert-parallel shards: partial outputs of disjoint expert ranges add up to the full result
    part = _ffn(kd, X, tabs, idx, wts, torch.float32, 0, 2) + _ffn(kd, X, tabs, idx, wts, torch.float32, 2, 4)
    assert np.abs(part - ref).max() <= 1e-3 * np.abs(ref).max()


def test_moe_decode_one_token_vs_reference_fp_kernel(kd, port):
    """One token against the reference's fused fp-path kernels (golden fixture): the int8 path stays within
    the documented ~1% activation-rounding distance; against the int8-aware checker within 1e-3."""
    g = np.load(os.path.join(GOLD, "moe_decode_fp.npz"))
    E, H, F, S = [int(v) for v in g["meta"]]
    dt3 = (O.Q4_K,) * 3
    lst = lambda a: [a[e] for e in range(E)]
    tabs = _tables(kd, lst(g["gate"]), lst(g["up"]), lst(g["down"]), dt3, H, F)
    X = torch.from_numpy(g["x"]).to(torch.bfloat16)[None, :]
    idx, wts = g["idx"][None, :], g["wts"][None, :]
    ws = torch.zeros(kd.moe_ffn_workspace_bytes(1, S, H, F, E), dtype=torch.uint8, device=DEV)
    Y = torch.empty((1, H), dtype=torch.float32, device=DEV)
    act = torch.empty((S, F), dtype=torch.bfloat16, device=DEV)
    kd.quant_moe_decode(X.to(DEV), *tabs, torch.from_numpy(idx).to(DEV), torch.from_numpy(wts).to(DEV), act, Y, ws)
    torch.cuda.synchronize()
    got = Y.cpu().numpy()[0]
    assert np.abs(got - g["Y"]).max() <= 3e-2 * np.abs(g["Y"]).max()
    al = lambda a: [O.aligned_copy(a[e]) for e in range(E)]
    ref = port.moe_ffn_int8(g["x"][None, :], al(g["gate"]), al(g["up"]), al(g["down"]), idx, wts, F, dt3, bf16=True)
    assert np.abs(got - ref[0]).max() <= 1e-3 * np.abs(ref).max()
    with pytest.raises(ValueError, match="expected one row"):          # tests/Test_MoeDecode.cpp:423-455
        kd.quant_moe_decode(torch.zeros(2, H, device=DEV), *tabs, torch.from_numpy(idx).to(DEV),
                            torch.from_numpy(wts).to(DEV), act, Y, ws)
    with pytest.raises(ValueError, match="act scratch too small"):
        kd.quant_moe_decode(X.to(DEV), *tabs, torch.from_numpy(idx).to(DEV), torch.from_numpy(wts).to(DEV),
                            act[:1], Y, ws)


@pytest.mark.parametrize("dtypes", [(O.Q5_K, O.Q5_K, O.Q5_K), (O.Q4_K, O.Q4_K, O.Q5_K)])
def test_moe_ffn_q5k_experts(kd, port, dtypes):
    """Q5_K expert matrices (random payloads: there is no Q5_K encoder here) through the batched kernels."""
    E, H, F, T, S = 5, 512, 256, 19, 2
    gate, up, down = _experts(kd, E, H, F, 70, dtypes, payload="random")
    tabs = _tables(kd, gate, up, down, dtypes, H, F)
    rng = np.random.default_rng(9)
    X = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32))
    idx = np.stack([rng.permutation(E)[:S] for _ in range(T)]).astype(np.int32)
    wts = rng.random((T, S)).astype(np.float32)
    al = lambda lst: [O.aligned_copy(a) for a in lst]
    ref = port.moe_ffn_int8(X.numpy(), al(gate), al(up), al(down), idx, wts, F, dtypes, bf16=False)
    got = _ffn(kd, X, tabs, idx, wts, torch.float32)
    assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()


@pytest.mark.parametrize("dtype,N,K", [(O.Q4_K, 300, 1024), (O.Q6_K, 130, 2048), (O.Q8_0, 257, 512), (O.Q5_K, 200, 1024)])
@pytest.mark.parametrize("M", [1, 2, 3, 5, 16, 17, 32, 33, 70])
def test_quant_gemm_rows_equal_gemv(kd, port, dtype, N, K, M, tile):
    if dtype != O.Q4_K and tile not in (3, 0):
        pytest.skip("the tile kind only matters for Q4_K")
    packed = kd.ggml_pack.random_payload(dtype, N, K, N + K)
    w = kd.QuantWeight.from_numpy(packed, dtype, N, K, DEV)
    X = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16)
    Y = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ws = torch.zeros(kd.quant_gemm_workspace_bytes(M, K), dtype=torch.uint8, device=DEV)
    kd.quant_gemm(X.to(DEV), w, Y, ws)
    torch.cuda.synchronize()
    host = O.aligned_copy(packed)
    got = Y.cpu().numpy()
    for m in range(M):
        ref, _ = port.gemv_int8(dtype, host, N, K, X[m].float().numpy())
        assert np.abs(got[m] - ref).max() <= 1e-3 * np.abs(ref).max()


def _full_layer(kd, port, E, k, H, F, T, seed):
    dt3 = (O.Q4_K,) * 3
    gate, up, down = _experts(kd, E, H, F, seed, dt3, payload="random")
    tabs = _tables(kd, gate, up, down, dt3, H, F)
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(T, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g).to(torch.bfloat16)
    idx_t = torch.empty((T, k), dtype=torch.int32, device=DEV)
    w_t = torch.empty((T, k), dtype=torch.float32, device=DEV)
    kd.moe_route(logits.to(DEV), None, k, True, 1.0, idx_t, w_t)
    torch.cuda.synchronize()
    idx, wts = idx_t.cpu().numpy(), w_t.cpu().numpy()
    ri, rw = port.moe_route(logits.float().numpy(), None, k, True)
    assert np.array_equal(idx, ri) and np.abs(wts - rw).max() <= 1e-5
    got = _ffn(kd, X, tabs, idx, wts, torch.float32)
    al = lambda lst: [O.aligned_copy(a) for a in lst]
    ref = port.moe_ffn_int8(X.float().numpy(), al(gate), al(up), al(down), idx, wts, F, dt3, bf16=True)
    assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()


def test_fine_grained_layer_full_size(kd, port, tensor_tile):
    """One layer of the 128-expert / top-8 / hidden 2048 / FFN 768 / 256-token configuration."""
    _full_layer(kd, port, 128, 8, 2048, 768, 256, 77)


def test_mixtral_style_layer_full_size(kd, port, tensor_tile):
    """8 experts / top-2 / hidden 4096 / FFN 14336 / 64 tokens: the coarse MoE configuration at its full
    shapes (792.7 MB of packed expert bytes)."""
    _full_layer(kd, port, 8, 2, 4096, 14336, 64, 78)


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32])
def test_batched_sweep_at_the_llama_ffn_shape(kd, port, M, tensor_tile):
    """Q4_K 14336 x 4096 with 1..32 activation rows: every output row equals the int8 GEMV of its
    activation row (the reference has no batched int8 kernel: src/KokkosDNN_GGUF.hpp:2564-2593 is fp)."""
    N, K = 14336, 4096
    packed = kd.ggml_pack.random_payload(O.Q4_K, N, K, 4242)
    w = kd.QuantWeight.from_numpy(packed, O.Q4_K, N, K, DEV)
    X = torch.randn(M, K, generator=torch.Generator().manual_seed(100 + M)).to(torch.bfloat16)
    Y = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ws = torch.zeros(kd.quant_gemm_workspace_bytes(M, K), dtype=torch.uint8, device=DEV)
    kd.quant_gemm(X.to(DEV), w, Y, ws)
    torch.cuda.synchronize()
    assert kd.device_status() == 0
    host = O.aligned_copy(packed)
    got = Y.cpu().numpy()
    for m in range(M):
        ref, _ = port.gemv_int8(O.Q4_K, host, N, K, X[m].float().numpy())
        assert np.abs(got[m] - ref).max() <= 1e-3 * np.abs(ref).max()


@pytest.mark.parametrize("N,K,M", [(128, 256, 1), (300, 1024, 5), (257, 2048, 32), (130, 512, 45)])
def test_tcgen05_sub_block_dots_bit_exact(kd, port, N, K, M):
    """The int32 sub-block dots the PRODUCTION tile kernel's tensor-core instructions leave in tensor memory,
    dumped by the kernel itself, equal the reference's unit integers summed per 32-element sub-block
    (src/KokkosDNN_GGUFGemvInt8.hpp:359-388: dotA / dotB of the two half units of a sub-block)."""
    prev = kd.tile_kind(2)
    try:
        packed = kd.ggml_pack.random_payload(O.Q4_K, N, K, N * 7 + K)
        w = kd.QuantWeight.from_numpy(packed, O.Q4_K, N, K, DEV)
        X = torch.randn(M, K, generator=torch.Generator().manual_seed(M + K))
        Y = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
        ws = torch.zeros(kd.quant_gemm_workspace_bytes(M, K), dtype=torch.uint8, device=DEV)
        dots = kd.quant_gemm_dots(X.to(DEV), w, Y, ws).cpu().numpy()
        torch.cuda.synchronize()
        assert kd.device_status() == 0
    finally:
        kd.tile_kind(prev)
    host = O.aligned_copy(packed)
    for m in range(M):
        ref, staging = port.gemv_int8(O.Q4_K, host, N, K, X[m].numpy())
        ints, _ = port.unit_table(O.Q4_K, host, N, K, staging)      # [N, K/32 units, {dotA, dotB}]
        u = ints.reshape(N, K // 256, 4, 2, 2)                      # [row, block, iter, half, A/B]
        want = u.sum(axis=3).reshape(N, K // 32)                    # sub-block 2*iter = A, 2*iter+1 = B
        assert np.array_equal(dots[m], want), m
        assert np.abs(Y[m].cpu().numpy() - ref).max() <= 1e-3 * np.abs(ref).max()


def test_duplicate_expert_in_one_token(kd, port, tensor_tile):
    """idx may name the same expert twice for one token (the reference treats every slot on its own,
    src/KokkosDNN_GGUF.hpp:2106-2110): both slots count."""
    E, H, F, T, S = 4, 512, 256, 9, 3
    dt3 = (O.Q4_K,) * 3
    gate, up, down = _experts(kd, E, H, F, 90, dt3)
    tabs = _tables(kd, gate, up, down, dt3, H, F)
    rng = np.random.default_rng(12)
    X = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32))
    idx = np.stack([rng.permutation(E)[:S] for _ in range(T)]).astype(np.int32)
    idx[2, 1] = idx[2, 0]
    idx[5, :] = 3
    wts = rng.random((T, S)).astype(np.float32)
    al = lambda lst: [O.aligned_copy(a) for a in lst]
    ref = port.moe_ffn_int8(X.numpy(), al(gate), al(up), al(down), idx, wts, F, dt3, bf16=False)
    got = _ffn(kd, X, tabs, idx, wts, torch.float32)
    assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()
