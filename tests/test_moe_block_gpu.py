"""The MoE block in four launches (kdnn_b200_moe_block) and the reference's small MoE operators, through the
C ABI, against the CPU checker.

Router: ids equal, weights within 1e-5 (tests/Test_MoE.cpp:117). Feed-forward: fp32 outputs within 1e-3 of
max|Y| of the int8-aware checker fed with the routing the block produced. Residual add: exact. Norm: against the
reference's own rmsnorm_noscale (src/KokkosDNN_RMSNorm.hpp:347-361) when its library is present, to fp32
reassociation / one bf16 ulp.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _experts(kd, E, H, F, seed):
    mk = lambda r, c, s: kd.ggml_pack.random_payload(O.Q4_K, r, c, s, scale_bits=0x1400)
    return ([mk(F, H, seed + e) for e in range(E)], [mk(F, H, seed + 1000 + e) for e in range(E)],
            [mk(H, F, seed + 2000 + e) for e in range(E)])


def _tables(kd, gate, up, down, H, F):
    mkq = lambda lst, r, c: [kd.QuantWeight.from_numpy(a, O.Q4_K, r, c, DEV) for a in lst]
    return (kd.make_quant_weight_table(mkq(gate, F, H), "gate"), kd.make_quant_weight_table(mkq(up, F, H), "up"),
            kd.make_quant_weight_table(mkq(down, H, F), "down"))


def _block_case(kd, port, E, k, H, F, T, dtype, seed, kind=3, sigmoid=False, bias=False, ref=None):
    prev = kd.tile_kind(kind)
    try:
        gate, up, down = _experts(kd, E, H, F, seed)
        tabs = _tables(kd, gate, up, down, H, F)
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(T, H, generator=g).to(dtype)
        h = torch.randn(T, H, generator=g).to(dtype)
        rw = (torch.randn(E, H, generator=g) / H ** 0.5).to(dtype)
        rb = (torch.randn(E, generator=g) * 0.1).to(dtype) if bias else None
        ws = torch.zeros(kd.moe_block_workspace_bytes(T, 1, k, H, F, E, True), dtype=torch.uint8, device=DEV)
        y = torch.full((T, H), float("nan"), dtype=torch.float32, device=DEV)
        h2 = torch.empty((T, H), dtype=dtype, device=DEV)
        x2 = torch.empty((T, H), dtype=dtype, device=DEV)
        for rep in range(2):     # the second call runs on the first call's left-over workspace
            y.fill_(float("nan"))
            kd.moe_block(x.to(DEV), rw.to(DEV), None if rb is None else rb.to(DEV), k, True, 1.0, *tabs, ws, y=y,
                         resid=h.to(DEV), h_out=h2, xn_out=x2, sigmoid=sigmoid)
            idx_t, w_t = kd.moe_block_routing(ws, T, 1, k, H, F, E)
            torch.cuda.synchronize()
            assert kd.device_status() == 0
            idx, wts = idx_t.cpu().numpy(), w_t.cpu().numpy()
            # router: logits in the Scalar type, then the reference's selection
            logits = (x.float() @ rw.float().t()).to(dtype).float().numpy()
            ri, rwt = port.moe_route(logits, None if rb is None else rb.float().numpy(), k, True, 1.0, sigmoid)
            assert np.array_equal(idx, ri)
            assert np.abs(wts - rwt).max() <= 1e-5
            al = lambda lst: [O.aligned_copy(a) for a in lst]
            yref = port.moe_ffn_int8(x.float().numpy(), al(gate), al(up), al(down), idx, wts, F, (O.Q4_K,) * 3,
                                     bf16=(dtype == torch.bfloat16))
            got = y.cpu().numpy()
            assert np.abs(got - yref).max() <= 1e-3 * np.abs(yref).max()
            # residual add: Scalar(float(h) + y), exact
            want_h = (h.float() + y.cpu()).to(dtype)
            assert torch.equal(h2.cpu(), want_h)
            # un-scaled RMS norm of the new residual stream
            hf = want_h.float().numpy()
            if ref is not None:
                want_x = ref.rmsnorm_noscale(hf, 1e-6, bf16=(dtype == torch.bfloat16))
            else:
                want_x = hf / np.sqrt((hf.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-6)
            gx = x2.float().cpu().numpy()
            tol = 2.0 ** -7 if dtype == torch.bfloat16 else 1e-5
            assert np.all(np.abs(gx - want_x) <= tol * np.maximum(np.abs(want_x), 1e-3))
    finally:
        kd.tile_kind(prev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", [3, 2, 1], ids=["auto", "tcgen05", "mma.sync"])
def test_moe_block_small(kd, port, dtype, kind):
    ref = O.Ref() if O.Ref.available() else None
    _block_case(kd, port, 8, 2, 512, 512, 13, dtype, 11, kind, ref=ref)


def test_moe_block_sigmoid_router_with_bias(kd, port):
    _block_case(kd, port, 16, 4, 512, 256, 9, torch.float32, 12, sigmoid=True, bias=True)


@pytest.mark.parametrize("kind", [3, 2], ids=["auto", "tcgen05"])
def test_moe_block_fine_grained_full_size(kd, port, kind):
    """128 experts / top-8 / hidden 2048 / FFN 768 / 256 tokens: one block of the benchmark's stack."""
    _block_case(kd, port, 128, 8, 2048, 768, 256, torch.float32, 13, kind)


def test_peer_that_never_signals_ends_in_a_status_not_a_hang(kd):
    """Failure injection on the host: the block is called as rank 0 of 2 while nobody runs rank 1 (its launch is
    simply never made; its region is a plain buffer on this GPU). Every device-side wait for the peer is bounded:
    the call returns, the status word says KDNN_ERR_DEVICE_WAIT, and the next ordinary call works."""
    E, k, H, F, Tl = 4, 2, 512, 256, 4
    gate, up, down = _experts(kd, E, H, F, 21)
    tabs = _tables(kd, gate, up, down, H, F)
    nbytes = kd.MoeExchange.region_bytes(Tl, 2, k, H)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(2)]
    ex = kd.MoeExchange.local(0, 2, bufs, wait_ns=20_000_000)       # 20 ms per wait
    x = torch.randn(Tl, H, generator=torch.Generator().manual_seed(1)).to(DEV)
    rw = torch.randn(E, H, generator=torch.Generator().manual_seed(2)).to(DEV)
    ws = torch.zeros(kd.moe_block_workspace_bytes(Tl, 2, k, H, F, E, False), dtype=torch.uint8, device=DEV)
    y = torch.zeros((Tl, H), dtype=torch.float32, device=DEV)
    kd.moe_block(x, rw, None, k, True, 1.0, *tabs, ws, y=y, expert_first=0, expert_count=2, exchange=ex)
    torch.cuda.synchronize()
    assert kd.device_status() == kd.KDNN_ERR_DEVICE_WAIT
    assert kd.device_status() == 0                                     # reading the status clears it
    ws1 = torch.zeros(kd.moe_block_workspace_bytes(Tl, 1, k, H, F, E, True), dtype=torch.uint8, device=DEV)
    kd.moe_block(x, rw, None, k, True, 1.0, *tabs, ws1, y=y)
    torch.cuda.synchronize()
    assert kd.device_status() == 0 and bool(torch.isfinite(y).all())


# ---- the reference's small MoE operators (tests/Test_MoE.cpp:201-341) -------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_moe_operators(kd, dtype):
    ref = O.Ref() if O.Ref.available() else None
    bf16 = dtype == torch.bfloat16
    rng = np.random.default_rng(3)
    T, K, D = 7, 3, 130
    eo = torch.from_numpy(rng.standard_normal((T, K, D)).astype(np.float32)).to(dtype)
    w = torch.from_numpy(rng.random((T, K)).astype(np.float32))
    y = torch.empty((T, D), dtype=dtype, device=DEV)
    kd.moe_expert_weighted_sum(eo.to(DEV), w.to(DEV), y)
    want = ref.moe_weighted_sum(eo.float().numpy(), w.numpy(), bf16) if ref else \
        (w.numpy()[:, :, None] * eo.float().numpy()).sum(1)
    tol = 2.0 ** -7 if bf16 else 1e-6
    assert np.all(np.abs(y.float().cpu().numpy() - want) <= tol * np.maximum(np.abs(want), 1.0))
    # gather: exact
    C_, N = 11, 6
    src = torch.from_numpy(rng.standard_normal((C_, D)).astype(np.float32)).to(dtype)
    rows = torch.tensor([5, 0, 10, 3, 3, 7], dtype=torch.int32)
    dst = torch.empty((N, D), dtype=dtype, device=DEV)
    kd.moe_gather_rows(src.to(DEV), rows.to(DEV), dst)
    assert torch.equal(dst.cpu(), src[rows.long()])
    # scatter-add: dst rows keep what they had plus w * src, cast per add
    base = torch.from_numpy(rng.standard_normal((C_, D)).astype(np.float32)).to(dtype)
    urows = torch.tensor([9, 2, 4], dtype=torch.int32)
    sv = torch.from_numpy(rng.standard_normal((3, D)).astype(np.float32)).to(dtype)
    wv = torch.tensor([0.5, -1.25, 2.0])
    d2 = base.clone().to(DEV)
    kd.moe_scatter_add_weighted(sv.to(DEV), urows.to(DEV), wv.to(DEV), d2)
    want = base.clone().float()
    want[urows.long()] = (base[urows.long()].float() + wv[:, None] * sv.float())
    want = want.to(dtype)
    if ref:
        want_ref = ref.moe_scatter_add_weighted(sv.float().numpy(), urows.numpy(), wv.numpy(), base.float().numpy(), bf16)
        assert np.array_equal(want.float().numpy(), want_ref)
    assert torch.equal(d2.cpu(), want)
    # swiglu
    Tn, Fn = 5, 200
    gt = torch.from_numpy(rng.standard_normal((Tn, Fn)).astype(np.float32) * 3).to(dtype)
    ut = torch.from_numpy(rng.standard_normal((Tn, Fn)).astype(np.float32)).to(dtype)
    out = torch.empty((Tn, Fn), dtype=dtype, device=DEV)
    kd.swiglu(gt.to(DEV), ut.to(DEV), out)
    want = ref.swiglu(gt.float().numpy(), ut.float().numpy(), bf16) if ref else \
        (gt.float() / (1 + torch.exp(-gt.float())) * ut.float()).numpy()
    tol = 2.0 ** -7 if bf16 else 2e-6
    assert np.all(np.abs(out.float().cpu().numpy() - want) <= tol * np.maximum(np.abs(want), 1e-3))
    torch.cuda.synchronize()
    with pytest.raises(ValueError):
        kd.swiglu(gt.to(DEV), ut.to(DEV)[:, :10], out)
