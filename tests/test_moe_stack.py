"""MoE layer stack: residual + RMS norm kernel, expert-parallel sharding arithmetic (gloo, CPU, world 2)
and a two-layer stack on the GPU against the CPU checker."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _stack_module():
    import __graft_entry__ as ge
    name = "dnn_for_kokkos_b200.moe_stack"
    if name in sys.modules:
        return sys.modules[name]
    ge.load_package()
    import importlib
    return importlib.import_module(name)


def test_expert_range():
    ms = _stack_module()
    assert ms.expert_range(0, 1, 128) == (0, 128)
    assert [ms.expert_range(r, 8, 128) for r in range(8)] == [(16 * r, 16) for r in range(8)]
    assert ms.expert_range(3, 4, 8) == (6, 2)
    with pytest.raises(ValueError):
        ms.expert_range(0, 3, 128)
    cfg = ms.StackConfig()
    assert cfg.layer_bytes() == 128 * (2 * 768 * 1152 + 2048 * 432) == 339738624


def _ep_worker(rank, world, port_q, tmpdir):
    """Each rank computes only its experts' slots (CPU checker as the compute), partial outputs are summed
    with an all-reduce: must equal the single-rank result up to fp32 reassociation."""
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_q)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as ge
    pack = ge._load_module("_gp_ep", os.path.join(ge.PKG_DIR, "ggml_pack.py"))
    ms_spec = ge._load_module("_ms_ep", os.path.join(ge.PKG_DIR, "moe_stack.py"))
    port = O.Port()
    port.set_threads(2)
    E, H, F, T, S = 8, 256, 256, 10, 2
    rng = np.random.default_rng(0)
    gate = [O.aligned_copy(pack.synth_weight(O.Q4_K, F, H, 10 + e, std=0.05)) for e in range(E)]
    up = [O.aligned_copy(pack.synth_weight(O.Q4_K, F, H, 20 + e, std=0.05)) for e in range(E)]
    down = [O.aligned_copy(pack.synth_weight(O.Q4_K, H, F, 30 + e, std=0.05)) for e in range(E)]
    X = O.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    idx, wts = port.moe_route(O.bf16_round(rng.standard_normal((T, E)).astype(np.float32)), None, S, True)
    full = port.moe_ffn_int8(X, gate, up, down, idx, wts, F, bf16=True)
    first, count = ms_spec.expert_range(rank, world, E)
    local_idx = np.where((idx >= first) & (idx < first + count), idx, -1).astype(np.int32)
    part = torch.from_numpy(port.moe_ffn_int8(X, gate, up, down, local_idx, wts, F, bf16=True))
    dist.all_reduce(part)
    ok = np.abs(part.numpy() - full).max() <= 1e-5 * np.abs(full).max()
    open(os.path.join(tmpdir, f"ok{rank}"), "w").write("1" if ok else "0")
    dist.destroy_process_group()


def test_expert_parallel_partials_sum_to_full_gloo(tmp_path):
    import torch.multiprocessing as mp
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port_q = s.getsockname()[1]
    s.close()
    mp.spawn(_ep_worker, args=(2, port_q, str(tmp_path)), nprocs=2, join=True)
    assert all(open(tmp_path / f"ok{r}").read() == "1" for r in range(2))


def test_token_range():
    ms = _stack_module()
    assert [ms.token_range(r, 8, 256) for r in range(8)] == [(32 * r, 32) for r in range(8)]
    assert ms.token_range(0, 1, 7) == (0, 7)
    with pytest.raises(ValueError):
        ms.token_range(0, 3, 256)


@pytest.mark.gpu
def test_residual_rmsnorm(kd):
    """out = Scalar(rmsnorm_noscale(Scalar(h + y))) against the reference's own rmsnorm_noscale
    (src/KokkosDNN_RMSNorm.hpp:347-361, through its compiled headers when present) applied to the residual sum."""
    dev = "cuda:0"
    ref = O.Ref() if O.Ref.available() else None
    for dt in (torch.float32, torch.bfloat16):
        g = torch.Generator().manual_seed(1)
        h = torch.randn(37, 2048, generator=g).to(dt)
        y = torch.randn(37, 2048, generator=g) * 3
        out = torch.empty(37, 2048, dtype=dt, device=dev)
        kd.residual_rmsnorm(h.to(dev), y.to(dev), out, 1e-6)
        torch.cuda.synchronize()
        r = (h.float() + y).to(dt).float()
        if ref is not None:
            want = torch.from_numpy(ref.rmsnorm_noscale(r.numpy(), 1e-6, bf16=(dt == torch.bfloat16)))
        else:
            want = (r / torch.sqrt((r * r).mean(dim=1, keepdim=True) + 1e-6)).to(dt).float()
        tol = 1e-5 if dt == torch.float32 else 2.0 ** -7
        assert (out.float().cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["push", "allreduce"])
def test_two_layer_stack_matches_checker(kd, port, mode):
    """x = rmsnorm(h); y = ffn(route(x W_r^T), x); h' = h + y, two layers, against the CPU checker."""
    ms = _stack_module()
    dev = torch.device("cuda:0")
    cfg = ms.StackConfig(layers=2, hidden=512, ffn=256, experts=8, top_k=2, tokens=12, seed=5)
    stack = ms.MoeStack(kd, dev, cfg, exchange=mode)
    g = torch.Generator(device=dev).manual_seed(cfg.seed)
    h0 = torch.randn(cfg.tokens, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
    out = stack.forward(h0)
    torch.cuda.synchronize()
    assert kd.device_status() == 0
    # same stack on the CPU checker
    norm = lambda r: O.bf16_round(r / np.sqrt((r * r).mean(axis=1, keepdims=True) + 1e-6))
    h = h0.float().cpu().numpy()
    x = norm(h)
    for l in range(cfg.layers):
        logits = O.bf16_round((torch.from_numpy(x).to(torch.bfloat16).to(dev) @ stack.routers[l].t()).float().cpu().numpy())
        idx, wts = port.moe_route(logits, None, cfg.top_k, True)
        tg, tu, td = stack.layers[l]
        eb_g = cfg.ffn * (cfg.hidden // 256 * 144)
        eb_d = cfg.hidden * (cfg.ffn // 256 * 144)
        gbuf, ubuf, dbuf = (t.keepalive[0].cpu().numpy() for t in (tg, tu, td))
        gate = [O.aligned_copy(gbuf[e * eb_g:(e + 1) * eb_g]) for e in range(cfg.experts)]
        up = [O.aligned_copy(ubuf[e * eb_g:(e + 1) * eb_g]) for e in range(cfg.experts)]
        down = [O.aligned_copy(dbuf[e * eb_d:(e + 1) * eb_d]) for e in range(cfg.experts)]
        y = port.moe_ffn_int8(x, gate, up, down, idx, wts, cfg.ffn, bf16=True)
        h = O.bf16_round(h + y)
        x = norm(h)
    got = out.float().cpu().numpy()
    assert np.abs(got - h).max() <= 2.0 ** -6 * np.abs(h).max()


@pytest.mark.gpu
def test_expert_parallel_stack_on_two_gpus(kd):
    """The push exchange and the all-reduce design on two ranks (one process per GPU, peer memory through IPC
    handles) against the same stack on one rank. Needs two GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import subprocess
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.join(ROOT, "bench.py"),
                        "--gpus", "2", "--check-multi-rank"], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    import json
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert line["push"] <= 1e-3 and line["allreduce"] <= 2.0 ** -6 and line["device_status"] == 0, line
