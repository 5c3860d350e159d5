"""Run one kernel of the library on one benchmark shape a few times -- a small, bounded
workload for profilers (ncu) and for quick checks on a new machine.

    python dnn-for-kokkos_b200/probe.py gemv q4k        # Q4_K 14336x4096, cold weights every launch
    python dnn-for-kokkos_b200/probe.py gemv q6k | q80 | q4k_small | q5k
    python dnn-for-kokkos_b200/probe.py moe             # one fine-grained MoE layer, three times

The GEMV probe keeps about 0.4 GB of copies of the matrix on the device and walks them, so
every launch reads weights that are not in L2; the MoE probe holds one layer (0.34 GB).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as ge  # noqa: E402


def gemv(kd, which: str, passes: int = 2) -> None:
    dev = torch.device("cuda:0")
    shapes = {"q4k": (kd.Q4_K, 14336, 4096), "q6k": (kd.Q6_K, 4096, 14336), "q80": (kd.Q8_0, 4096, 4096),
              "q4k_small": (kd.Q4_K, 4096, 4096), "q5k": (kd.Q5_K, 16000, 4096)}
    dt, rows, K = shapes[which]
    nbytes = rows * kd.ggml_row_bytes(dt, K)
    if dt == kd.Q5_K:
        packed = kd.ggml_pack.random_payload(dt, rows, K, 1)
    else:
        packed = kd.ggml_pack.synth_weight(dt, rows, K, 1)
    base = torch.from_numpy(packed.reshape(-1)).to(dev)
    copies = [kd.QuantWeight(base.clone(), dt, rows, K) for _ in range(int(400e6 // nbytes) + 1)]
    x = torch.randn(K, device=dev).to(torch.bfloat16)
    y = torch.empty(rows, dtype=torch.float32, device=dev)
    s = torch.empty(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device=dev)
    for _ in range(passes):
        for w in copies:
            kd.quant_gemv(x, w, y, s)
    torch.cuda.synchronize()
    print(f"gemv {which}: {len(copies)} copies x {passes} passes, status {kd.device_status()}")


def moe(kd, calls: int = 3) -> None:
    dev = torch.device("cuda:0")
    E, k, H, F, T = 128, 8, 2048, 768, 256
    rb_g, rb_d = kd.ggml_row_bytes(kd.Q4_K, H), kd.ggml_row_bytes(kd.Q4_K, F)
    bufs = []
    for rows, rb, nb in ((F, rb_g, F * H // 256), (F, rb_g, F * H // 256), (H, rb_d, H * F // 256)):
        buf = torch.randint(0, 256, (E, rows * rb), dtype=torch.uint8, device=dev)
        v = buf.view(E, nb, 144)
        v[:, :, 0], v[:, :, 1], v[:, :, 2], v[:, :, 3] = 0, 0x14, 0, 0x14   # d = dmin = 2^-10
        bufs.append(buf)
    mk = lambda buf, r, c: kd.make_quant_weight_table([kd.QuantWeight(buf[e], kd.Q4_K, r, c) for e in range(E)])
    tg, tu, td = mk(bufs[0], F, H), mk(bufs[1], F, H), mk(bufs[2], H, F)
    X = torch.randn(T, H, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev).to(torch.bfloat16)
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    wts = torch.empty((T, k), dtype=torch.float32, device=dev)
    Y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    ws = torch.zeros(kd.moe_ffn_workspace_bytes(T, k, H, F, E), dtype=torch.uint8, device=dev)
    for _ in range(calls):
        kd.moe_route(logits, None, k, True, 1.0, idx, wts)
        kd.moe_ffn(X, tg, tu, td, idx, wts, Y, ws)
    torch.cuda.synchronize()
    print(f"moe: {calls} calls, status {kd.device_status()}")


if __name__ == "__main__":
    kd = ge.load_package()
    if len(sys.argv) >= 2 and sys.argv[1] == "moe":
        moe(kd)
    elif len(sys.argv) >= 3 and sys.argv[1] == "gemv":
        gemv(kd, sys.argv[2])
    else:
        sys.exit(__doc__)
