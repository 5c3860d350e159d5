"""MoE decode layer stack on top of the library's MoE entry points, single GPU or
expert-parallel over the ranks of one node.

One layer:  logits = bf16(h W_r^T)  ->  moe_route (softmax over the selected k,
renormalised)  ->  moe_ffn over the rank's experts  ->  [sum of the ranks' partial
outputs]  ->  h' = bf16(rmsnorm(h + y)).

Expert parallelism: expert e lives on rank e // (E / world). Every rank holds the
full token block (T x H, 1 MB at the benchmark shape) and routes redundantly (the
router is deterministic), computes only its own experts' slots, and the partial
outputs are summed across ranks with one NCCL all-reduce per layer. The reference
has no multi-GPU code at all; this file is new design, not a mirror of it.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

Q4_K = 12


@dataclass
class StackConfig:
    layers: int = 48
    hidden: int = 2048
    ffn: int = 768
    experts: int = 128
    top_k: int = 8
    tokens: int = 256
    seed: int = 20261125

    def expert_bytes(self) -> int:
        rb_h = self.hidden // 256 * 144
        rb_f = self.ffn // 256 * 144
        return 2 * self.ffn * rb_h + self.hidden * rb_f

    def layer_bytes(self) -> int:
        return self.experts * self.expert_bytes()


def expert_range(rank: int, world: int, n_experts: int) -> Tuple[int, int]:
    """(first, count) of the contiguous expert block owned by `rank`."""
    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not split over {world} ranks")
    per = n_experts // world
    return rank * per, per


def random_q4k_payload(n_rows_total: int, cols: int, gen: torch.Generator, device) -> torch.Tensor:
    """Random Q4_K bytes with sanitized fp16 super-block scales (d = dmin = 2^-10), the payload style of
    the reference's benchmarks (benchmarks/Bench_MoeDecode.cpp:54-84)."""
    nb = n_rows_total * (cols // 256)
    raw = torch.randint(0, 256, (nb, 144), dtype=torch.uint8, device=device, generator=gen)
    raw[:, 0] = 0x00
    raw[:, 1] = 0x14
    raw[:, 2] = 0x00
    raw[:, 3] = 0x14
    return raw.reshape(-1)


class MoeStack:
    def __init__(self, kd, device, cfg: StackConfig, rank: int = 0, world: int = 1, group=None):
        self.kd, self.dev, self.cfg, self.rank, self.world, self.group = kd, device, cfg, rank, world, group
        self.e_first, self.e_count = expert_range(rank, world, cfg.experts)
        c = cfg
        self.layers: List[tuple] = []
        self.routers: List[torch.Tensor] = []
        for l in range(c.layers):
            # router weights are identical on every rank; expert payloads are seeded per (layer, expert)
            g = torch.Generator(device=device).manual_seed(c.seed + 7919 * l)
            self.routers.append((torch.randn(c.experts, c.hidden, device=device, generator=g) /
                                 c.hidden ** 0.5).to(torch.bfloat16))
            ge = torch.Generator(device=device).manual_seed(c.seed + 104729 * l + 31 * self.e_first + 1)
            gate = random_q4k_payload(self.e_count * c.ffn, c.hidden, ge, device)
            up = random_q4k_payload(self.e_count * c.ffn, c.hidden, ge, device)
            down = random_q4k_payload(self.e_count * c.hidden, c.ffn, ge, device)
            self.layers.append(self._tables(gate, up, down))
        T, S = c.tokens, c.top_k
        self.logits = torch.empty((T, c.experts), dtype=torch.bfloat16, device=device)
        self.idx = torch.empty((T, S), dtype=torch.int32, device=device)
        self.wts = torch.empty((T, S), dtype=torch.float32, device=device)
        self.y = torch.empty((T, c.hidden), dtype=torch.float32, device=device)
        self.ws = torch.zeros(kd.moe_ffn_workspace_bytes(T, S, c.hidden, c.ffn, c.experts), dtype=torch.uint8,
                              device=device)

    def _tables(self, gate, up, down):
        """Pointer tables over ALL experts; entries of experts this rank does not own are null."""
        kd, c = self.kd, self.cfg
        eb_g = c.ffn * (c.hidden // 256 * 144)
        eb_d = c.hidden * (c.ffn // 256 * 144)

        def table(buf, per, rows, cols):
            base = torch.zeros(c.experts, dtype=torch.int64, device=self.dev)
            own = torch.arange(self.e_count, device=self.dev, dtype=torch.int64) * per + buf.data_ptr()
            base[self.e_first:self.e_first + self.e_count] = own
            return kd.QuantWeightTable(base, Q4_K, rows, cols, cols // 256 * 144, (buf,))

        return (table(gate, eb_g, c.ffn, c.hidden), table(up, eb_g, c.ffn, c.hidden),
                table(down, eb_d, c.hidden, c.ffn))

    def layer(self, l: int, h: torch.Tensor) -> torch.Tensor:
        kd, c = self.kd, self.cfg
        torch.matmul(h, self.routers[l].t(), out=self.logits)          # plain library GEMM for the router logits
        kd.moe_route(self.logits, None, c.top_k, True, 1.0, self.idx, self.wts)
        tg, tu, td = self.layers[l]
        kd.moe_ffn(h, tg, tu, td, self.idx, self.wts, self.y, self.ws, self.e_first, self.e_count)
        if self.world > 1:
            torch.distributed.all_reduce(self.y, group=self.group)     # sum of the ranks' partial outputs
        out = torch.empty_like(h)
        kd.residual_rmsnorm(h, self.y, out)
        return out

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        for l in range(self.cfg.layers):
            h = self.layer(l, h)
        return h

    def kernels_per_layer(self) -> int:
        return 7   # route, sort, quantize x, gate/up tile (+ act quantizer), down tile, combine, residual+norm


def bench_moe_stack(kd, dev, rank: int, world: int, steps: int = 5, warmup: int = 3, peak: float = 6553.0,
                    cfg: Optional[StackConfig] = None) -> dict:
    """Tokens/s of the whole stack, timed with CUDA events, max over ranks."""
    import torch.distributed as dist
    cfg = cfg or StackConfig()
    stack = MoeStack(kd, dev, cfg, rank, world)
    g = torch.Generator(device=dev).manual_seed(cfg.seed)
    h0 = torch.randn(cfg.tokens, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        out = stack.forward(h0)
        torch.cuda.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                out = stack.forward(h0)
        except Exception:
            graph = None
            torch.cuda.synchronize()
    run = (lambda: graph.replay()) if graph is not None else (lambda: stack.forward(h0))
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            run()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(steps):
            run()
        e1.record(stream)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    finite = bool(torch.isfinite(out.float()).all().item())
    status = kd.device_status()
    layer_bytes = cfg.layer_bytes()
    return {
        "metric": "moe_decode_tokens_per_s", "value": cfg.tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "ms_per_step": ms, "scaling": "strong",
        "config": {"workload": "fine-grained MoE decode stack", "layers": cfg.layers, "hidden": cfg.hidden,
                   "experts": cfg.experts, "top_k": cfg.top_k, "ffn": cfg.ffn, "tokens": cfg.tokens,
                   "experts_per_gpu": cfg.experts // world, "weights": "random Q4_K payloads (seeded)",
                   "exchange": "replicated tokens, one NCCL all-reduce of partial outputs per layer"
                   if world > 1 else "none", "cuda_graph": graph is not None},
        "us_per_layer": ms * 1e3 / cfg.layers,
        "weight_GBps_per_gpu": layer_bytes / world * cfg.layers / (ms * 1e-3) / 1e9,
        "hbm_frac_per_gpu": layer_bytes / world * cfg.layers / (ms * 1e-3) / 1e9 / peak,
        "gpu_launches_per_step": stack.kernels_per_layer() * cfg.layers,
        "outputs_finite": finite, "device_status": status,
    }
