"""MoE decode layer stack on top of the library's MoE entry points, single GPU or
expert-parallel over the ranks of one node.

One layer (``exchange="push"``, the default; four kernel launches, see kdnn_b200_moe_block):
    x = rmsnorm(h)  [from the previous layer's combine]
    logits = Scalar(x W_r^T) -> top-k routing -> expert feed-forward -> y
    h' = Scalar(h + y),  x' = Scalar(rmsnorm(h'))

Expert parallelism: expert e lives on rank e // (E / world) and every rank owns tokens_local = T / world
tokens of the batch. The first kernel of a layer writes its tokens' quantized rows and routing into every
rank's exchange region (plain stores over NVLink: the dispatch), every rank runs its experts for the routed
slots of all tokens, the down-projection kernel stores each output row straight into the token owner's region
(the combine exchange) and the owner sums its tokens' slots in slot order. Flags with bounded waits order the
steps; no collective library call is on the path.

``exchange="allreduce"`` is the simpler design kept for comparison: every rank holds the full token block,
routes redundantly, computes its own experts' slots, and the partial outputs are summed with one NCCL
all-reduce per layer.

The reference has no multi-GPU code at all; this file is new design, not a mirror of it.
"""
from __future__ import annotations

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


def token_range(rank: int, world: int, tokens: int) -> Tuple[int, int]:
    """(first, count) of the contiguous token block owned by `rank`."""
    if tokens % world:
        raise ValueError(f"{tokens} tokens do not split over {world} ranks")
    per = tokens // world
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


def make_exchange(kd, rank: int, world: int, tokens_local: int, top_k: int, hidden: int, wait_ns: int = 0):
    """Allocates this rank's exchange region and opens the peers' (IPC handles travel through
    torch.distributed). Returns None for a single rank: the region then lives in the workspace."""
    if world == 1:
        return None
    import torch.distributed as dist
    nbytes = kd.MoeExchange.region_bytes(tokens_local, world, top_k, hidden)
    ptr, handle = kd.MoeExchange.alloc(nbytes)
    handles: List[Optional[bytes]] = [None] * world
    dist.all_gather_object(handles, handle)
    regions = [ptr if r == rank else kd.MoeExchange.open(handles[r]) for r in range(world)]
    dist.barrier()
    return kd.MoeExchange(rank, world, regions, wait_ns, ipc=True)


class MoeStack:
    def __init__(self, kd, device, cfg: StackConfig, rank: int = 0, world: int = 1, group=None,
                 exchange: str = "push"):
        self.kd, self.dev, self.cfg, self.rank, self.world, self.group = kd, device, cfg, rank, world, group
        self.mode = exchange
        self.e_first, self.e_count = expert_range(rank, world, cfg.experts)
        self.t_first, self.t_count = token_range(rank, world, cfg.tokens)
        c = cfg
        self.layers: List[tuple] = []
        self.routers: List[torch.Tensor] = []
        for l in range(c.layers):
            # router weights are identical on every rank; expert payloads are seeded per (layer, expert)
            g = torch.Generator(device=device).manual_seed(c.seed + 7919 * l)
            self.routers.append((torch.randn(c.experts, c.hidden, device=device, generator=g) /
                                 c.hidden ** 0.5).to(torch.bfloat16))
            gate, up, down = [], [], []
            for e in range(self.e_first, self.e_first + self.e_count):
                ge = torch.Generator(device=device).manual_seed(c.seed + 104729 * l + 31 * e + 1)
                gate.append(random_q4k_payload(c.ffn, c.hidden, ge, device))
                up.append(random_q4k_payload(c.ffn, c.hidden, ge, device))
                down.append(random_q4k_payload(c.hidden, c.ffn, ge, device))
            self.layers.append(self._tables(torch.cat(gate), torch.cat(up), torch.cat(down)))
        T, S = c.tokens, c.top_k
        if exchange == "push":
            self.ex = make_exchange(kd, rank, world, self.t_count, S, c.hidden)
            self.ws = torch.zeros(kd.moe_block_workspace_bytes(self.t_count, world, S, c.hidden, c.ffn, c.experts,
                                                               world == 1), dtype=torch.uint8, device=device)
        else:
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

    # ---- push exchange: this rank's tokens only -----------------------------------------------------
    def layer_push(self, l: int, h: torch.Tensor, x: torch.Tensor):
        """(h', x') of this rank's tokens: one kdnn_b200_moe_block call, four launches."""
        kd, c = self.kd, self.cfg
        tg, tu, td = self.layers[l]
        h2, x2 = torch.empty_like(h), torch.empty_like(x)
        kd.moe_block(x, self.routers[l], None, c.top_k, True, 1.0, tg, tu, td, self.ws, resid=h, h_out=h2, xn_out=x2,
                     expert_first=self.e_first, expert_count=self.e_count, exchange=self.ex)
        return h2, x2

    # ---- replicated tokens + all-reduce (comparison design) --------------------------------------------
    def layer_allreduce(self, l: int, h: torch.Tensor, x: torch.Tensor):
        kd, c = self.kd, self.cfg
        torch.matmul(x, self.routers[l].t(), out=self.logits)          # plain library GEMM for the router logits
        kd.moe_route(self.logits, None, c.top_k, True, 1.0, self.idx, self.wts)
        tg, tu, td = self.layers[l]
        kd.moe_ffn(x, tg, tu, td, self.idx, self.wts, self.y, self.ws, self.e_first, self.e_count)
        if self.world > 1:
            torch.distributed.all_reduce(self.y, group=self.group)     # sum of the ranks' partial outputs
        h2 = (h.float() + self.y).to(h.dtype)
        x2 = torch.empty_like(x)
        kd.residual_rmsnorm(h, self.y, x2)
        return h2, x2

    def close(self) -> None:
        """Gives the exchange regions back. Collective: every rank calls it, after its last forward."""
        ex = getattr(self, "ex", None)
        if ex is None:
            return
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)     # nobody reads or writes a peer's region after this
            torch.cuda.synchronize(self.dev)
        ex.close()
        self.ex = None

    def forward(self, h0: torch.Tensor) -> torch.Tensor:
        """h0: the full [tokens, hidden] block (identical on every rank). Returns the final residual stream of
        this rank's tokens (push) or of all tokens (allreduce)."""
        if self.mode == "push":
            h = h0[self.t_first:self.t_first + self.t_count].contiguous()
        else:
            h = h0
        x = torch.empty_like(h)
        self.kd.residual_rmsnorm(h, torch.zeros(h.shape, dtype=torch.float32, device=h.device), x)
        step = self.layer_push if self.mode == "push" else self.layer_allreduce
        for l in range(self.cfg.layers):
            h, x = step(l, h, x)
        return h

    def kernels_per_layer(self) -> int:
        # push: gate (logits + route + quantize + sort), gate/up tiles, down tiles, combine (+ residual + norm)
        # allreduce: route, prep (sort + quantize), gate/up, down, combine, residual + norm (+ the library GEMM and NCCL)
        return 4 if self.mode == "push" else 6


def bench_moe_stack(kd, dev, rank: int, world: int, steps: int = 5, warmup: int = 3, peak: float = 6553.0,
                    cfg: Optional[StackConfig] = None, exchange: str = "push", tile_kind: int = 3) -> dict:
    """Tokens/s of the whole stack, timed with CUDA events, max over ranks."""
    import torch.distributed as dist
    cfg = cfg or StackConfig()
    prev_kind = kd.tile_kind(tile_kind)
    stack = MoeStack(kd, dev, cfg, rank, world, exchange=exchange)
    g = torch.Generator(device=dev).manual_seed(cfg.seed)
    h0 = torch.randn(cfg.tokens, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        out = stack.forward(h0)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = stack.forward(h0)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            graph.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    finite = bool(torch.isfinite(out.float()).all().item())
    status = kd.device_status()
    kd.tile_kind(prev_kind)
    del graph          # its kernels name the exchange regions
    stack.close()
    layer_bytes = cfg.layer_bytes()
    names = {3: "auto (mma.sync for the MoE tiles)", 2: "tcgen05 + TMEM", 1: "mma.sync", 0: "dp4a"}
    return {
        "metric": "moe_decode_tokens_per_s", "value": cfg.tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "ms_per_step": ms, "scaling": "strong",
        "config": {"workload": "fine-grained MoE decode stack", "layers": cfg.layers, "hidden": cfg.hidden,
                   "experts": cfg.experts, "top_k": cfg.top_k, "ffn": cfg.ffn, "tokens": cfg.tokens,
                   "experts_per_gpu": cfg.experts // world, "tokens_per_gpu": cfg.tokens // world,
                   "weights": "random Q4_K payloads (seeded)", "tile_kernel": names[tile_kind],
                   "exchange": ("none" if world == 1 else
                                "dispatch: quantized rows pushed to every rank by the gate kernel; combine: output "
                                "rows pushed to the token owner by the down kernel (peer stores + bounded flag waits)")
                   if exchange == "push" else "replicated tokens, one NCCL all-reduce of partial outputs per layer",
                   "cuda_graph": True},
        "us_per_layer": ms * 1e3 / cfg.layers,
        "weight_GBps_per_gpu": layer_bytes / world * cfg.layers / (ms * 1e-3) / 1e9,
        "hbm_frac_per_gpu": layer_bytes / world * cfg.layers / (ms * 1e-3) / 1e9 / peak,
        "gpu_launches_per_step": stack.kernels_per_layer() * cfg.layers,
        "outputs_finite": finite, "device_status": status,
    }


def check_multi_rank(kd, dev, rank: int, world: int, layers: int = 2, cfg: Optional[StackConfig] = None) -> dict:
    """Correctness of the expert-parallel stack: every rank's tokens against the same stack run on ONE rank
    (all experts local, no exchange) inside this process. Returns the largest error relative to max|h|."""
    import torch.distributed as dist
    base = cfg or StackConfig()
    cfg = StackConfig(layers=layers, hidden=base.hidden, ffn=base.ffn, experts=base.experts, top_k=base.top_k,
                      tokens=base.tokens, seed=base.seed)
    g = torch.Generator(device=dev).manual_seed(cfg.seed)
    h0 = torch.randn(cfg.tokens, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
    out = {}
    single = MoeStack(kd, dev, cfg, 0, 1, exchange="push").forward(h0).float()
    torch.cuda.synchronize()
    for mode in ("push", "allreduce"):
        if world > 1:
            dist.barrier()
        stack = MoeStack(kd, dev, cfg, rank, world, exchange=mode)
        got = stack.forward(h0).float()
        torch.cuda.synchronize()
        want = single[stack.t_first:stack.t_first + stack.t_count] if mode == "push" else single
        err = (got - want).abs().max() / single.abs().max()
        t = torch.tensor([float(err)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[mode] = float(t.item())
        stack.close()
        del stack
    out["device_status"] = kd.device_status()
    return out
