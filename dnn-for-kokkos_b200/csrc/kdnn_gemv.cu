// Decode GEMV y = W x for GGUF block-quantized W (Q4_K, Q6_K, Q8_0) against
// per-32 int8 activations, for sm_100a.
//
// One kernel per call. Every CTA first starts streaming its packed weight rows
// with 1-D bulk copies (TMA, cp.async.bulk -> shared memory, completion on
// mbarriers), then quantizes the activation row into shared memory (the
// reference's separate stage-1 launch, src/KokkosDNN_GGUFGemvInt8.hpp:198-239,
// folded into the prologue; CTA 0 also writes the reference's staging layout to
// the caller's scratch), then consumes the weight stages with dp4a.
//
// Each lane handles one 64-element item of a 2048-element chunk per row, so the
// activation window and its block scales are loaded from shared memory once per
// RW weight rows (the cross-row reuse of the reference's row-blocked kernel,
// :525-599).
//
// HBM traffic per call: rows*row_bytes (each weight byte exactly once) +
// K*sizeof(x) per CTA from L2 + rows*sizeof(y).
#include "kdnn_common.cuh"

#include <limits.h>
#include <stdlib.h>

#include <atomic>
#include <string>

namespace kdnn {

__device__ int g_gemv_status = 0;

constexpr int kChunkItems = 32;    // one item per lane

template <uint32_t DT>
__host__ __device__ constexpr int chunk_bytes_full() {
  return DT == KDNN_GGML_Q4_K ? 8 * 144 : DT == KDNN_GGML_Q6_K ? 8 * 210 : 64 * 34;
}
// bytes of a chunk holding `items` 64-element items
template <uint32_t DT>
__host__ __device__ constexpr int chunk_bytes(int items) {
  return DT == KDNN_GGML_Q4_K ? items * 36 : DT == KDNN_GGML_Q6_K ? (items / 4) * 210 : items * 68;
}

// ---- activation staging in shared memory -------------------------------------
// xg[g][item]: the item's g-th 16-byte int8 granule, g = 0..3 (SoA so a warp's
// 128-bit loads are conflict-free). hd[item]: fp32 block scales (+ for Q4_K the
// scaled block sums). hs[item] (Q6_K): 32 * part sums for the "-32" term.
template <uint32_t DT>
__device__ __forceinline__ void granule_of(int b, int p, int& item, int& g) {
  if (DT == KDNN_GGML_Q6_K) {
    const int j8 = b & 7;
    item         = (b >> 3) * 4 + (j8 >> 2) * 2 + p;
    g            = j8 & 3;
  } else {
    const int k16 = b * 2 + p;
    item          = k16 >> 2;
    g             = k16 & 3;
  }
}

template <uint32_t DT, class XT>
__device__ __forceinline__ void stage_activations(const XT* __restrict__ x, int K, int nitems,
                                                  int4* xg, float4* hd, int4* hs,
                                                  uint8_t* gscratch) {
  const int nblk     = K / 32;
  const int lane     = threadIdx.x & 31;
  const int l4       = lane & 3;          // four lanes per 32-element block, eight elements each
  const int warps    = blockDim.x >> 5;
  const bool vec_ok  = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  int8_t* gq         = reinterpret_cast<int8_t*>(gscratch);
  ActHdr* gh         = gscratch ? reinterpret_cast<ActHdr*>(gscratch + act_hdr_offset(K)) : nullptr;
  // U independent loads in flight per thread before any of them is consumed: the
  // prologue is one memory round trip, not one per block.
  constexpr int U = 4;
  const int step  = warps * 8;
  for (int base0 = (threadIdx.x >> 5) * 8; base0 < nblk; base0 += step * U) {
    float v[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int b = base0 + u * step + (lane >> 2);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
      if (b < nblk) load8<XT>(x, static_cast<size_t>(b) * 32 + l4 * 8, vec_ok, v[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (base0 + u * step >= nblk) break;  // uniform across the warp
      const int b = base0 + u * step + (lane >> 2);
      float d;
      int part, total;
      const uint2 packed = quantize_block_lane8(v[u], d, part, total);
      if (b >= nblk) continue;
      const int p = l4 >> 1;
      int item, g;
      granule_of<DT>(b, p, item, g);
      reinterpret_cast<uint2*>(xg + static_cast<size_t>(g) * nitems + item)[l4 & 1] = packed;
      if ((l4 & 1) == 0) {
        if (DT == KDNN_GGML_Q6_K) {
          reinterpret_cast<float*>(hd + item)[g] = d;
          reinterpret_cast<int*>(hs + item)[g]   = part << 5;
        } else if (p == 0) {
          float* h = reinterpret_cast<float*>(hd + (b >> 1));
          h[b & 1] = d;
          if (DT == KDNN_GGML_Q4_K) h[2 + (b & 1)] = __fmul_rn(static_cast<float>(total), d);
        }
      }
      if (gscratch) {
        reinterpret_cast<uint2*>(gq + static_cast<size_t>(b) * 32)[l4] = packed;
        if (l4 == 0) gh[b] = ActHdr{d, part, total - part, 0};
      }
    }
  }
}

// ---- per-format item evaluation ------------------------------------------------
// `rowp`: shared-memory byte address of this row's chunk segment; `il`: item index
// inside the chunk (= lane). Returns the item's fp32 contribution to the row sum.

__device__ __forceinline__ int4 lds128(uint32_t a) {
  int4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
// 16 bytes at a 2-byte-aligned shared address as four words.
__device__ __forceinline__ void lds16_u2(uint32_t a, uint32_t (&w)[4]) {
  const uint32_t base = a & ~3u, sh = (a & 2u) * 8u;
  uint32_t t[5];
#pragma unroll
  for (int i = 0; i < 5; ++i) t[i] = lds32(base + 4 * i);
#pragma unroll
  for (int i = 0; i < 4; ++i) w[i] = __funnelshift_r(t[i], t[i + 1], sh);
}

// Q4_K 6-bit (scale, min) pairs of sub-blocks 2*it and 2*it+1 from the 12 scale
// bytes (s0 = bytes 0-3, s1 = 4-7, s2 = 8-11). Result: byte 0 = first sub-block,
// byte 1 = second.
__device__ __forceinline__ void q4k_scales(uint32_t s0, uint32_t s1, uint32_t s2, int it,
                                           uint32_t& scp, uint32_t& mnp) {
  const uint32_t sh = (it & 1) * 16;
  const uint32_t u0 = (s0 >> sh) & 0xFFFFu, u1 = (s1 >> sh) & 0xFFFFu, u2 = (s2 >> sh) & 0xFFFFu;
  if (it < 2) {
    scp = u0 & 0x3F3Fu;
    mnp = u1 & 0x3F3Fu;
  } else {
    scp = (u2 & 0x0F0Fu) | ((u0 >> 2) & 0x3030u);
    mnp = ((u2 >> 4) & 0x0F0Fu) | ((u1 >> 2) & 0x3030u);
  }
}

struct ItemX {   // one item's activation side, loaded once per RW rows
  int4 g[4];
  float4 hd;
  int4 hs;
};

template <uint32_t DT>
__device__ __forceinline__ float item_dot(uint32_t rowp, int il, const ItemX& x);

template <>
__device__ __forceinline__ float item_dot<KDNN_GGML_Q4_K>(uint32_t rowp, int il, const ItemX& x) {
  const uint32_t blk = rowp + (il >> 2) * 144;
  const int4 h       = lds128(blk);
  const int4 qa      = lds128(blk + 16 + (il & 3) * 32);
  const int4 qb      = lds128(blk + 32 + (il & 3) * 32);
  uint32_t scp, mnp;
  q4k_scales(h.y, h.z, h.w, il & 3, scp, mnp);
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
  const uint32_t q[8] = {(uint32_t)qa.x, (uint32_t)qa.y, (uint32_t)qa.z, (uint32_t)qa.w,
                         (uint32_t)qb.x, (uint32_t)qb.y, (uint32_t)qb.z, (uint32_t)qb.w};
  uint32_t lo0[4], lo1[4], hi0[4], hi1[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo0[i] = q[i] & 0x0F0F0F0Fu;
    hi0[i] = q[i] & 0xF0F0F0F0u;      // 16 * high nibble, used as unsigned bytes
    lo1[i] = q[4 + i] & 0x0F0F0F0Fu;
    hi1[i] = q[4 + i] & 0xF0F0F0F0u;
  }
  // low nibbles <-> elements 0..31 of the item (granules 0,1), high <-> 32..63 (2,3)
  const int dotA = dot16(lo1, x.g[1], dot16(lo0, x.g[0], 0));
  const int dotB = dot16_us(hi1, x.g[3], dot16_us(hi0, x.g[2], 0)) >> 4;  // exact: the sum is a multiple of 16
  const int sc0 = scp & 0xFF, sc1 = scp >> 8, mn0 = mnp & 0xFF, mn1 = mnp >> 8;
  const float p = static_cast<float>(sc0 * dotA) * x.hd.x + static_cast<float>(sc1 * dotB) * x.hd.y;
  const float m = static_cast<float>(mn0) * x.hd.z + static_cast<float>(mn1) * x.hd.w;
  return dd.x * p - dd.y * m;
}

template <>
__device__ __forceinline__ float item_dot<KDNN_GGML_Q6_K>(uint32_t rowp, int il, const ItemX& x) {
  const int chunk = (il >> 1) & 1, half = il & 1;
  const uint32_t blk = rowp + (il >> 2) * 210;
  uint32_t ql0[4], ql1[4], qh[4];
  lds16_u2(blk + chunk * 64 + half * 16, ql0);
  lds16_u2(blk + chunk * 64 + half * 16 + 32, ql1);
  lds16_u2(blk + 128 + chunk * 32 + half * 16, qh);
  uint32_t w0[4], w1[4], w2[4], w3[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    w0[i] = (ql0[i] & 0x0F0F0F0Fu) | ((qh[i] << 4) & 0x30303030u);
    w1[i] = (ql1[i] & 0x0F0F0F0Fu) | ((qh[i] << 2) & 0x30303030u);
    w2[i] = ((ql0[i] >> 4) & 0x0F0F0F0Fu) | (qh[i] & 0x30303030u);
    w3[i] = ((ql1[i] >> 4) & 0x0F0F0F0Fu) | ((qh[i] >> 2) & 0x30303030u);
  }
  const int d0 = dot16(w0, x.g[0], 0) - x.hs.x;
  const int d1 = dot16(w1, x.g[1], 0) - x.hs.y;
  const int d2 = dot16(w2, x.g[2], 0) - x.hs.z;
  const int d3 = dot16(w3, x.g[3], 0) - x.hs.w;
  // int8 scales of the four 16-element groups: scales[chunk*8 + half + 2g]
  const uint32_t sa = blk + 192 + chunk * 8 + half;
  int s[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    int v;
    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(sa + 2 * g));
    s[g] = v;
  }
  uint32_t db;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(db) : "r"(blk + 208));
  const float acc = static_cast<float>(s[0] * d0) * x.hd.x + static_cast<float>(s[1] * d1) * x.hd.y +
                    static_cast<float>(s[2] * d2) * x.hd.z + static_cast<float>(s[3] * d3) * x.hd.w;
  return h2f(db) * acc;
}

template <>
__device__ __forceinline__ float item_dot<KDNN_GGML_Q8_0>(uint32_t rowp, int il, const ItemX& x) {
  const uint32_t a = rowp + il * 68;  // two 34-byte blocks, 4-byte aligned
  uint32_t t[17];
#pragma unroll
  for (int i = 0; i < 17; ++i) t[i] = lds32(a + 4 * i);
  uint32_t q0[4], q1[4], q2[4], q3[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    q0[i] = __funnelshift_r(t[i], t[i + 1], 16);
    q1[i] = __funnelshift_r(t[4 + i], t[5 + i], 16);
    q2[i] = t[9 + i];
    q3[i] = t[13 + i];
  }
  const int dot0 = dot16(q1, x.g[1], dot16(q0, x.g[0], 0));
  const int dot1 = dot16(q3, x.g[3], dot16(q2, x.g[2], 0));
  return (h2f(t[0] & 0xFFFFu) * x.hd.x) * static_cast<float>(dot0) +
         (h2f(t[8] >> 16) * x.hd.y) * static_cast<float>(dot1);
}

// ---- the streaming kernel --------------------------------------------------------
constexpr int kGemvWarps  = 16;
constexpr int kTraceSlots = 8;   // timestamps per warp when tracing

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define KDNN_TRACE(slot)                                                                   \
  do {                                                                                     \
    if (p.trace && lane == 0)                                                              \
      p.trace[(static_cast<size_t>(blockIdx.x) * kGemvWarps + warp) * kTraceSlots + (slot)] = globaltimer_ns(); \
  } while (0)

// One 16-warp CTA per SM. Every warp is an independent streaming engine with a private
// ring of shared-memory stages (bulk copies, mbarrier completion, bounded waits): it takes
// whole row groups (RW rows, their 2048-element chunks in sequence), keeps the row sums in
// registers and does one shuffle reduction per group. The first group of every warp is
// fixed (gw = warp * gridDim + blockIdx, so the GPU sweeps the matrix in address order and
// the weights can be requested before the previous kernel in the stream has finished);
// the rest are handed out by a ticket counter, requested one group ahead so the atomic's
// round trip is off the critical path and all warps finish within one group of each other.
// The warp reconverges (__syncwarp) after lane 0 has refilled a stage and before anybody
// waits on the next one.
constexpr int kTicketSlots = 64;
__device__ unsigned int g_gemv_tickets[kTicketSlots];

struct GemvParams {
  const uint8_t* w;
  const void* x;
  void* y;
  uint8_t* scratch;
  int rows, K, row_bytes, nitems, nchunks;
  int ngroups, stages, stage_bytes, ticket_slot;
  unsigned long long* trace;
};

template <uint32_t DT, int RW, class XT, class YT>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) gemv_stream_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int4* xg      = reinterpret_cast<int4*>(smem);
  float4* hd    = reinterpret_cast<float4*>(smem + static_cast<size_t>(p.nitems) * 64);
  int4* hs      = reinterpret_cast<int4*>(smem + static_cast<size_t>(p.nitems) * 80);
  size_t off    = static_cast<size_t>(p.nitems) * (DT == KDNN_GGML_Q6_K ? 96 : 80);
  off           = (off + 127) & ~size_t(127);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off) + warp * 8;
  int2* meta     = reinterpret_cast<int2*>(smem + off + kGemvWarps * 64) + warp * 8;   // {group, chunk} per stage
  off += kGemvWarps * 128;
  uint8_t* ring = smem + off + static_cast<size_t>(warp) * p.stages * p.stage_bytes;
  const uint32_t ring_u32 = smem_u32(ring), bar_u32 = smem_u32(bars);
  KDNN_TRACE(0);

  const int G  = gridDim.x * kGemvWarps;
  const int gw = warp * gridDim.x + blockIdx.x;
  int is_group = gw, is_chunk = 0, is_n = 0;
  bool is_done = gw >= p.ngroups;
  int is_next  = 0x7fffffff;
  auto fetch_next = [&]() {
    is_next = G + static_cast<int>(atomicAdd(&g_gemv_tickets[p.ticket_slot], 1u));
  };
  auto issue = [&]() {  // lane 0 only
    const int s = is_n % p.stages;
    ++is_n;
    if (is_done) {
      meta[s] = make_int2(-1, 0);
      return;
    }
    meta[s] = make_int2(is_group, is_chunk);
    const int items   = min(kChunkItems, p.nitems - is_chunk * kChunkItems);
    const uint32_t cb = chunk_bytes<DT>(items);
    const int row0 = is_group * RW;
    const int nrow = min(RW, p.rows - row0);
    const uint32_t bar = bar_u32 + s * 8;
    mbar_expect_tx(bar, cb * nrow);
    const uint8_t* src = p.w + static_cast<size_t>(row0) * p.row_bytes +
                         static_cast<size_t>(is_chunk) * chunk_bytes_full<DT>();
    const uint32_t dst = ring_u32 + s * p.stage_bytes;
#pragma unroll
    for (int r = 0; r < RW; ++r)
      if (r < nrow)
        bulk_g2s(dst + r * chunk_bytes_full<DT>(), src + static_cast<size_t>(r) * p.row_bytes, cb, bar);
    if (++is_chunk == p.nchunks) {
      is_chunk = 0;
      is_group = is_next;
      if (is_group >= p.ngroups) is_done = true; else fetch_next();
    }
  };
  if (lane == 0) {
    for (int s = 0; s < p.stages; ++s) mbar_init(bar_u32 + s * 8, 1);
    fence_barrier_init();
    fence_proxy_async();
    if (!is_done) fetch_next();
    for (int s = 0; s < p.stages; ++s) issue();
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    g_gemv_tickets[(p.ticket_slot + kTicketSlots / 2) % kTicketSlots] = 0;  // a slot not in use
  KDNN_TRACE(1);
  pdl_launch_dependents();
  pdl_wait();
  KDNN_TRACE(2);
  stage_activations<DT, XT>(static_cast<const XT*>(p.x), p.K, p.nitems, xg, hd, hs,
                            blockIdx.x == 0 ? p.scratch : nullptr);
  __syncthreads();
  KDNN_TRACE(3);

  float acc[RW];
#pragma unroll
  for (int r = 0; r < RW; ++r) acc[r] = 0.f;
  YT* y = static_cast<YT*>(p.y);
  for (int n = 0;; ++n) {
    const int s  = n % p.stages;
    const int2 m = meta[s];
    if (m.x < 0) break;
    if (!mbar_wait_bounded(bar_u32 + s * 8, (n / p.stages) & 1)) {
      if (lane == 0) atomicExch(&g_gemv_status, KDNN_ERR_DEVICE_WAIT);
      return;
    }
    if (n == 0) KDNN_TRACE(4);
    const int item = m.y * kChunkItems + lane;
    if (item < p.nitems) {
      ItemX x;
#pragma unroll
      for (int g = 0; g < 4; ++g) x.g[g] = xg[static_cast<size_t>(g) * p.nitems + item];
      x.hd = hd[item];
      if (DT == KDNN_GGML_Q6_K) x.hs = hs[item];
      const uint32_t st = ring_u32 + s * p.stage_bytes;
#pragma unroll
      for (int r = 0; r < RW; ++r) acc[r] += item_dot<DT>(st + r * chunk_bytes_full<DT>(), lane, x);
    }
    if (m.y == p.nchunks - 1) {
      const int row0 = m.x * RW;
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float v = warp_sum(acc[r]);
        if (lane == 0 && row0 + r < p.rows) store_scalar(y + row0 + r, v);
        acc[r] = 0.f;
      }
    }
    __syncwarp();
    if (lane == 0) issue();
    __syncwarp();
  }
  KDNN_TRACE(6);
}

// ---- generic kernels (any alignment; also the parity probe) ------------------------
// Reference-shaped unit evaluation straight from global memory with 16-bit
// loads; windows and integer dots exactly as
// src/KokkosDNN_GGUFGemvInt8.hpp:280-466 defines them.
__device__ __forceinline__ uint32_t ldg_u16x2(const uint8_t* p) {
  const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
  return static_cast<uint32_t>(q[0]) | (static_cast<uint32_t>(q[1]) << 16);
}

template <uint32_t DT>
__device__ float unit_eval_generic(const uint8_t* row, int c, const int8_t* xq, const ActHdr* xh,
                                   int* ints) {
  const int blk = c >> 3, half = c & 1;
  int k0, kb, h0, h1;
  if (DT == KDNN_GGML_Q4_K) {
    k0 = blk * 256 + ((c >> 1) & 3) * 64 + half * 16; kb = k0 + 32; h0 = k0 >> 5; h1 = h0 + 1;
  } else if (DT == KDNN_GGML_Q6_K) {
    k0 = blk * 256 + ((c >> 2) & 1) * 128 + ((c >> 1) & 1) * 32 + half * 16; kb = k0 + 64;
    h0 = k0 >> 5; h1 = h0 + 2;
  } else {
    k0 = c * 32; kb = k0 + 16; h0 = h1 = c;
  }
  const int4 xa = *reinterpret_cast<const int4*>(xq + k0);
  const int4 xb = *reinterpret_cast<const int4*>(xq + kb);
  const float dx0 = xh[h0].d, dx1 = xh[h1].d;
  const int sum0 = half ? xh[h0].sum_hi : xh[h0].sum_lo;
  const int sum1 = half ? xh[h1].sum_hi : xh[h1].sum_lo;
  if (DT == KDNN_GGML_Q4_K) {
    const int it     = (c >> 1) & 3;
    const uint8_t* b = row + static_cast<size_t>(blk) * 144;
    const uint8_t* q = b + 16 + it * 32 + half * 16;
    uint32_t scp, mnp;
    q4k_scales(ldg_u16x2(b + 4), ldg_u16x2(b + 8), ldg_u16x2(b + 12), it, scp, mnp);
    const float dw = h2f(ldg_u16x2(b) & 0xFFFFu), dm = h2f(ldg_u16x2(b) >> 16);
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w = ldg_u16x2(q + 4 * i);
      lo[i] = w & 0x0F0F0F0Fu;
      hi[i] = (w >> 4) & 0x0F0F0F0Fu;
    }
    const int dotA = dot16(lo, xa, 0), dotB = dot16(hi, xb, 0);
    ints[0] = dotA; ints[1] = dotB;
    const float fa = dw * (float)(scp & 0xFF) * dx0, ma = dm * (float)(mnp & 0xFF) * dx0;
    const float fb = dw * (float)(scp >> 8) * dx1, mb = dm * (float)(mnp >> 8) * dx1;
    return fa * (float)dotA - ma * (float)sum0 + fb * (float)dotB - mb * (float)sum1;
  } else if (DT == KDNN_GGML_Q6_K) {
    const int chunk = (c >> 2) & 1, pair = (c >> 1) & 1;
    const uint8_t* b  = row + static_cast<size_t>(blk) * 210;
    const uint8_t* ql = b + chunk * 64 + pair * 32 + half * 16;
    const uint8_t* qh = b + 128 + chunk * 32 + half * 16;
    const int8_t* scl = reinterpret_cast<const int8_t*>(b + 192);
    const uint32_t sh = pair ? 2u : 0u;
    uint32_t wA[4], wB[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t l = ldg_u16x2(ql + 4 * i), h = ldg_u16x2(qh + 4 * i);
      wA[i] = (l & 0x0F0F0F0Fu) | (((h >> sh) & 0x03030303u) << 4);
      wB[i] = ((l >> 4) & 0x0F0F0F0Fu) | (((h >> (sh + 4u)) & 0x03030303u) << 4);
    }
    ints[0] = dot16(wA, xa, 0) - (sum0 << 5);
    ints[1] = dot16(wB, xb, 0) - (sum1 << 5);
    const float d  = h2f(*reinterpret_cast<const uint16_t*>(b + 208));
    const float s0 = d * (float)scl[chunk * 8 + 2 * pair + half] * dx0;
    const float s1 = d * (float)scl[chunk * 8 + 2 * pair + half + 4] * dx1;
    return s0 * (float)ints[0] + s1 * (float)ints[1];
  } else {
    const uint8_t* b = row + static_cast<size_t>(c) * 34;
    uint32_t q0[4], q1[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      q0[i] = ldg_u16x2(b + 2 + 4 * i);
      q1[i] = ldg_u16x2(b + 18 + 4 * i);
    }
    ints[0] = dot16(q1, xb, dot16(q0, xa, 0));
    ints[1] = 0;
    return h2f(*reinterpret_cast<const uint16_t*>(b)) * dx0 * (float)ints[0];
  }
}

template <class XT>
__global__ void quantize_act_kernel(const XT* __restrict__ x, int K, uint8_t* scratch) {
  const int nblk    = K / 32;
  const int lane    = threadIdx.x & 31, l8 = lane & 7;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & (sizeof(XT) * 4 - 1)) == 0;
  int8_t* gq        = reinterpret_cast<int8_t*>(scratch);
  ActHdr* gh        = reinterpret_cast<ActHdr*>(scratch + act_hdr_offset(K));
  const int gwarp   = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarp   = (gridDim.x * blockDim.x) >> 5;
  for (int base = gwarp * 4; base < nblk; base += nwarp * 4) {
    const int b      = base + (lane >> 3);
    const bool valid = b < nblk;
    float v[4]       = {0.f, 0.f, 0.f, 0.f};
    if (valid) load4<XT>(x, static_cast<size_t>(b) * 32 + l8 * 4, vec_ok, v);
    float d;
    int part, total;
    const uint32_t packed = quantize_block_lane(v, d, part, total);
    if (!valid) continue;
    reinterpret_cast<uint32_t*>(gq + static_cast<size_t>(b) * 32)[l8] = packed;
    if (l8 == 0) gh[b] = ActHdr{d, part, total - part, 0};
  }
}

// one warp per row over a staged activation row in global memory
template <uint32_t DT, class YT>
__global__ void gemv_generic_kernel(const uint8_t* __restrict__ w, size_t row_bytes, int rows,
                                    int K, const uint8_t* __restrict__ scratch, YT* y) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int8_t* xq = reinterpret_cast<const int8_t*>(scratch);
  const ActHdr* xh = reinterpret_cast<const ActHdr*>(scratch + act_hdr_offset(K));
  float acc        = 0.f;
  for (int c = lane; c < K / 32; c += 32) {
    int ints[2];
    acc += unit_eval_generic<DT>(w + static_cast<size_t>(row) * row_bytes, c, xq, xh, ints);
  }
  acc = warp_sum(acc);
  if (lane == 0) store_scalar(y + row, acc);
}

template <uint32_t DT>
__global__ void unit_dots_kernel(const uint8_t* __restrict__ w, size_t row_bytes, int rows, int K,
                                 const uint8_t* __restrict__ scratch, int32_t* out) {
  const int nu       = K / 32;
  const size_t total = static_cast<size_t>(rows) * nu;
  const int8_t* xq   = reinterpret_cast<const int8_t*>(scratch);
  const ActHdr* xh   = reinterpret_cast<const ActHdr*>(scratch + act_hdr_offset(K));
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / nu), c = static_cast<int>(i % nu);
    int ints[2];
    unit_eval_generic<DT>(w + static_cast<size_t>(r) * row_bytes, c, xq, xh, ints);
    out[2 * i]     = ints[0];
    out[2 * i + 1] = ints[1];
  }
}

// ---- host side ------------------------------------------------------------------
struct DeviceInfo {
  int sms = 0, max_smem = 0, smem_per_sm = 0;
};
static const DeviceInfo& device_info() {
  static thread_local DeviceInfo cache[64];
  int dev = 0;
  cudaGetDevice(&dev);
  DeviceInfo& d = cache[dev & 63];
  if (d.sms == 0) {
    cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&d.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaDeviceGetAttribute(&d.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
  }
  return d;
}

// KDNN_NO_PDL=1 launches without programmatic stream serialization (A/B aid).
static bool use_pdl() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("KDNN_NO_PDL");
    v             = (e && e[0] == '1') ? 0 : 1;
  }
  return v != 0;
}

static int env_int(const char* name, int dflt) {
  const char* e = getenv(name);
  return (e && *e) ? atoi(e) : dflt;
}

// Debug aid: when set (kdnn_b200_debug_set_trace), every warp of the streaming kernel
// writes kTraceSlots globaltimer stamps per launch into this device buffer.
static unsigned long long* g_trace_buffer = nullptr;
void gemv_set_trace(void* buf) { g_trace_buffer = static_cast<unsigned long long*>(buf); }

static std::atomic<unsigned> g_launch_counter{0};

template <uint32_t DT, int RW, class XT, class YT>
static cudaError_t launch_stream(const GemvParams& base, cudaStream_t stream) {
  const DeviceInfo& di = device_info();
  GemvParams p = base;
  p.ngroups     = (p.rows + RW - 1) / RW;
  p.stage_bytes = (RW * chunk_bytes_full<DT>() + 127) & ~127;
  const size_t act = ((static_cast<size_t>(p.nitems) * (DT == KDNN_GGML_Q6_K ? 96 : 80)) + 127) & ~size_t(127);
  auto smem_need = [&](int st) {
    return act + kGemvWarps * 128 + static_cast<size_t>(kGemvWarps) * st * p.stage_bytes + 128;
  };
  // Two stages per warp keep about one bandwidth-delay product in flight per SM; deeper
  // rings measured slower (their requests queue ahead of the activation loads).
  int stages = env_int("KDNN_GEMV_STAGES", 2);
  stages     = stages < 2 ? 2 : (stages > 8 ? 8 : stages);
  while (stages > 2 && smem_need(stages) > static_cast<size_t>(di.max_smem)) --stages;
  if (smem_need(stages) > static_cast<size_t>(di.max_smem)) return cudaErrorInvalidConfiguration;
  p.stages      = stages;
  p.ticket_slot = static_cast<int>(g_launch_counter.fetch_add(1) % kTicketSlots);
  p.trace       = g_trace_buffer;
  const int grid = min(di.sms, (p.ngroups + kGemvWarps - 1) / kGemvWarps);
  const size_t smem = smem_need(stages);
  auto kern = gemv_stream_kernel<DT, RW, XT, YT>;
  static thread_local size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem);
    if (e != cudaSuccess) return e;
    configured = di.max_smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kGemvWarps * 32); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = use_pdl() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <uint32_t DT, class XT, class YT>
static cudaError_t launch_stream_rw(const GemvParams& p, cudaStream_t stream) {
  const DeviceInfo& di = device_info();
  // Rows per group. One row per group gives the finest work units and measured fastest
  // for tall matrices; when there are at most two rows per warp, two-row groups (one
  // group per warp, shared activation window) win for the 144- and 34-byte formats.
  int rw = env_int("KDNN_GEMV_RW", 0);
  if (rw == 0) {
    const int warps = di.sms * kGemvWarps;
    rw = (DT != KDNN_GGML_Q6_K && p.rows > warps && p.rows <= 2 * warps) ? 2 : 1;
  }
  if (rw >= 2) return launch_stream<DT, 2, XT, YT>(p, stream);
  return launch_stream<DT, 1, XT, YT>(p, stream);
}

template <uint32_t DT>
static cudaError_t launch_stream_dt(const GemvParams& p, int xs, int ys, cudaStream_t stream) {
  if (xs == KDNN_F32 && ys == KDNN_F32) return launch_stream_rw<DT, float, float>(p, stream);
  if (xs == KDNN_BF16 && ys == KDNN_BF16)
    return launch_stream_rw<DT, __nv_bfloat16, __nv_bfloat16>(p, stream);
  if (xs == KDNN_BF16 && ys == KDNN_F32) return launch_stream_rw<DT, __nv_bfloat16, float>(p, stream);
  return launch_stream_rw<DT, float, __nv_bfloat16>(p, stream);
}

template <uint32_t DT>
static cudaError_t launch_generic_dt(const uint8_t* w, size_t rb, int rows, int K, const void* x,
                                     int xs, void* y, int ys, uint8_t* scratch, cudaStream_t st) {
  const int qblocks = max(1, min(64, (K / 32 + 31) / 32));
  if (xs == KDNN_F32)
    quantize_act_kernel<float><<<qblocks, 256, 0, st>>>(static_cast<const float*>(x), K, scratch);
  else
    quantize_act_kernel<__nv_bfloat16><<<qblocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), K, scratch);
  const int blocks = (rows + 7) / 8;
  if (ys == KDNN_F32)
    gemv_generic_kernel<DT, float><<<blocks, 256, 0, st>>>(w, rb, rows, K, scratch, static_cast<float*>(y));
  else
    gemv_generic_kernel<DT, __nv_bfloat16><<<blocks, 256, 0, st>>>(w, rb, rows, K, scratch, static_cast<__nv_bfloat16*>(y));
  return cudaGetLastError();
}

// Entry used by the C ABI. `force_generic` != 0 selects the plain-load kernels.
cudaError_t gemv_launch(uint32_t dt, const void* w, size_t rows, size_t cols, const void* x, int xs,
                        void* y, int ys, void* scratch, int force_generic, cudaStream_t stream) {
  const size_t rb = row_bytes_of(dt, cols);
  const bool w16  = (reinterpret_cast<uintptr_t>(w) & 15u) == 0;
  // bulk copies need 16-byte aligned row segments: every row start and every
  // 2048-element chunk start, and chunk sizes that are multiples of 16.
  bool fast = w16 && rb % 16 == 0 && cols % 64 == 0 && !force_generic && rb <= INT_MAX;
  if (dt == KDNN_GGML_Q6_K) fast = fast && cols % 2048 == 0;
  if (dt == KDNN_GGML_Q8_0) fast = fast && cols % 256 == 0;
  if (fast) {
    GemvParams p{};
    p.w         = static_cast<const uint8_t*>(w);
    p.x         = x;
    p.y         = y;
    p.scratch   = static_cast<uint8_t*>(scratch);
    p.rows      = static_cast<int>(rows);
    p.K         = static_cast<int>(cols);
    p.row_bytes = static_cast<int>(rb);
    p.nitems    = static_cast<int>(cols / 64);
    p.nchunks   = (p.nitems + kChunkItems - 1) / kChunkItems;
    cudaError_t e;
    switch (dt) {
      case KDNN_GGML_Q4_K: e = launch_stream_dt<KDNN_GGML_Q4_K>(p, xs, ys, stream); break;
      case KDNN_GGML_Q6_K: e = launch_stream_dt<KDNN_GGML_Q6_K>(p, xs, ys, stream); break;
      default: e = launch_stream_dt<KDNN_GGML_Q8_0>(p, xs, ys, stream); break;
    }
    if (e != cudaErrorInvalidConfiguration) return e;
    (void)cudaGetLastError();  // row too long for the shared-memory ring: plain loads
  }
  const uint8_t* wb = static_cast<const uint8_t*>(w);
  uint8_t* sb       = static_cast<uint8_t*>(scratch);
  switch (dt) {
    case KDNN_GGML_Q4_K: return launch_generic_dt<KDNN_GGML_Q4_K>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, sb, stream);
    case KDNN_GGML_Q6_K: return launch_generic_dt<KDNN_GGML_Q6_K>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, sb, stream);
    default: return launch_generic_dt<KDNN_GGML_Q8_0>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, sb, stream);
  }
}

cudaError_t quantize_act_launch(const void* x, int xs, size_t K, void* scratch, cudaStream_t st) {
  const int qblocks = max(1, min(64, (int)((K / 32 + 31) / 32)));
  if (xs == KDNN_F32)
    quantize_act_kernel<float><<<qblocks, 256, 0, st>>>(static_cast<const float*>(x), (int)K, static_cast<uint8_t*>(scratch));
  else
    quantize_act_kernel<__nv_bfloat16><<<qblocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), (int)K, static_cast<uint8_t*>(scratch));
  return cudaGetLastError();
}

cudaError_t unit_dots_launch(uint32_t dt, const void* w, size_t rows, size_t cols,
                             const void* scratch, int32_t* out, cudaStream_t st) {
  const size_t rb    = row_bytes_of(dt, cols);
  const size_t total = rows * (cols / 32);
  const size_t want   = (total + 255) / 256;
  const int blocks    = (int)(want < 4096 ? want : 4096);
  const uint8_t* wb  = static_cast<const uint8_t*>(w);
  const uint8_t* sb  = static_cast<const uint8_t*>(scratch);
  switch (dt) {
    case KDNN_GGML_Q4_K: unit_dots_kernel<KDNN_GGML_Q4_K><<<blocks, 256, 0, st>>>(wb, rb, (int)rows, (int)cols, sb, out); break;
    case KDNN_GGML_Q6_K: unit_dots_kernel<KDNN_GGML_Q6_K><<<blocks, 256, 0, st>>>(wb, rb, (int)rows, (int)cols, sb, out); break;
    default: unit_dots_kernel<KDNN_GGML_Q8_0><<<blocks, 256, 0, st>>>(wb, rb, (int)rows, (int)cols, sb, out); break;
  }
  return cudaGetLastError();
}

int gemv_take_status() {
  int v = 0, zero = 0;
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(&v, g_gemv_status, sizeof(int));
  if (v != 0) cudaMemcpyToSymbol(g_gemv_status, &zero, sizeof(int));
  return v;
}

// ---- allocation-free entry point --------------------------------------------------
// Activation staging for callers that cannot hand us a scratch buffer: a fixed array in
// device memory that every GPU loading this library carries until the process exits.
// Host code must not pass the array's name to a kernel (on the host the name is only a
// stand-in for the symbol); the device address is looked up once per device with
// cudaGetSymbolAddress and cached.
constexpr size_t kNoAllocMaxCols = 32768;                                  // largest K served
constexpr size_t kNoAllocBytes   = kNoAllocMaxCols + kNoAllocMaxCols / 2;  // = act_bytes(32768) = 49152
static __device__ __align__(256) uint8_t g_noalloc_staging[kNoAllocBytes];

void set_last_error(const char* msg);  // kdnn_capi.cu

static cudaError_t noalloc_staging_address(uint8_t** out) {
  constexpr int kMaxDevices = 64;
  static uint8_t* cache[kMaxDevices] = {};
  static std::atomic<bool> ready[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (!ready[dev].load(std::memory_order_acquire)) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_staging);  // resolved for the current device
    if (e != cudaSuccess) return e;
    cache[dev] = static_cast<uint8_t*>(p);
    ready[dev].store(true, std::memory_order_release);
  }
  *out = cache[dev];
  return cudaSuccess;
}

}  // namespace kdnn

extern "C" int kdnn_b200_quant_gemv_noalloc(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                                            const void* x, int x_scalar, void* y, int y_scalar,
                                            void* stream) {
  using namespace kdnn;
  if ((x_scalar != KDNN_F32 && x_scalar != KDNN_BF16) || (y_scalar != KDNN_F32 && y_scalar != KDNN_BF16)) {
    set_last_error("quant_gemv_noalloc: scalar must be KDNN_F32 or KDNN_BF16");
    return KDNN_ERR_INVALID;
  }
  if (cols > kNoAllocMaxCols) {
    set_last_error("quant_gemv_noalloc: cols exceeds the built-in staging (32768 columns); "
                   "use kdnn_b200_quant_gemv with a caller-owned scratch buffer");
    return KDNN_ERR_INVALID;
  }
  // the same decline list as kdnn_b200_quant_gemv, minus the scratch checks
  if (ggml_type != KDNN_GGML_Q4_K && ggml_type != KDNN_GGML_Q6_K && ggml_type != KDNN_GGML_Q8_0)
    return KDNN_DECLINED;
  if (w == nullptr || x == nullptr || y == nullptr) return KDNN_DECLINED;
  if (!block_aligned(ggml_type, cols)) return KDNN_DECLINED;
  if (rows == 0 || rows > static_cast<size_t>(INT_MAX)) return KDNN_DECLINED;
  if ((reinterpret_cast<uintptr_t>(w) & 1u) != 0u) return KDNN_DECLINED;
  if (ggml_type == KDNN_GGML_Q4_K && (reinterpret_cast<uintptr_t>(w) & 15u) != 0u) return KDNN_DECLINED;
  uint8_t* staging = nullptr;
  cudaError_t e = noalloc_staging_address(&staging);
  if (e == cudaSuccess)
    e = gemv_launch(ggml_type, w, rows, cols, x, x_scalar, y, y_scalar, staging, 0,
                    static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    set_last_error((std::string("quant_gemv_noalloc: ") + cudaGetErrorString(e)).c_str());
    return KDNN_ERR_CUDA;
  }
  return KDNN_OK;
}
