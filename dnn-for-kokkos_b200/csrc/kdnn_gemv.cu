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

// Tuning of the call in flight on this host thread (kdnn_b200_gemv_layout; all zero = the defaults).
static thread_local kdnn_b200_gemv_layout t_lay = {};

constexpr int kChunkItems = 32;    // one item per lane

template <uint32_t DT>
__host__ __device__ constexpr int chunk_bytes_full() {
  return DT == KDNN_GGML_Q4_K ? 8 * 144 : DT == KDNN_GGML_Q5_K ? 8 * 176 : DT == KDNN_GGML_Q6_K ? 8 * 210 : 64 * 34;
}
// bytes of a chunk holding `items` 64-element items
template <uint32_t DT>
__host__ __device__ constexpr int chunk_bytes(int items) {
  return DT == KDNN_GGML_Q4_K ? items * 36 : DT == KDNN_GGML_Q5_K ? items * 44 : DT == KDNN_GGML_Q6_K ? (items / 4) * 210 : items * 68;
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

struct NoHook { __device__ void operator()() const {} };
// `after_loads` runs once, after this thread's first batch of global loads has been issued
// and before their values are used: work that needs no activation bytes goes there.
template <uint32_t DT, class XT, class Hook = NoHook>
__device__ __forceinline__ void stage_activations(const XT* x, int K, int nitems,
                                                  int4* xg, float4* hd, int4* hs,
                                                  uint8_t* gscratch, Hook after_loads = Hook()) {
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
  bool first_batch = true;
  // (the loop always runs its first round -- with no block in range nothing is loaded or written in it -- so the hook,
  // the caller's weight requests, is inlined at ONE place; a second call site behind the loop doubled that code)
  for (int base0 = (threadIdx.x >> 5) * 8; base0 < nblk || first_batch; base0 += step * U) {
    float v[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int b = base0 + u * step + (lane >> 2);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
      if (b < nblk) load8<XT>(x, static_cast<size_t>(b) * 32 + l4 * 8, vec_ok, v[u]);
    }
    if (first_batch) after_loads();
    first_batch = false;
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
          if (DT == KDNN_GGML_Q4_K || DT == KDNN_GGML_Q5_K) h[2 + (b & 1)] = __fmul_rn(static_cast<float>(total), d);
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

// Q5_K: the low four bits as in Q4_K, the fifth bit of sub-block j is bit j of qh[l]. The
// dot is linear in the weight, so the bit plane gets its own dp4a against the same
// activation words (kept in place as 2^j * bit, unsigned, the factor removed exactly
// afterwards) instead of being merged into the nibbles first.
template <>
__device__ __forceinline__ float item_dot<KDNN_GGML_Q5_K>(uint32_t rowp, int il, const ItemX& x) {
  const uint32_t blk = rowp + (il >> 2) * 176;
  const int it       = il & 3;
  const int4 h   = lds128(blk);
  const int4 h0  = lds128(blk + 16), h1 = lds128(blk + 32);           // qh[0..15], qh[16..31]
  const int4 qa  = lds128(blk + 48 + it * 32), qb = lds128(blk + 64 + it * 32);
  uint32_t scp, mnp;
  q4k_scales(h.y, h.z, h.w, it, scp, mnp);
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
  const uint32_t q[8]  = {(uint32_t)qa.x, (uint32_t)qa.y, (uint32_t)qa.z, (uint32_t)qa.w,
                          (uint32_t)qb.x, (uint32_t)qb.y, (uint32_t)qb.z, (uint32_t)qb.w};
  const uint32_t hh[8] = {(uint32_t)h0.x, (uint32_t)h0.y, (uint32_t)h0.z, (uint32_t)h0.w,
                          (uint32_t)h1.x, (uint32_t)h1.y, (uint32_t)h1.z, (uint32_t)h1.w};
  uint32_t lo0[4], lo1[4], hi0[4], hi1[4], ba0[4], ba1[4], bb0[4], bb1[4];
  const uint32_t sh = 2 * it;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo0[i] = q[i] & 0x0F0F0F0Fu;
    hi0[i] = q[i] & 0xF0F0F0F0u;          // 16 * high nibble, unsigned bytes
    lo1[i] = q[4 + i] & 0x0F0F0F0Fu;
    hi1[i] = q[4 + i] & 0xF0F0F0F0u;
    const uint32_t t0 = hh[i] >> sh, t1 = hh[4 + i] >> sh;
    ba0[i] = t0 & 0x01010101u;            // fifth bit of sub-block 2*it
    ba1[i] = t1 & 0x01010101u;
    bb0[i] = t0 & 0x02020202u;            // 2 * fifth bit of sub-block 2*it + 1
    bb1[i] = t1 & 0x02020202u;
  }
  const int dotA = dot16(lo1, x.g[1], dot16(lo0, x.g[0], 0)) + 16 * dot16(ba1, x.g[1], dot16(ba0, x.g[0], 0));
  const int dotB = (dot16_us(hi1, x.g[3], dot16_us(hi0, x.g[2], 0)) >> 4) +
                   8 * dot16(bb1, x.g[3], dot16(bb0, x.g[2], 0));   // 16 * (sum of 2 * bit * x) / 2
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
constexpr int kGemvMaxWarps = 16;
constexpr int kXregMaxWarps = 18;   // the Q4_K register-window kernel may run up to 18 warps (576 threads, <= 113 registers)
constexpr int kGemvStages   = 2;   // ring depth per warp: about one bandwidth-delay product per SM in flight

// One CTA per SM, up to 16 warps. Every warp is an independent streaming engine with a
// private two-stage ring in shared memory (bulk copies, mbarrier completion, bounded
// waits); a stage holds one 2048-element chunk of RW consecutive weight rows.
//
// Work split. The row groups (RW rows) are divided evenly and contiguously over the CTAs,
// so nothing is carried between launches and each CTA sweeps its slice in address order.
// Inside a CTA the unit of work is (row group, range of `cpu` chunks): a warp accumulates
// its unit in registers, reduces it across lanes once, and writes either y (the unit
// covers the whole row) or a partial sum in shared memory that the CTA adds up, in chunk
// order, at the end. The host picks `cpu` and the warp count so that every warp gets many
// units and the last round is nearly full. The first unit of every warp is fixed, so its
// weights are requested before the previous kernel in the stream has finished
// (programmatic dependent launch); the rest come from a shared-memory counter, drawn one
// unit ahead.
struct GemvParams {
  const uint8_t* w;
  const void* x;
  void* y;
  uint8_t* scratch;
  int rows, K, row_bytes, nitems, nchunks;
  int ngroups;         // ceil(rows / RW)
  int gq, gr;          // ngroups / grid and ngroups % grid
  int cpu;             // chunks per unit
  int upg;             // units per group = ceil(nchunks / cpu)
  uint32_t upg_magic;  // ceil(2^32 / upg): u / upg == umulhi(u, magic) for the unit counts that occur
  int part_floats;     // partial sums kept in shared memory (upg > 1)
  int stage_bytes;
  int nmat;                 // 0 / 1: one matrix; 2..4: matrices of one shape against the same x in ONE launch
  const uint8_t* w_more[3]; // matrices 1..3
  void* y_more[3];
};

// Sum RW per-lane values across the warp. Afterwards lane l (l < RW) holds the total of
// row rev(l) for RW = 4 -- see row_of_lane -- and of row l for RW <= 2.
template <int RW>
__device__ __forceinline__ float reduce_rows(const float (&a)[RW], int lane) {
  constexpr unsigned full = 0xFFFFFFFFu;
  float v;
  if (RW == 4) {
    const bool hi = lane & 1;
    float k0 = hi ? a[2] : a[0], k1 = hi ? a[3] : a[1];
    const float s0 = hi ? a[0] : a[2], s1 = hi ? a[1] : a[3];
    k0 += __shfl_xor_sync(full, s0, 1);
    k1 += __shfl_xor_sync(full, s1, 1);
    const bool hi2 = lane & 2;
    v = hi2 ? k1 : k0;
    v += __shfl_xor_sync(full, hi2 ? k0 : k1, 2);
    v += __shfl_xor_sync(full, v, 4);
  } else if (RW == 2) {
    const bool hi = lane & 1;
    v = hi ? a[1] : a[0];
    v += __shfl_xor_sync(full, hi ? a[0] : a[1], 1);
    v += __shfl_xor_sync(full, v, 2);
    v += __shfl_xor_sync(full, v, 4);
  } else {
    v = a[0];
    v += __shfl_xor_sync(full, v, 1);
    v += __shfl_xor_sync(full, v, 2);
    v += __shfl_xor_sync(full, v, 4);
  }
  v += __shfl_xor_sync(full, v, 8);
  v += __shfl_xor_sync(full, v, 16);
  return v;
}
template <int RW>
__device__ __forceinline__ int row_of_lane(int lane) {
  return RW == 4 ? ((lane & 1) * 2 + ((lane >> 1) & 1)) : lane;
}

template <uint32_t DT, int RW, class XT, class YT>
__global__ void __launch_bounds__(kGemvMaxWarps * 32, 1) gemv_stream_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
  int4* xg      = reinterpret_cast<int4*>(smem);
  float4* hd    = reinterpret_cast<float4*>(smem + static_cast<size_t>(p.nitems) * 64);
  int4* hs      = reinterpret_cast<int4*>(smem + static_cast<size_t>(p.nitems) * 80);
  size_t off    = static_cast<size_t>(p.nitems) * (DT == KDNN_GGML_Q6_K ? 96 : 80);
  off           = (off + 127) & ~size_t(127);
  const uint32_t bar_u32 = smem_u32(smem + off) + warp * (kGemvStages * 8);
  off += kGemvMaxWarps * kGemvStages * 8;
  int& s_next_unit = *reinterpret_cast<int*>(smem + off);   // work counter of this CTA
  off += 128;
  float* part = reinterpret_cast<float*>(smem + off);        // [local row][unit of the row]
  off += (static_cast<size_t>(p.part_floats) * 4 + 127) & ~size_t(127);
  const uint32_t ring_u32 = smem_u32(smem + off) + warp * (kGemvStages * p.stage_bytes);

  // this CTA's slice of the row groups and its units
  // even contiguous split of the row groups over the CTAs (quotient and remainder from the host)
  const int c0 = static_cast<int>(blockIdx.x) * p.gq + min(static_cast<int>(blockIdx.x), p.gr);
  const int c1 = c0 + p.gq + (static_cast<int>(blockIdx.x) < p.gr ? 1 : 0);
  const int U  = (c1 - c0) * p.upg;
  if (threadIdx.x == 0) s_next_unit = W;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kGemvStages; ++s) mbar_init(bar_u32 + s * 8, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  // ---- producer state (uniform across the warp; lane 0 issues the copies) ----
  int pu = warp, pnext = 0x7fffffff, pg = 0, pchunk0 = 0, pchunks = 1, pc = 0, pui = 0;
  bool pdone = pu >= U;
  auto decode = [&](int u) {
    pg      = p.upg == 1 ? u : static_cast<int>(__umulhi(static_cast<uint32_t>(u), p.upg_magic));
    pui     = u - pg * p.upg;
    pchunk0 = pui * p.cpu;
    pchunks = min(p.cpu, p.nchunks - pchunk0);
  };
  auto draw = [&]() {
    int v = 0;
    if (lane == 0) v = atomicAdd(&s_next_unit, 1);
    pnext = __shfl_sync(0xFFFFFFFFu, v, 0);
  };
  // per-stage description of what the consumer will find: first local row (or -1),
  // chunk index, partial-sum slot (or -1 when the unit ends elsewhere / writes y).
  int m_row[kGemvStages], m_chunk[kGemvStages], m_end[kGemvStages];
  auto issue = [&](int s) {
    if (pdone) {
      m_row[s] = -1;
      return;
    }
    const int chunk = pchunk0 + pc;
    m_row[s]        = pg * RW;
    m_chunk[s]      = chunk;
    m_end[s]        = (pc == pchunks - 1) ? pui : -1;
    const int items   = min(kChunkItems, p.nitems - chunk * kChunkItems);
    const uint32_t cb = chunk_bytes<DT>(items);
    const int row0    = (c0 + pg) * RW;
    const int nrow    = min(RW, p.rows - row0);
    if (lane == 0) {
      const uint32_t bar = bar_u32 + s * 8;
      mbar_expect_tx(bar, cb * nrow);
      const uint8_t* src = p.w + static_cast<size_t>(row0) * p.row_bytes +
                           static_cast<size_t>(chunk) * chunk_bytes_full<DT>();
      const uint32_t dst = ring_u32 + s * p.stage_bytes;
#pragma unroll
      for (int r = 0; r < RW; ++r)
        if (r < nrow)
          bulk_g2s(dst + r * chunk_bytes_full<DT>(), src + static_cast<size_t>(r) * p.row_bytes, cb, bar);
    }
    if (++pc == pchunks) {
      pc = 0;
      pu = pnext;
      if (pu >= U) {
        pdone = true;
      } else {
        decode(pu);
        draw();
      }
    }
  };
  if (!pdone) {
    decode(pu);
    draw();
  }
  // Only the first stage is requested before the dependency: a deeper burst ahead of the
  // activation loads makes those loads (a few KB that everything waits for) queue behind
  // megabytes of weights. The rest of the ring follows once those loads are in flight.
  issue(0);
  pdl_launch_dependents();
  pdl_wait();
  stage_activations<DT, XT>(static_cast<const XT*>(p.x), p.K, p.nitems, xg, hd, hs,
                            blockIdx.x == 0 ? p.scratch : nullptr, [&]() {
#pragma unroll
                              for (int s = 1; s < kGemvStages; ++s) issue(s);
                            });
  __syncthreads();

  float acc[RW];
#pragma unroll
  for (int r = 0; r < RW; ++r) acc[r] = 0.f;
  YT* y         = static_cast<YT*>(p.y);
  const int my_r = row_of_lane<RW>(lane);
  uint32_t phase = 0;
  bool ok = true, more = true;
  while (more) {
#pragma unroll
    for (int s = 0; s < kGemvStages; ++s) {
      if (!more) break;
      if (m_row[s] < 0) {
        more = false;
        break;
      }
      if (!mbar_wait_bounded(bar_u32 + s * 8, phase)) {
        ok = more = false;
        break;
      }
      const int item = m_chunk[s] * kChunkItems + lane;
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
      if (m_end[s] >= 0) {   // last chunk of the unit
        const float v = reduce_rows<RW>(acc, lane);
        const int lrow = m_row[s] + my_r;
        if (lane < RW && c0 * RW + lrow < p.rows) {
          if (p.upg == 1) store_scalar(y + c0 * RW + lrow, v);
          else part[lrow * p.upg + m_end[s]] = v;
        }
#pragma unroll
        for (int r = 0; r < RW; ++r) acc[r] = 0.f;
      }
      __syncwarp();   // every lane has read this stage
      issue(s);
      __syncwarp();
    }
    phase ^= 1u;
  }
  if (!ok && lane == 0) atomicExch(&g_gemv_status, KDNN_ERR_DEVICE_WAIT);
  if (p.upg > 1) {   // add up the partial sums of every local row in chunk order
    __syncthreads();
    const int nloc = min((c1 - c0) * RW, p.rows - c0 * RW);
    for (int r = threadIdx.x; r < nloc; r += blockDim.x) {
      float v = 0.f;
      for (int j = 0; j < p.upg; ++j) v += part[r * p.upg + j];
      store_scalar(y + c0 * RW + r, v);
    }
  }
}

// ---- Q4_K: one lane per (row, super-block) ----------------------------------------
// The item mapping above spends most of its instructions on work that four lanes repeat
// for the same super-block (header load, 6-bit scale unpack) and on loop bookkeeping per
// 1152 bytes. Here a lane owns a whole 144-byte super-block of one row: nine 128-bit
// shared-memory loads, one unpack of all eight (scale, min) pairs, 64 dp4a. A stage holds
// two rows x up to 16 super-blocks (lanes 0..csb-1: row 0, csb..2csb-1: row 1), so a
// warp iteration consumes up to 4608 bytes.
//
// Activations in shared memory: one 336-byte record per super-block -- 256 int8, the eight
// block scales d, the eight products d * block sum, 16 bytes of padding (21 granules: an
// odd pitch, so the lanes of a row hit different banks and every load is base + constant).
constexpr int kWideRec     = 336;
constexpr int kWideSb      = 16;                 // super-blocks per row per stage
constexpr int kWideRowPitch = kWideSb * 144;
constexpr int kWideStage   = 2 * kWideRowPitch;  // bytes

template <class XT, class Hook = NoHook>
__device__ __forceinline__ void stage_activations_wide(const XT* x, int K, uint8_t* xrec,
                                                       uint8_t* gscratch, Hook after_loads = Hook()) {
  const int nblk    = K / 32;
  const int lane    = threadIdx.x & 31;
  const int l4      = lane & 3;
  const int warps   = blockDim.x >> 5;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  int8_t* gq        = reinterpret_cast<int8_t*>(gscratch);
  ActHdr* gh        = gscratch ? reinterpret_cast<ActHdr*>(gscratch + act_hdr_offset(K)) : nullptr;
  constexpr int U = 4;
  const int step  = warps * 8;
  bool first_batch = true;
  // (the loop always runs its first round -- with no block in range nothing is loaded or written in it -- so the hook,
  // the caller's weight requests, is inlined at ONE place; a second call site behind the loop doubled that code)
  for (int base0 = (threadIdx.x >> 5) * 8; base0 < nblk || first_batch; base0 += step * U) {
    float v[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int b = base0 + u * step + (lane >> 2);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
      if (b < nblk) load8<XT>(x, static_cast<size_t>(b) * 32 + l4 * 8, vec_ok, v[u]);
    }
    if (first_batch) after_loads();
    first_batch = false;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (base0 + u * step >= nblk) break;  // uniform across the warp
      const int b = base0 + u * step + (lane >> 2);
      float d;
      int part, total;
      const uint2 packed = quantize_block_lane8(v[u], d, part, total);
      if (b >= nblk) continue;
      const int sb = b >> 3, jb = b & 7;
      uint8_t* rec = xrec + static_cast<size_t>(sb) * kWideRec;
      reinterpret_cast<uint2*>(rec + (jb * 2 + (l4 >> 1)) * 16)[l4 & 1] = packed;
      if (l4 == 0) {
        reinterpret_cast<float*>(rec + 256)[jb] = d;
        reinterpret_cast<float*>(rec + 288)[jb] = __fmul_rn(static_cast<float>(total), d);
      }
      if (gscratch) {
        reinterpret_cast<uint2*>(gq + static_cast<size_t>(b) * 32)[l4] = packed;
        if (l4 == 0) gh[b] = ActHdr{d, part, total - part, 0};
      }
    }
  }
}

// One super-block (144 bytes at shared address `blk`) against its activation record `xr`.
__device__ __forceinline__ float q4k_superblock_dot(uint32_t blk, uint32_t xr) {
  const int4 h = lds128(blk);
  const uint32_t s0 = h.y, s1 = h.z, s2 = h.w;
  // all eight 6-bit scales / mins as bytes: [0] sub-blocks 0-3, [1] sub-blocks 4-7
  const uint32_t sc[2] = {s0 & 0x3F3F3F3Fu, (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u)};
  const uint32_t mn[2] = {s1 & 0x3F3F3F3Fu, ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u)};
  float dxs[8], dss[8];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int4 a = lds128(xr + 256 + 16 * i), c = lds128(xr + 288 + 16 * i);
    dxs[4 * i] = __int_as_float(a.x); dxs[4 * i + 1] = __int_as_float(a.y);
    dxs[4 * i + 2] = __int_as_float(a.z); dxs[4 * i + 3] = __int_as_float(a.w);
    dss[4 * i] = __int_as_float(c.x); dss[4 * i + 1] = __int_as_float(c.y);
    dss[4 * i + 2] = __int_as_float(c.z); dss[4 * i + 3] = __int_as_float(c.w);
  }
  float p = 0.f, m = 0.f;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int4 qa = lds128(blk + 16 + it * 32), qb = lds128(blk + 32 + it * 32);
    const int4 x0 = lds128(xr + 64 * it), x1 = lds128(xr + 64 * it + 16);
    const int4 x2 = lds128(xr + 64 * it + 32), x3 = lds128(xr + 64 * it + 48);
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
    const int dotA = dot16(lo1, x1, dot16(lo0, x0, 0));
    const int dotB = dot16_us(hi1, x3, dot16_us(hi0, x2, 0)) >> 4;  // exact: the sum is a multiple of 16
    const int jA = 2 * it, jB = 2 * it + 1;
    const int scA = (sc[jA >> 2] >> (8 * (jA & 3))) & 0xFF, scB = (sc[jB >> 2] >> (8 * (jB & 3))) & 0xFF;
    const int mnA = (mn[jA >> 2] >> (8 * (jA & 3))) & 0xFF, mnB = (mn[jB >> 2] >> (8 * (jB & 3))) & 0xFF;
    p = fmaf(static_cast<float>(scA * dotA), dxs[jA], p);
    p = fmaf(static_cast<float>(scB * dotB), dxs[jB], p);
    m = fmaf(static_cast<float>(mnA), dss[jA], m);
    m = fmaf(static_cast<float>(mnB), dss[jB], m);
  }
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
  return dd.x * p - dd.y * m;
}

struct WideParams {
  const uint8_t* w;
  const void* x;
  void* y;
  uint8_t* scratch;
  int rows, K, row_bytes, nsb;
  int nchunks, csb;    // chunks per row and super-blocks per chunk (the last chunk may hold fewer)
  int ngroups;         // ceil(rows / 2)
  int gq, gr;          // ngroups / grid and ngroups % grid
  int cpu, upg;        // chunks per unit, units per group
  uint32_t upg_magic;
  int part_floats;
};

// MAXW = 16: one CTA per SM. MAXW = 8: two CTAs per SM, so the next GEMV in the stream is
// resident (weights requested, waiting for its dependency) while this one still streams.
template <class XT, class YT, int MAXW, int STAGES>
__global__ void __launch_bounds__(MAXW * 32, MAXW == 8 ? 2 : 1) gemv_q4k_wide_kernel(const WideParams p) {
  constexpr int RW = 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
  const uint32_t x_u32 = smem_u32(smem);   // activation records
  size_t off    = (static_cast<size_t>(p.nsb) * kWideRec + 127) & ~size_t(127);
  const uint32_t bar_u32 = smem_u32(smem + off) + warp * (STAGES * 8);
  off += MAXW * STAGES * 8;
  int& s_next_unit = *reinterpret_cast<int*>(smem + off);
  off += 128;
  float* part = reinterpret_cast<float*>(smem + off);
  off += (static_cast<size_t>(p.part_floats) * 4 + 127) & ~size_t(127);
  const uint32_t ring_u32 = smem_u32(smem + off) + warp * (STAGES * kWideStage);

  // even contiguous split of the row groups over the CTAs (quotient and remainder from the host)
  const int c0 = static_cast<int>(blockIdx.x) * p.gq + min(static_cast<int>(blockIdx.x), p.gr);
  const int c1 = c0 + p.gq + (static_cast<int>(blockIdx.x) < p.gr ? 1 : 0);
  const int U  = (c1 - c0) * p.upg;
  if (threadIdx.x == 0) s_next_unit = W;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bar_u32 + s * 8, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  int pu = warp, pnext = 0x7fffffff, pg = 0, pchunk0 = 0, pchunks = 1, pc = 0, pui = 0;
  bool pdone = pu >= U;
  auto decode = [&](int u) {
    pg      = p.upg == 1 ? u : static_cast<int>(__umulhi(static_cast<uint32_t>(u), p.upg_magic));
    pui     = u - pg * p.upg;
    pchunk0 = pui * p.cpu;
    pchunks = min(p.cpu, p.nchunks - pchunk0);
  };
  auto draw = [&]() {
    int v = 0;
    if (lane == 0) v = atomicAdd(&s_next_unit, 1);
    pnext = __shfl_sync(0xFFFFFFFFu, v, 0);
  };
  int m_row[STAGES], m_chunk[STAGES], m_end[STAGES];
  auto issue = [&](int s) {
    if (pdone) {
      m_row[s] = -1;
      return;
    }
    const int chunk = pchunk0 + pc;
    m_row[s]        = pg * RW;
    m_chunk[s]      = chunk;
    m_end[s]        = (pc == pchunks - 1) ? pui : -1;
    const uint32_t cb = static_cast<uint32_t>(min(p.csb, p.nsb - chunk * p.csb)) * 144u;
    const int row0    = (c0 + pg) * RW;
    const int nrow    = min(RW, p.rows - row0);
    if (lane == 0) {
      const uint32_t bar = bar_u32 + s * 8;
      mbar_expect_tx(bar, cb * nrow);
      const uint8_t* src = p.w + static_cast<size_t>(row0) * p.row_bytes + static_cast<size_t>(chunk) * p.csb * 144;
      const uint32_t dst = ring_u32 + s * kWideStage;
      bulk_g2s(dst, src, cb, bar);
      if (nrow > 1) bulk_g2s(dst + kWideRowPitch, src + p.row_bytes, cb, bar);
    }
    if (++pc == pchunks) {
      pc = 0;
      pu = pnext;
      if (pu >= U) {
        pdone = true;
      } else {
        decode(pu);
        draw();
      }
    }
  };
  if (!pdone) {
    decode(pu);
    draw();
  }
#pragma unroll
  for (int s = 0; s < STAGES; ++s) issue(s);
  pdl_launch_dependents();
  pdl_wait();
  stage_activations_wide<XT>(static_cast<const XT*>(p.x), p.K, smem, blockIdx.x == 0 ? p.scratch : nullptr);
  __syncthreads();

  float acc[RW] = {0.f, 0.f};   // per-lane sums of this unit: [0] as a row-0 lane, [1] as a row-1 lane
  YT* y = static_cast<YT*>(p.y);
  uint32_t phase = 0;
  bool ok = true, more = true, first_round = true;
  while (more) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      if (!more) break;
      if (m_row[s] < 0) {
        more = false;
        break;
      }
      if (!mbar_wait_bounded(bar_u32 + s * 8, phase)) {
        ok = more = false;
        break;
      }
      const int lrow0 = m_row[s];
      const int nrow  = min(RW, p.rows - (c0 * RW + lrow0));
      const int sb0   = m_chunk[s] * p.csb;
      const int csb   = min(p.csb, p.nsb - sb0);
      const int r     = lane >= csb ? 1 : 0;
      const int sb    = lane - r * csb;
      if (sb < csb && r < nrow) {
        const float v = q4k_superblock_dot(ring_u32 + s * kWideStage + r * kWideRowPitch + sb * 144,
                                           x_u32 + (sb0 + sb) * kWideRec);
        if (r == 0) acc[0] += v; else acc[1] += v;
      }
      if (m_end[s] >= 0) {   // last chunk of the unit
        const float v = reduce_rows<RW>(acc, lane);
        const int lrow = lrow0 + lane;
        if (lane < nrow) {
          if (p.upg == 1) store_scalar(y + c0 * RW + lrow, v);
          else part[lrow * p.upg + m_end[s]] = v;
        }
        acc[0] = acc[1] = 0.f;
      }
      __syncwarp();   // every lane has read this stage
      issue(s);
      __syncwarp();
    }
    first_round = false;
    phase ^= 1u;
  }
  if (!ok && lane == 0) atomicExch(&g_gemv_status, KDNN_ERR_DEVICE_WAIT);
  if (p.upg > 1) {
    __syncthreads();
    const int nloc = min((c1 - c0) * RW, p.rows - c0 * RW);
    for (int r = threadIdx.x; r < nloc; r += blockDim.x) {
      float v = 0.f;
      for (int j = 0; j < p.upg; ++j) v += part[r * p.upg + j];
      store_scalar(y + c0 * RW + r, v);
    }
  }
}

// ---- Q4_K with the activation window in registers --------------------------------------
// In the kernel above two thirds of the shared-memory reads are activation bytes that
// every warp iteration fetches again. Here a warp is bound to one chunk of K (up to 16
// super-blocks) for the whole launch and each lane keeps its half super-block of the
// quantized activations (128 int8, four scales, four scaled sums: 40 registers) from the
// prologue on, so the main loop reads only weight bytes from shared memory: one header
// and four 16-byte nibble words per lane and row.
//   lane = (sb, half): sb = lane / 2 super-block inside the chunk, half = sub-blocks
//   4*half .. 4*half+3. A stage holds RW rows x one chunk (RW * 2304 bytes).
// Warps w, w + nchunks, ... share chunk w % nchunks and draw row groups from that chunk's
// counter; with more than one chunk the per-chunk row sums meet in shared memory and are
// added in chunk order at the end.
struct XregParams {
  const uint8_t* w;
  const void* x;
  void* y;
  uint8_t* scratch;
  int rows, K, row_bytes, nsb, nitems;
  int nchunks, csb;   // chunks per row (<= 16) and super-blocks per chunk (<= 16; the last chunk may hold fewer)
  int ngroups;        // ceil(rows / RW)
  int gq, gr;         // ngroups / grid and ngroups % grid
  int wpc;            // warps per chunk
  uint32_t nch_magic; // ceil(65536 / nchunks): warp / nchunks == (warp * magic) >> 16 for warp < 16
  int part_floats;
  int early;          // ring stages requested before the activation window is quantized
  int split_first;    // request only the first row of the first stage before the dependency
  int nmat, gpm;      // matrices in this launch (same shape, same x) and row groups per matrix; row group g belongs
                      // to matrix g / gpm
  const uint8_t* w_more[3];
  void* y_more[3];
};

// Half a super-block of one row: 128 weights against the lane's register window.
__device__ __forceinline__ float q4k_half_dot(uint32_t blk, uint32_t qoff, int half, const int4 (&xg)[8],
                                              const float4& dxv, const float4& dsv) {
  const int4 h = lds128(blk);
  const uint32_t s0 = h.y, s1 = h.z, s2 = h.w;
  const uint32_t sc4 = half ? ((s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u)) : (s0 & 0x3F3F3F3Fu);
  const uint32_t mn4 = half ? (((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u)) : (s1 & 0x3F3F3F3Fu);
  const float dx[4] = {dxv.x, dxv.y, dxv.z, dxv.w}, ds[4] = {dsv.x, dsv.y, dsv.z, dsv.w};
  // int -> float without the conversion unit: for |i| < 2^22, bits(i + 0x4B400000) is the
  // float 12582912 + i, and one exact subtraction gives float(i). The integer add rides
  // on the multiply-add that forms scale * dot; the 6-bit mins go straight from their byte
  // into the mantissa of 8388608.0f with one byte permute.
  constexpr int kMagicI   = 0x4B400000;
  constexpr float kMagicF = 12582912.0f;
  float p = 0.f, m = 0.f;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int4 qa = lds128(blk + qoff + 32 * t), qb = lds128(blk + qoff + 32 * t + 16);
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
    const int dotA = dot16(lo0, xg[4 * t], 0) + dot16(lo1, xg[4 * t + 1], 0);
    const int dotB = (dot16_us(hi0, xg[4 * t + 2], 0) + dot16_us(hi1, xg[4 * t + 3], 0)) >> 4;  // exact
    const int jA = 2 * t, jB = 2 * t + 1;
    const int scA = static_cast<int>(__byte_perm(sc4, 0u, 0x4440u | jA));
    const int scB = static_cast<int>(__byte_perm(sc4, 0u, 0x4440u | jB));
    const float fA = __int_as_float(scA * dotA + kMagicI) - kMagicF;   // |scale * dot| <= 63 * 60960 < 2^22
    const float fB = __int_as_float(scB * dotB + kMagicI) - kMagicF;
    const float mA = __uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7650u | jA)) - 8388608.0f;
    const float mB = __uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7650u | jB)) - 8388608.0f;
    p = fmaf(fA, dx[jA], p);
    p = fmaf(fB, dx[jB], p);
    m = fmaf(mA, ds[jA], m);
    m = fmaf(mB, ds[jB], m);
  }
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
  return dd.x * p - dd.y * m;
}

template <class XT, class YT, int RW, int STAGES, bool MULTI>
__global__ void __launch_bounds__(kXregMaxWarps * 32, 1) gemv_q4k_xreg_kernel(const XregParams p) {
  constexpr int kStage = RW * kWideRowPitch;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t x_u32 = smem_u32(smem);   // activation records (see kWideRec)
  size_t off = (static_cast<size_t>(p.nsb) * kWideRec + 127) & ~size_t(127);
  const uint32_t bar_u32 = smem_u32(smem + off) + warp * (STAGES * 8);
  off += kXregMaxWarps * STAGES * 8;
  int* s_next = reinterpret_cast<int*>(smem + off);   // [chunk] next local row group
  off += 128;
  float* part = reinterpret_cast<float*>(smem + off);  // [local row][chunk]
  off += (static_cast<size_t>(p.part_floats) * 4 + 127) & ~size_t(127);
  const uint32_t ring_u32 = smem_u32(smem + off) + warp * (STAGES * kStage);

  // even contiguous split of the row groups over the CTAs (quotient and remainder from the host)
  const int c0 = static_cast<int>(blockIdx.x) * p.gq + min(static_cast<int>(blockIdx.x), p.gr);
  const int c1 = c0 + p.gq + (static_cast<int>(blockIdx.x) < p.gr ? 1 : 0);
  const int G  = c1 - c0;                       // row groups of this CTA = units per chunk
  const int widx = static_cast<int>((static_cast<uint32_t>(warp) * p.nch_magic) >> 16), chunk = warp - widx * p.nchunks;
  const int sb0   = chunk * p.csb;
  const int csb   = min(p.csb, p.nsb - sb0);
  const uint32_t cb = static_cast<uint32_t>(csb) * 144u;
  if (threadIdx.x < p.nchunks) s_next[threadIdx.x] = p.wpc;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bar_u32 + s * 8, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncwarp();

  // ---- producer (state uniform across the warp; lane 0 issues the copies) ----
  int m_group[STAGES];
  auto mg_get = [&](int st) {   // register array read / written with a run-time stage index
    int v = m_group[0];
#pragma unroll
    for (int i = 1; i < STAGES; ++i)
      if (st == i) v = m_group[i];
    return v;
  };
  auto mg_set = [&](int st, int v) {
#pragma unroll
    for (int i = 0; i < STAGES; ++i)
      if (st == i) m_group[i] = v;
  };
  // several matrices in one launch: row group g of the launch is row group g % gpm of matrix g / gpm
  auto matrix_of = [&](int g, int& lg) {
    if (!MULTI) { lg = g; return 0; }
    const int m = g / p.gpm;
    lg = g - m * p.gpm;
    return m;
  };
  auto w_of = [&](int m) { return !MULTI || m == 0 ? p.w : m == 1 ? p.w_more[0] : m == 2 ? p.w_more[1] : p.w_more[2]; };
  auto y_of = [&](int m) {
    return static_cast<YT*>(!MULTI || m == 0 ? p.y : m == 1 ? p.y_more[0] : m == 2 ? p.y_more[1] : p.y_more[2]);
  };
  const bool contiguous = p.nchunks == 1 && p.row_bytes == kWideRowPitch;
  // part 0: the whole unit; part 1: its first row only (the barrier already expects all bytes);
  // part 2: the remaining rows of a unit started with part 1
  auto issue_unit = [&](int s, int u, int part = 0) {
    mg_set(s, u);
    int lg;
    const int mat  = matrix_of(c0 + u, lg);
    const int row0 = lg * RW;
    const int nrow = min(RW, p.rows - row0);
    if (lane == 0) {
      const uint32_t bar = bar_u32 + s * 8;
      if (part != 2) mbar_expect_tx(bar, cb * nrow);
      const uint8_t* src = w_of(mat) + static_cast<size_t>(sb0) * 144 + static_cast<size_t>(row0) * p.row_bytes;
      const uint32_t dst = ring_u32 + s * kStage;
      if (contiguous && part == 0) {   // one chunk per row and full rows: the unit is one run of bytes
        bulk_g2s(dst, src, cb * nrow, bar);
      } else {
#pragma unroll
        for (int r = 0; r < RW; ++r)
          if (r < nrow && (part == 0 || (part == 1) == (r == 0)))
            bulk_g2s(dst + r * kWideRowPitch, src + static_cast<size_t>(r) * p.row_bytes, cb, bar);
      }
    }
  };
  // The first unit of every warp is fixed and requested at once, before the CTA has even
  // synchronised. Only this one stage goes out before the dependency: a deeper burst ahead
  // of the activation loads makes those loads (a few KB that everything waits for) queue
  // behind megabytes of weights. The rest of the ring is requested right after the
  // activation loads have been issued.
  bool pdone = widx >= G;
  const bool split_first = RW > 1 && p.split_first;   // half of the first stage now, the rest behind the activation loads
  if (!pdone) issue_unit(0, widx, split_first ? 1 : 0); else m_group[0] = -1;
  __syncthreads();   // the chunk counters are set
  int pu = 0, pnext = 0x7fffffff;
  auto draw = [&]() {
    int v = 0;
    if (lane == 0) v = atomicAdd(&s_next[chunk], 1);
    pnext = __shfl_sync(0xFFFFFFFFu, v, 0);
  };
  auto advance = [&]() {
    pu = pnext;
    if (pu >= G) pdone = true; else draw();
  };
  auto issue = [&](int s) {
    if (pdone) {
      mg_set(s, -1);
      return;
    }
    issue_unit(s, pu);
    advance();
  };
  if (!pdone) {
    draw();
    advance();
  }
  pdl_launch_dependents();
  pdl_wait();
  // ring stages 1 .. early-1 are requested once the activation loads are in flight, the
  // rest after the quantized window has been written
  const bool first_live = m_group[0] >= 0;
  stage_activations_wide<XT>(static_cast<const XT*>(p.x), p.K, smem, blockIdx.x == 0 ? p.scratch : nullptr, [&]() {
    if (split_first && first_live) issue_unit(0, widx, 2);
#pragma unroll
    for (int s = 1; s < STAGES; ++s)
      if (s < p.early) issue(s);
  });
#pragma unroll
  for (int s = 1; s < STAGES; ++s)
    if (s >= p.early) issue(s);
  __syncthreads();

  // ---- this lane's activation window: registers for the rest of the kernel ----
  const int half = lane & 1;
  const int sbl  = lane >> 1;
  const bool active = sbl < csb;
  const int sb   = active ? sbl : 0;
  const uint32_t xr = x_u32 + (sb0 + sb) * kWideRec;
  int4 xg[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) xg[j] = lds128(xr + (8 * half + j) * 16);
  const int4 dxi = lds128(xr + 256 + 16 * half), dsi = lds128(xr + 288 + 16 * half);
  const float4 dxv = make_float4(__int_as_float(dxi.x), __int_as_float(dxi.y), __int_as_float(dxi.z), __int_as_float(dxi.w));
  const float4 dsv = make_float4(__int_as_float(dsi.x), __int_as_float(dsi.y), __int_as_float(dsi.z), __int_as_float(dsi.w));
  const uint32_t lane_blk = sb * 144, qoff = 16 + 64 * half;

  uint32_t phase = 0;
  bool ok = true, more = true, first_round = true;
  while (more) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      if (!more) break;
      if (mg_get(s) < 0) {
        more = false;
        break;
      }
      if (!mbar_wait_bounded(bar_u32 + s * 8, phase)) {
        ok = more = false;
        break;
      }
      const int lrow0 = mg_get(s) * RW;
      int lg;
      const int mat   = matrix_of(c0 + mg_get(s), lg);
      const int nrow  = min(RW, p.rows - lg * RW);
      float acc[RW];
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        acc[r] = 0.f;
        if (r < nrow) {
          const float v = q4k_half_dot(ring_u32 + s * kStage + r * kWideRowPitch + lane_blk, qoff, half, xg, dxv, dsv);
          acc[r] = active ? v : 0.f;
        }
      }
      const float v = reduce_rows<RW>(acc, lane);
      if (lane < nrow) {
        const int lrow = lrow0 + lane;
        if (p.nchunks == 1) store_scalar(y_of(mat) + lg * RW + lane, v);
        else part[lrow * p.nchunks + chunk] = v;
      }
      __syncwarp();   // every lane has read this stage
      issue(s);
      __syncwarp();
    }
    phase ^= 1u;
    first_round = false;
  }
  if (!ok && lane == 0) atomicExch(&g_gemv_status, KDNN_ERR_DEVICE_WAIT);
  if (p.nchunks > 1) {
    __syncthreads();
    const int nloc = min(G * RW, p.rows - c0 * RW);
    for (int r = threadIdx.x; r < nloc; r += blockDim.x) {
      float v = 0.f;
      for (int j = 0; j < p.nchunks; ++j) v += part[r * p.nchunks + j];
      store_scalar(static_cast<YT*>(p.y) + c0 * RW + r, v);   // one matrix per launch on this path
    }
  }
}

// The same structure for the formats evaluated per 64-element item (Q6_K, Q8_0): a warp is
// bound to one 2048-element chunk, lane = item, and the item's activation window (64 int8,
// block scales, for Q6_K the 32 * partial sums) stays in 20-24 registers.
template <uint32_t DT, class XT, class YT, int RW, int STAGES>
__global__ void __launch_bounds__(kGemvMaxWarps * 32, 1) gemv_item_xreg_kernel(const XregParams p) {
  constexpr int kRowPitch = chunk_bytes_full<DT>();
  constexpr int kStage = RW * kRowPitch;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int4* xg      = reinterpret_cast<int4*>(smem);
  float4* hd    = reinterpret_cast<float4*>(smem + static_cast<size_t>(p.nitems) * 64);
  int4* hs      = reinterpret_cast<int4*>(smem + static_cast<size_t>(p.nitems) * 80);
  size_t off    = (static_cast<size_t>(p.nitems) * (DT == KDNN_GGML_Q6_K ? 96 : 80) + 127) & ~size_t(127);
  const uint32_t bar_u32 = smem_u32(smem + off) + warp * (STAGES * 8);
  off += kGemvMaxWarps * STAGES * 8;
  int* s_next = reinterpret_cast<int*>(smem + off);   // [chunk] next local row group
  off += 128;
  float* part = reinterpret_cast<float*>(smem + off);  // [local row][chunk]
  off += (static_cast<size_t>(p.part_floats) * 4 + 127) & ~size_t(127);
  const uint32_t ring_u32 = smem_u32(smem + off) + warp * (STAGES * kStage);

  // even contiguous split of the row groups over the CTAs (quotient and remainder from the host)
  const int c0 = static_cast<int>(blockIdx.x) * p.gq + min(static_cast<int>(blockIdx.x), p.gr);
  const int c1 = c0 + p.gq + (static_cast<int>(blockIdx.x) < p.gr ? 1 : 0);
  const int G  = c1 - c0;                       // row groups of this CTA = units per chunk
  const int widx = static_cast<int>((static_cast<uint32_t>(warp) * p.nch_magic) >> 16), chunk = warp - widx * p.nchunks;
  const int items = min(kChunkItems, p.nitems - chunk * kChunkItems);
  const uint32_t cb = chunk_bytes<DT>(items);
  if (threadIdx.x < p.nchunks) s_next[threadIdx.x] = p.wpc;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bar_u32 + s * 8, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncwarp();

  // ---- producer (state uniform across the warp; lane 0 issues the copies) ----
  int m_group[STAGES];
  auto mg_get = [&](int st) {   // register array read / written with a run-time stage index
    int v = m_group[0];
#pragma unroll
    for (int i = 1; i < STAGES; ++i)
      if (st == i) v = m_group[i];
    return v;
  };
  auto mg_set = [&](int st, int v) {
#pragma unroll
    for (int i = 0; i < STAGES; ++i)
      if (st == i) m_group[i] = v;
  };
  const uint8_t* wsrc = p.w + static_cast<size_t>(chunk) * kRowPitch;
  const bool contiguous = p.nchunks == 1 && p.row_bytes == kRowPitch && cb == static_cast<uint32_t>(kRowPitch);
  auto issue_unit = [&](int s, int u) {
    mg_set(s, u);
    const int row0 = (c0 + u) * RW;
    const int nrow = min(RW, p.rows - row0);
    if (lane == 0) {
      const uint32_t bar = bar_u32 + s * 8;
      mbar_expect_tx(bar, cb * nrow);
      const uint8_t* src = wsrc + static_cast<size_t>(row0) * p.row_bytes;
      const uint32_t dst = ring_u32 + s * kStage;
      if (contiguous) {   // one chunk per row and full rows: the unit is one run of bytes
        bulk_g2s(dst, src, cb * nrow, bar);
      } else {
#pragma unroll
        for (int r = 0; r < RW; ++r)
          if (r < nrow) bulk_g2s(dst + r * kRowPitch, src + static_cast<size_t>(r) * p.row_bytes, cb, bar);
      }
    }
  };
  // The first unit of every warp is fixed and requested at once, before the CTA has even
  // synchronised. Only this one stage goes out before the dependency: a deeper burst ahead
  // of the activation loads makes those loads (a few KB that everything waits for) queue
  // behind megabytes of weights. The rest of the ring is requested right after the
  // activation loads have been issued.
  bool pdone = widx >= G;
  if (!pdone) issue_unit(0, widx); else m_group[0] = -1;
  __syncthreads();   // the chunk counters are set
  int pu = 0, pnext = 0x7fffffff;
  auto draw = [&]() {
    int v = 0;
    if (lane == 0) v = atomicAdd(&s_next[chunk], 1);
    pnext = __shfl_sync(0xFFFFFFFFu, v, 0);
  };
  auto advance = [&]() {
    pu = pnext;
    if (pu >= G) pdone = true; else draw();
  };
  auto issue = [&](int s) {
    if (pdone) {
      mg_set(s, -1);
      return;
    }
    issue_unit(s, pu);
    advance();
  };
  if (!pdone) {
    draw();
    advance();
  }
  pdl_launch_dependents();
  pdl_wait();
  // ring stages 1 .. early-1 are requested once the activation loads are in flight, the
  // rest after the quantized window has been written
  stage_activations<DT, XT>(static_cast<const XT*>(p.x), p.K, p.nitems, xg, hd, hs, blockIdx.x == 0 ? p.scratch : nullptr, [&]() {
#pragma unroll
    for (int s = 1; s < STAGES; ++s)
      if (s < p.early) issue(s);
  });
#pragma unroll
  for (int s = 1; s < STAGES; ++s)
    if (s >= p.early) issue(s);
  __syncthreads();

  // ---- this lane's activation window: registers for the rest of the kernel ----
  const bool active = lane < items;
  const int item = chunk * kChunkItems + (active ? lane : 0);
  ItemX x;
#pragma unroll
  for (int g = 0; g < 4; ++g) x.g[g] = xg[static_cast<size_t>(g) * p.nitems + item];
  x.hd = hd[item];
  x.hs = make_int4(0, 0, 0, 0);
  if (DT == KDNN_GGML_Q6_K) x.hs = hs[item];

  YT* y = static_cast<YT*>(p.y);
  uint32_t phase = 0;
  bool ok = true, more = true, first_round = true;
  // Code size matters here: three big kernels taking turns on a stream (a decoder's Q8_0 / Q4_K / Q6_K projections)
  // evict one another from the instruction cache -- 27.5 us per triple against 24.0 us for the sum of the
  // single-kernel sequences. The stage loop is therefore unrolled only for Q6_K (whose integer-bound inner loop loses
  // 5 % to a run-time stage index); the Q8_0 kernel runs it with a run-time index and is a third smaller.
  constexpr int kUnroll = DT == KDNN_GGML_Q6_K ? STAGES : 1;
  while (more) {
#pragma unroll kUnroll
    for (int s = 0; s < STAGES; ++s) {
      if (!more) break;
      if (mg_get(s) < 0) {
        more = false;
        break;
      }
      if (!mbar_wait_bounded(bar_u32 + s * 8, phase)) {
        ok = more = false;
        break;
      }
      const int lrow0 = mg_get(s) * RW;
      const int nrow  = min(RW, p.rows - (c0 * RW + lrow0));
      float acc[RW];
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        acc[r] = 0.f;
        if (r < nrow) {
          if (active) acc[r] = item_dot<DT>(ring_u32 + s * kStage + r * kRowPitch, lane, x);
        }
      }
      const float v = reduce_rows<RW>(acc, lane);
      if (lane < nrow) {
        const int lrow = lrow0 + lane;
        if (p.nchunks == 1) store_scalar(y + c0 * RW + lrow, v);
        else part[lrow * p.nchunks + chunk] = v;
      }
      __syncwarp();   // every lane has read this stage
      issue(s);
      __syncwarp();
    }
    phase ^= 1u;
    first_round = false;
  }
  if (!ok && lane == 0) atomicExch(&g_gemv_status, KDNN_ERR_DEVICE_WAIT);
  if (p.nchunks > 1) {
    __syncthreads();
    const int nloc = min(G * RW, p.rows - c0 * RW);
    for (int r = threadIdx.x; r < nloc; r += blockDim.x) {
      float v = 0.f;
      for (int j = 0; j < p.nchunks; ++j) v += part[r * p.nchunks + j];
      store_scalar(y + c0 * RW + r, v);
    }
  }
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
  } else if (DT == KDNN_GGML_Q5_K) {   // one whole 32-element sub-block, src/KokkosDNN_GGUFGemvInt8.hpp:389-422
    k0 = c * 32; kb = k0 + 16; h0 = h1 = c;
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
  } else if (DT == KDNN_GGML_Q5_K) {
    const int sub = c & 7, iter = sub >> 1;
    const bool low = (sub & 1) == 0;
    const uint8_t* b  = row + static_cast<size_t>(blk) * 176;
    const uint8_t* qh = b + 16;
    const uint8_t* ql = b + 48 + iter * 32;
    uint32_t scp, mnp;
    q4k_scales(ldg_u16x2(b + 4), ldg_u16x2(b + 8), ldg_u16x2(b + 12), iter, scp, mnp);
    const int sc = low ? (scp & 0xFF) : (scp >> 8), mn = low ? (mnp & 0xFF) : (mnp >> 8);
    const float dw = h2f(ldg_u16x2(b) & 0xFFFFu) * (float)sc * dx0;
    const float dm = h2f(ldg_u16x2(b) >> 16) * (float)mn * dx0;
    const uint32_t sh = low ? 0u : 4u, bitsh = static_cast<uint32_t>(sub);
    uint32_t w0[4], w1[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w0[i] = ((ldg_u16x2(ql + 4 * i) >> sh) & 0x0F0F0F0Fu) | (((ldg_u16x2(qh + 4 * i) >> bitsh) & 0x01010101u) << 4);
      w1[i] = ((ldg_u16x2(ql + 16 + 4 * i) >> sh) & 0x0F0F0F0Fu) |
              (((ldg_u16x2(qh + 16 + 4 * i) >> bitsh) & 0x01010101u) << 4);
    }
    ints[0] = dot16(w1, xb, dot16(w0, xa, 0));
    ints[1] = 0;
    return dw * (float)ints[0] - dm * (float)(xh[h0].sum_lo + xh[h0].sum_hi);
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
__global__ void quantize_act_kernel(const XT* x, int K, uint8_t* scratch) {
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
__global__ void gemv_generic_kernel(const uint8_t* w, size_t row_bytes, int rows,
                                    int K, const uint8_t* scratch, YT* y) {
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
__global__ void unit_dots_kernel(const uint8_t* w, size_t row_bytes, int rows, int K,
                                 const uint8_t* scratch, int32_t* out) {
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

static bool use_pdl() { return pdl_enabled() && t_lay.no_pdl == 0; }


static thread_local bool t_ring_does_not_fit = false;

// Work split of one launch. All 16 warps (the kernel is bound by instruction issue, and
// fewer warps measured slower even where they would fill the last round better); a unit is
// a whole row group when every warp gets several of them, otherwise the rows are cut into
// chunk ranges until there are about two units per warp.
struct GemvSplit { int cpu, upg, warps; };
static GemvSplit choose_split(int ngroups, int nchunks, int grid) {
  const int gpc = (ngroups + grid - 1) / grid;   // row groups of the largest CTA slice
  int upg = 1;
  if (gpc < kGemvMaxWarps) upg = min(nchunks, (2 * kGemvMaxWarps + gpc - 1) / gpc);
  const int cpu = (nchunks + upg - 1) / upg;
  return GemvSplit{cpu, (nchunks + cpu - 1) / cpu, kGemvMaxWarps};
}

template <uint32_t DT, int RW, class XT, class YT>
static cudaError_t launch_stream(const GemvParams& base, cudaStream_t stream) {
  const DeviceInfo& di = device_info();
  GemvParams p = base;
  p.ngroups     = (p.rows + RW - 1) / RW;
  p.stage_bytes = (RW * chunk_bytes_full<DT>() + 127) & ~127;
  const int grid = max(1, min(di.sms, p.ngroups));
  p.gq = p.ngroups / grid;
  p.gr = p.ngroups % grid;
  GemvSplit sp = choose_split(p.ngroups, p.nchunks, grid);
  if (const int w = t_lay.warps) sp.warps = max(1, min(kGemvMaxWarps, w));
  const int gpc = (p.ngroups + grid - 1) / grid;
  if (sp.upg > 1 && static_cast<size_t>(gpc + 1) * RW * sp.upg * 4 > 48 * 1024) {   // partial sums would not fit
    sp.cpu = p.nchunks;
    sp.upg = 1;
  }
  p.cpu         = sp.cpu;
  p.upg         = sp.upg;
  p.upg_magic   = static_cast<uint32_t>((0x100000000ull + sp.upg - 1) / sp.upg);
  p.part_floats = sp.upg > 1 ? (gpc + 1) * RW * sp.upg : 0;
  const size_t act = ((static_cast<size_t>(p.nitems) * (DT == KDNN_GGML_Q6_K ? 96 : 80)) + 127) & ~size_t(127);
  const size_t smem = act + kGemvMaxWarps * kGemvStages * 8 + 128 +
                      ((static_cast<size_t>(p.part_floats) * 4 + 127) & ~size_t(127)) +
                      static_cast<size_t>(kGemvMaxWarps) * kGemvStages * p.stage_bytes + 128;
  if (smem > static_cast<size_t>(di.max_smem)) {
    t_ring_does_not_fit = true;   // the caller takes the plain-load kernel instead
    return cudaSuccess;
  }
  auto kern = gemv_stream_kernel<DT, RW, XT, YT>;
  static SmemAttrOnce once;
  if (const cudaError_t e = set_max_smem_once(once, kern, di.max_smem)) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(sp.warps * 32); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = use_pdl() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

// Returns false when the shape is outside what the register-window kernel covers.
template <class XT, class YT, int RW>
static bool launch_q4k_xreg(const GemvParams& base, cudaStream_t stream, cudaError_t& err) {
  const DeviceInfo& di = device_info();
  XregParams p{};
  p.w = base.w; p.x = base.x; p.y = base.y; p.scratch = base.scratch;
  p.rows = base.rows; p.K = base.K; p.row_bytes = base.row_bytes;
  p.nsb     = base.K / 256;
  p.nchunks = (p.nsb + kWideSb - 1) / kWideSb;
  if (p.nchunks > kGemvMaxWarps) return false;
  p.csb     = (p.nsb + p.nchunks - 1) / p.nchunks;   // near-equal chunks
  p.nchunks = (p.nsb + p.csb - 1) / p.csb;
  p.gpm     = (p.rows + RW - 1) / RW;
  p.nmat    = base.nmat > 1 ? base.nmat : 1;
  if (p.nmat > 1 && p.nchunks != 1) return false;   // several matrices per launch: rows of one chunk only
  for (int i = 0; i < 3; ++i) { p.w_more[i] = base.w_more[i]; p.y_more[i] = base.y_more[i]; }
  p.ngroups = p.gpm * p.nmat;
  const int grid  = max(1, min(di.sms, p.ngroups));
  const int gpc0  = (p.ngroups + grid - 1) / grid;
  // Warps per chunk: units are equal-sized and handed out dynamically, so a CTA takes
  // ceil(units / warps) unit times; with one chunk per row one or two warps beyond 16 are added when
  // that saves a round (49 row groups: 17 warps finish in 3 rounds, 16 need a fourth).
  p.wpc = kGemvMaxWarps / p.nchunks;
  if (p.nchunks == 1) {
    int best = kGemvMaxWarps, best_rounds = (gpc0 + kGemvMaxWarps - 1) / kGemvMaxWarps;
    for (int w = kGemvMaxWarps + 1; w <= kXregMaxWarps; ++w) {
      const int rounds = (gpc0 + w - 1) / w;
      if (rounds < best_rounds) {
        best = w;
        best_rounds = rounds;
      }
    }
    p.wpc = best;
  }
  if (const int w = t_lay.warps) p.wpc = max(1, max(1, min(kXregMaxWarps, w)) / p.nchunks);
  const int warps = p.wpc * p.nchunks;
  p.gq = p.ngroups / grid;
  p.gr = p.ngroups % grid;
  p.nch_magic = static_cast<uint32_t>((65536 + p.nchunks - 1) / p.nchunks);
  const int gpc   = (p.ngroups + grid - 1) / grid;
  p.part_floats   = p.nchunks > 1 ? (gpc + 1) * RW * p.nchunks : 0;
  if (static_cast<size_t>(p.part_floats) * 4 > 32 * 1024) return false;
  const size_t fixed = ((static_cast<size_t>(p.nsb) * kWideRec + 127) & ~size_t(127)) + 128 +
                       ((static_cast<size_t>(p.part_floats) * 4 + 127) & ~size_t(127)) + 128;
  constexpr int kStage = RW * kWideRowPitch;
  auto smem_for = [&](int st) { return fixed + static_cast<size_t>(kXregMaxWarps) * st * 8 + static_cast<size_t>(warps) * st * kStage; };
  const int units_per_warp = (gpc + p.wpc - 1) / p.wpc;
  int stages = t_lay.stages;
  if (stages == 0) stages = 3;
  stages = max(2, min(4, min(stages, max(2, units_per_warp))));
  while (stages > 2 && smem_for(stages) > static_cast<size_t>(di.max_smem)) --stages;
  if (smem_for(stages) > static_cast<size_t>(di.max_smem)) return false;
  const size_t smem = smem_for(stages);
  p.early  = t_lay.early_stages > 0 ? t_lay.early_stages : 2;
  // When every warp has at most one unit the whole matrix would be requested before the dependency and
  // the activation loads would queue behind all of it: request half of it first, the rest behind those loads.
  p.split_first = gpc <= p.wpc ? 1 : 0;
  using Kern = void (*)(const XregParams);
  const bool multi = p.nmat > 1;
  const Kern kern = multi ? (stages == 2 ? gemv_q4k_xreg_kernel<XT, YT, RW, 2, true>
                             : stages == 3 ? gemv_q4k_xreg_kernel<XT, YT, RW, 3, true> : gemv_q4k_xreg_kernel<XT, YT, RW, 4, true>)
                          : (stages == 2 ? gemv_q4k_xreg_kernel<XT, YT, RW, 2, false>
                             : stages == 3 ? gemv_q4k_xreg_kernel<XT, YT, RW, 3, false> : gemv_q4k_xreg_kernel<XT, YT, RW, 4, false>);
  static SmemAttrOnce once[2][5];
  err = set_max_smem_once(once[multi][stages], kern, di.max_smem);
  if (err != cudaSuccess) return true;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(warps * 32); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = use_pdl() ? 1 : 0;
  err = cudaLaunchKernelEx(&cfg, kern, p);
  return true;
}

// Register-window kernel for the item formats. Returns false when the shape is outside what it covers.
template <uint32_t DT, class XT, class YT, int RW>
static bool launch_item_xreg(const GemvParams& base, cudaStream_t stream, cudaError_t& err) {
  const DeviceInfo& di = device_info();
  XregParams p{};
  p.w = base.w; p.x = base.x; p.y = base.y; p.scratch = base.scratch;
  p.rows = base.rows; p.K = base.K; p.row_bytes = base.row_bytes;
  p.nitems  = base.nitems;
  p.nchunks = base.nchunks;
  if (p.nchunks > kGemvMaxWarps) return false;
  p.ngroups = (p.rows + RW - 1) / RW;
  p.wpc     = kGemvMaxWarps / p.nchunks;
  const int warps = p.wpc * p.nchunks;
  const int grid  = max(1, min(di.sms, p.ngroups));
  p.gq = p.ngroups / grid;
  p.gr = p.ngroups % grid;
  p.nch_magic = static_cast<uint32_t>((65536 + p.nchunks - 1) / p.nchunks);
  const int gpc   = (p.ngroups + grid - 1) / grid;
  p.part_floats   = p.nchunks > 1 ? (gpc + 1) * RW * p.nchunks : 0;
  if (static_cast<size_t>(p.part_floats) * 4 > 32 * 1024) return false;
  const size_t fixed = ((static_cast<size_t>(p.nitems) * (DT == KDNN_GGML_Q6_K ? 96 : 80) + 127) & ~size_t(127)) + 128 +
                       ((static_cast<size_t>(p.part_floats) * 4 + 127) & ~size_t(127)) + 128;
  constexpr int kStage = RW * chunk_bytes_full<DT>();
  auto smem_for = [&](int st) { return fixed + static_cast<size_t>(kGemvMaxWarps) * st * (8 + kStage); };
  const int units_per_warp = (gpc + p.wpc - 1) / p.wpc;
  int stages = t_lay.stages;
  if (stages == 0) stages = DT == KDNN_GGML_Q6_K ? 2 : 3;   // measured: two stages are the best Q6_K point (11.9 against 12.4 us)
  stages = max(2, min(4, min(stages, max(2, units_per_warp))));
  while (stages > 2 && smem_for(stages) > static_cast<size_t>(di.max_smem)) --stages;
  if (smem_for(stages) > static_cast<size_t>(di.max_smem)) return false;
  const size_t smem = smem_for(stages);
  p.early  = t_lay.early_stages > 0 ? t_lay.early_stages : 2;
  using Kern = void (*)(const XregParams);
  const Kern kern = stages == 2 ? gemv_item_xreg_kernel<DT, XT, YT, RW, 2>
                  : stages == 3 ? gemv_item_xreg_kernel<DT, XT, YT, RW, 3> : gemv_item_xreg_kernel<DT, XT, YT, RW, 4>;
  static SmemAttrOnce once[5];
  err = set_max_smem_once(once[stages], kern, di.max_smem);
  if (err != cudaSuccess) return true;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(warps * 32); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = use_pdl() ? 1 : 0;
  err = cudaLaunchKernelEx(&cfg, kern, p);
  return true;
}

template <class XT, class YT>
static cudaError_t launch_q4k_wide(const GemvParams& base, cudaStream_t stream) {
  const DeviceInfo& di = device_info();
  WideParams p{};
  p.w = base.w; p.x = base.x; p.y = base.y; p.scratch = base.scratch;
  p.rows = base.rows; p.K = base.K; p.row_bytes = base.row_bytes;
  p.nsb     = base.K / 256;
  p.nchunks = (p.nsb + kWideSb - 1) / kWideSb;
  p.csb     = (p.nsb + p.nchunks - 1) / p.nchunks;   // near-equal chunks
  p.nchunks = (p.nsb + p.csb - 1) / p.csb;
  p.ngroups = (p.rows + 1) / 2;
  const int grid = max(1, min(di.sms, p.ngroups));
  p.gq = p.ngroups / grid;
  p.gr = p.ngroups % grid;
  GemvSplit sp = choose_split(p.ngroups, p.nchunks, grid);
  if (const int w = t_lay.warps) sp.warps = max(1, min(kGemvMaxWarps, w));
  const int gpc = (p.ngroups + grid - 1) / grid;
  if (sp.upg > 1 && static_cast<size_t>(gpc + 1) * 2 * sp.upg * 4 > 32 * 1024) {
    sp.cpu = p.nchunks;
    sp.upg = 1;
  }
  p.cpu         = sp.cpu;
  p.upg         = sp.upg;
  p.upg_magic   = static_cast<uint32_t>((0x100000000ull + sp.upg - 1) / sp.upg);
  p.part_floats = sp.upg > 1 ? (gpc + 1) * 2 * sp.upg : 0;
  const int maxw = sp.warps <= 8 ? 8 : kGemvMaxWarps;
  // Ring depth: as many stages as fit (up to 4) but no more than a warp has units to fetch;
  // with few units per warp the whole slice is requested at kernel entry.
  const size_t fixed = ((static_cast<size_t>(p.nsb) * kWideRec + 127) & ~size_t(127)) + 128 +
                       ((static_cast<size_t>(p.part_floats) * 4 + 127) & ~size_t(127)) + 128;
  auto smem_for = [&](int st) { return fixed + static_cast<size_t>(maxw) * st * (8 + kWideStage); };
  const size_t cap = maxw == 8 ? static_cast<size_t>(di.max_smem) / 2 - 1024 : static_cast<size_t>(di.max_smem);
  const int chunks_per_warp = (gpc * p.nchunks + sp.warps - 1) / sp.warps;
  int stages = t_lay.stages;
  if (stages == 0) stages = max(2, min(4, chunks_per_warp));
  stages = max(2, min(4, stages));
  while (stages > 2 && smem_for(stages) > cap) --stages;
  if (smem_for(stages) > cap) {
    t_ring_does_not_fit = true;
    return cudaSuccess;
  }
  const size_t smem = smem_for(stages);
  using Kern = void (*)(const WideParams);
  Kern kern;
  if (maxw == 8)
    kern = stages == 2 ? gemv_q4k_wide_kernel<XT, YT, 8, 2> : stages == 3 ? gemv_q4k_wide_kernel<XT, YT, 8, 3>
                                                                            : gemv_q4k_wide_kernel<XT, YT, 8, 4>;
  else
    kern = stages == 2 ? gemv_q4k_wide_kernel<XT, YT, 16, 2> : stages == 3 ? gemv_q4k_wide_kernel<XT, YT, 16, 3>
                                                                             : gemv_q4k_wide_kernel<XT, YT, 16, 4>;
  static SmemAttrOnce once[2][5];
  if (const cudaError_t e = set_max_smem_once(once[maxw == 8][stages], kern, static_cast<int>(cap))) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(sp.warps * 32); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = use_pdl() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <uint32_t DT, class XT, class YT>
static cudaError_t launch_stream_rw(const GemvParams& p, cudaStream_t stream) {
  // Rows per group: two rows share one load of the activation window and one pass of
  // the loop bookkeeping.
  int rw = t_lay.rows_per_group;
  const int kk = t_lay.kernel;   // 0 / 1: register window, 2: shared-memory window, 3: item mapping with the window in shared memory
  if (DT == KDNN_GGML_Q4_K && kk != 3) {
    cudaError_t err = cudaSuccess;
    if (kk != 2) {
      if (rw == 1 ? launch_q4k_xreg<XT, YT, 1>(p, stream, err) : launch_q4k_xreg<XT, YT, 2>(p, stream, err)) return err;
    }
    return launch_q4k_wide<XT, YT>(p, stream);
  }
  if (DT != KDNN_GGML_Q4_K && kk != 2 && kk != 3) {   // register-window kernel for Q6_K / Q8_0
    cudaError_t err = cudaSuccess;
    if (rw == 1 ? launch_item_xreg<DT, XT, YT, 1>(p, stream, err) : launch_item_xreg<DT, XT, YT, 2>(p, stream, err)) return err;
  }
  if (rw == 0) rw = p.rows >= 2 ? 2 : 1;
  if (rw >= 4 && DT == KDNN_GGML_Q4_K) return launch_stream<DT, 4, XT, YT>(p, stream);
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

// Entry used by the C ABI. `layout` (may be null) carries the caller's tuning; kernel 4 selects the
// plain-load kernels.
cudaError_t gemv_launch(uint32_t dt, const void* w, size_t rows, size_t cols, const void* x, int xs,
                        void* y, int ys, void* scratch, const kdnn_b200_gemv_layout* layout, cudaStream_t stream) {
  t_lay = layout != nullptr ? *layout : kdnn_b200_gemv_layout{};
  const bool force_generic = t_lay.kernel == 4;
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
    t_ring_does_not_fit = false;
    switch (dt) {
      case KDNN_GGML_Q4_K: e = launch_stream_dt<KDNN_GGML_Q4_K>(p, xs, ys, stream); break;
      case KDNN_GGML_Q5_K: e = launch_stream_dt<KDNN_GGML_Q5_K>(p, xs, ys, stream); break;
      case KDNN_GGML_Q6_K: e = launch_stream_dt<KDNN_GGML_Q6_K>(p, xs, ys, stream); break;
      default: e = launch_stream_dt<KDNN_GGML_Q8_0>(p, xs, ys, stream); break;
    }
    if (!t_ring_does_not_fit) return e;   // launched, or a real error: never masked by the plain-load kernel
    // activation row too long for shared memory next to the ring: plain loads
  }
  const uint8_t* wb = static_cast<const uint8_t*>(w);
  uint8_t* sb       = static_cast<uint8_t*>(scratch);
  switch (dt) {
    case KDNN_GGML_Q4_K: return launch_generic_dt<KDNN_GGML_Q4_K>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, sb, stream);
    case KDNN_GGML_Q5_K: return launch_generic_dt<KDNN_GGML_Q5_K>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, sb, stream);
    case KDNN_GGML_Q6_K: return launch_generic_dt<KDNN_GGML_Q6_K>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, sb, stream);
    default: return launch_generic_dt<KDNN_GGML_Q8_0>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, sb, stream);
  }
}

// n (2..4) matrices of one format and shape against the SAME activation row in one launch (a decoder's gate
// and up projections, or q / k / v of equal width): the launch-sized ramp and tail are paid once. Covered by
// the Q4_K register-window kernel for rows of one chunk (K <= 4096); everything else runs as n launches.
cudaError_t gemv_multi_launch(uint32_t dt, int n, const void* const* w, size_t rows, size_t cols, const void* x, int xs,
                              void* const* y, int ys, void* scratch, const kdnn_b200_gemv_layout* layout,
                              cudaStream_t stream) {
  const size_t rb = row_bytes_of(dt, cols);
  bool fused = dt == KDNN_GGML_Q4_K && n >= 2 && n <= 4 && rb % 16 == 0 && cols % 256 == 0 && rb <= INT_MAX &&
               rows * static_cast<size_t>(n) <= static_cast<size_t>(INT_MAX) && !(layout && layout->kernel >= 2);
  for (int i = 0; i < n && fused; ++i) fused = (reinterpret_cast<uintptr_t>(w[i]) & 15u) == 0;
  if (fused) {
    t_lay = layout != nullptr ? *layout : kdnn_b200_gemv_layout{};
    GemvParams p{};
    p.w = static_cast<const uint8_t*>(w[0]); p.x = x; p.y = y[0]; p.scratch = static_cast<uint8_t*>(scratch);
    p.rows = static_cast<int>(rows); p.K = static_cast<int>(cols); p.row_bytes = static_cast<int>(rb);
    p.nitems = static_cast<int>(cols / 64); p.nchunks = (p.nitems + kChunkItems - 1) / kChunkItems;
    p.nmat = n;
    for (int i = 1; i < n; ++i) { p.w_more[i - 1] = static_cast<const uint8_t*>(w[i]); p.y_more[i - 1] = y[i]; }
    cudaError_t err = cudaSuccess;
    bool done = false;
    const int rw = t_lay.rows_per_group == 1 ? 1 : 2;
    if (xs == KDNN_F32 && ys == KDNN_F32)
      done = rw == 1 ? launch_q4k_xreg<float, float, 1>(p, stream, err) : launch_q4k_xreg<float, float, 2>(p, stream, err);
    else if (xs == KDNN_BF16 && ys == KDNN_BF16)
      done = rw == 1 ? launch_q4k_xreg<__nv_bfloat16, __nv_bfloat16, 1>(p, stream, err)
                     : launch_q4k_xreg<__nv_bfloat16, __nv_bfloat16, 2>(p, stream, err);
    else if (xs == KDNN_BF16 && ys == KDNN_F32)
      done = rw == 1 ? launch_q4k_xreg<__nv_bfloat16, float, 1>(p, stream, err)
                     : launch_q4k_xreg<__nv_bfloat16, float, 2>(p, stream, err);
    else
      done = rw == 1 ? launch_q4k_xreg<float, __nv_bfloat16, 1>(p, stream, err)
                     : launch_q4k_xreg<float, __nv_bfloat16, 2>(p, stream, err);
    if (done) return err;
  }
  for (int i = 0; i < n; ++i) {
    const cudaError_t e = gemv_launch(dt, w[i], rows, cols, x, xs, y[i], ys, scratch, layout, stream);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
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
    case KDNN_GGML_Q5_K: unit_dots_kernel<KDNN_GGML_Q5_K><<<blocks, 256, 0, st>>>(wb, rb, (int)rows, (int)cols, sb, out); break;
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

extern "C" int kdnn_b200_quant_gemv_noalloc_ex(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                                               const void* x, int x_scalar, void* y, int y_scalar,
                                               const kdnn_b200_gemv_layout* layout, void* stream) {
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
  if (ggml_type != KDNN_GGML_Q4_K && ggml_type != KDNN_GGML_Q5_K && ggml_type != KDNN_GGML_Q6_K && ggml_type != KDNN_GGML_Q8_0)
    return KDNN_DECLINED;
  if (w == nullptr || x == nullptr || y == nullptr) return KDNN_DECLINED;
  if (!block_aligned(ggml_type, cols)) return KDNN_DECLINED;
  if (rows == 0 || rows > static_cast<size_t>(INT_MAX)) return KDNN_DECLINED;
  if ((reinterpret_cast<uintptr_t>(w) & 1u) != 0u) return KDNN_DECLINED;
  if ((ggml_type == KDNN_GGML_Q4_K || ggml_type == KDNN_GGML_Q5_K) && (reinterpret_cast<uintptr_t>(w) & 15u) != 0u) return KDNN_DECLINED;
  uint8_t* staging = nullptr;
  cudaError_t e = noalloc_staging_address(&staging);
  if (e == cudaSuccess)
    e = gemv_launch(ggml_type, w, rows, cols, x, x_scalar, y, y_scalar, staging, layout,
                    static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    set_last_error((std::string("quant_gemv_noalloc: ") + cudaGetErrorString(e)).c_str());
    return KDNN_ERR_CUDA;
  }
  return KDNN_OK;
}

extern "C" int kdnn_b200_quant_gemv_noalloc(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                                            const void* x, int x_scalar, void* y, int y_scalar,
                                            void* stream) {
  return kdnn_b200_quant_gemv_noalloc_ex(ggml_type, w, rows, cols, x, x_scalar, y, y_scalar, nullptr, stream);
}
