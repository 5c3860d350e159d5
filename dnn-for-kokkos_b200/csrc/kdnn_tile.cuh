// Shared pieces of the batched (several activation rows per weight row) int8
// kernels: the per-token activation item staged in shared memory and the
// per-format weight item held in registers.
//
// Work split: one LANE owns one weight row and walks its 64-element items; the
// activation side of an item is the same for every lane of the warp, so its
// shared-memory loads are broadcasts. Per item the lane unpacks the weights to
// int8 words once and reuses them for every token of the tile.
#pragma once

#include "kdnn_common.cuh"

namespace kdnn {

// One token's view of one 64-element item: four 16-byte int8 granules, the
// fp32 scale of the 32-block each granule lies in, and each granule's int sum.
struct __align__(16) ActItem {
  int4 g[4];
  float dx[4];
  int sum[4];
};
static_assert(sizeof(ActItem) == 96, "ActItem is six 16-byte loads");

template <uint32_t DT>
__device__ __forceinline__ void granule_map(int b, int p, int& item, int& g) {
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

// ---- weight item in registers ------------------------------------------------
// w[g][i]: int8 words of granule g. The fp32 fields are the weight-side factors.
template <uint32_t DT>
struct WItem;

__device__ __forceinline__ int4 ldg128(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_u16x2_nc(const uint8_t* p) {
  const unsigned short* q = reinterpret_cast<const unsigned short*>(p);
  return static_cast<uint32_t>(__ldg(q)) | (static_cast<uint32_t>(__ldg(q + 1)) << 16);
}

__device__ __forceinline__ void q4k_scale_pair(uint32_t s0, uint32_t s1, uint32_t s2, int it,
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

template <>
struct WItem<KDNN_GGML_Q4_K> {
  uint32_t w[4][4];
  float s0, s1, m0, m1;  // d*sc0, d*sc1, dmin*mn0, dmin*mn1
  // row: first byte of the packed row (16-byte aligned); item: index in the row
  __device__ __forceinline__ void load(const uint8_t* row, int item) {
    const uint8_t* blk = row + static_cast<size_t>(item >> 2) * 144;
    const int4 h       = ldg128(blk);
    const int4 qa      = ldg128(blk + 16 + (item & 3) * 32);
    const int4 qb      = ldg128(blk + 32 + (item & 3) * 32);
    uint32_t scp, mnp;
    q4k_scale_pair(h.y, h.z, h.w, item & 3, scp, mnp);
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
    s0 = dd.x * static_cast<float>(scp & 0xFF);
    s1 = dd.x * static_cast<float>(scp >> 8);
    m0 = dd.y * static_cast<float>(mnp & 0xFF);
    m1 = dd.y * static_cast<float>(mnp >> 8);
    const uint32_t q[8] = {(uint32_t)qa.x, (uint32_t)qa.y, (uint32_t)qa.z, (uint32_t)qa.w,
                           (uint32_t)qb.x, (uint32_t)qb.y, (uint32_t)qb.z, (uint32_t)qb.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[0][i] = q[i] & 0x0F0F0F0Fu;
      w[1][i] = q[4 + i] & 0x0F0F0F0Fu;
      w[2][i] = (q[i] >> 4) & 0x0F0F0F0Fu;
      w[3][i] = (q[4 + i] >> 4) & 0x0F0F0F0Fu;
    }
  }
  __device__ __forceinline__ float dot(const ActItem& a) const {
    const int dA = dot16(w[1], a.g[1], dot16(w[0], a.g[0], 0));
    const int dB = dot16(w[3], a.g[3], dot16(w[2], a.g[2], 0));
    const float p = s0 * (static_cast<float>(dA) * a.dx[0]) + s1 * (static_cast<float>(dB) * a.dx[2]);
    const float m = m0 * (static_cast<float>(a.sum[0] + a.sum[1]) * a.dx[0]) +
                    m1 * (static_cast<float>(a.sum[2] + a.sum[3]) * a.dx[2]);
    return p - m;
  }
};

// Q5_K: Q4_K's nibbles plus the fifth bit of sub-block j in bit j of qh[l] (src/KokkosDNN_GGUFGemvInt8.hpp:389-422);
// the words hold the complete 5-bit values, the rest is the Q4_K arithmetic.
template <>
struct WItem<KDNN_GGML_Q5_K> {
  uint32_t w[4][4];
  float s0, s1, m0, m1;  // d*sc0, d*sc1, dmin*mn0, dmin*mn1
  __device__ __forceinline__ void load(const uint8_t* row, int item) {
    const uint8_t* blk = row + static_cast<size_t>(item >> 2) * 176;
    const int it       = item & 3;
    const int4 h       = ldg128(blk);
    const int4 h0      = ldg128(blk + 16), h1 = ldg128(blk + 32);
    const int4 qa      = ldg128(blk + 48 + it * 32);
    const int4 qb      = ldg128(blk + 64 + it * 32);
    uint32_t scp, mnp;
    q4k_scale_pair(h.y, h.z, h.w, it, scp, mnp);
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
    s0 = dd.x * static_cast<float>(scp & 0xFF);
    s1 = dd.x * static_cast<float>(scp >> 8);
    m0 = dd.y * static_cast<float>(mnp & 0xFF);
    m1 = dd.y * static_cast<float>(mnp >> 8);
    const uint32_t q[8]  = {(uint32_t)qa.x, (uint32_t)qa.y, (uint32_t)qa.z, (uint32_t)qa.w,
                            (uint32_t)qb.x, (uint32_t)qb.y, (uint32_t)qb.z, (uint32_t)qb.w};
    const uint32_t hh[8] = {(uint32_t)h0.x, (uint32_t)h0.y, (uint32_t)h0.z, (uint32_t)h0.w,
                            (uint32_t)h1.x, (uint32_t)h1.y, (uint32_t)h1.z, (uint32_t)h1.w};
    const uint32_t sh = 2 * it;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t t0 = hh[i] >> sh, t1 = hh[4 + i] >> sh;
      w[0][i] = (q[i] & 0x0F0F0F0Fu) | ((t0 & 0x01010101u) << 4);
      w[1][i] = (q[4 + i] & 0x0F0F0F0Fu) | ((t1 & 0x01010101u) << 4);
      w[2][i] = ((q[i] >> 4) & 0x0F0F0F0Fu) | ((t0 & 0x02020202u) << 3);
      w[3][i] = ((q[4 + i] >> 4) & 0x0F0F0F0Fu) | ((t1 & 0x02020202u) << 3);
    }
  }
  __device__ __forceinline__ float dot(const ActItem& a) const {
    const int dA = dot16(w[1], a.g[1], dot16(w[0], a.g[0], 0));
    const int dB = dot16(w[3], a.g[3], dot16(w[2], a.g[2], 0));
    const float p = s0 * (static_cast<float>(dA) * a.dx[0]) + s1 * (static_cast<float>(dB) * a.dx[2]);
    const float m = m0 * (static_cast<float>(a.sum[0] + a.sum[1]) * a.dx[0]) +
                    m1 * (static_cast<float>(a.sum[2] + a.sum[3]) * a.dx[2]);
    return p - m;
  }
};

template <>
struct WItem<KDNN_GGML_Q6_K> {
  uint32_t w[4][4];
  float s[4];  // d * scales[...] of the four 16-element groups
  __device__ __forceinline__ void load(const uint8_t* row, int item) {
    const int chunk = (item >> 1) & 1, half = item & 1;
    const uint8_t* blk = row + static_cast<size_t>(item >> 2) * 210;
    const uint8_t* ql  = blk + chunk * 64 + half * 16;
    const uint8_t* qh  = blk + 128 + chunk * 32 + half * 16;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t l0 = ldg_u16x2_nc(ql + 4 * i), l1 = ldg_u16x2_nc(ql + 32 + 4 * i);
      const uint32_t h  = ldg_u16x2_nc(qh + 4 * i);
      w[0][i] = (l0 & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
      w[1][i] = (l1 & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
      w[2][i] = ((l0 >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
      w[3][i] = ((l1 >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
    }
    const float d     = h2f(__ldg(reinterpret_cast<const unsigned short*>(blk + 208)));
    const int8_t* scl = reinterpret_cast<const int8_t*>(blk + 192 + chunk * 8 + half);
#pragma unroll
    for (int g = 0; g < 4; ++g) s[g] = d * static_cast<float>(__ldg(scl + 2 * g));
  }
  __device__ __forceinline__ float dot(const ActItem& a) const {
    float acc = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int v = dot16(w[g], a.g[g], 0) - (a.sum[g] << 5);
      acc += s[g] * (static_cast<float>(v) * a.dx[g]);
    }
    return acc;
  }
};

template <>
struct WItem<KDNN_GGML_Q8_0> {
  uint32_t w[4][4];
  float d0, d1;
  __device__ __forceinline__ void load(const uint8_t* row, int item) {
    const uint8_t* b = row + static_cast<size_t>(item) * 68;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[0][i] = ldg_u16x2_nc(b + 2 + 4 * i);
      w[1][i] = ldg_u16x2_nc(b + 18 + 4 * i);
      w[2][i] = ldg_u16x2_nc(b + 36 + 4 * i);
      w[3][i] = ldg_u16x2_nc(b + 52 + 4 * i);
    }
    d0 = h2f(__ldg(reinterpret_cast<const unsigned short*>(b)));
    d1 = h2f(__ldg(reinterpret_cast<const unsigned short*>(b + 34)));
  }
  __device__ __forceinline__ float dot(const ActItem& a) const {
    const int x0 = dot16(w[1], a.g[1], dot16(w[0], a.g[0], 0));
    const int x1 = dot16(w[3], a.g[3], dot16(w[2], a.g[2], 0));
    return (d0 * a.dx[0]) * static_cast<float>(x0) + (d1 * a.dx[2]) * static_cast<float>(x1);
  }
};

// shared-memory ActItem as six broadcast 128-bit loads
__device__ __forceinline__ ActItem lds_item(const ActItem* p) {
  ActItem a;
  const int4* q = reinterpret_cast<const int4*>(p);
#pragma unroll
  for (int g = 0; g < 4; ++g) a.g[g] = q[g];
  const int4 d = q[4], s = q[5];
  a.dx[0] = __int_as_float(d.x); a.dx[1] = __int_as_float(d.y);
  a.dx[2] = __int_as_float(d.z); a.dx[3] = __int_as_float(d.w);
  a.sum[0] = s.x; a.sum[1] = s.y; a.sum[2] = s.z; a.sum[3] = s.w;
  return a;
}

}  // namespace kdnn
