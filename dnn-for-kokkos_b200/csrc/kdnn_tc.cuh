// Grouped int8 tile GEMM for Q4_K weights on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory), as ONE persistent,
// warp-specialised kernel per launch: a CTA per SM walks the tiles
// (group of <= 32 activation rows) x (128 weight rows) and never drains its
// pipeline between tiles, so the next tile's packed rows are already in flight
// while the current tile is being folded.
//
//   warp 12      producer: per 256-element super-block of K one stage of the ring =
//                128 packed rows x 144 bytes by tensor-map TMA (cp.async.bulk.tensor.2d,
//                32-row boxes, this GPU's memory only, no multicast) + the group's
//                quantized activation bytes and block scales by 1-D bulk copies
//   warps 8-11   unpack: thread = weight row; nibbles -> int8 in the K-major core-matrix
//                layout the MMA reads (eight 128 x 32 A tiles per stage), the 6-bit scales
//                and mins -> fp32 tables, activations -> eight 32 x 32 B tiles
//   warp 13      one thread issues eight tcgen05.mma per stage (one per 32-element
//                sub-block, each into its own 32-column TMEM slot: every sub-block has its
//                own scale on both sides, so nothing accumulates across them in TMEM) and
//                commits them to an mbarrier; two slot groups (2 x 256 columns) rotate
//   warps 0-7    drain: thread = (weight row, half of the activation rows); tcgen05.ld of
//                its TMEM lane, fold  acc += (d*sc) * dx * dot - (dmin*mn) * dx * sum  in
//                fp32 registers while the other slot group is being filled, then the
//                epilogue (SwiGLU + per-32 int8 quantization of the result for the
//                gate/up call; plain stores otherwise)
//
// The integer sub-block dots are exact (one MMA = one sub-block), as on the dp4a and
// mma.sync paths. Every wait is bounded; a wait that gives up raises a CTA-wide abort
// flag, records KDNN_ERR_DEVICE_WAIT in the status word, the producer waits (bounded) for
// its copies in flight, and the CTA frees its TMEM and returns.
#pragma once

#include <cuda.h>

#include <atomic>

#include "kdnn_mma.cuh"

namespace kdnn {

constexpr int kTcNT       = 32;                 // activation rows per group (MMA N)
constexpr int kTcBoxRows  = 32;                 // rows of one TMA box
constexpr int kTcWStage   = 128 * 144;          // packed rows of one stage
constexpr int kTcXq       = kTcNT * 256;        // int8 activations of one stage
constexpr int kTcXs       = kTcNT * 64;         // {d, d * sum} of the stage's eight 32-blocks per row
constexpr int kTcXStage   = kTcXq + kTcXs;
constexpr int kTcATile    = 128 * 32;
constexpr int kTcBTile    = kTcNT * 32;
constexpr int kTcThreads  = 14 * 32;
constexpr uint32_t kTcCols = 512;               // TMEM columns: 2 slot groups x 8 slots x 32

struct alignas(64) TcParams {
  CUtensorMap one;            // the matrix of a single-matrix call (maps0 == nullptr)
  const CUtensorMap* maps0;   // per-expert tensor maps, indexed like the weight table (gate / down / the one matrix)
  const CUtensorMap* maps1;   // up (MODE 1)
  int N, K;                   // weight rows of each matrix, elements per row
  int tile_rows;              // weight rows per tile (<= 128; MODE 1: 64 gate + the same 64 up rows)
  int row_tiles;              // ceil(N / tile_rows)
  const int4* groups;         // {table index of the expert, first position, rows (<= 32), 0}
  const int* n_groups;
  const int* list;            // slot id at each position
  int S;                      // slots per token
  const uint8_t* xrows;       // quantized activation rows (layout: act_row_pitch); MODE 0 by position, else by slot / S
  size_t x_pitch;
  void* dst;                  // MODE 0: float [npos, N]; MODE 1 without qdst: float [npos, N]; MODE 2: YT [rows, ld_dst]
  size_t ld_dst;
  int round_bf16;
  uint8_t* qdst;              // MODE 1: quantized rows by position
  size_t q_pitch;
  int* status;
  int32_t* dots;              // debug/parity: when set, raw int32 sub-block dots [pos][N][K/32] are stored too
};

template <int MODE>
struct TcLayout {
  static constexpr int kStages = MODE == 1 ? 3 : 4;
  static constexpr uint32_t w    = 0;
  static constexpr uint32_t x    = w + kStages * kTcWStage;
  static constexpr uint32_t a    = x + kStages * kTcXStage;
  static constexpr uint32_t b    = a + 2 * 8 * kTcATile;
  static constexpr uint32_t ws   = b + 2 * 8 * kTcBTile;          // [2][16][128] float: d*sc of 8 sub-blocks, dmin*mn of 8
  static constexpr uint32_t dx   = ws + 2 * 16 * 128 * 4;         // [2][16][32] float: dx of 8 blocks, dx*sum of 8
  static constexpr uint32_t ex   = dx + 2 * 16 * kTcNT * 4;       // MODE 1: [2][2 halves][2 warps][16][32] float
  static constexpr uint32_t bar  = ex + (MODE == 1 ? 2 * 2048 * 4 : 0);
  static constexpr uint32_t total = bar + 256 + 128;              // + slack for the 128-byte alignment of the base
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tensormap_acquire(const CUtensorMap* map) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(map) : "memory");
}
// shared-memory matrix descriptor: K-major, no swizzle, 8 x 16-byte core matrices,
// next 16 bytes of K at +128 B, next 8 rows at +256 B, descriptor version 1
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>(128u >> 4) << 16;
  d |= static_cast<uint64_t>(256u >> 4) << 32;
  d |= static_cast<uint64_t>(1u) << 46;
  return d;
}
// instruction descriptor: D = S32, A = B = signed 8-bit, both K-major, N = 32, M = 128
constexpr uint32_t kTcIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((kTcNT >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kTcIdesc), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, int (&v)[16], int o) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[o + 0]), "=r"(v[o + 1]), "=r"(v[o + 2]), "=r"(v[o + 3]), "=r"(v[o + 4]), "=r"(v[o + 5]),
                 "=r"(v[o + 6]), "=r"(v[o + 7])
               : "r"(taddr));
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, int (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void sts128(uint32_t a, const int4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts32f(uint32_t a, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
__device__ __forceinline__ float lds32f(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}

// MODE 0: dst[pos, j]  = W0[j,:] . q(x[pos,:])                        (down projection)
// MODE 1: act[pos, j]  = Scalar(silu(W0 . q(x)) * (W1 . q(x)))        (gate / up + SwiGLU; quantized when qdst is set)
// MODE 2: dst[row, j]  = YT(W0[j,:] . q(x[row,:]))                    (plain batched GEMM)
template <int MODE, class YT>
__global__ void __launch_bounds__(kTcThreads, 1) grouped_tc_q4k_kernel(const __grid_constant__ TcParams p) {
  using L = TcLayout<MODE>;
  constexpr int kStages = L::kStages;
  extern __shared__ __align__(128) uint8_t tc_smem_raw[];
  const uint32_t base = (smem_u32(tc_smem_raw) + 127u) & ~127u;
  uint8_t* smem = tc_smem_raw + (base - smem_u32(tc_smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // barriers: w_full[4], w_empty[4], a_full[2], mma_done[2], t_empty[2], ex_full[2]
  const uint32_t bars = base + L::bar;
  auto w_full   = [&](int s) { return bars + 8u * s; };
  auto w_empty  = [&](int s) { return bars + 32u + 8u * s; };
  auto a_full   = [&](int b) { return bars + 64u + 8u * b; };
  auto mma_done = [&](int b) { return bars + 80u + 8u * b; };
  auto t_empty  = [&](int b) { return bars + 96u + 8u * b; };
  auto ex_full  = [&](int b) { return bars + 112u + 8u * b; };
  uint32_t* tmem_slot      = reinterpret_cast<uint32_t*>(smem + L::bar + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::bar + 132);

  if (warp == 13) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTcCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 4; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), 128);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(a_full(b), 128);
      mbar_init(mma_done(b), 1);
      mbar_init(t_empty(b), 256);
      mbar_init(ex_full(b), 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  tc_before();
  __syncthreads();
  tc_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  // Bounded wait shared by every role: gives up when the barrier does not complete or when
  // another role of this CTA has already given up.
  auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
    for (uint32_t i = 0; i < (1u << 21); ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((i & 31u) == 31u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
  };

  const int n_groups    = __ldg(p.n_groups);
  const int total_tiles = n_groups * p.row_tiles;
  const int nks         = p.K / 256;
  bool ok = true;

  if (warp == 12) {
    // ------------------------------------------------------------------ producer
    const size_t scale_off = act_bytes(static_cast<size_t>(p.K));
    uint32_t seq = 0;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int g = t / p.row_tiles, rb = t - g * p.row_tiles;
      const int4 gi = __ldg(p.groups + g);
      const CUtensorMap* m0 = p.maps0 ? p.maps0 + gi.x : &p.one;
      const CUtensorMap* m1 = MODE == 1 ? p.maps1 + gi.x : m0;
      if (lane == 0 && p.maps0) {
        tensormap_acquire(m0);
        if (MODE == 1) tensormap_acquire(m1);
      }
      const int r0 = rb * p.tile_rows;
      const int nbox = MODE == 1 ? 4 : (min(p.tile_rows, p.N - r0) + kTcBoxRows - 1) / kTcBoxRows;
      const uint8_t* xrow = nullptr;
      if (lane < gi.z) {
        const int srow = MODE == 0 ? gi.y + lane : __ldg(p.list + gi.y + lane) / p.S;
        xrow = p.xrows + static_cast<size_t>(srow) * p.x_pitch;
      }
      for (int ks = 0; ks < nks; ++ks, ++seq) {
        const int s = static_cast<int>(seq % kStages);
        const uint32_t use = seq / kStages;
        if (!wait(w_empty(s), (use & 1u) ^ 1u)) { ok = false; break; }
        const uint32_t bar = w_full(s);
        const uint32_t wdst = base + L::w + s * kTcWStage, xdst = base + L::x + s * kTcXStage;
        if (lane == 0) {
          mbar_expect_tx(bar, static_cast<uint32_t>(nbox) * (kTcBoxRows * 144) + static_cast<uint32_t>(gi.z) * 320u);
          if (MODE == 1) {
            tma_load_2d(wdst, m0, ks * 144, r0, bar);
            tma_load_2d(wdst + 4608, m0, ks * 144, r0 + 32, bar);
            tma_load_2d(wdst + 9216, m1, ks * 144, r0, bar);
            tma_load_2d(wdst + 13824, m1, ks * 144, r0 + 32, bar);
          } else {
            for (int bx = 0; bx < nbox; ++bx) tma_load_2d(wdst + bx * 4608, m0, ks * 144, r0 + bx * kTcBoxRows, bar);
          }
        }
        __syncwarp();
        if (xrow) {
          bulk_g2s(xdst + lane * 256, xrow + static_cast<size_t>(ks) * 256, 256, bar);
          bulk_g2s(xdst + kTcXq + lane * 64, xrow + scale_off + static_cast<size_t>(ks) * 64, 64, bar);
        }
      }
    }
    if (!ok || *abort_flag) {
      // copies of the last stages may still be in flight: give them time to land before the CTA's
      // shared memory is handed to somebody else (bounded, the result of the launch is void anyway)
      for (int s = 0; s < kStages; ++s)
        for (uint32_t i = 0; i < (1u << 16); ++i)
          if (mbar_try_wait(w_full(s), 0u) || mbar_try_wait(w_full(s), 1u)) break;
    }
  } else if (warp >= 8 && warp < 12) {
    // ------------------------------------------------------------------ unpack
    const int u = threadIdx.x - 256;
    uint32_t seq = 0;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int g = t / p.row_tiles;
      const int ntok = __ldg(p.groups + g).z;
      for (int ks = 0; ks < nks; ++ks, ++seq) {
        const int s = static_cast<int>(seq % kStages);
        const uint32_t use = seq / kStages;
        const int b = seq & 1u;
        const uint32_t j = seq >> 1;
        if (!wait(w_full(s), use & 1u) || !wait(mma_done(b), (j & 1u) ^ 1u) || !wait(t_empty(b), (j & 1u) ^ 1u)) {
          ok = false;
          break;
        }
        const uint32_t mine = base + L::w + s * kTcWStage + u * 144;
        const int4 hdr = lds128_g(mine);
        const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
        const uint32_t wsb = base + L::ws + b * (16 * 128 * 4) + u * 4;
        const uint32_t abase = base + L::a + b * (8 * kTcATile) + (u >> 3) * 256 + (u & 7) * 16;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          uint32_t scp, mnp;
          q4k_scale_pair(hdr.y, hdr.z, hdr.w, it, scp, mnp);
          sts32f(wsb + (2 * it) * 512, dd.x * static_cast<float>(scp & 0xFF));
          sts32f(wsb + (2 * it + 1) * 512, dd.x * static_cast<float>(scp >> 8));
          sts32f(wsb + (8 + 2 * it) * 512, dd.y * static_cast<float>(mnp & 0xFF));
          sts32f(wsb + (9 + 2 * it) * 512, dd.y * static_cast<float>(mnp >> 8));
          const int4 qa = lds128_g(mine + 16 + it * 32), qb = lds128_g(mine + 32 + it * 32);
          // sub-block 2*it: low nibbles, 2*it+1: high nibbles; K bytes 0-15 then 16-31
          const int4 lo0 = make_int4(qa.x & 0x0F0F0F0F, qa.y & 0x0F0F0F0F, qa.z & 0x0F0F0F0F, qa.w & 0x0F0F0F0F);
          const int4 lo1 = make_int4(qb.x & 0x0F0F0F0F, qb.y & 0x0F0F0F0F, qb.z & 0x0F0F0F0F, qb.w & 0x0F0F0F0F);
          const int4 hi0 = make_int4((qa.x >> 4) & 0x0F0F0F0F, (qa.y >> 4) & 0x0F0F0F0F, (qa.z >> 4) & 0x0F0F0F0F,
                                     (qa.w >> 4) & 0x0F0F0F0F);
          const int4 hi1 = make_int4((qb.x >> 4) & 0x0F0F0F0F, (qb.y >> 4) & 0x0F0F0F0F, (qb.z >> 4) & 0x0F0F0F0F,
                                     (qb.w >> 4) & 0x0F0F0F0F);
          sts128(abase + (2 * it) * kTcATile, lo0);
          sts128(abase + (2 * it) * kTcATile + 128, lo1);
          sts128(abase + (2 * it + 1) * kTcATile, hi0);
          sts128(abase + (2 * it + 1) * kTcATile + 128, hi1);
        }
        // activations of the group: 32 rows x 16 pieces of 16 bytes -> eight B tiles
        const uint32_t xsrc = base + L::x + s * kTcXStage;
        const uint32_t bdst = base + L::b + b * (8 * kTcBTile);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int pc = u + 128 * i, n = pc >> 4, c16 = pc & 15;
          int4 v = make_int4(0, 0, 0, 0);
          if (n < ntok) v = lds128_g(xsrc + n * 256 + c16 * 16);
          sts128(bdst + (c16 >> 1) * kTcBTile + (n >> 3) * 256 + (c16 & 1) * 128 + (n & 7) * 16, v);
        }
        const uint32_t dxb = base + L::dx + b * (16 * kTcNT * 4);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int f = u + 128 * i, n = f >> 3, jj = f & 7;
          uint2 v = make_uint2(0u, 0u);
          if (n < ntok) v = lds64_g(xsrc + kTcXq + n * 64 + jj * 8);
          sts32f(dxb + (jj * kTcNT + n) * 4, __uint_as_float(v.x));
          sts32f(dxb + ((8 + jj) * kTcNT + n) * 4, __uint_as_float(v.y));
        }
        fence_proxy_async();   // generic-proxy writes (A, B tiles) -> async-proxy reads by the MMA
        mbar_arrive(a_full(b));
        mbar_arrive(w_empty(s));
      }
    }
  } else if (warp == 13) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      uint32_t seq = 0;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (int ks = 0; ks < nks; ++ks, ++seq) {
          const int b = seq & 1u;
          const uint32_t j = seq >> 1;
          if (!wait(a_full(b), j & 1u)) { ok = false; break; }
          tc_after();
          const uint32_t a0 = base + L::a + b * (8 * kTcATile), b0 = base + L::b + b * (8 * kTcBTile);
#pragma unroll
          for (int s8 = 0; s8 < 8; ++s8)
            tc_mma_i8(tmem_base + b * 256 + s8 * kTcNT, tc_desc(a0 + s8 * kTcATile), tc_desc(b0 + s8 * kTcBTile));
          tc_commit(mma_done(b));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ drain + epilogue
    const int q = warp & 3, hf = warp >> 2;
    const int row = q * 32 + lane;
    const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + hf * 16;
    uint32_t seq = 0, tile_no = 0;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_no) {
      const int g = t / p.row_tiles, rb = t - g * p.row_tiles;
      const int4 gi = __ldg(p.groups + g);
      const int ncol = max(0, min(16, gi.z - 16 * hf));
      const int n8 = (ncol + 7) >> 3;
      const int r0 = rb * p.tile_rows;
      float acc[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) acc[c] = 0.f;
      for (int ks = 0; ks < nks; ++ks, ++seq) {
        const int b = seq & 1u;
        const uint32_t j = seq >> 1;
        if (!wait(a_full(b), j & 1u) || !wait(mma_done(b), j & 1u)) { ok = false; break; }
        tc_after();
        if (n8 > 0) {
          const uint32_t wsb = base + L::ws + b * (16 * 128 * 4) + row * 4;
          const uint32_t dxb = base + L::dx + b * (16 * kTcNT * 4) + hf * 64;
#pragma unroll
          for (int s8 = 0; s8 < 8; ++s8) {
            int d[16];
            if (n8 == 2) tc_ld16(taddr0 + b * 256 + s8 * kTcNT, d);
            else tc_ld8(taddr0 + b * 256 + s8 * kTcNT, d, 0);
            tc_wait_ld();
            const float sw = lds32f(wsb + s8 * 512), mw = lds32f(wsb + (8 + s8) * 512);
            if (p.dots != nullptr) {   // parity probe: the exact integer sub-block dots of the production MMAs
              const int jrow = MODE == 1 ? (row < 64 ? r0 + row : -1) : (row < p.tile_rows ? r0 + row : -1);
              if (jrow >= 0 && jrow < p.N) {
#pragma unroll
                for (int c = 0; c < 16; ++c)
                  if (c < ncol)
                    p.dots[(static_cast<size_t>(gi.y + 16 * hf + c) * p.N + jrow) * (p.K / 32) + ks * 8 + s8] = d[c];
              }
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (v < 2 * n8) {
                const float4 a = lds128f(dxb + (s8 * kTcNT + 4 * v) * 4);
                const float4 m = lds128f(dxb + ((8 + s8) * kTcNT + 4 * v) * 4);
                const float2 sw2 = make_float2(sw, sw), nmw2 = make_float2(-mw, -mw);
                const float2 p0 = fmul2(make_float2(static_cast<float>(d[4 * v]), static_cast<float>(d[4 * v + 1])),
                                        make_float2(a.x, a.y));
                const float2 p1 = fmul2(make_float2(static_cast<float>(d[4 * v + 2]), static_cast<float>(d[4 * v + 3])),
                                        make_float2(a.z, a.w));
                float2 r = ffma2(sw2, p0, make_float2(acc[4 * v], acc[4 * v + 1]));
                r = ffma2(nmw2, make_float2(m.x, m.y), r);
                acc[4 * v] = r.x; acc[4 * v + 1] = r.y;
                r = ffma2(sw2, p1, make_float2(acc[4 * v + 2], acc[4 * v + 3]));
                r = ffma2(nmw2, make_float2(m.z, m.w), r);
                acc[4 * v + 2] = r.x; acc[4 * v + 3] = r.y;
              }
            }
          }
        }
        tc_before();
        mbar_arrive(t_empty(b));
      }
      if (!ok) break;
      // ---- epilogue of the tile ----
      if (MODE == 1) {
        const int tp = tile_no & 1u;
        const uint32_t exb = base + L::ex + tp * 8192 + ((hf * 2 + (q & 1)) * 16 * 32 + lane) * 4;
        if (q >= 2) {
#pragma unroll
          for (int c = 0; c < 16; ++c) sts32f(exb + c * 128, acc[c]);
          mbar_arrive(ex_full(tp));
        } else {
          if (!wait(ex_full(tp), (tile_no >> 1) & 1u)) { ok = false; break; }
          const int jcol = r0 + row;          // row < 64: this thread's gate row
          const int blk = jcol >> 5;          // 32-block of the act row this warp's lanes form
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            if (c < ncol) {                   // uniform across the warp
              const float up = lds32f(exb + c * 128);
              float v = acc[c];
              v = (v / (1.0f + expf(-v))) * up;
              if (p.round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
              if (jcol >= p.N) v = 0.f;
              const size_t ps = static_cast<size_t>(gi.y + 16 * hf + c);
              if (p.qdst != nullptr) {
                // the reference's stage-1 quantizer on the 32 values the warp holds (one whole block)
                float amax = fabsf(v);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                const float dq  = __fdiv_rn(amax, 127.0f);
                const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
                int qv = __float2int_rn(__fmul_rn(v, inv));
                qv = max(-127, min(127, qv));
                int sm = qv;
                sm += __shfl_xor_sync(0xffffffffu, sm, 1);
                sm += __shfl_xor_sync(0xffffffffu, sm, 2);
                sm += __shfl_xor_sync(0xffffffffu, sm, 4);
                sm += __shfl_xor_sync(0xffffffffu, sm, 8);
                const int other = __shfl_xor_sync(0xffffffffu, sm, 16);
                uint8_t* qrow = p.qdst + ps * p.q_pitch;
                if ((blk + 1) * 32 <= p.N) {
                  reinterpret_cast<int8_t*>(qrow)[blk * 32 + lane] = static_cast<int8_t>(qv);
                  if (lane == 0) {
                    reinterpret_cast<ActHdr*>(qrow + act_hdr_offset(static_cast<size_t>(p.N)))[blk] = ActHdr{dq, sm, other, 0};
                    const float ds = __fmul_rn(static_cast<float>(sm + other), dq);
                    reinterpret_cast<float2*>(qrow + act_bytes(static_cast<size_t>(p.N)))[blk] = make_float2(dq, ds);
                    store_sum_parts(qrow, act_parts_offset(static_cast<size_t>(p.N)), blk, ds);
                  }
                }
              } else if (jcol < p.N) {
                static_cast<float*>(p.dst)[ps * p.N + jcol] = v;
              }
            }
          }
        }
      } else {
        const int jrow = r0 + row;
        if (row < p.tile_rows && jrow < p.N) {
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            if (c < ncol) {
              const int ps = gi.y + 16 * hf + c;
              if (MODE == 2) {
                const int srow = __ldg(p.list + ps) / p.S;
                store_scalar(static_cast<YT*>(p.dst) + static_cast<size_t>(srow) * p.ld_dst + jrow, acc[c]);
              } else {
                static_cast<float*>(p.dst)[static_cast<size_t>(ps) * p.N + jrow] = acc[c];
              }
            }
          }
        }
      }
    }
  }
  if (!ok && lane == 0) atomicExch(p.status, KDNN_ERR_DEVICE_WAIT);
  tc_before();
  __syncthreads();
  if (warp == 13)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTcCols) : "memory");
}

// ---- host side ---------------------------------------------------------------------------
// cuTensorMapEncodeTiled is a driver entry point: fetched through the runtime, so the library
// does not link against libcuda.
using TcEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TcEncodeFn tc_encode_fn();   // kdnn_moe.cu

// Tensor map of one packed Q4_K matrix: bytes as the inner dimension, rows as the outer, boxes of
// 32 rows x one 144-byte super-block.
inline cudaError_t tc_encode_matrix(CUtensorMap* out, const void* w, size_t rows, size_t row_bytes) {
  TcEncodeFn fn = tc_encode_fn();
  if (fn == nullptr) return cudaErrorNotSupported;
  const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  const cuuint32_t box[2]     = {144u, static_cast<cuuint32_t>(kTcBoxRows)};
  const cuuint32_t estr[2]    = {1u, 1u};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

int device_sm_count();   // kdnn_moe.cu

template <int MODE, class YT>
static cudaError_t launch_grouped_tc(const TcParams& p, int max_tiles, cudaStream_t st) {
  using L = TcLayout<MODE>;
  auto kern = grouped_tc_q4k_kernel<MODE, YT>;
  static SmemAttrOnce once;
  const cudaError_t e = set_max_smem_once(once, kern, (int)L::total);
  if (e != cudaSuccess) return e;
  const int grid = max(1, min(device_sm_count(), max_tiles));
  return launch_chained(kern, dim3(grid), dim3(kTcThreads), L::total, st, p);
}

}  // namespace kdnn
