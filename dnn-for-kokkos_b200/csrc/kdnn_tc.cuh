// Grouped int8 tile GEMM for Q4_K weights on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory), as ONE persistent,
// warp-specialised kernel per launch: a CTA per SM walks the tiles
// (group of <= 32 activation rows) x (128 weight rows) and never drains its
// pipeline between tiles, so the next tile's packed rows are already in flight
// while the current tile is being folded.
//
//   warp 24      producer: per 256-element super-block of K one stage of the ring =
//                128 packed rows x 144 bytes by tensor-map TMA (cp.async.bulk.tensor.2d,
//                32-row boxes, this GPU's memory only, one destination CTA)
//   warps 16-23  unpack: thread = (weight row, half of its sub-blocks); nibbles -> int8 in the K-major core-matrix
//                layout the MMA reads (eight 128 x 32 A tiles per stage), the 6-bit scales
//                and mins -> fp32 tables; the group's quantized activations (a few KB per stage,
//                L2 hits) come by plain loads one stage ahead -> eight 32 x 32 B tiles
//   warp 25      one thread issues eight tcgen05.mma per stage (one per 32-element
//                sub-block, each into its own 32-column TMEM slot: every sub-block has its
//                own scale on both sides, so nothing accumulates across them in TMEM) and
//                commits them to an mbarrier; two slot groups (2 x 256 columns) rotate
//   warps 0-15   drain: thread = (weight row, half of the activation rows, half of the sub-blocks) --
//                four warps per TMEM lane quadrant, because the fold is a chain of dependent FP32
//                instructions that needs several warps per scheduler to issue at rate; tcgen05.ld
//                of its TMEM lane, fold  acc += (d*sc) * dx * dot - (dmin*mn) * dx * sum  in
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
constexpr int kTcATile    = 128 * 32;
constexpr int kTcBTile    = kTcNT * 32;
constexpr int kTcThreads  = 26 * 32;
constexpr int kTcDrainWarps = 16, kTcUnpackWarp0 = 16, kTcWarpProducer = 24, kTcWarpMma = 25;
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
  PeerOut po;                 // MODE 0: po.out != null writes the rows into this rank's slot-indexed buffer (read by the token owners)
};


template <int MODE>
struct TcLayout {
  static constexpr int kStages = MODE == 1 ? 5 : 6;   // as many as fit next to the other buffers
  static constexpr uint32_t w    = 0;
  static constexpr uint32_t a    = w + kStages * kTcWStage;
  static constexpr uint32_t b    = a + 2 * 8 * kTcATile;
  static constexpr uint32_t ws   = b + 2 * 8 * kTcBTile;          // [2][2 sub-block halves][sw, mw][128 rows][4] float: d*sc, dmin*mn
  static constexpr uint32_t dx   = ws + 2 * 2 * 2 * 128 * 16;     // [2][16][32] float: dx of 8 blocks, dx*sum of 8
  static constexpr uint32_t red  = dx + 2 * 16 * kTcNT * 4;       // [4 quadrants][2 column halves][16][32] float: partial sums of sub-blocks 4-7
  static constexpr uint32_t ex   = red + 4 * 2 * 16 * 32 * 4;     // MODE 1: [2 column halves][2 warps][16][32] float: the up rows' sums
  static constexpr uint32_t bar  = ex + (MODE == 1 ? 2048 * 4 : 0);
  static constexpr uint32_t total = bar + 256 + 128;              // + slack for the 128-byte alignment of the base
};

// Loads of what the PREVIOUS kernel in the stream wrote (group records, slot list, quantized rows). They must
// not be __ldg / invariant loads: the compiler may move an invariant load above griddepcontrol.wait, i.e. in
// front of the moment the producer's data exists (seen as groups read as zero on every call but the first).
__device__ __forceinline__ int ld_dep(const int* p) {
  int v;
  asm volatile("ld.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int4 ld_dep(const int4* p) {
  int4 v;
  asm volatile("ld.global.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_dep(const uint2* p) {
  uint2 v;
  asm volatile("ld.global.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int4 ld_dep128(const void* p) { return ld_dep(static_cast<const int4*>(p)); }

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
__device__ __forceinline__ void tc_ld8(uint32_t taddr, int (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
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

// One sub-block of one TMEM lane, already in registers, folded into the thread's accumulators:
//   acc[c] += sw * (float(D[c]) * dx[c]) - mw * dxs[c],  c < 8 * NC8.
template <int NC8>
__device__ __forceinline__ void tc_fold(float (&acc)[16], const int (&d)[8 * NC8], float sw, float mw, uint32_t dxs) {
  // all of the sub-block's activation scales first (one shared-memory round trip, not one per use)
  float4 a[2 * NC8], m[2 * NC8];
#pragma unroll
  for (int v = 0; v < 2 * NC8; ++v) {
    a[v] = lds128f(dxs + 16 * v);
    m[v] = lds128f(dxs + 8 * kTcNT * 4 + 16 * v);
  }
  const float2 sw2 = make_float2(sw, sw), nmw2 = make_float2(-mw, -mw);
  const float2 nmagic = make_float2(-kM2MagicF, -kM2MagicF);
#pragma unroll
  for (int v = 0; v < 2 * NC8; ++v) {
    // int -> float on the integer and FP32 pipes (no conversion instruction): for |i| < 2^22 the bits of
    // i + 0x4B400000 are the float 12582912 + i, one exact subtraction gives float(i); a sub-block dot is
    // at most 32 * 15 * 127 in magnitude. (Presetting the TMEM slots to that constant and letting the MMA
    // accumulate onto it saves the integer add but costs a tcgen05.st per slot and use: measured slower.)
    const float2 f0 = fadd2(make_float2(__int_as_float(d[4 * v] + kM2MagicI), __int_as_float(d[4 * v + 1] + kM2MagicI)), nmagic);
    const float2 f1 = fadd2(make_float2(__int_as_float(d[4 * v + 2] + kM2MagicI), __int_as_float(d[4 * v + 3] + kM2MagicI)), nmagic);
    const float2 p0 = fmul2(f0, make_float2(a[v].x, a[v].y));
    const float2 p1 = fmul2(f1, make_float2(a[v].z, a[v].w));
    float2 r = ffma2(sw2, p0, make_float2(acc[4 * v], acc[4 * v + 1]));
    r = ffma2(nmw2, make_float2(m[v].x, m[v].y), r);
    acc[4 * v] = r.x; acc[4 * v + 1] = r.y;
    r = ffma2(sw2, p1, make_float2(acc[4 * v + 2], acc[4 * v + 3]));
    r = ffma2(nmw2, make_float2(m[v].z, m[v].w), r);
    acc[4 * v + 2] = r.x; acc[4 * v + 3] = r.y;
  }
}

// Four sub-block slots of one TMEM lane: the loads come first and the slot group is handed back to the MMA
// warp (`t_empty_bar`) as soon as the values are in registers -- the arithmetic then overlaps the next MMAs
// into the same slots. Eight columns per thread: all four slots at once (32 registers); sixteen: two and two.
// `taddr` / `dxb` already point at the first of the four sub-blocks.
template <int NC8>
__device__ __forceinline__ void tc_drain_half(float (&acc)[16], uint32_t taddr, const float (&sws)[4], const float (&mws)[4],
                                              uint32_t dxb, uint32_t t_empty_bar, int lane) {
  if (NC8 == 1) {
    int d[4][8];
#pragma unroll
    for (int g = 0; g < 4; ++g) tc_ld8(taddr + g * kTcNT, d[g]);
    tc_wait_ld();
    tc_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(t_empty_bar);
#pragma unroll
    for (int g = 0; g < 4; ++g) tc_fold<1>(acc, d[g], sws[g], mws[g], dxb + g * kTcNT * 4);
  } else {
    int d[2][16];
    tc_ld16(taddr, d[0]);
    tc_ld16(taddr + kTcNT, d[1]);
    tc_wait_ld();
    tc_fold<2>(acc, d[0], sws[0], mws[0], dxb);
    tc_fold<2>(acc, d[1], sws[1], mws[1], dxb + kTcNT * 4);
    tc_ld16(taddr + 2 * kTcNT, d[0]);
    tc_ld16(taddr + 3 * kTcNT, d[1]);
    tc_wait_ld();
    tc_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(t_empty_bar);
    tc_fold<2>(acc, d[0], sws[2], mws[2], dxb + 2 * kTcNT * 4);
    tc_fold<2>(acc, d[1], sws[3], mws[3], dxb + 3 * kTcNT * 4);
  }
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

  // barriers: w_full[8], w_empty[8], a_full[2], mma_done[2], t_empty[2], red_full, red_empty, ex_full, ex_empty, s_free[2]
  const uint32_t bars = base + L::bar;
  auto w_full   = [&](int s) { return bars + 8u * s; };
  auto w_empty  = [&](int s) { return bars + 64u + 8u * s; };
  auto a_full   = [&](int b) { return bars + 128u + 8u * b; };
  auto mma_done = [&](int b) { return bars + 144u + 8u * b; };
  auto t_empty  = [&](int b) { return bars + 160u + 8u * b; };
  const uint32_t red_full = bars + 176u, red_empty = bars + 184u, ex_full = bars + 192u, ex_empty = bars + 200u;
  auto s_free   = [&](int b) { return bars + 208u + 8u * b; };
  uint32_t* tmem_slot      = reinterpret_cast<uint32_t*>(smem + L::bar + 224);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::bar + 228);

  if (warp == kTcWarpMma) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTcCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x == 0) {
    // one arrival per WARP on the barriers several warps feed (lane 0, after __syncwarp): hundreds of
    // per-thread arrivals on one shared-memory word serialise
    for (int s = 0; s < kStages; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), 8);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(a_full(b), 8);
      mbar_init(mma_done(b), 1);
      mbar_init(t_empty(b), kTcDrainWarps);
      mbar_init(s_free(b), kTcDrainWarps);
    }
    mbar_init(red_full, 8);
    mbar_init(red_empty, 8);
    mbar_init(ex_full, 4);
    mbar_init(ex_empty, 4);
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
      if (mbar_try_wait(bar, parity)) {
        return true;
      }
      if ((i & 31u) == 31u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
  };

  const int n_groups    = ld_dep(p.n_groups);
  const int total_tiles = n_groups * p.row_tiles;
  const int nks         = p.K / 256;
  bool ok = true;

  if (warp == kTcWarpProducer) {
    // ------------------------------------------------------------------ producer (one thread)
    if (lane == 0) {
      uint32_t seq = 0;
      int e_next = blockIdx.x < total_tiles ? ld_dep(p.groups + blockIdx.x / p.row_tiles).x : 0;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int g = t / p.row_tiles, rb = t - g * p.row_tiles;
        const int e = e_next;   // requested a tile ago
        if (t + static_cast<int>(gridDim.x) < total_tiles) e_next = ld_dep(p.groups + (t + gridDim.x) / p.row_tiles).x;
        const CUtensorMap* m0 = p.maps0 ? p.maps0 + e : &p.one;
        const CUtensorMap* m1 = MODE == 1 ? p.maps1 + e : m0;
        if (p.maps0) {
          tensormap_acquire(m0);
          if (MODE == 1) tensormap_acquire(m1);
        }
        const int r0 = rb * p.tile_rows;
        const int nbox = MODE == 1 ? 4 : (min(p.tile_rows, p.N - r0) + kTcBoxRows - 1) / kTcBoxRows;
        for (int ks = 0; ks < nks; ++ks, ++seq) {
          const int s = static_cast<int>(seq % kStages);
          const uint32_t use = seq / kStages;
          if (!wait(w_empty(s), (use & 1u) ^ 1u)) { ok = false; break; }
          const uint32_t bar = w_full(s);
          const uint32_t wdst = base + L::w + s * kTcWStage;
          mbar_expect_tx(bar, static_cast<uint32_t>(nbox) * (kTcBoxRows * 144));
          if (MODE == 1) {
            tma_load_2d(wdst, m0, ks * 144, r0, bar);
            tma_load_2d(wdst + 4608, m0, ks * 144, r0 + 32, bar);
            tma_load_2d(wdst + 9216, m1, ks * 144, r0, bar);
            tma_load_2d(wdst + 13824, m1, ks * 144, r0 + 32, bar);
          } else {
            for (int bx = 0; bx < nbox; ++bx) tma_load_2d(wdst + bx * 4608, m0, ks * 144, r0 + bx * kTcBoxRows, bar);
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
    }
  } else if (warp >= kTcUnpackWarp0 && warp < kTcUnpackWarp0 + 8) {
    // ------------------------------------------------------------------ unpack
    // thread = (weight row u of the tile, half uh of its nibble groups) for the weights; for the group's
    // activations it owns two 16-byte pieces (rows ut / 16 and ut / 16 + 16, piece ut % 16 of the stage's
    // 256 bytes) and one {d, d * sum} pair (row ut / 8, block ut % 8), fetched from global memory (L2) with
    // plain loads ONE STAGE AHEAD into registers: bulk copies of a few hundred bytes cost the copy engine
    // about as much as a 4 KB box each.
    const int ut = threadIdx.x - kTcUnpackWarp0 * 32;
    const int u = ut & 127, uh = ut >> 7;
    const size_t scale_off = act_bytes(static_cast<size_t>(p.K));
    // Metadata runs two tiles ahead so that no load waits for another load on the way: the group record of
    // tile i + 2 is requested when tile i is entered, the row ids of tile i + 1 (which need its group record,
    // here since a tile ago) at the same moment, and the pieces of stage s + 1 while stage s is unpacked.
    struct Rows { const uint8_t* r0; const uint8_t* r1; const uint8_t* rs; };   // null past the group's rows
    const int xn = ((ut >> 7) << 3) | (ut & 7), xc16 = (ut >> 3) & 15;   // this thread's pieces: rows xn, xn + 16, 16-byte piece xc16
    auto group_of = [&](int t) { return t < total_tiles ? ld_dep(p.groups + t / p.row_tiles) : make_int4(0, 0, 0, 0); };
    auto rows_of = [&](const int4& gi) {
      auto row_of = [&](int n) -> const uint8_t* {
        if (n >= gi.z) return nullptr;
        const int srow = MODE == 0 ? gi.y + n : ld_dep(p.list + gi.y + n) / p.S;
        return p.xrows + static_cast<size_t>(srow) * p.x_pitch;
      };
      return Rows{row_of(xn), row_of(xn + 16), row_of(ut & 31)};
    };
    // (piece mapping chosen for the STORES: eight consecutive lanes fill one 128-byte core matrix of a
    // B tile, 32 consecutive lanes fill 32 consecutive scale words -- no bank conflicts)
    struct Pieces { int4 x0, x1; uint2 sv; };
    int f_t = blockIdx.x, f_ks = 0;                 // fetch cursor: the stage whose pieces are requested next
    int4 gi2 = group_of(f_t + 2 * gridDim.x);
    Rows rows0 = rows_of(group_of(f_t)), rows1 = rows_of(group_of(f_t + gridDim.x));
    auto fetch = [&](Pieces& f) {
      f.x0 = f.x1 = make_int4(0, 0, 0, 0);
      f.sv = make_uint2(0u, 0u);
      if (f_t < total_tiles) {
        const size_t ko = static_cast<size_t>(f_ks) * 256 + xc16 * 16;
        if (rows0.r0) f.x0 = ld_dep128(rows0.r0 + ko);
        if (rows0.r1) f.x1 = ld_dep128(rows0.r1 + ko);
        if (rows0.rs) f.sv = ld_dep(reinterpret_cast<const uint2*>(rows0.rs + scale_off + static_cast<size_t>(f_ks) * 64 + (ut >> 5) * 8));
      }
      if (++f_ks == nks) {   // the cursor enters the next tile
        f_ks = 0;
        f_t += gridDim.x;
        rows0 = rows1;
        rows1 = rows_of(gi2);
        gi2 = group_of(f_t + 2 * gridDim.x);
      }
    };
    auto stage = [&](uint32_t seq, const Pieces& have) -> bool {
      const int s = static_cast<int>(seq % kStages);
      const uint32_t use = seq / kStages;
      const int b = seq & 1u;
      const uint32_t j = seq >> 1;
      bool okw = wait(w_full(s), use & 1u);
      okw = okw && wait(mma_done(b), (j & 1u) ^ 1u);
      if (!okw) return false;
      const uint32_t mine = base + L::w + s * kTcWStage + u * 144;
      const int4 hdr = lds128_g(mine);
      int4 qa[2], qb[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        qa[i] = lds128_g(mine + 16 + (2 * uh + i) * 32);
        qb[i] = lds128_g(mine + 32 + (2 * uh + i) * 32);
      }
      const uint32_t abase = base + L::a + b * (8 * kTcATile) + (u >> 3) * 256 + (u & 7) * 16;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int it = 2 * uh + i;
        // sub-block 2*it: low nibbles, 2*it+1: high nibbles; K bytes 0-15 then 16-31
        const int4 a4 = qa[i], b4 = qb[i];
        const int4 lo0 = make_int4(a4.x & 0x0F0F0F0F, a4.y & 0x0F0F0F0F, a4.z & 0x0F0F0F0F, a4.w & 0x0F0F0F0F);
        const int4 lo1 = make_int4(b4.x & 0x0F0F0F0F, b4.y & 0x0F0F0F0F, b4.z & 0x0F0F0F0F, b4.w & 0x0F0F0F0F);
        const int4 hi0 = make_int4((a4.x >> 4) & 0x0F0F0F0F, (a4.y >> 4) & 0x0F0F0F0F, (a4.z >> 4) & 0x0F0F0F0F,
                                   (a4.w >> 4) & 0x0F0F0F0F);
        const int4 hi1 = make_int4((b4.x >> 4) & 0x0F0F0F0F, (b4.y >> 4) & 0x0F0F0F0F, (b4.z >> 4) & 0x0F0F0F0F,
                                   (b4.w >> 4) & 0x0F0F0F0F);
        sts128(abase + (2 * it) * kTcATile, lo0);
        sts128(abase + (2 * it) * kTcATile + 128, lo1);
        sts128(abase + (2 * it + 1) * kTcATile, hi0);
        sts128(abase + (2 * it + 1) * kTcATile + 128, hi1);
      }
      // activations of the group (rows past its end are zeros): two pieces -> the B tile of their sub-block
      const uint32_t bdst = base + L::b + b * (8 * kTcBTile) + (xc16 >> 1) * kTcBTile + (xc16 & 1) * 128;
      sts128(bdst + (xn >> 3) * 256 + (xn & 7) * 16, have.x0);
      sts128(bdst + ((xn + 16) >> 3) * 256 + (xn & 7) * 16, have.x1);
      // the scale tables of this buffer are free once the drain warps are through with stage seq - 2
      if (!wait(s_free(b), (j & 1u) ^ 1u)) return false;
      {  // d * sc and dmin * mn of this thread's four sub-blocks (6-bit integers -> float through the mantissa
         // of 8388608.0f, no conversion instruction), 16 bytes per row and kind: conflict-free both ways
        const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
        float sw[4], mw[4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          uint32_t scp, mnp;
          q4k_scale_pair(hdr.y, hdr.z, hdr.w, 2 * uh + i, scp, mnp);
          sw[2 * i]     = dd.x * (__uint_as_float(0x4B000000u | (scp & 0xFFu)) - 8388608.0f);
          sw[2 * i + 1] = dd.x * (__uint_as_float(0x4B000000u | (scp >> 8)) - 8388608.0f);
          mw[2 * i]     = dd.y * (__uint_as_float(0x4B000000u | (mnp & 0xFFu)) - 8388608.0f);
          mw[2 * i + 1] = dd.y * (__uint_as_float(0x4B000000u | (mnp >> 8)) - 8388608.0f);
        }
        const uint32_t wsb = base + L::ws + ((b * 2 + uh) * 2 * 128 + u) * 16;
        asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(wsb), "f"(sw[0]), "f"(sw[1]), "f"(sw[2]), "f"(sw[3]) : "memory");
        asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(wsb + 128 * 16), "f"(mw[0]), "f"(mw[1]), "f"(mw[2]), "f"(mw[3]) : "memory");
      }
      const uint32_t dxb = base + L::dx + b * (16 * kTcNT * 4);
      sts32f(dxb + ((ut >> 5) * kTcNT + (ut & 31)) * 4, __uint_as_float(have.sv.x));
      sts32f(dxb + ((8 + (ut >> 5)) * kTcNT + (ut & 31)) * 4, __uint_as_float(have.sv.y));
      fence_proxy_async();   // generic-proxy writes (A, B tiles) -> async-proxy reads by the MMA
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(a_full(b));
        mbar_arrive(w_empty(s));
      }
      return true;
    };
    const int my_tiles = blockIdx.x < total_tiles ? (total_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const uint32_t nstages = static_cast<uint32_t>(my_tiles) * nks;
    // two stages per trip with the piece registers swapping roles, so that a stage's loads land in the
    // registers they are used from (no register move has to wait for a load in flight)
    Pieces pa, pb;
    fetch(pa);
    for (uint32_t seq = 0; seq < nstages && ok; seq += 2) {
      fetch(pb);
      ok = stage(seq, pa);
      if (ok && seq + 1 < nstages) {
        fetch(pa);
        ok = stage(seq + 1, pb);
      }
    }
  } else if (warp == kTcWarpMma) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      uint32_t seq = 0;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (int ks = 0; ks < nks; ++ks, ++seq) {
          const int b = seq & 1u;
          const uint32_t j = seq >> 1;
          if (!wait(a_full(b), j & 1u) || !wait(t_empty(b), (j & 1u) ^ 1u)) { ok = false; break; }
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
    const int q = warp & 3, hf = (warp >> 2) & 1, sh = warp >> 3;   // lane quadrant, column half, sub-block half
    const int row = q * 32 + lane;
    const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + sh * (4 * kTcNT);
    uint32_t seq = 0, tile_no = 0;
    int4 gi_next = blockIdx.x < total_tiles ? ld_dep(p.groups + blockIdx.x / p.row_tiles) : make_int4(0, 0, 0, 0);
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_no) {
      const int g = t / p.row_tiles, rb = t - g * p.row_tiles;
      const int4 gi = gi_next;   // requested a tile ago
      if (t + static_cast<int>(gridDim.x) < total_tiles) gi_next = ld_dep(p.groups + (t + gridDim.x) / p.row_tiles);
      // the group's activation rows are split between the warps that share a TMEM lane quadrant:
      // columns [0, h0) and [h0, n), h0 a multiple of 8
      const int h0 = min(gi.z, (((gi.z + 1) >> 1) + 7) & ~7);
      const int c0 = hf ? h0 : 0;
      const int ncol = hf ? gi.z - h0 : h0;
      const int n8 = (ncol + 7) >> 3;
      const int r0 = rb * p.tile_rows;
      float acc[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) acc[c] = 0.f;
      for (int ks = 0; ks < nks; ++ks, ++seq) {
        const int b = seq & 1u;
        const uint32_t j = seq >> 1;
        const int s = static_cast<int>(seq % kStages);
        if (!wait(a_full(b), j & 1u) || !wait(mma_done(b), j & 1u)) { ok = false; break; }
        tc_after();
        if (p.dots != nullptr && n8 > 0) {   // parity probe: the exact integer sub-block dots of the production MMAs, read before the slots are preset again
          const int jrow = MODE == 1 ? (row < 64 ? r0 + row : -1) : (row < p.tile_rows ? r0 + row : -1);
          for (int s4 = 0; s4 < 4; ++s4) {
            int d[16];
            tc_ld16(taddr0 + b * 256 + c0 + s4 * kTcNT, d);   // columns past the group's rows are read but not stored
            tc_wait_ld();
            if (jrow >= 0 && jrow < p.N) {
#pragma unroll
              for (int c = 0; c < 16; ++c)
                if (c < ncol)
                  p.dots[(static_cast<size_t>(gi.y + c0 + c) * p.N + jrow) * (p.K / 32) + ks * 8 + sh * 4 + s4] = d[c];
            }
          }
        }
        const uint32_t wsb = base + L::ws + ((b * 2 + sh) * 2 * 128 + row) * 16;
        const float4 swv = lds128f(wsb), mwv = lds128f(wsb + 128 * 16);
        const float sws[4] = {swv.x, swv.y, swv.z, swv.w}, mws[4] = {mwv.x, mwv.y, mwv.z, mwv.w};
        const uint32_t slot0 = taddr0 + b * 256;
        const uint32_t taddr = slot0 + c0;
        const uint32_t dxb = base + L::dx + b * (16 * kTcNT * 4) + (sh * 4 * kTcNT + c0) * 4;
        if (n8 == 1) {
          tc_drain_half<1>(acc, taddr, sws, mws, dxb, t_empty(b), lane);
        } else if (n8 == 2) {
          tc_drain_half<2>(acc, taddr, sws, mws, dxb, t_empty(b), lane);
        } else {
          tc_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(t_empty(b));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free(b));   // done with this stage's scale tables
      }
      if (!ok) break;
      // ---- the two sub-block halves meet: warps of half 1 hand their sums to the warps of half 0 ----
      {
        const uint32_t rb_ = base + L::red + ((q * 2 + hf) * 16 * 32 + lane) * 4;
        if (sh == 1) {
          if (!wait(red_empty, (tile_no & 1u) ^ 1u)) { ok = false; break; }
#pragma unroll
          for (int c = 0; c < 16; ++c) sts32f(rb_ + c * 128, acc[c]);
          __syncwarp();
          if (lane == 0) mbar_arrive(red_full);
          continue;
        }
        if (!wait(red_full, tile_no & 1u)) { ok = false; break; }
#pragma unroll
        for (int c = 0; c < 16; ++c) acc[c] += lds32f(rb_ + c * 128);
        __syncwarp();
        if (lane == 0) mbar_arrive(red_empty);
      }
      // ---- epilogue of the tile (warps of sub-block half 0) ----
      if (MODE == 1) {
        const uint32_t exb = base + L::ex + ((hf * 2 + (q & 1)) * 16 * 32 + lane) * 4;
        if (q >= 2) {
          if (!wait(ex_empty, (tile_no & 1u) ^ 1u)) { ok = false; break; }
#pragma unroll
          for (int c = 0; c < 16; ++c) sts32f(exb + c * 128, acc[c]);
          __syncwarp();
          if (lane == 0) mbar_arrive(ex_full);
        } else {
          if (!wait(ex_full, tile_no & 1u)) { ok = false; break; }
          float upv[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) upv[c] = lds32f(exb + c * 128);
          __syncwarp();
          if (lane == 0) mbar_arrive(ex_empty);
          const int jcol = r0 + row;          // row < 64: this thread's gate row
          const int blk = jcol >> 5;          // 32-block of the act row this warp's lanes form
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            if (c < ncol) {                   // uniform across the warp
              float v = acc[c];
              v = (v / (1.0f + expf(-v))) * upv[c];
              if (p.round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
              if (jcol >= p.N) v = 0.f;
              const size_t ps = static_cast<size_t>(gi.y + c0 + c);
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
              const int ps = gi.y + c0 + c;
              if (MODE == 2) {
                const int srow = ld_dep(p.list + ps) / p.S;
                store_scalar(static_cast<YT*>(p.dst) + static_cast<size_t>(srow) * p.ld_dst + jrow, acc[c]);
              } else if (MODE == 0 && p.po.out != nullptr) {
                peer_out_row(p.po, ld_dep(p.list + ps), p.N)[jrow] = acc[c];
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
  if (MODE == 0) peer_out_finish(p.po, gridDim.x);
  tc_before();
  __syncthreads();
  if (warp == kTcWarpMma)
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
