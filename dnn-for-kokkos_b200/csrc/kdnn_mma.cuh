// Grouped int8 tile GEMM for Q4_K weights on the tensor cores (mma.sync m16n8k32,
// u8 x s8 -> s32), used when a weight row meets several activation rows (batched
// GEMM, MoE experts).
//
//   dst[pos, j] = sum_k W_g[j, k] * x[row(pos), k]
//
// with the reference's int8 numerics: activations are per-32 int8 blocks, every
// 32-element sub-block product is an exact int32 (one MMA k-step = one Q4_K
// sub-block), and the fp32 fold  acc += (d*sc) * dx * dot - (dmin*mn) * dx * sum
// happens in registers right after the MMA -- the accumulator of mma.sync already
// lives there, which is what a rescale every 32 elements wants.
#pragma once

#include <atomic>

#include "kdnn_tile.cuh"

namespace kdnn {

struct MmaParams {
  const uintptr_t* w0;   // per-group payload addresses
  const uintptr_t* w1;   // up (MODE 1)
  int row_bytes;         // K / 256 * 144
  int N, K;
  const int* offs;       // [groups + 1]
  const int* list;       // slot id at each position
  int S;                 // slots per token
  int g_first;
  const uint8_t* xrows;  // quantized activation rows (layout: see act_row_pitch)
  size_t x_pitch;        // bytes between rows
                         // MODE 0 indexed by position, MODE 1 / 2 by slot / S
  void* dst;             // MODE 0, 1: float [npos, N]; MODE 2: YT [rows, ld_dst] indexed by slot / S
  size_t ld_dst;
  int round_bf16;
  uint8_t* qdst;         // MODE 1: when set, the epilogue writes quantized activation rows (by position)
  size_t q_pitch;        //         here instead of floats to dst
  int* status;
  int passes_z;          // CTAs along z that share a group's 32-row passes (0 = 1)
  int early;             // launch as a programmatic dependent (only worth it behind a tiny kernel, see launch_chained_if)
  PeerOut po;            // MODE 0: po.out != null writes the rows into this rank's slot-indexed buffer (read by the token owners)
};

__device__ __forceinline__ int4 lds128_g(uint32_t a) {
  int4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

// Structure:
//  * a warp owns 16 rows of ONE matrix (MODE 1: even warps gate, odd warps up, the two
//    meet in shared memory for the SwiGLU epilogue), so a CTA needs half the shared memory
//    and registers and two CTAs fit on an SM;
//  * up to 32 activation rows per pass (1..4 n8 tiles chosen at run time), staged in
//    512-element chunks with cp.async, double buffered: one __syncthreads per chunk;
//    the packed weight rows come the same way (16-byte cp.async pieces into a three-stage
//    ring per warp), awaited together with the activation chunk;
//  * the 6-bit scales of a super-block are expanded once per warp (one lane per row and
//    half) into a per-warp table instead of by every lane that needs them;
//  * packed bytes are read 64 bits at a time in a K order that both operands share
//    (mma k-slot 4*tig+i <- element 8*tig+i, slot 16+4*tig+i <- element 8*tig+4+i);
//  * the MMA accumulator starts at the bit pattern of 12582912.0f, so the int32 result is
//    already the float 12582912 + dot and one exact subtraction replaces the int->float
//    conversion; the high nibbles are used in place as unsigned bytes (16 * nibble), their
//    factor 16 goes into the scale.
//  * the min term  -dmin * sum_sb mn[row, sb] * (dx * sum)[token, sb]  of a super-block is a
//    16 x 8 x 8 matrix product of its own: the 6-bit mn are exact in bf16, the row quantizers
//    leave dx * sum split into three bf16 parts (24 bits), so three mma.sync m16n8k8 bf16 and
//    one fma per accumulator replace eight fmas per accumulator.
constexpr int kM2Warps   = 8;
constexpr int kM2NT      = 32;                 // activation rows per pass
constexpr int kM2KC      = 512;                // activation elements per staged chunk
constexpr int kM2XPitch  = kM2KC + 32;         // int8 row pitch: 8 words mod 32 (conflict-free 64-bit B loads)
constexpr int kM2WPitch  = 160;                // packed row pitch in a weight stage (same property)
constexpr int kM2Stages  = 3;                  // weight ring depth per warp, in super-blocks
constexpr int kM2StageBytes = 16 * kM2WPitch;
constexpr int kM2MagicI  = 0x4B400000;
constexpr float kM2MagicF = 12582912.0f;

__device__ __forceinline__ void mma_u8s8_magic(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(kM2MagicI));
}
// Shared loads with a compile-time byte offset folded into the instruction.
template <int OFF>
__device__ __forceinline__ uint2 lds64_o(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ int4 lds128_o(uint32_t a) {
  int4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFF));
  return v;
}
__device__ __forceinline__ uint2 lds64_g(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;   // 0: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 8 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
template <int OFF>
__device__ __forceinline__ uint32_t lds32_o(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
  return v;
}
// d = a (16 x 8, bf16) * b (8 x 8, bf16) + c, fp32 accumulation
__device__ __forceinline__ void mma_bf16_k8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b, float c0, float c1,
                                            float c2, float c3) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(b), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}
// Quantized activation row: the reference staging layout (int8 xq[K], at align16(K) one {d, sum_lo, sum_hi,
// pad} per 32), then one float2 {d, d * block sum} per 32, then per 256 elements 48 bytes: d * block sum of
// its eight blocks as three bf16 parts (8 high parts, 8 middle parts, 8 low parts; their sum is the float
// to 24 bits), the form the tile kernels consume.
__host__ __device__ inline size_t act_parts_offset(size_t K) { return act_bytes(K) + 8 * (K / 32); }
__device__ __forceinline__ void store_sum_parts(uint8_t* row, size_t parts_off, int b, float ds) {
  const __nv_bfloat16 p0 = __float2bfloat16_rn(ds);
  const float r1 = ds - __bfloat162float(p0);
  const __nv_bfloat16 p1 = __float2bfloat16_rn(r1);
  const __nv_bfloat16 p2 = __float2bfloat16_rn(r1 - __bfloat162float(p1));
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(row + parts_off + static_cast<size_t>(b >> 3) * 48) + (b & 7);
  dst[0] = p0; dst[8] = p1; dst[16] = p2;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

template <int MODE>
struct M2Layout {
  static constexpr int kRowsPerCta = MODE == 1 ? 64 : 128;
  static constexpr size_t xq    = 0;                                                   // [2][NT][XPitch] int8
  static constexpr size_t xs    = xq + 2 * kM2NT * kM2XPitch;                          // [2][KC/32][NT] float dx
  static constexpr size_t xp    = xs + 2 * (kM2KC / 32) * kM2NT * 4;                   // [2][KC/256][3 parts][NT][8 bf16]
  static constexpr size_t rowp  = xp + 2 * (kM2KC / 256) * 3 * kM2NT * 16;             // [NT] activation row offsets
  static constexpr size_t outp  = rowp + kM2NT * 8;                                    // [NT] output rows in the owners' buffers (scatter mode)
  static constexpr size_t tab   = outp + kM2NT * 8;                                    // [warps][16 rows]{sw[8], mn[8] bf16, -dmin, pad}
  static constexpr size_t ring  = (tab + kM2Warps * 16 * 4 * 16 + 127) & ~size_t(127); // [warps][stages][16][WPitch]
  static constexpr size_t total = ring + kM2Warps * kM2Stages * kM2StageBytes + 128;
};

#ifndef KDNN_M2_F32X2
#define KDNN_M2_F32X2 1   // fold with the packed fp32x2 instructions of sm_100 (0: scalar fma, for A/B runs)
#endif
// Packed fp32 pairs (one instruction, two lanes of arithmetic): d = a * b + c, a * b, a + b.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rc, rd;\n"
      "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rc, {%6, %7};\n"
      "fma.rn.f32x2 rd, ra, rb, rc;\n"
      "mov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rd;\n"
      "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\n"
      "mul.rn.f32x2 rd, ra, rb;\n"
      "mov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rd;\n"
      "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\n"
      "add.rn.f32x2 rd, ra, rb;\n"
      "mov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// One sub-block MMA of n8 tile T and its fold: acc += (sw * dx) * dot.
template <int IT, int PAR, int T>
__device__ __forceinline__ void m2_tile(float (&acc)[4][4], const uint32_t (&a)[4], float swA, float swB,
                                        uint32_t b_addr, uint32_t s_addr) {
  constexpr int blk = 2 * IT + PAR;
  const uint2 b   = lds64_o<T * (8 * kM2XPitch) + blk * 32>(b_addr);
  const uint2 dxv = lds64_o<(blk * kM2NT + 8 * T) * 4>(s_addr);   // dx of tokens 2 tig, 2 tig + 1
  int cfrag[4];
  mma_u8s8_magic(cfrag, a, b.x, b.y);
#if KDNN_M2_F32X2
  // the two tokens of a row as one packed pair: six instructions instead of twelve
  const float2 dx = make_float2(__uint_as_float(dxv.x), __uint_as_float(dxv.y));
  const float2 nm = make_float2(-kM2MagicF, -kM2MagicF);
  const float2 fA = fadd2(make_float2(__int_as_float(cfrag[0]), __int_as_float(cfrag[1])), nm);
  const float2 fB = fadd2(make_float2(__int_as_float(cfrag[2]), __int_as_float(cfrag[3])), nm);
  const float2 rA = ffma2(fmul2(make_float2(swA, swA), dx), fA, make_float2(acc[T][0], acc[T][1]));
  const float2 rB = ffma2(fmul2(make_float2(swB, swB), dx), fB, make_float2(acc[T][2], acc[T][3]));
  acc[T][0] = rA.x; acc[T][1] = rA.y; acc[T][2] = rB.x; acc[T][3] = rB.y;
#else
  const float dx0 = __uint_as_float(dxv.x), dx1 = __uint_as_float(dxv.y);
  const float f0 = __int_as_float(cfrag[0]) - kM2MagicF, f1 = __int_as_float(cfrag[1]) - kM2MagicF;
  const float f2 = __int_as_float(cfrag[2]) - kM2MagicF, f3 = __int_as_float(cfrag[3]) - kM2MagicF;
  acc[T][0] = fmaf(swA * dx0, f0, acc[T][0]);
  acc[T][1] = fmaf(swA * dx1, f1, acc[T][1]);
  acc[T][2] = fmaf(swB * dx0, f2, acc[T][2]);
  acc[T][3] = fmaf(swB * dx1, f3, acc[T][3]);
#endif
}

template <int NTILES, int IT>
__device__ __forceinline__ void m2_it(float (&acc)[4][4], uint32_t wa_addr, uint32_t ta_addr, uint32_t b_addr,
                                      uint32_t s_addr) {
  const uint2 wa = lds64_o<IT * 32>(wa_addr);
  const uint2 wb = lds64_o<8 * kM2WPitch + IT * 32>(wa_addr);
  const uint2 ta = lds64_o<IT * 8>(ta_addr);            // sw of sub-blocks 2 IT, 2 IT + 1, row gid
  const uint2 tb = lds64_o<8 * 64 + IT * 8>(ta_addr);   // row gid + 8
  {
    const uint32_t a[4] = {wa.x & 0x0F0F0F0Fu, wb.x & 0x0F0F0F0Fu, wa.y & 0x0F0F0F0Fu, wb.y & 0x0F0F0F0Fu};
    const float swA = __uint_as_float(ta.x), swB = __uint_as_float(tb.x);
    m2_tile<IT, 0, 0>(acc, a, swA, swB, b_addr, s_addr);
    if (NTILES > 1) m2_tile<IT, 0, 1>(acc, a, swA, swB, b_addr, s_addr);
    if (NTILES > 2) m2_tile<IT, 0, 2>(acc, a, swA, swB, b_addr, s_addr);
    if (NTILES > 3) m2_tile<IT, 0, 3>(acc, a, swA, swB, b_addr, s_addr);
  }
  {
    const uint32_t a[4] = {wa.x & 0xF0F0F0F0u, wb.x & 0xF0F0F0F0u, wa.y & 0xF0F0F0F0u, wb.y & 0xF0F0F0F0u};
    const float swA = __uint_as_float(ta.y), swB = __uint_as_float(tb.y);
    m2_tile<IT, 1, 0>(acc, a, swA, swB, b_addr, s_addr);
    if (NTILES > 1) m2_tile<IT, 1, 1>(acc, a, swA, swB, b_addr, s_addr);
    if (NTILES > 2) m2_tile<IT, 1, 2>(acc, a, swA, swB, b_addr, s_addr);
    if (NTILES > 3) m2_tile<IT, 1, 3>(acc, a, swA, swB, b_addr, s_addr);
  }
}

// Min term of one super-block for n8 tile T: acc -= dmin[row] * sum_sb mn[row, sb] * (dx * sum)[token, sb].
template <int T>
__device__ __forceinline__ void m2_min(float (&acc)[4][4], uint32_t a0, uint32_t a1, float ndA, float ndB,
                                       uint32_t p_addr) {
  const uint32_t b0 = lds32_o<(0 * kM2NT + 8 * T) * 16>(p_addr);
  const uint32_t b1 = lds32_o<(1 * kM2NT + 8 * T) * 16>(p_addr);
  const uint32_t b2 = lds32_o<(2 * kM2NT + 8 * T) * 16>(p_addr);
  float m[4];
  mma_bf16_k8(m, a0, a1, b2, 0.f, 0.f, 0.f, 0.f);   // low parts first
  mma_bf16_k8(m, a0, a1, b1, m[0], m[1], m[2], m[3]);
  mma_bf16_k8(m, a0, a1, b0, m[0], m[1], m[2], m[3]);
#if KDNN_M2_F32X2
  const float2 rA = ffma2(make_float2(ndA, ndA), make_float2(m[0], m[1]), make_float2(acc[T][0], acc[T][1]));
  const float2 rB = ffma2(make_float2(ndB, ndB), make_float2(m[2], m[3]), make_float2(acc[T][2], acc[T][3]));
  acc[T][0] = rA.x; acc[T][1] = rA.y; acc[T][2] = rB.x; acc[T][3] = rB.y;
#else
  acc[T][0] = fmaf(ndA, m[0], acc[T][0]);
  acc[T][1] = fmaf(ndA, m[1], acc[T][1]);
  acc[T][2] = fmaf(ndB, m[2], acc[T][2]);
  acc[T][3] = fmaf(ndB, m[3], acc[T][3]);
#endif
}

// One super-block (16 rows in stage `st`, scale table `tab`) against NTILES n8 tiles of
// activations: `xb` / `sx` point at the super-block's first 32-block in the staged chunk,
// `xp` at its three rows of bf16 sum parts.
template <int NTILES>
__device__ __forceinline__ void m2_superblock(float (&acc)[4][4], uint32_t st, uint32_t tab, uint32_t xb, uint32_t sx,
                                              uint32_t xp, int gid, int tig) {
  const uint32_t wa_addr = st + gid * kM2WPitch + 16 + 8 * tig;
  const uint32_t ta_addr = tab + gid * 64;
  const uint32_t b_addr  = xb + gid * kM2XPitch + 8 * tig;
  const uint32_t s_addr  = sx + tig * 8;
  m2_it<NTILES, 0>(acc, wa_addr, ta_addr, b_addr, s_addr);
  m2_it<NTILES, 1>(acc, wa_addr, ta_addr, b_addr, s_addr);
  m2_it<NTILES, 2>(acc, wa_addr, ta_addr, b_addr, s_addr);
  m2_it<NTILES, 3>(acc, wa_addr, ta_addr, b_addr, s_addr);
  const uint32_t m_addr = ta_addr + 32 + 4 * tig;       // mn of sub-blocks 2 tig, 2 tig + 1 as a bf16 pair
  const uint32_t a0 = lds32_o<0>(m_addr), a1 = lds32_o<8 * 64>(m_addr);
  const float ndA = __uint_as_float(lds32_o<48>(ta_addr)), ndB = __uint_as_float(lds32_o<8 * 64 + 48>(ta_addr));
  const uint32_t p_addr = xp + gid * 16 + 4 * tig;      // token gid of a tile, blocks 2 tig, 2 tig + 1
  m2_min<0>(acc, a0, a1, ndA, ndB, p_addr);
  if (NTILES > 1) m2_min<1>(acc, a0, a1, ndA, ndB, p_addr);
  if (NTILES > 2) m2_min<2>(acc, a0, a1, ndA, ndB, p_addr);
  if (NTILES > 3) m2_min<3>(acc, a0, a1, ndA, ndB, p_addr);
}

template <int MODE, class YT>
__global__ void __launch_bounds__(kM2Warps * 32, 2) grouped_mma2_q4k_kernel(const MmaParams p) {
  using L = M2Layout<MODE>;
  extern __shared__ __align__(128) uint8_t m2_smem[];
  pdl_chain_entry();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int g   = blockIdx.y;
  const int beg = p.offs[g], n_g = p.offs[g + 1] - beg;
  if (n_g <= 0) {
    if (MODE == 0) peer_out_finish(p.po, gridDim.x * gridDim.y * gridDim.z);
    return;
  }

  const uint32_t xq_u32 = smem_u32(m2_smem + L::xq), xs_u32 = smem_u32(m2_smem + L::xs);
  const uint32_t xp_u32 = smem_u32(m2_smem + L::xp);
  long long* rowp = reinterpret_cast<long long*>(m2_smem + L::rowp);
  float** outp = reinterpret_cast<float**>(m2_smem + L::outp);
  const uint32_t tab_u32 = smem_u32(m2_smem + L::tab) + warp * (16 * 4 * 16);
  const uint32_t ring_u32 = smem_u32(m2_smem + L::ring) + warp * (kM2Stages * kM2StageBytes);

  const int mat  = MODE == 1 ? (warp & 1) : 0;
  const int slab = MODE == 1 ? (warp >> 1) : warp;
  const int row_base = blockIdx.x * L::kRowsPerCta + slab * 16;
  const int nsb  = p.K / 256;
  // Weight stages are filled with 16-byte cp.async pieces (a stage is 16 rows x 144 bytes = 144 pieces,
  // spread over the lanes): bulk copies of 144 bytes each were limited by their per-copy cost.
  // Rows past the end re-read the last row.
  const uint8_t* wbase = reinterpret_cast<const uint8_t*>((mat == 0 ? p.w0 : p.w1)[p.g_first + g]);
  uint32_t psrc[5], pdst[5];   // byte offsets of this lane's pieces: source (from wbase), destination (stage 0)
#pragma unroll
  for (int j = 0; j < 5; ++j) {
    const int pc = lane + 32 * j;                      // piece index, valid below 144
    const int r = (pc * 7282) >> 16, c = pc - 9 * r;   // pc / 9 for pc < 160
    psrc[j] = static_cast<uint32_t>(min(row_base + min(r, 15), p.N - 1)) * static_cast<uint32_t>(p.row_bytes) + c * 16;
    pdst[j] = ring_u32 + min(r, 15) * kM2WPitch + c * 16;
  }
  // Stage sb % 3 holds super-block sb. Every call commits exactly one group (an empty one past the
  // last super-block), so at the top of chunk c the groups still allowed to be pending are always the
  // same: the one stage requested last. What is in flight during a chunk's arithmetic is the next
  // chunk's bytes plus one stage of the chunk after it.
  auto issue = [&](int sb) {   // whole warp
    if (sb < nsb) {
      const uint32_t so = (sb % kM2Stages) * kM2StageBytes;
      const uint8_t* srcb = wbase + static_cast<size_t>(sb) * 144;
#pragma unroll
      for (int j = 0; j < 5; ++j)
        if (j < 4 || lane < 16) cp_async16(pdst[j] + so, srcb + psrc[j], true);
    }
    cp_async_commit();
  };

  const int nchunk = (p.K + kM2KC - 1) / kM2KC;
  const size_t scale_off = act_bytes(static_cast<size_t>(p.K));
  const size_t parts_off = act_parts_offset(static_cast<size_t>(p.K));
  // cp.async of one activation chunk: NT rows x kc int8, NT x kc/32 scales d, and per row and
  // super-block the three 16-byte rows of bf16 sum parts
  auto stage_chunk = [&](int c) {
    const int k0 = c * kM2KC, kc = min(kM2KC, p.K - k0);
    const uint32_t xb = xq_u32 + (c & 1) * (kM2NT * kM2XPitch);
    const int lg = kc == kM2KC ? 5 : 31 - __clz(kc / 16);   // 16-byte pieces per row: a power of two
    const int per_row = 1 << lg;
    for (int f = threadIdx.x; f < kM2NT * per_row; f += blockDim.x) {
      const int t = f >> lg, c16 = f & (per_row - 1);
      const long long ro = rowp[t];
      cp_async16(xb + t * kM2XPitch + c16 * 16, p.xrows + (ro < 0 ? 0 : ro) + k0 + c16 * 16, ro >= 0);
    }
    const uint32_t sbuf = xs_u32 + (c & 1) * ((kM2KC / 32) * kM2NT * 4);
    const int nb = kc / 32;
    for (int f = threadIdx.x; f < kM2NT * nb; f += blockDim.x) {
      const int b = f / kM2NT, t = f - b * kM2NT;   // consecutive threads fill consecutive 4-byte slots
      const long long ro = rowp[t];
      cp_async4(sbuf + (b * kM2NT + t) * 4, p.xrows + (ro < 0 ? 0 : ro) + scale_off + static_cast<size_t>(k0 / 32 + b) * 8,
                ro >= 0);
    }
    const uint32_t pbuf = xp_u32 + (c & 1) * ((kM2KC / 256) * 3 * kM2NT * 16);
    const int npc = 3 * (kc / 256);               // 16-byte pieces per row: [super-block][part]
    for (int f = threadIdx.x; f < kM2NT * npc; f += blockDim.x) {
      const int pc = f / kM2NT, t = f - pc * kM2NT;
      const long long ro = rowp[t];
      cp_async16(pbuf + (pc * kM2NT + t) * 16,
                 p.xrows + (ro < 0 ? 0 : ro) + parts_off + static_cast<size_t>(k0 / 256) * 48 + pc * 16, ro >= 0);
    }
    cp_async_commit();
  };

  // passes of 32 activation rows: pass z, z + gridDim.z, ... belong to this CTA, so a group with many rows
  // is spread over several CTAs instead of keeping one CTA for several passes
  for (int t0 = blockIdx.z * kM2NT; t0 < n_g; t0 += gridDim.z * kM2NT) {
    const int nt = min(kM2NT, n_g - t0);
    const int ntiles = (nt + 7) >> 3;
    __syncthreads();   // the previous pass is done with every buffer
    if (threadIdx.x < kM2NT) {
      long long ro = -1;
      if (threadIdx.x < nt) {
        const int srow = MODE == 0 ? beg + t0 + threadIdx.x : p.list[beg + t0 + threadIdx.x] / p.S;
        ro = static_cast<long long>(srow) * static_cast<long long>(p.x_pitch);
      }
      rowp[threadIdx.x] = ro;
      if (MODE == 0 && p.po.out != nullptr)
        outp[threadIdx.x] = threadIdx.x < nt ? peer_out_row(p.po, p.list[beg + t0 + threadIdx.x], p.N) : nullptr;
    }
    __syncthreads();
    stage_chunk(0);
    for (int q = 0; q < kM2Stages; ++q) issue(q);

    float acc[4][4];
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;

    for (int c = 0; c < nchunk; ++c) {
      cp_async_wait_but_one();
      __syncthreads();   // chunk c has landed for everybody; everybody is done with chunk c - 1
      if (c + 1 < nchunk) stage_chunk(c + 1); else cp_async_commit();
      const uint32_t xb = xq_u32 + (c & 1) * (kM2NT * kM2XPitch);
      const uint32_t sbuf = xs_u32 + (c & 1) * ((kM2KC / 32) * kM2NT * 4);
      const uint32_t pbuf = xp_u32 + (c & 1) * ((kM2KC / 256) * 3 * kM2NT * 16);
      const int sb_first = c * (kM2KC / 256), sb_last = min(nsb, sb_first + kM2KC / 256);
      for (int sb = sb_first; sb < sb_last; ++sb) {
        const uint32_t st = ring_u32 + (sb % kM2Stages) * kM2StageBytes;
        {  // expand the 6-bit scales: lane = (row, half) -> {sw0, mw0, sw1, mw1} pairs of its four sub-blocks
          const int r = lane >> 1, half = lane & 1;
          const int4 h = lds128_g(st + r * kM2WPitch);
          const uint32_t s0 = h.y, s1 = h.z, s2 = h.w;
          const uint32_t sc4 = half ? ((s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u)) : (s0 & 0x3F3F3F3Fu);
          const uint32_t mn4 = half ? (((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u)) : (s1 & 0x3F3F3F3Fu);
          const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
          float sw[4];
          uint32_t mb[4];   // fp32 bits of the 6-bit mins: small integers, so the high half is the exact bf16
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float fs = __uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7650u | j)) - 8388608.0f;
            const float fm = __uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7650u | j)) - 8388608.0f;
            sw[j] = dd.x * fs * ((j & 1) ? 0.0625f : 1.0f);   // odd sub-blocks: high nibbles carry a factor 16
            mb[j] = __float_as_uint(fm);
          }
          // table entry [row] = {sw[8] floats, mn[8] bf16, -dmin, pad}; this lane owns sub-blocks 4 half .. 4 half + 3
          const uint32_t ta = tab_u32 + r * 64;
          asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(ta + half * 16), "f"(sw[0]), "f"(sw[1]), "f"(sw[2]), "f"(sw[3]) : "memory");
          asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(ta + 32 + half * 8), "r"(__byte_perm(mb[0], mb[1], 0x7632)),
                       "r"(__byte_perm(mb[2], mb[3], 0x7632)) : "memory");
          if (half == 0) asm volatile("st.shared.f32 [%0], %1;" ::"r"(ta + 48), "f"(-dd.y) : "memory");
        }
        __syncwarp();
        const int blk0 = (sb - sb_first) * 8;   // first 32-block of this super-block inside the chunk
        switch (ntiles) {
          case 1: m2_superblock<1>(acc, st, tab_u32, xb + blk0 * 32, sbuf + blk0 * (kM2NT * 4), pbuf + (sb - sb_first) * (3 * kM2NT * 16), gid, tig); break;
          case 2: m2_superblock<2>(acc, st, tab_u32, xb + blk0 * 32, sbuf + blk0 * (kM2NT * 4), pbuf + (sb - sb_first) * (3 * kM2NT * 16), gid, tig); break;
          case 3: m2_superblock<3>(acc, st, tab_u32, xb + blk0 * 32, sbuf + blk0 * (kM2NT * 4), pbuf + (sb - sb_first) * (3 * kM2NT * 16), gid, tig); break;
          default: m2_superblock<4>(acc, st, tab_u32, xb + blk0 * 32, sbuf + blk0 * (kM2NT * 4), pbuf + (sb - sb_first) * (3 * kM2NT * 16), gid, tig); break;
        }
        __syncwarp();   // every lane has read this stage and the table
        issue(sb + kM2Stages);
      }
    }
    // ---- epilogue ----
    if (MODE == 1) {
      __syncthreads();   // activation buffers are free: the up warps hand their tile to the gate warps
      float* ex = reinterpret_cast<float*>(m2_smem + L::xq) + slab * (16 * 32 + 32);
      if (mat == 1) {
#pragma unroll
        for (int t = 0; t < 4; ++t)
          if (t < ntiles)
#pragma unroll
            for (int i = 0; i < 4; ++i) ex[(t * 4 + i) * 32 + lane] = acc[t][i];
      }
      __syncthreads();
      // act tile of this CTA for the fused quantizer: [token][64 columns], behind the exchange area
      float* tile = reinterpret_cast<float*>(m2_smem + L::xq) + 4 * (16 * 32 + 32);
      if (mat == 0) {
#pragma unroll
        for (int t = 0; t < 4; ++t)
          if (t < ntiles)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int tok = 8 * t + 2 * tig + (i & 1);
            const int jl  = slab * 16 + gid + 8 * (i >> 1);
            const int j   = blockIdx.x * L::kRowsPerCta + jl;
            const float u = ex[(t * 4 + i) * 32 + lane];
            float v = acc[t][i];
            v = (v / (1.0f + expf(-v))) * u;
            if (p.round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
            if (p.qdst) tile[tok * 64 + jl] = j < p.N ? v : 0.f;
            else if (tok < nt && j < p.N) static_cast<float*>(p.dst)[static_cast<size_t>(beg + t0 + tok) * p.N + j] = v;
          }
      }
      if (p.qdst) {
        // per-32 int8 quantization of the tile (the reference's stage-1 quantizer, four lanes per
        // block) straight into the rows the down projection reads
        __syncthreads();
        const int pair = threadIdx.x >> 2, l4 = threadIdx.x & 3;
        const int tok = pair >> 1, blk = pair & 1;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = tile[tok * 64 + blk * 32 + l4 * 8 + i];
        float d;
        int part, total;
        const uint2 packed = quantize_block_lane8(v, d, part, total);
        const int b = blockIdx.x * 2 + blk;   // 32-block index inside the row
        if (tok < nt && (b + 1) * 32 <= p.N) {
          uint8_t* row = p.qdst + static_cast<size_t>(beg + t0 + tok) * p.q_pitch;
          reinterpret_cast<uint2*>(row + static_cast<size_t>(b) * 32)[l4] = packed;
          if (l4 == 0) {
            reinterpret_cast<ActHdr*>(row + act_hdr_offset(static_cast<size_t>(p.N)))[b] = ActHdr{d, part, total - part, 0};
            const float ds = __fmul_rn(static_cast<float>(total), d);
            reinterpret_cast<float2*>(row + act_bytes(static_cast<size_t>(p.N)))[b] = make_float2(d, ds);
            store_sum_parts(row, act_parts_offset(static_cast<size_t>(p.N)), b, ds);
          }
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tok = 8 * t + 2 * tig + (i & 1);
          const int j   = row_base + gid + 8 * (i >> 1);
          if (tok < nt && j < p.N) {
            if (MODE == 2) {
              const int srow = p.list[beg + t0 + tok] / p.S;
              store_scalar(static_cast<YT*>(p.dst) + static_cast<size_t>(srow) * p.ld_dst + j, acc[t][i]);
            } else if (MODE == 0 && p.po.out != nullptr) {
              outp[tok][j] = acc[t][i];
            } else {
              static_cast<float*>(p.dst)[static_cast<size_t>(beg + t0 + tok) * p.N + j] = acc[t][i];
            }
          }
        }
    }
  }
  if (MODE == 0) peer_out_finish(p.po, gridDim.x * gridDim.y * gridDim.z);
}

template <int MODE, class YT>
static cudaError_t launch_grouped_mma(const MmaParams& p, int groups, cudaStream_t st) {
  using L = M2Layout<MODE>;
  auto kern = grouped_mma2_q4k_kernel<MODE, YT>;
  static SmemAttrOnce once;
  const cudaError_t e = set_max_smem_once(once, kern, (int)L::total);
  if (e != cudaSuccess) return e;
  dim3 grid((p.N + L::kRowsPerCta - 1) / L::kRowsPerCta, groups, p.passes_z > 0 ? p.passes_z : 1);
  return launch_chained_if(p.early != 0, kern, grid, dim3(kM2Warps * 32), L::total, st, p);
}

// Batched form of the reference's stage-1 quantizer: row r of `src` (pitch ld
// elements) -> reference staging layout at dst + r * pitch_bytes. Rows at or past
// *nrows_dev (when given) are skipped.
template <class SRC>
__global__ void quantize_rows_kernel(const SRC* src, size_t ld, int nrows, int K,
                                     const int* nrows_dev, uint8_t* dst,
                                     size_t pitch_bytes) {
  pdl_chain_entry();
  const int row = blockIdx.y;
  if (row >= nrows || (nrows_dev && row >= *nrows_dev)) return;
  const int nblk    = K / 32;
  const int lane    = threadIdx.x & 31, l4 = lane & 3;
  const SRC* x      = src + static_cast<size_t>(row) * ld;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  uint8_t* out      = dst + static_cast<size_t>(row) * pitch_bytes;
  ActHdr* gh        = reinterpret_cast<ActHdr*>(out + act_hdr_offset(K));
  float2* gs        = reinterpret_cast<float2*>(out + act_bytes(K));
  const int gwarp   = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarp   = (gridDim.x * blockDim.x) >> 5;
  for (int base = gwarp * 8; base < nblk; base += nwarp * 8) {
    const int b = base + (lane >> 2);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (b < nblk) load8<SRC>(x, static_cast<size_t>(b) * 32 + l4 * 8, vec_ok, v);
    float d;
    int part, total;
    const uint2 packed = quantize_block_lane8(v, d, part, total);
    if (b >= nblk) continue;
    reinterpret_cast<uint2*>(out + static_cast<size_t>(b) * 32)[l4] = packed;
    if (l4 == 0) {
      gh[b] = ActHdr{d, part, total - part, 0};
      const float ds = __fmul_rn(static_cast<float>(total), d);
      gs[b] = make_float2(d, ds);
      store_sum_parts(out, act_parts_offset(static_cast<size_t>(K)), b, ds);
    }
  }
}

template <class SRC>
static cudaError_t launch_quantize_rows(const SRC* src, size_t ld, int nrows, int K, const int* nrows_dev,
                                        uint8_t* dst, size_t pitch_bytes, cudaStream_t st) {
  if (nrows <= 0) return cudaSuccess;
  const int bx = max(1, min(8, (K / 32 + 63) / 64));
  return launch_chained(quantize_rows_kernel<SRC>, dim3(bx, nrows), dim3(256), 0, st, src, ld, nrows, K, nrows_dev, dst,
                        pitch_bytes);
}

// Bytes between quantized activation rows (layout: see act_parts_offset).
inline size_t act_row_pitch(size_t K) { return (act_parts_offset(K) + 48 * ((K / 32 + 7) / 8) + 255) & ~size_t(255); }

}  // namespace kdnn
