// Grouped int8 tile GEMM for Q4_K weights on the tensor cores (mma.sync m16n8k32,
// s8 x s8 -> s32), used when a weight row meets several activation rows (batched
// GEMM, MoE experts).
//
//   dst[pos, j] = sum_k W_g[j, k] * x[row(pos), k]
//
// with the reference's int8 numerics: activations are per-32 int8 blocks, every
// 32-element sub-block product is an exact int32 (one MMA k-step = one Q4_K
// sub-block), and the fp32 fold  acc += (d*sc) * dx * dot - (dmin*mn) * dx * sum
// happens in registers right after the MMA -- the accumulator of mma.sync already
// lives there, which is what a rescale every 32 elements wants.
//
// CTA = 8 warps = 128 weight rows of one group (MODE 1: the same 128 rows of gate
// and of up). Each warp owns 16 rows and streams their packed bytes through a
// private ring of shared-memory stages filled by bulk copies (one 288-byte copy
// per row per stage = two super-blocks); the 16 activation rows of the current
// token tile sit in shared memory as int8 plus per-block scales, staged in
// 2048-element chunks.
#pragma once

#include "kdnn_tile.cuh"

namespace kdnn {

constexpr int kMmaWarps   = 8;
constexpr int kMmaRows    = 16 * kMmaWarps;  // weight rows per CTA
constexpr int kMmaNT      = 16;              // activation rows per tile (two n8 tiles)
constexpr int kMmaKC      = 2048;            // activation elements staged per chunk
constexpr int kMmaSB      = 2;               // super-blocks per weight stage
constexpr int kMmaSeg     = kMmaSB * 144;    // packed bytes per row per stage
constexpr int kMmaSegPad  = kMmaSeg + 16;    // shared-memory pitch (conflict-free A loads)
constexpr int kMmaXPitch  = kMmaKC + 16;     // int8 activation row pitch (conflict-free B loads)
constexpr int kMmaStages  = 2;

struct MmaParams {
  const uintptr_t* w0;   // per-group payload addresses
  const uintptr_t* w1;   // up (MODE 1)
  int row_bytes;         // K / 256 * 144
  int N, K;
  const int* offs;       // [groups + 1]
  const int* list;       // slot id at each position
  int S;                 // slots per token
  int g_first;
  const uint8_t* xrows;  // quantized activation rows, reference staging layout per row:
                         // int8 xq[K], then at align16(K) one {d, sum_lo, sum_hi, pad} per 32
  size_t x_pitch;        // bytes between rows
                         // MODE 0 indexed by position, MODE 1 / 2 by slot / S
  void* dst;             // MODE 0, 1: float [npos, N]; MODE 2: YT [rows, ld_dst] indexed by slot / S
  size_t ld_dst;
  int round_bf16;
  int* status;
};

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%12,%13};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

__device__ __forceinline__ uint32_t lds32_g(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ int4 lds128_g(uint32_t a) {
  int4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

template <int MODE, class YT>
__global__ void __launch_bounds__(kMmaWarps * 32, 1) grouped_mma_q4k_kernel(const MmaParams p) {
  constexpr int NMAT = MODE == 1 ? 2 : 1;
  extern __shared__ __align__(128) uint8_t mma_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;  // fragment coordinates
  const int g   = blockIdx.y;
  const int beg = p.offs[g], n_g = p.offs[g + 1] - beg;
  if (n_g <= 0) return;

  // shared layout
  int8_t* xq    = reinterpret_cast<int8_t*>(mma_smem);                          // [NT][kMmaXPitch]
  float* dx     = reinterpret_cast<float*>(mma_smem + kMmaNT * kMmaXPitch);     // [64][NT]
  float* dxs    = dx + (kMmaKC / 32) * kMmaNT;                                  // [64][NT]
  size_t off    = kMmaNT * kMmaXPitch + 2 * (kMmaKC / 32) * kMmaNT * sizeof(float);
  uint64_t* bars = reinterpret_cast<uint64_t*>(mma_smem + off) + warp * kMmaStages;
  off += kMmaWarps * kMmaStages * 8;
  off = (off + 127) & ~size_t(127);
  constexpr int kStageBytes = NMAT * 16 * kMmaSegPad;
  uint8_t* ring = mma_smem + off + static_cast<size_t>(warp) * kMmaStages * kStageBytes;
  const uint32_t ring_u32 = smem_u32(ring), bar_u32 = smem_u32(bars), xq_u32 = smem_u32(xq);

  const int nsb = p.K / 256;                          // super-blocks per row
  const int nq  = (nsb + kMmaSB - 1) / kMmaSB;        // weight stages per row
  const int row_base = blockIdx.x * kMmaRows + warp * 16;
  // this lane's copy source: lanes 0-15 rows of matrix 0, lanes 16-31 rows of matrix 1
  const int my_mat = lane >> 4, my_r = lane & 15;
  const bool my_copy = my_mat < NMAT;
  const int src_row = min(row_base + my_r, p.N - 1);  // rows past the end re-read the last row
  const uint8_t* src = nullptr;
  if (my_copy)
    src = reinterpret_cast<const uint8_t*>((my_mat == 0 ? p.w0 : p.w1)[p.g_first + g]) +
          static_cast<size_t>(src_row) * p.row_bytes;

  int issued = 0, consumed = 0;
  auto issue = [&](int q) {  // whole warp
    const int s  = issued % kMmaStages;
    ++issued;
    const int sb0 = q * kMmaSB;
    const uint32_t bytes = static_cast<uint32_t>(min(kMmaSB, nsb - sb0)) * 144u;
    const uint32_t bar = bar_u32 + s * 8;
    if (lane == 0) mbar_expect_tx(bar, bytes * 16u * NMAT);
    __syncwarp();
    if (my_copy)
      bulk_g2s(ring_u32 + s * kStageBytes + (my_mat * 16 + my_r) * kMmaSegPad,
               src + static_cast<size_t>(sb0) * 144, bytes, bar);
  };

  if (lane == 0) {
    for (int s = 0; s < kMmaStages; ++s) mbar_init(bar_u32 + s * 8, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncwarp();

  for (int t0 = 0; t0 < n_g; t0 += kMmaNT) {
    const int nt = min(kMmaNT, n_g - t0);
    float acc[NMAT][2][4];
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][t][i] = 0.f;

    for (int q = 0; q < kMmaStages && q < nq; ++q) issue(q);

    for (int k0 = 0; k0 < p.K; k0 += kMmaKC) {
      const int kc = min(kMmaKC, p.K - k0);
      __syncthreads();  // the previous chunk's readers are done
      // ---- stage the activation chunk: int8 rows + per-block scales ----
      for (int f = threadIdx.x; f < kMmaNT * (kc / 16); f += blockDim.x) {
        const int t = f / (kc / 16), c16 = f - t * (kc / 16);
        int4 v = make_int4(0, 0, 0, 0);
        if (t < nt) {
          const int srow = MODE == 0 ? beg + t0 + t : p.list[beg + t0 + t] / p.S;
          v = __ldg(reinterpret_cast<const int4*>(p.xrows + static_cast<size_t>(srow) * p.x_pitch + k0) + c16);
        }
        *reinterpret_cast<int4*>(xq + t * kMmaXPitch + c16 * 16) = v;
      }
      for (int f = threadIdx.x; f < kMmaNT * (kc / 32); f += blockDim.x) {
        const int b = f / kMmaNT, t = f - b * kMmaNT;
        float d = 0.f, ds = 0.f;
        if (t < nt) {
          const int srow = MODE == 0 ? beg + t0 + t : p.list[beg + t0 + t] / p.S;
          const int4 h = __ldg(reinterpret_cast<const int4*>(p.xrows + static_cast<size_t>(srow) * p.x_pitch +
                                                              act_hdr_offset(p.K)) + (k0 / 32 + b));
          d  = __int_as_float(h.x);
          ds = __fmul_rn(static_cast<float>(h.y + h.z), d);
        }
        dx[b * kMmaNT + t]  = d;
        dxs[b * kMmaNT + t] = ds;
      }
      __syncthreads();

      // ---- consume the weight stages that cover this chunk ----
      const int q_first = k0 / (256 * kMmaSB), q_last = min(nq, (k0 + kc) / (256 * kMmaSB) + ((k0 + kc) % (256 * kMmaSB) ? 1 : 0));
      for (int q = q_first; q < q_last; ++q) {
        const int s = consumed % kMmaStages;
        if (!mbar_wait_bounded(bar_u32 + s * 8, (consumed / kMmaStages) & 1)) {
          if (lane == 0) atomicExch(p.status, KDNN_ERR_DEVICE_WAIT);
          return;
        }
        ++consumed;
        const uint32_t st = ring_u32 + s * kStageBytes;
        const int nsb_here = min(kMmaSB, nsb - q * kMmaSB);
        for (int sbi = 0; sbi < nsb_here; ++sbi) {
          const int blk0 = ((q * kMmaSB + sbi) * 256 - k0) / 32;  // first 32-block of this super-block in the chunk
          // headers of this lane's two rows, per matrix
          int4 hdr[NMAT][2];
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            hdr[m][0] = lds128_g(st + (m * 16 + gid) * kMmaSegPad + sbi * 144);
            hdr[m][1] = lds128_g(st + (m * 16 + gid + 8) * kMmaSegPad + sbi * 144);
          }
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            // packed words: rows gid / gid+8, byte offsets 4*tig and 16 + 4*tig of the 32-byte group
            uint32_t wlo[NMAT][2], whi[NMAT][2];
            float sw[NMAT][2][2], mw[NMAT][2][2];  // [mat][row half][sub-block parity]
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const uint32_t a = st + (m * 16 + gid + 8 * h) * kMmaSegPad + sbi * 144 + 16 + it * 32 + 4 * tig;
                wlo[m][h] = lds32_g(a);
                whi[m][h] = lds32_g(a + 16);
                uint32_t scp, mnp;
                q4k_scale_pair(hdr[m][h].y, hdr[m][h].z, hdr[m][h].w, it, scp, mnp);
                const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr[m][h].x));
                sw[m][h][0] = dd.x * static_cast<float>(scp & 0xFF);
                sw[m][h][1] = dd.x * static_cast<float>(scp >> 8);
                mw[m][h][0] = dd.y * static_cast<float>(mnp & 0xFF);
                mw[m][h][1] = dd.y * static_cast<float>(mnp >> 8);
              }
#pragma unroll
            for (int par = 0; par < 2; ++par) {  // sub-block 2*it + par: low / high nibbles
              const int blk = blk0 + 2 * it + par;
              uint32_t a[NMAT][4];
#pragma unroll
              for (int m = 0; m < NMAT; ++m) {
                a[m][0] = (wlo[m][0] >> (4 * par)) & 0x0F0F0F0Fu;
                a[m][1] = (wlo[m][1] >> (4 * par)) & 0x0F0F0F0Fu;
                a[m][2] = (whi[m][0] >> (4 * par)) & 0x0F0F0F0Fu;
                a[m][3] = (whi[m][1] >> (4 * par)) & 0x0F0F0F0Fu;
              }
#pragma unroll
              for (int t = 0; t < 2; ++t) {  // n8 tiles: tokens 8t .. 8t+7
                const uint32_t xa = xq_u32 + (8 * t + gid) * kMmaXPitch + blk * 32 + 4 * tig;
                const uint32_t b0 = lds32_g(xa), b1 = lds32_g(xa + 16);
                const float2 dxv  = *reinterpret_cast<const float2*>(dx + blk * kMmaNT + 8 * t + 2 * tig);
                const float2 dsv  = *reinterpret_cast<const float2*>(dxs + blk * kMmaNT + 8 * t + 2 * tig);
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                  int c[4];
                  mma_s8(c, a[m], b0, b1);
                  // c0,c1: row gid, tokens 2*tig, 2*tig+1; c2,c3: row gid+8
                  acc[m][t][0] += sw[m][0][par] * (static_cast<float>(c[0]) * dxv.x) - mw[m][0][par] * dsv.x;
                  acc[m][t][1] += sw[m][0][par] * (static_cast<float>(c[1]) * dxv.y) - mw[m][0][par] * dsv.y;
                  acc[m][t][2] += sw[m][1][par] * (static_cast<float>(c[2]) * dxv.x) - mw[m][1][par] * dsv.x;
                  acc[m][t][3] += sw[m][1][par] * (static_cast<float>(c[3]) * dxv.y) - mw[m][1][par] * dsv.y;
                }
              }
            }
          }
        }
        __syncwarp();  // every lane has read this stage
        const int qn = q + kMmaStages;
        if (qn < nq) issue(qn);
      }
    }

    // ---- epilogue ----
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tok = 8 * t + 2 * tig + (i & 1);
        const int j   = row_base + gid + 8 * (i >> 1);
        if (tok < nt && j < p.N) {
          float v = acc[0][t][i];
          if (MODE == 1) {
            const float u = acc[NMAT - 1][t][i];
            v = (v / (1.0f + expf(-v))) * u;
            if (p.round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
          }
          if (MODE == 2) {
            const int srow = p.list[beg + t0 + tok] / p.S;
            store_scalar(static_cast<YT*>(p.dst) + static_cast<size_t>(srow) * p.ld_dst + j, v);
          } else {
            static_cast<float*>(p.dst)[static_cast<size_t>(beg + t0 + tok) * p.N + j] = v;
          }
        }
      }
  }
}

template <int MODE>
constexpr size_t mma_smem_bytes() {
  size_t off = kMmaNT * kMmaXPitch + 2 * (kMmaKC / 32) * kMmaNT * sizeof(float) + kMmaWarps * kMmaStages * 8;
  off        = (off + 127) & ~size_t(127);
  return off + static_cast<size_t>(kMmaWarps) * kMmaStages * (MODE == 1 ? 2 : 1) * 16 * kMmaSegPad + 128;
}

template <int MODE, class YT>
static cudaError_t launch_grouped_mma(const MmaParams& p, int groups, cudaStream_t st) {
  auto kern = grouped_mma_q4k_kernel<MODE, YT>;
  constexpr size_t smem = mma_smem_bytes<MODE>();
  static thread_local bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid((p.N + kMmaRows - 1) / kMmaRows, groups);
  kern<<<grid, kMmaWarps * 32, smem, st>>>(p);
  return cudaGetLastError();
}

// Batched form of the reference's stage-1 quantizer: row r of `src` (pitch ld
// elements) -> reference staging layout at dst + r * pitch_bytes. Rows at or past
// *nrows_dev (when given) are skipped.
template <class SRC>
__global__ void quantize_rows_kernel(const SRC* __restrict__ src, size_t ld, int nrows, int K,
                                     const int* __restrict__ nrows_dev, uint8_t* __restrict__ dst,
                                     size_t pitch_bytes) {
  const int row = blockIdx.y;
  if (row >= nrows || (nrows_dev && row >= *nrows_dev)) return;
  const int nblk    = K / 32;
  const int lane    = threadIdx.x & 31, l4 = lane & 3;
  const SRC* x      = src + static_cast<size_t>(row) * ld;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  uint8_t* out      = dst + static_cast<size_t>(row) * pitch_bytes;
  ActHdr* gh        = reinterpret_cast<ActHdr*>(out + act_hdr_offset(K));
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
    if (l4 == 0) gh[b] = ActHdr{d, part, total - part, 0};
  }
}

template <class SRC>
static cudaError_t launch_quantize_rows(const SRC* src, size_t ld, int nrows, int K, const int* nrows_dev,
                                        uint8_t* dst, size_t pitch_bytes, cudaStream_t st) {
  if (nrows <= 0) return cudaSuccess;
  const int bx = max(1, min(8, (K / 32 + 63) / 64));
  quantize_rows_kernel<SRC><<<dim3(bx, nrows), 256, 0, st>>>(src, ld, nrows, K, nrows_dev, dst, pitch_bytes);
  return cudaGetLastError();
}

inline size_t act_row_pitch(size_t K) { return (act_bytes(K) + 255) & ~size_t(255); }

}  // namespace kdnn
