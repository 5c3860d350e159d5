// Grouped int8 tile GEMM for Q4_K weights on the 5th-generation tensor cores:
// tcgen05.mma kind::i8 with the accumulators in tensor memory (TMEM).
//
// CTA = 128 threads = 128 weight rows of one group (the MMA's M; thread t owns row t
// and TMEM lane t) x a tile of 16 activation rows (the MMA's N).
// Per 256-element super-block of K:
//   1. the rows' packed bytes arrive in shared memory by bulk copies (one 144-byte copy
//      per row, issued by the row's thread, completion on an mbarrier);
//   2. every thread expands its row's nibbles to int8 and writes them into eight
//      128 x 32 operand tiles in the K-major, un-swizzled core-matrix layout the MMA
//      reads (8 rows x 16 bytes per core matrix), then fence.proxy.async;
//   3. one thread issues eight tcgen05.mma (one per 32-element sub-block, each into its
//      own 16-column TMEM slot, no accumulation across sub-blocks because every
//      sub-block has its own scales on both sides) and commits them to an mbarrier;
//   4. every thread reads its TMEM lane back (tcgen05.ld 32x32b.x16 per slot) and folds
//      acc[n] += (d*sc) * dx[n] * D[n] - (dmin*mn) * dx[n] * sum[n] in fp32 registers.
// The integer sub-block dots are exact, as on the dp4a and mma.sync paths.
//
// Every wait is bounded: a wait that gives up records KDNN_ERR_DEVICE_WAIT in the
// status word and execution continues to the common exit, where the TMEM columns are
// freed (results of that launch are then garbage, the GPU is not left hanging).
#pragma once

#include "kdnn_mma.cuh"

namespace kdnn {

constexpr int kUmmaRows   = 128;
constexpr int kUmmaNT     = 16;
constexpr int kUmmaKC     = 2048;                 // activation elements staged per chunk
constexpr int kUmmaATile  = 128 * 32;             // bytes of one sub-block operand tile
constexpr int kUmmaBTile  = kUmmaNT * 32;         // 512
constexpr int kUmmaPacked = 128 * 144;            // one super-block of packed rows
constexpr uint32_t kUmmaCols = 128;               // TMEM columns: 8 slots x 16

// shared-memory matrix descriptor: K-major, no swizzle, 8x16-byte core matrices,
// LBO (next 16 bytes of K) = 128 B, SBO (next 8 rows) = 256 B, descriptor version 1
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>(128u >> 4) << 16;
  d |= static_cast<uint64_t>(256u >> 4) << 32;
  d |= static_cast<uint64_t>(1u) << 46;
  return d;
}
// instruction descriptor: D = S32, A = B = signed 8-bit, both K-major, N = 16, M = 128
constexpr uint32_t kUmmaIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((kUmmaNT >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kUmmaIdesc), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <int MODE, class YT>
__global__ void __launch_bounds__(kUmmaRows, 1) grouped_umma_q4k_kernel(const MmaParams p) {
  constexpr int NMAT = MODE == 1 ? 2 : 1;
  extern __shared__ __align__(1024) uint8_t umma_smem[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ __align__(8) uint64_t bars[3];  // [0],[1]: packed buffers; [2]: MMA completion
  const int tid = threadIdx.x, warp = tid >> 5;
  const int g   = blockIdx.y;
  const int beg = p.offs[g], n_g = p.offs[g + 1] - beg;
  if (n_g <= 0) return;  // uniform for the CTA, before any allocation

  uint8_t* a_tiles = umma_smem;                                   // 8 x 4 KB
  uint8_t* b_tiles = a_tiles + 8 * kUmmaATile;                    // 64 x 512 B
  float* dx        = reinterpret_cast<float*>(b_tiles + (kUmmaKC / 32) * kUmmaBTile);  // [64][16]
  float* dxs       = dx + (kUmmaKC / 32) * kUmmaNT;
  uint8_t* packed  = reinterpret_cast<uint8_t*>(dxs + (kUmmaKC / 32) * kUmmaNT);       // 2 x 18 KB
  const uint32_t a_u32 = smem_u32(a_tiles), b_u32 = smem_u32(b_tiles), pk_u32 = smem_u32(packed);
  const uint32_t bar_u32 = smem_u32(bars);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kUmmaCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    mbar_init(bar_u32, 1);
    mbar_init(bar_u32 + 8, 1);
    mbar_init(bar_u32 + 16, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t my_taddr  = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

  const int nsb     = p.K / 256;
  const int row     = blockIdx.x * kUmmaRows + tid;
  const int src_row = min(row, p.N - 1);  // rows past the end re-read the last row
  const uint8_t* src0 =
      reinterpret_cast<const uint8_t*>(p.w0[p.g_first + g]) + static_cast<size_t>(src_row) * p.row_bytes;
  const uint8_t* src1 = NMAT == 2 ? reinterpret_cast<const uint8_t*>(p.w1[p.g_first + g]) +
                                        static_cast<size_t>(src_row) * p.row_bytes
                                  : src0;

  uint32_t pk_uses0 = 0, pk_uses1 = 0, mma_uses = 0;
  bool failed = false;
  // job j: MODE 1 -> (super-block j / 2, matrix j % 2); else (super-block j, matrix 0); buffer j & 1
  auto issue_job = [&](int j, int njobs) {
    if (j >= njobs) return;
    const int sb = NMAT == 2 ? j >> 1 : j, mat = NMAT == 2 ? j & 1 : 0;
    const uint32_t bar = bar_u32 + (j & 1) * 8;
    if (tid == 0) mbar_expect_tx(bar, kUmmaPacked);
    __syncthreads();  // the expectation is posted before any copy can complete
    bulk_g2s(pk_u32 + (j & 1) * kUmmaPacked + tid * 144, (mat ? src1 : src0) + static_cast<size_t>(sb) * 144, 144, bar);
  };

  for (int t0 = 0; t0 < n_g; t0 += kUmmaNT) {
    const int nt = min(kUmmaNT, n_g - t0);
    float acc[NMAT][kUmmaNT];
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int n = 0; n < kUmmaNT; ++n) acc[m][n] = 0.f;
    const int njobs = nsb * NMAT;
    issue_job(0, njobs);
    issue_job(1, njobs);

    for (int j0 = 0; j0 < njobs; j0 += NMAT) {
#pragma unroll
     for (int mat = 0; mat < NMAT; ++mat) {   // matrix index is a compile-time constant (register accumulators)
      const int j  = j0 + mat;
      const int sb = NMAT == 2 ? j >> 1 : j;
      const int k0 = (sb * 256 / kUmmaKC) * kUmmaKC;   // activation chunk of this super-block
      if (sb * 256 == k0 && mat == 0) {
        // ---- stage the activation chunk in the MMA's B layout, plus the block scales ----
        const int kc = min(kUmmaKC, p.K - k0);
        __syncthreads();  // nobody still reads the previous chunk's scales
        for (int f = tid; f < kUmmaNT * (kc / 16); f += kUmmaRows) {
          const int n = f / (kc / 16), c16 = f - n * (kc / 16);
          int4 v = make_int4(0, 0, 0, 0);
          if (n < nt) {
            const int srow = MODE == 0 ? beg + t0 + n : p.list[beg + t0 + n] / p.S;
            v = __ldg(reinterpret_cast<const int4*>(p.xrows + static_cast<size_t>(srow) * p.x_pitch + k0) + c16);
          }
          const int b = c16 >> 1, half = c16 & 1;
          *reinterpret_cast<int4*>(b_tiles + b * kUmmaBTile + (n >> 3) * 256 + half * 128 + (n & 7) * 16) = v;
        }
        for (int f = tid; f < kUmmaNT * (kc / 32); f += kUmmaRows) {
          const int b = f / kUmmaNT, n = f - b * kUmmaNT;
          float d = 0.f, ds = 0.f;
          if (n < nt) {
            const int srow = MODE == 0 ? beg + t0 + n : p.list[beg + t0 + n] / p.S;
            const int4 h = __ldg(reinterpret_cast<const int4*>(p.xrows + static_cast<size_t>(srow) * p.x_pitch +
                                                                act_hdr_offset(p.K)) + (k0 / 32 + b));
            d  = __int_as_float(h.x);
            ds = __fmul_rn(static_cast<float>(h.y + h.z), d);
          }
          dx[b * kUmmaNT + n]  = d;
          dxs[b * kUmmaNT + n] = ds;
        }
        // visibility to the MMA (async proxy) is established by the fence before the MMA below
      }
      // ---- packed rows of this job ----
      const int buf = j & 1;
      if (!mbar_wait_bounded(bar_u32 + buf * 8, (buf ? pk_uses1 : pk_uses0) & 1u)) failed = true;
      if (buf) ++pk_uses1; else ++pk_uses0;
      const uint32_t mine = pk_u32 + buf * kUmmaPacked + tid * 144;
      const int4 hdr = lds128_g(mine);
      const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
      float sw[8], mw[8];
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        uint32_t scp, mnp;
        q4k_scale_pair(hdr.y, hdr.z, hdr.w, it, scp, mnp);
        sw[2 * it]     = dd.x * static_cast<float>(scp & 0xFF);
        sw[2 * it + 1] = dd.x * static_cast<float>(scp >> 8);
        mw[2 * it]     = dd.y * static_cast<float>(mnp & 0xFF);
        mw[2 * it + 1] = dd.y * static_cast<float>(mnp >> 8);
        const int4 qa = lds128_g(mine + 16 + it * 32), qb = lds128_g(mine + 32 + it * 32);
        const uint32_t q[8] = {(uint32_t)qa.x, (uint32_t)qa.y, (uint32_t)qa.z, (uint32_t)qa.w,
                               (uint32_t)qb.x, (uint32_t)qb.y, (uint32_t)qb.z, (uint32_t)qb.w};
        // sub-block 2*it: low nibbles, 2*it+1: high nibbles; K bytes 0-15 then 16-31
        const uint32_t base = (tid >> 3) * 256 + (tid & 7) * 16;
        int4 lo0 = make_int4(q[0] & 0x0F0F0F0Fu, q[1] & 0x0F0F0F0Fu, q[2] & 0x0F0F0F0Fu, q[3] & 0x0F0F0F0Fu);
        int4 lo1 = make_int4(q[4] & 0x0F0F0F0Fu, q[5] & 0x0F0F0F0Fu, q[6] & 0x0F0F0F0Fu, q[7] & 0x0F0F0F0Fu);
        int4 hi0 = make_int4((q[0] >> 4) & 0x0F0F0F0Fu, (q[1] >> 4) & 0x0F0F0F0Fu, (q[2] >> 4) & 0x0F0F0F0Fu,
                             (q[3] >> 4) & 0x0F0F0F0Fu);
        int4 hi1 = make_int4((q[4] >> 4) & 0x0F0F0F0Fu, (q[5] >> 4) & 0x0F0F0F0Fu, (q[6] >> 4) & 0x0F0F0F0Fu,
                             (q[7] >> 4) & 0x0F0F0F0Fu);
        *reinterpret_cast<int4*>(a_tiles + (2 * it) * kUmmaATile + base)           = lo0;
        *reinterpret_cast<int4*>(a_tiles + (2 * it) * kUmmaATile + base + 128)     = lo1;
        *reinterpret_cast<int4*>(a_tiles + (2 * it + 1) * kUmmaATile + base)       = hi0;
        *reinterpret_cast<int4*>(a_tiles + (2 * it + 1) * kUmmaATile + base + 128) = hi1;
      }
      fence_proxy_async();  // generic-proxy writes (A tiles, B tiles) -> async-proxy reads by the MMA
      tc_fence_before();
      __syncthreads();       // operands complete; every thread has finished reading this packed buffer
      issue_job(j + 2, njobs);  // refill the buffer just consumed (contains a __syncthreads)
      // ---- eight MMAs, one per sub-block, each into its own TMEM slot ----
      if (tid == 0) {
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          const int blk = (sb * 256 - k0) / 32 + s;
          umma_i8(tmem_base + s * kUmmaNT, umma_desc(a_u32 + s * kUmmaATile), umma_desc(b_u32 + blk * kUmmaBTile));
        }
        umma_commit(bar_u32 + 16);
      }
      if (!mbar_wait_bounded(bar_u32 + 16, mma_uses & 1u)) failed = true;
      ++mma_uses;
      tc_fence_after();
      // ---- fold this thread's row ----
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        int d[16];
        tmem_ld16(my_taddr + s * kUmmaNT, d);
        tmem_wait_ld();
        const int blk = (sb * 256 - k0) / 32 + s;
        const float4* dxp = reinterpret_cast<const float4*>(dx + blk * kUmmaNT);
        const float4* dsp = reinterpret_cast<const float4*>(dxs + blk * kUmmaNT);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float4 a = dxp[v], b = dsp[v];
          acc[mat][4 * v + 0] += sw[s] * (static_cast<float>(d[4 * v + 0]) * a.x) - mw[s] * b.x;
          acc[mat][4 * v + 1] += sw[s] * (static_cast<float>(d[4 * v + 1]) * a.y) - mw[s] * b.y;
          acc[mat][4 * v + 2] += sw[s] * (static_cast<float>(d[4 * v + 2]) * a.z) - mw[s] * b.z;
          acc[mat][4 * v + 3] += sw[s] * (static_cast<float>(d[4 * v + 3]) * a.w) - mw[s] * b.w;
        }
      }
      tc_fence_before();  // TMEM reads are ordered before the next job's MMAs (after its __syncthreads)
     }
    }

    // ---- epilogue ----
    if (row < p.N) {
#pragma unroll
      for (int n = 0; n < kUmmaNT; ++n) {
        if (n < nt) {
          float v = acc[0][n];
          if (MODE == 1) {
            v = (v / (1.0f + expf(-v))) * acc[NMAT - 1][n];
            if (p.round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
          }
          if (MODE == 2) {
            const int srow = p.list[beg + t0 + n] / p.S;
            store_scalar(static_cast<YT*>(p.dst) + static_cast<size_t>(srow) * p.ld_dst + row, v);
          } else {
            static_cast<float*>(p.dst)[static_cast<size_t>(beg + t0 + n) * p.N + row] = v;
          }
        }
      }
    }
  }
  if (failed) atomicExch(p.status, KDNN_ERR_DEVICE_WAIT);
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kUmmaCols) : "memory");
}

constexpr size_t umma_smem_bytes() {
  return 8 * kUmmaATile + (kUmmaKC / 32) * kUmmaBTile + 2 * (kUmmaKC / 32) * kUmmaNT * sizeof(float) +
         2 * kUmmaPacked + 1024;
}

template <int MODE, class YT>
static cudaError_t launch_grouped_umma(const MmaParams& p, int groups, cudaStream_t st) {
  auto kern = grouped_umma_q4k_kernel<MODE, YT>;
  constexpr size_t smem = umma_smem_bytes();
  static thread_local bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid((p.N + kUmmaRows - 1) / kUmmaRows, groups);
  kern<<<grid, kUmmaRows, smem, st>>>(p);
  return cudaGetLastError();
}

}  // namespace kdnn
