// Grouped int8 GEMM, lane-per-row dp4a form: for every group (expert) g and every
// activation row assigned to it, dst[pos, j] = W_g[j, :] . q(src row), with the
// activation row quantized per 32 elements while it is staged into shared memory.
// Used by the MoE feed-forward (kdnn_moe.cu) and by the batched GEMM (kdnn_gemm.cu).
#pragma once

#include "kdnn_tile.cuh"

namespace kdnn {

constexpr int kMT      = 16;   // activation rows per tile (accumulators per lane)
constexpr int kRowsCta = 128;  // weight rows per CTA (one per thread)
constexpr int kKChunk  = 32;   // items (64 elements each) staged per pass over K

struct GroupedParams {
  const uintptr_t* w0;   // per-group payload addresses (gate, down, or the one matrix)
  const uintptr_t* w1;   // up (MODE 1 only)
  int row_bytes0, row_bytes1;
  int N;                 // weight rows per group
  int K;                 // elements per row
  const int* offs;       // [groups + 1] positions
  const int* list;       // slot id at each position
  int S;                 // slots per token (source row of a slot = slot / S)
  int g_first;           // first group's index into w0 / w1
  const ActItem* src;    // quantized activation rows, K/64 items each:
                         // MODE 0 indexed by position, MODE 1, 2 by slot / S
  void* dst;             // MODE 0, 1: float [npos, N]; MODE 2: YT [rows, ld_dst] indexed by slot / S
  size_t ld_dst;
  int round_bf16;        // MODE 1: round the SwiGLU result to bf16 (Scalar = bf16)
};

// MODE 0: dst[pos, j]  = W0[j,:] . q(src[pos,:])                      (down projection)
// MODE 1: dst[pos, j]  = Scalar(silu(W0 . q(x)) * (W1 . q(x)))        (gate / up + SwiGLU)
// MODE 2: dst[row, j]  = YT(W0[j,:] . q(x[row,:]))                    (plain batched GEMM)
template <uint32_t DT, int MODE, class XT, class YT>
__global__ void __launch_bounds__(kRowsCta) grouped_gemm_kernel(const GroupedParams p) {
  extern __shared__ __align__(16) uint8_t grouped_smem[];
  ActItem* items = reinterpret_cast<ActItem*>(grouped_smem);  // [kMT][kKChunk]
  const int g    = blockIdx.y;
  const int beg = p.offs[g], n_g = p.offs[g + 1] - beg;
  if (n_g <= 0) return;
  const int j       = blockIdx.x * kRowsCta + threadIdx.x;
  const bool row_ok = j < p.N;
  const int jr      = row_ok ? j : p.N - 1;
  const uint8_t* r0 = reinterpret_cast<const uint8_t*>(p.w0[p.g_first + g]) +
                      static_cast<size_t>(jr) * p.row_bytes0;
  const uint8_t* r1 = MODE == 1 ? reinterpret_cast<const uint8_t*>(p.w1[p.g_first + g]) +
                                      static_cast<size_t>(jr) * p.row_bytes1
                                : nullptr;
  const int nitems = p.K / 64;
  for (int t0 = 0; t0 < n_g; t0 += kMT) {
    const int nt = min(kMT, n_g - t0);
    float acc0[kMT], acc1[kMT];
#pragma unroll
    for (int t = 0; t < kMT; ++t) acc0[t] = acc1[t] = 0.f;
    for (int c0 = 0; c0 < nitems; c0 += kKChunk) {
      const int ci = min(kKChunk, nitems - c0);
      __syncthreads();
      {  // copy the tile's ActItems (nt rows x ci items, six 16-byte words each)
        const int words = nt * ci * 6;
        for (int f = threadIdx.x; f < words; f += blockDim.x) {
          const int t = f / (ci * 6), r = f - t * (ci * 6);
          const int srow = MODE == 0 ? beg + t0 + t : p.list[beg + t0 + t] / p.S;
          const int4* from = reinterpret_cast<const int4*>(p.src + static_cast<size_t>(srow) * nitems + c0);
          reinterpret_cast<int4*>(items + t * kKChunk)[r] = __ldg(from + r);
        }
      }
      __syncthreads();
      for (int i = 0; i < ci; ++i) {
        WItem<DT> wa, wb;
        wa.load(r0, c0 + i);
        if (MODE == 1) wb.load(r1, c0 + i);
#pragma unroll
        for (int t = 0; t < kMT; ++t) {
          if (t < nt) {
            const ActItem a = lds_item(items + t * kKChunk + i);
            acc0[t] += wa.dot(a);
            if (MODE == 1) acc1[t] += wb.dot(a);
          }
        }
      }
    }
    if (row_ok) {
#pragma unroll
      for (int t = 0; t < kMT; ++t) {
        if (t < nt) {
          if (MODE == 2) {
            const int slot = p.list[beg + t0 + t];
            store_scalar(static_cast<YT*>(p.dst) + static_cast<size_t>(slot / p.S) * p.ld_dst + j, acc0[t]);
          } else {
            float v = acc0[t];
            if (MODE == 1) {
              v = (acc0[t] / (1.0f + expf(-acc0[t]))) * acc1[t];
              if (p.round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
            }
            static_cast<float*>(p.dst)[static_cast<size_t>(beg + t0 + t) * p.N + j] = v;
          }
        }
      }
    }
  }
}

// Quantizes activation rows per 32 elements into ActItem rows (K/64 items each) in
// the granule order format DT consumes. src row r is `src + r * ld`; rows beyond
// *nrows_dev (when given) are skipped, so the grid can be sized for the maximum.
template <uint32_t DT, class SRC>
__global__ void quantize_items_kernel(const SRC* __restrict__ src, size_t ld, int nrows, int K,
                                      const int* __restrict__ nrows_dev, ActItem* __restrict__ dst) {
  const int row = blockIdx.y;
  if (row >= nrows || (nrows_dev && row >= *nrows_dev)) return;
  const int nblk = K / 32, nitems = K / 64;
  const int lane = threadIdx.x & 31, l8 = lane & 7;
  const SRC* x   = src + static_cast<size_t>(row) * ld;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & (sizeof(SRC) * 4 - 1)) == 0;
  ActItem* out   = dst + static_cast<size_t>(row) * nitems;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarp = (gridDim.x * blockDim.x) >> 5;
  for (int base = gwarp * 4; base < nblk; base += nwarp * 4) {
    const int b      = base + (lane >> 3);
    const bool valid = b < nblk;
    float v[4]       = {0.f, 0.f, 0.f, 0.f};
    if (valid) load4<SRC>(x, static_cast<size_t>(b) * 32 + l8 * 4, vec_ok, v);
    float d;
    int part, total;
    const uint32_t packed = quantize_block_lane(v, d, part, total);
    if (!valid) continue;
    int item, g;
    granule_map<DT>(b, l8 >> 2, item, g);
    ActItem& a = out[item];
    reinterpret_cast<uint32_t*>(&a.g[g])[l8 & 3] = packed;
    if ((l8 & 3) == 0) {
      a.dx[g]  = d;
      a.sum[g] = part;
    }
  }
}

template <class SRC>
static cudaError_t launch_quantize_items(uint32_t dt, const SRC* src, size_t ld, int nrows, int K,
                                         const int* nrows_dev, ActItem* dst, cudaStream_t st) {
  if (nrows <= 0) return cudaSuccess;
  const int bx = max(1, min(8, (K / 32 + 31) / 32));
  dim3 grid(bx, nrows);
  switch (dt) {
    case KDNN_GGML_Q4_K:
    case KDNN_GGML_Q5_K:   // same item order as Q4_K
      quantize_items_kernel<KDNN_GGML_Q4_K, SRC><<<grid, 256, 0, st>>>(src, ld, nrows, K, nrows_dev, dst); break;
    case KDNN_GGML_Q6_K: quantize_items_kernel<KDNN_GGML_Q6_K, SRC><<<grid, 256, 0, st>>>(src, ld, nrows, K, nrows_dev, dst); break;
    default: quantize_items_kernel<KDNN_GGML_Q8_0, SRC><<<grid, 256, 0, st>>>(src, ld, nrows, K, nrows_dev, dst); break;
  }
  return cudaGetLastError();
}

template <uint32_t DT, int MODE, class XT, class YT>
static cudaError_t launch_grouped(const GroupedParams& p, int groups, cudaStream_t st) {
  const size_t smem = sizeof(ActItem) * kMT * kKChunk;  // 48 KB
  auto kern = grouped_gemm_kernel<DT, MODE, XT, YT>;
  static SmemAttrOnce once;
  const cudaError_t e = set_max_smem_once(once, kern, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid((p.N + kRowsCta - 1) / kRowsCta, groups);
  kern<<<grid, kRowsCta, smem, st>>>(p);
  return cudaGetLastError();
}

template <int MODE, class XT, class YT>
static cudaError_t launch_grouped_dt(uint32_t dt, const GroupedParams& p, int groups, cudaStream_t st) {
  switch (dt) {
    case KDNN_GGML_Q4_K: return launch_grouped<KDNN_GGML_Q4_K, MODE, XT, YT>(p, groups, st);
    case KDNN_GGML_Q5_K: return launch_grouped<KDNN_GGML_Q5_K, MODE, XT, YT>(p, groups, st);
    case KDNN_GGML_Q6_K: return launch_grouped<KDNN_GGML_Q6_K, MODE, XT, YT>(p, groups, st);
    default: return launch_grouped<KDNN_GGML_Q8_0, MODE, XT, YT>(p, groups, st);
  }
}

}  // namespace kdnn
