// Packed GGUF rows -> dense Scalar matrix, for sm_100a:
//   Y[r, k] = Scalar(dequant(W[r, k]))
// the operator the reference's batched MoE and prefill paths stage their GEMMs
// through (src/KokkosDNN_GGUF.hpp:2637-2934, block formulas :300-384).
//
// HBM-bound on the dense side (4 or 2 bytes written per 0.56-1.06 bytes read). A warp
// converts 256 consecutive elements of one row per step (one K-quant super-block, or
// eight Q8_0 blocks): lane l produces elements 8l .. 8l+7, so a warp's stores are one
// contiguous 1 KB (fp32) or 512 B (bf16) run. Every expression is evaluated with the
// reference's association and without fused multiply-add, so fp32 outputs are
// bit-identical to it.
#include "kdnn_common.cuh"

namespace kdnn {

// 6-bit (scale, min) of sub-block j from the 12 scale bytes (ggml get_scale_min_k4,
// src/KokkosDNN_GGUF.hpp:286-296).
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int& sc, int& mn) {
  if (j < 4) {
    sc = q[j] & 63;
    mn = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

template <uint32_t DT>
__device__ __forceinline__ void dequant8(const uint8_t* __restrict__ blk, int l, float (&v)[8]) {
  if (DT == KDNN_GGML_Q8_0) {
    // blk: first of eight 34-byte blocks; lane l -> block l / 4, elements 8 * (l % 4) ..
    const uint8_t* b = blk + (l >> 2) * 34;
    const float d    = h2f(static_cast<uint32_t>(b[0]) | (static_cast<uint32_t>(b[1]) << 8));
    const int8_t* q  = reinterpret_cast<const int8_t*>(b + 2 + (l & 3) * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(d, static_cast<float>(q[i]));
  } else if (DT == KDNN_GGML_Q4_K || DT == KDNN_GGML_Q5_K) {
    const int j = l >> 2, o = (l & 3) * 8;   // sub-block, offset inside it
    const float d  = h2f(static_cast<uint32_t>(blk[0]) | (static_cast<uint32_t>(blk[1]) << 8));
    const float dm = h2f(static_cast<uint32_t>(blk[2]) | (static_cast<uint32_t>(blk[3]) << 8));
    int sc, mn;
    scale_min_k4(j, blk + 4, sc, mn);
    const float d1 = __fmul_rn(d, static_cast<float>(sc));
    const int sh   = (j & 1) * 4;
    if (DT == KDNN_GGML_Q4_K) {
      const float o1   = __fmul_rn(-dm, static_cast<float>(mn));
      const uint8_t* q = blk + 16 + 32 * (j >> 1) + o;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __fadd_rn(__fmul_rn(d1, static_cast<float>((q[i] >> sh) & 0xF)), o1);
    } else {
      const float o1    = __fmul_rn(dm, static_cast<float>(mn));
      const uint8_t* qh = blk + 16 + o;
      const uint8_t* q  = blk + 48 + 32 * (j >> 1) + o;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int hi = (qh[i] >> j) & 1;
        v[i] = __fsub_rn(__fmul_rn(d1, static_cast<float>(((q[i] >> sh) & 0xF) + 16 * hi)), o1);
      }
    }
  } else {  // Q6_K
    const int e = 8 * l, n = e >> 7, g = (e >> 5) & 3, lp = e & 31;   // half, quarter, offset in the quarter
    const float d     = h2f(static_cast<uint32_t>(blk[208]) | (static_cast<uint32_t>(blk[209]) << 8));
    const uint8_t* ql = blk + 64 * n + (g & 1) * 32 + lp;
    const uint8_t* qh = blk + 128 + 32 * n + lp;
    const int8_t sc   = reinterpret_cast<const int8_t*>(blk + 192)[8 * n + (lp >> 4) + 2 * g];
    const float ds    = __fmul_rn(d, static_cast<float>(sc));
    const int lsh = (g >> 1) * 4, hsh = 2 * g;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = static_cast<int>(((ql[i] >> lsh) & 0xF) | (((qh[i] >> hsh) & 3) << 4)) - 32;
      v[i] = __fmul_rn(ds, static_cast<float>(q));
    }
  }
}

template <uint32_t DT, class YT>
__global__ void dequant_to_dense_kernel(const uint8_t* __restrict__ w, size_t row_bytes, int rows, int cols,
                                        YT* __restrict__ y, size_t ldy) {
  constexpr int kGroupBytes = DT == KDNN_GGML_Q4_K ? 144 : DT == KDNN_GGML_Q5_K ? 176 : DT == KDNN_GGML_Q6_K ? 210 : 8 * 34;
  const int lane   = threadIdx.x & 31;
  const int groups = (cols + 255) / 256;                  // 256-element groups per row
  const long long total = static_cast<long long>(rows) * groups;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarp = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long u = warp0; u < total; u += nwarp) {
    const int r = static_cast<int>(u / groups), gi = static_cast<int>(u - static_cast<long long>(r) * groups);
    const int k = gi * 256 + 8 * lane;
    if (k >= cols) continue;                              // Q8_0 rows that are not a multiple of 256
    float v[8];
    dequant8<DT>(w + static_cast<size_t>(r) * row_bytes + static_cast<size_t>(gi) * kGroupBytes, lane, v);
    YT* dst = y + static_cast<size_t>(r) * ldy + k;
    if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      if (sizeof(YT) == 4) {
        reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
      } else {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(h);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) store_scalar(dst + i, v[i]);
    }
  }
}

template <uint32_t DT>
static cudaError_t dequant_dt(const uint8_t* w, size_t rb, int rows, int cols, void* y, size_t ldy, int ys,
                              cudaStream_t st) {
  const long long warps = static_cast<long long>(rows) * ((cols + 255) / 256);
  static thread_local int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const long long want = (warps + 7) / 8;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > static_cast<long long>(sms) * 16 ? sms * 16 : want));
  if (ys == KDNN_F32)
    dequant_to_dense_kernel<DT, float><<<blocks, 256, 0, st>>>(w, rb, rows, cols, static_cast<float*>(y), ldy);
  else
    dequant_to_dense_kernel<DT, __nv_bfloat16><<<blocks, 256, 0, st>>>(w, rb, rows, cols, static_cast<__nv_bfloat16*>(y), ldy);
  return cudaGetLastError();
}

// ---- fp-path GEMV ------------------------------------------------------------------------
// y[r] = Scalar(sum_k dequant(W[r, k]) * float(x[k])), fp32 accumulation: the operator behind
// Gguf::quant_gemv(handle, x, w, y) without a staging buffer (src/KokkosDNN_GGUF.hpp:2394-2493),
// which is also where a declined int8 call lands. The activation row sits in shared memory as
// fp32 (in pieces of kFpChunk elements), a warp owns one row at a time and converts 256 weights
// per step with the dequantizer above, so the weights are exactly the reference's dequantized
// values and only the order of the fp32 additions differs from its FMA chains.
constexpr int kFpChunk = 8192;   // activation elements resident per pass (32 KB)

template <uint32_t DT, class XT, class YT>
__global__ void __launch_bounds__(256) gemv_fp_kernel(const uint8_t* __restrict__ w, size_t row_bytes, int rows,
                                                       int cols, const XT* __restrict__ x, YT* __restrict__ y) {
  constexpr int kGroupBytes = DT == KDNN_GGML_Q4_K ? 144 : DT == KDNN_GGML_Q5_K ? 176 : DT == KDNN_GGML_Q6_K ? 210 : 8 * 34;
  __shared__ float xs[kFpChunk];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int rows_per_cta = (rows + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  // rows of this CTA are spread over its warps; partial sums over the chunks stay in registers
  // (at most kMaxRowsPerWarp rows per warp, the host sizes the grid accordingly)
  constexpr int kMaxRowsPerWarp = 8;
  float acc[kMaxRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kMaxRowsPerWarp; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 < cols; k0 += kFpChunk) {
    const int kc = min(kFpChunk, cols - k0);
    __syncthreads();
    for (int i = threadIdx.x; i < kc; i += blockDim.x) xs[i] = to_f32(x[k0 + i]);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kMaxRowsPerWarp; ++i) {
      const int r = r0 + warp + i * nwarp;
      if (r >= r1) break;
      const uint8_t* row = w + static_cast<size_t>(r) * row_bytes;
      float a = 0.f;
      for (int g = 0; g * 256 < kc; ++g) {
        const int k = g * 256 + 8 * lane;
        if (k >= kc) continue;   // Q8_0 rows that are not a multiple of 256
        float v[8];
        dequant8<DT>(row + static_cast<size_t>(k0 / 256 + g) * kGroupBytes, lane, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) a = fmaf(v[j], xs[k + j], a);
      }
      acc[i] += a;
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxRowsPerWarp; ++i) {
    const int r = r0 + warp + i * nwarp;
    if (r >= r1) break;
    const float v = warp_sum(acc[i]);
    if (lane == 0) store_scalar(y + r, v);
  }
}

template <uint32_t DT>
static cudaError_t gemv_fp_dt(const uint8_t* w, size_t rb, int rows, int cols, const void* x, int xs, void* y, int ys,
                              cudaStream_t st) {
  // 8 warps per CTA, at most 8 rows per warp: 64 rows per CTA at most
  const int grid = max(max(1, (rows + 63) / 64), min((rows + 7) / 8, 4 * 148));
  if (xs == KDNN_F32 && ys == KDNN_F32)
    gemv_fp_kernel<DT, float, float><<<grid, 256, 0, st>>>(w, rb, rows, cols, static_cast<const float*>(x), static_cast<float*>(y));
  else if (xs == KDNN_BF16 && ys == KDNN_BF16)
    gemv_fp_kernel<DT, __nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(w, rb, rows, cols, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y));
  else if (xs == KDNN_BF16)
    gemv_fp_kernel<DT, __nv_bfloat16, float><<<grid, 256, 0, st>>>(w, rb, rows, cols, static_cast<const __nv_bfloat16*>(x), static_cast<float*>(y));
  else
    gemv_fp_kernel<DT, float, __nv_bfloat16><<<grid, 256, 0, st>>>(w, rb, rows, cols, static_cast<const float*>(x), static_cast<__nv_bfloat16*>(y));
  return cudaGetLastError();
}

cudaError_t gemv_fp_launch(uint32_t dt, const void* w, size_t rows, size_t cols, const void* x, int xs, void* y, int ys,
                           cudaStream_t st) {
  const uint8_t* wb = static_cast<const uint8_t*>(w);
  const size_t rb   = row_bytes_of(dt, cols);
  switch (dt) {
    case KDNN_GGML_Q4_K: return gemv_fp_dt<KDNN_GGML_Q4_K>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, st);
    case KDNN_GGML_Q5_K: return gemv_fp_dt<KDNN_GGML_Q5_K>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, st);
    case KDNN_GGML_Q6_K: return gemv_fp_dt<KDNN_GGML_Q6_K>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, st);
    default: return gemv_fp_dt<KDNN_GGML_Q8_0>(wb, rb, (int)rows, (int)cols, x, xs, y, ys, st);
  }
}

cudaError_t dequant_launch(uint32_t dt, const void* w, size_t rows, size_t cols, void* y, size_t ldy, int ys,
                           cudaStream_t st) {
  const uint8_t* wb = static_cast<const uint8_t*>(w);
  const size_t rb   = row_bytes_of(dt, cols);
  switch (dt) {
    case KDNN_GGML_Q4_K: return dequant_dt<KDNN_GGML_Q4_K>(wb, rb, (int)rows, (int)cols, y, ldy, ys, st);
    case KDNN_GGML_Q5_K: return dequant_dt<KDNN_GGML_Q5_K>(wb, rb, (int)rows, (int)cols, y, ldy, ys, st);
    case KDNN_GGML_Q6_K: return dequant_dt<KDNN_GGML_Q6_K>(wb, rb, (int)rows, (int)cols, y, ldy, ys, st);
    default: return dequant_dt<KDNN_GGML_Q8_0>(wb, rb, (int)rows, (int)cols, y, ldy, ys, st);
  }
}

}  // namespace kdnn
