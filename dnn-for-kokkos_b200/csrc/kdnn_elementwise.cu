// The small MoE operators of the reference as stand-alone kernels, for callers that keep the structure of its
// per-expert loop (models/lfm2_5/KokkosDNN_LFM25Model.hpp:441-547): swiglu, the weighted sum over a token's
// expert outputs, row gather and weighted scatter-add. All are bound by memory traffic: 16-byte accesses
// where the rows allow it, one launch each, chained like every kernel of the library.
#include "kdnn_common.cuh"

namespace kdnn {

// out[t, f] = Scalar(silu(float(gate)) * float(up))   (src/KokkosDNN_SwiGLU.hpp:24-38)
template <class ST>
__global__ void swiglu_kernel(const ST* gate, size_t ldg, const ST* up, size_t ldu,
                              ST* out, size_t ldo, int T, int F) {
  pdl_chain_entry();
  const int t = blockIdx.y;
  for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < F; f += gridDim.x * blockDim.x) {
    const float g = to_f32(gate[static_cast<size_t>(t) * ldg + f]);
    const float v = (g / (1.0f + expf(-g))) * to_f32(up[static_cast<size_t>(t) * ldu + f]);
    store_scalar(out + static_cast<size_t>(t) * ldo + f, v);
  }
}

// y[t, d] = Scalar(sum_k w[t, k] * float(expert_out[t, k, d])), k ascending   (src/KokkosDNN_MoE.hpp:313-332)
template <class ST>
__global__ void weighted_sum_kernel(const ST* eo, const float* w, ST* y,
                                    size_t ldy, int T, int K, int D) {
  pdl_chain_entry();
  const int t = blockIdx.y;
  for (int d = blockIdx.x * blockDim.x + threadIdx.x; d < D; d += gridDim.x * blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) acc += w[static_cast<size_t>(t) * K + k] * to_f32(eo[(static_cast<size_t>(t) * K + k) * D + d]);
    store_scalar(y + static_cast<size_t>(t) * ldy + d, acc);
  }
}

// dst[n, :] = src[rows[n], :]   (src/KokkosDNN_MoE.hpp:337-351)
template <class ST>
__global__ void gather_rows_kernel(const ST* src, size_t lds, const int* rows,
                                   ST* dst, size_t ldd, int N, int D) {
  pdl_chain_entry();
  const int n = blockIdx.y;
  const ST* s = src + static_cast<size_t>(rows[n]) * lds;
  ST* o = dst + static_cast<size_t>(n) * ldd;
  const bool vec = ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(o)) & 15u) == 0;
  constexpr int per16 = 16 / sizeof(ST);
  const int nv = vec ? D / per16 : 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += gridDim.x * blockDim.x)
    reinterpret_cast<uint4*>(o)[i] = reinterpret_cast<const uint4*>(s)[i];
  for (int d = nv * per16 + blockIdx.x * blockDim.x + threadIdx.x; d < D; d += gridDim.x * blockDim.x) o[d] = s[d];
}

// dst[rows[n], d] = Scalar(float(dst[rows[n], d]) + w[n] * float(src[n, d])); rows unique per call, so no
// atomics (src/KokkosDNN_MoE.hpp:360-381)
template <class ST>
__global__ void scatter_add_kernel(const ST* src, size_t lds, const int* rows,
                                   const float* w, ST* dst, size_t ldd, int N, int D) {
  pdl_chain_entry();
  const int n = blockIdx.y;
  const float wn = w[n];
  ST* o = dst + static_cast<size_t>(rows[n]) * ldd;
  for (int d = blockIdx.x * blockDim.x + threadIdx.x; d < D; d += gridDim.x * blockDim.x)
    store_scalar(o + d, __fadd_rn(to_f32(o[d]), __fmul_rn(wn, to_f32(src[static_cast<size_t>(n) * lds + d]))));   // product and sum rounded separately, as written in the reference
}

// Read-only streaming probe: every 16 bytes of [src, src + bytes) are loaded once (grid-stride, 128-bit
// loads, eight in flight per thread) and folded into one word per thread, so the loads cannot be dropped.
// The counterpart of the reference benchmarks' ceiling kernels (benchmarks/Bench_GGUFGemv.cpp:65-81,
// benchmarks/Bench_MoeDecode.cpp:217-257): what a kernel that only READS packed weights can reach.
__global__ void __launch_bounds__(512) read_probe_kernel(const uint4* src, size_t n16, uint32_t* sink) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  uint32_t acc = 0;
  for (; i + 7 * stride < n16; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcs(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < 8; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  for (; i < n16; i += stride) {
    const uint4 v = __ldcs(src + i);
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  if (acc == 0x9E3779B9u) sink[0] = acc;   // practically never: keeps the loads observable
}
cudaError_t read_probe_launch(const void* src, size_t bytes, uint32_t* sink, int ctas, cudaStream_t st) {
  read_probe_kernel<<<ctas, 512, 0, st>>>(static_cast<const uint4*>(src), bytes / 16, sink);
  return cudaGetLastError();
}

static dim3 row_grid(size_t cols, size_t rows) {
  const unsigned bx = static_cast<unsigned>((cols + 1023) / 1024);
  return dim3(bx < 1 ? 1 : (bx > 32 ? 32 : bx), static_cast<unsigned>(rows));
}

cudaError_t swiglu_launch(const void* gate, size_t ldg, const void* up, size_t ldu, void* out, size_t ldo, size_t T,
                          size_t F, int scalar, cudaStream_t st) {
  if (scalar == KDNN_F32)
    return launch_chained(swiglu_kernel<float>, row_grid(F, T), dim3(256), 0, st, static_cast<const float*>(gate), ldg,
                          static_cast<const float*>(up), ldu, static_cast<float*>(out), ldo, (int)T, (int)F);
  return launch_chained(swiglu_kernel<__nv_bfloat16>, row_grid(F, T), dim3(256), 0, st,
                        static_cast<const __nv_bfloat16*>(gate), ldg, static_cast<const __nv_bfloat16*>(up), ldu,
                        static_cast<__nv_bfloat16*>(out), ldo, (int)T, (int)F);
}
cudaError_t weighted_sum_launch(const void* eo, const float* w, void* y, size_t ldy, size_t T, size_t K, size_t D,
                                int scalar, cudaStream_t st) {
  if (scalar == KDNN_F32)
    return launch_chained(weighted_sum_kernel<float>, row_grid(D, T), dim3(256), 0, st, static_cast<const float*>(eo), w,
                          static_cast<float*>(y), ldy, (int)T, (int)K, (int)D);
  return launch_chained(weighted_sum_kernel<__nv_bfloat16>, row_grid(D, T), dim3(256), 0, st,
                        static_cast<const __nv_bfloat16*>(eo), w, static_cast<__nv_bfloat16*>(y), ldy, (int)T, (int)K, (int)D);
}
cudaError_t gather_rows_launch(const void* src, size_t lds, const int* rows, void* dst, size_t ldd, size_t N, size_t D,
                               int scalar, cudaStream_t st) {
  if (scalar == KDNN_F32)
    return launch_chained(gather_rows_kernel<float>, row_grid(D / 4 + 1, N), dim3(256), 0, st, static_cast<const float*>(src),
                          lds, rows, static_cast<float*>(dst), ldd, (int)N, (int)D);
  return launch_chained(gather_rows_kernel<__nv_bfloat16>, row_grid(D / 8 + 1, N), dim3(256), 0, st,
                        static_cast<const __nv_bfloat16*>(src), lds, rows, static_cast<__nv_bfloat16*>(dst), ldd, (int)N, (int)D);
}
cudaError_t scatter_add_launch(const void* src, size_t lds, const int* rows, const float* w, void* dst, size_t ldd,
                               size_t N, size_t D, int scalar, cudaStream_t st) {
  if (scalar == KDNN_F32)
    return launch_chained(scatter_add_kernel<float>, row_grid(D, N), dim3(256), 0, st, static_cast<const float*>(src), lds,
                          rows, w, static_cast<float*>(dst), ldd, (int)N, (int)D);
  return launch_chained(scatter_add_kernel<__nv_bfloat16>, row_grid(D, N), dim3(256), 0, st,
                        static_cast<const __nv_bfloat16*>(src), lds, rows, w, static_cast<__nv_bfloat16*>(dst), ldd, (int)N, (int)D);
}

}  // namespace kdnn
