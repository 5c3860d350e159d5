// extern "C" entry points of libkdnn_b200.so (declared in include/kdnn_b200.h):
// argument validation with the reference's decline / throw split, then the
// kernel launchers of kdnn_gemv.cu, kdnn_gemm.cu and kdnn_moe.cu.
#include "kdnn_common.cuh"

#include <limits.h>
#include <stdio.h>
#include <string.h>
#include <string>

namespace kdnn {
cudaError_t gemv_launch(uint32_t dt, const void* w, size_t rows, size_t cols, const void* x, int xs,
                        void* y, int ys, void* scratch, const kdnn_b200_gemv_layout* layout, cudaStream_t stream);
cudaError_t gemv_multi_launch(uint32_t dt, int n, const void* const* w, size_t rows, size_t cols, const void* x, int xs,
                              void* const* y, int ys, void* scratch, const kdnn_b200_gemv_layout* layout,
                              cudaStream_t stream);
cudaError_t quantize_act_launch(const void* x, int xs, size_t K, void* scratch, cudaStream_t st);
cudaError_t unit_dots_launch(uint32_t dt, const void* w, size_t rows, size_t cols,
                             const void* scratch, int32_t* out, cudaStream_t st);
int gemv_take_status();

size_t gemm_workspace_bytes(size_t M, size_t K);
cudaError_t gemm_launch(uint32_t dt, const void* w, size_t N, size_t K, const void* X, size_t ldx,
                        size_t M, int xs, void* Y, size_t ldy, int ys, void* ws, int32_t* dots, cudaStream_t st);
int tile_kind();
int set_tile_kind(int k);
int device_sm_count();
cudaError_t read_probe_launch(const void* src, size_t bytes, uint32_t* sink, int ctas, cudaStream_t st);
cudaError_t swiglu_launch(const void* gate, size_t ldg, const void* up, size_t ldu, void* out, size_t ldo, size_t T,
                          size_t F, int scalar, cudaStream_t st);
cudaError_t weighted_sum_launch(const void* eo, const float* w, void* y, size_t ldy, size_t T, size_t K, size_t D,
                                int scalar, cudaStream_t st);
cudaError_t gather_rows_launch(const void* src, size_t lds, const int* rows, void* dst, size_t ldd, size_t N, size_t D,
                               int scalar, cudaStream_t st);
cudaError_t scatter_add_launch(const void* src, size_t lds, const int* rows, const float* w, void* dst, size_t ldd,
                               size_t N, size_t D, int scalar, cudaStream_t st);
size_t moe_exchange_bytes(size_t tokens_local, size_t world, size_t S, size_t H);
size_t moe_block_workspace_bytes(size_t tokens_local, size_t world, size_t S, size_t H, size_t F, size_t n_experts,
                                 int with_region);
cudaError_t moe_block_launch(const BlockArgs& a, cudaStream_t st);
void moe_block_routing(void* const* regions, int rank, void* ws, size_t Tl, size_t world, size_t S, size_t H, size_t F,
                       size_t E, const int32_t** idx, const float** wts);
cudaError_t tc_encode_matrix_host(void* out128, const void* w, size_t rows, size_t row_bytes);

cudaError_t moe_route_launch(const void* logits, size_t ld, size_t T, size_t E, int scalar,
                             const void* bias, int top_k, int norm_topk, float routed_scale,
                             int sigmoid, int32_t* top_idx, float* top_w, cudaStream_t st);
size_t moe_workspace_bytes(size_t T, size_t S, size_t H, size_t F, size_t n_experts);
cudaError_t moe_ffn_launch(const void* X, size_t ldx, size_t T, int xs,
                           const kdnn_b200_weight_table* gate, const kdnn_b200_weight_table* up,
                           const kdnn_b200_weight_table* down, const int32_t* idx, const float* wts,
                           size_t S, void* Y, size_t ldy, int ys, size_t e_first, size_t e_count,
                           void* ws, cudaStream_t st);
int moe_take_status();
cudaError_t gemv_fp_launch(uint32_t dt, const void* w, size_t rows, size_t cols, const void* x, int xs, void* y, int ys,
                           cudaStream_t st);
cudaError_t dequant_launch(uint32_t dt, const void* w, size_t rows, size_t cols, void* y, size_t ldy, int ys,
                           cudaStream_t st);
cudaError_t residual_rmsnorm_launch(const void* h, size_t ldh, const float* y, size_t ldy, void* out,
                                    size_t ldo, size_t T, size_t H, float eps, int scalar, cudaStream_t st);
}  // namespace kdnn

namespace {
thread_local std::string g_last_error;
}  // namespace
namespace kdnn {
void set_last_error(const char* msg) { g_last_error = msg; }
}  // namespace kdnn
namespace {

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}
int cuda_result(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return KDNN_OK;
  return fail(KDNN_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
bool scalar_ok(int s) { return s == KDNN_F32 || s == KDNN_BF16; }
bool int8_type(uint32_t t) {
  return t == KDNN_GGML_Q4_K || t == KDNN_GGML_Q5_K || t == KDNN_GGML_Q6_K || t == KDNN_GGML_Q8_0;
}
bool tile_type(uint32_t t) { return int8_type(t); }
// Copies between page-locked host memory and device memory done by a kernel over the mapped host
// pointer instead of by the copy engine: on a stream that alternates small copies and short kernels the
// engine hand-offs cost more than the kernels. Chained like every other kernel of the library, so the GEMV
// that follows a pull prefetches its weights while the pull is in flight.
__global__ void copy_bytes_kernel(const uint8_t* src, uint8_t* dst, size_t bytes) {
  kdnn::pdl_chain_entry();
  const size_t n16 = bytes / 16;
  const size_t i0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = i0; i < n16; i += stride)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  for (size_t i = n16 * 16 + i0; i < bytes; i += stride) dst[i] = src[i];
}
cudaError_t copy_bytes_launch(const void* src, void* dst, size_t bytes, cudaStream_t st) {
  const unsigned blocks = static_cast<unsigned>(bytes / 16 / 256 + 1);
  return kdnn::launch_chained(copy_bytes_kernel, dim3(blocks > 64 ? 64 : blocks), dim3(256), 0, st,
                              static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), bytes);
}
// The device-side address of a host buffer when a kernel may touch it (page-locked or registered memory,
// 16-byte aligned), else nullptr: pageable memory goes through cudaMemcpyAsync.
void* mapped_host_pointer(const void* host) {
  cudaPointerAttributes a{};
  if (cudaPointerGetAttributes(&a, host) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (a.type != cudaMemoryTypeHost || a.devicePointer == nullptr) return nullptr;
  if ((reinterpret_cast<uintptr_t>(a.devicePointer) & 15u) != 0u) return nullptr;
  return a.devicePointer;
}
// kdnn_b200_quant_gemv_host moves x and y with copy_bytes_kernel when the host buffers allow it
// (measured on the three decode GEMVs: 1972 GB/s end to end against 1245 GB/s with the copy engine);
// kdnn_b200_host_copy_by_kernel(0) keeps cudaMemcpyAsync for everything.
std::atomic<int> g_host_copy_kernel{1};
bool host_copy_by_kernel() { return g_host_copy_kernel.load(std::memory_order_relaxed) != 0; }
}  // namespace

extern "C" {

const char* kdnn_b200_last_error(void) { return g_last_error.c_str(); }

int kdnn_b200_device_status(void) {
  const int a = kdnn::gemv_take_status();
  const int b = kdnn::moe_take_status();
  return a != 0 ? a : b;
}

size_t kdnn_b200_gemv_scratch_bytes(size_t K) { return kdnn::act_bytes(K); }

int kdnn_b200_gemv_supported(uint32_t ggml_type, size_t K, int scalar) {
  return scalar_ok(scalar) && int8_type(ggml_type) && kdnn::act_bytes(K) != 0 &&
         kdnn::block_aligned(ggml_type, K);
}

int kdnn_b200_quant_gemv(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                         const void* x, int x_scalar, void* y, int y_scalar, void* act_scratch,
                         size_t act_scratch_bytes, void* stream) {
  return kdnn_b200_quant_gemv_ex(ggml_type, w, rows, cols, x, x_scalar, y, y_scalar, act_scratch, act_scratch_bytes,
                                 nullptr, stream);
}

int kdnn_b200_quant_gemv_ex(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                            const void* x, int x_scalar, void* y, int y_scalar, void* act_scratch,
                            size_t act_scratch_bytes, const kdnn_b200_gemv_layout* layout, void* stream) {
  if (!scalar_ok(x_scalar) || !scalar_ok(y_scalar))
    return fail(KDNN_ERR_INVALID, "quant_gemv: scalar must be KDNN_F32 or KDNN_BF16");
  // the reference launcher's decline list, src/KokkosDNN_GGUFGemvInt8.hpp:724-745
  if (!int8_type(ggml_type)) return KDNN_DECLINED;
  if (w == nullptr || act_scratch == nullptr || x == nullptr || y == nullptr) return KDNN_DECLINED;
  if (!kdnn::block_aligned(ggml_type, cols)) return KDNN_DECLINED;
  if (rows == 0 || rows > static_cast<size_t>(INT_MAX)) return KDNN_DECLINED;
  if (cols > static_cast<size_t>(INT_MAX)) return KDNN_DECLINED;
  if (act_scratch_bytes < kdnn::act_bytes(cols)) return KDNN_DECLINED;
  if ((reinterpret_cast<uintptr_t>(act_scratch) & 15u) != 0u) return KDNN_DECLINED;
  if ((reinterpret_cast<uintptr_t>(w) & 1u) != 0u) return KDNN_DECLINED;
  if ((ggml_type == KDNN_GGML_Q4_K || ggml_type == KDNN_GGML_Q5_K) && (reinterpret_cast<uintptr_t>(w) & 15u) != 0u)
    return KDNN_DECLINED;
  return cuda_result(kdnn::gemv_launch(ggml_type, w, rows, cols, x, x_scalar, y, y_scalar,
                                       act_scratch, layout,
                                       static_cast<cudaStream_t>(stream)),
                     "quant_gemv");
}

int kdnn_b200_host_copy_by_kernel(int on) {
  const int prev = g_host_copy_kernel.load(std::memory_order_relaxed);
  if (on >= 0) g_host_copy_kernel.store(on != 0, std::memory_order_relaxed);
  return prev;
}

int kdnn_b200_launch_chaining(int on) {
  std::atomic<int>& f = kdnn::pdl_flag();
  const int prev = f.load(std::memory_order_relaxed);
  if (on >= 0) f.store(on != 0, std::memory_order_relaxed);
  return prev;
}

int kdnn_b200_quant_gemv_multi(uint32_t ggml_type, size_t n, const void* const* w, size_t rows, size_t cols,
                               const void* x, int x_scalar, void* const* y, int y_scalar, void* act_scratch,
                               size_t act_scratch_bytes, const kdnn_b200_gemv_layout* layout, void* stream) {
  if (!scalar_ok(x_scalar) || !scalar_ok(y_scalar))
    return fail(KDNN_ERR_INVALID, "quant_gemv_multi: scalar must be KDNN_F32 or KDNN_BF16");
  if (n == 0) return KDNN_OK;
  if (w == nullptr || y == nullptr) return fail(KDNN_ERR_INVALID, "quant_gemv_multi: null pointer array");
  // per matrix the decline list of kdnn_b200_quant_gemv; nothing is launched unless every matrix passes
  if (!int8_type(ggml_type) || act_scratch == nullptr || x == nullptr) return KDNN_DECLINED;
  if (!kdnn::block_aligned(ggml_type, cols) || rows == 0 || rows > static_cast<size_t>(INT_MAX) ||
      cols > static_cast<size_t>(INT_MAX) || act_scratch_bytes < kdnn::act_bytes(cols) ||
      (reinterpret_cast<uintptr_t>(act_scratch) & 15u) != 0u)
    return KDNN_DECLINED;
  for (size_t i = 0; i < n; ++i) {
    if (w[i] == nullptr || y[i] == nullptr || (reinterpret_cast<uintptr_t>(w[i]) & 1u) != 0u) return KDNN_DECLINED;
    if ((ggml_type == KDNN_GGML_Q4_K || ggml_type == KDNN_GGML_Q5_K) && (reinterpret_cast<uintptr_t>(w[i]) & 15u) != 0u)
      return KDNN_DECLINED;
  }
  for (size_t i = 0; i < n; i += 4) {
    const int m = static_cast<int>(n - i < 4 ? n - i : 4);
    const int rc = cuda_result(kdnn::gemv_multi_launch(ggml_type, m, w + i, rows, cols, x, x_scalar, y + i, y_scalar,
                                                       act_scratch, layout, static_cast<cudaStream_t>(stream)),
                               "quant_gemv_multi");
    if (rc != KDNN_OK) return rc;
  }
  return KDNN_OK;
}

int kdnn_b200_quant_gemv_host(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                              const void* x_host, int x_scalar, void* y_host, int y_scalar, void* x_dev,
                              void* y_dev, void* act_scratch, size_t act_scratch_bytes, void* stream) {
  if (!scalar_ok(x_scalar) || !scalar_ok(y_scalar))
    return fail(KDNN_ERR_INVALID, "quant_gemv_host: scalar must be KDNN_F32 or KDNN_BF16");
  if (x_host == nullptr || y_host == nullptr) return fail(KDNN_ERR_INVALID, "quant_gemv_host: null host buffer");
  // everything that can decline is checked before the first copy is enqueued
  if (!int8_type(ggml_type) || w == nullptr || act_scratch == nullptr || x_dev == nullptr || y_dev == nullptr ||
      !kdnn::block_aligned(ggml_type, cols) || rows == 0 || rows > static_cast<size_t>(INT_MAX) ||
      cols > static_cast<size_t>(INT_MAX) || act_scratch_bytes < kdnn::act_bytes(cols) ||
      (reinterpret_cast<uintptr_t>(act_scratch) & 15u) != 0u || (reinterpret_cast<uintptr_t>(w) & 1u) != 0u ||
      ((ggml_type == KDNN_GGML_Q4_K || ggml_type == KDNN_GGML_Q5_K) && (reinterpret_cast<uintptr_t>(w) & 15u) != 0u))
    return KDNN_DECLINED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t xb = x_scalar == KDNN_F32 ? 4 : 2, yb = y_scalar == KDNN_F32 ? 4 : 2;
  void* xm = nullptr;
  void* ym = nullptr;
  if (host_copy_by_kernel() && (reinterpret_cast<uintptr_t>(x_dev) & 15u) == 0u &&
      (reinterpret_cast<uintptr_t>(y_dev) & 15u) == 0u) {
    xm = mapped_host_pointer(x_host);
    ym = mapped_host_pointer(y_host);
  }
  cudaError_t e = xm ? copy_bytes_launch(xm, x_dev, cols * xb, st)
                     : cudaMemcpyAsync(x_dev, x_host, cols * xb, cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) return cuda_result(e, "quant_gemv_host: copy of x");
  const int rc = kdnn_b200_quant_gemv(ggml_type, w, rows, cols, x_dev, x_scalar, y_dev, y_scalar, act_scratch,
                                      act_scratch_bytes, stream);
  if (rc != KDNN_OK) return rc;
  e = ym ? copy_bytes_launch(y_dev, ym, rows * yb, st)
         : cudaMemcpyAsync(y_host, y_dev, rows * yb, cudaMemcpyDeviceToHost, st);
  return cuda_result(e, "quant_gemv_host: copy of y");
}

int kdnn_b200_quantize_act_q8(const void* x, int x_scalar, size_t K, void* scratch,
                              size_t scratch_bytes, void* stream) {
  if (!scalar_ok(x_scalar)) return fail(KDNN_ERR_INVALID, "quantize_act_q8: bad scalar");
  if (K == 0 || K % 32 != 0 || K > static_cast<size_t>(INT_MAX)) return KDNN_DECLINED;
  if (x == nullptr || scratch == nullptr || scratch_bytes < kdnn::act_bytes(K) ||
      (reinterpret_cast<uintptr_t>(scratch) & 15u) != 0u)
    return KDNN_DECLINED;
  return cuda_result(
      kdnn::quantize_act_launch(x, x_scalar, K, scratch, static_cast<cudaStream_t>(stream)),
      "quantize_act_q8");
}

int kdnn_b200_unit_dots(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                        const void* staged_scratch, int32_t* out, void* stream) {
  if (!int8_type(ggml_type) || !kdnn::block_aligned(ggml_type, cols))
    return fail(KDNN_ERR_INVALID, "unit_dots: unsupported dtype or K not block aligned");
  if (!w || !staged_scratch || !out || rows == 0 || rows > INT_MAX || cols > INT_MAX)
    return fail(KDNN_ERR_INVALID, "unit_dots: bad argument");
  if ((reinterpret_cast<uintptr_t>(staged_scratch) & 15u) || (reinterpret_cast<uintptr_t>(w) & 1u))
    return fail(KDNN_ERR_INVALID, "unit_dots: misaligned buffer");
  return cuda_result(kdnn::unit_dots_launch(ggml_type, w, rows, cols, staged_scratch, out,
                                            static_cast<cudaStream_t>(stream)),
                     "unit_dots");
}

size_t kdnn_b200_gemm_workspace_bytes(size_t M, size_t K) {
  return kdnn::gemm_workspace_bytes(M, K);
}

int kdnn_b200_tile_kind(int kind) { return kdnn::set_tile_kind(kind); }

size_t kdnn_b200_weight_table_tma_bytes(size_t n_experts) { return n_experts * 128; }

int kdnn_b200_weight_table_tma_encode(const uintptr_t* host_base, uint32_t ggml_type, size_t rows, size_t cols,
                                      size_t n_experts, void* host_out) {
  if (!host_base || !host_out) return fail(KDNN_ERR_INVALID, "weight_table_tma_encode: null argument");
  if (ggml_type != KDNN_GGML_Q4_K || cols == 0 || cols % 256 != 0 || rows == 0) return KDNN_DECLINED;
  const size_t rb = kdnn::row_bytes_of(ggml_type, cols);
  for (size_t e = 0; e < n_experts; ++e) {
    if (host_base[e] == 0) {   // an expert this rank does not hold: never addressed by the kernels
      memset(static_cast<uint8_t*>(host_out) + e * 128, 0, 128);
      continue;
    }
    if (host_base[e] & 15u) return KDNN_DECLINED;
    const cudaError_t err = kdnn::tc_encode_matrix_host(static_cast<uint8_t*>(host_out) + e * 128,
                                                        reinterpret_cast<const void*>(host_base[e]), rows, rb);
    if (err == cudaErrorNotSupported) return KDNN_DECLINED;   // driver without the tensor-map encoder
    if (err != cudaSuccess) return fail(KDNN_ERR_CUDA, "weight_table_tma_encode: cuTensorMapEncodeTiled failed");
  }
  return KDNN_OK;
}

int kdnn_b200_quant_gemm(uint32_t ggml_type, const void* w, size_t N, size_t K, const void* X,
                         size_t ldx, size_t M, int x_scalar, void* Y, size_t ldy, int y_scalar,
                         void* workspace, size_t workspace_bytes, void* stream) {
  return kdnn_b200_quant_gemm_dots(ggml_type, w, N, K, X, ldx, M, x_scalar, Y, ldy, y_scalar, nullptr, workspace,
                                   workspace_bytes, stream);
}

int kdnn_b200_quant_gemm_dots(uint32_t ggml_type, const void* w, size_t N, size_t K, const void* X,
                              size_t ldx, size_t M, int x_scalar, void* Y, size_t ldy, int y_scalar, int32_t* dots,
                              void* workspace, size_t workspace_bytes, void* stream) {
  if (!scalar_ok(x_scalar) || !scalar_ok(y_scalar))
    return fail(KDNN_ERR_INVALID, "quant_gemm: scalar must be KDNN_F32 or KDNN_BF16");
  if (M == 0 || N == 0 || K == 0) return KDNN_OK;  // src/KokkosDNN_GGUF.hpp:2576
  if (ldx < K || ldy < N) return fail(KDNN_ERR_INVALID, "quant_gemm: dimension mismatch");
  if (M * N > static_cast<size_t>(INT_MAX)) return fail(KDNN_ERR_INVALID, "quant_gemm: M*N too large");
  if (!tile_type(ggml_type) || !kdnn::block_aligned(ggml_type, K)) return KDNN_DECLINED;
  if (!w || !X || !Y || !workspace) return KDNN_DECLINED;
  if (workspace_bytes < kdnn::gemm_workspace_bytes(M, K)) return KDNN_DECLINED;
  if ((reinterpret_cast<uintptr_t>(workspace) & 15u) || (reinterpret_cast<uintptr_t>(w) & 1u))
    return KDNN_DECLINED;
  if ((ggml_type == KDNN_GGML_Q4_K || ggml_type == KDNN_GGML_Q5_K) && (reinterpret_cast<uintptr_t>(w) & 15u) != 0u)
    return KDNN_DECLINED;   // 16-byte loads of the super-blocks, src/KokkosDNN_GGUFGemvInt8.hpp:741-743
  if (dots != nullptr && (ggml_type != KDNN_GGML_Q4_K || kdnn::tile_kind() < 2)) return KDNN_DECLINED;
  return cuda_result(kdnn::gemm_launch(ggml_type, w, N, K, X, ldx, M, x_scalar, Y, ldy, y_scalar,
                                       workspace, dots, static_cast<cudaStream_t>(stream)),
                     "quant_gemm");
}

int kdnn_b200_moe_route(const void* logits, size_t ld, size_t T, size_t E, int scalar,
                        const void* bias, int top_k, int norm_topk, float routed_scale,
                        int sigmoid, int32_t* top_idx, float* top_w, void* stream) {
  if (!scalar_ok(scalar)) return fail(KDNN_ERR_INVALID, "moe_route: bad scalar");
  if (T == 0) return KDNN_OK;  // src/KokkosDNN_MoE.hpp:256
  if (top_k <= 0 || static_cast<size_t>(top_k) > E)
    return fail(KDNN_ERR_INVALID, "moe_route: need 1 <= top_k <= E");  // :257-258
  if (!logits || !top_idx || !top_w || ld < E || T > INT_MAX || E > INT_MAX)
    return fail(KDNN_ERR_INVALID, "moe_route: bad argument");
  return cuda_result(kdnn::moe_route_launch(logits, ld, T, E, scalar, bias, top_k, norm_topk,
                                            routed_scale, sigmoid, top_idx, top_w,
                                            static_cast<cudaStream_t>(stream)),
                     "moe_route");
}

size_t kdnn_b200_moe_workspace_bytes(size_t T, size_t S, size_t H, size_t F, size_t n_experts) {
  return kdnn::moe_workspace_bytes(T, S, H, F, n_experts);
}

int kdnn_b200_moe_ffn(const void* X, size_t ldx, size_t T, int x_scalar,
                      const kdnn_b200_weight_table* gate, const kdnn_b200_weight_table* up,
                      const kdnn_b200_weight_table* down, const int32_t* idx, const float* wts,
                      size_t S, void* Y, size_t ldy, int y_scalar, size_t expert_first,
                      size_t expert_count, void* workspace, size_t workspace_bytes, void* stream) {
  if (!scalar_ok(x_scalar) || !scalar_ok(y_scalar))
    return fail(KDNN_ERR_INVALID, "moe_ffn: scalar must be KDNN_F32 or KDNN_BF16");
  if (!gate || !up || !down) return fail(KDNN_ERR_INVALID, "moe_ffn: null weight table");
  const size_t H = gate->cols, F = gate->rows;
  // src/KokkosDNN_GGUF.hpp:2352-2357
  if (up->cols != H || up->rows != F || down->rows != H || down->cols != F)
    return fail(KDNN_ERR_INVALID, "moe_ffn: dimension mismatch");
  if (gate->n_experts == 0 || gate->n_experts != up->n_experts || gate->n_experts != down->n_experts)
    return fail(KDNN_ERR_INVALID, "moe_ffn: expert table mismatch");
  if (T == 0 || S == 0 || H == 0 || F == 0) return KDNN_OK;  // :2362
  if (ldx < H || ldy < H) return fail(KDNN_ERR_INVALID, "moe_ffn: dimension mismatch");
  if (!tile_type(gate->ggml_type) || !tile_type(up->ggml_type) || !tile_type(down->ggml_type))
    return KDNN_DECLINED;
  // :2369-2381
  if (H % 256 != 0 || F % 256 != 0)
    return fail(KDNN_ERR_INVALID, "moe_ffn: K-quant rows must be a multiple of 256 elements");
  if (gate->row_bytes != kdnn::row_bytes_of(gate->ggml_type, H) ||
      up->row_bytes != kdnn::row_bytes_of(up->ggml_type, H) ||
      down->row_bytes != kdnn::row_bytes_of(down->ggml_type, F))
    return fail(KDNN_ERR_INVALID, "moe_ffn: bad packed row");
  if (!X || !Y || !idx || !wts || !workspace || !gate->base || !up->base || !down->base)
    return fail(KDNN_ERR_INVALID, "moe_ffn: null argument");
  if (expert_first + expert_count > gate->n_experts)
    return fail(KDNN_ERR_INVALID, "moe_ffn: expert range outside the table");
  if (workspace_bytes < kdnn::moe_workspace_bytes(T, S, H, F, gate->n_experts) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return fail(KDNN_ERR_INVALID, "moe_ffn: workspace too small or not 256-byte aligned");
  if (T * S > static_cast<size_t>(INT_MAX) / 4)
    return fail(KDNN_ERR_INVALID, "moe_ffn: T*S too large");
  return cuda_result(kdnn::moe_ffn_launch(X, ldx, T, x_scalar, gate, up, down, idx, wts, S, Y, ldy,
                                          y_scalar, expert_first, expert_count, workspace,
                                          static_cast<cudaStream_t>(stream)),
                     "moe_ffn");
}

size_t kdnn_b200_moe_exchange_bytes(size_t tokens_local, size_t world, size_t top_k, size_t H) {
  return kdnn::moe_exchange_bytes(tokens_local, world, top_k, H);
}
size_t kdnn_b200_moe_block_workspace_bytes(size_t tokens_local, size_t world, size_t top_k, size_t H, size_t F,
                                           size_t n_experts, int with_region) {
  return kdnn::moe_block_workspace_bytes(tokens_local, world, top_k, H, F, n_experts, with_region);
}

int kdnn_b200_moe_block(const void* x, size_t ldx, size_t tokens_local, int scalar, const void* router_w, size_t ldr,
                        const void* router_bias, int top_k, int norm_topk, float routed_scale, int sigmoid,
                        const kdnn_b200_weight_table* gate, const kdnn_b200_weight_table* up,
                        const kdnn_b200_weight_table* down, size_t expert_first, size_t expert_count, float* y,
                        size_t ldy, const void* resid, size_t ldres, void* h_out, size_t ldh, void* xn_out,
                        size_t ldxn, float eps, const kdnn_b200_moe_exchange* ex, void* workspace,
                        size_t workspace_bytes, void* stream) {
  if (!scalar_ok(scalar)) return fail(KDNN_ERR_INVALID, "moe_block: scalar must be KDNN_F32 or KDNN_BF16");
  if (!gate || !up || !down) return fail(KDNN_ERR_INVALID, "moe_block: null weight table");
  const size_t H = gate->cols, F = gate->rows, E = gate->n_experts;
  if (up->cols != H || up->rows != F || down->rows != H || down->cols != F)
    return fail(KDNN_ERR_INVALID, "moe_block: dimension mismatch");
  if (E == 0 || E != up->n_experts || E != down->n_experts)
    return fail(KDNN_ERR_INVALID, "moe_block: expert table mismatch");
  if (tokens_local == 0) return KDNN_OK;
  if (top_k <= 0 || static_cast<size_t>(top_k) > E) return fail(KDNN_ERR_INVALID, "moe_block: need 1 <= top_k <= E");
  const int world = ex ? ex->world : 1, rank = ex ? ex->rank : 0;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || (ex && !ex->regions))
    return fail(KDNN_ERR_INVALID, "moe_block: bad exchange descriptor");
  if (gate->ggml_type != KDNN_GGML_Q4_K || up->ggml_type != KDNN_GGML_Q4_K || down->ggml_type != KDNN_GGML_Q4_K)
    return KDNN_DECLINED;
  if (H % 256 != 0 || F % 256 != 0 || F % 64 != 0) return fail(KDNN_ERR_INVALID, "moe_block: K-quant rows must be a multiple of 256 elements");
  if (!x || !router_w || !workspace || !gate->base || !up->base || !down->base || ldx < H || ldr < H)
    return fail(KDNN_ERR_INVALID, "moe_block: null argument or short row");
  const size_t sb = scalar == KDNN_F32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(router_w) & 15u) || (ldr * sb) % 16 != 0) return KDNN_DECLINED;
  if (y && ((reinterpret_cast<uintptr_t>(y) & 15u) || ldy % 4 != 0 || ldy < H)) return KDNN_DECLINED;
  if ((resid && ldres < H) || (h_out && ldh < H) || (xn_out && ldxn < H) || ((h_out || xn_out) && !resid))
    return fail(KDNN_ERR_INVALID, "moe_block: residual outputs need resid and rows of at least H");
  if (expert_first + expert_count > E) return fail(KDNN_ERR_INVALID, "moe_block: expert range outside the table");
  if (world > 1 && expert_count == 0) return fail(KDNN_ERR_INVALID, "moe_block: every rank needs at least one expert");
  const size_t T = tokens_local * static_cast<size_t>(world);
  if (T * static_cast<size_t>(top_k) > static_cast<size_t>(INT_MAX) / 4) return fail(KDNN_ERR_INVALID, "moe_block: T*S too large");
  if (world > 1 && (expert_count * static_cast<size_t>(world) != E || expert_first != static_cast<size_t>(rank) * expert_count))
    return fail(KDNN_ERR_INVALID, "moe_block: with several ranks the experts split evenly, rank r owning [r*E/world, (r+1)*E/world)");
  if (expert_count > 4096 || (H + 2 * E + 2 * static_cast<size_t>(top_k) + 512) * 4 + 16 * (H + 32) > 200 * 1024) return KDNN_DECLINED;
  if (workspace_bytes < kdnn::moe_block_workspace_bytes(tokens_local, world, top_k, H, F, E, ex == nullptr) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return fail(KDNN_ERR_INVALID, "moe_block: workspace too small or not 256-byte aligned");
  kdnn::BlockArgs a{};
  a.x = x; a.ldx = ldx; a.Tl = tokens_local; a.scalar = scalar; a.rw = router_w; a.ldr = ldr; a.bias = router_bias;
  a.top_k = top_k; a.norm_topk = norm_topk; a.sigmoid = sigmoid; a.routed_scale = routed_scale;
  a.gate = gate; a.up = up; a.down = down; a.e_first = expert_first; a.e_count = expert_count;
  a.resid = resid; a.ldres = ldres; a.h_out = h_out; a.ldh = ldh; a.xn_out = xn_out; a.ldxn = ldxn; a.eps = eps;
  a.y = y; a.ldy = ldy; a.world = world; a.rank = rank; a.regions = ex ? ex->regions : nullptr;
  a.wait_ns = ex && ex->wait_ns ? ex->wait_ns : 2000000000ull; a.ws = workspace;
  return cuda_result(kdnn::moe_block_launch(a, static_cast<cudaStream_t>(stream)), "moe_block");
}

int kdnn_b200_moe_block_routing(const kdnn_b200_moe_exchange* ex, void* workspace, size_t tokens_local, size_t world,
                                size_t top_k, size_t H, size_t F, size_t n_experts, int32_t* idx_out, float* wts_out,
                                void* stream) {
  if (!workspace || !idx_out || !wts_out) return fail(KDNN_ERR_INVALID, "moe_block_routing: null argument");
  const int32_t* idx = nullptr;
  const float* wts = nullptr;
  kdnn::moe_block_routing(ex ? ex->regions : nullptr, ex ? ex->rank : 0, workspace, tokens_local, world, top_k, H, F,
                          n_experts, &idx, &wts);
  const size_t n = tokens_local * world * top_k;
  cudaError_t e = cudaMemcpyAsync(idx_out, idx, n * sizeof(int32_t), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(wts_out, wts, n * sizeof(float), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
  return cuda_result(e, "moe_block_routing");
}

int kdnn_b200_peer_alloc(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes == 0) return fail(KDNN_ERR_INVALID, "peer_alloc: bad argument");
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaSuccess) e = cudaMemset(*ptr, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, *ptr);
  if (e == cudaSuccess) memcpy(handle64, &h, sizeof(h));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  return cuda_result(e, "peer_alloc");
}
int kdnn_b200_peer_open(const void* handle64, void** ptr) {
  if (!ptr || !handle64) return fail(KDNN_ERR_INVALID, "peer_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return cuda_result(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "peer_open");
}
int kdnn_b200_peer_close(void* ptr) { return cuda_result(cudaIpcCloseMemHandle(ptr), "peer_close"); }
int kdnn_b200_peer_free(void* ptr) { return cuda_result(cudaFree(ptr), "peer_free"); }

int kdnn_b200_residual_rmsnorm(const void* h, size_t ldh, const float* y, size_t ldy, void* out, size_t ldo,
                               size_t T, size_t H, float eps, int scalar, void* stream) {
  if (!scalar_ok(scalar)) return fail(KDNN_ERR_INVALID, "residual_rmsnorm: bad scalar");
  if (T == 0 || H == 0) return KDNN_OK;
  if (!h || !y || !out || ldh < H || ldy < H || ldo < H || T > INT_MAX || H > INT_MAX)
    return fail(KDNN_ERR_INVALID, "residual_rmsnorm: bad argument");
  return cuda_result(kdnn::residual_rmsnorm_launch(h, ldh, y, ldy, out, ldo, T, H, eps, scalar,
                                                   static_cast<cudaStream_t>(stream)),
                     "residual_rmsnorm");
}

int kdnn_b200_swiglu(const void* gate, size_t ldg, const void* up, size_t ldu, void* out, size_t ldo, size_t T, size_t F,
                     int scalar, void* stream) {
  if (!scalar_ok(scalar)) return fail(KDNN_ERR_INVALID, "swiglu: bad scalar");
  if (T == 0 || F == 0) return KDNN_OK;
  if (!gate || !up || !out || ldg < F || ldu < F || ldo < F || T > 65535 || F > INT_MAX)
    return fail(KDNN_ERR_INVALID, "swiglu: dimension mismatch");
  return cuda_result(kdnn::swiglu_launch(gate, ldg, up, ldu, out, ldo, T, F, scalar, static_cast<cudaStream_t>(stream)), "swiglu");
}

int kdnn_b200_moe_expert_weighted_sum(const void* expert_out, const float* top_w, void* y, size_t ldy, size_t T, size_t K,
                                      size_t D, int scalar, void* stream) {
  if (!scalar_ok(scalar)) return fail(KDNN_ERR_INVALID, "moe_expert_weighted_sum: bad scalar");
  if (T == 0 || D == 0 || K == 0) return KDNN_OK;   // src/KokkosDNN_MoE.hpp:323
  if (!expert_out || !top_w || !y || ldy < D || T > 65535 || D > INT_MAX || K > INT_MAX)
    return fail(KDNN_ERR_INVALID, "moe_expert_weighted_sum: dimension mismatch");
  return cuda_result(kdnn::weighted_sum_launch(expert_out, top_w, y, ldy, T, K, D, scalar, static_cast<cudaStream_t>(stream)),
                     "moe_expert_weighted_sum");
}

int kdnn_b200_moe_gather_rows(const void* src, size_t lds, size_t C, const int32_t* rows, void* dst, size_t ldd, size_t N,
                              size_t D, int scalar, void* stream) {
  if (!scalar_ok(scalar)) return fail(KDNN_ERR_INVALID, "moe_gather_rows: bad scalar");
  if (N == 0 || D == 0) return KDNN_OK;   // :347
  if (!src || !rows || !dst || lds < D || ldd < D || C == 0 || N > 65535 || D > INT_MAX)
    return fail(KDNN_ERR_INVALID, "moe_gather_rows: dimension mismatch");
  return cuda_result(kdnn::gather_rows_launch(src, lds, rows, dst, ldd, N, D, scalar, static_cast<cudaStream_t>(stream)),
                     "moe_gather_rows");
}

int kdnn_b200_moe_scatter_add_weighted(const void* src, size_t lds, const int32_t* rows, const float* weights, void* dst,
                                       size_t ldd, size_t C, size_t N, size_t D, int scalar, void* stream) {
  if (!scalar_ok(scalar)) return fail(KDNN_ERR_INVALID, "moe_scatter_add_weighted: bad scalar");
  if (N == 0 || D == 0 || C == 0) return KDNN_OK;   // :372
  if (!src || !rows || !weights || !dst || lds < D || ldd < D || N > 65535 || D > INT_MAX)
    return fail(KDNN_ERR_INVALID, "moe_scatter_add_weighted: dimension mismatch");
  return cuda_result(kdnn::scatter_add_launch(src, lds, rows, weights, dst, ldd, N, D, scalar, static_cast<cudaStream_t>(stream)),
                     "moe_scatter_add_weighted");
}

int kdnn_b200_read_probe(const void* src, size_t bytes, void* sink, void* stream) {
  if (!src || !sink || (reinterpret_cast<uintptr_t>(src) & 15u)) return fail(KDNN_ERR_INVALID, "read_probe: bad argument");
  if (bytes < 16) return KDNN_OK;
  return cuda_result(kdnn::read_probe_launch(src, bytes, static_cast<uint32_t*>(sink), 4 * kdnn::device_sm_count(),
                                             static_cast<cudaStream_t>(stream)), "read_probe");
}

int kdnn_b200_dequant_to_dense(uint32_t ggml_type, const void* w, size_t rows, size_t cols, void* y, size_t ldy,
                               int y_scalar, void* stream) {
  if (!scalar_ok(y_scalar)) return fail(KDNN_ERR_INVALID, "dequant_to_dense: bad scalar");
  if (ggml_type != KDNN_GGML_Q4_K && ggml_type != KDNN_GGML_Q5_K && ggml_type != KDNN_GGML_Q6_K &&
      ggml_type != KDNN_GGML_Q8_0)
    return fail(KDNN_ERR_INVALID, "dequant_to_dense: unsupported dtype");
  if (rows == 0 || cols == 0) return KDNN_OK;
  if (!kdnn::block_aligned(ggml_type, cols))
    return fail(KDNN_ERR_INVALID, "dequant_to_dense: cols must be a whole number of blocks");
  if (ldy < cols || !w || !y || rows > static_cast<size_t>(INT_MAX) || cols > static_cast<size_t>(INT_MAX))
    return fail(KDNN_ERR_INVALID, "dequant_to_dense: dimension mismatch");
  return cuda_result(kdnn::dequant_launch(ggml_type, w, rows, cols, y, ldy, y_scalar,
                                          static_cast<cudaStream_t>(stream)),
                     "dequant_to_dense");
}

int kdnn_b200_quant_gemv_fp(uint32_t ggml_type, const void* w, size_t rows, size_t cols, const void* x,
                            int x_scalar, void* y, int y_scalar, void* stream) {
  if (!scalar_ok(x_scalar) || !scalar_ok(y_scalar)) return fail(KDNN_ERR_INVALID, "quant_gemv_fp: bad scalar");
  if (!int8_type(ggml_type)) return fail(KDNN_ERR_INVALID, "quant_gemv_fp: unsupported dtype");
  if (rows == 0 || cols == 0) return KDNN_OK;
  if (!kdnn::block_aligned(ggml_type, cols))
    return fail(KDNN_ERR_INVALID, "quant_gemv_fp: cols must be a whole number of blocks");
  if (!w || !x || !y || rows > static_cast<size_t>(INT_MAX) || cols > static_cast<size_t>(INT_MAX))
    return fail(KDNN_ERR_INVALID, "quant_gemv_fp: bad argument");
  return cuda_result(kdnn::gemv_fp_launch(ggml_type, w, rows, cols, x, x_scalar, y, y_scalar,
                                          static_cast<cudaStream_t>(stream)),
                     "quant_gemv_fp");
}

}  // extern "C"
