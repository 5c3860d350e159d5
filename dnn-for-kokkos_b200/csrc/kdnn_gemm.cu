// Batched GEMV / skinny GEMM Y[M,N] = X[M,K] W[N,K]^T with packed W and per-row
// int8 activations: the grouped kernel of kdnn_grouped.cuh with one group that
// holds all M activation rows. Row m of Y equals the decode GEMV applied to row m.
#include "kdnn_grouped.cuh"
#include "kdnn_mma.cuh"
#include "kdnn_umma.cuh"

namespace kdnn {

bool tile_mma_enabled();
int tile_kind();
int* moe_status_ptr();

// workspace: [offs: 2 ints | pad to 256][wptr: 1 address | pad to 256][list: M ints][items: M x K/64]
static size_t gemm_items_offset(size_t M) { return 512 + ((M * sizeof(int) + 255) & ~size_t(255)); }
size_t gemm_workspace_bytes(size_t M, size_t K) {
  const size_t a = M * (K / 64) * sizeof(ActItem), b = M * act_row_pitch(K);
  return gemm_items_offset(M) + (a > b ? a : b);
}

__global__ void gemm_setup_kernel(int M, uintptr_t w, int* offs, uintptr_t* wptr, int* list) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) {
    offs[0] = 0;
    offs[1] = M;
    wptr[0] = w;
  }
  if (i < M) list[i] = i;
}

cudaError_t gemm_launch(uint32_t dt, const void* w, size_t N, size_t K, const void* X, size_t ldx,
                        size_t M, int xs, void* Y, size_t ldy, int ys, void* ws, cudaStream_t st) {
  uint8_t* b      = static_cast<uint8_t*>(ws);
  int* offs       = reinterpret_cast<int*>(b);
  uintptr_t* wptr = reinterpret_cast<uintptr_t*>(b + 256);
  int* list       = reinterpret_cast<int*>(b + 512);
  gemm_setup_kernel<<<(unsigned)((M + 255) / 256), 256, 0, st>>>((int)M, reinterpret_cast<uintptr_t>(w),
                                                                 offs, wptr, list);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  if (dt == KDNN_GGML_Q4_K && tile_mma_enabled() && (reinterpret_cast<uintptr_t>(w) & 15u) == 0) {
    uint8_t* xrows = b + gemm_items_offset(M);
    err = xs == KDNN_F32
              ? launch_quantize_rows<float>(static_cast<const float*>(X), ldx, (int)M, (int)K, nullptr, xrows, act_row_pitch(K), st)
              : launch_quantize_rows<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(X), ldx, (int)M, (int)K, nullptr, xrows, act_row_pitch(K), st);
    if (err != cudaSuccess) return err;
    MmaParams q{};
    q.w0 = wptr; q.row_bytes = (int)row_bytes_of(dt, K);
    q.N = (int)N; q.K = (int)K; q.offs = offs; q.list = list; q.S = 1; q.g_first = 0;
    q.xrows = xrows; q.x_pitch = act_row_pitch(K); q.dst = Y; q.ld_dst = ldy; q.status = moe_status_ptr();
    q.passes_z = static_cast<int>(M <= 32 ? 1 : (M + 31) / 32 > 4 ? 4 : (M + 31) / 32);
    q.early = M <= 8;   // the row quantizer in front of it is then a handful of CTAs
    if (tile_kind() == 2)
      return ys == KDNN_F32 ? launch_grouped_umma<2, float>(q, 1, st) : launch_grouped_umma<2, __nv_bfloat16>(q, 1, st);
    return ys == KDNN_F32 ? launch_grouped_mma<2, float>(q, 1, st) : launch_grouped_mma<2, __nv_bfloat16>(q, 1, st);
  }
  ActItem* items = reinterpret_cast<ActItem*>(b + gemm_items_offset(M));
  err = xs == KDNN_F32
            ? launch_quantize_items<float>(dt, static_cast<const float*>(X), ldx, (int)M, (int)K, nullptr, items, st)
            : launch_quantize_items<__nv_bfloat16>(dt, static_cast<const __nv_bfloat16*>(X), ldx, (int)M, (int)K, nullptr, items, st);
  if (err != cudaSuccess) return err;
  GroupedParams p{};
  p.w0 = wptr;
  p.row_bytes0 = (int)row_bytes_of(dt, K);
  p.N = (int)N; p.K = (int)K;
  p.offs = offs; p.list = list; p.S = 1; p.g_first = 0;
  p.src = items; p.dst = Y; p.ld_dst = ldy;
  if (xs == KDNN_F32 && ys == KDNN_F32) return launch_grouped_dt<2, float, float>(dt, p, 1, st);
  if (xs == KDNN_BF16 && ys == KDNN_BF16) return launch_grouped_dt<2, __nv_bfloat16, __nv_bfloat16>(dt, p, 1, st);
  if (xs == KDNN_BF16 && ys == KDNN_F32) return launch_grouped_dt<2, __nv_bfloat16, float>(dt, p, 1, st);
  return launch_grouped_dt<2, float, __nv_bfloat16>(dt, p, 1, st);
}

}  // namespace kdnn
