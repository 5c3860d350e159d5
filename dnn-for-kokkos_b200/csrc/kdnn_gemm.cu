// Batched GEMV / skinny GEMM Y[M,N] = X[M,K] W[N,K]^T with packed W and per-row
// int8 activations: the grouped kernel of kdnn_grouped.cuh with one group that
// holds all M activation rows. Row m of Y equals the decode GEMV applied to row m.
#include "kdnn_grouped.cuh"
#include "kdnn_mma.cuh"
#include "kdnn_tc.cuh"

namespace kdnn {

int tile_kind();
cudaError_t moe_status_ptr(int** out);
cudaError_t gemv_launch(uint32_t dt, const void* w, size_t rows, size_t cols, const void* x, int xs,
                        void* y, int ys, void* scratch, const kdnn_b200_gemv_layout* layout, cudaStream_t stream);

// workspace: [offs: 2 ints, group count | pad to 256][wptr: 1 address | pad to 256][list: M ints][groups][items: M x K/64]
static size_t gemm_groups_offset(size_t M) { return 512 + ((M * sizeof(int) + 255) & ~size_t(255)); }
static size_t gemm_items_offset(size_t M) {
  return gemm_groups_offset(M) + (((M + kTcNT - 1) / kTcNT * sizeof(int4) + 255) & ~size_t(255));
}
size_t gemm_workspace_bytes(size_t M, size_t K) {
  const size_t a = M * (K / 64) * sizeof(ActItem), b = M * act_row_pitch(K);
  return gemm_items_offset(M) + (a > b ? a : b);
}

__global__ void gemm_setup_kernel(int M, uintptr_t w, int* offs, uintptr_t* wptr, int* list, int4* groups) {
  pdl_chain_entry();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) {
    offs[0] = 0;
    offs[1] = M;
    offs[2] = (M + kTcNT - 1) / kTcNT;   // groups of the tensor-core tile kernel: 32 activation rows each
    wptr[0] = w;
  }
  if (i < M) list[i] = i;
  if (i * kTcNT < M) groups[i] = make_int4(0, i * kTcNT, min(kTcNT, M - i * kTcNT), 0);
}

// Weight rows per tile of the tcgen05 kernel for a single matrix: as close to 128 as gives every SM the
// same number of tiles (a 14336-row matrix on 148 SMs: 97 rows, one tile each).
static int gemm_tile_rows(size_t N, size_t groups) {
  const size_t sms = static_cast<size_t>(device_sm_count());
  for (size_t rounds = 1; rounds <= 64; ++rounds) {
    const size_t per = (sms * rounds + groups - 1) / groups;   // row tiles per group for `rounds` full waves
    const size_t tr = (N + per - 1) / per;
    if (tr <= 128) return static_cast<int>(tr < 32 ? 32 : tr);
  }
  return 128;
}

// `dots` (parity probe, tcgen05 kernel only): int32 [M][N][K/32] raw sub-block dots, or nullptr.
cudaError_t gemm_launch(uint32_t dt, const void* w, size_t N, size_t K, const void* X, size_t ldx,
                        size_t M, int xs, void* Y, size_t ldy, int ys, void* ws, int32_t* dots, cudaStream_t st) {
  uint8_t* b      = static_cast<uint8_t*>(ws);
  // Crossover measured on a 14336 x 4096 Q4_K matrix: one GEMV kernel per activation row (6.9 us each) beats
  // the tile kernels (24 us and up) for up to three rows; the tcgen05 kernel is the faster tile kernel up
  // to eight rows (24-27 us against 30-31 us), the mma.sync kernel beyond (28 / 37 us against 31 / 42 us
  // at 16 / 32 rows).
  int kind = tile_kind();
  if (kind == 3 && dots == nullptr) {
    if (M <= 3) {
      uint8_t* scratch = b + gemm_items_offset(M);   // room for one staged row: the workspace holds M of them
      const size_t xb = xs == KDNN_F32 ? 4 : 2, yb = ys == KDNN_F32 ? 4 : 2;
      for (size_t m = 0; m < M; ++m) {
        const cudaError_t e = gemv_launch(dt, w, N, K, static_cast<const uint8_t*>(X) + m * ldx * xb, xs,
                                          static_cast<uint8_t*>(Y) + m * ldy * yb, ys, scratch, nullptr, st);
        if (e != cudaSuccess) return e;
      }
      return cudaSuccess;
    }
    kind = M <= 8 ? 2 : 1;
  } else if (kind == 3) {
    kind = 2;
  }
  int* offs       = reinterpret_cast<int*>(b);
  uintptr_t* wptr = reinterpret_cast<uintptr_t*>(b + 256);
  int* list       = reinterpret_cast<int*>(b + 512);
  int4* groups    = reinterpret_cast<int4*>(b + gemm_groups_offset(M));
  cudaError_t err = launch_chained(gemm_setup_kernel, dim3((unsigned)((M + 255) / 256)), dim3(256), 0, st, (int)M,
                                   reinterpret_cast<uintptr_t>(w), offs, wptr, list, groups);
  if (err != cudaSuccess) return err;
  if (dt == KDNN_GGML_Q4_K && kind != 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0) {
    uint8_t* xrows = b + gemm_items_offset(M);
    int* status = nullptr;
    err = moe_status_ptr(&status);
    if (err != cudaSuccess) return err;
    err = xs == KDNN_F32
              ? launch_quantize_rows<float>(static_cast<const float*>(X), ldx, (int)M, (int)K, nullptr, xrows, act_row_pitch(K), st)
              : launch_quantize_rows<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(X), ldx, (int)M, (int)K, nullptr, xrows, act_row_pitch(K), st);
    if (err != cudaSuccess) return err;
    if (kind == 2) {
      TcParams t{};
      err = tc_encode_matrix(&t.one, w, N, row_bytes_of(dt, K));
      if (err == cudaSuccess) {
        const size_t ngroups = (M + kTcNT - 1) / kTcNT;
        t.N = (int)N; t.K = (int)K;
        t.tile_rows = gemm_tile_rows(N, ngroups);
        t.row_tiles = (int)((N + t.tile_rows - 1) / t.tile_rows);
        t.groups = groups; t.n_groups = offs + 2; t.list = list; t.S = 1;
        t.xrows = xrows; t.x_pitch = act_row_pitch(K); t.dst = Y; t.ld_dst = ldy; t.status = status;
        t.dots = dots;
        const int tiles = (int)(ngroups * t.row_tiles);
        return ys == KDNN_F32 ? launch_grouped_tc<2, float>(t, tiles, st) : launch_grouped_tc<2, __nv_bfloat16>(t, tiles, st);
      }
      // no tensor-map encoder in this driver: the mma.sync kernel serves the call
    }
    MmaParams q{};
    q.w0 = wptr; q.row_bytes = (int)row_bytes_of(dt, K);
    q.N = (int)N; q.K = (int)K; q.offs = offs; q.list = list; q.S = 1; q.g_first = 0;
    q.xrows = xrows; q.x_pitch = act_row_pitch(K); q.dst = Y; q.ld_dst = ldy; q.status = status;
    q.passes_z = static_cast<int>(M <= 32 ? 1 : (M + 31) / 32 > 4 ? 4 : (M + 31) / 32);
    q.early = M <= 8;   // the row quantizer in front of it is then a handful of CTAs
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
