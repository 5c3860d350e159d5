// MoE kernels for sm_100a: router (top-k + weights), slot sort by expert, the
// packed expert feed-forward with per-32 int8 activations (gate/up + SwiGLU,
// down), and the weighted combine.
//
// Launch sequence of kdnn_b200_moe_ffn (no host synchronisation anywhere; the
// routing result is consumed on the device, as in the reference's fused decode
// kernels, src/KokkosDNN_GGUF.hpp:2329-2332):
//   1. moe_sort_kernel      slots (t,s) grouped by expert -> offsets, slot list
//   2. quantize rows        x rows -> per-32 int8
//   3. tile GEMM, MODE 1    act[pos, j] = Scalar(silu(gate_e x_t)_j * (up_e x_t)_j)
//   4. quantize rows        act rows -> per-32 int8 (inside step 3's epilogue on the mma.sync path)
//   5. tile GEMM, MODE 0    out[pos, d] = down_e[d,:] . act[pos,:]
//   6. moe_combine_kernel   Y[t, d] = Scalar(sum_s w[t,s] * out[pos(t,s), d])
// Workspace (caller-owned): offsets, slot list, slot positions, int8 items, act, out.
#include <type_traits>
#include "kdnn_grouped.cuh"
#include "kdnn_mma.cuh"
#include "kdnn_tc.cuh"

#include <limits.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>

namespace kdnn {

__device__ int g_moe_status = 0;
// Device address of the status word, looked up once per device (outside any stream capture when the first
// call on a device is) and cached; a failed lookup is reported to the caller instead of handing the kernels
// a null pointer.
cudaError_t moe_status_ptr(int** out) {
  constexpr int kMaxDevices = 64;
  static int* cache[kMaxDevices] = {};
  static std::atomic<bool> ready[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (!ready[dev].load(std::memory_order_acquire)) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_moe_status);
    if (e != cudaSuccess) return e;
    cache[dev] = static_cast<int*>(p);
    ready[dev].store(true, std::memory_order_release);
  }
  *out = cache[dev];
  return cudaSuccess;
}

int device_sm_count() {
  static std::atomic<int> cache[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int v = cache[dev & 63].load(std::memory_order_relaxed);
  if (v == 0) {
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    cache[dev & 63].store(v, std::memory_order_relaxed);
  }
  return v;
}

TcEncodeFn tc_encode_fn() {
  static std::atomic<TcEncodeFn> fn{nullptr};
  TcEncodeFn f = fn.load(std::memory_order_acquire);
  if (f == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    f = reinterpret_cast<TcEncodeFn>(p);
    fn.store(f, std::memory_order_release);
  }
  return f;
}

cudaError_t tc_encode_matrix_host(void* out128, const void* w, size_t rows, size_t row_bytes) {
  CUtensorMap m;
  const cudaError_t e = tc_encode_matrix(&m, w, rows, row_bytes);
  if (e == cudaSuccess) memcpy(out128, &m, 128);
  return e;
}

// Which Q4_K tile kernel the batched calls use: 3 = by measured crossover (default: the GEMV kernel per row
// up to 3 activation rows, the tcgen05 kernel up to 8, the mma.sync kernel beyond and for the MoE
// feed-forward), 2 = tcgen05 + TMEM everywhere it applies, 1 = mma.sync, 0 = the CUDA-core dp4a kernel
// (which also serves every other format). Process-wide, read per call.
static std::atomic<int> g_tile_kind{3};
int tile_kind() { return g_tile_kind.load(std::memory_order_relaxed); }
int set_tile_kind(int k) { return k >= 0 && k <= 3 ? g_tile_kind.exchange(k) : g_tile_kind.load(); }

// ---- router ----------------------------------------------------------------------
// One warp per token; the E scores live in shared memory (src/KokkosDNN_MoE.hpp:
// 161-200 stages them the same way), selection is a warp arg-max repeated top_k
// times with the reference's tie rule (strict '>' scanning ids upward = lowest id
// among equals), weights are recomputed from the logits by lane 0 in the
// reference's order (:114-146).
// Top-k selection and weights of ONE token by one warp. `lg(e)` / `bs(e)`: the logit and the bias of expert e
// as floats (already rounded to the Scalar they are stored in); `score`: E floats of shared memory.
template <class GetLogit, class GetBias>
__device__ __forceinline__ void route_warp(GetLogit lg, GetBias bs, bool has_bias, int E, int top_k, int norm_topk,
                                           float routed_scale, int sigmoid, float* score, int32_t* idx, float* w,
                                           int lane) {
  constexpr float NEG = -3.4028235e38f;
  for (int e = lane; e < E; e += 32) {
    const float raw = lg(e);
    const float b   = has_bias ? bs(e) : 0.0f;
    score[e]        = sigmoid ? (1.0f / (1.0f + expf(-raw))) + b : raw + b;
  }
  __syncwarp();
  float gmx = NEG, gsum = 0.0f;
  if (!sigmoid && !norm_topk) {  // global softmax denominator, sequential like the reference
    if (lane == 0) {
      for (int e = 0; e < E; ++e)
        if (score[e] > gmx) gmx = score[e];
      for (int e = 0; e < E; ++e) gsum += expf(score[e] - gmx);
    }
  }
  for (int k = 0; k < top_k; ++k) {
    float best = NEG;
    int be     = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float s = score[e];
      if (s > best) {
        best = s;
        be   = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe   = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) {
        best = ob;
        be   = oe;
      }
    }
    if (be == 0x7fffffff) be = -1;  // nothing above the sentinel
    if (lane == 0) {
      idx[k] = be;
      if (be >= 0) score[be] = NEG;
    }
    __syncwarp();
  }
  if (lane != 0) return;
  auto logit = [&](int k) {
    const int i     = idx[k];
    const float raw = lg(i < 0 ? 0 : i);
    return sigmoid ? 1.0f / (1.0f + expf(-raw)) : raw + (has_bias ? bs(i < 0 ? 0 : i) : 0.0f);
  };
  if (sigmoid) {
    if (norm_topk) {
      float sum = 0.0f;
      for (int k = 0; k < top_k; ++k) sum += logit(k);
      const float denom = sum + 1e-6f;
      for (int k = 0; k < top_k; ++k) w[k] = logit(k) / denom * routed_scale;
    } else {
      for (int k = 0; k < top_k; ++k) w[k] = logit(k) * routed_scale;
    }
  } else if (norm_topk) {
    float mx = NEG, sum = 0.0f;
    for (int k = 0; k < top_k; ++k) mx = logit(k) > mx ? logit(k) : mx;
    for (int k = 0; k < top_k; ++k) sum += expf(logit(k) - mx);
    for (int k = 0; k < top_k; ++k) w[k] = expf(logit(k) - mx) / sum * routed_scale;
  } else {
    for (int k = 0; k < top_k; ++k) w[k] = expf(logit(k) - gmx) / gsum * routed_scale;
  }
}

// The same selection and weights for E <= 256 and top_k <= 32 with the scores in registers (lane l holds the
// experts l, l + 32, ...): a selection round is two warp reductions (largest score, then smallest expert id among
// the lanes that hold it -- the reference's first-maximum rule), the weights are formed by lanes 0..top_k-1 in
// parallel and summed in slot order. The global-softmax denominator (neither sigmoid nor norm_topk) is a lane-wise
// then tree sum instead of the reference's sequential one: within 1e-6 relative of it.
// On return lane k < top_k holds slot k: sel_e (expert id or -1) and sel_w.
template <int J, class GetLogit, class GetBias>
__device__ __forceinline__ void route_warp_regs(GetLogit lg, GetBias bs, bool has_bias, int E, int top_k, int norm_topk,
                                                float routed_scale, int sigmoid, int lane, int& sel_e, float& sel_w) {
  constexpr float NEG = -3.4028235e38f;   // J = experts per lane (E <= 32 * J)
  float raw[J], bia[J], sc[J];
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int e = lane + 32 * j;
    raw[j] = 0.f; bia[j] = 0.f; sc[j] = NEG;
    if (e < E) {
      raw[j] = lg(e);
      bia[j] = has_bias ? bs(e) : 0.0f;
      sc[j] = sigmoid ? (1.0f / (1.0f + expf(-raw[j]))) + bia[j] : raw[j] + bia[j];
    }
  }
  float gmx = NEG, gsum = 0.0f;
  if (!sigmoid && !norm_topk) {
#pragma unroll
    for (int j = 0; j < J; ++j)
      if (lane + 32 * j < E && sc[j] > gmx) gmx = sc[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) gmx = fmaxf(gmx, __shfl_xor_sync(0xffffffffu, gmx, o));
#pragma unroll
    for (int j = 0; j < J; ++j)
      if (lane + 32 * j < E) gsum += expf(sc[j] - gmx);
    gsum = warp_sum(gsum);
  }
  const float raw0 = __shfl_sync(0xffffffffu, raw[0], 0), bia0 = __shfl_sync(0xffffffffu, bia[0], 0);
  int my_e = -1;
  float my_raw = raw0, my_b = bia0;   // an empty slot reads expert 0, like the reference's weight pass
  for (int k = 0; k < top_k; ++k) {
    float best = NEG, braw = 0.f, bb = 0.f;
    int bj = -1;
#pragma unroll
    for (int j = 0; j < J; ++j)
      if (sc[j] > best) { best = sc[j]; bj = j; braw = raw[j]; bb = bia[j]; }
    const uint32_t u = __float_as_uint(best + 0.0f);
    const uint32_t key = bj < 0 ? 0u : ((u & 0x80000000u) ? ~u : (u | 0x80000000u));
    const uint32_t top = __reduce_max_sync(0xffffffffu, key);
    const uint32_t mine = (top != 0u && key == top) ? static_cast<uint32_t>(lane + 32 * bj) : 0xffffffffu;
    const uint32_t be = __reduce_min_sync(0xffffffffu, mine);
    const int src = static_cast<int>(be & 31u);
    const float wraw = __shfl_sync(0xffffffffu, braw, src), wb = __shfl_sync(0xffffffffu, bb, src);
    if (be != 0xffffffffu) {
      if (lane == src) {
#pragma unroll
        for (int j = 0; j < J; ++j)
          if (j == static_cast<int>(be >> 5)) sc[j] = NEG;
      }
      if (lane == k) { my_e = static_cast<int>(be); my_raw = wraw; my_b = wb; }
    }
  }
  const float l = sigmoid ? 1.0f / (1.0f + expf(-my_raw)) : my_raw + (has_bias ? my_b : 0.0f);
  float wgt = 0.f;
  if (sigmoid) {
    if (norm_topk) {
      float sum = 0.0f;
      for (int k = 0; k < top_k; ++k) sum += __shfl_sync(0xffffffffu, l, k);
      wgt = l / (sum + 1e-6f) * routed_scale;
    } else {
      wgt = l * routed_scale;
    }
  } else if (norm_topk) {
    float mx = NEG;
    for (int k = 0; k < top_k; ++k) mx = fmaxf(mx, __shfl_sync(0xffffffffu, l, k));
    const float ex = expf(l - mx);
    float sum = 0.0f;
    for (int k = 0; k < top_k; ++k) sum += __shfl_sync(0xffffffffu, ex, k);
    wgt = ex / sum * routed_scale;
  } else {
    wgt = expf(l - gmx) / gsum * routed_scale;
  }
  sel_e = my_e;
  sel_w = wgt;
}

template <class ST>
__global__ void moe_route_kernel(const ST* logits, size_t ld, int T, int E,
                                 const ST* bias, int top_k, int norm_topk,
                                 float routed_scale, int sigmoid, int32_t* top_idx,
                                 float* top_w) {
  pdl_chain_entry();
  extern __shared__ float route_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int t = blockIdx.x * wpb + warp;
  if (t >= T) return;
  const ST* lg = logits + static_cast<size_t>(t) * ld;
  route_warp([&](int e) { return to_f32(lg[e]); }, [&](int e) { return to_f32(bias[e]); }, bias != nullptr, E, top_k,
             norm_topk, routed_scale, sigmoid, route_smem + static_cast<size_t>(warp) * E,
             top_idx + static_cast<size_t>(t) * top_k, top_w + static_cast<size_t>(t) * top_k, lane);
}

cudaError_t moe_route_launch(const void* logits, size_t ld, size_t T, size_t E, int scalar,
                             const void* bias, int top_k, int norm_topk, float routed_scale,
                             int sigmoid, int32_t* top_idx, float* top_w, cudaStream_t st) {
  int wpb = 4;
  while (wpb > 1 && static_cast<size_t>(wpb) * E * sizeof(float) > 48 * 1024) wpb >>= 1;
  const size_t smem = static_cast<size_t>(wpb) * E * sizeof(float);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  const int blocks = static_cast<int>((T + wpb - 1) / wpb);
  if (scalar == KDNN_F32)
    return launch_chained(moe_route_kernel<float>, dim3(blocks), dim3(wpb * 32), smem, st,
                          static_cast<const float*>(logits), ld, (int)T, (int)E, static_cast<const float*>(bias),
                          top_k, norm_topk, routed_scale, sigmoid, top_idx, top_w);
  return launch_chained(moe_route_kernel<__nv_bfloat16>, dim3(blocks), dim3(wpb * 32), smem, st,
                        static_cast<const __nv_bfloat16*>(logits), ld, (int)T, (int)E,
                        static_cast<const __nv_bfloat16*>(bias), top_k, norm_topk, routed_scale, sigmoid, top_idx,
                        top_w);
}

// ---- slot sort ---------------------------------------------------------------------
// Groups the T*S routed slots by expert for experts in [e_first, e_first+e_count).
//   offs[e_count + 1]  start of each local expert's run in `list`
//   list[n]            slot id (t*S + s) of the n-th position
//   pos[t*S + s]       position of the slot in `list`, or -1 when the slot's expert
//                      is out of range / not local (it then contributes nothing,
//                      src/KokkosDNN_GGUF.hpp:2106-2110)
// Order inside an expert's run is by slot id (token-major), as the reference's host-side
// counting sort produces (models/lfm2_5/KokkosDNN_LFM25Model.hpp:455-486); results do not
// depend on it. Several small CTAs: every CTA counts all slots (shared-memory atomics) and
// forms the same prefix sums, then places only its own experts -- a warp per expert sweeps
// the slot ids upward 32 at a time, ranks come from one ballot per sweep step.
__global__ void moe_sort_kernel(const int32_t* idx, int n_slots, int e_first,
                                int e_count, int* offs, int* list,
                                int* pos, int cache_slots) {
  pdl_chain_entry();
  extern __shared__ int sort_smem[];  // counts[e_count], cursor[e_count], then (when it fits) the local expert of every slot
  int* counts = sort_smem;
  int* cursor = sort_smem + e_count;
  int* local  = sort_smem + 2 * (e_count + 1);
  for (int e = threadIdx.x; e < e_count; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_slots; i += blockDim.x) {
    const int e = idx[i] - e_first;
    if (cache_slots) local[i] = e;
    if (e >= 0 && e < e_count) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x < 32) {   // exclusive prefix sums by one warp, 32 experts per step
    int run = 0;
    for (int e0 = 0; e0 < e_count; e0 += 32) {
      const int e = e0 + static_cast<int>(threadIdx.x);
      const int c = e < e_count ? counts[e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (static_cast<int>(threadIdx.x) >= o) incl += v;
      }
      if (e < e_count) {
        cursor[e] = run + incl - c;
        if (blockIdx.x == 0) offs[e] = run + incl - c;
      }
      run += __shfl_sync(0xFFFFFFFFu, incl, 31);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) offs[e_count] = run;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const unsigned below = (1u << lane) - 1u;
  for (int e = blockIdx.x * nwarps + warp; e < e_count; e += gridDim.x * nwarps) {
    if (counts[e] == 0) continue;
    int c = cursor[e];
    for (int base = 0; base < n_slots; base += 32) {
      const int i = base + lane;
      const bool hit = i < n_slots && (cache_slots ? local[i] : idx[i] - e_first) == e;
      const unsigned m = __ballot_sync(0xFFFFFFFFu, hit);
      if (hit) {
        const int ps = c + __popc(m & below);
        list[ps] = i;
        pos[i]   = ps;
      }
      c += __popc(m);
    }
  }
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_slots; i += gridDim.x * blockDim.x) {
    const int e = idx[i] - e_first;
    if (e < 0 || e >= e_count) pos[i] = -1;
  }
}


// ---- prep: slot sort + activation quantizer in ONE launch ------------------------------------
// CTA 0 groups the routed slots by expert (same outputs as moe_sort_kernel plus the tile kernels' group
// list), every other CTA quantizes activation rows. The sort is a counting sort over a bit matrix in shared
// memory: bit t of mask[e][t / 32] says token t routed a slot to local expert e, so a slot's position inside
// its expert's run is a prefix popcount -- every slot is placed independently, in token order, by its own
// thread (no sweep per expert). A token that names the same expert twice (callers may pass any idx) is
// detected by the atomicOr that sets the bit; the kernel then places sequentially per expert instead.
//   groups[g] = {table index of the expert, first position, rows (<= 32), 0}: one entry per 32 rows of an
//   expert's run, experts without rows have none.
struct PrepParams {
  const int32_t* idx;
  int n_slots, S, e_first, e_count, words;   // words = ceil(T / 32)
  int* offs; int* list; int* pos; int4* groups; int* n_groups;
  const void* X; size_t ldx; int T, H; uint8_t* xrows; size_t x_pitch;   // X == nullptr: no rows to quantize
};

__device__ void moe_sort_block(const PrepParams& p, uint32_t* sm) {
  const int tid = threadIdx.x, nt = blockDim.x, E = p.e_count, W = p.words;
  uint32_t* mask = sm;
  uint32_t* wpre = mask + E * W;
  int* counts = reinterpret_cast<int*>(wpre + E * W);
  int* starts = counts + E;
  int* gst    = starts + E + 1;
  int* dup    = gst + E + 1;
  // the routed expert of up to eight slots per thread is read once, all loads in flight together, and kept
  // in registers for the placement pass (a single CTA lives on memory latency here)
  constexpr int kPer = 8;
  const bool cached = p.n_slots <= nt * kPer;
  int ev[kPer];
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int i = tid + j * nt;
    ev[j] = cached && i < p.n_slots ? p.idx[i] - p.e_first : -1;
  }
  for (int i = tid; i < E * W; i += nt) mask[i] = 0u;
  if (tid == 0) *dup = 0;
  __syncthreads();
  for (int i = tid, j = 0; i < p.n_slots; i += nt, ++j) {
    const int e = cached ? ev[j < kPer ? j : 0] : p.idx[i] - p.e_first;
    if (e >= 0 && e < E) {
      const int t = i / p.S;
      const uint32_t bit = 1u << (t & 31);
      const uint32_t old = atomicOr(&mask[e * W + (t >> 5)], bit);
      if (old & bit) *dup = 1;
    }
  }
  __syncthreads();
  const bool has_dup = *dup != 0;
  for (int e = tid; e < E; e += nt) {
    int run = 0;
    if (!has_dup) {
      for (int w = 0; w < W; ++w) {
        wpre[e * W + w] = run;
        run += __popc(mask[e * W + w]);
      }
    } else {
      for (int i = 0; i < p.n_slots; ++i) run += (p.idx[i] - p.e_first == e);
    }
    counts[e] = run;
  }
  __syncthreads();
  if (tid < 32) {   // exclusive prefix sums of the row counts and of the group counts, 32 experts per step
    int run = 0, grun = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + tid;
      const int c = e < E ? counts[e] : 0;
      const int gc = (c + kTcNT - 1) / kTcNT;
      int incl = c, gincl = gc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, o), gv = __shfl_up_sync(0xFFFFFFFFu, gincl, o);
        if (tid >= o) { incl += v; gincl += gv; }
      }
      if (e < E) { starts[e] = run + incl - c; gst[e] = grun + gincl - gc; }
      run += __shfl_sync(0xFFFFFFFFu, incl, 31);
      grun += __shfl_sync(0xFFFFFFFFu, gincl, 31);
    }
    if (tid == 0) {
      starts[E] = run;
      p.offs[E] = run;
      *p.n_groups = grun;
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += nt) {
    p.offs[e] = starts[e];
    const int c = counts[e];
    for (int q = 0; q * kTcNT < c; ++q)
      p.groups[gst[e] + q] = make_int4(p.e_first + e, starts[e] + q * kTcNT, min(kTcNT, c - q * kTcNT), 0);
    if (has_dup) {   // sequential, stable placement of this expert's slots
      int c2 = starts[e];
      for (int i = 0; i < p.n_slots; ++i)
        if (p.idx[i] - p.e_first == e) { p.list[c2] = i; p.pos[i] = c2; ++c2; }
    }
  }
  for (int i = tid, j = 0; i < p.n_slots; i += nt, ++j) {
    const int e = cached ? ev[j < kPer ? j : 0] : p.idx[i] - p.e_first;
    if (e < 0 || e >= E) {
      p.pos[i] = -1;
    } else if (!has_dup) {
      const int t = i / p.S, w = t >> 5;
      const uint32_t bit = 1u << (t & 31);
      const int ps = starts[e] + static_cast<int>(wpre[e * W + w]) + __popc(mask[e * W + w] & (bit - 1u));
      p.list[ps] = i;
      p.pos[i]   = ps;
    }
  }
}
inline size_t moe_sort_smem(size_t e_count, size_t T) {
  return (2 * e_count * ((T + 31) / 32) + 3 * e_count + 8) * sizeof(int);
}

// One warp-iteration = eight 32-blocks of one row (four lanes per block), as quantize_rows_kernel.
template <class SRC>
__device__ void quantize_rows_part(const SRC* src, size_t ld, int nrows, int K, uint8_t* dst,
                                   size_t pitch_bytes, int gwarp, int nwarp) {
  const int nblk = K / 32, per_row = (nblk + 7) / 8;
  const int lane = threadIdx.x & 31, l4 = lane & 3;
  for (int it = gwarp; it < nrows * per_row; it += nwarp) {
    const int row = it / per_row, b = (it - row * per_row) * 8 + (lane >> 2);
    const SRC* x = src + static_cast<size_t>(row) * ld;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    uint8_t* out = dst + static_cast<size_t>(row) * pitch_bytes;
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
      reinterpret_cast<ActHdr*>(out + act_hdr_offset(K))[b] = ActHdr{d, part, total - part, 0};
      const float ds = __fmul_rn(static_cast<float>(total), d);
      reinterpret_cast<float2*>(out + act_bytes(K))[b] = make_float2(d, ds);
      store_sum_parts(out, act_parts_offset(static_cast<size_t>(K)), b, ds);
    }
  }
}

template <class SRC>
__global__ void __launch_bounds__(1024, 1) moe_prep_kernel(const PrepParams p) {
  pdl_chain_entry();
  extern __shared__ uint32_t prep_smem[];
  if (blockIdx.x == 0) {
    moe_sort_block(p, prep_smem);
  } else if (p.X != nullptr) {
    quantize_rows_part<SRC>(static_cast<const SRC*>(p.X), p.ldx, p.T, p.H, p.xrows, p.x_pitch,
                            (blockIdx.x - 1) * (blockDim.x >> 5) + (threadIdx.x >> 5), (gridDim.x - 1) * (blockDim.x >> 5));
  }
}

static cudaError_t moe_prep_launch(const PrepParams& p, int xs, cudaStream_t st) {
  const size_t smem = moe_sort_smem(p.e_count, p.T);
  int qctas = 0;
  if (p.X != nullptr) {
    const int items = p.T * ((p.H / 32 + 7) / 8);
    qctas = max(1, min(4 * device_sm_count(), (items + 31) / 32));
  }
  auto kern = xs == KDNN_F32 ? moe_prep_kernel<float> : moe_prep_kernel<__nv_bfloat16>;
  if (smem > 48 * 1024) {   // once per device, at the largest size this kernel is ever given (kPrepSmemLimit)
    static SmemAttrOnce once[2];
    const cudaError_t e = set_max_smem_once(once[xs == KDNN_F32], kern, 160 * 1024);
    if (e != cudaSuccess) return e;
  }
  return launch_chained(kern, dim3(1 + qctas), dim3(1024), smem, st, p);
}
constexpr size_t kPrepSmemLimit = 160 * 1024;

// Y[t, d] = Scalar(sum_s w[t,s] * out[pos(t,s), d]), slots ascending, fp32
// (src/KokkosDNN_MoE.hpp:326-331; zero-weight and unrouted slots skipped,
// src/KokkosDNN_GGUF.hpp:2205-2207).
template <class YT>
__global__ void moe_combine_kernel(const float* out, const int* pos,
                                   const float* wts, int T, int S, int H, YT* Y,
                                   size_t ldy) {
  pdl_chain_entry();
  const int t = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= H) return;
  float acc = 0.f;
  for (int s = 0; s < S; ++s) {
    const int ps  = pos[t * S + s];
    const float w = wts[t * S + s];
    if (ps < 0 || w == 0.0f) continue;
    acc += w * out[static_cast<size_t>(ps) * H + d];
  }
  store_scalar(Y + static_cast<size_t>(t) * ldy + d, acc);
}

// The same sums, four columns per thread (16-byte loads of `out`; H % 4 == 0 and 16-byte / 8-byte
// aligned output rows): every element is accumulated in the same slot order as above.
template <class YT>
__global__ void moe_combine4_kernel(const float* out, const int* pos,
                                    const float* wts, int T, int S, int H, YT* Y,
                                    size_t ldy) {
  pdl_chain_entry();
  const int t = blockIdx.y;
  const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (d >= H) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < S; ++s) {
    const int ps  = pos[t * S + s];
    const float w = wts[t * S + s];
    if (ps < 0 || w == 0.0f) continue;
    const float4 v = *reinterpret_cast<const float4*>(out + static_cast<size_t>(ps) * H + d);
    acc.x += w * v.x;
    acc.y += w * v.y;
    acc.z += w * v.z;
    acc.w += w * v.w;
  }
  YT* dst = Y + static_cast<size_t>(t) * ldy + d;
  if (sizeof(YT) == 4) {
    *reinterpret_cast<float4*>(dst) = acc;
  } else {
    __nv_bfloat162 h[2] = {__floats2bfloat162_rn(acc.x, acc.y), __floats2bfloat162_rn(acc.z, acc.w)};
    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(h);
  }
}

// ---- workspace layout -------------------------------------------------------------------
struct MoeWs {
  size_t offs, list, pos, groups, ngroups, xq, act, actq, out, total;
};
static size_t max_sz(size_t a, size_t b) { return a > b ? a : b; }
static MoeWs moe_ws_layout(size_t T, size_t S, size_t H, size_t F, size_t n_experts) {
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  MoeWs w{};
  size_t o = 0;
  w.offs = o; o += up((n_experts + 1) * sizeof(int));
  w.list = o; o += up(T * S * sizeof(int));
  w.pos  = o; o += up(T * S * sizeof(int));
  w.groups = o; o += up((n_experts + T * S / kTcNT + 1) * sizeof(int4));
  w.ngroups = o; o += 256;
  w.xq   = o; o += up(T * max_sz((H / 64) * sizeof(ActItem), act_row_pitch(H)));
  w.act  = o; o += up(T * S * F * sizeof(float));
  w.actq = o; o += up(T * S * max_sz((F / 64) * sizeof(ActItem), act_row_pitch(F)));
  w.out  = o; o += up(T * S * H * sizeof(float));
  w.total = o;
  return w;
}
size_t moe_workspace_bytes(size_t T, size_t S, size_t H, size_t F, size_t n_experts) {
  return moe_ws_layout(T, S, H, F, n_experts).total;
}

// The expert feed-forward between the slot sort and the combine, Q4_K on the tensor cores:
// gate/up + SwiGLU (+ per-32 quantization of the result) and the down projection, two launches.
// `kind` 2 = tcgen05 kernel (needs the tables' TMA descriptors), 1 = mma.sync kernel.
static cudaError_t moe_tiles_q4k(int kind, const kdnn_b200_weight_table* gate, const kdnn_b200_weight_table* up,
                                 const kdnn_b200_weight_table* down, size_t T, size_t S, int xs, size_t e_first,
                                 size_t e_count, uint8_t* b, const MoeWs& L, cudaStream_t st) {
  const size_t H = gate->cols, F = gate->rows;
  const int n_slots = static_cast<int>(T * S);
  int* offs = reinterpret_cast<int*>(b + L.offs);
  int* list = reinterpret_cast<int*>(b + L.list);
  float* act = reinterpret_cast<float*>(b + L.act);
  float* out = reinterpret_cast<float*>(b + L.out);
  uint8_t* xrows = b + L.xq;
  uint8_t* arows = b + L.actq;
  int* status = nullptr;
  cudaError_t err = moe_status_ptr(&status);
  if (err != cudaSuccess) return err;
  if (kind == 2) {
    const int max_groups = static_cast<int>(e_count) + n_slots / kTcNT;
    TcParams g{};
    g.maps0 = static_cast<const CUtensorMap*>(gate->tma); g.maps1 = static_cast<const CUtensorMap*>(up->tma);
    g.N = (int)F; g.K = (int)H; g.tile_rows = 64; g.row_tiles = (int)((F + 63) / 64);
    g.groups = reinterpret_cast<const int4*>(b + L.groups); g.n_groups = reinterpret_cast<const int*>(b + L.ngroups);
    g.list = list; g.S = (int)S; g.xrows = xrows; g.x_pitch = act_row_pitch(H);
    g.dst = act; g.ld_dst = F; g.round_bf16 = xs == KDNN_BF16; g.qdst = arows; g.q_pitch = act_row_pitch(F);
    g.status = status;
    err = launch_grouped_tc<1, float>(g, max_groups * g.row_tiles, st);
    if (err != cudaSuccess) return err;
    TcParams d{};
    d.maps0 = static_cast<const CUtensorMap*>(down->tma);
    d.N = (int)H; d.K = (int)F; d.tile_rows = 128; d.row_tiles = (int)((H + 127) / 128);
    d.groups = g.groups; d.n_groups = g.n_groups; d.list = list; d.S = (int)S;
    d.xrows = arows; d.x_pitch = act_row_pitch(F); d.dst = out; d.ld_dst = H; d.status = status;
    return launch_grouped_tc<0, float>(d, max_groups * d.row_tiles, st);
  }
  MmaParams g{};
  g.w0 = gate->base; g.w1 = up->base; g.row_bytes = (int)gate->row_bytes;
  g.N = (int)F; g.K = (int)H; g.offs = offs; g.list = list; g.S = (int)S; g.g_first = (int)e_first;
  g.xrows = xrows; g.x_pitch = act_row_pitch(H); g.dst = act; g.ld_dst = F;
  g.round_bf16 = xs == KDNN_BF16; g.status = status;
  // A group has n_slots / n_experts rows on average; routing is never uniform, so give every group one
  // CTA more along z than the mean needs (CTAs without a pass return at once).
  const int mean_rows = static_cast<int>((static_cast<size_t>(n_slots) + gate->n_experts - 1) / gate->n_experts);
  const int passes_z  = max(1, min(4, 1 + (2 * mean_rows) / 32));
  g.passes_z = passes_z;
  g.early = T <= 8;   // one-token decode: the kernel in front of it is a handful of CTAs
  const bool fused_q = F % 64 == 0;   // the epilogue quantizes whole 32-blocks of the result
  if (fused_q) {
    g.qdst    = arows;
    g.q_pitch = act_row_pitch(F);
  }
  err = launch_grouped_mma<1, float>(g, (int)e_count, st);
  if (err != cudaSuccess) return err;
  if (!fused_q) {
    err = launch_quantize_rows<float>(act, F, n_slots, (int)F, offs + e_count, arows, act_row_pitch(F), st);
    if (err != cudaSuccess) return err;
  }
  MmaParams d{};
  d.w0 = down->base; d.w1 = nullptr; d.row_bytes = (int)down->row_bytes;
  d.N = (int)H; d.K = (int)F; d.offs = offs; d.list = list; d.S = (int)S; d.g_first = (int)e_first;
  d.xrows = arows; d.x_pitch = act_row_pitch(F); d.dst = out; d.ld_dst = H; d.status = status;
  d.passes_z = passes_z;
  return launch_grouped_mma<0, float>(d, (int)e_count, st);
}

// Whether the tcgen05 kernel covers this call (otherwise the mma.sync kernel runs it).
static bool tc_covers(const kdnn_b200_weight_table* gate, const kdnn_b200_weight_table* up,
                      const kdnn_b200_weight_table* down) {
  const size_t H = gate->cols, F = gate->rows;
  return gate->tma != nullptr && up->tma != nullptr && down->tma != nullptr && F % 64 == 0 && H >= 512 && F >= 256;
}

template <class YT>
static cudaError_t moe_combine_launch(const float* out, const int* pos, const float* wts, size_t T, size_t S, size_t H,
                                      void* Y, size_t ldy, cudaStream_t st) {
  const size_t ybytes = sizeof(YT);
  const bool vec4 = H % 4 == 0 && (reinterpret_cast<uintptr_t>(Y) % (4 * ybytes)) == 0 && (ldy * ybytes) % (4 * ybytes) == 0;
  if (vec4)
    return launch_chained(moe_combine4_kernel<YT>, dim3((unsigned)((H / 4 + 127) / 128), (unsigned)T), dim3(128), 0, st,
                          out, pos, wts, (int)T, (int)S, (int)H, static_cast<YT*>(Y), ldy);
  return launch_chained(moe_combine_kernel<YT>, dim3((unsigned)((H + 255) / 256), (unsigned)T), dim3(256), 0, st, out,
                        pos, wts, (int)T, (int)S, (int)H, static_cast<YT*>(Y), ldy);
}

cudaError_t moe_ffn_launch(const void* X, size_t ldx, size_t T, int xs,
                           const kdnn_b200_weight_table* gate, const kdnn_b200_weight_table* up,
                           const kdnn_b200_weight_table* down, const int32_t* idx, const float* wts,
                           size_t S, void* Y, size_t ldy, int ys, size_t e_first, size_t e_count,
                           void* ws, cudaStream_t st) {
  const size_t H = gate->cols, F = gate->rows;
  if (gate->ggml_type != up->ggml_type) return cudaErrorNotSupported;  // mixed gate/up recipe
  const MoeWs L = moe_ws_layout(T, S, H, F, gate->n_experts);
  uint8_t* b    = static_cast<uint8_t*>(ws);
  int* offs = reinterpret_cast<int*>(b + L.offs);
  int* list = reinterpret_cast<int*>(b + L.list);
  int* pos  = reinterpret_cast<int*>(b + L.pos);
  float* act = reinterpret_cast<float*>(b + L.act);
  ActItem* xq   = reinterpret_cast<ActItem*>(b + L.xq);
  ActItem* actq = reinterpret_cast<ActItem*>(b + L.actq);
  float* out = reinterpret_cast<float*>(b + L.out);
  const int n_slots = static_cast<int>(T * S);
  const bool all_q4k = gate->ggml_type == KDNN_GGML_Q4_K && down->ggml_type == KDNN_GGML_Q4_K &&
                       (reinterpret_cast<uintptr_t>(ws) & 15u) == 0;
  const int want = tile_kind() == 3 ? 1 : tile_kind();   // measured: the mma.sync kernel is the faster one here
  const int kind = !all_q4k ? 0 : (want == 2 && !tc_covers(gate, up, down)) ? 1 : want;
  cudaError_t err;
  if (kind != 0 && moe_sort_smem(e_count, T) <= kPrepSmemLimit) {
    // one launch: slot sort (CTA 0) + row quantizer (the other CTAs)
    PrepParams pp{};
    pp.idx = idx; pp.n_slots = n_slots; pp.S = (int)S; pp.e_first = (int)e_first; pp.e_count = (int)e_count;
    pp.words = (int)((T + 31) / 32);
    pp.offs = offs; pp.list = list; pp.pos = pos;
    pp.groups = reinterpret_cast<int4*>(b + L.groups); pp.n_groups = reinterpret_cast<int*>(b + L.ngroups);
    pp.X = e_count > 0 ? X : nullptr; pp.ldx = ldx; pp.T = (int)T; pp.H = (int)H;
    pp.xrows = b + L.xq; pp.x_pitch = act_row_pitch(H);
    err = moe_prep_launch(pp, xs, st);
    if (err != cudaSuccess) return err;
    if (e_count > 0) {
      err = moe_tiles_q4k(kind, gate, up, down, T, S, xs, e_first, e_count, b, L, st);
      if (err != cudaSuccess) return err;
    }
  } else {
    const int sort_ctas = static_cast<int>(e_count < 4 ? 1 : (e_count + 3) / 4 > 64 ? 64 : (e_count + 3) / 4);
    const int cache_slots = n_slots <= 8192;   // the sweeps then read shared memory instead of global memory
    err = launch_chained(moe_sort_kernel, dim3(sort_ctas), dim3(128),
                         (2 * (e_count + 1) + (cache_slots ? n_slots : 0)) * sizeof(int), st, idx, n_slots,
                         (int)e_first, (int)e_count, offs, list, pos, cache_slots);
    if (err != cudaSuccess) return err;
    if (e_count > 0 && kind != 0) {   // slot matrix too large for the one-CTA sort: mma.sync kernel behind the plain sort
      err = xs == KDNN_F32
                ? launch_quantize_rows<float>(static_cast<const float*>(X), ldx, (int)T, (int)H, nullptr, b + L.xq, act_row_pitch(H), st)
                : launch_quantize_rows<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(X), ldx, (int)T, (int)H, nullptr, b + L.xq, act_row_pitch(H), st);
      if (err != cudaSuccess) return err;
      err = moe_tiles_q4k(1, gate, up, down, T, S, xs, e_first, e_count, b, L, st);
      if (err != cudaSuccess) return err;
    } else if (e_count > 0) {
      err = xs == KDNN_F32
                ? launch_quantize_items<float>(gate->ggml_type, static_cast<const float*>(X), ldx, (int)T, (int)H, nullptr, xq, st)
                : launch_quantize_items<__nv_bfloat16>(gate->ggml_type, static_cast<const __nv_bfloat16*>(X), ldx, (int)T, (int)H, nullptr, xq, st);
      if (err != cudaSuccess) return err;
      GroupedParams g{};
      g.w0 = gate->base; g.w1 = up->base;
      g.row_bytes0 = (int)gate->row_bytes; g.row_bytes1 = (int)up->row_bytes;
      g.N = (int)F; g.K = (int)H;
      g.offs = offs; g.list = list; g.S = (int)S; g.g_first = (int)e_first;
      g.src = xq; g.dst = act; g.ld_dst = F; g.round_bf16 = xs == KDNN_BF16;
      err = xs == KDNN_F32 ? launch_grouped_dt<1, float, float>(gate->ggml_type, g, (int)e_count, st)
                           : launch_grouped_dt<1, __nv_bfloat16, float>(gate->ggml_type, g, (int)e_count, st);
      if (err != cudaSuccess) return err;
      err = launch_quantize_items<float>(down->ggml_type, act, F, n_slots, (int)F, offs + e_count, actq, st);
      if (err != cudaSuccess) return err;
      GroupedParams d{};
      d.w0 = down->base; d.w1 = nullptr;
      d.row_bytes0 = (int)down->row_bytes;
      d.N = (int)H; d.K = (int)F;
      d.offs = offs; d.list = list; d.S = (int)S; d.g_first = (int)e_first;
      d.src = actq; d.dst = out; d.ld_dst = H;
      err = launch_grouped_dt<0, float, float>(down->ggml_type, d, (int)e_count, st);
      if (err != cudaSuccess) return err;
    }
  }
  return ys == KDNN_F32 ? moe_combine_launch<float>(out, pos, wts, T, S, H, Y, ldy, st)
                        : moe_combine_launch<__nv_bfloat16>(out, pos, wts, T, S, H, Y, ldy, st);
}

// out[t,:] = Scalar(r / sqrt(mean(r^2) + eps)) with r = Scalar(float(h[t,:]) + y[t,:]): the residual
// add after the MoE block (models/lfm2_5/KokkosDNN_LFM25Model.hpp:812-816) fused with the next block's
// un-scaled RMS norm (src/KokkosDNN_RMSNorm.hpp:347-361). One CTA per row, fp32 statistics.
template <class ST>
__global__ void residual_rmsnorm_kernel(const ST* h, size_t ldh, const float* y,
                                        size_t ldy, ST* out, size_t ldo, int H, float eps) {
  pdl_chain_entry();
  __shared__ float red[32];
  const int t = blockIdx.x;
  float ss = 0.f;
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    ST r;
    store_scalar(&r, to_f32(h[static_cast<size_t>(t) * ldh + d]) + y[static_cast<size_t>(t) * ldy + d]);
    const float v = to_f32(r);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = 1.0f / sqrtf(v / static_cast<float>(H) + eps);
  }
  __syncthreads();
  const float inv = red[0];
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    ST r;
    store_scalar(&r, to_f32(h[static_cast<size_t>(t) * ldh + d]) + y[static_cast<size_t>(t) * ldy + d]);
    store_scalar(out + static_cast<size_t>(t) * ldo + d, to_f32(r) * inv);
  }
}

cudaError_t residual_rmsnorm_launch(const void* h, size_t ldh, const float* y, size_t ldy, void* out,
                                    size_t ldo, size_t T, size_t H, float eps, int scalar, cudaStream_t st) {
  if (scalar == KDNN_F32)
    return launch_chained(residual_rmsnorm_kernel<float>, dim3((unsigned)T), dim3(256), 0, st,
                          static_cast<const float*>(h), ldh, y, ldy, static_cast<float*>(out), ldo, (int)H, eps);
  return launch_chained(residual_rmsnorm_kernel<__nv_bfloat16>, dim3((unsigned)T), dim3(256), 0, st,
                        static_cast<const __nv_bfloat16*>(h), ldh, y, ldy, static_cast<__nv_bfloat16*>(out), ldo,
                        (int)H, eps);
}


// ===== the MoE block in four launches, single GPU or expert-parallel over peer memory ================
//   1. moe_gate_kernel     router logits (x . Wr^T, fp32 accumulation, rounded to Scalar like the caller's
//                          gemm, models/lfm2_5/KokkosDNN_LFM25Model.hpp:788-797), top-k + weights, per-32
//                          quantization of the token rows -- written into EVERY rank's exchange region
//                          (plain peer stores: the dispatch is an all-gather by push, 4 KB per token and
//                          rank at hidden 2048); the last CTA to finish tells the peers, waits for theirs
//                          and sorts all routed slots for the local experts
//   2. gate/up tile kernel, 3. down tile kernel (its epilogue stores every output row straight into the
//                          token owner's slot-indexed buffer and its last CTA raises the owners' flags)
//   4. moe_combine_norm_kernel   waits for every rank's flag, sums the slots in slot order, adds the
//                          residual and forms the next block's un-scaled RMS norm
// Exchange region of one rank (all ranks use the same layout; T = tokens_local * world):
//   xrows  [T] quantized token rows        written by every rank's gate kernel (its own tokens)
//   idx    [T][S] routed expert ids        written by every rank's gate kernel (its own tokens)
//   rel    [T][S] rank of the slot inside its expert's run on the expert's owner (only the owner's copy
//                 of a slot's entry is written)
//   wts    [T][S] routing weights          local use only (the owner's combine)
//   out    [T][S][H] down-projection rows of the slots whose expert lives HERE; the token owners read them
//   cnt    [kMaxLocalExperts] rows routed to each local expert this call (peers add with system-scope atomics)
//   xflag / oflag  [world] epochs: "rank r's rows and routing are here" / "rank r's out rows are complete"
constexpr size_t kMaxLocalExperts = 4096;
struct ExLayout {
  size_t xrows, idx, rel, wts, out, cnt, xflag, oflag, total;
};
static ExLayout ex_layout(size_t Tl, size_t world, size_t S, size_t H) {
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  const size_t T = Tl * world;
  ExLayout L{};
  size_t o = 0;
  L.xrows = o; o += up(T * act_row_pitch(H));
  L.idx   = o; o += up(T * S * sizeof(int32_t));
  L.rel   = o; o += up(T * S * sizeof(int32_t));
  L.wts   = o; o += up(T * S * sizeof(float));
  L.out   = o; o += up(T * S * H * sizeof(float));
  L.cnt   = o; o += up(kMaxLocalExperts * sizeof(int));
  L.xflag = o; o += 256;
  L.oflag = o; o += 256;
  L.total = o;
  return L;
}
size_t moe_exchange_bytes(size_t tokens_local, size_t world, size_t S, size_t H) {
  return ex_layout(tokens_local, world, S, H).total;
}

constexpr int kGateThreads = 512;   // 16 warps
constexpr int kGateCluster = 4;     // CTAs of one cluster split the experts of the logit product
struct GateParams {
  const void* x; size_t ldx;
  const void* rw; size_t ldr; const void* bias;
  int Tl, H, E, top_k, norm_topk, sigmoid, world, rank;
  float routed_scale;
  int e_per_rank;               // experts per rank (world > 1: E / world), owner of expert e = e / e_per_rank
  uint8_t* region[kMaxRanks];   // every rank's exchange region
  ExLayout L;
  size_t x_pitch;
  int e_first, e_count;         // this rank's experts
  int* offs; int* list; int4* groups; int* n_groups;   // outputs of the last CTA (this rank's workspace)
  int* pos;                     // single rank: position of every slot in `list` (the down rows are kept by position)
  int* ticket; uint32_t* epoch; int* status;
  unsigned long long wait_ns;
};

__device__ __forceinline__ unsigned cluster_cta_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `p` (a shared-memory pointer of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ float* cluster_map(float* p, unsigned rank) {
  uint64_t out;
  asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"(reinterpret_cast<uint64_t>(p)), "r"(rank));
  return reinterpret_cast<float*>(out);
}

// One cluster of kGateCluster CTAs owns TPC tokens. Every CTA of the cluster holds the tokens' rows in
// shared memory and forms the logits of ITS quarter of the experts (so a CTA streams a quarter of the
// router matrix from L2); the logits land, through distributed shared memory, in the CTA that routes the
// token (token i of the cluster belongs to CTA i % kGateCluster), which then also quantizes its row.
template <class ST, int TPC>
__global__ void __launch_bounds__(kGateThreads) moe_gate_kernel(const GateParams p) {
  pdl_chain_entry();
  constexpr int C = kGateCluster, RT = (TPC + C - 1) / C, TH = TPC > 4 ? 4 : TPC;
  extern __shared__ __align__(16) uint8_t gate_smem[];
  float* xs = reinterpret_cast<float*>(gate_smem);                       // [TPC][H]
  float* lgs = xs + static_cast<size_t>(TPC) * p.H;                      // [RT][E] rounded logits of the tokens routed here
  float* score = lgs + static_cast<size_t>(RT) * p.E;                    // [RT][E] (only the router for E > 256)
  int32_t* ridx = reinterpret_cast<int32_t*>(score + static_cast<size_t>(RT) * p.E);   // [RT][top_k]
  float* rwts = reinterpret_cast<float*>(ridx + RT * p.top_k);                          // [RT][top_k]
  float* part = rwts + RT * p.top_k;                                     // [16 warps][TPC][32] partial logits
  // bf16 tokens: a second copy of the rows as stored, [8][H + 32] (rows past nt are zero), for the tensor-core product
  __nv_bfloat16* xb = reinterpret_cast<__nv_bfloat16*>(part + (kGateThreads / 32) * TPC * 32);
  constexpr bool kTensor = std::is_same<ST, __nv_bfloat16>::value;
  const int xb_pitch = p.H + 32;
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned crank = cluster_cta_rank();
  const uint32_t epoch = *p.epoch + 1u;                                  // this block call's epoch
  const int t_first = static_cast<int>(blockIdx.x / C) * TPC;            // local token index of the cluster's first token
  const int nt = max(0, min(TPC, p.Tl - t_first));
  const ST* x = static_cast<const ST*>(p.x);
  {
    const int h8 = p.H / 8;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (p.ldx * sizeof(ST)) % 16 == 0;
    for (int i = threadIdx.x; i < nt * h8; i += kGateThreads) {
      const int t = i / h8, k = (i - t * h8) * 8;
      float v[8];
      load8<ST>(x + static_cast<size_t>(t_first + t) * p.ldx, static_cast<size_t>(k), vec_ok, v);
      *reinterpret_cast<float4*>(xs + t * p.H + k) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(xs + t * p.H + k + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    for (int i = nt * p.H + threadIdx.x; i < TPC * p.H; i += kGateThreads) xs[i] = 0.f;
    if (kTensor) {
      for (int i = threadIdx.x; i < 8 * h8; i += kGateThreads) {
        const int t = i / h8, k = (i - t * h8) * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (t < nt) {
          const ST* src = x + static_cast<size_t>(t_first + t) * p.ldx + k;
          if (vec_ok) v = *reinterpret_cast<const uint4*>(src);
          else memcpy(&v, src, 16);
        }
        *reinterpret_cast<uint4*>(xb + t * xb_pitch + k) = v;
      }
    }
  }
  __syncthreads();
  // ---- router logits of this CTA's experts: lane = expert (32 at a time), warp = one sixteenth of the hidden
  // dimension. A lane streams its expert's row piece 16 bytes at a time and meets the tokens' values as
  // shared-memory broadcasts; partial sums (even and odd elements apart, packed fp32 FMA) go through shared
  // memory and are added warp 0 first. The order is the same for every grid shape, so the logits do not
  // depend on how many ranks share the tokens.
  {
    const ST* rw = static_cast<const ST*>(p.rw);
    constexpr int kWarps = kGateThreads / 32;
    const int Ec = (p.E + C - 1) / C, e_lo = static_cast<int>(crank) * Ec, e_hi = min(p.E, e_lo + Ec);
    const int kw = p.H / kWarps, k_lo = warp * kw;          // this warp's piece of K (a multiple of 16 elements)
    if (kTensor) {
      // bf16: the product runs on the tensor cores (mma.sync m16n8k16, fp32 accumulators): experts are the M
      // rows, the (up to eight) tokens the N columns. A lane takes 16 bytes of an expert row and of a token row
      // at the same place, which is the fragment of TWO k-steps under one fixed permutation of the 32 elements
      // of that piece of K (the same permutation on both operands leaves the dot product unchanged).
      const int g = lane >> 2, tq = lane & 3;
      const __nv_bfloat16* rwb = reinterpret_cast<const __nv_bfloat16*>(rw);
      for (int eb = e_lo; eb < e_hi; eb += 32) {
        float d[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        for (int k = 0; k < kw; k += 128) {               // up to four 32-element pieces with all loads in flight
          uint4 av[4][2][2];
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const int er = min(eb + 16 * mt + 8 * hh + g, e_hi - 1);
                const int kk = k + 32 * u < kw ? k + 32 * u : k;
                av[u][mt][hh] = *reinterpret_cast<const uint4*>(rwb + static_cast<size_t>(er) * p.ldr + k_lo + kk + 8 * tq);
              }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (k + 32 * u >= kw) break;
            const uint4 bv = *reinterpret_cast<const uint4*>(xb + g * xb_pitch + k_lo + k + 32 * u + 8 * tq);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
              const uint4 lo = av[u][mt][0], hi = av[u][mt][1];
              asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                           : "+f"(d[mt][0]), "+f"(d[mt][1]), "+f"(d[mt][2]), "+f"(d[mt][3])
                           : "r"(lo.x), "r"(hi.x), "r"(lo.y), "r"(hi.y), "r"(bv.x), "r"(bv.y));
              asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                           : "+f"(d[mt][0]), "+f"(d[mt][1]), "+f"(d[mt][2]), "+f"(d[mt][3])
                           : "r"(lo.z), "r"(hi.z), "r"(lo.w), "r"(hi.w), "r"(bv.z), "r"(bv.w));
            }
          }
        }
        __syncthreads();                                     // `part` free again (previous block of experts)
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int tok = 2 * tq + (i & 1), el = 16 * mt + 8 * (i >> 1) + g;
            if (tok < TPC) part[(warp * TPC + tok) * 32 + el] = d[mt][i];
          }
        __syncthreads();
        for (int i = threadIdx.x; i < TPC * 32; i += kGateThreads) {
          const int t = i >> 5, el = i & 31;
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) v += part[(w * TPC + t) * 32 + el];
          if (t < nt && eb + el < e_hi) {
            ST r;
            store_scalar(&r, v);          // the logits reach the router in the Scalar type
            cluster_map(lgs, static_cast<unsigned>(t % C))[(t / C) * p.E + eb + el] = to_f32(r);
          }
        }
      }
    } else
    for (int eb = e_lo; eb < e_hi; eb += 32) {
      const int e = eb + lane;
      const bool live = e < e_hi;
      const ST* row = rw + static_cast<size_t>(live ? e : eb) * p.ldr + k_lo;
      float2 acc[TPC];
#pragma unroll
      for (int t = 0; t < TPC; ++t) acc[t] = make_float2(0.f, 0.f);
      for (int k = 0; k < kw; k += 32) {
        float wv[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) load8<ST>(row, static_cast<size_t>(k + 8 * u < kw ? k + 8 * u : k), true, wv[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (k + 8 * u >= kw) break;
#pragma unroll
          for (int t = 0; t < TPC; ++t) {
            const float4 xa = *reinterpret_cast<const float4*>(xs + t * p.H + k_lo + k + 8 * u);
            const float4 xb = *reinterpret_cast<const float4*>(xs + t * p.H + k_lo + k + 8 * u + 4);
            float2 a = acc[t];
            a = ffma2(make_float2(wv[u][0], wv[u][1]), make_float2(xa.x, xa.y), a);
            a = ffma2(make_float2(wv[u][2], wv[u][3]), make_float2(xa.z, xa.w), a);
            a = ffma2(make_float2(wv[u][4], wv[u][5]), make_float2(xb.x, xb.y), a);
            a = ffma2(make_float2(wv[u][6], wv[u][7]), make_float2(xb.z, xb.w), a);
            acc[t] = a;
          }
        }
      }
      __syncthreads();                                       // `part` free again (previous block of experts)
#pragma unroll
      for (int t = 0; t < TPC; ++t) part[(warp * TPC + t) * 32 + lane] = acc[t].x + acc[t].y;
      __syncthreads();
      for (int i = threadIdx.x; i < TPC * 32; i += kGateThreads) {
        const int t = i >> 5, el = i & 31;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) v += part[(w * TPC + t) * 32 + el];
        if (t < nt && eb + el < e_hi) {
          ST r;
          store_scalar(&r, v);          // the logits reach the router in the Scalar type
          cluster_map(lgs, static_cast<unsigned>(t % C))[(t / C) * p.E + eb + el] = to_f32(r);
        }
      }
    }
  }
  cluster_sync_all();
  // ---- routing: one warp per token of this CTA (cluster token crank + C * warp) ----
  const ST* bias = static_cast<const ST*>(p.bias);
  const int my_tokens = nt > static_cast<int>(crank) ? (nt - static_cast<int>(crank) + C - 1) / C : 0;
  if (warp < my_tokens) {
    const int tl = t_first + static_cast<int>(crank) + C * warp;   // local token index
    const int tg = p.rank * p.Tl + tl;                              // global token index
    const float* lgt = lgs + warp * p.E;
    int e = -1;
    float wk = 0.f;
    if (p.E <= 256 && p.top_k <= 32) {
      if (p.E <= 128)
        route_warp_regs<4>([&](int i) { return lgt[i]; }, [&](int i) { return to_f32(bias[i]); }, bias != nullptr, p.E,
                           p.top_k, p.norm_topk, p.routed_scale, p.sigmoid, lane, e, wk);
      else
        route_warp_regs<8>([&](int i) { return lgt[i]; }, [&](int i) { return to_f32(bias[i]); }, bias != nullptr, p.E,
                           p.top_k, p.norm_topk, p.routed_scale, p.sigmoid, lane, e, wk);
    } else {
      int32_t* my_idx = ridx + warp * p.top_k;
      float* my_w = rwts + warp * p.top_k;
      route_warp([&](int i) { return lgt[i]; }, [&](int i) { return to_f32(bias[i]); }, bias != nullptr, p.E, p.top_k,
                 p.norm_topk, p.routed_scale, p.sigmoid, score + warp * p.E, my_idx, my_w, lane);
      __syncwarp();
    }
    for (int k = lane; k < p.top_k; k += 32) {
      if (!(p.E <= 256 && p.top_k <= 32)) { e = ridx[warp * p.top_k + k]; wk = rwts[warp * p.top_k + k]; }
      const size_t slot = static_cast<size_t>(tg) * p.top_k + k;
      reinterpret_cast<float*>(p.region[p.rank] + p.L.wts)[slot] = wk;
      for (int r = 0; r < p.world; ++r) reinterpret_cast<int32_t*>(p.region[r] + p.L.idx)[slot] = e;
      if (e >= 0 && e < p.E) {
        // the slot takes the next row of its expert on the expert's owner
        const int owner = p.world > 1 ? e / p.e_per_rank : 0;
        const int el = e - (p.world > 1 ? owner * p.e_per_rank : p.e_first);
        if (el >= 0 && el < (p.world > 1 ? p.e_per_rank : p.e_count)) {
          int* cnt = reinterpret_cast<int*>(p.region[owner] + p.L.cnt) + el;
          const int rel = owner == p.rank ? atomicAdd(cnt, 1) : atomicAdd_system(cnt, 1);
          reinterpret_cast<int32_t*>(p.region[owner] + p.L.rel)[slot] = rel;
        }
      }
    }
  }
  // ---- per-32 quantization of this CTA's token rows (the reference's stage-1 quantizer), to every rank ----
  {
    const int nblk = p.H / 32, per_row = (nblk + 7) / 8, l4 = lane & 3;
    for (int it = warp; it < my_tokens * per_row; it += kGateThreads / 32) {
      const int tq = it / per_row, b = (it - tq * per_row) * 8 + (lane >> 2);
      const int tc = static_cast<int>(crank) + C * tq;   // token of the cluster
      float v[8];
      if (b < nblk) {
        const float4 a = *reinterpret_cast<const float4*>(xs + tc * p.H + b * 32 + l4 * 8);
        const float4 c = *reinterpret_cast<const float4*>(xs + tc * p.H + b * 32 + l4 * 8 + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      }
      float d;
      int part, total;
      const uint2 packed = quantize_block_lane8(v, d, part, total);
      if (b >= nblk) continue;
      const size_t row_off = p.L.xrows + static_cast<size_t>(p.rank * p.Tl + t_first + tc) * p.x_pitch;
      const float ds = __fmul_rn(static_cast<float>(total), d);
      for (int r = 0; r < p.world; ++r) {
        uint8_t* out = p.region[r] + row_off;
        reinterpret_cast<uint2*>(out + static_cast<size_t>(b) * 32)[l4] = packed;
        if (l4 == 0) {
          reinterpret_cast<ActHdr*>(out + act_hdr_offset(p.H))[b] = ActHdr{d, part, total - part, 0};
          reinterpret_cast<float2*>(out + act_bytes(p.H))[b] = make_float2(d, ds);
          store_sum_parts(out, act_parts_offset(static_cast<size_t>(p.H)), b, ds);
        }
      }
    }
  }
  // ---- the last CTA: tell the peers, wait for them, turn the counts into runs ----
  // every thread's stores are ordered at device scope before the CTA's barrier; one thread then extends the
  // order to system scope (the peers) before it takes the ticket -- a system-scope fence by every thread of
  // every CTA costs tens of microseconds
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (p.world > 1) __threadfence_system();
    s_last = atomicAdd(p.ticket, 1) == static_cast<int>(gridDim.x) - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (p.world > 1) {
    if (threadIdx.x < p.world && static_cast<int>(threadIdx.x) != p.rank)   // one thread per peer: the fences overlap
      st_release_sys(reinterpret_cast<uint32_t*>(p.region[threadIdx.x] + p.L.xflag) + p.rank, epoch);
    if (threadIdx.x < p.world && static_cast<int>(threadIdx.x) != p.rank) {
      if (!wait_epoch(reinterpret_cast<const uint32_t*>(p.region[p.rank] + p.L.xflag) + threadIdx.x, epoch, p.wait_ns))
        atomicExch(p.status, KDNN_ERR_DEVICE_WAIT);
    }
    __syncthreads();
  }
  // counts -> exclusive prefix sums (runs and 32-row groups), by one warp, 32 experts per step; the counts are
  // cleared for the next call (no peer touches them before this rank's down kernel of THIS call has signalled)
  int* starts = reinterpret_cast<int*>(gate_smem);   // [e_count + 1]  (the token rows are no longer needed)
  int* cnt = reinterpret_cast<int*>(p.region[p.rank] + p.L.cnt);
  const int n_slots = p.Tl * p.world * p.top_k;
  // the first 4 * 512 slots' expert and rank are fetched now, together with the counts: one trip to L2, not two
  const int32_t* idx = reinterpret_cast<const int32_t*>(p.region[p.rank] + p.L.idx);
  const int32_t* rel = reinterpret_cast<const int32_t*>(p.region[p.rank] + p.L.rel);
  int ev0[4], rv0[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = threadIdx.x + u * kGateThreads;
    ev0[u] = i < n_slots ? __ldcg(idx + i) - p.e_first : -1;
    rv0[u] = i < n_slots ? __ldcg(rel + i) : 0;
  }
  if (warp == 0) {
    int run = 0, grun = 0;
    int pre[8];   // the first 256 counts are fetched together
#pragma unroll
    for (int j = 0; j < 8; ++j) pre[j] = lane + 32 * j < p.e_count ? __ldcg(cnt + lane + 32 * j) : 0;
    for (int eb = 0; eb < p.e_count; eb += 32) {
      const int e = eb + lane;
      int c = 0;
      if (e < p.e_count) {
        int raw = 0;
        if (eb < 256) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j == (eb >> 5)) raw = pre[j];
        } else {
          raw = __ldcg(cnt + e);
        }
        c = min(max(raw, 0), n_slots);
        cnt[e] = 0;
      }
      const int gc = (c + kTcNT - 1) / kTcNT;
      int incl = c, gincl = gc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, o), gv = __shfl_up_sync(0xFFFFFFFFu, gincl, o);
        if (lane >= o) { incl += v; gincl += gv; }
      }
      if (e < p.e_count) {
        const int st = run + incl - c, g0 = grun + gincl - gc;
        starts[e] = st;
        p.offs[e] = st;
        for (int q = 0; q * kTcNT < c; ++q)
          p.groups[g0 + q] = make_int4(p.e_first + e, st + q * kTcNT, min(kTcNT, c - q * kTcNT), 0);
      }
      run += __shfl_sync(0xFFFFFFFFu, incl, 31);
      grun += __shfl_sync(0xFFFFFFFFu, gincl, 31);
    }
    if (lane == 0) {
      starts[p.e_count] = run;
      p.offs[p.e_count] = run;
      *p.n_groups = grun;
    }
  }
  __syncthreads();
  {
    const int total = starts[p.e_count];
    for (int i0 = threadIdx.x; i0 < n_slots; i0 += 4 * kGateThreads) {
      int ev[4], rv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kGateThreads;
        if (i0 == static_cast<int>(threadIdx.x)) {
          ev[u] = ev0[u]; rv[u] = rv0[u];
        } else {
          ev[u] = i < n_slots ? __ldcg(idx + i) - p.e_first : -1;
          rv[u] = i < n_slots ? __ldcg(rel + i) : 0;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kGateThreads;
        if (ev[u] >= 0 && ev[u] < p.e_count) {
          const int ps = starts[ev[u]] + rv[u];
          if (ps >= starts[ev[u]] && ps < starts[ev[u] + 1] && ps < total) {
            p.list[ps] = i;
            if (p.pos) p.pos[i] = ps;
          }
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *p.epoch = epoch;
    *p.ticket = 0;
  }
}

// Y[t,:] = sum over the slots of w * out[slot,:] (slots ascending, fp32, src/KokkosDNN_MoE.hpp:326-331; slots
// whose expert id is outside [0, E) or whose weight is zero are skipped, src/KokkosDNN_GGUF.hpp:2106-2110,
// :2205-2207), then optionally the residual add and the next block's un-scaled RMS norm
// (models/lfm2_5/KokkosDNN_LFM25Model.hpp:812-816, :770; src/KokkosDNN_RMSNorm.hpp:347-361):
//   h_out = Scalar(float(resid) + Y),  xn_out = Scalar(h_out / sqrt(mean(h_out^2) + eps)).
// One CTA per local token. With world > 1 the CTA first waits (bounded) for every rank's output flag.
struct CombineParams {
  const float* out[kMaxRanks];             // every rank's slot-indexed rows [T*S][H] (a slot's row lives on its expert's owner)
  const int32_t* idx; const float* wts;    // this rank's region, [T][S]
  const int* pos;                          // single rank: row of slot i is out[0] + pos[i] * H (null: row i)
  int stage_slots;                         // > 0: the slot rows come in as bulk copies (TMA, 1-D) into shared memory, this many at a time
  int Tl, S, H, e_lo, e_hi, e_per_rank, world, rank;   // slots of experts in [e_lo, e_hi) have a row; owner = e / e_per_rank
  const uint32_t* oflag; const uint32_t* epoch; int* status;
  unsigned long long wait_ns;
  float* y; size_t ldy;
  const void* resid; size_t ldres; void* h_out; size_t ldh; void* xn_out; size_t ldxn;
  float eps;
};
template <class ST>
__global__ void __launch_bounds__(512) moe_combine_norm_kernel(const CombineParams p) {
  pdl_chain_entry();
  extern __shared__ float comb_smem[];   // [H] the row after the residual add
  __shared__ float red[32];
  __shared__ int s_e[64];
  __shared__ float s_w[64];
  __shared__ int s_p[64];
  __shared__ __align__(8) unsigned long long s_bar;
  if (p.stage_slots > 0 && threadIdx.x == 0) {
    mbar_init(smem_u32(&s_bar), 1);
    fence_barrier_init();
  }
  const int t = blockIdx.x;
  const int tg = p.rank * p.Tl + t;
  const int32_t* idx = p.idx + static_cast<size_t>(tg) * p.S;
  const float* wts = p.wts + static_cast<size_t>(tg) * p.S;
  const bool cached = p.S <= 64;         // the token's routing (written by this rank's gate kernel) is read before the wait
  if (cached && static_cast<int>(threadIdx.x) < p.S) {
    s_e[threadIdx.x] = idx[threadIdx.x];
    s_w[threadIdx.x] = wts[threadIdx.x];
    s_p[threadIdx.x] = p.pos ? p.pos[static_cast<size_t>(tg) * p.S + threadIdx.x] : 0;
  }
  // all slots staged in one round: thread r waits for rank r's flag and requests that rank's rows at once, so the
  // transfers from the early ranks run under the wait for the late ones
  const bool eager = p.world > 1 && cached && p.stage_slots >= p.S && static_cast<int>(blockDim.x >> 5) >= p.world;
  if (eager) {
    __syncthreads();   // the routing is cached, the barrier is initialised
    const uint32_t bar = smem_u32(&s_bar);
    const uint32_t row_bytes = static_cast<uint32_t>(p.H) * 4u;
    if (threadIdx.x == 0) {
      int nlive = 0;
      for (int s = 0; s < p.S; ++s) nlive += (s_e[s] >= p.e_lo && s_e[s] < p.e_hi && s_w[s] != 0.0f);
      if (nlive > 0) mbar_expect_tx(bar, row_bytes * static_cast<uint32_t>(nlive));
    }
    __syncthreads();   // the bytes are expected before any warp can have them arrive
    if ((threadIdx.x & 31) == 0 && static_cast<int>(threadIdx.x >> 5) < p.world) {   // one WARP per rank: they do not wait for one another
      const int r = static_cast<int>(threadIdx.x >> 5);
      if (!wait_epoch(p.oflag + r, *p.epoch, p.wait_ns)) atomicExch(p.status, KDNN_ERR_DEVICE_WAIT);
      asm volatile("fence.proxy.async;" ::: "memory");        // the rows were published to the generic proxy
      float* rows = comb_smem + p.H;
      for (int s = 0; s < p.S; ++s) {
        const int e = s_e[s];
        if (e < p.e_lo || e >= p.e_hi || s_w[s] == 0.0f || e / p.e_per_rank != r) continue;
        bulk_g2s(smem_u32(rows + static_cast<size_t>(s) * p.H), p.out[r] + (static_cast<size_t>(tg) * p.S + s) * p.H,
                 row_bytes, bar);
      }
    }
  } else if (p.world > 1) {
    if (static_cast<int>(threadIdx.x) < p.world) {
      if (!wait_epoch(p.oflag + threadIdx.x, *p.epoch, p.wait_ns)) atomicExch(p.status, KDNN_ERR_DEVICE_WAIT);
    }
  }
  __syncthreads();
  // ---- the slot rows as bulk copies: one request per 8 KB row instead of 16 bytes per thread (rows that cross
  // NVLink arrive several times faster that way); sums in slot order, as below ----
  const int SC = cached ? p.stage_slots : 0;
  if (SC > 0) {
    float* rows = comb_smem + p.H;                            // [SC][H]
    const uint32_t bar = smem_u32(&s_bar);
    const uint32_t row_bytes = static_cast<uint32_t>(p.H) * 4u;
    for (int d = threadIdx.x * 4; d < p.H; d += blockDim.x * 4)
      *reinterpret_cast<float4*>(comb_smem + d) = make_float4(0.f, 0.f, 0.f, 0.f);
    uint32_t phase = 0;
    bool ok = true;
    for (int s0 = 0; s0 < p.S; s0 += SC) {
      int nlive = 0;
      for (int u = 0; u < SC && s0 + u < p.S; ++u) {
        const int e = s_e[s0 + u];
        nlive += (e >= p.e_lo && e < p.e_hi && s_w[s0 + u] != 0.0f);
      }
      if (nlive == 0) continue;                               // the same for every thread
      if (threadIdx.x == 0 && !eager) {
        asm volatile("fence.proxy.async;" ::: "memory");      // the rows were published to the generic proxy (flag acquire)
        mbar_expect_tx(bar, row_bytes * static_cast<uint32_t>(nlive));
        for (int u = 0; u < SC && s0 + u < p.S; ++u) {
          const int s = s0 + u, e = s_e[s];
          if (e < p.e_lo || e >= p.e_hi || s_w[s] == 0.0f) continue;
          const float* src = p.out[p.world > 1 ? e / p.e_per_rank : 0];
          const size_t rowi = p.pos ? static_cast<size_t>(s_p[s]) : static_cast<size_t>(tg) * p.S + s;
          bulk_g2s(smem_u32(rows + static_cast<size_t>(u) * p.H), src + rowi * p.H, row_bytes, bar);
        }
      }
      if (ok && !mbar_wait_bounded(bar, phase)) {
        ok = false;
        if (threadIdx.x == 0) atomicExch(p.status, KDNN_ERR_DEVICE_WAIT);
      }
      phase ^= 1u;
      for (int d = threadIdx.x * 4; d < p.H; d += blockDim.x * 4) {
        float4 acc = *reinterpret_cast<const float4*>(comb_smem + d);
        for (int u = 0; u < SC && s0 + u < p.S; ++u) {
          const int s = s0 + u, e = s_e[s];
          const float w = s_w[s];
          if (e < p.e_lo || e >= p.e_hi || w == 0.0f) continue;
          const float4 v = *reinterpret_cast<const float4*>(rows + static_cast<size_t>(u) * p.H + d);
          acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
        }
        *reinterpret_cast<float4*>(comb_smem + d) = acc;
      }
      if (s0 + SC < p.S) {                                    // the staging rows are overwritten by the next round
        __syncthreads();
        if (threadIdx.x == 0) fence_proxy_async();
      }
    }
  }
  const ST* resid = static_cast<const ST*>(p.resid);
  float ss = 0.f;
  for (int d = threadIdx.x * 4; d < p.H; d += blockDim.x * 4) {
    float4 acc = SC > 0 ? *reinterpret_cast<const float4*>(comb_smem + d) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; SC == 0 && s0 < p.S; s0 += 8) {   // plain loads: eight rows in flight, summed in slot order
      float4 v[8];
      float w[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int s = s0 + u;
        const int e = s < p.S ? (cached ? s_e[s] : idx[s]) : -1;
        w[u] = s < p.S ? (cached ? s_w[s] : wts[s]) : 0.0f;
        if (e < p.e_lo || e >= p.e_hi) w[u] = 0.0f;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (w[u] != 0.0f) {
          const float* src = p.out[p.world > 1 ? e / p.e_per_rank : 0];
          const size_t rowi = p.pos ? static_cast<size_t>(s_p[s & 63]) : static_cast<size_t>(tg) * p.S + s;
          v[u] = __ldcg(reinterpret_cast<const float4*>(src + rowi * p.H + d));
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (w[u] == 0.0f) continue;
        acc.x += w[u] * v[u].x; acc.y += w[u] * v[u].y; acc.z += w[u] * v[u].z; acc.w += w[u] * v[u].w;
      }
    }
    if (p.y) *reinterpret_cast<float4*>(p.y + static_cast<size_t>(t) * p.ldy + d) = acc;
    if (resid) {
      const float a[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ST r;
        store_scalar(&r, to_f32(resid[static_cast<size_t>(t) * p.ldres + d + i]) + a[i]);
        if (p.h_out) static_cast<ST*>(p.h_out)[static_cast<size_t>(t) * p.ldh + d + i] = r;
        const float v = to_f32(r);
        comb_smem[d + i] = v;
        ss += v * v;
      }
    }
  }
  if (!resid || !p.xn_out) return;
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = 1.0f / sqrtf(v / static_cast<float>(p.H) + p.eps);
  }
  __syncthreads();
  const float inv = red[0];
  for (int d = threadIdx.x; d < p.H; d += blockDim.x)
    store_scalar(static_cast<ST*>(p.xn_out) + static_cast<size_t>(t) * p.ldxn + d, comb_smem[d] * inv);
}

// Local (not peer-visible) workspace of the block call.
struct BlockWs {
  size_t offs, list, pos, groups, ngroups, act, actq, sync, region, total;
};
static BlockWs block_ws_layout(size_t T, size_t S, size_t H, size_t F, size_t n_experts, size_t region_bytes) {
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  BlockWs w{};
  size_t o = 0;
  w.offs = o; o += up((n_experts + 1) * sizeof(int));
  w.list = o; o += up(T * S * sizeof(int));
  w.pos  = o; o += up(T * S * sizeof(int));
  w.groups = o; o += up((n_experts + T * S / kTcNT + 1) * sizeof(int4));
  w.ngroups = o; o += 256;
  w.act  = o; o += up(T * S * F * sizeof(float));
  w.actq = o; o += up(T * S * act_row_pitch(F));
  w.sync = o; o += 256;          // gate ticket, down ticket, epoch
  w.region = o; o += region_bytes;
  w.total = o;
  return w;
}
size_t moe_block_workspace_bytes(size_t tokens_local, size_t world, size_t S, size_t H, size_t F, size_t n_experts,
                                 int with_region) {
  const size_t T = tokens_local * world;
  return block_ws_layout(T, S, H, F, n_experts, with_region ? moe_exchange_bytes(tokens_local, world, S, H) : 0).total;
}


cudaError_t moe_block_launch(const BlockArgs& a, cudaStream_t st) {
  const size_t H = a.gate->cols, F = a.gate->rows, S = static_cast<size_t>(a.top_k), E = a.gate->n_experts;
  const size_t world = static_cast<size_t>(a.world), T = a.Tl * world;
  const ExLayout XL = ex_layout(a.Tl, world, S, H);
  const BlockWs L = block_ws_layout(T, S, H, F, E, a.regions ? 0 : XL.total);
  uint8_t* b = static_cast<uint8_t*>(a.ws);
  int* sync = reinterpret_cast<int*>(b + L.sync);
  int* status = nullptr;
  cudaError_t err = moe_status_ptr(&status);
  if (err != cudaSuccess) return err;
  uint8_t* regions[kMaxRanks] = {};
  for (size_t r = 0; r < world; ++r) regions[r] = a.regions ? static_cast<uint8_t*>(a.regions[r]) : b + L.region;
  uint8_t* mine = regions[a.rank];

  GateParams g{};
  g.x = a.x; g.ldx = a.ldx; g.rw = a.rw; g.ldr = a.ldr; g.bias = a.bias;
  g.Tl = (int)a.Tl; g.H = (int)H; g.E = (int)E; g.top_k = a.top_k; g.norm_topk = a.norm_topk; g.sigmoid = a.sigmoid;
  g.world = a.world; g.rank = a.rank; g.routed_scale = a.routed_scale;
  for (size_t r = 0; r < world; ++r) g.region[r] = regions[r];
  g.L = XL; g.x_pitch = act_row_pitch(H);
  g.e_per_rank = a.world > 1 ? (int)a.e_count : 0; g.e_first = (int)a.e_first; g.e_count = (int)a.e_count;
  g.offs = reinterpret_cast<int*>(b + L.offs); g.list = reinterpret_cast<int*>(b + L.list);
  g.groups = reinterpret_cast<int4*>(b + L.groups); g.n_groups = reinterpret_cast<int*>(b + L.ngroups);
  const bool by_position = a.world == 1 && S <= 64;   // where the down rows go, see below
  g.pos = by_position ? reinterpret_cast<int*>(b + L.pos) : nullptr;
  g.ticket = sync; g.epoch = reinterpret_cast<uint32_t*>(sync + 2); g.status = status; g.wait_ns = a.wait_ns;
  // tokens per cluster: about 128 CTAs whatever the token count (a CTA streams a quarter of the router matrix)
  int tpc = a.Tl >= 256 ? 8 : a.Tl >= 128 ? 4 : a.Tl >= 64 ? 2 : 1;
  auto gate_smem = [&](int n) {
    const size_t rt = (n + kGateCluster - 1) / kGateCluster;
    return std::max(((size_t)n * H + rt * (2 * E + 2 * S) + (size_t)(kGateThreads / 32) * n * 32) * sizeof(float),
                    (a.e_count + 1) * sizeof(int)) + (a.scalar == KDNN_BF16 ? 8 * (H + 32) * 2 : 0);
  };
  while (tpc > 1 && gate_smem(tpc) > 200 * 1024) tpc >>= 1;
  const size_t gsm = gate_smem(tpc);
  using GateKern = void (*)(const GateParams);
  const bool f32 = a.scalar == KDNN_F32;
  const GateKern gk = tpc == 8 ? (f32 ? moe_gate_kernel<float, 8> : moe_gate_kernel<__nv_bfloat16, 8>)
                    : tpc == 4 ? (f32 ? moe_gate_kernel<float, 4> : moe_gate_kernel<__nv_bfloat16, 4>)
                    : tpc == 2 ? (f32 ? moe_gate_kernel<float, 2> : moe_gate_kernel<__nv_bfloat16, 2>)
                               : (f32 ? moe_gate_kernel<float, 1> : moe_gate_kernel<__nv_bfloat16, 1>);
  if (gsm > 48 * 1024) {   // once per device and kernel, at the cap the token count is trimmed to above
    static SmemAttrOnce once[2][4];
    err = set_max_smem_once(once[f32][tpc == 8 ? 3 : tpc == 4 ? 2 : tpc == 2 ? 1 : 0], gk, 200 * 1024 + 8 * 1024);
    if (err != cudaSuccess) return err;
  }
  err = launch_chained_cluster(gk, dim3((unsigned)((a.Tl + tpc - 1) / tpc) * kGateCluster), dim3(kGateThreads), gsm,
                               kGateCluster, st, g);
  if (err != cudaSuccess) return err;

  // ---- expert tiles over all T tokens' slots, local experts ----
  PeerOut po{};
  // several ranks: rows by slot (the token owners find them without asking); one rank: rows by position in the
  // sorted list, as the tile kernels produce them (the scattered row pointers cost 6 us per block)
  po.out = by_position ? nullptr : reinterpret_cast<float*>(mine + XL.out);
  for (size_t r = 0; r < world; ++r) po.oflag[r] = reinterpret_cast<uint32_t*>(regions[r] + XL.oflag);
  po.world = a.world; po.rank = a.rank;
  po.ticket = a.world > 1 ? sync + 1 : nullptr;
  po.epoch = reinterpret_cast<const uint32_t*>(sync + 2);
  if (a.e_count > 0) {
    const int want = tile_kind() == 3 ? 1 : tile_kind();
    const int kind = (want == 2 && !tc_covers(a.gate, a.up, a.down)) || want == 0 ? 1 : want;
    const int n_slots = (int)(T * S);
    int* offs = reinterpret_cast<int*>(b + L.offs);
    int* list = reinterpret_cast<int*>(b + L.list);
    uint8_t* xrows = mine + XL.xrows;
    uint8_t* arows = b + L.actq;
    float* act = reinterpret_cast<float*>(b + L.act);
    if (kind == 2) {
      const int max_groups = (int)a.e_count + n_slots / kTcNT;
      TcParams t1{};
      t1.maps0 = static_cast<const CUtensorMap*>(a.gate->tma); t1.maps1 = static_cast<const CUtensorMap*>(a.up->tma);
      t1.N = (int)F; t1.K = (int)H; t1.tile_rows = 64; t1.row_tiles = (int)((F + 63) / 64);
      t1.groups = reinterpret_cast<const int4*>(b + L.groups); t1.n_groups = reinterpret_cast<const int*>(b + L.ngroups);
      t1.list = list; t1.S = (int)S; t1.xrows = xrows; t1.x_pitch = act_row_pitch(H);
      t1.dst = act; t1.ld_dst = F; t1.round_bf16 = a.scalar == KDNN_BF16; t1.qdst = arows; t1.q_pitch = act_row_pitch(F);
      t1.status = status;
      err = launch_grouped_tc<1, float>(t1, max_groups * t1.row_tiles, st);
      if (err != cudaSuccess) return err;
      TcParams t0{};
      t0.maps0 = static_cast<const CUtensorMap*>(a.down->tma);
      t0.N = (int)H; t0.K = (int)F; t0.tile_rows = 128; t0.row_tiles = (int)((H + 127) / 128);
      t0.groups = t1.groups; t0.n_groups = t1.n_groups; t0.list = list; t0.S = (int)S;
      t0.xrows = arows; t0.x_pitch = act_row_pitch(F); t0.dst = by_position ? mine + XL.out : nullptr; t0.ld_dst = H; t0.status = status; t0.po = po;
      err = launch_grouped_tc<0, float>(t0, max_groups * t0.row_tiles, st);
      if (err != cudaSuccess) return err;
    } else {
      MmaParams m1{};
      m1.w0 = a.gate->base; m1.w1 = a.up->base; m1.row_bytes = (int)a.gate->row_bytes;
      m1.N = (int)F; m1.K = (int)H; m1.offs = offs; m1.list = list; m1.S = (int)S; m1.g_first = (int)a.e_first;
      m1.xrows = xrows; m1.x_pitch = act_row_pitch(H); m1.dst = act; m1.ld_dst = F;
      m1.round_bf16 = a.scalar == KDNN_BF16; m1.status = status;
      const int mean_rows = (int)((T * S + E - 1) / E);
      // CTAs along z share an expert's 32-row passes. Routing is uneven (an expert may get several times the
      // mean), and a CTA without a pass leaves at once, so a small grid (few local experts) gets up to eight.
      const int row_ctas = (int)((F + 63) / 64 * a.e_count);
      const int passes_z = max(max(1, min(4, 1 + (2 * mean_rows) / 32)), min(8, 2048 / max(1, row_ctas)));
      m1.passes_z = passes_z; m1.qdst = arows; m1.q_pitch = act_row_pitch(F);
      err = launch_grouped_mma<1, float>(m1, (int)a.e_count, st);
      if (err != cudaSuccess) return err;
      MmaParams m0{};
      m0.w0 = a.down->base; m0.row_bytes = (int)a.down->row_bytes;
      m0.N = (int)H; m0.K = (int)F; m0.offs = offs; m0.list = list; m0.S = (int)S; m0.g_first = (int)a.e_first;
      m0.xrows = arows; m0.x_pitch = act_row_pitch(F); m0.dst = by_position ? mine + XL.out : nullptr; m0.ld_dst = H; m0.status = status;
      m0.passes_z = passes_z; m0.po = po;
      err = launch_grouped_mma<0, float>(m0, (int)a.e_count, st);
      if (err != cudaSuccess) return err;
    }
  }
  // ---- combine on the token owner ----
  CombineParams c{};
  for (size_t r = 0; r < world; ++r) c.out[r] = reinterpret_cast<const float*>(regions[r] + XL.out);
  c.e_per_rank = a.world > 1 ? (int)a.e_count : 1;
  c.pos = by_position ? reinterpret_cast<const int*>(b + L.pos) : nullptr;
  c.idx = reinterpret_cast<const int32_t*>(mine + XL.idx); c.wts = reinterpret_cast<const float*>(mine + XL.wts);
  c.Tl = (int)a.Tl; c.S = (int)S; c.H = (int)H; c.world = a.world; c.rank = a.rank;
  c.e_lo = a.world > 1 ? 0 : (int)a.e_first; c.e_hi = a.world > 1 ? (int)E : (int)(a.e_first + a.e_count);
  c.oflag = reinterpret_cast<const uint32_t*>(mine + XL.oflag); c.epoch = reinterpret_cast<const uint32_t*>(sync + 2);
  c.status = status; c.wait_ns = a.wait_ns;
  c.y = a.y; c.ldy = a.ldy; c.resid = a.resid; c.ldres = a.ldres; c.h_out = a.h_out; c.ldh = a.ldh;
  c.xn_out = a.xn_out; c.ldxn = a.ldxn; c.eps = a.eps;
  auto ck = a.scalar == KDNN_F32 ? moe_combine_norm_kernel<float> : moe_combine_norm_kernel<__nv_bfloat16>;
  const unsigned cthreads = (unsigned)std::min<size_t>(512, std::max<size_t>(a.world > 1 ? 256 : 128, (H / 4 + 31) / 32 * 32));
  // staged rows: as many slots at a time as fit next to the row itself (two CTAs per SM kept when they fit in half)
  size_t stage = std::min<size_t>(S, 8);
  while (stage > 0 && (1 + stage) * H * sizeof(float) > 200 * 1024) --stage;
  if (S > 64 || H % 4 != 0 || a.world == 1) stage = 0;   // local rows: plain loads by every thread are faster (6.5 against 13 us)
  c.stage_slots = (int)stage;
  const size_t csm = (1 + stage) * H * sizeof(float);
  if (csm > 48 * 1024) {
    static SmemAttrOnce once_f, once_b;
    err = set_max_smem_once(a.scalar == KDNN_F32 ? once_f : once_b, ck, 200 * 1024);
    if (err != cudaSuccess) return err;
  }
  return launch_chained(ck, dim3((unsigned)a.Tl), dim3(cthreads), csm, st, c);
}

void moe_block_routing(void* const* regions, int rank, void* ws, size_t Tl, size_t world, size_t S, size_t H, size_t F,
                       size_t E, const int32_t** idx, const float** wts) {
  const ExLayout XL = ex_layout(Tl, world, S, H);
  const BlockWs L = block_ws_layout(Tl * world, S, H, F, E, regions ? 0 : XL.total);
  uint8_t* mine = regions ? static_cast<uint8_t*>(regions[rank]) : static_cast<uint8_t*>(ws) + L.region;
  *idx = reinterpret_cast<const int32_t*>(mine + XL.idx);
  *wts = reinterpret_cast<const float*>(mine + XL.wts);
}

int moe_take_status() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_moe_status, sizeof(int));
  if (v != 0) cudaMemcpyToSymbol(g_moe_status, &zero, sizeof(int));
  return v;
}

}  // namespace kdnn
