// Shared device helpers for the sm_100a quantized-decode kernels: ggml block
// geometry, the per-32 int8 activation quantizer, and the mbarrier / bulk-copy
// (TMA 1-D) wrappers.
#pragma once
#include <stdlib.h>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/kdnn_b200.h"

namespace kdnn {

// ---- ggml block geometry --------------------------------------------------
// "Item" = 64 consecutive-in-the-format weight elements, the work one lane does
// per row: Q4_K one 32-byte nibble group (low nibbles = sub-block 2i, high
// nibbles = sub-block 2i+1), Q6_K one (128-chunk, half) slice (two ql windows
// sharing one qh window), Q8_0 two 34-byte blocks.
template <uint32_t DT>
struct Fmt;
template <>
struct Fmt<KDNN_GGML_Q4_K> {
  static constexpr int kBlockElems = 256, kBlockBytes = 144;
};
template <>
struct Fmt<KDNN_GGML_Q6_K> {
  static constexpr int kBlockElems = 256, kBlockBytes = 210;
};
template <>
struct Fmt<KDNN_GGML_Q8_0> {
  static constexpr int kBlockElems = 32, kBlockBytes = 34;
};

__host__ __device__ inline size_t row_bytes_of(uint32_t dt, size_t cols) {
  switch (dt) {
    case KDNN_GGML_Q8_0: return cols / 32 * 34;
    case KDNN_GGML_Q4_K: return cols / 256 * 144;
    case KDNN_GGML_Q5_K: return cols / 256 * 176;
    case KDNN_GGML_Q6_K: return cols / 256 * 210;
  }
  return 0;
}
__host__ __device__ inline bool block_aligned(uint32_t dt, size_t cols) {
  if (cols == 0 || cols % 32 != 0) return false;
  return dt == KDNN_GGML_Q8_0 ? true : cols % 256 == 0;
}

// Activation staging layout of the reference (int8 row, then 16-byte headers).
struct ActHdr {
  float d;
  int32_t sum_lo, sum_hi, pad;
};
__host__ __device__ inline size_t act_hdr_offset(size_t K) { return (K + 15) & ~size_t(15); }
__host__ __device__ inline size_t act_bytes(size_t K) {
  return K % 32 ? 0 : act_hdr_offset(K) + 16 * (K / 32);
}

// ---- scalar helpers ---------------------------------------------------------
__device__ __forceinline__ float h2f(uint32_t bits16) {
  // cvt.f32.f16 is exact for every fp16 value (subnormals, inf, nan payloads).
  return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void store_scalar(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_scalar(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// dp4a over one 16-byte window (four words each side).
__device__ __forceinline__ int dot16(const uint32_t (&w)[4], const int4& x, int acc) {
  acc = __dp4a(static_cast<int>(w[0]), x.x, acc);
  acc = __dp4a(static_cast<int>(w[1]), x.y, acc);
  acc = __dp4a(static_cast<int>(w[2]), x.z, acc);
  acc = __dp4a(static_cast<int>(w[3]), x.w, acc);
  return acc;
}

// dp4a with unsigned bytes on the weight side: lets the high nibbles of a packed Q4_K
// word be used in place (w & 0xF0F0F0F0 = 16 * nibble, bytes up to 240), the exact
// factor 16 is removed from the int32 sum afterwards.
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dot16_us(const uint32_t (&w)[4], const int4& x, int acc) {
  acc = dp4a_us(w[0], x.x, acc);
  acc = dp4a_us(w[1], x.y, acc);
  acc = dp4a_us(w[2], x.z, acc);
  acc = dp4a_us(w[3], x.w, acc);
  return acc;
}

// ---- per-32 int8 activation quantizer ---------------------------------------
// Eight lanes cooperate on one 32-element block (four elements each). Returns
// this lane's four quantized values packed into one word; d / part sums come
// back through references. All 32 lanes of the warp must call it together.
//   d = amax / 127 and inv = 127 / amax are IEEE divisions, q = rint(v * inv)
//   clamped to +-127: the same roundings as the reference's stage 1.
__device__ __forceinline__ uint32_t quantize_block_lane(const float (&v)[4], float& d,
                                                        int& part_sum, int& block_sum) {
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  d                = __fdiv_rn(amax, 127.0f);
  const float inv  = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
  uint32_t packed  = 0;
  int s            = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int q = __float2int_rn(__fmul_rn(v[i], inv));
    q     = max(-127, min(127, q));
    s += q;
    packed |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * i);
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  part_sum  = s;  // lanes 0-3 of the group: elements 0..15, lanes 4-7: 16..31
  block_sum = s + __shfl_xor_sync(0xffffffffu, s, 4);
  return packed;
}

// Four lanes cooperate on one 32-element block (eight elements each): half the
// per-block fixed cost (divisions, shuffles, addressing) of the eight-lane form.
// Returns the lane's eight quantized values as two words (elements 0-3, 4-7).
__device__ __forceinline__ uint2 quantize_block_lane8(const float (&v)[8], float& d, int& part_sum,
                                                      int& block_sum) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  d               = __fdiv_rn(amax, 127.0f);
  const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
  uint32_t w[2]   = {0u, 0u};
  int s           = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int q = __float2int_rn(__fmul_rn(v[i], inv));
    q     = max(-127, min(127, q));
    s += q;
    w[i >> 2] |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * (i & 3));
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  part_sum  = s;  // lanes 0-1 of the group: elements 0..15, lanes 2-3: 16..31
  block_sum = s + __shfl_xor_sync(0xffffffffu, s, 2);
  return make_uint2(w[0], w[1]);
}

template <class XT>
__device__ __forceinline__ void load8(const XT* x, size_t k, bool vec_ok, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* x, size_t k, bool vec_ok, float (&v)[8]) {
  if (vec_ok) {
    const float4 a = *reinterpret_cast<const float4*>(x + k);
    const float4 b = *reinterpret_cast<const float4*>(x + k + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = x[k + i];
  }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* x, size_t k, bool vec_ok,
                                                     float (&v)[8]) {
  if (vec_ok) {
    const uint4 t = *reinterpret_cast<const uint4*>(x + k);
    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i]     = __uint_as_float(u[i] << 16);
      v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(x[k + i]);
  }
}

template <class XT>
__device__ __forceinline__ void load4(const XT* x, size_t k, bool vec_ok, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* x, size_t k, bool vec_ok, float (&v)[4]) {
  if (vec_ok) {
    const float4 t = *reinterpret_cast<const float4*>(x + k);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = x[k + i];
  }
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* x, size_t k, bool vec_ok,
                                                     float (&v)[4]) {
  if (vec_ok) {
    const uint2 t = *reinterpret_cast<const uint2*>(x + k);
    v[0] = __uint_as_float(t.x << 16);
    v[1] = __uint_as_float(t.x & 0xFFFF0000u);
    v[2] = __uint_as_float(t.y << 16);
    v[3] = __uint_as_float(t.y & 0xFFFF0000u);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __bfloat162float(x[k + i]);
  }
}

// ---- mbarrier + bulk copy (TMA 1-D, one destination CTA) ----------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same probe with a suspend-time hint (ns): a thread whose phase is not complete is parked by the
// hardware for up to that long (it resumes at once when the phase completes) instead of coming back to
// spin -- a CTA with many waiting warps otherwise spends its issue slots on their polling loops.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` probes (each probe itself blocks for a
// hardware-defined slice), so a copy that never lands cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  uint32_t limit = (1u << 22)) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// global -> shared bulk copy completing on an mbarrier. Both addresses 16-byte
// aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start its
// prologue / wait for the previous kernel's memory before touching its outputs.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Both at the top of a kernel of a chain: the next kernel may be scheduled as soon as SM resources free up
// (it then sits in its own wait), and nothing of this kernel runs before everything earlier in the stream
// has completed and is visible. Without the launch attribute below both are no-ops.
__device__ __forceinline__ void pdl_chain_entry() {
  pdl_launch_dependents();
  pdl_wait();
}
// Programmatic dependent launch for the library's launches: on unless kdnn_b200_launch_chaining(0) was called
// (a caller that writes packed weights on the same stream right before a call needs it off, see kdnn_b200.h).
inline std::atomic<int>& pdl_flag() {
  static std::atomic<int> on{1};
  return on;
}
inline bool pdl_enabled() { return pdl_flag().load(std::memory_order_relaxed) != 0; }
// Launches a kernel that begins with pdl_chain_entry() (never one that does not: it would start early).
// `early` = false gives a plain launch: a grid of about one wave placed while the previous kernel still
// holds some SMs lands two CTAs on the free SMs and none on the busy ones, and stays that unbalanced.
template <class... KArgs, class... Args>
inline cudaError_t launch_chained_if(bool early, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = early && pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
// The same with a thread-block cluster of `cluster` CTAs along x (grid.x must be a multiple of it).
template <class... KArgs, class... Args>
inline cudaError_t launch_chained_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, unsigned cluster,
                                          cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
template <class... KArgs, class... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args&&... args) {
  return launch_chained_if(true, kern, grid, block, smem, st, static_cast<Args&&>(args)...);
}


// ---- expert-parallel exchange over peer memory ---------------------------------------------------
// Every rank owns one exchange region that its peers can write (plain stores over NVLink into the
// CONSUMER's memory; consumers only ever read their own memory). Flags are 32-bit epochs that only grow:
// a producer writes its data, then the epoch with release semantics at system scope; a consumer polls
// with acquire loads until the flag has reached the epoch it expects. Every poll loop is bounded by the
// global timer: a wait that runs out records KDNN_ERR_DEVICE_WAIT and the kernel carries on to its exit.
constexpr int kMaxRanks = 8;
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// true when *flag reached `epoch` within `limit_ns`
__device__ __forceinline__ bool wait_epoch(const uint32_t* flag, uint32_t epoch, unsigned long long limit_ns) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const unsigned long long t0 = global_timer_ns();
  while (global_timer_ns() - t0 < limit_ns) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
    __nanosleep(64);
  }
  return false;
}
// What the down-projection kernels of the MoE block need: where their rows go and whom to tell.
struct PeerOut {
  float* out;                   // THIS rank's slot-indexed output rows [all tokens * S][N] (the token owners read
                                // them from here); null = plain position-indexed dst
  uint32_t* oflag[kMaxRanks];   // every rank's "outputs of rank r are complete" flags [world]
  int world, rank;
  int* ticket;                  // grid-completion counter (this GPU), null when world == 1
  const uint32_t* epoch;        // this GPU's current epoch
};
// Called by every CTA of a down-projection kernel on its way out (all threads): the last CTA to arrive
// publishes this rank's epoch to every rank's flag array.
__device__ __forceinline__ void peer_out_finish(const PeerOut& po, unsigned total_ctas) {
  if (po.ticket == nullptr) return;
  __shared__ int s_fin;
  __threadfence();   // device scope by everybody, system scope by the threads that raise the flags
  __syncthreads();
  if (threadIdx.x == 0) {
    s_fin = atomicAdd(po.ticket, 1) == static_cast<int>(total_ctas) - 1;
    if (s_fin) *po.ticket = 0;
  }
  __syncthreads();
  // one thread per peer, so that the release fences run side by side: one thread storing to eight peers
  // in turn spent 2 us per peer
  if (s_fin && static_cast<int>(threadIdx.x) < po.world) {
    __threadfence();
    st_release_sys(po.oflag[threadIdx.x] + po.rank, *po.epoch);
  }
}
// Output row of slot `slot` (token-major slot id over ALL tokens) in this rank's buffer.
__device__ __forceinline__ float* peer_out_row(const PeerOut& po, int slot, int N) {
  return po.out + static_cast<size_t>(slot) * N;
}

// Arguments of one MoE block call (kdnn_capi.cu validates and fills them, kdnn_moe.cu launches).
struct BlockArgs {
  const void* x; size_t ldx; size_t Tl; int scalar;
  const void* rw; size_t ldr; const void* bias; int top_k, norm_topk, sigmoid; float routed_scale;
  const kdnn_b200_weight_table *gate, *up, *down;
  size_t e_first, e_count;
  const void* resid; size_t ldres; void* h_out; size_t ldh; void* xn_out; size_t ldxn; float eps;
  float* y; size_t ldy;
  int world, rank; void* const* regions;   // host array [world] of exchange regions (null: single GPU, region in the workspace)
  unsigned long long wait_ns;
  void* ws;
};

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to the (kernel, device) pair, so a host thread that
// moves to another device must set it there too: one bit per device, set on the first launch there.
struct SmemAttrOnce {
  std::atomic<unsigned long long> done{0};
};
template <class Kern>
inline cudaError_t set_max_smem_once(SmemAttrOnce& once, Kern kern, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned long long bit = 1ull << (dev & 63);
  if (once.done.load(std::memory_order_acquire) & bit) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) once.done.fetch_or(bit, std::memory_order_release);
  return e;
}

}  // namespace kdnn
