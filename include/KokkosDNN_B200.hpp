// C++ layer that keeps the reference library's operator signatures
// (Kokkos::View in and out, QuantWeight / QuantWeightTable, DNNHandle, exceptions
// for bad arguments, `false` for a declined fast path) on top of the C ABI in
// kdnn_b200.h.
//
// Every template below is duck-typed on the view / weight classes: it needs only
// `data()`, `extent(i)`, `stride(i)` from views and the public fields of
// Gguf::QuantWeight (`data`, `dtype`, `rows`, `cols`) and Gguf::QuantWeightTable
// (`base`, `dtype`, `rows`, `cols`, `row_bytes`, `size()`), so the same header
// compiles inside the reference library (real Kokkos, ExecSpace = Kokkos::Cuda)
// and against a test stand-in. Paths in comments are relative to the reference
// project root.
//
// Stream: the reference launches on the default instance of ExecSpace. Pass that
// instance's stream (Kokkos::Cuda().cuda_stream()) through `StreamOf`, or rely on
// the default (the legacy default stream, which is what a default-constructed
// Kokkos::Cuda uses unless Kokkos was initialised with its own stream).
#ifndef KOKKOSDNN_B200_HPP
#define KOKKOSDNN_B200_HPP

#include <climits>
#include <cstddef>
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include <cuda_runtime.h>
#if defined(KDNN_B200_NVTX)
#include <nvtx3/nvToolsExt.h>
#endif

#include "kdnn_b200.h"

namespace KokkosDNN {
namespace B200 {

// Scalar -> C ABI tag. float and any 2-byte type (Kokkos::Experimental::bhalf_t on
// a CUDA build is __nv_bfloat16) are accepted; everything else declines.
template <class Scalar>
constexpr int scalar_tag() {
  return std::is_same<Scalar, float>::value ? KDNN_F32 : (sizeof(Scalar) == 2 ? KDNN_BF16 : -1);
}

// Where the launches go. Specialise / overload for your execution space; the
// default is the legacy default stream.
template <class ExecSpace>
struct StreamOf {
  static void* get(const ExecSpace&) { return nullptr; }
};
#if defined(KOKKOS_ENABLE_CUDA)
template <>
struct StreamOf<Kokkos::Cuda> {
  static void* get(const Kokkos::Cuda& e) { return static_cast<void*>(e.cuda_stream()); }
};
#endif

inline void throw_on_error(int rc, const char* what) {
  if (rc == KDNN_ERR_INVALID) throw std::invalid_argument(kdnn_b200_last_error());
  if (rc < 0) throw std::runtime_error(std::string(what) + ": " + kdnn_b200_last_error());
}

// Gguf::quant_gemv_int8_scratch_bytes, src/KokkosDNN_GGUF.hpp:2496-2499
inline std::size_t quant_gemv_int8_scratch_bytes(std::size_t K) {
  return kdnn_b200_gemv_scratch_bytes(K);
}

// Gguf::quant_gemv_int8_supported, src/KokkosDNN_GGUF.hpp:2522-2529
template <class ExecSpace, class Scalar, class GgmlType>
inline bool quant_gemv_int8_supported(GgmlType dtype, std::size_t K) {
  return scalar_tag<Scalar>() >= 0 &&
         kdnn_b200_gemv_supported(static_cast<uint32_t>(dtype), K, scalar_tag<Scalar>()) != 0;
}

// Impl::GgufMvq::launch_quant_gemv_int8, src/KokkosDNN_GGUFGemvInt8.hpp:711-777.
// Same contract: returns false (nothing launched) when the fast path does not cover
// the call, so the caller keeps its portable kernel; never throws for a decline.
template <class ExecSpace, class XView, class YView>
bool launch_quant_gemv_int8(const ExecSpace& space, const XView& x, const std::uint8_t* wdata,
                            std::uint32_t ggml_type, std::size_t rows, std::size_t cols,
                            const YView& y, std::uint8_t* scratch, std::size_t scratch_bytes) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(x.data())>::type>::type;
  if (scalar_tag<Scalar>() < 0) return false;
  if (x.stride(0) != 1 || y.stride(0) != 1) return false;  // :730
  const int rc = kdnn_b200_quant_gemv(ggml_type, wdata, rows, cols, x.data(), scalar_tag<Scalar>(),
                                      y.data(), scalar_tag<Scalar>(), scratch, scratch_bytes,
                                      StreamOf<ExecSpace>::get(space));
  throw_on_error(rc, "quant_gemv");
  return rc == KDNN_OK;
}

// Gguf::quant_gemv(handle, x, w, y, act_scratch, label), src/KokkosDNN_GGUF.hpp:2531-2551.
// `fallback` is what the reference runs when the int8 path declines (its
// quant_gemv(handle, x, w, y, label)); it is called with no arguments.
template <class ExecSpace, class XView, class QuantWeight, class YView, class SView, class Fallback>
void quant_gemv(const ExecSpace& space, const XView& x, const QuantWeight& w, const YView& y,
                const SView& act_scratch, Fallback&& fallback) {
  if (x.extent(0) != w.cols || y.extent(0) != w.rows)
    throw std::invalid_argument("quant_gemv: dimension mismatch");  // :2538-2539
  if (w.rows == 0 || w.cols == 0) return;                          // :2541
  const std::size_t need = quant_gemv_int8_scratch_bytes(w.cols);
  if (need > 0 && act_scratch.extent(0) >= need &&
      launch_quant_gemv_int8(space, x, w.data.data(), static_cast<std::uint32_t>(w.dtype), w.rows,
                             w.cols, y, act_scratch.data(), act_scratch.extent(0)))
    return;
  fallback();
}

// The host's deep_copy(x_dev, x_host); quant_gemv(...); deep_copy(y_host, y_dev) around
// src/KokkosDNN_GGUF.hpp:2531-2551 as one call: x_host / y_host are host views (page-locked for the
// copies to be asynchronous), x_dev / y_dev / act_scratch device views. Returns false when the int8
// path declined (nothing was enqueued); y_host is valid once the space has been fenced.
template <class ExecSpace, class XHost, class QuantWeight, class YHost, class XView, class YView, class SView>
bool quant_gemv_host(const ExecSpace& space, const XHost& x_host, const QuantWeight& w, const YHost& y_host,
                     const XView& x_dev, const YView& y_dev, const SView& act_scratch) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(x_dev.data())>::type>::type;
  if (x_host.extent(0) != w.cols || y_host.extent(0) != w.rows || x_dev.extent(0) != w.cols ||
      y_dev.extent(0) != w.rows)
    throw std::invalid_argument("quant_gemv: dimension mismatch");
  if (w.rows == 0 || w.cols == 0) return true;
  if (scalar_tag<Scalar>() < 0) throw std::invalid_argument("quant_gemv: Scalar must be float or bhalf_t");
  const int rc = kdnn_b200_quant_gemv_host(static_cast<std::uint32_t>(w.dtype), w.data.data(), w.rows, w.cols,
                                           x_host.data(), scalar_tag<Scalar>(), y_host.data(), scalar_tag<Scalar>(),
                                           x_dev.data(), y_dev.data(), act_scratch.data(), act_scratch.extent(0),
                                           StreamOf<ExecSpace>::get(space));
  throw_on_error(rc, "quant_gemv_host");
  return rc == KDNN_OK;
}

// Several projections of ONE activation row in one call (the model's wgate / wup or wk / wv,
// models/glimmer/KokkosDNN_GlimmerModel.hpp:650-653, :523-526): ys[i] = ws[i] . x for matrices of one format and
// shape. `ws` and `ys` are any ranges of QuantWeight / views (std::array, std::vector, initializer_list).
// Returns false when the int8 path declined (nothing launched): the caller then makes its single calls.
template <class ExecSpace, class XView, class WRange, class YRange, class SView>
bool quant_gemv_multi(const ExecSpace& space, const XView& x, const WRange& ws, const YRange& ys,
                      const SView& act_scratch) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(x.data())>::type>::type;
  const void* wp[16];
  void* yp[16];
  std::size_t n = 0, rows = 0, cols = 0;
  std::uint32_t dtype = 0;
  for (const auto& w : ws) {
    if (n == 16) throw std::invalid_argument("quant_gemv_multi: at most 16 matrices per call");
    if (n == 0) { rows = w.rows; cols = w.cols; dtype = static_cast<std::uint32_t>(w.dtype); }
    if (w.rows != rows || w.cols != cols || static_cast<std::uint32_t>(w.dtype) != dtype)
      throw std::invalid_argument("quant_gemv_multi: matrices of one format and shape");
    wp[n++] = w.data.data();
  }
  std::size_t m = 0;
  for (const auto& y : ys) {
    if (m == n) break;
    if (y.extent(0) != rows) throw std::invalid_argument("quant_gemv_multi: dimension mismatch");
    if (y.stride(0) != 1) return false;
    yp[m++] = y.data();
  }
  if (m != n || x.extent(0) != cols) throw std::invalid_argument("quant_gemv_multi: dimension mismatch");
  if (n == 0 || rows == 0 || cols == 0) return true;
  if (scalar_tag<Scalar>() < 0 || x.stride(0) != 1) return false;
  const int rc = kdnn_b200_quant_gemv_multi(dtype, n, wp, rows, cols, x.data(), scalar_tag<Scalar>(), yp,
                                            scalar_tag<Scalar>(), act_scratch.data(), act_scratch.extent(0), nullptr,
                                            StreamOf<ExecSpace>::get(space));
  throw_on_error(rc, "quant_gemv_multi");
  return rc == KDNN_OK;
}

// Gguf::quant_gemv(handle, x, w, y) without staging (fp path), src/KokkosDNN_GGUF.hpp:2394-2493.
template <class ExecSpace, class XView, class QuantWeight, class YView>
void quant_gemv_fp(const ExecSpace& space, const XView& x, const QuantWeight& w, const YView& y) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(x.data())>::type>::type;
  if (x.extent(0) != w.cols || y.extent(0) != w.rows) throw std::invalid_argument("quant_gemv: dimension mismatch");
  if (w.rows == 0 || w.cols == 0) return;
  if (scalar_tag<Scalar>() < 0) throw std::invalid_argument("quant_gemv: Scalar must be float or bhalf_t");
  const int rc = kdnn_b200_quant_gemv_fp(static_cast<std::uint32_t>(w.dtype), w.data.data(), w.rows, w.cols, x.data(),
                                         scalar_tag<Scalar>(), y.data(), scalar_tag<Scalar>(),
                                         StreamOf<ExecSpace>::get(space));
  throw_on_error(rc, "quant_gemv_fp");
}

// Gguf::dequant_to_dense, src/KokkosDNN_GGUF.hpp:2839-2934.
template <class ExecSpace, class QuantWeight, class YView>
void dequant_to_dense(const ExecSpace& space, const QuantWeight& w, const YView& Y) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(Y.data())>::type>::type;
  if (Y.extent(0) != w.rows || Y.extent(1) != w.cols)
    throw std::invalid_argument("dequant_to_dense: dimension mismatch");
  if (w.rows == 0 || w.cols == 0) return;
  if (scalar_tag<Scalar>() < 0 || Y.stride(1) != 1)
    throw std::invalid_argument("dequant_to_dense: Y must be a LayoutRight float or bhalf_t view");
  const int rc = kdnn_b200_dequant_to_dense(static_cast<std::uint32_t>(w.dtype), w.data.data(), w.rows, w.cols,
                                            Y.data(), Y.stride(0), scalar_tag<Scalar>(),
                                            StreamOf<ExecSpace>::get(space));
  throw_on_error(rc, "dequant_to_dense");
}

// Gguf::quant_gemm, src/KokkosDNN_GGUF.hpp:2564-2593 (int8 activations per row).
// `workspace` is a caller-owned byte view of at least kdnn_b200_gemm_workspace_bytes(M, K).
template <class ExecSpace, class XView, class QuantWeight, class YView, class WsView, class Fallback>
void quant_gemm(const ExecSpace& space, const XView& X, const QuantWeight& w, const YView& Y,
                const WsView& workspace, Fallback&& fallback) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(X.data())>::type>::type;
  const std::size_t M = X.extent(0), K = X.extent(1), N = w.rows;
  if (w.cols != K || Y.extent(0) != M || Y.extent(1) != N)
    throw std::invalid_argument("quant_gemm: dimension mismatch");
  if (M == 0 || N == 0 || K == 0) return;
  if (M * N > static_cast<std::size_t>(INT_MAX)) throw std::invalid_argument("quant_gemm: M*N too large");
  int rc = KDNN_DECLINED;
  if (scalar_tag<Scalar>() >= 0 && X.stride(1) == 1 && Y.stride(1) == 1)
    rc = kdnn_b200_quant_gemm(static_cast<std::uint32_t>(w.dtype), w.data.data(), N, K, X.data(),
                              X.stride(0), M, scalar_tag<Scalar>(), Y.data(), Y.stride(0),
                              scalar_tag<Scalar>(), workspace.data(), workspace.extent(0),
                              StreamOf<ExecSpace>::get(space));
  throw_on_error(rc, "quant_gemm");
  if (rc == KDNN_DECLINED) fallback();
}

// KokkosDNN::moe_route / moe_route_sigmoid, src/KokkosDNN_MoE.hpp:240-304.
template <class ExecSpace, class LView, class BView, class IView, class WView>
void moe_route(const ExecSpace& space, const LView& logits, const BView& expert_bias, int top_k,
               bool norm_topk, float routed_scale, const IView& top_idx, const WView& top_w,
               bool sigmoid = false) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(logits.data())>::type>::type;
  const char* name    = sigmoid ? "moe_route_sigmoid" : "moe_route";
  const std::size_t T = logits.extent(0), E = logits.extent(1);
  const std::size_t K = top_k < 0 ? 0 : static_cast<std::size_t>(top_k);
  const bool have_bias = expert_bias.extent(0) != 0;
  if (have_bias && expert_bias.extent(0) != E)
    throw std::invalid_argument(std::string(name) + ": expert_bias extent must be E");
  if (top_idx.extent(0) != T || top_idx.extent(1) != K || top_w.extent(0) != T || top_w.extent(1) != K)
    throw std::invalid_argument(std::string(name) + ": output dimension mismatch");
  if (T == 0) return;
  if (top_k <= 0 || K > E) throw std::invalid_argument(std::string(name) + ": need 1 <= top_k <= E");
  static_assert(sizeof(Scalar) == 4 || sizeof(Scalar) == 2, "Scalar must be float or a 2-byte bfloat16");
  throw_on_error(kdnn_b200_moe_route(logits.data(), logits.stride(0), T, E, scalar_tag<Scalar>(),
                                     have_bias ? expert_bias.data() : nullptr, top_k, norm_topk ? 1 : 0,
                                     routed_scale, sigmoid ? 1 : 0, top_idx.data(), top_w.data(),
                                     StreamOf<ExecSpace>::get(space)),
                 name);
}

// Gguf::QuantWeightTable -> C struct (src/KokkosDNN_GGUF.hpp:2020-2029).
template <class Table>
kdnn_b200_weight_table table_of(const Table& t) {
  kdnn_b200_weight_table c;
  c.base      = reinterpret_cast<const uintptr_t*>(t.base.data());
  c.ggml_type = static_cast<std::uint32_t>(t.dtype);
  c.rows      = t.rows;
  c.cols      = t.cols;
  c.row_bytes = t.row_bytes;
  c.n_experts = t.size();
  c.tma       = nullptr;
  return c;
}

// Gguf::quant_moe_decode, src/KokkosDNN_GGUF.hpp:2335-2391, with the int8 activation
// numerics of the GEMV. Same argument checks and messages. `workspace`: caller-owned
// bytes, at least kdnn_b200_moe_workspace_bytes(1, S, K, MI, n_experts), 256-byte aligned.
template <class ExecSpace, class XView, class Table, class IView, class WView, class AView, class YView,
          class WsView>
void quant_moe_decode(const ExecSpace& space, const XView& X, const Table& gate, const Table& up,
                      const Table& down, const IView& idx, const WView& wts, const AView& act,
                      const YView& Y, const WsView& workspace) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(X.data())>::type>::type;
  if (X.extent(0) != 1 || Y.extent(0) != 1) throw std::invalid_argument("quant_moe_decode: expected one row");
  const std::size_t K = X.extent(1), MI = gate.rows;
  const std::size_t S = idx.extent(0) == 0 ? 0 : idx.extent(1);
  if (gate.cols != K || up.cols != K || up.rows != MI || down.rows != K || down.cols != MI ||
      Y.extent(1) != K)
    throw std::invalid_argument("quant_moe_decode: dimension mismatch");
  if (gate.size() == 0 || gate.size() != up.size() || gate.size() != down.size())
    throw std::invalid_argument("quant_moe_decode: expert table mismatch");
  if (idx.extent(0) != 1 || wts.extent(0) != 1 || wts.extent(1) != S)
    throw std::invalid_argument("quant_moe_decode: routing dimension mismatch");
  if (act.extent(0) < S || (S > 0 && act.extent(1) != MI))
    throw std::invalid_argument("quant_moe_decode: act scratch too small");
  if (S == 0 || K == 0 || MI == 0) return;
  const kdnn_b200_weight_table g = table_of(gate), u = table_of(up), d = table_of(down);
  throw_on_error(kdnn_b200_moe_ffn(X.data(), X.stride(0), 1, scalar_tag<Scalar>(), &g, &u, &d, idx.data(),
                                   wts.data(), S, Y.data(), Y.stride(0), scalar_tag<Scalar>(), 0,
                                   gate.size(), workspace.data(), workspace.extent(0),
                                   StreamOf<ExecSpace>::get(space)),
                 "quant_moe_decode");
}

// Batched form (T tokens): the device-side replacement of LFM2.5's
// moe_forward_sparse loop, models/lfm2_5/KokkosDNN_LFM25Model.hpp:441-547.
template <class ExecSpace, class XView, class Table, class IView, class WView, class YView, class WsView>
void moe_ffn(const ExecSpace& space, const XView& X, const Table& gate, const Table& up, const Table& down,
             const IView& idx, const WView& wts, const YView& Y, const WsView& workspace,
             std::size_t expert_first = 0, std::size_t expert_count = static_cast<std::size_t>(-1)) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(X.data())>::type>::type;
  const std::size_t T = X.extent(0), S = idx.extent(0) == 0 ? 0 : idx.extent(1);
  if (Y.extent(0) != T || Y.extent(1) != X.extent(1)) throw std::invalid_argument("moe_ffn: dimension mismatch");
  if (idx.extent(0) != T || wts.extent(0) != T || wts.extent(1) != S)
    throw std::invalid_argument("moe_ffn: routing dimension mismatch");
  const kdnn_b200_weight_table g = table_of(gate), u = table_of(up), d = table_of(down);
  if (expert_count == static_cast<std::size_t>(-1)) expert_count = gate.size() - expert_first;
  throw_on_error(kdnn_b200_moe_ffn(X.data(), X.stride(0), T, scalar_tag<Scalar>(), &g, &u, &d, idx.data(),
                                   wts.data(), S, Y.data(), Y.stride(0), scalar_tag<Scalar>(), expert_first,
                                   expert_count, workspace.data(), workspace.extent(0),
                                   StreamOf<ExecSpace>::get(space)),
                 "moe_ffn");
}


// The model's MoE block for a chunk of tokens in ONE call (router product, moe_route / moe_route_sigmoid, experts,
// residual add, the next block's un-scaled RMS norm; models/lfm2_5/KokkosDNN_LFM25Model.hpp:770-816):
//   h_out = h + MoE(x),  x_next = rmsnorm_noscale(h_out).
// x, h, h_out, x_next: [tokens, H] Scalar views; router_w [E, H]; router_bias [E] or a view of extent 0.
// `workspace`: caller-owned bytes, kdnn_b200_moe_block_workspace_bytes(tokens, 1, S, H, F, E, 1), 256-byte aligned,
// zeroed once; one workspace per stream. `exchange` (null: one GPU) as kdnn_b200.h describes.
// Returns false when the call is not covered (tables other than Q4_K): compose moe_route + moe_ffn instead.
template <class ExecSpace, class XView, class RView, class BView, class Table, class HView, class WsView>
bool moe_block(const ExecSpace& space, const XView& x, const RView& router_w, const BView& router_bias, int top_k,
               bool norm_topk, float routed_scale, bool sigmoid, const Table& gate, const Table& up, const Table& down,
               const HView& h, const HView& h_out, const XView& x_next, float eps, const WsView& workspace,
               const kdnn_b200_moe_exchange* exchange = nullptr, std::size_t expert_first = 0,
               std::size_t expert_count = static_cast<std::size_t>(-1), const void* tma_gate = nullptr,
               const void* tma_up = nullptr, const void* tma_down = nullptr) {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(x.data())>::type>::type;
  const std::size_t T = x.extent(0), H = x.extent(1);
  if (h.extent(0) != T || h.extent(1) != H || h_out.extent(0) != T || h_out.extent(1) != H ||
      x_next.extent(0) != T || x_next.extent(1) != H || router_w.extent(1) != H || router_w.extent(0) != gate.size())
    throw std::invalid_argument("moe_block: dimension mismatch");
  if (scalar_tag<Scalar>() < 0) throw std::invalid_argument("moe_block: Scalar must be float or bhalf_t");
  kdnn_b200_weight_table g = table_of(gate), u = table_of(up), d = table_of(down);
  g.tma = tma_gate; u.tma = tma_up; d.tma = tma_down;
  if (expert_count == static_cast<std::size_t>(-1)) expert_count = gate.size() - expert_first;
  const int rc = kdnn_b200_moe_block(x.data(), x.stride(0), T, scalar_tag<Scalar>(), router_w.data(), router_w.stride(0),
                                     router_bias.extent(0) ? router_bias.data() : nullptr, top_k, norm_topk ? 1 : 0,
                                     routed_scale, sigmoid ? 1 : 0, &g, &u, &d, expert_first, expert_count, nullptr, 0,
                                     h.data(), h.stride(0), h_out.data(), h_out.stride(0), x_next.data(),
                                     x_next.stride(0), eps, exchange, workspace.data(), workspace.extent(0),
                                     StreamOf<ExecSpace>::get(space));
  throw_on_error(rc, "moe_block");
  return rc == KDNN_OK;
}

// ---- the reference's own signatures -------------------------------------------------------------------
// Gguf::quant_gemv / quant_gemm / quant_moe_decode exactly as the reference declares them
// (src/KokkosDNN_GGUF.hpp:2531-2537, :2564-2570, :2335-2346): handle first, views, label last, no extra
// arguments. They are templates over the argument types, so they accept the reference's
// DNNHandle<ExecSpace>, Gguf::QuantWeight<ExecSpace>, Gguf::QuantWeightTable<ExecSpace> and Kokkos::View
// objects unchanged. What the C ABI needs beyond those arguments lives in a per-thread cache that grows on
// first use and is then reused (like the handle's lazily created members, src/KokkosDNN_Handle.hpp:186-193):
// the batched calls' workspace, and per weight table the TMA descriptors of its experts. A declined int8
// GEMV lands in this library's fp kernel (the reference lands in its own, :2550).
namespace Gguf {
namespace detail {

#if defined(KDNN_B200_NVTX)
struct Range {
  explicit Range(const std::string& label) { nvtxRangePushA(label.c_str()); }
  ~Range() { nvtxRangePop(); }
};
#else
struct Range {
  explicit Range(const std::string&) {}
};
#endif

// Device bytes that only grow; one buffer per host thread (a thread drives one stream at a time, as the
// reference's one-handle-per-thread rule has it).
inline void* workspace(std::size_t bytes) {
  struct Buf { void* p = nullptr; std::size_t n = 0; };
  static thread_local Buf b;
  if (bytes > b.n) {
    if (b.p) cudaFree(b.p);
    b.p = nullptr;
    b.n = 0;
    const std::size_t want = (bytes + (std::size_t(1) << 20)) & ~((std::size_t(1) << 20) - 1);
    if (cudaMalloc(&b.p, want) != cudaSuccess) throw std::runtime_error("KokkosDNN::B200: workspace allocation failed");
    cudaMemset(b.p, 0, want);
    b.n = want;
  }
  return b.p;
}

// TMA descriptors of a table's experts, built once per table (keyed by the device address of its pointer
// array: payloads never move after load, models/lfm2_5/KokkosDNN_LFM25Model.hpp:557-560).
template <class Table>
inline const void* table_tma(const Table& t) {
  static thread_local std::map<const void*, void*> cache;
  const void* key = t.base.data();
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  void* dev = nullptr;
  const std::size_t n = t.size();
  std::vector<std::uintptr_t> host(n);
  cudaMemcpy(host.data(), t.base.data(), n * sizeof(std::uintptr_t), cudaMemcpyDeviceToHost);
  std::vector<unsigned char> maps(kdnn_b200_weight_table_tma_bytes(n));
  if (kdnn_b200_weight_table_tma_encode(host.data(), static_cast<std::uint32_t>(t.dtype), t.rows, t.cols, n,
                                        maps.data()) == KDNN_OK &&
      cudaMalloc(&dev, maps.size()) == cudaSuccess)
    cudaMemcpy(dev, maps.data(), maps.size(), cudaMemcpyHostToDevice);
  cache[key] = dev;   // nullptr: no tensor-core descriptors for this table, the mma.sync kernel serves it
  return dev;
}

template <class Table>
inline kdnn_b200_weight_table table_c(const Table& t) {
  kdnn_b200_weight_table c = table_of(t);
  c.tma = table_tma(t);
  return c;
}

template <class Handle>
inline void* stream_of(const Handle&) { return nullptr; }   // the reference's quant ops ignore the handle and
                                                            // launch on the default instance (:2347, :2400, :2571)
}  // namespace detail

// src/KokkosDNN_GGUF.hpp:2531-2551
template <class Handle, class XView, class QuantWeight, class YView, class SView>
void quant_gemv(const Handle& handle, const XView& x, const QuantWeight& w, const YView& y, const SView& act_scratch,
                const std::string& label = "KokkosDNN::Gguf::quant_gemv") {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(x.data())>::type>::type;
  detail::Range range(label);
  if (x.extent(0) != w.cols || y.extent(0) != w.rows) throw std::invalid_argument("quant_gemv: dimension mismatch");
  if (w.rows == 0 || w.cols == 0) return;
  if (scalar_tag<Scalar>() < 0) throw std::invalid_argument("quant_gemv: Scalar must be float or bhalf_t");
  int rc = KDNN_DECLINED;
  if (x.stride(0) == 1 && y.stride(0) == 1)
    rc = kdnn_b200_quant_gemv(static_cast<std::uint32_t>(w.dtype), w.data.data(), w.rows, w.cols, x.data(),
                              scalar_tag<Scalar>(), y.data(), scalar_tag<Scalar>(), act_scratch.data(),
                              act_scratch.extent(0), detail::stream_of(handle));
  throw_on_error(rc, "quant_gemv");
  if (rc == KDNN_DECLINED)   // the staging-free path, as the reference falls back to its own
    throw_on_error(kdnn_b200_quant_gemv_fp(static_cast<std::uint32_t>(w.dtype), w.data.data(), w.rows, w.cols, x.data(),
                                           scalar_tag<Scalar>(), y.data(), scalar_tag<Scalar>(),
                                           detail::stream_of(handle)),
                   "quant_gemv");
}

// src/KokkosDNN_GGUF.hpp:2564-2593
template <class Handle, class XView, class QuantWeight, class YView>
void quant_gemm(const Handle& handle, const XView& X, const QuantWeight& w, const YView& Y,
                const std::string& label = "KokkosDNN::Gguf::quant_gemm") {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(X.data())>::type>::type;
  detail::Range range(label);
  const std::size_t M = X.extent(0), K = X.extent(1), N = w.rows;
  if (w.cols != K || Y.extent(0) != M || Y.extent(1) != N) throw std::invalid_argument("quant_gemm: dimension mismatch");
  if (M == 0 || N == 0 || K == 0) return;
  if (scalar_tag<Scalar>() < 0 || X.stride(1) != 1 || Y.stride(1) != 1)
    throw std::invalid_argument("quant_gemm: views must be LayoutRight float or bhalf_t");
  const std::size_t wsb = kdnn_b200_gemm_workspace_bytes(M, K);
  const int rc = kdnn_b200_quant_gemm(static_cast<std::uint32_t>(w.dtype), w.data.data(), N, K, X.data(), X.stride(0), M,
                                      scalar_tag<Scalar>(), Y.data(), Y.stride(0), scalar_tag<Scalar>(),
                                      detail::workspace(wsb), wsb, detail::stream_of(handle));
  throw_on_error(rc, "quant_gemm");
  if (rc == KDNN_DECLINED) throw std::invalid_argument("quant_gemm: unsupported dtype");   // :2573-2574
}

// src/KokkosDNN_GGUF.hpp:2335-2391 (int8 activation numerics, see kdnn_b200_moe_ffn)
template <class Handle, class XView, class Table, class IView, class WView, class AView, class YView>
void quant_moe_decode(const Handle& handle, const XView& X, const Table& gate, const Table& up, const Table& down,
                      const IView& idx, const WView& wts, const AView& act, const YView& Y,
                      const std::string& label = "KokkosDNN::Gguf::quant_moe_decode") {
  using Scalar = typename std::remove_cv<typename std::remove_pointer<decltype(X.data())>::type>::type;
  detail::Range range(label);
  if (X.extent(0) != 1 || Y.extent(0) != 1) throw std::invalid_argument("quant_moe_decode: expected one row");
  const std::size_t K = X.extent(1), MI = gate.rows;
  const std::size_t S = idx.extent(0) == 0 ? 0 : idx.extent(1);
  if (gate.cols != K || up.cols != K || up.rows != MI || down.rows != K || down.cols != MI || Y.extent(1) != K)
    throw std::invalid_argument("quant_moe_decode: dimension mismatch");
  if (gate.size() == 0 || gate.size() != up.size() || gate.size() != down.size())
    throw std::invalid_argument("quant_moe_decode: expert table mismatch");
  if (idx.extent(0) != 1 || wts.extent(0) != 1 || wts.extent(1) != S)
    throw std::invalid_argument("quant_moe_decode: routing dimension mismatch");
  if (act.extent(0) < S || (S > 0 && act.extent(1) != MI))
    throw std::invalid_argument("quant_moe_decode: act scratch too small");
  if (S == 0 || K == 0 || MI == 0) return;
  const kdnn_b200_weight_table g = detail::table_c(gate), u = detail::table_c(up), d = detail::table_c(down);
  const std::size_t wsb = kdnn_b200_moe_workspace_bytes(1, S, K, MI, gate.size());
  throw_on_error(kdnn_b200_moe_ffn(X.data(), X.stride(0), 1, scalar_tag<Scalar>(), &g, &u, &d, idx.data(), wts.data(), S,
                                   Y.data(), Y.stride(0), scalar_tag<Scalar>(), 0, gate.size(), detail::workspace(wsb),
                                   wsb, detail::stream_of(handle)),
                 "quant_moe_decode");
}

}  // namespace Gguf

}  // namespace B200
}  // namespace KokkosDNN

#endif  // KOKKOSDNN_B200_HPP
