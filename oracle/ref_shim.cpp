// C entry points around the REFERENCE's own quantized-decode operators, compiled
// from the reference's header files where they lie (never copied) against the
// host stand-in in oracle/kokkos_standin/. Built by oracle/Makefile into
// oracle/_ref/libkdnn_ref.so.
//
// TEST INFRASTRUCTURE ONLY: this library is the parity checker and the timed
// CPU baseline. Nothing in the product path may load it.
//
// Every function below forwards to the reference operator named in its comment
// (paths are relative to the reference project root).
#include <Kokkos_Core.hpp>

#include "KokkosDNN_GGUF.hpp"
#include "KokkosDNN_GGUF_Synthetic.hpp"
#include "KokkosDNN_MoE.hpp"
#include "KokkosDNN_RMSNorm.hpp"
#include "KokkosDNN_SwiGLU.hpp"

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

namespace {
using Exec   = Kokkos::DefaultExecutionSpace;
using BHalf  = Kokkos::Experimental::bhalf_t;
namespace G  = KokkosDNN::Gguf;
namespace MV = KokkosDNN::Impl::GgufMvq;

thread_local std::string g_err;

template <class T>
using V1 = Kokkos::View<T*, Exec>;
template <class T>
using V2 = Kokkos::View<T**, Kokkos::LayoutRight, Exec>;
template <class T>
using V3 = Kokkos::View<T***, Kokkos::LayoutRight, Exec>;

G::QuantWeight<Exec> wrap_weight(uint32_t dtype, const uint8_t* w, size_t rows,
                                 size_t cols, size_t bytes) {
  G::QuantWeight<Exec> q;
  q.dtype = static_cast<G::GgmlType>(dtype);
  q.rows  = rows;
  q.cols  = cols;
  q.data  = V1<uint8_t>(const_cast<uint8_t*>(w), bytes);
  return q;
}

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::invalid_argument& e) {
    g_err = e.what();
    return -1;
  } catch (const std::exception& e) {
    g_err = e.what();
    return -2;
  }
}
}  // namespace

extern "C" {

const char* kref_last_error() { return g_err.c_str(); }

int kref_num_threads() {
#if defined(_OPENMP)
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void kref_set_num_threads(int n) {
#if defined(_OPENMP)
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

// src/KokkosDNN_GGUF.hpp:2496 quant_gemv_int8_scratch_bytes
size_t kref_int8_scratch_bytes(size_t K) {
  return G::quant_gemv_int8_scratch_bytes(K);
}

// src/KokkosDNN_GGUF.hpp:2522 quant_gemv_int8_supported (Scalar = float / bf16)
int kref_int8_supported(uint32_t dtype, size_t K, int bf16) {
  return bf16 ? G::quant_gemv_int8_supported<Exec, BHalf>(
                    static_cast<G::GgmlType>(dtype), K)
              : G::quant_gemv_int8_supported<Exec, float>(
                    static_cast<G::GgmlType>(dtype), K);
}

// src/KokkosDNN_GGUF.hpp:187 ggml_row_bytes (returns 0 instead of throwing)
size_t kref_row_bytes(uint32_t dtype, size_t cols) {
  try {
    return G::ggml_row_bytes(static_cast<G::GgmlType>(dtype), cols);
  } catch (...) {
    return 0;
  }
}

// src/KokkosDNN_GGUFGemvInt8.hpp:198 QuantizeActQ8Functor — stage 1 alone.
// x: K floats or K bf16 bit patterns; scratch: act_q8_bytes(K), 16-byte aligned.
int kref_quantize_act(const void* x, int bf16, size_t K, uint8_t* scratch) {
  return guarded([&] {
    int8_t* xq        = reinterpret_cast<int8_t*>(scratch);
    MV::ActQ8Hdr* xh  = reinterpret_cast<MV::ActQ8Hdr*>(scratch + MV::act_q8_hdr_offset(K));
    const int nblk    = static_cast<int>(K / 32);
    if (bf16) {
      MV::QuantizeActQ8Functor<Exec, BHalf> f{static_cast<const BHalf*>(x), xq, xh, nblk};
      for (int b = 0; b < nblk; ++b) f(b);
    } else {
      MV::QuantizeActQ8Functor<Exec, float> f{static_cast<const float*>(x), xq, xh, nblk};
      for (int b = 0; b < nblk; ++b) f(b);
    }
  });
}

// src/KokkosDNN_GGUFGemvInt8.hpp:468 gemv_int8_unit_dot — one unit's fp32 value
// for every (row, unit) of a packed matrix: out[row * nunits + c].
int kref_unit_values(int wd, const uint8_t* w, size_t rows, size_t cols,
                     size_t row_bytes, const uint8_t* scratch, float* out) {
  return guarded([&] {
    const int8_t* xq       = reinterpret_cast<const int8_t*>(scratch);
    const MV::ActQ8Hdr* xh = reinterpret_cast<const MV::ActQ8Hdr*>(
        scratch + MV::act_q8_hdr_offset(cols));
    const int nu = static_cast<int>(cols / 32);
    for (size_t r = 0; r < rows; ++r)
      for (int c = 0; c < nu; ++c) {
        const uint8_t* row = w + r * row_bytes;
        float v            = 0;
        switch (static_cast<MV::Wd>(wd)) {
          case MV::Wd::Q4K: v = MV::gemv_int8_unit_dot<Exec, MV::Wd::Q4K>(row, c, xq, xh); break;
          case MV::Wd::Q5K: v = MV::gemv_int8_unit_dot<Exec, MV::Wd::Q5K>(row, c, xq, xh); break;
          case MV::Wd::Q6K: v = MV::gemv_int8_unit_dot<Exec, MV::Wd::Q6K>(row, c, xq, xh); break;
          case MV::Wd::Q80: v = MV::gemv_int8_unit_dot<Exec, MV::Wd::Q80>(row, c, xq, xh); break;
        }
        out[r * (size_t)nu + (size_t)c] = v;
      }
  });
}

// src/KokkosDNN_GGUFGemvInt8.hpp:280 mvq_load_unit_window — the activation
// window of unit c, flattened as {w[0..7], sum0, sum1} int32 and {d0, d1} fp32.
int kref_unit_window(int wd, const uint8_t* scratch, size_t cols, int c,
                     int32_t* words10, float* d2) {
  return guarded([&] {
    const int8_t* xq       = reinterpret_cast<const int8_t*>(scratch);
    const MV::ActQ8Hdr* xh = reinterpret_cast<const MV::ActQ8Hdr*>(
        scratch + MV::act_q8_hdr_offset(cols));
    MV::Int8UnitWindow x{};
    switch (static_cast<MV::Wd>(wd)) {
      case MV::Wd::Q4K: x = MV::mvq_load_unit_window<Exec, MV::Wd::Q4K>(xq, xh, c); break;
      case MV::Wd::Q5K: x = MV::mvq_load_unit_window<Exec, MV::Wd::Q5K>(xq, xh, c); break;
      case MV::Wd::Q6K: x = MV::mvq_load_unit_window<Exec, MV::Wd::Q6K>(xq, xh, c); break;
      case MV::Wd::Q80: x = MV::mvq_load_unit_window<Exec, MV::Wd::Q80>(xq, xh, c); break;
    }
    for (int i = 0; i < 8; ++i) words10[i] = x.w[i];
    words10[8] = x.sum0;
    words10[9] = x.sum1;
    d2[0]      = x.d0;
    d2[1]      = x.d1;
  });
}

// src/KokkosDNN_IntDot.hpp:101 IntDot<ExecSpace>::dot4
int32_t kref_dot4(int32_t a, int32_t b, int32_t acc) {
  return KokkosDNN::Impl::IntDot<Exec>::dot4(a, b, acc);
}

// src/KokkosDNN_GGUF.hpp:2531 quant_gemv(handle, x, w, y, act_scratch) — int8
// path when scratch != null and large enough, else
// src/KokkosDNN_GGUF.hpp:2394 quant_gemv(handle, x, w, y) — fp path.
// x, y are float or bf16 bit patterns according to `bf16`.
int kref_quant_gemv(uint32_t dtype, const uint8_t* w, size_t wbytes, size_t rows,
                    size_t cols, const void* x, void* y, int bf16,
                    uint8_t* scratch, size_t scratch_bytes) {
  return guarded([&] {
    KokkosDNN::DNNHandle<Exec> h;
    auto q = wrap_weight(dtype, w, rows, cols, wbytes);
    if (bf16) {
      V1<BHalf> xv(static_cast<BHalf*>(const_cast<void*>(x)), cols);
      V1<BHalf> yv(static_cast<BHalf*>(y), rows);
      if (scratch)
        G::quant_gemv(h, xv, q, yv, V1<uint8_t>(scratch, scratch_bytes));
      else
        G::quant_gemv(h, xv, q, yv);
    } else {
      V1<float> xv(static_cast<float*>(const_cast<void*>(x)), cols);
      V1<float> yv(static_cast<float*>(y), rows);
      if (scratch)
        G::quant_gemv(h, xv, q, yv, V1<uint8_t>(scratch, scratch_bytes));
      else
        G::quant_gemv(h, xv, q, yv);
    }
  });
}

// src/KokkosDNN_GGUF.hpp:2564 quant_gemm — Y[M,N] = X[M,K] W[N,K]^T (fp path).
int kref_quant_gemm(uint32_t dtype, const uint8_t* w, size_t wbytes, size_t rows,
                    size_t cols, const void* X, size_t M, void* Y, int bf16) {
  return guarded([&] {
    KokkosDNN::DNNHandle<Exec> h;
    auto q = wrap_weight(dtype, w, rows, cols, wbytes);
    if (bf16) {
      V2<BHalf> xv(static_cast<BHalf*>(const_cast<void*>(X)), M, cols);
      V2<BHalf> yv(static_cast<BHalf*>(Y), M, rows);
      G::quant_gemm(h, xv, q, yv);
    } else {
      V2<float> xv(static_cast<float*>(const_cast<void*>(X)), M, cols);
      V2<float> yv(static_cast<float*>(Y), M, rows);
      G::quant_gemm(h, xv, q, yv);
    }
  });
}

// src/KokkosDNN_GGUF.hpp:2839 dequant_to_dense
int kref_dequant_to_dense(uint32_t dtype, const uint8_t* w, size_t wbytes,
                          size_t rows, size_t cols, void* Y, int bf16) {
  return guarded([&] {
    auto q = wrap_weight(dtype, w, rows, cols, wbytes);
    if (bf16) {
      V2<BHalf> yv(static_cast<BHalf*>(Y), rows, cols);
      G::dequant_to_dense(q, yv);
    } else {
      V2<float> yv(static_cast<float*>(Y), rows, cols);
      G::dequant_to_dense(q, yv);
    }
  });
}

// src/KokkosDNN_MoE.hpp:240 moe_route / :280 moe_route_sigmoid
int kref_moe_route(const void* logits, int bf16, size_t T, size_t E,
                   const void* bias, size_t bias_len, int top_k, int norm_topk,
                   float routed_scale, int sigmoid, int* top_idx, float* top_w) {
  return guarded([&] {
    const size_t K = top_k < 0 ? 0 : static_cast<size_t>(top_k);
    V2<int> iv(top_idx, T, K);
    V2<float> wv(top_w, T, K);
    if (bf16) {
      V2<BHalf> lv(static_cast<BHalf*>(const_cast<void*>(logits)), T, E);
      V1<BHalf> bv(static_cast<BHalf*>(const_cast<void*>(bias)), bias_len);
      if (sigmoid)
        KokkosDNN::moe_route_sigmoid<Exec, BHalf>(lv, bv, top_k, norm_topk != 0, routed_scale, iv, wv);
      else
        KokkosDNN::moe_route<Exec, BHalf>(lv, bv, top_k, norm_topk != 0, routed_scale, iv, wv);
    } else {
      V2<float> lv(static_cast<float*>(const_cast<void*>(logits)), T, E);
      V1<float> bv(static_cast<float*>(const_cast<void*>(bias)), bias_len);
      if (sigmoid)
        KokkosDNN::moe_route_sigmoid<Exec, float>(lv, bv, top_k, norm_topk != 0, routed_scale, iv, wv);
      else
        KokkosDNN::moe_route<Exec, float>(lv, bv, top_k, norm_topk != 0, routed_scale, iv, wv);
    }
  });
}

// src/KokkosDNN_GGUF.hpp:2335 quant_moe_decode (one token, fp path) with
// src/KokkosDNN_GGUF.hpp:2031 make_quant_weight_table for the three tables.
// gate/up/down: arrays of n_experts payload pointers.
int kref_quant_moe_decode(const void* X, int bf16, size_t K, size_t MI,
                          size_t n_experts, uint32_t gdtype, uint32_t udtype,
                          uint32_t ddtype, const uint8_t* const* gate,
                          const uint8_t* const* up, const uint8_t* const* down,
                          const int* idx, const float* wts, size_t S, void* act,
                          void* Y) {
  return guarded([&] {
    KokkosDNN::DNNHandle<Exec> h;
    auto rb = [](uint32_t dt, size_t cols) {
      return G::ggml_row_bytes(static_cast<G::GgmlType>(dt), cols);
    };
    std::vector<G::QuantWeight<Exec>> g, u, d;
    for (size_t e = 0; e < n_experts; ++e) {
      g.push_back(wrap_weight(gdtype, gate[e], MI, K, MI * rb(gdtype, K)));
      u.push_back(wrap_weight(udtype, up[e], MI, K, MI * rb(udtype, K)));
      d.push_back(wrap_weight(ddtype, down[e], K, MI, K * rb(ddtype, MI)));
    }
    auto tg = G::make_quant_weight_table(g, "gate");
    auto tu = G::make_quant_weight_table(u, "up");
    auto td = G::make_quant_weight_table(d, "down");
    V2<int> iv(const_cast<int*>(idx), 1, S);
    V2<float> wv(const_cast<float*>(wts), 1, S);
    if (bf16) {
      V2<BHalf> xv(static_cast<BHalf*>(const_cast<void*>(X)), 1, K);
      V2<BHalf> av(static_cast<BHalf*>(act), S, MI);
      V2<BHalf> yv(static_cast<BHalf*>(Y), 1, K);
      G::quant_moe_decode<Exec, BHalf>(h, xv, tg, tu, td, iv, wv, av, yv);
    } else {
      V2<float> xv(static_cast<float*>(const_cast<void*>(X)), 1, K);
      V2<float> av(static_cast<float*>(act), S, MI);
      V2<float> yv(static_cast<float*>(Y), 1, K);
      G::quant_moe_decode<Exec, float>(h, xv, tg, tu, td, iv, wv, av, yv);
    }
  });
}

// src/KokkosDNN_MoE.hpp:313 moe_expert_weighted_sum
int kref_moe_weighted_sum(const void* expert_out, const float* top_w, size_t T,
                          size_t K, size_t D, void* y, int bf16) {
  return guarded([&] {
    V2<float> wv(const_cast<float*>(top_w), T, K);
    if (bf16) {
      V3<BHalf> ev(static_cast<BHalf*>(const_cast<void*>(expert_out)), T, K, D);
      V2<BHalf> yv(static_cast<BHalf*>(y), T, D);
      KokkosDNN::moe_expert_weighted_sum<Exec, BHalf>(ev, wv, yv);
    } else {
      V3<float> ev(static_cast<float*>(const_cast<void*>(expert_out)), T, K, D);
      V2<float> yv(static_cast<float*>(y), T, D);
      KokkosDNN::moe_expert_weighted_sum<Exec, float>(ev, wv, yv);
    }
  });
}

// src/KokkosDNN_MoE.hpp:337 moe_gather_rows
int kref_moe_gather_rows(const void* src, size_t C, size_t D, const int* rows,
                         size_t N, void* dst, int bf16) {
  return guarded([&] {
    V1<int> rv(const_cast<int*>(rows), N);
    if (bf16) {
      V2<BHalf> sv(static_cast<BHalf*>(const_cast<void*>(src)), C, D);
      V2<BHalf> dv(static_cast<BHalf*>(dst), N, D);
      KokkosDNN::moe_gather_rows<Exec, BHalf>(sv, rv, dv);
    } else {
      V2<float> sv(static_cast<float*>(const_cast<void*>(src)), C, D);
      V2<float> dv(static_cast<float*>(dst), N, D);
      KokkosDNN::moe_gather_rows<Exec, float>(sv, rv, dv);
    }
  });
}

// src/KokkosDNN_MoE.hpp:360 moe_scatter_add_weighted
int kref_moe_scatter_add_weighted(const void* src, size_t N, size_t D,
                                  const int* rows, const float* weights,
                                  void* dst, size_t C, int bf16) {
  return guarded([&] {
    V1<int> rv(const_cast<int*>(rows), N);
    V1<float> wv(const_cast<float*>(weights), N);
    if (bf16) {
      V2<BHalf> sv(static_cast<BHalf*>(const_cast<void*>(src)), N, D);
      V2<BHalf> dv(static_cast<BHalf*>(dst), C, D);
      KokkosDNN::moe_scatter_add_weighted<Exec, BHalf>(sv, rv, wv, dv);
    } else {
      V2<float> sv(static_cast<float*>(const_cast<void*>(src)), N, D);
      V2<float> dv(static_cast<float*>(dst), C, D);
      KokkosDNN::moe_scatter_add_weighted<Exec, float>(sv, rv, wv, dv);
    }
  });
}

// src/KokkosDNN_SwiGLU.hpp:12 silu
float kref_silu(float v) { return KokkosDNN::silu(v); }

// src/KokkosDNN_GGUF.hpp:201 fp16_to_float
float kref_fp16_to_float(uint16_t h) { return G::fp16_to_float(h); }

// src/KokkosDNN_GGUF.hpp:287 get_scale_min_k4
void kref_scale_min_k4(int j, const uint8_t* scales, uint8_t* sc, uint8_t* mn) {
  G::get_scale_min_k4(j, scales, sc, mn);
}

// src/KokkosDNN_GGUF.hpp:300/324/329/362 dequant_q4k/q80/q6k/q5k_block over a
// packed row of `cols` elements.
int kref_dequant_row(uint32_t dtype, const uint8_t* row, size_t cols, float* out) {
  return guarded([&] {
    switch (static_cast<G::GgmlType>(dtype)) {
      case G::GgmlType::Q4_K:
        for (size_t b = 0; b < cols / 256; ++b)
          G::dequant_q4k_block(reinterpret_cast<const G::BlockQ4K*>(row + b * 144), out + b * 256);
        break;
      case G::GgmlType::Q5_K:
        for (size_t b = 0; b < cols / 256; ++b)
          G::dequant_q5k_block(reinterpret_cast<const G::BlockQ5K*>(row + b * 176), out + b * 256);
        break;
      case G::GgmlType::Q6_K:
        for (size_t b = 0; b < cols / 256; ++b)
          G::dequant_q6k_block(reinterpret_cast<const G::BlockQ6K*>(row + b * 210), out + b * 256);
        break;
      case G::GgmlType::Q8_0:
        for (size_t b = 0; b < cols / 32; ++b)
          G::dequant_q80_block(reinterpret_cast<const G::BlockQ80*>(row + b * 34), out + b * 32);
        break;
      default: throw std::invalid_argument("kref_dequant_row: unsupported dtype");
    }
  });
}

// src/KokkosDNN_GGUF_Synthetic.hpp:49 write_synthetic_gguf — the reference's own container writer,
// driven with flat arrays: tensor t has n_dims[t] extents at dims[4*t..], payload raw[t] of raw_bytes[t].
int kref_gguf_write(const char* path, size_t n_tensors, const char* const* names, const uint32_t* dtypes,
                    const uint32_t* n_dims, const uint64_t* dims, const uint8_t* const* raw,
                    const size_t* raw_bytes, size_t n_str, const char* const* str_keys,
                    const char* const* str_vals, size_t n_f32, const char* const* f32_keys,
                    const float* f32_vals, size_t n_u32, const char* const* u32_keys,
                    const uint32_t* u32_vals) {
  return guarded([&] {
    std::vector<G::SyntheticTensor> ts(n_tensors);
    for (size_t t = 0; t < n_tensors; ++t) {
      ts[t].name  = names[t];
      ts[t].dtype = static_cast<G::GgmlType>(dtypes[t]);
      ts[t].dims.assign(dims + 4 * t, dims + 4 * t + n_dims[t]);
      ts[t].raw.assign(raw[t], raw[t] + raw_bytes[t]);
    }
    G::SyntheticKV kv;
    for (size_t i = 0; i < n_str; ++i) kv.strings[str_keys[i]] = str_vals[i];
    for (size_t i = 0; i < n_f32; ++i) kv.f32[f32_keys[i]] = f32_vals[i];
    for (size_t i = 0; i < n_u32; ++i) kv.u32[u32_keys[i]] = u32_vals[i];
    G::write_synthetic_gguf(path, ts, kv);
  });
}

// src/KokkosDNN_GGUF.hpp:462 GgufFile(path) + :516 find + :584 payload — the reference's own reader on
// a file. out8 = {dtype, n_dims, dims[0..3], offset, nbytes}; copies up to `cap` payload bytes.
int kref_gguf_read_tensor(const char* path, const char* name, uint64_t* out8, uint64_t* data_start,
                          uint8_t* payload, size_t cap) {
  return guarded([&] {
    G::GgufFile f(path);
    const G::GgufTensorInfo& ti = f.find(name);
    out8[0] = static_cast<uint64_t>(ti.dtype);
    out8[1] = ti.n_dims;
    for (uint32_t d = 0; d < 4; ++d) out8[2 + d] = d < ti.n_dims ? ti.dims[d] : 0;
    out8[6] = ti.offset;
    out8[7] = ti.nbytes;
    *data_start = f.data_start();
    const size_t n = cap < (size_t)ti.nbytes ? cap : (size_t)ti.nbytes;
    if (n) std::memcpy(payload, f.payload(ti), n);
  });
}

// src/KokkosDNN_GGUF.hpp:527/543/554 kv_string / kv_f32 / kv_u32. kind 0 string (into buf), 1 f32, 2 u32.
int kref_gguf_read_kv(const char* path, const char* key, int kind, char* buf, size_t cap, float* f32,
                      uint32_t* u32) {
  return guarded([&] {
    G::GgufFile f(path);
    if (kind == 0) {
      std::snprintf(buf, cap, "%s", f.kv_string(key).c_str());
    } else if (kind == 1) {
      *f32 = f.kv_f32(key);
    } else {
      *u32 = f.kv_u32(key);
    }
  });
}

// src/KokkosDNN_RMSNorm.hpp:347 rmsnorm_noscale: y = x / sqrt(mean(x^2) + eps), rows of a [T, D] view
int kref_rmsnorm_noscale(const void* x, int bf16, size_t T, size_t D, float eps, void* y) {
  return guarded([&] {
    if (bf16) {
      V2<BHalf> xv(static_cast<BHalf*>(const_cast<void*>(x)), T, D), yv(static_cast<BHalf*>(y), T, D);
      KokkosDNN::rmsnorm_noscale<Exec, BHalf>(xv, eps, yv);
    } else {
      V2<float> xv(static_cast<float*>(const_cast<void*>(x)), T, D), yv(static_cast<float*>(y), T, D);
      KokkosDNN::rmsnorm_noscale<Exec, float>(xv, eps, yv);
    }
  });
}

// src/KokkosDNN_SwiGLU.hpp:24 swiglu: out = Scalar(silu(gate) * up), [T, F]
int kref_swiglu(const void* gate, const void* up, int bf16, size_t T, size_t F, void* out) {
  return guarded([&] {
    if (bf16) {
      V2<BHalf> g(static_cast<BHalf*>(const_cast<void*>(gate)), T, F), u(static_cast<BHalf*>(const_cast<void*>(up)), T, F),
          o(static_cast<BHalf*>(out), T, F);
      KokkosDNN::swiglu<Exec, BHalf>(g, u, o);
    } else {
      V2<float> g(static_cast<float*>(const_cast<void*>(gate)), T, F), u(static_cast<float*>(const_cast<void*>(up)), T, F),
          o(static_cast<float*>(out), T, F);
      KokkosDNN::swiglu<Exec, float>(g, u, o);
    }
  });
}

}  // extern "C"
