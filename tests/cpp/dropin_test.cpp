// Drives the C++ drop-in layer (include/KokkosDNN_B200.hpp) the way the reference's
// own tests drive its operators (tests/Test_GGUF.cpp:849-932, tests/Test_MoE.cpp:
// 99-124, tests/Test_MoeDecode.cpp:423-455): Kokkos::View arguments, QuantWeight /
// QuantWeightTable structs, std::invalid_argument for bad arguments, fallback on a
// declined fast path. Views here are the host stand-in's View class wrapped around
// cudaMalloc'd memory; results are checked against the CPU checker
// (oracle/libkdnn_oracle.so). Exit code 0 = all checks passed.
#include <Kokkos_Core.hpp>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <array>
#include <vector>

#include "KokkosDNN_B200.hpp"

extern "C" {
size_t ko_act_q8_bytes(size_t K);
int ko_gemv_int8(uint32_t dtype, const uint8_t* w, size_t rows, size_t cols, const float* x, float* y,
                 uint8_t* scratch);
int ko_moe_route(const float* logits, size_t T, size_t E, const float* bias, int top_k, int norm_topk,
                 float routed_scale, int sigmoid, int* top_idx, float* top_w);
int ko_moe_ffn_int8(const float* X, size_t T, size_t H, size_t F, size_t n_experts, uint32_t gdt,
                    uint32_t udt, uint32_t ddt, const uint8_t* const* gate, const uint8_t* const* up,
                    const uint8_t* const* down, const int* idx, const float* wts, size_t S, int bf16,
                    float* Y, float* act_out);
}

namespace {
struct Dev {};  // execution-space tag of this test (launches go to the default stream)
template <class T> using V1 = Kokkos::View<T*, Dev>;
template <class T> using V2 = Kokkos::View<T**, Kokkos::LayoutRight, Dev>;
enum class GgmlType : uint32_t { Q8_0 = 8, Q4_K = 12, Q6_K = 14 };
struct QuantWeight { V1<uint8_t> data; GgmlType dtype; size_t rows, cols; };
struct QuantWeightTable {
  V1<uintptr_t> base; GgmlType dtype; size_t rows, cols, row_bytes;
  size_t size() const { return base.extent(0); }
};

int failures = 0;
#define CHECK(cond) do { if (!(cond)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); ++failures; } } while (0)

template <class T> T* dmalloc(size_t n) { void* p = nullptr; cudaMalloc(&p, (n ? n : 1) * sizeof(T)); return static_cast<T*>(p); }
template <class T> T* upload(const std::vector<T>& h) { T* d = dmalloc<T>(h.size()); cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice); return d; }
template <class T> std::vector<T> download(const T* d, size_t n) { std::vector<T> h(n); cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost); return h; }

// random payload with sanitized fp16 scales (tests/Test_GGUF.cpp:941-971)
std::vector<uint8_t> payload(GgmlType dt, size_t rows, size_t cols, uint32_t seed) {
  const size_t bs = dt == GgmlType::Q4_K ? 144 : dt == GgmlType::Q6_K ? 210 : 34;
  const size_t nb = cols / (dt == GgmlType::Q8_0 ? 32 : 256);
  std::vector<uint8_t> raw(rows * nb * bs);
  std::mt19937 rng(seed);
  for (auto& b : raw) b = (uint8_t)(rng() & 0xFF);
  const uint16_t small = 0x1400;
  for (size_t i = 0; i < rows * nb; ++i) {
    uint8_t* blk = raw.data() + i * bs;
    if (dt == GgmlType::Q6_K) std::memcpy(blk + 208, &small, 2);
    else { std::memcpy(blk, &small, 2); if (dt == GgmlType::Q4_K) std::memcpy(blk + 2, &small, 2); }
  }
  return raw;
}
float max_abs(const std::vector<float>& v) { float m = 0; for (float f : v) m = std::fmax(m, std::fabs(f)); return m; }
}  // namespace

int main() {
  namespace B = KokkosDNN::B200;
  Dev space;
  std::mt19937 rng(7);
  std::normal_distribution<float> nd(0.f, 1.f);

  // ---- quant_gemv: int8 path taken, result equals the checker; fallback on decline ----
  for (GgmlType dt : {GgmlType::Q4_K, GgmlType::Q6_K, GgmlType::Q8_0}) {
    const size_t N = 37, K = 2048;
    auto raw = payload(dt, N, K, 11);
    std::vector<float> x(K);
    for (auto& v : x) v = nd(rng);
    QuantWeight w{V1<uint8_t>(upload(raw), raw.size()), dt, N, K};
    V1<float> xv(upload(x), K), yv(dmalloc<float>(N), N);
    V1<uint8_t> scratch(dmalloc<uint8_t>(B::quant_gemv_int8_scratch_bytes(K)), B::quant_gemv_int8_scratch_bytes(K));
    bool fell_back = false;
    B::quant_gemv(space, xv, w, yv, scratch, [&] { fell_back = true; });
    cudaDeviceSynchronize();
    CHECK(!fell_back);
    std::vector<float> ref(N);
    std::vector<uint8_t> hs(ko_act_q8_bytes(K) + 64);
    uint8_t* hsa = hs.data() + ((64 - (reinterpret_cast<uintptr_t>(hs.data()) & 63)) & 63);
    ko_gemv_int8((uint32_t)dt, raw.data(), N, K, x.data(), ref.data(), hsa);
    auto got = download(yv.data(), N);
    float err = 0;
    for (size_t i = 0; i < N; ++i) err = std::fmax(err, std::fabs(got[i] - ref[i]));
    CHECK(err <= 1e-3f * max_abs(ref));
    CHECK(std::memcmp(download(scratch.data(), ko_act_q8_bytes(K)).data(), hsa, ko_act_q8_bytes(K)) == 0);
    // undersized staging must decline and run the caller's portable path (Test_GGUF.cpp:1026-1052)
    V1<uint8_t> tiny(scratch.data(), B::quant_gemv_int8_scratch_bytes(K) / 2);
    B::quant_gemv(space, xv, w, yv, tiny, [&] { fell_back = true; });
    CHECK(fell_back);
    // dimension mismatch throws before any launch (Test_GGUF.cpp:1253-1259)
    bool threw = false;
    try { V1<float> bad(xv.data(), K / 2); B::quant_gemv(space, bad, w, yv, scratch, [] {}); }
    catch (const std::invalid_argument&) { threw = true; }
    CHECK(threw);
    // host-resident activations: copy in, GEMV, copy out as one call; same bits as the device call
    {
      std::vector<float> yh(N, -1.f);
      V1<float> xh(x.data(), K), yhv(yh.data(), N), yd(dmalloc<float>(N), N);
      CHECK(B::quant_gemv_host(space, xh, w, yhv, xv, yd, scratch));
      cudaDeviceSynchronize();
      CHECK(std::memcmp(yh.data(), got.data(), N * sizeof(float)) == 0);
    }
    CHECK((B::quant_gemv_int8_supported<Dev, float>(dt, K)));
    CHECK(!(B::quant_gemv_int8_supported<Dev, double>(dt, K)));
  }
  CHECK(B::quant_gemv_int8_scratch_bytes(500) == 0);

  // ---- moe_route: ids exact, weights 1e-5 (Test_MoE.cpp:99-124) ----
  {
    const size_t T = 3, E = 6;
    std::vector<float> lg = {0.1f, 2.0f, -1.0f, 0.5f, 1.2f, -0.3f, 1.5f, 1.5f, 1.5f, -2.0f, 0.0f, 3.0f,
                             -0.5f, -0.2f, -0.8f, -0.1f, -1.5f, -0.4f};
    V2<float> lv(upload(lg), T, E);
    V1<float> bias;
    V2<int> iv(dmalloc<int>(T * 2), T, 2);
    V2<float> wv(dmalloc<float>(T * 2), T, 2);
    B::moe_route(space, lv, bias, 2, true, 1.0f, iv, wv);
    cudaDeviceSynchronize();
    std::vector<int> ri(T * 2);
    std::vector<float> rw(T * 2);
    ko_moe_route(lg.data(), T, E, nullptr, 2, 1, 1.0f, 0, ri.data(), rw.data());
    auto gi = download(iv.data(), T * 2);
    auto gw = download(wv.data(), T * 2);
    for (size_t i = 0; i < T * 2; ++i) { CHECK(gi[i] == ri[i]); CHECK(std::fabs(gw[i] - rw[i]) <= 1e-5f); }
    CHECK(gi[2] == 5 && gi[3] == 0);  // 3-way tie keeps the lowest id
    bool threw = false;
    try { B::moe_route(space, lv, bias, 7, true, 1.0f, iv, wv); } catch (const std::invalid_argument&) { threw = true; }
    CHECK(threw);
  }

  // ---- quant_gemv_multi: two projections of one row in one call, each equal to the checker ----
  {
    const size_t N = 130, K = 1024;
    auto r0 = payload(GgmlType::Q4_K, N, K, 51), r1 = payload(GgmlType::Q4_K, N, K, 52);
    std::vector<float> x(K);
    for (auto& v : x) v = nd(rng);
    std::array<QuantWeight, 2> ws = {QuantWeight{V1<uint8_t>(upload(r0), r0.size()), GgmlType::Q4_K, N, K},
                                     QuantWeight{V1<uint8_t>(upload(r1), r1.size()), GgmlType::Q4_K, N, K}};
    std::array<V1<float>, 2> ys = {V1<float>(dmalloc<float>(N), N), V1<float>(dmalloc<float>(N), N)};
    V1<float> xv(upload(x), K);
    V1<uint8_t> scratch(dmalloc<uint8_t>(B::quant_gemv_int8_scratch_bytes(K)), B::quant_gemv_int8_scratch_bytes(K));
    CHECK(B::quant_gemv_multi(space, xv, ws, ys, scratch));
    cudaDeviceSynchronize();
    std::vector<uint8_t> hs(ko_act_q8_bytes(K) + 64);
    uint8_t* hsa = hs.data() + ((64 - (reinterpret_cast<uintptr_t>(hs.data()) & 63)) & 63);
    for (int i = 0; i < 2; ++i) {
      std::vector<float> ref(N);
      ko_gemv_int8(12, i ? r1.data() : r0.data(), N, K, x.data(), ref.data(), hsa);
      auto got = download(ys[i].data(), N);
      float err = 0;
      for (size_t j = 0; j < N; ++j) err = std::fmax(err, std::fabs(got[j] - ref[j]));
      CHECK(err <= 1e-3f * max_abs(ref));
    }
    bool threw = false;
    try {
      std::array<V1<float>, 2> bad = {ys[0], V1<float>(ys[1].data(), N - 1)};
      B::quant_gemv_multi(space, xv, ws, bad, scratch);
    } catch (const std::invalid_argument&) { threw = true; }
    CHECK(threw);
  }

  // ---- quant_moe_decode: one token, dead slot, argument errors (Test_MoeDecode.cpp:368-455) ----
  {
    const size_t E = 3, H = 512, F = 256, S = 3;
    std::vector<std::vector<uint8_t>> g(E), u(E), d(E);
    std::vector<uintptr_t> gp(E), up(E), dp(E);
    std::vector<const uint8_t*> gh(E), uh(E), dh(E);
    for (size_t e = 0; e < E; ++e) {
      g[e] = payload(GgmlType::Q4_K, F, H, 100 + e); u[e] = payload(GgmlType::Q4_K, F, H, 200 + e);
      d[e] = payload(GgmlType::Q4_K, H, F, 300 + e);
      gp[e] = (uintptr_t)upload(g[e]); up[e] = (uintptr_t)upload(u[e]); dp[e] = (uintptr_t)upload(d[e]);
      gh[e] = g[e].data(); uh[e] = u[e].data(); dh[e] = d[e].data();
    }
    QuantWeightTable tg{V1<uintptr_t>(upload(gp), E), GgmlType::Q4_K, F, H, H / 256 * 144};
    QuantWeightTable tu{V1<uintptr_t>(upload(up), E), GgmlType::Q4_K, F, H, H / 256 * 144};
    QuantWeightTable td{V1<uintptr_t>(upload(dp), E), GgmlType::Q4_K, H, F, F / 256 * 144};
    std::vector<float> x(H);
    for (auto& v : x) v = nd(rng);
    std::vector<int> idx = {2, -1, 0};
    std::vector<float> wts = {0.5f, 0.3f, 0.2f};
    V2<float> X(upload(x), 1, H), Y(dmalloc<float>(H), 1, H), act(dmalloc<float>(S * F), S, F);
    V2<int> iv(upload(idx), 1, S);
    V2<float> wv(upload(wts), 1, S);
    const size_t wsb = kdnn_b200_moe_workspace_bytes(1, S, H, F, E);
    V1<uint8_t> ws(dmalloc<uint8_t>(wsb), wsb);
    B::quant_moe_decode(space, X, tg, tu, td, iv, wv, act, Y, ws);
    cudaDeviceSynchronize();
    std::vector<float> ref(H);
    ko_moe_ffn_int8(x.data(), 1, H, F, E, 12, 12, 12, gh.data(), uh.data(), dh.data(), idx.data(), wts.data(), S, 0,
                    ref.data(), nullptr);
    auto got = download(Y.data(), H);
    float err = 0;
    for (size_t i = 0; i < H; ++i) err = std::fmax(err, std::fabs(got[i] - ref[i]));
    CHECK(err <= 1e-3f * max_abs(ref));
    bool threw = false;
    try { V2<float> X2(X.data(), 2, H / 2); B::quant_moe_decode(space, X2, tg, tu, td, iv, wv, act, Y, ws); }
    catch (const std::invalid_argument&) { threw = true; }
    CHECK(threw);
    threw = false;
    try { V2<float> small(act.data(), 1, F); B::quant_moe_decode(space, X, tg, tu, td, iv, wv, small, Y, ws); }
    catch (const std::invalid_argument&) { threw = true; }
    CHECK(threw);
  }
  // ---- moe_block: router + experts + residual + norm in one call; the experts' part against the checker fed with
  // the routing the block produced ----
  {
    const size_t E = 4, H = 512, F = 256, S = 2, T = 5;
    std::vector<std::vector<uint8_t>> g(E), u(E), d(E);
    std::vector<uintptr_t> gp(E), up(E), dp(E);
    std::vector<const uint8_t*> gh(E), uh(E), dh(E);
    for (size_t e = 0; e < E; ++e) {
      g[e] = payload(GgmlType::Q4_K, F, H, 400 + e); u[e] = payload(GgmlType::Q4_K, F, H, 500 + e);
      d[e] = payload(GgmlType::Q4_K, H, F, 600 + e);
      gp[e] = (uintptr_t)upload(g[e]); up[e] = (uintptr_t)upload(u[e]); dp[e] = (uintptr_t)upload(d[e]);
      gh[e] = g[e].data(); uh[e] = u[e].data(); dh[e] = d[e].data();
    }
    QuantWeightTable tg{V1<uintptr_t>(upload(gp), E), GgmlType::Q4_K, F, H, H / 256 * 144};
    QuantWeightTable tu{V1<uintptr_t>(upload(up), E), GgmlType::Q4_K, F, H, H / 256 * 144};
    QuantWeightTable td{V1<uintptr_t>(upload(dp), E), GgmlType::Q4_K, H, F, F / 256 * 144};
    std::vector<float> x(T * H), h(T * H), rw(E * H);
    for (auto& v : x) v = nd(rng);
    for (auto& v : h) v = nd(rng);
    for (auto& v : rw) v = nd(rng) / std::sqrt((float)H);
    V2<float> X(upload(x), T, H), Hin(upload(h), T, H), Hout(dmalloc<float>(T * H), T, H), Xn(dmalloc<float>(T * H), T, H);
    V2<float> RW(upload(rw), E, H);
    V1<float> nobias(nullptr, 0);
    const size_t wsb = kdnn_b200_moe_block_workspace_bytes(T, 1, S, H, F, E, 1);
    V1<uint8_t> ws(dmalloc<uint8_t>(wsb), wsb);
    cudaMemset(ws.data(), 0, wsb);
    CHECK(B::moe_block(space, X, RW, nobias, (int)S, true, 1.0f, false, tg, tu, td, Hin, Hout, Xn, 1e-6f, ws));
    V2<int> iv(dmalloc<int>(T * S), T, S);
    V2<float> wv(dmalloc<float>(T * S), T, S);
    CHECK(kdnn_b200_moe_block_routing(nullptr, ws.data(), T, 1, S, H, F, E, iv.data(), wv.data(), nullptr) == KDNN_OK);
    cudaDeviceSynchronize();
    auto idx = download(iv.data(), T * S);
    auto wts = download(wv.data(), T * S);
    std::vector<float> yref(T * H);
    ko_moe_ffn_int8(x.data(), T, H, F, E, 12, 12, 12, gh.data(), uh.data(), dh.data(), idx.data(), wts.data(), S, 0,
                    yref.data(), nullptr);
    auto hout = download(Hout.data(), T * H);
    auto xn = download(Xn.data(), T * H);
    float err = 0;
    for (size_t i = 0; i < T * H; ++i) err = std::fmax(err, std::fabs((hout[i] - h[i]) - yref[i]));
    CHECK(err <= 1e-3f * max_abs(yref) + 1e-5f * max_abs(h));
    for (size_t t = 0; t < T; ++t) {   // un-scaled RMS norm of the new residual row
      double ss = 0;
      for (size_t k = 0; k < H; ++k) ss += (double)hout[t * H + k] * hout[t * H + k];
      const float inv = (float)(1.0 / std::sqrt(ss / H + 1e-6));
      float e2 = 0;
      for (size_t k = 0; k < H; ++k) e2 = std::fmax(e2, std::fabs(xn[t * H + k] - hout[t * H + k] * inv));
      CHECK(e2 <= 1e-5f * (1.0f + std::fabs(inv) * max_abs(hout)));
    }
  }
  CHECK(kdnn_b200_device_status() == 0);
  std::printf(failures ? "dropin_test: %d FAILURES\n" : "dropin_test: all checks passed\n", failures);
  return failures ? 1 : 0;
}
