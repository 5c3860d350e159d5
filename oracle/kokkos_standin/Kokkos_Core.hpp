// Host-only stand-in for the slice of the Kokkos API that the reference's
// quantized-decode headers use (KokkosDNN_GGUF.hpp, KokkosDNN_GGUFGemvInt8.hpp,
// KokkosDNN_IntDot.hpp, KokkosDNN_MoE.hpp, KokkosDNN_SwiGLU.hpp,
// KokkosDNN_Handle.hpp, KokkosDNN_Occupancy.hpp).
//
// TEST INFRASTRUCTURE ONLY. It exists so the reference's own functor bodies
// can be compiled and executed on CPU cores as the parity oracle and as the
// timed CPU baseline. It is not Kokkos: teams always have exactly one thread
// (the reference's kernels all stride on the runtime team size, so a
// one-thread team runs each functor body as a serial loop), and the league
// loop of every parallel_for is distributed over OpenMP threads when built
// with -fopenmp. Integer results are schedule-independent; fp32 sums follow
// the serial order of a one-thread team.
#pragma once

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define KOKKOS_INLINE_FUNCTION inline
#define KOKKOS_FUNCTION
#define KOKKOS_LAMBDA [=]

namespace Kokkos {

// ---- math ---------------------------------------------------------------
// rint follows the current rounding mode (round-to-nearest-even by default),
// which is what Kokkos::rint lowers to on every backend.
inline float rint(float v) { return ::nearbyintf(v); }
inline float expf(float v) { return ::expf(v); }
inline float sqrtf(float v) { return ::sqrtf(v); }
inline float cosf(float v) { return ::cosf(v); }
inline float sinf(float v) { return ::sinf(v); }

// ---- spaces -------------------------------------------------------------
struct HostSpace {};

// Bump allocator over one league member's scratch arena.
class ScratchArena {
 public:
  ScratchArena() = default;
  ScratchArena(char* base, std::size_t cap) : base_(base), cap_(cap) {}
  void* get_shmem(std::size_t bytes) const {
    const std::size_t need = (bytes + 15) & ~std::size_t(15);
    if (used_ + need > cap_) throw std::runtime_error("standin: team scratch overflow");
    void* p = base_ + used_;
    used_ += need;
    return p;
  }

 private:
  char* base_             = nullptr;
  std::size_t cap_        = 0;
  mutable std::size_t used_ = 0;
};

// The one execution space: host cores, OpenMP over the league when available.
struct HostThreads {
  using memory_space         = HostSpace;
  using scratch_memory_space = ScratchArena;
  using execution_space      = HostThreads;
  std::uint32_t impl_instance_id() const { return 1u; }
  void fence() const {}
  void fence(const std::string&) const {}
};
using Serial                = HostThreads;
using DefaultExecutionSpace = HostThreads;
using DefaultHostExecutionSpace = HostThreads;

inline void fence() {}
inline void fence(const std::string&) {}

// ---- policies -----------------------------------------------------------
struct AUTO_t {};
static constexpr AUTO_t AUTO{};
struct ParallelForTag {};
struct PerTeamValue {
  std::size_t bytes;
};
struct PerThreadValue {
  std::size_t bytes;
};
inline PerTeamValue PerTeam(std::size_t b) { return {b}; }
inline PerThreadValue PerThread(std::size_t b) { return {b}; }

class TeamHandle {
 public:
  TeamHandle(int rank, int size, char* scratch, std::size_t cap)
      : league_rank_(rank), league_size_(size), arena_(scratch, cap) {}
  int league_rank() const { return league_rank_; }
  int league_size() const { return league_size_; }
  int team_rank() const { return 0; }
  int team_size() const { return 1; }
  void team_barrier() const {}
  const ScratchArena& team_shmem() const { return arena_; }
  const ScratchArena& team_scratch(int) const { return arena_; }
  const ScratchArena& thread_scratch(int) const { return arena_; }

 private:
  int league_rank_, league_size_;
  ScratchArena arena_;
};

template <class... Props>
class TeamPolicy {
 public:
  using member_type = TeamHandle;
  TeamPolicy(int league, int team) : league_(league) {
    if (team != 1)
      throw std::runtime_error("standin: host teams have exactly one thread");
  }
  TeamPolicy(int league, AUTO_t) : league_(league) {}
  template <class Space>
  TeamPolicy(const Space&, int league, int team) : TeamPolicy(league, team) {}
  TeamPolicy& set_scratch_size(int, PerTeamValue v) {
    scratch_ += v.bytes;
    return *this;
  }
  TeamPolicy& set_scratch_size(int, PerThreadValue v) {
    scratch_ += v.bytes;
    return *this;
  }
  TeamPolicy& set_scratch_size(int, PerTeamValue a, PerThreadValue b) {
    scratch_ += a.bytes + b.bytes;
    return *this;
  }
  template <class F>
  int team_size_max(const F&, ParallelForTag) const {
    return 1;
  }
  int league_size() const { return league_; }
  std::size_t scratch_bytes() const { return scratch_; }

 private:
  int league_;
  std::size_t scratch_ = 0;
};

template <class... Props>
struct RangePolicy {
  std::size_t begin, end;
  RangePolicy(std::size_t b, std::size_t e) : begin(b), end(e) {}
  template <class Space>
  RangePolicy(const Space&, std::size_t b, std::size_t e) : begin(b), end(e) {}
};

template <int N>
struct Rank {};
template <class... Props>
struct MDRangePolicy {
  std::size_t lo[2], hi[2];
  template <class A, class B>
  MDRangePolicy(std::initializer_list<A> l, std::initializer_list<B> h) {
    int i = 0;
    for (auto v : l) lo[i++] = static_cast<std::size_t>(v);
    i = 0;
    for (auto v : h) hi[i++] = static_cast<std::size_t>(v);
  }
};

struct TeamThreadRangeSpan {
  std::size_t begin, end;
};
inline TeamThreadRangeSpan TeamThreadRange(const TeamHandle&, std::size_t n) {
  return {0, n};
}
inline TeamThreadRangeSpan TeamThreadRange(const TeamHandle&, std::size_t b,
                                           std::size_t e) {
  return {b, e};
}
inline TeamThreadRangeSpan ThreadVectorRange(const TeamHandle&, std::size_t n) {
  return {0, n};
}

// ---- dispatch -----------------------------------------------------------
template <class F, class... P>
void parallel_for(const std::string&, const TeamPolicy<P...>& pol, const F& f) {
  const int league      = pol.league_size();
  const std::size_t cap = pol.scratch_bytes() + 256;
#if defined(_OPENMP)
#pragma omp parallel
  {
    std::vector<char> arena(cap);
#pragma omp for schedule(static)
    for (int i = 0; i < league; ++i) {
      TeamHandle m(i, league, arena.data(), cap);
      f(m);
    }
  }
#else
  std::vector<char> arena(cap);
  for (int i = 0; i < league; ++i) {
    TeamHandle m(i, league, arena.data(), cap);
    f(m);
  }
#endif
}
template <class F, class... P>
void parallel_for(const TeamPolicy<P...>& pol, const F& f) {
  parallel_for(std::string(), pol, f);
}

template <class F, class... P>
void parallel_for(const std::string&, const RangePolicy<P...>& pol, const F& f) {
  const long b = static_cast<long>(pol.begin), e = static_cast<long>(pol.end);
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
  for (long i = b; i < e; ++i) f(static_cast<int>(i));
}

template <class F, class... P>
void parallel_for(const std::string&, const MDRangePolicy<P...>& pol,
                  const F& f) {
  const long b0 = static_cast<long>(pol.lo[0]), e0 = static_cast<long>(pol.hi[0]);
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
  for (long i = b0; i < e0; ++i)
    for (std::size_t j = pol.lo[1]; j < pol.hi[1]; ++j)
      f(static_cast<std::size_t>(i), j);
}

// Nested (inside a team): serial, because the team has one thread.
template <class F>
void parallel_for(const TeamThreadRangeSpan& r, const F& f) {
  for (std::size_t i = r.begin; i < r.end; ++i) f(i);
}
template <class F, class T>
void parallel_reduce(const TeamThreadRangeSpan& r, const F& f, T& out) {
  T acc = T();
  for (std::size_t i = r.begin; i < r.end; ++i) f(i, acc);
  out = acc;
}

// ---- View ---------------------------------------------------------------
struct LayoutRight {};
struct LayoutLeft {};
struct Unmanaged {};
template <class T>
struct MemoryTraits {};

namespace detail {
template <class D>
struct peel {
  static constexpr int rank = 0;
  using type                = D;
};
template <class D>
struct peel<D*> {
  static constexpr int rank = 1 + peel<D>::rank;
  using type                = typename peel<D>::type;
};
}  // namespace detail

// Row-major (LayoutRight) dense array of rank 0..3, shared ownership for
// labelled allocations, non-owning when wrapped around a pointer.
template <class DataType, class... Props>
class View {
 public:
  using value_type           = typename detail::peel<DataType>::type;
  using non_const_value_type = std::remove_const_t<value_type>;
  static constexpr int rank  = detail::peel<DataType>::rank;
  using HostMirror           = View;
  using host_mirror_type     = View;
  using execution_space      = HostThreads;
  using memory_space         = HostSpace;

  View() { ext_[0] = ext_[1] = ext_[2] = 0; }
  explicit View(const std::string&, std::size_t a = 1, std::size_t b = 1,
                std::size_t c = 1) {
    set_extents(a, b, c);
    const std::size_t n = span();
    // 64-byte aligned like a real Kokkos allocation (the reference's int8
    // path declines unless payload and staging are 16-byte aligned).
    void* raw = nullptr;
    if (posix_memalign(&raw, 64, (n ? n : 1) * sizeof(non_const_value_type)) != 0)
      throw std::bad_alloc();
    std::memset(raw, 0, (n ? n : 1) * sizeof(non_const_value_type));
    owner_ = std::shared_ptr<void>(raw, [](void* p) { std::free(p); });
    ptr_   = static_cast<value_type*>(raw);
  }
  View(value_type* p, std::size_t a = 1, std::size_t b = 1, std::size_t c = 1)
      : ptr_(p) {
    set_extents(a, b, c);
  }
  View(const ScratchArena& arena, std::size_t a)
      : ptr_(static_cast<value_type*>(arena.get_shmem(a * sizeof(value_type)))) {
    set_extents(a, 1, 1);
  }
  template <class D2, class... P2>
  View(const View<D2, P2...>& o) : owner_(o.owner()), ptr_(o.data()) {
    ext_[0] = o.raw_extent(0);
    ext_[1] = o.raw_extent(1);
    ext_[2] = o.raw_extent(2);
  }

  value_type* data() const { return ptr_; }
  std::size_t extent(int i) const { return i < rank ? ext_[i] : 1; }
  int extent_int(int i) const { return static_cast<int>(extent(i)); }
  std::size_t raw_extent(int i) const { return ext_[i]; }
  std::size_t size() const { return span(); }
  std::size_t span() const {
    std::size_t n = 1;
    for (int i = 0; i < rank; ++i) n *= ext_[i];
    return n;
  }
  std::size_t stride(int i) const {
    std::size_t s = 1;
    for (int j = rank - 1; j > i; --j) s *= ext_[j];
    return s;
  }
  const std::shared_ptr<void>& owner() const { return owner_; }

  value_type& operator()() const { return ptr_[0]; }
  value_type& operator()(std::size_t i) const { return ptr_[i]; }
  value_type& operator()(std::size_t i, std::size_t j) const {
    return ptr_[i * ext_[1] + j];
  }
  value_type& operator()(std::size_t i, std::size_t j, std::size_t k) const {
    return ptr_[(i * ext_[1] + j) * ext_[2] + k];
  }

 private:
  void set_extents(std::size_t a, std::size_t b, std::size_t c) {
    ext_[0] = rank > 0 ? a : 1;
    ext_[1] = rank > 1 ? b : 1;
    ext_[2] = rank > 2 ? c : 1;
  }
  std::shared_ptr<void> owner_;
  value_type* ptr_ = nullptr;
  std::size_t ext_[3];
};

template <class V>
V create_mirror_view(const V& v) {
  return v;
}
template <class Space, class V>
V create_mirror_view_and_copy(const Space&, const V& v) {
  return v;
}
template <class A, class B>
void deep_copy(const A& dst, const B& src) {
  if (static_cast<const void*>(dst.data()) == static_cast<const void*>(src.data()))
    return;
  std::memcpy(dst.data(), src.data(),
              sizeof(typename A::non_const_value_type) * dst.span());
}

// ---- reduced-precision scalar --------------------------------------------
namespace Experimental {
// True 16-bit bfloat16 storage with round-to-nearest-even conversion from
// float, so a "bf16" instantiation of a reference op sees the values a CUDA
// build (__float2bfloat16_rn) would see.
struct bhalf_t {
  std::uint16_t bits = 0;
  bhalf_t()          = default;
  explicit bhalf_t(float f) {
    std::uint32_t u;
    std::memcpy(&u, &f, 4);
    if (((u >> 23) & 0xFFu) == 0xFFu && (u & 0x7FFFFFu) != 0u) {
      bits = static_cast<std::uint16_t>((u >> 16) | 0x40u);  // quiet NaN
    } else {
      u += 0x7FFFu + ((u >> 16) & 1u);
      bits = static_cast<std::uint16_t>(u >> 16);
    }
  }
  explicit operator float() const {
    const std::uint32_t u = static_cast<std::uint32_t>(bits) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
  }
};
}  // namespace Experimental

}  // namespace Kokkos
