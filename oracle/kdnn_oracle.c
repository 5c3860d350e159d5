/* CPU restatement of the reference's quantized-decode arithmetic, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the parity checker for the CUDA
 * library (and, when the reference itself cannot be compiled, the timed CPU
 * baseline). Nothing in the product path may call, link or load it.
 *
 * Parity pin: oracle/pin_oracle.py checks every function here bit-for-bit
 * (integers) and bit-for-bit or to fp32 reassociation (floats) against the
 * reference's own functions compiled from its headers (oracle/_ref), and
 * against the known-answer vectors of the reference's tests restated in
 * tests/test_oracle_kat.py.
 *
 * Each function cites the reference file:line it restates (paths relative to
 * the reference project root). Build with -ffp-contract=off so fp32 products
 * and sums round exactly where the expression tree says.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define KO_Q8_0 8u
#define KO_Q4_K 12u
#define KO_Q5_K 13u
#define KO_Q6_K 14u

/* ---- threads ---------------------------------------------------------- */
int ko_num_threads(void) {
#if defined(_OPENMP)
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void ko_set_num_threads(int n) {
#if defined(_OPENMP)
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ---- scalar helpers ----------------------------------------------------- */

/* fp16 bit pattern -> fp32, exact, including subnormals, inf and nan payloads.
 * src/KokkosDNN_GGUF.hpp:201-227, src/KokkosDNN_GGUFGemvInt8.hpp:154-179 */
float ko_fp16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t ex   = ((uint32_t)h >> 10) & 0x1Fu;
  uint32_t man  = (uint32_t)h & 0x3FFu;
  uint32_t bits;
  if (ex == 0u) {
    if (man == 0u) {
      bits = sign;
    } else {
      int e = 1;
      while ((man & 0x400u) == 0u) {
        man <<= 1;
        --e;
      }
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(e + 112) << 23) | (man << 13);
    }
  } else if (ex == 31u) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((ex + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* bf16 bit pattern -> fp32. src/KokkosDNN_GGUF.hpp:229-234 */
float ko_bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* fp32 -> bf16 bit pattern, round to nearest even (what a CUDA build's
 * float -> bhalf_t conversion does; tests/Test_GGUF.cpp:53-61 uses the same
 * rounding for its bf16 fixtures). */
uint16_t ko_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if (((u >> 23) & 0xFFu) == 0xFFu && (u & 0x7FFFFFu) != 0u)
    return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
float ko_bf16_round(float f) { return ko_bf16_to_f32(ko_f32_to_bf16(f)); }

/* 6-bit (scale, min) pair j of a Q4_K / Q5_K super-block.
 * src/KokkosDNN_GGUF.hpp:287-296, src/KokkosDNN_GGUFGemvInt8.hpp:184-193 */
void ko_scale_min_k4(int j, const uint8_t* s, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = (uint8_t)(s[j] & 63u);
    *mn = (uint8_t)(s[j + 4] & 63u);
  } else {
    *sc = (uint8_t)((s[j + 4] & 0x0Fu) | ((s[j - 4] >> 6) << 4));
    *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
  }
}

/* Bytes of one packed row; 0 when cols is not a whole number of blocks or the
 * dtype is not one of the int8-path formats.
 * src/KokkosDNN_GGUF.hpp:90-138, :187-195 */
size_t ko_row_bytes(uint32_t dtype, size_t cols) {
  switch (dtype) {
    case KO_Q8_0: return cols % 32 ? 0 : cols / 32 * 34;
    case KO_Q4_K: return cols % 256 ? 0 : cols / 256 * 144;
    case KO_Q5_K: return cols % 256 ? 0 : cols / 256 * 176;
    case KO_Q6_K: return cols % 256 ? 0 : cols / 256 * 210;
    default: return 0;
  }
}

/* silu(x) = x / (1 + expf(-x)). src/KokkosDNN_SwiGLU.hpp:12-14 */
float ko_silu(float x) { return x / (1.0f + expf(-x)); }

/* 4-way signed int8 dot with int32 accumulator.
 * src/KokkosDNN_IntDot.hpp:53-66 */
int32_t ko_dot4(int32_t a, int32_t b, int32_t acc) {
  uint32_t ua = (uint32_t)a, ub = (uint32_t)b;
  for (int l = 0; l < 4; ++l) {
    int32_t x = (int8_t)(uint8_t)(ua >> (8 * l));
    int32_t y = (int8_t)(uint8_t)(ub >> (8 * l));
    acc += x * y;
  }
  return acc;
}

static uint32_t ld32(const uint8_t* p) {
  return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) |
         ((uint32_t)p[3] << 24);
}

/* ---- activation staging --------------------------------------------------
 * Layout (src/KokkosDNN_GGUFGemvInt8.hpp:108-129): int8 xq[K] at offset 0,
 * then at align16(K) one 16-byte header {float d; int32 sum_lo; int32 sum_hi;
 * int32 pad} per 32 elements. */
typedef struct {
  float d;
  int32_t sum_lo, sum_hi, pad;
} ko_act_hdr;

size_t ko_act_hdr_offset(size_t K) { return (K + 15) & ~(size_t)15; }
size_t ko_act_q8_bytes(size_t K) {
  return K % 32 ? 0 : ko_act_hdr_offset(K) + 16 * (K / 32);
}

/* Per-32 symmetric int8 quantization of one activation row (already widened
 * to fp32 from its Scalar). src/KokkosDNN_GGUFGemvInt8.hpp:198-239 */
void ko_quantize_act_q8(const float* x, size_t K, uint8_t* scratch) {
  int8_t* xq     = (int8_t*)scratch;
  ko_act_hdr* xh = (ko_act_hdr*)(scratch + ko_act_hdr_offset(K));
  for (size_t b = 0; b < K / 32; ++b) {
    const float* v = x + b * 32;
    float amax     = 0.0f;
    for (int i = 0; i < 32; ++i) {
      float a = v[i] >= 0.0f ? v[i] : -v[i];
      if (a > amax) amax = a;
    }
    const float d   = amax / 127.0f;
    const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
    int lo = 0, hi = 0;
    for (int i = 0; i < 32; ++i) {
      int q = (int)nearbyintf(v[i] * inv);
      if (q > 127) q = 127;
      if (q < -127) q = -127;
      xq[b * 32 + i] = (int8_t)q;
      if (i < 16) lo += q; else hi += q;
    }
    xh[b].d      = d;
    xh[b].sum_lo = lo;
    xh[b].sum_hi = hi;
    xh[b].pad    = 0;
  }
}

/* ---- decode units --------------------------------------------------------
 * A unit is 32 weight elements of one packed row; c = unit index in the row. */
typedef struct {
  int32_t w[8]; /* two 16-element int8 windows, four words each */
  float d0, d1;
  int32_t sum0, sum1;
} ko_window;

/* Activation window of unit c. src/KokkosDNN_GGUFGemvInt8.hpp:280-353 */
static ko_window load_window(uint32_t dtype, const uint8_t* scratch, size_t K,
                             int c) {
  const int8_t* xq     = (const int8_t*)scratch;
  const ko_act_hdr* xh = (const ko_act_hdr*)(scratch + ko_act_hdr_offset(K));
  ko_window x;
  int k0, kb, h0, h1, half = c & 1;
  switch (dtype) {
    case KO_Q4_K: {
      int blk = c >> 3, iter = (c >> 1) & 3;
      k0 = blk * 256 + iter * 64 + half * 16;
      kb = k0 + 32;
      h0 = k0 >> 5;
      h1 = h0 + 1;
      x.sum0 = half ? xh[h0].sum_hi : xh[h0].sum_lo;
      x.sum1 = half ? xh[h1].sum_hi : xh[h1].sum_lo;
      break;
    }
    case KO_Q6_K: {
      int blk = c >> 3, chunk = (c >> 2) & 1, pair = (c >> 1) & 1;
      k0 = blk * 256 + chunk * 128 + pair * 32 + half * 16;
      kb = k0 + 64;
      h0 = k0 >> 5;
      h1 = h0 + 2;
      x.sum0 = half ? xh[h0].sum_hi : xh[h0].sum_lo;
      x.sum1 = half ? xh[h1].sum_hi : xh[h1].sum_lo;
      break;
    }
    case KO_Q5_K: {
      int blk = c >> 3, sub = c & 7, iter = sub >> 1;
      k0 = blk * 256 + iter * 64 + ((sub & 1) ? 32 : 0);
      kb = k0 + 16;
      h0 = h1 = k0 >> 5;
      x.sum0 = x.sum1 = xh[h0].sum_lo + xh[h0].sum_hi;
      break;
    }
    default: /* Q8_0 */
      k0 = c * 32;
      kb = k0 + 16;
      h0 = h1 = c;
      x.sum0 = x.sum1 = 0;
      break;
  }
  for (int i = 0; i < 4; ++i) {
    x.w[i]     = (int32_t)ld32((const uint8_t*)xq + k0 + 4 * i);
    x.w[4 + i] = (int32_t)ld32((const uint8_t*)xq + kb + 4 * i);
  }
  x.d0 = xh[h0].d;
  x.d1 = xh[h1].d;
  return x;
}

void ko_unit_window(uint32_t dtype, const uint8_t* scratch, size_t K, int c,
                    int32_t* words10, float* d2) {
  ko_window x = load_window(dtype, scratch, K, c);
  for (int i = 0; i < 8; ++i) words10[i] = x.w[i];
  words10[8] = x.sum0;
  words10[9] = x.sum1;
  d2[0]      = x.d0;
  d2[1]      = x.d1;
}

/* Integer dots of one unit against its window, and the unit's fp32 value.
 * ints[0], ints[1] are what the reference multiplies by its fp32 scales:
 *   Q4_K: dotA, dotB;  Q6_K: dotA - 32*sum0, dotB - 32*sum1;
 *   Q5_K: dot, 0;      Q8_0: dot, 0.
 * src/KokkosDNN_GGUFGemvInt8.hpp:359-466 */
static float unit_eval(uint32_t dtype, const uint8_t* row, int c,
                       const ko_window* x, int32_t* ints) {
  int blk = c >> 3, half = c & 1;
  switch (dtype) {
    case KO_Q4_K: {
      int iter          = (c >> 1) & 3;
      const uint8_t* b  = row + (size_t)blk * 144;
      const uint8_t* qw = b + 16 + iter * 32 + half * 16;
      uint8_t sc0, mn0, sc1, mn1;
      ko_scale_min_k4(2 * iter, b + 4, &sc0, &mn0);
      ko_scale_min_k4(2 * iter + 1, b + 4, &sc1, &mn1);
      const float dw = ko_fp16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
      const float dm = ko_fp16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
      const float fa = dw * (float)sc0 * x->d0;
      const float ma = dm * (float)mn0 * x->d0;
      const float fb = dw * (float)sc1 * x->d1;
      const float mb = dm * (float)mn1 * x->d1;
      int32_t dotA = 0, dotB = 0;
      for (int i = 0; i < 4; ++i) {
        uint32_t w = ld32(qw + 4 * i);
        dotA = ko_dot4((int32_t)(w & 0x0F0F0F0Fu), x->w[i], dotA);
        dotB = ko_dot4((int32_t)((w >> 4) & 0x0F0F0F0Fu), x->w[4 + i], dotB);
      }
      ints[0] = dotA;
      ints[1] = dotB;
      return fa * (float)dotA - ma * (float)x->sum0 + fb * (float)dotB -
             mb * (float)x->sum1;
    }
    case KO_Q5_K: {
      int sub = c & 7, iter = sub >> 1, low = (sub & 1) == 0;
      const uint8_t* b  = row + (size_t)blk * 176;
      const uint8_t* qh = b + 16;
      const uint8_t* ql = b + 48 + iter * 32;
      uint8_t sc, mn;
      ko_scale_min_k4(sub, b + 4, &sc, &mn);
      const float dw = ko_fp16_to_f32((uint16_t)(b[0] | (b[1] << 8))) * (float)sc * x->d0;
      const float dm = ko_fp16_to_f32((uint16_t)(b[2] | (b[3] << 8))) * (float)mn * x->d0;
      const uint32_t sh = low ? 0u : 4u, bitsh = (uint32_t)(2 * iter + (low ? 0 : 1));
      int32_t dot = 0;
      for (int i = 0; i < 4; ++i) {
        uint32_t w0 = ((ld32(ql + 4 * i) >> sh) & 0x0F0F0F0Fu) |
                      (((ld32(qh + 4 * i) >> bitsh) & 0x01010101u) << 4);
        uint32_t w1 = ((ld32(ql + 16 + 4 * i) >> sh) & 0x0F0F0F0Fu) |
                      (((ld32(qh + 16 + 4 * i) >> bitsh) & 0x01010101u) << 4);
        dot = ko_dot4((int32_t)w0, x->w[i], dot);
        dot = ko_dot4((int32_t)w1, x->w[4 + i], dot);
      }
      ints[0] = dot;
      ints[1] = 0;
      return dw * (float)dot - dm * (float)x->sum0;
    }
    case KO_Q6_K: {
      int chunk = (c >> 2) & 1, pair = (c >> 1) & 1;
      const uint8_t* b  = row + (size_t)blk * 210;
      const uint8_t* ql = b + chunk * 64 + pair * 32 + half * 16;
      const uint8_t* qh = b + 128 + chunk * 32 + half * 16;
      const int8_t* scl = (const int8_t*)(b + 192);
      const float d     = ko_fp16_to_f32((uint16_t)(b[208] | (b[209] << 8)));
      const float s0    = d * (float)scl[chunk * 8 + 2 * pair + half] * x->d0;
      const float s1    = d * (float)scl[chunk * 8 + 2 * pair + half + 4] * x->d1;
      const uint32_t sh = pair ? 2u : 0u;
      int32_t dotA = 0, dotB = 0;
      for (int i = 0; i < 4; ++i) {
        uint32_t qlw = ld32(ql + 4 * i), qhw = ld32(qh + 4 * i);
        uint32_t wA  = (qlw & 0x0F0F0F0Fu) | (((qhw >> sh) & 0x03030303u) << 4);
        uint32_t wB  = ((qlw >> 4) & 0x0F0F0F0Fu) |
                      (((qhw >> (sh + 4u)) & 0x03030303u) << 4);
        dotA = ko_dot4((int32_t)wA, x->w[i], dotA);
        dotB = ko_dot4((int32_t)wB, x->w[4 + i], dotB);
      }
      ints[0] = dotA - (x->sum0 << 5);
      ints[1] = dotB - (x->sum1 << 5);
      return s0 * (float)ints[0] + s1 * (float)ints[1];
    }
    default: { /* Q8_0 */
      const uint8_t* b = row + (size_t)c * 34;
      const float dw   = ko_fp16_to_f32((uint16_t)(b[0] | (b[1] << 8))) * x->d0;
      int32_t dot      = 0;
      for (int i = 0; i < 8; ++i)
        dot = ko_dot4((int32_t)ld32(b + 2 + 4 * i), x->w[i], dot);
      ints[0] = dot;
      ints[1] = 0;
      return dw * (float)dot;
    }
  }
}

/* Per-unit integer dots and fp32 values for a whole packed matrix:
 * ints[(row*nunits + c)*2 + {0,1}], vals[row*nunits + c] (either may be NULL). */
void ko_unit_table(uint32_t dtype, const uint8_t* w, size_t rows, size_t cols,
                   const uint8_t* scratch, int32_t* ints, float* vals) {
  const size_t rb = ko_row_bytes(dtype, cols);
  const int nu    = (int)(cols / 32);
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
  for (long r = 0; r < (long)rows; ++r)
    for (int c = 0; c < nu; ++c) {
      ko_window x = load_window(dtype, scratch, cols, c);
      int32_t two[2];
      float v = unit_eval(dtype, w + (size_t)r * rb, c, &x, two);
      if (ints) {
        ints[((size_t)r * nu + c) * 2]     = two[0];
        ints[((size_t)r * nu + c) * 2 + 1] = two[1];
      }
      if (vals) vals[(size_t)r * nu + c] = v;
    }
}

/* Stage 2 of the int8 GEMV over an already-staged activation row:
 * y[row] = sum over units c ascending, fp32 (the order a one-thread team
 * produces). src/KokkosDNN_GGUFGemvInt8.hpp:480-505 */
void ko_gemv_int8_staged(uint32_t dtype, const uint8_t* w, size_t rows,
                         size_t cols, const uint8_t* scratch, float* y) {
  const size_t rb = ko_row_bytes(dtype, cols);
  const int nu    = (int)(cols / 32);
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
  for (long r = 0; r < (long)rows; ++r) {
    float sum = 0.0f;
    for (int c = 0; c < nu; ++c) {
      ko_window x = load_window(dtype, scratch, cols, c);
      int32_t two[2];
      sum += unit_eval(dtype, w + (size_t)r * rb, c, &x, two);
    }
    y[r] = sum;
  }
}

/* Both stages: quantize x (fp32 values of the Scalar activations) into
 * scratch, then the integer-dot GEMV. y is the fp32 row sum BEFORE the cast to
 * Scalar. src/KokkosDNN_GGUFGemvInt8.hpp:711-777, src/KokkosDNN_GGUF.hpp:2531-2551 */
int ko_gemv_int8(uint32_t dtype, const uint8_t* w, size_t rows, size_t cols,
                 const float* x, float* y, uint8_t* scratch) {
  if (ko_row_bytes(dtype, cols) == 0 || rows == 0) return 1;
  ko_quantize_act_q8(x, cols, scratch);
  ko_gemv_int8_staged(dtype, w, rows, cols, scratch, y);
  return 0;
}

/* ---- block dequantizers -------------------------------------------------- */

/* One packed row -> fp32. src/KokkosDNN_GGUF.hpp:300-384 */
int ko_dequant_row(uint32_t dtype, const uint8_t* row, size_t cols, float* out) {
  switch (dtype) {
    case KO_Q4_K:
      for (size_t b = 0; b < cols / 256; ++b, row += 144, out += 256) {
        const float d  = ko_fp16_to_f32((uint16_t)(row[0] | (row[1] << 8)));
        const float mn = -ko_fp16_to_f32((uint16_t)(row[2] | (row[3] << 8)));
        for (int j = 0; j < 4; ++j) {
          uint8_t s1, m1, s2, m2;
          ko_scale_min_k4(2 * j, row + 4, &s1, &m1);
          ko_scale_min_k4(2 * j + 1, row + 4, &s2, &m2);
          const float d1 = d * (float)s1, o1 = mn * (float)m1;
          const float d2 = d * (float)s2, o2 = mn * (float)m2;
          const uint8_t* q = row + 16 + 32 * j;
          for (int l = 0; l < 32; ++l) {
            out[64 * j + l]      = d1 * (float)(q[l] & 0xF) + o1;
            out[64 * j + 32 + l] = d2 * (float)(q[l] >> 4) + o2;
          }
        }
      }
      return 0;
    case KO_Q5_K:
      for (size_t b = 0; b < cols / 256; ++b, row += 176, out += 256) {
        const float d  = ko_fp16_to_f32((uint16_t)(row[0] | (row[1] << 8)));
        const float mn = ko_fp16_to_f32((uint16_t)(row[2] | (row[3] << 8)));
        const uint8_t* qh = row + 16;
        for (int j = 0; j < 4; ++j) {
          uint8_t s1, m1, s2, m2;
          ko_scale_min_k4(2 * j, row + 4, &s1, &m1);
          ko_scale_min_k4(2 * j + 1, row + 4, &s2, &m2);
          const float d1 = d * (float)s1, o1 = mn * (float)m1;
          const float d2 = d * (float)s2, o2 = mn * (float)m2;
          const uint8_t* q = row + 48 + 32 * j;
          const uint8_t u1 = (uint8_t)(1u << (2 * j)), u2 = (uint8_t)(2u << (2 * j));
          for (int l = 0; l < 32; ++l) {
            out[64 * j + l]      = d1 * (float)((q[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - o1;
            out[64 * j + 32 + l] = d2 * (float)((q[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - o2;
          }
        }
      }
      return 0;
    case KO_Q6_K:
      for (size_t b = 0; b < cols / 256; ++b, row += 210, out += 256) {
        const float d     = ko_fp16_to_f32((uint16_t)(row[208] | (row[209] << 8)));
        const int8_t* scl = (const int8_t*)(row + 192);
        for (int n = 0; n < 2; ++n) {
          const uint8_t* ql = row + 64 * n;
          const uint8_t* qh = row + 128 + 32 * n;
          const int8_t* sc  = scl + 8 * n;
          float* o          = out + 128 * n;
          for (int l = 0; l < 32; ++l) {
            const int is = l / 16;
            const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
            const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            o[l]      = d * (float)sc[is + 0] * (float)q1;
            o[l + 32] = d * (float)sc[is + 2] * (float)q2;
            o[l + 64] = d * (float)sc[is + 4] * (float)q3;
            o[l + 96] = d * (float)sc[is + 6] * (float)q4;
          }
        }
      }
      return 0;
    case KO_Q8_0:
      for (size_t b = 0; b < cols / 32; ++b, row += 34, out += 32) {
        const float d = ko_fp16_to_f32((uint16_t)(row[0] | (row[1] << 8)));
        for (int i = 0; i < 32; ++i) out[i] = d * (float)(int8_t)row[2 + i];
      }
      return 0;
    default: return -1;
  }
}

/* y[row] = sum_k dequant(W[row,k]) * x[k] accumulated in double: the
 * independent reference the reference's own GEMV tests compare against
 * (tests/Test_GGUF.cpp:744-752, :916-925). mag[row] = sum |terms| (may be NULL). */
int ko_gemv_dequant_f64(uint32_t dtype, const uint8_t* w, size_t rows,
                        size_t cols, const float* x, double* y, double* mag) {
  const size_t rb = ko_row_bytes(dtype, cols);
  if (rb == 0) return -1;
#if defined(_OPENMP)
#pragma omp parallel
#endif
  {
    float* tmp = (float*)malloc(sizeof(float) * cols);
#if defined(_OPENMP)
#pragma omp for schedule(static)
#endif
    for (long r = 0; r < (long)rows; ++r) {
      ko_dequant_row(dtype, w + (size_t)r * rb, cols, tmp);
      double acc = 0, m = 0;
      for (size_t k = 0; k < cols; ++k) {
        const double v = (double)tmp[k] * (double)x[k];
        acc += v;
        m += fabs(v);
      }
      y[r] = acc;
      if (mag) mag[r] = m;
    }
    free(tmp);
  }
  return 0;
}

/* Values the int8 staging represents: out[k] = d_block * q[k]
 * (the "dqx" array of tests/Test_GGUF.cpp:868-881). */
void ko_dequant_act(const uint8_t* scratch, size_t K, float* out) {
  const int8_t* xq     = (const int8_t*)scratch;
  const ko_act_hdr* xh = (const ko_act_hdr*)(scratch + ko_act_hdr_offset(K));
  for (size_t k = 0; k < K; ++k) out[k] = xh[k / 32].d * (float)xq[k];
}

/* ---- router ---------------------------------------------------------------
 * Greedy top-k with strict '>' (ties keep the lower expert id), then weights
 * recomputed from the logits at the selected ids.
 * src/KokkosDNN_MoE.hpp:84-147 (select + weights), :161-200 (scores).
 * logits: [T,E] fp32 values of the Scalar logits; bias: E values or NULL. */
int ko_moe_route(const float* logits, size_t T, size_t E, const float* bias,
                 int top_k, int norm_topk, float routed_scale, int sigmoid,
                 int* top_idx, float* top_w) {
  const float NEG = -3.4028235e38f;
  if (T == 0) return 0;
  if (top_k <= 0 || (size_t)top_k > E) return -1;
#if defined(_OPENMP)
#pragma omp parallel
#endif
  {
    float* score = (float*)malloc(sizeof(float) * (E ? E : 1));
    float* lk    = (float*)malloc(sizeof(float) * (size_t)top_k);
#if defined(_OPENMP)
#pragma omp for schedule(static)
#endif
    for (long t = 0; t < (long)T; ++t) {
      const float* lg = logits + (size_t)t * E;
      int* idx        = top_idx + (size_t)t * top_k;
      float* w        = top_w + (size_t)t * top_k;
      for (size_t e = 0; e < E; ++e) {
        const float b = bias ? bias[e] : 0.0f;
        score[e] = sigmoid ? (1.0f / (1.0f + expf(-lg[e]))) + b : lg[e] + b;
      }
      float gmx = NEG, gsum = 0.0f;
      if (!sigmoid && !norm_topk) {
        for (size_t e = 0; e < E; ++e)
          if (score[e] > gmx) gmx = score[e];
        for (size_t e = 0; e < E; ++e) gsum += expf(score[e] - gmx);
      }
      for (int k = 0; k < top_k; ++k) {
        float best = NEG;
        int be     = -1;
        for (size_t e = 0; e < E; ++e)
          if (score[e] > best) {
            best = score[e];
            be   = (int)e;
          }
        idx[k] = be;
        if (be >= 0) score[be] = NEG;
      }
      for (int k = 0; k < top_k; ++k) {
        const size_t i  = (size_t)idx[k];
        const float raw = lg[i];
        lk[k] = sigmoid ? 1.0f / (1.0f + expf(-raw)) : raw + (bias ? bias[i] : 0.0f);
      }
      if (sigmoid) {
        if (norm_topk) {
          float sum = 0.0f;
          for (int k = 0; k < top_k; ++k) sum += lk[k];
          const float denom = sum + 1e-6f;
          for (int k = 0; k < top_k; ++k) w[k] = lk[k] / denom * routed_scale;
        } else {
          for (int k = 0; k < top_k; ++k) w[k] = lk[k] * routed_scale;
        }
      } else if (norm_topk) {
        float mx = NEG, sum = 0.0f;
        for (int k = 0; k < top_k; ++k)
          if (lk[k] > mx) mx = lk[k];
        for (int k = 0; k < top_k; ++k) sum += expf(lk[k] - mx);
        for (int k = 0; k < top_k; ++k) w[k] = expf(lk[k] - mx) / sum * routed_scale;
      } else {
        for (int k = 0; k < top_k; ++k) w[k] = expf(lk[k] - gmx) / gsum * routed_scale;
      }
    }
    free(score);
    free(lk);
  }
  return 0;
}

/* ---- MoE feed-forward with int8 activations --------------------------------
 * Composition of the reference's pieces for T tokens (the reference has no
 * batched int8 kernel; its fused one-token kernel src/KokkosDNN_GGUF.hpp:
 * 2075-2223 has this structure with fp dots):
 *   per (token t, slot s), e = idx[t,s]; slots with e out of range or w == 0
 *   contribute nothing (:2106-2110, :2205-2207);
 *   g = int8 GEMV(gate_e, x_t), u = int8 GEMV(up_e, x_t)   (fp32 row sums)
 *   act = Scalar(silu(g) * u)                               (:2152)
 *   o   = int8 GEMV(down_e, act)                            (fp32 row sums)
 *   Y[t,:] = sum_s w[t,s] * o_s, s ascending, fp32          (:2201-2220,
 *                                   src/KokkosDNN_MoE.hpp:326-331)
 * X: [T,H] fp32 values of the Scalar activations. bf16 != 0 rounds act to
 * bf16 (Scalar = bf16). Y: [T,H] fp32, before the cast to Scalar.
 * act_out (optional): [T,S,F] the Scalar-rounded activations as fp32. */
int ko_moe_ffn_int8(const float* X, size_t T, size_t H, size_t F,
                    size_t n_experts, uint32_t gdt, uint32_t udt, uint32_t ddt,
                    const uint8_t* const* gate, const uint8_t* const* up,
                    const uint8_t* const* down, const int* idx,
                    const float* wts, size_t S, int bf16, float* Y,
                    float* act_out) {
  if (!ko_row_bytes(gdt, H) || !ko_row_bytes(udt, H) || !ko_row_bytes(ddt, F))
    return -1;
  const size_t sx = ko_act_q8_bytes(H), sa = ko_act_q8_bytes(F);
#if defined(_OPENMP)
#pragma omp parallel
#endif
  {
    uint8_t* xs = (uint8_t*)aligned_alloc(64, (sx + 63) & ~(size_t)63);
    uint8_t* as = (uint8_t*)aligned_alloc(64, (sa + 63) & ~(size_t)63);
    float* g    = (float*)malloc(sizeof(float) * F);
    float* u    = (float*)malloc(sizeof(float) * F);
    float* a    = (float*)malloc(sizeof(float) * F);
    float* o    = (float*)malloc(sizeof(float) * H);
#if defined(_OPENMP)
#pragma omp for schedule(dynamic, 1)
#endif
    for (long t = 0; t < (long)T; ++t) {
      float* y = Y + (size_t)t * H;
      for (size_t d = 0; d < H; ++d) y[d] = 0.0f;
      ko_quantize_act_q8(X + (size_t)t * H, H, xs);
      for (size_t s = 0; s < S; ++s) {
        const int e   = idx[(size_t)t * S + s];
        const float w = wts[(size_t)t * S + s];
        const int bad = e < 0 || (size_t)e >= n_experts;
        if (act_out)
          for (size_t j = 0; j < F; ++j) act_out[((size_t)t * S + s) * F + j] = 0.0f;
        if (bad) continue;
        /* nested parallelism is off: these run serially inside the token loop */
        for (size_t j = 0; j < F; ++j) {
          float sg = 0.0f, su = 0.0f;
          const uint8_t* gr = gate[e] + j * ko_row_bytes(gdt, H);
          const uint8_t* ur = up[e] + j * ko_row_bytes(udt, H);
          for (int c = 0; c < (int)(H / 32); ++c) {
            int32_t two[2];
            ko_window xw = load_window(gdt, xs, H, c);
            sg += unit_eval(gdt, gr, c, &xw, two);
            if (udt != gdt) xw = load_window(udt, xs, H, c);
            su += unit_eval(udt, ur, c, &xw, two);
          }
          g[j] = sg;
          u[j] = su;
          const float v = ko_silu(sg) * su;
          a[j]          = bf16 ? ko_bf16_round(v) : v;
        }
        if (act_out) memcpy(act_out + ((size_t)t * S + s) * F, a, sizeof(float) * F);
        if (w == 0.0f) continue;
        ko_quantize_act_q8(a, F, as);
        for (size_t d = 0; d < H; ++d) {
          float sum = 0.0f;
          const uint8_t* dr = down[e] + d * ko_row_bytes(ddt, F);
          for (int c = 0; c < (int)(F / 32); ++c) {
            int32_t two[2];
            ko_window aw = load_window(ddt, as, F, c);
            sum += unit_eval(ddt, dr, c, &aw, two);
          }
          o[d] = sum;
        }
        for (size_t d = 0; d < H; ++d) y[d] += w * o[d];
      }
    }
    free(xs); free(as); free(g); free(u); free(a); free(o);
  }
  return 0;
}

/* y[t,d] = sum_k w[t,k] * out[t,k,d], k ascending, fp32.
 * src/KokkosDNN_MoE.hpp:313-332 */
void ko_moe_weighted_sum(const float* out, const float* w, size_t T, size_t K,
                         size_t D, float* y) {
  for (size_t t = 0; t < T; ++t)
    for (size_t d = 0; d < D; ++d) {
      float acc = 0.0f;
      for (size_t k = 0; k < K; ++k) acc += w[t * K + k] * out[(t * K + k) * D + d];
      y[t * D + d] = acc;
    }
}
