/*
 * kq_oracle — CPU restatement of karume's quantized `linear` path.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke
 * check and the CPU-baseline / reference legs of the benchmark may load this
 * library; the CUDA library never links or calls it and has no CPU fallback.
 *
 * The reference implementation is TypeScript + WGSL and cannot run where this is
 * built (no Deno / WebGPU), so every function below restates one reference
 * function in plain C and names the reference file:line it follows (paths are
 * relative to the karume repository root).  The restatement is pinned against
 *   - the known-answer vectors of the reference's own tests
 *     (packages/runtime/tests/format_i4_test.ts, gpu_i8_weights_test.ts,
 *      tools/exporter/tests/test_emit.py),
 *   - the reference's committed torch-derived golden model with an i8 `linear`
 *     (packages/runtime/tests/fixtures/golden/i8_weights), and
 *   - vectors produced by importing the reference's Python exporter
 *     (karume.quantize / karume.emit), whose `dequantize_int4/int8` are the
 *     producer-side witnesses of the same single-rounding dequant rule,
 *   - the known answers of packages/runtime/tests/i8a8_reference_test.ts for the
 *     integer-dot functions.
 * The neighbour formulas at the end of the file (rms_norm, sigmoid / silu-mul, add) have
 * no golden output in the reference's tests: for those three, PARITY IS UNPINNED (they are
 * restated formulas checked against hand-computed values).
 *
 * Build: -O2/-O3 WITHOUT -ffast-math.  FP contraction is irrelevant to the f64
 * paths (an f32*f32 product is exact in f64) and is pinned off by the Makefile
 * (-ffp-contract=off) so that the explicit fmaf()/non-fmaf variants of the f32
 * replay mean what they say.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define KQO_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------------------
 * f16 / bf16 helpers
 * ------------------------------------------------------------------------- */

/* IEEE binary16 bit pattern -> f32 value.  Always exact.
 * Follows packages/runtime/src/format/f16.ts:23-36 (f16BitsToF32): exponent 0 is
 * +-0 / subnormal (mantissa * 2^-24), exponent 31 is Inf / NaN (payload not kept),
 * else (1 + mantissa/1024) * 2^(exp-15). */
KQO_API float kqo_f16_bits_to_f32(uint16_t bits) {
  const int sign = (bits & 0x8000u) ? -1 : 1;
  const int exponent = (bits >> 10) & 0x1f;
  const int mantissa = bits & 0x3ff;
  if (exponent == 0) return (float)sign * (float)mantissa * 0x1p-24f;
  if (exponent == 0x1f) return mantissa == 0 ? (float)sign * INFINITY : NAN;
  return (float)sign * (1.0f + (float)mantissa / 1024.0f) * ldexpf(1.0f, exponent - 15);
}

/* f32 -> binary16 bit pattern, round-to-nearest-even, overflow to Inf, gradual
 * underflow.  This is the rounding `Math.f16round` performs in
 * packages/runtime/src/format/f16.ts:56-68 (roundToF16). */
KQO_API uint16_t kqo_f32_to_f16_bits(float value) {
  uint32_t x;
  memcpy(&x, &value, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t absx = x & 0x7fffffffu;
  if (absx > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);  /* NaN */
  if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* >= 65520 -> Inf */
  if (absx < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25 -> 0 (tie to even) */
  int exponent = (int)(absx >> 23) - 127;
  uint32_t mantissa = (absx & 0x7fffffu) | 0x800000u; /* 24-bit significand */
  int shift;                                          /* bits dropped from the significand */
  uint32_t base;
  if (exponent < -14) {
    shift = 13 + (-14 - exponent); /* subnormal: align to 2^-24 units */
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(exponent + 15) << 10;
    mantissa &= 0x7fffffu;
  }
  uint32_t kept = mantissa >> shift;
  const uint32_t rem = mantissa & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (kept & 1u))) kept += 1; /* carry may bump the exponent: intended */
  return (uint16_t)(sign | (base + kept));
}

KQO_API float kqo_round_to_f16(float value) {
  return kqo_f16_bits_to_f32(kqo_f32_to_f16_bits(value));
}

/* f32 -> bfloat16 -> f32 (round-to-nearest-even).  The reference has no bf16
 * compute variant; this supplies the "reference math on pre-rounded inputs"
 * construction (the one packages/runtime/src/kernels/gemm.ts:177-197 uses for its
 * f16-compute variant) for bf16 activations / bf16 dequant tiles. */
KQO_API float kqo_round_to_bf16(float value) {
  uint32_t x;
  memcpy(&x, &value, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) {
    x = (x | 0x00400000u) & 0xffff0000u;
  } else {
    x += 0x7fffu + ((x >> 16) & 1u);
    x &= 0xffff0000u;
  }
  float out;
  memcpy(&out, &x, 4);
  return out;
}

KQO_API void kqo_f16_array_to_f32(const uint16_t* bits, size_t count, float* out) {
  for (size_t i = 0; i < count; ++i) out[i] = kqo_f16_bits_to_f32(bits[i]);
}

KQO_API void kqo_round_array(const float* in, size_t count, int kind /*1=f16, 2=bf16*/, float* out) {
  for (size_t i = 0; i < count; ++i)
    out[i] = kind == 1 ? kqo_round_to_f16(in[i]) : kind == 2 ? kqo_round_to_bf16(in[i]) : in[i];
}

/* ---------------------------------------------------------------------------
 * Storage decoders
 * ------------------------------------------------------------------------- */

/* Packed int4 -> f32.  Follows packages/runtime/src/format/i4.ts:63-118 (decodeI4):
 * flat element i lives in byte i>>1, LOW nibble when i is even, HIGH nibble when
 * odd; stored value u = q + 8; result = fround((u - 8) * scale[row*groups + group])
 * with exactly one f32 rounding (i4.ts:113).  `width` is the row length
 * (numel / shape[0], i4.ts:31) and must be divisible by group_size; the scale is
 * the rank-2 group form [rows, width/group_size] (i4.ts:46-52).
 * Returns 0, or a negative code for the contract violations the reference throws on
 * (byte length is the caller's to check: it is rows*width/2). */
KQO_API int kqo_decode_i4(const uint8_t* bytes, size_t rows, size_t width, const float* scale,
                          size_t group_size, float* out) {
  if (((rows * width) & 1u) != 0) return -1;
  if (group_size < 1 || width % group_size != 0) return -2;
  const size_t groups = width / group_size;
  size_t i = 0;
  for (size_t row = 0; row < rows; ++row) {
    for (size_t group = 0; group < groups; ++group) {
      const float s = scale[row * groups + group];
      for (size_t element = 0; element < group_size; ++element, ++i) {
        const uint8_t byte = bytes[i >> 1];
        const int u = (i & 1u) ? (byte >> 4) : (byte & 0x0f);
        /* (u - 8) * s evaluated exactly in f64, rounded once to f32 (Math.fround) */
        out[i] = (float)((double)(u - 8) * (double)s);
      }
    }
  }
  return 0;
}

/* Signed int8 -> f32 with a keepdim-broadcast scale over a rank-2 view.
 * Follows packages/runtime/src/format/i8.ts:80-117 (decodeI8) and its stride rule
 * i8.ts:49-73 (scaleStrides): an axis of extent 1 has stride 0.  For `linear` the
 * scale is [rows,1] (scale_rows=rows, scale_cols=1).  result = fround(q * s), one
 * rounding (i8.ts:107). */
KQO_API int kqo_decode_i8(const int8_t* bytes, size_t rows, size_t cols, const float* scale,
                          size_t scale_rows, size_t scale_cols, float* out) {
  if ((scale_rows != 1 && scale_rows != rows) || (scale_cols != 1 && scale_cols != cols)) return -1;
  const size_t stride_col = scale_cols == 1 ? 0 : 1;
  const size_t stride_row = scale_rows == 1 ? 0 : scale_cols;
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c)
      out[r * cols + c] =
          (float)((double)bytes[r * cols + c] * (double)scale[r * stride_row + c * stride_col]);
  return 0;
}

/* ---------------------------------------------------------------------------
 * linear
 * ------------------------------------------------------------------------- */

/* out[row,col] = fround( sum_i x[row,i]*w[col,i]  (f64, i ascending)  + bias[col] ).
 * Follows packages/runtime/src/reference/ops.ts:879-897 (referenceLinear): weight is
 * [n,k] un-transposed, accumulation is a plain f64 loop, one fround at the end. */
KQO_API void kqo_linear_f64(const float* x, const float* w, const float* bias, size_t m, size_t n,
                            size_t k, float* out) {
#pragma omp parallel for schedule(static) if (n * k > 65536)
  for (ptrdiff_t col = 0; col < (ptrdiff_t)n; ++col) {
    for (size_t row = 0; row < m; ++row) {
      double acc = 0.0;
      for (size_t i = 0; i < k; ++i) acc += (double)x[row * k + i] * (double)w[(size_t)col * k + i];
      out[row * n + (size_t)col] = (float)(acc + (double)bias[col]);
    }
  }
}

/* Replay of ONE shader invocation's arithmetic in f32: k ascending, acc = acc + a*b,
 * bias added once after the K loop.  Order follows the generated kernel text
 * packages/runtime/tests/fixtures/wgsl/linear_wi4_v4.wgsl:151-171 (inner loop) and
 * :193-215 (bias at store); packages/runtime/src/kernels/gemm-geometry.ts:13-16
 * states that this per-output order does not depend on the tile geometry.
 * fused != 0 evaluates acc + a*b as one fmaf (WGSL lets the compiler contract,
 * packages/runtime/src/kernels/gemm.ts:918-920); fused == 0 rounds the product first. */
KQO_API void kqo_linear_f32_seq(const float* x, const float* w, const float* bias, size_t m,
                                size_t n, size_t k, int fused, float* out) {
#pragma omp parallel for schedule(static) if (n * k > 65536)
  for (ptrdiff_t col = 0; col < (ptrdiff_t)n; ++col) {
    for (size_t row = 0; row < m; ++row) {
      float acc = 0.0f;
      if (fused) {
        for (size_t i = 0; i < k; ++i) acc = fmaf(x[row * k + i], w[(size_t)col * k + i], acc);
      } else {
        for (size_t i = 0; i < k; ++i) {
          volatile float p = x[row * k + i] * w[(size_t)col * k + i];
          acc = acc + p;
        }
      }
      out[row * n + (size_t)col] = acc + bias[col];
    }
  }
}

/* The same f64 linear computed straight from the packed bytes, dequantising each
 * weight with the decodeI4 rule on the fly (so no [n,k] f32 matrix is materialised).
 * Value-identical to kqo_decode_i4 followed by kqo_linear_f64; exists because the
 * large benchmark shapes would need gigabytes expanded.  threads <= 0 means "all
 * the OpenMP runtime gives"; threads == 1 is the scalar port. */
KQO_API void kqo_linear_i4_f64(const float* x, const uint8_t* bytes, const float* scale,
                               const float* bias, size_t m, size_t n, size_t k, size_t group_size,
                               int threads, float* out) {
  const size_t groups = k / group_size;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
#pragma omp parallel for schedule(static)
  for (ptrdiff_t col = 0; col < (ptrdiff_t)n; ++col) {
    const uint8_t* wrow = bytes + ((size_t)col * k >> 1);
    for (size_t row = 0; row < m; ++row) {
      double acc = 0.0;
      for (size_t i = 0; i < k; ++i) {
        const uint8_t byte = wrow[i >> 1];
        const int u = (i & 1u) ? (byte >> 4) : (byte & 0x0f);
        const float wv = (float)((double)(u - 8) * (double)scale[(size_t)col * groups + i / group_size]);
        acc += (double)x[row * k + i] * (double)wv;
      }
      out[row * n + (size_t)col] = (float)(acc + (double)bias[col]);
    }
  }
}

/* Packed-int4 linear in f32, sequential K — the shader's arithmetic, value for value
 * (dequant per element with one f32 multiply as in
 * packages/runtime/src/kernels/weight-storage.ts:159-187, then acc = fma(a, b, acc),
 * bias last).  This is the variant timed as the CPU baseline: it does the work one
 * reference invocation does, on host cores. */
KQO_API void kqo_linear_i4_f32(const float* x, const uint8_t* bytes, const float* scale,
                               const float* bias, size_t m, size_t n, size_t k, size_t group_size,
                               int threads, float* out) {
  const size_t groups = k / group_size;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
#pragma omp parallel for schedule(static)
  for (ptrdiff_t col = 0; col < (ptrdiff_t)n; ++col) {
    const uint8_t* wrow = bytes + ((size_t)col * k >> 1);
    const float* srow = scale + (size_t)col * groups;
    for (size_t row = 0; row < m; ++row) {
      const float* xr = x + row * k;
      float acc = 0.0f;
      for (size_t g = 0; g < groups; ++g) {
        const float s = srow[g];
        for (size_t e = 0; e < group_size; e += 2) {
          const size_t i = g * group_size + e;
          const uint8_t byte = wrow[i >> 1];
          const float w0 = (float)((int)(byte & 0x0f) - 8) * s;
          const float w1 = (float)((int)(byte >> 4) - 8) * s;
          acc = fmaf(xr[i], w0, acc);
          acc = fmaf(xr[i + 1], w1, acc);
        }
      }
      out[row * n + (size_t)col] = acc + bias[col];
    }
  }
}

/* int8 per-output-channel linear, f64 accumulate, from the raw bytes. */
KQO_API void kqo_linear_i8_f64(const float* x, const int8_t* bytes, const float* scale,
                               const float* bias, size_t m, size_t n, size_t k, int threads,
                               float* out) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
#pragma omp parallel for schedule(static)
  for (ptrdiff_t col = 0; col < (ptrdiff_t)n; ++col) {
    const int8_t* wrow = bytes + (size_t)col * k;
    const float s = scale[col];
    for (size_t row = 0; row < m; ++row) {
      double acc = 0.0;
      for (size_t i = 0; i < k; ++i) {
        const float wv = (float)((double)wrow[i] * (double)s);
        acc += (double)x[row * k + i] * (double)wv;
      }
      out[row * n + (size_t)col] = (float)(acc + (double)bias[col]);
    }
  }
}

/* int8 linear in f32, sequential K (shader arithmetic:
 * packages/runtime/src/kernels/weight-storage.ts:191-209). */
KQO_API void kqo_linear_i8_f32(const float* x, const int8_t* bytes, const float* scale,
                               const float* bias, size_t m, size_t n, size_t k, int threads,
                               float* out) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
#pragma omp parallel for schedule(static)
  for (ptrdiff_t col = 0; col < (ptrdiff_t)n; ++col) {
    const int8_t* wrow = bytes + (size_t)col * k;
    const float s = scale[col];
    for (size_t row = 0; row < m; ++row) {
      const float* xr = x + row * k;
      float acc = 0.0f;
      for (size_t i = 0; i < k; ++i) acc = fmaf(xr[i], (float)wrow[i] * s, acc);
      out[row * n + (size_t)col] = acc + bias[col];
    }
  }
}

/* ---------------------------------------------------------------------------
 * allclose
 * ------------------------------------------------------------------------- */

/* |actual - expected| <= atol + rtol*|expected| element-wise; NaN/Inf on either side
 * fails.  Follows packages/runtime/src/reference/allclose.ts:47-82.  report[0] =
 * fail count, [1] = max abs error, [2] = max rel error (denominator floored at
 * 1e-12), [3] = worst index, [4] = non-finite count.  Returns 1 on pass. */
KQO_API int kqo_allclose(const float* actual, const float* expected, size_t count, double atol,
                         double rtol, double* report) {
  size_t fail = 0, non_finite = 0, worst = 0;
  double max_abs = 0.0, max_rel = 0.0;
  for (size_t i = 0; i < count; ++i) {
    const double x = actual[i], y = expected[i];
    if (!isfinite(x) || !isfinite(y)) {
      if (non_finite == 0) worst = i;
      non_finite += 1;
      fail += 1;
      max_abs = INFINITY;
      max_rel = INFINITY;
      continue;
    }
    const double abs_err = fabs(x - y);
    if (abs_err > max_abs && non_finite == 0) {
      max_abs = abs_err;
      worst = i;
    }
    const double denom = fabs(y) > 1e-12 ? fabs(y) : 1e-12;
    if (abs_err / denom > max_rel) max_rel = abs_err / denom;
    if (abs_err > atol + rtol * fabs(y)) fail += 1;
  }
  if (report) {
    report[0] = (double)fail;
    report[1] = max_abs;
    report[2] = max_rel;
    report[3] = (double)worst;
    report[4] = (double)non_finite;
  }
  return fail == 0;
}

/* ---------------------------------------------------------------------------
 * Integer-dot contracts (opt-in `linearCompute: "i8a8"` of the reference)
 * ------------------------------------------------------------------------- */

static float kqo_round_ties_even(float v) { return nearbyintf(v); } /* default FE_TONEAREST */

/* Per-row symmetric int8 activation quantisation.
 * Follows packages/runtime/src/reference/i8a8.ts:87-113 (quantizeRowsReference):
 * s = max(fround(amax * fround(1/127)), f32 tiny), NaN poisons the row scale;
 * q = clamp(round_half_even(fround(x / s)), +-127). */
KQO_API void kqo_quantize_rows(const float* x, size_t rows, size_t dim, int8_t* q, float* scale) {
  const float inv = (float)(1.0 / 127.0);
  const float tiny = 1.1754943508222875e-38f;
  for (size_t row = 0; row < rows; ++row) {
    const float* xr = x + row * dim;
    float amax = 0.0f;
    int saw_nan = 0;
    for (size_t i = 0; i < dim; ++i) {
      const float v = fabsf(xr[i]);
      if (isnan(v)) saw_nan = 1;
      else if (v > amax) amax = v;
    }
    float s = amax * inv;
    if (s < tiny) s = tiny;
    if (saw_nan) s = NAN;
    scale[row] = s;
    for (size_t i = 0; i < dim; ++i) {
      float r = kqo_round_ties_even(xr[i] / s);
      if (!(r >= -127.0f)) r = -127.0f; /* also maps NaN, outside the contract, to a fixed value */
      if (r > 127.0f) r = 127.0f;
      q[row * dim + i] = (int8_t)r;
    }
  }
}

/* w8a8: out = fround(fround(sum xq*wq) * fround(xs[row]*ws[col]) + bias[col]).
 * Follows packages/runtime/src/reference/i8a8.ts:159-175 (referenceLinearI8a8). */
KQO_API void kqo_linear_w8a8(const float* x, const int8_t* wq, const float* wscale,
                             const float* bias, size_t m, size_t n, size_t k, int8_t* xq_scratch,
                             float* xs_scratch, float* out) {
  kqo_quantize_rows(x, m, k, xq_scratch, xs_scratch);
  for (size_t row = 0; row < m; ++row)
    for (size_t col = 0; col < n; ++col) {
      int64_t acc = 0;
      for (size_t i = 0; i < k; ++i) acc += (int64_t)xq_scratch[row * k + i] * (int64_t)wq[col * k + i];
      const float combined = xs_scratch[row] * wscale[col];
      out[row * n + col] = (float)((double)(float)acc * (double)combined + (double)bias[col]);
    }
}

/* w4a8: per group an exact integer sum flushed with one fma, groups ascending;
 * the row scale enters only in the last fma.
 * Follows packages/runtime/src/reference/i8a8.ts:209-229 (referenceLinearW4a8).
 * `wq` holds the signed values (u - 8), one per byte. */
KQO_API void kqo_linear_w4a8(const float* x, const int8_t* wq, const float* wscale,
                             const float* bias, size_t m, size_t n, size_t k, size_t group_size,
                             int8_t* xq_scratch, float* xs_scratch, float* out) {
  const size_t groups = k / group_size;
  kqo_quantize_rows(x, m, k, xq_scratch, xs_scratch);
  for (size_t row = 0; row < m; ++row)
    for (size_t col = 0; col < n; ++col) {
      float accf = 0.0f;
      for (size_t g = 0; g < groups; ++g) {
        int64_t acci = 0;
        for (size_t i = g * group_size; i < (g + 1) * group_size; ++i)
          acci += (int64_t)xq_scratch[row * k + i] * (int64_t)wq[col * k + i];
        accf = (float)((double)(float)acci * (double)wscale[col * groups + g] + (double)accf);
      }
      out[row * n + col] = (float)((double)accf * (double)xs_scratch[row] + (double)bias[col]);
    }
}

/* ---------------------------------------------------------------------------
 * The matmul's neighbours in a decoder layer (rms_norm, SiLU gate, residual add)
 * ------------------------------------------------------------------------- */

/* rms_norm over the last dimension, weight only.
 * Follows packages/runtime/src/reference/ops.ts:948-972 (referenceRmsNorm): the squares are
 * summed in f64, inv = 1 / sqrt(mean + eps) (the mean is NOT subtracted, eps sits inside
 * the root), and each output is x * inv * weight evaluated in f64 and rounded to f32 once. */
KQO_API void kqo_rms_norm(const float* x, const float* weight, size_t rows, size_t dim, double eps, float* out) {
  for (size_t row = 0; row < rows; ++row) {
    const float* xr = x + row * dim;
    double squares = 0.0;
    for (size_t i = 0; i < dim; ++i) squares += (double)xr[i] * (double)xr[i];
    const double inv = 1.0 / sqrt(squares / (double)dim + eps);
    for (size_t i = 0; i < dim; ++i) out[row * dim + i] = (float)((double)xr[i] * inv * (double)weight[i]);
  }
}

/* sigmoid, the reference's unary table entry: f32(1 / (1 + exp(-x))) with the exponential in
 * f64 (packages/runtime/src/reference/ops.ts:150). */
KQO_API void kqo_sigmoid(const float* x, size_t n, float* out) {
  for (size_t i = 0; i < n; ++i) out[i] = (float)(1.0 / (1.0 + exp(-(double)x[i])));
}

/* SwiGLU as the reference's graph spells it: sigmoid(gate) -> mul(gate, sigmoid) -> mul(.., up),
 * three f32 nodes, each result rounded to f32 (the SiLU pair is what the fusion rule `silu`
 * of packages/runtime/src/runtime/fusion.ts:453-511 replaces; it keeps the intermediate
 * f32 rounding of the sigmoid, packages/runtime/src/kernels/silu.ts:1-20). */
KQO_API void kqo_silu_mul(const float* gate, const float* up, size_t n, float* out) {
  for (size_t i = 0; i < n; ++i) {
    const float s = (float)(1.0 / (1.0 + exp(-(double)gate[i])));
    const float a = (float)((double)gate[i] * (double)s);
    out[i] = (float)((double)a * (double)up[i]);
  }
}

/* residual add: one f32 addition per element (the `add` node). */
KQO_API void kqo_add(const float* a, const float* b, size_t n, float* out) {
  for (size_t i = 0; i < n; ++i) out[i] = (float)((double)a[i] + (double)b[i]);
}


KQO_API int kqo_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
