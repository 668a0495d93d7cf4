/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference's NVFP4 CPU path.
 *
 * This file is the parity oracle for the sm_100a kernels.  It is not part of
 * the product: only the test-suite, the smoke check and the CPU-baseline legs
 * of the benchmark may load it.  Every function cites the reference source it
 * restates (paths are relative to the reference project root).
 *
 * Parity status: PINNED.  The codec is checked against the reference's own
 * known-answer tests (crates/nml-parameter/tests/parameter_contract.rs:84-131),
 * the quantizer byte-for-byte against the reference's Python quantizer
 * (tools/nvfp4/convert.py:357-410) through committed golden fixtures, and the
 * kernels against the closed-form cases of
 * crates/nml-kernel-nvfp4/tests/cpu_contract.rs and
 * crates/nml/tests/nvfp4_contract.rs.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: the reference multiplies and then adds (no FMA)
 * in its AVX2 dot product, and the routing exponential below must evaluate
 * with exactly the operations written.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define NML_BLOCK 16

#if defined(__x86_64__)
#include <immintrin.h>
#define NML_HAVE_AVX2_PATH 1
#else
#define NML_HAVE_AVX2_PATH 0
#endif

/* ------------------------------------------------------------------ codec */

/* crates/nml-parameter/src/lib.rs:391 (E2M1_MAGNITUDES) and :416-426. */
static const float kE2M1Magnitude[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

float nml_oracle_decode_e2m1(uint8_t code) {
  const float magnitude = kE2M1Magnitude[code & 0x07];
  return (code & 0x08) ? -magnitude : magnitude;
}

/* crates/nml-parameter/src/lib.rs:448-461.  Returns 0 when the byte is not a
 * valid unsigned E4M3FN scale (sign bit set or the NaN pattern 0x7f). */
int nml_oracle_decode_e4m3fn_scale(uint8_t bits, float *value) {
  if (bits & 0x80) return 0;
  const int exponent = (bits >> 3) & 0x0f;
  const int fraction = bits & 0x07;
  if (exponent == 0x0f && fraction == 0x07) return 0;
  if (exponent == 0) {
    *value = (float)fraction * 0x1p-9f;
  } else {
    *value = (1.0f + (float)fraction / 8.0f) * ldexpf(1.0f, exponent - 7);
  }
  return 1;
}

/* crates/nml-parameter/src/lib.rs:463-481: nearest of the 127 valid codes,
 * ties to the even code.  The search visits codes in increasing order, which
 * is also increasing value order, so a later candidate wins only when it is
 * strictly closer or equally close with an even code replacing an odd one. */
uint8_t nml_oracle_encode_e4m3fn_scale(float value) {
  uint8_t best = 0;
  float best_distance = INFINITY;
  for (int bits = 0; bits <= 0x7e; ++bits) {
    float candidate;
    nml_oracle_decode_e4m3fn_scale((uint8_t)bits, &candidate);
    const float distance = fabsf(value - candidate);
    if (distance < best_distance ||
        (distance == best_distance && (bits & 1) == 0 && (best & 1) != 0)) {
      best = (uint8_t)bits;
      best_distance = distance;
    }
  }
  return best;
}

/* crates/nml-parameter/src/lib.rs:428-446. */
uint8_t nml_oracle_encode_e2m1(float value) {
  const uint8_t sign = (uint8_t)(signbit(value) ? 0x08 : 0x00);
  const float magnitude = fabsf(value);
  uint8_t best = 0;
  float best_distance = INFINITY;
  for (int code = 0; code < 8; ++code) {
    const float distance = fabsf(magnitude - kE2M1Magnitude[code]);
    if (distance < best_distance ||
        (distance == best_distance && (code & 1) == 0 && (best & 1) != 0)) {
      best = (uint8_t)code;
      best_distance = distance;
    }
  }
  return (uint8_t)(sign | best);
}

/* crates/nml-parameter/src/lib.rs:483-500: amax / (448 * 6), 1.0 when all zero.
 * Returns NaN when a value is not finite (the reference returns an error). */
float nml_oracle_global_scale(const float *values, size_t count) {
  float maximum = 0.0f;
  for (size_t i = 0; i < count; ++i) {
    if (!isfinite(values[i])) return NAN;
    const float magnitude = fabsf(values[i]);
    if (magnitude > maximum) maximum = magnitude;
  }
  return maximum == 0.0f ? 1.0f : maximum / (448.0f * 6.0f);
}

/* crates/nml-parameter/src/lib.rs:502-538.  payload has ceil(width/2) bytes,
 * scales ceil(width/16) bytes.  Low nibble holds the even column. */
void nml_oracle_quantize_row(const float *values, size_t width, float global_scale,
                             uint8_t *payload, uint8_t *scales) {
  memset(payload, 0, (width + 1) / 2);
  const size_t blocks = (width + NML_BLOCK - 1) / NML_BLOCK;
  for (size_t block = 0; block < blocks; ++block) {
    const size_t start = block * NML_BLOCK;
    const size_t end = start + NML_BLOCK < width ? start + NML_BLOCK : width;
    float block_amax = 0.0f;
    for (size_t i = start; i < end; ++i) {
      const float magnitude = fabsf(values[i]);
      if (magnitude > block_amax) block_amax = magnitude;
    }
    const float unrounded = (block_amax / 6.0f) / global_scale;
    const uint8_t scale_bits = nml_oracle_encode_e4m3fn_scale(unrounded);
    float block_scale;
    nml_oracle_decode_e4m3fn_scale(scale_bits, &block_scale);
    scales[block] = scale_bits;
    for (size_t i = start; i < end; ++i) {
      const uint8_t code =
          block_scale == 0.0f ? 0 : nml_oracle_encode_e2m1(values[i] / (block_scale * global_scale));
      if ((i & 1) == 0) {
        payload[i / 2] = code;
      } else {
        payload[i / 2] |= (uint8_t)(code << 4);
      }
    }
  }
}

/* Whole-tensor quantizer in the way the reference tests drive the row codec
 * (crates/nml-kernel-nvfp4/tests/cpu_contract.rs:12-28): one global scale for
 * the tensor, then row by row.  Returns the global scale. */
float nml_oracle_quantize_tensor(const float *values, size_t rows, size_t width,
                                 uint8_t *payload, uint8_t *scales) {
  const float global = nml_oracle_global_scale(values, rows * width);
  const size_t packed = (width + 1) / 2, scale_width = (width + NML_BLOCK - 1) / NML_BLOCK;
#pragma omp parallel for schedule(static)
  for (long long row = 0; row < (long long)rows; ++row) {
    nml_oracle_quantize_row(values + (size_t)row * width, width, global,
                            payload + (size_t)row * packed, scales + (size_t)row * scale_width);
  }
  return global;
}

static inline uint8_t nibble_at(const uint8_t *payload, size_t row_offset, size_t column) {
  const uint8_t byte = payload[row_offset + column / 2];
  return (column & 1) == 0 ? (uint8_t)(byte & 0x0f) : (uint8_t)(byte >> 4);
}

/* crates/nml-kernel-nvfp4/src/lib.rs:110-187 (Weight::new).  Return codes:
 * 0 ok, 1 invalid global scale, 2 nonzero pad nibble, 3 invalid scale byte,
 * 4 zero-scale block with a nonzero magnitude. */
int nml_oracle_validate_weight(const uint8_t *payload, const uint8_t *scales, float global_scale,
                               size_t rows, size_t width) {
  if (!isfinite(global_scale) || global_scale <= 0.0f) return 1;
  const size_t packed = (width + 1) / 2, scale_width = (width + NML_BLOCK - 1) / NML_BLOCK;
  for (size_t row = 0; row < rows; ++row) {
    if ((width & 1) && (payload[row * packed + packed - 1] & 0xf0)) return 2;
    for (size_t block = 0; block < scale_width; ++block) {
      float scale;
      if (!nml_oracle_decode_e4m3fn_scale(scales[row * scale_width + block], &scale)) return 3;
      if (scale == 0.0f) {
        const size_t start = block * NML_BLOCK;
        const size_t end = start + NML_BLOCK < width ? start + NML_BLOCK : width;
        for (size_t column = start; column < end; ++column) {
          if (nibble_at(payload, row * packed, column) & 0x07) return 4;
        }
      }
    }
  }
  return 0;
}

/* crates/nml-kernel-nvfp4/src/lib.rs:193-200 (Weight::value): the effective
 * scale fl(block_scale * global_scale) is formed first, then multiplied by the
 * code value.  crates/nml-parameter/src/lib.rs:574-578 documents the same
 * association for dequantize_row. */
static inline float weight_value(const uint8_t *payload, const uint8_t *scales, float global_scale,
                                 size_t packed, size_t scale_width, size_t row, size_t column) {
  float scale = 0.0f;
  nml_oracle_decode_e4m3fn_scale(scales[row * scale_width + column / NML_BLOCK], &scale);
  return nml_oracle_decode_e2m1(nibble_at(payload, row * packed, column)) * (scale * global_scale);
}

/* crates/nml-parameter/src/lib.rs:540-588.  Returns 0 on success, nonzero for
 * the error cases the reference rejects (pad nibble, invalid scale byte,
 * zero scale with a nonzero magnitude). */
int nml_oracle_dequantize_row(const uint8_t *payload, const uint8_t *scales, float global_scale,
                              size_t width, float *out) {
  if (!isfinite(global_scale) || global_scale <= 0.0f) return 1;
  if ((width & 1) && (payload[(width + 1) / 2 - 1] & 0xf0)) return 2;
  for (size_t i = 0; i < width; ++i) {
    float scale;
    if (!nml_oracle_decode_e4m3fn_scale(scales[i / NML_BLOCK], &scale)) return 3;
    const uint8_t code = nibble_at(payload, 0, i);
    if (scale == 0.0f && (code & 0x07)) return 4;
    out[i] = nml_oracle_decode_e2m1(code) * (scale * global_scale);
  }
  return 0;
}

/* --------------------------------------------------------- 16-bit floats */

/* crates/nml-types/src/lib.rs:117-125: round to nearest even, NaN kept quiet. */
uint16_t nml_oracle_bf16_from_f32(float value) {
  uint32_t bits;
  memcpy(&bits, &value, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040);
  const uint32_t upper = bits >> 16;
  const uint32_t rounding_bias = 0x7fffu + (upper & 1u);
  return (uint16_t)((bits + rounding_bias) >> 16);
}

float nml_oracle_bf16_to_f32(uint16_t bits) {
  const uint32_t wide = (uint32_t)bits << 16;
  float value;
  memcpy(&value, &wide, 4);
  return value;
}

/* IEEE binary16, round to nearest even (the reference's F16::from_f32,
 * crates/nml-types/src/lib.rs, is the same standard conversion). */
uint16_t nml_oracle_f16_from_f32(float value) {
  uint32_t bits;
  memcpy(&bits, &value, 4);
  const uint32_t sign = (bits >> 16) & 0x8000u;
  const uint32_t magnitude = bits & 0x7fffffffu;
  if (magnitude > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
  if (magnitude >= 0x47800000u) return (uint16_t)(sign | 0x7c00u); /* >= 65536 -> inf */
  if (magnitude < 0x38800000u) {                                   /* below 2^-14: subnormal */
    if (magnitude < 0x33000000u) return (uint16_t)sign;           /* below 2^-25 */
    const int exponent = (int)(magnitude >> 23);
    const uint32_t mantissa = (magnitude & 0x7fffffu) | 0x800000u;
    const int shift = 126 - exponent; /* 14..24 */
    uint32_t result = mantissa >> shift;
    const uint32_t remainder = mantissa & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    if (remainder > halfway || (remainder == halfway && (result & 1u))) ++result;
    return (uint16_t)(sign | result);
  }
  uint32_t result = (magnitude - 0x38000000u) >> 13;
  const uint32_t remainder = magnitude & 0x1fffu;
  if (remainder > 0x1000u || (remainder == 0x1000u && (result & 1u))) ++result;
  return (uint16_t)(sign | result); /* a carry into 0x7c00 is the correct infinity */
}

float nml_oracle_f16_to_f32(uint16_t bits) {
  const uint32_t sign = ((uint32_t)bits & 0x8000u) << 16;
  const uint32_t exponent = (bits >> 10) & 0x1fu;
  const uint32_t mantissa = bits & 0x3ffu;
  uint32_t wide;
  if (exponent == 0) {
    if (mantissa == 0) {
      wide = sign;
    } else {
      float value = (float)mantissa * 0x1p-24f;
      memcpy(&wide, &value, 4);
      wide |= sign;
    }
  } else if (exponent == 0x1f) {
    wide = sign | 0x7f800000u | (mantissa << 13);
  } else {
    wide = sign | ((exponent + 112u) << 23) | (mantissa << 13);
  }
  float value;
  memcpy(&value, &wide, 4);
  return value;
}

/* dtype codes follow the kernel ABI: 1 = f16, 2 = bf16. */
static inline float load16(const uint16_t *data, size_t index, int dtype) {
  return dtype == 1 ? nml_oracle_f16_to_f32(data[index]) : nml_oracle_bf16_to_f32(data[index]);
}
static inline uint16_t store16(float value, int dtype) {
  return dtype == 1 ? nml_oracle_f16_from_f32(value) : nml_oracle_bf16_from_f32(value);
}

void nml_oracle_to_f32(const uint16_t *data, size_t count, int dtype, float *out) {
  for (size_t i = 0; i < count; ++i) out[i] = load16(data, i, dtype);
}
void nml_oracle_from_f32(const float *data, size_t count, int dtype, uint16_t *out) {
  for (size_t i = 0; i < count; ++i) out[i] = store16(data[i], dtype);
}

/* -------------------------------------------------------------- kernels */

/* crates/nml-kernel-nvfp4/src/lib.rs:204-224,466-485 and x86.rs:61-75.
 * Returns 0, or 1 + the offending position when an index is out of range
 * (the reference returns IndexOutOfBounds). */
long long nml_oracle_embedding(const int64_t *indices, size_t count, const uint8_t *payload,
                               const uint8_t *scales, float global_scale, size_t vocabulary,
                               size_t width, float *out) {
  const size_t packed = (width + 1) / 2, scale_width = (width + NML_BLOCK - 1) / NML_BLOCK;
  for (size_t i = 0; i < count; ++i) {
    if (indices[i] < 0 || (uint64_t)indices[i] >= vocabulary) return 1 + (long long)i;
  }
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)count; ++i) {
    const size_t row = (size_t)indices[i];
    for (size_t column = 0; column < width; ++column) {
      out[(size_t)i * width + column] =
          weight_value(payload, scales, global_scale, packed, scale_width, row, column);
    }
  }
  return 0;
}

/* crates/nml-kernel-nvfp4/src/x86.rs:82-100 (dot_row, the implementation the
 * reference selects on any AVX2 host, lib.rs:35-43): eight f32 lanes, each
 * block contributes lanes += x[0..8]*w[0..8] then lanes += x[8..16]*w[8..16]
 * as separate multiply and add; lanes are then summed in lane order and the
 * columns past the last whole block are added one by one. */
static float dot_row_scalar_order(const uint8_t *payload, const uint8_t *scales,
                                  float global_scale, size_t packed, size_t scale_width,
                                  size_t width, size_t row, const float *input) {
  float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const size_t vector_width = width / NML_BLOCK * NML_BLOCK;
  for (size_t block_start = 0; block_start < vector_width; block_start += NML_BLOCK) {
    float scale = 0.0f;
    nml_oracle_decode_e4m3fn_scale(scales[row * scale_width + block_start / NML_BLOCK], &scale);
    const float effective = scale * global_scale;
    const uint8_t *bytes = payload + row * packed + block_start / 2;
    float decoded[16];
    for (int i = 0; i < 8; ++i) {
      decoded[2 * i] = nml_oracle_decode_e2m1((uint8_t)(bytes[i] & 0x0f)) * effective;
      decoded[2 * i + 1] = nml_oracle_decode_e2m1((uint8_t)(bytes[i] >> 4)) * effective;
    }
    for (int lane = 0; lane < 8; ++lane) {
      const float product = input[block_start + lane] * decoded[lane];
      lanes[lane] = lanes[lane] + product;
    }
    for (int lane = 0; lane < 8; ++lane) {
      const float product = input[block_start + 8 + lane] * decoded[8 + lane];
      lanes[lane] = lanes[lane] + product;
    }
  }
  float sum = 0.0f;
  for (int lane = 0; lane < 8; ++lane) sum += lanes[lane];
  for (size_t column = vector_width; column < width; ++column) {
    sum += input[column] *
           weight_value(payload, scales, global_scale, packed, scale_width, row, column);
  }
  return sum;
}

#if NML_HAVE_AVX2_PATH
/* The same arithmetic with AVX2 registers, so that the CPU baseline runs at the speed class
 * of the reference's own AVX2 kernel: identical operations in identical order (one multiply
 * by the effective scale per value, then multiply and add per lane), hence identical bits to
 * dot_row_scalar_order.  Magnitudes come from an in-register 8-entry table and the sign bit
 * is OR-ed in, instead of the reference's 16-entry memory gather. */
__attribute__((target("avx2"))) static float dot_row_avx2(
    const uint8_t *payload, const uint8_t *scales, float global_scale, size_t packed,
    size_t scale_width, size_t width, size_t row, const float *input,
    const float *scale_table) {
  const __m256 magnitudes = _mm256_setr_ps(0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f);
  const __m256i seven = _mm256_set1_epi32(7);
  const __m256i eight = _mm256_set1_epi32(8);
  const __m128i nibble_mask = _mm_set1_epi8(0x0f);
  __m256 lanes = _mm256_setzero_ps();
  const size_t vector_width = width / NML_BLOCK * NML_BLOCK;
  const uint8_t *row_payload = payload + row * packed;
  const uint8_t *row_scales = scales + row * scale_width;
  for (size_t block_start = 0; block_start < vector_width; block_start += NML_BLOCK) {
    const __m256 effective =
        _mm256_set1_ps(scale_table[row_scales[block_start / NML_BLOCK]] * global_scale);
    const __m128i bytes = _mm_loadl_epi64((const __m128i *)(row_payload + block_start / 2));
    const __m128i low = _mm_and_si128(bytes, nibble_mask);
    const __m128i high = _mm_and_si128(_mm_srli_epi16(bytes, 4), nibble_mask);
    const __m128i codes = _mm_unpacklo_epi8(low, high); /* 16 codes in column order */
    const __m256i first = _mm256_cvtepu8_epi32(codes);
    const __m256i second = _mm256_cvtepu8_epi32(_mm_srli_si128(codes, 8));
    const __m256 sign_first =
        _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_and_si256(first, eight), 28));
    const __m256 sign_second =
        _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_and_si256(second, eight), 28));
    const __m256 value_first = _mm256_or_ps(
        _mm256_permutevar8x32_ps(magnitudes, _mm256_and_si256(first, seven)), sign_first);
    const __m256 value_second = _mm256_or_ps(
        _mm256_permutevar8x32_ps(magnitudes, _mm256_and_si256(second, seven)), sign_second);
    const __m256 weight_first = _mm256_mul_ps(value_first, effective);
    const __m256 weight_second = _mm256_mul_ps(value_second, effective);
    lanes = _mm256_add_ps(lanes, _mm256_mul_ps(_mm256_loadu_ps(input + block_start),
                                               weight_first));
    lanes = _mm256_add_ps(lanes, _mm256_mul_ps(_mm256_loadu_ps(input + block_start + 8),
                                               weight_second));
  }
  float lane_values[8];
  _mm256_storeu_ps(lane_values, lanes);
  float sum = 0.0f;
  for (int lane = 0; lane < 8; ++lane) sum += lane_values[lane];
  for (size_t column = vector_width; column < width; ++column) {
    sum += input[column] *
           weight_value(payload, scales, global_scale, packed, scale_width, row, column);
  }
  return sum;
}
#endif

static float g_scale_table[256];
static int g_scale_table_ready = 0;
static int g_use_avx2 = -1;

static void prepare_tables(void) {
  if (!g_scale_table_ready) {
    for (int bits = 0; bits < 256; ++bits) {
      float value = 0.0f;
      if (!nml_oracle_decode_e4m3fn_scale((uint8_t)bits, &value)) value = NAN;
      g_scale_table[bits] = value;
    }
    g_scale_table_ready = 1;
  }
  if (g_use_avx2 < 0) {
#if NML_HAVE_AVX2_PATH
    g_use_avx2 = __builtin_cpu_supports("avx2") ? 1 : 0;
#else
    g_use_avx2 = 0;
#endif
  }
}

/* 1: use the AVX2 evaluation when the host has it (default); 0: scalar evaluation. */
void nml_oracle_set_avx2(int enabled) {
  prepare_tables();
#if NML_HAVE_AVX2_PATH
  g_use_avx2 = (enabled && __builtin_cpu_supports("avx2")) ? 1 : 0;
#else
  (void)enabled;
#endif
}

static float dot_row_avx2_order(const uint8_t *payload, const uint8_t *scales, float global_scale,
                                size_t packed, size_t scale_width, size_t width, size_t row,
                                const float *input) {
#if NML_HAVE_AVX2_PATH
  if (g_use_avx2 == 1) {
    return dot_row_avx2(payload, scales, global_scale, packed, scale_width, width, row, input,
                        g_scale_table);
  }
#endif
  return dot_row_scalar_order(payload, scales, global_scale, packed, scale_width, width, row,
                              input);
}

/* f64 accumulation of the same terms, the independent oracle the reference's
 * own tests use (crates/nml-kernel-nvfp4/tests/cpu_contract.rs:44-85). */
static double dot_row_f64(const uint8_t *payload, const uint8_t *scales, float global_scale,
                          size_t packed, size_t scale_width, size_t width, size_t row,
                          const float *input) {
  double sum = 0.0;
  for (size_t column = 0; column < width; ++column) {
    float scale = 0.0f;
    nml_oracle_decode_e4m3fn_scale(scales[row * scale_width + column / NML_BLOCK], &scale);
    const double value = (double)nml_oracle_decode_e2m1(nibble_at(payload, row * packed, column)) *
                         (double)scale * (double)global_scale;
    sum += (double)input[column] * value;
  }
  return sum;
}

/* crates/nml-kernel-nvfp4/src/lib.rs:227-266.  input [rows, inputs] f32,
 * weight [outputs, inputs], bias [outputs] or NULL, out [rows, outputs].
 * mode 0: the reference's f32 order; mode 1: f64 accumulation. */
void nml_oracle_linear(const float *input, size_t rows, const uint8_t *payload,
                       const uint8_t *scales, float global_scale, size_t outputs, size_t inputs,
                       const float *bias, float *out, int mode) {
  prepare_tables();
  const size_t packed = (inputs + 1) / 2, scale_width = (inputs + NML_BLOCK - 1) / NML_BLOCK;
#pragma omp parallel for schedule(static) collapse(2)
  for (long long row = 0; row < (long long)rows; ++row) {
    for (long long output = 0; output < (long long)outputs; ++output) {
      const float *input_row = input + (size_t)row * inputs;
      const float b = bias ? bias[output] : 0.0f;
      if (mode == 0) {
        out[(size_t)row * outputs + (size_t)output] =
            b + dot_row_avx2_order(payload, scales, global_scale, packed, scale_width, inputs,
                                   (size_t)output, input_row);
      } else {
        out[(size_t)row * outputs + (size_t)output] =
            (float)((double)b + dot_row_f64(payload, scales, global_scale, packed, scale_width,
                                            inputs, (size_t)output, input_row));
      }
    }
  }
}

/* The CPU custom-call handler around `linear`
 * (crates/nml-kernel-nvfp4/src/ffi.rs:104-226,556-613): 16-bit activations and
 * bias widen to f32, the f32 result narrows with round-to-nearest-even.
 * out16 receives the narrowed output, out32 (optional) the f32 values before
 * narrowing. */
void nml_oracle_linear_16(const uint16_t *input, size_t rows, const uint8_t *payload,
                          const uint8_t *scales, float global_scale, size_t outputs,
                          size_t inputs, const uint16_t *bias, int dtype, uint16_t *out16,
                          float *out32, int mode) {
  float *wide = (float *)malloc(sizeof(float) * rows * inputs);
  float *result = out32 ? out32 : (float *)malloc(sizeof(float) * rows * outputs);
  float *wide_bias = NULL;
  nml_oracle_to_f32(input, rows * inputs, dtype, wide);
  if (bias) {
    wide_bias = (float *)malloc(sizeof(float) * outputs);
    nml_oracle_to_f32(bias, outputs, dtype, wide_bias);
  }
  nml_oracle_linear(wide, rows, payload, scales, global_scale, outputs, inputs, wide_bias, result,
                    mode);
  if (out16) nml_oracle_from_f32(result, rows * outputs, dtype, out16);
  free(wide);
  free(wide_bias);
  if (!out32) free(result);
}

/* crates/nml-kernel-nvfp4/src/lib.rs:450-464 (project_expert). */
static void project_expert(const float *input, size_t expert, const uint8_t *payload,
                           const uint8_t *scales, float global_scale, size_t outputs,
                           size_t inputs, const float *bias, float *out, int mode) {
  const size_t packed = (inputs + 1) / 2, scale_width = (inputs + NML_BLOCK - 1) / NML_BLOCK;
  for (size_t output = 0; output < outputs; ++output) {
    const size_t row = expert * outputs + output;
    const float b = bias ? bias[output] : 0.0f;
    if (mode == 0) {
      out[output] = b + dot_row_avx2_order(payload, scales, global_scale, packed, scale_width,
                                           inputs, row, input);
    } else {
      out[output] = (float)((double)b + dot_row_f64(payload, scales, global_scale, packed,
                                                    scale_width, inputs, row, input));
    }
  }
}

/* crates/nml-kernel-nvfp4/src/lib.rs:272-324.  Returns 0 or 1 + assignment
 * index of an out-of-range expert. */
long long nml_oracle_grouped_projection(const float *input, const int64_t *expert_indices,
                                        size_t assignments, const uint8_t *payload,
                                        const uint8_t *scales, float global_scale, size_t experts,
                                        size_t outputs, size_t inputs, const float *bias,
                                        float *out, int mode) {
  prepare_tables();
  for (size_t a = 0; a < assignments; ++a) {
    if (expert_indices[a] < 0 || (uint64_t)expert_indices[a] >= experts) return 1 + (long long)a;
  }
#pragma omp parallel for schedule(dynamic)
  for (long long a = 0; a < (long long)assignments; ++a) {
    const size_t expert = (size_t)expert_indices[a];
    project_expert(input + (size_t)a * inputs, expert, payload, scales, global_scale, outputs,
                   inputs, bias ? bias + expert * outputs : NULL, out + (size_t)a * outputs, mode);
  }
  return 0;
}

/* crates/nml-kernel-nvfp4/src/lib.rs:333-448.  hidden [tokens, H] f32, router
 * indices/weights [tokens*k], gate_up [E, 2I, H] with gate/up rows
 * interleaved, down [E, H, I]; out [tokens, H] f32.  The activation stays f32
 * between the two projections.  Accumulation over routes follows route order.
 * Returns 0 or 1 + assignment index of an out-of-range expert. */
long long nml_oracle_routed_clamped_swiglu(
    const float *hidden, size_t tokens, const int64_t *router_indices,
    const float *routing_weights, size_t top_k, const uint8_t *gate_payload,
    const uint8_t *gate_scales, float gate_global, const float *gate_bias,
    const uint8_t *down_payload, const uint8_t *down_scales, float down_global,
    const float *down_bias, size_t experts, size_t hidden_size, size_t intermediate, float *out,
    int mode) {
  prepare_tables();
  const size_t doubled = 2 * intermediate;
  for (size_t a = 0; a < tokens * top_k; ++a) {
    if (router_indices[a] < 0 || (uint64_t)router_indices[a] >= experts) return 1 + (long long)a;
  }
  memset(out, 0, sizeof(float) * tokens * hidden_size);
#pragma omp parallel
  {
    float *gate_up = (float *)malloc(sizeof(float) * doubled);
    float *activated = (float *)malloc(sizeof(float) * intermediate);
    float *projected = (float *)malloc(sizeof(float) * hidden_size);
#pragma omp for schedule(dynamic)
    for (long long token = 0; token < (long long)tokens; ++token) {
      const float *input = hidden + (size_t)token * hidden_size;
      for (size_t route = 0; route < top_k; ++route) {
        const size_t assignment = (size_t)token * top_k + route;
        const size_t expert = (size_t)router_indices[assignment];
        project_expert(input, expert, gate_payload, gate_scales, gate_global, doubled, hidden_size,
                       gate_bias + expert * doubled, gate_up, mode);
        for (size_t i = 0; i < intermediate; ++i) {
          const float gate = fminf(gate_up[2 * i], 7.0f);
          float up = gate_up[2 * i + 1];
          up = up < -7.0f ? -7.0f : (up > 7.0f ? 7.0f : up);
          const float swish = gate * (1.0f / (1.0f + expf(-1.702f * gate)));
          activated[i] = (up + 1.0f) * swish;
        }
        project_expert(activated, expert, down_payload, down_scales, down_global, hidden_size,
                       intermediate, down_bias + expert * hidden_size, projected, mode);
        const float weight = routing_weights[assignment];
        for (size_t h = 0; h < hidden_size; ++h) {
          out[(size_t)token * hidden_size + h] += weight * projected[h];
        }
      }
    }
    free(gate_up);
    free(activated);
    free(projected);
  }
  return 0;
}

/* The device kernels split the routed layer in two custom calls and round the
 * intermediate tensors to the activation dtype (reference GPU semantics,
 * crates/nml-kernel-nvfp4/src/turing_adapter.cu:344-365 for gate/up,
 * :438-455 for down, and crates/nml-ir/src/nvfp4_backend.rs:486-508 for the
 * k-way sum in the activation dtype).  These two helpers restate exactly those
 * stages so each device kernel can be checked on its own.
 *
 * gate/up: activated[a, i] for every assignment a with expert_ids[a] >= 0;
 * rows of masked assignments (expert -1) are left untouched. */
void nml_oracle_expert_gate_up(const float *hidden, const int32_t *expert_ids, size_t assignments,
                               size_t top_k, const uint8_t *payload, const uint8_t *scales,
                               float global_scale, const float *bias, size_t hidden_size,
                               size_t intermediate, float *activated, int mode) {
  prepare_tables();
  const size_t doubled = 2 * intermediate;
#pragma omp parallel
  {
    float *gate_up = (float *)malloc(sizeof(float) * doubled);
#pragma omp for schedule(dynamic)
    for (long long a = 0; a < (long long)assignments; ++a) {
      if (expert_ids[a] < 0) continue;
      const size_t expert = (size_t)expert_ids[a];
      project_expert(hidden + ((size_t)a / top_k) * hidden_size, expert, payload, scales,
                     global_scale, doubled, hidden_size, bias + expert * doubled, gate_up, mode);
      for (size_t i = 0; i < intermediate; ++i) {
        const float gate = fminf(gate_up[2 * i], 7.0f);
        float up = gate_up[2 * i + 1];
        up = up < -7.0f ? -7.0f : (up > 7.0f ? 7.0f : up);
        /* turing_adapter.cu:360 divides; lib.rs:427 multiplies by the
         * reciprocal.  The two differ by at most one f32 ulp. */
        const float swish = gate * (1.0f / (1.0f + expf(-1.702f * gate)));
        activated[(size_t)a * intermediate + i] = (up + 1.0f) * swish;
      }
    }
    free(gate_up);
  }
}

/* down: weighted[a, h] = (act[a,:] . W_down[e, h, :] + bias[e, h]) * w[a]. */
void nml_oracle_expert_down(const float *activated, const int32_t *expert_ids,
                            const float *routing_weights, size_t assignments,
                            const uint8_t *payload, const uint8_t *scales, float global_scale,
                            const float *bias, size_t hidden_size, size_t intermediate,
                            float *weighted, int mode) {
  prepare_tables();
#pragma omp parallel
  {
    float *projected = (float *)malloc(sizeof(float) * hidden_size);
#pragma omp for schedule(dynamic)
    for (long long a = 0; a < (long long)assignments; ++a) {
      if (expert_ids[a] < 0) continue;
      const size_t expert = (size_t)expert_ids[a];
      project_expert(activated + (size_t)a * intermediate, expert, payload, scales, global_scale,
                     hidden_size, intermediate, bias + expert * hidden_size, projected, mode);
      for (size_t h = 0; h < hidden_size; ++h) {
        weighted[(size_t)a * hidden_size + h] = projected[h] * routing_weights[a];
      }
    }
    free(projected);
  }
}

/* ---------------------------------------------------------------- routing */

/* A base-e exponential built only from IEEE operations that are correctly
 * rounded everywhere (fmaf, multiply, add, rintf, exponent-field arithmetic),
 * so the CPU oracle and the CUDA routing kernel produce the same bits and
 * therefore the same ties.  The reference lowers softmax to stablehlo.exp
 * (crates/nml-ir/src/lib.rs:4109-4137), whose bits depend on the XLA backend;
 * what the reference fixes is the selection rule applied to those values.
 * Valid for x <= 0 (softmax arguments after the row maximum is subtracted);
 * returns 0 below -87.3.  Relative error about 1e-7. */
float nml_oracle_exp_det(float x) {
  if (!(x > -87.3f)) return 0.0f; /* also maps NaN to 0 */
  if (x > 0.0f) x = 0.0f;
  const float n = rintf(x * 1.44269504088896341f);
  float r = fmaf(n, -0.693359375f, x);       /* ln2 high part, exact product */
  r = fmaf(n, 2.12194440e-4f, r);            /* minus ln2 low part */
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  p = fmaf(p, r * r, r);
  p = p + 1.0f;
  /* scale by 2^n, n in [-126, 0]: p is in [0.5, 2), so adding n to the
   * exponent field stays in the normal range except at the very bottom,
   * where the product form below is used. */
  const int ni = (int)n;
  uint32_t scale_bits = (uint32_t)(ni + 127) << 23;
  float scale;
  memcpy(&scale, &scale_bits, 4);
  return p * scale;
}

/* Routing of routed_clamped_swiglu_impl (crates/nml-ir/src/lib.rs:1411-1437):
 * softmax over all experts in f32 (:4109-4137), top-k by descending
 * probability with ties going to the lower expert index (total comparator,
 * :3534-3605 and :9884-10014), renormalise by max(sum, f32 epsilon), masked
 * tokens get expert -1 and weight 0, weights narrow to the activation dtype.
 * logits [tokens, experts] f32; active (optional) [tokens] bytes;
 * ids [tokens, k] i32; weights32 (optional) f32 before narrowing; weights16
 * (optional) narrowed to dtype (1 = f16, 2 = bf16). */
void nml_oracle_route(const float *logits, const uint8_t *active, size_t tokens, size_t experts,
                      size_t top_k, int dtype, int32_t *ids, float *weights32,
                      uint16_t *weights16) {
#pragma omp parallel
  {
    float *probability = (float *)malloc(sizeof(float) * experts);
    uint8_t *taken = (uint8_t *)malloc(experts);
#pragma omp for schedule(static)
    for (long long token = 0; token < (long long)tokens; ++token) {
      const float *row = logits + (size_t)token * experts;
      float maximum = -INFINITY;
      for (size_t e = 0; e < experts; ++e) maximum = row[e] > maximum ? row[e] : maximum;
      if (maximum > -INFINITY) {
        float denominator = 0.0f;
        for (size_t e = 0; e < experts; ++e) {
          probability[e] = nml_oracle_exp_det(row[e] - maximum);
          denominator = denominator + probability[e];
        }
        for (size_t e = 0; e < experts; ++e) probability[e] = probability[e] / denominator;
      } else {
        for (size_t e = 0; e < experts; ++e) probability[e] = 0.0f;
      }
      memset(taken, 0, experts);
      float selected[64];
      int32_t selected_id[64];
      float sum = 0.0f;
      for (size_t route = 0; route < top_k; ++route) {
        long long best = -1;
        for (size_t e = 0; e < experts; ++e) {
          if (taken[e]) continue;
          if (best < 0 || probability[e] > probability[best]) best = (long long)e;
        }
        taken[best] = 1;
        selected[route] = probability[best];
        selected_id[route] = (int32_t)best;
        sum = sum + probability[best];
      }
      const float normalizer = sum > 1.1920928955078125e-7f ? sum : 1.1920928955078125e-7f;
      const int is_active = active ? active[token] != 0 : 1;
      for (size_t route = 0; route < top_k; ++route) {
        const size_t a = (size_t)token * top_k + route;
        const float weight = is_active ? selected[route] / normalizer : 0.0f;
        ids[a] = is_active ? selected_id[route] : -1;
        if (weights32) weights32[a] = weight;
        if (weights16) weights16[a] = store16(weight, dtype);
      }
    }
    free(probability);
    free(taken);
  }
}

/* moe_assignment_plan (crates/nml-ir/src/lib.rs:5644-5779).  expert_ids holds
 * A = tokens*k entries, -1 for masked routes.  Capacity:
 *   max_blocks = ceil((A + min(A, E) * (block-1)) / block), positions =
 *   max_blocks * block.  sorted [positions] is filled with the sentinel A,
 * block_experts [max_blocks] with -1.
 * If A <= E: block b holds assignment b in its first slot and block_experts
 * is the flat id list (including -1), active_blocks = A.
 * Otherwise experts are laid out in index order, each padded to a multiple of
 * `block`, assignments in ascending order inside an expert.
 * Returns active_blocks. */
int32_t nml_oracle_assignment_plan(const int32_t *expert_ids, size_t assignments, size_t experts,
                                   size_t block, int32_t *sorted, int32_t *block_experts) {
  const size_t nonempty = assignments < experts ? assignments : experts;
  const size_t max_blocks = (assignments + nonempty * (block - 1) + block - 1) / block;
  const size_t positions = max_blocks * block;
  for (size_t i = 0; i < positions; ++i) sorted[i] = (int32_t)assignments;
  for (size_t b = 0; b < max_blocks; ++b) block_experts[b] = -1;
  if (assignments <= experts) {
    for (size_t a = 0; a < assignments; ++a) {
      sorted[a * block] = (int32_t)a;
      block_experts[a] = expert_ids[a];
    }
    return (int32_t)assignments;
  }
  size_t prefix = 0;
  for (size_t e = 0; e < experts; ++e) {
    size_t count = 0;
    for (size_t a = 0; a < assignments; ++a) {
      if (expert_ids[a] == (int32_t)e) {
        sorted[prefix + count] = (int32_t)a;
        ++count;
      }
    }
    const size_t padded = (count + block - 1) / block * block;
    for (size_t b = prefix / block; b < (prefix + padded) / block; ++b) {
      block_experts[b] = (int32_t)e;
    }
    prefix += padded;
  }
  return (int32_t)(prefix / block);
}

/* The k-way combine of the device path (crates/nml-ir/src/nvfp4_backend.rs:
 * 486-508): weighted [tokens, k, H] in the activation dtype is summed over k
 * in route order, each partial sum narrowed to the activation dtype (XLA
 * evaluates the bf16 reduce in f32 per add and narrows per step on CPU; the
 * device kernel here accumulates in f32 and narrows once, which is never less
 * accurate).  mode 0: one narrowing at the end; mode 1: narrow every add. */
void nml_oracle_combine(const uint16_t *weighted, size_t tokens, size_t top_k, size_t hidden_size,
                        int dtype, int mode, uint16_t *out) {
#pragma omp parallel for schedule(static)
  for (long long token = 0; token < (long long)tokens; ++token) {
    for (size_t h = 0; h < hidden_size; ++h) {
      float sum = 0.0f;
      for (size_t route = 0; route < top_k; ++route) {
        sum += load16(weighted, ((size_t)token * top_k + route) * hidden_size + h, dtype);
        if (mode == 1) {
          const uint16_t narrowed = store16(sum, dtype);
          sum = load16(&narrowed, 0, dtype);
        }
      }
      out[(size_t)token * hidden_size + h] = store16(sum, dtype);
    }
  }
}

int nml_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void nml_oracle_set_threads(int threads) {
#ifdef _OPENMP
  omp_set_num_threads(threads > 0 ? threads : 1);
#else
  (void)threads;
#endif
}
