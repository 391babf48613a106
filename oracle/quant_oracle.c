/* TEST INFRASTRUCTURE ONLY — CPU restatement of the quantisers on the routed-MoE path.
 * Never linked into, imported by or executed from the product path.
 *
 * Blockwise FP8 E4M3 (reference: src/cuda/fp8/quantization.cuh:35-81, tests/test_fp8.py:20-36):
 *   scale = 2^ceil(log2(amax / 448)), never below the smallest normal FP32; an all-zero block
 *   has scale 1; a block holding a non-finite value has a NaN scale; q = e4m3_rn(x / scale).
 *   Blocks are 1 x 128 (activations) or 128 x 128 (weights); `transpose` quantises x^T.
 * NVFP4 (reference: weftmoe/nvfp4.py:14-31, tests/torchrun_sm100_nvfp4.py:13-27):
 *   per 16 values sf = e4m3( min(amax / (6 s), 448) ), code = e2m1_rn_even( |v| / (sf s) ),
 *   0 when sf == 0; two codes per byte, even element in the low nibble.
 * Pinned against tests/golden/fp8_quant.pt and tests/golden/nvfp4_round.pt, which were produced
 * by the reference's own quant_reference / round_nvfp4_blocks.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float u32_as_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f32_as_u32(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* FP32 -> E4M3 (fn variant: no infinities, 0x7f = NaN, max 448), round to nearest even,
 * magnitudes beyond the largest finite code saturate to 448. */
uint8_t wm_oracle_e4m3(float f) {
  const uint8_t sign = (f32_as_u32(f) >> 31) ? 0x80 : 0x00;
  if (isnan(f)) return (uint8_t)(sign | 0x7f);
  const float a = fabsf(f);
  if (a >= 464.0f) return (uint8_t)(sign | 0x7e); /* 464 is the midpoint 448..480: ties to even = 480 -> sat */
  if (a < 0.015625f) { /* below 2^-6: subnormal grid of 2^-9 */
    const int q = (int)rintf(a * 512.0f);
    return (uint8_t)(sign | q); /* q == 8 is the smallest normal */
  }
  int e;
  const float m = frexpf(a, &e); /* a = m * 2^e, m in [0.5, 1) */
  int q = (int)rintf((m * 2.0f - 1.0f) * 8.0f);
  int exp = e - 1;
  if (q == 8) { q = 0; ++exp; }
  int code = ((exp + 7) << 3) | q;
  if (code > 0x7e) code = 0x7e;
  return (uint8_t)(sign | code);
}

float wm_oracle_e4m3_to_f32(uint8_t c) {
  const float sign = (c & 0x80) ? -1.0f : 1.0f;
  const int exp = (c >> 3) & 0xf, man = c & 7;
  if (exp == 0xf && man == 7) return NAN;
  if (exp == 0) return sign * ldexpf((float)man, -9);
  return sign * ldexpf(1.0f + man / 8.0f, exp - 7);
}

/* Power-of-two dequantisation scale of one block. */
float wm_oracle_fp8_block_scale(float amax, int nonfinite) {
  if (nonfinite || !isfinite(amax)) return NAN;
  if (amax == 0.0f) return 1.0f;
  const uint32_t bits = f32_as_u32(amax);
  /* amax / 448 = amax * 2^-9 * (512/448); 448 = 1.75 * 2^8, so ceil(log2(amax/448)) is
   * exponent - 8 when the mantissa is <= 1.75 and exponent - 7 above it. */
  int exponent = (int)(bits >> 23) - 8 + ((bits & 0x7fffffu) > 0x600000u);
  if (exponent < 1) exponent = 1;
  return u32_as_f32((uint32_t)exponent << 23);
}

/* x: [batch][rows][cols] float (already widened from BF16 if needed).
 * transpose = 0: out q [batch][rows][cols_p], scales [batch][rows_b][cols/128 ceil]
 * transpose = 1: quantises x^T: q [batch][cols][rows_p128cols], i.e. m = cols, k = rows.
 * block_rows is 1 or 128.  cols_p = k rounded up to 128 (padding bytes are zero codes). */
void wm_oracle_fp8_quantize(const float* x, int batch, int rows, int cols, int block_rows,
                            int transpose, uint8_t* q, float* scales) {
  const int m = transpose ? cols : rows, k = transpose ? rows : cols;
  const int kb = (k + 127) / 128, kp = kb * 128;
  const int mb = (m + block_rows - 1) / block_rows;
  for (int b = 0; b < batch; ++b) {
    const float* xb = x + (size_t)b * rows * cols;
    uint8_t* qb = q + (size_t)b * m * kp;
    float* sb = scales + (size_t)b * mb * kb;
    memset(qb, 0, (size_t)m * kp);
    for (int bi = 0; bi < mb; ++bi)
      for (int bj = 0; bj < kb; ++bj) {
        float amax = 0.0f;
        int bad = 0;
        for (int i = bi * block_rows; i < (bi + 1) * block_rows && i < m; ++i)
          for (int j = bj * 128; j < (bj + 1) * 128 && j < k; ++j) {
            const float v = transpose ? xb[(size_t)j * cols + i] : xb[(size_t)i * cols + j];
            if (!isfinite(v)) bad = 1;
            else if (fabsf(v) > amax) amax = fabsf(v);
          }
        const float scale = wm_oracle_fp8_block_scale(amax, bad);
        sb[bi * kb + bj] = scale;
        for (int i = bi * block_rows; i < (bi + 1) * block_rows && i < m; ++i)
          for (int j = bj * 128; j < (bj + 1) * 128 && j < k; ++j) {
            const float v = transpose ? xb[(size_t)j * cols + i] : xb[(size_t)i * cols + j];
            /* dividing by a power of two is exact; NaN scale gives NaN codes */
            qb[(size_t)i * kp + j] = wm_oracle_e4m3(v / scale);
          }
      }
  }
}

/* E2M1 code (0..7 magnitude index) of a non-negative value, round to nearest, ties to even code. */
static int e2m1_code(float a) {
  static const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  int code = 0;
  while (code < 7 && a > mid[code]) ++code; /* first midpoint >= a */
  if (code < 7 && a == mid[code] && (code & 1)) ++code; /* tie with odd lower code rounds up */
  return code;
}

/* x [rows][cols], cols % 16 == 0.  Outputs: packed [rows][cols/2] (low nibble = even element,
 * bit 3 of a nibble = sign), sf [rows][cols/16] E4M3 bytes, rounded [rows][cols] = the value the
 * tensor core sees times the block scale (without the layer scale), as round_nvfp4_blocks returns. */
void wm_oracle_nvfp4_quantize(const float* x, int rows, int cols, double layer_scale,
                              uint8_t* packed, uint8_t* sf_out, float* rounded) {
  static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  const float denom = (float)(6.0 * layer_scale);
  const float ls = (float)layer_scale;
  for (int r = 0; r < rows; ++r)
    for (int g = 0; g < cols / 16; ++g) {
      const float* v = x + (size_t)r * cols + g * 16;
      float amax = 0.0f;
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
      float s = amax / denom;
      if (s > 448.0f) s = 448.0f;
      const uint8_t sb = wm_oracle_e4m3(s);
      const float sf = wm_oracle_e4m3_to_f32(sb);
      if (sf_out) sf_out[(size_t)r * (cols / 16) + g] = sb;
      for (int i = 0; i < 16; ++i) {
        const float a = sf > 0.0f ? fabsf(v[i]) / (sf * ls) : 0.0f;
        const int code = e2m1_code(a);
        const int neg = v[i] < 0.0f;
        if (rounded) rounded[(size_t)r * cols + g * 16 + i] = mag[code] * (neg ? -1.0f : (v[i] > 0.0f ? 1.0f : 0.0f)) * sf;
        if (packed) {
          uint8_t* p = packed + (size_t)r * (cols / 2) + (g * 16 + i) / 2;
          const uint8_t nib = (uint8_t)(code | (neg ? 8 : 0));
          if (i & 1) *p = (uint8_t)((*p & 0x0f) | (nib << 4));
          else *p = (uint8_t)((*p & 0xf0) | nib);
        }
      }
    }
}
