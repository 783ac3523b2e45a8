/*
 * CPU oracle for the quantized-linear + fused-MoE path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic the reference defines for the path:
 * the GGML block formats and the router / alignment / grouped-GEMM / combine steps.
 * It is the checker the GPU parity tests compare against and the CPU arm of the
 * benchmark.  Nothing in the shipped library links, loads or calls it.
 *
 * Parity status: PARITY UNPINNED against the reference itself.  The reference holds
 * no golden vectors or known-answer tests for any function here and none of its
 * kernels can be built without the vendor toolchain, so there is nothing of the
 * reference to run or compare with.  The block-format functions are pinned instead
 * against the independent `gguf` python package (bit-exact on dequantisation) and
 * against hand-computed known-answer blocks stored with the tests.
 *
 * Reference locations each function follows (paths inside the reference project):
 *   block_q8_0                 kernels/quant.cpp:98-104
 *   block_q4_K, QK_K           kernels/quant.cpp:50-51,145-150
 *   get_scale_min_k4           kernels/quant.cpp:356-363
 *   Q4_K affine formula        kernels/quant.cpp:392-412  (format only: the vector
 *                              code there reuses the first sub-block's min for the
 *                              second sub-block, which is not followed)
 *   quantize_q8_0              kernels/quant.cpp:270-292
 *   topk_softmax               kernels/topk_softmax_host.cpp:121-172
 *   moe_align_block_size       kernels/moe_align_host.cpp:51-58,587-764,766-935
 *   invoke_fused_moe           kernels/fused_moe_host.cpp:43-250
 *   silu_and_mul               kernels/topsaten_ops_wrapper.cpp:375-391
 *   moe (weighted combine)     kernels/moe_host.cpp:26-81
 *   indexed_moe CPU loop       kernels/moe_host.cpp:325-353
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK8_0 32
#define QK_K 256
#define Q8_0_BYTES 34
#define Q4K_BYTES 144

/* ---------------------------------------------------------------- scalar type helpers */

static float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while (!(man & 0x400u));
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* round-to-nearest-even f32 -> f16 */
static uint16_t f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7FFFFFFFu;
  if (absx >= 0x7F800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0));
  }
  if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7C00u);
  }
  if (absx < 0x33000001u) { /* below half of the smallest subnormal */
    return (uint16_t)sign;
  }
  int32_t exp = (int32_t)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
  uint32_t shift;
  uint32_t hexp;
  if (exp < -14) { /* subnormal result */
    shift = (uint32_t)(13 + (-14 - exp));
    hexp = 0;
  } else {
    shift = 13;
    hexp = (uint32_t)(exp + 15);
  }
  uint32_t halfway = 1u << (shift - 1);
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t q = man >> shift;
  if (rem > halfway || (rem == halfway && (q & 1u))) q++;
  uint32_t out;
  if (hexp == 0) {
    out = q; /* may carry into the exponent field, which is correct */
  } else {
    out = ((hexp - 1u) << 10) + q; /* q carries the implicit 1 */
  }
  return (uint16_t)(sign | out);
}

static float bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static uint16_t f32_to_bf16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7FFFu + lsb;
  return (uint16_t)(x >> 16);
}

/* dtype codes follow the reference's DATATYPE enum (src/lib.rs:87-106) */
enum { UB_F16 = 4, UB_BF16 = 5, UB_F32 = 8 };

static float load_as_f32(const void* p, size_t i, int dtype) {
  if (dtype == UB_F32) return ((const float*)p)[i];
  if (dtype == UB_F16) return f16_to_f32(((const uint16_t*)p)[i]);
  return bf16_to_f32(((const uint16_t*)p)[i]);
}

static void store_from_f32(void* p, size_t i, int dtype, float v) {
  if (dtype == UB_F32)
    ((float*)p)[i] = v;
  else if (dtype == UB_F16)
    ((uint16_t*)p)[i] = f32_to_f16(v);
  else
    ((uint16_t*)p)[i] = f32_to_bf16(v);
}

/* round a float through the storage type T (what a cast to T and back does) */
static float round_through(float v, int dtype) {
  if (dtype == UB_F32) return v;
  if (dtype == UB_F16) return f16_to_f32(f32_to_f16(v));
  return bf16_to_f32(f32_to_bf16(v));
}

void ub_oracle_f32_to_f16(const float* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = f32_to_f16(in[i]);
}
void ub_oracle_f16_to_f32(const uint16_t* in, float* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = f16_to_f32(in[i]);
}
void ub_oracle_f32_to_bf16(const float* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = f32_to_bf16(in[i]);
}
void ub_oracle_bf16_to_f32(const uint16_t* in, float* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = bf16_to_f32(in[i]);
}

/* ---------------------------------------------------------------- block formats */

/* kernels/quant.cpp:356-363 */
static void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
  if (j < 4) {
    *sc = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

/* One interleaved 34-byte Q8_0 block -> 32 floats: y = d * q */
static void dequant_block_q8_0(const uint8_t* blk, float* y) {
  uint16_t dh;
  memcpy(&dh, blk, 2);
  const float d = f16_to_f32(dh);
  const int8_t* qs = (const int8_t*)(blk + 2);
  for (int i = 0; i < QK8_0; i++) y[i] = d * (float)qs[i];
}

/* One interleaved 144-byte Q4_K super-block -> 256 floats.
 * 64-value group g: low nibbles of qs[32g..32g+31] are values 64g..64g+31 with
 * (scale, min) pair 2g; high nibbles are values 64g+32..64g+63 with pair 2g+1.
 * y = (d*sc)*q - (dmin*m), each product exact in f32, one rounding in the subtract. */
static void dequant_block_q4k(const uint8_t* blk, float* y) {
  uint16_t dh, mh;
  memcpy(&dh, blk, 2);
  memcpy(&mh, blk + 2, 2);
  const float d = f16_to_f32(dh);
  const float dmin = f16_to_f32(mh);
  const uint8_t* scales = blk + 4;
  const uint8_t* qs = blk + 16;
  for (int g = 0; g < 4; g++) {
    uint8_t sc, m;
    scale_min_k4(2 * g, scales, &sc, &m);
    const float d1 = d * (float)sc, m1 = dmin * (float)m;
    scale_min_k4(2 * g + 1, scales, &sc, &m);
    const float d2 = d * (float)sc, m2 = dmin * (float)m;
    for (int l = 0; l < 32; l++) {
      y[64 * g + l] = d1 * (float)(qs[32 * g + l] & 0xF) - m1;
      y[64 * g + 32 + l] = d2 * (float)(qs[32 * g + l] >> 4) - m2;
    }
  }
}

/* One interleaved 210-byte Q6_K super-block -> 256 floats (layout declared at kernels/quant.cpp:170-177:
 * ql[128] low nibbles, qh[64] upper two bits, int8 scales[16], f16 d; the reference has no kernel for it, the
 * arithmetic is the published GGML one).  Element i = 128h + 32j + l: low nibble in ql[64h + 32(j&1) + l]
 * (upper half of the byte when j >= 2), top two bits at bit 2j of qh[32h + l]; y = (d * scales[i/16]) * (q - 32). */
#define Q6K_BYTES 210
static void dequant_block_q6k(const uint8_t* blk, float* y) {
  uint16_t dh;
  memcpy(&dh, blk + 208, 2);
  const float d = f16_to_f32(dh);
  const int8_t* sc = (const int8_t*)(blk + 192);
  for (int h = 0; h < 2; h++)
    for (int j = 0; j < 4; j++) {
      const uint8_t* ql = blk + 64 * h + 32 * (j & 1);
      const uint8_t* qh = blk + 128 + 32 * h;
      const int shift = j >= 2 ? 4 : 0;
      for (int half = 0; half < 2; half++) { /* 16 positions share one scale */
        const float ds = d * (float)sc[8 * h + 2 * j + half];
        for (int l = 16 * half; l < 16 * half + 16; l++) {
          const int q = ((ql[l] >> shift) & 0xF) | (((qh[l] >> (2 * j)) & 3) << 4);
          y[128 * h + 32 * j + l] = ds * (float)(q - 32);
        }
      }
    }
}

/* One interleaved 176-byte Q5_K super-block -> 256 floats (layout declared at kernels/quant.cpp:154-161: f16 d,
 * f16 dmin, twelve scale bytes packed as in Q4_K, qh[32], qs[128]; the reference has no kernel for it, the
 * arithmetic is the published GGML one).  64-value group g: values 0..31 = low nibbles of qs[32g..] + 16 * bit 2g
 * of qh[l] with pair 2g, values 32..63 = high nibbles + 16 * bit 2g+1 with pair 2g+1; y = (d*sc)*q - dmin*m. */
#define Q5K_BYTES 176
static void dequant_block_q5k(const uint8_t* blk, float* y) {
  uint16_t dh, mh;
  memcpy(&dh, blk, 2);
  memcpy(&mh, blk + 2, 2);
  const float d = f16_to_f32(dh);
  const float dmin = f16_to_f32(mh);
  const uint8_t* scales = blk + 4;
  const uint8_t* qh = blk + 16;
  const uint8_t* qs = blk + 48;
  for (int g = 0; g < 4; g++) {
    uint8_t sc, m;
    scale_min_k4(2 * g, scales, &sc, &m);
    const float d1 = d * (float)sc, m1 = dmin * (float)m;
    scale_min_k4(2 * g + 1, scales, &sc, &m);
    const float d2 = d * (float)sc, m2 = dmin * (float)m;
    for (int l = 0; l < 32; l++) {
      const int q1 = (qs[32 * g + l] & 0xF) + (((qh[l] >> (2 * g)) & 1) << 4);
      const int q2 = (qs[32 * g + l] >> 4) + (((qh[l] >> (2 * g + 1)) & 1) << 4);
      y[64 * g + l] = d1 * (float)q1 - m1;
      y[64 * g + 32 + l] = d2 * (float)q2 - m2;
    }
  }
}

/* One interleaved 18-byte Q4_0 block -> 32 floats (kernels/quant.cpp:64-69: f16 d and sixteen bytes; value i in
 * the low nibble of byte i, value 16 + i in its high nibble); y = d * (q - 8). */
#define Q4_0_BYTES 18
static void dequant_block_q4_0(const uint8_t* blk, float* y) {
  uint16_t dh;
  memcpy(&dh, blk, 2);
  const float d = f16_to_f32(dh);
  for (int i = 0; i < 16; i++) {
    y[i] = d * (float)((int)(blk[2 + i] & 0xF) - 8);
    y[16 + i] = d * (float)((int)(blk[2 + i] >> 4) - 8);
  }
}

/* Format codes of the functions below: 0 = Q8_0, 1 = Q4_K, 2 = Q6_K, 3 = Q5_K, 4 = Q4_0. */
static int fmt_per(int fmt) { return (fmt == 0 || fmt == 4) ? QK8_0 : QK_K; }
static int fmt_bytes(int fmt) {
  return fmt == 0 ? Q8_0_BYTES : fmt == 1 ? Q4K_BYTES : fmt == 2 ? Q6K_BYTES : fmt == 3 ? Q5K_BYTES : Q4_0_BYTES;
}
static void dequant_block(int fmt, const uint8_t* blk, float* y) {
  if (fmt == 0)
    dequant_block_q8_0(blk, y);
  else if (fmt == 1)
    dequant_block_q4k(blk, y);
  else if (fmt == 2)
    dequant_block_q6k(blk, y);
  else if (fmt == 3)
    dequant_block_q5k(blk, y);
  else
    dequant_block_q4_0(blk, y);
}

void ub_oracle_dequant_q6k(const uint8_t* blocks, float* out, size_t nblocks) {
#pragma omp parallel for schedule(static)
  for (long b = 0; b < (long)nblocks; b++) dequant_block_q6k(blocks + (size_t)b * Q6K_BYTES, out + (size_t)b * QK_K);
}

void ub_oracle_dequant_q8_0(const uint8_t* blocks, float* out, size_t nblocks) {
#pragma omp parallel for schedule(static)
  for (long b = 0; b < (long)nblocks; b++) dequant_block_q8_0(blocks + (size_t)b * Q8_0_BYTES, out + (size_t)b * QK8_0);
}

void ub_oracle_dequant_q4k(const uint8_t* blocks, float* out, size_t nblocks) {
#pragma omp parallel for schedule(static)
  for (long b = 0; b < (long)nblocks; b++) dequant_block_q4k(blocks + (size_t)b * Q4K_BYTES, out + (size_t)b * QK_K);
}

/* Dequantise then round once to the storage type (f16 / bf16 / f32). */
void ub_oracle_dequant_to(const uint8_t* blocks, void* out, size_t nblocks, int is_q4k, int dtype) {
  const int per = is_q4k ? QK_K : QK8_0;
  const int bytes = is_q4k ? Q4K_BYTES : Q8_0_BYTES;
#pragma omp parallel for schedule(static)
  for (long b = 0; b < (long)nblocks; b++) {
    float tmp[QK_K];
    if (is_q4k)
      dequant_block_q4k(blocks + (size_t)b * bytes, tmp);
    else
      dequant_block_q8_0(blocks + (size_t)b * bytes, tmp);
    for (int i = 0; i < per; i++) store_from_f32(out, (size_t)b * per + i, dtype, tmp[i]);
  }
}

/* The reference keeps device tensors de-interleaved (kernels/quant.cpp:219-220, 441-442):
 *   Q8_0: [nb x f16 d][nb x 32 int8]        Q4_K: [nb x 16-byte header][nb x 128-byte qs]
 * These two convert between the interleaved GGUF bytes and that split layout. */
void ub_oracle_split_layout(const uint8_t* inter, uint8_t* split, size_t nb, int is_q4k) {
  const size_t hb = is_q4k ? 16 : 2, qb = is_q4k ? 128 : 32;
  for (size_t b = 0; b < nb; b++) {
    memcpy(split + b * hb, inter + b * (hb + qb), hb);
    memcpy(split + nb * hb + b * qb, inter + b * (hb + qb) + hb, qb);
  }
}
void ub_oracle_interleave_layout(const uint8_t* split, uint8_t* inter, size_t nb, int is_q4k) {
  const size_t hb = is_q4k ? 16 : 2, qb = is_q4k ? 128 : 32;
  for (size_t b = 0; b < nb; b++) {
    memcpy(inter + b * (hb + qb), split + b * hb, hb);
    memcpy(inter + b * (hb + qb) + hb, split + nb * hb + b * qb, qb);
  }
}

/* kernels/quant.cpp:270-292: d = amax/127, id = 1/d (0 when d == 0), q = round(x*id),
 * stored d is f16(d).  Rounding is half-away-from-zero (roundf), as GGML does. */
void ub_oracle_quantize_q8_0(const float* x, uint8_t* blocks, size_t nblocks) {
#pragma omp parallel for schedule(static)
  for (long b = 0; b < (long)nblocks; b++) {
    const float* xb = x + (size_t)b * QK8_0;
    float amax = 0.f;
    for (int i = 0; i < QK8_0; i++) {
      float a = fabsf(xb[i]);
      if (a > amax) amax = a;
    }
    const float d = amax / 127.f;
    const float id = (d != 0.f) ? 1.f / d : 0.f;
    uint16_t dh = f32_to_f16(d);
    uint8_t* blk = blocks + (size_t)b * Q8_0_BYTES;
    memcpy(blk, &dh, 2);
    for (int i = 0; i < QK8_0; i++) ((int8_t*)(blk + 2))[i] = (int8_t)roundf(xb[i] * id);
  }
}

/* ---------------------------------------------------------------- quantized matmul */

/* y[M,N] = x[M,K] . W^T, W = N rows of interleaved blocks.  "exact" arm: weights
 * dequantised to f32 exactly as above, products and sums in double, one rounding
 * to f32 at the end.  This is the parity oracle (not a timed path). */
void ub_oracle_qmatmul_exact(const float* x, const uint8_t* wq, float* y, int M, int N, int K, int is_q4k) {
  const int per = fmt_per(is_q4k), bytes = fmt_bytes(is_q4k);  /* is_q4k is the format code (0 .. 4) */
  const int nb = K / per;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; n++) {
    float* wrow = (float*)malloc((size_t)K * sizeof(float));
    for (int b = 0; b < nb; b++) {
      const uint8_t* blk = wq + ((size_t)n * nb + b) * bytes;
      dequant_block(is_q4k, blk, wrow + (size_t)b * per);
    }
    for (int m = 0; m < M; m++) {
      const float* xr = x + (size_t)m * K;
      double acc = 0.0;
      for (int k = 0; k < K; k++) acc += (double)xr[k] * (double)wrow[k];
      y[(size_t)m * N + n] = (float)acc;
    }
    free(wrow);
  }
}

/* Timed CPU arm: the same block-wise dequant-dot with f32 accumulation, one pass over
 * the packed weights per call, OpenMP over rows.  Per block the integer part is summed
 * first and scaled once, the usual CPU formulation of a GGML-style vec-dot with a
 * floating-point activation row. */
void ub_oracle_qmatmul_f32(const float* x, const uint8_t* wq, float* y, int M, int N, int K, int is_q4k) {
  const int per = fmt_per(is_q4k), bytes = fmt_bytes(is_q4k);  /* is_q4k is the format code (0 .. 4) */
  const int nb = K / per;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; n++) {
    float wtmp[QK_K];
    for (int m0 = 0; m0 < M; m0 += 16) {
      const int mt = (M - m0) < 16 ? (M - m0) : 16;
      float acc[16];
      for (int m = 0; m < mt; m++) acc[m] = 0.f;
      for (int b = 0; b < nb; b++) {
        const uint8_t* blk = wq + ((size_t)n * nb + b) * bytes;
        dequant_block(is_q4k, blk, wtmp);
        for (int m = 0; m < mt; m++) {
          const float* xr = x + (size_t)(m0 + m) * K + (size_t)b * per;
          float s = 0.f;
          for (int i = 0; i < per; i++) s += xr[i] * wtmp[i];
          acc[m] += s;
        }
      }
      for (int m = 0; m < mt; m++) y[(size_t)(m0 + m) * N + n] = acc[m];
    }
  }
}

/* ---------------------------------------------------------------- "q8act" arm (informational)
 * GGML-family CPU back ends (candle's quantized matmul among them, the parity target the task names) do not
 * multiply f32 activations with dequantised weights: they first quantise every activation row to 8-bit blocks
 * and take integer dot products per block.  This arm restates that published algorithm so that the distance
 * between it and the exact arm above can be reported:
 *   Q8_0 weights: activations -> Q8_0 blocks of 32 (d = amax/127 kept in f16, q = round(x/d); the quantiser of
 *                 kernels/quant.cpp:280-289), block result d_w * d_x * sum(q_w * q_x);
 *   Q4_K weights: activations -> 256-wide int8 blocks with an f32 scale (GGML's Q8_K: iscale = -128/max where
 *                 max is the SIGNED value of largest magnitude, q = min(127, round(iscale * x)), d = 1/iscale),
 *                 block result d_w*d_x*sum_j sc_j*sum(q4*q8) - dmin_w*d_x*sum_j m_j*sum_j(q8).
 * No version of candle is pinned by the reference, so this arm is not a gate. */
static float round_half_away(float v) { return roundf(v); }

void ub_oracle_qmatmul_q8act_f32(const float* x, const uint8_t* wq, float* y, int M, int N, int K, int fmt) {
  if (fmt == 0) {
    const int nb = K / QK8_0;
    int8_t* xq = (int8_t*)malloc((size_t)M * K);
    float* xd = (float*)malloc((size_t)M * nb * sizeof(float));
    for (int m = 0; m < M; m++)
      for (int b = 0; b < nb; b++) {
        const float* xr = x + (size_t)m * K + (size_t)b * QK8_0;
        float amax = 0.f;
        for (int i = 0; i < QK8_0; i++) amax = fmaxf(amax, fabsf(xr[i]));
        const float d = amax / 127.f, id = d != 0.f ? 1.f / d : 0.f;
        for (int i = 0; i < QK8_0; i++) xq[(size_t)m * K + (size_t)b * QK8_0 + i] = (int8_t)round_half_away(xr[i] * id);
        xd[(size_t)m * nb + b] = f16_to_f32(f32_to_f16(d));
      }
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++)
      for (int m = 0; m < M; m++) {
        float acc = 0.f;
        for (int b = 0; b < nb; b++) {
          const uint8_t* blk = wq + ((size_t)n * nb + b) * Q8_0_BYTES;
          uint16_t dh;
          memcpy(&dh, blk, 2);
          const int8_t* qw = (const int8_t*)(blk + 2);
          const int8_t* qx = xq + (size_t)m * K + (size_t)b * QK8_0;
          int s = 0;
          for (int i = 0; i < QK8_0; i++) s += (int)qw[i] * (int)qx[i];
          acc += f16_to_f32(dh) * xd[(size_t)m * nb + b] * (float)s;
        }
        y[(size_t)m * N + n] = acc;
      }
    free(xq);
    free(xd);
    return;
  }
  /* Q4_K weights x 256-wide int8 activation blocks */
  const int nb = K / QK_K;
  int8_t* xq = (int8_t*)malloc((size_t)M * K);
  float* xd = (float*)malloc((size_t)M * nb * sizeof(float));
  int* bs = (int*)malloc((size_t)M * nb * 8 * sizeof(int)); /* sums of q over the 8 sub-blocks of 32 */
  for (int m = 0; m < M; m++)
    for (int b = 0; b < nb; b++) {
      const float* xr = x + (size_t)m * K + (size_t)b * QK_K;
      float max = 0.f, amax = 0.f;
      for (int i = 0; i < QK_K; i++) {
        const float ax = fabsf(xr[i]);
        if (ax > amax) amax = ax, max = xr[i];
      }
      int8_t* q = xq + (size_t)m * K + (size_t)b * QK_K;
      if (amax == 0.f) {
        memset(q, 0, QK_K);
        xd[(size_t)m * nb + b] = 0.f;
      } else {
        const float iscale = -128.f / max;
        for (int i = 0; i < QK_K; i++) {
          int v = (int)lrintf(iscale * xr[i]); /* nearest, ties to even, as GGML's nearest_int */
          q[i] = (int8_t)(v > 127 ? 127 : v);
        }
        xd[(size_t)m * nb + b] = 1.f / iscale;
      }
      for (int j = 0; j < 8; j++) {
        int sacc = 0;
        for (int i = 0; i < 32; i++) sacc += q[32 * j + i];
        bs[((size_t)m * nb + b) * 8 + j] = sacc;
      }
    }
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; n++)
    for (int m = 0; m < M; m++) {
      float acc = 0.f;
      for (int b = 0; b < nb; b++) {
        const uint8_t* blk = wq + ((size_t)n * nb + b) * Q4K_BYTES;
        uint16_t dh, mh;
        memcpy(&dh, blk, 2);
        memcpy(&mh, blk + 2, 2);
        const uint8_t* scales = blk + 4;
        const uint8_t* qs = blk + 16;
        const int8_t* q8 = xq + (size_t)m * K + (size_t)b * QK_K;
        const int* bsum = bs + ((size_t)m * nb + b) * 8;
        int sumi = 0, summ = 0;
        for (int g = 0; g < 4; g++) {
          uint8_t sc0, m0, sc1, m1;
          scale_min_k4(2 * g, scales, &sc0, &m0);
          scale_min_k4(2 * g + 1, scales, &sc1, &m1);
          int lo = 0, hi = 0;
          for (int i = 0; i < 32; i++) {
            lo += (int)(qs[32 * g + i] & 0xF) * (int)q8[64 * g + i];
            hi += (int)(qs[32 * g + i] >> 4) * (int)q8[64 * g + 32 + i];
          }
          sumi += (int)sc0 * lo + (int)sc1 * hi;
          summ += (int)m0 * bsum[2 * g] + (int)m1 * bsum[2 * g + 1];
        }
        const float dx = xd[(size_t)m * nb + b];
        acc += f16_to_f32(dh) * dx * (float)sumi - f16_to_f32(mh) * dx * (float)summ;
      }
      y[(size_t)m * N + n] = acc;
    }
  free(xq);
  free(xd);
  free(bs);
}

/* OpenMP thread count of the CPU arm: launchers such as torch.distributed.run export OMP_NUM_THREADS=1, so the
 * arm sets its thread count explicitly and reports what it got. */
#ifdef _OPENMP
#include <omp.h>
int ub_oracle_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}
#else
int ub_oracle_set_threads(int n) {
  (void)n;
  return 1;
}
#endif

/* ---------------------------------------------------------------- MoE router */

/* kernels/topk_softmax_host.cpp:121-172.  f32 softmax, k rounds of strict-greater arg-max
 * (ties to the lowest index), weight = prob cast to T; when norm_topk_prob the cast value
 * is read back, multiplied by 1/sum(selected probs, f32) and cast again. */
void ub_oracle_topk_softmax(const void* in, void* out_w, int32_t* out_idx, int T, int E, int k, int norm, int dtype) {
  float* prob = (float*)malloc((size_t)E * sizeof(float));
  float* wtmp = (float*)malloc((size_t)E * sizeof(float));
  float* sel = (float*)malloc((size_t)k * sizeof(float));
  for (int t = 0; t < T; t++) {
    float maxv = -INFINITY;
    for (int e = 0; e < E; e++) {
      float v = load_as_f32(in, (size_t)t * E + e, dtype);
      if (v > maxv) maxv = v;
    }
    float sum = 0.f;
    for (int e = 0; e < E; e++) sum += expf(load_as_f32(in, (size_t)t * E + e, dtype) - maxv);
    const float inv_sum = sum > 0.f ? 1.f / sum : 1.f;
    for (int e = 0; e < E; e++) {
      prob[e] = expf(load_as_f32(in, (size_t)t * E + e, dtype) - maxv) * inv_sum;
      wtmp[e] = prob[e];
    }
    float wsum = 0.f;
    int got = 0;
    for (int j = 0; j < k; j++) {
      float best = -INFINITY;
      int bi = -1;
      for (int e = 0; e < E; e++)
        if (wtmp[e] > best) {
          best = wtmp[e];
          bi = e;
        }
      if (bi < 0) break;
      sel[j] = round_through(prob[bi], dtype);
      out_idx[(size_t)t * k + j] = bi;
      wsum += prob[bi];
      wtmp[bi] = -INFINITY;
      got++;
    }
    if (norm && wsum > 0.f) {
      const float inv = 1.f / wsum;
      for (int j = 0; j < got; j++) sel[j] = sel[j] * inv;
    }
    for (int j = 0; j < got; j++) store_from_f32(out_w, (size_t)t * k + j, dtype, sel[j]);
  }
  free(prob);
  free(wtmp);
  free(sel);
}

/* ---------------------------------------------------------------- MoE alignment */

/* kernels/moe_align_host.cpp.  Stable counting sort of the T*k flat slots by expert id,
 * every non-empty expert padded up to a multiple of block_size.
 *   sorted_ids[ T*k + E*(block-1) ]   pad value = T*k (the ORIGINAL T, :775-781)
 *   experts_ids[ max_padded / block ] zero beyond the used blocks (:779-781), entry =
 *                                     expert_map[e] when a map is given (:535-543,703-707)
 *   num_tokens_post_pad[1]
 * real_token_num (nullable) limits the slots read to real*k (:786-799).
 * Returns 0, or -1 when an id is outside [0,E) / a map entry outside [-1,E) (the
 * reference traps the device there, :101-163). */
int ub_oracle_moe_align(int32_t* sorted_ids, int32_t* experts_ids, int32_t* num_post_pad, const int32_t* topk_ids,
                        const int32_t* real_token_num, const int32_t* expert_map, int E, int block, int T, int k) {
  const int pad_value = T * k;
  const int max_padded = T * k + E * (block - 1);
  const int max_blocks = max_padded / block;
  for (int i = 0; i < max_padded; i++) sorted_ids[i] = pad_value;
  for (int i = 0; i < max_blocks; i++) experts_ids[i] = 0;
  int tn = T;
  if (real_token_num) {
    tn = *real_token_num;
    if (tn < 0 || tn > T) return -1;
  }
  const int slots = tn * k;
  if (slots == 0) {
    *num_post_pad = 0;
    return 0;
  }
  int* cnt = (int*)calloc((size_t)E, sizeof(int));
  int* off = (int*)calloc((size_t)E + 1, sizeof(int));
  for (int i = 0; i < slots; i++) {
    int e = topk_ids[i];
    if (e < 0 || e >= E) {
      free(cnt);
      free(off);
      return -1;
    }
    cnt[e]++;
  }
  if (expert_map)
    for (int e = 0; e < E; e++)
      if (expert_map[e] < -1 || expert_map[e] >= E) {
        free(cnt);
        free(off);
        return -1;
      }
  int blk = 0;
  for (int e = 0; e < E; e++) {
    off[e] = blk * block;
    int nblk = (cnt[e] + block - 1) / block;
    for (int j = 0; j < nblk; j++) experts_ids[blk + j] = expert_map ? expert_map[e] : e;
    blk += nblk;
  }
  *num_post_pad = blk * block;
  for (int e = 0; e < E; e++) cnt[e] = 0;
  for (int i = 0; i < slots; i++) {
    int e = topk_ids[i];
    sorted_ids[off[e] + cnt[e]] = i;
    cnt[e]++;
  }
  free(cnt);
  free(off);
  return 0;
}

/* ---------------------------------------------------------------- grouped expert GEMM */

/* kernels/fused_moe_host.cpp:43-250 with dense f32 expert weights B[E,N,K] (the caller
 * dequantises Q4_K experts first).  For block b with expert e = experts_ids[b]:
 *   C[sorted_id, :] = A[sorted_id / topk_str, :] . B[e]^T (+ bias[e]),
 *   topk_str = top_k when mul_routed_weight == 0 (A is [T,K]) else 1 (A is [T*k,K]);
 *   when mul_routed_weight the f32 accumulator is multiplied by topk_weights[sorted_id];
 *   e == -1 zero-fills the rows; slots >= topk_ids_size are padding and skipped.
 * Accumulates in double, rounds once to `dtype`.  Rows of C not named by a slot are left
 * untouched. */
void ub_oracle_fused_moe(void* C, const void* A, const float* B, const float* bias, const float* topk_w,
                         const int32_t* sorted_ids, const int32_t* experts_ids, const int32_t* num_post_pad, int K,
                         int N, int E, int topk_ids_size, int top_k, int block, int mul_routed_weight, int bias_flag,
                         int dtype) {
  (void)E;
  const int padded = *num_post_pad;
  if (padded == 0) return;
  const int nblocks = padded / block;
  const int topk_str = mul_routed_weight ? 1 : top_k;
  for (int b = 0; b < nblocks; b++) {
    const int e = experts_ids[b];
#pragma omp parallel for schedule(static)
    for (int i = 0; i < block; i++) {
      const int sid = sorted_ids[b * block + i];
      if (sid < 0 || sid >= topk_ids_size) continue;
      if (e == -1) {
        for (int n = 0; n < N; n++) store_from_f32(C, (size_t)sid * N + n, dtype, 0.f);
        continue;
      }
      const size_t arow = (size_t)(sid / topk_str) * K;
      for (int n = 0; n < N; n++) {
        const float* wrow = B + ((size_t)e * N + n) * K;
        double acc = 0.0;
        for (int kk = 0; kk < K; kk++) acc += (double)load_as_f32(A, arow + kk, dtype) * (double)wrow[kk];
        if (bias_flag) acc += (double)bias[(size_t)e * N + n];
        if (mul_routed_weight) acc *= (double)topk_w[sid];
        store_from_f32(C, (size_t)sid * N + n, dtype, (float)acc);
      }
    }
  }
}

/* kernels/topsaten_ops_wrapper.cpp:375-391: out[t, :D] = silu(in[t, :D]) * in[t, D:2D] */
void ub_oracle_silu_and_mul(const void* in, void* out, int rows, int D, int dtype) {
  for (int t = 0; t < rows; t++)
    for (int j = 0; j < D; j++) {
      const float g = load_as_f32(in, (size_t)t * 2 * D + j, dtype);
      const float u = load_as_f32(in, (size_t)t * 2 * D + D + j, dtype);
      const float s = g / (1.f + expf(-g));
      store_from_f32(out, (size_t)t * D + j, dtype, s * u);
    }
}

/* Sum over the top-k axis: out[t,:] = sum_j in[t,j,:] (f32 sum in slot order, one cast). */
void ub_oracle_topk_sum(const void* in, void* out, int T, int topk, int H, int dtype) {
  for (int t = 0; t < T; t++)
    for (int h = 0; h < H; h++) {
      float s = 0.f;
      for (int j = 0; j < topk; j++) s += load_as_f32(in, ((size_t)t * topk + j) * H + h, dtype);
      store_from_f32(out, (size_t)t * H + h, dtype, s);
    }
}

/* kernels/moe_host.cpp:26-81: for k in [0,K): r = idx[k]; if r < N and top[k] < topk:
 *   y[r,:] = T( y[r,:] + T(e_out[k,:] * w[r*topk + top[k]]) )     (rows of length M) */
void ub_oracle_moe_combine(void* y, const void* e_out, const float* w, const uint32_t* idx, const uint32_t* top, int N,
                           int K, int M, int topk, int dtype) {
  for (int k = 0; k < K; k++) {
    const uint32_t r = idx[k];
    if (r >= (uint32_t)N) continue;
    const uint32_t tp = top[k];
    if (tp >= (uint32_t)topk) continue;
    const float wv = w[(size_t)r * topk + tp];
    for (int j = 0; j < M; j++) {
      const float prod = round_through(load_as_f32(e_out, (size_t)k * M + j, dtype) * wv, dtype);
      const float cur = load_as_f32(y, (size_t)r * M + j, dtype);
      store_from_f32(y, (size_t)r * M + j, dtype, cur + prod);
    }
  }
}

/* kernels/moe_host.cpp:325-353: out[b,t,:] = in[b, (M==1 ? 0 : t), :] . w[indices[b,t]]^T */
void ub_oracle_indexed_moe(const void* in, const float* w, void* out, const uint32_t* indices, int N, int K, int M,
                           int batch, int topk, int num_experts, int dtype) {
  (void)num_experts;
#pragma omp parallel for schedule(static)
  for (int b = 0; b < batch; b++)
    for (int t = 0; t < topk; t++) {
      const uint32_t e = indices[(size_t)b * topk + t];
      const int m = (M == 1) ? 0 : t;
      const size_t arow = ((size_t)b * M + m) * K;
      for (int n = 0; n < N; n++) {
        const float* wrow = w + ((size_t)e * N + n) * K;
        double acc = 0.0;
        for (int kk = 0; kk < K; kk++) acc += (double)load_as_f32(in, arow + kk, dtype) * (double)wrow[kk];
        store_from_f32(out, ((size_t)b * topk + t) * N + n, dtype, (float)acc);
      }
    }
}
