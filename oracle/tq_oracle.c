/*
 * CPU oracle for the TurboQuant paged-KV path.  TEST INFRASTRUCTURE ONLY: nothing under anna_b200/ may
 * link, load or call this file; only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline /
 * --impl reference legs use it, and only as the checker / the timed CPU baseline.
 *
 * What it restates (plain scalar C, one thread unless the caller splits the rows):
 *
 *  - value quantizer  : anna.model.turboquant.quantize_turboquant_values / _pack_value_data
 *                       (src/anna/model/turboquant.py:199-230, :164-175) and its inverse
 *                       dequantize_turboquant_values / _unpack_value_data (:233-252, :178-196).
 *  - key quantizer    : the arithmetic behind _quantize_turboquant_keys (turboquant.py:255-272), which the
 *                       reference delegates to the un-vendored PyPI package `turboquant` (pinned
 *                       >=0.2,<0.3 in pyproject.toml:25; classes turboquant.core.TurboQuantMSE / TurboQuantIP,
 *                       constructed with seed=42 at turboquant.py:80,:90).  That package is absent, so this
 *                       file restates the published TurboQuant algorithm (normalise -> random rotation ->
 *                       per-coordinate Lloyd-Max index -> 1-bit QJL sign of the residual + residual norm) with
 *                       a structured rotation (random-sign Walsh-Hadamard) and fixes every rounding step so
 *                       that a GPU implementation can match it bit for bit.  Parity of the key codes against
 *                       the real package is UNPINNED (the reference holds no golden vectors for them); the
 *                       estimator structure follows turboquant_key_attention_scores (turboquant.py:316-332).
 *  - decode attention : TurboQuantKVRow.decode_attention, CPU branch (turboquant.py:1275-1293) and
 *                       grouped_query_attention (src/anna/model/ops.py:1552-1574), in fp32.
 *
 * Key quantizer, exact definition (all arithmetic IEEE binary32, round-to-nearest, no fused multiply-add):
 *   tree(v)  : pairwise sum, adjacent pairs first: strides 1, 2, 4, ..., D/2.
 *   fwht(v)  : in-place butterflies for stride h = 1, 2, ..., D/2: (lo, hi) -> (lo + hi, lo - hi).
 *   norm     = sqrtf(tree(x_i * x_i));      inv = 1.0f / fmaxf(norm, 1e-20f)
 *   w        = fwht(s1 * x) * inv           (s1_i = +-1; w_i is ~N(0,1) for a generic x)
 *   idx_i    = #{k : w_i > boundary_k}      (boundaries = float32 midpoints of the sorted centroids)
 *   e_i      = w_i - centroid[idx_i]
 *   rnorm    = sqrtf(tree(e_i * e_i)) * (float)(1/sqrt(D))
 *   sign_i   = (fwht(s2 * e)_i >= 0) ? 1 : 0
 * De-quantisation (original basis):
 *   k_hat = norm * (1/D) * s1 * fwht( centroid[idx] + sqrt(pi/2)/sqrt(D) * rnorm * s2 * fwht(2*sign - 1) )
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TQO_MAX_DIM 1024
#define TQO_PI 3.14159265358979323846

/* ------------------------------------------------------------------------------------------------ */
/* small helpers                                                                                    */

static float f32_from_bits(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

uint16_t tqo_f32_to_bf16(float f) {
  uint32_t b = f32_bits(f);
  if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x0040u); /* quiet NaN */
  uint32_t lsb = (b >> 16) & 1u;
  b += 0x7fffu + lsb;
  return (uint16_t)(b >> 16);
}
float tqo_bf16_to_f32(uint16_t h) { return f32_from_bits(((uint32_t)h) << 16); }

uint16_t tqo_f32_to_f16(float f) {
  uint32_t x = f32_bits(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t mant = x & 0x007fffffu;
  int32_t exp = (int32_t)((x >> 23) & 0xffu);
  if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (mant ? 0x0200u : 0u));
  exp = exp - 127 + 15;
  if (exp >= 0x1f) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    mant |= 0x00800000u;
    uint32_t shift = (uint32_t)(14 - exp);
    uint32_t half = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1u);
    uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1u))) half++;
    return (uint16_t)(sign | half);
  }
  uint32_t half = (uint32_t)(exp << 10) | (mant >> 13);
  uint32_t rem = mant & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
  return (uint16_t)(sign | half);
}
float tqo_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t mant = h & 0x3ffu;
  if (exp == 0) {
    if (mant == 0) return f32_from_bits(sign);
    float m = (float)mant * (1.0f / 16777216.0f); /* mant * 2^-24 */
    return sign ? -m : m;
  }
  if (exp == 0x1f) return f32_from_bits(sign | 0x7f800000u | (mant << 13));
  return f32_from_bits(sign | ((exp + 112u) << 23) | (mant << 13));
}

/* dtype codes shared with the C ABI: 0 = float32, 1 = float16, 2 = bfloat16 */
static float round_to_dtype(float v, int dtype) {
  if (dtype == 1) return tqo_f16_to_f32(tqo_f32_to_f16(v));
  if (dtype == 2) return tqo_bf16_to_f32(tqo_f32_to_bf16(v));
  return v;
}

/* +-1 sign vector from a splitmix64 stream keyed by (seed, stream, dim). */
void tqo_signs(int dim, uint64_t seed, int stream, float* out) {
  uint64_t x = seed ^ (0xD1B54A32D192ED03ull * (uint64_t)(stream + 1)) ^ ((uint64_t)dim * 0x9E3779B97F4A7C15ull);
  for (int i = 0; i < dim; ++i) {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    out[i] = (z >> 63) ? -1.0f : 1.0f;
  }
}

void tqo_fwht(float* v, int dim) {
  for (int h = 1; h < dim; h <<= 1) {
    for (int base = 0; base < dim; base += 2 * h) {
      for (int j = base; j < base + h; ++j) {
        volatile float lo = v[j];
        volatile float hi = v[j + h];
        v[j] = lo + hi;
        v[j + h] = lo - hi;
      }
    }
  }
}

static float tree_sum(float* scratch, int dim) {
  for (int h = 1; h < dim; h <<= 1) {
    for (int j = 0; j < dim; j += 2 * h) {
      volatile float s = scratch[j] + scratch[j + h];
      scratch[j] = s;
    }
  }
  return scratch[0];
}

/* ------------------------------------------------------------------------------------------------ */
/* key quantizer                                                                                    */

/*
 * x        : [n, dim] float32 (bf16 / fp16 inputs are widened exactly by the caller)
 * idx      : [n, dim] uint8   Lloyd-Max index of each rotated coordinate (0 .. 2^index_bits - 1)
 * sign     : [n, dim] uint8   QJL sign bit, 1 when the projected residual is >= 0 (may be NULL: MSE-only)
 * norms    : [n] float32      ||x||
 * rnorms   : [n] float32      norm of the quantisation residual of x / ||x||   (may be NULL: MSE-only)
 */
int tqo_quantize_keys(const float* x, int64_t n, int dim, int index_bits, const float* s1, const float* s2,
                      const float* centroids, const float* boundaries, uint8_t* idx, uint8_t* sign,
                      float* norms, float* rnorms) {
  if (dim <= 0 || dim > TQO_MAX_DIM || (dim & (dim - 1)) != 0) return 1;
  if (index_bits < 1 || index_bits > 4) return 2;
  const int nb = (1 << index_bits) - 1;
  const float rsqrt_dim = (float)(1.0 / sqrt((double)dim));
  float w[TQO_MAX_DIM], e[TQO_MAX_DIM], t[TQO_MAX_DIM];
  for (int64_t r = 0; r < n; ++r) {
    const float* row = x + r * dim;
    for (int i = 0; i < dim; ++i) { volatile float p = row[i] * row[i]; t[i] = p; }
    const float norm = sqrtf(tree_sum(t, dim));
    const float inv = 1.0f / fmaxf(norm, 1e-20f);
    for (int i = 0; i < dim; ++i) w[i] = s1[i] < 0.0f ? -row[i] : row[i];
    tqo_fwht(w, dim);
    for (int i = 0; i < dim; ++i) {
      volatile float scaled = w[i] * inv;
      w[i] = scaled;
      int code = 0;
      for (int k = 0; k < nb; ++k) code += (scaled > boundaries[k]) ? 1 : 0;
      idx[r * dim + i] = (uint8_t)code;
      volatile float err = scaled - centroids[code];
      e[i] = err;
    }
    norms[r] = norm;
    if (sign != NULL && rnorms != NULL) {
      for (int i = 0; i < dim; ++i) { volatile float p = e[i] * e[i]; t[i] = p; }
      volatile float rn = sqrtf(tree_sum(t, dim)) * rsqrt_dim;
      rnorms[r] = rn;
      for (int i = 0; i < dim; ++i) t[i] = s2[i] < 0.0f ? -e[i] : e[i];
      tqo_fwht(t, dim);
      for (int i = 0; i < dim; ++i) sign[r * dim + i] = (t[i] >= 0.0f) ? 1 : 0;
    }
  }
  return 0;
}

/* De-quantise to the original basis (float32).  sign / rnorms may be NULL (MSE-only reconstruction). */
int tqo_dequantize_keys(const uint8_t* idx, const uint8_t* sign, const float* norms, const float* rnorms,
                        int64_t n, int dim, const float* s1, const float* s2, const float* centroids,
                        float* out) {
  if (dim <= 0 || dim > TQO_MAX_DIM || (dim & (dim - 1)) != 0) return 1;
  const float kappa = (float)(sqrt(TQO_PI / 2.0) / sqrt((double)dim));
  const float inv_dim = 1.0f / (float)dim;
  float a[TQO_MAX_DIM], c[TQO_MAX_DIM];
  for (int64_t r = 0; r < n; ++r) {
    for (int i = 0; i < dim; ++i) a[i] = centroids[idx[r * dim + i]];
    if (sign != NULL && rnorms != NULL) {
      for (int i = 0; i < dim; ++i) c[i] = sign[r * dim + i] ? 1.0f : -1.0f;
      tqo_fwht(c, dim);
      const float coef = kappa * rnorms[r];
      for (int i = 0; i < dim; ++i) a[i] += coef * (s2[i] < 0.0f ? -c[i] : c[i]);
    }
    tqo_fwht(a, dim);
    const float scale = norms[r] * inv_dim;
    for (int i = 0; i < dim; ++i) out[r * dim + i] = scale * (s1[i] < 0.0f ? -a[i] : a[i]);
  }
  return 0;
}

/* Rotate queries into the code basis: q1 = fwht(s1*q), q2 = fwht(s2*q1)  (both un-normalised). */
int tqo_rotate_queries(const float* q, int64_t n, int dim, const float* s1, const float* s2, float* q1,
                       float* q2) {
  if (dim <= 0 || dim > TQO_MAX_DIM || (dim & (dim - 1)) != 0) return 1;
  for (int64_t r = 0; r < n; ++r) {
    float* a = q1 + r * dim;
    float* b = q2 + r * dim;
    for (int i = 0; i < dim; ++i) a[i] = s1[i] < 0.0f ? -q[r * dim + i] : q[r * dim + i];
    tqo_fwht(a, dim);
    for (int i = 0; i < dim; ++i) b[i] = s2[i] < 0.0f ? -a[i] : a[i];
    tqo_fwht(b, dim);
  }
  return 0;
}

/* ------------------------------------------------------------------------------------------------ */
/* value quantizer (turboquant.py:199-230)                                                          */

/*
 * x      : [n, dim] float32 holding values that are exactly representable in `dtype`
 * data   : [n, dim / per_byte] uint8, per_byte = 4 for bits == 2 else 2 (3-bit codes use 4-bit storage)
 * scales : [n, dim / group] float32 holding the dtype-rounded scale; zeros likewise
 */
int tqo_quantize_values(const float* x, int64_t n, int dim, int group, int bits, int dtype, uint8_t* data,
                        float* scales, float* zeros) {
  if (bits < 2 || bits > 4) return 1;
  if (group <= 0 || dim % group != 0) return 2;
  const int storage = (bits == 2) ? 2 : 4;
  const int per_byte = 8 / storage;
  if (dim % per_byte != 0) return 3;
  const float levels = (float)((1 << bits) - 1);
  const int groups = dim / group;
  for (int64_t r = 0; r < n; ++r) {
    const float* row = x + r * dim;
    uint8_t* out = data + r * (dim / per_byte);
    memset(out, 0, (size_t)(dim / per_byte));
    for (int g = 0; g < groups; ++g) {
      float lo = row[g * group], hi = row[g * group];
      for (int j = 1; j < group; ++j) {
        const float v = row[g * group + j];
        lo = v < lo ? v : lo;
        hi = v > hi ? v : hi;
      }
      volatile float span = hi - lo;
      volatile float raw = span / levels;
      float sc = raw < 1e-8f ? 1e-8f : raw;
      sc = round_to_dtype(sc, dtype);
      const float zp = round_to_dtype(lo, dtype);
      scales[r * groups + g] = sc;
      zeros[r * groups + g] = zp;
      for (int j = 0; j < group; ++j) {
        const int d = g * group + j;
        volatile float shifted = row[d] - zp;
        volatile float ratio = shifted / sc;
        float q = rintf(ratio);
        if (!(q >= 0.0f)) q = 0.0f; /* also maps NaN (0/0 when an fp16 scale underflows to 0) to 0 */
        if (q > levels) q = levels;
        const unsigned code = (unsigned)q;
        out[d / per_byte] |= (uint8_t)(code << (storage * (d % per_byte)));
      }
    }
  }
  return 0;
}

int tqo_dequantize_values(const uint8_t* data, const float* scales, const float* zeros, int64_t n, int dim,
                          int group, int bits, float* out) {
  if (bits < 2 || bits > 4) return 1;
  const int storage = (bits == 2) ? 2 : 4;
  const int per_byte = 8 / storage;
  const unsigned mask = (1u << storage) - 1u;
  const int groups = dim / group;
  for (int64_t r = 0; r < n; ++r) {
    for (int d = 0; d < dim; ++d) {
      const unsigned code = (data[r * (dim / per_byte) + d / per_byte] >> (storage * (d % per_byte))) & mask;
      volatile float prod = (float)code * scales[r * groups + d / group];
      out[r * dim + d] = prod + zeros[r * groups + d / group];
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------------------------------ */
/* single-token GQA decode over dense K/V (fp32), one (batch row) at a time                          */

/*
 * q      : [hq, dim]            k, v : [hkv, len, dim]        gate : [hq, dim] or NULL
 * out    : [hq, dim]            softmax in fp32, scores = (q . k) * scaling, out *= sigmoid(gate)
 * A row with len == 0 yields zeros (ops.py:1046-1047, .sycl:4461).
 */
int tqo_gqa_decode(const float* q, const float* k, const float* v, const float* gate, int hq, int hkv,
                   int64_t len, int dim, float scaling, float* out) {
  if (hkv <= 0 || hq % hkv != 0) return 1;
  const int groups = hq / hkv;
  float* scores = (float*)malloc(sizeof(float) * (size_t)(len > 0 ? len : 1));
  if (!scores) return 2;
  for (int h = 0; h < hq; ++h) {
    const int kh = h / groups;
    float* o = out + (int64_t)h * dim;
    for (int d = 0; d < dim; ++d) o[d] = 0.0f;
    if (len <= 0) continue;
    float best = -INFINITY;
    for (int64_t t = 0; t < len; ++t) {
      const float* kr = k + ((int64_t)kh * len + t) * dim;
      float acc = 0.0f;
      for (int d = 0; d < dim; ++d) acc += q[(int64_t)h * dim + d] * kr[d];
      scores[t] = acc * scaling;
      if (scores[t] > best) best = scores[t];
    }
    double denom = 0.0;
    for (int64_t t = 0; t < len; ++t) { scores[t] = expf(scores[t] - best); denom += scores[t]; }
    for (int64_t t = 0; t < len; ++t) {
      const float p = (float)(scores[t] / denom);
      const float* vr = v + ((int64_t)kh * len + t) * dim;
      for (int d = 0; d < dim; ++d) o[d] += p * vr[d];
    }
    if (gate) {
      for (int d = 0; d < dim; ++d) o[d] *= 1.0f / (1.0f + expf(-gate[(int64_t)h * dim + d]));
    }
  }
  free(scores);
  return 0;
}

int tqo_version(void) { return 1; }
