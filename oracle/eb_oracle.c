/*
 * eb_oracle.c — CPU restatement of Forward's EmbeddingBag plugin kernels.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product (the CUDA library, the
 * plugin, the host session) links, loads or calls this file; it exists so the
 * tests, the smoke check and the bench's CPU-baseline leg have an independent
 * answer to compare the GPU path with.
 *
 * What it follows (paths inside the Tencent/Forward tree):
 *   source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/embedding_bag_plugin.cu
 *     :66-118   EmbeddingBagCuda                (1-D indices + offsets)
 *     :120-168  EmbeddingBagCudaWithFixedOffset (2-D [batch, L] indices)
 *     :170-181  GatherKernel
 *     :39-64    atomicOp / atomicMax            (the op switch)
 *   .../embedding_bag_plugin.h:39  enum ReduceOperation {SUM=0, MEAN=1, MAX=2, SQUARE_SUM=3, GATHER=999}
 *
 * Two semantics are offered because the reference kernel's op switch and the
 * reference enum disagree (the kernel treats 1 as max and 2 as a plain add,
 * while the enum — and torch's mode integer that the parser copies into it —
 * says 1 = mean, 2 = max):
 *   ORACLE_SEM_ENUM (0)    what the plugin is specified to compute: enum
 *                          meanings, max starts from the first element, mean
 *                          divides by the non-padding count, gather subtracts
 *                          the window origin.  This is the parity target and
 *                          equals torch CPU EmbeddingBag.
 *   ORACLE_SEM_KERNEL (1)  the literal behaviour of the reference .cu, kept so
 *                          a test can show where the two differ: op 1 =
 *                          max(0, max_i x) / max(len,1), op 2 = sum, mean
 *                          denominators count skipped indices, gather does not
 *                          subtract data_offset and leaves skipped rows as
 *                          they were.
 *
 * Pins: checked against the reference's only loadable fixture for this path
 * (data/torch_unit_tests/nodes/embedding_bag.pth with the inputs of
 * source/unit_test/test_torch_nodes.h:178-185) and against torch CPU
 * EmbeddingBag outputs committed under tests/golden/.  For mean, max, fp16,
 * padding and per-sample weights the reference has no test of its own; those
 * are pinned by torch CPU only.
 *
 * Arithmetic: fp32 accumulation in bag order (the reference's shared-memory
 * atomics have no defined order; bag order is the deterministic choice and is
 * what torch CPU produces), fp16 read exactly, results rounded once to the
 * output type (fp16 mean: torch's round / divide / round unless the
 * single-rounding flag is set), weighted sum with fused multiply-add.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_SEM_ENUM 0
#define ORACLE_SEM_KERNEL 1

#define MODE_SUM 0
#define MODE_MEAN 1
#define MODE_MAX 2
#define MODE_SQUARE_SUM 3
#define MODE_GATHER 999

#define FLAG_MEAN_RAW_LENGTH 1u
#define FLAG_GATHER_KEEP_SKIPPED 2u
#define FLAG_MEAN_SINGLE_ROUNDING 4u

/* ---- IEEE binary16 <-> binary32, round to nearest even ------------------- */

static float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
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

static uint16_t float_to_half(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t abs = x & 0x7FFFFFFFu;
  if (abs >= 0x7F800000u) { /* inf / nan */
    if (abs > 0x7F800000u) return (uint16_t)(sign | 0x7FFFu);
    return (uint16_t)(sign | 0x7C00u);
  }
  if (abs >= 0x477FF000u) { /* >= 65520 rounds to inf */
    return (uint16_t)(sign | 0x7C00u);
  }
  if (abs < 0x33000001u) { /* <= 2^-25 rounds to zero */
    return (uint16_t)sign;
  }
  int32_t e = (int32_t)(abs >> 23) - 127;
  uint32_t m = (abs & 0x7FFFFFu) | 0x800000u;
  uint32_t shift, half_e;
  if (e < -14) { /* subnormal result */
    shift = (uint32_t)(13 + (-14 - e));
    half_e = 0;
  } else {
    shift = 13;
    half_e = (uint32_t)(e + 15);
  }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
  uint32_t out;
  if (half_e == 0) {
    out = q; /* may carry into exponent 1: correct by construction */
  } else {
    out = ((half_e - 1) << 10) + q; /* q has the implicit bit at 0x400 */
  }
  return (uint16_t)(sign | out);
}

/* exported for the Python side's own checks */
float oracle_half_to_float(uint16_t h) { return half_to_float(h); }
uint16_t oracle_float_to_half(float f) { return float_to_half(f); }

/* ---- counter-based table generator (host twin of fwd_eb_fill_table) ------ */

static uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

/* Sum of eight 16-bit uniforms, centred: an Irwin-Hall bell with unit
 * variance after the constant scale.  Integer until the final multiply, so
 * host and device agree bit for bit. */
float oracle_table_value(uint64_t seed, int64_t row, int32_t col, float scale) {
  uint64_t a = mix64(seed ^ mix64((uint64_t)row * 0xD1342543DE82EF95ull + (uint64_t)(uint32_t)col));
  uint64_t b = mix64(a);
  int32_t s = 0;
  for (int i = 0; i < 4; ++i) {
    s += (int32_t)((a >> (16 * i)) & 0xFFFFu);
    s += (int32_t)((b >> (16 * i)) & 0xFFFFu);
  }
  s -= 4 * 65535; /* centre: mean of eight U{0..65535} */
  /* variance of one term = (65536^2 - 1)/12; eight terms */
  const float inv_sigma = 1.0f / 53509.92f;
  float unit = (float)s * inv_sigma;
  return unit * scale;
}

void oracle_fill_rows(void* table, int32_t table_dtype, const int64_t* rows, int64_t n_rows,
                      int32_t dim, uint64_t seed, float scale) {
  for (int64_t r = 0; r < n_rows; ++r) {
    for (int32_t c = 0; c < dim; ++c) {
      float v = oracle_table_value(seed, rows[r], c, scale);
      if (table_dtype == 1) {
        ((uint16_t*)table)[r * dim + c] = float_to_half(v);
      } else {
        ((float*)table)[r * dim + c] = v;
      }
    }
  }
}

/* ---- pooling ----------------------------------------------------------- */

static int64_t load_idx(const void* p, int32_t dtype, int64_t i) {
  return dtype == 1 ? ((const int64_t*)p)[i] : (int64_t)((const int32_t*)p)[i];
}

static float load_elem(const void* table, int32_t dtype, int64_t pos) {
  return dtype == 1 ? half_to_float(((const uint16_t*)table)[pos]) : ((const float*)table)[pos];
}

static void store_elem(void* out, int32_t dtype, int64_t pos, float v) {
  if (dtype == 1) {
    ((uint16_t*)out)[pos] = float_to_half(v);
  } else {
    ((float*)out)[pos] = v;
  }
}

/*
 * Returns 0, or -1 on bad arguments.  `acc` scratch is allocated per call.
 * Argument meanings match fwd_eb_params field for field.
 */
int oracle_eb_forward(const void* table, int32_t table_dtype, int32_t dim, int64_t num_rows,
                      int64_t row_lo, int64_t table_stride, const void* indices,
                      const void* offsets, int32_t index_dtype, int32_t fixed_len,
                      int64_t num_indices, int64_t num_bags, const float* psw, int32_t mode,
                      int32_t include_last_offset, int64_t padding_idx, void* out,
                      int32_t out_dtype, int64_t out_stride, uint32_t flags, int32_t semantics) {
  if (dim <= 0 || num_bags < 0 || num_indices < 0) return -1;
  if (table_stride == 0) table_stride = dim;
  if (out_stride == 0) out_stride = dim;

  if (mode == MODE_GATHER) {
    /* embedding_bag_plugin.cu:170-181 */
    for (int64_t t = 0; t < num_indices; ++t) {
      int64_t idx = load_idx(indices, index_dtype, t);
      int in_window = idx >= row_lo && idx < row_lo + num_rows;
      if (in_window) {
        /* the literal kernel addresses data[input_id * dim] without removing
         * data_offset (.cu:178); only defined here when that stays in range */
        int64_t row = (semantics == ORACLE_SEM_KERNEL) ? idx : idx - row_lo;
        if (row < 0 || row >= num_rows) return -1;
        for (int32_t c = 0; c < dim; ++c) {
          store_elem(out, out_dtype, t * out_stride + c,
                     load_elem(table, table_dtype, row * table_stride + c));
        }
      } else if (semantics != ORACLE_SEM_KERNEL && !(flags & FLAG_GATHER_KEEP_SKIPPED)) {
        for (int32_t c = 0; c < dim; ++c) store_elem(out, out_dtype, t * out_stride + c, 0.0f);
      }
    }
    return 0;
  }

  if (psw && mode != MODE_SUM) return -1;
  float* acc = (float*)malloc(sizeof(float) * (size_t)dim);
  if (!acc) return -1;

  for (int64_t b = 0; b < num_bags; ++b) {
    int64_t start, end;
    if (fixed_len > 0) { /* .cu:135-136 */
      start = b * (int64_t)fixed_len;
      end = start + fixed_len;
    } else { /* .cu:80-86 */
      start = load_idx(offsets, index_dtype, b);
      if (include_last_offset || b + 1 < num_bags) {
        end = load_idx(offsets, index_dtype, b + 1);
      } else {
        end = num_indices;
      }
    }
    if (start < 0 || end > num_indices || end < start) {
      free(acc);
      return -1;
    }

    for (int32_t c = 0; c < dim; ++c) acc[c] = 0.0f; /* .cu:71-75 */
    int64_t n_counted = 0; /* non-padding indices, in or out of the window */
    int have = 0;          /* a row has been taken (max mode) */

    for (int64_t i = start; i < end; ++i) {
      int64_t idx = load_idx(indices, index_dtype, i);
      if (semantics != ORACLE_SEM_KERNEL && padding_idx >= 0 && idx == padding_idx) continue;
      ++n_counted;
      if (!(idx >= row_lo && idx < row_lo + num_rows)) continue; /* .cu:94 */
      int64_t base = (idx - row_lo) * table_stride;              /* .cu:95 */
      if (semantics == ORACLE_SEM_KERNEL) {
        /* literal op switch, .cu:50-64 */
        for (int32_t c = 0; c < dim; ++c) {
          float x = load_elem(table, table_dtype, base + c);
          if (mode == 1) {
            acc[c] = fmaxf(acc[c], x);
          } else if (mode == 3) {
            acc[c] += x * x;
          } else {
            acc[c] += x;
          }
        }
        continue;
      }
      switch (mode) {
        case MODE_SUM:
          if (psw) {
            float w = psw[i];
            for (int32_t c = 0; c < dim; ++c) {
              acc[c] = fmaf(w, load_elem(table, table_dtype, base + c), acc[c]);
            }
            break;
          }
          /* fall through */
        case MODE_MEAN:
          for (int32_t c = 0; c < dim; ++c) acc[c] += load_elem(table, table_dtype, base + c);
          break;
        case MODE_SQUARE_SUM:
          for (int32_t c = 0; c < dim; ++c) {
            float x = load_elem(table, table_dtype, base + c);
            float sq = x * x;
            acc[c] += sq;
          }
          break;
        case MODE_MAX:
          for (int32_t c = 0; c < dim; ++c) {
            float x = load_elem(table, table_dtype, base + c);
            if (!have || x > acc[c]) acc[c] = x; /* strict: first of equals wins */
          }
          have = 1;
          break;
        default:
          free(acc);
          return -1;
      }
    }

    if (semantics == ORACLE_SEM_KERNEL) {
      /* .cu:109-117: op 1 divides by the raw bag length */
      float denom = (float)((end - start) > 1 ? (end - start) : 1);
      for (int32_t c = 0; c < dim; ++c) {
        store_elem(out, out_dtype, b * out_stride + c, mode == 1 ? acc[c] / denom : acc[c]);
      }
      continue;
    }

    if (mode == MODE_MEAN) {
      int64_t d = (flags & FLAG_MEAN_RAW_LENGTH) ? (end - start) : n_counted;
      if (d < 1) d = 1;
      float denom = (float)d;
      for (int32_t c = 0; c < dim; ++c) {
        float v;
        if (out_dtype == 1 && table_dtype == 1 && !(flags & FLAG_MEAN_SINGLE_ROUNDING)) {
          v = half_to_float(float_to_half(acc[c])) / denom; /* torch CPU Half path */
        } else {
          v = acc[c] / denom;
        }
        store_elem(out, out_dtype, b * out_stride + c, v);
      }
    } else {
      for (int32_t c = 0; c < dim; ++c) store_elem(out, out_dtype, b * out_stride + c, acc[c]);
    }
  }
  free(acc);
  return 0;
}

/* Sum of partials in slot order, fp32 math: twin of fwd_eb_combine_partials. */
void oracle_combine_partials(const void* parts, int32_t part_dtype, int32_t num_parts,
                             int64_t part_stride, int64_t count, void* out, int32_t out_dtype) {
  for (int64_t i = 0; i < count; ++i) {
    float s = 0.0f;
    for (int32_t r = 0; r < num_parts; ++r) s += load_elem(parts, part_dtype, r * part_stride + i);
    store_elem(out, out_dtype, i, s);
  }
}
