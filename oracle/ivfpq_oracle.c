/*
 * CPU oracle for IVF-PQ search.  TEST INFRASTRUCTURE ONLY: nothing in the shipped library links,
 * loads or calls this file.  It is used by the parity tests, by the smoke check and by the timed CPU
 * baseline of the benchmark.
 *
 * It restates, in plain C, the arithmetic of the reference search path
 * (cuvs::neighbors::ivf_pq::search) so that a GPU result can be compared number by number:
 *
 *   - query cast / padding ............ cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:103-125,
 *                                       cpp/src/neighbors/detail/ann_utils.cuh:133-199 (mapping<float>)
 *   - coarse scores + probe selection .. cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:127-167
 *   - query rotation ................... cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:996-1025
 *   - per-probe sample offsets ......... cpp/src/neighbors/ivf_common.cu:21-50
 *   - base diff ........................ detail/jit_lto_kernels/precompute_base_diff_impl.cuh:14-39
 *   - look-up table .................... detail/jit_lto_kernels/create_lut_impl.cuh:17-79
 *   - custom 8-bit float ............... cpp/src/neighbors/ivf_pq/ivf_pq_fp_8bit.cuh:31-100
 *   - code unpack + score .............. detail/jit_lto_kernels/compute_score_impl.cuh:20-79,
 *                                       cpp/src/neighbors/ivf_pq/ivf_pq_codepacking.cuh:30-117
 *   - cosine increment ................. detail/jit_lto_kernels/increment_score_impl.cuh
 *   - final selection, id translation .. cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:646-674,
 *                                       cpp/src/neighbors/ivf_common.cuh:94-252
 *
 * PINNED against the reference's own code: the 8-bit float and the bit-field code layout (host build
 * of two reference headers, oracle/ref_pin.cpp); base differences, look-up tables in their three
 * storage types, code unpack + per-vector scores in both internal distance types, the cosine
 * increment, the value mappings, distance post-processing and the sample-index -> source-id
 * translation (device build of the reference's headers by nvcc, oracle/ref_pin_dev.cu, run on a B200;
 * its outputs are the golden vectors tests/golden/ref_dev.npz, and the GPU tests compare the three
 * implementations live).  NOT PINNED, because the reference has no code of its own to pin against:
 * the summation order of the two library GEMMs (coarse scores, query rotation: binary-only cuBLAS in
 * the reference; here sequential fused multiply-adds over the inner dimension, which is also what the
 * GPU rescoring pass computes), the order of equal scores in select_k (un-vendored RAFT; the
 * reference calls it with sorted=false, so the order is unspecified; fixed here to (score, sample
 * index) ascending), and the .npy framing of index files (un-vendored RAFT serializer; checked against
 * numpy instead).  The reference's inner-product table has a second variant, taken when shared
 * memory is short (base differences not precomputed), in which nvcc contracts q * c into the
 * subtraction: its tables differ from the precomputed variant in the last bit of some entries.  This
 * file, and the engine, follow the precomputed variant (the reference's first choice).
 * The reference's pruning (per-query k-th bound, L2 early exit) is dropped: it only discards
 * candidates that cannot reach the top-k.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#if defined(__x86_64__) && defined(__GNUC__) && !defined(ORC_NO_CLONES)
#define ORC_HOT __attribute__((target_clones("default", "arch=x86-64-v3")))
#else
#define ORC_HOT
#endif

#define ORC_EXPORT __attribute__((visibility("default")))

/* ---- metric codes (c/include/cuvs/distance/distance.h) ------------------------------------ */
enum { M_L2 = 0, M_L2SQRT = 1, M_COSINE = 2, M_IP = 6 };
/* ---- lut / internal dtypes, values of cudaDataType_t ---------------------------------------- */
enum { DT_F16 = 2, DT_F32 = 0, DT_U8 = 8 };
/* ---- query element types --------------------------------------------------------------------- */
enum { Q_F32 = 0, Q_F16 = 1, Q_I8 = 2, Q_U8 = 3 };

typedef struct {
  int32_t metric;
  int32_t codebook_kind; /* 0 = per subspace, 1 = per cluster */
  uint32_t n_lists, dim, dim_ext, rot_dim, pq_dim, pq_len, pq_bits;
  uint32_t _pad;
  const float* pq_centers;     /* [pq_dim or n_lists, pq_len, 1<<pq_bits] */
  const float* centers;        /* [n_lists, dim_ext] */
  const float* centers_rot;    /* [n_lists, rot_dim] */
  const float* rotation;       /* [rot_dim, dim] */
  const uint32_t* list_sizes;  /* [n_lists] */
  const uint64_t* code_offsets; /* [n_lists] byte offset of each list in `codes` */
  const uint8_t* codes;        /* interleaved list data, lists back to back */
  const uint64_t* id_offsets;  /* [n_lists] element offset of each list in `ids` */
  const int64_t* ids;
} orc_index;

/* ============================ half precision helpers ========================================== */

static inline uint32_t f2u(float f)
{
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static inline float u2f(uint32_t u)
{
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* fp32 -> fp16 bits, round to nearest even (what `half(float)` does on the GPU). */
static inline uint16_t f32_to_f16(float f)
{
  uint32_t x    = f2u(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t ax   = x & 0x7fffffffu;
  if (ax >= 0x7f800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u : 0));
  }
  if (ax >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (ax < 0x38800000u) { /* subnormal half or zero */
    if (ax < 0x33000000u) { return (uint16_t)sign; } /* < 2^-25 -> 0 (2^-25 itself ties to even 0) */
    uint32_t e    = ax >> 23;
    uint32_t m    = (ax & 0x7fffffu) | 0x800000u;
    uint32_t sh   = 126u - e; /* 14..24 */
    uint32_t half = m >> sh;
    uint32_t rem  = m & ((1u << sh) - 1u);
    uint32_t mid  = 1u << (sh - 1u);
    if (rem > mid || (rem == mid && (half & 1u))) { half++; }
    return (uint16_t)(sign | half);
  }
  uint32_t h   = ((ax - 0x38000000u) >> 13);
  uint32_t rem = ax & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) { h++; }
  return (uint16_t)(sign | h);
}

static float g_h2f[65536];
static int g_h2f_ready = 0;

static float f16_to_f32_slow(uint16_t h)
{
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e    = (h >> 10) & 0x1fu;
  uint32_t m    = h & 0x3ffu;
  if (e == 0) {
    if (m == 0) { return u2f(sign); }
    float v = (float)m * (1.0f / 16777216.0f); /* m * 2^-24 */
    return sign ? -v : v;
  }
  if (e == 31) { return u2f(sign | 0x7f800000u | (m << 13)); }
  return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

static void init_tables(void)
{
  if (g_h2f_ready) { return; }
  for (uint32_t i = 0; i < 65536; i++) { g_h2f[i] = f16_to_f32_slow((uint16_t)i); }
  g_h2f_ready = 1;
}
static inline float f16_to_f32(uint16_t h) { return g_h2f[h]; }

/* half + half, correctly rounded: the exact sum is rounded once to fp32 and once more to fp16;
 * with 24 >= 2*11+2 significand bits the double rounding is innocuous. */
static inline uint16_t f16_add(uint16_t a, uint16_t b)
{
  return f32_to_f16(f16_to_f32(a) + f16_to_f32(b));
}

ORC_EXPORT uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
ORC_EXPORT float orc_f16_to_f32(uint16_t h)
{
  init_tables();
  return f16_to_f32(h);
}

/* ============================ 8-bit float (ivf_pq_fp_8bit.cuh:31-100) ========================= */
/* ExpBits = 5: ExpMask = 15, ValBits = 3. */
#define FP8_EXPMASK 15u
#define FP8_VALBITS 3u
#define FP8_EXPBITS 5u

static inline uint8_t fp8_encode_unsigned(float v)
{
  const float kMin = 1.0f / (float)(1u << FP8_EXPMASK);
  const float kMax = (float)(1u << (FP8_EXPMASK + 1u)) * (2.0f - 1.0f / (float)(1u << FP8_VALBITS));
  if (v < kMin) { return 0; } /* also catches negatives; NaN compares false and falls through */
  if (v >= kMax) { return 0xffu; }
  return (uint8_t)((f2u(v) + (FP8_EXPMASK << 23u) - 0x3f800000u) >> (15u + FP8_EXPBITS));
}
static inline uint8_t fp8_encode(float v, int is_signed)
{
  if (is_signed) {
    uint8_t u = fp8_encode_unsigned(fabsf(v));
    return (uint8_t)((u & 0xfeu) | (v < 0 ? 1u : 0u));
  }
  return fp8_encode_unsigned(v);
}
static inline float fp8_decode(uint8_t b, int is_signed)
{
  uint32_t u = b;
  if (is_signed) { u &= ~1u; }
  const uint32_t kBase32 = (0x3f800000u | (0x00400000u >> FP8_VALBITS)) - (FP8_EXPMASK << 23);
  float r                = u2f(kBase32 + (u << (15u + FP8_EXPBITS)));
  if (is_signed && (b & 1u)) { r = -r; }
  return r;
}
static inline uint16_t fp8_decode_half(uint8_t b, int is_signed)
{
  uint16_t u = b;
  if (is_signed) { u &= (uint16_t)~1u; }
  const uint16_t kBase16 = (uint16_t)((0x3c00u | (0x0200u >> FP8_VALBITS)) - (FP8_EXPMASK << 10));
  uint16_t r             = (uint16_t)(kBase16 + (u << (2u + FP8_EXPBITS)));
  if (is_signed && (b & 1u)) { r ^= 0x8000u; }
  return r;
}
ORC_EXPORT uint8_t orc_fp8_encode(float v, int is_signed) { return fp8_encode(v, is_signed); }
ORC_EXPORT float orc_fp8_decode(uint8_t b, int is_signed) { return fp8_decode(b, is_signed); }
ORC_EXPORT uint16_t orc_fp8_decode_half(uint8_t b, int is_signed)
{
  return fp8_decode_half(b, is_signed);
}

/* ============================ interleaved code layout ======================================== */
/* ivf_pq.hpp:235-296, ivf_pq_codepacking.cuh:30-168: vector i sits in group i/32, lane i%32;
 * its codes form a little-endian bit stream cut into 16-byte pieces of floor(128/bits) codes;
 * piece c lives at byte ((group*n_pieces + c)*32 + lane)*16. */

static inline uint32_t codes_per_piece(uint32_t bits) { return 128u / bits; }
static inline uint32_t n_pieces(uint32_t pq_dim, uint32_t bits)
{
  uint32_t cpp = codes_per_piece(bits);
  return (pq_dim + cpp - 1u) / cpp;
}
ORC_EXPORT uint64_t orc_list_bytes(uint32_t n_rows, uint32_t pq_dim, uint32_t bits)
{
  return (uint64_t)((n_rows + 31u) / 32u) * n_pieces(pq_dim, bits) * 512u;
}

static inline uint32_t read_code(const uint8_t* list, uint32_t i, uint32_t j, uint32_t pq_dim,
                                 uint32_t bits)
{
  uint32_t cpp      = codes_per_piece(bits);
  uint32_t np       = n_pieces(pq_dim, bits);
  uint32_t piece    = j / cpp;
  uint32_t k        = j % cpp;
  const uint8_t* p  = list + (((uint64_t)(i / 32u) * np + piece) * 32u + (i % 32u)) * 16u;
  uint32_t bit      = k * bits;
  uint32_t byte     = bit >> 3;
  uint32_t sh       = bit & 7u;
  uint32_t pair     = p[byte];
  if (sh + bits > 8u) { pair |= (uint32_t)p[byte + 1] << 8; }
  return (pair >> sh) & ((1u << bits) - 1u);
}
static inline void write_code(uint8_t* list, uint32_t i, uint32_t j, uint32_t pq_dim, uint32_t bits,
                              uint32_t code)
{
  uint32_t cpp   = codes_per_piece(bits);
  uint32_t np    = n_pieces(pq_dim, bits);
  uint32_t piece = j / cpp;
  uint32_t k     = j % cpp;
  uint8_t* p     = list + (((uint64_t)(i / 32u) * np + piece) * 32u + (i % 32u)) * 16u;
  uint32_t bit   = k * bits;
  uint32_t byte  = bit >> 3;
  uint32_t sh    = bit & 7u;
  uint32_t mask  = (1u << bits) - 1u;
  if (sh + bits > 8u) {
    uint32_t pair = p[byte] | ((uint32_t)p[byte + 1] << 8);
    pair &= ~(mask << sh);
    pair |= (code & mask) << sh;
    p[byte]     = (uint8_t)(pair & 0xffu);
    p[byte + 1] = (uint8_t)(pair >> 8);
  } else {
    p[byte] = (uint8_t)((p[byte] & ~(mask << sh)) | ((code & mask) << sh));
  }
}

/* codes: [n_rows, pq_dim] one code per byte -> interleaved list (must be zero-initialised). */
ORC_EXPORT void orc_pack_list(const uint8_t* codes, uint32_t n_rows, uint32_t pq_dim, uint32_t bits,
                              uint32_t first_row, uint8_t* list)
{
  for (uint32_t i = 0; i < n_rows; i++) {
    for (uint32_t j = 0; j < pq_dim; j++) {
      write_code(list, first_row + i, j, pq_dim, bits, codes[(uint64_t)i * pq_dim + j]);
    }
  }
}
ORC_EXPORT void orc_unpack_list(const uint8_t* list, uint32_t n_rows, uint32_t pq_dim, uint32_t bits,
                                uint32_t first_row, uint8_t* codes)
{
  for (uint32_t i = 0; i < n_rows; i++) {
    for (uint32_t j = 0; j < pq_dim; j++) {
      codes[(uint64_t)i * pq_dim + j] = (uint8_t)read_code(list, first_row + i, j, pq_dim, bits);
    }
  }
}

/* ============================ query preparation ============================================== */

/* mapping<float> (ann_utils.cuh:168-199): uint8 / 256, int8 / 128, half and float unchanged. */
static void map_query(const void* q, int qtype, uint32_t dim, float* out)
{
  switch (qtype) {
    case Q_F32: memcpy(out, q, (size_t)dim * 4); break;
    case Q_F16:
      for (uint32_t i = 0; i < dim; i++) { out[i] = f16_to_f32(((const uint16_t*)q)[i]); }
      break;
    case Q_I8:
      for (uint32_t i = 0; i < dim; i++) { out[i] = (float)((const int8_t*)q)[i] * (1.0f / 128.0f); }
      break;
    default:
      for (uint32_t i = 0; i < dim; i++) { out[i] = (float)((const uint8_t*)q)[i] * (1.0f / 256.0f); }
  }
}
static size_t qtype_size(int qtype) { return qtype == Q_F32 ? 4 : (qtype == Q_F16 ? 2 : 1); }

static int is_l2(int metric) { return metric == M_L2 || metric == M_L2SQRT; }

/* ============================ coarse stage =================================================== */

/* qc[l] = alpha * sum_k centers[l,k] * fq[k], fq padded with -0.5 (L2) or 0 at column dim. */
ORC_HOT static void coarse_scores(const orc_index* ix, const float* fq_ext, float* qc)
{
  const float alpha = is_l2(ix->metric) ? -2.0f : -1.0f;
  const uint32_t de = ix->dim_ext;
  for (uint32_t l = 0; l < ix->n_lists; l++) {
    const float* c = ix->centers + (size_t)l * de;
    float acc      = 0.0f;
    for (uint32_t k = 0; k < de; k++) { acc = fmaf(c[k], fq_ext[k], acc); }
    qc[l] = alpha * acc;
  }
}

typedef struct {
  float s;
  uint32_t i;
} cand_t;

static inline int cand_less(cand_t a, cand_t b) { return a.s < b.s || (a.s == b.s && a.i < b.i); }

/* bounded max-heap keeping the `cap` smallest candidates */
static void heap_push(cand_t* h, uint32_t* n, uint32_t cap, cand_t c)
{
  if (*n < cap) {
    uint32_t i = (*n)++;
    h[i]       = c;
    while (i > 0) {
      uint32_t p = (i - 1) / 2;
      if (cand_less(h[p], h[i])) {
        cand_t t = h[p];
        h[p]     = h[i];
        h[i]     = t;
        i        = p;
      } else {
        break;
      }
    }
    return;
  }
  if (!cand_less(c, h[0])) { return; }
  h[0]       = c;
  uint32_t i = 0;
  for (;;) {
    uint32_t l = 2 * i + 1, r = l + 1, m = i;
    if (l < cap && cand_less(h[m], h[l])) { m = l; }
    if (r < cap && cand_less(h[m], h[r])) { m = r; }
    if (m == i) { break; }
    cand_t t = h[m];
    h[m]     = h[i];
    h[i]     = t;
    i        = m;
  }
}
static int cand_cmp(const void* a, const void* b)
{
  cand_t x = *(const cand_t*)a, y = *(const cand_t*)b;
  return cand_less(x, y) ? -1 : (cand_less(y, x) ? 1 : 0);
}

/* ============================ LUT ============================================================ */

/* One LUT, kept in the storage type it would have on the GPU. */
typedef struct {
  int lut_dtype;
  int is_signed;
  float* f32;
  uint16_t* f16;
  uint8_t* u8;
} lut_t;

ORC_HOT static void build_lut(const orc_index* ix, uint32_t label, const float* rot_q, lut_t* lut,
                              float* base /* [rot_dim] or [2*rot_dim] scratch */)
{
  const uint32_t book = 1u << ix->pq_bits;
  const uint32_t len  = ix->pq_len;
  const float* c      = ix->centers_rot + (size_t)label * ix->rot_dim;
  const int l2        = is_l2(ix->metric);
  /* precompute_base_diff_impl.cuh */
  if (l2) {
    for (uint32_t i = 0; i < ix->rot_dim; i++) { base[i] = rot_q[i] - c[i]; }
  } else {
    for (uint32_t i = 0; i < ix->rot_dim; i++) {
      base[2 * i]     = rot_q[i];
      base[2 * i + 1] = c[i] * rot_q[i];
    }
  }
  const float* pqc0 = ix->codebook_kind == 0 ? ix->pq_centers
                                             : ix->pq_centers + (size_t)label * len * book;
  for (uint32_t j = 0; j < ix->pq_dim; j++) {
    const float* pqc = pqc0 + (ix->codebook_kind == 0 ? (size_t)j * len * book : 0);
    for (uint32_t b = 0; b < book; b++) {
      float score = 0.0f;
      for (uint32_t k = 0; k < len; k++) {
        float pq_c = pqc[(size_t)k * book + b];
        uint32_t d = j * len + k;
        if (l2) {
          float diff = base[d] - pq_c;
          score      = fmaf(diff, diff, score);
        } else {
          score = score - base[2 * d + 1];
          score = fmaf(-base[2 * d], pq_c, score);
        }
      }
      size_t e = (size_t)j * book + b;
      switch (lut->lut_dtype) {
        case DT_F32: lut->f32[e] = score; break;
        case DT_F16: lut->f16[e] = f32_to_f16(score); break;
        default: lut->u8[e] = fp8_encode(score, lut->is_signed);
      }
    }
  }
}

/* Decode the LUT into fp32 (f32 internal distances) or into fp16 bits (f16 internal). */
static void decode_lut(const lut_t* lut, size_t n, int internal_dtype, float* outf, uint16_t* outh)
{
  for (size_t e = 0; e < n; e++) {
    if (internal_dtype == DT_F32) {
      switch (lut->lut_dtype) {
        case DT_F32: outf[e] = lut->f32[e]; break;
        case DT_F16: outf[e] = f16_to_f32(lut->f16[e]); break;
        default: outf[e] = fp8_decode(lut->u8[e], lut->is_signed);
      }
    } else {
      switch (lut->lut_dtype) {
        case DT_F16: outh[e] = lut->f16[e]; break;
        default: outh[e] = fp8_decode_half(lut->u8[e], lut->is_signed);
      }
    }
  }
}

/* ============================ scan =========================================================== */

/* Scores of every vector of one list, in the order stored.  compute_score_impl.cuh:55-79 sums the
 * looked-up entries sequentially over the subspaces in the internal distance type. */
ORC_HOT static void scan_list_f32(const orc_index* ix, uint32_t label, const float* lutf, int cosine,
                                  float* scores)
{
  const uint32_t n    = ix->list_sizes[label];
  const uint32_t bits = ix->pq_bits, pq_dim = ix->pq_dim, book = 1u << bits;
  const uint8_t* list = ix->codes + ix->code_offsets[label];
  if (bits == 8) {
    const uint32_t np = (pq_dim + 15u) / 16u;
    for (uint32_t i = 0; i < n; i++) {
      const uint8_t* p = list + ((uint64_t)(i / 32u) * np * 32u + (i % 32u)) * 16u;
      float s          = 0.0f;
      for (uint32_t j = 0; j < pq_dim; j++) {
        s += lutf[(size_t)j * 256u + p[(size_t)(j >> 4) * 512u + (j & 15u)]];
      }
      scores[i] = cosine ? s + 1.0f : s;
    }
    return;
  }
  for (uint32_t i = 0; i < n; i++) {
    float s = 0.0f;
    for (uint32_t j = 0; j < pq_dim; j++) {
      s += lutf[(size_t)j * book + read_code(list, i, j, pq_dim, bits)];
    }
    scores[i] = cosine ? s + 1.0f : s;
  }
}

static void scan_list_f16(const orc_index* ix, uint32_t label, const uint16_t* luth, int cosine,
                          float* scores)
{
  const uint32_t n    = ix->list_sizes[label];
  const uint32_t bits = ix->pq_bits, pq_dim = ix->pq_dim, book = 1u << bits;
  const uint8_t* list = ix->codes + ix->code_offsets[label];
  for (uint32_t i = 0; i < n; i++) {
    uint16_t s = 0;
    for (uint32_t j = 0; j < pq_dim; j++) {
      s = f16_add(s, luth[(size_t)j * book + read_code(list, i, j, pq_dim, bits)]);
    }
    if (cosine) { s = f16_add(s, 0x3c00u); }
    scores[i] = f16_to_f32(s);
  }
}

/* ============================ distances post-processing ====================================== */
/* ivf_common.cuh:175-252 with scaling_factor = kDivisor<T> (ivf_pq_search.cuh:1043). */
static float postprocess(float score, int metric, float scale)
{
  switch (metric) {
    case M_L2: return scale != 1.0f ? score * (scale * scale) : score;
    case M_L2SQRT: return scale != 1.0f ? sqrtf(score) * scale : sqrtf(score);
    case M_IP: {
      float factor = -1.0f * scale * scale;
      return score * factor;
    }
    default: { /* cosine: no sign flip */
      float factor = scale * scale;
      return factor != 1.0f ? score * factor : score;
    }
  }
}

/* ============================ stage entry points (used by stage-wise parity tests) =========== */

ORC_EXPORT void orc_prepare_queries(const orc_index* ix, const void* queries, int qtype, uint32_t n_q,
                                    float* fq_ext /* [n_q, dim_ext] */, float* rot_q /* [n_q, rot_dim] */)
{
  init_tables();
  const size_t qs = qtype_size(qtype);
  for (uint32_t q = 0; q < n_q; q++) {
    float* f = fq_ext + (size_t)q * ix->dim_ext;
    map_query((const uint8_t*)queries + (size_t)q * ix->dim * qs, qtype, ix->dim, f);
    for (uint32_t k = ix->dim; k < ix->dim_ext; k++) { f[k] = 0.0f; }
    if (is_l2(ix->metric)) { f[ix->dim] = -0.5f; }
    float* r = rot_q + (size_t)q * ix->rot_dim;
    for (uint32_t i = 0; i < ix->rot_dim; i++) {
      const float* row = ix->rotation + (size_t)i * ix->dim;
      float acc        = 0.0f;
      for (uint32_t k = 0; k < ix->dim; k++) { acc = fmaf(row[k], f[k], acc); }
      r[i] = acc;
    }
    if (ix->metric == M_COSINE) {
      float ss = 0.0f;
      for (uint32_t i = 0; i < ix->rot_dim; i++) { ss = fmaf(r[i], r[i], ss); }
      float nrm = sqrtf(ss);
      if (nrm > 0.0f) {
        for (uint32_t i = 0; i < ix->rot_dim; i++) { r[i] = r[i] / nrm; }
      }
    }
  }
}

/* probes sorted by (score, list id) ascending; scores optional. */
ORC_EXPORT void orc_select_clusters(const orc_index* ix, const float* fq_ext, uint32_t n_q,
                                    uint32_t n_probes, uint32_t* probes, float* probe_scores,
                                    float* all_scores /* optional [n_q, n_lists] */)
{
  if (n_probes > ix->n_lists) { n_probes = ix->n_lists; }
#pragma omp parallel
  {
    float* qc   = (float*)malloc((size_t)ix->n_lists * sizeof(float));
    cand_t* hp  = (cand_t*)malloc((size_t)n_probes * sizeof(cand_t));
#pragma omp for schedule(dynamic, 4)
    for (int64_t q = 0; q < (int64_t)n_q; q++) {
      coarse_scores(ix, fq_ext + (size_t)q * ix->dim_ext, qc);
      if (all_scores) { memcpy(all_scores + (size_t)q * ix->n_lists, qc, (size_t)ix->n_lists * 4); }
      uint32_t n = 0;
      for (uint32_t l = 0; l < ix->n_lists; l++) {
        cand_t c = {qc[l], l};
        heap_push(hp, &n, n_probes, c);
      }
      qsort(hp, n, sizeof(cand_t), cand_cmp);
      for (uint32_t p = 0; p < n_probes; p++) {
        probes[(size_t)q * n_probes + p] = hp[p].i;
        if (probe_scores) { probe_scores[(size_t)q * n_probes + p] = hp[p].s; }
      }
    }
    free(qc);
    free(hp);
  }
}

/* ============================ int8 coarse search (coarse_search_dtype = CUDA_R_8I) =========== */

/* mapping<int8_t> of a float after the scaling (ann_utils.cuh:211-217): clamped to [-128, 127], then
 * converted toward zero.  The half-precision source takes the generic path, whose device
 * conversion half -> int8 saturates to the same range. */
static int8_t f32_to_i8(float x)
{
  if (x != x) { return 0; }
  if (x >= 127.0f) { return 127; }
  if (x <= -128.0f) { return -128; }
  return (int8_t)x;
}

ORC_EXPORT uint32_t orc_dim_ext_int8(uint32_t dim) { return (dim + 2 + 15) / 16 * 16; } /* ivf_pq_index.cu:667 */

/* centers_int8 (cpp/src/neighbors/ivf_pq_index.cu:661-738): out [n_lists, dim_ext_int8]. */
ORC_EXPORT void orc_centers_int8(const orc_index* ix, int8_t* out)
{
  const uint32_t d8 = orc_dim_ext_int8(ix->dim);
  for (uint32_t row = 0; row < ix->n_lists; row++) {
    const float* in = ix->centers + (size_t)row * ix->dim_ext;
    for (uint32_t col = 0; col < d8; col++) {
      int8_t v;
      if (col < ix->dim) {
        v = (int8_t)fmaxf(-128.0f, fminf(127.0f, in[col] * 128.0f));
      } else {
        const float x = in[ix->dim];
        const float c = 64.0f / (float)(d8 - ix->dim - 1);
        const float y = fmaxf(-128.0f, fminf(127.0f, x * c));
        const float z = fmaxf(-128.0f, fminf(127.0f, (y - roundf(y)) * 128.0f));
        v             = col > ix->dim ? (int8_t)roundf(y) : (int8_t)z;
      }
      out[(size_t)row * d8 + col] = v;
    }
  }
}

/* rotation_matrix_int8 (ivf_pq_index.cu:624-658): mapping<int8_t> of every element. */
ORC_EXPORT void orc_rotation_int8(const orc_index* ix, int8_t* out)
{
  const size_t n = (size_t)ix->rot_dim * ix->dim;
  for (size_t i = 0; i < n; i++) { out[i] = f32_to_i8(ix->rotation[i] * 128.0f); }
}

/* mapping<int8_t> of a query (ann_utils.cuh:178-209). */
static void map_query_int8(const void* q, int qtype, uint32_t dim, int8_t* out)
{
  switch (qtype) {
    case Q_F32:
      for (uint32_t i = 0; i < dim; i++) { out[i] = f32_to_i8(((const float*)q)[i] * 128.0f); }
      break;
    case Q_F16: /* the product with 128 is exact in half precision */
      for (uint32_t i = 0; i < dim; i++) { out[i] = f32_to_i8(f16_to_f32(((const uint16_t*)q)[i]) * 128.0f); }
      break;
    case Q_I8: memcpy(out, q, dim); break;
    default:
      for (uint32_t i = 0; i < dim; i++) { out[i] = (int8_t)(((const uint8_t*)q)[i] >> 1); }
  }
}

/* Queries of the int8 coarse search (ivf_pq_search.cuh:171-256) and their rotation
 * (:996-1025, alpha = 1/128/128): q8_ext [n_q, dim_ext_int8], rot_q [n_q, rot_dim]. */
ORC_EXPORT void orc_prepare_queries_int8(const orc_index* ix, const void* queries, int qtype, uint32_t n_q,
                                         const int8_t* rot8, int8_t* q8_ext, float* rot_q)
{
  init_tables();
  const uint32_t d8 = orc_dim_ext_int8(ix->dim);
  const uint32_t m  = d8 - ix->dim;
  const int8_t norm_factor = is_l2(ix->metric) ? -128 : 0;
  const size_t qs   = qtype_size(qtype);
  for (uint32_t q = 0; q < n_q; q++) {
    int8_t* f = q8_ext + (size_t)q * d8;
    map_query_int8((const uint8_t*)queries + (size_t)q * ix->dim * qs, qtype, ix->dim, f);
    for (uint32_t col = ix->dim; col < d8; col++) {
      f[col] = (m == 1 || col > ix->dim) ? norm_factor : (int8_t)(1 - (int)m);
    }
    float* r = rot_q + (size_t)q * ix->rot_dim;
    for (uint32_t i = 0; i < ix->rot_dim; i++) {
      const int8_t* row = rot8 + (size_t)i * ix->dim;
      int32_t acc       = 0;
      for (uint32_t k = 0; k < ix->dim; k++) { acc += (int32_t)row[k] * (int32_t)f[k]; }
      r[i] = (float)acc * (1.0f / 128.0f / 128.0f);
    }
    if (ix->metric == M_COSINE) {
      float ss = 0.0f;
      for (uint32_t i = 0; i < ix->rot_dim; i++) { ss = fmaf(r[i], r[i], ss); }
      float nrm = sqrtf(ss);
      if (nrm > 0.0f) {
        for (uint32_t i = 0; i < ix->rot_dim; i++) { r[i] = r[i] / nrm; }
      }
    }
  }
}

typedef struct {
  int32_t s;
  uint32_t i;
} icand_t;
static int icand_cmp(const void* a, const void* b)
{
  const icand_t x = *(const icand_t*)a, y = *(const icand_t*)b;
  if (x.s != y.s) { return x.s < y.s ? -1 : 1; }
  return x.i < y.i ? -1 : (x.i > y.i ? 1 : 0);
}

/* int32 scores alpha * <c8, q8> (alpha = -2 for L2, -1 otherwise), the n_probes smallest by
 * (score, list id).  The reference's selection does not define the order of equal scores. */
ORC_EXPORT void orc_select_clusters_int8(const orc_index* ix, const int8_t* c8, const int8_t* q8_ext,
                                         uint32_t n_q, uint32_t n_probes, uint32_t* probes, int32_t* probe_scores)
{
  const uint32_t d8   = orc_dim_ext_int8(ix->dim);
  const int32_t alpha = is_l2(ix->metric) ? -2 : -1;
  if (n_probes > ix->n_lists) { n_probes = ix->n_lists; }
  icand_t* all = (icand_t*)malloc((size_t)ix->n_lists * sizeof(icand_t));
  for (uint32_t q = 0; q < n_q; q++) {
    const int8_t* f = q8_ext + (size_t)q * d8;
    for (uint32_t l = 0; l < ix->n_lists; l++) {
      const int8_t* c = c8 + (size_t)l * d8;
      int32_t acc     = 0;
      for (uint32_t k = 0; k < d8; k++) { acc += (int32_t)c[k] * (int32_t)f[k]; }
      all[l].s = alpha * acc;
      all[l].i = l;
    }
    qsort(all, ix->n_lists, sizeof(icand_t), icand_cmp);
    for (uint32_t p = 0; p < n_probes; p++) {
      probes[(size_t)q * n_probes + p] = all[p].i;
      if (probe_scores) { probe_scores[(size_t)q * n_probes + p] = all[p].s; }
    }
  }
  free(all);
}

/* ============================ fp16 coarse search (coarse_search_dtype = CUDA_R_16F) ========== */
/* ivf_pq_search.cuh:259-340 and :996-1025: queries, centers (with their norm column) and the rotation
 * matrix are rounded to half precision, the products are library GEMMs whose accumulation the
 * reference does not define, the scores are half-precision numbers and select_k leaves equal scores in
 * unspecified order.  The rule restated here (and computed by the GPU path): fp32 fused multiply-adds
 * over ascending k on the half-rounded operands, the scaled sum rounded once to half precision, probes
 * ordered by (half score, list id); rotated queries by the same chain, kept in fp32. */
static float round_to_half(float x) { return f16_to_f32(f32_to_f16(x)); }

/* mapping<half> of one query element (ann_utils.cuh:168-199), widened to fp32 */
static float map_query_f16(const void* q, int qtype, uint32_t i)
{
  switch (qtype) {
    case Q_F32: return round_to_half(((const float*)q)[i]);
    case Q_F16: return f16_to_f32(((const uint16_t*)q)[i]);
    case Q_I8: return (float)((const int8_t*)q)[i] * (1.0f / 128.0f); /* exact in half precision */
    default: return (float)((const uint8_t*)q)[i] * (1.0f / 256.0f);
  }
}

ORC_EXPORT void orc_prepare_queries_f16(const orc_index* ix, const void* queries, int qtype, uint32_t n_q,
                                        float* fq_ext /* [n_q, dim_ext] half values */, float* rot_q)
{
  init_tables();
  const size_t qs = qtype_size(qtype);
  for (uint32_t q = 0; q < n_q; q++) {
    float* f = fq_ext + (size_t)q * ix->dim_ext;
    const uint8_t* src = (const uint8_t*)queries + (size_t)q * ix->dim * qs;
    for (uint32_t k = 0; k < ix->dim; k++) { f[k] = map_query_f16(src, qtype, k); }
    for (uint32_t k = ix->dim; k < ix->dim_ext; k++) { f[k] = 0.0f; }
    if (is_l2(ix->metric)) { f[ix->dim] = -0.5f; }
    float* r = rot_q + (size_t)q * ix->rot_dim;
    for (uint32_t i = 0; i < ix->rot_dim; i++) {
      const float* row = ix->rotation + (size_t)i * ix->dim;
      float acc        = 0.0f;
      for (uint32_t k = 0; k < ix->dim; k++) { acc = fmaf(round_to_half(row[k]), f[k], acc); }
      r[i] = acc;
    }
    if (ix->metric == M_COSINE) {
      float ss = 0.0f;
      for (uint32_t i = 0; i < ix->rot_dim; i++) { ss = fmaf(r[i], r[i], ss); }
      float nrm = sqrtf(ss);
      if (nrm > 0.0f) {
        for (uint32_t i = 0; i < ix->rot_dim; i++) { r[i] = r[i] / nrm; }
      }
    }
  }
}

ORC_EXPORT void orc_select_clusters_f16(const orc_index* ix, const float* fq_ext, uint32_t n_q,
                                        uint32_t n_probes, uint32_t* probes, float* probe_scores)
{
  init_tables();
  if (n_probes > ix->n_lists) { n_probes = ix->n_lists; }
  const float alpha = is_l2(ix->metric) ? -2.0f : -1.0f;
  float* ch = (float*)malloc((size_t)ix->n_lists * ix->dim_ext * sizeof(float));
  for (size_t i = 0; i < (size_t)ix->n_lists * ix->dim_ext; i++) { ch[i] = round_to_half(ix->centers[i]); }
#pragma omp parallel
  {
    cand_t* all = (cand_t*)malloc((size_t)ix->n_lists * sizeof(cand_t));
#pragma omp for schedule(dynamic, 4)
    for (int64_t q = 0; q < (int64_t)n_q; q++) {
      const float* f = fq_ext + (size_t)q * ix->dim_ext;
      for (uint32_t l = 0; l < ix->n_lists; l++) {
        const float* c = ch + (size_t)l * ix->dim_ext;
        float acc      = 0.0f;
        for (uint32_t k = 0; k < ix->dim_ext; k++) { acc = fmaf(c[k], f[k], acc); }
        all[l].s = round_to_half(alpha * acc);
        all[l].i = l;
      }
      qsort(all, ix->n_lists, sizeof(cand_t), cand_cmp);
      for (uint32_t p = 0; p < n_probes; p++) {
        probes[(size_t)q * n_probes + p] = all[p].i;
        if (probe_scores) { probe_scores[(size_t)q * n_probes + p] = all[p].s; }
      }
    }
    free(all);
  }
  free(ch);
}

/* LUT of one (query, list) pair in its storage type (4, 2 or 1 bytes per entry). */
ORC_EXPORT void orc_build_lut(const orc_index* ix, uint32_t label, const float* rot_q, int lut_dtype,
                              void* out)
{
  init_tables();
  lut_t lut;
  lut.lut_dtype = lut_dtype;
  lut.is_signed = !is_l2(ix->metric);
  lut.f32       = (float*)out;
  lut.f16       = (uint16_t*)out;
  lut.u8        = (uint8_t*)out;
  float* base   = (float*)malloc((size_t)ix->rot_dim * 2 * sizeof(float));
  build_lut(ix, label, rot_q, &lut, base);
  free(base);
}

/* Internal scores of every vector of one (query, list) pair, widened to fp32, in stored order:
 * what compute_distances_impl.cuh:73-90 produces before the top-k.  Returns -1 for the one invalid
 * pairing (fp32 table with fp16 internal distances). */
ORC_EXPORT int orc_pair_scores(const orc_index* ix, uint32_t label, const float* rot_q, int lut_dtype,
                               int internal_dtype, float* scores)
{
  init_tables();
  if (internal_dtype == DT_F16 && lut_dtype == DT_F32) { return -1; }
  const size_t lut_n = (size_t)ix->pq_dim << ix->pq_bits;
  lut_t lut;
  void* lut_raw  = malloc(lut_n * 4);
  lut.lut_dtype  = lut_dtype;
  lut.is_signed  = !is_l2(ix->metric);
  lut.f32        = (float*)lut_raw;
  lut.f16        = (uint16_t*)lut_raw;
  lut.u8         = (uint8_t*)lut_raw;
  float* lutf    = (float*)malloc(lut_n * 4);
  uint16_t* luth = (uint16_t*)malloc(lut_n * 2);
  float* base    = (float*)malloc((size_t)ix->rot_dim * 2 * sizeof(float));
  build_lut(ix, label, rot_q, &lut, base);
  decode_lut(&lut, lut_n, internal_dtype, lutf, luth);
  if (internal_dtype == DT_F32) {
    scan_list_f32(ix, label, lutf, ix->metric == M_COSINE, scores);
  } else {
    scan_list_f16(ix, label, luth, ix->metric == M_COSINE, scores);
  }
  free(lut_raw);
  free(lutf);
  free(luth);
  free(base);
  return 0;
}

ORC_EXPORT float orc_postprocess(float score, int metric, float scale) { return postprocess(score, metric, scale); }

/* Fine search given the probes: neighbours [n_q,k] int64, distances [n_q,k] f32.
 * Optional raw outputs: internal scores before post-processing. */
/* Bitset sample filter (cpp/src/neighbors/sample_filter.cuh:162-176): a vector is searched only if
 * bit `source id` of the bitset is set.  NULL = no filter. */
static const uint32_t* g_filter_bits = NULL;
static uint64_t g_filter_nbits       = 0;
ORC_EXPORT void orc_set_filter(const uint32_t* bits, uint64_t nbits)
{
  g_filter_bits  = bits;
  g_filter_nbits = nbits;
}
static inline int filter_pass(int64_t id)
{
  if (!g_filter_bits) { return 1; }
  if (id < 0 || (uint64_t)id >= g_filter_nbits) { return 0; }
  return (g_filter_bits[id >> 5] >> (id & 31)) & 1u;
}

ORC_EXPORT int orc_search_probes(const orc_index* ix, const float* rot_q, const uint32_t* probes,
                                 uint32_t n_q, uint32_t n_probes, uint32_t k, int lut_dtype,
                                 int internal_dtype, float scale, int64_t* neighbors,
                                 float* distances, float* raw_scores)
{
  init_tables();
  if (internal_dtype == DT_F16 && lut_dtype == DT_F32) { return -1; }
  const size_t lut_n = (size_t)ix->pq_dim << ix->pq_bits;
  uint32_t max_list  = 0;
  for (uint32_t l = 0; l < ix->n_lists; l++) {
    if (ix->list_sizes[l] > max_list) { max_list = ix->list_sizes[l]; }
  }
  const int cosine = ix->metric == M_COSINE;
#pragma omp parallel
  {
    lut_t lut;
    lut.lut_dtype  = lut_dtype;
    lut.is_signed  = !is_l2(ix->metric);
    void* lut_raw  = malloc(lut_n * 4);
    lut.f32        = (float*)lut_raw;
    lut.f16        = (uint16_t*)lut_raw;
    lut.u8         = (uint8_t*)lut_raw;
    float* lutf    = (float*)malloc(lut_n * 4);
    uint16_t* luth = (uint16_t*)malloc(lut_n * 2);
    float* base    = (float*)malloc((size_t)ix->rot_dim * 2 * sizeof(float));
    float* scores  = (float*)malloc(((size_t)max_list + 1) * sizeof(float));
    cand_t* hp     = (cand_t*)malloc((size_t)k * sizeof(cand_t));
    uint32_t* chunk = (uint32_t*)malloc((size_t)n_probes * sizeof(uint32_t));
#pragma omp for schedule(dynamic, 1)
    for (int64_t q = 0; q < (int64_t)n_q; q++) {
      const uint32_t* pr = probes + (size_t)q * n_probes;
      const float* rq    = rot_q + (size_t)q * ix->rot_dim;
      uint32_t nh        = 0;
      uint32_t offset    = 0;
      for (uint32_t p = 0; p < n_probes; p++) {
        uint32_t label = pr[p];
        uint32_t n     = ix->list_sizes[label];
        if (n > 0) {
          build_lut(ix, label, rq, &lut, base);
          decode_lut(&lut, lut_n, internal_dtype, lutf, luth);
          if (internal_dtype == DT_F32) {
            scan_list_f32(ix, label, lutf, cosine, scores);
          } else {
            scan_list_f16(ix, label, luth, cosine, scores);
          }
          for (uint32_t i = 0; i < n; i++) {
            if (!filter_pass(ix->ids[ix->id_offsets[label] + i])) { continue; }
            cand_t c = {scores[i], offset + i};
            heap_push(hp, &nh, k, c);
          }
        }
        offset += n;
        chunk[p] = offset; /* calc_chunk_indices: inclusive prefix sum */
      }
      qsort(hp, nh, sizeof(cand_t), cand_cmp);
      for (uint32_t r = 0; r < k; r++) {
        size_t o = (size_t)q * k + r;
        if (r < nh) {
          /* postprocess_neighbors_kernel: find the probe whose range holds the sample */
          uint32_t s = hp[r].i, p = 0;
          while (chunk[p] <= s) { p++; }
          uint32_t in_list = s - (p > 0 ? chunk[p - 1] : 0);
          neighbors[o]     = ix->ids[ix->id_offsets[pr[p]] + in_list];
          distances[o]     = postprocess(hp[r].s, ix->metric, scale);
          if (raw_scores) { raw_scores[o] = hp[r].s; }
        } else {
          neighbors[o] = INT64_MAX; /* kOutOfBoundsRecord<int64_t> */
          distances[o] = postprocess(INFINITY, ix->metric, scale);
          if (raw_scores) { raw_scores[o] = INFINITY; }
        }
      }
    }
    free(lut_raw);
    free(lutf);
    free(luth);
    free(base);
    free(scores);
    free(hp);
    free(chunk);
  }
  return 0;
}

/* Whole search: ivf_pq_search.cuh:881-1058. */
ORC_EXPORT int orc_search(const orc_index* ix, const void* queries, int qtype, uint32_t n_q,
                          uint32_t n_probes, uint32_t k, int lut_dtype, int internal_dtype,
                          int64_t* neighbors, float* distances, uint32_t* probes_out)
{
  if (n_probes > ix->n_lists) { n_probes = ix->n_lists; }
  if (n_probes == 0 || k == 0) { return -2; }
  float* fq      = (float*)malloc((size_t)n_q * ix->dim_ext * sizeof(float));
  float* rq      = (float*)malloc((size_t)n_q * ix->rot_dim * sizeof(float));
  uint32_t* prb  = probes_out ? probes_out : (uint32_t*)malloc((size_t)n_q * n_probes * 4);
  orc_prepare_queries(ix, queries, qtype, n_q, fq, rq);
  orc_select_clusters(ix, fq, n_q, n_probes, prb, NULL, NULL);
  float scale = qtype == Q_U8 ? 256.0f : (qtype == Q_I8 ? 128.0f : 1.0f);
  int rc = orc_search_probes(ix, rq, prb, n_q, n_probes, k, lut_dtype, internal_dtype, scale,
                             neighbors, distances, NULL);
  free(fq);
  free(rq);
  if (!probes_out) { free(prb); }
  return rc;
}

/* ============================ encoder used by the CPU index builder ========================== */
/* Same choice rule as ivf_pq_process_and_fill_codes.cuh:84-126: for each subspace the code whose
 * codebook entry has the smallest squared distance to the rotated residual, lowest code on ties. */
ORC_EXPORT void orc_encode(const orc_index* ix, const float* dataset_f32 /* [n, dim] already mapped */,
                           const uint32_t* labels, uint32_t n, uint8_t* codes /* [n, pq_dim] */)
{
  const uint32_t book = 1u << ix->pq_bits, len = ix->pq_len;
#pragma omp parallel
  {
    float* res = (float*)malloc((size_t)ix->rot_dim * sizeof(float));
    float* xc  = (float*)malloc((size_t)ix->dim * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; i++) {
      const uint32_t l = labels[i];
      const float* x   = dataset_f32 + (size_t)i * ix->dim;
      const float* c   = ix->centers + (size_t)l * ix->dim_ext;
      for (uint32_t d = 0; d < ix->dim; d++) { xc[d] = x[d] - c[d]; }
      for (uint32_t r = 0; r < ix->rot_dim; r++) {
        const float* row = ix->rotation + (size_t)r * ix->dim;
        float acc        = 0.0f;
        for (uint32_t d = 0; d < ix->dim; d++) { acc = fmaf(row[d], xc[d], acc); }
        res[r] = acc;
      }
      const float* pqc0 = ix->codebook_kind == 0 ? ix->pq_centers
                                                 : ix->pq_centers + (size_t)l * len * book;
      for (uint32_t j = 0; j < ix->pq_dim; j++) {
        const float* pqc = pqc0 + (ix->codebook_kind == 0 ? (size_t)j * len * book : 0);
        float best       = INFINITY;
        uint32_t best_b  = 0;
        for (uint32_t b = 0; b < book; b++) {
          float d2 = 0.0f;
          for (uint32_t k = 0; k < len; k++) {
            float t = res[j * len + k] - pqc[(size_t)k * book + b];
            d2      = fmaf(t, t, d2);
          }
          if (d2 < best) {
            best   = d2;
            best_b = b;
          }
        }
        codes[(size_t)i * ix->pq_dim + j] = (uint8_t)best_b;
      }
    }
    free(res);
    free(xc);
  }
}

ORC_EXPORT int orc_num_threads(void)
{
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
ORC_EXPORT void orc_set_num_threads(int n)
{
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}
