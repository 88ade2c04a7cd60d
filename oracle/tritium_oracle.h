/*
 * CPU oracle for the packed additive-ternary linear layer.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference project's scalar algorithms.  It is
 * linked or loaded only by the test suite, the smoke check and the CPU-baseline leg of
 * the benchmark; the product library never calls it.
 *
 * Parity pinning: the reference is Rust and cannot be compiled in the build image, so the
 * oracle is pinned by the known-answer vectors and formula fixtures of the reference's own
 * unit tests (see tests/test_oracle_golden.py).  Each function cites the reference source
 * it follows (paths are relative to the reference workspace root).
 */
#ifndef TRITIUM_ORACLE_H
#define TRITIUM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OR_TILE 256u      /* crates/tritium-format/src/salt_v2_package.rs:44 */
#define OR_MAX_PLANES 3u  /* salt_v2_package.rs:47 */
#define OR_RANK_STRIDE 256u /* salt_v2_package.rs:83 */

/* Codec identifiers as stored in a package header (salt_v2_package.rs:2747-2762). */
enum { OR_CODEC_D2 = 1, OR_CODEC_B3 = 2, OR_CODEC_S34 = 3 };

/* Error codes (negative = failure). */
enum {
  OR_OK = 0,
  OR_ERR_LENGTH = -1,         /* wrong packed length / declared size mismatch */
  OR_ERR_INVALID_CODE = -2,   /* D2 code 11, B3 byte >= 243 */
  OR_ERR_PADDING = -3,        /* non-canonical padding trit / bit / map padding */
  OR_ERR_S34_SHAPE = -4,      /* S34 needs a multiple of four trits / one zero per group */
  OR_ERR_PLANE_LEN = -5,
  OR_ERR_TRIT = -6,
  OR_ERR_SCALE_COUNT = -7,
  OR_ERR_SCALE_NONFINITE = -8,
  OR_ERR_SCALE_NEGATIVE = -9,
  OR_ERR_SCALE_ZERO_NONZERO_GROUP = -10,
  OR_ERR_PLANE_COUNT = -11,
  OR_ERR_GROUP_SIZE = -12,
  OR_ERR_SHAPE = -13,
  OR_ERR_MAGIC = -14,
  OR_ERR_VERSION = -15,
  OR_ERR_CODEC = -16,
  OR_ERR_FLAGS = -17,
  OR_ERR_TRUNCATED = -18,
  OR_ERR_TRAILING = -19,
  OR_ERR_NON_NESTED_MAP = -20,
  OR_ERR_NAME = -21,
  OR_ERR_TRANSFORM = -22,
  OR_ERR_NONFINITE_ACTIVATION = -23,
  OR_ERR_NONFINITE_OUTPUT = -24,
  OR_ERR_ALLOC = -25,
  OR_ERR_DUPLICATE_NAME = -26
};

/* ---- f16 <-> f32 (IEEE binary16, round to nearest even), as `half` 2.7.1 does ---- */
uint16_t or_f32_to_f16(float value);
float or_f16_to_f32(uint16_t bits);

/* ---- codecs: crates/tritium-format/src/salt_v2.rs ---- */
/* ledger():  out = {physical_bytes, canonical_padding_trits, canonical_padding_bits, encoded_bits} */
int or_codec_ledger(int codec, size_t logical_trits, uint64_t out[4]);
/* pack_d2 / pack_b3 / pack_s34; returns bytes written or an error. `out` may be NULL to size. */
long or_codec_pack(int codec, const int8_t* trits, size_t n, uint8_t* out, size_t out_cap);
/* unpack_*: canonical decode with every rejection rule of the reference. */
int or_codec_unpack(int codec, const uint8_t* packed, size_t packed_len, size_t logical_trits,
                    int8_t* trits_out);
/* Plane-level pack/unpack including the S34 shape padding of a ragged final tile
 * (salt_v2_package.rs:2383-2456). */
long or_plane_pack(int codec, const int8_t* trits, size_t logical_len, uint8_t* out, size_t out_cap);
int or_plane_unpack(int codec, const uint8_t* packed, size_t packed_len, size_t logical_len,
                    int8_t* trits_out);
size_t or_plane_payload_bytes(int codec, size_t logical_len);

/* ---- semantic tensor: crates/tritium-format/src/salt_v2_package.rs:94-251,582-641 ----
 * Dense host representation used by the oracle: tile t, plane p, element e live at
 * trits[(t*3+p)*256+e] and scales[(t*3+p)*4+g] (f16 bits). */
typedef struct {
  uint64_t rows, cols;       /* matrix dims; coefficients = rows*cols */
  uint32_t rank;             /* 2 (matrix) or 1 (vector: rows must be 1); 0 means 2 */
  uint32_t group;            /* 64 or 128 */
  uint64_t tiles;            /* ceil(coefficients/256) */
  const uint8_t* plane_count; /* [tiles], 1..3 */
  const int8_t* trits;
  const uint16_t* scales;
} or_tensor;

int or_tensor_validate(const or_tensor* t);

/* ---- indexed runtime (resident) layout: salt_v2_package.rs:889-962 and
 * crates/tritium-cuda/src/cuda/backend.rs:7463-7651 ---- */
typedef struct {
  uint64_t payload_bytes, scale_bytes, map_bytes, rank_prefix_bytes;
  uint64_t tiles, present_planes;
  uint32_t terminal_map_value;
} or_resident_sizes;
int or_resident_plan(const or_tensor* t, int codec, or_resident_sizes* out);
/* index_metadata = map bytes followed by LE u32 rank prefixes. Map code = planes-1. */
int or_resident_build(const or_tensor* t, int codec, uint8_t* payload, uint16_t* scales,
                      uint8_t* index_metadata, uint32_t* terminal_map_value);

/* ---- package bytes: salt_v2_package.rs:1526-1668 (write), 1679-1978 (read) ---- */
typedef struct {
  const char* name;
  or_tensor tensor;
} or_named_tensor;
/* Returns total bytes (or error). `out` may be NULL to size. */
long or_package_write(int codec, const or_named_tensor* tensors, size_t count, uint8_t* out,
                      size_t out_cap);
/* Header probe: tensor count / codec. */
int or_package_probe(const uint8_t* bytes, size_t len, int* codec, uint32_t* tensor_count);
/* Describe tensor `index`: fills rows, cols, group, tiles and name (up to name_cap-1 bytes). */
int or_package_tensor_info(const uint8_t* bytes, size_t len, uint32_t index, uint64_t* rows,
                           uint64_t* cols, uint32_t* group, uint64_t* tiles, uint32_t* rank,
                           char* name, size_t name_cap);
/* Decode tensor `index` into caller arrays sized from or_package_tensor_info. Validates the
 * whole package (every rejection rule). */
int or_package_read_tensor(const uint8_t* bytes, size_t len, uint32_t index, uint8_t* plane_count,
                           int8_t* trits, uint16_t* scales);

/* ---- the operator: crates/tritium-cpu/src/salt_v2.rs:316-423 ---- */
typedef struct {
  uint64_t row, column;      /* NonFiniteOutput{row,column} / NonFiniteActivation{index=column} */
  uint32_t bits;
} or_fail;
int or_matvec(const or_tensor* t, const float* x, float* y, or_fail* fail);
/* Same arithmetic over the resident arenas: crates/tritium-nn/src/layers/salt_v2_host.rs:235-354 */
int or_forward_packed(int codec, uint32_t group, uint64_t rows, uint64_t cols,
                      const uint8_t* payload, const uint16_t* scales, const uint8_t* index_metadata,
                      uint64_t map_bytes, uint32_t terminal_map_value, const float* x, uint64_t m,
                      float* y, or_fail* fail);
/* Row-parallel (POSIX threads) variant of or_matvec for timing; identical per-row arithmetic. */
int or_matmul_mt(const or_tensor* t, const float* x, uint64_t m, float* y, int threads);
/* salt_v2_gather_rows: salt_v2_host.rs:277-294,356-387 */
int or_gather_rows(const or_tensor* t, const uint32_t* rows, uint64_t count, float* out);

/* ---- int8 activation quantisation: crates/tritium-spec/src/lib.rs:351-378 ---- */
void or_quantize_act_int8(const float* act, uint64_t m, uint64_t k, float* q_out, float* scale_out);
/* quant -> contraction (exact integers) -> fold; I_dump is [m][rows][groups_per_row][3] int32
 * (zero where a plane is absent) or NULL.  groups_per_row = number of scale segments a row
 * crosses (cols/group when cols is a multiple of the group size). */
int or_a8_linear(const or_tensor* t, const float* x, uint64_t m, float* y, int32_t* i_dump,
                 float* act_scale_out);

/* ---- TQ2_0 trait path ---- */
/* crates/tritium-format/src/tq2.rs:21-83, src/rows.rs:61-77 */
int or_tq2_pack_row(const int8_t* trits, uint64_t k, const uint16_t* block_scales, uint8_t* out);
int or_tq2_unpack_row(const uint8_t* packed, uint64_t k, int8_t* trits_out, uint16_t* scales_out);
/* crates/tritium-core/src/reference.rs:25-55 */
int or_tq1_pack_row(const int8_t* trits, uint64_t k, const uint16_t* block_scales, uint8_t* out);
int or_tq1_unpack_row(const uint8_t* packed, uint64_t k, int8_t* trits_out, uint16_t* scales_out);
int or_salt_v1_matmul(const uint8_t* planes, uint32_t t_planes, uint64_t n, uint64_t k, const float* act,
                      uint64_t m, float* out);
/* crates/tritium-nn/src/ops/rmsnorm.rs:20-94 */
float or_sum_squares_canonical(const float* x, uint64_t n);
void or_rmsnorm(const float* x, const float* w, float eps, int zero_centered, uint64_t n, float* out);
void or_reference_mpgemm(const float* act, const int8_t* w, const float* scale_n, uint64_t m,
                         uint64_t n, uint64_t k, float* out);
/* crates/tritium-spec/src/lib.rs:266-318 (default host path) */
void or_mpgemm_with_act_quant(const float* act, const int8_t* w, const float* scale_n, uint64_t m,
                              uint64_t n, uint64_t k, float* out);

/* ---- conformance generator: crates/tritium-testkit/src/generate.rs:18-56 ---- */
typedef struct { uint64_t state; } or_xorshift;
void or_xs_seed(or_xorshift* r, uint64_t seed);
uint64_t or_xs_next(or_xorshift* r);
uint64_t or_xs_below(or_xorshift* r, uint64_t n);
float or_xs_activation(or_xorshift* r);
float or_xs_scale(or_xorshift* r);
int8_t or_xs_trit(or_xorshift* r);

#ifdef __cplusplus
}
#endif
#endif
