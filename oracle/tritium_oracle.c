/*
 * CPU oracle for the packed additive-ternary linear layer.  TEST INFRASTRUCTURE ONLY:
 * a plain-C restatement of the reference project's scalar algorithms, used by the tests,
 * the smoke check and the CPU-baseline leg of the benchmark as the checker.  The product
 * library does not link, load or call anything in this file.
 *
 * Build with -O2 -ffp-contract=off: every float operation below must stay a separate IEEE
 * single-precision operation (the reference order contract, crates/tritium-cpu/src/salt_v2.rs:10-23).
 *
 * Parity pinning: the reference (Rust) cannot be built in this image.  The oracle is pinned
 * against the known-answer vectors and formula fixtures in the reference's own unit tests;
 * the int8-activation x multi-plane composition is pinned part by part only (quantiser and
 * contraction separately), because the reference holds no test that runs the two together.
 */
#include "tritium_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ f16 <-> f32 */

static uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

/* IEEE binary32 -> binary16, round to nearest even (the `half` crate's from_f32). */
uint16_t or_f32_to_f16(float value) {
  uint32_t x = f32_bits(value);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t exp = (x >> 23) & 0xffu;
  uint32_t man = x & 0x7fffffu;
  if (exp == 0xffu) {
    if (man == 0) return (uint16_t)(sign | 0x7c00u);
    return (uint16_t)(sign | 0x7c00u | 0x0200u | (man >> 13));
  }
  int32_t e = (int32_t)exp - 127 + 15;
  if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign;
    man |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - e);
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
    return (uint16_t)(sign | half_man);
  }
  uint32_t half = sign | ((uint32_t)e << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
  return (uint16_t)half;
}

float or_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_f32(sign);
    int e = -1;
    do { e++; man <<= 1; } while ((man & 0x400u) == 0);
    man &= 0x3ffu;
    return bits_f32(sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13));
  }
  if (exp == 0x1f) return bits_f32(sign | 0x7f800000u | (man << 13));
  return bits_f32(sign | ((exp - 15 + 127) << 23) | (man << 13));
}

/* ------------------------------------------------------------------ codecs */
/* crates/tritium-format/src/salt_v2.rs:185-257 */
int or_codec_ledger(int codec, size_t n, uint64_t out[4]) {
  uint64_t bytes, pad_trits = 0, pad_bits = 0, bits;
  if (codec == OR_CODEC_D2) {
    bytes = (n + 3) / 4; bits = bytes * 8;
    if (n % 4) pad_trits = 4 - n % 4;
  } else if (codec == OR_CODEC_B3) {
    bytes = (n + 4) / 5; bits = bytes * 8;
    if (n % 5) pad_trits = 5 - n % 5;
  } else if (codec == OR_CODEC_S34) {
    if (n % 4) return OR_ERR_S34_SHAPE;
    bits = (uint64_t)(n / 4) * 5;
    bytes = (bits + 7) / 8;
    pad_bits = (8 - bits % 8) % 8;
  } else {
    return OR_ERR_CODEC;
  }
  out[0] = bytes; out[1] = pad_trits; out[2] = pad_bits; out[3] = bits;
  return OR_OK;
}

/* salt_v2.rs:268-281 (D2), 333-351 (B3), 411-440 (S34) */
long or_codec_pack(int codec, const int8_t* trits, size_t n, uint8_t* out, size_t out_cap) {
  uint64_t led[4];
  int rc = or_codec_ledger(codec, n, led);
  if (rc) return rc;
  size_t bytes = (size_t)led[0];
  if (!out) return (long)bytes;
  if (out_cap < bytes) return OR_ERR_LENGTH;
  for (size_t i = 0; i < n; i++)
    if (trits[i] < -1 || trits[i] > 1) return OR_ERR_TRIT;
  if (codec == OR_CODEC_D2) {
    memset(out, 0x55, bytes);
    for (size_t i = 0; i < n; i++) {
      unsigned shift = 2u * (unsigned)(i % 4);
      out[i / 4] = (uint8_t)((out[i / 4] & ~(3u << shift)) | ((unsigned)(trits[i] + 1) << shift));
    }
  } else if (codec == OR_CODEC_B3) {
    for (size_t b = 0; b < bytes; b++) {
      unsigned code = 0, place = 1;
      for (unsigned s = 0; s < 5; s++) {
        size_t ti = b * 5 + s;
        unsigned digit = ti < n ? (unsigned)(trits[ti] + 1) : 1u;
        code += digit * place;
        place *= 3;
      }
      out[b] = (uint8_t)code;
    }
  } else {
    memset(out, 0, bytes);
    for (size_t g = 0; g < n / 4; g++) {
      const int8_t* grp = trits + g * 4;
      int zeros = 0, zero_index = -1;
      for (int s = 0; s < 4; s++)
        if (grp[s] == 0) { zeros++; if (zero_index < 0) zero_index = s; }
      if (zeros != 1) return OR_ERR_S34_SHAPE;
      unsigned code = (unsigned)zero_index, sign_index = 0;
      for (int s = 0; s < 4; s++) {
        if (grp[s] == 0) continue;
        if (grp[s] == 1) code |= 1u << (2 + sign_index);
        sign_index++;
      }
      size_t bit = g * 5, byte = bit / 8;
      unsigned shift = (unsigned)(bit % 8);
      unsigned shifted = code << shift;
      out[byte] |= (uint8_t)shifted;
      if (shift + 5 > 8) out[byte + 1] |= (uint8_t)(shifted >> 8);
    }
  }
  return (long)bytes;
}

/* salt_v2.rs:294-322 (D2), 364-399 (B3), 453-482,503-524 (S34) */
int or_codec_unpack(int codec, const uint8_t* packed, size_t packed_len, size_t n, int8_t* out) {
  uint64_t led[4];
  int rc = or_codec_ledger(codec, n, led);
  if (rc) return rc;
  if (packed_len != (size_t)led[0]) return OR_ERR_LENGTH;
  if (codec == OR_CODEC_D2) {
    size_t physical = packed_len * 4, w = 0;
    for (size_t i = 0; i < physical; i++) {
      unsigned code = (packed[i / 4] >> (2 * (i % 4))) & 3u;
      if (code == 3u) return OR_ERR_INVALID_CODE;
      if (i >= n) { if (code != 1u) return OR_ERR_PADDING; continue; }
      out[w++] = (int8_t)((int)code - 1);
    }
  } else if (codec == OR_CODEC_B3) {
    size_t w = 0;
    for (size_t b = 0; b < packed_len; b++) {
      unsigned code = packed[b];
      if (code >= 243u) return OR_ERR_INVALID_CODE;
      for (unsigned s = 0; s < 5; s++) {
        unsigned digit = code % 3u;
        code /= 3u;
        size_t ti = b * 5 + s;
        if (ti >= n) { if (digit != 1u) return OR_ERR_PADDING; continue; }
        out[w++] = (int8_t)((int)digit - 1);
      }
    }
  } else {
    if (led[2]) {
      unsigned used = 8u - (unsigned)led[2];
      if (packed[packed_len - 1] & (uint8_t)(0xffu << used)) return OR_ERR_PADDING;
    }
    size_t w = 0;
    for (size_t g = 0; g < n / 4; g++) {
      size_t bit = g * 5, byte = bit / 8;
      unsigned shift = (unsigned)(bit % 8);
      unsigned word = packed[byte] | ((byte + 1 < packed_len ? (unsigned)packed[byte + 1] : 0u) << 8);
      unsigned code = (word >> shift) & 31u;
      unsigned zero_index = code & 3u, sign_index = 0;
      for (unsigned s = 0; s < 4; s++) {
        if (s == zero_index) { out[w++] = 0; continue; }
        out[w++] = (code & (1u << (2 + sign_index))) ? 1 : -1;
        sign_index++;
      }
    }
  }
  return OR_OK;
}

/* stored_trit_count: salt_v2_package.rs:2458-2467 */
static size_t stored_trits(int codec, size_t logical_len) {
  return codec == OR_CODEC_S34 ? (logical_len + 3) / 4 * 4 : logical_len;
}

size_t or_plane_payload_bytes(int codec, size_t logical_len) {
  uint64_t led[4];
  if (or_codec_ledger(codec, stored_trits(codec, logical_len), led)) return 0;
  return (size_t)led[0];
}

/* pack_salt_v2_plane + canonical_s34_trits: salt_v2_package.rs:2420-2456 */
long or_plane_pack(int codec, const int8_t* trits, size_t logical_len, uint8_t* out, size_t out_cap) {
  if (codec != OR_CODEC_S34) return or_codec_pack(codec, trits, logical_len, out, out_cap);
  int8_t canonical[OR_TILE + 4];
  if (logical_len > OR_TILE) return OR_ERR_PLANE_LEN;
  size_t stored = stored_trits(codec, logical_len);
  memcpy(canonical, trits, logical_len);
  size_t full = logical_len / 4 * 4, len = logical_len;
  if (full != logical_len) {
    int zeros = 0;
    for (size_t i = full; i < logical_len; i++) zeros += trits[i] == 0;
    if (zeros > 1) return OR_ERR_S34_SHAPE;
    if (zeros == 0) canonical[len++] = 0;
    while (len < stored) canonical[len++] = -1;
  }
  return or_codec_pack(codec, canonical, stored, out, out_cap);
}

/* unpack_salt_v2_plane_into + validate_s34_shape_padding: salt_v2_package.rs:2360-2418 */
int or_plane_unpack(int codec, const uint8_t* packed, size_t packed_len, size_t logical_len,
                    int8_t* out) {
  if (codec != OR_CODEC_S34) return or_codec_unpack(codec, packed, packed_len, logical_len, out);
  int8_t decoded[OR_TILE + 4];
  if (logical_len > OR_TILE) return OR_ERR_PLANE_LEN;
  size_t stored = stored_trits(codec, logical_len);
  int rc = or_codec_unpack(codec, packed, packed_len, stored, decoded);
  if (rc) return rc;
  if (stored != logical_len) {
    size_t start = logical_len / 4 * 4, pad = logical_len;
    int zeros = 0;
    for (size_t i = start; i < logical_len; i++) zeros += decoded[i] == 0;
    if (zeros > 1) return OR_ERR_S34_SHAPE;
    if (zeros == 0) { if (decoded[pad] != 0) return OR_ERR_PADDING; pad++; }
    for (size_t i = pad; i < stored; i++) if (decoded[i] != -1) return OR_ERR_PADDING;
  }
  memcpy(out, decoded, logical_len);
  return OR_OK;
}

/* ------------------------------------------------------------------ semantic tensor */

static size_t tile_len(uint64_t coeffs, uint64_t tile) {
  uint64_t rest = coeffs - tile * OR_TILE;
  return (size_t)(rest < OR_TILE ? rest : OR_TILE);
}
static const int8_t* t_trits(const or_tensor* t, uint64_t tile, unsigned p) {
  return t->trits + (tile * 3 + p) * OR_TILE;
}
static const uint16_t* t_scales(const or_tensor* t, uint64_t tile, unsigned p) {
  return t->scales + (tile * 3 + p) * 4;
}

/* SaltV2Plane::new_with_scale_group_size (salt_v2_package.rs:130-187), SaltV2Tile::new
 * (:222-251), SaltV2Tensor::new_with_layout (:582-641). */
int or_tensor_validate(const or_tensor* t) {
  if (t->group != 64 && t->group != 128) return OR_ERR_GROUP_SIZE;
  if (t->rows == 0 || t->cols == 0) return OR_ERR_SHAPE;
  uint64_t coeffs = t->rows * t->cols;
  if (t->tiles != (coeffs + OR_TILE - 1) / OR_TILE) return OR_ERR_SHAPE;
  for (uint64_t tile = 0; tile < t->tiles; tile++) {
    unsigned planes = t->plane_count[tile];
    if (planes < 1 || planes > OR_MAX_PLANES) return OR_ERR_PLANE_COUNT;
    size_t len = tile_len(coeffs, tile);
    size_t groups = (len + t->group - 1) / t->group;
    for (unsigned p = 0; p < planes; p++) {
      const int8_t* tr = t_trits(t, tile, p);
      const uint16_t* sc = t_scales(t, tile, p);
      for (size_t i = 0; i < len; i++)
        if (tr[i] < -1 || tr[i] > 1) return OR_ERR_TRIT;
      for (size_t g = 0; g < groups; g++) {
        float v = or_f16_to_f32(sc[g]);
        if (!isfinite(v)) return OR_ERR_SCALE_NONFINITE;
        if (sc[g] & 0x8000u) return OR_ERR_SCALE_NEGATIVE;
        if (sc[g] == 0) {
          size_t end = (g + 1) * t->group < len ? (g + 1) * t->group : len;
          for (size_t i = g * t->group; i < end; i++)
            if (tr[i] != 0) return OR_ERR_SCALE_ZERO_NONZERO_GROUP;
        }
      }
    }
  }
  return OR_OK;
}

/* ------------------------------------------------------------------ resident layout */
/* SaltV2IndexedRuntimeLedger::for_tensor: salt_v2_package.rs:889-962 */
int or_resident_plan(const or_tensor* t, int codec, or_resident_sizes* out) {
  uint64_t coeffs = t->rows * t->cols;
  memset(out, 0, sizeof *out);
  out->tiles = t->tiles;
  for (uint64_t tile = 0; tile < t->tiles; tile++) {
    unsigned planes = t->plane_count[tile];
    size_t len = tile_len(coeffs, tile);
    out->present_planes += planes;
    out->payload_bytes += (uint64_t)planes * or_plane_payload_bytes(codec, len);
    out->scale_bytes += (uint64_t)planes * ((len + t->group - 1) / t->group) * 2;
  }
  uint64_t map_bits = t->tiles * 2;
  out->map_bytes = map_bits / 8;
  uint64_t prefixes = (t->tiles ? t->tiles - 1 : 0) / OR_RANK_STRIDE;
  out->rank_prefix_bytes = prefixes * 4;
  if (out->tiles > 0xffffffffull || out->present_planes > 0xffffffffull ||
      out->payload_bytes > 0xffffffffull || out->scale_bytes / 2 > 0xffffffffull)
    return OR_ERR_LENGTH;
  return OR_OK;
}

/* upload_salt_v2: crates/tritium-cuda/src/cuda/backend.rs:7544-7611 */
int or_resident_build(const or_tensor* t, int codec, uint8_t* payload, uint16_t* scales,
                      uint8_t* index_metadata, uint32_t* terminal_map_value) {
  or_resident_sizes plan;
  int rc = or_resident_plan(t, codec, &plan);
  if (rc) return rc;
  uint64_t coeffs = t->rows * t->cols;
  memset(index_metadata, 0, (size_t)(plan.map_bytes + plan.rank_prefix_bytes));
  uint32_t terminal = 0;
  uint64_t planes_before = 0, pay = 0, sc = 0, prefix = 0;
  for (uint64_t tile = 0; tile < t->tiles; tile++) {
    if (tile != 0 && tile % OR_RANK_STRIDE == 0) {
      uint32_t v = (uint32_t)planes_before;
      uint8_t* dst = index_metadata + plan.map_bytes + prefix * 4;
      dst[0] = (uint8_t)v; dst[1] = (uint8_t)(v >> 8); dst[2] = (uint8_t)(v >> 16); dst[3] = (uint8_t)(v >> 24);
      prefix++;
    }
    unsigned planes = t->plane_count[tile];
    unsigned code = planes - 1;
    uint64_t bit = tile * 2;
    if (bit < plan.map_bytes * 8) index_metadata[bit / 8] |= (uint8_t)(code << (bit % 8));
    else terminal |= code << (bit - plan.map_bytes * 8);
    size_t len = tile_len(coeffs, tile);
    size_t groups = (len + t->group - 1) / t->group;
    for (unsigned p = 0; p < planes; p++) {
      long n = or_plane_pack(codec, t_trits(t, tile, p), len, payload + pay, 64);
      if (n < 0) return (int)n;
      pay += (uint64_t)n;
      memcpy(scales + sc, t_scales(t, tile, p), groups * 2);
      sc += groups;
    }
    planes_before += planes;
  }
  *terminal_map_value = terminal;
  return OR_OK;
}

/* ------------------------------------------------------------------ package bytes */

static void put16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
static void put32(uint8_t* p, uint32_t v) { for (int i = 0; i < 4; i++) p[i] = (uint8_t)(v >> (8 * i)); }
static void put64(uint8_t* p, uint64_t v) { for (int i = 0; i < 8; i++) p[i] = (uint8_t)(v >> (8 * i)); }
static uint16_t get16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static uint32_t get32(const uint8_t* p) { uint32_t v = 0; for (int i = 0; i < 4; i++) v |= (uint32_t)p[i] << (8 * i); return v; }
static uint64_t get64(const uint8_t* p) { uint64_t v = 0; for (int i = 0; i < 8; i++) v |= (uint64_t)p[i] << (8 * i); return v; }

/* plane_count_map_value: salt_v2_package.rs:2680-2687 */
static unsigned presence_bits(unsigned planes) { return planes == 1 ? 0u : planes == 2 ? 1u : 3u; }

/* write_salt_v2_package: salt_v2_package.rs:1526-1668; encode_tensor :1980-2066;
 * encode_presence_maps :2478-2558; push_layout :2828-2858 */
long or_package_write(int codec, const or_named_tensor* ts, size_t count, uint8_t* out, size_t cap) {
  if (count == 0 || count >= (1u << 26)) return OR_ERR_SHAPE;
  if (codec < OR_CODEC_D2 || codec > OR_CODEC_S34) return OR_ERR_CODEC;
  uint16_t version = 1;
  uint64_t full_tiles = 0, total = 24;
  for (size_t i = 0; i < count; i++) {
    const or_tensor* t = &ts[i].tensor;
    int rc = or_tensor_validate(t);
    if (rc) return rc;
    if (!ts[i].name || !ts[i].name[0]) return OR_ERR_NAME;
    for (size_t j = 0; j < i; j++)
      if (strcmp(ts[i].name, ts[j].name) == 0) return OR_ERR_DUPLICATE_NAME;
    if (t->group != 128) version = 2;
    or_resident_sizes plan;
    rc = or_resident_plan(t, codec, &plan);
    if (rc && rc != OR_ERR_LENGTH) return rc;
    full_tiles += (t->rows * t->cols) / OR_TILE;
    total += 64 + strlen(ts[i].name) + (t->rank == 1 ? 8 : 16) + plan.payload_bytes + plan.scale_bytes;
    if (t->rank == 1 && t->rows != 1) return OR_ERR_SHAPE;
  }
  uint64_t map_bytes = full_tiles * 2 / 8;
  total += map_bytes;
  uint64_t padded = (total + 7) / 8 * 8;
  if (!out) return (long)padded;
  if (cap < padded) return OR_ERR_LENGTH;
  memset(out, 0, (size_t)padded);

  /* global presence map over full tiles; trailing bits ride in the tensor-count word */
  uint8_t* map = (uint8_t*)calloc((size_t)map_bytes + 1, 1);
  if (!map) return OR_ERR_ALLOC;
  unsigned embedded = 0;
  uint64_t gt = 0, complete_bits = map_bytes * 8;
  for (size_t i = 0; i < count; i++) {
    const or_tensor* t = &ts[i].tensor;
    uint64_t tf = (t->rows * t->cols) / OR_TILE;
    for (uint64_t tile = 0; tile < tf; tile++, gt++) {
      unsigned bits = presence_bits(t->plane_count[tile]);
      for (unsigned b = 0; b < 2; b++) {
        if (!(bits & (1u << b))) continue;
        uint64_t bit = gt * 2 + b;
        if (bit < complete_bits) map[bit / 8] |= (uint8_t)(1u << (bit % 8));
        else embedded |= 1u << (bit - complete_bits);
      }
    }
  }

  uint8_t* p = out;
  memcpy(p, "TSLT2PKG", 8); p += 8;
  put16(p, version); p += 2;
  *p++ = (uint8_t)codec;
  *p++ = 0;
  put32(p, (uint32_t)count | (embedded << 26)); p += 4;
  put64(p, padded); p += 8;
  for (size_t i = 0; i < count; i++) {
    const or_tensor* t = &ts[i].tensor;
    uint64_t coeffs = t->rows * t->cols;
    or_resident_sizes plan;
    or_resident_plan(t, codec, &plan);
    size_t name_len = strlen(ts[i].name);
    unsigned ragged = coeffs % OR_TILE ? presence_bits(t->plane_count[t->tiles - 1]) : 0u;
    put32(p, (uint32_t)name_len); p += 4;
    put32(p, t->rank == 1 ? 1u : 2u); p += 4;
    put64(p, coeffs); p += 8;
    put64(p, t->tiles | ((uint64_t)ragged << 62)); p += 8;
    put64(p, plan.payload_bytes); p += 8;
    put64(p, plan.scale_bytes); p += 8;
    *p++ = 0;                               /* transform tag: None */
    *p++ = (uint8_t)(t->group == 64 ? 1 : 0); /* scale geometry */
    p += 6;                                 /* reserved zero */
    put64(p, 0); p += 8;                    /* seed */
    put64(p, 0); p += 8;                    /* domain */
    memcpy(p, ts[i].name, name_len); p += name_len;
    if (t->rank != 1) { put64(p, t->rows); p += 8; }
    put64(p, t->cols); p += 8;
    uint8_t* sc = p + plan.payload_bytes;
    for (uint64_t tile = 0; tile < t->tiles; tile++) {
      size_t len = tile_len(coeffs, tile);
      size_t groups = (len + t->group - 1) / t->group;
      for (unsigned pl = 0; pl < t->plane_count[tile]; pl++) {
        long n = or_plane_pack(codec, t_trits(t, tile, pl), len, p, 64);
        if (n < 0) { free(map); return n; }
        p += n;
        for (size_t g = 0; g < groups; g++) { put16(sc, t_scales(t, tile, pl)[g]); sc += 2; }
      }
    }
    p = sc;
  }
  memcpy(p, map, (size_t)map_bytes);
  free(map);
  return (long)padded;
}

typedef struct {
  uint64_t rows, cols, coeffs, tiles, full_tiles;
  uint32_t group, rank;
  int ragged_planes;      /* 0 = none */
  uint64_t payload_len, scales_len;
  const uint8_t *name, *payload, *scales;
  uint32_t name_len;
  uint64_t first_full_tile; /* offset into the global map */
} raw_tensor;

typedef struct {
  int codec;
  uint16_t version;
  uint32_t count;
  unsigned embedded;
  const uint8_t* map;
  uint64_t map_bytes, total_full_tiles;
  raw_tensor* tensors;
} parsed_package;

static unsigned map_planes(const parsed_package* pk, uint64_t global_tile, int* nested_ok) {
  unsigned bits = 0;
  for (unsigned b = 0; b < 2; b++) {
    uint64_t bit = global_tile * 2 + b;
    unsigned v = bit < pk->map_bytes * 8 ? (pk->map[bit / 8] >> (bit % 8)) & 1u
                                          : (pk->embedded >> (bit - pk->map_bytes * 8)) & 1u;
    bits |= v << b;
  }
  if (bits == 2u) *nested_ok = 0;
  return 1 + (bits & 1u) + ((bits >> 1) & 1u);
}

static unsigned raw_tile_planes(const parsed_package* pk, const raw_tensor* r, uint64_t tile, int* ok) {
  if (tile < r->full_tiles) return map_planes(pk, r->first_full_tile + tile, ok);
  return (unsigned)r->ragged_planes;
}

/* read_salt_v2_package: salt_v2_package.rs:1679-1978 (header, per-tensor, map, padding rules) */
static int parse_package(const uint8_t* b, size_t len, parsed_package* pk) {
  memset(pk, 0, sizeof *pk);
  size_t pos = 0;
#define NEED(n) do { if (len - pos < (size_t)(n)) return OR_ERR_TRUNCATED; } while (0)
  NEED(8);
  if (memcmp(b, "TSLT2PKG", 8)) return OR_ERR_MAGIC;
  pos = 8;
  NEED(2); pk->version = get16(b + pos); pos += 2;
  if (pk->version != 1 && pk->version != 2) return OR_ERR_VERSION;
  NEED(1); pk->codec = b[pos++];
  if (pk->codec < OR_CODEC_D2 || pk->codec > OR_CODEC_S34) return OR_ERR_CODEC;
  NEED(1); if (b[pos++] != 0) return OR_ERR_FLAGS;
  NEED(4); uint32_t word = get32(b + pos); pos += 4;
  pk->count = word & ((1u << 26) - 1);
  pk->embedded = word >> 26;
  NEED(8); uint64_t declared_total = get64(b + pos); pos += 8;
  if (declared_total != len) return OR_ERR_LENGTH;
  if (pk->count == 0) return OR_ERR_SHAPE;
  if (pk->count > (len - pos) / 64) return OR_ERR_TRUNCATED;
  pk->tensors = (raw_tensor*)calloc(pk->count, sizeof(raw_tensor));
  if (!pk->tensors) return OR_ERR_ALLOC;
  int any_g64 = 0;
  uint64_t full_total = 0;
  for (uint32_t i = 0; i < pk->count; i++) {
    raw_tensor* r = &pk->tensors[i];
    NEED(64);
    r->name_len = get32(b + pos); r->rank = get32(b + pos + 4);
    uint64_t declared_coeffs = get64(b + pos + 8);
    uint64_t tile_word = get64(b + pos + 16);
    r->payload_len = get64(b + pos + 24);
    r->scales_len = get64(b + pos + 32);
    uint8_t tag = b[pos + 40], geom = b[pos + 41];
    for (int z = 0; z < 6; z++) if (b[pos + 42 + z]) return OR_ERR_TRANSFORM;
    uint64_t seed = get64(b + pos + 48), domain = get64(b + pos + 56);
    pos += 64;
    if (pk->version == 1) { if (geom != 0) return OR_ERR_TRANSFORM; r->group = 128; }
    else { if (geom > 1) return OR_ERR_GROUP_SIZE; r->group = geom ? 64 : 128; }
    if (tag == 0) { if (seed || domain) return OR_ERR_TRANSFORM; }
    else return OR_ERR_TRANSFORM; /* SignedRht: not executable by the oracle */
    if (r->group == 64) any_g64 = 1;
    NEED(r->name_len);
    r->name = b + pos; pos += r->name_len;
    if (r->name_len == 0) return OR_ERR_NAME;
    for (uint32_t j = 0; j < i; j++)
      if (pk->tensors[j].name_len == r->name_len && !memcmp(pk->tensors[j].name, r->name, r->name_len))
        return OR_ERR_DUPLICATE_NAME;
    if (r->rank == 0 || r->rank > 2) return OR_ERR_SHAPE;
    NEED((size_t)r->rank * 8);
    if (r->rank == 1) { r->rows = 1; r->cols = get64(b + pos); }
    else { r->rows = get64(b + pos); r->cols = get64(b + pos + 8); }
    pos += (size_t)r->rank * 8;
    if (r->rows == 0 || r->cols == 0) return OR_ERR_SHAPE;
    r->coeffs = r->rows * r->cols;
    if (declared_coeffs != r->coeffs) return OR_ERR_LENGTH;
    r->tiles = (r->coeffs + OR_TILE - 1) / OR_TILE;
    if ((tile_word & ((1ull << 62) - 1)) != r->tiles) return OR_ERR_LENGTH;
    unsigned ragged_value = (unsigned)(tile_word >> 62);
    r->full_tiles = r->coeffs / OR_TILE;
    if (r->coeffs % OR_TILE == 0) {
      if (ragged_value) return OR_ERR_PADDING;
      r->ragged_planes = 0;
    } else {
      if (ragged_value == 2u) return OR_ERR_NON_NESTED_MAP;
      r->ragged_planes = 1 + (int)(ragged_value & 1u) + (int)(ragged_value >> 1);
    }
    if (r->payload_len + r->scales_len > len - pos) return OR_ERR_TRUNCATED;
    r->payload = b + pos; pos += (size_t)r->payload_len;
    r->scales = b + pos; pos += (size_t)r->scales_len;
    r->first_full_tile = full_total;
    full_total += r->full_tiles;
  }
  if (pk->version != (any_g64 ? 2 : 1)) return OR_ERR_VERSION;
  pk->total_full_tiles = full_total;
  pk->map_bytes = full_total * 2 / 8;
  NEED(pk->map_bytes);
  pk->map = b + pos; pos += (size_t)pk->map_bytes;
  unsigned embedded_bits = (unsigned)(full_total * 2 % 8);
  if (embedded_bits < 6 && (pk->embedded >> embedded_bits)) return OR_ERR_PADDING;
  size_t pad = (8 - pos % 8) % 8;
  if (len - pos != pad) return OR_ERR_TRAILING;
  for (size_t i = 0; i < pad; i++) if (b[pos + i]) return OR_ERR_PADDING;
  int nested = 1;
  for (uint64_t g = 0; g < full_total; g++) map_planes(pk, g, &nested);
  if (!nested) return OR_ERR_NON_NESTED_MAP;
  /* declared section sizes are re-derived, never trusted (:1921-1926) */
  for (uint32_t i = 0; i < pk->count; i++) {
    raw_tensor* r = &pk->tensors[i];
    uint64_t pay = 0, sc = 0;
    for (uint64_t tile = 0; tile < r->tiles; tile++) {
      unsigned planes = raw_tile_planes(pk, r, tile, &nested);
      size_t tl = tile_len(r->coeffs, tile);
      pay += (uint64_t)planes * or_plane_payload_bytes(pk->codec, tl);
      sc += (uint64_t)planes * ((tl + r->group - 1) / r->group) * 2;
    }
    if (pay != r->payload_len || sc != r->scales_len) return OR_ERR_LENGTH;
  }
#undef NEED
  return OR_OK;
}

int or_package_probe(const uint8_t* bytes, size_t len, int* codec, uint32_t* tensor_count) {
  parsed_package pk;
  int rc = parse_package(bytes, len, &pk);
  if (rc == OR_OK) { *codec = pk.codec; *tensor_count = pk.count; }
  free(pk.tensors);
  return rc;
}

int or_package_tensor_info(const uint8_t* bytes, size_t len, uint32_t index, uint64_t* rows,
                           uint64_t* cols, uint32_t* group, uint64_t* tiles, uint32_t* rank,
                           char* name, size_t name_cap) {
  parsed_package pk;
  int rc = parse_package(bytes, len, &pk);
  if (rc == OR_OK) {
    if (index >= pk.count) rc = OR_ERR_SHAPE;
    else {
      raw_tensor* r = &pk.tensors[index];
      *rows = r->rows; *cols = r->cols; *group = r->group; *tiles = r->tiles; *rank = r->rank;
      if (name && name_cap) {
        size_t n = r->name_len < name_cap - 1 ? r->name_len : name_cap - 1;
        memcpy(name, r->name, n); name[n] = 0;
      }
    }
  }
  free(pk.tensors);
  return rc;
}

int or_package_read_tensor(const uint8_t* bytes, size_t len, uint32_t index, uint8_t* plane_count,
                           int8_t* trits, uint16_t* scales) {
  parsed_package pk;
  int rc = parse_package(bytes, len, &pk);
  if (rc) { free(pk.tensors); return rc; }
  /* every tensor is decoded so that a defect anywhere fails the read, as the reference does */
  for (uint32_t i = 0; i < pk.count && rc == OR_OK; i++) {
    raw_tensor* r = &pk.tensors[i];
    const uint8_t* pay = r->payload;
    const uint8_t* sc = r->scales;
    int ok = 1;
    for (uint64_t tile = 0; tile < r->tiles && rc == OR_OK; tile++) {
      unsigned planes = raw_tile_planes(&pk, r, tile, &ok);
      size_t tl = tile_len(r->coeffs, tile);
      size_t pb = or_plane_payload_bytes(pk.codec, tl);
      size_t groups = (tl + r->group - 1) / r->group;
      if (i == index) plane_count[tile] = (uint8_t)planes;
      for (unsigned p = 0; p < planes; p++) {
        int8_t tmp[OR_TILE];
        rc = or_plane_unpack(pk.codec, pay, pb, tl, tmp);
        if (rc) break;
        uint16_t s4[4] = {0, 0, 0, 0};
        for (size_t g = 0; g < groups; g++) s4[g] = get16(sc + 2 * g);
        /* plane validation: same rules as the semantic constructor */
        for (size_t g = 0; g < groups && rc == OR_OK; g++) {
          float v = or_f16_to_f32(s4[g]);
          if (!isfinite(v)) rc = OR_ERR_SCALE_NONFINITE;
          else if (s4[g] & 0x8000u) rc = OR_ERR_SCALE_NEGATIVE;
          else if (s4[g] == 0) {
            size_t end = (g + 1) * r->group < tl ? (g + 1) * r->group : tl;
            for (size_t e = g * r->group; e < end; e++)
              if (tmp[e]) { rc = OR_ERR_SCALE_ZERO_NONZERO_GROUP; break; }
          }
        }
        if (rc) break;
        if (i == index) {
          int8_t* dst = trits + (tile * 3 + p) * OR_TILE;
          memset(dst, 0, OR_TILE);
          memcpy(dst, tmp, tl);
          memcpy(scales + (tile * 3 + p) * 4, s4, sizeof s4);
        }
        pay += pb; sc += groups * 2;
      }
    }
  }
  if (rc == OR_OK && index >= pk.count) rc = OR_ERR_SHAPE;
  free(pk.tensors);
  return rc;
}

/* ------------------------------------------------------------------ the operator */

/* salt_v2_matvec_into, one row: crates/tritium-cpu/src/salt_v2.rs:341-420.
 * `ints` (optional) receives each group accumulator as an integer, laid out
 * [segment_index_in_row][3]; used only when the activation is integer valued. */
static int row_dot(const or_tensor* t, uint64_t row, const float* x, float* out, or_fail* fail,
                   int32_t* ints) {
  uint64_t cols = t->cols, row_base = row * cols, row_end = row_base + cols;
  uint64_t coeffs = t->rows * t->cols;
  float accumulator = 0.0f;
  uint64_t c = row_base, segment = 0;
  while (c < row_end) {
    uint64_t tile = c / OR_TILE, tile_base = tile * OR_TILE;
    size_t local_start = (size_t)(c - tile_base);
    size_t tl = tile_len(coeffs, tile);
    size_t group = local_start / t->group;
    size_t group_end = (group + 1) * t->group;
    if (group_end > tl) group_end = tl;
    uint64_t seg_len = group_end - local_start;
    if (seg_len > row_end - c) seg_len = row_end - c;
    uint64_t seg_end = c + seg_len;
    uint64_t terminal_column = seg_end - row_base - 1;
    unsigned planes = t->plane_count[tile];
    for (unsigned p = 0; p < planes; p++) {
      const int8_t* tr = t_trits(t, tile, p);
      float scale = or_f16_to_f32(t_scales(t, tile, p)[group]);
      float ga = 0.0f;
      for (uint64_t cur = c; cur < seg_end; cur++) {
        uint64_t column = cur - row_base;
        int8_t trit = tr[cur - tile_base];
        if (trit == -1) ga -= x[column];
        else if (trit == 1) ga += x[column];
        if (!isfinite(ga)) { if (fail) { fail->row = row; fail->column = column; } return OR_ERR_NONFINITE_OUTPUT; }
      }
      if (ints) ints[segment * 3 + p] = (int32_t)ga;
      float contribution = ga * scale;
      if (!isfinite(contribution)) { if (fail) { fail->row = row; fail->column = terminal_column; } return OR_ERR_NONFINITE_OUTPUT; }
      accumulator += contribution;
      if (!isfinite(accumulator)) { if (fail) { fail->row = row; fail->column = terminal_column; } return OR_ERR_NONFINITE_OUTPUT; }
    }
    c = seg_end;
    segment++;
  }
  *out = accumulator;
  return OR_OK;
}

/* validate_activation: crates/tritium-cpu/src/salt_v2.rs:461-477 */
static int check_activation(const float* x, uint64_t n, or_fail* fail) {
  for (uint64_t i = 0; i < n; i++)
    if (!isfinite(x[i])) {
      if (fail) { fail->row = 0; fail->column = i; fail->bits = f32_bits(x[i]); }
      return OR_ERR_NONFINITE_ACTIVATION;
    }
  return OR_OK;
}

int or_matvec(const or_tensor* t, const float* x, float* y, or_fail* fail) {
  int rc = check_activation(x, t->cols, fail);
  if (rc) return rc;
  for (uint64_t row = 0; row < t->rows; row++) {
    float v;
    rc = row_dot(t, row, x, &v, fail, NULL);
    if (rc) return rc;
    y[row] = v;
  }
  return OR_OK;
}

typedef struct {
  const or_tensor* t; const float* x; float* y; uint64_t m, row0, row1; int failed;
} mt_job;

static void* mt_worker(void* arg) {
  mt_job* j = (mt_job*)arg;
  for (uint64_t row = j->row0; row < j->row1; row++)
    for (uint64_t mi = 0; mi < j->m; mi++) {
      float v = 0.0f;
      if (row_dot(j->t, row, j->x + mi * j->t->cols, &v, NULL, NULL)) j->failed = 1;
      j->y[mi * j->t->rows + row] = v;
    }
  return NULL;
}

/* Rows are split into `threads` contiguous ranges (POSIX threads); per-row arithmetic is
 * row_dot, unchanged.  The reference itself is single threaded on this path. */
int or_matmul_mt(const or_tensor* t, const float* x, uint64_t m, float* y, int threads) {
  int rc = check_activation(x, m * t->cols, NULL);
  if (rc) return rc;
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  pthread_t tid[256];
  mt_job jobs[256];
  uint64_t per = (t->rows + (uint64_t)threads - 1) / (uint64_t)threads;
  int started = 0, failed = 0;
  for (int i = 0; i < threads; i++) {
    uint64_t r0 = per * (uint64_t)i, r1 = r0 + per;
    if (r0 >= t->rows) break;
    if (r1 > t->rows) r1 = t->rows;
    jobs[i] = (mt_job){t, x, y, m, r0, r1, 0};
    if (pthread_create(&tid[i], NULL, mt_worker, &jobs[i])) { mt_worker(&jobs[i]); tid[i] = 0; }
    started = i + 1;
  }
  for (int i = 0; i < started; i++) {
    if (tid[i]) pthread_join(tid[i], NULL);
    failed |= jobs[i].failed;
  }
  return failed ? OR_ERR_NONFINITE_OUTPUT : OR_OK;
}

/* Resident-arena addressing: crates/tritium-nn/src/layers/salt_v2_host.rs:389-469 */
typedef struct {
  int codec; uint32_t group; uint64_t rows, cols, coeffs, tiles;
  const uint8_t* payload; const uint16_t* scales; const uint8_t* meta;
  uint64_t map_bytes; uint32_t terminal;
} packed_view;

static unsigned pv_planes(const packed_view* v, uint64_t tile) {
  uint64_t bit = tile * 2;
  unsigned code = bit < v->map_bytes * 8 ? (v->meta[bit / 8] >> (bit % 8)) & 3u
                                         : (v->terminal >> (bit - v->map_bytes * 8)) & 3u;
  return code + 1;
}
static uint64_t pv_rank(const packed_view* v, uint64_t tile) {
  uint64_t block = tile / OR_RANK_STRIDE, rank = 0;
  if (block) rank = get32(v->meta + v->map_bytes + (block - 1) * 4);
  for (uint64_t cur = block * OR_RANK_STRIDE; cur < tile; cur++) rank += pv_planes(v, cur);
  return rank;
}

int or_forward_packed(int codec, uint32_t group, uint64_t rows, uint64_t cols,
                      const uint8_t* payload, const uint16_t* scales, const uint8_t* meta,
                      uint64_t map_bytes, uint32_t terminal, const float* x, uint64_t m, float* y,
                      or_fail* fail) {
  packed_view v = {codec, group, rows, cols, rows * cols, (rows * cols + OR_TILE - 1) / OR_TILE,
                   payload, scales, meta, map_bytes, terminal};
  int rc = check_activation(x, m * cols, fail);
  if (rc) return rc;
  size_t full_bytes = or_plane_payload_bytes(codec, OR_TILE);
  for (uint64_t mi = 0; mi < m; mi++) {
    const float* xr = x + mi * cols;
    for (uint64_t row = 0; row < rows; row++) {
      uint64_t row_base = row * cols, row_end = row_base + cols, c = row_base;
      float accumulator = 0.0f;
      while (c < row_end) {
        uint64_t tile = c / OR_TILE, tile_base = tile * OR_TILE;
        size_t local_start = (size_t)(c - tile_base), tl = tile_len(v.coeffs, tile);
        size_t g = local_start / group, g_end = (g + 1) * group;
        if (g_end > tl) g_end = tl;
        uint64_t seg_len = g_end - local_start;
        if (seg_len > row_end - c) seg_len = row_end - c;
        uint64_t seg_end = c + seg_len, rank = pv_rank(&v, tile);
        unsigned planes = pv_planes(&v, tile);
        if (planes > OR_MAX_PLANES) return OR_ERR_PLANE_COUNT;
        size_t pb = or_plane_payload_bytes(codec, tl), sc_count = (tl + group - 1) / group;
        for (unsigned p = 0; p < planes; p++) {
          int8_t decoded[OR_TILE];
          rc = or_plane_unpack(codec, payload + rank * full_bytes + p * pb, pb, tl, decoded);
          if (rc) return rc;
          float scale = or_f16_to_f32(scales[rank * (OR_TILE / group) + p * sc_count + g]);
          float ga = 0.0f;
          for (uint64_t cur = c; cur < seg_end; cur++) {
            int8_t trit = decoded[cur - tile_base];
            if (trit == -1) ga -= xr[cur - row_base];
            else if (trit == 1) ga += xr[cur - row_base];
            if (!isfinite(ga)) { if (fail) { fail->row = row; fail->column = cur - row_base; } return OR_ERR_NONFINITE_OUTPUT; }
          }
          float contribution = ga * scale;
          if (!isfinite(contribution)) { if (fail) { fail->row = row; fail->column = seg_end - row_base - 1; } return OR_ERR_NONFINITE_OUTPUT; }
          accumulator += contribution;
          if (!isfinite(accumulator)) { if (fail) { fail->row = row; fail->column = seg_end - row_base - 1; } return OR_ERR_NONFINITE_OUTPUT; }
        }
        c = seg_end;
      }
      y[mi * rows + row] = accumulator;
    }
  }
  return OR_OK;
}

/* reconstruct_row / gather_rows: salt_v2_host.rs:277-294,356-387 */
int or_gather_rows(const or_tensor* t, const uint32_t* rows, uint64_t count, float* out) {
  uint64_t cols = t->cols, coeffs = t->rows * t->cols;
  for (uint64_t i = 0; i < count; i++) if (rows[i] >= t->rows) return OR_ERR_SHAPE;
  memset(out, 0, (size_t)(count * cols) * sizeof(float));
  for (uint64_t i = 0; i < count; i++) {
    uint64_t base = (uint64_t)rows[i] * cols;
    for (uint64_t col = 0; col < cols; col++) {
      uint64_t c = base + col, tile = c / OR_TILE;
      size_t local = (size_t)(c % OR_TILE);
      (void)coeffs;
      for (unsigned p = 0; p < t->plane_count[tile]; p++)
        out[i * cols + col] += (float)t_trits(t, tile, p)[local] *
                               or_f16_to_f32(t_scales(t, tile, p)[local / t->group]);
    }
  }
  return OR_OK;
}

/* ------------------------------------------------------------------ A8 */
/* quantize_act_int8: crates/tritium-spec/src/lib.rs:351-378 */
void or_quantize_act_int8(const float* act, uint64_t m, uint64_t k, float* q, float* scale) {
  for (uint64_t r = 0; r < m; r++) {
    const float* row = act + r * k;
    float gamma = 0.0f;
    for (uint64_t i = 0; i < k; i++) { float a = fabsf(row[i]); if (a > gamma) gamma = a; }
    float* out = q + r * k;
    if (gamma == 0.0f) {
      for (uint64_t i = 0; i < k; i++) out[i] = 0.0f;
      scale[r] = 0.0f;
      continue;
    }
    float s = 127.0f / gamma;
    for (uint64_t i = 0; i < k; i++) {
      float v = nearbyintf(row[i] * s); /* round half to even under the default rounding mode */
      if (v < -128.0f) v = -128.0f;
      if (v > 127.0f) v = 127.0f;
      out[i] = v;
    }
    scale[r] = gamma / 127.0f;
  }
}

static uint64_t segments_per_row(const or_tensor* t) {
  /* number of (tile, group) segments row 0.. crosses; equal for every row only when cols is a
   * multiple of the group size, which the A8 dump requires */
  return (t->cols + t->group - 1) / t->group;
}

/* The W1.58A8 composition: quantise (lib.rs:351-378), contract with the SALT V2 order
 * (salt_v2.rs:316-423) on the integer-valued activation, fold act_scale last (lib.rs:310-316). */
int or_a8_linear(const or_tensor* t, const float* x, uint64_t m, float* y, int32_t* dump,
                 float* act_scale_out) {
  if (dump && t->cols % t->group) return OR_ERR_SHAPE;
  float* q = (float*)malloc((size_t)(m * t->cols) * sizeof(float));
  float* a = (float*)malloc((size_t)m * sizeof(float));
  if (!q || !a) { free(q); free(a); return OR_ERR_ALLOC; }
  int rc = check_activation(x, m * t->cols, NULL);
  if (rc == OR_OK) {
    or_quantize_act_int8(x, m, t->cols, q, a);
    uint64_t segs = segments_per_row(t);
    if (dump) memset(dump, 0, (size_t)(m * t->rows * segs * 3) * sizeof(int32_t));
    for (uint64_t mi = 0; mi < m && rc == OR_OK; mi++)
      for (uint64_t row = 0; row < t->rows; row++) {
        float v;
        rc = row_dot(t, row, q + mi * t->cols, &v, NULL,
                     dump ? dump + (mi * t->rows + row) * segs * 3 : NULL);
        if (rc) break;
        y[mi * t->rows + row] = v * a[mi];
      }
    if (act_scale_out) memcpy(act_scale_out, a, (size_t)m * sizeof(float));
  }
  free(q); free(a);
  return rc;
}

/* ------------------------------------------------------------------ TQ2_0 */
/* pack_tq2_0_block / pack_tq2_0_row: crates/tritium-format/src/tq2.rs:21-46, rows.rs:61-77 */
int or_tq2_pack_row(const int8_t* trits, uint64_t k, const uint16_t* block_scales, uint8_t* out) {
  uint64_t nb = (k + 255) / 256;
  for (uint64_t b = 0; b < nb; b++) {
    int8_t block[256];
    memset(block, 0, sizeof block);
    uint64_t n = k - b * 256 < 256 ? k - b * 256 : 256;
    memcpy(block, trits + b * 256, (size_t)n);
    uint8_t* o = out + b * 66;
    for (int c = 0; c < 2; c++)
      for (int mm = 0; mm < 32; mm++) {
        unsigned qv = 0;
        for (int n4 = 0; n4 < 4; n4++) {
          int8_t tv = block[c * 128 + n4 * 32 + mm];
          if (tv < -1 || tv > 1) return OR_ERR_TRIT;
          qv |= ((unsigned)(tv + 1) & 3u) << (2 * n4);
        }
        o[c * 32 + mm] = (uint8_t)qv;
      }
    put16(o + 64, block_scales[b]);
  }
  return OR_OK;
}

/* unpack_tq2_0_block: tq2.rs:52-83 */
int or_tq2_unpack_row(const uint8_t* packed, uint64_t k, int8_t* trits_out, uint16_t* scales_out) {
  uint64_t nb = (k + 255) / 256;
  for (uint64_t b = 0; b < nb; b++) {
    const uint8_t* qs = packed + b * 66;
    int8_t block[256];
    for (int c = 0; c < 2; c++)
      for (int l = 0; l < 4; l++)
        for (int mm = 0; mm < 32; mm++) {
          int qv = (qs[c * 32 + mm] >> (2 * l)) & 3;
          if (qv == 3) return OR_ERR_INVALID_CODE;
          block[c * 128 + l * 32 + mm] = (int8_t)(qv - 1);
        }
    uint64_t n = k - b * 256 < 256 ? k - b * 256 : 256;
    memcpy(trits_out + b * 256, block, (size_t)n);
    if (scales_out) scales_out[b] = get16(qs + 64);
  }
  return OR_OK;
}

/* TQ1_0 block (54 bytes = 48 qs + 4 qh + f16 scale): pack_tq1_0_block / unpack_tq1_0_block,
 * crates/tritium-format/src/tq1.rs:16-122.  Five trits per byte in ggml's fixed-point base-3 code:
 * encode = ceil(acc * 256 / 243), decode digit n = (((byte * 3^n) mod 256) * 3) >> 8. */
static uint8_t tq1_encode(unsigned acc) { return (uint8_t)((acc * 256u + 242u) / 243u); }
static int8_t tq1_decode(uint8_t byte, int n) {
  static const uint8_t pow3[6] = {1, 3, 9, 27, 81, 243};
  uint8_t q = (uint8_t)(byte * pow3[n]);
  return (int8_t)((((unsigned)q * 3u) >> 8) - 1);
}
int or_tq1_pack_row(const int8_t* trits, uint64_t k, const uint16_t* block_scales, uint8_t* out) {
  uint64_t nb = (k + 255) / 256;
  for (uint64_t b = 0; b < nb; b++) {
    int8_t blk[256];
    for (int i = 0; i < 256; i++) blk[i] = b * 256 + i < k ? trits[b * 256 + i] : 0;
    uint8_t* o = out + b * 54;
    for (int m = 0; m < 32; m++) { unsigned acc = 0; for (int n = 0; n < 5; n++) acc = acc * 3 + (unsigned)(blk[m + n * 32] + 1); o[m] = tq1_encode(acc); }
    for (int m = 0; m < 16; m++) { unsigned acc = 0; for (int n = 0; n < 5; n++) acc = acc * 3 + (unsigned)(blk[160 + m + n * 16] + 1); o[32 + m] = tq1_encode(acc); }
    for (int j = 0; j < 4; j++) { unsigned acc = 0; for (int m = 0; m < 4; m++) acc = acc * 3 + (unsigned)(blk[240 + j + m * 4] + 1); acc *= 3; o[48 + j] = tq1_encode(acc); }
    put16(o + 52, block_scales ? block_scales[b] : 0x3C00);
  }
  return OR_OK;
}
int or_tq1_unpack_row(const uint8_t* packed, uint64_t k, int8_t* trits_out, uint16_t* scales_out) {
  uint64_t nb = (k + 255) / 256;
  for (uint64_t b = 0; b < nb; b++) {
    const uint8_t* qs = packed + b * 54;
    int8_t blk[256];
    for (int n = 0; n < 5; n++) for (int m = 0; m < 32; m++) blk[n * 32 + m] = tq1_decode(qs[m], n);
    for (int n = 0; n < 5; n++) for (int m = 0; m < 16; m++) blk[160 + n * 16 + m] = tq1_decode(qs[32 + m], n);
    for (int n = 0; n < 4; n++) for (int j = 0; j < 4; j++) blk[240 + n * 4 + j] = tq1_decode(qs[48 + j], n);
    uint64_t len = k - b * 256 < 256 ? k - b * 256 : 256;
    memcpy(trits_out + b * 256, blk, (size_t)len);
    if (scales_out) scales_out[b] = get16(qs + 52);
  }
  return OR_OK;
}

/* SALT V1 multi-plane forward.  PackedSaltMatrix::row_dot with reconstruct_block over dense planes
 * (crates/tritium-nn/src/layers/packed_salt.rs:612-661): per 256-block the weights are rebuilt in
 * f32 as w[i] = sum over planes (plane order) of scale_p * trit_p[i], then acc += act[i] * w[i] in
 * ascending k.  `planes` is plane-major [t_planes][n][ceil(k/256) * 66] TQ2_0 rows whose block
 * scale carries the plane's per-block scale (kernel twin: tq2_0_add.cu:661-719). */
int or_salt_v1_matmul(const uint8_t* planes, uint32_t t_planes, uint64_t n, uint64_t k, const float* act,
                      uint64_t m, float* out) {
  uint64_t nb = (k + 255) / 256, row_bytes = nb * 66;
  for (uint64_t mi = 0; mi < m; mi++)
    for (uint64_t ni = 0; ni < n; ni++) {
      float acc = 0.0f;
      for (uint64_t b = 0; b < nb; b++) {
        float weight[256];
        for (int i = 0; i < 256; i++) weight[i] = 0.0f;
        uint64_t len = k - b * 256 < 256 ? k - b * 256 : 256;
        for (uint32_t p = 0; p < t_planes; p++) {
          const uint8_t* qs = planes + ((uint64_t)p * n + ni) * row_bytes + b * 66;
          float scale = or_f16_to_f32(get16(qs + 64));
          for (int c = 0; c < 2; c++)
            for (int l = 0; l < 4; l++)
              for (int mm = 0; mm < 32; mm++) {
                int qv = (qs[c * 32 + mm] >> (2 * l)) & 3;
                if (qv == 3) return OR_ERR_INVALID_CODE;
                int idx = c * 128 + l * 32 + mm;
                if ((uint64_t)idx < len) weight[idx] += scale * (float)(qv - 1);
              }
        }
        for (uint64_t i = 0; i < len; i++) acc += act[mi * k + b * 256 + i] * weight[i];
      }
      out[mi * n + ni] = acc;
    }
  return OR_OK;
}

/* sum_squares_canonical: crates/tritium-nn/src/ops/rmsnorm.rs:20-34 (256 slots, slot t folds
 * x[t], x[t+256], ... in ascending order; then a power-of-two tree part[t] += part[t+off]) */
float or_sum_squares_canonical(const float* x, uint64_t n) {
  float part[256];
  for (int t = 0; t < 256; t++) part[t] = 0.0f;
  for (uint64_t i = 0; i < n; i++) part[i % 256] += x[i] * x[i];
  for (int off = 128; off > 0; off >>= 1)
    for (int t = 0; t < off; t++) part[t] += part[t + off];
  return part[0];
}

/* rmsnorm / rmsnorm_zero_centered: crates/tritium-nn/src/ops/rmsnorm.rs:43-94.  One row of n
 * values; zero_centered selects the (1 + w) scale. */
void or_rmsnorm(const float* x, const float* w, float eps, int zero_centered, uint64_t n, float* out) {
  if (!n) return;
  float mean_sq = or_sum_squares_canonical(x, n) / (float)n;
  float inv = 1.0f / sqrtf(mean_sq + eps);
  for (uint64_t i = 0; i < n; i++) {
    float scale = zero_centered ? 1.0f + w[i] : w[i];
    out[i] = x[i] * inv * scale;
  }
}

/* reference_mpgemm: crates/tritium-core/src/reference.rs:25-55 */
void or_reference_mpgemm(const float* act, const int8_t* w, const float* scale_n, uint64_t m,
                         uint64_t n, uint64_t k, float* out) {
  for (uint64_t mi = 0; mi < m; mi++)
    for (uint64_t ni = 0; ni < n; ni++) {
      float acc = 0.0f;
      for (uint64_t ki = 0; ki < k; ki++) {
        int8_t tv = w[ni * k + ki];
        if (tv == 1) acc += act[mi * k + ki];
        else if (tv == -1) acc -= act[mi * k + ki];
      }
      out[mi * n + ni] = acc * scale_n[ni];
    }
}

/* TernaryBackend::mpgemm_with_act_quant default: crates/tritium-spec/src/lib.rs:266-318 */
void or_mpgemm_with_act_quant(const float* act, const int8_t* w, const float* scale_n, uint64_t m,
                              uint64_t n, uint64_t k, float* out) {
  float* q = (float*)malloc((size_t)(m * k) * sizeof(float));
  float* a = (float*)malloc((size_t)m * sizeof(float));
  if (!q || !a) { free(q); free(a); return; }
  or_quantize_act_int8(act, m, k, q, a);
  or_reference_mpgemm(q, w, scale_n, m, n, k, out);
  for (uint64_t mi = 0; mi < m; mi++)
    for (uint64_t ni = 0; ni < n; ni++) out[mi * n + ni] *= a[mi];
  free(q); free(a);
}

/* ------------------------------------------------------------------ conformance PRNG */
/* XorShift64: crates/tritium-testkit/src/generate.rs:18-56 */
void or_xs_seed(or_xorshift* r, uint64_t seed) { r->state = seed | 1; }
uint64_t or_xs_next(or_xorshift* r) {
  uint64_t x = r->state;
  x ^= x << 13; x ^= x >> 7; x ^= x << 17;
  r->state = x;
  return x;
}
uint64_t or_xs_below(or_xorshift* r, uint64_t n) { return or_xs_next(r) % n; }
float or_xs_activation(or_xorshift* r) { return ((float)or_xs_below(r, 2000) - 1000.0f) / 100.0f; }
float or_xs_scale(or_xorshift* r) { return ((float)or_xs_below(r, 200) + 1.0f) / 100.0f; }
int8_t or_xs_trit(or_xorshift* r) { return (int8_t)((int)or_xs_below(r, 3) - 1); }
