// Host-side byte layouts of the packed ternary artifact.
//
// Layout facts implemented here (reference: crates/tritium-format/src/salt_v2.rs and
// src/salt_v2_package.rs):
//   D2   4 trits per byte, 2-bit code = trit+1, slot 0 in the low bits, tail slots hold code 01.
//   B3   5 trits per byte, byte = sum (trit_i+1)*3^i, byte < 243, tail digits are 1.
//   S34  one 5-bit code per 4 trits (2 bits: position of the single zero, 3 bits: signs),
//        little-endian bit stream, zero bit padding; a ragged final tile is completed with
//        (0 if it has no zero yet) then -1.
//   A tensor is cut every 256 coefficients of its flattened row-major index into tiles of 1..3
//   planes; each plane carries ceil(len/group) f16 scales (finite, non-negative, zero only over
//   an all-zero group).  The resident arenas are: payload (tile-major, then plane), scales (same
//   order), a 2-bit-per-tile map holding planes-1 whose last partial byte rides in a scalar, and
//   one u32 cumulative plane count per 256 tiles after the first.
#include "tb_format.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace tbf {

Err invalid(const std::string& m) { return Err{5, m}; }
Err shape(const std::string& m) { return Err{2, m}; }

// ---------------------------------------------------------------- f16
uint16_t f32_to_f16(float v) {
  uint32_t x;
  std::memcpy(&x, &v, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp = int32_t((x >> 23) & 0xff) - 112;  // rebias 127 -> 15
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return uint16_t(sign | 0x7c00u | (man ? 0x200u | (man >> 13) : 0));
  if (exp >= 31) return uint16_t(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return uint16_t(sign);
    man |= 0x800000u;
    const uint32_t drop = uint32_t(14 - exp);
    uint32_t keep = man >> drop;
    const uint32_t rest = man & ((1u << drop) - 1), half = 1u << (drop - 1);
    keep += (rest > half) || (rest == half && (keep & 1u));
    return uint16_t(sign | keep);
  }
  uint32_t out = sign | (uint32_t(exp) << 10) | (man >> 13);
  const uint32_t rest = man & 0x1fffu;
  out += (rest > 0x1000u) || (rest == 0x1000u && (out & 1u));
  return uint16_t(out);
}

float f16_to_f32(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, bits;
  if (exp == 0) {
    if (!man) bits = sign;
    else {
      int shift = 0;
      while (!(man & 0x400u)) { man <<= 1; ++shift; }
      bits = sign | (uint32_t(113 - shift) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
  else bits = sign | ((exp + 112) << 23) | (man << 13);
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// ---------------------------------------------------------------- codecs
namespace {

// byte -> five digits, built once.
struct B3Table {
  uint8_t digit[243][5];
  B3Table() {
    for (int b = 0; b < 243; ++b) {
      int v = b;
      for (int i = 0; i < 5; ++i) { digit[b][i] = uint8_t(v % 3); v /= 3; }
    }
  }
};
const B3Table& b3_table() { static const B3Table t; return t; }

inline size_t stored_len(int codec, size_t logical) { return codec == kS34 ? (logical + 3) / 4 * 4 : logical; }

}  // namespace

size_t codec_bytes(int codec, size_t n) {
  switch (codec) {
    case kD2: return (n + 3) / 4;
    case kB3: return (n + 4) / 5;
    case kS34: return (n / 4 * 5 + 7) / 8;
    default: return 0;
  }
}
size_t plane_bytes(int codec, size_t logical_len) { return codec_bytes(codec, stored_len(codec, logical_len)); }

Err pack(int codec, const int8_t* t, size_t n, uint8_t* out) {
  for (size_t i = 0; i < n; ++i)
    if (t[i] < -1 || t[i] > 1) return invalid("trit " + std::to_string(i) + " is outside {-1,0,+1}");
  const size_t bytes = codec_bytes(codec, n);
  if (codec == kD2) {
    for (size_t b = 0; b < bytes; ++b) {
      unsigned v = 0x55;
      for (unsigned s = 0; s < 4 && b * 4 + s < n; ++s)
        v = (v & ~(3u << (2 * s))) | (unsigned(t[b * 4 + s] + 1) << (2 * s));
      out[b] = uint8_t(v);
    }
  } else if (codec == kB3) {
    static const unsigned place[5] = {1, 3, 9, 27, 81};
    for (size_t b = 0; b < bytes; ++b) {
      unsigned v = 0;
      for (unsigned s = 0; s < 5; ++s) v += place[s] * (b * 5 + s < n ? unsigned(t[b * 5 + s] + 1) : 1u);
      out[b] = uint8_t(v);
    }
  } else if (codec == kS34) {
    if (n % 4) return invalid("S34 requires a multiple of four trits, got " + std::to_string(n));
    std::memset(out, 0, bytes);
    for (size_t g = 0; g < n / 4; ++g) {
      unsigned code = 0, signs = 0, zeros = 0;
      for (unsigned s = 0; s < 4; ++s) {
        const int8_t v = t[g * 4 + s];
        if (v == 0) { if (!zeros) code |= s; ++zeros; }
        else { if (v > 0) code |= 1u << (2 + signs); ++signs; }
      }
      if (zeros != 1) return invalid("S34 group " + std::to_string(g) + " requires exactly one zero, got " + std::to_string(zeros));
      const size_t bit = g * 5;
      const unsigned wide = code << (bit & 7);
      out[bit >> 3] |= uint8_t(wide);
      if (wide >> 8) out[(bit >> 3) + 1] |= uint8_t(wide >> 8);
    }
  } else {
    return Err{3, "unknown codec tag " + std::to_string(codec)};
  }
  return ok();
}

Err unpack(int codec, const uint8_t* p, size_t len, size_t n, int8_t* out) {
  if (codec == kS34 && n % 4) return invalid("S34 requires a multiple of four trits, got " + std::to_string(n));
  if (codec != kD2 && codec != kB3 && codec != kS34) return Err{3, "unknown codec tag " + std::to_string(codec)};
  if (len != codec_bytes(codec, n))
    return invalid("wrong packed length: expected " + std::to_string(codec_bytes(codec, n)) + ", got " + std::to_string(len));
  if (codec == kD2) {
    for (size_t i = 0; i < len * 4; ++i) {
      const unsigned c = (p[i >> 2] >> (2 * (i & 3))) & 3u;
      if (c == 3) return invalid("reserved D2 code 11 at trit slot " + std::to_string(i));
      if (i < n) out[i] = int8_t(int(c) - 1);
      else if (c != 1) return invalid("noncanonical D2 padding at trit slot " + std::to_string(i));
    }
  } else if (codec == kB3) {
    const B3Table& tab = b3_table();
    for (size_t b = 0; b < len; ++b) {
      if (p[b] >= 243) return invalid("B3 byte " + std::to_string(b) + " holds code " + std::to_string(p[b]) + " >= 243");
      for (unsigned s = 0; s < 5; ++s) {
        const size_t i = b * 5 + s;
        if (i < n) out[i] = int8_t(int(tab.digit[p[b]][s]) - 1);
        else if (tab.digit[p[b]][s] != 1) return invalid("noncanonical B3 padding at trit slot " + std::to_string(i));
      }
    }
  } else {
    const size_t bits = n / 4 * 5;
    if (bits % 8 && (p[len - 1] >> (bits % 8))) return invalid("noncanonical S34 terminal padding bits");
    for (size_t g = 0; g < n / 4; ++g) {
      const size_t bit = g * 5;
      unsigned w = p[bit >> 3];
      if ((bit >> 3) + 1 < len) w |= unsigned(p[(bit >> 3) + 1]) << 8;
      const unsigned code = (w >> (bit & 7)) & 31u, zero = code & 3u;
      unsigned sign = 2;
      for (unsigned s = 0; s < 4; ++s) {
        if (s == zero) out[g * 4 + s] = 0;
        else { out[g * 4 + s] = (code >> sign) & 1u ? 1 : -1; ++sign; }
      }
    }
  }
  return ok();
}

Err plane_pack(int codec, const int8_t* t, size_t logical, uint8_t* out) {
  if (codec != kS34 || logical % 4 == 0) return pack(codec, t, logical, out);
  int8_t buf[kTile + 4];
  if (logical > kTile) return invalid("plane longer than a tile");
  std::memcpy(buf, t, logical);
  size_t len = logical;
  const size_t tail = logical / 4 * 4;
  const auto zeros = std::count(t + tail, t + logical, int8_t(0));
  if (zeros > 1) return invalid("S34 ragged tail holds more than one zero");
  if (zeros == 0) buf[len++] = 0;
  while (len % 4) buf[len++] = -1;
  return pack(codec, buf, len, out);
}

Err plane_unpack(int codec, const uint8_t* p, size_t len, size_t logical, int8_t* out) {
  if (codec != kS34 || logical % 4 == 0) return unpack(codec, p, len, logical, out);
  int8_t buf[kTile + 4];
  if (logical > kTile) return invalid("plane longer than a tile");
  const size_t stored = stored_len(codec, logical);
  if (Err e = unpack(codec, p, len, stored, buf)) return e;
  const size_t tail = logical / 4 * 4;
  const auto zeros = std::count(buf + tail, buf + logical, int8_t(0));
  if (zeros > 1) return invalid("S34 ragged tail holds more than one zero");
  size_t pad = logical;
  if (zeros == 0 && buf[pad++] != 0) return invalid("noncanonical S34 shape padding");
  for (; pad < stored; ++pad)
    if (buf[pad] != -1) return invalid("noncanonical S34 shape padding");
  std::memcpy(out, buf, logical);
  return ok();
}

// ---------------------------------------------------------------- resident arenas
uint8_t Resident::planes_of(uint64_t tile) const {
  if (uniform_planes) return uint8_t(uniform_planes);
  const uint64_t bit = tile * 2;
  const unsigned code = bit < map.size() * 8 ? (map[bit >> 3] >> (bit & 7)) & 3u
                                             : (terminal_map >> (bit - map.size() * 8)) & 3u;
  return uint8_t(code + 1);
}

namespace {

inline size_t tile_len(uint64_t coeffs, uint64_t tile) { return size_t(std::min<uint64_t>(kTile, coeffs - tile * kTile)); }

Err check_geometry(int codec, uint32_t group, uint64_t n, uint64_t k) {
  if (codec != kD2 && codec != kB3 && codec != kS34) return Err{3, "unknown codec tag " + std::to_string(codec)};
  if (group != 64 && group != 128) return invalid("unsupported scale group size " + std::to_string(group));
  if (n == 0 || k == 0) return invalid("tensor dimensions must be positive");
  if (n > 0xffffffffull || k > 0xffffffffull) return invalid("dimension exceeds the u32 kernel ABI");
  if (n * k / kTile + 1 > 0xffffffffull) return invalid("tile count exceeds the u32 kernel ABI");
  return ok();
}

Err check_scale(uint16_t bits, const int8_t* t, size_t begin, size_t end, uint64_t tile, unsigned plane, size_t g) {
  const std::string where = " (tile " + std::to_string(tile) + ", plane " + std::to_string(plane) + ", group " + std::to_string(g) + ")";
  if ((bits & 0x7c00u) == 0x7c00u) return invalid("non-finite scale" + where);
  if (bits & 0x8000u) return invalid("negative scale" + where);
  if (bits == 0 && t)
    for (size_t i = begin; i < end; ++i)
      if (t[i]) return invalid("zero scale over a nonzero group" + where);
  return ok();
}

void finish_index(Resident* r, const std::vector<uint8_t>& counts) {
  const uint64_t tiles = counts.size();
  r->tiles = tiles;
  r->map.assign(size_t(tiles * 2 / 8), 0);
  r->rank_prefix.clear();
  r->terminal_map = 0;
  r->present_planes = 0;
  bool uniform = true;
  for (uint64_t t = 0; t < tiles; ++t) {
    if (t && t % kRankStride == 0) r->rank_prefix.push_back(uint32_t(r->present_planes));
    const unsigned code = counts[t] - 1u;
    const uint64_t bit = t * 2;
    if (bit < r->map.size() * 8) r->map[bit >> 3] |= uint8_t(code << (bit & 7));
    else r->terminal_map |= code << (bit - r->map.size() * 8);
    r->present_planes += counts[t];
    uniform = uniform && counts[t] == counts[0];
  }
  r->uniform_planes = uniform ? counts[0] : 0;
}

}  // namespace

Err resident_sizes(int codec, uint32_t group, uint64_t n, uint64_t k, const uint8_t* pc, Sizes* out) {
  if (Err e = check_geometry(codec, group, n, k)) return e;
  const uint64_t coeffs = n * k, tiles = (coeffs + kTile - 1) / kTile;
  Sizes s;
  s.tiles = tiles;
  for (uint64_t t = 0; t < tiles; ++t) {
    if (pc[t] < 1 || pc[t] > kMaxPlanes) return invalid("tile " + std::to_string(t) + " has " + std::to_string(pc[t]) + " planes");
    const size_t len = tile_len(coeffs, t);
    s.present_planes += pc[t];
    s.payload_bytes += uint64_t(pc[t]) * plane_bytes(codec, len);
    s.scale_count += uint64_t(pc[t]) * ((len + group - 1) / group);
  }
  s.map_bytes = tiles * 2 / 8;
  s.rank_prefix_bytes = (tiles ? tiles - 1 : 0) / kRankStride * 4;
  if (s.payload_bytes > 0xffffffffull || s.scale_count > 0xffffffffull || s.present_planes > 0xffffffffull)
    return invalid("resident arenas exceed the u32 kernel ABI");
  *out = s;
  return ok();
}

Err resident_from_planes(int codec, uint32_t group, uint64_t n, uint64_t k, const uint8_t* pc,
                         const int8_t* trits, const uint16_t* scales, Resident* out) {
  Sizes sz;
  if (Err e = resident_sizes(codec, group, n, k, pc, &sz)) return e;
  const uint64_t coeffs = n * k;
  Resident r;
  r.codec = codec; r.group = group; r.n = n; r.k = k;
  r.payload.resize(size_t(sz.payload_bytes));
  r.scales.resize(size_t(sz.scale_count));
  size_t pay = 0, sc = 0;
  for (uint64_t t = 0; t < sz.tiles; ++t) {
    const size_t len = tile_len(coeffs, t), groups = (len + group - 1) / group;
    for (unsigned p = 0; p < pc[t]; ++p) {
      const int8_t* tr = trits + (t * 3 + p) * kTile;
      const uint16_t* s = scales + (t * 3 + p) * 4;
      for (size_t g = 0; g < groups; ++g)
        if (Err e = check_scale(s[g], tr, g * group, std::min(len, (g + 1) * group), t, p, g)) return e;
      if (Err e = plane_pack(codec, tr, len, r.payload.data() + pay)) return e;
      pay += plane_bytes(codec, len);
      std::copy(s, s + groups, r.scales.begin() + sc);
      sc += groups;
    }
  }
  finish_index(&r, std::vector<uint8_t>(pc, pc + sz.tiles));
  *out = std::move(r);
  return ok();
}

namespace {
// Shapes on which a tensor with varying plane counts is padded to uniform plane slots; odd shapes
// (a single row, very long rows) stay on the general route.
bool pads_to_uniform(const Resident& r) {
  return !r.uniform_planes && r.k % 256 == 0 && r.group == 128 && r.n >= 16 && r.k <= 65536;
}
}  // namespace

Err device_layout(const Resident& in, Resident* out, bool* recoded, bool* map_counts) {
  *recoded = *map_counts = false;
  const Resident* cur = &in;
  if (in.codec == kS34 && in.k % 256 == 0 && in.group == 128 && (in.uniform_planes || pads_to_uniform(in))) {
    const size_t slots = size_t(in.present_planes), from = plane_bytes(kS34, 256), to = plane_bytes(kB3, 256);
    if (in.payload.size() == slots * from) {
      *out = in;
      out->codec = kB3;
      out->payload.assign(slots * to, 0);
      int8_t trits[256];
      for (size_t i = 0; i < slots; ++i) {
        if (Err e = unpack(kS34, in.payload.data() + i * from, from, 256, trits)) return e;
        if (Err e = pack(kB3, trits, 256, out->payload.data() + i * to)) return e;
      }
      *recoded = true;
      cur = out;
    }
  }
  if (pads_to_uniform(*cur) && (cur->codec == kB3 || cur->codec == kD2)) {
    const Resident src = *cur;   // `out` may be the source
    uint32_t most = 1;
    for (uint64_t t = 0; t < src.tiles; ++t) most = std::max<uint32_t>(most, src.planes_of(t));
    const size_t pb = plane_bytes(src.codec, 256);
    *out = src;
    out->payload.assign(size_t(src.tiles) * most * pb, uint8_t(src.codec == kB3 ? 121 : 0x55));
    out->scales.assign(size_t(src.tiles) * most * 2, 0);
    size_t at = 0;
    for (uint64_t t = 0; t < src.tiles; ++t) {
      const uint32_t have = src.planes_of(t);
      std::memcpy(out->payload.data() + size_t(t) * most * pb, src.payload.data() + at * pb, size_t(have) * pb);
      std::memcpy(out->scales.data() + size_t(t) * most * 2, src.scales.data() + at * 2, size_t(have) * 2 * sizeof(uint16_t));
      at += have;
    }
    out->uniform_planes = most;
    *map_counts = true;
  }
  return ok();
}

Err resident_from_arenas(int codec, uint32_t group, uint64_t n, uint64_t k, const uint8_t* payload,
                         size_t payload_len, const uint16_t* scales, size_t scale_count,
                         const uint8_t* map, size_t map_len, uint32_t terminal, Resident* out) {
  if (Err e = check_geometry(codec, group, n, k)) return e;
  const uint64_t coeffs = n * k, tiles = (coeffs + kTile - 1) / kTile;
  if (map_len != tiles * 2 / 8)
    return shape("plane map holds " + std::to_string(map_len) + " bytes, expected " + std::to_string(tiles * 2 / 8));
  std::vector<uint8_t> counts(size_t(tiles), 1);
  for (uint64_t t = 0; t < tiles; ++t) {
    const uint64_t bit = t * 2;
    const unsigned code = bit < map_len * 8 ? (map[bit >> 3] >> (bit & 7)) & 3u : (terminal >> (bit - map_len * 8)) & 3u;
    if (code > 2) return invalid("plane map encodes four planes at tile " + std::to_string(t));
    counts[t] = uint8_t(code + 1);
  }
  const unsigned used_terminal_bits = unsigned(tiles * 2 % 8);
  if (used_terminal_bits < 32 && (terminal >> used_terminal_bits)) return invalid("terminal map value has bits beyond the last tile");
  Sizes sz;
  if (Err e = resident_sizes(codec, group, n, k, counts.data(), &sz)) return e;
  if (payload_len != sz.payload_bytes)
    return shape("payload holds " + std::to_string(payload_len) + " bytes, expected " + std::to_string(sz.payload_bytes));
  if (scale_count != sz.scale_count)
    return shape("scale arena holds " + std::to_string(scale_count) + " values, expected " + std::to_string(sz.scale_count));
  // canonicity: every plane must decode, and zero scales must sit over all-zero groups
  size_t pay = 0, sc = 0;
  int8_t decoded[kTile];
  for (uint64_t t = 0; t < tiles; ++t) {
    const size_t len = tile_len(coeffs, t), groups = (len + group - 1) / group, pb = plane_bytes(codec, len);
    for (unsigned p = 0; p < counts[t]; ++p) {
      bool need_trits = false;
      for (size_t g = 0; g < groups; ++g) need_trits |= scales[sc + g] == 0;
      if (codec == kB3 && len == kTile && !need_trits) {
        for (size_t b = 0; b < pb; ++b)
          if (payload[pay + b] >= 243) return invalid("B3 byte holds a code >= 243 in tile " + std::to_string(t));
        if (b3_table().digit[payload[pay + 51]][1] != 1 || b3_table().digit[payload[pay + 51]][2] != 1 ||
            b3_table().digit[payload[pay + 51]][3] != 1 || b3_table().digit[payload[pay + 51]][4] != 1)
          return invalid("noncanonical B3 padding in tile " + std::to_string(t));
      } else if (codec == kD2 && len == kTile && !need_trits) {
        for (size_t b = 0; b < pb; ++b)
          if (payload[pay + b] & (payload[pay + b] >> 1) & 0x55) return invalid("reserved D2 code 11 in tile " + std::to_string(t));
      } else {
        if (Err e = plane_unpack(codec, payload + pay, pb, len, decoded)) return e;
      }
      for (size_t g = 0; g < groups; ++g)
        if (Err e = check_scale(scales[sc + g], need_trits ? decoded : nullptr, g * group, std::min(len, (g + 1) * group), t, p, g)) return e;
      pay += pb; sc += groups;
    }
  }
  Resident r;
  r.codec = codec; r.group = group; r.n = n; r.k = k;
  r.payload.assign(payload, payload + payload_len);
  r.scales.assign(scales, scales + scale_count);
  finish_index(&r, counts);
  *out = std::move(r);
  return ok();
}

// ---------------------------------------------------------------- package container
namespace {

struct Reader {
  const uint8_t* b; size_t len, pos = 0; bool fail = false;
  const uint8_t* take(size_t n) { if (len - pos < n) { fail = true; return nullptr; } const uint8_t* p = b + pos; pos += n; return p; }
  uint64_t le(size_t n) { const uint8_t* p = take(n); uint64_t v = 0; if (p) for (size_t i = 0; i < n; ++i) v |= uint64_t(p[i]) << (8 * i); return v; }
};

void put(std::vector<uint8_t>* o, uint64_t v, size_t n) { for (size_t i = 0; i < n; ++i) o->push_back(uint8_t(v >> (8 * i))); }

inline unsigned presence_bits(unsigned planes) { return planes == 1 ? 0u : planes == 2 ? 1u : 3u; }

struct RawTensor {
  std::string name;
  uint64_t rows = 1, cols = 0, coeffs = 0, tiles = 0, full_tiles = 0, first_full = 0;
  uint32_t group = 128;
  int ragged_planes = 0;
  const uint8_t* payload = nullptr; const uint8_t* scales = nullptr;
  uint64_t payload_len = 0, scales_len = 0;
};

}  // namespace

// write_salt_v2_package (crates/tritium-format/src/salt_v2_package.rs:1526-1668): tensors in the
// given order, one presence map over the full tiles of all of them behind the last tensor, its
// trailing bits in the tensor-count word, version 2 as soon as one tensor uses 64-wide groups.
Err package_write_multi(int codec, const PackageTensorIn* ts, size_t count, std::vector<uint8_t>* out) {
  if (count == 0 || count >= (1u << 26)) return shape("a package holds 1 .. 2^26 - 1 tensors");
  std::vector<Resident> rs(count);
  uint64_t full_total = 0, raw = 24;
  bool any64 = false;
  for (size_t i = 0; i < count; ++i) {
    const PackageTensorIn& t = ts[i];
    if (!t.name || !*t.name) return invalid("tensor name is empty");
    for (size_t j = 0; j < i; ++j)
      if (std::strcmp(ts[j].name, t.name) == 0) return invalid(std::string("duplicate tensor name ") + t.name);
    if (Err e = resident_from_planes(codec, t.group, t.n, t.k, t.plane_count, t.trits, t.scales, &rs[i])) return e;
    any64 |= t.group == 64;
    full_total += t.n * t.k / kTile;
    raw += 64 + std::strlen(t.name) + 16 + rs[i].payload.size() + rs[i].scales.size() * 2;
  }
  std::vector<uint8_t> map(size_t(full_total * 2 / 8), 0);
  unsigned embedded = 0;
  uint64_t g = 0;
  for (size_t i = 0; i < count; ++i) {
    const uint64_t full = ts[i].n * ts[i].k / kTile;
    for (uint64_t t = 0; t < full; ++t, ++g) {
      const unsigned bits = presence_bits(ts[i].plane_count[t]);
      for (unsigned b = 0; b < 2; ++b)
        if (bits >> b & 1u) {
          const uint64_t bit = g * 2 + b;
          if (bit < map.size() * 8) map[bit >> 3] |= uint8_t(1u << (bit & 7));
          else embedded |= 1u << (bit - map.size() * 8);
        }
    }
  }
  raw += map.size();
  const uint64_t total = (raw + 7) / 8 * 8;
  std::vector<uint8_t>& o = *out;
  o.clear();
  o.reserve(size_t(total));
  o.insert(o.end(), {'T', 'S', 'L', 'T', '2', 'P', 'K', 'G'});
  put(&o, any64 ? 2 : 1, 2);
  o.push_back(uint8_t(codec));
  o.push_back(0);
  put(&o, uint32_t(count) | (embedded << 26), 4);
  put(&o, total, 8);
  for (size_t i = 0; i < count; ++i) {
    const PackageTensorIn& t = ts[i];
    const Resident& r = rs[i];
    const uint64_t coeffs = t.n * t.k;
    const size_t name_len = std::strlen(t.name);
    put(&o, name_len, 4);
    put(&o, 2, 4);
    put(&o, coeffs, 8);
    put(&o, r.tiles | (uint64_t(coeffs % kTile ? presence_bits(t.plane_count[r.tiles - 1]) : 0u) << 62), 8);
    put(&o, r.payload.size(), 8);
    put(&o, r.scales.size() * 2, 8);
    o.push_back(0);
    o.push_back(t.group == 64 ? 1 : 0);
    o.insert(o.end(), 6 + 16, 0);
    o.insert(o.end(), t.name, t.name + name_len);
    put(&o, t.n, 8);
    put(&o, t.k, 8);
    o.insert(o.end(), r.payload.begin(), r.payload.end());
    for (uint16_t s : r.scales) put(&o, s, 2);
  }
  o.insert(o.end(), map.begin(), map.end());
  o.resize(size_t(total), 0);
  return ok();
}

Err package_write(int codec, const char* name, uint32_t group, uint64_t n, uint64_t k,
                  const uint8_t* pc, const int8_t* trits, const uint16_t* scales, std::vector<uint8_t>* out) {
  const PackageTensorIn one{name, group, n, k, pc, trits, scales};
  return package_write_multi(codec, &one, 1, out);
}

// ---------------------------------------------------------------- package reader over a byte source
// SaltV2PackageReader (crates/tritium-format/src/salt_v2_package/reader.rs:333,790,841): the
// header table is walked with small reads, the sections of other tensors are skipped, and only the
// named tensor's payload, scales and its slice of the presence map are fetched.
namespace {
struct SourceReader {
  ReadAtFn read_at; void* user; uint64_t len; uint64_t pos = 0; bool fail = false;
  bool fetch(uint64_t off, void* dst, size_t n) {
    if (off > len || len - off < n) { fail = true; return false; }
    if (n && read_at(user, off, dst, n) != 0) { fail = true; return false; }
    return true;
  }
  bool take(void* dst, size_t n) { if (!fetch(pos, dst, n)) return false; pos += n; return true; }
  uint64_t le(size_t n) { uint8_t b[8] = {0}; take(b, n); uint64_t v = 0; for (size_t i = 0; i < n; ++i) v |= uint64_t(b[i]) << (8 * i); return v; }
  void skip(uint64_t n) { if (len - pos < n) fail = true; else pos += n; }
};
}  // namespace

Err resident_from_reader(ReadAtFn read_at, void* user, uint64_t len, const char* want, Resident* out) {
  if (!read_at || !want) return invalid("null reader or tensor name");
  SourceReader rd{read_at, user, len};
  uint8_t magic[8];
  if (!rd.take(magic, 8) || std::memcmp(magic, "TSLT2PKG", 8)) return invalid("bad package magic");
  const unsigned version = unsigned(rd.le(2));
  if (rd.fail || (version != 1 && version != 2)) return invalid("unsupported package version " + std::to_string(version));
  const int codec = int(rd.le(1));
  if (rd.fail || codec < kD2 || codec > kS34) return Err{3, "unsupported package codec tag " + std::to_string(codec)};
  if (rd.le(1) != 0 || rd.fail) return invalid("package flags must be zero");
  const uint32_t word = uint32_t(rd.le(4));
  const uint32_t count = word & ((1u << 26) - 1), embedded = word >> 26;
  const uint64_t declared_total = rd.le(8);
  if (rd.fail) return invalid("truncated package header");
  if (declared_total != len) return invalid("package declares " + std::to_string(declared_total) + " bytes but holds " + std::to_string(len));
  if (count == 0) return invalid("package holds no tensor");
  RawTensor hit;
  uint64_t hit_payload_off = 0, hit_scales_off = 0, full_total = 0;
  bool found = false, any64 = false;
  std::vector<std::string> names;
  for (uint32_t i = 0; i < count; ++i) {
    RawTensor t;
    const uint32_t name_len = uint32_t(rd.le(4)), rank = uint32_t(rd.le(4));
    const uint64_t declared_coeffs = rd.le(8), tile_word = rd.le(8);
    t.payload_len = rd.le(8); t.scales_len = rd.le(8);
    const unsigned tag = unsigned(rd.le(1)), geom = unsigned(rd.le(1));
    uint8_t zero6[6] = {1, 1, 1, 1, 1, 1};
    rd.take(zero6, 6);
    const uint64_t seed = rd.le(8), domain = rd.le(8);
    if (rd.fail) return invalid("truncated tensor header");
    if (std::any_of(zero6, zero6 + 6, [](uint8_t v) { return v != 0; })) return invalid("noncanonical transform metadata");
    if (version == 1 ? geom != 0 : geom > 1) return invalid("unsupported scale geometry tag " + std::to_string(geom));
    t.group = geom ? 64 : 128;
    any64 |= geom != 0;
    if (tag == 0 && (seed || domain)) return invalid("noncanonical transform metadata");
    if (tag > 1) return invalid("unsupported transform tag " + std::to_string(tag));
    if (!name_len) return invalid("empty tensor name");
    if (name_len > rd.len - rd.pos) return invalid("truncated tensor name");
    t.name.resize(name_len);
    if (!rd.take(&t.name[0], name_len)) return invalid("truncated tensor name");
    if (std::find(names.begin(), names.end(), t.name) != names.end()) return invalid("duplicate tensor name " + t.name);
    names.push_back(t.name);
    if (rank == 0) return invalid("tensor has no dimensions");
    uint64_t prod = 1, last = 1;
    for (uint32_t d = 0; d < rank; ++d) {
      last = rd.le(8);
      if (rd.fail) return invalid("truncated tensor dimensions");
      if (!last || (prod && last > UINT64_MAX / prod)) return invalid("invalid tensor dimensions");
      prod *= last;
    }
    t.cols = last; t.rows = prod / last; t.coeffs = prod;
    if (declared_coeffs != prod) return invalid("declared coefficient count disagrees with the dimensions");
    t.tiles = (prod + kTile - 1) / kTile;
    if ((tile_word & ((1ull << 62) - 1)) != t.tiles) return invalid("declared tile count disagrees with the dimensions");
    const unsigned ragged = unsigned(tile_word >> 62);
    t.full_tiles = prod / kTile;
    if (prod % kTile == 0) { if (ragged) return invalid("noncanonical map padding"); }
    else { if (ragged == 2) return invalid("plane map is not nested"); t.ragged_planes = 1 + int(ragged & 1) + int(ragged >> 1); }
    const bool is_hit = t.name == want;
    if (tag == 1 && is_hit) return invalid("tensor transform SignedRht is not implemented; only None is accepted");
    if (rank != 2 && is_hit) return invalid("SALT V2 forward requires rank 2, got rank " + std::to_string(rank));
    if (t.payload_len > rd.len - rd.pos || t.scales_len > rd.len - rd.pos - t.payload_len) return invalid("truncated tensor sections");
    t.first_full = full_total;
    if (is_hit) { hit = t; hit_payload_off = rd.pos; hit_scales_off = rd.pos + t.payload_len; found = true; }
    rd.skip(t.payload_len + t.scales_len);
    full_total += t.full_tiles;
  }
  if (version != (any64 ? 2u : 1u)) return invalid("noncanonical package version");
  const uint64_t map_off = rd.pos, map_len = full_total * 2 / 8;
  rd.skip(map_len);
  if (rd.fail) return invalid("truncated presence map");
  if (full_total * 2 % 8 < 6 && (embedded >> (full_total * 2 % 8))) return invalid("noncanonical map padding");
  const uint64_t pad = (8 - rd.pos % 8) % 8;
  if (rd.len - rd.pos != pad) return invalid("unexpected trailing data");
  uint8_t padding[8] = {0};
  if (pad && !rd.take(padding, size_t(pad))) return invalid("truncated file padding");
  for (uint64_t i = 0; i < pad; ++i) if (padding[i]) return invalid("noncanonical file padding");
  if (!found) return invalid(std::string("package holds no tensor named ") + want);
  // the tensor's slice of the presence map
  const uint64_t bit0 = hit.first_full * 2, bit1 = (hit.first_full + hit.full_tiles) * 2;
  const uint64_t byte0 = bit0 / 8, byte1 = std::min<uint64_t>((bit1 + 7) / 8, map_len);
  std::vector<uint8_t> map(size_t(byte1 > byte0 ? byte1 - byte0 : 0));
  if (!map.empty() && !rd.fetch(map_off + byte0, map.data(), map.size())) return invalid("presence map cannot be read");
  auto planes_at = [&](uint64_t gtile) -> int {
    unsigned bits = 0;
    for (unsigned b = 0; b < 2; ++b) {
      const uint64_t bit = gtile * 2 + b;
      bits |= (bit < map_len * 8 ? (map[size_t((bit >> 3) - byte0)] >> (bit & 7)) & 1u : (embedded >> (bit - map_len * 8)) & 1u) << b;
    }
    return bits == 2 ? -1 : 1 + int(bits & 1) + int(bits >> 1);
  };
  std::vector<uint8_t> counts(size_t(hit.tiles));
  for (uint64_t i = 0; i < hit.tiles; ++i) {
    const int pcount = i < hit.full_tiles ? planes_at(hit.first_full + i) : hit.ragged_planes;
    if (pcount < 0) return invalid("plane map is not nested");
    counts[i] = uint8_t(pcount);
  }
  Sizes sz;
  if (Err e = resident_sizes(codec, hit.group, hit.rows, hit.cols, counts.data(), &sz)) return e;
  if (sz.payload_bytes != hit.payload_len || sz.scale_count * 2 != hit.scales_len)
    return invalid("declared section sizes of tensor " + hit.name + " disagree with the derived sizes");
  std::vector<uint8_t> payload(size_t(hit.payload_len)), scale_bytes(size_t(hit.scales_len));
  if (!payload.empty() && !rd.fetch(hit_payload_off, payload.data(), payload.size())) return invalid("tensor payload cannot be read");
  if (!scale_bytes.empty() && !rd.fetch(hit_scales_off, scale_bytes.data(), scale_bytes.size())) return invalid("tensor scales cannot be read");
  std::vector<uint16_t> sc(scale_bytes.size() / 2);
  for (size_t i = 0; i < sc.size(); ++i) sc[i] = uint16_t(scale_bytes[2 * i] | (scale_bytes[2 * i + 1] << 8));
  std::vector<uint8_t> rmap(size_t(hit.tiles * 2 / 8), 0);
  uint32_t terminal = 0;
  for (uint64_t i = 0; i < hit.tiles; ++i) {
    const uint64_t bit = i * 2;
    const unsigned code = counts[i] - 1u;
    if (bit < rmap.size() * 8) rmap[bit >> 3] |= uint8_t(code << (bit & 7));
    else terminal |= code << (bit - rmap.size() * 8);
  }
  return resident_from_arenas(codec, hit.group, hit.rows, hit.cols, payload.data(), payload.size(), sc.data(), sc.size(),
                              rmap.data(), rmap.size(), terminal, out);
}

Err resident_from_package(const uint8_t* bytes, size_t len, const char* want, Resident* out) {
  Reader rd{bytes, len};
  const uint8_t* magic = rd.take(8);
  if (!magic || std::memcmp(magic, "TSLT2PKG", 8)) return invalid("bad package magic");
  const unsigned version = unsigned(rd.le(2));
  if (rd.fail || (version != 1 && version != 2)) return invalid("unsupported package version " + std::to_string(version));
  const int codec = int(rd.le(1));
  if (rd.fail || codec < kD2 || codec > kS34) return Err{3, "unsupported package codec tag " + std::to_string(codec)};
  if (rd.le(1) != 0 || rd.fail) return invalid("package flags must be zero");
  const uint32_t word = uint32_t(rd.le(4));
  const uint32_t count = word & ((1u << 26) - 1), embedded = word >> 26;
  const uint64_t declared_total = rd.le(8);
  if (rd.fail) return invalid("truncated package header");
  if (declared_total != len) return invalid("package declares " + std::to_string(declared_total) + " bytes but holds " + std::to_string(len));
  if (count == 0) return invalid("package holds no tensor");
  if (count > (len - rd.pos) / 64) return invalid("truncated tensor table");
  std::vector<RawTensor> ts(count);
  uint64_t full_total = 0;
  bool any64 = false;
  for (uint32_t i = 0; i < count; ++i) {
    RawTensor& t = ts[i];
    const uint32_t name_len = uint32_t(rd.le(4)), rank = uint32_t(rd.le(4));
    const uint64_t declared_coeffs = rd.le(8), tile_word = rd.le(8);
    t.payload_len = rd.le(8); t.scales_len = rd.le(8);
    const unsigned tag = unsigned(rd.le(1)), geom = unsigned(rd.le(1));
    const uint8_t* zero6 = rd.take(6);
    const uint64_t seed = rd.le(8), domain = rd.le(8);
    if (rd.fail) return invalid("truncated tensor header");
    if (std::any_of(zero6, zero6 + 6, [](uint8_t v) { return v != 0; })) return invalid("noncanonical transform metadata");
    if (version == 1 ? geom != 0 : geom > 1) return invalid("unsupported scale geometry tag " + std::to_string(geom));
    t.group = geom ? 64 : 128;
    any64 |= geom != 0;
    if (tag == 0 && (seed || domain)) return invalid("noncanonical transform metadata");
    if (tag > 1) return invalid("unsupported transform tag " + std::to_string(tag));
    const uint8_t* nm = rd.take(name_len);
    if (rd.fail) return invalid("truncated tensor name");
    if (!name_len) return invalid("empty tensor name");
    t.name.assign(reinterpret_cast<const char*>(nm), name_len);
    for (uint32_t j = 0; j < i; ++j)
      if (ts[j].name == t.name) return invalid("duplicate tensor name " + t.name);
    if (rank == 0) return invalid("tensor has no dimensions");
    uint64_t prod = 1, last = 1;
    for (uint32_t d = 0; d < rank; ++d) {
      last = rd.le(8);
      if (rd.fail) return invalid("truncated tensor dimensions");
      if (!last || (prod && last > UINT64_MAX / prod)) return invalid("invalid tensor dimensions");
      prod *= last;
    }
    t.cols = last; t.rows = prod / last; t.coeffs = prod;
    if (declared_coeffs != prod) return invalid("declared coefficient count disagrees with the dimensions");
    t.tiles = (prod + kTile - 1) / kTile;
    if ((tile_word & ((1ull << 62) - 1)) != t.tiles) return invalid("declared tile count disagrees with the dimensions");
    const unsigned ragged = unsigned(tile_word >> 62);
    t.full_tiles = prod / kTile;
    if (prod % kTile == 0) { if (ragged) return invalid("noncanonical map padding"); }
    else { if (ragged == 2) return invalid("plane map is not nested"); t.ragged_planes = 1 + int(ragged & 1) + int(ragged >> 1); }
    if (tag == 1 && std::strcmp(want, t.name.c_str()) == 0) return invalid("tensor transform SignedRht is not implemented; only None is accepted");
    if (rank != 2 && std::strcmp(want, t.name.c_str()) == 0) return invalid("SALT V2 forward requires rank 2, got rank " + std::to_string(rank));
    if (t.payload_len + t.scales_len > len - rd.pos) return invalid("truncated tensor sections");
    t.payload = rd.take(size_t(t.payload_len));
    t.scales = rd.take(size_t(t.scales_len));
    t.first_full = full_total;
    full_total += t.full_tiles;
  }
  if (version != (any64 ? 2u : 1u)) return invalid("noncanonical package version");
  const size_t map_len = size_t(full_total * 2 / 8);
  const uint8_t* map = rd.take(map_len);
  if (rd.fail) return invalid("truncated presence map");
  if (full_total * 2 % 8 < 6 && (embedded >> (full_total * 2 % 8))) return invalid("noncanonical map padding");
  const size_t pad = (8 - rd.pos % 8) % 8;
  if (len - rd.pos != pad) return invalid("unexpected trailing data");
  for (size_t i = 0; i < pad; ++i) if (bytes[rd.pos + i]) return invalid("noncanonical file padding");
  auto planes_at = [&](uint64_t g) -> int {
    unsigned bits = 0;
    for (unsigned b = 0; b < 2; ++b) {
      const uint64_t bit = g * 2 + b;
      bits |= (bit < map_len * 8 ? (map[bit >> 3] >> (bit & 7)) & 1u : (embedded >> (bit - map_len * 8)) & 1u) << b;
    }
    return bits == 2 ? -1 : 1 + int(bits & 1) + int(bits >> 1);
  };
  const RawTensor* hit = nullptr;
  std::vector<uint8_t> hit_counts;
  for (const RawTensor& t : ts) {
    std::vector<uint8_t> counts(size_t(t.tiles));
    for (uint64_t i = 0; i < t.tiles; ++i) {
      const int p = i < t.full_tiles ? planes_at(t.first_full + i) : t.ragged_planes;
      if (p < 0) return invalid("plane map is not nested");
      counts[i] = uint8_t(p);
    }
    Sizes sz;
    if (Err e = resident_sizes(codec, t.group, t.rows, t.cols, counts.data(), &sz)) return e;
    if (sz.payload_bytes != t.payload_len || sz.scale_count * 2 != t.scales_len)
      return invalid("declared section sizes of tensor " + t.name + " disagree with the derived sizes");
    if (t.name == want) { hit = &t; hit_counts = counts; }
  }
  if (!hit) return invalid(std::string("package holds no tensor named ") + want);
  std::vector<uint16_t> sc(size_t(hit->scales_len / 2));
  for (size_t i = 0; i < sc.size(); ++i) sc[i] = uint16_t(hit->scales[2 * i] | (hit->scales[2 * i + 1] << 8));
  // runtime map (planes-1) from the presence bits
  std::vector<uint8_t> rmap(size_t(hit->tiles * 2 / 8), 0);
  uint32_t terminal = 0;
  for (uint64_t i = 0; i < hit->tiles; ++i) {
    const uint64_t bit = i * 2;
    const unsigned code = hit_counts[i] - 1u;
    if (bit < rmap.size() * 8) rmap[bit >> 3] |= uint8_t(code << (bit & 7));
    else terminal |= code << (bit - rmap.size() * 8);
  }
  return resident_from_arenas(codec, hit->group, hit->rows, hit->cols, hit->payload, size_t(hit->payload_len),
                              sc.data(), sc.size(), rmap.data(), rmap.size(), terminal, out);
}

// ---------------------------------------------------------------- TQ2_0
// 66-byte block: byte c*32+m holds elements c*128 + n*32 + m (n = 0..3) at bit 2n, code = trit+1,
// followed by an f16 block scale (crates/tritium-format/src/tq2.rs:21-46).
Err tq2_pack_rows(const int8_t* trits, uint64_t n, uint64_t k, uint8_t* out) {
  const uint64_t nb = (k + 255) / 256;
  for (uint64_t r = 0; r < n; ++r)
    for (uint64_t b = 0; b < nb; ++b) {
      uint8_t* o = out + (r * nb + b) * 66;
      for (unsigned byte = 0; byte < 64; ++byte) {
        unsigned v = 0;
        for (unsigned s = 0; s < 4; ++s) {
          const uint64_t e = b * 256 + (byte / 32) * 128 + s * 32 + byte % 32;
          const int8_t t = e < k ? trits[r * k + e] : int8_t(0);
          if (t < -1 || t > 1) return invalid("trit outside {-1,0,+1}");
          v |= unsigned(t + 1) << (2 * s);
        }
        o[byte] = uint8_t(v);
      }
      o[64] = 0x00; o[65] = 0x3c;  // f16 1.0
    }
  return ok();
}

Err resident_from_tq2(const uint8_t* packed, size_t len, uint64_t n, uint64_t k, Resident* out) {
  if (Err e = check_geometry(kD2, 128, std::max<uint64_t>(n, 1), std::max<uint64_t>(k, 1))) return e;
  const uint64_t nb = (k + 255) / 256;
  if (len != n * nb * 66)
    return invalid("packed len " + std::to_string(len) + " != expected " + std::to_string(n * nb * 66));
  // Rows are padded to whole 256-trit blocks with zero trits, so the D2 tensor is [n, nb*256].
  const uint64_t kp = nb * 256;
  Resident r;
  r.codec = kD2; r.group = 128; r.n = n; r.k = kp;
  r.payload.assign(size_t(n * nb * 64), 0x55);
  r.scales.assign(size_t(n * nb * 2), 0x3c00);
  for (uint64_t blk = 0; blk < n * nb; ++blk) {
    const uint8_t* qs = packed + blk * 66;
    uint8_t* o = r.payload.data() + blk * 64;
    for (unsigned byte = 0; byte < 64; ++byte) {
      if (qs[byte] & (qs[byte] >> 1) & 0x55) return invalid("TQ2_0 block holds the reserved code 11");
      for (unsigned s = 0; s < 4; ++s) {
        const unsigned e = (byte / 32) * 128 + s * 32 + byte % 32, code = (qs[byte] >> (2 * s)) & 3u;
        o[e >> 2] = uint8_t((o[e >> 2] & ~(3u << (2 * (e & 3)))) | (code << (2 * (e & 3))));
      }
    }
  }
  finish_index(&r, std::vector<uint8_t>(size_t(n * nb), 1));
  *out = std::move(r);
  return ok();
}

// TQ1_0 rows (54-byte blocks: 48 + 4 bytes of five / four trits in ggml's fixed-point base-3 code,
// f16 scale; crates/tritium-format/src/tq1.rs:16-122) -> a 1-plane D2 tensor with unit group scales,
// like resident_from_tq2.  Digit n of a byte: (((byte * 3^n) mod 256) * 3) >> 8.
Err resident_from_tq1(const uint8_t* packed, size_t len, uint64_t n, uint64_t k, Resident* out) {
  if (Err e = check_geometry(kD2, 128, std::max<uint64_t>(n, 1), std::max<uint64_t>(k, 1))) return e;
  const uint64_t nb = (k + 255) / 256;
  if (len != n * nb * 54)
    return invalid("packed len " + std::to_string(len) + " != expected " + std::to_string(n * nb * 54));
  Resident r;
  r.codec = kD2; r.group = 128; r.n = n; r.k = nb * 256;
  r.payload.assign(size_t(n * nb * 64), 0);
  r.scales.assign(size_t(n * nb * 2), 0x3c00);
  static const uint8_t pow3[5] = {1, 3, 9, 27, 81};
  auto digit = [](uint8_t byte, unsigned d) { return unsigned((unsigned(uint8_t(byte * pow3[d])) * 3u) >> 8); };
  for (uint64_t blk = 0; blk < n * nb; ++blk) {
    const uint8_t* qs = packed + blk * 54;
    uint8_t* o = r.payload.data() + blk * 64;
    auto put_code = [&](unsigned e, unsigned code) { o[e >> 2] = uint8_t(o[e >> 2] | (code << (2 * (e & 3)))); };
    for (unsigned d = 0; d < 5; ++d) for (unsigned m = 0; m < 32; ++m) put_code(d * 32 + m, digit(qs[m], d));
    for (unsigned d = 0; d < 5; ++d) for (unsigned m = 0; m < 16; ++m) put_code(160 + d * 16 + m, digit(qs[32 + m], d));
    for (unsigned d = 0; d < 4; ++d) for (unsigned j = 0; j < 4; ++j) put_code(240 + d * 4 + j, digit(qs[48 + j], d));
  }
  finish_index(&r, std::vector<uint8_t>(size_t(n * nb), 1));
  *out = std::move(r);
  return ok();
}

// SALT V1: `planes` plane-major TQ2_0 rows [t][n][ceil(k/256) * 66] whose f16 block scale is that
// plane's scale for the block (crates/tritium-cuda/kernels/tq2_0_add.cu:640-660,
// crates/tritium-nn/src/layers/packed_salt.rs:630-645).  Re-laid as a t-plane D2 tensor whose two
// 128-wide groups of a tile both carry the block scale.
Err resident_from_salt_v1(const uint8_t* packed, size_t len, uint32_t t_planes, uint64_t n, uint64_t k, Resident* out) {
  if (t_planes < 1 || t_planes > kMaxPlanes) return Err{3, "SALT V1 upload takes 1..3 planes, got " + std::to_string(t_planes)};
  if (Err e = check_geometry(kD2, 128, std::max<uint64_t>(n, 1), std::max<uint64_t>(k, 1))) return e;
  const uint64_t nb = (k + 255) / 256;
  if (len != uint64_t(t_planes) * n * nb * 66)
    return invalid("packed len " + std::to_string(len) + " != expected " + std::to_string(uint64_t(t_planes) * n * nb * 66));
  Resident r;
  r.codec = kD2; r.group = 128; r.n = n; r.k = nb * 256;
  r.payload.assign(size_t(n * nb * t_planes * 64), 0x55);
  r.scales.assign(size_t(n * nb * t_planes * 2), 0);
  for (uint64_t row = 0; row < n; ++row)
    for (uint64_t b = 0; b < nb; ++b)
      for (uint32_t p = 0; p < t_planes; ++p) {
        const uint8_t* qs = packed + ((uint64_t(p) * n + row) * nb + b) * 66;
        const uint64_t tile_plane = (row * nb + b) * t_planes + p;
        uint8_t* o = r.payload.data() + tile_plane * 64;
        bool any = false;
        for (unsigned byte = 0; byte < 64; ++byte) {
          if (qs[byte] & (qs[byte] >> 1) & 0x55) return invalid("TQ2_0 block holds the reserved code 11");
          for (unsigned s = 0; s < 4; ++s) {
            const unsigned e = (byte / 32) * 128 + s * 32 + byte % 32, code = (qs[byte] >> (2 * s)) & 3u;
            any |= code != 1u;
            o[e >> 2] = uint8_t((o[e >> 2] & ~(3u << (2 * (e & 3)))) | (code << (2 * (e & 3))));
          }
        }
        const uint16_t bits = uint16_t(qs[64] | (qs[65] << 8));
        const bool finite = (bits & 0x7c00) != 0x7c00, negative = (bits & 0x8000) != 0;
        if (!finite || negative) return invalid("SALT V1 block scale must be a finite, non-negative f16");
        if ((bits & 0x7fff) == 0 && any) return invalid("SALT V1 block scale is zero over a block that holds trits");
        r.scales[size_t(tile_plane * 2)] = bits;
        r.scales[size_t(tile_plane * 2 + 1)] = bits;
      }
  finish_index(&r, std::vector<uint8_t>(size_t(n * nb), uint8_t(t_planes)));
  *out = std::move(r);
  return ok();
}

// ---------------------------------------------------------------- tensor-parallel shards
Err shard_sizes(int codec, uint32_t group, uint32_t n, uint32_t k, uint32_t planes, bool row_parallel,
                uint32_t world, uint32_t rank, ShardSizes* out) {
  if (Err e = check_geometry(codec, group, n, k)) return e;
  if (planes < 1 || planes > kMaxPlanes) return invalid("plane count must be 1..3");
  if (!world || rank >= world) return invalid("rank must be below the world size");
  if (k % kTile) return invalid("tensor-parallel sharding needs k to be a multiple of 256");
  ShardSizes s;
  if (row_parallel) {
    if (k % (uint64_t(world) * group)) return invalid("k is not divisible into scale-group aligned shards");
    s.n = n; s.k = (k / world + kTile - 1) / kTile * kTile;  // padded to whole tiles with zero trits
  } else {
    if (n % world) return invalid("n is not divisible by the world size");
    s.n = n / world; s.k = k;
  }
  const uint64_t tiles = uint64_t(s.n) * s.k / kTile;
  s.payload_bytes = tiles * planes * plane_bytes(codec, kTile);
  s.scale_count = tiles * planes * (kTile / group);
  s.map_bytes = tiles * 2 / 8;
  *out = s;
  return ok();
}

Err shard(int codec, uint32_t group, uint32_t n, uint32_t k, uint32_t planes, const uint8_t* payload,
          const uint16_t* scales, bool row_parallel, uint32_t world, uint32_t rank,
          uint8_t* sp, uint16_t* ss, uint8_t* smap, uint32_t* terminal) {
  ShardSizes sz;
  if (Err e = shard_sizes(codec, group, n, k, planes, row_parallel, world, rank, &sz)) return e;
  const size_t pb = plane_bytes(codec, kTile), gpt = kTile / group;
  const uint64_t tpr = k / kTile;  // tiles per source row
  if (!row_parallel) {
    const uint64_t first_tile = uint64_t(rank) * sz.n * tpr, tiles = uint64_t(sz.n) * tpr;
    std::memcpy(sp, payload + first_tile * planes * pb, size_t(tiles * planes * pb));
    std::memcpy(ss, scales + first_tile * planes * gpt, size_t(tiles * planes * gpt) * 2);
  } else {
    const uint64_t kv = k / world, k0 = uint64_t(rank) * kv, stpr = sz.k / kTile;
    std::vector<int8_t> row(static_cast<size_t>(k), 0), piece(kTile, 0);
    for (uint64_t r = 0; r < n; ++r)
      for (uint32_t p = 0; p < planes; ++p) {
        for (uint64_t t = 0; t < tpr; ++t)
          if (Err e = unpack(codec, payload + ((r * tpr + t) * planes + p) * pb, pb, kTile, row.data() + t * kTile)) return e;
        for (uint64_t t = 0; t < stpr; ++t) {
          std::fill(piece.begin(), piece.end(), int8_t(0));
          const uint64_t begin = t * kTile, end = std::min<uint64_t>(kv, begin + kTile);
          if (end > begin) std::copy(row.begin() + k0 + begin, row.begin() + k0 + end, piece.begin());
          if (codec == kS34)  // padded coefficients must keep the one-zero-per-four structure
            for (uint64_t e = end > begin ? end - begin : 0; e < kTile; ++e) piece[e] = (e % 4) ? int8_t(-1) : int8_t(0);
          if (Err e = pack(codec, piece.data(), kTile, sp + ((r * stpr + t) * planes + p) * pb)) return e;
          for (uint64_t g = 0; g < gpt; ++g) {
            const uint64_t col = k0 + begin + g * group;  // source column of this scale group
            const bool live = begin + g * group < kv;
            const uint64_t st = col / kTile, sg = (col % kTile) / group;
            // S34 padding carries nonzero trits, so its (unused) groups take a unit scale and
            // rely on zero activations; D2/B3 padding is all-zero and takes a zero scale.
            ss[((r * stpr + t) * planes + p) * gpt + g] =
                live ? scales[((r * tpr + st) * planes + p) * gpt + sg] : (codec == kS34 ? uint16_t(0x3c00) : uint16_t(0));
          }
        }
      }
  }
  const uint64_t tiles = uint64_t(sz.n) * sz.k / kTile;
  std::memset(smap, 0, size_t(sz.map_bytes));
  *terminal = 0;
  for (uint64_t t = 0; t < tiles; ++t) {
    const uint64_t bit = t * 2;
    if (bit < sz.map_bytes * 8) smap[bit >> 3] |= uint8_t((planes - 1) << (bit & 7));
    else *terminal |= (planes - 1) << (bit - sz.map_bytes * 8);
  }
  return ok();
}

// ---------------------------------------------------------------- host activation quantiser
// per token: gamma = max|x|; zero row -> zeros and zero scale; q = clamp(rint(x * (127/gamma)));
// scale = gamma/127 (crates/tritium-spec/src/lib.rs:351-378).
void quantize_act_int8(const float* act, uint64_t m, uint64_t k, float* q, float* scale) {
  for (uint64_t r = 0; r < m; ++r) {
    const float* x = act + r * k;
    float gamma = 0.f;
    for (uint64_t i = 0; i < k; ++i) gamma = std::max(gamma, std::fabs(x[i]));
    if (gamma == 0.f) { std::fill(q + r * k, q + (r + 1) * k, 0.f); scale[r] = 0.f; continue; }
    const float s = 127.0f / gamma;
    for (uint64_t i = 0; i < k; ++i) q[r * k + i] = std::min(127.f, std::max(-128.f, std::nearbyintf(x[i] * s)));
    scale[r] = gamma / 127.0f;
  }
}

}  // namespace tbf
