// Host-side byte layouts of the packed ternary artifact (tritium-format's SALT V2 codecs,
// package container, indexed runtime arenas and TQ2_0 rows).  Pure C++17, no device code.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace tbf {

constexpr uint32_t kTile = 256;        // coefficients per allocation tile
constexpr uint32_t kMaxPlanes = 3;
constexpr uint32_t kRankStride = 256;  // tiles per rank prefix

enum Codec : int { kD2 = 1, kB3 = 2, kS34 = 3 };

// Error carrier: code follows tb_status numbering (0 ok, 2 shape, 3 format, 5 invalid input).
struct Err {
  int code = 0;
  std::string msg;
  explicit operator bool() const { return code != 0; }
};
inline Err ok() { return {}; }
Err invalid(const std::string& m);
Err shape(const std::string& m);

uint16_t f32_to_f16(float v);
float f16_to_f32(uint16_t h);

size_t codec_bytes(int codec, size_t trits);               // codec ledger (trits must suit S34)
size_t plane_bytes(int codec, size_t logical_len);         // incl. S34 shape padding
Err pack(int codec, const int8_t* trits, size_t n, uint8_t* out);
Err unpack(int codec, const uint8_t* packed, size_t len, size_t n, int8_t* out);
Err plane_pack(int codec, const int8_t* trits, size_t logical_len, uint8_t* out);
Err plane_unpack(int codec, const uint8_t* packed, size_t len, size_t logical_len, int8_t* out);

// Resident ("indexed runtime") arenas of one [n,k] tensor.
struct Resident {
  int codec = kB3;
  uint32_t group = 128;
  uint64_t n = 0, k = 0, tiles = 0, present_planes = 0;
  uint32_t uniform_planes = 0;  // 1..3 when every tile has that many planes, else 0
  std::vector<uint8_t> payload;
  std::vector<uint16_t> scales;
  std::vector<uint8_t> map;          // complete bytes of the 2-bit runtime map (value planes-1)
  std::vector<uint32_t> rank_prefix; // cumulative planes before tile 256, 512, ...
  uint32_t terminal_map = 0;
  uint8_t planes_of(uint64_t tile) const;
};

struct Sizes {
  uint64_t payload_bytes = 0, scale_count = 0, map_bytes = 0, rank_prefix_bytes = 0, tiles = 0,
           present_planes = 0;
};
Err resident_sizes(int codec, uint32_t group, uint64_t n, uint64_t k, const uint8_t* plane_count,
                   Sizes* out);
// From dense planes (semantic validation included).
Err resident_from_planes(int codec, uint32_t group, uint64_t n, uint64_t k,
                         const uint8_t* plane_count, const int8_t* trits, const uint16_t* scales,
                         Resident* out);
// From caller-supplied arenas; re-derives every size and checks codec canonicity and scales.
Err resident_from_arenas(int codec, uint32_t group, uint64_t n, uint64_t k, const uint8_t* payload,
                         size_t payload_len, const uint16_t* scales, size_t scale_count,
                         const uint8_t* map, size_t map_len, uint32_t terminal, Resident* out);
// The arenas as the device holds them.  Two re-layouts let the fast kernels (uniform plane
// counts, k % 256 == 0, groups of 128, B3 or D2) take more artifacts:
//  * S34 (one 5-bit code per four trits) has no tile expander of its own: on such a shape the
//    same trits are stored as B3 (52 instead of 40 bytes per plane of a tile), so every kernel,
//    the bit-exact one included, sees the trits the artifact holds;
//  * a tensor whose tiles hold different plane counts (n >= 16, k <= 65536) gets every tile
//    padded to the largest count by all-zero planes (zero-trit bytes, zero scales); the 2-bit map
//    keeps the true counts (*map_counts), which the bit-exact kernel follows: a zero plane would
//    add +0.0, and that can flip the sign of a zero sum.
// `out` is filled only when *recoded or *map_counts is set; otherwise the input is the layout.
Err device_layout(const Resident& in, Resident* out, bool* recoded, bool* map_counts);
// From package bytes (whole-package validation), tensor selected by name.
Err resident_from_package(const uint8_t* bytes, size_t len, const char* name, Resident* out);
// From a byte source read at arbitrary offsets (a seekable file): the header table is walked, the
// named tensor's sections and its slice of the presence map are fetched, nothing else is read.
// `read_at` returns 0 on success.
using ReadAtFn = int (*)(void* user, uint64_t offset, void* dst, size_t len);
Err resident_from_reader(ReadAtFn read_at, void* user, uint64_t len, const char* name, Resident* out);
// Package bytes for matrix tensors in the given order.
struct PackageTensorIn {
  const char* name; uint32_t group; uint64_t n, k;
  const uint8_t* plane_count; const int8_t* trits; const uint16_t* scales;
};
Err package_write_multi(int codec, const PackageTensorIn* tensors, size_t count, std::vector<uint8_t>* out);
// Package bytes for one matrix tensor.
Err package_write(int codec, const char* name, uint32_t group, uint64_t n, uint64_t k,
                  const uint8_t* plane_count, const int8_t* trits, const uint16_t* scales,
                  std::vector<uint8_t>* out);

// TQ2_0 rows (66-byte blocks) -> a 1-plane D2 resident tensor with unit group scales.
Err resident_from_tq2(const uint8_t* packed, size_t len, uint64_t n, uint64_t k, Resident* out);
Err tq2_pack_rows(const int8_t* trits, uint64_t n, uint64_t k, uint8_t* out);
// TQ1_0 rows (54-byte blocks) -> a 1-plane D2 resident tensor with unit group scales.
Err resident_from_tq1(const uint8_t* packed, size_t len, uint64_t n, uint64_t k, Resident* out);
// SALT V1 plane-major TQ2_0 planes (per-block f16 scales inside the blocks) -> a t-plane D2 resident tensor.
Err resident_from_salt_v1(const uint8_t* packed, size_t len, uint32_t t_planes, uint64_t n, uint64_t k, Resident* out);

// Tensor-parallel shard of a uniform-plane tensor.
struct ShardSizes { uint32_t n = 0, k = 0; uint64_t payload_bytes = 0, scale_count = 0, map_bytes = 0; };
Err shard_sizes(int codec, uint32_t group, uint32_t n, uint32_t k, uint32_t planes, bool row_parallel,
                uint32_t world, uint32_t rank, ShardSizes* out);
Err shard(int codec, uint32_t group, uint32_t n, uint32_t k, uint32_t planes, const uint8_t* payload,
          const uint16_t* scales, bool row_parallel, uint32_t world, uint32_t rank,
          uint8_t* shard_payload, uint16_t* shard_scales, uint8_t* shard_map, uint32_t* terminal);

void quantize_act_int8(const float* act, uint64_t m, uint64_t k, float* q, float* scale);

}  // namespace tbf
