// Internal declarations shared by the C-ABI layer and the kernel translation units.
#pragma once

#include <cuda_runtime.h>

#include <atomic>

#include <cstdint>
#include <string>

#include "../../include/tritium_b200.h"
#include "tb_format.h"

// Device status word layout (uint32 x 8), written by kernels, read by tb_backend_check.
enum : uint32_t {
  TBS_FLAGS = 0,       // bit mask below
  TBS_INFO0 = 1,       // row / stage
  TBS_INFO1 = 2,       // column / barrier id
  TBS_INFO2 = 3,
};
enum : uint32_t {
  TBF_NONFINITE_ACT = 1u,
  TBF_NONFINITE_OUT = 2u,
  TBF_WAIT_TIMEOUT = 4u,
  TBF_BAD_CONFIG = 8u,
};

struct tb_backend {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  cudaDeviceProp prop{};
  char physical_id[96]{};
  uint32_t* d_status = nullptr;   // 8 words
  uint32_t* h_status = nullptr;   // pinned mirror
  // grow-on-demand staging for the host-pointer entry points
  void* d_x = nullptr; size_t d_x_cap = 0;
  void* d_y = nullptr; size_t d_y_cap = 0;
  void* d_aux = nullptr; size_t d_aux_cap = 0;   // act scales / row scales / acc dump
  void* h_pin = nullptr; size_t h_pin_cap = 0;   // pinned bounce buffer
  // scratch for the prefill path: quantised activations (permuted int8) + token scales
  void* d_q = nullptr; size_t d_q_cap = 0;
  // scratch for the decode path: activation tables built by the prepare kernel
  void* d_prep = nullptr; size_t d_prep_cap = 0;
  // normalised activations, for norm+linear calls whose tables the decode kernel does not build itself
  void* d_norm = nullptr; size_t d_norm_cap = 0;
  // fp32 activations split into int8 limbs, their multipliers and the limbs' outputs
  void* d_limb = nullptr; size_t d_limb_cap = 0;
  uint32_t* d_tile_counters = nullptr;   // 256 words, zero between launches (the tensor-core kernel's K splits)
  int max_smem_optin = 0;
  // Weights, stacks and communicators point back at their backend.  tb_backend_free only marks
  // the context released while such objects are alive; the last of them to go destroys it, so that
  // a caller may drop its handles in any order.
  std::atomic<uint32_t> dependants{0};
  std::atomic<bool> released{false};
  uint32_t inject_missing_tx = 0;   // test hook: armed by tb_backend_inject_wait_timeout, used once
};

// How the decode kernel walks one weight tensor (fixed at upload).
struct DecodePlan {
  uint32_t rows_per_stage = 0;   // R: multiple of 4 (16-byte chunks) with R*planes % 16 == 0
  uint32_t row_bytes = 0;        // tiles_per_row * planes * plane_bytes
  uint32_t stage_bytes = 0;      // R * row_bytes
  uint32_t scale_stage_bytes = 0;
  uint32_t blocks = 0;           // ceil(n / R)
};

struct tb_weights {
  tb_backend* owner = nullptr;
  int codec = 0;                 // tbf::Codec
  uint32_t group = 128, uniform_planes = 0;
  // Tiles with different plane counts (aligned shapes only) are stored padded to the largest
  // count with all-zero planes, so that the fast kernels see a uniform tensor: uniform_planes is
  // then that count, and map_counts tells the bit-exact kernel to take each tile's true count
  // from the 2-bit map (a zero plane would add +0.0, which can flip the sign of a zero sum).
  bool map_counts = false;
  uint64_t n = 0, k = 0, tiles = 0, present_planes = 0;
  uint64_t payload_bytes = 0, scale_count = 0, map_bytes = 0, rank_prefix_bytes = 0;
  uint32_t terminal_map = 0;
  uint64_t source_len = 0;
  uint64_t logical_k = 0;        // k the caller sees (TQ2_0 rows are padded to whole blocks)
  bool is_tq2 = false;
  bool fast = false;             // uniform planes, k % 256 == 0, group 128, codec D2/B3
  uint8_t* d_payload = nullptr;  // padded to whole decode stages with zero-trit bytes
  uint16_t* d_scales = nullptr;
  uint8_t* d_meta = nullptr;     // map bytes followed by LE u32 rank prefixes
  uint32_t* d_tile_rank = nullptr;  // planes before each tile (ragged tensors only)
  DecodePlan plan;
};

void tb_set_error(const std::string& message);
void tb_clear_error();
// An object that keeps a pointer to `b` calls retain when it is created and release when it is freed.
void tb_backend_retain(tb_backend* b);
void tb_backend_release(tb_backend* b);
tb_status tb_fail(tb_status code, const std::string& message);
tb_status tb_cuda_fail(cudaError_t err, const char* what);

// ---- kernel launchers (each returns a cudaError_t from the launch) ----
struct ExactArgs {
  const tb_weights* w;
  const float* x; float* y; uint32_t m;
  const float* row_scale;   // nullable
  uint32_t* status;
};
cudaError_t tb_launch_exact(const ExactArgs& a, cudaStream_t stream);
cudaError_t tb_launch_gather_rows(const tb_weights* w, const uint32_t* rows, uint32_t count, float* out,
                                  cudaStream_t stream);
// RMSNorm of m rows of k values into fp32 `out` (canonical 256-slot reduction order).
cudaError_t tb_launch_rmsnorm(const void* x, tb_dtype dtype, const float* weight, float eps, bool zero_centered, uint32_t m,
                              uint32_t k, float* out, cudaStream_t stream);
// The int8 path of layouts without a fast kernel: codes as fp32 values for the exact kernel, and
// the token scale (and residual) applied to its output.
cudaError_t tb_launch_quantize_to_float(const void* x, tb_dtype dtype, uint32_t m, uint32_t k, float* q, float* act_scale, uint32_t* status,
                                        cudaStream_t stream);
// fp32 activations through the int8 kernels: four int8 limbs per element (pseudo-tokens 4t..4t+3
// with their own dequantisation multipliers), and the sum of the four outputs of a token.
cudaError_t tb_launch_limb_split(const float* x, uint32_t m, uint32_t k, int8_t* q, float* act_scale, uint32_t* status, cudaStream_t stream);
cudaError_t tb_launch_limb_sum(const float* y4, uint32_t m, uint32_t n, float* y, cudaStream_t stream);
cudaError_t tb_launch_scale_tokens(const float* y, const float* act_scale, const float* residual, uint32_t m, uint32_t n, void* out,
                                   tb_dtype out_dtype, cudaStream_t stream);
cudaError_t tb_launch_row_absmax(const void* x, tb_dtype dtype, uint32_t m, uint32_t k, float* out, cudaStream_t stream);
cudaError_t tb_launch_check_finite(const float* x, uint64_t count, uint32_t* status, cudaStream_t stream);

// One slot of a peer-memory communicator as the kernels see it: every rank's copy of the slot and of
// its flag words (this rank's own pointers at index `rank`).  world <= 1 means "no peers".
// Flag words of a slot: [0,8) one-shot flags, 8 epoch, 9 block counter (one-shot reduce);
// 10 epoch, 11 block counter (fused kernels); 16.. arrival counters, one per token or row block.
// 12 epoch, 13 block counter (exchanges inside the decode kernel).
constexpr uint32_t kCommMaxWorld = 8, kCommFusedEpoch = 10, kCommFusedDone = 11, kCommDecodeEpoch = 12, kCommDecodeDone = 13,
                   kCommCounters = 16;
// Byte offset, inside the absmax slot, of the words the decode kernel's absmax exchange uses:
// uint64 [round parity][source rank][token] = (round << 32) | float bits.
// (the decode kernel's words first, then the preparation kernel's: the two count rounds separately)
constexpr uint32_t kCommAbsmaxWords = 64, kCommAbsmaxWordsPrepare = kCommAbsmaxWords + 2 * kCommMaxWorld * 4 * 8,
                   kCommAbsmaxBytes = kCommAbsmaxWordsPrepare + 2 * kCommMaxWorld * 4 * 8;
struct TbCommView {
  float* data[kCommMaxWorld];
  uint32_t* flags[kCommMaxWorld];
  uint32_t world, rank, counters;   // counters: arrival counters the slot's flag area holds
  long long wait_cycles;            // bound of every wait on a peer, in SM clocks
};

// Device-resident descriptor of one layer of a grouped launch.
struct TbLayerDesc { const uint8_t* payload; const uint16_t* scales; };

struct DecodeArgs {
  const tb_weights* w;
  const void* x; tb_dtype x_dtype; const float* act_scale_in; const float* act_absmax_in;
  uint32_t m;                 // 1..4 tokens per launch
  void* y; tb_dtype y_dtype; uint32_t y_row_stride;  // elements between tokens in y
  int32_t* acc_dump; uint32_t dump_token_offset, dump_tokens_total;
  const float* row_scale;
  uint32_t* status;
  bool pdl;
  // fused: the decode kernel quantises x and builds its activation tables itself (x 16-byte
  // aligned; no scratch, no prepare launch).  Otherwise the tables come from `scratch`, which
  // tb_launch_prepare filled on the same stream.
  bool fused;
  void* scratch; size_t scratch_bytes;   // activation tables (written by the prepare kernel)
  bool tables_shared;   // the tables in scratch were prepared for an earlier launch of the same input
  // grouped launch: `layer_count` layers shaped like `w` read the same activations; outputs are
  // written as [layer][m][n] with `y_layer_stride` elements between layers
  const TbLayerDesc* layers; uint32_t layer_count; uint32_t y_layer_stride;
  // tensor-parallel row shard (single layer): the prepare kernel exchanges the per-token absmax
  // through `comm_absmax`.  Null = no peers.
  const TbCommView* comm_absmax;
  // Row shard whose outputs are summed over the ranks inside the decode kernel: every CTA pushes
  // its partial rows, each value tagged with the round, into all ranks' copies of this slot, and
  // sums a row block once all ranks' values of this round have arrived.  Fused launches exchange the absmax the same
  // way (through comm_absmax).  Null = no peers.  Every rank must make the same launch.
  const TbCommView* comm_y;
  uint32_t inject_missing_tx;   // test hook (non-fused launches): the table barrier expects this many bytes too many
  // fused launches: RMSNorm over each token's row in front of the quantiser (weight [k] fp32,
  // 16-byte aligned; null = none).  Any launch: out = residual + y (fp32, indexed like y).
  const float* norm_weight; float norm_eps; bool norm_zero_centered;
  const float* residual;
  // squared-ReLU gate in front of the quantiser (fp32 x = gate projection, relu2_up = up
  // projection, both [m][k]; 16-byte aligned for fused launches; not together with the norm)
  const float* relu2_up;
};
cudaError_t tb_launch_prepare(const DecodeArgs& a, cudaStream_t stream);
// Whether a decode launch of `m` tokens should build its activation tables itself (one launch)
// rather than read them from scratch that tb_launch_prepare filled.  Every CTA repeats the
// construction, so this pays only for small tables; x must be 16-byte aligned.
bool tb_decode_builds_tables(const tb_weights* w, uint32_t m, const void* x);
size_t tb_decode_scratch_bytes(const tb_weights* w, uint32_t m);
// Returns false (and leaves *err untouched) when the layout/shape does not fit the kernel.
bool tb_decode_supported(const tb_weights* w, uint32_t m, int max_smem, size_t* smem_bytes);
cudaError_t tb_launch_decode(const DecodeArgs& a, int sm_count, int max_smem, cudaStream_t stream);
void tb_make_decode_plan(tb_weights* w, int max_smem);

struct PrefillArgs {
  const tb_weights* w;
  const void* x; tb_dtype x_dtype; const float* act_scale_in; const float* act_absmax_in;
  uint32_t m;
  void* y; tb_dtype y_dtype;
  int32_t* acc_dump;
  const float* row_scale;
  void* scratch; size_t scratch_bytes;   // permuted int8 activations, slab start values, token scales
  uint32_t* status;
  const float* residual = nullptr;       // [m][n] fp32, nullable: out = residual + y
  const float* relu2_up = nullptr;       // squared-ReLU gate: activation = (max(x, 0)^2) * relu2_up (x fp32)
  uint32_t* tile_counters = nullptr;     // 256 zeroed words (few-token launches split K and count the splits of a tile in)
};
bool tb_prefill_supported(const tb_weights* w, uint32_t m);
size_t tb_prefill_scratch_bytes(const tb_weights* w, uint32_t m);
cudaError_t tb_launch_prefill(const PrefillArgs& a, int sm_count, cudaStream_t stream);

// peer-memory communicator (kernels_comm.cu)
struct tb_comm;
bool tb_comm_view(const tb_comm* c, uint32_t slot, TbCommView* out);
size_t tb_comm_slot_bytes(const tb_comm* c);
const tb_backend* tb_comm_owner(const tb_comm* c);
