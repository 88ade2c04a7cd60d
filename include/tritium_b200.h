/*
 * tritium_b200 — C ABI of the B200 (sm_100a) backend for Tritium's packed additive-ternary
 * linear layer  Y = X · Σ_p diag(s_p)·T_p.
 *
 * Conventions follow the reference project's own C ABI (crates/tritium-ffi/src/lib.rs:8-26,
 * 42-75,82-100,362-376): every fallible call returns a tb_status (TB_OK == 0); the message of
 * the last failure on the calling thread is kept in thread-local storage and returned by
 * tb_last_error() until the next call on that thread; handles are opaque, owned by the caller
 * and released by a null-safe *_free; every pointer is null-checked; nothing unwinds across
 * the boundary.  A handle may move between threads but must not be used from two threads at
 * once.  Status codes mirror BackendError (crates/tritium-spec/src/lib.rs:384-405).
 *
 * There is no CPU fallback: every compute entry point fails with TB_BACKEND when no CUDA
 * device is present.  Host-side format helpers (tb_fmt_*) run anywhere.
 */
#ifndef TRITIUM_B200_H
#define TRITIUM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB_ABI_VERSION 1u

typedef enum tb_status {
  TB_OK = 0,
  TB_NULL_ARG = 1,
  TB_SHAPE_MISMATCH = 2,     /* BackendError::ShapeMismatch */
  TB_UNSUPPORTED_FORMAT = 3, /* BackendError::UnsupportedFormat */
  TB_OUT_OF_MEMORY = 4,      /* BackendError::OutOfMemory */
  TB_INVALID_INPUT = 5,      /* BackendError::InvalidInput */
  TB_BACKEND = 6,            /* BackendError::Backend (driver / device failure) */
  TB_TIMEOUT = 7             /* a bounded device-side wait gave up; the context stays usable */
} tb_status;

/* Codec tags as written in a package header (crates/tritium-format/src/salt_v2_package.rs:2747-2762). */
typedef enum tb_codec { TB_CODEC_D2 = 1, TB_CODEC_B3 = 2, TB_CODEC_S34 = 3 } tb_codec;

typedef enum tb_dtype { TB_F32 = 0, TB_BF16 = 1, TB_I8 = 2 } tb_dtype;

typedef struct tb_backend tb_backend;
typedef struct tb_weights tb_weights;
typedef struct tb_stack tb_stack;

/* DeviceCaps (crates/tritium-spec/src/caps.rs:7-68). */
typedef struct tb_caps {
  char backend[16];      /* "b200" */
  char device_name[128];
  char device_id[32];    /* "b200:<ordinal>" */
  char physical_id[96];  /* "b200:<ordinal>:GPU-<uuid>" */
  char features[192];    /* comma separated: sm_100a,salt_v2_d2,salt_v2_b3,salt_v2_s34,tq2_0,int8_tcgen05 */
  uint64_t total_memory_bytes;
  uint32_t sm_count;
  uint32_t supports_imma;
  uint32_t supports_fp8;
} tb_caps;

/* Byte receipt of one forward call: the algorithmic bytes the call had to move
 * (SaltV2ForwardReceipt, crates/tritium-cuda/src/cuda/backend.rs:321-405).  dense_weight_bytes
 * is always 0: no dequantised weight copy exists on the device. */
typedef struct tb_receipt {
  uint64_t payload_bytes, scale_bytes, map_bytes, rank_prefix_bytes;
  uint64_t activation_bytes, output_bytes, dense_weight_bytes;
  uint32_t kernel; /* 0 exact, 1 decode (mma.sync), 2 prefill (tcgen05) */
  uint32_t launches;
} tb_receipt;

typedef struct tb_weights_info {
  uint32_t codec, group, planes_uniform; /* codec: the codec resident on the device (an S34 artifact on a
                                            256-aligned g128 shape is stored as B3 with the same trits);
                                            planes_uniform: plane slots per tile as stored on the device, 1..3
                                            (tiles with fewer planes on a 256-aligned B3/D2 g128 shape are padded
                                            with zero planes to the largest count), or 0 for the ragged layout */
  uint64_t n, k, tiles, present_planes;
  uint64_t payload_bytes, scale_bytes, map_bytes, rank_prefix_bytes;
  uint64_t source_len_bytes; /* DeviceBuffer::len_bytes(): the caller's packed input length */
  uint32_t fast_path;        /* 1 when the decode/prefill kernels accept this layout */
} tb_weights_info;

/* ------------------------------------------------------------------ library */
uint32_t tb_abi_version(void);
const char* tb_last_error(void);
/* The two lengths of the calling thread's last failure when it was a TB_SHAPE_MISMATCH that knows
 * them (BackendError::ShapeMismatch { expected, got }, crates/tritium-spec/src/lib.rs:384-391;
 * callers such as crates/tritium-nn/src/layers/projection.rs:207-209 match on the variant).
 * Returns TB_INVALID_INPUT when the last failure carries no lengths. */
tb_status tb_last_shape_mismatch(uint64_t* expected, uint64_t* got);

/* ------------------------------------------------------------------ backend
 * Replaces CudaBackend::new / the BackendEntry init function
 * (crates/tritium-cuda/src/cuda/backend.rs:9087-9100, crates/tritium-runtime/src/lib.rs:74-86).
 * Returns TB_BACKEND (never aborts) when no device exists. */
tb_status tb_backend_create(int ordinal, tb_backend** out);
/* Handles may be dropped in any order (a Rust binding's Drop order is the owner's, not ours):
 * while weights, stacks or communicators of this backend are alive, tb_backend_free only marks
 * the context released (every later call on it fails with TB_INVALID_INPUT, except the free calls
 * of its objects) and the last of those objects to be freed destroys it. */
void tb_backend_free(tb_backend* backend);
/* TernaryBackend::capabilities (crates/tritium-spec/src/lib.rs:166-185). */
tb_status tb_backend_caps(const tb_backend* backend, tb_caps* out);
tb_status tb_backend_synchronize(tb_backend* backend);

/* ------------------------------------------------------------------ weights
 * TernaryBackend::upload_weights for TernaryFormat::Tq2_0 (crates/tritium-spec/src/lib.rs:186-199,
 * crates/tritium-cuda/src/cuda/backend.rs:8581-8650).  `len` must equal n*ceil(k/256)*66. */
tb_status tb_tq2_upload(tb_backend* backend, const uint8_t* packed, size_t len, uint32_t n,
                        uint32_t k, tb_weights** out);
/* The same for TernaryFormat::Tq1_0 (54-byte blocks, crates/tritium-format/src/tq1.rs:16-122; the
 * reference's kernels for it: crates/tritium-cuda/kernels/tq2_0_add.cu:796-913).  `len` must equal
 * n*ceil(k/256)*54.  The handle runs through tb_mpgemm / tb_mpgemm_with_act_quant like a TQ2_0 one. */
tb_status tb_tq1_upload(tb_backend* backend, const uint8_t* packed, size_t len, uint32_t n,
                        uint32_t k, tb_weights** out);
/* SALT V1 multi-plane weights: `t_planes` (1..3) plane-major TQ2_0 planes [t][n][ceil(k/256)*66]
 * whose f16 block scale is the plane's scale for that block; W = sum_p scale_p * trit_p.  Replaces
 * the upload behind salt_mpgemm_tiled_f32 (crates/tritium-cuda/kernels/tq2_0_add.cu:640-719, host
 * crates/tritium-cuda/src/cuda/backend.rs:7807-7811) and PackedSaltMatrix
 * (crates/tritium-nn/src/layers/packed_salt.rs:612-678).  The handle then runs through the same
 * forward entry points: tb_linear_forward_a8 is SaltLinear::forward (layers/salt.rs:114-147: quantise,
 * project, scale), tb_linear_forward_f32 the kernel's fp32-activation form.  Rows are padded to whole
 * 256-blocks with zero trits: activations and info.k use the padded width. */
tb_status tb_salt_v1_upload(tb_backend* backend, const uint8_t* planes, size_t len, uint32_t t_planes,
                            uint32_t n, uint32_t k, tb_weights** out);
/* CudaBackend::upload_salt_v2 (crates/tritium-cuda/src/cuda/backend.rs:7463-7651), taking the
 * resident arenas: payload (tile-major then plane), f16 scale bits, the runtime plane map
 * (2 bits per tile, value planes-1) and its terminal partial byte.  Sizes are re-derived from
 * (n, k, group, map) and compared. */
tb_status tb_salt_v2_upload(tb_backend* backend, tb_codec codec, uint32_t group, uint32_t n,
                            uint32_t k, const uint8_t* payload, size_t payload_len,
                            const uint16_t* scales, size_t scale_count, const uint8_t* plane_map,
                            size_t map_len, uint32_t terminal_map_value, tb_weights** out);
/* CudaBackend::upload_salt_v2_from_reader (crates/tritium-cuda/src/cuda/backend/salt_v2_reader_upload.rs:32):
 * whole package bytes plus a tensor name. */
tb_status tb_salt_v2_upload_package(tb_backend* backend, const uint8_t* package, size_t len,
                                    const char* tensor_name, tb_weights** out);
/* The same from a byte source that is read at arbitrary offsets (a seekable file), so that a
 * multi-gigabyte package is never held in memory: SaltV2PackageReader::new_strict / tensor_info /
 * visit_packed_tensor (crates/tritium-format/src/salt_v2_package/reader.rs:333,790,841) as used by
 * upload_salt_v2_from_reader (crates/tritium-cuda/src/cuda/backend/salt_v2_reader_upload.rs:32).  The
 * header table is walked with small reads; only the named tensor's payload, scales and its slice of
 * the presence map are fetched.  `read_at` copies `len` bytes at `offset` into `dst` and returns 0,
 * or non-zero on failure (reported as TB_INVALID_INPUT).  `package_len` is the source's length. */
typedef int (*tb_read_at_fn)(void* user, uint64_t offset, void* dst, size_t len);
tb_status tb_salt_v2_upload_reader(tb_backend* backend, tb_read_at_fn read_at, void* user, uint64_t package_len,
                                   const char* tensor_name, tb_weights** out);
tb_status tb_weights_info_get(const tb_weights* weights, tb_weights_info* out);
void tb_weights_free(tb_weights* weights);

/* ------------------------------------------------------------------ forward, host pointers
 * CudaBackend::salt_v2_forward_exact_into (crates/tritium-cuda/src/cuda/backend/salt_v2_runtime.rs:212-381):
 * fp32 activations [m,k] -> fp32 [m,n], bit-identical to the CPU reference order
 * (crates/tritium-cpu/src/salt_v2.rs:316-423).  Non-finite activations and outputs are rejected
 * as TB_INVALID_INPUT and `y` is left untouched on any error. */
tb_status tb_salt_v2_forward_exact(tb_backend* backend, const tb_weights* weights, const float* x,
                                   uint32_t m, float* y, tb_receipt* receipt);
/* CudaBackend::salt_v2_forward_fast (backend.rs:7672-7687): same contract, reassociated sums; not
 * bit-exact but within 1e-5 relative L2.  Tensors with a fast kernel run every fp32 activation as
 * four int8 limbs relative to its token's absmax (representation error below 2e-9 of the absmax)
 * through the int8 kernels, exact int32 sums per limb; other layouts run the bit-exact kernel. */
tb_status tb_linear_forward_f32(tb_backend* backend, const tb_weights* weights, const float* x,
                                uint32_t m, float* y, tb_receipt* receipt);
/* The fused W1.58A8 path (TernaryBackend::mpgemm_with_act_quant, crates/tritium-spec/src/lib.rs:266-318,
 * applied to the SALT V2 contraction): per-token absmax int8 quantisation, exact int32
 * contraction per (scale group, plane), fold of f16 group scales and the token scale.
 * `x` is [m,k] of x_dtype; `y` is [m,n] of y_dtype (TB_F32 or TB_BF16).  `acc_dump`, when not
 * NULL, receives the int32 accumulators as [m][n][k/group][planes]. */
tb_status tb_linear_forward_a8(tb_backend* backend, const tb_weights* weights, const void* x,
                               tb_dtype x_dtype, uint32_t m, void* y, tb_dtype y_dtype,
                               int32_t* acc_dump, tb_receipt* receipt);
/* CudaBackend::salt_v2_gather_rows (backend.rs:7689-7701, kernels/salt_v2.cu:221-304). */
tb_status tb_salt_v2_gather_rows(tb_backend* backend, const tb_weights* weights,
                                 const uint32_t* rows, size_t row_count, float* out);

/* ------------------------------------------------------------------ forward, device pointers
 * Same operators on device memory, launched on `stream` (a cudaStream_t, NULL = the backend's
 * stream) without any host synchronisation or allocation beyond the backend's own scratch.
 * The backend's stream is non-blocking: work on it is NOT ordered with the legacy default stream.
 * A caller whose tensors are produced on the default stream passes cudaStreamLegacy (the handle
 * 0x1), not NULL, and keeps every buffer of a call alive until the stream has run it.
 * flags: */
#define TB_FWD_A8 1u          /* int8-quantise activations (x_dtype F32 or BF16), or consume int8 */
#define TB_FWD_EXACT 2u       /* force the bit-exact kernel (fp32 activations only) */
#define TB_FWD_PDL 4u         /* launch with programmatic dependent launch (weights prefetch early) */
#define TB_FWD_FORCE_DECODE 8u   /* streaming kernel whatever m; TB_UNSUPPORTED_FORMAT when a row block does not fit */
#define TB_FWD_FORCE_PREFILL 16u /* tensor-core kernel whatever m */
/* Without a force flag: up to 8 tokens take the streaming (decode) kernel, more the tensor-core
 * kernels; a tensor whose rows are too long for the streaming kernel's shared-memory ring takes the
 * tensor-core kernel at every m (so a device-pointer caller reserves with tb_backend_reserve). */
typedef struct tb_forward_args {
  const void* x;            /* [m,k] device */
  tb_dtype x_dtype;
  const float* act_scale;   /* [m] device; dequantisation multiplier, required when x_dtype == TB_I8 */
  const float* act_absmax;  /* [m] device, nullable: per-token max|x| over the FULL row; a
                               row-parallel shard passes the global value so that its int8
                               codes equal the unsharded ones */
  uint32_t m;
  void* y;                  /* [m,n] device */
  tb_dtype y_dtype;
  int32_t* acc_dump;        /* device, nullable */
  const float* row_scale;   /* [n] device, nullable: per-output-channel scale (trait path) */
  uint32_t flags;
  void* stream;
} tb_forward_args;
tb_status tb_linear_forward_dev(tb_backend* backend, const tb_weights* weights,
                                const tb_forward_args* args, tb_receipt* receipt);
/* The decode block's fused step around a packed linear, on device pointers: RMSNorm in front of
 * the int8 quantiser and `residual + y` behind the token scale.  Replaces the reference's
 * rmsnorm_quant_i8 launch in front of its int8 GEMV (crates/tritium-cuda/kernels/decode.cu:533-640;
 * arithmetic of crates/tritium-nn/src/ops/rmsnorm.rs:20-94, including the canonical 256-slot
 * reduction order, so the int8 codes equal the reference's) and the residual epilogue of its
 * TQ2_0 kernels (crates/tritium-cuda/kernels/tq2_0_add.cu:577-637: one rounding for
 * residual + acc * scale).  Up to four tokens with small activation tables run as ONE launch
 * (the norm happens inside the decode kernel's table builder); other shapes normalise with a
 * kernel of their own into backend scratch, which the first such call of a size allocates.
 *   norm_weight NULL = no norm (residual epilogue only); residual NULL = none; relu2_up: the MLP's
 *   squared-ReLU gate in front of the down projection (see the field).
 *   x fp32 or bf16 (bf16 is widened exactly); norm_weight fp32 [k]; residual fp32 [m][n]. */
#define TB_NORM_ZERO_CENTERED 1u   /* scale by (1 + w): rmsnorm_zero_centered, rmsnorm.rs:49-63 */
typedef struct tb_norm_linear_args {
  const void* x;             /* [m,k] device */
  tb_dtype x_dtype;
  const float* norm_weight;  /* [k] device, nullable */
  float norm_eps;
  uint32_t norm_flags;
  const float* residual;     /* [m,n] device fp32, nullable; may alias y only when y is fp32 */
  uint32_t m;
  void* y;                   /* [m,n] device */
  tb_dtype y_dtype;
  uint32_t flags;            /* TB_FWD_PDL, TB_FWD_FORCE_DECODE, TB_FWD_FORCE_PREFILL */
  void* stream;
  const float* relu2_up;     /* [m,k] device fp32, nullable: squared-ReLU gate in front of the quantiser.
                                x then holds the gate projection's fp32 output, relu2_up the up
                                projection's, and the linear's input is (max(x,0)^2) * relu2_up, the
                                reference's relu2_gate_f32 (crates/tritium-cuda/kernels/decode.cu:772-780),
                                computed where the activations are quantised: no launch of its own.
                                Not together with norm_weight. */
} tb_norm_linear_args;
tb_status tb_norm_linear_forward_dev(tb_backend* backend, const tb_weights* weights,
                                     const tb_norm_linear_args* args, tb_receipt* receipt);
/* No counterpart in the reference: an int8-path forward (1..4 tokens, device pointers) for
 * callers that are not allowed to allocate device memory while they run — a serving loop whose
 * memory is fully planned up front, a latency-critical thread that must not enter the driver's
 * allocator (cudaMalloc and cudaFree serialise the whole device), or code that runs while every
 * byte of HBM is already spoken for.  This call performs no cudaMalloc, cudaFree or any other
 * allocating call: its only working memory, the activation tables, sits in a fixed 256 KiB array
 * that is part of the library image on every GPU that loads it (held until the process exits).
 *   - Shapes whose tables do not fit (roughly m * k above 40k elements for B3, m <= 4 always) are
 *     refused with TB_INVALID_INPUT and a message that states both sizes.
 *   - The first call on a device looks up the array's device address; make that first call
 *     before starting any stream capture, and from one thread.
 *   - All calls share the one array.  Each call rewrites every table entry it later reads, so
 *     nothing has to be cleared, but two calls that overlap on the GPU (different streams, or the
 *     same stream with programmatic overlap) race on it: keep them ordered.
 * `act_scale` is needed only for int8 activations.  Results equal tb_linear_forward_dev with
 * TB_FWD_A8.  Timeouts and finite checks are reported by tb_backend_check as usual. */
tb_status tb_linear_forward_a8_static(tb_backend* backend, const tb_weights* weights, const void* x,
                                      tb_dtype x_dtype, const float* act_scale, uint32_t m, void* y,
                                      tb_dtype y_dtype, void* stream);
/* Per-token max|x| of `x` [m,k] (fp32 or bf16, device) into `out` [m] (fp32, device).  A
 * row-parallel shard runs this on its slice of the activations, takes the maximum over the
 * tensor-parallel group and passes the result as `act_absmax`, which reproduces the
 * quantisation scale of quantize_act_int8 over the whole row
 * (crates/tritium-spec/src/lib.rs:351-378; no sharded counterpart exists in the reference). */
tb_status tb_act_absmax_dev(tb_backend* backend, const void* x, tb_dtype x_dtype, uint32_t m, uint32_t k,
                            float* out, void* stream);
/* Reserves the backend's device scratch for `weights` at up to `max_m` tokens, so that later
 * tb_linear_forward_dev calls allocate nothing. */
tb_status tb_backend_reserve(tb_backend* backend, const tb_weights* weights, uint32_t max_m);
/* Reads and clears the device status word written by bounded waits / finite checks. */
tb_status tb_backend_check(tb_backend* backend, void* stream);
/* Test hook, no counterpart in the reference: when `enable` is non-zero, the NEXT
 * tb_linear_forward_a8_static call makes its kernel wait for table bytes that nobody sends.  The
 * bounded wait runs out (about two seconds), the kernel returns by itself, tb_backend_check
 * reports TB_TIMEOUT, and the context stays usable.  Nothing faults, traps or spins without a
 * limit.  The hook disarms itself after that one call. */
tb_status tb_backend_inject_wait_timeout(tb_backend* backend, uint32_t enable);

/* ------------------------------------------------------------------ trait path (1 plane, per-channel scale)
 * TernaryBackend::mpgemm (crates/tritium-spec/src/lib.rs:200-215; host crates/tritium-cuda/src/cuda/backend.rs:7175-7315)
 * out[m,n] = scales[n] · Σ_k act[m,k]·w[n,k].  Integer-valued activations in [-128,127] take the
 * exact int8 kernel (as crates/tritium-cpu/src/kernel.rs:833-837 does); others the fp32 kernel. */
tb_status tb_mpgemm(tb_backend* backend, const tb_weights* weights, const float* act,
                    const float* scales, uint32_t m, uint32_t n, uint32_t k, float* out);
/* TernaryBackend::mpgemm_with_act_quant (lib.rs:216-318; CUDA override backend.rs:8868-8954). */
tb_status tb_mpgemm_with_act_quant(tb_backend* backend, const tb_weights* weights,
                                   const float* act, const float* scales, uint32_t m, uint32_t n,
                                   uint32_t k, float* out);

/* ------------------------------------------------------------------ layer stack (decoder linears)
 * A sequence of resident linears run back to back on one stream, each layer's weight stream
 * overlapping the previous layer's tail.  `weights[i]` consumes the output of layer i-1 when
 * chain[i] != 0, else the stack input.  Used by the 2B / 27B stack configurations. */
tb_status tb_stack_create(tb_backend* backend, const tb_weights* const* weights,
                          const uint8_t* chain, uint32_t layers, uint32_t max_m, tb_stack** out);
tb_status tb_stack_forward_dev(tb_stack* stack, const void* x, tb_dtype x_dtype, uint32_t m,
                               void* y_last, tb_dtype y_dtype, uint32_t flags, void* stream);
/* Host-pointer pass over a stack whose layers all read the stack input (up to 4 tokens): x in,
 * every layer's bf16 output out as [layer][m][n]; one synchronisation; `y_bf16` is written only
 * on success.  No counterpart in the reference: it replaces one tb_linear_forward_a8 call per
 * projection when several projections (a QKV or gate/up group) read the same activations. */
tb_status tb_stack_forward_host(tb_stack* stack, const void* x, tb_dtype x_dtype, uint32_t m, void* y_bf16, uint32_t flags);
uint64_t tb_stack_bytes_per_step(const tb_stack* stack, uint32_t m);
/* Consecutive unchained layers of one geometry form a group that runs as a single launch;
 * their bf16 outputs ([m][n] per layer) are read back with this call (synchronises). */
tb_status tb_stack_read_output(tb_stack* stack, uint32_t layer, uint32_t m, void* out_bf16);
void tb_stack_free(tb_stack* stack);

/* ------------------------------------------------------------------ tensor-parallel reduce over peer memory
 * No counterpart in the reference (its only collective is the host-staged NCCL gradient
 * all-reduce, crates/tritium-cuda/src/nccl.rs:530-625).  A communicator owns `slots` buffers of
 * `slot_bytes` on this rank's GPU; the ranks of one node exchange the 64-byte handles
 * (tb_comm_export -> all-gather by any means -> tb_comm_connect) and then reduce a slot with one
 * kernel launch that reads every rank's copy with plain peer loads: the row-parallel kernel
 * writes its fp32 partial outputs straight into tb_comm_slot(), tb_comm_allreduce_f32 combines
 * them in rank order into `out` (local device memory).  Waits on peers are bounded; a peer that
 * does not arrive is reported as TB_TIMEOUT by tb_backend_check.  A slot's content may be
 * rewritten only after a later reduce on the same communicator has been launched behind it. */
#define TB_COMM_HANDLE_BYTES 64
typedef struct tb_comm tb_comm;
tb_status tb_comm_create(tb_backend* backend, uint32_t world, uint32_t rank, size_t slot_bytes, uint32_t slots,
                         uint32_t counters_per_slot, tb_comm** out);
tb_status tb_comm_export(const tb_comm* comm, uint8_t* handle_out /* TB_COMM_HANDLE_BYTES */);
tb_status tb_comm_connect(tb_comm* comm, const uint8_t* all_handles /* world x TB_COMM_HANDLE_BYTES */);
void* tb_comm_slot(const tb_comm* comm, uint32_t slot);
tb_status tb_comm_allreduce_f32(tb_comm* comm, uint32_t slot, uint32_t count, int op_max, float* out, void* stream);
/* Row-parallel int8 forward (1..8 tokens, at most four per launch), with both exchanges inside
 * the kernels:
 *   - the per-token absmax, so that every shard quantises with the scale of the whole row: each
 *     rank pushes its slice's value, tagged with the round number, into the peers' copies of
 *     `slot_absmax` and finds the peers' values in its own memory (small activation tables: inside
 *     the decode kernel's table builder; large ones: in the preparation kernel);
 *   - the output sum: every CTA pushes its fp32 partial rows into all ranks' copies of `slot_y`
 *     and, once the peers' partials of a row block have arrived, adds them in rank order and
 *     stores `y` (fp32 or bf16; every rank ends with the same bits of the full result).
 * Every value travels with its round number in one 8-byte word, so the exchanges need no flag,
 * no fence and no second kernel: a row-parallel linear with small tables is ONE launch.  Only
 * plain peer stores (and loads of the rank's own memory) are used.  `slot_y` must hold
 * 2 x world x min(m,4) x n 8-byte words, `slot_absmax` 2 KiB.  flags: 0 or TB_FWD_PDL.
 * Every rank must make the same call (same m) on its shard; the two slots belong to this linear
 * alone; use tb_comm_allreduce_f32 on them only after every rank has gone idle (a host barrier).  After a TB_TIMEOUT the
 * round counters of the ranks no longer agree: free the communicator and build a new one. */
tb_status tb_linear_forward_tp_dev(tb_backend* backend, const tb_weights* weights, tb_comm* comm, uint32_t slot_absmax,
                                   uint32_t slot_y, const void* x, tb_dtype x_dtype, uint32_t m, void* y, tb_dtype y_dtype,
                                   uint32_t flags, void* stream);
/* The same with the block's fused steps of tb_norm_linear_args: `relu2_up` (the squared-ReLU gate
 * acts on this rank's slice of the row: x and relu2_up are the local shards of the gate and up
 * projections' outputs) and `residual` (added once, behind the sum over the ranks, so every rank
 * stores the same bits).  `norm_weight` must be NULL: RMSNorm acts on the whole row and belongs in
 * front of the column-parallel linear.  At most 8 tokens; flags: 0 or TB_FWD_PDL. */
tb_status tb_block_linear_forward_tp_dev(tb_backend* backend, const tb_weights* weights, tb_comm* comm, uint32_t slot_absmax,
                                         uint32_t slot_y, const tb_norm_linear_args* args);
/* Bound of every wait on a peer, in SM clock cycles (default 4e9, about two seconds).  A wait
 * that runs out sets the backend's status word (TB_TIMEOUT at the next tb_backend_check) and the
 * kernel returns; nothing traps. */
tb_status tb_comm_set_wait_limit(tb_comm* comm, uint64_t sm_cycles);
/* Teardown across ranks, in this order: (1) every rank synchronises its device and meets the
 * others at a host barrier, so that no kernel anywhere still reads or writes peer memory;
 * (2) every rank calls tb_comm_disconnect, which unmaps the peers' buffers; (3) a second host
 * barrier; (4) tb_comm_free releases this rank's buffer.  Freeing a buffer that a peer still has
 * mapped, or is still reading, is an error the library cannot detect.  tb_comm_free alone
 * performs (2) and (4) for this rank and is enough for world == 1. */
tb_status tb_comm_disconnect(tb_comm* comm);
void tb_comm_free(tb_comm* comm);

/* ------------------------------------------------------------------ tensor-parallel sharding (host)
 * Cuts one tensor's resident arenas into the shard for `rank` of `world`:
 * column-parallel (split n; QKV, gate/up) or row-parallel (split k; O, down).  Row-parallel
 * shards are re-encoded so that each shard is itself a valid [n, k/world] tensor.  Output
 * buffers are sized by tb_tp_shard_sizes. */
typedef struct tb_shard_sizes {
  uint32_t n, k;
  uint64_t payload_bytes, scale_count, map_bytes;
} tb_shard_sizes;
tb_status tb_tp_shard_sizes(tb_codec codec, uint32_t group, uint32_t n, uint32_t k, uint32_t planes,
                            int row_parallel, uint32_t world, uint32_t rank, tb_shard_sizes* out);
tb_status tb_tp_shard(tb_codec codec, uint32_t group, uint32_t n, uint32_t k, uint32_t planes,
                      const uint8_t* payload, const uint16_t* scales, int row_parallel,
                      uint32_t world, uint32_t rank, uint8_t* shard_payload,
                      uint16_t* shard_scales, uint8_t* shard_map, uint32_t* shard_terminal);

/* ------------------------------------------------------------------ host format helpers
 * Byte-for-byte the tritium-format layouts; no device needed. */
/* pack_d2/pack_b3/pack_s34 and unpack_* (crates/tritium-format/src/salt_v2.rs:268-482).
 * tb_fmt_pack returns bytes written (negative tb_status on error; out may be NULL to size). */
int64_t tb_fmt_pack(tb_codec codec, const int8_t* trits, size_t n, uint8_t* out, size_t cap);
tb_status tb_fmt_unpack(tb_codec codec, const uint8_t* packed, size_t len, size_t n, int8_t* trits);
size_t tb_fmt_plane_bytes(tb_codec codec, size_t logical_len);
/* Builds the resident arenas from dense planes: trits[(tile*3+p)*256+e], scales[(tile*3+p)*4+g]
 * (f16 bits), plane_count[tile]; validates the semantic rules of
 * salt_v2_package.rs:130-187,222-251,582-641.  Sizes come from tb_fmt_resident_sizes. */
typedef struct tb_resident_sizes {
  uint64_t payload_bytes, scale_count, map_bytes, rank_prefix_bytes, tiles, present_planes;
} tb_resident_sizes;
tb_status tb_fmt_resident_sizes(tb_codec codec, uint32_t group, uint64_t n, uint64_t k,
                                const uint8_t* plane_count, tb_resident_sizes* out);
tb_status tb_fmt_resident_build(tb_codec codec, uint32_t group, uint64_t n, uint64_t k,
                                const uint8_t* plane_count, const int8_t* trits,
                                const uint16_t* scales, uint8_t* payload, uint16_t* scale_out,
                                uint8_t* plane_map, uint32_t* terminal_map_value);
/* Host-only twin of the re-layout the uploads apply: the payload and scale arenas as the device
 * holds them.  They are the artifact's own, except that (a) an S34 tensor on a shape the fast
 * kernels take (k % 256 == 0, groups of 128) is stored as B3 with the same trits, and (b) a
 * tensor whose tiles hold different plane counts on such a shape (n >= 16, k <= 65536) has
 * every tile padded to the largest count by all-zero planes (zero-trit bytes, zero scales; the
 * plane map keeps the true counts).  Call with NULL output buffers to learn the sizes. */
typedef struct tb_device_layout {
  uint32_t codec, planes_uniform; /* as resident: codec tag; plane slots per tile, 0 for the ragged layout */
  uint32_t recoded;               /* 1 when S34 was stored as B3 */
  uint32_t counts_from_map;       /* 1 when tiles were padded: true plane counts live in the map */
  uint64_t payload_bytes, scale_count;
} tb_device_layout;
tb_status tb_fmt_device_layout(tb_codec codec, uint32_t group, uint32_t n, uint32_t k, const uint8_t* payload,
                               size_t payload_len, const uint16_t* scales, size_t scale_count,
                               const uint8_t* plane_map, size_t map_len, uint32_t terminal_map_value,
                               tb_device_layout* info, uint8_t* payload_out, uint16_t* scales_out);
/* write_salt_v2_package for one matrix tensor (salt_v2_package.rs:1526-1668); returns total
 * bytes (negative tb_status on error; out may be NULL to size). */
int64_t tb_fmt_package_write(tb_codec codec, const char* name, uint32_t group, uint64_t n,
                             uint64_t k, const uint8_t* plane_count, const int8_t* trits,
                             const uint16_t* scales, uint8_t* out, size_t cap);
/* write_salt_v2_package for several matrix tensors in the given order (salt_v2_package.rs:1526-1668):
 * one presence map over the full tiles of all tensors behind the last one, its trailing bits in the
 * tensor-count word, version 2 as soon as one tensor uses 64-wide scale groups.  Arrays hold `count`
 * entries; trits / scales / plane_count are laid out per tensor as for tb_fmt_resident_build. */
int64_t tb_fmt_package_write_multi(tb_codec codec, uint32_t count, const char* const* names, const uint32_t* groups,
                                   const uint64_t* n, const uint64_t* k, const uint8_t* const* plane_count,
                                   const int8_t* const* trits, const uint16_t* const* scales, uint8_t* out, size_t cap);
/* Host-only twin of tb_salt_v2_upload_reader: fetches the resident arenas of one tensor from a byte
 * source.  Call with NULL buffers to learn the sizes, then with buffers of those sizes. */
typedef struct tb_package_tensor {
  uint32_t codec, group, terminal_map_value, planes_uniform;
  uint64_t n, k, payload_bytes, scale_count, map_bytes;
} tb_package_tensor;
tb_status tb_fmt_package_extract(tb_read_at_fn read_at, void* user, uint64_t package_len, const char* tensor_name,
                                 tb_package_tensor* info, uint8_t* payload, uint16_t* scales, uint8_t* plane_map);
/* pack_tq2_0_row (crates/tritium-format/src/rows.rs:61-77) with unit block scales. */
tb_status tb_fmt_tq2_pack_rows(const int8_t* trits, uint64_t n, uint64_t k, uint8_t* out);
/* quantize_act_int8 (crates/tritium-spec/src/lib.rs:351-378), host. */
void tb_fmt_quantize_act_int8(const float* act, uint64_t m, uint64_t k, float* q, float* scale);

#ifdef __cplusplus
}
#endif
#endif
