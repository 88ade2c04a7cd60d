// C ABI of the B200 backend: handles, uploads, forward entry points, stack driver, host format
// helpers.  Host logic only; kernels live in kernels_*.cu.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "tb_internal.h"

// ---------------------------------------------------------------- errors
namespace {
thread_local std::string g_last_error;
thread_local bool g_has_error = false;
thread_local bool g_has_shape = false;          // the last error carries the two lengths of a shape mismatch
thread_local uint64_t g_shape_expected = 0, g_shape_got = 0;
}  // namespace

void tb_set_error(const std::string& message) { g_last_error = message; g_has_error = true; g_has_shape = false; }
void tb_clear_error() { g_has_error = false; g_has_shape = false; }
// BackendError::ShapeMismatch { expected, got } (crates/tritium-spec/src/lib.rs:384-391)
static tb_status fail_shape(uint64_t expected, uint64_t got) {
  tb_set_error("shape mismatch: expected " + std::to_string(expected) + ", got " + std::to_string(got));
  g_has_shape = true; g_shape_expected = expected; g_shape_got = got;
  return TB_SHAPE_MISMATCH;
}
static void clear_error() { tb_clear_error(); }
tb_status tb_fail(tb_status code, const std::string& message) { tb_set_error(message); return code; }
tb_status tb_cuda_fail(cudaError_t err, const char* what) {
  const tb_status code = err == cudaErrorMemoryAllocation ? TB_OUT_OF_MEMORY : TB_BACKEND;
  return tb_fail(code, std::string(what) + ": " + cudaGetErrorName(err) + " (" + cudaGetErrorString(err) + ")");
}
static tb_status from_fmt(const tbf::Err& e) {
  const tb_status code = e.code == 2 ? TB_SHAPE_MISMATCH : e.code == 3 ? TB_UNSUPPORTED_FORMAT : TB_INVALID_INPUT;
  return tb_fail(code, e.msg);
}
#define TB_CUDA(call, what)                                   \
  do {                                                        \
    cudaError_t err__ = (call);                               \
    if (err__ != cudaSuccess) return tb_cuda_fail(err__, what); \
  } while (0)

extern "C" uint32_t tb_abi_version(void) { return TB_ABI_VERSION; }
extern "C" const char* tb_last_error(void) { return g_has_error ? g_last_error.c_str() : nullptr; }
extern "C" tb_status tb_last_shape_mismatch(uint64_t* expected, uint64_t* got) {
  if (!expected || !got) return TB_NULL_ARG;
  if (!g_has_error || !g_has_shape) return TB_INVALID_INPUT;
  *expected = g_shape_expected; *got = g_shape_got;
  return TB_OK;
}

// ---------------------------------------------------------------- backend
namespace {

tb_status ensure(void** ptr, size_t* cap, size_t need, bool pinned_host = false) {
  if (*cap >= need) return TB_OK;
  if (*ptr) { if (pinned_host) cudaFreeHost(*ptr); else cudaFree(*ptr); *ptr = nullptr; *cap = 0; }
  const size_t want = std::max<size_t>(need, 4096);
  cudaError_t err = pinned_host ? cudaMallocHost(ptr, want) : cudaMalloc(ptr, want);
  if (err != cudaSuccess) { *ptr = nullptr; return tb_cuda_fail(err, "allocate staging buffer"); }
  *cap = want;
  return TB_OK;
}

tb_status use_device(const tb_backend* b) {
  TB_CUDA(cudaSetDevice(b->ordinal), "select device");
  return TB_OK;
}

}  // namespace

extern "C" tb_status tb_backend_create(int ordinal, tb_backend** out) {
  clear_error();
  if (!out) return tb_fail(TB_NULL_ARG, "out is null");
  *out = nullptr;
  int count = 0;
  cudaError_t err = cudaGetDeviceCount(&count);
  if (err != cudaSuccess || count == 0) {
    cudaGetLastError();
    return tb_fail(TB_BACKEND, std::string("no CUDA device available") +
                                   (err != cudaSuccess ? std::string(": ") + cudaGetErrorString(err) : ""));
  }
  if (ordinal < 0 || ordinal >= count) return tb_fail(TB_INVALID_INPUT, "device ordinal out of range");
  tb_backend* b = new (std::nothrow) tb_backend();
  if (!b) return tb_fail(TB_OUT_OF_MEMORY, "host allocation failed");
  b->ordinal = ordinal;
  auto bail = [&](cudaError_t e, const char* what) { tb_backend_free(b); return tb_cuda_fail(e, what); };
  if ((err = cudaSetDevice(ordinal)) != cudaSuccess) return bail(err, "select device");
  if ((err = cudaGetDeviceProperties(&b->prop, ordinal)) != cudaSuccess) return bail(err, "query device");
  if (b->prop.major != 10) {
    const std::string msg = "device " + std::string(b->prop.name) + " is sm_" + std::to_string(b->prop.major) +
                            std::to_string(b->prop.minor) + "; this backend carries sm_100a code only";
    tb_backend_free(b);
    return tb_fail(TB_BACKEND, msg);
  }
  if ((err = cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking)) != cudaSuccess) return bail(err, "create stream");
  if ((err = cudaMalloc(&b->d_status, 8 * sizeof(uint32_t))) != cudaSuccess) return bail(err, "allocate status");
  if ((err = cudaMemset(b->d_status, 0, 8 * sizeof(uint32_t))) != cudaSuccess) return bail(err, "clear status");
  if ((err = cudaMallocHost(&b->h_status, 8 * sizeof(uint32_t))) != cudaSuccess) return bail(err, "allocate status mirror");
  cudaDeviceGetAttribute(&b->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, ordinal);
  b->d_prep_cap = 2u << 20;   // activation tables of the decode path: up to 4 tokens x k = 32768
  if ((err = cudaMalloc(&b->d_prep, b->d_prep_cap)) != cudaSuccess) return bail(err, "allocate decode scratch");
  if ((err = cudaMalloc(reinterpret_cast<void**>(&b->d_tile_counters), 256 * sizeof(uint32_t))) != cudaSuccess ||
      (err = cudaMemset(b->d_tile_counters, 0, 256 * sizeof(uint32_t))) != cudaSuccess)
    return bail(err, "allocate tile counters");
  const unsigned char* u = reinterpret_cast<const unsigned char*>(b->prop.uuid.bytes);
  std::snprintf(b->physical_id, sizeof b->physical_id,
                "b200:%d:GPU-%02x%02x%02x%02x-%02x%02x-%02x%02x-%02x%02x-%02x%02x%02x%02x%02x%02x", ordinal, u[0], u[1],
                u[2], u[3], u[4], u[5], u[6], u[7], u[8], u[9], u[10], u[11], u[12], u[13], u[14], u[15]);
  *out = b;
  return TB_OK;
}

namespace {
void destroy_backend(tb_backend* b);
}
void tb_backend_retain(tb_backend* b) { if (b) b->dependants.fetch_add(1); }
void tb_backend_release(tb_backend* b) {
  if (b && b->dependants.fetch_sub(1) == 1 && b->released.load()) destroy_backend(b);
}

extern "C" void tb_backend_free(tb_backend* b) {
  if (!b || b->released.exchange(true)) return;
  if (b->dependants.load() == 0) destroy_backend(b);   // otherwise the last dependant does it
}

namespace {
void destroy_backend(tb_backend* b) {
  cudaSetDevice(b->ordinal);
  if (b->stream) { cudaStreamSynchronize(b->stream); cudaStreamDestroy(b->stream); }
  cudaFree(b->d_status); cudaFreeHost(b->h_status);
  cudaFree(b->d_x); cudaFree(b->d_y); cudaFree(b->d_aux); cudaFree(b->d_q); cudaFree(b->d_prep); cudaFree(b->d_norm); cudaFree(b->d_limb); cudaFree(b->d_tile_counters); cudaFreeHost(b->h_pin);
  delete b;
}
}  // namespace

extern "C" tb_status tb_backend_caps(const tb_backend* b, tb_caps* out) {
  clear_error();
  if (!b || !out) return tb_fail(TB_NULL_ARG, "null argument");
  std::memset(out, 0, sizeof *out);
  std::snprintf(out->backend, sizeof out->backend, "b200");
  std::snprintf(out->device_name, sizeof out->device_name, "%.*s", int(sizeof out->device_name) - 1, b->prop.name);
  std::snprintf(out->device_id, sizeof out->device_id, "b200:%d", b->ordinal);
  std::snprintf(out->physical_id, sizeof out->physical_id, "%s", b->physical_id);
  std::snprintf(out->features, sizeof out->features, "sm_100a,salt_v2_d2,salt_v2_b3,salt_v2_s34,tq2_0,int8_tcgen05");
  out->total_memory_bytes = b->prop.totalGlobalMem;
  out->sm_count = uint32_t(b->prop.multiProcessorCount);
  out->supports_imma = 1;
  out->supports_fp8 = 1;
  return TB_OK;
}

extern "C" tb_status tb_backend_synchronize(tb_backend* b) {
  clear_error();
  if (!b) return tb_fail(TB_NULL_ARG, "backend is null");
  if (tb_status s = use_device(b)) return s;
  TB_CUDA(cudaStreamSynchronize(b->stream), "synchronize stream");
  return TB_OK;
}

extern "C" tb_status tb_backend_check(tb_backend* b, void* stream) {
  clear_error();
  if (!b) return tb_fail(TB_NULL_ARG, "backend is null");
  if (tb_status s = use_device(b)) return s;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : b->stream;
  TB_CUDA(cudaMemcpyAsync(b->h_status, b->d_status, 8 * sizeof(uint32_t), cudaMemcpyDeviceToHost, st), "read status");
  TB_CUDA(cudaMemsetAsync(b->d_status, 0, 8 * sizeof(uint32_t), st), "clear status");
  TB_CUDA(cudaStreamSynchronize(st), "synchronize stream");
  const uint32_t flags = b->h_status[TBS_FLAGS];
  if (!flags) return TB_OK;
  char msg[192];
  if (flags & TBF_WAIT_TIMEOUT) {
    // a tensor-core launch that gave up may have left the arrival counters of its K splits part
    // way: the next launch must find them at zero again
    cudaMemsetAsync(b->d_tile_counters, 0, 256 * sizeof(uint32_t), st);
    std::snprintf(msg, sizeof msg, "a bounded device wait gave up (stage %u, barrier %u)", b->h_status[TBS_INFO0], b->h_status[TBS_INFO1]);
    return tb_fail(TB_TIMEOUT, msg);
  }
  if (flags & TBF_NONFINITE_ACT) {
    std::snprintf(msg, sizeof msg, "SALT V2 activation %u is non-finite (%#010x)", b->h_status[TBS_INFO0], b->h_status[TBS_INFO1]);
    return tb_fail(TB_INVALID_INPUT, msg);
  }
  if (flags & TBF_NONFINITE_OUT) {
    std::snprintf(msg, sizeof msg, "SALT V2 output row %u became non-finite at column %u", b->h_status[TBS_INFO0], b->h_status[TBS_INFO1]);
    return tb_fail(TB_INVALID_INPUT, msg);
  }
  return tb_fail(TB_BACKEND, "kernel reported an invalid configuration");
}

extern "C" tb_status tb_backend_inject_wait_timeout(tb_backend* b, uint32_t enable) {
  clear_error();
  if (!b) return tb_fail(TB_NULL_ARG, "backend is null");
  b->inject_missing_tx = enable ? 16u : 0u;
  return TB_OK;
}

// ---------------------------------------------------------------- weights
namespace {

tb_status upload_resident(tb_backend* b, const tbf::Resident& r_artifact, uint64_t source_len, bool is_tq2, uint64_t logical_k,
                          tb_weights** out) {
  if (tb_status s = use_device(b)) return s;
  // the arenas as the device holds them: S34 recoded as B3, varying plane counts padded (tb_format.h)
  tbf::Resident relaid;
  bool recoded = false, map_counts = false;
  if (tbf::Err e = tbf::device_layout(r_artifact, &relaid, &recoded, &map_counts)) return from_fmt(e);
  const tbf::Resident& r = (recoded || map_counts) ? relaid : r_artifact;
  tb_weights* w = new (std::nothrow) tb_weights();
  if (!w) return tb_fail(TB_OUT_OF_MEMORY, "host allocation failed");
  w->owner = b; tb_backend_retain(b); w->codec = r.codec; w->group = r.group; w->uniform_planes = r.uniform_planes;
  w->map_counts = map_counts;
  w->n = r.n; w->k = r.k; w->tiles = r.tiles; w->present_planes = r.present_planes;
  w->payload_bytes = r.payload.size(); w->scale_count = r.scales.size();
  w->map_bytes = r.map.size(); w->rank_prefix_bytes = r.rank_prefix.size() * 4;
  w->terminal_map = r.terminal_map; w->source_len = source_len; w->is_tq2 = is_tq2; w->logical_k = logical_k;
  w->fast = r.uniform_planes != 0 && r.k % 256 == 0 && r.group == 128 && (r.codec == tbf::kB3 || r.codec == tbf::kD2);
  tb_make_decode_plan(w, b->max_smem_optin);
  // Arenas are padded so that the last row block is a full, valid stage: zero-trit bytes
  // (B3 121, D2 0x55) and zero scales.  The padding is never stored to an output.
  size_t pay_alloc = r.payload.size() + 64, sc_alloc = r.scales.size() * 2 + 64;
  if (w->fast) {
    pay_alloc = std::max<size_t>(pay_alloc, size_t(w->plan.blocks) * w->plan.stage_bytes + 64);
    sc_alloc = std::max<size_t>(sc_alloc, size_t(w->plan.blocks) * w->plan.scale_stage_bytes + 64);
  }
  auto bail = [&](cudaError_t e, const char* what) { tb_weights_free(w); return tb_cuda_fail(e, what); };
  cudaError_t err;
  if ((err = cudaMalloc(&w->d_payload, pay_alloc)) != cudaSuccess) return bail(err, "upload SALT V2 payload");
  if ((err = cudaMalloc(&w->d_scales, sc_alloc)) != cudaSuccess) return bail(err, "upload SALT V2 scales");
  const int fill = r.codec == tbf::kB3 ? 121 : r.codec == tbf::kD2 ? 0x55 : 0;
  if ((err = cudaMemsetAsync(w->d_payload, fill, pay_alloc, b->stream)) != cudaSuccess) return bail(err, "pad payload");
  if ((err = cudaMemsetAsync(w->d_scales, 0, sc_alloc, b->stream)) != cudaSuccess) return bail(err, "pad scales");
  if ((err = cudaMemcpyAsync(w->d_payload, r.payload.data(), r.payload.size(), cudaMemcpyHostToDevice, b->stream)) != cudaSuccess)
    return bail(err, "upload SALT V2 payload");
  if ((err = cudaMemcpyAsync(w->d_scales, r.scales.data(), r.scales.size() * 2, cudaMemcpyHostToDevice, b->stream)) != cudaSuccess)
    return bail(err, "upload SALT V2 scales");
  std::vector<uint8_t> meta(r.map);
  for (uint32_t v : r.rank_prefix) for (int i = 0; i < 4; ++i) meta.push_back(uint8_t(v >> (8 * i)));
  if ((err = cudaMalloc(&w->d_meta, meta.size() + 16)) != cudaSuccess) return bail(err, "upload SALT V2 compact index");
  if (!meta.empty() && (err = cudaMemcpyAsync(w->d_meta, meta.data(), meta.size(), cudaMemcpyHostToDevice, b->stream)) != cudaSuccess)
    return bail(err, "upload SALT V2 compact index");
  std::vector<uint32_t> ranks;
  if (!r.uniform_planes) {
    ranks.resize(size_t(r.tiles));
    uint32_t acc = 0;
    for (uint64_t t = 0; t < r.tiles; ++t) { ranks[t] = acc; acc += r.planes_of(t); }
    if ((err = cudaMalloc(&w->d_tile_rank, ranks.size() * 4)) != cudaSuccess) return bail(err, "upload tile ranks");
    if ((err = cudaMemcpyAsync(w->d_tile_rank, ranks.data(), ranks.size() * 4, cudaMemcpyHostToDevice, b->stream)) != cudaSuccess)
      return bail(err, "upload tile ranks");
  }
  if ((err = cudaStreamSynchronize(b->stream)) != cudaSuccess) return bail(err, "finish upload");
  *out = w;
  return TB_OK;
}

}  // namespace

extern "C" tb_status tb_tq2_upload(tb_backend* b, const uint8_t* packed, size_t len, uint32_t n, uint32_t k, tb_weights** out) {
  clear_error();
  if (!b || !out || (!packed && len)) return tb_fail(TB_NULL_ARG, "null argument");
  *out = nullptr;
  if (n == 0 || k == 0) return tb_fail(TB_INVALID_INPUT, "packed len 0: shape must be positive");
  tbf::Resident r;
  if (tbf::Err e = tbf::resident_from_tq2(packed, len, n, k, &r)) return from_fmt(e);
  return upload_resident(b, r, len, true, k, out);
}

extern "C" tb_status tb_tq1_upload(tb_backend* b, const uint8_t* packed, size_t len, uint32_t n, uint32_t k, tb_weights** out) {
  clear_error();
  if (!b || !out || (!packed && len)) return tb_fail(TB_NULL_ARG, "null argument");
  *out = nullptr;
  if (n == 0 || k == 0) return tb_fail(TB_INVALID_INPUT, "packed len 0: shape must be positive");
  tbf::Resident r;
  if (tbf::Err e = tbf::resident_from_tq1(packed, len, n, k, &r)) return from_fmt(e);
  return upload_resident(b, r, len, true, k, out);
}

extern "C" tb_status tb_salt_v1_upload(tb_backend* b, const uint8_t* planes, size_t len, uint32_t t_planes, uint32_t n, uint32_t k,
                                       tb_weights** out) {
  clear_error();
  if (!b || !out || (!planes && len)) return tb_fail(TB_NULL_ARG, "null argument");
  *out = nullptr;
  if (n == 0 || k == 0) return tb_fail(TB_INVALID_INPUT, "shape must be positive");
  tbf::Resident r;
  if (tbf::Err e = tbf::resident_from_salt_v1(planes, len, t_planes, n, k, &r)) return from_fmt(e);
  return upload_resident(b, r, len, false, k, out);
}

extern "C" tb_status tb_salt_v2_upload(tb_backend* b, tb_codec codec, uint32_t group, uint32_t n, uint32_t k,
                                       const uint8_t* payload, size_t payload_len, const uint16_t* scales, size_t scale_count,
                                       const uint8_t* plane_map, size_t map_len, uint32_t terminal, tb_weights** out) {
  clear_error();
  if (!b || !out || !payload || !scales || (!plane_map && map_len)) return tb_fail(TB_NULL_ARG, "null argument");
  *out = nullptr;
  tbf::Resident r;
  if (tbf::Err e = tbf::resident_from_arenas(int(codec), group, n, k, payload, payload_len, scales, scale_count, plane_map, map_len, terminal, &r))
    return from_fmt(e);
  return upload_resident(b, r, payload_len, false, k, out);
}

extern "C" tb_status tb_salt_v2_upload_package(tb_backend* b, const uint8_t* package, size_t len, const char* name, tb_weights** out) {
  clear_error();
  if (!b || !out || !package || !name) return tb_fail(TB_NULL_ARG, "null argument");
  *out = nullptr;
  tbf::Resident r;
  if (tbf::Err e = tbf::resident_from_package(package, len, name, &r)) return from_fmt(e);
  return upload_resident(b, r, r.payload.size(), false, r.k, out);
}

extern "C" tb_status tb_salt_v2_upload_reader(tb_backend* b, tb_read_at_fn read_at, void* user, uint64_t package_len, const char* name,
                                              tb_weights** out) {
  clear_error();
  if (!b || !out || !read_at || !name) return tb_fail(TB_NULL_ARG, "null argument");
  *out = nullptr;
  tbf::Resident r;
  if (tbf::Err e = tbf::resident_from_reader(read_at, user, package_len, name, &r)) return from_fmt(e);
  return upload_resident(b, r, r.payload.size(), false, r.k, out);
}

extern "C" tb_status tb_weights_info_get(const tb_weights* w, tb_weights_info* out) {
  clear_error();
  if (!w || !out) return tb_fail(TB_NULL_ARG, "null argument");
  std::memset(out, 0, sizeof *out);
  out->codec = uint32_t(w->codec); out->group = w->group; out->planes_uniform = w->uniform_planes;
  out->n = w->n; out->k = w->k; out->tiles = w->tiles; out->present_planes = w->present_planes;
  out->payload_bytes = w->payload_bytes; out->scale_bytes = w->scale_count * 2; out->map_bytes = w->map_bytes;
  out->rank_prefix_bytes = w->rank_prefix_bytes; out->source_len_bytes = w->source_len; out->fast_path = w->fast;
  return TB_OK;
}

extern "C" void tb_weights_free(tb_weights* w) {
  if (!w) return;
  if (w->owner) cudaSetDevice(w->owner->ordinal);
  cudaFree(w->d_payload); cudaFree(w->d_scales); cudaFree(w->d_meta); cudaFree(w->d_tile_rank);
  tb_backend* owner = w->owner;
  delete w;
  tb_backend_release(owner);
}

// ---------------------------------------------------------------- forward
namespace {

void fill_receipt(const tb_weights* w, uint32_t m, size_t x_elem, size_t y_elem, uint32_t kernel, uint32_t launches, tb_receipt* r) {
  if (!r) return;
  std::memset(r, 0, sizeof *r);
  r->payload_bytes = w->payload_bytes; r->scale_bytes = w->scale_count * 2; r->map_bytes = w->map_bytes;
  r->rank_prefix_bytes = w->rank_prefix_bytes;
  r->activation_bytes = uint64_t(m) * w->k * x_elem; r->output_bytes = uint64_t(m) * w->n * y_elem;
  r->kernel = kernel; r->launches = launches;
}

size_t dtype_size(tb_dtype t) { return t == TB_F32 ? 4 : t == TB_BF16 ? 2 : 1; }

tb_status check_handles(const tb_backend* b, const tb_weights* w) {
  if (!b || !w) return tb_fail(TB_NULL_ARG, "null argument");
  if (b->released.load()) return tb_fail(TB_INVALID_INPUT, "the backend context was freed; only its objects' free calls are still valid");
  if (w->owner != b) return tb_fail(TB_INVALID_INPUT, "weights handle belongs to another backend context");
  return TB_OK;
}

tb_status reserve_prefill(tb_backend* b, const tb_weights* w, uint32_t m);

// The decode kernel keeps two row blocks of a tensor in shared memory at least.  Rows too long for
// that (three planes beyond k of about 9 K, two planes beyond about 28 K) go to the tensor-core
// kernel at every token count.
bool decode_fits(const tb_backend* b, const tb_weights* w, uint32_t m) {
  return tb_decode_supported(w, std::min<uint32_t>(std::max<uint32_t>(m, 1u), 4u), b->max_smem_optin, nullptr);
}
bool takes_tensor_cores(const tb_backend* b, const tb_weights* w, uint32_t m, uint32_t flags, uint32_t decode_limit = 8) {
  if (flags & TB_FWD_FORCE_PREFILL) return true;
  if (flags & TB_FWD_FORCE_DECODE) return false;
  return m > decode_limit || (w->fast && !decode_fits(b, w, m));
}

// What a decode block wraps around the linear: RMSNorm in front of the quantiser, residual behind.
struct BlockExtras {
  const float* norm_weight = nullptr; float norm_eps = 0.f; bool norm_zero_centered = false;
  const float* residual = nullptr;
  const float* relu2_up = nullptr;   // squared-ReLU gate: activation = (max(x, 0)^2) * relu2_up
};

// Device-pointer dispatch shared by every entry point.  Returns the kernel family used.
tb_status forward_dev(tb_backend* b, const tb_weights* w, const tb_forward_args& a_in, cudaStream_t st, tb_receipt* receipt,
                      const BlockExtras& ex = BlockExtras{}) {
  tb_forward_args a = a_in;
  if (a.m == 0 || w->n == 0) { fill_receipt(w, 0, 0, 0, 0, 0, receipt); return TB_OK; }
  if (!a.x || !a.y) return tb_fail(TB_NULL_ARG, "null activation or output pointer");
  const bool a8 = (a.flags & TB_FWD_A8) != 0 || a.x_dtype == TB_I8;
  if ((ex.norm_weight || ex.residual) && !a8) return tb_fail(TB_INVALID_INPUT, "the norm and residual steps belong to the int8 path");
  if (ex.norm_weight && a.x_dtype == TB_I8) return tb_fail(TB_INVALID_INPUT, "RMSNorm takes fp32 or bf16 activations");
  if (ex.relu2_up) {
    if (a.x_dtype != TB_F32) return tb_fail(TB_INVALID_INPUT, "the squared-ReLU gate takes the fp32 outputs of the gate and up projections");
    if (ex.norm_weight || a.act_absmax) return tb_fail(TB_INVALID_INPUT, "the squared-ReLU gate is not combined with RMSNorm or a supplied absmax");
    if (!w->fast) return tb_fail(TB_UNSUPPORTED_FORMAT, "the squared-ReLU gate needs uniform plane counts, k % 256 == 0, group 128 and codec D2 or B3");
  }
  if (!a8) {
    if (a.x_dtype != TB_F32 || a.y_dtype != TB_F32) return tb_fail(TB_INVALID_INPUT, "the fp32 path takes fp32 activations and outputs");
    if (!(a.flags & TB_FWD_EXACT) && w->fast && a.m <= (1u << 20)) {
      // Not bit-exact, but fast: every activation as four int8 limbs relative to its token's
      // absmax (error below 2e-9 of the absmax), the limbs as pseudo-tokens through the int8
      // kernels (exact int32 sums per limb), the four outputs of a token added in a fixed order.
      const uint32_t m4 = a.m * 4;
      const size_t qb = (size_t(m4) * w->k + 255) & ~size_t(255), sb = (size_t(m4) * 4 + 255) & ~size_t(255);
      if (tb_status s = ensure(&b->d_limb, &b->d_limb_cap, qb + sb + size_t(m4) * w->n * 4 + 256)) return s;
      if (takes_tensor_cores(b, w, m4, a.flags)) if (tb_status s = reserve_prefill(b, w, m4)) return s;
      uint8_t* base = static_cast<uint8_t*>(b->d_limb);
      int8_t* q = reinterpret_cast<int8_t*>(base);
      float* scales = reinterpret_cast<float*>(base + qb);
      float* y4 = reinterpret_cast<float*>(base + qb + sb);
      TB_CUDA(tb_launch_limb_split(static_cast<const float*>(a.x), a.m, uint32_t(w->k), q, scales, b->d_status, st), "launch limb split");
      tb_forward_args l{};
      l.x = q; l.x_dtype = TB_I8; l.act_scale = scales; l.m = m4; l.y = y4; l.y_dtype = TB_F32; l.row_scale = a.row_scale;
      l.flags = TB_FWD_A8 | (a.flags & (TB_FWD_PDL | TB_FWD_FORCE_DECODE | TB_FWD_FORCE_PREFILL));
      tb_receipt inner{};
      if (tb_status s = forward_dev(b, w, l, st, &inner)) return s;
      TB_CUDA(tb_launch_limb_sum(y4, a.m, uint32_t(w->n), static_cast<float*>(a.y), st), "launch limb sum");
      fill_receipt(w, a.m, 4, 4, inner.kernel, inner.launches + 2, receipt);
      return TB_OK;
    }
    ExactArgs e{w, static_cast<const float*>(a.x), static_cast<float*>(a.y), a.m, a.row_scale, b->d_status};
    TB_CUDA(tb_launch_check_finite(e.x, uint64_t(a.m) * w->k, b->d_status, st), "launch finite check");
    TB_CUDA(tb_launch_exact(e, st), "launch salt_v2_exact");
    fill_receipt(w, a.m, 4, 4, 0, 2, receipt);
    return TB_OK;
  }
  if (a.x_dtype == TB_I8 && !a.act_scale) return tb_fail(TB_NULL_ARG, "int8 activations need act_scale");
  if (a.y_dtype == TB_I8) return tb_fail(TB_INVALID_INPUT, "output dtype must be fp32 or bf16");
  if (!w->fast) {
    // Scale groups of 64, ragged shapes, S34 and mixed plane counts have no fast kernel: quantise
    // to int8 codes kept as fp32 values, run the bit-exact kernel on them (its group sums of small
    // integers are exact and it keeps the reference's order, so the result equals the CPU path bit
    // for bit), apply the token scale.  Slow by design; the accumulator dump is not offered here.
    if (a.acc_dump) return tb_fail(TB_UNSUPPORTED_FORMAT, "the accumulator dump needs uniform plane counts, k % 256 == 0, group 128 and codec D2 or B3");
    if (a.x_dtype == TB_I8 || a.act_absmax) return tb_fail(TB_UNSUPPORTED_FORMAT, "this layout takes fp32 or bf16 activations without a supplied absmax");
    const size_t qf = (size_t(a.m) * w->k * 4 + 255) & ~size_t(255), yf = (size_t(a.m) * w->n * 4 + 255) & ~size_t(255);
    if (tb_status s = ensure(&b->d_norm, &b->d_norm_cap, 2 * qf + yf + size_t(a.m) * 4 + 256)) return s;
    uint8_t* base = static_cast<uint8_t*>(b->d_norm);
    float* q = reinterpret_cast<float*>(base + qf);           // the first qf bytes may hold normalised rows
    float* y32 = reinterpret_cast<float*>(base + 2 * qf);
    float* scale = reinterpret_cast<float*>(base + 2 * qf + yf);
    const void* src = a.x; tb_dtype src_dtype = a.x_dtype;
    if (ex.norm_weight) {
      TB_CUDA(tb_launch_rmsnorm(a.x, a.x_dtype, ex.norm_weight, ex.norm_eps, ex.norm_zero_centered, a.m, uint32_t(w->k),
                                reinterpret_cast<float*>(base), st), "launch rmsnorm");
      src = base; src_dtype = TB_F32;
    }
    TB_CUDA(tb_launch_quantize_to_float(src, src_dtype, a.m, uint32_t(w->k), q, scale, b->d_status, st), "launch quantise");
    ExactArgs e{w, q, y32, a.m, a.row_scale, b->d_status};
    TB_CUDA(tb_launch_exact(e, st), "launch salt_v2_exact");
    TB_CUDA(tb_launch_scale_tokens(y32, scale, ex.residual, a.m, uint32_t(w->n), a.y, a.y_dtype, st), "launch token scale");
    fill_receipt(w, a.m, dtype_size(a.x_dtype), dtype_size(a.y_dtype), 0, ex.norm_weight ? 4 : 3, receipt);
    return TB_OK;
  }
  // measured crossover (C2, 27B and 2B linears alike): two chained 4-token decode passes are level with
  // one call of the few-token tensor-core kernel (about 25 us on C2), three passes are slower
  const bool want_prefill = takes_tensor_cores(b, w, a.m, a.flags);
  uint32_t extra_launches = 0;
  // The decode kernel normalises inside its table builder.  Every other route (the tensor-core
  // kernel, tables from the preparation kernel) takes rows normalised by a kernel of its own; the
  // arithmetic is the same, so the codes are too.
  const auto normalise = [&](uint32_t m0, uint32_t mc) -> tb_status {
    if (tb_status s = ensure(&b->d_norm, &b->d_norm_cap, size_t(a.m) * w->k * 4)) return s;
    float* dst = static_cast<float*>(b->d_norm) + size_t(m0) * w->k;
    const uint8_t* src = static_cast<const uint8_t*>(a_in.x) + size_t(m0) * w->k * dtype_size(a_in.x_dtype);
    TB_CUDA(tb_launch_rmsnorm(src, a_in.x_dtype, ex.norm_weight, ex.norm_eps, ex.norm_zero_centered, mc, uint32_t(w->k), dst, st),
            "launch rmsnorm");
    ++extra_launches;
    return TB_OK;
  };
  if (want_prefill && tb_prefill_supported(w, a.m)) {
    const size_t need = tb_prefill_scratch_bytes(w, a.m);
    if (b->d_q_cap < need) return tb_fail(TB_OUT_OF_MEMORY, "prefill scratch is not reserved; call through a host entry point or tb_stack first");
    if (ex.norm_weight) {
      if (tb_status s = normalise(0, a.m)) return s;
      a.x = b->d_norm; a.x_dtype = TB_F32;
    }
    PrefillArgs pa{w, a.x, a.x_dtype, a.act_scale, a.act_absmax, a.m, a.y, a.y_dtype, a.acc_dump, a.row_scale,
                   b->d_q, b->d_q_cap, b->d_status};
    pa.residual = ex.residual; pa.tile_counters = b->d_tile_counters; pa.relu2_up = ex.relu2_up;
    TB_CUDA(tb_launch_prefill(pa, b->prop.multiProcessorCount, st), "launch prefill");
    fill_receipt(w, a.m, dtype_size(a_in.x_dtype), dtype_size(a.y_dtype), 2, 2 + extra_launches, receipt);
    return TB_OK;
  }
  if (a.flags & TB_FWD_FORCE_PREFILL) return tb_fail(TB_UNSUPPORTED_FORMAT, "the prefill kernel does not take this shape");
  uint32_t launches = 0;
  // One pass per four tokens.  Small activation tables are built inside the decode kernel (one
  // launch); large ones, and activations that are not 16-byte aligned, by the separate preparation
  // kernel into the backend's scratch (see tb_decode_builds_tables).
  for (uint32_t m0 = 0; m0 < a.m; m0 += 4) {
    const uint32_t mc = std::min<uint32_t>(4, a.m - m0);
    const bool fused = tb_decode_builds_tables(w, mc, a.x) &&
                       (!ex.norm_weight || (reinterpret_cast<uintptr_t>(ex.norm_weight) & 15u) == 0) &&
                       (!ex.relu2_up || (reinterpret_cast<uintptr_t>(ex.relu2_up) & 15u) == 0);
    if (!tb_decode_supported(w, mc, b->max_smem_optin, nullptr))
      return tb_fail(TB_UNSUPPORTED_FORMAT, "the decode kernel's shared-memory plan does not fit this shape");
    DecodeArgs d{};
    d.w = w; d.x_dtype = a.x_dtype; d.m = mc; d.y_dtype = a.y_dtype; d.y_row_stride = uint32_t(w->n);
    d.x = static_cast<const uint8_t*>(a.x) + size_t(m0) * w->k * dtype_size(a.x_dtype);
    if (ex.norm_weight) {
      if (fused) {
        d.norm_weight = ex.norm_weight; d.norm_eps = ex.norm_eps; d.norm_zero_centered = ex.norm_zero_centered;
      } else {
        if (tb_status s = normalise(m0, mc)) return s;
        d.x = static_cast<const float*>(b->d_norm) + size_t(m0) * w->k; d.x_dtype = TB_F32;
      }
    }
    d.residual = ex.residual ? ex.residual + size_t(m0) * w->n : nullptr;
    d.relu2_up = ex.relu2_up ? ex.relu2_up + size_t(m0) * w->k : nullptr;
    d.act_scale_in = a.act_scale ? a.act_scale + m0 : nullptr;
    d.act_absmax_in = a.act_absmax ? a.act_absmax + m0 : nullptr;
    d.y = static_cast<uint8_t*>(a.y) + size_t(m0) * w->n * dtype_size(a.y_dtype);
    d.acc_dump = a.acc_dump; d.dump_token_offset = m0; d.dump_tokens_total = a.m;
    // passes after the first always chain with programmatic dependent launch: their weight
    // stream starts under the previous pass's tail
    d.row_scale = a.row_scale; d.status = b->d_status; d.pdl = (a.flags & TB_FWD_PDL) != 0 || m0 > 0;
    d.fused = fused;
    d.scratch = b->d_prep; d.scratch_bytes = b->d_prep_cap;
    d.tables_shared = false;
    if (!fused) { TB_CUDA(tb_launch_prepare(d, st), "launch prepare"); ++launches; }
    TB_CUDA(tb_launch_decode(d, b->prop.multiProcessorCount, b->max_smem_optin, st), "launch decode");
    ++launches;
  }
  fill_receipt(w, a.m, dtype_size(a.x_dtype), dtype_size(a.y_dtype), 1, launches + extra_launches, receipt);
  return TB_OK;
}

tb_status reserve_prefill(tb_backend* b, const tb_weights* w, uint32_t m) {
  if (!w->fast || !tb_prefill_supported(w, m)) return TB_OK;
  // batches of up to 64 tokens split K and keep partial sums in the scratch as well, so the need
  // does not grow monotonically with m: reserve for the largest of the kernel's token-tile classes
  size_t need = tb_prefill_scratch_bytes(w, m);
  for (uint32_t edge : {32u, 64u})
    if (m > edge) need = std::max(need, tb_prefill_scratch_bytes(w, edge));
  return ensure(&b->d_q, &b->d_q_cap, need);
}

// Host-pointer wrapper: stage in, run, check, stage out.  `y` is written only on success.
tb_status forward_host(tb_backend* b, const tb_weights* w, const void* x, tb_dtype xd, uint32_t m, void* y, tb_dtype yd,
                       int32_t* acc_dump, const float* row_scale_host, uint32_t flags, tb_receipt* receipt) {
  if (tb_status s = check_handles(b, w)) return s;
  if (m == 0 || w->n == 0) { fill_receipt(w, 0, 0, 0, 0, 0, receipt); return TB_OK; }
  if (!x || !y) return tb_fail(TB_NULL_ARG, "null activation or output pointer");
  if (tb_status s = use_device(b)) return s;
  const size_t xb = size_t(m) * w->k * dtype_size(xd), yb = size_t(m) * w->n * dtype_size(yd);
  const size_t groups = w->k / w->group;
  const size_t dump_b = acc_dump ? size_t(m) * w->n * groups * w->uniform_planes * 4 : 0;
  const size_t rs_b = row_scale_host ? w->n * 4 : 0;
  if (tb_status s = ensure(&b->d_x, &b->d_x_cap, xb)) return s;
  if (tb_status s = ensure(&b->d_y, &b->d_y_cap, yb)) return s;
  if (tb_status s = ensure(&b->d_aux, &b->d_aux_cap, dump_b + rs_b + 256)) return s;
  if (flags & TB_FWD_A8) if (tb_status s = reserve_prefill(b, w, m)) return s;
  uint8_t* aux = static_cast<uint8_t*>(b->d_aux);
  // Activations and outputs travel through one pinned bounce buffer, so that both copies are truly
  // asynchronous and the call needs a single stream synchronisation: [x | y].
  const size_t x_off = 0, y_off = (xb + 255) / 256 * 256;
  if (tb_status s = ensure(&b->h_pin, &b->h_pin_cap, y_off + yb, true)) return s;
  uint8_t* pin = static_cast<uint8_t*>(b->h_pin);
  std::memcpy(pin + x_off, x, xb);
  TB_CUDA(cudaMemcpyAsync(b->d_x, pin + x_off, xb, cudaMemcpyHostToDevice, b->stream), "copy activations to device");
  if (rs_b) TB_CUDA(cudaMemcpyAsync(aux + dump_b, row_scale_host, rs_b, cudaMemcpyHostToDevice, b->stream), "copy scales to device");
  tb_forward_args a{};
  a.x = b->d_x; a.x_dtype = xd; a.m = m; a.y = b->d_y; a.y_dtype = yd; a.flags = flags;
  a.acc_dump = acc_dump ? reinterpret_cast<int32_t*>(aux) : nullptr;
  a.row_scale = rs_b ? reinterpret_cast<const float*>(aux + dump_b) : nullptr;
  if (tb_status s = forward_dev(b, w, a, b->stream, receipt)) return s;
  // the device status word (bounded waits, finite checks) comes back with the output; the
  // caller's buffers are written only when it is clean
  TB_CUDA(cudaMemcpyAsync(pin + y_off, b->d_y, yb, cudaMemcpyDeviceToHost, b->stream), "copy output to host");
  TB_CUDA(cudaMemcpyAsync(b->h_status, b->d_status, 8 * sizeof(uint32_t), cudaMemcpyDeviceToHost, b->stream), "read status");
  TB_CUDA(cudaStreamSynchronize(b->stream), "synchronize stream");
  if (b->h_status[TBS_FLAGS]) return tb_backend_check(b, b->stream);   // reports and clears
  std::memcpy(y, pin + y_off, yb);
  if (dump_b) {
    TB_CUDA(cudaMemcpyAsync(acc_dump, aux, dump_b, cudaMemcpyDeviceToHost, b->stream), "copy accumulators to host");
    TB_CUDA(cudaStreamSynchronize(b->stream), "synchronize stream");
  }
  return TB_OK;
}

tb_status preflight_finite(const float* x, size_t count) {
  for (size_t i = 0; i < count; ++i)
    if (!std::isfinite(x[i])) {
      uint32_t bits;
      std::memcpy(&bits, &x[i], 4);
      char msg[96];
      std::snprintf(msg, sizeof msg, "SALT V2 activation %zu is non-finite (%#010x)", i, bits);
      return tb_fail(TB_INVALID_INPUT, msg);
    }
  return TB_OK;
}

}  // namespace

extern "C" tb_status tb_salt_v2_forward_exact(tb_backend* b, const tb_weights* w, const float* x, uint32_t m, float* y, tb_receipt* receipt) {
  clear_error();
  if (tb_status s = check_handles(b, w)) return s;
  if (m && w->n && x) if (tb_status s = preflight_finite(x, size_t(m) * w->k)) return s;
  return forward_host(b, w, x, TB_F32, m, y, TB_F32, nullptr, nullptr, TB_FWD_EXACT, receipt);
}

extern "C" tb_status tb_linear_forward_f32(tb_backend* b, const tb_weights* w, const float* x, uint32_t m, float* y, tb_receipt* receipt) {
  clear_error();
  if (tb_status s = check_handles(b, w)) return s;
  if (m && w->n && x) if (tb_status s = preflight_finite(x, size_t(m) * w->k)) return s;
  return forward_host(b, w, x, TB_F32, m, y, TB_F32, nullptr, nullptr, 0, receipt);
}

extern "C" tb_status tb_linear_forward_a8(tb_backend* b, const tb_weights* w, const void* x, tb_dtype xd, uint32_t m, void* y,
                                          tb_dtype yd, int32_t* acc_dump, tb_receipt* receipt) {
  clear_error();
  if (tb_status s = check_handles(b, w)) return s;
  if (xd == TB_I8) return tb_fail(TB_INVALID_INPUT, "host int8 activations are not accepted here; pass fp32 or bf16");
  if (xd == TB_F32 && m && w->n && x) if (tb_status s = preflight_finite(static_cast<const float*>(x), size_t(m) * w->k)) return s;
  return forward_host(b, w, x, xd, m, y, yd, acc_dump, nullptr, TB_FWD_A8, receipt);
}

extern "C" tb_status tb_linear_forward_dev(tb_backend* b, const tb_weights* w, const tb_forward_args* args, tb_receipt* receipt) {
  clear_error();
  if (tb_status s = check_handles(b, w)) return s;
  if (!args) return tb_fail(TB_NULL_ARG, "args is null");
  if (tb_status s = use_device(b)) return s;
  cudaStream_t st = args->stream ? static_cast<cudaStream_t>(args->stream) : b->stream;
  return forward_dev(b, w, *args, st, receipt);
}

extern "C" tb_status tb_norm_linear_forward_dev(tb_backend* b, const tb_weights* w, const tb_norm_linear_args* args, tb_receipt* receipt) {
  clear_error();
  if (tb_status s = check_handles(b, w)) return s;
  if (!args) return tb_fail(TB_NULL_ARG, "args is null");
  if (args->x_dtype != TB_F32 && args->x_dtype != TB_BF16) return tb_fail(TB_INVALID_INPUT, "activations must be fp32 or bf16");
  if (args->norm_flags & ~TB_NORM_ZERO_CENTERED) return tb_fail(TB_INVALID_INPUT, "unknown norm flag");
  if (args->norm_weight && !(args->norm_eps >= 0.f)) return tb_fail(TB_INVALID_INPUT, "norm_eps must be a non-negative number");
  if (tb_status s = use_device(b)) return s;
  cudaStream_t st = args->stream ? static_cast<cudaStream_t>(args->stream) : b->stream;
  tb_forward_args a{};
  a.x = args->x; a.x_dtype = args->x_dtype; a.m = args->m; a.y = args->y; a.y_dtype = args->y_dtype;
  a.flags = args->flags | TB_FWD_A8; a.stream = args->stream;
  if (takes_tensor_cores(b, w, a.m, a.flags)) if (tb_status s = reserve_prefill(b, w, a.m)) return s;
  BlockExtras ex;
  ex.norm_weight = args->norm_weight; ex.norm_eps = args->norm_eps;
  ex.norm_zero_centered = (args->norm_flags & TB_NORM_ZERO_CENTERED) != 0; ex.residual = args->residual;
  ex.relu2_up = args->relu2_up;
  return forward_dev(b, w, a, st, receipt, ex);
}

extern "C" tb_status tb_act_absmax_dev(tb_backend* b, const void* x, tb_dtype x_dtype, uint32_t m, uint32_t k, float* out, void* stream) {
  clear_error();
  if (!b) return tb_fail(TB_NULL_ARG, "null argument");
  if (m == 0) return TB_OK;
  if (!x || !out) return tb_fail(TB_NULL_ARG, "null activation or output pointer");
  if (x_dtype != TB_F32 && x_dtype != TB_BF16) return tb_fail(TB_INVALID_INPUT, "activations must be fp32 or bf16");
  if (tb_status s = use_device(b)) return s;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : b->stream;
  TB_CUDA(tb_launch_row_absmax(x, x_dtype, m, k, out, st), "launch row absmax");
  return TB_OK;
}

namespace {
tb_status forward_tp(tb_backend* b, const tb_weights* w, tb_comm* comm, uint32_t slot_absmax, uint32_t slot_y, const void* x,
                     tb_dtype x_dtype, uint32_t m, void* y, tb_dtype y_dtype, uint32_t flags, void* stream, const BlockExtras& ex);
}

extern "C" tb_status tb_linear_forward_tp_dev(tb_backend* b, const tb_weights* w, tb_comm* comm, uint32_t slot_absmax, uint32_t slot_y,
                                               const void* x, tb_dtype x_dtype, uint32_t m, void* y, tb_dtype y_dtype, uint32_t flags,
                                               void* stream) {
  clear_error();
  return forward_tp(b, w, comm, slot_absmax, slot_y, x, x_dtype, m, y, y_dtype, flags, stream, BlockExtras{});
}

extern "C" tb_status tb_block_linear_forward_tp_dev(tb_backend* b, const tb_weights* w, tb_comm* comm, uint32_t slot_absmax,
                                                     uint32_t slot_y, const tb_norm_linear_args* args) {
  clear_error();
  if (!args) return tb_fail(TB_NULL_ARG, "args is null");
  if (args->norm_weight) return tb_fail(TB_INVALID_INPUT, "RMSNorm acts on the whole row: apply it in front of the column-parallel linear, not on a row shard");
  BlockExtras ex;
  ex.residual = args->residual; ex.relu2_up = args->relu2_up;
  return forward_tp(b, w, comm, slot_absmax, slot_y, args->x, args->x_dtype, args->m, args->y, args->y_dtype, args->flags, args->stream, ex);
}

namespace {
tb_status forward_tp(tb_backend* b, const tb_weights* w, tb_comm* comm, uint32_t slot_absmax, uint32_t slot_y, const void* x,
                     tb_dtype x_dtype, uint32_t m, void* y, tb_dtype y_dtype, uint32_t flags, void* stream, const BlockExtras& ex) {
  if (tb_status s = check_handles(b, w)) return s;
  if (!comm) return tb_fail(TB_NULL_ARG, "communicator is null");
  if (tb_comm_owner(comm) != b) return tb_fail(TB_INVALID_INPUT, "communicator belongs to another backend context");
  if (m == 0 || w->n == 0) return TB_OK;
  if (!x || !y) return tb_fail(TB_NULL_ARG, "null activation or output pointer");
  if (x_dtype == TB_I8) return tb_fail(TB_INVALID_INPUT, "the tensor-parallel path quantises fp32 or bf16 activations itself");
  if (y_dtype == TB_I8) return tb_fail(TB_INVALID_INPUT, "output dtype must be fp32 or bf16");
  if (m > 8) return tb_fail(TB_INVALID_INPUT, "the fused tensor-parallel path takes at most 8 tokens per call");
  if (flags & ~TB_FWD_PDL) return tb_fail(TB_INVALID_INPUT, "unknown flag bits");
  if (ex.relu2_up && x_dtype != TB_F32) return tb_fail(TB_INVALID_INPUT, "the squared-ReLU gate takes the fp32 outputs of the gate and up projections");
  if (!w->fast) return tb_fail(TB_UNSUPPORTED_FORMAT, "the int8 path needs uniform plane counts, k % 256 == 0, group 128 and codec D2 or B3");
  if (slot_absmax == slot_y) return tb_fail(TB_INVALID_INPUT, "the absmax and the output slot must differ");
  TbCommView va{}, vy{};
  if (!tb_comm_view(comm, slot_absmax, &va) || !tb_comm_view(comm, slot_y, &vy))
    return tb_fail(TB_INVALID_INPUT, "communicator is not connected or a slot index is out of range");
  if (tb_status s = use_device(b)) return s;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : b->stream;
  if (va.world <= 1) {
    tb_forward_args a{};
    a.x = x; a.x_dtype = x_dtype; a.m = m; a.y = y; a.y_dtype = y_dtype; a.flags = TB_FWD_A8 | TB_FWD_FORCE_DECODE | flags;
    return forward_dev(b, w, a, st, nullptr, ex);
  }
  // every rank's partial rows of one pass (8-byte words: value and round), in two alternating copies
  const size_t need_y = size_t(2) * va.world * std::min<uint32_t>(4, m) * w->n * 8;
  if (need_y > tb_comm_slot_bytes(comm))
    return tb_fail(TB_INVALID_INPUT, "the output slot holds " + std::to_string(tb_comm_slot_bytes(comm)) + " bytes, 2 x world x tokens x n 8-byte words need " +
                                         std::to_string(need_y));
  if (tb_comm_slot_bytes(comm) < kCommAbsmaxBytes) return tb_fail(TB_INVALID_INPUT, "the absmax slot is smaller than 2 KiB");
  for (uint32_t m0 = 0; m0 < m; m0 += 4) {
    const uint32_t mc = std::min<uint32_t>(4, m - m0);
    if (!tb_decode_supported(w, mc, b->max_smem_optin, nullptr))
      return tb_fail(TB_UNSUPPORTED_FORMAT, "the decode kernel's shared-memory plan does not fit this shape");
    DecodeArgs d{};
    d.w = w; d.x_dtype = x_dtype; d.m = mc; d.y_row_stride = uint32_t(w->n);
    d.x = static_cast<const uint8_t*>(x) + size_t(m0) * w->k * dtype_size(x_dtype);
    d.y = static_cast<uint8_t*>(y) + size_t(m0) * w->n * dtype_size(y_dtype); d.y_dtype = y_dtype;
    d.status = b->d_status; d.pdl = (flags & TB_FWD_PDL) != 0 || m0 > 0;
    d.scratch = b->d_prep; d.scratch_bytes = b->d_prep_cap;
    d.comm_absmax = &va; d.comm_y = &vy;
    // the gate acts on this rank's slice of the row; the residual is added once, behind the sum over the ranks
    d.relu2_up = ex.relu2_up ? ex.relu2_up + size_t(m0) * w->k : nullptr;
    d.residual = ex.residual ? ex.residual + size_t(m0) * w->n : nullptr;
    // Small tables: ONE launch (absmax exchange in the table builder, output sum in the epilogue).
    // Large tables: the preparation kernel exchanges the absmax, the decode kernel sums the outputs.
    d.fused = tb_decode_builds_tables(w, mc, d.x);
    if (!d.fused) TB_CUDA(tb_launch_prepare(d, st), "launch prepare");
    TB_CUDA(tb_launch_decode(d, b->prop.multiProcessorCount, b->max_smem_optin, st), "launch decode");
  }
  return TB_OK;
}
}  // namespace

extern "C" tb_status tb_backend_reserve(tb_backend* b, const tb_weights* w, uint32_t max_m) {
  clear_error();
  if (tb_status s = check_handles(b, w)) return s;
  if (tb_status s = use_device(b)) return s;
  return reserve_prefill(b, w, max_m);
}

extern "C" tb_status tb_salt_v2_gather_rows(tb_backend* b, const tb_weights* w, const uint32_t* rows, size_t count, float* out) {
  clear_error();
  if (tb_status s = check_handles(b, w)) return s;
  if (count == 0) return TB_OK;
  if (!rows || !out) return tb_fail(TB_NULL_ARG, "null argument");
  for (size_t i = 0; i < count; ++i)
    if (rows[i] >= w->n) return tb_fail(TB_INVALID_INPUT, "token_embd row " + std::to_string(rows[i]) + " is out of range");
  if (tb_status s = use_device(b)) return s;
  const size_t ob = count * w->k * 4;
  if (tb_status s = ensure(&b->d_x, &b->d_x_cap, count * 4)) return s;
  if (tb_status s = ensure(&b->d_y, &b->d_y_cap, ob)) return s;
  TB_CUDA(cudaMemcpyAsync(b->d_x, rows, count * 4, cudaMemcpyHostToDevice, b->stream), "copy row ids");
  TB_CUDA(tb_launch_gather_rows(w, static_cast<const uint32_t*>(b->d_x), uint32_t(count), static_cast<float*>(b->d_y), b->stream), "launch gather");
  TB_CUDA(cudaMemcpyAsync(out, b->d_y, ob, cudaMemcpyDeviceToHost, b->stream), "copy rows to host");
  TB_CUDA(cudaStreamSynchronize(b->stream), "synchronize stream");
  return TB_OK;
}

// ---------------------------------------------------------------- trait path
namespace {
tb_status check_trait_shape(const tb_weights* w, uint32_t n, uint32_t k) {
  if (!w->is_tq2) return tb_fail(TB_INVALID_INPUT, "buffer is not a TQ2_0 upload");
  if (w->n != n || w->logical_k != k)
    return fail_shape(w->n * w->logical_k, uint64_t(n) * k);
  return TB_OK;
}
// Rows are stored padded to whole 256-trit blocks; widen [m,k] to [m,kp] with zeros.
void pad_rows(const float* src, uint32_t m, uint32_t k, uint64_t kp, std::vector<float>* dst) {
  dst->assign(size_t(m) * kp, 0.f);
  for (uint32_t r = 0; r < m; ++r) std::copy(src + size_t(r) * k, src + size_t(r + 1) * k, dst->begin() + size_t(r) * kp);
}
}  // namespace

extern "C" tb_status tb_mpgemm(tb_backend* b, const tb_weights* w, const float* act, const float* scales, uint32_t m, uint32_t n,
                               uint32_t k, float* out) {
  clear_error();
  if (tb_status s = check_handles(b, w)) return s;
  if (tb_status s = check_trait_shape(w, n, k)) return s;
  if (m == 0 || n == 0) return TB_OK;
  if (!act || !scales || !out) return tb_fail(TB_NULL_ARG, "null argument");
  // Integer-valued activations in [-128,127] (what TernaryLinear::forward hands over after its
  // host quantisation) take the exact int8 kernel with a unit token scale.
  bool a8 = true;
  for (size_t i = 0; i < size_t(m) * k && a8; ++i) a8 = act[i] >= -128.f && act[i] <= 127.f && act[i] == std::trunc(act[i]);
  std::vector<float> padded;
  const float* x = act;
  if (w->k != k) { pad_rows(act, m, k, w->k, &padded); x = padded.data(); }
  if (!a8) return forward_host(b, w, x, TB_F32, m, out, TB_F32, nullptr, scales, 0, nullptr);
  // int8 path: quantising integers with absmax 127 reproduces them exactly only when the row
  // maximum is 127, so feed the codes directly as int8 with act_scale = 1.
  if (tb_status s = use_device(b)) return s;
  std::vector<int8_t> q(size_t(m) * w->k);
  for (size_t i = 0; i < q.size(); ++i) q[i] = int8_t(int(x[i]));
  const size_t yb = size_t(m) * n * 4;
  if (tb_status s = ensure(&b->d_x, &b->d_x_cap, q.size())) return s;
  if (tb_status s = ensure(&b->d_y, &b->d_y_cap, yb)) return s;
  if (tb_status s = ensure(&b->d_aux, &b->d_aux_cap, size_t(n) * 4 + size_t(m) * 4 + 256)) return s;
  if (tb_status s = reserve_prefill(b, w, m)) return s;
  float* d_rs = static_cast<float*>(b->d_aux);
  float* d_as = d_rs + n;
  std::vector<float> ones(m, 1.0f);
  TB_CUDA(cudaMemcpyAsync(b->d_x, q.data(), q.size(), cudaMemcpyHostToDevice, b->stream), "copy activations to device");
  TB_CUDA(cudaMemcpyAsync(d_rs, scales, size_t(n) * 4, cudaMemcpyHostToDevice, b->stream), "copy scales to device");
  TB_CUDA(cudaMemcpyAsync(d_as, ones.data(), size_t(m) * 4, cudaMemcpyHostToDevice, b->stream), "copy token scales to device");
  tb_forward_args a{};
  a.x = b->d_x; a.x_dtype = TB_I8; a.act_scale = d_as; a.m = m; a.y = b->d_y; a.y_dtype = TB_F32; a.row_scale = d_rs; a.flags = TB_FWD_A8;
  if (tb_status s = forward_dev(b, w, a, b->stream, nullptr)) return s;
  if (tb_status s = tb_backend_check(b, b->stream)) return s;
  TB_CUDA(cudaMemcpyAsync(out, b->d_y, yb, cudaMemcpyDeviceToHost, b->stream), "copy output to host");
  TB_CUDA(cudaStreamSynchronize(b->stream), "synchronize stream");
  return TB_OK;
}

extern "C" tb_status tb_mpgemm_with_act_quant(tb_backend* b, const tb_weights* w, const float* act, const float* scales, uint32_t m,
                                              uint32_t n, uint32_t k, float* out) {
  clear_error();
  if (tb_status s = check_handles(b, w)) return s;
  if (tb_status s = check_trait_shape(w, n, k)) return s;
  if (m == 0 || n == 0) return TB_OK;
  if (!act || !scales || !out) return tb_fail(TB_NULL_ARG, "null argument");
  std::vector<float> padded;
  const float* x = act;
  if (w->k != k) { pad_rows(act, m, k, w->k, &padded); x = padded.data(); }
  return forward_host(b, w, x, TB_F32, m, out, TB_F32, nullptr, scales, TB_FWD_A8, nullptr);
}

// ---------------------------------------------------------------- layer stack
namespace {
// A run of consecutive layers that all read the stack input and share one geometry: launched
// as ONE grouped decode (a single persistent grid streams every layer's weights back to back).
struct StackGroup {
  size_t first = 0, count = 0;
  TbLayerDesc* d_descs = nullptr;
  void* y = nullptr;          // [count][max_m][n] bf16
};
}  // namespace

struct tb_stack {
  tb_backend* backend = nullptr;
  std::vector<const tb_weights*> layers;
  std::vector<uint8_t> chain;
  std::vector<StackGroup> groups;
  std::vector<int> group_of;           // layer -> group index or -1
  uint32_t max_m = 0;
  void* buf[2] = {nullptr, nullptr};   // ping-pong activations (bf16)
  size_t buf_bytes = 0;
};

extern "C" tb_status tb_stack_create(tb_backend* b, const tb_weights* const* weights, const uint8_t* chain, uint32_t layers,
                                     uint32_t max_m, tb_stack** out) {
  clear_error();
  if (!b || !weights || !out) return tb_fail(TB_NULL_ARG, "null argument");
  *out = nullptr;
  if (b->released.load()) return tb_fail(TB_INVALID_INPUT, "the backend context was freed");
  if (!layers || !max_m) return tb_fail(TB_INVALID_INPUT, "a stack needs at least one layer and one token");
  if (tb_status s = use_device(b)) return s;
  tb_stack* st = new (std::nothrow) tb_stack();
  if (!st) return tb_fail(TB_OUT_OF_MEMORY, "host allocation failed");
  st->backend = b; st->max_m = max_m;
  uint64_t widest = 0;
  for (uint32_t i = 0; i < layers; ++i) {
    const tb_weights* w = weights[i];
    if (!w || w->owner != b || !w->fast) { delete st; return tb_fail(TB_INVALID_INPUT, "stack layers must be fast-path weights of this backend"); }
    const bool chained = chain && chain[i];
    if (chained && (i == 0 || weights[i - 1]->n != w->k)) { delete st; return tb_fail(TB_SHAPE_MISMATCH, "chained layer input width differs from the previous output width"); }
    if (!chained && i > 0 && w->k != weights[0]->k) { delete st; return tb_fail(TB_SHAPE_MISMATCH, "unchained layers read the stack input and must share its width"); }
    st->layers.push_back(w);
    st->chain.push_back(chained ? 1 : 0);
    widest = std::max<uint64_t>(widest, w->n);
    if (tb_status s = reserve_prefill(b, w, max_m)) { delete st; return s; }
  }
  tb_backend_retain(b);   // from here on every exit goes through tb_stack_free
  st->group_of.assign(layers, -1);
  auto same_geometry = [](const tb_weights* p, const tb_weights* q) {
    return p->k == q->k && p->n == q->n && p->codec == q->codec && p->uniform_planes == q->uniform_planes &&
           p->plan.rows_per_stage == q->plan.rows_per_stage;
  };
  for (uint32_t i = 0; i < layers;) {
    uint32_t e = i + 1;
    // a grouped run must not feed a chained successor (its outputs live in the group buffer)
    if (!st->chain[i])
      while (e < layers && !st->chain[e] && same_geometry(st->layers[i], st->layers[e])) ++e;
    const bool feeds_chain = e < layers && st->chain[e];
    if (e - i > 128) e = i + 128;   // descriptor capacity of one grouped launch
    if (e - i >= 2 && !feeds_chain) {
      StackGroup g;
      g.first = i; g.count = e - i;
      std::vector<TbLayerDesc> descs;
      for (uint32_t l = i; l < e; ++l) descs.push_back(TbLayerDesc{st->layers[l]->d_payload, st->layers[l]->d_scales});
      cudaError_t err = cudaMalloc(&g.d_descs, descs.size() * sizeof(TbLayerDesc));
      if (err == cudaSuccess) err = cudaMemcpy(g.d_descs, descs.data(), descs.size() * sizeof(TbLayerDesc), cudaMemcpyHostToDevice);
      if (err == cudaSuccess) err = cudaMalloc(&g.y, g.count * size_t(max_m) * st->layers[i]->n * 2);
      if (err != cudaSuccess) { cudaFree(g.d_descs); cudaFree(g.y); tb_stack_free(st); return tb_cuda_fail(err, "allocate layer group"); }
      for (uint32_t l = i; l < e; ++l) st->group_of[l] = int(st->groups.size());
      st->groups.push_back(g);
    }
    i = e;
  }
  st->buf_bytes = size_t(max_m) * widest * 2;
  for (int i = 0; i < 2; ++i) {
    cudaError_t err = cudaMalloc(&st->buf[i], st->buf_bytes);
    if (err != cudaSuccess) { tb_stack_free(st); return tb_cuda_fail(err, "allocate stack activations"); }
  }
  *out = st;
  return TB_OK;
}

extern "C" tb_status tb_stack_forward_dev(tb_stack* st, const void* x, tb_dtype xd, uint32_t m, void* y_last, tb_dtype yd,
                                          uint32_t flags, void* stream) {
  clear_error();
  if (!st || !x) return tb_fail(TB_NULL_ARG, "null argument");
  if (m == 0) return TB_OK;
  if (m > st->max_m) return tb_fail(TB_SHAPE_MISMATCH, "token count exceeds the stack's max_m");
  tb_backend* b = st->backend;
  if (tb_status s = use_device(b)) return s;
  cudaStream_t cs = stream ? static_cast<cudaStream_t>(stream) : b->stream;
  const size_t n_layers = st->layers.size();
  if (y_last && st->group_of[n_layers - 1] >= 0)
    return tb_fail(TB_INVALID_INPUT, "the last layer belongs to a grouped run: its output is read with tb_stack_read_output, y_last must be NULL");
  for (size_t i = 0; i < n_layers; ++i) {
    const int gi = st->group_of[i];
    if (gi >= 0) {
      // A run of layers that read the stack input.  Outputs go to the group buffer as
      // [layer][m][n] bf16, whichever kernel family runs.
      const StackGroup& g = st->groups[gi];
      const tb_weights* w = st->layers[i];
      const bool prefill = takes_tensor_cores(b, w, m, flags, 16);
      if (prefill) {
        for (size_t l = 0; l < g.count; ++l) {
          tb_forward_args a{};
          a.x = x; a.x_dtype = xd; a.m = m;
          a.y = static_cast<uint8_t*>(g.y) + l * size_t(m) * w->n * 2; a.y_dtype = TB_BF16;
          a.flags = TB_FWD_A8 | (flags & (TB_FWD_PDL | TB_FWD_FORCE_DECODE | TB_FWD_FORCE_PREFILL));
          a.stream = cs;
          if (tb_status s = forward_dev(b, st->layers[i + l], a, cs, nullptr)) return s;
        }
      } else {
        // one grouped decode launch per pass of up to four tokens
        for (uint32_t m0 = 0; m0 < m; m0 += 4) {
          const uint32_t mc = std::min<uint32_t>(4, m - m0);
          DecodeArgs d{};
          d.w = w; d.x_dtype = xd; d.m = mc; d.y_dtype = TB_BF16; d.y_row_stride = uint32_t(w->n);
          d.x = static_cast<const uint8_t*>(x) + size_t(m0) * w->k * dtype_size(xd);
          d.y = static_cast<uint8_t*>(g.y) + size_t(m0) * w->n * 2;
          d.status = b->d_status; d.pdl = (flags & TB_FWD_PDL) != 0 || m0 > 0;
          d.fused = tb_decode_builds_tables(w, mc, d.x);
          d.scratch = b->d_prep; d.scratch_bytes = b->d_prep_cap;
          d.layers = g.d_descs; d.layer_count = uint32_t(g.count); d.y_layer_stride = uint32_t(size_t(m) * w->n);
          if (!tb_decode_supported(w, mc, b->max_smem_optin, nullptr))
            return tb_fail(TB_UNSUPPORTED_FORMAT, "the decode kernel's shared-memory plan does not fit this shape");
          if (!d.fused) TB_CUDA(tb_launch_prepare(d, cs), "launch prepare");
          TB_CUDA(tb_launch_decode(d, b->prop.multiProcessorCount, b->max_smem_optin, cs), "launch grouped decode");
        }
      }
      i += g.count - 1;
      continue;
    }
    tb_forward_args a{};
    const bool chained = st->chain[i] != 0, last = i + 1 == n_layers;
    a.x = chained ? st->buf[(i + 1) & 1] : x;
    a.x_dtype = chained ? TB_BF16 : xd;
    a.m = m;
    a.y = (last && y_last) ? y_last : st->buf[i & 1];
    a.y_dtype = (last && y_last) ? yd : TB_BF16;
    a.flags = TB_FWD_A8 | (flags & (TB_FWD_PDL | TB_FWD_FORCE_DECODE | TB_FWD_FORCE_PREFILL));
    a.stream = cs;
    if (tb_status s = forward_dev(b, st->layers[i], a, cs, nullptr)) return s;
  }
  return TB_OK;
}

/* Host-pointer pass over a stack whose layers all read the stack input (every layer belongs to a
 * grouped run, m <= 4): one copy of x to the device, one prepare + one grouped launch per run,
 * one copy of every layer's bf16 output ([layer][m][n], layers in stack order) back, one
 * synchronisation.  `y` is written only when the device status is clean. */
extern "C" tb_status tb_stack_forward_host(tb_stack* st, const void* x, tb_dtype xd, uint32_t m, void* y_bf16, uint32_t flags) {
  clear_error();
  if (!st || !x || !y_bf16) return tb_fail(TB_NULL_ARG, "null argument");
  if (m == 0) return TB_OK;
  if (m > st->max_m) return tb_fail(TB_SHAPE_MISMATCH, "token count exceeds the stack's max_m");
  if (xd == TB_I8) return tb_fail(TB_INVALID_INPUT, "host int8 activations are not accepted here; pass fp32 or bf16");
  for (int gi : st->group_of)
    if (gi < 0) return tb_fail(TB_INVALID_INPUT, "every layer of the stack must belong to a grouped run");
  tb_backend* b = st->backend;
  if (tb_status s = use_device(b)) return s;
  const size_t xb = size_t(m) * st->layers[0]->k * dtype_size(xd);
  size_t yb = 0;
  for (const tb_weights* w : st->layers) yb += size_t(m) * w->n * 2;
  const size_t y_off = (xb + 255) / 256 * 256;
  if (tb_status s = ensure(&b->d_x, &b->d_x_cap, xb)) return s;
  if (tb_status s = ensure(&b->h_pin, &b->h_pin_cap, y_off + yb, true)) return s;
  uint8_t* pin = static_cast<uint8_t*>(b->h_pin);
  std::memcpy(pin, x, xb);
  TB_CUDA(cudaMemcpyAsync(b->d_x, pin, xb, cudaMemcpyHostToDevice, b->stream), "copy activations to device");
  if (tb_status s = tb_stack_forward_dev(st, b->d_x, xd, m, nullptr, TB_BF16, flags, b->stream)) return s;
  size_t off = y_off;
  for (const StackGroup& g : st->groups) {
    const size_t bytes = g.count * size_t(m) * st->layers[g.first]->n * 2;
    TB_CUDA(cudaMemcpyAsync(pin + off, g.y, bytes, cudaMemcpyDeviceToHost, b->stream), "copy group outputs to host");
    off += bytes;
  }
  TB_CUDA(cudaMemcpyAsync(b->h_status, b->d_status, 8 * sizeof(uint32_t), cudaMemcpyDeviceToHost, b->stream), "read status");
  TB_CUDA(cudaStreamSynchronize(b->stream), "synchronize stream");
  if (b->h_status[TBS_FLAGS]) return tb_backend_check(b, b->stream);
  std::memcpy(y_bf16, pin + y_off, yb);
  return TB_OK;
}

/* Copies the bf16 outputs of grouped layer `layer` (as [m][n]) to `out` on the host; used by
 * tests and by callers that consume every projection of a group. */
extern "C" tb_status tb_stack_read_output(tb_stack* st, uint32_t layer, uint32_t m, void* out_bf16) {
  clear_error();
  if (!st || !out_bf16) return tb_fail(TB_NULL_ARG, "null argument");
  if (layer >= st->layers.size() || st->group_of[layer] < 0) return tb_fail(TB_INVALID_INPUT, "layer is not part of a grouped run");
  if (m == 0 || m > st->max_m) return tb_fail(TB_SHAPE_MISMATCH, "token count exceeds the stack's max_m");
  if (tb_status s = use_device(st->backend)) return s;
  const StackGroup& g = st->groups[st->group_of[layer]];
  const size_t per_layer = size_t(m) * st->layers[layer]->n * 2;
  TB_CUDA(cudaStreamSynchronize(st->backend->stream), "synchronize stream");
  TB_CUDA(cudaMemcpy(out_bf16, static_cast<const uint8_t*>(g.y) + (layer - g.first) * per_layer, per_layer, cudaMemcpyDeviceToHost), "copy group output");
  return TB_OK;
}

extern "C" uint64_t tb_stack_bytes_per_step(const tb_stack* st, uint32_t m) {
  if (!st) return 0;
  uint64_t total = 0;
  for (const tb_weights* w : st->layers)
    total += w->payload_bytes + w->scale_count * 2 + w->map_bytes + w->rank_prefix_bytes + uint64_t(m) * (w->k + w->n) * 2;
  return total;
}

extern "C" void tb_stack_free(tb_stack* st) {
  if (!st) return;
  if (st->backend) cudaSetDevice(st->backend->ordinal);
  for (StackGroup& g : st->groups) { cudaFree(g.d_descs); cudaFree(g.y); }
  cudaFree(st->buf[0]); cudaFree(st->buf[1]);
  tb_backend* owner = st->backend;
  delete st;
  tb_backend_release(owner);
}

// ---------------------------------------------------------------- tensor-parallel shards (host)
extern "C" tb_status tb_tp_shard_sizes(tb_codec codec, uint32_t group, uint32_t n, uint32_t k, uint32_t planes, int row_parallel,
                                       uint32_t world, uint32_t rank, tb_shard_sizes* out) {
  clear_error();
  if (!out) return tb_fail(TB_NULL_ARG, "out is null");
  tbf::ShardSizes s;
  if (tbf::Err e = tbf::shard_sizes(int(codec), group, n, k, planes, row_parallel != 0, world, rank, &s)) return from_fmt(e);
  out->n = s.n; out->k = s.k; out->payload_bytes = s.payload_bytes; out->scale_count = s.scale_count; out->map_bytes = s.map_bytes;
  return TB_OK;
}

extern "C" tb_status tb_tp_shard(tb_codec codec, uint32_t group, uint32_t n, uint32_t k, uint32_t planes, const uint8_t* payload,
                                 const uint16_t* scales, int row_parallel, uint32_t world, uint32_t rank, uint8_t* sp, uint16_t* ss,
                                 uint8_t* smap, uint32_t* terminal) {
  clear_error();
  if (!payload || !scales || !sp || !ss || !terminal) return tb_fail(TB_NULL_ARG, "null argument");
  uint8_t dummy = 0;
  if (tbf::Err e = tbf::shard(int(codec), group, n, k, planes, payload, scales, row_parallel != 0, world, rank, sp, ss,
                              smap ? smap : &dummy, terminal))
    return from_fmt(e);
  return TB_OK;
}

// ---------------------------------------------------------------- host format helpers
extern "C" int64_t tb_fmt_pack(tb_codec codec, const int8_t* trits, size_t n, uint8_t* out, size_t cap) {
  clear_error();
  if (!trits && n) { tb_fail(TB_NULL_ARG, "trits is null"); return -TB_NULL_ARG; }
  if (codec == TB_CODEC_S34 && n % 4) { tb_fail(TB_INVALID_INPUT, "S34 requires a multiple of four trits"); return -TB_INVALID_INPUT; }
  const size_t bytes = tbf::codec_bytes(int(codec), n);
  if (!out) return int64_t(bytes);
  if (cap < bytes) { tb_fail(TB_SHAPE_MISMATCH, "output buffer too small"); return -TB_SHAPE_MISMATCH; }
  if (tbf::Err e = tbf::pack(int(codec), trits, n, out)) return -int64_t(from_fmt(e));
  return int64_t(bytes);
}

extern "C" tb_status tb_fmt_unpack(tb_codec codec, const uint8_t* packed, size_t len, size_t n, int8_t* trits) {
  clear_error();
  if ((!packed && len) || (!trits && n)) return tb_fail(TB_NULL_ARG, "null argument");
  if (tbf::Err e = tbf::unpack(int(codec), packed, len, n, trits)) return from_fmt(e);
  return TB_OK;
}

extern "C" size_t tb_fmt_plane_bytes(tb_codec codec, size_t logical_len) { return tbf::plane_bytes(int(codec), logical_len); }

extern "C" tb_status tb_fmt_resident_sizes(tb_codec codec, uint32_t group, uint64_t n, uint64_t k, const uint8_t* pc, tb_resident_sizes* out) {
  clear_error();
  if (!pc || !out) return tb_fail(TB_NULL_ARG, "null argument");
  tbf::Sizes s;
  if (tbf::Err e = tbf::resident_sizes(int(codec), group, n, k, pc, &s)) return from_fmt(e);
  out->payload_bytes = s.payload_bytes; out->scale_count = s.scale_count; out->map_bytes = s.map_bytes;
  out->rank_prefix_bytes = s.rank_prefix_bytes; out->tiles = s.tiles; out->present_planes = s.present_planes;
  return TB_OK;
}

extern "C" tb_status tb_fmt_resident_build(tb_codec codec, uint32_t group, uint64_t n, uint64_t k, const uint8_t* pc, const int8_t* trits,
                                           const uint16_t* scales, uint8_t* payload, uint16_t* scale_out, uint8_t* plane_map,
                                           uint32_t* terminal) {
  clear_error();
  if (!pc || !trits || !scales || !payload || !scale_out || !terminal) return tb_fail(TB_NULL_ARG, "null argument");
  tbf::Resident r;
  if (tbf::Err e = tbf::resident_from_planes(int(codec), group, n, k, pc, trits, scales, &r)) return from_fmt(e);
  std::copy(r.payload.begin(), r.payload.end(), payload);
  std::copy(r.scales.begin(), r.scales.end(), scale_out);
  if (plane_map) std::copy(r.map.begin(), r.map.end(), plane_map);
  *terminal = r.terminal_map;
  return TB_OK;
}

extern "C" tb_status tb_fmt_device_layout(tb_codec codec, uint32_t group, uint32_t n, uint32_t k, const uint8_t* payload,
                                          size_t payload_len, const uint16_t* scales, size_t scale_count, const uint8_t* plane_map,
                                          size_t map_len, uint32_t terminal, tb_device_layout* info, uint8_t* payload_out,
                                          uint16_t* scales_out) {
  clear_error();
  if (!payload || !scales || !info || (!plane_map && map_len)) return tb_fail(TB_NULL_ARG, "null argument");
  tbf::Resident r, relaid;
  if (tbf::Err e = tbf::resident_from_arenas(int(codec), group, n, k, payload, payload_len, scales, scale_count, plane_map, map_len, terminal, &r))
    return from_fmt(e);
  bool recoded = false, map_counts = false;
  if (tbf::Err e = tbf::device_layout(r, &relaid, &recoded, &map_counts)) return from_fmt(e);
  const tbf::Resident& d = (recoded || map_counts) ? relaid : r;
  info->codec = uint32_t(d.codec); info->planes_uniform = d.uniform_planes; info->counts_from_map = map_counts ? 1u : 0u;
  info->recoded = recoded ? 1u : 0u; info->payload_bytes = d.payload.size(); info->scale_count = d.scales.size();
  if (payload_out) std::copy(d.payload.begin(), d.payload.end(), payload_out);
  if (scales_out) std::copy(d.scales.begin(), d.scales.end(), scales_out);
  return TB_OK;
}

extern "C" int64_t tb_fmt_package_write(tb_codec codec, const char* name, uint32_t group, uint64_t n, uint64_t k, const uint8_t* pc,
                                        const int8_t* trits, const uint16_t* scales, uint8_t* out, size_t cap) {
  clear_error();
  if (!name || !pc || !trits || !scales) { tb_fail(TB_NULL_ARG, "null argument"); return -TB_NULL_ARG; }
  std::vector<uint8_t> bytes;
  if (tbf::Err e = tbf::package_write(int(codec), name, group, n, k, pc, trits, scales, &bytes)) return -int64_t(from_fmt(e));
  if (!out) return int64_t(bytes.size());
  if (cap < bytes.size()) { tb_fail(TB_SHAPE_MISMATCH, "output buffer too small"); return -TB_SHAPE_MISMATCH; }
  std::copy(bytes.begin(), bytes.end(), out);
  return int64_t(bytes.size());
}

extern "C" int64_t tb_fmt_package_write_multi(tb_codec codec, uint32_t count, const char* const* names, const uint32_t* groups,
                                              const uint64_t* n, const uint64_t* k, const uint8_t* const* pc, const int8_t* const* trits,
                                              const uint16_t* const* scales, uint8_t* out, size_t cap) {
  clear_error();
  if (!names || !groups || !n || !k || !pc || !trits || !scales) { tb_fail(TB_NULL_ARG, "null argument"); return -TB_NULL_ARG; }
  std::vector<tbf::PackageTensorIn> ts(count);
  for (uint32_t i = 0; i < count; ++i) {
    if (!names[i] || !pc[i] || !trits[i] || !scales[i]) { tb_fail(TB_NULL_ARG, "null tensor argument"); return -TB_NULL_ARG; }
    ts[i] = tbf::PackageTensorIn{names[i], groups[i], n[i], k[i], pc[i], trits[i], scales[i]};
  }
  std::vector<uint8_t> bytes;
  if (tbf::Err e = tbf::package_write_multi(int(codec), ts.data(), ts.size(), &bytes)) return -int64_t(from_fmt(e));
  if (!out) return int64_t(bytes.size());
  if (cap < bytes.size()) { tb_fail(TB_SHAPE_MISMATCH, "output buffer too small"); return -TB_SHAPE_MISMATCH; }
  std::copy(bytes.begin(), bytes.end(), out);
  return int64_t(bytes.size());
}

extern "C" tb_status tb_fmt_package_extract(tb_read_at_fn read_at, void* user, uint64_t package_len, const char* name,
                                            tb_package_tensor* info, uint8_t* payload, uint16_t* scales, uint8_t* plane_map) {
  clear_error();
  if (!read_at || !name || !info) return tb_fail(TB_NULL_ARG, "null argument");
  tbf::Resident r;
  if (tbf::Err e = tbf::resident_from_reader(read_at, user, package_len, name, &r)) return from_fmt(e);
  info->codec = uint32_t(r.codec); info->group = r.group; info->terminal_map_value = r.terminal_map; info->planes_uniform = r.uniform_planes;
  info->n = r.n; info->k = r.k; info->payload_bytes = r.payload.size(); info->scale_count = r.scales.size(); info->map_bytes = r.map.size();
  if (payload) std::copy(r.payload.begin(), r.payload.end(), payload);
  if (scales) std::copy(r.scales.begin(), r.scales.end(), scales);
  if (plane_map) std::copy(r.map.begin(), r.map.end(), plane_map);
  return TB_OK;
}

extern "C" tb_status tb_fmt_tq2_pack_rows(const int8_t* trits, uint64_t n, uint64_t k, uint8_t* out) {
  clear_error();
  if (!trits || !out) return tb_fail(TB_NULL_ARG, "null argument");
  if (tbf::Err e = tbf::tq2_pack_rows(trits, n, k, out)) return from_fmt(e);
  return TB_OK;
}

extern "C" void tb_fmt_quantize_act_int8(const float* act, uint64_t m, uint64_t k, float* q, float* scale) {
  if (!act || !q || !scale) return;
  tbf::quantize_act_int8(act, m, k, q, scale);
}
