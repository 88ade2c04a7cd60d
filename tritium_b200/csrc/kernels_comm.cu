// One-shot all-reduce over peer memory for the small messages of tensor-parallel decode.
//
// Every rank owns one device allocation (data slots followed by flag words) that its peers map
// with CUDA IPC.  A reduce of slot s:
//   1. each rank (block 0) raises flag[s][rank] = seq in every peer's allocation with a
//      system-scope release store: "my partial for this round is in my memory";
//   2. every block waits (bounded) until all peers' flags in its OWN memory have reached seq;
//   3. every block reads its slice of all ranks' partials with ordinary peer loads (no TMA, no
//      multicast), combines them in rank order (so every rank gets the same bits) and writes
//      the result to local memory;
//   4. the last block to finish publishes seq as the slot's epoch for the next launch.
// seq comes from device memory, so the same launch can be replayed from a CUDA graph.
// A slot's partial may be overwritten again only after another reduce of the same group has
// been passed (every rank has then finished reading it); callers rotate at least two slots.
#include <cuda_runtime.h>

#include <cstring>
#include <new>
#include <string>

#include "tb_internal.h"

namespace {

constexpr uint32_t kMaxWorld = 8;
constexpr long long kCommWaitCycles = 4000000000ll;   // about two seconds of SM clocks

struct ReduceParams {
  const float* data[kMaxWorld];   // every rank's slot (own pointer for this rank)
  uint32_t* peer_flags[kMaxWorld];   // every rank's flag row for this slot
  uint32_t* my_flags;             // this rank's flag row for the slot: [world]
  uint32_t* epoch;                // this rank's epoch word for the slot
  uint32_t* done;                 // this rank's block counter for the slot
  float* out;
  uint32_t* status;
  uint32_t rank, world, count, op;   // op: 0 sum, 1 max
  long long wait_cycles;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_peer1(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) oneshot_reduce_kernel(const ReduceParams p) {
  __shared__ uint32_t failed;
  const uint32_t tid = threadIdx.x;
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(p.epoch) + 1u;
  if (tid == 0) failed = 0;
  __syncthreads();
  if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
    __threadfence_system();
    st_release_sys(p.peer_flags[tid] + p.rank, seq);
  }
  if (tid < p.world && tid != p.rank) {
    const long long t0 = clock64();
    for (uint32_t i = 0;; ++i) {
      // flags only grow; a peer that is already one round ahead has passed this one
      if (int32_t(ld_acquire_sys(p.my_flags + tid) - seq) >= 0) break;
      if ((i & 63u) == 63u && clock64() - t0 > p.wait_cycles) {
        failed = 1;
        if (atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = tid; p.status[TBS_INFO1] = 400; }
        break;
      }
    }
  }
  __syncthreads();
  if (!failed) {
    const uint32_t vec = p.count / 4;
    for (uint32_t i = blockIdx.x * blockDim.x + tid; i < vec; i += gridDim.x * blockDim.x) {
      float4 acc = p.rank == 0 ? *reinterpret_cast<const float4*>(p.data[0] + 4 * size_t(i)) : ld_peer4(p.data[0] + 4 * size_t(i));
      for (uint32_t r = 1; r < p.world; ++r) {
        const float4 v = r == p.rank ? *reinterpret_cast<const float4*>(p.data[r] + 4 * size_t(i)) : ld_peer4(p.data[r] + 4 * size_t(i));
        if (p.op == 0) { acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w); }
        else { acc.x = fmaxf(acc.x, v.x); acc.y = fmaxf(acc.y, v.y); acc.z = fmaxf(acc.z, v.z); acc.w = fmaxf(acc.w, v.w); }
      }
      *reinterpret_cast<float4*>(p.out + 4 * size_t(i)) = acc;
    }
    for (uint32_t i = vec * 4 + blockIdx.x * blockDim.x + tid; i < p.count; i += gridDim.x * blockDim.x) {
      float acc = p.rank == 0 ? p.data[0][i] : ld_peer1(p.data[0] + i);
      for (uint32_t r = 1; r < p.world; ++r) {
        const float v = r == p.rank ? p.data[r][i] : ld_peer1(p.data[r] + i);
        acc = p.op == 0 ? __fadd_rn(acc, v) : fmaxf(acc, v);
      }
      p.out[i] = acc;
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.done, 1u) == gridDim.x - 1) {
      *p.done = 0;
      // also after a timeout: the next launch must not wait for a round that was given up
      *reinterpret_cast<volatile uint32_t*>(p.epoch) = seq;
    }
  }
}

}  // namespace

struct tb_comm {
  tb_backend* owner = nullptr;
  uint32_t world = 1, rank = 0, slots = 0, flag_words = 16;
  size_t slot_bytes = 0, data_bytes = 0, total_bytes = 0;
  uint8_t* base[kMaxWorld] = {};   // base[rank] is the local allocation, the others are IPC mappings
  bool connected = false;
  long long wait_cycles = kCommWaitCycles;
};

namespace {
uint32_t* flag_row(uint8_t* base, const tb_comm* c, uint32_t slot) {
  return reinterpret_cast<uint32_t*>(base + c->data_bytes) + size_t(slot) * c->flag_words;
}
}  // namespace

extern "C" tb_status tb_comm_create(tb_backend* b, uint32_t world, uint32_t rank, size_t slot_bytes, uint32_t slots,
                                    uint32_t counters_per_slot, tb_comm** out) {
  if (!b || !out) return tb_fail(TB_NULL_ARG, "null argument");
  *out = nullptr;
  if (b->released.load()) return tb_fail(TB_INVALID_INPUT, "the backend context was freed");
  if (world == 0 || world > kMaxWorld || rank >= world) return tb_fail(TB_INVALID_INPUT, "world must be 1..8 and rank below it");
  if (slots == 0 || slot_bytes == 0) return tb_fail(TB_INVALID_INPUT, "a communicator needs at least one slot of at least one byte");
  if (cudaSetDevice(b->ordinal) != cudaSuccess) return tb_fail(TB_BACKEND, "select device");
  tb_comm* c = new (std::nothrow) tb_comm();
  if (!c) return tb_fail(TB_OUT_OF_MEMORY, "host allocation failed");
  c->owner = b; c->world = world; c->rank = rank; c->slots = slots;
  c->slot_bytes = (slot_bytes + 255) / 256 * 256;
  c->data_bytes = c->slot_bytes * slots;
  c->flag_words = (kCommCounters + counters_per_slot + 15) / 16 * 16;
  c->total_bytes = c->data_bytes + size_t(slots) * c->flag_words * 4;
  void* mem = nullptr;
  cudaError_t err = cudaMalloc(&mem, c->total_bytes);
  if (err != cudaSuccess) { delete c; return tb_cuda_fail(err, "allocate communicator memory"); }
  if ((err = cudaMemset(mem, 0, c->total_bytes)) != cudaSuccess || (err = cudaDeviceSynchronize()) != cudaSuccess) {
    cudaFree(mem); delete c; return tb_cuda_fail(err, "clear communicator memory");
  }
  c->base[rank] = static_cast<uint8_t*>(mem);
  c->connected = world == 1;
  tb_backend_retain(b);
  *out = c;
  return TB_OK;
}

extern "C" tb_status tb_comm_export(const tb_comm* c, uint8_t* handle_out) {
  if (!c || !handle_out) return tb_fail(TB_NULL_ARG, "null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == TB_COMM_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  if (cudaSetDevice(c->owner->ordinal) != cudaSuccess) return tb_fail(TB_BACKEND, "select device");
  cudaError_t err = cudaIpcGetMemHandle(&h, c->base[c->rank]);
  if (err != cudaSuccess) return tb_cuda_fail(err, "export communicator memory");
  std::memcpy(handle_out, &h, sizeof h);
  return TB_OK;
}

extern "C" tb_status tb_comm_connect(tb_comm* c, const uint8_t* all_handles) {
  if (!c || !all_handles) return tb_fail(TB_NULL_ARG, "null argument");
  if (c->connected) return TB_OK;
  if (cudaSetDevice(c->owner->ordinal) != cudaSuccess) return tb_fail(TB_BACKEND, "select device");
  for (uint32_t r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, all_handles + size_t(r) * TB_COMM_HANDLE_BYTES, sizeof h);
    void* mapped = nullptr;
    cudaError_t err = cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess) return tb_cuda_fail(err, "map a peer's communicator memory");
    c->base[r] = static_cast<uint8_t*>(mapped);
  }
  c->connected = true;
  return TB_OK;
}

extern "C" void* tb_comm_slot(const tb_comm* c, uint32_t slot) {
  if (!c || slot >= c->slots) return nullptr;
  return c->base[c->rank] + size_t(slot) * c->slot_bytes;
}

extern "C" tb_status tb_comm_allreduce_f32(tb_comm* c, uint32_t slot, uint32_t count, int op_max, float* out, void* stream) {
  if (!c || !out) return tb_fail(TB_NULL_ARG, "null argument");
  if (!c->connected) return tb_fail(TB_INVALID_INPUT, "communicator is not connected to its peers");
  if (slot >= c->slots || size_t(count) * 4 > c->slot_bytes) return tb_fail(TB_INVALID_INPUT, "slot index or element count out of range");
  if (count == 0) return TB_OK;
  if (cudaSetDevice(c->owner->ordinal) != cudaSuccess) return tb_fail(TB_BACKEND, "select device");
  ReduceParams p{};
  for (uint32_t r = 0; r < c->world; ++r) {
    p.data[r] = reinterpret_cast<const float*>(c->base[r] + size_t(slot) * c->slot_bytes);
    p.peer_flags[r] = flag_row(c->base[r], c, slot);
  }
  uint32_t* mine = flag_row(c->base[c->rank], c, slot);
  p.my_flags = mine; p.epoch = mine + kMaxWorld; p.done = mine + kMaxWorld + 1;
  p.out = out; p.status = c->owner->d_status;
  p.rank = c->rank; p.world = c->world; p.count = count; p.op = op_max ? 1u : 0u;
  p.wait_cycles = c->wait_cycles;
  const uint32_t blocks = std::min<uint32_t>(32, (count / 4 + 255) / 256 + 1);
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : c->owner->stream;
  oneshot_reduce_kernel<<<blocks, 256, 0, st>>>(p);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return tb_cuda_fail(err, "launch one-shot reduce");
  return TB_OK;
}

bool tb_comm_view(const tb_comm* c, uint32_t slot, TbCommView* out) {
  if (!c || !c->connected || slot >= c->slots) return false;
  for (uint32_t r = 0; r < c->world; ++r) {
    out->data[r] = reinterpret_cast<float*>(c->base[r] + size_t(slot) * c->slot_bytes);
    out->flags[r] = flag_row(c->base[r], c, slot);
  }
  out->world = c->world; out->rank = c->rank; out->counters = c->flag_words - kCommCounters;
  out->wait_cycles = c->wait_cycles;
  return true;
}
size_t tb_comm_slot_bytes(const tb_comm* c) { return c ? c->slot_bytes : 0; }
const tb_backend* tb_comm_owner(const tb_comm* c) { return c ? c->owner : nullptr; }

extern "C" tb_status tb_comm_set_wait_limit(tb_comm* c, uint64_t sm_cycles) {
  if (!c) return tb_fail(TB_NULL_ARG, "null argument");
  if (sm_cycles == 0 || sm_cycles > (uint64_t(1) << 40)) return tb_fail(TB_INVALID_INPUT, "the wait limit must be between 1 and 2^40 SM cycles");
  c->wait_cycles = static_cast<long long>(sm_cycles);
  return TB_OK;
}

extern "C" tb_status tb_comm_disconnect(tb_comm* c) {
  if (!c) return tb_fail(TB_NULL_ARG, "null argument");
  if (cudaSetDevice(c->owner->ordinal) != cudaSuccess) return tb_fail(TB_BACKEND, "select device");
  cudaError_t err = cudaDeviceSynchronize();   // none of this rank's kernels may still read a peer
  for (uint32_t r = 0; r < c->world; ++r) {
    if (r == c->rank || !c->base[r]) continue;
    const cudaError_t e = cudaIpcCloseMemHandle(c->base[r]);
    if (err == cudaSuccess) err = e;
    c->base[r] = nullptr;
  }
  c->connected = c->world == 1;
  if (err != cudaSuccess) return tb_cuda_fail(err, "unmap the peers' communicator memory");
  return TB_OK;
}

extern "C" void tb_comm_free(tb_comm* c) {
  if (!c) return;
  tb_comm_disconnect(c);
  cudaFree(c->base[c->rank]);
  tb_backend* owner = c->owner;
  delete c;
  tb_backend_release(owner);
}
