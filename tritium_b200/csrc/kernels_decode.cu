// Decode GEMV (1..4 tokens) straight from the packed B3 / D2 arenas, sm_100a.
//
// Data movement: a CTA owns blocks of R consecutive output rows.  A row's tile-planes are
// contiguous in the payload arena and rows follow one another, so a block is ONE contiguous byte
// range; a producer warp streams it (and the matching f16 scale range) into a shared-memory ring
// with cp.async.bulk + mbarrier transaction counts.  Weights are read from HBM exactly once.
//
// Arithmetic: activations are int8 (per-token absmax quantisation fused into the prologue).
// B3 bytes are never expanded to trits.  For a byte b = sum d_i 3^i the five floor quotients
// q_i = floor(b / 3^i) come from half-precision FMAs on (1024 + b) (round-to-nearest of the FMA
// does the floor; constants verified exhaustively for b in [0,243)), and
//     sum_i d_i x_i = sum_i q_i (x_i - 3 x_{i-1})
// so the quotient bytes feed mma.sync.m16n8k32 (u8 x s8 -> s32) against pre-transformed
// activations z_i = x_i - 3 x_{i-1}, split as z = 4*zh + zl to fit int8 (two MMA columns per
// token).  q_0 is the raw byte: the packed word itself is an MMA operand.  Sums are exact int32
// per (row, 128-group, plane); the f16 group scale is applied once per sum in fp32.
// D2 words feed the MMA as unsigned 2-bit codes (t = code - 1) with z = x.
//
// Fragment roles (m16n8k32): MMA rows are 16 consecutive row-planes; lane (g = lane/4, c = lane%4)
// supplies rows g and g+8 from packed words c, 4+c, 8+c (and half of word 12 for B3).  The B
// operand (activations) is laid out in shared memory in exactly that k-slot order.  Trits that
// belong to the other scale group of a straddling byte, and B3 padding digits, are removed on
// the activation side (their z entries are zero), never by masking weights.
//
// Every wait is bounded; on timeout the kernel records TBF_WAIT_TIMEOUT and returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <string>

#include "tb_internal.h"

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxStages = 4;
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr int kMaxGroupLayers = 128;   // layers of one grouped launch (descriptors live in shared memory)

struct DecodeParams {
  const uint8_t* payload; const uint16_t* scales;   // single layer (layers == nullptr)
  const TbLayerDesc* layers; uint32_t layer_count; uint32_t y_layer_stride;   // grouped launch: outputs [layer][m][n]
  const uint8_t* tables; uint32_t table_bytes;   // z tables | accumulator start values | token scales
  void* y; int32_t* acc_dump; const float* row_scale;
  uint32_t* status;
  uint32_t m, n, k, planes, tpr;            // tpr = k / 256
  uint32_t rows_per_stage, row_bytes, stage_bytes, scale_stage_bytes, blocks;
  uint32_t stages, y_dtype, y_row_stride;
  uint32_t dump_token_offset, dump_tokens_total;
  uint32_t pdl, wait_tables, ctas_per_sm;
  // shared memory offsets (bytes)
  uint32_t off_ring, off_scale_ring, off_z, off_cinit, off_part, off_actscale, off_zero;
  TbCommView comm;   // world > 1: write fp32 partial rows into the slot and finish the all-reduce here
};

// ---- peer-memory helpers (tensor-parallel row shards)
constexpr long long kPeerWaitCycles = 4000000000ll;   // about two seconds of SM clocks
__device__ __forceinline__ void peer_signal(uint32_t* counter) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
}
__device__ __forceinline__ uint32_t peer_poll(const uint32_t* counter) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
  return v;
}
__device__ __forceinline__ float peer_load(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
// Waits (bounded) until `counter` has received `target` arrivals since the slot was created.
__device__ __forceinline__ bool peer_wait(const uint32_t* counter, uint32_t target) {
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    if (int32_t(peer_poll(counter) - target) >= 0) return true;
    if ((i & 255u) == 255u && clock64() - t0 > kPeerWaitCycles) return false;
  }
}

template <int CODEC> struct Traits;
// kMmas: MMAs per (16 row-planes x tile-plane) when the two scale groups use separate
// accumulators; kMmasDual: when they use separate MMA columns instead (1 or 2 tokens).
template <> struct Traits<tbf::kB3> { static constexpr int kMmas = 13, kMmasDual = 10, kPlaneBytes = 52; };
template <> struct Traits<tbf::kD2> { static constexpr int kMmas = 8, kMmasDual = 8, kPlaneBytes = 64; };
template <int CODEC, bool DUAL> struct MmaCount { static constexpr int value = DUAL ? Traits<CODEC>::kMmasDual : Traits<CODEC>::kMmas; };

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false after kSpinLimit polls or when another thread flagged an abort.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i >= 4) __nanosleep(100);   // waiting warps should not take issue slots from working ones
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A*B with a zero accumulator (starts a chain without clearing four registers first).
__device__ __forceinline__ void mma_u8s8_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// int -> float for |v| < 2^22 without the conversion unit: the integer is added into the mantissa
// of 1.5 * 2^23 and the constant is subtracted again (both steps exact).
__device__ __forceinline__ float group_sum_to_float(int v) {
  return __fsub_rn(__int_as_float(0x4B400000 + v), 12582912.0f);
}

// ---------------------------------------------------------------- B3 quotients
// Half constants (bit patterns, both halves).  For V = 1024 + v:
//   fma(V, 0x3553, 0x6156) = 1024 + floor(v/3)   for v in [0,242]
//   fma(V, 0x2f19, 0x631e) = 1025 + floor(v/9)   for v in [0,242]   (and for v in [0,80])
//   fma(1025+v, 0x2f1f, 0x631d) = 1025 + floor(v/9) for v in [0,26]
// so with Q1 = 1024+q1, Q2 = 1025+q2, Q3 = fma(Q1, ./9) = 1025+q3, Q4 = fma(Q2, ./9) = 1025+q4
// the low bytes are q1, 1+q2, 1+q3, 1+q4.  The "+1" offsets are folded into the accumulator
// start value on the activation side.
constexpr uint32_t kC3 = 0x35533553u, kK3 = 0x61566156u;
constexpr uint32_t kC9 = 0x2f192f19u, kK9 = 0x631e631eu;
constexpr uint32_t kC9b = 0x2f1f2f1fu, kK9b = 0x631d631du;
__device__ __forceinline__ void b3_quads(uint32_t w, uint32_t (&q)[5]) {
  const uint32_t h01 = prmt(w, 0x64646464u, 0x4140u);  // halves 1024+b0, 1024+b1
  const uint32_t h23 = prmt(w, 0x64646464u, 0x4342u);  // halves 1024+b2, 1024+b3
  const uint32_t a1 = hfma2_bits(h01, kC3, kK3), b1 = hfma2_bits(h23, kC3, kK3);
  const uint32_t a2 = hfma2_bits(h01, kC9, kK9), b2 = hfma2_bits(h23, kC9, kK9);
  const uint32_t a3 = hfma2_bits(a1, kC9, kK9), b3 = hfma2_bits(b1, kC9, kK9);
  const uint32_t a4 = hfma2_bits(a2, kC9b, kK9b), b4 = hfma2_bits(b2, kC9b, kK9b);
  q[0] = w;
  q[1] = prmt(a1, b1, 0x6420u);
  q[2] = prmt(a2, b2, 0x6420u);
  q[3] = prmt(a3, b3, 0x6420u);
  q[4] = prmt(a4, b4, 0x6420u);
}

// ---------------------------------------------------------------- activation-side tables
// Which packed word / digits / scale-group variant MMA number `mma` of a tile-plane consumes for
// the lane column c (0..3).
// bytewise: the MMA takes ONE packed byte per lane column (byte c of the word): register byte i of
// the first operand quad is digit i (0..3), byte 0 of the second quad is digit 4.
template <int CODEC> struct Slot { int word, variant, d0, d1, lane_lo, lane_hi; bool bytewise; };
template <int CODEC, bool DUAL> __device__ __forceinline__ Slot<CODEC> slot_of(int mma, int c);
template <> __device__ __forceinline__ Slot<tbf::kB3> slot_of<tbf::kB3, false>(int mma, int c) {
  // mma 0-2: words c (group 0); 3-5: words 4+c into group 0; 6-8: words 4+c into group 1;
  // 9-11: words 8+c (group 1); 12: byte c of word 12 (group 1).
  const int slot = mma < 3 ? 0 : mma < 9 ? 1 : mma < 12 ? 2 : 3;
  const int pair = mma % 3;
  Slot<tbf::kB3> s;
  s.variant = mma < 6 ? 0 : 1;
  s.d0 = pair * 2; s.d1 = pair == 2 ? -1 : pair * 2 + 1;
  s.word = slot < 3 ? slot * 4 + c : 12;
  s.lane_lo = 0; s.lane_hi = 4;
  s.bytewise = slot == 3;
  return s;
}
template <> __device__ __forceinline__ Slot<tbf::kB3> slot_of<tbf::kB3, true>(int mma, int c) {
  // three MMAs per packed word; the scale group is chosen by the MMA column, not by the MMA
  // (the tenth MMA takes byte c of word 12)
  const int slot = mma / 3, pair = mma % 3;
  Slot<tbf::kB3> s;
  s.variant = -1;
  s.d0 = pair * 2; s.d1 = pair == 2 ? -1 : pair * 2 + 1;
  s.word = slot < 3 ? slot * 4 + c : 12;
  s.lane_lo = 0; s.lane_hi = 4;
  s.bytewise = slot == 3;
  return s;
}
template <> __device__ __forceinline__ Slot<tbf::kD2> slot_of<tbf::kD2, false>(int mma, int c) {
  const int slot = mma >> 1;  // words c, 4+c (group 0), 8+c, 12+c (group 1)
  Slot<tbf::kD2> s;
  s.variant = slot >> 1;
  s.d0 = (mma & 1) * 2; s.d1 = s.d0 + 1;
  s.word = slot * 4 + c;
  s.lane_lo = 0; s.lane_hi = 4;
  s.bytewise = false;
  return s;
}
template <> __device__ __forceinline__ Slot<tbf::kD2> slot_of<tbf::kD2, true>(int mma, int c) {
  Slot<tbf::kD2> s = slot_of<tbf::kD2, false>(mma, c);
  s.variant = -1;
  return s;
}

// z value of (byte-lane e of packed word `word`, digit/slot i) for scale-group `variant`.
template <int CODEC>
__device__ __forceinline__ int z_value(const int8_t* xq_tile, int word, int e, int i, int variant) {
  if (CODEC == tbf::kB3) {
    const int t = 5 * (4 * word + e) + i;
    const int cur = (t < 256 && (t >> 7) == variant) ? xq_tile[t] : 0;
    const int prev = (i > 0 && t - 1 < 256 && ((t - 1) >> 7) == variant) ? xq_tile[t - 1] : 0;
    return cur - 3 * prev;
  } else {
    const int t = 16 * word + 4 * e + i;
    return ((t >> 7) == variant) ? xq_tile[t] : 0;
  }
}

template <int CODEC>
__device__ __forceinline__ uint32_t z_quad(const int8_t* xq_tile, const Slot<CODEC>& s, int digit, int hl, int variant) {
  if (digit < 0) return 0;
  uint32_t out = 0;
  for (int e = s.lane_lo; e < s.lane_hi; ++e) {
    const int z = z_value<CODEC>(xq_tile, s.word, e, digit, variant);
    const int v = hl == 0 ? (z >> 2) : (z & 3);
    out |= uint32_t(v & 0xff) << (8 * e);
  }
  return out;
}

// B operand of a bytewise MMA for lane column c: quad 0 = digits 0..3 of byte c of the word,
// quad 1 = digit 4 in its first byte.
template <int CODEC>
__device__ __forceinline__ uint2 z_bytewise(const int8_t* xq_tile, const Slot<CODEC>& s, int c, int hl, int variant) {
  uint32_t q0 = 0, q1 = 0;
  for (int i = 0; i < 5; ++i) {
    const int z = z_value<CODEC>(xq_tile, s.word, c, i, variant);
    const uint32_t v = uint32_t((hl == 0 ? (z >> 2) : (z & 3)) & 0xff);
    if (i < 4) q0 |= v << (8 * i); else q1 = v;
  }
  return make_uint2(q0, q1);
}

// ---------------------------------------------------------------- activation preparation
// One CTA per (tile column j, token t): per-token absmax int8 quantisation of the 256
// activations of column j (each CTA re-reduces the whole row for the absmax: the row is a few
// KB), then the B-fragment table entries and accumulator start values of that column.
// Table layout in global scratch (bytes): z entries uint2[tpr][mmas][ncol][4] | start values
// int[m][tpr][2] (padded to 16) | token scales float[m] (padded to 16).
struct PrepareParams {
  const void* x; const float* act_scale_in; const float* act_absmax_in;
  uint8_t* tables; uint32_t* status;
  uint32_t m, k, tpr, x_dtype, off_cinit, off_actscale, pdl;
  TbCommView comm;   // world > 1: the per-token absmax is the maximum over the ranks' slices
};

__device__ __forceinline__ float load_act(const void* x, uint32_t dtype, size_t i) {
  return dtype == TB_F32 ? static_cast<const float*>(x)[i] : __bfloat162float(static_cast<const __nv_bfloat16*>(x)[i]);
}

template <int CODEC, bool DUAL>
__global__ void __launch_bounds__(256) prepare_kernel(const PrepareParams p) {
  constexpr int kNM = MmaCount<CODEC, DUAL>::value;
  __shared__ int8_t xq[256];
  __shared__ float red[8];
  if (p.pdl) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t j = blockIdx.x, t = blockIdx.y, ncol = (DUAL ? 4 : 2) * p.m;
  float scale_out;
  uint32_t comm_seq = 0;   // thread 0 only
  if (p.x_dtype == TB_I8) {
    xq[tid] = static_cast<const int8_t*>(p.x)[size_t(t) * p.k + j * 256 + tid];
    scale_out = p.act_scale_in[t];
  } else {
    float gamma;
    if (p.act_absmax_in) {
      gamma = p.act_absmax_in[t];   // absmax over the full (unsharded) row, supplied by the caller
    } else {
      float mx = 0.f;
      for (uint32_t i = tid; i < p.k; i += 256) mx = fmaxf(mx, fabsf(load_act(p.x, p.x_dtype, size_t(t) * p.k + i)));
      for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) red[warp] = mx;
      __syncthreads();
      gamma = 0.f;
      for (int w2 = 0; w2 < 8; ++w2) gamma = fmaxf(gamma, red[w2]);
    }
    if (p.comm.world > 1) {
      // every rank holds a slice of the row: publish this slice's absmax (tile column 0 does it),
      // wait for the peers' arrivals, take the maximum
      __shared__ float gamma_all;
      __syncthreads();
      if (tid == 0) {
        uint32_t* mine = p.comm.flags[p.comm.rank];
        comm_seq = *reinterpret_cast<volatile uint32_t*>(mine + kCommFusedEpoch) + 1u;
        if (j == 0) {
          p.comm.data[p.comm.rank][t] = gamma;
          __threadfence_system();
          // a launch of fewer than four tokens still advances all four token counters, so that
          // "arrivals = peers x rounds" holds for every counter whatever the token counts were
          for (uint32_t r = 0; r < p.comm.world; ++r)
            if (r != p.comm.rank) {
              peer_signal(p.comm.flags[r] + kCommCounters + t);
              if (t == 0)
                for (uint32_t unused = p.m; unused < 4; ++unused) peer_signal(p.comm.flags[r] + kCommCounters + unused);
            }
        }
        float gmax = gamma;
        if (peer_wait(mine + kCommCounters + t, (p.comm.world - 1) * comm_seq)) {
          for (uint32_t r = 0; r < p.comm.world; ++r)
            if (r != p.comm.rank) gmax = fmaxf(gmax, peer_load(p.comm.data[r] + t));
        } else if (atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) {
          p.status[TBS_INFO0] = t; p.status[TBS_INFO1] = 500;
        }
        gamma_all = gmax;
      }
      __syncthreads();
      gamma = gamma_all;
    }
    const float scale_q = gamma > 0.f ? __fdiv_rn(127.0f, gamma) : 0.f;
    scale_out = __fdiv_rn(gamma, 127.0f);
    const float v = load_act(p.x, p.x_dtype, size_t(t) * p.k + j * 256 + tid);
    xq[tid] = int8_t(int(fminf(127.f, fmaxf(-128.f, rintf(__fmul_rn(v, scale_q))))));
  }
  __syncthreads();
  uint2* ztab = reinterpret_cast<uint2*>(p.tables);
  // entries of this (tile column, token): mma x [scale group] x {high, low part} x lane column.
  // MMA column = 2*token + hl, plus 2*m for the second scale group in the dual layout.
  constexpr uint32_t kPerMma = DUAL ? 16 : 8;
  if (tid < kNM * kPerMma) {
    const uint32_t c = tid & 3, hl = (tid >> 2) & 1, v = DUAL ? (tid >> 3) & 1 : 0, mma = tid / kPerMma;
    const Slot<CODEC> s = slot_of<CODEC, DUAL>(int(mma), int(c));
    const int variant = DUAL ? int(v) : s.variant;
    const uint32_t col = v * 2 * p.m + 2 * t + hl;
    ztab[((size_t(j) * kNM + mma) * ncol + col) * 4 + c] =
        s.bytewise ? z_bytewise<CODEC>(xq, s, int(c), int(hl), variant)
                   : make_uint2(z_quad<CODEC>(xq, s, s.d0, int(hl), variant), z_quad<CODEC>(xq, s, s.d1, int(hl), variant));
  }
  // accumulator start value of (token, column, group v):
  //   B3: -(sum over the group of x_t * c5[t mod 5]), c5 = {1,-2,-1,-1,2}: the group sum of x plus
  //       the operand offsets (q2,q3,q4 carry +1) times z = x_i - 3 x_{i-1};   D2: -(sum of x_t).
  if (warp < 2) {
    int sum = 0;
    for (int e = 0; e < 4; ++e) {
      const int tt = int(warp) * 128 + int(lane) * 4 + e;
      int coef = 1;
      if (CODEC == tbf::kB3) { const int d = tt % 5; coef = d == 0 ? 1 : d == 1 ? -2 : d == 4 ? 2 : -1; }
      sum += int(xq[tt]) * coef;
    }
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) reinterpret_cast<int*>(p.tables + p.off_cinit)[(t * p.tpr + j) * 2 + warp] = -sum;
  }
  if (j == 0 && tid == 0) reinterpret_cast<float*>(p.tables + p.off_actscale)[t] = scale_out;
  if (j == 0 && t == 0 && tid < 4) reinterpret_cast<uint32_t*>(p.tables + p.off_actscale + 16)[tid] = 0u;
  if (p.comm.world > 1 && tid == 0 && comm_seq) {
    // the last CTA of the launch closes the round
    uint32_t* mine = p.comm.flags[p.comm.rank];
    __threadfence();
    if (atomicAdd(mine + kCommFusedDone, 1u) == gridDim.x * gridDim.y - 1) {
      mine[kCommFusedDone] = 0;
      *reinterpret_cast<volatile uint32_t*>(mine + kCommFusedEpoch) = comm_seq;
    }
  }
}

// ---------------------------------------------------------------- the kernel
template <int CODEC, int PLANES, int M>
__global__ void __launch_bounds__(kThreads, 2) decode_kernel(const DecodeParams p) {
  using T = Traits<CODEC>;
  constexpr bool DUAL = M <= 2;
  constexpr int kNM = MmaCount<CODEC, DUAL>::value;
  constexpr uint32_t ncol = (DUAL ? 4 : 2) * M;   // MMA columns in use
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], table_bar;
  __shared__ uint32_t abort_flag, comm_ok;
  __shared__ TbLayerDesc layer_desc[kMaxGroupLayers];

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* ring = smem + p.off_ring;
  uint8_t* scale_ring = smem + p.off_scale_ring;
  uint2* ztab = reinterpret_cast<uint2*>(smem + p.off_z);
  int* cinit = reinterpret_cast<int*>(smem + p.off_cinit);
  float* part = reinterpret_cast<float*>(smem + p.off_part);
  float* act_scale = reinterpret_cast<float*>(smem + p.off_actscale);

  if (tid == 0) {
    abort_flag = 0;
    for (uint32_t s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kConsumerWarps); }
    mbar_init(&table_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (uint32_t l = tid; l < p.layer_count; l += kThreads) {
    if (p.layers) { layer_desc[l].payload = p.layers[l].payload; layer_desc[l].scales = p.layers[l].scales; }
    else { layer_desc[l].payload = p.payload; layer_desc[l].scales = p.scales; }
  }
  __syncthreads();
  // The next kernel on the stream may begin once every CTA has passed this point.  When this
  // launch has to wait for its tables, the trigger is raised only after that wait, so that a
  // later launch which shares the tables (and therefore does not wait) cannot outrun them.
  if (p.pdl && !p.wait_tables) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const uint32_t total_blocks = p.blocks * p.layer_count;
  const uint32_t my_blocks = blockIdx.x < total_blocks ? (total_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (warp == kConsumerWarps) {
    // ------------------------------------------------ producer: weights do not depend on the
    // previous kernel, so the stream starts before griddepcontrol.wait.
    if (lane == 0) {
      uint32_t fills[kMaxStages] = {0, 0, 0, 0};
      for (uint32_t it = 0; it < my_blocks; ++it) {
        const uint32_t s = it % p.stages, round = it / p.stages;
        if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1, &abort_flag)) {
          abort_flag = 1;
          if (atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = it; p.status[TBS_INFO1] = 100 + s; }
          break;
        }
        const uint32_t gblk = blockIdx.x + it * gridDim.x;
        const uint32_t layer = gblk / p.blocks, blk = gblk - layer * p.blocks;
        const uint8_t* pay = layer_desc[layer].payload;
        const uint8_t* scs = reinterpret_cast<const uint8_t*>(layer_desc[layer].scales);
        mbar_expect_tx(&full_bar[s], p.stage_bytes + p.scale_stage_bytes);
        bulk_g2s(ring + size_t(s) * p.stage_bytes, pay + size_t(blk) * p.stage_bytes, p.stage_bytes, &full_bar[s]);
        bulk_g2s(scale_ring + size_t(s) * p.scale_stage_bytes, scs + size_t(blk) * p.scale_stage_bytes,
                 p.scale_stage_bytes, &full_bar[s]);
        ++fills[s];
      }
      // Do not leave the CTA while a copy may still be landing in its shared memory: wait
      // (bounded) for the latest fill of every slot.  In the normal path these have all
      // completed already, because the consumers waited on them.
      for (uint32_t s = 0; s < p.stages; ++s)
        if (fills[s])
          for (uint32_t i = 0; i < kSpinLimit && !mbar_try_wait(&full_bar[s], (fills[s] - 1) & 1); ++i) {}
    }
    return;
  }

  // -------------------------------------------------- consumers: fetch the activation tables
  // The prepare kernel (previous launch on this stream) wrote z tables, accumulator start values
  // and token scales to global scratch; one bulk copy brings them in.
  const uint32_t ctid = tid;  // 0 .. kConsumerWarps*32-1
  constexpr uint32_t kCT = kConsumerWarps * 32;
  if (p.pdl && p.wait_tables) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  if (ctid == 0) {
    mbar_expect_tx(&table_bar, p.table_bytes);
    bulk_g2s(smem + p.off_z, p.tables, p.table_bytes, &table_bar);
  }
  {
    const bool tables_ok = mbar_wait(&table_bar, 0, &abort_flag);
    if (!tables_ok) {
      abort_flag = 1;
      if (lane == 0 && atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = 0; p.status[TBS_INFO1] = 200; }
    }
    consumer_sync();
    if (abort_flag) return;
  }

  // -------------------------------------------------- consumers: main loop
  const uint32_t g = lane >> 2, c = lane & 3;
  const uint32_t rp_per_stage = p.rows_per_stage * PLANES;        // multiple of 16
  const uint32_t sets = rp_per_stage >> 4;
  const uint32_t items = p.tpr * sets;   // (set, tile column) pairs, set-major
  const uint32_t per_warp = (items + kConsumerWarps - 1) / kConsumerWarps;
  const uint32_t item_lo = warp * per_warp, item_hi = min(items, item_lo + per_warp);
  const uint32_t first_set = item_lo / p.tpr, first_j = item_lo - first_set * p.tpr;
  const uint32_t part_stride = rp_per_stage * M;                  // floats per warp slice
  // Which (scale group, token) cell of the C fragment this lane finishes.
  //   separate accumulators: lane column c holds token c, both groups;
  //   dual columns:          lane column c holds group c / m, token c % m.
  const bool lane_has_cell = DUAL ? c < 2 * M : c < M;
  const uint32_t cell_group = DUAL ? (c >= M ? 1u : 0u) : 0u;
  const uint32_t cell_token = DUAL ? c - cell_group * M : c;
  // MMA columns beyond `ncol` produce sums nobody reads, so their lanes may load any valid
  // table entry: fold them onto the used columns instead of masking.
  const uint32_t bcol = g % ncol;
  const uint32_t byte_sel = c | (c << 4) | ((4u + c) << 8) | ((4u + c) << 12);   // byte c of two words -> bytes 0 and 2
  constexpr uint32_t zstep = ncol * 4;
  const uint32_t groups_per_row = p.tpr * 2;

  // Tensor-parallel row shard: the fp32 partial rows go to the peer-visible slot and the
  // all-reduce is finished at the end of this kernel.
  const bool fused = p.comm.world > 1;
  const uint32_t comm_seq = fused ? *reinterpret_cast<volatile uint32_t*>(p.comm.flags[p.comm.rank] + kCommFusedEpoch) + 1u : 0u;
  for (uint32_t it = 0; it < my_blocks; ++it) {
    const uint32_t s = it % p.stages;
    float* my_part = part + ((it & 1) * kConsumerWarps + warp) * part_stride;
    for (uint32_t i = lane; i < part_stride; i += 32) my_part[i] = 0.f;
    __syncwarp();
    const bool landed = mbar_wait(&full_bar[s], (it / p.stages) & 1, &abort_flag);
    if (!landed) {
      abort_flag = 1;
      if (lane == 0 && atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = it; p.status[TBS_INFO1] = s; }
    }
    const uint32_t* words = reinterpret_cast<const uint32_t*>(ring + size_t(s) * p.stage_bytes);
    const uint32_t* scl = reinterpret_cast<const uint32_t*>(scale_ring + size_t(s) * p.scale_stage_bytes);
    const uint32_t gblk = blockIdx.x + it * gridDim.x;
    const uint32_t layer = gblk / p.blocks, blk = gblk - layer * p.blocks;
    const uint32_t row0 = blk * p.rows_per_stage;

    // Items are (row set, tile column) pairs in set-major order; a warp's range is contiguous, so
    // it walks the columns of one set with running pointers and keeps the two rows' partial
    // sums in registers until the set changes.
    uint32_t item = item_lo, set = first_set, j = first_j;
    for (; landed && item < item_hi; ++set, j = 0) {
      const uint32_t j_end = min(p.tpr, j + (item_hi - item));
      item += j_end - j;
      const uint32_t rpa = set * 16 + g, rpb = rpa + 8;
      const uint32_t na = rpa / PLANES, pa = rpa - na * PLANES;
      const uint32_t nb = rpb / PLANES, pb = rpb - nb * PLANES;
      constexpr uint32_t kWordsPerPlane = T::kPlaneBytes / 4, kColStride = PLANES * kWordsPerPlane;
      const uint32_t* wa = words + ((na * p.tpr + j) * PLANES + pa) * kWordsPerPlane + c;
      const uint32_t* wb = words + ((nb * p.tpr + j) * PLANES + pb) * kWordsPerPlane + c;
      // f16 scales of (row-plane, tile): two per u32, [group 0 | group 1]
      const uint16_t* sca = reinterpret_cast<const uint16_t*>(scl + (na * p.tpr + j) * PLANES + pa) + (DUAL ? cell_group : 0);
      const uint16_t* scb = reinterpret_cast<const uint16_t*>(scl + (nb * p.tpr + j) * PLANES + pb) + (DUAL ? cell_group : 0);
      const int* cin = cinit + ((DUAL ? cell_token : c) * p.tpr + j) * 2 + (DUAL ? cell_group : 0);
      const uint2* zlane = ztab + (size_t(j) * kNM * ncol + bcol) * 4 + c;
      constexpr uint32_t zcol = kNM * ncol * 4;
#define TB_BFRAG(mm) (zlane[(mm) * zstep])
      float ya = 0.f, yb = 0.f;

      for (; j < j_end; ++j, wa += kColStride, wb += kColStride, sca += 2 * PLANES, scb += 2 * PLANES, cin += 2, zlane += zcol) {
        int acc0[4], acc1[4];   // group 0 / group 1 sums (dual layout: acc0 holds this lane's group)
        if (CODEC == tbf::kB3) {
          // Two accumulation chains, fed alternately, so that consecutive MMAs rarely depend on
          // each other.  Dual layout: chain A takes words c and 8+c, chain B words 4+c and 12, and
          // their sum is the cell.  Separate accumulators: chain A is scale group 0, chain B group 1.
          int sA[4], sB[4];
          uint32_t qa[5], qb[5];
          uint2 b;
          b3_quads(wa[0], qa); b3_quads(wb[0], qb);
          b = TB_BFRAG(0); mma_u8s8_first(sA, qa[0], qb[0], qa[1], qb[1], b.x, b.y);
          b = TB_BFRAG(1); mma_u8s8(sA, qa[2], qb[2], qa[3], qb[3], b.x, b.y);
          b = TB_BFRAG(2); mma_u8s8(sA, qa[4], qb[4], 0u, 0u, b.x, b.y);
          b3_quads(wa[4], qa); b3_quads(wb[4], qb);
          if (DUAL) {
            b = TB_BFRAG(3); mma_u8s8_first(sB, qa[0], qb[0], qa[1], qb[1], b.x, b.y);
            b = TB_BFRAG(4); mma_u8s8(sB, qa[2], qb[2], qa[3], qb[3], b.x, b.y);
            b = TB_BFRAG(5); mma_u8s8(sB, qa[4], qb[4], 0u, 0u, b.x, b.y);
          } else {
            // the words 4..7 straddle the two scale groups: once per group, masked on the B side
            b = TB_BFRAG(3); mma_u8s8(sA, qa[0], qb[0], qa[1], qb[1], b.x, b.y);
            b = TB_BFRAG(6); mma_u8s8_first(sB, qa[0], qb[0], qa[1], qb[1], b.x, b.y);
            b = TB_BFRAG(4); mma_u8s8(sA, qa[2], qb[2], qa[3], qb[3], b.x, b.y);
            b = TB_BFRAG(7); mma_u8s8(sB, qa[2], qb[2], qa[3], qb[3], b.x, b.y);
            b = TB_BFRAG(5); mma_u8s8(sA, qa[4], qb[4], 0u, 0u, b.x, b.y);
            b = TB_BFRAG(8); mma_u8s8(sB, qa[4], qb[4], 0u, 0u, b.x, b.y);
          }
          constexpr int o2 = DUAL ? 6 : 9, o3 = DUAL ? 9 : 12;
          b3_quads(wa[8], qa); b3_quads(wb[8], qb);
          if (DUAL) {
            b = TB_BFRAG(o2); mma_u8s8(sA, qa[0], qb[0], qa[1], qb[1], b.x, b.y);
            b = TB_BFRAG(o2 + 1); mma_u8s8(sA, qa[2], qb[2], qa[3], qb[3], b.x, b.y);
            b = TB_BFRAG(o2 + 2); mma_u8s8(sA, qa[4], qb[4], 0u, 0u, b.x, b.y);
          } else {
            b = TB_BFRAG(o2); mma_u8s8(sB, qa[0], qb[0], qa[1], qb[1], b.x, b.y);
            b = TB_BFRAG(o2 + 1); mma_u8s8(sB, qa[2], qb[2], qa[3], qb[3], b.x, b.y);
            b = TB_BFRAG(o2 + 2); mma_u8s8(sB, qa[4], qb[4], 0u, 0u, b.x, b.y);
          }
          {
            // word 12: lane column c takes byte c of both rows through one half2 chain; its five
            // quotients fill the lane's eight k-slots of a single MMA
            const uint32_t h = (prmt(wa[12 - c], wb[12 - c], byte_sel) & 0x00ff00ffu) | 0x64006400u;
            const uint32_t q1 = hfma2_bits(h, kC3, kK3), q2 = hfma2_bits(h, kC9, kK9);
            const uint32_t q3 = hfma2_bits(q1, kC9, kK9), q4 = hfma2_bits(q2, kC9b, kK9b);
            const uint32_t u = prmt(h, q1, 0x6240u), v = prmt(q2, q3, 0x6240u);
            b = TB_BFRAG(o3);
            mma_u8s8(sB, prmt(u, v, 0x5410u), prmt(u, v, 0x7632u), prmt(q4, 0u, 0x4440u), prmt(q4, 0u, 0x4442u), b.x, b.y);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (DUAL) acc0[e] = sA[e] + sB[e];
            else { acc0[e] = sA[e]; acc1[e] = sB[e]; }
          }
        } else {
          int sq[4][4];
#pragma unroll
          for (int sl = 0; sl < 4; ++sl) {
            const uint32_t va = wa[sl * 4], vb = wb[sl * 4];
            uint2 b = TB_BFRAG(sl * 2);
            mma_u8s8_first(sq[sl], va & 0x03030303u, vb & 0x03030303u, (va >> 2) & 0x03030303u, (vb >> 2) & 0x03030303u, b.x, b.y);
            b = TB_BFRAG(sl * 2 + 1);
            mma_u8s8(sq[sl], (va >> 4) & 0x03030303u, (vb >> 4) & 0x03030303u, (va >> 6) & 0x03030303u,
                     (vb >> 6) & 0x03030303u, b.x, b.y);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (DUAL) acc0[e] = (sq[0][e] + sq[1][e]) + (sq[2][e] + sq[3][e]);
            else { acc0[e] = sq[0][e] + sq[1][e]; acc1[e] = sq[2][e] + sq[3][e]; }
          }
        }

        // finish the cells: columns (2c, 2c+1) are the high / low activation parts of one cell
        if (DUAL) {
          if (lane_has_cell) {
            const int ci = cin[0];
            const int ia = 4 * acc0[0] + acc0[1] + ci, ib = 4 * acc0[2] + acc0[3] + ci;
            ya = __fmaf_rn(group_sum_to_float(ia), __half2float(__ushort_as_half(sca[0])), ya);
            yb = __fmaf_rn(group_sum_to_float(ib), __half2float(__ushort_as_half(scb[0])), yb);
            if (p.acc_dump) {
              const uint32_t tok = p.dump_token_offset + cell_token;
              if (row0 + na < p.n)
                p.acc_dump[((size_t(tok) * p.n + row0 + na) * groups_per_row + 2 * j + cell_group) * PLANES + pa] = ia;
              if (row0 + nb < p.n)
                p.acc_dump[((size_t(tok) * p.n + row0 + nb) * groups_per_row + 2 * j + cell_group) * PLANES + pb] = ib;
            }
          }
        } else if (lane_has_cell) {
          const int ci0 = cin[0], ci1 = cin[1];
          const int ia0 = 4 * acc0[0] + acc0[1] + ci0, ia1 = 4 * acc1[0] + acc1[1] + ci1;
          const int ib0 = 4 * acc0[2] + acc0[3] + ci0, ib1 = 4 * acc1[2] + acc1[3] + ci1;
          ya = __fmaf_rn(group_sum_to_float(ia1), __half2float(__ushort_as_half(sca[1])),
                         __fmaf_rn(group_sum_to_float(ia0), __half2float(__ushort_as_half(sca[0])), ya));
          yb = __fmaf_rn(group_sum_to_float(ib1), __half2float(__ushort_as_half(scb[1])),
                         __fmaf_rn(group_sum_to_float(ib0), __half2float(__ushort_as_half(scb[0])), yb));
          if (p.acc_dump) {
            const uint32_t tok = p.dump_token_offset + c;
            if (row0 + na < p.n) {
              int32_t* d = p.acc_dump + ((size_t(tok) * p.n + row0 + na) * groups_per_row + 2 * j) * PLANES + pa;
              d[0] = ia0; d[PLANES] = ia1;
            }
            if (row0 + nb < p.n) {
              int32_t* d = p.acc_dump + ((size_t(tok) * p.n + row0 + nb) * groups_per_row + 2 * j) * PLANES + pb;
              d[0] = ib0; d[PLANES] = ib1;
            }
          }
        }
      }
#undef TB_BFRAG
      // hand the set's partial sums to the stage combine
      if (DUAL) {
        // the two scale groups of a (row, token) sit p.m lanes apart: group 0 + group 1
        ya = __fadd_rn(ya, __shfl_xor_sync(0xffffffffu, ya, M));
        yb = __fadd_rn(yb, __shfl_xor_sync(0xffffffffu, yb, M));
        if (lane_has_cell && cell_group == 0) {
          my_part[rpa * M + cell_token] += ya;
          my_part[rpb * M + cell_token] += yb;
        }
      } else if (lane_has_cell) {
        my_part[rpa * M + c] += ya;
        my_part[rpb * M + c] += yb;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);   // slot may be refilled

    // combine the warps' partial sums (fixed order: plane ascending, warp ascending).  Every
    // consumer warp reaches this barrier, also after a failed wait, and all leave together.
    consumer_sync();
    if (abort_flag) return;
    const float* stage_part = part + (it & 1) * kConsumerWarps * part_stride;
    for (uint32_t e = ctid; e < p.rows_per_stage * M; e += kCT) {
      const uint32_t t = e / p.rows_per_stage, r = e - t * p.rows_per_stage;
      if (row0 + r >= p.n) continue;
      float sum = 0.f;
#pragma unroll
      for (uint32_t q = 0; q < PLANES; ++q)
        for (int w2 = 0; w2 < kConsumerWarps; ++w2)
          sum = __fadd_rn(sum, stage_part[w2 * part_stride + (r * PLANES + q) * M + t]);
      float out = __fmul_rn(sum, act_scale[t]);
      if (p.row_scale) out = __fmul_rn(out, p.row_scale[row0 + r]);
      if (fused) {
        // this rank's partial row, peer-visible; the sum over ranks follows one block later
        p.comm.data[p.comm.rank][size_t(t) * p.n + row0 + r] = out;
        continue;
      }
      const size_t idx = size_t(layer) * p.y_layer_stride + size_t(t) * p.y_row_stride + row0 + r;
      if (p.y_dtype == TB_F32) static_cast<float*>(p.y)[idx] = out;
      else static_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(out);
    }
  }
  if (fused) {
    // Every rank's CTA number b walks the same row blocks.  Once all of this CTA's partial rows are
    // written, ONE arrival is raised on every peer's counter b; when the peers' arrivals are in,
    // the CTA's rows are summed over the ranks in rank order (one NVLink round trip per kernel).
    consumer_sync();
    if (ctid == 0) {
      // the barrier orders the other threads' stores before this fence; the fence and the release
      // additions publish them to the peers
      __threadfence_system();
      for (uint32_t r = 0; r < p.comm.world; ++r)
        if (r != p.comm.rank) peer_signal(p.comm.flags[r] + kCommCounters + blockIdx.x);
      const bool arrived = peer_wait(p.comm.flags[p.comm.rank] + kCommCounters + blockIdx.x, (p.comm.world - 1) * comm_seq);
      if (!arrived) {
        abort_flag = 1;
        if (atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = blockIdx.x; p.status[TBS_INFO1] = 501; }
      }
      comm_ok = arrived ? 1u : 0u;
    }
    consumer_sync();
    if (!comm_ok) return;
    const uint32_t per_block = p.rows_per_stage * M;
    for (uint32_t e = ctid; e < my_blocks * per_block; e += kCT) {
      const uint32_t it = e / per_block, rem = e - it * per_block;
      const uint32_t t = rem / p.rows_per_stage, r = rem - t * p.rows_per_stage;
      const uint32_t row = (blockIdx.x + it * gridDim.x) * p.rows_per_stage + r;
      if (row >= p.n) continue;
      const size_t at = size_t(t) * p.n + row;
      float sum = p.comm.rank == 0 ? p.comm.data[0][at] : peer_load(p.comm.data[0] + at);
      for (uint32_t q = 1; q < p.comm.world; ++q)
        sum = __fadd_rn(sum, q == p.comm.rank ? p.comm.data[q][at] : peer_load(p.comm.data[q] + at));
      const size_t idx = size_t(t) * p.y_row_stride + row;
      if (p.y_dtype == TB_F32) static_cast<float*>(p.y)[idx] = sum;
      else static_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(sum);
    }
    if (ctid == 0) {
      // the last CTA of the launch closes the round
      uint32_t* mine = p.comm.flags[p.comm.rank];
      __threadfence();
      if (atomicAdd(mine + kCommFusedDone, 1u) == gridDim.x - 1) {
        mine[kCommFusedDone] = 0;
        *reinterpret_cast<volatile uint32_t*>(mine + kCommFusedEpoch) = comm_seq;
      }
    }
  }
}

uint32_t round_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

// Byte layout of the activation tables (identical in global scratch and in shared memory).
struct TableLayout { uint32_t z_bytes, off_cinit, off_actscale, total; };
bool use_dual(uint32_t m) { return m <= 2; }
TableLayout table_layout(const tb_weights* w, uint32_t m) {
  const bool dual = use_dual(m);
  const uint32_t tpr = uint32_t(w->k / 256);
  const uint32_t mmas = w->codec == tbf::kB3 ? (dual ? 10 : 13) : 8;
  TableLayout t;
  t.z_bytes = tpr * mmas * ((dual ? 4 : 2) * m) * 4 * 8;
  t.off_cinit = t.z_bytes;
  t.off_actscale = t.off_cinit + round_up(m * tpr * 2 * 4, 16);
  t.total = t.off_actscale + 32;   // token scales (16 bytes) then a zero entry read by idle MMA columns
  return t;
}

// Shared-memory layout for (weights, m); returns total bytes or 0 when it cannot fit.
size_t layout(const tb_weights* w, uint32_t m, int max_smem, DecodeParams* p) {
  const DecodePlan& pl = w->plan;
  const uint32_t planes = w->uniform_planes;
  const TableLayout tl = table_layout(w, m);
  uint32_t off = 0;
  const uint32_t part = round_up(2 * kConsumerWarps * pl.rows_per_stage * planes * m * 4, 16);
  const uint32_t fixed = tl.total + part;
  const uint32_t per_stage = pl.stage_bytes + pl.scale_stage_bytes;
  if (fixed + 2 * per_stage > uint32_t(max_smem)) return 0;
  // Prefer a footprint that lets two CTAs share an SM (one of this launch, one of the next launch
  // on the stream, whose weight stream then starts under this launch's tail).
  const uint32_t half_sm = 110u * 1024u;   // two CTAs (dynamic + static + 1 KB reserved each) within 228 KB
  const uint32_t budget = fixed + 2 * per_stage <= half_sm ? half_sm : uint32_t(max_smem);
  uint32_t stages = std::min<uint32_t>(kMaxStages, (budget - fixed) / per_stage);
  if (p) {
    p->stages = stages;
    p->off_ring = off; off += stages * pl.stage_bytes;
    p->off_scale_ring = off; off += stages * pl.scale_stage_bytes;
    p->off_z = off;
    p->off_cinit = off + tl.off_cinit;
    p->off_actscale = off + tl.off_actscale;
    p->off_zero = off + tl.off_actscale + 16;
    off += tl.total;
    p->off_part = off; off += part;
    p->table_bytes = tl.total;
    p->ctas_per_sm = budget == half_sm ? 2 : 1;
  }
  return size_t(fixed) + size_t(stages) * per_stage;
}

}  // namespace

void tb_make_decode_plan(tb_weights* w, int max_smem) {
  DecodePlan pl{};
  if (!w->fast) { w->plan = pl; return; }
  const uint32_t planes = w->uniform_planes, tpr = uint32_t(w->k / 256);
  const uint32_t pb = w->codec == tbf::kB3 ? 52 : 64;
  pl.row_bytes = tpr * planes * pb;
  const uint32_t base = planes == 2 ? 8 : 16;   // R % 4 == 0 and R*planes % 16 == 0
  const uint32_t target = 40 * 1024;
  uint32_t r = std::max(base, (target / pl.row_bytes) / base * base);
  r = std::min<uint32_t>(r, 128);
  // keep enough blocks to cover every SM at least three times when the tensor allows it
  while (r > base && (w->n + r - 1) / r < 444) r -= base;
  pl.rows_per_stage = r;
  pl.stage_bytes = r * pl.row_bytes;
  pl.scale_stage_bytes = r * tpr * planes * 4;
  pl.blocks = uint32_t((w->n + r - 1) / r);
  (void)max_smem;
  w->plan = pl;
}

bool tb_decode_supported(const tb_weights* w, uint32_t m, int max_smem, size_t* smem_bytes) {
  if (!w->fast || m < 1 || m > 4) return false;
  const size_t bytes = layout(w, m, max_smem, nullptr);
  if (!bytes) return false;
  if (smem_bytes) *smem_bytes = bytes;
  return true;
}

size_t tb_decode_scratch_bytes(const tb_weights* w, uint32_t m) { return table_layout(w, m).total; }

cudaError_t tb_launch_prepare(const DecodeArgs& a, cudaStream_t stream) {
  const tb_weights* w = a.w;
  const TableLayout tl = table_layout(w, a.m);
  if (!a.scratch || a.scratch_bytes < tl.total) return cudaErrorInvalidValue;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  PrepareParams pp{};
  pp.x = a.x; pp.act_scale_in = a.act_scale_in; pp.act_absmax_in = a.act_absmax_in;
  pp.tables = static_cast<uint8_t*>(a.scratch);
  pp.m = a.m; pp.k = uint32_t(w->k); pp.tpr = uint32_t(w->k / 256); pp.x_dtype = uint32_t(a.x_dtype);
  pp.off_cinit = tl.off_cinit; pp.off_actscale = tl.off_actscale; pp.pdl = a.pdl ? 1u : 0u;
  pp.status = a.status;
  if (a.comm_absmax) {
    if (a.comm_absmax->counters < a.m) return cudaErrorInvalidValue;
    pp.comm = *a.comm_absmax;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pp.tpr, a.m);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = a.pdl ? 1 : 0;
  const bool dual = use_dual(a.m);
  if (w->codec == tbf::kB3)
    return dual ? cudaLaunchKernelEx(&cfg, prepare_kernel<tbf::kB3, true>, pp) : cudaLaunchKernelEx(&cfg, prepare_kernel<tbf::kB3, false>, pp);
  return dual ? cudaLaunchKernelEx(&cfg, prepare_kernel<tbf::kD2, true>, pp) : cudaLaunchKernelEx(&cfg, prepare_kernel<tbf::kD2, false>, pp);
}

using DecodeKernel = void (*)(const DecodeParams);
template <int CODEC, int PLANES> DecodeKernel pick_tokens(uint32_t m) {
  return m == 1 ? decode_kernel<CODEC, PLANES, 1> : m == 2 ? decode_kernel<CODEC, PLANES, 2>
       : m == 3 ? decode_kernel<CODEC, PLANES, 3> : decode_kernel<CODEC, PLANES, 4>;
}
template <int CODEC> DecodeKernel pick_planes(uint32_t planes, uint32_t m) {
  return planes == 1 ? pick_tokens<CODEC, 1>(m) : planes == 2 ? pick_tokens<CODEC, 2>(m) : pick_tokens<CODEC, 3>(m);
}

cudaError_t tb_launch_decode(const DecodeArgs& a, int sm_count, int max_smem, cudaStream_t stream) {
  const tb_weights* w = a.w;
  DecodeParams p{};
  const size_t smem = layout(w, a.m, max_smem, &p);
  if (!smem) return cudaErrorInvalidConfiguration;
  const TableLayout tl = table_layout(w, a.m);
  if (!a.scratch || a.scratch_bytes < tl.total) return cudaErrorInvalidValue;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  p.payload = w->d_payload; p.scales = w->d_scales;
  p.layers = a.layers; p.layer_count = a.layers ? a.layer_count : 1; p.y_layer_stride = a.y_layer_stride;
  p.tables = static_cast<const uint8_t*>(a.scratch);
  p.y = a.y; p.acc_dump = a.acc_dump; p.row_scale = a.row_scale;
  p.status = a.status;
  p.m = a.m; p.n = uint32_t(w->n); p.k = uint32_t(w->k); p.planes = w->uniform_planes; p.tpr = uint32_t(w->k / 256);
  p.rows_per_stage = w->plan.rows_per_stage; p.row_bytes = w->plan.row_bytes;
  p.stage_bytes = w->plan.stage_bytes; p.scale_stage_bytes = w->plan.scale_stage_bytes; p.blocks = w->plan.blocks;
  p.y_dtype = uint32_t(a.y_dtype); p.y_row_stride = a.y_row_stride;
  p.dump_token_offset = a.dump_token_offset; p.dump_tokens_total = a.dump_tokens_total;
  p.pdl = a.pdl ? 1u : 0u;
  p.wait_tables = a.tables_shared ? 0u : 1u;
  if (a.comm_y) {
    // one arrival counter per CTA (up to two CTAs per SM); single layer, fp32 partials of [m, n]
    if (a.layers || a.comm_y->counters < 2u * uint32_t(sm_count)) return cudaErrorInvalidValue;
    p.comm = *a.comm_y;
  }
  DecodeKernel kernel = w->codec == tbf::kB3 ? pick_planes<tbf::kB3>(w->uniform_planes, a.m) : pick_planes<tbf::kD2>(w->uniform_planes, a.m);
  if (a.layers && a.layer_count > uint32_t(kMaxGroupLayers)) return cudaErrorInvalidValue;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (err != cudaSuccess) return err;
  cudaLaunchConfig_t cfg{};
  // A grouped launch keeps two CTAs per SM busy.  A single small layer keeps one, so that the next
  // launch on the stream can move in beside it; a layer with many row blocks per SM is better
  // served by two CTAs per SM of its own.
  const bool wide = a.layers != nullptr || p.blocks >= 2u * uint32_t(sm_count);
  const uint32_t resident = uint32_t(sm_count) * (wide ? p.ctas_per_sm : 1u);
  cfg.gridDim = dim3(std::min<uint32_t>(p.blocks * p.layer_count, resident));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = a.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

// ---------------------------------------------------------------- allocation-free entry point
// Scratch for callers that must not allocate: the activation tables normally live in a buffer the
// backend obtained from cudaMalloc; here they live in this fixed array, which every GPU that loads
// the library carries until the process exits.
constexpr size_t kStaticTableBytes = 256u * 1024u;
static __device__ __align__(256) uint8_t g_static_tables[kStaticTableBytes];

namespace {
// Device address of g_static_tables per device ordinal, resolved on the first call on that device.
// In host code the array's name is only a handle for the runtime, never a device pointer.
void* g_static_tables_ptr[64] = {};
}  // namespace

extern "C" tb_status tb_linear_forward_a8_static(tb_backend* backend, const tb_weights* weights, const void* x,
                                                 tb_dtype x_dtype, const float* act_scale, uint32_t m, void* y,
                                                 tb_dtype y_dtype, void* stream) {
  if (!backend || !weights) return tb_fail(TB_NULL_ARG, "null argument");
  if (weights->owner != backend) return tb_fail(TB_INVALID_INPUT, "weights handle belongs to another backend context");
  if (m == 0 || weights->n == 0) return TB_OK;
  if (!x || !y) return tb_fail(TB_NULL_ARG, "null activation or output pointer");
  if (x_dtype == TB_I8 && !act_scale) return tb_fail(TB_NULL_ARG, "int8 activations need act_scale");
  if (y_dtype == TB_I8) return tb_fail(TB_INVALID_INPUT, "output dtype must be fp32 or bf16");
  if (m > 4) return tb_fail(TB_INVALID_INPUT, "the allocation-free entry point takes at most 4 tokens per call, got " + std::to_string(m));
  if (!weights->fast) return tb_fail(TB_UNSUPPORTED_FORMAT, "the int8 path needs uniform plane counts, k % 256 == 0, group 128 and codec D2 or B3");
  if (backend->ordinal < 0 || backend->ordinal >= 64) return tb_fail(TB_INVALID_INPUT, "device ordinal out of range");
  const TableLayout tl = table_layout(weights, m);
  if (tl.total > kStaticTableBytes)
    return tb_fail(TB_INVALID_INPUT, "activation tables need " + std::to_string(tl.total) + " bytes but the fixed scratch holds " +
                                         std::to_string(kStaticTableBytes) + " (k = " + std::to_string(weights->k) + ", m = " + std::to_string(m) + ")");
  if (!tb_decode_supported(weights, m, backend->max_smem_optin, nullptr))
    return tb_fail(TB_UNSUPPORTED_FORMAT, "the decode kernel's shared-memory plan does not fit this shape");
  cudaError_t err = cudaSetDevice(backend->ordinal);
  if (err != cudaSuccess) return tb_cuda_fail(err, "select device");
  void*& tables = g_static_tables_ptr[backend->ordinal];
  if (!tables) {
    // once per device, with that device current
    err = cudaGetSymbolAddress(&tables, g_static_tables);
    if (err != cudaSuccess) { tables = nullptr; return tb_cuda_fail(err, "resolve the fixed scratch array"); }
  }
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : backend->stream;
  DecodeArgs d{};
  d.w = weights; d.x = x; d.x_dtype = x_dtype; d.act_scale_in = act_scale; d.m = m;
  d.y = y; d.y_dtype = y_dtype; d.y_row_stride = uint32_t(weights->n);
  d.status = backend->d_status; d.pdl = false;
  d.scratch = tables; d.scratch_bytes = kStaticTableBytes;
  // Nothing in the tables has to start at zero: the prepare kernel rewrites every entry the decode
  // kernel of the same call reads (z entries, start values, token scales) before it is read.
  err = tb_launch_prepare(d, st);
  if (err != cudaSuccess) return tb_cuda_fail(err, "launch prepare");
  err = tb_launch_decode(d, backend->prop.multiProcessorCount, backend->max_smem_optin, st);
  if (err != cudaSuccess) return tb_cuda_fail(err, "launch decode");
  return TB_OK;
}
