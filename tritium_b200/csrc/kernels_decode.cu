// Decode GEMV (1..4 tokens per pass) straight from the packed B3 / D2 arenas, sm_100a.
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
// Roles inside a CTA: eight consumer warps share every row block (each takes a run of
// (tile column, 16 row-planes) items, tile column outermost, so that the B fragments of a column
// stay in registers while the row-planes change), one producer warp feeds the ring, one combiner
// warp adds the consumers' partial sums of a finished block in a fixed order and stores the
// outputs.  The hand-offs are mbarriers: no warp waits for another consumer warp.
//
// The activation tables (B fragments, accumulator start values, token scales) are either built by
// the CTA itself from the activations (one launch per linear) or copied from global scratch that
// prepare_kernel filled (tensor-parallel shards that exchange the absmax, callers that supply
// their own scratch).
//
// Every wait is bounded; on timeout the kernel records TBF_WAIT_TIMEOUT and returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cfloat>
#include <cstdlib>
#include <string>

#include "tb_internal.h"

namespace {

constexpr int kWarps = 8;                       // consumer warps; then one producer and one combiner warp
constexpr int kThreads = (kWarps + 2) * 32;
constexpr int kConsumerThreads = kWarps * 32;
constexpr int kMaxStages = 4;
constexpr int kPartBufs = 4;   // row blocks whose partial sums may wait for the combiner
constexpr int kMaxGroupLayers = 128;   // layers of one grouped launch (descriptors live in shared memory)
constexpr uint32_t kBuildStagingBytes = 32 * 272 + 8 * 16 + 16 + 128;   // fused prologue: quantised activations of one pass of pairs, absmax partials, 1/rms per token, the peers' absmax

struct DecodeParams {
  const uint8_t* payload; const uint16_t* scales;   // single layer (layers == nullptr)
  const TbLayerDesc* layers; uint32_t layer_count; uint32_t y_layer_stride;   // grouped launch: outputs [layer][m][n]
  const uint8_t* tables; uint32_t table_bytes;   // z tables | accumulator start values | token scales
  // fused prologue (fused != 0): the CTA quantises x and builds its tables itself
  const void* x; const float* act_scale_in; const float* act_absmax_in; uint32_t x_dtype, fused;
  // fused RMSNorm in front of the quantiser (fused launches only; null = none) and `residual + y`
  // behind the token scale (fp32, indexed like y; null = none)
  const float* norm_weight; float norm_eps; uint32_t norm_zero_centered;
  const float* residual;
  // squared-ReLU gate in front of the quantiser (null = none): x holds the gate projection's fp32
  // output, relu2_up the up projection's, and the activation is (max(x, 0)^2) * up, the
  // reference's relu2_gate_f32 (crates/tritium-cuda/kernels/decode.cu:772-780)
  const float* relu2_up;
  // tensor-parallel row shard (tp != 0): absmax exchange of the fused prologue, output sum over the ranks
  TbCommView comm_absmax, comm_y; uint32_t tp;
  void* y; int32_t* acc_dump; const float* row_scale;
  uint32_t* status;
  uint32_t m, n, k, planes, tpr;            // m: valid tokens; tpr = k / 256
  uint32_t rows_per_stage, row_bytes, stage_bytes, scale_stage_bytes, blocks;
  uint32_t stages, y_dtype, y_row_stride;
  uint32_t dump_token_offset, dump_tokens_total;
  uint32_t pdl, wait_tables, ctas_per_sm;
  uint32_t inject_missing_tx;   // test hook: bytes the table barrier expects but nobody copies
  // shared memory offsets (bytes)
  uint32_t off_ring, off_scale_ring, off_z, off_cinit, off_part, off_actscale, off_xq;
};


// ---- peer-memory helpers (tensor-parallel row shards)
// One 8-byte word carries a value and the round it belongs to: a single store publishes both.
__device__ __forceinline__ void peer_store_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t peer_load_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
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
// The same with a time hint: the hardware may keep the thread suspended for up to `ns` nanoseconds
// before it reports "not yet", which keeps a waiting warp out of the issue slots.
__device__ __forceinline__ bool mbar_try_wait_for(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity), "r"(ns) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about two seconds of SM clocks or when another thread flagged an
// abort.  Returns false in both cases.
constexpr uint32_t kWaitHintNs = 20000;
constexpr long long kWaitLimitCycles = 4000000000ll;   // about two seconds of SM clocks
constexpr long long kDrainLimitCycles = 4000000ll;     // about two milliseconds: copies in flight after an abort
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, long long limit) {
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait_for(bar, parity, kWaitHintNs)) return true;
    if ((abort_flag && *abort_flag) || clock64() - t0 > limit) return false;
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, long long limit = kWaitLimitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, limit);
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// Shared-memory loads through 32-bit addresses (the generic 64-bit pointer arithmetic otherwise
// doubles every address computation in the inner loop).
template <int OFF = 0> __device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
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
// For the packed words of two rows, in MMA operand order: A[2i] = q_i of row a,
// A[2i+1] = q_i of row b.  A[10] and A[11] pad the third MMA; they meet zero B entries, so their
// value does not matter and they are left unwritten.
__device__ __forceinline__ void b3_quads2(uint32_t wa, uint32_t wb, uint32_t (&A)[12]) {
  const uint32_t ha01 = prmt(wa, 0x64646464u, 0x4140u), ha23 = prmt(wa, 0x64646464u, 0x4342u);
  const uint32_t hb01 = prmt(wb, 0x64646464u, 0x4140u), hb23 = prmt(wb, 0x64646464u, 0x4342u);
  const uint32_t a1 = hfma2_bits(ha01, kC3, kK3), a1h = hfma2_bits(ha23, kC3, kK3);
  const uint32_t b1 = hfma2_bits(hb01, kC3, kK3), b1h = hfma2_bits(hb23, kC3, kK3);
  const uint32_t a2 = hfma2_bits(ha01, kC9, kK9), a2h = hfma2_bits(ha23, kC9, kK9);
  const uint32_t b2 = hfma2_bits(hb01, kC9, kK9), b2h = hfma2_bits(hb23, kC9, kK9);
  const uint32_t a3 = hfma2_bits(a1, kC9, kK9), a3h = hfma2_bits(a1h, kC9, kK9);
  const uint32_t b3 = hfma2_bits(b1, kC9, kK9), b3h = hfma2_bits(b1h, kC9, kK9);
  const uint32_t a4 = hfma2_bits(a2, kC9b, kK9b), a4h = hfma2_bits(a2h, kC9b, kK9b);
  const uint32_t b4 = hfma2_bits(b2, kC9b, kK9b), b4h = hfma2_bits(b2h, kC9b, kK9b);
  A[0] = wa; A[1] = wb;
  A[2] = prmt(a1, a1h, 0x6420u); A[3] = prmt(b1, b1h, 0x6420u);
  A[4] = prmt(a2, a2h, 0x6420u); A[5] = prmt(b2, b2h, 0x6420u);
  A[6] = prmt(a3, a3h, 0x6420u); A[7] = prmt(b3, b3h, 0x6420u);
  A[8] = prmt(a4, a4h, 0x6420u); A[9] = prmt(b4, b4h, 0x6420u);
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
  const float* relu2_up;   // squared-ReLU gate: activation = (max(x, 0)^2) * relu2_up (x fp32); null = none
  uint8_t* tables; uint32_t* status;
  uint32_t m, mk, k, tpr, x_dtype, off_cinit, off_actscale, pdl;   // m valid tokens (grid.y), tables laid out for mk
  TbCommView comm;   // world > 1: the per-token absmax is the maximum over the ranks' slices
};

// (max(g, 0)^2) * u with the reference's association and no contraction
__device__ __forceinline__ float relu2_gate(float g, float u) {
  const float r = fmaxf(g, 0.0f);
  return __fmul_rn(__fmul_rn(r, r), u);
}
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
  const uint32_t j = blockIdx.x, t = blockIdx.y, ncol = (DUAL ? 4 : 2) * p.mk;
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
      for (uint32_t i = tid; i < p.k; i += 256) {
        const size_t at = size_t(t) * p.k + i;
        float v = load_act(p.x, p.x_dtype, at);
        if (p.relu2_up) v = relu2_gate(v, p.relu2_up[at]);
        mx = fmaxf(mx, fabsf(v));
      }
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
        // value and round number travel in one 8-byte word ([round parity][source rank][token]):
        // no flag, no fence; a word tagged with this round holds this round's value
        const uint32_t par = comm_seq & 1u;
        if (j == 0)
          for (uint32_t r = 0; r < p.comm.world; ++r)
            if (r != p.comm.rank)
              peer_store_u64(reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(p.comm.data[r]) + kCommAbsmaxWordsPrepare) +
                                 (par * kCommMaxWorld + p.comm.rank) * 4 + t,
                             (uint64_t(comm_seq) << 32) | __float_as_uint(gamma));
        float gmax = gamma;
        const uint64_t* own = reinterpret_cast<const uint64_t*>(reinterpret_cast<const uint8_t*>(p.comm.data[p.comm.rank]) + kCommAbsmaxWordsPrepare);
        const long long t0 = clock64();
        for (uint32_t r = 0; r < p.comm.world; ++r) {
          if (r == p.comm.rank) continue;
          for (uint32_t i = 0;; ++i) {
            const uint64_t word = peer_load_u64(own + (par * kCommMaxWorld + r) * 4 + t);
            if (uint32_t(word >> 32) == comm_seq) { gmax = fmaxf(gmax, __uint_as_float(uint32_t(word))); break; }
            if ((i & 63u) == 63u && clock64() - t0 > p.comm.wait_cycles) {
              if (atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = t; p.status[TBS_INFO1] = 500 + r; }
              break;
            }
          }
        }
        gamma_all = gmax;
      }
      __syncthreads();
      gamma = gamma_all;
    }
    const float scale_q = gamma > 0.f ? __fdiv_rn(127.0f, gamma) : 0.f;
    scale_out = __fdiv_rn(gamma, 127.0f);
    float v = load_act(p.x, p.x_dtype, size_t(t) * p.k + j * 256 + tid);
    if (p.relu2_up) v = relu2_gate(v, p.relu2_up[size_t(t) * p.k + j * 256 + tid]);
    if (!(fabsf(v) <= FLT_MAX) && atomicOr(&p.status[TBS_FLAGS], TBF_NONFINITE_ACT) == 0) {
      p.status[TBS_INFO0] = t * p.k + j * 256 + tid; p.status[TBS_INFO1] = __float_as_uint(v);
    }
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
    const uint32_t col = v * 2 * p.mk + 2 * t + hl;
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
// ---------------------------------------------------------------- fused prologue
// Eight elements of a row starting at element `idx` (a multiple of 8; rows are 16-byte aligned).
__device__ __forceinline__ void load8(const void* x, uint32_t dtype, size_t idx, float (&v)[8]) {
  if (dtype == TB_F32) {
    const float4 a = reinterpret_cast<const float4*>(x)[idx / 4], b = reinterpret_cast<const float4*>(x)[idx / 4 + 1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else if (dtype == TB_BF16) {
    const uint4 u = reinterpret_cast<const uint4*>(x)[idx / 8];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  } else {
    const uint2 u = reinterpret_cast<const uint2*>(x)[idx / 8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = float(int(int8_t(u.x >> (8 * i))));
      v[4 + i] = float(int(int8_t(u.y >> (8 * i))));
    }
  }
}

// MMA number that consumes digit pair `pair` of the packed words of `slot` (words 4*slot .. 4*slot+3;
// slot 3 of B3 is the bytewise MMA on word 12) for scale group `v`, or -1 when that combination holds
// only zeros (the inverse of slot_of).
template <int CODEC, bool DUAL> __device__ __forceinline__ int mma_of(uint32_t slot, uint32_t pair, uint32_t v) {
  if (CODEC == tbf::kB3) {
    if (DUAL) return slot < 3 ? int(slot * 3 + pair) : 9;
    if (slot == 0) return v == 0 ? int(pair) : -1;
    if (slot == 1) return int((v == 0 ? 3 : 6) + pair);
    if (slot == 2) return v == 1 ? int(9 + pair) : -1;
    return v == 1 ? 12 : -1;
  }
  if (DUAL) return int(slot * 2 + pair);
  return (slot >> 1) == v ? int(slot * 2 + pair) : -1;
}

constexpr uint32_t kChunkPairs = 32;    // (tile column, token) pairs quantised per pass of the table builder
constexpr uint32_t kPairStride = 272;   // staged bytes per pair: 256 codes + zero padding (B3 digits 256..259)

__device__ __forceinline__ int sbyte(uint32_t w, int b) { return int(int8_t(w >> (8 * b))); }

// Builds this CTA's activation tables in shared memory (same contents as prepare_kernel writes to
// global scratch): per-token absmax int8 quantisation of x, B-fragment entries, accumulator start
// values, token scales.  Called by the eight consumer warps (tid 0..255).
//
// Work item of the entry construction = one packed word position w of one (tile column, token,
// scale group): the 20 (B3) or 16 (D2) activations that meet the word's digits are five (four)
// aligned 32-bit words of the staged codes, every one of them inside a single scale group; their
// transformed values z = x_t - 3 x_(t-1) (B3; x_t for D2), split as 4*high + low, are the table
// words of that position.  Items are independent, so the whole CTA works on them at once.
// y = (x * inv) * w (or (1 + w)) for eight consecutive columns: the reference's rmsnorm expression
// (crates/tritium-nn/src/ops/rmsnorm.rs:88-91), one rounding per operation.
__device__ __forceinline__ void apply_norm(const DecodeParams& p, float inv, uint32_t col, float (&v)[8]) {
  float w[8];
  load8(p.norm_weight, TB_F32, col, w);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float scale = p.norm_zero_centered ? __fadd_rn(1.0f, w[e]) : w[e];
    v[e] = __fmul_rn(__fmul_rn(v[e], inv), scale);
  }
}

// squared-ReLU gate for eight consecutive activations (see relu2_gate)
__device__ __forceinline__ void apply_gate(const DecodeParams& p, size_t at, float (&v)[8]) {
  float u[8];
  load8(p.relu2_up, TB_F32, at, u);
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = relu2_gate(v[e], u[e]);
}

template <int CODEC, bool DUAL, int M>
__device__ __forceinline__ void build_tables(const DecodeParams& p, uint8_t* smem, uint32_t tid, uint32_t tp_seq) {
  constexpr int kNM = MmaCount<CODEC, DUAL>::value;
  constexpr uint32_t ncol = (DUAL ? 4 : 2) * M;
  constexpr bool B3 = CODEC == tbf::kB3;
  constexpr uint32_t kDigits = B3 ? 5 : 4, kWords = B3 ? 13 : 16;   // digits per packed byte, packed words per tile-plane
  const uint32_t warp = tid >> 5, lane = tid & 31;
  uint8_t* xq = smem + p.off_xq;                                                             // [kChunkPairs][kPairStride]
  float* red = reinterpret_cast<float*>(smem + p.off_xq + kChunkPairs * kPairStride);       // [warp][4]
  uint32_t* ztab = reinterpret_cast<uint32_t*>(smem + p.off_z);
  int* cinit = reinterpret_cast<int*>(smem + p.off_cinit);
  float* act_scale = reinterpret_cast<float*>(smem + p.off_actscale);
  float scale_q[M], scale_out[M], inv_rms[M];
  const uint32_t pairs = p.tpr * M;
  const bool norm = p.norm_weight != nullptr;
#pragma unroll
  for (int t = 0; t < M; ++t) inv_rms[t] = 1.f;
  if (norm) {
    // RMSNorm prologue, in the reference's canonical order (crates/tritium-nn/src/ops/rmsnorm.rs:20-34,
    // crates/tritium-cuda/kernels/decode.cu:533-640): 256 slots, slot t folds x[t], x[t+256], ...
    // ascending; then the power-of-two tree part[t] += part[t+off].  The 256 consumer threads are
    // the 256 slots.  The staging area is free until the quantise phase.
    float* part = reinterpret_cast<float*>(xq);
    float* inv_s = red + kWarps * 4;
#pragma unroll
    for (int t = 0; t < M; ++t) {
      if (uint32_t(t) >= p.m) break;
      float acc = 0.f;
      for (uint32_t i = tid; i < p.k; i += kConsumerThreads) {
        const size_t at = size_t(t) * p.k + i;
        const float v = p.x_dtype == TB_F32 ? static_cast<const float*>(p.x)[at]
                                            : __bfloat162float(static_cast<const __nv_bfloat16*>(p.x)[at]);
        acc = __fadd_rn(acc, __fmul_rn(v, v));
      }
      part[tid] = acc;
      consumer_sync();
      if (tid < 128) part[tid] = __fadd_rn(part[tid], part[tid + 128]);
      consumer_sync();
      if (tid < 64) part[tid] = __fadd_rn(part[tid], part[tid + 64]);
      consumer_sync();
      if (tid < 32) {
        float v = __fadd_rn(part[tid], part[tid + 32]);
        for (int o = 16; o; o >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, o));   // lane t pairs with t + o
        if (tid == 0) inv_s[t] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(v, float(p.k)), p.norm_eps)));
      }
      consumer_sync();
    }
#pragma unroll
    for (int t = 0; t < M; ++t) inv_rms[t] = uint32_t(t) < p.m ? inv_s[t] : 1.f;
    consumer_sync();   // the slots turn back into staging
  }
  if (tid < kChunkPairs) *reinterpret_cast<uint4*>(xq + tid * kPairStride + 256) = make_uint4(0, 0, 0, 0);
  if (p.x_dtype == TB_I8) {
#pragma unroll
    for (int t = 0; t < M; ++t) { scale_q[t] = 1.f; scale_out[t] = uint32_t(t) < p.m ? p.act_scale_in[t] : 0.f; }
  } else {
    if (!p.act_absmax_in) {
#pragma unroll
      for (int t = 0; t < M; ++t) {
        float mx = 0.f;
        for (uint32_t i = tid * 8; i < p.k && uint32_t(t) < p.m; i += kConsumerThreads * 8) {
          float v[8];
          load8(p.x, p.x_dtype, size_t(t) * p.k + i, v);
          if (p.relu2_up) apply_gate(p, size_t(t) * p.k + i, v);
          if (norm) apply_norm(p, inv_rms[t], i, v);
#pragma unroll
          for (int e = 0; e < 8; ++e) mx = fmaxf(mx, fabsf(v[e]));
        }
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red[warp * 4 + t] = mx;
      }
      consumer_sync();
    }
    float* peer_gamma = red + kWarps * 4 + 4;   // [rank][token]
    if (p.tp && !p.act_absmax_in) {
      // Row shard: the row's absmax is the maximum over the ranks' slices.  CTA 0 pushes this
      // slice's value, tagged with the round, into every peer's copy of the slot; every CTA then
      // finds the peers' values in its own GPU's memory.  Two parities alternate, so a rank that
      // is one round ahead cannot overwrite a value still being read.
      const TbCommView& cv = p.comm_absmax;
      const uint32_t par = tp_seq & 1u;
      if (tid < cv.world && tid != cv.rank) {
        if (blockIdx.x == 0) {
          uint64_t* dst = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(cv.data[tid]) + kCommAbsmaxWords) + (par * kCommMaxWorld + cv.rank) * 4;
          for (uint32_t t = 0; t < p.m; ++t) {
            float mine = 0.f;
            for (uint32_t w2 = 0; w2 < uint32_t(kWarps); ++w2) mine = fmaxf(mine, red[w2 * 4 + t]);
            peer_store_u64(dst + t, (uint64_t(tp_seq) << 32) | __float_as_uint(mine));
          }
        }
        const uint64_t* src = reinterpret_cast<const uint64_t*>(reinterpret_cast<const uint8_t*>(cv.data[cv.rank]) + kCommAbsmaxWords) + (par * kCommMaxWorld + tid) * 4;
        const long long t0 = clock64();
        for (uint32_t t = 0; t < p.m; ++t) {
          float got = 0.f;
          for (uint32_t i = 0;; ++i) {
            const uint64_t v = peer_load_u64(src + t);
            if (uint32_t(v >> 32) == tp_seq) { got = __uint_as_float(uint32_t(v)); break; }
            if ((i & 63u) == 63u && clock64() - t0 > cv.wait_cycles) {
              if (atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = tid; p.status[TBS_INFO1] = 600 + t; }
              break;
            }
          }
          peer_gamma[tid * 4 + t] = got;
        }
      }
      consumer_sync();
    }
#pragma unroll
    for (int t = 0; t < M; ++t) {
      float gamma = 0.f;
      if (p.act_absmax_in) gamma = uint32_t(t) < p.m ? p.act_absmax_in[t] : 0.f;   // absmax over the full (unsharded) row, supplied by the caller
      else {
        for (uint32_t w2 = 0; w2 < uint32_t(kWarps); ++w2) gamma = fmaxf(gamma, red[w2 * 4 + t]);
        if (p.tp && uint32_t(t) < p.m)
          for (uint32_t r = 0; r < p.comm_absmax.world; ++r)
            if (r != p.comm_absmax.rank) gamma = fmaxf(gamma, peer_gamma[r * 4 + t]);
      }
      scale_q[t] = gamma > 0.f ? __fdiv_rn(127.0f, gamma) : 0.f;
      scale_out[t] = __fdiv_rn(gamma, 127.0f);
    }
  }
  for (uint32_t base = 0; base < pairs; base += kChunkPairs) {
    const uint32_t chunk = min(kChunkPairs, pairs - base);
    // ---- quantise: a warp takes whole pairs (lane = eight consecutive activations), and adds up
    // the accumulator start values of the pair's two scale groups on the way
#pragma unroll
    for (uint32_t r = 0; r < kChunkPairs / kWarps; ++r) {
      const uint32_t lp = warp + r * kWarps;
      if (lp >= chunk) continue;
      const uint32_t pr = base + lp, j = pr / M, t = pr - j * M;
      if (t >= p.m) continue;   // table entries of absent tokens are never read for an output
      float v[8];
      load8(p.x, p.x_dtype, size_t(t) * p.k + j * 256 + lane * 8, v);
      float sq = scale_q[0], inv = inv_rms[0];
#pragma unroll
      for (int tt = 1; tt < M; ++tt) { sq = t == uint32_t(tt) ? scale_q[tt] : sq; inv = t == uint32_t(tt) ? inv_rms[tt] : inv; }
      if (p.relu2_up) apply_gate(p, size_t(t) * p.k + j * 256 + lane * 8, v);
      if (norm) apply_norm(p, inv, j * 256 + lane * 8, v);
      int q[8];
      bool bad = false;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        bad |= !(fabsf(v[e]) <= FLT_MAX);
        q[e] = p.x_dtype == TB_I8 ? int(v[e]) : int(fminf(127.f, fmaxf(-128.f, rintf(__fmul_rn(v[e], sq)))));
      }
      if (bad && atomicOr(&p.status[TBS_FLAGS], TBF_NONFINITE_ACT) == 0) {
        p.status[TBS_INFO0] = t * p.k + j * 256 + lane * 8; p.status[TBS_INFO1] = 0x7fc00000u;
      }
      uint2 packed;
      packed.x = uint32_t(q[0] & 0xff) | (uint32_t(q[1] & 0xff) << 8) | (uint32_t(q[2] & 0xff) << 16) | (uint32_t(q[3] & 0xff) << 24);
      packed.y = uint32_t(q[4] & 0xff) | (uint32_t(q[5] & 0xff) << 8) | (uint32_t(q[6] & 0xff) << 16) | (uint32_t(q[7] & 0xff) << 24);
      reinterpret_cast<uint2*>(xq + lp * kPairStride)[lane] = packed;
      // accumulator start values (see prepare_kernel): lanes 0..15 hold scale group 0, 16..31 group 1
      int sum = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int coef = 1;
        if (B3) { const int d = int(lane * 8 + e) % 5; coef = d == 0 ? 1 : d == 1 ? -2 : d == 4 ? 2 : -1; }
        sum += q[e] * coef;
      }
      for (int o = 8; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if ((lane & 15) == 0) cinit[(t * p.tpr + j) * 2 + (lane >> 4)] = -sum;
    }
    consumer_sync();
    // ---- entries: item = (pair of the chunk, scale group, packed word position)
    for (uint32_t item = tid; item < chunk * 2 * kWords; item += kConsumerThreads) {
      const uint32_t lp = item / (2 * kWords), rem = item - lp * (2 * kWords), v = rem / kWords, w = rem - v * kWords;
      const uint32_t pr = base + lp, j = pr / M, t = pr - j * M;
      if (t >= p.m) continue;
      const uint32_t slot = w >> 2, c = w & 3;
      const bool bytewise = B3 && slot == 3;
      if (!DUAL && mma_of<CODEC, false>(slot, 0, v) < 0) continue;   // no MMA reads this word for this scale group
      // the activations that meet the digits of packed word w: words of four, each inside one scale group
      const uint32_t t0 = 4 * kDigits * w;
      const uint32_t* src = reinterpret_cast<const uint32_t*>(xq + lp * kPairStride + t0);
      int a[4 * 5];
#pragma unroll
      for (uint32_t kw = 0; kw < kDigits; ++kw) {
        const uint32_t word = (((t0 + 4 * kw) >> 7) == v) ? src[kw] : 0u;   // trits 256..259 read the zero padding
#pragma unroll
        for (int b = 0; b < 4; ++b) a[4 * kw + b] = sbyte(word, b);
      }
      // z of (byte e, digit i) and its parts
      uint32_t hi[5][4], lo[5][4];   // [digit][byte]
#pragma unroll
      for (uint32_t e = 0; e < 4; ++e) {
#pragma unroll
        for (uint32_t i = 0; i < kDigits; ++i) {
          const int cur = a[kDigits * e + i];
          const int z = (B3 && i > 0) ? cur - 3 * a[kDigits * e + i - 1] : cur;
          hi[i][e] = uint32_t(z >> 2) & 0xffu;
          lo[i][e] = uint32_t(z) & 3u;
        }
      }
      const uint32_t col0 = (DUAL ? v * 2 * M : 0) + 2 * t;
      if (bytewise) {
        // byte e of word 12 belongs to lane column e: operand quad 0 = digits 0..3, quad 1 byte 0 = digit 4
        const uint32_t mma = uint32_t(mma_of<CODEC, DUAL>(3, 0, v));
#pragma unroll
        for (uint32_t e = 0; e < 4; ++e) {
          uint32_t* at = ztab + (((j * kNM + mma) * ncol + col0) * 4 + e) * 2;
          at[0] = hi[0][e] | (hi[1][e] << 8) | (hi[2][e] << 16) | (hi[3][e] << 24); at[1] = hi[4][e];
          at[8] = lo[0][e] | (lo[1][e] << 8) | (lo[2][e] << 16) | (lo[3][e] << 24); at[9] = lo[4][e];
        }
      } else {
#pragma unroll
        for (uint32_t i = 0; i < kDigits; ++i) {
          // digit i: MMA of (slot, digit pair i/2), operand quad i%2; bytes e = 0..3
          const uint32_t mma = uint32_t(mma_of<CODEC, DUAL>(slot, i >> 1, v));
          uint32_t* at = ztab + (((j * kNM + mma) * ncol + col0) * 4 + c) * 2 + (i & 1);
          at[0] = hi[i][0] | (hi[i][1] << 8) | (hi[i][2] << 16) | (hi[i][3] << 24);
          at[8] = lo[i][0] | (lo[i][1] << 8) | (lo[i][2] << 16) | (lo[i][3] << 24);   // low part: the next column
          if (B3 && i == 4) { at[1] = 0u; at[9] = 0u; }                                 // the fifth digit has no partner
        }
      }
    }
    consumer_sync();
  }
  if (tid < uint32_t(M)) {
    float so = scale_out[0];
#pragma unroll
    for (int tt = 1; tt < M; ++tt) so = tid == uint32_t(tt) ? scale_out[tt] : so;
    act_scale[tid] = so;
  }
}

// ---------------------------------------------------------------- the kernel
// M: token columns the tables are laid out for (1, 2 or 4; p.m <= M tokens are valid).
// SETS: blocks of 16 row-planes in one row block (rows_per_stage * PLANES / 16).
template <int CODEC, int PLANES, int M, int SETS>
__global__ void __launch_bounds__(kThreads, 2) decode_kernel(const DecodeParams p) {
  using T = Traits<CODEC>;
  constexpr bool DUAL = M <= 2;
  constexpr int kNM = MmaCount<CODEC, DUAL>::value;
  constexpr uint32_t ncol = (DUAL ? 4 : 2) * M;   // MMA columns in use
  constexpr uint32_t NC = DUAL ? 2 * M : M;       // (scale group, token) cells a lane quad finishes
  constexpr bool kPlaneSets = PLANES == 3;        // a set is one plane of 16 rows: the lane adds a row's planes itself
  constexpr int YN = kPlaneSets ? 1 : SETS;       // partial sums a lane keeps for each of its two rows
  constexpr uint32_t kSliceFloats = YN * 16 * NC;   // one consumer warp's partial sums of a row block
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], table_bar, part_full[kPartBufs], part_empty[kPartBufs];
  __shared__ uint32_t abort_flag, tp_round;
  __shared__ TbLayerDesc layer_desc[kMaxGroupLayers];

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* ring = smem + p.off_ring;
  uint8_t* scale_ring = smem + p.off_scale_ring;
  const uint2* ztab = reinterpret_cast<const uint2*>(smem + p.off_z);
  const int* cinit = reinterpret_cast<const int*>(smem + p.off_cinit);
  float* part = reinterpret_cast<float*>(smem + p.off_part);
  const float* act_scale = reinterpret_cast<const float*>(smem + p.off_actscale);

  if (tid == 0) {
    abort_flag = 0;
    for (uint32_t s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kWarps); }
    mbar_init(&table_bar, 1);
    for (int b = 0; b < kPartBufs; ++b) { mbar_init(&part_full[b], kWarps); mbar_init(&part_empty[b], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (uint32_t l = tid; l < p.layer_count; l += kThreads) {
    if (p.layers) { layer_desc[l].payload = p.layers[l].payload; layer_desc[l].scales = p.layers[l].scales; }
    else { layer_desc[l].payload = p.payload; layer_desc[l].scales = p.scales; }
  }
  __syncthreads();
  // The next kernel on the stream may begin once every CTA has passed this point.  A launch that
  // builds its own tables shares no scratch with its neighbours, so it raises the trigger at
  // once.  A launch that waits for tables in global scratch raises it only after that wait, so
  // that a later launch which shares the tables (and does not wait) cannot outrun them.
  if (p.pdl && (p.fused || !p.wait_tables)) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const uint32_t total_blocks = p.blocks * p.layer_count;
  const uint32_t my_blocks = blockIdx.x < total_blocks ? (total_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (warp == kWarps) {
    // ------------------------------------------------ producer: weights do not depend on the
    // previous kernel, so the stream starts before griddepcontrol.wait.
    if (lane != 0) return;
    uint32_t fills[kMaxStages] = {0, 0, 0, 0};
    uint32_t s = 0, round = 0;
    uint32_t layer = blockIdx.x / p.blocks, blk = blockIdx.x - layer * p.blocks;
    for (uint32_t it = 0; it < my_blocks; ++it) {
      if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1, &abort_flag)) {
        abort_flag = 1;
        if (atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = it; p.status[TBS_INFO1] = 100 + s; }
        break;
      }
      const uint8_t* pay = layer_desc[layer].payload;
      const uint8_t* scs = reinterpret_cast<const uint8_t*>(layer_desc[layer].scales);
      mbar_expect_tx(&full_bar[s], p.stage_bytes + p.scale_stage_bytes);
      bulk_g2s(ring + size_t(s) * p.stage_bytes, pay + size_t(blk) * p.stage_bytes, p.stage_bytes, &full_bar[s]);
      bulk_g2s(scale_ring + size_t(s) * p.scale_stage_bytes, scs + size_t(blk) * p.scale_stage_bytes,
               p.scale_stage_bytes, &full_bar[s]);
      ++fills[s];
      if (++s == p.stages) { s = 0; ++round; }
      for (blk += gridDim.x; blk >= p.blocks; blk -= p.blocks) ++layer;
    }
    // Do not leave the CTA while a copy may still be landing in its shared memory: wait
    // (bounded) for the latest fill of every slot.  In the normal path these have all
    // completed already, because the consumers waited on them.
    for (uint32_t sl = 0; sl < p.stages; ++sl)
      if (fills[sl]) mbar_wait(&full_bar[sl], (fills[sl] - 1) & 1, nullptr, kDrainLimitCycles);
    return;
  }

  if (warp == kWarps + 1) {
    // ------------------------------------------------ combiner: adds the eight consumer warps'
    // partial sums of a finished row block (fixed order: plane, scale-group cell, warp), applies
    // the token scale and stores the outputs, while the consumers work on later blocks.
    // Round of the exchanges between the ranks: one more than the rounds this slot has completed.
    // The word lives in device memory, so a replayed CUDA graph counts on by itself; the previous
    // launch on the stream may be the one that completes the round before, so wait for it first.
    uint32_t tp_seq = 0;
    if (p.tp) {
      if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
      tp_seq = *reinterpret_cast<volatile uint32_t*>(p.comm_y.flags[p.comm_y.rank] + kCommDecodeEpoch) + 1u;
    }
    if (!mbar_wait(&table_bar, 0, &abort_flag)) return;   // token scales live in the tables
    uint32_t buf = 0, parity = 0;
    uint32_t layer = blockIdx.x / p.blocks, blk = blockIdx.x - layer * p.blocks;
    for (uint32_t it = 0; it < my_blocks; ++it) {
      if (!mbar_wait(&part_full[buf], parity, &abort_flag)) {
        abort_flag = 1;
        if (lane == 0 && atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = it; p.status[TBS_INFO1] = 300 + buf; }
        return;
      }
      const uint32_t row0 = blk * p.rows_per_stage;
      const float* stage_part = part + size_t(buf) * kWarps * kSliceFloats;
      for (uint32_t e = lane; e < p.rows_per_stage * p.m; e += 32) {
        const uint32_t t = e / p.rows_per_stage, r = e - t * p.rows_per_stage;
        if (row0 + r >= p.n) continue;
        float sum = 0.f;
        constexpr uint32_t kSplit = PLANES == 2 ? 2 : 1;   // planes that arrive as separate partial sums
#pragma unroll
        for (uint32_t q = 0; q < kSplit; ++q) {
#pragma unroll
          for (uint32_t grp = 0; grp < (DUAL ? 2u : 1u); ++grp) {
            const float* src = stage_part + (r * kSplit + q) * NC + grp * M + t;
            float v[kWarps];
#pragma unroll
            for (int w2 = 0; w2 < kWarps; ++w2) v[w2] = src[w2 * kSliceFloats];
#pragma unroll
            for (int w2 = 0; w2 < kWarps; ++w2) sum = __fadd_rn(sum, v[w2]);
          }
        }
        float out = __fmul_rn(sum, act_scale[t]);
        if (p.row_scale) out = __fmul_rn(out, p.row_scale[row0 + r]);
        if (p.tp) {
          // this rank's partial goes into every rank's copy of the slot: [round parity][source rank][token][row]
          // Each value travels with the round number in one 8-byte word, so the receiver needs no
          // flag, no counter and no fence: a word whose tag is this round is this round's value.
          const size_t at = (size_t((tp_seq & 1u) * p.comm_y.world + p.comm_y.rank) * p.m + t) * p.n + row0 + r;
          const uint64_t word = (uint64_t(tp_seq) << 32) | __float_as_uint(out);
          for (uint32_t dst = 0; dst < p.comm_y.world; ++dst) peer_store_u64(reinterpret_cast<uint64_t*>(p.comm_y.data[dst]) + at, word);
          continue;
        }
        const size_t idx = size_t(layer) * p.y_layer_stride + size_t(t) * p.y_row_stride + row0 + r;
        if (p.residual) out = __fadd_rn(p.residual[idx], out);   // crates/tritium-cuda/kernels/tq2_0_add.cu:577-637
        if (p.y_dtype == TB_F32) static_cast<float*>(p.y)[idx] = out;
        else static_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(out);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&part_empty[buf]);
      if (++buf == kPartBufs) { buf = 0; parity ^= 1; }
      for (blk += gridDim.x; blk >= p.blocks; blk -= p.blocks) ++layer;
    }
    if (p.tp) {
      // Second pass over this CTA's row blocks: wait until every rank's word of an output carries
      // this round's tag (each peer's CTA of the same index pushed it at about the same time), then
      // add the ranks' partials in rank order, so that every rank stores the same bits.
      const TbCommView& cv = p.comm_y;
      const uint64_t* base = reinterpret_cast<const uint64_t*>(cv.data[cv.rank]) + size_t((tp_seq & 1u) * cv.world) * p.m * p.n;
      const size_t src_stride = size_t(p.m) * p.n;
      const long long t0 = clock64();
      bool ok = true;
      blk = blockIdx.x;
      for (uint32_t it = 0; it < my_blocks && ok; ++it, blk += gridDim.x) {
        const uint32_t row0 = blk * p.rows_per_stage;
        for (uint32_t e = lane; e < p.rows_per_stage * p.m && ok; e += 32) {
          const uint32_t t = e / p.rows_per_stage, r = e - t * p.rows_per_stage;
          if (row0 + r >= p.n) continue;
          const uint64_t* src = base + size_t(t) * p.n + row0 + r;
          float part_of[kCommMaxWorld];
          uint32_t pending = (1u << cv.world) - 1u;
          for (uint32_t spin = 0; pending; ++spin) {
#pragma unroll
            for (uint32_t q = 0; q < kCommMaxWorld; ++q)
              if (pending & (1u << q)) {
                const uint64_t word = peer_load_u64(src + q * src_stride);
                if (uint32_t(word >> 32) == tp_seq) { part_of[q] = __uint_as_float(uint32_t(word)); pending &= ~(1u << q); }
              }
            if (pending && (spin & 63u) == 63u && clock64() - t0 > cv.wait_cycles) {
              if (atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = blk; p.status[TBS_INFO1] = 700 + pending; }
              ok = false;
              break;
            }
          }
          if (!ok) break;
          float out = part_of[0];
#pragma unroll
          for (uint32_t q = 1; q < kCommMaxWorld; ++q)
            if (q < cv.world) out = __fadd_rn(out, part_of[q]);
          const size_t idx = size_t(t) * p.y_row_stride + row0 + r;
          if (p.residual) out = __fadd_rn(p.residual[idx], out);
          if (p.y_dtype == TB_F32) static_cast<float*>(p.y)[idx] = out;
          else static_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(out);
        }
        ok = __all_sync(0xffffffffu, ok);
      }
      // the last CTA to get here closes the round (also after a wait that ran out: the next
      // launch must not wait for a round that was given up)
      __syncwarp();
      if (lane == 0) {
        __threadfence();
        uint32_t* flags = cv.flags[cv.rank];
        if (atomicAdd(flags + kCommDecodeDone, 1u) == gridDim.x - 1) {
          flags[kCommDecodeDone] = 0;
          *reinterpret_cast<volatile uint32_t*>(flags + kCommDecodeEpoch) = tp_seq;
        }
      }
    }
    return;
  }

  // -------------------------------------------------- consumers: activation tables
  if (p.fused) {
    // x may be the previous kernel's output: wait for it (the weight stream is already running)
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (p.tp) {
      if (tid == 0) tp_round = *reinterpret_cast<volatile uint32_t*>(p.comm_y.flags[p.comm_y.rank] + kCommDecodeEpoch) + 1u;
      consumer_sync();
    }
    build_tables<CODEC, DUAL, M>(p, smem, tid, p.tp ? tp_round : 0u);
    consumer_sync();
    if (tid == 0) mbar_arrive(&table_bar);   // releases the combiner
  } else {
    // The prepare kernel (previous launch on this stream) wrote the tables to global scratch; one
    // bulk copy brings them in.
    if (p.pdl && p.wait_tables) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    if (tid == 0) {
      mbar_expect_tx(&table_bar, p.table_bytes + p.inject_missing_tx);
      bulk_g2s(smem + p.off_z, p.tables, p.table_bytes, &table_bar);
    }
    if (!mbar_wait(&table_bar, 0, &abort_flag)) {
      abort_flag = 1;
      if (lane == 0 && atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = 0; p.status[TBS_INFO1] = 200; }
      return;
    }
  }

  // -------------------------------------------------- consumers: main loop
  const uint32_t g = lane >> 2, c = lane & 3;
  // Which (scale group, token) cell of the C fragment this lane finishes.
  //   separate accumulators: lane column c holds token c, both groups;
  //   dual columns:          lane column c holds group c / M, token c % M.
  // Lane columns beyond the cells in use compute sums that nobody reads.
  const bool lane_has_cell = c < NC;
  const uint32_t cell_group = DUAL ? ((c >= M && lane_has_cell) ? 1u : 0u) : 0u;
  const uint32_t cell_token = lane_has_cell ? (DUAL ? c - cell_group * M : c) : 0u;
  // MMA columns beyond `ncol` produce sums nobody reads, so their lanes may load any valid
  // table entry: fold them onto the used columns instead of masking.
  const uint32_t bcol = g % ncol;
  const uint32_t byte_sel = c | (c << 4) | ((4u + c) << 8) | ((4u + c) << 12);   // byte c of two words -> bytes 0 and 2
  constexpr uint32_t zstep = ncol * 4;
  const uint32_t groups_per_row = p.tpr * 2;
  const bool dump = p.acc_dump != nullptr;
  constexpr uint32_t kPlaneBytes = T::kPlaneBytes;
  constexpr int kMagic = 0x4B400000;   // bits of 1.5 * 2^23: an integer added here reads as float 12582912 + v

  // Lane -> weights.  A set is 16 MMA rows (row-planes) of one tile column:
  //   one plane:    set q = rows 16q .. 16q+15              (the lane holds rows g and g+8)
  //   two planes:   set q = rows 8q .. 8q+7, both planes    (the lane holds (row g/2, plane g%2) and row + 4)
  //   three planes: set q = plane q of the block's 16 rows  (rows g and g+8; the planes of a row add up in the lane)
  // so that every address is lane base + set stride + half stride, the same for every block.
  const uint32_t row_bytes = p.tpr * PLANES * kPlaneBytes, srow_bytes = p.tpr * PLANES * 4;
  const uint32_t lrow = PLANES == 2 ? g >> 1 : g, lplane = PLANES == 2 ? g & 1 : 0;
  const uint32_t lane_w = lrow * row_bytes + lplane * kPlaneBytes + c * 4;             // word c of the lane's first tile-plane
  const uint32_t lane_s = lrow * srow_bytes + lplane * 4 + (DUAL ? cell_group * 2 : 0);
  constexpr uint32_t kHalfRows = PLANES == 2 ? 4 : 8;
  const uint32_t db_w = kHalfRows * row_bytes, db_s = kHalfRows * srow_bytes;           // first -> second row of the lane
  const uint32_t dq_w = kPlaneSets ? kPlaneBytes : 2 * kHalfRows * row_bytes;           // set q -> set q + 1
  const uint32_t dq_s = kPlaneSets ? 4u : 2 * kHalfRows * srow_bytes;
  const uint32_t w12 = 48 - 4 * c;   // from word c to word 12 of a tile-plane
  const uint32_t zlane0 = smem_addr(ztab + bcol * 4 + c);
  const uint32_t cin0 = smem_addr(cinit + cell_token * p.tpr * 2 + cell_group);
  const uint32_t ring_addr = smem_addr(ring), scale_ring_addr = smem_addr(scale_ring);

  uint32_t s = 0, full_parity = 0, buf = 0, part_round = 0, vw = warp;
  for (uint32_t it = 0; it < my_blocks; ++it) {
    if (!mbar_wait(&full_bar[s], full_parity, &abort_flag)) {
      abort_flag = 1;
      if (lane == 0 && atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = it; p.status[TBS_INFO1] = s; }
      return;
    }
    const uint32_t wstage = ring_addr + s * p.stage_bytes + lane_w;
    const uint32_t sstage = scale_ring_addr + s * p.scale_stage_bytes + lane_s;

    float ya[YN], yb[YN];
#pragma unroll
    for (int q = 0; q < YN; ++q) { ya[q] = 0.f; yb[q] = 0.f; }

    // This warp takes the tile columns vw, vw + 8, ...  The assignment rotates from block to
    // block, so that one-column differences between warps even out.
    for (uint32_t j = vw; j < p.tpr; j += kWarps) {
      // B fragments of tile column j stay in registers while the row-planes change
      uint2 bf[kNM];
      {
        const uint32_t zlane = zlane0 + j * (kNM * ncol * 4 * 8);
#pragma unroll
        for (int mm = 0; mm < kNM; ++mm) bf[mm] = lds_u64(zlane + mm * (zstep * 8));
      }
      const int ci0 = int(lds_u32(cin0 + j * 8)) + kMagic, ci1 = DUAL ? 0 : int(lds_u32<4>(cin0 + j * 8)) + kMagic;
      const uint32_t wcol = wstage + j * (PLANES * kPlaneBytes);
      const uint32_t scol = sstage + j * (PLANES * 4);
#pragma unroll
      for (int q = 0; q < SETS; ++q) {
        const uint32_t wa = wcol + q * dq_w, wb = wa + db_w;
        int acc0[4], acc1[4];   // group 0 / group 1 sums (dual layout: acc0 holds this lane's group)
        if constexpr (CODEC == tbf::kB3) {
          // Two accumulation chains, fed alternately, so that consecutive MMAs rarely depend on
          // each other.  Dual layout: chain A takes words c and 8+c, chain B words 4+c and 12, and
          // their sum is the cell.  Separate accumulators: chain A is scale group 0, chain B group 1.
          int sA[4], sB[4];
          uint32_t A[12];
#define TB_MMA3(first, acc, i0)                                                          \
  first(acc, A[0], A[1], A[2], A[3], bf[i0].x, bf[i0].y);                                \
  mma_u8s8(acc, A[4], A[5], A[6], A[7], bf[(i0) + 1].x, bf[(i0) + 1].y);                 \
  mma_u8s8(acc, A[8], A[9], A[10], A[11], bf[(i0) + 2].x, bf[(i0) + 2].y)
          b3_quads2(lds_u32(wa), lds_u32(wb), A);
          TB_MMA3(mma_u8s8_first, sA, 0);
          b3_quads2(lds_u32(wa + 16), lds_u32(wb + 16), A);
          if constexpr (DUAL) {
            TB_MMA3(mma_u8s8_first, sB, 3);
          } else {
            // the words 4..7 straddle the two scale groups: once per group, masked on the B side
            TB_MMA3(mma_u8s8, sA, 3);
            TB_MMA3(mma_u8s8_first, sB, 6);
          }
          constexpr int o2 = DUAL ? 6 : 9, o3 = DUAL ? 9 : 12;
          b3_quads2(lds_u32(wa + 32), lds_u32(wb + 32), A);
          if constexpr (DUAL) {
            TB_MMA3(mma_u8s8, sA, o2);
          } else {
            TB_MMA3(mma_u8s8, sB, o2);
          }
#undef TB_MMA3
          {
            // word 12: lane column c takes byte c of both rows through one half2 chain; its five
            // quotients fill the lane's eight k-slots of a single MMA
            const uint32_t w12a = lds_u32(wa + w12), w12b = lds_u32(wb + w12);
            const uint32_t h = (prmt(w12a, w12b, byte_sel) & 0x00ff00ffu) | 0x64006400u;
            const uint32_t q1 = hfma2_bits(h, kC3, kK3), q2 = hfma2_bits(h, kC9, kK9);
            const uint32_t q3 = hfma2_bits(q1, kC9, kK9), q4 = hfma2_bits(q2, kC9b, kK9b);
            const uint32_t u = prmt(h, q1, 0x6240u), v = prmt(q2, q3, 0x6240u);
            mma_u8s8(sB, prmt(u, v, 0x5410u), prmt(u, v, 0x7632u), prmt(q4, 0u, 0x4440u), prmt(q4, 0u, 0x4442u), bf[o3].x, bf[o3].y);
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
            const uint32_t va = lds_u32(wa + sl * 16), vb = lds_u32(wb + sl * 16);
            mma_u8s8_first(sq[sl], va & 0x03030303u, vb & 0x03030303u, (va >> 2) & 0x03030303u, (vb >> 2) & 0x03030303u,
                           bf[sl * 2].x, bf[sl * 2].y);
            mma_u8s8(sq[sl], (va >> 4) & 0x03030303u, (vb >> 4) & 0x03030303u, (va >> 6) & 0x03030303u,
                     (vb >> 6) & 0x03030303u, bf[sl * 2 + 1].x, bf[sl * 2 + 1].y);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (DUAL) acc0[e] = (sq[0][e] + sq[1][e]) + (sq[2][e] + sq[3][e]);
            else { acc0[e] = sq[0][e] + sq[1][e]; acc1[e] = sq[2][e] + sq[3][e]; }
          }
        }

        // finish the cells: columns (2c, 2c+1) are the high / low activation parts of one cell.
        // Every lane runs this code (lanes without a cell produce values that are never read).
        const int yi = kPlaneSets ? 0 : q;
        const uint32_t sa_addr = scol + q * dq_s, sb_addr = sa_addr + db_s;
        int da0, da1 = 0, db0, db1 = 0;   // exact group sums + kMagic
        if constexpr (DUAL) {
          da0 = 4 * acc0[0] + acc0[1] + ci0; db0 = 4 * acc0[2] + acc0[3] + ci0;
          const float sa = __half2float(__ushort_as_half(uint16_t(lds_u16(sa_addr))));
          const float sb = __half2float(__ushort_as_half(uint16_t(lds_u16(sb_addr))));
          ya[yi] = __fmaf_rn(__fsub_rn(__int_as_float(da0), 12582912.0f), sa, ya[yi]);
          yb[yi] = __fmaf_rn(__fsub_rn(__int_as_float(db0), 12582912.0f), sb, yb[yi]);
        } else {
          da0 = 4 * acc0[0] + acc0[1] + ci0; da1 = 4 * acc1[0] + acc1[1] + ci1;
          db0 = 4 * acc0[2] + acc0[3] + ci0; db1 = 4 * acc1[2] + acc1[3] + ci1;
          const uint32_t s2a = lds_u32(sa_addr), s2b = lds_u32(sb_addr);   // f16 scales [group 0 | group 1]
          ya[yi] = __fmaf_rn(__fsub_rn(__int_as_float(da0), 12582912.0f), __half2float(__ushort_as_half(uint16_t(s2a & 0xffffu))), ya[yi]);
          ya[yi] = __fmaf_rn(__fsub_rn(__int_as_float(da1), 12582912.0f), __half2float(__ushort_as_half(uint16_t(s2a >> 16))), ya[yi]);
          yb[yi] = __fmaf_rn(__fsub_rn(__int_as_float(db0), 12582912.0f), __half2float(__ushort_as_half(uint16_t(s2b & 0xffffu))), yb[yi]);
          yb[yi] = __fmaf_rn(__fsub_rn(__int_as_float(db1), 12582912.0f), __half2float(__ushort_as_half(uint16_t(s2b >> 16))), yb[yi]);
        }
        if (dump) {
          if (lane_has_cell && cell_token < p.m) {
            const uint32_t gblk = blockIdx.x + it * gridDim.x;
            const uint32_t row0 = (gblk % p.blocks) * p.rows_per_stage;
            // (row, plane) of the lane's first row-plane in set q; the second one is kHalfRows rows further
            const uint32_t na = kPlaneSets ? g : q * 2 * kHalfRows + lrow, nb = na + kHalfRows;
            const uint32_t pl = kPlaneSets ? uint32_t(q) : lplane;
            const uint32_t tok = p.dump_token_offset + cell_token;
            if (row0 + na < p.n) {
              int32_t* d = p.acc_dump + ((size_t(tok) * p.n + row0 + na) * groups_per_row + 2 * j + cell_group) * PLANES + pl;
              d[0] = da0 - kMagic;
              if (!DUAL) d[PLANES] = da1 - kMagic;
            }
            if (row0 + nb < p.n) {
              int32_t* d = p.acc_dump + ((size_t(tok) * p.n + row0 + nb) * groups_per_row + 2 * j + cell_group) * PLANES + pl;
              d[0] = db0 - kMagic;
              if (!DUAL) d[PLANES] = db1 - kMagic;
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);      // slot may be refilled

    // hand this warp's partial sums of the block to the combiner: [row-plane (three planes: row)][cell]
    if (part_round > 0 && !mbar_wait(&part_empty[buf], (part_round - 1) & 1, &abort_flag)) {
      abort_flag = 1;
      if (lane == 0 && atomicOr(&p.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { p.status[TBS_INFO0] = it; p.status[TBS_INFO1] = 400 + buf; }
      return;
    }
    float* my_part = part + (size_t(buf) * kWarps + warp) * kSliceFloats;
    if (lane_has_cell) {
#pragma unroll
      for (int q = 0; q < YN; ++q) {
        my_part[(q * 16 + g) * NC + c] = ya[q];
        my_part[(q * 16 + 8 + g) * NC + c] = yb[q];
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&part_full[buf]);
    if (++s == p.stages) { s = 0; full_parity ^= 1; }
    if (++buf == kPartBufs) { buf = 0; ++part_round; }
    if (++vw == kWarps) vw = 0;
  }
}

uint32_t round_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

// Byte layout of the activation tables (identical in global scratch and in shared memory).
struct TableLayout { uint32_t z_bytes, off_cinit, off_actscale, total; };
// Token columns the tables and the kernel are laid out for: three tokens run in the four-token kernel.
uint32_t layout_tokens(uint32_t m) { return m == 3 ? 4u : m; }
bool use_dual(uint32_t m) { return m <= 2; }
TableLayout table_layout(const tb_weights* w, uint32_t m_valid) {
  const uint32_t m = layout_tokens(m_valid);
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
  const uint32_t cw = kWarps;
  uint32_t off = 0;
  const uint32_t mk = layout_tokens(m), cells = use_dual(mk) ? 2 * mk : mk;
  // a consumer warp's partial sums per row block: one per row-plane (three planes: one per row)
  const uint32_t part = kPartBufs * cw * pl.rows_per_stage * (planes == 3 ? 1 : planes) * cells * 4;
  const uint32_t xq = kBuildStagingBytes;   // fused prologue staging
  const uint32_t fixed = tl.total + part + xq;
  const uint32_t per_stage = pl.stage_bytes + pl.scale_stage_bytes;
  if (fixed + 2 * per_stage > uint32_t(max_smem)) return 0;
  // Prefer a footprint that lets two CTAs share an SM (of this launch, or one of this launch and
  // one of the next launch on the stream, whose weight stream then starts under this launch's
  // tail).  Each CTA adds its static shared memory and 1 KB of reserved space to the 228 KB of an SM.
  const uint32_t half_sm = 110u * 1024u;
  uint32_t budget = uint32_t(max_smem), ctas = 1;
  if (fixed + 2 * per_stage <= half_sm) { budget = half_sm; ctas = 2; }
  uint32_t stages = std::min<uint32_t>(kMaxStages, (budget - fixed) / per_stage);
  if (p) {
    p->stages = stages;
    p->off_ring = off; off += stages * pl.stage_bytes;
    p->off_scale_ring = off; off += stages * pl.scale_stage_bytes;
    p->off_z = off;
    p->off_cinit = off + tl.off_cinit;
    p->off_actscale = off + tl.off_actscale;
    off += tl.total;
    p->off_part = off; off += part;
    p->off_xq = off; off += xq;
    p->table_bytes = tl.total;
    p->ctas_per_sm = ctas;
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
  // A row block is `sets` blocks of 16 row-planes: 16*sets/planes rows (1, 2 or 4 sets for one and
  // two planes, 3 sets = 16 rows for three), so that R % 4 == 0 (16-byte chunks).  Take the
  // largest block up to about 40 KB that still leaves every SM three blocks when the tensor allows it.
  const uint32_t target = 40 * 1024;
  uint32_t sets = planes == 3 ? 3 : 1;
  if (planes != 3)
    for (uint32_t cand : {2u, 4u}) {
      const uint32_t r = 16 * cand / planes;
      if (r * pl.row_bytes <= target && (w->n + r - 1) / r >= 444) sets = cand;
    }
  const uint32_t r = 16 * sets / planes;
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

bool tb_decode_builds_tables(const tb_weights* w, uint32_t m, const void* x) {
  // (tile column, token) pairs every CTA would have to quantise and lay out; measured on B200: up
  // to about a dozen pairs the single launch wins, beyond that the separate kernel
  const uint32_t pairs = uint32_t(w->k / 256) * layout_tokens(m);
  return pairs <= 12 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
}

cudaError_t tb_launch_prepare(const DecodeArgs& a, cudaStream_t stream) {
  const tb_weights* w = a.w;
  const TableLayout tl = table_layout(w, a.m);
  if (!a.scratch || a.scratch_bytes < tl.total) return cudaErrorInvalidValue;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  PrepareParams pp{};
  pp.x = a.x; pp.act_scale_in = a.act_scale_in; pp.act_absmax_in = a.act_absmax_in;
  if (a.relu2_up) {
    if (a.x_dtype != TB_F32) return cudaErrorInvalidValue;
    pp.relu2_up = a.relu2_up;
  }
  pp.tables = static_cast<uint8_t*>(a.scratch);
  pp.m = a.m; pp.mk = layout_tokens(a.m); pp.k = uint32_t(w->k); pp.tpr = uint32_t(w->k / 256); pp.x_dtype = uint32_t(a.x_dtype);
  pp.off_cinit = tl.off_cinit; pp.off_actscale = tl.off_actscale; pp.pdl = a.pdl ? 1u : 0u;
  pp.status = a.status;
  if (a.comm_absmax) pp.comm = *a.comm_absmax;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pp.tpr, a.m);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = a.pdl ? 1 : 0;
  const bool dual = use_dual(layout_tokens(a.m));
  if (w->codec == tbf::kB3)
    return dual ? cudaLaunchKernelEx(&cfg, prepare_kernel<tbf::kB3, true>, pp) : cudaLaunchKernelEx(&cfg, prepare_kernel<tbf::kB3, false>, pp);
  return dual ? cudaLaunchKernelEx(&cfg, prepare_kernel<tbf::kD2, true>, pp) : cudaLaunchKernelEx(&cfg, prepare_kernel<tbf::kD2, false>, pp);
}

using DecodeKernel = void (*)(const DecodeParams);
template <int CODEC, int PLANES, int SETS> DecodeKernel pick_tokens(uint32_t mk) {
  return mk == 1 ? decode_kernel<CODEC, PLANES, 1, SETS> : mk == 2 ? decode_kernel<CODEC, PLANES, 2, SETS> : decode_kernel<CODEC, PLANES, 4, SETS>;
}
template <int CODEC, int PLANES> DecodeKernel pick_sets(uint32_t sets, uint32_t mk) {
  return sets == 1 ? pick_tokens<CODEC, PLANES, 1>(mk) : sets == 2 ? pick_tokens<CODEC, PLANES, 2>(mk) : pick_tokens<CODEC, PLANES, 4>(mk);
}
template <int CODEC> DecodeKernel pick_planes(uint32_t planes, uint32_t sets, uint32_t mk) {
  return planes == 1 ? pick_sets<CODEC, 1>(sets, mk) : planes == 2 ? pick_sets<CODEC, 2>(sets, mk) : pick_tokens<CODEC, 3, 3>(mk);
}

cudaError_t tb_launch_decode(const DecodeArgs& a, int sm_count, int max_smem, cudaStream_t stream) {
  const tb_weights* w = a.w;
  DecodeParams p{};
  const size_t smem = layout(w, a.m, max_smem, &p);
  if (!smem) return cudaErrorInvalidConfiguration;
  const TableLayout tl = table_layout(w, a.m);
  if (a.fused) {
    // the prologue reads x with 16-byte loads
    if (!a.x || (reinterpret_cast<uintptr_t>(a.x) & 15u)) return cudaErrorInvalidValue;
    // a row shard that builds its own tables exchanges the absmax in the same launch, which needs the output slot's round
    if (a.comm_absmax && !a.comm_y) return cudaErrorInvalidValue;
    if (a.comm_y && a.comm_y->world > 1 && !a.comm_absmax && !a.act_absmax_in && a.x_dtype != TB_I8) return cudaErrorInvalidValue;
    if (a.x_dtype == TB_I8 && !a.act_scale_in) return cudaErrorInvalidValue;
    p.fused = 1; p.x = a.x; p.act_scale_in = a.act_scale_in; p.act_absmax_in = a.act_absmax_in; p.x_dtype = uint32_t(a.x_dtype);
    if (a.relu2_up) {
      if (a.x_dtype != TB_F32 || (reinterpret_cast<uintptr_t>(a.relu2_up) & 15u) || a.norm_weight) return cudaErrorInvalidValue;
      p.relu2_up = a.relu2_up;
    }
    if (a.norm_weight) {
      if (a.x_dtype == TB_I8 || (reinterpret_cast<uintptr_t>(a.norm_weight) & 15u)) return cudaErrorInvalidValue;
      p.norm_weight = a.norm_weight; p.norm_eps = a.norm_eps; p.norm_zero_centered = a.norm_zero_centered ? 1u : 0u;
    }
  } else if (!a.scratch || a.scratch_bytes < tl.total || a.norm_weight) {
    return cudaErrorInvalidValue;   // the norm prologue lives in the fused builder; other launches take normalised input
  }
  p.residual = a.residual;
  if (a.comm_y && a.comm_y->world > 1) {
    if (a.layers || a.layer_count > 1 || a.acc_dump) return cudaErrorInvalidValue;
    p.tp = 1; p.comm_y = *a.comm_y;
    if (a.fused && a.comm_absmax) p.comm_absmax = *a.comm_absmax;
  }
  cudaLaunchAttribute attr[2];
  unsigned num_attrs = 0;
  if (a.pdl) {
    attr[num_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[num_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++num_attrs;
  }
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
  p.inject_missing_tx = a.inject_missing_tx;
  const uint32_t sets = w->plan.rows_per_stage * w->uniform_planes / 16, mk = layout_tokens(a.m);
  DecodeKernel kernel = w->codec == tbf::kB3 ? pick_planes<tbf::kB3>(w->uniform_planes, sets, mk) : pick_planes<tbf::kD2>(w->uniform_planes, sets, mk);
  if (!kernel) return cudaErrorInvalidConfiguration;
  if (a.layers && a.layer_count > uint32_t(kMaxGroupLayers)) return cudaErrorInvalidValue;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (err != cudaSuccess) return err;
  cudaLaunchConfig_t cfg{};
  // A grouped launch keeps two CTAs per SM busy.  A single small layer keeps one, so that the next
  // launch on the stream can move in beside it; a layer with many row blocks per SM is better
  // served by two CTAs per SM of its own.
  const bool wide = a.layers != nullptr || p.blocks >= 2u * uint32_t(sm_count);
  const uint32_t resident = uint32_t(sm_count) * (wide ? p.ctas_per_sm : 1u);
  uint32_t grid = std::min<uint32_t>(p.blocks * p.layer_count, resident);
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = num_attrs;
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
  tb_clear_error();
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
  d.inject_missing_tx = backend->inject_missing_tx;   // test hook, one call only
  backend->inject_missing_tx = 0;
  // Nothing in the tables has to start at zero: the prepare kernel rewrites every entry the decode
  // kernel of the same call reads (z entries, start values, token scales) before it is read.
  err = tb_launch_prepare(d, st);
  if (err != cudaSuccess) return tb_cuda_fail(err, "launch prepare");
  err = tb_launch_decode(d, backend->prop.multiProcessorCount, backend->max_smem_optin, st);
  if (err != cudaSuccess) return tb_cuda_fail(err, "launch decode");
  return TB_OK;
}

