// Prefill GEMM (many tokens) from the packed B3 / D2 arenas on the tcgen05 INT8 tensor cores.
//
//   Y[m,n] = a[m] * sum over (tile column j, plane p, group g) of s[n,j,p,g] * I[m,n,j,p,g],
//   I = sum over the 128 trits of the group of t * q          (exact int32)
//
// One CTA owns a 128 (weight rows) x 2*HW (tokens) output tile, HW = 128 (64 for up to 128 tokens),
// and walks the K dimension in slabs of one (tile column, plane, scale group) = 128 trits:
//   * expander warps read each row's packed words, turn them into int8 operands (B3: a
//     half-precision-FMA chain gives the quotients floor(b / 3^i), one 32-bit multiply-add per
//     digit gives the four lanes' digits; no table, no division) and write the slab as a K-major,
//     128-byte-swizzled tile in shared memory (A operand, UMMA M = 128);
//   * a TMA warp loads the int8 activations of the tile column (B operand) from the scratch
//     written by the quantisation pre-pass, already in the expander's k-slot order, together with
//     the per-token start values of its two slabs;
//   * two MMA warps, one per half of the token tile, each issue four tcgen05.mma (kind::i8,
//     N = HW, K = 32 each) per slab into their TMEM accumulator.  The accumulator was pre-loaded by
//     the epilogue with 0x4B400000 - (sum of the slab's activations): operands are the unsigned
//     codes c = trit + 1, so after the MMAs the accumulator's BITS are the float 12582912 + I and
//     int -> float costs one FADD.  While one half is drained the tensor core works on the other;
//   * epilogue warps (one TMEM lane = one weight row per thread; a warp owns one half and a
//     column range of it) drain the accumulator, multiply by the row's f16 group scale, add into
//     fp32 running sums that also live in TMEM (packed two-lane FADD2 / FFMA2), store the next
//     slab's start values and hand the half back.
//
// TMEM columns: [0,HW) and [HW,2HW) accumulator halves, [2HW,4HW) fp32 running sums.
// All waits are bounded; a timeout sets TBF_WAIT_TIMEOUT and every role leaves its loop, the
// allocating warp frees TMEM, and the kernel returns.  No TMA multicast is used.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "tb_internal.h"

namespace {

constexpr int kRows = 128;        // weight rows per tile (UMMA M)
// Expanded slabs in flight.  With several expander groups working on consecutive tile-planes at
// once, a group's wait on a ring slot must never be more than one phase ahead of the slot's
// barrier: eight slots for three groups (six slabs in flight) keep it so.
__host__ __device__ constexpr int stages_a(int exp_groups) { return exp_groups > 1 ? 8 : 4; }
constexpr int kStagesB = 2;       // tile columns of activations in flight (two slabs each)
// Warps: 0 TMA, 1-2 MMA issue (1 owns TMEM), 3 idle, then EPI epilogue warps, then 4 x EXP expander
// warps (a group of four warps expands one 128-row slab).  Two configurations, both 768 threads:
//   many tokens (tiles of 128 or 256): EPI = 16 (two column parts per accumulator half and lane
//     quadrant: the drain bounds the kernel), EXP = 1;
//   few tokens (tiles of 32 or 64):    EPI = 8 (the drain is small), EXP = 3 (the kernel is bound by
//     how fast the weights can be expanded, which has to keep up with HBM).
constexpr int kFirstEpilogueWarp = 4, kGroupWarps = 4;
__host__ __device__ constexpr int threads_of(int epi, int exp_groups) { return 32 * (kFirstEpilogueWarp + epi + kGroupWarps * exp_groups); }
constexpr uint32_t kSpin = 1u << 22;
constexpr uint32_t kBarFull = 1, kBarEmpty = 3;                 // named barriers kBarFull + half, kBarEmpty + half
constexpr uint32_t kBarEpilogue = 5;                              // all epilogue warps (split-K combine)
constexpr long long kWaitCycles = 2000000000ll;
constexpr uint32_t kMagicBits = 0x4B400000u;   // float 12582912 = 2^23 + 2^22
constexpr uint32_t kTileABytes = kRows * 128;
constexpr uint32_t kMaxSplitTiles = 256;   // arrival counters the backend keeps for split output tiles

struct PrefillParams {
  const uint8_t* payload; const uint16_t* scales;
  const int8_t* qperm; const int32_t* qinit; const float* ascale;   // scratch from the pre-pass
  void* y; int32_t* acc_dump; const float* row_scale; const float* residual;
  uint32_t* status;
  uint32_t m, m_pad, n, k, tpr, y_dtype;
  uint32_t n_tiles, m_tiles;
  // Split K: `splits` CTAs share an output tile, each walks a range of tile columns and leaves its
  // fp32 running sums in `partial` [split][m_pad][n]; the last of them to finish (a counter per
  // tile) adds the parts in split order and finishes the outputs.  splits == 1: none of this.
  uint32_t splits;
  float* partial; uint32_t* tile_counters;
};

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t saddr(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t c) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(b)), "r"(c)); }
__device__ __forceinline__ void mbar_arrive(uint64_t* b) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(b)) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(saddr(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(saddr(b)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  After kWaitCycles SM clocks (about a second) it records TBF_WAIT_TIMEOUT and raises
// the CTA's abort flag; from then on NO wait in this CTA blocks any more: every role runs its
// loops to the end on whatever data is there (the host discards the result), so that all
// barrier arrivals still happen and the kernel ends.  `backoff_ns` > 0 sleeps between polls:
// roles that run ahead of the pipeline (copy producer, expanders) must not take issue slots from
// the warps that bound it.
struct WaitCtx { volatile uint32_t* abort_flag; uint32_t* status; };
__device__ __forceinline__ void mbar_wait(uint64_t* b, uint32_t parity, const WaitCtx& ctx, uint32_t where, uint32_t backoff_ns = 0) {
  if (mbar_try(b, parity) || *ctx.abort_flag) return;
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    if (backoff_ns) __nanosleep(backoff_ns);
    if (mbar_try(b, parity)) return;
    if ((i & 63u) == 63u) {
      if (*ctx.abort_flag) return;
      if (clock64() - t0 > kWaitCycles) {
        *ctx.abort_flag = 1;
        if (atomicOr(&ctx.status[TBS_FLAGS], TBF_WAIT_TIMEOUT) == 0) { ctx.status[TBS_INFO0] = parity; ctx.status[TBS_INFO1] = where; }
        return;
      }
    }
  }
}
// Named barriers hand an accumulator half back and forth between its MMA warp and its epilogue
// warps without polling: every participant makes the same number of calls whatever happens.
__device__ __forceinline__ void named_sync(uint32_t id, uint32_t count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void named_arrive(uint32_t id, uint32_t count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r; asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel)); return r;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(saddr(dst)), "l"(map), "r"(x), "r"(y), "r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(saddr(dst)), "l"(src), "r"(bytes), "r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], int8 operands, int32 accumulate.  The many-token kernel always
// accumulates (its epilogue pre-loads the accumulator); the few-token kernel overwrites with the
// first K step of a slab.
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate = 1u) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
#define TB_R16(a, o) "=r"(a[o+0]), "=r"(a[o+1]), "=r"(a[o+2]), "=r"(a[o+3]), "=r"(a[o+4]), "=r"(a[o+5]), "=r"(a[o+6]), "=r"(a[o+7]), \
                     "=r"(a[o+8]), "=r"(a[o+9]), "=r"(a[o+10]), "=r"(a[o+11]), "=r"(a[o+12]), "=r"(a[o+13]), "=r"(a[o+14]), "=r"(a[o+15])
#define TB_S16(a, o) "r"(a[o+0]), "r"(a[o+1]), "r"(a[o+2]), "r"(a[o+3]), "r"(a[o+4]), "r"(a[o+5]), "r"(a[o+6]), "r"(a[o+7]), \
                     "r"(a[o+8]), "r"(a[o+9]), "r"(a[o+10]), "r"(a[o+11]), "r"(a[o+12]), "r"(a[o+13]), "r"(a[o+14]), "r"(a[o+15])
// 32 lanes x 16 columns of 32 bits: this thread's lane, 16 consecutive columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : TB_R16(r, 0) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), TB_S16(r, 0) : "memory");
}
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_stn(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st16(taddr, r); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte swizzle, 8-row groups
// 1024 bytes apart; `k_chunk` selects the 32-byte K slice of one MMA inside the swizzled row.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t k_chunk) {
  uint64_t d = 0;
  d |= uint64_t(((addr + k_chunk * 32u) & 0x3ffffu) >> 4);   // start address
  d |= uint64_t(1) << 16;                                    // leading byte offset (unused for swizzled K-major)
  d |= uint64_t(1024 >> 4) << 32;                            // stride byte offset
  d |= uint64_t(1) << 46;                                    // descriptor version
  d |= uint64_t(2) << 61;                                    // SWIZZLE_128B
  return d;
}
// Instruction descriptor: s32 accumulate, A/B formats, K-major both, N, M.
__host__ __device__ constexpr uint32_t instr_desc_n(uint32_t n) {
  return (2u << 4)                    // s32 accumulator
         | (1u << 7) | (1u << 10)     // A and B are signed 8-bit
         | ((n >> 3) << 17) | ((uint32_t(kRows) >> 4) << 24);
}

// ---------------------------------------------------------------- k-slot order of a slab
// slot (0..127) of trit t (0..255 of the tile) inside its group's slab: packed words are expanded
// digit-major (quad = 5*word + digit, byte lane = byte of the word); the word that straddles the
// group boundary (bytes 24..27) and the last word (bytes 48..51, four padding digits) are laid
// out in natural trit order.
__host__ __device__ inline uint32_t b3_slot(uint32_t t) {
  if (t < 120) { const uint32_t w = t / 20, r = t % 20; return 4 * (5 * w + r % 5) + r / 5; }
  if (t < 128) return t;
  if (t < 140) return t - 128;
  if (t < 240) { const uint32_t w = t / 20, r = t % 20; return 4 * (3 + 5 * (w - 7) + r % 5) + r / 5; }
  return 112 + (t - 240);
}
__host__ __device__ inline uint32_t d2_slot(uint32_t t) {
  const uint32_t u = t & 127, w = u >> 4, e = (u & 15) >> 2, s = u & 3;
  return 4 * (4 * w + s) + e;
}

// ---------------------------------------------------------------- quantisation pre-pass
struct QuantParams {
  const void* x; const float* act_scale_in; const float* act_absmax_in;
  const float* relu2_up;   // squared-ReLU gate (x fp32): activation = (max(x, 0)^2) * relu2_up; null = none
  int8_t* qperm; int32_t* qinit; float* ascale;
  uint32_t m, m_pad, k, x_dtype, codec;
  uint32_t* status;
};

__global__ void __launch_bounds__(256) prefill_quant_kernel(const QuantParams p) {
  __shared__ float red[8];
  // The tensor-core kernel behind this one may start now: its expanders do not depend on the
  // activations, only its copy warp waits (griddepcontrol.wait) for this grid to complete.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t slabs = p.k / 128;
  int8_t* qrow = p.qperm + size_t(t) * p.k;
  if (t >= p.m) {   // padding tokens: zero codes, neutral start values
    for (uint32_t i = tid; i < p.k; i += 256) qrow[i] = 0;
    for (uint32_t s = tid; s < slabs; s += 256) p.qinit[size_t(s) * p.m_pad + t] = int(kMagicBits);
    if (tid == 0) p.ascale[t] = 0.f;
    return;
  }
  float scale_q = 0.f;
  if (p.x_dtype != TB_I8) {
    float gamma;
    if (p.act_absmax_in) gamma = p.act_absmax_in[t];
    else {
      float mx = 0.f;
      for (uint32_t i = tid; i < p.k; i += 256) {
        float v = p.x_dtype == TB_F32 ? static_cast<const float*>(p.x)[size_t(t) * p.k + i]
                                      : __bfloat162float(static_cast<const __nv_bfloat16*>(p.x)[size_t(t) * p.k + i]);
        if (p.relu2_up) { const float r = fmaxf(v, 0.0f); v = __fmul_rn(__fmul_rn(r, r), p.relu2_up[size_t(t) * p.k + i]); }
        mx = fmaxf(mx, fabsf(v));
      }
      for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) red[warp] = mx;
      __syncthreads();
      gamma = 0.f;
      for (int w = 0; w < 8; ++w) gamma = fmaxf(gamma, red[w]);
    }
    scale_q = gamma > 0.f ? __fdiv_rn(127.0f, gamma) : 0.f;
    if (tid == 0) p.ascale[t] = __fdiv_rn(gamma, 127.0f);
  } else if (tid == 0) {
    p.ascale[t] = p.act_scale_in[t];
  }
  // one warp per 128-trit group: quantise, scatter into slot order, sum
  for (uint32_t grp = warp; grp < slabs; grp += 8) {
    int sum = 0;
    for (uint32_t e = 0; e < 4; ++e) {
      const uint32_t u = lane * 4 + e, i = grp * 128 + u, tt = (grp & 1) * 128 + u;   // tt: trit index in its tile
      int q;
      if (p.x_dtype == TB_I8) q = static_cast<const int8_t*>(p.x)[size_t(t) * p.k + i];
      else {
        float v = p.x_dtype == TB_F32 ? static_cast<const float*>(p.x)[size_t(t) * p.k + i]
                                      : __bfloat162float(static_cast<const __nv_bfloat16*>(p.x)[size_t(t) * p.k + i]);
        if (p.relu2_up) { const float r = fmaxf(v, 0.0f); v = __fmul_rn(__fmul_rn(r, r), p.relu2_up[size_t(t) * p.k + i]); }
        // a NaN would clamp to a finite code: report non-finite activations instead
        if (!(fabsf(v) <= 3.402823466e+38f) && atomicOr(&p.status[TBS_FLAGS], TBF_NONFINITE_ACT) == 0) {
          p.status[TBS_INFO0] = t * p.k + i; p.status[TBS_INFO1] = __float_as_uint(v);
        }
        q = int(fminf(127.f, fmaxf(-128.f, rintf(__fmul_rn(v, scale_q)))));
      }
      sum += q;
      qrow[grp * 128 + (p.codec == tbf::kB3 ? b3_slot(tt) : d2_slot(tt))] = int8_t(q);
    }
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) p.qinit[size_t(grp) * p.m_pad + t] = int(kMagicBits) - sum;
  }
}

// ---------------------------------------------------------------- weight expansion
// B3 word (four bytes) -> five registers of operand bytes: digit i (0..2, i.e. trit + 1) of bytes
// 0..3 in byte lanes 0..3.  The quotients q_i = floor(b / 3^i) come from a half-precision FMA
// chain on 1024 + b (exact: every intermediate is an integer below 2048); packed as bytes,
// d_i = q_i - 3 q_(i+1) is one 32-bit multiply-add for all four lanes (no lane ever borrows).
__device__ __forceinline__ void b3_digits(uint32_t w, uint32_t (&r)[5]) {
  constexpr uint32_t c1 = 0x35533553u, k1 = 0x61566156u;   // 1024+v -> 1024+floor(v/3), v <= 242
  constexpr uint32_t c2 = 0x354d354du, k2 = 0x61596159u;   // v <= 80
  constexpr uint32_t c3 = 0x354b354bu, k3 = 0x615a615au;   // v <= 26
  const uint32_t h01 = prmt(w, 0x64646464u, 0x4140u), h23 = prmt(w, 0x64646464u, 0x4342u);
  const uint32_t a1 = hfma2(h01, c1, k1), b1 = hfma2(h23, c1, k1);
  const uint32_t a2 = hfma2(a1, c2, k2), b2 = hfma2(b1, c2, k2);
  const uint32_t a3 = hfma2(a2, c3, k3), b3 = hfma2(b2, c3, k3);
  const uint32_t a4 = hfma2(a3, c3, k3), b4 = hfma2(b3, c3, k3);
  const uint32_t q1 = prmt(a1, b1, 0x6420u), q2 = prmt(a2, b2, 0x6420u), q3 = prmt(a3, b3, 0x6420u), q4 = prmt(a4, b4, 0x6420u);
  r[0] = w - 3u * q1;
  r[1] = q1 - 3u * q2;
  r[2] = q2 - 3u * q3;
  r[3] = q3 - 3u * q4;
  r[4] = q4;
}
// (a.byte[ea], b.byte[eb], c.byte[ec], d.byte[ed])
__device__ __forceinline__ uint32_t pack4(uint32_t a, uint32_t ea, uint32_t b, uint32_t eb, uint32_t c, uint32_t ec, uint32_t d, uint32_t ed) {
  return prmt(prmt(a, b, ea | ((4u + eb) << 4)), prmt(c, d, ec | ((4u + ed) << 4)), 0x5410u);
}
// natural-order trit quad number `nq` of a word whose digit registers are r[0..4]: trits 4nq..4nq+3
// of the sequence T[5*byte + digit]
__device__ __forceinline__ uint32_t natural_quad(const uint32_t (&r)[5], int nq) {
  const int t0 = 4 * nq;
  return pack4(r[t0 % 5], t0 / 5, r[(t0 + 1) % 5], (t0 + 1) / 5, r[(t0 + 2) % 5], (t0 + 2) / 5, r[(t0 + 3) % 5], (t0 + 3) / 5);
}
// store 16 bytes = quads 4*chunk .. 4*chunk+3 of row `row` into a swizzled K-major tile
__device__ __forceinline__ void store_chunk(uint8_t* tile, uint32_t row, uint32_t chunk, uint32_t q0, uint32_t q1, uint32_t q2, uint32_t q3) {
  *reinterpret_cast<uint4*>(tile + row * 128u + ((chunk ^ (row & 7u)) << 4)) = make_uint4(q0, q1, q2, q3);
}

// y{0,1} += (as_float(d{0,1}) - 12582912) * s, two lanes per instruction
__device__ __forceinline__ void scale_add2(uint32_t d0, uint32_t d1, float2 neg_magic, float2 scale, uint32_t& y0, uint32_t& y1) {
  const float2 d = __fadd2_rn(make_float2(__uint_as_float(d0), __uint_as_float(d1)), neg_magic);
  const float2 y = __ffma2_rn(d, scale, make_float2(__uint_as_float(y0), __uint_as_float(y1)));
  y0 = __float_as_uint(y.x); y1 = __float_as_uint(y.y);
}
__device__ __forceinline__ void lds128(uint32_t addr, uint32_t* v) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
}

// work item = (row tile, token tile, K split); a split walks tile columns [j0, j1)
__device__ __forceinline__ void split_range(const PrefillParams& p, uint32_t tile, uint32_t& j0, uint32_t& j1) {
  const uint32_t sp = tile % p.splits;
  j0 = uint32_t(uint64_t(p.tpr) * sp / p.splits);
  j1 = uint32_t(uint64_t(p.tpr) * (sp + 1) / p.splits);
}

// ---------------------------------------------------------------- roles shared by the two kernels
// Copy warp: the int8 activations of a tile column (two slabs of TILE_TOKENS x 128 bytes) and the
// per-token start values of its two slabs, into a ring of STAGES_B columns.
template <uint32_t TILE_TOKENS, int STAGES_B>
__device__ __forceinline__ void tma_role(const PrefillParams& p, const CUtensorMap& map_q, uint32_t tiles, uint8_t* tile_b, int32_t* qinit_s,
                                         uint64_t* b_full, uint64_t* b_empty, const WaitCtx& wctx, uint32_t lane) {
  constexpr uint32_t kTileTokens = TILE_TOKENS, kTileBBytes = TILE_TOKENS * 128;
  constexpr int kStagesB = STAGES_B;
  // launched with programmatic stream serialisation: everything this warp loads was written by
  // the quantisation pre-pass, the previous grid on the stream
  asm volatile("griddepcontrol.wait;" ::: "memory");
    // ------------------------------------------------ TMA: activations + start values of a tile column
    if (lane == 0) {
      uint32_t fill = 0;
      for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const uint32_t mt = (tile / p.splits) % p.m_tiles;
        uint32_t j0, j1;
        split_range(p, tile, j0, j1);
        for (uint32_t j = j0; j < j1; ++j, ++fill) {
          const uint32_t s = fill % kStagesB, round = fill / kStagesB;
          if (round > 0) mbar_wait(&b_empty[s], (round - 1) & 1, wctx, 300, 400);
          mbar_expect_tx(&b_full[s], 2 * kTileBBytes + 2 * kTileTokens * 4);
          for (int gsel = 0; gsel < 2; ++gsel) {
            tma_load_2d(tile_b + (s * 2 + gsel) * kTileBBytes, &map_q, int((2 * j + gsel) * 128), int(mt * kTileTokens), &b_full[s]);
            bulk_g2s(qinit_s + (s * 2 + gsel) * kTileTokens, p.qinit + size_t(2 * j + gsel) * p.m_pad + mt * kTileTokens,
                     kTileTokens * 4, &b_full[s]);
          }
        }
      }
      // copies in flight must land before the CTA's shared memory goes away
      for (uint32_t back = 0; back < kStagesB && back < fill; ++back) {
        const uint32_t f = fill - 1 - back;
        for (uint32_t i = 0; i < kSpin && !mbar_try(&b_full[f % kStagesB], (f / kStagesB) & 1); ++i) {}
      }
    }
}

// Expander warps (groups of four: one lane per weight row of the 128-row slab).
template <int CODEC, int PLANES, int EXP, int STAGES_A>
__device__ __forceinline__ void expander_role(const PrefillParams& p, uint32_t tiles, uint32_t wexp_all, uint32_t lane, uint8_t* tile_a,
                                              uint32_t* stage_s, uint64_t* a_full, uint64_t* a_empty, const WaitCtx& wctx) {
  constexpr int kStagesA = STAGES_A;
  constexpr uint32_t kPlaneBytes = CODEC == tbf::kB3 ? 52 : 64;
    // ------------------------------------------------ expanders: one weight row per thread
    // Rows are 1.5 KB apart in the arena, so a lane that fetched its own row word by word would
    // touch one sector per load.  Instead the warp fetches its 32 rows' words of a tile-plane as a
    // flattened (row, word) sequence -- consecutive lanes read consecutive words -- parks them in a
    // per-warp staging area, and every lane picks up its own row from there (stride kWords words:
    // odd for B3, conflict-free).  The next tile-plane's words are requested before the current
    // one is expanded.
    // With EXP > 1 groups, group g expands the tile-planes whose running number is g modulo EXP:
    // consecutive slabs are then built by different groups at the same time, and the MMA warps
    // still consume them in order from the ring.
    constexpr uint32_t kWords = kPlaneBytes / 4;
    const uint32_t grp = wexp_all / kGroupWarps, wexp = wexp_all % kGroupWarps;
    const uint32_t r = wexp * 32 + lane;
    uint32_t* stage = stage_s + wexp_all * 32 * kWords;
    const uint32_t row_stride = p.tpr * PLANES * kWords;   // words per weight row
    uint32_t tp_seq = 0;                                   // tile-planes handed to the ring so far (all groups count alike)
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      const uint32_t nt = tile / (p.m_tiles * p.splits);
      uint32_t j0, j1;
      split_range(p, tile, j0, j1);
      const uint32_t count = (j1 - j0) * PLANES, tp0 = j0 * PLANES;   // this item's tile-planes: tp0 .. tp0 + count - 1 of the row
      const uint32_t first = (grp + EXP - tp_seq % EXP) % EXP;        // the group's first one among them
      const uint32_t* tile_words = reinterpret_cast<const uint32_t*>(p.payload);
      const uint32_t row0 = nt * kRows + wexp * 32;
      // One load instruction brings the words of kRowsPerIt whole rows (lane -> (row, word) is fixed,
      // so the address of iteration `it` is a lane constant plus it x a launch constant; lanes past
      // the last whole row idle: 26 of 32 for B3, all for D2).
      constexpr uint32_t kRowsPerIt = 32 / kWords, kLanesUsed = kRowsPerIt * kWords, kIts = 32 / kRowsPerIt;
      const uint32_t lrow = lane / kWords, lwd = lane - lrow * kWords;
      const bool lane_used = lane < kLanesUsed;
      const bool whole = row0 + 31 < p.n;   // otherwise rows past the end repeat the last row; never stored
      const uint32_t* lane_words = tile_words + size_t(min(row0 + lrow, p.n - 1)) * row_stride + lwd;
      uint32_t pf[kIts];
      auto fetch = [&](uint32_t tp) {
#pragma unroll
        for (uint32_t it = 0; it < kIts; ++it) {
          if (!lane_used) continue;
          const uint32_t* at = whole ? lane_words + size_t(it * kRowsPerIt) * row_stride
                                     : tile_words + size_t(min(row0 + it * kRowsPerIt + lrow, p.n - 1)) * row_stride + lwd;
          pf[it] = __ldg(at + tp * kWords);
        }
      };
      if (EXP > 1 && grp == 0) {
        // Few-token kernel: the expansion is bound by how fast the words arrive.  Ask for this item's
        // whole share of the lane's row (contiguous in the arena) to be brought into L2 now, so that
        // the loads below meet L2 latency, not HBM latency.
        const uint32_t n = min(row0 + lane, p.n - 1);
        const uint8_t* from = reinterpret_cast<const uint8_t*>(tile_words + size_t(n) * row_stride + tp0 * kWords);
        const uint32_t bytes = count * kWords * 4;
        for (uint32_t off = 0; off < bytes + 127; off += 128)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(from + min(off, bytes - 4)));
      }
      if (first < count) fetch(tp0 + first);
      {
        for (uint32_t i = first; i < count; i += EXP) {
          const uint32_t slab = 2 * (tp_seq + i);
          uint32_t w[kWords];
#pragma unroll
          for (uint32_t it = 0; it < kIts; ++it)
            if (lane_used) stage[it * kLanesUsed + lane] = pf[it];
          __syncwarp();
          if (i + EXP < count) fetch(tp0 + i + EXP);
#pragma unroll
          for (uint32_t i = 0; i < kWords; ++i) w[i] = stage[lane * kWords + i];
          __syncwarp();
          const uint32_t s0 = slab % kStagesA, s1 = (slab + 1) % kStagesA;
          if (slab >= kStagesA) mbar_wait(&a_empty[s0], ((slab / kStagesA) - 1) & 1, wctx, 302, 100);
          uint8_t* t0 = tile_a + s0 * kTileABytes;
          if (CODEC == tbf::kB3) {
            uint32_t d[5], e[5], f[5], g2[5];
            // group 0: words 0..5 digit-major (quads 0..29), then trits 120..127 in natural order
            b3_digits(w[0], d); b3_digits(w[1], e); b3_digits(w[2], f); b3_digits(w[3], g2);
            store_chunk(t0, r, 0, d[0], d[1], d[2], d[3]);
            store_chunk(t0, r, 1, d[4], e[0], e[1], e[2]);
            store_chunk(t0, r, 2, e[3], e[4], f[0], f[1]);
            store_chunk(t0, r, 3, f[2], f[3], f[4], g2[0]);
            b3_digits(w[4], d); b3_digits(w[5], e); b3_digits(w[6], f);
            store_chunk(t0, r, 4, g2[1], g2[2], g2[3], g2[4]);
            store_chunk(t0, r, 5, d[0], d[1], d[2], d[3]);
            store_chunk(t0, r, 6, d[4], e[0], e[1], e[2]);
            store_chunk(t0, r, 7, e[3], e[4], natural_quad(f, 0), natural_quad(f, 1));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_full[s0]);
            if (slab + 1 >= kStagesA) mbar_wait(&a_empty[s1], (((slab + 1) / kStagesA) - 1) & 1, wctx, 302, 100);
            uint8_t* t1 = tile_a + s1 * kTileABytes;
            // group 1: trits 128..139 in natural order (quads 0..2), words 7..11, trits 240..255
            b3_digits(w[7], d); b3_digits(w[8], e);
            store_chunk(t1, r, 0, natural_quad(f, 2), natural_quad(f, 3), natural_quad(f, 4), d[0]);
            store_chunk(t1, r, 1, d[1], d[2], d[3], d[4]);
            b3_digits(w[9], f); b3_digits(w[10], g2);
            store_chunk(t1, r, 2, e[0], e[1], e[2], e[3]);
            store_chunk(t1, r, 3, e[4], f[0], f[1], f[2]);
            store_chunk(t1, r, 4, f[3], f[4], g2[0], g2[1]);
            b3_digits(w[11], d); b3_digits(w[12], e);
            store_chunk(t1, r, 5, g2[2], g2[3], g2[4], d[0]);
            store_chunk(t1, r, 6, d[1], d[2], d[3], d[4]);
            store_chunk(t1, r, 7, natural_quad(e, 0), natural_quad(e, 1), natural_quad(e, 2), natural_quad(e, 3));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_full[s1]);
          } else {
            // D2: word i of the tile-plane holds trits 16i..16i+15; quad (4w + s) = slot s of its bytes
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) {
              const uint32_t v = w[c];
              store_chunk(t0, r, c, v & 0x03030303u, (v >> 2) & 0x03030303u, (v >> 4) & 0x03030303u, (v >> 6) & 0x03030303u);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_full[s0]);
            if (slab + 1 >= kStagesA) mbar_wait(&a_empty[s1], (((slab + 1) / kStagesA) - 1) & 1, wctx, 302, 100);
            uint8_t* t1 = tile_a + s1 * kTileABytes;
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) {
              const uint32_t v = w[8 + c];
              store_chunk(t1, r, c, v & 0x03030303u, (v >> 2) & 0x03030303u, (v >> 4) & 0x03030303u, (v >> 6) & 0x03030303u);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_full[s1]);
          }
        }
      }
      tp_seq += count;
    }
}

// HW = tokens per accumulator half (64 or 128); a CTA tile is 128 weight rows x 2*HW tokens.
template <int CODEC, int PLANES, int HW, bool DUMP, int EPI, int EXP>
__global__ void __launch_bounds__(threads_of(EPI, EXP), 1) prefill_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap map_q) {
  constexpr int kStagesA = stages_a(EXP);
  constexpr int kEpilogueWarps = EPI, kFirstExpandWarp = kFirstEpilogueWarp + EPI;
  constexpr uint32_t kHandoffThreads = 32 + 32 * EPI / 2;      // one MMA warp + the epilogue warps of its half
  constexpr uint32_t kTileTokens = 2 * HW;
  constexpr uint32_t kTileBBytes = kTileTokens * 128;          // one slab of activations
  constexpr uint32_t kParts = kEpilogueWarps / 8;              // epilogue warps per (half, lane quadrant)
  constexpr uint32_t kCW = HW / kParts;                        // columns per epilogue thread
  constexpr int kChunk = 16;
  static_assert(kCW % kChunk == 0, "an epilogue thread drains whole 16-column chunks");
  constexpr uint32_t kSlabsPerCol = 2 * PLANES;
  constexpr uint32_t kIdesc = instr_desc_n(HW);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tile_a = smem;                                       // kStagesA * 16 KB
  uint8_t* tile_b = tile_a + kStagesA * kTileABytes;            // kStagesB * 2 slabs
  int32_t* qinit_s = reinterpret_cast<int32_t*>(tile_b + kStagesB * 2 * kTileBBytes);   // kStagesB * 2 * kTileTokens
  uint32_t* stage_s = reinterpret_cast<uint32_t*>(qinit_s + kStagesB * 2 * kTileTokens);   // kExpandWarps * 32 rows * 16 words
  __shared__ uint64_t a_full[kStagesA], a_empty[kStagesA], b_full[kStagesB], b_empty[kStagesB], acc_full[2];
  __shared__ uint32_t tmem_base_s, abort_flag, combine_flag;

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStagesA; ++s) { mbar_init(&a_full[s], kGroupWarps); mbar_init(&a_empty[s], 2); }
    for (int s = 0; s < kStagesB; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 2 + kEpilogueWarps); }
    for (int s = 0; s < 2; ++s) mbar_init(&acc_full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_base_s)), "r"(4u * HW) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  // work item = (row tile, token tile, K split); a split walks tile columns [j0, j1)
  const uint32_t tiles = p.n_tiles * p.m_tiles * p.splits;

  const WaitCtx wctx{&abort_flag, p.status};
  if (warp == 0) {
    tma_role<kTileTokens, kStagesB>(p, map_q, tiles, tile_b, qinit_s, b_full, b_empty, wctx, lane);
  } else if (warp == 1 || warp == 2) {
    // ------------------------------------------------ MMA issuers, one warp per accumulator half (issuing a
    // tcgen05.mma keeps the thread busy for about as long as the MMA runs, so one thread cannot
    // keep the tensor core fed and also do the waiting); the whole warp walks the loop (so
    // that addresses and descriptors stay in uniform registers); one elected lane issues
    const uint32_t h = warp - 1;
    uint32_t slab = 0, colfill = 0;
    const uint64_t a_desc0 = smem_desc(saddr(tile_a), 0), b_desc0 = smem_desc(saddr(tile_b), 0);
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      uint32_t j0, j1;
      split_range(p, tile, j0, j1);
      for (uint32_t j = j0; j < j1; ++j, ++colfill) {
        const uint32_t sb = colfill % kStagesB;
        mbar_wait(&b_full[sb], (colfill / kStagesB) & 1, wctx, 301);
        for (uint32_t q = 0; q < kSlabsPerCol; ++q, ++slab) {
          const uint32_t sa = slab % kStagesA, gsel = q & 1;
          mbar_wait(&a_full[sa], (slab / kStagesA) & 1, wctx, 301);
          // descriptor start addresses are in 16-byte units
          const uint64_t a_desc = a_desc0 + uint64_t(sa * (kTileABytes >> 4));
          const uint64_t b_desc = b_desc0 + uint64_t((sb * 2 + gsel) * (kTileBBytes >> 4)) + uint64_t(h * (HW * 128u >> 4));
          named_sync(kBarEmpty + h, kHandoffThreads);   // the epilogue has stored the start values
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (uint32_t kc = 0; kc < 4; ++kc) tc_mma_i8(tmem_base + h * HW, a_desc + 2 * kc, b_desc + 2 * kc, kIdesc);
            tc_commit(&acc_full[h]);
            tc_commit(&a_empty[sa]);
          }
          __syncwarp();
          mbar_wait(&acc_full[h], slab & 1, wctx, 301);
          tc_fence_before();
          named_arrive(kBarFull + h, kHandoffThreads);
        }
        if (elect_one()) tc_commit(&b_empty[sb]);
        __syncwarp();
      }
    }
  } else if (warp >= kFirstExpandWarp) {
    expander_role<CODEC, PLANES, EXP, kStagesA>(p, tiles, warp - kFirstExpandWarp, lane, tile_a, stage_s, a_full, a_empty, wctx);
  } else if (warp >= kFirstEpilogueWarp) {
    // ------------------------------------------------ epilogue: TMEM lane = weight row; a warp owns one
    // accumulator half, one lane quadrant and a column range of it
    const uint32_t quad = warp & 3, sub = (warp - kFirstEpilogueWarp) >> 2, wh = sub & 1, part = sub >> 1, r = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((quad * 32u) << 16) + part * kCW;
    uint32_t slab = 0, colfill = 0;
    // start values of slab 0 (first tile column, group 0) for both halves
    {
      mbar_wait(&b_full[0], 0, wctx, 303);
      {
        const uint32_t h = wh;
        const uint32_t qi = saddr(qinit_s + h * HW + part * kCW);
#pragma unroll 1
        for (uint32_t c = 0; c < kCW; c += kChunk) {
          uint32_t v[kChunk];
#pragma unroll
          for (int i = 0; i < kChunk; i += 4) lds128(qi + (c + i) * 4u, &v[i]);
          tmem_stn(lane_addr + h * HW + c, v);
#pragma unroll
          for (int i = 0; i < kChunk; ++i) v[i] = 0u;
          tmem_stn(lane_addr + (2 + h) * HW + c, v);       // running sums start at zero
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        named_arrive(kBarEmpty + h, kHandoffThreads);
      }
    }
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      const uint32_t sp = tile % p.splits, out_tile = tile / p.splits, nt = out_tile / p.m_tiles, mt = out_tile % p.m_tiles;
      uint32_t j0, j1;
      split_range(p, tile, j0, j1);
      const uint32_t n = nt * kRows + r;
      const uint32_t nc = min(n, p.n - 1);
      const uint16_t* srow = p.scales + size_t(nc) * p.tpr * PLANES * 2;
      const bool more_tiles = tile + gridDim.x < tiles;
      // the row's group scales of a tile column (two f16 per plane) are fetched one column ahead,
      // so that no slab's drain waits for a load
      const uint32_t* srow2 = reinterpret_cast<const uint32_t*>(srow);
      uint32_t sc_next[PLANES];
#pragma unroll
      for (int pl2 = 0; pl2 < PLANES; ++pl2) sc_next[pl2] = __ldg(srow2 + j0 * PLANES + pl2);
      for (uint32_t j = j0; j < j1; ++j, ++colfill) {
        const uint32_t sb = colfill % kStagesB;
        uint32_t sc[PLANES];
#pragma unroll
        for (int pl2 = 0; pl2 < PLANES; ++pl2) {
          sc[pl2] = sc_next[pl2];
          if (j + 1 < j1) sc_next[pl2] = __ldg(srow2 + (j + 1) * PLANES + pl2);
        }
#pragma unroll
        for (uint32_t q = 0; q < kSlabsPerCol; ++q, ++slab) {
          const uint32_t gsel = q & 1, pl = q >> 1;
          const float sv = __half2float(__ushort_as_half(uint16_t(gsel ? sc[pl] >> 16 : sc[pl] & 0xffffu)));
          const float2 scale2 = make_float2(sv, sv), neg_magic2 = make_float2(-12582912.0f, -12582912.0f);
          const bool last = (j + 1 == j1 && q + 1 == kSlabsPerCol);
          // where the next slab's start values are
          const bool next_col = q + 1 == kSlabsPerCol;
          const bool has_next = !(last && !more_tiles);
          const uint32_t ncol = next_col ? colfill + 1 : colfill;
          if (has_next && next_col) mbar_wait(&b_full[ncol % kStagesB], (ncol / kStagesB) & 1, wctx, 303);
          const uint32_t qnext = saddr(qinit_s + ((ncol % kStagesB) * 2 + (next_col ? 0u : (q + 1) & 1u)) * kTileTokens + part * kCW);
          {
            const uint32_t h = wh;
            named_sync(kBarFull + h, kHandoffThreads);   // the MMA warp saw this half's MMAs complete
            tc_fence_after();
            const uint32_t d_addr = lane_addr + h * HW, y_addr = lane_addr + (2 + h) * HW;
            const uint32_t tok0 = mt * kTileTokens + h * HW + part * kCW;
#pragma unroll 1
            for (uint32_t c = 0; c < kCW; c += kChunk) {
              uint32_t dv[kChunk], yv[kChunk];
              tmem_ldn(d_addr + c, dv);
              tmem_ldn(y_addr + c, yv);      // zero at the first slab of a tile (see below)
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < kChunk; i += 2) scale_add2(dv[i], dv[i + 1], neg_magic2, scale2, yv[i], yv[i + 1]);
              if (DUMP) {
                if (n < p.n) {
#pragma unroll
                  for (int i = 0; i < kChunk; ++i) {
                    const uint32_t mtok = tok0 + c + i;
                    if (mtok < p.m)
                      p.acc_dump[((size_t(mtok) * p.n + n) * (p.tpr * 2) + 2 * j + gsel) * PLANES + pl] = int(dv[i]) - int(kMagicBits);
                  }
                }
              }
              if (has_next) {
#pragma unroll
                for (int i = 0; i < kChunk; i += 4) lds128(qnext + (h * HW + c + i) * 4u, &dv[i]);
                tmem_stn(d_addr + c, dv);
              }
              if (!last) tmem_stn(y_addr + c, yv);
              else {
                if (p.splits > 1) {
                  // this split's running sums; the last split of the tile to finish adds them up
                  if (n < p.n) {
#pragma unroll
                    for (int i = 0; i < kChunk; ++i) {
                      const uint32_t mtok = tok0 + c + i;
                      if (mtok < p.m) p.partial[(size_t(sp) * p.m_pad + mtok) * p.n + n] = __uint_as_float(yv[i]);
                    }
                  }
                } else if (n < p.n) {
                  const float rs = p.row_scale ? p.row_scale[n] : 1.0f;
#pragma unroll
                  for (int i = 0; i < kChunk; ++i) {
                    const uint32_t mtok = tok0 + c + i;
                    if (mtok < p.m) {
                      float out = __fmul_rn(__uint_as_float(yv[i]), __ldg(p.ascale + mtok));
                      if (p.row_scale) out = __fmul_rn(out, rs);
                      const size_t idx = size_t(mtok) * p.n + n;
                      if (p.residual) out = __fadd_rn(__ldg(p.residual + idx), out);
                      if (p.y_dtype == TB_F32) static_cast<float*>(p.y)[idx] = out;
                      else static_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(out);
                    }
                  }
                }
                // the next tile starts from zero running sums
#pragma unroll
                for (int i = 0; i < kChunk; ++i) yv[i] = 0u;
                tmem_stn(y_addr + c, yv);
              }
            }
            tmem_wait_st();
            tc_fence_before();
            if (has_next) named_arrive(kBarEmpty + h, kHandoffThreads);
          }
          // the column's start values and activations are no longer needed by this warp
          if (lane == 0 && next_col) mbar_arrive(&b_empty[sb]);
          if (last && p.splits > 1) {
            // Split K: count this split in; whoever completes the count adds the splits' sums in
            // split order (every run gives the same bits) and finishes the tile's outputs.
            __threadfence();
            named_sync(kBarEpilogue, 32 * EPI);
            if (warp == kFirstEpilogueWarp && lane == 0) {
              const uint32_t arrived = atomicAdd(p.tile_counters + out_tile, 1u);
              combine_flag = arrived == p.splits - 1 ? 1u : 0u;
              if (combine_flag) p.tile_counters[out_tile] = 0u;   // ready for the next launch
            }
            named_sync(kBarEpilogue, 32 * EPI);
            if (combine_flag && n < p.n) {
              __threadfence();
              const float rs = p.row_scale ? p.row_scale[n] : 1.0f;
              const uint32_t tok0 = mt * kTileTokens + wh * HW + part * kCW;
              for (uint32_t c = 0; c < kCW; ++c) {
                const uint32_t mtok = tok0 + c;
                if (mtok >= p.m) break;
                float sum = __ldcg(p.partial + size_t(mtok) * p.n + n);
                for (uint32_t s2 = 1; s2 < p.splits; ++s2) sum = __fadd_rn(sum, __ldcg(p.partial + (size_t(s2) * p.m_pad + mtok) * p.n + n));
                float out = __fmul_rn(sum, __ldg(p.ascale + mtok));
                if (p.row_scale) out = __fmul_rn(out, rs);
                const size_t idx = size_t(mtok) * p.n + n;
                if (p.residual) out = __fadd_rn(__ldg(p.residual + idx), out);
                if (p.y_dtype == TB_F32) static_cast<float*>(p.y)[idx] = out;
                else static_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(out);
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(4u * HW) : "memory");
}

// ---------------------------------------------------------------- few tokens (up to 64): fewtok_kernel
// With few tokens the drain is small and the fixed cost of handing an accumulator back and forth
// once per slab would bound the kernel.  So here: one token tile (TT = 32 or 64 tokens, N of the MMA),
// a ring of four accumulators in TMEM that the single MMA warp fills without waiting for the
// epilogue, the first MMA of a slab overwrites (no start values are stored), the running sums live
// in the epilogue threads' registers (no TMEM traffic but the accumulator loads), and three
// expander groups build consecutive slabs at once, because what bounds this kernel is how fast the
// packed weights can be expanded: that has to keep up with HBM.  K is split over CTAs when there
// are fewer output tiles than SMs.
//   int -> float of an accumulator: bits(D + (0x4B400000 - sum of the slab's activations)) is the
//   float 12582912 + I, as in the many-token kernel, but the addend meets D in the epilogue.
// Warps: 0 copy, 1-2 MMA issue (alternate slabs; 1 owns TMEM), 3 idle, 4..11 epilogue (lane quadrant =
// warp % 4; warps 4-7 take the first half of the tokens, 8-11 the second), 12..23 expanders.
constexpr int kFewEpilogueWarps = 8, kFewExpGroups = 3, kFewStagesA = stages_a(kFewExpGroups), kFewStagesB = 4, kFewAccBufs = 4;
constexpr int kFewFirstExpandWarp = kFirstEpilogueWarp + kFewEpilogueWarps;
constexpr int kFewThreads = threads_of(kFewEpilogueWarps, kFewExpGroups);

template <int CODEC, int PLANES, int TT, bool DUMP>
__global__ void __launch_bounds__(kFewThreads, 1) fewtok_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap map_q) {
  constexpr uint32_t kTileBBytes = TT * 128;
  constexpr uint32_t kCW = TT / 2;                  // columns (tokens) per epilogue thread
  constexpr uint32_t kChunks = kCW / 16;
  constexpr uint32_t kSlabsPerCol = 2 * PLANES;
  constexpr uint32_t kIdesc = instr_desc_n(TT);
  constexpr uint32_t kTmemCols = kFewAccBufs * TT;  // 128 or 256
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tile_a = smem;
  uint8_t* tile_b = tile_a + kFewStagesA * kTileABytes;
  int32_t* qinit_s = reinterpret_cast<int32_t*>(tile_b + kFewStagesB * 2 * kTileBBytes);
  uint32_t* stage_s = reinterpret_cast<uint32_t*>(qinit_s + kFewStagesB * 2 * TT);
  __shared__ uint64_t a_full[kFewStagesA], a_empty[kFewStagesA], b_full[kFewStagesB], b_empty[kFewStagesB];
  __shared__ uint64_t acc_full[kFewAccBufs], acc_empty[kFewAccBufs];
  __shared__ uint32_t tmem_base_s, abort_flag, combine_flag;

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < kFewStagesA; ++s) { mbar_init(&a_full[s], kGroupWarps); mbar_init(&a_empty[s], 1); }
    for (int s = 0; s < kFewStagesB; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 2 + kFewEpilogueWarps); }
    for (int s = 0; s < kFewAccBufs; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], kFewEpilogueWarps); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_base_s)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t tiles = p.n_tiles * p.m_tiles * p.splits;
  const WaitCtx wctx{&abort_flag, p.status};

  // Registers follow the work.  The pool is what the CTA got at launch, 768 x 80: the first
  // warpgroup (copy, MMA issue, idle) gives back 40 per thread, the two epilogue warpgroups take
  // 16 more each; 128 x 40 + 256 x 96 + 384 x 80 fits, so no request can block.
  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    tma_role<TT, kFewStagesB>(p, map_q, tiles, tile_b, qinit_s, b_full, b_empty, wctx, lane);
  } else if (warp == 1 || warp == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    // ------------------------------------------------ MMA issue: two warps take alternate slabs (issuing the four
    // MMAs of a slab occupies the issuing thread for several hundred clocks, more than the
    // slab's share of the weight stream allows), each up to two slabs ahead of the epilogue
    const uint32_t mine = warp - 1;
    uint32_t slab = 0, colfill = 0;
    const uint64_t a_desc0 = smem_desc(saddr(tile_a), 0), b_desc0 = smem_desc(saddr(tile_b), 0);
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      uint32_t j0, j1;
      split_range(p, tile, j0, j1);
      for (uint32_t j = j0; j < j1; ++j, ++colfill) {
        const uint32_t sb = colfill % kFewStagesB;
        mbar_wait(&b_full[sb], (colfill / kFewStagesB) & 1, wctx, 311);
        for (uint32_t q = 0; q < kSlabsPerCol; ++q, ++slab) {
          if ((slab & 1u) != mine) continue;
          const uint32_t sa = slab % kFewStagesA, gsel = q & 1, buf = slab % kFewAccBufs;
          mbar_wait(&a_full[sa], (slab / kFewStagesA) & 1, wctx, 312, 32);
          if (slab >= uint32_t(kFewAccBufs)) mbar_wait(&acc_empty[buf], ((slab / kFewAccBufs) - 1) & 1, wctx, 313);
          tc_fence_after();
          const uint64_t a_desc = a_desc0 + uint64_t(sa * (kTileABytes >> 4));
          const uint64_t b_desc = b_desc0 + uint64_t((sb * 2 + gsel) * (kTileBBytes >> 4));
          if (elect_one()) {
#pragma unroll
            for (uint32_t kc = 0; kc < 4; ++kc) tc_mma_i8(tmem_base + buf * TT, a_desc + 2 * kc, b_desc + 2 * kc, kIdesc, kc > 0 ? 1u : 0u);
            tc_commit(&acc_full[buf]);
            tc_commit(&a_empty[sa]);
          }
          __syncwarp();
        }
        if (elect_one()) tc_commit(&b_empty[sb]);
        __syncwarp();
      }
    }
  } else if (warp >= kFewFirstExpandWarp) {
    expander_role<CODEC, PLANES, kFewExpGroups, kFewStagesA>(p, tiles, warp - kFewFirstExpandWarp, lane, tile_a, stage_s, a_full, a_empty, wctx);
  } else if (warp >= kFirstEpilogueWarp) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 96;");
    // ------------------------------------------------ epilogue: TMEM lane = weight row, running sums in registers
    const uint32_t quad = warp & 3, colhalf = (warp - kFirstEpilogueWarp) >> 2, r = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((quad * 32u) << 16) + colhalf * kCW;
    float y[kCW];
#pragma unroll
    for (uint32_t i = 0; i < kCW; ++i) y[i] = 0.f;
    uint32_t slab = 0, colfill = 0;
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      const uint32_t sp = tile % p.splits, out_tile = tile / p.splits, nt = out_tile / p.m_tiles, mt = out_tile % p.m_tiles;
      uint32_t j0, j1;
      split_range(p, tile, j0, j1);
      const uint32_t n = nt * kRows + r;
      const uint32_t nc = min(n, p.n - 1);
      const uint16_t* srow = p.scales + size_t(nc) * p.tpr * PLANES * 2;
      const uint32_t tok0 = mt * TT + colhalf * kCW;
      // The row's group scales of a tile column (two f16 per plane) are fetched one column ahead:
      // a load issued where the scale is needed would stall every slab for a trip to L2.
      const uint32_t* srow2 = reinterpret_cast<const uint32_t*>(srow);
      uint32_t sc_next[PLANES];
#pragma unroll
      for (int pl = 0; pl < PLANES; ++pl) sc_next[pl] = __ldg(srow2 + j0 * PLANES + pl);
      for (uint32_t j = j0; j < j1; ++j, ++colfill) {
        const uint32_t sb = colfill % kFewStagesB;
        uint32_t sc[PLANES];
#pragma unroll
        for (int pl = 0; pl < PLANES; ++pl) {
          sc[pl] = sc_next[pl];
          if (j + 1 < j1) sc_next[pl] = __ldg(srow2 + (j + 1) * PLANES + pl);
        }
        mbar_wait(&b_full[sb], (colfill / kFewStagesB) & 1, wctx, 314, 64);   // the column's start values are in shared memory
#pragma unroll
        for (uint32_t q = 0; q < kSlabsPerCol; ++q, ++slab) {
          const uint32_t gsel = q & 1, pl = q >> 1, buf = slab % kFewAccBufs;
          const float sv = __half2float(__ushort_as_half(uint16_t(gsel ? sc[pl] >> 16 : sc[pl] & 0xffffu)));
          const float2 scale2 = make_float2(sv, sv), neg_magic2 = make_float2(-12582912.0f, -12582912.0f);
          mbar_wait(&acc_full[buf], (slab / kFewAccBufs) & 1, wctx, 315, 64);   // sleeps between polls: the issue slots belong to the expanders
          tc_fence_after();
          uint32_t dv[kChunks][16];
#pragma unroll
          for (uint32_t c = 0; c < kChunks; ++c) tmem_ldn(lane_addr + buf * TT + c * 16, dv[c]);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);   // the MMA warp may overwrite this accumulator
          const uint32_t qi = saddr(qinit_s + (sb * 2 + gsel) * TT + colhalf * kCW);
#pragma unroll
          for (uint32_t c = 0; c < kChunks; ++c) {
            uint32_t iv[16];
#pragma unroll
            for (int i = 0; i < 16; i += 4) lds128(qi + (c * 16 + i) * 4u, &iv[i]);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const uint32_t b0 = dv[c][i] + iv[i], b1 = dv[c][i + 1] + iv[i + 1];   // bits of 12582912 + I
              const float2 d = __fadd2_rn(make_float2(__uint_as_float(b0), __uint_as_float(b1)), neg_magic2);
              const float2 acc = __ffma2_rn(d, scale2, make_float2(y[c * 16 + i], y[c * 16 + i + 1]));
              y[c * 16 + i] = acc.x; y[c * 16 + i + 1] = acc.y;
              if (DUMP) {
                if (n < p.n) {
                  const uint32_t mtok = tok0 + c * 16 + i;
                  if (mtok < p.m) p.acc_dump[((size_t(mtok) * p.n + n) * (p.tpr * 2) + 2 * j + gsel) * PLANES + pl] = int(b0) - int(kMagicBits);
                  if (mtok + 1 < p.m) p.acc_dump[((size_t(mtok + 1) * p.n + n) * (p.tpr * 2) + 2 * j + gsel) * PLANES + pl] = int(b1) - int(kMagicBits);
                }
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&b_empty[sb]);
      }
      // ---- the tile (or this split of it) is complete
      if (n < p.n) {
        const float rs = p.row_scale ? p.row_scale[n] : 1.0f;
#pragma unroll
        for (uint32_t i = 0; i < kCW; ++i) {
          const uint32_t mtok = tok0 + i;
          if (mtok < p.m) {
            if (p.splits > 1) {
              p.partial[(size_t(sp) * p.m_pad + mtok) * p.n + n] = y[i];
            } else {
              float out = __fmul_rn(y[i], __ldg(p.ascale + mtok));
              if (p.row_scale) out = __fmul_rn(out, rs);
              const size_t idx = size_t(mtok) * p.n + n;
              if (p.residual) out = __fadd_rn(__ldg(p.residual + idx), out);
              if (p.y_dtype == TB_F32) static_cast<float*>(p.y)[idx] = out;
              else static_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(out);
            }
          }
        }
      }
#pragma unroll
      for (uint32_t i = 0; i < kCW; ++i) y[i] = 0.f;
      if (p.splits > 1) {
        // Split K: count this split in; whoever completes the count adds the splits' sums in split
        // order (every run gives the same bits) and finishes the tile's outputs.
        __threadfence();
        named_sync(kBarEpilogue, 32 * kFewEpilogueWarps);
        if (warp == kFirstEpilogueWarp && lane == 0) {
          const uint32_t arrived = atomicAdd(p.tile_counters + out_tile, 1u);
          combine_flag = arrived == p.splits - 1 ? 1u : 0u;
          if (combine_flag) p.tile_counters[out_tile] = 0u;   // ready for the next launch
        }
        named_sync(kBarEpilogue, 32 * kFewEpilogueWarps);
        if (combine_flag && n < p.n) {
          __threadfence();
          const float rs = p.row_scale ? p.row_scale[n] : 1.0f;
          for (uint32_t c = 0; c < kCW; ++c) {
            const uint32_t mtok = tok0 + c;
            if (mtok >= p.m) break;
            float sum = __ldcg(p.partial + size_t(mtok) * p.n + n);
            for (uint32_t s2 = 1; s2 < p.splits; ++s2) sum = __fadd_rn(sum, __ldcg(p.partial + (size_t(s2) * p.m_pad + mtok) * p.n + n));
            float out = __fmul_rn(sum, __ldg(p.ascale + mtok));
            if (p.row_scale) out = __fmul_rn(out, rs);
            const size_t idx = size_t(mtok) * p.n + n;
            if (p.residual) out = __fadd_rn(__ldg(p.residual + idx), out);
            if (p.y_dtype == TB_F32) static_cast<float*>(p.y)[idx] = out;
            else static_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(out);
          }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");   // the idle warp of the first warpgroup
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// ---------------------------------------------------------------- host side
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_tiled_fn() {
  static EncodeTiled fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeTiled>(sym);
  }();
  return fn;
}

// tokens per accumulator half: one token tile of 32, 64 or 128 tokens for that many tokens, else
// tiles of 256.  Tiles of 32 and 64 tokens run the few-token configuration of the kernel.
uint32_t half_width(uint32_t m) { return m <= 32 ? 16 : m <= 64 ? 32 : m <= 128 ? 64 : 128; }
uint32_t pad_tokens(uint32_t m) { const uint32_t t = 2 * half_width(m); return (m + t - 1) / t * t; }
// K splits of an output tile: as many as keep every CTA of one wave busy, at most one per tile column.
uint32_t k_splits(uint32_t out_tiles, uint32_t tpr, uint32_t sm_count, uint32_t hw) {
  if (hw > 32 || out_tiles >= sm_count || out_tiles > kMaxSplitTiles) return 1;
  return std::max(1u, std::min(std::min(sm_count / out_tiles, tpr), 8u));
}
uint32_t splits_of(const tb_weights* w, uint32_t m, uint32_t sm_count) {
  const uint32_t hw = half_width(m), tile_tokens = 2 * hw;
  const uint32_t out_tiles = uint32_t((w->n + kRows - 1) / kRows) * (pad_tokens(m) / tile_tokens);
  return k_splits(out_tiles, uint32_t(w->k / 256), sm_count, hw);
}

struct Scratch { int8_t* qperm; int32_t* qinit; float* ascale; float* partial; };
Scratch carve(void* base, uint32_t m_pad, uint32_t k) {
  uint8_t* b = static_cast<uint8_t*>(base);
  Scratch s;
  s.qperm = reinterpret_cast<int8_t*>(b);
  size_t off = (size_t(m_pad) * k + 255) & ~size_t(255);
  s.qinit = reinterpret_cast<int32_t*>(b + off);
  off += (size_t(k / 128) * m_pad * 4 + 255) & ~size_t(255);
  s.ascale = reinterpret_cast<float*>(b + off);
  off += (size_t(m_pad) * 4 + 255) & ~size_t(255);
  s.partial = reinterpret_cast<float*>(b + off);   // [splits][m_pad][n], only when K is split
  return s;
}

size_t smem_of(uint32_t hw) {
  const uint32_t tile_tokens = 2 * hw;
  if (hw <= 32)   // few-token kernel
    return 1024 + size_t(kFewStagesA) * kTileABytes + size_t(kFewStagesB) * 2 * tile_tokens * 128 + size_t(kFewStagesB) * 2 * tile_tokens * 4 +
           size_t(kGroupWarps * kFewExpGroups) * 32 * 16 * 4;
  return 1024 + size_t(stages_a(1)) * kTileABytes + size_t(kStagesB) * 2 * tile_tokens * 128 + size_t(kStagesB) * 2 * tile_tokens * 4 +
         size_t(kGroupWarps) * 32 * 16 * 4;
}

template <typename Kernel>
cudaError_t launch_kernel(Kernel kernel, dim3 grid, int threads, size_t smem, cudaStream_t st, const PrefillParams& pp, const CUtensorMap& map) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (e != cudaSuccess) return e;
  // may start under the tail of the quantisation pre-pass (see tma_role)
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = dim3(unsigned(threads)); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, pp, map);
}

template <int CODEC, int HW, bool DUMP>
cudaError_t launch_planes(uint32_t planes, dim3 grid, size_t smem, cudaStream_t st, const PrefillParams& pp, const CUtensorMap& map) {
  if constexpr (HW <= 32) {
    constexpr int TT = 2 * HW;
    if (planes == 1) return launch_kernel(fewtok_kernel<CODEC, 1, TT, DUMP>, grid, kFewThreads, smem, st, pp, map);
    if (planes == 2) return launch_kernel(fewtok_kernel<CODEC, 2, TT, DUMP>, grid, kFewThreads, smem, st, pp, map);
    return launch_kernel(fewtok_kernel<CODEC, 3, TT, DUMP>, grid, kFewThreads, smem, st, pp, map);
  } else {
    constexpr int EPI = 16, EXP = 1;
    if (planes == 1) return launch_kernel(prefill_kernel<CODEC, 1, HW, DUMP, EPI, EXP>, grid, threads_of(EPI, EXP), smem, st, pp, map);
    if (planes == 2) return launch_kernel(prefill_kernel<CODEC, 2, HW, DUMP, EPI, EXP>, grid, threads_of(EPI, EXP), smem, st, pp, map);
    return launch_kernel(prefill_kernel<CODEC, 3, HW, DUMP, EPI, EXP>, grid, threads_of(EPI, EXP), smem, st, pp, map);
  }
}

template <int CODEC>
cudaError_t launch_shape(uint32_t hw, bool dump, uint32_t planes, dim3 grid, size_t smem, cudaStream_t st, const PrefillParams& pp,
                         const CUtensorMap& map) {
#define TB_HW_CASE(W) \
  if (hw == W) return dump ? launch_planes<CODEC, W, true>(planes, grid, smem, st, pp, map) \
                           : launch_planes<CODEC, W, false>(planes, grid, smem, st, pp, map)
  TB_HW_CASE(16);
  TB_HW_CASE(32);
  TB_HW_CASE(64);
  TB_HW_CASE(128);
#undef TB_HW_CASE
  return cudaErrorInvalidValue;
}

}  // namespace

bool tb_prefill_supported(const tb_weights* w, uint32_t m) {
  return w->fast && m >= 1 && w->k >= 256 && encode_tiled_fn() != nullptr;
}

size_t tb_prefill_scratch_bytes(const tb_weights* w, uint32_t m) {
  const uint32_t m_pad = pad_tokens(m);
  const uint32_t sm_count = w->owner ? uint32_t(w->owner->prop.multiProcessorCount) : 148u;
  const uint32_t splits = splits_of(w, m, sm_count);
  return ((size_t(m_pad) * w->k + 255) & ~size_t(255)) + ((size_t(w->k / 128) * m_pad * 4 + 255) & ~size_t(255)) +
         ((size_t(m_pad) * 4 + 255) & ~size_t(255)) + (splits > 1 ? size_t(splits) * m_pad * w->n * 4 : 0) + 256;
}

cudaError_t tb_launch_prefill(const PrefillArgs& a, int sm_count, cudaStream_t stream) {
  const tb_weights* w = a.w;
  const uint32_t m_pad = pad_tokens(a.m), k = uint32_t(w->k);
  if (!a.scratch || a.scratch_bytes < tb_prefill_scratch_bytes(w, a.m)) return cudaErrorInvalidValue;
  const Scratch sc = carve(a.scratch, m_pad, k);

  QuantParams qp{};
  qp.x = a.x; qp.act_scale_in = a.act_scale_in; qp.act_absmax_in = a.act_absmax_in;
  if (a.relu2_up) {
    if (a.x_dtype != TB_F32) return cudaErrorInvalidValue;
    qp.relu2_up = a.relu2_up;
  }
  qp.qperm = sc.qperm; qp.qinit = sc.qinit; qp.ascale = sc.ascale;
  qp.m = a.m; qp.m_pad = m_pad; qp.k = k; qp.x_dtype = uint32_t(a.x_dtype); qp.codec = uint32_t(w->codec); qp.status = a.status;
  prefill_quant_kernel<<<m_pad, 256, 0, stream>>>(qp);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;

  // activations as a 2-D int8 tensor [m_pad rows][k bytes]; a box is one slab of one token tile
  CUtensorMap map;
  const cuuint64_t dims[2] = {k, m_pad};
  const cuuint64_t strides[1] = {k};
  const uint32_t hw = half_width(a.m), tile_tokens = 2 * hw;
  const cuuint32_t box[2] = {128, tile_tokens};
  const cuuint32_t elem[2] = {1, 1};
  if (encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, sc.qperm, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;

  PrefillParams pp{};
  pp.payload = w->d_payload; pp.scales = w->d_scales;
  pp.qperm = sc.qperm; pp.qinit = sc.qinit; pp.ascale = sc.ascale;
  pp.y = a.y; pp.acc_dump = a.acc_dump; pp.row_scale = a.row_scale; pp.status = a.status; pp.residual = a.residual;
  pp.m = a.m; pp.m_pad = m_pad; pp.n = uint32_t(w->n); pp.k = k; pp.tpr = k / 256; pp.y_dtype = uint32_t(a.y_dtype);
  pp.n_tiles = (pp.n + kRows - 1) / kRows; pp.m_tiles = m_pad / tile_tokens;
  pp.splits = splits_of(w, a.m, uint32_t(sm_count));
  if (pp.splits > 1) {
    if (!a.tile_counters) return cudaErrorInvalidValue;
    pp.partial = sc.partial; pp.tile_counters = a.tile_counters;
  }
  const size_t smem = smem_of(hw);
  const dim3 grid(std::min<uint32_t>(pp.n_tiles * pp.m_tiles * pp.splits, uint32_t(sm_count)));
  const bool dump = a.acc_dump != nullptr;
  return w->codec == tbf::kB3 ? launch_shape<tbf::kB3>(hw, dump, w->uniform_planes, grid, smem, stream, pp, map)
                              : launch_shape<tbf::kD2>(hw, dump, w->uniform_planes, grid, smem, stream, pp, map);
}
