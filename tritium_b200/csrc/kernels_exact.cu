// Bit-exact SALT V2 forward for any valid layout (ragged plane counts, g64/g128, rows that
// straddle tiles, D2/B3/S34), plus row gather.
//
// Arithmetic contract (crates/tritium-cpu/src/salt_v2.rs:10-23,316-423): per output row, walk
// the scale-group segments in ascending coefficient order; per segment and per plane (ascending)
// fold ga = ga ± x[col] sequentially in fp32, multiply once by the f16 scale, add to the row
// accumulator.  No FMA, no reassociation.  Here one warp owns one output row: each lane folds
// whole (segment, plane) sums on its own — the sequential order inside a sum is kept — and the
// contributions are then added in segment/plane order, so the result is bit-identical.
//
// Compiled with --fmad=false; the explicit _rn intrinsics pin the rounding as well.
#include <cuda_fp16.h>

#include <cuda_bf16.h>

#include "tb_internal.h"

namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kTokens = 4;  // tokens folded per decode pass

struct ExactParams {
  const uint8_t* payload; const uint16_t* scales; const uint8_t* meta; const uint32_t* tile_rank;
  uint64_t map_bytes, coeffs, tiles;
  uint32_t terminal, uniform_planes, codec, group, m, n, k;
  uint32_t pad_planes;   // != 0: every tile occupies this many plane slots; its true count comes from the map
  const float* x; float* y; const float* row_scale;
  uint32_t* status;
};

__device__ __forceinline__ uint32_t plane_bytes_dev(uint32_t codec, uint32_t len) {
  if (codec == tbf::kD2) return (len + 3u) >> 2;
  if (codec == tbf::kB3) return (len + 4u) / 5u;
  return (((len + 3u) >> 2) * 5u + 7u) >> 3;
}

__device__ __forceinline__ uint32_t planes_of(const ExactParams& p, uint64_t tile) {
  if (p.uniform_planes) return p.uniform_planes;
  const uint64_t bit = tile * 2;
  const uint32_t code = bit < p.map_bytes * 8 ? (p.meta[bit >> 3] >> (bit & 7)) & 3u
                                              : (p.terminal >> (bit - p.map_bytes * 8)) & 3u;
  return code + 1;
}

__device__ __forceinline__ uint64_t rank_of(const ExactParams& p, uint64_t tile) {
  if (p.pad_planes) return tile * p.pad_planes;
  return p.uniform_planes ? tile * p.uniform_planes : p.tile_rank[tile];
}

// One trit of a plane whose bytes start at `base`.  `lut` maps a B3 byte to five 2-bit digits.
__device__ __forceinline__ int trit_at(const uint8_t* base, uint32_t codec, uint32_t local,
                                       const uint16_t* lut) {
  if (codec == tbf::kD2) return int((base[local >> 2] >> (2 * (local & 3))) & 3u) - 1;
  if (codec == tbf::kB3) {
    const uint32_t byte = local / 5u;
    return int((lut[base[byte]] >> (2 * (local - byte * 5u))) & 3u) - 1;
  }
  const uint32_t bit = (local >> 2) * 5u, byte = bit >> 3;
  const uint32_t word = base[byte] | (uint32_t(base[byte + 1]) << 8);  // arena is padded by one byte
  const uint32_t code = (word >> (bit & 7)) & 31u, slot = local & 3u, zero = code & 3u;
  if (slot == zero) return 0;
  return (code >> (2 + slot - (slot > zero))) & 1u ? 1 : -1;
}

// Acc = float reproduces the reference order bit for bit.  Acc = double is the trait path's
// accumulator (the reference's own CUDA kernel for that path folds in f64,
// crates/tritium-cuda/kernels/tq2_0_add.cu:107-175): the only rounding left is the final one.
template <typename Acc> __device__ __forceinline__ Acc acc_add(Acc a, float b);
template <> __device__ __forceinline__ float acc_add<float>(float a, float b) { return __fadd_rn(a, b); }
template <> __device__ __forceinline__ double acc_add<double>(double a, float b) { return __dadd_rn(a, double(b)); }
template <typename Acc> __device__ __forceinline__ Acc acc_mul(Acc a, float b);
template <> __device__ __forceinline__ float acc_mul<float>(float a, float b) { return __fmul_rn(a, b); }
template <> __device__ __forceinline__ double acc_mul<double>(double a, float b) { return __dmul_rn(a, double(b)); }
__device__ __forceinline__ float shfl_acc(float v, int l) { return __shfl_sync(0xffffffffu, v, l); }
__device__ __forceinline__ double shfl_acc(double v, int l) { return __shfl_sync(0xffffffffu, v, l); }

template <typename Acc>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) salt_v2_exact_kernel(const ExactParams p) {
  __shared__ uint16_t lut[243];
  for (int b = threadIdx.x; b < 243; b += blockDim.x) {
    int v = b; uint32_t packed = 0;
    for (int i = 0; i < 5; ++i) { packed |= uint32_t(v % 3) << (2 * i); v /= 3; }
    lut[b] = uint16_t(packed);
  }
  __syncthreads();
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t row = blockIdx.x * kWarpsPerBlock + warp;
  const uint32_t m0 = blockIdx.y * kTokens;
  if (row >= p.n) return;
  const uint32_t tokens = min(uint32_t(kTokens), p.m - m0);
  const uint64_t row_base = uint64_t(row) * p.k, row_end = row_base + p.k;
  const uint32_t full_bytes = plane_bytes_dev(p.codec, 256), full_scales = 256u / p.group;

  Acc acc[kTokens];
#pragma unroll
  for (int t = 0; t < kTokens; ++t) acc[t] = Acc(0);
  bool bad = false;
  uint32_t bad_col = 0;

  // Segment s of this row: boundaries are the row start, every tile-local group boundary, and
  // the row end.  first_boundary = distance from the row start to the next group boundary.
  const uint32_t head = p.group - uint32_t(row_base % p.group);  // group divides 256
  const uint32_t first_len = min(head, p.k);
  const uint32_t segments = 1 + (p.k > first_len ? (p.k - first_len + p.group - 1) / p.group : 0);

  for (uint32_t seg0 = 0; seg0 < segments; seg0 += 32) {
    const uint32_t seg = seg0 + lane;
    Acc contrib[3][kTokens];
    uint32_t planes = 0;
#pragma unroll
    for (int q = 0; q < 3; ++q)
#pragma unroll
      for (int t = 0; t < kTokens; ++t) contrib[q][t] = Acc(0);
    if (seg < segments) {
      const uint32_t col0 = seg == 0 ? 0 : first_len + (seg - 1) * p.group;
      const uint32_t len = seg == 0 ? first_len : min(p.group, p.k - col0);
      const uint64_t c = row_base + col0, tile = c >> 8;
      const uint32_t local0 = uint32_t(c & 255);
      const uint32_t tlen = uint32_t(min(uint64_t(256), p.coeffs - (tile << 8)));
      const uint32_t g = local0 / p.group;
      planes = planes_of(p, tile);
      const uint64_t rank = rank_of(p, tile);
      const uint32_t cur_bytes = plane_bytes_dev(p.codec, tlen);
      const uint32_t cur_scales = (tlen + p.group - 1) / p.group;
      for (uint32_t q = 0; q < planes; ++q) {
        const uint8_t* base = p.payload + rank * full_bytes + uint64_t(q) * cur_bytes;
        const float scale = __half2float(__ushort_as_half(p.scales[rank * full_scales + q * cur_scales + g]));
        Acc ga[kTokens];
#pragma unroll
        for (int t = 0; t < kTokens; ++t) ga[t] = Acc(0);
        for (uint32_t e = 0; e < len; ++e) {
          const int trit = trit_at(base, p.codec, local0 + e, lut);
          if (trit == 0) continue;
#pragma unroll
          for (int t = 0; t < kTokens; ++t)
            if (t < int(tokens)) {
              const float xv = p.x[uint64_t(m0 + t) * p.k + col0 + e];
              ga[t] = acc_add<Acc>(ga[t], trit > 0 ? xv : -xv);
              if (!isfinite(ga[t]) && !bad) { bad = true; bad_col = col0 + e; }
            }
        }
#pragma unroll
        for (int t = 0; t < kTokens; ++t) {
          contrib[q][t] = acc_mul<Acc>(ga[t], scale);
          if (!isfinite(contrib[q][t]) && !bad) { bad = true; bad_col = col0 + len - 1; }
        }
      }
      (void)row_end;
    }
    // ordered fold: segment ascending, plane ascending
    for (int l = 0; l < 32; ++l) {
      const uint32_t lp = __shfl_sync(0xffffffffu, planes, l);
      if (lp == 0) break;  // uniform: lanes past the last segment hold zero planes
#pragma unroll
      for (int q = 0; q < 3; ++q) {
        if (uint32_t(q) < lp) {
#pragma unroll
          for (int t = 0; t < kTokens; ++t) {
            const Acc v = shfl_acc(contrib[q][t], l);
            acc[t] = acc[t] + v;
          }
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kTokens; ++t)
    if (!isfinite(acc[t]) && !bad) { bad = true; bad_col = p.k - 1; }
  if (__any_sync(0xffffffffu, bad)) {
    if (bad && atomicOr(&p.status[TBS_FLAGS], TBF_NONFINITE_OUT) == 0) {
      p.status[TBS_INFO0] = row;
      p.status[TBS_INFO1] = bad_col;
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int t = 0; t < kTokens; ++t)
      if (t < int(tokens)) {
        float v = float(acc[t]);
        if (p.row_scale) v = __fmul_rn(v, p.row_scale[row]);
        p.y[uint64_t(m0 + t) * p.n + row] = v;
      }
  }
}

__global__ void gather_rows_kernel(const ExactParams p, const uint32_t* rows, uint32_t count, float* out) {
  __shared__ uint16_t lut[243];
  for (int b = threadIdx.x; b < 243; b += blockDim.x) {
    int v = b; uint32_t packed = 0;
    for (int i = 0; i < 5; ++i) { packed |= uint32_t(v % 3) << (2 * i); v /= 3; }
    lut[b] = uint16_t(packed);
  }
  __syncthreads();
  const uint64_t idx = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= uint64_t(count) * p.k) return;
  const uint32_t which = uint32_t(idx / p.k), col = uint32_t(idx % p.k);
  const uint64_t c = uint64_t(rows[which]) * p.k + col, tile = c >> 8;
  const uint32_t local = uint32_t(c & 255);
  const uint32_t tlen = uint32_t(min(uint64_t(256), p.coeffs - (tile << 8)));
  const uint32_t full_bytes = plane_bytes_dev(p.codec, 256), cur_bytes = plane_bytes_dev(p.codec, tlen);
  const uint32_t full_scales = 256u / p.group, cur_scales = (tlen + p.group - 1) / p.group;
  const uint64_t rank = rank_of(p, tile);
  float w = 0.f;
  for (uint32_t q = 0; q < planes_of(p, tile); ++q) {
    const int trit = trit_at(p.payload + rank * full_bytes + uint64_t(q) * cur_bytes, p.codec, local, lut);
    const float scale = __half2float(__ushort_as_half(p.scales[rank * full_scales + q * cur_scales + local / p.group]));
    w = __fadd_rn(w, __fmul_rn(float(trit), scale));
  }
  out[idx] = w;
}

__global__ void check_finite_kernel(const float* x, uint64_t count, uint32_t* status) {
  const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
    if (!isfinite(x[i]) && atomicOr(&status[TBS_FLAGS], TBF_NONFINITE_ACT) == 0) {
      status[TBS_INFO0] = uint32_t(i);
      status[TBS_INFO1] = __float_as_uint(x[i]);
    }
}

// max |x| of each token's row: one CTA per token
__global__ void __launch_bounds__(256) row_absmax_kernel(const void* x, uint32_t dtype, uint32_t k, float* out) {
  __shared__ float red[8];
  const uint32_t t = blockIdx.x, tid = threadIdx.x;
  float mx = 0.f;
  for (uint32_t i = tid; i < k; i += 256) {
    const size_t idx = size_t(t) * k + i;
    const float v = dtype == TB_F32 ? static_cast<const float*>(x)[idx]
                                    : __bfloat162float(static_cast<const __nv_bfloat16*>(x)[idx]);
    mx = fmaxf(mx, fabsf(v));
  }
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
    out[t] = mx;
  }
}

// RMSNorm of one token's row per CTA, in the reference's canonical order
// (crates/tritium-nn/src/ops/rmsnorm.rs:20-94): the 256 threads are the 256 slots, slot t folds
// x[t], x[t+256], ... ascending, then the power-of-two tree; out = (x * inv) * w, or (1 + w).
__global__ void __launch_bounds__(256) rmsnorm_kernel(const void* x, uint32_t dtype, const float* weight, float eps,
                                                      uint32_t zero_centered, uint32_t k, float* out) {
  __shared__ float part[256];
  __shared__ float inv_s;
  const uint32_t t = blockIdx.x, tid = threadIdx.x;
  const auto at = [&](uint32_t i) {
    const size_t idx = size_t(t) * k + i;
    return dtype == TB_F32 ? static_cast<const float*>(x)[idx] : __bfloat162float(static_cast<const __nv_bfloat16*>(x)[idx]);
  };
  float acc = 0.f;
  for (uint32_t i = tid; i < k; i += 256) { const float v = at(i); acc = __fadd_rn(acc, __fmul_rn(v, v)); }
  part[tid] = acc;
  __syncthreads();
  for (uint32_t off = 128; off >= 32; off >>= 1) {
    if (tid < off) part[tid] = __fadd_rn(part[tid], part[tid + off]);
    __syncthreads();
  }
  if (tid < 32) {
    float v = part[tid];
    for (int o = 16; o; o >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, o));
    if (tid == 0) inv_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(v, float(k)), eps)));
  }
  __syncthreads();
  const float inv = inv_s;
  for (uint32_t i = tid; i < k; i += 256) {
    const float scale = zero_centered ? __fadd_rn(1.0f, weight[i]) : weight[i];
    out[size_t(t) * k + i] = __fmul_rn(__fmul_rn(at(i), inv), scale);
  }
}

// Per-token absmax int8 quantisation with the codes kept as fp32 values (quantize_act_int8,
// crates/tritium-spec/src/lib.rs:239-264): the input of the exact kernel when a layout without a
// fast kernel takes the int8 path.  One CTA per token.
__global__ void __launch_bounds__(256) quantize_to_float_kernel(const void* x, uint32_t dtype, uint32_t k, float* q, float* act_scale,
                                                                uint32_t* status) {
  __shared__ float red[8];
  const uint32_t t = blockIdx.x, tid = threadIdx.x;
  const auto at = [&](uint32_t i) {
    const size_t idx = size_t(t) * k + i;
    return dtype == TB_F32 ? static_cast<const float*>(x)[idx] : __bfloat162float(static_cast<const __nv_bfloat16*>(x)[idx]);
  };
  float mx = 0.f;
  bool bad = false;
  for (uint32_t i = tid; i < k; i += 256) { const float v = at(i); bad |= !(fabsf(v) <= 3.402823466e+38f); mx = fmaxf(mx, fabsf(v)); }
  if (bad && atomicOr(&status[TBS_FLAGS], TBF_NONFINITE_ACT) == 0) { status[TBS_INFO0] = t * k; status[TBS_INFO1] = 0x7fc00000u; }
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  float gamma = 0.f;
  for (int w = 0; w < 8; ++w) gamma = fmaxf(gamma, red[w]);
  const float scale_q = gamma > 0.f ? __fdiv_rn(127.0f, gamma) : 0.f;
  if (tid == 0) act_scale[t] = __fdiv_rn(gamma, 127.0f);
  for (uint32_t i = tid; i < k; i += 256) q[size_t(t) * k + i] = fminf(127.f, fmaxf(-128.f, rintf(__fmul_rn(at(i), scale_q))));
}

// fp32 activations as four int8 limbs per element, for the int8 kernels: with gamma = max |x| of
// the token and u = x * 127 / gamma, q0 = rint(u), then three times r <- (r - q) * 128, q = rint(r):
//   x = (gamma / 127) * (q0 + q1 / 128 + q2 / 128^2 + q3 / 128^3) + e,  |e| <= gamma * 2e-9,
// every step after u exact in fp32.  Limb l of token t becomes pseudo-token 4 t + l with the
// dequantisation multiplier gamma / 127 / 128^l; the four outputs are added afterwards.
__global__ void __launch_bounds__(256) limb_split_kernel(const float* x, uint32_t k, int8_t* q, float* act_scale, uint32_t* status) {
  __shared__ float red[8];
  const uint32_t t = blockIdx.x, tid = threadIdx.x;
  const float* row = x + size_t(t) * k;
  float mx = 0.f;
  bool bad = false;
  for (uint32_t i = tid; i < k; i += 256) { const float v = row[i]; bad |= !(fabsf(v) <= 3.402823466e+38f); mx = fmaxf(mx, fabsf(v)); }
  if (bad && atomicOr(&status[TBS_FLAGS], TBF_NONFINITE_ACT) == 0) { status[TBS_INFO0] = t * k; status[TBS_INFO1] = 0x7fc00000u; }
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  float gamma = 0.f;
  for (int w = 0; w < 8; ++w) gamma = fmaxf(gamma, red[w]);
  const float scale_q = gamma > 0.f ? __fdiv_rn(127.0f, gamma) : 0.f;
  if (tid < 4) {
    float a = __fdiv_rn(gamma, 127.0f);
    for (uint32_t l = 0; l < tid; ++l) a = __fmul_rn(a, 0.0078125f);   // exact: a power of two
    act_scale[4 * t + tid] = a;
  }
  for (uint32_t i = tid; i < k; i += 256) {
    float r = __fmul_rn(row[i], scale_q);
#pragma unroll
    for (uint32_t l = 0; l < 4; ++l) {
      const float ql = fminf(127.f, fmaxf(-127.f, rintf(r)));
      q[(size_t(4 * t + l)) * k + i] = int8_t(int(ql));
      r = __fmul_rn(__fsub_rn(r, ql), 128.0f);
    }
  }
}

// y[t][i] = ((y4[4t][i] + y4[4t+1][i]) + y4[4t+2][i]) + y4[4t+3][i]
__global__ void __launch_bounds__(256) limb_sum_kernel(const float* y4, uint32_t n, float* y) {
  const uint32_t t = blockIdx.y;
  for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256) {
    const float* src = y4 + size_t(4 * t) * n + i;
    y[size_t(t) * n + i] = __fadd_rn(__fadd_rn(__fadd_rn(src[0], src[n]), src[2 * size_t(n)]), src[3 * size_t(n)]);
  }
}

// y_out[t][i] = y[t][i] * act_scale[t] (one rounding), fp32 or bf16
__global__ void __launch_bounds__(256) scale_tokens_kernel(const float* y, const float* act_scale, const float* residual, uint32_t n,
                                                           void* out, uint32_t out_dtype) {
  const uint32_t t = blockIdx.y;
  const float a = act_scale[t];
  for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256) {
    const size_t idx = size_t(t) * n + i;
    float v = __fmul_rn(y[idx], a);
    if (residual) v = __fadd_rn(residual[idx], v);
    if (out_dtype == TB_F32) static_cast<float*>(out)[idx] = v;
    else static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  }
}

ExactParams make_params(const tb_weights* w) {
  ExactParams p{};
  p.payload = w->d_payload; p.scales = w->d_scales; p.meta = w->d_meta; p.tile_rank = w->d_tile_rank;
  p.map_bytes = w->map_bytes; p.coeffs = w->n * w->k; p.tiles = w->tiles;
  p.terminal = w->terminal_map;
  p.uniform_planes = w->map_counts ? 0u : w->uniform_planes;
  p.pad_planes = w->map_counts ? w->uniform_planes : 0u;
  p.codec = uint32_t(w->codec); p.group = w->group; p.n = uint32_t(w->n); p.k = uint32_t(w->k);
  return p;
}

}  // namespace

cudaError_t tb_launch_exact(const ExactArgs& a, cudaStream_t stream) {
  ExactParams p = make_params(a.w);
  p.x = a.x; p.y = a.y; p.m = a.m; p.row_scale = a.row_scale; p.status = a.status;
  if (a.m == 0 || p.n == 0) return cudaSuccess;
  const dim3 grid((p.n + kWarpsPerBlock - 1) / kWarpsPerBlock, (a.m + kTokens - 1) / kTokens);
  if (a.w->is_tq2) salt_v2_exact_kernel<double><<<grid, kWarpsPerBlock * 32, 0, stream>>>(p);
  else salt_v2_exact_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t tb_launch_gather_rows(const tb_weights* w, const uint32_t* rows, uint32_t count, float* out,
                                  cudaStream_t stream) {
  ExactParams p = make_params(w);
  const uint64_t total = uint64_t(count) * p.k;
  if (!total) return cudaSuccess;
  gather_rows_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>(p, rows, count, out);
  return cudaGetLastError();
}

cudaError_t tb_launch_row_absmax(const void* x, tb_dtype dtype, uint32_t m, uint32_t k, float* out, cudaStream_t stream) {
  if (!m) return cudaSuccess;
  row_absmax_kernel<<<m, 256, 0, stream>>>(x, uint32_t(dtype), k, out);
  return cudaGetLastError();
}

cudaError_t tb_launch_rmsnorm(const void* x, tb_dtype dtype, const float* weight, float eps, bool zero_centered, uint32_t m,
                              uint32_t k, float* out, cudaStream_t stream) {
  if (!m) return cudaSuccess;
  rmsnorm_kernel<<<m, 256, 0, stream>>>(x, uint32_t(dtype), weight, eps, zero_centered ? 1u : 0u, k, out);
  return cudaGetLastError();
}

cudaError_t tb_launch_quantize_to_float(const void* x, tb_dtype dtype, uint32_t m, uint32_t k, float* q, float* act_scale, uint32_t* status,
                                        cudaStream_t stream) {
  if (!m) return cudaSuccess;
  quantize_to_float_kernel<<<m, 256, 0, stream>>>(x, uint32_t(dtype), k, q, act_scale, status);
  return cudaGetLastError();
}

cudaError_t tb_launch_limb_split(const float* x, uint32_t m, uint32_t k, int8_t* q, float* act_scale, uint32_t* status, cudaStream_t stream) {
  if (!m) return cudaSuccess;
  limb_split_kernel<<<m, 256, 0, stream>>>(x, k, q, act_scale, status);
  return cudaGetLastError();
}

cudaError_t tb_launch_limb_sum(const float* y4, uint32_t m, uint32_t n, float* y, cudaStream_t stream) {
  if (!m || !n) return cudaSuccess;
  limb_sum_kernel<<<dim3(std::min<uint32_t>((n + 255) / 256, 64), m), 256, 0, stream>>>(y4, n, y);
  return cudaGetLastError();
}

cudaError_t tb_launch_scale_tokens(const float* y, const float* act_scale, const float* residual, uint32_t m, uint32_t n, void* out,
                                   tb_dtype out_dtype, cudaStream_t stream) {
  if (!m || !n) return cudaSuccess;
  scale_tokens_kernel<<<dim3(std::min<uint32_t>((n + 255) / 256, 64), m), 256, 0, stream>>>(y, act_scale, residual, n, out, uint32_t(out_dtype));
  return cudaGetLastError();
}

cudaError_t tb_launch_check_finite(const float* x, uint64_t count, uint32_t* status, cudaStream_t stream) {
  if (!count) return cudaSuccess;
  const unsigned blocks = unsigned(std::min<uint64_t>((count + 255) / 256, 1184));
  check_finite_kernel<<<blocks, 256, 0, stream>>>(x, count, status);
  return cudaGetLastError();
}
