// Device helpers of the sparse MoE decode reader (sm_100a).
//
// The arithmetic in this file is *pinned*: every operation is an IEEE-754
// single-precision add, multiply, divide or fused multiply-add issued through
// an explicit intrinsic, so the compiler can neither reassociate nor contract
// it, and a host restatement using the same operation sequence reproduces the
// results bit for bit.  Channel selection depends only on pinned arithmetic and
// on exact integer dot products.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cfm {

constexpr int kBlock = 128;          // coordinates per rotation block
constexpr int kWordRows = 16;        // sketch rows per 32-bit word
constexpr int kQuantBits = 21;       // block maximum maps into [2^21, 2^22]
constexpr int kDownTileRows = 64;    // kept rows per down tile
constexpr int kEncodeTileRows = 256; // channels per encoder tile
constexpr unsigned kFull = 0xffffffffu;

// Round an FP32 value to BF16 (nearest even) and widen it again.
__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

// exp(x) from Cody-Waite reduction and a degree-7 Horner polynomial.
// exp(x) = 2^n * p(r), n = rint(x * log2 e), r = x - n * ln 2 (two-term split).
// Saturates to +inf from 88 and to 0 below -87; NaN propagates.
__device__ __forceinline__ float pinned_exp(float x) {
  if (!(x == x)) return x;
  if (x >= 88.0f) return __int_as_float(0x7f800000);
  if (x <= -87.0f) return 0.0f;
  const float n = rintf(__fmul_rn(x, 1.44269502f));
  float r = __fmaf_rn(n, -0.693145752f, x);
  r = __fmaf_rn(n, -1.42860677e-06f, r);
  float p = 1.98412701e-04f;
  p = __fmaf_rn(p, r, 1.38888892e-03f);
  p = __fmaf_rn(p, r, 8.33333377e-03f);
  p = __fmaf_rn(p, r, 4.16666679e-02f);
  p = __fmaf_rn(p, r, 1.66666672e-01f);
  p = __fmaf_rn(p, r, 0.5f);
  p = __fmaf_rn(p, r, 1.0f);
  p = __fmaf_rn(p, r, 1.0f);
  const int e = static_cast<int>(n);  // in [-126, 127]
  return __fmul_rn(p, __int_as_float((e + 127) << 23));
}

// SiLU: x / (1 + exp(-x)).
__device__ __forceinline__ float pinned_silu(float x) {
  return __fdiv_rn(x, __fadd_rn(1.0f, pinned_exp(-x)));
}

// GELU, tanh form: 0.5 x (1 + tanh(z)), z = sqrt(2/pi) (x + 0.044715 x^3),
// with tanh(z) = 1 - 2 / (exp(2 z) + 1).
__device__ __forceinline__ float pinned_gelu_tanh(float x) {
  const float x3 = __fmul_rn(__fmul_rn(x, x), x);
  const float inner = __fmaf_rn(0.044715f, x3, x);
  const float z = __fmul_rn(0.797884583f, inner);
  const float ez = pinned_exp(__fmul_rn(2.0f, z));
  const float th = __fsub_rn(1.0f, __fdiv_rn(2.0f, __fadd_rn(ez, 1.0f)));
  return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, th));
}

__device__ __forceinline__ float pinned_activate(float x, int activation) {
  return activation == 1 ? pinned_gelu_tanh(x) : pinned_silu(x);
}

// The gated feature with the reference's rounding points for an exactly
// computed channel: bf16(bf16(phi(bf16 g)) * bf16 u).
__device__ __forceinline__ float exact_feature(float g, float u, int activation) {
  const float gb = bf16_round(g), ub = bf16_round(u);
  return bf16_round(__fmul_rn(bf16_round(pinned_activate(gb, activation)), ub));
}

// The feature of a skipped channel from its sketch projections: one rounding,
// bf16(phi(bf16 g) * bf16 u).
__device__ __forceinline__ float sketch_feature(float g, float u, int activation) {
  const float gb = bf16_round(g), ub = bf16_round(u);
  return bf16_round(__fmul_rn(pinned_activate(gb, activation), ub));
}

// Point score: ((norm * phi(g)) * u)^2 * w^2 on BF16-rounded projections.
__device__ __forceinline__ float point_score(float g, float u, float norm, float w,
                                             int activation) {
  const float gb = bf16_round(g), ub = bf16_round(u);
  const float t = __fmul_rn(__fmul_rn(norm, pinned_activate(gb, activation)), ub);
  return __fadd_rn(__fmul_rn(__fmul_rn(t, t), __fmul_rn(w, w)), 0.0f);
}

// Recovery-aware score: w^2 times the expected squared output error of skipping
// the channel, with the gate modelled as Gaussian around g (five Gauss-Hermite
// nodes), sketch residual variances vg and vu, down-column norm n and the
// recovery response split into alpha (along the down column) and beta (across):
//   n^2 max(E[a^2] - E[a]^2, 0) + ((n E[a] - alpha p)^2 + (beta p)^2),
// p = bf16(phi(g) u), on BF16-rounded projections.
__device__ __forceinline__ float risk_score(float g, float u, float vg, float vu, float norm,
                                            float alpha, float beta, float w, int activation) {
  const float gb = bf16_round(g), ub = bf16_round(u);
  const float sg = __fsqrt_rn(vg), su = __fsqrt_rn(vu);
  const float spread = __fadd_rn(__fmul_rn(ub, ub), __fmul_rn(su, su));
  const float nodes[5] = {-2.85697007f, -1.35562618f, 0.0f, 1.35562618f, 2.85697007f};
  const float mass[5] = {0.0112574113f, 0.222075922f, 0.533333333f, 0.222075922f,
                         0.0112574113f};
  float mu = 0.0f, second = 0.0f;
#pragma unroll
  for (int j = 0; j < 5; ++j) {
    const float a = pinned_activate(__fadd_rn(gb, __fmul_rn(nodes[j], sg)), activation);
    mu = __fadd_rn(mu, __fmul_rn(__fmul_rn(mass[j], a), ub));
    second = __fadd_rn(second, __fmul_rn(__fmul_rn(mass[j], __fmul_rn(a, a)), spread));
  }
  const float p = bf16_round(__fmul_rn(pinned_activate(gb, activation), ub));
  const float spread_error = fmaxf(__fsub_rn(second, __fmul_rn(mu, mu)), 0.0f);
  float risk = __fmul_rn(__fmul_rn(norm, norm), spread_error);
  const float along = __fsub_rn(__fmul_rn(norm, mu), __fmul_rn(alpha, p));
  const float across = __fmul_rn(beta, p);
  risk = __fadd_rn(risk, __fadd_rn(__fmul_rn(along, along), __fmul_rn(across, across)));
  return __fadd_rn(__fmul_rn(risk, __fmul_rn(w, w)), 0.0f);
}

// 16-byte read-only load that does not allocate in L1 (streamed weights).
__device__ __forceinline__ uint4 load_stream16(const void* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t load_stream4(const void* p) {
  uint32_t v;
  asm("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Two BF16 values packed in a 32-bit word -> two floats (exact).
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) {
  return __uint_as_float(w & 0xffff0000u);
}

// Programmatic dependent launch.  A kernel launched with programmatic stream
// serialisation may start while its predecessor in the stream is still running;
// grid_dependency_wait() returns once that predecessor has completed and its writes
// are visible, and must precede the first access to anything the predecessor wrote.
// grid_dependency_release() lets the successor of the calling grid be scheduled once
// every CTA of this grid has called it or exited.  Both do nothing in ordinary launches.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_release() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Exclusive scan of `value` over the CTA (blockDim.x a multiple of 32, at most
// 1024); `scratch` holds 33 ints.  Returns the sum of the earlier threads and
// writes the CTA total to `*total`.  Ends with a barrier.
__device__ __forceinline__ int block_exclusive_scan(int value, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  int scan = value;
#pragma unroll
  for (int w = 1; w < 32; w <<= 1) {
    const int o = __shfl_up_sync(kFull, scan, w);
    if (lane >= w) scan += o;
  }
  __syncthreads();  // earlier users of the scratch are done
  if (lane == 31) scratch[warp] = scan;
  __syncthreads();
  if (warp == 0) {
    int t = lane < warps ? scratch[lane] : 0;
#pragma unroll
    for (int w = 1; w < 32; w <<= 1) {
      const int o = __shfl_up_sync(kFull, t, w);
      if (lane >= w) t += o;
    }
    scratch[lane] = t;  // inclusive scan of the warp totals
  }
  __syncthreads();
  *total = scratch[warps - 1];
  return scan - value + (warp ? scratch[warp - 1] : 0);
}

}  // namespace cfm
