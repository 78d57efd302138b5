// Construction-time kernel: the ternary sketch of the native gate/up rows,
// written straight into the two layouts the screen kernels read (sm_100a).
//
// Per expert, row and 128-coordinate rotation block (reference
// reader/sketch.py:84-150): rotate the row's block (signs, seven butterfly
// stages, 1/sqrt(128)); a coordinate keeps its sign when |v| > 0.7 mean|v|; the
// block's scale is the mean magnitude of the kept coordinates (over max(count,
// 1)), its residual variance mean((v - sign scale)^2); both stored FP16.
//
// One warp per (row, block), lane l holding coordinates 4 l .. 4 l + 3; a CTA of
// sixteen warps takes sixteen consecutive rows of one block, so that it can
// assemble the coordinate-major words (sixteen rows per 32-bit word) in shared
// memory.  The rotation is the reference's butterfly, bit for bit.  The three
// reductions over a block's 128 values (sum of magnitudes, sum of kept
// magnitudes, sum of squared residuals) are FP32 sums in a fixed order of their
// own (four values per lane, then a lane butterfly), which is not the order of a
// torch reduction: a coordinate whose magnitude sits within rounding of the
// threshold can come out differently from the reference builder's, and a scale
// can differ in its last FP16 bit.  The readers take either sketch; parity tests
// use the reference builder's.  Included by cfm_reader.cu inside namespace cfm.
#pragma once

constexpr int kBuildRows = 16;  // rows per CTA = rows per coordinate-major word

// Bit position of coordinate c (0..15) of a word of the row-major layout: four
// masked shifts of the word give the byte-permute selectors of coordinates 0-3,
// 4-7, 8-11 and 12-15 (see decode_word).
__device__ __forceinline__ int grouped_bit(int c) {
  return c < 4 ? 4 * c : c < 8 ? 4 * (c - 4) + 2 : c < 12 ? 16 + 4 * (c - 8) : 18 + 4 * (c - 12);
}

// grid (B, 2I / 16, E), 512 threads.
__global__ void __launch_bounds__(kBuildRows * 32)
    k_build_sketch(int H, int I, const __nv_bfloat16* gate_up, const int8_t* signs,
                   uint32_t* words, uint32_t* grouped, __half* statistics) {
  __shared__ uint8_t code[kBuildRows][kBlock];  // trit + 1 of every (row, coordinate)
  const int b = blockIdx.x, group = blockIdx.y, e = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rows = 2 * I, B = H / kBlock;
  const int row = group * kBuildRows + warp;
  // ---- load and rotate: lane holds coordinates 4 lane .. 4 lane + 3 ----
  const __nv_bfloat16* source =
      gate_up + (static_cast<size_t>(e) * rows + row) * H + b * kBlock + 4 * lane;
  const uint2 raw = *reinterpret_cast<const uint2*>(source);
  const char4 sign = *reinterpret_cast<const char4*>(signs + b * kBlock + 4 * lane);
  float v[4] = {__fmul_rn(bf16_lo(raw.x), static_cast<float>(sign.x)),
                __fmul_rn(bf16_hi(raw.x), static_cast<float>(sign.y)),
                __fmul_rn(bf16_lo(raw.y), static_cast<float>(sign.z)),
                __fmul_rn(bf16_hi(raw.y), static_cast<float>(sign.w))};
  {  // half-widths 1 and 2 inside the lane: the lower member takes the sum
    float a = __fadd_rn(v[0], v[1]), d = __fsub_rn(v[0], v[1]);
    float c = __fadd_rn(v[2], v[3]), f = __fsub_rn(v[2], v[3]);
    v[0] = __fadd_rn(a, c);
    v[2] = __fsub_rn(a, c);
    v[1] = __fadd_rn(d, f);
    v[3] = __fsub_rn(d, f);
  }
#pragma unroll
  for (int w = 1; w < 32; w <<= 1) {  // half-widths 4 .. 64 across lanes
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(kFull, v[i], w);
      v[i] = (lane & w) ? __fsub_rn(o, v[i]) : __fadd_rn(v[i], o);
    }
  }
  float size[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = __fmul_rn(v[i], 0.0883883461f);  // float(1 / sqrt(128))
    size[i] = fabsf(v[i]);
  }
  auto warp_sum = [&](float x) {
#pragma unroll
    for (int w = 16; w; w >>= 1) x = __fadd_rn(x, __shfl_xor_sync(kFull, x, w));
    return x;
  };
  // ---- ternary weight network rule ----
  const float mean =
      __fdiv_rn(warp_sum(__fadd_rn(__fadd_rn(size[0], size[1]), __fadd_rn(size[2], size[3]))),
                128.0f);
  const float cut = __fmul_rn(0.7f, mean);
  float kept_sum = 0.0f;
  int kept = 0;
  float trit[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool member = size[i] > cut;
    trit[i] = member ? (v[i] > 0.0f ? 1.0f : v[i] < 0.0f ? -1.0f : 0.0f) : 0.0f;
    kept_sum = __fadd_rn(kept_sum, member ? size[i] : 0.0f);
    kept += member;
  }
  kept_sum = warp_sum(kept_sum);
#pragma unroll
  for (int w = 16; w; w >>= 1) kept += __shfl_xor_sync(kFull, kept, w);
  const float scale = __fdiv_rn(kept_sum, static_cast<float>(max(kept, 1)));
  float residual = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float d = __fsub_rn(v[i], __fmul_rn(trit[i], scale));
    residual = __fadd_rn(residual, __fmul_rn(d, d));
  }
  residual = __fdiv_rn(warp_sum(residual), 128.0f);
  if (lane == 0) {
    __half* plane = statistics + (static_cast<size_t>(e) * B + b) * 2 * rows + row;
    plane[0] = __float2half_rn(scale);
    plane[rows] = __float2half_rn(residual);
  }
  // ---- row-major layout: the row's 128 coordinates of this block in eight words ----
  uint32_t part = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t c = static_cast<uint32_t>(static_cast<int>(trit[i]) + 1);
    code[warp][4 * lane + i] = static_cast<uint8_t>(c);
    part |= c << grouped_bit(4 * (lane & 3) + i);
  }
  part |= __shfl_xor_sync(kFull, part, 1);
  part |= __shfl_xor_sync(kFull, part, 2);
  if ((lane & 3) == 0)
    grouped[((static_cast<size_t>(e) * B + b) * rows + row) * 8 + (lane >> 2)] = part;
  __syncthreads();
  // ---- coordinate-major layout: one word per coordinate holds the CTA's sixteen rows ----
  if (tid < kBlock) {
    uint32_t word = 0;
#pragma unroll
    for (int r = 0; r < kBuildRows; ++r) word |= static_cast<uint32_t>(code[r][tid]) << (2 * r);
    words[(static_cast<size_t>(e) * H + b * kBlock + tid) * (rows / kBuildRows) + group] = word;
  }
}
