// Expert-major screen, two 16-row tiles per warp (sm_100a).  Same arithmetic as
// k_screen_grouped (int8 trits x int8 digits on the m16n8k32 tensor-core path,
// exact int32 block dots, the per-block FP32 rescale in block order): results are
// bit-identical.  What differs is the work a warp shares and how its operands
// arrive:
//
//   * a warp owns 32 sketch rows (tiles X: rows g, g + 8 and Y: rows g + 16,
//     g + 24 of its range), so the digit fragments of the expert's tokens, their
//     exponents and all address arithmetic are loaded once for two tiles, and the
//     two tiles give the scheduler two independent decode / MMA / rescale chains;
//   * at its start a warp asks L2 for the codes and scales of all its rotation
//     blocks (one bulk prefetch of 1 KiB and one of 64 bytes per block, issued by
//     lanes 0 .. B-1), so the register loads, one block ahead, find them in L2 and
//     the HBM latency of the sketch stream is paid once per warp, not per block;
//   * the scales travel with the codes; digits and exponents are loaded at the top
//     of the block that uses them (L1 hits; the decode of the codes covers their
//     latency), which keeps the registers for two tiles' fragments and accumulators.
//
// grid (ceil(2I / 128), E, passes), 128 threads, no shared memory, no barrier.  Included by cfm_reader.cu inside namespace cfm.
#pragma once

// Asks L2 for `bytes` (a multiple of 16) from `p` (16-byte aligned); no data returns.
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

constexpr int kRows32Warps = 4;  // 128 rows per CTA, four CTAs per SM

__global__ void __launch_bounds__(kRows32Warps * 32, 16 / kRows32Warps)
    k_screen_rows32(Layer L, Workspace ws) {
  grid_dependency_release();  // the selection may be scheduled; it waits for this grid
  constexpr int kRows = kRows32Warps * 32;  // rows per CTA
  const int e = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int first = ws.group_offsets[e], total = ws.group_offsets[e + 1] - first;
  const int rows = 2 * L.I, B = L.B;
  const int r0 = blockIdx.x * kRows + warp * 32;
  if (total == 0 || r0 >= rows) return;  // whole warps are in or out: 2I is a multiple of 32
  if (8 * static_cast<int>(blockIdx.z) >= total) return;
  const size_t row_words = kBlock / 32;  // uint2 per row and block
  const size_t block_words = static_cast<size_t>(rows) * row_words;
  const uint2* codes = reinterpret_cast<const uint2*>(L.sketch_grouped) +
                       (static_cast<size_t>(e) * B * rows + r0) * row_words;
  const __half* scales = L.statistics + static_cast<size_t>(e) * B * 2 * rows + r0;
  for (int b = lane; b < B; b += 32) {
    prefetch_l2(codes + b * block_words, 32 * 32);
    prefetch_l2(scales + static_cast<size_t>(b) * 2 * rows, 32 * 2);
  }
  codes += g * row_words + tq;
  scales += g;

  for (int base = 8 * blockIdx.z; base < total; base += 8 * gridDim.z) {
    const int count = min(8, total - base);
    // Pair of the token whose digits this lane feeds (column g of the tiles).
    const int pair_g = g < count ? ws.group_pairs[first + base + g] : -1;
    // Pairs of the two tokens whose results this lane finishes.
    const int pair_0 = __shfl_sync(kFull, pair_g, (2 * tq) * 4);
    const int pair_1 = __shfl_sync(kFull, pair_g, (2 * tq + 1) * 4);
    const uint2* next_codes = codes;
    const __half* scale = scales;
    const uint4* digits = reinterpret_cast<const uint4*>(
        (pair_g >= 0 ? ws.limbs + static_cast<size_t>(pair_g / L.K) * B * 3 * kBlock
                     : ws.zero_limbs) + 32 * tq);
    const float* unscale_0 = ws.unscales + static_cast<size_t>(max(pair_0, 0) / L.K) * B;
    const float* unscale_1 = ws.unscales + static_cast<size_t>(max(pair_1, 0) / L.K) * B;
    struct Words {
      uint2 row[4];     // 32 coordinates of rows g, g + 8, g + 16, g + 24
      __half scale[4];  // and the block scales of those rows
    };
    auto fetch = [&]() {
      Words w;
#pragma unroll
      for (int i = 0; i < 4; ++i) w.row[i] = next_codes[i * 8 * row_words];
      next_codes += block_words;
#pragma unroll
      for (int i = 0; i < 4; ++i) w.scale[i] = scale[8 * i];
      scale += 2 * rows;
      return w;
    };
    float run[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    auto compute = [&](const Words& cur) {
      uint4 digit[3][2];
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        digit[j][0] = digits[j * (kBlock / 16)];
        digit[j][1] = digits[j * (kBlock / 16) + 1];
      }
      const float unscale[2] = {*unscale_0++, *unscale_1++};
      digits += 3 * kBlock / 16;
#pragma unroll
      for (int tile = 0; tile < 2; ++tile) {
        uint32_t fa[8], fb[8];
        decode_word(cur.row[2 * tile].x, fa[0], fa[1], fa[2], fa[3]);
        decode_word(cur.row[2 * tile].y, fa[4], fa[5], fa[6], fa[7]);
        decode_word(cur.row[2 * tile + 1].x, fb[0], fb[1], fb[2], fb[3]);
        decode_word(cur.row[2 * tile + 1].y, fb[4], fb[5], fb[6], fb[7]);
        int acc[3][4];
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const uint4 lo = digit[j][0], hi = digit[j][1];
          mma_s8_first(acc[j], fa[0], fb[0], fa[1], fb[1], lo.x, lo.y);
          mma_s8(acc[j], fa[2], fb[2], fa[3], fb[3], lo.z, lo.w);
          mma_s8(acc[j], fa[4], fb[4], fa[5], fb[5], hi.x, hi.y);
          mma_s8(acc[j], fa[6], fb[6], fa[7], fb[7], hi.z, hi.w);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int dot = acc[0][i] + acc[1][i] * 256 + acc[2][i] * 65536;
          const float d = __fmul_rn(__int2float_rn(dot), unscale[i & 1]);
          run[4 * tile + i] = __fadd_rn(
              run[4 * tile + i], __fmul_rn(__half2float(cur.scale[2 * tile + (i >> 1)]), d));
        }
      }
    };
    // Two code buffers used in turn: while one block computes, the next block's
    // codes are on their way from L2.
    Words even = fetch(), odd;
    for (int b = 0; b < B; b += 2) {
      if (b + 1 < B) odd = fetch();
      compute(even);
      if (b + 2 < B) even = fetch();
      if (b + 1 < B) compute(odd);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int pair = (i & 1) ? pair_1 : pair_0;
      if (pair < 0) continue;
      const int row = r0 + g + 8 * (2 * (i >> 2) + ((i >> 1) & 1));
      const int t = pair / L.K, slot = pair - t * L.K;
      float* out = ws.partial + static_cast<size_t>(t) * 2 * L.N + static_cast<size_t>(slot) * L.I;
      (row < L.I ? out[row] : out[L.N + row - L.I]) = run[i];
    }
  }
}
