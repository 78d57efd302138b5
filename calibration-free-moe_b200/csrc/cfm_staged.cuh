// Expert-major screen whose sketch operand is staged in shared memory by bulk
// asynchronous copies (sm_100a).  Same arithmetic as k_screen_grouped: int8 trits x
// int8 digits on the m16n8k32 tensor-core path, exact int32 block dots, the
// per-block FP32 rescale in block order; results are bit-identical.
//
// What differs is how the 2-bit codes and FP16 scales reach the warps.  Loading
// them into registers one rotation block ahead keeps about 9 KB per SM in flight,
// which bounds the kernel near 1.4 TB/s whatever else it does.  Here thread 0 of a
// CTA issues, up front, one bulk copy per rotation block for the CTA's 128 rows
// (4 KiB of codes, 256 bytes of scales; both contiguous in the row-major layout),
// each completing on its own mbarrier, so a CTA has up to 68 KiB in flight and the
// warps find a block's operand in shared memory when they get to it.  With B <= 16
// rotation blocks every block keeps its own stage: experts with more than eight
// tokens run their further passes from shared memory.  Wider layers reuse the
// sixteen stages as a ring (one CTA barrier per block hands a stage back).
//
// Every mbarrier wait is bounded (about a second); a wait that runs out sets
// status[0] and the CTA leaves.  Included by cfm_reader.cu inside namespace cfm.
#pragma once

namespace staged {

constexpr int kWarps = 8;                  // 16 sketch rows per warp
constexpr int kRows = kWarps * 16;         // rows per CTA
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 16;
constexpr int kCodeBytes = kRows * 32;     // 128 two-bit codes per row
constexpr int kScaleBytes = kRows * 2;     // FP16 scale per row
constexpr int kStageBytes = kCodeBytes + kScaleBytes;
constexpr size_t kSharedBytes = static_cast<size_t>(kStages) * kStageBytes + kStages * 8 + 16;

__device__ __forceinline__ void expect_bytes(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

// Bulk copy global -> shared memory of this CTA, completing `bytes` on `bar`.
// Both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t destination, const void* source, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          destination),
      "l"(source), "r"(bytes), "r"(bar)
      : "memory");
}

}  // namespace staged

// grid (ceil(2I / 128), E, passes), 256 threads, dynamic shared memory
// staged::kSharedBytes.  `L.sketch_grouped` and `L.statistics` 16-byte aligned.
__global__ void __launch_bounds__(staged::kThreads, 2) k_screen_staged(Layer L, Workspace ws) {
  using namespace staged;
  extern __shared__ __align__(128) uint8_t staged_shared[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(staged_shared + kStages * kStageBytes);
  volatile int* abort = reinterpret_cast<volatile int*>(bars + kStages);
  const int e = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int first = ws.group_offsets[e], total = ws.group_offsets[e + 1] - first;
  const int rows = 2 * L.I, B = L.B;
  const int cta_row = blockIdx.x * kRows;
  const int start = 8 * blockIdx.z, stride = 8 * gridDim.z;
  if (start >= total) return;  // the whole CTA: nothing of this expert for it
  const int passes = (total - start + stride - 1) / stride;
  const int cta_rows = min(kRows, rows - cta_row);  // a multiple of 32
  const bool resident = B <= kStages;               // every block has a stage of its own
  const int copies = resident ? B : passes * B;     // bulk-copy pairs this CTA issues in all

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) tc::barrier_init(tc::shared_address(bars + s), 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const uint8_t* code_source = reinterpret_cast<const uint8_t*>(L.sketch_grouped) +
                               (static_cast<size_t>(e) * B * rows + cta_row) * 32;
  const __half* scale_source = L.statistics + static_cast<size_t>(e) * B * 2 * rows + cta_row;
  auto issue = [&](int q) {  // thread 0: the operand of rotation block q mod B into stage q mod 16
    const int b = q % B, stage = q % kStages;
    const uint32_t bar = tc::shared_address(bars + stage);
    const uint32_t destination = tc::shared_address(staged_shared + stage * kStageBytes);
    const uint32_t code_bytes = cta_rows * 32, scale_bytes = cta_rows * 2;
    expect_bytes(bar, code_bytes + scale_bytes);
    bulk_load(destination, code_source + static_cast<size_t>(b) * rows * 32, code_bytes, bar);
    bulk_load(destination + kCodeBytes, scale_source + static_cast<size_t>(b) * 2 * rows,
              scale_bytes, bar);
  };
  if (tid == 0)
    for (int q = 0; q < min(copies, kStages); ++q) issue(q);

  const int r0 = warp * 16;                 // first row of this warp inside the CTA
  const bool active = r0 < cta_rows;        // whole warps are in or out
  if (resident && !active) return;          // no CTA barrier below in that mode
  const int row_a = cta_row + r0 + g, row_b = row_a + 8;

  struct DigitFetch {
    uint4 digit[3][2];  // this lane's 32 coordinates of the three digits of token g
    float unscale[2];   // 2^(e - 21) of the two tokens this lane finishes
  };
  int q = 0;
  bool failed = false;
  for (int base = start; base < total && !failed; base += stride) {
    const int count = min(8, total - base);
    const int pair_g = g < count ? ws.group_pairs[first + base + g] : -1;
    const int pair_0 = __shfl_sync(kFull, pair_g, (2 * tq) * 4);
    const int pair_1 = __shfl_sync(kFull, pair_g, (2 * tq + 1) * 4);
    const uint4* next_digits = reinterpret_cast<const uint4*>(
        (pair_g >= 0 ? ws.limbs + static_cast<size_t>(pair_g / L.K) * B * 3 * kBlock
                     : ws.zero_limbs) + 32 * tq);
    const float* next_unscale_0 = ws.unscales + static_cast<size_t>(max(pair_0, 0) / L.K) * B;
    const float* next_unscale_1 = ws.unscales + static_cast<size_t>(max(pair_1, 0) / L.K) * B;
    auto fetch = [&]() {
      DigitFetch f;
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        f.digit[j][0] = next_digits[j * (kBlock / 16)];
        f.digit[j][1] = next_digits[j * (kBlock / 16) + 1];
      }
      f.unscale[0] = *next_unscale_0++;
      f.unscale[1] = *next_unscale_1++;
      next_digits += 3 * kBlock / 16;
      return f;
    };
    float run[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // One rotation block: wait for its stage, multiply, rescale; in ring mode hand the
    // stage back and let thread 0 refill it.
    auto block = [&](const DigitFetch& cur) {
      const int stage = q % kStages;
      const uint32_t parity = resident ? 0u : static_cast<uint32_t>(q / kStages) & 1u;
      const bool ready = tc::barrier_wait(tc::shared_address(bars + stage), parity, abort);
      if (ready && active) {
        const uint8_t* codes = staged_shared + stage * kStageBytes;
        const uint2 word_a = *reinterpret_cast<const uint2*>(codes + (r0 + g) * 32 + tq * 8);
        const uint2 word_b = *reinterpret_cast<const uint2*>(codes + (r0 + g + 8) * 32 + tq * 8);
        const __half* scales = reinterpret_cast<const __half*>(codes + kCodeBytes);
        const float scale_a = __half2float(scales[r0 + g]);
        const float scale_b = __half2float(scales[r0 + g + 8]);
        uint32_t fa[8], fb[8];
        decode_word(word_a.x, fa[0], fa[1], fa[2], fa[3]);
        decode_word(word_a.y, fa[4], fa[5], fa[6], fa[7]);
        decode_word(word_b.x, fb[0], fb[1], fb[2], fb[3]);
        decode_word(word_b.y, fb[4], fb[5], fb[6], fb[7]);
        int acc[3][4];
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const uint4 lo = cur.digit[j][0], hi = cur.digit[j][1];
          mma_s8_first(acc[j], fa[0], fb[0], fa[1], fb[1], lo.x, lo.y);
          mma_s8(acc[j], fa[2], fb[2], fa[3], fb[3], lo.z, lo.w);
          mma_s8(acc[j], fa[4], fb[4], fa[5], fb[5], hi.x, hi.y);
          mma_s8(acc[j], fa[6], fb[6], fa[7], fb[7], hi.z, hi.w);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int dot = acc[0][i] + acc[1][i] * 256 + acc[2][i] * 65536;
          const float d = __fmul_rn(__int2float_rn(dot), cur.unscale[i & 1]);
          run[i] = __fadd_rn(run[i], __fmul_rn(i < 2 ? scale_a : scale_b, d));
        }
      }
      if (!resident) {
        // Every warp is done with this stage, or some warp gave up: the same answer for all.
        failed = __syncthreads_or(!ready);
        if (tid == 0 && !failed && q + kStages < copies) issue(q + kStages);
      } else if (!ready) {
        failed = true;
      }
      ++q;
    };
    DigitFetch even = fetch(), odd;
    for (int b = 0; b < B && !failed; b += 2) {
      if (b + 1 < B) odd = fetch();
      block(even);
      if (b + 2 < B) even = fetch();
      if (b + 1 < B && !failed) block(odd);
    }
    if (resident) q = 0;  // further passes read the same stages again
    if (failed || !active) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int pair = (i & 1) ? pair_1 : pair_0;
      if (pair < 0) continue;
      const int row = (i < 2) ? row_a : row_b;
      const int t = pair / L.K, slot = pair - t * L.K;
      float* out = ws.partial + static_cast<size_t>(t) * 2 * L.N + static_cast<size_t>(slot) * L.I;
      (row < L.I ? out[row] : out[L.N + row - L.I]) = run[i];
    }
  }
  if (failed && lane == 0) atomicExch(&ws.status[0], 1);
}
