// Expert-parallel dispatch of the kept-channel lists and combine of the partial
// output rows over peer memory (NVLink / NVSwitch), sm_100a.
//
// Every rank owns one exchange block in its own HBM that all ranks of the box
// have mapped (CUDA IPC).  Layout, identical on all ranks (P ranks, T tokens per
// rank and step, F kept channels, H columns):
//
//   header   256 x u32   [0] epoch of the last finished step, [1] arrivals of the
//                        finish kernel, [2] status (non-zero: a wait ran out),
//                        [16 + p] lists of rank p have landed for this epoch,
//                        [32 + p] rows of owner p have landed for this epoch,
//                        [48 + p], [64 + p] arrival counters of this rank's own
//                        sending CTAs (lists, rows), per destination
//   lists    i32 [P][T][F]  kept-channel lists of every rank's tokens
//   rows     f32 [P][T][H]  per owner rank, its partial output rows of THIS
//                           rank's tokens
//
// One layer call is one epoch.  The home rank of a token stores its kept list
// into every rank's `lists` (the tail of k_select when the call carries the
// exchange); owners wait for the lists they adopt
// (k_adopt), compute, and store each token's partial output row straight into
// slot [owner] of the home rank's `rows` (k_partial_output); the home rank waits
// for all owners' rows and adds them in rank order (k_finish_rows), so the sum
// does not depend on arrival order.  Data is written with plain peer stores,
// made visible with a system-scope fence, and announced by the last CTA to
// arrive with a release store of the epoch into the destination's flag; readers
// poll their own flag with acquire loads and read the data past L1.  Every wait
// is bounded (about a second); when one runs out the kernel records it in the
// local status word and goes on with whatever is there, so no launch can hang.
// Included by cfm_reader.cu inside namespace cfm.
#pragma once

constexpr int kExchangeHeaderWords = 256;
constexpr int kExchangeEpoch = 0, kExchangeFinished = 1, kExchangeStatus = 2;
constexpr int kExchangeListsFlag = 16, kExchangeRowsFlag = 32;
constexpr int kExchangeListsArrive = 48, kExchangeRowsArrive = 64;
constexpr long long kExchangeWaitCycles = 2000000000LL;

struct Exchange {  // device-visible copy of cfm_exchange
  int world, rank, tokens;
  char* block[CFM_MAX_RANKS];
};

__host__ __device__ inline size_t exchange_lists_offset() {
  return sizeof(uint32_t) * kExchangeHeaderWords;
}
__host__ __device__ inline size_t exchange_rows_offset(int world, int tokens, int F) {
  const size_t lists = sizeof(int32_t) * static_cast<size_t>(world) * tokens * F;
  return exchange_lists_offset() + (lists + 255) / 256 * 256;
}
__host__ __device__ inline size_t exchange_bytes(int world, int tokens, int F, int H) {
  return exchange_rows_offset(world, tokens, F) +
         sizeof(float) * static_cast<size_t>(world) * tokens * H;
}

__device__ __forceinline__ uint32_t* exchange_header(const Exchange& x, int rank) {
  return reinterpret_cast<uint32_t*>(x.block[rank]);
}

__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void store_release_system(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until *flag reaches `epoch` (flags only grow).  One thread calls it.
// Returns false, after recording it in `status`, when the wait ran out.
__device__ __forceinline__ bool exchange_wait(const uint32_t* flag, uint32_t epoch,
                                              uint32_t* status, uint32_t what) {
  const long long start = clock64();
  for (;;) {
    // Signed distance: correct across the wrap of the 32-bit epoch.
    if (static_cast<int32_t>(load_acquire_system(flag) - epoch) >= 0) return true;
    if (clock64() - start > kExchangeWaitCycles) {
      atomicOr(status, what);
      return false;
    }
    __nanosleep(64);
  }
}

// All threads of the CTA call this after their peer stores.  The last CTA of
// `expected` to arrive at `counter` (local memory) announces `epoch` at `flag`
// (the destination's memory).
__device__ __forceinline__ void exchange_announce(uint32_t* counter, unsigned expected,
                                                  uint32_t* flag, uint32_t epoch) {
  // The CTA barrier orders every thread's stores before thread 0's system-scope fence,
  // which is cumulative: one fence per CTA publishes them all.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned old = atomicAdd(counter, 1u);
    if (old == expected - 1) {
      *counter = 0;
      __threadfence_system();
      store_release_system(flag, epoch);
    }
  }
}

// grid (H / 128, T), 128 threads: the home rank's output rows.  Waits for the
// partial rows of all owners, adds them in rank order, adds the decoder term of
// the home rank's own latent and stores BF16.  The last CTA closes the epoch.
__global__ void __launch_bounds__(128) k_finish_rows(Layer L, Exchange x, const float* latent_rows,
                                                     __nv_bfloat16* out) {
  __shared__ float latent[256];
  const int t = blockIdx.y, tid = threadIdx.x, h = blockIdx.x * 128 + tid;
  uint32_t* header = exchange_header(x, x.rank);
  const uint32_t epoch = header[kExchangeEpoch] + 1u;
  if (tid < x.world)
    exchange_wait(header + kExchangeRowsFlag + tid, epoch, header + kExchangeStatus, 2u);
  const bool recover = L.R > 0 && L.decoder && latent_rows;
  if (recover)
    for (int r = tid; r < L.R; r += 128)
      latent[r] = bf16_round(latent_rows[static_cast<size_t>(t) * L.R + r]);
  __syncthreads();
  const float* rows = reinterpret_cast<const float*>(
      x.block[x.rank] + exchange_rows_offset(x.world, x.tokens, L.F));
  float routed = 0.0f;
  for (int p = 0; p < x.world; ++p)
    routed += __ldcg(rows + (static_cast<size_t>(p) * x.tokens + t) * L.H + h);
  float correction = 0.0f;
  if (recover) {
    const uint4* row = reinterpret_cast<const uint4*>(L.decoder + static_cast<size_t>(h) * L.R);
    float dot = 0.0f;
    for (int i = 0; i < L.R / 8; ++i) {
      const uint4 w = row[i];
      const float* z = latent + i * 8;
      dot = fmaf(bf16_lo(w.x), z[0], dot);
      dot = fmaf(bf16_hi(w.x), z[1], dot);
      dot = fmaf(bf16_lo(w.y), z[2], dot);
      dot = fmaf(bf16_hi(w.y), z[3], dot);
      dot = fmaf(bf16_lo(w.z), z[4], dot);
      dot = fmaf(bf16_hi(w.z), z[5], dot);
      dot = fmaf(bf16_lo(w.w), z[6], dot);
      dot = fmaf(bf16_hi(w.w), z[7], dot);
    }
    correction = bf16_round(dot);
  }
  out[static_cast<size_t>(t) * L.H + h] = __float2bfloat16_rn(routed + correction);
  // Every CTA has read the epoch by now; the last one to finish closes it.
  __syncthreads();
  if (tid == 0) {
    const unsigned all = gridDim.x * gridDim.y;
    const unsigned old = atomicAdd(header + kExchangeFinished, 1u);
    if (old == all - 1) {
      header[kExchangeFinished] = 0;
      __threadfence();
      header[kExchangeEpoch] = epoch;
    }
  }
}
