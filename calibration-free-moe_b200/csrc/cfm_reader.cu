// Sparse MoE decode reader for B200 (sm_100a): kernels and C ABI.
//
// One call processes T decode tokens of one MoE layer:
//   prepare  rotate the input (block Hadamard), keep the KEEP largest rotated
//            coordinates per 128-block, make a fixed-point copy of them
//   route    sort each token's K experts ascending, map to local ids
//   screen   exact integer dot products of the 2-bit ternary sketch with the
//            fixed-point rotated input -> projections -> selection scores
//   select   per token the F best scores (radix select), ties to the lower
//            candidate index; read-cost counters
//   exact    gathered BF16 gate/up rows of the kept channels, phi(g) * u
//   down     gathered channel-major down rows of the kept channels
//   encode   low-rank recovery encoder over the skipped channels
//   output   router-weighted mix + decoder term, BF16 store
//
// Selection depends only on integer dot products and pinned FP32 operations
// (see cfm_device.cuh), so it does not change with batch size, split count or
// launch shape.  No kernel waits on another: cross-CTA reductions use the
// "last CTA to arrive finishes" pattern with an atomic counter and no spin.
#include "cfm_device.cuh"

#include "cfm_b200.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <mutex>

namespace cfm {

// ---------------------------------------------------------------------------
// Workspace binding
// ---------------------------------------------------------------------------
struct Workspace {
  int32_t* ids;
  float* weights;
  float* norms;
  float* planes;
  int32_t* coordinates;
  int32_t* quantized;
  int32_t* exponents;
  float* parts;
  uint32_t* counters;
  float* partial;
  float* scores;
  uint8_t* selected;
  uint8_t* completed;
  int32_t* candidate_ids;
  int32_t* counts;
  int32_t* starts;
  int32_t* tile_starts;
  __nv_bfloat16* activations;
  float* exact;
  float* down_parts;
  float* encoder_parts;
  float* latent;
  int32_t* status;
  int8_t* limbs;
  int32_t* group_offsets;
  int32_t* group_pairs;
  int32_t* cuts;
  float* variances;
  float* unscales;
  int8_t* zero_limbs;
  int32_t* tile_list;
  int32_t* tile_count;
  int32_t parts_tokens;
  int32_t down_tiles;
  int32_t encoder_tiles;
  int32_t capacity;
};

struct Layer {  // device-visible copy of cfm_layer with typed pointers
  int H, I, E, K, F, KEEP, R, activation, score, global_experts, owner, tensor_engine, row_engine;
  int B, N, W;  // blocks, candidates, sketch words per coordinate
  uint32_t width_magic;  // floor(2^32 / I) + 1, or 0 where the multiplication is not exact
  const __nv_bfloat16* gate_up;
  const __nv_bfloat16* down;
  const uint32_t* sketch;
  const uint32_t* sketch_grouped;
  const __half* statistics;
  const float* norms;
  const float* geometry;
  const __nv_bfloat16* encoder;
  const __nv_bfloat16* decoder;
  const int8_t* signs;
  const int32_t* expert_map;
  double* read_work;
  const float* threshold;  // device scalar of the threshold mode, or nullptr
};

// Slot of candidate i, i / I, by multiplication where that is exact for the layer.
__device__ __forceinline__ int slot_of(const Layer& L, int i) {
  return L.width_magic ? static_cast<int>(__umulhi(static_cast<uint32_t>(i), L.width_magic))
                       : i / L.I;
}

// Score of candidate i (slot's channel c of local expert e) of token t; defined with the select kernel.
__device__ __forceinline__ float candidate_score(const Layer& L, const Workspace& ws, int t, int i,
                                                 int e, int c, float weight);

static int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

// Most partial sums per (token, slot) the expert-major down kernel writes.
constexpr int64_t kDownGroupedMaxParts = 8;

// Most candidates per token (N = K * I) the selection kernels take: their scans pack two
// counts of at most N into the halves of one 32-bit integer.
constexpr int64_t kMaxCandidates = 32767;

static int make_layout(const cfm_layer* l, int32_t capacity, cfm_workspace_layout* o) {
  if (!l || !o) return CFM_E_NULL;
  const int64_t H = l->hidden, I = l->width, K = l->top_k, F = l->final_count;
  const int64_t KEEP = l->keep, R = l->rank, C = capacity;
  if (H <= 0 || H % kBlock || I <= 0 || I % 16 || K <= 0 || K > 32 || KEEP < 1 ||
      KEEP > kBlock || R < 0 || R > 256 || (R % 8) || (R && (256 % R)) || F < 1 ||
      F > K * I || K * I > kMaxCandidates)
    return CFM_E_SHAPE;
  if (C < 1) return CFM_E_CAPACITY;
  const int64_t B = H / kBlock, N = K * I;
  int64_t at = 0;
  auto take = [&](int64_t bytes) {
    const int64_t here = at;
    at = align256(at + bytes);
    return here;
  };
  o->parts_tokens = static_cast<int32_t>(C < 16 ? C : 16);
  o->down_tiles = static_cast<int32_t>(std::max<int64_t>(
      (F + kDownTileRows - 1) / kDownTileRows + K - 1, kDownGroupedMaxParts * K));
  o->encoder_tiles = static_cast<int32_t>((I + kEncodeTileRows - 1) / kEncodeTileRows);
  o->reserved = 0;
  o->ids = take(4 * C * K);
  o->weights = take(4 * C * K);
  o->norms = take(4 * C * B);
  o->planes = take(4 * C * B * KEEP);
  o->coordinates = take(4 * C * B * KEEP);
  o->quantized = take(4 * C * B * KEEP);
  o->exponents = take(4 * C * B * 2);
  o->parts = take(4 * o->parts_tokens * K * B * 2 * I);
  o->counters = take(4 * (2 * C * K + 2 * C));
  o->partial = take(4 * C * 2 * N);
  o->scores = take(4 * C * N);
  o->selected = take(C * N);
  o->completed = take(C * N);
  o->candidate_ids = take(4 * C * F);
  o->counts = take(4 * C * K);
  o->starts = take(4 * C * K);
  o->tile_starts = take(4 * C * K);
  o->activations = take(2 * C * N);
  o->exact = take(4 * C * 2 * F);
  o->down_parts = take(4 * C * o->down_tiles * H);
  o->encoder_parts = take(4 * C * K * o->encoder_tiles * (R ? R : 1));
  o->latent = take(4 * C * (R ? R : 1));
  o->status = take(16);
  o->limbs = take(C * B * 3 * kBlock);
  o->group_offsets = take(4 * (static_cast<int64_t>(l->experts > 0 ? l->experts : 1) + 1));
  o->group_pairs = take(4 * C * K);
  o->cuts = take(4 * C * (K + 1));
  o->variances = take(4 * C * 2 * N);
  o->unscales = take(4 * C * B);
  o->zero_limbs = take(B * 3 * kBlock);
  o->tile_list = take(32 * C * ((F + kDownTileRows - 1) / kDownTileRows + K));
  o->tile_count = take(16);
  o->bytes = at;
  return 0;
}

static Workspace bind(const cfm_workspace_layout& o, void* base, int32_t capacity) {
  char* p = static_cast<char*>(base);
  Workspace w;
  w.ids = reinterpret_cast<int32_t*>(p + o.ids);
  w.weights = reinterpret_cast<float*>(p + o.weights);
  w.norms = reinterpret_cast<float*>(p + o.norms);
  w.planes = reinterpret_cast<float*>(p + o.planes);
  w.coordinates = reinterpret_cast<int32_t*>(p + o.coordinates);
  w.quantized = reinterpret_cast<int32_t*>(p + o.quantized);
  w.exponents = reinterpret_cast<int32_t*>(p + o.exponents);
  w.parts = reinterpret_cast<float*>(p + o.parts);
  w.counters = reinterpret_cast<uint32_t*>(p + o.counters);
  w.partial = reinterpret_cast<float*>(p + o.partial);
  w.scores = reinterpret_cast<float*>(p + o.scores);
  w.selected = reinterpret_cast<uint8_t*>(p + o.selected);
  w.completed = reinterpret_cast<uint8_t*>(p + o.completed);
  w.candidate_ids = reinterpret_cast<int32_t*>(p + o.candidate_ids);
  w.counts = reinterpret_cast<int32_t*>(p + o.counts);
  w.starts = reinterpret_cast<int32_t*>(p + o.starts);
  w.tile_starts = reinterpret_cast<int32_t*>(p + o.tile_starts);
  w.activations = reinterpret_cast<__nv_bfloat16*>(p + o.activations);
  w.exact = reinterpret_cast<float*>(p + o.exact);
  w.down_parts = reinterpret_cast<float*>(p + o.down_parts);
  w.encoder_parts = reinterpret_cast<float*>(p + o.encoder_parts);
  w.latent = reinterpret_cast<float*>(p + o.latent);
  w.status = reinterpret_cast<int32_t*>(p + o.status);
  w.limbs = reinterpret_cast<int8_t*>(p + o.limbs);
  w.group_offsets = reinterpret_cast<int32_t*>(p + o.group_offsets);
  w.group_pairs = reinterpret_cast<int32_t*>(p + o.group_pairs);
  w.cuts = reinterpret_cast<int32_t*>(p + o.cuts);
  w.variances = reinterpret_cast<float*>(p + o.variances);
  w.unscales = reinterpret_cast<float*>(p + o.unscales);
  w.zero_limbs = reinterpret_cast<int8_t*>(p + o.zero_limbs);
  w.tile_list = reinterpret_cast<int32_t*>(p + o.tile_list);
  w.tile_count = reinterpret_cast<int32_t*>(p + o.tile_count);
  w.parts_tokens = o.parts_tokens;
  w.down_tiles = o.down_tiles;
  w.encoder_tiles = o.encoder_tiles;
  w.capacity = capacity;
  return w;
}

static Layer device_layer(const cfm_layer* l) {
  Layer d;
  d.H = l->hidden;
  d.I = l->width;
  d.E = l->experts;
  d.K = l->top_k;
  d.F = l->final_count;
  d.KEEP = l->keep;
  d.R = l->rank;
  d.activation = l->activation;
  d.score = l->score;
  d.global_experts = l->global_experts;
  d.owner = l->recovery_owner;
  d.tensor_engine = l->tensor_engine;
  d.row_engine = l->row_engine;
  d.B = d.H / kBlock;
  d.N = d.K * d.I;
  d.W = 2 * d.I / kWordRows;
  // i / I == umulhi(i, magic) for every candidate i < N as long as N * I <= 2^32.
  const uint64_t width = static_cast<uint64_t>(d.I);
  d.width_magic = static_cast<uint64_t>(d.N) * width <= (1ull << 32)
                      ? static_cast<uint32_t>((1ull << 32) / width + 1) : 0u;
  d.gate_up = static_cast<const __nv_bfloat16*>(l->gate_up);
  d.down = static_cast<const __nv_bfloat16*>(l->down);
  d.sketch = l->sketch;
  d.sketch_grouped = l->sketch_grouped;
  d.statistics = static_cast<const __half*>(l->statistics);
  d.norms = l->norms;
  d.geometry = l->geometry;
  d.encoder = static_cast<const __nv_bfloat16*>(l->encoder);
  d.decoder = static_cast<const __nv_bfloat16*>(l->decoder);
  d.signs = l->signs;
  d.expert_map = l->expert_map;
  d.read_work = l->read_work;
  d.threshold = l->selection_threshold;
  return d;
}

#include "cfm_exchange.cuh"

// ---------------------------------------------------------------------------
// prepare: rotation, partial-screen mask, fixed-point copy
// ---------------------------------------------------------------------------
// grid (T, B), 128 threads: one thread per coordinate of one rotation block.
__global__ void __launch_bounds__(kBlock) k_prepare(Layer L, Workspace ws,
                                                    const __nv_bfloat16* hidden,
                                                    const uint8_t* padding) {
  const int t = blockIdx.x, b = blockIdx.y, c = threadIdx.x;
  if (padding && padding[t]) return;
  __shared__ float sm[kBlock];
  __shared__ int warp_i[4];
  __shared__ float warp_f[4];
  const int lane = c & 31, warp = c >> 5;

  const size_t at = static_cast<size_t>(t) * L.H + b * kBlock + c;
  float v = __fmul_rn(__bfloat162float(hidden[at]),
                      static_cast<float>(L.signs[b * kBlock + c]));
  // Butterfly, half-widths 1..64: the member with the bit clear takes the sum,
  // the member with the bit set takes (partner - own).
#pragma unroll
  for (int w = 1; w < 32; w <<= 1) {
    const float o = __shfl_xor_sync(kFull, v, w);
    v = (c & w) ? __fsub_rn(o, v) : __fadd_rn(v, o);
  }
#pragma unroll
  for (int w = 32; w < kBlock; w <<= 1) {
    sm[c] = v;
    __syncthreads();
    const float o = sm[c ^ w];
    __syncthreads();
    v = (c & w) ? __fsub_rn(o, v) : __fadd_rn(v, o);
  }
  v = __fmul_rn(v, 0.0883883461f);  // float(1 / sqrt(128))

  // Rank by magnitude, ties to the lower coordinate.
  const float a = fabsf(v);
  sm[c] = a;
  __syncthreads();
  bool kept = true;
  if (L.KEEP < kBlock) {
    int rank = 0;
#pragma unroll 8
    for (int j = 0; j < kBlock; ++j) {
      const float o = sm[j];
      rank += (o > a) || (o == a && j < c);
    }
    kept = rank < L.KEEP;
  }
  // Compact kept coordinates in ascending coordinate order.
  const unsigned ballot = __ballot_sync(kFull, kept);
  if (lane == 0) warp_i[warp] = __popc(ballot);
  // Block maximum magnitude (kept values are the largest, so this is theirs).
  float m = a;
#pragma unroll
  for (int w = 16; w; w >>= 1) m = fmaxf(m, __shfl_xor_sync(kFull, m, w));
  if (lane == 0) warp_f[warp] = m;
  __syncthreads();
  int position = __popc(ballot & ((1u << lane) - 1));
  for (int w = 0; w < warp; ++w) position += warp_i[w];
  m = fmaxf(fmaxf(warp_f[0], warp_f[1]), fmaxf(warp_f[2], warp_f[3]));
  __syncthreads();

  // Fixed point: q = rint(v * 2^(21 - e)), e = floor(log2 m) clamped to +-100.
  int e = static_cast<int>((__float_as_uint(m) >> 23) & 0xff) - 127;
  e = max(-100, min(100, e));
  int q = 0;
  float energy = 0.0f;
  if (kept) {
    const float scale = __uint_as_float(static_cast<uint32_t>(127 + kQuantBits - e) << 23);
    q = (m > 0.0f) ? __float2int_rn(__fmul_rn(v, scale)) : 0;
    q = max(-(1 << 22), min(1 << 22, q));
    energy = __fmul_rn(v, v);
    const size_t out = (static_cast<size_t>(t) * L.B + b) * L.KEEP + position;
    ws.planes[out] = v;
    ws.coordinates[out] = c;
    ws.quantized[out] = q;
  }
  {
    // Balanced base-256 digits of q (zero for dropped coordinates), in natural
    // coordinate order: q = l0 + 256 l1 + 65536 l2, each digit an int8.
    const int l0 = static_cast<int8_t>(q & 0xff);
    const int q1 = (q - l0) >> 8;
    const int l1 = static_cast<int8_t>(q1 & 0xff);
    const int l2 = (q1 - l1) >> 8;
    int8_t* limb = ws.limbs + (static_cast<size_t>(t) * L.B + b) * 3 * kBlock + c;
    limb[0] = static_cast<int8_t>(l0);
    limb[kBlock] = static_cast<int8_t>(l1);
    limb[2 * kBlock] = static_cast<int8_t>(l2);
  }
  int qsum = q;
#pragma unroll
  for (int w = 16; w; w >>= 1) qsum += __shfl_xor_sync(kFull, qsum, w);
  if (lane == 0) warp_i[warp] = qsum;
  sm[c] = energy;  // squares of the kept values, zero elsewhere
  __syncthreads();
  if (c == 0) {
    const size_t row = static_cast<size_t>(t) * L.B + b;
    ws.exponents[2 * row] = e;
    ws.exponents[2 * row + 1] = warp_i[0] + warp_i[1] + warp_i[2] + warp_i[3];
    ws.unscales[row] = __uint_as_float(static_cast<uint32_t>(127 + e - kQuantBits) << 23);
    // Energy of the kept coordinates, summed in coordinate order (pinned).
    float total = 0.0f;
    for (int j = 0; j < kBlock; ++j) total = __fadd_rn(total, sm[j]);
    ws.norms[row] = total;
  }
}

// ---------------------------------------------------------------------------
// route: stable ascending sort of a token's experts
// ---------------------------------------------------------------------------
// grid (T), 32 threads.
__global__ void __launch_bounds__(32) k_route(Layer L, Workspace ws, const void* ids,
                                              int ids64, const void* weights, int wbf16) {
  const int t = blockIdx.x, lane = threadIdx.x;
  long long id = 0x7fffffffffffffffLL;
  float w = 0.0f;
  if (lane < L.K) {
    const size_t at = static_cast<size_t>(t) * L.K + lane;
    id = ids64 ? static_cast<const long long*>(ids)[at]
               : static_cast<long long>(static_cast<const int32_t*>(ids)[at]);
    w = wbf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(weights)[at])
              : static_cast<const float*>(weights)[at];
  }
  int rank = 0;
  for (int j = 0; j < L.K; ++j) {
    const long long o = __shfl_sync(kFull, id, j);
    rank += (o < id) || (o == id && j < lane);
  }
  if (lane < L.K) {
    int local = -1;
    if (L.expert_map) {
      if (id >= 0 && id < L.global_experts) local = L.expert_map[id];
    } else if (id >= 0 && id < L.E) {
      local = static_cast<int>(id);
    }
    if (local >= L.E) local = -1;
    const size_t out = static_cast<size_t>(t) * L.K + rank;
    ws.ids[out] = local;
    ws.weights[out] = w;
  }
}

// ---------------------------------------------------------------------------
// adopt: a selection made on the token's home rank, cut down to this rank's experts
// ---------------------------------------------------------------------------
// grid (T), 256 threads.  Expert parallelism with a replicated sketch: the home
// rank of a token has chosen its kept channels and sent them as a list of
// candidate ids (slot * I + channel, slots in ascending expert order; ascending,
// -1 after the last).  This rank orders and maps the router's experts exactly as
// k_route does, keeps the entries of the slots it owns in their order, and
// derives the per-slot counts, list starts and down-tile starts for them.
// With `peers` the lists are those the home ranks stored into this rank's exchange
// block; the CTA first waits (bounded) until the lists of its row's home rank have
// landed for the current epoch.
__global__ void __launch_bounds__(256) k_adopt(Layer L, Workspace ws, const void* ids, int ids64,
                                               const void* weights, int wbf16,
                                               const uint8_t* padding, const int32_t* lists,
                                               Exchange x, int peers) {
  __shared__ int route[32];
  __shared__ int count[32];
  __shared__ int warp_total[8];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool padded = padding && padding[t];
  if (peers) {
    uint32_t* header = exchange_header(x, x.rank);
    if (tid == 0)
      exchange_wait(header + kExchangeListsFlag + t / x.tokens, header[kExchangeEpoch] + 1u,
                    header + kExchangeStatus, 1u);
    lists = reinterpret_cast<const int32_t*>(x.block[x.rank] + exchange_lists_offset());
    __syncthreads();
  }
  if (warp == 0) {
    long long id = 0x7fffffffffffffffLL;
    float w = 0.0f;
    if (lane < L.K) {
      const size_t at = static_cast<size_t>(t) * L.K + lane;
      id = ids64 ? static_cast<const long long*>(ids)[at]
                 : static_cast<long long>(static_cast<const int32_t*>(ids)[at]);
      w = wbf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(weights)[at])
                : static_cast<const float*>(weights)[at];
    }
    int rank = 0;
    for (int j = 0; j < L.K; ++j) {
      const long long o = __shfl_sync(kFull, id, j);
      rank += (o < id) || (o == id && j < lane);
    }
    count[lane] = 0;
    if (lane < L.K) {
      int local = -1;
      if (L.expert_map) {
        if (id >= 0 && id < L.global_experts) local = L.expert_map[id];
      } else if (id >= 0 && id < L.E) {
        local = static_cast<int>(id);
      }
      if (local >= L.E) local = -1;
      const size_t out = static_cast<size_t>(t) * L.K + rank;
      ws.ids[out] = local;
      ws.weights[out] = w;
      route[rank] = padded ? -1 : local;
    }
  }
  __syncthreads();
  const int32_t* in = lists + static_cast<size_t>(t) * L.F;
  int32_t* out = ws.candidate_ids + static_cast<size_t>(t) * L.F;
  int kept = 0;
  for (int base = 0; base < L.F; base += 256) {
    const int i = base + tid;
    const int cid = i < L.F ? __ldcg(in + i) : -1;  // past L1: a peer may have written it
    const int slot = cid >= 0 ? min(cid / L.I, L.K - 1) : 0;
    const bool keep = cid >= 0 && route[slot] >= 0;
    const unsigned ballot = __ballot_sync(kFull, keep);
    if (lane == 0) warp_total[warp] = __popc(ballot);
    __syncthreads();
    int before = kept, all = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      before += w < warp ? warp_total[w] : 0;
      all += warp_total[w];
    }
    if (keep) {
      out[before + __popc(ballot & ((1u << lane) - 1))] = cid;
      atomicAdd(&count[slot], 1);
    }
    kept += all;
    __syncthreads();
  }
  for (int i = kept + tid; i < L.F; i += 256) out[i] = -1;
  if (warp == 0) {
    const bool live = lane < L.K;
    const int mine = live ? count[lane] : 0;
    const int tiles = (mine + kDownTileRows - 1) / kDownTileRows;
    int rows = mine, scan = tiles;
#pragma unroll
    for (int w = 1; w < 32; w <<= 1) {
      const int r = __shfl_up_sync(kFull, rows, w), o = __shfl_up_sync(kFull, scan, w);
      if (lane >= w) {
        rows += r;
        scan += o;
      }
    }
    if (live) {
      const size_t pair = static_cast<size_t>(t) * L.K + lane;
      ws.counts[pair] = mine;
      ws.starts[pair] = rows - mine;
      ws.tile_starts[pair] = scan - tiles;
    }
  }
}

// ---------------------------------------------------------------------------
// screen: sketch GEMV + score
// ---------------------------------------------------------------------------
// grid (T*K pairs, S splits of the rotation blocks), W*CG threads.  Thread
// (cg, wi) owns sketch word wi (16 rows) and the kept coordinates j = cg mod CG
// of each block.  Integer partial dots are summed across coordinate groups in
// shared memory; each thread then finishes 16/CG rows.
template <int CG>
__global__ void __launch_bounds__(512) k_screen(Layer L, Workspace ws, const uint8_t* padding, int S) {
  grid_dependency_release();  // the selection may be scheduled; it waits for this grid
  constexpr int RPT = kWordRows / CG;  // rows a thread finishes per block
  constexpr int U = 8;                 // words in flight per thread
  extern __shared__ int smem[];
  const int rows = 2 * L.I, W = L.W, threads = W * CG;
  int* sq = smem;              // [128] fixed-point values of the block
  int* sc = sq + kBlock;       // [128] their coordinates
  int* red = sc + kBlock;      // [CG * 16 * W] partial dots (CG > 1)
  __shared__ int s_last;

  const int pair = blockIdx.x, split = blockIdx.y;
  const int t = pair / L.K, slot = pair - t * L.K;
  const int tid = threadIdx.x, wi = tid % W, cg = tid / W;
  const int e = ws.ids[pair];
  if ((padding && padding[t]) || e < 0) {
    if (split == 0) {
      for (int c = tid; c < L.I; c += threads) {
        ws.partial[static_cast<size_t>(t) * 2 * L.N + slot * L.I + c] = 0.0f;
        ws.partial[static_cast<size_t>(t) * 2 * L.N + L.N + slot * L.I + c] = 0.0f;
      }
    }
    return;
  }
  const int per = (L.B + S - 1) / S;
  const int b0 = split * per, b1 = min(L.B, b0 + per);
  float run[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) run[r] = 0.0f;
  const int row0 = wi * kWordRows + cg * RPT;  // first row this thread finishes

  for (int b = b0; b < b1; ++b) {
    const size_t tb = static_cast<size_t>(t) * L.B + b;
    __syncthreads();
    for (int j = tid; j < L.KEEP; j += threads) {
      sq[j] = ws.quantized[tb * L.KEEP + j];
      sc[j] = ws.coordinates[tb * L.KEEP + j];
    }
    // Scales of the rows this thread finishes, fetched ahead of the dots.
    float scale[RPT];
    {
      const __half* st = L.statistics +
                         (static_cast<size_t>(e) * L.B + b) * 2 * rows + row0;
#pragma unroll
      for (int r = 0; r < RPT; ++r) scale[r] = __half2float(st[r]);
    }
    const int be = ws.exponents[2 * tb], qsum = ws.exponents[2 * tb + 1];
    __syncthreads();

    int acc[kWordRows];
#pragma unroll
    for (int j = 0; j < kWordRows; ++j) acc[j] = 0;
    const uint32_t* base =
        L.sketch + (static_cast<size_t>(e) * L.H + static_cast<size_t>(b) * kBlock) * W + wi;
    for (int j0 = cg; j0 < L.KEEP; j0 += CG * U) {
      uint32_t word[U];
      int q[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int j = j0 + u * CG;
        if (j < L.KEEP) {
          word[u] = load_stream4(base + static_cast<size_t>(sc[j]) * W);
          q[u] = sq[j];
        } else {
          word[u] = 0;
          q[u] = 0;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int j = 0; j < kWordRows; ++j)
          acc[j] += static_cast<int>((word[u] >> (2 * j)) & 3u) * q[u];
      }
    }
    int dot[RPT];
    if (CG > 1) {
#pragma unroll
      for (int j = 0; j < kWordRows; ++j) red[(cg * kWordRows + j) * W + wi] = acc[j];
      __syncthreads();
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        int s = 0;
#pragma unroll
        for (int g = 0; g < CG; ++g) s += red[(g * kWordRows + cg * RPT + r) * W + wi];
        dot[r] = s;
      }
    } else {
#pragma unroll
      for (int r = 0; r < RPT; ++r) dot[r] = acc[r];
    }
    // code = trit + 1, so sum(trit * q) = sum(code * q) - sum(q).
    const float unscale = __uint_as_float(static_cast<uint32_t>(127 + be - kQuantBits) << 23);
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const float d = __fmul_rn(__int2float_rn(dot[r] - qsum), unscale);
      const float prod = __fmul_rn(scale[r], d);
      if (S == 1) {
        run[r] = __fadd_rn(run[r], prod);
      } else {
        ws.parts[(static_cast<size_t>(pair) * L.B + b) * rows + row0 + r] = prod;
      }
    }
  }

  float* gate_out = ws.partial + static_cast<size_t>(t) * 2 * L.N + static_cast<size_t>(slot) * L.I;
  float* up_out = gate_out + L.N;
  if (S == 1) {
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int row = row0 + r;
      (row < L.I ? gate_out[row] : up_out[row - L.I]) = run[r];
    }
    return;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned old = atomicAdd(&ws.counters[pair], 1u);
    s_last = (old == static_cast<unsigned>(S - 1));
    if (s_last) ws.counters[pair] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // The last split to arrive sums the per-block products in block order.
  for (int row = tid; row < rows; row += threads) {
    float s = 0.0f;
    const float* p = ws.parts + static_cast<size_t>(pair) * L.B * rows + row;
    for (int b = 0; b < L.B; ++b) s = __fadd_rn(s, __ldcg(p + static_cast<size_t>(b) * rows));
    (row < L.I ? gate_out[row] : up_out[row - L.I]) = s;
  }
}

// ---------------------------------------------------------------------------
// grouped screen: pairs grouped by expert, int8 tensor-core dot products
// ---------------------------------------------------------------------------
// Lists the active (token, slot) pairs of every local expert.  One CTA; dynamic
// shared memory: 2 * E counters.  The order of an expert's pairs is whatever the
// atomics produce; every pair's result is independent of it.
__global__ void __launch_bounds__(1024) k_group(Layer L, Workspace ws, const uint8_t* padding,
                                                int T) {
  extern __shared__ int group_smem[];
  int* count = group_smem;
  int* cursor = group_smem + L.E;
  const int tid = threadIdx.x, pairs = T * L.K;
  for (int e = tid; e < L.E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = tid; p < pairs; p += blockDim.x) {
    const int e = ws.ids[p];
    if (e >= 0 && !(padding && padding[p / L.K])) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (tid < 32) {  // exclusive scan over experts, one warp
    int carry = 0;
    for (int base = 0; base < L.E; base += 32) {
      const int e = base + tid;
      const int mine = e < L.E ? count[e] : 0;
      int scan = mine;
#pragma unroll
      for (int w = 1; w < 32; w <<= 1) {
        const int o = __shfl_up_sync(kFull, scan, w);
        if (tid >= w) scan += o;
      }
      if (e < L.E) {
        cursor[e] = carry + scan - mine;
        ws.group_offsets[e] = carry + scan - mine;
      }
      carry += __shfl_sync(kFull, scan, 31);
    }
    if (tid == 0) ws.group_offsets[L.E] = carry;
  }
  __syncthreads();
  for (int p = tid; p < pairs; p += blockDim.x) {
    const int e = ws.ids[p];
    if (e >= 0 && !(padding && padding[p / L.K])) {
      ws.group_pairs[atomicAdd(&cursor[e], 1)] = p;
    }
  }
}

// Sixteen 2-bit codes of one 32-bit word -> four int8x4 registers of trits.
// The grouped layout stores coordinate c of a word at bit 4c (c < 4),
// 4(c-4)+2 (c < 8), 16+4(c-8) (c < 12), 18+4(c-12) otherwise, so that four
// masked shifts yield byte-permute selectors; the permute picks -1, 0, +1 from
// a register table.
__device__ __forceinline__ void decode_word(uint32_t w, uint32_t& c0, uint32_t& c1, uint32_t& c2,
                                            uint32_t& c3) {
  constexpr uint32_t table = 0x000100ffu;  // byte 0 = -1, byte 1 = 0, byte 2 = +1
  c0 = __byte_perm(table, 0u, w & 0x3333u);
  c1 = __byte_perm(table, 0u, (w >> 2) & 0x3333u);
  c2 = __byte_perm(table, 0u, (w >> 16) & 0x3333u);
  c3 = __byte_perm(table, 0u, (w >> 18) & 0x3333u);
}

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#include "cfm_build.cuh"

constexpr int kGroupWarps = 8;  // 16 sketch rows per warp

// m16n8k32 int8 MMA whose accumulator starts at zero.
__device__ __forceinline__ void mma_s8_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Everything a lane needs for one rotation block, fetched one block ahead.
struct GroupFetch {
  uint2 word_a, word_b;  // 32 coordinates of rows g and g + 8
  uint4 digit[3][2];     // this lane's 32 coordinates of the three digits of token g
  __half scale_a, scale_b;
  float unscale[2];      // 2^(e - 21) of the two tokens this lane finishes (2 tq, 2 tq + 1)
};

// grid (ceil(2I / 128), E, passes), 256 threads, no shared memory, no barrier.  A warp
// owns 16 sketch rows of one expert and walks the rotation blocks in order.  Per
// block it decodes 16 rows x 128 coordinates into int8 fragments and multiplies
// them with the int8 digits of up to eight of the expert's tokens (m16n8k32,
// exact int32 sums; one 8-column tile per digit).  Lane (g, tq) holds
// coordinates 32 tq .. 32 tq + 31 of rows g and g + 8 and of token g's digits,
// so k-step m uses coordinates 32 tq + 8 m .. + 7 of all of them; the digits
// come straight from global memory (L1/L2 resident, 32 contiguous bytes per
// lane and digit).  The next block's words, digits, scales and exponents are
// in flight in registers while the current block computes.  Experts with more
// than eight tokens take further passes of eight, spread over grid.z.
__global__ void __launch_bounds__(kGroupWarps * 32, 2) k_screen_grouped(Layer L, Workspace ws) {
  grid_dependency_release();  // the selection may be scheduled; it waits for this grid
  constexpr int kGroupRows = kGroupWarps * 16;  // rows per CTA
  const int e = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int first = ws.group_offsets[e], total = ws.group_offsets[e + 1] - first;
  const int rows = 2 * L.I;
  const int r0 = blockIdx.x * kGroupRows + warp * 16;
  if (total == 0 || r0 >= rows) return;  // whole warps are in or out: 2I is a multiple of 32
  const int row_a = r0 + g, row_b = r0 + g + 8;
  const uint2* sketch = reinterpret_cast<const uint2*>(L.sketch_grouped) + tq;
  const size_t sketch_block = static_cast<size_t>(rows) * (kBlock / 32);  // uint2 per block
  const size_t sketch_a = (static_cast<size_t>(e) * L.B * rows + row_a) * (kBlock / 32);
  const size_t sketch_b = (static_cast<size_t>(e) * L.B * rows + row_b) * (kBlock / 32);
  const __half* scales = L.statistics + static_cast<size_t>(e) * L.B * 2 * rows;

  for (int base = 8 * blockIdx.z; base < total; base += 8 * gridDim.z) {
    const int count = min(8, total - base);
    // Pair of the token whose digits this lane feeds (column g of the tiles).
    const int pair_g = g < count ? ws.group_pairs[first + base + g] : -1;
    // Pairs of the two tokens whose results this lane finishes.
    const int pair_0 = __shfl_sync(kFull, pair_g, (2 * tq) * 4);
    const int pair_1 = __shfl_sync(kFull, pair_g, (2 * tq + 1) * 4);
    // Running pointers, advanced by one rotation block per fetch.  Empty token
    // slots read a block of zero digits kept in the workspace (never written).
    const uint2* next_a = sketch + sketch_a;
    const uint2* next_b = sketch + sketch_b;
    const __half* next_scale_a = scales + row_a;
    const __half* next_scale_b = scales + row_b;
    const uint4* next_digits = reinterpret_cast<const uint4*>(
        (pair_g >= 0 ? ws.limbs + static_cast<size_t>(pair_g / L.K) * L.B * 3 * kBlock
                     : ws.zero_limbs) + 32 * tq);
    const float* next_unscale_0 = ws.unscales + static_cast<size_t>(max(pair_0, 0) / L.K) * L.B;
    const float* next_unscale_1 = ws.unscales + static_cast<size_t>(max(pair_1, 0) / L.K) * L.B;
    auto fetch = [&]() {
      GroupFetch f;
      f.word_a = *next_a;
      f.word_b = *next_b;
      f.scale_a = *next_scale_a;
      f.scale_b = *next_scale_b;
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        f.digit[j][0] = next_digits[j * (kBlock / 16)];
        f.digit[j][1] = next_digits[j * (kBlock / 16) + 1];
      }
      f.unscale[0] = *next_unscale_0;
      f.unscale[1] = *next_unscale_1;
      next_a += sketch_block;
      next_b += sketch_block;
      next_scale_a += 2 * rows;
      next_scale_b += 2 * rows;
      next_digits += 3 * kBlock / 16;
      ++next_unscale_0;
      ++next_unscale_1;
      return f;
    };

    float run[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    auto compute = [&](const GroupFetch& cur) {
      uint32_t fa[8], fb[8];
      decode_word(cur.word_a.x, fa[0], fa[1], fa[2], fa[3]);
      decode_word(cur.word_a.y, fa[4], fa[5], fa[6], fa[7]);
      decode_word(cur.word_b.x, fb[0], fb[1], fb[2], fb[3]);
      decode_word(cur.word_b.y, fb[4], fb[5], fb[6], fb[7]);
      int acc[3][4];
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const uint4 lo = cur.digit[j][0], hi = cur.digit[j][1];
        mma_s8_first(acc[j], fa[0], fb[0], fa[1], fb[1], lo.x, lo.y);
        mma_s8(acc[j], fa[2], fb[2], fa[3], fb[3], lo.z, lo.w);
        mma_s8(acc[j], fa[4], fb[4], fa[5], fb[5], hi.x, hi.y);
        mma_s8(acc[j], fa[6], fb[6], fa[7], fb[7], hi.z, hi.w);
      }
      const float scale_a = __half2float(cur.scale_a), scale_b = __half2float(cur.scale_b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int dot = acc[0][i] + acc[1][i] * 256 + acc[2][i] * 65536;
        const float d = __fmul_rn(__int2float_rn(dot), cur.unscale[i & 1]);
        run[i] = __fadd_rn(run[i], __fmul_rn(i < 2 ? scale_a : scale_b, d));
      }
    };
    // Two fetch buffers used in turn, so that no block's data is copied between
    // registers: while one block computes the next one's loads are in flight.
    GroupFetch even = fetch(), odd;
    for (int b = 0; b < L.B; b += 2) {
      if (b + 1 < L.B) odd = fetch();
      compute(even);
      if (b + 2 < L.B) even = fetch();
      if (b + 1 < L.B) compute(odd);
    }
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
}

// ---------------------------------------------------------------------------
// grouped screen on the 5th-generation tensor cores (tcgen05, TMEM accumulators)
// ---------------------------------------------------------------------------
// Same arithmetic as k_screen_grouped (int8 trits x int8 digits -> exact int32
// block dots), as one M128 x N32 x K32 `tcgen05.mma.kind::i8` per 32 coordinates.
// A CTA owns 128 sketch rows of one expert and up to ten of its tokens per pass.
// Per rotation block one ring stage in shared memory holds
//   A  the 128 rows x 128 coordinates decoded to int8 (K-major canonical layout,
//      no swizzle: core matrices of 8 rows x 16 bytes, 128 bytes apart along K,
//      256 bytes apart along M; four K = 32 steps of 4 KiB), and
//   B  the three int8 digits of the tokens for those 128 coordinates (column
//      3 token + digit, same layout, four steps of 1 KiB);
// both written by eight producer warps (a thread decodes 64 coordinates of one
// row and forwards one 16-byte piece of digits, all fetched one block ahead).
// One warp issues the MMAs into one of four 32-column int32 accumulators in
// tensor memory; four epilogue warps read them back (`tcgen05.ld`), rescale per
// block and keep the running projections in registers.  Stages and
// accumulators are handed over with mbarriers; every wait is bounded (about a
// second) and on expiry sets `status[0]`, makes all roles leave, and the CTA
// still frees its tensor memory.
namespace tc {

constexpr int kRows = 128;            // sketch rows per CTA (MMA M)
constexpr int kCols = 32;             // accumulator columns (MMA N)
constexpr int kTokens = 10;           // tokens per pass: 3 digit columns each
constexpr int kStages = 4;            // ring stages = accumulators in flight
constexpr int kStepBytes = kRows * 32;          // one K = 32 step of A
constexpr int kDigitStepBytes = kCols * 32;     // one K = 32 step of B
constexpr int kStageBytes = 4 * (kStepBytes + kDigitStepBytes);  // one rotation block
constexpr int kProducers = 256;                 // eight producer warps
constexpr int kThreads = 13 * 32;               // 8 producer, 4 epilogue, 1 MMA warp
constexpr long long kWaitCycles = 2000000000LL;  // bound of every barrier wait

__device__ __forceinline__ uint32_t shared_address(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void barrier_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void barrier_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Waits for the phase with the given parity; false when the wait ran out or
// another role already gave up.
__device__ __forceinline__ bool barrier_wait(uint32_t bar, uint32_t parity, volatile int* abort) {
  const long long start = clock64();
  for (;;) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if (*abort || clock64() - start > kWaitCycles) {
      *abort = 1;
      return false;
    }
  }
}

// Shared-memory matrix descriptor: K-major, no swizzle, 128 bytes between the
// two 16-byte K chunks of a core-matrix row group, 256 bytes between row groups.
__device__ __forceinline__ uint64_t matrix_descriptor(uint32_t address) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((address & 0x3ffffu) >> 4);  // start address
  d |= static_cast<uint64_t>(128 >> 4) << 16;             // leading (K) byte offset
  d |= static_cast<uint64_t>(256 >> 4) << 32;             // stride (M/N) byte offset
  d |= static_cast<uint64_t>(1) << 46;                    // descriptor version of sm_100
  return d;
}

// Instruction descriptor: int32 accumulate, signed int8 A and B, both K-major.
__host__ __device__ constexpr uint32_t instruction_descriptor() {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kCols >> 3) << 17) |
         (static_cast<uint32_t>(kRows >> 4) << 24);
}

__device__ __forceinline__ void mma_i8(uint32_t tmem, uint64_t a, uint64_t b, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem), "l"(a), "l"(b), "r"(instruction_descriptor()), "r"(accumulate), "r"(0)
      : "memory");
}

__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

__host__ __device__ inline size_t shared_bytes(int B) {
  return static_cast<size_t>(kStages) * kStageBytes + sizeof(float) * kTokens * B + 256;
}

}  // namespace tc

// grid (ceil(2I / 128), E, passes), 416 threads, dynamic shared memory
// tc::shared_bytes(B).
__global__ void __launch_bounds__(tc::kThreads) k_screen_tc(Layer L, Workspace ws) {
  using namespace tc;
  extern __shared__ __align__(1024) uint8_t tc_shared[];
  uint8_t* ring = tc_shared;  // [kStages][A 16 KiB | B 4 KiB]
  float* unscale = reinterpret_cast<float*>(ring + kStages * kStageBytes);  // [kTokens][B]
  uint8_t* tail = reinterpret_cast<uint8_t*>(unscale + kTokens * L.B);
  uint64_t* barriers = reinterpret_cast<uint64_t*>(tail);  // full, empty, ready, freed x stages
  int* pairs = reinterpret_cast<int*>(tail + 128);         // [kTokens]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tail + 192);
  volatile int* abort = reinterpret_cast<volatile int*>(tail + 196);

  const int e = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int first = ws.group_offsets[e], total = ws.group_offsets[e + 1] - first;
  if (total <= static_cast<int>(blockIdx.z) * kTokens) return;  // no pass for this CTA
  const int rows = 2 * L.I;
  const uint32_t full = shared_address(barriers), empty = full + 8 * kStages,
                 ready = empty + 8 * kStages, freed = ready + 8 * kStages;

  if (tid == 0) {
    *abort = 0;
    for (int s = 0; s < kStages; ++s) {
      barrier_init(full + 8 * s, kProducers / 32);  // one lane of every producer warp arrives
      barrier_init(empty + 8 * s, 1);               // the MMA commit arrives
      barrier_init(ready + 8 * s, 1);               // the MMA commit arrives
      barrier_init(freed + 8 * s, 4);               // one lane of every epilogue warp arrives
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 12) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     shared_address(tmem_holder)),
                 "r"(kStages * kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_holder;

  int iteration = 0;  // rotation blocks processed so far, over all passes
  for (int base = kTokens * blockIdx.z; base < total; base += kTokens * gridDim.z) {
    const int count = min(kTokens, total - base);
    if (tid < kTokens) pairs[tid] = tid < count ? ws.group_pairs[first + base + tid] : -1;
    __syncthreads();
    for (int index = tid; index < kTokens * L.B; index += kThreads) {
      const int token = index / L.B, b = index - token * L.B;
      const int pair = pairs[token];
      const int be =
          pair >= 0 ? ws.exponents[2 * (static_cast<size_t>(pair / L.K) * L.B + b)] : kQuantBits;
      unscale[index] = __uint_as_float(static_cast<uint32_t>(127 + be - kQuantBits) << 23);
    }
    __syncthreads();

    if (warp < 8) {
      // ---- producers.  Thread (half, local row): coordinates 64 half .. + 63 of
      // the row (four words, K steps 2 half and 2 half + 1); it also forwards the
      // 16-byte piece `piece` of digit column `column` of the block.
      const int half = tid >> 7, local = tid & 127;
      const int row = blockIdx.x * kRows + local;
      const bool inside = row < rows;
      const uint4* source =
          reinterpret_cast<const uint4*>(L.sketch_grouped +
                                         (static_cast<size_t>(e) * L.B * rows + (inside ? row : 0)) *
                                             (kBlock / 16)) + half;
      const size_t block_stride = static_cast<size_t>(rows) * (kBlock / 16) / 4;  // uint4 per block
      const int column = tid >> 3, piece = tid & 7;  // 32 columns x 8 pieces
      const int token = column / 3, digit = column - 3 * token;
      const int pair = token < kTokens ? pairs[token] : -1;
      const uint4* digits =
          pair >= 0 ? reinterpret_cast<const uint4*>(
                          ws.limbs + (static_cast<size_t>(pair / L.K) * L.B * 3 + digit) * kBlock) + piece
                    : nullptr;
      const size_t digit_stride = 3 * kBlock / 16;  // uint4 per block
      uint8_t* a_dst = ring + (2 * half) * kStepBytes + (local >> 3) * 256 + (local & 7) * 16;
      uint8_t* b_dst = ring + 4 * kStepBytes + (piece >> 1) * kDigitStepBytes + (column >> 3) * 256 +
                       (piece & 1) * 128 + (column & 7) * 16;
      uint4 next_words = inside ? source[0] : make_uint4(0, 0, 0, 0);
      uint4 next_digits = digits ? digits[0] : make_uint4(0, 0, 0, 0);
      for (int b = 0; b < L.B && !*abort; ++b) {
        const int it = iteration + b, stage = it % kStages;
        const uint4 words = next_words, piece_bytes = next_digits;
        if (b + 1 < L.B) {
          if (inside) next_words = source[(b + 1) * block_stride];
          if (digits) next_digits = digits[(b + 1) * digit_stride];
        }
        if (!barrier_wait(empty + 8 * stage, ((it / kStages) & 1) ^ 1, abort)) break;
        uint8_t* a_out = a_dst + stage * kStageBytes;
        const uint32_t four[4] = {words.x, words.y, words.z, words.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {  // word w = coordinates 64 half + 16 w .. + 15
          uint4 bytes;
          decode_word(four[w], bytes.x, bytes.y, bytes.z, bytes.w);
          *reinterpret_cast<uint4*>(a_out + (w >> 1) * kStepBytes + (w & 1) * 128) = bytes;
        }
        *reinterpret_cast<uint4*>(b_dst + stage * kStageBytes) = piece_bytes;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) barrier_arrive(full + 8 * stage);
      }
    } else if (warp == 12) {
      // ---- MMA issue: one lane; four K = 32 steps per rotation block.
      if (lane == 0) {
        for (int b = 0; b < L.B && !*abort; ++b) {
          const int it = iteration + b, stage = it % kStages;
          const uint32_t parity = (it / kStages) & 1;
          if (!barrier_wait(full + 8 * stage, parity, abort)) break;
          if (!barrier_wait(freed + 8 * stage, parity ^ 1, abort)) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_base = shared_address(ring + stage * kStageBytes);
          const uint32_t b_base = a_base + 4 * kStepBytes;
#pragma unroll
          for (int step = 0; step < 4; ++step)
            mma_i8(tmem + stage * kCols, matrix_descriptor(a_base + step * kStepBytes),
                   matrix_descriptor(b_base + step * kDigitStepBytes), step > 0);
          mma_commit(empty + 8 * stage);  // the stage may be refilled
          mma_commit(ready + 8 * stage);  // the accumulator may be read
        }
      }
    } else {
      // ---- epilogue: thread = accumulator lane = sketch row.
      const int quarter = warp - 8, local = quarter * 32 + lane;
      const int row = blockIdx.x * kRows + local;
      const bool inside = row < rows;
      const __half* scales =
          L.statistics + static_cast<size_t>(e) * L.B * 2 * rows + (inside ? row : 0);
      float run[kTokens];
#pragma unroll
      for (int t = 0; t < kTokens; ++t) run[t] = 0.0f;
      float scale = inside ? __half2float(scales[0]) : 0.0f;
      for (int b = 0; b < L.B && !*abort; ++b) {
        const int it = iteration + b, stage = it % kStages;
        const float scale_now = scale;
        if (inside && b + 1 < L.B)
          scale = __half2float(scales[static_cast<size_t>(b + 1) * 2 * rows]);
        if (!barrier_wait(ready + 8 * stage, (it / kStages) & 1, abort)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t c[kCols];
        const uint32_t address = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + stage * kCols;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]), "=r"(c[4]), "=r"(c[5]), "=r"(c[6]),
              "=r"(c[7]), "=r"(c[8]), "=r"(c[9]), "=r"(c[10]), "=r"(c[11]), "=r"(c[12]),
              "=r"(c[13]), "=r"(c[14]), "=r"(c[15]), "=r"(c[16]), "=r"(c[17]), "=r"(c[18]),
              "=r"(c[19]), "=r"(c[20]), "=r"(c[21]), "=r"(c[22]), "=r"(c[23]), "=r"(c[24]),
              "=r"(c[25]), "=r"(c[26]), "=r"(c[27]), "=r"(c[28]), "=r"(c[29]), "=r"(c[30]),
              "=r"(c[31])
            : "r"(address)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) barrier_arrive(freed + 8 * stage);
#pragma unroll
        for (int t = 0; t < kTokens; ++t) {
          if (t < count) {
            const int dot = static_cast<int>(c[3 * t]) + static_cast<int>(c[3 * t + 1]) * 256 +
                            static_cast<int>(c[3 * t + 2]) * 65536;
            const float d = __fmul_rn(__int2float_rn(dot), unscale[t * L.B + b]);
            run[t] = __fadd_rn(run[t], __fmul_rn(scale_now, d));
          }
        }
      }
      if (inside && !*abort) {
#pragma unroll
        for (int t = 0; t < kTokens; ++t) {
          if (t < count) {
            const int pair = pairs[t];
            const int token = pair / L.K, slot = pair - token * L.K;
            float* out = ws.partial + static_cast<size_t>(token) * 2 * L.N +
                         static_cast<size_t>(slot) * L.I;
            (row < L.I ? out[row] : out[L.N + row - L.I]) = run[t];
          }
        }
      }
    }
    iteration += L.B;
    __syncthreads();
    if (*abort) break;
  }
  if (*abort && tid == 0) atomicExch(&ws.status[0], 1);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 12) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"(kStages * kCols)
                 : "memory");
  }
}

#include "cfm_screen_rows32.cuh"

// grid (T, ceil(N / 256)), 256 threads: zero the projections of remote or padded
// slots (the grouped screen writes only live pairs).
__global__ void k_clear_dead(Layer L, Workspace ws, const uint8_t* padding) {
  const int t = blockIdx.x, i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= L.N) return;
  const int slot = i / L.I;
  if ((padding && padding[t]) || ws.ids[static_cast<size_t>(t) * L.K + slot] < 0) {
    ws.partial[static_cast<size_t>(t) * 2 * L.N + i] = 0.0f;
    ws.partial[static_cast<size_t>(t) * 2 * L.N + L.N + i] = 0.0f;
  }
}

// grid (T, ceil(N / 256)), 256 threads: scores from projections (used when the
// scores are exchanged between ranks before selection).
__global__ void k_score(Layer L, Workspace ws, const uint8_t* padding) {
  const int t = blockIdx.x, i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= L.N) return;
  const int slot = i / L.I, c = i - slot * L.I;
  const int e = ws.ids[static_cast<size_t>(t) * L.K + slot];
  float value = 0.0f;
  if (e >= 0 && !(padding && padding[t]))
    value = candidate_score(L, ws, t, i, e, c, ws.weights[static_cast<size_t>(t) * L.K + slot]);
  ws.scores[static_cast<size_t>(t) * L.N + i] = value;
}

// Residual variance of every candidate's sketch projections (recovery-aware
// score): sum over blocks, in block order, of the row's FP16 residual variance
// times the energy of the token's kept coordinates in that block.
// grid (T*K pairs, ceil(2I / 256)), 256 threads, one sketch row per thread.
__global__ void __launch_bounds__(256) k_variance(Layer L, Workspace ws, const uint8_t* padding) {
  const int pair = blockIdx.x, row = blockIdx.y * 256 + threadIdx.x;
  const int rows = 2 * L.I;
  if (row >= rows) return;
  const int t = pair / L.K, slot = pair - t * L.K;
  const int e = ws.ids[pair];
  float sum = 0.0f;
  if (e >= 0 && !(padding && padding[t])) {
    const __half* variance = L.statistics + (static_cast<size_t>(e) * L.B * 2 + 1) * rows + row;
    const float* energy = ws.norms + static_cast<size_t>(t) * L.B;
    for (int b = 0; b < L.B; ++b)
      sum = __fadd_rn(sum, __fmul_rn(__half2float(variance[static_cast<size_t>(b) * 2 * rows]),
                                     energy[b]));
  }
  float* out = ws.variances + static_cast<size_t>(t) * 2 * L.N + static_cast<size_t>(slot) * L.I;
  (row < L.I ? out[row] : out[L.N + row - L.I]) = sum;
}

// Score of candidate i of token t from its projections (and variances).
__device__ __forceinline__ float candidate_score(const Layer& L, const Workspace& ws, int t, int i,
                                                 int e, int c, float weight) {
  const float* gate = ws.partial + static_cast<size_t>(t) * 2 * L.N;
  const float norm = L.norms[static_cast<size_t>(e) * L.I + c];
  if (L.score == CFM_SCORE_POINT) return point_score(gate[i], gate[L.N + i], norm, weight, L.activation);
  const float* variance = ws.variances + static_cast<size_t>(t) * 2 * L.N;
  float alpha = 0.0f, beta = 0.0f;
  if (L.geometry) {
    alpha = L.geometry[(static_cast<size_t>(e) * L.I + c) * 2];
    beta = L.geometry[(static_cast<size_t>(e) * L.I + c) * 2 + 1];
  }
  return risk_score(gate[i], gate[L.N + i], variance[i], variance[L.N + i], norm, alpha, beta,
                    weight, L.activation);
}

// ---------------------------------------------------------------------------
// select: top-F per token, read-cost counters
// ---------------------------------------------------------------------------
constexpr int kSelectThreads = 1024;

#include "cfm_select.cuh"

__device__ __forceinline__ int64_t sector_run(int64_t bytes) { return (bytes + 31) / 32 * 32; }

// Read-cost counters of one token (integers, so FP64 atomics are exact): lane
// `lane` of one warp adds slot `lane` of `read_work`.  `local_slots` of the
// token's experts are held here and `kept_local` of its kept channels are theirs.
__device__ __forceinline__ void account_reads(const Layer& L, int lane, int local_slots,
                                              int kept_local, bool screened) {
  const int I = L.I, K = L.K;
  if (L.read_work && lane < CFM_READ_WORK_SLOTS) {
    const bool ep = L.expert_map != nullptr;
    const int64_t H = L.H, R = L.R;
    const int64_t candidates = static_cast<int64_t>(local_slots) * I;
    const int64_t native = 2 * (2 * kept_local * H + kept_local * H);
    const int64_t dense_slot = 6 * static_cast<int64_t>(I) * H;
    const int64_t reference = ep ? local_slots * dense_slot : K * dense_slot;
    const int64_t recovery = 2 * R * (candidates - kept_local + (L.owner ? H : 0));
    const bool residual = L.score != CFM_SCORE_POINT;
    const int64_t code = 2 * ((I + 4) / 5), plane = 4 * I;
    const int64_t sketch_exact =
        screened ? local_slots * L.B * (L.KEEP * code + plane * (1 + residual)) : 0;
    const int64_t sketch_sector =
        screened ? local_slots * L.B *
                       (L.KEEP * sector_run(code) + sector_run(plane) * (1 + residual))
                 : 0;
    // Bytes the screen kernel itself requests: 2-bit codes (I / 2 bytes per
    // kept coordinate) and the FP16 scale plane.
    const int64_t sketch_issued =
        screened ? local_slots * L.B * (static_cast<int64_t>(L.KEEP) * (I / 2) + plane) : 0;
    const int64_t selection =
        screened ? ((L.geometry ? 12 : 4) * candidates) : 0;
    // Threshold mode: every token also reads the FP32 layer threshold (one sector).
    const int64_t threshold_exact = L.threshold ? 4 : 0, threshold_sector = L.threshold ? 32 : 0;
    int64_t value = 0;
    switch (lane) {
      case 0: case 6: value = native; break;
      case 1: value = reference; break;
      case 3: case 7: value = recovery; break;
      case 4: value = selection + threshold_exact; break;
      case 9: value = selection + threshold_sector; break;
      case 19: value = L.threshold ? 1 : 0; break;
      case 5: value = sketch_exact; break;
      case 10: value = screened ? H : 0; break;
      case 11: value = sketch_issued; break;
      case 17: value = sketch_sector; break;
      case 12: value = 4 * H * kept_local; break;
      case 13: value = 2 * H * kept_local; break;
      case 14: value = 2 * R * (candidates - kept_local); break;
      default: value = 0;
  }
    if (value) atomicAdd(L.read_work + lane, static_cast<double>(value));
  }
}

// grid (T), 1024 threads, dynamic shared memory: N keys.
// With `peers` (expert parallelism over peer memory; row_offset 0, T = x.tokens) a
// CTA ends by storing its token's kept list into slot [rank] of every rank's exchange
// block; the last CTA to arrive releases each destination's flag with the call's epoch.
// Without PEERS the exchange argument is a dummy, so that the single-GPU kernel carries
// neither the parameter block nor the code of the hand-over.
struct NoExchange {
  int world, rank, tokens;
  char* block[1];
};
template <bool PEERS>
__global__ void __launch_bounds__(kSelectThreads)
    k_select(Layer L, Workspace ws, const uint8_t* padding, int scores_ready, int row_offset,
             typename std::conditional<PEERS, Exchange, NoExchange>::type x) {
  constexpr bool peers = PEERS;
  grid_dependency_release();  // the exact gather may be scheduled; it waits for this grid
  grid_dependency_wait();     // the screen's projections are complete
  extern __shared__ uint32_t keys[];
  __shared__ int hist[2048];
  __shared__ int warp_above[33], warp_ties[32];
  __shared__ int s_digit, s_remaining;
  __shared__ int s_starts[33], s_tie_start[33], s_budget[32];
  const int t = blockIdx.x + row_offset, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = L.N, F = L.F, K = L.K, I = L.I;
  const bool cut_given = scores_ready == 2, cut_only = scores_ready == 3;
  int32_t* counts = ws.counts + static_cast<size_t>(t) * K;
  int32_t* starts = ws.starts + static_cast<size_t>(t) * K;
  int32_t* tile_starts = ws.tile_starts + static_cast<size_t>(t) * K;
  // All threads of the CTA call this once the token's list is complete (or has
  // nothing to say: a padding row, whose list the owners ignore).
  auto publish = [&](bool send) {
    if constexpr (PEERS) {
    __syncthreads();  // the list is complete in global memory for this CTA's threads
    uint32_t* header = exchange_header(x, x.rank);
    const uint32_t epoch = header[kExchangeEpoch] + 1u;
    if (send) {
      const int32_t* mine = ws.candidate_ids + static_cast<size_t>(t) * F;
      const size_t at = (static_cast<size_t>(x.rank) * x.tokens + t) * F;
      if (F % 4 == 0) {
        const int quads = F / 4;
        for (int j = tid; j < x.world * quads; j += kSelectThreads) {
          const int d = j / quads, i = j - d * quads;
          int4* out = reinterpret_cast<int4*>(
              reinterpret_cast<int32_t*>(x.block[d] + exchange_lists_offset()) + at);
          out[i] = reinterpret_cast<const int4*>(mine)[i];
        }
      } else {
        for (int j = tid; j < x.world * F; j += kSelectThreads) {
          const int d = j / F, i = j - d * F;
          (reinterpret_cast<int32_t*>(x.block[d] + exchange_lists_offset()) + at)[i] = mine[i];
        }
      }
    }
    // The CTA barrier orders every thread's stores before the fences of the few threads
    // that announce; a system-scope fence is cumulative.
    __syncthreads();
    if (tid < x.world) {
      __threadfence_system();
      uint32_t* counter = header + kExchangeListsArrive + tid;
      if (atomicAdd(counter, 1u) == gridDim.x - 1) {
        *counter = 0;
        __threadfence_system();
        store_release_system(exchange_header(x, tid) + kExchangeListsFlag + x.rank, epoch);
      }
    }
    }
  };
  if (padding && padding[t]) {
    if (tid < K) counts[tid] = starts[tid] = tile_starts[tid] = 0;
    if (tid <= K) ws.cuts[static_cast<size_t>(t) * (K + 1) + tid] = 0;
    if (peers) publish(false);
    return;
  }
  const bool screened = F < N;
  uint32_t cut = 0;
  int take_ties = 0;
  if (screened) {
    float* score = ws.scores + static_cast<size_t>(t) * N;
    if (scores_ready) {
      for (int i = tid; i < N; i += kSelectThreads) keys[i] = __float_as_uint(score[i]);
    } else {
      // Score every candidate from its sketch projections (zero for remote slots).
      for (int i = tid; i < N; i += kSelectThreads) {
        const int slot = slot_of(L, i), c = i - slot * I;
        const int e = ws.ids[static_cast<size_t>(t) * K + slot];
        float value = 0.0f;
        if (e >= 0)
          value = candidate_score(L, ws, t, i, e, c, ws.weights[static_cast<size_t>(t) * K + slot]);
        score[i] = value;
        keys[i] = __float_as_uint(value);
      }
    }
    // Radix search for the F-th largest key: digits of 11, 11 and 10 bits from
    // the top.  Each pass histograms the keys that match the prefix found so far,
    // then a block-wide scan from the highest digit down locates the digit in
    // which the running count reaches the number still wanted.
    uint32_t prefix = 0, mask = 0;
    int remaining = F;
#pragma unroll 1
    for (int pass = 0; pass < (cut_given ? 0 : 3); ++pass) {
      const int shift = pass == 0 ? 21 : pass == 1 ? 10 : 0;
      const int bins = pass == 2 ? 1024 : 2048;
      for (int i = tid; i < bins; i += kSelectThreads) hist[i] = 0;
      __syncthreads();
      for (int i = tid; i < N; i += kSelectThreads) {
        const uint32_t k = keys[i];
        if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & (bins - 1)], 1);
      }
      __syncthreads();
      // Thread tid owns digits bins-1-2*tid and bins-2-2*tid (descending order).
      const int d0 = bins - 1 - 2 * tid;
      const int c0 = d0 >= 0 ? hist[d0] : 0;
      const int c1 = d0 >= 1 ? hist[d0 - 1] : 0;
      const int total = c0 + c1;
      int scan = total;
#pragma unroll
      for (int w = 1; w < 32; w <<= 1) {
        const int o = __shfl_up_sync(kFull, scan, w);
        if (lane >= w) scan += o;
      }
      if (lane == 31) warp_above[warp] = scan;
      __syncthreads();
      if (warp == 0) {
        int totals = warp_above[lane];
#pragma unroll
        for (int w = 1; w < 32; w <<= 1) {
          const int o = __shfl_up_sync(kFull, totals, w);
          if (lane >= w) totals += o;
        }
        warp_ties[lane] = totals;  // inclusive scan of the warp totals
      }
      __syncthreads();
      const int before = scan - total + (warp ? warp_ties[warp - 1] : 0);
      if (before < remaining && before + total >= remaining) {
        const bool first = before + c0 >= remaining;
        s_digit = first ? d0 : d0 - 1;
        s_remaining = remaining - (first ? before : before + c0);
      }
      __syncthreads();
      prefix |= static_cast<uint32_t>(s_digit) << shift;
      mask |= static_cast<uint32_t>(bins - 1) << shift;
      remaining = s_remaining;
    }
    cut = prefix;
    take_ties = remaining;
    if (L.threshold && !cut_given) {
      // Threshold mode: every score at or above the layer threshold, at most F
      // (best first).  When fewer than F reach it, the cut moves up to just below
      // the threshold's key and no tie budget is needed.
      const uint32_t floor_key = __float_as_uint(__fadd_rn(*L.threshold, 0.0f));
      if (cut < floor_key) {
        cut = floor_key - 1u;
        take_ties = 0;
      }
    }
  }

  // Compaction in candidate order: a thread owns a contiguous chunk.  Ties at
  // the cut are kept in candidate order; that rule is applied slot by slot with a
  // per-slot tie budget, so that a rank holding only some of a token's slots can
  // repeat the selection from the cut and the budgets alone.
  const int chunk = (N + kSelectThreads - 1) / kSelectThreads;
  const int begin = min(N, tid * chunk), end = min(N, begin + chunk);
  const int32_t* route = ws.ids + static_cast<size_t>(t) * K;
  int32_t* cuts = ws.cuts + static_cast<size_t>(t) * (K + 1);
  if (cut_given) cut = static_cast<uint32_t>(cuts[0]);
  auto block_exclusive = [&](int value, int* total) {
    return block_exclusive_scan(value, warp_above, total);
  };
  // Counts above the cut and tied with it, packed into one scan (N < 65536).
  const bool budgets = cut_given || cut_only;
  int counted = 0;
  if (screened)
    for (int i = begin; i < end; ++i) {
      const uint32_t k = keys[i];
      counted += (k > cut ? 0x10000 : 0) + (k == cut ? 1 : 0);
    }
  int all_counted = 0;
  const int counted_before = block_exclusive(counted, &all_counted);
  const int ties_before = counted_before & 0xffff, above_before = counted_before >> 16;
  if (budgets) {
    int running = ties_before;
    for (int i = begin; i < end; ++i) {
      const int slot = slot_of(L, i);
      if (i == slot * I) s_tie_start[slot] = running;
      running += screened && keys[i] == cut;
    }
    if (tid == 0) s_tie_start[K] = all_counted & 0xffff;
    __syncthreads();
    if (tid < K) {
      int budget;
      if (cut_given) {
        budget = cuts[1 + tid];
      } else {
        const int in_slot = s_tie_start[tid + 1] - s_tie_start[tid];
        budget = max(0, min(in_slot, take_ties - s_tie_start[tid]));
        cuts[1 + tid] = budget;
        if (tid == 0) cuts[0] = static_cast<int32_t>(cut);
      }
      s_budget[tid] = budget;
    }
    if (cut_only) return;  // the token's home rank only publishes the cut and the budgets
    __syncthreads();
  }
  auto keeps = [&](int i, int running) {
    const int slot = slot_of(L, i);
    if (cut_given && route[slot] < 0) return false;  // another rank's slot
    if (!screened) return true;
    const uint32_t k = keys[i];
    if (k != cut) return k > cut;
    return budgets ? running - s_tie_start[slot] < s_budget[slot] : running < take_ties;
  };
  int total_kept = screened ? (all_counted >> 16) + min(all_counted & 0xffff, take_ties) : F;
  int position = above_before + min(ties_before, take_ties);
  if (!screened) position = begin;
  if (budgets) {
    int kept = 0, running = ties_before;
    for (int i = begin; i < end; ++i) {
      kept += keeps(i, running);
      running += screened && keys[i] == cut;
    }
    position = block_exclusive(kept, &total_kept);
  }
  uint8_t* selected = ws.selected + static_cast<size_t>(t) * N;
  uint8_t* completed = ws.completed + static_cast<size_t>(t) * N;
  int32_t* list = ws.candidate_ids + static_cast<size_t>(t) * F;
  {
    int running = ties_before;
    for (int i = begin; i < end; ++i) {
      const bool keep = keeps(i, running);
      running += screened && keys[i] == cut;
      const int slot = slot_of(L, i);
      if (i - slot * I == 0) s_starts[slot] = position;
      selected[i] = keep;
      completed[i] = keep && route[slot] >= 0;
      if (keep) list[position++] = i;
    }
  }
  for (int i = total_kept + tid; i < F; i += kSelectThreads) list[i] = -1;
  if (tid == 0) s_starts[K] = total_kept;
  __syncthreads();
  if (warp == 0) {
    const bool live = lane < K;
    const int count = live ? s_starts[lane + 1] - s_starts[lane] : 0;
    const bool local = live && route[lane] >= 0;
    const int tiles = local ? (count + kDownTileRows - 1) / kDownTileRows : 0;
    int scan = tiles;
#pragma unroll
    for (int w = 1; w < 32; w <<= 1) {
      const int o = __shfl_up_sync(kFull, scan, w);
      if (lane >= w) scan += o;
    }
    if (live) {
      counts[lane] = count;
      starts[lane] = s_starts[lane];
      tile_starts[lane] = scan - tiles;
    }
    // Read-cost counters of this token (integers, so FP64 atomics are exact).
    int local_slots = local, kept_local = local ? count : 0;
#pragma unroll
    for (int w = 16; w; w >>= 1) {
      local_slots += __shfl_xor_sync(kFull, local_slots, w);
      kept_local += __shfl_xor_sync(kFull, kept_local, w);
    }
    account_reads(L, lane, local_slots, kept_local, screened);
  }
  if (peers) publish(true);
}

// ---------------------------------------------------------------------------
// exact: gathered gate/up rows
// ---------------------------------------------------------------------------
constexpr int kExactWarps = 4;

// One warp's dot products of a gate row and an up row with the input staged in
// shared memory (`xs`, `chunks` 16-byte pieces): eight pieces of each row in
// flight per lane (2048 columns per sweep), FP32 FMAs in a fixed order, then a
// butterfly over the lanes.  Every lane returns the sums.  The loads of a sweep and
// the arithmetic on them are separate steps, so that a kernel can issue a row's
// first sweep before the barrier that publishes `xs`.
constexpr int kExactSweep = 8;  // 16-byte pieces of each row per lane and sweep

__device__ __forceinline__ void exact_load(const uint4* gate, const uint4* up, int base, int chunks,
                                           uint4 (&gw)[kExactSweep], uint4 (&uw)[kExactSweep]) {
  if (base + 32 * (kExactSweep - 1) < chunks) {
#pragma unroll
    for (int k = 0; k < kExactSweep; ++k) {
      gw[k] = load_stream16(gate + base + 32 * k);
      uw[k] = load_stream16(up + base + 32 * k);
    }
  } else {
#pragma unroll
    for (int k = 0; k < kExactSweep; ++k) {
      const int i = base + 32 * k;
      gw[k] = uw[k] = make_uint4(0, 0, 0, 0);
      if (i < chunks) {
        gw[k] = load_stream16(gate + i);
        uw[k] = load_stream16(up + i);
      }
    }
  }
}

__device__ __forceinline__ void exact_consume(const uint4 (&gw)[kExactSweep],
                                              const uint4 (&uw)[kExactSweep], const uint4* xs,
                                              int base, int chunks, float& g, float& u) {
#pragma unroll
  for (int k = 0; k < kExactSweep; ++k) {
    const int i = min(base + 32 * k, chunks - 1);
    const uint4 xw = xs[i];
    g = fmaf(bf16_lo(gw[k].x), bf16_lo(xw.x), g);
    g = fmaf(bf16_hi(gw[k].x), bf16_hi(xw.x), g);
    g = fmaf(bf16_lo(gw[k].y), bf16_lo(xw.y), g);
    g = fmaf(bf16_hi(gw[k].y), bf16_hi(xw.y), g);
    g = fmaf(bf16_lo(gw[k].z), bf16_lo(xw.z), g);
    g = fmaf(bf16_hi(gw[k].z), bf16_hi(xw.z), g);
    g = fmaf(bf16_lo(gw[k].w), bf16_lo(xw.w), g);
    g = fmaf(bf16_hi(gw[k].w), bf16_hi(xw.w), g);
    u = fmaf(bf16_lo(uw[k].x), bf16_lo(xw.x), u);
    u = fmaf(bf16_hi(uw[k].x), bf16_hi(xw.x), u);
    u = fmaf(bf16_lo(uw[k].y), bf16_lo(xw.y), u);
    u = fmaf(bf16_hi(uw[k].y), bf16_hi(xw.y), u);
    u = fmaf(bf16_lo(uw[k].z), bf16_lo(xw.z), u);
    u = fmaf(bf16_hi(uw[k].z), bf16_hi(xw.z), u);
    u = fmaf(bf16_lo(uw[k].w), bf16_lo(xw.w), u);
    u = fmaf(bf16_hi(uw[k].w), bf16_hi(xw.w), u);
  }
}

// The rest of a row pair whose first sweep (`gw`, `uw`) is loaded already when
// `loaded`, else the whole pair; same order of operations either way.
__device__ __forceinline__ void exact_dot(const uint4* gate, const uint4* up, const uint4* xs,
                                          int chunks, int lane, bool loaded,
                                          uint4 (&gw)[kExactSweep], uint4 (&uw)[kExactSweep],
                                          float& g_out, float& u_out) {
  float g = 0.0f, u = 0.0f;
  for (int base = lane; base < chunks; base += 32 * kExactSweep) {
    if (!(loaded && base == lane)) exact_load(gate, up, base, chunks, gw, uw);
    exact_consume(gw, uw, xs, base, chunks, g, u);
  }
#pragma unroll
  for (int w = 16; w; w >>= 1) {
    g += __shfl_xor_sync(kFull, g, w);
    u += __shfl_xor_sync(kFull, u, w);
  }
  g_out = g;
  u_out = u;
}

// grid (ceil(F / 4), T), 128 threads; one warp per kept candidate.
__global__ void __launch_bounds__(kExactWarps * 32) k_exact(Layer L, Workspace ws,
                                                            const __nv_bfloat16* hidden,
                                                            const uint8_t* padding) {
  grid_dependency_wait();  // the selection is complete
  extern __shared__ uint4 xs[];  // H bf16 values of the token
  const int t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (padding && padding[t]) return;
  const int32_t* list = ws.candidate_ids + static_cast<size_t>(t) * L.F;
  const bool strided = gridDim.x * kExactWarps < L.F;  // CTAs walk the list in strides
  if (L.expert_map) {
    // Expert parallel: leave before staging the input when this CTA has nothing
    // to do.  A list cut down to the local slots ends with -1 entries; a full list
    // is probed for candidates of local experts.
    if (list[blockIdx.x * kExactWarps] < 0) return;
    if (!strided) {
      const int probe = blockIdx.x * kExactWarps + warp;
      bool mine = false;
      if (probe < L.F) {
        const int cid = list[probe];
        mine = cid >= 0 && ws.ids[static_cast<size_t>(t) * L.K + cid / L.I] >= 0;
      }
      if (!__syncthreads_or(mine)) return;
    }
  }
  const int chunks = L.H / 8;
  const size_t up_offset = static_cast<size_t>(L.I) * L.H / 8;
  // The rows of a candidate of a local expert, or null.
  auto rows_of = [&](int index) -> const uint4* {
    if (index >= L.F) return nullptr;
    const int cid = list[index];
    if (cid < 0) return nullptr;
    const int slot = cid / L.I, c = cid - slot * L.I;
    const int e = ws.ids[static_cast<size_t>(t) * L.K + slot];
    if (e < 0) return nullptr;
    return reinterpret_cast<const uint4*>(L.gate_up + (static_cast<size_t>(e) * 2 * L.I + c) * L.H);
  };
  // The first row pair's first sweep is on its way while the input row is staged.
  const int first = blockIdx.x * kExactWarps + warp;
  uint4 gw[kExactSweep], uw[kExactSweep];
  const uint4* first_rows = rows_of(first);
  if (first_rows) exact_load(first_rows, first_rows + up_offset, lane, chunks, gw, uw);
  const uint4* x = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(t) * L.H);
  for (int i = tid; i < chunks; i += kExactWarps * 32) xs[i] = x[i];
  __syncthreads();
  for (int index = first; index < L.F; index += gridDim.x * kExactWarps) {
  const int cid = list[index];
  if (cid < 0) break;  // lists end with -1 entries
  const uint4* gate = index == first ? first_rows : rows_of(index);
  if (!gate) continue;
  float g, u;
  exact_dot(gate, gate + up_offset, xs, chunks, lane, index == first, gw, uw, g, u);
  if (lane == 0) {
    ws.activations[static_cast<size_t>(t) * L.N + cid] =
        __float2bfloat16_rn(exact_feature(g, u, L.activation));
    ws.exact[static_cast<size_t>(t) * 2 * L.F + index] = g;
    ws.exact[static_cast<size_t>(t) * 2 * L.F + L.F + index] = u;
  }
  }
}

// The same gather with the (token, expert) pairs walked in expert order:
// grid (X, T * K), 128 threads.  CTA row y takes the y-th pair of the list
// grouped by expert (k_group), so the tokens of one expert run next to each
// other in time and a row several of them kept comes from HBM once and from L2
// after that.  The X CTAs of a pair share its kept rows, one warp per row.  Same
// arithmetic, same order, same bits as k_exact.
// The kept rows of the y-th pair of the list grouped by expert, for the CTA column
// blockIdx.x; all threads of the CTA call it with the staged row `xs` free.
__device__ __forceinline__ void exact_pair(const Layer& L, const Workspace& ws,
                                           const __nv_bfloat16* hidden, uint4* xs, int y) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pair = ws.group_pairs[y];
  const int count = ws.counts[pair];
  if (static_cast<int>(blockIdx.x) * kExactWarps >= count) return;  // the whole CTA
  const int t = pair / L.K, slot = pair - t * L.K, e = ws.ids[pair];
  const int start = ws.starts[pair];
  const int32_t* list = ws.candidate_ids + static_cast<size_t>(t) * L.F + start;
  const int chunks = L.H / 8;
  const size_t up_offset = static_cast<size_t>(L.I) * L.H / 8;
  const uint4* expert_rows =
      reinterpret_cast<const uint4*>(L.gate_up + static_cast<size_t>(e) * 2 * L.I * L.H);
  // The first row pair's first sweep is on its way while the input row is staged.
  const int first = blockIdx.x * kExactWarps + warp;
  uint4 gw[kExactSweep], uw[kExactSweep];
  if (first < count) {
    const uint4* gate = expert_rows + static_cast<size_t>(list[first] - slot * L.I) * chunks;
    exact_load(gate, gate + up_offset, lane, chunks, gw, uw);
  }
  const uint4* x = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(t) * L.H);
  for (int i = tid; i < chunks; i += kExactWarps * 32) xs[i] = x[i];
  __syncthreads();
  for (int index = first; index < count; index += gridDim.x * kExactWarps) {
    const int cid = list[index];
    const uint4* gate = expert_rows + static_cast<size_t>(cid - slot * L.I) * chunks;
    float g, u;
    exact_dot(gate, gate + up_offset, xs, chunks, lane, index == first, gw, uw, g, u);
    if (lane == 0) {
      ws.activations[static_cast<size_t>(t) * L.N + cid] =
          __float2bfloat16_rn(exact_feature(g, u, L.activation));
      ws.exact[static_cast<size_t>(t) * 2 * L.F + start + index] = g;
      ws.exact[static_cast<size_t>(t) * 2 * L.F + L.F + start + index] = u;
    }
  }
}

// STRIDED: under expert parallelism fewer CTA rows than (token, slot) pairs are launched,
// since a rank owns few of them; row y then takes pairs y, y + gridDim.y, ...
template <bool STRIDED>
__global__ void __launch_bounds__(kExactWarps * 32) k_exact_pairs(Layer L, Workspace ws,
                                                                  const __nv_bfloat16* hidden) {
  grid_dependency_wait();  // the selection is complete
  extern __shared__ uint4 xs[];  // H bf16 values of the token
  const int pairs = ws.group_offsets[L.E];
  if (!STRIDED) {
    if (static_cast<int>(blockIdx.y) < pairs) exact_pair(L, ws, hidden, xs, blockIdx.y);
    return;
  }
  for (int y = blockIdx.y; y < pairs; y += gridDim.y) {
    exact_pair(L, ws, hidden, xs, y);
    __syncthreads();  // the staged row may be overwritten by the next pair
  }
}

// ---------------------------------------------------------------------------
// down: gathered channel-major down rows
// ---------------------------------------------------------------------------
constexpr int kDownColumns = 1024;  // output columns per CTA: 32 accumulators per lane
constexpr int kDownStages = 4;      // rows in flight per warp (3, 4 and 6 measured alike)
constexpr int kDownRowBytes = kDownColumns * 2;  // one row's share of a CTA: 2 KiB per warp and row
constexpr int down_ring_bytes(int stages) { return 4 * stages * kDownRowBytes; }  // per CTA

// 16 bytes global -> shared memory, past L1, completing in the thread's current
// cp.async group.
__device__ __forceinline__ void copy_async16(void* shared, const void* global) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                   static_cast<uint32_t>(__cvta_generic_to_shared(shared))),
               "l"(global)
               : "memory");
}
__device__ __forceinline__ void copy_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int PENDING>
__device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// grid (ceil(H / 1024), tiles, T), 128 threads, down_ring_bytes(kDownStages) of dynamic
// shared memory.  One CTA sums up to 64 kept rows of one expert, each scaled by its
// activation, over 1024 output columns.  A warp takes every fourth row of the
// tile.  Rows travel through a ring in shared memory, four per warp in flight:
// per row a lane copies four 16-byte pieces 512 bytes apart (2 KiB contiguous per
// warp and row) with cp.async and later reads back exactly the pieces it copied,
// so a lane only ever waits for its own copy groups and the ring needs no barrier.
// The row is accumulated into 32 FP32 registers per lane in row order; the four
// warps' sums are added in warp order through shared memory (the ring's, once
// all copies have landed).  Under expert parallelism (STRIDED) fewer CTAs than
// tiles are launched per token, since a rank owns few of a token's slots; they
// walk the tiles in strides.
// One tile: `rows` (at most 64) kept rows of slot `slot` of token t, an expert-e
// slot, whose candidate ids start at `list`, summed into down tile `tile`.
// Called by all 128 threads of a CTA; begins and ends with the shared arrays free.
template <int STAGES>
__device__ __forceinline__ void down_tile(const Layer& L, const Workspace& ws, int t, int slot,
                                          int e, int rows, const int32_t* list, int tile,
                                          int* tile_channel, float* tile_activation,
                                          uint8_t* ring) {
  constexpr int CHUNKS = kDownColumns / 256;  // 16-byte pieces per lane and row
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int column0 = blockIdx.x * kDownColumns + lane * 8;  // this lane's first column
  const __nv_bfloat16* act = ws.activations + static_cast<size_t>(t) * L.N;
  if (tid < rows) {
    const int cid = list[tid];
    tile_channel[tid] = cid - slot * L.I;
    tile_activation[tid] = __bfloat162float(act[cid]);
  }
  __syncthreads();
  const __nv_bfloat16* base = L.down + static_cast<size_t>(e) * L.I * L.H + column0;
  bool live[CHUNKS];
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) live[j] = column0 + 256 * j < L.H;
  float acc[CHUNKS][8];
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[j][i] = 0.0f;
  // This lane's pieces of ring slot s of its warp.
  uint8_t* mine = ring + warp * (STAGES * kDownRowBytes) + lane * 16;
  auto fetch = [&](int r, int s) {  // row r of the tile into slot s; one copy group
    if (r < rows) {
      const __nv_bfloat16* row = base + static_cast<size_t>(tile_channel[r]) * L.H;
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j)
        if (live[j]) copy_async16(mine + s * kDownRowBytes + 512 * j, row + 256 * j);
    }
    copy_async_commit();  // also when empty: the group count per iteration stays fixed
  };
  auto add = [&](int r, int s) {
    const float a = tile_activation[r];
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      const uint4 w = live[j] ? *reinterpret_cast<const uint4*>(mine + s * kDownRowBytes + 512 * j)
                              : make_uint4(0, 0, 0, 0);
      acc[j][0] = fmaf(bf16_lo(w.x), a, acc[j][0]);
      acc[j][1] = fmaf(bf16_hi(w.x), a, acc[j][1]);
      acc[j][2] = fmaf(bf16_lo(w.y), a, acc[j][2]);
      acc[j][3] = fmaf(bf16_hi(w.y), a, acc[j][3]);
      acc[j][4] = fmaf(bf16_lo(w.z), a, acc[j][4]);
      acc[j][5] = fmaf(bf16_hi(w.z), a, acc[j][5]);
      acc[j][6] = fmaf(bf16_lo(w.w), a, acc[j][6]);
      acc[j][7] = fmaf(bf16_hi(w.w), a, acc[j][7]);
    }
  };
#pragma unroll
  for (int s = 0; s < STAGES; ++s) fetch(warp + 4 * s, s);
  int s = 0;
  for (int r = warp; r < rows; r += 4) {
    copy_async_wait<STAGES - 1>();  // the oldest group, row r, has landed
    add(r, s);
    fetch(r + 4 * STAGES, s);  // the slot is free again: its pieces are in registers
    s = s + 1 == STAGES ? 0 : s + 1;
  }
  copy_async_wait<0>();
  __syncthreads();  // every warp is done with the ring: it now holds the warps' sums
  float(*red)[kDownColumns] = reinterpret_cast<float(*)[kDownColumns]>(ring);
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    float4* out = reinterpret_cast<float4*>(&red[warp][256 * j + lane * 8]);
    out[0] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
    out[1] = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
  }
  __syncthreads();
  float* parts = ws.down_parts + (static_cast<size_t>(t) * ws.down_tiles + tile) * L.H +
                 blockIdx.x * kDownColumns;
  for (int c = tid * 4; c < kDownColumns; c += 128 * 4) {
    if (blockIdx.x * kDownColumns + c < L.H) {
      const float4 a = *reinterpret_cast<const float4*>(&red[0][c]);
      const float4 b = *reinterpret_cast<const float4*>(&red[1][c]);
      const float4 d = *reinterpret_cast<const float4*>(&red[2][c]);
      const float4 g = *reinterpret_cast<const float4*>(&red[3][c]);
      *reinterpret_cast<float4*>(parts + c) =
          make_float4(((a.x + b.x) + d.x) + g.x, ((a.y + b.y) + d.y) + g.y,
                      ((a.z + b.z) + d.z) + g.z, ((a.w + b.w) + d.w) + g.w);
    }
  }
  __syncthreads();  // the shared arrays may be reused
}

template <bool STRIDED, int STAGES>
__global__ void __launch_bounds__(128, 4) k_down(Layer L, Workspace ws, const uint8_t* padding) {
  extern __shared__ __align__(128) uint8_t down_ring[];
  __shared__ int tile_channel[kDownTileRows];
  __shared__ float tile_activation[kDownTileRows];
  __shared__ int s_slot, s_first;
  const int t = blockIdx.z, tid = threadIdx.x;
  if (padding && padding[t]) return;
  const size_t token_pairs = static_cast<size_t>(t) * L.K;
  int used;
  {
    // Tiles are laid out slot after slot; leave at once beyond the last one.
    const size_t last = token_pairs + L.K - 1;
    const int tail =
        ws.ids[last] >= 0 ? (ws.counts[last] + kDownTileRows - 1) / kDownTileRows : 0;
    used = ws.tile_starts[last] + tail;
  }
  int tile = blockIdx.y;
  if (tile >= used) return;
  do {
    if (tid == 0) s_slot = -1;
    __syncthreads();
    if (tid < L.K) {  // the slot whose tile range holds this tile, if any
      const int e = ws.ids[token_pairs + tid];
      const int tiles =
          e >= 0 ? (ws.counts[token_pairs + tid] + kDownTileRows - 1) / kDownTileRows : 0;
      const int begin = ws.tile_starts[token_pairs + tid];
      if (tile >= begin && tile < begin + tiles) {
        s_slot = tid;
        s_first = (tile - begin) * kDownTileRows;
      }
    }
    __syncthreads();
    const int slot = s_slot, first = s_first;
    if (slot < 0) continue;  // uniform: every thread read the same slot
    down_tile<STAGES>(L, ws, t, slot, ws.ids[token_pairs + slot],
              min(kDownTileRows, ws.counts[token_pairs + slot] - first),
              ws.candidate_ids + static_cast<size_t>(t) * L.F + ws.starts[token_pairs + slot] + first,
              tile, tile_channel, tile_activation, down_ring);
  } while (STRIDED && (tile += gridDim.y) < used);
}

// The same tiles from the list of the call's tiles in expert order
// (cfm_select.cuh): grid (ceil(H / 1024), most tiles a call can have), 128
// threads.  A CTA reads its 32-byte record and goes straight to the tile's rows.
// Same tiles, same sums, same bits as k_down.
template <int STAGES>
__global__ void __launch_bounds__(128, 4) k_down_tiles(Layer L, Workspace ws) {
  extern __shared__ __align__(128) uint8_t down_ring[];
  __shared__ int tile_channel[kDownTileRows];
  __shared__ float tile_activation[kDownTileRows];
  const int tiles = ws.tile_count[0];
  for (int y = blockIdx.y; y < tiles; y += gridDim.y) {  // strides under expert parallelism
    const int4* record = reinterpret_cast<const int4*>(ws.tile_list) + 2 * y;
    const int4 a = record[0], b = record[1];  // t, slot, expert, rows | list, tile
    down_tile<STAGES>(L, ws, a.x, a.y, a.z, a.w, ws.candidate_ids + b.x, b.y, tile_channel,
                      tile_activation, down_ring);
  }
}

// ---------------------------------------------------------------------------
// encode: recovery encoder over skipped channels, then the latent
// ---------------------------------------------------------------------------
// grid (encoder_tiles, T*K), 256 threads.  A CTA owns 256 channels of one
// (token, expert) pair.  Phase 1 turns the sketch projections of the skipped
// channels into features in shared memory (0 for kept channels); phase 2
// streams the encoder rows: LPR = R / 8 lanes cover one row (16 bytes each),
// 256 / LPR row groups walk the channels with eight rows in flight per thread;
// phase 3 folds the row groups (shuffles inside a warp, shared memory across
// warps).  The last CTA of a token to arrive mixes the latent.
constexpr int kEncodeThreads = 256;

__global__ void __launch_bounds__(kEncodeThreads) k_encode(Layer L, Workspace ws,
                                                           const uint8_t* padding) {
  __shared__ float feature[kEncodeTileRows];
  __shared__ float red[kEncodeThreads / 32][256];
  __shared__ int s_last;
  const int tile = blockIdx.x, pair = blockIdx.y, tid = threadIdx.x;
  const int t = pair / L.K, slot = pair - t * L.K;
  const int R = L.R, lpr = R / 8, groups = kEncodeThreads / lpr;
  const int e = ws.ids[pair];
  const bool dead = (padding && padding[t]) || e < 0;
  const int c0 = tile * kEncodeTileRows, c1 = min(L.I, c0 + kEncodeTileRows);
  const int group = tid / lpr, col = (tid - group * lpr) * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  if (!dead) {
    const float* pg = ws.partial + static_cast<size_t>(t) * 2 * L.N + slot * L.I;
    const float* pu = pg + L.N;
    const uint8_t* sel = ws.selected + static_cast<size_t>(t) * L.N + slot * L.I;
    for (int c = c0 + tid; c < c1; c += kEncodeThreads)
      feature[c - c0] = sel[c] ? 0.0f : sketch_feature(pg[c], pu[c], L.activation);
    __syncthreads();
    const __nv_bfloat16* enc = L.encoder + static_cast<size_t>(e) * L.I * R + col;
    constexpr int U = 8;
    for (int base = c0 + group; base < c1; base += groups * U) {
      uint4 w[U];
      float p[U];
      if (base + (U - 1) * groups < c1) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = base + u * groups;
          p[u] = feature[c - c0];
          w[u] = *reinterpret_cast<const uint4*>(enc + static_cast<size_t>(c) * R);
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = base + u * groups;
          p[u] = 0.0f;
          w[u] = make_uint4(0, 0, 0, 0);
          if (c < c1) {
            p[u] = feature[c - c0];
            w[u] = *reinterpret_cast<const uint4*>(enc + static_cast<size_t>(c) * R);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        acc[0] = fmaf(bf16_lo(w[u].x), p[u], acc[0]);
        acc[1] = fmaf(bf16_hi(w[u].x), p[u], acc[1]);
        acc[2] = fmaf(bf16_lo(w[u].y), p[u], acc[2]);
        acc[3] = fmaf(bf16_hi(w[u].y), p[u], acc[3]);
        acc[4] = fmaf(bf16_lo(w[u].z), p[u], acc[4]);
        acc[5] = fmaf(bf16_hi(w[u].z), p[u], acc[5]);
        acc[6] = fmaf(bf16_lo(w[u].w), p[u], acc[6]);
        acc[7] = fmaf(bf16_hi(w[u].w), p[u], acc[7]);
      }
    }
  }
  // Fold the row groups that share a warp (lanes lpr apart hold the same columns).
  for (int w = lpr; w < 32; w <<= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(kFull, acc[j], w);
  }
  const int lane = tid & 31, warp = tid >> 5;
  if (lpr >= 32) {
    // One row spans the whole warp or more: lane owns columns (tid % lpr) * 8.
#pragma unroll
    for (int j = 0; j < 8; ++j) red[group][col + j] = acc[j];
  } else if (lane < lpr) {
#pragma unroll
    for (int j = 0; j < 8; ++j) red[warp][col + j] = acc[j];
  }
  __syncthreads();
  const int folds = lpr >= 32 ? groups : kEncodeThreads / 32;
  float* parts = ws.encoder_parts + (static_cast<size_t>(pair) * ws.encoder_tiles + tile) * R;
  for (int r = tid; r < R; r += kEncodeThreads) {
    float sum = 0.0f;
    for (int f = 0; f < folds; ++f) sum += red[f][r];
    parts[r] = sum;
  }
  // Last CTA of the token mixes the latent.
  __threadfence();
  __syncthreads();
  uint32_t* counter = ws.counters + 2 * static_cast<size_t>(ws.capacity) * L.K + t;
  if (tid == 0) {
    const unsigned total = static_cast<unsigned>(L.K * ws.encoder_tiles);
    const unsigned old = atomicAdd(counter, 1u);
    s_last = (old == total - 1);
    if (s_last) *counter = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int r = tid; r < R; r += kEncodeThreads) {
    float latent = 0.0f;
    for (int s2 = 0; s2 < L.K; ++s2) {
      const int pe = ws.ids[static_cast<size_t>(t) * L.K + s2];
      if (pe < 0 || (padding && padding[t])) continue;
      const float* p = ws.encoder_parts +
                       (static_cast<size_t>(t) * L.K + s2) * ws.encoder_tiles * R + r;
      float sum = 0.0f;
      for (int j = 0; j < ws.encoder_tiles; ++j) sum += __ldcg(p + static_cast<size_t>(j) * R);
      latent = fmaf(bf16_round(sum), ws.weights[static_cast<size_t>(t) * L.K + s2], latent);
    }
    ws.latent[static_cast<size_t>(t) * R + r] = latent;
  }
}

// grid (T), 128 threads: latent = 0 (no skipped channels, or no map).
__global__ void k_zero_latent(Layer L, Workspace ws) {
  for (int r = threadIdx.x; r < L.R; r += blockDim.x)
    ws.latent[static_cast<size_t>(blockIdx.x) * L.R + r] = 0.0f;
}

#include "cfm_grouped.cuh"

// One past the last down tile of slot `slot` of token t.  The per-token down
// kernel lays a token's tiles out slot after slot, ceil(count / 64) tiles per
// local slot, starting at `tile_starts`; the expert-major one writes `fixed`
// partial sums for every local slot, slot after slot.
__device__ __forceinline__ int down_slot_end(const Layer& L, const Workspace& ws, int t, int slot,
                                             int fixed) {
  const size_t pairs = static_cast<size_t>(t) * L.K;
  if (fixed == 0) {
    const int tiles = ws.ids[pairs + slot] >= 0
                          ? (ws.counts[pairs + slot] + kDownTileRows - 1) / kDownTileRows : 0;
    return ws.tile_starts[pairs + slot] + tiles;
  }
  int local = 0;
  for (int s = 0; s <= slot; ++s) local += ws.ids[pairs + s] >= 0;
  return local * fixed;
}

// ---------------------------------------------------------------------------
// output: router mix + decoder term
// ---------------------------------------------------------------------------
// One output column of one token: the per-slot sums of its down-tile partials in
// tile order, each rounded to BF16 and mixed with the slot's router weight in slot
// order.  `parts` points at the column in the token's first tile; `slot_end` and
// `slot_weight` are the token's slot table in shared memory.  Sixteen tile loads are
// in flight at a time; the additions keep their order.
__device__ __forceinline__ float mix_down_tiles(const float* parts, int used, size_t stride,
                                                const int* slot_end, const float* slot_weight) {
  constexpr int kInFlight = 16;
  float routed = 0.0f, sum = 0.0f;
  int slot = 0;
  for (int base = 0; base < used; base += kInFlight) {
    float v[kInFlight];
#pragma unroll
    for (int j = 0; j < kInFlight; ++j)
      v[j] = base + j < used ? __ldcg(parts + static_cast<size_t>(base + j) * stride) : 0.0f;
#pragma unroll
    for (int j = 0; j < kInFlight; ++j) {
      const int tile = base + j;
      if (tile < used) {
        while (tile >= slot_end[slot]) {  // close the finished slots
          routed = fmaf(bf16_round(sum), slot_weight[slot], routed);
          sum = 0.0f;
          ++slot;
        }
        sum += v[j];
      }
    }
  }
  if (used > 0) routed = fmaf(bf16_round(sum), slot_weight[slot], routed);
  return routed;
}

// The same for four adjacent columns (16-byte loads); each column's additions keep
// the order of the one-column version.
__device__ __forceinline__ float4 mix_down_tiles4(const float* parts, int used, size_t stride,
                                                  const int* slot_end, const float* slot_weight) {
  constexpr int kInFlight = 8;
  float4 routed = make_float4(0.0f, 0.0f, 0.0f, 0.0f), sum = routed;
  int slot = 0;
  auto close = [&]() {
    const float w = slot_weight[slot];
    routed.x = fmaf(bf16_round(sum.x), w, routed.x);
    routed.y = fmaf(bf16_round(sum.y), w, routed.y);
    routed.z = fmaf(bf16_round(sum.z), w, routed.z);
    routed.w = fmaf(bf16_round(sum.w), w, routed.w);
    sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    ++slot;
  };
  for (int base = 0; base < used; base += kInFlight) {
    float4 v[kInFlight];
#pragma unroll
    for (int j = 0; j < kInFlight; ++j)
      v[j] = base + j < used
                 ? __ldcg(reinterpret_cast<const float4*>(parts + static_cast<size_t>(base + j) * stride))
                 : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < kInFlight; ++j) {
      const int tile = base + j;
      if (tile < used) {
        while (tile >= slot_end[slot]) close();  // close the finished slots
        sum.x += v[j].x;
        sum.y += v[j].y;
        sum.z += v[j].z;
        sum.w += v[j].w;
      }
    }
  }
  if (used > 0) close();
  return routed;
}

// grid (H / 128, T), 128 threads, one output column per thread.  `fixed` is the
// number of partial sums per local slot the expert-major down kernel wrote, or 0
// after the per-token down kernel.
__global__ void __launch_bounds__(128) k_output(Layer L, Workspace ws, const uint8_t* padding,
                                                __nv_bfloat16* out, int fixed) {
  __shared__ float latent[256];
  __shared__ int slot_end[32];       // one past the last down tile of every slot
  __shared__ float slot_weight[32];
  const int t = blockIdx.y, tid = threadIdx.x, h = blockIdx.x * 128 + tid;
  if (padding && padding[t]) {
    out[static_cast<size_t>(t) * L.H + h] = __float2bfloat16_rn(0.0f);
    return;
  }
  const bool recover = L.R > 0 && L.owner && L.decoder;
  if (tid < L.K) {
    const size_t pair = static_cast<size_t>(t) * L.K + tid;
    slot_end[tid] = down_slot_end(L, ws, t, tid, fixed);
    slot_weight[tid] = ws.weights[pair];
  }
  if (recover)
    for (int r = tid; r < L.R; r += 128)
      latent[r] = bf16_round(ws.latent[static_cast<size_t>(t) * L.R + r]);
  // The decoder row does not depend on the slot table: its first chunks are on their
  // way before the barrier.
  constexpr int kAhead = 8;  // 16-byte chunks of the decoder row fetched ahead (R <= 64: all)
  float correction = 0.0f;
  const uint4* decoder_row = reinterpret_cast<const uint4*>(L.decoder + static_cast<size_t>(h) * L.R);
  uint4 ahead[kAhead];
  if (recover) {
#pragma unroll
    for (int i = 0; i < kAhead; ++i)
      ahead[i] = i < L.R / 8 ? decoder_row[i] : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  const int used = slot_end[L.K - 1];  // tiles are laid out slot after slot
  const float routed = mix_down_tiles(
      ws.down_parts + static_cast<size_t>(t) * ws.down_tiles * L.H + h, used, L.H, slot_end,
      slot_weight);
  if (recover) {
    float dot = 0.0f;
    auto fold = [&](const uint4 w, int i) {
      const float* z = latent + i * 8;
      dot = fmaf(bf16_lo(w.x), z[0], dot);
      dot = fmaf(bf16_hi(w.x), z[1], dot);
      dot = fmaf(bf16_lo(w.y), z[2], dot);
      dot = fmaf(bf16_hi(w.y), z[3], dot);
      dot = fmaf(bf16_lo(w.z), z[4], dot);
      dot = fmaf(bf16_hi(w.z), z[5], dot);
      dot = fmaf(bf16_lo(w.w), z[6], dot);
      dot = fmaf(bf16_hi(w.w), z[7], dot);
    };
#pragma unroll
    for (int i = 0; i < kAhead; ++i)
      if (i < L.R / 8) fold(ahead[i], i);
    for (int i0 = kAhead; i0 < L.R / 8; i0 += 4) {
      uint4 row[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        row[i] = i0 + i < L.R / 8 ? decoder_row[i0 + i] : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i0 + i < L.R / 8) fold(row[i], i0 + i);
    }
    correction = bf16_round(dot);
  }
  out[static_cast<size_t>(t) * L.H + h] = __float2bfloat16_rn(routed + correction);
}

// Expert parallelism splits the output stage in two.  k_partial_output runs on
// the rank that owns experts: the router-weighted FP32 sum of its local slots'
// BF16-rounded expert sums, no decoder term.  k_finish runs on the token's home
// rank after the partial sums and latents of all ranks have been added: decoder
// term and BF16 store.  grid (H / 128, T), 128 threads each.
// With `peers` row t goes straight into slot [this rank] of the `rows` of its home
// rank's exchange block (no latent: the home rank computes its own), and the last
// CTA of a home rank's rows announces the epoch there.
__global__ void __launch_bounds__(128) k_partial_output(Layer L, Workspace ws,
                                                        const uint8_t* padding, float* combined,
                                                        int fixed, Exchange x, int peers) {
  __shared__ int slot_end[32];
  __shared__ float slot_weight[32];
  const int t = blockIdx.y, tid = threadIdx.x, h = blockIdx.x * 128 + tid;
  float* routed_out = combined + static_cast<size_t>(t) * (L.H + L.R);
  const bool padded = padding && padding[t];
  if (peers) {
    // grid (ceil(H / 512), T): four adjacent columns per thread, so that a row crosses
    // NVLink in 16-byte stores and a quarter of the CTAs fence and arrive.
    const int h4 = (blockIdx.x * 128 + tid) * 4;
    const int home = t / x.tokens, row = t - home * x.tokens;
    routed_out = reinterpret_cast<float*>(x.block[home] +
                                          exchange_rows_offset(x.world, x.tokens, L.F)) +
                 (static_cast<size_t>(x.rank) * x.tokens + row) * L.H;
    float4 routed = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (!padded) {
      if (tid < L.K) {
        slot_end[tid] = down_slot_end(L, ws, t, tid, fixed);
        slot_weight[tid] = ws.weights[static_cast<size_t>(t) * L.K + tid];
      }
      __syncthreads();
      if (h4 < L.H)
        routed = mix_down_tiles4(
            ws.down_parts + static_cast<size_t>(t) * ws.down_tiles * L.H + h4, slot_end[L.K - 1],
            L.H, slot_end, slot_weight);
    }
    if (h4 < L.H) *reinterpret_cast<float4*>(routed_out + h4) = routed;
    uint32_t* header = exchange_header(x, x.rank);
    exchange_announce(header + kExchangeRowsArrive + home, gridDim.x * x.tokens,
                      exchange_header(x, home) + kExchangeRowsFlag + x.rank,
                      header[kExchangeEpoch] + 1u);
    return;
  }
  if (blockIdx.x == 0)  // this rank's share of the latent rides behind the H outputs
    for (int r = tid; r < L.R; r += 128)
      routed_out[L.H + r] = padded ? 0.0f : ws.latent[static_cast<size_t>(t) * L.R + r];
  if (padded) {
    routed_out[h] = 0.0f;
    return;
  }
  if (tid < L.K) {
    const size_t pair = static_cast<size_t>(t) * L.K + tid;
    slot_end[tid] = down_slot_end(L, ws, t, tid, fixed);
    slot_weight[tid] = ws.weights[pair];
  }
  __syncthreads();
  routed_out[h] = mix_down_tiles(
      ws.down_parts + static_cast<size_t>(t) * ws.down_tiles * L.H + h, slot_end[L.K - 1], L.H,
      slot_end, slot_weight);
}

__global__ void __launch_bounds__(128) k_finish(Layer L, const float* combined,
                                                const float* latent_rows, __nv_bfloat16* out) {
  __shared__ float latent[256];
  const int t = blockIdx.y, tid = threadIdx.x, h = blockIdx.x * 128 + tid;
  // The latent rides behind the H sums of a row unless it is given on its own.
  const float* row_in = combined + static_cast<size_t>(t) * (latent_rows ? L.H : L.H + L.R);
  const float* latent_in = latent_rows ? latent_rows + static_cast<size_t>(t) * L.R : row_in + L.H;
  const bool recover = L.R > 0 && L.decoder;
  float correction = 0.0f;
  if (recover) {
    for (int r = tid; r < L.R; r += 128)
      latent[r] = bf16_round(latent_in[r]);
    __syncthreads();
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
  out[static_cast<size_t>(t) * L.H + h] =
      __float2bfloat16_rn(row_in[h] + correction);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
struct Bound {
  Layer L;
  Workspace ws;
  cudaStream_t stream;
  int T;
  int row_offset;  // first workspace row of the call (cfm_select only)
  const uint8_t* padding;
};

static int bind_call(const cfm_layer* layer, void* workspace, int32_t capacity,
                     const cfm_call* call, void* stream, Bound* b) {
  if (!layer || !workspace || !call) return CFM_E_NULL;
  cfm_workspace_layout layout;
  const int rc = make_layout(layer, capacity, &layout);
  if (rc) return rc;
  if (call->tokens < 1 || call->row_offset < 0 || call->tokens + call->row_offset > capacity)
    return CFM_E_CAPACITY;
  if (layer->experts < 1) return CFM_E_SHAPE;
  if (layer->activation != CFM_ACT_SILU && layer->activation != CFM_ACT_GELU_TANH)
    return CFM_E_UNSUPPORTED;
  if (layer->score != CFM_SCORE_POINT && layer->score != CFM_SCORE_RECOVERY_AWARE)
    return CFM_E_UNSUPPORTED;
  if (layer->row_engine < CFM_ROWS_AUTO || layer->row_engine > CFM_ROWS_EXPERT_MAJOR)
    return CFM_E_UNSUPPORTED;
  const bool screened = layer->final_count < layer->top_k * layer->width;
  if (screened && (!layer->sketch || !layer->statistics || !layer->norms || !layer->signs))
    return CFM_E_NULL;
  if (layer->rank && (!layer->encoder || !layer->decoder)) return CFM_E_NULL;
  b->L = device_layer(layer);
  b->ws = bind(layout, workspace, capacity);
  b->stream = static_cast<cudaStream_t>(stream);
  b->T = call->tokens;
  b->row_offset = call->row_offset;
  b->padding = call->padding;
  return 0;
}

// Launch with programmatic stream serialisation: the kernel may be scheduled while its
// predecessor in the stream is finishing and waits for it at grid_dependency_wait().
// Used for the selection after the screen and for the exact gather after the selection
// (measured: 0.6 to 1.3 us per call).  CFM_PDL=0 in the environment makes these ordinary
// launches.
template <typename... Params, typename... Args>
static void launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
  static const bool on = [] {
    const char* v = std::getenv("CFM_PDL");
    return !v || std::atoi(v) != 0;
  }();
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = on ? 1 : 0;
  (void)cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

static int launched() {
  const cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? 0 : static_cast<int>(err);
}

static int run_prepare(const Bound& b, const cfm_call* call) {
  if (b.L.F >= b.L.N) return 0;
  if (!call->hidden) return CFM_E_NULL;
  k_prepare<<<dim3(b.T, b.L.B), kBlock, 0, b.stream>>>(
      b.L, b.ws, static_cast<const __nv_bfloat16*>(call->hidden), b.padding);
  return launched();
}

// Batch size from which the screen runs expert-major on the tensor cores.
constexpr int kGroupedScreenTokens = 8;

static bool screens_grouped(const Bound& b) {
  return b.L.F < b.L.N && b.L.sketch_grouped && b.T >= kGroupedScreenTokens && b.L.E <= 4096;
}

static int run_route(const Bound& b, const cfm_call* call) {
  if (!call->ids || !call->weights) return CFM_E_NULL;
  k_route<<<b.T, 32, 0, b.stream>>>(b.L, b.ws, call->ids, call->ids_are_int64, call->weights,
                                    call->weights_are_bf16);
  int rc = launched();
  if (rc || !screens_grouped(b)) return rc;
  // The expert-major screen reads the (token, slot) pairs grouped by expert.
  k_group<<<1, 1024, 2 * sizeof(int) * b.L.E, b.stream>>>(b.L, b.ws, b.padding, b.T);
  return launched();
}

template <int CG>
static int launch_screen(const Bound& b, int S) {
  const int threads = b.L.W * CG;
  const size_t smem = sizeof(int) * (2 * kBlock + (CG > 1 ? CG * kWordRows * b.L.W : 0));
  if (smem > 48 * 1024) {
    const cudaError_t err = cudaFuncSetAttribute(
        k_screen<CG>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  k_screen<CG><<<dim3(b.T * b.L.K, S), threads, smem, b.stream>>>(b.L, b.ws, b.padding, S);
  return launched();
}

static int run_screen_grouped(const Bound& b) {
  int rc = 0;
  // Experts with many tokens (few local experts under expert parallelism) spread
  // their passes of eight tokens over grid.z.
  const int64_t per_expert = (static_cast<int64_t>(b.T) * b.L.K + b.L.E - 1) / b.L.E;
  const int passes = static_cast<int>(std::min<int64_t>(8, std::max<int64_t>(1, (per_expert + 7) / 8)));
  const dim3 grid((2 * b.L.I + kGroupWarps * 16 - 1) / (kGroupWarps * 16), b.L.E, passes);
  const size_t tc_bytes = tc::shared_bytes(b.L.B);
  if (b.L.tensor_engine == CFM_ENGINE_TCGEN05 && tc_bytes <= 200 * 1024) {
    const cudaError_t err = cudaFuncSetAttribute(
        k_screen_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(tc_bytes));
    if (err != cudaSuccess) return static_cast<int>(err);
    const int tc_passes = static_cast<int>(
        std::min<int64_t>(8, std::max<int64_t>(1, (per_expert + tc::kTokens - 1) / tc::kTokens)));
    k_screen_tc<<<dim3(grid.x, grid.y, tc_passes), tc::kThreads, tc_bytes, b.stream>>>(b.L, b.ws);
  } else if (per_expert < 8 && (reinterpret_cast<uintptr_t>(b.L.sketch_grouped) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(b.L.statistics) & 15) == 0) {
    // Up to eight tokens per expert on average (one pass for most experts): two row
    // tiles per warp share the digit fragments.  Measured on the benchmark shapes
    // against the one-tile kernel: 61 vs 67 us (128 experts of width 768, 64 tokens),
    // 157 vs 257 us (hidden 4096, width 1536, 32 tokens); with eight and more tokens
    // per expert (256 experts of width 512, 256 tokens) the one-tile kernel, which
    // has the digits of the next block in registers, is ahead (214 vs 231 us).
    const dim3 wide((2 * b.L.I + kRows32Warps * 32 - 1) / (kRows32Warps * 32), b.L.E, passes);
    k_screen_rows32<<<wide, kRows32Warps * 32, 0, b.stream>>>(b.L, b.ws);
  } else {
    k_screen_grouped<<<grid, kGroupWarps * 32, 0, b.stream>>>(b.L, b.ws);
  }
  if ((rc = launched())) return rc;
  if (b.padding || b.L.expert_map) {
    k_clear_dead<<<dim3(b.T, (b.L.N + 255) / 256), 256, 0, b.stream>>>(b.L, b.ws, b.padding);
    rc = launched();
  }
  return rc;
}

static int run_screen_projections(const Bound& b);

static int run_screen(const Bound& b) {
  if (b.L.F >= b.L.N) return 0;
  if (b.L.score == CFM_SCORE_RECOVERY_AWARE) {
    k_variance<<<dim3(b.T * b.L.K, (2 * b.L.I + 255) / 256), 256, 0, b.stream>>>(b.L, b.ws,
                                                                                 b.padding);
    const int rc = launched();
    if (rc) return rc;
  }
  return run_screen_projections(b);
}

static int run_screen_projections(const Bound& b) {
  if (screens_grouped(b)) return run_screen_grouped(b);
  // Split the rotation blocks across CTAs while the batch is too small to fill
  // the 148 SMs; large batches keep each pair's blocks in one CTA.
  const int pairs = b.T * b.L.K;
  int S = 1;
  if (b.T <= b.ws.parts_tokens) {
    while (S < b.L.B && pairs * S < 2 * 148) S *= 2;
    if (S > b.L.B) S = b.L.B;
  }
  // Coordinate groups: as many as keep the CTA within 512 threads, at most 4.
  int cg = 4;
  while (cg > 1 && b.L.W * cg > 512) cg >>= 1;
  if (b.L.W > 512) return CFM_E_SHAPE;  // I > 4096
  switch (cg) {
    case 4: return launch_screen<4>(b, S);
    case 2: return launch_screen<2>(b, S);
    default: return launch_screen<1>(b, S);
  }
}

static bool pairs_grouped(const Bound& b);

static int run_select(const Bound& b, int scores_ready, const Exchange* exchange = nullptr) {
  const size_t smem = sizeof(uint32_t) * b.L.N;
  if (smem + 10240 > 48 * 1024) {  // static shared memory counts against the default limit
    cudaError_t err = cudaFuncSetAttribute(
        k_select<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(k_select<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  if (exchange)
    launch_dependent(k_select<true>, dim3(b.T), dim3(kSelectThreads), smem, b.stream, b.L, b.ws,
                     b.padding, scores_ready, b.row_offset, *exchange);
  else
    launch_dependent(k_select<false>, dim3(b.T), dim3(kSelectThreads), smem, b.stream, b.L, b.ws,
                     b.padding, scores_ready, b.row_offset, NoExchange{});
  return launched();
}

// The down tiles of the call in expert order, once the selection is done.
static int run_list_tiles(const Bound& b) {
  if (!pairs_grouped(b) || !b.L.down) return 0;  // a layer without native rows has no down stage
  k_list_tiles<<<1, 1024, 0, b.stream>>>(b.L, b.ws);
  return launched();
}

static int run_score(const Bound& b) {
  if (b.L.F >= b.L.N) return 0;
  k_score<<<dim3(b.T, (b.L.N + 255) / 256), 256, 0, b.stream>>>(b.L, b.ws, b.padding);
  return launched();
}

// Batches whose pairs are grouped by expert also read the experts' native rows
// expert-major (the groups come from k_group, launched by route and adopt).
static bool pairs_grouped(const Bound& b) { return screens_grouped(b); }  // see run_select

// Expert-major exact, down and encode: a row is read once for all the tokens of
// its expert that kept it.  On the shapes measured so far (4 to 16 tokens per
// expert) the per-token kernels walking the pairs in expert order are faster: the
// rows several tokens share come from HBM once either way (from L2 after the
// first), and the per-token kernels keep more loads in flight.  So the automatic
// choice is per-token; the expert-major kernels run on request.
static bool rows_grouped(const Bound& b) {
  return pairs_grouped(b) && b.L.row_engine == CFM_ROWS_EXPERT_MAJOR;
}

// Partial sums per (token, local slot) of the expert-major down kernel: enough
// CTAs to fill the device, at most what the workspace has room for.
static int down_grouped_parts(const Bound& b) {
  const int64_t column_blocks = (b.L.H + kDownGroupedColumns - 1) / kDownGroupedColumns;
  const int64_t wanted = (8 * 148 + column_blocks * b.L.E - 1) / (column_blocks * b.L.E);
  const int64_t room = std::min<int64_t>(kDownGroupedMaxParts, b.ws.down_tiles / b.L.K);
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::max<int64_t>(2, wanted), room)));
}

static int run_exact_grouped(const Bound& b, const cfm_call* call) {
  // Entries of the per-channel token table: four times the mean number of kept
  // channels per expert, at least one expert's width (the largest one token can need).
  const int64_t mean = (static_cast<int64_t>(b.T) * b.L.F + b.L.E - 1) / b.L.E;
  const int entries = static_cast<int>(
      std::min<int64_t>(16384, std::max<int64_t>(b.L.I, 4 * mean)));
  const size_t smem = exact_grouped_bytes(b.L.I, entries);
  if (smem > 48 * 1024) {
    const cudaError_t err = cudaFuncSetAttribute(
        k_exact_grouped, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  const int parts = static_cast<int>(
      std::max<int64_t>(1, std::min<int64_t>(32, (4 * 148 + b.L.E - 1) / b.L.E)));
  k_exact_grouped<<<dim3(parts, b.L.E), kExactGroupedThreads, smem, b.stream>>>(
      b.L, b.ws, static_cast<const __nv_bfloat16*>(call->hidden), entries);
  return launched();
}

static int run_exact(const Bound& b, const cfm_call* call) {
  if (!call->hidden || !b.L.gate_up) return CFM_E_NULL;
  if (rows_grouped(b)) return run_exact_grouped(b, call);
  const size_t smem = static_cast<size_t>(b.L.H) * 2;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(
        k_exact, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(k_exact_pairs<false>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(k_exact_pairs<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  if (pairs_grouped(b)) {
    // One warp per kept row of a pair when the pair keeps the mean number of rows.
    const int per_pair = (b.L.F + b.L.K - 1) / b.L.K;
    const int ctas = std::max(1, (per_pair + kExactWarps - 1) / kExactWarps);
    int64_t rows = static_cast<int64_t>(b.T) * b.L.K;
    if (b.L.expert_map && b.L.global_experts > 0)  // twice the expected share of the pairs
      rows = std::max<int64_t>(8, std::min<int64_t>(
                                      rows, (2 * rows * b.L.E + b.L.global_experts - 1) /
                                                b.L.global_experts));
    if (rows < static_cast<int64_t>(b.T) * b.L.K)
      launch_dependent(k_exact_pairs<true>, dim3(ctas, static_cast<unsigned>(rows)),
                       dim3(kExactWarps * 32), smem, b.stream, b.L, b.ws,
                       static_cast<const __nv_bfloat16*>(call->hidden));
    else
      launch_dependent(k_exact_pairs<false>, dim3(ctas, static_cast<unsigned>(rows)),
                       dim3(kExactWarps * 32), smem, b.stream, b.L, b.ws,
                       static_cast<const __nv_bfloat16*>(call->hidden));
    return launched();
  }
  int ctas = (b.L.F + kExactWarps - 1) / kExactWarps;
  if (b.L.expert_map && b.L.global_experts > 0) {
    // Expert parallel: a rank holds E of the global experts, so about that share
    // of a token's kept channels; CTAs stride through the list, twice the
    // expected share of them are launched.
    const int64_t share = (2LL * ctas * b.L.E + b.L.global_experts - 1) / b.L.global_experts;
    ctas = static_cast<int>(std::max<int64_t>(8, std::min<int64_t>(ctas, share)));
  }
  launch_dependent(k_exact, dim3(ctas, b.T), dim3(kExactWarps * 32), smem, b.stream, b.L, b.ws,
                   static_cast<const __nv_bfloat16*>(call->hidden), b.padding);
  return launched();
}

// Passes the ring depth of the down kernels to `launch` as a compile-time constant.
template <typename Launch>
static int launch_down(Launch launch) {
  return launch(std::integral_constant<int, kDownStages>{});
}

static int run_down(const Bound& b) {
  if (!b.L.down) return CFM_E_NULL;
  if (rows_grouped(b)) {
    const size_t smem = down_grouped_bytes(b.L.I);
    if (smem > 48 * 1024) {
      const cudaError_t err = cudaFuncSetAttribute(
          k_down_grouped, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (err != cudaSuccess) return static_cast<int>(err);
    }
    const int parts = down_grouped_parts(b);
    const dim3 grid((b.L.H + kDownGroupedColumns - 1) / kDownGroupedColumns, b.L.E, parts);
    k_down_grouped<<<grid, kDownGroupedThreads, smem, b.stream>>>(b.L, b.ws, parts);
    return launched();
  }
  if (pairs_grouped(b)) {
    // The call's tiles were listed in expert order after the selection.
    int64_t most = static_cast<int64_t>(b.T) * ((b.L.F + kDownTileRows - 1) / kDownTileRows + b.L.K);
    if (b.L.expert_map && b.L.global_experts > 0)  // twice the expected share of the tiles
      most = std::max<int64_t>(8, std::min<int64_t>(
                                      most, (2 * most * b.L.E + b.L.global_experts - 1) /
                                                b.L.global_experts));
    const dim3 grid((b.L.H + kDownColumns - 1) / kDownColumns, static_cast<unsigned>(most));
    return launch_down([&](auto stages) {
      constexpr int S = decltype(stages)::value;
      cudaError_t err = cudaFuncSetAttribute(
          k_down_tiles<S>, cudaFuncAttributeMaxDynamicSharedMemorySize, down_ring_bytes(S));
      if (err != cudaSuccess) return static_cast<int>(err);
      k_down_tiles<S><<<grid, 128, down_ring_bytes(S), b.stream>>>(b.L, b.ws);
      return launched();
    });
  }
  int tiles = b.ws.down_tiles;
  if (b.L.expert_map && b.L.global_experts > 0) {
    // Expert parallel: about E / global of a token's tiles are local; twice that
    // share of CTAs is launched per token and walks the tiles in strides.
    const int64_t share = (2LL * tiles * b.L.E + b.L.global_experts - 1) / b.L.global_experts;
    tiles = static_cast<int>(std::max<int64_t>(2, std::min<int64_t>(tiles, share)));
  }
  const dim3 grid((b.L.H + kDownColumns - 1) / kDownColumns, tiles, b.T);
  return launch_down([&](auto stages) {
    constexpr int S = decltype(stages)::value;
    cudaError_t err = cudaFuncSetAttribute(
        k_down<true, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, down_ring_bytes(S));
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(k_down<false, S>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 down_ring_bytes(S));
    if (err != cudaSuccess) return static_cast<int>(err);
    if (tiles < b.ws.down_tiles)
      k_down<true, S><<<grid, 128, down_ring_bytes(S), b.stream>>>(b.L, b.ws, b.padding);
    else
      k_down<false, S><<<grid, 128, down_ring_bytes(S), b.stream>>>(b.L, b.ws, b.padding);
    return launched();
  });

}

static int run_encode(const Bound& b) {
  if (b.L.R == 0) return 0;
  if (b.L.F >= b.L.N) {
    k_zero_latent<<<b.T, 128, 0, b.stream>>>(b.L, b.ws);
    return launched();
  }
  if (rows_grouped(b) && !b.L.expert_map) {
    const size_t smem = encode_grouped_bytes(b.L.R);
    if (smem > 48 * 1024) {
      const cudaError_t err = cudaFuncSetAttribute(
          k_encode_grouped, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (err != cudaSuccess) return static_cast<int>(err);
    }
    k_encode_grouped<<<dim3(b.ws.encoder_tiles, b.L.E), kEncodeThreads, smem, b.stream>>>(b.L, b.ws);
    return launched();
  }
  k_encode<<<dim3(b.ws.encoder_tiles, b.T * b.L.K), kEncodeThreads, 0, b.stream>>>(b.L, b.ws, b.padding);
  return launched();
}

static int run_output(const Bound& b, const cfm_call* call) {
  if (!call->out) return CFM_E_NULL;
  k_output<<<dim3(b.L.H / 128, b.T), 128, 0, b.stream>>>(
      b.L, b.ws, b.padding, static_cast<__nv_bfloat16*>(call->out),
      rows_grouped(b) ? down_grouped_parts(b) : 0);
  return launched();
}

// One side stream and two events per device, created on the first whole-layer
// call on that device (make that call outside stream capture).
struct SideStream {
  cudaStream_t stream;
  cudaEvent_t fork, join, tiles;
  std::mutex* sequence;  // held while a whole-layer call enqueues its fork .. join sequence
  bool ready;
};
static SideStream g_side[64];
static std::mutex g_side_sequence[64];
static std::mutex g_side_lock;

static int side_stream(SideStream* out) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return -1;
  std::lock_guard<std::mutex> guard(g_side_lock);
  SideStream& slot = g_side[device];
  if (!slot.ready) {
    int low = 0, high = 0;
    if (cudaDeviceGetStreamPriorityRange(&low, &high) != cudaSuccess) return -1;
    if (cudaStreamCreateWithPriority(&slot.stream, cudaStreamNonBlocking, high) != cudaSuccess) {
      (void)cudaGetLastError();
      return -1;
    }
    if (cudaEventCreateWithFlags(&slot.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&slot.join, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&slot.tiles, cudaEventDisableTiming) != cudaSuccess) {
      (void)cudaGetLastError();
      return -1;
    }
    slot.sequence = &g_side_sequence[device];
    slot.ready = true;
  }
  *out = slot;
  return 0;
}

// Checks an exchange description against the layer and the call (`rows` = tokens
// of all ranks) and makes the device-visible copy.
static int bind_exchange(const cfm_exchange* e, const cfm_layer* layer, int rows, Exchange* out) {
  if (!e || !layer) return CFM_E_NULL;
  if (e->world < 1 || e->world > CFM_MAX_RANKS || e->rank < 0 || e->rank >= e->world ||
      e->tokens < 1)
    return CFM_E_SHAPE;
  if (rows != e->world * e->tokens) return CFM_E_CAPACITY;
  out->world = e->world;
  out->rank = e->rank;
  out->tokens = e->tokens;
  for (int p = 0; p < CFM_MAX_RANKS; ++p) {
    out->block[p] = p < e->world ? static_cast<char*>(e->blocks[p]) : nullptr;
    if (p < e->world && !e->blocks[p]) return CFM_E_NULL;
  }
  return 0;
}

}  // namespace cfm

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
using namespace cfm;

extern "C" {

int cfm_abi_version(void) { return CFM_ABI_VERSION; }

const char* cfm_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case CFM_E_NULL: return "a required pointer is NULL";
    case CFM_E_SHAPE: return "a dimension violates the layer contract";
    case CFM_E_CAPACITY: return "token count outside the workspace capacity";
    case CFM_E_UNSUPPORTED: return "option not supported by this build";
    case CFM_E_STATIC_CAPACITY: return "batch exceeds the library-owned scratch of cfm_screen_static";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error";
  }
}

int cfm_workspace_layout_for(const cfm_layer* layer, int32_t capacity,
                             cfm_workspace_layout* layout) {
  return make_layout(layer, capacity, layout);
}

#define CFM_STAGE(name, body)                                                      \
  int name(const cfm_layer* layer, void* workspace, int32_t capacity,             \
           const cfm_call* call, void* stream) {                                   \
    Bound b;                                                                       \
    const int rc = bind_call(layer, workspace, capacity, call, stream, &b);        \
    if (rc) return rc;                                                             \
    body                                                                           \
  }

CFM_STAGE(cfm_prepare_input, return run_prepare(b, call);)
CFM_STAGE(cfm_route, return run_route(b, call);)
CFM_STAGE(cfm_screen, return run_screen(b);)
CFM_STAGE(cfm_select, {
  // With an exchange in the call (home rank of an expert-parallel layer, plain
  // selection of its own rows) the kernel also sends the kept lists to all ranks.
  Exchange x = {};
  const bool send = call->exchange != nullptr && call->scores_ready == 0;
  if (send) {
    const int bound = bind_exchange(call->exchange, layer, call->exchange->world * b.T, &x);
    if (bound) return bound;
    if (b.row_offset != 0) return CFM_E_CAPACITY;
  }
  const int code = run_select(b, call->scores_ready, send ? &x : nullptr);
  // Mode 3 only publishes the cut; every other mode leaves final counts behind.
  return code || call->scores_ready == 3 ? code : run_list_tiles(b);
})
CFM_STAGE(cfm_score, return run_score(b);)
CFM_STAGE(cfm_list_tiles, return run_list_tiles(b);)
CFM_STAGE(cfm_exact, return run_exact(b, call);)
CFM_STAGE(cfm_down, return run_down(b);)
CFM_STAGE(cfm_encode, return run_encode(b);)
CFM_STAGE(cfm_output, return run_output(b, call);)

int cfm_partial_output(const cfm_layer* layer, void* workspace, int32_t capacity,
                       const cfm_call* call, void* stream) {
  Bound b;
  const int rc = bind_call(layer, workspace, capacity, call, stream, &b);
  if (rc) return rc;
  Exchange x = {};
  const int peers = call->exchange != nullptr;
  if (peers) {
    const int code = bind_exchange(call->exchange, layer, b.T, &x);
    if (code) return code;
  } else if (!call->out) {
    return CFM_E_NULL;
  }
  k_partial_output<<<dim3(peers ? (b.L.H + 511) / 512 : b.L.H / 128, b.T), 128, 0, b.stream>>>(
      b.L, b.ws, b.padding, static_cast<float*>(call->out),
      rows_grouped(b) ? down_grouped_parts(b) : 0, x, peers);
  return launched();
}

int cfm_finish(const cfm_layer* layer, int32_t tokens, const float* combined,
               const float* latent, void* out, void* stream) {
  if (!layer || !combined || !out) return CFM_E_NULL;
  cfm_workspace_layout layout;
  const int rc = make_layout(layer, 1, &layout);  // validates the dimensions
  if (rc) return rc;
  if (tokens < 1) return CFM_E_CAPACITY;
  const Layer L = device_layer(layer);
  k_finish<<<dim3(L.H / 128, tokens), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      L, combined, latent, static_cast<__nv_bfloat16*>(out));
  return launched();
}

int cfm_adopt(const cfm_layer* layer, void* workspace, int32_t capacity, const cfm_call* call,
              void* stream) {
  Bound b;
  const int rc = bind_call(layer, workspace, capacity, call, stream, &b);
  if (rc) return rc;
  if (!call->ids || !call->weights || (!call->lists && !call->exchange)) return CFM_E_NULL;
  Exchange x = {};
  const int peers = call->exchange != nullptr;
  if (peers) {
    const int bound = bind_exchange(call->exchange, layer, b.T, &x);
    if (bound) return bound;
  }
  k_adopt<<<b.T, 256, 0, b.stream>>>(b.L, b.ws, call->ids, call->ids_are_int64, call->weights,
                                     call->weights_are_bf16, b.padding, call->lists, x, peers);
  int code = launched();
  if (code || !pairs_grouped(b)) return code;
  // The exact and down kernels read the pairs grouped by expert; the down tiles are
  // listed by cfm_list_tiles, which may run beside cfm_exact.
  k_group<<<1, 1024, 2 * sizeof(int) * b.L.E, b.stream>>>(b.L, b.ws, b.padding, b.T);
  return launched();
}

int cfm_build_sketch(const cfm_layer* layer, const void* gate_up, const int8_t* signs,
                     uint32_t* sketch, uint32_t* sketch_grouped, void* statistics, void* stream) {
  if (!layer || !gate_up || !signs || !sketch || !sketch_grouped || !statistics) return CFM_E_NULL;
  const int64_t H = layer->hidden, I = layer->width, E = layer->experts;
  if (H <= 0 || H % kBlock || I <= 0 || I % 16 || E < 1 || E > 65535 || 2 * I / kBuildRows > 65535)
    return CFM_E_SHAPE;
  const dim3 grid(static_cast<unsigned>(H / kBlock), static_cast<unsigned>(2 * I / kBuildRows),
                  static_cast<unsigned>(E));
  k_build_sketch<<<grid, kBuildRows * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<int>(H), static_cast<int>(I), static_cast<const __nv_bfloat16*>(gate_up), signs,
      sketch, sketch_grouped, static_cast<__half*>(statistics));
  return launched();
}

int64_t cfm_exchange_bytes(const cfm_layer* layer, int32_t world, int32_t tokens) {
  if (!layer || world < 1 || world > CFM_MAX_RANKS || tokens < 1) return 0;
  return static_cast<int64_t>(
      exchange_bytes(world, tokens, layer->final_count, layer->hidden));
}

int cfm_peer_alloc(int64_t bytes, void** block) {
  if (!block || bytes < 1) return CFM_E_NULL;
  cudaError_t err = cudaMalloc(block, static_cast<size_t>(bytes));
  if (err == cudaSuccess) err = cudaMemset(*block, 0, static_cast<size_t>(bytes));
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  return static_cast<int>(err);
}

int cfm_peer_export(void* block, void* handle) {
  if (!block || !handle) return CFM_E_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == CFM_PEER_HANDLE_BYTES, "handle size");
  return static_cast<int>(
      cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle), block));
}

int cfm_peer_import(const void* handle, void** block) {
  if (!block || !handle) return CFM_E_NULL;
  cudaIpcMemHandle_t copy;
  memcpy(&copy, handle, sizeof(copy));
  return static_cast<int>(cudaIpcOpenMemHandle(block, copy, cudaIpcMemLazyEnablePeerAccess));
}

int cfm_peer_release(void* block, int32_t imported) {
  if (!block) return 0;
  return static_cast<int>(imported ? cudaIpcCloseMemHandle(block) : cudaFree(block));
}

int cfm_exchange_status(const cfm_exchange* exchange, int32_t* status) {
  if (!exchange || !status || exchange->rank < 0 || exchange->rank >= CFM_MAX_RANKS ||
      !exchange->blocks[exchange->rank])
    return CFM_E_NULL;
  uint32_t word = 0;
  const cudaError_t err = cudaMemcpy(
      &word, static_cast<const uint32_t*>(exchange->blocks[exchange->rank]) + kExchangeStatus,
      sizeof(word), cudaMemcpyDeviceToHost);
  *status = static_cast<int32_t>(word);
  return static_cast<int>(err);
}

int cfm_finish_rows(const cfm_layer* layer, const cfm_exchange* exchange, const float* latent,
                    void* out, void* stream) {
  if (!layer || !exchange || !out) return CFM_E_NULL;
  cfm_workspace_layout layout;
  const int rc = make_layout(layer, 1, &layout);  // validates the dimensions
  if (rc) return rc;
  Exchange x = {};
  const int bound = bind_exchange(exchange, layer, exchange->world * exchange->tokens, &x);
  if (bound) return bound;
  const Layer L = device_layer(layer);
  k_finish_rows<<<dim3(L.H / 128, x.tokens), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      L, x, latent, static_cast<__nv_bfloat16*>(out));
  return launched();
}

int cfm_reader_forward(const cfm_layer* layer, void* workspace, int32_t capacity,
                       const cfm_call* call, void* stream) {
  Bound b;
  int rc = bind_call(layer, workspace, capacity, call, stream, &b);
  if (rc) return rc;
  if (!layer->gate_up || !layer->down) return CFM_E_NULL;
  SideStream side;
  const bool have_side = b.L.F < b.L.N && side_stream(&side) == 0;
  // The side stream and its two events are shared by every whole-layer call on the
  // device: the enqueue sequence below runs under the device's lock, so calls from
  // several host threads do not interleave their fork and join points.
  std::unique_lock<std::mutex> sequence;
  if (have_side) sequence = std::unique_lock<std::mutex>(*side.sequence);
  // After a fork the caller's stream must wait for the side stream again whatever
  // happens, or a capture of the caller's stream would be left with an unjoined branch.
  bool forked = false;
  auto leave = [&](int code) {
    if (forked) {
      (void)cudaEventRecord(side.join, side.stream);
      (void)cudaStreamWaitEvent(b.stream, side.join, 0);
      forked = false;
    }
    return code;
  };
  auto fork_side = [&]() {
    cudaError_t err = cudaEventRecord(side.fork, b.stream);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(side.stream, side.fork, 0);
    if (err == cudaSuccess) forked = true;
    return static_cast<int>(err);
  };
  auto join_side = [&]() {
    cudaError_t err = cudaEventRecord(side.join, side.stream);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(b.stream, side.join, 0);
    forked = false;
    return static_cast<int>(err);
  };
  Bound on_side = b;
  if (have_side) on_side.stream = side.stream;
  if (have_side && !call->input_prepared) {
    // Routing (and the grouping by expert) does not depend on the rotated input:
    // it runs on the side stream beside the rotation.
    if ((rc = fork_side())) return leave(rc);
    if ((rc = run_route(on_side, call))) return leave(rc);
    if ((rc = run_prepare(b, call))) return leave(rc);
    if ((rc = join_side())) return leave(rc);
  } else {
    if (!call->input_prepared && (rc = run_prepare(b, call))) return rc;
    if ((rc = run_route(b, call))) return rc;
  }
  if ((rc = run_screen(b))) return rc;
  if ((rc = run_select(b, 0))) return rc;
  // The listing of the down tiles and the recovery encoder (L2-resident rows,
  // arithmetic) run on the side stream beside the two HBM-bound gathers; the down
  // kernel waits for the list, the output mix for the encoder.
  const bool fork = have_side && (b.L.R > 0 || pairs_grouped(b));
  if (fork) {
    if ((rc = fork_side())) return leave(rc);
    if ((rc = run_list_tiles(on_side))) return leave(rc);
    if (cudaEventRecord(side.tiles, side.stream) != cudaSuccess) return leave(static_cast<int>(cudaGetLastError()));
    if ((rc = run_encode(on_side))) return leave(rc);
  } else if ((rc = run_list_tiles(b))) {
    return rc;
  }
  if ((rc = run_exact(b, call))) return leave(rc);
  if (fork && cudaStreamWaitEvent(b.stream, side.tiles, 0) != cudaSuccess)
    return leave(static_cast<int>(cudaGetLastError()));
  if ((rc = run_down(b))) return leave(rc);
  if (fork) {
    if ((rc = join_side())) return leave(rc);
  } else if ((rc = run_encode(b))) {
    return rc;
  }
  return run_output(b, call);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Screen with library-owned scratch (no allocation by anyone at call time)
// ---------------------------------------------------------------------------
// Scratch of cfm_screen_static: the per-block products of the split screen and
// its arrival counters.  The arrays live in the library image, so every GPU
// that loads the library holds them (4 MiB + 4 KiB) until the process exits.
// All calls on a device share them.
static __device__ __align__(256) float g_static_parts[CFM_STATIC_PARTS_FLOATS];
static __device__ __align__(256) unsigned int g_static_counters[CFM_STATIC_MAX_PAIRS];

namespace {
constexpr int kMaxDevices = 64;
struct StaticScratch {
  float* parts;
  unsigned int* counters;
  bool ready;
};
StaticScratch g_scratch[kMaxDevices];
std::mutex g_scratch_lock;

// Resolves the device addresses of the two arrays for the current device.  In
// host code the array names are only handles; kernels need the addresses
// cudaGetSymbolAddress returns for the device that is current.
int static_scratch(StaticScratch* out) {
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (device < 0 || device >= kMaxDevices) return CFM_E_UNSUPPORTED;
  std::lock_guard<std::mutex> guard(g_scratch_lock);
  StaticScratch& slot = g_scratch[device];
  if (!slot.ready) {
    void* parts = nullptr;
    void* counters = nullptr;
    err = cudaGetSymbolAddress(&parts, g_static_parts);
    if (err != cudaSuccess) return static_cast<int>(err);
    err = cudaGetSymbolAddress(&counters, g_static_counters);
    if (err != cudaSuccess) return static_cast<int>(err);
    slot.parts = static_cast<float*>(parts);
    slot.counters = static_cast<unsigned int*>(counters);
    slot.ready = true;
  }
  *out = slot;
  return 0;
}
}  // namespace

extern "C" int cfm_screen_static(const cfm_layer* layer, const cfm_static_screen* io,
                                 void* stream) {
  if (!layer || !io) return CFM_E_NULL;
  if (!io->ids || !io->quantized || !io->coordinates || !io->exponents || !io->partial ||
      !layer->sketch || !layer->statistics)
    return CFM_E_NULL;
  cfm_workspace_layout layout;
  int rc = make_layout(layer, 1, &layout);  // validates the dimensions
  if (rc) return rc;
  const Layer L = device_layer(layer);
  if (L.F >= L.N) return CFM_E_SHAPE;  // unscreened plans have no screen
  if (L.W > 512) return CFM_E_SHAPE;
  if (io->tokens < 1) return CFM_E_CAPACITY;
  const int64_t pairs = static_cast<int64_t>(io->tokens) * L.K;
  if (pairs > CFM_STATIC_MAX_PAIRS ||
      pairs * L.B * 2 * L.I > static_cast<int64_t>(CFM_STATIC_PARTS_FLOATS))
    return CFM_E_STATIC_CAPACITY;
  StaticScratch scratch;
  if ((rc = static_scratch(&scratch))) return rc;

  Workspace ws = {};
  ws.ids = const_cast<int32_t*>(io->ids);
  ws.quantized = const_cast<int32_t*>(io->quantized);
  ws.coordinates = const_cast<int32_t*>(io->coordinates);
  ws.exponents = const_cast<int32_t*>(io->exponents);
  ws.parts = scratch.parts;
  ws.counters = scratch.counters;
  ws.partial = io->partial;
  ws.parts_tokens = io->tokens;
  ws.capacity = io->tokens;
  Bound b;
  b.L = L;
  b.ws = ws;
  b.stream = static_cast<cudaStream_t>(stream);
  b.T = io->tokens;
  b.row_offset = 0;
  b.padding = io->padding;
  // The arrival counters must start at zero; the products need no clearing
  // (every entry that is read has been written by this call).
  const cudaError_t err = cudaMemsetAsync(scratch.counters, 0, sizeof(unsigned int) * pairs,
                                          b.stream);
  if (err != cudaSuccess) return static_cast<int>(err);
  // The recovery-aware score also reads the residual variances of the projections;
  // that kernel needs no scratch and runs when the caller asks for them.
  if (io->variances) {
    if (!io->energies) return CFM_E_NULL;
    b.ws.norms = const_cast<float*>(io->energies);
    b.ws.variances = io->variances;
    k_variance<<<dim3(b.T * L.K, (2 * L.I + 255) / 256), 256, 0, b.stream>>>(b.L, b.ws, b.padding);
    if ((rc = launched())) return rc;
  }
  // Always split the rotation blocks across CTAs, so the scratch is what joins them.
  int S = 2;
  while (S < L.B && pairs * S < 2 * 148) S *= 2;
  if (S > L.B) S = L.B;
  if (L.B == 1) S = 1;
  int cg = 4;
  while (cg > 1 && L.W * cg > 512) cg >>= 1;
  switch (cg) {
    case 4: return launch_screen<4>(b, S);
    case 2: return launch_screen<2>(b, S);
    default: return launch_screen<1>(b, S);
  }
}
