// Expert-major exact gate/up, down and recovery-encode kernels (sm_100a).
//
// From eight tokens per call the (token, expert) pairs are grouped by expert
// (k_group).  The kernels here walk one expert at a time: a row of the expert's
// weights that several of its tokens kept is read from HBM once and applied to
// all of them, instead of once per token as the per-token kernels do.
//
//   k_exact_grouped   gate and up rows of the union of the kept channels
//   k_down_grouped    channel-major down rows of the same union
//   k_encode_grouped  recovery-encoder rows, applied to every token of the expert
//
// Every CTA rebuilds, in shared memory, what it needs to know about its expert
// from the kept lists of the expert's tokens (a few hundred list entries): no
// kernel of its own and no global scratch for the unions.  Included by
// cfm_reader.cu inside namespace cfm, after Layer and Workspace.
#pragma once

// Tokens of one expert a CTA of k_exact_grouped tabulates at a time.
constexpr int kExactChunkTokens = 128;
constexpr int kExactGroupedThreads = 256;
// Tokens whose dot products share one pass over a row's registers.
constexpr int kExactTogether = 4;

// Tokens of one expert whose partial sums a CTA of k_down_grouped (and of
// k_encode_grouped) keeps in registers at a time.
constexpr int kDownChunkTokens = 8;
constexpr int kDownGroupedColumns = 256;  // output columns per CTA: 8 per lane
constexpr int kDownGroupedThreads = 128;

// (token, slot) of the j-th pair of expert e, and where its kept list starts.
struct GroupedToken {
  int t, slot, start, count;
};

__device__ __forceinline__ GroupedToken grouped_token(const Layer& L, const Workspace& ws,
                                                      int pair) {
  GroupedToken g;
  g.t = pair / L.K;
  g.slot = pair - g.t * L.K;
  g.start = ws.starts[pair];
  g.count = ws.counts[pair];
  return g;
}

// ---------------------------------------------------------------------------
// exact, expert-major
// ---------------------------------------------------------------------------
// grid (parts, E), 256 threads, dynamic shared memory exact_grouped_bytes().
// The CTAs of one expert each tabulate, per channel of the expert, the tokens
// that kept it (a compressed-row table built from the tokens' kept lists with
// shared-memory atomics), list the channels some token kept (the union) and
// share the union's rows round-robin: CTA `part` takes every parts-th row, its
// warps every eighth of those.  A warp holds one sweep (2048 columns) of the gate
// and the up row in registers, 16 bytes per lane and load, and runs the dot
// products of up to four of the row's tokens against the tokens' inputs (read
// through L1) in the order the per-token kernel uses, so both give the same
// bits.  Experts with more tokens or kept channels than the table holds are
// done in several chunks of tokens.
__host__ __device__ inline size_t exact_grouped_bytes(int I, int entries) {
  return sizeof(int) * (static_cast<size_t>(3) * I + 1 + 4 * kExactChunkTokens + 40) +
         sizeof(uint32_t) * static_cast<size_t>(entries);
}

__global__ void __launch_bounds__(kExactGroupedThreads, 2)
    k_exact_grouped(Layer L, Workspace ws, const __nv_bfloat16* hidden, int entries) {
  extern __shared__ int exact_smem[];
  const int I = L.I;
  int* offset = exact_smem;                    // [I + 1]
  int* cursor = offset + I + 1;                // [I]
  int* unions = cursor + I;                    // [I]
  int* tok_t = unions + I;                     // [kExactChunkTokens] each
  int* tok_slot = tok_t + kExactChunkTokens;
  int* tok_start = tok_slot + kExactChunkTokens;
  int* tok_count = tok_start + kExactChunkTokens;
  int* scratch = tok_count + kExactChunkTokens;  // [40]
  uint32_t* entry = reinterpret_cast<uint32_t*>(scratch + 40);

  const int e = blockIdx.y, part = blockIdx.x, parts = gridDim.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kWarps = kExactGroupedThreads / 32;
  const int first = ws.group_offsets[e], total = ws.group_offsets[e + 1] - first;
  if (total <= 0) return;
  const int chunks = L.H / 8;  // 16-byte pieces per row
  const int per = (I + kExactGroupedThreads - 1) / kExactGroupedThreads;

  for (int begin = 0; begin < total;) {
    // ---- the chunk of tokens: as many as the table holds ----
    int mine = 0;
    if (tid < kExactChunkTokens && begin + tid < total) {
      const GroupedToken g = grouped_token(L, ws, ws.group_pairs[first + begin + tid]);
      tok_t[tid] = g.t;
      tok_slot[tid] = g.slot;
      tok_start[tid] = g.start;
      tok_count[tid] = g.count;
      mine = g.count;
    }
    int all = 0;
    const int before = block_exclusive_scan(mine, scratch, &all);
    // Tokens whose entries end within the table; the first always fits (a token
    // keeps at most I channels of one expert and the table holds at least I).
    const bool fits = tid < kExactChunkTokens && begin + tid < total &&
                      (tid == 0 || before + mine <= entries);
    const int tokens = __syncthreads_count(fits && tid < kExactChunkTokens);
    // `fits` is monotone (prefix sums grow), so the count is the chunk's length.
    for (int c = tid; c <= I; c += kExactGroupedThreads) offset[c] = 0;
    __syncthreads();
    // ---- how many tokens kept each channel ----
    for (int j = warp; j < tokens; j += kWarps) {
      const int32_t* list =
          ws.candidate_ids + static_cast<size_t>(tok_t[j]) * L.F + tok_start[j];
      const int base = tok_slot[j] * I;
      for (int k = lane; k < tok_count[j]; k += 32) atomicAdd(&offset[list[k] - base], 1);
    }
    __syncthreads();
    // ---- first entry of every channel; the union of kept channels ----
    int local = 0, kept = 0;
    for (int c = tid * per; c < min(I, (tid + 1) * per); ++c) {
      local += offset[c];
      kept += offset[c] > 0;
    }
    int rows = 0, sum = 0;
    int at = block_exclusive_scan(local, scratch, &sum);
    int row = block_exclusive_scan(kept, scratch, &rows);
    for (int c = tid * per; c < min(I, (tid + 1) * per); ++c) {
      const int count = offset[c];
      offset[c] = at;
      cursor[c] = at;
      if (count > 0) unions[row++] = c;
      at += count;
    }
    if (tid == 0) offset[I] = sum;
    __syncthreads();
    // ---- fill: token index within the chunk and position in its kept list ----
    for (int j = warp; j < tokens; j += kWarps) {
      const int32_t* list =
          ws.candidate_ids + static_cast<size_t>(tok_t[j]) * L.F + tok_start[j];
      const int base = tok_slot[j] * I;
      for (int k = lane; k < tok_count[j]; k += 32) {
        const int at_entry = atomicAdd(&cursor[list[k] - base], 1);
        entry[at_entry] = static_cast<uint32_t>(j) |
                          (static_cast<uint32_t>(tok_start[j] + k) << 8);
      }
    }
    __syncthreads();

    // ---- the union's rows ----
    for (int u = part + parts * warp; u < rows; u += parts * kWarps) {
      const int c = unions[u];
      const uint4* gate = reinterpret_cast<const uint4*>(
          L.gate_up + (static_cast<size_t>(e) * 2 * I + c) * L.H);
      const uint4* up = gate + static_cast<size_t>(I) * L.H / 8;
      const int lo = offset[c], hi = offset[c + 1];
      for (int g0 = lo; g0 < hi; g0 += kExactTogether) {
        const int count = min(kExactTogether, hi - g0);
        float g[kExactTogether], v[kExactTogether];
        const uint4* x[kExactTogether];
#pragma unroll
        for (int q = 0; q < kExactTogether; ++q) {
          g[q] = v[q] = 0.0f;
          const int j = static_cast<int>(entry[g0 + min(q, count - 1)] & 0xffu);
          x[q] = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(tok_t[j]) * L.H);
        }
        constexpr int U = 8;  // 16-byte pieces of each row in flight per lane
        for (int base = lane; base < chunks; base += 32 * U) {
          uint4 gw[U], uw[U];
          if (base + 32 * (U - 1) < chunks) {
#pragma unroll
            for (int k = 0; k < U; ++k) {
              gw[k] = load_stream16(gate + base + 32 * k);
              uw[k] = load_stream16(up + base + 32 * k);
            }
          } else {
#pragma unroll
            for (int k = 0; k < U; ++k) {
              const int i = base + 32 * k;
              gw[k] = uw[k] = make_uint4(0, 0, 0, 0);
              if (i < chunks) {
                gw[k] = load_stream16(gate + i);
                uw[k] = load_stream16(up + i);
              }
            }
          }
#pragma unroll
          for (int q = 0; q < kExactTogether; ++q) {
            if (q < count) {  // uniform over the warp
              float gq = g[q], vq = v[q];
#pragma unroll
              for (int k = 0; k < U; ++k) {
                const uint4 xw = __ldg(x[q] + min(base + 32 * k, chunks - 1));
                gq = fmaf(bf16_lo(gw[k].x), bf16_lo(xw.x), gq);
                gq = fmaf(bf16_hi(gw[k].x), bf16_hi(xw.x), gq);
                gq = fmaf(bf16_lo(gw[k].y), bf16_lo(xw.y), gq);
                gq = fmaf(bf16_hi(gw[k].y), bf16_hi(xw.y), gq);
                gq = fmaf(bf16_lo(gw[k].z), bf16_lo(xw.z), gq);
                gq = fmaf(bf16_hi(gw[k].z), bf16_hi(xw.z), gq);
                gq = fmaf(bf16_lo(gw[k].w), bf16_lo(xw.w), gq);
                gq = fmaf(bf16_hi(gw[k].w), bf16_hi(xw.w), gq);
                vq = fmaf(bf16_lo(uw[k].x), bf16_lo(xw.x), vq);
                vq = fmaf(bf16_hi(uw[k].x), bf16_hi(xw.x), vq);
                vq = fmaf(bf16_lo(uw[k].y), bf16_lo(xw.y), vq);
                vq = fmaf(bf16_hi(uw[k].y), bf16_hi(xw.y), vq);
                vq = fmaf(bf16_lo(uw[k].z), bf16_lo(xw.z), vq);
                vq = fmaf(bf16_hi(uw[k].z), bf16_hi(xw.z), vq);
                vq = fmaf(bf16_lo(uw[k].w), bf16_lo(xw.w), vq);
                vq = fmaf(bf16_hi(uw[k].w), bf16_hi(xw.w), vq);
              }
              g[q] = gq;
              v[q] = vq;
            }
          }
        }
#pragma unroll
        for (int q = 0; q < kExactTogether; ++q) {
          if (q < count) {
            float gq = g[q], vq = v[q];
#pragma unroll
            for (int w = 16; w; w >>= 1) {
              gq += __shfl_xor_sync(kFull, gq, w);
              vq += __shfl_xor_sync(kFull, vq, w);
            }
            if (lane == 0) {
              const uint32_t packed = entry[g0 + q];
              const int j = static_cast<int>(packed & 0xffu), position = static_cast<int>(packed >> 8);
              const size_t t = static_cast<size_t>(tok_t[j]);
              ws.activations[t * L.N + static_cast<size_t>(tok_slot[j]) * I + c] =
                  __float2bfloat16_rn(exact_feature(gq, vq, L.activation));
              ws.exact[t * 2 * L.F + position] = gq;
              ws.exact[t * 2 * L.F + L.F + position] = vq;
            }
          }
        }
      }
    }
    begin += tokens;
    __syncthreads();  // the table is rebuilt for the next chunk
  }
}

// ---------------------------------------------------------------------------
// down, expert-major
// ---------------------------------------------------------------------------
// grid (ceil(H / 256), E, parts), 128 threads, dynamic shared memory
// down_grouped_bytes(I).  A CTA owns 256 output columns of one expert and one of
// `parts` contiguous ranges of its channels.  For up to eight of the expert's
// tokens at a time it tabulates the activations of their kept channels in shared
// memory ([I][8] BF16, zero where a token did not keep the channel), then its
// four warps walk the channels of the range (warp w takes channels w, w + 4, ...):
// a channel some token kept is loaded once, 16 bytes per lane with up to eight
// rows in flight, and added to the FP32 sums of every token that kept it, which
// live in registers.  Which warp and which range a channel belongs to depends on
// the channel alone, so a token's sums are added in the same order whatever other
// tokens share its expert.  The four warps' sums are added in warp order through
// shared memory and stored as that token's partial sum of slot and part; the
// output kernel adds the parts in order.
__host__ __device__ inline size_t down_grouped_bytes(int I) {
  return (sizeof(uint4) + sizeof(int)) * static_cast<size_t>(I) +
         sizeof(float) * 4 * kDownChunkTokens * kDownGroupedColumns + 16 * sizeof(int) * 5;
}

// acc += s * (the eight BF16 values of w).
__device__ __forceinline__ void down_add_row(float (&acc)[8], const uint4& w, float s) {
  acc[0] = fmaf(bf16_lo(w.x), s, acc[0]);
  acc[1] = fmaf(bf16_hi(w.x), s, acc[1]);
  acc[2] = fmaf(bf16_lo(w.y), s, acc[2]);
  acc[3] = fmaf(bf16_hi(w.y), s, acc[3]);
  acc[4] = fmaf(bf16_lo(w.z), s, acc[4]);
  acc[5] = fmaf(bf16_hi(w.z), s, acc[5]);
  acc[6] = fmaf(bf16_lo(w.w), s, acc[6]);
  acc[7] = fmaf(bf16_hi(w.w), s, acc[7]);
}

__global__ void __launch_bounds__(kDownGroupedThreads, 4)
    k_down_grouped(Layer L, Workspace ws, int parts) {
  extern __shared__ uint4 down_smem[];
  const int I = L.I;
  uint4* table = down_smem;  // [I] eight BF16 activations per channel
  float* red = reinterpret_cast<float*>(table + I);  // [4][8][256]
  int* kept_by = reinterpret_cast<int*>(red + 4 * kDownChunkTokens * kDownGroupedColumns);  // [I]
  int* tok_t = kept_by + I;
  int* tok_slot = tok_t + 16;
  int* tok_start = tok_slot + 16;
  int* tok_count = tok_start + 16;
  int* tok_tile = tok_count + 16;

  const int e = blockIdx.y, part = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int first = ws.group_offsets[e], total = ws.group_offsets[e + 1] - first;
  if (total <= 0) return;
  const int column0 = blockIdx.x * kDownGroupedColumns + lane * 8;
  const bool live = column0 < L.H;
  // This CTA's channel range: equal shares, multiples of four channels.
  const int share = ((I + parts - 1) / parts + 3) / 4 * 4;
  const int c_begin = min(I, part * share), c_end = min(I, c_begin + share);
  const __nv_bfloat16* base = L.down + static_cast<size_t>(e) * I * L.H + (live ? column0 : 0);
  __nv_bfloat16* cells = reinterpret_cast<__nv_bfloat16*>(table);

  for (int begin = 0; begin < total; begin += kDownChunkTokens) {
    const int tokens = min(kDownChunkTokens, total - begin);
    __syncthreads();  // the previous chunk's table and sums are no longer read
    if (tid < tokens) {
      const GroupedToken g = grouped_token(L, ws, ws.group_pairs[first + begin + tid]);
      tok_t[tid] = g.t;
      tok_slot[tid] = g.slot;
      tok_start[tid] = g.start;
      tok_count[tid] = g.count;
      // Partial sums are laid out local slot after local slot, `parts` each.
      int local = 0;
      for (int s = 0; s < g.slot; ++s) local += ws.ids[static_cast<size_t>(g.t) * L.K + s] >= 0;
      tok_tile[tid] = local * parts + part;
    }
    for (int c = c_begin + tid; c < c_end; c += kDownGroupedThreads) {
      table[c] = make_uint4(0, 0, 0, 0);
      kept_by[c] = 0;
    }
    __syncthreads();
    // Activations of the kept channels inside the range (lists are ascending).
    for (int j = warp; j < tokens; j += 4) {
      const size_t t = static_cast<size_t>(tok_t[j]);
      const int32_t* list = ws.candidate_ids + t * L.F + tok_start[j];
      const __nv_bfloat16* act = ws.activations + t * L.N;
      const int slot_base = tok_slot[j] * I;
      for (int k = lane; k < tok_count[j]; k += 32) {
        const int cid = list[k], c = cid - slot_base;
        if (c >= c_begin && c < c_end) {
          cells[c * kDownChunkTokens + j] = act[cid];
          atomicOr(&kept_by[c], 1 << j);
        }
      }
    }
    __syncthreads();

    float acc[kDownChunkTokens][8];
#pragma unroll
    for (int j = 0; j < kDownChunkTokens; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[j][i] = 0.0f;
    // Channels c_begin + warp + 4 (32 round + lane): a ballot finds the kept ones.
    for (int round = 0; c_begin + warp + 128 * round < c_end; ++round) {
      const int mine = c_begin + warp + 4 * (32 * round + lane);
      const bool any = mine < c_end && kept_by[mine] != 0;
      unsigned pending = __ballot_sync(kFull, any);
      while (pending) {
        int channel[8];
        uint4 row[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          channel[q] = -1;
          if (pending) {
            const int bit = __ffs(pending) - 1;
            pending &= pending - 1;
            channel[q] = c_begin + warp + 4 * (32 * round + bit);
          }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
          row[q] = (channel[q] >= 0 && live)
                       ? load_stream16(base + static_cast<size_t>(channel[q]) * L.H)
                       : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (channel[q] < 0) continue;  // uniform over the warp
          const uint4 a = table[channel[q]];
          const uint4 w = row[q];
          // The tokens that kept the channel, one after the other (uniform over the warp).
          for (unsigned keepers = static_cast<unsigned>(kept_by[channel[q]]); keepers;
               keepers &= keepers - 1) {
            switch (__ffs(keepers) - 1) {
              case 0: down_add_row(acc[0], w, bf16_lo(a.x)); break;
              case 1: down_add_row(acc[1], w, bf16_hi(a.x)); break;
              case 2: down_add_row(acc[2], w, bf16_lo(a.y)); break;
              case 3: down_add_row(acc[3], w, bf16_hi(a.y)); break;
              case 4: down_add_row(acc[4], w, bf16_lo(a.z)); break;
              case 5: down_add_row(acc[5], w, bf16_hi(a.z)); break;
              case 6: down_add_row(acc[6], w, bf16_lo(a.w)); break;
              default: down_add_row(acc[7], w, bf16_hi(a.w)); break;
            }
          }
        }
      }
    }
    // The four warps' sums, added in warp order.
#pragma unroll
    for (int j = 0; j < kDownChunkTokens; ++j) {
      if (j < tokens) {
        float4* out = reinterpret_cast<float4*>(
            red + (static_cast<size_t>(warp) * kDownChunkTokens + j) * kDownGroupedColumns + lane * 8);
        out[0] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        out[1] = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
      }
    }
    __syncthreads();
    for (int index = tid; index < tokens * (kDownGroupedColumns / 4); index += kDownGroupedThreads) {
      const int j = index / (kDownGroupedColumns / 4), c4 = (index - j * (kDownGroupedColumns / 4)) * 4;
      const int column = blockIdx.x * kDownGroupedColumns + c4;
      if (column >= L.H) continue;
      const float* r0 = red + static_cast<size_t>(j) * kDownGroupedColumns + c4;
      const size_t stride = static_cast<size_t>(kDownChunkTokens) * kDownGroupedColumns;
      const float4 a = *reinterpret_cast<const float4*>(r0);
      const float4 b = *reinterpret_cast<const float4*>(r0 + stride);
      const float4 d = *reinterpret_cast<const float4*>(r0 + 2 * stride);
      const float4 g = *reinterpret_cast<const float4*>(r0 + 3 * stride);
      float* parts_out = ws.down_parts +
                         (static_cast<size_t>(tok_t[j]) * ws.down_tiles + tok_tile[j]) * L.H + column;
      *reinterpret_cast<float4*>(parts_out) =
          make_float4(((a.x + b.x) + d.x) + g.x, ((a.y + b.y) + d.y) + g.y,
                      ((a.z + b.z) + d.z) + g.z, ((a.w + b.w) + d.w) + g.w);
    }
  }
}

// ---------------------------------------------------------------------------
// encode, expert-major
// ---------------------------------------------------------------------------
// Element r of the router-weighted latent of token t from the per-(pair, tile)
// encoder sums: per live slot the tiles are added in order, rounded to BF16 and
// mixed by the router weight.
__device__ __forceinline__ float mix_latent(const Layer& L, const Workspace& ws, int t, int r) {
  float latent = 0.0f;
  for (int s = 0; s < L.K; ++s) {
    if (ws.ids[static_cast<size_t>(t) * L.K + s] < 0) continue;
    const float* p =
        ws.encoder_parts + (static_cast<size_t>(t) * L.K + s) * ws.encoder_tiles * L.R + r;
    float sum = 0.0f;
    for (int j = 0; j < ws.encoder_tiles; ++j) sum += __ldcg(p + static_cast<size_t>(j) * L.R);
    latent = fmaf(bf16_round(sum), ws.weights[static_cast<size_t>(t) * L.K + s], latent);
  }
  return latent;
}

// grid (encoder_tiles, E), 256 threads, dynamic shared memory
// encode_grouped_bytes(R).  A CTA owns 256 channels of one expert: it reads their
// encoder rows once for up to eight of the expert's tokens at a time.  Features
// of the skipped channels (zero for kept ones) go to shared memory; LPR = R / 8
// lanes cover one encoder row (16 bytes each) and 256 / LPR row groups walk the
// channels, every row applied to the eight tokens' sums in registers; the row
// groups are folded as in the per-pair kernel (shuffles, then shared memory in
// warp order), so both give the same bits.  The last CTA to arrive for a token
// mixes its latent.  Single-device readers only: every slot of every token is
// local, so a token expects K * encoder_tiles arrivals.
__host__ __device__ inline size_t encode_grouped_bytes(int R) {
  return sizeof(float) * (static_cast<size_t>(kDownChunkTokens) * kEncodeTileRows +
                          static_cast<size_t>(kDownChunkTokens) * (kEncodeThreads / 32) * R);
}

__global__ void __launch_bounds__(kEncodeThreads)
    k_encode_grouped(Layer L, Workspace ws) {
  extern __shared__ float encode_smem[];
  float (*feature)[kEncodeTileRows] = reinterpret_cast<float (*)[kEncodeTileRows]>(encode_smem);
  float* red = encode_smem + kDownChunkTokens * kEncodeTileRows;  // [token][fold][R]
  __shared__ int tok_t[kDownChunkTokens], tok_slot[kDownChunkTokens], tok_last[kDownChunkTokens];
  const int tile = blockIdx.x, e = blockIdx.y, tid = threadIdx.x;
  const int first = ws.group_offsets[e], total = ws.group_offsets[e + 1] - first;
  if (total <= 0) return;
  const int R = L.R, lpr = R / 8, groups = kEncodeThreads / lpr;
  const int c0 = tile * kEncodeTileRows, c1 = min(L.I, c0 + kEncodeTileRows);
  const int group = tid / lpr, col = (tid - group * lpr) * 8;
  const int lane = tid & 31, warp = tid >> 5;
  constexpr int kFolds = kEncodeThreads / 32;
  const __nv_bfloat16* enc = L.encoder + static_cast<size_t>(e) * L.I * R + col;

  for (int begin = 0; begin < total; begin += kDownChunkTokens) {
    const int tokens = min(kDownChunkTokens, total - begin);
    __syncthreads();
    if (tid < tokens) {
      const int pair = ws.group_pairs[first + begin + tid];
      tok_t[tid] = pair / L.K;
      tok_slot[tid] = pair - tok_t[tid] * L.K;
    }
    __syncthreads();
    for (int index = tid; index < tokens * (c1 - c0); index += kEncodeThreads) {
      const int j = index / (c1 - c0), c = c0 + index - j * (c1 - c0);
      const size_t t = static_cast<size_t>(tok_t[j]);
      const size_t at = t * 2 * L.N + static_cast<size_t>(tok_slot[j]) * L.I + c;
      feature[j][c - c0] =
          ws.selected[t * L.N + static_cast<size_t>(tok_slot[j]) * L.I + c]
              ? 0.0f : sketch_feature(ws.partial[at], ws.partial[at + L.N], L.activation);
    }
    __syncthreads();
    float acc[kDownChunkTokens][8];
#pragma unroll
    for (int j = 0; j < kDownChunkTokens; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[j][i] = 0.0f;
    constexpr int U = 4;
    for (int base = c0 + group; base < c1; base += groups * U) {
      uint4 w[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = base + u * groups;
        w[u] = c < c1 ? *reinterpret_cast<const uint4*>(enc + static_cast<size_t>(c) * R)
                      : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = min(base + u * groups, c1 - 1) - c0;
#pragma unroll
        for (int j = 0; j < kDownChunkTokens; ++j)
          if (j < tokens) down_add_row(acc[j], w[u], feature[j][c]);  // uniform over the CTA
      }
    }
    // Fold the row groups that share a warp (lanes lpr apart hold the same columns),
    // then the warps (or, for rows wider than a warp, the row groups) in order.
#pragma unroll
    for (int j = 0; j < kDownChunkTokens; ++j) {
      if (j < tokens) {
        for (int w = lpr; w < 32; w <<= 1) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[j][i] += __shfl_xor_sync(kFull, acc[j][i], w);
        }
        float* mine = red + (static_cast<size_t>(j) * kFolds + (lpr >= 32 ? group : warp)) * R + col;
        if (lpr >= 32 || lane < lpr) {
#pragma unroll
          for (int i = 0; i < 8; ++i) mine[i] = acc[j][i];
        }
      }
    }
    __syncthreads();
    const int folds = lpr >= 32 ? groups : kFolds;
    for (int index = tid; index < tokens * R; index += kEncodeThreads) {
      const int j = index / R, r = index - j * R;
      float sum = 0.0f;
      for (int f = 0; f < folds; ++f) sum += red[(static_cast<size_t>(j) * kFolds + f) * R + r];
      const size_t pair = static_cast<size_t>(tok_t[j]) * L.K + tok_slot[j];
      ws.encoder_parts[(pair * ws.encoder_tiles + tile) * R + r] = sum;
    }
    // The last CTA to arrive for a token mixes its latent.
    __threadfence();
    __syncthreads();
    if (tid < tokens) {
      uint32_t* counter = ws.counters + 2 * static_cast<size_t>(ws.capacity) * L.K + tok_t[tid];
      const unsigned expected = static_cast<unsigned>(L.K * ws.encoder_tiles);
      const unsigned old = atomicAdd(counter, 1u);
      tok_last[tid] = old == expected - 1;
      if (tok_last[tid]) *counter = 0;
    }
    __syncthreads();
    for (int index = tid; index < tokens * R; index += kEncodeThreads) {
      const int j = index / R, r = index - j * R;
      if (!tok_last[j]) continue;
      __threadfence();
      ws.latent[static_cast<size_t>(tok_t[j]) * R + r] = mix_latent(L, ws, tok_t[j], r);
    }
  }
}
