// The list of down tiles of a call, in expert order (sm_100a).
//
// The down kernel sums up to 64 kept rows of one (token, expert) pair per CTA.
// Which tiles exist is known once every token's selection is done.  One CTA then
// walks the pairs in expert order (k_group's list), counts their tiles with a
// block-wide scan and writes one 32-byte record per tile; the down kernel's CTAs
// read their record and go straight to the rows.  Tiles of one expert run next to
// each other in time, so a down row several tokens kept comes from HBM once and
// from L2 after that, and every CTA has one tile however unevenly a token's kept
// channels spread over its experts.  The whole-layer call runs the listing on its
// side stream beside the exact gate/up gather, so it costs the layer nothing.
// Included by cfm_reader.cu inside namespace cfm.
#pragma once

// One tile of the down kernel: up to 64 kept rows of one (token, slot) pair; 32 bytes.
struct DownTile {
  int32_t t, slot, expert, rows;
  int32_t list;   // first of the tile's entries in `candidate_ids`, as an index into the whole array
  int32_t tile;   // index of the tile's partial sum among the token's down tiles
  int32_t reserved[2];
};

// Called by all threads of ONE CTA once counts, starts and tile_starts of every
// pair are final.  `scratch` holds 33 ints of shared memory.
__device__ __forceinline__ void list_down_tiles(const Layer& L, const Workspace& ws,
                                                int* scratch) {
  const int tid = threadIdx.x, threads = blockDim.x, K = L.K, F = L.F;
  const int pairs = ws.group_offsets[L.E];
  DownTile* out = reinterpret_cast<DownTile*>(ws.tile_list);
  int base = 0;
  for (int first = 0; first < pairs; first += threads) {
    const int p = first + tid;
    int pair = 0, kept = 0, tiles = 0;
    if (p < pairs) {
      pair = ws.group_pairs[p];
      kept = ws.counts[pair];
      tiles = (kept + kDownTileRows - 1) / kDownTileRows;
    }
    int all = 0;
    const int at = base + block_exclusive_scan(tiles, scratch, &all);
    if (p < pairs) {
      const int token = pair / K, slot = pair - token * K;
      const int start = ws.starts[pair], tile0 = ws.tile_starts[pair], expert = ws.ids[pair];
      for (int j = 0; j < tiles; ++j) {
        DownTile d;
        d.t = token;
        d.slot = slot;
        d.expert = expert;
        d.rows = min(kDownTileRows, kept - j * kDownTileRows);
        d.list = token * F + start + j * kDownTileRows;
        d.tile = tile0 + j;
        d.reserved[0] = d.reserved[1] = 0;
        out[at + j] = d;
      }
    }
    base += all;
  }
  if (tid == 0) ws.tile_count[0] = base;
}

// grid (1), 1024 threads.
__global__ void __launch_bounds__(1024) k_list_tiles(Layer L, Workspace ws) {
  __shared__ int scratch[33];
  list_down_tiles(L, ws, scratch);
}
