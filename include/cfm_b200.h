/*
 * C ABI of the B200 (sm_100a) sparse MoE decode reader.
 *
 * Every per-call entry point takes plain device pointers, sizes and a CUDA
 * stream, enqueues work on that stream and returns without synchronising, and
 * allocates no device memory: the caller owns weights, sketch, workspace and
 * outputs.  (The set-up calls of the peer-memory exchange, cfm_peer_*, are the
 * exception and say so.)  Return value 0 is success, a negative value is one of the
 * CFM_E_* argument errors (nothing was launched), a positive value is a
 * cudaError_t from a launch.  The host-side Python operator
 * (`ProgressiveReader`) is the only intended caller; it raises ValueError
 * before calling for every contract violation the reference rejects.
 *
 * The functions replace, stage by stage, the Triton launches of the
 * reference's `calibration_free_moe/reader/progressive.py`; each declaration
 * cites the reference code it stands for.
 *
 * Symbols: H hidden size, I channels per expert, E local experts, K experts
 * per token, N = K * I candidates per token, F channels kept per token,
 * R recovery rank, B = H / 128 rotation blocks, KEEP kept rotated coordinates
 * per block, T tokens in a call, C workspace capacity in tokens.
 */
#ifndef CFM_B200_H
#define CFM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CFM_ABI_VERSION 10

/* argument errors */
#define CFM_E_NULL -1       /* a required pointer is NULL                      */
#define CFM_E_SHAPE -2      /* a dimension violates the layer contract          */
#define CFM_E_CAPACITY -3   /* T outside [1, C] or workspace too small          */
#define CFM_E_UNSUPPORTED -4 /* option not built (e.g. an unknown score code)   */

#define CFM_ACT_SILU 0
#define CFM_ACT_GELU_TANH 1
#define CFM_SCORE_POINT 0
#define CFM_SCORE_RECOVERY_AWARE 1
#define CFM_ENGINE_MMA_SYNC 0 /* warp-level mma.sync.m16n8k32 (default: measured faster) */
#define CFM_ENGINE_TCGEN05 1  /* tcgen05.mma kind::i8, accumulators in tensor memory     */
#define CFM_ROWS_AUTO 0        /* the library's choice (per token, pairs in expert order) */
#define CFM_ROWS_PER_TOKEN 1   /* native rows always gathered per token                 */
#define CFM_ROWS_EXPERT_MAJOR 2 /* expert-major whenever the pairs are grouped (T >= 8) */
#define CFM_READ_WORK_SLOTS 20

/* One MoE layer: dimensions and resident tensors.  Mirrors the state
 * `ProgressiveReader.__init__` prepares (reference progressive.py:3133-3515). */
typedef struct cfm_layer {
  int32_t hidden;         /* H, multiple of 128                                */
  int32_t width;          /* I, multiple of 16                                 */
  int32_t experts;        /* E, experts resident on this device                */
  int32_t top_k;          /* K <= 32                                           */
  int32_t final_count;    /* F, 1 <= F <= N; F == N disables the screen        */
  int32_t keep;           /* KEEP in [1, 128]                                  */
  int32_t rank;           /* R, 0 = no recovery map; else multiple of 8, <= 256 */
  int32_t activation;     /* CFM_ACT_*                                         */
  int32_t score;          /* CFM_SCORE_*                                       */
  int32_t global_experts; /* length of expert_map, 0 when expert_map is NULL   */
  int32_t recovery_owner; /* 1 if this rank adds the decoder term              */
  int32_t tensor_engine;  /* CFM_ENGINE_*: tensor-core path of the grouped screen */
  int32_t row_engine;     /* CFM_ROWS_*: how exact, down and encode walk the native rows */
  int32_t reserved;
  const void* gate_up;       /* bf16 [E, 2I, H] contiguous                      */
  const void* down;          /* bf16 physical [E, I, H] (channel-major)         */
  const uint32_t* sketch;    /* coordinate-major layout [E, H, 2I/16], 2 bits per trit */
  const uint32_t* sketch_grouped; /* row-major layout [E, B, 2I, 8] or NULL     */
  const void* statistics;    /* fp16 physical [E, B, 2, 2I]: scale, variance    */
  const float* norms;        /* f32 [E, I], down-column norms                   */
  const float* geometry;     /* f32 [E, I, 2] or NULL (recovery-aware score)    */
  const void* encoder;       /* bf16 [E, I, R] or NULL                          */
  const void* decoder;       /* bf16 [H, R] or NULL                             */
  const int8_t* signs;       /* int8 [H], +-1                                   */
  const int32_t* expert_map; /* i32 [global_experts] global->local, -1 remote   */
  double* read_work;         /* f64 [20] read-cost counters, accumulated        */
  const float* selection_threshold; /* device f32 scalar: keep scores >= it, at most F
                                       per token; NULL = plain top-F                 */
} cfm_layer;

/* Expert parallelism over peer memory: every rank of the box owns one exchange
 * block of cfm_exchange_bytes() bytes in its own device memory, and all ranks have
 * mapped all blocks (cfm_peer_alloc / cfm_peer_export / cfm_peer_import, CUDA IPC).
 * `blocks[p]` is rank p's block as this process sees it.  One layer call is one
 * epoch of the exchange; all ranks must make the same sequence of calls. */
#define CFM_MAX_RANKS 16
#define CFM_PEER_HANDLE_BYTES 64
typedef struct cfm_exchange {
  int32_t world;          /* P, ranks of the box sharing the experts            */
  int32_t rank;           /* this rank                                          */
  int32_t tokens;         /* T, tokens every rank brings per call (fixed)       */
  int32_t reserved;
  void* blocks[CFM_MAX_RANKS];
} cfm_exchange;

/* One call.  Mirrors the arguments of `ProgressiveReader.__call__`
 * (reference progressive.py:3875-3926). */
typedef struct cfm_call {
  int32_t tokens;         /* T                                                 */
  int32_t ids_are_int64;  /* ids element type: 0 int32, 1 int64                */
  int32_t weights_are_bf16; /* router weight type: 0 float32, 1 bfloat16       */
  int32_t input_prepared; /* 1: cfm_prepare_input already ran for these rows   */
  int32_t scores_ready;   /* cfm_select: 0 computes the scores, 1 reads `scores`,
                             2 reads `scores`, takes cut and tie budgets from
                             `cuts` and keeps local slots only, 3 reads `scores`
                             and only writes cut and tie budgets to `cuts`      */
  int32_t row_offset;     /* cfm_select only: first workspace row to process   */
  const void* hidden;     /* bf16 [T, H]                                       */
  const void* ids;        /* [T, K] router expert ids (global ids under EP)    */
  const void* weights;    /* [T, K] router weights                             */
  const uint8_t* padding; /* bool [T] or NULL; 1 marks a padding row           */
  void* out;              /* bf16 [T, H]                                       */
  const int32_t* lists;   /* cfm_adopt only: i32 [T, F] kept candidate ids chosen
                             by the tokens' home ranks, ascending, -1 after the
                             last; NULL elsewhere                               */
  const struct cfm_exchange* exchange; /* expert parallelism over peer memory, or NULL:
                             cfm_adopt then reads the lists the home ranks stored
                             into this rank's exchange block and
                             cfm_partial_output stores its rows into the home
                             ranks' blocks (see cfm_exchange below)              */
} cfm_call;

/* Byte offsets of every scratch array inside one workspace allocation of
 * `bytes` bytes (256-byte aligned).  Mirrors the tensors of `ReaderWorkspace`
 * (reference progressive.py:2868-3121); names follow the reference where the
 * array has a counterpart. */
typedef struct cfm_workspace_layout {
  int64_t bytes;
  int64_t ids;            /* i32 [C, K]  experts sorted ascending, local ids    */
  int64_t weights;        /* f32 [C, K]  router weights in the same order       */
  int64_t norms;          /* f32 [C, B]  energy of the kept rotated coordinates */
  int64_t planes;         /* f32 [C, B, KEEP] kept rotated values               */
  int64_t coordinates;    /* i32 [C, B, KEEP] their coordinates, ascending      */
  int64_t quantized;      /* i32 [C, B, KEEP] fixed-point kept values           */
  int64_t exponents;      /* i32 [C, B, 2] fixed-point exponent, sum of values  */
  int64_t parts;          /* f32 [PARTS_TOKENS * K, B, 2I] per-block products   */
  int64_t counters;       /* u32 [2 * C * K + 2 * C] arrival counters (zero)    */
  int64_t partial;        /* f32 [C, 2, N] sketch projections (gate, up)        */
  int64_t scores;         /* f32 [C, N]                                         */
  int64_t selected;       /* u8  [C, N]                                         */
  int64_t completed;      /* u8  [C, N]                                         */
  int64_t candidate_ids;  /* i32 [C, F] kept candidates, ascending              */
  int64_t counts;         /* i32 [C, K]                                         */
  int64_t starts;         /* i32 [C, K]                                         */
  int64_t tile_starts;    /* i32 [C, K]                                         */
  int64_t activations;    /* bf16 [C, N] exact phi(g) u of kept candidates      */
  int64_t exact;          /* f32 [C, 2, F] exact gate and up projections        */
  int64_t down_parts;     /* f32 [C, down_tiles, H]                             */
  int64_t encoder_parts;  /* f32 [C, K, encoder_tiles, R]                       */
  int64_t latent;         /* f32 [C, R]                                         */
  int64_t status;         /* i32 [4] device-side error flags (zero = healthy)   */
  int64_t limbs;          /* i8  [C, B, 3, 128] base-256 digits of `quantized`  */
  int64_t group_offsets;  /* i32 [E + 1] first pair of every expert             */
  int64_t group_pairs;    /* i32 [C * K] (token, slot) pairs grouped by expert  */
  int64_t cuts;           /* i32 [C, 1 + K] score cut and per-slot tie budgets   */
  int64_t variances;      /* f32 [C, 2, N] residual variances of the projections */
  int64_t unscales;       /* f32 [C, B] 2^(exponent - 21), undoes the fixed point */
  int64_t zero_limbs;     /* i8  [B, 3, 128] zero digits for empty token slots    */
  int64_t tile_list;      /* i32 [C * (ceil(F / 64) + K), 8] down tiles in expert order */
  int64_t tile_count;     /* i32 [4] number of listed tiles                        */
  int32_t parts_tokens;   /* tokens the split screen can serve                  */
  int32_t down_tiles;     /* max(ceil(F / 64) + K - 1, 8 K) partial sums per token */
  int32_t encoder_tiles;  /* ceil(I / 256)                                      */
  int32_t reserved;
} cfm_workspace_layout;

/* ABI version of the loaded library (== CFM_ABI_VERSION of this header). */
int cfm_abi_version(void);

/* Text for a return code of this library. */
const char* cfm_error_string(int code);

/* Fill `layout` for a layer's dimensions and a capacity of C tokens.  Reads
 * only hidden/width/top_k/final_count/keep/rank of `layer`.
 * Replaces: ReaderWorkspace.__init__ sizing (progressive.py:2885-3121). */
int cfm_workspace_layout_for(const cfm_layer* layer, int32_t capacity,
                             cfm_workspace_layout* layout);

/* Construction: the ternary sketch of the native gate/up rows (`gate_up` bf16
 * [E, 2I, H], `signs` int8 [H]) written straight into the two kernel layouts
 * (`sketch`, `sketch_grouped`) and the FP16 statistics (physical [E, B, 2, 2I]).
 * Reads only hidden, width and experts of `layer`.  Same rotation and rule as the
 * reference builder; its three FP32 sums per block are added in another order,
 * so a coordinate within rounding of the threshold, or the last FP16 bit of a
 * scale, can differ from the reference builder's output.
 * Replaces: build_sketch (reader/sketch.py:84-150) for construction on the GPU. */
int cfm_build_sketch(const cfm_layer* layer, const void* gate_up, const int8_t* signs,
                     uint32_t* sketch, uint32_t* sketch_grouped, void* statistics, void* stream);

/* Input rotation: BF16 rows -> sign flip, 128-point Hadamard butterfly, keep
 * the KEEP largest |v| per block (ties to the lower coordinate), fixed-point
 * copy of the kept values.  Replaces: _prepare_input / _rotate_sketch_block
 * (progressive.py:304-346,389-453), launched by prepare_input (:3829-3873). */
int cfm_prepare_input(const cfm_layer* layer, void* workspace, int32_t capacity,
                      const cfm_call* call, void* stream);

/* Route: per token, sort the K expert ids ascending (stable), carry the
 * weights, map global to local ids; for batches the screen runs expert-major
 * (8 tokens and more, row-major sketch present) also group the (token, slot)
 * pairs by expert.  Independent of cfm_prepare_input: the two may run on
 * different streams.  Replaces: _prepare / _route (progressive.py:143-239,
 * 349-386), _group_sort (:2329-2382). */
int cfm_route(const cfm_layer* layer, void* workspace, int32_t capacity,
              const cfm_call* call, void* stream);

/* Screen: sketch projections of every candidate channel of every routed local
 * expert.  Writes `partial`; rows of remote or padded slots are zero.  Small
 * batches run one GEMV per (token, expert) over the coordinate-major sketch;
 * from 8 tokens the pairs, grouped by expert by cfm_route, run on the tensor
 * cores over the row-major sketch (when the layer has one).  Both give the same
 * bits.  Needs cfm_prepare_input and cfm_route of the same rows.
 * Replaces: _sketch_screen and its helpers (progressive.py:478-1066),
 * _group_screen (:2428-2606). */
int cfm_screen(const cfm_layer* layer, void* workspace, int32_t capacity,
               const cfm_call* call, void* stream);

/* Score: selection scores from the projections (zero for remote or padded
 * slots).  Only needed when scores are exchanged between ranks before the
 * selection; cfm_select computes them itself unless call->scores_ready.
 * Replaces: _screen_score (progressive.py:1274-1353). */
int cfm_score(const cfm_layer* layer, void* workspace, int32_t capacity,
              const cfm_call* call, void* stream);

/* Select: per token the F best scores, ties to the lower candidate index;
 * writes selected, candidate_ids, counts, starts, tile_starts and adds the
 * call's read-cost counters.  When the pairs are grouped by expert (cfm_route of
 * a batch of eight tokens and more) it also leaves the list of the call's down
 * tiles in expert order that cfm_down then reads (cfm_reader_forward builds that
 * list on its side stream beside the exact gather).  Replaces: _select
 * (progressive.py:1584-1775), _account_fixed (:242-276), _count_reads
 * (:2114-2317). */
int cfm_select(const cfm_layer* layer, void* workspace, int32_t capacity,
               const cfm_call* call, void* stream);

/* Exact gate/up: native BF16 rows of the kept candidates against the input,
 * FP32 accumulation, phi(g) u with the reference's BF16 rounding points.  With
 * the pairs grouped by expert, the (token, expert) pairs are walked in expert
 * order, so a row several tokens of one expert kept is fetched from HBM once
 * (row engine "per token"), or each expert's union of kept rows is read once and
 * applied to all its tokens (row engine "expert major").  Same bits either way.
 * Replaces: _acquire with END == H (progressive.py:1372-1581), _group_union
 * (:2609-2652), _group_complete (:2655-2718). */
int cfm_exact(const cfm_layer* layer, void* workspace, int32_t capacity,
              const cfm_call* call, void* stream);

/* Down: channel-major down rows of the kept candidates, weighted by their
 * activations, FP32 partial sums per tile of 64 kept rows (per token, tiles in
 * expert order when the pairs are grouped) or per (token, slot, channel range)
 * with the expert's union of kept rows read once (row engine "expert major").
 * Replaces: _down (progressive.py:1778-1856), _group_down (:2721-2801). */
int cfm_down(const cfm_layer* layer, void* workspace, int32_t capacity,
             const cfm_call* call, void* stream);

/* Recovery encode: sketch features of the skipped channels through the
 * encoder rows, then the router-weighted latent; per (token, expert) pair, or
 * with an expert's encoder rows read once for all its tokens (row engine "expert
 * major"; same bits).  Replaces: _encode and _latent (progressive.py:1859-2016),
 * _group_encode (:2804-2865). */
int cfm_encode(const cfm_layer* layer, void* workspace, int32_t capacity,
               const cfm_call* call, void* stream);

/* Output: mix the per-expert down sums by router weight, add the decoder
 * term, store BF16.  Replaces: _output (progressive.py:2019-2111). */
int cfm_output(const cfm_layer* layer, void* workspace, int32_t capacity,
               const cfm_call* call, void* stream);

/* Expert parallelism, owner side: like cfm_output but call->out is f32
 * [T, H + R]: per row the router-weighted sum of this rank's local slots (each
 * expert sum rounded to BF16 first, as in _output; no decoder term) followed by
 * this rank's share of the latent.  The caller adds the rows of all ranks.
 * Replaces: the per-rank part of _output (progressive.py:2019-2111). */
int cfm_partial_output(const cfm_layer* layer, void* workspace, int32_t capacity,
                       const cfm_call* call, void* stream);

/* Expert parallelism, home side: out = bf16(routed + bf16(U bf16(latent))) for
 * `tokens` rows.  With `latent` NULL, `combined` is f32 [T, H + R]: the sums
 * over the ranks of the rows cfm_partial_output wrote.  With `latent` f32
 * [T, R] (the home rank computed the whole latent itself), `combined` is f32
 * [T, H].  Needs only hidden, rank and decoder of `layer`.
 * Replaces: the tail of _output (:2096-2111). */
int cfm_finish(const cfm_layer* layer, int32_t tokens, const float* combined,
               const float* latent, void* out, void* stream);

/* Expert parallelism with the sketch replicated on every rank: the home rank of
 * a token screens and selects over all K experts and sends the kept candidate
 * ids; the ranks that own the experts adopt them.  From call->ids, call->weights
 * (as cfm_route) and call->lists this writes the workspace's routing order, the
 * list cut down to the local slots, and their counts, starts and down-tile
 * starts, after which cfm_exact, cfm_list_tiles, cfm_down and cfm_partial_output run.
 * No reference counterpart: the reference replicates the tokens and all-reduces
 * the scores instead (progressive.py:4245-4251). */
int cfm_adopt(const cfm_layer* layer, void* workspace, int32_t capacity, const cfm_call* call,
              void* stream);

/* Lists the down tiles of the call in expert order (batches of eight tokens and
 * more; nothing to do below that).  cfm_select does this itself; after cfm_adopt the
 * caller runs it anywhere between cfm_adopt and cfm_down, for instance on a second
 * stream beside cfm_exact, which does not read the list. */
int cfm_list_tiles(const cfm_layer* layer, void* workspace, int32_t capacity,
                   const cfm_call* call, void* stream);

/* Expert parallelism over peer memory (NVLink), replacing the collectives around
 * cfm_adopt and cfm_partial_output.  Per layer call and rank: cfm_select with
 * call->exchange (home side; plain selection, scores_ready 0) ends by storing the
 * kept lists of this rank's T tokens into every rank's block; cfm_adopt with
 * call->exchange waits for the lists of each row's home rank; cfm_partial_output with call->exchange stores each row's FP32
 * partial sums into the block of the row's home rank; cfm_finish_rows (home side)
 * waits for the rows of all ranks, adds them in rank order, adds the decoder term
 * of `latent` (f32 [T, R], or NULL) and stores BF16 `out` [T, H].  Every device-side
 * wait is bounded (about a second); a wait that ran out sets a bit in the status
 * word cfm_exchange_status reads (1: lists, 2: rows; the call synchronises) and
 * the results of that call are not to be trusted.  No reference counterpart: the
 * reference replicates the tokens and all-reduces (progressive.py:4245-4251,
 * 4444-4445).  cfm_peer_alloc allocates (and zeroes) a block with cudaMalloc;
 * cfm_peer_export writes its CFM_PEER_HANDLE_BYTES-byte IPC handle, which
 * cfm_peer_import opens in another process of the same box; these four are set-up
 * calls and synchronise. */
int64_t cfm_exchange_bytes(const cfm_layer* layer, int32_t world, int32_t tokens);
int cfm_peer_alloc(int64_t bytes, void** block);
int cfm_peer_export(void* block, void* handle);
int cfm_peer_import(const void* handle, void** block);
int cfm_peer_release(void* block, int32_t imported);
int cfm_exchange_status(const cfm_exchange* exchange, int32_t* status);
int cfm_finish_rows(const cfm_layer* layer, const cfm_exchange* exchange, const float* latent,
                    void* out, void* stream);

/* The whole layer on one stream: prepare (unless input_prepared), route,
 * screen, select, exact, down, encode, output.  Single-device readers only;
 * expert-parallel readers call the stages with their collectives between.
 * Replaces: ProgressiveReader.__call__ (progressive.py:3875-4472). */
int cfm_reader_forward(const cfm_layer* layer, void* workspace, int32_t capacity,
                       const cfm_call* call, void* stream);

/* ---- screen with library-owned scratch ----------------------------------- */
#define CFM_E_STATIC_CAPACITY -5 /* batch beyond the library-owned scratch       */
#define CFM_STATIC_PARTS_FLOATS (1 << 20) /* 4 MiB of per-block products          */
#define CFM_STATIC_MAX_PAIRS 1024         /* (token, expert) pairs per call       */

/* Inputs and output of cfm_screen_static: arrays in the formats cfm_route and
 * cfm_prepare_input write (a caller may point into its own workspace). */
typedef struct cfm_static_screen {
  int32_t tokens;             /* T >= 1                                         */
  int32_t reserved;
  const int32_t* ids;         /* i32 [T, K] local expert ids, ascending per token */
  const int32_t* quantized;   /* i32 [T, B, KEEP] fixed-point kept values        */
  const int32_t* coordinates; /* i32 [T, B, KEEP] their coordinates              */
  const int32_t* exponents;   /* i32 [T, B, 2] exponent and sum per block        */
  const uint8_t* padding;     /* bool [T] or NULL                                */
  float* partial;             /* out: f32 [T, 2, N] sketch projections           */
  const float* energies;      /* f32 [T, B] energy of the kept coordinates per block
                                 (the workspace's `norms`); needed with `variances` */
  float* variances;           /* out: f32 [T, 2, N] residual variances of the
                                 projections, or NULL to skip them               */
} cfm_static_screen;

/* The split screen (one GEMV per (token, expert) pair, rotation blocks spread
 * over CTAs) for callers that cannot provide scratch memory of their own and
 * must not cause an allocation: a decode step inside a serving engine that has
 * already handed all free device memory to its cache pool, or a host plugin
 * whose contract forbids touching the allocator.  The per-block products and
 * the arrival counters that join the CTAs live in two arrays inside the library
 * image (4 MiB + 4 KiB on every GPU that loads the library, held until exit);
 * this function, and everything it calls, allocates nothing.
 *
 * Limits: T * K <= CFM_STATIC_MAX_PAIRS and T * K * B * 2I <=
 * CFM_STATIC_PARTS_FLOATS, else CFM_E_STATIC_CAPACITY and nothing is launched.
 * The arrays are part of the library's device image: the CUDA runtime reserves
 * them when it loads that image on a device, which happens at the latest on the
 * first call of any entry point there.  A host whose memory pool takes all free
 * device memory must therefore load the library and make one call on the device
 * BEFORE the pool grabs its memory; from then on no call changes the amount of
 * free device memory.  The first call on a device also looks up the arrays'
 * device addresses; make it once, with the device current, before any stream
 * capture begins.  All calls on a device share the arrays, which keep the previous
 * call's contents: the counters are cleared on the stream at the start of every
 * call, and two calls whose kernels overlap on the GPU (different streams) race.
 * `partial` equals what cfm_screen writes, bit for bit.  cfm_screen on a layer with
 * the recovery-aware score also fills the workspace's `variances`, which
 * cfm_select and cfm_score then read: pass `energies` and `variances` to get them
 * from this call too (that kernel needs no scratch); with `variances` NULL only
 * `partial` is written and such a caller must provide the variances itself.
 * No counterpart in the reference, whose scratch is always caller-allocated
 * (ReaderWorkspace). */
int cfm_screen_static(const cfm_layer* layer, const cfm_static_screen* io, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CFM_B200_H */
