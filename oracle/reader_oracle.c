/*
 * CPU oracle of the sparse MoE decode reader.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithm of the reference's
 * calibration_free_moe/reader/{sketch,progressive}.py as its own tests define it
 * (tests/test_progressive_reader.py:102-267, `_reference_screen` and
 * `_reference_output`).  It is the checker for the CUDA library: only tests,
 * the smoke check and the CPU-baseline leg of the benchmark may call it, and
 * the product never does.  Its results are pinned against golden vectors
 * produced by the reference's own PyTorch functions (tests/golden/).
 *
 * It is written independently of the CUDA code: it decodes the reference's
 * five-trits-per-byte sketch layout directly (not the kernel's 2-bit layout),
 * finds the kept coordinates and the top-F by sorting (not by ranking or radix
 * search), and takes the encoder in the reference API layout [E, R, I].
 *
 * Arithmetic that decides channel selection follows one pinned order, which the
 * CUDA kernels reproduce bit for bit:
 *   1. rotation: sign flip, seven butterfly stages (half-widths 1..64,
 *      (l + r, l - r)), one multiply by float(1/sqrt(128))   [sketch.py:38-50]
 *   2. partial screen: keep the KEEP largest |v| per block, ties to the lower
 *      coordinate                                            [sketch.py:53-68]
 *   3. fixed point: with m the block's largest |v| and e = floor(log2 m)
 *      clamped to [-100, 100], q = rint(v * 2^(21-e)); block dots of trits with
 *      q are exact integers; dot = float(sum) * 2^(e-21)
 *   4. projection = sum over blocks in ascending order of fl(scale_b * dot_b),
 *      scale_b the FP16 block scale                          [progressive.py:600-669]
 *   5. point score = fl(fl(fl(fl(norm * phi(g)) * u)^2) * fl(w*w)) with g, u
 *      the BF16-rounded projections                          [tests/...:170-182]
 *   6. phi from the pinned exp below.
 * Step 3 replaces the reference's FP32 dot by an exact fixed-point one of the
 * same accuracy; that makes selections independent of summation order.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -pthread).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define BLOCK 128
#define QUANT_BITS 21

typedef struct oracle_layer {
  int32_t hidden, width, experts, top_k, final_count, keep, rank, activation;
  int32_t global_experts, recovery_owner;
  const uint16_t* gate_up;    /* bf16 [E, 2I, H] */
  const uint16_t* down;       /* bf16 physical [E, I, H] */
  const uint8_t* codes;       /* reference sketch codes [E, code_bytes] */
  int64_t code_bytes;         /* bytes per expert */
  const uint16_t* statistics; /* fp16 physical [E, B, 2, 2I] */
  const float* norms;         /* f32 [E, I] */
  const uint16_t* encoder;    /* bf16 [E, R, I] (reference API layout) or NULL */
  const uint16_t* decoder;    /* bf16 [H, R] or NULL */
  const int8_t* signs;        /* [H] */
  const int32_t* expert_map;  /* [global_experts] or NULL */
  int32_t score;              /* 0 point, 1 recovery-aware */
  int32_t reserved;
  const float* geometry;      /* f32 [E, I, 2] (alpha, beta) or NULL */
  const float* threshold;     /* threshold mode: keep scores >= *threshold, at most F; or NULL */
} oracle_layer;

typedef struct oracle_result {
  float* partial;         /* [T, 2, N] sketch projections, or NULL */
  float* scores;          /* [T, N] or NULL */
  uint8_t* selected;      /* [T, N] or NULL */
  int32_t* candidate_ids; /* [T, F] or NULL */
  int32_t* sorted_ids;    /* [T, K] local ids in slot order, or NULL */
  float* sorted_weights;  /* [T, K] or NULL */
  float* planes;          /* [T, B, KEEP] kept rotated values, or NULL */
  int32_t* coordinates;   /* [T, B, KEEP] or NULL */
  float* latent;          /* [T, R] or NULL */
  float* output;          /* [T, H] output (BF16-rounded unless fp32 mode) */
  float* routed;          /* [T, H] router-weighted sum of the local slots before the
                             decoder term and the final rounding, or NULL */
  const float* given_scores; /* [T, N] scores to select by instead of the computed ones
                                (expert parallelism: sums over ranks), or NULL */
  const uint8_t* given_selected; /* [T, N] kept-channel mask to use instead of selecting
                                    (expert parallelism: a rank's own slots), or NULL */
} oracle_result;

/* ---- number formats ---------------------------------------------------- */
static float bf16_to_float(uint16_t v) {
  uint32_t bits = (uint32_t)v << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static float bf16_round(float x) { /* round to nearest even, keep as float */
  uint32_t bits;
  memcpy(&bits, &x, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
  bits += 0x7fffu + ((bits >> 16) & 1u);
  bits &= 0xffff0000u;
  memcpy(&x, &bits, 4);
  return x;
}

static float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const int exponent = (h >> 10) & 0x1f;
  const uint32_t fraction = h & 0x3ffu;
  float value;
  if (exponent == 0) {
    value = ldexpf((float)fraction, -24);
  } else if (exponent == 31) {
    value = fraction ? NAN : INFINITY;
  } else {
    value = ldexpf((float)(fraction | 0x400u), exponent - 25);
  }
  uint32_t bits;
  memcpy(&bits, &value, 4);
  bits |= sign;
  memcpy(&value, &bits, 4);
  return value;
}

static float pow2f(int e) { /* 2^e for e in [-126, 127] */
  uint32_t bits = (uint32_t)(e + 127) << 23;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* ---- pinned activation ------------------------------------------------- */
static float pinned_exp(float x) {
  if (!(x == x)) return x;
  if (x >= 88.0f) return INFINITY;
  if (x <= -87.0f) return 0.0f;
  const float n = rintf(x * 1.44269502f);
  float r = fmaf(n, -0.693145752f, x);
  r = fmaf(n, -1.42860677e-06f, r);
  float p = 1.98412701e-04f;
  p = fmaf(p, r, 1.38888892e-03f);
  p = fmaf(p, r, 8.33333377e-03f);
  p = fmaf(p, r, 4.16666679e-02f);
  p = fmaf(p, r, 1.66666672e-01f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  return p * pow2f((int)n);
}

static float activate(float x, int activation) {
  if (activation == 1) { /* GELU, tanh form (reference activation.py:24-27) */
    const float x3 = (x * x) * x;
    const float inner = fmaf(0.044715f, x3, x);
    const float z = 0.797884583f * inner;
    const float ez = pinned_exp(2.0f * z);
    const float th = 1.0f - 2.0f / (ez + 1.0f);
    return (0.5f * x) * (1.0f + th);
  }
  return x / (1.0f + pinned_exp(-x)); /* SiLU */
}

/* Recovery-aware score (reference tests/test_progressive_reader.py:146-182,
 * progressive.py:1304-1353): five-node Gauss-Hermite expectation over the gate. */
static float risk_score(float g, float u, float vg, float vu, float norm, float alpha, float beta,
                        float w, int activation) {
  static const float nodes[5] = {-2.85697007f, -1.35562618f, 0.0f, 1.35562618f, 2.85697007f};
  static const float mass[5] = {0.0112574113f, 0.222075922f, 0.533333333f, 0.222075922f,
                                0.0112574113f};
  const float gb = bf16_round(g), ub = bf16_round(u);
  const float sg = sqrtf(vg), su = sqrtf(vu);
  const float spread = (ub * ub) + (su * su);
  float mu = 0.0f, second = 0.0f;
  for (int j = 0; j < 5; ++j) {
    const float a = activate(gb + nodes[j] * sg, activation);
    mu = mu + (mass[j] * a) * ub;
    second = second + (mass[j] * (a * a)) * spread;
  }
  const float p = bf16_round(activate(gb, activation) * ub);
  float spread_error = second - mu * mu;
  if (!(spread_error > 0.0f)) spread_error = 0.0f;
  float risk = (norm * norm) * spread_error;
  const float along = norm * mu - alpha * p;
  const float across = beta * p;
  risk = risk + ((along * along) + (across * across));
  return (risk * (w * w)) + 0.0f;
}

static double activate_f64(double x, int activation) {
  if (activation == 1) {
    return 0.5 * x * (1.0 + tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)));
  }
  return x / (1.0 + exp(-x));
}

/* ---- sketch decoding (reference sketch.py:209-232) --------------------- */
static int code_stride(int width) { return (2 * ((width + 4) / 5) + 15) / 16 * 16; }

/* Byte offset of code byte j of rotated coordinate h inside one expert. */
static int64_t code_offset(int hidden, int width, int h, int j) {
  const int stride = code_stride(width);
  const int body = stride / 32 * 32;
  const int blocks = hidden / BLOCK;
  if (j < body) return (int64_t)h * body + j;
  return (int64_t)blocks * BLOCK * body + ((int64_t)(h / 256) * BLOCK + h % BLOCK) * 32 +
         (int64_t)((h / BLOCK) % 2) * 16 + (j - body);
}

/* Trits of all 2I rows at rotated coordinate h of expert e. */
static void decode_coordinate(const oracle_layer* L, int e, int h, int8_t* trits) {
  const int I = L->width;
  const uint8_t* codes = L->codes + (int64_t)e * L->code_bytes;
  static const int place[5] = {1, 3, 9, 27, 81};
  for (int plane = 0; plane < 2; ++plane) {
    for (int c = 0; c < I; ++c) {
      const int byte = codes[code_offset(L->hidden, I, h, 2 * (c / 5) + plane)];
      trits[plane * I + c] = (int8_t)((byte / place[c % 5]) % 3 - 1);
    }
  }
}

/* ---- rotation and partial screen (reference sketch.py:38-68) ----------- */
static int compare_desc(const void* a, const void* b) {
  const float x = *(const float*)a, y = *(const float*)b;
  return (x < y) - (x > y);
}

/* Rotates one 128-block; writes kept values/coordinates (ascending), their
 * fixed-point copies, the exponent and the sum of the fixed-point values. */
static void rotate_block(const uint16_t* x, const int8_t* signs, int keep, float* planes,
                         int32_t* coordinates, int32_t* quantized, int* exponent, int* qsum,
                         float* energy) {
  float v[BLOCK], next[BLOCK], magnitude[BLOCK], sorted[BLOCK];
  for (int c = 0; c < BLOCK; ++c) v[c] = bf16_to_float(x[c]) * (float)signs[c];
  for (int half = 1; half < BLOCK; half *= 2) {
    for (int start = 0; start < BLOCK; start += 2 * half) {
      for (int j = 0; j < half; ++j) {
        const float left = v[start + j], right = v[start + half + j];
        next[start + j] = left + right;
        next[start + half + j] = left - right;
      }
    }
    memcpy(v, next, sizeof v);
  }
  for (int c = 0; c < BLOCK; ++c) {
    v[c] = v[c] * 0.0883883461f;
    magnitude[c] = fabsf(v[c]);
    sorted[c] = magnitude[c];
  }
  qsort(sorted, BLOCK, sizeof(float), compare_desc);
  const float cut = sorted[keep - 1];
  const float top = sorted[0];
  int above = 0;
  for (int c = 0; c < BLOCK; ++c) above += magnitude[c] > cut;
  int room = keep - above;
  uint32_t bits;
  memcpy(&bits, &top, 4);
  int e = (int)((bits >> 23) & 0xffu) - 127;
  if (e < -100) e = -100;
  if (e > 100) e = 100;
  const float scale = pow2f(QUANT_BITS - e);
  int count = 0, sum = 0;
  float kept_energy = 0.0f; /* squares of the kept values, in coordinate order */
  for (int c = 0; c < BLOCK; ++c) {
    int member = magnitude[c] > cut;
    if (!member && magnitude[c] == cut && room > 0) {
      member = 1;
      --room;
    }
    kept_energy = kept_energy + (member ? v[c] * v[c] : 0.0f);
    if (!member) continue;
    long q = top > 0.0f ? lrintf(v[c] * scale) : 0;
    if (q > (1 << 22)) q = 1 << 22;
    if (q < -(1 << 22)) q = -(1 << 22);
    planes[count] = v[c];
    coordinates[count] = c;
    quantized[count] = (int32_t)q;
    sum += (int)q;
    ++count;
  }
  *exponent = e;
  *qsum = sum;
  *energy = kept_energy;
}

/* ---- selection (reference tests/test_progressive_reader.py:240-246) ---- */
typedef struct {
  uint32_t key;
  int32_t index;
} ranked;

static int compare_ranked(const void* a, const void* b) {
  const ranked* x = (const ranked*)a;
  const ranked* y = (const ranked*)b;
  if (x->key != y->key) return x->key < y->key ? 1 : -1;
  return (x->index > y->index) - (x->index < y->index);
}

static int compare_int(const void* a, const void* b) {
  const int32_t x = *(const int32_t*)a, y = *(const int32_t*)b;
  return (x > y) - (x < y);
}

/* ---- one token ---------------------------------------------------------- */
static void token_forward(const oracle_layer* L, int t, const uint16_t* hidden,
                          const int64_t* ids, const float* weights, int fp32_mode,
                          const oracle_result* out) {
  const int H = L->hidden, I = L->width, K = L->top_k, F = L->final_count;
  const int KEEP = L->keep, R = L->rank, B = H / BLOCK, N = K * I, rows = 2 * I;
  const int screened = F < N;
  const uint16_t* x = hidden + (int64_t)t * H;

  /* route: stable ascending sort by global id (progressive.py:349-386) */
  int order[32], local[32];
  float route[32];
  for (int s = 0; s < K; ++s) {
    int rank = 0;
    for (int j = 0; j < K; ++j)
      rank += ids[(int64_t)t * K + j] < ids[(int64_t)t * K + s] ||
              (ids[(int64_t)t * K + j] == ids[(int64_t)t * K + s] && j < s);
    order[rank] = s;
  }
  for (int s = 0; s < K; ++s) {
    const int64_t id = ids[(int64_t)t * K + order[s]];
    int mapped = -1;
    if (L->expert_map) {
      if (id >= 0 && id < L->global_experts) mapped = L->expert_map[id];
    } else if (id >= 0 && id < L->experts) {
      mapped = (int)id;
    }
    local[s] = mapped;
    route[s] = weights[(int64_t)t * K + order[s]];
    if (out->sorted_ids) out->sorted_ids[(int64_t)t * K + s] = mapped;
    if (out->sorted_weights) out->sorted_weights[(int64_t)t * K + s] = route[s];
  }

  float* projection = (float*)calloc((size_t)2 * N, sizeof(float));
  float* score = (float*)calloc((size_t)N, sizeof(float));
  uint8_t* chosen = (uint8_t*)calloc((size_t)N, 1);

  if (screened) {
    /* rotation + partial screen + fixed point */
    float* planes = (float*)malloc(sizeof(float) * B * KEEP);
    int32_t* coordinates = (int32_t*)malloc(sizeof(int32_t) * B * KEEP);
    int32_t* quantized = (int32_t*)malloc(sizeof(int32_t) * B * KEEP);
    int* exponent = (int*)malloc(sizeof(int) * B);
    int* qsum = (int*)malloc(sizeof(int) * B);
    float* energy = (float*)malloc(sizeof(float) * B);
    for (int b = 0; b < B; ++b)
      rotate_block(x + b * BLOCK, L->signs + b * BLOCK, KEEP, planes + b * KEEP,
                   coordinates + b * KEEP, quantized + b * KEEP, exponent + b, qsum + b,
                   energy + b);
    if (out->planes) memcpy(out->planes + (int64_t)t * B * KEEP, planes, sizeof(float) * B * KEEP);
    if (out->coordinates)
      memcpy(out->coordinates + (int64_t)t * B * KEEP, coordinates, sizeof(int32_t) * B * KEEP);

    /* screen (progressive.py:478-786; tests/...:102-145) */
    int8_t* trits = (int8_t*)malloc((size_t)rows);
    int32_t* dot = (int32_t*)malloc(sizeof(int32_t) * rows);
    float* sum = (float*)malloc(sizeof(float) * rows);
    for (int s = 0; s < K; ++s) {
      const int e = local[s];
      if (e < 0) continue; /* remote slot: projections and scores stay zero */
      for (int r = 0; r < rows; ++r) sum[r] = 0.0f;
      for (int b = 0; b < B; ++b) {
        memset(dot, 0, sizeof(int32_t) * rows);
        for (int j = 0; j < KEEP; ++j) {
          decode_coordinate(L, e, b * BLOCK + coordinates[b * KEEP + j], trits);
          const int32_t q = quantized[b * KEEP + j];
          for (int r = 0; r < rows; ++r) dot[r] += trits[r] * q;
        }
        const float unscale = pow2f(exponent[b] - QUANT_BITS);
        const uint16_t* stat = L->statistics + ((int64_t)e * B + b) * 2 * rows;
        for (int r = 0; r < rows; ++r) {
          const float d = (float)dot[r] * unscale;
          const float product = half_to_float(stat[r]) * d;
          sum[r] = sum[r] + product;
        }
      }
      for (int c = 0; c < I; ++c) {
        const float g = sum[c], u = sum[I + c];
        projection[s * I + c] = g;
        projection[N + s * I + c] = u;
        const float gb = bf16_round(g), ub = bf16_round(u);
        const float norm = L->norms[(int64_t)e * I + c];
        if (L->score == 1) {
          /* residual variances: sum over blocks, in order, of variance_b * energy_b */
          float vg = 0.0f, vu = 0.0f;
          for (int b = 0; b < B; ++b) {
            const uint16_t* stat = L->statistics + (((int64_t)e * B + b) * 2 + 1) * rows;
            vg = vg + half_to_float(stat[c]) * energy[b];
            vu = vu + half_to_float(stat[I + c]) * energy[b];
          }
          const float alpha = L->geometry ? L->geometry[((int64_t)e * I + c) * 2] : 0.0f;
          const float beta = L->geometry ? L->geometry[((int64_t)e * I + c) * 2 + 1] : 0.0f;
          score[s * I + c] = risk_score(g, u, vg, vu, norm, alpha, beta, route[s], L->activation);
        } else {
          const float v = (norm * activate(gb, L->activation)) * ub;
          score[s * I + c] = ((v * v) * (route[s] * route[s])) + 0.0f;
        }
      }
    }
    free(trits);
    free(dot);
    free(sum);
    free(planes);
    free(coordinates);
    free(quantized);
    free(exponent);
    free(qsum);
    free(energy);
  }
  if (out->partial) memcpy(out->partial + (int64_t)t * 2 * N, projection, sizeof(float) * 2 * N);
  if (out->scores) memcpy(out->scores + (int64_t)t * N, score, sizeof(float) * N);

  if (out->given_scores) memcpy(score, out->given_scores + (int64_t)t * N, sizeof(float) * N);

  /* select: F best, ties to the lower candidate index */
  int32_t* kept = (int32_t*)malloc(sizeof(int32_t) * F);
  if (out->given_selected) {
    int count = 0;
    for (int i = 0; i < F; ++i) kept[i] = -1;
    for (int i = 0; i < N && count < F; ++i)
      if (out->given_selected[(int64_t)t * N + i]) kept[count++] = i;
  } else if (screened) {
    ranked* order_by_score = (ranked*)malloc(sizeof(ranked) * N);
    for (int i = 0; i < N; ++i) {
      memcpy(&order_by_score[i].key, &score[i], 4);
      order_by_score[i].index = i;
    }
    qsort(order_by_score, N, sizeof(ranked), compare_ranked);
    int keep_count = F;
    if (L->threshold) { /* every score at or above the threshold, at most F, best first
                           (tests/test_progressive_reader.py:229-239) */
      int passing = 0;
      for (int i = 0; i < N; ++i) passing += score[i] >= *L->threshold;
      if (passing < keep_count) keep_count = passing;
    }
    for (int i = 0; i < F; ++i) kept[i] = i < keep_count ? order_by_score[i].index : 0x7fffffff;
    qsort(kept, F, sizeof(int32_t), compare_int);
    for (int i = keep_count; i < F; ++i) kept[i] = -1;
    free(order_by_score);
  } else {
    for (int i = 0; i < F; ++i) kept[i] = i;
  }
  for (int i = 0; i < F; ++i)
    if (kept[i] >= 0) chosen[kept[i]] = 1;
  if (out->candidate_ids) memcpy(out->candidate_ids + (int64_t)t * F, kept, sizeof(int32_t) * F);
  if (out->selected) memcpy(out->selected + (int64_t)t * N, chosen, (size_t)N);

  /* exact gate/up, down, recovery, output (tests/...:212-266) */
  double* routed = (double*)calloc((size_t)H, sizeof(double));
  double* latent = (double*)calloc((size_t)(R ? R : 1), sizeof(double));
  double* expert_sum = (double*)malloc(sizeof(double) * H);
  double* expert_latent = (double*)malloc(sizeof(double) * (R ? R : 1));
  for (int s = 0; s < K; ++s) {
    const int e = local[s];
    if (e < 0) continue;
    for (int h = 0; h < H; ++h) expert_sum[h] = 0.0;
    for (int r = 0; r < R; ++r) expert_latent[r] = 0.0;
    for (int c = 0; c < I; ++c) {
      const int cand = s * I + c;
      if (chosen[cand]) {
        const uint16_t* gate = L->gate_up + ((int64_t)e * rows + c) * H;
        const uint16_t* up = gate + (int64_t)I * H;
        double g = 0.0, u = 0.0;
        for (int h = 0; h < H; ++h) {
          const double xv = bf16_to_float(x[h]);
          g += (double)bf16_to_float(gate[h]) * xv;
          u += (double)bf16_to_float(up[h]) * xv;
        }
        double a;
        if (fp32_mode) {
          a = activate_f64(g, L->activation) * u;
        } else {
          const float gb = bf16_round((float)g), ub = bf16_round((float)u);
          a = bf16_round(bf16_round(activate(gb, L->activation)) * ub);
        }
        const uint16_t* row = L->down + ((int64_t)e * I + c) * H;
        for (int h = 0; h < H; ++h) expert_sum[h] += (double)bf16_to_float(row[h]) * a;
      } else if (R > 0 && L->encoder) {
        double p;
        if (fp32_mode) {
          p = activate_f64(projection[cand], L->activation) * projection[N + cand];
        } else {
          const float gb = bf16_round(projection[cand]), ub = bf16_round(projection[N + cand]);
          p = bf16_round(activate(gb, L->activation) * ub);
        }
        const uint16_t* enc = L->encoder + (int64_t)e * R * I + c;
        for (int r = 0; r < R; ++r) expert_latent[r] += (double)bf16_to_float(enc[(int64_t)r * I]) * p;
      }
    }
    for (int h = 0; h < H; ++h)
      routed[h] += (fp32_mode ? expert_sum[h] : (double)bf16_round((float)expert_sum[h])) * route[s];
    for (int r = 0; r < R; ++r)
      latent[r] += (fp32_mode ? expert_latent[r] : (double)bf16_round((float)expert_latent[r])) * route[s];
  }
  if (out->latent)
    for (int r = 0; r < R; ++r) out->latent[(int64_t)t * R + r] = (float)latent[r];
  if (out->routed)
    for (int h = 0; h < H; ++h) out->routed[(int64_t)t * H + h] = (float)routed[h];
  for (int h = 0; h < H; ++h) {
    double recovery = 0.0;
    if (R > 0 && L->decoder && L->recovery_owner) {
      const uint16_t* row = L->decoder + (int64_t)h * R;
      for (int r = 0; r < R; ++r)
        recovery += (double)bf16_to_float(row[r]) *
                    (fp32_mode ? latent[r] : (double)bf16_round((float)latent[r]));
      if (!fp32_mode) recovery = bf16_round((float)recovery);
    }
    const double value = routed[h] + recovery;
    out->output[(int64_t)t * H + h] = fp32_mode ? (float)value : bf16_round((float)value);
  }
  free(routed);
  free(latent);
  free(expert_sum);
  free(expert_latent);
  free(kept);
  free(projection);
  free(score);
  free(chosen);
}

/* ---- driver: tokens spread over POSIX threads ---------------------------- */
typedef struct {
  const oracle_layer* L;
  int tokens;
  const uint16_t* hidden;
  const int64_t* ids;
  const float* weights;
  const uint8_t* padding;
  int fp32_mode;
  const oracle_result* out;
  int next; /* next token to take, guarded by lock */
  pthread_mutex_t lock;
} job;

static void* worker(void* arg) {
  job* j = (job*)arg;
  const int H = j->L->hidden, N = j->L->top_k * j->L->width;
  for (;;) {
    pthread_mutex_lock(&j->lock);
    const int t = j->next++;
    pthread_mutex_unlock(&j->lock);
    if (t >= j->tokens) return NULL;
    const oracle_result* out = j->out;
    if (j->padding && j->padding[t]) {
      memset(out->output + (int64_t)t * H, 0, sizeof(float) * H);
      if (out->routed) memset(out->routed + (int64_t)t * H, 0, sizeof(float) * H);
      if (out->latent && j->L->rank)
        memset(out->latent + (int64_t)t * j->L->rank, 0, sizeof(float) * j->L->rank);
      if (out->scores) memset(out->scores + (int64_t)t * N, 0, sizeof(float) * N);
      if (out->partial) memset(out->partial + (int64_t)t * 2 * N, 0, sizeof(float) * 2 * N);
      if (out->selected) memset(out->selected + (int64_t)t * N, 0, (size_t)N);
      continue;
    }
    token_forward(j->L, t, j->hidden, j->ids, j->weights, j->fp32_mode, out);
  }
}

/* Runs T tokens on `threads` POSIX threads (at least 1); padded rows produce
 * zeros.  fp32_mode evaluates the sparse operator on the same selection without
 * the BF16 rounding points.  Returns 0, or -1 for invalid dimensions. */
int oracle_forward(const oracle_layer* L, int tokens, const uint16_t* hidden, const int64_t* ids,
                   const float* weights, const uint8_t* padding, int fp32_mode, int threads,
                   const oracle_result* out) {
  if (!L || !out || !out->output || L->hidden % BLOCK || L->top_k > 32 || L->keep < 1 ||
      L->keep > BLOCK)
    return -1;
  job j = {L, tokens, hidden, ids, weights, padding, fp32_mode, out, 0, PTHREAD_MUTEX_INITIALIZER};
  if (threads > tokens) threads = tokens;
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  pthread_t pool[256];
  int started = 0;
  for (int i = 1; i < threads; ++i)
    if (pthread_create(&pool[started], NULL, worker, &j) == 0) ++started;
  worker(&j);
  for (int i = 0; i < started; ++i) pthread_join(pool[i], NULL);
  pthread_mutex_destroy(&j.lock);
  return 0;
}

int oracle_abi_version(void) { return 1; }
