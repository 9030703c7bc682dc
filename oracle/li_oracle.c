/* CPU restatement of the lightning-indexer score and the canonical TopK-2048 in plain C.
 *
 * TEST INFRASTRUCTURE ONLY: used by tests/, the smoke check and the CPU arms of bench.py;
 * never linked into or called from the product library.
 *
 * Follows (paths inside the reference project zxdgongjue-spec/KVIP):
 *   - op_kernel/indexer/indexer_score.h:59-140, 384-426 - W = f32(bf16 w) * qscale; two fp32
 *     accumulators for even / odd heads updated in ascending head order with a fused
 *     multiply-add of relu(q.k) and W; score = (even + odd) * kscale; optional bf16 rounding
 *     with ties away from zero;
 *   - op_kernel/indexer/indexer_cube.h:344-371 - keys are gathered one 128-token page at a
 *     time through block_table;
 *   - op_kernel/indexer/topk_common.h:1136-1187 and indexer_vector.h:826-957 - TopK order.
 * Golden for the formula: tests/operators/lifetch/support/workloads.py:406-413, 1228-1237.
 * The dot product accumulates d = 0..127 in ascending order with fmaf, which is also what the
 * CUDA-core cross-check kernel does, so the two agree bit for bit.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static float e4m3_value[256];
static int table_ready = 0;

static void build_table(void) {
  for (int c = 0; c < 256; ++c) {
    int e = (c >> 3) & 15, m = c & 7;
    float v = e == 0 ? (float)m * 0x1p-9f : (1.0f + (float)m / 8.0f) * ldexpf(1.0f, e - 7);
    if ((c & 0x7f) == 0x7f) v = NAN;
    e4m3_value[c] = (c & 0x80) ? -v : v;
  }
  table_ready = 1;
}

static inline float bf16_bits_to_float(uint16_t bits) {
  uint32_t u = (uint32_t)bits << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline float bf16_away(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  u = (u + 0x8000u) & 0xffff0000u;
  memcpy(&v, &u, 4);
  return v;
}

/* scores[t, s] for every active query row t and s < ceil128(valid length).
 * query: [T, heads, 128]; keys: [rows, 128]; both u8 E4M3 codes (key_is_bf16 = 0) or bf16 bits.
 * weights: bf16 bits (weight_is_bf16 = 1) or fp32. query_scale / key_scale may be NULL. */
void kvip_oracle_li_scores(const void* query, const void* keys, const void* weights, const float* query_scale,
                           const float* key_scale, const int32_t* key_lengths, const int32_t* query_ends,
                           const int32_t* block_table, float* scores, int batch, int queries, int heads, int pages,
                           int score_stride, int key_is_bf16, int weight_is_bf16, int score_mode) {
  if (!table_ready) build_table();
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
  for (int b = 0; b < batch; ++b) {
    for (int page_i = 0; page_i < pages; ++page_i) {
      int longest = 0;
      for (int q = 0; q < queries; ++q)
        if (query_ends[b * queries + q] > longest) longest = query_ends[b * queries + q];
      int len = key_lengths[b] < longest ? key_lengths[b] : longest;
      if (len > pages * 128) len = pages * 128;
      if (page_i * 128 >= len) continue;
      const int64_t page = block_table[(int64_t)b * pages + page_i];
      float kf[128];
      for (int q = 0; q < queries; ++q) {
        const int t = b * queries + q;
        if (query_ends[t] <= 0) continue;
        float qf[64 * 128], w[64];
        for (int i = 0; i < heads * 128; ++i)
          qf[i] = key_is_bf16 ? bf16_bits_to_float(((const uint16_t*)query)[(int64_t)t * heads * 128 + i])
                              : e4m3_value[((const uint8_t*)query)[(int64_t)t * heads * 128 + i]];
        for (int h = 0; h < heads; ++h) {
          float v = weight_is_bf16 ? bf16_bits_to_float(((const uint16_t*)weights)[t * heads + h])
                                   : ((const float*)weights)[t * heads + h];
          if (query_scale) v *= query_scale[t * heads + h];
          w[h] = v;
        }
        for (int row = 0; row < 128; ++row) {
          const int64_t key_row = page * 128 + row;
          for (int d = 0; d < 128; ++d)
            kf[d] = key_is_bf16 ? bf16_bits_to_float(((const uint16_t*)keys)[key_row * 128 + d])
                                : e4m3_value[((const uint8_t*)keys)[key_row * 128 + d]];
          float even = 0.f, odd = 0.f;
          for (int h = 0; h < heads; ++h) {
            float dot = 0.f;
            for (int d = 0; d < 128; ++d) dot = fmaf(qf[h * 128 + d], kf[d], dot);
            const float relu = dot > 0.f ? dot : 0.f;
            if (h & 1) odd = fmaf(relu, w[h], odd);
            else even = fmaf(relu, w[h], even);
          }
          float score = (even + odd) * (key_scale ? key_scale[key_row] : 1.0f);
          if (score_mode == 1) score = bf16_away(score);
          scores[(int64_t)t * score_stride + page_i * 128 + row] = score;
        }
      }
    }
  }
}

static inline uint32_t sortable(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

static int cmp_u32_desc(const void* a, const void* b) {
  uint32_t x = *(const uint32_t*)a, y = *(const uint32_t*)b;
  return x < y ? 1 : (x > y ? -1 : 0);
}

/* Canonical TopK-2048 of one row: positions with key > v ascending, then key == v ascending. */
void kvip_oracle_topk_row(const float* row, int valid_len, int base_index, int32_t* out) {
  const int K = 2048;
  for (int i = 0; i < K; ++i) out[i] = -1;
  if (valid_len <= 0) return;
  if (valid_len <= K) {
    for (int i = 0; i < valid_len; ++i) out[i] = i + base_index;
    return;
  }
  uint32_t* keys = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)valid_len);
  for (int i = 0; i < valid_len; ++i) keys[i] = sortable(row[i]);
  uint32_t* sorted = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)valid_len);
  memcpy(sorted, keys, sizeof(uint32_t) * (size_t)valid_len);
  qsort(sorted, (size_t)valid_len, sizeof(uint32_t), cmp_u32_desc);
  const uint32_t kth = sorted[K - 1];
  int n = 0;
  for (int i = 0; i < valid_len; ++i)
    if (keys[i] > kth) out[n++] = i + base_index;
  for (int i = 0; i < valid_len && n < K; ++i)
    if (keys[i] == kth) out[n++] = i + base_index;
  free(sorted);
  free(keys);
}

void kvip_oracle_topk(const float* scores, const int32_t* key_lengths, const int32_t* query_ends, int32_t* out,
                      int rows, int queries, int score_stride, int base_index) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int t = 0; t < rows; ++t) {
    int len = key_lengths[t / queries] < query_ends[t] ? key_lengths[t / queries] : query_ends[t];
    if (len > score_stride) len = score_stride;
    kvip_oracle_topk_row(scores + (int64_t)t * score_stride, len, base_index, out + (int64_t)t * 2048);
  }
}
