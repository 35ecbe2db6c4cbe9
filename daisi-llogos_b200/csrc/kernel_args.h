// Argument blocks of the kernels' entry points that take more than a handful of values: plain structs that a caller
// fills and passes by address (Python through ctypes, the block runner in C++).  Every field is a device pointer, an
// int or a float; the layouts are part of the libraries' interface.
#pragma once

// What a norm leaves to the consumer of its output when it does not divide by the root mean square itself: the norm
// wrote x * weight and, per row, the sum of the row's squares, whole (parts = 1) or as `parts` partial sums (one per
// block of columns of whoever produced the row).  The consumer multiplies the rows of its product by
// 1 / sqrt(sum / width + eps): a product is linear in its rows, so the result is that of the normalised input, and
// nobody had to wait for a whole row before the product's operand could be written.
struct RowScale {
  const float* ss;            // [rows][parts], or null: rows are used as they are
  int parts;
  float inv_width;            // 1 / (elements of a row)
  float eps;
};

#ifdef __CUDACC__
__device__ __forceinline__ float row_scale_of(const RowScale& s, long long row) {
  if (!s.ss) return 1.0f;
  const float* p = s.ss + row * s.parts;
  float t = 0.f;
  for (int j0 = 0; j0 < s.parts; j0 += 8) {           // eight loads under way at a time; added in their order, so
    float v[8];                                       // the scale is the same whoever computes it
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = j0 + j < s.parts ? p[j0 + j] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += v[j];
  }
  return 1.0f / sqrtf(t * s.inv_width + s.eps);
}
#endif

struct QkPrepArgs {
  const void* qkv;            // [n_partials][n_tokens][(nh + 2 nkv) * hd], float32 or bfloat16
  int qkv_dtype;
  int n_partials;
  long long partial_stride;   // elements between partials
  const void* q_norm_w;       // [hd] or null
  const void* k_norm_w;       // [hd] or null
  int norm_w_dtype;
  float norm_eps;
  const void* bias;           // [(nh + 2 nkv) * hd] or null
  int bias_dtype;
  const float* cos_table;     // [positions][rotary_dim / 2] or null
  const float* sin_table;
  int rotary_dim;
  int pairing;                // 0: (i, i + rotary_dim/2), 1: (2i, 2i+1)
  int table_positions;
  const int* positions;       // [n_tokens]
  void* q_out;                // [n_tokens][nh][hd]
  void* k_new;                // [n_tokens][nkv][hd] or null
  void* v_new;
  void* k_pages;              // paged store or null
  void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* seq_of_token;    // [n_tokens] -> index into slots
  const int* slots;
  int n_tokens, nh, nkv, hd;
  RowScale row_scale;         // of the token rows of qkv (applied to the summed partials, before anything else)
};

// Attention for a step with several tokens per sequence (attention_simt.cu, attention_mma.cu, attention_tc.cu).
struct PrefillArgs {
  const void* q;            // [n_tokens][nh][hd]
  const void* k_new;        // [n_tokens][nkv][hd]
  const void* v_new;
  const void* k_pages;      // [pages][nkv][LLG_PAGE][hd]
  const void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* tiles;         // [n_tiles][2]: (sequence index in the batch, first query among its step tokens)
  const int* cu_tokens;     // [B + 1]
  const int* len_before;    // [B]
  const int* slots;         // [B]
  void* out;                // [n_tokens][nh * hd]
  int n_tiles, nh, nkv, hd;
  float scale;
  int window;               // 0 = all keys
  int n_tokens, n_pages;    // rows of k_new / v_new, pages of k_pages / v_pages
};

// Attention of one new token per sequence, split kernels (attention_simt.cu, attention_mma.cu).
struct DecodeArgs {
  const void* q;            // [B][nh][hd]
  const void* k_pages;
  const void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* slots;         // [B]
  const int* len_before;    // [B]; the new token's key is already in the cache at this position
  float* part_o;            // [B][nh][n_splits][hd]  un-normalised
  float* part_ml;           // [B][nh][n_splits][2]   running maximum, sum
  int n_seqs, nh, nkv, hd, n_splits;
  float scale;
  int window;
};

// Attention of one new token per sequence, TMA kernel (attention_decode_tma.cu).
struct DecodeTmaArgs {
  const void* q;              // [n_seqs][nh][hd]
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* slots;
  const int* len_before;
  float* part;                // [part_slots][G][hd + PART_PAD]
  int* counters;              // [n_seqs][nh], zero
  void* out;                  // [n_seqs][nh * hd]
  int n_seqs, nh, nkv, hd;
  float scale;
  int window;
};
