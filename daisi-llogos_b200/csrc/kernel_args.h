// Argument blocks of the kernels' entry points that take more than a handful of values: plain structs that a caller
// fills and passes by address (Python through ctypes, the block runner in C++).  Every field is a device pointer, an
// int or a float; the layouts are part of the libraries' interface.
#pragma once

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
