// Choosing the next token on the device, one block per sequence, all arithmetic in float32.
//
// The pipeline is the reference sampler's (Inference/Sampler.cs:26-85): penalties over the
// recent tokens (:89-143), greedy shortcut, temperature, top-k (:249-276), min-p (:150-170),
// softmax over the candidates (:278-295), typical-p (:178-230), top-p (:297-332), and a draw by
// inverse CDF from one uniform number (:334-345).  The reference sorts candidates on the host;
// here every filter is a threshold found by bisection over the whole vocabulary, so no sort is
// needed and nothing is truncated.  Differences that follow from that: elements that tie with
// the threshold of min-p, typical-p or top-p are all kept (the reference's sort leaves their order
// open; top-k keeps exactly k, the smallest tokens among ties, as the reference does), and the draw
// walks the kept tokens in index order (the reference walks them by descending probability); the
// distribution drawn from is the same.
//
// The uniform number of (seed, sequence id, step) comes from a counter-based generator, so a
// sequence's tokens do not depend on what else is in its batch.
//
// Two ways through the pipeline.  The general one works on the whole vocabulary in global memory,
// one block per sequence (some seventy passes).  With top-k up to 64, the common case, the
// vocabulary is first cut into slices of 8192 logits, one block per (slice, sequence): a block
// keeps its logits in registers, finds its own k-th largest and passes on what reaches it, in index
// order.  No slice can hold k logits above the k-th largest of the whole row, so every token that
// top-k keeps is among these candidates; a second kernel runs the same filters and the same draw
// on the candidates alone (a few thousand at most, in shared memory).  A slice with more than 64
// candidates (ties) sends its row through the general way.
//
// Without top-k the same two kernels serve as long as the 64 largest logits of every slice can decide the
// outcome.  The first kernel then also leaves each slice's maximum and its sum of exp(v - maximum), from which
// the second has the softmax's normaliser over the whole row, and the scaled logits in the work row.  Pure
// temperature sampling draws over the whole row: the slice that holds the drawn point is found from the slices'
// masses, the point within it by one pass over that slice.  With top-p or min-p the filters run on the candidates
// with the whole row's normaliser, after a check that no token outside the candidates can belong to the kept set
// (every such token is no larger than its slice's 64th largest); if the check fails, the general way runs.
#include "common.cuh"

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Uniform in [0, 1) with 24 bits, a function of (seed, sequence id, step) only.
__device__ __forceinline__ float uniform_of(unsigned long long seed, int seq_id, int step) {
  unsigned long long h = splitmix64(seed);
  h = splitmix64(h ^ (0xD1B54A32D192ED03ull * (unsigned long long)(seq_id + 1)));
  h = splitmix64(h ^ (0x8CB92BA72F3D8DD7ull * (unsigned long long)(step + 1)));
  return (float)(h >> 40) * (1.0f / 16777216.0f);
}

// Monotone map float -> unsigned: a < b  <=>  key(a) < key(b)  (no NaNs expected).
__device__ __forceinline__ unsigned f2key(float f) {
  unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(unsigned k) {
  unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  int t = lane < (THREADS >> 5) ? scratch[lane] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// Lowest index among the maxima of x[0..n).
__device__ int block_argmax(const float* __restrict__ x, int n, float* fs, int* is) {
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += THREADS) {
    const float v = x[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) {
    fs[warp] = best;
    is[warp] = bi;
  }
  __syncthreads();
  best = lane < (THREADS >> 5) ? fs[lane] : -INFINITY;
  bi = lane < (THREADS >> 5) ? is[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (bi == 0x7fffffff) bi = 0;  // all NaN or n == 0
  return bi;
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, int vocab,
                                                         int* __restrict__ out) {
  __shared__ float fs[32];
  __shared__ int is[32];
  const int b = blockIdx.x;
  const int r = block_argmax(logits + (long long)b * vocab, vocab, fs, is);
  if (threadIdx.x == 0) out[b] = r;
}

struct SampleArgs {
  const float* logits;     // [B][V]
  float* work;             // [B][V] scratch: scaled logits, then probabilities
  int* out;                // [B]
  float* probs_out;        // [B][V] or null: the distribution drawn from (for tests)
  const int* seq_ids;      // [B] or null (then the row index)
  int* history;            // [rows][history_stride] recent tokens, or null; row of sequence b: history_rows[b], else b
  int* history_len;        // [rows] tokens seen so far (the row holds the last min(len, stride) of them, as a ring)
  int history_stride;
  int n_seqs, vocab;
  float temperature;
  int top_k;
  float top_p, min_p, typical_p;
  int min_keep;
  float repetition_penalty, frequency_penalty, presence_penalty;
  int penalize_newline;
  unsigned long long seed;
  int step;
  const int* banned;       // [n_banned] tokens whose logit becomes -inf (PreventEOS), or null
  int n_banned;
  float* cand_val;         // [B][n_slices][CAND_CAP] scaled logits of the candidates, or null
  int* cand_idx;           // [B][n_slices][CAND_CAP] their tokens
  int* cand_count;         // [B][n_slices] candidates found (more than CAND_CAP: the row takes the general way)
  int n_slices;
  const int* history_rows; // [B] or null
  int history_append;      // 1: the drawn token is written into the sequence's ring and its count goes up
  float* slice_stats;      // [B][n_slices][3] or null: a slice's maximum, its sum of exp(v - maximum), its least candidate
};

__device__ __forceinline__ int history_row(const SampleArgs& a, int b) { return a.history_rows ? a.history_rows[b] : b; }

// The kernel that has drawn `token` for sequence b keeps the ring of recent tokens up to date, so that the host
// need not send the history again (one thread calls this, after every read of the ring in this launch).
__device__ __forceinline__ void history_push(const SampleArgs& a, int b, int token) {
  if (!a.history || !a.history_append) return;
  const int row = history_row(a, b);
  const int len = a.history_len[row];
  a.history[(long long)row * a.history_stride + len % a.history_stride] = token;
  a.history_len[row] = len + 1;
}

constexpr int SLICE_PER = 8;                       // logits per thread of a slice's block
constexpr int SLICE_LEN = THREADS * SLICE_PER;     // logits per slice
constexpr int CAND_CAP = 64;                       // candidates a slice may pass on (and largest top-k of this way)
constexpr int MAX_SLICES = 64;
constexpr int HIST_MAX = 256;                      // recent tokens the slice kernel takes
constexpr int BANNED_MAX = 64;

// k-th largest value (k >= 1) of key(x[i]) over elements with keep(i); bisection over the 32 key bits.
template <typename KeyFn>
__device__ unsigned kth_largest_key(int n, int k, KeyFn key, int* is) {
  unsigned lo = 0u;  // largest t such that count(key >= t) >= k
  for (int bit = 31; bit >= 0; --bit) {
    const unsigned t = lo | (1u << bit);
    int c = 0;
    for (int i = threadIdx.x; i < n; i += THREADS) c += key(i) >= t ? 1 : 0;
    c = block_sum_int(c, is);
    if (c >= k) lo = t;
  }
  return lo;
}

// New value of token t's logit `v` that occurs `count` times among the recent tokens.
__device__ __forceinline__ float penalised(const SampleArgs& a, float v, int count) {
  if (a.repetition_penalty != 1.0f) {
    // applied once per occurrence in the window, as the reference's loop does
    for (int c = 0; c < count; ++c) v = v > 0.f ? v / a.repetition_penalty : v * a.repetition_penalty;
  }
  if (a.frequency_penalty != 0.f || a.presence_penalty != 0.f)
    v -= a.frequency_penalty * (float)count + a.presence_penalty;
  return v;
}

// Exclusive prefix sum of v over the block's threads; *total gets the sum.
__device__ int block_exclusive_scan_int(int v, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  int wsum = lane < (THREADS >> 5) ? scratch[lane] : 0;
  int wincl = wsum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, wincl, o);
    if (lane >= o) wincl += t;
  }
  *total = __shfl_sync(0xffffffffu, wincl, 31);
  const int before_warp = __shfl_sync(0xffffffffu, wincl - wsum, warp);
  return before_warp + incl - v;
}

// Filters and draw for sequence b over w[0..n): scaled logits in, probabilities left behind.  `map` (or null)
// gives the token of entry i; entries are in the order of their tokens.  mx = the largest scaled logit.
// `z_row` > 0: the entries are a part of a larger row whose sum of exp(v - mx) is z_row (that is the softmax's
// normaliser then), and sums of probabilities are whole only over entries of probability `whole_above` and more; when
// the entries cannot decide the outcome, *undecided is set and nothing is drawn.
__device__ void filter_and_draw(const SampleArgs& a, int b, float* w, int n, const int* map, float mx,
                                float* fs, int* is, int* chosen_slot, float* scan, float z_row = 0.f,
                                float whole_above = 0.f, int* undecided = nullptr) {
  const int tid = threadIdx.x;
  int& chosen = *chosen_slot;

  const int min_keep = a.min_keep > 1 ? a.min_keep : 1;

  // 4. top-k and min-p as one lower bound on the scaled logit
  float bound = -INFINITY;
  if (a.top_k > 0 && a.top_k < n) {
    bound = key2f(kth_largest_key(n, a.top_k, [&](int i) { return f2key(w[i]); }, is));
    // Exactly top_k stay: of the logits equal to the k-th largest, those with the smallest tokens, as the
    // reference's selection keeps the first it meets (Sampler.cs:249-276).  The ordered pass over the
    // vocabulary runs only when there are more ties than places.
    int gt = 0, eq = 0;
    for (int i = tid; i < n; i += THREADS) {
      gt += w[i] > bound ? 1 : 0;
      eq += w[i] == bound ? 1 : 0;
    }
    gt = block_sum_int(gt, is);
    eq = block_sum_int(eq, is);
    const int places = a.top_k - gt;
    if (eq > places) {
      int seen = 0;
      for (int i0 = 0; i0 < n; i0 += THREADS) {
        const int i = i0 + tid;
        const int mine = (i < n && w[i] == bound) ? 1 : 0;
        int total;
        const int before = block_exclusive_scan_int(mine, is, &total);
        if (mine && seen + before >= places) w[i] = -INFINITY;
        seen += total;
        __syncthreads();
      }
    }
  }
  if (a.min_p > 0.f && a.min_p < 1.0f) {
    float mb = mx + logf(a.min_p);
    if (min_keep > 1) {
      const float kb = key2f(kth_largest_key(n, min(min_keep, n), [&](int i) { return f2key(w[i]); }, is));
      mb = fminf(mb, kb);
    }
    bound = fmaxf(bound, mb);
  }

  // 5. softmax over the kept tokens
  float z = 0.f;
  for (int i = tid; i < n; i += THREADS) {
    const float v = w[i];
    const float e = v >= bound ? expf(v - mx) : 0.f;
    w[i] = e;
    z += e;
  }
  z = block_sum(z, fs);
  const float inv_z = 1.0f / (z_row > 0.f ? z_row : z);
  for (int i = tid; i < n; i += THREADS) w[i] *= inv_z;
  __syncthreads();

  // 6. typical-p: keep the tokens whose surprise is nearest the entropy until their mass reaches typical_p
  if (a.typical_p > 0.f && a.typical_p < 1.0f) {
    float ent = 0.f;
    for (int i = tid; i < n; i += THREADS) {
      const float p = w[i];
      if (p > 0.f) ent -= p * logf(p);
    }
    ent = block_sum(ent, fs);
    auto dev = [&](int i) -> float {
      const float p = w[i];
      return p > 0.f ? fabsf(-logf(p) - ent) : INFINITY;
    };
    // least deviation (as float bits; deviations are >= 0) whose inclusive mass reaches typical_p:
    // the largest t with mass(bits < t) < typical_p
    unsigned thr = 0u;
    for (int bit = 30; bit >= 0; --bit) {
      const unsigned t = thr | (1u << bit);
      float mass = 0.f;
      for (int i = tid; i < n; i += THREADS)
        if (__float_as_uint(dev(i)) < t) mass += w[i];
      mass = block_sum(mass, fs);
      if (mass < a.typical_p) thr = t;
    }
    if (min_keep > 1) {  // at least min_keep tokens: the min_keep-th smallest deviation
      const unsigned kk = kth_largest_key(n, min(min_keep, n), [&](int i) { return ~__float_as_uint(dev(i)); }, is);
      thr = max(thr, ~kk);
    }
    float s = 0.f;
    for (int i = tid; i < n; i += THREADS) {
      const float d = dev(i);
      const float p = (__float_as_uint(d) <= thr) ? w[i] : 0.f;
      s += p;
      w[i] = p;
    }
    s = block_sum(s, fs);
    if (s > 0.f) {
      const float r = 1.0f / s;
      for (int i = tid; i < n; i += THREADS) w[i] *= r;
    }
    __syncthreads();
  }

  // 7. top-p: the smallest set of most probable tokens whose mass exceeds top_p
  if (a.top_p > 0.f && a.top_p < 1.0f) {
    // largest t (a float's bits, probabilities are >= 0) with mass(p >= t) > top_p
    unsigned cur = 0u;
    // Entries of a larger row: below `whole_above` the sums miss tokens that are not among the entries.  If the mass
    // from there up does not exceed top_p, the kept set reaches further down than the entries can tell; if it does,
    // every threshold at or below it is known to pass without a sum.
    const unsigned whole_key = whole_above > 0.f ? __float_as_uint(whole_above) : 0u;
    if (whole_key) {
      float mass = 0.f;
      for (int i = tid; i < n; i += THREADS) {
        const float p = w[i];
        if (p > 0.f && __float_as_uint(p) >= whole_key) mass += p;
      }
      mass = block_sum(mass, fs);
      if (!(mass > a.top_p)) {
        if (tid == 0) *undecided = 1;
        __syncthreads();
        return;
      }
    }
    for (int bit = 30; bit >= 0; --bit) {
      const unsigned t = cur | (1u << bit);
      if (t <= whole_key) {
        cur = t;
        continue;
      }
      float mass = 0.f;
      for (int i = tid; i < n; i += THREADS) {
        const float p = w[i];
        if (p > 0.f && __float_as_uint(p) >= t) mass += p;
      }
      mass = block_sum(mass, fs);
      if (mass > a.top_p) cur = t;
    }
    unsigned thr = cur;
    if (min_keep > 1) {
      const unsigned kk = kth_largest_key(n, min(min_keep, n), [&](int i) { return __float_as_uint(w[i]); }, is);
      thr = min(thr, kk);
    }
    float s = 0.f;
    for (int i = tid; i < n; i += THREADS) {
      const float p = w[i];
      const float q = (p > 0.f && __float_as_uint(p) >= thr) ? p : 0.f;
      w[i] = q;
      s += q;
    }
    s = block_sum(s, fs);
    if (s > 0.f) {
      const float r = 1.0f / s;
      for (int i = tid; i < n; i += THREADS) w[i] *= r;
    }
    __syncthreads();
  }
  if (a.probs_out) {
    float* po = a.probs_out + (long long)b * a.vocab;
    if (map) {
      for (int i = tid; i < a.vocab; i += THREADS) po[i] = 0.f;
      __syncthreads();
      for (int i = tid; i < n; i += THREADS) po[map[i]] = w[i];
    } else {
      for (int i = tid; i < n; i += THREADS) po[i] = w[i];
    }
  }

  // 8. draw: first index whose cumulative probability exceeds u * total
  const int seq = a.seq_ids ? a.seq_ids[b] : b;
  const float u = uniform_of(a.seed, seq, a.step);
  const int per = (n + THREADS - 1) / THREADS;
  const int i0 = tid * per, i1 = min(n, i0 + per);
  float mine = 0.f;
  for (int i = i0; i < i1; ++i) mine += w[i];
  // inclusive scan of the per-thread sums
  scan[tid] = mine;
  __syncthreads();
  for (int o = 1; o < THREADS; o <<= 1) {
    const float add = tid >= o ? scan[tid - o] : 0.f;
    __syncthreads();
    scan[tid] += add;
    __syncthreads();
  }
  const float total = scan[THREADS - 1];
  const float target = u * total;
  if (tid == 0) chosen = 0x7fffffff;
  __syncthreads();
  const float before = scan[tid] - mine;
  if (target >= before && target < scan[tid]) {
    float c = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      c += w[i];
      if (w[i] > 0.f && target < c) {
        pick = i;
        break;
      }
    }
    if (pick < 0)  // rounding left the target past the last token of this chunk: take its last kept token
      for (int i = i1 - 1; i >= i0; --i)
        if (w[i] > 0.f) {
          pick = i;
          break;
        }
    if (pick >= 0) atomicMin(&chosen, pick);
  }
  __syncthreads();
  if (chosen == 0x7fffffff) {
    // target == total through rounding: take the most probable token
    const int r = block_argmax(w, n, fs, is);
    if (tid == 0) chosen = r;
    __syncthreads();
  }
  if (tid == 0) {
    const int token = map ? map[chosen] : chosen;
    a.out[b] = token;
    history_push(a, b, token);
  }
}

// The general way: the whole vocabulary of sequence b, in global memory.
__device__ void sample_full(const SampleArgs& a, int b, float* fs, int* is, int* chosen_slot, float* scan) {
  const int n = a.vocab, tid = threadIdx.x;
  const float* logits = a.logits + (long long)b * n;
  float* w = a.work + (long long)b * n;

  // 1. copy, penalties over the recent tokens, banned tokens
  for (int i = tid; i < n; i += THREADS) w[i] = logits[i];
  __syncthreads();
  const bool penal = a.history && (a.repetition_penalty != 1.0f || a.frequency_penalty != 0.f ||
                                   a.presence_penalty != 0.f);
  if (penal) {
    const int hl = min(a.history_len[history_row(a, b)], a.history_stride);
    const int* hist = a.history + (long long)history_row(a, b) * a.history_stride;
    // One thread per distinct recent token: the first occurrence owns the token.
    for (int j = tid; j < hl; j += THREADS) {
      const int t = hist[j];
      if (t < 0 || t >= n) continue;
      if (!a.penalize_newline && (t == 10 || t == 13)) continue;
      int count = 0;
      bool first = true;
      for (int q = 0; q < hl; ++q)
        if (hist[q] == t) {
          if (q < j) first = false;
          ++count;
        }
      if (!first) continue;
      w[t] = penalised(a, w[t], count);
    }
    __syncthreads();
  }
  for (int j = tid; j < a.n_banned; j += THREADS) {
    const int t = a.banned[j];
    if (t >= 0 && t < n) w[t] = -INFINITY;
  }
  __syncthreads();

  // 2. greedy
  if (a.temperature == 0.f) {
    const int r = block_argmax(w, n, fs, is);
    if (tid == 0) {
      a.out[b] = r;
      history_push(a, b, r);
    }
    if (a.probs_out)
      for (int i = tid; i < n; i += THREADS) a.probs_out[(long long)b * n + i] = i == r ? 1.f : 0.f;
    return;
  }

  // 3. temperature
  const float inv_t = 1.0f / a.temperature;
  float mx = -INFINITY;
  for (int i = tid; i < n; i += THREADS) {
    const float v = w[i] * inv_t;
    w[i] = v;
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, fs);
  filter_and_draw(a, b, w, n, nullptr, mx, fs, is, chosen_slot, scan);
}

__global__ void __launch_bounds__(THREADS) sample_kernel(SampleArgs a) {
  __shared__ float fs[32];
  __shared__ int is[32];
  __shared__ int chosen;
  __shared__ float scan[THREADS];
  sample_full(a, blockIdx.x, fs, is, &chosen, scan);
}

// First stage of the candidate way: block (slice, sequence) keeps SLICE_LEN scaled logits in registers and
// passes on those that reach its own top_k-th largest, in index order.
__global__ void __launch_bounds__(THREADS) sample_candidates_kernel(SampleArgs a) {
  __shared__ int is[32];
  __shared__ float fs[32];
  // without a top-k of its own the slice passes on its 64 largest, and what the second kernel needs of the rest
  const bool wide = !(a.top_k > 0 && a.top_k <= CAND_CAP);
  const int k_eff = wide ? CAND_CAP : a.top_k;
  __shared__ int pen_tok[HIST_MAX];
  __shared__ float pen_val[HIST_MAX];
  const int s = blockIdx.x, b = blockIdx.y, n = a.vocab, tid = threadIdx.x;
  const float* logits = a.logits + (long long)b * n;
  const int i0 = s * SLICE_LEN + tid * SLICE_PER;
  float v[SLICE_PER];
#pragma unroll
  for (int e = 0; e < SLICE_PER; ++e) v[e] = i0 + e < n ? logits[i0 + e] : -INFINITY;
  const bool penal = a.history && (a.repetition_penalty != 1.0f || a.frequency_penalty != 0.f ||
                                   a.presence_penalty != 0.f);
  if (penal) {
    const int hl = min(min(a.history_len[history_row(a, b)], a.history_stride), HIST_MAX);
    const int* hist = a.history + (long long)history_row(a, b) * a.history_stride;
    for (int j = tid; j < hl; j += THREADS) {      // the first occurrence of a token owns it
      const int t = hist[j];
      int owner = t;
      int count = 0;
      if (t < 0 || t >= n || (!a.penalize_newline && (t == 10 || t == 13))) owner = -1;
      for (int q = 0; q < hl; ++q)
        if (hist[q] == t) {
          if (q < j) owner = -1;
          ++count;
        }
      pen_tok[j] = owner;
      pen_val[j] = owner >= 0 ? penalised(a, logits[t], count) : 0.f;
    }
    __syncthreads();
    for (int j = 0; j < hl; ++j) {
      const int d = pen_tok[j] - i0;
      if (pen_tok[j] >= 0 && d >= 0 && d < SLICE_PER) {
#pragma unroll
        for (int e = 0; e < SLICE_PER; ++e)
          if (e == d) v[e] = pen_val[j];
      }
    }
  }
  for (int j = 0; j < a.n_banned; ++j) {
    const int d = a.banned[j] - i0;
    if (d >= 0 && d < SLICE_PER) {
#pragma unroll
      for (int e = 0; e < SLICE_PER; ++e)
        if (e == d) v[e] = -INFINITY;
    }
  }
  const float inv_t = 1.0f / a.temperature;
#pragma unroll
  for (int e = 0; e < SLICE_PER; ++e) v[e] *= inv_t;
  // the slice's top_k-th largest (bisection over the key bits, counts from registers)
  unsigned lo = 0u;
  for (int bit = 31; bit >= 0; --bit) {
    const unsigned t = lo | (1u << bit);
    int c = 0;
#pragma unroll
    for (int e = 0; e < SLICE_PER; ++e) c += f2key(v[e]) >= t ? 1 : 0;
    c = block_sum_int(c, is);
    if (c >= k_eff) lo = t;
  }
  const float thr = key2f(lo);
  if (wide) {
    float* w = a.work + (long long)b * n;
    float m = -INFINITY;
#pragma unroll
    for (int e = 0; e < SLICE_PER; ++e) {
      if (i0 + e < n) w[i0 + e] = v[e];
      m = fmaxf(m, v[e]);
    }
    m = block_max(m, fs);
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < SLICE_PER; ++e) sum += v[e] > -INFINITY ? expf(v[e] - m) : 0.f;
    sum = block_sum(sum, fs);
    if (tid == 0) {
      float* st = a.slice_stats + ((long long)b * a.n_slices + s) * 3;
      st[0] = m;
      st[1] = m > -INFINITY ? sum : 0.f;
      st[2] = thr;
    }
  }
  int cnt = 0;
#pragma unroll
  for (int e = 0; e < SLICE_PER; ++e) cnt += (v[e] >= thr && v[e] > -INFINITY) ? 1 : 0;
  int total;
  int pos = block_exclusive_scan_int(cnt, is, &total);
  const long long base = ((long long)b * a.n_slices + s) * CAND_CAP;
#pragma unroll
  for (int e = 0; e < SLICE_PER; ++e) {
    if (v[e] >= thr && v[e] > -INFINITY) {
      if (pos < CAND_CAP) {
        a.cand_val[base + pos] = v[e];
        a.cand_idx[base + pos] = i0 + e;
      }
      ++pos;
    }
  }
  if (tid == 0) a.cand_count[(long long)b * a.n_slices + s] = total;
}

// Second stage: the candidates of sequence b, gathered in index order, go through the filters and the draw.
__global__ void __launch_bounds__(THREADS) sample_from_candidates_kernel(SampleArgs a) {
  __shared__ float fs[32];
  __shared__ int is[32];
  __shared__ int chosen;
  __shared__ float scan[THREADS];
  __shared__ float cw[MAX_SLICES * CAND_CAP];
  __shared__ int cidx[MAX_SLICES * CAND_CAP];
  __shared__ int offs[MAX_SLICES + 1];
  __shared__ int overflow;
  const int b = blockIdx.x, tid = threadIdx.x, ns = a.n_slices;
  if (tid == 0) {
    int o = 0, ov = 0;
    for (int s = 0; s < ns; ++s) {
      const int c = a.cand_count[(long long)b * ns + s];
      if (c > CAND_CAP) ov = 1;
      offs[s] = o;
      o += min(c, CAND_CAP);
    }
    offs[ns] = o;
    overflow = ov;
  }
  __syncthreads();
  if (overflow) {                                  // uniform over the block
    sample_full(a, b, fs, is, &chosen, scan);
    return;
  }
  const int n_c = offs[ns];
  for (int g = tid; g < ns * CAND_CAP; g += THREADS) {
    const int s = g / CAND_CAP, j = g % CAND_CAP;
    if (j < offs[s + 1] - offs[s]) {
      cw[offs[s] + j] = a.cand_val[((long long)b * ns + s) * CAND_CAP + j];
      cidx[offs[s] + j] = a.cand_idx[((long long)b * ns + s) * CAND_CAP + j];
    }
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int i = tid; i < n_c; i += THREADS) mx = fmaxf(mx, cw[i]);
  mx = block_max(mx, fs);
  const bool wide = !(a.top_k > 0 && a.top_k <= CAND_CAP);
  if (!wide) {
    filter_and_draw(a, b, cw, n_c, cidx, mx, fs, is, &chosen, scan);
    return;
  }

  // ---- no top-k: the candidates are the 64 largest of every slice, the slices' sums give the whole row's ----
  __shared__ float smass[MAX_SLICES];       // a slice's sum of exp(v - mx)
  __shared__ float z_row_s, whole_s, target_s;
  __shared__ int slice_s, undecided;
  const float* st = a.slice_stats + (long long)b * ns * 3;
  if (tid < ns) smass[tid] = st[3 * tid] > -INFINITY ? st[3 * tid + 1] * expf(st[3 * tid] - mx) : 0.f;
  __syncthreads();
  const bool top_p_on = a.top_p > 0.f && a.top_p < 1.0f, min_p_on = a.min_p > 0.f && a.min_p < 1.0f;
  if (tid == 0) {
    float z = 0.f, least = -INFINITY;
    for (int s = 0; s < ns; ++s) {            // in slice order, by one thread: the same sum whatever else runs
      z += smass[s];
      least = fmaxf(least, st[3 * s + 2]);    // the largest of the slices' least candidates
    }
    z_row_s = z;
    whole_s = expf(least - mx) / z;           // every token outside the candidates is at most this probable
    // min-p keeps v >= mx + log(min_p): decidable when that bound lies above every slice's least candidate
    undecided = (min_p_on && !(mx + logf(a.min_p) > least)) ? 1 : 0;
  }
  __syncthreads();
  if (top_p_on || min_p_on) {
    if (!undecided)        // with min-p the kept tokens are all candidates, and the softmax is over them alone
      filter_and_draw(a, b, cw, n_c, cidx, mx, fs, is, &chosen, scan, min_p_on ? 0.f : z_row_s, min_p_on ? 0.f : whole_s, &undecided);
    __syncthreads();
    if (undecided) sample_full(a, b, fs, is, &chosen, scan);      // uniform over the block
    return;
  }

  // ---- temperature alone: a draw over the whole row ----
  const int n = a.vocab;
  const float* w = a.work + (long long)b * n;
  const int seq = a.seq_ids ? a.seq_ids[b] : b;
  const float u = uniform_of(a.seed, seq, a.step);
  if (tid == 0) {
    const float target = u * z_row_s;
    float before = 0.f;
    int pick = ns - 1;
    for (int s = 0; s < ns; ++s) {
      if (target < before + smass[s]) {
        pick = s;
        break;
      }
      if (s < ns - 1) before += smass[s];
    }
    slice_s = pick;
    target_s = target - before;               // where the drawn point lies within the slice's own mass
    chosen = 0x7fffffff;
  }
  __syncthreads();
  if (a.probs_out) {
    const float inv = 1.0f / z_row_s;
    for (int i = tid; i < n; i += THREADS) a.probs_out[(long long)b * n + i] = w[i] > -INFINITY ? expf(w[i] - mx) * inv : 0.f;
  }
  {
    const int i0 = slice_s * SLICE_LEN + tid * SLICE_PER;
    float p[SLICE_PER], mine = 0.f;
#pragma unroll
    for (int e = 0; e < SLICE_PER; ++e) {
      p[e] = (i0 + e < n && w[i0 + e] > -INFINITY) ? expf(w[i0 + e] - mx) : 0.f;
      mine += p[e];
    }
    scan[tid] = mine;
    __syncthreads();
    for (int o = 1; o < THREADS; o <<= 1) {
      const float add = tid >= o ? scan[tid - o] : 0.f;
      __syncthreads();
      scan[tid] += add;
      __syncthreads();
    }
    const float target = target_s, before = scan[tid] - mine;
    if (target >= before && target < scan[tid]) {
      float c = before;
      int pick = -1;
#pragma unroll
      for (int e = 0; e < SLICE_PER; ++e) {
        c += p[e];
        if (pick < 0 && p[e] > 0.f && target < c) pick = i0 + e;
      }
      if (pick < 0)          // rounding left the point past this thread's last token: its last token that can be drawn
        for (int e = SLICE_PER - 1; e >= 0; --e)
          if (pick < 0 && p[e] > 0.f) pick = i0 + e;
      if (pick >= 0) atomicMin(&chosen, pick);
    }
    __syncthreads();
    if (chosen == 0x7fffffff) {
      // rounding left the point past the slice's last token: the most probable token of the row
      const int r = block_argmax(cw, n_c, fs, is);
      if (tid == 0) chosen = cidx[r];
      __syncthreads();
    }
    if (tid == 0) {
      a.out[b] = chosen;
      history_push(a, b, chosen);
    }
  }
}

}  // namespace

// out[b] = lowest index among the maxima of logits[b][:]  (greedy; Inference/Sampler.cs:234-247)
LLG_API int llg_argmax(const float* logits, int n_seqs, int vocab, int* out, cudaStream_t stream) {
  LLG_REQUIRE(n_seqs >= 0 && vocab > 0, "argmax: bad sizes");
  if (n_seqs == 0) return 0;
  argmax_kernel<<<n_seqs, THREADS, 0, stream>>>(logits, vocab, out);
  return llg_check_launch("argmax");
}

// Slices that the candidate way cuts a vocabulary into, and the candidates a slice may pass on: the caller
// gives cand_val / cand_idx as [n_seqs][slices][cap] and cand_count as [n_seqs][slices] (or leaves them null).
LLG_API int llg_sample_slices(int vocab) { return (vocab + SLICE_LEN - 1) / SLICE_LEN; }
LLG_API int llg_sample_candidate_cap() { return CAND_CAP; }

LLG_API int llg_sample(const SampleArgs* args, cudaStream_t stream) {
  const SampleArgs& a = *args;
  LLG_REQUIRE(a.n_seqs >= 0 && a.vocab > 0, "sample: bad sizes");
  LLG_REQUIRE(a.temperature >= 0.f, "sample: temperature must not be negative");
  LLG_REQUIRE(a.work != nullptr, "sample: needs a work buffer of n_seqs * vocab floats");
  LLG_REQUIRE(!(a.history) || (a.history_len && a.history_stride > 0), "sample: history needs lengths and a stride");
  LLG_REQUIRE(a.repetition_penalty > 0.f, "sample: repetition penalty must be positive");
  if (a.n_seqs == 0) return 0;
  const int slices = (a.vocab + SLICE_LEN - 1) / SLICE_LEN;
  const bool scratch = a.cand_val && a.cand_idx && a.cand_count && a.n_slices == slices && slices <= MAX_SLICES &&
                       a.temperature > 0.f && (!a.history || a.history_stride <= HIST_MAX) && a.n_banned <= BANNED_MAX &&
                       a.n_seqs <= 65535;
  const bool narrow = a.top_k > 0 && a.top_k <= CAND_CAP && a.top_k < a.vocab && a.min_keep <= a.top_k;
  // no top-k at all, no typical-p (its entropy is over the whole row), at least one token kept is all min_keep asks
  const bool wide = (a.top_k <= 0 || a.top_k >= a.vocab) && !(a.typical_p > 0.f && a.typical_p < 1.0f) && a.min_keep <= 1 &&
                    a.slice_stats != nullptr && a.vocab >= CAND_CAP &&
                    // one block per (slice, row): worth it while they all run at once; a large batch fills the GPU with
                    // one block per row anyway (measured: 64 rows 136 us this way, 88 us the general way)
                    8LL * a.n_seqs * slices <= 18LL * llg_sm_count();        // two resident blocks per multiprocessor, and a few more
  const bool by_candidates = scratch && (narrow || wide);
  if (by_candidates) {
    sample_candidates_kernel<<<dim3(slices, a.n_seqs), THREADS, 0, stream>>>(a);
    if (llg_check_launch("sample (candidates)")) return 1;
    sample_from_candidates_kernel<<<a.n_seqs, THREADS, 0, stream>>>(a);
  } else {
    sample_kernel<<<a.n_seqs, THREADS, 0, stream>>>(a);
  }
  return llg_check_launch("sample");
}
