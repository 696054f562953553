// Softmax attention over a sliding window with optional kept first tokens, a sink in the denominator, a learned bias
// by distance, capped scores and a gate a head.
//
// The cache holds one vector per token, [k: kv_heads x dim | v: kv_heads x vdim], in pages: cache[page][offset][width].
// A row at position p sees the keys j <= p with p - j < window (window 0: all) or j < keep_first.
//
//   score  = (q . k) scale;  cap > 0: cap tanh(score / cap);  bias: + bias[head][min(p - j, distances - 1)]
//   weight = exp(score) / (sum over the seen keys of exp(score) + exp(sink[head]))        (sink null: no such term)
//   out    = sum weight v, times sigmoid(gate[row][head]) where there is a gate
//
//   window_qk_prepare        per row: RMS norm over the WHOLE q (and k) projection with a weight a column, rotation of the
//                            first columns of every head in neighbouring pairs or in halves, by a table of (cos, sin) or
//                            by angles position * f_i computed in 32-bit from frequencies; without write_kv the rows
//                            hold q alone and nothing goes to the cache (a mixer that reads another's keys and values);
//                            q goes to a buffer of its own, k and v (v: its own columns, or the key columns as they
//                            came, before norm and rotation) to the row's slot of the cache
//   window_attention_generic a warp a (row, head): keys in chunks of 32 at multiples of 32 (a lane a key for the
//                            scores, a lane a value column for the sums), 32-bit throughout; the result does not
//                            depend on the step's make-up by a single bit.  With splits the keys of a (row, head) of a
//                            request of at most 16 rows are cut into parts side by side, folded in order by
//                            window_attention_merge
//   window_attention_tile    bf16, tensor cores (mma.sync m16n8k16), requests of more than 16 rows: a block is 128 rows
//                            of a (request, head), a warp 16 of them; tiles of 64 keys by cp.async into two buffers, the
//                            tiles of the kept first tokens before those of the window; scores, softmax and sums
//                            32-bit; the weights enter the product with the values as a bf16 pair (rounding and remainder)
#include "common.cuh"
#include "mma.cuh"

namespace pih {

constexpr int kWinMaxPerLane = 16;          // value columns a lane at most: vdim <= 512 (instances: 2, 4, 8, 16)

// What a row may see, and how a score is finished: shared by all kernels of the file.
struct WindowRule {
  int window;            // 0: every earlier key
  int keep_first;        // keys below this place stay seen
  float scale;
  float cap;             // 0: scores are not capped
  const float* bias;     // [heads][distances] or null
  int distances;
};

template <bool kExact>
__device__ __forceinline__ float capped(float s, float cap) {
  if (kExact) return cap * tanhf(s / cap);
  // 1 - 2 / (e^{2x} + 1): the special-function unit's exponential; its error is far below a bf16 rounding of q or k
  return cap * (1.0f - __fdividef(2.0f, __expf(2.0f * s / cap) + 1.0f));
}

template <bool kExact>
__device__ __forceinline__ float finish_score(float dot, const WindowRule& rule, const float* bias_of_head, int distance) {
  float s = dot * rule.scale;
  if (rule.cap > 0.0f) s = capped<kExact>(s, rule.cap);
  if (bias_of_head != nullptr) s += bias_of_head[min(max(distance, 0), rule.distances - 1)];
  return s;
}

// WORDS (1, 2 or 4) 32-bit words from an address that is a multiple of their size, as one load; and element i of type T
// out of such words.
template <int WORDS>
__device__ __forceinline__ void load_words(uint32_t (&w)[WORDS], const void* src) {
  static_assert(WORDS == 1 || WORDS == 2 || WORDS == 4, "one load");
  if constexpr (WORDS == 4) {
    const uint4 r = *reinterpret_cast<const uint4*>(src);
    w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
  } else if constexpr (WORDS == 2) {
    const uint2 r = *reinterpret_cast<const uint2*>(src);
    w[0] = r.x; w[1] = r.y;
  } else {
    w[0] = *reinterpret_cast<const uint32_t*>(src);
  }
}
template <typename T, int WORDS>
__device__ __forceinline__ float element_of_words(const uint32_t (&w)[WORDS], int i) {
  if constexpr (sizeof(T) == 4) return __uint_as_float(w[i]);
  else return __uint_as_float((i & 1) ? (w[i >> 1] & 0xffff0000u) : (w[i >> 1] << 16));     // bf16: the upper half of a float
}

// A block is a (row, part): part 0 the row's q, part 1 its k, part 2 its v.  src [rows, ld]: q [heads x dim] |
// k [kv_heads x dim] | v [kv_heads x vdim] (v absent with values_from_keys).  table: fp32 [max_positions][rot / 2][2]
// (cos, sin) or null.  Where the sizes keep 16-byte pieces aligned and inside a head (and the rotation pairs
// neighbours), a thread keeps its pieces in registers between the sum of squares and the writing; else element by
// element.
template <typename T>
__global__ void __launch_bounds__(256)
window_qk_prepare_kernel(const T* __restrict__ src, long long ld, T* __restrict__ q_out, const float* __restrict__ q_norm,
                         const float* __restrict__ k_norm, float eps, const float* __restrict__ table,
                         const float* __restrict__ freq, int rot,
                         int interleaved, int max_positions, const int* __restrict__ positions,
                         const int* __restrict__ slot_mapping, T* __restrict__ cache, long long cache_slots, int heads,
                         int kv_heads, int dim, int vdim, int values_from_keys, uint32_t* __restrict__ error) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));         // elements a piece
  constexpr int kWords = 4;
  constexpr int kHeld = 2;                                     // pieces a thread keeps
  constexpr int kTurnPairs = 128;                              // computed angles: their cosines and sines, once a block
  __shared__ float scratch[33];
  __shared__ float turn_s[2 * kTurnPairs];
  wait_for_prior_kernels();
  launch_dependents();
  const long long row = blockIdx.x;
  const int part = blockIdx.y;
  const int nq = heads * dim, nk = kv_heads * dim, nv = kv_heads * vdim;
  const long long width = nk + nv;
  int slot = slot_mapping[row];
  if (slot != kPaddingSlot && (slot < 0 || slot >= cache_slots)) {
    if (threadIdx.x == 0 && part == 0) publish_error(error, kRowWithoutPage);
    slot = kPaddingSlot;
  }
  const T* x = src + row * ld;
  const bool aligned = ld % V == 0 && nq % V == 0 && nk % V == 0 && width % V == 0;
  if (part == 2) {                                             // the values: a copy
    if (slot < 0) return;
    const T* v = values_from_keys ? x + nq : x + nq + nk;
    T* dst = cache + slot * width + nk;
    if (aligned && nv % V == 0) {
      for (int e = threadIdx.x * V; e < nv; e += blockDim.x * V)
        *reinterpret_cast<uint4*>(dst + e) = *reinterpret_cast<const uint4*>(v + e);
    } else {
      for (int e = threadIdx.x; e < nv; e += blockDim.x) dst[e] = v[e];
    }
    return;
  }
  int pos = positions[row];
  if (table != nullptr && (pos < 0 || pos >= max_positions)) {
    if (threadIdx.x == 0 && part == 0) publish_error(error, kBadPosition);
    pos = 0;
  }
  const float* cs = table != nullptr ? table + static_cast<long long>(pos) * rot : nullptr;   // (rot / 2) pairs of 2
  const bool turns = rot > 0 && (cs != nullptr || freq != nullptr);
  const float place = static_cast<float>(pos);
  const int half = rot >> 1;
  const T* xp = part == 0 ? x : x + nq;
  const int n = part == 0 ? nq : nk;
  const float* w = part == 0 ? q_norm : k_norm;
  T* dst = part == 0 ? q_out + row * nq : (slot >= 0 ? cache + slot * width : nullptr);
  if (dst == nullptr) return;
  if (turns && cs == nullptr && half <= kTurnPairs) {
    // the row's angles serve every head: their cosines and sines are formed once and read like a table's row
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(place * freq[i], &turn_s[2 * i + 1], &turn_s[2 * i]);
    __syncthreads();
    cs = turn_s;
  }
  const bool pieces = aligned && dim % V == 0 && (!turns || (interleaved ? rot % V == 0 : half % V == 0)) &&
                      n <= static_cast<int>(blockDim.x) * V * kHeld;
  if (pieces) {
    float held[kHeld][V];
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < kHeld; ++u) {
      const int e = (threadIdx.x + u * blockDim.x) * V;
      uint32_t raw[kWords] = {0u, 0u, 0u, 0u};
      if (e < n) load_words<kWords>(raw, xp + e);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        held[u][i] = element_of_words<T, kWords>(raw, i);
        ss = fmaf(held[u][i], held[u][i], ss);
      }
    }
    float inv = 1.0f;
    if (w != nullptr) {
      ss = block_sum(ss, scratch);
      inv = 1.0f / sqrtf(ss / static_cast<float>(n) + eps);
    }
#pragma unroll
    for (int u = 0; u < kHeld; ++u) {
      const int e = (threadIdx.x + u * blockDim.x) * V;
      if (e >= n) continue;
      float o[V];
#pragma unroll
      for (int i = 0; i < V; ++i) o[i] = w != nullptr ? held[u][i] * inv * w[e + i] : held[u][i];
      const int c = e % dim;                                   // the piece lies inside a head, and inside or outside the rotation
      if (turns && c < rot && interleaved) {
#pragma unroll
        for (int i = 0; i < V; i += 2) {
          float cosine, sine;                                     // pair (c + i) / 2
          if (cs != nullptr) { cosine = cs[c + i]; sine = cs[c + i + 1]; }
          else sincosf(place * freq[(c + i) >> 1], &sine, &cosine);
          const float a = o[i], b = o[i + 1];
          o[i] = a * cosine - b * sine;
          o[i + 1] = b * cosine + a * sine;
        }
      } else if (turns && c < rot) {
        // pairs of halves: the partners of this piece are the piece half a rotation away, in the same head
        const bool first = c < half;
        const int pe = first ? e + half : e - half;
        const int pair0 = first ? c : c - half;
        uint32_t raw[kWords];
        load_words<kWords>(raw, xp + pe);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float p = element_of_words<T, kWords>(raw, i);
          if (w != nullptr) p = p * inv * w[pe + i];
          float cosine, sine;
          if (cs != nullptr) { cosine = cs[2 * (pair0 + i)]; sine = cs[2 * (pair0 + i) + 1]; }
          else sincosf(place * freq[pair0 + i], &sine, &cosine);
          o[i] = first ? o[i] * cosine - p * sine : o[i] * cosine + p * sine;
        }
      }
      T out[V];
#pragma unroll
      for (int i = 0; i < V; ++i) out[i] = from_float<T>(o[i]);
      *reinterpret_cast<uint4*>(dst + e) = *reinterpret_cast<const uint4*>(out);
    }
    return;
  }
  float inv = 1.0f;
  if (w != nullptr) {
    float ss = 0.0f;
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      const float v = to_float<T>(xp[e]);
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    inv = 1.0f / sqrtf(ss / static_cast<float>(n) + eps);
  }
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const int c = e % dim;                                     // column within the head
    float o = to_float<T>(xp[e]);
    if (w != nullptr) o = o * inv * w[e];
    if (turns && c < rot) {
      int pair, other;
      bool first;                                              // whether e is the first number of its pair
      if (interleaved) { pair = c >> 1; first = (c & 1) == 0; other = first ? e + 1 : e - 1; }
      else { pair = c < half ? c : c - half; first = c < half; other = first ? e + half : e - half; }
      float p = to_float<T>(xp[other]);
      if (w != nullptr) p = p * inv * w[other];
      float cosine, sine;
      if (cs != nullptr) { cosine = cs[2 * pair]; sine = cs[2 * pair + 1]; }
      else sincosf(place * freq[pair], &sine, &cosine);
      o = first ? o * cosine - p * sine : o * cosine + p * sine;
    }
    dst[e] = from_float<T>(o);
  }
}

// The sums of one (row, head) over the keys first .. last (absolute places; chunks of 32 at multiples of 32): a lane a key
// for the scores, a lane PL neighbouring value columns (PL lane + e) for the sums.  q: 32-bit.
template <typename T, int PL>
__device__ __forceinline__ void window_stretch(const float* q, const T* __restrict__ cache, const int* __restrict__ table,
                                               int first, int last, int pos, int g, int kv_heads, int dim, int vdim,
                                               int page_size, int num_pages, const WindowRule& rule,
                                               const float* bias_of_head, int lane, float (&a)[PL], float& m, float& l,
                                               uint32_t* __restrict__ error) {
  constexpr bool kExact = sizeof(T) == 4;
  const long long width = static_cast<long long>(kv_heads) * (dim + vdim);
  for (int j0 = first & ~31; j0 <= last; j0 += 32) {
    const int j = j0 + lane;
    const bool live = j >= first && j <= last;
    long long at = -1;
    if (live) {
      const int page = table[j / page_size];
      if (page < 0 || page >= num_pages) publish_error(error, kRowWithoutPage);
      else at = (static_cast<long long>(page) * page_size + j % page_size) * width;
    }
    float s = -INFINITY;
    if (at >= 0) {
      const T* k = cache + at + static_cast<long long>(g) * dim;
      // four sums side by side (column e joins sum e % 4), folded at the end: the chain of dependent additions is a
      // quarter as long, and both ways of loading add in the same order
      float d4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      constexpr int kVec = 16 / sizeof(T);
      if (dim % kVec == 0 && width % kVec == 0) {             // 16-byte loads
        for (int e0 = 0; e0 < dim; e0 += 8 * kVec) {
          uint4 r[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) r[u] = *reinterpret_cast<const uint4*>(k + min(e0 + u * kVec, dim - kVec));
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int e = e0 + u * kVec;
            if (e < dim) {
              const T* kk = reinterpret_cast<const T*>(&r[u]);
#pragma unroll
              for (int i = 0; i < kVec; ++i) d4[i & 3] = fmaf(q[e + i], to_float<T>(kk[i]), d4[i & 3]);
            }
          }
        }
      } else {
        int e = 0;
        for (; e + 3 < dim; e += 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) d4[i] = fmaf(q[e + i], to_float<T>(k[e + i]), d4[i]);
        }
#pragma unroll
        for (int i = 0; i < 3; ++i)
          if (e + i < dim) d4[i] = fmaf(q[e + i], to_float<T>(k[e + i]), d4[i]);
      }
      const float d = (d4[0] + d4[1]) + (d4[2] + d4[3]);
      s = finish_score<kExact>(d, rule, bias_of_head, pos - j);
    }
    const float top = fmaxf(m, warp_max(s));
    if (top == -INFINITY) continue;                            // no live key in the chunk
    const float p = at >= 0 ? expf(s - top) : 0.0f;
    const float fix = expf(m - top);                           // exp(-inf) = 0 at the first chunk
    l = fmaf(l, fix, warp_sum(p));
    m = top;
#pragma unroll
    for (int e = 0; e < PL; ++e) a[e] *= fix;
    const long long v_at = at >= 0 ? at + static_cast<long long>(kv_heads) * dim + static_cast<long long>(g) * vdim : -1;
    // the values of kBatch keys are asked for together: shuffles first, then all loads, then the sums in the keys' order.
    // A lane holds the PL neighbouring columns from PL * lane on and loads them in pieces of up to 16 bytes where the
    // sizes keep every piece aligned.
    constexpr int kPiece = PL * sizeof(T) <= 16 ? PL : 16 / static_cast<int>(sizeof(T));
    constexpr int kWords = kPiece * static_cast<int>(sizeof(T)) / 4;
    constexpr int kBatch = PL <= 4 ? 16 : (PL <= 8 ? 8 : 4);
    const bool pieces = vdim % kPiece == 0 && width % kPiece == 0 && (static_cast<long long>(kv_heads) * dim) % kPiece == 0;
    for (int j8 = 0; j8 < 32; j8 += kBatch) {
      long long va[kBatch];
      float wgt[kBatch], x[kBatch][PL];
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        va[b] = __shfl_sync(0xffffffffu, v_at, j8 + b);
        wgt[b] = __shfl_sync(0xffffffffu, p, j8 + b);
      }
      if (pieces) {
        uint32_t raw[kBatch][PL / kPiece][kWords];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          const T* v = cache + (va[b] >= 0 ? va[b] : 0) + PL * lane;
#pragma unroll
          for (int c = 0; c < PL / kPiece; ++c) {
            if (PL * lane + c * kPiece < vdim) load_words<kWords>(raw[b][c], v + c * kPiece);
            else
#pragma unroll
              for (int i = 0; i < kWords; ++i) raw[b][c][i] = 0u;
          }
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b)
#pragma unroll
          for (int e = 0; e < PL; ++e) x[b][e] = element_of_words<T, kWords>(raw[b][e / kPiece], e % kPiece);
      } else {
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          const T* v = cache + (va[b] >= 0 ? va[b] : 0) + PL * lane;
#pragma unroll
          for (int e = 0; e < PL; ++e) x[b][e] = (PL * lane + e < vdim) ? to_float<T>(v[e]) : 0.0f;
        }
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const bool there = va[b] >= 0;
#pragma unroll
        for (int e = 0; e < PL; ++e) a[e] = fmaf(wgt[b], there ? x[b][e] : 0.0f, a[e]);
      }
    }
  }
}

// The sink joins the denominator, the sums are divided, the gate multiplies; a lane holds columns PL lane + e.
template <typename T, int PL>
__device__ __forceinline__ void window_finish(float (&a)[PL], float m, float l, const float* __restrict__ sink, int head,
                                              const T* __restrict__ gate, int vdim, int lane, T* __restrict__ out,
                                              uint32_t* __restrict__ error) {
  float fix = 1.0f;
  if (sink != nullptr) {
    const float s = sink[head];
    const float top = fmaxf(m, s);
    fix = expf(m - top);
    l = fmaf(l, fix, expf(s - top));
  }
  if (!(l > 0.0f) || l > 3.0e38f) {
    if (lane == 0) publish_error(error, kAttentionDenominator);
    l = 1.0f;
  }
  float f = fix / l;
  if (gate != nullptr) f *= 1.0f / (1.0f + expf(-to_float<T>(*gate)));
#pragma unroll
  for (int e = 0; e < PL; ++e)
    if (PL * lane + e < vdim) out[PL * lane + e] = from_float<T>(a[e] * f);
}

// A warp a (row, head) and a part of its keys.  splits == 1: the whole row, finished here.  More: part blockIdx.y of the
// keys of rows whose request brings at most small_rows rows, its sums to partial [row][head][split][2 + 32 PL]: m, l, a (lane by lane).
template <typename T, int PL>
__global__ void __launch_bounds__(128)
window_attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ cache,
                                const int* __restrict__ block_table, int table_width,
                                const int* __restrict__ request_of_row, const int* __restrict__ positions,
                                const int* __restrict__ cu_q, int rows, int heads, int kv_heads, int dim, int vdim,
                                int page_size, int num_pages, WindowRule rule, const float* __restrict__ sink,
                                const T* __restrict__ gate, long long ld_gate, int splits, int small_rows,
                                float* __restrict__ partial, uint32_t* __restrict__ error) {
  extern __shared__ float smem[];
  wait_for_prior_kernels();
  launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (unit >= static_cast<long long>(rows) * heads) return;
  const int row = static_cast<int>(unit / heads), head = static_cast<int>(unit % heads);
  const int req = request_of_row[row];
  T* o = out + unit * vdim;
  if (req < 0) {                                               // a row of padding: zeros, so that nothing unset travels on
    if (blockIdx.y == 0)
      for (int e = lane; e < vdim; e += 32) o[e] = from_float<T>(0.0f);
    return;
  }
  if (splits > 1 && cu_q[req + 1] - cu_q[req] > small_rows) return;
  const int g = head / (heads / kv_heads);
  float* qs = smem + warp * dim;
  const T* qr = q + unit * dim;
  for (int e = lane; e < dim; e += 32) qs[e] = to_float<T>(qr[e]);
  __syncwarp();
  const int pos = positions[row];
  const int first = rule.window > 0 ? max(0, pos - rule.window + 1) : 0;
  const int kept = min(rule.keep_first, first);                // keys 0 .. kept - 1 lie before the window and stay seen
  const int* table = block_table + static_cast<long long>(req) * table_width;
  const float* bias_of_head = rule.bias != nullptr ? rule.bias + static_cast<long long>(head) * rule.distances : nullptr;
  float a[PL];
#pragma unroll
  for (int e = 0; e < PL; ++e) a[e] = 0.0f;
  float m = -INFINITY, l = 0.0f;
  // the chunks of the kept keys and of the window, numbered through; a part takes a stretch of them
  const int kept_chunks = kept > 0 ? ((kept - 1) >> 5) + 1 : 0;
  const int chunk0 = first >> 5, win_chunks = (pos >> 5) - chunk0 + 1;
  int c_lo = 0, c_hi = kept_chunks + win_chunks;
  if (splits > 1) {
    const int per = (c_hi + splits - 1) / splits;
    c_lo = static_cast<int>(blockIdx.y) * per;
    c_hi = min(c_hi, c_lo + per);
  }
  if (c_lo < kept_chunks) {
    const int lo = c_lo << 5, hi = min(kept, min(c_hi, kept_chunks) << 5) - 1;
    if (lo <= hi)
      window_stretch<T, PL>(qs, cache, table, lo, hi, pos, g, kv_heads, dim, vdim, page_size, num_pages, rule, bias_of_head,
                            lane, a, m, l, error);
  }
  if (c_hi > kept_chunks) {
    const int lo = max(first, (chunk0 + max(c_lo, kept_chunks) - kept_chunks) << 5);
    const int hi = min(pos, ((chunk0 + c_hi - kept_chunks) << 5) - 1);
    if (lo <= hi)
      window_stretch<T, PL>(qs, cache, table, lo, hi, pos, g, kv_heads, dim, vdim, page_size, num_pages, rule, bias_of_head,
                            lane, a, m, l, error);
  }
  if (splits > 1) {
    float* p = partial + (unit * splits + blockIdx.y) * (2 + 32 * PL);
    if (lane == 0) { p[0] = m; p[1] = l; }
#pragma unroll
    for (int e = 0; e < PL; ++e)
      p[2 + 32 * e + lane] = a[e];                             // (column PL lane + e; beyond vdim: zero)
    return;
  }
  window_finish<T, PL>(a, m, l, sink, head, gate != nullptr ? gate + row * ld_gate + head : nullptr, vdim, lane, o, error);
}

// A warp a (row, head): the parts' sums folded in order, then the sink, the division and the gate.
template <typename T, int PL>
__global__ void __launch_bounds__(128)
window_attention_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, const int* __restrict__ request_of_row,
                              const int* __restrict__ cu_q, int rows, int heads, int vdim, int splits, int small_rows,
                              const float* __restrict__ sink, const T* __restrict__ gate, long long ld_gate,
                              uint32_t* __restrict__ error) {
  wait_for_prior_kernels();
  launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (unit >= static_cast<long long>(rows) * heads) return;
  const int row = static_cast<int>(unit / heads), head = static_cast<int>(unit % heads);
  const int req = request_of_row[row];
  if (req < 0 || cu_q[req + 1] - cu_q[req] > small_rows) return;
  const float* base = partial + unit * splits * (2 + 32 * PL);
  float pm = -INFINITY, pl = 0.0f;
  if (lane < splits) {
    const float* p = base + static_cast<long long>(lane) * (2 + 32 * PL);
    pm = p[0]; pl = p[1];
  }
  const float m = warp_max(pm);
  const float f = pm == -INFINITY ? 0.0f : expf(pm - m);
  const float l = warp_sum(pl * f);
  float a[PL];
#pragma unroll
  for (int e = 0; e < PL; ++e) a[e] = 0.0f;
#pragma unroll 8
  for (int s = 0; s < splits; ++s) {
    const float* p = base + static_cast<long long>(s) * (2 + 32 * PL);
    const float d = __shfl_sync(0xffffffffu, f, s);
#pragma unroll
    for (int e = 0; e < PL; ++e)
      a[e] = fmaf(p[2 + 32 * e + lane], d, a[e]);
  }
  window_finish<T, PL>(a, m, l, sink, head, gate != nullptr ? gate + row * ld_gate + head : nullptr, vdim, lane,
                       out + unit * vdim, error);
}

// Tensor cores for requests of more than small_rows rows (bf16).  A block is kTileRows consecutive rows of one request and one
// head (found on the device from cu_q: block x of the grid is the x-th such tile of the step, blocks beyond the last
// leave); a warp is 16 of the rows.  Key tiles of 64 (the keys and values of the head's key/value head) come by
// cp.async into two buffers: first the tiles that hold kept first tokens before the window, then the window's; columns
// beyond dim / vdim up to the instance's DIM / VDIM are zeros.  Per warp: S = Q K^T (32-bit), the score finished (scale,
// cap, bias by distance), the running maximum and sum of a row in the exp2 domain, P as a bf16 pair (rounding,
// remainder) into O += P V.  At the end the sink joins the sum and the gate multiplies.
constexpr int kTileWarps = 8;                               // 16 rows a warp: 128 rows a block, two blocks a multiprocessor
constexpr int kTileRows = 16 * kTileWarps, kTileThreads = 32 * kTileWarps;

template <int DIM, int VDIM>
__global__ void __launch_bounds__(kTileThreads, 2)
window_attention_tile_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                             const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int table_width,
                             const int* __restrict__ cu_q, const int* __restrict__ q_start, int requests, int heads,
                             int kv_heads, int dim, int vdim, int page_size, int num_pages, WindowRule rule,
                             const float* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, long long ld_gate,
                             int small_rows, uint32_t* __restrict__ error) {
  typedef __nv_bfloat16 bf16;
  constexpr int QLD = DIM + 8, VLD = VDIM + 8;                // row strides that keep ldmatrix free of bank conflicts
  constexpr int QC = DIM / 8, VC = VDIM / 8, PER = QC + VC;   // 16-byte pieces of a row of q or k, of v, of a key
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(16) unsigned char window_tile_smem[];
  bf16* Qs = reinterpret_cast<bf16*>(window_tile_smem);       // [kTileRows][QLD]
  bf16* Ks = Qs + kTileRows * QLD;                                   // [2][64][QLD]
  bf16* Vs = Ks + 2 * 64 * QLD;                               // [2][64][VLD]
  __shared__ int tile_info[2];
  __shared__ float bias_s[2][kTileRows + 64];                 // the bias of a key tile by (row - key) + 63 of the block
  wait_for_prior_kernels();
  launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    // the last tiles of a request have the most keys: they start first, so that the short ones fill the end
    int t = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x), found = -1, at = 0;
    for (int r = 0; r < requests; ++r) {
      const int n = cu_q[r + 1] - cu_q[r];
      if (n <= small_rows) continue;
      const int tiles = (n + kTileRows - 1) / kTileRows;
      if (t < tiles) { found = r; at = cu_q[r] + t * kTileRows; break; }
      t -= tiles;
    }
    tile_info[0] = found;
    tile_info[1] = at;
  }
  __syncthreads();
  const int req = tile_info[0];
  if (req < 0) return;
  const int row0 = tile_info[1];
  const int nrows = min(kTileRows, cu_q[req + 1] - row0);
  const int pos0 = q_start[req] + (row0 - cu_q[req]);
  const int head = blockIdx.y, g = head / (heads / kv_heads);
  const long long width = static_cast<long long>(kv_heads) * (dim + vdim);
  const int* table = block_table + static_cast<long long>(req) * table_width;
  const int key_last = pos0 + nrows - 1;
  const int key_first = rule.window > 0 ? max(0, pos0 - rule.window + 1) : 0;
  const int kept = min(rule.keep_first, key_first);           // kept keys that lie before the first row's window
  const float* bias_of_head = rule.bias != nullptr ? rule.bias + static_cast<long long>(head) * rule.distances : nullptr;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

  for (int c = tid; c < kTileRows * QC; c += kTileThreads) {
    const int rr = c / QC, col = (c % QC) * 8;
    bf16* dst = Qs + rr * QLD + col;
    if (rr < nrows && col < dim) mma::copy_async_16(dst, q + (static_cast<long long>(row0 + rr) * heads + head) * dim + col);
    else *reinterpret_cast<uint4*>(dst) = zero;
  }
  // kTileThreads / 64 threads a key: each looks the key's place in the cache up, the pieces are dealt round
  constexpr int kPerKey = kTileThreads / 64;
  auto load_keys = [&](int buf, int j0) {
    const int key = tid / kPerKey, j = j0 + key;
    bf16* kb = Ks + (buf * 64 + key) * QLD;
    bf16* vb = Vs + (buf * 64 + key) * VLD;
    long long at = -1;
    if (j <= key_last && (j >= key_first || j < kept)) {
      const int page = table[page_shift >= 0 ? j >> page_shift : j / page_size];
      const int offset = page_shift >= 0 ? j & (page_size - 1) : j % page_size;
      if (page < 0 || page >= num_pages) publish_error(error, kRowWithoutPage);
      else at = (static_cast<long long>(page) * page_size + offset) * width;
    }
    const bf16* ksrc = cache + at + static_cast<long long>(g) * dim;
    const bf16* vsrc = cache + at + static_cast<long long>(kv_heads) * dim + static_cast<long long>(g) * vdim;
#pragma unroll
    for (int cc = tid % kPerKey; cc < PER; cc += kPerKey) {
      if (cc < QC) {
        const int col = cc * 8;
        if (at >= 0 && col < dim) mma::copy_async_16(kb + col, ksrc + col);
        else *reinterpret_cast<uint4*>(kb + col) = zero;
      } else {
        const int col = (cc - QC) * 8;
        if (at >= 0 && col < vdim) mma::copy_async_16(vb + col, vsrc + col);
        else *reinterpret_cast<uint4*>(vb + col) = zero;
      }
    }
    if (bias_of_head != nullptr && tid < kTileRows + 63)      // distance (pos0 + row) - (j0 + key), row - key = tid - 63
      mma::copy_async_4(&bias_s[buf][tid], bias_of_head + min(max(pos0 - j0 + tid - 63, 0), rule.distances - 1));
    mma::copy_async_commit();
  };
  // the tiles in the order they are visited: those of the kept keys that end before the window's first tile, then the window's
  const int tile_lo = key_first >> 6, tile_hi = key_last >> 6;
  const int kept_tiles = kept > 0 ? min(((kept - 1) >> 6) + 1, tile_lo) : 0;
  const int visits = kept_tiles + (tile_hi - tile_lo + 1);
  auto tile_of = [&](int v) { return v < kept_tiles ? v : tile_lo + (v - kept_tiles); };
  load_keys(0, tile_of(0) * 64);                              // (the group also holds the copies of q)

  const int wr0 = warp * 16;
  const int ra = wr0 + (lane >> 2), rb = ra + 8;
  const int pos_a = ra < nrows ? pos0 + ra : -1, pos_b = rb < nrows ? pos0 + rb : -1;
  const int warp_first = pos0 + wr0, warp_last = pos0 + min(wr0 + 15, nrows - 1);
  const bool plain = rule.cap <= 0.0f && bias_of_head == nullptr;
  float O[VDIM / 8][4];
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
#pragma unroll
  for (int n = 0; n < VDIM / 8; ++n) O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.0f;
  for (int v = 0; v < visits; ++v) {
    const int buf = v & 1;
    mma::copy_async_wait<0>();
    __syncthreads();
    const int j0 = tile_of(v) * 64;
    // the warp's rows see something of this tile: a key of their windows, or a kept key
    const bool any = wr0 < nrows && j0 <= warp_last &&
                     (rule.window <= 0 || j0 + 63 > warp_first - rule.window || j0 < rule.keep_first);
    const bf16* kb = Ks + buf * 64 * QLD;
    const bf16* vb = Vs + buf * 64 * VLD;
    float S[8][4];
    if (any) {
#pragma unroll
      for (int n = 0; n < 8; ++n) S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.0f;
      {
        // the fragments of step kk + 1 are asked for before the products of step kk: a load is never waited for
        uint32_t a[2][4], b[2][4][4];
        auto fetch = [&](int kk, int f) {
          mma::load_matrices(a[f], Qs + (wr0 + (lane & 15)) * QLD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int np = 0; np < 4; ++np)
            mma::load_matrices(b[f][np], kb + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * QLD + kk * 16 + ((lane >> 3) & 1) * 8);
        };
        fetch(0, 0);
#pragma unroll
        for (int kk = 0; kk < DIM / 16; ++kk) {
          if (kk + 1 < DIM / 16) fetch(kk + 1, (kk + 1) & 1);
#pragma unroll
          for (int np = 0; np < 4; ++np) {
            mma::multiply_add(S[2 * np], a[kk & 1], b[kk & 1][np][0], b[kk & 1][np][1]);
            mma::multiply_add(S[2 * np + 1], a[kk & 1], b[kk & 1][np][2], b[kk & 1][np][3]);
          }
        }
      }
    }
    // the next tile is asked for while the tensor cores work on this tile's scores (its buffer was let go of at the end
    // of the step before)
    if (v + 1 < visits) load_keys(buf ^ 1, tile_of(v + 1) * 64);
    if (any) {
      // a tile that every row of the warp sees whole needs no mask
      const bool whole = j0 + 63 <= warp_first && (rule.window <= 0 || j0 > warp_last - rule.window || j0 + 63 < rule.keep_first);
      const float* bias_t = bias_of_head != nullptr ? bias_s[buf] + 63 : nullptr;
      const int la = ra - 2 * (lane & 3), lb = rb - 2 * (lane & 3);   // row - key of the thread's first column
      float top_a = -INFINITY, top_b = -INFINITY;
      auto finish = [&](float dot, int rel) {                  // rel: row - key inside the block's tile
        float s = dot * rule.scale;
        if (rule.cap > 0.0f) s = capped<false>(s, rule.cap);
        if (bias_t != nullptr) s += bias_t[rel];
        return s * kLog2e;
      };
      if (whole) {
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (plain) {
              S[n][c] *= rule.scale * kLog2e;
              S[n][2 + c] *= rule.scale * kLog2e;
            } else {
              S[n][c] = finish(S[n][c], la - n * 8 - c);
              S[n][2 + c] = finish(S[n][2 + c], lb - n * 8 - c);
            }
            top_a = fmaxf(top_a, S[n][c]);
            top_b = fmaxf(top_b, S[n][2 + c]);
          }
        }
      } else {
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int key = j0 + n * 8 + 2 * (lane & 3) + c;
            const bool see_a = key <= pos_a && (rule.window <= 0 || key > pos_a - rule.window || key < rule.keep_first);
            const bool see_b = key <= pos_b && (rule.window <= 0 || key > pos_b - rule.window || key < rule.keep_first);
            const float sa = plain ? S[n][c] * (rule.scale * kLog2e) : finish(S[n][c], la - n * 8 - c);
            const float sb = plain ? S[n][2 + c] * (rule.scale * kLog2e) : finish(S[n][2 + c], lb - n * 8 - c);
            S[n][c] = see_a ? sa : -INFINITY;
            S[n][2 + c] = see_b ? sb : -INFINITY;
            top_a = fmaxf(top_a, S[n][c]);
            top_b = fmaxf(top_b, S[n][2 + c]);
          }
        }
      }
      top_a = fmaxf(top_a, __shfl_xor_sync(0xffffffffu, top_a, 1));
      top_a = fmaxf(top_a, __shfl_xor_sync(0xffffffffu, top_a, 2));
      top_b = fmaxf(top_b, __shfl_xor_sync(0xffffffffu, top_b, 1));
      top_b = fmaxf(top_b, __shfl_xor_sync(0xffffffffu, top_b, 2));
      const float new_a = fmaxf(m_a, top_a), new_b = fmaxf(m_b, top_b);
      const float ref_a = new_a == -INFINITY ? 0.0f : new_a, ref_b = new_b == -INFINITY ? 0.0f : new_b;
      const float fix_a = mma::exp2_fast(m_a - ref_a), fix_b = mma::exp2_fast(m_b - ref_b);
      m_a = new_a;
      m_b = new_b;
      float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        S[n][0] = mma::exp2_fast(S[n][0] - ref_a);
        S[n][1] = mma::exp2_fast(S[n][1] - ref_a);
        S[n][2] = mma::exp2_fast(S[n][2] - ref_b);
        S[n][3] = mma::exp2_fast(S[n][3] - ref_b);
        sum_a += S[n][0] + S[n][1];
        sum_b += S[n][2] + S[n][3];
      }
      l_a = fmaf(l_a, fix_a, sum_a);
      l_b = fmaf(l_b, fix_b, sum_b);
      if (__any_sync(0xffffffffu, fix_a != 1.0f || fix_b != 1.0f)) {   // (a maximum that stays leaves the sums as they are)
#pragma unroll
        for (int n = 0; n < VDIM / 8; ++n) {
          O[n][0] *= fix_a;
          O[n][1] *= fix_a;
          O[n][2] *= fix_b;
          O[n][3] *= fix_b;
        }
      }
      {
        // 16 keys by 64 value columns a step: the values of the next step are asked for before this step's products;
        // the eight products with the roundings come before the eight with the remainders, so that none waits for
        // the one before it
        constexpr int kGroups = VDIM / 64, kSteps = 4 * kGroups;
        uint32_t b[2][4][4];
        auto fetch = [&](int t, int f) {
          const int kk = t / kGroups, v0 = (t % kGroups) * 4;
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mma::load_matrices_transposed(b[f][u], vb + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * VLD + (v0 + u) * 16 + (lane >> 4) * 8);
        };
        fetch(0, 0);
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int t = 0; t < kSteps; ++t) {
          const int kk = t / kGroups, v0 = (t % kGroups) * 4;
          if (t + 1 < kSteps) fetch(t + 1, (t + 1) & 1);
          if (t % kGroups == 0) {
            hi[0] = mma::pack(S[2 * kk][0], S[2 * kk][1]);
            hi[1] = mma::pack(S[2 * kk][2], S[2 * kk][3]);
            hi[2] = mma::pack(S[2 * kk + 1][0], S[2 * kk + 1][1]);
            hi[3] = mma::pack(S[2 * kk + 1][2], S[2 * kk + 1][3]);
            lo[0] = mma::pack_remainder(S[2 * kk][0], S[2 * kk][1], hi[0]);
            lo[1] = mma::pack_remainder(S[2 * kk][2], S[2 * kk][3], hi[1]);
            lo[2] = mma::pack_remainder(S[2 * kk + 1][0], S[2 * kk + 1][1], hi[2]);
            lo[3] = mma::pack_remainder(S[2 * kk + 1][2], S[2 * kk + 1][3], hi[3]);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            mma::multiply_add(O[2 * (v0 + u)], hi, b[t & 1][u][0], b[t & 1][u][1]);
            mma::multiply_add(O[2 * (v0 + u) + 1], hi, b[t & 1][u][2], b[t & 1][u][3]);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            mma::multiply_add(O[2 * (v0 + u)], lo, b[t & 1][u][0], b[t & 1][u][1]);
            mma::multiply_add(O[2 * (v0 + u) + 1], lo, b[t & 1][u][2], b[t & 1][u][3]);
          }
        }
      }
    }
    // (no barrier here: the next copies into this tile's buffers are issued behind the next step's barrier, which no
    // warp passes before every warp has left this step)
  }
  if (wr0 >= nrows) return;
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  float fix_a = 1.0f, fix_b = 1.0f;
  if (sink != nullptr) {                                      // the sink's term, in the exp2 domain like the others
    const float s = sink[head] * kLog2e;
    const float top_a = fmaxf(m_a, s), top_b = fmaxf(m_b, s);
    fix_a = exp2f(m_a - top_a);
    fix_b = exp2f(m_b - top_b);
    l_a = fmaf(l_a, fix_a, exp2f(s - top_a));
    l_b = fmaf(l_b, fix_b, exp2f(s - top_b));
  }
  const bool bad = (ra < nrows && (!(l_a > 0.0f) || l_a > 3.0e38f)) || (rb < nrows && (!(l_b > 0.0f) || l_b > 3.0e38f));
  if (bad) publish_error(error, kAttentionDenominator);
  float f_a = l_a > 0.0f ? fix_a / l_a : 0.0f, f_b = l_b > 0.0f ? fix_b / l_b : 0.0f;
  if (gate != nullptr) {
    if (ra < nrows) f_a *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[(row0 + ra) * ld_gate + head])));
    if (rb < nrows) f_b *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[(row0 + rb) * ld_gate + head])));
  }
#pragma unroll
  for (int n = 0; n < VDIM / 8; ++n) {
    const int col = n * 8 + 2 * (lane & 3);
    if (col >= vdim) continue;                                // vdim is a multiple of 8: the pair is inside
    if (ra < nrows)
      *reinterpret_cast<__nv_bfloat162*>(out + (static_cast<long long>(row0 + ra) * heads + head) * vdim + col) =
          __floats2bfloat162_rn(O[n][0] * f_a, O[n][1] * f_a);
    if (rb < nrows)
      *reinterpret_cast<__nv_bfloat162*>(out + (static_cast<long long>(row0 + rb) * heads + head) * vdim + col) =
          __floats2bfloat162_rn(O[n][2] * f_b, O[n][3] * f_b);
  }
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

// src [rows, ld]: q [heads x dim] | k [kv_heads x dim] | v [kv_heads x vdim] (no v columns with values_from_keys: the
// key columns as they are become the values); q_out [rows, heads x dim]; q_norm fp32 [heads x dim], k_norm fp32
// [kv_heads x dim] or null; table fp32 [max_positions, rot / 2, 2] or null, and then freq fp32 [rot / 2] or null (angles
// computed from the position); cache [num_pages, page_size, kv_heads (dim + vdim)].  write_kv 0: the rows hold q alone and
// nothing goes to the cache.
extern "C" int pih_window_qk_prepare(int dtype, const void* src, long long ld, void* q_out, const void* q_norm,
                                     const void* k_norm, float eps, const void* table, const void* freq, int rot,
                                     int interleaved, int max_positions, const void* positions, const void* slot_mapping,
                                     void* cache, int page_size, int num_pages, int rows, int heads, int kv_heads, int dim,
                                     int vdim, int values_from_keys, int write_kv, void* error, void* stream) {
  if (rows <= 0) return 0;
  if (table != nullptr && freq != nullptr) return PIH_ERR_BAD_ARGUMENT;
  if (rot < 0 || rot > dim || (rot & 1) || heads < 1 || kv_heads < 1 || (values_from_keys && vdim != dim))
    return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long slots = static_cast<long long>(num_pages) * page_size;
  const int threads = heads * dim >= 1024 ? 256 : 128;
#define PIH_WQK(T)                                                                                                     \
  launch_kernel(window_qk_prepare_kernel<T>, dim3(rows, write_kv ? 3 : 1), dim3(threads), 0, s,                        \
                static_cast<const T*>(src), ld,                                                                        \
                static_cast<T*>(q_out), static_cast<const float*>(q_norm), static_cast<const float*>(k_norm), eps,     \
                static_cast<const float*>(rot > 0 ? table : nullptr), static_cast<const float*>(rot > 0 ? freq : nullptr), \
                rot, interleaved, max_positions,                                                                       \
                static_cast<const int*>(positions), static_cast<const int*>(slot_mapping), static_cast<T*>(cache), slots, \
                heads, kv_heads, dim, vdim, values_from_keys, static_cast<uint32_t*>(error))
  if (dtype == PIH_F32) PIH_WQK(float);
  else if (dtype == PIH_BF16) PIH_WQK(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_WQK
  PIH_LAUNCH_CHECK();
  return 0;
}

template <int DIM, int VDIM>
static int launch_window_tile(cudaStream_t s, unsigned tiles, const void* q, void* out, const void* cache,
                              const void* block_table, int table_width, const void* cu_q, const void* q_start, int requests,
                              int heads, int kv_heads, int dim, int vdim, int page_size, int num_pages, const WindowRule& rule,
                              const void* sink, const void* gate, long long ld_gate, int small_rows, void* error) {
  const size_t smem = ((static_cast<size_t>(kTileRows) + 2 * 64) * (DIM + 8) + 2 * 64 * (VDIM + 8)) * sizeof(bf16);
  static bool raised = false;
  if (!raised && smem > 48 * 1024) {
    cudaFuncSetAttribute(window_attention_tile_kernel<DIM, VDIM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(smem));
    raised = true;
  }
  launch_kernel(window_attention_tile_kernel<DIM, VDIM>, dim3(tiles, heads), dim3(kTileThreads), smem, s, static_cast<const bf16*>(q),
                static_cast<bf16*>(out), static_cast<const bf16*>(cache), static_cast<const int*>(block_table), table_width,
                static_cast<const int*>(cu_q), static_cast<const int*>(q_start), requests, heads, kv_heads, dim, vdim,
                page_size, num_pages, rule, static_cast<const float*>(sink), static_cast<const bf16*>(gate), ld_gate,
                small_rows, static_cast<uint32_t*>(error));
  PIH_LAUNCH_CHECK();
  return 0;
}

// 1 when the tensor-core kernel has an instance for these sizes (bf16; dim and vdim multiples of 8 up to 128).
extern "C" int pih_window_attention_tile_takes(int dim, int vdim) {
  return dim >= 8 && vdim >= 8 && dim % 8 == 0 && vdim % 8 == 0 && dim <= 128 && vdim <= 128;
}

// The attention of the step's rows: q [rows, heads x dim] (prepared), out [rows, heads x vdim].  bias fp32
// [heads, distances] or null; sink fp32 [heads] or null; gate [rows, ld_gate] of the compute dtype (column h: head h's
// logit) or null.  ``tile`` (bf16 only, sizes that pih_window_attention_tile_takes): requests of more than 16 rows run
// on the tensor-core kernel.  ``small``: the other rows (all rows without ``tile``) run on the warp kernel, their keys
// cut into ``splits`` parts (1: uncut) through ``partial`` (fp32 [rows, heads, splits, 2 + 32 x the value columns a lane]).
extern "C" int pih_window_attention(int dtype, const void* q, void* out, const void* cache, const void* block_table,
                                    int table_width, const void* request_of_row, const void* positions, const void* cu_q,
                                    const void* q_start, int rows, int requests, int heads, int kv_heads, int dim, int vdim,
                                    int page_size, int num_pages, float scale, float cap, const void* bias, int distances,
                                    int window, int keep_first, const void* sink, const void* gate, long long ld_gate,
                                    int tile, int small, int splits, void* partial, void* error, void* stream) {
  if (rows <= 0) return 0;
  if (dim > 1024 || vdim > 32 * kWinMaxPerLane || heads % kv_heads || splits < 1) return PIH_ERR_UNSUPPORTED;
  if (tile && (dtype != PIH_BF16 || !pih_window_attention_tile_takes(dim, vdim))) return PIH_ERR_UNSUPPORTED;
  if (splits > 32 || (splits > 1 && partial == nullptr) || window < 0 || keep_first < 0 || (bias != nullptr && distances < 1))
    return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  WindowRule rule;
  rule.window = window;
  rule.keep_first = window > 0 ? keep_first : 0;
  rule.scale = scale;
  rule.cap = cap;
  rule.bias = static_cast<const float*>(bias);
  rule.distances = distances;
  const int small_rows = tile ? 16 : 0x7fffffff;
  if (tile) {
    const unsigned tiles = static_cast<unsigned>((rows + kTileRows - 1) / kTileRows + requests);
    int rc;
#define PIH_TILE(D, V)                                                                                                 \
  rc = launch_window_tile<D, V>(s, tiles, q, out, cache, block_table, table_width, cu_q, q_start, requests, heads,    \
                                kv_heads, dim, vdim, page_size, num_pages, rule, sink, gate, ld_gate, small_rows, error)
    if (dim <= 32) { if (vdim <= 64) PIH_TILE(32, 64); else PIH_TILE(32, 128); }
    else if (dim <= 64) { if (vdim <= 64) PIH_TILE(64, 64); else PIH_TILE(64, 128); }
    else { if (vdim <= 64) PIH_TILE(128, 64); else PIH_TILE(128, 128); }
#undef PIH_TILE
    if (rc != 0) return rc;
  }
  if (!small) return 0;
  const long long units = static_cast<long long>(rows) * heads;
  const size_t smem = 4 * static_cast<size_t>(dim) * sizeof(float);
  const dim3 grid(static_cast<unsigned>((units + 3) / 4), splits);
#define PIH_WAG_PL(T, PL)                                                                                              \
  do {                                                                                                                 \
    launch_kernel(window_attention_generic_kernel<T, PL>, grid, dim3(128), smem, s, static_cast<const T*>(q),          \
                  static_cast<T*>(out), static_cast<const T*>(cache), static_cast<const int*>(block_table), table_width, \
                  static_cast<const int*>(request_of_row), static_cast<const int*>(positions),                         \
                  static_cast<const int*>(cu_q), rows, heads, kv_heads, dim, vdim, page_size, num_pages, rule,         \
                  static_cast<const float*>(sink), static_cast<const T*>(gate), ld_gate, splits, small_rows,           \
                  static_cast<float*>(partial), static_cast<uint32_t*>(error));                                        \
    PIH_LAUNCH_CHECK();                                                                                                \
    if (splits > 1)                                                                                                    \
      launch_kernel(window_attention_merge_kernel<T, PL>, dim3(grid.x), dim3(128), 0, s,                               \
                    static_cast<const float*>(partial), static_cast<T*>(out), static_cast<const int*>(request_of_row), \
                    static_cast<const int*>(cu_q), rows, heads, vdim, splits, small_rows,                              \
                    static_cast<const float*>(sink), static_cast<const T*>(gate), ld_gate, static_cast<uint32_t*>(error)); \
  } while (0)
#define PIH_WAG(T)                                                                                                     \
  do {                                                                                                                 \
    if (vdim <= 64) PIH_WAG_PL(T, 2);                                                                                  \
    else if (vdim <= 128) PIH_WAG_PL(T, 4);                                                                            \
    else if (vdim <= 256) PIH_WAG_PL(T, 8);                                                                            \
    else PIH_WAG_PL(T, 16);                                                                                            \
  } while (0)
  if (dtype == PIH_F32) PIH_WAG(float);
  else if (dtype == PIH_BF16) PIH_WAG(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_WAG_PL
#undef PIH_WAG
  PIH_LAUNCH_CHECK();
  return 0;
}
