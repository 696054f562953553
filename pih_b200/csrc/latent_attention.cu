// Attention over a cached latent: every token caches ONE vector c of ``rank`` numbers, and a head's key and value
// are products of c with that head's matrices.  Because both are linear in c, the head's key matrix is folded into
// the query (q' = W_k^T q, ``rank`` numbers) and its value matrix is applied after the weighted sum of latents:
//
//   score_j = (q' . c_j) * scale        o' = sum_j p_j c_j        head output = W_v o'
//
// so the kernels here see one shared "key = value = c_j" for all heads (the folded products are batched matrix
// products outside).  The softmax denominator may hold a sink: a learned logit per head that has no key and no value;
// it is the state the running softmax starts from (maximum = sink, sum = 1, accumulator = 0).  A sigmoid gate per
// (row, head) may scale the output.  Scores, weights and sums are 32-bit; keys are visited in ascending position, so a
// row's result does not depend on how its prompt was cut or batched.
//
//   latent_write              c = rmsnorm(raw latent) * w  ->  the paged cache [pages, page_size, rank]
//   latent_attention_generic  one warp a (row, head), keys in order: any rank up to 512; the 32-bit path
//   latent_attention_split    a block a (row, part of its keys, 8 heads) and a merge: bf16, any rank
//   latent_attention_mma      the same cut on tensor cores (the heads are the rows of the MMA): bf16, rank 64 .. 512
#include "common.cuh"

namespace pih {

template <typename T>
__global__ void __launch_bounds__(128)
latent_write_kernel(const T* __restrict__ raw, long long ld, const float* __restrict__ weight, float eps,
                    T* __restrict__ cache, const int* __restrict__ slot_mapping, int rows, int rank, long long cache_rows,
                    int cache_width, int rot, int interleaved, const float* __restrict__ freq,
                    const int* __restrict__ positions, const T* __restrict__ q_raw, long long ldq,
                    const float* __restrict__ q_weight, T* __restrict__ q_out, int q_rank, uint32_t* err) {
  wait_for_prior_kernels();
  launch_dependents();
  int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) {
    // the warps behind the rows' own: the queries' latent of row ``row - rows``, normed into a buffer of its own
    row -= rows;
    if (q_raw == nullptr || row >= rows) return;
    const T* src = q_raw + static_cast<long long>(row) * ldq;
    float ss = 0.0f;
    for (int i = lane; i < q_rank; i += 32) { const float a = to_float<T>(src[i]); ss = fmaf(a, a, ss); }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / static_cast<float>(q_rank) + eps);
    T* dst = q_out + static_cast<long long>(row) * q_rank;
    for (int i = lane; i < q_rank; i += 32) dst[i] = from_float<T>(to_float<T>(src[i]) * scale * q_weight[i]);
    return;
  }
  const int slot = slot_mapping[row];
  if (slot == kPaddingSlot) return;
  if (slot < 0 || slot >= cache_rows) {
    if (lane == 0) publish_error(err, kRowWithoutPage);
    return;
  }
  const T* src = raw + static_cast<long long>(row) * ld;
  float ss = 0.0f;
  for (int i = lane; i < rank; i += 32) { const float a = to_float<T>(src[i]); ss = fmaf(a, a, ss); }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / static_cast<float>(rank) + eps);
  T* dst = cache + static_cast<long long>(slot) * cache_width;      // (columns behind rank + rot are left as they are)
  for (int i = lane; i < rank; i += 32) dst[i] = from_float<T>(to_float<T>(src[i]) * scale * weight[i]);
  if (rot > 0) {
    // behind the latent: ``rot`` more numbers, not normed, rotated by the row's position (32-bit angles)
    const float place = static_cast<float>(positions[row]);
    const int half = rot >> 1;
    for (int c = lane; c < rot; c += 32) {
      int pair, other;
      bool first;
      if (interleaved) { pair = c >> 1; first = (c & 1) == 0; other = first ? c + 1 : c - 1; }
      else { pair = c < half ? c : c - half; first = c < half; other = first ? c + half : c - half; }
      float sn, cs;
      sincosf(place * freq[pair], &sn, &cs);
      const float a = to_float<T>(src[rank + c]), b = to_float<T>(src[rank + other]);
      dst[rank + c] = from_float<T>(first ? a * cs - b * sn : a * cs + b * sn);
    }
  }
}

constexpr int kLatentPerLane = 32;          // rank <= 32 * 32 (instances: 2, 4, 8, 16, 24, 32)

// q: [rows, heads, rank] (the folded queries); gate: [rows, ldg] logits, column h, or null; sink: fp32 [heads] or null.
template <typename T, int kPerLane>
__global__ void __launch_bounds__(128)
latent_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ gate, long long ldg,
                                const float* __restrict__ sink, const T* __restrict__ cache,
                                const int* __restrict__ block_table, int table_width, const int* __restrict__ request_of_row,
                                const int* __restrict__ positions, T* __restrict__ out, int rows, int heads, int rank,
                                int page_size, int num_pages, float scale, int window, uint32_t* err) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(rows) * heads) return;
  const int lane = threadIdx.x & 31;
  const int row = static_cast<int>(item / heads), h = static_cast<int>(item % heads);
  const int req = request_of_row[row];
  if (req < 0) return;                                           // a row of padding
  const int pos = positions[row];
  float qr[kPerLane], acc[kPerLane];
#pragma unroll
  for (int e = 0; e < kPerLane; ++e) {
    const int i = lane + 32 * e;
    qr[e] = i < rank ? to_float<T>(q[item * rank + i]) : 0.0f;
    acc[e] = 0.0f;
  }
  float m = sink != nullptr ? sink[h] : -INFINITY;
  float l = sink != nullptr ? 1.0f : 0.0f;
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = block_table + static_cast<long long>(req) * table_width;
  bool bad = false;
  for (int j = first; j <= pos; ++j) {
    const int pi = j / page_size;
    const int page = pi < table_width ? table[pi] : -1;
    if (page < 0 || page >= num_pages) { bad = true; continue; }
    const T* c = cache + (static_cast<long long>(page) * page_size + (j - pi * page_size)) * rank;
    float cr[kPerLane];
    float s = 0.0f;
#pragma unroll
    for (int e = 0; e < kPerLane; ++e) {
      const int i = lane + 32 * e;
      cr[e] = (e * 32 < rank && i < rank) ? to_float<T>(c[i]) : 0.0f;
      s = fmaf(qr[e], cr[e], s);
    }
    s = warp_sum(s) * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);                          // exp(-inf) = 0 at the first key without a sink
    const float p = expf(s - m_new);
    l = fmaf(l, corr, p);
#pragma unroll
    for (int e = 0; e < kPerLane; ++e) acc[e] = fmaf(acc[e], corr, p * cr[e]);
    m = m_new;
  }
  if (bad && lane == 0) publish_error(err, kRowWithoutPage);
  if (!(l > 0.0f) || !isfinite(l)) {
    if (lane == 0) publish_error(err, kAttentionDenominator);
    l = 1.0f;
  }
  float factor = 1.0f / l;
  if (gate != nullptr) {
    const float z = to_float<T>(gate[static_cast<long long>(row) * ldg + h]);
    factor *= 1.0f / (1.0f + expf(-z));
  }
#pragma unroll
  for (int e = 0; e < kPerLane; ++e) {
    const int i = lane + 32 * e;
    if (i < rank) out[item * rank + i] = from_float<T>(acc[e] * factor);
  }
}


// The same attention for the serving dtype, cut over keys.  Block (row, split of the row's keys, group of 8 heads):
// 8 warps, a head each; a tile of 32 cached latents is brought into shared memory ONCE for the 8 heads.  Scores: a
// lane a key (the folded query is read as a broadcast, the latent row with a padded pitch, conflict-free); weights
// and running sums in 32-bit; the weighted sum of latents: a lane a column.  A split leaves (maximum, sum, weighted
// sum) per head; latent_merge folds the splits in order, starting from the sink, and applies 1 / sum and the gate.
// rank a multiple of 4.
template <typename T, int kPerLane>
__global__ void __launch_bounds__(256)
latent_attention_split_kernel(const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ block_table,
                              int table_width, const int* __restrict__ request_of_row, const int* __restrict__ positions,
                              float* __restrict__ partial, int heads, int rank, int page_size, int num_pages, float scale,
                              int window, int splits, uint32_t* err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ long long src_row[32];
  constexpr int kUnit = 4 / sizeof(T);                           // elements in a 32-bit unit
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x, split = blockIdx.y, h0 = blockIdx.z * 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, h = h0 + warp;
  const int req = request_of_row[row];
  if (req < 0) return;                                           // a row of padding
  float* qs = reinterpret_cast<float*>(smem_raw);                // [8][rank]
  T* tile = reinterpret_cast<T*>(qs + 8 * rank);                 // [32][pitch]
  const int pitch = rank + (sizeof(T) == 2 ? 2 : 1);             // an odd number of 32-bit words
  const int pos = positions[row];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int chunk = (((pos - first + 1) + splits - 1) / splits + 31) / 32 * 32;
  const int k0 = first + split * chunk, k1 = min(pos + 1, k0 + chunk);
  for (int i = tid; i < 8 * rank; i += 256) {
    const int hh = h0 + i / rank;
    qs[i] = hh < heads ? to_float<T>(q[(static_cast<long long>(row) * heads + hh) * rank + i % rank]) : 0.0f;
  }
  float m = -INFINITY, l = 0.0f, acc[kPerLane];
#pragma unroll
  for (int e = 0; e < kPerLane; ++e) acc[e] = 0.0f;
  const int* table = block_table + static_cast<long long>(req) * table_width;
  const int units = rank / kUnit;
  for (int t0 = k0; t0 < k1; t0 += 32) {
    __syncthreads();                                             // the tile before this one has been used
    if (tid < 32) {
      const int key = t0 + tid;
      long long src = -1;
      if (key < k1) {
        const int pi = key / page_size;
        const int page = pi < table_width ? table[pi] : -1;
        if (page < 0 || page >= num_pages) publish_error(err, kRowWithoutPage);
        else src = (static_cast<long long>(page) * page_size + (key - pi * page_size)) * rank;
      }
      src_row[tid] = src;
    }
    __syncthreads();
    for (int i = tid; i < 32 * units; i += 256) {
      const int j = i / units, un = i - j * units;
      const long long src = src_row[j];
      uint32_t word = 0u;
      if (src >= 0) word = *reinterpret_cast<const uint32_t*>(cache + src + un * kUnit);
      *reinterpret_cast<uint32_t*>(tile + j * pitch + un * kUnit) = word;
    }
    __syncthreads();
    if (h < heads) {
      const T* cj = tile + lane * pitch;
      const float* qh = qs + warp * rank;
      float s0 = 0.0f, s1 = 0.0f;
      for (int r = 0; r < rank; r += 4) {
        const float4 qv = *reinterpret_cast<const float4*>(qh + r);
        s0 = fmaf(qv.x, to_float<T>(cj[r + 0]), s0);
        s1 = fmaf(qv.y, to_float<T>(cj[r + 1]), s1);
        s0 = fmaf(qv.z, to_float<T>(cj[r + 2]), s0);
        s1 = fmaf(qv.w, to_float<T>(cj[r + 3]), s1);
      }
      const bool valid = t0 + lane < k1 && src_row[lane] >= 0;
      const float sc = valid ? (s0 + s1) * scale : -INFINITY;
      const float m_new = fmaxf(m, warp_max(sc));
      if (m_new > -INFINITY) {
        const float corr = expf(m - m_new);
        const float p = valid ? expf(sc - m_new) : 0.0f;
        l = fmaf(l, corr, warp_sum(p));
#pragma unroll
        for (int e = 0; e < kPerLane; ++e) acc[e] *= corr;
        for (int j = 0; j < 32; ++j) {
          const float pj = __shfl_sync(0xffffffffu, p, j);
          const T* c = tile + j * pitch;
#pragma unroll
          for (int e = 0; e < kPerLane; ++e) {
            const int i = lane + 32 * e;
            if (e * 32 < rank && i < rank) acc[e] = fmaf(pj, to_float<T>(c[i]), acc[e]);
          }
        }
        m = m_new;
      }
    }
  }
  if (h < heads) {
    float* dst = partial + ((static_cast<long long>(row) * heads + h) * splits + split) * (rank + 2);
    if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
    for (int e = 0; e < kPerLane; ++e) {
      const int i = lane + 32 * e;
      if (i < rank) dst[2 + i] = acc[e];
    }
  }
}


// ---- the tensor-core kernel (bf16, rank 64 / 128 / 192 / 256 / 384 / 512) ------------------------------------------------------
// Block (row, split of the row's keys, group of 16 heads), 8 warps.  The 16 heads of the row are the 16 rows of an
// m16n8k16 MMA: scores S[16 heads x 16 keys] = Q'[16 x rank] . C^T and sums O'[16 x rank] += P[16 x 16] . C[16 x rank],
// so one tile of latents feeds every head's score AND weighted sum.  A tile of 128 latents is staged in shared memory
// (16-byte copies, padded pitch); warp w takes keys 16 w .. 16 w + 15 of every tile and runs a softmax stream of its
// own over them (32-bit maximum, sum and accumulators in registers; P goes from the score accumulators straight into
// the A operand).  Each warp leaves (maximum, sum, weighted sum) per head as one more split for latent_merge.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

constexpr int kMmaTileKeys = 128;

// kRowsPerBlock = 1: the block is one row (blockIdx.x), its 8 warps take the tile's 8 groups of 16 keys.
// kRowsPerBlock = 4: the block is 4 consecutive rows of ONE request (blockIdx.x counts the requests' row tiles, found
// by walking cu_q; blocks beyond the last tile leave), so a tile of latents is fetched once for 4 rows: warp w is row
// w % 4 and takes every second group of 16 keys.  Parts a (row, head): splits * 8 / kRowsPerBlock.
template <int kRank, int kOut, int kRowsPerBlock>
__global__ void __launch_bounds__(256)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                            const int* __restrict__ block_table, int table_width, const int* __restrict__ request_of_row,
                            const int* __restrict__ positions, const int* __restrict__ cu_q, int requests,
                            float* __restrict__ partial, int heads, int page_size, int num_pages, float scale, int window,
                            int splits, uint32_t* err) {
  typedef __nv_bfloat16 bf;
  constexpr int kPitch = kRank + 8;                              // elements; rows 16 bytes apart in the banks
  constexpr int kStreams = 8 / kRowsPerBlock;                    // warps a row, each a stream of its own over keys
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ long long src_row[kMmaTileKeys];
  wait_for_prior_kernels();
  launch_dependents();
  // a latent wider than 256: the block computes every score but only kOut of the sum's columns (the accumulators of
  // all of them would not fit a thread's registers); blockIdx.z counts (group of heads, stretch of columns)
  constexpr int kStretches = kRank / kOut;
  const int split = blockIdx.y, h0 = (blockIdx.z / kStretches) * 16;
  const int cbase = (blockIdx.z % kStretches) * kOut;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  int row0, n_rows, req;
  if (kRowsPerBlock == 1) {
    row0 = blockIdx.x;
    n_rows = 1;
    req = request_of_row[row0];
    if (req < 0) return;                                         // a row of padding
  } else {
    int b = blockIdx.x;
    req = 0;
    for (; req < requests; ++req) {
      const int tiles = (cu_q[req + 1] - cu_q[req] + kRowsPerBlock - 1) / kRowsPerBlock;
      if (b < tiles) break;
      b -= tiles;
    }
    if (req >= requests) return;                                 // beyond the last row tile
    row0 = cu_q[req] + b * kRowsPerBlock;
    n_rows = min(kRowsPerBlock, cu_q[req + 1] - row0);
  }
  bf* Qs = reinterpret_cast<bf*>(smem_raw);                      // [kRowsPerBlock * 16][kPitch]
  bf* tile = Qs + kRowsPerBlock * 16 * kPitch;                   // [128][kPitch]
  // the block's keys: from the first row's first key to the last row's position, cut into ``splits``
  const int pos_last = positions[row0 + n_rows - 1];
  const int first_0 = window > 0 ? max(0, positions[row0] - window + 1) : 0;
  const int chunk = (((pos_last - first_0 + 1) + splits - 1) / splits + kMmaTileKeys - 1) / kMmaTileKeys * kMmaTileKeys;
  const int k0 = first_0 + split * chunk, k1 = min(pos_last + 1, k0 + chunk);
  constexpr int kUnits = kRank / 8;                              // 16-byte units a row
  for (int i = tid; i < kRowsPerBlock * 16 * kUnits; i += 256) {
    const int rr = i / kUnits, un = i - rr * kUnits;
    const int ri = rr / 16, hh = rr % 16;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (ri < n_rows && h0 + hh < heads)
      v = *reinterpret_cast<const uint4*>(q + (static_cast<long long>(row0 + ri) * heads + h0 + hh) * kRank + un * 8);
    *reinterpret_cast<uint4*>(Qs + rr * kPitch + un * 8) = v;
  }
  // this warp's row and its share of a tile's groups of 16 keys
  const int ri = warp % kRowsPerBlock, stream = warp / kRowsPerBlock;
  const bool active = ri < n_rows;
  const int pos = active ? positions[row0 + ri] : -1;
  const int first = (active && window > 0) ? max(0, pos - window + 1) : 0;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
  float O[kOut / 8][4];
#pragma unroll
  for (int n = 0; n < kOut / 8; ++n) { O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.0f; }
  const int* table = block_table + static_cast<long long>(req) * table_width;
  const int mi = lane >> 3, lr = lane & 7;
  for (int t0 = k0; t0 < k1; t0 += kMmaTileKeys) {
    __syncthreads();                                             // the tile before this one has been used
    if (tid < kMmaTileKeys) {
      const int key = t0 + tid;
      long long src = -1;
      if (key < k1) {
        const int pi = key / page_size;
        const int page = pi < table_width ? table[pi] : -1;
        if (page < 0 || page >= num_pages) publish_error(err, kRowWithoutPage);
        else src = (static_cast<long long>(page) * page_size + (key - pi * page_size)) * kRank;
      }
      src_row[tid] = src;
    }
    __syncthreads();
    for (int i = tid; i < kMmaTileKeys * kUnits; i += 256) {
      const int j = i / kUnits, un = i - j * kUnits;
      const long long src = src_row[j];
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (src >= 0) v = *reinterpret_cast<const uint4*>(cache + src + un * 8);
      *reinterpret_cast<uint4*>(tile + j * kPitch + un * 8) = v;
    }
    __syncthreads();
    if (!active) continue;
    for (int kl = stream * 16; kl < kMmaTileKeys; kl += kStreams * 16) {      // this warp's keys within the tile
      if (t0 + kl >= k1 || t0 + kl > pos || t0 + kl + 15 < first) continue;
      float S[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll
      for (int ks = 0; ks < kRank / 16; ++ks) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, Qs + (ri * 16 + lr + (mi & 1) * 8) * kPitch + ks * 16 + (mi >> 1) * 8);
        ldmatrix_x4(b, tile + (kl + lr + (mi >> 1) * 8) * kPitch + ks * 16 + (mi & 1) * 8);
        mma_bf16(S[0], a, b[0], b[1]);
        mma_bf16(S[1], a, b[2], b[3]);
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int kk = kl + nt * 8 + 2 * t4 + (c & 1);
          const int key = t0 + kk;
          const bool valid = key < k1 && key <= pos && key >= first && src_row[kk] >= 0;
          S[nt][c] = valid ? S[nt][c] * scale : -INFINITY;
          if (c < 2) mx0 = fmaxf(mx0, S[nt][c]); else mx1 = fmaxf(mx1, S[nt][c]);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float corr0 = n0 == -INFINITY ? 1.0f : expf(m0 - n0), corr1 = n1 == -INFINITY ? 1.0f : expf(m1 - n1);
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float nn = c < 2 ? n0 : n1;
          const float pv = nn == -INFINITY ? 0.0f : expf(S[nt][c] - nn);
          S[nt][c] = pv;
          if (c < 2) sum0 += pv; else sum1 += pv;
        }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      l0 = fmaf(l0, corr0, sum0);
      l1 = fmaf(l1, corr1, sum1);
      m0 = n0;
      m1 = n1;
      uint32_t pa[4];
      pa[0] = pack_bf16(S[0][0], S[0][1]);
      pa[1] = pack_bf16(S[0][2], S[0][3]);
      pa[2] = pack_bf16(S[1][0], S[1][1]);
      pa[3] = pack_bf16(S[1][2], S[1][3]);
#pragma unroll
      for (int nb = 0; nb < kOut / 16; ++nb) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, tile + (kl + lr + (mi & 1) * 8) * kPitch + cbase + nb * 16 + (mi >> 1) * 8);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float (&o)[4] = O[2 * nb + half];
          o[0] *= corr0; o[1] *= corr0; o[2] *= corr1; o[3] *= corr1;
          mma_bf16(o, pa, b[2 * half], b[2 * half + 1]);
        }
      }
    }
  }
  if (!active) return;
  const int parts = splits * kStreams;
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const int h = h0 + g + hr * 8;
    if (h >= heads) continue;
    float* dst = partial + ((static_cast<long long>(row0 + ri) * heads + h) * parts + split * kStreams + stream) * (kRank + 2);
    if (t4 == 0 && cbase == 0) { dst[0] = hr ? m1 : m0; dst[1] = hr ? l1 : l0; }
#pragma unroll
    for (int n = 0; n < kOut / 8; ++n) {
      dst[2 + cbase + n * 8 + 2 * t4] = O[n][2 * hr];
      dst[2 + cbase + n * 8 + 2 * t4 + 1] = O[n][2 * hr + 1];
    }
  }
}

// One block a (row, head): the parts' maxima give the common maximum (the sink's logit among them), every part its
// factor exp(maximum of the part - common maximum) (first warp, kept in shared memory), then a thread a column adds the
// parts' columns in order, eight loads under way at a time.  At most kMergeParts parts.
constexpr int kMergeParts = 256;

template <typename T>
__global__ void __launch_bounds__(256)
latent_merge_kernel(const float* __restrict__ partial, const T* __restrict__ gate, long long ldg,
                    const float* __restrict__ sink, const int* __restrict__ request_of_row, T* __restrict__ out, int rows,
                    int heads, int rank, int splits, uint32_t* err) {
  __shared__ float factor_of[kMergeParts];
  __shared__ float scale_s;
  wait_for_prior_kernels();
  launch_dependents();
  const long long item = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int row = static_cast<int>(item / heads), h = static_cast<int>(item % heads);
  if (request_of_row[row] < 0) return;
  const float* base = partial + item * splits * (rank + 2);
  if (threadIdx.x < 32) {
    float m_all = sink != nullptr ? sink[h] : -INFINITY;
    for (int s = lane; s < splits; s += 32)
      if (base[s * (rank + 2) + 1] > 0.0f) m_all = fmaxf(m_all, base[s * (rank + 2)]);
    m_all = warp_max(m_all);
    float l = 0.0f;
    for (int s = lane; s < splits; s += 32) {
      const float ls = base[s * (rank + 2) + 1];
      const float f = ls > 0.0f ? expf(base[s * (rank + 2)] - m_all) : 0.0f;
      factor_of[s] = f;
      l = fmaf(ls, f, l);
    }
    l = warp_sum(l);
    if (sink != nullptr) l += expf(sink[h] - m_all);
    if (!(l > 0.0f) || !isfinite(l)) {
      if (lane == 0) publish_error(err, kAttentionDenominator);
      l = 1.0f;
    }
    float scale_out = 1.0f / l;
    if (gate != nullptr) {
      const float z = to_float<T>(gate[static_cast<long long>(row) * ldg + h]);
      scale_out *= 1.0f / (1.0f + expf(-z));
    }
    if (lane == 0) scale_s = scale_out;
  }
  __syncthreads();
  const float scale_out = scale_s;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    float a = 0.0f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) a = fmaf(base[s * (rank + 2) + 2 + i], factor_of[s], a);   // (loads run ahead)
    out[item * rank + i] = from_float<T>(a * scale_out);
  }
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

// raw [rows, ld]: ``rank`` numbers that are normed and, behind them, ``rot`` numbers that are rotated by
// positions[row] * freq[pair] (pairs of neighbours with ``interleaved``, else halves); cache [slots, cache_width] with
// cache_width >= rank + rot (columns of padding behind them are not written).  With q_raw [rows, ldq] the same launch
// norms its first q_rank columns with q_weight (fp32) and the same eps into q_out [rows, q_rank]: the queries' latent.
extern "C" int pih_latent_write(int dtype, const void* raw, long long ld, const void* weight, float eps, void* cache,
                                const void* slot_mapping, int rows, int rank, int page_size, int num_pages,
                                int cache_width, int rot, int interleaved, const void* freq, const void* positions,
                                const void* q_raw, long long ldq, const void* q_weight, void* q_out, int q_rank,
                                void* err, void* stream) {
  if (rows <= 0) return 0;
  if (rot < 0 || (rot & 1) || (rot > 0 && (freq == nullptr || positions == nullptr)) || cache_width < rank + rot)
    return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long cache_rows = static_cast<long long>(page_size) * num_pages;
#define PIH_LW(T)                                                                                                      \
  launch_kernel(latent_write_kernel<T>, dim3(((q_raw != nullptr ? 2 * rows : rows) + 3) / 4), dim3(128), 0, s,         \
                static_cast<const T*>(raw), ld,                                                                        \
                static_cast<const float*>(weight), eps, static_cast<T*>(cache), static_cast<const int*>(slot_mapping), \
                rows, rank, cache_rows, cache_width, rot, interleaved, static_cast<const float*>(freq),                \
                static_cast<const int*>(positions), static_cast<const T*>(q_raw), ldq,                                 \
                static_cast<const float*>(q_weight), static_cast<T*>(q_out), q_rank, static_cast<uint32_t*>(err))
  if (dtype == PIH_F32) PIH_LW(float);
  else if (dtype == PIH_BF16) PIH_LW(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_LW
  PIH_LAUNCH_CHECK();
  return 0;
}

extern "C" int pih_latent_attention_generic(int dtype, const void* q, const void* gate, long long ldg, const void* sink,
                                            const void* cache, const void* block_table, int table_width,
                                            const void* request_of_row, const void* positions, void* out, int rows,
                                            int heads, int rank, int page_size, int num_pages, float scale, int window,
                                            void* err, void* stream) {
  if (rows <= 0) return 0;
  if (rank > 32 * kLatentPerLane) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long items = static_cast<long long>(rows) * heads;
  dim3 grid(static_cast<unsigned>((items + 3) / 4));
#define PIH_LA1(T, NE)                                                                                                 \
  launch_kernel(latent_attention_generic_kernel<T, NE>, grid, dim3(128), 0, s, static_cast<const T*>(q),                   \
                static_cast<const T*>(gate), ldg, static_cast<const float*>(sink), static_cast<const T*>(cache),       \
                static_cast<const int*>(block_table), table_width, static_cast<const int*>(request_of_row),            \
                static_cast<const int*>(positions), static_cast<T*>(out), rows, heads, rank, page_size, num_pages,     \
                scale, window, static_cast<uint32_t*>(err))
#define PIH_LA(T)                                                                                                      \
  do {                                                                                                                 \
    if (rank <= 64) PIH_LA1(T, 2);                                                                                     \
    else if (rank <= 128) PIH_LA1(T, 4);                                                                               \
    else if (rank <= 256) PIH_LA1(T, 8);                                                                               \
    else if (rank <= 512) PIH_LA1(T, 16);                                                                              \
    else if (rank <= 768) PIH_LA1(T, 24);                                                                              \
    else PIH_LA1(T, 32);                                                                                               \
  } while (0)
  if (dtype == PIH_F32) PIH_LA(float);
  else if (dtype == PIH_BF16) PIH_LA(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_LA
#undef PIH_LA1
  PIH_LAUNCH_CHECK();
  return 0;
}

// Splits of a row's keys for a step of ``rows`` rows: enough blocks to fill the GPU, a function of the step's shape only.
extern "C" int pih_latent_attention_splits(int rows, int heads) {
  const int groups = (heads + 7) / 8;
  const int per_row = (2 * 148) / (rows * groups > 0 ? rows * groups : 1);
  return per_row < 1 ? 1 : (per_row > 32 ? 32 : per_row);
}

// partial: fp32 scratch, rows * heads * splits * (rank + 2)
extern "C" int pih_latent_attention_split(int dtype, const void* q, const void* gate, long long ldg, const void* sink,
                                          const void* cache, const void* block_table, int table_width,
                                          const void* request_of_row, const void* positions, void* partial, void* out,
                                          int rows, int heads, int rank, int page_size, int num_pages, float scale,
                                          int window, int splits, void* err, void* stream) {
  if (rows <= 0) return 0;
  if (rank > 32 * kLatentPerLane || rank % 4 || splits < 1 || splits > kMergeParts || rows > 65535 * 32)
    return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int esize = dtype == PIH_F32 ? 4 : 2;
  const size_t smem = 8 * static_cast<size_t>(rank) * 4 + 32 * static_cast<size_t>(rank + (esize == 2 ? 2 : 1)) * esize;
  dim3 grid(rows, splits, (heads + 7) / 8);
  const long long items = static_cast<long long>(rows) * heads;
#define PIH_LS1(T, NE)                                                                                                 \
  do {                                                                                                                 \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(latent_attention_split_kernel<T, NE>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                           static_cast<int>(smem));                                                                    \
    launch_kernel(latent_attention_split_kernel<T, NE>, grid, dim3(256), smem, s, static_cast<const T*>(q),            \
                  static_cast<const T*>(cache), static_cast<const int*>(block_table), table_width,                     \
                  static_cast<const int*>(request_of_row), static_cast<const int*>(positions),                         \
                  static_cast<float*>(partial), heads, rank, page_size, num_pages, scale, window, splits,              \
                  static_cast<uint32_t*>(err));                                                                        \
  } while (0)
#define PIH_LS(T)                                                                                                      \
  do {                                                                                                                 \
    if (rank <= 64) PIH_LS1(T, 2);                                                                                     \
    else if (rank <= 128) PIH_LS1(T, 4);                                                                               \
    else if (rank <= 256) PIH_LS1(T, 8);                                                                               \
    else if (rank <= 512) PIH_LS1(T, 16);                                                                              \
    else if (rank <= 768) PIH_LS1(T, 24);                                                                              \
    else PIH_LS1(T, 32);                                                                                               \
    PIH_LAUNCH_CHECK();                                                                                                \
    launch_kernel(latent_merge_kernel<T>, dim3(static_cast<unsigned>(items)), dim3(rank >= 256 ? 256 : (rank + 31) / 32 * 32), 0, s, \
                  static_cast<const float*>(partial), static_cast<const T*>(gate), ldg, static_cast<const float*>(sink), \
                  static_cast<const int*>(request_of_row), static_cast<T*>(out), rows, heads, rank, splits,            \
                  static_cast<uint32_t*>(err));                                                                        \
  } while (0)
  if (dtype == PIH_F32) PIH_LS(float);
  else if (dtype == PIH_BF16) PIH_LS(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_LS
#undef PIH_LS1
  PIH_LAUNCH_CHECK();
  return 0;
}

// The tensor-core kernel: bf16, rank 64, 128, 192, 256, 384 or 512.  rows_per_block 1 or 4 (4: blocks are row tiles
// of a request, for steps of prompt portions).  partial: fp32 scratch, rows * heads * parts * (rank + 2) with
// parts = splits * 8 / rows_per_block.
extern "C" int pih_latent_attention_mma(const void* q, const void* gate, long long ldg, const void* sink, const void* cache,
                                        const void* block_table, int table_width, const void* request_of_row,
                                        const void* positions, const void* cu_q, int requests, void* partial, void* out,
                                        int rows, int heads, int rank, int page_size, int num_pages, float scale,
                                        int window, int splits, int rows_per_block, void* err, void* stream) {
  if (rows <= 0) return 0;
  if ((rank != 64 && rank != 128 && rank != 192 && rank != 256 && rank != 384 && rank != 512) || splits < 1 ||
      (rows_per_block != 1 && rows_per_block != 4) || splits * 8 / rows_per_block > kMergeParts || rows > 65535 * 32)
    return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = (16 * rows_per_block + kMmaTileKeys) * static_cast<size_t>(rank + 8) * 2;
  const unsigned blocks_x = rows_per_block == 1 ? rows : (rows + 3) / 4 + requests;
  dim3 grid(blocks_x, splits, (heads + 15) / 16 * (rank > 256 ? 2 : 1));
  const long long items = static_cast<long long>(rows) * heads;
#define PIH_LM1(R, C, B)                                                                                               \
  do {                                                                                                                 \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(latent_attention_mma_kernel<R, C, B>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                           static_cast<int>(smem));                                                                    \
    launch_kernel(latent_attention_mma_kernel<R, C, B>, grid, dim3(256), smem, s, static_cast<const bf16*>(q),         \
                  static_cast<const bf16*>(cache), static_cast<const int*>(block_table), table_width,                  \
                  static_cast<const int*>(request_of_row), static_cast<const int*>(positions),                         \
                  static_cast<const int*>(cu_q), requests, static_cast<float*>(partial), heads, page_size, num_pages,  \
                  scale, window, splits, static_cast<uint32_t*>(err));                                                 \
  } while (0)
#define PIH_LM(R, C)                                                                                                   \
  do {                                                                                                                 \
    if (rows_per_block == 1) PIH_LM1(R, C, 1); else PIH_LM1(R, C, 4);                                                  \
  } while (0)
  if (rank == 64) PIH_LM(64, 64);
  else if (rank == 128) PIH_LM(128, 128);
  else if (rank == 192) PIH_LM(192, 192);
  else if (rank == 256) PIH_LM(256, 256);
  else if (rank == 384) PIH_LM(384, 192);
  else PIH_LM(512, 256);
#undef PIH_LM
#undef PIH_LM1
  PIH_LAUNCH_CHECK();
  launch_kernel(latent_merge_kernel<bf16>, dim3(static_cast<unsigned>(items)), dim3(rank >= 256 ? 256 : (rank + 31) / 32 * 32), 0, s,
                static_cast<const float*>(partial), static_cast<const bf16*>(gate), ldg, static_cast<const float*>(sink),
                static_cast<const int*>(request_of_row), static_cast<bf16*>(out), rows, heads, rank,
                splits * 8 / rows_per_block, static_cast<uint32_t*>(err));
  PIH_LAUNCH_CHECK();
  return 0;
}
