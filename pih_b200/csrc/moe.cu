// Mixture of experts: routing and the experts' products over rows grouped by expert.
//
//   moe_route      per row: the ``top`` largest router logits (32-bit), softmax over the chosen ones, and the row's
//                  place among the rows of each chosen expert
//   moe_plan       per expert: where its rows start, and where its row tiles start (one block)
//   moe_scatter    (row, choice) -> a position in expert order, and back
//   moe_gate_up    grouped product: act[pos] = silu(x[row] . Wg_e^T) * (x[row] . Wu_e^T)
//   moe_down       grouped product: y[pos] = act[pos] . Wd_e^T  (32-bit)
//   moe_combine    out[row] = sum_k weight[row][k] * y[pos(row, k)], k ascending
//
// Nothing returns to the host: a grouped product is launched for the most row tiles that the step could need
// (ceil(rows * top / 64) + experts), a block looks up its expert and rows in the plan, and blocks beyond the plan
// leave.  Every output element is accumulated by one thread in ascending k exactly as the single product does, and a
// row's result depends on that row alone: the rows an expert happens to share a tile with change no bit.
#include "common.cuh"

namespace pih {

constexpr int kMoeTile = 64;

// One warp a row.  A logit that is not a number counts as the smallest; ties go to the smaller index.
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int rows, int experts, int top, int* __restrict__ expert_of,
                 float* __restrict__ weight_of, int* __restrict__ rank_of, int* __restrict__ counts,
                 int* __restrict__ pos_of) {
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  constexpr int kPer = 32;                                       // experts <= 1024
  float v[kPer];
  uint32_t taken = 0;
#pragma unroll
  for (int e = 0; e < kPer; ++e) {
    const int i = lane + 32 * e;
    float a = (e * 32 < experts && i < experts) ? logits[static_cast<long long>(row) * experts + i] : -INFINITY;
    v[e] = (a == a) ? a : -INFINITY;
  }
  float first = 0.0f, denom = 0.0f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
#pragma unroll
    for (int e = 0; e < kPer; ++e) {
      const int i = lane + 32 * e;
      if (e * 32 < experts && i < experts && !((taken >> e) & 1u) && (v[e] > best || best_i == 0x7fffffff)) {
        best = v[e];
        best_i = i;
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, d);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, d);
      if (oi != 0x7fffffff && (best_i == 0x7fffffff || ob > best || (ob == best && oi < best_i))) { best = ob; best_i = oi; }
    }
    if ((best_i & 31) == lane) taken |= 1u << (best_i >> 5);
    if (k == 0) first = best;
    const float e_k = (best == -INFINITY) ? (first == -INFINITY ? 1.0f : 0.0f) : expf(best - first);
    denom += e_k;
    if (lane == 0) {
      expert_of[static_cast<long long>(row) * top + k] = best_i;
      weight_of[static_cast<long long>(row) * top + k] = e_k;
      // grouped by expert: the row's place among the expert's rows; not grouped (counts null): a slot stays where it is
      if (counts != nullptr) rank_of[static_cast<long long>(row) * top + k] = atomicAdd(&counts[best_i], 1);
      else pos_of[static_cast<long long>(row) * top + k] = row * top + k;
    }
  }
  __syncwarp();
  if (lane < top) {
    for (int k = lane; k < top; k += 32) weight_of[static_cast<long long>(row) * top + k] /= denom;
  }
}

// Routing by scores over ALL outputs: s = softmax(logits), or with ``scoring`` 1 the sigmoid of each logit by itself;
// the choice goes by s + correction, among the outputs of the
// ``keep`` best of ``groups`` equal groups of neighbours (a group's score: its largest choice score; the others count
// as minus infinity); the ``top`` largest are chosen (ties: the smaller index) and weigh with their s, divided by the
// chosen ones' sum only with ``renormalize``.  One warp a row; ``flags``: [warps][groups] ints of shared memory.
__global__ void __launch_bounds__(128)
moe_route_scored_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ correction, int rows,
                        int experts, int top, int groups, int keep, int renormalize, int scoring, int* __restrict__ expert_of,
                        float* __restrict__ weight_of, int* __restrict__ rank_of, int* __restrict__ counts,
                        int* __restrict__ pos_of) {
  extern __shared__ float route_smem[];
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int kPer = 32;                                       // experts <= 1024
  float sc[kPer], ch[kPer];
  uint32_t taken = 0;
  float mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < kPer; ++e) {
    const int i = lane + 32 * e;
    float a = (e * 32 < experts && i < experts) ? logits[row * ld + i] : -INFINITY;
    sc[e] = (a == a) ? a : -INFINITY;
    mx = fmaxf(mx, sc[e]);
  }
  mx = warp_max(mx);
  float sum = 0.0f;
#pragma unroll
  for (int e = 0; e < kPer; ++e) {
    if (scoring == 1) sc[e] = (e * 32 < experts && sc[e] != -INFINITY) ? 1.0f / (1.0f + expf(-sc[e])) : 0.0f;
    else sc[e] = (e * 32 < experts && sc[e] != -INFINITY) ? expf(sc[e] - mx) : 0.0f;
    sum += sc[e];
  }
  sum = warp_sum(sum);
  const float inv = scoring == 1 ? 1.0f : 1.0f / sum;         // (a sigmoid score stands for itself)
#pragma unroll
  for (int e = 0; e < kPer; ++e) {
    const int i = lane + 32 * e;
    sc[e] *= inv;
    ch[e] = (e * 32 < experts && i < experts) ? sc[e] + (correction != nullptr ? correction[i] : 0.0f) : -INFINITY;
  }
  if (groups > 1) {
    float* score = route_smem + warp * 2 * groups;               // a group's score, then whether it is kept
    int* kept = reinterpret_cast<int*>(score + groups);
    const int size = experts / groups;
    for (int g = 0; g < groups; ++g) {
      float best = -INFINITY;
#pragma unroll
      for (int e = 0; e < kPer; ++e) {
        const int i = lane + 32 * e;
        if (e * 32 < experts && i < experts && i / size == g) best = fmaxf(best, ch[e]);
      }
      best = warp_max(best);
      if (lane == 0) score[g] = best;
    }
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {
      int ahead = 0;
      for (int o = 0; o < groups; ++o) ahead += (score[o] > score[g] || (score[o] == score[g] && o < g)) ? 1 : 0;
      kept[g] = ahead < keep ? 1 : 0;
    }
    __syncwarp();
#pragma unroll
    for (int e = 0; e < kPer; ++e) {
      const int i = lane + 32 * e;
      if (e * 32 < experts && i < experts && !kept[i / size]) ch[e] = -INFINITY;
    }
  }
  float chosen_sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, best_s = 0.0f;
    int best_i = 0x7fffffff;
#pragma unroll
    for (int e = 0; e < kPer; ++e) {
      const int i = lane + 32 * e;
      if (e * 32 < experts && i < experts && !((taken >> e) & 1u) && (ch[e] > best || best_i == 0x7fffffff)) {
        best = ch[e];
        best_s = sc[e];
        best_i = i;
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, d);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, d);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, d);
      if (oi != 0x7fffffff && (best_i == 0x7fffffff || ob > best || (ob == best && oi < best_i))) { best = ob; best_s = os; best_i = oi; }
    }
    if ((best_i & 31) == lane) taken |= 1u << (best_i >> 5);
    chosen_sum += best_s;
    if (lane == 0) {
      expert_of[static_cast<long long>(row) * top + k] = best_i;
      weight_of[static_cast<long long>(row) * top + k] = best_s;
      if (counts != nullptr) rank_of[static_cast<long long>(row) * top + k] = atomicAdd(&counts[best_i], 1);
      else pos_of[static_cast<long long>(row) * top + k] = row * top + k;
    }
  }
  __syncwarp();
  if (renormalize)
    for (int k = lane; k < top; k += 32) weight_of[static_cast<long long>(row) * top + k] /= chosen_sum;
}

// plan: [0 .. experts] first position of an expert's rows; [experts+1 .. 2 experts+1] first tile of an expert.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int experts, int* __restrict__ plan) {
  wait_for_prior_kernels();
  launch_dependents();
  if (threadIdx.x != 0) return;
  int pos = 0, tile = 0;
  for (int e = 0; e < experts; ++e) {
    plan[e] = pos;
    plan[experts + 1 + e] = tile;
    pos += counts[e];
    tile += (counts[e] + kMoeTile - 1) / kMoeTile;
  }
  plan[experts] = pos;
  plan[2 * experts + 1] = tile;
}

__global__ void moe_scatter_kernel(const int* __restrict__ expert_of, const int* __restrict__ rank_of,
                                   const int* __restrict__ plan, int slots, int top, int* __restrict__ pos_of,
                                   int* __restrict__ row_of, int* __restrict__ slot_of) {
  wait_for_prior_kernels();
  launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= slots) return;
  const int pos = plan[expert_of[i]] + rank_of[i];
  pos_of[i] = pos;
  row_of[pos] = i / top;
  slot_of[pos] = i;
}

// The grouped product.  kForm 1: two weight matrices per expert and silu(a) * b in the epilogue; 2: one matrix and the
// square of max(a, 0); 0: one matrix, the product as it is.  A's rows are gathered through ``row_of`` when it is given
// (else row = position); with ``in_weight`` a gathered row is multiplied by the weight of its slot (``slot_of`` by
// position) and rounded to the storage type: the expert reads the weighted row.  Expert e's matrices [N, K] start
// ``e * expert_stride`` elements behind W0 and W1.
template <typename TA, typename TC, int kForm>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const TA* __restrict__ A, long long lda, const int* __restrict__ row_of, const TA* __restrict__ W0,
                   const TA* __restrict__ W1, long long expert_stride, TC* __restrict__ C, long long ldc,
                   const int* __restrict__ plan, int experts, int with_matrices, int N, int K,
                   const float* __restrict__ in_weight, const int* __restrict__ slot_of) {
  constexpr bool kGated = kForm == 1;
  constexpr int BM = kMoeTile, BN = 64, BK = 16, TM = 4, TN = 4;
  wait_for_prior_kernels();
  launch_dependents();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[kGated ? 2 : 1][BK][BN + 4];
  __shared__ int rows_s[BM];
  __shared__ float weight_s[BM];
  __shared__ int info[3];
  const int tid = threadIdx.x;
  if (tid == 0) {
    const int tile = blockIdx.y;
    const int* tiles = plan + experts + 1;
    int e = -1;
    if (tile < tiles[experts]) {
      int lo = 0, hi = experts - 1;                              // the last expert whose first tile is <= tile and that has tiles
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tiles[mid] <= tile) lo = mid; else hi = mid - 1;
      }
      e = lo;
    }
    info[0] = e;
    if (e >= 0) {
      info[1] = plan[e] + (tile - tiles[e]) * BM;                // first position of the tile
      info[2] = min(BM, plan[e + 1] - info[1]);                  // its rows
    }
  }
  __syncthreads();
  const int e = info[0];
  if (e < 0 || e >= with_matrices) return;                      // (an identity expert has no matrices: its rows are the combine's)
  const int p0 = info[1], m_rows = info[2];
  if (tid < BM) {
    rows_s[tid] = tid < m_rows ? (row_of != nullptr ? row_of[p0 + tid] : p0 + tid) : -1;
    weight_s[tid] = (tid < m_rows && in_weight != nullptr) ? in_weight[slot_of[p0 + tid]] : 1.0f;
  }
  __syncthreads();
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int n0 = blockIdx.x * BN;
  const TA* w0 = W0 + e * expert_stride;
  const TA* w1 = kGated ? W1 + e * expert_stride : nullptr;
  float acc[kGated ? 2 : 1][TM][TN];
#pragma unroll
  for (int g = 0; g < (kGated ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[g][i][j] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int el = tid + i * 256;
      const int r = el / BK, c = el % BK;
      const int gk = k0 + c, gn = n0 + r;
      const int src = rows_s[r];
      float a = (src >= 0 && gk < K) ? to_float<TA>(A[static_cast<long long>(src) * lda + gk]) : 0.0f;
      if (in_weight != nullptr) a = round_to<TA>(a * weight_s[r]);
      As[c][r] = a;
      Ws[0][c][r] = (gn < N && gk < K) ? to_float<TA>(w0[static_cast<long long>(gn) * K + gk]) : 0.0f;
      if (kGated) Ws[1][c][r] = (gn < N && gk < K) ? to_float<TA>(w1[static_cast<long long>(gn) * K + gk]) : 0.0f;
    }
    __syncthreads();
    float part[kGated ? 2 : 1][TM][TN];
#pragma unroll
    for (int g = 0; g < (kGated ? 2 : 1); ++g)
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) part[g][i][j] = 0.0f;
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int g = 0; g < (kGated ? 2 : 1); ++g) {
        float w[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j) w[j] = Ws[g][k][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) part[g][i][j] = fmaf(a[i], w[j], part[g][i][j]);
      }
    }
#pragma unroll
    for (int g = 0; g < (kGated ? 2 : 1); ++g)
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[g][i][j] += part[g][i][j];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = ty * TM + i;
    if (m >= m_rows) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float val;
      if (kGated) {
        // the two products are rounded to the storage type before the activation, as separate products would be
        const float a = round_to<TA>(acc[0][i][j]), b = round_to<TA>(acc[kGated ? 1 : 0][i][j]);
        val = (a / (1.0f + expf(-a))) * b;
      } else if (kForm == 2) {
        const float a = fmaxf(round_to<TA>(acc[0][i][j]), 0.0f);
        val = a * a;
      } else {
        val = acc[0][i][j];
      }
      C[static_cast<long long>(p0 + m) * ldc + gn] = from_float<TC>(val);
    }
  }
}


// Few rows (a decode step): every (row, choice) slot on its own, a warp an output column, the expert's weight rows
// read with 16-byte loads, four columns in flight a warp.  x row of slot s: s / row_div.  kForm 1: act[s][n] =
// silu(x . W0_e[n]) * (x . W1_e[n]); 2: act[s][n] = max(x . W0_e[n], 0)^2; 0: out[out_index[s]][n] = x . W0_e[n]
// (32-bit).  With ``in_weight`` the row is multiplied by the slot's weight and rounded to the storage type first.
// K a multiple of 8 (4 in 32-bit).
template <typename T, typename TC, int kForm>
__global__ void __launch_bounds__(256)
moe_gemv_kernel(const T* __restrict__ x, long long ldx, int row_div, const int* __restrict__ expert_of,
                const T* __restrict__ W0, const T* __restrict__ W1, long long expert_stride, TC* __restrict__ out,
                long long ldo, const int* __restrict__ out_index, int with_matrices, int N, int K,
                const float* __restrict__ in_weight) {
  constexpr bool kGated = kForm == 1;
  constexpr int kVec = 16 / sizeof(T), kCols = 4;
  extern __shared__ float xs[];
  wait_for_prior_kernels();
  launch_dependents();
  const int slot = blockIdx.x;
  const int e = expert_of[slot];
  if (e >= with_matrices) return;                               // an identity expert: the combine takes the row itself
  const T* xr = x + static_cast<long long>(slot / row_div) * ldx;
  const float scale_in = in_weight != nullptr ? in_weight[slot] : 1.0f;
  for (int k = threadIdx.x; k < K; k += blockDim.x)
    xs[k] = in_weight != nullptr ? round_to<T>(to_float<T>(xr[k]) * scale_in) : to_float<T>(xr[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = (blockIdx.y * (blockDim.x >> 5) + warp) * kCols;
  if (n0 >= N) return;
  const T* w0 = W0 + e * expert_stride;
  const T* w1 = kGated ? W1 + e * expert_stride : nullptr;
  float a0[kCols], a1[kCols];
#pragma unroll
  for (int c = 0; c < kCols; ++c) a0[c] = a1[c] = 0.0f;
  for (int k = lane * kVec; k < K; k += 32 * kVec) {
    float xv[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) xv[i] = xs[k + i];
#pragma unroll
    for (int c = 0; c < kCols; ++c) {
      const int n = min(n0 + c, N - 1);
      __align__(16) T wv[kVec];
      *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(w0 + static_cast<long long>(n) * K + k);
#pragma unroll
      for (int i = 0; i < kVec; ++i) a0[c] = fmaf(to_float<T>(wv[i]), xv[i], a0[c]);
      if (kGated) {
        *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(w1 + static_cast<long long>(n) * K + k);
#pragma unroll
        for (int i = 0; i < kVec; ++i) a1[c] = fmaf(to_float<T>(wv[i]), xv[i], a1[c]);
      }
    }
  }
  const long long orow = out_index != nullptr ? out_index[slot] : slot;
#pragma unroll
  for (int c = 0; c < kCols; ++c) {
    float g = warp_sum(a0[c]);
    float u = kGated ? warp_sum(a1[c]) : 0.0f;
    if (lane == 0 && n0 + c < N) {
      if (kGated) {
        g = round_to<T>(g);
        u = round_to<T>(u);
        out[orow * ldo + n0 + c] = from_float<TC>((g / (1.0f + expf(-g))) * u);
      } else if (kForm == 2) {
        g = fmaxf(round_to<T>(g), 0.0f);
        out[orow * ldo + n0 + c] = from_float<TC>(g * g);
      } else {
        out[orow * ldo + n0 + c] = from_float<TC>(g);
      }
    }
  }
}

// Few rows, many small matrices (a head's or a diagonal block's): out[t][b][n] = x[t][b] . W[b][n], a warp four output
// columns, the matrix rows read with 16-byte loads.  K a multiple of 8 (bf16).  Two optional steps of the mixers that use
// it for their folds: ``freq`` — the columns rot_offset .. rot_offset + rot of every x[t][b] are rotated by
// positions[t] * freq[pair] on their way into shared memory (32-bit angles, rounded to T like a rotation's own kernel
// would leave them; pairs of neighbours with ``interleaved``, else halves); ``gate`` — the output, rounded, is multiplied
// by sigmoid(gate[t * ldg + b * N + n]).
template <typename T, typename TC>
__global__ void __launch_bounds__(256)
batched_gemv_kernel(const T* __restrict__ x, long long ldx, long long batch_x, const T* __restrict__ W, TC* __restrict__ out,
                    int batches, int N, int K, const float* __restrict__ freq, const int* __restrict__ positions,
                    int rot_offset, int rot, int interleaved, const T* __restrict__ gate, long long ldg) {
  constexpr int kVec = 16 / sizeof(T), kCols = 4;
  extern __shared__ float xs[];
  wait_for_prior_kernels();
  launch_dependents();
  const int t = blockIdx.x / batches, b = blockIdx.x % batches;
  const T* xr = x + t * ldx + b * batch_x;
  if (freq == nullptr) {
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_float<T>(xr[k]);
  } else {
    const float place = static_cast<float>(positions[t]);
    const int half = rot >> 1;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      float v = to_float<T>(xr[k]);
      const int c = k - rot_offset;
      if (c >= 0 && c < rot) {
        int pair, other;
        bool first;
        if (interleaved) { pair = c >> 1; first = (c & 1) == 0; other = first ? k + 1 : k - 1; }
        else { pair = c < half ? c : c - half; first = c < half; other = first ? k + half : k - half; }
        float sn, cs;
        sincosf(place * freq[pair], &sn, &cs);
        const float p = to_float<T>(xr[other]);
        v = round_to<T>(first ? v * cs - p * sn : v * cs + p * sn);
      }
      xs[k] = v;
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = (blockIdx.y * (blockDim.x >> 5) + warp) * kCols;
  if (n0 >= N) return;
  const T* w = W + static_cast<long long>(b) * N * K;
  float acc[kCols];
#pragma unroll
  for (int c = 0; c < kCols; ++c) acc[c] = 0.0f;
  for (int k = lane * kVec; k < K; k += 32 * kVec) {
    float xv[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) xv[i] = xs[k + i];
#pragma unroll
    for (int c = 0; c < kCols; ++c) {
      const int n = min(n0 + c, N - 1);
      __align__(16) T wv[kVec];
      *reinterpret_cast<uint4*>(wv) = *reinterpret_cast<const uint4*>(w + static_cast<long long>(n) * K + k);
#pragma unroll
      for (int i = 0; i < kVec; ++i) acc[c] = fmaf(to_float<T>(wv[i]), xv[i], acc[c]);
    }
  }
#pragma unroll
  for (int c = 0; c < kCols; ++c) {
    float v = warp_sum(acc[c]);
    if (lane == 0 && n0 + c < N) {
      if (gate != nullptr) {
        const float g = to_float<T>(gate[t * ldg + static_cast<long long>(b) * N + n0 + c]);
        v = round_to<TC>(v) * (1.0f / (1.0f + expf(-g)));
      }
      out[(static_cast<long long>(blockIdx.x)) * N + n0 + c] = from_float<TC>(v);
    }
  }
}

// An expert from ``with_matrices`` on is an identity expert: its output is the row of x itself.  ``unit_weights``: the
// weights were applied to what the experts read; the outputs are summed as they are.
template <typename T, typename TY>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ pos_of,
                                   const float* __restrict__ weight_of, T* __restrict__ out, int rows, int hidden, int top,
                                   const int* __restrict__ expert_of, int with_matrices, const T* __restrict__ x,
                                   long long ldx, int unit_weights) {
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < top; ++k) {
      const long long i = static_cast<long long>(row) * top + k;
      const float v = expert_of[i] >= with_matrices ? to_float<T>(x[row * ldx + c])
                                                    : to_float<TY>(y[static_cast<long long>(pos_of[i]) * hidden + c]);
      acc = unit_weights ? acc + v : fmaf(weight_of[i], v, acc);
    }
    out[static_cast<long long>(row) * hidden + c] = from_float<T>(acc);
  }
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

// ints: expert_of[slots] | rank_of[slots] | pos_of[slots] | row_of[slots] | counts[experts] | plan[2 experts + 2] |
// slot_of[slots] (the (row, choice) slot at each position in expert order);
// the caller zeroes counts.  weight_of: fp32 [slots].
extern "C" long long pih_moe_route_words(int rows, int experts, int top) {
  return 5LL * rows * top + experts + 2LL * experts + 2;
}

// grouped 0: only the choice and the weights (for the kernels that take every slot on its own; ints need no zeroing)
extern "C" int pih_moe_route(const void* logits, int rows, int experts, int top, void* ints, void* weight_of, int grouped,
                             void* stream) {
  if (rows <= 0) return 0;
  if (experts < 1 || experts > 1024 || top < 1 || top > experts) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long slots = static_cast<long long>(rows) * top;
  int* expert_of = static_cast<int*>(ints);
  int* rank_of = expert_of + slots;
  int* pos_of = rank_of + slots;
  int* row_of = pos_of + slots;
  int* counts = row_of + slots;
  int* plan = counts + experts;
  launch_kernel(moe_route_kernel, dim3((rows + 3) / 4), dim3(128), 0, s, static_cast<const float*>(logits), rows, experts,
                top, expert_of, static_cast<float*>(weight_of), rank_of, grouped ? counts : static_cast<int*>(nullptr), pos_of);
  PIH_LAUNCH_CHECK();
  if (!grouped) return 0;
  launch_kernel(moe_plan_kernel, dim3(1), dim3(32), 0, s, static_cast<const int*>(counts), experts, plan);
  PIH_LAUNCH_CHECK();
  launch_kernel(moe_scatter_kernel, dim3(static_cast<unsigned>((slots + 255) / 256)), dim3(256), 0, s,
                static_cast<const int*>(expert_of), static_cast<const int*>(rank_of), static_cast<const int*>(plan),
                static_cast<int>(slots), top, pos_of, row_of, plan + 2 * experts + 2);
  PIH_LAUNCH_CHECK();
  return 0;
}

// The same outputs as pih_moe_route from the scored routing (see moe_route_scored_kernel); logits fp32 [rows, ld] of which
// the first ``experts`` columns are the router's outputs; correction fp32 [experts] or null.
extern "C" int pih_moe_route_scored(const void* logits, long long ld, const void* correction, int rows, int experts, int top,
                                    int groups, int keep, int renormalize, int scoring, void* ints, void* weight_of,
                                    int grouped, void* stream) {
  if (rows <= 0) return 0;
  if (experts < 1 || experts > 1024 || top < 1 || top > experts || groups < 1 || groups > 1024 || experts % groups ||
      keep < 1 || keep > groups)
    return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long slots = static_cast<long long>(rows) * top;
  int* expert_of = static_cast<int*>(ints);
  int* rank_of = expert_of + slots;
  int* pos_of = rank_of + slots;
  int* row_of = pos_of + slots;
  int* counts = row_of + slots;
  int* plan = counts + experts;
  launch_kernel(moe_route_scored_kernel, dim3((rows + 3) / 4), dim3(128), 4 * 2 * groups * sizeof(float), s,
                static_cast<const float*>(logits), ld, static_cast<const float*>(correction), rows, experts, top, groups,
                keep, renormalize, scoring, expert_of, static_cast<float*>(weight_of), rank_of,
                grouped ? counts : static_cast<int*>(nullptr), pos_of);
  PIH_LAUNCH_CHECK();
  if (!grouped) return 0;
  launch_kernel(moe_plan_kernel, dim3(1), dim3(32), 0, s, static_cast<const int*>(counts), experts, plan);
  PIH_LAUNCH_CHECK();
  launch_kernel(moe_scatter_kernel, dim3(static_cast<unsigned>((slots + 255) / 256)), dim3(256), 0, s,
                static_cast<const int*>(expert_of), static_cast<const int*>(rank_of), static_cast<const int*>(plan),
                static_cast<int>(slots), top, pos_of, row_of, plan + 2 * experts + 2);
  PIH_LAUNCH_CHECK();
  return 0;
}

// x [rows, lda]; w_gate_up [experts, 2 ff, hidden]: an expert's gate rows, then its up rows; w_down [experts, hidden, ff];
// act [slots, ff] (storage type); y fp32 [slots, hidden]; out [rows, hidden] (storage type).  few_rows: every slot on
// its own (the weight rows streamed with 16-byte loads) instead of the grouped product; needs hidden and ff to be
// multiples of 8 (bf16) or 4 (32-bit) and hidden, ff <= 12288.  ``experts`` counts the router's outputs, of which the
// last ``identity`` have no matrices: their output is the row of x itself.
// ``gated`` 0: an expert is W_down max(W_up x, 0)^2 and w_gate_up is [experts, ff, hidden].  ``weigh_input`` 1: an expert
// reads its row times the slot's weight (rounded to the storage type) and the outputs are summed as they are.
extern "C" int pih_moe_experts(int dtype, const void* x, long long lda, const void* w_gate_up, const void* w_down, void* act,
                               void* y, void* out, const void* ints, const void* weight_of, int rows, int experts, int top,
                               int hidden, int ff, int few_rows, int identity, int gated, int weigh_input, void* stream) {
  if (rows <= 0) return 0;
  if (identity < 0 || identity > experts) return PIH_ERR_BAD_ARGUMENT;
  if (weigh_input && identity > 0) return PIH_ERR_UNSUPPORTED;
  const int with_matrices = experts - identity;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long slots = static_cast<long long>(rows) * top;
  const int* expert_of = static_cast<const int*>(ints);
  const int* pos_of = expert_of + 2 * slots;
  const int* row_of = pos_of + slots;
  const int* plan = row_of + slots + experts;
  const int* slot_of = plan + 2 * experts + 2;
  const float* in_w = weigh_input ? static_cast<const float*>(weight_of) : nullptr;
  const unsigned tiles = static_cast<unsigned>((slots + kMoeTile - 1) / kMoeTile + experts);
  if (tiles > 65535) return PIH_ERR_UNSUPPORTED;
  const long long gu_stride = (gated ? 2LL : 1LL) * ff * hidden, down_stride = static_cast<long long>(hidden) * ff;
  if (few_rows) {
    const int vec = dtype == PIH_F32 ? 4 : 8;
    if (hidden % vec || ff % vec || hidden > 12288 || ff > 12288 || slots > 65535) return PIH_ERR_UNSUPPORTED;
  }
#define PIH_MOE_FIRST(T, FORM)                                                                                         \
  do {                                                                                                                 \
    if (few_rows) {                                                                                                    \
      launch_kernel(moe_gemv_kernel<T, T, FORM>, dim3(static_cast<unsigned>(slots), (ff + 31) / 32), dim3(256),        \
                    hidden * sizeof(float), s, static_cast<const T*>(x), lda, top, expert_of, wgu,                     \
                    wgu + static_cast<long long>(ff) * hidden, gu_stride, static_cast<T*>(act),                        \
                    static_cast<long long>(ff), static_cast<const int*>(nullptr), with_matrices, ff, hidden, in_w);    \
    } else {                                                                                                           \
      launch_kernel(moe_grouped_kernel<T, T, FORM>, dim3((ff + 63) / 64, tiles), dim3(256), 0, s,                      \
                    static_cast<const T*>(x), lda, row_of, wgu, wgu + static_cast<long long>(ff) * hidden, gu_stride,  \
                    static_cast<T*>(act), static_cast<long long>(ff), plan, experts, with_matrices, ff, hidden, in_w,  \
                    slot_of);                                                                                          \
    }                                                                                                                  \
  } while (0)
#define PIH_MOE(T)                                                                                                     \
  do {                                                                                                                 \
    const T* wgu = static_cast<const T*>(w_gate_up);                                                                   \
    if (gated) PIH_MOE_FIRST(T, 1); else PIH_MOE_FIRST(T, 2);                                                          \
    PIH_LAUNCH_CHECK();                                                                                                \
    if (few_rows) {                                                                                                    \
      launch_kernel(moe_gemv_kernel<T, float, 0>, dim3(static_cast<unsigned>(slots), (hidden + 31) / 32),              \
                    dim3(256), ff * sizeof(float), s, static_cast<const T*>(act), static_cast<long long>(ff), 1,       \
                    expert_of, static_cast<const T*>(w_down), static_cast<const T*>(nullptr), down_stride,             \
                    static_cast<float*>(y), static_cast<long long>(hidden), pos_of, with_matrices, hidden, ff,         \
                    static_cast<const float*>(nullptr));                                                               \
    } else {                                                                                                           \
      launch_kernel(moe_grouped_kernel<T, float, 0>, dim3((hidden + 63) / 64, tiles), dim3(256), 0, s,                 \
                    static_cast<const T*>(act), static_cast<long long>(ff), static_cast<const int*>(nullptr),          \
                    static_cast<const T*>(w_down), static_cast<const T*>(nullptr), down_stride,                        \
                    static_cast<float*>(y), static_cast<long long>(hidden), plan, experts, with_matrices, hidden, ff,  \
                    static_cast<const float*>(nullptr), static_cast<const int*>(nullptr));                             \
    }                                                                                                                  \
    PIH_LAUNCH_CHECK();                                                                                                \
    launch_kernel(moe_combine_kernel<T, float>, dim3(rows), dim3(hidden >= 256 ? 256 : 128), 0, s,                     \
                  static_cast<const float*>(y), pos_of, static_cast<const float*>(weight_of), static_cast<T*>(out),    \
                  rows, hidden, top, expert_of, with_matrices, static_cast<const T*>(x), lda, weigh_input);            \
  } while (0)
  if (dtype == PIH_F32) PIH_MOE(float);
  else if (dtype == PIH_BF16) PIH_MOE(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_MOE
#undef PIH_MOE_FIRST
  PIH_LAUNCH_CHECK();
  return 0;
}

// xs[pos] = round(x[row_of[pos]] * weight_of[slot_of[pos]]) for the positions of experts with matrices, in expert order:
// what a library's grouped product reads when the weights multiply the experts' input.  xs [slots, hidden].
namespace pih {
template <typename T>
__global__ void moe_gather_scaled_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ row_of,
                                         const int* __restrict__ slot_of, const float* __restrict__ weight_of,
                                         T* __restrict__ xs, int hidden) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long pos = blockIdx.x;
  const float w = weight_of[slot_of[pos]];
  const T* src = x + static_cast<long long>(row_of[pos]) * ldx;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    xs[pos * hidden + c] = from_float<T>(to_float<T>(src[c]) * w);
}
}  // namespace pih

extern "C" int pih_moe_gather_scaled(int dtype, const void* x, long long ldx, const void* ints, const void* weight_of,
                                     void* xs, int rows, int experts, int top, int hidden, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long slots = static_cast<long long>(rows) * top;
  const int* row_of = static_cast<const int*>(ints) + 3 * slots;
  const int* slot_of = row_of + slots + experts + 2 * experts + 2;
  if (dtype == PIH_BF16)
    launch_kernel(moe_gather_scaled_kernel<bf16>, dim3(static_cast<unsigned>(slots)), dim3(hidden >= 1024 ? 256 : 128), 0, s,
                  static_cast<const bf16*>(x), ldx, row_of, slot_of, static_cast<const float*>(weight_of),
                  static_cast<bf16*>(xs), hidden);
  else if (dtype == PIH_F32)
    launch_kernel(moe_gather_scaled_kernel<float>, dim3(static_cast<unsigned>(slots)), dim3(hidden >= 1024 ? 256 : 128), 0, s,
                  static_cast<const float*>(x), ldx, row_of, slot_of, static_cast<const float*>(weight_of),
                  static_cast<float*>(xs), hidden);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}

// out[row] = sum_k weight_of[row][k] * y[pos_of[row][k]] for y in bf16 (the output of a library's grouped product)
// (x [rows, ldx] and with_matrices: see moe_combine_kernel)
extern "C" int pih_moe_combine_bf16(const void* y, const void* ints, const void* weight_of, void* out, int rows, int top,
                                    int hidden, int with_matrices, const void* x, long long ldx, int unit_weights,
                                    void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int* expert_of = static_cast<const int*>(ints);
  const int* pos_of = expert_of + 2LL * rows * top;
  launch_kernel(moe_combine_kernel<bf16, bf16>, dim3(rows), dim3(hidden >= 256 ? 256 : 128), 0, s,
                static_cast<const bf16*>(y), pos_of, static_cast<const float*>(weight_of), static_cast<bf16*>(out), rows,
                hidden, top, expert_of, with_matrices, static_cast<const bf16*>(x), ldx, unit_weights);
  PIH_LAUNCH_CHECK();
  return 0;
}

// out[t][b] = x[t][b] . W[b]^T for few rows t in bf16: x element (t, b, k) at t * ldx + b * batch_x + k, W [batches, N, K],
// out [rows, batches, N] contiguous, bf16 or fp32.  freq fp32 [rot / 2] with positions int32 [rows]: the columns
// rot_offset .. rot_offset + rot of every x[t][b] are rotated first.  gate bf16 [rows, ldg] (column b * N + n): the
// rounded output times its sigmoid.  Both nullable.
extern "C" int pih_batched_gemv(int out_dtype, const void* x, long long ldx, long long batch_x, const void* W, void* out,
                                int rows, int batches, int N, int K, const void* freq, const void* positions,
                                int rot_offset, int rot, int interleaved, const void* gate, long long ldg, void* stream) {
  if (rows <= 0 || batches <= 0 || N <= 0) return 0;
  if (K % 8 || K > 12288 || static_cast<long long>(rows) * batches > 65535 * 16) return PIH_ERR_UNSUPPORTED;
  if (freq != nullptr && (positions == nullptr || rot < 0 || (rot & 1) || rot_offset < 0 || rot_offset + rot > K))
    return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(rows * batches, (N + 31) / 32);
  if (out_dtype == PIH_BF16)
    launch_kernel(batched_gemv_kernel<bf16, bf16>, grid, dim3(256), K * sizeof(float), s, static_cast<const bf16*>(x), ldx,
                  batch_x, static_cast<const bf16*>(W), static_cast<bf16*>(out), batches, N, K,
                  static_cast<const float*>(freq), static_cast<const int*>(positions), rot_offset, rot, interleaved,
                  static_cast<const bf16*>(gate), ldg);
  else if (out_dtype == PIH_F32)
    launch_kernel(batched_gemv_kernel<bf16, float>, grid, dim3(256), K * sizeof(float), s, static_cast<const bf16*>(x), ldx,
                  batch_x, static_cast<const bf16*>(W), static_cast<float*>(out), batches, N, K,
                  static_cast<const float*>(freq), static_cast<const int*>(positions), rot_offset, rot, interleaved,
                  static_cast<const bf16*>(gate), ldg);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}
