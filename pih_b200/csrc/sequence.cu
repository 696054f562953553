// Kernels of mixers that carry a state from token to token, and of a residual stream kept in 32-bit.
//
//   embedding_stream      table rows (bf16 or fp32) -> a 32-bit stream
//   rmsnorm_stream        h (fp32) += delta; out = h / sqrt(mean(h^2) + eps) * w, w a vector or ONE number
//   causal_conv           short causal convolution per channel over each request's rows, the last taps-1 inputs
//                         carried in the request's state slot
//   delta_prepare         unit-norm q and k per head, decay and write strength per head (32-bit)
//   delta_recurrence      gated delta rule: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q
//   gated_rmsnorm         per-head RMS norm of the read-out, times a weight, times silu(gate)
//   rglru_gates, _chain   real-gated linear recurrent unit: S <- a S + sqrt(1 - a^2) (i u), out = S * gelu(y)
//
// A step's rows are packed: request r owns rows cu_q[r] .. cu_q[r+1]-1 in the order of their positions, and
// state_slots[r] is its slot in the state tensor (fp32, ``state_stride`` numbers a slot).  Kernels that carry state
// are driven by requests, so rows of padding (no request) are never touched and requests of padding (no rows, slot -1)
// do nothing.  Everything that enters a recurrence is 32-bit: states, decays, gates, unit norms; only the inputs that
// come from projections and convolutions have the storage type T.  A request's result depends on its own rows and
// state alone, in an order of operations fixed by the row: cutting a prompt or batching it changes no bit.
#include "common.cuh"

namespace pih {

constexpr int kMaxTaps = 16;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void embedding_stream_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                        int hidden, int vocab, uint32_t* err) {
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x;
  int id = ids[row];
  const bool bad = id < 0 || id >= vocab;
  if (bad) {
    if (threadIdx.x == 0) publish_error(err, kTokenOutOfVocabulary);
    id = 0;
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    out[static_cast<long long>(row) * hidden + c] = bad ? 0.0f : to_float<T>(table[static_cast<long long>(id) * hidden + c]);
}

// One block a row.  Without ``rows``: h[row] += delta[row] is stored back and normed.  With ``rows`` (a gather of the
// rows whose logits are wanted) nothing is stored: the sum is formed for the norm alone.
template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_stream_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ weight, int weight_len,
                      TO* __restrict__ out, const int* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[33];
  wait_for_prior_kernels();
  launch_dependents();
  const int row = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  float* hr = h + static_cast<long long>(row) * width;
  const TD* dr = delta != nullptr ? delta + static_cast<long long>(row) * width : nullptr;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = hr[c];
    if (dr != nullptr) {
      v += to_float<TD>(dr[c]);
      if (rows == nullptr) hr[c] = v;
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  TO* o = out + static_cast<long long>(blockIdx.x) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = hr[c];
    if (dr != nullptr && rows != nullptr) v += to_float<TD>(dr[c]);
    o[c] = from_float<TO>(v * scale * (weight_len == 1 ? weight[0] : weight[c]));
  }
}

// Block (32 channels, 8 token lanes) computes 128 rows of a request for 32 channels; blockIdx.z counts the stretches of
// 128 rows (launched for the step's row count; stretches beyond a request's rows leave).
// in(s) = x[s] + in_bias for s >= 0, the history for -(taps-1) <= s < 0 (zeros at the start of a sequence).
// out[t] = act( sum_j w[c][j] in(t - (taps-1) + j) + out_bias ).  The history is only read here; causal_conv_history
// replaces it afterwards.
constexpr int kConvRows = 128;

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w, const float* __restrict__ in_bias,
                   const float* __restrict__ out_bias, T* __restrict__ out, long long ldo, int channels, int taps,
                   int activation, const float* __restrict__ state, long long state_stride, long long state_offset,
                   const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
  wait_for_prior_kernels();
  launch_dependents();
  const int r = blockIdx.x;
  const int c = blockIdx.y * 32 + threadIdx.x;
  const int lo = cu_q[r], n = cu_q[r + 1] - lo;
  const int slot = state_slots[r];
  const int t_first = blockIdx.z * kConvRows;
  if (n <= t_first || slot < 0 || c >= channels) return;
  const int hist_n = taps - 1;
  const float* st = state + slot * state_stride + state_offset;       // [taps-1][channels]
  float wr[kMaxTaps];
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j) wr[j] = j < taps ? to_float<T>(w[static_cast<long long>(c) * taps + j]) : 0.0f;
  const float ib = in_bias != nullptr ? in_bias[c] : 0.0f;
  const float ob = out_bias != nullptr ? out_bias[c] : 0.0f;
  // a token lane takes a run of consecutive rows and keeps the last taps inputs in registers: every input is read once
  const int per = kConvRows / static_cast<int>(blockDim.y);
  const int t0 = t_first + static_cast<int>(threadIdx.y) * per, t1 = min(n, t0 + per);
  if (t0 >= t1) return;
  auto input = [&](int s) {
    return s >= 0 ? to_float<T>(x[static_cast<long long>(lo + s) * ldx + c]) + ib
                  : st[static_cast<long long>(hist_n + s) * channels + c];
  };
  float held[kMaxTaps];                                       // held[j] = in(t - hist_n + j), j < taps
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j) held[j] = (j + 1 < taps) ? input(t0 - hist_n + j) : 0.0f;
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const float newest = input(t);
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
      if (j < taps) {
        const float v = j + 1 == taps ? newest : held[j];
        acc = fmaf(wr[j], v, acc);
      }
    }
#pragma unroll
    for (int j = 0; j + 1 < kMaxTaps; ++j) held[j] = j + 2 == taps ? newest : held[j + 1];
    acc += ob;
    if (activation == 1) acc = acc / (1.0f + expf(-acc));
    out[static_cast<long long>(lo + t) * ldo + c] = from_float<T>(acc);
  }
}

// Thread a (request, channel): the history becomes the last taps-1 inputs of [old history, the step's rows].
template <typename T>
__global__ void __launch_bounds__(128)
causal_conv_history_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ in_bias, int channels, int taps,
                           float* __restrict__ state, long long state_stride, long long state_offset,
                           const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
  wait_for_prior_kernels();
  launch_dependents();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int lo = cu_q[r], n = cu_q[r + 1] - lo;
  const int slot = state_slots[r];
  if (n <= 0 || slot < 0 || c >= channels) return;
  const int hist_n = taps - 1;
  float* st = state + slot * state_stride + state_offset;
  const float ib = in_bias != nullptr ? in_bias[c] : 0.0f;
  float keep[kMaxTaps];
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j) {
    keep[j] = 0.0f;
    if (j < hist_n) {
      const int s = n - hist_n + j;
      keep[j] = s >= 0 ? to_float<T>(x[static_cast<long long>(lo + s) * ldx + c]) + ib
                       : st[static_cast<long long>(hist_n + s) * channels + c];
    }
  }
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j)
    if (j < hist_n) st[static_cast<long long>(j) * channels + c] = keep[j];
}

// One block a row.  qk: [rows, ld] with q heads at column 0 and k heads at column kv_heads*dim (after convolution and
// activation); ba: [rows, ldb] with the write-strength logits at column 0 and the decay logits at column ``heads``.
// qn, kn: fp32 [rows, kv_heads, dim]; decay (as g - 1), beta: fp32 [rows, heads].
template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const T* __restrict__ qk, long long ld, const T* __restrict__ ba, long long ldb,
                     const float* __restrict__ decay_log, const float* __restrict__ decay_bias, float* __restrict__ qn,
                     float* __restrict__ kn, float* __restrict__ decay, float* __restrict__ beta, int heads, int kv_heads,
                     int dim, float unit_eps, float q_scale) {
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int v = warp; v < 2 * kv_heads; v += warps) {             // vector v: q head v, or k head v - kv_heads
    const T* src = qk + static_cast<long long>(row) * ld + static_cast<long long>(v) * dim;
    float ss = 0.0f;
    for (int i = lane; i < dim; i += 32) { const float a = to_float<T>(src[i]); ss = fmaf(a, a, ss); }
    ss = warp_sum(ss);
    const float scale = (1.0f / sqrtf(ss + unit_eps)) * (v < kv_heads ? q_scale : 1.0f);
    float* dst = (v < kv_heads ? qn : kn) + (static_cast<long long>(row) * kv_heads + (v < kv_heads ? v : v - kv_heads)) * dim;
    for (int i = lane; i < dim; i += 32) dst[i] = to_float<T>(src[i]) * scale;
  }
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    const float b = to_float<T>(ba[static_cast<long long>(row) * ldb + h]);
    const float a = to_float<T>(ba[static_cast<long long>(row) * ldb + heads + h]);
    beta[static_cast<long long>(row) * heads + h] = sigmoid_f(b);
    // g - 1 rather than g: a decay next to 1 keeps its distance from 1 to full precision (see rglru_scan_kernel)
    decay[static_cast<long long>(row) * heads + h] = expm1f(-expf(decay_log[h]) * softplus_f(a + decay_bias[h]));
  }
}

// Block (request, head, slice of value columns); thread j owns column v0 + j of S (all ``dim`` rows, in shared memory:
// S[i][j], conflict-free).  The next token's k and q are fetched into registers while this token is computed.
template <typename T>
__global__ void delta_recurrence_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const T* __restrict__ v,
                                        long long ldv, const float* __restrict__ decay, const float* __restrict__ beta,
                                        float* __restrict__ out, float* __restrict__ state, long long state_stride,
                                        const int* __restrict__ cu_q, const int* __restrict__ state_slots, int heads,
                                        int kv_heads, int dim, int vdim) {
  extern __shared__ float smem[];
  wait_for_prior_kernels();
  launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y;
  const int cols = blockDim.x;
  const int j = threadIdx.x, col = blockIdx.z * cols + j;
  const int lo = cu_q[r], hi = cu_q[r + 1];
  const int slot = state_slots[r];
  if (hi <= lo || slot < 0) return;
  const int kh = h / (heads / kv_heads);
  float* S = smem;                          // [dim][cols]
  float* kq = smem + dim * cols;            // [2 buffers][k: dim | q: dim]
  const bool live = col < vdim;
  float* Sg = state + slot * state_stride + (static_cast<long long>(h) * dim) * vdim;
  for (int i = 0; i < dim; ++i) S[i * cols + j] = live ? Sg[static_cast<long long>(i) * vdim + col] : 0.0f;
  const int per = (2 * dim + cols - 1) / cols;                   // numbers of k|q a thread fetches
  auto fetch = [&](int t, int e) -> float {
    const int idx = j + e * cols;
    if (idx >= 2 * dim) return 0.0f;
    const float* src = idx < dim ? kn : qn;
    return src[(static_cast<long long>(t) * kv_heads + kh) * dim + (idx < dim ? idx : idx - dim)];
  };
  constexpr int kMaxPer = 16;               // dim <= 8 * cols
  float nxt[kMaxPer];
#pragma unroll
  for (int e = 0; e < kMaxPer; ++e) nxt[e] = e < per ? fetch(lo, e) : 0.0f;
  for (int t = lo; t < hi; ++t) {
    float* cur = kq + (t & 1) * 2 * dim;
#pragma unroll
    for (int e = 0; e < kMaxPer; ++e)
      if (e < per && j + e * cols < 2 * dim) cur[j + e * cols] = nxt[e];
    __syncthreads();
    if (t + 1 < hi) {
#pragma unroll
      for (int e = 0; e < kMaxPer; ++e) nxt[e] = e < per ? fetch(t + 1, e) : 0.0f;
    }
    const float gm1 = decay[static_cast<long long>(t) * heads + h];        // g - 1; g x is formed as x + (g - 1) x
    const float b = beta[static_cast<long long>(t) * heads + h];
    const float vj = live ? to_float<T>(v[static_cast<long long>(t) * ldv + static_cast<long long>(h) * vdim + col]) : 0.0f;
    const float* k = cur;
    const float* q = cur + dim;
    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    int i = 0;
    for (; i + 4 <= dim; i += 4) {
      a0 = fmaf(S[(i + 0) * cols + j], k[i + 0], a0);
      a1 = fmaf(S[(i + 1) * cols + j], k[i + 1], a1);
      a2 = fmaf(S[(i + 2) * cols + j], k[i + 2], a2);
      a3 = fmaf(S[(i + 3) * cols + j], k[i + 3], a3);
    }
    for (; i < dim; ++i) a0 = fmaf(S[i * cols + j], k[i], a0);
    const float dot = (a0 + a1) + (a2 + a3);
    const float u = b * (vj - fmaf(gm1, dot, dot));
    float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
    i = 0;
    for (; i + 4 <= dim; i += 4) {
      const float s0 = fmaf(k[i + 0], u, fmaf(gm1, S[(i + 0) * cols + j], S[(i + 0) * cols + j]));
      const float s1 = fmaf(k[i + 1], u, fmaf(gm1, S[(i + 1) * cols + j], S[(i + 1) * cols + j]));
      const float s2 = fmaf(k[i + 2], u, fmaf(gm1, S[(i + 2) * cols + j], S[(i + 2) * cols + j]));
      const float s3 = fmaf(k[i + 3], u, fmaf(gm1, S[(i + 3) * cols + j], S[(i + 3) * cols + j]));
      S[(i + 0) * cols + j] = s0; S[(i + 1) * cols + j] = s1; S[(i + 2) * cols + j] = s2; S[(i + 3) * cols + j] = s3;
      o0 = fmaf(s0, q[i + 0], o0); o1 = fmaf(s1, q[i + 1], o1); o2 = fmaf(s2, q[i + 2], o2); o3 = fmaf(s3, q[i + 3], o3);
    }
    for (; i < dim; ++i) {
      const float s0 = fmaf(k[i], u, fmaf(gm1, S[i * cols + j], S[i * cols + j]));
      S[i * cols + j] = s0;
      o0 = fmaf(s0, q[i], o0);
    }
    if (live) out[(static_cast<long long>(t) * heads + h) * vdim + col] = (o0 + o1) + (o2 + o3);
  }
  if (live)
    for (int i = 0; i < dim; ++i) Sg[static_cast<long long>(i) * vdim + col] = S[i * cols + j];
}

// The same recurrence with S in registers, for the key sizes that have an instance.  Block (request, head, 32 value
// columns); a column of S is held by 8 threads (4 for small keys), thread (column c = tid / parts, part p = tid % parts)
// the rows p * kDim / parts ..., so the parts of a column sit in neighbouring lanes and meet through shuffles.  What the recurrence reads of a
// token (k, q, the block's 32 values, decay, write strength) is staged in shared memory a chunk of tokens at a time,
// two buffers: the next chunk's numbers are copied asynchronously while this chunk is computed, so no load from
// memory and only one barrier a chunk lie on the chain from token to token.  The order of the
// additions is fixed by the kernel, not by the step's make-up or by where a chunk begins.
__device__ __forceinline__ void async_copy_16(void* smem_dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(src));
}
__device__ __forceinline__ void async_copy_4(void* smem_dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(src));
}
__device__ __forceinline__ void async_copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void async_copies_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <typename T, int kDim>
__global__ void __launch_bounds__(kDim >= 64 ? 256 : 128)
delta_recurrence_reg_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const T* __restrict__ v,
                            long long ldv, const float* __restrict__ decay, const float* __restrict__ beta,
                            float* __restrict__ out, float* __restrict__ state, long long state_stride,
                            const int* __restrict__ cu_q, const int* __restrict__ state_slots, int heads, int kv_heads,
                            int vdim) {
  constexpr int kParts = kDim >= 64 ? 8 : 4;              // threads a column of S
  constexpr int kThreads = 32 * kParts;
  constexpr int kRows = kDim / kParts;                    // rows of S a thread holds
  constexpr int kSeg = kRows + 4;                         // a part's stretch of k (or q) in the staging buffer: the parts'
                                                          // 16-byte reads fall into different banks
  constexpr int kChunk = kDim <= 128 ? 16 : 8;            // tokens staged at a time (even)
  constexpr int kVWords = 32 * sizeof(T) / 4;             // the block's 32 values of a token, in 32-bit words
  constexpr int kTok = 2 * kParts * kSeg + 4 + kVWords;   // words staged a token: k | q | decay - 1, write strength, pad | values
  constexpr int kCopies = 2 * (kDim / 4) + 2 + kVWords;   // asynchronous copies a token
  extern __shared__ __align__(16) float stage[];          // [2][kChunk][kTok]
  wait_for_prior_kernels();
  launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, part = tid % kParts, cl = tid / kParts, col0 = blockIdx.z * 32, col = col0 + cl;
  const int lo = cu_q[r], hi = cu_q[r + 1];
  const int slot = state_slots[r];
  if (hi <= lo || slot < 0) return;
  const int kh = h / (heads / kv_heads);
  const bool live = col < vdim;
  float* Sg = state + slot * state_stride + (static_cast<long long>(h) * kDim + part * kRows) * vdim;
  float S[kRows];
#pragma unroll
  for (int i = 0; i < kRows; ++i) S[i] = live ? Sg[static_cast<long long>(i) * vdim + col] : 0.0f;
  // the copies of the chunk that starts at token t0, into buffer b: straight from memory into shared memory, so that
  // they are under way while the chunk before is computed
  auto issue = [&](int t0, int b) {
    const int n_tok = min(kChunk, hi - t0);
    for (int i = tid; i < n_tok * kCopies; i += kThreads) {
      const int tok = i / kCopies, c = i - tok * kCopies;
      const int t = t0 + tok;
      float* dst = stage + (b * kChunk + tok) * kTok;
      if (c < 2 * (kDim / 4)) {
        const bool is_q = c >= kDim / 4;
        const int e = (is_q ? c - kDim / 4 : c) * 4;             // element of k (or q)
        const float* src = (is_q ? qn : kn) + (static_cast<long long>(t) * kv_heads + kh) * kDim + e;
        async_copy_16(dst + (is_q ? kParts * kSeg : 0) + (e / kRows) * kSeg + e % kRows, src);
      } else if (c < 2 * (kDim / 4) + 2) {
        const int which = c - 2 * (kDim / 4);
        async_copy_4(dst + 2 * kParts * kSeg + which, (which ? beta : decay) + static_cast<long long>(t) * heads + h);
      } else {
        const int w = c - 2 * (kDim / 4) - 2;                    // word w holds 4 / sizeof(T) values
        const int first_col = col0 + w * (4 / static_cast<int>(sizeof(T)));
        if (first_col < vdim)
          async_copy_4(dst + 2 * kParts * kSeg + 4 + w,
                       v + static_cast<long long>(t) * ldv + static_cast<long long>(h) * vdim + first_col);
      }
    }
    async_copies_commit();
  };
  // a token's numbers from the staging buffer into registers, one token ahead of the arithmetic
  struct Tok { float k[kRows], q[kRows], gm1, b, v; };
  auto load = [&](Tok& x, const float* cur) {
#pragma unroll
    for (int i = 0; i < kRows; i += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(cur + part * kSeg + i);
      const float4 q4 = *reinterpret_cast<const float4*>(cur + kParts * kSeg + part * kSeg + i);
      x.k[i] = k4.x; x.k[i + 1] = k4.y; x.k[i + 2] = k4.z; x.k[i + 3] = k4.w;
      x.q[i] = q4.x; x.q[i + 1] = q4.y; x.q[i + 2] = q4.z; x.q[i + 3] = q4.w;
    }
    x.gm1 = cur[2 * kParts * kSeg];
    x.b = cur[2 * kParts * kSeg + 1];
    x.v = to_float<T>(reinterpret_cast<const T*>(cur + 2 * kParts * kSeg + 4)[cl]);
  };
  auto reduce = [&](float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    if (kParts == 8) x += __shfl_xor_sync(0xffffffffu, x, 4);
    return x;
  };
  auto compute = [&](const Tok& x, int t) {
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int i = 0; i < kRows; i += 2) {
      a0 = fmaf(S[i], x.k[i], a0);
      a1 = fmaf(S[i + 1], x.k[i + 1], a1);
    }
    const float dot = reduce(a0 + a1);
    const float u = x.b * (x.v - fmaf(x.gm1, dot, dot));
    float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
    for (int i = 0; i < kRows; i += 2) {
      S[i] = fmaf(x.k[i], u, fmaf(x.gm1, S[i], S[i]));
      S[i + 1] = fmaf(x.k[i + 1], u, fmaf(x.gm1, S[i + 1], S[i + 1]));
      o0 = fmaf(S[i], x.q[i], o0);
      o1 = fmaf(S[i + 1], x.q[i + 1], o1);
    }
    const float o = reduce(o0 + o1);
    if (live && part == 0) out[(static_cast<long long>(t) * heads + h) * vdim + col] = o;
  };
  issue(lo, 0);
  async_copies_wait();
  __syncthreads();
  int buf = 0;
  for (int t0 = lo; t0 < hi; t0 += kChunk) {
    if (t0 + kChunk < hi) issue(t0 + kChunk, buf ^ 1);
    const int n_tok = min(kChunk, hi - t0);
    const float* base = stage + buf * kChunk * kTok;
    Tok x0, x1;
    load(x0, base);
    for (int tok = 0; tok < n_tok; tok += 2) {
      if (tok + 1 < n_tok) load(x1, base + (tok + 1) * kTok);
      compute(x0, t0 + tok);
      if (tok + 1 < n_tok) {
        if (tok + 2 < n_tok) load(x0, base + (tok + 2) * kTok);
        compute(x1, t0 + tok + 1);
      }
    }
    async_copies_wait();
    __syncthreads();
    buf ^= 1;
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < kRows; ++i) Sg[static_cast<long long>(i) * vdim + col] = S[i];
  }
}

// One warp a (row, head): o fp32 [rows, heads, vdim]; gate [rows, ldg] with head h at column h * vdim.
template <typename T>
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long ldg, const float* __restrict__ weight,
                     T* __restrict__ out, long long rows_heads, int heads, int vdim, float eps) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= rows_heads) return;
  const int lane = threadIdx.x & 31;
  const long long row = item / heads;
  const int h = static_cast<int>(item % heads);
  const float* src = o + item * vdim;
  float ss = 0.0f;
  for (int i = lane; i < vdim; i += 32) ss = fmaf(src[i], src[i], ss);
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / static_cast<float>(vdim) + eps);
  const T* g = gate + row * ldg + static_cast<long long>(h) * vdim;
  T* dst = out + item * vdim;
  for (int i = lane; i < vdim; i += 32) {
    const float z = to_float<T>(g[i]);
    dst[i] = from_float<T>(src[i] * scale * weight[i] * (z / (1.0f + expf(-z))));
  }
}

// The unit in two kernels.  rglru_gates (a thread a (row, channel), every row at once): from the gate logits
// (gates: fp32 [rows, blocks, 2 * bw]: block b's decay-gate logits, then its input-gate logits, without their biases),
// the convolution's output u and the other branch y_pre [rows, ldy] before its bias and GELU, the three numbers that
// the recurrence needs of a token: coef[row][c] = (a - 1, sqrt(1 - a^2) * i * u, gelu(y), 0).  rglru_chain (a thread a
// (request, channel)): S <- S + (a - 1) S + b, out = S * y over the request's rows in order, eight tokens' numbers in
// flight ahead of the chain (sixteen tokens fetched while sixteen are computed).
template <typename T>
__global__ void __launch_bounds__(256)
rglru_gates_kernel(const T* __restrict__ u, long long ldu, const float* __restrict__ gates, const T* __restrict__ y_pre,
                   long long ldy, const float* __restrict__ y_bias, const float* __restrict__ r_bias,
                   const float* __restrict__ i_bias, const float* __restrict__ lam, float decay_scale,
                   float4* __restrict__ coef, int rows, int width, int blocks) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(rows) * width) return;
  const int t = static_cast<int>(idx / width), c = static_cast<int>(idx % width);
  const int bw = width / blocks, b = c / bw, o = c % bw;
  const float* g = gates + (static_cast<long long>(t) * blocks + b) * (2 * bw);
  const float rg = sigmoid_f(g[o] + r_bias[c]);
  const float ig = sigmoid_f(g[bw + o] + i_bias[c]);
  const float log_a = -(decay_scale * softplus_f(lam[c])) * rg;
  // a = exp(log_a) lies next to 1 for a channel that remembers long, where 32-bit numbers are 6e-8 apart: a rounded
  // there would be off by a few percent of 1 - a, and a thousand steps would multiply that up.  So a - 1 and
  // 1 - a^2 come from expm1, and a S is formed as S + (a - 1) S.
  const float am1 = expm1f(log_a);
  const float mult = sqrtf(-expm1f(2.0f * log_a));
  const float y = gelu_tanh_f(to_float<T>(y_pre[static_cast<long long>(t) * ldy + c]) + y_bias[c]);
  coef[idx] = make_float4(am1, mult, ig * to_float<T>(u[static_cast<long long>(t) * ldu + c]), y);
}

template <typename T>
__global__ void __launch_bounds__(128)
rglru_chain_kernel(const float4* __restrict__ coef, T* __restrict__ out, long long ldo, float* __restrict__ state,
                   long long state_stride, const int* __restrict__ cu_q, const int* __restrict__ state_slots, int width) {
  wait_for_prior_kernels();
  launch_dependents();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int lo = cu_q[r], hi = cu_q[r + 1];
  const int slot = state_slots[r];
  if (hi <= lo || slot < 0 || c >= width) return;
  float S = state[slot * state_stride + c];
  constexpr int kAhead = 16;
  float4 cur[kAhead], nxt[kAhead];
  auto fetch = [&](float4 (&f)[kAhead], int t0) {
#pragma unroll
    for (int i = 0; i < kAhead; ++i)
      f[i] = t0 + i < hi ? coef[static_cast<long long>(t0 + i) * width + c] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  };
  auto chain = [&](const float4 (&f)[kAhead], int t0) {
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      if (t0 + i < hi) {
        S = fmaf(f[i].x, S, fmaf(f[i].y, f[i].z, S));
        out[static_cast<long long>(t0 + i) * ldo + c] = from_float<T>(S * f[i].w);
      }
    }
  };
  fetch(cur, lo);
  for (int t0 = lo; t0 < hi; t0 += 2 * kAhead) {           // the next sixteen tokens' numbers are under way during the chain
    fetch(nxt, t0 + kAhead);
    chain(cur, t0);
    fetch(cur, t0 + 2 * kAhead);
    chain(nxt, t0 + kAhead);
  }
  state[slot * state_stride + c] = S;
}


}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

extern "C" int pih_embedding_stream(int dtype, const void* table, const void* ids, void* out, int rows, int hidden,
                                    int vocab, void* err, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = hidden >= 256 ? 256 : 64;
  if (dtype == PIH_F32)
    launch_kernel(embedding_stream_kernel<float>, dim3(rows), dim3(threads), 0, s, static_cast<const float*>(table),
                  static_cast<const int*>(ids), static_cast<float*>(out), hidden, vocab, static_cast<uint32_t*>(err));
  else if (dtype == PIH_BF16)
    launch_kernel(embedding_stream_kernel<bf16>, dim3(rows), dim3(threads), 0, s, static_cast<const bf16*>(table),
                  static_cast<const int*>(ids), static_cast<float*>(out), hidden, vocab, static_cast<uint32_t*>(err));
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}

extern "C" int pih_rmsnorm_stream(int delta_dtype, int out_dtype, void* h, const void* delta, const void* weight,
                                  int weight_len, void* out, const void* rows, int n_out, int width, float eps,
                                  void* stream) {
  if (n_out <= 0) return 0;
  if (weight_len != 1 && weight_len != width) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = width >= 1024 ? 256 : 128;
#define PIH_NORM(TD, TO)                                                                                              \
  launch_kernel(rmsnorm_stream_kernel<TD, TO>, dim3(n_out), dim3(threads), 0, s, static_cast<float*>(h),               \
                static_cast<const TD*>(delta), static_cast<const float*>(weight), weight_len, static_cast<TO*>(out),   \
                static_cast<const int*>(rows), width, eps)
  if (delta_dtype == PIH_F32 && out_dtype == PIH_F32) PIH_NORM(float, float);
  else if (delta_dtype == PIH_BF16 && out_dtype == PIH_BF16) PIH_NORM(bf16, bf16);
  else if (delta_dtype == PIH_F32 && out_dtype == PIH_BF16) PIH_NORM(float, bf16);
  else if (delta_dtype == PIH_BF16 && out_dtype == PIH_F32) PIH_NORM(bf16, float);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_NORM
  PIH_LAUNCH_CHECK();
  return 0;
}

extern "C" int pih_causal_conv(int dtype, const void* x, long long ldx, const void* w, const void* in_bias,
                               const void* out_bias, void* out, long long ldo, int channels, int taps, int activation,
                               void* state, long long state_stride, long long state_offset, const void* cu_q,
                               const void* state_slots, int rows, int requests, void* stream) {
  if (requests <= 0 || channels <= 0 || rows <= 0) return 0;
  if (taps < 1 || taps > kMaxTaps) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(requests, (channels + 31) / 32, (rows + kConvRows - 1) / kConvRows), block(32, 8);
  dim3 grid_h(requests, (channels + 127) / 128);
  if (grid.y > 65535 || grid.z > 65535) return PIH_ERR_UNSUPPORTED;
#define PIH_CONV(T)                                                                                                    \
  do {                                                                                                                 \
    launch_kernel(causal_conv_kernel<T>, grid, block, 0, s, static_cast<const T*>(x), ldx, static_cast<const T*>(w),    \
                  static_cast<const float*>(in_bias), static_cast<const float*>(out_bias), static_cast<T*>(out), ldo,  \
                  channels, taps, activation, static_cast<const float*>(state), state_stride, state_offset,            \
                  static_cast<const int*>(cu_q), static_cast<const int*>(state_slots));                                \
    PIH_LAUNCH_CHECK();                                                                                                \
    if (taps > 1)                                                                                                      \
      launch_kernel(causal_conv_history_kernel<T>, grid_h, dim3(128), 0, s, static_cast<const T*>(x), ldx,             \
                    static_cast<const float*>(in_bias), channels, taps, static_cast<float*>(state), state_stride,      \
                    state_offset, static_cast<const int*>(cu_q), static_cast<const int*>(state_slots));                \
  } while (0)
  if (dtype == PIH_F32) PIH_CONV(float);
  else if (dtype == PIH_BF16) PIH_CONV(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_CONV
  PIH_LAUNCH_CHECK();
  return 0;
}

// The gated delta rule over a step's rows.  qkv [rows, ld]: q heads, k heads, v heads (after convolution and SiLU);
// ba [rows, ldb]: write-strength logits, decay logits.  scratch: fp32, rows * (2 * kv_heads * dim + 2 * heads).
// out: fp32 [rows, heads, vdim].  The state S [heads, dim, vdim] lies at the start of a request's slot.
extern "C" int pih_gated_delta_rule(int dtype, const void* qkv, long long ld, const void* ba, long long ldb,
                                    const void* decay_log, const void* decay_bias, void* scratch, void* out, void* state,
                                    long long state_stride, const void* cu_q, const void* state_slots, int rows,
                                    int requests, int heads, int kv_heads, int dim, int vdim, float unit_eps,
                                    float q_scale, void* stream) {
  if (rows <= 0 || requests <= 0) return 0;
  if (heads % kv_heads) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int cols = vdim >= 64 ? 64 : 32;
  if (dim > 8 * cols) return PIH_ERR_UNSUPPORTED;
  const size_t smem = (static_cast<size_t>(dim) * cols + 4 * static_cast<size_t>(dim)) * sizeof(float);
  if (smem > 200 * 1024) return PIH_ERR_UNSUPPORTED;
  float* qn = static_cast<float*>(scratch);
  float* kn = qn + static_cast<long long>(rows) * kv_heads * dim;
  float* decay = kn + static_cast<long long>(rows) * kv_heads * dim;
  float* beta = decay + static_cast<long long>(rows) * heads;
  dim3 grid(requests, heads, (vdim + cols - 1) / cols);
  if (grid.y > 65535 || grid.z > 65535) return PIH_ERR_UNSUPPORTED;
  const long long qk_size = static_cast<long long>(kv_heads) * dim;
  int dim_instance = dim;
#define PIH_DELTA_REG(T, D)                                                                                            \
  do {                                                                                                                 \
    const int parts = (D) >= 64 ? 8 : 4;                                                                               \
    const size_t staged = 2 * static_cast<size_t>((D) <= 128 ? 16 : 8) *                                               \
                          (2 * parts * ((D) / parts + 4) + 4 + 32 * sizeof(T) / 4) * sizeof(float);                    \
    if (staged > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(delta_recurrence_reg_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                           static_cast<int>(staged));                                                                  \
    launch_kernel(delta_recurrence_reg_kernel<T, D>, dim3(requests, heads, (vdim + 31) / 32), dim3(32 * parts), staged, s, \
                  static_cast<const float*>(qn), static_cast<const float*>(kn),                                        \
                  static_cast<const T*>(qkv) + 2 * qk_size, ld, static_cast<const float*>(decay),                      \
                  static_cast<const float*>(beta), static_cast<float*>(out), static_cast<float*>(state), state_stride, \
                  static_cast<const int*>(cu_q), static_cast<const int*>(state_slots), heads, kv_heads, vdim);         \
  } while (0)
#define PIH_DELTA(T)                                                                                                   \
  do {                                                                                                                 \
    launch_kernel(delta_prepare_kernel<T>, dim3(rows), dim3(128), 0, s, static_cast<const T*>(qkv), ld,                \
                  static_cast<const T*>(ba), ldb, static_cast<const float*>(decay_log),                                \
                  static_cast<const float*>(decay_bias), qn, kn, decay, beta, heads, kv_heads, dim, unit_eps, q_scale); \
    PIH_LAUNCH_CHECK();                                                                                                \
    const bool words = sizeof(T) == 4 || (ld % 2 == 0 && vdim % 2 == 0);      /* values are copied in 32-bit words */  \
    if (!words) dim_instance = 0;                                                                                      \
    if (dim_instance == 16) PIH_DELTA_REG(T, 16);                                                                      \
    else if (dim_instance == 32) PIH_DELTA_REG(T, 32);                                                                          \
    else if (dim_instance == 64) PIH_DELTA_REG(T, 64);                                                                          \
    else if (dim_instance == 128) PIH_DELTA_REG(T, 128);                                                                        \
    else if (dim_instance == 256) PIH_DELTA_REG(T, 256);                                                                        \
    else {                                                                                                             \
      if (smem > 48 * 1024)                                                                                            \
        cudaFuncSetAttribute(delta_recurrence_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
      launch_kernel(delta_recurrence_kernel<T>, grid, dim3(cols), smem, s, static_cast<const float*>(qn),              \
                    static_cast<const float*>(kn), static_cast<const T*>(qkv) + 2 * qk_size, ld,                       \
                    static_cast<const float*>(decay), static_cast<const float*>(beta), static_cast<float*>(out),       \
                    static_cast<float*>(state), state_stride, static_cast<const int*>(cu_q),                           \
                    static_cast<const int*>(state_slots), heads, kv_heads, dim, vdim);                                 \
    }                                                                                                                  \
  } while (0)
  if (dtype == PIH_F32) PIH_DELTA(float);
  else if (dtype == PIH_BF16) PIH_DELTA(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_DELTA
#undef PIH_DELTA_REG
  PIH_LAUNCH_CHECK();
  return 0;
}

extern "C" int pih_gated_rmsnorm(int dtype, const void* o, const void* gate, long long ldg, const void* weight, void* out,
                                 int rows, int heads, int vdim, float eps, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long items = static_cast<long long>(rows) * heads;
  dim3 grid(static_cast<unsigned>((items + 3) / 4));
#define PIH_GN(T)                                                                                                      \
  launch_kernel(gated_rmsnorm_kernel<T>, grid, dim3(128), 0, s, static_cast<const float*>(o), static_cast<const T*>(gate), \
                ldg, static_cast<const float*>(weight), static_cast<T*>(out), items, heads, vdim, eps)
  if (dtype == PIH_F32) PIH_GN(float);
  else if (dtype == PIH_BF16) PIH_GN(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_GN
  PIH_LAUNCH_CHECK();
  return 0;
}

// coef: scratch, 4 * rows * width floats (16-byte aligned)
extern "C" int pih_rglru_scan(int dtype, const void* u, long long ldu, const void* gates, const void* y_pre, long long ldy,
                              const void* y_bias, const void* r_bias, const void* i_bias, const void* lam,
                              float decay_scale, void* coef, void* out, long long ldo, void* state, long long state_stride,
                              const void* cu_q, const void* state_slots, int rows, int requests, int width, int blocks,
                              void* stream) {
  if (requests <= 0 || width <= 0 || rows <= 0) return 0;
  if (blocks < 1 || width % blocks) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(requests, (width + 127) / 128);
  const long long items = static_cast<long long>(rows) * width;
  if (grid.y > 65535 || (items + 255) / 256 > 2147483647LL) return PIH_ERR_UNSUPPORTED;
#define PIH_SCAN(T)                                                                                                    \
  do {                                                                                                                 \
    launch_kernel(rglru_gates_kernel<T>, dim3(static_cast<unsigned>((items + 255) / 256)), dim3(256), 0, s,            \
                  static_cast<const T*>(u), ldu, static_cast<const float*>(gates), static_cast<const T*>(y_pre), ldy,  \
                  static_cast<const float*>(y_bias), static_cast<const float*>(r_bias),                                \
                  static_cast<const float*>(i_bias), static_cast<const float*>(lam), decay_scale,                      \
                  static_cast<float4*>(coef), rows, width, blocks);                                                    \
    PIH_LAUNCH_CHECK();                                                                                                \
    launch_kernel(rglru_chain_kernel<T>, grid, dim3(128), 0, s, static_cast<const float4*>(coef), static_cast<T*>(out), \
                  ldo, static_cast<float*>(state), state_stride, static_cast<const int*>(cu_q),                        \
                  static_cast<const int*>(state_slots), width);                                                        \
  } while (0)
  if (dtype == PIH_F32) PIH_SCAN(float);
  else if (dtype == PIH_BF16) PIH_SCAN(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_SCAN
  PIH_LAUNCH_CHECK();
  return 0;
}
