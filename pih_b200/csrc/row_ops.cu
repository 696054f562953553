// Row-wise kernels that several mixers and feed-forwards share.
//
//   embed_bigram    out = embed[token] + bigram[(previous * mul_prev + token * mul_cur) mod buckets], the sum in 32-bit;
//                   a sequence's first token takes the bigram table's last row.  The token before a step's first row is
//                   the request's state (one int32 in its state slot), which the kernel also leaves for the next step
//   rmsnorm_rows    x / sqrt(mean(x^2) + eps) * w over the columns of a strided view, a weight a column
//   rotate_heads    the columns offset .. offset + rot of every head rotated by position * f_i (32-bit angles), the
//                   pairs being halves (i, i + rot / 2) or neighbours (2i, 2i + 1)
//   gate_mul        a * sigmoid(g) or a * silu(g), the gate a strided view
//   unary_act       relu(z)^2
//   scale_rows      x *= s in place (32-bit)
#include "common.cuh"

namespace pih {

// One block a row.  The block of a request's FIRST row of the step reads the request's last token from its state slot
// and leaves the step's last token there: no other block touches that slot.
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
embed_bigram_kernel(const T* __restrict__ embed, const T* __restrict__ bigram, const int* __restrict__ ids,
                    const int* __restrict__ positions, const int* __restrict__ request_of_row,
                    const int* __restrict__ cu_q, const int* __restrict__ state_slots, int* __restrict__ last_token,
                    long long ld_state, int slots, TO* __restrict__ out, int width, int vocab, long long buckets,
                    long long mul_prev, long long mul_cur, uint32_t* __restrict__ error) {
  __shared__ int prev_s;
  wait_for_prior_kernels();
  launch_dependents();
  const long long row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) publish_error(error, kTokenOutOfVocabulary);
    id = 0;
  }
  if (threadIdx.x == 0) {
    int prev = -1;                                               // none: the sequence's first token
    const int req = request_of_row[row];
    if (req >= 0) {
      const int first = cu_q[req], end = cu_q[req + 1];
      if (row == first) {
        const int slot = state_slots[req];
        if (slot >= 0 && slot < slots) {
          if (positions[row] > 0) prev = last_token[slot * ld_state];
          int last = ids[end - 1];
          last_token[slot * ld_state] = (last < 0 || last >= vocab) ? 0 : last;
        }
      } else if (positions[row] > 0) {
        prev = ids[row - 1];
        if (prev < 0 || prev >= vocab) prev = 0;                 // (reported by the row that brought it)
      }
      if (prev >= vocab) prev = 0;
    }
    prev_s = prev;
  }
  __syncthreads();
  const int prev = prev_s;
  // every factor is below ``buckets``, so no product leaves 64 bits whatever the multipliers are
  const long long pick = prev < 0 ? buckets
                                  : ((prev % buckets) * mul_prev + (static_cast<long long>(id) % buckets) * mul_cur) % buckets;
  const T* a = embed + static_cast<long long>(id) * width;
  const T* b = bigram + pick * width;
  TO* o = out + row * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_float<TO>(to_float<T>(a[c]) + to_float<T>(b[c]));
}

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const T* __restrict__ x, long long ld, const float* __restrict__ weight, T* __restrict__ out, int n,
                    float eps) {
  __shared__ float scratch[33];
  wait_for_prior_kernels();
  launch_dependents();
  const T* xr = x + static_cast<long long>(blockIdx.x) * ld;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = to_float<T>(xr[c]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(n) + eps);
  T* o = out + static_cast<long long>(blockIdx.x) * n;
  for (int c = threadIdx.x; c < n; c += blockDim.x) o[c] = from_float<T>(to_float<T>(xr[c]) * inv * weight[c]);
}

// 16 bytes as V numbers of T, and back
template <typename T, int V>
__device__ __forceinline__ void load_piece(float (&v)[V], const T* src) {
  __align__(16) T raw[V];
  *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int i = 0; i < V; ++i) v[i] = to_float<T>(raw[i]);
}
template <typename T, int V>
__device__ __forceinline__ void store_piece(T* dst, const float (&v)[V]) {
  __align__(16) T raw[V];
#pragma unroll
  for (int i = 0; i < V; ++i) raw[i] = from_float<T>(v[i]);
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(raw);
}

// x [rows, ld]: heads x width columns; out [rows, heads, width] contiguous.  A block is a row: the cosines and sines
// of the row's rot / 2 angles are formed once, in shared memory (rot <= 2 * kMaxPairs), and serve every head.
// kPieces: a thread moves 16-byte pieces (width, offset, rot / 2 — or rot with neighbouring pairs — and ld multiples
// of a piece).
constexpr int kMaxPairs = 256;
template <typename T, bool kPieces>
__global__ void __launch_bounds__(256)
rotate_heads_kernel(const T* __restrict__ x, long long ld, T* __restrict__ out, const float* __restrict__ freq,
                    const int* __restrict__ positions, int heads, int width, int offset, int rot, int interleaved) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  __shared__ float cos_s[kMaxPairs], sin_s[kMaxPairs];
  wait_for_prior_kernels();
  launch_dependents();
  const long long row = blockIdx.x;
  const int half = rot >> 1;
  const float place = static_cast<float>(positions[row]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(place * freq[i], &sin_s[i], &cos_s[i]);   // (half <= kMaxPairs)
  __syncthreads();
  const T* xr = x + row * ld;
  T* o = out + row * heads * width;
  const int n = heads * width;
  if constexpr (kPieces) {
    for (int e = threadIdx.x * V; e < n; e += blockDim.x * V) {
      const int c = e % width - offset;
      float v[V];
      load_piece<T, V>(v, xr + e);
      if (c >= 0 && c < rot) {
        if (interleaved) {
#pragma unroll
          for (int i = 0; i < V; i += 2) {
            const float cs = cos_s[(c + i) >> 1], sn = sin_s[(c + i) >> 1];
            const float a = v[i], b = v[i + 1];
            v[i] = a * cs - b * sn;
            v[i + 1] = b * cs + a * sn;
          }
        } else {
          const bool first = c < half;
          float p[V];
          load_piece<T, V>(p, xr + (first ? e + half : e - half));
          const int pair0 = first ? c : c - half;
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float cs = cos_s[pair0 + i], sn = sin_s[pair0 + i];
            v[i] = first ? v[i] * cs - p[i] * sn : v[i] * cs + p[i] * sn;
          }
        }
      }
      store_piece<T, V>(o + e, v);
    }
  } else {
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      const int c = e % width - offset;                           // column within the rotated part
      float v = to_float<T>(xr[e]);
      if (c >= 0 && c < rot) {
        int pair, other;
        bool first;
        if (interleaved) { pair = c >> 1; first = (c & 1) == 0; other = first ? e + 1 : e - 1; }
        else { pair = c < half ? c : c - half; first = c < half; other = first ? e + half : e - half; }
        const float p = to_float<T>(xr[other]);
        v = first ? v * cos_s[pair] - p * sin_s[pair] : v * cos_s[pair] + p * sin_s[pair];
      }
      o[e] = from_float<T>(v);
    }
  }
}

// kind 1: sigmoid(g); 2: silu(g).  kPieces: 16 bytes a thread (width and ldg multiples of a piece).
template <typename T, bool kPieces>
__global__ void gate_mul_kernel(const T* __restrict__ a, const T* __restrict__ gate, long long ldg, T* __restrict__ out,
                                long long rows, int width, int kind) {
  constexpr int V = kPieces ? 16 / static_cast<int>(sizeof(T)) : 1;
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
  if (i >= rows * width) return;
  const long long gi = (i / width) * ldg + i % width;
  if (kPieces) {
    float av[V], gv[V];
    load_piece<T, V>(av, a + i);
    load_piece<T, V>(gv, gate + gi);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float s = 1.0f / (1.0f + expf(-gv[j]));
      av[j] *= kind == 2 ? gv[j] * s : s;
    }
    store_piece<T, V>(out + i, av);
    return;
  }
  const float g = to_float<T>(gate[gi]);
  const float s = 1.0f / (1.0f + expf(-g));
  out[i] = from_float<T>(to_float<T>(a[i]) * (kind == 2 ? g * s : s));
}

// kind 1: the square of max(z, 0).  kPieces: 16 bytes a thread (width and ld multiples of a piece).
template <typename T, bool kPieces>
__global__ void unary_act_kernel(const T* __restrict__ z, long long ld, T* __restrict__ out, long long rows, int width,
                                 int kind) {
  constexpr int V = kPieces ? 16 / static_cast<int>(sizeof(T)) : 1;
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
  if (i >= rows * width) return;
  const long long zi = (i / width) * ld + i % width;
  if (kPieces) {
    float v[V];
    load_piece<T, V>(v, z + zi);
#pragma unroll
    for (int j = 0; j < V; ++j) { v[j] = fmaxf(v[j], 0.0f); v[j] *= v[j]; }
    store_piece<T, V>(out + i, v);
    return;
  }
  const float v = fmaxf(to_float<T>(z[zi]), 0.0f);
  out[i] = from_float<T>(v * v);
}

__global__ void scale_rows_kernel(float* __restrict__ x, long long n, float s) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= s;
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

static inline dim3 flat_grid(long long n) { return dim3(static_cast<unsigned>((n + 255) / 256)); }

// embed [vocab, width], bigram [buckets + 1, width] of ``dtype``; out [rows, width] of ``out_dtype``; last_token int32
// [slots, ld_state] (element 0 of a slot's row); ids, positions, request_of_row [rows]; cu_q, state_slots per request.
extern "C" int pih_embed_bigram(int dtype, int out_dtype, const void* embed, const void* bigram, const void* ids,
                                const void* positions, const void* request_of_row, const void* cu_q,
                                const void* state_slots, void* last_token, long long ld_state, int slots, void* out, int rows,
                                int width, int vocab, long long buckets, long long mul_prev, long long mul_cur, void* error,
                                void* stream) {
  if (rows <= 0) return 0;
  if (buckets < 1 || width < 1 || buckets > (1LL << 31) || mul_prev < 0 || mul_cur < 0) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define PIH_EB(T, TO)                                                                                                  \
  launch_kernel(embed_bigram_kernel<T, TO>, dim3(rows), dim3(width >= 1024 ? 256 : 128), 0, s,                         \
                static_cast<const T*>(embed), static_cast<const T*>(bigram), static_cast<const int*>(ids),             \
                static_cast<const int*>(positions), static_cast<const int*>(request_of_row),                           \
                static_cast<const int*>(cu_q), static_cast<const int*>(state_slots), static_cast<int*>(last_token),    \
                ld_state, slots, static_cast<TO*>(out), width, vocab, buckets, mul_prev % buckets, mul_cur % buckets,  \
                static_cast<uint32_t*>(error))
  if (dtype == PIH_F32 && out_dtype == PIH_F32) PIH_EB(float, float);
  else if (dtype == PIH_BF16 && out_dtype == PIH_F32) PIH_EB(bf16, float);
  else if (dtype == PIH_BF16 && out_dtype == PIH_BF16) PIH_EB(bf16, bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_EB
  PIH_LAUNCH_CHECK();
  return 0;
}

// x [rows, ld] (n columns read), weight fp32 [n], out [rows, n] contiguous
extern "C" int pih_rmsnorm_rows(int dtype, const void* x, long long ld, const void* weight, void* out, int rows, int n,
                                float eps, void* stream) {
  if (rows <= 0 || n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 block(n >= 1024 ? 256 : 128);
  if (dtype == PIH_BF16)
    launch_kernel(rmsnorm_rows_kernel<bf16>, dim3(rows), block, 0, s, static_cast<const bf16*>(x), ld,
                  static_cast<const float*>(weight), static_cast<bf16*>(out), n, eps);
  else if (dtype == PIH_F32)
    launch_kernel(rmsnorm_rows_kernel<float>, dim3(rows), block, 0, s, static_cast<const float*>(x), ld,
                  static_cast<const float*>(weight), static_cast<float*>(out), n, eps);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// x [rows, ld] holding heads x width columns; out [rows, heads, width]; freq fp32 [rot / 2]
extern "C" int pih_rotate_heads(int dtype, const void* x, long long ld, void* out, const void* freq, const void* positions,
                                int rows, int heads, int width, int offset, int rot, int interleaved, void* stream) {
  if (rows <= 0 || heads <= 0 || width <= 0) return 0;
  if (rot < 0 || (rot & 1) || offset < 0 || offset + rot > width) return PIH_ERR_BAD_ARGUMENT;
  if (rot > 2 * kMaxPairs) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int V = dtype == PIH_F32 ? 4 : 8;
  const bool pieces = width % V == 0 && offset % V == 0 && ld % V == 0 && (interleaved ? rot % V == 0 : (rot / 2) % V == 0) &&
                      aligned16(x) && aligned16(out);
  const dim3 block(heads * width >= 2048 ? 256 : 128);
#define PIH_RH(T, P)                                                                                                   \
  launch_kernel(rotate_heads_kernel<T, P>, dim3(rows), block, 0, s, static_cast<const T*>(x), ld, static_cast<T*>(out), \
                static_cast<const float*>(freq), static_cast<const int*>(positions), heads, width, offset, rot, interleaved)
  if (dtype == PIH_BF16) { if (pieces) PIH_RH(bf16, true); else PIH_RH(bf16, false); }
  else if (dtype == PIH_F32) { if (pieces) PIH_RH(float, true); else PIH_RH(float, false); }
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_RH
  PIH_LAUNCH_CHECK();
  return 0;
}

// out = a * act(gate): a, out [rows, width] contiguous, gate [rows, ldg]; kind 1 sigmoid, 2 silu
extern "C" int pih_gate_mul(int dtype, const void* a, const void* gate, long long ldg, void* out, long long rows, int width,
                            int kind, void* stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (kind != 1 && kind != 2) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int V = dtype == PIH_F32 ? 4 : 8;
  const bool pieces = width % V == 0 && ldg % V == 0 && aligned16(a) && aligned16(gate) && aligned16(out);
  const long long n = rows * width / (pieces ? V : 1);
#define PIH_GM(T, P)                                                                                                   \
  launch_kernel(gate_mul_kernel<T, P>, flat_grid(n), dim3(256), 0, s, static_cast<const T*>(a),                        \
                static_cast<const T*>(gate), ldg, static_cast<T*>(out), rows, width, kind)
  if (dtype == PIH_BF16) { if (pieces) PIH_GM(bf16, true); else PIH_GM(bf16, false); }
  else if (dtype == PIH_F32) { if (pieces) PIH_GM(float, true); else PIH_GM(float, false); }
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_GM
  PIH_LAUNCH_CHECK();
  return 0;
}

// out [rows, width] contiguous = act(z [rows, ld]); kind 1: relu(z)^2
extern "C" int pih_unary_act(int dtype, const void* z, long long ld, void* out, long long rows, int width, int kind,
                             void* stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (kind != 1) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int V = dtype == PIH_F32 ? 4 : 8;
  const bool pieces = width % V == 0 && ld % V == 0 && aligned16(z) && aligned16(out);
  const long long n = rows * width / (pieces ? V : 1);
#define PIH_UA(T, P)                                                                                                   \
  launch_kernel(unary_act_kernel<T, P>, flat_grid(n), dim3(256), 0, s, static_cast<const T*>(z), ld,                   \
                static_cast<T*>(out), rows, width, kind)
  if (dtype == PIH_BF16) { if (pieces) PIH_UA(bf16, true); else PIH_UA(bf16, false); }
  else if (dtype == PIH_F32) { if (pieces) PIH_UA(float, true); else PIH_UA(float, false); }
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_UA
  PIH_LAUNCH_CHECK();
  return 0;
}

extern "C" int pih_scale_rows(void* x, long long n, float scale, void* stream) {
  if (n <= 0) return 0;
  launch_kernel(scale_rows_kernel, flat_grid(n), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<float*>(x), n,
                scale);
  PIH_LAUNCH_CHECK();
  return 0;
}
