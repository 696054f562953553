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

// x [rows, ld]: heads x width columns; out [rows, heads, width] contiguous.
template <typename T>
__global__ void rotate_heads_kernel(const T* __restrict__ x, long long ld, T* __restrict__ out, const float* __restrict__ freq,
                                    const int* __restrict__ positions, long long rows, int heads, int width, int offset,
                                    int rot, int interleaved) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long per_row = static_cast<long long>(heads) * width;
  if (i >= rows * per_row) return;
  const long long row = i / per_row;
  const int e = static_cast<int>(i % per_row);
  const int c = e % width - offset;                               // column within the rotated part
  const T* xr = x + row * ld;
  float v = to_float<T>(xr[e]);
  if (c >= 0 && c < rot) {
    const int half = rot >> 1;
    int pair, other;
    bool first;
    if (interleaved) { pair = c >> 1; first = (c & 1) == 0; other = first ? e + 1 : e - 1; }
    else { pair = c < half ? c : c - half; first = c < half; other = first ? e + half : e - half; }
    float sn, cs;
    sincosf(static_cast<float>(positions[row]) * freq[pair], &sn, &cs);
    const float p = to_float<T>(xr[other]);
    v = first ? v * cs - p * sn : v * cs + p * sn;
  }
  out[i] = from_float<T>(v);
}

// kind 1: sigmoid(g); 2: silu(g)
template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ a, const T* __restrict__ gate, long long ldg, T* __restrict__ out,
                                long long rows, int width, int kind) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * width) return;
  const float g = to_float<T>(gate[(i / width) * ldg + i % width]);
  const float s = 1.0f / (1.0f + expf(-g));
  out[i] = from_float<T>(to_float<T>(a[i]) * (kind == 2 ? g * s : s));
}

// kind 1: the square of max(z, 0)
template <typename T>
__global__ void unary_act_kernel(const T* __restrict__ z, long long ld, T* __restrict__ out, long long rows, int width,
                                 int kind) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * width) return;
  const float v = fmaxf(to_float<T>(z[(i / width) * ld + i % width]), 0.0f);
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

// x [rows, ld] holding heads x width columns; out [rows, heads, width]; freq fp32 [rot / 2]
extern "C" int pih_rotate_heads(int dtype, const void* x, long long ld, void* out, const void* freq, const void* positions,
                                int rows, int heads, int width, int offset, int rot, int interleaved, void* stream) {
  if (rows <= 0 || heads <= 0 || width <= 0) return 0;
  if (rot < 0 || (rot & 1) || offset < 0 || offset + rot > width) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long n = static_cast<long long>(rows) * heads * width;
  if (dtype == PIH_BF16)
    launch_kernel(rotate_heads_kernel<bf16>, flat_grid(n), dim3(256), 0, s, static_cast<const bf16*>(x), ld,
                  static_cast<bf16*>(out), static_cast<const float*>(freq), static_cast<const int*>(positions),
                  static_cast<long long>(rows), heads, width, offset, rot, interleaved);
  else if (dtype == PIH_F32)
    launch_kernel(rotate_heads_kernel<float>, flat_grid(n), dim3(256), 0, s, static_cast<const float*>(x), ld,
                  static_cast<float*>(out), static_cast<const float*>(freq), static_cast<const int*>(positions),
                  static_cast<long long>(rows), heads, width, offset, rot, interleaved);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}

// out = a * act(gate): a, out [rows, width] contiguous, gate [rows, ldg]; kind 1 sigmoid, 2 silu
extern "C" int pih_gate_mul(int dtype, const void* a, const void* gate, long long ldg, void* out, long long rows, int width,
                            int kind, void* stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (kind != 1 && kind != 2) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PIH_BF16)
    launch_kernel(gate_mul_kernel<bf16>, flat_grid(rows * width), dim3(256), 0, s, static_cast<const bf16*>(a),
                  static_cast<const bf16*>(gate), ldg, static_cast<bf16*>(out), rows, width, kind);
  else if (dtype == PIH_F32)
    launch_kernel(gate_mul_kernel<float>, flat_grid(rows * width), dim3(256), 0, s, static_cast<const float*>(a),
                  static_cast<const float*>(gate), ldg, static_cast<float*>(out), rows, width, kind);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}

// out [rows, width] contiguous = act(z [rows, ld]); kind 1: relu(z)^2
extern "C" int pih_unary_act(int dtype, const void* z, long long ld, void* out, long long rows, int width, int kind,
                             void* stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (kind != 1) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PIH_BF16)
    launch_kernel(unary_act_kernel<bf16>, flat_grid(rows * width), dim3(256), 0, s, static_cast<const bf16*>(z), ld,
                  static_cast<bf16*>(out), rows, width, kind);
  else if (dtype == PIH_F32)
    launch_kernel(unary_act_kernel<float>, flat_grid(rows * width), dim3(256), 0, s, static_cast<const float*>(z), ld,
                  static_cast<float*>(out), rows, width, kind);
  else
    return PIH_ERR_BAD_ARGUMENT;
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
