// Row-wise kernels around a 32-bit residual stream whose norms sit on the sub-layers' outputs.
//
//   stream_cast       the stream rounded to the compute dtype (what a sub-layer reads)
//   stream_norm_add   h += rmsnorm(y + bias) * w in 32-bit, and beside it the new h rounded to the compute dtype
//   bias_xielu        act(z + b): for u > 0  ap u^2 + u / 2,  else  an (exp(u) - 1 - u) + u / 2   (32-bit inside)
//   add_gated         out = a + sigmoid(g[row]) * b   (a shared expert behind its one-number gate)
//   embed_positions   several copies of embed[token] + positions[place] as 32-bit streams
//   hyper_stream      several residual streams a row: the pending sub-layer output is written into them through a mixing
//                     matrix, and the next sub-layer's input is read out of them and normed, in one pass over the row
#include "common.cuh"

namespace pih {

template <typename TO>
__global__ void stream_cast_kernel(const float* __restrict__ h, TO* __restrict__ out, long long n) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_float<TO>(h[i]);
}

// One block a row.  The sum of squares is taken over y + bias as it is (32-bit); the order of additions depends on the
// block's size alone.
template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
stream_norm_add_kernel(float* __restrict__ h, const TY* __restrict__ y, long long ldy, const float* __restrict__ bias,
                       const float* __restrict__ weight, TO* __restrict__ copy, int width, float eps) {
  __shared__ float scratch[33];
  wait_for_prior_kernels();
  launch_dependents();
  const long long row = blockIdx.x;
  const TY* yr = y + row * ldy;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_float<TY>(yr[c]) + (bias != nullptr ? bias[c] : 0.0f);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  float* hr = h + row * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_float<TY>(yr[c]) + (bias != nullptr ? bias[c] : 0.0f);
    const float s = hr[c] + v * inv * weight[c];
    hr[c] = s;
    if (copy != nullptr) copy[row * width + c] = from_float<TO>(s);
  }
}

template <typename T>
__global__ void bias_xielu_kernel(const T* __restrict__ z, long long ldz, const float* __restrict__ bias, T* __restrict__ out,
                                  long long rows, int width, float alpha_positive, float alpha_negative) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * width) return;
  const long long row = i / width;
  const int c = static_cast<int>(i - row * width);
  const float u = to_float<T>(z[row * ldz + c]) + (bias != nullptr ? bias[c] : 0.0f);
  const float v = u > 0.0f ? fmaf(alpha_positive * u, u, 0.5f * u) : fmaf(alpha_negative, expm1f(u) - u, 0.5f * u);
  out[i] = from_float<T>(v);
}

// The same, 16 bytes a thread (width and the row stride multiples of 16 bytes).
template <typename T>
__global__ void bias_xielu_vec_kernel(const T* __restrict__ z, long long ldz, const float* __restrict__ bias, T* __restrict__ out,
                                      long long rows, int width, float alpha_positive, float alpha_negative) {
  constexpr int kVec = 16 / sizeof(T);
  wait_for_prior_kernels();
  launch_dependents();
  const int per_row = width / kVec;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * per_row) return;
  const long long row = i / per_row;
  const int c = static_cast<int>(i - row * per_row) * kVec;
  __align__(16) T v[kVec];
  *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(z + row * ldz + c);
#pragma unroll
  for (int k = 0; k < kVec; ++k) {
    const float u = to_float<T>(v[k]) + (bias != nullptr ? bias[c + k] : 0.0f);
    v[k] = from_float<T>(u > 0.0f ? fmaf(alpha_positive * u, u, 0.5f * u) : fmaf(alpha_negative, expm1f(u) - u, 0.5f * u));
  }
  *reinterpret_cast<uint4*>(out + row * width + c) = *reinterpret_cast<const uint4*>(v);
}

template <typename T>
__global__ void add_gated_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ gate,
                                 long long ldg, T* __restrict__ out, long long rows, int width) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * width) return;
  const long long row = i / width;
  const float g = gate != nullptr ? 1.0f / (1.0f + expf(-gate[row * ldg])) : 1.0f;      // no gate: a + b
  out[i] = from_float<T>(fmaf(g, to_float<T>(b[i]), to_float<T>(a[i])));
}

// out [rows][streams][width] = embed[token] + positions[place], the same in every stream (32-bit sums).
template <typename T, typename TO>
__global__ void embed_positions_kernel(const T* __restrict__ embed, const T* __restrict__ places, const int* __restrict__ ids,
                                       const int* __restrict__ positions, TO* __restrict__ out, int width, int streams,
                                       int vocab, int max_positions, uint32_t* __restrict__ error) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long row = blockIdx.x;
  int id = ids[row], pos = positions[row];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) publish_error(error, kTokenOutOfVocabulary);
    id = 0;
  }
  if (places != nullptr && (pos < 0 || pos >= max_positions)) {
    if (threadIdx.x == 0) publish_error(error, kBadPosition);
    pos = 0;
  }
  const T* e = embed + static_cast<long long>(id) * width;
  const T* p = places != nullptr ? places + static_cast<long long>(pos) * width : nullptr;
  TO* o = out + row * streams * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const TO v = from_float<TO>(to_float<T>(e[c]) + (p != nullptr ? to_float<T>(p[c]) : 0.0f));
    for (int s = 0; s < streams; ++s) o[static_cast<long long>(s) * width + c] = v;
  }
}

constexpr int kMaxStreams = 8;

// One block a row of x [rows][S][width] (32-bit).  With y (the output of the sub-layer that ran last, not yet written):
//   x_t <- sum_s mix[s][t] x_s + spread[t] y        for all t at once, from the old streams
// (stored back unless ``gather`` selects rows: then the row is only read).  With ``collect``:
//   u = sum_t collect[t] x_t;   out = u / sqrt(mean(u^2) + eps) * weight                (weight null: out = u)
// rounded to TO.  All sums 32-bit, in the order of the streams.  SC: the number of streams where the instance knows it
// (0: any number up to kMaxStreams); V: columns a thread takes at a time (4: 16-byte loads of the streams).
template <typename TY, typename TO, int SC, int V>
__global__ void __launch_bounds__(256)
hyper_stream_kernel(float* __restrict__ x, const TY* __restrict__ y, long long ldy, const float* __restrict__ mix,
                    const float* __restrict__ spread, const float* __restrict__ collect, const float* __restrict__ weight,
                    const int* __restrict__ gather, TO* __restrict__ out, int streams, int width, float eps) {
  constexpr int NS = SC > 0 ? SC : kMaxStreams;
  const int S = SC > 0 ? SC : streams;
  extern __shared__ __align__(16) float hyper_u[];             // [width]
  __shared__ float scratch[33];
  __shared__ float coef[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
  wait_for_prior_kernels();
  launch_dependents();
  const long long row = gather != nullptr ? gather[blockIdx.x] : blockIdx.x;
  float* m = coef;
  float* sp = coef + kMaxStreams * kMaxStreams;
  float* co = sp + kMaxStreams;
  if (threadIdx.x < S * S && y != nullptr) m[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < S) {
    sp[threadIdx.x] = y != nullptr ? spread[threadIdx.x] : 0.0f;
    co[threadIdx.x] = collect != nullptr ? collect[threadIdx.x] : 0.0f;
  }
  __syncthreads();
  float* xr = x + row * S * width;
  const TY* yr = y != nullptr ? y + row * ldy : nullptr;
  float ss = 0.0f;
  for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
    float v[NS][V];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      if (s < S) {
        if constexpr (V == 4) {
          const float4 r = *reinterpret_cast<const float4*>(xr + static_cast<long long>(s) * width + c);
          v[s][0] = r.x; v[s][1] = r.y; v[s][2] = r.z; v[s][3] = r.w;
        } else {
          v[s][0] = xr[static_cast<long long>(s) * width + c];
        }
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) v[s][i] = 0.0f;
      }
    }
    if (yr != nullptr) {
      float yv[V];
      if constexpr (V == 4 && sizeof(TY) == 2) {
        const uint2 r = *reinterpret_cast<const uint2*>(yr + c);
        yv[0] = __uint_as_float(r.x << 16); yv[1] = __uint_as_float(r.x & 0xffff0000u);
        yv[2] = __uint_as_float(r.y << 16); yv[3] = __uint_as_float(r.y & 0xffff0000u);
      } else if constexpr (V == 4) {
        const float4 r = *reinterpret_cast<const float4*>(yr + c);
        yv[0] = r.x; yv[1] = r.y; yv[2] = r.z; yv[3] = r.w;
      } else {
        yv[0] = to_float<TY>(yr[c]);
      }
      float n[NS][V];
#pragma unroll
      for (int t = 0; t < NS; ++t) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float acc = 0.0f;
          if (t < S) {
#pragma unroll
            for (int s = 0; s < NS; ++s)
              if (s < S) acc = fmaf(m[s * S + t], v[s][i], acc);
            acc = fmaf(sp[t], yv[i], acc);
          }
          n[t][i] = acc;
        }
      }
#pragma unroll
      for (int t = 0; t < NS; ++t) {
#pragma unroll
        for (int i = 0; i < V; ++i) v[t][i] = n[t][i];
        if (t < S && gather == nullptr) {
          if constexpr (V == 4)
            *reinterpret_cast<float4*>(xr + static_cast<long long>(t) * width + c) = make_float4(n[t][0], n[t][1], n[t][2], n[t][3]);
          else
            xr[static_cast<long long>(t) * width + c] = n[t][0];
        }
      }
    }
    if (collect != nullptr) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float u = 0.0f;
#pragma unroll
        for (int t = 0; t < NS; ++t)
          if (t < S) u = fmaf(co[t], v[t][i], u);
        hyper_u[c + i] = u;
        ss = fmaf(u, u, ss);
      }
    }
  }
  if (collect == nullptr) return;
  float inv = 1.0f;
  if (weight != nullptr) {
    ss = block_sum(ss, scratch);
    inv = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  }
  TO* o = out + static_cast<long long>(blockIdx.x) * width;
  for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {  // (a thread reads back what it wrote itself)
#pragma unroll
    for (int i = 0; i < V; ++i)
      o[c + i] = from_float<TO>(weight != nullptr ? hyper_u[c + i] * inv * weight[c + i] : hyper_u[c + i]);
  }
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

extern "C" int pih_stream_cast(int out_dtype, const void* h, void* out, long long n, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>((n + 255) / 256));
  if (out_dtype == PIH_BF16)
    launch_kernel(stream_cast_kernel<bf16>, grid, dim3(256), 0, s, static_cast<const float*>(h), static_cast<bf16*>(out), n);
  else if (out_dtype == PIH_F32)
    launch_kernel(stream_cast_kernel<float>, grid, dim3(256), 0, s, static_cast<const float*>(h), static_cast<float*>(out), n);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}

// h fp32 [rows, width] (in place); y [rows, ldy] of y_dtype; bias, weight fp32 [width] (bias may be null); copy
// [rows, width] of copy_dtype or null.
extern "C" int pih_stream_norm_add(int y_dtype, int copy_dtype, void* h, const void* y, long long ldy, const void* bias,
                                   const void* weight, void* copy, int rows, int width, float eps, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(rows), block(width >= 1024 ? 256 : 128);
#define PIH_SNA(TY, TO)                                                                                                \
  launch_kernel(stream_norm_add_kernel<TY, TO>, grid, block, 0, s, static_cast<float*>(h), static_cast<const TY*>(y), \
                ldy, static_cast<const float*>(bias), static_cast<const float*>(weight), static_cast<TO*>(copy), width, eps)
  if (y_dtype == PIH_BF16 && copy_dtype == PIH_BF16) PIH_SNA(bf16, bf16);
  else if (y_dtype == PIH_F32 && copy_dtype == PIH_F32) PIH_SNA(float, float);
  else if (y_dtype == PIH_BF16 && copy_dtype == PIH_F32) PIH_SNA(bf16, float);
  else if (y_dtype == PIH_F32 && copy_dtype == PIH_BF16) PIH_SNA(float, bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_SNA
  PIH_LAUNCH_CHECK();
  return 0;
}

extern "C" int pih_bias_xielu(int dtype, const void* z, long long ldz, const void* bias, void* out, long long rows, int width,
                              float alpha_positive, float alpha_negative, void* stream) {
  if (rows <= 0 || width <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int vec = dtype == PIH_F32 ? 4 : 8;
  if ((dtype == PIH_F32 || dtype == PIH_BF16) && width % vec == 0 && ldz % vec == 0 &&
      reinterpret_cast<uintptr_t>(z) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    const dim3 vgrid(static_cast<unsigned>((rows * (width / vec) + 255) / 256));
    if (dtype == PIH_BF16)
      launch_kernel(bias_xielu_vec_kernel<bf16>, vgrid, dim3(256), 0, s, static_cast<const bf16*>(z), ldz,
                    static_cast<const float*>(bias), static_cast<bf16*>(out), rows, width, alpha_positive, alpha_negative);
    else
      launch_kernel(bias_xielu_vec_kernel<float>, vgrid, dim3(256), 0, s, static_cast<const float*>(z), ldz,
                    static_cast<const float*>(bias), static_cast<float*>(out), rows, width, alpha_positive, alpha_negative);
    PIH_LAUNCH_CHECK();
    return 0;
  }
  const dim3 grid(static_cast<unsigned>((rows * width + 255) / 256));
  if (dtype == PIH_BF16)
    launch_kernel(bias_xielu_kernel<bf16>, grid, dim3(256), 0, s, static_cast<const bf16*>(z), ldz,
                  static_cast<const float*>(bias), static_cast<bf16*>(out), rows, width, alpha_positive, alpha_negative);
  else if (dtype == PIH_F32)
    launch_kernel(bias_xielu_kernel<float>, grid, dim3(256), 0, s, static_cast<const float*>(z), ldz,
                  static_cast<const float*>(bias), static_cast<float*>(out), rows, width, alpha_positive, alpha_negative);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}

// out = a + sigmoid(gate[row * ldg]) * b; a, b, out [rows, width] contiguous; gate fp32
extern "C" int pih_add_gated(int dtype, const void* a, const void* b, const void* gate, long long ldg, void* out,
                             long long rows, int width, void* stream) {
  if (rows <= 0 || width <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>((rows * width + 255) / 256));
  if (dtype == PIH_BF16)
    launch_kernel(add_gated_kernel<bf16>, grid, dim3(256), 0, s, static_cast<const bf16*>(a), static_cast<const bf16*>(b),
                  static_cast<const float*>(gate), ldg, static_cast<bf16*>(out), rows, width);
  else if (dtype == PIH_F32)
    launch_kernel(add_gated_kernel<float>, grid, dim3(256), 0, s, static_cast<const float*>(a), static_cast<const float*>(b),
                  static_cast<const float*>(gate), ldg, static_cast<float*>(out), rows, width);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}

// out [rows, streams, width] of out_dtype = embed[ids] + places[positions] (places null: the embedding alone).
extern "C" int pih_embed_positions(int dtype, int out_dtype, const void* embed, const void* places, const void* ids,
                                   const void* positions, void* out, int rows, int width, int streams, int vocab,
                                   int max_positions, void* error, void* stream) {
  if (rows <= 0) return 0;
  if (streams < 1 || width < 1) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define PIH_EP(T, TO)                                                                                                  \
  launch_kernel(embed_positions_kernel<T, TO>, dim3(rows), dim3(width >= 1024 ? 256 : 128), 0, s,                      \
                static_cast<const T*>(embed), static_cast<const T*>(places), static_cast<const int*>(ids),             \
                static_cast<const int*>(positions), static_cast<TO*>(out), width, streams, vocab, max_positions,       \
                static_cast<uint32_t*>(error))
  if (dtype == PIH_BF16 && out_dtype == PIH_F32) PIH_EP(bf16, float);
  else if (dtype == PIH_F32 && out_dtype == PIH_F32) PIH_EP(float, float);
  else if (dtype == PIH_BF16 && out_dtype == PIH_BF16) PIH_EP(bf16, bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_EP
  PIH_LAUNCH_CHECK();
  return 0;
}

// x fp32 [*, streams, width] in place; y [rows, ldy] of y_dtype or null (then mix and spread are not read); mix fp32
// [streams, streams] indexed [from, to]; spread, collect fp32 [streams]; weight fp32 [width] or null; gather int32
// [out_rows] or null (null: out_rows rows from the first); out [out_rows, width] of out_dtype (null without collect).
extern "C" int pih_hyper_stream(int y_dtype, int out_dtype, void* x, const void* y, long long ldy, const void* mix,
                                const void* spread, const void* collect, const void* weight, const void* gather, void* out,
                                int out_rows, int streams, int width, float eps, void* stream) {
  if (out_rows <= 0) return 0;
  if (streams < 1 || streams > kMaxStreams || (collect != nullptr && out == nullptr) || (y == nullptr && collect == nullptr))
    return PIH_ERR_BAD_ARGUMENT;
  if (static_cast<size_t>(width) * sizeof(float) > 96 * 1024) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = collect != nullptr ? static_cast<size_t>(width) * sizeof(float) : 0;
  const dim3 grid(out_rows), block(width >= 2048 ? 256 : 128);
  const bool wide = width % 4 == 0 && ldy % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(y) % 16 == 0;
#define PIH_HS_I(TY, TO, SC, V)                                                                                        \
  do {                                                                                                                 \
    static bool raised = false;                                                                                        \
    if (!raised && smem > 48 * 1024) {                                                                                 \
      cudaFuncSetAttribute(hyper_stream_kernel<TY, TO, SC, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
      raised = true;                                                                                                   \
    }                                                                                                                  \
    launch_kernel(hyper_stream_kernel<TY, TO, SC, V>, grid, block, smem, s, static_cast<float*>(x),                    \
                  static_cast<const TY*>(y), ldy, static_cast<const float*>(mix), static_cast<const float*>(spread),   \
                  static_cast<const float*>(collect), static_cast<const float*>(weight), static_cast<const int*>(gather), \
                  static_cast<TO*>(out), streams, width, eps);                                                         \
  } while (0)
#define PIH_HS(TY, TO)                                                                                                 \
  do {                                                                                                                 \
    if (wide && streams == 2) PIH_HS_I(TY, TO, 2, 4);                                                                  \
    else if (wide && streams == 4) PIH_HS_I(TY, TO, 4, 4);                                                             \
    else if (wide) PIH_HS_I(TY, TO, 0, 4);                                                                             \
    else PIH_HS_I(TY, TO, 0, 1);                                                                                       \
  } while (0)
  if (y_dtype == PIH_BF16 && out_dtype == PIH_BF16) PIH_HS(bf16, bf16);
  else if (y_dtype == PIH_F32 && out_dtype == PIH_F32) PIH_HS(float, float);
  else if (y_dtype == PIH_BF16 && out_dtype == PIH_F32) PIH_HS(bf16, float);
  else if (y_dtype == PIH_F32 && out_dtype == PIH_BF16) PIH_HS(float, bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_HS_I
#undef PIH_HS
  PIH_LAUNCH_CHECK();
  return 0;
}
