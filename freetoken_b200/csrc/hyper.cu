// Several residual streams (hyper-connections), and the mean of normed branch outputs.
//
// hyper_step, a block per token: the token's S <= 8 streams pass through registers once.  A sub-layer's result y is
// written into every stream while the streams are mixed (x_t <- sum_s mix[s][t] x_s + out[t] y, all new streams from
// the old ones), the next sub-layer's input u = sum_s in[s] x_s is formed from the new streams, kept in shared
// memory, RMS-normed (plain weight) and written; the last layer's call leaves the streams' sum in the one-stream
// residual, the first one's starts every stream as a copy of it.  Each of these steps is optional, so one launch
// serves "write the result of the sub-layer before and read for the next one".  All sums are 32-bit, added in the
// order s = 0, 1, ...
//
// norm_mean, a block per token: out = (1 / n) sum_i x_i / rms(x_i) * w_i over n <= 4 branch outputs.
#include "common.cuh"

namespace ftk {

constexpr int kHyperMaxStreams = 8;
constexpr int kHyperThreads = 256;

struct HyperArgs {
  float* streams; long long stream_stride; int S, T, C;
  const float* init_from; const void* y; const float* mix; const float* out_w; const float* in_w; const float* norm_w;
  float eps; void* h_out; float* sum_out;
};

// MAXS: the smallest of 1, 2, 4, 8 that holds the streams (a token's streams stay in registers: the fewer the kernel
// sets aside, the more blocks an SM holds)
template <typename TY, typename TH, int MAXS>
__global__ void __launch_bounds__(kHyperThreads) hyper_step_kernel(HyperArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float sm[];  // [C] the sub-layer's input before its norm, then 33 floats of scratch
  __shared__ float coef[kHyperMaxStreams * kHyperMaxStreams + 2 * kHyperMaxStreams];
  const int S = a.S, C = a.C;
  float* cmix = coef; float* cout = coef + kHyperMaxStreams * kHyperMaxStreams; float* cin = cout + kHyperMaxStreams;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) cmix[i] = a.mix ? a.mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) { cout[i] = a.out_w ? a.out_w[i] : 0.f; cin[i] = a.in_w ? a.in_w[i] : 0.f; }
  __syncthreads();
  const size_t t = blockIdx.x;
  const TY* y = a.y ? (const TY*)a.y + t * C : nullptr;
  const float* init = a.init_from ? a.init_from + t * C : nullptr;
  float* u_row = sm;
  float* scratch = sm + ((C + 3) & ~3);
  const bool vec = (C & 3) == 0 && (a.stream_stride & 3) == 0;
  const bool writes = y != nullptr || init != nullptr;
  float ss = 0.f;
  for (int c0 = threadIdx.x * 4; c0 < C; c0 += blockDim.x * 4) {
    const int nc = min(4, C - c0);
    float x[MAXS][4];
    if (init) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (vec) Vec4<float>::load(init + c0, v);
      else for (int i = 0; i < nc; ++i) v[i] = init[c0 + i];
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
#pragma unroll
        for (int i = 0; i < 4; ++i) x[s][i] = v[i];
    } else {
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) {
          const float* src = a.streams + (size_t)s * a.stream_stride + t * C + c0;
          if (vec) Vec4<float>::load(src, x[s]);
          else for (int i = 0; i < 4; ++i) x[s][i] = i < nc ? src[i] : 0.f;
        }
    }
    float yv[4] = {0.f, 0.f, 0.f, 0.f};
    if (y) {
      if (vec) Vec4<TY>::load(y + c0, yv);
      else for (int i = 0; i < nc; ++i) yv[i] = to_float(y[c0 + i]);
    }
    // one new stream after the other, each from all the old ones: stored, and added to what is read from the new streams
    float u[4] = {0.f, 0.f, 0.f, 0.f}, z[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int to = 0; to < MAXS; ++to)
      if (to < S) {
        float v[4];
        if (y) {
#pragma unroll
          for (int i = 0; i < 4; ++i) v[i] = 0.f;
#pragma unroll
          for (int s = 0; s < MAXS; ++s)
            if (s < S)
#pragma unroll
              for (int i = 0; i < 4; ++i) v[i] = fmaf(cmix[s * S + to], x[s][i], v[i]);
#pragma unroll
          for (int i = 0; i < 4; ++i) v[i] = fmaf(cout[to], yv[i], v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) v[i] = x[to][i];
        }
        if (writes) {
          float* dst = a.streams + (size_t)to * a.stream_stride + t * C + c0;
          if (vec) Vec4<float>::store(dst, v);
          else for (int i = 0; i < nc; ++i) dst[i] = v[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) { u[i] = fmaf(cin[to], v[i], u[i]); z[i] += v[i]; }
      }
    if (a.in_w) {
      for (int i = 0; i < nc; ++i) { u_row[c0 + i] = u[i]; ss = fmaf(u[i], u[i], ss); }
    }
    if (a.sum_out) {
      float* dst = a.sum_out + t * C + c0;
      if (vec) Vec4<float>::store(dst, z);
      else for (int i = 0; i < nc; ++i) dst[i] = z[i];
    }
  }
  if (!a.in_w) return;
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / (float)C + a.eps);
  TH* h = (TH*)a.h_out + t * C;
  for (int c0 = threadIdx.x * 4; c0 < C; c0 += blockDim.x * 4) {
    const int nc = min(4, C - c0);
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < nc; ++i) v[i] = u_row[c0 + i] * r * a.norm_w[c0 + i];
    if ((C & 3) == 0) Vec4<TH>::store(h + c0, v);
    else for (int i = 0; i < nc; ++i) h[c0 + i] = from_float<TH>(v[i]);
  }
}

struct NormMeanArgs { const void* xs[4]; const float* ws[4]; int n, C; float eps; void* out; int keep; };

// keep: the rows stay in shared memory between the pass that takes their mean squares and the pass that adds them up
// (n * C values of T behind the scratch); otherwise the second pass reads them again
template <typename T>
__global__ void __launch_bounds__(kHyperThreads) norm_mean_kernel(NormMeanArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float nm_sm[];
  float* scratch = nm_sm;  // 33 floats (36 set aside)
  T* kept = reinterpret_cast<T*>(nm_sm + 36);
  const size_t t = blockIdx.x;
  const int C = a.C;
  const bool vec = (C & 3) == 0;
  float r[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j >= a.n) break;
    const T* x = (const T*)a.xs[j] + t * C;
    float ss = 0.f;
    for (int c0 = threadIdx.x * 4; c0 < C; c0 += blockDim.x * 4) {
      const int nc = min(4, C - c0);
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (vec) Vec4<T>::load(x + c0, v);
      else for (int i = 0; i < nc; ++i) v[i] = to_float(x[c0 + i]);
      for (int i = 0; i < 4; ++i) ss = fmaf(v[i], v[i], ss);
      if (a.keep) {
        if (vec) Vec4<T>::store(kept + (size_t)j * C + c0, v);
        else for (int i = 0; i < nc; ++i) kept[(size_t)j * C + c0 + i] = from_float<T>(v[i]);
      }
    }
    ss = block_sum(ss, scratch);
    r[j] = rsqrtf(ss / (float)C + a.eps);
  }
  const float inv_n = 1.f / (float)a.n;
  T* out = (T*)a.out + t * C;
  for (int c0 = threadIdx.x * 4; c0 < C; c0 += blockDim.x * 4) {
    const int nc = min(4, C - c0);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j >= a.n) break;
      const T* x = a.keep ? kept + (size_t)j * C : (const T*)a.xs[j] + t * C;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (vec) Vec4<T>::load(x + c0, v);
      else for (int i = 0; i < nc; ++i) v[i] = to_float(x[c0 + i]);
      for (int i = 0; i < nc; ++i) acc[i] = fmaf(v[i] * r[j], a.ws[j][c0 + i], acc[i]);
    }
    for (int i = 0; i < 4; ++i) acc[i] *= inv_n;
    if (vec) Vec4<T>::store(out + c0, acc);
    else for (int i = 0; i < nc; ++i) out[c0 + i] = from_float<T>(acc[i]);
  }
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_hyper_step(float* streams, long long stream_stride, int n_streams, int n_tokens, int channels,
                              const float* init_from, const void* y, int y_dtype, const float* mix, const float* out_w,
                              const float* in_w, const float* norm_w, float eps, void* h_out, int h_dtype,
                              float* sum_out, void* stream) {
  FTK_REQUIRE(dtype_ok(y_dtype) && dtype_ok(h_dtype), "hyper_step: bad dtype");
  FTK_REQUIRE(n_streams >= 1 && n_streams <= kHyperMaxStreams, "hyper_step: %d streams (1 to %d taken)", n_streams,
              kHyperMaxStreams);
  FTK_REQUIRE(n_tokens >= 0 && channels >= 1 && stream_stride >= (long long)n_tokens * channels, "hyper_step: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(streams, "hyper_step: null pointer");
  FTK_REQUIRE((y == nullptr) == (mix == nullptr) && (y == nullptr) == (out_w == nullptr),
              "hyper_step: a result to write comes with its mix matrix and output weights");
  FTK_REQUIRE((in_w == nullptr) == (norm_w == nullptr) && (in_w == nullptr) == (h_out == nullptr),
              "hyper_step: a read comes with input weights, a norm weight and an output");
  FTK_REQUIRE((((uintptr_t)streams | (uintptr_t)init_from | (uintptr_t)y | (uintptr_t)h_out | (uintptr_t)sum_out) & 15) == 0,
              "hyper_step: 16-byte aligned rows only");
  HyperArgs a{streams, stream_stride, n_streams, n_tokens, channels, init_from, y, mix, out_w, in_w, norm_w, eps, h_out, sum_out};
  const size_t smem = ((size_t)((channels + 3) & ~3) + 33) * sizeof(float);
  FTK_REQUIRE(smem <= 200 * 1024, "hyper_step: rows of %d channels do not fit shared memory", channels);
  cudaStream_t s = (cudaStream_t)stream;
#define FTK_HYPER_N(TY, TH, N)                                                                     \
  do {                                                                                             \
    auto kern = hyper_step_kernel<TY, TH, N>;                                                      \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    FTK_LAUNCH(kern, n_tokens, kHyperThreads, smem, s, a);                                         \
  } while (0)
#define FTK_HYPER(TY, TH)                          \
  do {                                             \
    if (n_streams == 1) FTK_HYPER_N(TY, TH, 1);    \
    else if (n_streams == 2) FTK_HYPER_N(TY, TH, 2); \
    else if (n_streams <= 4) FTK_HYPER_N(TY, TH, 4); \
    else FTK_HYPER_N(TY, TH, 8);                   \
  } while (0)
  if (y_dtype == FTK_F32 && h_dtype == FTK_F32) FTK_HYPER(float, float);
  else if (y_dtype == FTK_F32) FTK_HYPER(float, __nv_bfloat16);
  else if (h_dtype == FTK_F32) FTK_HYPER(__nv_bfloat16, float);
  else FTK_HYPER(__nv_bfloat16, __nv_bfloat16);
#undef FTK_HYPER
#undef FTK_HYPER_N
  FTK_LAUNCH_CHECK("hyper_step");
  return 0;
}

extern "C" int ftk_norm_mean(const void* const* xs, const float* const* ws, int n, int dtype, float eps, void* out,
                             int n_tokens, int channels, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "norm_mean: bad dtype %d", dtype);
  FTK_REQUIRE(n >= 1 && n <= 4 && n_tokens >= 0 && channels >= 1, "norm_mean: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(xs && ws && out, "norm_mean: null pointer");
  NormMeanArgs a;
  uintptr_t bits = (uintptr_t)out;
  for (int i = 0; i < 4; ++i) {
    a.xs[i] = i < n ? xs[i] : nullptr;
    a.ws[i] = i < n ? ws[i] : nullptr;
    FTK_REQUIRE(i >= n || (xs[i] && ws[i]), "norm_mean: null pointer");
    bits |= (uintptr_t)a.xs[i];
  }
  FTK_REQUIRE((bits & 15) == 0, "norm_mean: 16-byte aligned rows only");
  a.n = n; a.C = channels; a.eps = eps; a.out = out;
  const size_t rows = (size_t)n * channels * dtype_size(dtype);
  a.keep = rows <= 40 * 1024 && channels % 4 == 0 ? 1 : 0;  // (what fits beside the scratch without asking for more shared memory)
  const size_t smem = 36 * sizeof(float) + (a.keep ? rows : 0);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == FTK_F32) FTK_LAUNCH(norm_mean_kernel<float>, n_tokens, kHyperThreads, smem, s, a);
  else FTK_LAUNCH(norm_mean_kernel<__nv_bfloat16>, n_tokens, kHyperThreads, smem, s, a);
  FTK_LAUNCH_CHECK("norm_mean");
  return 0;
}
