// What a state-space layer (and any layer that convolves its projections) needs around the recurrence.
//
// conv_act: out[t, c] = act(bias[c] + sum_j w[c, j] * in(t - taps + 1 + j, c)) over each request's own inputs, on
// rows of the engine's type that may be a view of a projection's columns.  As in short_conv, tiles are aligned to
// requests: tile 0 of a request reads the request's last taps - 1 inputs from its state slot (zeros before the
// sequence starts), and the same threads write the new ones afterwards.  Sums and the activation are 32-bit.
//
// ssm_gates: step sizes dt = softplus(dt_raw + dt_bias) and decays exp(-exp(A_log) dt) per (token, head), 32-bit.
//
// ssm_output, a block per (token, norm group): y = (o + D_h x) silu(z), divided by the root mean square of its
// group, times a weight.
#include "common.cuh"

namespace ftk {

constexpr int kCaTile = 32;      // tokens per tile (at least taps - 1)
constexpr int kCaMaxTaps = 16;
constexpr int kCaThreads = 128;  // four channels a thread

__device__ __forceinline__ float softplus_f(float z) { return z > 0.f ? z + log1pf(expf(-z)) : log1pf(expf(z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

template <typename T, int TAPS>
__global__ void __launch_bounds__(kCaThreads)
conv_act_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ w, const float* __restrict__ bias,
                int taps, int act, float* __restrict__ state, const int32_t* __restrict__ state_slots,
                const int32_t* __restrict__ seg_info, int n_segs, int n_slots, T* __restrict__ out, int n_tokens, int C,
                int vec_ok) {
  pdl_wait();
  pdl_trigger();
  const int c0 = (blockIdx.y * kCaThreads + threadIdx.x) * 4;
  if (c0 >= C) return;
  const int nc = min(4, C - c0);
  const bool vec = vec_ok && nc == 4;
  if (TAPS > 0) taps = TAPS;
  // the thread's taps and bias first: they wait for nothing, and the search for the block's request runs beside them
  constexpr int kMost = TAPS > 0 ? TAPS : kCaMaxTaps;
  float wt[kMost][4], bs[4];
#pragma unroll
  for (int j = 0; j < (TAPS > 0 ? TAPS : taps); ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) wt[j][i] = i < nc ? w[(size_t)(c0 + i) * taps + j] : 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) bs[i] = (bias && i < nc) ? bias[c0 + i] : 0.f;
  int tile = blockIdx.x, seg = 0, q_start = 0, q_len = 0, kv_len = 0;
  for (; seg < n_segs; ++seg) {
    q_start = seg_info[seg * 4]; q_len = seg_info[seg * 4 + 1]; kv_len = seg_info[seg * 4 + 2];
    const int n = q_len > 0 ? (q_len + kCaTile - 1) / kCaTile : 0;
    if (tile < n) break;
    tile -= n;
  }
  if (seg >= n_segs || q_start < 0 || q_start + q_len > n_tokens || kv_len < q_len) return;
  const int keep = taps - 1;
  const int slot = state_slots[seg];
  const bool has_slot = state && slot >= 0 && slot < n_slots;
  const int before = kv_len - q_len;
  float* st = has_slot ? state + ((size_t)slot * keep) * C + c0 : nullptr;  // row r: the input `keep - r` places back
  const bool first = tile == 0;
  const int t0 = tile * kCaTile, t1 = min(q_len, t0 + kCaTile);
  // input `s` places into the request's tokens of this step (negative: before them)
  auto input = [&](int s, float (&v)[4]) {
    if (s >= 0) {
      const T* r = x + (size_t)(q_start + s) * x_stride + c0;
      if (vec) Vec4<T>::load(r, v);
      else for (int i = 0; i < 4; ++i) v[i] = i < nc ? to_float(r[i]) : 0.f;
    } else {
      const int r = keep + s;  // the slot's row
      for (int i = 0; i < 4; ++i) v[i] = (st && before > 0 && r >= 0 && -s <= before && i < nc) ? st[(size_t)r * C + i] : 0.f;
    }
  };
  constexpr int K = TAPS > 1 ? TAPS - 1 : 1;
  float win[K][4];  // TAPS > 1: the inputs t - K .. t - 1, oldest first
  float tail[kMost][4];  // what tile 0 read of the slot and must hand on when the step is shorter than the state
  if (first) {
    for (int r = 0; r < keep; ++r) input(r - keep, tail[r]);
  }
  if (TAPS > 1) {
#pragma unroll
    for (int r = 0; r < K; ++r) {
      if (first) {
#pragma unroll
        for (int i = 0; i < 4; ++i) win[r][i] = tail[r][i];
      } else {
        input(t0 - K + r, win[r]);
      }
    }
  }
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {  // (unrolled: several rows' loads are then in flight per thread)
    float cur[4], acc[4];
    input(t, cur);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = bs[i];
    if (TAPS > 1) {
#pragma unroll
      for (int r = 0; r < K; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = fmaf(wt[r][i], win[r][i], acc[i]);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(wt[K][i], cur[i], acc[i]);
#pragma unroll
      for (int r = 0; r + 1 < K; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) win[r][i] = win[r + 1][i];
#pragma unroll
      for (int i = 0; i < 4; ++i) win[K - 1][i] = cur[i];
    } else {
      for (int j = 0; j < taps; ++j) {
        const int s = t - keep + j;
        float in[4];
        if (s >= 0 || !first) {
          if (s < 0) continue;  // (tiles hold at least `keep` tokens: never reached)
          if (j == keep) { for (int i = 0; i < 4; ++i) in[i] = cur[i]; }
          else input(s, in);
        } else {
          for (int i = 0; i < 4; ++i) in[i] = tail[keep + s][i];
        }
        for (int i = 0; i < 4; ++i) acc[i] = fmaf(wt[j][i], in[i], acc[i]);
      }
    }
    if (act == 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = silu_f(acc[i]);
    }
    T* o = out + (size_t)(q_start + t) * C + c0;
    if (vec) Vec4<T>::store(o, acc);
    else for (int i = 0; i < nc; ++i) o[i] = from_float<T>(acc[i]);
  }
  if (first && st) {  // the new state: the request's last `keep` inputs, oldest first
    for (int r = 0; r < keep; ++r) {
      const int s = q_len - keep + r;
      float v[4];
      if (s >= 0) input(s, v);
      else for (int i = 0; i < 4; ++i) v[i] = tail[keep + s][i];
      for (int i = 0; i < nc; ++i) st[(size_t)r * C + i] = v[i];
    }
  }
}

template <typename T>
__global__ void ssm_gates_kernel(const T* __restrict__ dt, long long dt_stride, const float* __restrict__ dt_bias,
                                 const float* __restrict__ a_log, float* __restrict__ dt_out, float* __restrict__ decay_out,
                                 int n_tokens, int H) {
  pdl_wait();
  pdl_trigger();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_tokens * H) return;
  const int t = (int)(i / H), h = (int)(i % H);
  const float step = softplus_f(to_float(dt[(size_t)t * dt_stride + h]) + dt_bias[h]);
  dt_out[i] = step;
  decay_out[i] = expf(-expf(a_log[h]) * step);
}

template <typename T>
__global__ void __launch_bounds__(256)
ssm_output_kernel(const float* __restrict__ o32, const T* __restrict__ x, long long x_stride, const float* __restrict__ d_skip,
                  const T* __restrict__ z, long long z_stride, const float* __restrict__ norm_w, int norm_groups, float eps,
                  T* __restrict__ out, int H, int P) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float sm[];  // [L] the gated values of this group, then 33 floats of scratch
  const size_t t = blockIdx.x;
  const int g = blockIdx.y;
  const int I = H * P, L = I / norm_groups, base = g * L;
  float* scratch = sm + ((L + 3) & ~3);
  float ss = 0.f;
  for (int j = threadIdx.x; j < L; j += blockDim.x) {
    const int c = base + j;
    const float xv = to_float(x[t * x_stride + c]), zv = to_float(z[t * z_stride + c]);
    const float y = fmaf(d_skip[c / P], xv, o32[t * I + c]) * silu_f(zv);
    sm[j] = y;
    ss = fmaf(y, y, ss);
  }
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / (float)L + eps);
  for (int j = threadIdx.x; j < L; j += blockDim.x)
    out[t * I + base + j] = from_float<T>(sm[j] * r * norm_w[base + j]);
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_conv_act(const void* x, long long x_stride, int dtype, const float* w, const float* bias, int taps,
                            int act, float* state, int n_slots, const int32_t* state_slots, const int32_t* seg_info,
                            int n_segs, void* out, int n_tokens, int channels, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "conv_act: bad dtype %d", dtype);
  FTK_REQUIRE(taps >= 1 && taps <= kCaMaxTaps && taps - 1 <= kCaTile, "conv_act: %d taps (1 to %d taken)", taps, kCaMaxTaps);
  FTK_REQUIRE(n_tokens >= 0 && channels >= 1 && n_segs >= 1 && x_stride >= channels && (act == 0 || act == 1),
              "conv_act: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(x && w && out && seg_info && state_slots && (taps == 1 || state), "conv_act: null pointer");
  const int quad = 4 * dtype_size(dtype);
  const int vec_ok = channels % 4 == 0 && x_stride % 4 == 0 && (uintptr_t)x % quad == 0 && (uintptr_t)out % quad == 0;
  dim3 grid((n_tokens + kCaTile - 1) / kCaTile + n_segs, (channels + kCaThreads * 4 - 1) / (kCaThreads * 4));
  cudaStream_t s = (cudaStream_t)stream;
#define FTK_CA(TY, N)                                                                                                  \
  FTK_LAUNCH((conv_act_kernel<TY, N>), grid, kCaThreads, 0, s, (const TY*)x, x_stride, w, bias, taps, act, state,    \
             state_slots, seg_info, n_segs, n_slots, (TY*)out, n_tokens, channels, vec_ok)
#define FTK_CA_TAPS(TY)                \
  do {                                 \
    if (taps == 2) FTK_CA(TY, 2);      \
    else if (taps == 3) FTK_CA(TY, 3); \
    else if (taps == 4) FTK_CA(TY, 4); \
    else FTK_CA(TY, 0);                \
  } while (0)
  if (dtype == FTK_F32) FTK_CA_TAPS(float);
  else FTK_CA_TAPS(__nv_bfloat16);
#undef FTK_CA_TAPS
#undef FTK_CA
  FTK_LAUNCH_CHECK("conv_act");
  return 0;
}

extern "C" int ftk_ssm_gates(const void* dt, long long dt_stride, int dtype, const float* dt_bias, const float* a_log,
                             float* dt_out, float* decay_out, int n_tokens, int n_heads, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "ssm_gates: bad dtype %d", dtype);
  FTK_REQUIRE(n_tokens >= 0 && n_heads >= 1 && dt_stride >= n_heads, "ssm_gates: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(dt && dt_bias && a_log && dt_out && decay_out, "ssm_gates: null pointer");
  const long long n = (long long)n_tokens * n_heads;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == FTK_F32) FTK_LAUNCH(ssm_gates_kernel<float>, blocks, 256, 0, s, (const float*)dt, dt_stride, dt_bias, a_log, dt_out, decay_out, n_tokens, n_heads);
  else FTK_LAUNCH(ssm_gates_kernel<__nv_bfloat16>, blocks, 256, 0, s, (const __nv_bfloat16*)dt, dt_stride, dt_bias, a_log, dt_out, decay_out, n_tokens, n_heads);
  FTK_LAUNCH_CHECK("ssm_gates");
  return 0;
}

extern "C" int ftk_ssm_output(const float* o32, const void* x, long long x_stride, const float* d_skip, const void* z,
                              long long z_stride, int dtype, const float* norm_w, int norm_groups, float eps, void* out,
                              int n_tokens, int n_heads, int vdim, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "ssm_output: bad dtype %d", dtype);
  const long long inner = (long long)n_heads * vdim;
  FTK_REQUIRE(n_tokens >= 0 && n_heads >= 1 && vdim >= 1 && norm_groups >= 1 && norm_groups <= 65535 &&
              inner % norm_groups == 0 && x_stride >= inner && z_stride >= inner, "ssm_output: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(o32 && x && d_skip && z && norm_w && out, "ssm_output: null pointer");
  const int L = (int)(inner / norm_groups);
  const size_t smem = ((size_t)((L + 3) & ~3) + 33) * sizeof(float);
  FTK_REQUIRE(smem <= 200 * 1024, "ssm_output: norm groups of %d channels do not fit shared memory", L);
  dim3 grid(n_tokens, norm_groups);
  cudaStream_t s = (cudaStream_t)stream;
#define FTK_SSM_OUT(TY)                                                                                         \
  do {                                                                                                          \
    auto kern = ssm_output_kernel<TY>;                                                                          \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    FTK_LAUNCH(kern, grid, 256, smem, s, o32, (const TY*)x, x_stride, d_skip, (const TY*)z, z_stride, norm_w,  \
               norm_groups, eps, (TY*)out, n_heads, vdim);                                                      \
  } while (0)
  if (dtype == FTK_F32) FTK_SSM_OUT(float);
  else FTK_SSM_OUT(__nv_bfloat16);
#undef FTK_SSM_OUT
  FTK_LAUNCH_CHECK("ssm_output");
  return 0;
}
