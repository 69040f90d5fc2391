// Short causal convolution over time with a per-request state, and the learned mix of all layer outputs so far.
//
// short_conv: out[t, c] = x[t, c] + sum_j w[c, j] * in(t - taps + 1 + j, c), where in() is the request's own input at
// that place: a row of this step, or, before the step's first token, one of the request's last taps - 1 inputs
// kept in its state slot (zeros before the sequence starts).  x is the 32-bit stream, the sum is 32-bit, the
// result is rounded once to the engine's type.  Tiles are aligned to requests: tile 0 of a request is the only
// one that reads the old state, and the same threads (a thread owns its channels) write the new one afterwards,
// so one launch both uses and advances the state.
//
// depth_mix: hist[n] = x; x = sum_{j <= n} mix[j] * hist[j], all 32-bit, in the order j = 0, 1, ..., n.
#include "common.cuh"

namespace ftk {

constexpr int kConvTile = 16;     // tokens per tile (at least taps - 1)
constexpr int kConvMaxTaps = 16;
constexpr int kConvThreads = 128; // four channels a thread

// TAPS > 0: the tap count at compile time.  A thread then keeps its channels' last TAPS - 1 inputs in registers and
// fetches every row of the stream once; TAPS == 0 takes any count and fetches a row once per tap (from L1).
template <typename T, int TAPS>
__global__ void __launch_bounds__(kConvThreads)
short_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, int taps, float* __restrict__ state,
                  const int32_t* __restrict__ state_slots, const int32_t* __restrict__ seg_info, int n_segs, int n_slots,
                  T* __restrict__ out, int n_tokens, int C) {
  pdl_wait();
  pdl_trigger();
  // which request and which of its tiles
  int tile = blockIdx.x, seg = 0, q_start = 0, q_len = 0, kv_len = 0;
  for (; seg < n_segs; ++seg) {
    q_start = seg_info[seg * 4]; q_len = seg_info[seg * 4 + 1]; kv_len = seg_info[seg * 4 + 2];
    const int n = q_len > 0 ? (q_len + kConvTile - 1) / kConvTile : 0;
    if (tile < n) break;
    tile -= n;
  }
  if (seg >= n_segs || q_start < 0 || q_start + q_len > n_tokens || kv_len < q_len) return;
  const int c0 = (blockIdx.y * kConvThreads + threadIdx.x) * 4;
  if (c0 >= C) return;
  const int nc = min(4, C - c0);
  const bool vec = nc == 4 && (C & 3) == 0;
  if (TAPS > 0) taps = TAPS;
  const int keep = taps - 1;
  const int slot = state_slots[seg];
  const bool has_slot = slot >= 0 && slot < n_slots;
  const int before = kv_len - q_len;                       // tokens the request held before this step
  float* st = has_slot ? state + ((size_t)slot * keep) * C + c0 : nullptr;  // row i: the input `keep - i` places back
  constexpr int kMost = TAPS > 0 ? TAPS : kConvMaxTaps;
  float wt[kMost][4];
#pragma unroll
  for (int j = 0; j < (TAPS > 0 ? TAPS : taps); ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) wt[j][i] = i < nc ? w[(size_t)(c0 + i) * taps + j] : 0.f;
  float old[kMost][4];                                     // the slot's rows, read by tile 0 only
  const bool first = tile == 0;
  if (first) {
#pragma unroll
    for (int r = 0; r < (TAPS > 0 ? TAPS - 1 : keep); ++r)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        old[r][i] = (st && before > 0 && i < nc && keep - r <= before) ? st[(size_t)r * C + i] : 0.f;
  }
  const int t0 = tile * kConvTile, t1 = min(q_len, t0 + kConvTile);
  if (TAPS > 1 && vec) {
    constexpr int K = TAPS > 1 ? TAPS - 1 : 1;
    float win[K][4];                                       // inputs t - K .. t - 1, oldest first
#pragma unroll
    for (int r = 0; r < K; ++r) {
      if (first) {
#pragma unroll
        for (int i = 0; i < 4; ++i) win[r][i] = old[r][i];
      } else {
        Vec4<float>::load(x + (size_t)(q_start + t0 - K + r) * C + c0, win[r]);
      }
    }
    const float* row = x + (size_t)(q_start + t0) * C + c0;
    T* o = out + (size_t)(q_start + t0) * C + c0;
#pragma unroll 4
    for (int t = t0; t < t1; ++t, row += C, o += C) {
      float cur[4], acc[4];
      Vec4<float>::load(row, cur);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = cur[i];        // the same order of sums as the form for any count
#pragma unroll
      for (int r = 0; r < K; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = fmaf(wt[r][i], win[r][i], acc[i]);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(wt[K][i], cur[i], acc[i]);
      Vec4<T>::store(o, acc);
#pragma unroll
      for (int r = 0; r + 1 < K; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) win[r][i] = win[r + 1][i];
#pragma unroll
      for (int i = 0; i < 4; ++i) win[K - 1][i] = cur[i];
    }
  } else
  for (int t = t0; t < t1; ++t) {
    float acc[4];
    const float* row = x + (size_t)(q_start + t) * C + c0;
    if (vec) Vec4<float>::load(row, acc);
    else for (int i = 0; i < 4; ++i) acc[i] = i < nc ? row[i] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int s = t - keep + j;                          // place among the step's tokens of this request
      float in[4];
      if (s >= 0) {
        const float* r2 = x + (size_t)(q_start + s) * C + c0;
        if (vec) Vec4<float>::load(r2, in);
        else for (int i = 0; i < 4; ++i) in[i] = i < nc ? r2[i] : 0.f;
      } else if (first) {                                  // s in [-keep, -1]: the slot's row keep + s
        for (int i = 0; i < 4; ++i) in[i] = old[keep + s][i];
      } else {
        continue;                                          // (tiles hold at least `keep` tokens: never reached)
      }
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(wt[j][i], in[i], acc[i]);
    }
    T* o = out + (size_t)(q_start + t) * C + c0;
    if (vec) Vec4<T>::store(o, acc);
    else for (int i = 0; i < nc; ++i) o[i] = from_float<T>(acc[i]);
  }
  if (first && st) {  // the new state: the last `keep` inputs of the request, oldest first
    for (int r = 0; r < keep; ++r) {
      const int s = q_len - keep + r;                      // place among the step's tokens, negative: an old row
      float v[4];
      if (s >= 0) {
        const float* r2 = x + (size_t)(q_start + s) * C + c0;
        for (int i = 0; i < 4; ++i) v[i] = i < nc ? r2[i] : 0.f;
      } else {
        for (int i = 0; i < 4; ++i) v[i] = old[keep + s][i];
      }
      for (int i = 0; i < nc; ++i) st[(size_t)r * C + i] = v[i];
    }
  }
}

__global__ void depth_mix_kernel(float* __restrict__ hist, long long layer_stride, int n_prev,
                                 const float* __restrict__ mix, float* __restrict__ x, long long n) {
  pdl_wait();
  pdl_trigger();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float cur[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
  const bool vec = i + 4 <= n;
  if (vec) Vec4<float>::load(x + i, cur);
  else for (int k = 0; k < 4; ++k) cur[k] = i + k < n ? x[i + k] : 0.f;
  for (int j = 0; j < n_prev; ++j) {
    const float m = __ldg(mix + j);
    float v[4];
    const float* src = hist + (size_t)j * layer_stride + i;
    if (vec) Vec4<float>::load(src, v);
    else for (int k = 0; k < 4; ++k) v[k] = i + k < n ? src[k] : 0.f;
    for (int k = 0; k < 4; ++k) acc[k] = fmaf(m, v[k], acc[k]);
  }
  const float m = __ldg(mix + n_prev);
  float* dst = hist + (size_t)n_prev * layer_stride + i;
  if (vec) Vec4<float>::store(dst, cur);
  else for (int k = 0; k < 4; ++k) if (i + k < n) dst[k] = cur[k];
  for (int k = 0; k < 4; ++k) acc[k] = fmaf(m, cur[k], acc[k]);
  if (vec) Vec4<float>::store(x + i, acc);
  else for (int k = 0; k < 4; ++k) if (i + k < n) x[i + k] = acc[k];
}

// out[r, :] = weights[sorted_routes[r]] * h[sorted_routes[r] / top_k, :] (32-bit product, rounded once)
template <typename T>
__global__ void moe_gather_scaled_kernel(const T* __restrict__ h, const int32_t* __restrict__ sorted_routes,
                                         const float* __restrict__ weights, int top_k, int hidden, int n_tokens,
                                         T* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int route = sorted_routes[r];
  const int t = route / top_k;
  if (route < 0 || t >= n_tokens) return;
  const float wgt = weights[route];
  const T* src = h + (size_t)t * hidden;
  T* dst = out + (size_t)r * hidden;
  if ((hidden & 3) == 0 && ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float v[4];
      Vec4<T>::load(src + i, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] *= wgt;
      Vec4<T>::store(dst + i, v);
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_float<T>(wgt * to_float(src[i]));
}

// x <- max(x, 0)^2 in place
template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, long long n) {
  pdl_wait();
  pdl_trigger();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  if (i + 4 <= n && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    float v[4];
    Vec4<T>::load(x + i, v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[k] = fmaxf(v[k], 0.f);
      v[k] *= v[k];
    }
    Vec4<T>::store(x + i, v);
    return;
  }
  for (long long j = i; j < n && j < i + 4; ++j) {
    const float v = fmaxf(to_float(x[j]), 0.f);
    x[j] = from_float<T>(v * v);
  }
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_short_conv(const float* x, const float* w, int taps, float* state, int n_slots,
                              const int32_t* state_slots, const int32_t* seg_info, int n_segs, void* out, int dtype,
                              int n_tokens, int channels, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "short_conv: bad dtype %d", dtype);
  FTK_REQUIRE(taps >= 1 && taps <= kConvMaxTaps && taps - 1 <= kConvTile, "short_conv: %d taps (1 to %d taken)", taps,
              kConvMaxTaps);
  FTK_REQUIRE(n_tokens >= 0 && channels >= 1 && n_segs >= 1, "short_conv: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(x && w && out && seg_info && state_slots && (taps == 1 || state), "short_conv: null pointer");
  FTK_REQUIRE((((uintptr_t)x | (uintptr_t)out) & 15) == 0, "short_conv: 16-byte aligned rows only");
  // tiles: every request's tokens rounded up, so at most n_tokens / tile + n_segs
  dim3 grid((n_tokens + kConvTile - 1) / kConvTile + n_segs, (channels + kConvThreads * 4 - 1) / (kConvThreads * 4));
  cudaStream_t s = (cudaStream_t)stream;
#define FTK_CONV(TY, N)                                                                                              \
  FTK_LAUNCH((short_conv_kernel<TY, N>), grid, kConvThreads, 0, s, x, w, taps, state, state_slots, seg_info, n_segs, \
             n_slots, (TY*)out, n_tokens, channels)
#define FTK_CONV_TAPS(TY)                  \
  do {                                     \
    if (taps == 2) FTK_CONV(TY, 2);        \
    else if (taps == 3) FTK_CONV(TY, 3);   \
    else if (taps == 4) FTK_CONV(TY, 4);   \
    else FTK_CONV(TY, 0);                  \
  } while (0)
  if (dtype == FTK_F32) FTK_CONV_TAPS(float);
  else FTK_CONV_TAPS(__nv_bfloat16);
#undef FTK_CONV_TAPS
#undef FTK_CONV
  FTK_LAUNCH_CHECK("short_conv");
  return 0;
}

extern "C" int ftk_depth_mix(float* hist, long long layer_stride, int n_prev, const float* mix, float* x, long long n,
                             void* stream) {
  FTK_REQUIRE(n_prev >= 0 && n >= 0 && layer_stride >= n, "depth_mix: bad sizes");
  if (n == 0) return 0;
  FTK_REQUIRE(hist && mix && x, "depth_mix: null pointer");
  FTK_REQUIRE((((uintptr_t)hist | (uintptr_t)x) & 15) == 0 && layer_stride % 4 == 0, "depth_mix: 16-byte aligned rows only");
  const long long quads = (n + 3) / 4;
  FTK_LAUNCH(depth_mix_kernel, (unsigned)((quads + 255) / 256), 256, 0, (cudaStream_t)stream, hist, layer_stride, n_prev, mix, x,
             n);
  FTK_LAUNCH_CHECK("depth_mix");
  return 0;
}

extern "C" int ftk_moe_gather_scaled(const void* h, int dtype, const int32_t* sorted_routes, const float* weights,
                                     int n_routes, int top_k, int hidden, void* out, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "moe_gather_scaled: bad dtype %d", dtype);
  FTK_REQUIRE(n_routes >= 0 && top_k > 0 && hidden > 0 && n_routes % top_k == 0, "moe_gather_scaled: bad sizes");
  if (n_routes == 0) return 0;
  FTK_REQUIRE(h && sorted_routes && weights && out, "moe_gather_scaled: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int n_tokens = n_routes / top_k;
  const int threads = hidden >= 2048 ? 256 : 128;
  if (dtype == FTK_F32)
    FTK_LAUNCH(moe_gather_scaled_kernel<float>, n_routes, threads, 0, s, (const float*)h, sorted_routes, weights, top_k, hidden,
               n_tokens, (float*)out);
  else
    FTK_LAUNCH(moe_gather_scaled_kernel<__nv_bfloat16>, n_routes, threads, 0, s, (const __nv_bfloat16*)h, sorted_routes, weights,
               top_k, hidden, n_tokens, (__nv_bfloat16*)out);
  FTK_LAUNCH_CHECK("moe_gather_scaled");
  return 0;
}

extern "C" int ftk_relu2(void* x, int dtype, long long n, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype) && n >= 0, "relu2: bad arguments");
  if (n == 0) return 0;
  FTK_REQUIRE(x, "relu2: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)(((n + 3) / 4 + 255) / 256);
  if (dtype == FTK_F32) FTK_LAUNCH(relu2_kernel<float>, blocks, 256, 0, s, (float*)x, n);
  else FTK_LAUNCH(relu2_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)x, n);
  FTK_LAUNCH_CHECK("relu2");
  return 0;
}
