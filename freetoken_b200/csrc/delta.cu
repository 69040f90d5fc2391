// Gated delta rule: a matrix state per (request, head) that every token first decays, then corrects towards its
// value along its key, then reads with its query:
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
// beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)); q and k are made unit vectors per head first
// (x / sqrt(sum x^2 + eps)), q also scaled.  State, gates, norms and all sums are 32-bit.
//
// The correction u needs S^T k of the state as the token finds it, so a request's tokens run one after the other.
// What runs side by side are the state's columns: a block owns 32 value columns of one (request, head); four
// neighbouring lanes share a column, each keeping a quarter of its key channels in registers, so that S^T k and
// S^T q are a thread's own sums plus two shuffles and no thread waits for another warp.  The tokens' q, k (normed
// as they are staged), v and gates come through shared memory 16 tokens at a time; the outputs of a batch leave
// together.  A decode step is the same kernel with one token per request.
#include "common.cuh"

namespace ftk {

constexpr int kDeltaBatch = 16;   // tokens staged at a time
constexpr int kDeltaCols = 32;    // value columns per block
constexpr int kDeltaThreads = 128;

struct DeltaArgs {
  const void* q; const void* k; const void* v; const void* b; const void* a;
  long long q_stride, k_stride, v_stride, b_stride, a_stride;
  const float* a_log; const float* dt_bias;
  float q_scale, unit_eps;
  float* state; int n_slots;
  const int32_t* state_slots; const int32_t* seg_info; int n_segs;
  float* out; int n_tokens, H, G, D, Dv;
};

__device__ __forceinline__ float delta_softplus(float z) { return z > 0.f ? z + log1pf(expf(-z)) : log1pf(expf(z)); }

template <typename T, int DPT>
__global__ void __launch_bounds__(kDeltaThreads) delta_scan_kernel(DeltaArgs a) {
  pdl_wait();
  pdl_trigger();
  constexpr int Dp = DPT * 4;  // padded key channels
  __shared__ __align__(16) float sq[kDeltaBatch][Dp];
  __shared__ __align__(16) float sk[kDeltaBatch][Dp];
  __shared__ float sv[kDeltaBatch][kDeltaCols];
  __shared__ float so[kDeltaBatch][kDeltaCols];
  __shared__ float sbeta[kDeltaBatch], sg[kDeltaBatch];
  const int seg = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * kDeltaCols;
  const int D = a.D, Dv = a.Dv;
  const int q_start = a.seg_info[seg * 4], q_len = a.seg_info[seg * 4 + 1], kv_len = a.seg_info[seg * 4 + 2];
  if (q_len <= 0 || q_start < 0 || q_start + q_len > a.n_tokens || kv_len < q_len) return;
  const int slot = a.state_slots[seg];
  if (slot < 0 || slot >= a.n_slots) return;
  const int hqk = h / (a.H / a.G);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slice = lane & 3, lcol = warp * 8 + (lane >> 2), col = col0 + lcol;
  const int d0 = slice * DPT;
  const bool live = col < Dv;
  float* st = a.state + ((size_t)slot * a.H + h) * D * Dv;
  const bool fresh = kv_len == q_len;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) s[i] = (!fresh && live && d0 + i < D) ? st[(size_t)(d0 + i) * Dv + col] : 0.f;
  const T* qb = (const T*)a.q; const T* kb = (const T*)a.k; const T* vb = (const T*)a.v;
  const T* bb = (const T*)a.b; const T* ab = (const T*)a.a;
  const float neg_rate = -expf(a.a_log[h]), bias = a.dt_bias[h];
  for (int b0 = 0; b0 < q_len; b0 += kDeltaBatch) {
    const int nb = min(kDeltaBatch, q_len - b0);
    __syncthreads();  // the batch before is read
    for (int i = threadIdx.x; i < nb * Dp; i += kDeltaThreads) {
      const int t = i / Dp, d = i % Dp;
      const size_t tok = (size_t)(q_start + b0 + t);
      sq[t][d] = d < D ? to_float(qb[tok * a.q_stride + (size_t)hqk * D + d]) : 0.f;
      sk[t][d] = d < D ? to_float(kb[tok * a.k_stride + (size_t)hqk * D + d]) : 0.f;
    }
    for (int i = threadIdx.x; i < nb * kDeltaCols; i += kDeltaThreads) {
      const int t = i / kDeltaCols, j = i % kDeltaCols;
      const size_t tok = (size_t)(q_start + b0 + t);
      sv[t][j] = col0 + j < Dv ? to_float(vb[tok * a.v_stride + (size_t)h * Dv + col0 + j]) : 0.f;
    }
    if (threadIdx.x < nb) {
      const size_t tok = (size_t)(q_start + b0 + threadIdx.x);
      const float bl = to_float(bb[tok * a.b_stride + h]), al = to_float(ab[tok * a.a_stride + h]);
      sbeta[threadIdx.x] = 1.f / (1.f + expf(-bl));
      sg[threadIdx.x] = expf(neg_rate * delta_softplus(al + bias));
    }
    __syncthreads();
    // unit vectors: a warp takes a token at a time
    for (int t = warp; t < nb; t += kDeltaThreads / 32) {
      float s2q = 0.f, s2k = 0.f;
      for (int d = lane; d < Dp; d += 32) { s2q = fmaf(sq[t][d], sq[t][d], s2q); s2k = fmaf(sk[t][d], sk[t][d], s2k); }
      s2q = warp_sum(s2q); s2k = warp_sum(s2k);
      const float rq = rsqrtf(s2q + a.unit_eps) * a.q_scale, rk = rsqrtf(s2k + a.unit_eps);
      for (int d = lane; d < Dp; d += 32) { sq[t][d] *= rq; sk[t][d] *= rk; }
    }
    __syncthreads();
    for (int t = 0; t < nb; ++t) {
      const float g = sg[t], beta = sbeta[t], vj = sv[t][lcol];
      const float4* k4 = reinterpret_cast<const float4*>(&sk[t][d0]);
      const float4* q4 = reinterpret_cast<const float4*>(&sq[t][d0]);
      float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {
        const float4 kv = k4[i];
        r0 = fmaf(s[4 * i + 0], kv.x, r0); r1 = fmaf(s[4 * i + 1], kv.y, r1);
        r2 = fmaf(s[4 * i + 2], kv.z, r2); r3 = fmaf(s[4 * i + 3], kv.w, r3);
      }
      float r = (r0 + r1) + (r2 + r3);
      r += __shfl_xor_sync(0xffffffffu, r, 1);
      r += __shfl_xor_sync(0xffffffffu, r, 2);
      const float u = beta * (vj - g * r);  // S^T k of the decayed state is g times that of the state as found
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {
        const float4 kv = k4[i], qv = q4[i];
        s[4 * i + 0] = fmaf(g, s[4 * i + 0], kv.x * u); o0 = fmaf(s[4 * i + 0], qv.x, o0);
        s[4 * i + 1] = fmaf(g, s[4 * i + 1], kv.y * u); o1 = fmaf(s[4 * i + 1], qv.y, o1);
        s[4 * i + 2] = fmaf(g, s[4 * i + 2], kv.z * u); o2 = fmaf(s[4 * i + 2], qv.z, o2);
        s[4 * i + 3] = fmaf(g, s[4 * i + 3], kv.w * u); o3 = fmaf(s[4 * i + 3], qv.w, o3);
      }
      float o = (o0 + o1) + (o2 + o3);
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (slice == 0) so[t][lcol] = o;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nb * kDeltaCols; i += kDeltaThreads) {
      const int t = i / kDeltaCols, j = i % kDeltaCols;
      if (col0 + j < Dv) a.out[((size_t)(q_start + b0 + t) * a.H + h) * Dv + col0 + j] = so[t][j];
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < D) st[(size_t)(d0 + i) * Dv + col] = s[i];
  }
}

template <typename T>
static int launch_delta(const DeltaArgs& a, cudaStream_t s) {
  dim3 grid(a.n_segs, a.H, (a.Dv + kDeltaCols - 1) / kDeltaCols);
  if (a.D <= 16) FTK_LAUNCH((delta_scan_kernel<T, 4>), grid, kDeltaThreads, 0, s, a);
  else if (a.D <= 32) FTK_LAUNCH((delta_scan_kernel<T, 8>), grid, kDeltaThreads, 0, s, a);
  else if (a.D <= 64) FTK_LAUNCH((delta_scan_kernel<T, 16>), grid, kDeltaThreads, 0, s, a);
  else if (a.D <= 128) FTK_LAUNCH((delta_scan_kernel<T, 32>), grid, kDeltaThreads, 0, s, a);
  else FTK_LAUNCH((delta_scan_kernel<T, 64>), grid, kDeltaThreads, 0, s, a);
  FTK_LAUNCH_CHECK("delta_scan");
  return 0;
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_delta_scan(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                              long long v_stride, const void* b, long long b_stride, const void* a, long long a_stride,
                              int dtype, const float* a_log, const float* dt_bias, float q_scale, float unit_eps,
                              float* state, int n_slots, const int32_t* state_slots, const int32_t* seg_info, int n_segs,
                              float* out, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "delta_scan: bad dtype %d", dtype);
  FTK_REQUIRE(n_tokens >= 0 && n_segs >= 0, "delta_scan: bad counts");
  if (n_tokens == 0 || n_segs == 0) return 0;
  FTK_REQUIRE(n_heads >= 1 && n_heads <= 65535 && n_kv_heads >= 1 && n_heads % n_kv_heads == 0 && dim >= 1 && dim <= 256 &&
              vdim >= 1 && vdim <= 65535 * kDeltaCols,
              "delta_scan: %d heads on %d key heads of %d key and %d value channels are not taken (at most 256 key channels)",
              n_heads, n_kv_heads, dim, vdim);
  FTK_REQUIRE(q && k && v && b && a && a_log && dt_bias && state && state_slots && seg_info && out, "delta_scan: null pointer");
  DeltaArgs d;
  d.q = q; d.k = k; d.v = v; d.b = b; d.a = a;
  d.q_stride = q_stride; d.k_stride = k_stride; d.v_stride = v_stride; d.b_stride = b_stride; d.a_stride = a_stride;
  d.a_log = a_log; d.dt_bias = dt_bias; d.q_scale = q_scale; d.unit_eps = unit_eps;
  d.state = state; d.n_slots = n_slots; d.state_slots = state_slots; d.seg_info = seg_info; d.n_segs = n_segs;
  d.out = out; d.n_tokens = n_tokens; d.H = n_heads; d.G = n_kv_heads; d.D = dim; d.Dv = vdim;
  cudaStream_t s = (cudaStream_t)stream;
  return dtype == FTK_F32 ? launch_delta<float>(d, s) : launch_delta<__nv_bfloat16>(d, s);
}
