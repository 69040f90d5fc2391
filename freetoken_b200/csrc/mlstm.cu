// Matrix memory with exponential gates (the mLSTM of xLSTM) on top of the gated-linear-attention recurrence.
//
// Per head, with log gates i_t (input) and f_t (forget) and the running maximum m_t = max(f_t + m_(t-1), i_t), m_0 = 0:
//   S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T,  n_t likewise with k_t alone,
//   o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6).
// This is a linear recurrence with one decay per head and token, a_t = e^(f_t + m_(t-1) - m_t) <= 1, and keys times
// e^(i_t - m_t) <= 1: the gated-linear-attention kernel runs it, chunk by chunk for long portions, and whatever the cap
// of the gates, S and n stay bounded.  n is the recurrence of one more value column that is 1 for every token.  Two
// kernels around the recurrence kernel, which reads q, k and v where the projection left them, multiplies the keys by
// their factor in 32 bits as it stages them, takes a_t as the head's decay and adds the column of ones itself:
//   gates    per (request, head), a block: m_t, the key factor and the decay of the step's tokens (scans over lanes and warps:
//            F_t = f_1 + ... + f_t, m_t = F_t + max(m_0, max_(s <= t) (i_s - F_s))), m left in the request's slot;
//   output   per (token, head): the division, the head's unit norm, the weight, the sigmoid gate.
#include "common.cuh"

namespace ftk {

__device__ __forceinline__ float capped(float x, float cap) { return cap * tanhf(x / cap); }
__device__ __forceinline__ float log_sigmoid(float z) { return z > 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }

// A block per (request, head); its warps take 128 tokens each, four consecutive ones a lane.  A stretch of tokens
// is summed up by (F, B) = (sum of its forget gates, max over its tokens of i_s - F_s with F_s counted from the stretch's
// start); stretch a in front of stretch b gives (F_a + F_b, max(B_a, B_b - F_a)).  Lanes, then warps, then passes are put
// together that way, and m_t = F_t + max(m_0, B_t) over everything up to t.
__global__ void mlstm_gates_kernel(const float* __restrict__ pre, const float* __restrict__ bias_i,
                                   const float* __restrict__ bias_f, float cap, float* __restrict__ m_state, int n_slots,
                                   const int32_t* __restrict__ state_slots, const int32_t* __restrict__ seg_info, int n_segs,
                                   int H, int n_tokens, float* __restrict__ key_fac, float* __restrict__ decay,
                                   float* __restrict__ m_out) {
  pdl_wait();
  pdl_trigger();
  __shared__ float warp_f[2][8], warp_b[2][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int seg = blockIdx.x / H, h = blockIdx.x - seg * H;
  if (seg >= n_segs) return;
  const int q_start = seg_info[seg * 4], q_len = seg_info[seg * 4 + 1], kv_len = seg_info[seg * 4 + 2];
  if (q_start < 0 || q_len <= 0 || q_start + q_len > n_tokens) return;
  const int slot = state_slots[seg];
  const bool has_slot = slot >= 0 && slot < n_slots;
  float m = (has_slot && kv_len > q_len) ? m_state[(size_t)slot * H + h] : 0.f;
  constexpr int K = 4;
  int pass = 0;
  for (int t0 = 0; t0 < q_len; t0 += (int)blockDim.x * K, pass ^= 1) {
    const int mine = t0 + (int)threadIdx.x * K;
    float gi[K], F[K], log_f[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      gi[j] = -INFINITY;
      F[j] = 0.f;
      if (mine + j < q_len) {
        const float* row = pre + (size_t)(q_start + mine + j) * 2 * H;
        gi[j] = row[h] + bias_i[h];
        F[j] = row[H + h] + bias_f[h];
      }
    }
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const bool on = mine + j < q_len;
      gi[j] = on ? capped(gi[j], cap) : -INFINITY;
      const float f = on ? log_sigmoid(capped(F[j], cap)) : 0.f;
      log_f[j] = f;
      F[j] = f + (j ? F[j - 1] : 0.f);  // within the lane
    }
    const float tot = F[K - 1];
    float incl = tot;  // over the lanes of the warp, inclusive
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const float before = incl - tot;
    float best[K];  // max of i_s - F_s up to each token, F counted from the warp's first token
#pragma unroll
    for (int j = 0; j < K; ++j) {
      F[j] += before;
      best[j] = gi[j] - F[j];
      if (j) best[j] = fmaxf(best[j], best[j - 1]);
    }
    float upto = best[K - 1];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, upto, o);
      if (lane >= o) upto = fmaxf(upto, v);
    }
    float front = __shfl_up_sync(0xffffffffu, upto, 1);
    if (lane == 0) front = -INFINITY;
    if (lane == 31) {
      warp_f[pass][warp] = incl;
      warp_b[pass][warp] = upto;
    }
    __syncthreads();  // (the other pair of arrays is written in the next pass: one barrier a pass is enough)
    float f_pre = 0.f, b_pre = -INFINITY, f_all = 0.f, b_all = -INFINITY;
    for (int w = 0; w < n_warps; ++w) {
      if (w == warp) { f_pre = f_all; b_pre = b_all; }
      b_all = fmaxf(b_all, warp_b[pass][w] - f_all);
      f_all += warp_f[pass][w];
    }
    float mt[K];
#pragma unroll
    for (int j = 0; j < K; ++j) mt[j] = f_pre + F[j] + fmaxf(m, fmaxf(b_pre, fmaxf(front, best[j]) - f_pre));
    // the maximum in front of the lane's first token: the lane's before, the warp's before, or the pass's start
    float m_prev = __shfl_up_sync(0xffffffffu, mt[K - 1], 1);
    if (lane == 0) m_prev = f_pre + fmaxf(m, b_pre);
#pragma unroll
    for (int j = 0; j < K; ++j) {
      if (mine + j < q_len) {
        const size_t at = (size_t)(q_start + mine + j) * H + h;
        key_fac[at] = expf(gi[j] - mt[j]);
        decay[at] = expf(log_f[j] + m_prev - mt[j]);
        m_out[at] = mt[j];
      }
      m_prev = mt[j];
    }
    m = f_all + fmaxf(m, b_all);  // tokens past the end count as f = 0, i = -inf
  }
  if (has_slot && threadIdx.x == 0) m_state[(size_t)slot * H + h] = m;
}

// a warp per (token, head)
template <typename T>
__global__ void mlstm_output_kernel(const float* __restrict__ o32, const float* __restrict__ nq, const float* __restrict__ m,
                                    const T* __restrict__ gates, long long gate_stride, const float* __restrict__ norm_w,
                                    float eps, T* __restrict__ out, int n_tokens, int H, int Dv) {
  pdl_wait();
  pdl_trigger();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n_tokens * H) return;
  const int t = warp / H, h = warp - t * H;
  const float* src = o32 + ((size_t)t * H + h) * Dv;
  const float den = fmaxf(fabsf(nq[(size_t)t * H + h]), expf(-m[(size_t)t * H + h])) + 1e-6f;
  float ss = 0.f;
  for (int d = lane; d < Dv; d += 32) {
    const float v = src[d] / den;
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)Dv + eps);
  const T* g = gates + (size_t)t * gate_stride + h * Dv;
  T* dst = out + ((size_t)t * H + h) * Dv;
  for (int d = lane; d < Dv; d += 32) {
    const float v = src[d] / den * r * norm_w[h * Dv + d];
    const float gate = 1.f / (1.f + expf(-to_float(g[d])));
    dst[d] = from_float<T>(v * gate);
  }
}

// The same for bfloat16 heads of 8 x 2^k values (k <= 5) whose rows allow 16-byte accesses: a thread takes eight
// consecutive values, the TPR threads of a (token, head) sit side by side in a warp and add their squares by shuffles.
template <int TPR>
__global__ void __launch_bounds__(256) mlstm_output_vec_kernel(const float* __restrict__ o32, const float* __restrict__ nq,
                                                               const float* __restrict__ m,
                                                               const __nv_bfloat16* __restrict__ gates, long long gate_stride,
                                                               const float* __restrict__ norm_w, float eps,
                                                               __nv_bfloat16* __restrict__ out, int n_tokens, int H) {
  pdl_wait();
  pdl_trigger();
  constexpr int Dv = TPR * 8;
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / TPR;
  const int d = (threadIdx.x % TPR) * 8;
  const bool ok = w < (long long)n_tokens * H;
  const long long wr = ok ? w : 0;
  const long long t = wr / H;
  const int h = (int)(wr % H);
  const float* src = o32 + (size_t)wr * Dv + d;
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  const uint4 graw = *reinterpret_cast<const uint4*>(gates + t * gate_stride + (size_t)h * Dv + d);
  const float4 w0 = *reinterpret_cast<const float4*>(norm_w + h * Dv + d), w1 = *reinterpret_cast<const float4*>(norm_w + h * Dv + d + 4);
  const float den = fmaxf(fabsf(nq[wr]), expf(-m[wr])) + 1e-6f;
  float v[8] = {a.x / den, a.y / den, a.z / den, a.w / den, b.x / den, b.y / den, b.z / den, b.w / den};
  const float wt[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 8; ++u) ss += v[u] * v[u];
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = rsqrtf(ss / (float)Dv + eps);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
  uint4 res;
  __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const float2 g = __bfloat1622float2(g2[u]);
    const float y0 = v[2 * u] * r * wt[2 * u] / (1.f + expf(-g.x));
    const float y1 = v[2 * u + 1] * r * wt[2 * u + 1] / (1.f + expf(-g.y));
    r2[u] = __floats2bfloat162_rn(y0, y1);
  }
  if (ok) *reinterpret_cast<uint4*>(out + (size_t)wr * Dv + d) = res;
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_mlstm_gates(const float* pre, const float* bias_i, const float* bias_f, float cap, float* m_state,
                               int n_slots, const int32_t* state_slots, const int32_t* seg_info, int n_segs, int n_heads,
                               int n_tokens, float* key_fac, float* decay, float* m_out, void* stream) {
  FTK_REQUIRE(n_segs >= 1 && n_heads >= 1 && n_tokens >= 0 && cap > 0.f, "mlstm_gates: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(pre && bias_i && bias_f && m_state && state_slots && seg_info && key_fac && decay && m_out,
              "mlstm_gates: null pointer");
  FTK_REQUIRE((long long)n_segs * n_heads <= 0x7fffffffLL, "mlstm_gates: too many (request, head) pairs");
  const int threads = n_tokens / n_segs <= 128 ? 32 : 256;  // a warp where requests bring a few tokens, eight for portions
  FTK_LAUNCH(mlstm_gates_kernel, n_segs * n_heads, threads, 0, (cudaStream_t)stream, pre, bias_i, bias_f, cap, m_state, n_slots,
             state_slots, seg_info, n_segs, n_heads, n_tokens, key_fac, decay, m_out);
  FTK_LAUNCH_CHECK("mlstm_gates");
  return 0;
}

extern "C" int ftk_mlstm_output(const float* o32, const float* nq, const float* m, const void* gates, long long gate_stride,
                                const float* norm_w, float eps, void* out, int dtype, int n_tokens, int n_heads, int vdim,
                                void* stream) {
  FTK_REQUIRE(dtype_ok(dtype) && n_heads >= 1 && vdim >= 1 && n_tokens >= 0, "mlstm_output: bad arguments");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(o32 && nq && m && gates && norm_w && out, "mlstm_output: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const long long warps = (long long)n_tokens * n_heads;
  const int tpr = vdim / 8;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (dtype == FTK_BF16 && vdim % 8 == 0 && tpr <= 32 && (tpr & (tpr - 1)) == 0 && gate_stride % 8 == 0 && al16(o32) &&
      al16(gates) && al16(norm_w) && al16(out)) {
    const unsigned blocks = (unsigned)((warps * tpr + 255) / 256);
#define FTK_MO(N) FTK_LAUNCH(mlstm_output_vec_kernel<N>, blocks, 256, 0, s, o32, nq, m, (const __nv_bfloat16*)gates, gate_stride, \
                             norm_w, eps, (__nv_bfloat16*)out, n_tokens, n_heads)
    (tpr == 1 ? FTK_MO(1) : tpr == 2 ? FTK_MO(2) : tpr == 4 ? FTK_MO(4) : tpr == 8 ? FTK_MO(8) : tpr == 16 ? FTK_MO(16) : FTK_MO(32));
#undef FTK_MO
    FTK_LAUNCH_CHECK("mlstm_output");
    return 0;
  }
  const unsigned blocks = (unsigned)((warps + 3) / 4);
  if (dtype == FTK_F32)
    FTK_LAUNCH(mlstm_output_kernel<float>, blocks, 128, 0, s, o32, nq, m, (const float*)gates, gate_stride, norm_w, eps, (float*)out,
               n_tokens, n_heads, vdim);
  else
    FTK_LAUNCH(mlstm_output_kernel<__nv_bfloat16>, blocks, 128, 0, s, o32, nq, m, (const __nv_bfloat16*)gates, gate_stride, norm_w,
               eps, (__nv_bfloat16*)out, n_tokens, n_heads, vdim);
  FTK_LAUNCH_CHECK("mlstm_output");
  return 0;
}
