// Gated delta rule: a matrix state per (request, head) that every token first decays, then corrects towards its
// value along its key, then reads with its query:
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
// beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)); q and k are made unit vectors per head first
// (x / sqrt(sum x^2 + eps)), q also scaled.  State, gates, norms and all sums are 32-bit.  The state is kept
// column by column, [value column][key channel], so that a thread's share of a column is one stretch of memory.
//
// The correction u needs S^T k of the state as the token finds it, so a request's tokens run one after the other.
// What runs side by side are the state's columns: a block owns 16 to 64 value columns of one (request, head); eight
// (or four, or two) neighbouring lanes share a column, each keeping its share of the column's key channels in
// registers.  One pass over a thread's share of the state gives both S^T k and S^T q of the state as found (a few
// shuffle rounds, interleaved), and the token's output follows without a second pass: with r = S^T k, p = S^T q of
// the state before the decay,
//   u = beta (v - g r),   o = g p + (k . q) u,   S <- g S + k u^T.
// Tokens go in pairs: the sums over the state for both come from the state as the first finds it, in one pass and one
// set of shuffle rounds, and the second token's follow from them with the dots k_a . k_b and k_a . q_b; that halves the
// chain of sums, shuffles and updates that a token cannot start before the one before has ended.
// The tokens' q, k, v come through shared memory 16 tokens at a time: rows that allow 16-byte copies are fetched a
// batch ahead with cp.async as they lie in memory while the current batch runs, and a pass from shared to shared
// memory widens them, makes q and k unit vectors (eight lanes a token) and takes k . q; every slice's channels are
// set off by 16 bytes (and every raw row by 16 bytes) so that lanes that read side by side fall into different
// banks.  The outputs of a batch leave together.  A decode step is the same kernel with one token per request.
#include "common.cuh"

namespace ftk {

constexpr int kDeltaBatch = 16;   // tokens staged at a time
constexpr int kDeltaThreads = 128;

struct DeltaArgs {
  const void* q; const void* k; const void* v; const void* b; const void* a;
  long long q_stride, k_stride, v_stride, b_stride, a_stride;
  const float* a_log; const float* dt_bias;
  float q_scale, unit_eps;
  float* state; int n_slots;
  const int32_t* state_slots; const int32_t* seg_info; int n_segs;
  float* out; int n_tokens, H, G, D, Dv;
  int wide;  // q, k and v rows allow 16-byte copies
};

__device__ __forceinline__ float delta_softplus(float z) { return z > 0.f ? z + log1pf(expf(-z)) : log1pf(expf(z)); }
__device__ __forceinline__ void delta_cp16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // fewer source bytes than 16: the rest is written as zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void delta_cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void delta_cp_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// DPT key channels a thread, LPC lanes a column
template <int DPT, int LPC>
__host__ __device__ constexpr int delta_row_len() { return DPT * LPC + 4 * LPC; }  // a slice's channels start 16 bytes behind the slice before
template <int LPC>
__host__ __device__ constexpr int delta_cols() { return kDeltaThreads / LPC; }  // value columns per block
template <typename T, int DPT, int LPC>
__host__ __device__ constexpr size_t delta_smem_bytes() {
  return ((size_t)2 * kDeltaBatch * delta_row_len<DPT, LPC>() + kDeltaBatch * delta_cols<LPC>() + 4 * kDeltaBatch) * sizeof(float) +
         ((size_t)2 * kDeltaBatch * (DPT * LPC + 16 / sizeof(T)) + kDeltaBatch * delta_cols<LPC>()) * sizeof(T);
}

template <typename T, int DPT, int LPC>
__global__ void __launch_bounds__(kDeltaThreads) delta_scan_kernel(DeltaArgs a) {
  pdl_wait();
  pdl_trigger();
  constexpr int Dp = DPT * LPC;  // padded key channels
  constexpr int RL = delta_row_len<DPT, LPC>();
  constexpr int E = 16 / (int)sizeof(T);  // elements per 16-byte copy
  constexpr int RAWL = Dp + E;            // a raw row and its 16 bytes of padding
  constexpr int kDeltaCols = delta_cols<LPC>();
  constexpr int CPW = 32 / LPC;           // columns per warp
  extern __shared__ __align__(16) float sm[];
  float* sq = sm;                                   // [batch][RL]: channel d of a token at d + 4 (d / DPT)
  float* sk = sq + kDeltaBatch * RL;
  float* sv = sk + kDeltaBatch * RL;                // [batch][cols]
  // (the outputs of a batch lie in an array of their own: the token loop's loads may then pass its stores)
  __shared__ float so[kDeltaBatch * kDeltaCols];
  float* sbeta = sv + kDeltaBatch * kDeltaCols;     // [batch]
  float* sg = sbeta + kDeltaBatch;
  float* skq = sg + kDeltaBatch;
  float* skk = skq + kDeltaBatch;                   // [batch / 2]: k_a . k_b of the pair of tokens (2j, 2j + 1)
  float* skq2 = skk + kDeltaBatch / 2;              // [batch / 2]: k_a . q_b
  T* qraw = reinterpret_cast<T*>(skq2 + kDeltaBatch / 2);  // [batch][RAWL]: the next batch as it lies in memory
  T* kraw = qraw + kDeltaBatch * RAWL;
  T* vraw = kraw + kDeltaBatch * RAWL;              // [batch][cols]
  const int seg = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * kDeltaCols;
  const int D = a.D, Dv = a.Dv;
  const int q_start = a.seg_info[seg * 4], q_len = a.seg_info[seg * 4 + 1], kv_len = a.seg_info[seg * 4 + 2];
  if (q_len <= 0 || q_start < 0 || q_start + q_len > a.n_tokens || kv_len < q_len) return;
  const int slot = a.state_slots[seg];
  if (slot < 0 || slot >= a.n_slots) return;
  const int hqk = h / (a.H / a.G);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slice = lane % LPC, lcol = warp * CPW + lane / LPC, col = col0 + lcol;
  const int d0 = slice * DPT;
  const bool live = col < Dv;
  // the state lies column by column ([Dv][D]): a thread's channels of its column are neighbours in memory
  float* st = a.state + (((size_t)slot * a.H + h) * Dv + (live ? col : 0)) * D + d0;
  const bool fresh = kv_len == q_len;
  const bool quads = (D & 3) == 0;  // (the state's rows then start on 16 bytes: float4 accesses)
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; i += 4) {
    if (!fresh && live && quads && d0 + i + 4 <= D) {
      const float4 f = *reinterpret_cast<const float4*>(st + i);
      s[i] = f.x; s[i + 1] = f.y; s[i + 2] = f.z; s[i + 3] = f.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[i + e] = (!fresh && live && d0 + i + e < D) ? st[i + e] : 0.f;
    }
  }
  const T* qb = (const T*)a.q; const T* kb = (const T*)a.k; const T* vb = (const T*)a.v;
  const T* bb = (const T*)a.b; const T* ab = (const T*)a.a;
  const float neg_rate = -expf(a.a_log[h]), bias = a.dt_bias[h];
  const bool wide = a.wide != 0;
  // the batch from token b0n on, as it lies in memory, into the raw buffers (16 bytes a copy; zeros past the rows' ends)
  auto fetch = [&](int b0n) {
    const int nbn = min(kDeltaBatch, q_len - b0n);
    constexpr int per_row = Dp / E;
    for (int i = threadIdx.x; i < kDeltaBatch * per_row; i += kDeltaThreads) {
      const int t = i / per_row, d = (i % per_row) * E;
      const bool in = t < nbn && d < D;
      const size_t tok = (size_t)(q_start + b0n + (in ? t : 0));
      delta_cp16(qraw + t * RAWL + d, in ? qb + tok * a.q_stride + (size_t)hqk * D + d : qb, in);
      delta_cp16(kraw + t * RAWL + d, in ? kb + tok * a.k_stride + (size_t)hqk * D + d : kb, in);
    }
    constexpr int vper = kDeltaCols / E;
    for (int i = threadIdx.x; i < kDeltaBatch * vper; i += kDeltaThreads) {
      const int t = i / vper, j = (i % vper) * E;
      const bool in = t < nbn && col0 + j < Dv;
      const size_t tok = (size_t)(q_start + b0n + (in ? t : 0));
      delta_cp16(vraw + t * kDeltaCols + j, in ? vb + tok * a.v_stride + (size_t)h * Dv + col0 + j : vb, in);
    }
    delta_cp_commit();
  };
  // the gate logits of a batch: a thread a token, fetched a batch ahead into registers
  float bl_next = 0.f, al_next = 0.f;
  auto fetch_gates = [&](int b0n) {
    const int t = threadIdx.x;
    if (t < kDeltaBatch && b0n + t < q_len) {
      const size_t tok = (size_t)(q_start + b0n + t);
      bl_next = to_float(bb[tok * a.b_stride + h]);
      al_next = to_float(ab[tok * a.a_stride + h]);
    }
  };
  if (wide) fetch(0);
  fetch_gates(0);
  for (int b0 = 0; b0 < q_len; b0 += kDeltaBatch) {
    const int nb = min(kDeltaBatch, q_len - b0);
    if (wide) delta_cp_wait_all();
    __syncthreads();  // the raw rows have landed; the batch before is read and its outputs are written
    if (threadIdx.x < nb) {
      sbeta[threadIdx.x] = 1.f / (1.f + expf(-bl_next));
      sg[threadIdx.x] = expf(neg_rate * delta_softplus(al_next + bias));
    }
    if (!wide) {  // rows that do not allow 16-byte copies: element by element, straight from memory
      for (int i = threadIdx.x; i < kDeltaBatch * Dp; i += kDeltaThreads) {
        const int t = i / Dp, d = i % Dp;
        const bool in = t < nb && d < D;
        const size_t tok = (size_t)(q_start + b0 + (in ? t : 0));
        qraw[t * RAWL + d] = in ? qb[tok * a.q_stride + (size_t)hqk * D + d] : from_float<T>(0.f);
        kraw[t * RAWL + d] = in ? kb[tok * a.k_stride + (size_t)hqk * D + d] : from_float<T>(0.f);
      }
      for (int i = threadIdx.x; i < kDeltaBatch * kDeltaCols; i += kDeltaThreads) {
        const int t = i / kDeltaCols, j = i % kDeltaCols;
        const bool in = t < nb && col0 + j < Dv;
        const size_t tok = (size_t)(q_start + b0 + (in ? t : 0));
        vraw[i] = in ? vb[tok * a.v_stride + (size_t)h * Dv + col0 + j] : from_float<T>(0.f);
      }
      __syncthreads();
    }
    // widen; unit vectors and k . q: eight lanes a token, a warp four tokens at a time
    for (int t = warp * 4 + (lane >> 3); t < kDeltaBatch; t += kDeltaThreads / 8) {
      const int sub = lane & 7;
      float s2q = 0.f, s2k = 0.f, dkq = 0.f, dkk = 0.f, dkq2 = 0.f;
      const int tp = t > 0 ? t - 1 : 0;  // the token before (its dots are used by the odd tokens of a pair)
      for (int d = sub; d < Dp; d += 8) {
        const float qv = to_float(qraw[t * RAWL + d]), kv = to_float(kraw[t * RAWL + d]);
        const float kp = to_float(kraw[tp * RAWL + d]);
        s2q = fmaf(qv, qv, s2q); s2k = fmaf(kv, kv, s2k); dkq = fmaf(qv, kv, dkq);
        dkk = fmaf(kp, kv, dkk); dkq2 = fmaf(kp, qv, dkq2);
      }
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) {
        s2q += __shfl_xor_sync(0xffffffffu, s2q, o);
        s2k += __shfl_xor_sync(0xffffffffu, s2k, o);
        dkq += __shfl_xor_sync(0xffffffffu, dkq, o);
        dkk += __shfl_xor_sync(0xffffffffu, dkk, o);
        dkq2 += __shfl_xor_sync(0xffffffffu, dkq2, o);
      }
      const float rq = rsqrtf(s2q + a.unit_eps) * a.q_scale, rk = rsqrtf(s2k + a.unit_eps);
      const float rk_before = __shfl_up_sync(0xffffffffu, rk, 8);  // (an odd token's partner lies eight lanes down)
      if (sub == 0 && (t & 1)) { skk[t >> 1] = dkk * rk_before * rk; skq2[t >> 1] = dkq2 * rk_before * rq; }
      for (int d = sub; d < Dp; d += 8) {
        const int at = t * RL + d + 4 * (d / DPT);
        sq[at] = to_float(qraw[t * RAWL + d]) * rq;
        sk[at] = to_float(kraw[t * RAWL + d]) * rk;
      }
      if (sub == 0) skq[t] = dkq * rq * rk;
    }
    for (int i = threadIdx.x; i < kDeltaBatch * kDeltaCols; i += kDeltaThreads) sv[i] = to_float(vraw[i]);
    __syncthreads();  // the raw buffers are read: the next batch may land
    if (b0 + kDeltaBatch < q_len) {
      if (wide) fetch(b0 + kDeltaBatch);
      fetch_gates(b0 + kDeltaBatch);
    }
    // two tokens at a time: S^T k and S^T q of both from the state as the first finds it (one pass, one set of shuffle
    // rounds); with the pair's dots k_a . k_b and k_a . q_b the second token's sums over the state the first leaves follow:
    //   S_a^T k_b = g_a S^T k_b + (k_a . k_b) u_a,   S_a^T q_b = g_a S^T q_b + (k_a . q_b) u_a
    int t_done = 0;
#pragma unroll 2
    for (int t = 0; t + 1 < nb; t += 2) {
      const float ga = sg[t], gb = sg[t + 1], ba = sbeta[t], bb2 = sbeta[t + 1], kqa = skq[t], kqb = skq[t + 1];
      const float kk = skk[t >> 1], kqab = skq2[t >> 1];
      const float va = sv[t * kDeltaCols + lcol], vb2 = sv[(t + 1) * kDeltaCols + lcol];
      const float4* ka4 = reinterpret_cast<const float4*>(sk + t * RL + d0 + 4 * slice);
      const float4* qa4 = reinterpret_cast<const float4*>(sq + t * RL + d0 + 4 * slice);
      const float4* kb4 = reinterpret_cast<const float4*>(sk + (t + 1) * RL + d0 + 4 * slice);
      const float4* qb4 = reinterpret_cast<const float4*>(sq + (t + 1) * RL + d0 + 4 * slice);
      float ra[2] = {0.f, 0.f}, pa[2] = {0.f, 0.f}, rb[2] = {0.f, 0.f}, pb[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {
        const float4 ka = ka4[i], qa = qa4[i], kb = kb4[i], qb = qb4[i];
        ra[0] = fmaf(s[4 * i + 0], ka.x, ra[0]); pa[0] = fmaf(s[4 * i + 0], qa.x, pa[0]);
        rb[0] = fmaf(s[4 * i + 0], kb.x, rb[0]); pb[0] = fmaf(s[4 * i + 0], qb.x, pb[0]);
        ra[1] = fmaf(s[4 * i + 1], ka.y, ra[1]); pa[1] = fmaf(s[4 * i + 1], qa.y, pa[1]);
        rb[1] = fmaf(s[4 * i + 1], kb.y, rb[1]); pb[1] = fmaf(s[4 * i + 1], qb.y, pb[1]);
        ra[0] = fmaf(s[4 * i + 2], ka.z, ra[0]); pa[0] = fmaf(s[4 * i + 2], qa.z, pa[0]);
        rb[0] = fmaf(s[4 * i + 2], kb.z, rb[0]); pb[0] = fmaf(s[4 * i + 2], qb.z, pb[0]);
        ra[1] = fmaf(s[4 * i + 3], ka.w, ra[1]); pa[1] = fmaf(s[4 * i + 3], qa.w, pa[1]);
        rb[1] = fmaf(s[4 * i + 3], kb.w, rb[1]); pb[1] = fmaf(s[4 * i + 3], qb.w, pb[1]);
      }
      float ras = ra[0] + ra[1], pas = pa[0] + pa[1], rbs = rb[0] + rb[1], pbs = pb[0] + pb[1];
#pragma unroll
      for (int o = 1; o < LPC; o <<= 1) {
        ras += __shfl_xor_sync(0xffffffffu, ras, o);
        rbs += __shfl_xor_sync(0xffffffffu, rbs, o);
        pas += __shfl_xor_sync(0xffffffffu, pas, o);
        pbs += __shfl_xor_sync(0xffffffffu, pbs, o);
      }
      const float ua = ba * (va - ga * ras);
      const float ub = bb2 * (vb2 - gb * fmaf(ga, rbs, kk * ua));
      const float gab = ga * gb, wa = gb * ua;
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {  // S <- g_b (g_a S + k_a u_a^T) + k_b u_b^T
        const float4 ka = ka4[i], kb = kb4[i];
        s[4 * i + 0] = fmaf(gab, s[4 * i + 0], fmaf(wa, ka.x, ub * kb.x));
        s[4 * i + 1] = fmaf(gab, s[4 * i + 1], fmaf(wa, ka.y, ub * kb.y));
        s[4 * i + 2] = fmaf(gab, s[4 * i + 2], fmaf(wa, ka.z, ub * kb.z));
        s[4 * i + 3] = fmaf(gab, s[4 * i + 3], fmaf(wa, ka.w, ub * kb.w));
      }
      if (slice == 0) {
        so[t * kDeltaCols + lcol] = fmaf(ga, pas, kqa * ua);
        so[(t + 1) * kDeltaCols + lcol] = fmaf(gb, fmaf(ga, pbs, kqab * ua), kqb * ub);
      }
      t_done = t + 2;
    }
    for (int t = t_done; t < nb; ++t) {  // (a batch's odd last token)
      const float g = sg[t], beta = sbeta[t], kq = skq[t], vj = sv[t * kDeltaCols + lcol];
      const float4* k4 = reinterpret_cast<const float4*>(sk + t * RL + d0 + 4 * slice);
      const float4* q4 = reinterpret_cast<const float4*>(sq + t * RL + d0 + 4 * slice);
      float4 kr[DPT / 4];
      float r[4] = {0.f, 0.f, 0.f, 0.f}, pp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {
        const float4 kv = k4[i], qv = q4[i];
        kr[i] = kv;
        r[0] = fmaf(s[4 * i + 0], kv.x, r[0]); pp[0] = fmaf(s[4 * i + 0], qv.x, pp[0]);
        r[1] = fmaf(s[4 * i + 1], kv.y, r[1]); pp[1] = fmaf(s[4 * i + 1], qv.y, pp[1]);
        r[2] = fmaf(s[4 * i + 2], kv.z, r[2]); pp[2] = fmaf(s[4 * i + 2], qv.z, pp[2]);
        r[3] = fmaf(s[4 * i + 3], kv.w, r[3]); pp[3] = fmaf(s[4 * i + 3], qv.w, pp[3]);
      }
      float rs = (r[0] + r[1]) + (r[2] + r[3]), ps = (pp[0] + pp[1]) + (pp[2] + pp[3]);
#pragma unroll
      for (int o = 1; o < LPC; o <<= 1) {
        rs += __shfl_xor_sync(0xffffffffu, rs, o);
        ps += __shfl_xor_sync(0xffffffffu, ps, o);
      }
      const float u = beta * (vj - g * rs);  // S^T k of the decayed state is g times that of the state as found
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {
        s[4 * i + 0] = fmaf(g, s[4 * i + 0], kr[i].x * u);
        s[4 * i + 1] = fmaf(g, s[4 * i + 1], kr[i].y * u);
        s[4 * i + 2] = fmaf(g, s[4 * i + 2], kr[i].z * u);
        s[4 * i + 3] = fmaf(g, s[4 * i + 3], kr[i].w * u);
      }
      if (slice == 0) so[t * kDeltaCols + lcol] = fmaf(g, ps, kq * u);  // S_new^T q = g S^T q + (k . q) u
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nb * kDeltaCols; i += kDeltaThreads) {
      const int t = i / kDeltaCols, j = i % kDeltaCols;
      if (col0 + j < Dv) a.out[((size_t)(q_start + b0 + t) * a.H + h) * Dv + col0 + j] = so[i];
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DPT; i += 4) {
      if (quads && d0 + i + 4 <= D) {
        *reinterpret_cast<float4*>(st + i) = make_float4(s[i], s[i + 1], s[i + 2], s[i + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (d0 + i + e < D) st[i + e] = s[i + e];
      }
    }
  }
}

template <typename T, int DPT, int LPC>
static int launch_delta_sized(const DeltaArgs& a, cudaStream_t s) {
  constexpr int kDeltaCols = delta_cols<LPC>();
  dim3 grid(a.n_segs, a.H, (a.Dv + kDeltaCols - 1) / kDeltaCols);
  constexpr size_t smem = delta_smem_bytes<T, DPT, LPC>();
  auto kern = delta_scan_kernel<T, DPT, LPC>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  FTK_LAUNCH(kern, grid, kDeltaThreads, smem, s, a);
  FTK_LAUNCH_CHECK("delta_scan");
  return 0;
}

template <typename T>
static int launch_delta(DeltaArgs a, cudaStream_t s) {
  const long long e = 16 / (long long)sizeof(T);
  a.wide = a.D % e == 0 && a.Dv % e == 0 && a.q_stride % e == 0 && a.k_stride % e == 0 && a.v_stride % e == 0 &&
           (((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v) & 15) == 0;
  if (a.D <= 16) return launch_delta_sized<T, 4, 4>(a, s);
  if (a.D <= 32) return launch_delta_sized<T, 4, 8>(a, s);
  if (a.D <= 64) return launch_delta_sized<T, 8, 8>(a, s);
  if (a.D <= 128) {
    // two lanes a column (64 channels a thread, one shuffle round) once the step has columns enough for every SM that way;
    // measured on B200, 48 heads of 128 x 128, 2,048 tokens: 856 us against 988 (four lanes) and 910 (eight)
    if ((long long)a.n_segs * a.H * a.Dv >= 148 * 32) return launch_delta_sized<T, 64, 2>(a, s);
    return launch_delta_sized<T, 16, 8>(a, s);
  }
  return launch_delta_sized<T, 32, 8>(a, s);
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
              vdim >= 1 && vdim <= 65535 * 16 && (long long)n_heads <= 65535,
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
