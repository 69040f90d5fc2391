// Gated linear attention: a matrix state per (request, head), S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t,
// with a decay a_t = sigmoid(z_t)^(1 / tau) per key channel.  State, decays and all sums are 32-bit.
//
// A step's tokens are cut into chunks of at most `chunk` consecutive tokens of one request (the host
// lists them: 4 int32 per chunk = segment, first token within the segment's tokens, tokens, place of
// the chunk among the segment's chunks; and per segment: first chunk, chunks).  A request with one
// chunk (every decode step) takes one launch: the recurrence runs from the request's state slot and
// leaves the new state there.  Longer portions take three launches, so that chunks run side by side:
//   1. every chunk but a segment's last runs the recurrence from a zero state: its own contribution
//      L_c = sum_s (prod_{r > s} a_r) k_s v_s^T, and the product of its decays P_c;
//   2. per segment and state element, one after the other: S_(c+1) = P_c S_c + L_c, with S_0 the slot's
//      state (zero for a request's first tokens); S_(c+1) overwrites L_c, and S_0 goes where the last chunk's
//      L would lie, so that step 3 never reads a slot that its last chunk is writing;
//   3. every chunk runs the recurrence from its start state and writes its tokens' outputs; a
//      segment's last chunk leaves the final state in the slot.
// The recurrence itself is the plain one, token by token, so the result differs from a pure scan only
// by the rounding of step 2's sums.
//
// A block owns 64 (or 32) value columns of one (chunk, head): per group of that many columns, 4 warps split the
// key channels, a thread keeps its share of two (or one) state columns in registers, and the tokens' q, k and
// decays are staged in shared memory 16 tokens at a time for all of the block's columns (float4 reads, the same
// address for the whole warp).  Portions of several chunks turn their decay logits into decays once, in place, before
// the chunks run; a decode step does it while it stages its one token.
#include "common.cuh"

namespace ftk {

constexpr int kGlaSlices = 4;    // warps per column group: each takes a quarter of the key channels
constexpr int kGlaBatch = 16;    // tokens staged at a time
// value columns per thread: two (columns lane and lane + 32 of the group's 64) while a thread's share of the key
// channels leaves the registers for it; every q, k and decay read from shared memory then serves two columns
__host__ __device__ constexpr int gla_cols_per_thread(int dpt) { return dpt <= 32 ? 2 : 1; }
// column groups (of four warps) per block: one (measured on B200 at 16 heads of 128 x 128, 2,048 tokens: 276 us
// against 306 with two groups, whose 256 threads of 150 to 170 registers leave an SM a single block)
__host__ __device__ constexpr int gla_max_groups(int dpt) { return 1; }

struct GlaArgs {
  const void* q; const void* k; const void* v;  // rows of the engine's type: token t at + t * stride, head h at + h * dim
  long long q_stride, k_stride, v_stride;
  float* z;                // [T, H * D] decay logits (before the bias); decays once gla_decay_kernel has run
  const float* z_bias;     // [H * D] or null
  int z_is_decay;
  float inv_tau, q_scale;
  float* state;            // [slots, H, D, Dv]
  const int32_t* state_slots;  // [S]
  const int32_t* seg_info;     // [S, 4]: q_start, q_len, kv_len, -
  const int32_t* chunks;       // [n_chunks, 4]
  const int32_t* seg_chunks;   // [S, 2]: first chunk, chunks
  int n_chunks, n_segs, n_slots;
  float* carry;            // [n_chunks, H, D, Dv]: L_c, then the start state of chunk c + 1
  float* decay_prod;       // [n_chunks, H, D]
  float* out;              // [T, H, Dv]
  int H, D, Dv, n_tokens, groups;
  const float* k_fac;      // [T, H] or null: a factor on token t's keys of head h (applied in 32 bits while they are staged)
  const float* a_head;     // [T, H] or null: one decay per (token, head) for all key channels, in place of z
  int ones_col;            // 1: the last of the Dv value columns is 1 for every token, and v holds Dv - 1 columns per head
  float* out_ones;         // [T, H] or null: with ones_col, that column's outputs go here and out is [T, H, Dv - 1]
  int qk_div;              // queries and keys are shared by groups of this many heads: head h reads q/k head h / qk_div
};

// 16 bytes from global to shared memory without a trip through registers; `valid` false writes zeros
__device__ __forceinline__ void gla_cp16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void gla_cp4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void gla_cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void gla_cp_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

__device__ __forceinline__ float decay_of(float z, float inv_tau) {
  // sigmoid(z)^(1 / tau) = exp(-softplus(-z) / tau)
  const float sp = z > 0.f ? log1pf(expf(-z)) : -z + log1pf(expf(z));
  return expf(-sp * inv_tau);
}

__global__ void gla_decay_kernel(float* z, const float* __restrict__ bias, long long n, int hd, float inv_tau) {
  pdl_wait();
  pdl_trigger();
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) z[i] = decay_of(z[i] + (bias ? bias[i % hd] : 0.f), inv_tau);
}

// MODE 0: one launch for segments of one chunk (state slot -> outputs -> state slot)
// MODE 1: local contribution of a chunk from a zero state (no outputs)
// MODE 3: outputs of a chunk from its start state
template <typename T, int DPT, int MODE>
__global__ void __launch_bounds__(gla_max_groups(DPT) * kGlaSlices * 32) gla_chunk_kernel(GlaArgs a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float sm[];
  const int D = a.D, Dv = a.Dv;
  const int Dvin = Dv - a.ones_col;             // value columns that v holds
  const int Dp = DPT * kGlaSlices;              // padded key channels
  constexpr int NC = gla_cols_per_thread(DPT);
  constexpr int kGlaCols = 32 * NC;             // value columns per group of four warps
  const int cols = a.groups * kGlaCols;         // value columns of this block
  float* sq = sm;                               // [batch][Dp]
  float* sk = sq + kGlaBatch * Dp;
  float* sa = sk + kGlaBatch * Dp;
  float* sv = sa + kGlaBatch * Dp;              // [batch][cols]
  float* part = sv + kGlaBatch * cols;          // [slices][batch][cols]
  const int c = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cols;
  const int hqk = h / a.qk_div;
  const int32_t* ch = a.chunks + (size_t)c * 4;
  const int seg = ch[0], tok0 = ch[1], ntok = ch[2], place = ch[3];
  if (seg < 0 || seg >= a.n_segs || ntok <= 0) return;
  const int q_start = a.seg_info[seg * 4], q_len = a.seg_info[seg * 4 + 1], kv_len = a.seg_info[seg * 4 + 2];
  const int n_seg_chunks = a.seg_chunks[seg * 2 + 1];
  if (tok0 < 0 || tok0 + ntok > q_len || q_start < 0 || q_start + q_len > a.n_tokens) return;
  const bool single = n_seg_chunks == 1, last = place == n_seg_chunks - 1;
  if (MODE == 0 && !single) return;
  if (MODE == 1 && (single || last)) return;
  if (MODE == 3 && single) return;
  const int slot = a.state_slots[seg];
  if (slot < 0 || slot >= a.n_slots) return;
  const int lane = threadIdx.x & 31, slice = (threadIdx.x >> 5) % kGlaSlices, group = threadIdx.x / (kGlaSlices * 32);
  const int lcol = group * kGlaCols + lane;     // the thread's first column within the block (the second: + 32)
  const int col = col0 + lcol;
  const int d0 = slice * DPT;
  float s[NC][DPT];
  // the start state
  const bool fresh = kv_len - q_len == 0;
  const float* src = nullptr;
  if (MODE == 0) {
    if (!fresh) src = a.state + ((size_t)slot * a.H + h) * D * Dv;
  } else if (MODE == 3) {  // chunk 0 finds its start state in the last chunk's place, the others in the chunk's before
    const int from = place == 0 ? c + n_seg_chunks - 1 : c - 1;
    src = a.carry + ((size_t)from * a.H + h) * D * Dv;
  }
#pragma unroll
  for (int n = 0; n < NC; ++n)
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      s[n][i] = (src && col + 32 * n < Dvin && d0 + i < D) ? src[(size_t)(d0 + i) * Dv + col + 32 * n] : 0.f;
  // The column of ones (a normaliser: the decayed sum of the keys) is no value column of any thread: in the block of
  // the first columns, lane l of a slice's warp keeps its key channels l, l + 32, ... of it, and the warp adds up n . q.
  constexpr int NPL = (DPT + 31) / 32;
  const bool norm_here = a.ones_col && blockIdx.z == 0 && group == 0;
  float nn[NPL];
#pragma unroll
  for (int u = 0; u < NPL; ++u) {
    const int i = lane + 32 * u;
    nn[u] = (norm_here && src && i < DPT && d0 + i < D) ? src[(size_t)(d0 + i) * Dv + Dvin] : 0.f;
  }
  float pa[MODE == 1 ? DPT : 1];  // MODE 1: the product of the chunk's decays (the lanes of a warp hold the same values)
  if (MODE == 1) {
#pragma unroll
    for (int i = 0; i < DPT; ++i) pa[i] = 1.f;
  }
  const T* qb = (const T*)a.q;
  const T* kb = (const T*)a.k;
  const T* vb = (const T*)a.v;
  // eight bfloat16 at a time where the rows allow it
  const bool wide = sizeof(T) == 2 && D % 8 == 0 && a.q_stride % 8 == 0 && a.k_stride % 8 == 0 &&
                    ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) |
                      reinterpret_cast<uintptr_t>(a.z)) & 15) == 0;
  // bfloat16 rows that allow it are fetched a batch ahead: cp.async brings the next 16 tokens' q, k, decay logits and
  // values as they lie in memory into a second set of buffers while the current 16 are worked on, and a pass
  // from shared to shared memory widens them
  // (a chunk of one batch has nothing to fetch ahead of: it takes the direct way)
  const bool ahead = wide && ntok > kGlaBatch && Dvin % 8 == 0 && a.v_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(a.v) & 15) == 0;
  float* npart = part + kGlaSlices * kGlaBatch * cols;  // [slices][batch]: the ones column's share of each slice
  __nv_bfloat16* kraw = reinterpret_cast<__nv_bfloat16*>(npart + kGlaSlices * kGlaBatch);        // [batch][Dp]
  __nv_bfloat16* qraw = kraw + kGlaBatch * Dp;
  float* zraw = reinterpret_cast<float*>(qraw + kGlaBatch * Dp);                                  // [batch][Dp]
  __nv_bfloat16* vraw = reinterpret_cast<__nv_bfloat16*>(zraw + kGlaBatch * Dp);                  // [batch][cols]
  float* hraw = reinterpret_cast<float*>(vraw + kGlaBatch * cols);                                // [2][batch]: key factors, head decays
  auto fetch = [&](int b0n) {
    const int nbn = min(kGlaBatch, ntok - b0n);
    const int per_row = Dp / 8;
    const __nv_bfloat16* kg = reinterpret_cast<const __nv_bfloat16*>(a.k);
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.q);
    const __nv_bfloat16* vg = reinterpret_cast<const __nv_bfloat16*>(a.v);
    for (int i = threadIdx.x; i < nbn * per_row; i += blockDim.x) {
      const int t = i / per_row, d = (i % per_row) * 8;
      const size_t tok = (size_t)(q_start + tok0 + b0n + t);
      const bool in = d < D;
      gla_cp16(kraw + t * Dp + d, in ? kg + tok * a.k_stride + (size_t)hqk * D + d : kg, in);
      if (MODE != 1) gla_cp16(qraw + t * Dp + d, in ? qg + tok * a.q_stride + (size_t)hqk * D + d : qg, in);
      if (!a.a_head) {
        const float* zr = in ? a.z + (tok * a.H + h) * D + d : a.z;
        gla_cp16(zraw + t * Dp + d, zr, in);
        gla_cp16(zraw + t * Dp + d + 4, in ? zr + 4 : zr, in);
      }
    }
    if (a.k_fac || a.a_head) {
      for (int t = threadIdx.x; t < nbn; t += blockDim.x) {
        const size_t at = (size_t)(q_start + tok0 + b0n + t) * a.H + h;
        if (a.k_fac) gla_cp4(hraw + t, a.k_fac + at);
        if (a.a_head) gla_cp4(hraw + kGlaBatch + t, a.a_head + at);
      }
    }
    const int vper = cols / 8;
    for (int i = threadIdx.x; i < nbn * vper; i += blockDim.x) {
      const int t = i / vper, j = (i % vper) * 8;
      const size_t tok = (size_t)(q_start + tok0 + b0n + t);
      const bool in = col0 + j < Dvin;
      gla_cp16(vraw + t * cols + j, in ? vg + tok * a.v_stride + (size_t)h * Dvin + col0 + j : vg, in);
    }
    gla_cp_commit();
  };
  if (sizeof(T) == 2 && ahead) fetch(0);
  for (int b0 = 0; b0 < ntok; b0 += kGlaBatch) {
    const int nb = min(kGlaBatch, ntok - b0);
    if (sizeof(T) == 2 && ahead) gla_cp_wait_all();
    __syncthreads();
    if (sizeof(T) == 2 && ahead) {
      for (int i = threadIdx.x * 4; i < nb * Dp; i += blockDim.x * 4) {
        const int d = i % Dp, t = i / Dp;
        const float kf = a.k_fac ? hraw[t] : 1.f;
        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(kraw + i);
        const float2 k01 = __bfloat1622float2(k2[0]), k23 = __bfloat1622float2(k2[1]);
        *reinterpret_cast<float4*>(sk + i) = make_float4(k01.x * kf, k01.y * kf, k23.x * kf, k23.y * kf);
        if (MODE != 1) {
          const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(qraw + i);
          const float2 q01 = __bfloat1622float2(q2[0]), q23 = __bfloat1622float2(q2[1]);
          *reinterpret_cast<float4*>(sq + i) = make_float4(q01.x * a.q_scale, q01.y * a.q_scale, q23.x * a.q_scale, q23.y * a.q_scale);
        }
        float4 av;
        if (d >= D) {
          av = make_float4(1.f, 1.f, 1.f, 1.f);
        } else if (a.a_head) {
          const float ah = hraw[kGlaBatch + t];
          av = make_float4(ah, ah, ah, ah);
        } else {
          av = *reinterpret_cast<const float4*>(zraw + i);
        }
        if (d < D && !a.a_head && !a.z_is_decay) {
          const float* bz = a.z_bias ? a.z_bias + (size_t)h * D + d : nullptr;
          av.x = decay_of(av.x + (bz ? bz[0] : 0.f), a.inv_tau);
          av.y = decay_of(av.y + (bz ? bz[1] : 0.f), a.inv_tau);
          av.z = decay_of(av.z + (bz ? bz[2] : 0.f), a.inv_tau);
          av.w = decay_of(av.w + (bz ? bz[3] : 0.f), a.inv_tau);
        }
        *reinterpret_cast<float4*>(sa + i) = av;
      }
      for (int i = threadIdx.x * 2; i < nb * cols; i += blockDim.x * 2) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vraw + i));
        sv[i] = f.x;
        sv[i + 1] = f.y;
      }
      __syncthreads();
      if (b0 + kGlaBatch < ntok) fetch(b0 + kGlaBatch);  // the buffers are read: the next batch may land
    } else {
    if (wide) {
      const int per_row = Dp / 8;
      for (int i = threadIdx.x; i < nb * per_row; i += blockDim.x) {
        const int t = i / per_row, d = (i % per_row) * 8;
        const size_t tok = (size_t)(q_start + tok0 + b0 + t);
        float qv[8], kv[8], av[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) { qv[u] = 0.f; kv[u] = 0.f; av[u] = 1.f; }
        if (d < D) {
          const uint4 kr = *reinterpret_cast<const uint4*>(kb + tok * a.k_stride + (size_t)hqk * D + d);
          const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kr);
#pragma unroll
          const float kf = a.k_fac ? a.k_fac[tok * a.H + h] : 1.f;
#pragma unroll
          for (int u = 0; u < 4; ++u) { const float2 f = __bfloat1622float2(k2[u]); kv[2 * u] = f.x * kf; kv[2 * u + 1] = f.y * kf; }
          if (MODE != 1) {
            const uint4 qr = *reinterpret_cast<const uint4*>(qb + tok * a.q_stride + (size_t)hqk * D + d);
            const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&qr);
#pragma unroll
            for (int u = 0; u < 4; ++u) { const float2 f = __bfloat1622float2(q2[u]); qv[2 * u] = f.x * a.q_scale; qv[2 * u + 1] = f.y * a.q_scale; }
          }
          if (a.a_head) {
            const float ah = a.a_head[tok * a.H + h];
#pragma unroll
            for (int u = 0; u < 8; ++u) av[u] = ah;
          } else {
            const float* zr = a.z + (tok * a.H + h) * D + d;
            const float4 z0 = *reinterpret_cast<const float4*>(zr), z1 = *reinterpret_cast<const float4*>(zr + 4);
            av[0] = z0.x; av[1] = z0.y; av[2] = z0.z; av[3] = z0.w; av[4] = z1.x; av[5] = z1.y; av[6] = z1.z; av[7] = z1.w;
          }
          if (!a.a_head && !a.z_is_decay) {
#pragma unroll
            for (int u = 0; u < 8; ++u) av[u] = decay_of(av[u] + (a.z_bias ? a.z_bias[(size_t)h * D + d + u] : 0.f), a.inv_tau);
          }
        }
        float* dq = sq + t * Dp + d; float* dk = sk + t * Dp + d; float* da = sa + t * Dp + d;
        *reinterpret_cast<float4*>(dq) = make_float4(qv[0], qv[1], qv[2], qv[3]);
        *reinterpret_cast<float4*>(dq + 4) = make_float4(qv[4], qv[5], qv[6], qv[7]);
        *reinterpret_cast<float4*>(dk) = make_float4(kv[0], kv[1], kv[2], kv[3]);
        *reinterpret_cast<float4*>(dk + 4) = make_float4(kv[4], kv[5], kv[6], kv[7]);
        *reinterpret_cast<float4*>(da) = make_float4(av[0], av[1], av[2], av[3]);
        *reinterpret_cast<float4*>(da + 4) = make_float4(av[4], av[5], av[6], av[7]);
      }
    } else {
      for (int i = threadIdx.x; i < nb * Dp; i += blockDim.x) {
        const int t = i / Dp, d = i % Dp;
        const size_t tok = (size_t)(q_start + tok0 + b0 + t);
        float qv = 0.f, kv = 0.f, av = 1.f;
        if (d < D) {
          if (MODE != 1) qv = to_float(qb[tok * a.q_stride + (size_t)hqk * D + d]) * a.q_scale;
          kv = to_float(kb[tok * a.k_stride + (size_t)hqk * D + d]) * (a.k_fac ? a.k_fac[tok * a.H + h] : 1.f);
          av = a.a_head ? a.a_head[tok * a.H + h] : a.z[(tok * a.H + h) * D + d];
          if (!a.a_head && !a.z_is_decay) av = decay_of(av + (a.z_bias ? a.z_bias[(size_t)h * D + d] : 0.f), a.inv_tau);
        }
        sq[i] = qv; sk[i] = kv; sa[i] = av;
      }
    }
    for (int i = threadIdx.x; i < nb * cols; i += blockDim.x) {
      const int t = i / cols, j = i % cols;
      const size_t tok = (size_t)(q_start + tok0 + b0 + t);
      sv[i] = col0 + j < Dvin ? to_float(vb[tok * a.v_stride + (size_t)h * Dvin + col0 + j]) : 0.f;
    }
    __syncthreads();
    }
    for (int t = 0; t < nb; ++t) {
      float vj[NC], acc[NC][4];  // four chains per column, added in a fixed order
#pragma unroll
      for (int n = 0; n < NC; ++n) {
        vj[n] = sv[t * cols + lcol + 32 * n];
        acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      }
      const float4* q4 = reinterpret_cast<const float4*>(sq + t * Dp + d0);
      const float4* k4 = reinterpret_cast<const float4*>(sk + t * Dp + d0);
      const float4* a4 = reinterpret_cast<const float4*>(sa + t * Dp + d0);
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {
        const float4 av = a4[i], kv = k4[i];
        float4 qv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (MODE != 1) qv = q4[i];
#pragma unroll
        for (int n = 0; n < NC; ++n) {
          s[n][4 * i + 0] = fmaf(av.x, s[n][4 * i + 0], kv.x * vj[n]);
          s[n][4 * i + 1] = fmaf(av.y, s[n][4 * i + 1], kv.y * vj[n]);
          s[n][4 * i + 2] = fmaf(av.z, s[n][4 * i + 2], kv.z * vj[n]);
          s[n][4 * i + 3] = fmaf(av.w, s[n][4 * i + 3], kv.w * vj[n]);
          if (MODE != 1) {
            acc[n][0] = fmaf(s[n][4 * i + 0], qv.x, acc[n][0]);
            acc[n][1] = fmaf(s[n][4 * i + 1], qv.y, acc[n][1]);
            acc[n][2] = fmaf(s[n][4 * i + 2], qv.z, acc[n][2]);
            acc[n][3] = fmaf(s[n][4 * i + 3], qv.w, acc[n][3]);
          }
        }
        if (MODE == 1) {
          pa[4 * i + 0] *= av.x; pa[4 * i + 1] *= av.y; pa[4 * i + 2] *= av.z; pa[4 * i + 3] *= av.w;
        }
      }
      if (MODE != 1) {
#pragma unroll
        for (int n = 0; n < NC; ++n)
          part[(slice * kGlaBatch + t) * cols + lcol + 32 * n] = (acc[n][0] + acc[n][1]) + (acc[n][2] + acc[n][3]);
      }
      if (norm_here) {
        float nq = 0.f;
#pragma unroll
        for (int u = 0; u < NPL; ++u) {
          const int i = lane + 32 * u;
          if (i < DPT) {
            nn[u] = fmaf(sa[t * Dp + d0 + i], nn[u], sk[t * Dp + d0 + i]);
            if (MODE != 1) nq = fmaf(nn[u], sq[t * Dp + d0 + i], nq);
          }
        }
        if (MODE != 1) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) nq += __shfl_xor_sync(0xffffffffu, nq, o);
          if (lane == 0) npart[slice * kGlaBatch + t] = nq;
        }
      }
    }
    if (MODE != 1) {
      __syncthreads();
      for (int i = threadIdx.x; i < nb * cols; i += blockDim.x) {
        const int t = i / cols, j = i % cols;
        if (col0 + j < Dvin) {
          float o = 0.f;
#pragma unroll
          for (int w = 0; w < kGlaSlices; ++w) o += part[(w * kGlaBatch + t) * cols + j];  // slices in order
          const size_t row = (size_t)(q_start + tok0 + b0 + t) * a.H + h;
          a.out[row * (a.out_ones ? Dvin : Dv) + col0 + j] = o;
        }
      }
      if (norm_here && threadIdx.x < nb) {  // (group 0's threads: the first ones of the block)
        const int t = threadIdx.x;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kGlaSlices; ++w) o += npart[w * kGlaBatch + t];
        const size_t row = (size_t)(q_start + tok0 + b0 + t) * a.H + h;
        if (a.out_ones) a.out_ones[row] = o;
        else a.out[row * Dv + Dvin] = o;
      }
    }
  }
  // where the state goes
  float* dst = nullptr;
  if (MODE == 0 || (MODE == 3 && last)) dst = a.state + ((size_t)slot * a.H + h) * D * Dv;
  if (MODE == 1) dst = a.carry + ((size_t)c * a.H + h) * D * Dv;
  if (dst) {
#pragma unroll
    for (int n = 0; n < NC; ++n)
#pragma unroll
      for (int i = 0; i < DPT; ++i)
        if (d0 + i < D && col + 32 * n < Dvin) dst[(size_t)(d0 + i) * Dv + col + 32 * n] = s[n][i];
    if (norm_here) {
#pragma unroll
      for (int u = 0; u < NPL; ++u) {
        const int i = lane + 32 * u;
        if (i < DPT && d0 + i < D) dst[(size_t)(d0 + i) * Dv + Dvin] = nn[u];
      }
    }
  }
  if (MODE == 1 && blockIdx.z == 0 && group == 0 && lane == 0) {
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < D) a.decay_prod[((size_t)c * a.H + h) * D + d0 + i] = pa[i];
  }
}

// Step 2: a thread per state element of a (segment, head) walks the segment's chunks.
__global__ void gla_carry_kernel(GlaArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.y, h = blockIdx.z;
  const int first = a.seg_chunks[seg * 2], n = a.seg_chunks[seg * 2 + 1];
  if (n <= 1 || first < 0 || first + n > a.n_chunks) return;
  const int slot = a.state_slots[seg];
  if (slot < 0 || slot >= a.n_slots) return;
  const size_t DV = (size_t)a.D * a.Dv;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= DV) return;
  const int d = (int)(e / a.Dv);
  const bool fresh = a.seg_info[seg * 4 + 2] - a.seg_info[seg * 4 + 1] == 0;
  float s = fresh ? 0.f : a.state[((size_t)slot * a.H + h) * DV + e];
  a.carry[((size_t)(first + n - 1) * a.H + h) * DV + e] = s;
  for (int c = first; c < first + n - 1; ++c) {
    float* l = a.carry + ((size_t)c * a.H + h) * DV + e;
    s = fmaf(a.decay_prod[((size_t)c * a.H + h) * a.D + d], s, *l);
    *l = s;
  }
}

template <typename T, int DPT>
static int launch_gla(GlaArgs a, bool any_single, bool any_multi, cudaStream_t s) {
  const int Dp = DPT * kGlaSlices;
  constexpr int kGlaCols = 32 * gla_cols_per_thread(DPT);
  const int dv_real = a.Dv - a.ones_col;  // the column of ones rides in the block of the first columns
  const int tiles = (dv_real + kGlaCols - 1) / kGlaCols;
  a.groups = min(tiles, gla_max_groups(DPT));
  const int cols = a.groups * kGlaCols;
  const int threads = a.groups * kGlaSlices * 32;
  size_t smem = ((size_t)3 * kGlaBatch * Dp + (size_t)kGlaBatch * cols + (size_t)kGlaSlices * kGlaBatch * cols +
                 (size_t)kGlaSlices * kGlaBatch) * sizeof(float);
  if (sizeof(T) == 2)  // the next batch as it lies in memory: q, k (bfloat16), decay logits (float), values (bfloat16)
    smem += (size_t)kGlaBatch * Dp * (2 + 2 + 4) + (size_t)kGlaBatch * cols * 2 + (size_t)2 * kGlaBatch * 4;
  dim3 grid(a.n_chunks, a.H, (dv_real + cols - 1) / cols);
  auto k0 = gla_chunk_kernel<T, DPT, 0>;
  auto k1 = gla_chunk_kernel<T, DPT, 1>;
  auto k3 = gla_chunk_kernel<T, DPT, 3>;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  if (any_multi && !a.a_head) {  // the decays of all of the step's tokens, once, where the logits lay
    const long long n = (long long)a.n_tokens * a.H * a.D;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    FTK_LAUNCH(gla_decay_kernel, blocks, 256, 0, s, a.z, a.z_bias, n, a.H * a.D, a.inv_tau);
    FTK_LAUNCH_CHECK("gla_scan (decays)");
    a.z_is_decay = 1;
  }
  if (any_single) {
    FTK_LAUNCH(k0, grid, threads, smem, s, a);
    FTK_LAUNCH_CHECK("gla_scan (one chunk per request)");
  }
  if (any_multi) {
    FTK_LAUNCH(k1, grid, threads, smem, s, a);
    FTK_LAUNCH_CHECK("gla_scan (chunk contributions)");
    const size_t DV = (size_t)a.D * a.Dv;
    dim3 cgrid((unsigned)((DV + 255) / 256), a.n_segs, a.H);
    FTK_LAUNCH(gla_carry_kernel, cgrid, 256, 0, s, a);
    FTK_LAUNCH_CHECK("gla_scan (carry)");
    FTK_LAUNCH(k3, grid, threads, smem, s, a);
    FTK_LAUNCH_CHECK("gla_scan (chunk outputs)");
  }
  return 0;
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_gla_scan(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                            long long v_stride, int dtype, float* z, const float* z_bias, float tau,
                            float q_scale, float* state, int n_slots, const int32_t* state_slots,
                            const int32_t* seg_info, int n_segs, const int32_t* chunks, int n_chunks,
                            const int32_t* seg_chunks, int any_single, int any_multi, float* carry,
                            float* decay_prod, float* out, int n_tokens, int n_heads, int dim, int vdim,
                            const float* k_fac, const float* a_head, int ones_col, float* out_ones, int qk_div,
                            void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "gla_scan: bad dtype %d", dtype);
  FTK_REQUIRE(n_tokens >= 0 && n_segs >= 0 && n_chunks >= 0, "gla_scan: bad counts");
  if (n_tokens == 0 || n_chunks == 0) return 0;
  FTK_REQUIRE(n_heads >= 1 && n_heads <= 65535 && dim >= 1 && dim <= 256 && vdim >= 1 && vdim <= 65535 * 32,
              "gla_scan: %d heads of %d key and %d value channels are not taken (at most 256 key channels)", n_heads,
              dim, vdim);
  FTK_REQUIRE(n_segs <= 65535, "gla_scan: too many segments");
  FTK_REQUIRE(tau > 0.f, "gla_scan: tau must be positive");
  FTK_REQUIRE(ones_col == 0 || (ones_col == 1 && vdim >= 2), "gla_scan: a column of ones needs a value column beside it");
  FTK_REQUIRE(q && k && v && (z || a_head) && state && state_slots && seg_info && chunks && seg_chunks && out,
              "gla_scan: null pointer");
  FTK_REQUIRE(!any_multi || (carry && decay_prod), "gla_scan: portions of several chunks need scratch");
  GlaArgs a;
  a.q = q; a.k = k; a.v = v; a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
  a.z = z; a.z_bias = z_bias; a.z_is_decay = 0; a.groups = 1; a.inv_tau = 1.f / tau; a.q_scale = q_scale;
  a.state = state; a.state_slots = state_slots; a.seg_info = seg_info; a.chunks = chunks; a.seg_chunks = seg_chunks;
  a.n_chunks = n_chunks; a.n_segs = n_segs; a.n_slots = n_slots; a.carry = carry; a.decay_prod = decay_prod;
  FTK_REQUIRE(!out_ones || ones_col, "gla_scan: outputs of a column of ones that is not there");
  FTK_REQUIRE(qk_div >= 1 && n_heads % qk_div == 0 && (qk_div == 1 || a_head),
              "gla_scan: heads that share queries and keys come in groups that divide the heads, with a decay per head");
  a.k_fac = k_fac; a.a_head = a_head; a.ones_col = ones_col; a.out_ones = out_ones; a.qk_div = qk_div;
  a.out = out; a.H = n_heads; a.D = dim; a.Dv = vdim; a.n_tokens = n_tokens;
  cudaStream_t s = (cudaStream_t)stream;
  note_variant(any_multi ? "gla_scan: chunks side by side" : "gla_scan: one chunk per request");
  const bool f32 = dtype == FTK_F32;
  if (dim <= 32) return f32 ? launch_gla<float, 8>(a, any_single, any_multi, s) : launch_gla<__nv_bfloat16, 8>(a, any_single, any_multi, s);
  if (dim <= 64) return f32 ? launch_gla<float, 16>(a, any_single, any_multi, s) : launch_gla<__nv_bfloat16, 16>(a, any_single, any_multi, s);
  if (dim <= 128) return f32 ? launch_gla<float, 32>(a, any_single, any_multi, s) : launch_gla<__nv_bfloat16, 32>(a, any_single, any_multi, s);
  return f32 ? launch_gla<float, 64>(a, any_single, any_multi, s) : launch_gla<__nv_bfloat16, 64>(a, any_single, any_multi, s);
}
