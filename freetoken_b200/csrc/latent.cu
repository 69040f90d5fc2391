// Latent attention: what a token leaves in the cache and what its query looks like.
//
// latent_store, a block per token, from the row of the one input projection [query latent | key/value latent |
// rotated key part]: the query latent is RMS-normed (plain weight) into a dense row for the up-projection; the
// key/value latent is RMS-normed, the shared key part rotated by the token's position, and both go into the
// token's cache row as [latent | rotated part | zeros up to the padded size].  Norms and rotation are 32-bit.
//
// latent_query_rotate: the rotated part of every head's query is turned by the token's position and written
// behind the latent part of the query row that the attention kernel reads ([latent | rotated part | zeros]).
//
// Rotation: among the first n_rot dimensions of the part, pair i is (2i, 2i + 1) in the interleaved layout and
// (i, i + n_rot / 2) otherwise; the table holds cos || sin of position * base^(-2i / n_rot) per position.
#include "common.cuh"

namespace ftk {

__device__ __forceinline__ float rotated_at(const float* v, int d, int n_rot, int interleaved, const float* tab) {
  // `v` holds the part's values, `tab` the position's row of the table (cos[n_rot/2] || sin[n_rot/2])
  if (d >= n_rot) return v[d];
  const int half = n_rot >> 1;
  int i, partner;
  bool is_first;
  if (interleaved) { i = d >> 1; is_first = (d & 1) == 0; partner = is_first ? d + 1 : d - 1; }
  else { is_first = d < half; i = is_first ? d : d - half; partner = is_first ? d + half : d - half; }
  const float c = tab[i], s = tab[half + i];
  return is_first ? v[d] * c - v[partner] * s : v[d] * c + v[partner] * s;
}

template <typename T>
__global__ void latent_store_kernel(const T* __restrict__ proj, long long row_stride, int q_rank, int kv_rank, int rot_dim,
                                    int n_rot, int interleaved, const float* __restrict__ wq, const float* __restrict__ wkv,
                                    float eps, const int32_t* __restrict__ positions, const float* __restrict__ table,
                                    int max_pos, T* __restrict__ cq_out, T* __restrict__ slab, long long slab_rows,
                                    const int32_t* __restrict__ slot_map, int pad_dim) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sm[];  // the row in 32-bit, then 33 floats of scratch
  const int t = blockIdx.x;
  const int width = q_rank + kv_rank + rot_dim;
  float* row = sm;
  float* scratch = sm + width;
  const T* src = proj + (size_t)t * row_stride;
  float sq = 0.f, skv = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_float(src[i]);
    row[i] = v;
    if (i < q_rank) sq += v * v;
    else if (i < q_rank + kv_rank) skv += v * v;
  }
  sq = block_sum(sq, scratch);
  skv = block_sum(skv, scratch);
  const float rq = q_rank ? rsqrtf(sq / (float)q_rank + eps) : 0.f, rkv = rsqrtf(skv / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq_out[(size_t)t * q_rank + i] = from_float<T>(row[i] * rq * wq[i]);
  const long long slot = slot_map[t];
  if (slot < 0 || slot >= slab_rows) return;  // a position whose page a window has already passed is not stored
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const float* tab = table ? table + (size_t)pos * n_rot : nullptr;
  T* dst = slab + (size_t)slot * pad_dim;
  const float* c = row + q_rank;
  const float* kr = c + kv_rank;
  for (int i = threadIdx.x; i < pad_dim; i += blockDim.x) {
    float v = 0.f;
    if (i < kv_rank) v = c[i] * rkv * wkv[i];
    else if (i < kv_rank + rot_dim) v = tab ? rotated_at(kr, i - kv_rank, n_rot, interleaved, tab) : kr[i - kv_rank];
    dst[i] = from_float<T>(v);
  }
}

__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store2(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
__device__ __forceinline__ void store2(__nv_bfloat16* p, float2 v) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
}

template <typename T>
__global__ void latent_query_rotate_kernel(const T* __restrict__ q, int n_heads, int flat_dim, int rot_dim, int n_rot,
                                           int interleaved, const int32_t* __restrict__ positions,
                                           const float* __restrict__ table, int max_pos, T* __restrict__ q_out,
                                           int kv_rank, int pad_dim, int heads_per_block) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sm[];  // [heads of this block][rot_dim]
  const int t = blockIdx.x, h0 = blockIdx.y * heads_per_block;
  const int qd = flat_dim + rot_dim;
  const T* src = q + ((size_t)t * n_heads + h0) * qd;
  const int all_heads = n_heads;
  n_heads = min(heads_per_block, n_heads - h0);  // from here on: the block's heads
  // two values at a time where every offset is even (the rows themselves start on a multiple of their even widths)
  const bool pairs = ((rot_dim | flat_dim | kv_rank | pad_dim) & 1) == 0;
  if (pairs) {
    const int half = rot_dim / 2;
    for (int i = threadIdx.x; i < n_heads * half; i += blockDim.x) {
      const int h = i / half, d = (i - h * half) * 2;
      const float2 v = load2(src + (size_t)h * qd + flat_dim + d);
      sm[h * rot_dim + d] = v.x;
      sm[h * rot_dim + d + 1] = v.y;
    }
  } else {
    for (int i = threadIdx.x; i < n_heads * rot_dim; i += blockDim.x) {
      const int h = i / rot_dim, d = i - h * rot_dim;
      sm[i] = to_float(src[(size_t)h * qd + flat_dim + d]);
    }
  }
  __syncthreads();
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const float* tab = table ? table + (size_t)pos * n_rot : nullptr;
  const int tail = pad_dim - kv_rank;
  T* dst = q_out + ((size_t)t * all_heads + h0) * pad_dim;
  if (pairs) {
    const int half = tail / 2;
    for (int i = threadIdx.x; i < n_heads * half; i += blockDim.x) {
      const int h = i / half, d = (i - h * half) * 2;
      float2 v = make_float2(0.f, 0.f);
      if (d < rot_dim) {
        v.x = tab ? rotated_at(sm + h * rot_dim, d, n_rot, interleaved, tab) : sm[h * rot_dim + d];
        v.y = tab ? rotated_at(sm + h * rot_dim, d + 1, n_rot, interleaved, tab) : sm[h * rot_dim + d + 1];
      }
      store2(dst + (size_t)h * pad_dim + kv_rank + d, v);
    }
    return;
  }
  for (int i = threadIdx.x; i < n_heads * tail; i += blockDim.x) {
    const int h = i / tail, d = i - h * tail;
    float v = 0.f;
    if (d < rot_dim) v = tab ? rotated_at(sm + h * rot_dim, d, n_rot, interleaved, tab) : sm[h * rot_dim + d];
    dst[(size_t)h * pad_dim + kv_rank + d] = from_float<T>(v);
  }
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_latent_store(const void* proj, int dtype, long long row_stride, int q_rank, int kv_rank, int rot_dim,
                                int n_rot, int interleaved, const float* wq, const float* wkv, float eps,
                                const int32_t* positions, const float* table, int max_pos, void* cq_out, void* slab,
                                long long slab_rows, const int32_t* slot_map, int pad_dim, int n_tokens, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "latent_store: bad dtype %d", dtype);
  FTK_REQUIRE(q_rank >= 0 && kv_rank >= 1 && rot_dim >= 0 && n_rot >= 0 && n_rot <= rot_dim && n_rot % 2 == 0 &&
              pad_dim >= kv_rank + rot_dim && n_tokens >= 0, "latent_store: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(proj && (q_rank == 0 || (wq && cq_out)) && wkv && positions && slab && slot_map && (n_rot == 0 || table),
              "latent_store: null pointer");
  const int width = q_rank + kv_rank + rot_dim;
  const size_t smem = (size_t)(width + 33) * sizeof(float);
  FTK_REQUIRE(smem <= 48 * 1024, "latent_store: rows of %d values do not fit", width);
  const int threads = width >= 1024 ? 256 : 128;
  cudaStream_t s = (cudaStream_t)stream;
  const float* tab = n_rot ? table : nullptr;
  if (dtype == FTK_F32)
    FTK_LAUNCH(latent_store_kernel<float>, n_tokens, threads, smem, s, (const float*)proj, row_stride, q_rank, kv_rank, rot_dim,
               n_rot, interleaved, wq, wkv, eps, positions, tab, max_pos, (float*)cq_out, (float*)slab, slab_rows, slot_map,
               pad_dim);
  else
    FTK_LAUNCH(latent_store_kernel<__nv_bfloat16>, n_tokens, threads, smem, s, (const __nv_bfloat16*)proj, row_stride, q_rank,
               kv_rank, rot_dim, n_rot, interleaved, wq, wkv, eps, positions, tab, max_pos, (__nv_bfloat16*)cq_out,
               (__nv_bfloat16*)slab, slab_rows, slot_map, pad_dim);
  FTK_LAUNCH_CHECK("latent_store");
  return 0;
}

extern "C" int ftk_latent_query_rotate(const void* q, int dtype, int n_heads, int flat_dim, int rot_dim, int n_rot,
                                       int interleaved, const int32_t* positions, const float* table, int max_pos,
                                       void* q_out, int kv_rank, int pad_dim, int n_tokens, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "latent_query_rotate: bad dtype %d", dtype);
  FTK_REQUIRE(n_heads >= 1 && flat_dim >= 0 && rot_dim >= 0 && n_rot >= 0 && n_rot <= rot_dim && n_rot % 2 == 0 &&
              pad_dim >= kv_rank + rot_dim && n_tokens >= 0, "latent_query_rotate: bad sizes");
  if (n_tokens == 0 || pad_dim == kv_rank) return 0;
  FTK_REQUIRE(q && positions && q_out && (n_rot == 0 || table), "latent_query_rotate: null pointer");
  // a block takes a token's heads in groups that give its 128 threads two values each to read and pad_dim - kv_rank to write
  const int per = max(1, min(n_heads, 256 / max(rot_dim, 1)));
  const size_t smem = (size_t)per * rot_dim * sizeof(float) + 16;
  FTK_REQUIRE(smem <= 48 * 1024, "latent_query_rotate: %d rotated values a head do not fit", rot_dim);
  FTK_REQUIRE((n_heads + per - 1) / per <= 65535, "latent_query_rotate: too many heads");
  const dim3 grid(n_tokens, (n_heads + per - 1) / per);
  cudaStream_t s = (cudaStream_t)stream;
  const float* tab = n_rot ? table : nullptr;
  if (dtype == FTK_F32)
    FTK_LAUNCH(latent_query_rotate_kernel<float>, grid, 128, smem, s, (const float*)q, n_heads, flat_dim, rot_dim, n_rot,
               interleaved, positions, tab, max_pos, (float*)q_out, kv_rank, pad_dim, per);
  else
    FTK_LAUNCH(latent_query_rotate_kernel<__nv_bfloat16>, grid, 128, smem, s, (const __nv_bfloat16*)q, n_heads, flat_dim,
               rot_dim, n_rot, interleaved, positions, tab, max_pos, (__nv_bfloat16*)q_out, kv_rank, pad_dim, per);
  FTK_LAUNCH_CHECK("latent_query_rotate");
  return 0;
}
