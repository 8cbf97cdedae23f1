// Unit norm of query and key heads (each head divided by its root mean square, no gain), fused
// with the write of the new keys and values into the paged cache.  A value head may have another
// width than a key head.
//
//   y = x / sqrt(mean(x^2) + eps)  per head, statistics in float32
//
// One block per token, one warp per head in turn.  Query heads are normed in place; key heads are
// normed and stored into the cache (what the cache holds is the normed key), values are copied.
// Without a cache (a run that reads another run's keys and values) only the query heads are touched.
#include "common.cuh"

#define UN_THREADS 256

template <typename T>
__global__ void unit_norm_append_kernel(T* __restrict__ x, int row_stride, int n_q_heads, int head_dim, float eps,
                                        int k_off, int v_off, int n_kv_heads, int v_dim,
                                        const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                        const int* __restrict__ slots, const int* __restrict__ page_table,
                                        int pt_stride, T* __restrict__ k_cache, T* __restrict__ v_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  T* row = x + (size_t)t * row_stride;
  const int n_k = k_cache ? n_kv_heads : 0;
  const int pos = k_cache ? tok_pos[t] : 0;
  const int* pt = k_cache ? page_table + (size_t)slots[tok_seq[t]] * pt_stride : nullptr;
  for (int h = warp; h < n_q_heads + n_k; h += n_warps) {
    bool is_key = h >= n_q_heads;
    T* hd = is_key ? row + k_off + (size_t)(h - n_q_heads) * head_dim : row + (size_t)h * head_dim;
    float ss = 0.f;
    for (int d = lane; d < head_dim; d += 32) {
      float v = to_f32<T>(hd[d]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    float scale = 1.0f / sqrtf(ss / (float)head_dim + eps);
    T* dst = is_key ? k_cache + cache_row_offset(pt, pos, n_kv_heads, h - n_q_heads, head_dim) : hd;
    for (int d = lane; d < head_dim; d += 32) {
      T y = from_f32<T>(to_f32<T>(hd[d]) * scale);
      dst[d] = y;
      if (is_key) hd[d] = y;
    }
  }
  if (k_cache) {
    for (int e = threadIdx.x; e < n_kv_heads * v_dim; e += blockDim.x) {
      int kvh = e / v_dim, d = e - kvh * v_dim;
      v_cache[cache_row_offset(pt, pos, n_kv_heads, kvh, v_dim) + d] = row[v_off + e];
    }
  }
}

extern "C" int bn_unit_norm_append(void* x, int dtype, int n_tokens, int row_stride, int n_q_heads, int head_dim,
                                   float eps, int k_off, int v_off, int n_kv_heads, int v_dim, const int* tok_seq,
                                   const int* tok_pos, const int* slots, const int* page_table, int pt_stride,
                                   void* k_cache, void* v_cache, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!x || head_dim <= 0 || n_q_heads < 0 || !(eps > 0.f) || (k_cache && (!v_cache || n_kv_heads <= 0 || v_dim <= 0)))
    return BN_ERR_BAD_ARG;
  if (dtype == BN_F32)
    BN_LAUNCH(unit_norm_append_kernel<float>, n_tokens, UN_THREADS, 0, stream, (float*)x, row_stride, n_q_heads, head_dim,
              eps, k_off, v_off, n_kv_heads, v_dim, tok_seq, tok_pos, slots, page_table, pt_stride, (float*)k_cache,
              (float*)v_cache);
  else if (dtype == BN_BF16)
    BN_LAUNCH(unit_norm_append_kernel<__nv_bfloat16>, n_tokens, UN_THREADS, 0, stream, (__nv_bfloat16*)x, row_stride,
              n_q_heads, head_dim, eps, k_off, v_off, n_kv_heads, v_dim, tok_seq, tok_pos, slots, page_table, pt_stride,
              (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// RMS norms over whole slices of a row (all query heads of a token at once, and all key heads), each with a
// gain; values optionally blended with another tensor's rows; keys and values written into the paged cache.
//
//   q <- q / sqrt(mean(q^2) + eps) * wq   over q_len numbers at q_off;   k likewise over k_len at k_off
//   v <- (1 - blend) v + blend v_other    when v_other is given (row t of v_other lies at v_other + t * other_stride)
//
// One block per token.  Statistics and the blend are float32; what the cache gets is what the row then holds.
// Without a cache only the row is rewritten.
template <typename T>
__global__ void slice_norm_append_kernel(T* __restrict__ x, int row_stride, int q_off, int q_len, const void* __restrict__ wq,
                                         int k_off, int k_len, const void* __restrict__ wk, int w_dtype, float eps, int v_off,
                                         const T* __restrict__ v_other, int other_stride, float blend, int n_kv_heads,
                                         int head_dim, int v_dim, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                         const int* __restrict__ slots, const int* __restrict__ page_table, int pt_stride,
                                         T* __restrict__ k_cache, T* __restrict__ v_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  T* row = x + (size_t)t * row_stride;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < q_len; i += blockDim.x) {
    float a = to_f32<T>(row[q_off + i]);
    sq += a * a;
  }
  for (int i = threadIdx.x; i < k_len; i += blockDim.x) {
    float a = to_f32<T>(row[k_off + i]);
    sk += a * a;
  }
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);
  const int pos = k_cache ? tok_pos[t] : 0;
  const int* pt = k_cache ? page_table + (size_t)slots[tok_seq[t]] * pt_stride : nullptr;
  if (q_len > 0) {
    const float scale = 1.0f / sqrtf(sq / (float)q_len + eps);
    for (int i = threadIdx.x; i < q_len; i += blockDim.x)
      row[q_off + i] = from_f32<T>(to_f32<T>(row[q_off + i]) * scale * load_as_f32(wq, w_dtype, i));
  }
  const float kscale = k_len > 0 && wk ? 1.0f / sqrtf(sk / (float)k_len + eps) : 1.0f;
  for (int i = threadIdx.x; i < k_len; i += blockDim.x) {
    T y = wk ? from_f32<T>(to_f32<T>(row[k_off + i]) * kscale * load_as_f32(wk, w_dtype, i)) : row[k_off + i];
    row[k_off + i] = y;
    if (k_cache) {
      const int kvh = i / head_dim, d = i - kvh * head_dim;
      k_cache[cache_row_offset(pt, pos, n_kv_heads, kvh, head_dim) + d] = y;
    }
  }
  for (int i = threadIdx.x; i < n_kv_heads * v_dim; i += blockDim.x) {
    T y = row[v_off + i];
    if (v_other) {
      y = from_f32<T>((1.0f - blend) * to_f32<T>(y) + blend * to_f32<T>(v_other[(size_t)t * other_stride + i]));
      row[v_off + i] = y;
    }
    if (v_cache) {
      const int kvh = i / v_dim, d = i - kvh * v_dim;
      v_cache[cache_row_offset(pt, pos, n_kv_heads, kvh, v_dim) + d] = y;
    }
  }
}

extern "C" int bn_slice_norm_append(void* x, int dtype, int n_tokens, int row_stride, int q_off, int q_len, const void* wq,
                                    int k_off, int k_len, const void* wk, int w_dtype, float eps, int v_off, const void* v_other,
                                    int other_stride, float blend, int n_kv_heads, int head_dim, int v_dim, const int* tok_seq,
                                    const int* tok_pos, const int* slots, const int* page_table, int pt_stride, void* k_cache,
                                    void* v_cache, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!x || q_len < 0 || (q_len > 0 && !wq) || k_len != n_kv_heads * head_dim || n_kv_heads <= 0 || head_dim <= 0 || v_dim <= 0 ||
      !(eps > 0.f) || (k_cache && (!v_cache || !tok_seq || !tok_pos || !slots || !page_table)) ||
      (w_dtype != BN_F32 && w_dtype != BN_BF16))
    return BN_ERR_BAD_ARG;
  if (dtype == BN_F32)
    BN_LAUNCH(slice_norm_append_kernel<float>, n_tokens, UN_THREADS, 0, stream, (float*)x, row_stride, q_off, q_len, wq, k_off, k_len,
              wk, w_dtype, eps, v_off, (const float*)v_other, other_stride, blend, n_kv_heads, head_dim, v_dim, tok_seq, tok_pos,
              slots, page_table, pt_stride, (float*)k_cache, (float*)v_cache);
  else if (dtype == BN_BF16)
    BN_LAUNCH(slice_norm_append_kernel<__nv_bfloat16>, n_tokens, UN_THREADS, 0, stream, (__nv_bfloat16*)x, row_stride, q_off, q_len,
              wq, k_off, k_len, wk, w_dtype, eps, v_off, (const __nv_bfloat16*)v_other, other_stride, blend, n_kv_heads, head_dim,
              v_dim, tok_seq, tok_pos, slots, page_table, pt_stride, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}
