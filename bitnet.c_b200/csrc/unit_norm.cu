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

// Queries, keys and values of a token from the float32 rows of their projection: a bias added, RMS norms with gains
// over spans of the query slice and of the key slice, a factor on the queries that grows with the position, the
// row written out in the compute type, keys and values into the paged cache.
//
//   r = src + bias                                                     (float32)
//   q_j <- q_j / sqrt(mean over its span (q^2) + eps) * wq[j mod q_span] * (1 + coef ln(floor((p + 1) / every) + 1))
//   k_j <- k_j / sqrt(mean over its span (k^2) + eps) * wk[j mod k_span]
//
// A span of head_dim numbers norms every head by itself with one gain for all heads; a span of the whole slice
// norms all heads of a token at once.  Span 0: no norm.  every 0: no factor.  The value plane may have fewer heads
// than the key plane (n_v_heads).  One block per token; the row waits in shared memory between the phases.
// VEC: every slice, span and head begins and ends at a multiple of four numbers and all addresses are multiples of
// 16 bytes, so rows are read, written and placed into the pages four numbers at a time.
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const unsigned*>(&a);
  raw.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float4 gain4(const void* w, int dtype, int i) {
  if (dtype == BN_F32) return *reinterpret_cast<const float4*>((const float*)w + i);
  const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)w + i);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T, bool VEC>
__global__ void qk_norm_append_kernel(const float* __restrict__ src, int src_stride, const void* __restrict__ bias, int bias_dtype,
                                      T* __restrict__ out, int out_stride, int row_len, int q_len, int q_span,
                                      const void* __restrict__ wq, int k_off, int k_len, int k_span, const void* __restrict__ wk,
                                      int w_dtype, float eps, float temp_coef, int temp_every, int v_off, int n_kv_heads,
                                      int head_dim, int n_v_heads, int v_dim, const int* __restrict__ tok_seq,
                                      const int* __restrict__ tok_pos, const int* __restrict__ slots,
                                      const int* __restrict__ page_table, int pt_stride, T* __restrict__ k_cache,
                                      T* __restrict__ v_cache) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float qk_row[];  // row_len numbers, then one inverse root mean square per span
  float* inv = qk_row + row_len;
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const float* s = src + (size_t)t * src_stride;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < row_len; i += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(s + i);
      if (bias) {
        const float4 b = gain4(bias, bias_dtype, i);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      *reinterpret_cast<float4*>(qk_row + i) = a;
    }
  } else {
    for (int i = threadIdx.x; i < row_len; i += blockDim.x) qk_row[i] = s[i] + (bias ? load_as_f32(bias, bias_dtype, i) : 0.f);
  }
  __syncthreads();
  const int nq = q_span > 0 ? q_len / q_span : 0, nk = k_span > 0 ? k_len / k_span : 0;
  for (int g = warp; g < nq + nk; g += n_warps) {
    const bool is_k = g >= nq;
    const int span = is_k ? k_span : q_span;
    const float* p = qk_row + (is_k ? k_off + (g - nq) * k_span : g * q_span);
    float ss = 0.f;
    for (int d = lane; d < span; d += 32) ss = fmaf(p[d], p[d], ss);
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.0f / sqrtf(ss / (float)span + eps);
  }
  __syncthreads();
  const int pos = tok_pos[t];
  const float temp = temp_every > 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f) : 1.0f;
  const int* pt = k_cache ? page_table + (size_t)slots[tok_seq[t]] * pt_stride : nullptr;
  T* o = out + (size_t)t * out_stride;
  const int v_len = n_v_heads * v_dim;
  if constexpr (VEC) {
    for (int i = threadIdx.x * 4; i < row_len; i += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(qk_row + i);
      if (i < q_len) {
        float f = temp;
        if (q_span > 0) {
          const float4 g = gain4(wq, w_dtype, i % q_span);
          f *= inv[i / q_span];
          a.x *= g.x; a.y *= g.y; a.z *= g.z; a.w *= g.w;
        }
        a.x *= f; a.y *= f; a.z *= f; a.w *= f;
        store4<T>(o + i, a);
      } else if (i >= k_off && i < k_off + k_len) {
        const int j = i - k_off;
        if (k_span > 0) {
          const float4 g = gain4(wk, w_dtype, j % k_span);
          const float f = inv[nq + j / k_span];
          a.x *= g.x * f; a.y *= g.y * f; a.z *= g.z * f; a.w *= g.w * f;
        }
        store4<T>(o + i, a);
        if (k_cache) {
          const int kvh = j / head_dim, d = j - kvh * head_dim;
          store4<T>(k_cache + cache_row_offset(pt, pos, n_kv_heads, kvh, head_dim) + d, a);
        }
      } else {
        store4<T>(o + i, a);
        if (v_cache && i >= v_off && i < v_off + v_len) {
          const int j = i - v_off, vh = j / v_dim, d = j - vh * v_dim;
          store4<T>(v_cache + cache_row_offset(pt, pos, n_v_heads, vh, v_dim) + d, a);
        }
      }
    }
  } else {
  for (int i = threadIdx.x; i < row_len; i += blockDim.x) {
    float a = qk_row[i];
    if (i < q_len) {
      if (q_span > 0) a = a * inv[i / q_span] * load_as_f32(wq, w_dtype, i % q_span);
      a *= temp;
      o[i] = from_f32<T>(a);
    } else if (i >= k_off && i < k_off + k_len) {
      const int j = i - k_off;
      if (k_span > 0) a = a * inv[nq + j / k_span] * load_as_f32(wk, w_dtype, j % k_span);
      const T y = from_f32<T>(a);
      o[i] = y;
      if (k_cache) {
        const int kvh = j / head_dim, d = j - kvh * head_dim;
        k_cache[cache_row_offset(pt, pos, n_kv_heads, kvh, head_dim) + d] = y;
      }
    } else {
      const T y = from_f32<T>(a);
      o[i] = y;
      if (v_cache && i >= v_off && i < v_off + v_len) {
        const int j = i - v_off, vh = j / v_dim, d = j - vh * v_dim;
        v_cache[cache_row_offset(pt, pos, n_v_heads, vh, v_dim) + d] = y;
      }
    }
  }
  }
}

extern "C" int bn_qk_norm_append(const float* src, int src_stride, const void* bias, int bias_dtype, void* out, int dtype, int out_stride,
                                 int n_tokens, int row_len, int q_len, int q_span, const void* wq, int k_off, int k_len, int k_span,
                                 const void* wk, int w_dtype, float eps, float temp_coef, int temp_every, int v_off, int n_kv_heads,
                                 int head_dim, int n_v_heads, int v_dim, const int* tok_seq, const int* tok_pos, const int* slots,
                                 const int* page_table, int pt_stride, void* k_cache, void* v_cache, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!src || !out || !tok_pos || row_len <= 0 || row_len > src_stride || row_len > out_stride || q_len < 0 || k_len < 0 ||
      q_len > k_off || k_off + k_len > row_len || q_span < 0 || k_span < 0 || (q_span > 0 && (!wq || q_len % q_span)) ||
      (k_span > 0 && (!wk || k_len % k_span)) || !(eps > 0.f) || temp_every < 0 ||
      (k_cache && (!v_cache || !tok_seq || !slots || !page_table || n_kv_heads <= 0 || head_dim <= 0 || n_v_heads <= 0 || v_dim <= 0 ||
                   k_len != n_kv_heads * head_dim || v_off < k_off + k_len || v_off + n_v_heads * v_dim > row_len)))
    return BN_ERR_BAD_ARG;
  const int spans = (q_span > 0 ? q_len / q_span : 0) + (k_span > 0 ? k_len / k_span : 0);
  const size_t smem = ((size_t)row_len + spans) * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;
  // four numbers at a time when nothing begins or ends inside a group of four and every address is a multiple of 16 bytes
  const bool vec = !((row_len | src_stride | out_stride | q_len | k_off | k_len | v_off | q_span | k_span) & 3) &&
                   (!k_cache || !((head_dim | v_dim) & 3)) &&
                   !(((uintptr_t)src | (uintptr_t)bias | (uintptr_t)out | (uintptr_t)wq | (uintptr_t)wk | (uintptr_t)k_cache |
                      (uintptr_t)v_cache) & 15);
#define BN_QK_LAUNCH(TT, VV)                                                                                                   \
  BN_LAUNCH((qk_norm_append_kernel<TT, VV>), n_tokens, UN_THREADS, smem, stream, src, src_stride, bias, bias_dtype, (TT*)out,  \
            out_stride, row_len, q_len, q_span, wq, k_off, k_len, k_span, wk, w_dtype, eps, temp_coef, temp_every, v_off,      \
            n_kv_heads, head_dim, n_v_heads, v_dim, tok_seq, tok_pos, slots, page_table, pt_stride, (TT*)k_cache,              \
            (TT*)v_cache)
#define BN_QK_PREP(TT)                                                                                                         \
  do {                                                                                                                         \
    if (smem > 48 * 1024) {                                                                                                    \
      static size_t granted = 0;                                                                                               \
      if (smem > granted) {                                                                                                    \
        cudaError_t e = cudaFuncSetAttribute(qk_norm_append_kernel<TT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e == cudaSuccess)                                                                                                  \
          e = cudaFuncSetAttribute(qk_norm_append_kernel<TT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;                                                                   \
        granted = smem;                                                                                                        \
      }                                                                                                                        \
    }                                                                                                                          \
    if (vec) BN_QK_LAUNCH(TT, true);                                                                                           \
    else BN_QK_LAUNCH(TT, false);                                                                                              \
  } while (0)
  if (dtype == BN_F32) BN_QK_PREP(float);
  else if (dtype == BN_BF16) BN_QK_PREP(__nv_bfloat16);
  else return BN_ERR_BAD_ARG;
#undef BN_QK_PREP
#undef BN_QK_LAUNCH
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// Two maps of attention over the same values, combined: per token and head
//   o = a1 - lambda a2;   o <- o / sqrt(mean(o^2) + eps) * post
// a1 and a2 are float32 rows of v_dim numbers; the maps of the heads that share a key/value head lie as
// [group][map][head in group][v_dim] in a row of `in`.  One warp per (token, head).  tail > 0: behind the heads
// every row of out gets a one and tail - 1 zeros, so that the product that reads the rows adds a bias that is
// stored as a column of its matrix.
template <typename T>
__global__ void diff_combine_kernel(const float* __restrict__ in, int in_stride, T* __restrict__ out, int out_stride, int n_tokens,
                                    int n_heads, int per_group, int v_dim, float lambda, float eps, float post, int tail) {
  pdl_launch_dependents();
  pdl_wait();
  const int item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (item >= n_tokens * n_heads) return;
  const int t = item / n_heads, h = item - t * n_heads;
  const int g = h / per_group, hg = h - g * per_group;
  const float* a1 = in + (size_t)t * in_stride + ((size_t)(2 * g) * per_group + hg) * v_dim;
  const float* a2 = a1 + (size_t)per_group * v_dim;
  float ss = 0.f;
  for (int d = lane; d < v_dim; d += 32) {
    const float o = a1[d] - lambda * a2[d];
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  const float scale = post / sqrtf(ss / (float)v_dim + eps);
  T* orow = out + (size_t)t * out_stride + (size_t)h * v_dim;
  for (int d = lane; d < v_dim; d += 32) orow[d] = from_f32<T>((a1[d] - lambda * a2[d]) * scale);
  if (h == 0 && lane < tail) out[(size_t)t * out_stride + (size_t)n_heads * v_dim + lane] = from_f32<T>(lane == 0 ? 1.f : 0.f);
}

extern "C" int bn_diff_combine(const float* in, int in_stride, void* out, int dtype, int out_stride, int n_tokens, int n_heads,
                               int per_group, int v_dim, float lambda, float eps, float post, int tail, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!in || !out || n_heads <= 0 || per_group <= 0 || n_heads % per_group || v_dim <= 0 || !(eps > 0.f) || tail < 0 || tail > 32 ||
      in_stride < 2 * n_heads * v_dim || out_stride < n_heads * v_dim + tail)
    return BN_ERR_BAD_ARG;
  const long long items = (long long)n_tokens * n_heads;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  if (dtype == BN_F32)
    BN_LAUNCH(diff_combine_kernel<float>, blocks, 256, 0, stream, in, in_stride, (float*)out, out_stride, n_tokens, n_heads, per_group,
              v_dim, lambda, eps, post, tail);
  else if (dtype == BN_BF16)
    BN_LAUNCH(diff_combine_kernel<__nv_bfloat16>, blocks, 256, 0, stream, in, in_stride, (__nv_bfloat16*)out, out_stride, n_tokens,
              n_heads, per_group, v_dim, lambda, eps, post, tail);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}
