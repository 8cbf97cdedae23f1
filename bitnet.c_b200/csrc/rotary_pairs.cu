// Rotary position encoding with a table of frequencies, fused with the write of the new keys (and
// values) into the paged cache.
//
// Dimension 2i of the rotated part of a head is paired with dimension 2i + 1 (or, with split_halves,
// dimension i with dimension i + half); at position p the pair (u, v) becomes
// (u cos a - v sin a, v cos a + u sin a) with a = p * freq[i] in float32 (in double precision when the table comes
// as doubles, freqs64), cos and sin both times `magnitude`.  The
// frequencies come as a table, so that whoever builds it decides base, scaling of long
// wavelengths and the like (parts/position.py).  The rotated part may lie anywhere inside a head
// (rot_off), so heads of the form [plain | rotated] and keys whose last numbers are a rotated part
// shared by all heads take the same kernel.
//
// One block per token, phases with a barrier between them:
//   0  (optional) the first norm_len numbers of the key row divided by their root mean square, times a gain:
//      a latent that is cached normed, with its rotated part behind it (one key head)
//   1  value heads -> cache, as they are (they may be the key heads before rotation: v_off == k_off)
//   2  pairs of the query heads and of the key heads rotated in place
//   3  key heads -> cache
#include "common.cuh"

#define RP_THREADS 256
#define RP_MAX_HALF 256

template <typename T>
__global__ void rotary_pairs_append_kernel(T* xq, int q_row_stride, T* xk, int row_stride, const float* __restrict__ freqs, int half,
                                           const int* __restrict__ tok_pos, int q_off, int n_q_heads, int q_head_stride,
                                           int q_rot_off, int k_off, int n_k_heads, int k_head_stride, int k_rot_off,
                                           int k_row, int v_off, int v_head_stride, int v_row,
                                           const int* __restrict__ tok_seq, const int* __restrict__ slots,
                                           const int* __restrict__ page_table, int pt_stride, T* __restrict__ k_cache,
                                           T* __restrict__ v_cache, int norm_len, const void* __restrict__ norm_w,
                                           int norm_w_dtype, float norm_eps, int split_halves, float magnitude,
                                           const double* __restrict__ freqs64) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float cs[RP_MAX_HALF], sn[RP_MAX_HALF];
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  T* row = xk + (size_t)t * row_stride;    // the row that holds the key (and value) heads
  T* qrow = xq + (size_t)t * q_row_stride;  // the row that holds the query heads (may be the same)
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sv, cv;
    if (freqs64) {
      // the table in double precision: the angle is taken there too (at position p a float32 angle is off by up to
      // p * 6e-8 radians), a few hundred values per token
      double sd, cd;
      sincos((double)pos * freqs64[i], &sd, &cd);
      sv = (float)sd;
      cv = (float)cd;
    } else {
      sincosf((float)pos * freqs[i], &sv, &cv);
    }
    sn[i] = sv * magnitude;
    cs[i] = cv * magnitude;
  }
  const int* pt = k_cache ? page_table + (size_t)slots[tok_seq[t]] * pt_stride : nullptr;
  if (norm_len > 0) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < norm_len; i += blockDim.x) {
      const float a = to_f32<T>(row[k_off + i]);
      ss += a * a;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)norm_len + norm_eps);
    for (int i = threadIdx.x; i < norm_len; i += blockDim.x)
      row[k_off + i] = from_f32<T>(to_f32<T>(row[k_off + i]) * scale * load_as_f32(norm_w, norm_w_dtype, i));
    __syncthreads();
  }
  if (v_cache) {
    for (int e = threadIdx.x; e < n_k_heads * v_row; e += blockDim.x) {
      const int h = e / v_row, d = e - h * v_row;
      v_cache[cache_row_offset(pt, pos, n_k_heads, h, v_row) + d] = row[v_off + h * v_head_stride + d];
    }
  }
  __syncthreads();
  const int n_q = n_q_heads * half, n_k = n_k_heads * half;
  for (int item = threadIdx.x; item < n_q + n_k; item += blockDim.x) {
    const bool is_q = item < n_q;
    const int it = is_q ? item : item - n_q;
    const int h = it / half, i = it - h * half;
    T* p = (is_q ? qrow + q_off + h * q_head_stride + q_rot_off : row + k_off + h * k_head_stride + k_rot_off);
    // the pair's two numbers: neighbours (2i, 2i + 1), or number i of the first half with number i of the second
    T* pu = p + (split_halves ? i : 2 * i);
    T* pv = p + (split_halves ? i + half : 2 * i + 1);
    const float u = to_f32<T>(*pu), v = to_f32<T>(*pv), c = cs[i], s = sn[i];
    *pu = from_f32<T>(u * c - v * s);
    *pv = from_f32<T>(v * c + u * s);
  }
  if (!k_cache) return;
  __syncthreads();
  for (int e = threadIdx.x; e < n_k_heads * k_row; e += blockDim.x) {
    const int h = e / k_row, d = e - h * k_row;
    k_cache[cache_row_offset(pt, pos, n_k_heads, h, k_row) + d] = row[k_off + h * k_head_stride + d];
  }
}

// xq [n, q_row_stride] and xk [n, row_stride] of `dtype` (they may be one tensor); freqs [half] float32.  Query heads: n_q_heads heads from element q_off,
// q_head_stride apart, the rotated part 2 * half wide from q_rot_off inside each; key heads likewise.
// With k_cache: head h of the keys (its first k_row numbers, after rotation) goes to the cache
// [pages, n_k_heads, BN_PAGE, k_row]; with v_cache the first v_row numbers of the heads at v_off go,
// unrotated, to [pages, n_k_heads, BN_PAGE, v_row].  norm_len > 0 (one key head, norm_len <= k_rot_off): the key row's
// first norm_len numbers are RMS-normed with the gain norm_w first, in place.
extern "C" int bn_rotary_pairs_append(void* xq, int q_row_stride, void* xk, int dtype, int n, int row_stride, const float* freqs, int half,
                                      const int* tok_pos, int q_off, int n_q_heads, int q_head_stride, int q_rot_off,
                                      int k_off, int n_k_heads, int k_head_stride, int k_rot_off, int k_row, int v_off,
                                      int v_head_stride, int v_row, const int* tok_seq, const int* slots,
                                      const int* page_table, int pt_stride, void* k_cache, void* v_cache,
                                      int norm_len, const void* norm_w, int norm_w_dtype, float norm_eps,
                                      int split_halves, float magnitude, const double* freqs64, cudaStream_t stream) {
  if (n <= 0) return BN_OK;
  if (norm_len < 0 || (norm_len > 0 && (!norm_w || n_k_heads != 1 || norm_len > k_rot_off || !(norm_eps > 0.f) ||
                                        (norm_w_dtype != BN_F32 && norm_w_dtype != BN_BF16))))
    return BN_ERR_BAD_ARG;
  if ((n_q_heads > 0 && !xq) || (n_k_heads > 0 && !xk) || !tok_pos || half < 0 || half > RP_MAX_HALF || (half > 0 && !freqs) || n_q_heads < 0 || n_k_heads < 0 ||
      (n_q_heads > 0 && (q_off < 0 || q_rot_off < 0 || q_rot_off + 2 * half > q_head_stride ||
                         q_off + n_q_heads * q_head_stride > q_row_stride)) ||
      (n_k_heads > 0 && (k_off < 0 || k_rot_off < 0 || k_rot_off + 2 * half > k_head_stride ||
                         k_off + n_k_heads * k_head_stride > row_stride)))
    return BN_ERR_BAD_ARG;
  if (k_cache && (!tok_seq || !slots || !page_table || n_k_heads <= 0 || k_row <= 0 || k_row > k_head_stride)) return BN_ERR_BAD_ARG;
  if (v_cache && (!k_cache || v_row <= 0 || v_off < 0 || v_row > v_head_stride || v_off + n_k_heads * v_head_stride > row_stride))
    return BN_ERR_BAD_ARG;
  if (dtype == BN_F32)
    BN_LAUNCH(rotary_pairs_append_kernel<float>, n, RP_THREADS, 0, stream, (float*)xq, q_row_stride, (float*)xk, row_stride, freqs, half, tok_pos, q_off,
              n_q_heads, q_head_stride, q_rot_off, k_off, n_k_heads, k_head_stride, k_rot_off, k_row, v_off, v_head_stride,
              v_row, tok_seq, slots, page_table, pt_stride, (float*)k_cache, (float*)v_cache, norm_len, norm_w, norm_w_dtype, norm_eps,
              split_halves, magnitude, freqs64);
  else if (dtype == BN_BF16)
    BN_LAUNCH(rotary_pairs_append_kernel<__nv_bfloat16>, n, RP_THREADS, 0, stream, (__nv_bfloat16*)xq, q_row_stride,
              (__nv_bfloat16*)xk, row_stride, freqs, half,
              tok_pos, q_off, n_q_heads, q_head_stride, q_rot_off, k_off, n_k_heads, k_head_stride, k_rot_off, k_row, v_off,
              v_head_stride, v_row, tok_seq, slots, page_table, pt_stride, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, norm_len,
              norm_w, norm_w_dtype, norm_eps, split_halves, magnitude, freqs64);
  else
    return BN_ERR_BAD_ARG;
  return BN_OK;
}
