// Causal softmax attention over the paged cache, for any mix of new tokens: whole
// prompts, pieces of prompts, or one token per sequence.  One block per (token, head).
// This is the general kernel: it serves the float32 path and every shape; the
// bfloat16 path uses the specialised kernels in attention_prefill.cu and
// attention_decode.cu where they apply.
//
// Reference: for query head h the key/value head is h / (n_heads / n_kv_heads);
// s_i = (q . K[t_i]) * scale over the causal range only, p = softmax(s) with the
// maximum subtracted, out = sum_i p_i V[t_i]   (src/transformer/gqa_scalar.c:61-121,
// prefill: src/transformer/batched_attn_scalar.c:97-169).  The online form with a
// running maximum and sum is the reference's flash variant (gqa_scalar.c:127-207).
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_CHUNK 128

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* o) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float* o) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
  }
};

// 1 / (l + e^(sink - m)) for sums l taken relative to the maximum m, also when the sink exceeds every score
__device__ __forceinline__ float sink_inverse(float m, float l, float sink) {
  const float top = fmaxf(m, sink);
  const float a = expf(m - top);
  return a / (l * a + expf(sink - top));
}

// a result number: in the compute type, or (out_wide) as float32 into an output that is a float32 array
template <typename T>
__device__ __forceinline__ void store_result(T* out, int out_wide, size_t at, float v) {
  if (out_wide) reinterpret_cast<float*>(out)[at] = v;
  else out[at] = from_f32<T>(v);
}

// Optional extras, each off when its pointer is null or its number zero, so that one kernel
// serves every softmax attention of the library:
//   v_dim        width of a value head when it differs from a key head's
//   keep_first   with a window: keys at positions below keep_first stay visible however far back
//   rel, n_rel   additive bias by distance, rel[min(pos - p, n_rel - 1) * n_heads + h] (float32; the
//                scale does not multiply it)
//   gate         per token and head a number whose logistic function multiplies the head's output
//   chunk        positions are cut into chunks of this many and a token sees the earlier keys of its own
//                chunk only (takes the place of the window)
//   v_row        width of a row of the value plane when it is more than v_dim: the values are the first
//                v_dim numbers of each row (the key plane itself, for values that are a part of the keys)
//   sink         per head a score (float32) that stands in the softmax's denominator once, without a key and
//                without a value: the weights then sum to less than one
//   out_wide     the output is a float32 array whatever the compute type (what follows wants the sums unrounded)
//   v_share      so many consecutive key heads read one value head (the value plane has n_kv_heads / v_share
//                heads): several maps of scores over the same values
template <typename T>
__global__ void attention_general_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                                         int out_stride, int n_heads, int n_kv_heads, int head_dim, int v_dim,
                                         float scale, int window, int keep_first, int chunk, int v_row,
                                         const float* __restrict__ rel, int n_rel, const T* __restrict__ gate, int gate_stride,
                                         const int* __restrict__ tok_seq,
                                         const int* __restrict__ tok_pos, const int* __restrict__ slots,
                                         const int* __restrict__ page_table, int pt_stride,
                                         const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                         float* __restrict__ part, int n_splits, const float* __restrict__ sink, int v_share, int out_wide) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  extern __shared__ __align__(16) float sm[];
  float* qs = sm;                    // head_dim
  float* ps = qs + head_dim;         // ATT_CHUNK scores, then probabilities
  float* scratch = ps + ATT_CHUNK;   // 32
  int t = blockIdx.x, h = blockIdx.y;
  int kvh = h / (n_heads / n_kv_heads);
  const int vh = kvh / v_share, n_v_heads = n_kv_heads / v_share;
  int pos = tok_pos[t];
  const int* pt = page_table + (size_t)slots[tok_seq[t]] * pt_stride;
  int lo = chunk > 0 ? (pos / chunk) * chunk : (window > 0 ? max(0, pos - window + 1) : 0);
  // visible keys: positions [0, n_first) and [lo, pos]; u counts through both ranges
  int n_first = min(keep_first, lo);
  int n_keys = n_first + pos - lo + 1;

  const T* qrow = q + (size_t)t * q_stride + (size_t)h * head_dim;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) qs[d] = to_f32<T>(qrow[d]);
  __syncthreads();

  constexpr int VN = Vec16<T>::N;
  constexpr int MAX_D = 8;  // output dims per thread when a row is not read in 16-byte pieces: v_dim <= 1024
  // Weighted sum of the values.  Rows of whole 16-byte pieces: a row is read by v_dim / VN threads,
  // one piece each, and the rows of a chunk are shared out over the groups of such threads; the
  // groups' sums meet in shared memory at the end.  Other widths: one thread per dimension.
  const bool wide = (v_dim % VN) == 0 && (v_row % VN) == 0 && v_dim / VN <= ATT_THREADS;
  const int per_row = wide ? v_dim / VN : 1, groups = wide ? ATT_THREADS / per_row : 1;
  const int piece = threadIdx.x % per_row, group = threadIdx.x / per_row;
  float acc[MAX_D];
#pragma unroll
  for (int r = 0; r < MAX_D; ++r) acc[r] = 0.f;
  float accv[VN];
#pragma unroll
  for (int e = 0; e < VN; ++e) accv[e] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  // with n_splits > 1 the chunks of keys are dealt out to the blocks blockIdx.z = 0 .. n_splits - 1, which
  // leave their running maximum, sum and unnormalised output in `part` for attention_merge_kernel
  for (int base = blockIdx.z * ATT_CHUNK; base < n_keys; base += ATT_CHUNK * n_splits) {
    int n = min(ATT_CHUNK, n_keys - base);
    float s = -INFINITY;
    if ((int)threadIdx.x < n) {
      int u = base + threadIdx.x;
      int p = u < n_first ? u : lo + (u - n_first);
      const T* krow = k_cache + cache_row_offset(pt, p, n_kv_heads, kvh, head_dim);
      float dot = 0.f;
      if (head_dim % VN == 0) {  // rows of whole 16-byte pieces
        for (int d = 0; d < head_dim; d += VN) {
          float kv[VN];
          Vec16<T>::load(krow + d, kv);
          const float4* q4 = reinterpret_cast<const float4*>(qs + d);  // four numbers of q per read
#pragma unroll
          for (int e = 0; e < VN / 4; ++e) {
            const float4 a = q4[e];
            dot = fmaf(a.x, kv[4 * e], dot); dot = fmaf(a.y, kv[4 * e + 1], dot);
            dot = fmaf(a.z, kv[4 * e + 2], dot); dot = fmaf(a.w, kv[4 * e + 3], dot);
          }
        }
      } else {
        for (int d = 0; d < head_dim; ++d) dot = fmaf(qs[d], to_f32<T>(krow[d]), dot);
      }
      s = dot * scale;
      if (rel) s += rel[(size_t)min(pos - p, n_rel - 1) * n_heads + h];
    }
    float m_chunk = block_max(s, scratch);
    float m_new = fmaxf(m_run, m_chunk);
    float alpha = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
    float p_mine = ((int)threadIdx.x < n) ? expf(s - m_new) : 0.f;
    ps[threadIdx.x] = p_mine;
    float l_chunk = block_sum(p_mine, scratch);  // has the barrier that publishes ps[]
    l_run = l_run * alpha + l_chunk;
    m_run = m_new;
    if (wide) {
#pragma unroll
      for (int e = 0; e < VN; ++e) accv[e] *= alpha;
      if (group < groups) {
        for (int j = group; j < n; j += groups) {
          int u = base + j;
          int p = u < n_first ? u : lo + (u - n_first);
          float vv[VN];
          Vec16<T>::load(v_cache + cache_row_offset(pt, p, n_v_heads, vh, v_row) + piece * VN, vv);
          float w = ps[j];
#pragma unroll
          for (int e = 0; e < VN; ++e) accv[e] = fmaf(w, vv[e], accv[e]);
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < MAX_D; ++r) {
        int d = threadIdx.x + r * ATT_THREADS;
        if (d < v_dim) {
          float a = acc[r] * alpha;
          for (int j = 0; j < n; ++j) {
            int u = base + j;
            int p = u < n_first ? u : lo + (u - n_first);
            const T* vrow = v_cache + cache_row_offset(pt, p, n_v_heads, vh, v_row);
            a = fmaf(ps[j], to_f32<T>(vrow[d]), a);
          }
          acc[r] = a;
        }
      }
    }
    __syncthreads();  // ps[] is rewritten by the next chunk
  }
  float inv = sink && !part ? sink_inverse(m_run, l_run, sink[h]) : 1.0f / l_run;
  if (gate) inv *= 1.0f / (1.0f + expf(-to_f32<T>(gate[(size_t)t * gate_stride + h])));
  const size_t orow = (size_t)t * out_stride + (size_t)h * v_dim;
  float* prow = part ? part + (((size_t)t * n_heads + h) * n_splits + blockIdx.z) * (v_dim + 2) : nullptr;
  if (prow && threadIdx.x == 0) { prow[0] = m_run; prow[1] = l_run; }
  if (wide) {
    // groups * v_dim <= ATT_THREADS * VN floats, kept behind the scores
    float* red = scratch + 32;
    if (group < groups) {
#pragma unroll
      for (int e = 0; e < VN; ++e) red[(size_t)group * v_dim + piece * VN + e] = accv[e];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < v_dim; d += ATT_THREADS) {
      float a = 0.f;
      for (int g = 0; g < groups; ++g) a += red[(size_t)g * v_dim + d];
      if (prow) prow[2 + d] = a;
      else store_result<T>(out, out_wide, orow + d, a * inv);
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < MAX_D; ++r) {
    int d = threadIdx.x + r * ATT_THREADS;
    if (d < v_dim) {
      if (prow) prow[2 + d] = acc[r];
      else store_result<T>(out, out_wide, orow + d, acc[r] * inv);
    }
  }
}

// The same for R query heads of one key/value head at once (a block per token and group of R heads): every key
// and value row is read once for the R heads instead of once per head, which is what bounds the kernel above when
// many heads share few rows (one token per sequence, grouped or multi-query heads: the rows come from the L2 R
// times less often).  Rows of whole 16-byte pieces only (head_dim, v_dim, v_row multiples of the piece).
template <int R>
__device__ __forceinline__ void block_max_sum_r(float* v, float* scratch, bool is_max) {
  // v[R] per thread -> the block's maximum (or sum) of each, to every thread; scratch holds 32 * R floats
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int r = 0; r < R; ++r) v[r] = is_max ? warp_max(v[r]) : warp_sum(v[r]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) scratch[warp * R + r] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float a = is_max ? -INFINITY : 0.f;
    for (int w = 0; w < nwarp; ++w) a = is_max ? fmaxf(a, scratch[w * R + r]) : a + scratch[w * R + r];
    v[r] = a;
  }
}

template <typename T, int R>
__global__ void __launch_bounds__(ATT_THREADS)
attention_grouped_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride, int n_heads,
                         int n_kv_heads, int head_dim, int v_dim, float scale, int window, int keep_first, int chunk,
                         int v_row, const float* __restrict__ rel, int n_rel, const T* __restrict__ gate, int gate_stride,
                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ slots,
                         const int* __restrict__ page_table, int pt_stride, const T* __restrict__ k_cache,
                         const T* __restrict__ v_cache, float* __restrict__ part, int n_splits,
                         const float* __restrict__ sink, int v_share, int out_wide) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  float* qs = sm;                           // [R][head_dim]
  float* ps = qs + (size_t)R * head_dim;    // [R][ATT_CHUNK] probabilities
  float* scratch = ps + R * ATT_CHUNK;      // [32 * R]
  float* red = scratch + 32 * R;            // [R][groups * v_dim] at the end
  const int t = blockIdx.x, h0 = blockIdx.y * R;
  const int kvh = h0 / (n_heads / n_kv_heads);
  const int vh = kvh / v_share, n_v_heads = n_kv_heads / v_share;
  const int pos = tok_pos[t];
  const int* pt = page_table + (size_t)slots[tok_seq[t]] * pt_stride;
  const int lo = chunk > 0 ? (pos / chunk) * chunk : (window > 0 ? max(0, pos - window + 1) : 0);
  const int n_first = min(keep_first, lo);
  const int n_keys = n_first + pos - lo + 1;
  constexpr int VN = Vec16<T>::N;
  for (int i = threadIdx.x; i < R * head_dim; i += blockDim.x)
    qs[i] = to_f32<T>(q[(size_t)t * q_stride + (size_t)h0 * head_dim + i]);
  __syncthreads();
  const int per_row = v_dim / VN, groups = ATT_THREADS / per_row;
  const int piece = threadIdx.x % per_row, group = threadIdx.x / per_row;
  float accv[R][VN];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int e = 0; e < VN; ++e) accv[r][e] = 0.f;
  float m_run[R], l_run[R];
#pragma unroll
  for (int r = 0; r < R; ++r) { m_run[r] = -INFINITY; l_run[r] = 0.f; }

  for (int base = blockIdx.z * ATT_CHUNK; base < n_keys; base += ATT_CHUNK * n_splits) {
    const int n = min(ATT_CHUNK, n_keys - base);
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = -INFINITY;
    if ((int)threadIdx.x < n) {
      const int u = base + threadIdx.x;
      const int p = u < n_first ? u : lo + (u - n_first);
      const T* krow = k_cache + cache_row_offset(pt, p, n_kv_heads, kvh, head_dim);
      float dot[R];
#pragma unroll
      for (int r = 0; r < R; ++r) dot[r] = 0.f;
#pragma unroll 8
      for (int d = 0; d < head_dim; d += VN) {
        float kv[VN];
        Vec16<T>::load(krow + d, kv);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float4* q4 = reinterpret_cast<const float4*>(qs + r * head_dim + d);  // four numbers of q per read
#pragma unroll
          for (int e = 0; e < VN / 4; ++e) {
            const float4 a = q4[e];
            dot[r] = fmaf(a.x, kv[4 * e], dot[r]); dot[r] = fmaf(a.y, kv[4 * e + 1], dot[r]);
            dot[r] = fmaf(a.z, kv[4 * e + 2], dot[r]); dot[r] = fmaf(a.w, kv[4 * e + 3], dot[r]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        s[r] = dot[r] * scale;
        if (rel) s[r] += rel[(size_t)min(pos - p, n_rel - 1) * n_heads + h0 + r];
      }
    }
    float m_new[R], alpha[R], p_mine[R];
#pragma unroll
    for (int r = 0; r < R; ++r) m_new[r] = s[r];
    block_max_sum_r<R>(m_new, scratch, true);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      m_new[r] = fmaxf(m_run[r], m_new[r]);
      alpha[r] = (m_run[r] == -INFINITY) ? 0.f : expf(m_run[r] - m_new[r]);
      p_mine[r] = ((int)threadIdx.x < n) ? expf(s[r] - m_new[r]) : 0.f;
      ps[r * ATT_CHUNK + threadIdx.x] = p_mine[r];
    }
    block_max_sum_r<R>(p_mine, scratch, false);  // has the barriers that publish ps[]
#pragma unroll
    for (int r = 0; r < R; ++r) {
      l_run[r] = l_run[r] * alpha[r] + p_mine[r];
      m_run[r] = m_new[r];
#pragma unroll
      for (int e = 0; e < VN; ++e) accv[r][e] *= alpha[r];
    }
    if (group < groups) {
      // eight rows of values in flight at a time: a row alone leaves the thread waiting for its one load
      constexpr int VB = 8;
      for (int j0 = group; j0 < n; j0 += VB * groups) {
        float vv[VB][VN];
#pragma unroll
        for (int b = 0; b < VB; ++b) {
          const int j = j0 + b * groups;
          if (j < n) {
            const int u = base + j;
            const int p = u < n_first ? u : lo + (u - n_first);
            Vec16<T>::load(v_cache + cache_row_offset(pt, p, n_v_heads, vh, v_row) + piece * VN, vv[b]);
          }
        }
#pragma unroll
        for (int b = 0; b < VB; ++b) {
          const int j = j0 + b * groups;
          if (j < n) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const float w = ps[r * ATT_CHUNK + j];
#pragma unroll
              for (int e = 0; e < VN; ++e) accv[r][e] = fmaf(w, vv[b][e], accv[r][e]);
            }
          }
        }
      }
    }
    __syncthreads();  // ps[] is rewritten by the next chunk
  }
  // the groups' sums meet in shared memory: red[r][group][v_dim]
  if (group < groups) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int e = 0; e < VN; ++e) red[((size_t)r * groups + group) * v_dim + piece * VN + e] = accv[r][e];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int h = h0 + r;
    float inv = sink && !part ? sink_inverse(m_run[r], l_run[r], sink[h]) : 1.0f / l_run[r];
    if (gate) inv *= 1.0f / (1.0f + expf(-to_f32<T>(gate[(size_t)t * gate_stride + h])));
    const size_t orow = (size_t)t * out_stride + (size_t)h * v_dim;
    float* prow = part ? part + (((size_t)t * n_heads + h) * n_splits + blockIdx.z) * (v_dim + 2) : nullptr;
    if (prow && threadIdx.x == 0) { prow[0] = m_run[r]; prow[1] = l_run[r]; }
    for (int d = threadIdx.x; d < v_dim; d += ATT_THREADS) {
      float a = 0.f;
      for (int g = 0; g < groups; ++g) a += red[((size_t)r * groups + g) * v_dim + d];
      if (prow) prow[2 + d] = a;
      else store_result<T>(out, out_wide, orow + d, a * inv);
    }
  }
}

// out[t][h] = sum_z e^{m_z - M} acc_z / sum_z e^{m_z - M} l_z (times the logistic function of the gate), M = max_z m_z
template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part, int n_splits, int n_heads, int v_dim,
                                       const T* __restrict__ gate, int gate_stride, T* __restrict__ out, int out_stride,
                                       const float* __restrict__ sink, int out_wide) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* p = part + ((size_t)t * n_heads + h) * n_splits * (v_dim + 2);
  float M = -INFINITY;
  for (int z = 0; z < n_splits; ++z) M = fmaxf(M, p[(size_t)z * (v_dim + 2)]);
  float L = 0.f;
  for (int z = 0; z < n_splits; ++z) {
    float m = p[(size_t)z * (v_dim + 2)];
    if (m != -INFINITY) L += expf(m - M) * p[(size_t)z * (v_dim + 2) + 1];
  }
  float inv = sink ? sink_inverse(M, L, sink[h]) : 1.0f / L;
  if (gate) inv *= 1.0f / (1.0f + expf(-to_f32<T>(gate[(size_t)t * gate_stride + h])));
  for (int d = threadIdx.x; d < v_dim; d += blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < n_splits; ++z) {
      float m = p[(size_t)z * (v_dim + 2)];
      if (m != -INFINITY) a = fmaf(expf(m - M), p[(size_t)z * (v_dim + 2) + 2 + d], a);
    }
    store_result<T>(out, out_wide, (size_t)t * out_stride + (size_t)h * v_dim + d, a * inv);
  }
}

// q: [n_tokens, q_stride] with head h at element h*head_dim; out [n_tokens, out_stride] with head h at
// element h*v_dim.  The keys and values of the new tokens must already be in the cache.
extern "C" int bn_attention_general_ex(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                       int n_tokens, int n_heads, int n_kv_heads, int head_dim, int v_dim, float scale,
                                       int window, int keep_first, int chunk, int v_row, const float* rel, int n_rel,
                                       const void* gate, int gate_stride, const int* tok_seq, const int* tok_pos, const int* slots,
                                       const int* page_table, int pt_stride,
                                       const void* k_cache, const void* v_cache, float* part, int n_splits,
                                       const float* sink, int v_share, int out_wide, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (v_share < 1 || n_kv_heads % v_share || (v_share > 1 && v_row > 0)) return BN_ERR_BAD_ARG;
  if (n_splits < 1 || n_splits > 64 || (n_splits > 1 && !part)) return BN_ERR_BAD_ARG;
  if (n_splits == 1) part = nullptr;
  if (v_row <= 0) v_row = v_dim;
  // value rows of whole 16-byte pieces may be up to 128 pieces wide; others are one dimension per thread, eight times
  const int vn = dtype == BN_F32 ? 4 : 8;
  const bool wide = v_dim % vn == 0 && v_row % vn == 0 && v_dim / vn <= ATT_THREADS;
  if (head_dim <= 0 || head_dim > 2048 || n_kv_heads <= 0 || n_heads % n_kv_heads || window < 0 || keep_first < 0 ||
      chunk < 0 || (chunk > 0 && (window > 0 || keep_first > 0)) || v_dim <= 0 || v_row < v_dim ||
      (!wide && v_dim > 8 * ATT_THREADS) || (rel && n_rel <= 0))
    return BN_ERR_BAD_ARG;
  if (n_heads > 65535) return BN_ERR_BAD_ARG;
  // few tokens whose heads share rows: the heads of a key/value head four (or two) at a time, rows read once for them
  const int gq = n_heads / n_kv_heads;
  const int R = (gq % 4 == 0) ? 4 : ((gq % 2 == 0) ? 2 : 1);
  if (R > 1 && wide && head_dim % vn == 0 && n_tokens <= 256) {
    dim3 ggrid(n_tokens, n_heads / R, n_splits);
    const size_t gsmem = ((size_t)R * head_dim + R * ATT_CHUNK + 32 * R + (size_t)R * ATT_THREADS * vn) * sizeof(float);
#define BN_GROUPED(TT, RR)                                                                                                  \
  do {                                                                                                                      \
    if (gsmem > 48 * 1024) {                                                                                                \
      static size_t granted = 0;                                                                                            \
      if (gsmem > granted) {                                                                                                \
        cudaError_t e = cudaFuncSetAttribute(attention_grouped_kernel<TT, RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gsmem); \
        if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;                                                                \
        granted = gsmem;                                                                                                    \
      }                                                                                                                     \
    }                                                                                                                       \
    BN_LAUNCH((attention_grouped_kernel<TT, RR>), ggrid, ATT_THREADS, gsmem, stream, (const TT*)q, q_stride, (TT*)out,       \
              out_stride, n_heads, n_kv_heads, head_dim, v_dim, scale, window, keep_first, chunk, v_row, rel, n_rel,        \
              (const TT*)gate, gate_stride, tok_seq, tok_pos, slots, page_table, pt_stride, (const TT*)k_cache,              \
              (const TT*)v_cache, part, n_splits, sink, v_share, out_wide);                                                           \
  } while (0)
    if (gsmem <= 160 * 1024 && (dtype == BN_F32 || dtype == BN_BF16)) {
      if (dtype == BN_F32) { if (R == 4) BN_GROUPED(float, 4); else BN_GROUPED(float, 2); }
      else { if (R == 4) BN_GROUPED(__nv_bfloat16, 4); else BN_GROUPED(__nv_bfloat16, 2); }
#undef BN_GROUPED
      if (part) {
        dim3 mgrid(n_tokens, n_heads);
        if (dtype == BN_F32)
          BN_LAUNCH((attention_merge_kernel<float>), mgrid, 128, 0, stream, (const float*)part, n_splits, n_heads, v_dim,
                    (const float*)gate, gate_stride, (float*)out, out_stride, sink, out_wide);
        else
          BN_LAUNCH((attention_merge_kernel<__nv_bfloat16>), mgrid, 128, 0, stream, (const float*)part, n_splits, n_heads, v_dim,
                    (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_stride, sink, out_wide);
      }
      BN_CHECK_LAUNCH();
      return BN_OK;
    }
  }
  dim3 grid(n_tokens, n_heads, n_splits);
  size_t smem = (head_dim + ATT_CHUNK + 32 + ATT_THREADS * 8) * sizeof(float);  // q, scores, reduction scratch, the groups' sums
  if (dtype == BN_F32)
    BN_LAUNCH((attention_general_kernel<float>), grid, ATT_THREADS, smem, stream, 
        (const float*)q, q_stride, (float*)out, out_stride, n_heads, n_kv_heads, head_dim, v_dim, scale, window,
        keep_first, chunk, v_row, rel, n_rel, (const float*)gate, gate_stride,
        tok_seq, tok_pos, slots, page_table, pt_stride, (const float*)k_cache, (const float*)v_cache, part, n_splits, sink, v_share, out_wide);
  else if (dtype == BN_BF16)
    BN_LAUNCH((attention_general_kernel<__nv_bfloat16>), grid, ATT_THREADS, smem, stream, 
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, n_heads, n_kv_heads, head_dim, v_dim,
        scale, window, keep_first, chunk, v_row, rel, n_rel, (const __nv_bfloat16*)gate, gate_stride,
        tok_seq, tok_pos, slots, page_table, pt_stride,
        (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, part, n_splits, sink, v_share, out_wide);
  else
    return BN_ERR_BAD_ARG;
  if (part) {
    dim3 mgrid(n_tokens, n_heads);
    if (dtype == BN_F32)
      BN_LAUNCH((attention_merge_kernel<float>), mgrid, 128, 0, stream, (const float*)part, n_splits, n_heads, v_dim,
                (const float*)gate, gate_stride, (float*)out, out_stride, sink, out_wide);
    else
      BN_LAUNCH((attention_merge_kernel<__nv_bfloat16>), mgrid, 128, 0, stream, (const float*)part, n_splits, n_heads, v_dim,
                (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_stride, sink, out_wide);
  }
  BN_CHECK_LAUNCH();
  return BN_OK;
}

extern "C" int bn_attention_general(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                    int n_tokens, int n_heads, int n_kv_heads, int head_dim, float scale,
                                    int window, const int* tok_seq, const int* tok_pos, const int* slots,
                                    const int* page_table, int pt_stride,
                                    const void* k_cache, const void* v_cache, cudaStream_t stream) {
  return bn_attention_general_ex(q, q_stride, out, out_stride, dtype, n_tokens, n_heads, n_kv_heads, head_dim, head_dim,
                                 scale, window, 0, 0, 0, nullptr, 0, nullptr, 0, tok_seq, tok_pos, slots, page_table,
                                 pt_stride, k_cache, v_cache, nullptr, 1, nullptr, 1, 0, stream);
}
