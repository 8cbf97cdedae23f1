// Causal attention without a softmax over the paged cache, for any mix of new tokens (whole prompts,
// pieces of prompts, one token per sequence), in both element types.
//
//   a_g(i, j) = sigmoid(q_g(i) . k_c(j) * scale + rel[min(i - j, n_rel - 1)][g])      for 0 <= i - j < window
//   w_h(i, j) = sum_g mix[h][g] a_g(i, j)                                             (mix null: w = a)
//   out_h(i)  = gate_h(i) * sum_j w_h(i, j) v_c(h)(j)
//
// c(h) = h / (heads / kv_heads); rel holds the learned bias by distance with whatever is constant per head
// added in (float32; the scale does not multiply it); the gate is the logistic function of one number per
// head or per output number.  Scores, weights, the mixing and the value sums are float32.
//
// Nothing is normalised over the keys, so the heads of a token cannot be treated apart: the mixing needs
// every head's weight of a key.  One block takes a token and all its heads: a thread computes the scores of
// one key for every head (the key rows of all key/value heads), mixes them, and leaves the mixed weights in
// shared memory; then the value rows are summed in 16-byte pieces by groups of threads, the heads of a
// key/value head RB at a time so that a row is read once for them.  The keys of a token may be dealt out
// over several blocks (n_splits), whose partial sums a second kernel adds up.
#include "common.cuh"

#define SA_THREADS 128
#define SA_CHUNK 128

template <typename T>
struct Piece;
template <>
struct Piece<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* o) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <>
struct Piece<__nv_bfloat16> {
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

// N numbers of a row from element d0 on; beyond `len` zeros.  `vec`: the row is made of whole 16-byte pieces.
template <typename T>
__device__ __forceinline__ void load_piece(const T* row, int d0, int len, bool vec, float* o) {
  constexpr int N = Piece<T>::N;
  if (vec) {
    Piece<T>::load(row + d0, o);
  } else {
#pragma unroll
    for (int e = 0; e < N; ++e) o[e] = d0 + e < len ? to_f32<T>(row[d0 + e]) : 0.f;
  }
}

__device__ __forceinline__ float logistic(float z) { return 1.0f / (1.0f + expf(-z)); }

// gate_mode: 0 none, 1 one number per head (gate[t][h]), 2 one per output number (gate[t][h * v_dim + d])
template <typename T>
__device__ __forceinline__ float gate_of(const T* gate, int gate_stride, int gate_mode, int t, int h, int idx) {
  if (gate_mode == 0) return 1.0f;
  return logistic(to_f32<T>(gate[(size_t)t * gate_stride + (gate_mode == 1 ? h : idx)]));
}

template <typename T, int RB>
__global__ void __launch_bounds__(SA_THREADS)
sigmoid_attention_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride, int n_heads, int n_kv_heads,
                         int head_dim, int v_dim, float scale, int window, const float* __restrict__ rel, int n_rel,
                         const float* __restrict__ mix, const T* __restrict__ gate, int gate_stride, int gate_mode,
                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ slots,
                         const int* __restrict__ page_table, int pt_stride, const T* __restrict__ k_cache,
                         const T* __restrict__ v_cache, float* __restrict__ part, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int VN = Piece<T>::N;
  extern __shared__ __align__(16) float sm[];
  const int H = n_heads, R = n_heads / n_kv_heads;
  const int per_row = (v_dim + VN - 1) / VN, groups = SA_THREADS / per_row, v_pad = per_row * VN;
  float* qs = sm;                                   // [H][head_dim]
  float* araw = qs + (size_t)H * head_dim;          // [H][SA_CHUNK] weights before the mixing
  float* ps = mix ? araw + H * SA_CHUNK : araw;     // [H][SA_CHUNK] weights after it
  float* mixs = ps + H * SA_CHUNK;                  // [H][H]
  float* outs = mixs + (mix ? H * H : 0);           // [H][v_dim]
  float* red = outs + (size_t)H * v_dim;            // [RB][groups][v_pad]
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = tok_pos[t];
  const int* pt = page_table + (size_t)slots[tok_seq[t]] * pt_stride;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int n_keys = pos - lo + 1;
  const bool k_vec = head_dim % VN == 0, v_vec = v_dim % VN == 0;
  for (int i = tid; i < H * head_dim; i += SA_THREADS) qs[i] = to_f32<T>(q[(size_t)t * q_stride + i]);
  if (mix)
    for (int i = tid; i < H * H; i += SA_THREADS) mixs[i] = mix[i];
  for (int i = tid; i < H * v_dim; i += SA_THREADS) outs[i] = 0.f;
  __syncthreads();
  const int piece = tid % per_row, group = tid / per_row;

  for (int base = blockIdx.y * SA_CHUNK; base < n_keys; base += SA_CHUNK * n_splits) {
    const int n = min(SA_CHUNK, n_keys - base);
    if (tid < n) {
      const int p = lo + base + tid;
      const float* bias = rel ? rel + (size_t)min(pos - p, n_rel - 1) * H : nullptr;
      for (int c = 0; c < n_kv_heads; ++c) {
        const T* krow = k_cache + cache_row_offset(pt, p, n_kv_heads, c, head_dim);
        for (int r0 = 0; r0 < R; r0 += RB) {
          float dot[RB];
#pragma unroll
          for (int r = 0; r < RB; ++r) dot[r] = 0.f;
          const float* q0 = qs + (size_t)(c * R + r0) * head_dim;
          for (int d = 0; d < head_dim; d += VN) {
            float kv[VN];
            load_piece<T>(krow, d, head_dim, k_vec, kv);
#pragma unroll
            for (int r = 0; r < RB; ++r) {
#pragma unroll
              for (int e = 0; e < VN; ++e)
                if (k_vec || d + e < head_dim) dot[r] = fmaf(q0[r * head_dim + d + e], kv[e], dot[r]);
            }
          }
#pragma unroll
          for (int r = 0; r < RB; ++r) {
            const int h = c * R + r0 + r;
            araw[h * SA_CHUNK + tid] = logistic(dot[r] * scale + (bias ? bias[h] : 0.f));
          }
        }
      }
      // the mixing reads what this thread wrote itself: its key's weights of all heads
      if (mix) {
        for (int h = 0; h < H; ++h) {
          float w = 0.f;
          for (int g = 0; g < H; ++g) w = fmaf(mixs[h * H + g], araw[g * SA_CHUNK + tid], w);
          ps[h * SA_CHUNK + tid] = w;
        }
      }
    }
    __syncthreads();
    // ---- values: the heads of key/value head c, RB at a time
    for (int c = 0; c < n_kv_heads; ++c) {
      for (int r0 = 0; r0 < R; r0 += RB) {
        float accv[RB][VN];
#pragma unroll
        for (int r = 0; r < RB; ++r)
#pragma unroll
          for (int e = 0; e < VN; ++e) accv[r][e] = 0.f;
        if (group < groups) {
          constexpr int VB = 4;  // rows of values in flight per thread
          for (int j0 = group; j0 < n; j0 += VB * groups) {
            float vv[VB][VN];
#pragma unroll
            for (int b = 0; b < VB; ++b) {
              const int j = j0 + b * groups;
              if (j < n)
                load_piece<T>(v_cache + cache_row_offset(pt, lo + base + j, n_kv_heads, c, v_dim), piece * VN, v_dim, v_vec, vv[b]);
            }
#pragma unroll
            for (int b = 0; b < VB; ++b) {
              const int j = j0 + b * groups;
              if (j < n) {
#pragma unroll
                for (int r = 0; r < RB; ++r) {
                  const float w = ps[(c * R + r0 + r) * SA_CHUNK + j];
#pragma unroll
                  for (int e = 0; e < VN; ++e) accv[r][e] = fmaf(w, vv[b][e], accv[r][e]);
                }
              }
            }
          }
#pragma unroll
          for (int r = 0; r < RB; ++r)
#pragma unroll
            for (int e = 0; e < VN; ++e) red[((size_t)r * groups + group) * v_pad + piece * VN + e] = accv[r][e];
        }
        __syncthreads();
        for (int i = tid; i < RB * v_dim; i += SA_THREADS) {
          const int r = i / v_dim, d = i - r * v_dim;
          float a = 0.f;
          for (int g = 0; g < groups; ++g) a += red[((size_t)r * groups + g) * v_pad + d];
          outs[(size_t)(c * R + r0 + r) * v_dim + d] += a;
        }
        __syncthreads();
      }
    }
  }
  if (part) {
    float* prow = part + ((size_t)t * n_splits + blockIdx.y) * H * v_dim;
    for (int i = tid; i < H * v_dim; i += SA_THREADS) prow[i] = outs[i];
  } else {
    for (int i = tid; i < H * v_dim; i += SA_THREADS)
      out[(size_t)t * out_stride + i] = from_f32<T>(outs[i] * gate_of<T>(gate, gate_stride, gate_mode, t, i / v_dim, i));
  }
}

// out[t][i] = gate * sum_z part[t][z][i]
template <typename T>
__global__ void sigmoid_attention_merge_kernel(const float* __restrict__ part, int n_splits, int row, int v_dim,
                                               const T* __restrict__ gate, int gate_stride, int gate_mode, T* __restrict__ out,
                                               int out_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < row; i += blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < n_splits; ++z) a += part[((size_t)t * n_splits + z) * row + i];
    out[(size_t)t * out_stride + i] = from_f32<T>(a * gate_of<T>(gate, gate_stride, gate_mode, t, i / v_dim, i));
  }
}

static size_t sa_smem_floats(int H, int head_dim, int v_dim, int rb, int vn, bool mixed) {
  const int per_row = (v_dim + vn - 1) / vn, groups = SA_THREADS / per_row;
  return (size_t)H * head_dim + (size_t)(mixed ? 2 : 1) * H * SA_CHUNK + (mixed ? (size_t)H * H : 0) + (size_t)H * v_dim +
         (size_t)rb * groups * per_row * vn;
}

template <typename T, int RB>
static int sa_launch(const void* q, int q_stride, void* out, int out_stride, int n_tokens, int n_heads, int n_kv_heads,
                     int head_dim, int v_dim, float scale, int window, const float* rel, int n_rel, const float* mix,
                     const void* gate, int gate_stride, int gate_mode, const int* tok_seq, const int* tok_pos, const int* slots,
                     const int* page_table, int pt_stride, const void* k_cache, const void* v_cache, float* part, int n_splits,
                     cudaStream_t stream) {
  const size_t smem = sa_smem_floats(n_heads, head_dim, v_dim, RB, Piece<T>::N, mix != nullptr) * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;
  if (smem > 48 * 1024) {
    static size_t granted = 0;
    if (smem > granted) {
      cudaError_t e = cudaFuncSetAttribute(sigmoid_attention_kernel<T, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted = smem;
    }
  }
  dim3 grid(n_tokens, n_splits);
  BN_LAUNCH((sigmoid_attention_kernel<T, RB>), grid, SA_THREADS, smem, stream, (const T*)q, q_stride, (T*)out, out_stride, n_heads,
            n_kv_heads, head_dim, v_dim, scale, window, rel, n_rel, mix, (const T*)gate, gate_stride, gate_mode, tok_seq, tok_pos,
            slots, page_table, pt_stride, (const T*)k_cache, (const T*)v_cache, part, n_splits);
  if (part)
    BN_LAUNCH((sigmoid_attention_merge_kernel<T>), n_tokens, 256, 0, stream, (const float*)part, n_splits, n_heads * v_dim, v_dim,
              (const T*)gate, gate_stride, gate_mode, (T*)out, out_stride);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// Bytes of shared memory a launch takes (the caller may refuse sizes that do not fit before it launches).
extern "C" int bn_sigmoid_attention_smem(int dtype, int n_heads, int n_kv_heads, int head_dim, int v_dim, int mixed) {
  const int R = n_heads / n_kv_heads, rb = R % 4 == 0 ? 4 : (R % 2 == 0 ? 2 : 1);
  return (int)(sa_smem_floats(n_heads, head_dim, v_dim, rb, dtype == BN_F32 ? 4 : 8, mixed != 0) * sizeof(float));
}

// q: [n_tokens, q_stride] with head h at element h * head_dim; out [n_tokens, out_stride] with head h at element
// h * v_dim.  The keys and values of the new tokens must already be in the cache.  part: float32
// [n_tokens, n_splits, n_heads * v_dim] when n_splits > 1.
extern "C" int bn_sigmoid_attention(const void* q, int q_stride, void* out, int out_stride, int dtype, int n_tokens, int n_heads,
                                    int n_kv_heads, int head_dim, int v_dim, float scale, int window, const float* rel, int n_rel,
                                    const float* mix, const void* gate, int gate_stride, int gate_mode, const int* tok_seq,
                                    const int* tok_pos, const int* slots, const int* page_table, int pt_stride,
                                    const void* k_cache, const void* v_cache, float* part, int n_splits, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && !part)) return BN_ERR_BAD_ARG;
  if (n_splits == 1) part = nullptr;
  const int vn = dtype == BN_F32 ? 4 : 8;
  if (!q || !out || !k_cache || !v_cache || head_dim <= 0 || v_dim <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || window < 0 ||
      (v_dim + vn - 1) / vn > SA_THREADS || (rel && n_rel <= 0) || gate_mode < 0 || gate_mode > 2 || (gate_mode && !gate))
    return BN_ERR_BAD_ARG;
  const int R = n_heads / n_kv_heads;
#define BN_SA_ARGS q, q_stride, out, out_stride, n_tokens, n_heads, n_kv_heads, head_dim, v_dim, scale, window, rel, n_rel, mix, gate, \
                   gate_stride, gate_mode, tok_seq, tok_pos, slots, page_table, pt_stride, k_cache, v_cache, part, n_splits, stream
  if (dtype == BN_F32) {
    if (R % 4 == 0) return sa_launch<float, 4>(BN_SA_ARGS);
    if (R % 2 == 0) return sa_launch<float, 2>(BN_SA_ARGS);
    return sa_launch<float, 1>(BN_SA_ARGS);
  }
  if (dtype == BN_BF16) {
    if (R % 4 == 0) return sa_launch<__nv_bfloat16, 4>(BN_SA_ARGS);
    if (R % 2 == 0) return sa_launch<__nv_bfloat16, 2>(BN_SA_ARGS);
    return sa_launch<__nv_bfloat16, 1>(BN_SA_ARGS);
  }
#undef BN_SA_ARGS
  return BN_ERR_BAD_ARG;
}
