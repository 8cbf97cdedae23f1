// SwiGLU over rows of width 2 I that hold, alternating, 8 gate values and the 8 up values of the
// same indices: out[t, i] = silu(h[t, 16 (i / 8) + i % 8]) * h[t, 16 (i / 8) + 8 + i % 8].
// (The stacked gate/up weight is laid out that way so that the small-batch product can apply
// the activation in its epilogue, linear_tc.cu.)  One thread takes a block of 8: it reads the 8
// gate and 8 up values as whole 16- or 32-byte pieces and writes 8 results.
// Reference: silu(z) = z / (1 + exp(-z)) with exact expf on the reference-activation
// path (src/transformer/cpu_backend.c:365-392, src/transformer/prefill_backend.c:25-49).
#include "common.cuh"

__device__ __forceinline__ float glu_mul_one(float g, float u, int act) { return glu_activation(g, act) * u; }

__global__ void silu_mul_bf16_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ out,
                                     int blocks_per_row, size_t total_blocks, int act) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_blocks) return;
  size_t t = idx / blocks_per_row;
  size_t j = idx - t * blocks_per_row;
  const uint4* src = reinterpret_cast<const uint4*>(h + (t * blocks_per_row + j) * 16);
  uint4 gr = src[0], ur = src[1];
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gr);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&ur);
  uint4 res;
  __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
    r2[i] = __floats2bfloat162_rn(glu_mul_one(g.x, u.x, act), glu_mul_one(g.y, u.y, act));
  }
  *reinterpret_cast<uint4*>(out + (t * blocks_per_row + j) * 8) = res;
}

__global__ void silu_mul_f32_kernel(const float* __restrict__ h, float* __restrict__ out, int blocks_per_row,
                                    size_t total_blocks, int act) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_blocks) return;
  size_t t = idx / blocks_per_row;
  size_t j = idx - t * blocks_per_row;
  const float4* src = reinterpret_cast<const float4*>(h + (t * blocks_per_row + j) * 16);
  float4 g0 = src[0], g1 = src[1], u0 = src[2], u1 = src[3];
  float4* dst = reinterpret_cast<float4*>(out + (t * blocks_per_row + j) * 8);
  dst[0] = make_float4(glu_mul_one(g0.x, u0.x, act), glu_mul_one(g0.y, u0.y, act), glu_mul_one(g0.z, u0.z, act), glu_mul_one(g0.w, u0.w, act));
  dst[1] = make_float4(glu_mul_one(g1.x, u1.x, act), glu_mul_one(g1.y, u1.y, act), glu_mul_one(g1.z, u1.z, act), glu_mul_one(g1.w, u1.w, act));
}

// h: [n_rows, 2 * inter], out: [n_rows, inter]; inter a multiple of 8, both 16-byte aligned.
// act: the gate's activation (BN_ACT_SILU, BN_ACT_GELU_TANH)
extern "C" int bn_glu_mul(const void* h, void* out, int dtype, int n_rows, int inter, int act, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (act != BN_ACT_SILU && act != BN_ACT_GELU_TANH) return BN_ERR_BAD_ARG;
  if (inter <= 0 || inter % 8 || (((uintptr_t)h | (uintptr_t)out) & 15)) return BN_ERR_BAD_ARG;
  int bpr = inter / 8;
  size_t total = (size_t)n_rows * bpr;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == BN_F32)
    BN_LAUNCH(silu_mul_f32_kernel, blocks, 256, 0, stream, (const float*)h, (float*)out, bpr, total, act);
  else if (dtype == BN_BF16)
    BN_LAUNCH(silu_mul_bf16_kernel, blocks, 256, 0, stream, (const __nv_bfloat16*)h, (__nv_bfloat16*)out, bpr, total, act);
  else
    return BN_ERR_BAD_ARG;
  return BN_OK;
}

extern "C" int bn_silu_mul(const void* h, void* out, int dtype, int n_rows, int inter, cudaStream_t stream) {
  return bn_glu_mul(h, out, dtype, n_rows, inter, BN_ACT_SILU, stream);
}

// x = x * scale, then (cap != 0) x = tanhf(x / cap) * cap: an output head's logit scale and the
// reference's final soft-cap (src/transformer/logits.c:325-333), float32 in place.
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t n, float scale, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = x[i] * scale;
  if (cap != 0.0f) v = tanhf(v * (1.0f / cap)) * cap;
  x[i] = v;
}

extern "C" int bn_scale_softcap(float* x, long long n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return BN_OK;
  if (!x) return BN_ERR_BAD_ARG;
  unsigned blocks = (unsigned)(((size_t)n + 255) / 256);
  BN_LAUNCH(scale_softcap_kernel, blocks, 256, 0, stream, x, (size_t)n, scale, cap);
  return BN_OK;
}

// Clamped gated unit: rows of h hold `inter` gate values and then `inter` up values;
// g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(slope * g) * (u + 1).
__device__ __forceinline__ float glu_limited_one(float g, float u, float limit, float slope) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-slope * g)) * (u + 1.0f);
}

template <typename T>
__global__ void glu_limited_kernel(const T* __restrict__ h, T* __restrict__ out, int inter, size_t total, float limit,
                                   float slope) {
  pdl_launch_dependents();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  size_t t = idx / inter;
  size_t j = idx - t * inter;
  out[idx] = from_f32<T>(glu_limited_one(to_f32<T>(h[t * 2 * inter + j]), to_f32<T>(h[t * 2 * inter + inter + j]), limit, slope));
}

// inter a multiple of 8, both buffers 16-byte aligned: a thread takes 8 gate and 8 up values in 16-byte pieces
__global__ void glu_limited_bf16x8_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ out, int inter,
                                          size_t total8, float limit, float slope) {
  pdl_launch_dependents();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int per_row = inter / 8;
  size_t t = idx / per_row;
  size_t j = (idx - t * per_row) * 8;
  uint4 gr = *reinterpret_cast<const uint4*>(h + t * 2 * inter + j), ur = *reinterpret_cast<const uint4*>(h + t * 2 * inter + inter + j);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gr);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&ur);
  uint4 res;
  __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
    r2[i] = __floats2bfloat162_rn(glu_limited_one(g.x, u.x, limit, slope), glu_limited_one(g.y, u.y, limit, slope));
  }
  *reinterpret_cast<uint4*>(out + t * inter + j) = res;
}

extern "C" int bn_glu_limited(const void* h, void* out, int dtype, int n_rows, int inter, float limit, float slope,
                              cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (inter <= 0 || !h || !out) return BN_ERR_BAD_ARG;
  size_t total = (size_t)n_rows * inter;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == BN_F32)
    BN_LAUNCH(glu_limited_kernel<float>, blocks, 256, 0, stream, (const float*)h, (float*)out, inter, total, limit, slope);
  else if (dtype == BN_BF16 && inter % 8 == 0 && ((((uintptr_t)h) | ((uintptr_t)out)) & 15) == 0)
    BN_LAUNCH(glu_limited_bf16x8_kernel, (unsigned)((total / 8 + 255) / 256), 256, 0, stream, (const __nv_bfloat16*)h,
              (__nv_bfloat16*)out, inter, total / 8, limit, slope);
  else if (dtype == BN_BF16)
    BN_LAUNCH(glu_limited_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)h, (__nv_bfloat16*)out,
              inter, total, limit, slope);
  else
    return BN_ERR_BAD_ARG;
  return BN_OK;
}

// The plain gated unit on rows that hold `inter` gate values and then `inter` up values: out = act(gate) * up.
template <typename T>
__global__ void glu_halves_kernel(const T* __restrict__ h, T* __restrict__ out, int inter, size_t total, int act) {
  pdl_launch_dependents();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  size_t t = idx / inter;
  size_t j = idx - t * inter;
  out[idx] = from_f32<T>(glu_activation(to_f32<T>(h[t * 2 * inter + j]), act) * to_f32<T>(h[t * 2 * inter + inter + j]));
}

// inter a multiple of 8, both buffers 16-byte aligned: a thread takes 8 gate and 8 up values in 16-byte pieces
__global__ void glu_halves_bf16x8_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ out, int inter,
                                         size_t total8, int act) {
  pdl_launch_dependents();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int per_row = inter / 8;
  size_t t = idx / per_row;
  size_t j = (idx - t * per_row) * 8;
  uint4 gr = *reinterpret_cast<const uint4*>(h + t * 2 * inter + j), ur = *reinterpret_cast<const uint4*>(h + t * 2 * inter + inter + j);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gr);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&ur);
  uint4 res;
  __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
    r2[i] = __floats2bfloat162_rn(glu_activation(g.x, act) * u.x, glu_activation(g.y, act) * u.y);
  }
  *reinterpret_cast<uint4*>(out + t * inter + j) = res;
}

extern "C" int bn_glu_halves(const void* h, void* out, int dtype, int n_rows, int inter, int act, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (inter <= 0 || !h || !out || (act != BN_ACT_SILU && act != BN_ACT_GELU_TANH)) return BN_ERR_BAD_ARG;
  size_t total = (size_t)n_rows * inter;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == BN_F32)
    BN_LAUNCH(glu_halves_kernel<float>, blocks, 256, 0, stream, (const float*)h, (float*)out, inter, total, act);
  else if (dtype == BN_BF16 && inter % 8 == 0 && ((((uintptr_t)h) | ((uintptr_t)out)) & 15) == 0)
    BN_LAUNCH(glu_halves_bf16x8_kernel, (unsigned)((total / 8 + 255) / 256), 256, 0, stream, (const __nv_bfloat16*)h,
              (__nv_bfloat16*)out, inter, total / 8, act);
  else if (dtype == BN_BF16)
    BN_LAUNCH(glu_halves_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)h, (__nv_bfloat16*)out, inter, total, act);
  else
    return BN_ERR_BAD_ARG;
  return BN_OK;
}

// A gated row of a second embedding: out[t, j] = act(pre[t, j]) * table[tokens[t], col0 + j], j < dim.
// pre [n, pre_stride] and out [n, dim] of type `dtype`; the table [vocab, table_stride] of type
// `table_dtype`; an id outside the table gives zeros.
__global__ void gated_lookup_kernel(const void* __restrict__ pre, int pre_stride, int dtype, const void* __restrict__ table,
                                    int table_dtype, int table_stride, int col0, int vocab, const int* __restrict__ tokens,
                                    void* __restrict__ out, int dim, size_t total, int act) {
  pdl_launch_dependents();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  size_t t = idx / dim;
  int j = (int)(idx - t * dim);
  int tok = tokens[t];
  float e = (tok >= 0 && tok < vocab) ? load_as_f32(table, table_dtype, (size_t)tok * table_stride + col0 + j) : 0.f;
  store_from_f32(out, dtype, idx, glu_activation(load_as_f32(pre, dtype, t * pre_stride + j), act) * e);
}

extern "C" int bn_gated_lookup(const void* pre, int pre_stride, int dtype, const void* table, int table_dtype,
                               int table_stride, int col0, int vocab, const int* tokens, void* out, int n, int dim, int act,
                               cudaStream_t stream) {
  if (n <= 0) return BN_OK;
  if (dim <= 0 || col0 < 0 || col0 + dim > table_stride || pre_stride < dim || !pre || !table || !tokens || !out ||
      (dtype != BN_F32 && dtype != BN_BF16) || (table_dtype != BN_F32 && table_dtype != BN_BF16) ||
      (act != BN_ACT_SILU && act != BN_ACT_GELU_TANH))
    return BN_ERR_BAD_ARG;
  size_t total = (size_t)n * dim;
  BN_LAUNCH(gated_lookup_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, pre, pre_stride, dtype, table, table_dtype,
            table_stride, col0, vocab, tokens, out, dim, total, act);
  return BN_OK;
}

// x[t, i] <- x[t, i] * sigmoid(g[t, i]) for i < n, in place: an output gate on every number of a row.  x and g are
// views into rows of `dtype` with strides of their own; the logistic function is taken in float32.
template <typename T>
__global__ void gate_rows_kernel(T* __restrict__ x, int x_stride, const T* __restrict__ g, int g_stride, int n, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / n, c = i - t * n;
    const float z = to_f32<T>(g[t * g_stride + c]);
    x[t * x_stride + c] = from_f32<T>(to_f32<T>(x[t * x_stride + c]) / (1.0f + expf(-z)));
  }
}

extern "C" int bn_gate_rows(void* x, int x_stride, const void* g, int g_stride, int dtype, int n_rows, int n, cudaStream_t stream) {
  if (n_rows <= 0 || n <= 0) return BN_OK;
  if (!x || !g || x_stride < n || g_stride < n) return BN_ERR_BAD_ARG;
  const size_t total = (size_t)n_rows * n;
  const unsigned blocks = (unsigned)min((size_t)4096, (total + 255) / 256);
  if (dtype == BN_F32)
    BN_LAUNCH(gate_rows_kernel<float>, blocks, 256, 0, stream, (float*)x, x_stride, (const float*)g, g_stride, n, total);
  else if (dtype == BN_BF16)
    BN_LAUNCH(gate_rows_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)g,
              g_stride, n, total);
  else
    return BN_ERR_BAD_ARG;
  return BN_OK;
}
