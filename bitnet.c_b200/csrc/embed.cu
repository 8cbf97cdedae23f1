// Token embedding: ids -> rows of the table, written as the float32 residual stream.
// Reference: bn_model_embed_token bounds-checks the id, zero-fills and logs on a bad
// one, and converts the row to float32 (src/model_embed.c:6-28).
#include "common.cuh"

template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                    float* __restrict__ out, int width, int vocab, float scale,
                                    int* __restrict__ bad_token) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  int t = blockIdx.x;
  int id = tokens[t];
  float* o = out + (size_t)t * width;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicExch(bad_token, 1);
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_f32<T>(row[i]) * scale;
}

// bad_token: one int on the device, set to 1 when an id lies outside [0, vocab).
extern "C" int bn_embed_gather(const void* table, int table_dtype, const int* tokens, float* out,
                               int n_tokens, int width, int vocab, float scale, int* bad_token,
                               cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (width <= 0 || vocab <= 0) return BN_ERR_BAD_ARG;
  int threads = width >= 1024 ? 256 : 128;
  if (table_dtype == BN_F32)
    BN_LAUNCH((embed_gather_kernel<float>), n_tokens, threads, 0, stream, (const float*)table, tokens, out, width, vocab, scale, bad_token);
  else if (table_dtype == BN_BF16)
    BN_LAUNCH((embed_gather_kernel<__nv_bfloat16>), n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, tokens, out, width, vocab, scale, bad_token);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// The same with the rows normed before anybody reads them: out[t] = v / sqrt(mean(v^2) + eps) * w with
// v = table[tokens[t]] * scale (the float32 stream starts as the normed embedding), and in the same pass the norm
// of the first reader, h[t] = out[t] / sqrt(mean(out[t]^2) + eps1) * w1, in the compute type (w1 null: none).
// One block per token; the row waits in shared memory between the passes.  A bad id gives rows of zeros.
template <typename T>
__global__ void embed_gather_normed_kernel(const T* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ out,
                                           int width, int vocab, float scale, const void* __restrict__ w, int w_dtype, float eps,
                                           const void* __restrict__ w1, int w1_dtype, float eps1, void* __restrict__ h, int h_dtype,
                                           int* __restrict__ bad_token) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float emb_row[];  // width floats, then 32 for the reductions
  float* scratch = emb_row + width;
  const int t = blockIdx.x;
  const int id = tokens[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicExch(bad_token, 1);
  const T* row = table + (size_t)(bad ? 0 : id) * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float a = bad ? 0.f : to_f32<T>(row[i]) * scale;
    emb_row[i] = a;
    ss += a * a;
  }
  ss = block_sum(ss, scratch);
  const float s0 = 1.0f / sqrtf(ss / (float)width + eps);
  float* o = out + (size_t)t * width;
  float s2 = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float a = emb_row[i] * s0 * load_as_f32(w, w_dtype, i);
    o[i] = a;
    emb_row[i] = a;
    s2 += a * a;
  }
  if (!w1) return;
  s2 = block_sum(s2, scratch);
  const float s1 = 1.0f / sqrtf(s2 / (float)width + eps1);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    store_from_f32(h, h_dtype, (size_t)t * width + i, emb_row[i] * s1 * load_as_f32(w1, w1_dtype, i));
}

extern "C" int bn_embed_gather_normed(const void* table, int table_dtype, const int* tokens, float* out, int n_tokens, int width,
                                      int vocab, float scale, const void* w, int w_dtype, float eps, const void* w1, int w1_dtype,
                                      float eps1, void* h, int h_dtype, int* bad_token, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (width <= 0 || vocab <= 0 || !w || !(eps > 0.f) || (w1 && (!h || !(eps1 > 0.f)))) return BN_ERR_BAD_ARG;
  const size_t smem = ((size_t)width + 32) * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;
  const int threads = width >= 1024 ? 256 : 128;
#define BN_EMB_NORMED(TT)                                                                                                       \
  do {                                                                                                                          \
    if (smem > 48 * 1024) {                                                                                                     \
      static size_t granted = 0;                                                                                                \
      if (smem > granted) {                                                                                                     \
        cudaError_t e = cudaFuncSetAttribute(embed_gather_normed_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;                                                                    \
        granted = smem;                                                                                                         \
      }                                                                                                                         \
    }                                                                                                                           \
    BN_LAUNCH((embed_gather_normed_kernel<TT>), n_tokens, threads, smem, stream, (const TT*)table, tokens, out, width, vocab,    \
              scale, w, w_dtype, eps, w1, w1_dtype, eps1, h, h_dtype, bad_token);                                               \
  } while (0)
  if (table_dtype == BN_F32) BN_EMB_NORMED(float);
  else if (table_dtype == BN_BF16) BN_EMB_NORMED(__nv_bfloat16);
  else return BN_ERR_BAD_ARG;
#undef BN_EMB_NORMED
  BN_CHECK_LAUNCH();
  return BN_OK;
}
