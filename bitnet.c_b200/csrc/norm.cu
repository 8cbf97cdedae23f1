// Residual add fused with RMSNorm.
//
//   v = x[row] (+ delta[row]);  x[row] = v (when write_x);  out[r] = v * rsqrt(mean(v^2) + eps) * w
//
// x is the float32 residual stream; delta is the output of the part that ran
// before (any element type), possibly as n_parts partial sums [n_parts, rows, width] left by
// a product that split its inner dimension (linear_mma.cu); they are added in order of the
// part index.  The sum and the statistics are float32.  With a
// row index the kernel reads only the listed rows and writes them densely: this
// serves the final norm, which is needed at the wanted positions only.
// Reference: eps is added to the mean inside the root, out = x * scale * w
// (src/transformer/rmsnorm_scalar.c:4-13); the residual add fused in front is the
// reference's residual_rmsnorm kernel (src/gpu_cuda.cu:5077).
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

// Few rows (decode): one row per block would leave most SMs idle and each block with a long
// chain of loads, so a row is spread over a thread-block cluster of NORM_CLUSTER blocks.  Each
// block holds its columns in registers, the sums of squares meet through distributed shared
// memory, and every block adds them in rank order, so all see the same scale.
#define NORM_CLUSTER 8
#define NORM_CL_THREADS 128
#define NORM_CL_VEC 4  // float4 groups per thread: up to 128 * 4 * 4 = 2048 columns per block

__device__ __forceinline__ float4 load4_as_f32(const void* p, int dtype, size_t i) {
  if (dtype == BN_F32) return *reinterpret_cast<const float4*>((const float*)p + i);
  uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p + i);
  float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4_from_f32(void* p, int dtype, size_t i, float4 v) {
  if (dtype == BN_F32) {
    *reinterpret_cast<float4*>((float*)p + i) = v;
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>((__nv_bfloat16*)p + i) = raw;
  }
}

__global__ void __cluster_dims__(1, NORM_CLUSTER, 1) __launch_bounds__(NORM_CL_THREADS)
add_rmsnorm_cluster_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype, int n_parts,
                           size_t part_stride, const void* __restrict__ w, int w_dtype, void* __restrict__ out,
                           int out_dtype, const int* __restrict__ rows, int width, int cols_per_block, float eps,
                           int write_x) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  __shared__ float scratch[32];
  __shared__ float block_ss;
  cg::cluster_group cluster = cg::this_cluster();
  const int r = blockIdx.x, rank = blockIdx.y;  // the cluster spans gridDim.y == NORM_CLUSTER
  const size_t row = rows ? (size_t)rows[r] : (size_t)r;
  const int c0 = rank * cols_per_block, c1 = min(width, c0 + cols_per_block);
  float4 v[NORM_CL_VEC];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < NORM_CL_VEC; ++u) {
    int c = c0 + (u * NORM_CL_THREADS + threadIdx.x) * 4;
    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < c1) {
      float4 a = *reinterpret_cast<const float4*>(x + row * width + c);
      if (delta) {
        for (int p = 0; p < n_parts; ++p) {
          float4 d = load4_as_f32(delta, delta_dtype, p * part_stride + row * width + c);
          a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        }
      }
      v[u] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) block_ss = ss;
  cluster.sync();
  float total = 0.f;
  for (int k = 0; k < NORM_CLUSTER; ++k) total += *cluster.map_shared_rank(&block_ss, k);
  float scale = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
  for (int u = 0; u < NORM_CL_VEC; ++u) {
    int c = c0 + (u * NORM_CL_THREADS + threadIdx.x) * 4;
    if (c < c1) {
      float4 a = v[u];
      if (write_x) *reinterpret_cast<float4*>(x + row * width + c) = a;
      float4 g = load4_as_f32(w, w_dtype, c);
      store4_from_f32(out, out_dtype, (size_t)r * width + c,
                      make_float4(a.x * scale * g.x, a.y * scale * g.y, a.z * scale * g.z, a.w * scale * g.w));
    }
  }
  cluster.sync();  // no block may leave while another still reads its sum
}

__global__ void add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype,
                                   int n_parts, size_t part_stride, const void* __restrict__ w, int w_dtype, void* __restrict__ out,
                                   int out_dtype, const int* __restrict__ rows, int width, float eps,
                                   int write_x, int vec4) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  extern __shared__ __align__(16) float v[];  // width floats, then 32 for the reduction
  float* scratch = v + width;
  int r = blockIdx.x;
  size_t row = rows ? (size_t)rows[r] : (size_t)r;
  float* xr = x + row * width;
  float ss = 0.f;
  if (vec4) {
    // groups of four columns, whole 8- or 16-byte pieces (the launcher checked the alignment)
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(xr + i);
      if (delta) {
        for (int p = 0; p < n_parts; ++p) {
          float4 d = load4_as_f32(delta, delta_dtype, p * part_stride + row * width + i);
          a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        }
      }
      *reinterpret_cast<float4*>(v + i) = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float a = xr[i];
      if (delta) {
        for (int p = 0; p < n_parts; ++p) a += load_as_f32(delta, delta_dtype, p * part_stride + row * width + i);
      }
      v[i] = a;
      ss += a * a;
    }
  }
  ss = block_sum(ss, scratch);
  float scale = 1.0f / sqrtf(ss / (float)width + eps);
  if (vec4) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(v + i);
      if (write_x) *reinterpret_cast<float4*>(xr + i) = a;
      float4 g = load4_as_f32(w, w_dtype, i);
      store4_from_f32(out, out_dtype, (size_t)r * width + i,
                      make_float4(a.x * scale * g.x, a.y * scale * g.y, a.z * scale * g.z, a.w * scale * g.w));
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float a = v[i];
      if (write_x) xr[i] = a;
      store_from_f32(out, out_dtype, (size_t)r * width + i, a * scale * load_as_f32(w, w_dtype, i));
    }
  }
}

extern "C" int bn_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_parts, long long part_stride,
                              const void* w, int w_dtype,
                              void* out, int out_dtype, const int* rows, int n_rows, int width, float eps,
                              int write_x, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (width <= 0 || !(eps > 0.f) || (delta && n_parts < 1)) return BN_ERR_BAD_ARG;
  // few rows of a wide model: a cluster of blocks per row (columns in multiples of 4, all pointers
  // and row strides 16-byte aligned)
  int cols = ((width + NORM_CLUSTER - 1) / NORM_CLUSTER + 3) / 4 * 4;
  bool aligned = width % 8 == 0 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)w | (uintptr_t)delta) & 15) == 0 &&
                 (part_stride % 8) == 0;
  if (n_rows <= 256 && width >= 1024 && aligned && cols <= NORM_CL_THREADS * NORM_CL_VEC * 4) {
    BN_LAUNCH(add_rmsnorm_cluster_kernel, dim3(n_rows, NORM_CLUSTER), NORM_CL_THREADS, 0, stream, 
        x, delta, delta_dtype, n_parts, (size_t)part_stride, w, w_dtype, out, out_dtype, rows, width, cols, eps,
        write_x);
    BN_CHECK_LAUNCH();
    return BN_OK;
  }
  size_t smem = ((size_t)width + 32) * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;  // width beyond 51,168: refused
  if (smem > 48 * 1024) {
    static size_t granted = 0;
    if (smem > granted) {
      cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted = smem;
    }
  }
  int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  BN_LAUNCH(add_rmsnorm_kernel, n_rows, threads, smem, stream, x, delta, delta_dtype, n_parts, (size_t)part_stride, w,
                                                       w_dtype, out, out_dtype,
                                                       rows, width, eps, write_x, aligned ? 1 : 0);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// Norm after the sum (post-norm blocks): v = alpha * x + delta, x = v * rsqrt(mean(v^2) + eps) * w.
// The float32 residual x is rewritten in place with the norm's output, and `out` (optional)
// receives the same values in the compute type for the products that read them next.
__global__ void scaled_add_rmsnorm_kernel(float* __restrict__ x, float alpha, const void* __restrict__ delta,
                                          int delta_dtype, const void* __restrict__ w, int w_dtype,
                                          void* __restrict__ out, int out_dtype, int width, float eps, int vec4) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float v[];  // width floats, then 32 for the reduction
  float* scratch = v + width;
  size_t row = blockIdx.x;
  float* xr = x + row * width;
  float ss = 0.f;
  if (vec4) {  // groups of four columns in whole 8- or 16-byte pieces (the launcher checked the alignment)
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(xr + i);
      a.x *= alpha; a.y *= alpha; a.z *= alpha; a.w *= alpha;
      if (delta) {
        float4 d = load4_as_f32(delta, delta_dtype, row * width + i);
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
      }
      *reinterpret_cast<float4*>(v + i) = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float a = alpha * xr[i];
      if (delta) a += load_as_f32(delta, delta_dtype, row * width + i);
      v[i] = a;
      ss += a * a;
    }
  }
  ss = block_sum(ss, scratch);
  float scale = 1.0f / sqrtf(ss / (float)width + eps);
  if (vec4) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(v + i);
      float4 g = load4_as_f32(w, w_dtype, i);
      float4 y = make_float4(a.x * scale * g.x, a.y * scale * g.y, a.z * scale * g.z, a.w * scale * g.w);
      *reinterpret_cast<float4*>(xr + i) = y;
      if (out) store4_from_f32(out, out_dtype, row * width + i, y);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float y = v[i] * scale * load_as_f32(w, w_dtype, i);
      xr[i] = y;
      if (out) store_from_f32(out, out_dtype, row * width + i, y);
    }
  }
}

extern "C" int bn_scaled_add_rmsnorm(float* x, float alpha, const void* delta, int delta_dtype, const void* w,
                                     int w_dtype, void* out, int out_dtype, int n_rows, int width, float eps,
                                     cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (width <= 0 || !(eps > 0.f) || !x || !w) return BN_ERR_BAD_ARG;
  size_t smem = ((size_t)width + 32) * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;
  if (smem > 48 * 1024) {
    static size_t granted = 0;
    if (smem > granted) {
      cudaError_t e = cudaFuncSetAttribute(scaled_add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted = smem;
    }
  }
  int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  int vec4 = width % 8 == 0 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)w | (uintptr_t)delta) & 15) == 0;
  BN_LAUNCH(scaled_add_rmsnorm_kernel, n_rows, threads, smem, stream, x, alpha, delta, delta_dtype, w, w_dtype, out,
            out_dtype, width, eps, vec4);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// ---- parallel blocks ---------------------------------------------------------------------------
// x += a (+ b): the deltas of the two sublayers of a parallel block (any element type) meet in the
// float32 residual; `cast` (optional) receives the new rows in the compute type for the product
// that reads them next.
__global__ void residual_add_kernel(float* __restrict__ x, const void* __restrict__ a, int a_dtype,
                                    const void* __restrict__ b, int b_dtype, void* __restrict__ cast, int cast_dtype,
                                    size_t total, int vec4) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * (vec4 ? 4 : 1);
  if (i >= total) return;
  if (vec4) {
    float4 v = *reinterpret_cast<const float4*>(x + i);
    float4 d = load4_as_f32(a, a_dtype, i);
    if (b) {
      float4 e = load4_as_f32(b, b_dtype, i);
      d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;  // the sublayers' sum first, then onto the stream
    }
    v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    *reinterpret_cast<float4*>(x + i) = v;
    if (cast) store4_from_f32(cast, cast_dtype, i, v);
  } else {
    float d = load_as_f32(a, a_dtype, i);
    if (b) d += load_as_f32(b, b_dtype, i);
    float v = x[i] + d;
    x[i] = v;
    if (cast) store_from_f32(cast, cast_dtype, i, v);
  }
}

extern "C" int bn_residual_add(float* x, const void* a, int a_dtype, const void* b, int b_dtype, void* cast, int cast_dtype,
                               long long total, cudaStream_t stream) {
  if (total <= 0) return BN_OK;
  if (!x || !a) return BN_ERR_BAD_ARG;
  int vec4 = total % 4 == 0 && (((uintptr_t)x | (uintptr_t)a | (uintptr_t)b | (uintptr_t)cast) & 15) == 0;
  size_t threads = vec4 ? (size_t)total / 4 : (size_t)total;
  BN_LAUNCH(residual_add_kernel, (unsigned)((threads + 255) / 256), 256, 0, stream, x, a, a_dtype, b, b_dtype, cast,
            cast_dtype, (size_t)total, vec4);
  return BN_OK;
}

// x += a (+ b) as above, then the norms that read the stream next, in the same pass: out1 = x * rsqrt(mean(x^2) + eps) * w1
// and, if w2 is given, out2 = the same rows times w2 (two norms of one stream share their statistics).  One block
// per row; float32 sums and statistics; out1 / out2 in the compute type.
__global__ void residual_add_norms_kernel(float* __restrict__ x, const void* __restrict__ a, int a_dtype, const void* __restrict__ b,
                                          int b_dtype, const void* __restrict__ w1, const void* __restrict__ w2, int w_dtype,
                                          float eps, void* __restrict__ out1, void* __restrict__ out2, int out_dtype, int width) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float v[];  // width floats, then 32 for the reduction
  float* scratch = v + width;
  const size_t row = blockIdx.x;
  float* xr = x + row * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float d = load_as_f32(a, a_dtype, row * width + i);
    if (b) d += load_as_f32(b, b_dtype, row * width + i);  // the sublayers' sum first, then onto the stream
    const float t = xr[i] + d;
    xr[i] = t;
    v[i] = t;
    ss += t * t;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float t = v[i] * scale;
    store_from_f32(out1, out_dtype, row * width + i, t * load_as_f32(w1, w_dtype, i));
    if (w2) store_from_f32(out2, out_dtype, row * width + i, t * load_as_f32(w2, w_dtype, i));
  }
}

extern "C" int bn_residual_add_norms(float* x, const void* a, int a_dtype, const void* b, int b_dtype, const void* w1, const void* w2,
                                     int w_dtype, float eps, void* out1, void* out2, int out_dtype, int n_rows, int width,
                                     cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (width <= 0 || !(eps > 0.f) || !x || !a || !w1 || !out1 || (w2 && !out2)) return BN_ERR_BAD_ARG;
  size_t smem = ((size_t)width + 32) * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;
  if (smem > 48 * 1024) {
    static size_t granted = 0;
    if (smem > granted) {
      cudaError_t e = cudaFuncSetAttribute(residual_add_norms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted = smem;
    }
  }
  int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  BN_LAUNCH(residual_add_norms_kernel, n_rows, threads, smem, stream, x, a, a_dtype, b, b_dtype, w1, w2, w_dtype, eps, out1, out2,
            out_dtype, width);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// x += y / sqrt(mean(y^2) + eps_y) * wy: a delta that enters the stream through a norm of its own.
// Then, if `w` is given, out[r] = x * rsqrt(mean(x^2) + eps) * w: the norm that reads the stream next,
// in the same pass (out in the compute type).  One block per row; float32 statistics.  VEC: rows of whole
// 16-byte pieces at aligned addresses are read and written four numbers at a time.
template <bool VEC>
__global__ void add_normed_kernel(float* __restrict__ x, const void* __restrict__ y, int y_dtype,
                                  const void* __restrict__ wy, int wy_dtype, float eps_y, const void* __restrict__ w,
                                  int w_dtype, float eps, void* __restrict__ out, int out_dtype, int width) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float v[];  // width floats, then 32 for the reductions
  float* scratch = v + width;
  const size_t row = blockIdx.x;
  float* xr = x + row * width;
  if (VEC) {
    const int n4 = width >> 2;
    const size_t r4 = row * n4;
    float4* v4 = reinterpret_cast<float4*>(v);
    float4* x4 = reinterpret_cast<float4*>(xr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 a = load4_as_f32(y, y_dtype, (r4 + i) * 4);
      v4[i] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
    ss = block_sum(ss, scratch);
    const float scale_y = 1.0f / sqrtf(ss / (float)width + eps_y);
    float sx = 0.f;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 g = load4_as_f32(wy, wy_dtype, (size_t)i * 4), b = v4[i];
      float4 a = x4[i];
      a.x += b.x * scale_y * g.x; a.y += b.y * scale_y * g.y; a.z += b.z * scale_y * g.z; a.w += b.w * scale_y * g.w;
      x4[i] = a;
      v4[i] = a;
      sx += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
    if (!w) return;
    sx = block_sum(sx, scratch);
    const float scale = 1.0f / sqrtf(sx / (float)width + eps);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 g = load4_as_f32(w, w_dtype, (size_t)i * 4), a = v4[i];
      store4_from_f32(out, out_dtype, (r4 + i) * 4, make_float4(a.x * scale * g.x, a.y * scale * g.y, a.z * scale * g.z, a.w * scale * g.w));
    }
    return;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float a = load_as_f32(y, y_dtype, row * width + i);
    v[i] = a;
    ss += a * a;
  }
  ss = block_sum(ss, scratch);
  const float scale_y = 1.0f / sqrtf(ss / (float)width + eps_y);
  float sx = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float a = xr[i] + v[i] * scale_y * load_as_f32(wy, wy_dtype, i);
    xr[i] = a;
    v[i] = a;
    sx += a * a;
  }
  if (!w) return;
  sx = block_sum(sx, scratch);
  const float scale = 1.0f / sqrtf(sx / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    store_from_f32(out, out_dtype, row * width + i, v[i] * scale * load_as_f32(w, w_dtype, i));
}

extern "C" int bn_add_normed(float* x, const void* y, int y_dtype, const void* wy, int wy_dtype, float eps_y, const void* w,
                             int w_dtype, float eps, void* out, int out_dtype, int n_rows, int width, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (width <= 0 || !(eps_y > 0.f) || !x || !y || !wy || (w && (!out || !(eps > 0.f)))) return BN_ERR_BAD_ARG;
  size_t smem = ((size_t)width + 32) * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;
  const bool vec = width % 4 == 0 && !(((uintptr_t)x | (uintptr_t)y | (uintptr_t)wy | (uintptr_t)w | (uintptr_t)out) & 15);
  if (smem > 48 * 1024) {
    static size_t granted = 0;
    if (smem > granted) {
      cudaError_t e = cudaFuncSetAttribute(add_normed_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(add_normed_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted = smem;
    }
  }
  int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  if (vec)
    BN_LAUNCH(add_normed_kernel<true>, n_rows, threads, smem, stream, x, y, y_dtype, wy, wy_dtype, eps_y, w, w_dtype, eps, out,
              out_dtype, width);
  else
    BN_LAUNCH(add_normed_kernel<false>, n_rows, threads, smem, stream, x, y, y_dtype, wy, wy_dtype, eps_y, w, w_dtype, eps, out,
              out_dtype, width);
  return BN_OK;
}

// RMS norms of up to two slices of every row, in place: x[t, off_s : off_s + len_s] becomes
// v * rsqrt(mean(v^2) + eps) * w_s (the latents of a low-rank projection, each with its own gain).
// One warp per (row, slice); float32 statistics; x and the gains of type `dtype` / `w_dtype`.
__global__ void rmsnorm_slices_kernel(void* __restrict__ x, int dtype, int stride, int n_rows, int off0, int len0,
                                      const void* __restrict__ w0, int off1, int len1, const void* __restrict__ w1,
                                      int w_dtype, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int n_slices = len1 > 0 ? 2 : 1;
  const int item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (item >= n_rows * n_slices) return;
  const int row = item / n_slices, s = item - row * n_slices;
  const int off = s ? off1 : off0, len = s ? len1 : len0;
  const void* w = s ? w1 : w0;
  const size_t base = (size_t)row * stride + off;
  float ss = 0.f;
  for (int i = lane; i < len; i += 32) {
    float a = load_as_f32(x, dtype, base + i);
    ss += a * a;
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)len + eps);
  for (int i = lane; i < len; i += 32)
    store_from_f32(x, dtype, base + i, load_as_f32(x, dtype, base + i) * scale * load_as_f32(w, w_dtype, i));
}

extern "C" int bn_rmsnorm_slices(void* x, int dtype, int stride, int n_rows, int off0, int len0, const void* w0, int off1,
                                 int len1, const void* w1, int w_dtype, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (!x || !w0 || len0 <= 0 || off0 < 0 || off0 + len0 > stride || !(eps > 0.f) ||
      (len1 > 0 && (!w1 || off1 < 0 || off1 + len1 > stride)) || len1 < 0)
    return BN_ERR_BAD_ARG;
  const int items = n_rows * (len1 > 0 ? 2 : 1);
  BN_LAUNCH(rmsnorm_slices_kernel, (unsigned)((items + 7) / 8), 256, 0, stream, x, dtype, stride, n_rows, off0, len0, w0, off1,
            len1, w1, w_dtype, eps);
  return BN_OK;
}
