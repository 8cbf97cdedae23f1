// Mixture of experts with sigmoid scores: routing, and the expert products for few tokens.
//
//   z = W_router h (float32), s = sigmoid(z); each token takes the `top` experts with the largest
//   scores; its weight for an expert is that expert's score, taken as it is (or renormalised over the
//   chosen ones), and multiplies either the expert's input or its output.
//
//   bn_moe_route     ids[t][k], weights[t][k] for every token
//   bn_moe_gate_up   y[t * top + k] = act(W_gate[e] x, W_up[e] x) with x = h[t] (times the weight, when it
//                    scales the input) for e = ids[t][k]
//   bn_moe_down      out[t] = sum_k (weight) W_down[e] y[t * top + k] (+ what a shared expert gave), float32
//   bn_moe_scale_rows  x[t * top + k] = weight[t][k] * h[t], for the path that multiplies expert by expert
//
// The two product kernels stream an expert's matrices once per (token, expert) and are meant for the
// few rows of a decode step; they read everything they need from device memory, so a step that
// uses them can be recorded.  With many rows the tokens are sorted by expert instead and every
// expert's rows go through the library's ordinary products (parts/moe.py).
//
// The activation is the clamped gated unit of act.cu: g = min(gate, limit), u = clamp(up, +-limit),
// y = g * sigmoid(slope * g) * (u + 1).
#include "common.cuh"

#define MOE_MAX_EXPERTS 1024

template <typename T, typename W>
__global__ void moe_route_kernel(const T* __restrict__ h, int width, const W* __restrict__ w, int n_experts, int top,
                                 int renormalise, int softmax, float weight_scale, float sum_eps, int* __restrict__ ids,
                                 float* __restrict__ weights) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float z[MOE_MAX_EXPERTS];
  extern __shared__ __align__(16) float xs[];  // width
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const T* row = h + (size_t)t * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32<T>(row[c]);
  __syncthreads();
  for (int e = warp; e < n_experts; e += n_warps) {
    float dot = warp_dot(xs, w + (size_t)e * width, width, lane);
    if (lane == 0) z[e] = dot;
  }
  __syncthreads();
  if (warp == 0) {
    // softmax scores: e^(z - max) over the sum of all experts' (the order of the scores is the logits')
    float z_max = -INFINITY, z_sum = 0.f;
    if (softmax) {
      for (int e = lane; e < n_experts; e += 32) z_max = fmaxf(z_max, z[e]);
      z_max = warp_max(z_max);
      for (int e = lane; e < n_experts; e += 32) z_sum += expf(z[e] - z_max);
      z_sum = warp_sum(z_sum);
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
      // the largest logit left; among equal ones the lowest index
      float best = -INFINITY;
      int arg = n_experts;
      for (int e = lane; e < n_experts; e += 32)
        if (z[e] > best) { best = z[e]; arg = e; }
      for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
      }
      float s = softmax ? expf(best - z_max) / z_sum : 1.0f / (1.0f + expf(-best));
      total += s;
      if (lane == 0) {
        ids[(size_t)t * top + k] = arg;
        weights[(size_t)t * top + k] = s;
        z[arg] = -INFINITY;
      }
      __syncwarp();
    }
    __syncwarp();
    if (lane < top && (renormalise || weight_scale != 1.0f)) {
      float wt = weights[(size_t)t * top + lane];
      if (renormalise) wt /= total + sum_eps;
      weights[(size_t)t * top + lane] = wt * weight_scale;
    }
  }
}

// softmax: the scores are the softmax over all experts instead of each logit's logistic function; the chosen
// experts' scores are divided by their sum + sum_eps with `renormalise`, then multiplied by weight_scale
extern "C" int bn_moe_route_ex(const void* h, int h_dtype, int n_tokens, int width, const void* w, int w_dtype,
                               int n_experts, int top, int renormalise, int softmax, float weight_scale, float sum_eps,
                               int* ids, float* weights, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!h || !w || !ids || !weights || width <= 0 || n_experts <= 0 || n_experts > MOE_MAX_EXPERTS || top <= 0 ||
      top > n_experts || top > 32 || (size_t)width * sizeof(float) > 40 * 1024)
    return BN_ERR_BAD_ARG;
  const size_t smem = (size_t)width * sizeof(float);
  if (h_dtype == BN_F32 && w_dtype == BN_F32)
    BN_LAUNCH((moe_route_kernel<float, float>), n_tokens, 256, smem, stream, (const float*)h, width, (const float*)w,
              n_experts, top, renormalise, softmax, weight_scale, sum_eps, ids, weights);
  else if (h_dtype == BN_BF16 && w_dtype == BN_BF16)
    BN_LAUNCH((moe_route_kernel<__nv_bfloat16, __nv_bfloat16>), n_tokens, 256, smem, stream, (const __nv_bfloat16*)h, width,
              (const __nv_bfloat16*)w, n_experts, top, renormalise, softmax, weight_scale, sum_eps, ids, weights);
  else if (h_dtype == BN_BF16 && w_dtype == BN_F32)
    BN_LAUNCH((moe_route_kernel<__nv_bfloat16, float>), n_tokens, 256, smem, stream, (const __nv_bfloat16*)h, width,
              (const float*)w, n_experts, top, renormalise, softmax, weight_scale, sum_eps, ids, weights);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}

extern "C" int bn_moe_route(const void* h, int h_dtype, int n_tokens, int width, const void* w, int w_dtype,
                            int n_experts, int top, int renormalise, int* ids, float* weights, cudaStream_t stream) {
  return bn_moe_route_ex(h, h_dtype, n_tokens, width, w, w_dtype, n_experts, top, renormalise, 0, 1.0f, 0.0f, ids, weights, stream);
}

#define MOE_THREADS 256
#define MOE_ROWS_PER_BLOCK 32  // outputs per block of the product kernels

// grid (tokens * top, ceil(ff / MOE_ROWS_PER_BLOCK)); row j of expert e's gate matrix lies at
// w_gate + e * expert_stride + j * width, of its up matrix at w_up + the same (so that one tensor
// [experts, 2 * ff, width] with the gate rows first serves both)
template <typename T>
__global__ void moe_gate_up_kernel(const T* __restrict__ h, int width, const int* __restrict__ ids,
                                   const float* __restrict__ weights, int scale_input, const T* __restrict__ w_gate,
                                   const T* __restrict__ w_up, size_t expert_stride, int ff, int top, float limit,
                                   float slope, int act, T* __restrict__ y) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float xs[];  // width
  const int item = blockIdx.x, t = item / top;
  const int e = ids[item];
  const float wt = scale_input ? weights[item] : 1.0f;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  // the expert's input in the compute type, as the path that sorts tokens by expert stores it
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    xs[c] = to_f32<T>(from_f32<T>(to_f32<T>(h[(size_t)t * width + c]) * wt));
  __syncthreads();
  const int j0 = blockIdx.y * MOE_ROWS_PER_BLOCK, j1 = min(ff, j0 + MOE_ROWS_PER_BLOCK);
  // a warp takes four neighbouring rows of both matrices at a time
  for (int j = j0 + warp * 4; j < j1; j += n_warps * 4) {
    float g4[4], u4[4];
    const T* gr = w_gate + (size_t)e * expert_stride + (size_t)j * width;
    const T* ur = w_up + (size_t)e * expert_stride + (size_t)j * width;
    if (j + 4 <= j1) {
      warp_dot_rows<4>(xs, gr, (size_t)width, width, lane, g4);
      warp_dot_rows<4>(xs, ur, (size_t)width, width, lane, u4);
    } else {
      for (int r = 0; r < j1 - j; ++r) {
        g4[r] = warp_dot(xs, gr + (size_t)r * width, width, lane);
        u4[r] = warp_dot(xs, ur + (size_t)r * width, width, lane);
      }
    }
    if (lane < 4 && j + lane < j1) {
      // the products' results pass through the compute type, as they do on the sorted path
      float g = lane == 0 ? g4[0] : lane == 1 ? g4[1] : lane == 2 ? g4[2] : g4[3];
      float u = lane == 0 ? u4[0] : lane == 1 ? u4[1] : lane == 2 ? u4[2] : u4[3];
      g = to_f32<T>(from_f32<T>(g));
      u = to_f32<T>(from_f32<T>(u));
      if (act >= 0) {  // the plain gated unit: act(g) * u
        y[(size_t)item * ff + j + lane] = from_f32<T>(glu_activation(g, act) * u);
      } else {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        y[(size_t)item * ff + j + lane] = from_f32<T>(g / (1.0f + expf(-slope * g)) * (u + 1.0f));
      }
    }
  }
}

// grid (tokens, ceil(width / MOE_ROWS_PER_BLOCK)); w_down: [experts, width, ff]
template <typename T>
__global__ void moe_down_kernel(const T* __restrict__ y, int ff, const int* __restrict__ ids,
                                const float* __restrict__ weights, int scale_output, const T* __restrict__ w_down,
                                int width, int top, const void* __restrict__ add, int add_dtype, float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float ys[];  // top * ff: the token's activations, expert by expert
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < top * ff; i += blockDim.x) ys[i] = to_f32<T>(y[(size_t)t * top * ff + i]);
  __syncthreads();
  const int c0 = blockIdx.y * MOE_ROWS_PER_BLOCK, c1 = min(width, c0 + MOE_ROWS_PER_BLOCK);
  for (int c = c0 + warp * 4; c < c1; c += n_warps * 4) {
    float total[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top; ++k) {
      const int e = ids[(size_t)t * top + k];
      const T* wr = w_down + ((size_t)e * width + c) * ff;
      float d4[4] = {0.f, 0.f, 0.f, 0.f};
      if (c + 4 <= c1) {
        warp_dot_rows<4>(ys + (size_t)k * ff, wr, (size_t)ff, ff, lane, d4);
      } else {
        for (int r = 0; r < c1 - c; ++r) d4[r] = warp_dot(ys + (size_t)k * ff, wr + (size_t)r * ff, ff, lane);
      }
      const float wt = scale_output ? weights[(size_t)t * top + k] : 1.0f;
#pragma unroll
      for (int r = 0; r < 4; ++r) total[r] += d4[r] * wt;
    }
    if (lane < 4 && c + lane < c1) {
      float v = lane == 0 ? total[0] : lane == 1 ? total[1] : lane == 2 ? total[2] : total[3];
      if (add) v += load_as_f32(add, add_dtype, (size_t)t * width + c + lane);
      out[(size_t)t * width + c + lane] = v;
    }
  }
}

// Shared memory beyond the default 48 KB is asked for once per kernel and size (up to MOE_SMEM_MAX bytes).
#define MOE_SMEM_MAX (200 * 1024)
template <typename K>
static int moe_grant_smem(K kernel, size_t smem, size_t* granted) {
  if (smem > MOE_SMEM_MAX) return BN_ERR_BAD_ARG;
  if (smem > 48 * 1024 && smem > *granted) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    *granted = smem;
  }
  return BN_OK;
}

// act < 0: the clamped unit with `limit` and `slope`; act >= 0 (BN_ACT_*): act(gate) * up without clamps
extern "C" int bn_moe_gate_up_ex(const void* h, int dtype, int n_tokens, int width, const int* ids, const float* weights,
                                 int scale_input, const void* w_gate, const void* w_up, long long expert_stride, int ff, int top,
                                 float limit, float slope, int act, void* y, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!h || !ids || !weights || !w_gate || !w_up || !y || width <= 0 || ff <= 0 || top <= 0) return BN_ERR_BAD_ARG;
  size_t smem = (size_t)width * sizeof(float);
  static size_t granted[2] = {0, 0};
  int rc = dtype == BN_F32 ? moe_grant_smem(moe_gate_up_kernel<float>, smem, &granted[0])
                           : moe_grant_smem(moe_gate_up_kernel<__nv_bfloat16>, smem, &granted[1]);
  if (rc != BN_OK) return rc;
  dim3 grid(n_tokens * top, (ff + MOE_ROWS_PER_BLOCK - 1) / MOE_ROWS_PER_BLOCK);
  if (dtype == BN_F32)
    BN_LAUNCH(moe_gate_up_kernel<float>, grid, MOE_THREADS, smem, stream, (const float*)h, width, ids, weights, scale_input,
              (const float*)w_gate, (const float*)w_up, (size_t)expert_stride, ff, top, limit, slope, act, (float*)y);
  else if (dtype == BN_BF16)
    BN_LAUNCH(moe_gate_up_kernel<__nv_bfloat16>, grid, MOE_THREADS, smem, stream, (const __nv_bfloat16*)h, width, ids,
              weights, scale_input, (const __nv_bfloat16*)w_gate, (const __nv_bfloat16*)w_up, (size_t)expert_stride, ff, top, limit,
              slope, act, (__nv_bfloat16*)y);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}

extern "C" int bn_moe_gate_up(const void* h, int dtype, int n_tokens, int width, const int* ids, const float* weights,
                              int scale_input, const void* w_gate, const void* w_up, long long expert_stride, int ff, int top,
                              float limit, float slope, void* y, cudaStream_t stream) {
  return bn_moe_gate_up_ex(h, dtype, n_tokens, width, ids, weights, scale_input, w_gate, w_up, expert_stride, ff, top, limit, slope,
                           -1, y, stream);
}

extern "C" int bn_moe_down(const void* y, int dtype, int n_tokens, int ff, const int* ids, const float* weights,
                           int scale_output, const void* w_down, int width, int top, const void* add, int add_dtype,
                           float* out, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!y || !ids || !weights || !w_down || !out || width <= 0 || ff <= 0 || top <= 0) return BN_ERR_BAD_ARG;
  dim3 grid(n_tokens, (width + MOE_ROWS_PER_BLOCK - 1) / MOE_ROWS_PER_BLOCK);
  const size_t smem = (size_t)top * ff * sizeof(float);
  static size_t granted[2] = {0, 0};
  int rc = dtype == BN_F32 ? moe_grant_smem(moe_down_kernel<float>, smem, &granted[0])
                           : moe_grant_smem(moe_down_kernel<__nv_bfloat16>, smem, &granted[1]);
  if (rc != BN_OK) return rc;
  if (dtype == BN_F32)
    BN_LAUNCH(moe_down_kernel<float>, grid, MOE_THREADS, smem, stream, (const float*)y, ff, ids, weights, scale_output,
              (const float*)w_down, width, top, add, add_dtype, out);
  else if (dtype == BN_BF16)
    BN_LAUNCH(moe_down_kernel<__nv_bfloat16>, grid, MOE_THREADS, smem, stream, (const __nv_bfloat16*)y, ff, ids, weights,
              scale_output, (const __nv_bfloat16*)w_down, width, top, add, add_dtype, out);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// ---- sorting tokens by expert (many rows) --------------------------------------------------------
// counts[e] = how many (token, k) items chose expert e; one thread per item.
__global__ void moe_count_kernel(const int* __restrict__ ids, int n_items, int* __restrict__ counts) {
  pdl_launch_dependents();
  pdl_wait();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_items) atomicAdd(&counts[ids[i]], 1);
}

// offsets[e] = first row of expert e in the sorted order: the experts' rows packed one behind another
// (cap == 0; offsets[n_experts] = n_items), or every expert in a block of cap rows of its own; one block.
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int n_experts, int cap, int* __restrict__ offsets,
                                   int* __restrict__ cursor) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < n_experts; ++e) {
      offsets[e] = at;
      cursor[e] = at;
      at += cap > 0 ? cap : counts[e];
    }
    offsets[n_experts] = at;
  }
}

// place[i] = row of item i in the sorted order, and x_sorted[place[i]] = weight * h[token of i] (or h itself).
// Rows of one expert come in any order; every row is computed alone, so the order changes no result.
template <typename T>
__global__ void moe_scatter_kernel(const T* __restrict__ h, int width, const int* __restrict__ ids,
                                   const float* __restrict__ weights, int scale_input, int top, int* __restrict__ cursor,
                                   int* __restrict__ place, T* __restrict__ x_sorted) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int row;
  const int item = blockIdx.x, t = item / top;
  if (threadIdx.x == 0) {
    row = atomicAdd(&cursor[ids[item]], 1);
    place[item] = row;
  }
  __syncthreads();
  const float wt = scale_input ? weights[item] : 1.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    x_sorted[(size_t)row * width + c] = from_f32<T>(to_f32<T>(h[(size_t)t * width + c]) * wt);
}

// out[t] = sum_k (weight) y_sorted[place[t * top + k]] (+ add[t]), float32
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ y_sorted, int width, const int* __restrict__ place,
                                  const float* __restrict__ weights, int scale_output, int top,
                                  const void* __restrict__ add, int add_dtype, float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
      float v = to_f32<T>(y_sorted[(size_t)place[(size_t)t * top + k] * width + c]);
      total += scale_output ? v * weights[(size_t)t * top + k] : v;
    }
    if (add) total += load_as_f32(add, add_dtype, (size_t)t * width + c);
    out[(size_t)t * width + c] = total;
  }
}

// counts: [n_experts], zeroed by the caller: how many (token, expert) items chose each expert
extern "C" int bn_moe_count(const int* ids, int n_items, int* counts, cudaStream_t stream) {
  if (n_items <= 0) return BN_OK;
  if (!ids || !counts) return BN_ERR_BAD_ARG;
  BN_LAUNCH(moe_count_kernel, (n_items + 255) / 256, 256, 0, stream, ids, n_items, counts);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// counts as bn_moe_count left them; offsets: [n_experts + 1]; cursor: [n_experts]; place: [n_items];
// x_sorted: [n_items, width] (cap == 0) or [n_experts * cap, width] (cap >= the largest count)
extern "C" int bn_moe_scatter(const void* h, int dtype, int n_tokens, int width, const int* ids, const float* weights,
                              int scale_input, int top, int n_experts, int cap, const int* counts, int* offsets,
                              int* cursor, int* place, void* x_sorted, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!h || !ids || !weights || !counts || !offsets || !cursor || !place || !x_sorted || width <= 0 || top <= 0 ||
      n_experts <= 0 || cap < 0)
    return BN_ERR_BAD_ARG;
  int n_items = n_tokens * top;
  BN_LAUNCH(moe_offsets_kernel, 1, 32, 0, stream, counts, n_experts, cap, offsets, cursor);
  if (dtype == BN_F32)
    BN_LAUNCH(moe_scatter_kernel<float>, n_items, 128, 0, stream, (const float*)h, width, ids, weights, scale_input, top,
              cursor, place, (float*)x_sorted);
  else if (dtype == BN_BF16)
    BN_LAUNCH(moe_scatter_kernel<__nv_bfloat16>, n_items, 128, 0, stream, (const __nv_bfloat16*)h, width, ids, weights,
              scale_input, top, cursor, place, (__nv_bfloat16*)x_sorted);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}

extern "C" int bn_moe_gather(const void* y_sorted, int dtype, int n_tokens, int width, const int* place,
                             const float* weights, int scale_output, int top, const void* add, int add_dtype, float* out,
                             cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!y_sorted || !place || !weights || !out || width <= 0 || top <= 0) return BN_ERR_BAD_ARG;
  if (dtype == BN_F32)
    BN_LAUNCH(moe_gather_kernel<float>, n_tokens, 256, 0, stream, (const float*)y_sorted, width, place, weights,
              scale_output, top, add, add_dtype, out);
  else if (dtype == BN_BF16)
    BN_LAUNCH(moe_gather_kernel<__nv_bfloat16>, n_tokens, 256, 0, stream, (const __nv_bfloat16*)y_sorted, width, place,
              weights, scale_output, top, add, add_dtype, out);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// Experts by a table instead of a router: token id -> the `top` experts of its row, each with the same weight.
// table [vocab, table_stride] int32; an id outside the table, or an entry outside the experts, takes expert 0
// with weight 0 (it adds nothing).
__global__ void moe_table_route_kernel(const int* __restrict__ tokens, int n_tokens, const int* __restrict__ table, int vocab,
                                       int table_stride, int top, int n_experts, float weight, int* __restrict__ ids,
                                       float* __restrict__ weights) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * top) return;
  const int t = i / top, k = i - t * top;
  const int tok = tokens[t];
  int e = tok >= 0 && tok < vocab ? table[(size_t)tok * table_stride + k] : -1;
  const bool ok = e >= 0 && e < n_experts;
  ids[i] = ok ? e : 0;
  weights[i] = ok ? weight : 0.f;
}

extern "C" int bn_moe_table_route(const int* tokens, int n_tokens, const int* table, int vocab, int table_stride, int top,
                                  int n_experts, float weight, int* ids, float* weights, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!tokens || !table || !ids || !weights || top <= 0 || top > table_stride || vocab <= 0 || n_experts <= 0) return BN_ERR_BAD_ARG;
  BN_LAUNCH(moe_table_route_kernel, (n_tokens * top + 255) / 256, 256, 0, stream, tokens, n_tokens, table, vocab, table_stride, top,
            n_experts, weight, ids, weights);
  BN_CHECK_LAUNCH();
  return BN_OK;
}
