// Attention without a softmax for runs of new tokens in bfloat16, on the tensor cores, one thread-block
// cluster per 16 new tokens of a sequence.
//
//   a_g(i, j) = sigmoid(q_g(i) . k_c(g)(j) * scale + rel[min(i - j, n_rel - 1)][g])   for 0 <= i - j < window
//   w_h(i, j) = sum_g mix[h][g] a_g(i, j)                                             (mix null: w = a)
//   out_h(i)  = gate_h(i) * sum_j w_h(i, j) v_c(h)(j)
//
// Nothing is normalised over the keys, but the mixing needs every head's weight of a (query, key) pair, so the
// heads cannot run apart.  The cluster has one block per key/value head c; a block has WPH warps per query head
// of c (1, 2 or 4, so that a block has about eight).  Per page of 64 keys: the warps of a head compute its
// 16 x 64 scores with m16n8k16 MMAs, each 64 / WPH of the keys (queries held in registers as A fragments, the
// key page in shared memory), and leave the logistic weights in their block's shared memory as float32; after a cluster barrier every warp takes some of the page's eight 8-key column
// groups, reads all heads' weights of those columns from all blocks (distributed shared memory), mixes them
// for the heads of its own block (float32 FMAs) and leaves them in local shared memory; then the warps of a head
// multiply its mixed weights with the value page, each for 1 / WPH of the value columns, the weights entering the tensor cores as the sum
// of two bfloat16 terms (16 bits of mantissa), accumulating in float32 registers over all pages.  The second
// cluster barrier of a page (no block overwrites weights another still reads) is split: arrive after the
// mixing, wait before the next page's weights are written.
// With four or eight key/value heads of up to four query heads each the exchange runs the other way (SLICE below):
// a block mixes all heads' weights of its share of the page's keys, and every block then fetches its own heads'
// mixed weights, which moves a fraction of the bytes between the blocks.
// The new tokens' keys and values must already be in the cache; pages are [page][kv head][64][width].
#include "mma.cuh"

#define SP_M 16
#define SP_N 64
#define SP_LD 72        // floats per row of a weight tile: 64 + 8, so that float2 accesses of a quad pattern spread over all banks
#define SP_MAX_R 8      // query heads per key/value head (warps per block)
#define SP_BIAS 80      // distances one tile's scores can have: 16 + 64 - 1, rounded up

template <int HD>
__device__ __forceinline__ unsigned sp_off(int row, int chunk) {
  return (unsigned)(row * HD * 2 + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ void sp_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void sp_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ unsigned sp_map(unsigned local_addr, unsigned rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
// volatile keeps it between the cluster barriers (which clobber memory); without a clobber of its own several may be in flight
__device__ __forceinline__ float4 sp_ld4(unsigned cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(cluster_addr));
  return v;
}
__device__ __forceinline__ float sp_ld1(unsigned cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr));
  return v;
}
__device__ __forceinline__ float sp_rest(float p) { return p - __bfloat162float(__float2bfloat16_rn(p)); }

struct SpArgs {
  const __nv_bfloat16* q;
  int q_stride;
  __nv_bfloat16* out;
  int out_stride, n_heads, n_kv_heads, head_dim, v_dim;
  float scale;
  int window;
  const float* rel;
  int n_rel;
  const float* mix;
  const __nv_bfloat16* gate;
  int gate_stride, gate_mode;
  const int *tile_seq, *tile_row0, *seq_start, *seq_pos0, *slots, *page_table;
  int pt_stride;
  const __nv_bfloat16 *k_cache, *v_cache;
  float* part;   // not null: the pages of a block of rows are dealt out over n_splits clusters (blockIdx.z), which
  int n_splits;  // leave their sums here, float32 [tokens][n_splits][n_heads * v_dim], for the kernel that adds them up
};

// RP: the query heads per key/value head, rounded up to a power of two (the mixing keeps so many accumulators
// per column); the warps per query head follow from it, so that a block has about eight warps.
// SLICE (4 or 8 key/value heads, up to 4 query heads each): the mixing is dealt out by keys instead.  Block c
// reads all heads' weights of its 64 / G keys only, mixes them for *all* heads, and leaves the mixed weights in its
// shared memory, from where every block fetches its own heads' (a second cluster barrier in between): every weight
// crosses the SM-to-SM network about twice instead of once per block of the cluster.  The values have one
// stage then (asked for at the top of their page's turn, needed at its end).
template <int HD, int VD, int RP, bool SLICE>
__global__ void __launch_bounds__(32 * SP_MAX_R, RP <= 4 ? 2 : 1)
sigmoid_attention_prefill_kernel(const SpArgs a) {
  constexpr int WPH = RP <= 2 ? 4 : (RP <= 4 ? 2 : 1);
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int KTILE = SP_N * HD * 2, VTILE = SP_N * VD * 2;
  constexpr int CHUNKS = HD / 8, VCHUNKS = VD / 8, KSTEPS = HD / 16;
  constexpr int NJ = SP_N / 8 / WPH;  // 8-key column groups whose scores a warp computes
  constexpr int NO = VD / 8 / WPH;    // 8-wide column tiles of the output that a warp sums
  const int R = a.n_heads / a.n_kv_heads, H = a.n_heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g4 = lane >> 2, t4 = lane & 3;
  const int n_warps = R * WPH, n_threads = 32 * n_warps;
  const int hr = warp / WPH, wq = warp % WPH;  // this warp's head within the block, and its share of that head's work
  const int c = blockIdx.x;  // key/value head = rank in the cluster
  const int h = c * R + hr;
  const unsigned s_k = (unsigned)__cvta_generic_to_shared(smem);   // two stages
  const unsigned s_v = s_k + 2 * KTILE;                            // two stages (SLICE: one)
  constexpr int V_STAGES = SLICE ? 1 : 2;
  const int G = a.n_kv_heads;
  float* s_a = reinterpret_cast<float*>(smem + 2 * KTILE + V_STAGES * VTILE);  // [R][16][SP_LD] this block's heads' weights
  float* s_w = s_a + R * SP_M * SP_LD;                                  // [R][16][SP_LD] the same heads' mixed weights
  // [H][SP_MAX_R]: mix[c * R + r][g] at [g][r]; SLICE: [H][G][SP_MAX_R]: mix[c2 * R + r][g] at [g][c2][r]
  float* s_mix = s_w + R * SP_M * SP_LD;
  float* s_bias = s_mix + H * SP_MAX_R * (SLICE ? G : 1);               // [warps][SP_BIAS]
  float* s_ws = s_bias + n_warps * SP_BIAS;                             // SLICE: [H][16][64 / G] all heads' mixed weights of this block's keys
  const unsigned s_a_addr = (unsigned)__cvta_generic_to_shared(s_a);
  const unsigned s_ws_addr = (unsigned)__cvta_generic_to_shared(s_ws);

  const int blk = gridDim.y - 1 - blockIdx.y;
  const int seq = a.tile_seq[blk], row0 = (a.tile_row0 ? a.tile_row0[blk] : 0) + (a.part ? 0 : blockIdx.z * SP_M);
  const int split = a.part ? blockIdx.z : 0, stride = a.part ? a.n_splits : 1;
  const int start = a.seq_start[seq], n_new = a.seq_start[seq + 1] - start, pos0 = a.seq_pos0[seq];
  if (row0 >= n_new) return;  // the whole cluster alike
  const int* pt = a.page_table + (size_t)a.slots[seq] * a.pt_stride;
  const int rows_here = min(SP_M, n_new - row0);
  const int seq_last = pos0 + n_new - 1;
  const int q_first = pos0 + row0, q_last = q_first + rows_here - 1;
  const int lo_first = a.window > 0 ? max(0, q_first - a.window + 1) : 0;
  const int tile_lo = lo_first / SP_N + split;
  const int n_walk = max(0, (q_last / SP_N - tile_lo + stride) / stride);  // pages tile_lo, tile_lo + stride, ...
  const int real_chunks = a.head_dim / 8, real_vchunks = a.v_dim / 8;

  // ---- queries: through shared memory (the mixed weights' place) into A fragments
  {
    const unsigned s_q = (unsigned)__cvta_generic_to_shared(s_w);
    for (int p = tid; p < R * SP_M * CHUNKS; p += n_threads) {
      const int r = p / (SP_M * CHUNKS), rem = p % (SP_M * CHUNKS), row = rem / CHUNKS, ch = rem % CHUNKS;
      const bool ok = row < rows_here && ch < real_chunks;
      const __nv_bfloat16* src = ok ? a.q + (size_t)(start + row0 + row) * a.q_stride + (size_t)(c * R + r) * a.head_dim + ch * 8 : a.q;
      cp_async16(s_q + r * SP_M * HD * 2 + sp_off<HD>(row, ch), src, ok);
    }
    cp_async_commit();
  }
  for (int i = tid; i < H * SP_MAX_R * (SLICE ? G : 1); i += n_threads) {
    const int r = i % SP_MAX_R, c2 = SLICE ? (i / SP_MAX_R) % G : c, g = i / (SP_MAX_R * (SLICE ? G : 1));
    s_mix[i] = r < R ? (a.mix ? a.mix[(size_t)(c2 * R + r) * H + g] : (g == c2 * R + r ? 1.f : 0.f)) : 0.f;
  }
  cp_async_wait<0>();
  __syncthreads();
  unsigned qf[KSTEPS][4];
  {
    const unsigned s_q = (unsigned)__cvta_generic_to_shared(s_w) + hr * SP_M * HD * 2;
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) ldsm_x4(s_q + sp_off<HD>(r + (mi & 1) * 8, ks * 2 + (mi >> 1)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }
  __syncthreads();  // the mixed weights' place is free again

  // the page's number is asked for one page ahead of its rows, the bias of a page's distances one page ahead of
  // its scores: no warp waits for either
  auto load_k = [&](int page, int stage) {
    const __nv_bfloat16* kb = a.k_cache + ((size_t)page * a.n_kv_heads + c) * BN_PAGE * a.head_dim;
    for (int p = tid; p < SP_N * CHUNKS; p += n_threads) {
      const int r = p / CHUNKS, ch = p % CHUNKS;
      const bool ok = ch < real_chunks;
      cp_async16(s_k + stage * KTILE + sp_off<HD>(r, ch), ok ? kb + (size_t)r * a.head_dim + ch * 8 : kb, ok);
    }
  };
  auto load_v = [&](int tile, int page, int stage) {
    const __nv_bfloat16* vb = a.v_cache + ((size_t)page * a.n_kv_heads + c) * BN_PAGE * a.v_dim;
    for (int p = tid; p < SP_N * VCHUNKS; p += n_threads) {
      const int r = p / VCHUNKS, ch = p % VCHUNKS;
      // rows behind the sequence's last position are zero, whatever the cache holds: zero weights times anything stay zero
      const bool ok = ch < real_vchunks && tile * SP_N + r <= seq_last;
      cp_async16(s_v + stage * VTILE + sp_off<VD>(r, ch), ok ? vb + (size_t)r * a.v_dim + ch * 8 : vb, ok);
    }
  };
  int page_cur = n_walk > 0 ? pt[tile_lo] : 0;
  if (n_walk > 0) {
    load_k(page_cur, 0);
    if (!SLICE) load_v(tile_lo, page_cur, 0);
  }
  cp_async_commit();
  int page_next = n_walk > 1 ? pt[tile_lo + stride] : 0;
  auto bias_of = [&](int tile, int x) {  // of distance (q_first - the tile's last key) + lane + 32 x, for this warp's head
    const int dist = q_first - (tile * SP_N + SP_N - 1) + lane + 32 * x;
    return a.rel[(size_t)min(max(dist, 0), a.n_rel - 1) * H + h];
  };
  float bias_next[3] = {0.f, 0.f, 0.f};
  if (a.rel && n_walk > 0) {
#pragma unroll
    for (int x = 0; x < 3; ++x) bias_next[x] = bias_of(tile_lo, x);
  }

  float o[NO][4];
#pragma unroll
  for (int j = 0; j < NO; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  int qpos[2], qlo[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = g4 + e * 8;
    qpos[e] = r < rows_here ? q_first + r : q_first;
    qlo[e] = a.window > 0 ? max(0, qpos[e] - a.window + 1) : 0;
  }
  float* my_a = s_a + hr * SP_M * SP_LD;
  float* my_w = s_w + hr * SP_M * SP_LD;
  float* my_bias = s_bias + warp * SP_BIAS;

  for (int u = 0; u < n_walk; ++u) {
    const int tile = tile_lo + u * stride, stage = u & 1;
    cp_async_wait<0>();
    __syncthreads();  // this page is here; everybody is done with the other stage and with the mixed weights
    if (SLICE) load_v(tile, page_cur, 0);  // everybody is done with the page before
    if (u + 1 < n_walk) {
      load_k(page_next, stage ^ 1);
      if (!SLICE) load_v(tile + stride, page_next, stage ^ 1);
      page_cur = page_next;
      if (u + 2 < n_walk) page_next = pt[tile + 2 * stride];
    }
    cp_async_commit();
    const int dist0 = q_first - (tile * SP_N + SP_N - 1);
    if (a.rel) {
#pragma unroll
      for (int x = 0; x < 3; ++x)
        if (lane + 32 * x < SP_BIAS) my_bias[lane + 32 * x] = bias_next[x];
      __syncwarp();
      if (u + 1 < n_walk) {
#pragma unroll
        for (int x = 0; x < 3; ++x) bias_next[x] = bias_of(tile + stride, x);
      }
    }
    // ---- scores of this warp's head and keys
    float s[NJ][4];
#pragma unroll
    for (int j = 0; j < NJ; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    const unsigned kb = s_k + stage * KTILE, vb = s_v + (SLICE ? 0 : stage * VTILE);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int j = 0; j < NJ; j += 2) {
        unsigned b0, b1, b2, b3;
        const int mi = lane >> 3, r = lane & 7;
        ldsm_x4(kb + sp_off<HD>((wq * NJ + j + (mi >> 1)) * 8 + r, ks * 2 + (mi & 1)), b0, b1, b2, b3);
        mma_bf16(s[j], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
        mma_bf16(s[j + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
      }
    }
    if (!SLICE && u > 0) sp_cluster_wait();  // every block has read the weights of the page before
    const int kbase = tile * SP_N;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float w2[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int kpos = kbase + (wq * NJ + j) * 8 + 2 * t4 + x;
          const bool ok = kpos <= qpos[e] && kpos >= qlo[e];
          float z = s[j][2 * e + x] * a.scale;
          if (a.rel && ok) z += my_bias[qpos[e] - kpos - dist0];
          w2[x] = ok ? __fdividef(1.0f, 1.0f + __expf(-z)) : 0.f;
        }
        *reinterpret_cast<float2*>(my_a + (g4 + e * 8) * SP_LD + (wq * NJ + j) * 8 + 2 * t4) = make_float2(w2[0], w2[1]);
      }
    }
    sp_cluster_arrive();
    sp_cluster_wait();  // all heads' weights of this page are written
    // ---- mixing: this warp's column groups, all heads in, this block's heads out
    if (SLICE) {
      // ---- mixing by keys: this block's 64 / G keys, all heads in, all heads out, four blocks' heads at a time
      const int KS = SP_N / G, P = SP_M * KS, n_dg = (G + 3) / 4;
      for (int it = tid; it < P * n_dg; it += n_threads) {
        const int pair = it % P, dg = it / P, row = pair / KS, k = pair % KS;
        float acc[4][RP];
#pragma unroll
        for (int d = 0; d < 4; ++d)
#pragma unroll
          for (int r = 0; r < RP; ++r) acc[d][r] = 0.f;
        const unsigned at = (unsigned)((row * SP_LD + c * KS + k) * 4);
        for (int cg = 0; cg < G; ++cg) {
          const unsigned base = sp_map(s_a_addr, (unsigned)cg) + at;
          float v[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) v[x] = sp_ld1(base + (unsigned)(min(x, R - 1) * SP_M * SP_LD * 4));
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            if (x < R) {
              const float* mrow = s_mix + ((cg * R + x) * G + dg * 4) * SP_MAX_R;  // the factors of heads beyond R are zeros
#pragma unroll
              for (int d = 0; d < 4; ++d) {
                float m[4];
                *reinterpret_cast<float4*>(m) = *reinterpret_cast<const float4*>(mrow + d * SP_MAX_R);
#pragma unroll
                for (int r = 0; r < RP; ++r) acc[d][r] = fmaf(m[r], v[x], acc[d][r]);
              }
            }
          }
        }
#pragma unroll
        for (int d = 0; d < 4; ++d)
#pragma unroll
          for (int r = 0; r < RP; ++r)
            if (dg * 4 + d < G && r < R) s_ws[(((dg * 4 + d) * R + r) * SP_M + row) * KS + k] = acc[d][r];
      }
      sp_cluster_arrive();
      sp_cluster_wait();  // all blocks' mixed weights of this page are written
      // ---- this block's heads' mixed weights of all keys, 16 bytes at a time
      for (int idx = tid; idx < R * SP_M * (SP_N / 4); idx += n_threads) {
        const int r = idx / (SP_M * (SP_N / 4)), rem = idx % (SP_M * (SP_N / 4)), row = rem / (SP_N / 4), key0 = (rem % (SP_N / 4)) * 4;
        const float4 v = sp_ld4(sp_map(s_ws_addr, (unsigned)(key0 / KS)) + (unsigned)(((((c * R + r) * SP_M + row) * KS) + key0 % KS) * 4));
        *reinterpret_cast<float4*>(s_w + (r * SP_M + row) * SP_LD + key0) = v;
      }
      cp_async_wait<0>();  // this page's values (and the next page's keys) are here
    }
    // a lane takes four neighbouring keys of one row: a 16 x 8 group of a head is one 16-byte read per lane
    for (int j = SLICE ? SP_N : warp; j < SP_N / 8; j += n_warps) {
      float acc[RP][4];
#pragma unroll
      for (int r = 0; r < RP; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
      const int at_f = (lane >> 1) * SP_LD + j * 8 + (lane & 1) * 4;
      const unsigned at = (unsigned)(at_f * 4);
      // up to four heads' weights of a block are asked for at a time, then mixed in
      for (int cg = 0; cg < a.n_kv_heads; ++cg) {
        const unsigned base = sp_map(s_a_addr, (unsigned)cg) + at;
        for (int rg0 = 0; rg0 < R; rg0 += 4) {
          float4 v[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) v[x] = sp_ld4(base + (unsigned)(min(rg0 + x, R - 1) * SP_M * SP_LD * 4));
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            if (rg0 + x < R) {
              // the factors of heads beyond R are zeros
              const float* mrow = s_mix + (cg * R + rg0 + x) * SP_MAX_R;
              float m[SP_MAX_R];
              *reinterpret_cast<float4*>(m) = *reinterpret_cast<const float4*>(mrow);
              if (RP > 4) *reinterpret_cast<float4*>(m + 4) = *reinterpret_cast<const float4*>(mrow + 4);
#pragma unroll
              for (int r = 0; r < RP; ++r) {
                acc[r][0] = fmaf(m[r], v[x].x, acc[r][0]);
                acc[r][1] = fmaf(m[r], v[x].y, acc[r][1]);
                acc[r][2] = fmaf(m[r], v[x].z, acc[r][2]);
                acc[r][3] = fmaf(m[r], v[x].w, acc[r][3]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RP; ++r)
        if (r < R) *reinterpret_cast<float4*>(s_w + r * SP_M * SP_LD + at_f) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
    if (!SLICE) sp_cluster_arrive();  // this block reads no other's weights of this page any more
    __syncthreads();                  // the mixed weights of all column groups are written
    // ---- O += W V, the weights as two bfloat16 terms
#pragma unroll
    for (int ks = 0; ks < SP_N / 16; ++ks) {
      const float2 w00 = *reinterpret_cast<const float2*>(my_w + g4 * SP_LD + ks * 16 + 2 * t4);
      const float2 w10 = *reinterpret_cast<const float2*>(my_w + (g4 + 8) * SP_LD + ks * 16 + 2 * t4);
      const float2 w01 = *reinterpret_cast<const float2*>(my_w + g4 * SP_LD + ks * 16 + 8 + 2 * t4);
      const float2 w11 = *reinterpret_cast<const float2*>(my_w + (g4 + 8) * SP_LD + ks * 16 + 8 + 2 * t4);
      const unsigned a0 = pack_bf16(w00.x, w00.y), a1 = pack_bf16(w10.x, w10.y), a2 = pack_bf16(w01.x, w01.y), a3 = pack_bf16(w11.x, w11.y);
      const unsigned r0 = pack_bf16(sp_rest(w00.x), sp_rest(w00.y)), r1 = pack_bf16(sp_rest(w10.x), sp_rest(w10.y));
      const unsigned r2 = pack_bf16(sp_rest(w01.x), sp_rest(w01.y)), r3 = pack_bf16(sp_rest(w11.x), sp_rest(w11.y));
#pragma unroll
      for (int j = 0; j < NO; j += 2) {
        unsigned b0, b1, b2, b3;
        const int mi = lane >> 3, r = lane & 7;
        ldsm_x4_trans(vb + sp_off<VD>(ks * 16 + (mi & 1) * 8 + r, wq * NO + j + (mi >> 1)), b0, b1, b2, b3);
        mma_bf16(o[j], a0, a1, a2, a3, b0, b1);
        mma_bf16(o[j + 1], a0, a1, a2, a3, b2, b3);
        mma_bf16(o[j], r0, r1, r2, r3, b0, b1);
        mma_bf16(o[j + 1], r0, r1, r2, r3, b2, b3);
      }
    }
  }
  if (SLICE && n_walk > 0) sp_cluster_arrive();
  if (n_walk > 0) sp_cluster_wait();  // no block leaves while another still reads its weights
  if (a.part) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int r = g4 + e * 8;
      if (r >= rows_here) continue;
      float* prow = a.part + ((size_t)(start + row0 + r) * a.n_splits + split) * H * a.v_dim + (size_t)h * a.v_dim;
#pragma unroll
      for (int j = 0; j < NO; ++j) {
        const int d = (wq * NO + j) * 8 + 2 * t4;
        if (d < a.v_dim) *reinterpret_cast<float2*>(prow + d) = make_float2(o[j][2 * e], o[j][2 * e + 1]);
      }
    }
    return;
  }

  // ---- gate and store
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = g4 + e * 8;
    if (r >= rows_here) continue;
    const size_t trow = (size_t)(start + row0 + r);
    __nv_bfloat16* orow = a.out + trow * a.out_stride + (size_t)h * a.v_dim;
    const __nv_bfloat16* grow = a.gate ? a.gate + trow * a.gate_stride : nullptr;
    float gh = 1.f;
    if (a.gate_mode == 1) gh = 1.0f / (1.0f + expf(-__bfloat162float(grow[h])));
#pragma unroll
    for (int j = 0; j < NO; ++j) {
      const int d = (wq * NO + j) * 8 + 2 * t4;
      if (d < a.v_dim) {
        float g0 = gh, g1 = gh;
        if (a.gate_mode == 2) {
          const float2 gz = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(grow + (size_t)h * a.v_dim + d));
          g0 = 1.0f / (1.0f + expf(-gz.x));
          g1 = 1.0f / (1.0f + expf(-gz.y));
        }
        *reinterpret_cast<__nv_bfloat162*>(orow + d) = __floats2bfloat162_rn(o[j][2 * e] * g0, o[j][2 * e + 1] * g1);
      }
    }
  }
}

// out[t][i] = gate * sum_z part[t][z][i]
__global__ void sigmoid_attention_sum_kernel(const float* __restrict__ part, int n_splits, int row, int v_dim,
                                             const __nv_bfloat16* __restrict__ gate, int gate_stride, int gate_mode,
                                             __nv_bfloat16* __restrict__ out, int out_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < row; i += blockDim.x) {
    float s = 0.f;
    for (int z = 0; z < n_splits; ++z) s += part[((size_t)t * n_splits + z) * row + i];
    if (gate_mode) s *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * gate_stride + (gate_mode == 1 ? i / v_dim : i)])));
    out[(size_t)t * out_stride + i] = __float2bfloat16_rn(s);
  }
}

// Warps per query head: so that a block has about eight warps (the kernel's WPH).
static int sp_wph(int R) { return R <= 2 ? 4 : (R <= 4 ? 2 : 1); }

// The mixing is dealt out by keys (the kernel's SLICE) where that moves fewer bytes between the blocks.
static bool sp_slice(int n_kv_heads, int R) { return (n_kv_heads == 4 || n_kv_heads == 8) && R <= 4; }

static size_t sp_smem_bytes(int hd, int vd, int n_heads, int n_kv_heads) {
  const int R = n_heads / n_kv_heads;
  const bool slice = sp_slice(n_kv_heads, R);
  return 2 * (size_t)SP_N * hd * 2 + (slice ? 1 : 2) * (size_t)SP_N * vd * 2 +
         ((size_t)2 * R * SP_M * SP_LD + (size_t)n_heads * SP_MAX_R * (slice ? n_kv_heads : 1) + (size_t)R * sp_wph(R) * SP_BIAS +
          (slice ? (size_t)n_heads * SP_M * (SP_N / n_kv_heads) : 0)) * sizeof(float);
}

template <int HD, int VD, int RP, bool SLICE>
static int sp_launch_w(const SpArgs& a, int n_tiles, cudaStream_t stream) {
  const int WPH = sp_wph(RP);
  const int R = a.n_heads / a.n_kv_heads;
  const size_t smem = sp_smem_bytes(HD, VD, a.n_heads, a.n_kv_heads);
  static size_t granted = 0;
  if (smem > granted) {
    cudaError_t e = cudaFuncSetAttribute(sigmoid_attention_prefill_kernel<HD, VD, RP, SLICE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    granted = smem;
  }
  // one cluster per 16 rows: the blocks of 64 rows of the step's list, four deep; or, with the pages dealt out,
  // one cluster per block of (at most 16) rows and share of the pages
  dim3 grid(a.n_kv_heads, n_tiles, a.part ? a.n_splits : 64 / SP_M);
  cudaError_t e = bn_launch_cluster(sigmoid_attention_prefill_kernel<HD, VD, RP, SLICE>, grid, dim3(32 * R * WPH), smem, stream,
                                    dim3(a.n_kv_heads, 1, 1), a);
  if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
  BN_CHECK_LAUNCH();
  return BN_OK;
}

template <int HD, int VD>
static int sp_launch(const SpArgs& a, int n_tiles, cudaStream_t stream) {
  const int R = a.n_heads / a.n_kv_heads;
  if (sp_slice(a.n_kv_heads, R)) {
    if (R == 1) return sp_launch_w<HD, VD, 1, true>(a, n_tiles, stream);
    if (R == 2) return sp_launch_w<HD, VD, 2, true>(a, n_tiles, stream);
    return sp_launch_w<HD, VD, 4, true>(a, n_tiles, stream);
  }
  if (R == 1) return sp_launch_w<HD, VD, 1, false>(a, n_tiles, stream);
  if (R == 2) return sp_launch_w<HD, VD, 2, false>(a, n_tiles, stream);
  if (R <= 4) return sp_launch_w<HD, VD, 4, false>(a, n_tiles, stream);
  return sp_launch_w<HD, VD, 8, false>(a, n_tiles, stream);
}

// Whether the sizes fit this kernel (1) or want the general one (0): bfloat16 rows in whole 16-element steps up
// to 128, up to 8 query heads per key/value head, up to 8 key/value heads (a portable cluster), and the shared
// memory of one block.
extern "C" int bn_sigmoid_attention_prefill_fits(int n_heads, int n_kv_heads, int head_dim, int v_dim) {
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || n_kv_heads > 8 || n_heads / n_kv_heads > SP_MAX_R) return 0;
  if (head_dim <= 0 || head_dim % 16 || head_dim > 128 || v_dim <= 0 || v_dim % 16 || v_dim > 128) return 0;
  return sp_smem_bytes(head_dim <= 64 ? 64 : 128, v_dim <= 64 ? 64 : 128, n_heads, n_kv_heads) <= 200 * 1024;
}

// q: [tokens, q_stride] bfloat16 (head h at element h * head_dim), out [tokens, out_stride] (head h at element
// h * v_dim).  tile_seq / tile_row0: for each block of 64 new-token rows its sequence and first row; seq_start
// [n_seqs + 1]: first packed row of each sequence; seq_pos0: its length before the step.  rel [n_rel, n_heads]
// float32 by distance (the last row for every longer one) or null; mix [n_heads, n_heads] float32 or null;
// gate_mode 0 none, 1 one number per head, 2 one per output number (logistic function applied here).
// n_splits > 1 (every listed block of rows then holds at most 16 rows, tile_row0 may be null for rows from 0 on):
// the pages a block of rows sees are dealt out over so many clusters, whose float32 sums in part
// [n_tokens, n_splits, n_heads * v_dim] a second kernel adds up: for steps of few tokens behind long contexts.
extern "C" int bn_sigmoid_attention_prefill(const void* q, int q_stride, void* out, int out_stride, int n_tiles, int n_heads,
                                            int n_kv_heads, int head_dim, int v_dim, float scale, int window, const float* rel,
                                            int n_rel, const float* mix, const void* gate, int gate_stride, int gate_mode,
                                            const int* tile_seq, const int* tile_row0, const int* seq_start, const int* seq_pos0,
                                            const int* slots, const int* page_table, int pt_stride, const void* k_cache,
                                            const void* v_cache, float* part, int n_splits, int n_tokens, cudaStream_t stream) {
  if (n_tiles <= 0) return BN_OK;
  if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && (!part || n_tokens <= 0))) return BN_ERR_BAD_ARG;
  if (n_splits == 1) part = nullptr;
  if (!bn_sigmoid_attention_prefill_fits(n_heads, n_kv_heads, head_dim, v_dim) || n_tiles > 65535 || !q || !out || !k_cache || !v_cache ||
      window < 0 || (q_stride % 8) || (out_stride % 2) || (((uintptr_t)q) & 15) || (rel && n_rel <= 0) || gate_mode < 0 || gate_mode > 2 ||
      (gate_mode && (!gate || (gate_stride % 2) || (((uintptr_t)gate) & 3))))
    return BN_ERR_BAD_ARG;
  SpArgs a;
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride; a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
  a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.v_dim = v_dim; a.scale = scale; a.window = window;
  a.rel = rel; a.n_rel = n_rel; a.mix = mix; a.gate = gate_mode ? (const __nv_bfloat16*)gate : nullptr; a.gate_stride = gate_stride;
  a.gate_mode = gate_mode; a.tile_seq = tile_seq; a.tile_row0 = tile_row0; a.seq_start = seq_start; a.seq_pos0 = seq_pos0;
  a.slots = slots; a.page_table = page_table; a.pt_stride = pt_stride;
  a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
  a.part = part; a.n_splits = n_splits;
  const bool k64 = head_dim <= 64, v64 = v_dim <= 64;
  int rc;
  if (k64 && v64) rc = sp_launch<64, 64>(a, n_tiles, stream);
  else if (k64) rc = sp_launch<64, 128>(a, n_tiles, stream);
  else if (v64) rc = sp_launch<128, 64>(a, n_tiles, stream);
  else rc = sp_launch<128, 128>(a, n_tiles, stream);
  if (rc != BN_OK || !part) return rc;
  BN_LAUNCH(sigmoid_attention_sum_kernel, n_tokens, 256, 0, stream, (const float*)part, n_splits, n_heads * v_dim, v_dim, a.gate, gate_stride,
            gate_mode, a.out, out_stride);
  BN_CHECK_LAUNCH();
  return BN_OK;
}
