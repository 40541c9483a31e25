// A feed-forward of routed experts.
//
//   route    logits = Wr h + b in float32 (one warp per token); the ``top`` largest (the lower index wins a tie);
//            weights = softmax over the chosen logits; also sigmoid(Wsg h), the gate of a shared expert
//   sort     the (token, choice) pairs ordered by expert: for each expert the range of its pairs, for each pair its
//            place, and a table of row tiles (expert, first row, rows) for the grouped products
//   gate_up  act[place] = silu(Wg_e x) * (Wu_e x) for every pair, x = the pair's token        } grouped products:
//   down     y[place] = Wd_e act[place]                                    float32            } a tile = one expert
//   combine  out[t] = sum_k weight[t, k] y[place(t, k)] + gate[t] * shared[t]                  float32
//
// Nothing comes back to the host between these: counts, places and tiles stay on the device, so a step with
// routed experts is captured in a CUDA graph like any other.  The products run on float32 FMA with the
// weights in the engine's dtype; a tile's rows are pairs of one expert, its sums one FMA chain over k each.
#include "common.cuh"

#define MOE_MAX_TOP 32

// ----------------------------------------------------------------------------- route
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ h, const T* __restrict__ wr, const float* __restrict__ br,
                 const T* __restrict__ wsg, int n_tokens, int D, int E, int top, int* __restrict__ idx,
                 float* __restrict__ wt, float* __restrict__ sgate) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float lg[];                 // [warps][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n_tokens) return;
  float* my = lg + (size_t)warp * E;
  const T* x = h + (size_t)t * D;
  for (int e = 0; e < E; e++) {
    float acc = 0.f;
    for (int i = lane; i < D; i += 32) acc = fmaf(to_float(x[i]), to_float(wr[(size_t)e * D + i]), acc);
    acc = warp_sum(acc);
    if (lane == 0) my[e] = acc + br[e];
  }
  if (wsg) {
    float acc = 0.f;
    for (int i = lane; i < D; i += 32) acc = fmaf(to_float(x[i]), to_float(wsg[i]), acc);
    acc = warp_sum(acc);
    if (lane == 0) sgate[t] = 1.0f / (1.0f + expf(-acc));
  }
  __syncwarp();
  if (lane == 0) {
    float v[MOE_MAX_TOP];
    for (int k = 0; k < top; k++) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; e++) {
        float z = my[e];
        if (best < 0 || z > bv) { best = e; bv = z; }
      }
      idx[(size_t)t * top + k] = best;
      v[k] = bv;
      my[best] = -INFINITY;
    }
    float sum = 0.f;
    const float vmax = v[0];                      // the first chosen is the largest
    for (int k = 0; k < top; k++) { v[k] = expf(v[k] - vmax); sum += v[k]; }
    for (int k = 0; k < top; k++) wt[(size_t)t * top + k] = v[k] / sum;
  }
}

// ----------------------------------------------------------------------------- sort
// One CTA.  meta: [0, E] offsets (E + 1), then n_tiles, then tiles (expert, first row, rows) x max_tiles.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ idx, int n_pairs, int E, int tile_rows, int max_tiles, int* __restrict__ place,
                int* __restrict__ pair_at, int* __restrict__ meta) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int cnt[];                  // [E] counts, then [E] cursors
  int* cur = cnt + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&cnt[idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    int* tiles = meta + E + 2;
    for (int e = 0; e < E; e++) {
      meta[e] = off;
      cur[e] = off;
      for (int r0 = 0; r0 < cnt[e] && nt < max_tiles; r0 += tile_rows) {
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = off + r0;
        tiles[3 * nt + 2] = min(tile_rows, cnt[e] - r0);
        nt++;
      }
      off += cnt[e];
    }
    meta[E] = off;
    meta[E + 1] = nt;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    int at = atomicAdd(&cur[idx[p]], 1);
    place[p] = at;
    pair_at[at] = p;
  }
}

// ----------------------------------------------------------------------------- grouped products
// Tile of TM rows x 64 columns; 256 threads, each (TM / 16) x 4 outputs.  GATED: two weight matrices and the
// SwiGLU of their sums.  Rows of A: the pair's token (``pair_at[row] / top``) when ``by_token``, else the row itself.
template <typename TI, typename TW, typename TO, int TM, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TI* __restrict__ A, long long lda, const int* __restrict__ pair_at, int top, int by_token,
                const TW* __restrict__ W1, const TW* __restrict__ W2, TO* __restrict__ out, int N, int K,
                const int* __restrict__ meta, int E) {
  pdl_launch_dependents();
  pdl_wait();
  const int n_tiles = meta[E + 1];
  if ((int)blockIdx.y >= n_tiles) return;
  const int* tile = meta + E + 2 + 3 * blockIdx.y;
  const int e = tile[0], row0 = tile[1], rows = tile[2];
  constexpr int RPT = TM / 16;                  // rows per thread
  __shared__ float As[16][TM + 4];
  __shared__ float B1[16][64 + 4];
  __shared__ float B2[GATED ? 16 : 1][64 + 4];
  __shared__ int src[TM];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int n0 = blockIdx.x * 64;
  if (tid < TM) {
    int r = row0 + tid;
    src[tid] = tid < rows ? (by_token ? pair_at[r] / top : r) : -1;
  }
  __syncthreads();
  const TW* w1 = W1 + (size_t)e * N * K;
  const TW* w2 = GATED ? W2 + (size_t)e * N * K : nullptr;
  float acc1[RPT][4], acc2[RPT][4];
#pragma unroll
  for (int i = 0; i < RPT; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc1[i][j] = acc2[i][j] = 0.f;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int gk = k0 + lk + j, gn = n0 + lr;
      if (lr < TM) As[lk + j][lr] = (src[lr] >= 0 && gk < K) ? to_float(A[(size_t)src[lr] * lda + gk]) : 0.f;
      B1[lk + j][lr] = (gn < N && gk < K) ? to_float(w1[(size_t)gn * K + gk]) : 0.f;
      if (GATED) B2[lk + j][lr] = (gn < N && gk < K) ? to_float(w2[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; kk++) {
      float a[RPT], b1[4], b2[4];
#pragma unroll
      for (int i = 0; i < RPT; i++) a[i] = As[kk][ty * RPT + i];
#pragma unroll
      for (int j = 0; j < 4; j++) { b1[j] = B1[kk][tx * 4 + j]; b2[j] = GATED ? B2[kk][tx * 4 + j] : 0.f; }
#pragma unroll
      for (int i = 0; i < RPT; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
          acc1[i][j] = fmaf(a[i], b1[j], acc1[i][j]);
          if (GATED) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RPT; i++) {
    int r = ty * RPT + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc1[i][j];
      if (GATED) v = v / (1.0f + expf(-v)) * acc2[i][j];
      out[(size_t)(row0 + r) * N + gn] = from_float<TO>(v);
    }
  }
}

// ----------------------------------------------------------------------------- combine
// out[t, :] = sum_k wt[t, k] * y[place[t * top + k], :] + sgate[t] * sum_p shared[p, t, :]   (float32 out)
template <typename TS>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ wt, int top,
                   const TS* __restrict__ shared, int n_parts, size_t part_stride, const float* __restrict__ sgate,
                   float* __restrict__ out, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; k++)
      acc = fmaf(wt[(size_t)t * top + k], y[(size_t)place[(size_t)t * top + k] * D + i], acc);
    if (shared) {
      float s = to_float(shared[(size_t)t * D + i]);
      for (int p = 1; p < n_parts; p++) s += to_float(shared[p * part_stride + (size_t)t * D + i]);
      acc = fmaf(sgate[t], s, acc);
    }
    out[(size_t)t * D + i] = acc;
  }
}

// ----------------------------------------------------------------------------- launchers
extern "C" int qd_moe_route(const void* h, const void* wr, const float* br, const void* wsg, int dtype, int T, int D,
                            int E, int top, int* idx, float* wt, float* sgate, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top < 1 || top > E || top > MOE_MAX_TOP || E > 2048) return QD_ERR_UNSUPPORTED;
  size_t smem = (size_t)4 * E * sizeof(float);
  dim3 grid((T + 3) / 4);
  if (dtype == QD_F32)
    qd_launch(moe_route_kernel<float>, grid, dim3(128), smem, stream, (const float*)h, (const float*)wr, br,
              (const float*)wsg, T, D, E, top, idx, wt, sgate);
  else if (dtype == QD_BF16)
    qd_launch(moe_route_kernel<bf16>, grid, dim3(128), smem, stream, (const bf16*)h, (const bf16*)wr, br,
              (const bf16*)wsg, T, D, E, top, idx, wt, sgate);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

extern "C" int qd_moe_sort(const int* idx, int n_pairs, int E, int tile_rows, int max_tiles, int* place, int* pair_at,
                           int* meta, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (E > 4096) return QD_ERR_UNSUPPORTED;
  qd_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, idx, n_pairs, E, tile_rows,
            max_tiles, place, pair_at, meta);
  return qd_last_error();
}

// gated != 0: out[place, N] = silu(A W1_e^T) * (A W2_e^T) in ``out_dtype``; else out = A W1_e^T.
extern "C" int qd_moe_gemm(const void* A, long long lda, int a_dtype, const int* pair_at, int top, int by_token,
                           const void* W1, const void* W2, int w_dtype, void* out, int out_dtype, int N, int K,
                           const int* meta, int E, int tile_rows, int max_tiles, int gated, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (max_tiles > 65535 || (tile_rows != 16 && tile_rows != 64)) return QD_ERR_UNSUPPORTED;
  dim3 grid((N + 63) / 64, max_tiles);
#define MOE_GO(TI, TW, TO, TM, G)                                                                                   \
  qd_launch(moe_gemm_kernel<TI, TW, TO, TM, G>, grid, dim3(256), 0, stream, (const TI*)A, lda, pair_at, top, by_token, \
            (const TW*)W1, (const TW*)W2, (TO*)out, N, K, meta, E)
#define MOE_PICK(TI, TW, TO)                                                     \
  do {                                                                           \
    if (tile_rows == 16) { if (gated) MOE_GO(TI, TW, TO, 16, true); else MOE_GO(TI, TW, TO, 16, false); } \
    else { if (gated) MOE_GO(TI, TW, TO, 64, true); else MOE_GO(TI, TW, TO, 64, false); }                 \
  } while (0)
  if (a_dtype == QD_F32 && w_dtype == QD_F32 && out_dtype == QD_F32) MOE_PICK(float, float, float);
  else if (a_dtype == QD_BF16 && w_dtype == QD_BF16 && out_dtype == QD_BF16) MOE_PICK(bf16, bf16, bf16);
  else if (a_dtype == QD_BF16 && w_dtype == QD_BF16 && out_dtype == QD_F32) MOE_PICK(bf16, bf16, float);
  else return QD_ERR_UNSUPPORTED;
#undef MOE_PICK
#undef MOE_GO
  return qd_last_error();
}

extern "C" int qd_moe_combine(const float* y, const int* place, const float* wt, int top, const void* shared,
                              int shared_dtype, int n_parts, long long part_stride, const float* sgate, float* out,
                              int T, int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (shared && shared_dtype == QD_BF16 && n_parts == 1)
    qd_launch(moe_combine_kernel<bf16>, dim3(T), dim3(256), 0, stream, y, place, wt, top, (const bf16*)shared, 1,
              (size_t)0, sgate, out, D);
  else if (!shared || shared_dtype == QD_F32)
    qd_launch(moe_combine_kernel<float>, dim3(T), dim3(256), 0, stream, y, place, wt, top, (const float*)shared,
              n_parts, (size_t)part_stride, sgate, out, D);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}
