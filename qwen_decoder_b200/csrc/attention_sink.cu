// Grouped-query attention whose softmax has a sink, whose values may have another size than its keys, and whose
// queries and keys are unit-normalised per head before they turn:
//
//   prep      per token: q_h <- unit(q_h) * wq, k_g <- unit(k_g) * wk (unit(y) = y / sqrt(mean(y^2) + eps), over the
//             head; skipped without weights), the first ``rotary_dim`` elements of each turn by the token's
//             position (table rows of cos and sin), v_g <- (1 - lam) v_g + lam v0_g when a source of earlier values
//             is given; q goes to a dense [T, H * d] tensor, k and v to the token's slot of the paged cache
//   attend    p_j = exp(s_j) / (sum_j exp(s_j) + exp(sink_h)) over the keys j <= position (or the last ``window``),
//             s_j = (q . k_j) * scale; the sink has no key and no value.  One warp per (token, head), float32
//             arithmetic, any sizes; tiles of 32 keys counted from key 0, so the order of every sum depends on the
//             token's position only
//
// A page of the cache holds the keys [G, page_size, d] and then the values [G, page_size, vd].
#include "common.cuh"
#include <math.h>

#define AS_MAX_D 512
#define AS_WARPS 4

__device__ __forceinline__ float as_ld(const void* p, int code, size_t i) {
  return code == QD_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}
__device__ __forceinline__ void as_st(void* p, int code, size_t i, float v) {
  if (code == QD_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------------------------------------------------- prep
// One warp per (token, slot): slots 0..H-1 the query heads, H..H+G-1 the key heads, H+G..H+2G-1 the value heads.
// qkv [T, ld]: row = [q (H*d) | k (G*d) | v (G*vd)].
__global__ void __launch_bounds__(AS_WARPS * 32)
qk_norm_rope_write_kernel(const void* __restrict__ qkv, int in_dtype, long long ld, int T, int H, int G, int d, int vd,
                          const float* __restrict__ wq, const float* __restrict__ wk, float eps, int rotary_dim,
                          int pairing, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                          const int* __restrict__ positions, void* __restrict__ q_out, int q_dtype,
                          void* __restrict__ kv, int kv_dtype, const int* __restrict__ slot_map, int page_size,
                          int write_kv, const void* __restrict__ v0, long long v0_ld, const float* __restrict__ lam_p) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = H + 2 * G;
  const long long item = (long long)blockIdx.x * AS_WARPS + warp;
  if (item >= (long long)T * slots) return;
  const int t = (int)(item / slots), s = (int)(item - (long long)t * slots);
  const size_t row = (size_t)t * ld;
  const size_t page_elems = (size_t)G * page_size * (d + vd);
  size_t slot = 0, page = 0, off = 0;
  if (s >= H) {
    if (!write_kv) return;
    slot = (size_t)slot_map[t];
    page = slot / page_size;
    off = slot - page * page_size;
  }
  if (s >= H + G) {                                   // a value head
    const int g = s - H - G;
    const size_t src = row + (size_t)H * d + (size_t)G * d + (size_t)g * vd;
    const size_t dst = page * page_elems + (size_t)G * page_size * d + ((size_t)g * page_size + off) * vd;
    const float lam = v0 ? *lam_p : 0.f;
    for (int i = lane; i < vd; i += 32) {
      float v = as_ld(qkv, in_dtype, src + i);
      if (v0) v = (1.0f - lam) * v + lam * as_ld(v0, in_dtype, (size_t)t * v0_ld + (size_t)g * vd + i);
      as_st(kv, kv_dtype, dst + i, v);
    }
    return;
  }
  const bool is_q = s < H;
  const size_t src = row + (is_q ? (size_t)s * d : (size_t)H * d + (size_t)(s - H) * d);
  const float* w = is_q ? wq : wk;
  // pairs (a, b) of the head: pair j = lane + 32 * i holds elements (2j, 2j+1) when the pairing is adjacent, and
  // (j, j + rotary_dim / 2) within the rotated part when it is half-split (elements past the rotated part: adjacent)
  float a[AS_MAX_D / 64], b[AS_MAX_D / 64];
  int ia[AS_MAX_D / 64], ib[AS_MAX_D / 64];
  const int half = rotary_dim / 2, pairs = d / 2;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 64; i++) {
    const int j = lane + 32 * i;
    a[i] = b[i] = 0.f;
    ia[i] = ib[i] = -1;
    if (j < pairs) {
      if (pairing == 1 && j < half) { ia[i] = j; ib[i] = j + half; }
      else { ia[i] = 2 * j; ib[i] = 2 * j + 1; }
      a[i] = as_ld(qkv, in_dtype, src + ia[i]);
      b[i] = as_ld(qkv, in_dtype, src + ib[i]);
      ss = fmaf(a[i], a[i], fmaf(b[i], b[i], ss));
    }
  }
  float last = 0.f;                                   // an odd head size leaves one element without a partner
  if ((d & 1) && lane == 0) { last = as_ld(qkv, in_dtype, src + d - 1); ss = fmaf(last, last, ss); }
  float f = 1.f;
  if (w) f = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
  const int pos = positions[t];
  const size_t dst = is_q ? (size_t)t * H * d + (size_t)s * d
                          : page * page_elems + ((size_t)(s - H) * page_size + off) * d;
  void* out = is_q ? q_out : kv;
  const int oc = is_q ? q_dtype : kv_dtype;
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 64; i++) {
    const int j = lane + 32 * i;
    if (j >= pairs) continue;
    float x = a[i] * f, y = b[i] * f;
    if (w) { x *= w[ia[i]]; y *= w[ib[i]]; }
    if (j < half) {
      const float c = cos_t[(size_t)pos * half + j], sn = sin_t[(size_t)pos * half + j];
      const float xr = x * c - y * sn, yr = y * c + x * sn;
      x = xr; y = yr;
    }
    as_st(out, oc, dst + ia[i], x);
    as_st(out, oc, dst + ib[i], y);
  }
  if ((d & 1) && lane == 0) as_st(out, oc, dst + d - 1, w ? last * f * w[d - 1] : last);
}

extern "C" int qd_qk_norm_rope_write(const void* qkv, int in_dtype, long long ld, int T, int H, int G, int d, int vd,
                                     const float* wq, const float* wk, float eps, int rotary_dim, int pairing,
                                     const float* cos_t, const float* sin_t, const int* positions, void* q_out,
                                     int q_dtype, void* kv, int kv_dtype, const int* slot_map, int page_size,
                                     int write_kv, const void* v0, long long v0_ld, const float* lam,
                                     cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d <= 0 || d > AS_MAX_D || vd <= 0 || rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || (!wq) != (!wk))
    return QD_ERR_UNSUPPORTED;
  if (pairing == 1 && (d & 1)) return QD_ERR_UNSUPPORTED;
  const long long items = (long long)T * (H + 2 * G);
  qd_launch(qk_norm_rope_write_kernel, dim3((unsigned)((items + AS_WARPS - 1) / AS_WARPS)), dim3(AS_WARPS * 32), 0,
            stream, qkv, in_dtype, ld, T, H, G, d, vd, wq, wk, eps, rotary_dim, pairing, cos_t, sin_t, positions, q_out,
            q_dtype, kv, kv_dtype, slot_map, page_size, write_kv, v0, v0_ld, lam);
  return qd_last_error();
}

// ----------------------------------------------------------------------------------------------------------- attend
template <typename T>
__global__ void __launch_bounds__(AS_WARPS * 32)
sink_attention_generic_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                              const T* __restrict__ kv, const int* __restrict__ block_table, int max_blocks,
                              const int* __restrict__ token_req, const int* __restrict__ positions, int n_tokens,
                              int H, int G, int d, int vd, int page_size, float scale, int window,
                              const float* __restrict__ sinks) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * AS_WARPS + warp;
  if (item >= (long long)n_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item - (long long)t * H);
  const int g = h / (H / G);
  float* qs = smem + (size_t)warp * d;
  const T* qr = q + (size_t)t * q_stride + (size_t)h * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_float(qr[i]);
  __syncwarp();

  const int pos = positions[t];
  const int* bt = block_table + (size_t)token_req[t] * max_blocks;
  const int key_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const size_t page_elems = (size_t)G * page_size * (d + vd);
  const size_t k_head = (size_t)g * page_size * d;
  const size_t v_head = (size_t)G * page_size * d + (size_t)g * page_size * vd;

  float m = -INFINITY, l = 0.0f;
  float o[AS_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 32; i++) o[i] = 0.0f;

  for (int base = key_lo & ~31; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key >= key_lo && key <= pos;
    float s = -INFINITY;
    if (valid) {
      const int page = bt[key / page_size];
      const T* kr = kv + (size_t)page * page_elems + k_head + (size_t)(key % page_size) * d;
      float acc = 0.0f;
      for (int i = 0; i < d; i++) acc = fmaf(qs[i], to_float(kr[i]), acc);
      s = acc * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float c = expf(m - m_new);  // m = -inf on the first tile gives 0
    const float p = valid ? expf(s - m_new) : 0.0f;
    l = l * c + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < AS_MAX_D / 32; i++) o[i] *= c;
    const int jend = pos - base + 1 < 32 ? pos - base + 1 : 32;
    for (int j = 0; j < jend; j++) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = base + j;
      if (kj < key_lo) continue;
      const int page = bt[kj / page_size];
      const T* vr = kv + (size_t)page * page_elems + v_head + (size_t)(kj % page_size) * vd;
#pragma unroll
      for (int i = 0; i < AS_MAX_D / 32; i++) {
        const int idx = lane + 32 * i;
        if (idx < vd) o[i] = fmaf(pj, to_float(vr[idx]), o[i]);
      }
    }
  }
  if (sinks) {                                        // the sink joins the denominator once, unscaled
    const float sk = sinks[h];
    const float m_new = fmaxf(m, sk);
    const float c = expf(m - m_new);
    l = l * c + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < AS_MAX_D / 32; i++) o[i] *= c;
  }
  T* orow = out + (size_t)t * out_stride + (size_t)h * vd;
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 32; i++) {
    const int idx = lane + 32 * i;
    if (idx < vd) orow[idx] = from_float<T>(o[i] * inv);
  }
}

// q: first query element, rows q_stride elements apart, head h at h * d; out [n_tokens, H * vd] rows out_stride apart;
// kv: pages of [G, page_size, d] keys then [G, page_size, vd] values; sinks float32 [H] or null.
extern "C" int qd_sink_attention_generic(const void* q, long long q_stride, void* out, long long out_stride,
                                         const void* kv, int dtype, const int* block_table, int max_blocks,
                                         const int* token_req, const int* positions, int n_tokens, int H, int G, int d,
                                         int vd, int page_size, float scale, int window, const float* sinks,
                                         cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || d > AS_MAX_D || vd <= 0 || vd > AS_MAX_D || G <= 0 || H % G != 0 || page_size <= 0)
    return QD_ERR_UNSUPPORTED;
  const long long items = (long long)n_tokens * H;
  const unsigned blocks = (unsigned)((items + AS_WARPS - 1) / AS_WARPS);
  const size_t smem = (size_t)AS_WARPS * d * sizeof(float);
  if (dtype == QD_F32)
    qd_launch(sink_attention_generic_kernel<float>, dim3(blocks), dim3(AS_WARPS * 32), smem, stream, (const float*)q,
              q_stride, (float*)out, out_stride, (const float*)kv, block_table, max_blocks, token_req, positions,
              n_tokens, H, G, d, vd, page_size, scale, window, sinks);
  else if (dtype == QD_BF16)
    qd_launch(sink_attention_generic_kernel<bf16>, dim3(blocks), dim3(AS_WARPS * 32), smem, stream, (const bf16*)q,
              q_stride, (bf16*)out, out_stride, (const bf16*)kv, block_table, max_blocks, token_req, positions,
              n_tokens, H, G, d, vd, page_size, scale, window, sinks);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}
