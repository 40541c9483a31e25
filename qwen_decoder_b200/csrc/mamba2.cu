// The selective state-space mixer (Mamba-2 form): a short causal convolution with its activation, the
// recurrence over a per-head state, and the gated grouped norm of its output.
//
//   conv      xbc[t, c] = silu(b_c + sum_k w[c, k] in[t - (taps-1) + k, c]); inputs before the step's first token come
//             from the request's state (the last taps-1 inputs), which conv_state then moves on
//   scan      per request and head, token after token:
//               dt = softplus(dt_raw + dt_bias); a = exp(-exp(A_log) dt); S <- a S + dt B x^T; y = S^T C + D x
//             S [P, N] float32 lives in the request's state slot (N contiguous); a CTA owns some of the P value
//             columns of one (request, head) -- columns never mix -- and a thread keeps a slice of N in registers
//   gate_norm out = (y silu(z)) / rms over each of ``groups`` equal parts * w
//
// Everything here is float32 (inputs arrive as the float32 result of the input projection); only the
// gated, normed output takes the engine's dtype for the output projection.  A request's portion may be of
// any length and start anywhere: the same kernels serve prompts, portions and single decoded tokens.
#include "common.cuh"

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ----------------------------------------------------------------------------- convolution
// u [T, ldu] float32, channels at column x_off; state row of request slot s: conv part at conv_off, laid out
// [taps - 1][C] (oldest first).  One thread per (token, channel).
__global__ void __launch_bounds__(256)
mamba_conv_kernel(const float* __restrict__ u, long long ldu, int x_off, int C, int taps, const float* __restrict__ w,
                  const float* __restrict__ bias, const float* __restrict__ state, long long state_stride,
                  long long conv_off, const int* __restrict__ token_req, const int* __restrict__ cu_tokens,
                  const int* __restrict__ slots, float* __restrict__ xbc, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x, t = blockIdx.x;
  if (c >= C) return;
  const int rq = token_req[t], first = cu_tokens[rq];
  const int i = t - first;                                     // place within the request's portion
  const float* st = state + (size_t)slots[rq] * state_stride + conv_off;
  float acc = bias[c];
  for (int k = 0; k < taps; k++) {
    int src = i - (taps - 1) + k;                              // place of the tap's input; negative: before the portion
    float v = src >= 0 ? u[(size_t)(first + src) * ldu + x_off + c] : st[(size_t)(taps - 1 + src) * C + c];
    acc = fmaf(w[(size_t)c * taps + k], v, acc);
  }
  xbc[(size_t)t * C + c] = silu_f(acc);
}

// The state after a portion of n tokens: the last taps - 1 of (old state ++ the portion's inputs).  One thread per
// (request, channel); a thread reads an old entry before it overwrites a lower one.
__global__ void __launch_bounds__(256)
mamba_conv_state_kernel(const float* __restrict__ u, long long ldu, int x_off, int C, int taps,
                        float* __restrict__ state, long long state_stride, long long conv_off,
                        const int* __restrict__ cu_tokens, const int* __restrict__ slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, rq = blockIdx.y;
  if (c >= C) return;
  const int first = cu_tokens[rq], n = cu_tokens[rq + 1] - first;
  float* st = state + (size_t)slots[rq] * state_stride + conv_off;
  for (int j = 0; j < taps - 1; j++) {
    int src = n - (taps - 1) + j;                              // place in the portion; negative: still the old state
    st[(size_t)j * C + c] = src >= 0 ? u[(size_t)(first + src) * ldu + x_off + c] : st[(size_t)(j + n) * C + c];
  }
}

// ----------------------------------------------------------------------------- recurrence
#define MS_THREADS 256
#define MS_TOKENS 16        // tokens staged per round

// grid (ceil(P / PB), heads, requests); PB = MS_THREADS / NS value columns a CTA; thread (pl, ns): column p0 + pl,
// state elements n = ns + NS * j, j < SPT.  xbc row: [x (heads * P) | B (G * N) | C (G * N)].
template <int SPT>
__global__ void __launch_bounds__(MS_THREADS)
mamba_scan_kernel(const float* __restrict__ xbc, int Cw, const float* __restrict__ u, long long ldu, int dt_off,
                  const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dp,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ cu_tokens,
                  const int* __restrict__ slots, float* __restrict__ y, int nh, int P, int N, int G, int NS,
                  int write_state) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int PB = MS_THREADS / NS;
  float* Bs = sm;                                // [MS_TOKENS][N]
  float* Cs = Bs + MS_TOKENS * N;                // [MS_TOKENS][N]
  float* xs = Cs + MS_TOKENS * N;                // [MS_TOKENS][PB]
  float* dts = xs + MS_TOKENS * PB;              // [MS_TOKENS] step sizes
  float* as = dts + MS_TOKENS;                   // [MS_TOKENS] decays
  const int hd = blockIdx.y, rq = blockIdx.z, p0 = blockIdx.x * PB;
  const int ns = threadIdx.x % NS, pl = threadIdx.x / NS;
  const int p = p0 + pl;
  const int g = hd / (nh / G);
  const int first = cu_tokens[rq], n_tok = cu_tokens[rq + 1] - first;
  const int inner = nh * P;
  float* S = state + (size_t)slots[rq] * state_stride + ((size_t)hd * P + (p < P ? p : 0)) * N;
  float s[SPT];
#pragma unroll
  for (int j = 0; j < SPT; j++) {
    int n = ns + NS * j;
    s[j] = (p < P && n < N) ? S[n] : 0.f;
  }
  const float negA = -expf(A_log[hd]), Dh = Dp[hd], bias = dt_bias[hd];
  for (int t0 = 0; t0 < n_tok; t0 += MS_TOKENS) {
    const int nt = min(MS_TOKENS, n_tok - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * N; i += MS_THREADS) {
      int tt = i / N, n = i - tt * N;
      const float* row = xbc + (size_t)(first + t0 + tt) * Cw;
      Bs[tt * N + n] = row[inner + g * N + n];
      Cs[tt * N + n] = row[inner + G * N + g * N + n];
    }
    for (int i = threadIdx.x; i < nt * PB; i += MS_THREADS) {
      int tt = i / PB, q = i - tt * PB;
      xs[tt * PB + q] = p0 + q < P ? xbc[(size_t)(first + t0 + tt) * Cw + (size_t)hd * P + p0 + q] : 0.f;
    }
    if (threadIdx.x < nt) {
      float dt = softplus_f(u[(size_t)(first + t0 + threadIdx.x) * ldu + dt_off + hd] + bias);
      dts[threadIdx.x] = dt;
      as[threadIdx.x] = expf(negA * dt);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; tt++) {
      const float a = as[tt], xv = xs[tt * PB + pl], dx = dts[tt] * xv;
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < SPT; j++) {
        int n = ns + NS * j;
        if (n < N) {
          s[j] = fmaf(a, s[j], dx * Bs[tt * N + n]);
          acc = fmaf(s[j], Cs[tt * N + n], acc);
        }
      }
      for (int o = NS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (ns == 0 && p < P) y[(size_t)(first + t0 + tt) * inner + (size_t)hd * P + p] = fmaf(Dh, xv, acc);
    }
  }
  if (p < P && write_state) {
#pragma unroll
    for (int j = 0; j < SPT; j++) {
      int n = ns + NS * j;
      if (n < N) S[n] = s[j];
    }
  }
}

// ----------------------------------------------------------------------------- gate and grouped norm
// grid (tokens, groups): out[t, part] = v / sqrt(mean(v^2) + eps) * w with v = y * silu(z); z at column z_off of u.
template <typename TO>
__global__ void __launch_bounds__(256)
mamba_gate_norm_kernel(const float* __restrict__ y, const float* __restrict__ u, long long ldu, int z_off,
                       const float* __restrict__ w, TO* __restrict__ out, int inner, int groups, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[40];
  const int t = blockIdx.x, part = inner / groups, lo = blockIdx.y * part;
  float ss = 0.f;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    float v = y[(size_t)t * inner + lo + i] * silu_f(u[(size_t)t * ldu + z_off + lo + i]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)part + eps);
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    float v = y[(size_t)t * inner + lo + i] * silu_f(u[(size_t)t * ldu + z_off + lo + i]);
    out[(size_t)t * inner + lo + i] = from_float<TO>(v * inv * w[lo + i]);
  }
}

// ----------------------------------------------------------------------------- launchers
extern "C" int qd_mamba_conv(const float* u, long long ldu, int x_off, int C, int taps, const float* w,
                             const float* bias, float* state, long long state_stride, long long conv_off,
                             const int* token_req, const int* cu_tokens, const int* slots, float* xbc, int T, int R,
                             int update_state, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps < 1 || C > 65535 * 256 || R > 65535) return QD_ERR_UNSUPPORTED;
  dim3 grid(T, (C + 255) / 256);
  qd_launch(mamba_conv_kernel, grid, dim3(256), 0, stream, u, ldu, x_off, C, taps, w, bias, (const float*)state,
            state_stride, conv_off, token_req, cu_tokens, slots, xbc, T);
  if (update_state && taps > 1)
    qd_launch(mamba_conv_state_kernel, dim3((C + 255) / 256, R), dim3(256), 0, stream, u, ldu, x_off, C, taps, state,
              state_stride, conv_off, cu_tokens, slots);
  return qd_last_error();
}

extern "C" int qd_mamba_scan(const float* xbc, int Cw, const float* u, long long ldu, int dt_off, const float* dt_bias,
                             const float* A_log, const float* Dp, float* state, long long state_stride,
                             const int* cu_tokens, const int* slots, float* y, int R, int nh, int P, int N, int G,
                             int write_state, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (N <= 0 || N > 512 || nh % G || nh > 65535 || R > 65535) return QD_ERR_UNSUPPORTED;
  int NS = 1;                                     // lanes that share a value column: a power of two, at most 32
  while (NS < 32 && (N + NS - 1) / NS > 8) NS *= 2;
  const int spt = (N + NS - 1) / NS;              // up to 8, or up to 16 for N above 256
  const int PB = MS_THREADS / NS;
  dim3 grid((P + PB - 1) / PB, nh, R);
  size_t smem = ((size_t)MS_TOKENS * (2 * N + PB + 2)) * sizeof(float);
#define MS_GO(SPT)                                                                                                   \
  qd_launch(mamba_scan_kernel<SPT>, grid, dim3(MS_THREADS), smem, stream, xbc, Cw, u, ldu, dt_off, dt_bias, A_log, Dp, \
            state, state_stride, cu_tokens, slots, y, nh, P, N, G, NS, write_state)
  if (spt <= 4) MS_GO(4);
  else if (spt <= 8) MS_GO(8);
  else MS_GO(16);
#undef MS_GO
  return qd_last_error();
}

extern "C" int qd_mamba_gate_norm(const float* y, const float* u, long long ldu, int z_off, const float* w, void* out,
                                  int out_dtype, int T, int inner, int groups, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (groups < 1 || groups > 65535 || inner % groups) return QD_ERR_UNSUPPORTED;
  dim3 grid(T, groups);
  if (out_dtype == QD_F32)
    qd_launch(mamba_gate_norm_kernel<float>, grid, dim3(256), 0, stream, y, u, ldu, z_off, w, (float*)out, inner,
              groups, eps);
  else if (out_dtype == QD_BF16)
    qd_launch(mamba_gate_norm_kernel<bf16>, grid, dim3(256), 0, stream, y, u, ldu, z_off, w, (bf16*)out, inner, groups,
              eps);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}
