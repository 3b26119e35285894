// Kernels of the mixers that carry a state of fixed size from token to token instead of (or beside)
// cached keys and values: a short causal convolution per channel, the selective state-space scan
// (S <- exp(dt A) S + dt x B, y = S C + D x), and a matrix recurrence per head
// (S <- diag(a) S + b v^T, o = S^T q) that serves both gated linear attention (a = f, b = 1 - f) and a
// matrix memory with exponential gates held stable by a running maximum (a = scalar keep, b = take * k).
//
// The flat batch holds prompt portions of any length beside single tokens.  Request r owns the rows
// cu_q[r] .. cu_q[r+1]-1; its state lives in row state_slots[r] of each state tensor, is read at the
// start of the step and written back at its end, so a prompt may be cut anywhere.  States, decays,
// gates, step sizes and every sum over a state are fp32 whatever the activations' type; the order of
// the sums depends on nothing but the sizes of the model.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// --------------------------------------------------------------- causal convolution + SiLU
// out[i, c] = silu(bias[c] + sum_j w[c, taps-1-j] * x[i-j, c]) over the request's own earlier tokens;
// what lies before this step's first token comes from conv_state[slot, taps-1, channels] (the last
// taps-1 inputs of the request, oldest first; zero for a new request).  The state itself is brought
// up to date by the scan kernel that follows.
constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(256)
conv_silu_kernel(const T* __restrict__ x, int64_t x_stride, const float* __restrict__ w, const float* __restrict__ bias,
                 const float* __restrict__ conv_state, const int* __restrict__ positions,
                 const int* __restrict__ token_row, T* __restrict__ out, int n_tokens, int channels, int taps) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int i = blockIdx.x;
  if (c >= channels) return;
  const int row = token_row[i], pos = positions[i];
  float acc = bias ? bias[c] : 0.f;
  int j0 = -1;   // first distance at which the batch no longer holds the request's token
  for (int j = 0; j < taps; ++j) {
    float v = 0.f;
    if (j0 < 0) {
      const int k = i - j;
      const bool here = k >= 0 && token_row[k] == row && positions[k] == pos - j;
      if (here) {
        v = to_float(x[(int64_t)k * x_stride + c]);
      } else {
        j0 = j;
      }
    }
    if (j0 >= 0) {
      const int idx = taps - 2 - (j - j0);
      v = conv_state[((int64_t)row * (taps - 1) + idx) * channels + c];
    }
    acc = fmaf(w[(int64_t)c * taps + (taps - 1 - j)], v, acc);
  }
  out[(int64_t)i * channels + c] = from_float<T>(siluf_(acc));
}

// --------------------------------------------------------------- selective scan
// One group of `lanes` threads per (request, channel); each thread keeps NPT of the channel's states.
constexpr int SCAN_NPT = 8;
constexpr int SCAN_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const T* __restrict__ xc,            // [n, channels]  convolved, activated input
                      const float* __restrict__ dt_raw,    // [n, channels]  step-size projection, before bias
                      const float* __restrict__ dt_bias,   // [channels]
                      const float* __restrict__ A,         // [channels, n_state]  (negative)
                      const T* __restrict__ bc, int64_t bc_stride, int b_off, int c_off,   // B, C rows
                      const float* __restrict__ D,         // [channels]
                      const T* __restrict__ xz, int64_t xz_stride, int z_off,              // raw input and gate
                      float* __restrict__ ssm_state,       // [slots, channels, n_state]
                      float* __restrict__ conv_state,      // [slots, taps-1, channels]
                      const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                      T* __restrict__ out,                 // [n, channels]  y * silu(z)
                      int channels, int n_state, int taps, int lanes) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int per_block = SCAN_THREADS / lanes;
  const int c = blockIdx.x * per_block + threadIdx.x / lanes;
  const int sub = threadIdx.x % lanes;
  const int start = cu_q[r], end = cu_q[r + 1];
  const int slot = state_slots[r];
  const bool live = c < channels;
  const int cc = live ? c : 0;
  float S[SCAN_NPT], a[SCAN_NPT];
  float* sp = ssm_state + ((int64_t)slot * channels + cc) * n_state;
#pragma unroll
  for (int k = 0; k < SCAN_NPT; ++k) {
    const int n = sub * SCAN_NPT + k;
    const bool ok = live && n < n_state;
    S[k] = ok ? sp[n] : 0.f;
    a[k] = ok ? A[(int64_t)cc * n_state + n] : 0.f;
  }
  const float bias = dt_bias[cc], dskip = D[cc];
  for (int t = start; t < end; ++t) {
    const float dt = softplusf_(dt_raw[(int64_t)t * channels + cc] + bias);
    const float x = to_float(xc[(int64_t)t * channels + cc]);
    const float dx = dt * x;
    const T* brow = bc + (int64_t)t * bc_stride;
    float y = 0.f;
#pragma unroll
    for (int k = 0; k < SCAN_NPT; ++k) {
      const int n = sub * SCAN_NPT + k;
      if (n < n_state) {
        S[k] = expf(dt * a[k]) * S[k] + dx * to_float(brow[b_off + n]);
        y = fmaf(S[k], to_float(brow[c_off + n]), y);
      }
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
    if (sub == 0 && live) {
      const float z = to_float(xz[(int64_t)t * xz_stride + z_off + cc]);
      out[(int64_t)t * channels + cc] = from_float<T>((y + dskip * x) * siluf_(z));
    }
  }
  if (live) {
#pragma unroll
    for (int k = 0; k < SCAN_NPT; ++k) {
      const int n = sub * SCAN_NPT + k;
      if (n < n_state) sp[n] = S[k];
    }
  }
  // the convolution's memory: the request's last taps-1 raw inputs, oldest first
  if (live && sub == 0 && taps > 1) {
    const int keep = taps - 1, q_len = end - start;
    float* cs = conv_state + (int64_t)slot * keep * channels + cc;
    float fresh[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) {
      if (k < keep) {
        const int from_batch = q_len - keep + k;     // index among this step's tokens
        fresh[k] = from_batch >= 0 ? to_float(xz[(int64_t)(start + from_batch) * xz_stride + cc])
                                   : cs[(int64_t)(k + q_len) * channels];
      }
    }
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k)
      if (k < keep) cs[(int64_t)k * channels] = fresh[k];
  }
}

// --------------------------------------------------------------- matrix recurrence per head
// S [dk, dvx] per (request, head).  mode 0 (gated linear attention): a[d] = f[d], b[d] = 1 - f[d] with
// f = lower + (1 - lower) * sigmoid(f_raw + f_bias) and q = silu(q_raw).  mode 1 (matrix memory with
// exponential gates): i = cap * tanh((i_raw + i_bias) / cap), f = logsigmoid(cap * tanh((f_raw + f_bias) / cap)),
// m' = max(f + m, i), a = exp(f + m - m'), b[d] = exp(i - m') * k[d], q = q_raw * q_scale; the state
// has one column more than there are value columns, fed with ones, which carries the normaliser n, and
// the output gets two columns more: n . q and exp(-m').
// A block owns COLS columns of one (request, head); `lanes` threads share a column, each keeping DPT rows.
constexpr int REC_DPT = 16;
constexpr int REC_THREADS = 256;
constexpr int REC_CHUNK = 8;

template <typename T>
__global__ void __launch_bounds__(REC_THREADS)
matrix_recurrence_kernel(int mode,
                         const T* __restrict__ q, int64_t q_stride,       // [n, heads * dk] at its offset
                         const T* __restrict__ k, int64_t k_stride,       // mode 1
                         const T* __restrict__ v, int64_t v_stride,       // [n, heads * dv]
                         const float* __restrict__ gates, int64_t gates_stride,
                         // mode 0: f_raw [n, heads * dk]; mode 1: [n, 2 * heads]: i_raw | f_raw
                         const float* __restrict__ gate_bias,             // same layout as one row of gates
                         const float* __restrict__ lower,                 // mode 0: [heads * dk]
                         float cap, float q_scale,
                         float* __restrict__ state,                       // [slots, heads, dk, dvx]
                         float* __restrict__ mstate,                      // mode 1: [slots, heads]
                         const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                         float* __restrict__ out, int64_t out_stride,     // [n, heads * out_cols]
                         int heads, int dk, int dv, int lanes) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int cols = REC_THREADS / lanes;
  const int dvx = dv + (mode == 1 ? 1 : 0);
  const int out_cols = dv + (mode == 1 ? 2 : 0);
  const int r = blockIdx.z, h = blockIdx.y;
  const int col = blockIdx.x * cols + threadIdx.x / lanes;
  const int sub = threadIdx.x % lanes;
  const int start = cu_q[r], end = cu_q[r + 1];
  const int slot = state_slots[r];
  const bool live = col < dvx;
  float* q_s = smem;                              // [CHUNK, dk]
  float* a_s = q_s + REC_CHUNK * dk;              // [CHUNK, dk]  (mode 0)
  float* b_s = a_s + REC_CHUNK * dk;              // [CHUNK, dk]
  float* v_s = b_s + REC_CHUNK * dk;              // [CHUNK, cols]
  float* keep_s = v_s + REC_CHUNK * cols;         // [CHUNK]  mode 1: exp(f + m - m')
  float* take_s = keep_s + REC_CHUNK;             // [CHUNK]  mode 1: exp(i - m')
  float* e_s = take_s + REC_CHUNK;                // [CHUNK]  mode 1: exp(-m')
  __shared__ float m_run;

  float S[REC_DPT];
  float* sp = state + (((int64_t)slot * heads + h) * dk) * dvx + (live ? col : 0);
#pragma unroll
  for (int i = 0; i < REC_DPT; ++i) {
    const int d = sub * REC_DPT + i;
    S[i] = (live && d < dk) ? sp[(int64_t)d * dvx] : 0.f;
  }
  if (threadIdx.x == 0) m_run = mode == 1 ? mstate[(int64_t)slot * heads + h] : 0.f;
  __syncthreads();

  for (int t0 = start; t0 < end; t0 += REC_CHUNK) {
    const int nt = min(REC_CHUNK, end - t0);
    // ---- stage the chunk: effective q, a, b per (token, row), v per (token, column)
    if (mode == 1) {
      if (threadIdx.x == 0) {          // the scalar gates run in sequence: the maximum is carried
        float m = m_run;
        for (int tt = 0; tt < nt; ++tt) {
          const float* g = gates + (int64_t)(t0 + tt) * gates_stride;
          const float ig = cap * tanhf((g[h] + gate_bias[h]) / cap);
          const float fg = logsigmoidf_(cap * tanhf((g[heads + h] + gate_bias[heads + h]) / cap));
          const float m_new = fmaxf(fg + m, ig);
          keep_s[tt] = expf(fg + m - m_new);
          take_s[tt] = expf(ig - m_new);
          e_s[tt] = expf(-m_new);
          m = m_new;
        }
        m_run = m;
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < nt * dk; idx += REC_THREADS) {
        const int tt = idx / dk, d = idx - tt * dk;
        const int64_t t = t0 + tt;
        q_s[idx] = to_float(q[t * q_stride + (int64_t)h * dk + d]) * q_scale;
        b_s[idx] = take_s[tt] * to_float(k[t * k_stride + (int64_t)h * dk + d]);
      }
    } else {
      for (int idx = threadIdx.x; idx < nt * dk; idx += REC_THREADS) {
        const int tt = idx / dk, d = idx - tt * dk;
        const int64_t t = t0 + tt;
        const int hd = h * dk + d;
        const float lo = lower[hd];
        const float f = lo + (1.0f - lo) * sigmoidf_(gates[t * gates_stride + hd] + gate_bias[hd]);
        a_s[idx] = f;
        b_s[idx] = 1.0f - f;
        q_s[idx] = siluf_(to_float(q[t * q_stride + hd]));
      }
    }
    for (int idx = threadIdx.x; idx < nt * cols; idx += REC_THREADS) {
      const int tt = idx / cols, cix = idx - tt * cols;
      const int cg = blockIdx.x * cols + cix;
      v_s[idx] = cg < dv ? to_float(v[(int64_t)(t0 + tt) * v_stride + (int64_t)h * dv + cg]) : 1.0f;
    }
    __syncthreads();
    // ---- the recurrence over the chunk's tokens
    for (int tt = 0; tt < nt; ++tt) {
      const float vj = v_s[tt * cols + threadIdx.x / lanes];
      const float keep = mode == 1 ? keep_s[tt] : 0.f;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < REC_DPT; ++i) {
        const int d = sub * REC_DPT + i;
        if (d < dk) {
          const float a = mode == 1 ? keep : a_s[tt * dk + d];
          S[i] = a * S[i] + b_s[tt * dk + d] * vj;
          o = fmaf(S[i], q_s[tt * dk + d], o);
        }
      }
      for (int off = lanes >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (sub == 0 && live) out[(int64_t)(t0 + tt) * out_stride + (int64_t)h * out_cols + col] = o;
      if (mode == 1 && blockIdx.x == 0 && threadIdx.x == 0)
        out[(int64_t)(t0 + tt) * out_stride + (int64_t)h * out_cols + dv + 1] = e_s[tt];
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < REC_DPT; ++i) {
      const int d = sub * REC_DPT + i;
      if (d < dk) sp[(int64_t)d * dvx] = S[i];
    }
  }
  if (mode == 1 && blockIdx.x == 0 && threadIdx.x == 0) mstate[(int64_t)slot * heads + h] = m_run;
}

// --------------------------------------------------------------- per-head output norm
// One warp per (token, head): o [dv] (fp32, optionally divided by max(|o[dv]|, o[dv+1]) + den_eps, the
// two extra columns the recurrence wrote), divided by its root mean square, times a weight (shared by
// the heads when w_head_stride is 0), times sigmoid(gate) when a gate is given.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_kernel(const float* __restrict__ o, int64_t o_stride, int o_cols, int with_den, float den_eps,
                 const float* __restrict__ w, int w_head_stride, const T* __restrict__ gate, int64_t gate_stride,
                 T* __restrict__ out, int64_t out_stride, int n_tokens, int heads, int dv, float eps) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * 4 + warp;
  if (item >= (int64_t)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (int64_t)t * heads);
  const float* row = o + (int64_t)t * o_stride + (int64_t)h * o_cols;
  float inv_den = 1.0f;
  if (with_den) inv_den = 1.0f / (fmaxf(fabsf(row[dv]), row[dv + 1]) + den_eps);
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) {
    const float x = with_den ? row[c] * inv_den : row[c];
    ss = fmaf(x, x, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    float x = (with_den ? row[c] * inv_den : row[c]) * inv * w[(int64_t)h * w_head_stride + c];
    if (gate) x *= sigmoidf_(to_float(gate[(int64_t)t * gate_stride + (int64_t)h * dv + c]));
    out[(int64_t)t * out_stride + (int64_t)h * dv + c] = from_float<T>(x);
  }
}

inline int pow2_at_least(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

template <typename T>
int conv_silu_launch(const T* x, int64_t x_stride, const float* w, const float* bias, const float* conv_state,
                     const int* positions, const int* token_row, T* out, int n_tokens, int channels, int taps,
                     cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS || (channels + 255) / 256 > 65535) return (int)cudaErrorInvalidValue;
  return gllm_launch(conv_silu_kernel<T>, dim3(n_tokens, (channels + 255) / 256), dim3(256), 0, stream, x, x_stride, w,
                     bias, conv_state, positions, token_row, out, n_tokens, channels, taps);
}

template <typename T>
int selective_scan_launch(const T* xc, const float* dt_raw, const float* dt_bias, const float* A, const T* bc,
                          int64_t bc_stride, int b_off, int c_off, const float* D, const T* xz, int64_t xz_stride,
                          int z_off, float* ssm_state, float* conv_state, const int* cu_q, const int* state_slots,
                          T* out, int num_requests, int channels, int n_state, int taps, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  const int lanes = pow2_at_least((n_state + SCAN_NPT - 1) / SCAN_NPT);
  if (lanes > 32 || taps < 1 || taps > MAX_TAPS || num_requests > 65535) return (int)cudaErrorInvalidValue;
  const int per_block = SCAN_THREADS / lanes;
  return gllm_launch(selective_scan_kernel<T>, dim3((channels + per_block - 1) / per_block, num_requests),
                     dim3(SCAN_THREADS), 0, stream, xc, dt_raw, dt_bias, A, bc, bc_stride, b_off, c_off, D, xz, xz_stride,
                     z_off, ssm_state, conv_state, cu_q, state_slots, out, channels, n_state, taps, lanes);
}

template <typename T>
int matrix_recurrence_launch(int mode, const T* q, int64_t q_stride, const T* k, int64_t k_stride, const T* v,
                             int64_t v_stride, const float* gates, int64_t gates_stride, const float* gate_bias,
                             const float* lower, float cap, float q_scale, float* state, float* mstate,
                             const int* cu_q, const int* state_slots, float* out, int64_t out_stride,
                             int num_requests, int heads, int dk, int dv, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  const int lanes = pow2_at_least((dk + REC_DPT - 1) / REC_DPT);
  if (lanes > 32 || heads > 65535 || num_requests > 65535 || dk < 1 || dv < 1) return (int)cudaErrorInvalidValue;
  const int cols = REC_THREADS / lanes;
  const int dvx = dv + (mode == 1 ? 1 : 0);
  const size_t smem = sizeof(float) * ((size_t)3 * REC_CHUNK * dk + (size_t)REC_CHUNK * cols + 3 * REC_CHUNK);
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  return gllm_launch(matrix_recurrence_kernel<T>, dim3((dvx + cols - 1) / cols, heads, num_requests), dim3(REC_THREADS),
                     smem, stream, mode, q, q_stride, k, k_stride, v, v_stride, gates, gates_stride, gate_bias, lower, cap,
                     q_scale, state, mstate, cu_q, state_slots, out, out_stride, heads, dk, dv, lanes);
}

template <typename T>
int head_norm_launch(const float* o, int64_t o_stride, int o_cols, int with_den, float den_eps, const float* w,
                     int w_head_stride, const T* gate, int64_t gate_stride, T* out, int64_t out_stride, int n_tokens,
                     int heads, int dv, float eps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int64_t blocks = ((int64_t)n_tokens * heads + 3) / 4;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return gllm_launch(head_norm_kernel<T>, dim3((unsigned)blocks), dim3(128), 0, stream, o, o_stride, o_cols, with_den,
                     den_eps, w, w_head_stride, gate, gate_stride, out, out_stride, n_tokens, heads, dv, eps);
}
}  // namespace

#define GLLM_RECURRENT_EXPORTS(T, S)                                                                                  \
  GLLM_API int gllm_conv_silu_##S(const T* x, int64_t x_stride, const float* w, const float* bias,                    \
                                  const float* conv_state, const int* positions, const int* token_row, T* out,        \
                                  int n_tokens, int channels, int taps, cudaStream_t stream) {                        \
    return conv_silu_launch<T>(x, x_stride, w, bias, conv_state, positions, token_row, out, n_tokens, channels, taps, \
                               stream);                                                                               \
  }                                                                                                                   \
  GLLM_API int gllm_selective_scan_##S(const T* xc, const float* dt_raw, const float* dt_bias, const float* A,        \
                                       const T* bc, int64_t bc_stride, int b_off, int c_off, const float* D,          \
                                       const T* xz, int64_t xz_stride, int z_off, float* ssm_state, float* conv_state, \
                                       const int* cu_q, const int* state_slots, T* out, int num_requests,             \
                                       int channels, int n_state, int taps, cudaStream_t stream) {                    \
    return selective_scan_launch<T>(xc, dt_raw, dt_bias, A, bc, bc_stride, b_off, c_off, D, xz, xz_stride, z_off,     \
                                    ssm_state, conv_state, cu_q, state_slots, out, num_requests, channels, n_state,   \
                                    taps, stream);                                                                    \
  }                                                                                                                   \
  GLLM_API int gllm_matrix_recurrence_##S(int mode, const T* q, int64_t q_stride, const T* k, int64_t k_stride,       \
                                          const T* v, int64_t v_stride, const float* gates, int64_t gates_stride,     \
                                          const float* gate_bias, const float* lower, float cap, float q_scale,       \
                                          float* state, float* mstate, const int* cu_q, const int* state_slots,       \
                                          float* out, int64_t out_stride, int num_requests, int heads, int dk,        \
                                          int dv, cudaStream_t stream) {                                              \
    return matrix_recurrence_launch<T>(mode, q, q_stride, k, k_stride, v, v_stride, gates, gates_stride, gate_bias,   \
                                       lower, cap, q_scale, state, mstate, cu_q, state_slots, out, out_stride,        \
                                       num_requests, heads, dk, dv, stream);                                          \
  }                                                                                                                   \
  GLLM_API int gllm_head_norm_##S(const float* o, int64_t o_stride, int o_cols, int with_den, float den_eps,          \
                                  const float* w, int w_head_stride, const T* gate, int64_t gate_stride, T* out,      \
                                  int64_t out_stride, int n_tokens, int heads, int dv, float eps,                     \
                                  cudaStream_t stream) {                                                              \
    return head_norm_launch<T>(o, o_stride, o_cols, with_den, den_eps, w, w_head_stride, gate, gate_stride, out,      \
                               out_stride, n_tokens, heads, dv, eps, stream);                                         \
  }

GLLM_RECURRENT_EXPORTS(float, f32)
GLLM_RECURRENT_EXPORTS(__nv_bfloat16, bf16)
