// Causal attention over the paged cache whose weights are not a softmax: the weight of a visible key
// is sigmoid(q . k * scale + bias[head]), and the weights are not normalised over the keys.  Keys and
// values may differ in width.  Beside it, the kernel that prepares its operands: an RMS norm of every
// query and key head (one weight per column, shared by the heads), a multiplier on the queries that
// grows with the logarithm of the position, 1 + coef * ln(floor((p + 1) / every) + 1), and the store of
// the new keys and values into their pages.
//
// Page layout: [kv_heads, block_size, dk] keys, then [kv_heads, block_size, dv] values.
// Scores, weights and the output sum are fp32; keys are taken in blocks of 32 aligned to absolute
// positions and added in ascending order, so a result depends neither on how the request was cut into
// steps nor on the rest of the batch.  One warp per (token, query head).
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_DK = 256;
constexpr int MAX_DV = 256;

// One warp per (token, head) of the stacked [q | k | v] row.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_store_kernel(T* __restrict__ qkv, int64_t stride, const float* __restrict__ q_weight,
                     const float* __restrict__ k_weight, float eps, float temp_coef, float temp_every,
                     const int* __restrict__ positions, const int* __restrict__ slot_mapping, T* __restrict__ cache,
                     int n_tokens, int hq, int hkv, int dk, int dv, int block_size, int num_pages,
                     int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_token = hq + 2 * hkv;
  const int64_t item = (int64_t)blockIdx.x * WARPS + warp;
  if (item >= (int64_t)n_tokens * per_token) return;
  const int n = (int)(item / per_token), h = (int)(item - (int64_t)n * per_token);
  T* row = qkv + (int64_t)n * stride;
  const size_t page_elems = (size_t)hkv * block_size * (dk + dv);
  int64_t dst = -1;
  if (h >= hq && slot_mapping != nullptr) {
    const int slot = slot_mapping[n];
    if (slot < 0) return;
    const int page = slot / block_size, off = slot % block_size;
    if (page >= num_pages) {
      if (lane == 0) atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      return;
    }
    if (h < hq + hkv)
      dst = (int64_t)((size_t)page * page_elems + ((size_t)(h - hq) * block_size + off) * dk);
    else
      dst = (int64_t)((size_t)page * page_elems + (size_t)hkv * block_size * dk +
                      ((size_t)(h - hq - hkv) * block_size + off) * dv);
  }
  if (h >= hq + hkv) {                       // a value head: stored as it is
    if (dst < 0) return;
    const T* src = row + (int64_t)hq * dk + (int64_t)hkv * dk + (int64_t)(h - hq - hkv) * dv;
    for (int c = lane; c < dv; c += 32) cache[dst + c] = src[c];
    return;
  }
  T* x = row + (int64_t)h * dk;
  float ss = 0.f;
  for (int c = lane; c < dk; c += 32) {
    const float v = to_float(x[c]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  float mult = 1.0f / sqrtf(ss / (float)dk + eps);
  const float* w = h < hq ? q_weight : k_weight;
  float after = 1.0f;
  if (h < hq && temp_coef != 0.f) {
    const float steps = floorf((float)(positions[n] + 1) / temp_every);
    after = 1.0f + temp_coef * logf(steps + 1.0f);
  }
  for (int c = lane; c < dk; c += 32) {
    const float v = to_float(x[c]) * mult * w[c] * after;
    if (h < hq) x[c] = from_float<T>(v);
    else if (dst >= 0) cache[dst + c] = from_float<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_sigmoid_kernel(const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, int64_t out_stride,
                         const T* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
                         const int* __restrict__ positions, const int* __restrict__ token_row,
                         const float* __restrict__ head_bias, int n_tokens, int hq, int hkv, int dk, int dv,
                         int block_size, int num_pages, float scale, int* __restrict__ status) {
  __shared__ float q_s[WARPS][MAX_DK];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * WARPS + warp;
  if (item >= (int64_t)n_tokens * hq) return;
  const int n = (int)(item / hq), h = (int)(item - (int64_t)n * hq);
  const int kvh = h / (hq / hkv);
  const int qpos = positions[n];
  const int* bt = block_table + (int64_t)token_row[n] * bt_stride;
  const T* qv = q + (int64_t)n * q_stride + (int64_t)h * dk;
  for (int i = lane; i < dk; i += 32) q_s[warp][i] = to_float(qv[i]);
  __syncwarp();
  const float bias = head_bias ? head_bias[h] : 0.f;
  const size_t page_elems = (size_t)hkv * block_size * (dk + dv);
  const size_t v_base = (size_t)hkv * block_size * dk;
  float acc[MAX_DV / 32], lost[MAX_DV / 32];
#pragma unroll
  for (int i = 0; i < MAX_DV / 32; ++i) acc[i] = lost[i] = 0.f;
  for (int j0 = 0; j0 <= qpos; j0 += 32) {
    const int j = j0 + lane;
    float p = 0.f;
    int64_t vbase = -1;
    if (j <= qpos) {
      const int page = bt[j / block_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      } else {
        const int off = j % block_size;
        const T* kp = cache + (size_t)page * page_elems + ((size_t)kvh * block_size + off) * dk;
        float dot = 0.f;
        for (int i = 0; i < dk; ++i) dot = fmaf(q_s[warp][i], to_float(kp[i]), dot);
        p = 1.0f / (1.0f + expf(-(dot * scale + bias)));
        vbase = (int64_t)((size_t)page * page_elems + v_base + ((size_t)kvh * block_size + off) * dv);
      }
    }
    // the block's 32 terms are added up by themselves and then added to the total with the low-order bits that
    // the addition drops carried along (compensated summation): the rounding error of a long context stays that
    // of one block
    float part[MAX_DV / 32];
#pragma unroll
    for (int i = 0; i < MAX_DV / 32; ++i) part[i] = 0.f;
    const int count = min(32, qpos - j0 + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int64_t vb = __shfl_sync(0xffffffffu, vbase, jj);
      if (vb < 0) continue;
      const T* vp = cache + vb;
#pragma unroll
      for (int i = 0; i < MAX_DV / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) part[i] = fmaf(pj, to_float(vp[c]), part[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_DV / 32; ++i) {
      const float y = part[i] - lost[i];
      const float t = acc[i] + y;
      lost[i] = (t - acc[i]) - y;
      acc[i] = t;
    }
  }
  T* o = out + (int64_t)n * out_stride + (int64_t)h * dv;
#pragma unroll
  for (int i = 0; i < MAX_DV / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) o[c] = from_float<T>(acc[i]);
  }
}

template <typename T>
int qk_norm_store_launch(T* qkv, int64_t stride, const float* q_weight, const float* k_weight, float eps,
                         float temp_coef, float temp_every, const int* positions, const int* slot_mapping, T* cache,
                         int n_tokens, int hq, int hkv, int dk, int dv, int block_size, int num_pages, int* status,
                         cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hq <= 0 || hkv <= 0 || dk <= 0 || dv <= 0 || (temp_coef != 0.f && !(temp_every > 0.f)))
    return (int)cudaErrorInvalidValue;
  const int64_t blocks = ((int64_t)n_tokens * (hq + 2 * hkv) + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return gllm_launch(qk_norm_store_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, qkv, stride, q_weight,
                     k_weight, eps, temp_coef, temp_every, positions, slot_mapping, cache, n_tokens, hq, hkv, dk, dv,
                     block_size, num_pages, status);
}

template <typename T>
int attention_sigmoid_launch(const T* q, int64_t q_stride, T* out, int64_t out_stride, const T* cache,
                             const int* block_table, int bt_stride, const int* positions, const int* token_row,
                             const float* head_bias, int n_tokens, int hq, int hkv, int dk, int dv, int block_size,
                             int num_pages, float scale, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dk <= 0 || dk > MAX_DK || dv <= 0 || dv > MAX_DV || hq <= 0 || hkv <= 0 || hq % hkv)
    return (int)cudaErrorInvalidValue;
  const int64_t blocks = ((int64_t)n_tokens * hq + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return gllm_launch(attention_sigmoid_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, q, q_stride, out,
                     out_stride, cache, block_table, bt_stride, positions, token_row, head_bias, n_tokens, hq, hkv, dk,
                     dv, block_size, num_pages, scale, status);
}
}  // namespace

#define GLLM_SIGMOID_EXPORTS(T, S)                                                                                    \
  GLLM_API int gllm_qk_norm_store_##S(T* qkv, int64_t stride, const float* q_weight, const float* k_weight, float eps, \
                                      float temp_coef, float temp_every, const int* positions,                        \
                                      const int* slot_mapping, T* cache, int n_tokens, int hq, int hkv, int dk,       \
                                      int dv, int block_size, int num_pages, int* status, cudaStream_t stream) {      \
    return qk_norm_store_launch<T>(qkv, stride, q_weight, k_weight, eps, temp_coef, temp_every, positions,            \
                                   slot_mapping, cache, n_tokens, hq, hkv, dk, dv, block_size, num_pages, status,     \
                                   stream);                                                                           \
  }                                                                                                                   \
  GLLM_API int gllm_attention_sigmoid_##S(const T* q, int64_t q_stride, T* out, int64_t out_stride, const T* cache,   \
                                          const int* block_table, int bt_stride, const int* positions,                \
                                          const int* token_row, const float* head_bias, int n_tokens, int hq,         \
                                          int hkv, int dk, int dv, int block_size, int num_pages, float scale,        \
                                          int* status, cudaStream_t stream) {                                         \
    return attention_sigmoid_launch<T>(q, q_stride, out, out_stride, cache, block_table, bt_stride, positions,        \
                                       token_row, head_bias, n_tokens, hq, hkv, dk, dv, block_size, num_pages, scale, \
                                       status, stream);                                                               \
  }

GLLM_SIGMOID_EXPORTS(float, f32)
GLLM_SIGMOID_EXPORTS(__nv_bfloat16, bf16)
