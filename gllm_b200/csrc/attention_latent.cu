// Attention over one cached latent vector per token (multi-head latent attention).
//
// Every token caches c (rank numbers, the RMS-normed down-projection) followed by one rotated key part
// kr (rot numbers) that all heads share: rank + rot numbers per token and layer instead of keys and values
// for every head.  Head h's key is [W_uk[h] c ; kr] and its value W_uv[h] c.  Both up-projections are moved
// to the query's side so that the cached vectors are used as they are:
//
//   score(i, j) = ((W_uk[h]^T q_i) . c_j + qr_i . kr_j) * scale        qa = W_uk[h]^T q : rank numbers
//   out_i       = W_uv[h] (sum_j p_ij c_j)                             the sum over keys: rank numbers
//
// i.e. attention with ONE key/value head of width rank + rot whose values are the first rank columns of
// the keys.  Kernels here:
//   latent_prep       per token: c = rms(down[:rank]) * w, kr = rotate(down[rank:]), both stored into the
//                     token's cache slot; the rotated part of every query head is rotated in place
//   head_linear       out[n, h, :] = W[h] x[n, h, :] for every head (qa from q; values from the summed latents)
//   attention_latent  softmax attention of every (token, head) over the request's cached [c ; kr], with an
//                     optional sigmoid gate per (token, head) on the result; CUDA cores, any widths
// Positions, angles, norm statistics, scores, softmax statistics and accumulators are fp32.  Keys are taken in
// blocks of 32 aligned to absolute positions, so a token's result does not depend on how its request was cut
// into steps or on the rest of the batch.
#include "common.cuh"

namespace {

// ------------------------------------------------------------------ latent_prep
// The projection may arrive as `n_parts` unsummed fp32 splits of the product: they are summed into `rows` first.
// row: [n, stride] of T; the query heads start at column 0, each `q_head` wide with its rotated part at
// column `q_plain` of the head; the down-projection (rank + rot columns) starts at column `down_col`.
// Rotation: neighbours (2i, 2i+1) of the first `rot_dims` columns of a rotated part, angle p * inv_freq[i].
// Cache layer: [page][block_size][rank + rot].
template <typename T>
__global__ void __launch_bounds__(256)
latent_prep_kernel(T* __restrict__ rows, int64_t stride, const float* __restrict__ parts, int n_parts,
                   int64_t part_stride, int width, const float* __restrict__ norm_w, float eps,
                   const int* __restrict__ positions, const float* __restrict__ inv_freq,
                   const int* __restrict__ slot_mapping, T* __restrict__ cache, int n_tokens, int heads, int q_head,
                   int q_plain, int down_col, int rank, int rot, int rot_dims, int block_size, int num_pages,
                   int* __restrict__ status) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  T* row = rows + (size_t)n * stride;
  if (parts) {     // the projection arrives as unsummed splits [part][token][width]: summed in ascending order first
    const float* src = parts + (size_t)n * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
      row[c] = from_float<T>(sum_parts16(src + c, n_parts, part_stride));
    __syncthreads();
  }
  const float pos = (float)positions[n];
  const int half = rot_dims / 2;
  // the rotated part of every query head, in place
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    T* part = row + (size_t)h * q_head + q_plain;
    const float u = to_float(part[2 * i]), v = to_float(part[2 * i + 1]);
    part[2 * i] = from_float<T>(u * c - v * s);
    part[2 * i + 1] = from_float<T>(v * c + u * s);
  }
  const T* down = row + down_col;
  float ss = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    const float x = to_float(down[c]);
    ss += x * x;
  }
  const float total = block_sum(ss, scratch);
  const int slot = slot_mapping ? slot_mapping[n] : -1;
  if (slot < 0) return;
  const int page = slot / block_size, off = slot - page * block_size;
  if (page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, GLLM_STATUS_PAGE_RANGE);
    return;
  }
  const float inv = 1.0f / sqrtf(total / (float)rank + eps);
  T* dst = cache + ((size_t)page * block_size + off) * (rank + rot);
  for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_float<T>(to_float(down[c]) * inv * norm_w[c]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    const float u = to_float(down[rank + 2 * i]), v = to_float(down[rank + 2 * i + 1]);
    dst[rank + 2 * i] = from_float<T>(u * c - v * s);
    dst[rank + 2 * i + 1] = from_float<T>(v * c + u * s);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = down[rank + c];
}

// ------------------------------------------------------------------ head_linear
// out[n * out_stride + h * out_head + j] = sum_i x[n * x_stride + h * x_head + i] * w[(h * J + j) * I + i]
// for j < J, i < I: one small product per head, all heads in one launch (blockIdx.z = head).  Every output is
// summed by one thread over i in ascending order whatever the number of tokens is.
constexpr int HL_BM = 64, HL_BN = 64, HL_BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ x, int64_t x_stride, int x_head, const T* __restrict__ w,
                   T* __restrict__ out, int64_t out_stride, int out_head, int n_tokens, int I, int J) {
  __shared__ float xs[HL_BK][HL_BM + 4];
  __shared__ float ws[HL_BK][HL_BN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * HL_BM, n0 = blockIdx.x * HL_BN, h = blockIdx.z;
  const T* xh = x + (size_t)h * x_head;
  const T* wh = w + (size_t)h * J * I;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < I; k0 += HL_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int m = m0 + lrow, j = n0 + lrow;
      xs[lk + e][lrow] = (m < n_tokens && k < I) ? to_float(xh[(size_t)m * x_stride + k]) : 0.f;
      ws[lk + e][lrow] = (j < J && k < I) ? to_float(wh[(size_t)j * I + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HL_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= n_tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx * 4 + j;
      if (c < J) out[(size_t)m * out_stride + (size_t)h * out_head + c] = from_float<T>(acc[i][j]);
    }
  }
}

// ------------------------------------------------------------------ attention_latent
// One warp per (token, head).  qa: [n, heads, rank] (stride per token / per head given); qr: the rotated query
// parts inside the projection rows.  gate: one logit per (token, head) at gate[n * gate_stride + h] (null: no
// gate); the result is multiplied by sigmoid(gate).  out: [n, heads, rank].
constexpr int LA_WARPS = 4;
constexpr int LA_MAX_K = 640;        // rank + rot
template <typename T, int CHUNKS>    // CHUNKS * 32 >= rank
__global__ void __launch_bounds__(LA_WARPS * 32)
attention_latent_kernel(const T* __restrict__ qa, int64_t qa_stride, int qa_head, const T* __restrict__ qr,
                        int64_t qr_stride, int qr_head, const T* __restrict__ gate, int64_t gate_stride,
                        T* __restrict__ out, int64_t out_stride, int out_head, const T* __restrict__ cache,
                        const int* __restrict__ block_table, int bt_stride, const int* __restrict__ positions,
                        const int* __restrict__ token_row, int n_tokens, int heads, int rank, int rot,
                        int block_size, int num_pages, float scale, int window, int* __restrict__ status) {
  __shared__ float q_s[LA_WARPS][LA_MAX_K];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * LA_WARPS + warp;
  if (item >= (int64_t)n_tokens * heads) return;
  const int n = (int)(item / heads), h = (int)(item - (int64_t)n * heads);
  const int qpos = positions[n];
  const int* bt = block_table + (int64_t)token_row[n] * bt_stride;
  const int dk = rank + rot;
  const T* qav = qa + (int64_t)n * qa_stride + (int64_t)h * qa_head;
  const T* qrv = qr + (int64_t)n * qr_stride + (int64_t)h * qr_head;
  for (int i = lane; i < rank; i += 32) q_s[warp][i] = to_float(qav[i]);
  for (int i = lane; i < rot; i += 32) q_s[warp][rank + i] = to_float(qrv[i]);
  __syncwarp();

  const int kstart = window > 0 ? max(0, qpos - window + 1) : 0;
  float m = -INFINITY, l = 0.f;
  float acc[CHUNKS];
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) acc[i] = 0.f;

  for (int j0 = kstart & ~31; j0 <= qpos; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j >= kstart && j <= qpos;
    float s = -INFINITY;
    int64_t kbase = -1;
    if (valid) {
      const int page = bt[j / block_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      } else {
        kbase = (int64_t)(((size_t)page * block_size + (size_t)(j % block_size)) * dk);
        const T* kp = cache + kbase;
        float dot = 0.f;
        for (int i = 0; i < dk; ++i) dot = fmaf(q_s[warp][i], to_float(kp[i]), dot);
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;      // only after a bad page id
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) acc[i] *= corr;
    const int count = min(32, qpos - j0 + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int64_t kb = __shfl_sync(0xffffffffu, kbase, jj);
      if (kb < 0) continue;  // uniform across the warp
      const T* vp = cache + kb;
#pragma unroll
      for (int i = 0; i < CHUNKS; ++i) {
        const int c = lane + 32 * i;
        if (c < rank) acc[i] = fmaf(pj, to_float(vp[c]), acc[i]);
      }
    }
    m = m_new;
  }
  float mult = l > 0.f ? 1.0f / l : 0.f;
  if (gate) mult *= 1.0f / (1.0f + expf(-to_float(gate[(int64_t)n * gate_stride + h])));
  T* o = out + (int64_t)n * out_stride + (int64_t)h * out_head;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = lane + 32 * i;
    if (c < rank) o[c] = from_float<T>(acc[i] * mult);
  }
}

template <typename T>
int latent_prep_launch(T* rows, int64_t stride, const float* parts, int n_parts, int64_t part_stride, int width,
                       const float* norm_w, float eps, const int* positions,
                       const float* inv_freq, const int* slot_mapping, T* cache, int n_tokens, int heads, int q_head,
                       int q_plain, int down_col, int rank, int rot, int rot_dims, int block_size, int num_pages,
                       int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (rank <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2 || q_plain + rot > q_head ||
      n_parts > 16 || (parts && width > stride))
    return (int)cudaErrorInvalidValue;
  return gllm_launch(latent_prep_kernel<T>, dim3((unsigned)n_tokens), dim3(256), 0, stream, rows, stride, parts,
                     n_parts, part_stride, width, norm_w, eps,
                     positions, inv_freq, slot_mapping, cache, n_tokens, heads, q_head, q_plain, down_col, rank, rot,
                     rot_dims, block_size, num_pages, status);
}

template <typename T>
int head_linear_launch(const T* x, int64_t x_stride, int x_head, const T* w, T* out, int64_t out_stride,
                       int out_head, int n_tokens, int heads, int I, int J, cudaStream_t stream) {
  if (n_tokens <= 0 || heads <= 0) return 0;
  if (I <= 0 || J <= 0 || heads > 65535) return (int)cudaErrorInvalidValue;
  const dim3 grid((J + HL_BN - 1) / HL_BN, (n_tokens + HL_BM - 1) / HL_BM, heads);
  if (grid.y > 65535) return (int)cudaErrorInvalidValue;
  return gllm_launch(head_linear_kernel<T>, grid, dim3(256), 0, stream, x, x_stride, x_head, w, out, out_stride,
                     out_head, n_tokens, I, J);
}

template <typename T>
int attention_latent_launch(const T* qa, int64_t qa_stride, int qa_head, const T* qr, int64_t qr_stride, int qr_head,
                            const T* gate, int64_t gate_stride, T* out, int64_t out_stride, int out_head,
                            const T* cache, const int* block_table, int bt_stride, const int* positions,
                            const int* token_row, int n_tokens, int heads, int rank, int rot, int block_size,
                            int num_pages, float scale, int window, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (rank <= 0 || rot < 0 || rank + rot > LA_MAX_K || rank > 512 || heads <= 0) return (int)cudaErrorInvalidValue;
  const int64_t items = (int64_t)n_tokens * heads;
  const int64_t blocks = (items + LA_WARPS - 1) / LA_WARPS;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
#define GLLM_LA_LAUNCH(C)                                                                                        \
  return gllm_launch(attention_latent_kernel<T, C>, dim3((unsigned)blocks), dim3(LA_WARPS * 32), 0, stream, qa,   \
                     qa_stride, qa_head, qr, qr_stride, qr_head, gate, gate_stride, out, out_stride, out_head,    \
                     cache, block_table, bt_stride, positions, token_row, n_tokens, heads, rank, rot, block_size, \
                     num_pages, scale, window, status)
  if (rank <= 128) GLLM_LA_LAUNCH(4);
  if (rank <= 256) GLLM_LA_LAUNCH(8);
  GLLM_LA_LAUNCH(16);
#undef GLLM_LA_LAUNCH
}
}  // namespace

#define GLLM_LATENT_EXPORTS(T, S)                                                                                \
  GLLM_API int gllm_latent_prep_##S(T* rows, int64_t stride, const float* parts, int n_parts, int64_t part_stride, \
                                    int width, const float* norm_w, float eps, const int* positions,             \
                                    const float* inv_freq, const int* slot_mapping, T* cache, int n_tokens,      \
                                    int heads, int q_head, int q_plain, int down_col, int rank, int rot,         \
                                    int rot_dims, int block_size, int num_pages, int* status,                    \
                                    cudaStream_t stream) {                                                       \
    return latent_prep_launch<T>(rows, stride, parts, n_parts, part_stride, width, norm_w, eps, positions,       \
                                 inv_freq, slot_mapping, cache, n_tokens,                                        \
                                 heads, q_head, q_plain, down_col, rank, rot, rot_dims, block_size, num_pages,   \
                                 status, stream);                                                                \
  }                                                                                                              \
  GLLM_API int gllm_head_linear_##S(const T* x, int64_t x_stride, int x_head, const T* w, T* out,                \
                                    int64_t out_stride, int out_head, int n_tokens, int heads, int I, int J,     \
                                    cudaStream_t stream) {                                                       \
    return head_linear_launch<T>(x, x_stride, x_head, w, out, out_stride, out_head, n_tokens, heads, I, J, stream); \
  }                                                                                                              \
  GLLM_API int gllm_attention_latent_##S(const T* qa, int64_t qa_stride, int qa_head, const T* qr,               \
                                         int64_t qr_stride, int qr_head, const T* gate, int64_t gate_stride,     \
                                         T* out, int64_t out_stride, int out_head, const T* cache,               \
                                         const int* block_table, int bt_stride, const int* positions,            \
                                         const int* token_row, int n_tokens, int heads, int rank, int rot,       \
                                         int block_size, int num_pages, float scale, int window, int* status,    \
                                         cudaStream_t stream) {                                                  \
    return attention_latent_launch<T>(qa, qa_stride, qa_head, qr, qr_stride, qr_head, gate, gate_stride, out,    \
                                      out_stride, out_head, cache, block_table, bt_stride, positions, token_row, \
                                      n_tokens, heads, rank, rot, block_size, num_pages, scale, window, status,  \
                                      stream);                                                                   \
  }
GLLM_LATENT_EXPORTS(float, f32)
GLLM_LATENT_EXPORTS(__nv_bfloat16, bf16)
