// A residual that is kept as several parallel streams (hyper-connections), and the embedding that
// starts it.
//
// Layout: X [tokens, streams, width] fp32.  A sublayer reads u = sum_s read[s] * X[:, s], runs on the
// RMS norm of u, and its result y is written back as X'[:, t] = sum_s mix[s, t] * X[:, s] + write[t] * y
// (all streams at once, from the old ones).  As with the single residual stream, whose add is fused
// into the norm kernel that follows it, the write of one sublayer and the read + norm of the next are
// one kernel here: one block per token, every sum in fp32 and in a fixed order (streams ascending).
// With streams = 1, mix = [[1]], write = [1], read = [1] this is add + RMSNorm.
#include "common.cuh"

namespace {
constexpr int MAX_STREAMS = 16;

// Token embedding (+ a sinusoid of the position: column 2i = sin(p f_i), 2i+1 = cos(p f_i), with the
// frequencies f_i given in fp32 and the angle formed in fp32), copied into every stream.  A negative
// token id stands for sampled[token_row[i]] (the token the previous step left on the device).
template <typename T>
__global__ void __launch_bounds__(256)
embed_streams_kernel(const int* __restrict__ tokens, const int* __restrict__ sampled, const int* __restrict__ token_row,
                     const T* __restrict__ table, const int* __restrict__ positions, const float* __restrict__ freq,
                     float* __restrict__ out, int width, int vocab, int streams, float scale, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  int tok = tokens[i];
  if (tok < 0 && sampled != nullptr) tok = sampled[token_row[i]];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, GLLM_STATUS_TOKEN_RANGE);
    tok = 0;
  }
  const float p = freq ? (float)positions[i] : 0.f;
  const T* row = table + (int64_t)tok * width;
  float* o = out + (int64_t)i * streams * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = to_float(row[c]) * scale;
    if (freq) {
      const float ang = p * freq[c >> 1];
      v += (c & 1) ? cosf(ang) : sinf(ang);
    }
    for (int s = 0; s < streams; ++s) o[(int64_t)s * width + c] = v;
  }
}

// rows == nullptr: token i = blockIdx.x, X is updated in place.  rows given: only those tokens, X untouched.
template <typename T, int STREAMS>
__global__ void __launch_bounds__(256)
stream_mix_norm_kernel(const T* __restrict__ y, float* __restrict__ X, const float* __restrict__ mix,
                       const float* __restrict__ write, const float* __restrict__ read,
                       const float* __restrict__ weight, T* __restrict__ out, float* __restrict__ sum_out,
                       const int* __restrict__ rows, int width, float eps) {
  constexpr int streams = STREAMS;
  extern __shared__ float u_s[];          // [width]
  __shared__ float scratch[32];
  __shared__ float mix_s[STREAMS * STREAMS], write_s[STREAMS], read_s[STREAMS];
  if (threadIdx.x < streams * streams) mix_s[threadIdx.x] = mix ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < streams) {
    write_s[threadIdx.x] = write ? write[threadIdx.x] : 0.f;
    read_s[threadIdx.x] = read ? read[threadIdx.x] : 1.0f;
  }
  pdl_trigger();
  pdl_wait();
  __syncthreads();
  const int i = rows ? rows[blockIdx.x] : blockIdx.x;
  float* x = X + (int64_t)i * streams * width;
  const bool has_y = y != nullptr;
  float ss = 0.f;
  // four columns a thread at a time: all their loads are asked for before the first store (the streams are
  // read and written through the same pointer, so the compiler keeps loads behind earlier stores)
  constexpr int UNROLL = STREAMS > 8 ? 1 : 4;
  for (int c0 = threadIdx.x; c0 < width; c0 += UNROLL * blockDim.x) {
    float old[UNROLL][STREAMS], yv[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const int c = c0 + k * blockDim.x;
      const bool ok = c < width;
#pragma unroll
      for (int s = 0; s < STREAMS; ++s) old[k][s] = (ok && s < streams) ? x[(int64_t)s * width + c] : 0.f;
      yv[k] = (ok && has_y) ? to_float(y[(int64_t)i * width + c]) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const int c = c0 + k * blockDim.x;
      if (c >= width) break;
      float u = 0.f;
      if (has_y) {
#pragma unroll
        for (int t = 0; t < STREAMS; ++t) {
          if (t < streams) {
            float nv = 0.f;
#pragma unroll
            for (int s = 0; s < STREAMS; ++s)
              if (s < streams) nv = fmaf(mix_s[s * streams + t], old[k][s], nv);
            nv = fmaf(write_s[t], yv[k], nv);
            if (!rows) x[(int64_t)t * width + c] = nv;
            u = fmaf(read_s[t], nv, u);
          }
        }
      } else {
#pragma unroll
        for (int t = 0; t < STREAMS; ++t)
          if (t < streams) u = fmaf(read_s[t], old[k][t], u);
      }
      u_s[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (sum_out) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) sum_out[(int64_t)blockIdx.x * width + c] = u_s[c];
  }
  if (out == nullptr) return;
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(int64_t)blockIdx.x * width + c] = from_float<T>(u_s[c] * inv * weight[c]);
}

template <typename T>
int embed_streams_launch(const int* tokens, const int* sampled, const int* token_row, const T* table,
                         const int* positions, const float* freq, float* out, int n, int width, int vocab, int streams,
                         float scale, int* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (streams < 1 || width < 1) return (int)cudaErrorInvalidValue;
  return gllm_launch(embed_streams_kernel<T>, dim3(n), dim3(256), 0, stream, tokens, sampled, token_row, table,
                     positions, freq, out, width, vocab, streams, scale, status);
}

template <typename T>
int stream_mix_norm_launch(const T* y, float* X, const float* mix, const float* write, const float* read,
                           const float* weight, T* out, float* sum_out, const int* rows, int n_rows, int width,
                           int streams, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (streams < 1 || streams > MAX_STREAMS || width < 1 || (size_t)width * 4 > 160 * 1024)
    return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)width * sizeof(float);
  void (*kernel)(const T*, float*, const float*, const float*, const float*, const float*, T*, float*, const int*, int,
                 float) = nullptr;
  switch (streams) {
    case 1: kernel = stream_mix_norm_kernel<T, 1>; break;
    case 2: kernel = stream_mix_norm_kernel<T, 2>; break;
    case 3: kernel = stream_mix_norm_kernel<T, 3>; break;
    case 4: kernel = stream_mix_norm_kernel<T, 4>; break;
    case 5: kernel = stream_mix_norm_kernel<T, 5>; break;
    case 6: kernel = stream_mix_norm_kernel<T, 6>; break;
    case 7: kernel = stream_mix_norm_kernel<T, 7>; break;
    case 8: kernel = stream_mix_norm_kernel<T, 8>; break;
    case 9: kernel = stream_mix_norm_kernel<T, 9>; break;
    case 10: kernel = stream_mix_norm_kernel<T, 10>; break;
    case 11: kernel = stream_mix_norm_kernel<T, 11>; break;
    case 12: kernel = stream_mix_norm_kernel<T, 12>; break;
    case 13: kernel = stream_mix_norm_kernel<T, 13>; break;
    case 14: kernel = stream_mix_norm_kernel<T, 14>; break;
    case 15: kernel = stream_mix_norm_kernel<T, 15>; break;
    default: kernel = stream_mix_norm_kernel<T, 16>; break;
  }
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return gllm_launch(kernel, dim3(n_rows), dim3(256), smem, stream, y, X, mix, write, read, weight, out, sum_out, rows,
                     width, eps);
}
}  // namespace

#define GLLM_STREAMS_EXPORTS(T, S)                                                                                     \
  GLLM_API int gllm_embed_streams_##S(const int* tokens, const int* sampled, const int* token_row, const T* table,     \
                                      const int* positions, const float* freq, float* out, int n, int width,           \
                                      int vocab, int streams, float scale, int* status, cudaStream_t stream) {         \
    return embed_streams_launch<T>(tokens, sampled, token_row, table, positions, freq, out, n, width, vocab, streams,  \
                                   scale, status, stream);                                                             \
  }                                                                                                                    \
  GLLM_API int gllm_stream_mix_norm_##S(const T* y, float* X, const float* mix, const float* write, const float* read, \
                                        const float* weight, T* out, float* sum_out, const int* rows, int n_rows,      \
                                        int width, int streams, float eps, cudaStream_t stream) {                      \
    return stream_mix_norm_launch<T>(y, X, mix, write, read, weight, out, sum_out, rows, n_rows, width, streams, eps,  \
                                     stream);                                                                          \
  }

GLLM_STREAMS_EXPORTS(float, f32)
GLLM_STREAMS_EXPORTS(__nv_bfloat16, bf16)
