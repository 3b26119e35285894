// Sigmoid-weighted causal attention of the bf16 path on the tensor cores, over the paged cache:
// out[i, h] = sum_{j <= p_i} sigmoid(q_i . k_j * scale + bias[h]) v_j, keys dk wide and values dv wide.
//
// The arrangement is that of the softmax prefill kernel (attention_prefill_bf16.cu): one CTA (4 warps)
// owns 64 rows = (64 / G') query tokens x G' query heads that share one kv head, K/V tiles of 64 keys are
// fetched page by page with cp.async in two stages, Q K^T and P V run as mma.sync m16n8k16 with fp32
// accumulation.  Without a softmax there is no running maximum and no rescaling: the weights are formed in
// fp32, rounded to bf16 for the second product, and summed in fp32.  For the same reason a request's keys
// can be cut into ranges whose partial results simply add: with `splits` > 1 the CTA of (tile, split s)
// visits the key tiles [s * tiles_per_split, (s + 1) * tiles_per_split) and writes an fp32 partial
// [split][token][head * dv] (zeros when its range is empty), which a later kernel adds in ascending order;
// that is how single decoded tokens get enough CTAs to stream a long context.
// Page layout: [kv_heads, block_size, dk] keys, then [kv_heads, block_size, dv] values.
#include "mma_utils.cuh"

namespace {
constexpr int BM = 64, BN = 64, SG_THREADS = 128;

// piece index XORed with row bits inside its own group of 8 (rows of a multiple of 8 pieces) or of 4
template <int C>
__device__ __forceinline__ int swz(int row, int piece) {
  if (C % 8 == 0) return piece ^ (row & 7);
  return piece ^ ((row >> 1) & 3);
}

template <int DK, int DV>
__global__ void __launch_bounds__(SG_THREADS)
sigmoid_mma_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_stride, __nv_bfloat16* __restrict__ out,
                   int64_t out_stride, float* __restrict__ partial, int64_t partial_stride,
                   const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
                   const int* __restrict__ cu_q, const int* __restrict__ ctx_lens, const int* __restrict__ slots,
                   const float* __restrict__ head_bias, int hq, int hkv, int gp, int block_size, int num_pages,
                   float half_scale, int splits, int tiles_per_split, int* __restrict__ status) {
  constexpr int CK = DK / 8, CV = DV / 8;
  constexpr int K_BYTES = BN * DK * 2, V_BYTES = BN * DV * 2;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* q_sm = smem_raw;                       // [BM][DK]
  unsigned char* kv_sm = smem_raw + BM * DK * 2;        // [2 stages][K [BN][DK] | V [BN][DV]]

  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.z;
  const int group = hq / hkv;
  const int tiles_per_kv = group / gp;
  const int kvh = blockIdx.y / tiles_per_kv;
  const int h0 = kvh * group + (blockIdx.y - kvh * tiles_per_kv) * gp;
  const int qt = BM / gp;
  const int tok_begin = cu_q[r], q_len = cu_q[r + 1] - tok_begin;
  const int n_qtiles = (q_len + qt - 1) / qt;
  const int split = blockIdx.x % splits;
  const int xt = blockIdx.x / splits;
  if (xt >= n_qtiles) return;
  const int qtile = n_qtiles - 1 - xt;                  // longest rows first
  const int t0 = qtile * qt;
  const int t_count = min(qt, q_len - t0);
  const int ctx = ctx_lens[r];
  const int* bt = block_table + (int64_t)slots[r] * bt_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, t4 = lane & 3;

  const int pos_first = ctx + t0, pos_last = ctx + t0 + t_count - 1;
  int tile_first = 0, tile_last = pos_last / BN;
  if (splits > 1) {
    tile_first = split * tiles_per_split;
    tile_last = min(tile_last, tile_first + tiles_per_split - 1);
  }

  const int64_t page_elems = (int64_t)hkv * block_size * (DK + DV);
  const int64_t v_region = (int64_t)hkv * block_size * DK;

  int qpos[2];
  bool row_ok[2];
  float bias2[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = warp * 16 + g8 + 8 * i;
    const int tl = rr / gp;
    row_ok[i] = tl < t_count;
    qpos[i] = pos_first + tl;
    bias2[i] = (head_bias ? head_bias[h0 + rr - tl * gp] : 0.f) * 0.5f;
  }
  float o[DV / 8][4];
#pragma unroll
  for (int nd = 0; nd < DV / 8; ++nd)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nd][e] = 0.f;

  if (tile_first <= tile_last) {
    for (int idx = threadIdx.x; idx < BM * CK; idx += SG_THREADS) {
      const int rr = idx / CK, piece = idx - rr * CK;
      const int tl = rr / gp, g = rr - tl * gp;
      const bool ok = tl < t_count;
      const __nv_bfloat16* src =
          q + (int64_t)(tok_begin + t0 + (ok ? tl : 0)) * q_stride + (int64_t)(h0 + g) * DK + piece * 8;
      cp_async16(smem_u32(q_sm + (rr * CK + swz<CK>(rr, piece)) * 16), src, ok);
    }
    auto load_kv = [&](int tile, int stage) {
      unsigned char* k_dst = kv_sm + stage * (K_BYTES + V_BYTES);
      unsigned char* v_dst = k_dst + K_BYTES;
      for (int idx = threadIdx.x; idx < BN * (CK + CV); idx += SG_THREADS) {
        const int row = idx / (CK + CV), piece = idx - row * (CK + CV);
        const int key = tile * BN + row;
        bool ok = key <= pos_last;
        int page = 0;
        if (ok) {
          page = bt[key / block_size];
          if (page < 0 || page >= num_pages) {
            atomicOr(status, GLLM_STATUS_PAGE_RANGE);
            ok = false;
            page = 0;
          }
        }
        const int off = key % block_size;
        if (piece < CK) {
          const __nv_bfloat16* src = cache + (int64_t)page * page_elems + ((int64_t)kvh * block_size + off) * DK + piece * 8;
          cp_async16(smem_u32(k_dst + (row * CK + swz<CK>(row, piece)) * 16), ok ? src : cache, ok);
        } else {
          const int pv = piece - CK;
          const __nv_bfloat16* src =
              cache + (int64_t)page * page_elems + v_region + ((int64_t)kvh * block_size + off) * DV + pv * 8;
          cp_async16(smem_u32(v_dst + (row * CV + swz<CV>(row, pv)) * 16), ok ? src : cache, ok);
        }
      }
    };
    load_kv(tile_first, 0);
    cp_async_commit();
    uint32_t qf[DK / 16][4];

    for (int tile = tile_first; tile <= tile_last; ++tile) {
      const int stage = (tile - tile_first) & 1;
      if (tile < tile_last) {
        load_kv(tile + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      if (tile == tile_first) {
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
          const int mat = lane >> 3, rl = lane & 7;
          const int row = warp * 16 + (mat & 1) * 8 + rl;
          const int piece = 2 * ks + (mat >> 1);
          ldmatrix_x4(qf[ks], smem_u32(q_sm + (row * CK + swz<CK>(row, piece)) * 16));
        }
      }
      const unsigned char* k_sm = kv_sm + stage * (K_BYTES + V_BYTES);
      const unsigned char* v_sm = k_sm + K_BYTES;
      const int kv0 = tile * BN;

      float s[BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          const int mat = lane >> 3, rl = lane & 7;
          const int row = np * 16 + (mat >> 1) * 8 + rl;
          const int piece = 2 * ks + (mat & 1);
          uint32_t b[4];
          ldmatrix_x4(b, smem_u32(k_sm + (row * CK + swz<CK>(row, piece)) * 16));
          mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
          mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
        }
      }
      // ---- weights: sigmoid(x) = 0.5 + 0.5 tanh(x / 2), x = s * scale + bias (one special-function
      // instruction per score; its error is below the bf16 rounding of the weight); hidden keys weigh nothing
      const bool need_mask = (kv0 + BN - 1 > pos_first) || (t_count < qt);
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          float p;
          asm("tanh.approx.f32 %0, %1;" : "=f"(p) : "f"(fmaf(s[nt][e], half_scale, bias2[i])));
          p = fmaf(0.5f, p, 0.5f);
          if (need_mask) {
            const int key = kv0 + nt * 8 + 2 * t4 + (e & 1);
            if (!row_ok[i] || key > qpos[i]) p = 0.f;
          }
          s[nt][e] = p;
        }
      // ---- O += P V
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int nd2 = 0; nd2 < DV / 16; ++nd2) {
          const int mat = lane >> 3, rl = lane & 7;
          const int row = kk * 16 + (mat & 1) * 8 + rl;
          const int piece = 2 * nd2 + (mat >> 1);
          uint32_t b[4];
          ldmatrix_x4_trans(b, smem_u32(v_sm + (row * CV + swz<CV>(row, piece)) * 16));
          mma_bf16(o[2 * nd2], a, b[0], b[1]);
          mma_bf16(o[2 * nd2 + 1], a, b[2], b[3]);
        }
      }
      __syncthreads();
    }
  }
  // ---- store
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!row_ok[i]) continue;
    const int rr = warp * 16 + g8 + 8 * i;
    const int tl = rr / gp, g = rr - tl * gp;
    const int64_t token = tok_begin + t0 + tl;
    if (splits > 1) {
      float* dst = partial + (int64_t)split * partial_stride + token * (int64_t)hq * DV + (int64_t)(h0 + g) * DV;
#pragma unroll
      for (int nd = 0; nd < DV / 8; ++nd)
        *reinterpret_cast<float2*>(dst + nd * 8 + 2 * t4) = make_float2(o[nd][2 * i], o[nd][2 * i + 1]);
    } else {
      __nv_bfloat16* dst = out + token * out_stride + (int64_t)(h0 + g) * DV;
#pragma unroll
      for (int nd = 0; nd < DV / 8; ++nd)
        *reinterpret_cast<__nv_bfloat162*>(dst + nd * 8 + 2 * t4) = __floats2bfloat162_rn(o[nd][2 * i], o[nd][2 * i + 1]);
    }
  }
}

template <int DK, int DV>
int sigmoid_mma_launch(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out, int64_t out_stride, float* partial,
                       int64_t partial_stride, const __nv_bfloat16* cache, const int* block_table, int bt_stride,
                       const int* cu_q, const int* ctx_lens, const int* slots, const float* head_bias,
                       int num_requests, int max_q_len, int hq, int hkv, int block_size, int num_pages, float scale,
                       int splits, int tiles_per_split, int* status, cudaStream_t stream) {
  const int group = hq / hkv;
  const int gp = (group <= BM && BM % group == 0) ? group : 1;
  const int qt = BM / gp;
  const size_t smem = (size_t)BM * DK * 2 + 2 * (size_t)BN * (DK + DV) * 2;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(sigmoid_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(((max_q_len + qt - 1) / qt) * splits, hkv * (group / gp), num_requests);
  return gllm_launch(sigmoid_mma_kernel<DK, DV>, grid, dim3(SG_THREADS), smem, stream, q, q_stride, out, out_stride,
                     partial, partial_stride, cache, block_table, bt_stride, cu_q, ctx_lens, slots, head_bias, hq, hkv,
                     gp, block_size, num_pages, 0.5f * scale, splits, tiles_per_split, status);
}
}  // namespace

GLLM_API int gllm_attention_sigmoid_mma_supports(int dk, int dv) {
  auto ok = [](int d) { return d == 32 || d == 64 || d == 96 || d == 128; };
  return ok(dk) && ok(dv);
}

// How many query tokens one CTA covers (the caller sizes its split decision with it).
GLLM_API int gllm_attention_sigmoid_mma_tokens_per_tile(int hq, int hkv) {
  const int group = hq / hkv;
  return (group <= BM && BM % group == 0) ? BM / group : BM;
}

GLLM_API int gllm_attention_sigmoid_mma(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out, int64_t out_stride,
                                        float* partial, int64_t partial_stride, const __nv_bfloat16* cache,
                                        const int* block_table, int bt_stride, const int* cu_q, const int* ctx_lens,
                                        const int* slots, const float* head_bias, int num_requests, int max_q_len,
                                        int hq, int hkv, int dk, int dv, int block_size, int num_pages, float scale,
                                        int splits, int tiles_per_split, int* status, cudaStream_t stream) {
  if (num_requests <= 0 || max_q_len <= 0) return 0;
  if (hq <= 0 || hkv <= 0 || hq % hkv || num_requests > 65535 || (q_stride % 8) || (out_stride % 2) || splits < 1 ||
      (splits > 1 && (partial == nullptr || tiles_per_split < 1)))
    return (int)cudaErrorInvalidValue;
#define GLLM_SG(A, B)                                                                                                \
  if (dk == A && dv == B)                                                                                            \
    return sigmoid_mma_launch<A, B>(q, q_stride, out, out_stride, partial, partial_stride, cache, block_table,       \
                                    bt_stride, cu_q, ctx_lens, slots, head_bias, num_requests, max_q_len, hq, hkv,   \
                                    block_size, num_pages, scale, splits, tiles_per_split, status, stream);
#define GLLM_SG_ROW(A) GLLM_SG(A, 32) GLLM_SG(A, 64) GLLM_SG(A, 96) GLLM_SG(A, 128)
  GLLM_SG_ROW(32) GLLM_SG_ROW(64) GLLM_SG_ROW(96) GLLM_SG_ROW(128)
#undef GLLM_SG_ROW
#undef GLLM_SG
  return (int)cudaErrorInvalidValue;
}
