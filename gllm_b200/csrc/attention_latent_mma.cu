// Latent attention of the bf16 path on the tensor cores: softmax attention of every (token, head) over its
// request's cached [c ; kr] vectors (RANK + ROT numbers per token, one "key head" for all query heads), the
// values being the first RANK columns of the keys (see attention_latent.cu for the algebra).
//
// One CTA of 8 warps owns 64 rows = (64 / H') tokens x H' heads (H' = all heads when there are at most 64 of
// them, so that a key tile is fetched once for all heads of a token).  The rows' queries [qa ; qr] stay in
// shared memory; key tiles of 32 tokens come page by page with cp.async in two stages and serve both products:
//   S = Q K^T     warp w: rows 16 (w & 3) .., keys 16 (w >> 2) ..           mma.sync m16n8k16, fp32
//   softmax       four threads per row over the tile's 32 scores (fp32, base 2): running maximum and sum,
//                 probabilities to shared memory as bf16, the rescaling factor of the row beside them
//   O = O c + P V warp w: rows 16 (w & 3) .., columns (w >> 2) RANK / 2 ..   V = the tile's first RANK columns
// Key tiles are aligned to absolute positions, so a token's result does not depend on how its request was cut
// into steps.  With `splits` > 1 a CTA visits the key tiles [s * tiles_per_split, (s + 1) * tiles_per_split)
// only and leaves (unnormalised O, maximum, sum) in fp32; latent_merge combines the ranges (single decoded
// tokens over a long context get enough CTAs that way).  The per-head sigmoid gate multiplies the result.
#include "mma_utils.cuh"

namespace {
constexpr int LM_BM = 64, LM_BN = 32, LM_THREADS = 256;
constexpr float LOG2E = 1.4426950408889634f;

template <int C>
__device__ __forceinline__ int lswz(int row, int piece) {
  if (C % 8 == 0) return piece ^ (row & 7);
  return piece ^ ((row >> 1) & 3);
}

__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}

// FEW: no CTA of the launch has more than 16 rows (single tokens of up to 16 heads).  The eight warps then share
// the one block of 16 rows: in S = Q K^T a warp takes 8 of the tile's keys and one half of the width (the halves
// are added by the softmax threads), in P V it takes every eighth block of 16 value columns.  The accumulators are
// a quarter of the general form's, so that two CTAs fit an SM.
template <int RANK, int ROT, bool FEW>
__global__ void __launch_bounds__(LM_THREADS, FEW ? 2 : 1)
latent_mma_kernel(const __nv_bfloat16* __restrict__ qa, int64_t qa_stride, const __nv_bfloat16* __restrict__ qr,
                  int64_t qr_stride, int qr_head, const __nv_bfloat16* __restrict__ gate, int64_t gate_stride,
                  __nv_bfloat16* __restrict__ out, int64_t out_stride, float* __restrict__ part_o,
                  float* __restrict__ part_ml, const __nv_bfloat16* __restrict__ cache,
                  const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q,
                  const int* __restrict__ ctx_lens, const int* __restrict__ slots, int n_tokens, int heads, int gp,
                  int qt, int q_rows, int block_size, int num_pages, float scale_log2, int splits,
                  int tiles_per_split, int* __restrict__ status) {
  constexpr int DK = RANK + ROT, CK = DK / 8, CR = RANK / 8, CP = LM_BN / 8;
  constexpr int K_BYTES = LM_BN * DK * 2;
  // q_rows: a multiple of 16 that no CTA of the launch uses more rows than (16 for single tokens of 16 heads: the
  // queries then take a quarter of the room and two CTAs fit an SM)
  const int Q_BYTES = q_rows * DK * 2;
  constexpr int S_LD = LM_BN + 2;
  constexpr int NV = FEW ? 2 : RANK / 16;  // n8 tiles of a warp's half of the value columns
  constexpr int PAIRS = RANK / 16;         // FEW: blocks of 16 value columns, dealt out to the warps in turn
  constexpr int MAXP = FEW ? (PAIRS + 7) / 8 : 1;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* q_sm = smem_raw;                                   // [q_rows][DK] bf16
  unsigned char* k_sm0 = q_sm + Q_BYTES;                            // 2 x [32][DK] bf16
  float* s_sm = reinterpret_cast<float*>(k_sm0 + 2 * K_BYTES);      // [64][S_LD]
  unsigned char* p_sm = reinterpret_cast<unsigned char*>(s_sm + LM_BM * S_LD);   // [64][32] bf16
  float* corr_sm = reinterpret_cast<float*>(p_sm + LM_BM * LM_BN * 2);           // [64] rescale, then [64] m, [64] l
  float* m_sm = corr_sm + LM_BM;
  float* l_sm = m_sm + LM_BM;

  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.z;
  const int h0 = blockIdx.y * gp;
  const int tok_begin = cu_q[r], q_len = cu_q[r + 1] - tok_begin;
  const int n_qtiles = (q_len + qt - 1) / qt;
  const int split = blockIdx.x % splits;
  const int xt = blockIdx.x / splits;
  if (xt >= n_qtiles) return;
  const int qtile = n_qtiles - 1 - xt;                  // longest rows first
  const int t0 = qtile * qt;
  const int t_count = min(qt, q_len - t0);
  const int rows_used = t_count * gp;
  const int ctx = ctx_lens[r];
  const int* bt = block_table + (int64_t)slots[r] * bt_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int rb = (warp & 3) * 16, half = warp >> 2;

  const int pos_first = ctx + t0, pos_last = ctx + t0 + t_count - 1;
  int tile_first = 0, tile_last = pos_last / LM_BN;
  if (splits > 1) {
    tile_first = split * tiles_per_split;
    tile_last = min(tile_last, tile_first + tiles_per_split - 1);
  }

  // softmax role: thread t owns row t >> 2, keys 8 (t & 3) .. of every tile
  const int srow = threadIdx.x >> 2, squart = threadIdx.x & 3;
  const int s_tl = srow / gp;
  const bool s_ok = srow < rows_used;
  const int s_qpos = pos_first + s_tl;
  float m_run = -INFINITY, l_run = 0.f;

  float o[NV][4];
#pragma unroll
  for (int nd = 0; nd < NV; ++nd)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nd][e] = 0.f;
  float of[MAXP][2][4];
#pragma unroll
  for (int j = 0; j < MAXP; ++j)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) of[j][nt][e] = 0.f;

  if (tile_first <= tile_last) {
    {   // four threads a row: one division per thread
      const int rr = threadIdx.x >> 2;
      if (rr < q_rows) {
        const int tl = rr / gp, g = rr - tl * gp;
        const bool ok = rr < rows_used;
        const int64_t token = tok_begin + t0 + (ok ? tl : 0);
        const __nv_bfloat16* a_src = qa + token * qa_stride + (int64_t)(h0 + (ok ? g : 0)) * RANK;
        const __nv_bfloat16* r_src = qr + token * qr_stride + (int64_t)(h0 + (ok ? g : 0)) * qr_head;
        for (int piece = threadIdx.x & 3; piece < CK; piece += 4)
          cp_async16(smem_u32(q_sm + (rr * CK + lswz<CK>(rr, piece)) * 16),
                     piece < CR ? a_src + piece * 8 : r_src + (piece - CR) * 8, ok);
      }
    }
    auto load_k = [&](int tile, int stage) {     // eight threads a key: one look-up of its page per thread
      unsigned char* dst = k_sm0 + stage * K_BYTES;
      const int row = threadIdx.x >> 3;
      const int key = tile * LM_BN + row;
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
      const __nv_bfloat16* src = ok ? cache + ((int64_t)page * block_size + key % block_size) * DK : cache;
      for (int piece = threadIdx.x & 7; piece < CK; piece += 8)
        cp_async16(smem_u32(dst + (row * CK + lswz<CK>(row, piece)) * 16), ok ? src + piece * 8 : cache, ok);
    };
    load_k(tile_first, 0);
    cp_async_commit();

    for (int tile = tile_first; tile <= tile_last; ++tile) {
      const int stage = (tile - tile_first) & 1;
      if (tile < tile_last) {
        load_k(tile + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const unsigned char* k_sm = k_sm0 + stage * K_BYTES;
      const int kv0 = tile * LM_BN;
      // ---- S = Q K^T: 16 rows x 16 keys per warp (a warp whose rows are all unused sits the products out);
      // even and odd steps along the width add into accumulators of their own: two shorter chains
      if constexpr (FEW) {
        float s2[2][4];
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 4; ++e) s2[c][e] = 0.f;
        constexpr int KS_HALF = DK / 32;
        const int mat = lane >> 3, rl = lane & 7;
        const int arow = (mat & 1) * 8 + rl;
        const int key8 = (warp & 3) * 8, kh = warp >> 2;
        const int brow = key8 + rl;
        auto step = [&](int k, float (&acc)[4]) {
          const int ks = kh * KS_HALF + k;
          uint32_t a[4], b0, b1;
          ldmatrix_x4(a, smem_u32(q_sm + (arow * CK + lswz<CK>(arow, 2 * ks + (mat >> 1))) * 16));
          ldmatrix_x2(b0, b1, smem_u32(k_sm + (brow * CK + lswz<CK>(brow, 2 * ks + (mat & 1))) * 16));
          mma_bf16(acc, a, b0, b1);
        };
#pragma unroll 2
        for (int k = 0; k + 1 < KS_HALF; k += 2) {       // two chains of additions
          step(k, s2[0]);
          step(k + 1, s2[1]);
        }
        if (KS_HALF & 1) step(KS_HALF - 1, s2[0]);
#pragma unroll
        for (int i = 0; i < 2; ++i)
          *reinterpret_cast<float2*>(s_sm + (kh * 16 + g8 + 8 * i) * S_LD + key8 + 2 * t4) =
              make_float2(s2[0][2 * i] + s2[1][2 * i], s2[0][2 * i + 1] + s2[1][2 * i + 1]);
      } else if (rb < rows_used) {
        float s[2][2][4];
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[c][nt][e] = 0.f;
        const int mat = lane >> 3, rl = lane & 7;
        const int arow = rb + (mat & 1) * 8 + rl;
        const int brow = half * 16 + (mat >> 1) * 8 + rl;
#pragma unroll 4
        for (int ks = 0; ks < DK / 16; ++ks) {
          uint32_t a[4], b[4];
          ldmatrix_x4(a, smem_u32(q_sm + (arow * CK + lswz<CK>(arow, 2 * ks + (mat >> 1))) * 16));
          ldmatrix_x4(b, smem_u32(k_sm + (brow * CK + lswz<CK>(brow, 2 * ks + (mat & 1))) * 16));
          mma_bf16(s[ks & 1][0], a, b[0], b[1]);
          mma_bf16(s[ks & 1][1], a, b[2], b[3]);
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int i = 0; i < 2; ++i)
            *reinterpret_cast<float2*>(s_sm + (rb + g8 + 8 * i) * S_LD + half * 16 + nt * 8 + 2 * t4) =
                make_float2(s[0][nt][2 * i] + s[1][nt][2 * i], s[0][nt][2 * i + 1] + s[1][nt][2 * i + 1]);
      }
      __syncthreads();
      // ---- softmax of the tile: four threads a row
      if (!FEW || warp < 2) {
        float v[8];
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int key = kv0 + squart * 8 + e;
          float x = s_sm[srow * S_LD + squart * 8 + e];
          if (FEW) x += s_sm[(16 + srow) * S_LD + squart * 8 + e];      // the other half of the width
          x *= scale_log2;
          v[e] = (s_ok && key <= s_qpos) ? x : -INFINITY;
          mx = fmaxf(mx, v[e]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        float sum = 0.f;
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float p0 = (m_new == -INFINITY) ? 0.f : fast_exp2(v[e] - m_new);
          const float p1 = (m_new == -INFINITY) ? 0.f : fast_exp2(v[e + 1] - m_new);
          sum += p0 + p1;
          packed[e >> 1] = pack_bf16(p0, p1);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float corr = (m_run == -INFINITY) ? ((m_new == -INFINITY) ? 1.f : 0.f) : fast_exp2(m_run - m_new);
        l_run = l_run * corr + sum;
        m_run = m_new;
        *reinterpret_cast<uint4*>(p_sm + (srow * CP + lswz<CP>(srow, squart)) * 16) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
        if (squart == 0) corr_sm[srow] = corr;
      }
      __syncthreads();
      // ---- O = O * corr + P V: 16 rows x RANK / 2 columns per warp
      if constexpr (FEW) {
        const float c0 = corr_sm[g8], c1 = corr_sm[g8 + 8];
#pragma unroll
        for (int j = 0; j < MAXP; ++j)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            of[j][nt][0] *= c0; of[j][nt][1] *= c0; of[j][nt][2] *= c1; of[j][nt][3] *= c1;
          }
        const int mat = lane >> 3, rl = lane & 7;
#pragma unroll
        for (int kk = 0; kk < LM_BN / 16; ++kk) {
          uint32_t a[4];
          const int arow = (mat & 1) * 8 + rl;
          ldmatrix_x4(a, smem_u32(p_sm + (arow * CP + lswz<CP>(arow, 2 * kk + (mat >> 1))) * 16));
#pragma unroll
          for (int j = 0; j < MAXP; ++j) {
            const int pair = warp + 8 * j;
            if (pair < PAIRS) {
              const int row = kk * 16 + (mat & 1) * 8 + rl;
              uint32_t b[4];
              ldmatrix_x4_trans(b, smem_u32(k_sm + (row * CK + lswz<CK>(row, 2 * pair + (mat >> 1))) * 16));
              mma_bf16(of[j][0], a, b[0], b[1]);
              mma_bf16(of[j][1], a, b[2], b[3]);
            }
          }
        }
      } else if (rb < rows_used) {
        const float c0 = corr_sm[rb + g8], c1 = corr_sm[rb + g8 + 8];
#pragma unroll
        for (int nd = 0; nd < NV; ++nd) {
          o[nd][0] *= c0; o[nd][1] *= c0; o[nd][2] *= c1; o[nd][3] *= c1;
        }
        const int mat = lane >> 3, rl = lane & 7;
#pragma unroll
        for (int kk = 0; kk < LM_BN / 16; ++kk) {
          uint32_t a[4];
          const int arow = rb + (mat & 1) * 8 + rl;
          ldmatrix_x4(a, smem_u32(p_sm + (arow * CP + lswz<CP>(arow, 2 * kk + (mat >> 1))) * 16));
#pragma unroll
          for (int nd2 = 0; nd2 < NV / 2; ++nd2) {
            const int row = kk * 16 + (mat & 1) * 8 + rl;
            const int piece = half * (CR / 2) + 2 * nd2 + (mat >> 1);
            uint32_t b[4];
            ldmatrix_x4_trans(b, smem_u32(k_sm + (row * CK + lswz<CK>(row, piece)) * 16));
            mma_bf16(o[2 * nd2], a, b[0], b[1]);
            mma_bf16(o[2 * nd2 + 1], a, b[2], b[3]);
          }
        }
      }
      __syncthreads();
    }
  }
  if (squart == 0) {
    m_sm[srow] = m_run;
    l_sm[srow] = l_run;
  }
  __syncthreads();
  // ---- store
  if constexpr (FEW) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int rr = g8 + 8 * i;
      if (rr >= rows_used) continue;
      const int tl = rr / gp, g = rr - tl * gp;
      const int64_t token = tok_begin + t0 + tl;
      const int head = h0 + g;
      float mult = 1.f;
      if (splits == 1) {
        const float l = l_sm[rr];
        mult = l > 0.f ? 1.0f / l : 0.f;
        if (gate) mult *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[token * gate_stride + head])));
      } else if (warp == 0 && t4 == 0) {
        float* ml = part_ml + (((int64_t)split * n_tokens + token) * heads + head) * 2;
        ml[0] = m_sm[rr];
        ml[1] = l_sm[rr];
      }
#pragma unroll
      for (int j = 0; j < MAXP; ++j) {
        const int pair = warp + 8 * j;
        if (pair >= PAIRS) continue;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int col = pair * 16 + nt * 8 + 2 * t4;
          if (splits > 1)
            *reinterpret_cast<float2*>(part_o + (((int64_t)split * n_tokens + token) * heads + head) * RANK + col) =
                make_float2(of[j][nt][2 * i], of[j][nt][2 * i + 1]);
          else
            *reinterpret_cast<__nv_bfloat162*>(out + token * out_stride + (int64_t)head * RANK + col) =
                __floats2bfloat162_rn(of[j][nt][2 * i] * mult, of[j][nt][2 * i + 1] * mult);
        }
      }
    }
  } else {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = rb + g8 + 8 * i;
    if (rr >= rows_used) continue;
    const int tl = rr / gp, g = rr - tl * gp;
    const int64_t token = tok_begin + t0 + tl;
    const int head = h0 + g;
    const int col0 = half * (RANK / 2);
    if (splits > 1) {
      float* dst = part_o + (((int64_t)split * n_tokens + token) * heads + head) * RANK + col0;
#pragma unroll
      for (int nd = 0; nd < NV; ++nd)
        *reinterpret_cast<float2*>(dst + nd * 8 + 2 * t4) = make_float2(o[nd][2 * i], o[nd][2 * i + 1]);
      if (half == 0 && t4 == 0) {
        float* ml = part_ml + (((int64_t)split * n_tokens + token) * heads + head) * 2;
        ml[0] = m_sm[rr];
        ml[1] = l_sm[rr];
      }
    } else {
      const float l = l_sm[rr];
      float mult = l > 0.f ? 1.0f / l : 0.f;
      if (gate) mult *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[token * gate_stride + head])));
      __nv_bfloat16* dst = out + token * out_stride + (int64_t)head * RANK + col0;
#pragma unroll
      for (int nd = 0; nd < NV; ++nd)
        *reinterpret_cast<__nv_bfloat162*>(dst + nd * 8 + 2 * t4) =
            __floats2bfloat162_rn(o[nd][2 * i] * mult, o[nd][2 * i + 1] * mult);
    }
  }
  }
}

// Combines the ranges of latent_mma_kernel: out = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s, times the gate.
// One block per (token, head).
__global__ void __launch_bounds__(512)
latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                    const __nv_bfloat16* __restrict__ gate, int64_t gate_stride, __nv_bfloat16* __restrict__ out,
                    int64_t out_stride, int n_tokens, int heads, int rank, int splits) {
  __shared__ float w_s[64];          // weight of every range: 2^(m_s - m) / l, times the gate
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x / heads, head = blockIdx.x - token * heads;
  const int64_t base = (int64_t)token * heads + head, step = (int64_t)n_tokens * heads;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float ms[2], ls[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int s = lane + 32 * k;
      ms[k] = s < splits ? part_ml[(base + s * step) * 2] : -INFINITY;
      ls[k] = s < splits ? part_ml[(base + s * step) * 2 + 1] : 0.f;
    }
    const float m = warp_max(fmaxf(ms[0], ms[1]));
    float e[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) e[k] = ms[k] == -INFINITY ? 0.f : fast_exp2(ms[k] - m);
    const float l = warp_sum(e[0] * ls[0] + e[1] * ls[1]);
    float mult = l > 0.f ? 1.0f / l : 0.f;
    if (gate) mult *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[token * gate_stride + head])));
    w_s[lane] = e[0] * mult;
    w_s[lane + 32] = e[1] * mult;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float acc = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 16) {          // sixteen loads in flight, then the additions in ascending order
      float v[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) v[k] = s0 + k < splits ? __ldcg(part_o + (base + (s0 + k) * step) * rank + c) : 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k) acc = fmaf(w_s[(s0 + k) & 63], v[k], acc);
    }
    out[token * out_stride + (int64_t)head * rank + c] = __float2bfloat16_rn(acc);
  }
}

// ------------------------------------------------------------------ one small product per head
// out[n, h, j] = sum_i x[n, h, i] * w[h, j, i] (the same job as head_linear in attention_latent.cu) on the tensor
// cores: a CTA of 4 warps owns 64 tokens x 64 outputs of one head, operand tiles of 32 columns come with
// cp.async in two stages, every warp multiplies its 16 tokens by all 64 outputs.  I a multiple of 8.
constexpr int HM_BM = 64, HM_BN = 64, HM_BK = 32, HM_THREADS = 128;

__global__ void __launch_bounds__(HM_THREADS)
head_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_stride, int x_head,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, int64_t out_stride,
                       int out_head, int n_tokens, int I, int J) {
  constexpr int C = HM_BK / 8;
  __shared__ __align__(128) unsigned char x_sm[2][HM_BM * HM_BK * 2];
  __shared__ __align__(128) unsigned char w_sm[2][HM_BN * HM_BK * 2];
  pdl_trigger();
  const int m0 = blockIdx.y * HM_BM, n0 = blockIdx.x * HM_BN, h = blockIdx.z;
  const __nv_bfloat16* xh = x + (int64_t)h * x_head;
  const __nv_bfloat16* wh = w + (int64_t)h * J * I;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, t4 = lane & 3;
  auto load_w = [&](int k0, int stage) {
    for (int idx = threadIdx.x; idx < HM_BN * C; idx += HM_THREADS) {
      const int row = idx / C, piece = idx - row * C;
      const bool ok = n0 + row < J && k0 + piece * 8 < I;
      cp_async16(smem_u32(w_sm[stage] + (row * C + lswz<C>(row, piece)) * 16),
                 ok ? wh + (int64_t)(n0 + row) * I + k0 + piece * 8 : wh, ok);
    }
  };
  auto load_x = [&](int k0, int stage) {
    for (int idx = threadIdx.x; idx < HM_BM * C; idx += HM_THREADS) {
      const int row = idx / C, piece = idx - row * C;
      const bool ok = m0 + row < n_tokens && k0 + piece * 8 < I;
      cp_async16(smem_u32(x_sm[stage] + (row * C + lswz<C>(row, piece)) * 16),
                 ok ? xh + (int64_t)(m0 + row) * x_stride + k0 + piece * 8 : xh, ok);
    }
  };
  load_w(0, 0);              // the weight does not depend on the kernel before this one
  pdl_wait();
  load_x(0, 0);
  cp_async_commit();
  float acc[HM_BN / 8][4];
#pragma unroll
  for (int nt = 0; nt < HM_BN / 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
  const int steps = (I + HM_BK - 1) / HM_BK;
  const int mat = lane >> 3, rl = lane & 7;
  for (int it = 0; it < steps; ++it) {
    const int stage = it & 1;
    if (it + 1 < steps) {
      load_w((it + 1) * HM_BK, stage ^ 1);
      load_x((it + 1) * HM_BK, stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < HM_BK / 16; ++ks) {
      uint32_t a[4];
      const int arow = warp * 16 + (mat & 1) * 8 + rl;
      ldmatrix_x4(a, smem_u32(x_sm[stage] + (arow * C + lswz<C>(arow, 2 * ks + (mat >> 1))) * 16));
#pragma unroll
      for (int np = 0; np < HM_BN / 16; ++np) {
        uint32_t b[4];
        const int brow = np * 16 + (mat >> 1) * 8 + rl;
        ldmatrix_x4(b, smem_u32(w_sm[stage] + (brow * C + lswz<C>(brow, 2 * ks + (mat & 1))) * 16));
        mma_bf16(acc[2 * np], a, b[0], b[1]);
        mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + warp * 16 + g8 + 8 * i;
    if (m >= n_tokens) continue;
    __nv_bfloat16* dst = out + (int64_t)m * out_stride + (int64_t)h * out_head;
#pragma unroll
    for (int nt = 0; nt < HM_BN / 8; ++nt) {
      const int c = n0 + nt * 8 + 2 * t4;
      if (c + 1 < J) *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(acc[nt][2 * i], acc[nt][2 * i + 1]);
      else if (c < J) dst[c] = __float2bfloat16_rn(acc[nt][2 * i]);
    }
  }
}

template <int RANK, int ROT>
size_t latent_mma_smem(int q_rows) {
  return (size_t)q_rows * (RANK + ROT) * 2 + 2 * (size_t)LM_BN * (RANK + ROT) * 2 + (size_t)LM_BM * (LM_BN + 2) * 4 +
         (size_t)LM_BM * LM_BN * 2 + 3 * LM_BM * 4;
}

template <int RANK, int ROT>
int latent_mma_launch(const __nv_bfloat16* qa, int64_t qa_stride, const __nv_bfloat16* qr, int64_t qr_stride,
                      int qr_head, const __nv_bfloat16* gate, int64_t gate_stride, __nv_bfloat16* out,
                      int64_t out_stride, float* part_o, float* part_ml, const __nv_bfloat16* cache,
                      const int* block_table, int bt_stride, const int* cu_q, const int* ctx_lens, const int* slots,
                      int num_requests, int max_q_len, int n_tokens, int heads, int block_size, int num_pages,
                      float scale, int splits, int tiles_per_split, int* status, cudaStream_t stream) {
  const int gp = heads <= LM_BM ? heads : 1;
  const int qt = LM_BM / gp;
  const int rows_most = (max_q_len < qt ? max_q_len : qt) * gp;
  const int q_rows = rows_most >= LM_BM ? LM_BM : ((rows_most + 15) / 16) * 16;
  const size_t smem = latent_mma_smem<RANK, ROT>(q_rows);
  static bool attr_set = false;
  if (!attr_set && latent_mma_smem<RANK, ROT>(LM_BM) > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(latent_mma_kernel<RANK, ROT, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)latent_mma_smem<RANK, ROT>(LM_BM));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(latent_mma_kernel<RANK, ROT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)latent_mma_smem<RANK, ROT>(16));
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid(((max_q_len + qt - 1) / qt) * splits, heads / gp, num_requests);
  auto kernel = q_rows == 16 ? latent_mma_kernel<RANK, ROT, true> : latent_mma_kernel<RANK, ROT, false>;
  int code = gllm_launch(kernel, grid, dim3(LM_THREADS), smem, stream, qa, qa_stride, qr,
                         qr_stride, qr_head, gate, gate_stride, out, out_stride, part_o, part_ml, cache, block_table,
                         bt_stride, cu_q, ctx_lens, slots, n_tokens, heads, gp, qt, q_rows, block_size, num_pages,
                         scale * LOG2E, splits, tiles_per_split, status);
  if (code != 0 || splits <= 1) return code;
  return gllm_launch(latent_merge_kernel, dim3((unsigned)(n_tokens * heads)), dim3(RANK >= 512 ? 512 : 256), 0, stream,
                     (const float*)part_o, (const float*)part_ml, gate, gate_stride, out, out_stride, n_tokens, heads,
                     RANK, splits);
}
}  // namespace

#define GLLM_LATENT_SIZES(X) X(64, 32) X(64, 64) X(96, 32) X(128, 32) X(128, 64) X(256, 32) X(256, 64) X(512, 64)

GLLM_API int gllm_attention_latent_mma_supports(int rank, int rot) {
#define GLLM_LM_OK(A, B) if (rank == A && rot == B) return 1;
  GLLM_LATENT_SIZES(GLLM_LM_OK)
#undef GLLM_LM_OK
  return 0;
}

// Query tokens per CTA (the caller sizes its split decision with it).
GLLM_API int gllm_attention_latent_mma_tokens_per_tile(int heads) { return heads <= LM_BM ? LM_BM / heads : LM_BM; }

GLLM_API int gllm_attention_latent_mma(const __nv_bfloat16* qa, int64_t qa_stride, const __nv_bfloat16* qr,
                                       int64_t qr_stride, int qr_head, const __nv_bfloat16* gate,
                                       int64_t gate_stride, __nv_bfloat16* out, int64_t out_stride, float* part_o,
                                       float* part_ml, const __nv_bfloat16* cache, const int* block_table,
                                       int bt_stride, const int* cu_q, const int* ctx_lens, const int* slots,
                                       int num_requests, int max_q_len, int n_tokens, int heads, int rank, int rot,
                                       int block_size, int num_pages, float scale, int splits, int tiles_per_split,
                                       int* status, cudaStream_t stream) {
  if (num_requests <= 0 || max_q_len <= 0) return 0;
  if (heads <= 0 || num_requests > 65535 || (qa_stride % 8) || (qr_stride % 8) || (qr_head % 8) || (out_stride % 2) ||
      splits < 1 || splits > 64 || (splits > 1 && (part_o == nullptr || part_ml == nullptr || tiles_per_split < 1)))
    return (int)cudaErrorInvalidValue;
#define GLLM_LM(A, B)                                                                                              \
  if (rank == A && rot == B)                                                                                       \
    return latent_mma_launch<A, B>(qa, qa_stride, qr, qr_stride, qr_head, gate, gate_stride, out, out_stride,      \
                                   part_o, part_ml, cache, block_table, bt_stride, cu_q, ctx_lens, slots,          \
                                   num_requests, max_q_len, n_tokens, heads, block_size, num_pages, scale, splits, \
                                   tiles_per_split, status, stream);
  GLLM_LATENT_SIZES(GLLM_LM)
#undef GLLM_LM
  return (int)cudaErrorInvalidValue;
}

GLLM_API int gllm_head_linear_mma(const __nv_bfloat16* x, int64_t x_stride, int x_head, const __nv_bfloat16* w,
                                  __nv_bfloat16* out, int64_t out_stride, int out_head, int n_tokens, int heads, int I,
                                  int J, cudaStream_t stream) {
  if (n_tokens <= 0 || heads <= 0) return 0;
  if (I <= 0 || J <= 0 || heads > 65535 || (I % 8) || (x_stride % 8) || (x_head % 8) || (out_stride % 2) ||
      (out_head % 2))
    return (int)cudaErrorInvalidValue;
  const dim3 grid((J + HM_BN - 1) / HM_BN, (n_tokens + HM_BM - 1) / HM_BM, heads);
  if (grid.y > 65535) return (int)cudaErrorInvalidValue;
  return gllm_launch(head_linear_mma_kernel, grid, dim3(HM_THREADS), 0, stream, x, x_stride, x_head, w, out,
                     out_stride, out_head, n_tokens, I, J);
}
