// Flash attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), head dim 128.
//
// One CTA = 128 query rows of one (sequence, head).  Per 128-key tile:
//   S = Q K^T        tcgen05.mma 128x128x16 (both operands K-major, TMA-staged with 128-byte swizzle)
//                    into one of two TMEM score buffers, so the next tile's scores are computed
//                    while this tile's soft-max runs;
//   soft-max         eight warps, two threads per query row (64 key columns each): tcgen05.ld the
//                    row, mask, running max / sum in the exp2 domain, P (bf16) written to shared
//                    memory in the UMMA K-major swizzled layout, O rescaled in TMEM (tcgen05.ld /
//                    tcgen05.st) only when a row maximum moved by more than 2^8;
//   O += P V         tcgen05.mma with V as an MN-major operand straight from its [keys, d] tile.
// Warp roles (320 threads): warps 0-7 soft-max / epilogue (TMEM lane quarter = warp id % 4), warp 8
// TMA producer, warp 9 TMEM allocation + MMA issue.  Causal masking is bottom-right aligned when the
// key sequence is longer than the query sequence, as in the mma.sync kernel of attention.cu,
// which stays the fallback (other head sizes, backward).
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in the status word, skips the
// rest, frees TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>

#include "tcgen05_utils.cuh"

namespace msrl {
namespace fa5 {

using namespace t5;

constexpr int BM = 128, D = 128;
constexpr uint32_t TILE_HALF = 128 * 64 * 2;          // one [128 rows x 64 cols] bf16 swizzled half tile
constexpr uint32_t TILE_BYTES = 2 * TILE_HALF;         // 32 KiB
constexpr uint32_t SMEM_Q = 0;
constexpr uint32_t TMEM_COLS = 512;                    // backward kernels
constexpr uint32_t fwd_smem_bytes(int bn) { return TILE_BYTES + 4u * (2u * bn * 64 * 2) + 128u * bn * 2; }
constexpr int OUT_PITCH = 144;
constexpr int SOFTMAX_WARPS = 8, TMA_WARP = 8, MMA_WARP = 9, THREADS = 320;

enum { ERR_SMEM = 10, ERR_Q = 11, ERR_K = 12, ERR_V = 13, ERR_S = 14, ERR_P = 15, ERR_PV = 16, ERR_EMPTY = 17 };

struct Params {
  __nv_bfloat16* o;
  long long o_stride_t;
  float* lse;
  const int* cu_q;
  const int* cu_k;
  int nh, nkv;
  long long Tq;
  float scale_log2;
  int causal;
  int q_col0, q_group_stride, q_hpg, q_head_stride;    // column of head h inside a row of the Q tensor map
  int k_col0, k_group_stride, k_hpg, k_head_stride;
  int v_col0, v_group_stride, v_hpg, v_head_stride;
  int* error;
};

__device__ __forceinline__ int head_col(int col0, int gs, int hpg, int hs, int h) {
  return col0 + (h / hpg) * gs + (h % hpg) * hs;
}

// BN = keys per tile.  128: one CTA per SM (192 KiB of shared memory, 512 TMEM columns).  64: two
// CTAs per SM (112 KiB, 256 columns each), so that one CTA's soft-max, prologue and epilogue overlap
// the other's tensor work.
template <int BN>
__global__ void __launch_bounds__(THREADS, BN == 128 ? 1 : 2)
fa_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], s_free[2], p_ready, pv_done;
  __shared__ uint32_t tmem_slot;
  constexpr uint32_t KV_HALF = BN * 64 * 2, KV_BYTES = 2 * KV_HALF;
  constexpr uint32_t SMEM_K = TILE_BYTES, SMEM_V = SMEM_K + 2 * KV_BYTES, SMEM_P = SMEM_V + 2 * KV_BYTES;
  constexpr uint32_t TMEM_COLS = BN == 128 ? 512 : 256;      // S0 [0,BN) S1 [BN,2BN) O [2BN, 2BN+128)
  constexpr int HALF = BN / 2, NCH = HALF / 32;              // key columns per soft-max thread

  const int b = blockIdx.z, h = blockIdx.y, mt = blockIdx.x;
  const int q0 = p.cu_q[b], qlen = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], klen = p.cu_k[b + 1] - k0;
  const int m0 = mt * BM;
  if (m0 >= qlen) return;                         // uniform for the CTA, before any allocation
  const int hk = h / (p.nh / p.nkv);
  const int off = klen - qlen;
  int kmax = klen;
  if (p.causal) kmax = min(klen, m0 + BM + off);
  const int n_tiles = kmax > 0 ? (kmax + BN - 1) / BN : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    // the tiles must fit behind the 1024-byte alignment of the dynamic segment (the launch leaves
    // less than a full KiB of slack when two CTAs share an SM)
    uint32_t dyn;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;\n" : "=r"(dyn));
    if ((uint32_t)(smem - smem_raw) + fwd_smem_bytes(BN) > dyn) {
      if (threadIdx.x == 0) atomicCAS(p.error, 0, ERR_SMEM);
      return;
    }
  }
  float (*l_part)[BM] = reinterpret_cast<float (*)[BM]>(smem + SMEM_P);   // used after the last P V product

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], SOFTMAX_WARPS);
    }
    mbar_init(&p_ready, SOFTMAX_WARPS);
    mbar_init(&pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_o = tmem + 2 * BN;

  if (warp == TMA_WARP) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      const int qc = head_col(p.q_col0, p.q_group_stride, p.q_hpg, p.q_head_stride, h);
      const int kc = head_col(p.k_col0, p.k_group_stride, p.k_hpg, p.k_head_stride, hk);
      const int vc = head_col(p.v_col0, p.v_group_stride, p.v_hpg, p.v_head_stride, hk);
      mbar_expect_tx(&q_full, TILE_BYTES);
      tma_load_2d(smem + SMEM_Q, &map_q, &q_full, qc, q0 + m0);
      tma_load_2d(smem + SMEM_Q + TILE_HALF, &map_q, &q_full, qc + 64, q0 + m0);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const uint32_t use = j >> 1;
        if (use > 0) ok = mbar_wait(&k_empty[st], (use - 1) & 1, p.error, ERR_EMPTY);
        if (!ok) break;
        mbar_expect_tx(&k_full[st], KV_BYTES);
        unsigned char* sk = smem + SMEM_K + st * KV_BYTES;
        tma_load_2d(sk, &map_k, &k_full[st], kc, k0 + j * BN);
        tma_load_2d(sk + KV_HALF, &map_k, &k_full[st], kc + 64, k0 + j * BN);
        if (use > 0) ok = mbar_wait(&v_empty[st], (use - 1) & 1, p.error, ERR_EMPTY);
        if (!ok) break;
        mbar_expect_tx(&v_full[st], KV_BYTES);
        unsigned char* sv = smem + SMEM_V + st * KV_BYTES;
        tma_load_2d(sv, &map_v, &v_full[st], vc, k0 + j * BN);
        tma_load_2d(sv + KV_HALF, &map_v, &v_full[st], vc + 64, k0 + j * BN);
      }
    }
  } else if (warp == MMA_WARP) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t id_s = idesc_bf16(BM, BN, false);
      constexpr uint32_t id_o = idesc_bf16(BM, D, true);
      const uint32_t q_addr = smem_u32(smem + SMEM_Q), p_addr = smem_u32(smem + SMEM_P);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1, p.error, ERR_K)) return false;
        if (j >= 2 && !mbar_wait(&s_free[st], ((j >> 1) - 1) & 1, p.error, ERR_S)) return false;
        fence_after();
        const uint32_t k_addr = smem_u32(smem + SMEM_K + st * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          umma(tmem + st * BN, desc_sw128(q_addr + (kk >> 2) * TILE_HALF + (kk & 3) * 32, 16, 1024),
               desc_sw128(k_addr + (kk >> 2) * KV_HALF + (kk & 3) * 32, 16, 1024), id_s,
               kk > 0 ? 1u : 0u);
        }
        commit(&s_full[st]);
        commit(&k_empty[st]);
        return true;
      };
      bool ok = n_tiles > 0 && mbar_wait(&q_full, 0, p.error, ERR_Q);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);            // next tile's scores run during this soft-max
        if (!ok) break;
        ok = mbar_wait(&p_ready, j & 1, p.error, ERR_P) && mbar_wait(&v_full[st], (j >> 1) & 1, p.error, ERR_V);
        if (!ok) break;
        fence_after();
        const uint32_t v_addr = smem_u32(smem + SMEM_V + st * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint32_t pa = p_addr + (kk >> 2) * TILE_HALF + (kk & 3) * 32;
          umma(tmem_o, desc_sw128(pa, 16, 1024), desc_sw128(v_addr + kk * 2048, KV_HALF, 1024), id_o,
               (j > 0 || kk > 0) ? 1u : 0u);
        }
        commit(&pv_done);
        commit(&v_empty[st]);
      }
    }
  } else {
    // ---------------- soft-max + epilogue ----------------
    // Two threads per query row: warps 0-3 own key columns [0, 64) of the tile, warps 4-7 columns
    // [64, 128) (a warp reaches the TMEM lanes of its quarter, warp % 4).  Both read the whole
    // score row for its maximum, so they agree on the running maximum without talking; each keeps
    // the partial sum of its own columns, rescales its half of the O columns and writes its half
    // of P.
    const int wg = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;                    // row inside the tile
    const int grow = m0 + row;                              // row inside the sequence
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    unsigned char* sp = smem + SMEM_P + ((wg * HALF) >> 6) * TILE_HALF;   // the 64-column half tile of P
    constexpr int NCHUNK = HALF / 8;
    const int chunk0 = ((wg * HALF) & 63) >> 3;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      ok = mbar_wait_warp(&s_full[sb], (j >> 1) & 1, p.error, ERR_S);
      if (!ok) break;
      fence_after();
      const int kbase = j * BN;
      const bool need_mask = (kbase + BN > klen) || (p.causal && (kbase + BN - 1 > m0 + off));
      const int limit = min(klen, p.causal ? grow + off + 1 : klen) - kbase;   // valid columns of this row
      float s[HALF], t[32];
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      // the other half: maximum only
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col0 = (wg ^ 1) * HALF + c * 32;
        tmem_ld32(tmem + lane_base + sb * BN + col0, t);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = (col0 + i < limit) ? t[i] : -INFINITY;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmaxf(mx0, t[i]);
          mx1 = fmaxf(mx1, t[i + 1]);
          mx2 = fmaxf(mx2, t[i + 2]);
          mx3 = fmaxf(mx3, t[i + 3]);
        }
      }
      // this thread's half
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col0 = wg * HALF + c * 32;
        tmem_ld32(tmem + lane_base + sb * BN + col0, t);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = t[i];
          if (need_mask) v = (col0 + i < limit) ? v : -INFINITY;
          s[c * 32 + i] = v;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmaxf(mx0, s[c * 32 + i]);
          mx1 = fmaxf(mx1, s[c * 32 + i + 1]);
          mx2 = fmaxf(mx2, s[c * 32 + i + 2]);
          mx3 = fmaxf(mx3, s[c * 32 + i + 3]);
        }
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);              // the score buffer may be overwritten
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;   // scale > 0
      // The running maximum follows the row maximum lazily: it moves only when the row maximum
      // passed it by more than 8 (a factor 256, harmless in fp32 sums and bf16 P), so that O is
      // rescaled in TMEM on few tiles only.
      float m_new = fmaxf(m_run, mx);
      if (m_run != -INFINITY && m_new - m_run <= 8.f) m_new = m_run;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m_run - m_use);
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
      for (int i = 0; i < HALF; i += 4) {
        s[i] = exp2f(fmaf(s[i], p.scale_log2, -m_use));
        s[i + 1] = exp2f(fmaf(s[i + 1], p.scale_log2, -m_use));
        s[i + 2] = exp2f(fmaf(s[i + 2], p.scale_log2, -m_use));
        s[i + 3] = exp2f(fmaf(s[i + 3], p.scale_log2, -m_use));
        sum0 += s[i];
        sum1 += s[i + 1];
        sum2 += s[i + 2];
        sum3 += s[i + 3];
      }
      l_run = l_run * corr + ((sum0 + sum1) + (sum2 + sum3));
      m_run = m_new;
      if (j > 0) {
        // the previous P V product must be finished before P is overwritten or O is rescaled
        ok = mbar_wait_warp(&pv_done, (j - 1) & 1, p.error, ERR_PV);
        if (!ok) break;
        fence_after();
        if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            tmem_ld32(tmem_o + lane_base + wg * 64 + c * 32, t);
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] *= corr;
            tmem_st32(tmem_o + lane_base + wg * 64 + c * 32, t);
          }
        }
      }
      // P half row -> shared memory, K-major, 128-byte swizzle: 16-byte chunk index XOR (row % 8)
#pragma unroll
      for (int chunk = 0; chunk < NCHUNK; ++chunk) {
        unsigned char* dst = sp + (row >> 3) * 1024 + (row & 7) * 128 + (((chunk0 + chunk) ^ (row & 7)) << 4);
        *reinterpret_cast<bf16x8*>(dst) = pack8(&s[chunk * 8]);
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic smem writes -> UMMA reads
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready);
    }
    if (ok && n_tiles > 0) ok = mbar_wait_warp(&pv_done, (n_tiles - 1) & 1, p.error, ERR_PV);
    // the two partial sums of a row meet in shared memory
    l_part[wg][row] = l_run;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");        // every soft-max thread reaches this once
    if (ok) {
      fence_after();
      const float l_row = l_part[0][row] + l_part[1][row];
      const float inv_l = l_row > 0.f ? 1.f / l_row : 0.f;
      // O: 32 rows x 64 columns through this warp's patch (all tiles are consumed: any stage is free)
      unsigned char* patch = smem + warp * (32 * OUT_PITCH);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float v[32];
        if (n_tiles > 0) {
          tmem_ld32(tmem_o + lane_base + wg * 64 + hh * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= inv_l;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<bf16x8*>(patch + lane * OUT_PITCH + hh * 64 + q * 16) = pack8(v + q * 8);
      }
      __syncwarp();
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + (lane >> 3);
        const int gr = m0 + quarter * 32 + r;
        if (gr < qlen)
          st8(p.o + (long long)(q0 + gr) * p.o_stride_t + (long long)h * D + wg * 64 + (lane & 7) * 8,
              *reinterpret_cast<const bf16x8*>(patch + r * OUT_PITCH + (lane & 7) * 16));
      }
      if (wg == 0 && grow < qlen) p.lse[(long long)h * p.Tq + q0 + grow] = (m_run + log2f(l_row)) * 0.6931471805599453f;
    }
  }
  fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
  }
}

// =====================================================================================================
// Backward.  Two kernels, as in attention.cu (no atomics, bit-reproducible):
//   fa_bwd_dq_tcgen05_kernel    CTA = 128 query rows of one head, loop over 64-key tiles:
//                               S = Q K^T, dP = dO V^T (TMEM, double-buffered), dS = P o (dP - delta)
//                               to shared memory, dQ += dS K (K as MN-major operand), dQ in TMEM.
//   fa_bwd_dkdv_tcgen05_kernel  CTA = 128 keys of one KV head, loop over the query heads of the
//                               group and their 64-row query tiles: S^T = K Q^T, dP^T = V dO^T,
//                               P^T and dS^T to shared memory, dV += P^T dO, dK += dS^T Q (dO and Q
//                               as MN-major operands), dK and dV in TMEM.
// P is recomputed from the saved log-sum-exp; delta = rowsum(dO o O) comes from a small kernel.
// =====================================================================================================
constexpr uint32_t T64_HALF = 64 * 64 * 2;             // [64 rows x 64 cols] bf16 swizzled half tile, 8 KiB
constexpr uint32_t T64_BYTES = 2 * T64_HALF;           // 16 KiB
constexpr int BWD_STAGES = 3;
constexpr uint32_t BWD_STAGE_BYTES = 2 * T64_BYTES;    // two 64-row tiles per stage (K+V or Q+dO)
constexpr uint32_t DQ_SMEM_Q = 0, DQ_SMEM_DO = TILE_BYTES, DQ_SMEM_KV = 2 * TILE_BYTES,
                   DQ_SMEM_DS = DQ_SMEM_KV + BWD_STAGES * BWD_STAGE_BYTES, DQ_SMEM_TOTAL = DQ_SMEM_DS + T64_BYTES;
constexpr uint32_t KV_SMEM_K = 0, KV_SMEM_V = TILE_BYTES, KV_SMEM_QDO = 2 * TILE_BYTES,
                   KV_SMEM_P = KV_SMEM_QDO + BWD_STAGES * BWD_STAGE_BYTES, KV_SMEM_DS = KV_SMEM_P + T64_BYTES,
                   KV_SMEM_TOTAL = KV_SMEM_DS + T64_BYTES;
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
  const __nv_bfloat16* o;
  const __nv_bfloat16* dout;
  long long o_stride_t;
  const float* lse;      // [nh, Tq], natural log
  float* delta;          // [nh, Tq]
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long q_stride_t, k_stride_t, v_stride_t;
  const int* cu_q;
  const int* cu_k;
  int nh, nkv;
  long long Tq;
  float scale, scale_log2;
  int causal;
  int q_group_stride, q_hpg, q_head_stride;
  int k_group_stride, k_hpg, k_head_stride;
  int v_group_stride, v_hpg, v_head_stride;
  int* error;
};

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h), head size 128.
__global__ void fa_delta128_kernel(const BwdParams p) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= p.Tq * p.nh) return;
  const long long t = w / p.nh;
  const int h = (int)(w % p.nh);
  const long long base = t * p.o_stride_t + (long long)h * D + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(p.o + base);
  const uint2 b = *reinterpret_cast<const uint2*>(p.dout + base);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(b2[i]);
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) p.delta[(long long)h * p.Tq + t] = s;
}

// One warp's 32 TMEM lanes x 64 accumulator columns -> bf16, through a shared-memory patch, stored
// as whole 128-byte row segments.  `dst` points at (first row of the warp, first of the 64 columns).
__device__ __forceinline__ void store_half_tile(uint32_t taddr, float scale, bool zero, unsigned char* patch, int lane,
                                                __nv_bfloat16* dst, long long row_stride, int rows_valid) {
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    float v[32];
    if (!zero) {
      tmem_ld32(taddr + hh * 32, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= scale;
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0.f;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
      *reinterpret_cast<bf16x8*>(patch + lane * OUT_PITCH + hh * 64 + q * 16) = pack8(v + q * 8);
  }
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3);
    if (r < rows_valid)
      st8(dst + (long long)r * row_stride + (lane & 7) * 8,
          *reinterpret_cast<const bf16x8*>(patch + r * OUT_PITCH + (lane & 7) * 16));
  }
  __syncwarp();
}

// 32 values of one row -> four 16-byte chunks of a K-major, 128-byte-swizzled [128 x 64] bf16 tile.
__device__ __forceinline__ void write_row_chunks(unsigned char* tile, int row, int first_chunk, const float* v) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    unsigned char* dst = tile + (row >> 3) * 1024 + (row & 7) * 128 + (((first_chunk + c) ^ (row & 7)) << 4);
    *reinterpret_cast<bf16x8*>(dst) = pack8(v + c * 8);
  }
}

__global__ void __launch_bounds__(THREADS, 1)
fa_bwd_dq_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                         const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const __grid_constant__ BwdParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t qdo_full, kv_full[BWD_STAGES], kv_empty[BWD_STAGES], s_full[2], s_free[2], ds_ready, ds_free;
  __shared__ uint32_t tmem_slot;

  const int b = blockIdx.z, h = blockIdx.y, mt = blockIdx.x;
  const int q0 = p.cu_q[b], qlen = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], klen = p.cu_k[b + 1] - k0;
  const int m0 = mt * BM;
  if (m0 >= qlen) return;
  const int hk = h / (p.nh / p.nkv);
  const int off = klen - qlen;
  int kmax = klen;
  if (p.causal) kmax = min(klen, m0 + BM + off);
  const int n_tiles = kmax > 0 ? (kmax + 63) / 64 : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&qdo_full, 1);
    for (int i = 0; i < BWD_STAGES; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], SOFTMAX_WARPS);
    }
    mbar_init(&ds_ready, SOFTMAX_WARPS);
    mbar_init(&ds_free, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;                 // S: [0,64) [64,128)   dP: [128,192) [192,256)   dQ: [256,384)
  const uint32_t tmem_dp = tmem + 128, tmem_dq = tmem + 256;

  if (warp == TMA_WARP) {
    if (elect_one()) {
      const int qc = head_col(0, p.q_group_stride, p.q_hpg, p.q_head_stride, h);
      const int kc = head_col(0, p.k_group_stride, p.k_hpg, p.k_head_stride, hk);
      const int vc = head_col(0, p.v_group_stride, p.v_hpg, p.v_head_stride, hk);
      mbar_expect_tx(&qdo_full, 2 * TILE_BYTES);
      tma_load_2d(smem + DQ_SMEM_Q, &map_q, &qdo_full, qc, q0 + m0);
      tma_load_2d(smem + DQ_SMEM_Q + TILE_HALF, &map_q, &qdo_full, qc + 64, q0 + m0);
      tma_load_2d(smem + DQ_SMEM_DO, &map_do, &qdo_full, h * D, q0 + m0);
      tma_load_2d(smem + DQ_SMEM_DO + TILE_HALF, &map_do, &qdo_full, h * D + 64, q0 + m0);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % BWD_STAGES;
        const uint32_t use = j / BWD_STAGES;
        if (use > 0 && !mbar_wait(&kv_empty[st], (use - 1) & 1, p.error, ERR_EMPTY)) break;
        mbar_expect_tx(&kv_full[st], BWD_STAGE_BYTES);
        unsigned char* sk = smem + DQ_SMEM_KV + st * BWD_STAGE_BYTES;
        tma_load_2d(sk, &map_k, &kv_full[st], kc, k0 + j * 64);
        tma_load_2d(sk + T64_HALF, &map_k, &kv_full[st], kc + 64, k0 + j * 64);
        tma_load_2d(sk + T64_BYTES, &map_v, &kv_full[st], vc, k0 + j * 64);
        tma_load_2d(sk + T64_BYTES + T64_HALF, &map_v, &kv_full[st], vc + 64, k0 + j * 64);
      }
    }
  } else if (warp == MMA_WARP) {
    if (elect_one()) {
      constexpr uint32_t id_s = idesc_bf16(BM, 64, false);
      constexpr uint32_t id_o = idesc_bf16(BM, D, true);
      const uint32_t q_addr = smem_u32(smem + DQ_SMEM_Q), do_addr = smem_u32(smem + DQ_SMEM_DO);
      const uint32_t ds_addr = smem_u32(smem + DQ_SMEM_DS);
      auto issue_s = [&](int j) -> bool {
        const int st = j % BWD_STAGES, sb = j & 1;
        if (!mbar_wait(&kv_full[st], (j / BWD_STAGES) & 1, p.error, ERR_K)) return false;
        if (j >= 2 && !mbar_wait(&s_free[sb], ((j >> 1) - 1) & 1, p.error, ERR_S)) return false;
        fence_after();
        const uint32_t k_addr = smem_u32(smem + DQ_SMEM_KV + st * BWD_STAGE_BYTES), v_addr = k_addr + T64_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma(tmem + sb * 64, desc_sw128(q_addr + (kk >> 2) * TILE_HALF + (kk & 3) * 32, 16, 1024),
               desc_sw128(k_addr + (kk >> 2) * T64_HALF + (kk & 3) * 32, 16, 1024), id_s, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma(tmem_dp + sb * 64, desc_sw128(do_addr + (kk >> 2) * TILE_HALF + (kk & 3) * 32, 16, 1024),
               desc_sw128(v_addr + (kk >> 2) * T64_HALF + (kk & 3) * 32, 16, 1024), id_s, kk > 0 ? 1u : 0u);
        commit(&s_full[sb]);
        return true;
      };
      bool ok = n_tiles > 0 && mbar_wait(&qdo_full, 0, p.error, ERR_Q);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % BWD_STAGES;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        ok = mbar_wait(&ds_ready, j & 1, p.error, ERR_P);
        if (!ok) break;
        fence_after();
        const uint32_t k_addr = smem_u32(smem + DQ_SMEM_KV + st * BWD_STAGE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)                 // dQ += dS[128 x 64 keys] K[64 keys x 128]
          umma(tmem_dq, desc_sw128(ds_addr + kk * 32, 16, 1024), desc_sw128(k_addr + kk * 2048, T64_HALF, 1024), id_o,
               (j > 0 || kk > 0) ? 1u : 0u);
        commit(&ds_free);
        commit(&kv_empty[st]);
      }
    }
  } else {
    const int wg = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int grow = m0 + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const bool row_ok = grow < qlen;
    // a row outside the sequence gets lse = +inf, so that its P is exactly 0
    const float lse2 = row_ok ? p.lse[(long long)h * p.Tq + q0 + grow] * LOG2E : INFINITY;
    const float delta = row_ok ? p.delta[(long long)h * p.Tq + q0 + grow] : 0.f;
    unsigned char* ds_tile = smem + DQ_SMEM_DS;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      ok = mbar_wait_warp(&s_full[sb], (j >> 1) & 1, p.error, ERR_S);
      if (!ok) break;
      fence_after();
      float s[32], dp[32];
      tmem_ld32(tmem + lane_base + sb * 64 + wg * 32, s);
      tmem_ld32(tmem_dp + lane_base + sb * 64 + wg * 32, dp);
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);
      const int kbase = j * 64 + wg * 32;
      const int limit = min(klen, p.causal ? grow + off + 1 : klen) - kbase;   // valid columns of this thread
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float pr = (i < limit) ? exp2f(fmaf(s[i], p.scale_log2, -lse2)) : 0.f;
        s[i] = pr * (dp[i] - delta);
      }
      if (j > 0) {
        ok = mbar_wait_warp(&ds_free, (j - 1) & 1, p.error, ERR_PV);
        if (!ok) break;
      }
      write_row_chunks(ds_tile, row, wg * 4, s);
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_ready);
    }
    if (ok && n_tiles > 0) ok = mbar_wait_warp(&ds_free, (n_tiles - 1) & 1, p.error, ERR_PV);
    if (ok) {
      fence_after();
      const int qc = head_col(0, p.q_group_stride, p.q_hpg, p.q_head_stride, h);
      store_half_tile(tmem_dq + lane_base + wg * 64, p.scale, n_tiles == 0, smem + warp * (32 * OUT_PITCH), lane,
                      p.dq + (long long)(q0 + m0 + quarter * 32) * p.q_stride_t + qc + wg * 64, p.q_stride_t,
                      qlen - (m0 + quarter * 32));
    }
  }
  fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
  }
}

__global__ void __launch_bounds__(THREADS, 1)
fa_bwd_dkdv_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                           const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                           const __grid_constant__ BwdParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t kv_full, qdo_full[BWD_STAGES], qdo_empty[BWD_STAGES], s_full[2], s_free[2], p_ready, p_free;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(16) float stat_s[BWD_STAGES][2][64];   // per stage: log2-domain lse and delta of its 64 query rows

  const int b = blockIdx.z, hk = blockIdx.y, nt = blockIdx.x;
  const int q0 = p.cu_q[b], qlen = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], klen = p.cu_k[b + 1] - k0;
  const int kb = nt * BM;                                  // first key of this CTA
  if (kb >= klen) return;
  const int rep = p.nh / p.nkv;
  const int off = klen - qlen;
  // 64-row query tiles that see any of these keys: rows r with r + off >= kb (causal), r < qlen
  int i_start = 0;
  if (p.causal) i_start = max(0, kb - off) / 64;
  const int i_end = (qlen + 63) / 64;
  const int nq = max(0, i_end - i_start);
  const int n_it = nq * rep;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&kv_full, 1);
    for (int i = 0; i < BWD_STAGES; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], SOFTMAX_WARPS);
    }
    mbar_init(&p_ready, SOFTMAX_WARPS);
    mbar_init(&p_free, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;           // S^T: [0,64) [64,128)   dP^T: [128,192) [192,256)   dV: [256,384)   dK: [384,512)
  const uint32_t tmem_dp = tmem + 128, tmem_dv = tmem + 256, tmem_dk = tmem + 384;

  if (warp == TMA_WARP) {
    // lane 0 issues the TMA loads; all lanes stage the per-query statistics of the tile (two rows each)
    const int kc = head_col(0, p.k_group_stride, p.k_hpg, p.k_head_stride, hk);
    const int vc = head_col(0, p.v_group_stride, p.v_hpg, p.v_head_stride, hk);
    if (lane == 0) {
      mbar_expect_tx(&kv_full, 2 * TILE_BYTES);
      tma_load_2d(smem + KV_SMEM_K, &map_k, &kv_full, kc, k0 + kb);
      tma_load_2d(smem + KV_SMEM_K + TILE_HALF, &map_k, &kv_full, kc + 64, k0 + kb);
      tma_load_2d(smem + KV_SMEM_V, &map_v, &kv_full, vc, k0 + kb);
      tma_load_2d(smem + KV_SMEM_V + TILE_HALF, &map_v, &kv_full, vc + 64, k0 + kb);
    }
    for (int it = 0; it < n_it; ++it) {
      const int st = it % BWD_STAGES;
      const uint32_t use = it / BWD_STAGES;
      if (use > 0 && !mbar_wait(&qdo_empty[st], (use - 1) & 1, p.error, ERR_EMPTY)) break;
      const int hq = hk * rep + it / nq, qi = i_start + it % nq;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int q = qi * 64 + half * 32 + lane;
        const bool okq = q < qlen;
        const long long gi = (long long)hq * p.Tq + q0 + q;
        stat_s[st][0][half * 32 + lane] = okq ? __ldg(p.lse + gi) * LOG2E : INFINITY;   // +inf: P is exactly 0
        stat_s[st][1][half * 32 + lane] = okq ? __ldg(p.delta + gi) : 0.f;
      }
      __syncwarp();
      if (lane == 0) {
        const int qc = head_col(0, p.q_group_stride, p.q_hpg, p.q_head_stride, hq);
        mbar_expect_tx(&qdo_full[st], BWD_STAGE_BYTES);
        unsigned char* sq = smem + KV_SMEM_QDO + st * BWD_STAGE_BYTES;
        tma_load_2d(sq, &map_q, &qdo_full[st], qc, q0 + qi * 64);
        tma_load_2d(sq + T64_HALF, &map_q, &qdo_full[st], qc + 64, q0 + qi * 64);
        tma_load_2d(sq + T64_BYTES, &map_do, &qdo_full[st], hq * D, q0 + qi * 64);
        tma_load_2d(sq + T64_BYTES + T64_HALF, &map_do, &qdo_full[st], hq * D + 64, q0 + qi * 64);
      }
      __syncwarp();
    }
  } else if (warp == MMA_WARP) {
    if (elect_one()) {
      constexpr uint32_t id_s = idesc_bf16(BM, 64, false);
      constexpr uint32_t id_o = idesc_bf16(BM, D, true);
      const uint32_t k_addr = smem_u32(smem + KV_SMEM_K), v_addr = smem_u32(smem + KV_SMEM_V);
      const uint32_t p_addr = smem_u32(smem + KV_SMEM_P), ds_addr = smem_u32(smem + KV_SMEM_DS);
      auto issue_s = [&](int it) -> bool {
        const int st = it % BWD_STAGES, sb = it & 1;
        if (!mbar_wait(&qdo_full[st], (it / BWD_STAGES) & 1, p.error, ERR_Q)) return false;
        if (it >= 2 && !mbar_wait(&s_free[sb], ((it >> 1) - 1) & 1, p.error, ERR_S)) return false;
        fence_after();
        const uint32_t q_addr = smem_u32(smem + KV_SMEM_QDO + st * BWD_STAGE_BYTES), do_addr = q_addr + T64_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)              // S^T[keys, q] = K Q^T
          umma(tmem + sb * 64, desc_sw128(k_addr + (kk >> 2) * TILE_HALF + (kk & 3) * 32, 16, 1024),
               desc_sw128(q_addr + (kk >> 2) * T64_HALF + (kk & 3) * 32, 16, 1024), id_s, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)              // dP^T[keys, q] = V dO^T
          umma(tmem_dp + sb * 64, desc_sw128(v_addr + (kk >> 2) * TILE_HALF + (kk & 3) * 32, 16, 1024),
               desc_sw128(do_addr + (kk >> 2) * T64_HALF + (kk & 3) * 32, 16, 1024), id_s, kk > 0 ? 1u : 0u);
        commit(&s_full[sb]);
        return true;
      };
      bool ok = n_it > 0 && mbar_wait(&kv_full, 0, p.error, ERR_K);
      if (ok) ok = issue_s(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % BWD_STAGES;
        if (it + 1 < n_it) ok = issue_s(it + 1);
        if (!ok) break;
        ok = mbar_wait(&p_ready, it & 1, p.error, ERR_P);
        if (!ok) break;
        fence_after();
        const uint32_t q_addr = smem_u32(smem + KV_SMEM_QDO + st * BWD_STAGE_BYTES), do_addr = q_addr + T64_BYTES;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)                   // dV += P^T[keys x 64 q] dO[64 q x 128]
          umma(tmem_dv, desc_sw128(p_addr + kk * 32, 16, 1024), desc_sw128(do_addr + kk * 2048, T64_HALF, 1024), id_o,
               (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)                   // dK += dS^T[keys x 64 q] Q[64 q x 128]
          umma(tmem_dk, desc_sw128(ds_addr + kk * 32, 16, 1024), desc_sw128(q_addr + kk * 2048, T64_HALF, 1024), id_o,
               (it > 0 || kk > 0) ? 1u : 0u);
        commit(&p_free);
        commit(&qdo_empty[st]);
      }
    }
  } else {
    const int wg = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;                   // key row of this thread
    const int key = kb + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int sb = it & 1;
      const int hq = hk * rep + it / nq, qi = i_start + it % nq;
      const int qbase = qi * 64 + wg * 32;                 // first query row of this thread's 32 columns
      const int st = it % BWD_STAGES;
      ok = mbar_wait_warp(&s_full[sb], (it >> 1) & 1, p.error, ERR_S);
      if (!ok) break;
      fence_after();
      // the statistics of this stage were written before its "full" arrival, which the MMA thread saw
      // before it issued the MMAs this wait is about; waiting on the stage barrier as well makes the
      // ordering direct (the phase cannot advance before this iteration's P is handed over)
      ok = mbar_wait_warp(&qdo_full[st], (it / BWD_STAGES) & 1, p.error, ERR_Q);
      if (!ok) break;
      float lse2[32], dl[32];
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 a = *reinterpret_cast<const float4*>(&stat_s[st][0][wg * 32 + i]);
        const float4 b4 = *reinterpret_cast<const float4*>(&stat_s[st][1][wg * 32 + i]);
        lse2[i] = a.x; lse2[i + 1] = a.y; lse2[i + 2] = a.z; lse2[i + 3] = a.w;
        dl[i] = b4.x; dl[i + 1] = b4.y; dl[i + 2] = b4.z; dl[i + 3] = b4.w;
      }
      float s[32], dp[32];
      tmem_ld32(tmem + lane_base + sb * 64 + wg * 32, s);
      tmem_ld32(tmem_dp + lane_base + sb * 64 + wg * 32, dp);
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);
      // column i (query qbase + i) sees this key iff key <= q + off
      const int first = p.causal ? key - off - qbase : 0;   // columns below `first` are masked
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float pr = (i >= first) ? exp2f(fmaf(s[i], p.scale_log2, -lse2[i])) : 0.f;
        s[i] = pr;
        dp[i] = pr * (dp[i] - dl[i]);
      }
      if (it > 0) {
        ok = mbar_wait_warp(&p_free, (it - 1) & 1, p.error, ERR_PV);
        if (!ok) break;
      }
      write_row_chunks(smem + KV_SMEM_P, row, wg * 4, s);
      write_row_chunks(smem + KV_SMEM_DS, row, wg * 4, dp);
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready);
    }
    if (ok && n_it > 0) ok = mbar_wait_warp(&p_free, (n_it - 1) & 1, p.error, ERR_PV);
    if (ok) {
      fence_after();
      const int kc = head_col(0, p.k_group_stride, p.k_hpg, p.k_head_stride, hk);
      const int vc = head_col(0, p.v_group_stride, p.v_hpg, p.v_head_stride, hk);
      unsigned char* patch = smem + KV_SMEM_QDO + warp * (32 * OUT_PITCH);
      const int rows_valid = klen - (kb + quarter * 32);
      store_half_tile(tmem_dv + lane_base + wg * 64, 1.f, n_it == 0, patch, lane,
                      p.dv + (long long)(k0 + kb + quarter * 32) * p.v_stride_t + vc + wg * 64, p.v_stride_t, rows_valid);
      store_half_tile(tmem_dk + lane_base + wg * 64, p.scale, n_it == 0, patch, lane,
                      p.dk + (long long)(k0 + kb + quarter * 32) * p.k_stride_t + kc + wg * 64, p.k_stride_t, rows_valid);
    }
  }
  fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
  }
}

}  // namespace fa5
}  // namespace msrl

using namespace msrl;

static PFN_cuTensorMapEncodeTiled_v12000 fa5_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// [rows, width] bf16 view with a row pitch of `stride_t` elements; box = 64 columns x `box_rows` rows.
static bool fa5_make_map(CUtensorMap* map, const void* base, long long rows, long long width, long long stride_t,
                         unsigned box_rows = 128u) {
  auto fn = fa5_encode_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (stride_t * 2) % 16 != 0 || width % 8 != 0) return false;
  cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(stride_t * 2)};
  cuuint32_t box[2] = {64u, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static long long fa5_width(int heads, long long gs, long long hpg, long long hs) {
  long long w = 0;
  for (int h = 0; h < heads; ++h) {
    const long long c = (h / hpg) * gs + (h % hpg) * hs + fa5::D;
    w = c > w ? c : w;
  }
  return w;
}

// Same contract as msrl_flash_attn_varlen_fwd (attention.cu) for head dim 128, plus the number of
// key rows `Tk` and a device status word (0 = ok; 11..17 = a bounded wait ran out).  Layout
// arrays: {stride_t, group_stride, heads_per_group, head_stride} for q, k, v (12 values).
// Returns cudaErrorNotSupported for shapes this kernel does not cover: the caller falls back.
MSRL_API int msrl_flash_attn_varlen_fwd_tcgen05(const void* q, const void* k, const void* v,
                                                const long long* lay, void* o, long long o_stride_t,
                                                float* lse, const int* cu_q, const int* cu_k, int batch,
                                                int max_q, int nh, int nkv, long long Tq, long long Tk,
                                                int D, int causal, int* error, cudaStream_t st) {
  if (batch == 0 || Tq == 0) return 0;
  if (D != fa5::D || nh % nkv != 0 || (o_stride_t % 8) != 0 || (reinterpret_cast<uintptr_t>(o) & 15) != 0)
    return (int)cudaErrorNotSupported;
  for (int i = 0; i < 3; ++i) {
    const long long* l = lay + 4 * i;
    if (l[0] % 8 != 0 || l[1] % 8 != 0 || l[3] % 8 != 0 || l[2] <= 0) return (int)cudaErrorNotSupported;
  }
  static int bn = 0;
  if (bn == 0) {
    const char* e = getenv("MSRL_ATTN_KEY_TILE");
    bn = (e != nullptr && atoi(e) == 128) ? 128 : 64;
  }
  CUtensorMap mq, mk, mv;
  if (!fa5_make_map(&mq, q, Tq, fa5_width(nh, lay[1], lay[2], lay[3]), lay[0]) ||
      !fa5_make_map(&mk, k, Tk, fa5_width(nkv, lay[5], lay[6], lay[7]), lay[4], bn) ||
      !fa5_make_map(&mv, v, Tk, fa5_width(nkv, lay[9], lay[10], lay[11]), lay[8], bn))
    return (int)cudaErrorNotSupported;
  fa5::Params p{};
  p.o = (__nv_bfloat16*)o;
  p.o_stride_t = o_stride_t;
  p.lse = lse;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.nh = nh;
  p.nkv = nkv;
  p.Tq = Tq;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)D);
  p.causal = causal;
  p.q_col0 = 0; p.q_group_stride = (int)lay[1]; p.q_hpg = (int)lay[2]; p.q_head_stride = (int)lay[3];
  p.k_col0 = 0; p.k_group_stride = (int)lay[5]; p.k_hpg = (int)lay[6]; p.k_head_stride = (int)lay[7];
  p.v_col0 = 0; p.v_group_stride = (int)lay[9]; p.v_hpg = (int)lay[10]; p.v_head_stride = (int)lay[11];
  p.error = error;
  static bool attr_set = false;
  const int smem = (int)fa5::fwd_smem_bytes(bn) + (bn == 128 ? 1024 : 896);   // 64: two CTAs in 228 KiB
  if (!attr_set) {
    cudaError_t e = bn == 128
        ? cudaFuncSetAttribute(fa5::fa_fwd_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
        : cudaFuncSetAttribute(fa5::fa_fwd_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((max_q + fa5::BM - 1) / fa5::BM, nh, batch);
  if (bn == 128)
    fa5::fa_fwd_tcgen05_kernel<128><<<grid, fa5::THREADS, smem, st>>>(mq, mk, mv, p);
  else
    fa5::fa_fwd_tcgen05_kernel<64><<<grid, fa5::THREADS, smem, st>>>(mq, mk, mv, p);
  return (int)cudaGetLastError();
}

// Same contract as msrl_flash_attn_varlen_bwd (attention.cu) for head size 128, plus `Tk` and a
// device status word.  delta: fp32 scratch [nh, Tq]; dq/dk/dv use the layouts of q/k/v.
MSRL_API int msrl_flash_attn_varlen_bwd_tcgen05(const void* q, const void* k, const void* v, const long long* lay,
                                                const void* o, const void* dout, long long o_stride_t,
                                                const float* lse, float* delta, void* dq, void* dk, void* dv,
                                                const int* cu_q, const int* cu_k, int batch, int max_q, int max_k,
                                                int nh, int nkv, long long Tq, long long Tk, int D, int causal,
                                                int* error, cudaStream_t st) {
  if (batch == 0 || Tq == 0) return 0;
  if (D != fa5::D || nh % nkv != 0 || (o_stride_t % 8) != 0 || (reinterpret_cast<uintptr_t>(o) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(dout) & 15) != 0 || (reinterpret_cast<uintptr_t>(dq) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(dk) & 15) != 0 || (reinterpret_cast<uintptr_t>(dv) & 15) != 0)
    return (int)cudaErrorNotSupported;
  for (int i = 0; i < 3; ++i) {
    const long long* l = lay + 4 * i;
    if (l[0] % 8 != 0 || l[1] % 8 != 0 || l[3] % 8 != 0 || l[2] <= 0) return (int)cudaErrorNotSupported;
  }
  const long long wq = fa5_width(nh, lay[1], lay[2], lay[3]), wk = fa5_width(nkv, lay[5], lay[6], lay[7]),
                  wv = fa5_width(nkv, lay[9], lay[10], lay[11]);
  CUtensorMap q128, q64, do128, do64, k128, k64, v128, v64;
  if (!fa5_make_map(&q128, q, Tq, wq, lay[0], 128) || !fa5_make_map(&q64, q, Tq, wq, lay[0], 64) ||
      !fa5_make_map(&do128, dout, Tq, (long long)nh * D, o_stride_t, 128) ||
      !fa5_make_map(&do64, dout, Tq, (long long)nh * D, o_stride_t, 64) ||
      !fa5_make_map(&k128, k, Tk, wk, lay[4], 128) || !fa5_make_map(&k64, k, Tk, wk, lay[4], 64) ||
      !fa5_make_map(&v128, v, Tk, wv, lay[8], 128) || !fa5_make_map(&v64, v, Tk, wv, lay[8], 64))
    return (int)cudaErrorNotSupported;
  fa5::BwdParams p{};
  p.o = (const __nv_bfloat16*)o;
  p.dout = (const __nv_bfloat16*)dout;
  p.o_stride_t = o_stride_t;
  p.lse = lse;
  p.delta = delta;
  p.dq = (__nv_bfloat16*)dq;
  p.dk = (__nv_bfloat16*)dk;
  p.dv = (__nv_bfloat16*)dv;
  p.q_stride_t = lay[0];
  p.k_stride_t = lay[4];
  p.v_stride_t = lay[8];
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.nh = nh;
  p.nkv = nkv;
  p.Tq = Tq;
  p.scale = 1.f / sqrtf((float)D);
  p.scale_log2 = p.scale * fa5::LOG2E;
  p.causal = causal;
  p.q_group_stride = (int)lay[1]; p.q_hpg = (int)lay[2]; p.q_head_stride = (int)lay[3];
  p.k_group_stride = (int)lay[5]; p.k_hpg = (int)lay[6]; p.k_head_stride = (int)lay[7];
  p.v_group_stride = (int)lay[9]; p.v_hpg = (int)lay[10]; p.v_head_stride = (int)lay[11];
  p.error = error;
  static bool attr_set = false;
  const int smem_dq = (int)fa5::DQ_SMEM_TOTAL + 1024, smem_kv = (int)fa5::KV_SMEM_TOTAL + 1024;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fa5::fa_bwd_dq_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(fa5::fa_bwd_dkdv_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_kv);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const long long warps = Tq * nh;
  fa5::fa_delta128_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(p);
  dim3 grid_kv((max_k + fa5::BM - 1) / fa5::BM, nkv, batch);
  fa5::fa_bwd_dkdv_tcgen05_kernel<<<grid_kv, fa5::THREADS, smem_kv, st>>>(q64, do64, k128, v128, p);
  dim3 grid_q((max_q + fa5::BM - 1) / fa5::BM, nh, batch);
  fa5::fa_bwd_dq_tcgen05_kernel<<<grid_q, fa5::THREADS, smem_dq, st>>>(q128, do128, k64, v64, p);
  return (int)cudaGetLastError();
}
