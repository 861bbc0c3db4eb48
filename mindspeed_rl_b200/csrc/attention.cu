// Variable-length ("packed", THD) causal flash attention, forward and backward, with GQA.
//
// Sequences are delimited by cu_seqlens (int32 [B+1]); Q/K/V are addressed through HeadLayout
// so they can be read straight out of the fused QKV projection output (either [q|k|v] or the
// per-KV-group interleave) and the gradients are written straight into a dQKV buffer of the
// same shape.  When q_len < k_len the causal mask is bottom-right aligned (a prefill chunk
// attending to its cached prefix).
//
// Forward: 64 query rows per CTA (4 warps x 16 rows), 64-key tiles double-buffered with
// cp.async, online softmax in the exp2 domain, fp32 accumulation on mma.sync tensor cores.
// Backward is split in two kernels that each own their output tile (no atomics, bitwise
// deterministic): `dkdv` (one CTA per 64-key tile, sweeps query tiles and the q heads of the
// KV group) and `dq` (one CTA per 64-query tile, sweeps key tiles).
//
// Replaces the reference's dependency on an external fused attention with
// `set_actual_seq_len` (mindspeed_rl/models/base/base_training_engine.py:384-391).
#include "mma_utils.cuh"

namespace msrl {

struct AttnParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  HeadLayout Lq, Lk, Lv;
  __nv_bfloat16* o;        // [Tq, nh*D] (row stride o_stride_t)
  long long o_stride_t;
  float* lse;              // [nh, Tq] natural-log sum-exp of the scaled scores
  const int* cu_q;
  const int* cu_k;
  int nh, nkv;
  long long Tq;
  float scale;             // 1/sqrt(D)
  float scale_log2;        // scale * log2(e)
  int causal;
  // backward only
  const __nv_bfloat16* dout;  // same layout as o
  float* delta;               // [nh, Tq] rowsum(dO * O)
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
};

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) fa_fwd_kernel(const AttnParams p) {
  constexpr int BM = 64, BN = 64, LD = D + 8, THREADS = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sK = sQ + BM * LD;           // 2 stages
  __nv_bfloat16* sV = sK + 2 * BN * LD;       // 2 stages

  const int b = blockIdx.z, h = blockIdx.y, mt = blockIdx.x;
  const int q0 = p.cu_q[b], qlen = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], klen = p.cu_k[b + 1] - k0;
  const int m0 = mt * BM;
  if (m0 >= qlen) return;
  const int hk = h / (p.nh / p.nkv);
  const int off = klen - qlen;
  int kmax = klen;
  if (p.causal) kmax = min(klen, m0 + BM + off);
  const int n_tiles = (kmax + BN - 1) / BN;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qrow = lane >> 2, qcol = (lane & 3) * 2;

  load_tile_async<BM, D, LD, THREADS>(sQ, p.q, p.Lq, h, q0, m0, qlen);
  if (n_tiles > 0) {
    load_tile_async<BN, D, LD, THREADS>(sK, p.k, p.Lk, hk, k0, 0, klen);
    load_tile_async<BN, D, LD, THREADS>(sV, p.v, p.Lv, hk, k0, 0, klen);
  }
  cp_async_commit();

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  for (int it = 0; it < n_tiles; ++it) {
    const int st = it & 1;
    if (it + 1 < n_tiles) {
      load_tile_async<BN, D, LD, THREADS>(sK + (st ^ 1) * BN * LD, p.k, p.Lk, hk, k0, (it + 1) * BN, klen);
      load_tile_async<BN, D, LD, THREADS>(sV + (st ^ 1) * BN * LD, p.v, p.Lv, hk, k0, (it + 1) * BN, klen);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    const __nv_bfloat16* tK = sK + st * BN * LD;
    const __nv_bfloat16* tV = sV + st * BN * LD;

    // S = Q K^T  (16 x 64 per warp)
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, smem_u32(sQ + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8));
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        uint32_t bfr[4];
        ldmatrix_x4(bfr, smem_u32(tK + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + kk * 16 +
                                  ((lane >> 3) & 1) * 8));
        mma_16816(s[2 * np], a, bfr[0], bfr[1]);
        mma_16816(s[2 * np + 1], a, bfr[2], bfr[3]);
      }
    }

    // mask + online softmax (exp2 domain)
    const int kbase = it * BN;
    const bool need_mask = (kbase + BN > klen) || (p.causal && (kbase + BN - 1 > m0 + off));
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = s[nt][j] * p.scale_log2;
        if (need_mask) {
          const int key = kbase + nt * 8 + qcol + (j & 1);
          const int row = m0 + warp * 16 + qrow + ((j >> 1) << 3);
          const bool ok = (key < klen) && (!p.causal || key <= row + off);
          v = ok ? v : -INFINITY;
        }
        s[nt][j] = v;
        mx[j >> 1] = fmaxf(mx[j >> 1], v);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      corr[r] = exp2f(m_run[r] - m_use[r]);  // m_run = -inf -> 0
      m_run[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = exp2f(s[nt][j] - m_use[j >> 1]);
        s[nt][j] = e;
        rs[j >> 1] += e;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + rs[r];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      o_acc[dt][0] *= corr[0];
      o_acc[dt][1] *= corr[0];
      o_acc[dt][2] *= corr[1];
      o_acc[dt][3] *= corr[1];
    }

    // O += P V
#pragma unroll
    for (int kc = 0; kc < BN / 16; ++kc) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kc][0], s[2 * kc][1]);
      a[1] = pack_bf16(s[2 * kc][2], s[2 * kc][3]);
      a[2] = pack_bf16(s[2 * kc + 1][0], s[2 * kc + 1][1]);
      a[3] = pack_bf16(s[2 * kc + 1][2], s[2 * kc + 1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t bfr[4];
        ldmatrix_x4_trans(bfr, smem_u32(tV + (kc * 16 + (lane & 15)) * LD + dp * 16 + (lane >> 4) * 8));
        mma_16816(o_acc[2 * dp], a, bfr[0], bfr[1]);
        mma_16816(o_acc[2 * dp + 1], a, bfr[2], bfr[3]);
      }
    }
    __syncthreads();
  }

  // finalize
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = m0 + warp * 16 + qrow + r * 8;
    if (row >= qlen) continue;
    const float inv = (l_run[r] > 0.f) ? 1.f / l_run[r] : 0.f;
    __nv_bfloat16* orow = p.o + (long long)(q0 + row) * p.o_stride_t + (long long)h * D;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      *reinterpret_cast<__nv_bfloat162*>(orow + dt * 8 + qcol) =
          __floats2bfloat162_rn(o_acc[dt][2 * r] * inv, o_acc[dt][2 * r + 1] * inv);
    }
    if ((lane & 3) == 0) {
      const float m_fin = (m_run[r] == -INFINITY) ? 0.f : m_run[r];
      p.lse[(long long)h * p.Tq + q0 + row] =
          (l_run[r] > 0.f) ? (m_fin + log2f(l_run[r])) * kLn2 : -INFINITY;
    }
  }
}

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]   (one warp per (t, h))
template <int D>
__global__ void fa_delta_kernel(const AttnParams p) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= p.Tq * p.nh) return;
  const long long t = gw / p.nh;
  const int h = (int)(gw % p.nh);
  const __nv_bfloat16* o = p.o + t * p.o_stride_t + (long long)h * D;
  const __nv_bfloat16* d = p.dout + t * p.o_stride_t + (long long)h * D;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + i));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(d + i));
    s += a.x * c.x + a.y * c.y;
  }
  s = warp_sum(s);
  if (lane == 0) p.delta[(long long)h * p.Tq + t] = s;
}

// ---------------------------------------------------------------------------------------------
// Backward, dK / dV.  CTA = 64 keys of one KV head (4 warps x 16 keys); sweeps the q heads of
// the group and 32-row query tiles.  Works on transposed tiles: S^T = K Q^T so that each warp
// owns the rows (keys) of its dK / dV accumulators.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) fa_bwd_dkdv_kernel(const AttnParams p) {
  constexpr int BN = 64, BM = 32, LD = D + 8, THREADS = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sV = sK + BN * LD;
  __nv_bfloat16* sQ = sV + BN * LD;            // 2 stages of BM rows
  __nv_bfloat16* sdO = sQ + 2 * BM * LD;       // 2 stages
  float* sLse = reinterpret_cast<float*>(sdO + 2 * BM * LD);  // 2 x BM
  float* sDelta = sLse + 2 * BM;                              // 2 x BM

  const int b = blockIdx.z, hk = blockIdx.y, nt0 = blockIdx.x;
  const int q0 = p.cu_q[b], qlen = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], klen = p.cu_k[b + 1] - k0;
  const int n0 = nt0 * BN;
  if (n0 >= klen) return;
  const int rep = p.nh / p.nkv;
  const int off = klen - qlen;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int frow = lane >> 2, fcol = (lane & 3) * 2;

  // first query row that can see key n0: row + off >= n0
  int m_start = 0;
  if (p.causal) m_start = max(0, n0 - off);
  m_start = (m_start / BM) * BM;
  const int q_tiles = (qlen > m_start) ? (qlen - m_start + BM - 1) / BM : 0;
  const int total_iters = q_tiles * rep;

  load_tile_async<BN, D, LD, THREADS>(sK, p.k, p.Lk, hk, k0, n0, klen);
  load_tile_async<BN, D, LD, THREADS>(sV, p.v, p.Lv, hk, k0, n0, klen);

  auto issue = [&](int iter, int stage) {
    const int hq = hk * rep + iter / q_tiles;
    const int m0 = m_start + (iter % q_tiles) * BM;
    load_tile_async<BM, D, LD, THREADS>(sQ + stage * BM * LD, p.q, p.Lq, hq, q0, m0, qlen);
    // dO has the plain [T, nh*D] layout
    HeadLayout Ldo{p.o_stride_t, 0, p.nh, D};
    load_tile_async<BM, D, LD, THREADS>(sdO + stage * BM * LD, p.dout, Ldo, hq, q0, m0, qlen);
    for (int i = threadIdx.x; i < BM; i += THREADS) {
      const int r = m0 + i;
      const bool ok = r < qlen;
      sLse[stage * BM + i] = ok ? p.lse[(long long)hq * p.Tq + q0 + r] : INFINITY;
      sDelta[stage * BM + i] = ok ? p.delta[(long long)hq * p.Tq + q0 + r] : 0.f;
    }
  };
  if (total_iters > 0) issue(0, 0);
  cp_async_commit();

  float dk_acc[D / 8][4], dv_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) dk_acc[i][j] = dv_acc[i][j] = 0.f;

  for (int iter = 0; iter < total_iters; ++iter) {
    const int st = iter & 1;
    if (iter + 1 < total_iters) {
      issue(iter + 1, st ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int m0 = m_start + (iter % q_tiles) * BM;
    const __nv_bfloat16* tQ = sQ + st * BM * LD;
    const __nv_bfloat16* tdO = sdO + st * BM * LD;
    const float* tLse = sLse + st * BM;
    const float* tDelta = sDelta + st * BM;

    // S^T = K Q^T and dP^T = V dO^T : [16 keys x 32 queries] per warp
    float sT[BM / 8][4], dpT[BM / 8][4];
#pragma unroll
    for (int i = 0; i < BM / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) sT[i][j] = dpT[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t ak[4], av[4];
      const int arow = warp * 16 + (lane & 15), acol = kk * 16 + (lane >> 4) * 8;
      ldmatrix_x4(ak, smem_u32(sK + arow * LD + acol));
      ldmatrix_x4(av, smem_u32(sV + arow * LD + acol));
#pragma unroll
      for (int np = 0; np < BM / 16; ++np) {
        const int brow = np * 16 + (lane & 7) + (lane >> 4) * 8, bcol = kk * 16 + ((lane >> 3) & 1) * 8;
        uint32_t bq[4], bd[4];
        ldmatrix_x4(bq, smem_u32(tQ + brow * LD + bcol));
        ldmatrix_x4(bd, smem_u32(tdO + brow * LD + bcol));
        mma_16816(sT[2 * np], ak, bq[0], bq[1]);
        mma_16816(sT[2 * np + 1], ak, bq[2], bq[3]);
        mma_16816(dpT[2 * np], av, bd[0], bd[1]);
        mma_16816(dpT[2 * np + 1], av, bd[2], bd[3]);
      }
    }
    // P^T = exp2(S^T*scale_log2 - lse*log2e) ; dS^T = P^T * (dP^T - delta) * scale
#pragma unroll
    for (int nt = 0; nt < BM / 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int qi = nt * 8 + fcol + (j & 1);            // query index in tile (column)
        const int key = n0 + warp * 16 + frow + ((j >> 1) << 3);
        const int row = m0 + qi;
        const bool ok = (key < klen) && (row < qlen) && (!p.causal || key <= row + off);
        const float pv = ok ? exp2f(sT[nt][j] * p.scale_log2 - tLse[qi] * kLog2e) : 0.f;
        sT[nt][j] = pv;
        dpT[nt][j] = pv * (dpT[nt][j] - tDelta[qi]) * p.scale;
      }
    }
    // dV += P^T dO ; dK += dS^T Q   (A from registers, B = [q][d] tiles via transposed ldmatrix)
#pragma unroll
    for (int kc = 0; kc < BM / 16; ++kc) {
      uint32_t ap[4], ads[4];
      ap[0] = pack_bf16(sT[2 * kc][0], sT[2 * kc][1]);
      ap[1] = pack_bf16(sT[2 * kc][2], sT[2 * kc][3]);
      ap[2] = pack_bf16(sT[2 * kc + 1][0], sT[2 * kc + 1][1]);
      ap[3] = pack_bf16(sT[2 * kc + 1][2], sT[2 * kc + 1][3]);
      ads[0] = pack_bf16(dpT[2 * kc][0], dpT[2 * kc][1]);
      ads[1] = pack_bf16(dpT[2 * kc][2], dpT[2 * kc][3]);
      ads[2] = pack_bf16(dpT[2 * kc + 1][0], dpT[2 * kc + 1][1]);
      ads[3] = pack_bf16(dpT[2 * kc + 1][2], dpT[2 * kc + 1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        const int brow = kc * 16 + (lane & 15), bcol = dp * 16 + (lane >> 4) * 8;
        uint32_t bdo[4], bq[4];
        ldmatrix_x4_trans(bdo, smem_u32(tdO + brow * LD + bcol));
        ldmatrix_x4_trans(bq, smem_u32(tQ + brow * LD + bcol));
        mma_16816(dv_acc[2 * dp], ap, bdo[0], bdo[1]);
        mma_16816(dv_acc[2 * dp + 1], ap, bdo[2], bdo[3]);
        mma_16816(dk_acc[2 * dp], ads, bq[0], bq[1]);
        mma_16816(dk_acc[2 * dp + 1], ads, bq[2], bq[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int key = n0 + warp * 16 + frow + r * 8;
    if (key >= klen) continue;
    __nv_bfloat16* dkrow = p.dk + head_offset(p.Lk, (long long)k0 + key, hk);
    __nv_bfloat16* dvrow = p.dv + head_offset(p.Lv, (long long)k0 + key, hk);
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      *reinterpret_cast<__nv_bfloat162*>(dkrow + dt * 8 + fcol) =
          __floats2bfloat162_rn(dk_acc[dt][2 * r], dk_acc[dt][2 * r + 1]);
      *reinterpret_cast<__nv_bfloat162*>(dvrow + dt * 8 + fcol) =
          __floats2bfloat162_rn(dv_acc[dt][2 * r], dv_acc[dt][2 * r + 1]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Backward, dQ.  CTA = 64 query rows of one q head; sweeps key tiles up to the diagonal.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) fa_bwd_dq_kernel(const AttnParams p) {
  constexpr int BM = 64, BN = 64, LD = D + 8, THREADS = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sdO = sQ + BM * LD;
  __nv_bfloat16* sK = sdO + BM * LD;          // 2 stages
  __nv_bfloat16* sV = sK + 2 * BN * LD;       // 2 stages

  const int b = blockIdx.z, h = blockIdx.y, mt = blockIdx.x;
  const int q0 = p.cu_q[b], qlen = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], klen = p.cu_k[b + 1] - k0;
  const int m0 = mt * BM;
  if (m0 >= qlen) return;
  const int hk = h / (p.nh / p.nkv);
  const int off = klen - qlen;
  int kmax = klen;
  if (p.causal) kmax = min(klen, m0 + BM + off);
  const int n_tiles = (kmax + BN - 1) / BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int frow = lane >> 2, fcol = (lane & 3) * 2;

  HeadLayout Ldo{p.o_stride_t, 0, p.nh, D};
  load_tile_async<BM, D, LD, THREADS>(sQ, p.q, p.Lq, h, q0, m0, qlen);
  load_tile_async<BM, D, LD, THREADS>(sdO, p.dout, Ldo, h, q0, m0, qlen);
  if (n_tiles > 0) {
    load_tile_async<BN, D, LD, THREADS>(sK, p.k, p.Lk, hk, k0, 0, klen);
    load_tile_async<BN, D, LD, THREADS>(sV, p.v, p.Lv, hk, k0, 0, klen);
  }
  cp_async_commit();

  float lse_r[2], delta_r[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = m0 + warp * 16 + frow + r * 8;
    const bool ok = row < qlen;
    lse_r[r] = ok ? p.lse[(long long)h * p.Tq + q0 + row] : INFINITY;
    delta_r[r] = ok ? p.delta[(long long)h * p.Tq + q0 + row] : 0.f;
  }

  float dq_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) dq_acc[i][j] = 0.f;

  for (int it = 0; it < n_tiles; ++it) {
    const int st = it & 1;
    if (it + 1 < n_tiles) {
      load_tile_async<BN, D, LD, THREADS>(sK + (st ^ 1) * BN * LD, p.k, p.Lk, hk, k0, (it + 1) * BN, klen);
      load_tile_async<BN, D, LD, THREADS>(sV + (st ^ 1) * BN * LD, p.v, p.Lv, hk, k0, (it + 1) * BN, klen);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* tK = sK + st * BN * LD;
    const __nv_bfloat16* tV = sV + st * BN * LD;

    float s[BN / 8][4], dp[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t aq[4], ado[4];
      const int arow = warp * 16 + (lane & 15), acol = kk * 16 + (lane >> 4) * 8;
      ldmatrix_x4(aq, smem_u32(sQ + arow * LD + acol));
      ldmatrix_x4(ado, smem_u32(sdO + arow * LD + acol));
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        const int brow = np * 16 + (lane & 7) + (lane >> 4) * 8, bcol = kk * 16 + ((lane >> 3) & 1) * 8;
        uint32_t bk[4], bv[4];
        ldmatrix_x4(bk, smem_u32(tK + brow * LD + bcol));
        ldmatrix_x4(bv, smem_u32(tV + brow * LD + bcol));
        mma_16816(s[2 * np], aq, bk[0], bk[1]);
        mma_16816(s[2 * np + 1], aq, bk[2], bk[3]);
        mma_16816(dp[2 * np], ado, bv[0], bv[1]);
        mma_16816(dp[2 * np + 1], ado, bv[2], bv[3]);
      }
    }
    const int kbase = it * BN;
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = kbase + nt * 8 + fcol + (j & 1);
        const int r = j >> 1;
        const int row = m0 + warp * 16 + frow + r * 8;
        const bool ok = (key < klen) && (row < qlen) && (!p.causal || key <= row + off);
        const float pv = ok ? exp2f(s[nt][j] * p.scale_log2 - lse_r[r] * kLog2e) : 0.f;
        dp[nt][j] = pv * (dp[nt][j] - delta_r[r]) * p.scale;
      }
    }
    // dQ += dS K
#pragma unroll
    for (int kc = 0; kc < BN / 16; ++kc) {
      uint32_t a[4];
      a[0] = pack_bf16(dp[2 * kc][0], dp[2 * kc][1]);
      a[1] = pack_bf16(dp[2 * kc][2], dp[2 * kc][3]);
      a[2] = pack_bf16(dp[2 * kc + 1][0], dp[2 * kc + 1][1]);
      a[3] = pack_bf16(dp[2 * kc + 1][2], dp[2 * kc + 1][3]);
#pragma unroll
      for (int dd = 0; dd < D / 16; ++dd) {
        uint32_t bk[4];
        ldmatrix_x4_trans(bk, smem_u32(tK + (kc * 16 + (lane & 15)) * LD + dd * 16 + (lane >> 4) * 8));
        mma_16816(dq_acc[2 * dd], a, bk[0], bk[1]);
        mma_16816(dq_acc[2 * dd + 1], a, bk[2], bk[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = m0 + warp * 16 + frow + r * 8;
    if (row >= qlen) continue;
    __nv_bfloat16* dqrow = p.dq + head_offset(p.Lq, (long long)q0 + row, h);
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      *reinterpret_cast<__nv_bfloat162*>(dqrow + dt * 8 + fcol) =
          __floats2bfloat162_rn(dq_acc[dt][2 * r], dq_acc[dt][2 * r + 1]);
    }
  }
}

template <int D>
static int launch_fwd(const AttnParams& p, int batch, int max_q, cudaStream_t st) {
  constexpr int LD = D + 8;
  const size_t smem = (size_t)(64 + 4 * 64) * LD * sizeof(__nv_bfloat16);
  cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((max_q + 63) / 64, p.nh, batch);
  fa_fwd_kernel<D><<<grid, 128, smem, st>>>(p);
  return (int)cudaGetLastError();
}

template <int D>
static int launch_bwd(const AttnParams& p, int batch, int max_q, int max_k, cudaStream_t st) {
  constexpr int LD = D + 8;
  {
    const long long warps = p.Tq * p.nh;
    const long long blocks = ceil_div(warps * 32, 256);
    fa_delta_kernel<D><<<(unsigned)blocks, 256, 0, st>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  {
    const size_t smem = (size_t)(2 * 64 + 4 * 32) * LD * sizeof(__nv_bfloat16) + 4 * 32 * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_dkdv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((max_k + 63) / 64, p.nkv, batch);
    fa_bwd_dkdv_kernel<D><<<grid, 128, smem, st>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  {
    const size_t smem = (size_t)(2 * 64 + 4 * 64) * LD * sizeof(__nv_bfloat16);
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((max_q + 63) / 64, p.nh, batch);
    fa_bwd_dq_kernel<D><<<grid, 128, smem, st>>>(p);
    return (int)cudaGetLastError();
  }
}

}  // namespace msrl

using namespace msrl;

// layout arrays: {stride_t, group_stride, heads_per_group, head_stride} for q, k, v (12 values)
static AttnParams make_params(const void* q, const void* k, const void* v, const long long* lay,
                              void* o, long long o_stride_t, float* lse, const int* cu_q,
                              const int* cu_k, int nh, int nkv, long long Tq, int D, int causal) {
  AttnParams p{};
  p.q = (const __nv_bfloat16*)q;
  p.k = (const __nv_bfloat16*)k;
  p.v = (const __nv_bfloat16*)v;
  p.Lq = HeadLayout{lay[0], (int)lay[1], (int)lay[2], (int)lay[3]};
  p.Lk = HeadLayout{lay[4], (int)lay[5], (int)lay[6], (int)lay[7]};
  p.Lv = HeadLayout{lay[8], (int)lay[9], (int)lay[10], (int)lay[11]};
  p.o = (__nv_bfloat16*)o;
  p.o_stride_t = o_stride_t;
  p.lse = lse;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.nh = nh;
  p.nkv = nkv;
  p.Tq = Tq;
  p.scale = 1.f / sqrtf((float)D);
  p.scale_log2 = p.scale * kLog2e;
  p.causal = causal;
  return p;
}

MSRL_API int msrl_flash_attn_varlen_fwd(const void* q, const void* k, const void* v,
                                        const long long* layouts12, void* o, long long o_stride_t,
                                        float* lse, const int* cu_q, const int* cu_k, int batch,
                                        int max_q, int nh, int nkv, long long Tq, int D,
                                        int causal, cudaStream_t st) {
  if (batch == 0 || Tq == 0) return 0;
  if (nh % nkv != 0) return (int)cudaErrorInvalidValue;
  AttnParams p = make_params(q, k, v, layouts12, o, o_stride_t, lse, cu_q, cu_k, nh, nkv, Tq, D, causal);
  if (D == 128) return launch_fwd<128>(p, batch, max_q, st);
  if (D == 64) return launch_fwd<64>(p, batch, max_q, st);
  return (int)cudaErrorInvalidValue;
}

// delta: fp32 scratch [nh, Tq]; dq/dk/dv use the same layouts as q/k/v.
MSRL_API int msrl_flash_attn_varlen_bwd(const void* q, const void* k, const void* v,
                                        const long long* layouts12, const void* o,
                                        const void* dout, long long o_stride_t, const float* lse,
                                        float* delta, void* dq, void* dk, void* dv,
                                        const int* cu_q, const int* cu_k, int batch, int max_q,
                                        int max_k, int nh, int nkv, long long Tq, int D, int causal,
                                        cudaStream_t st) {
  if (batch == 0 || Tq == 0) return 0;
  if (nh % nkv != 0) return (int)cudaErrorInvalidValue;
  AttnParams p = make_params(q, k, v, layouts12, const_cast<void*>(o), o_stride_t,
                             const_cast<float*>(lse), cu_q, cu_k, nh, nkv, Tq, D, causal);
  p.dout = (const __nv_bfloat16*)dout;
  p.delta = delta;
  p.dq = (__nv_bfloat16*)dq;
  p.dk = (__nv_bfloat16*)dk;
  p.dv = (__nv_bfloat16*)dv;
  if (D == 128) return launch_bwd<128>(p, batch, max_q, max_k, st);
  if (D == 64) return launch_bwd<64>(p, batch, max_q, max_k, st);
  return (int)cudaErrorInvalidValue;
}
