// Memory-bound fused ops: RMSNorm (fwd/bwd, optional residual add, per-head variant),
// RoPE (in place, fwd/bwd), SwiGLU (fwd/bwd), residual add, bias-grad column sums.
// All tensors bf16 with fp32 math; rows are moved with 128-bit loads/stores.
//
// Reference call sites these replace: flags use_fused_rmsnorm / use_fused_rotary_pos_emb /
// use_fused_swiglu / qk_layernorm (mindspeed_rl/config_cls/megatron_config.py:209-212,332).
#include "mma_utils.cuh"  // HeadLayout: addressing of heads inside fused QKV rows

namespace msrl {

// --------------------------------------------------------------------------------------------
// RMSNorm forward, one block per row.  Optional residual: s = x + res is written to sum_out
// and normalised (the "add + norm" pair between sub-layers).
// --------------------------------------------------------------------------------------------
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd_out, int H,
                   float eps) {
  __shared__ float red[32];
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  float* row = reinterpret_cast<float*>(dyn_smem);  // H floats: the (summed) row in fp32
  const long long r = blockIdx.x;
  const __nv_bfloat16* xr = x + r * H;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += THREADS) {
    float f[8];
    unpack8(ld8(xr + i * 8), f);
    if (res != nullptr) {
      float g[8];
      unpack8(ld8(res + r * H + i * 8), g);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += g[k];
      if (sum_out != nullptr) {
        bf16x8 s = pack8(f);
        st8(sum_out + r * H + i * 8, s);
        unpack8(s, f);  // normalise exactly what was stored
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      row[i * 8 + k] = f[k];
      ss += f[k] * f[k];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)H + eps);
  if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[r] = rstd;
  for (int i = threadIdx.x; i < nvec; i += THREADS) {
    float wv[8], o[8];
    unpack8(ld8(w + i * 8), wv);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = row[i * 8 + k] * rstd * wv[k];
    st8(y + r * H + i * 8, pack8(o));
  }
}

// Warp-per-row form (H <= 32 * VPT * 8): every warp owns whole rows (blockIdx / warp strided), reads a row
// into registers with VPT independent 16-byte loads per lane, reduces it with shuffles only (no block
// barrier anywhere), scales and stores it.  With five 128-thread blocks per SM about 140 KB of loads are in
// flight per SM, which is what a streaming kernel with a reduction in the middle needs to stay near the
// copy bandwidth.
template <int VPT, bool RES>
__global__ void __launch_bounds__(128)
rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                        const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                        __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd_out, long long rows,
                        int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  const long long warps = (long long)gridDim.x * 4;
  for (long long r = (long long)blockIdx.x * 4 + (threadIdx.x >> 5); r < rows; r += warps) {
    bf16x8 raw[VPT], raw_res[RES ? VPT : 1];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        raw[j] = ld8(x + r * H + i * 8);
        if (RES) raw_res[j] = ld8(res + r * H + i * 8);
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        float f[8];
        unpack8(raw[j], f);
        if (RES) {
          float g[8];
          unpack8(raw_res[j], g);
#pragma unroll
          for (int k = 0; k < 8; ++k) f[k] += g[k];
          raw[j] = pack8(f);                       // the rounded sum is what gets stored and normalised
          if (sum_out != nullptr) st8(sum_out + r * H + i * 8, raw[j]);
          unpack8(raw[j], f);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (lane == 0 && rstd_out != nullptr) rstd_out[r] = rstd;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        float f[8], wv[8], o[8];
        unpack8(raw[j], f);
        unpack8(ld8(w + i * 8), wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = f[k] * rstd * wv[k];
        st8(y + r * H + i * 8, pack8(o));
      }
    }
  }
}

// One-pass form for rows that fit the block's registers (H <= THREADS * VPT * 8).  Persistent blocks
// walk rows blockIdx.x, +gridDim.x, ...; the loads of the next row are issued before the current row
// is reduced, scaled and stored, so that a block always has a row in flight (no shared-memory staging
// of the row; with the optional residual the rounded sum is written back and normalised).
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_regs_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                        const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                        __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd_out, long long rows,
                        int H, float eps) {
  __shared__ float red[2][32];
  const int nvec = H >> 3;
  bf16x8 cur[VPT], cur_res[VPT], nxt[VPT], nxt_res[VPT];
  auto fetch = [&](long long r, bf16x8 (&dst)[VPT], bf16x8 (&dst_res)[VPT]) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nvec) {
        dst[j] = ld8(x + r * H + i * 8);
        if (res != nullptr) dst_res[j] = ld8(res + r * H + i * 8);
      }
    }
  };
  long long r = blockIdx.x;
  if (r < rows) fetch(r, cur, cur_res);
  int flip = 0;
  for (; r < rows; r += gridDim.x, flip ^= 1) {
    const long long rn = r + gridDim.x;
    if (rn < rows) fetch(rn, nxt, nxt_res);          // in flight while this row is processed
    float f[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nvec) {
        unpack8(cur[j], f[j]);
        if (res != nullptr) {
          float g[8];
          unpack8(cur_res[j], g);
#pragma unroll
          for (int k = 0; k < 8; ++k) f[j][k] += g[k];
          if (sum_out != nullptr) {
            const bf16x8 s = pack8(f[j]);
            st8(sum_out + r * H + i * 8, s);
            unpack8(s, f[j]);  // normalise exactly what was stored
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += f[j][k] * f[j][k];
      }
    }
    {   // block sum with alternating scratch: one barrier per row is enough
      const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
      ss = warp_sum(ss);
      if (lane == 0) red[flip][wid] = ss;
      __syncthreads();
      ss = warp_sum(lane < THREADS / 32 ? red[flip][lane] : 0.f);
    }
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[r] = rstd;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nvec) {
        float wv[8], o[8];
        unpack8(ld8(w + i * 8), wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = f[j][k] * rstd * wv[k];
        st8(y + r * H + i * 8, pack8(o));
      }
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      cur[j] = nxt[j];
      cur_res[j] = nxt_res[j];
    }
  }
}

// RMSNorm backward, stage 1: each block walks rows blockIdx.x, +gridDim.x, ... and
//   dx = rstd * (dy*w) - x * rstd^3 * mean(dy*w*x)   (optionally dx += dres)
// while keeping partial sums of dw = sum_rows dy * x * rstd in registers; the partials go to
// `dw_partial[gridDim.x, H]` (scratch) and stage 2 reduces them over blocks.
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, long long rows, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float dw_acc[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j)
#pragma unroll
    for (int k = 0; k < 8; ++k) dw_acc[j][k] = 0.f;

  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float rs = rstd[r];
    float g[VPT][8], xv[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nvec) {
        float d[8], wv[8];
        unpack8(ld8(dy + r * H + i * 8), d);
        unpack8(ld8(x + r * H + i * 8), xv[j]);
        unpack8(ld8(w + i * 8), wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          g[j][k] = d[k] * wv[k];
          dot += g[j][k] * xv[j][k];
          dw_acc[j][k] += d[k] * xv[j][k] * rs;
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * rs * rs * rs / (float)H;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = g[j][k] * rs - xv[j][k] * c;
        if (dres != nullptr) {
          float e[8];
          unpack8(ld8(dres + r * H + i * 8), e);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += e[k];
        }
        st8(dx + r * H + i * 8, pack8(o));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) dw_partial[(long long)blockIdx.x * H + i * 8 + k] = dw_acc[j][k];
    }
  }
}

// Stage 2: dw[h] (+)= sum_b partial[b, h].
__global__ void colsum_partials_kernel(const float* __restrict__ partial, int nblocks, int H,
                                       float* __restrict__ out_f32,
                                       __nv_bfloat16* __restrict__ out_bf16, int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[(long long)b * H + h];
  if (out_f32 != nullptr) out_f32[h] = accumulate ? out_f32[h] + s : s;
  if (out_bf16 != nullptr)
    out_bf16[h] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[h]) + s : s);
}

// --------------------------------------------------------------------------------------------
// Per-head RMSNorm (QK-norm): one warp per (token, head), head_dim <= 256, in place capable.
// --------------------------------------------------------------------------------------------
__global__ void headnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, HeadLayout L,
                                    const __nv_bfloat16* __restrict__ w,
                                    __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                    long long T, int nheads, int hd, float eps) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= T * nheads) return;
  const long long t = gw / nheads;
  const int h = (int)(gw % nheads);
  const long long off = head_offset(L, t, h);
  float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const bool act = lane * 8 < hd;
  if (act) unpack8(ld8(x + off + lane * 8), f);
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / (float)hd + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[gw] = rs;
  if (act) {
    float wv[8], o[8];
    unpack8(ld8(w + lane * 8), wv);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = f[k] * rs * wv[k];
    st8(y + off + lane * 8, pack8(o));
  }
}

// Backward of the per-head norm. dx overwrites dy in place (same layout); dw partial sums are
// accumulated per block into dw_partial[gridDim.x, hd].
__global__ void headnorm_bwd_kernel(__nv_bfloat16* __restrict__ dy_dx,
                                    const __nv_bfloat16* __restrict__ x, HeadLayout L,
                                    const __nv_bfloat16* __restrict__ w,
                                    const float* __restrict__ rstd, float* __restrict__ dw_partial,
                                    long long T, int nheads, int hd) {
  __shared__ float sdw[8][256];    // one row per warp (256 threads): summed in warp order, so that the
                                   // result does not depend on which warp finishes first
  const int lane = threadIdx.x & 31;
  const long long warps_total = ((long long)gridDim.x * blockDim.x) >> 5;
  const bool act = lane * 8 < hd;
  float dw_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; gw < T * nheads;
       gw += warps_total) {
    const long long t = gw / nheads;
    const int h = (int)(gw % nheads);
    const long long off = head_offset(L, t, h);
    const float rs = rstd[gw];
    float d[8] = {0, 0, 0, 0, 0, 0, 0, 0}, xv[8] = {0, 0, 0, 0, 0, 0, 0, 0}, wv[8], g[8];
    float dot = 0.f;
    if (act) {
      unpack8(ld8(dy_dx + off + lane * 8), d);
      unpack8(ld8(x + off + lane * 8), xv);
      unpack8(ld8(w + lane * 8), wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        g[k] = d[k] * wv[k];
        dot += g[k] * xv[k];
        dw_acc[k] += d[k] * xv[k] * rs;
      }
    }
    dot = warp_sum(dot);
    const float c = dot * rs * rs * rs / (float)hd;
    if (act) {
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = g[k] * rs - xv[k] * c;
      st8(dy_dx + off + lane * 8, pack8(o));
    }
  }
  const int warp = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < 8; ++k) sdw[warp][lane * 8 + k] = act ? dw_acc[k] : 0.f;
  __syncthreads();
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sdw[w][i];
    dw_partial[(long long)blockIdx.x * hd + i] = t;
  }
}

// --------------------------------------------------------------------------------------------
// RoPE (rotate-half / "neox" pairing: element i pairs with i + hd/2), in place.
// cos_sin table: [max_pos, hd] fp32 = [cos(0..hd/2) | sin(0..hd/2)] per position.
// sign = +1 forward, -1 backward (the inverse rotation applied to gradients).
// --------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ q, HeadLayout Lq, int nq,
                            __nv_bfloat16* __restrict__ k, HeadLayout Lk, int nk,
                            const int* __restrict__ positions, const float* __restrict__ cos_sin,
                            long long T, int hd, float sign) {
  // one thread rotates 4 pairs: (i..i+3, i+hd/2..i+hd/2+3)
  const int half = hd >> 1;
  const int per_head = half >> 2;
  const long long total = T * (long long)(nq + nk) * per_head;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % per_head);
    const long long th = idx / per_head;
    const int h = (int)(th % (nq + nk));
    const long long t = th / (nq + nk);
    __nv_bfloat16* base = (h < nq) ? q + head_offset(Lq, t, h) : k + head_offset(Lk, t, h - nq);
    const int pos = positions[t];
    const float4 cs = *reinterpret_cast<const float4*>(cos_sin + (long long)pos * hd + c * 4);
    const float4 sn = *reinterpret_cast<const float4*>(cos_sin + (long long)pos * hd + half + c * 4);
    uint2 lo_raw = *reinterpret_cast<const uint2*>(base + c * 4);
    uint2 hi_raw = *reinterpret_cast<const uint2*>(base + half + c * 4);
    __nv_bfloat162* lo = reinterpret_cast<__nv_bfloat162*>(&lo_raw);
    __nv_bfloat162* hi = reinterpret_cast<__nv_bfloat162*>(&hi_raw);
    const float cc[4] = {cs.x, cs.y, cs.z, cs.w};
    const float s4[4] = {sn.x * sign, sn.y * sign, sn.z * sign, sn.w * sign};
    float a[4], b[4];
    float2 t0 = __bfloat1622float2(lo[0]), t1 = __bfloat1622float2(lo[1]);
    float2 u0 = __bfloat1622float2(hi[0]), u1 = __bfloat1622float2(hi[1]);
    a[0] = t0.x; a[1] = t0.y; a[2] = t1.x; a[3] = t1.y;
    b[0] = u0.x; b[1] = u0.y; b[2] = u1.x; b[3] = u1.y;
    float ra[4], rb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      ra[j] = a[j] * cc[j] - b[j] * s4[j];
      rb[j] = b[j] * cc[j] + a[j] * s4[j];
    }
    lo[0] = __floats2bfloat162_rn(ra[0], ra[1]);
    lo[1] = __floats2bfloat162_rn(ra[2], ra[3]);
    hi[0] = __floats2bfloat162_rn(rb[0], rb[1]);
    hi[1] = __floats2bfloat162_rn(rb[2], rb[3]);
    *reinterpret_cast<uint2*>(base + c * 4) = lo_raw;
    *reinterpret_cast<uint2*>(base + half + c * 4) = hi_raw;
  }
}

// --------------------------------------------------------------------------------------------
// SwiGLU: in [T, 2F] = [gate | up] -> out [T, F] = silu(gate) * up
// --------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in,
                                  __nv_bfloat16* __restrict__ out, long long T, int F) {
  const int nvec = F >> 3;
  const long long total = T * nvec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int i = (int)(idx % nvec);
    float g[8], u[8], o[8];
    unpack8(ld8(in + t * 2 * F + i * 8), g);
    unpack8(ld8(in + t * 2 * F + F + i * 8), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    st8(out + t * F + i * 8, pack8(o));
  }
}

// dgate = dy * up * s * (1 + g*(1-s)),  dup = dy * g * s  with s = sigmoid(g); writes [T, 2F].
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ in,
                                  const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ din, long long T, int F) {
  const int nvec = F >> 3;
  const long long total = T * nvec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int i = (int)(idx % nvec);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(ld8(in + t * 2 * F + i * 8), g);
    unpack8(ld8(in + t * 2 * F + F + i * 8), u);
    unpack8(ld8(dy + t * F + i * 8), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = 1.f / (1.f + __expf(-g[k]));
      dg[k] = d[k] * u[k] * s * (1.f + g[k] * (1.f - s));
      du[k] = d[k] * g[k] * s;
    }
    st8(din + t * 2 * F + i * 8, pack8(dg));
    st8(din + t * 2 * F + F + i * 8, pack8(du));
  }
}

// out = a + b (bf16), n multiple of 8
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    unpack8(ld8(a + i * 8), x);
    unpack8(ld8(b + i * 8), y);
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] += y[k];
    st8(out + i * 8, pack8(x));
  }
}

// Column sums of a [rows, C] bf16 matrix into partial[gridDim.y, C] (bias gradients).
__global__ void colsum_rows_kernel(const __nv_bfloat16* __restrict__ m, long long rows, int C,
                                   float* __restrict__ partial) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (long long r = blockIdx.y; r < rows; r += gridDim.y) s += __bfloat162float(m[r * C + c]);
  partial[(long long)blockIdx.y * C + c] = s;
}

// Embedding gradient: g[id] += sum of the rows d[t] with ids[t] == id, rows of one id added in fp32 in
// token order (no atomics: bit-reproducible).  `order` lists the tokens sorted by id (stable), segment s
// covers order[seg_start[s] .. seg_start[s + 1]) and belongs to row seg_id[s] of g.  One block per
// segment, 16-byte column vectors strided over the threads.
template <typename G>
__global__ void __launch_bounds__(128)
embedding_grad_kernel(const __nv_bfloat16* __restrict__ d, long long ldd, const long long* __restrict__ order,
                      const long long* __restrict__ seg_start, const long long* __restrict__ seg_id,
                      G* __restrict__ g, long long ldg, int H) {
  const long long s = blockIdx.x;
  const long long t0 = seg_start[s], t1 = seg_start[s + 1];
  G* row = g + seg_id[s] * ldg;
  for (int c = threadIdx.x * 8; c < H; c += 128 * 8) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (long long t = t0; t < t1; ++t) {
      float f[8];
      unpack8(ld8(d + order[t] * ldd + c), f);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += f[k];
    }
    if (sizeof(G) == 2) {
      __nv_bfloat16* r16 = reinterpret_cast<__nv_bfloat16*>(row);
      float cur[8];
      unpack8(ld8(r16 + c), cur);
#pragma unroll
      for (int k = 0; k < 8; ++k) cur[k] += acc[k];
      st8(r16 + c, pack8(cur));
    } else {
      float* r32 = reinterpret_cast<float*>(row);
#pragma unroll
      for (int k = 0; k < 8; ++k) r32[c + k] += acc[k];
    }
  }
}

}  // namespace msrl

using namespace msrl;

static inline int grid_for(long long work_items, int threads, int per_sm = 8) {
  long long b = ceil_div(work_items, threads);
  long long cap = (long long)sm_count() * per_sm;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

MSRL_API int msrl_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out,
                              float* rstd, long long rows, int H, float eps, cudaStream_t st) {
  if (rows == 0) return 0;
  if (H % 8 != 0 || H > 16384) return (int)cudaErrorInvalidValue;
  if (H <= 32 * 16 * 8 && rows >= 4LL * sm_count()) {        // the usual hidden sizes, enough rows: a warp per row
    const long long cap = (long long)sm_count() * 3;        // three blocks fit the registers of an SM
    const long long want = (rows + 3) / 4;
    const unsigned blocks = (unsigned)(want < cap ? want : cap);
#define MSRL_RMS_WARP(V, R)                                                                            \
    rmsnorm_fwd_warp_kernel<V, R><<<blocks, 128, 0, st>>>(                                             \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, \
        (__nv_bfloat16*)sum_out, rstd, rows, H, eps)
    if (res != nullptr) {
      if (H <= 32 * 8 * 8) MSRL_RMS_WARP(8, true);
      else if (H <= 32 * 14 * 8) MSRL_RMS_WARP(14, true);
      else MSRL_RMS_WARP(16, true);
    } else {
      if (H <= 32 * 8 * 8) MSRL_RMS_WARP(8, false);
      else if (H <= 32 * 14 * 8) MSRL_RMS_WARP(14, false);
      else MSRL_RMS_WARP(16, false);
    }
#undef MSRL_RMS_WARP
    MSRL_LAUNCH_CHECK();
  }
  if (H <= 256 * 4 * 8) {        // few rows (decode steps) or wider rows: a block per row, the row in registers
    // one wave of persistent blocks: four 128-thread (two 256-thread) blocks fit the registers of an SM
    const long long cap = (long long)sm_count() * (H <= 128 * 4 * 8 ? 4 : 2);
    const unsigned blocks = (unsigned)(rows < cap ? rows : cap);
    if (H <= 128 * 4 * 8)
      rmsnorm_fwd_regs_kernel<128, 4><<<blocks, 128, 0, st>>>(
          (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,
          (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, rstd, rows, H, eps);
    else
      rmsnorm_fwd_regs_kernel<256, 4><<<blocks, 256, 0, st>>>(
          (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,
          (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, rstd, rows, H, eps);
    MSRL_LAUNCH_CHECK();
  }
  size_t smem = (size_t)H * sizeof(float);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(rmsnorm_fwd_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    attr_set = true;
  }
  rmsnorm_fwd_kernel<256><<<(unsigned)rows, 256, smem, st>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,
      (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, rstd, H, eps);
  MSRL_LAUNCH_CHECK();
}

// Number of blocks (= rows of the dw scratch) the backward uses for a given problem.
MSRL_API int msrl_rmsnorm_bwd_blocks(long long rows) {
  long long cap = (long long)sm_count() * 2;      // more blocks were measured slower (the partial sums cost cap x H floats)
  return (int)(rows < cap ? (rows < 1 ? 1 : rows) : cap);
}

// dw_partial: fp32 scratch of msrl_rmsnorm_bwd_blocks(rows) * H elements.
// dw_f32 / dw_bf16: either may be null; `accumulate` adds to the existing value.
MSRL_API int msrl_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                              const void* dres, void* dx, float* dw_partial, float* dw_f32,
                              void* dw_bf16, int accumulate, long long rows, int H,
                              cudaStream_t st) {
  if (rows == 0) return 0;
  if (H % 8 != 0 || H > 8192) return (int)cudaErrorInvalidValue;
  const int nb = msrl_rmsnorm_bwd_blocks(rows);
  const int nvec = H / 8;
#define LAUNCH_BWD(VPT)                                                                        \
  rmsnorm_bwd_kernel<256, VPT><<<nb, 256, 0, st>>>(                                            \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,        \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dw_partial, rows, H)
  if (nvec <= 256) LAUNCH_BWD(1);
  else if (nvec <= 512) LAUNCH_BWD(2);
  else if (nvec <= 768) LAUNCH_BWD(3);
  else LAUNCH_BWD(4);
#undef LAUNCH_BWD
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  colsum_partials_kernel<<<(H + 255) / 256, 256, 0, st>>>(dw_partial, nb, H, dw_f32,
                                                          (__nv_bfloat16*)dw_bf16, accumulate);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_headnorm_fwd(const void* x, long long stride_t, int group_stride, int hpg,
                               int head_stride, const void* w, void* y, float* rstd, long long T,
                               int nheads, int hd, float eps, cudaStream_t st) {
  if (T == 0) return 0;
  if (hd % 8 != 0 || hd > 256) return (int)cudaErrorInvalidValue;
  HeadLayout L{stride_t, group_stride, hpg, head_stride};
  const long long warps = T * nheads;
  const int threads = 256;
  const long long blocks = ceil_div(warps * 32, threads);
  headnorm_fwd_kernel<<<(unsigned)blocks, threads, 0, st>>>(
      (const __nv_bfloat16*)x, L, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, T, nheads, hd,
      eps);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_headnorm_bwd_blocks() { return sm_count() * 4; }

MSRL_API int msrl_headnorm_bwd(void* dy_dx, const void* x, long long stride_t, int group_stride,
                               int hpg, int head_stride, const void* w, const float* rstd,
                               float* dw_partial, float* dw_f32, void* dw_bf16, int accumulate,
                               long long T, int nheads, int hd, cudaStream_t st) {
  if (T == 0) return 0;
  if (hd % 8 != 0 || hd > 256) return (int)cudaErrorInvalidValue;
  HeadLayout L{stride_t, group_stride, hpg, head_stride};
  const int nb = msrl_headnorm_bwd_blocks();
  headnorm_bwd_kernel<<<nb, 256, 0, st>>>((__nv_bfloat16*)dy_dx, (const __nv_bfloat16*)x, L,
                                          (const __nv_bfloat16*)w, rstd, dw_partial, T, nheads, hd);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  colsum_partials_kernel<<<(hd + 255) / 256, 256, 0, st>>>(dw_partial, nb, hd, dw_f32,
                                                           (__nv_bfloat16*)dw_bf16, accumulate);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_rope(void* q, long long q_stride_t, int q_group_stride, int q_hpg,
                       int q_head_stride, int nq, void* k, long long k_stride_t, int k_group_stride,
                       int k_hpg, int k_head_stride, int nk, const int* positions,
                       const float* cos_sin, long long T, int hd, float sign, cudaStream_t st) {
  if (T == 0) return 0;
  if (hd % 8 != 0) return (int)cudaErrorInvalidValue;
  HeadLayout Lq{q_stride_t, q_group_stride, q_hpg, q_head_stride};
  HeadLayout Lk{k_stride_t, k_group_stride, k_hpg > 0 ? k_hpg : 1, k_head_stride};
  const long long total = T * (long long)(nq + nk) * (hd / 8);
  rope_kernel<<<grid_for(total, 256), 256, 0, st>>>((__nv_bfloat16*)q, Lq, nq, (__nv_bfloat16*)k,
                                                    Lk, nk, positions, cos_sin, T, hd, sign);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_swiglu_fwd(const void* in, void* out, long long T, int F, cudaStream_t st) {
  if (T == 0) return 0;
  if (F % 8 != 0) return (int)cudaErrorInvalidValue;
  swiglu_fwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)in,
                                                                (__nv_bfloat16*)out, T, F);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_swiglu_bwd(const void* in, const void* dy, void* din, long long T, int F,
                             cudaStream_t st) {
  if (T == 0) return 0;
  if (F % 8 != 0) return (int)cudaErrorInvalidValue;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, st>>>(
      (const __nv_bfloat16*)in, (const __nv_bfloat16*)dy, (__nv_bfloat16*)din, T, F);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_add(const void* a, const void* b, void* out, long long n, cudaStream_t st) {
  if (n == 0) return 0;
  if (n % 8 != 0) return (int)cudaErrorInvalidValue;
  add_kernel<<<grid_for(n / 8, 256), 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                   (__nv_bfloat16*)out, n / 8);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_colsum_blocks() { return 64; }

// Bias gradient: out[c] (+)= sum_r m[r, c]; partial is fp32 scratch [msrl_colsum_blocks(), C].
MSRL_API int msrl_colsum(const void* m, long long rows, int C, float* partial, float* out_f32,
                         void* out_bf16, int accumulate, cudaStream_t st) {
  if (rows == 0 || C == 0) return 0;
  const int nb = msrl_colsum_blocks();
  dim3 grid((C + 127) / 128, nb);
  colsum_rows_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)m, rows, C, partial);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  colsum_partials_kernel<<<(C + 255) / 256, 256, 0, st>>>(partial, nb, C, out_f32,
                                                          (__nv_bfloat16*)out_bf16, accumulate);
  MSRL_LAUNCH_CHECK();
}

// g[seg_id[s]] += sum over t in [seg_start[s], seg_start[s+1]) of d[order[t]]   (see embedding_grad_kernel).
// d bf16 [T, H] (row pitch ldd), g bf16 or fp32 [V, H] (row pitch ldg); H a multiple of 8, rows 16-byte aligned.
MSRL_API int msrl_embedding_grad(const void* d, long long ldd, const long long* order, const long long* seg_start,
                                 const long long* seg_id, long long n_seg, void* g, long long ldg, int g_is_f32,
                                 int H, cudaStream_t st) {
  if (n_seg == 0) return 0;
  if (H % 8 != 0 || ldd % 8 != 0 || ldg % 8 != 0 || n_seg > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (g_is_f32)
    embedding_grad_kernel<float><<<(unsigned)n_seg, 128, 0, st>>>((const __nv_bfloat16*)d, ldd, order, seg_start,
                                                                  seg_id, (float*)g, ldg, H);
  else
    embedding_grad_kernel<__nv_bfloat16><<<(unsigned)n_seg, 128, 0, st>>>((const __nv_bfloat16*)d, ldd, order,
                                                                          seg_start, seg_id, (__nv_bfloat16*)g, ldg, H);
  MSRL_LAUNCH_CHECK();
}
