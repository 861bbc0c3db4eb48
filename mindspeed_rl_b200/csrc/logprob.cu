// Row-wise log-softmax statistics over (a shard of) the vocabulary: per token the running
// max, sum-exp, target logit and sum e^{z-m} z, from which log p(label) and the entropy
// follow after a tiny cross-shard combine; and the matching backward that overwrites the logits
// with d loss / d logits.  Used by the chunked LM-head path (logits of a token chunk live only
// between the two GEMMs) and as the epilogue maths of the fused tcgen05 LM-head kernel.
//
// Reference semantics: vocab-parallel cross entropy and entropy with 3 all-reduces each
// (mindspeed_rl/utils/compute.py:29-97); here the shards' 4-float records are combined once.
#include "common.cuh"

namespace msrl {

struct RowStat {
  float m;    // max of z over the shard
  float s;    // sum exp(z - m)
  float zy;   // z[label] if the label lives in this shard else 0
  float spz;  // sum exp(z - m) * z
};

__global__ void __launch_bounds__(256)
logprob_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long row_stride, int V,
                     int vocab_offset, const long long* __restrict__ labels, float inv_temp,
                     RowStat* __restrict__ out) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  const __nv_bfloat16* row = logits + r * row_stride;
  const int nvec = V >> 3;
  float m = -INFINITY, s = 0.f, spz = 0.f;
  for (int i = threadIdx.x; i < nvec; i += 256) {
    float f[8];
    unpack8(ld8(row + i * 8), f);
    float lm = -INFINITY;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      f[k] *= inv_temp;
      lm = fmaxf(lm, f[k]);
    }
    if (lm > m) {
      const float c = __expf(m - lm);
      s *= c;
      spz *= c;
      m = lm;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float e = __expf(f[k] - m);
      s += e;
      spz += e * f[k];
    }
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += 256) {  // tail (V % 8)
    const float z = __bfloat162float(row[i]) * inv_temp;
    if (z > m) {
      const float c = __expf(m - z);
      s *= c;
      spz *= c;
      m = z;
    }
    const float e = __expf(z - m);
    s += e;
    spz += e * z;
  }
  const float bm = block_max(m, red);
  const float c = (m == -INFINITY) ? 0.f : __expf(m - bm);
  const float bs = block_sum(s * c, red);
  const float bspz = block_sum(spz * c, red);
  if (threadIdx.x == 0) {
    const long long y = labels[r] - vocab_offset;
    RowStat o;
    o.m = bm;
    o.s = bs;
    o.spz = bspz;
    o.zy = (y >= 0 && y < V) ? __bfloat162float(row[y]) * inv_temp : 0.f;
    out[r] = o;
  }
}

// Combine `nshard` records per row ([nshard, T] layout) -> logp, entropy, lse.
__global__ void logprob_finish_kernel(const RowStat* __restrict__ st, int nshard, long long T,
                                      float* __restrict__ logp, float* __restrict__ entropy,
                                      float* __restrict__ lse_out) {
  const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= T) return;
  float m = -INFINITY;
  for (int k = 0; k < nshard; ++k) m = fmaxf(m, st[(long long)k * T + r].m);
  float s = 0.f, spz = 0.f, zy = 0.f;
  for (int k = 0; k < nshard; ++k) {
    const RowStat a = st[(long long)k * T + r];
    const float c = __expf(a.m - m);
    s += a.s * c;
    spz += a.spz * c;
    zy += a.zy;
  }
  const float lse = m + __logf(s);
  logp[r] = zy - lse;
  if (entropy != nullptr) entropy[r] = lse - spz / s;
  if (lse_out != nullptr) lse_out[r] = lse;
}

// In place: logits <- d loss / d logits
//   dz_j = dlogp * (1[j == y] - p_j) + dent * p_j * ((lse - H) - z_j),  dlogit = dz * inv_temp
__global__ void __launch_bounds__(256)
logprob_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long row_stride, int V,
                   int vocab_offset, const long long* __restrict__ labels, float inv_temp,
                   const float* __restrict__ lse, const float* __restrict__ entropy,
                   const float* __restrict__ dlogp, const float* __restrict__ dent) {
  const long long r = blockIdx.x;
  __nv_bfloat16* row = logits + r * row_stride;
  const float l = lse[r];
  const float g = dlogp[r];
  const float ge = (dent != nullptr) ? dent[r] : 0.f;
  const float mean_z = (entropy != nullptr) ? (l - entropy[r]) : 0.f;
  const long long y = labels[r] - vocab_offset;
  const int nvec = V >> 3;
  for (int i = threadIdx.x; i < nvec; i += 256) {
    float f[8];
    unpack8(ld8(row + i * 8), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float z = f[k] * inv_temp;
      const float pj = __expf(z - l);
      float d = -g * pj + ge * pj * (mean_z - z);
      if ((long long)(i * 8 + k) == y) d += g;
      f[k] = d * inv_temp;
    }
    st8(row + i * 8, pack8(f));
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += 256) {
    const float z = __bfloat162float(row[i]) * inv_temp;
    const float pj = __expf(z - l);
    float d = -g * pj + ge * pj * (mean_z - z);
    if ((long long)i == y) d += g;
    row[i] = __float2bfloat16(d * inv_temp);
  }
}

}  // namespace msrl

using namespace msrl;

MSRL_API int msrl_logprob_stats(const void* logits, long long row_stride, long long T, int V,
                                int vocab_offset, const long long* labels, float inv_temp,
                                void* stats_out, cudaStream_t st) {
  if (T == 0) return 0;
  if (row_stride % 8 != 0) return (int)cudaErrorInvalidValue;
  logprob_stats_kernel<<<(unsigned)T, 256, 0, st>>>((const __nv_bfloat16*)logits, row_stride, V,
                                                    vocab_offset, labels, inv_temp,
                                                    (RowStat*)stats_out);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_logprob_finish(const void* stats, int nshard, long long T, float* logp,
                                 float* entropy, float* lse, cudaStream_t st) {
  if (T == 0) return 0;
  logprob_finish_kernel<<<(unsigned)ceil_div(T, 256), 256, 0, st>>>((const RowStat*)stats, nshard, T,
                                                                   logp, entropy, lse);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_logprob_bwd(void* logits, long long row_stride, long long T, int V,
                              int vocab_offset, const long long* labels, float inv_temp,
                              const float* lse, const float* entropy, const float* dlogp,
                              const float* dent, cudaStream_t st) {
  if (T == 0) return 0;
  if (row_stride % 8 != 0) return (int)cudaErrorInvalidValue;
  logprob_bwd_kernel<<<(unsigned)T, 256, 0, st>>>((__nv_bfloat16*)logits, row_stride, V,
                                                  vocab_offset, labels, inv_temp, lse, entropy,
                                                  dlogp, dent);
  MSRL_LAUNCH_CHECK();
}
