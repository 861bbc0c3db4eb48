// RL objective kernels: clipped policy loss (GRPO / DAPO / PPO) with KL penalty evaluated
// forward and backward in one pass, clipped value loss, GAE reverse scan, group-normalised
// advantages.  fp32 throughout; inputs are the per-token [B, L] response tensors.
//
// Formulas follow the reference loss functions
// (mindspeed_rl/models/loss/grpo_actor_loss_func.py:100-144, dapo_actor_loss_func.py:105-152,
//  ppo_actor_loss_func.py:91-132, critic_loss_func.py:82-111, utils/compute.py:100-133,
//  trainer/utils/compute_utils.py:107-191).
#include "common.cuh"

namespace msrl {

enum KlKind { KL_NONE = 0, KL_PLAIN = 1, KL_ABS = 2, KL_MSE = 3, KL_LOW_VAR = 4 };

__device__ __forceinline__ void kl_value_grad(int kind, float lp, float ref, float& val, float& g) {
  const float d = lp - ref;
  switch (kind) {
    case KL_PLAIN: val = d; g = 1.f; break;
    case KL_ABS: val = fabsf(d); g = (d > 0.f) ? 1.f : ((d < 0.f) ? -1.f : 0.f); break;
    case KL_MSE: val = 0.5f * d * d; g = d; break;
    case KL_LOW_VAR: {
      const float kraw = -d;
      const float k = fminf(fmaxf(kraw, -20.f), 20.f);
      const float e = expf(k);
      const float v = e - k - 1.f;
      val = fminf(fmaxf(v, -10.f), 10.f);
      const bool pass = (kraw > -20.f && kraw < 20.f) && (v > -10.f && v < 10.f);
      g = pass ? -(e - 1.f) : 0.f;
      break;
    }
    default: val = 0.f; g = 0.f;
  }
}

// stats[0]=sum w_loss*pg  [1]=sum w_stat*clipped  [2]=sum w_stat*(old-lp)  [3]=sum w_stat*kl
// dlogp = w_loss * d pg/d lp + w_stat * kl_scale * kl_coef * d kl/d lp   (the KL term is always a
// token mean; kl_scale carries the gradient-accumulation scale that w_loss already contains)
// w_loss / w_stat already contain mask / normaliser (token-mean or seq-mean-token-mean).
__global__ void policy_loss_kernel(const float* __restrict__ logp, const float* __restrict__ old_logp,
                                   const float* __restrict__ ref_logp, const float* __restrict__ adv,
                                   const float* __restrict__ w_loss, const float* __restrict__ w_stat,
                                   float* __restrict__ dlogp, float* __restrict__ stats,
                                   long long n, float ratio_lo, float ratio_hi, float kl_coef,
                                   float kl_scale, int kl_kind) {
  __shared__ float red[32];
  float s_pg = 0.f, s_clip = 0.f, s_kl_old = 0.f, s_kl = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float wl = w_loss[i], ws = w_stat[i];
    float grad = 0.f;
    if (wl != 0.f || ws != 0.f) {
      const float lp = logp[i];
      const float old = (old_logp != nullptr) ? old_logp[i] : lp;
      const float a = adv[i];
      const float ratio = expf(lp - old);
      const float rc = fminf(fmaxf(ratio, ratio_lo), ratio_hi);
      const float l1 = -a * ratio, l2 = -a * rc;
      const bool in_range = (ratio >= ratio_lo) && (ratio <= ratio_hi);
      const float pg = fmaxf(l1, l2);
      // gradient of max(l1, l2): l1 branch -> -a*ratio ; l2 branch -> -a*ratio inside the
      // clamp range, 0 outside
      float dpg;
      if (l1 > l2) dpg = -a * ratio;
      else if (l2 > l1) dpg = in_range ? -a * ratio : 0.f;
      else dpg = in_range ? -a * ratio : 0.5f * (-a * ratio);
      s_pg += wl * pg;
      s_clip += ws * ((l2 > l1) ? 1.f : 0.f);
      s_kl_old += ws * (old - lp);
      grad = wl * dpg;
      if (kl_kind != KL_NONE && ref_logp != nullptr) {
        float kv, kg;
        kl_value_grad(kl_kind, lp, ref_logp[i], kv, kg);
        s_kl += ws * kv;
        grad += ws * kl_scale * kl_coef * kg;
      }
    }
    dlogp[i] = grad;
  }
  s_pg = block_sum(s_pg, red);
  s_clip = block_sum(s_clip, red);
  s_kl_old = block_sum(s_kl_old, red);
  s_kl = block_sum(s_kl, red);
  if (threadIdx.x == 0) {
    atomicAdd(&stats[0], s_pg);
    atomicAdd(&stats[1], s_clip);
    atomicAdd(&stats[2], s_kl_old);
    atomicAdd(&stats[3], s_kl);
  }
}

// Clipped value loss: 0.5 * sum w * max((v-R)^2, (clamp(v, vo-c, vo+c)-R)^2) ; dv per token.
__global__ void value_loss_kernel(const float* __restrict__ v, const float* __restrict__ v_old,
                                  const float* __restrict__ ret, const float* __restrict__ w,
                                  float* __restrict__ dv, float* __restrict__ stats, long long n,
                                  float clip) {
  __shared__ float red[32];
  float s_loss = 0.f, s_clip = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float wi = w[i];
    float g = 0.f;
    if (wi != 0.f) {
      const float vi = v[i], vo = v_old[i], r = ret[i];
      const float lo = vo - clip, hi = vo + clip;
      const float vc = fminf(fmaxf(vi, lo), hi);
      const float l1 = (vi - r) * (vi - r), l2 = (vc - r) * (vc - r);
      const bool in_range = (vi >= lo) && (vi <= hi);
      s_loss += 0.5f * wi * fmaxf(l1, l2);
      s_clip += wi * ((l2 > l1) ? 1.f : 0.f);
      if (l1 > l2) g = (vi - r);
      else if (l2 > l1) g = in_range ? (vc - r) : 0.f;
      else g = in_range ? (vi - r) : 0.5f * (vi - r);
      g *= wi;
    }
    dv[i] = g;
  }
  s_loss = block_sum(s_loss, red);
  s_clip = block_sum(s_clip, red);
  if (threadIdx.x == 0) {
    atomicAdd(&stats[0], s_loss);
    atomicAdd(&stats[1], s_clip);
  }
}

// GAE: one thread per row, reverse scan over the padded width (no mask inside the scan).
//   delta_t = r_t + gamma*v_{t+1} - v_t ; A_t = delta_t + gamma*lam*A_{t+1} ; ret = A + v
__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                           float* __restrict__ adv, float* __restrict__ ret, int B, int L,
                           float gamma, float lam) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const float* r = rewards + (long long)b * L;
  const float* v = values + (long long)b * L;
  float last = 0.f, next_v = 0.f;
  for (int t = L - 1; t >= 0; --t) {
    const float vt = v[t];
    const float delta = r[t] + gamma * next_v - vt;
    last = delta + gamma * lam * last;
    adv[(long long)b * L + t] = last;
    ret[(long long)b * L + t] = last + vt;
    next_v = vt;
  }
}

// Group-normalised advantage: scores [G, n]; a = (s - mean_g) / (std_g(unbiased) + eps),
// broadcast over L tokens and multiplied by mask. One block per sample row.
__global__ void group_norm_adv_kernel(const float* __restrict__ scores,
                                      const float* __restrict__ mask, float* __restrict__ adv,
                                      int n, int L, float eps) {
  const int row = blockIdx.x;
  const int g = row / n;
  double mean = 0.0;
  for (int j = 0; j < n; ++j) mean += (double)scores[g * n + j];
  mean /= (double)n;
  double var = 0.0;
  for (int j = 0; j < n; ++j) {
    const double d = (double)scores[g * n + j] - mean;
    var += d * d;
  }
  // torch.std of a single element is NaN; a group of one keeps that behaviour out of the way
  const double sd = (n > 1) ? sqrt(var / (double)(n - 1)) : 0.0;
  const float a = (float)(((double)scores[row] - mean) / (sd + (double)eps));
  for (int t = threadIdx.x; t < L; t += blockDim.x)
    adv[(long long)row * L + t] = a * mask[(long long)row * L + t];
}

}  // namespace msrl

using namespace msrl;

MSRL_API int msrl_policy_loss(const float* logp, const float* old_logp, const float* ref_logp,
                              const float* adv, const float* w_loss, const float* w_stat,
                              float* dlogp, float* stats4, long long n, float ratio_lo,
                              float ratio_hi, float kl_coef, float kl_scale, int kl_kind,
                              cudaStream_t st) {
  cudaMemsetAsync(stats4, 0, 4 * sizeof(float), st);
  if (n == 0) return 0;
  long long blocks = ceil_div(n, 256);
  if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
  policy_loss_kernel<<<(unsigned)blocks, 256, 0, st>>>(logp, old_logp, ref_logp, adv, w_loss, w_stat,
                                                       dlogp, stats4, n, ratio_lo, ratio_hi,
                                                       kl_coef, kl_scale, kl_kind);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_value_loss(const float* v, const float* v_old, const float* ret, const float* w,
                             float* dv, float* stats2, long long n, float clip, cudaStream_t st) {
  cudaMemsetAsync(stats2, 0, 2 * sizeof(float), st);
  if (n == 0) return 0;
  long long blocks = ceil_div(n, 256);
  if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
  value_loss_kernel<<<(unsigned)blocks, 256, 0, st>>>(v, v_old, ret, w, dv, stats2, n, clip);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_gae(const float* rewards, const float* values, float* adv, float* ret, int B,
                      int L, float gamma, float lam, cudaStream_t st) {
  if (B == 0 || L == 0) return 0;
  gae_kernel<<<(B + 63) / 64, 64, 0, st>>>(rewards, values, adv, ret, B, L, gamma, lam);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_group_norm_adv(const float* scores, const float* mask, float* adv, int rows,
                                 int n, int L, float eps, cudaStream_t st) {
  if (rows == 0 || L == 0) return 0;
  group_norm_adv_kernel<<<rows, 128, 0, st>>>(scores, mask, adv, n, L, eps);
  MSRL_LAUNCH_CHECK();
}
