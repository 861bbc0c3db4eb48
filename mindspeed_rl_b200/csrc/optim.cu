// Optimizer kernels over flat buffers: global grad-norm (sum of squares), clip coefficient on
// the device (no host round trip), fused AdamW that reads bf16/fp32 grads, updates fp32
// master weights + moments and emits the bf16 working copy in the same pass.
//
// Replaces the reference's `optimizer_selection: fused_adamw` dependency
// (docs/zh/features/swap_optimizer.md:25-33) and Megatron's clip_grad_norm.
#include "common.cuh"

namespace msrl {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = to_f32<T>(g[i]);
    s += v * v;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// Order-independent variant: every block stores its partial sum, then one block adds the partials in
// index order (a fixed tree), so the result is the same bit pattern on every run.
template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ g, long long n, float* __restrict__ partials) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = to_f32<T>(g[i]);
    s += v * v;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

__global__ void sumsq_finish_kernel(const float* __restrict__ partials, int n_part, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n_part; i += blockDim.x) s += partials[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) *out += s;
}

// coef = min(1, max_norm / (sqrt(sumsq) + 1e-6)) * extra_scale ; norm_out = sqrt(sumsq)
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float extra_scale,
                                 float* __restrict__ coef, float* __restrict__ norm_out) {
  const float norm = sqrtf(*sumsq);
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (norm + 1e-6f));
  *coef = c * extra_scale;
  *norm_out = norm;
}

template <typename G>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ g, __nv_bfloat16* __restrict__ p16, long long n,
                             float lr, float b1, float b2, float eps, float wd, float bc1,
                             float bc2, const float* __restrict__ grad_scale) {
  const float gs = (grad_scale != nullptr) ? *grad_scale : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gi = to_f32<G>(g[i]) * gs;
    float mi = m[i], vi = v[i], pi = p[i];
    mi = b1 * mi + (1.f - b1) * gi;
    vi = b2 * vi + (1.f - b2) * gi * gi;
    const float mhat = mi / bc1;
    const float vhat = vi / bc2;
    pi = pi * (1.f - lr * wd) - lr * mhat / (sqrtf(vhat) + eps);
    m[i] = mi;
    v[i] = vi;
    p[i] = pi;
    if (p16 != nullptr) p16[i] = __float2bfloat16(pi);
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                        long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}

}  // namespace msrl

using namespace msrl;

static inline unsigned stream_grid(long long n) {
  long long b = ceil_div(n, 256);
  long long cap = (long long)sm_count() * 8;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

// out must be zeroed by the caller before the first call of a norm computation; calls add up.
MSRL_API int msrl_sumsq(const void* g, int is_bf16, long long n, float* out, cudaStream_t st) {
  if (n == 0) return 0;
  if (is_bf16)
    sumsq_kernel<__nv_bfloat16><<<stream_grid(n), 256, 0, st>>>((const __nv_bfloat16*)g, n, out);
  else
    sumsq_kernel<float><<<stream_grid(n), 256, 0, st>>>((const float*)g, n, out);
  MSRL_LAUNCH_CHECK();
}

// partials: scratch of at least `max_blocks` floats
MSRL_API int msrl_sumsq_ordered(const void* g, int is_bf16, long long n, float* partials, int max_blocks, float* out,
                                cudaStream_t st) {
  if (n == 0) return 0;
  int grid = (int)stream_grid(n);
  if (grid > max_blocks) grid = max_blocks;
  if (grid < 1) return (int)cudaErrorInvalidValue;
  if (is_bf16)
    sumsq_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)g, n, partials);
  else
    sumsq_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)g, n, partials);
  sumsq_finish_kernel<<<1, 256, 0, st>>>(partials, grid, out);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_clip_coef(const float* sumsq, float max_norm, float extra_scale, float* coef,
                            float* norm_out, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(sumsq, max_norm, extra_scale, coef, norm_out);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_adamw(float* p, float* m, float* v, const void* g, int g_is_bf16, void* p16,
                        long long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                        float bc2, const float* grad_scale, cudaStream_t st) {
  if (n == 0) return 0;
  if (g_is_bf16)
    adamw_kernel<__nv_bfloat16><<<stream_grid(n), 256, 0, st>>>(
        p, m, v, (const __nv_bfloat16*)g, (__nv_bfloat16*)p16, n, lr, b1, b2, eps, wd, bc1, bc2,
        grad_scale);
  else
    adamw_kernel<float><<<stream_grid(n), 256, 0, st>>>(p, m, v, (const float*)g,
                                                        (__nv_bfloat16*)p16, n, lr, b1, b2, eps, wd,
                                                        bc1, bc2, grad_scale);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t st) {
  if (n == 0) return 0;
  cast_f32_to_bf16_kernel<<<stream_grid(n), 256, 0, st>>>(src, (__nv_bfloat16*)dst, n);
  MSRL_LAUNCH_CHECK();
}
