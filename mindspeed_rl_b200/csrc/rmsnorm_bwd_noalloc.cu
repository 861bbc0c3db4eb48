// Allocation-free RMSNorm backward: same mathematics as msrl_rmsnorm_bwd (elementwise.cu), with
// the partial weight-gradient sums kept in a scratch array that belongs to the library instead
// of a buffer the caller has to provide.  See rmsnorm_bwd_noalloc.h for who this is for, the size
// limit, the first-call set-up and the rule about overlapping calls.
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "rmsnorm_bwd_noalloc.h"

// One slab per GPU that loads this library: [MSRL_RMSNORM_NOALLOC_BLOCKS, MSRL_RMSNORM_NOALLOC_MAX_H]
// fp32 partial sums.  In host code this name is only a handle -- the device address is obtained
// once per device with cudaGetSymbolAddress and handed to the kernels as a pointer.
static __device__ __align__(256) float
    g_rmsnorm_noalloc_scratch[MSRL_RMSNORM_NOALLOC_BLOCKS * MSRL_RMSNORM_NOALLOC_MAX_H];

namespace {

using namespace msrl;

constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// Stage 1: block b walks rows b, b+gridDim.x, ...; writes dx and leaves its partial dw row in
// partial[b, 0..H).  Each block (re)writes its whole row, so stale contents are never read.
template <int VPT>
__global__ void __launch_bounds__(kThreads)
noalloc_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                           const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                           const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                           float* __restrict__ partial, long long rows, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float acc[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[j][k] = 0.f;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float rs = rstd[r];
    float g[VPT][8], xv[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = threadIdx.x + j * kThreads;
      if (i < nvec) {
        float d[8], wv[8];
        unpack8(ld8(dy + r * H + i * 8), d);
        unpack8(ld8(x + r * H + i * 8), xv[j]);
        unpack8(ld8(w + i * 8), wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          g[j][k] = d[k] * wv[k];
          dot += g[j][k] * xv[j][k];
          acc[j][k] += d[k] * xv[j][k] * rs;
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * rs * rs * rs / (float)H;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = threadIdx.x + j * kThreads;
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
    const int i = threadIdx.x + j * kThreads;
    if (i < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) partial[(long long)blockIdx.x * H + i * 8 + k] = acc[j][k];
    }
  }
}

// Stage 2: dw[h] (+)= sum_b partial[b, h] over the nblocks rows stage 1 just wrote.
__global__ void noalloc_reduce_kernel(const float* __restrict__ partial, int nblocks, int H,
                                      float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16,
                                      int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[(long long)b * H + h];
  if (out_f32 != nullptr) out_f32[h] = accumulate ? out_f32[h] + s : s;
  if (out_bf16 != nullptr)
    out_bf16[h] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[h]) + s : s);
}

std::mutex g_setup_mutex;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of this GPU's copy of the scratch array (looked up once per device, with that
// device current -- which it is, because the caller's launch targets the current device).
cudaError_t scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_noalloc_scratch);
    if (e != cudaSuccess) return e;
    if (p == nullptr) return cudaErrorInvalidSymbol;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int msrl_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                             const void* dres, void* dx, float* dw_f32, void* dw_bf16, int accumulate,
                             long long rows, int H, cudaStream_t stream) {
  if (H <= 0 || H % 8 != 0 || H > MSRL_RMSNORM_NOALLOC_MAX_H) {
    std::fprintf(stderr,
                 "msrl_rmsnorm_bwd_noalloc: hidden size %d is not supported (need a multiple of 8, at most "
                 "%d: the built-in scratch holds %d x %d floats). Use msrl_rmsnorm_bwd with a caller-provided "
                 "scratch buffer for larger rows.\n",
                 H, MSRL_RMSNORM_NOALLOC_MAX_H, MSRL_RMSNORM_NOALLOC_BLOCKS, MSRL_RMSNORM_NOALLOC_MAX_H);
    return (int)cudaErrorInvalidValue;
  }
  if (rows < 0) {
    std::fprintf(stderr, "msrl_rmsnorm_bwd_noalloc: negative row count %lld\n", rows);
    return (int)cudaErrorInvalidValue;
  }
  if (rows == 0) return (int)cudaSuccess;
  // The kernels move 128-bit vectors through these buffers: a missing or misaligned pointer must
  // become an error code here, not a fault on the GPU.
  const struct { const void* p; const char* name; bool required; } ptrs[] = {
      {dy, "dy", true}, {x, "x", true}, {w, "w", true}, {dx, "dx", true}, {dres, "dres", false}};
  for (const auto& a : ptrs) {
    if (a.p == nullptr ? a.required : (reinterpret_cast<uintptr_t>(a.p) & 15) != 0) {
      std::fprintf(stderr, "msrl_rmsnorm_bwd_noalloc: %s must be %s16-byte aligned device memory\n", a.name,
                   a.required ? "non-null, " : "null or ");
      return (int)cudaErrorInvalidValue;
    }
  }
  if (rstd == nullptr || (reinterpret_cast<uintptr_t>(rstd) & 3) != 0) {
    std::fprintf(stderr, "msrl_rmsnorm_bwd_noalloc: rstd must be non-null fp32 device memory\n");
    return (int)cudaErrorInvalidValue;
  }
  float* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) {
    std::fprintf(stderr, "msrl_rmsnorm_bwd_noalloc: cannot resolve the scratch array on this device: %s\n",
                 cudaGetErrorString(e));
    return (int)e;
  }
  const int nb = rows < MSRL_RMSNORM_NOALLOC_BLOCKS ? (int)rows : MSRL_RMSNORM_NOALLOC_BLOCKS;
  const int nvec = H / 8;
  const __nv_bfloat16* dyb = static_cast<const __nv_bfloat16*>(dy);
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wb = static_cast<const __nv_bfloat16*>(w);
  const __nv_bfloat16* rb = static_cast<const __nv_bfloat16*>(dres);
  __nv_bfloat16* dxb = static_cast<__nv_bfloat16*>(dx);
  if (nvec <= kThreads)
    noalloc_rmsnorm_bwd_kernel<1><<<nb, kThreads, 0, stream>>>(dyb, xb, wb, rstd, rb, dxb, scratch, rows, H);
  else if (nvec <= 2 * kThreads)
    noalloc_rmsnorm_bwd_kernel<2><<<nb, kThreads, 0, stream>>>(dyb, xb, wb, rstd, rb, dxb, scratch, rows, H);
  else if (nvec <= 3 * kThreads)
    noalloc_rmsnorm_bwd_kernel<3><<<nb, kThreads, 0, stream>>>(dyb, xb, wb, rstd, rb, dxb, scratch, rows, H);
  else
    noalloc_rmsnorm_bwd_kernel<4><<<nb, kThreads, 0, stream>>>(dyb, xb, wb, rstd, rb, dxb, scratch, rows, H);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (dw_f32 == nullptr && dw_bf16 == nullptr) return (int)cudaSuccess;   // weight gradient not wanted
  noalloc_reduce_kernel<<<(H + 255) / 256, 256, 0, stream>>>(scratch, nb, H, dw_f32,
                                                            static_cast<__nv_bfloat16*>(dw_bf16), accumulate);
  return (int)cudaGetLastError();
}
