// Merge of two partial attention results over disjoint key sets (ring attention, split-KV):
//   lse' = log(exp(lse_a) + exp(lse_b)),  out' = out_a * exp(lse_a - lse') + out_b * exp(lse_b - lse')
// The running result (fp32 out [T, nh, hd], lse [nh, T]) is updated in place with a block result
// (bf16 out [Tb, nh*hd], fp32 lse [nh, Tb]); `rows` optionally maps block row i to running row rows[i].
// One warp per (block row, head).
#include "common.cuh"

namespace msrl {

__global__ void attn_merge_kernel(float* __restrict__ acc_o, float* __restrict__ acc_l, long long T,
                                  const __nv_bfloat16* __restrict__ o, const float* __restrict__ l, long long Tb,
                                  const long long* __restrict__ rows, int nh, int hd) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= Tb * nh) return;
  const long long i = w / nh;
  const int h = (int)(w % nh);
  const long long t = rows != nullptr ? rows[i] : i;
  const float la = acc_l[(long long)h * T + t], lb = l[(long long)h * Tb + i];
  const float m = fmaxf(la, lb);
  float wa, wb, lt;
  if (m == -INFINITY) {          // neither side saw a key
    wa = wb = 0.f;
    lt = -INFINITY;
  } else {
    const float ea = __expf(la - m), eb = __expf(lb - m);
    lt = m + __logf(ea + eb);
    wa = ea / (ea + eb);
    wb = eb / (ea + eb);
  }
  float* pa = acc_o + (t * nh + h) * hd;
  const __nv_bfloat16* pb = o + (i * nh + h) * hd;
  for (int c = lane * 8; c < hd; c += 256) {
    float f[8];
    unpack8(ld8(pb + c), f);
    float4 a0 = *reinterpret_cast<float4*>(pa + c), a1 = *reinterpret_cast<float4*>(pa + c + 4);
    a0.x = a0.x * wa + f[0] * wb; a0.y = a0.y * wa + f[1] * wb; a0.z = a0.z * wa + f[2] * wb; a0.w = a0.w * wa + f[3] * wb;
    a1.x = a1.x * wa + f[4] * wb; a1.y = a1.y * wa + f[5] * wb; a1.z = a1.z * wa + f[6] * wb; a1.w = a1.w * wa + f[7] * wb;
    *reinterpret_cast<float4*>(pa + c) = a0;
    *reinterpret_cast<float4*>(pa + c + 4) = a1;
  }
  __syncwarp();
  if (lane == 0) acc_l[(long long)h * T + t] = lt;
}

}  // namespace msrl

using namespace msrl;

// hd must be a multiple of 8; acc_o and o 16-byte aligned.
MSRL_API int msrl_attn_merge(float* acc_o, float* acc_l, long long T, const void* o, const float* l, long long Tb,
                             const long long* rows, int nh, int hd, cudaStream_t st) {
  if (hd % 8 != 0) return (int)cudaErrorInvalidValue;
  const long long warps = Tb * nh;
  if (warps == 0) return 0;
  attn_merge_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(acc_o, acc_l, T, (const __nv_bfloat16*)o, l, Tb, rows,
                                                                 nh, hd);
  return (int)cudaGetLastError();
}
