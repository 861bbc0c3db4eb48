// Remove-padding packing on the device.
//
//  * pack_tokens:  padded [B, S] token ids + per-row prompt / response lengths + the (tiny, host
//    built) block offsets cu[B+1]  ->  packed ids [T], next-token labels [T] (0 at the last token
//    of a sequence and in padding) and position ids [T] that restart in every block;
//  * unpack_response: a per-token quantity of the packed stream (log-probs, entropies, values)
//    -> [B, W] rows that start at the position predicting the first response token
//    (prompt_len - 1) and are zero beyond the response length.
//
// One thread per output element; the owning sequence of a packed position is found by binary
// search in cu.  Replaces the Python index arithmetic of the reference
// (mindspeed_rl/utils/remove_padding.py:55-79,118-134; models/base/base_training_engine.py:367-371).
#include "common.cuh"

namespace msrl {

__device__ __forceinline__ int find_block(const int* __restrict__ cu, int nb, long long pos) {
  int lo = 0, hi = nb;                 // cu[lo] <= pos < cu[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu[mid] <= pos) lo = mid; else hi = mid;
  }
  return lo;
}

template <typename IdT>
__global__ void pack_tokens_kernel(const IdT* __restrict__ ids2d, long long ld, const int* __restrict__ p_len,
                                   const int* __restrict__ r_len, const int* __restrict__ cu, int B, int S,
                                   long long T, long long* __restrict__ out_ids, long long* __restrict__ out_labels,
                                   int* __restrict__ out_pos) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < T; t += stride) {
    const int b = find_block(cu, B, t);
    const int off = (int)(t - cu[b]);
    int len = p_len[b] + r_len[b];
    len = len < S ? len : S;
    const IdT* row = ids2d + (long long)b * ld;
    out_ids[t] = off < len ? (long long)row[off] : 0;
    out_labels[t] = off + 1 < len ? (long long)row[off + 1] : 0;
    out_pos[t] = off;
  }
}

template <typename T>
__global__ void unpack_response_kernel(const T* __restrict__ src, const int* __restrict__ cu, const int* __restrict__ p_len,
                                       const int* __restrict__ r_len, int B, int W, long long total,
                                       float* __restrict__ out) {
  const long long n = (long long)B * W;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int b = (int)(i / W), j = (int)(i % W);
    const long long t = (long long)cu[b] + p_len[b] - 1 + j;
    float v = 0.f;
    if (j < r_len[b] && t >= 0 && t < total) v = (float)src[t];
    out[i] = v;
  }
}

}  // namespace msrl

using namespace msrl;

// ids2d: [B, S] int32 (ids_are_i64 = 0) or int64 (1), row pitch ld elements.
MSRL_API int msrl_pack_tokens(const void* ids2d, int ids_are_i64, long long ld, const int* p_len, const int* r_len,
                              const int* cu, int B, int S, long long T, long long* out_ids, long long* out_labels,
                              int* out_pos, cudaStream_t st) {
  if (T <= 0 || B <= 0) return 0;
  const int threads = 256;
  const int blocks = (int)((T + threads - 1) / threads < 65535 ? (T + threads - 1) / threads : 65535);
  if (ids_are_i64)
    pack_tokens_kernel<long long><<<blocks, threads, 0, st>>>((const long long*)ids2d, ld, p_len, r_len, cu, B, S, T,
                                                              out_ids, out_labels, out_pos);
  else
    pack_tokens_kernel<int><<<blocks, threads, 0, st>>>((const int*)ids2d, ld, p_len, r_len, cu, B, S, T, out_ids,
                                                        out_labels, out_pos);
  MSRL_LAUNCH_CHECK();
}

// src: [total] fp32 (src_is_bf16 = 0) or bf16 (1); out: [B, W] fp32.
MSRL_API int msrl_unpack_response(const void* src, int src_is_bf16, const int* cu, const int* p_len, const int* r_len,
                                  int B, int W, long long total, float* out, cudaStream_t st) {
  const long long n = (long long)B * W;
  if (n <= 0) return 0;
  const int threads = 256;
  const int blocks = (int)((n + threads - 1) / threads < 65535 ? (n + threads - 1) / threads : 65535);
  if (src_is_bf16)
    unpack_response_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>((const __nv_bfloat16*)src, cu, p_len, r_len, B, W,
                                                                      total, out);
  else
    unpack_response_kernel<float><<<blocks, threads, 0, st>>>((const float*)src, cu, p_len, r_len, B, W, total, out);
  MSRL_LAUNCH_CHECK();
}
