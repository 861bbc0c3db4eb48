// Token movement of mixture-of-experts layers: dispatch plan, permute, combine.
//
//   plan      expert id of every (token, k) slot -> per-expert counts, 128-row padded segment
//             offsets, the destination row of every slot (stable: slots of an expert keep their
//             order), the expert of every 128-row tile.  Three small kernels, no host round trip:
//             the grouped GEMM's row count is bounded by slots + 128 * experts on the host side.
//   permute   x[token] (optionally scaled by the slot's weight) -> rows of the expert-grouped
//             buffer; pad rows of every segment are zeroed.
//   combine   out[token] = sum_k w[token, k] * y[row(token, k)]   (fp32 accumulation; w optional)
//   slot_dot  dw[token, k] = <dout[token], y[row(token, k)]>      (gradient of the combine weights)
//
// Reference behaviour: permute / unpermute around the grouped expert MLP in
// mindspeed_rl/models/rollout/vllm_adapter/fused_moe.py:230-373.
#include "common.cuh"

namespace msrl {

constexpr int PLAN_THREADS = 256;
constexpr int MOE_PAD = 128;

// A: per-block histogram + stable rank of each slot inside its block.
__global__ void __launch_bounds__(PLAN_THREADS)
moe_plan_local_kernel(const long long* expert_of, int n_slots, int n_experts, int* block_hist, int* local_rank) {
  extern __shared__ int sh[];                       // [warps][n_experts]
  const int warps = PLAN_THREADS / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < warps * n_experts; i += PLAN_THREADS) sh[i] = 0;
  __syncthreads();
  const int slot = blockIdx.x * PLAN_THREADS + threadIdx.x;
  const int e = slot < n_slots ? (int)expert_of[slot] : -1;
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) sh[warp * n_experts + e] = __popc(peers);
  __syncthreads();
  // exclusive scan over the warps, per expert
  for (int x = threadIdx.x; x < n_experts; x += PLAN_THREADS) {
    int run = 0;
    for (int w = 0; w < warps; ++w) {
      const int c = sh[w * n_experts + x];
      sh[w * n_experts + x] = run;
      run += c;
    }
    block_hist[(long long)blockIdx.x * n_experts + x] = run;
  }
  __syncthreads();
  if (e >= 0) local_rank[slot] = sh[warp * n_experts + e] + rank_in_warp;
}

// B: one block.  Scan the block histograms per expert (in place -> block offsets), pad the counts to
// 128 rows, scan them, fill the tile table.
__global__ void __launch_bounds__(1024)
moe_plan_scan_kernel(int* block_hist, int n_blocks, int n_experts, int* counts, int* offsets, int* tile_expert,
                     int max_tiles) {
  __shared__ int padded[1024];
  const int e = threadIdx.x;
  int total = 0;
  if (e < n_experts) {
    for (int b = 0; b < n_blocks; ++b) {
      const int c = block_hist[(long long)b * n_experts + e];
      block_hist[(long long)b * n_experts + e] = total;
      total += c;
    }
    counts[e] = total;
  }
  padded[e] = e < n_experts ? (total + MOE_PAD - 1) / MOE_PAD * MOE_PAD : 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < n_experts; ++i) {
      offsets[i] = run;
      run += padded[i];
    }
    offsets[n_experts] = run;
  }
  __syncthreads();
  if (e < n_experts) {
    const int t0 = offsets[e] / MOE_PAD, t1 = offsets[e + 1] / MOE_PAD;
    for (int t = t0; t < t1 && t < max_tiles; ++t) tile_expert[t] = e;
  }
  const int used = offsets[n_experts] / MOE_PAD;
  for (int t = used + threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
}

// C: destination row of every slot.
__global__ void moe_plan_pos_kernel(const long long* expert_of, int n_slots, int n_experts, const int* block_hist,
                                    const int* local_rank, const int* offsets, int* pos) {
  const int slot = blockIdx.x * PLAN_THREADS + threadIdx.x;
  if (slot >= n_slots) return;
  const int e = (int)expert_of[slot];
  pos[slot] = offsets[e] + block_hist[(long long)blockIdx.x * n_experts + e] + local_rank[slot];
}

// One block per token (blocks [0, T)) or per expert (blocks [T, T + E): zero the pad rows).
__global__ void __launch_bounds__(128)
moe_permute_kernel(const __nv_bfloat16* x, long long ldx, const int* pos, const float* w, int T, int k, int H,
                   const int* counts, const int* offsets, __nv_bfloat16* xp, long long ldp) {
  const int b = blockIdx.x;
  if (b < T) {
    for (int c = threadIdx.x * 8; c < H; c += 128 * 8) {
      const bf16x8 v = ld8(x + (long long)b * ldx + c);
      for (int j = 0; j < k; ++j) {
        const int r = pos[b * k + j];
        if (w == nullptr) {
          st8(xp + (long long)r * ldp + c, v);
        } else {
          float f[8];
          unpack8(v, f);
          const float s = w[b * k + j];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] *= s;
          st8(xp + (long long)r * ldp + c, pack8(f));
        }
      }
    }
  } else {
    const int e = b - T;
    const int r0 = offsets[e] + counts[e], r1 = offsets[e + 1];
    bf16x8 z;
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    z = pack8(f);
    for (int r = r0; r < r1; ++r)
      for (int c = threadIdx.x * 8; c < H; c += 128 * 8) st8(xp + (long long)r * ldp + c, z);
  }
}

__global__ void __launch_bounds__(128)
moe_combine_kernel(const __nv_bfloat16* y, long long ldy, const int* pos, const float* w, int k, int H,
                   __nv_bfloat16* out, long long ldo, int accumulate) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < H; c += 128 * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (accumulate) unpack8(ld8(out + (long long)t * ldo + c), acc);
    for (int j = 0; j < k; ++j) {
      float f[8];
      unpack8(ld8(y + (long long)pos[t * k + j] * ldy + c), f);
      const float s = w != nullptr ? w[t * k + j] : 1.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += s * f[i];
    }
    st8(out + (long long)t * ldo + c, pack8(acc));
  }
}

// one warp per slot
__global__ void moe_slot_dot_kernel(const __nv_bfloat16* dout, long long ldd, const __nv_bfloat16* y, long long ldy,
                                    const int* pos, int n_slots, int k, int H, float* dw) {
  const int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (slot >= n_slots) return;
  const __nv_bfloat16* a = dout + (long long)(slot / k) * ldd;
  const __nv_bfloat16* b = y + (long long)pos[slot] * ldy;
  float s = 0.f;
  for (int c = lane * 8; c < H; c += 32 * 8) {
    float fa[8], fb[8];
    unpack8(ld8(a + c), fa);
    unpack8(ld8(b + c), fb);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += fa[i] * fb[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) dw[slot] = s;
}

}  // namespace msrl

using namespace msrl;

// scratch: ints, at least moe_plan_scratch(n_slots, n_experts) of them
MSRL_API long long msrl_moe_plan_scratch(int n_slots, int n_experts) {
  const long long blocks = (n_slots + PLAN_THREADS - 1) / PLAN_THREADS;
  return blocks * n_experts + n_slots;
}

// expert_of [n_slots] int64 -> counts [E], offsets [E+1] (padded to 128), pos [n_slots],
// tile_expert [max_tiles]
MSRL_API int msrl_moe_plan(const long long* expert_of, int n_slots, int n_experts, int* scratch, int* counts,
                           int* offsets, int* pos, int* tile_expert, int max_tiles, cudaStream_t st) {
  if (n_experts > 1024 || n_experts <= 0) return (int)cudaErrorInvalidValue;
  const int blocks = (n_slots + PLAN_THREADS - 1) / PLAN_THREADS;
  int* block_hist = scratch;
  int* local_rank = scratch + (long long)blocks * n_experts;
  if (blocks > 0)
    moe_plan_local_kernel<<<blocks, PLAN_THREADS, (PLAN_THREADS / 32) * n_experts * sizeof(int), st>>>(
        expert_of, n_slots, n_experts, block_hist, local_rank);
  moe_plan_scan_kernel<<<1, 1024, 0, st>>>(block_hist, blocks, n_experts, counts, offsets, tile_expert, max_tiles);
  if (blocks > 0)
    moe_plan_pos_kernel<<<blocks, PLAN_THREADS, 0, st>>>(expert_of, n_slots, n_experts, block_hist, local_rank,
                                                         offsets, pos);
  return (int)cudaGetLastError();
}

// H and the leading dimensions must be multiples of 8, pointers 16-byte aligned.
MSRL_API int msrl_moe_permute(const void* x, long long ldx, const int* pos, const float* w, int T, int k, int H,
                              int n_experts, const int* counts, const int* offsets, void* xp, long long ldp,
                              cudaStream_t st) {
  if (H % 8 != 0 || ldx % 8 != 0 || ldp % 8 != 0) return (int)cudaErrorInvalidValue;
  if (T + n_experts == 0) return 0;
  moe_permute_kernel<<<T + n_experts, 128, 0, st>>>((const __nv_bfloat16*)x, ldx, pos, w, T, k, H, counts, offsets,
                                                    (__nv_bfloat16*)xp, ldp);
  return (int)cudaGetLastError();
}

MSRL_API int msrl_moe_combine(const void* y, long long ldy, const int* pos, const float* w, int T, int k, int H,
                              void* out, long long ldo, int accumulate, cudaStream_t st) {
  if (H % 8 != 0 || ldy % 8 != 0 || ldo % 8 != 0) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  moe_combine_kernel<<<T, 128, 0, st>>>((const __nv_bfloat16*)y, ldy, pos, w, k, H, (__nv_bfloat16*)out, ldo, accumulate);
  return (int)cudaGetLastError();
}

MSRL_API int msrl_moe_slot_dot(const void* dout, long long ldd, const void* y, long long ldy, const int* pos, int T,
                               int k, int H, float* dw, cudaStream_t st) {
  if (H % 8 != 0 || ldd % 8 != 0 || ldy % 8 != 0) return (int)cudaErrorInvalidValue;
  const int n = T * k;
  if (n == 0) return 0;
  moe_slot_dot_kernel<<<(n + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)dout, ldd, (const __nv_bfloat16*)y, ldy, pos,
                                                   n, k, H, dw);
  return (int)cudaGetLastError();
}
