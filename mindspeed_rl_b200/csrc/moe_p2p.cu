// Expert-parallel token dispatch and combine over peer-mapped memory (one NVSwitch domain).
//
// Instead of an all-to-all collective, every rank writes its routed token rows straight into the
// expert slabs of the destination ranks (plain 16-byte stores over NVLink), and pulls the expert
// outputs it needs back with plain loads while it combines them:
//
//   publish   my per-expert slot counts -> row `me` of every peer's count table       (peer stores)
//   -- device barrier --
//   layout    from the full count table every rank derives, without further talk, where its own
//             slots start inside every destination's slab (segments per local expert, ordered by
//             source rank, padded to 128 rows), and for itself as destination: counts, padded
//             offsets and the expert of every 128-row tile (the grouped GEMM's plan)
//   dispatch  x[token] (optionally scaled) -> destination slab rows; the route (rank, row) of every
//             slot is kept for the way back; the destination zeroes its own pad rows
//   -- device barrier --     grouped expert GEMMs on the slab     -- device barrier --
//   combine   out[token] = sum_k w * y_peer[rank(slot)][row(slot)]                     (peer loads)
//
// The barriers are the symmetric arena's (symm.cu); buffers are reused layer after layer, which the
// barrier order makes safe.  A slab that would overflow raises a status code instead of writing.
// Reference behaviour: all-to-all token dispatcher of the expert-parallel MoE layer
// (mindspeed_rl/models/rollout/vllm_adapter/fused_moe.py:230-503; flag moe_token_dispatcher_type).
#include "common.cuh"

namespace msrl {

constexpr int P2P_MAX_RANKS = 16;
constexpr int P2P_PAD = 128;
struct P2PPeers {
  void* p[P2P_MAX_RANKS];
};

__global__ void moe_p2p_publish_kernel(const __grid_constant__ P2PPeers tables, const int* counts, int n_total, int me) {
  int* dst = reinterpret_cast<int*>(tables.p[blockIdx.x]) + (long long)me * n_total;
  for (int i = threadIdx.x; i < n_total; i += blockDim.x) dst[i] = counts[i];
}

// One block of 1024 threads.  all_counts [ep][ep * e_local] (row = source rank).
__global__ void __launch_bounds__(1024)
moe_p2p_layout_kernel(const int* all_counts, int ep, int e_local, int me, int cap_rows, int* my_base, int* counts_l,
                      int* offsets_l, int* tile_expert, int* status, int* overflow) {
  __shared__ int padded[1024];
  const int n_total = ep * e_local;
  // every (destination, local expert) pair g: rows before mine, total rows
  for (int g = threadIdx.x; g < n_total; g += blockDim.x) {
    int before = 0, total = 0;
    for (int s = 0; s < ep; ++s) {
      const int c = all_counts[(long long)s * n_total + g];
      if (s < me) before += c;
      total += c;
    }
    my_base[g] = before;                      // completed below with the segment offset
    padded[g] = (total + P2P_PAD - 1) / P2P_PAD * P2P_PAD;
    if (g / e_local == me) counts_l[g % e_local] = total;
  }
  __syncthreads();
  // per destination: exclusive scan of the padded segment sizes over its local experts
  for (int d = threadIdx.x; d < ep; d += blockDim.x) {
    int run = 0;
    for (int e = 0; e < e_local; ++e) {
      const int g = d * e_local + e;
      const int sz = padded[g];
      my_base[g] += run;
      if (d == me) offsets_l[e] = run;
      run += sz;
    }
    // every member evaluates every destination from the same table, so all of them reach the same
    // verdict and can leave the peer-memory path together
    if (overflow != nullptr && run > cap_rows) atomicMax(overflow, 1);
    if (d == me) {
      offsets_l[e_local] = run;
      if (status != nullptr && run > cap_rows) atomicCAS(status, 0, 300 + me);     // this rank's slab would overflow
    }
  }
  __syncthreads();
  const int max_tiles = cap_rows / P2P_PAD;
  const int used = min(offsets_l[e_local], cap_rows) / P2P_PAD;
  for (int e = threadIdx.x; e < e_local; e += blockDim.x)
    for (int t = offsets_l[e] / P2P_PAD; t < offsets_l[e + 1] / P2P_PAD && t < max_tiles; ++t) tile_expert[t] = e;
  for (int t = used + threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
}

// Blocks [0, T): one token each.  Blocks [T, T + e_local): zero the pad rows of my own slab.
__global__ void __launch_bounds__(128)
moe_p2p_dispatch_kernel(const __nv_bfloat16* x, long long ldx, const long long* expert_of, const int* plan_pos,
                        const int* plan_offsets, const float* w, int T, int k, int H, int e_local, int cap_rows,
                        const int* my_base, const __grid_constant__ P2PPeers slabs, int me, const int* counts_l,
                        const int* offsets_l, int* slot_rank, int* slot_row) {
  const int b = blockIdx.x;
  if (b < T) {
    for (int j = 0; j < k; ++j) {
      const int slot = b * k + j;
      const int g = (int)expert_of[slot];
      const int d = g / e_local;
      const int row = my_base[g] + (plan_pos[slot] - plan_offsets[g]);
      if (threadIdx.x == 0) {
        slot_rank[slot] = d;
        slot_row[slot] = row;
      }
      if (row >= cap_rows) continue;                         // overflow: flagged by the destination's layout
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(slabs.p[d]) + (long long)row * H;
      const float s = w != nullptr ? w[slot] : 1.f;
      for (int c = threadIdx.x * 8; c < H; c += 128 * 8) {
        bf16x8 v = ld8(x + (long long)b * ldx + c);
        if (w != nullptr) {
          float f[8];
          unpack8(v, f);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] *= s;
          v = pack8(f);
        }
        st8(dst + c, v);
      }
    }
  } else {
    const int e = b - T;
    const int r0 = offsets_l[e] + counts_l[e], r1 = min(offsets_l[e + 1], cap_rows);
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const bf16x8 z = pack8(f);
    __nv_bfloat16* mine = reinterpret_cast<__nv_bfloat16*>(slabs.p[me]);
    for (int r = r0; r < r1; ++r)
      for (int c = threadIdx.x * 8; c < H; c += 128 * 8) st8(mine + (long long)r * H + c, z);
  }
}

__global__ void __launch_bounds__(128)
moe_p2p_combine_kernel(const __grid_constant__ P2PPeers ybufs, const int* slot_rank, const int* slot_row, const float* w,
                       int k, int H, int cap_rows, __nv_bfloat16* out, long long ldo, __nv_bfloat16* keep_rows) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < H; c += 128 * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int slot = t * k + j;
      const int row = slot_row[slot];
      if (row >= cap_rows) continue;
      const bf16x8 v = ld8(reinterpret_cast<const __nv_bfloat16*>(ybufs.p[slot_rank[slot]]) + (long long)row * H + c);
      if (keep_rows != nullptr) st8(keep_rows + (long long)slot * H + c, v);
      float f[8];
      unpack8(v, f);
      const float s = w != nullptr ? w[slot] : 1.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += s * f[i];
    }
    st8(out + (long long)t * ldo + c, pack8(acc));
  }
}

}  // namespace msrl

using namespace msrl;

static P2PPeers p2p_peers(void* const* ptrs, int n) {
  P2PPeers p{};
  for (int i = 0; i < n && i < P2P_MAX_RANKS; ++i) p.p[i] = ptrs[i];
  return p;
}

MSRL_API int msrl_moe_p2p_max_ranks() { return P2P_MAX_RANKS; }

// tables: the ep members' addresses of the [ep, n_total] int count table
MSRL_API int msrl_moe_p2p_publish(void* const* tables, const int* counts, int n_total, int me, int ep, cudaStream_t st) {
  if (ep > P2P_MAX_RANKS) return (int)cudaErrorInvalidValue;
  moe_p2p_publish_kernel<<<ep, 256, 0, st>>>(p2p_peers(tables, ep), counts, n_total, me);
  return (int)cudaGetLastError();
}

MSRL_API int msrl_moe_p2p_layout(const int* all_counts, int ep, int e_local, int me, int cap_rows, int* my_base,
                                 int* counts_l, int* offsets_l, int* tile_expert, int* status, int* overflow,
                                 cudaStream_t st) {
  // `overflow` (optional, zeroed by the caller): set to 1 on EVERY member when any member's slab would
  // overflow; `status` (optional): 300 + me recorded when this rank's own slab would
  if (ep * e_local > 1024 || cap_rows % P2P_PAD != 0) return (int)cudaErrorInvalidValue;
  moe_p2p_layout_kernel<<<1, 1024, 0, st>>>(all_counts, ep, e_local, me, cap_rows, my_base, counts_l, offsets_l,
                                            tile_expert, status, overflow);
  return (int)cudaGetLastError();
}

MSRL_API int msrl_moe_p2p_dispatch(const void* x, long long ldx, const long long* expert_of, const int* plan_pos,
                                   const int* plan_offsets, const float* w, int T, int k, int H, int e_local,
                                   int cap_rows, const int* my_base, void* const* slabs, int me, int ep,
                                   const int* counts_l, const int* offsets_l, int* slot_rank, int* slot_row,
                                   cudaStream_t st) {
  if (H % 8 != 0 || ldx % 8 != 0 || ep > P2P_MAX_RANKS) return (int)cudaErrorInvalidValue;
  moe_p2p_dispatch_kernel<<<T + e_local, 128, 0, st>>>((const __nv_bfloat16*)x, ldx, expert_of, plan_pos, plan_offsets,
                                                       w, T, k, H, e_local, cap_rows, my_base, p2p_peers(slabs, ep),
                                                       me, counts_l, offsets_l, slot_rank, slot_row);
  return (int)cudaGetLastError();
}

MSRL_API int msrl_moe_p2p_combine(void* const* ybufs, int ep, const int* slot_rank, const int* slot_row, const float* w,
                                  int T, int k, int H, int cap_rows, void* out, long long ldo, void* keep_rows,
                                  cudaStream_t st) {
  if (H % 8 != 0 || ldo % 8 != 0 || ep > P2P_MAX_RANKS) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  moe_p2p_combine_kernel<<<T, 128, 0, st>>>(p2p_peers(ybufs, ep), slot_rank, slot_row, w, k, H, cap_rows,
                                            (__nv_bfloat16*)out, ldo, (__nv_bfloat16*)keep_rows);
  return (int)cudaGetLastError();
}
