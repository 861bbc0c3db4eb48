// Symmetric (peer-mapped) memory and the NVLink collectives built on it.
//
// Every rank of a team allocates one arena with cudaMalloc, exports it with a CUDA IPC handle and
// maps all peers' arenas; kernels then read / write peer memory directly with ordinary loads and
// stores over NVLink 5 / NVSwitch (no multicast TMA, no NCCL on these paths).
//
//  * device barrier: epoch flags in the arena, bounded spin, status word on expiry
//  * all-gather (pull):      dst[r*n .. ] = peer_r.src[0..n)
//  * reduce-scatter (pull):  out[i] = sum_r peer_r.src[shard*n + i]   (fp32 accumulation)
//  * copy plan (resharding): list of strided row-block copies peer -> local, optional
//    de-interleave is expressed through the plan itself
//
// Cross-GPU waits are bounded by a wall-clock limit; on expiry the kernel stores an error code
// in the caller's status word and returns.
#include <string.h>

#include "common.cuh"

namespace msrl {

constexpr int kMaxRanks = 16;
constexpr long long kBarrierCycles = 4000000000LL;   // ~2 s

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct Epochs {
  unsigned int e[kMaxRanks];
};

// flags.p[r] points at rank r's flag array (kMaxRanks x u32 at the start of its arena).  Slot
// [p] of my array is written only by peer p and counts the barriers p and I have shared, so
// barriers over different subsets of the team (mask) can interleave as long as every pair of
// ranks issues its common barriers in the same order.
__global__ void symm_barrier_kernel(const __grid_constant__ PeerPtrs flags, int rank, int world,
                                    const __grid_constant__ Epochs epochs, unsigned int mask, int* status) {
  const int r = threadIdx.x;
  __threadfence_system();   // earlier kernels' writes (local and peer) become visible first
  if (r < world && r != rank && ((mask >> r) & 1u)) {
    const unsigned int epoch = epochs.e[r];
    st_release_sys(reinterpret_cast<unsigned int*>(flags.p[r]) + rank, epoch);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(flags.p[rank]) + r;
    const long long t0 = clock64();
    // epochs only grow; ">=" in wrap-around arithmetic
    while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > kBarrierCycles) {
        atomicCAS(status, 0, 100 + r);
        break;
      }
    }
  }
  __syncthreads();
  __threadfence_system();
}

// 16-byte vector copy of n_vec uint4 from each peer's src into dst blocks.
__global__ void symm_all_gather_kernel(const __grid_constant__ PeerPtrs src, uint4* __restrict__ dst, long long n_vec, int world,
                                       int rank) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int i = 0; i < world; ++i) {
    const int r = (rank + i) % world;   // start with the local shard, then stagger peers
    const uint4* s = reinterpret_cast<const uint4*>(src.p[r]);
    uint4* d = dst + (long long)r * n_vec;
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < n_vec; k += stride) d[k] = s[k];
  }
}

// out[i] = scale * sum_r src_r[offset + i]; bf16 inputs, fp32 accumulate, bf16 and/or fp32 outputs.
__global__ void symm_reduce_scatter_bf16_kernel(const __grid_constant__ PeerPtrs src, long long offset, __nv_bfloat16* __restrict__ out16,
                                                float* __restrict__ out32, long long n_vec8, int world,
                                                int rank, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < n_vec8; k += stride) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int i = 0; i < world; ++i) {
      const int r = (rank + i) % world;
      const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + offset;
      float f[8];
      unpack8(ld8(s + k * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= scale;
    if (out16 != nullptr) st8(out16 + k * 8, pack8(acc));
    if (out32 != nullptr) {
      *reinterpret_cast<float4*>(out32 + k * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(out32 + k * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

__global__ void symm_reduce_scatter_f32_kernel(const __grid_constant__ PeerPtrs src, long long offset, float* __restrict__ out,
                                               long long n_vec4, int world, int rank, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < n_vec4; k += stride) {
    float4 acc = make_float4(0, 0, 0, 0);
    for (int i = 0; i < world; ++i) {
      const int r = (rank + i) % world;
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src.p[r]) + offset)[k];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(out)[k] = acc;
  }
}

// One entry of a reshard plan: copy `rows` rows of `row_bytes` bytes (multiple of 16) from
// peer `src_rank` at byte offset src_off (row pitch src_pitch) to local byte offset dst_off
// (row pitch dst_pitch).
struct CopyDesc {
  long long src_off, dst_off, src_pitch, dst_pitch;
  int src_rank, rows, row_bytes, pad;
};

__global__ void symm_copy_plan_kernel(const __grid_constant__ PeerPtrs src, unsigned char* __restrict__ dst,
                                      const CopyDesc* __restrict__ plan, int n_desc) {
  // blockIdx.y walks descriptors, blockIdx.x / threads walk the 16-byte vectors of one descriptor
  for (int d = blockIdx.y; d < n_desc; d += gridDim.y) {
    const CopyDesc c = plan[d];
    const unsigned char* s = reinterpret_cast<const unsigned char*>(src.p[c.src_rank]) + c.src_off;
    unsigned char* o = dst + c.dst_off;
    const int vec_per_row = c.row_bytes >> 4;
    const long long total = (long long)c.rows * vec_per_row;
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < total;
         k += (long long)gridDim.x * blockDim.x) {
      const long long row = k / vec_per_row;
      const int v = (int)(k % vec_per_row);
      *reinterpret_cast<uint4*>(o + row * c.dst_pitch + (long long)v * 16) =
          *reinterpret_cast<const uint4*>(s + row * c.src_pitch + (long long)v * 16);
    }
  }
}

// ---- all-reduce of small activations (rollout decode under tensor parallelism) -------------------
// Every rank owns a region [flags | slots] in its arena.  flags: 2 parities x kMaxRanks u32; slots:
// 2 parities x world x slot_bytes.  A call with sequence number q (kept in device memory, so that a
// CUDA graph can replay the launch unchanged) uses parity q & 1:
//   1. push: every CTA stores its part of x into slot [parity][me] of EVERY peer (posted remote
//      stores: one NVLink crossing, no round trip); the last CTA to finish releases
//      flags[parity][me] = q + 1 on every peer;
//   2. wait (bounded) until flags[parity][p] == q + 1 for every peer p in this rank's own region;
//   3. out = sum over ranks in rank order (own x at its own position), fp32 accumulation: every rank
//      adds the same numbers in the same order and gets bit-identical results;
//   4. the last CTA to leave re-arms the local counters and advances q.
// Parity double-buffering is enough: a rank can start call q + 2 (same parity as q) only after every
// peer has pushed for q + 1, which a peer does after it has finished reading its slots of call q.
struct ArState {
  unsigned int seq, pushed, left, pad;
};
constexpr int kArFlagBytes = 2 * kMaxRanks * 4;      // 128 B, padded to 256 by the host
constexpr int kArHeader = 256;

__global__ void symm_allreduce_push_kernel(const __grid_constant__ PeerPtrs region, int rank, int world,
                                           const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                           long long n_vec8, long long slot_bytes, ArState* state, int* status) {
  __shared__ unsigned int s_seq;
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_seq = *reinterpret_cast<volatile unsigned int*>(&state->seq);
  __syncthreads();
  const unsigned int q = s_seq, parity = q & 1u;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // 1. push my values into my slot on every peer
  for (int i = 1; i < world; ++i) {
    const int p = (rank + i) % world;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(region.p[p]) + kArHeader +
                                                          ((long long)parity * world + rank) * slot_bytes);
    for (long long k = first; k < n_vec8; k += stride) st8(dst + k * 8, ld8(x + k * 8));
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&state->pushed, 1u) == gridDim.x - 1) {
      for (int i = 1; i < world; ++i) {
        const int p = (rank + i) % world;
        st_release_sys(reinterpret_cast<unsigned int*>(region.p[p]) + parity * kMaxRanks + rank, q + 1);
      }
    }
    // 2. wait for every peer's push of this call
    int ok = 1;
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(region.p[rank]) + parity * kMaxRanks;
    const long long t0 = clock64();
    for (int i = 1; i < world && ok; ++i) {
      const int p = (rank + i) % world;
      while (ld_acquire_sys(mine + p) != q + 1) {
        if (clock64() - t0 > kBarrierCycles) {
          atomicCAS(status, 0, 200 + p);
          ok = 0;
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  // 3. reduce in rank order
  if (s_ok) {
    const unsigned char* slots = reinterpret_cast<const unsigned char*>(region.p[rank]) + kArHeader +
                                 (long long)parity * world * slot_bytes;
    for (long long k = first; k < n_vec8; k += stride) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < world; ++r) {
        const __nv_bfloat16* src = (r == rank) ? x : reinterpret_cast<const __nv_bfloat16*>(slots + r * slot_bytes);
        float f[8];
        unpack8(ld8(src + k * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
      st8(out + k * 8, pack8(acc));
    }
  }
  // 4. last CTA out re-arms the counters and advances the sequence number
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(&state->left, 1u) == gridDim.x - 1) {
    state->pushed = 0;
    state->left = 0;
    __threadfence();
    *reinterpret_cast<volatile unsigned int*>(&state->seq) = q + 1;
  }
}

}  // namespace msrl

using namespace msrl;

static PeerPtrs to_peers(void* const* ptrs, int world) {
  PeerPtrs p{};
  for (int i = 0; i < world && i < kMaxRanks; ++i) p.p[i] = ptrs[i];
  return p;
}

// ---- arena management (host) -------------------------------------------------------------------
MSRL_API int msrl_symm_alloc(long long bytes, void** ptr_out, unsigned char* handle64_out) {
  void* p = nullptr;
  // a failure here is an ordinary outcome (the caller falls back to collectives): leave no
  // allocation and no pending error behind
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return (int)e;
  }
  e = cudaMemset(p, 0, (size_t)bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    cudaGetLastError();
    return (int)e;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle64_out, &h, 64);
  *ptr_out = p;
  return 0;
}

MSRL_API int msrl_symm_open(const unsigned char* handle64, void** ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return (int)cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
}

MSRL_API int msrl_symm_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
MSRL_API int msrl_symm_free(void* ptr) { return (int)cudaFree(ptr); }
MSRL_API int msrl_symm_max_ranks() { return kMaxRanks; }

// ---- collectives ----------------------------------------------------------------------------------
MSRL_API int msrl_symm_barrier(void* const* flag_ptrs, int rank, int world, const unsigned int* epochs,
                               unsigned int mask, int* status, cudaStream_t st) {
  if (world > kMaxRanks) return (int)cudaErrorInvalidValue;
  Epochs e{};
  for (int i = 0; i < world; ++i) e.e[i] = epochs[i];
  symm_barrier_kernel<<<1, 32, 0, st>>>(to_peers(flag_ptrs, world), rank, world, e, mask, status);
  MSRL_LAUNCH_CHECK();
}

static inline unsigned copy_grid(long long n_vec) {
  long long b = ceil_div(n_vec, 256);
  long long cap = (long long)sm_count() * 4;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

MSRL_API int msrl_symm_all_gather(void* const* src_ptrs, void* dst, long long shard_bytes, int rank, int world,
                                  cudaStream_t st) {
  if (shard_bytes % 16 != 0 || world > kMaxRanks) return (int)cudaErrorInvalidValue;
  if (shard_bytes == 0) return 0;
  symm_all_gather_kernel<<<copy_grid(shard_bytes / 16), 256, 0, st>>>(to_peers(src_ptrs, world), (uint4*)dst,
                                                                     shard_bytes / 16, world, rank);
  MSRL_LAUNCH_CHECK();
}

// src_ptrs[r]: rank r's full gradient buffer; element_offset: first element of my shard.
MSRL_API int msrl_symm_reduce_scatter(void* const* src_ptrs, long long element_offset, void* out_bf16,
                                      float* out_f32, long long n, int is_bf16, int rank, int world, float scale,
                                      cudaStream_t st) {
  if (world > kMaxRanks || n % 8 != 0 || element_offset % 8 != 0) return (int)cudaErrorInvalidValue;
  if (n == 0) return 0;
  if (is_bf16)
    symm_reduce_scatter_bf16_kernel<<<copy_grid(n / 8), 256, 0, st>>>(
        to_peers(src_ptrs, world), element_offset, (__nv_bfloat16*)out_bf16, out_f32, n / 8, world, rank, scale);
  else
    symm_reduce_scatter_f32_kernel<<<copy_grid(n / 4), 256, 0, st>>>(to_peers(src_ptrs, world), element_offset,
                                                                    out_f32, n / 4, world, rank, scale);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_symm_allreduce_header_bytes() { return kArHeader; }
MSRL_API int msrl_symm_allreduce_state_bytes() { return (int)sizeof(ArState); }

// out = sum over the team of x (bf16, n elements, multiple of 8; x and out may alias).  region_ptrs[r]:
// rank r's all-reduce region (header + 2 x world x slot_bytes, zero-initialised once); state: this
// rank's ArState in ordinary device memory (zero-initialised once).  All ranks must issue the same
// sequence of calls on this region.  The launch reads its sequence number from `state`, so a CUDA
// graph may replay it.
MSRL_API int msrl_symm_allreduce_push(void* const* region_ptrs, int rank, int world, const void* x, void* out,
                                      long long n, long long slot_bytes, void* state, int* status, cudaStream_t st) {
  if (world > kMaxRanks || n % 8 != 0 || n * 2 > slot_bytes || slot_bytes % 16 != 0) return (int)cudaErrorInvalidValue;
  if (n == 0) return 0;
  // every CTA spins on the peers' flags: the grid must be resident at once
  long long blocks = ceil_div(n / 8, 256 * 4);
  const long long cap = sm_count();
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  symm_allreduce_push_kernel<<<(unsigned)blocks, 256, 0, st>>>(to_peers(region_ptrs, world), rank, world,
                                                              (const __nv_bfloat16*)x, (__nv_bfloat16*)out, n / 8,
                                                              slot_bytes, (ArState*)state, status);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_copy_desc_bytes() { return (int)sizeof(CopyDesc); }

// plan: device array of CopyDesc (n_desc entries); dst: local destination base.
MSRL_API int msrl_symm_copy_plan(void* const* src_ptrs, void* dst, const void* plan, int n_desc, int world,
                                 cudaStream_t st) {
  if (world > kMaxRanks) return (int)cudaErrorInvalidValue;
  if (n_desc == 0) return 0;
  dim3 grid(8, n_desc < 4096 ? n_desc : 4096);
  symm_copy_plan_kernel<<<grid, 256, 0, st>>>(to_peers(src_ptrs, world), (unsigned char*)dst,
                                              (const CopyDesc*)plan, n_desc);
  MSRL_LAUNCH_CHECK();
}
