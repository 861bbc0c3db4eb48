// Dense bf16 GEMM of the linear layers on CTA pairs:  C[M,N] (+)= op(A) * op(B)^T, fp32 accumulate.
//
// Two CTAs on the two SMs of one TPC form a cluster and run ONE tcgen05.mma.cta_group::2 per
// 256x256x16 step: each CTA stages its own 128 rows of A and its own 128 rows of B (half of what a
// single-CTA 128x256 tile has to pull from L2 for B) and holds the accumulator rows of its half in
// its own tensor memory.  Per stage a CTA moves 32 KiB, so six stages fit beside the epilogue
// patches and the tensor pipe reads only 64 bytes of shared memory per clock and SM.
//
//  * TMA (cp.async.bulk.tensor with .cta_group::2, every load from this GPU's own memory, each
//    CTA loading its own operand halves) fills a 6-stage ring; the transaction
//    bytes of both CTAs are counted on the leader CTA's "full" barrier;
//  * one thread of the leader CTA (cluster rank 0) issues the MMAs for the pair; tcgen05.commit
//    releases the ring slot in both CTAs and finally hands the accumulator to both epilogues;
//  * the accumulators are double-buffered in tensor memory (2 x 256 columns), so the epilogue of
//    tile i overlaps the main loop of tile i+1; the epilogue warps of both CTAs arrive on the
//    leader's "accumulator free" barrier (a remote arrive for the second CTA);
//  * operand forms: K-major (rows of K contiguous elements) and MN-major (the matrix stored
//    transposed, [K, rows]) for A and for B through the UMMA descriptors, so forward (x W^T), data
//    gradient (dy W) and weight gradient (dy^T x) all read the tensors where they are;
//  * epilogues: bf16 store (+ bias), or accumulate into an fp32 / bf16 C (weight gradients add
//    into the flat gradient buffer).
//
// Every wait is bounded; on expiry the status word is set, all roles drain and both CTAs still free
// their tensor memory.  Reference role: the column / row parallel linears of the training
// backend (mindspeed_rl/config_cls/megatron_config.py:365-368 selects their fused Ascend forms).
#include <cuda.h>
#include <cudaTypedefs.h>
#include <stdlib.h>

#include "tcgen05_utils.cuh"

namespace msrl {
namespace g2 {

using namespace t5;

constexpr int BM = 256, BN = 256, BK = 64;       // tile of the CTA pair
constexpr int HM = 128, HN = 128;                // rows of A / rows of B staged by one CTA
constexpr int STAGES = 6;
constexpr uint32_t SMEM_A = HM * BK * 2;          // 16 KiB
constexpr uint32_t SMEM_B = HN * BK * 2;          // 16 KiB
constexpr uint32_t STAGE_BYTES = SMEM_A + SMEM_B;
constexpr uint32_t TMEM_COLS = 512;               // two 128 x 256 fp32 accumulators per CTA
constexpr int EPI_PITCH = 144;
constexpr uint32_t EPI_BYTES = 4 * 32 * EPI_PITCH;
enum { ERR_FULL = 31, ERR_EMPTY = 32, ERR_ACC = 33 };
enum OutMode { OUT_BF16 = 0, OUT_ACC_F32 = 1, OUT_ACC_BF16 = 2 };

struct Params {
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;   // OUT_BF16 only, may be null
  int* error;
  int flags;                   // experiment switches (MSRL_G2_FLAGS): 1 fence per stage, 4 no stores, bits 4-7 ring depth
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// Tile load into this CTA's shared memory; the bytes are counted on the barrier at cluster address
// `bar_cluster_addr` (the leader CTA's).  Source: this GPU's own memory only.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
               ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
// Arrive (once the MMAs issued so far have completed) on the barrier at this shared-memory offset in
// both CTAs of the pair.
__device__ __forceinline__ void commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
constexpr uint32_t idesc_pair(bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// Tile order: panels of GROUP_M row tiles; inside a panel row tiles run fastest, then column tiles.
// The pairs working at the same time then share a few column tiles of B and at most GROUP_M row tiles
// of A (about 29 MB at K = 3584), which stay in L2 while the panel sweeps over all of B.
constexpr int GROUP_M = 16;
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_panel = GROUP_M * n_tiles;
  const int panel = tile / per_panel, rem = tile - panel * per_panel;
  const int first = panel * GROUP_M;
  const int rows = (m_tiles - first) < GROUP_M ? (m_tiles - first) : GROUP_M;
  mt = first + rem % rows;
  nt = rem / rows;
}

template <bool A_MN, bool B_MN, int OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();            // 0: leader (issues the MMAs), 1: its partner
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int RS = ((p.flags >> 4) & 15) ? ((p.flags >> 4) & 15) : STAGES;   // ring depth in use

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);      // the leader's producer arrives with the byte count of both CTAs
      mbar_init(&empty_bar[s], 1);     // one commit arrival per use
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);     // four epilogue warps in each of the two CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
  }
  fence_before();
  __syncthreads();
  cluster_sync();                       // both CTAs' barriers are initialised before anyone signals them
  fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 4) {
    // ---------------- TMA producer (one thread in each CTA) ----------------
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      const uint32_t full0 = map_to_rank(smem_u32(&full_bar[0]), 0);     // the leader's barriers
      for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, mt, nt);
        const int m0 = mt * BM + (int)rank * HM, n0 = nt * BN + (int)rank * HN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % RS;
          const uint32_t use = it / RS;
          if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, p.error, ERR_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t bar = full0 + (uint32_t)s * 8;
          unsigned char* sa = smem + (size_t)s * STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < HM / 64; ++i)       // [64 k rows x 64 m columns] blocks of 8 KiB
              tma_load_2d_pair(sa + i * 8192, &map_a, bar, m0 + i * 64, kb * BK);
          } else {
            tma_load_2d_pair(sa, &map_a, bar, kb * BK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < HN / 64; ++i)
              tma_load_2d_pair(sa + SMEM_A + i * 8192, &map_b, bar, n0 + i * 64, kb * BK);
          } else {
            tma_load_2d_pair(sa + SMEM_A, &map_b, bar, kb * BK, n0);
          }
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    // one elected lane of the converged warp runs the whole issue loop
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = idesc_pair(A_MN, B_MN);
      // descriptors of stage 0, k-step 0; a later stage / k-step only adds to the 14-bit address field
      // (shared memory ends below 256 KiB, so the sum never carries out of it)
      const uint32_t smem0 = smem_u32(smem);
      const uint64_t da0 = A_MN ? desc_sw128(smem0, 8192, 1024) : desc_sw128(smem0, 16, 1024);
      const uint64_t db0 = B_MN ? desc_sw128(smem0 + SMEM_A, 8192, 1024) : desc_sw128(smem0 + SMEM_A, 16, 1024);
      constexpr uint32_t KA = (A_MN ? 2048 : 32) >> 4, KB_ = (B_MN ? 2048 : 32) >> 4;
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters, ++local) {
        const uint32_t buf = local & 1;
        if (local >= 2) {      // both CTAs' epilogues must have drained this accumulator
          ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, p.error, ERR_ACC);
          if (!ok) break;
          fence_after();
        }
        const uint32_t tmem_acc = tmem + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % RS;
          ok = mbar_wait(&full_bar[s], (it / RS) & 1, p.error, ERR_FULL);
          if (!ok) break;
          // the operands were written by TMA and are ordered by the barrier itself; a tcgen05 fence
          // here would only hold back the MMA issue
          if (p.flags & 1) fence_after();
          const uint64_t so = (uint64_t)((uint32_t)s * (STAGE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_pair(tmem_acc, da0 + so + k * KA, db0 + so + k * KB_, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          commit_pair(&empty_bar[s]);     // the slot is free in both CTAs once these MMAs have read it
        }
        commit_pair(&acc_full[buf]);      // accumulator complete (or abandoned) for both epilogues
      }
    }
  } else {
    // ---------------- epilogue: warp w owns TMEM lanes 32w .. 32w+31 of this CTA's half ----------------
    uint32_t local = 0;
    bool ok = true;
    unsigned char* patch = smem + (size_t)STAGES * STAGE_BYTES + (size_t)warp * (32 * EPI_PITCH);
    const uint32_t acc_empty_leader0 = map_to_rank(smem_u32(&acc_empty[0]), 0);
    const uint32_t acc_empty_leader1 = map_to_rank(smem_u32(&acc_empty[1]), 0);
    for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters, ++local) {
      const uint32_t buf = local & 1;
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, mt, nt);
      const int m0 = mt * BM + (int)rank * HM, n0 = nt * BN;
      ok = mbar_wait(&acc_full[buf], (local >> 1) & 1, p.error, ERR_ACC) &&
           (*reinterpret_cast<volatile int*>(p.error) == 0);
      if (!ok) break;
      fence_after();
      const int row = m0 + warp * 32 + lane;
      const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16) + buf * BN;
      if (OUT == OUT_BF16) {
        __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C);
        const long long crow0 = m0 + warp * 32;
        const bool vec_ok = (p.N % 8 == 0) && (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          if (n0 + c * 64 >= p.N) break;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v[32];
            tmem_ld32(t_row + c * 64 + h * 32, v);
            if (p.bias != nullptr) {
              const int cb = n0 + c * 64 + h * 32;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (cb + j < p.N) v[j] += __bfloat162float(p.bias[cb + j]);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<bf16x8*>(patch + lane * EPI_PITCH + h * 64 + q * 16) = pack8(v + q * 8);
          }
          __syncwarp();
          if (p.flags & 4) {
          } else if (vec_ok) {
            // whole 128-byte row segments per store instruction: 4 rows x 8 lanes x 16 bytes
            const int col = n0 + c * 64 + (lane & 7) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + (lane >> 3);
              if (crow0 + r < p.M && col < p.N)
                st8(C + (crow0 + r) * p.ldc + col, *reinterpret_cast<const bf16x8*>(patch + r * EPI_PITCH + (lane & 7) * 16));
            }
          } else if (row < p.M) {
            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(patch + lane * EPI_PITCH);
            for (int j = 0; j < 64 && n0 + c * 64 + j < p.N; ++j) C[(long long)row * p.ldc + n0 + c * 64 + j] = src[j];
          }
          __syncwarp();
        }
      } else {
        // Accumulating epilogues (weight gradients): C += acc through the warp's shared-memory patch, so
        // that the read-modify-write of C moves whole 128-byte (fp32) / 64-byte (bf16) row segments per
        // group of lanes instead of one 16-byte piece per lane and row.  32 columns per step, fp32 staging.
        const long long crow0 = m0 + warp * 32;
        const bool f32 = (OUT == OUT_ACC_F32);
        const bool vec_ok = f32 ? ((p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)
                                : ((p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;
          float v[32];
          tmem_ld32(t_row + c * 32, v);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(patch + lane * EPI_PITCH + q * 16) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
          __syncwarp();
          if (vec_ok && col0 + 32 <= p.N) {
            if (f32) {
              float* C = reinterpret_cast<float*>(p.C);
              const int cc = (lane & 7) * 4;                    // 8 lanes x 16 B = one 128-byte row segment
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int r = i * 4 + (lane >> 3);
                if (crow0 + r < p.M) {
                  float* dst = C + (crow0 + r) * p.ldc + col0 + cc;
                  float4 o = *reinterpret_cast<const float4*>(dst);
                  const float4 a = *reinterpret_cast<const float4*>(patch + r * EPI_PITCH + cc * 4);
                  o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
                  *reinterpret_cast<float4*>(dst) = o;
                }
              }
            } else {
              __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C);
              const int cc = (lane & 3) * 8;                    // 4 lanes x 16 B = one 64-byte row segment
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int r = i * 8 + (lane >> 2);
                if (crow0 + r < p.M) {
                  __nv_bfloat16* dst = C + (crow0 + r) * p.ldc + col0 + cc;
                  float f[8];
                  unpack8(ld8(dst), f);
                  const float4 a0 = *reinterpret_cast<const float4*>(patch + r * EPI_PITCH + cc * 4);
                  const float4 a1 = *reinterpret_cast<const float4*>(patch + r * EPI_PITCH + cc * 4 + 16);
                  f[0] += a0.x; f[1] += a0.y; f[2] += a0.z; f[3] += a0.w;
                  f[4] += a1.x; f[5] += a1.y; f[6] += a1.z; f[7] += a1.w;
                  st8(dst, pack8(f));
                }
              }
            }
          } else if (row < p.M) {
            const float* src = reinterpret_cast<const float*>(patch + lane * EPI_PITCH);
            if (f32) {
              float* dst = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
              for (int jj = 0; jj < 32 && col0 + jj < p.N; ++jj) dst[jj] += src[jj];
            } else {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
              for (int jj = 0; jj < 32 && col0 + jj < p.N; ++jj) dst[jj] = __float2bfloat16(__bfloat162float(dst[jj]) + src[jj]);
            }
          }
          __syncwarp();
        }
      }
      // hand the accumulator back to the leader's MMA thread
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(buf ? acc_empty_leader1 : acc_empty_leader0);
    }
  }
  // Nobody leaves while its partner may still read its shared memory, signal its barriers or use the
  // paired tensor-memory allocation.
  fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
  }
}

// ---- host side ----------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// bf16 matrix stored as [outer, inner] with `inner` contiguous and leading dimension ld (elements).
static bool make_map(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld, int box_inner,
                     int box_outer) {
  auto fn = encode_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * 2)};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool A_MN, bool B_MN, int OUT>
static int launch(const void* A, long long lda, const void* B, long long ldb, const Params& p, cudaStream_t st) {
  CUtensorMap ma, mb;
  // K-major: [rows, K], box 64 k x 128 rows; MN-major: [K, rows], box 64 rows x 64 k
  const bool oka = A_MN ? make_map(&ma, A, p.M, p.K, lda, 64, 64) : make_map(&ma, A, p.K, p.M, lda, BK, HM);
  const bool okb = B_MN ? make_map(&mb, B, p.N, p.K, ldb, 64, 64) : make_map(&mb, B, p.K, p.N, ldb, BK, HN);
  if (!oka || !okb) return (int)cudaErrorInvalidValue;
  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT>;
  const size_t smem = (size_t)STAGES * STAGE_BYTES + EPI_BYTES + 1024;
  static int max_clusters = 0;   // per instantiation
  cudaLaunchConfig_t cfg = {};          // the pair (cluster of 2) is a compile-time attribute of the kernel
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  if (max_clusters == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cfg.gridDim = dim3(2 * (sm_count() / 2), 1, 1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = sm_count() / 2;
    max_clusters = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int clusters = tiles < max_clusters ? tiles : max_clusters;
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  return (int)cudaLaunchKernelEx(&cfg, kern, ma, mb, p);
}

}  // namespace g2
}  // namespace msrl

using namespace msrl;

// C[M,N] (+)= op(A) op(B)^T with bf16 operands and fp32 accumulation on CTA pairs.
//   a_mn = 0: A is [M, K] row-major (lda >= K);   a_mn = 1: A is stored transposed, [K, M] (lda >= M)
//   b_mn = 0: B is [N, K] row-major (ldb >= N.K); b_mn = 1: B is stored transposed, [K, N] (ldb >= N)
//   out_mode 0: C bf16 = result (+ bias[N], bf16, optional); 1: C fp32 += result; 2: C bf16 += result.
// Supported forms: (a_mn, b_mn) = (0,0) forward, (0,1) data gradient, (1,1) weight gradient.
// Leading dimensions and the contiguous extents must be multiples of 8 elements, bases 16-byte
// aligned.  `error` is a device int set non-zero when a bounded wait inside the kernel expired.
MSRL_API int msrl_gemm_pair_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                                 void* C, long long ldc, int out_mode, const void* bias, int M, int N, int K,
                                 int* error, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  if (K <= 0 || K % 8 != 0 || (a_mn && M % 8 != 0) || (b_mn && N % 8 != 0)) return (int)cudaErrorInvalidValue;
  g2::Params p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C;
  p.ldc = ldc;
  p.bias = out_mode == g2::OUT_BF16 ? reinterpret_cast<const __nv_bfloat16*>(bias) : nullptr;
  p.error = error;
  static const int flags = [] { const char* e = getenv("MSRL_G2_FLAGS"); return e ? atoi(e) : 0; }();
  p.flags = flags;
  if (!a_mn && !b_mn && out_mode == g2::OUT_BF16) return g2::launch<false, false, g2::OUT_BF16>(A, lda, B, ldb, p, st);
  if (!a_mn && b_mn && out_mode == g2::OUT_BF16) return g2::launch<false, true, g2::OUT_BF16>(A, lda, B, ldb, p, st);
  if (a_mn && b_mn && out_mode == g2::OUT_BF16) return g2::launch<true, true, g2::OUT_BF16>(A, lda, B, ldb, p, st);
  if (a_mn && b_mn && out_mode == g2::OUT_ACC_F32) return g2::launch<true, true, g2::OUT_ACC_F32>(A, lda, B, ldb, p, st);
  if (a_mn && b_mn && out_mode == g2::OUT_ACC_BF16) return g2::launch<true, true, g2::OUT_ACC_BF16>(A, lda, B, ldb, p, st);
  return (int)cudaErrorInvalidValue;
}
