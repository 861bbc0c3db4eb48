// Grouped (per-expert) GEMM for mixture-of-experts layers on the 5th-generation tensor cores.
//
//   C[r, :] = A[r, :] * B_e        for every row r of the 128-row tiles that belong to expert e
//
// A [P, K] holds the permuted tokens, grouped by expert, every group padded to a multiple of 128
// rows; `tile_expert[P / 128]` names the expert of each row tile (-1: tile not in use, skipped).
// The experts' weights stay where the model keeps them: B is ONE 2-D tensor map over the whole
// stacked weight, and expert e's operand starts at TMA coordinates (e * ex, e * ey).  Two operand
// forms cover forward and data-gradient of both expert linears without a transposed copy:
//   * B K-major  ([N rows, K contiguous]; box 64 x 256): dact = d w2[e]^T, dx = dgu w1[:, e]^T;
//   * B MN-major ([K rows, N contiguous]; four 64 x 64 boxes per stage): gu = x w1[:, e],
//     y = act w2[e].
// The pipeline is the one of gemm_tcgen05.cu: persistent CTAs, a 4-stage TMA ring, one thread
// issuing tcgen05.mma 128x256x16 into two TMEM accumulators, four epilogue warps storing bf16 rows
// as whole 128-byte segments.  Every wait is bounded and reports through the status word.
//
// Reference behaviour: the grouped expert computation of
// mindspeed_rl/models/rollout/vllm_adapter/fused_moe.py:55-373 (Ascend grouped matmul + SwiGLU).
#include <cuda.h>
#include <cudaTypedefs.h>

#include "tcgen05_utils.cuh"

namespace msrl {
namespace gg {

using namespace t5;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr uint32_t SMEM_A = BM * BK * 2;                 // 16 KiB
constexpr uint32_t SMEM_B = BN * BK * 2;                 // 32 KiB
constexpr uint32_t STAGE_BYTES = SMEM_A + SMEM_B;
constexpr uint32_t TMEM_COLS = 512;
constexpr int EPI_PITCH = 144;
constexpr uint32_t EPI_BYTES = 4 * 32 * EPI_PITCH;
enum { ERR_FULL = 21, ERR_EMPTY = 22, ERR_ACC = 23 };

struct Params {
  int n_m_tiles, N, K;
  const int* tile_expert;
  int ex, ey;                 // TMA coordinate offsets of expert e: (e * ex, e * ey)
  __nv_bfloat16* C;
  long long ldc;
  int* error;
};

template <bool B_MN>
__global__ void __launch_bounds__(192, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = p.n_m_tiles * n_tiles;
  const int num_kb = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;

  // tile order: column tiles fastest, so that the CTAs running together cover a few dozen row tiles of
  // one expert with all its weight columns: both stay in L2 and are read from DRAM once
  if (warp == 4) {
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mt = tile / n_tiles, nt = tile % n_tiles;
        const int e = p.tile_expert[mt];
        if (e < 0) continue;
        const int m0 = mt * BM, n0 = nt * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t use = it / STAGES;
          if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, p.error, ERR_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          unsigned char* sa = smem + (size_t)s * STAGE_BYTES;
          tma_load_2d(sa, &map_a, &full_bar[s], kb * BK, m0);
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)     // [64 k rows x 64 n columns] blocks, 8 KiB each
              tma_load_2d(sa + SMEM_A + i * 8192, &map_b, &full_bar[s], e * p.ex + n0 + i * 64, e * p.ey + kb * BK);
          } else {
            tma_load_2d(sa + SMEM_A, &map_b, &full_bar[s], e * p.ex + kb * BK, e * p.ey + n0);
          }
        }
      }
    }
  } else if (warp == 5) {
    if (elect_one()) {
      constexpr uint32_t idesc = idesc_bf16(BM, BN, B_MN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (p.tile_expert[tile / n_tiles] < 0) continue;
        const uint32_t buf = local & 1;
        if (local >= 2) {
          ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, p.error, ERR_ACC);
          if (!ok) break;
          fence_after();
        }
        const uint32_t tmem_acc = tmem + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, p.error, ERR_FULL);
          if (!ok) break;
          fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + SMEM_A;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t db = B_MN ? desc_sw128(b_addr + k * 2048, 8192, 1024) : desc_sw128(b_addr + k * 32, 16, 1024);
            umma(tmem_acc, desc_sw128(a_addr + k * 32, 16, 1024), db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          commit(&empty_bar[s]);
        }
        commit(&acc_full[buf]);
        ++local;
      }
    }
  } else {
    uint32_t local = 0;
    bool ok = true;
    unsigned char* patch = smem + (size_t)STAGES * STAGE_BYTES + (size_t)warp * (32 * EPI_PITCH);
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int mt = tile / n_tiles, nt = tile % n_tiles;
      if (p.tile_expert[mt] < 0) continue;
      const uint32_t buf = local & 1;
      const int m0 = mt * BM, n0 = nt * BN;
      ok = mbar_wait_warp(&acc_full[buf], (local >> 1) & 1, p.error, ERR_ACC);
      if (!ok) break;
      fence_after();
      const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16) + buf * BN;
      const long long crow0 = m0 + warp * 32;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        if (n0 + c * 64 >= p.N) break;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float v[32];
          tmem_ld32(t_row + c * 64 + h * 32, v);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<bf16x8*>(patch + lane * EPI_PITCH + h * 64 + q * 16) = pack8(v + q * 8);
        }
        __syncwarp();
        const int col = n0 + c * 64 + (lane & 7) * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + (lane >> 3);
          if (col < p.N)
            st8(p.C + (crow0 + r) * p.ldc + col, *reinterpret_cast<const bf16x8*>(patch + r * EPI_PITCH + (lane & 7) * 16));
        }
        __syncwarp();
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      ++local;
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
  }
}

}  // namespace gg
}  // namespace msrl

using namespace msrl;

static PFN_cuTensorMapEncodeTiled_v12000 gg_encode_fn() {
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

static bool gg_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                        unsigned box_cols, unsigned box_rows) {
  auto fn = gg_encode_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * 2)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A [n_m_tiles * 128, K] (lda), C [n_m_tiles * 128, N] (ldc), B: 2-D bf16 matrix [b_rows, b_cols]
// (ldb) holding all experts; expert e's operand starts at column e*ex, row e*ey.  b_mn_major = 0:
// B_e is [N, K] (K contiguous); 1: B_e is [K, N] (N contiguous).  K must be a multiple of 64, N, ex
// of 8.  `sm_count` CTAs at most.  Returns cudaErrorNotSupported for shapes outside this cover.
MSRL_API int msrl_moe_grouped_gemm(const void* A, long long lda, const void* B, long long b_rows, long long b_cols,
                                   long long ldb, int b_mn_major, int ex, int ey, void* C, long long ldc,
                                   const int* tile_expert, int n_m_tiles, int N, int K, int sm_count, int* error,
                                   cudaStream_t st) {
  if (n_m_tiles == 0 || N == 0) return 0;
  if (K % gg::BK != 0 || K == 0 || N % 8 != 0 || ex % 8 != 0 || ldc % 8 != 0 ||
      (reinterpret_cast<uintptr_t>(C) & 15) != 0)
    return (int)cudaErrorNotSupported;
  CUtensorMap ma, mb;
  if (!gg_make_map(&ma, A, (long long)n_m_tiles * gg::BM, K, lda, gg::BK, gg::BM)) return (int)cudaErrorNotSupported;
  if (!(b_mn_major ? gg_make_map(&mb, B, b_rows, b_cols, ldb, 64, 64) : gg_make_map(&mb, B, b_rows, b_cols, ldb, gg::BK, gg::BN)))
    return (int)cudaErrorNotSupported;
  gg::Params p{};
  p.n_m_tiles = n_m_tiles;
  p.N = N;
  p.K = K;
  p.tile_expert = tile_expert;
  p.ex = ex;
  p.ey = ey;
  p.C = (__nv_bfloat16*)C;
  p.ldc = ldc;
  p.error = error;
  const int smem = (int)(gg::STAGES * gg::STAGE_BYTES + gg::EPI_BYTES + 1024);
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gg::grouped_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gg::grouped_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int total = n_m_tiles * ((N + gg::BN - 1) / gg::BN);
  const int grid = total < sm_count ? total : sm_count;
  if (b_mn_major)
    gg::grouped_gemm_kernel<true><<<grid, 192, smem, st>>>(ma, mb, p);
  else
    gg::grouped_gemm_kernel<false><<<grid, 192, smem, st>>>(ma, mb, p);
  return (int)cudaGetLastError();
}
