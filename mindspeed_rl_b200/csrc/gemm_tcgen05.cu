// Blackwell tensor-core GEMM  C[M,N] = A[M,K] * B[N,K]^T  (bf16 in, fp32 accumulate in TMEM).
//
// * operands are staged by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into a
//   4-stage shared-memory ring guarded by full/empty mbarriers;
// * one elected thread issues tcgen05.mma (cta_group::1, 128x256x16) on UMMA shared-memory
//   descriptors; tcgen05.commit releases ring slots and finally signals the epilogue;
// * four epilogue warps read the 128x256 fp32 accumulator out of TMEM with tcgen05.ld and apply
//   a fused epilogue:
//     - STORE: convert to bf16 and store C;
//     - LOGPROB_STATS: LM-head fused with the log-softmax statistics -- every row's running
//       (max, sum-exp, target logit, sum e^z z) over this tile's 256 vocabulary columns is
//       written as one 16-byte record; the logits themselves never reach global memory.
//
// Every wait on an mbarrier is bounded (wall-clock limit); on expiry the kernel records an error
// code, skips the remaining work, still frees its TMEM allocation and returns, so the host sees
// a status instead of a hung device.
//
// Warp roles (192 threads): warps 0-3 epilogue (TMEM lane quarter = warp id), warp 4 TMA
// producer, warp 5 TMEM allocation + MMA issue.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace msrl {

constexpr int G_BM = 128, G_BN = 256, G_BK = 64, G_STAGES = 4;
constexpr uint32_t G_SMEM_A = G_BM * G_BK * 2;   // 16 KiB
constexpr uint32_t G_SMEM_B = G_BN * G_BK * 2;   // 32 KiB
constexpr uint32_t G_STAGE_BYTES = G_SMEM_A + G_SMEM_B;
constexpr uint32_t G_TMEM_COLS = 512;           // two 128x256 fp32 accumulators
constexpr long long G_WAIT_CYCLES = 4000000000LL;  // ~2 s at 2 GHz

enum GemmError { GEMM_OK = 0, GEMM_TIMEOUT_FULL = 1, GEMM_TIMEOUT_EMPTY = 2, GEMM_TIMEOUT_ACC = 3 };

struct RowStat4 {
  float m, s, zy, spz;
};

// ---- mbarrier / TMA / tcgen05 wrappers ----------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the limit expired or another role already reported an error.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 255u) == 0) {
      if (*reinterpret_cast<volatile int*>(err) != 0) return false;
      if (clock64() - t0 > G_WAIT_CYCLES) {
        atomicCAS(err, 0, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar))
               : "memory");
}
// K-major operand tile, 128-byte swizzle: rows are 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for SW128 K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                              // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                              // layout type: SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

constexpr uint32_t make_idesc_bf16(int m, int n) {
  return (1u << 4)                      // accumulator format: F32
         | (1u << 7)                    // A format: BF16
         | (1u << 10)                   // B format: BF16
         | ((uint32_t)(n >> 3) << 17)   // N / 8
         | ((uint32_t)(m >> 4) << 24);  // M / 16
}

enum Epilogue { EPI_STORE = 0, EPI_LOGPROB_STATS = 1 };

struct GemmParams {
  int M, N, K;
  // EPI_STORE
  __nv_bfloat16* C;
  long long ldc;
  // EPI_LOGPROB_STATS
  const long long* labels;  // [M] global vocabulary ids
  int vocab_offset;         // first vocabulary id of column 0
  float inv_temp;
  RowStat4* stats;          // [num_n_tiles, M]
  int* error;               // device status word (0 = ok)
};

template <int EPI>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
  // Persistent: each CTA walks tiles blockIdx.x, +gridDim.x, ... (M-tiles fastest so that CTAs
  // running together share B tiles through L2).  The TMEM allocation holds two 128x256 fp32
  // accumulators; the epilogue of tile i overlaps the main loop of tile i+1.
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t full_bar[G_STAGES], empty_bar[G_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + G_BM - 1) / G_BM, n_tiles = (p.N + G_BN - 1) / G_BN;
  const int total_tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + G_BK - 1) / G_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);   // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_u32(&tmem_base_slot)),
                 "r"(G_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;  // k-blocks issued so far (ring position)
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * G_BM, n0 = (tile / m_tiles) * G_BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % G_STAGES;
          const uint32_t use = it / G_STAGES;
          if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, p.error, GEMM_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], G_STAGE_BYTES);
          unsigned char* sa = smem + (size_t)s * G_STAGE_BYTES;
          tma_load_2d(sa, &map_a, &full_bar[s], kb * G_BK, m0);
          tma_load_2d(sa + G_SMEM_A, &map_b, &full_bar[s], kb * G_BK, n0);
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(G_BM, G_BN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        const uint32_t buf = local & 1;
        if (local >= 2) {  // the epilogue must have drained this accumulator
          ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, p.error, GEMM_TIMEOUT_ACC);
          if (!ok) break;
          tcgen05_fence_after();
        }
        const uint32_t tmem_acc = tmem_base + buf * G_BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % G_STAGES;
          ok = mbar_wait(&full_bar[s], (it / G_STAGES) & 1, p.error, GEMM_TIMEOUT_FULL);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * G_STAGE_BYTES);
          const uint32_t b_addr = a_addr + G_SMEM_A;
#pragma unroll
          for (int k = 0; k < G_BK / 16; ++k) {
            umma_bf16(tmem_acc, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(&empty_bar[s]);  // slot reusable once these MMAs have read it
        }
        tcgen05_commit(&acc_full[buf]);   // accumulator complete (or abandoned)
      }
    }
  } else {
    // ---------------- epilogue: warp w owns TMEM lanes / rows 32w .. 32w+31 ----------------
    uint32_t local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const uint32_t buf = local & 1;
      const int m0 = (tile % m_tiles) * G_BM, n0 = (tile / m_tiles) * G_BN;
      ok = mbar_wait(&acc_full[buf], (local >> 1) & 1, p.error, GEMM_TIMEOUT_ACC) &&
           (*reinterpret_cast<volatile int*>(p.error) == 0);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = m0 + warp * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * G_BN;
      if (EPI == EPI_STORE) {
#pragma unroll 1
        for (int c = 0; c < G_BN / 32; ++c) {
          float v[32];
          tmem_ld32(t_row + c * 32, v);
          const int col = n0 + c * 32;
          if (row < p.M && col < p.N) {
            __nv_bfloat16* dst = p.C + (long long)row * p.ldc + col;
            if (col + 32 <= p.N && (p.ldc % 8 == 0)) {
#pragma unroll
              for (int q = 0; q < 4; ++q) st8(dst + q * 8, pack8(v + q * 8));
            } else {
              for (int j = 0; j < 32 && col + j < p.N; ++j) dst[j] = __float2bfloat16(v[j]);
            }
          }
        }
      } else {
        float mx = -INFINITY, s = 0.f, spz = 0.f, zy = 0.f;
        const long long label = (row < p.M) ? p.labels[row] - p.vocab_offset : -1;
#pragma unroll 1
        for (int c = 0; c < G_BN / 32; ++c) {
          float v[32];
          tmem_ld32(t_row + c * 32, v);
          const int col = n0 + c * 32;
          float cm = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            // logits take the bf16 rounding the un-fused path would apply before the softmax
            v[j] = (col + j < p.N) ? __bfloat162float(__float2bfloat16(v[j])) * p.inv_temp : -INFINITY;
            cm = fmaxf(cm, v[j]);
          }
          if (cm > mx) {
            const float corr = __expf(mx - cm);
            s *= corr;
            spz *= corr;
            mx = cm;
          }
          if (mx > -INFINITY) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col + j < p.N) {
                const float e = __expf(v[j] - mx);
                s += e;
                spz += e * v[j];
              }
            }
          }
          if (label >= col && label < col + 32 && label < p.N) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (label == col + j) zy = v[j];
          }
        }
        if (row < p.M) {
          RowStat4 o{mx, s, zy, spz};
          p.stats[(long long)(tile / m_tiles) * p.M + row] = o;
        }
      }
      // hand the accumulator back to the MMA warp
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(G_TMEM_COLS));
  }
}

// ---- host side ----------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
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

// Row-major [rows, K] bf16 matrix with leading dimension `ld` (elements); box = 64 x box_rows.
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld,
                     int box_rows) {
  auto fn = get_encode_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * 2)};
  cuuint32_t box[2] = {(cuuint32_t)G_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int EPI>
static int launch_gemm(const void* A, long long lda, const void* B, long long ldb, const GemmParams& p,
                       cudaStream_t st) {
  CUtensorMap ma, mb;
  if (!make_map(&ma, A, p.M, p.K, lda, G_BM) || !make_map(&mb, B, p.N, p.K, ldb, G_BN))
    return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)G_STAGES * G_STAGE_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int tiles = ((p.M + G_BM - 1) / G_BM) * ((p.N + G_BN - 1) / G_BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_tcgen05_kernel<EPI><<<grid, 192, smem, st>>>(ma, mb, p);
  return (int)cudaGetLastError();
}

}  // namespace msrl

using namespace msrl;

// C[M,N] (bf16, leading dim ldc) = A[M,K] * B[N,K]^T.  `error` is a device int the kernel sets to a
// non-zero code when one of its bounded waits expired (the result is then invalid).
MSRL_API int msrl_gemm_bf16_tn(const void* A, long long lda, const void* B, long long ldb, void* C,
                               long long ldc, int M, int N, int K, int* error, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  if (K % 8 != 0) return (int)cudaErrorInvalidValue;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = (__nv_bfloat16*)C;
  p.ldc = ldc;
  p.error = error;
  return launch_gemm<EPI_STORE>(A, lda, B, ldb, p, st);
}

MSRL_API int msrl_lmhead_stats_tiles(int N) { return (N + G_BN - 1) / G_BN; }

// LM head fused with the log-softmax statistics: stats[tile_n, M] records over 256-column tiles
// of z = (H W^T) * inv_temp; combine them with msrl_logprob_finish(nshard = tiles * shards).
MSRL_API int msrl_lmhead_stats(const void* H, long long ldh, const void* W, long long ldw,
                               const long long* labels, int vocab_offset, float inv_temp, void* stats,
                               int M, int N, int K, int* error, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  if (K % 8 != 0) return (int)cudaErrorInvalidValue;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.labels = labels;
  p.vocab_offset = vocab_offset;
  p.inv_temp = inv_temp;
  p.stats = (RowStat4*)stats;
  p.error = error;
  return launch_gemm<EPI_LOGPROB_STATS>(H, ldh, W, ldw, p, st);
}
