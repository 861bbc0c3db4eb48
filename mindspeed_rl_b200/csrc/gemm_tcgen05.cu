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
//
// Two communication-fused variants add four "comm" warps (320 threads) that move data over
// NVLink through peer-mapped memory while the tensor cores work:
//   * COMM_AG  (all-gather -> GEMM, sequence-parallel column linear): A's row blocks live on the
//     peers.  The comm warps of all CTAs pull them piecewise into a local gathered buffer (every
//     remote byte crosses NVLink once) and count pieces per 128-row tile; the TMA producer waits
//     for a tile's count before loading it.  Tiles are visited own block first, then the peers
//     in ring order, the same order the pieces are copied in.
//   * COMM_RS  (GEMM -> reduce-scatter, row linear): the epilogue pushes each bf16 partial tile
//     straight into the staging area of the rank that owns those rows (remote stores) and bumps
//     that rank's per-row-tile counter with a release at system scope; the comm warps wait for
//     a row tile's counter to reach (ranks x column tiles x 4 warps) and sum the staged partials
//     in fp32 into the output shard.  Row tiles are visited in lock-step over the destination
//     ranks, so reduction of row tile i overlaps the main loop of row tile i+1.
// All cross-CTA and cross-GPU waits are bounded like the mbarrier waits.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace msrl {

constexpr int G_BM = 128, G_BN = 256, G_BK = 64, G_STAGES = 4;
constexpr uint32_t G_SMEM_A = G_BM * G_BK * 2;   // 16 KiB
constexpr uint32_t G_SMEM_B = G_BN * G_BK * 2;   // 32 KiB
constexpr uint32_t G_STAGE_BYTES = G_SMEM_A + G_SMEM_B;
constexpr uint32_t G_TMEM_COLS = 512;           // two 128x256 fp32 accumulators
constexpr int G_EPI_PITCH = 144;                // bytes per row of an epilogue warp's 32x64 bf16 patch
constexpr uint32_t G_EPI_BYTES = 4 * 32 * G_EPI_PITCH;
constexpr long long G_WAIT_CYCLES = 4000000000LL;  // ~2 s at 2 GHz

enum GemmError {
  GEMM_OK = 0, GEMM_TIMEOUT_FULL = 1, GEMM_TIMEOUT_EMPTY = 2, GEMM_TIMEOUT_ACC = 3,
  GEMM_TIMEOUT_GATHER = 4,   // a gathered A tile never became ready
  GEMM_TIMEOUT_PEERS = 5     // partial tiles from a peer never arrived
};
enum CommMode { COMM_NONE = 0, COMM_AG = 1, COMM_RS = 2 };
constexpr int G_MAX_RANKS = 16;
constexpr int G_COMM_THREADS = 128;
constexpr int G_AG_PIECES = 16;      // a 128-row tile is copied as 16 pieces of 8 rows
constexpr int G_RS_CHUNKS = 16;      // a row tile is reduced as 16 column chunks (spreads the tail over CTAs)

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
// One lane of a fully active, converged warp (lets the compiler keep the issue loop's state in
// uniform registers, unlike a `lane == 0` test).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
  return pred != 0;
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
  // communication-fused variants
  int rank, world;
  int m_local;              // rows owned by one rank (multiple of 128); M = world * m_local
  void* peer[G_MAX_RANKS];  // AG: every rank's A shard [m_local, K]; RS: every rank's staging area
                            //     [world, m_local, N] bf16 (slot s holds rank s's partials)
  unsigned int* peer_flag[G_MAX_RANKS];  // RS: every rank's per-row-tile arrival counters
  long long ld_peer;        // AG: leading dimension of the peers' A shards (elements)
  __nv_bfloat16* gathered;  // AG: local [M, K] buffer the shards are pulled into (ld = K)
  unsigned int* tile_ready; // AG: local per-row-tile piece counters (zeroed before launch)
  unsigned int rs_target;   // RS: counter value that means "all partials of this call arrived"
  unsigned int* rs_done;    // RS: local per-row-tile count of reducer units that passed their wait
  __nv_bfloat16* rs_out;    // RS: [m_local, N] reduced output shard
  long long ld_out;
};

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
// Bounded spin until *p >= target (wrap-around compare). `sys` selects system scope.
template <bool SYS>
__device__ __forceinline__ bool wait_counter(const unsigned int* p, unsigned int target, int* err, int code) {
  const long long t0 = clock64();
  uint32_t polls = 0;
  while ((int)((SYS ? ld_acquire_sys_u32(p) : ld_acquire_gpu_u32(p)) - target) < 0) {
    if ((++polls & 63u) == 0) {
      if (*reinterpret_cast<volatile int*>(err) != 0) return false;
      if (clock64() - t0 > G_WAIT_CYCLES) {
        atomicCAS(err, 0, code);
        return false;
      }
    }
  }
  return true;
}

// Tile order of the three variants: linear index -> (row tile, column tile).
template <int COMM>
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int rank, int world, int mt_local,
                                            int& mt, int& nt) {
  if (COMM == COMM_AG) {
    // own block first, then peers in ring order; inside a block row tiles ascend, column tiles fastest
    const int per_block = mt_local * n_tiles;
    const int pos = tile / per_block, rem = tile % per_block;
    mt = ((rank + pos) % world) * mt_local + rem / n_tiles;
    nt = rem % n_tiles;
  } else if (COMM == COMM_RS) {
    // local row-tile index slowest, destination rank fastest (starting with the next rank)
    const int per_row = n_tiles * world;
    const int i = tile / per_row, rem = tile % per_row;
    nt = rem / world;
    mt = ((rank + 1 + rem % world) % world) * mt_local + i;
  } else {
    mt = tile % m_tiles;   // row tiles fastest so that CTAs running together share B through L2
    nt = tile / m_tiles;
  }
}

template <int EPI, int COMM>
__global__ void __launch_bounds__(COMM == COMM_NONE ? 192 : 192 + G_COMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_a_local, const __grid_constant__ GemmParams p) {
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
  const int mt_local = (COMM == COMM_NONE) ? m_tiles : p.m_local / G_BM;

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
    if (elect_one()) {
      uint32_t it = 0;  // k-blocks issued so far (ring position)
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int mt, nt;
        tile_coords<COMM>(tile, m_tiles, n_tiles, p.rank, p.world, mt_local, mt, nt);
        const int m0 = mt * G_BM, n0 = nt * G_BN;
        const CUtensorMap* amap = &map_a;
        int a_row = m0;
        if (COMM == COMM_AG) {
          if (mt / mt_local == p.rank) {
            // tiles of this rank's own block read the shard where it already is: no wait
            amap = &map_a_local;
            a_row = (mt % mt_local) * G_BM;
          } else {
            // the comm warps of the grid must have landed all pieces of this row tile locally
            ok = wait_counter<false>(p.tile_ready + mt, G_AG_PIECES, p.error, GEMM_TIMEOUT_GATHER);
            if (!ok) break;
            asm volatile("fence.proxy.async;\n" ::: "memory");   // generic-proxy stores -> TMA reads
          }
        }
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % G_STAGES;
          const uint32_t use = it / G_STAGES;
          if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, p.error, GEMM_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], G_STAGE_BYTES);
          unsigned char* sa = smem + (size_t)s * G_STAGE_BYTES;
          tma_load_2d(sa, amap, &full_bar[s], kb * G_BK, a_row);
          tma_load_2d(sa + G_SMEM_A, &map_b, &full_bar[s], kb * G_BK, n0);
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
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
  } else if (warp < 4) {
    // ---------------- epilogue: warp w owns TMEM lanes / rows 32w .. 32w+31 ----------------
    uint32_t local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const uint32_t buf = local & 1;
      int mt, nt;
      tile_coords<COMM>(tile, m_tiles, n_tiles, p.rank, p.world, mt_local, mt, nt);
      const int m0 = mt * G_BM, n0 = nt * G_BN;
      // the lanes agree on the outcome: the tcgen05.ld below is a warp-wide instruction
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (local >> 1) & 1, p.error, GEMM_TIMEOUT_ACC) &&
                                       (*reinterpret_cast<volatile int*>(p.error) == 0));
      if (!ok) break;
      tcgen05_fence_after();
      const int row = m0 + warp * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * G_BN;
      if (EPI == EPI_STORE) {
        __nv_bfloat16* cbase = p.C;
        long long ldc = p.ldc, crow = row;
        if (COMM == COMM_RS) {
          // partial tile goes to slot `rank` of the staging area on the rank that owns these rows
          const int dest = mt / mt_local;
          cbase = reinterpret_cast<__nv_bfloat16*>(p.peer[dest]) + (long long)p.rank * p.m_local * p.N;
          ldc = p.N;
          crow = row - (long long)dest * p.m_local;
        }
        if (p.N % 8 == 0 && ldc % 8 == 0 && (reinterpret_cast<uintptr_t>(cbase) & 15) == 0) {
          // Coalesced path: a lane owns one accumulator row, but a global store instruction should
          // cover whole 128-byte row segments.  Each warp transposes 32 rows x 64 columns through
          // its private shared-memory patch (row pitch 144 B: conflict-free for 16-byte accesses)
          // and writes 4 rows x 128 B per instruction.
          unsigned char* patch = smem + (size_t)G_STAGES * G_STAGE_BYTES + (size_t)warp * (32 * G_EPI_PITCH);
          const long long crow0 = crow - lane;             // output row of this warp's TMEM lane 0
#pragma unroll 1
          for (int c = 0; c < G_BN / 64; ++c) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              float v[32];
              tmem_ld32(t_row + c * 64 + h * 32, v);
#pragma unroll
              for (int q = 0; q < 4; ++q)
                *reinterpret_cast<bf16x8*>(patch + lane * G_EPI_PITCH + h * 64 + q * 16) = pack8(v + q * 8);
            }
            __syncwarp();
            const int col = n0 + c * 64 + (lane & 7) * 8;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int r = it * 4 + (lane >> 3);
              if (m0 + warp * 32 + r < p.M && col < p.N)
                st8(cbase + (crow0 + r) * ldc + col,
                    *reinterpret_cast<const bf16x8*>(patch + r * G_EPI_PITCH + (lane & 7) * 16));
            }
            __syncwarp();
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < G_BN / 32; ++c) {
            float v[32];
            tmem_ld32(t_row + c * 32, v);
            const int col = n0 + c * 32;
            if (row < p.M && col < p.N) {
              __nv_bfloat16* dst = cbase + crow * ldc + col;
              for (int j = 0; j < 32 && col + j < p.N; ++j) dst[j] = __float2bfloat16(v[j]);
            }
          }
        }
        if (COMM == COMM_RS) {
          // publish: this warp's 32 rows of the tile are in place on the destination rank
          __threadfence_system();
          __syncwarp();
          if (lane == 0) red_release_sys_add(p.peer_flag[mt / mt_local] + (mt % mt_local), 1u);
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
          p.stats[(long long)nt * p.M + row] = o;
        }
      }
      // hand the accumulator back to the MMA warp
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  } else if (COMM == COMM_AG) {
    // ---------------- comm warps: pull the peers' A shards into the gathered buffer ----------------
    const int ct = threadIdx.x - 192;
    const int row_vecs = p.K / 8;                          // 16-byte vectors per row
    const int piece_vecs = (G_BM / G_AG_PIECES) * row_vecs;
    const int n_pieces = m_tiles * G_AG_PIECES;
    for (int piece = blockIdx.x; piece < n_pieces; piece += gridDim.x) {
      const int q = piece / G_AG_PIECES, sub = piece % G_AG_PIECES;
      // peers first (in the order their tiles are consumed), this rank's own shard last: nobody
      // waits for the self-copy, it only completes the gathered buffer for the weight gradient
      const int src_rank = (p.rank + 1 + q / mt_local) % p.world;
      const int mt = src_rank * mt_local + q % mt_local;
      const int r0 = (q % mt_local) * G_BM + sub * (G_BM / G_AG_PIECES);   // first row inside the shard
      const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.peer[src_rank]);
      __nv_bfloat16* dst = p.gathered + ((long long)src_rank * p.m_local + r0) * p.K;
      // batches of 8 independent 16-byte loads per thread before any store: the loads must all be
      // in flight together to cover the NVLink round trip
      for (int v0 = ct; v0 < piece_vecs; v0 += G_COMM_THREADS * 8) {
        bf16x8 buf[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int v = v0 + u * G_COMM_THREADS;
          if (v < piece_vecs) buf[u] = ld8(src + (long long)(r0 + v / row_vecs) * p.ld_peer + (v % row_vecs) * 8);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int v = v0 + u * G_COMM_THREADS;
          if (v < piece_vecs) st8(dst + (long long)(v / row_vecs) * p.K + (v % row_vecs) * 8, buf[u]);
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, %0;\n" ::"n"(G_COMM_THREADS) : "memory");
      if (ct == 0) red_release_gpu_add(p.tile_ready + mt, 1u);
    }
  } else if (COMM == COMM_RS) {
    // ---------------- comm warps: reduce the staged partial tiles of my row block ----------------
    __shared__ int comm_ok;
    const int ct = threadIdx.x - 192;
    const int chunk_cols = ((p.N / 8 + G_RS_CHUNKS - 1) / G_RS_CHUNKS) * 8;
    const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(p.peer[p.rank]);
    const long long slot = (long long)p.m_local * p.N;
    const int units = mt_local * G_RS_CHUNKS;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const int i = u / G_RS_CHUNKS, ch = u % G_RS_CHUNKS;
      if (ct == 0) {
        unsigned int* flag = p.peer_flag[p.rank] + i;
        comm_ok = wait_counter<true>(flag, p.rs_target, p.error, GEMM_TIMEOUT_PEERS) ? 1 : 0;
        // the last of the row tile's reducer units to get here re-arms the counters for the
        // call after next (the next call uses the other parity's counters)
        if (comm_ok && atomicAdd(p.rs_done + i, 1u) == G_RS_CHUNKS - 1) {
          p.rs_done[i] = 0;
          *reinterpret_cast<volatile unsigned int*>(flag) = 0;
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(G_COMM_THREADS) : "memory");
      const int good = comm_ok;
      asm volatile("bar.sync 1, %0;\n" ::"n"(G_COMM_THREADS) : "memory");
      if (!good) break;
      const int c0 = ch * chunk_cols;
      const int c1 = (c0 + chunk_cols < p.N) ? c0 + chunk_cols : p.N;
      const int vecs = (c1 - c0) / 8;
      const int total = G_BM * vecs;
      for (int v0 = ct; v0 < total; v0 += G_COMM_THREADS * 4) {
        // four independent 16-byte vectors per thread keep enough loads in flight
        float acc[4][8];
        long long off[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * G_COMM_THREADS;
          const int vv = v < total ? v : v0;
          off[u] = (long long)(i * G_BM + vv / vecs) * p.N + c0 + (vv % vecs) * 8;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
        }
        for (int s = 0; s < p.world; ++s) {
          bf16x8 raw[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) raw[u] = ld8(stage + s * slot + off[u]);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float f[8];
            unpack8(raw[u], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[u][j] += f[j];
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * G_COMM_THREADS;
          if (v < total) {
            const int rr = i * G_BM + v / vecs, cc = c0 + (v % vecs) * 8;
            st8(p.rs_out + (long long)rr * p.ld_out + cc, pack8(acc[u]));
          }
        }
      }
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

template <int EPI, int COMM = COMM_NONE>
static int launch_gemm(const void* A, long long lda, const void* B, long long ldb, const GemmParams& p,
                       cudaStream_t st, const void* A_local = nullptr, long long lda_local = 0) {
  CUtensorMap ma, mb, ml;
  if (!make_map(&ma, A, p.M, p.K, lda, G_BM) || !make_map(&mb, B, p.N, p.K, ldb, G_BN))
    return (int)cudaErrorInvalidValue;
  ml = ma;
  if (A_local != nullptr && !make_map(&ml, A_local, p.m_local, p.K, lda_local, G_BM))
    return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)G_STAGES * G_STAGE_BYTES + G_EPI_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI, COMM>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int tiles = ((p.M + G_BM - 1) / G_BM) * ((p.N + G_BN - 1) / G_BN);
  // The fused variants always launch one CTA per SM: their comm warps share the copy / reduce
  // work of the whole grid, and every CTA must be resident for the counters to advance.
  const int grid = (COMM != COMM_NONE || tiles >= sm_count()) ? sm_count() : tiles;
  const int threads = COMM == COMM_NONE ? 192 : 192 + G_COMM_THREADS;
  gemm_tcgen05_kernel<EPI, COMM><<<grid, threads, smem, st>>>(ma, mb, ml, p);
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

// ---- communication-fused GEMMs over peer-mapped memory ------------------------------------------
// C[world*m_local, N] = gather_r(A_r)[world*m_local, K] * B[N,K]^T where A_r is rank r's shard
// (peer_a[r], leading dimension ld_peer).  `gathered` ([world*m_local, K], local) receives the
// gathered A as a by-product; `tile_ready` holds world*m_local/128 counters and is zeroed here.
// The peers' shards must be complete before the launch (device barrier on the stream) and stay
// unchanged until every rank's kernel has finished.
MSRL_API int msrl_ag_gemm_bf16_tn(void* const* peer_a, long long ld_peer, void* gathered, const void* B,
                                  long long ldb, void* C, long long ldc, int m_local, int N, int K, int rank,
                                  int world, unsigned int* tile_ready, int* error, cudaStream_t st) {
  if (m_local == 0 || N == 0) return 0;
  if (K % 8 != 0 || m_local % G_BM != 0 || world > G_MAX_RANKS || ld_peer % 8 != 0)
    return (int)cudaErrorInvalidValue;
  GemmParams p{};
  p.M = m_local * world; p.N = N; p.K = K;
  p.C = (__nv_bfloat16*)C;
  p.ldc = ldc;
  p.error = error;
  p.rank = rank; p.world = world; p.m_local = m_local;
  for (int r = 0; r < world; ++r) p.peer[r] = peer_a[r];
  p.ld_peer = ld_peer;
  p.gathered = (__nv_bfloat16*)gathered;
  p.tile_ready = tile_ready;
  cudaError_t e = cudaMemsetAsync(tile_ready, 0, sizeof(unsigned int) * (size_t)(p.M / G_BM), st);
  if (e != cudaSuccess) return (int)e;
  return launch_gemm<EPI_STORE, COMM_AG>(gathered, K, B, ldb, p, st, peer_a[rank], ld_peer);
}

MSRL_API int msrl_gemm_rs_tiles(int N) { return (N + G_BN - 1) / G_BN; }

// out[m_local, N] (this rank's row block) = sum over ranks of (A_r[world*m_local, K] * B_r[N,K]^T).
// peer_stage[r]: rank r's staging area [world, m_local, N] bf16; peer_flag[r]: rank r's m_local/128
// arrival counters, `target` = world x msrl_gemm_rs_tiles(N) x 4 arrivals per row tile; `done`:
// local m_local/128 words (zero).  The reducer re-arms counters and `done` itself, so callers
// alternate between two sets of (staging, counters, done) from call to call and never clear them.
// Every rank must launch the same call in the same order.
MSRL_API int msrl_gemm_rs_bf16_tn(const void* A, long long lda, const void* B, long long ldb,
                                  void* const* peer_stage, void* const* peer_flag, unsigned int* done,
                                  void* out, long long ld_out,
                                  int m_local, int N, int K, int rank, int world, unsigned int target,
                                  int* error, cudaStream_t st) {
  if (m_local == 0 || N == 0) return 0;
  if (K % 8 != 0 || N % 8 != 0 || m_local % G_BM != 0 || world > G_MAX_RANKS || ld_out % 8 != 0)
    return (int)cudaErrorInvalidValue;
  GemmParams p{};
  p.M = m_local * world; p.N = N; p.K = K;
  p.error = error;
  p.rank = rank; p.world = world; p.m_local = m_local;
  for (int r = 0; r < world; ++r) {
    p.peer[r] = peer_stage[r];
    p.peer_flag[r] = (unsigned int*)peer_flag[r];
  }
  p.rs_target = target;
  p.rs_done = done;
  p.rs_out = (__nv_bfloat16*)out;
  p.ld_out = ld_out;
  return launch_gemm<EPI_STORE, COMM_RS>(A, lda, B, ldb, p, st);
}
