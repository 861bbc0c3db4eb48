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
enum OutMode { OUT_BF16 = 0, OUT_ACC_F32 = 1, OUT_ACC_BF16 = 2, OUT_PART_F32 = 3 };
enum CommMode { COMM_NONE = 0, COMM_AG = 1, COMM_RS = 2 };
enum { ERR_GATHER = 34, ERR_PEERS = 35 };
constexpr int MAX_RANKS = 16;
constexpr int COMM_THREADS = 128;     // four extra warps move data over NVLink while the tensor cores work
constexpr int AG_PIECES = 16;         // a 128-row unit is gathered as 16 pieces of 8 rows
constexpr int RS_CHUNKS = 16;         // a 128-row unit is reduced as 16 column chunks

struct Params {
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;   // OUT_BF16 only, may be null
  int* error;
  // grouped reduction (expert weight gradients): `groups` independent products share the operands' M and N
  // and split their rows: group g reduces over rows [seg[g], seg[g + 1]) (device array, multiples of 64,
  // read by the kernel: no host round trip) and accumulates into C + g * c_group_stride
  int groups;
  const int* seg;
  long long c_group_stride;
  int k_splits;                // OUT_PART_F32: pieces the reduction is cut into (one work item per tile and piece;
                               // piece s writes its fp32 partial tile into slab s of C, [k_splits, M, ldc])
  // communication-fused variants (tensor-parallel linears under sequence parallelism)
  int rank, world;
  int m_local;                 // rows owned by one rank (multiple of 256); M = world * m_local
  void* peer[MAX_RANKS];       // AG: every rank's A shard [m_local, K]; RS: every rank's staging area
                               //     [world, m_local, N] bf16 (slot s holds rank s's partial sums)
  unsigned int* peer_flag[MAX_RANKS];   // RS: every rank's arrival counters, one per 128-row unit
  long long ld_peer;           // AG: leading dimension of the peers' shards
  __nv_bfloat16* gathered;     // AG: local [M, K] buffer the shards are pulled into
  unsigned int* tile_ready;    // AG: local piece counters, one per 128-row unit (zeroed before launch)
  unsigned int rs_target;      // RS: counter value that means "all partial sums of this call arrived"
  unsigned int* rs_done;       // RS: reducer units that passed their wait, per 128-row unit
  __nv_bfloat16* rs_out;       // RS: [m_local, N] reduced output
  long long ld_out;
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
// Communication-fused orders.  AG: this rank's own row block first, then the peers' blocks in ring
// order (the order their shards arrive in), column tiles fastest.  RS: row tile i of every
// destination rank in turn (starting with the next rank), so that the owners can reduce row tile i
// while row tile i + 1 is being multiplied.
__device__ __forceinline__ void tile_coords_ag(int tile, int n_tiles, int rank, int world, int mt_local, int& mt,
                                               int& nt) {
  const int per_block = mt_local * n_tiles;
  const int pos = tile / per_block, rem = tile % per_block;
  mt = ((rank + pos) % world) * mt_local + rem / n_tiles;
  nt = rem % n_tiles;
}
__device__ __forceinline__ void tile_coords_rs(int tile, int n_tiles, int rank, int world, int mt_local, int& mt,
                                               int& nt) {
  const int per_row = n_tiles * world;
  const int i = tile / per_row, rem = tile % per_row;
  nt = rem / world;
  mt = ((rank + 1 + rem % world) % world) * mt_local + i;
}
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
// Bounded spin until *p >= target (wrap-around compare); SYS: the counter is bumped by other GPUs.
template <bool SYS>
__device__ __forceinline__ bool wait_counter(const unsigned int* p, unsigned int target, int* err, int code) {
  const long long t0 = clock64();
  uint32_t polls = 0;
  while ((int)((SYS ? ld_acquire_sys_u32(p) : ld_acquire_gpu_u32(p)) - target) < 0) {
    if ((++polls & 63u) == 0) {
      if (*reinterpret_cast<volatile int*>(err) != 0) return false;
      if (clock64() - t0 > WAIT_CYCLES) {
        atomicCAS(err, 0, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_panel = GROUP_M * n_tiles;
  const int panel = tile / per_panel, rem = tile - panel * per_panel;
  const int first = panel * GROUP_M;
  const int rows = (m_tiles - first) < GROUP_M ? (m_tiles - first) : GROUP_M;
  mt = first + rem % rows;
  nt = rem / rows;
}

template <bool A_MN, bool B_MN, int OUT, int COMM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(COMM == COMM_NONE ? 192 : 192 + COMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_a_local, const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();            // 0: leader (issues the MMAs), 1: its partner
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int tiles_per_group = m_tiles * n_tiles;
  const bool grouped = (OUT == OUT_ACC_F32 || OUT == OUT_ACC_BF16) && COMM == COMM_NONE && p.groups > 0;
  const int total_tiles = tiles_per_group * ((OUT == OUT_PART_F32) ? p.k_splits : (grouped ? p.groups : 1));
  const int num_kb = (p.K + BK - 1) / BK;
  // split reduction (small-M, weight-streaming problems): work item = (tile, piece of K)
  const int k_splits = (OUT == OUT_PART_F32) ? p.k_splits : 1;
  const int kb_per = (num_kb + k_splits - 1) / k_splits;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int mt_local = (COMM == COMM_NONE) ? m_tiles : p.m_local / BM;       // row tiles of one rank's block
  const int units_local = (COMM == COMM_NONE) ? 0 : p.m_local / HM;          // 128-row units of one rank's block
  // k-block range of a work item; an empty range (an expert without tokens) is skipped by every role alike
  auto krange = [&](int tile, int& kb0, int& kb1) {
    if (OUT == OUT_PART_F32) {
      kb0 = (tile % k_splits) * kb_per;
      kb1 = (kb0 + kb_per < num_kb) ? kb0 + kb_per : num_kb;
    } else if (grouped) {
      const int g = tile / tiles_per_group;
      kb0 = p.seg[g] / BK;
      kb1 = p.seg[g + 1] / BK;
    } else {
      kb0 = 0;
      kb1 = num_kb;
    }
  };
  auto coords = [&](int tile, int& mt, int& nt) {
    if (OUT == OUT_PART_F32) tile /= k_splits;
    if (grouped) tile %= tiles_per_group;
    if (COMM == COMM_AG) tile_coords_ag(tile, n_tiles, p.rank, p.world, mt_local, mt, nt);
    else if (COMM == COMM_RS) tile_coords_rs(tile, n_tiles, p.rank, p.world, mt_local, mt, nt);
    else tile_coords(tile, m_tiles, n_tiles, mt, nt);
  };
  constexpr int RS = STAGES;   // ring depth

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
        int mt, nt, kb0, kb1;
        krange(tile, kb0, kb1);
        if (grouped && kb1 <= kb0) continue;
        coords(tile, mt, nt);
        const int m0 = mt * BM + (int)rank * HM, n0 = nt * BN + (int)rank * HN;
        const CUtensorMap* amap = &map_a;
        int a_row = m0;
        if (COMM == COMM_AG) {
          const int unit = m0 / HM;                     // 128-row unit this CTA loads
          if (unit / units_local == p.rank) {
            // rows of this rank's own block are read from the shard where it already is: no wait
            amap = &map_a_local;
            a_row = (unit % units_local) * HM;
          } else {
            // the comm warps of the grid must have landed all pieces of this unit in the gathered buffer
            ok = wait_counter<false>(p.tile_ready + unit, AG_PIECES, p.error, ERR_GATHER);
            if (!ok) break;
            asm volatile("fence.proxy.async;\n" ::: "memory");   // generic-proxy stores -> TMA reads
          }
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
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
            tma_load_2d_pair(sa, amap, bar, kb * BK, a_row);
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
      for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
        int kb0, kb1;
        krange(tile, kb0, kb1);
        if (grouped && kb1 <= kb0) continue;
        const uint32_t buf = local & 1;
        if (local >= 2) {      // both CTAs' epilogues must have drained this accumulator
          ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, p.error, ERR_ACC);
          if (!ok) break;
          fence_after();
        }
        const uint32_t tmem_acc = tmem + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % RS;
          ok = mbar_wait(&full_bar[s], (it / RS) & 1, p.error, ERR_FULL);
          if (!ok) break;
          // the operands were written by TMA and are ordered by the barrier itself; a tcgen05 fence
          // here would only hold back the MMA issue (measured)
          const uint64_t so = (uint64_t)((uint32_t)s * (STAGE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_pair(tmem_acc, da0 + so + k * KA, db0 + so + k * KB_, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          commit_pair(&empty_bar[s]);     // the slot is free in both CTAs once these MMAs have read it
        }
        commit_pair(&acc_full[buf]);      // accumulator complete (or abandoned) for both epilogues
        ++local;
      }
    }
  } else if (warp < 4) {
    // ---------------- epilogue: warp w owns TMEM lanes 32w .. 32w+31 of this CTA's half ----------------
    uint32_t local = 0;
    bool ok = true;
    unsigned char* patch = smem + (size_t)STAGES * STAGE_BYTES + (size_t)warp * (32 * EPI_PITCH);
    const uint32_t acc_empty_leader0 = map_to_rank(smem_u32(&acc_empty[0]), 0);
    const uint32_t acc_empty_leader1 = map_to_rank(smem_u32(&acc_empty[1]), 0);
    for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
      {
        int kb0, kb1;
        krange(tile, kb0, kb1);
        if (grouped && kb1 <= kb0) continue;
      }
      const uint32_t buf = local & 1;
      int mt, nt;
      coords(tile, mt, nt);
      const int m0 = mt * BM + (int)rank * HM, n0 = nt * BN;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (local >> 1) & 1, p.error, ERR_ACC) &&
                                       (*reinterpret_cast<volatile int*>(p.error) == 0));
      if (!ok) break;
      fence_after();
      const int row = m0 + warp * 32 + lane;
      const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16) + buf * BN;
      if (OUT == OUT_BF16) {
        __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C);
        long long crow0 = m0 + warp * 32, ldc = p.ldc;
        long long row_limit = p.M;
        if (COMM == COMM_RS) {
          // the partial tile goes to slot `rank` of the staging area on the rank that owns these rows
          const int dest = mt / mt_local;
          C = reinterpret_cast<__nv_bfloat16*>(p.peer[dest]) + (long long)p.rank * p.m_local * p.N;
          ldc = p.N;
          crow0 -= (long long)dest * p.m_local;
          row_limit = p.m_local;
        }
        const bool vec_ok = (p.N % 8 == 0) && (ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
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
          if (vec_ok) {
            // whole 128-byte row segments per store instruction: 4 rows x 8 lanes x 16 bytes
            const int col = n0 + c * 64 + (lane & 7) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + (lane >> 3);
              if (crow0 + r < row_limit && col < p.N)
                st8(C + (crow0 + r) * ldc + col, *reinterpret_cast<const bf16x8*>(patch + r * EPI_PITCH + (lane & 7) * 16));
            }
          } else if (crow0 + lane < row_limit) {
            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(patch + lane * EPI_PITCH);
            for (int j = 0; j < 64 && n0 + c * 64 + j < p.N; ++j) C[(crow0 + lane) * ldc + n0 + c * 64 + j] = src[j];
          }
          __syncwarp();
        }
        if (COMM == COMM_RS) {
          // publish: this warp's 32 rows of the partial tile are in place on the destination rank
          __threadfence_system();
          __syncwarp();
          if (lane == 0) {
            const int unit = (mt % mt_local) * 2 + (int)rank;
            asm volatile("red.release.sys.global.add.u32 [%0], %1;\n" ::"l"(p.peer_flag[mt / mt_local] + unit), "r"(1u)
                         : "memory");
          }
        }
      } else {
        // Accumulating epilogues (weight gradients): C += acc through the warp's shared-memory patch, so
        // that the read-modify-write of C moves whole 128-byte (fp32) / 64-byte (bf16) row segments per
        // group of lanes instead of one 16-byte piece per lane and row.  32 columns per step, fp32 staging.
        const long long crow0 = m0 + warp * 32;
        const bool f32 = (OUT == OUT_ACC_F32 || OUT == OUT_PART_F32);
        // split reduction: this piece's slab of the partial-sum buffer; an empty piece (more pieces than
        // k-blocks) was never multiplied and stores zeros
        const long long group_off = grouped ? (long long)(tile / tiles_per_group) * p.c_group_stride : 0;
        float* const Cf = reinterpret_cast<float*>(p.C) + group_off +
                          ((OUT == OUT_PART_F32) ? (long long)(tile % k_splits) * p.M * p.ldc : 0);
        const bool empty_piece = (OUT == OUT_PART_F32) && (tile % k_splits) * kb_per >= num_kb;
        const bool vec_ok = f32 ? ((p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)
                                : ((p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;
          float v[32];
          tmem_ld32(t_row + c * 32, v);
          if (empty_piece) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(patch + lane * EPI_PITCH + q * 16) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
          __syncwarp();
          if (vec_ok && col0 + 32 <= p.N) {
            if (f32) {
              float* C = Cf;
              const int cc = (lane & 7) * 4;                    // 8 lanes x 16 B = one 128-byte row segment
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int r = i * 4 + (lane >> 3);
                if (crow0 + r < p.M) {
                  float* dst = C + (crow0 + r) * p.ldc + col0 + cc;
                  const float4 a = *reinterpret_cast<const float4*>(patch + r * EPI_PITCH + cc * 4);
                  if (OUT == OUT_PART_F32) {
                    *reinterpret_cast<float4*>(dst) = a;
                  } else {
                    float4 o = *reinterpret_cast<const float4*>(dst);
                    o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
                    *reinterpret_cast<float4*>(dst) = o;
                  }
                }
              }
            } else {
              __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C) + group_off;
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
              float* dst = Cf + (long long)row * p.ldc + col0;
              for (int jj = 0; jj < 32 && col0 + jj < p.N; ++jj) dst[jj] = (OUT == OUT_PART_F32) ? src[jj] : dst[jj] + src[jj];
            } else {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + group_off + (long long)row * p.ldc + col0;
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
      ++local;
    }
  }
  if (COMM == COMM_AG && warp >= 6) {
    // ---------------- comm warps: pull the peers' A shards into the gathered buffer ----------------
    const int ct = threadIdx.x - 192;
    const int row_vecs = p.K / 8;                          // 16-byte vectors per row
    const int piece_vecs = (HM / AG_PIECES) * row_vecs;
    const int n_units = p.M / HM;
    const int n_pieces = n_units * AG_PIECES;
    for (int piece = blockIdx.x; piece < n_pieces; piece += gridDim.x) {
      const int q = piece / AG_PIECES, sub = piece % AG_PIECES;
      // peers first (in the order their tiles are consumed), this rank's own shard last: nobody waits
      // for the self-copy, it only completes the gathered buffer for the weight gradient
      const int src_rank = (p.rank + 1 + q / units_local) % p.world;
      const int unit = src_rank * units_local + q % units_local;
      const int r0 = (q % units_local) * HM + sub * (HM / AG_PIECES);       // first row inside the shard
      const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.peer[src_rank]);
      __nv_bfloat16* dst = p.gathered + ((long long)src_rank * p.m_local + r0) * p.K;
      // batches of 8 independent 16-byte loads per thread before any store: the loads must all be in
      // flight together to cover the NVLink round trip
      for (int v0 = ct; v0 < piece_vecs; v0 += COMM_THREADS * 8) {
        bf16x8 buf[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int v = v0 + u * COMM_THREADS;
          if (v < piece_vecs) buf[u] = ld8(src + (long long)(r0 + v / row_vecs) * p.ld_peer + (v % row_vecs) * 8);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int v = v0 + u * COMM_THREADS;
          if (v < piece_vecs) st8(dst + (long long)(v / row_vecs) * p.K + (v % row_vecs) * 8, buf[u]);
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, %0;\n" ::"n"(COMM_THREADS) : "memory");
      if (ct == 0) asm volatile("red.release.gpu.global.add.u32 [%0], %1;\n" ::"l"(p.tile_ready + unit), "r"(1u) : "memory");
    }
  } else if (COMM == COMM_RS && warp >= 6) {
    // ---------------- comm warps: reduce the staged partial sums of my row block ----------------
    __shared__ int comm_ok;
    const int ct = threadIdx.x - 192;
    const int chunk_cols = ((p.N / 8 + RS_CHUNKS - 1) / RS_CHUNKS) * 8;
    const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(p.peer[p.rank]);
    const long long slot = (long long)p.m_local * p.N;
    const int units = units_local * RS_CHUNKS;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const int i = u / RS_CHUNKS, ch = u % RS_CHUNKS;
      if (ct == 0) {
        unsigned int* flag = p.peer_flag[p.rank] + i;
        comm_ok = wait_counter<true>(flag, p.rs_target, p.error, ERR_PEERS) ? 1 : 0;
        // the last of the unit's reducers to get here re-arms the counters for the call after next
        // (the next call uses the other parity's counters)
        if (comm_ok && atomicAdd(p.rs_done + i, 1u) == RS_CHUNKS - 1) {
          p.rs_done[i] = 0;
          *reinterpret_cast<volatile unsigned int*>(flag) = 0;
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(COMM_THREADS) : "memory");
      const int good = comm_ok;
      asm volatile("bar.sync 1, %0;\n" ::"n"(COMM_THREADS) : "memory");
      if (!good) break;
      const int c0 = ch * chunk_cols;
      const int c1 = (c0 + chunk_cols < p.N) ? c0 + chunk_cols : p.N;
      const int vecs = (c1 - c0) / 8;
      const int total = HM * vecs;
      for (int v0 = ct; v0 < total; v0 += COMM_THREADS * 4) {
        float acc[4][8];
        long long off[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int v = v0 + x * COMM_THREADS;
          const int vv = v < total ? v : v0;
          off[x] = (long long)(i * HM + vv / vecs) * p.N + c0 + (vv % vecs) * 8;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[x][j] = 0.f;
        }
        for (int sr = 0; sr < p.world; ++sr) {
          bf16x8 raw[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) raw[x] = ld8(stage + sr * slot + off[x]);
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            float f[8];
            unpack8(raw[x], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[x][j] += f[j];
          }
        }
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int v = v0 + x * COMM_THREADS;
          if (v < total) {
            const int rr = i * HM + v / vecs, cc = c0 + (v % vecs) * 8;
            st8(p.rs_out + (long long)rr * p.ld_out + cc, pack8(acc[x]));
          }
        }
      }
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

template <bool A_MN, bool B_MN, int OUT, int COMM = COMM_NONE>
static int launch(const void* A, long long lda, const void* B, long long ldb, const Params& p, cudaStream_t st,
                  const void* A_local = nullptr, long long lda_local = 0) {
  CUtensorMap ma, mb, ml;
  // K-major: [rows, K], box 64 k x 128 rows; MN-major: [K, rows], box 64 rows x 64 k
  const bool oka = A_MN ? make_map(&ma, A, p.M, p.K, lda, 64, 64) : make_map(&ma, A, p.K, p.M, lda, BK, HM);
  const bool okb = B_MN ? make_map(&mb, B, p.N, p.K, ldb, 64, 64) : make_map(&mb, B, p.K, p.N, ldb, BK, HN);
  if (!oka || !okb) return (int)cudaErrorInvalidValue;
  ml = ma;
  if (A_local != nullptr && !make_map(&ml, A_local, p.K, p.m_local, lda_local, BK, HM)) return (int)cudaErrorInvalidValue;
  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT, COMM>;
  const size_t smem = (size_t)STAGES * STAGE_BYTES + EPI_BYTES + 1024;
  static int max_clusters = 0;   // per instantiation
  cudaLaunchConfig_t cfg = {};          // the pair (cluster of 2) is a compile-time attribute of the kernel
  cfg.blockDim = dim3(COMM == COMM_NONE ? 192 : 192 + COMM_THREADS, 1, 1);
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
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) *
                    (OUT == OUT_PART_F32 ? p.k_splits : (p.groups > 0 ? p.groups : 1));
  // the fused variants always launch every pair: their comm warps share the copy / reduce work of the
  // whole grid, and every CTA must be resident for the counters to advance
  const int clusters = (COMM != COMM_NONE || tiles >= max_clusters) ? max_clusters : tiles;
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  return (int)cudaLaunchKernelEx(&cfg, kern, ma, mb, ml, p);
}

// Sum of the split-reduction slabs: out[M, N] bf16 = sum_s part[s][M, N] (+ bias[N]), slabs added in
// index order so that the result does not depend on which pair produced which piece.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, long long slab, int splits,
                                                             __nv_bfloat16* __restrict__ out, long long ldo,
                                                             const __nv_bfloat16* __restrict__ bias, int M, int N) {
  const int vec_per_row = N / 8;
  const long long total = (long long)M * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row), c = (int)(i % vec_per_row) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const float* src = part + (long long)r * N + c;
    for (int sidx = 0; sidx < splits; ++sidx) {
      const float4 a = *reinterpret_cast<const float4*>(src + sidx * slab);
      const float4 b = *reinterpret_cast<const float4*>(src + sidx * slab + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    if (bias != nullptr) {
      float f[8];
      unpack8(ld8(bias + c), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    st8(out + (long long)r * ldo + c, pack8(acc));
  }
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
  if (!a_mn && !b_mn && out_mode == g2::OUT_BF16) return g2::launch<false, false, g2::OUT_BF16>(A, lda, B, ldb, p, st);
  if (!a_mn && b_mn && out_mode == g2::OUT_BF16) return g2::launch<false, true, g2::OUT_BF16>(A, lda, B, ldb, p, st);
  if (a_mn && b_mn && out_mode == g2::OUT_BF16) return g2::launch<true, true, g2::OUT_BF16>(A, lda, B, ldb, p, st);
  if (a_mn && b_mn && out_mode == g2::OUT_ACC_F32) return g2::launch<true, true, g2::OUT_ACC_F32>(A, lda, B, ldb, p, st);
  if (a_mn && b_mn && out_mode == g2::OUT_ACC_BF16) return g2::launch<true, true, g2::OUT_ACC_BF16>(A, lda, B, ldb, p, st);
  return (int)cudaErrorInvalidValue;
}

// Split-reduction form for small M (decode): the reduction is cut into `splits` pieces so that
// tiles x pieces fills the machine, every piece writes an fp32 partial tile into `part`
// ([splits, M, N] floats), and a second kernel adds the slabs in order into C (bf16, + optional bias).
// A [M, K] and B [N, K] row-major; N a multiple of 8.  msrl_gemm_pair_splitk_plan suggests `splits`
// (0: the plain kernel or the library is the better choice).
MSRL_API int msrl_gemm_pair_splitk_plan(int M, int N, int K) {
  const int tiles = ((M + g2::BM - 1) / g2::BM) * ((N + g2::BN - 1) / g2::BN);
  const int pairs = sm_count() / 2;
  const int num_kb = (K + g2::BK - 1) / g2::BK;
  if (tiles == 0 || N % 8 != 0 || K % 8 != 0) return 0;
  int splits = pairs / tiles;
  if (splits > num_kb / 8) splits = num_kb / 8;                   // at least 8 k-blocks per piece
  // the partial sums are written and read back once: keep them under about a third of the weight bytes
  const long long cap = (long long)(0.35 * K) / (4LL * (M < 1 ? 1 : M));
  if (splits > cap) splits = (int)cap;
  if (splits > 16) splits = 16;
  if (splits < 2) return 0;
  const int kb_per = (num_kb + splits - 1) / splits;
  return (num_kb + kb_per - 1) / kb_per;                          // no empty piece
}

MSRL_API int msrl_gemm_pair_splitk_bf16(const void* A, long long lda, const void* B, long long ldb, float* part,
                                        void* C, long long ldc, const void* bias, int M, int N, int K, int splits,
                                        int* error, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  if (K <= 0 || K % 8 != 0 || N % 8 != 0 || ldc % 8 != 0 || splits < 1 || splits > 64 ||
      (reinterpret_cast<uintptr_t>(part) & 15) != 0 || (reinterpret_cast<uintptr_t>(C) & 15) != 0)
    return (int)cudaErrorInvalidValue;
  {   // no piece may be empty: the pipeline hands an accumulator over only after at least one MMA
    const int num_kb = (K + g2::BK - 1) / g2::BK;
    const int kb_per = (num_kb + splits - 1) / splits;
    splits = (num_kb + kb_per - 1) / kb_per;
  }
  g2::Params p{};
  p.M = M; p.N = N; p.K = K;
  p.C = part;
  p.ldc = N;
  p.k_splits = splits;
  p.error = error;
  int rc = g2::launch<false, false, g2::OUT_PART_F32>(A, lda, B, ldb, p, st);
  if (rc != 0) return rc;
  const long long vecs = (long long)M * (N / 8);
  long long blocks = (vecs + 255) / 256;
  if (blocks > 4LL * sm_count()) blocks = 4LL * sm_count();
  g2::splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, st>>>(part, (long long)M * N, splits, (__nv_bfloat16*)C, ldc,
                                                              (const __nv_bfloat16*)bias, M, N);
  return (int)cudaGetLastError();
}

// Grouped weight gradient (mixture-of-experts layers): for every group g,
//   C_g[M, N] += A[seg[g] : seg[g+1], :M]^T  B[seg[g] : seg[g+1], :N]
// with A [rows, M] and B [rows, N] row-major bf16 (both read as MN-major operands), C_g = C + g * c_group_stride
// (leading dimension ldc), out_mode 1: fp32 accumulate, 2: bf16 accumulate.  `seg` is a DEVICE array of
// groups + 1 row offsets, multiples of 64 (the padded expert segments of the permuted token layout; pad rows
// must be zero in A or B); groups without rows are skipped on the device, nothing is read back to the host.
MSRL_API int msrl_gemm_pair_grouped_wgrad(const void* A, long long lda, const void* B, long long ldb, void* C,
                                          long long ldc, long long c_group_stride, int out_mode, const int* seg,
                                          int groups, int M, int N, long long rows, int* error, cudaStream_t st) {
  if (groups <= 0 || M == 0 || N == 0 || rows == 0) return 0;
  if (M % 8 != 0 || N % 8 != 0 || rows % 8 != 0 || rows > 0x7fffffffLL ||
      (out_mode != g2::OUT_ACC_F32 && out_mode != g2::OUT_ACC_BF16))
    return (int)cudaErrorInvalidValue;
  g2::Params p{};
  p.M = M; p.N = N; p.K = (int)rows;
  p.C = C;
  p.ldc = ldc;
  p.error = error;
  p.groups = groups;
  p.seg = seg;
  p.c_group_stride = c_group_stride;
  if (out_mode == g2::OUT_ACC_F32) return g2::launch<true, true, g2::OUT_ACC_F32>(A, lda, B, ldb, p, st);
  return g2::launch<true, true, g2::OUT_ACC_BF16>(A, lda, B, ldb, p, st);
}

// ---- communication-fused forms on CTA pairs (same contracts as msrl_ag_gemm_bf16_tn / msrl_gemm_rs_bf16_tn,
// token shards in multiples of 256 rows) ------------------------------------------------------------
MSRL_API int msrl_ag_gemm_pair_bf16_tn(void* const* peer_a, long long ld_peer, void* gathered, const void* B,
                                       long long ldb, void* C, long long ldc, int m_local, int N, int K, int rank,
                                       int world, unsigned int* tile_ready, int* error, cudaStream_t st) {
  if (m_local == 0 || N == 0) return 0;
  if (K % 8 != 0 || m_local % g2::BM != 0 || world > g2::MAX_RANKS || ld_peer % 8 != 0) return (int)cudaErrorInvalidValue;
  g2::Params p{};
  p.M = m_local * world; p.N = N; p.K = K;
  p.C = C;
  p.ldc = ldc;
  p.error = error;
  p.rank = rank; p.world = world; p.m_local = m_local;
  for (int r = 0; r < world; ++r) p.peer[r] = peer_a[r];
  p.ld_peer = ld_peer;
  p.gathered = (__nv_bfloat16*)gathered;
  p.tile_ready = tile_ready;
  cudaError_t e = cudaMemsetAsync(tile_ready, 0, sizeof(unsigned int) * (size_t)(p.M / g2::HM), st);
  if (e != cudaSuccess) return (int)e;
  return g2::launch<false, false, g2::OUT_BF16, g2::COMM_AG>(gathered, K, B, ldb, p, st, peer_a[rank], ld_peer);
}

MSRL_API int msrl_gemm_rs_pair_bf16_tn(const void* A, long long lda, const void* B, long long ldb,
                                       void* const* peer_stage, void* const* peer_flag, unsigned int* done, void* out,
                                       long long ld_out, int m_local, int N, int K, int rank, int world,
                                       unsigned int target, int* error, cudaStream_t st) {
  if (m_local == 0 || N == 0) return 0;
  if (K % 8 != 0 || N % 8 != 0 || m_local % g2::BM != 0 || world > g2::MAX_RANKS || ld_out % 8 != 0)
    return (int)cudaErrorInvalidValue;
  g2::Params p{};
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
  return g2::launch<false, false, g2::OUT_BF16, g2::COMM_RS>(A, lda, B, ldb, p, st);
}
