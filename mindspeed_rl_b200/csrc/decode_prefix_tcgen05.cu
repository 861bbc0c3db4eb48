// Shared-prefix pass of grouped decode on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// head dim 128.
//
// The n samples of one prompt attend to the same prompt keys.  One CTA takes one (group, KV head,
// prefix split): the query rows of all members (members x q-heads-per-KV-head <= 128 rows, row =
// member * rep + head) form ONE 128-row A operand, so the prompt's K/V is read once per group and
// multiplied by every member in the same MMAs.  The mma.sync form of this pass (decode.cu) is bound
// by the legacy tensor path; here a 64- or 128-key tile costs two groups of eight tcgen05.mma.
//
//   Q            gathered by the soft-max warps from the decode step's [B, heads * 128] activations
//                into shared memory in the UMMA K-major 128-byte-swizzled layout (rows past the
//                group's members are zero);
//   K, V         straight from the paged cache: the cache is one 2-D tensor map
//                [num_blocks * block_size, n_kv_heads * 128]; a key tile is BN / block_size boxes of
//                [block_size rows x 64 columns], each landing at its rows of the swizzled tile;
//   S = Q K^T    into one of two TMEM score buffers; soft-max by eight warps (two threads per row),
//                P through shared memory, O += P V with V as MN-major operand, O resident in TMEM;
//   output       un-normalised partial (O, running max in the exp2 domain, sum) per member row into
//                the split slots that the merge kernel of decode.cu combines with the members' own
//                suffix partials.
//
// Contract: every group's shared prefix is a multiple of BN keys (the caller rounds the shared
// length down and leaves the remainder to the per-sequence suffix kernel), so no tile is ragged
// and no uninitialised cache slot is ever multiplied.  A prefix that breaks the contract sets the
// status word and writes empty partials.
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in the status word, skips the
// rest, frees TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>

#include "mma_utils.cuh"
#include "tcgen05_utils.cuh"

namespace msrl {
namespace dp5 {

using namespace t5;

constexpr int BM = 128, D = 128;
constexpr uint32_t TILE_HALF = 128 * 64 * 2;          // one [128 rows x 64 cols] bf16 swizzled half tile
constexpr uint32_t TILE_BYTES = 2 * TILE_HALF;         // 32 KiB
constexpr uint32_t SMEM_Q = 0;
constexpr uint32_t smem_bytes(int bn) { return TILE_BYTES + 4u * (2u * bn * 64 * 2) + 128u * bn * 2; }
constexpr int SOFTMAX_WARPS = 8, TMA_WARP = 8, MMA_WARP = 9, THREADS = 320;
constexpr int GROUP_MAX = 8;                           // members per group (rows of the group table)

enum { ERR_SMEM = 40, ERR_Q = 41, ERR_K = 42, ERR_V = 43, ERR_S = 44, ERR_P = 45, ERR_PV = 46, ERR_EMPTY = 47,
       ERR_PREFIX = 48 };

struct Params {
  const __nv_bfloat16* q;     // one token per sequence
  HeadLayout Lq;
  const int* block_tables;    // [B, max_blocks]
  int max_blocks, block_size;
  const int* group_rows;      // [n_groups, GROUP_MAX] batch rows (-1 = empty)
  const int* group_prefix;    // [n_groups] shared keys of the group (multiple of the key tile)
  float* part_o;              // [B, nh, slot_total, D]
  float* part_ml;             // [B, nh, slot_total, 2]
  int nh, nkv, slot_total, npre;
  float scale_log2;
  int* error;
};

// Empty partial (no keys): max -inf, sum 0, zeros, for every member row of this CTA.
__device__ __forceinline__ void write_empty(const Params& p, const int* rows, int rep, int hk, int sp) {
  for (int r = threadIdx.x; r < GROUP_MAX * rep; r += blockDim.x) {
    const int b = rows[r / rep];
    if (b < 0) continue;
    const long long pi = ((long long)b * p.nh + hk * rep + r % rep) * p.slot_total + sp;
    for (int d = 0; d < D; d += 4) *reinterpret_cast<float4*>(p.part_o + pi * D + d) = make_float4(0.f, 0.f, 0.f, 0.f);
    p.part_ml[pi * 2] = -INFINITY;
    p.part_ml[pi * 2 + 1] = 0.f;
  }
}

// BN = keys per tile.  128: one CTA per SM (192 KiB of shared memory, 512 TMEM columns).  64: two
// CTAs per SM (112 KiB, 256 columns each), so that one CTA's soft-max, prologue and epilogue overlap
// the other's tensor work.
template <int BN>
__global__ void __launch_bounds__(THREADS, BN == 128 ? 1 : 2)
prefix_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], s_free[2], p_ready, pv_done;
  __shared__ uint32_t tmem_slot;
  constexpr uint32_t KV_HALF = BN * 64 * 2, KV_BYTES = 2 * KV_HALF;
  constexpr uint32_t SMEM_K = TILE_BYTES, SMEM_V = SMEM_K + 2 * KV_BYTES, SMEM_P = SMEM_V + 2 * KV_BYTES;
  constexpr uint32_t TMEM_COLS = BN == 128 ? 512 : 256;      // S0 [0,BN) S1 [BN,2BN) O [2BN, 2BN+128)
  constexpr int HALF = BN / 2, NCH = HALF / 32;              // key columns per soft-max thread

  const int g = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  const int rep = p.nh / p.nkv;
  const int* rows = p.group_rows + (long long)g * GROUP_MAX;
  const int lead = rows[0];
  if (lead < 0) return;                           // unused group slot (uniform for the CTA)
  const int prefix = p.group_prefix[g];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int n_tiles = 0, t0 = 0;
  if (prefix % BN != 0) {
    if (threadIdx.x == 0) atomicCAS(p.error, 0, ERR_PREFIX);
  } else {
    const int tiles_total = prefix / BN;
    const int per = (tiles_total + p.npre - 1) / p.npre;
    t0 = sp * per;
    n_tiles = min(tiles_total, t0 + per) - t0;
  }
  if (n_tiles <= 0) {                             // nothing shared, or more splits than tiles
    write_empty(p, rows, rep, hk, sp);
    return;
  }
  {
    // the tiles must fit behind the 1024-byte alignment of the dynamic segment
    uint32_t dyn;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;\n" : "=r"(dyn));
    if ((uint32_t)(smem - smem_raw) + smem_bytes(BN) > dyn) {
      if (threadIdx.x == 0) atomicCAS(p.error, 0, ERR_SMEM);
      write_empty(p, rows, rep, hk, sp);
      return;
    }
  }
  float (*l_part)[BM] = reinterpret_cast<float (*)[BM]>(smem + SMEM_P);   // used after the last P V product

  if (threadIdx.x == 0) {
    mbar_init(&q_full, SOFTMAX_WARPS);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], SOFTMAX_WARPS);
    }
    mbar_init(&p_ready, SOFTMAX_WARPS);
    mbar_init(&pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_o = tmem + 2 * BN;

  if (warp == TMA_WARP) {
    // ---------------- TMA producer: the prompt's K/V blocks through the lead member's block table ----------------
    if (elect_one()) {
      const int* bt = p.block_tables + (long long)lead * p.max_blocks;
      const int bs = p.block_size;
      const int blocks_per_tile = BN / bs;
      const uint32_t blk_bytes = (uint32_t)bs * 128u;            // bytes of one block inside a half tile
      const int col = hk * D;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const uint32_t use = j >> 1;
        const int blk0 = (t0 + j) * blocks_per_tile;
        if (use > 0) ok = mbar_wait(&k_empty[st], (use - 1) & 1, p.error, ERR_EMPTY);
        if (!ok) break;
        mbar_expect_tx(&k_full[st], KV_BYTES);
        unsigned char* sk = smem + SMEM_K + st * KV_BYTES;
        for (int i = 0; i < blocks_per_tile; ++i) {
          const int row = __ldg(bt + blk0 + i) * bs;
          tma_load_2d(sk + i * blk_bytes, &map_k, &k_full[st], col, row);
          tma_load_2d(sk + KV_HALF + i * blk_bytes, &map_k, &k_full[st], col + 64, row);
        }
        if (use > 0) ok = mbar_wait(&v_empty[st], (use - 1) & 1, p.error, ERR_EMPTY);
        if (!ok) break;
        mbar_expect_tx(&v_full[st], KV_BYTES);
        unsigned char* sv = smem + SMEM_V + st * KV_BYTES;
        for (int i = 0; i < blocks_per_tile; ++i) {
          const int row = __ldg(bt + blk0 + i) * bs;
          tma_load_2d(sv + i * blk_bytes, &map_v, &v_full[st], col, row);
          tma_load_2d(sv + KV_HALF + i * blk_bytes, &map_v, &v_full[st], col + 64, row);
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t id_s = idesc_bf16(BM, BN, false);
      constexpr uint32_t id_o = idesc_bf16(BM, D, true);
      const uint32_t q_addr = smem_u32(smem + SMEM_Q), p_addr = smem_u32(smem + SMEM_P);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1, p.error, ERR_K)) return false;
        if (j >= 2 && !mbar_wait(&s_free[st], ((j >> 1) - 1) & 1, p.error, ERR_S)) return false;
        fence_after();
        const uint32_t k_addr = smem_u32(smem + SMEM_K + st * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          umma(tmem + st * BN, desc_sw128(q_addr + (kk >> 2) * TILE_HALF + (kk & 3) * 32, 16, 1024),
               desc_sw128(k_addr + (kk >> 2) * KV_HALF + (kk & 3) * 32, 16, 1024), id_s,
               kk > 0 ? 1u : 0u);
        }
        commit(&s_full[st]);
        commit(&k_empty[st]);
        return true;
      };
      bool ok = mbar_wait(&q_full, 0, p.error, ERR_Q);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);            // next tile's scores run during this soft-max
        if (!ok) break;
        ok = mbar_wait(&p_ready, j & 1, p.error, ERR_P) && mbar_wait(&v_full[st], (j >> 1) & 1, p.error, ERR_V);
        if (!ok) break;
        fence_after();
        const uint32_t v_addr = smem_u32(smem + SMEM_V + st * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint32_t pa = p_addr + (kk >> 2) * TILE_HALF + (kk & 3) * 32;
          umma(tmem_o, desc_sw128(pa, 16, 1024), desc_sw128(v_addr + kk * 2048, KV_HALF, 1024), id_o,
               (j > 0 || kk > 0) ? 1u : 0u);
        }
        commit(&pv_done);
        commit(&v_empty[st]);
      }
    }
  } else {
    // ---------------- Q gather, soft-max, partial output ----------------
    // Q: 128 rows x 16 chunks of 16 bytes; row r = member r / rep, head hk * rep + r % rep; K-major,
    // 128-byte swizzle: chunk index XOR (row % 8) inside the row's 128 bytes of its 64-column half.
    for (int idx = threadIdx.x; idx < BM * (D / 8); idx += SOFTMAX_WARPS * 32) {
      const int r = idx >> 4, chunk = idx & 15;
      const int mem = r / rep;
      const int b = (mem < GROUP_MAX) ? rows[mem] : -1;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (b >= 0) val = *reinterpret_cast<const uint4*>(p.q + head_offset(p.Lq, b, hk * rep + r % rep) + chunk * 8);
      unsigned char* dst = smem + SMEM_Q + (chunk >> 3) * TILE_HALF + (r >> 3) * 1024 + (r & 7) * 128 +
                           (((chunk & 7) ^ (r & 7)) << 4);
      *reinterpret_cast<uint4*>(dst) = val;
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic smem writes -> UMMA reads
    __syncwarp();
    if (lane == 0) mbar_arrive(&q_full);

    // Two threads per query row: warps 0-3 own key columns [0, BN/2) of the tile, warps 4-7 the other
    // half (a warp reaches the TMEM lanes of its quarter, warp % 4).  Both read the whole score row
    // for its maximum, so they agree on the running maximum without talking; each keeps the partial
    // sum of its own columns, rescales its half of the O columns and writes its half of P.
    const int wg = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;                    // row inside the tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    unsigned char* sp_ = smem + SMEM_P + ((wg * HALF) >> 6) * TILE_HALF;   // the 64-column half tile of P
    constexpr int NCHUNK = HALF / 8;
    const int chunk0 = ((wg * HALF) & 63) >> 3;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      // warp-uniform outcome: the tcgen05.ld / st below are warp-wide instructions
      ok = mbar_wait_warp(&s_full[sb], (j >> 1) & 1, p.error, ERR_S);
      if (!ok) break;
      fence_after();
      float s[HALF], t[32];
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      // the other half: maximum only
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        tmem_ld32(tmem + lane_base + sb * BN + (wg ^ 1) * HALF + c * 32, t);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmaxf(mx0, t[i]);
          mx1 = fmaxf(mx1, t[i + 1]);
          mx2 = fmaxf(mx2, t[i + 2]);
          mx3 = fmaxf(mx3, t[i + 3]);
        }
      }
      // this thread's half
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        tmem_ld32(tmem + lane_base + sb * BN + wg * HALF + c * 32, t);
#pragma unroll
        for (int i = 0; i < 32; ++i) s[c * 32 + i] = t[i];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmaxf(mx0, t[i]);
          mx1 = fmaxf(mx1, t[i + 1]);
          mx2 = fmaxf(mx2, t[i + 2]);
          mx3 = fmaxf(mx3, t[i + 3]);
        }
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);              // the score buffer may be overwritten
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;   // scale > 0
      // The running maximum follows the row maximum lazily: it moves only when the row maximum
      // passed it by more than 8 (a factor 256, harmless in fp32 sums and bf16 P), so that O is
      // rescaled in TMEM on few tiles only.  The partial is reported relative to this reference.
      float m_new = fmaxf(m_run, mx);
      if (m_run != -INFINITY && m_new - m_run <= 8.f) m_new = m_run;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m_run - m_use);
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
      for (int i = 0; i < HALF; i += 4) {
        s[i] = exp2f(fmaf(s[i], p.scale_log2, -m_use));
        s[i + 1] = exp2f(fmaf(s[i + 1], p.scale_log2, -m_use));
        s[i + 2] = exp2f(fmaf(s[i + 2], p.scale_log2, -m_use));
        s[i + 3] = exp2f(fmaf(s[i + 3], p.scale_log2, -m_use));
        sum0 += s[i];
        sum1 += s[i + 1];
        sum2 += s[i + 2];
        sum3 += s[i + 3];
      }
      l_run = l_run * corr + ((sum0 + sum1) + (sum2 + sum3));
      m_run = m_new;
      if (j > 0) {
        // the previous P V product must be finished before P is overwritten or O is rescaled
        ok = mbar_wait_warp(&pv_done, (j - 1) & 1, p.error, ERR_PV);
        if (!ok) break;
        fence_after();
        if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            tmem_ld32(tmem_o + lane_base + wg * 64 + c * 32, t);
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] *= corr;
            tmem_st32(tmem_o + lane_base + wg * 64 + c * 32, t);
          }
        }
      }
      // P half row -> shared memory, K-major, 128-byte swizzle: 16-byte chunk index XOR (row % 8)
#pragma unroll
      for (int chunk = 0; chunk < NCHUNK; ++chunk) {
        unsigned char* dst = sp_ + (row >> 3) * 1024 + (row & 7) * 128 + (((chunk0 + chunk) ^ (row & 7)) << 4);
        *reinterpret_cast<bf16x8*>(dst) = pack8(&s[chunk * 8]);
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic smem writes -> UMMA reads
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready);
    }
    if (ok) ok = mbar_wait_warp(&pv_done, (n_tiles - 1) & 1, p.error, ERR_PV);
    // the two partial sums of a row meet in shared memory
    l_part[wg][row] = l_run;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");        // every soft-max thread reaches this once
    // tcgen05.ld is a warp-wide (.sync.aligned) instruction: every lane of the warp takes the same path
    // through the loads; only the stores depend on whether the lane's row belongs to a member
    ok = __all_sync(0xffffffffu, ok);
    const int mem = row / rep;
    const int b = (mem < GROUP_MAX) ? rows[mem] : -1;
    const long long pi = ((long long)(b >= 0 ? b : 0) * p.nh + hk * rep + row % rep) * p.slot_total + sp;
    float* dst = p.part_o + pi * D + wg * 64;
    if (ok) {
      fence_after();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float v[32];
        tmem_ld32(tmem_o + lane_base + wg * 64 + hh * 32, v);
        if (b >= 0) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(dst + hh * 32 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
      }
      if (b >= 0 && wg == 0) {
        p.part_ml[pi * 2] = m_run;
        p.part_ml[pi * 2 + 1] = l_part[0][row] + l_part[1][row];
      }
    } else if (b >= 0) {
      // a wait gave up (the status word says which): leave a well-formed empty partial behind
      for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (wg == 0) {
        p.part_ml[pi * 2] = -INFINITY;
        p.part_ml[pi * 2 + 1] = 0.f;
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
  }
}

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

// The paged cache as [num_blocks * block_size rows, n_kv_heads * 128 columns] bf16; box = 64 columns x
// one block of rows.
static bool make_cache_map(CUtensorMap* map, const void* base, long long rows, long long width, unsigned box_rows) {
  auto fn = encode_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || width % 8 != 0) return false;
  cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(width * 2)};
  cuuint32_t box[2] = {64u, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace dp5
}  // namespace msrl

using namespace msrl;

// Keys per tile of the tcgen05 shared-prefix kernel, i.e. the multiple that the caller must round the
// groups' shared prefix down to; 0 when the kernel does not cover the shape (head size other than
// 128, more than 16 q heads per KV head, a block size that does not divide the tile or is below 8).
MSRL_API int msrl_paged_prefix_tcgen05_tile(int nh, int nkv, int D, int block_size) {
  if (D != dp5::D || nkv <= 0 || nh % nkv != 0 || (nh / nkv) * dp5::GROUP_MAX > dp5::BM) return 0;
  static int bn = 0;
  if (bn == 0) {
    const char* e = getenv("MSRL_PREFIX_KEY_TILE");
    bn = (e != nullptr && atoi(e) == 128) ? 128 : 64;
  }
  if (block_size < 8 || bn % block_size != 0) return 0;
  return bn;
}

// Shared-prefix partials of grouped decode (slots [0, npre) of every member row; same tables as
// msrl_paged_decode_grouped in decode.cu).  k_cache / v_cache: [num_blocks, block_size, nkv, 128] bf16.
// Returns cudaErrorNotSupported for shapes the kernel does not cover: the caller falls back.
MSRL_API int msrl_paged_prefix_tcgen05(const void* q, const long long* q_layout4, const void* k_cache,
                                       const void* v_cache, long long num_blocks, const int* block_tables,
                                       int max_blocks, const int* group_rows, const int* group_prefix, int n_groups,
                                       float* part_o, float* part_ml, int nh, int nkv, int D, int block_size,
                                       int slot_total, int npre, int* error, cudaStream_t st) {
  if (n_groups == 0) return 0;
  const int bn = msrl_paged_prefix_tcgen05_tile(nh, nkv, D, block_size);
  if (bn == 0 || npre < 1 || num_blocks <= 0 || q_layout4[0] % 8 != 0 || q_layout4[1] % 8 != 0 ||
      q_layout4[3] % 8 != 0 || q_layout4[2] <= 0 || (reinterpret_cast<uintptr_t>(q) & 15) != 0)
    return (int)cudaErrorNotSupported;
  CUtensorMap mk, mv;
  const long long rows = num_blocks * block_size, width = (long long)nkv * D;
  if (!dp5::make_cache_map(&mk, k_cache, rows, width, (unsigned)block_size) ||
      !dp5::make_cache_map(&mv, v_cache, rows, width, (unsigned)block_size))
    return (int)cudaErrorNotSupported;
  dp5::Params p{};
  p.q = (const __nv_bfloat16*)q;
  p.Lq = HeadLayout{q_layout4[0], (int)q_layout4[1], (int)q_layout4[2], (int)q_layout4[3]};
  p.block_tables = block_tables;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.group_rows = group_rows;
  p.group_prefix = group_prefix;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.nh = nh;
  p.nkv = nkv;
  p.slot_total = slot_total;
  p.npre = npre;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)D);
  p.error = error;
  static bool attr_set = false;
  const int smem = (int)dp5::smem_bytes(bn) + (bn == 128 ? 1024 : 896);   // 64: two CTAs in 228 KiB
  if (!attr_set) {
    cudaError_t e = bn == 128
        ? cudaFuncSetAttribute(dp5::prefix_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
        : cudaFuncSetAttribute(dp5::prefix_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid(n_groups, nkv, npre);
  if (bn == 128)
    dp5::prefix_tcgen05_kernel<128><<<grid, dp5::THREADS, smem, st>>>(mk, mv, p);
  else
    dp5::prefix_tcgen05_kernel<64><<<grid, dp5::THREADS, smem, st>>>(mk, mv, p);
  return (int)cudaGetLastError();
}
