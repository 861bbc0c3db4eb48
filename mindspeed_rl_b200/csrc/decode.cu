// Rollout-engine kernels: paged KV-cache write, paged GQA decode attention (split-KV with a
// merge pass), gather of cached K/V for chunked prefill, and the token sampler.
//
// Cache layout: k_cache / v_cache = [num_blocks, block_size, n_kv_heads, D] bf16; a token's
// slot is block * block_size + offset.  The decode kernel processes one (sequence, KV head,
// split) per CTA and serves all q heads of the KV group from one pass over K/V using
// mma.sync tiles (q heads padded to 16 rows).
//
// These replace the rollout engine the reference imports (vLLM paged attention + sampler;
// mindspeed_rl/models/rollout/vllm_engine.py:222-250,423-504).
#include "mma_utils.cuh"

namespace msrl {

constexpr float kLog2eD = 1.4426950408889634f;
constexpr float kLn2D = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------------
// KV-cache write
// ---------------------------------------------------------------------------------------------
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ k, HeadLayout Lk,
                                      const __nv_bfloat16* __restrict__ v, HeadLayout Lv,
                                      const long long* __restrict__ slots,
                                      __nv_bfloat16* __restrict__ k_cache,
                                      __nv_bfloat16* __restrict__ v_cache, long long T, int nkv,
                                      int D) {
  const int vec_per_head = D >> 3;
  const long long total = T * nkv * vec_per_head;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % vec_per_head);
    const long long th = idx / vec_per_head;
    const int h = (int)(th % nkv);
    const long long t = th / nkv;
    const long long slot = slots[t];
    if (slot < 0) continue;
    const long long dst = (slot * nkv + h) * D + c * 8;
    st8(k_cache + dst, ld8(k + head_offset(Lk, t, h) + c * 8));
    st8(v_cache + dst, ld8(v + head_offset(Lv, t, h) + c * 8));
  }
}

// Gather cached K/V of whole sequences into contiguous [Tk, nkv, D] buffers (prefill of a chunk
// that attends to an already cached prefix).  token_seq[t], token_pos[t] give the owning
// sequence row of the block table and the position inside the sequence.
__global__ void kv_cache_gather_kernel(const __nv_bfloat16* __restrict__ k_cache,
                                       const __nv_bfloat16* __restrict__ v_cache,
                                       const int* __restrict__ block_tables, int max_blocks,
                                       const int* __restrict__ token_seq,
                                       const int* __restrict__ token_pos,
                                       __nv_bfloat16* __restrict__ k_out,
                                       __nv_bfloat16* __restrict__ v_out, long long T, int nkv,
                                       int D, int block_size) {
  const int vec_per_tok = (nkv * D) >> 3;
  const long long total = T * vec_per_tok;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % vec_per_tok);
    const long long t = idx / vec_per_tok;
    const int pos = token_pos[t];
    const int blk = block_tables[(long long)token_seq[t] * max_blocks + pos / block_size];
    const long long src = ((long long)blk * block_size + pos % block_size) * nkv * D + c * 8;
    st8(k_out + t * nkv * D + c * 8, ld8(k_cache + src));
    st8(v_out + t * nkv * D + c * 8, ld8(v_cache + src));
  }
}

// ---------------------------------------------------------------------------------------------
// Paged decode attention
// ---------------------------------------------------------------------------------------------
struct DecodeParams {
  const __nv_bfloat16* q;  // one token per sequence
  HeadLayout Lq;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_tables;  // [B, max_blocks]
  const int* context_lens;  // [B] (includes the current token)
  __nv_bfloat16* out;       // [B, nh*D]
  long long out_stride;
  float* part_o;            // scratch [B, nh, nsplit, D]
  float* part_ml;           // scratch [B, nh, nsplit, 2]  (m in exp2 domain, l)
  int max_blocks, block_size, nh, nkv, nsplit;
  float scale_log2;
  // shared-prefix (grouped) decode: sequences that share their first key_start[b] keys with the
  // other members of their group skip those keys here; the group kernel covers them once.
  const int* key_start;     // [B] or nullptr
  int slot_base;            // first partial slot this kernel writes
  int slot_total;           // partial slots per (b, head); 1 = write `out` directly
  const int* group_rows;    // [n_groups, kGroupMax] batch rows (-1 = empty)
  const int* group_prefix;  // [n_groups] shared keys of the group
  int npre;                 // prefix splits (slots 0 .. npre-1)
  int block_shift;          // log2(block_size), or -1 when it is not a power of two
};

constexpr int kGroupMax = 8;

template <int D>
__global__ void __launch_bounds__(128) paged_decode_kernel(const DecodeParams p) {
  constexpr int CH = 64, LD = D + 8, THREADS = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // 16 x LD
  __nv_bfloat16* sK = sQ + 16 * LD;                                 // 2 x CH x LD
  __nv_bfloat16* sV = sK + 2 * CH * LD;                             // 2 x CH x LD

  const int b = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  const int rep = p.nh / p.nkv;
  const int ctx = p.context_lens[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int frow = lane >> 2, fcol = (lane & 3) * 2;

  const int k0 = (p.key_start != nullptr) ? min(p.key_start[b], ctx) : 0;
  int per_split = (ctx - k0 + p.nsplit - 1) / p.nsplit;
  per_split = ((per_split + CH - 1) / CH) * CH;
  const int kbeg = k0 + sp * per_split;
  const int kend = min(ctx, kbeg + per_split);
  const int n_chunks = (kend > kbeg) ? (kend - kbeg + CH - 1) / CH : 0;

  // Q rows: the `rep` heads of this KV group; rows >= rep are zero
  for (int i = threadIdx.x; i < 16 * (D / 8); i += THREADS) {
    const int r = i / (D / 8), c = i % (D / 8);
    const bool ok = r < rep;
    const __nv_bfloat16* src = p.q + head_offset(p.Lq, b, hk * rep + (ok ? r : 0)) + c * 8;
    cp_async16(sQ + r * LD + c * 8, src, ok);
  }
  const int* bt = p.block_tables + (long long)b * p.max_blocks;
  auto issue = [&](int chunk, int stage) {
    const int base = kbeg + chunk * CH;
    for (int i = threadIdx.x; i < CH * (D / 8); i += THREADS) {
      const int r = i / (D / 8), c = i % (D / 8);
      const int key = base + r;
      const bool ok = key < kend;
      const int kk = ok ? key : kbeg;
      int blk, off;
      if (p.block_shift >= 0) {
        blk = __ldg(bt + (kk >> p.block_shift));
        off = kk & (p.block_size - 1);
      } else {
        blk = __ldg(bt + kk / p.block_size);
        off = kk % p.block_size;
      }
      const long long src = (((long long)blk * p.block_size + off) * p.nkv + hk) * D + c * 8;
      cp_async16(sK + (stage * CH + r) * LD + c * 8, p.k_cache + src, ok);
      cp_async16(sV + (stage * CH + r) * LD + c * 8, p.v_cache + src, ok);
    }
  };
  if (n_chunks > 0) issue(0, 0);
  cp_async_commit();

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int ch = 0; ch < n_chunks; ++ch) {
    const int st = ch & 1;
    if (ch + 1 < n_chunks) {
      issue(ch + 1, st ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* tK = sK + (st * CH + warp * 16) * LD;  // this warp's 16 keys
    const __nv_bfloat16* tV = sV + (st * CH + warp * 16) * LD;
    float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4], bfr[4];
      ldmatrix_x4(a, smem_u32(sQ + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8));
      ldmatrix_x4(bfr, smem_u32(tK + ((lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8));
      mma_16816(s[0], a, bfr[0], bfr[1]);
      mma_16816(s[1], a, bfr[2], bfr[3]);
    }
    const int key0 = kbeg + ch * CH + warp * 16;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = key0 + nt * 8 + fcol + (j & 1);
        const float v = (key < kend) ? s[nt][j] * p.scale_log2 : -INFINITY;
        s[nt][j] = v;
        mx[j >> 1] = fmaxf(mx[j >> 1], v);
      }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      corr[r] = exp2f(m_run[r] - m_use[r]);
      m_run[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = exp2f(s[nt][j] - m_use[j >> 1]);
        s[nt][j] = e;
        rs[j >> 1] += e;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + rs[r];
    uint32_t a[4];
    a[0] = pack_bf16(s[0][0], s[0][1]);
    a[1] = pack_bf16(s[0][2], s[0][3]);
    a[2] = pack_bf16(s[1][0], s[1][1]);
    a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t bfr[4];
      ldmatrix_x4_trans(bfr, smem_u32(tV + (lane & 15) * LD + dp * 16 + (lane >> 4) * 8));
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        o_acc[2 * dp][j] *= corr[0];
        o_acc[2 * dp][2 + j] *= corr[1];
        o_acc[2 * dp + 1][j] *= corr[0];
        o_acc[2 * dp + 1][2 + j] *= corr[1];
      }
      mma_16816(o_acc[2 * dp], a, bfr[0], bfr[1]);
      mma_16816(o_acc[2 * dp + 1], a, bfr[2], bfr[3]);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the 4 warps through shared memory (re-using the K/V stages)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  float* sO = reinterpret_cast<float*>(sK);        // [4][16][D]
  float* sM = sO + 4 * 16 * D;                     // [4][16]
  float* sL = sM + 4 * 16;                         // [4][16]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = frow + r * 8;
    if ((lane & 3) == 0) {
      sM[warp * 16 + row] = m_run[r];
      sL[warp * 16 + row] = l_run[r];
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      sO[(warp * 16 + row) * D + dt * 8 + fcol] = o_acc[dt][2 * r];
      sO[(warp * 16 + row) * D + dt * 8 + fcol + 1] = o_acc[dt][2 * r + 1];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < rep * D; i += THREADS) {
    const int r = i / D, d = i % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, sM[w * 16 + r]);
    const float mu = (m == -INFINITY) ? 0.f : m;
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = exp2f(sM[w * 16 + r] - mu);
      l += sL[w * 16 + r] * c;
      o += sO[(w * 16 + r) * D + d] * c;
    }
    const int h = hk * rep + r;
    if (p.slot_total == 1) {
      p.out[(long long)b * p.out_stride + (long long)h * D + d] =
          __float2bfloat16(l > 0.f ? o / l : 0.f);
    } else {
      const long long pi = ((long long)b * p.nh + h) * p.slot_total + p.slot_base + sp;
      p.part_o[pi * D + d] = o;
      if (d == 0) {
        p.part_ml[pi * 2] = m;
        p.part_ml[pi * 2 + 1] = l;
      }
    }
  }
}

// Shared-prefix pass of grouped decode.  The n samples of one prompt share the prompt's KV
// blocks; instead of streaming them once per sample, one CTA handles a whole group for one KV
// head: the query rows of all members (members x heads-per-KV-head <= 64 rows, 16 per warp) run
// against each 64-key chunk of the shared prefix, which is therefore read from HBM once per group.
// Grid (group, kv head, prefix split); partial results go to slots [0, npre) of every member and
// are merged with the members' own suffix partials by the merge kernel.
// Pipeline of the shared-prefix kernel: 32 keys per stage, three stages (two chunks in flight while one
// is multiplied), 70 KB of shared memory per CTA at D = 128, so three CTAs share an SM.  The kernel is
// bound by instruction issue and load latency, not by bytes, hence: block ids by shift / mask when the
// block size is a power of two, the query fragments held in registers for the whole pass, and the
// rescale of the output accumulators skipped while no row of the warp raised its running maximum.
constexpr int kPrefixChunk = 32;
constexpr int kPrefixStages = 3;
template <int D>
__global__ void __launch_bounds__(128) paged_decode_prefix_kernel(const DecodeParams p) {
  constexpr int CH = kPrefixChunk, LD = D + 8, THREADS = 128, ROWS = 64, ST = kPrefixStages;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // 64 x LD
  __nv_bfloat16* sK = sQ + ROWS * LD;                               // ST x CH x LD
  __nv_bfloat16* sV = sK + ST * CH * LD;                            // ST x CH x LD

  const int g = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  const int rep = p.nh / p.nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int frow = lane >> 2, fcol = (lane & 3) * 2;
  const int* rows = p.group_rows + (long long)g * kGroupMax;
  const int prefix = p.group_prefix[g];
  const int lead = rows[0];
  if (lead < 0) return;   // unused group slot (uniform for the whole CTA)

  int per_split = (prefix + p.npre - 1) / p.npre;
  per_split = ((per_split + CH - 1) / CH) * CH;
  const int kbeg = sp * per_split;
  const int kend = min(prefix, kbeg + per_split);
  const int n_chunks = (kend > kbeg) ? (kend - kbeg + CH - 1) / CH : 0;

  // query rows: row = member * rep + head-in-group
  for (int i = threadIdx.x; i < ROWS * (D / 8); i += THREADS) {
    const int r = i / (D / 8), c = i % (D / 8);
    const int mem = r / rep;
    const int b = (mem < kGroupMax) ? rows[mem] : -1;
    const bool ok = b >= 0;
    const __nv_bfloat16* src = p.q + head_offset(p.Lq, ok ? b : lead, hk * rep + r % rep) + c * 8;
    cp_async16(sQ + r * LD + c * 8, src, ok);
  }
  cp_async_commit();
  const int* bt = p.block_tables + (long long)lead * p.max_blocks;
  const int shift = p.block_shift, mask = p.block_size - 1;
  const long long row_elems = (long long)p.nkv * D;
  const int my_r = threadIdx.x / (D / 8), my_c = (threadIdx.x % (D / 8)) * 8;   // first row / column of this thread
  constexpr int RSTEP = THREADS / (D / 8);                                      // rows between its copies
  auto issue = [&](int chunk, int stage) {
    const int base = kbeg + chunk * CH;
#pragma unroll
    for (int it = 0; it < CH / RSTEP; ++it) {
      const int r = my_r + it * RSTEP;
      const int key = base + r;
      const bool ok = key < kend;
      const int kk = ok ? key : kbeg;
      int blk, off;
      if (shift >= 0) {
        blk = __ldg(bt + (kk >> shift));
        off = kk & mask;
      } else {
        blk = __ldg(bt + kk / p.block_size);
        off = kk % p.block_size;
      }
      const long long src = ((long long)blk * p.block_size + off) * row_elems + (long long)hk * D + my_c;
      cp_async16(sK + (stage * CH + r) * LD + my_c, p.k_cache + src, ok);
      cp_async16(sV + (stage * CH + r) * LD + my_c, p.v_cache + src, ok);
    }
  };
  // prologue: ST - 1 chunks in flight (one commit group per chunk, empty groups keep the count uniform)
#pragma unroll
  for (int s = 0; s < ST - 1; ++s) {
    if (s < n_chunks) issue(s, s);
    cp_async_commit();
  }

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  // this warp's 16 query rows as A fragments, loaded once
  cp_async_wait<ST - 1>();          // the query group (the oldest) has landed
  __syncthreads();
  uint32_t qf[D / 16][4];
  {
    const __nv_bfloat16* tQ = sQ + warp * 16 * LD;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
      ldmatrix_x4(qf[kk], smem_u32(tQ + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8));
  }

  for (int ch = 0; ch < n_chunks; ++ch) {
    const int st = ch % ST;
    // chunk ch + ST - 1 goes into the stage that chunk ch - 1 has just left (all warps passed the
    // barrier at the end of the previous iteration)
    if (ch + ST - 1 < n_chunks) issue(ch + ST - 1, (ch + ST - 1) % ST);
    cp_async_commit();
    cp_async_wait<ST - 1>();        // chunk ch is complete; the ST - 1 younger groups may still fly
    __syncthreads();
    float s[CH / 8][4];
#pragma unroll
    for (int nt = 0; nt < CH / 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[nt][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int kt = 0; kt < CH / 16; ++kt) {
        uint32_t bfr[4];
        const __nv_bfloat16* tK = sK + (st * CH + kt * 16) * LD;
        ldmatrix_x4(bfr, smem_u32(tK + ((lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8));
        mma_16816(s[2 * kt], qf[kk], bfr[0], bfr[1]);
        mma_16816(s[2 * kt + 1], qf[kk], bfr[2], bfr[3]);
      }
    }
    const int key0 = kbeg + ch * CH;
    const bool ragged = key0 + CH > kend;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < CH / 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = s[nt][j] * p.scale_log2;
        if (ragged && key0 + nt * 8 + fcol + (j & 1) >= kend) v = -INFINITY;
        s[nt][j] = v;
        mx[j >> 1] = fmaxf(mx[j >> 1], v);
      }
    float corr[2], m_use[2];
    bool moved = false;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      corr[r] = exp2f(m_run[r] - m_use[r]);
      moved = moved || (m_new != m_run[r]);
      m_run[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < CH / 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = exp2f(s[nt][j] - m_use[j >> 1]);
        s[nt][j] = e;
        rs[j >> 1] += e;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + rs[r];
    if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt) {
        o_acc[dt][0] *= corr[0];
        o_acc[dt][1] *= corr[0];
        o_acc[dt][2] *= corr[1];
        o_acc[dt][3] *= corr[1];
      }
    }
#pragma unroll
    for (int kt = 0; kt < CH / 16; ++kt) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
      a[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
      a[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
      a[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
      const __nv_bfloat16* tV = sV + (st * CH + kt * 16) * LD;
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t bfr[4];
        ldmatrix_x4_trans(bfr, smem_u32(tV + (lane & 15) * LD + dp * 16 + (lane >> 4) * 8));
        mma_16816(o_acc[2 * dp], a, bfr[0], bfr[1]);
        mma_16816(o_acc[2 * dp + 1], a, bfr[2], bfr[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  // every warp owns its rows outright: write the partials of the members it covers
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + frow + r * 8;
    const int mem = row / rep;
    const int b = (mem < kGroupMax) ? rows[mem] : -1;
    if (b < 0) continue;
    const int h = hk * rep + row % rep;
    const long long pi = ((long long)b * p.nh + h) * p.slot_total + sp;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
      *reinterpret_cast<float2*>(p.part_o + pi * D + dt * 8 + fcol) = make_float2(o_acc[dt][2 * r], o_acc[dt][2 * r + 1]);
    if ((lane & 3) == 0) {
      p.part_ml[pi * 2] = m_run[r];
      p.part_ml[pi * 2 + 1] = l_run[r];
    }
  }
}

template <int D>
__global__ void paged_decode_merge_kernel(const DecodeParams p, int B) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= (long long)B * p.nh) return;
  const int ns = p.slot_total;
  const float* ml = p.part_ml + gw * ns * 2;
  float m = -INFINITY;
  for (int s = 0; s < ns; ++s) m = fmaxf(m, ml[2 * s]);
  const float mu = (m == -INFINITY) ? 0.f : m;
  float l = 0.f;
  for (int s = 0; s < ns; ++s) l += ml[2 * s + 1] * exp2f(ml[2 * s] - mu);
  const long long b = gw / p.nh;
  const int h = (int)(gw % p.nh);
  for (int d = lane; d < D; d += 32) {
    float o = 0.f;
    for (int s = 0; s < ns; ++s)
      o += p.part_o[(gw * ns + s) * D + d] * exp2f(ml[2 * s] - mu);
    p.out[b * p.out_stride + (long long)h * D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
  }
}

// ---------------------------------------------------------------------------------------------
// Sampler.  One CTA per row.  Distribution = softmax(logits / T) restricted to tokens that
// pass top-k / top-p / min-p expressed as one logit threshold `thresh[b]` computed by the
// filter kernel below (-inf = no filter).  Sampling uses the Gumbel-max trick with a
// counter-based Philox stream keyed by (seed, row key, global vocab index), so the result does
// not depend on how the vocabulary is sharded.  Emits per row a candidate record
//   {max, sumexp(z - max), best perturbed value, best index, z at best}
// which a combine step merges across vocabulary shards.
// `eos_prob[b] >= 0` forces P(eos) to that value (benchmark length control): the EOS token is
// removed from the softmax and re-inserted with logit lse + log(p/(1-p)).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mulhilo(uint32_t a, uint32_t b, uint32_t& hi) {
  const unsigned long long p = (unsigned long long)a * b;
  hi = (uint32_t)(p >> 32);
  return (uint32_t)p;
}
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    uint32_t hi0, hi1;
    const uint32_t lo0 = mulhilo(0xD2511F53u, ctr.x, hi0);
    const uint32_t lo1 = mulhilo(0xCD9E8D57u, ctr.z, hi1);
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return ctr;
}
__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
  // u in (0,1): (bits + 0.5) / 2^32
  const float u = ((float)(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -__logf(-__logf(u));
}

struct SampleRec {
  float m, s, best_val, best_z;
  int best_idx, pad;
};

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

// Grid (row, vocabulary split): every CTA makes ONE pass over its slice of the row (16-byte
// loads), tracking the soft-max statistics and the Gumbel arg-max together; one Philox call
// serves four consecutive vocabulary ids.  The per-split records are merged by the combine kernel
// exactly like records of vocabulary shards on different ranks.
template <typename T>
__global__ void __launch_bounds__(256)
sample_kernel(const T* __restrict__ logits, long long row_stride, int V, int vocab_offset,
              const float* __restrict__ inv_temp, const float* __restrict__ thresh,
              const float* __restrict__ eos_prob, int eos_id,
              const unsigned long long* __restrict__ row_keys, unsigned long long seed,
              SampleRec* __restrict__ rec, int B) {
  __shared__ float red[32];
  __shared__ int redi[32];
  const int b = blockIdx.x;
  const T* row = logits + (long long)b * row_stride;
  const float it = inv_temp[b];
  const bool greedy = it <= 0.f;               // temperature 0 -> argmax
  const float sc = greedy ? 1.f : it;
  const float th = (thresh != nullptr) ? thresh[b] : -INFINITY;
  const float pe = (eos_prob != nullptr) ? eos_prob[b] : -1.f;
  const int eos_local = (pe >= 0.f) ? eos_id - vocab_offset : -1;
  // this CTA's slice [lo, hi) of the row, in multiples of 8 elements
  const int per = ((V + (int)gridDim.y - 1) / (int)gridDim.y + 7) & ~7;
  const int lo = min(V, (int)blockIdx.y * per), hi = min(V, lo + per);
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(row) & 15) == 0);

  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  const unsigned long long rk = row_keys[b];
  float m = -INFINITY, s = 0.f;
  float best = -INFINITY, best_z = 0.f;
  int best_i = -1;
  uint4 rnd = make_uint4(0u, 0u, 0u, 0u);
  uint32_t rnd_group = 0xffffffffu;
  auto visit = [&](int i, float raw) {
    if (i == eos_local) return;
    const float z = raw * sc;
    if (z < th) return;
    if (z > m) {
      s = s * __expf(m - z) + 1.f;
      m = z;
    } else {
      s += __expf(z - m);
    }
    float val = z;
    if (!greedy) {
      const uint32_t gi = (uint32_t)(i + vocab_offset);
      if ((gi >> 2) != rnd_group) {
        rnd_group = gi >> 2;
        rnd = philox4x32_10(make_uint4(rnd_group, 0u, (uint32_t)rk, (uint32_t)(rk >> 32)), key);
      }
      const uint32_t c = gi & 3u;
      val = z + gumbel_from_bits(c == 0 ? rnd.x : (c == 1 ? rnd.y : (c == 2 ? rnd.z : rnd.w)));
    }
    if (val > best || (val == best && i < best_i)) {
      best = val;
      best_z = z;
      best_i = i;
    }
  };
  if (vec_ok) {
    for (int i0 = lo + threadIdx.x * 8; i0 < hi; i0 += blockDim.x * 8) {
      float f[8];
      if (i0 + 8 > hi) {                       // ragged tail of the row: never read past its end
        for (int j = 0; i0 + j < hi; ++j) visit(i0 + j, ld_logit<T>(row, i0 + j));
        continue;
      }
      if (sizeof(T) == 2) {
        unpack8(ld8(reinterpret_cast<const __nv_bfloat16*>(row) + i0), f);
      } else {
        const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(row) + i0);
        const float4 c = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(row) + i0 + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = c.x; f[5] = c.y; f[6] = c.z; f[7] = c.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (i0 + j < hi) visit(i0 + j, f[j]);
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) visit(i, ld_logit<T>(row, i));
  }
  const float bm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - bm);
  const float bs = block_sum(s, red);
  // block arg-max
  float wbest = best;
  int wi = best_i;
  float wz = best_z;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, wbest, o);
    const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
    const float oz = __shfl_xor_sync(0xffffffffu, wz, o);
    if (ov > wbest || (ov == wbest && oi >= 0 && (wi < 0 || oi < wi))) {
      wbest = ov; wi = oi; wz = oz;
    }
  }
  __shared__ float redz[32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { red[wid] = wbest; redi[wid] = wi; redz[wid] = wz; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float fb = -INFINITY, fz = 0.f;
    int fi = -1;
    for (int w = 0; w < nw; ++w) {
      if (red[w] > fb || (red[w] == fb && redi[w] >= 0 && (fi < 0 || redi[w] < fi))) {
        fb = red[w]; fi = redi[w]; fz = redz[w];
      }
    }
    SampleRec r;
    r.m = bm; r.s = bs; r.best_val = fb; r.best_z = fz;
    r.best_idx = (fi >= 0) ? fi + vocab_offset : -1;
    r.pad = 0;
    rec[(long long)blockIdx.y * B + b] = r;
  }
}

// Combine `nshard` candidate records per row into the sampled token and its log-probability.
// With a forced EOS probability the EOS decision is drawn from the same Philox stream
// (counter word 1 = 1) so every shard agrees.
__global__ void sample_combine_kernel(const SampleRec* __restrict__ rec, int nshard, int B,
                                      const float* __restrict__ eos_prob, int eos_id,
                                      const unsigned long long* __restrict__ row_keys,
                                      unsigned long long seed, long long* __restrict__ tokens,
                                      float* __restrict__ logprobs) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float m = -INFINITY;
  for (int s = 0; s < nshard; ++s) m = fmaxf(m, rec[(long long)s * B + b].m);
  float sum = 0.f, best = -INFINITY, bz = 0.f;
  int bi = -1;
  for (int s = 0; s < nshard; ++s) {
    const SampleRec r = rec[(long long)s * B + b];
    if (r.m > -INFINITY) sum += r.s * __expf(r.m - m);
    if (r.best_idx >= 0 && (r.best_val > best || (r.best_val == best && r.best_idx < bi))) {
      best = r.best_val; bz = r.best_z; bi = r.best_idx;
    }
  }
  const float lse = m + __logf(sum);
  float lp = bz - lse;
  const float pe = (eos_prob != nullptr) ? eos_prob[b] : -1.f;
  if (pe >= 0.f) {
    const unsigned long long rk = row_keys[b];
    const uint4 r = philox4x32_10(make_uint4(0u, 1u, (uint32_t)rk, (uint32_t)(rk >> 32)),
                                  make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    const float u = ((float)(r.x >> 8) + 0.5f) * (1.0f / 16777216.0f);
    if (u < pe || bi < 0) {
      bi = eos_id;
      lp = __logf(fmaxf(pe, 1e-30f));
    } else {
      lp += __logf(fmaxf(1.f - pe, 1e-30f));
    }
  }
  tokens[b] = bi;
  logprobs[b] = lp;
}

// top-k / top-p / min-p -> one logit threshold per row (in units of z = logit / T).
// k-th largest by radix-select over the order-preserving integer image of z (4 x 8-bit
// passes), nucleus threshold by bisection on z.  One CTA per row.
__device__ __forceinline__ uint32_t f32_ordered(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float f32_from_ordered(uint32_t o) {
  const uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
  return __uint_as_float(u);
}

template <typename T>
__global__ void __launch_bounds__(1024)
sample_filter_kernel(const T* __restrict__ logits, long long row_stride, int V,
                     const float* __restrict__ inv_temp, const int* __restrict__ top_k,
                     const float* __restrict__ top_p, const float* __restrict__ min_p,
                     float* __restrict__ thresh) {
  __shared__ float red[32];
  __shared__ unsigned int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  const int b = blockIdx.x;
  const T* row = logits + (long long)b * row_stride;
  const float it = inv_temp[b];
  const float sc = it <= 0.f ? 1.f : it;
  float th = -INFINITY;

  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, ld_logit<T>(row, i) * sc);
  m = block_max(m, red);

  const int k = top_k[b];
  if (k > 0 && k < V) {
    uint32_t prefix = 0, mask = 0;
    int remaining = k;
    for (int pass = 3; pass >= 0; --pass) {
      for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
      __syncthreads();
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const uint32_t o = f32_ordered(ld_logit<T>(row, i) * sc);
        if ((o & mask) == prefix) atomicAdd(&hist[(o >> (pass * 8)) & 255u], 1u);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int rem = remaining;
        int bin = 255;
        for (; bin > 0; --bin) {
          if ((int)hist[bin] >= rem) break;
          rem -= (int)hist[bin];
        }
        s_prefix = prefix | ((uint32_t)bin << (pass * 8));
        s_remaining = rem;
      }
      __syncthreads();
      prefix = s_prefix;
      remaining = s_remaining;
      mask |= 255u << (pass * 8);
      __syncthreads();
    }
    th = fmaxf(th, f32_from_ordered(prefix));
  }
  const float mp = min_p[b];
  if (mp > 0.f) th = fmaxf(th, m + __logf(mp));
  const float tp = top_p[b];
  if (tp > 0.f && tp < 1.f) {
    // total mass above the current threshold
    float tot = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float z = ld_logit<T>(row, i) * sc;
      if (z >= th) tot += __expf(z - m);
    }
    tot = block_sum(tot, red);
    // find the largest tau with mass(z >= tau) >= tp * tot  (bisection on z in [m-40, m])
    float lo = fmaxf(th, m - 40.f), hi = m;
    for (int iter = 0; iter < 26; ++iter) {
      const float mid = 0.5f * (lo + hi);
      float acc = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float z = ld_logit<T>(row, i) * sc;
        if (z >= mid) acc += __expf(z - m);
      }
      acc = block_sum(acc, red);
      if (acc >= tp * tot) lo = mid; else hi = mid;
    }
    th = fmaxf(th, lo);
  }
  if (threadIdx.x == 0) thresh[b] = th;
}

}  // namespace msrl

using namespace msrl;

MSRL_API int msrl_kv_cache_write(const void* k, const void* v, const long long* layouts8,
                                 const long long* slots, void* k_cache, void* v_cache,
                                 long long T, int nkv, int D, cudaStream_t st) {
  if (T == 0) return 0;
  if (D % 8 != 0) return (int)cudaErrorInvalidValue;
  HeadLayout Lk{layouts8[0], (int)layouts8[1], (int)layouts8[2], (int)layouts8[3]};
  HeadLayout Lv{layouts8[4], (int)layouts8[5], (int)layouts8[6], (int)layouts8[7]};
  const long long total = T * nkv * (D / 8);
  long long blocks = ceil_div(total, 256);
  if (blocks > 8LL * sm_count()) blocks = 8LL * sm_count();
  kv_cache_write_kernel<<<(unsigned)blocks, 256, 0, st>>>(
      (const __nv_bfloat16*)k, Lk, (const __nv_bfloat16*)v, Lv, slots, (__nv_bfloat16*)k_cache,
      (__nv_bfloat16*)v_cache, T, nkv, D);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_kv_cache_gather(const void* k_cache, const void* v_cache, const int* block_tables,
                                  int max_blocks, const int* token_seq, const int* token_pos,
                                  void* k_out, void* v_out, long long T, int nkv, int D,
                                  int block_size, cudaStream_t st) {
  if (T == 0) return 0;
  const long long total = T * (nkv * D / 8);
  long long blocks = ceil_div(total, 256);
  if (blocks > 8LL * sm_count()) blocks = 8LL * sm_count();
  kv_cache_gather_kernel<<<(unsigned)blocks, 256, 0, st>>>(
      (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_tables, max_blocks,
      token_seq, token_pos, (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, T, nkv, D, block_size);
  MSRL_LAUNCH_CHECK();
}

// Scratch requirement (floats) for a given problem: part_o = B*nh*nsplit*D, part_ml = B*nh*nsplit*2.
MSRL_API int msrl_paged_decode_nsplit(int B, int nkv, int max_ctx) {
  // Three CTAs of this kernel are resident per SM (shared memory); pick the smallest split count
  // that fills the machine and wastes under ~10% of the last wave, keeping >= 256 keys per split.
  const double slots = 3.0 * sm_count();
  int ns = 1;
  while (ns < 32 && (max_ctx + 2 * ns - 1) / (2 * ns) >= 256) {
    const double waves = B * (double)nkv * ns / slots;
    const double eff = waves / ceil(waves);
    if (waves >= 1.0 && eff >= 0.9) break;
    ns *= 2;
  }
  return ns;
}

// tcgen05 form of the shared-prefix pass (decode_prefix_tcgen05.cu)
extern "C" int msrl_paged_prefix_tcgen05(const void* q, const long long* q_layout4, const void* k_cache,
                                         const void* v_cache, long long num_blocks, const int* block_tables,
                                         int max_blocks, const int* group_rows, const int* group_prefix, int n_groups,
                                         float* part_o, float* part_ml, int nh, int nkv, int D, int block_size,
                                         int slot_total, int npre, int* error, cudaStream_t st);

static int launch_paged_decode(const void* q, const long long* q_layout4, const void* k_cache,
                               const void* v_cache, const int* block_tables, int max_blocks,
                               const int* context_lens, void* out, long long out_stride,
                               float* part_o, float* part_ml, int B, int nh, int nkv, int D,
                               int block_size, int nsplit, const int* key_start, const int* group_rows,
                               const int* group_prefix, int n_groups, int npre, cudaStream_t st,
                               long long num_blocks = 0, int prefix_tile = 0, int* error = nullptr) {
  if (B == 0) return 0;
  if (nh % nkv != 0 || nh / nkv > 16 || (D != 64 && D != 128) || nsplit < 1)
    return (int)cudaErrorInvalidValue;
  const bool grouped = n_groups > 0;
  if (grouped && (npre < 1 || key_start == nullptr || group_rows == nullptr || group_prefix == nullptr))
    return (int)cudaErrorInvalidValue;
  DecodeParams p{};
  p.key_start = grouped ? key_start : nullptr;
  p.group_rows = group_rows;
  p.group_prefix = group_prefix;
  p.npre = grouped ? npre : 0;
  p.slot_base = p.npre;
  p.slot_total = p.npre + nsplit;
  p.q = (const __nv_bfloat16*)q;
  p.Lq = HeadLayout{q_layout4[0], (int)q_layout4[1], (int)q_layout4[2], (int)q_layout4[3]};
  p.k_cache = (const __nv_bfloat16*)k_cache;
  p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_tables = block_tables;
  p.context_lens = context_lens;
  p.out = (__nv_bfloat16*)out;
  p.out_stride = out_stride;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.block_shift = -1;
  if (block_size > 0 && (block_size & (block_size - 1)) == 0)
    for (int sft = 0; sft < 31; ++sft)
      if ((1 << sft) == block_size) p.block_shift = sft;
  p.nh = nh;
  p.nkv = nkv;
  p.nsplit = nsplit;
  p.scale_log2 = kLog2eD / sqrtf((float)D);
  const int LD = D + 8;
  size_t smem = (size_t)(16 + 4 * 64) * LD * sizeof(__nv_bfloat16);
  const size_t merge_smem = (size_t)(4 * 16 * D + 2 * 4 * 16) * sizeof(float) + 16 * LD * sizeof(__nv_bfloat16);
  if (merge_smem > smem) smem = merge_smem;
  dim3 grid(B, nkv, nsplit);
  cudaError_t e;
  bool prefix_done = false;
  if (grouped && prefix_tile > 0 && error != nullptr) {
    // the caller rounded every shared prefix down to a multiple of the tensor-core kernel's key tile
    const int rc = msrl_paged_prefix_tcgen05(q, q_layout4, k_cache, v_cache, num_blocks, block_tables, max_blocks,
                                             group_rows, group_prefix, n_groups, part_o, part_ml, nh, nkv, D,
                                             block_size, p.slot_total, npre, error, st);
    if (rc == 0) prefix_done = true;
    else if (rc != (int)cudaErrorNotSupported) return rc;
  }
  if (grouped && !prefix_done) {
    const size_t psmem = (size_t)(64 + 2 * kPrefixStages * kPrefixChunk) * LD * sizeof(__nv_bfloat16);
    dim3 pgrid(n_groups, nkv, npre);
    if (D == 128) {
      e = cudaFuncSetAttribute(paged_decode_prefix_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)psmem);
      if (e != cudaSuccess) return (int)e;
      paged_decode_prefix_kernel<128><<<pgrid, 128, psmem, st>>>(p);
    } else {
      e = cudaFuncSetAttribute(paged_decode_prefix_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)psmem);
      if (e != cudaSuccess) return (int)e;
      paged_decode_prefix_kernel<64><<<pgrid, 128, psmem, st>>>(p);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  if (D == 128) {
    e = cudaFuncSetAttribute(paged_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    paged_decode_kernel<128><<<grid, 128, smem, st>>>(p);
  } else {
    e = cudaFuncSetAttribute(paged_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    paged_decode_kernel<64><<<grid, 128, smem, st>>>(p);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (p.slot_total > 1) {
    const long long warps = (long long)B * nh;
    const unsigned blocks = (unsigned)ceil_div(warps * 32, 128);
    if (D == 128) paged_decode_merge_kernel<128><<<blocks, 128, 0, st>>>(p, B);
    else paged_decode_merge_kernel<64><<<blocks, 128, 0, st>>>(p, B);
  }
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_paged_decode(const void* q, const long long* q_layout4, const void* k_cache,
                               const void* v_cache, const int* block_tables, int max_blocks,
                               const int* context_lens, void* out, long long out_stride,
                               float* part_o, float* part_ml, int B, int nh, int nkv, int D,
                               int block_size, int nsplit, cudaStream_t st) {
  return launch_paged_decode(q, q_layout4, k_cache, v_cache, block_tables, max_blocks, context_lens, out,
                             out_stride, part_o, part_ml, B, nh, nkv, D, block_size, nsplit, nullptr, nullptr,
                             nullptr, 0, 0, st);
}

MSRL_API int msrl_paged_decode_group_max(int nh, int nkv) {
  const int cap = 64 / (nh / nkv);
  return cap < kGroupMax ? cap : kGroupMax;
}

// Grouped decode: every batch row belongs to exactly one group (singletons allowed, prefix 0).
// group_rows [n_groups, 8] lists the members' batch rows (-1 padded, at most
// msrl_paged_decode_group_max members); the members of a group share their first group_prefix[g]
// keys (same tokens, hence the same K/V, read through the first member's block table);
// key_start[b] = prefix of b's group.  prefix_tile > 0 states that every group_prefix is a multiple of
// that many keys (msrl_paged_prefix_tcgen05_tile): the shared pass then runs on the tcgen05 kernel, which
// needs the number of cache blocks and a device status word.  Scratch: part_o B*nh*(npre+nsplit)*D floats, part_ml
// B*nh*(npre+nsplit)*2 floats.
MSRL_API int msrl_paged_decode_grouped(const void* q, const long long* q_layout4, const void* k_cache,
                                       const void* v_cache, const int* block_tables, int max_blocks,
                                       const int* context_lens, const int* key_start, const int* group_rows,
                                       const int* group_prefix, int n_groups, void* out, long long out_stride,
                                       float* part_o, float* part_ml, int B, int nh, int nkv, int D,
                                       int block_size, int nsplit, int npre, long long num_blocks,
                                       int prefix_tile, int* error, cudaStream_t st) {
  if (n_groups < 1) return (int)cudaErrorInvalidValue;
  return launch_paged_decode(q, q_layout4, k_cache, v_cache, block_tables, max_blocks, context_lens, out,
                             out_stride, part_o, part_ml, B, nh, nkv, D, block_size, nsplit, key_start, group_rows,
                             group_prefix, n_groups, npre, st, num_blocks, prefix_tile, error);
}

MSRL_API int msrl_sample_rec_bytes() { return (int)sizeof(SampleRec); }

MSRL_API int msrl_sample_filter(const void* logits, int is_bf16, long long row_stride, int B, int V,
                                const float* inv_temp, const int* top_k, const float* top_p,
                                const float* min_p, float* thresh, cudaStream_t st) {
  if (B == 0) return 0;
  if (is_bf16)
    sample_filter_kernel<__nv_bfloat16><<<B, 1024, 0, st>>>((const __nv_bfloat16*)logits, row_stride,
                                                            V, inv_temp, top_k, top_p, min_p, thresh);
  else
    sample_filter_kernel<float><<<B, 1024, 0, st>>>((const float*)logits, row_stride, V, inv_temp,
                                                    top_k, top_p, min_p, thresh);
  MSRL_LAUNCH_CHECK();
}

MSRL_API int msrl_sample(const void* logits, int is_bf16, long long row_stride, int B, int V,
                         int vocab_offset, const float* inv_temp, const float* thresh,
                         const float* eos_prob, int eos_id, const unsigned long long* row_keys,
                         unsigned long long seed, void* rec, int nsplit, cudaStream_t st) {
  // rec: nsplit * B records laid out [split][row]; merge them with msrl_sample_combine(nshard = nsplit)
  if (B == 0) return 0;
  if (nsplit < 1) return (int)cudaErrorInvalidValue;
  dim3 grid(B, nsplit);
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)logits, row_stride, V,
                                                       vocab_offset, inv_temp, thresh, eos_prob, eos_id,
                                                       row_keys, seed, (SampleRec*)rec, B);
  else
    sample_kernel<float><<<grid, 256, 0, st>>>((const float*)logits, row_stride, V, vocab_offset,
                                               inv_temp, thresh, eos_prob, eos_id, row_keys, seed,
                                               (SampleRec*)rec, B);
  MSRL_LAUNCH_CHECK();
}

// Vocabulary splits per row that fill the machine (about four CTAs per SM, >= 4096 ids per CTA).
MSRL_API int msrl_sample_nsplit(int B, int V) {
  int ns = (4 * sm_count() + B - 1) / (B > 0 ? B : 1);
  const int cap = (V + 4095) / 4096;
  if (ns > cap) ns = cap;
  if (ns > 32) ns = 32;
  return ns < 1 ? 1 : ns;
}

MSRL_API int msrl_sample_combine(const void* rec, int nshard, int B, const float* eos_prob,
                                 int eos_id, const unsigned long long* row_keys,
                                 unsigned long long seed, long long* tokens, float* logprobs,
                                 cudaStream_t st) {
  if (B == 0) return 0;
  sample_combine_kernel<<<(B + 127) / 128, 128, 0, st>>>((const SampleRec*)rec, nshard, B, eos_prob,
                                                         eos_id, row_keys, seed, tokens, logprobs);
  MSRL_LAUNCH_CHECK();
}
