// Warp-level tensor-core building blocks shared by the attention kernels:
// ldmatrix / mma.sync m16n8k16 (bf16 in, fp32 accumulate), cp.async tile loads.
#pragma once
#include "common.cuh"

namespace msrl {

// Addressing of heads inside fused QKV rows (see elementwise.cu for the derivation).
struct HeadLayout {
  long long stride_t;
  int group_stride;
  int heads_per_group;
  int head_stride;
};
__device__ __forceinline__ long long head_offset(const HeadLayout& L, long long t, int h) {
  return t * L.stride_t + (long long)(h / L.heads_per_group) * L.group_stride +
         (long long)(h % L.heads_per_group) * L.head_stride;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// d += a(16x16, row) * b(16x8, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// 16-byte async copy global -> shared; when !pred the destination is zero-filled.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  const uint32_t s = smem_u32(smem);
  const int bytes = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Load ROWS x D bf16 (D multiple of 8) rows [row0, row0+ROWS) of head `h` into smem with row
// stride LD; rows >= nrows are zero-filled. `tok0` is the first token of the sequence.
template <int ROWS, int D, int LD, int THREADS>
__device__ __forceinline__ void load_tile_async(__nv_bfloat16* smem, const __nv_bfloat16* base,
                                                const HeadLayout& L, int h, long long tok0,
                                                int row0, int nrows) {
  constexpr int VEC_PER_ROW = D / 8;
  constexpr int TOTAL = ROWS * VEC_PER_ROW;
  for (int i = threadIdx.x; i < TOTAL; i += THREADS) {
    const int r = i / VEC_PER_ROW, c = i % VEC_PER_ROW;
    const bool ok = (row0 + r) < nrows;
    const long long t = tok0 + (ok ? (row0 + r) : 0);
    const __nv_bfloat16* src = base + head_offset(L, t, h) + c * 8;
    cp_async16(smem + r * LD + c * 8, src, ok);
  }
}

}  // namespace msrl
