// A 64 x 64 output tile of C = A B^T on tensor cores (bfloat16 operands, fp32 sums), shared by the
// grouped products of the routed experts and the product batched over heads.  Four warps of 32 rows x
// 32 columns each (thread's element [m][mt][nt][2i+j]: row (warp/2)*32 + mt*16 + lane/4 + 8i, column
// (warp%2)*32 + nt*8 + 2*(lane%4) + j); operands come through a three-stage cp.async ring in shared memory (rows of 32 k-values,
// padded so that ldmatrix finds eight rows in eight different banks).  Rows of A are found through
// an index (gathered rows; a negative index is a row of zeros); rows of B are K elements apart.
#pragma once
#include "common.cuh"

namespace leone {

constexpr int TM = 64, TN = 64, TK = 32, TSTAGES = 3, TPITCH = TK * 2 + 16;

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// a_rows: row r of the tile reads a_base + a_index[r] * lda (a_index < 0: a row of zeros).
template <int NB>
__device__ __forceinline__ void grouped_mainloop(unsigned char* smem, const __nv_bfloat16* a_base, const int* a_index_s,
                                                 int lda, const __nv_bfloat16* b0_base, const __nv_bfloat16* b1_base,
                                                 int n_valid, int K, float (*acc)[2][4][4], int ldb = 0) {
  if (ldb == 0) ldb = K;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kStageBytes = (TM + NB * TN) * TPITCH;
  const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem);
  const int kblocks = (K + TK - 1) / TK;
  auto load = [&](int kb, int stage) {
    const uint32_t st = base + stage * kStageBytes;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * 128, row = c >> 2, kc = c & 3;
      const int k = kb * TK + kc * 8;
      const int ai = a_index_s[row];
      const bool av = ai >= 0 && k < K;
      cp_async16_zfill(st + row * TPITCH + kc * 16, av ? (const void*)(a_base + (size_t)ai * lda + k) : (const void*)a_base, av);
      const bool bv = row < n_valid && k < K;
      cp_async16_zfill(st + (TM + row) * TPITCH + kc * 16, bv ? (const void*)(b0_base + (size_t)row * ldb + k) : (const void*)b0_base, bv);
      if (NB == 2)
        cp_async16_zfill(st + (TM + TN + row) * TPITCH + kc * 16,
                         bv ? (const void*)(b1_base + (size_t)row * ldb + k) : (const void*)b1_base, bv);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  for (int s = 0; s < TSTAGES - 1; ++s) {
    if (s < kblocks) load(s, s);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // the warps are 2 x 2, each with 32 rows x 32 columns (of every B matrix): two A fragments and
  // two B fragment pairs a matrix serve eight MMAs a matrix
  const int mi = lane >> 3, wm = warp >> 1, wn = warp & 1;
  for (int kb = 0; kb < kblocks; ++kb) {
    asm volatile("cp.async.wait_group %0;" ::"n"(TSTAGES - 2) : "memory");
    __syncthreads();
    if (kb + TSTAGES - 1 < kblocks) load(kb + TSTAGES - 1, (kb + TSTAGES - 1) % TSTAGES);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const uint32_t st = base + (kb % TSTAGES) * kStageBytes;
#pragma unroll
    for (int ks = 0; ks < TK / 16; ++ks) {
      uint32_t a[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        ldsm4(st + (wm * 32 + mt * 16 + (lane & 15)) * TPITCH + (lane >> 4) * 16 + ks * 32, a[mt][0], a[mt][1], a[mt][2],
              a[mt][3]);
#pragma unroll
      for (int m = 0; m < NB; ++m) {
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm4(st + (TM + m * TN + wn * 32 + np * 16 + (lane & 7) + (mi >> 1) * 8) * TPITCH + (mi & 1) * 16 + ks * 32, b0,
                b1, b2, b3);
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            mma16816(acc[m][mt][2 * np], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
            mma16816(acc[m][mt][2 * np + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

}  // namespace leone
