// Small kernels shared by several parts: two RMS norms of the same rows in one pass, the squared
// ReLU, and a product batched over heads.
#include "common.cuh"
#include "mma_tile.cuh"

namespace leone {

// out_a = x * r * w_a, out_b = x * r * w_b with r = 1/sqrt(mean(x^2) + eps): both norms of a layer
// whose branches read the same residual rows share the row's sum of squares.
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
rms_norm_pair_kernel(const float* __restrict__ x, const TW* __restrict__ w_a, const TW* __restrict__ w_b,
                     T* __restrict__ out_a, T* __restrict__ out_b, int width, float eps) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(x[base + c], x[base + c], ss);
  ss = block_sum(ss, scratch);
  const float r = 1.f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = x[base + c] * r;
    out_a[base + c] = from_float<T>(v * to_float<TW>(w_a[c]));
    out_b[base + c] = from_float<T>(v * to_float<TW>(w_b[c]));
  }
}

template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ x, long long n) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = fmaxf(to_float<T>(x[i]), 0.f);
    x[i] = from_float<T>(v * v);
  }
}

// C_b[M, N] = A_b[M, K] W_b[N, K]^T for b < batch, fp32 accumulation with k ascending; the three
// operands of batch b start b * (their batch stride) elements after those of batch 0.
constexpr int BM = 64, BN = 64, BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_batched_kernel(const T* __restrict__ A, const T* __restrict__ W, T* __restrict__ C, int M, int N, int K,
                    int lda, int ldw, int ldc, long long a_bs, long long w_bs, long long c_bs) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  A += (size_t)blockIdx.z * a_bs;
  W += (size_t)blockIdx.z * w_bs;
  C += (size_t)blockIdx.z * c_bs;
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int ty = tid >> 4, tx = tid & 15;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const T* a_row = A + (size_t)(m0 + lr) * lda;
  const T* w_row = W + (size_t)(n0 + lr) * ldw;
  const bool a_ok = m0 + lr < M, w_ok = n0 + lr < N;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_ok && k < K) ? to_float<T>(a_row[k]) : 0.f;
      Ws[lk + i][lr] = (w_ok && k < K) ? to_float<T>(w_row[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = from_float<T>(acc[i][j]);
    }
  }
}

// The same product on tensor cores (bfloat16): a block owns 64 rows x 64 columns of one batch.
__global__ void __launch_bounds__(128)
gemm_batched_mma_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                        __nv_bfloat16* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc, long long a_bs,
                        long long w_bs, long long c_bs) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_m[];
  __shared__ int a_index[TM];
  A += (size_t)blockIdx.z * a_bs;
  W += (size_t)blockIdx.z * w_bs;
  C += (size_t)blockIdx.z * c_bs;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  for (int r = threadIdx.x; r < TM; r += 128) a_index[r] = m0 + r < M ? m0 + r : -1;
  __syncthreads();
  float acc[1][2][4][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[0][mt][n][i] = 0.f;
  grouped_mainloop<1>(smem_m, A, a_index, lda, W + (size_t)n0 * ldw, nullptr, min(TN, N - n0), K, acc, ldw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int wm = warp >> 1, wn = warp & 1;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int m = m0 + wm * 32 + mt * 16 + g + 8 * i;
      if (m >= M) continue;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = n0 + wn * 32 + n * 8 + 2 * tq;
        if (col >= N) continue;
        *reinterpret_cast<__nv_bfloat162*>(C + (size_t)m * ldc + col) =
            __floats2bfloat162_rn(acc[0][mt][n][2 * i], acc[0][mt][n][2 * i + 1]);
      }
    }
}

}  // namespace leone

using namespace leone;

extern "C" void leone_mixers_set_pdl(int enabled) { pdl_flag() = enabled ? 1 : 0; }

extern "C" int leone_rms_norm_pair(const float* x, const void* w_a, const void* w_b, int w_dtype, void* out_a,
                                   void* out_b, int out_dtype, int n, int width, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0) return kRefusedSize;
#define NP(T, TW)                                                                                            \
  launch_kernel(rms_norm_pair_kernel<T, TW>, dim3(n), dim3(256), 0, stream, x, (const TW*)w_a, (const TW*)w_b, (T*)out_a, (T*)out_b, \
                                                     width, eps)
  if (out_dtype == 0 && w_dtype == 0) NP(float, float);
  else if (out_dtype == 1 && w_dtype == 0) NP(__nv_bfloat16, float);
  else if (out_dtype == 1 && w_dtype == 1) NP(__nv_bfloat16, __nv_bfloat16);
  else if (out_dtype == 0 && w_dtype == 1) NP(float, __nv_bfloat16);
  else return kRefusedDtype;
#undef NP
  return launch_result();
}

extern "C" int leone_relu_squared(int dtype, void* x, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long want = (n + 255) / 256;
  const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == 0) launch_kernel(relu_squared_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, n);
  else if (dtype == 1) launch_kernel(relu_squared_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, n);
  else return kRefusedDtype;
  return launch_result();
}

extern "C" int leone_gemm_batched(int dtype, const void* a, const void* w, void* c, int m, int n, int k, int lda,
                                  int ldw, int ldc, long long a_bs, long long w_bs, long long c_bs, int batch,
                                  cudaStream_t stream) {
  if (m <= 0 || n <= 0 || batch <= 0) return 0;
  if (k <= 0 || lda < k || ldw < k || ldc < n || batch > 65535) return kRefusedSize;
  const dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM, batch);
  if (grid.y > 65535) return kRefusedSize;
  // bfloat16 with 16-byte aligned rows: tensor cores
  if (dtype == 1 && k % 8 == 0 && n % 2 == 0 && lda % 8 == 0 && ldw % 8 == 0 && ldc % 2 == 0 && a_bs % 8 == 0 &&
      w_bs % 8 == 0 && c_bs % 2 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)c % 4) == 0) {
    const dim3 tgrid((n + TN - 1) / TN, (m + TM - 1) / TM, batch);
    if (tgrid.y > 65535) return kRefusedSize;
    const size_t smem = (size_t)TSTAGES * (TM + TN) * TPITCH;
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(gemm_batched_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      configured = true;
    }
    launch_kernel(gemm_batched_mma_kernel, tgrid, dim3(128), smem, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                                                          (__nv_bfloat16*)c, m, n, k, lda, ldw, ldc, a_bs, w_bs, c_bs);
    return launch_result();
  }
  if (dtype == 0)
    launch_kernel(gemm_batched_kernel<float>, grid, dim3(256), 0, stream, (const float*)a, (const float*)w, (float*)c, m, n, k, lda,
                                                         ldw, ldc, a_bs, w_bs, c_bs);
  else if (dtype == 1)
    launch_kernel(gemm_batched_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                                                                 (__nv_bfloat16*)c, m, n, k, lda, ldw, ldc, a_bs,
                                                                 w_bs, c_bs);
  else
    return kRefusedDtype;
  return launch_result();
}
