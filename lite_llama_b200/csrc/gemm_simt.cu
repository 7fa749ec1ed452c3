// y[M, N] = x[M, K] . w[N, K]^T on the CUDA cores, fp32 accumulation, any shape and alignment.
//
// Two users: (1) true 32-bit models (B2L_F32): the tensor cores have no exact fp32 mode, so the exact path runs here;
// (2) 16-bit shapes the tcgen05 GEMM refuses (K not a multiple of 8 elements: the TMA 16-byte rule).
// Every output element is one k-ascending fp32 sum whatever M is, so a token's result does not depend on
// what else is in the batch.
#include "common.cuh"

namespace {

constexpr int kBM = 64, kBN = 64, kBK = 16, kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads) gemm_simt_kernel(T* __restrict__ y, const T* __restrict__ x,
                                                             const T* __restrict__ w, const T* __restrict__ bias,
                                                             int64_t m, int64_t n, int64_t k, int64_t xs, int64_t ws,
                                                             int64_t ys) {
  pdl_prologue();
  __shared__ float xt[kBK][kBM + 4];
  __shared__ float wt[kBK][kBN + 4];
  const int tid = threadIdx.x;
  const int64_t m0 = (int64_t)blockIdx.y * kBM, n0 = (int64_t)blockIdx.x * kBN;
  const int lr = tid >> 2, lk = (tid & 3) * 4;          // loader: row of the tile, first of 4 k values
  const int tr = (tid >> 4) * 4, tc = (tid & 15) * 4;   // compute: 4 x 4 outputs
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < k; k0 += kBK) {
    const int64_t xr = m0 + lr, wr = n0 + lr;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t kk = k0 + lk + i;
      xt[lk + i][lr] = (xr < m && kk < k) ? to_f32(x[xr * xs + kk]) : 0.f;
      wt[lk + i][lr] = (wr < n && kk < k) ? to_f32(w[wr * ws + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kBK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = xt[kk][tr + i]; b[i] = wt[kk][tc + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = m0 + tr + i;
    if (r >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t c = n0 + tc + j;
      if (c < n) y[r * ys + c] = from_f32<T>(acc[i][j] + (bias ? to_f32(bias[c]) : 0.f));
    }
  }
}

}  // namespace

extern "C" int b2l_gemm_simt(void* y, const void* x, const void* w, const void* bias, int64_t m, int64_t n, int64_t k,
                             int64_t x_row_stride, int64_t w_row_stride, int64_t y_row_stride, int dtype,
                             void* stream) {
  B2L_REQUIRE(y && x && w, "gemm_simt: null pointer");
  B2L_REQUIRE(m >= 0 && n > 0 && k > 0, "gemm_simt: bad shape m=%lld n=%lld k=%lld", (long long)m, (long long)n,
              (long long)k);
  if (m == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)cdiv64(n, kBN), (unsigned)cdiv64(m, kBM));
  B2L_DISPATCH_FLOAT(dtype, "gemm_simt", {
    b2l_launch(gemm_simt_kernel<T>, grid, dim3(kThreads), (size_t)0, st, (T*)y, (const T*)x, (const T*)w,
               (const T*)bias, m, n, k, x_row_stride, w_row_stride, y_row_stride);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
