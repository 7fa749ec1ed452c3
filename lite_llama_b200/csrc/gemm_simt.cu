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

// ---- per-head batched product: y[t, h, :] = W[h] . x[t, h, :]  (optionally * sigmoid(gate[t, h])) ------------------
// Same tile and the same k-ascending sums as above, blockIdx.z = head.  x / y rows hold the heads side by side
// (head strides in elements), W is [heads, N, K] dense.
template <typename T>
__global__ void __launch_bounds__(kThreads) head_linear_kernel(T* __restrict__ y, const T* __restrict__ x,
                                                               const T* __restrict__ w, const T* __restrict__ gate,
                                                               int64_t m, int64_t n, int64_t k, int64_t xs, int64_t xh,
                                                               int64_t ys, int64_t yh, int64_t gs) {
  pdl_prologue();
  __shared__ float xt[kBK][kBM + 4];
  __shared__ float wt[kBK][kBN + 4];
  const int tid = threadIdx.x, h = blockIdx.z;
  x += (int64_t)h * xh;
  y += (int64_t)h * yh;
  w += (int64_t)h * n * k;
  const int64_t m0 = (int64_t)blockIdx.y * kBM, n0 = (int64_t)blockIdx.x * kBN;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int tr = (tid >> 4) * 4, tc = (tid & 15) * 4;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < k; k0 += kBK) {
    const int64_t xr = m0 + lr, wr = n0 + lr;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t kk = k0 + lk + i;
      xt[lk + i][lr] = (xr < m && kk < k) ? to_f32(x[xr * xs + kk]) : 0.f;
      wt[lk + i][lr] = (wr < n && kk < k) ? to_f32(w[wr * k + kk]) : 0.f;
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
    const float g = gate ? 1.0f / (1.0f + expf(-to_f32(gate[r * gs + h]))) : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t c = n0 + tc + j;
      if (c < n) y[r * ys + c] = from_f32<T>(acc[i][j] * g);
    }
  }
}

// ---- grouped (per-expert) product over slots sorted by expert ----------------------------------------------------
// sorted_ids / expert_ids / num_post are moe_align_block_size's outputs for block_size = kGM: row block b holds up to
// kGM slots of expert expert_ids[b] (padding = a slot id >= num_valid_slots).  Slot s reads activation row s / top_k
// and writes output row s:   c[s, :] = act(W[e] . a[s / top_k, :]) * (slot_weight[s] if given, multiplied in fp32).
constexpr int kGM = 32;

__device__ __forceinline__ float gelu_erf_f(float v) { return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f)); }

template <typename T>
__global__ void __launch_bounds__(kThreads) moe_gemm_simt_kernel(T* __restrict__ c, const T* __restrict__ a,
                                                                 const T* __restrict__ w,
                                                                 const float* __restrict__ slot_weight,
                                                                 const int* __restrict__ sorted_ids,
                                                                 const int* __restrict__ expert_ids,
                                                                 const int* __restrict__ num_post, int64_t num_valid,
                                                                 int top_k, int64_t n, int64_t k, int64_t as, int64_t cs,
                                                                 int act) {
  pdl_prologue();
  __shared__ float xt[kBK][kGM + 4];
  __shared__ float wt[kBK][kBN + 4];
  __shared__ int slot_of[kGM];
  const int tid = threadIdx.x;
  const int64_t b0 = (int64_t)blockIdx.y * kGM;
  if (b0 >= num_post[0]) return;
  const int64_t n0 = (int64_t)blockIdx.x * kBN;
  const T* we = w + (int64_t)expert_ids[blockIdx.y] * n * k;
  if (tid < kGM) slot_of[tid] = sorted_ids[b0 + tid];
  __syncthreads();
  const int xr = tid >> 3, xk = (tid & 7) * 2;            // x loader: 32 rows x 16 k, two values per thread
  const int lr = tid >> 2, lk = (tid & 3) * 4;            // w loader: 64 rows x 16 k, four values per thread
  const int tr = (tid >> 4) * 2, tc = (tid & 15) * 4;     // compute: 2 x 4 outputs
  const int64_t xslot = slot_of[xr];
  const T* xrow = xslot < num_valid ? a + (xslot / top_k) * as : nullptr;
  float acc[2][4] = {};
  for (int64_t k0 = 0; k0 < k; k0 += kBK) {
    const int64_t wr = n0 + lr;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int64_t kk = k0 + xk + i;
      xt[xk + i][xr] = (xrow && kk < k) ? to_f32(xrow[kk]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t kk = k0 + lk + i;
      wt[lk + i][lr] = (wr < n && kk < k) ? to_f32(we[wr * k + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kBK; ++kk) {
      float av[2], bv[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) av[i] = xt[kk][tr + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = wt[kk][tc + j];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int64_t slot = slot_of[tr + i];
    if (slot >= num_valid) continue;
    const float g = slot_weight ? slot_weight[slot] : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t col = n0 + tc + j;
      if (col >= n) continue;
      float v = acc[i][j];
      if (act == 1) v = gelu_erf_f(v);
      c[slot * cs + col] = from_f32<T>(v * g);
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

/* y[t, h, :] = W[h] . x[t, h, :] for W [heads, n, k]; gate (nullable) [m, >= heads]: y *= sigmoid(gate[t, h]). */
extern "C" int b2l_head_linear(void* y, int64_t y_row_stride, int64_t y_head_stride, const void* x,
                               int64_t x_row_stride, int64_t x_head_stride, const void* w, const void* gate,
                               int64_t gate_row_stride, int64_t m, int heads, int64_t n, int64_t k, int dtype,
                               void* stream) {
  B2L_REQUIRE(y && x && w, "head_linear: null pointer");
  B2L_REQUIRE(m >= 0 && heads > 0 && heads <= 65535 && n > 0 && k > 0, "head_linear: bad shape");
  if (m == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)cdiv64(n, kBN), (unsigned)cdiv64(m, kBM), (unsigned)heads);
  B2L_DISPATCH_FLOAT(dtype, "head_linear", {
    b2l_launch(head_linear_kernel<T>, grid, dim3(kThreads), (size_t)0, st, (T*)y, (const T*)x, (const T*)w,
               (const T*)gate, m, n, k, x_row_stride, x_head_stride, y_row_stride, y_head_stride, gate_row_stride);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_moe_gemm_simt_block(void) { return kGM; }

/* Grouped product over expert-sorted slots (moe_align_block_size with block_size = b2l_moe_gemm_simt_block()):
 * c[s, :] = act(W[expert(s)] . a[s / top_k, :]) * slot_weight_f32[s];  act: 0 none, 1 exact gelu;  W [experts, n, k]. */
extern "C" int b2l_moe_gemm_simt(void* c, const void* a, const void* w, const void* slot_weight_f32,
                                 const void* sorted_token_ids, const void* expert_ids,
                                 const void* num_tokens_post_padded, int64_t em, int64_t num_valid_slots, int top_k,
                                 int64_t n, int64_t k, int64_t a_row_stride, int64_t c_row_stride, int act, int dtype,
                                 void* stream) {
  B2L_REQUIRE(c && a && w && sorted_token_ids && expert_ids && num_tokens_post_padded, "moe_gemm_simt: null pointer");
  B2L_REQUIRE(top_k >= 1 && n > 0 && k > 0 && em >= 0 && (act == 0 || act == 1), "moe_gemm_simt: bad shape");
  if (em == 0 || num_valid_slots == 0) return B2L_OK;
  B2L_REQUIRE(cdiv64(em, kGM) <= 65535, "moe_gemm_simt: %lld row blocks", (long long)cdiv64(em, kGM));
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)cdiv64(n, kBN), (unsigned)cdiv64(em, kGM));   // blocks at or past num_post leave at once
  B2L_DISPATCH_FLOAT(dtype, "moe_gemm_simt", {
    b2l_launch(moe_gemm_simt_kernel<T>, grid, dim3(kThreads), (size_t)0, st, (T*)c, (const T*)a, (const T*)w,
               (const float*)slot_weight_f32, (const int*)sorted_token_ids, (const int*)expert_ids,
               (const int*)num_tokens_post_padded, num_valid_slots, top_k, n, k, a_row_stride, c_row_stride, act);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
