// Selective state-space mixer (Mamba-2 form: scalar decay per head, state S[N, P] per head) over a RAGGED batch:
// sequence s owns tokens [seq_start[s], seq_start[s+1]) of the flat batch, has seq_ctx[s] earlier tokens whose
// effect lives in state slot seq_slot[s], and may bring any number of new tokens (1 = a decode step).
//
//   causal_conv_silu      out[t, c] = silu(bias[c] + sum_j w[c, K-1-j] * in[t-j, c]); inputs before the step come from
//                         the slot's conv tail (the last K-1 inputs), inputs before the sequence are zero
//   conv_tail_update      the slot's conv tail after the step (in place)
//   ssm_scan              dt = softplus(dt_raw + dt_bias); S <- exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + D x
//                         S in fp32 registers for the whole step, read from / written to the slot once
//   gated_group_norm      o = unit_rms_g(y * silu(z)) * w   in `groups` equal parts of the row
// A sequence with seq_ctx == 0 starts from zero: its slot is never read, so slots need no clearing when reused.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ---- seq lookup for a flat token: binary search in seq_start -------------------------------------------------------
__device__ __forceinline__ int find_seq(const int* __restrict__ seq_start, int nseq, int tok) {
  int lo = 0, hi = nseq - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (seq_start[mid] <= tok) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T>
__global__ void causal_conv_silu_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t in_stride,
                                        const T* __restrict__ w, const T* __restrict__ bias,
                                        const T* __restrict__ tail, const int* __restrict__ seq_start,
                                        const int* __restrict__ seq_ctx, const int* __restrict__ seq_slot, int nseq,
                                        int channels, int taps) {
  pdl_prologue();
  const int tok = blockIdx.y;
  const int s = find_seq(seq_start, nseq, tok);
  const int local = tok - seq_start[s], ctx = seq_ctx[s];
  const int64_t slot = seq_slot[s];
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float acc = to_f32(bias[c]);
  for (int j = 0; j < taps; ++j) {                 // j tokens back
    const int i = local - j;
    float v = 0.f;
    if (i >= 0) v = to_f32(in[(int64_t)(tok - j) * in_stride + c]);
    else if (ctx + i >= 0) v = to_f32(tail[(slot * (taps - 1) + (taps - 1 + i)) * channels + c]);
    acc = fmaf(to_f32(w[(int64_t)c * taps + (taps - 1 - j)]), v, acc);
  }
  out[(int64_t)tok * channels + c] = from_f32<T>(silu_f(acc));
}

template <typename T>
__global__ void conv_tail_update_kernel(T* __restrict__ tail, const T* __restrict__ in, int64_t in_stride,
                                        const int* __restrict__ seq_start, const int* __restrict__ seq_ctx,
                                        const int* __restrict__ seq_slot, int channels, int taps) {
  pdl_prologue();
  const int s = blockIdx.y;
  const int start = seq_start[s], len = seq_start[s + 1] - start, ctx = seq_ctx[s];
  const int64_t slot = seq_slot[s];
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels || len <= 0) return;
  const int keep = taps - 1;
  T* mine = tail + slot * keep * channels;
  // entry j holds the input at absolute index ctx + len - keep + j; ascending j only reads entries > j of the old tail
  for (int j = 0; j < keep; ++j) {
    const int a = ctx + len - keep + j;
    T v = from_f32<T>(0.f);
    if (a >= ctx) v = in[(int64_t)(start + a - ctx) * in_stride + c];
    else if (a >= 0) v = mine[(int64_t)(j + len) * channels + c];
    mine[(int64_t)j * channels + c] = v;
  }
}

// One warp = kCols columns p of one head; lane l holds state rows n = l + 32 j.  grid (ceil(P / (4 kCols)), H, nseq).
constexpr int kCols = 4, kScanWarps = 4;

template <typename T, int NJ>
__global__ void __launch_bounds__(kScanWarps * 32) ssm_scan_kernel(
    float* __restrict__ y, float* __restrict__ state, const T* __restrict__ xbc, int64_t xbc_stride,
    const T* __restrict__ dt_raw, int64_t dt_stride, const T* __restrict__ dt_bias, const T* __restrict__ a_log,
    const T* __restrict__ d_skip, const int* __restrict__ seq_start, const int* __restrict__ seq_ctx,
    const int* __restrict__ seq_slot, int heads, int groups, int N, int P) {
  pdl_prologue();
  const int s = blockIdx.z, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int p0 = (blockIdx.x * kScanWarps + warp) * kCols;
  if (p0 >= P) return;
  const int start = seq_start[s], len = seq_start[s + 1] - start, ctx = seq_ctx[s];
  if (len <= 0) return;
  const int64_t slot = seq_slot[s];
  const int g = h / (heads / groups), inner = heads * P;
  const float neg_a = -expf(to_f32(a_log[h])), bias = to_f32(dt_bias[h]), dsk = to_f32(d_skip[h]);
  float* st = state + ((slot * heads + h) * (int64_t)P) * N;            // [P, N], n contiguous
  float S[kCols][NJ];
#pragma unroll
  for (int c = 0; c < kCols; ++c)
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int n = lane + 32 * j;
      S[c][j] = (ctx > 0 && n < N && p0 + c < P) ? st[(int64_t)(p0 + c) * N + n] : 0.f;
    }
  const T* xrow = xbc + (int64_t)start * xbc_stride;
  const int boff = inner + g * N, coff = inner + groups * N + g * N;
  // software pipeline: the next token's operands are in flight while this token's state update runs
  float nb[NJ], nc[NJ], nx[kCols], ndt;
  auto fetch = [&](int t) {
    const T* r = xrow + (int64_t)t * xbc_stride;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int n = lane + 32 * j;
      nb[j] = n < N ? to_f32(r[boff + n]) : 0.f;
      nc[j] = n < N ? to_f32(r[coff + n]) : 0.f;
    }
#pragma unroll
    for (int c = 0; c < kCols; ++c) nx[c] = (p0 + c < P) ? to_f32(r[h * P + p0 + c]) : 0.f;
    ndt = to_f32(dt_raw[(int64_t)(start + t) * dt_stride + h]);
  };
  fetch(0);
  for (int t = 0; t < len; ++t) {
    float b[NJ], cc[NJ], x[kCols];
#pragma unroll
    for (int j = 0; j < NJ; ++j) { b[j] = nb[j]; cc[j] = nc[j]; }
#pragma unroll
    for (int c = 0; c < kCols; ++c) x[c] = nx[c];
    const float dt = softplus_f(ndt + bias);
    if (t + 1 < len) fetch(t + 1);
    const float decay = expf(neg_a * dt);
    float acc[kCols];
#pragma unroll
    for (int c = 0; c < kCols; ++c) {
      const float dx = dt * x[c];
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        S[c][j] = fmaf(decay, S[c][j], dx * b[j]);
        a = fmaf(S[c][j], cc[j], a);
      }
      acc[c] = warp_reduce_sum(a);
    }
    if (lane < kCols && p0 + lane < P) {
      float v = acc[0], xv = x[0];
#pragma unroll
      for (int c = 1; c < kCols; ++c) if (lane == c) { v = acc[c]; xv = x[c]; }
      y[(int64_t)(start + t) * inner + h * P + p0 + lane] = fmaf(dsk, xv, v);
    }
  }
#pragma unroll
  for (int c = 0; c < kCols; ++c)
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int n = lane + 32 * j;
      if (n < N && p0 + c < P) st[(int64_t)(p0 + c) * N + n] = S[c][j];
    }
}

template <typename T>
__global__ void gated_group_norm_kernel(T* __restrict__ o, const float* __restrict__ y, const T* __restrict__ z,
                                        int64_t z_stride, const T* __restrict__ w, int inner, int groups, float eps) {
  pdl_prologue();
  __shared__ float red[32];
  const int64_t t = blockIdx.y;
  const int gs = inner / groups, base = blockIdx.x * gs;
  float ss = 0.f;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float v = y[t * inner + base + i] * silu_f(to_f32(z[t * z_stride + base + i]));
    ss = fmaf(v, v, ss);
  }
  ss = warp_reduce_sum(ss);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = lane < nw ? red[lane] : 0.f;
  tot = warp_reduce_sum(tot);
  const float rr = 1.0f / sqrtf(tot / (float)gs + eps);
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float v = y[t * inner + base + i] * silu_f(to_f32(z[t * z_stride + base + i]));
    o[t * inner + base + i] = from_f32<T>(v * rr * to_f32(w[base + i]));
  }
}

}  // namespace

extern "C" int b2l_causal_conv_silu(void* out, const void* in, int64_t in_row_stride, const void* weight,
                                    const void* bias, void* tail, const void* seq_start, const void* seq_ctx,
                                    const void* seq_slot, int64_t num_seqs, int64_t tokens, int channels, int taps,
                                    int dtype, void* stream) {
  B2L_REQUIRE(out && in && weight && bias && (tail || taps == 1) && seq_start && seq_ctx && seq_slot, "causal_conv_silu: null pointer");
  B2L_REQUIRE(channels > 0 && taps >= 1 && num_seqs >= 0 && tokens >= 0, "causal_conv_silu: bad shape");
  if (tokens == 0 || num_seqs == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 block(128), grid((unsigned)cdiv64(channels, 128), (unsigned)tokens);
  const dim3 grid2((unsigned)cdiv64(channels, 128), (unsigned)num_seqs);
  B2L_DISPATCH_FLOAT(dtype, "causal_conv_silu", {
    b2l_launch(causal_conv_silu_kernel<T>, grid, block, (size_t)0, st, (T*)out, (const T*)in, in_row_stride,
               (const T*)weight, (const T*)bias, (const T*)tail, (const int*)seq_start, (const int*)seq_ctx,
               (const int*)seq_slot, (int)num_seqs, channels, taps);
    b2l_count_launch();
    if (taps > 1)
      b2l_launch(conv_tail_update_kernel<T>, grid2, block, (size_t)0, st, (T*)tail, (const T*)in, in_row_stride,
                 (const int*)seq_start, (const int*)seq_ctx, (const int*)seq_slot, channels, taps);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_ssm_scan(void* y_f32, void* state_f32, const void* xbc, int64_t xbc_row_stride, const void* dt_raw,
                            int64_t dt_row_stride, const void* dt_bias, const void* a_log, const void* d_skip,
                            const void* seq_start, const void* seq_ctx, const void* seq_slot, int64_t num_seqs,
                            int heads, int groups, int state_size, int head_dim, int dtype, void* stream) {
  B2L_REQUIRE(y_f32 && state_f32 && xbc && dt_raw && dt_bias && a_log && d_skip && seq_start && seq_ctx && seq_slot,
              "ssm_scan: null pointer");
  B2L_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0 && state_size > 0 && head_dim > 0,
              "ssm_scan: bad geometry heads=%d groups=%d state=%d head_dim=%d", heads, groups, state_size, head_dim);
  B2L_REQUIRE(state_size <= 256, "ssm_scan: state size %d > 256", state_size);
  if (num_seqs <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 block(kScanWarps * 32), grid((unsigned)cdiv64(head_dim, kScanWarps * kCols), (unsigned)heads,
                                          (unsigned)num_seqs);
  const int nj = (state_size + 31) / 32;
#define B2L_SCAN(NJV)                                                                                                \
  b2l_launch(ssm_scan_kernel<T, NJV>, grid, block, (size_t)0, st, (float*)y_f32, (float*)state_f32, (const T*)xbc,   \
             xbc_row_stride, (const T*)dt_raw, dt_row_stride, (const T*)dt_bias, (const T*)a_log, (const T*)d_skip,  \
             (const int*)seq_start, (const int*)seq_ctx, (const int*)seq_slot, heads, groups, state_size, head_dim)
  B2L_DISPATCH_FLOAT(dtype, "ssm_scan", {
    if (nj <= 1) B2L_SCAN(1);
    else if (nj <= 2) B2L_SCAN(2);
    else if (nj <= 4) B2L_SCAN(4);
    else B2L_SCAN(8);
  });
#undef B2L_SCAN
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_gated_group_norm(void* out, const void* y_f32, const void* z, int64_t z_row_stride,
                                    const void* weight, int64_t rows, int inner, int groups, float eps, int dtype,
                                    void* stream) {
  B2L_REQUIRE(out && y_f32 && z && weight, "gated_group_norm: null pointer");
  B2L_REQUIRE(inner > 0 && groups > 0 && inner % groups == 0, "gated_group_norm: %d columns in %d groups", inner, groups);
  if (rows <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int gs = inner / groups;
  const int threads = gs >= 1024 ? 256 : (gs >= 256 ? 128 : (gs >= 64 ? 64 : 32));
  B2L_DISPATCH_FLOAT(dtype, "gated_group_norm", {
    b2l_launch(gated_group_norm_kernel<T>, dim3((unsigned)groups, (unsigned)rows), dim3(threads), (size_t)0, st, (T*)out,
               (const float*)y_f32, (const T*)z, z_row_stride, (const T*)weight, inner, groups, eps);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
