// Tensor-core (mma.sync m16n8k16, fp32 accumulators) versions of the two row-mapped products of csrc/gemm_simt.cu for
// 16-bit activations:
//   * per-head product   y[t, h, :] = W[h] . x[t, h, :]          (* sigmoid(gate[t, h]))
//   * grouped product    c[s, :] = act(W[expert(s)] . a[s / top_k, :]) * slot_weight[s]     over expert-sorted slots
// One kernel, two row maps: a CTA owns BM rows (16, 64 or 128) x 64 output columns of one head / one expert block, its
// four warps hold 16-column slices (BM = 16), 16-row slices (BM = 64) or 32-row slices (BM = 128).  The rows' inputs are
// gathered and the weight tile streamed with 16-byte asynchronous copies into a padded shared-memory ring of 32 k
// values per stage: four stages for the 16-row tile (decode: the weights are what streams, so as many bytes as
// possible are in flight), three for 64 rows, two for 128.  Every output element is one k-ascending tensor-core sum, so
// a row's result does not depend on which other rows share its tile.  Needs k a multiple of 8 and 16-byte aligned rows
// (the callers fall back to the CUDA-core kernels otherwise); W is [heads or experts, n, k] dense.
#include "common.cuh"

namespace {

constexpr int kBN = 64, kBK = 32, kPitch = kBK + 8;          // elements; 80-byte rows: ldmatrix without bank conflicts

struct RowsArgs {
  const void* x; const void* w; void* y;
  int64_t n, k, xs, ys;
  // per-head map
  int64_t m, xh, yh, gs; const void* gate;
  // grouped map
  const float* slot_weight; const int* sorted_ids; const int* expert_ids; const int* num_post;
  int64_t num_valid; int top_k, act;
  int out_f32;                 // per-head map only: y is fp32 (router logits: 16-bit operands, 32-bit sums kept as they are)
};

__device__ __forceinline__ void cp16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float gelu_erf_m(float v) { return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f)); }

template <typename T, int BM, int GROUPED>
__global__ void __launch_bounds__(128) rows_gemm_mma_kernel(RowsArgs a) {
  pdl_prologue();
  constexpr int WM = BM >= 64 ? 4 : 1, WN = 4 / WM;          // warps along rows / columns
  constexpr int MT = BM / (16 * WM);                         // 16-row tiles per warp
  constexpr int NT = kBN / WN / 8;                           // 8-column tiles per warp
  constexpr int ST = BM == 16 ? 4 : (BM == 64 ? 3 : 2);      // ring stages
  __shared__ __align__(16) T As[ST][BM][kPitch];
  __shared__ __align__(16) T Ws[ST][kBN][kPitch];
  __shared__ const T* arow[BM];
  __shared__ void* crow[BM];
  __shared__ float mult[BM];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t n0 = (int64_t)blockIdx.x * kBN;
  const T* wb;
  if (GROUPED) {
    const int64_t b0 = (int64_t)blockIdx.y * BM;
    if (b0 >= a.num_post[0]) return;
    wb = (const T*)a.w + (int64_t)a.expert_ids[blockIdx.y] * a.n * a.k;
    if (tid < BM) {
      const int64_t slot = a.sorted_ids[b0 + tid];
      const bool ok = slot < a.num_valid;
      arow[tid] = ok ? (const T*)a.x + (slot / a.top_k) * a.xs : nullptr;
      crow[tid] = ok ? (void*)((T*)a.y + slot * a.ys) : nullptr;
      mult[tid] = (ok && a.slot_weight) ? a.slot_weight[slot] : 1.0f;
    }
  } else {
    const int h = blockIdx.z;
    wb = (const T*)a.w + (int64_t)h * a.n * a.k;
    if (tid < BM) {
      const int64_t row = (int64_t)blockIdx.y * BM + tid;
      const bool ok = row < a.m;
      arow[tid] = ok ? (const T*)a.x + row * a.xs + h * a.xh : nullptr;
      const int64_t off = row * a.ys + h * a.yh;
      crow[tid] = ok ? (a.out_f32 ? (void*)((float*)a.y + off) : (void*)((T*)a.y + off)) : nullptr;
      mult[tid] = (ok && a.gate) ? 1.0f / (1.0f + expf(-to_f32(((const T*)a.gate)[row * a.gs + h]))) : 1.0f;
    }
  }
  __syncthreads();
  auto issue = [&](int64_t k0, int st) {
    for (int i = tid; i < BM * (kBK / 8); i += 128) {
      const int r = i / (kBK / 8), c = (i % (kBK / 8)) * 8;
      const T* src = arow[r];
      if (src && k0 + c < a.k) cp16(smem_u32(&As[st][r][c]), src + k0 + c);
      else *reinterpret_cast<uint4*>(&As[st][r][c]) = make_uint4(0u, 0u, 0u, 0u);
    }
    for (int i = tid; i < kBN * (kBK / 8); i += 128) {
      const int r = i / (kBK / 8), c = (i % (kBK / 8)) * 8;
      if (n0 + r < a.n && k0 + c < a.k) cp16(smem_u32(&Ws[st][r][c]), wb + (n0 + r) * a.k + k0 + c);
      else *reinterpret_cast<uint4*>(&Ws[st][r][c]) = make_uint4(0u, 0u, 0u, 0u);
    }
    cp_commit();
  };
  const int wm = warp % WM, wn = warp / WM;
  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
  const int64_t kt_count = (a.k + kBK - 1) / kBK;
  // one copy group per k tile, committed even when it is empty, so that "all but the newest ST - 2 groups have
  // landed" always means "tile kt has landed"
#pragma unroll
  for (int s = 0; s < ST - 1; ++s) {
    if (s < kt_count) issue((int64_t)s * kBK, s); else cp_commit();
  }
  for (int64_t kt = 0; kt < kt_count; ++kt) {
    const int st = (int)(kt % ST);
    cp_wait<ST - 2>();
    __syncthreads();                                         // tile kt is visible; every warp is done with tile kt - 1,
    if (kt + ST - 1 < kt_count) issue((kt + ST - 1) * kBK, (int)((kt + ST - 1) % ST));      // whose stage is refilled
    else cp_commit();
#pragma unroll
    for (int kk = 0; kk < kBK / 16; ++kk) {
      uint32_t af[MT][4];
#pragma unroll
      for (int i = 0; i < MT; ++i)
        ldmatrix_x4(af[i], smem_u32(&As[st][(wm * MT + i) * 16 + (lane & 15)][kk * 16 + (lane >> 4) * 8]));
      const int mj = lane >> 3, r = lane & 7;
#pragma unroll
      for (int jp = 0; jp < NT / 2; ++jp) {
        uint32_t bf[4];
        ldmatrix_x4(bf, smem_u32(&Ws[st][wn * (NT * 8) + jp * 16 + (mj >> 1) * 8 + r][kk * 16 + (mj & 1) * 8]));
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          mma_m16n8k16<T>(acc[i][2 * jp], af[i], bf[0], bf[1]);
          mma_m16n8k16<T>(acc[i][2 * jp + 1], af[i], bf[2], bf[3]);
        }
      }
    }
  }
  const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int mh = 0; mh < MT * 2; ++mh) {
    const int mi = mh >> 1, half = mh & 1;
    const int r = (wm * MT + mi) * 16 + gq + half * 8;
    if (!crow[r]) continue;
    const float g = mult[r];
    if (!GROUPED && a.out_f32) {
      float* d32 = (float*)crow[r];
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int64_t col = n0 + wn * (NT * 8) + j * 8 + 2 * tq;
        if (col < a.n) d32[col] = acc[mi][j][half * 2] * g;
        if (col + 1 < a.n) d32[col + 1] = acc[mi][j][half * 2 + 1] * g;
      }
      continue;
    }
    T* dst = (T*)crow[r];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int64_t col = n0 + wn * (NT * 8) + j * 8 + 2 * tq;
      float v0 = acc[mi][j][half * 2], v1 = acc[mi][j][half * 2 + 1];
      if (GROUPED && a.act == 1) { v0 = gelu_erf_m(v0); v1 = gelu_erf_m(v1); }
      v0 *= g; v1 *= g;
      if (col + 1 < a.n && (((uintptr_t)(dst + col)) & 3) == 0) {
        *reinterpret_cast<uint32_t*>(dst + col) = pack2<T>(v0, v1);
      } else {
        if (col < a.n) dst[col] = from_f32<T>(v0);
        if (col + 1 < a.n) dst[col + 1] = from_f32<T>(v1);
      }
    }
  }
}

template <typename T, int GROUPED>
void launch_rows(const RowsArgs& a, int bm, dim3 grid, cudaStream_t st) {
  if (bm == 16) b2l_launch(rows_gemm_mma_kernel<T, 16, GROUPED>, grid, dim3(128), (size_t)0, st, a);
  else if (bm == 64) b2l_launch(rows_gemm_mma_kernel<T, 64, GROUPED>, grid, dim3(128), (size_t)0, st, a);
  else b2l_launch(rows_gemm_mma_kernel<T, 128, GROUPED>, grid, dim3(128), (size_t)0, st, a);
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// Rows per CTA of the per-head map: the largest tile that still gives every SM a CTA (a product with few output
// columns, the router's for instance, has few column tiles and needs many row tiles to fill the GPU).
inline int pick_rows(int64_t m, int64_t column_tiles) {
  const int64_t sms = b2l_num_sms();
  if (m > 256 && cdiv64(m, 128) * column_tiles >= sms) return 128;
  if (m > 16 && cdiv64(m, 64) * column_tiles >= sms) return 64;
  return m > 64 && cdiv64(m, 16) * column_tiles > 4 * sms ? 64 : 16;
}

}  // namespace

/* 1 when the tensor-core kernels take these operands (16-bit dtype, k and the row / head strides multiples of 8
 * elements, 16-byte aligned bases); the callers use the CUDA-core kernels of csrc/gemm_simt.cu otherwise. */
extern "C" int b2l_rows_gemm_mma_ok(const void* x, const void* w, int64_t k, int64_t x_row_stride, int64_t x_head_stride,
                                    int dtype) {
  return (dtype == B2L_F16 || dtype == B2L_BF16) && k > 0 && k % 8 == 0 && x_row_stride % 8 == 0 &&
         x_head_stride % 8 == 0 && aligned16(x) && aligned16(w);
}

extern "C" int b2l_head_linear_mma(void* y, int64_t y_row_stride, int64_t y_head_stride, const void* x,
                                   int64_t x_row_stride, int64_t x_head_stride, const void* w, const void* gate,
                                   int64_t gate_row_stride, int64_t m, int heads, int64_t n, int64_t k, int dtype,
                                   void* stream) {
  B2L_REQUIRE(y && x && w, "head_linear_mma: null pointer");
  B2L_REQUIRE(m >= 0 && heads > 0 && heads <= 65535 && n > 0, "head_linear_mma: bad shape");
  B2L_REQUIRE(b2l_rows_gemm_mma_ok(x, w, k, x_row_stride, x_head_stride, dtype), "head_linear_mma: operands not aligned");
  if (m == 0) return B2L_OK;
  RowsArgs a = {};
  a.x = x; a.w = w; a.y = y; a.n = n; a.k = k; a.xs = x_row_stride; a.ys = y_row_stride;
  a.m = m; a.xh = x_head_stride; a.yh = y_head_stride; a.gs = gate_row_stride; a.gate = gate;
  const int bm = pick_rows(m, cdiv64(n, kBN) * heads);
  const dim3 grid((unsigned)cdiv64(n, kBN), (unsigned)cdiv64(m, bm), (unsigned)heads);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == B2L_F16) launch_rows<__half, 0>(a, bm, grid, st);
  else launch_rows<__nv_bfloat16, 0>(a, bm, grid, st);
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

/* block_size (16, 64 or 128) is the block size the slots were aligned to (b2l_moe_align_block_size). */
extern "C" int b2l_moe_gemm_mma(void* c, const void* a_in, const void* w, const void* slot_weight_f32,
                                const void* sorted_token_ids, const void* expert_ids,
                                const void* num_tokens_post_padded, int64_t em, int64_t num_valid_slots, int top_k,
                                int block_size, int64_t n, int64_t k, int64_t a_row_stride, int64_t c_row_stride,
                                int act, int dtype, void* stream) {
  B2L_REQUIRE(c && a_in && w && sorted_token_ids && expert_ids && num_tokens_post_padded, "moe_gemm_mma: null pointer");
  B2L_REQUIRE(top_k >= 1 && n > 0 && em >= 0 && (act == 0 || act == 1) &&
                  (block_size == 16 || block_size == 64 || block_size == 128), "moe_gemm_mma: bad shape");
  B2L_REQUIRE(b2l_rows_gemm_mma_ok(a_in, w, k, a_row_stride, 0, dtype), "moe_gemm_mma: operands not aligned");
  if (em == 0 || num_valid_slots == 0) return B2L_OK;
  B2L_REQUIRE(cdiv64(em, block_size) <= 65535, "moe_gemm_mma: %lld row blocks", (long long)cdiv64(em, block_size));
  RowsArgs a = {};
  a.x = a_in; a.w = w; a.y = c; a.n = n; a.k = k; a.xs = a_row_stride; a.ys = c_row_stride;
  a.slot_weight = (const float*)slot_weight_f32; a.sorted_ids = (const int*)sorted_token_ids;
  a.expert_ids = (const int*)expert_ids; a.num_post = (const int*)num_tokens_post_padded;
  a.num_valid = num_valid_slots; a.top_k = top_k; a.act = act;
  const dim3 grid((unsigned)cdiv64(n, kBN), (unsigned)cdiv64(em, block_size));
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == B2L_F16) launch_rows<__half, 1>(a, block_size, grid, st);
  else launch_rows<__nv_bfloat16, 1>(a, block_size, grid, st);
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

/* y_f32[m, n] = x[m, k] . w[n, k]^T with 16-bit operands and the fp32 tensor-core sums stored unrounded. */
extern "C" int b2l_linear_f32out_mma(void* y_f32, const void* x, const void* w, int64_t m, int64_t n, int64_t k,
                                     int64_t x_row_stride, int64_t y_row_stride, int dtype, void* stream) {
  B2L_REQUIRE(y_f32 && x && w, "linear_f32out_mma: null pointer");
  B2L_REQUIRE(m >= 0 && n > 0, "linear_f32out_mma: bad shape");
  B2L_REQUIRE(b2l_rows_gemm_mma_ok(x, w, k, x_row_stride, 0, dtype), "linear_f32out_mma: operands not aligned");
  if (m == 0) return B2L_OK;
  RowsArgs a = {};
  a.x = x; a.w = w; a.y = y_f32; a.n = n; a.k = k; a.xs = x_row_stride; a.ys = y_row_stride; a.m = m; a.out_f32 = 1;
  const int bm = pick_rows(m, cdiv64(n, kBN));
  const dim3 grid((unsigned)cdiv64(n, kBN), (unsigned)cdiv64(m, bm), 1u);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == B2L_F16) launch_rows<__half, 0>(a, bm, grid, st);
  else launch_rows<__nv_bfloat16, 0>(a, bm, grid, st);
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
