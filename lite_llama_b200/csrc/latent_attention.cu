// Per-token preparation for LATENT attention: queries and keys/values go through low-rank latents, only the key/value
// latent and one rotated key part shared by all heads are cached, and the queries are multiplied into the latent space
// so that attention runs directly on the cached rows (csrc/attention_sink.cu with one kv head, value columns =
// the latent itself):
//
//   proj row  = [ a: q_rank | b: kv_rank | r: rot_dim | ... ]          (one fused down-projection of the mixer input)
//   a  <- a / rms(a) * wq                in place: the input of the query up-projection
//   pool row  = [ b / rms(b) * wkv | rotate(r, pos) ]
//
//   rope_heads: dst[t, h, :width] = src[t, h, :width] with the first `rot_dims` entries rotated by the token's position
//               (entry i pairs with entry i + rot_dims/2); the rest is copied.
//
//   rope_table: cs[t] = [cos(pos_t f_i), i < rot_dims/2 | sin(pos_t f_i)], f_i = base^(-2i/rot_dims), once per step: every
//               layer with the same rotary constants reads the same table.
//
// Statistics and the rotation are fp32; the angle and its sine / cosine are evaluated in fp64 (a position of a few
// thousand times a frequency near 1 loses the low bits of the angle in fp32) and stored as fp32.
#include "common.cuh"

namespace {

// cos / sin of pos * base^(-2i/dims) for pair i
__device__ __forceinline__ void pair_angle(int pos, int i, int dims, double log2_base, float& c, float& s) {
  const double f = exp2(-2.0 * (double)i / (double)dims * log2_base);
  double sd, cd;
  sincos((double)pos * f, &sd, &cd);
  c = (float)cd; s = (float)sd;
}

__global__ void rope_table_kernel(float* __restrict__ cs, const int* __restrict__ pos, int64_t tokens, int dims,
                                  double log2_base) {
  pdl_prologue();
  const int half = dims / 2;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= tokens * half) return;
  const int64_t t = i / half;
  const int k = (int)(i - t * half);
  float c, s;
  pair_angle(pos[t], k, dims, log2_base, c, s);
  cs[t * dims + k] = c;
  cs[t * dims + half + k] = s;
}

// One WARP per token (four tokens per CTA): the two statistics are warp reductions, nothing waits on a barrier.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(T* __restrict__ proj, int64_t stride, T* __restrict__ pool,
                                                             int64_t pool_stride, const int* __restrict__ rows,
                                                             const float* __restrict__ cs_table,
                                                             const T* __restrict__ wq, const T* __restrict__ wkv,
                                                             int64_t tokens, int q_rank, int kv_rank, int rot_dim,
                                                             int rot_dims, float eps) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= tokens) return;
  T* a = proj + t * stride;
  const T* b = a + q_rank;
  const T* r = b + kv_rank;
  T* dst = pool + (int64_t)rows[t] * pool_stride;
  float ss = 0.f;
  for (int i = lane; i < q_rank; i += 32) { const float v = to_f32(a[i]); ss = fmaf(v, v, ss); }
  float rstd = 1.0f / sqrtf(warp_reduce_sum(ss) / (float)q_rank + eps);
  for (int i = lane; i < q_rank; i += 32) a[i] = from_f32<T>(to_f32(a[i]) * rstd * to_f32(wq[i]));
  ss = 0.f;
  for (int i = lane; i < kv_rank; i += 32) { const float v = to_f32(b[i]); ss = fmaf(v, v, ss); }
  rstd = 1.0f / sqrtf(warp_reduce_sum(ss) / (float)kv_rank + eps);
  for (int i = lane; i < kv_rank; i += 32) dst[i] = from_f32<T>(to_f32(b[i]) * rstd * to_f32(wkv[i]));
  const int half = rot_dims / 2;
  const float* cs = cs_table + t * rot_dims;
  for (int i = lane; i < half; i += 32) {
    const float c = cs[i], s = cs[half + i];
    const float u = to_f32(r[i]), v = to_f32(r[i + half]);
    dst[kv_rank + i] = from_f32<T>(u * c - v * s);
    dst[kv_rank + i + half] = from_f32<T>(v * c + u * s);
  }
  for (int i = 2 * half + lane; i < rot_dim; i += 32) dst[kv_rank + i] = r[i];
}

// One thread per rotary pair (or per copied element) of one (token, head): the work is spread over the whole grid
// whatever the number of tokens.
template <typename T>
__global__ void __launch_bounds__(256) rope_heads_kernel(T* __restrict__ dst, int64_t dst_stride, int dst_head_stride,
                                                         const T* __restrict__ src, int64_t src_stride,
                                                         int src_head_stride, const float* __restrict__ cs_table,
                                                         int64_t tokens, int heads, int width, int rot_dims) {
  pdl_prologue();
  const int half = rot_dims / 2, per = width - half;            // items per (token, head): pairs, then the copied tail
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * heads * per) return;
  const int64_t th = idx / per;
  const int j = (int)(idx - th * per);
  const int64_t t = th / heads;
  const int h = (int)(th - t * heads);
  const T* sh = src + t * src_stride + (int64_t)h * src_head_stride;
  T* dh = dst + t * dst_stride + (int64_t)h * dst_head_stride;
  if (j < half) {
    const float c = cs_table[t * rot_dims + j], s = cs_table[t * rot_dims + half + j];
    const float u = to_f32(sh[j]), v = to_f32(sh[j + half]);
    dh[j] = from_f32<T>(u * c - v * s);
    dh[j + half] = from_f32<T>(v * c + u * s);
  } else {
    dh[j + half] = sh[j + half];
  }
}

}  // namespace

extern "C" int b2l_rope_table(void* cos_sin_f32, const void* pos_i32, int64_t tokens, int rot_dims, float rot_base,
                              void* stream) {
  B2L_REQUIRE(cos_sin_f32 && pos_i32, "rope_table: null pointer");
  B2L_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_base > 0.f, "rope_table: bad constants");
  if (tokens <= 0 || rot_dims == 0) return B2L_OK;
  const int64_t total = tokens * (rot_dims / 2);
  b2l_launch(rope_table_kernel, dim3((unsigned)cdiv64(total, 128)), dim3(128), (size_t)0, (cudaStream_t)stream,
             (float*)cos_sin_f32, (const int*)pos_i32, tokens, rot_dims, log2((double)rot_base));
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_latent_prepare(void* proj, int64_t proj_row_stride, void* pool, int64_t pool_row_stride,
                                  const void* kv_rows_i32, const void* cos_sin_f32, const void* q_norm_weight,
                                  const void* kv_norm_weight, int64_t tokens, int q_rank, int kv_rank, int rot_dim,
                                  int rot_dims, float eps, int dtype, void* stream) {
  B2L_REQUIRE(proj && pool && kv_rows_i32 && q_norm_weight && kv_norm_weight, "latent_prepare: null pointer");
  B2L_REQUIRE(q_rank > 0 && kv_rank > 0 && rot_dim >= 0 && rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0,
              "latent_prepare: bad shape (q_rank %d, kv_rank %d, rot_dim %d, rot_dims %d)", q_rank, kv_rank, rot_dim, rot_dims);
  B2L_REQUIRE(cos_sin_f32 || rot_dims == 0, "latent_prepare: no rotation table");
  if (tokens <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  B2L_DISPATCH_FLOAT(dtype, "latent_prepare", {
    b2l_launch(latent_prepare_kernel<T>, dim3((unsigned)cdiv64(tokens, 4)), dim3(128), (size_t)0, st, (T*)proj,
               proj_row_stride, (T*)pool, pool_row_stride, (const int*)kv_rows_i32, (const float*)cos_sin_f32,
               (const T*)q_norm_weight, (const T*)kv_norm_weight, tokens, q_rank, kv_rank, rot_dim, rot_dims, eps);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_rope_heads(void* dst, int64_t dst_row_stride, int dst_head_stride, const void* src,
                              int64_t src_row_stride, int src_head_stride, const void* cos_sin_f32, int64_t tokens,
                              int heads, int width, int rot_dims, int dtype, void* stream) {
  B2L_REQUIRE(dst && src, "rope_heads: null pointer");
  B2L_REQUIRE(heads > 0 && width >= 0 && rot_dims >= 0 && rot_dims <= width && rot_dims % 2 == 0,
              "rope_heads: bad shape (heads %d, width %d, rot_dims %d)", heads, width, rot_dims);
  B2L_REQUIRE(cos_sin_f32 || rot_dims == 0, "rope_heads: no rotation table");
  if (tokens <= 0 || width == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  B2L_DISPATCH_FLOAT(dtype, "rope_heads", {
    b2l_launch(rope_heads_kernel<T>, dim3((unsigned)cdiv64(tokens * heads * (width - rot_dims / 2), 256)), dim3(256),
               (size_t)0, st, (T*)dst, dst_row_stride,
               dst_head_stride, (const T*)src, src_row_stride, src_head_stride, (const float*)cos_sin_f32, tokens, heads,
               width, rot_dims);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
