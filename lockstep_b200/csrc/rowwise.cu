// Row-wise kernels of designs that norm after a sublayer as well as before it:
//   - layer norm with a gain and no bias, (x - mean) rsqrt(var + eps) gain, var the mean of the
//     squared deviations (rows may be gathered through row_index);
//   - the closing kernel of a sublayer: the RMS-normed results of mixers side by side, each with
//     a gain of its own, summed with one factor; optionally a layer norm of that sum; added to
//     the residual stream;
//   - an embedding with a factor on the token's row and a second table indexed by a hash of the
//     token and the one before it, whose last row serves a sequence's first token;
//   - float32 rows written into some columns of a wider row of the engine's type; logits times a
//     factor, then capped with tanh.
// All reductions run in float32 in an order fixed by the row's own width (a thread's elements
// ascending, the lanes by an xor tree, the warps ascending), so a row's result does not depend on the batch.
#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;  // a block per row

template <typename TG>
__device__ __forceinline__ float gain_of(const TG* g, int i) { return ls_to_float<TG>(g[i]); }

// Sum over the block in a fixed order (lanes by xor tree, warps ascending); every thread gets it.  `scratch`: 32 floats.
__device__ __forceinline__ float row_sum(float v, float* scratch) {
  const float total = ls_block_sum(v, scratch);
  __syncthreads();                 // scratch is free for the next sum
  return total;
}

// (x - mean) rsqrt(var + eps) gain over float32 rows.  A thread takes the elements tid, tid + 256, ... of the row and
// keeps up to eight of them in registers between the passes (rows up to 2,048 wide are read once).
template <typename TG, typename TO>
__global__ void __launch_bounds__(ROW_THREADS)
layernorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index, const TG* __restrict__ gain,
                 TO* __restrict__ out, int rows, int width, int x_rows, float eps, int* err) {
  __shared__ float scratch[32];
  ls_dependency_sync();
  const int r = blockIdx.x, tid = threadIdx.x;
  int src_row = r;
  if (row_index != nullptr) {
    src_row = row_index[r];
    if (src_row < 0 || src_row >= x_rows) {
      if (tid == 0) ls_record_fault(err, LS_DEV_ROW_RANGE, r);
      src_row = 0;
    }
  }
  const float* row = x + (int64_t)src_row * width;
  constexpr int KEEP = 8;
  float v[KEEP];
#pragma unroll
  for (int j = 0; j < KEEP; ++j) v[j] = tid + j * ROW_THREADS < width ? row[tid + j * ROW_THREADS] : 0.f;
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) s += v[j];
  for (int i = tid + KEEP * ROW_THREADS; i < width; i += ROW_THREADS) s += row[i];
  const float mean = row_sum(s, scratch) / (float)width;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const float d = tid + j * ROW_THREADS < width ? v[j] - mean : 0.f;
    q = fmaf(d, d, q);
  }
  for (int i = tid + KEEP * ROW_THREADS; i < width; i += ROW_THREADS) {
    const float d = row[i] - mean;
    q = fmaf(d, d, q);
  }
  const float rstd = 1.0f / sqrtf(row_sum(q, scratch) / (float)width + eps);
  TO* dst = out + (int64_t)r * width;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int i = tid + j * ROW_THREADS;
    if (i < width) dst[i] = ls_from_float<TO>((v[j] - mean) * rstd * gain_of<TG>(gain, i));
  }
  for (int i = tid + KEEP * ROW_THREADS; i < width; i += ROW_THREADS)
    dst[i] = ls_from_float<TO>((row[i] - mean) * rstd * gain_of<TG>(gain, i));
}

// residual += post(scale sum_b rms_b(x_b) gain_b), post = layer norm with post_gain, or nothing.  The merged row
// lies in shared memory between the passes.
__global__ void __launch_bounds__(ROW_THREADS)
norm_merge_add_kernel(float* __restrict__ residual, const float* __restrict__ branches, int n, int64_t branch_stride,
                      const float* __restrict__ branch_gain, float scale, const float* __restrict__ post_gain,
                      int rows, int width, float eps_branch, float eps_post) {
  extern __shared__ float merged[];                 // [width]
  __shared__ float scratch[32];
  ls_dependency_sync();
  const int r = blockIdx.x, tid = threadIdx.x;
  constexpr int MAX_N = 4;
  float rstd_b[MAX_N];
#pragma unroll
  for (int b = 0; b < MAX_N; ++b) {
    rstd_b[b] = 1.0f;
    if (b < n && branch_gain != nullptr) {
      const float* row = branches + b * branch_stride + (int64_t)r * width;
      float q = 0.f;
#pragma unroll 4
      for (int i = tid; i < width; i += ROW_THREADS) q = fmaf(row[i], row[i], q);
      rstd_b[b] = 1.0f / sqrtf(row_sum(q, scratch) / (float)width + eps_branch);
    }
  }
  float s = 0.f;
#pragma unroll 2
  for (int i = tid; i < width; i += ROW_THREADS) {
    float v = 0.f;
#pragma unroll
    for (int b = 0; b < MAX_N; ++b)
      if (b < n) {
        const float xb = branches[b * branch_stride + (int64_t)r * width + i];
        v += branch_gain != nullptr ? xb * rstd_b[b] * branch_gain[b * width + i] : xb;
      }
    v *= scale;
    merged[i] = v;                                  // (read back by this thread alone)
    s += v;
  }
  float* dst = residual + (int64_t)r * width;
  if (post_gain == nullptr) {
#pragma unroll 4
    for (int i = tid; i < width; i += ROW_THREADS) dst[i] += merged[i];
    return;
  }
  const float mean = row_sum(s, scratch) / (float)width;
  float q = 0.f;
  for (int i = tid; i < width; i += ROW_THREADS) {
    const float d = merged[i] - mean;
    q = fmaf(d, d, q);
  }
  const float rstd = 1.0f / sqrtf(row_sum(q, scratch) / (float)width + eps_post);
#pragma unroll 4
  for (int i = tid; i < width; i += ROW_THREADS) dst[i] += (merged[i] - mean) * rstd * post_gain[i];
}

// out[t] = table[id] factor + pairs[row(previous id, id)]
template <typename T>
__global__ void pair_embed_kernel(const int* __restrict__ ids, const int* __restrict__ token_slot,
                                  const int* __restrict__ carried, int64_t carried_stride, const T* __restrict__ table,
                                  const T* __restrict__ pairs, float* __restrict__ out, int width, int vocab, int buckets,
                                  long long mul_prev, long long mul_cur, float factor, int* err) {
  ls_dependency_sync();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + (int64_t)t * width;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) ls_record_fault(err, LS_DEV_TOKEN_RANGE, t);
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (int64_t)id * width;
  if (pairs == nullptr) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = ls_to_float<T>(src[i]) * factor;
    return;
  }
  // the token before: the one in front of it in the step where that belongs to the same request, else what the
  // request's slot keeps (the last token of its last portion, plus one; zero: the request has none yet)
  const int slot = token_slot[t];
  long long prev = (t > 0 && token_slot[t - 1] == slot) ? (long long)ids[t - 1] : (long long)carried[slot * carried_stride] - 1;
  if (prev >= vocab) prev = -1;
  const long long row = prev < 0 ? buckets : (prev * mul_prev + (long long)id * mul_cur) % buckets;
  const T* pair = pairs + row * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    dst[i] = fmaf(ls_to_float<T>(src[i]), factor, ls_to_float<T>(pair[i]));
}

// the last token of every request's portion, plus one, into the request's slot
__global__ void pair_carry_kernel(const int* __restrict__ ids, const int* __restrict__ token_slot,
                                  int* __restrict__ carried, int64_t carried_stride, int tokens) {
  ls_dependency_sync();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const int slot = token_slot[t];
  if (t == tokens - 1 || token_slot[t + 1] != slot) carried[slot * carried_stride] = ids[t] + 1;
}

template <typename TO>
__global__ void rows_cast_kernel(const float* __restrict__ src, TO* __restrict__ dst, int64_t rows, int width, int64_t ld) {
  ls_dependency_sync();
  const int64_t n = rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width;
    dst[r * ld + (i - r * width)] = ls_from_float<TO>(src[i]);
  }
}

__global__ void scale_cap_kernel(float* __restrict__ x, int64_t count, float factor, float cap) {
  ls_dependency_sync();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = x[i] * factor;
    x[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

inline int blocks_for(int64_t n) { return (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16); }

}  // namespace

LS_API int ls_layernorm(const float* x, const int* row_index, const void* gain, int gain_dtype, void* out, int out_dtype,
                        int rows, int width, int x_rows, float eps, int* err, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0) return LS_E_SIZE;
  const dim3 grid(rows), block(ROW_THREADS);
  LS_COUNT(LS_K_LAYERNORM);
#define LS_LN(TG, TO) \
  ls_launch(layernorm_kernel<TG, TO>, grid, block, 0, stream, x, row_index, (const TG*)gain, (TO*)out, rows, width, x_rows, eps, err)
  if (gain_dtype == LS_F32 && out_dtype == LS_F32) LS_LN(float, float);
  else if (gain_dtype == LS_F32 && out_dtype == LS_BF16) LS_LN(float, __nv_bfloat16);
  else if (gain_dtype == LS_BF16 && out_dtype == LS_BF16) LS_LN(__nv_bfloat16, __nv_bfloat16);
  else if (gain_dtype == LS_BF16 && out_dtype == LS_F32) LS_LN(__nv_bfloat16, float);
  else return LS_E_DTYPE;
#undef LS_LN
  return ls_launch_status();
}

LS_API int ls_norm_merge_add(float* residual, const float* branches, int n, long long branch_stride, const float* branch_gain,
                             float scale, const float* post_gain, int rows, int width, float eps_branch, float eps_post,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || n < 1 || n > 4) return LS_E_SIZE;
  const size_t smem = sizeof(float) * (size_t)width;
  if (smem > 200 * 1024) return LS_E_SMEM;
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    if (cudaFuncSetAttribute(norm_merge_add_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LS_E_SMEM;
    configured = smem;
  }
  LS_COUNT(LS_K_NORM_MERGE_ADD);
  ls_launch(norm_merge_add_kernel, dim3(rows), dim3(ROW_THREADS), smem, stream, residual, branches,
            n, (int64_t)branch_stride, branch_gain, scale, post_gain, rows, width, eps_branch, eps_post);
  return ls_launch_status();
}

LS_API int ls_pair_embed(const int* ids, const int* token_slot, int* carried, long long carried_stride, const void* table,
                         const void* pairs, int dtype, float* out, int tokens, int width, int vocab, int buckets,
                         long long mul_prev, long long mul_cur, float factor, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (pairs != nullptr && (buckets <= 0 || carried == nullptr || token_slot == nullptr)) return LS_E_SIZE;
  const int threads = width >= 1024 ? 256 : 128;
  LS_COUNT(LS_K_PAIR_EMBED);
  if (dtype == LS_F32)
    ls_launch(pair_embed_kernel<float>, tokens, threads, 0, stream, ids, token_slot, (const int*)carried, (int64_t)carried_stride,
              (const float*)table, (const float*)pairs, out, width, vocab, buckets, mul_prev, mul_cur, factor, err);
  else if (dtype == LS_BF16)
    ls_launch(pair_embed_kernel<__nv_bfloat16>, tokens, threads, 0, stream, ids, token_slot, (const int*)carried,
              (int64_t)carried_stride, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, out, width, vocab, buckets,
              mul_prev, mul_cur, factor, err);
  else
    return LS_E_DTYPE;
  if (ls_launch_status() != 0) return ls_launch_status();
  if (pairs != nullptr)
    ls_launch(pair_carry_kernel, dim3((tokens + 127) / 128), dim3(128), 0, stream, ids, token_slot, carried,
              (int64_t)carried_stride, tokens);
  return ls_launch_status();
}

LS_API int ls_rows_cast(const float* src, void* dst, int dst_dtype, long long rows, int width, long long ld, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || ld < width) return LS_E_SIZE;
  LS_COUNT(LS_K_ROWS_CAST);
  if (dst_dtype == LS_F32) ls_launch(rows_cast_kernel<float>, blocks_for(rows * width), 256, 0, stream, src, (float*)dst, (int64_t)rows, width, (int64_t)ld);
  else if (dst_dtype == LS_BF16) ls_launch(rows_cast_kernel<__nv_bfloat16>, blocks_for(rows * width), 256, 0, stream, src, (__nv_bfloat16*)dst, (int64_t)rows, width, (int64_t)ld);
  else return LS_E_DTYPE;
  return ls_launch_status();
}

LS_API int ls_scale_cap(float* x, long long count, float factor, float cap, cudaStream_t stream) {
  if (count <= 0) return 0;
  LS_COUNT(LS_K_SCALE_CAP);
  ls_launch(scale_cap_kernel, blocks_for(count), 256, 0, stream, x, (int64_t)count, factor, cap);
  return ls_launch_status();
}
