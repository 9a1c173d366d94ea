// Row-wise kernels of the step: embedding gather, RMSNorm, and the fused
// per-head norm + rotary position encoding + paged cache write.
//
// All reductions run in float32 in an order fixed by the row's own width, so
// a row's result does not depend on what else is in the batch.
#include "common.cuh"
#include "rope.cuh"

// --------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :]   (out is the float32 residual stream)
// --------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                    float* __restrict__ out, int width, int vocab, int accumulate, int* err) {
  ls_dependency_sync();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + (int64_t)t * width;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) ls_record_fault(err, LS_DEV_TOKEN_RANGE, t);
    if (!accumulate)
      for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (int64_t)id * width;
  if (accumulate) {
    // the token's embedding is added to a residual stream that already holds something (a
    // model that feeds the embedding in again before a later pass over some of its layers)
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] += ls_to_float<T>(src[i]);
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = ls_to_float<T>(src[i]);
  }
}

LS_API int ls_embed_gather(const int* ids, const void* table, int table_dtype, float* out,
                           int tokens, int width, int vocab, int accumulate, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (table_dtype == LS_F32)
    LS_COUNT(LS_K_EMBED_GATHER), ls_launch(embed_gather_kernel<float>, tokens, threads, 0, stream, ids, (const float*)table, out, width, vocab, accumulate, err);
  else if (table_dtype == LS_BF16)
    LS_COUNT(LS_K_EMBED_GATHER), ls_launch(embed_gather_kernel<__nv_bfloat16>, tokens, threads, 0, stream, ids, (const __nv_bfloat16*)table, out, width, vocab, accumulate, err);
  else
    return LS_E_DTYPE;
  return ls_launch_status();
}

// four gains as floats in one access, and four outputs out in one access (the row's and the
// gain's starts are 16-byte aligned where these are used)
template <typename TG>
__device__ __forceinline__ float4 ls_load4(const TG* p) {
  if constexpr (sizeof(TG) == 4) {
    return *reinterpret_cast<const float4*>(p);
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y));
  }
}
template <typename TO>
__device__ __forceinline__ void ls_store4(TO* p, float a, float b, float c, float d) {
  if constexpr (sizeof(TO) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
  }
}

// --------------------------------------------------------------------------
// RMSNorm over float32 rows: y = x * rsqrt(mean(x^2) + eps) * gain
// rows may be gathered through row_index (the rows whose logits are wanted).
// --------------------------------------------------------------------------
// One warp per row: lane l takes the float4 groups l, l + 32, ... of the row, keeps
// them in registers between the two passes (rows up to 8192 wide; wider rows are
// read twice), sums its squares in that order and the lanes by an xor tree.  The
// order depends on the width alone.
// y[0..4) = x * rstd * gain, in one access each for the gains and the outputs where `vec`
template <typename TO, typename TG>
__device__ __forceinline__ void rmsnorm_out4(TO* y, const TG* gain, const float* x, float rstd, bool vec) {
  if (vec) {
    const float4 gn = ls_load4<TG>(gain);
    ls_store4<TO>(y, x[0] * rstd * gn.x, x[1] * rstd * gn.y, x[2] * rstd * gn.z, x[3] * rstd * gn.w);
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) y[e] = ls_from_float<TO>(x[e] * rstd * ls_to_float<TG>(gain[e]));
  }
}

template <typename TO, typename TG>
__global__ void __launch_bounds__(128)
rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
               const TG* __restrict__ gain_all, TO* __restrict__ y, int rows, int width, int src_rows,
               float eps, int parts, int64_t x_ld, int* err) {
  ls_dependency_sync();
  constexpr int KEEP = 64;                    // floats a lane keeps: 16 float4
  const int lane = threadIdx.x & 31;
  // a row of `parts` equal consecutive parts, each normalised by its own root mean square, is
  // `parts` rows of `width` elements to this kernel (the gain runs over the whole row)
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= rows * parts) return;
  const int r = unit / parts, part = unit - r * parts;
  int src = row_index ? row_index[r] : r;
  if (src < 0 || src >= src_rows) {
    if (lane == 0) ls_record_fault(err, LS_DEV_ROW_RANGE, r);
    src = 0;
  }
  // (x_ld: the source rows' pitch, where the normed columns are the first of a wider row)
  const float* xr = x + (int64_t)src * x_ld + (int64_t)part * width;
  TO* yr = y + ((int64_t)r * parts + part) * width;
  const TG* gain = gain_all + (int64_t)part * width;
  const bool vec = (width & 3) == 0 && ((uintptr_t)xr & 15) == 0;
  // four outputs an access where the outputs and the gains allow it (this changes no sum)
  const bool vec_out = ((uintptr_t)y & (4 * sizeof(TO) - 1)) == 0 && ((uintptr_t)gain & (4 * sizeof(TG) - 1)) == 0;
  float keep[KEEP];
  float ss = 0.f;
  if (vec) {
    const int groups = width >> 2;
#pragma unroll
    for (int i = 0; i < KEEP / 4; ++i) {
      const int g = lane + 32 * i;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (g < groups) v = *reinterpret_cast<const float4*>(xr + 4 * g);
      keep[4 * i + 0] = v.x; keep[4 * i + 1] = v.y; keep[4 * i + 2] = v.z; keep[4 * i + 3] = v.w;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    for (int g = lane + 32 * (KEEP / 4); g < groups; g += 32) {
      const float4 v = *reinterpret_cast<const float4*>(xr + 4 * g);
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
  } else {
    for (int i = lane; i < width; i += 32) ss = fmaf(xr[i], xr[i], ss);
  }
  ss = ls_warp_sum(ss);
  const float rstd = 1.0f / sqrtf(ss / (float)width + eps);
  if (vec) {
    const int groups = width >> 2;
#pragma unroll
    for (int i = 0; i < KEEP / 4; ++i) {
      const int g = lane + 32 * i;
      if (g < groups) rmsnorm_out4<TO, TG>(yr + 4 * g, gain + 4 * g, keep + 4 * i, rstd, vec_out);
    }
    for (int g = lane + 32 * (KEEP / 4); g < groups; g += 32) {
      const float4 v = *reinterpret_cast<const float4*>(xr + 4 * g);
      const float four[4] = {v.x, v.y, v.z, v.w};
      rmsnorm_out4<TO, TG>(yr + 4 * g, gain + 4 * g, four, rstd, vec_out);
    }
  } else {
    for (int i = lane; i < width; i += 32)
      yr[i] = ls_from_float<TO>(xr[i] * rstd * ls_to_float<TG>(gain[i]));
  }
}

LS_API int ls_rmsnorm(const float* x, const int* row_index, const void* gain, int gain_dtype,
                      void* y, int y_dtype, int rows, int row_width, int src_rows, float eps,
                      int parts, int64_t x_ld, int* err, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (parts <= 0 || row_width % parts) return LS_E_SIZE;
  if (x_ld <= 0) x_ld = row_width;
  if (x_ld < row_width) return LS_E_SIZE;
  const int width = row_width / parts;
  // few rows: one warp per block, so that the rows spread over the device
  const int warps = (int64_t)rows * parts >= 1024 ? 4 : 1;
  const int blocks = (rows * parts + warps - 1) / warps;
#define LS_RMS(TO, TG)                                                                          \
  LS_COUNT(LS_K_RMSNORM), ls_launch(rmsnorm_kernel<TO, TG>, blocks, warps * 32, 0, stream, x, row_index, (const TG*)gain, (TO*)y, \
                                                            rows, width, src_rows, eps, parts, x_ld, err)
  if (y_dtype == LS_F32 && gain_dtype == LS_F32) LS_RMS(float, float);
  else if (y_dtype == LS_F32 && gain_dtype == LS_BF16) LS_RMS(float, __nv_bfloat16);
  else if (y_dtype == LS_BF16 && gain_dtype == LS_F32) LS_RMS(__nv_bfloat16, float);
  else if (y_dtype == LS_BF16 && gain_dtype == LS_BF16) LS_RMS(__nv_bfloat16, __nv_bfloat16);
  else return LS_E_DTYPE;
#undef LS_RMS
  return ls_launch_status();
}

// --------------------------------------------------------------------------
// Per-head RMSNorm (optional) + rotary position encoding (optional) of q and k,
// and the write of k and v into the paged cache.  A block per token, its warps over the heads.
//
// qkv:   [tokens, (nq + 2*nkv) * d]   projections of this step's tokens
// q_out: [tokens, nq * d]
// pages: [num_pages, 2, nkv, page_size, d]   one layer of one cache group
// The page of a token is block_table[req_row[token] * table_stride + pos / page_size].
// --------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_rope_store_kernel(const T* __restrict__ qkv, const LsQkvStore args, int tokens, int* err) {
  ls_dependency_sync();
  // the token's projections come into shared memory in 16-byte pieces; then a warp per head
  extern __shared__ uint4 row_smem[];
  const int t = blockIdx.x;
  const int heads_total = args.nq + 2 * args.nkv;
  const int row_elems = heads_total * args.d;
  const T* row = qkv + (int64_t)t * row_elems;
  constexpr int PER = 16 / (int)sizeof(T);
  if ((row_elems % PER) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    for (int i = threadIdx.x; i < row_elems / PER; i += blockDim.x)
      row_smem[i] = reinterpret_cast<const uint4*>(row)[i];
  } else {
    T* dst = reinterpret_cast<T*>(row_smem);
    for (int i = threadIdx.x; i < row_elems; i += blockDim.x) dst[i] = row[i];
  }
  __syncthreads();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int head = warp; head < heads_total; head += warps)
    ls_qkv_head_store<T>(args, reinterpret_cast<const T*>(row_smem) + head * args.d, t, head, lane, err);
}

// The same for bfloat16 heads of D = 64 or 128 elements that are rotated whole, at a fraction
// of the instructions: what belongs to the token (position, page, cosines, sines, gains) is
// looked up once per token and not once per head, a lane keeps its four (two) elements of a
// head in registers and writes the results over the staged row, and the row leaves in 16-byte
// pieces.  Every sum and product is ls_norm_rope_head's, in its order: the bits are the same.
template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_whole_kernel(const __nv_bfloat16* __restrict__ qkv, const LsQkvStore args, int tokens, int* err) {
  typedef __nv_bfloat16 bf16;
  constexpr int PER_LANE = D / 32;                // a lane's elements of a head: lane, lane + 32, ...
  constexpr int VEC = D / 8;                      // 16-byte pieces of a head
  ls_dependency_trigger();
  extern __shared__ uint4 row_smem[];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = args.nq, nkv = args.nkv;
  const int heads_total = nq + 2 * nkv;
  // weights first: they do not wait for the kernel before
  float gq[PER_LANE], gk[PER_LANE];
  const bool normed = args.q_gain != nullptr;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    gq[j] = gk[j] = 1.f;
    if (normed) {
      const int i = lane + 32 * j;
      if (args.gain_bf16) {
        gq[j] = __bfloat162float(reinterpret_cast<const bf16*>(args.q_gain)[i]);
        gk[j] = __bfloat162float(reinterpret_cast<const bf16*>(args.k_gain)[i]);
      } else {
        gq[j] = reinterpret_cast<const float*>(args.q_gain)[i];
        gk[j] = reinterpret_cast<const float*>(args.k_gain)[i];
      }
    }
  }
  ls_dependency_wait();
  const uint4* row = reinterpret_cast<const uint4*>(qkv + (int64_t)t * heads_total * D);
  for (int i = threadIdx.x; i < heads_total * VEC; i += blockDim.x) row_smem[i] = row[i];
  // the token's place: the same in every thread
  const int pos = args.positions[t];
  const bool pos_ok = pos >= 0 && pos < args.max_positions;
  int page = 0;
  bool page_ok = false;
  if (args.write_cache && pos_ok) {
    page = args.block_table[(int64_t)args.token_req[t] * args.table_stride + pos / args.page_size];
    page_ok = page >= 0 && page < args.num_pages;
  }
  float cs[PER_LANE / 2], sn[PER_LANE / 2];
#pragma unroll
  for (int j = 0; j < PER_LANE / 2; ++j) {
    cs[j] = sn[j] = 0.f;
    if (pos_ok) {
      cs[j] = args.cos_table[(int64_t)pos * (D / 2) + lane + 32 * j];
      sn[j] = args.sin_table[(int64_t)pos * (D / 2) + lane + 32 * j];
    }
  }
  if (threadIdx.x == 0) {
    if (!pos_ok) ls_record_fault(err, LS_DEV_POSITION_RANGE, t);
    else if (args.write_cache && !page_ok) ls_record_fault(err, LS_DEV_PAGE_RANGE, t);
  }
  __syncthreads();
  bf16* staged = reinterpret_cast<bf16*>(row_smem);
  if (pos_ok) {
    const int normed_heads = args.write_cache && page_ok ? nq + nkv : nq;      // v heads leave as they came
    for (int head = warp; head < normed_heads; head += 8) {
      bf16* h = staged + head * D;
      const float* gain = head < nq ? gq : gk;
      float v[PER_LANE];
      float rstd = 1.f;
#pragma unroll
      for (int j = 0; j < PER_LANE; ++j) v[j] = __bfloat162float(h[lane + 32 * j]);
      if (normed) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) ss = fmaf(v[j], v[j], ss);
        ss = ls_warp_sum(ss);
        rstd = 1.0f / sqrtf(ss / (float)D + args.eps);
      }
#pragma unroll
      for (int j = 0; j < PER_LANE / 2; ++j) {
        float lo = __fmul_rn(v[j], rstd);
        float hi = __fmul_rn(v[j + PER_LANE / 2], rstd);
        if (normed) {
          lo = __fmul_rn(lo, gain[j]);
          hi = __fmul_rn(hi, gain[j + PER_LANE / 2]);
        }
        h[lane + 32 * j] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(lo, cs[j]), __fmul_rn(hi, sn[j])));
        h[lane + 32 * j + D / 2] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(hi, cs[j]), __fmul_rn(lo, sn[j])));
      }
    }
  }
  __syncthreads();
  // out: q heads side by side into q_out's row; k and v heads each to its line of the page
  const int first = pos_ok ? 0 : nq * VEC;                                  // a bad position writes nothing
  const int last = args.write_cache && page_ok ? heads_total * VEC : nq * VEC;
  uint4* q_dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(args.q_out) + (int64_t)t * nq * D);
  const int slot = args.write_cache && page_ok ? pos % args.page_size : 0;
  for (int i = first + threadIdx.x; i < last; i += blockDim.x) {
    const int head = i / VEC, piece = i % VEC;
    if (head < nq) {
      q_dst[i] = row_smem[i];
    } else {
      const int is_v = head >= nq + nkv ? 1 : 0;
      const int kvh = head - nq - is_v * nkv;
      const int64_t line = (((int64_t)page * 2 + is_v) * nkv + kvh) * args.page_size + slot;
      reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(args.pages) + line * D)[piece] = row_smem[i];
    }
  }
}

LS_API int ls_qk_norm_rope_store(const void* qkv, void* q_out, void* pages, int dtype,
                                 const void* q_gain, const void* k_gain, int gain_dtype,
                                 const float* cos_table, const float* sin_table,
                                 const int* positions, const int* token_req,
                                 const int* block_table, int table_stride, int tokens, int nq,
                                 int nkv, int d, int rot_dim, int page_size, int num_pages,
                                 int max_positions, float eps, int write_cache, int interleaved,
                                 int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot_dim < 0 || rot_dim > d || (rot_dim & 1)) return LS_E_SIZE;
  const int heads = nq + 2 * nkv;
  const int warps = heads < 8 ? heads : 8;
  const size_t smem = (size_t)heads * d * (dtype == LS_F32 ? 4 : 2);
  if (smem > 200 * 1024) return LS_E_SIZE;          // a token's projections must fit shared memory
  if (smem > 48 * 1024) {
    static size_t allowed_f32 = 0, allowed_bf16 = 0;
    size_t& allowed = dtype == LS_F32 ? allowed_f32 : allowed_bf16;
    if (smem > allowed) {
      cudaError_t e = dtype == LS_F32
                          ? cudaFuncSetAttribute(qk_norm_rope_store_kernel<float>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                          : cudaFuncSetAttribute(qk_norm_rope_store_kernel<__nv_bfloat16>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return LS_E_SMEM;
      allowed = smem;
    }
  }
  dim3 grid(tokens);
  if (gain_dtype != LS_F32 && gain_dtype != LS_BF16) return LS_E_DTYPE;
  LsQkvStore args;
  args.q_out = q_out;
  args.pages = pages;
  args.q_gain = q_gain;
  args.k_gain = k_gain;
  args.cos_table = cos_table;
  args.sin_table = sin_table;
  args.positions = positions;
  args.token_req = token_req;
  args.block_table = block_table;
  args.gain_bf16 = gain_dtype == LS_BF16 ? 1 : 0;
  args.table_stride = table_stride;
  args.nq = nq;
  args.nkv = nkv;
  args.d = d;
  args.rot_dim = rot_dim;
  args.page_size = page_size;
  args.num_pages = num_pages;
  args.max_positions = max_positions;
  args.write_cache = write_cache;
  args.eps = eps;
  args.interleaved = interleaved ? 1 : 0;
  // whole heads of 64 or 128 bfloat16 in the half layout, rows and targets on 16-byte boundaries: the short kernel
  const bool whole = dtype == LS_BF16 && (d == 64 || d == 128) && rot_dim == d && !interleaved && (q_gain == nullptr) == (k_gain == nullptr) &&
                     (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)pages) & 15) == 0 && smem <= 48 * 1024;
  if (whole) {
    if (d == 64)
      LS_COUNT(LS_K_QK_NORM_ROPE_WHOLE), ls_launch(qk_norm_rope_store_whole_kernel<64>, grid, 256, smem, stream, (const __nv_bfloat16*)qkv, args, tokens, err);
    else
      LS_COUNT(LS_K_QK_NORM_ROPE_WHOLE), ls_launch(qk_norm_rope_store_whole_kernel<128>, grid, 256, smem, stream, (const __nv_bfloat16*)qkv, args, tokens, err);
    return ls_launch_status();
  }
  if (dtype == LS_F32)
    LS_COUNT(LS_K_QK_NORM_ROPE), ls_launch(qk_norm_rope_store_kernel<float>, grid, warps * 32, smem, stream, (const float*)qkv, args, tokens, err);
  else if (dtype == LS_BF16)
    LS_COUNT(LS_K_QK_NORM_ROPE), ls_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, grid, warps * 32, smem, stream, (const __nv_bfloat16*)qkv, args,
              tokens, err);
  else
    return LS_E_DTYPE;
  return ls_launch_status();
}

// --------------------------------------------------------------------------
// silu(gate) * up on [rows, 2*width] -> [rows, width]  (gate in the first half)
// used where the product is not fused into the GEMM that makes gate and up
// --------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int64_t rows,
                                int width) {
  ls_dependency_sync();
  const int64_t n = rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width;
    const int c = (int)(i - r * width);
    const float g = ls_to_float<T>(gate_up[r * 2 * width + c]);
    const float u = ls_to_float<T>(gate_up[r * 2 * width + width + c]);
    out[i] = ls_from_float<T>(g / (1.0f + expf(-g)) * u);
  }
}

LS_API int ls_silu_mul(const void* gate_up, void* out, int dtype, int rows, int width,
                       cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int64_t n = (int64_t)rows * width;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (dtype == LS_F32)
    LS_COUNT(LS_K_SILU_MUL), ls_launch(silu_mul_kernel<float>, blocks, 256, 0, stream, (const float*)gate_up, (float*)out, rows, width);
  else if (dtype == LS_BF16)
    LS_COUNT(LS_K_SILU_MUL), ls_launch(silu_mul_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, rows, width);
  else
    return LS_E_DTYPE;
  return ls_launch_status();
}


// --------------------------------------------------------------------------
// Gated feed-forward activation with clamps: from a product's float32 or engine-type output
// [rows, 2 * width] (gate columns, then up columns) and optional biases [2 * width]:
//   g = min(gate + b, limit), u = clamp(up + b, -limit, limit), out = g * sigmoid(alpha g) * (u + 1)
// computed in float32.  `residual` (or null): the bias of the projection that follows is added to
// the float32 residual stream [rows, res_width] by the same launch, so that the product that
// comes next only has to add itself.
// --------------------------------------------------------------------------
template <typename TI, typename TO, typename TB>
__global__ void clamped_glu_kernel(const TI* __restrict__ gate_up, const TB* __restrict__ bias, TO* __restrict__ out,
                                   int64_t rows, int width, int64_t in_ld, float limit, float alpha,
                                   float* __restrict__ residual, const TB* __restrict__ res_bias, int res_width, int vec,
                                   float up_offset, int gelu) {
  ls_dependency_sync();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  auto act = [&](float g, float u, int c) {
    if (bias != nullptr) {
      g += ls_to_float<TB>(bias[c]);
      u += ls_to_float<TB>(bias[width + c]);
    }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    // gelu: the tanh form, 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))
    if (gelu) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * (u + up_offset);
    return g / (1.0f + expf(-alpha * g)) * (u + up_offset);
  };
  if (vec) {
    // four columns a thread, 16 bytes a load (widths that are multiples of four, aligned rows)
    const int64_t n4 = rows * (width >> 2);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
      const int64_t r = i / (width >> 2);
      const int c = (int)(i - r * (width >> 2)) << 2;
      const float4 g4 = ls_load4<TI>(gate_up + r * in_ld + c);
      const float4 u4 = ls_load4<TI>(gate_up + r * in_ld + width + c);
      ls_store4<TO>(out + r * width + c, act(g4.x, u4.x, c), act(g4.y, u4.y, c + 1), act(g4.z, u4.z, c + 2),
                    act(g4.w, u4.w, c + 3));
    }
  } else {
    const int64_t n = rows * width;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      const int64_t r = i / width;
      const int c = (int)(i - r * width);
      out[i] = ls_from_float<TO>(act(ls_to_float<TI>(gate_up[r * in_ld + c]),
                                     ls_to_float<TI>(gate_up[r * in_ld + width + c]), c));
    }
  }
  if (residual != nullptr) {
    const int64_t m = rows * res_width;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += stride)
      residual[i] += ls_to_float<TB>(res_bias[i % res_width]);
  }
}

LS_API int ls_clamped_glu(const void* gate_up, long long in_ld, int in_dtype, const void* bias, int bias_dtype, void* out,
                          int out_dtype, int rows, int width, float limit, float alpha, float* residual,
                          const void* res_bias, int res_width, float up_offset, int gelu, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || in_ld < 2 * (long long)width || (residual != nullptr && (res_bias == nullptr || res_width <= 0)))
    return LS_E_SIZE;
  // (gate_up may be some columns of a wider row: in_ld is its row pitch in elements)
  const int in_bytes = in_dtype == LS_F32 ? 4 : 2;
  const int vec = (width & 3) == 0 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                  (in_ld * in_bytes) % 16 == 0;
  const int64_t n = (int64_t)rows * (width / (vec ? 4 : 1) > res_width ? width / (vec ? 4 : 1) : res_width);
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  LS_COUNT(LS_K_CLAMPED_GLU);
#define LS_GLU(TI, TO, TB)                                                                                        \
  ls_launch(clamped_glu_kernel<TI, TO, TB>, blocks, 256, 0, stream, (const TI*)gate_up, (const TB*)bias, (TO*)out, \
            (int64_t)rows, width, (int64_t)in_ld, limit, alpha, residual, (const TB*)res_bias, res_width, vec, up_offset, gelu)
  if (in_dtype == LS_F32 && out_dtype == LS_F32 && bias_dtype == LS_F32) LS_GLU(float, float, float);
  else if (in_dtype == LS_F32 && out_dtype == LS_BF16 && bias_dtype == LS_BF16) LS_GLU(float, __nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == LS_F32 && out_dtype == LS_BF16 && bias_dtype == LS_F32) LS_GLU(float, __nv_bfloat16, float);
  else if (in_dtype == LS_BF16 && out_dtype == LS_BF16 && bias_dtype == LS_BF16) LS_GLU(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == LS_BF16 && out_dtype == LS_BF16 && bias_dtype == LS_F32) LS_GLU(__nv_bfloat16, __nv_bfloat16, float);
  else return LS_E_DTYPE;
#undef LS_GLU
  return ls_launch_status();
}

// --------------------------------------------------------------------------
// rows of a float32 tensor set to a bias vector (or to zero), or the bias added to them:
// what a product that adds itself into its output starts from.
//   mode 0: x[r, :] = bias (zero where bias is null); mode 1: x[r, :] += bias
// --------------------------------------------------------------------------
template <typename TB>
__global__ void row_bias_kernel(float* __restrict__ x, const TB* __restrict__ bias, int64_t rows, int width, int mode) {
  ls_dependency_sync();
  const int64_t n = rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float b = bias != nullptr ? ls_to_float<TB>(bias[i % width]) : 0.f;
    x[i] = mode == 0 ? b : x[i] + b;
  }
}

LS_API int ls_row_bias(float* x, const void* bias, int bias_dtype, int rows, int width, int mode, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || (mode != 0 && mode != 1) || (mode == 1 && bias == nullptr)) return LS_E_SIZE;
  const int64_t n = (int64_t)rows * width;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  LS_COUNT(LS_K_ROW_BIAS);
  if (bias_dtype == LS_F32) ls_launch(row_bias_kernel<float>, blocks, 256, 0, stream, x, (const float*)bias, (int64_t)rows, width, mode);
  else if (bias_dtype == LS_BF16) ls_launch(row_bias_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, (const __nv_bfloat16*)bias, (int64_t)rows, width, mode);
  else return LS_E_DTYPE;
  return ls_launch_status();
}

// --------------------------------------------------------------------------
// residual += sum_b scale[b] * branch[b]  (float32; branches [n, count] one after the other):
// the results of mixers that run side by side on the same input, each with a weight of its own
// --------------------------------------------------------------------------
constexpr int MAX_BRANCHES = 4;
struct LsBranchScales { float s[MAX_BRANCHES]; };
__global__ void weighted_sum_kernel(float* __restrict__ residual, const float* __restrict__ branches, int64_t count,
                                    int n, LsBranchScales scales, const float* __restrict__ bias, int width) {
  ls_dependency_sync();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
    // bias (or null) [width]: the branches' output biases, already weighted and summed
    float sum = bias != nullptr ? bias[i % width] : 0.f;
#pragma unroll
    for (int b = 0; b < MAX_BRANCHES; ++b)
      if (b < n) sum = fmaf(scales.s[b], branches[(int64_t)b * count + i], sum);
    residual[i] += sum;
  }
}

LS_API int ls_weighted_sum(float* residual, const float* branches, long long count, int n, const float* scales,
                           const float* bias, int width, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (n <= 0 || n > MAX_BRANCHES || (bias != nullptr && width <= 0)) return LS_E_SIZE;
  LsBranchScales s;
  for (int b = 0; b < MAX_BRANCHES; ++b) s.s[b] = b < n ? scales[b] : 0.f;
  const int blocks = (int)((count + 255) / 256 < 148 * 16 ? (count + 255) / 256 : 148 * 16);
  LS_COUNT(LS_K_WEIGHTED_SUM);
  ls_launch(weighted_sum_kernel, blocks, 256, 0, stream, residual, branches, (int64_t)count, n, s, bias, width > 0 ? width : 1);
  return ls_launch_status();
}

// --------------------------------------------------------------------------
// The closing kernel of a layer whose sublayers run side by side on one normed row y:
//   residual[t, c] += sum_b gate_b[t, c] * branch[b, t, c],  gate_b = sigmoid(z[t, b * width + c] + bias[b * width + c])
// (float32; z the float32 result of the gates' product, or null for no gates), the sum made from
// zero in the order of the branches and then added to the stream.  With `carry`, the row y[t] of
// every token that is the last of its request's portion goes to carry[slot[t], :] in float32: what
// the next step's first token of that request is shifted towards.
// --------------------------------------------------------------------------
// (VEC = 4: four columns a thread with 16-byte loads, where the width is a multiple of four and every row
// starts on a 16-byte boundary; the arithmetic of a column is the same.)
template <typename TY, int VEC>
__global__ void __launch_bounds__(256) gated_sum_kernel(float* __restrict__ residual, const float* __restrict__ branches,
                                                        int n, const float* __restrict__ z, const float* __restrict__ bias,
                                                        int tokens, int width, const TY* __restrict__ y,
                                                        float* __restrict__ carry, int64_t carry_stride,
                                                        const int* __restrict__ token_slot) {
  ls_dependency_sync();
  const int t = blockIdx.x;
  const int64_t count = (int64_t)tokens * width;
  bool keep = false;
  int slot = 0;
  if (carry != nullptr) {
    slot = token_slot[t];
    keep = t + 1 == tokens || token_slot[t + 1] != slot;
  }
  for (int c = threadIdx.x * VEC; c < width; c += 256 * VEC) {
    const int64_t at = (int64_t)t * width + c;
    float sum[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) sum[i] = 0.f;
    for (int b = 0; b < n; ++b) {
      float v[VEC], logit[VEC], add[VEC];
      if constexpr (VEC == 4) {
        const float4 q = *reinterpret_cast<const float4*>(branches + (int64_t)b * count + at);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
      } else {
        v[0] = branches[(int64_t)b * count + at];
      }
      if (z != nullptr) {
        if constexpr (VEC == 4) {
          const float4 l = *reinterpret_cast<const float4*>(z + (int64_t)t * n * width + (int64_t)b * width + c);
          const float4 o = *reinterpret_cast<const float4*>(bias + b * width + c);
          logit[0] = l.x; logit[1] = l.y; logit[2] = l.z; logit[3] = l.w;
          add[0] = o.x; add[1] = o.y; add[2] = o.z; add[3] = o.w;
        } else {
          logit[0] = z[(int64_t)t * n * width + (int64_t)b * width + c];
          add[0] = bias[b * width + c];
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = v[i] * (1.0f / (1.0f + expf(-(logit[i] + add[i]))));
      }
#pragma unroll
      for (int i = 0; i < VEC; ++i) sum[i] += v[i];
    }
    if constexpr (VEC == 4) {
      float4 r = *reinterpret_cast<float4*>(residual + at);
      r.x += sum[0]; r.y += sum[1]; r.z += sum[2]; r.w += sum[3];
      *reinterpret_cast<float4*>(residual + at) = r;
    } else {
      residual[at] += sum[0];
    }
    if (keep) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) carry[(int64_t)slot * carry_stride + c + i] = ls_to_float<TY>(y[at + i]);
    }
  }
}

template <typename TY>
static void gated_sum_launch(float* residual, const float* branches, int n, const float* z, const float* bias, int tokens,
                             int width, const TY* y, float* carry, int64_t carry_stride, const int* token_slot,
                             cudaStream_t stream) {
  auto aligned = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (width % 4 == 0 && aligned(residual) && aligned(branches) && aligned(z) && aligned(bias))
    ls_launch(gated_sum_kernel<TY, 4>, dim3(tokens), dim3(256), 0, stream, residual, branches, n, z, bias, tokens, width, y,
              carry, carry_stride, token_slot);
  else
    ls_launch(gated_sum_kernel<TY, 1>, dim3(tokens), dim3(256), 0, stream, residual, branches, n, z, bias, tokens, width, y,
              carry, carry_stride, token_slot);
}

LS_API int ls_gated_sum(float* residual, const float* branches, int n, const float* z, const float* bias, int tokens,
                        int width, const void* y, int y_dtype, float* carry, long long carry_stride,
                        const int* token_slot, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n <= 0 || width <= 0 || (z != nullptr && bias == nullptr)) return LS_E_SIZE;
  if (carry != nullptr && (y == nullptr || token_slot == nullptr || carry_stride < width)) return LS_E_SIZE;
  LS_COUNT(LS_K_GATED_SUM);
  if (y_dtype == LS_F32)
    gated_sum_launch<float>(residual, branches, n, z, bias, tokens, width, (const float*)y, carry, (int64_t)carry_stride,
                            token_slot, stream);
  else if (y_dtype == LS_BF16)
    gated_sum_launch<__nv_bfloat16>(residual, branches, n, z, bias, tokens, width, (const __nv_bfloat16*)y, carry,
                                    (int64_t)carry_stride, token_slot, stream);
  else return LS_E_DTYPE;
  return ls_launch_status();
}

// --------------------------------------------------------------------------
// RMSNorm and token shift in one pass over the rows:
//   y[t] = h[t] * rsqrt(mean(h[t]^2) + eps) * gain,   x[t] = y[t] + (before - y[t]) * mu
// with `before` = y[t - 1] where token t - 1 belongs to the same slot (its norm is made again here, with the
// same sums), else the row carried in carry[slot[t]] from the step before (zeros for a new request).  A
// warp per row; the sums, products and roundings are those of rmsnorm_kernel followed by the shift of the
// rounded rows, so the bits are the same.
// --------------------------------------------------------------------------
template <typename TO, typename TG>
__global__ void __launch_bounds__(128)
rmsnorm_shift_kernel(const float* __restrict__ h, const TG* __restrict__ gain, const float* __restrict__ mu,
                     const float* __restrict__ carry, int64_t carry_stride, const int* __restrict__ token_slot,
                     TO* __restrict__ y, TO* __restrict__ x, int tokens, int width, float eps) {
  ls_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int slot = token_slot[t];
  const bool inside = t > 0 && token_slot[t - 1] == slot;
  const float* cur = h + (int64_t)t * width;
  const float* prev = h + (int64_t)(inside ? t - 1 : t) * width;
  const float* kept = carry + (int64_t)slot * carry_stride;
  const bool vec = (width & 3) == 0 && ((uintptr_t)h & 15) == 0;
  const bool vec_out = vec && ((uintptr_t)y & (4 * sizeof(TO) - 1)) == 0 && ((uintptr_t)x & (4 * sizeof(TO) - 1)) == 0 &&
                       ((uintptr_t)gain & (4 * sizeof(TG) - 1)) == 0 && ((uintptr_t)mu & 15) == 0 &&
                       ((uintptr_t)kept & 15) == 0 && (carry_stride & 3) == 0;
  auto sum_squares = [&](const float* r) {
    float ss = 0.f;
    if (vec) {
      for (int g = lane; g < (width >> 2); g += 32) {
        const float4 v = *reinterpret_cast<const float4*>(r + 4 * g);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
      }
    } else {
      for (int i = lane; i < width; i += 32) ss = fmaf(r[i], r[i], ss);
    }
    return ls_warp_sum(ss);
  };
  const float rstd = 1.0f / sqrtf(sum_squares(cur) / (float)width + eps);
  const float rstd_prev = inside ? 1.0f / sqrtf(sum_squares(prev) / (float)width + eps) : 0.f;
  auto rounded = [](float v) { return ls_to_float<TO>(ls_from_float<TO>(v)); };
  if (vec_out) {
    for (int g = lane; g < (width >> 2); g += 32) {
      const int c = 4 * g;
      const float4 v = *reinterpret_cast<const float4*>(cur + c);
      const float4 gn = ls_load4<TG>(gain + c);
      const float4 m = *reinterpret_cast<const float4*>(mu + c);
      const float own[4] = {rounded(v.x * rstd * gn.x), rounded(v.y * rstd * gn.y), rounded(v.z * rstd * gn.z),
                            rounded(v.w * rstd * gn.w)};
      float before[4];
      if (inside) {
        const float4 p = *reinterpret_cast<const float4*>(prev + c);
        before[0] = rounded(p.x * rstd_prev * gn.x); before[1] = rounded(p.y * rstd_prev * gn.y);
        before[2] = rounded(p.z * rstd_prev * gn.z); before[3] = rounded(p.w * rstd_prev * gn.w);
      } else {
        const float4 p = *reinterpret_cast<const float4*>(kept + c);
        before[0] = p.x; before[1] = p.y; before[2] = p.z; before[3] = p.w;
      }
      ls_store4<TO>(y + (int64_t)t * width + c, own[0], own[1], own[2], own[3]);
      ls_store4<TO>(x + (int64_t)t * width + c, fmaf(before[0] - own[0], m.x, own[0]), fmaf(before[1] - own[1], m.y, own[1]),
                    fmaf(before[2] - own[2], m.z, own[2]), fmaf(before[3] - own[3], m.w, own[3]));
    }
  } else {
    for (int c = lane; c < width; c += 32) {
      const float gn = ls_to_float<TG>(gain[c]);
      const float own = rounded(cur[c] * rstd * gn);
      const float before = inside ? rounded(prev[c] * rstd_prev * gn) : kept[c];
      y[(int64_t)t * width + c] = ls_from_float<TO>(own);
      x[(int64_t)t * width + c] = ls_from_float<TO>(fmaf(before - own, mu[c], own));
    }
  }
}

LS_API int ls_rmsnorm_shift(const float* h, const void* gain, int gain_dtype, const float* mu, const float* carry,
                            long long carry_stride, const int* token_slot, void* y, void* x, int out_dtype, int tokens,
                            int width, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || carry_stride < width) return LS_E_SIZE;
  const int warps = tokens >= 1024 ? 4 : 1;
  const int blocks = (tokens + warps - 1) / warps;
  LS_COUNT(LS_K_RMSNORM_SHIFT);
#define LS_RMS_SHIFT(TO, TG)                                                                                          \
  ls_launch(rmsnorm_shift_kernel<TO, TG>, blocks, warps * 32, 0, stream, h, (const TG*)gain, mu, carry,               \
            (int64_t)carry_stride, token_slot, (TO*)y, (TO*)x, tokens, width, eps)
  if (out_dtype == LS_F32 && gain_dtype == LS_F32) LS_RMS_SHIFT(float, float);
  else if (out_dtype == LS_F32 && gain_dtype == LS_BF16) LS_RMS_SHIFT(float, __nv_bfloat16);
  else if (out_dtype == LS_BF16 && gain_dtype == LS_F32) LS_RMS_SHIFT(__nv_bfloat16, float);
  else if (out_dtype == LS_BF16 && gain_dtype == LS_BF16) LS_RMS_SHIFT(__nv_bfloat16, __nv_bfloat16);
  else return LS_E_DTYPE;
#undef LS_RMS_SHIFT
  return ls_launch_status();
}

// Switches programmatic dependent launch of this library's kernels on or off.
LS_API void ls_set_dependent_launch_core(int on) { ls_dependent_launch = on ? 1 : 0; }
