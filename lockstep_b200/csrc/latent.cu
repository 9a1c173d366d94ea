// Attention over a cached latent: what lies between the projections and the attention kernels.
//
// A token's keys and values are functions of one small vector c (the latent, `rank` elements,
// RMS-normed) and of one rotated key part k_r (`dr` elements) that all heads share:
//   key of head h   = [W_uk,h c ; k_r],   value of head h = W_uv,h c.
// Only [c ; k_r] is cached.  A query head's score with a cached token is then
//   q_plain,h . (W_uk,h c) + q_rot,h . k_r = [W_uk,h^T q_plain,h ; q_rot,h] . [c ; k_r],
// so the attention kernels see one key head of size D >= rank + dr that every query head reads,
// with values [c ; 0]; the head's output sum_j p_j c_j goes through W_uv,h afterwards.
//
//   latent_finish:  a block per token: norm of c, rotation of k_r and of every head's q_rot, the
//                   cache write ([c ; k_r ; 0] as the key row, [c ; 0] as the value row) and the
//                   rotated and padded part of the folded queries.
//   heads_product:  out[t, h, :] = a[t, h, :] @ w[h]^T for every head at once (the fold of W_uk into
//                   the queries, and W_uv on the attention's output), an element one chain of fused
//                   multiply-adds over ascending k, so a row's bits do not depend on the batch.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

struct LatentArgs {
  const void* proj;        // [tokens, ld]: H heads of [d plain ; dr rotated] queries
  int64_t ld;
  const void* kv;          // [tokens, kv_ld]: [rank ; dr] of the keys' side (null for a layer that writes no cache)
  int64_t kv_ld;
  void* q_out;             // [tokens, H, D]: this kernel writes columns rank .. D of every head
  void* pages;             // [num_pages, 2, 1, page_size, D]
  const void* gain;        // [rank]
  int gain_bf16;
  const float* cos_table;  // [max_positions, dr / 2]
  const float* sin_table;
  const int* positions;
  const int* token_req;
  const int* block_table;
  int table_stride, H, d, dr, rank, D, page_size, num_pages, max_positions, interleaved, write_cache;
  float eps;
  const void* w_fold;      // null, or [H, rank, d]: this kernel also folds W_uk into the queries (few tokens)
};

// element i of a rotated vector x[0 .. dr): pairs (2j, 2j+1) when interleaved, else (j, j + dr/2);
// products and sums rounded one by one
template <typename T>
__device__ __forceinline__ float rotated(const T* x, int i, int dr, int interleaved, const float* cs, const float* sn) {
  const int half = dr >> 1;
  int j, lo, hi;
  bool first;
  if (interleaved) {
    j = i >> 1; lo = 2 * j; hi = lo + 1; first = (i & 1) == 0;
  } else {
    j = i < half ? i : i - half; lo = j; hi = j + half; first = i < half;
  }
  const float u = ls_to_float<T>(x[lo]), v = ls_to_float<T>(x[hi]);
  return first ? __fsub_rn(__fmul_rn(u, cs[j]), __fmul_rn(v, sn[j]))
               : __fadd_rn(__fmul_rn(v, cs[j]), __fmul_rn(u, sn[j]));
}

template <typename T>
__global__ void __launch_bounds__(THREADS) latent_finish_kernel(LatentArgs a, int* err) {
  __shared__ float scratch[32];
  extern __shared__ float q_plain[];       // with w_fold: the plain query part [d] of this block's head
  ls_dependency_sync();
  const int t = blockIdx.x;
  const T* row = reinterpret_cast<const T*>(a.proj) + (int64_t)t * a.ld;
  const int pos = a.positions[t];
  const int half = a.dr >> 1;
  if (half > 0 && (pos < 0 || pos >= a.max_positions)) {
    if (threadIdx.x == 0) ls_record_fault(err, LS_DEV_POSITION_RANGE, t);
    return;
  }
  const float* cs = a.cos_table + (int64_t)pos * half;
  const float* sn = a.sin_table + (int64_t)pos * half;
  const int qd = a.d + a.dr, tail = a.D - a.rank;
  // queries: the rotated part of every head behind the columns the fold will fill, then zeros
  T* q_dst = reinterpret_cast<T*>(a.q_out) + (int64_t)t * a.H * a.D;
  for (int e = threadIdx.x; e < a.H * tail && blockIdx.y == 0; e += THREADS) {
    const int h = e / tail, i = e - h * tail;
    const float v = i < a.dr ? rotated<T>(row + h * qd + a.d, i, a.dr, a.interleaved, cs, sn) : 0.f;
    q_dst[h * a.D + a.rank + i] = ls_from_float<T>(v);
  }
  if (a.w_fold != nullptr) {
    // columns 0 .. rank of head blockIdx.y: W_uk,h^T q_plain,h, an element one chain of fused multiply-adds
    // over ascending k from zero, as heads_product makes it (the same bits), for a step of few tokens; the
    // weights come 16 bytes at a time where the rows allow it, several loads in flight
    const int h = blockIdx.y;
    for (int e = threadIdx.x; e < a.d; e += THREADS) q_plain[e] = ls_to_float<T>(row[h * qd + e]);
    __syncthreads();
    const T* w = reinterpret_cast<const T*>(a.w_fold) + (int64_t)h * a.rank * a.d;
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool wide = a.d % VEC == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    for (int r = threadIdx.x; r < a.rank; r += THREADS) {
      const T* wr = w + (int64_t)r * a.d;
      float acc = 0.f;
      if (wide) {
        for (int k0 = 0; k0 < a.d; k0 += 4 * VEC) {
          uint4 raw[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            raw[u] = k0 + u * VEC < a.d ? *reinterpret_cast<const uint4*>(wr + k0 + u * VEC) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (k0 + u * VEC >= a.d) break;
            const T* wv = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
            for (int x = 0; x < VEC; ++x) acc = fmaf(q_plain[k0 + u * VEC + x], ls_to_float<T>(wv[x]), acc);
          }
        }
      } else {
        for (int k = 0; k < a.d; ++k) acc = fmaf(q_plain[k], ls_to_float<T>(wr[k]), acc);
      }
      q_dst[h * a.D + r] = ls_from_float<T>(acc);
    }
  }
  if (blockIdx.y != 0) return;
  if (!a.write_cache) return;
  const int req = a.token_req[t];
  const int page = a.block_table[(int64_t)req * a.table_stride + pos / a.page_size];
  if (page < 0 || page >= a.num_pages) {
    if (threadIdx.x == 0) ls_record_fault(err, LS_DEV_PAGE_RANGE, t);
    return;
  }
  const T* c = reinterpret_cast<const T*>(a.kv) + (int64_t)t * a.kv_ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < a.rank; i += THREADS) {
    const float v = ls_to_float<T>(c[i]);
    ss = fmaf(v, v, ss);
  }
  const float rstd = 1.0f / sqrtf(ls_block_sum(ss, scratch) / (float)a.rank + a.eps);
  T* pages = reinterpret_cast<T*>(a.pages);
  T* k_row = pages + (((int64_t)page * 2 + 0) * a.page_size + pos % a.page_size) * a.D;
  T* v_row = pages + (((int64_t)page * 2 + 1) * a.page_size + pos % a.page_size) * a.D;
  for (int i = threadIdx.x; i < a.D; i += THREADS) {
    float k = 0.f, v = 0.f;
    if (i < a.rank) {
      const float g = a.gain_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.gain)[i])
                                  : reinterpret_cast<const float*>(a.gain)[i];
      k = v = __fmul_rn(__fmul_rn(ls_to_float<T>(c[i]), rstd), g);
    } else if (i < a.rank + a.dr) {
      k = rotated<T>(c + a.rank, i - a.rank, a.dr, a.interleaved, cs, sn);
    }
    k_row[i] = ls_from_float<T>(k);
    v_row[i] = ls_from_float<T>(v);
  }
}

// ---------------------------------------------------------------------------------------
// out[t, h * out_hs + n] = sum_k a[t * a_ld + h * a_hs + k] * w[(h * N + n) * K + k]
// 64 x 64 outputs a block, 32 of k at a time, 4 x 4 outputs a thread.  Where the rows allow it
// (`vec`: pitches, head strides and K multiples of a 16-byte piece, aligned bases) both operands
// come 16 bytes a load, consecutive threads taking consecutive rows, so that the transposed
// stores into shared memory fall into different banks.
// ---------------------------------------------------------------------------------------
constexpr int HP_T = 64, HP_N = 64, HP_K = 32;

// 64 rows x HP_K columns of `src` (row r at src + r * ld, rows past `rows` and columns past K as zeros)
// into tile[k][r]
template <typename T>
__device__ __forceinline__ void hp_load_tile(float (*tile)[HP_T + 4], const T* __restrict__ src, int64_t ld, int rows,
                                             int k0, int K, int vec, int tid) {
  constexpr int VEC = 16 / (int)sizeof(T);
  if (vec) {
    for (int p = tid; p < 64 * (HP_K / VEC); p += 256) {
      const int r = p & 63, c = (p >> 6) * VEC;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);             // zero bits are 0.0 in either type
      if (r < rows && k0 + c < K) raw = *reinterpret_cast<const uint4*>(src + (int64_t)r * ld + k0 + c);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int x = 0; x < VEC; ++x) tile[c + x][r] = ls_to_float<T>(v[x]);
    }
  } else {
    for (int e = tid; e < 64 * HP_K; e += 256) {
      const int r = e / HP_K, k = e - r * HP_K;
      tile[k][r] = (r < rows && k0 + k < K) ? ls_to_float<T>(src[(int64_t)r * ld + k0 + k]) : 0.f;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) heads_product_kernel(const T* __restrict__ a, int64_t a_ld, int a_hs,
                                                            const T* __restrict__ w, T* __restrict__ out, int64_t out_ld,
                                                            int out_hs, int tokens, int N, int K, int vec) {
  __shared__ __align__(16) float As[HP_K][HP_T + 4];
  __shared__ __align__(16) float Ws[HP_K][HP_N + 4];
  ls_dependency_sync();
  const int h = blockIdx.z, t0 = blockIdx.x * HP_T, n0 = blockIdx.y * HP_N;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;     // outputs: tokens ty * 4 .., columns tx * 4 ..
  const T* ah = a + (int64_t)h * a_hs + (int64_t)t0 * a_ld;
  const T* wh = w + ((int64_t)h * N + n0) * K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HP_K) {
    __syncthreads();
    hp_load_tile<T>(As, ah, a_ld, tokens - t0, k0, K, vec, tid);
    hp_load_tile<T>(Ws, wh, K, N - n0, k0, K, vec, tid);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HP_K; ++k) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 w4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float av[4] = {a4.x, a4.y, a4.z, a4.w}, wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(int64_t)t * out_ld + (int64_t)h * out_hs + n] = ls_from_float<T>(acc[i][j]);
    }
  }
}

}  // namespace

LS_API int ls_latent_finish(const void* proj, int64_t ld, const void* kv, int64_t kv_ld, int dtype, void* q_out,
                            void* pages, const void* gain,
                            int gain_dtype, const float* cos_table, const float* sin_table, const int* positions,
                            const int* token_req, const int* block_table, int table_stride, int tokens, int H, int d,
                            int dr, int rank, int D, int page_size, int num_pages, int max_positions, int interleaved,
                            int write_cache, float eps, const void* w_fold, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || d <= 0 || dr < 0 || (dr & 1) || rank <= 0 || D < rank + dr) return LS_E_SIZE;
  if (ld < (int64_t)H * (d + dr)) return LS_E_SIZE;
  if (gain_dtype != LS_F32 && gain_dtype != LS_BF16) return LS_E_DTYPE;
  if (write_cache && (pages == nullptr || page_size <= 0 || kv == nullptr || kv_ld < rank + dr || gain == nullptr))
    return LS_E_SIZE;
  if (dr > 0 && (cos_table == nullptr || sin_table == nullptr)) return LS_E_SIZE;
  LatentArgs a;
  a.proj = proj; a.ld = ld; a.kv = kv; a.kv_ld = kv_ld; a.q_out = q_out; a.pages = pages; a.gain = gain; a.gain_bf16 = gain_dtype == LS_BF16 ? 1 : 0;
  a.cos_table = cos_table; a.sin_table = sin_table; a.positions = positions; a.token_req = token_req;
  a.block_table = block_table; a.table_stride = table_stride; a.H = H; a.d = d; a.dr = dr; a.rank = rank; a.D = D;
  a.page_size = page_size > 0 ? page_size : 1; a.num_pages = num_pages; a.max_positions = max_positions;
  a.interleaved = interleaved; a.write_cache = write_cache; a.eps = eps; a.w_fold = w_fold;
  const size_t smem = w_fold != nullptr ? sizeof(float) * (size_t)d : 0;
  if (smem > 40 * 1024 || (w_fold != nullptr && H > 65535)) return LS_E_SMEM;
  const dim3 grid(tokens, w_fold != nullptr ? H : 1);
  LS_COUNT(LS_K_LATENT_FINISH);
  cudaError_t e;
  if (dtype == LS_F32) e = ls_launch(latent_finish_kernel<float>, grid, dim3(THREADS), smem, stream, a, err);
  else if (dtype == LS_BF16) e = ls_launch(latent_finish_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream, a, err);
  else return LS_E_DTYPE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API int ls_heads_product(const void* a, int64_t a_ld, int a_hs, const void* w, void* out, int64_t out_ld, int out_hs,
                            int dtype, int tokens, int heads, int N, int K, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || heads > 65535 || N <= 0 || K <= 0) return LS_E_SIZE;
  const dim3 grid((tokens + HP_T - 1) / HP_T, (N + HP_N - 1) / HP_N, heads);
  if (grid.y > 65535) return LS_E_SIZE;
  LS_COUNT(LS_K_HEADS_PRODUCT);
  if (dtype != LS_F32 && dtype != LS_BF16) return LS_E_DTYPE;
  const int piece = dtype == LS_F32 ? 4 : 8;            // elements of 16 bytes
  const int vec = a_ld % piece == 0 && a_hs % piece == 0 && K % piece == 0 && ((uintptr_t)a & 15) == 0 &&
                  ((uintptr_t)w & 15) == 0;
  cudaError_t e;
  if (dtype == LS_F32)
    e = ls_launch(heads_product_kernel<float>, grid, dim3(256), 0, stream, (const float*)a, a_ld, a_hs, (const float*)w,
                  (float*)out, out_ld, out_hs, tokens, N, K, vec);
  else if (dtype == LS_BF16)
    e = ls_launch(heads_product_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)a, a_ld, a_hs,
                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_ld, out_hs, tokens, N, K, vec);
  else return LS_E_DTYPE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}
