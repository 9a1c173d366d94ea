// A feed-forward of routed experts: router scores, the choice of the top experts per token,
// the step's (token, choice) pairs sorted by expert, the experts' two products over the
// sorted rows, and the sum of a token's choices into the residual stream.
//
// Router logits arrive as float32 [tokens, experts].  The score is the sigmoid of the logit, or
// the softmax over all experts; the `top` largest scores (plus an optional correction per expert
// that only the choice sees) are chosen (ties to the lower index) and kept in order of rank; the
// weight is the score itself.  The last experts may be identities, which have no weights and no
// rows in the sorted order: the sum takes the token's own row for them.  A pair's
// row in the sorted order is handed out by a counter per expert, so which row a pair gets
// may differ from run to run, but no value depends on it: every element of a product is one
// chain of fused multiply-adds over ascending k, whatever tile its row lies in, and a token's
// choices are added in order of rank.
#include "common.cuh"

namespace {

constexpr int MAX_PER_LANE = 16;      // experts a lane looks after: up to 512 experts
constexpr int ROUTE_WARPS = 8;
constexpr int PLAN_THREADS = 1024;
constexpr int TILE_M = 64, TILE_N = 64, TILE_K = 16;

// ids [T, top] int32, weights [T, top] float32.  logits [T, ld]: the first `experts` columns of a row.
// softmax 0: weight = sigmoid(logit); 1: weight = softmax over the `experts` logits (the largest taken off, the
// exponentials summed lane by lane over ascending experts, then by an xor tree: an order the token alone fixes).
// correction (or null) [experts]: added to the weight for the choice only.
// (one warp: token t)
__device__ __forceinline__ void route_token(const float* __restrict__ logits, int64_t ld, int t, int experts, int top,
                                            int softmax, const float* __restrict__ correction, int* __restrict__ ids,
                                            float* __restrict__ weights) {
  const int lane = threadIdx.x & 31;
  float z[MAX_PER_LANE];     // the expert's score
  float pick[MAX_PER_LANE];  // what the choice compares
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    z[i] = e < experts ? logits[(int64_t)t * ld + e] : -INFINITY;
  }
  if (softmax == 2) {
    // the scores are the logits themselves; the weights become a softmax over the chosen ones below
  } else if (softmax) {
    float top_z = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) top_z = fmaxf(top_z, z[i]);
    top_z = ls_warp_max(top_z);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      z[i] = lane + 32 * i < experts ? expf(z[i] - top_z) : 0.f;
      sum += z[i];
    }
    sum = ls_warp_sum(sum);
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) z[i] = z[i] / sum;
  } else {
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) z[i] = 1.0f / (1.0f + expf(-z[i]));
  }
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    pick[i] = e < experts ? (correction != nullptr ? z[i] + correction[e] : z[i]) : -INFINITY;
  }
  unsigned taken = 0;
  for (int r = 0; r < top; ++r) {
    float best = -INFINITY, best_z = 0.f;
    int at = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && !((taken >> i) & 1u) && (pick[i] > best || (pick[i] == best && e < at))) {
        best = pick[i];
        best_z = z[i];
        at = e;
      }
    }
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const float oz = __shfl_xor_sync(0xffffffffu, best_z, off);
      const int oa = __shfl_xor_sync(0xffffffffu, at, off);
      if (ob > best || (ob == best && oa < at)) {
        best = ob;
        best_z = oz;
        at = oa;
      }
    }
    if ((at & 31) == lane) taken |= 1u << (at >> 5);
    if (lane == 0) {
      ids[(int64_t)t * top + r] = at;
      weights[(int64_t)t * top + r] = best_z;
    }
  }
  if (softmax == 2 && lane == 0) {
    // softmax over the chosen logits alone (the first is the largest), summed in order of rank
    float* w = weights + (int64_t)t * top;
    const float top_z = w[0];
    float sum = 0.f;
    for (int r = 0; r < top; ++r) {
      w[r] = expf(w[r] - top_z);
      sum += w[r];
    }
    for (int r = 0; r < top; ++r) w[r] = w[r] / sum;
  }
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_kernel(const float* __restrict__ logits, int64_t ld, int tokens,
                                                                 int experts, int top, int softmax,
                                                                 const float* __restrict__ correction,
                                                                 int* __restrict__ ids, float* __restrict__ weights) {
  ls_dependency_sync();
  const int t = blockIdx.x * ROUTE_WARPS + (threadIdx.x >> 5);
  if (t >= tokens) return;
  route_token(logits, ld, t, experts, top, softmax, correction, ids, weights);
}

// plan [0] = tiles, then (expert, first row, rows) per tile; row_token / row_weight per sorted
// row; pair_row [T * top]: the sorted row of a pair.  The work of one block of any size.
// (ids and weights are not marked restrict: the kernel that also makes them writes them before this reads them)
__device__ __forceinline__ void plan_block(const int* ids, const float* weights, int pairs,
                                           int top, int experts, int tile_rows, int* __restrict__ plan, int max_tiles,
                                           int* __restrict__ row_token, float* __restrict__ row_weight,
                                           int* __restrict__ pair_row, int* err) {
  // (ids outside 0 .. experts - 1 get no row: the caller's identity experts)
  extern __shared__ int sm[];
  int* count = sm;                  // [experts]
  int* first = count + experts;     // [experts]
  int* cursor = first + experts;    // [experts]
  __shared__ int sorted_rows;
  const int tid = threadIdx.x;
  const int PLAN_THREADS = blockDim.x;
  for (int e = tid; e < experts; e += PLAN_THREADS) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = tid; p < pairs; p += PLAN_THREADS) {
    const int e = ids[p];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      first[e] = at;
      for (int r0 = 0; r0 < count[e]; r0 += tile_rows) {
        if (tiles < max_tiles) {
          plan[1 + 3 * tiles] = e;
          plan[1 + 3 * tiles + 1] = at + r0;
          plan[1 + 3 * tiles + 2] = count[e] - r0 < tile_rows ? count[e] - r0 : tile_rows;
        }
        ++tiles;
      }
      at += count[e];
    }
    sorted_rows = at;
    if (tiles > max_tiles) {
      ls_record_fault(err, LS_DEV_ROW_RANGE, tiles);
      tiles = max_tiles;
    }
    plan[0] = tiles;
  }
  __syncthreads();
  for (int p = tid; p < pairs; p += PLAN_THREADS) {
    const int e = ids[p];
    if (e < 0 || e >= experts) continue;
    const int row = first[e] + atomicAdd(&cursor[e], 1);
    row_token[row] = p / top;
    row_weight[row] = weights[p];
    pair_row[p] = row;
  }
  // pairs whose expert has no rows (an identity expert) leave the sorted order shorter than the lists:
  // the rows past its end name token 0 with the weight zero, so that a kernel that walks all rows of
  // the lists reads nothing outside the step's tokens
  for (int row = sorted_rows + tid; row < pairs; row += PLAN_THREADS) {
    row_token[row] = 0;
    row_weight[row] = 0.f;
  }
}

__global__ void __launch_bounds__(PLAN_THREADS) plan_kernel(const int* __restrict__ ids, const float* __restrict__ weights,
                                                            int pairs, int top, int experts, int tile_rows,
                                                            int* __restrict__ plan, int max_tiles,
                                                            int* __restrict__ row_token,
                                                            float* __restrict__ row_weight, int* __restrict__ pair_row,
                                                            int* err) {
  ls_dependency_sync();
  plan_block(ids, weights, pairs, top, experts, tile_rows, plan, max_tiles, row_token, row_weight, pair_row, err);
}

// The choice and the plan of a step of few tokens in one block: its warps take the tokens in turn, then the
// block sorts the pairs.  `real`: the experts that have rows (the first of the `experts` the router scores).
__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_plan_kernel(
    const float* __restrict__ logits, int64_t ld, int tokens, int experts, int top, int softmax,
    const float* __restrict__ correction, int* ids, float* weights, int real, int tile_rows,
    int* __restrict__ plan, int max_tiles, int* __restrict__ row_token, float* __restrict__ row_weight,
    int* __restrict__ pair_row, int* err) {
  ls_dependency_sync();
  for (int t = threadIdx.x >> 5; t < tokens; t += ROUTE_WARPS)
    route_token(logits, ld, t, experts, top, softmax, correction, ids, weights);
  __syncthreads();                  // (the block's own writes to ids and weights are visible to it behind the barrier)
  plan_block(ids, weights, tokens * top, top, real, tile_rows, plan, max_tiles, row_token, row_weight, pair_row, err);
}

// One tile of an expert's product on the CUDA cores: C[rows, N] = A[rows, K] . W_e[N, K]^T.
//   MODE 0 (up):   A row = x[row_token] * row_weight, C = relu(.)^2 in the engine's type
//   MODE 1 (down): A row = act[row],                  C float32
//   MODE 2 (down, one expert a token): C[row_token[row], :] += the product, float32: the sum into
//   the residual stream, every element of which then has one writer
//   MODE 3 (up):   A row = x[row_token] (times row_weight where that is given), C float32: what an
//   activation kernel of its own reads
template <typename T, int MODE>
__global__ void __launch_bounds__(256) expert_product_kernel(const int* __restrict__ plan, const T* __restrict__ A,
                                                             const int* __restrict__ row_token,
                                                             const float* __restrict__ row_weight,
                                                             const T* __restrict__ W, void* __restrict__ Cout, int N,
                                                             int K) {
  __shared__ float As[TILE_K][TILE_M + 4];
  __shared__ float Bs[TILE_K][TILE_N + 4];
  ls_dependency_sync();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int e = plan[1 + 3 * tile], row0 = plan[1 + 3 * tile + 1], rows = plan[1 + 3 * tile + 2];
  const int n0 = blockIdx.x * TILE_N, tid = threadIdx.x;
  const T* We = W + (int64_t)e * N * K;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4] = {};
  // what this thread loads: four elements of A and of W per k-block
  const int lr = tid >> 2, lk = (tid & 3) * 4;       // row (or weight row) 0..63, k 0, 4, 8, 12
  int64_t a_row = -1;
  float a_scale = 1.f;
  constexpr bool GATHERS = MODE == 0 || MODE == 3;
  if (lr < rows) {
    a_row = GATHERS ? row_token[row0 + lr] : row0 + lr;
    if (GATHERS && row_weight != nullptr) a_scale = row_weight[row0 + lr];
  }
  const bool w_ok = n0 + lr < N;
  for (int k0 = 0; k0 < K; k0 += TILE_K) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      float av = 0.f, wv = 0.f;
      if (a_row >= 0 && k < K) {
        av = ls_to_float<T>(A[a_row * K + k]);
        if (GATHERS) av = av * a_scale;
      }
      if (w_ok && k < K) wv = ls_to_float<T>(We[(int64_t)(n0 + lr) * K + k]);
      As[lk + i][lr] = av;
      Bs[lk + i][lr] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TILE_K; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[kk][ty * 4 + i];
        b[i] = Bs[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      const int64_t at = (int64_t)(row0 + r) * N + n;
      if (MODE == 0) {
        const float v = fmaxf(acc[i][j], 0.f);
        reinterpret_cast<T*>(Cout)[at] = ls_from_float<T>(v * v);
      } else if (MODE == 1 || MODE == 3) {
        reinterpret_cast<float*>(Cout)[at] = acc[i][j];
      } else {
        float* to = reinterpret_cast<float*>(Cout) + (int64_t)row_token[row0 + r] * N + n;
        *to = *to + acc[i][j];
      }
    }
  }
}

// residual[t, :] += y[row of (t, 0), :] + y[row of (t, 1), :] + ... in order of rank
__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_row,
                                                      float* __restrict__ residual, int top, int width) {
  ls_dependency_sync();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += 256) {
    float sum = y[(int64_t)pair_row[(int64_t)t * top] * width + c];
    for (int r = 1; r < top; ++r) sum += y[(int64_t)pair_row[(int64_t)t * top + r] * width + c];
    residual[(int64_t)t * width + c] += sum;
  }
}

// The sum of a token's chosen experts, with all that may ride on it:
//   out[t, :] (+)= sum_r w[t, r] * (id[t, r] < real ? y[row of (t, r), :] : x[t, :])  +  sigmoid(gate[t]) * shared[t, :]
// in order of rank from zero, the shared expert's term last.  w null: weights of one (the scores went into
// the experts' inputs); ids >= `real` are identity experts; shared null: no shared expert; gate null: its
// weight is one.  store: out is written, else added to.
template <typename TX>
__global__ void __launch_bounds__(256) mix_kernel(const float* __restrict__ y, const int* __restrict__ pair_row,
                                                  const int* __restrict__ ids, const float* __restrict__ w, int real,
                                                  const TX* __restrict__ x, const float* __restrict__ shared,
                                                  const float* __restrict__ gate, int64_t gate_ld,
                                                  float* __restrict__ out, int top, int width, int store) {
  ls_dependency_sync();
  const int t = blockIdx.x;
  const float shared_w = shared == nullptr ? 0.f : gate == nullptr ? 1.f : 1.0f / (1.0f + expf(-gate[(int64_t)t * gate_ld]));
  for (int c = threadIdx.x; c < width; c += 256) {
    float sum = 0.f;
    for (int r = 0; r < top; ++r) {
      const int64_t p = (int64_t)t * top + r;
      const float v = ids[p] < real ? y[(int64_t)pair_row[p] * width + c] : ls_to_float<TX>(x[(int64_t)t * width + c]);
      sum = w != nullptr ? fmaf(w[p], v, sum) : sum + v;
    }
    if (shared != nullptr) sum = fmaf(shared_w, shared[(int64_t)t * width + c], sum);
    float* to = out + (int64_t)t * width + c;
    *to = store ? sum : *to + sum;
  }
}

}  // namespace

LS_API int ls_experts_tile_rows() { return TILE_M; }

LS_API int ls_experts_route(const float* logits, long long ld, int tokens, int experts, int top, int softmax,
                            const float* correction, int* ids, float* weights, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (experts <= 0 || experts > 32 * MAX_PER_LANE || top <= 0 || top > experts || ld < experts) return LS_E_SIZE;
  LS_COUNT(LS_K_EXPERTS_ROUTE);
  cudaError_t e = ls_launch(route_kernel, dim3((tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), 0, stream,
                            logits, (int64_t)ld, tokens, experts, top, softmax, correction, ids, weights);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

// Both in one launch of one block, for steps of few tokens (the same choices, weights and plan).
LS_API int ls_experts_route_plan(const float* logits, long long ld, int tokens, int experts, int top, int softmax,
                                 const float* correction, int* ids, float* weights, int real, int tile_rows, int* plan,
                                 int max_tiles, int* row_token, float* row_weight, int* pair_row, int* err,
                                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (experts <= 0 || experts > 32 * MAX_PER_LANE || top <= 0 || top > experts || ld < experts) return LS_E_SIZE;
  if (real <= 0 || real > experts || max_tiles <= 0 || tile_rows <= 0) return LS_E_SIZE;
  LS_COUNT(LS_K_EXPERTS_ROUTE);
  LS_COUNT(LS_K_EXPERTS_PLAN);
  cudaError_t e = ls_launch(route_plan_kernel, dim3(1), dim3(ROUTE_WARPS * 32), sizeof(int) * 3 * (size_t)real, stream,
                            logits, (int64_t)ld, tokens, experts, top, softmax, correction, ids, weights, real, tile_rows,
                            plan, max_tiles, row_token, row_weight, pair_row, err);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

// tile_rows: the most rows of a tile (what the product that reads the plan takes: ls_experts_tile_rows()
// for the CUDA-core product, the tensor-core product's own)
LS_API int ls_experts_plan(const int* ids, const float* weights, int tokens, int top, int experts, int tile_rows,
                           int* plan, int max_tiles, int* row_token, float* row_weight, int* pair_row, int* err,
                           cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (experts <= 0 || experts > 4096 || top <= 0 || max_tiles <= 0 || tile_rows <= 0) return LS_E_SIZE;
  LS_COUNT(LS_K_EXPERTS_PLAN);
  cudaError_t e = ls_launch(plan_kernel, dim3(1), dim3(PLAN_THREADS), sizeof(int) * 3 * (size_t)experts, stream, ids,
                            weights, tokens * top, top, experts, tile_rows, plan, max_tiles, row_token, row_weight, pair_row, err);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

// mode 0: act[rows, N] = relu(x[row_token] * row_weight . W_e^T)^2; mode 1: y[rows, N] = act . W_e^T (float32);
// mode 2: residual[row_token[row], :] += act . W_e^T (a token's one expert); mode 3: C[rows, N] = x[row_token]
// (* row_weight unless null) . W_e^T (float32).  W [experts, N, K] in the engine's type.
LS_API int ls_experts_product(int mode, int dtype, const int* plan, int max_tiles, const void* A, const int* row_token,
                              const float* row_weight, const void* W, void* C, int N, int K, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (N <= 0 || K <= 0 || max_tiles > 65535) return LS_E_SIZE;     // (the plan's tiles hold up to TILE_M rows)
  const dim3 grid((N + TILE_N - 1) / TILE_N, max_tiles);
  if (mode < 0 || mode > 3) return LS_E_SIZE;
  LS_COUNT(mode == 0 || mode == 3 ? LS_K_EXPERTS_UP : LS_K_EXPERTS_DOWN);
  cudaError_t e;
  typedef __nv_bfloat16 bf16;
  if (dtype == LS_F32 && mode == 0)
    e = ls_launch(expert_product_kernel<float, 0>, grid, dim3(256), 0, stream, plan, (const float*)A, row_token, row_weight, (const float*)W, C, N, K);
  else if (dtype == LS_F32 && mode == 1)
    e = ls_launch(expert_product_kernel<float, 1>, grid, dim3(256), 0, stream, plan, (const float*)A, row_token, row_weight, (const float*)W, C, N, K);
  else if (dtype == LS_BF16 && mode == 0)
    e = ls_launch(expert_product_kernel<bf16, 0>, grid, dim3(256), 0, stream, plan, (const bf16*)A, row_token, row_weight, (const bf16*)W, C, N, K);
  else if (dtype == LS_BF16 && mode == 1)
    e = ls_launch(expert_product_kernel<bf16, 1>, grid, dim3(256), 0, stream, plan, (const bf16*)A, row_token, row_weight, (const bf16*)W, C, N, K);
  else if (dtype == LS_F32 && mode == 2)
    e = ls_launch(expert_product_kernel<float, 2>, grid, dim3(256), 0, stream, plan, (const float*)A, row_token, row_weight, (const float*)W, C, N, K);
  else if (dtype == LS_BF16 && mode == 2)
    e = ls_launch(expert_product_kernel<bf16, 2>, grid, dim3(256), 0, stream, plan, (const bf16*)A, row_token, row_weight, (const bf16*)W, C, N, K);
  else if (dtype == LS_F32 && mode == 3)
    e = ls_launch(expert_product_kernel<float, 3>, grid, dim3(256), 0, stream, plan, (const float*)A, row_token, row_weight, (const float*)W, C, N, K);
  else if (dtype == LS_BF16 && mode == 3)
    e = ls_launch(expert_product_kernel<bf16, 3>, grid, dim3(256), 0, stream, plan, (const bf16*)A, row_token, row_weight, (const bf16*)W, C, N, K);
  else return LS_E_DTYPE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API int ls_experts_combine(const float* y, const int* pair_row, float* residual, int tokens, int top, int width,
                              cudaStream_t stream) {
  if (tokens <= 0) return 0;
  LS_COUNT(LS_K_EXPERTS_COMBINE);
  cudaError_t e = ls_launch(combine_kernel, dim3(tokens), dim3(256), 0, stream, y, pair_row, residual, top, width);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API int ls_experts_mix(const float* y, const int* pair_row, const int* ids, const float* w, int real, const void* x,
                          int x_dtype, const float* shared, const float* gate, long long gate_ld, float* out, int tokens,
                          int top, int width, int store, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (top <= 0 || width <= 0 || real < 0) return LS_E_SIZE;
  LS_COUNT(LS_K_EXPERTS_MIX);
  cudaError_t e;
  if (x_dtype == LS_F32)
    e = ls_launch(mix_kernel<float>, dim3(tokens), dim3(256), 0, stream, y, pair_row, ids, w, real, (const float*)x, shared,
                  gate, (int64_t)gate_ld, out, top, width, store);
  else if (x_dtype == LS_BF16)
    e = ls_launch(mix_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, y, pair_row, ids, w, real,
                  (const __nv_bfloat16*)x, shared, gate, (int64_t)gate_ld, out, top, width, store);
  else return LS_E_DTYPE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API const char* ls_constants_experts() {
  static char buf[256];
  static const LsConstant c[] = {{"experts.tile_rows", TILE_M}, {"experts.tile_features", TILE_N}, {"experts.k_block", TILE_K}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}
