// The routed experts' two products on the tcgen05 tensor cores (bfloat16 operands, float32
// accumulation in tensor memory).
//
// The step's (token, choice) pairs are sorted by expert (experts.cu) and cut into tiles of up
// to 128 rows of one expert.  A block takes one tile and 128 of the expert's weight rows: the
// weight rows are the MMA's M side (a lane of tensor memory each), the tile's rows its N side
// (a column each), K runs in blocks of 64 elements through a ring of TMA-fed, 128-byte-swizzled
// stages.  The weights of all experts are one 2-D tensor [experts * N, K], the sorted rows
// another [rows, K]; a box that reaches past an expert's weight rows or past the tile's rows
// reads its neighbour's (or zeros past the end), and those lanes and columns are not stored.
// An element is one accumulator over ascending K, so a row's result does not depend on the
// tile it lies in.  Warps: TMA producer, MMA issuer (one elected lane), four epilogue warps.
//   mode 0: C[row, n] = relu(acc)^2 as bfloat16;  mode 1: C[row, n] = acc as float32;
//   mode 2: C[row_token[row], n] += acc (float32): the sum into the residual stream where a token
//   chooses one expert, so that every element has one writer.
// ls_experts_gather writes the sorted, scaled rows that mode 0 reads.
#include "tc_common.cuh"

namespace {

constexpr int BM = 128;            // weight rows of a block (MMA M)
constexpr int BT = 128;            // rows of a tile (MMA N)
constexpr int BK = 64;             // K elements of a stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 3;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BT * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
constexpr uint32_t ACC_COLS = 128;

template <int MODE>
__global__ void __launch_bounds__(192) experts_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                         const __grid_constant__ CUtensorMap map_x,
                                                         const int* __restrict__ plan, const int* __restrict__ row_token,
                                                         void* __restrict__ C, int N, int K, int* err) {
  ls_dependency_sync();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;                    // the work list is sized for the worst case
  const int e = plan[1 + 3 * tile], row0 = plan[1 + 3 * tile + 1], rows = plan[1 + 3 * tile + 2];
  const int n0 = blockIdx.x * BM;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (size_t)STAGES * STAGE_BYTES);
  uint64_t* full = bars;                  // [STAGES]
  uint64_t* empty = bars + STAGES;        // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES; // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* failed = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(ACC_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int kb = 0;
      bool ok = true;
      for (; kb < total_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
        if (*failed || !mbar_wait(&empty[s], phase ^ 1u)) {
          *failed = 1;
          ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 500 + s);
          ok = false;
          break;
        }
        const uint32_t stage = base + (uint32_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        tma_load_2d(stage, &map_w, kb * BK, e * N + n0, &full[s]);
        tma_load_2d(stage + A_BYTES, &map_x, kb * BK, row0, &full[s]);
      }
      if (!ok) {
        // wait (bounded) for the copies still in flight before the block goes on to its end
        const int first = kb > STAGES ? kb - STAGES : 0;
        for (int j = first; j < kb; ++j) mbar_wait(&full[j % STAGES], (uint32_t)(j / STAGES) & 1u);
      }
    }
  } else if (warp == 1) {
    // the whole warp walks the loop and one elected lane issues
    constexpr uint32_t idesc = instr_desc(BM, BT);
    const bool issuer = elect_one();
    bool ok = true;
    for (int kb = 0; kb < total_kb; ++kb) {
      const int s = kb % STAGES;
      const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
      ok = __all_sync(0xffffffffu, !*failed && mbar_wait(&full[s], phase));
      if (!ok) {
        *failed = 1;
        if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 520 + s);
        break;
      }
      fence_after_sync();
      const uint32_t stage = base + (uint32_t)s * STAGE_BYTES;
      const uint64_t adesc = desc_k_major(stage), bdesc = desc_k_major(stage + A_BYTES);
      if (issuer) {
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) umma(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kb == 0 && k == 0) ? 0u : 1u);
        umma_commit(&empty[s]);
      }
      __syncwarp();
    }
    if (ok && issuer) umma_commit(acc_full);
    __syncwarp();
  } else {
    // epilogue: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 32
    const int quad = warp & 3;
    const int n = n0 + quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    bool got = mbar_wait(acc_full, 0u);
    if (!got) {
      *failed = 1;
      if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 540 + quad);
    }
    if (__all_sync(0xffffffffu, got)) {
      fence_after_sync();
      for (int c0 = 0; c0 < rows; c0 += 32) {
        uint32_t g[32];
        tmem_ld32(lane_base + (uint32_t)c0, g);
        tmem_ld_wait();
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j < rows) {
              const int64_t at = (int64_t)(row0 + c0 + j) * N + n;
              const float acc = __uint_as_float(g[j]);
              if (MODE == 0) {
                const float v = fmaxf(acc, 0.f);
                reinterpret_cast<__nv_bfloat16*>(C)[at] = __float2bfloat16_rn(v * v);
              } else if (MODE == 1) {
                reinterpret_cast<float*>(C)[at] = acc;
              } else {
                float* to = reinterpret_cast<float*>(C) + (int64_t)row_token[row0 + c0 + j] * N + n;
                *to = *to + acc;
              }
            }
          }
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_COLS) : "memory");
  }
}

// out[row, :] = x[row_token[row], :] * row_weight[row] (a copy where row_weight is null), rounded to bfloat16 once
__global__ void __launch_bounds__(256) gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_token,
                                                     const float* __restrict__ row_weight,
                                                     __nv_bfloat16* __restrict__ out, int width) {
  ls_dependency_sync();
  const int row = blockIdx.x;
  const int64_t src = (int64_t)row_token[row] * width;
  if (row_weight == nullptr) {
    for (int c = threadIdx.x; c < width; c += 256) out[(int64_t)row * width + c] = x[src + c];
    return;
  }
  const float w = row_weight[row];
  for (int c = threadIdx.x; c < width; c += 256)
    out[(int64_t)row * width + c] = __float2bfloat16_rn(__bfloat162float(x[src + c]) * w);
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
  }
  return fn;
}

// rows x K bfloat16, contiguous rows; box of box_rows x 64 elements with 128-byte swizzle
bool make_map(CUtensorMap* map, const void* ptr, long long rows, int K, int box_rows) {
  EncodeTiled enc = encode_fn();
  if (enc == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

LS_API int ls_experts_tc_tile_rows() { return BT; }

LS_API int ls_experts_gather(const void* x, const int* row_token, const float* row_weight, void* out, int rows,
                             int width, cudaStream_t stream) {
  if (rows <= 0) return 0;
  LS_COUNT(LS_K_EXPERTS_GATHER);
  cudaError_t e = ls_launch(gather_kernel, dim3(rows), dim3(256), 0, stream, (const __nv_bfloat16*)x, row_token,
                            row_weight, (__nv_bfloat16*)out, width);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

// A [rows, K] bfloat16 sorted by expert as `plan` says (tiles of up to 128 rows), W [experts, N, K]
// bfloat16; C [rows, N]: mode 0 bfloat16 relu(.)^2, mode 1 float32; mode 2: C [tokens, N] float32, added into
// at row_token[row].  Returns LS_E_ALIGN or LS_E_SIZE, having launched nothing, for what TMA cannot
// address; the caller then takes the CUDA-core product.
LS_API int ls_experts_product_tc(int mode, const int* plan, int max_tiles, const void* A, long long rows, const void* W,
                                 int experts, const int* row_token, void* C, int N, int K, int* err,
                                 cudaStream_t stream) {
  if (max_tiles <= 0 || rows <= 0) return 0;
  if (N <= 0 || K <= 0 || experts <= 0 || max_tiles > 65535 || mode < 0 || mode > 2) return LS_E_SIZE;
  if (mode == 2 && row_token == nullptr) return LS_E_SIZE;
  if ((K % 8) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return LS_E_ALIGN;
  CUtensorMap mw, mx;
  if (!make_map(&mw, W, (long long)experts * N, K, BM)) return LS_E_SIZE;
  if (!make_map(&mx, A, rows, K, BT)) return LS_E_SIZE;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(experts_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(experts_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(experts_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return LS_E_SMEM;
    configured = true;
  }
  const dim3 grid((N + BM - 1) / BM, max_tiles);
  LS_COUNT(mode == 0 ? LS_K_EXPERTS_UP_TC : LS_K_EXPERTS_DOWN_TC);
  cudaError_t e =
      mode == 0   ? ls_launch(experts_tc_kernel<0>, grid, dim3(192), SMEM, stream, mw, mx, plan, row_token, C, N, K, err)
      : mode == 1 ? ls_launch(experts_tc_kernel<1>, grid, dim3(192), SMEM, stream, mw, mx, plan, row_token, C, N, K, err)
                  : ls_launch(experts_tc_kernel<2>, grid, dim3(192), SMEM, stream, mw, mx, plan, row_token, C, N, K, err);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API const char* ls_constants_experts_tc() {
  static char buf[256];
  static const LsConstant c[] = {{"experts_tc.tile_rows", BT}, {"experts_tc.weight_rows", BM}, {"experts_tc.k_block", BK},
                                 {"experts_tc.stages", STAGES}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}
