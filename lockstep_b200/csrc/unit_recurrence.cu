// A gated linear recurrent unit per channel, and the rotation of a linear-attention layer's
// queries and keys.
//
// The unit (per channel c of `width` channels, cut into `blocks` equal parts):
//   u_t = conv(x)_t                       a causal convolution per channel over the projection x (+ its bias),
//                                         the inputs before a portion taken from the request's slot
//   r_t = sigmoid(A_b u_t,b + ba), i_t = sigmoid(I_b u_t,b + bi)     A_b, I_b square matrices of part b
//   log a_t = -c r_t softplus(lam),  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t
//   out_t = S_t gelu(y_t)                 y the second projection (+ its bias)
// unit_gates makes a_t and the input term b_t = sqrt(1 - a_t^2) i_t u_t for every token (float32);
// unit_scan walks every portion token by token, one thread a channel, writes S gelu(y) in the
// engine's type, and keeps S and the last taps - 1 inputs of the convolution in the slot
// (float32 [width + (taps - 1) width], the inputs oldest first).
// A token's arithmetic does not depend on the portion it arrives in: a gate's sum is four chains over
// ascending quarters of the input channels, added in ascending order; the walk is one fused multiply-add a token.
#include "common.cuh"

namespace {

constexpr int GATE_TOKENS = 16;     // tokens of one block of unit_gates
constexpr int GATE_COLS = 32;       // output channels of one block
constexpr int GATE_THREADS = 128;   // four warps: a quarter of the input channels each
constexpr int MAX_UNIT_TAPS = 16;

struct GateArgs {
  const void* proj;        // [T, ld]: the x projection at column x_at
  int64_t ld;
  int x_at;
  const float* x_bias;     // [width]
  const float* conv_w;     // [width, taps], last column the current token's
  const float* conv_b;     // [width]
  const float* state;      // per slot: S [width], then (taps - 1) rows of carried inputs
  int64_t state_stride;
  const int* token_slot;
  const void* w_r;         // [blocks, bw (in), bw (out)]: the matrices transposed, in the engine's type
  const void* w_i;
  const float* b_r;        // [width]
  const float* b_i;
  const float* rate;       // [width]: softplus(lam)
  float* a_out;            // [T, width]
  float* b_out;
  int T, width, blocks, taps;
  int runs;                // runs of GATE_COLS output channels that one block takes, one after the other
  float c;                 // the factor in log a
};

// A block: GATE_TOKENS tokens, one part, some runs of GATE_COLS output channels of it (all of them in a step of many
// tokens, where staging the convolution once pays; one run in a step of few, where more blocks do); its four warps
// each take a quarter of the input channels (ascending, one accumulator a token and matrix), the quarters are added
// in ascending order.
template <typename T>
__global__ void __launch_bounds__(GATE_THREADS) unit_gates_kernel(GateArgs g) {
  // u [bw][GATE_TOKENS], then the quarters' sums [4][2][GATE_TOKENS][GATE_COLS] (before them, there: the tile's inputs)
  extern __shared__ __align__(16) float us[];
  ls_dependency_sync();
  const int bw = g.width / g.blocks, part = blockIdx.y, t0 = blockIdx.x * GATE_TOKENS;
  const int nt = g.T - t0 < GATE_TOKENS ? g.T - t0 : GATE_TOKENS;
  const T* proj = reinterpret_cast<const T*>(g.proj);
  float* sums = us + bw * GATE_TOKENS;
  __shared__ int tok_slot[GATE_TOKENS], tok_inside[GATE_TOKENS];
  if (threadIdx.x < GATE_TOKENS) {
    const int t = t0 + threadIdx.x;
    int slot = 0, inside = 0;
    if (threadIdx.x < nt) {
      slot = g.token_slot[t];
      // how many of the tokens in front of t belong to its portion (up to taps - 1)
      while (inside < g.taps - 1 && t - inside - 1 >= 0 && g.token_slot[t - inside - 1] == slot) ++inside;
    }
    tok_slot[threadIdx.x] = slot;
    tok_inside[threadIdx.x] = inside;
  }
  __syncthreads();
  // the inputs (with their bias) of the tile's tokens and of the taps - 1 tokens in front of them, where the quarters'
  // sums will lie later: row r is token t0 - (taps - 1) + r.  Loads that do not wait for one another.
  const int lead = g.taps - 1;
  float* xs = sums;
#pragma unroll 4
  for (int e = threadIdx.x; e < (GATE_TOKENS + lead) * bw; e += blockDim.x) {
    const int r = e / bw, k = e - r * bw, t = t0 - lead + r;
    float x = 0.f;
    if (t >= 0 && t < g.T) x = ls_to_float<T>(proj[(int64_t)t * g.ld + g.x_at + part * bw + k]) + g.x_bias[part * bw + k];
    xs[e] = x;
  }
  __syncthreads();
  // the convolution: channel c of token t reads its own input and the taps - 1 before it (those in front of the
  // token's portion from the request's slot)
  for (int e = threadIdx.x; e < GATE_TOKENS * bw; e += blockDim.x) {
    const int tt = e / bw, k = e - tt * bw, c = part * bw + k;
    float acc = 0.f;
    if (tt < nt) {
      const int inside = tok_inside[tt];
      const float* carried = g.state + (int64_t)tok_slot[tt] * g.state_stride + g.width;
      acc = g.conv_b[c];
      for (int j = 0; j < g.taps; ++j) {
        const int back = lead - j;                 // tap j reads the input `back` tokens ago
        const float x = back <= inside ? xs[(lead + tt - back) * bw + k]
                                       : carried[(int64_t)(lead + inside - back) * g.width + c];
        acc = fmaf(g.conv_w[(int64_t)c * g.taps + j], x, acc);
      }
    }
    us[k * GATE_TOKENS + tt] = acc;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, quarter = threadIdx.x >> 5;
  const int per = (bw + 3) / 4, k_lo = quarter * per, k_hi = k_lo + per < bw ? k_lo + per : bw;
  const T* w_r = reinterpret_cast<const T*>(g.w_r) + (int64_t)part * bw * bw;
  const T* w_i = reinterpret_cast<const T*>(g.w_i) + (int64_t)part * bw * bw;
  // the block's runs of GATE_COLS output channels, one after the other
  for (int run = blockIdx.z * g.runs; run < (blockIdx.z + 1) * g.runs && run * GATE_COLS < bw; ++run) {
    const int j = run * GATE_COLS + lane;
    float ar[GATE_TOKENS], ai[GATE_TOKENS];
#pragma unroll
    for (int tt = 0; tt < GATE_TOKENS; ++tt) ar[tt] = ai[tt] = 0.f;
    if (j < bw) {
#pragma unroll 4
      for (int k = k_lo; k < k_hi; ++k) {
        const float wr = ls_to_float<T>(w_r[(int64_t)k * bw + j]), wi = ls_to_float<T>(w_i[(int64_t)k * bw + j]);
        const float4* u4 = reinterpret_cast<const float4*>(us + k * GATE_TOKENS);
#pragma unroll
        for (int q = 0; q < GATE_TOKENS / 4; ++q) {
          const float4 u = u4[q];
          ar[4 * q] = fmaf(wr, u.x, ar[4 * q]); ai[4 * q] = fmaf(wi, u.x, ai[4 * q]);
          ar[4 * q + 1] = fmaf(wr, u.y, ar[4 * q + 1]); ai[4 * q + 1] = fmaf(wi, u.y, ai[4 * q + 1]);
          ar[4 * q + 2] = fmaf(wr, u.z, ar[4 * q + 2]); ai[4 * q + 2] = fmaf(wi, u.z, ai[4 * q + 2]);
          ar[4 * q + 3] = fmaf(wr, u.w, ar[4 * q + 3]); ai[4 * q + 3] = fmaf(wi, u.w, ai[4 * q + 3]);
        }
      }
    }
    __syncthreads();                               // the run before is done with the quarters' sums
#pragma unroll
    for (int tt = 0; tt < GATE_TOKENS; ++tt) {
      sums[((quarter * 2 + 0) * GATE_TOKENS + tt) * GATE_COLS + lane] = ar[tt];
      sums[((quarter * 2 + 1) * GATE_TOKENS + tt) * GATE_COLS + lane] = ai[tt];
    }
    __syncthreads();
    if (j < bw) {
      const int c = part * bw + j;
      const float br = g.b_r[c], bi = g.b_i[c], rate = g.rate[c];
      // warp `quarter` finishes the tokens quarter, quarter + 4, ...
      for (int tt = quarter; tt < nt; tt += 4) {
        float zr = 0.f, zi = 0.f;
#pragma unroll
        for (int qq = 0; qq < 4; ++qq) {
          zr += sums[((qq * 2 + 0) * GATE_TOKENS + tt) * GATE_COLS + lane];
          zi += sums[((qq * 2 + 1) * GATE_TOKENS + tt) * GATE_COLS + lane];
        }
        const float r = 1.0f / (1.0f + expf(-(zr + br)));
        const float i = 1.0f / (1.0f + expf(-(zi + bi)));
        const float log_a = -g.c * r * rate;
        // sqrt(1 - a^2) through expm1: a decay near one keeps its digits
        const float in = sqrtf(-expm1f(2.0f * log_a)) * i * us[j * GATE_TOKENS + tt];
        g.a_out[(int64_t)(t0 + tt) * g.width + c] = expf(log_a);
        g.b_out[(int64_t)(t0 + tt) * g.width + c] = in;
      }
    }
  }
}

struct ScanArgs {
  const int* portions;     // from find_portions
  const float* a;          // [T, width]
  const float* b;
  const void* proj;        // [T, ld]: y at column y_at, x at column x_at
  int64_t ld;
  int y_at, x_at;
  const float* y_bias;
  const float* x_bias;
  float* state;
  int64_t state_stride;
  void* out;               // [T, width] in the engine's type
  int width, taps;
};

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(128) unit_scan_kernel(ScanArgs s) {
  ls_dependency_sync();
  const int p = blockIdx.x;
  if (p >= s.portions[0]) return;
  const int t0 = s.portions[1 + 3 * p], n = s.portions[1 + 3 * p + 1], slot = s.portions[1 + 3 * p + 2];
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= s.width) return;
  const T* proj = reinterpret_cast<const T*>(s.proj);
  T* out = reinterpret_cast<T*>(s.out);
  float* state = s.state + (int64_t)slot * s.state_stride;
  float S = state[c];
  const float yb = s.y_bias[c];
  constexpr int AHEAD = 8;
  for (int i0 = 0; i0 < n; i0 += AHEAD) {
    float a[AHEAD], b[AHEAD], y[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      const int64_t t = t0 + (i0 + k < n ? i0 + k : n - 1);
      a[k] = s.a[t * s.width + c];
      b[k] = s.b[t * s.width + c];
      y[k] = ls_to_float<T>(proj[t * s.ld + s.y_at + c]);
    }
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      if (i0 + k >= n) break;
      S = fmaf(a[k], S, b[k]);
      out[(int64_t)(t0 + i0 + k) * s.width + c] = ls_from_float<T>(S * gelu_tanh_f(y[k] + yb));
    }
  }
  state[c] = S;
  // the convolution's last taps - 1 inputs, oldest first: from the portion where it is long enough, else what
  // the slot held moves up
  float keep[MAX_UNIT_TAPS];
  const int rows = s.taps - 1;
  for (int i = 0; i < rows; ++i) {
    const int at = n - rows + i;           // the portion's token that row i holds afterwards
    keep[i] = at >= 0 ? ls_to_float<T>(proj[(int64_t)(t0 + at) * s.ld + s.x_at + c]) + s.x_bias[c]
                      : state[s.width + (int64_t)(rows + at) * s.width + c];
  }
  for (int i = 0; i < rows; ++i) state[s.width + (int64_t)i * s.width + c] = keep[i];
}

struct RotateArgs {
  const void* proj;        // [T, ld]: q at q_at, k at k_at (heads x dk each), v at v_at (heads x dv)
  int64_t ld;
  int q_at, k_at, v_at;
  const float* cos_table;  // [max_positions, rot_dim / 2]
  const float* sin_table;
  const int* positions;
  float* out;              // [T, 2 heads dk + heads dv]: rotated q, rotated k times k_scale, v
  int T, heads, dk, dv, rot_dim, max_positions;
  float k_scale;
};

template <typename T>
__global__ void __launch_bounds__(128) rotate_rows_kernel(RotateArgs r, int* err) {
  ls_dependency_sync();
  const int t = blockIdx.x;
  const T* row = reinterpret_cast<const T*>(r.proj) + (int64_t)t * r.ld;
  const int Kd = r.heads * r.dk, Vd = r.heads * r.dv, half = r.rot_dim >> 1;
  float* dst = r.out + (int64_t)t * (2 * Kd + Vd);
  int pos = r.positions[t];
  if (half > 0 && (pos < 0 || pos >= r.max_positions)) {
    if (threadIdx.x == 0) ls_record_fault(err, LS_DEV_POSITION_RANGE, t);
    pos = 0;
  }
  const float* cs = r.cos_table + (int64_t)pos * half;
  const float* sn = r.sin_table + (int64_t)pos * half;
  // element e of q or k: head e / dk, channel e % dk; a rotated pair is (i, i + rot_dim / 2); products and sums are
  // rounded one by one
  for (int e = threadIdx.x; e < 2 * Kd; e += blockDim.x) {
    const bool is_k = e >= Kd;
    const T* src = row + (is_k ? r.k_at : r.q_at);
    const int w = is_k ? e - Kd : e;
    const int i = w % r.dk;
    float v;
    if (i < half) {
      const float lo = ls_to_float<T>(src[w]), hi = ls_to_float<T>(src[w + half]);
      v = __fsub_rn(__fmul_rn(lo, cs[i]), __fmul_rn(hi, sn[i]));
    } else if (i < r.rot_dim) {
      const float lo = ls_to_float<T>(src[w - half]), hi = ls_to_float<T>(src[w]);
      v = __fadd_rn(__fmul_rn(hi, cs[i - half]), __fmul_rn(lo, sn[i - half]));
    } else {
      v = ls_to_float<T>(src[w]);
    }
    dst[e] = is_k ? __fmul_rn(v, r.k_scale) : v;
  }
  for (int e = threadIdx.x; e < Vd; e += blockDim.x) dst[2 * Kd + e] = ls_to_float<T>(row[r.v_at + e]);
}

}  // namespace

LS_API int ls_unit_gates(const void* proj, long long ld, int x_at, int dtype, const float* x_bias, const float* conv_w,
                         const float* conv_b, const float* state, long long state_stride, const int* token_slot,
                         const void* w_r, const void* w_i, const float* b_r, const float* b_i, const float* rate,
                         float* a_out, float* b_out, int tokens, int width, int blocks, int taps, float c,
                         cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || blocks <= 0 || width % blocks || taps < 1 || taps > MAX_UNIT_TAPS) return LS_E_SIZE;
  const int bw = width / blocks;
  const size_t quarters = 4 * 2 * GATE_TOKENS * GATE_COLS, inputs = (size_t)(GATE_TOKENS + taps - 1) * bw;
  const size_t smem = sizeof(float) * ((size_t)GATE_TOKENS * bw + (quarters > inputs ? quarters : inputs));
  if (smem > 200 * 1024 || blocks > 65535 || (bw + GATE_COLS - 1) / GATE_COLS > 65535) return LS_E_SMEM;
  GateArgs g;
  g.proj = proj; g.ld = ld; g.x_at = x_at; g.x_bias = x_bias; g.conv_w = conv_w; g.conv_b = conv_b; g.state = state;
  g.state_stride = state_stride; g.token_slot = token_slot; g.w_r = w_r; g.w_i = w_i; g.b_r = b_r; g.b_i = b_i; g.rate = rate;
  g.a_out = a_out; g.b_out = b_out; g.T = tokens; g.width = width; g.blocks = blocks; g.taps = taps; g.c = c;
  const int all_runs = (bw + GATE_COLS - 1) / GATE_COLS;
  g.runs = tokens > 2 * GATE_TOKENS ? all_runs : 1;
  const dim3 grid((tokens + GATE_TOKENS - 1) / GATE_TOKENS, blocks, (all_runs + g.runs - 1) / g.runs);
  const int threads = GATE_THREADS;
  LS_COUNT(LS_K_UNIT_GATES);
  if (dtype == LS_F32) {
    // (the kernel has a little static shared memory besides: the limit is asked for from 40 KB on)
    static size_t set_f32 = 40 * 1024;
    if (smem > set_f32) {
      if (cudaFuncSetAttribute(unit_gates_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return LS_E_SMEM;
      set_f32 = smem;
    }
    ls_launch(unit_gates_kernel<float>, grid, dim3(threads), smem, stream, g);
  } else if (dtype == LS_BF16) {
    static size_t set_bf16 = 40 * 1024;
    if (smem > set_bf16) {
      if (cudaFuncSetAttribute(unit_gates_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return LS_E_SMEM;
      set_bf16 = smem;
    }
    ls_launch(unit_gates_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, g);
  } else {
    return LS_E_DTYPE;
  }
  return ls_launch_status();
}

LS_API int ls_unit_scan(const int* portions, int max_portions, const float* a, const float* b, const void* proj, long long ld,
                        int y_at, int x_at, int dtype, const float* y_bias, const float* x_bias, float* state,
                        long long state_stride, void* out, int width, int taps, cudaStream_t stream) {
  if (max_portions <= 0) return 0;
  if (width <= 0 || taps < 1 || taps > MAX_UNIT_TAPS) return LS_E_SIZE;
  ScanArgs s;
  s.portions = portions; s.a = a; s.b = b; s.proj = proj; s.ld = ld; s.y_at = y_at; s.x_at = x_at; s.y_bias = y_bias;
  s.x_bias = x_bias; s.state = state; s.state_stride = state_stride; s.out = out; s.width = width; s.taps = taps;
  const dim3 grid(max_portions, (width + 127) / 128);
  LS_COUNT(LS_K_UNIT_SCAN);
  if (dtype == LS_F32) ls_launch(unit_scan_kernel<float>, grid, dim3(128), 0, stream, s);
  else if (dtype == LS_BF16) ls_launch(unit_scan_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, s);
  else return LS_E_DTYPE;
  return ls_launch_status();
}

LS_API int ls_rotate_rows(const void* proj, long long ld, int q_at, int k_at, int v_at, int dtype, const float* cos_table,
                          const float* sin_table, const int* positions, float* out, int tokens, int heads, int dk, int dv,
                          int rot_dim, int max_positions, float k_scale, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || dk <= 0 || dv <= 0 || rot_dim < 0 || rot_dim > dk || rot_dim % 2) return LS_E_SIZE;
  if (rot_dim > 0 && (cos_table == nullptr || sin_table == nullptr)) return LS_E_SIZE;
  RotateArgs r;
  r.proj = proj; r.ld = ld; r.q_at = q_at; r.k_at = k_at; r.v_at = v_at; r.cos_table = cos_table; r.sin_table = sin_table;
  r.positions = positions; r.out = out; r.T = tokens; r.heads = heads; r.dk = dk; r.dv = dv; r.rot_dim = rot_dim;
  r.max_positions = max_positions; r.k_scale = k_scale;
  LS_COUNT(LS_K_ROTATE_ROWS);
  if (dtype == LS_F32) ls_launch(rotate_rows_kernel<float>, dim3(tokens), dim3(128), 0, stream, r, err);
  else if (dtype == LS_BF16) ls_launch(rotate_rows_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, r, err);
  else return LS_E_DTYPE;
  return ls_launch_status();
}
