// Mixers that carry a matrix state from token to token, one state per request slot:
//   - the gated delta rule with a decay per head and key channel,
//   - an RWKV-style rule (decay per channel, a bonus for the current token),
// and what stands around them: the list of a step's portions made on the device, short
// causal convolutions with their carried inputs, the token shift, the decays from the outputs
// of their low-rank maps (which run as products), and the gated per-head RMSNorm of the read-out.
//
// A step's token axis packs portions of several requests; a request appears once, so token t
// continues the portion of token t - 1 exactly when both have the same slot.  Everything a
// kernel needs to know about portions it takes from `token_slot` on the device, so a recorded
// step replays with other portions in the same buffers.
//
// All state and everything that enters a recurrence is float32.  A token's arithmetic is the
// same whatever portion it arrives in: states are walked token by token, a dot product over
// the key channels is four interleaved chains of fused multiply-adds per thread (channel r of
// the thread's run goes to chain r mod 4), added as (c0 + c1) + (c2 + c3), then an xor-tree
// over the lanes that share a column.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------
// portions: out[0] = count, then (first token, tokens, slot) per portion, in token order
// ---------------------------------------------------------------------------------------
constexpr int PORTION_THREADS = 1024;

__global__ void __launch_bounds__(PORTION_THREADS) find_portions_kernel(const int* __restrict__ token_slot, int T,
                                                                       int* __restrict__ out, int cap, int* err) {
  __shared__ int warp_s[32], warp_e[32];
  __shared__ int base_s, base_e;
  ls_dependency_sync();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) base_s = base_e = 0;
  __syncthreads();
  for (int c0 = 0; c0 < T; c0 += PORTION_THREADS) {
    const int t = c0 + tid;
    int slot = 0;
    bool is_s = false, is_e = false;
    if (t < T) {
      slot = token_slot[t];
      is_s = t == 0 || token_slot[t - 1] != slot;
      is_e = t == T - 1 || token_slot[t + 1] != slot;
    }
    const unsigned bs = __ballot_sync(0xffffffffu, is_s), be = __ballot_sync(0xffffffffu, is_e);
    const unsigned below = (1u << lane) - 1u;
    if (lane == 0) {
      warp_s[warp] = __popc(bs);
      warp_e[warp] = __popc(be);
    }
    __syncthreads();
    int off_s = base_s, off_e = base_e, tot_s = 0, tot_e = 0;
    for (int w = 0; w < PORTION_THREADS / 32; ++w) {
      if (w < warp) {
        off_s += warp_s[w];
        off_e += warp_e[w];
      }
      tot_s += warp_s[w];
      tot_e += warp_e[w];
    }
    if (is_s) {
      const int p = off_s + __popc(bs & below);
      if (p < cap) {
        out[1 + 3 * p] = t;
        out[1 + 3 * p + 2] = slot;
      }
    }
    if (is_e) {
      const int p = off_e + __popc(be & below);
      if (p < cap) out[1 + 3 * p + 1] = t;     // the last token for now
    }
    __syncthreads();
    if (tid == 0) {
      base_s += tot_s;
      base_e += tot_e;
    }
    __syncthreads();
  }
  const int count = base_s;
  if (tid == 0) {
    out[0] = count < cap ? count : cap;
    if (count > cap) ls_record_fault(err, LS_DEV_ROW_RANGE, count);
  }
  __threadfence_block();
  __syncthreads();
  for (int p = tid; p < count && p < cap; p += PORTION_THREADS) out[1 + 3 * p + 1] = out[1 + 3 * p + 1] - out[1 + 3 * p] + 1;
}

// how many tokens before t lie in t's portion, at most `most`
__device__ __forceinline__ int tokens_before(const int* __restrict__ token_slot, int t, int most) {
  const int slot = token_slot[t];
  int m = 0;
  while (m < most && t - m - 1 >= 0 && token_slot[t - m - 1] == slot) ++m;
  return m;
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------------------
// gated delta rule: everything between the projections and the recurrence, one block a token
// ---------------------------------------------------------------------------------------
constexpr int PREP_THREADS = 256;
constexpr int MAX_TAPS = 8;

struct DeltaPrepArgs {
  const void* proj;        // [T, ld]: q (G dk) | k (G dk) | v (H dv) | beta (H) | ...
  int64_t ld;
  const float* conv_w;     // [C, taps], C = 2 G dk + H dv; the last tap is the current token's
  const float* dt_bias;    // [H dk]
  const float* a_log;      // [H]
  const float* state;      // per slot: S [H, dk, dv], then the last taps - 1 inputs of the convolution [taps - 1, C]
  int64_t state_stride;
  const int* token_slot;
  float* qkv;              // [T, C]: q (unit, scaled), k (unit), v, after convolution and silu
  float* decay;            // [T, H dk]: in, the output z of the decay's low-rank map; out, exp(-exp(A_log) softplus(z + dt_bias))
  float* beta;             // [T, H]
  int T, H, G, dk, dv, taps;
  float unit_eps;
};

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS) delta_prep_kernel(DeltaPrepArgs a) {
  extern __shared__ float smem[];
  ls_dependency_sync();
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int Kd = a.G * a.dk, Vd = a.H * a.dv, C = 2 * Kd + Vd;
  float* conv = smem;              // [C]
  float* head_scale = conv + C;    // [2 G]
  const T* proj = reinterpret_cast<const T*>(a.proj);
  const T* row = proj + (int64_t)t * a.ld;
  const int slot = a.token_slot[t];
  const int before = tokens_before(a.token_slot, t, a.taps - 1);
  const float* carried = a.state + (int64_t)slot * a.state_stride + (int64_t)a.H * a.dk * a.dv;

  for (int c = tid; c < C; c += PREP_THREADS) {
    float acc = 0.f;
    for (int j = 0; j < a.taps; ++j) {
      const int back = a.taps - 1 - j;
      float x;
      if (back <= before) x = ls_to_float<T>(proj[(int64_t)(t - back) * a.ld + c]);
      else x = carried[(int64_t)(a.taps - 2 - (back - before - 1)) * C + c];
      acc = fmaf(a.conv_w[c * a.taps + j], x, acc);
    }
    conv[c] = silu_f(acc);
  }
  __syncthreads();
  // q and k heads to unit length; q also by dk^(-1/2)
  for (int h = warp; h < 2 * a.G; h += PREP_THREADS / 32) {
    float ss = 0.f;
    for (int i = lane; i < a.dk; i += 32) {
      const float v = conv[h * a.dk + i];
      ss = fmaf(v, v, ss);
    }
    ss = ls_warp_sum(ss);
    if (lane == 0) head_scale[h] = (1.0f / sqrtf(ss + a.unit_eps)) * (h < a.G ? 1.0f / sqrtf((float)a.dk) : 1.0f);
  }
  __syncthreads();
  float* out = a.qkv + (int64_t)t * C;
  for (int c = tid; c < C; c += PREP_THREADS) out[c] = c < 2 * Kd ? conv[c] * head_scale[c / a.dk] : conv[c];
  for (int h = tid; h < a.H; h += PREP_THREADS) a.beta[(int64_t)t * a.H + h] = sigmoid_f(ls_to_float<T>(row[C + h]));
  float* decay = a.decay + (int64_t)t * a.H * a.dk;
  for (int i = tid; i < a.H * a.dk; i += PREP_THREADS)
    decay[i] = expf(-expf(a.a_log[i / a.dk]) * softplus_f(decay[i] + a.dt_bias[i]));
}

// z <- exp(-exp(z + bias[column])), element by element: a decay from its low-rank map's output
__global__ void __launch_bounds__(PREP_THREADS) double_exp_decay_kernel(float* __restrict__ z, const float* __restrict__ bias,
                                                                        int64_t count, int channels) {
  ls_dependency_sync();
  const int64_t i = (int64_t)blockIdx.x * PREP_THREADS + threadIdx.x;
  if (i < count) z[i] = expf(-expf(z[i] + bias[i % channels]));
}

// z <- sigmoid(z + bias[column])^(1 / tau), element by element, through its logarithm:
// exp(-softplus(-(z + bias)) / tau)
__global__ void __launch_bounds__(PREP_THREADS) sigmoid_power_decay_kernel(float* __restrict__ z, const float* __restrict__ bias,
                                                                           int64_t count, int channels, float inv_tau) {
  ls_dependency_sync();
  const int64_t i = (int64_t)blockIdx.x * PREP_THREADS + threadIdx.x;
  if (i < count) z[i] = expf(-softplus_f(-(z[i] + bias[i % channels])) * inv_tau);
}

// ---------------------------------------------------------------------------------------
// token shift: five mixes of a token with the one before it (the carried one at a portion's start)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(PREP_THREADS) shift_mix_kernel(const T* __restrict__ x, const float* __restrict__ mu,
                                                                 const float* __restrict__ state, int64_t state_stride,
                                                                 int64_t prev_offset, const int* __restrict__ token_slot,
                                                                 T* __restrict__ out, int tokens, int width, int mixes) {
  ls_dependency_sync();
  const int t = blockIdx.x;
  const int slot = token_slot[t];
  const bool inside = t > 0 && token_slot[t - 1] == slot;
  const float* carried = state + (int64_t)slot * state_stride + prev_offset;
  for (int c = threadIdx.x; c < width; c += PREP_THREADS) {
    const float cur = ls_to_float<T>(x[(int64_t)t * width + c]);
    const float prev = inside ? ls_to_float<T>(x[(int64_t)(t - 1) * width + c]) : carried[c];
    const float diff = prev - cur;
    for (int s = 0; s < mixes; ++s)
      out[((int64_t)s * tokens + t) * width + c] = ls_from_float<T>(fmaf(diff, mu[s * width + c], cur));
  }
}

// x <- tanh(x), element by element
template <typename T>
__global__ void __launch_bounds__(PREP_THREADS) tanh_kernel(T* __restrict__ x, int64_t count) {
  ls_dependency_sync();
  const int64_t i = (int64_t)blockIdx.x * PREP_THREADS + threadIdx.x;
  if (i < count) x[i] = ls_from_float<T>(tanhf(ls_to_float<T>(x[i])));
}

// ---------------------------------------------------------------------------------------
// the recurrences
// ---------------------------------------------------------------------------------------
constexpr int ROWS = 16;          // key channels of a column that one thread keeps in registers
constexpr int CHUNK = 8;          // tokens staged in shared memory at a time
// RULE_GLA: a decayed sum of outer products, S <- diag(decay_t) S + k_t v_t^T, o_t = out_scale S^T q_t
enum { RULE_DELTA = 0, RULE_WKV = 1, RULE_GLA = 2 };

struct RuleArgs {
  const int* portions;     // from find_portions_kernel
  float* state;            // per slot: S [H, dk, dv] first
  int64_t state_stride;
  // delta: qkv float32 [T, 2 G dk + H dv], decay [T, H dk], beta [T, H]
  // wkv:   r, k, v [T, H dk] in the engine's type, decay [T, H dk], bonus [H dk]
  const void* in_a;        // delta: qkv; wkv: r
  const void* in_b;        // wkv: k
  const void* in_v;        // wkv: v
  const float* decay;      // [T, H dk]
  const float* beta;       // delta
  const float* bonus;      // wkv
  float* out;              // [T, H dv] float32
  // what else the state carries, updated by one block per portion after the walk
  const void* carry_src;   // delta: the raw projection [T, ld] (its first C columns); wkv: the mixer's input [T, width]
  int64_t carry_ld;
  int carry_width;         // delta: C; wkv: width
  int carry_rows;          // delta: taps - 1; wkv: 1
  int H, G, dk, dv, lanes; // lanes: threads that share a column (a power of two, lanes * ROWS >= dk)
  int64_t in_ld;           // gla: q, k, v are columns of wider rows, this many elements apart
  float out_scale;         // gla: factor on the read-out (the queries' scale)
  int64_t decay_ld;        // elements between two tokens' decays (H dk), or 0: one decay [H dk] for every token
};

// One staged value's source: where token t's copy lies (p + t * stride), and its element type.
struct StageSrc {
  const char* p;
  int64_t stride;
  int kind;                // 0: nothing (zero), 1: float32, 2: the engine's type
};

constexpr int STAGE_SLOTS = 4;     // staged values of a token that one thread fetches (more: the plain loader)

template <int RULE, typename T>
__global__ void __launch_bounds__(128) rule_kernel(RuleArgs a) {
  extern __shared__ float smem[];
  ls_dependency_sync();
  const int p = blockIdx.x;
  if (p >= a.portions[0]) return;
  const int t0 = a.portions[1 + 3 * p], n = a.portions[1 + 3 * p + 1], slot = a.portions[1 + 3 * p + 2];
  const int h = blockIdx.y, tid = threadIdx.x, L = a.lanes, CB = blockDim.x / L;
  const int dk = a.dk, dv = a.dv;
  const int col0 = blockIdx.z * CB, cl = tid / L, part = tid % L;
  const int col = col0 + cl;
  const bool active = col < dv;
  const int g = h / (a.H / a.G);
  float* state = a.state + (int64_t)slot * a.state_stride + (int64_t)h * dk * dv;
  // a thread keeps the key channels i = part * ROWS + r of its column
  float S[ROWS], bonus[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int i = part * ROWS + r;
    S[r] = (active && i < dk) ? state[(int64_t)i * dv + col] : 0.f;
    bonus[r] = (RULE == RULE_WKV && i < dk) ? a.bonus[h * dk + i] : 0.f;
  }
  // What is fetched per token: A [dk] (q or r), B [dk] (k), D [dk] (decay), V [CB], beta.
  // In shared memory each of A, B, D lies as L runs of ROWS channels, a run padded by four
  // words: the lanes that share a column read 16 bytes each from different banks, the lanes of
  // other columns the same words.  Channels past dk stay zero (a zero key writes nothing).
  const int per_token = 3 * dk + CB + 1;
  const int run = ROWS + 4, dkp = L * run, cbp = (CB + 3) & ~3;
  const int stride = 3 * dkp + cbp + 4;              // words of a token in shared memory
  const int Kd = a.G * dk, C = 2 * Kd + a.H * dv;
  auto place = [&](int k) {                          // where fetched value k of a token lies
    if (k < 3 * dk) {
      const int which = k / dk, i = k - which * dk;
      return which * dkp + (i / ROWS) * run + (i % ROWS);
    }
    return k < 3 * dk + CB ? 3 * dkp + (k - 3 * dk) : 3 * dkp + cbp;
  };
  auto source = [&](int k) {
    StageSrc s;
    s.p = nullptr; s.stride = 0; s.kind = 0;
    if (k >= per_token) return s;
    if (k < 3 * dk) {
      const int which = k / dk, i = k - which * dk;
      if (which == 2) {
        s.p = reinterpret_cast<const char*>(a.decay + h * dk + i);
        s.stride = a.decay_ld * 4;
        s.kind = 1;
      } else if (RULE == RULE_DELTA) {
        s.p = reinterpret_cast<const char*>(reinterpret_cast<const float*>(a.in_a) + which * Kd + g * dk + i);
        s.stride = (int64_t)C * 4;
        s.kind = 1;
      } else {
        s.p = reinterpret_cast<const char*>(reinterpret_cast<const T*>(which == 0 ? a.in_a : a.in_b) + h * dk + i);
        s.stride = (RULE == RULE_GLA ? a.in_ld : (int64_t)a.H * dk) * sizeof(T);
        s.kind = 2;
      }
    } else if (k < 3 * dk + CB) {
      const int j = col0 + (k - 3 * dk);
      if (j < dv) {
        if (RULE == RULE_DELTA) {
          s.p = reinterpret_cast<const char*>(reinterpret_cast<const float*>(a.in_a) + 2 * Kd + h * dv + j);
          s.stride = (int64_t)C * 4;
          s.kind = 1;
        } else {
          s.p = reinterpret_cast<const char*>(reinterpret_cast<const T*>(a.in_v) + h * dv + j);
          s.stride = (RULE == RULE_GLA ? a.in_ld : (int64_t)a.H * dv) * sizeof(T);
          s.kind = 2;
        }
      }
    } else if (RULE == RULE_DELTA) {
      s.p = reinterpret_cast<const char*>(a.beta + h);
      s.stride = (int64_t)a.H * 4;
      s.kind = 1;
    }
    return s;
  };
  auto fetch = [&](const StageSrc& s, int64_t t) {
    if (s.kind == 0) return 0.f;
    const char* at = s.p + t * s.stride;
    if (s.kind == 2) return ls_to_float<T>(*reinterpret_cast<const T*>(at));
    return *reinterpret_cast<const float*>(at);
  };
  auto walk = [&](const float* buf, int c0, int cn) {
    // unrolled over the chunk: a token's read-out (its sums and the exchange between the lanes of a
    // column) does not feed the state, so the next tokens' updates are issued beside it
#pragma unroll
    for (int tt = 0; tt < CHUNK; ++tt) {
      if (tt >= cn) break;
      const float* tok = buf + tt * stride;
      const float4* A = reinterpret_cast<const float4*>(tok + part * run);
      const float4* B = reinterpret_cast<const float4*>(tok + dkp + part * run);
      const float4* D = reinterpret_cast<const float4*>(tok + 2 * dkp + part * run);
      const float vj = tok[3 * dkp + cl];
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
      if (RULE == RULE_DELTA) {
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
        float4 kk[ROWS / 4];
#pragma unroll
        for (int r = 0; r < ROWS / 4; ++r) {
          const float4 dd = D[r];
          kk[r] = B[r];
          S[4 * r] *= dd.x; d0 = fmaf(S[4 * r], kk[r].x, d0);
          S[4 * r + 1] *= dd.y; d1 = fmaf(S[4 * r + 1], kk[r].y, d1);
          S[4 * r + 2] *= dd.z; d2 = fmaf(S[4 * r + 2], kk[r].z, d2);
          S[4 * r + 3] *= dd.w; d3 = fmaf(S[4 * r + 3], kk[r].w, d3);
        }
        float dot = (d0 + d1) + (d2 + d3);
        for (int off = L >> 1; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float u = tok[3 * dkp + cbp] * (vj - dot);
#pragma unroll
        for (int r = 0; r < ROWS / 4; ++r) {
          const float4 qq = A[r];
          S[4 * r] = fmaf(kk[r].x, u, S[4 * r]); o0 = fmaf(S[4 * r], qq.x, o0);
          S[4 * r + 1] = fmaf(kk[r].y, u, S[4 * r + 1]); o1 = fmaf(S[4 * r + 1], qq.y, o1);
          S[4 * r + 2] = fmaf(kk[r].z, u, S[4 * r + 2]); o2 = fmaf(S[4 * r + 2], qq.z, o2);
          S[4 * r + 3] = fmaf(kk[r].w, u, S[4 * r + 3]); o3 = fmaf(S[4 * r + 3], qq.w, o3);
        }
      } else if (RULE == RULE_GLA) {
#pragma unroll
        for (int r = 0; r < ROWS / 4; ++r) {
          const float4 qq = A[r], kk = B[r], dd = D[r];
          S[4 * r] = fmaf(dd.x, S[4 * r], kk.x * vj); o0 = fmaf(qq.x, S[4 * r], o0);
          S[4 * r + 1] = fmaf(dd.y, S[4 * r + 1], kk.y * vj); o1 = fmaf(qq.y, S[4 * r + 1], o1);
          S[4 * r + 2] = fmaf(dd.z, S[4 * r + 2], kk.z * vj); o2 = fmaf(qq.z, S[4 * r + 2], o2);
          S[4 * r + 3] = fmaf(dd.w, S[4 * r + 3], kk.w * vj); o3 = fmaf(qq.w, S[4 * r + 3], o3);
        }
      } else {
#pragma unroll
        for (int r = 0; r < ROWS / 4; ++r) {
          const float4 rr = A[r], kk = B[r], dd = D[r];
          float kv = kk.x * vj;
          o0 = fmaf(rr.x, fmaf(bonus[4 * r], kv, S[4 * r]), o0); S[4 * r] = fmaf(dd.x, S[4 * r], kv);
          kv = kk.y * vj;
          o1 = fmaf(rr.y, fmaf(bonus[4 * r + 1], kv, S[4 * r + 1]), o1); S[4 * r + 1] = fmaf(dd.y, S[4 * r + 1], kv);
          kv = kk.z * vj;
          o2 = fmaf(rr.z, fmaf(bonus[4 * r + 2], kv, S[4 * r + 2]), o2); S[4 * r + 2] = fmaf(dd.z, S[4 * r + 2], kv);
          kv = kk.w * vj;
          o3 = fmaf(rr.w, fmaf(bonus[4 * r + 3], kv, S[4 * r + 3]), o3); S[4 * r + 3] = fmaf(dd.w, S[4 * r + 3], kv);
        }
      }
      float o = (o0 + o1) + (o2 + o3);
      for (int off = L >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (RULE == RULE_GLA) o *= a.out_scale;
      if (active && part == 0) a.out[(int64_t)(t0 + c0 + tt) * a.H * dv + h * dv + col] = o;
    }
  };

  for (int e = tid; e < 2 * CHUNK * stride; e += blockDim.x) smem[e] = 0.f;
  __syncthreads();
  if (per_token <= STAGE_SLOTS * (int)blockDim.x) {
    // every thread fetches the same few values of every token: the next chunk's are on their way
    // to registers while this chunk is walked, and go to the other buffer afterwards
    StageSrc src[STAGE_SLOTS];
    int at[STAGE_SLOTS];
#pragma unroll
    for (int m = 0; m < STAGE_SLOTS; ++m) {
      const int k = tid + m * (int)blockDim.x;
      src[m] = source(k);
      at[m] = k < per_token ? place(k) : -1;
    }
    // The loads of a chunk are issued together, without a branch between them (a slot that
    // fetches nothing reads a valid word and drops it; tokens past the portion's end read its
    // last token again); what they brought is converted when it goes to shared memory.
    const char* from[STAGE_SLOTS];
    bool half[STAGE_SLOTS];
#pragma unroll
    for (int m = 0; m < STAGE_SLOTS; ++m) {
      half[m] = src[m].kind == 2 && sizeof(T) == 2;
      from[m] = src[m].kind == 0 ? reinterpret_cast<const char*>(a.decay) : src[m].p;
      if (src[m].kind == 0) src[m].stride = 0;
    }
    uint32_t regs[STAGE_SLOTS][CHUNK];
    auto fetch_chunk = [&](int c0) {
#pragma unroll
      for (int tt = 0; tt < CHUNK; ++tt) {
        const int64_t t = t0 + (c0 + tt < n ? c0 + tt : n - 1);
#pragma unroll
        for (int m = 0; m < STAGE_SLOTS; ++m) {
          const char* at_t = from[m] + t * src[m].stride;
          regs[m][tt] = half[m] ? (uint32_t)*reinterpret_cast<const unsigned short*>(at_t)
                                : *reinterpret_cast<const uint32_t*>(at_t);
        }
      }
    };
    auto store_chunk = [&](float* buf) {
#pragma unroll
      for (int m = 0; m < STAGE_SLOTS; ++m) {
        if (at[m] < 0) continue;
#pragma unroll
        for (int tt = 0; tt < CHUNK; ++tt) {
          float v = half[m] ? __uint_as_float(regs[m][tt] << 16) : __uint_as_float(regs[m][tt]);
          if (src[m].kind == 0) v = 0.f;
          buf[tt * stride + at[m]] = v;
        }
      }
    };
    fetch_chunk(0);
    store_chunk(smem);
    __syncthreads();
    int turn = 0;
    for (int c0 = 0; c0 < n; c0 += CHUNK, turn ^= 1) {
      const bool more = c0 + CHUNK < n;
      if (more) fetch_chunk(c0 + CHUNK);
      walk(smem + turn * CHUNK * stride, c0, n - c0 < CHUNK ? n - c0 : CHUNK);
      if (more) store_chunk(smem + (turn ^ 1) * CHUNK * stride);
      __syncthreads();
    }
  } else {
    for (int c0 = 0; c0 < n; c0 += CHUNK) {
      const int cn = n - c0 < CHUNK ? n - c0 : CHUNK;
      __syncthreads();
      for (int e = tid; e < cn * per_token; e += blockDim.x) {
        const int tt = e / per_token, k = e - tt * per_token;
        smem[tt * stride + place(k)] = fetch(source(k), t0 + c0 + tt);
      }
      __syncthreads();
      walk(smem, c0, cn);
    }
  }
  if (active) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int i = part * ROWS + r;
      if (i < dk) state[(int64_t)i * dv + col] = S[r];
    }
  }
  // the rest of the state: the last inputs of this portion, behind those that were carried
  if (blockIdx.y == 0 && blockIdx.z == 0 && a.carry_rows > 0) {
    float* carried = a.state + (int64_t)slot * a.state_stride + (int64_t)a.H * dk * dv;
    const T* src = reinterpret_cast<const T*>(a.carry_src);
    const int rows = a.carry_rows, W = a.carry_width;
    for (int c = tid; c < W; c += blockDim.x) {
      float keep[MAX_TAPS];
      for (int s = 0; s < rows; ++s) {
        const int from = n - rows + s;
        keep[s] = from >= 0 ? ls_to_float<T>(src[(int64_t)(t0 + from) * a.carry_ld + c]) : carried[(int64_t)(s + n) * W + c];
      }
      for (int s = 0; s < rows; ++s) carried[(int64_t)s * W + c] = keep[s];
    }
  }
}

// ---------------------------------------------------------------------------------------
// read-out: per-head RMSNorm, a gain, a gate
// ---------------------------------------------------------------------------------------
// out[t, h, j] = o[t, h, j] * rsqrt(mean_j o^2 + eps) * gain[shared ? j : h dv + j] * gate
//   gate_mode 0: gate_f32[t, h dv + j] as it is; 1: silu(gate_x[t, h dv + j]) from the engine's type;
//   2: sigmoid(gate_f32[t, h dv + j])
template <typename T>
__global__ void __launch_bounds__(PREP_THREADS) head_rms_gate_kernel(const float* __restrict__ o, const float* __restrict__ gain,
                                                                     const float* __restrict__ gate_f32,
                                                                     const T* __restrict__ gate_x, T* __restrict__ out,
                                                                     int H, int dv, int gain_shared, int gate_mode, float eps,
                                                                     int64_t gate_ld) {
  ls_dependency_sync();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int h = warp; h < H; h += PREP_THREADS / 32) {
    const int64_t base = ((int64_t)t * H + h) * dv;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) {
      const float v = o[base + j];
      ss = fmaf(v, v, ss);
    }
    ss = ls_warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int j = lane; j < dv; j += 32) {
      const float gt = gate_mode == 0 ? gate_f32[base + j]
                       : gate_mode == 2 ? sigmoid_f(gate_f32[base + j]) : silu_f(ls_to_float<T>(gate_x[(int64_t)t * gate_ld + h * dv + j]));
      out[base + j] = ls_from_float<T>(o[base + j] * rstd * gain[gain_shared ? j : h * dv + j] * gt);
    }
  }
}

int lanes_for(int dk) {
  int lanes = 1;
  while (lanes * ROWS < dk) lanes *= 2;
  return lanes;
}

}  // namespace

LS_API int ls_find_portions(const int* token_slot, int tokens, int* out, int cap, int* err, cudaStream_t stream) {
  if (tokens <= 0 || cap <= 0) return LS_E_SIZE;
  LS_COUNT(LS_K_FIND_PORTIONS);
  cudaError_t e = ls_launch(find_portions_kernel, dim3(1), dim3(PORTION_THREADS), 0, stream, token_slot, tokens, out, cap, err);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API int ls_delta_prep(const void* proj, int64_t ld, int dtype, const float* conv_w, const float* dt_bias,
                         const float* a_log, const float* state, int64_t state_stride, const int* token_slot,
                         float* qkv, float* decay, float* beta, int tokens, int H, int G, int dk, int dv, int taps,
                         float unit_eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || taps < 1 || taps > MAX_TAPS) return LS_E_SIZE;
  DeltaPrepArgs a;
  a.proj = proj; a.ld = ld; a.conv_w = conv_w; a.dt_bias = dt_bias; a.a_log = a_log; a.state = state;
  a.state_stride = state_stride; a.token_slot = token_slot; a.qkv = qkv; a.decay = decay; a.beta = beta; a.T = tokens;
  a.H = H; a.G = G; a.dk = dk; a.dv = dv; a.taps = taps; a.unit_eps = unit_eps;
  const size_t smem = sizeof(float) * (size_t)(2 * G * dk + H * dv + 2 * G);
  if (smem > 200 * 1024) return LS_E_SMEM;
  LS_COUNT(LS_K_DELTA_PREP);
  cudaError_t e;
  if (dtype == LS_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = ls_launch(delta_prep_kernel<float>, dim3(tokens), dim3(PREP_THREADS), smem, stream, a);
  } else if (dtype == LS_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prep_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = ls_launch(delta_prep_kernel<__nv_bfloat16>, dim3(tokens), dim3(PREP_THREADS), smem, stream, a);
  } else return LS_E_DTYPE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API int ls_double_exp_decay(float* z, const float* bias, long long count, int channels, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (channels <= 0) return LS_E_SIZE;
  LS_COUNT(LS_K_DOUBLE_EXP_DECAY);
  const dim3 grid((unsigned)((count + PREP_THREADS - 1) / PREP_THREADS));
  cudaError_t e = ls_launch(double_exp_decay_kernel, grid, dim3(PREP_THREADS), 0, stream, z, bias, (int64_t)count, channels);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API int ls_shift_mix(const void* x, int dtype, const float* mu, const float* state, int64_t state_stride,
                        int64_t prev_offset, const int* token_slot, void* out, int tokens, int width, int mixes,
                        cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || mixes <= 0) return LS_E_SIZE;
  LS_COUNT(LS_K_SHIFT_MIX);
  cudaError_t e;
  if (dtype == LS_F32)
    e = ls_launch(shift_mix_kernel<float>, dim3(tokens), dim3(PREP_THREADS), 0, stream, (const float*)x, mu, state,
                  state_stride, prev_offset, token_slot, (float*)out, tokens, width, mixes);
  else if (dtype == LS_BF16)
    e = ls_launch(shift_mix_kernel<__nv_bfloat16>, dim3(tokens), dim3(PREP_THREADS), 0, stream, (const __nv_bfloat16*)x,
                  mu, state, state_stride, prev_offset, token_slot, (__nv_bfloat16*)out, tokens, width, mixes);
  else return LS_E_DTYPE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API int ls_tanh_rows(void* x, int dtype, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  LS_COUNT(LS_K_TANH);
  const dim3 grid((unsigned)((count + PREP_THREADS - 1) / PREP_THREADS));
  cudaError_t e;
  if (dtype == LS_F32) e = ls_launch(tanh_kernel<float>, grid, dim3(PREP_THREADS), 0, stream, (float*)x, (int64_t)count);
  else if (dtype == LS_BF16) e = ls_launch(tanh_kernel<__nv_bfloat16>, grid, dim3(PREP_THREADS), 0, stream, (__nv_bfloat16*)x, (int64_t)count);
  else return LS_E_DTYPE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

// rule 0: the gated delta rule; rule 1: the wkv rule.  `dtype`: the engine's type (of r, k, v for
// rule 1, and of carry_src for both).
LS_API int ls_sigmoid_power_decay(float* z, const float* bias, long long count, int channels, float tau, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (channels <= 0 || !(tau > 0.f)) return LS_E_SIZE;
  LS_COUNT(LS_K_SIGMOID_POWER_DECAY);
  const dim3 grid((unsigned)((count + PREP_THREADS - 1) / PREP_THREADS));
  cudaError_t e = ls_launch(sigmoid_power_decay_kernel, grid, dim3(PREP_THREADS), 0, stream, z, bias, (int64_t)count, channels,
                            1.0f / tau);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API int ls_state_rule(int rule, int dtype, const int* portions, int max_portions, float* state, int64_t state_stride,
                         const void* in_a, const void* in_b, const void* in_v, const float* decay,
                         const float* beta, const float* bonus, float* out, const void* carry_src, int64_t carry_ld, int carry_width,
                         int carry_rows, int H, int G, int dk, int dv, int64_t in_ld, float out_scale,
                         int64_t decay_ld, cudaStream_t stream) {
  if (max_portions <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || dk <= 0 || dk > 32 * ROWS || dv <= 0 || carry_rows < 0 || carry_rows >= MAX_TAPS) return LS_E_SIZE;
  if (H > 65535) return LS_E_SIZE;
  RuleArgs a;
  a.portions = portions; a.state = state; a.state_stride = state_stride; a.in_a = in_a; a.in_b = in_b; a.in_v = in_v;
  a.decay = decay; a.beta = beta; a.bonus = bonus; a.out = out; a.carry_src = carry_src; a.carry_ld = carry_ld;
  a.carry_width = carry_width; a.carry_rows = carry_rows; a.H = H; a.G = G; a.dk = dk; a.dv = dv;
  a.lanes = lanes_for(dk);
  a.in_ld = in_ld; a.out_scale = out_scale;
  a.decay_ld = decay_ld < 0 ? (int64_t)H * dk : decay_ld;
  // columns a block: as many as fill 128 threads, fewer where the head has fewer
  int threads = 128;
  while (threads > 32 && (threads / 2) / a.lanes >= dv) threads /= 2;
  const int cb = threads / a.lanes;
  const dim3 grid(max_portions, H, (dv + cb - 1) / cb);
  // two buffers of CHUNK tokens, a token as the kernel lays it out
  const size_t smem = sizeof(float) * 2 * (size_t)CHUNK * (3 * a.lanes * (ROWS + 4) + ((cb + 3) & ~3) + 4);
  static bool configured = false;
  if (!configured) {
    const int most = 96 * 1024;
    if (cudaFuncSetAttribute(rule_kernel<RULE_DELTA, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
        cudaFuncSetAttribute(rule_kernel<RULE_DELTA, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
        cudaFuncSetAttribute(rule_kernel<RULE_WKV, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
        cudaFuncSetAttribute(rule_kernel<RULE_WKV, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
        cudaFuncSetAttribute(rule_kernel<RULE_GLA, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
        cudaFuncSetAttribute(rule_kernel<RULE_GLA, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess)
      return LS_E_SMEM;
    configured = true;
  }
  if (smem > 96 * 1024) return LS_E_SMEM;
  cudaError_t e;
  if (rule == RULE_DELTA) {
    LS_COUNT(LS_K_DELTA_RULE);
    if (dtype == LS_F32) e = ls_launch(rule_kernel<RULE_DELTA, float>, grid, dim3(threads), smem, stream, a);
    else if (dtype == LS_BF16) e = ls_launch(rule_kernel<RULE_DELTA, __nv_bfloat16>, grid, dim3(threads), smem, stream, a);
    else return LS_E_DTYPE;
  } else if (rule == RULE_WKV) {
    LS_COUNT(LS_K_WKV_RULE);
    if (dtype == LS_F32) e = ls_launch(rule_kernel<RULE_WKV, float>, grid, dim3(threads), smem, stream, a);
    else if (dtype == LS_BF16) e = ls_launch(rule_kernel<RULE_WKV, __nv_bfloat16>, grid, dim3(threads), smem, stream, a);
    else return LS_E_DTYPE;
  } else if (rule == RULE_GLA) {
    if (H != G || in_ld <= 0) return LS_E_SIZE;
    LS_COUNT(LS_K_GLA_RULE);
    if (dtype == LS_F32) e = ls_launch(rule_kernel<RULE_GLA, float>, grid, dim3(threads), smem, stream, a);
    else if (dtype == LS_BF16) e = ls_launch(rule_kernel<RULE_GLA, __nv_bfloat16>, grid, dim3(threads), smem, stream, a);
    else return LS_E_DTYPE;
  } else return LS_E_SIZE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

// gate_logit: gate_f32 holds logits, the gate is their sigmoid
LS_API int ls_head_rms_gate(const float* o, const float* gain, const float* gate_f32, const void* gate_x, void* out,
                            int dtype, int tokens, int H, int dv, int gain_shared, int gate_logit, float eps,
                            int64_t gate_ld, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || dv <= 0 || (gate_f32 == nullptr) == (gate_x == nullptr)) return LS_E_SIZE;
  const int mode = gate_f32 != nullptr ? (gate_logit ? 2 : 0) : 1;
  if (gate_ld <= 0) gate_ld = (int64_t)H * dv;       // the gate's rows lie one after the other
  LS_COUNT(LS_K_HEAD_RMS_GATE);
  cudaError_t e;
  if (dtype == LS_F32)
    e = ls_launch(head_rms_gate_kernel<float>, dim3(tokens), dim3(PREP_THREADS), 0, stream, o, gain, gate_f32,
                  (const float*)gate_x, (float*)out, H, dv, gain_shared, mode, eps, gate_ld);
  else if (dtype == LS_BF16)
    e = ls_launch(head_rms_gate_kernel<__nv_bfloat16>, dim3(tokens), dim3(PREP_THREADS), 0, stream, o, gain, gate_f32,
                  (const __nv_bfloat16*)gate_x, (__nv_bfloat16*)out, H, dv, gain_shared, mode, eps, gate_ld);
  else return LS_E_DTYPE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

LS_API void ls_set_dependent_launch_seq(int on) { ls_dependent_launch = on ? 1 : 0; }
LS_API const char* ls_kernel_names_seq() { return LS_KERNEL_NAMES; }
LS_API int ls_kernel_launches_seq(unsigned long long* out, int n) {
  for (int i = 0; i < n && i < LS_K_COUNT; ++i) out[i] = ls_kernel_launches[i];
  return LS_K_COUNT;
}
LS_API const char* ls_constants_recurrent() {
  static char buf[256];
  static const LsConstant c[] = {{"recurrent.rows_per_thread", ROWS}, {"recurrent.chunk_tokens", CHUNK},
                                 {"recurrent.max_taps", MAX_TAPS}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}
