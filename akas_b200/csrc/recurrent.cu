// Mixers with a matrix state per head: gated linear attention and the gated delta rule, and what stands around
// their recurrences (low-rank decay gates, a causal depthwise convolution with silu, unit-length q and k, the
// step sizes and decays of the delta rule, the gated RMS norm of the read-out).
//
// Everything here is float32 arithmetic whatever the compute dtype; inputs that a matrix product wrote may be
// bfloat16 and are widened on load. The recurrences run token by token in one fixed order per (request, head,
// value channel), so a request's results do not depend on how its tokens were cut into steps or on what else
// is in the batch.
//
// State layouts (one row per request slot; only the slot stride is free, so a state may be part of a wider
// row): a matrix state is S^T, [heads, value_dim, key_dim] float32, so that the key channels a thread owns are
// contiguous; a convolution's state is its last taps - 1 inputs, [taps - 1, channels] float32, oldest first.
#include "common.cuh"

using namespace akas;

namespace {

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// ------------------------------------------------------------------------------------------------ decay gates
//
// out[n, o] = sigmoid(z)^(1 / tau), z = sum_r low[n, r] * wt[r, o] + bias[o]: the up projection of a low-rank pair in
// float32 (one ascending chain of fused multiply-adds per output), then exp(log sigmoid(z) / tau). The matrix comes
// transposed, [R, O], so that the threads of a warp read neighbouring words.
constexpr int kGateTokens = 8;

template <typename T>
__global__ void decay_gates_kernel(const T* __restrict__ low, long long ld, const float* __restrict__ w,
                                   const float* __restrict__ bias, float* __restrict__ out, int N, int O, int R,
                                   float inv_tau) {
  extern __shared__ float rows[];  // [kGateTokens][R]
  const int n0 = blockIdx.x * kGateTokens;
  for (int i = threadIdx.x; i < kGateTokens * R; i += blockDim.x) {
    const int t = i / R, r = i % R;
    rows[i] = n0 + t < N ? to_f32(low[(size_t)(n0 + t) * ld + r]) : 0.f;
  }
  __syncthreads();
  for (int o = blockIdx.y * blockDim.x + threadIdx.x; o < O; o += gridDim.y * blockDim.x) {
    float acc[kGateTokens];
#pragma unroll
    for (int t = 0; t < kGateTokens; ++t) acc[t] = 0.f;
    for (int r = 0; r < R; ++r) {
      const float wv = w[(size_t)r * O + o];
#pragma unroll
      for (int t = 0; t < kGateTokens; ++t) acc[t] = fmaf(rows[t * R + r], wv, acc[t]);
    }
    const float b = bias[o];
#pragma unroll
    for (int t = 0; t < kGateTokens; ++t)
      if (n0 + t < N) out[(size_t)(n0 + t) * O + o] = expf(-softplus_f(-(acc[t] + b)) * inv_tau);
  }
}

// ------------------------------------------------------------------------------------------------ the recurrences
//
// One block of TH threads per (head, request, tile of value channels). A thread owns R consecutive key channels of one value
// channel j: s[r] = S[ks * R + r][j]; the KS threads of a value channel are neighbouring lanes of a warp and add
// their partial sums by shuffles. The step's tokens come through shared memory in chunks of CH (fewer where rows are long).
//
//   GLA:    s <- alpha_t[kk] s + k_t[kk] v_t[j];                                  o_t[j] = sum_kk s q_t[kk]
//   FIXED:  the same with one constant decay per head in place of alpha_t[kk] (decay [H]); with `act`, q, k and v
//           pass silu on their way in (the mixer's activations, applied in float32).
//   DELTA:  s <- g_t s; u = beta_t (v_t[j] - sum_kk s k_t[kk]); s <- s + k_t[kk] u; o_t[j] = sum_kk s q_t[kk]
constexpr int kPad = 4;  // floats between the R-blocks of a shared row: neighbouring lanes' 16-byte reads miss each other's banks

template <int KS> __device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = KS / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T, int R, int KS, int CH, int TH, bool DELTA, bool FIXED = false>
__global__ void __launch_bounds__(TH)
scan_kernel(const T* __restrict__ q, long long ldq, const T* __restrict__ k, long long ldk, const T* __restrict__ v,
            long long ldv, const float* __restrict__ decay /* GLA: alpha [N, H * D]; DELTA: g [N, H] */,
            const float* __restrict__ beta /* DELTA: [N, H] */, float* __restrict__ state, long long slot_stride,
            const int* __restrict__ cu_seqlens, const int* __restrict__ slots, float* __restrict__ out, int H, int rep,
            int D, int V, float q_scale, int write, int act) {
  constexpr int VT = TH / KS;           // value channels of a block
  constexpr int ROW = KS * (R + kPad);  // floats of a padded shared row of key channels
  __shared__ __align__(16) float sq[CH][ROW];
  __shared__ __align__(16) float sk[CH][ROW];
  __shared__ __align__(16) float sa[DELTA || FIXED ? 1 : CH][DELTA || FIXED ? 4 : ROW];
  __shared__ float sv[CH][VT];
  __shared__ float sg[CH], sb[CH];

  const int h = blockIdx.x, req = blockIdx.y;
  const int slot = slots[req];
  const int t_begin = cu_seqlens[req], t_end = cu_seqlens[req + 1];
  if (slot < 0 || t_end <= t_begin) return;
  const int ks = threadIdx.x % KS, jl = threadIdx.x / KS;
  const int j = blockIdx.z * VT + jl;
  const bool live = j < V;
  const int hk = h / rep;  // the q/k head that this head reads
  const int kk0 = ks * R;

  float s[R];
  float* srow = state + (size_t)slot * slot_stride + ((size_t)h * V + (live ? j : 0)) * D;
  const bool vec = D % 4 == 0 && slot_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(state) & 15) == 0;
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    if (live && vec && kk0 + r + 3 < D) {
      const float4 x = *reinterpret_cast<const float4*>(srow + kk0 + r);
      s[r] = x.x; s[r + 1] = x.y; s[r + 2] = x.z; s[r + 3] = x.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[r + e] = live && kk0 + r + e < D ? srow[kk0 + r + e] : 0.f;
    }
  }

  // A chunk's inputs are fetched into registers while the chunk before it is computed, and put into shared memory
  // when that is done: the recurrence never waits for global memory except at its first chunk.
  constexpr int NQ = (CH * KS * R + TH - 1) / TH, NV = (CH * VT + TH - 1) / TH;
  T rq[NQ], rk[NQ], rv[NV];  // as fetched: widening them here would make the loop below wait for the loads at once
  float ra[DELTA || FIXED ? 1 : NQ], rg = 0.f, rb = 0.f;
  const float fixed = FIXED ? decay[h] : 0.f;
  const T zero = from_f32<T>(0.f);
  auto fetch = [&](int c0) {
    const int count = min(CH, t_end - c0);
#pragma unroll
    for (int u = 0; u < NQ; ++u) {
      const int i = threadIdx.x + u * TH;
      const int t = i / (KS * R), kk = i % (KS * R);
      const bool in = t < count && kk < D;
      const size_t n = (size_t)(c0 + t);
      rq[u] = in ? q[n * ldq + (size_t)hk * D + kk] : zero;
      rk[u] = in ? k[n * ldk + (size_t)hk * D + kk] : zero;
      if (!DELTA && !FIXED) ra[u] = in ? decay[n * ((size_t)H * D) + (size_t)h * D + kk] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      const int i = threadIdx.x + u * TH;
      const int t = i / VT, col = blockIdx.z * VT + i % VT;
      rv[u] = t < count && col < V ? v[(size_t)(c0 + t) * ldv + (size_t)h * V + col] : zero;
    }
    if (DELTA && threadIdx.x < count) {
      rg = decay[(size_t)(c0 + threadIdx.x) * H + h];
      rb = beta[(size_t)(c0 + threadIdx.x) * H + h];
    }
  };
  fetch(t_begin);
  for (int c0 = t_begin; c0 < t_end; c0 += CH) {
    const int count = min(CH, t_end - c0);
    __syncthreads();  // the chunk before has been read
#pragma unroll
    for (int u = 0; u < NQ; ++u) {
      const int i = threadIdx.x + u * TH;
      if (i < CH * KS * R) {
        const int t = i / (KS * R), kk = i % (KS * R);
        const int at = kk + (kk / R) * kPad;
        float qv = to_f32(rq[u]), kv = to_f32(rk[u]);
        if (FIXED && act) { qv *= sigmoid_f(qv); kv *= sigmoid_f(kv); }
        sq[t][at] = qv * q_scale;
        sk[t][at] = kv;
        if (!DELTA && !FIXED) sa[t][at] = ra[u];
      }
    }
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      const int i = threadIdx.x + u * TH;
      if (i < CH * VT) {
        float vv = to_f32(rv[u]);
        if (FIXED && act) vv *= sigmoid_f(vv);
        sv[i / VT][i % VT] = vv;
      }
    }
    if (DELTA && threadIdx.x < CH) {
      sg[threadIdx.x] = rg;
      sb[threadIdx.x] = rb;
    }
    __syncthreads();
    if (c0 + CH < t_end) fetch(c0 + CH);
#pragma unroll 2
    for (int t = 0; t < count; ++t) {
      const float* qr = &sq[t][ks * (R + kPad)];
      const float* kr = &sk[t][ks * (R + kPad)];
      const float vj = sv[t][jl];
      float acc = 0.f, acc2 = 0.f;  // two chains of sums, added before the lanes meet: always in this order
      if (DELTA) {
        const float g = sg[t];
        float pk = 0.f, pk2 = 0.f;
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(kr + r);
          s[r] *= g; s[r + 1] *= g; s[r + 2] *= g; s[r + 3] *= g;
          pk = fmaf(s[r], kv.x, pk); pk2 = fmaf(s[r + 1], kv.y, pk2); pk = fmaf(s[r + 2], kv.z, pk); pk2 = fmaf(s[r + 3], kv.w, pk2);
        }
        pk = group_sum<KS>(pk + pk2);
        const float u = sb[t] * (vj - pk);
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(kr + r);
          const float4 qv = *reinterpret_cast<const float4*>(qr + r);
          s[r] = fmaf(kv.x, u, s[r]); s[r + 1] = fmaf(kv.y, u, s[r + 1]);
          s[r + 2] = fmaf(kv.z, u, s[r + 2]); s[r + 3] = fmaf(kv.w, u, s[r + 3]);
          acc = fmaf(s[r], qv.x, acc); acc2 = fmaf(s[r + 1], qv.y, acc2); acc = fmaf(s[r + 2], qv.z, acc); acc2 = fmaf(s[r + 3], qv.w, acc2);
        }
      } else if (FIXED) {
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(kr + r);
          const float4 qv = *reinterpret_cast<const float4*>(qr + r);
          s[r] = fmaf(fixed, s[r], kv.x * vj); s[r + 1] = fmaf(fixed, s[r + 1], kv.y * vj);
          s[r + 2] = fmaf(fixed, s[r + 2], kv.z * vj); s[r + 3] = fmaf(fixed, s[r + 3], kv.w * vj);
          acc = fmaf(s[r], qv.x, acc); acc2 = fmaf(s[r + 1], qv.y, acc2); acc = fmaf(s[r + 2], qv.z, acc); acc2 = fmaf(s[r + 3], qv.w, acc2);
        }
      } else {
        const float* ar = &sa[t][ks * (R + kPad)];
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(kr + r);
          const float4 qv = *reinterpret_cast<const float4*>(qr + r);
          const float4 av = *reinterpret_cast<const float4*>(ar + r);
          s[r] = fmaf(av.x, s[r], kv.x * vj); s[r + 1] = fmaf(av.y, s[r + 1], kv.y * vj);
          s[r + 2] = fmaf(av.z, s[r + 2], kv.z * vj); s[r + 3] = fmaf(av.w, s[r + 3], kv.w * vj);
          acc = fmaf(s[r], qv.x, acc); acc2 = fmaf(s[r + 1], qv.y, acc2); acc = fmaf(s[r + 2], qv.z, acc); acc2 = fmaf(s[r + 3], qv.w, acc2);
        }
      }
      acc = group_sum<KS>(acc + acc2);
      if (ks == 0 && live) out[(size_t)(c0 + t) * ((size_t)H * V) + (size_t)h * V + j] = acc;
    }
  }
  if (write && live) {
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      if (vec && kk0 + r + 3 < D) {
        *reinterpret_cast<float4*>(srow + kk0 + r) = make_float4(s[r], s[r + 1], s[r + 2], s[r + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (kk0 + r + e < D) srow[kk0 + r + e] = s[r + e];
      }
    }
  }
}

template <typename T, bool DELTA, bool FIXED = false>
int launch_scan(const T* q, long long ldq, const T* k, long long ldk, const T* v, long long ldv, const float* decay,
                const float* beta, float* state, long long slot_stride, const int* cu_seqlens, const int* slots, float* out,
                int tokens, int requests, int H, int rep, int D, int V, float q_scale, int write, cudaStream_t stream,
                int act = 0) {
  if (requests <= 0 || H <= 0) return 0;
  if (D > 1024) return (int)cudaErrorInvalidValue;
  // (Blocks of 64 threads, which spread a head's value channels over four times as many SMs when a step holds few
  // long portions, were measured and dropped: a token's cost is the latency of its chain of shared-memory reads, sums
  // and shuffles, which fewer warps per SM hide less well. 2,048 tokens, 16 heads of 128 x 128: 0.94 against 0.75 ms.)
  (void)tokens;
#define AKAS_SCAN(R, KS, CH)                                                                                              \
  {                                                                                                                       \
    const dim3 grid(H, requests, (V + 256 / KS - 1) / (256 / KS));                                                        \
    return launch_ordinary(scan_kernel<T, R, KS, CH, 256, DELTA, FIXED>, grid, dim3(256), 0, stream, q, ldq, k, ldk, v, ldv,  \
                          decay, beta, state, slot_stride, cu_seqlens, slots, out, H, rep, D, V, q_scale, write, act);    \
  }
  if (D <= 8) AKAS_SCAN(8, 1, 16)
  if (D <= 16) AKAS_SCAN(8, 2, 16)
  if (D <= 32) AKAS_SCAN(8, 4, 16)
  if (D <= 64) AKAS_SCAN(16, 4, 16)
  if (D <= 128) AKAS_SCAN(16, 8, 16)
  if (D <= 256) AKAS_SCAN(16, 16, 8)
  if (D <= 512) AKAS_SCAN(16, 32, 4)
  AKAS_SCAN(32, 32, 2)
#undef AKAS_SCAN
}

// ------------------------------------------------------------------------------------------------ fixed decay, in chunks
//
// The recurrence with one constant decay per head, S <- a S + k v^T, o = S^T q, for prompt portions: a request's
// tokens of this step are cut into chunks of kChunk, and three kernels replace the walk token by token.
//   chunk_state   per (chunk, head, tile of value channels): U = sum_s a^(len - 1 - s) v_s k_s^T, what the chunk's
//                 tokens add to the state by the chunk's end;
//   chunk_carry   per (request, head): S_0 = the slot's state; the state at every chunk's start, S_(j+1) = a^len_j S_j
//                 + U_j, written where U_j stood; the last one back to the slot;
//   chunk_output  per (chunk, head, tile of value channels): o_t = a^(t + 1) S_j^T q_t + sum_(s <= t) a^(t - s) (q_t . k_s) v_s.
// Everything is float32 fused multiply-adds (the decays' powers come from a float64 pow, rounded once); sums run in
// a fixed order that depends on where a chunk starts in the step, so a result differs from the token-by-token
// kernel's, and between ways of cutting a prompt, by rounding only. Key sizes up to kChunkMaxD.
constexpr int kChunk = 64, kChunkVT = 64, kChunkMaxD = 128, kChunkThreads = 256;

// which (request, chunk of it) the block's chunk number is; false if there is none
__device__ __forceinline__ bool find_chunk(const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int R, int id,
                                           int& req, int& first, int& len, int& index) {
  for (int r = 0; r < R; ++r) {
    const int b = cu_seqlens[r], e = cu_seqlens[r + 1];
    const int chunks = slots[r] < 0 ? 0 : (e - b + kChunk - 1) / kChunk;
    if (id < chunks) {
      req = r; index = id; first = b + id * kChunk; len = min(kChunk, e - first);
      return true;
    }
    id -= chunks;
  }
  return false;
}

// Stages `live` rows of `cols` channels (src row pitch ld) into shared memory rows of `pitch` floats as float32, silu'd
// where `act`, times `scale` or, where `pw` is given, times pw[live - 1 - row]; rows from `live` to `rows` and the columns
// from `cols` to `pitch` become zero. Eight channels a load where the sizes allow: a chunk's inputs are then two or
// four loads a thread, all in flight together, where one channel a load made the block wait on memory most of its time.
template <typename T>
__device__ __forceinline__ void stage_rows(float* __restrict__ dst, int pitch, const T* __restrict__ src, long long ld, int live,
                                           int cols, int rows, float scale, const float* __restrict__ pw, int act) {
  const bool vec = cols % 8 == 0 && ld % 8 == 0 && ((uintptr_t)src % 16) == 0;
  if (vec) {
    const int per = cols / 8;
    for (int i = threadIdx.x; i < rows * per; i += kChunkThreads) {
      const int t = i / per, c = (i % per) * 8;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (t < live) {
        load8(src + (size_t)t * ld + c, v);
        const float f = pw != nullptr ? pw[live - 1 - t] : scale;
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (act ? v[j] * sigmoid_f(v[j]) : v[j]) * f;
      }
      *reinterpret_cast<float4*>(dst + t * pitch + c) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(dst + t * pitch + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    const int pad = pitch - cols;
    for (int i = threadIdx.x; i < rows * pad; i += kChunkThreads) dst[(i / pad) * pitch + cols + i % pad] = 0.f;
    return;
  }
  for (int i = threadIdx.x; i < rows * pitch; i += kChunkThreads) {
    const int t = i / pitch, c = i % pitch;
    float x = 0.f;
    if (t < live && c < cols) {
      x = to_f32(src[(size_t)t * ld + c]);
      x = (act ? x * sigmoid_f(x) : x) * (pw != nullptr ? pw[live - 1 - t] : scale);
    }
    dst[i] = x;
  }
}

template <typename T>
__global__ void __launch_bounds__(kChunkThreads)
chunk_state_kernel(const T* __restrict__ k, long long ldk, const T* __restrict__ v, long long ldv, const float* __restrict__ decay,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ slots, float* __restrict__ scratch, int R, int H,
                   int D, int V, int DP, int act) {
  extern __shared__ __align__(16) float sm[];
  float* sk = sm;                    // [kChunk][DP]
  float* sv = sk + kChunk * DP;      // [kChunk][kChunkVT], already times a^(len - 1 - s)
  float* pw = sv + kChunk * kChunkVT;  // [kChunk] powers of the decay
  int req, first, len, index;
  if (!find_chunk(cu_seqlens, slots, R, blockIdx.x, req, first, len, index)) return;
  const int h = blockIdx.y, v0 = blockIdx.z * kChunkVT;
  const double a = (double)decay[h];
  for (int i = threadIdx.x; i < kChunk; i += kChunkThreads) pw[i] = (float)pow(a, (double)i);
  __syncthreads();
  stage_rows(sk, DP, k + (size_t)first * ldk + (size_t)h * D, ldk, len, D, kChunk, 1.f, nullptr, act);
  stage_rows(sv, kChunkVT, v + (size_t)first * ldv + (size_t)h * V + v0, ldv, len, min(kChunkVT, V - v0), kChunk, 1.f, pw, act);
  __syncthreads();
  // a thread owns 4 value channels x 4 key channels at a time
  const int tv = (threadIdx.x / 16) * 4, td = (threadIdx.x % 16) * 4;  // 16 x 16 threads cover 64 x 64
  float* out = scratch + ((size_t)blockIdx.x * H + h) * V * D;
  for (int d0 = 0; d0 < DP; d0 += 64) {
    float acc[4][4] = {};
    if (d0 + td < DP) {
      for (int t = 0; t < kChunk; ++t) {
        const float4 kv = *reinterpret_cast<const float4*>(sk + t * DP + d0 + td);
        const float4 vv = *reinterpret_cast<const float4*>(sv + t * kChunkVT + tv);
        const float kk[4] = {kv.x, kv.y, kv.z, kv.w}, vs[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(vs[i], kk[j], acc[i][j]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (v0 + tv + i < V && d0 + td + j < D) out[(size_t)(v0 + tv + i) * D + d0 + td + j] = acc[i][j];
  }
}

// One block per (request, head): walks the request's chunks; every element of the state is one thread's chain.
__global__ void chunk_carry_kernel(const float* __restrict__ decay, float* __restrict__ state, long long slot_stride,
                                   const int* __restrict__ cu_seqlens, const int* __restrict__ slots, float* __restrict__ scratch,
                                   int R, int H, int D, int V, int write) {
  const int req = blockIdx.x, h = blockIdx.y;
  const int slot = slots[req];
  if (slot < 0) return;
  int base = 0;  // the number of the request's first chunk
  for (int r = 0; r < req; ++r) base += slots[r] < 0 ? 0 : (cu_seqlens[r + 1] - cu_seqlens[r] + kChunk - 1) / kChunk;
  const int n = cu_seqlens[req + 1] - cu_seqlens[req];
  const int chunks = (n + kChunk - 1) / kChunk;
  if (chunks == 0) return;
  const double a = (double)decay[h];
  const float whole = (float)pow(a, (double)kChunk), last = (float)pow(a, (double)(n - (chunks - 1) * kChunk));
  float* srow = state + (size_t)slot * slot_stride + (size_t)h * V * D;
  for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < V * D; i += gridDim.z * blockDim.x) {
    float s = srow[i];
    for (int j0 = 0; j0 < chunks; j0 += 8) {  // eight chunks' sums are fetched at once: the chain itself waits for no load
      float add[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) add[e] = j0 + e < chunks ? scratch[((size_t)(base + j0 + e) * H + h) * V * D + i] : 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (j0 + e < chunks) {
          scratch[((size_t)(base + j0 + e) * H + h) * V * D + i] = s;
          s = fmaf(j0 + e + 1 < chunks ? whole : last, s, add[e]);
        }
      }
    }
    if (write) srow[i] = s;
  }
}

template <typename T>
__global__ void __launch_bounds__(kChunkThreads)
chunk_output_kernel(const T* __restrict__ q, long long ldq, const T* __restrict__ k, long long ldk, const T* __restrict__ v,
                    long long ldv, const float* __restrict__ decay, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ slots, const float* __restrict__ scratch, float* __restrict__ out, int R, int H, int D,
                    int V, int DP, float q_scale, int act) {
  extern __shared__ __align__(16) float sm[];
  float* sq = sm;                        // [kChunk][DP]
  float* sk = sq + kChunk * DP;          // [kChunk][DP]
  float* ss = sk + kChunk * DP;          // [kChunkVT][DP] the state at the chunk's start (rows: value channels)
  float* sv = ss + kChunkVT * DP;        // [kChunk][kChunkVT]
  float* sa = sv + kChunk * kChunkVT;    // [kChunk][kChunk] decayed scores, zero above the diagonal
  float* pw = sa + kChunk * kChunk;      // [kChunk + 1] powers of the decay
  int req, first, len, index;
  if (!find_chunk(cu_seqlens, slots, R, blockIdx.x, req, first, len, index)) return;
  const int h = blockIdx.y, v0 = blockIdx.z * kChunkVT;
  const double a = (double)decay[h];
  for (int i = threadIdx.x; i <= kChunk; i += kChunkThreads) pw[i] = (float)pow(a, (double)i);
  stage_rows(sq, DP, q + (size_t)first * ldq + (size_t)h * D, ldq, len, D, kChunk, q_scale, nullptr, act);
  stage_rows(sk, DP, k + (size_t)first * ldk + (size_t)h * D, ldk, len, D, kChunk, 1.f, nullptr, act);
  // the state at the chunk's start: rows are this tile's value channels
  stage_rows(ss, DP, scratch + ((size_t)blockIdx.x * H + h) * V * D + (size_t)v0 * D, (long long)D, min(kChunkVT, V - v0), D, kChunkVT,
             1.f, nullptr, 0);
  stage_rows(sv, kChunkVT, v + (size_t)first * ldv + (size_t)h * V + v0, ldv, len, min(kChunkVT, V - v0), kChunk, 1.f, nullptr, act);
  __syncthreads();
  // A thread's part of a 64 x 64 result: rows tr .. tr + 3 and columns tc, tc + 16, tc + 32, tc + 48. Where a column
  // is a row of shared memory (a key, a value channel of the state), the 8 threads of a quarter of a warp read 8
  // neighbouring rows, whose 16-byte words lie in different banks (rows are DP = 4 mod 8 floats apart); with four
  // neighbouring columns a thread, they would read rows 4 apart and meet in two banks.
  const int tr = (threadIdx.x / 16) * 4, tc = threadIdx.x % 16;
  {  // scores of queries tr.. against keys tc + 16 j, times a^(t - s) on and below the diagonal
    float acc[4][4] = {};
    for (int d = 0; d < DP; d += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        qv[i] = *reinterpret_cast<const float4*>(sq + (tr + i) * DP + d);
        kv[i] = *reinterpret_cast<const float4*>(sk + (tc + 16 * i) * DP + d);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(qv[i].x, kv[j].x, acc[i][j]); acc[i][j] = fmaf(qv[i].y, kv[j].y, acc[i][j]);
          acc[i][j] = fmaf(qv[i].z, kv[j].z, acc[i][j]); acc[i][j] = fmaf(qv[i].w, kv[j].w, acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = tc + 16 * j;
        sa[(tr + i) * kChunk + key] = key <= tr + i ? acc[i][j] * pw[tr + i - key] : 0.f;
      }
  }
  __syncthreads();
  float acc[4][4] = {};  // tokens tr.. x value channels tc + 16 j
  for (int t = 0; t < min(tr + 4, len); ++t) {  // keys up to the thread's last query
    float vv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) vv[j] = sv[t * kChunkVT + tc + 16 * j];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float w = sa[(tr + i) * kChunk + t];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(w, vv[j], acc[i][j]);
    }
  }
  float carry[4][4] = {};  // what the state at the chunk's start gives: S^T q, times a^(t + 1) below
  for (int d = 0; d < DP; d += 4) {
    float4 qv[4], sr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      qv[i] = *reinterpret_cast<const float4*>(sq + (tr + i) * DP + d);
      sr[i] = *reinterpret_cast<const float4*>(ss + (tc + 16 * i) * DP + d);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        carry[i][j] = fmaf(qv[i].x, sr[j].x, carry[i][j]); carry[i][j] = fmaf(qv[i].y, sr[j].y, carry[i][j]);
        carry[i][j] = fmaf(qv[i].z, sr[j].z, carry[i][j]); carry[i][j] = fmaf(qv[i].w, sr[j].w, carry[i][j]);
      }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (tr + i < len && v0 + tc + 16 * j < V)
        out[(size_t)(first + tr + i) * ((size_t)H * V) + (size_t)h * V + v0 + tc + 16 * j] = fmaf(pw[tr + i + 1], carry[i][j], acc[i][j]);
}

template <typename T>
int launch_chunks(const T* q, long long ldq, const T* k, long long ldk, const T* v, long long ldv, const float* decay, float* state,
                  long long slot_stride, const int* cu_seqlens, const int* slots, float* out, float* scratch, int tokens,
                  int requests, int H, int D, int V, float q_scale, int act, int write, cudaStream_t stream) {
  const int DP = (D + 7) / 8 * 8 + 4;  // rows of key channels in shared memory: whole 16-byte words, 4 mod 8 floats apart (see chunk_output)
  const int chunks = (tokens + kChunk - 1) / kChunk + requests;  // at most: every request may end with a part of a chunk
  const int vt = (V + kChunkVT - 1) / kChunkVT;
  const size_t smem1 = sizeof(float) * ((size_t)kChunk * DP + kChunk * kChunkVT + kChunk);
  const size_t smem3 = sizeof(float) * ((size_t)2 * kChunk * DP + (size_t)kChunkVT * DP + kChunk * kChunkVT + kChunk * kChunk + kChunk + 4);
  static bool configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (!configured[device]) {
    const int most = (int)(sizeof(float) * ((size_t)2 * kChunk * (kChunkMaxD + 12) + (size_t)kChunkVT * (kChunkMaxD + 12) + kChunk * kChunkVT +
                                           kChunk * kChunk + kChunk + 4));
    cudaError_t e = cudaFuncSetAttribute(chunk_output_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(chunk_output_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(chunk_state_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(chunk_state_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  int err = launch_ordinary(chunk_state_kernel<T>, dim3(chunks, H, vt), dim3(kChunkThreads), smem1, stream, k, ldk, v, ldv, decay,
                            cu_seqlens, slots, scratch, requests, H, D, V, DP, act);
  if (err) return err;
  err = launch_ordinary(chunk_carry_kernel, dim3(requests, H, min(64, (V * D + 255) / 256)), dim3(256), 0, stream, decay, state,
                        slot_stride, cu_seqlens, slots, scratch, requests, H, D, V, write);
  if (err) return err;
  return launch_ordinary(chunk_output_kernel<T>, dim3(chunks, H, vt), dim3(kChunkThreads), smem3, stream, q, ldq, k, ldk, v, ldv, decay,
                         cu_seqlens, slots, (const float*)scratch, out, requests, H, D, V, DP, q_scale, act);
}

// ------------------------------------------------------------------------------------------------ causal convolution
//
// y[n, c] = silu(sum_j taps[c, j] * x_(i - L + 1 + j)) for the i-th token of its request in this step; inputs before
// the step's first token come from the request's state rows. One ascending chain of fused multiply-adds per output.
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ taps,
                                        const float* __restrict__ state, long long slot_stride,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ seq_of_token,
                                        const int* __restrict__ slots, float* __restrict__ y, int C, int L) {
  const int n = blockIdx.x;
  const int req = seq_of_token[n];
  if (req < 0) return;
  const int slot = slots[req];
  if (slot < 0) return;
  const int first = cu_seqlens[req];
  const int i = n - first;
  const float* st = state + (size_t)slot * slot_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < L; ++j) {
      const int src = i - (L - 1) + j;
      const float in = src >= 0 ? to_f32(x[(size_t)(first + src) * ldx + c]) : st[(size_t)(L - 1 + src) * C + c];
      acc = fmaf(taps[(size_t)c * L + j], in, acc);
    }
    y[(size_t)n * C + c] = acc * sigmoid_f(acc);
  }
}

// The same for four neighbouring channels a thread (C, the row pitches and the slot pitch multiples of 4, rows on 16
// bytes): inputs move 8 or 16 bytes at a time, results 16.
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
  const uint2 a = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xffff0000u);
  v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xffff0000u);
}

template <typename T>
__global__ void causal_conv_silu4_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ taps,
                                         const float* __restrict__ state, long long slot_stride,
                                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_of_token,
                                         const int* __restrict__ slots, float* __restrict__ y, int C, int L) {
  const int n = blockIdx.x;
  const int req = seq_of_token[n];
  if (req < 0) return;
  const int slot = slots[req];
  if (slot < 0) return;
  const int first = cu_seqlens[req];
  const int i = n - first;
  const float* st = state + (size_t)slot * slot_stride;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < C; c += gridDim.y * blockDim.x * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < L; ++j) {
      const int src = i - (L - 1) + j;
      float in[4];
      if (src >= 0) load4(x + (size_t)(first + src) * ldx + c, in);
      else load4(st + (size_t)(L - 1 + src) * C + c, in);
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] = fmaf(taps[(size_t)(c + e) * L + j], in[e], acc[e]);
    }
    *reinterpret_cast<float4*>(y + (size_t)n * C + c) =
        make_float4(acc[0] * sigmoid_f(acc[0]), acc[1] * sigmoid_f(acc[1]), acc[2] * sigmoid_f(acc[2]), acc[3] * sigmoid_f(acc[3]));
  }
}

// The state after the step: the last L - 1 inputs of each request, from the step's tokens and, where those are fewer,
// from the rows the state held. Row i takes what is n_r rows further on, so ascending i never overwrites a row that
// is still to be read.
template <typename T>
__global__ void causal_conv_state_kernel(const T* __restrict__ x, long long ldx, float* __restrict__ state,
                                         long long slot_stride, const int* __restrict__ cu_seqlens,
                                         const int* __restrict__ slots, int C, int L) {
  const int req = blockIdx.x;
  const int slot = slots[req];
  const int first = cu_seqlens[req], count = cu_seqlens[req + 1] - first;
  if (slot < 0 || count <= 0) return;
  float* st = state + (size_t)slot * slot_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    for (int i = 0; i < L - 1; ++i) {
      const int src = count - (L - 1) + i;  // index among the step's tokens
      st[(size_t)i * C + c] = src >= 0 ? to_f32(x[(size_t)(first + src) * ldx + c]) : st[(size_t)(i + count) * C + c];
    }
  }
}

// ------------------------------------------------------------------------------------------------ delta rule inputs
//
// One block per token. Heads of q (the first G * D columns of y) and of k (the next G * D) become unit vectors,
// x / sqrt(sum x^2 + unit_eps), q times q_scale too; beta = sigmoid(b); g = exp(-exp(A_log) * softplus(a + dt_bias)).
template <typename T>
__global__ void delta_prep_kernel(float* __restrict__ y, long long ldy, int G, int D, float q_scale, float unit_eps,
                                  const T* __restrict__ b, long long ldb, const T* __restrict__ a, long long lda,
                                  const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                  float* __restrict__ beta, float* __restrict__ g, int H) {
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int head = warp; head < 2 * G; head += warps) {
    float* row = y + (size_t)n * ldy + (size_t)head * D;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss = fmaf(row[d], row[d], ss);
    ss = warp_sum(ss);
    const float inv = (head < G ? q_scale : 1.f) / sqrtf(ss + unit_eps);
    for (int d = lane; d < D; d += 32) row[d] *= inv;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    beta[(size_t)n * H + h] = sigmoid_f(to_f32(b[(size_t)n * ldb + h]));
    g[(size_t)n * H + h] = expf(-expf(a_log[h]) * softplus_f(to_f32(a[(size_t)n * lda + h]) + dt_bias[h]));
  }
}

// ------------------------------------------------------------------------------------------------ gated RMS norm
//
// One warp per (token, head): out = o / sqrt(mean(o^2) + eps) * w * f(gate) * out_scale, f = silu or (sigmoid != 0)
// the sigmoid alone; the output's rows have a pitch of their own. A norm over all heads together is the call with one
// head of H * V channels. w may be null: the division alone, every weight one.
__device__ __forceinline__ float4 norm_weight4(const float* __restrict__ w, int j) {
  return w != nullptr ? *reinterpret_cast<const float4*>(w + j) : make_float4(1.f, 1.f, 1.f, 1.f);
}

template <typename TG, typename TO>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                                     const TG* __restrict__ gate, long long ldg, TO* __restrict__ out, int N, int H, int V,
                                     int sigmoid, float out_scale, long long ldo) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)N * H) return;
  const int n = (int)(item / H), h = (int)(item % H);
  const float* row = o + (size_t)n * H * V + (size_t)h * V;
  float ss = 0.f;
  if (V % 4 == 0 && ldg % 4 == 0 && ldo % 4 == 0 && sizeof(TO) == sizeof(TG) && (uintptr_t)gate % (4 * sizeof(TG)) == 0 &&
      (uintptr_t)out % (4 * sizeof(TO)) == 0) {
    // four channels a lane: 16-byte reads of o, 8- or 16-byte reads of the gate and writes of the result. A row of at
    // most 1,024 channels stays in registers between the sum and the result, with its weights and gates asked for in
    // the same trip to memory (a step of few tokens is a handful of warps that only wait).
    if (V <= 1024) {
      float4 x[8], wv[8];
      float gv[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int j = lane * 4 + i * 128;
        if (j < V) {
          x[i] = *reinterpret_cast<const float4*>(row + j);
          wv[i] = norm_weight4(w, j);
          load4(gate + (size_t)n * ldg + (size_t)h * V + j, gv[i]);
          ss = fmaf(x[i].x, x[i].x, ss); ss = fmaf(x[i].y, x[i].y, ss); ss = fmaf(x[i].z, x[i].z, ss); ss = fmaf(x[i].w, x[i].w, ss);
        }
      }
      ss = warp_sum(ss);
      const float inv = out_scale / sqrtf(ss / (float)V + eps);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int j = lane * 4 + i * 128;
        if (j < V) {
#pragma unroll
          for (int e = 0; e < 4; ++e) gv[i][e] = sigmoid ? sigmoid_f(gv[i][e]) : gv[i][e] * sigmoid_f(gv[i][e]);
          const float r[4] = {x[i].x * inv * wv[i].x * gv[i][0], x[i].y * inv * wv[i].y * gv[i][1], x[i].z * inv * wv[i].z * gv[i][2],
                              x[i].w * inv * wv[i].w * gv[i][3]};
          TO* dst = out + (size_t)n * ldo + (size_t)h * V + j;
          if (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
          } else {
            const __nv_bfloat162 a = __floats2bfloat162_rn(r[0], r[1]), b = __floats2bfloat162_rn(r[2], r[3]);
            *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
          }
        }
      }
      return;
    }
    // four channels a lane: 16-byte reads of o, 8- or 16-byte reads of the gate and writes of the result
    for (int j = lane * 4; j < V; j += 128) {
      const float4 x = *reinterpret_cast<const float4*>(row + j);
      ss = fmaf(x.x, x.x, ss); ss = fmaf(x.y, x.y, ss); ss = fmaf(x.z, x.z, ss); ss = fmaf(x.w, x.w, ss);
    }
    ss = warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)V + eps);
    for (int j = lane * 4; j < V; j += 128) {
      const float4 x = *reinterpret_cast<const float4*>(row + j);
      const float4 wv = norm_weight4(w, j);
      float gv[4];
      load4(gate + (size_t)n * ldg + (size_t)h * V + j, gv);
#pragma unroll
      for (int e = 0; e < 4; ++e) gv[e] = sigmoid ? sigmoid_f(gv[e]) : gv[e] * sigmoid_f(gv[e]);
      const float r[4] = {x.x * inv * wv.x * gv[0], x.y * inv * wv.y * gv[1], x.z * inv * wv.z * gv[2], x.w * inv * wv.w * gv[3]};
      TO* dst = out + (size_t)n * ldo + (size_t)h * V + j;
      if (sizeof(TO) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
      } else {
        const __nv_bfloat162 a = __floats2bfloat162_rn(r[0], r[1]), b = __floats2bfloat162_rn(r[2], r[3]);
        *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
      }
    }
    return;
  }
  for (int j = lane; j < V; j += 32) ss = fmaf(row[j], row[j], ss);
  ss = warp_sum(ss);
  const float inv = out_scale / sqrtf(ss / (float)V + eps);
  for (int j = lane; j < V; j += 32) {
    const float gv = to_f32(gate[(size_t)n * ldg + (size_t)h * V + j]);
    out[(size_t)n * ldo + (size_t)h * V + j] = from_f32<TO>(row[j] * inv * (w != nullptr ? w[j] : 1.f) * (sigmoid ? sigmoid_f(gv) : gv * sigmoid_f(gv)));
  }
}

}  // namespace

AKAS_API int akas_decay_gates(const void* low, long long ld, const float* w, const float* bias, float* out, int N, int O,
                              int R, float tau, int dtype, cudaStream_t stream) {
  if (N <= 0 || O <= 0) return 0;
  const dim3 grid((N + kGateTokens - 1) / kGateTokens, min((O + 127) / 128, 64));
  const size_t smem = (size_t)kGateTokens * R * sizeof(float);
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  if (dtype == AKAS_F32)
    return launch_ordinary(decay_gates_kernel<float>, grid, dim3(128), smem, stream, (const float*)low, ld, w, bias, out, N, O, R, 1.f / tau);
  return launch_ordinary(decay_gates_kernel<bf16>, grid, dim3(128), smem, stream, (const bf16*)low, ld, w, bias, out, N, O, R, 1.f / tau);
}

AKAS_API int akas_gla_scan(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                           const float* alpha, float* state, long long slot_stride, const int* cu_seqlens, const int* slots,
                           float* out, int tokens, int requests, int H, int D, int V, float q_scale, int write, int dtype,
                           cudaStream_t stream) {
  if (dtype == AKAS_F32)
    return launch_scan<float, false>((const float*)q, ldq, (const float*)k, ldk, (const float*)v, ldv, alpha, nullptr, state,
                                     slot_stride, cu_seqlens, slots, out, tokens, requests, H, 1, D, V, q_scale, write, stream);
  return launch_scan<bf16, false>((const bf16*)q, ldq, (const bf16*)k, ldk, (const bf16*)v, ldv, alpha, nullptr, state,
                                  slot_stride, cu_seqlens, slots, out, tokens, requests, H, 1, D, V, q_scale, write, stream);
}

// The recurrence with one constant decay per head (decay [H] float32); act != 0: silu on q, k and v on their way in.
AKAS_API int akas_decay_scan(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                             const float* decay, float* state, long long slot_stride, const int* cu_seqlens, const int* slots,
                             float* out, int tokens, int requests, int H, int D, int V, float q_scale, int act, int write,
                             int dtype, cudaStream_t stream) {
  if (dtype == AKAS_F32)
    return launch_scan<float, false, true>((const float*)q, ldq, (const float*)k, ldk, (const float*)v, ldv, decay, nullptr,
                                           state, slot_stride, cu_seqlens, slots, out, tokens, requests, H, 1, D, V, q_scale,
                                           write, stream, act);
  return launch_scan<bf16, false, true>((const bf16*)q, ldq, (const bf16*)k, ldk, (const bf16*)v, ldv, decay, nullptr, state,
                                        slot_stride, cu_seqlens, slots, out, tokens, requests, H, 1, D, V, q_scale, write,
                                        stream, act);
}

// Floats of scratch that akas_decay_scan_chunked needs; 0 where it does not take the sizes (the token-by-token kernel does).
AKAS_API long long akas_decay_chunk_scratch(int tokens, int requests, int H, int D, int V) {
  if (D > kChunkMaxD || tokens <= 0 || requests <= 0) return 0;
  return (long long)((tokens + kChunk - 1) / kChunk + requests) * H * D * V;
}

// The same recurrence as akas_decay_scan, in chunks (see above): for steps that bring many tokens a request.
AKAS_API int akas_decay_scan_chunked(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                                     const float* decay, float* state, long long slot_stride, const int* cu_seqlens,
                                     const int* slots, float* out, float* scratch, int tokens, int requests, int H, int D, int V,
                                     float q_scale, int act, int write, int dtype, cudaStream_t stream) {
  if (tokens <= 0 || requests <= 0 || H <= 0) return 0;
  if (D > kChunkMaxD || scratch == nullptr) return (int)cudaErrorInvalidValue;
  if (dtype == AKAS_F32)
    return launch_chunks((const float*)q, ldq, (const float*)k, ldk, (const float*)v, ldv, decay, state, slot_stride, cu_seqlens,
                         slots, out, scratch, tokens, requests, H, D, V, q_scale, act, write, stream);
  return launch_chunks((const bf16*)q, ldq, (const bf16*)k, ldk, (const bf16*)v, ldv, decay, state, slot_stride, cu_seqlens, slots,
                       out, scratch, tokens, requests, H, D, V, q_scale, act, write, stream);
}

AKAS_API int akas_delta_scan(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv,
                             const float* beta, const float* g, float* state, long long slot_stride, const int* cu_seqlens,
                             const int* slots, float* out, int tokens, int requests, int H, int G, int D, int V, int write,
                             cudaStream_t stream) {
  if (G <= 0 || H % G) return (int)cudaErrorInvalidValue;
  return launch_scan<float, true>(q, ldq, k, ldk, v, ldv, g, beta, state, slot_stride, cu_seqlens, slots, out, tokens,
                                  requests, H, H / G, D, V, 1.f, write, stream);
}

AKAS_API int akas_causal_conv_silu(const void* x, long long ldx, const float* taps, float* state, long long slot_stride,
                                   const int* cu_seqlens, const int* seq_of_token, const int* slots, float* y, int N,
                                   int requests, int C, int L, int write, int dtype, cudaStream_t stream) {
  if (N <= 0 || C <= 0) return 0;
  const dim3 grid(N, min((C + 255) / 256, 32));
  const float* old = state;
  const size_t elem = dtype == AKAS_F32 ? 4 : 2;
  const bool four = C % 4 == 0 && ldx % 4 == 0 && slot_stride % 4 == 0 && (uintptr_t)x % (4 * elem) == 0 &&
                    (uintptr_t)state % 16 == 0 && (uintptr_t)y % 16 == 0;
  const dim3 grid4(N, min((C / 4 + 127) / 128, 32));
  int err = four ? (dtype == AKAS_F32
      ? launch_ordinary(causal_conv_silu4_kernel<float>, grid4, dim3(128), 0, stream, (const float*)x, ldx, taps, old, slot_stride,
                        cu_seqlens, seq_of_token, slots, y, C, L)
      : launch_ordinary(causal_conv_silu4_kernel<bf16>, grid4, dim3(128), 0, stream, (const bf16*)x, ldx, taps, old, slot_stride,
                        cu_seqlens, seq_of_token, slots, y, C, L))
      : dtype == AKAS_F32
      ? launch_ordinary(causal_conv_silu_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, ldx, taps, old, slot_stride,
                       cu_seqlens, seq_of_token, slots, y, C, L)
      : launch_ordinary(causal_conv_silu_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, ldx, taps, old, slot_stride,
                       cu_seqlens, seq_of_token, slots, y, C, L);
  if (err || !write || requests <= 0) return err;
  const dim3 sgrid(requests, min((C + 255) / 256, 32));
  if (dtype == AKAS_F32)
    return launch_ordinary(causal_conv_state_kernel<float>, sgrid, dim3(256), 0, stream, (const float*)x, ldx, state, slot_stride,
                          cu_seqlens, slots, C, L);
  return launch_ordinary(causal_conv_state_kernel<bf16>, sgrid, dim3(256), 0, stream, (const bf16*)x, ldx, state, slot_stride,
                        cu_seqlens, slots, C, L);
}

AKAS_API int akas_delta_prep(float* y, long long ldy, int G, int D, float q_scale, float unit_eps, const void* b,
                             long long ldb, const void* a, long long lda, const float* a_log, const float* dt_bias,
                             float* beta, float* g, int N, int H, int dtype, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (dtype == AKAS_F32)
    return launch_ordinary(delta_prep_kernel<float>, dim3(N), dim3(128), 0, stream, y, ldy, G, D, q_scale, unit_eps,
                          (const float*)b, ldb, (const float*)a, lda, a_log, dt_bias, beta, g, H);
  return launch_ordinary(delta_prep_kernel<bf16>, dim3(N), dim3(128), 0, stream, y, ldy, G, D, q_scale, unit_eps, (const bf16*)b,
                        ldb, (const bf16*)a, lda, a_log, dt_bias, beta, g, H);
}

AKAS_API int akas_gated_rmsnorm(const float* o, const float* w, float eps, const void* gate, long long ldg, void* out, int N,
                                int H, int V, int gate_dtype, int out_dtype, int sigmoid, float out_scale, long long ldo,
                                cudaStream_t stream) {
  if (N <= 0 || H <= 0) return 0;
  const long long items = (long long)N * H;
  const int blocks = (int)((items + 7) / 8);
#define AKAS_GN(TG, TO) \
  return launch_ordinary(gated_rmsnorm_kernel<TG, TO>, dim3(blocks), dim3(256), 0, stream, o, w, eps, (const TG*)gate, ldg, (TO*)out, N, H, V, \
                         sigmoid, out_scale, ldo)
  if (gate_dtype == AKAS_F32 && out_dtype == AKAS_F32) AKAS_GN(float, float);
  if (gate_dtype == AKAS_F32) AKAS_GN(float, bf16);
  if (out_dtype == AKAS_F32) AKAS_GN(bf16, float);
  AKAS_GN(bf16, bf16);
#undef AKAS_GN
}
