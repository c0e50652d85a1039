// A routed feed-forward (mixture of experts): the router, and the experts for steps of few tokens and for float32.
//
// Router, per token, all in float32: logits z = W_r h over the R router outputs (one chain of sums per (token,
// output) whose order depends on the width only), s = softmax(z); the choice score is s + correction; the outputs
// form `groups` equal groups of neighbours, a group's score is its largest choice score, only outputs of the `keep`
// best groups can be chosen; the `top` largest choice scores among those are chosen (ties: the lower index); the
// weights are the chosen outputs' s over their sum (+ 1e-20). Router outputs from `experts` on are identity experts:
// they have no matrices and return their input. Options: `sigmoid`, s = 1 / (1 + exp(-z)) per output instead of the
// softmax; no correction (a null pointer); `renorm` 0, the weights are the chosen s as they are; `extra` more rows of
// W_r behind the R that compete, whose sigmoids are returned beside the choice (gates that read the router's input).
//
// Experts, token by token (moe_gate_up, moe_down): act[pair] = silu(W_gate h) * (W_up h) for every (token, chosen
// real expert) pair, then out[n] = sum over the token's chosen outputs of weight * (W_down act, or h for an identity
// expert), added in the order of the choice. Every output is one warp's sum over the inner size in a fixed order, so
// a token's result does not depend on what else the step holds. Weights of all experts are stacked: gate and up as
// [experts, 2 F, C] (gate rows first), down as [experts, C, F]. Where the weight multiplies the expert's INPUT
// (out[n] = sum expert(w h)), moe_gate_up gets the weights and scales both of its float32 sums (W (w h) = w (W h))
// before the activation, and moe_down gets none. moe_down can also add a dense result of every token (a shared
// expert's), times a gate per token.
#include "common.cuh"

using namespace akas;

namespace {

constexpr int kRouteTokens = 8;   // tokens of a router block = its warps
constexpr int kRouteChunk = 2048; // channels of h staged at a time (64 KB of float32 rows for the block's tokens)
constexpr int kRouteOutputs = 4;  // router outputs whose rows a warp reads at the same time

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(kRouteTokens * 32)
moe_route_kernel(const T* __restrict__ h, long long ldh, const float* __restrict__ w, const float* __restrict__ correction,
                 int* __restrict__ chosen, float* __restrict__ weights, int N, int C, int RC, int groups, int keep, int top,
                 int sigmoid, int renorm, int extra, float* __restrict__ extras) {
  extern __shared__ __align__(16) float smem[];
  int R = RC + extra;                              // rows of the matrix: the RC outputs that compete, then the extra ones
  float* rows = smem;                              // [kRouteTokens][kRouteChunk]
  float* z = rows + kRouteTokens * kRouteChunk;    // [kRouteTokens][R] logits, then scores
  float* pick = z + kRouteTokens * R;              // [kRouteTokens][R] choice scores
  float* gbest = pick + kRouteTokens * R;          // [kRouteTokens][groups]
  float* part = gbest + kRouteTokens * groups;     // [warps][kRouteOutputs][kRouteTokens] the warps' partial sums
  const int n0 = blockIdx.x * kRouteTokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kRouteTokens * R; i += blockDim.x) z[i] = 0.f;
  if (gridDim.x <= 16) {
    // a step of few tokens is a few blocks that wait for memory: the whole matrix is asked into the L2 at once, so that
    // the reads below, one group of outputs after another, do not each wait for DRAM
    const char* bytes = reinterpret_cast<const char*>(w);
    const size_t total = (size_t)R * C * sizeof(float);
    for (size_t off = (size_t)threadIdx.x * 128; off < total; off += (size_t)blockDim.x * 128)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(bytes + off));
  }
  for (int c0 = 0; c0 < C; c0 += kRouteChunk) {
    const int width = min(kRouteChunk, C - c0);
    __syncthreads();
    if (C % 8 == 0 && ldh % 8 == 0 && ((uintptr_t)h % 16) == 0) {  // eight channels a load
      const int per_row = width / 8;
      for (int i = threadIdx.x; i < kRouteTokens * per_row; i += blockDim.x) {
        const int t = i / per_row, c = (i % per_row) * 8;
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (n0 + t < N) load8(h + (size_t)(n0 + t) * ldh + c0 + c, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) rows[t * kRouteChunk + c + j] = v[j];
      }
    } else {
      for (int i = threadIdx.x; i < kRouteTokens * width; i += blockDim.x) {
        const int t = i / width, c = i % width;
        rows[t * kRouteChunk + c] = n0 + t < N ? to_f32(h[(size_t)(n0 + t) * ldh + c0 + c]) : 0.f;
      }
    }
    __syncthreads();
    // Warp w takes the w-th eighth of the staged channels for EVERY router output, so that all of a lane's loads of
    // the matrix are in flight at once (one trip to memory instead of one per output); the warps' partial sums meet
    // in shared memory and are added in the order of the warps: the order of a (token, output) sum depends on the
    // width only.
    const bool vec = C % 4 == 0 && ((uintptr_t)w % 16) == 0;
    const int slice = ((width + kRouteTokens - 1) / kRouteTokens + 3) / 4 * 4;
    const int s0 = min(width, warp * slice), s1 = min(width, s0 + slice);
    for (int e0 = 0; e0 < R; e0 += kRouteOutputs) {
      float acc[kRouteOutputs][kRouteTokens];
#pragma unroll
      for (int o = 0; o < kRouteOutputs; ++o)
#pragma unroll
        for (int t = 0; t < kRouteTokens; ++t) acc[o][t] = 0.f;
      if (vec) {
        for (int c = s0 + lane * 4; c < s1; c += 128) {
          float4 wv[kRouteOutputs];
#pragma unroll
          for (int o = 0; o < kRouteOutputs; ++o)
            wv[o] = e0 + o < R ? *reinterpret_cast<const float4*>(w + (size_t)(e0 + o) * C + c0 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int t = 0; t < kRouteTokens; ++t) {
            const float4 hv = *reinterpret_cast<const float4*>(rows + t * kRouteChunk + c);
#pragma unroll
            for (int o = 0; o < kRouteOutputs; ++o) {
              acc[o][t] = fmaf(hv.x, wv[o].x, acc[o][t]); acc[o][t] = fmaf(hv.y, wv[o].y, acc[o][t]);
              acc[o][t] = fmaf(hv.z, wv[o].z, acc[o][t]); acc[o][t] = fmaf(hv.w, wv[o].w, acc[o][t]);
            }
          }
        }
      } else {
        for (int c = s0 + lane; c < s1; c += 32) {
#pragma unroll
          for (int o = 0; o < kRouteOutputs; ++o) {
            const float wv = e0 + o < R ? w[(size_t)(e0 + o) * C + c0 + c] : 0.f;
#pragma unroll
            for (int t = 0; t < kRouteTokens; ++t) acc[o][t] = fmaf(rows[t * kRouteChunk + c], wv, acc[o][t]);
          }
        }
      }
      // the lanes' 32 sums each (4 outputs x 8 tokens) are added across the warp so that lane l ends with the total of
      // sum number l: every round a lane hands one half of what it still holds to its partner and keeps the other
      // (31 shuffles instead of 32 x 5); the order of the additions is the same for every token and batch
      static_assert(kRouteOutputs * kRouteTokens == 32, "one sum per lane");
      float* v = &acc[0][0];
#pragma unroll
      for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
          const float send = upper ? v[i] : v[i + n / 2];
          const float keep = upper ? v[i + n / 2] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
      }
      part[warp * 32 + lane] = v[0];  // [warp][output][token]
      __syncthreads();
      for (int i = threadIdx.x; i < kRouteOutputs * kRouteTokens; i += blockDim.x) {
        const int o = i / kRouteTokens, t = i % kRouteTokens;
        if (e0 + o < R) {
          float sum = z[t * R + e0 + o];
          for (int ww = 0; ww < kRouteTokens; ++ww) sum += part[(ww * kRouteOutputs + o) * kRouteTokens + t];
          z[t * R + e0 + o] = sum;
        }
      }
      __syncthreads();
    }
  }
  __syncthreads();
  // warp t chooses for token n0 + t
  const int n = n0 + warp;
  if (n >= N) return;
  float* zt = z + warp * R;
  float* pt = pick + warp * R;
  float* gt = gbest + warp * groups;
  for (int j = lane; j < extra; j += 32) extras[(size_t)n * extra + j] = 1.f / (1.f + expf(-zt[RC + j]));
  R = RC;  // from here on: the outputs that compete
  if (sigmoid) {
    // Without a correction the choice goes by the logits themselves: the same order as their sigmoids', and two large
    // logits whose sigmoids both round to one still compare.
    for (int e = lane; e < R; e += 32) {
      const float logit = zt[e];
      zt[e] = 1.f / (1.f + expf(-logit));
      pt[e] = correction != nullptr ? zt[e] + correction[e] : logit;
    }
  } else {
    float top_z = -INFINITY;
    for (int e = lane; e < R; e += 32) top_z = fmaxf(top_z, zt[e]);
    top_z = warp_max(top_z);
    float sum = 0.f;
    for (int e = lane; e < R; e += 32) {
      const float p = expf(zt[e] - top_z);
      zt[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < R; e += 32) {
      zt[e] *= inv;
      pt[e] = zt[e] + (correction != nullptr ? correction[e] : 0.f);
    }
  }
  __syncwarp();
  const int size = R / groups;
  if (groups > 1 && keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * size; e < (g + 1) * size; ++e) best = fmaxf(best, pt[e]);
      gt[g] = best;
    }
    __syncwarp();
    // a group stays iff fewer than `keep` groups beat it (a tie goes to the lower index)
    for (int g = lane; g < groups; g += 32) {
      int ahead = 0;
      for (int o = 0; o < groups; ++o) ahead += gt[o] > gt[g] || (gt[o] == gt[g] && o < g);
      if (ahead >= keep)
        for (int e = g * size; e < (g + 1) * size; ++e) pt[e] = -INFINITY;
    }
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < R; e += 32)
      if (pt[e] > best) { best = pt[e]; at = e; }  // ascending e: the first of equal scores stays
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;  // fewer choosable outputs than `top`: cannot happen for a valid configuration
    if (lane == 0) {
      chosen[(size_t)n * top + k] = at;
      weights[(size_t)n * top + k] = zt[at];
      pt[at] = -INFINITY;
    }
    total += zt[at];
    __syncwarp();
  }
  if (lane == 0 && renorm) {
    const float norm = 1.f / (total + 1e-20f);
    for (int k = 0; k < top; ++k) weights[(size_t)n * top + k] *= norm;
  }
}

// One warp per (pair, hidden channel f): both dots over C, act = silu(gate) * up. Pairs of identity experts do nothing.
// in_weights (or null): the pair's weight multiplies both sums before the activation.
template <typename T>
__global__ void __launch_bounds__(256)
moe_gate_up_kernel(const T* __restrict__ h, long long ldh, const T* __restrict__ w_gate_up, const int* __restrict__ chosen,
                   T* __restrict__ act, int pairs, int top, int C, int F, int experts, const float* __restrict__ in_weights) {
  const int pair = blockIdx.x;
  const int e = chosen[pair];
  if (e >= experts || e < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const T* x = h + (size_t)(pair / top) * ldh;
  const T* wg = w_gate_up + (size_t)e * 2 * F * C;
  const float scale = in_weights != nullptr ? in_weights[pair] : 1.f;
  constexpr int N = Vec<T>::N;
  const bool vec = C % N == 0 && ldh % N == 0 && ((uintptr_t)h % 16) == 0 && ((uintptr_t)w_gate_up % 16) == 0;
  for (int f = blockIdx.y * warps + warp; f < F; f += gridDim.y * warps) {
    const T* g_row = wg + (size_t)f * C;
    const T* u_row = wg + (size_t)(F + f) * C;
    float ag = 0.f, au = 0.f;
    if (vec) {
      for (int c = lane * N; c < C; c += 32 * N) {
        float xv[N], gv[N], uv[N];
        load_vec(x + c, xv);
        load_vec(g_row + c, gv);
        load_vec(u_row + c, uv);
#pragma unroll
        for (int i = 0; i < N; ++i) { ag = fmaf(xv[i], gv[i], ag); au = fmaf(xv[i], uv[i], au); }
      }
    } else {
      for (int c = lane; c < C; c += 32) {
        const float xv = to_f32(x[c]);
        ag = fmaf(xv, to_f32(g_row[c]), ag);
        au = fmaf(xv, to_f32(u_row[c]), au);
      }
    }
    ag = warp_sum(ag) * scale;
    au = warp_sum(au) * scale;
    if (lane == 0) act[(size_t)pair * F + f] = from_f32<T>(silu_f(ag) * au);
  }
}

// One warp per (token, output channel c): the weighted sum over the token's chosen outputs. With `x` the sum does not
// go to `out` but into the residual stream: x += mult * (ls_a * a + ls_b * sum), the update of a block whose mixer's
// result a and feed-forward meet the stream together (a null scale is all ones). Null weights: every weight is one.
// shared (or null): float32 [N, C] added to the sum, times shared_gate[n * ldsg] where that is given.
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ h, long long ldh, const T* __restrict__ w_down, const int* __restrict__ chosen,
                const float* __restrict__ weights, const T* __restrict__ act, float* __restrict__ out, int top, int C, int F,
                int experts, float* __restrict__ x, const float* __restrict__ a_res, const float* __restrict__ ls_a,
                const float* __restrict__ ls_b, float mult, const float* __restrict__ shared,
                const float* __restrict__ shared_gate, long long ldsg) {
  const int n = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  constexpr int N = Vec<T>::N;
  const bool vec = F % N == 0 && ((uintptr_t)act % 16) == 0 && ((uintptr_t)w_down % 16) == 0;
  for (int c = blockIdx.y * warps + warp; c < C; c += gridDim.y * warps) {
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = chosen[(size_t)n * top + k];
      const float g = weights != nullptr ? weights[(size_t)n * top + k] : 1.f;
      if (e >= experts) {
        total = fmaf(g, to_f32(h[(size_t)n * ldh + c]), total);
        continue;
      }
      const T* row = w_down + ((size_t)e * C + c) * F;
      const T* a = act + ((size_t)n * top + k) * F;
      float acc = 0.f;
      if (vec) {
        for (int f = lane * N; f < F; f += 32 * N) {
          float av[N], wv[N];
          load_vec(a + f, av);
          load_vec(row + f, wv);
#pragma unroll
          for (int i = 0; i < N; ++i) acc = fmaf(av[i], wv[i], acc);
        }
      } else {
        for (int f = lane; f < F; f += 32) acc = fmaf(to_f32(a[f]), to_f32(row[f]), acc);
      }
      total = fmaf(g, warp_sum(acc), total);
    }
    if (lane == 0) {
      if (shared != nullptr) total = fmaf(shared_gate != nullptr ? shared_gate[(size_t)n * ldsg] : 1.f, shared[(size_t)n * C + c], total);
      if (x != nullptr) {
        const size_t at = (size_t)n * C + c;
        x[at] = fmaf(mult, fmaf(ls_b ? ls_b[c] : 1.f, total, (ls_a ? ls_a[c] : 1.f) * a_res[at]), x[at]);
      } else {
        out[(size_t)n * C + c] = total;
      }
    }
  }
}

}  // namespace

// R: the outputs that compete; the matrix has R + extra rows.
AKAS_API int akas_moe_route(const void* h, long long ldh, const float* w, const float* correction, int* chosen, float* weights,
                            int N, int C, int R, int groups, int keep, int top, int dtype, int sigmoid, int renorm, int extra,
                            float* extras, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (R <= 0 || groups <= 0 || R % groups || keep <= 0 || keep > groups || top <= 0 || top > keep * (R / groups) || extra < 0 ||
      (extra > 0 && extras == nullptr))
    return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * ((size_t)kRouteTokens * kRouteChunk + 2 * (size_t)kRouteTokens * (R + extra) + (size_t)kRouteTokens * groups +
                                       (size_t)kRouteTokens * kRouteOutputs * kRouteTokens);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const dim3 grid((N + kRouteTokens - 1) / kRouteTokens);
  static size_t allowed[64][2] = {};
  int device = 0;
  cudaGetDevice(&device);
  const int which = dtype == AKAS_F32 ? 0 : 1;
  if (smem > 48 * 1024 && device < 64 && allowed[device][which] < smem) {
    const cudaError_t e = which == 0
        ? cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
        : cudaFuncSetAttribute(moe_route_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed[device][which] = smem;
  }
  if (dtype == AKAS_F32)
    return launch_ordinary(moe_route_kernel<float>, grid, dim3(kRouteTokens * 32), smem, stream, (const float*)h, ldh, w,
                           correction, chosen, weights, N, C, R, groups, keep, top, sigmoid, renorm, extra, extras);
  return launch_ordinary(moe_route_kernel<bf16>, grid, dim3(kRouteTokens * 32), smem, stream, (const bf16*)h, ldh, w, correction,
                         chosen, weights, N, C, R, groups, keep, top, sigmoid, renorm, extra, extras);
}

AKAS_API int akas_moe_gate_up(const void* h, long long ldh, const void* w_gate_up, const int* chosen, void* act, int N,
                              int top, int C, int F, int experts, int dtype, const float* in_weights, cudaStream_t stream) {
  if (N <= 0 || top <= 0 || experts <= 0) return 0;
  const int pairs = N * top;
  // warps enough to fill the GPU when the pairs are few (a row of F per warp), fewer and longer-lived when they are many
  const dim3 grid(pairs, max(1, min((F + 7) / 8, pairs >= 4096 ? 2 : pairs >= 256 ? 16 : 256)));
  if (dtype == AKAS_F32)
    return launch_ordinary(moe_gate_up_kernel<float>, grid, dim3(256), 0, stream, (const float*)h, ldh, (const float*)w_gate_up,
                           chosen, (float*)act, pairs, top, C, F, experts, in_weights);
  return launch_ordinary(moe_gate_up_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)h, ldh, (const bf16*)w_gate_up,
                         chosen, (bf16*)act, pairs, top, C, F, experts, in_weights);
}

AKAS_API int akas_moe_down(const void* h, long long ldh, const void* w_down, const int* chosen, const float* weights,
                           const void* act, float* out, int N, int top, int C, int F, int experts, int dtype, float* x,
                           const float* a_res, const float* ls_a, const float* ls_b, float mult, const float* shared,
                           const float* shared_gate, long long ldsg, cudaStream_t stream) {
  if (N <= 0) return 0;
  const dim3 grid(N, max(1, min((C + 7) / 8, N >= 2048 ? 2 : N >= 64 ? 32 : 256)));
  if (dtype == AKAS_F32)
    return launch_ordinary(moe_down_kernel<float>, grid, dim3(256), 0, stream, (const float*)h, ldh, (const float*)w_down, chosen,
                           weights, (const float*)act, out, top, C, F, experts, x, a_res, ls_a, ls_b, mult, shared, shared_gate, ldsg);
  return launch_ordinary(moe_down_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)h, ldh, (const bf16*)w_down, chosen,
                         weights, (const bf16*)act, out, top, C, F, experts, x, a_res, ls_a, ls_b, mult, shared, shared_gate, ldsg);
}
