// Embedding gather, RMSNorm (optionally of gathered rows), SwiGLU and the reset of state rows.
//
// The residual stream is float32 in both precisions: the embedding writes float32, RMSNorm reads
// it and writes the compute dtype that the next matrix product takes. All sums are float32.
#include "common.cuh"

using namespace akas;

// out[n, :] = float(table[token[n], :])
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                 float* __restrict__ out, int C) {
  chain_release();
  chain_wait();
  const int n = blockIdx.x;
  const T* row = table + (size_t)tokens[n] * C;
  float* dst = out + (size_t)n * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) dst[c] = to_f32(row[c]);
}

AKAS_API int akas_embedding(const int* tokens, const void* table, float* out, int N, int C, int dtype,
                            cudaStream_t stream) {
  if (N <= 0) return 0;
  const int threads = C >= 1024 ? 256 : 128;
  if (dtype == AKAS_F32)
    return launch_chained(embedding_kernel<float>, dim3(N), dim3(threads), 0, stream, tokens, (const float*)table, out, C);
  return launch_chained(embedding_kernel<bf16>, dim3(N), dim3(threads), 0, stream, tokens, (const bf16*)table, out, C);
}

// y[i, :] = x[row(i), :] * rsqrt(mean(x^2) + eps) * (w or 1 + w); row(i) = rows[i] if rows else i.
// One block per row; the row is read twice (the second read hits L1/L2).
template <typename TI, typename TO>
__global__ void rmsnorm_kernel(const TI* __restrict__ x, const float* __restrict__ w, TO* __restrict__ y,
                               const int* __restrict__ rows, int C, float eps, int zero_centered) {
  chain_release();  // a kernel after this one that was launched as its programmatic dependent may set itself up meanwhile
  __shared__ float scratch[32];
  const int i = blockIdx.x;
  const TI* src = x + (size_t)(rows ? rows[i] : i) * C;
  float ss = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = to_f32(src[c]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)C + eps);
  TO* dst = y + (size_t)i * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float g = zero_centered ? 1.f + w[c] : w[c];
    dst[c] = from_f32<TO>(to_f32(src[c]) * inv * g);
  }
}

// The same for float32 rows whose width is a multiple of 8 and at most 8192: the row is read once, with
// 16-byte loads, and stays in registers between the sum of squares and the scaling.
template <typename TO, int PER_THREAD>  // PER_THREAD groups of 8 elements per thread, 256 threads
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ y,
                    const int* __restrict__ rows, int C, float eps, int zero_centered) {
  chain_release();  // a kernel after this one that was launched as its programmatic dependent may set itself up meanwhile
  __shared__ float scratch[32];
  const int i = blockIdx.x;
  // the weights and (what the host wrote for this step) the row's number do not wait for the kernel ahead
  const size_t row = rows ? rows[i] : i;
  float v[PER_THREAD][8], g[PER_THREAD][8];
#pragma unroll
  for (int p = 0; p < PER_THREAD; ++p) {
    const int c = (p * 256 + threadIdx.x) * 8;
    if (c < C) {
      const float4 wa = *reinterpret_cast<const float4*>(w + c);
      const float4 wb = *reinterpret_cast<const float4*>(w + c + 4);
      g[p][0] = wa.x; g[p][1] = wa.y; g[p][2] = wa.z; g[p][3] = wa.w;
      g[p][4] = wb.x; g[p][5] = wb.y; g[p][6] = wb.z; g[p][7] = wb.w;
    }
  }
  chain_wait();
  const float* src = x + row * C;
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < PER_THREAD; ++p) {
    const int c = (p * 256 + threadIdx.x) * 8;
    if (c < C) {
      const float4 a = *reinterpret_cast<const float4*>(src + c);
      const float4 b = *reinterpret_cast<const float4*>(src + c + 4);
      v[p][0] = a.x; v[p][1] = a.y; v[p][2] = a.z; v[p][3] = a.w;
      v[p][4] = b.x; v[p][5] = b.y; v[p][6] = b.z; v[p][7] = b.w;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(v[p][e], v[p][e], ss);
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)C + eps);
  TO* dst = y + (size_t)i * C;
#pragma unroll
  for (int p = 0; p < PER_THREAD; ++p) {
    const int c = (p * 256 + threadIdx.x) * 8;
    if (c < C) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[p][e] * inv * (zero_centered ? 1.f + g[p][e] : g[p][e]);
      store8(dst + c, o);
    }
  }
}

AKAS_API int akas_rmsnorm(const void* x, const float* w, void* y, const int* rows, int M, int C, float eps,
                          int zero_centered, int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (in_dtype == AKAS_F32 && C % 8 == 0 && C >= 1024 && C <= 8192 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
#define AKAS_ROWS(TO, P) \
  return launch_chained(rmsnorm_rows_kernel<TO, P>, dim3(M), dim3(256), 0, stream, (const float*)x, w, (TO*)y, rows, C, eps, zero_centered)
    if (out_dtype == AKAS_F32) { if (C <= 2048) AKAS_ROWS(float, 1); else if (C <= 4096) AKAS_ROWS(float, 2); else AKAS_ROWS(float, 4); }
    else { if (C <= 2048) AKAS_ROWS(bf16, 1); else if (C <= 4096) AKAS_ROWS(bf16, 2); else AKAS_ROWS(bf16, 4); }
#undef AKAS_ROWS
  }
  const int threads = C >= 2048 ? 512 : C >= 512 ? 256 : 128;
#define AKAS_NORM(TI, TO) \
  rmsnorm_kernel<TI, TO><<<M, threads, 0, stream>>>((const TI*)x, w, (TO*)y, rows, C, eps, zero_centered)
  if (in_dtype == AKAS_F32 && out_dtype == AKAS_F32) AKAS_NORM(float, float);
  else if (in_dtype == AKAS_F32) AKAS_NORM(float, bf16);
  else if (out_dtype == AKAS_F32) AKAS_NORM(bf16, float);
  else AKAS_NORM(bf16, bf16);
#undef AKAS_NORM
  return launch_status();
}

// out[n, f] = silu(gu[n, f]) * gu[n, F + f], silu(g) = g / (1 + exp(-g)), in float32
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t n = i / F;
  const int f = (int)(i - n * F);
  const float g = to_f32(gu[n * 2 * F + f]);
  const float u = to_f32(gu[n * 2 * F + F + f]);
  out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
}

// Eight (bfloat16) or four (float32) neighbours per thread with 16-byte loads, for F a multiple of that.
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t groups) {
  constexpr int V = Vec<T>::N;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= groups) return;
  const int per_row = F / V;
  const size_t n = i / per_row;
  const int f = (int)(i - n * per_row) * V;
  float g[V], u[V], o[V];
  load_vec(gu + n * 2 * F + f, g);
  load_vec(gu + n * 2 * F + F + f, u);
#pragma unroll
  for (int e = 0; e < V; ++e) o[e] = g[e] / (1.f + expf(-g[e])) * u[e];
  store_vec(out + n * F + f, o);
}

AKAS_API int akas_swiglu(const void* gu, void* out, int N, int F, int dtype, cudaStream_t stream) {
  const size_t total = (size_t)N * F;
  if (total == 0) return 0;
  const int threads = 256;
  const int v = dtype == AKAS_F32 ? 4 : 8;
  if (F % v == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0) {
    const size_t groups = total / v;
    const unsigned blocks = (unsigned)((groups + threads - 1) / threads);
    if (dtype == AKAS_F32)
      swiglu_vec_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, F, groups);
    else
      swiglu_vec_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, F, groups);
    return launch_status();
  }
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  if (dtype == AKAS_F32)
    swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, F, total);
  else
    swiglu_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, F, total);
  return launch_status();
}

// state[g, slot, :] = 0 for one slot of a [groups, slots, row] float32 tensor (groups: the layers whose states
// of one shape share an allocation)
__global__ void zero_row_kernel(float* __restrict__ state, size_t row, size_t group_stride, int slot) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < row) state[blockIdx.y * group_stride + (size_t)slot * row + i] = 0.f;
}

AKAS_API int akas_zero_row(float* state, long long row_elems, int slot, int groups, long long group_stride,
                           cudaStream_t stream) {
  if (row_elems <= 0 || groups <= 0) return 0;
  if (groups > 65535) return (int)cudaErrorInvalidValue;
  const int threads = 256;
  zero_row_kernel<<<dim3((unsigned)((row_elems + threads - 1) / threads), groups), threads, 0, stream>>>(
      state, (size_t)row_elems, (size_t)group_stride, slot);
  return launch_status();
}

// token_ids[i] = previous[source[i]] where source[i] >= 0: tokens that the step before sampled and that never
// went to the host.
__global__ void take_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ source,
                                   const int* __restrict__ previous, int previous_count, int N) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const int s = source[i];
  if (s >= 0 && s < previous_count) token_ids[i] = previous[s];
}

AKAS_API int akas_take_tokens(int* token_ids, const int* source, const int* previous, int previous_count, int N,
                              cudaStream_t stream) {
  if (N <= 0) return 0;
  take_tokens_kernel<<<(N + 255) / 256, 256, 0, stream>>>(token_ids, source, previous, previous_count, N);
  return launch_status();
}

// out[n, c] = x[n, c] + bias[c], x float32, out float32 or bfloat16 (out may be x): the bias of a product whose
// result was left in float32, added before the one rounding.
template <typename TO>
__global__ void add_bias_kernel(const float* __restrict__ x, const float* __restrict__ bias, TO* __restrict__ out, int C,
                                size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = from_f32<TO>(x[i] + bias[i % C]);
}

AKAS_API int akas_add_bias(const float* x, const float* bias, void* out, int N, int C, int out_dtype, cudaStream_t stream) {
  const size_t total = (size_t)N * C;
  if (total == 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dtype == AKAS_F32) add_bias_kernel<float><<<blocks, 256, 0, stream>>>(x, bias, (float*)out, C, total);
  else add_bias_kernel<bf16><<<blocks, 256, 0, stream>>>(x, bias, (bf16*)out, C, total);
  return launch_status();
}

// In place on float32: x = x * scale, then x = cap * tanh(x / cap) where cap > 0 (an embedding multiplier, a
// logit scale, a logit softcap).
__global__ void scale_cap_kernel(float* __restrict__ x, float scale, float cap, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = x[i] * scale;
  if (cap > 0.f) v = cap * tanhf(v / cap);
  x[i] = v;
}

AKAS_API int akas_scale_cap(float* x, float scale, float cap, long long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  scale_cap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, scale, cap, (size_t)total);
  return launch_status();
}

// h[n, :] += float(table[index[n], :]) in place on float32 h: learned absolute positions on top of the embedding.
template <typename T>
__global__ void add_rows_kernel(float* __restrict__ h, const T* __restrict__ table, const int* __restrict__ index, int C) {
  const int n = blockIdx.x;
  const T* row = table + (size_t)index[n] * C;
  float* dst = h + (size_t)n * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) dst[c] += to_f32(row[c]);
}

AKAS_API int akas_add_rows(float* h, const void* table, const int* index, int N, int C, int dtype, cudaStream_t stream) {
  if (N <= 0) return 0;
  const int threads = C >= 1024 ? 256 : 128;
  if (dtype == AKAS_F32) return launch_ordinary(add_rows_kernel<float>, dim3(N), dim3(threads), 0, stream, h, (const float*)table, index, C);
  return launch_ordinary(add_rows_kernel<bf16>, dim3(N), dim3(threads), 0, stream, h, (const bf16*)table, index, C);
}

// x[n, c] += mult * (ls_a[c] * a[n, c] + ls_b[c] * b[n, c]) in place on the float32 residual stream: the update of a
// block whose sublayers all read one norm of x and whose results meet, each through a learned scale per channel,
// in one sum. b may be null: a block without the second sublayer; a null scale is all ones. Four channels a thread
// where C allows.
__global__ void scaled_add_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ ls_a,
                                  const float* __restrict__ b, const float* __restrict__ ls_b, float mult, long long total,
                                  int C, int vec) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * (vec ? 4 : 1);
  if (i >= total) return;
  if (vec) {
    const int c = (int)(i % C);
    float4 xv = *reinterpret_cast<float4*>(x + i);
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 av = *reinterpret_cast<const float4*>(a + i), la = ls_a ? *reinterpret_cast<const float4*>(ls_a + c) : one;
    float4 sum = make_float4(la.x * av.x, la.y * av.y, la.z * av.z, la.w * av.w);
    if (b != nullptr) {
      const float4 bv = *reinterpret_cast<const float4*>(b + i), lb = ls_b ? *reinterpret_cast<const float4*>(ls_b + c) : one;
      sum.x = fmaf(lb.x, bv.x, sum.x); sum.y = fmaf(lb.y, bv.y, sum.y); sum.z = fmaf(lb.z, bv.z, sum.z); sum.w = fmaf(lb.w, bv.w, sum.w);
    }
    xv.x = fmaf(mult, sum.x, xv.x); xv.y = fmaf(mult, sum.y, xv.y); xv.z = fmaf(mult, sum.z, xv.z); xv.w = fmaf(mult, sum.w, xv.w);
    *reinterpret_cast<float4*>(x + i) = xv;
  } else {
    const int c = (int)(i % C);
    float sum = (ls_a ? ls_a[c] : 1.f) * a[i];
    if (b != nullptr) sum = fmaf(ls_b ? ls_b[c] : 1.f, b[i], sum);
    x[i] = fmaf(mult, sum, x[i]);
  }
}

AKAS_API int akas_scaled_add(float* x, const float* a, const float* ls_a, const float* b, const float* ls_b, float mult, int N,
                             int C, cudaStream_t stream) {
  const long long total = (long long)N * C;
  if (total <= 0) return 0;
  const bool aligned = ((uintptr_t)x | (uintptr_t)a | (uintptr_t)ls_a | (uintptr_t)b | (uintptr_t)ls_b) % 16 == 0;
  const int vec = C % 4 == 0 && aligned;
  const long long threads = vec ? total / 4 : total;
  return launch_ordinary(scaled_add_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, stream, x, a, ls_a, b, ls_b,
                         mult, total, C, vec);
}

// PolyNorm of rows: out = a N(z) + b N(z^2) + c N(z^3) + e with N(x) = x / sqrt(mean(x^2) + eps) over the row and
// the powers taken element by element; coeffs = (a, b, c, e). One block per row; powers and sums are float32. VEC: the
// row's width is a multiple of 8 and rows start on 16 bytes, so 8 elements move at a time.
template <typename TI, typename TO, bool VEC>
__global__ void polynorm_kernel(const TI* __restrict__ z, const float* __restrict__ coeffs, float eps,
                                TO* __restrict__ out, int F) {
  __shared__ float scratch[3][32];
  const TI* row = z + (size_t)blockIdx.x * F;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (VEC) {
    for (int c = threadIdx.x * 8; c < F; c += blockDim.x * 8) {
      float x[8];
      load8(row + c, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x2 = x[e] * x[e], x3 = x2 * x[e];
        s1 = fmaf(x[e], x[e], s1);
        s2 = fmaf(x2, x2, s2);
        s3 = fmaf(x3, x3, s3);
      }
    }
  } else {
    for (int c = threadIdx.x; c < F; c += blockDim.x) {
      const float x = to_f32(row[c]), x2 = x * x, x3 = x2 * x;
      s1 = fmaf(x, x, s1);
      s2 = fmaf(x2, x2, s2);
      s3 = fmaf(x3, x3, s3);
    }
  }
  // the three sums meet together: one pair of barriers instead of three
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  s1 = warp_sum(s1); s2 = warp_sum(s2); s3 = warp_sum(s3);
  if (lane == 0) { scratch[0][warp] = s1; scratch[1][warp] = s2; scratch[2][warp] = s3; }
  __syncthreads();
  s1 = warp_sum(lane < warps ? scratch[0][lane] : 0.f);
  s2 = warp_sum(lane < warps ? scratch[1][lane] : 0.f);
  s3 = warp_sum(lane < warps ? scratch[2][lane] : 0.f);
  const float i1 = coeffs[0] / sqrtf(s1 / (float)F + eps);
  const float i2 = coeffs[1] / sqrtf(s2 / (float)F + eps);
  const float i3 = coeffs[2] / sqrtf(s3 / (float)F + eps);
  const float e0 = coeffs[3];
  TO* dst = out + (size_t)blockIdx.x * F;
  if (VEC) {
    for (int c = threadIdx.x * 8; c < F; c += blockDim.x * 8) {
      float x[8], y[8];
      load8(row + c, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x2 = x[e] * x[e];
        y[e] = fmaf(x[e], i1, fmaf(x2, i2, fmaf(x2 * x[e], i3, e0)));
      }
      store8(dst + c, y);
    }
  } else {
    for (int c = threadIdx.x; c < F; c += blockDim.x) {
      const float x = to_f32(row[c]), x2 = x * x;
      dst[c] = from_f32<TO>(fmaf(x, i1, fmaf(x2, i2, fmaf(x2 * x, i3, e0))));
    }
  }
}

AKAS_API int akas_polynorm(const void* z, const float* coeffs, float eps, void* out, int N, int F, int in_dtype,
                           int out_dtype, cudaStream_t stream) {
  if (N <= 0) return 0;
  const int threads = F >= 4096 ? 512 : F >= 1024 ? 256 : 128;
  const bool vec = F % 8 == 0 && (uintptr_t)z % 16 == 0 && (uintptr_t)out % 16 == 0;
#define AKAS_POLY(TI, TO)                                                                                              \
  {                                                                                                                    \
    if (vec) return launch_ordinary(polynorm_kernel<TI, TO, true>, dim3(N), dim3(threads), 0, stream, (const TI*)z, coeffs, eps, (TO*)out, F);  \
    return launch_ordinary(polynorm_kernel<TI, TO, false>, dim3(N), dim3(threads), 0, stream, (const TI*)z, coeffs, eps, (TO*)out, F);          \
  }
  if (in_dtype == AKAS_F32 && out_dtype == AKAS_F32) AKAS_POLY(float, float)
  else if (in_dtype == AKAS_F32) AKAS_POLY(float, bf16)
  else if (out_dtype == AKAS_F32) AKAS_POLY(bf16, float)
  else AKAS_POLY(bf16, bf16)
#undef AKAS_POLY
}

// Dynamic Tanh, a norm without statistics: y[m, c] = tanh(alpha * x[row(m), c]) * w[c] + b[c], float32 throughout,
// rounded once on the way out. alpha is one number on the device. rows: optional gather of the rows to norm.
// ADD (float32 y only): y += the result, the norm behind a sublayer and the residual sum in one pass.
template <typename TO, bool ADD>
__global__ void dynamic_tanh_kernel(const float* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ w,
                                    const float* __restrict__ b, TO* __restrict__ y, const int* __restrict__ rows, int C,
                                    size_t total) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= total) return;
  const float a = alpha[0];
  if (C % 4 == 0) {  // four channels of one row, 16 bytes in
    const size_t m = i / C;
    const int c = (int)(i % C);
    const size_t src = (rows != nullptr ? (size_t)rows[m] : m) * C + c;
    const float4 v = *reinterpret_cast<const float4*>(x + src);
    const float4 wv = *reinterpret_cast<const float4*>(w + c), bv = *reinterpret_cast<const float4*>(b + c);
    if constexpr (ADD) {
      float4 r = *reinterpret_cast<const float4*>(y + i);
      r.x += fmaf(tanhf(a * v.x), wv.x, bv.x);
      r.y += fmaf(tanhf(a * v.y), wv.y, bv.y);
      r.z += fmaf(tanhf(a * v.z), wv.z, bv.z);
      r.w += fmaf(tanhf(a * v.w), wv.w, bv.w);
      *reinterpret_cast<float4*>(y + i) = r;
      return;
    }
    y[i] = from_f32<TO>(fmaf(tanhf(a * v.x), wv.x, bv.x));
    y[i + 1] = from_f32<TO>(fmaf(tanhf(a * v.y), wv.y, bv.y));
    y[i + 2] = from_f32<TO>(fmaf(tanhf(a * v.z), wv.z, bv.z));
    y[i + 3] = from_f32<TO>(fmaf(tanhf(a * v.w), wv.w, bv.w));
    return;
  }
  for (size_t j = i; j < total && j < i + 4; ++j) {
    const size_t m = j / C;
    const int c = (int)(j % C);
    const size_t src = (rows != nullptr ? (size_t)rows[m] : m) * C + c;
    const float value = fmaf(tanhf(a * x[src]), w[c], b[c]);
    if constexpr (ADD) y[j] += value;
    else y[j] = from_f32<TO>(value);
  }
}

AKAS_API int akas_dynamic_tanh(const float* x, const float* alpha, const float* w, const float* b, void* y, const int* rows,
                               int M, int C, int out_dtype, int add, cudaStream_t stream) {
  const size_t total = (size_t)M * C;
  if (total == 0) return 0;
  if (add && out_dtype != AKAS_F32) return (int)cudaErrorInvalidValue;
  const unsigned blocks = (unsigned)((total + 1023) / 1024);
  if (add) dynamic_tanh_kernel<float, true><<<blocks, 256, 0, stream>>>(x, alpha, w, b, (float*)y, rows, C, total);
  else if (out_dtype == AKAS_F32) dynamic_tanh_kernel<float, false><<<blocks, 256, 0, stream>>>(x, alpha, w, b, (float*)y, rows, C, total);
  else dynamic_tanh_kernel<bf16, false><<<blocks, 256, 0, stream>>>(x, alpha, w, b, (bf16*)y, rows, C, total);
  return launch_status();
}

// The middle of a gated feed-forward whose first product left float32: out[n, f] = act(g + b_g) * (u + b_u) with
// g = gu[n, f], u = gu[n, F + f] (rows of pitch ld), biases optional, act the tanh form of gelu (0) or silu (1);
// float32 until the one rounding. The same launch adds the last product's bias to the residual stream
// (res[n, c] += res_bias[c], float32 [N, C]) where one is given, so that product can accumulate into it.
__device__ __forceinline__ float gelu_tanh_f32(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// An activation without a gate on a product's rows: out[n, f] = act(z[n, f]) for z float32 or bfloat16 with a row
// pitch, act the square of max(z, 0) (0), the tanh form of gelu (1) or silu (2); float32 until the one rounding.
template <typename TI, typename TO>
__global__ void activation_kernel(const TI* __restrict__ z, long long ld, TO* __restrict__ out, int N, int F, int act) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * F) return;
  const size_t n = i / F;
  const int f = (int)(i % F);
  const float v = to_f32(z[n * ld + f]);
  float a;
  if (act == 0) { const float r = fmaxf(v, 0.f); a = r * r; }
  else if (act == 1) a = gelu_tanh_f32(v);
  else a = v / (1.f + expf(-v));
  out[i] = from_f32<TO>(a);
}

AKAS_API int akas_activation(const void* z, long long ld, int in_dtype, void* out, int out_dtype, int N, int F, int act,
                             cudaStream_t stream) {
  if (N <= 0 || F <= 0) return 0;
  if (act < 0 || act > 2) return (int)cudaErrorInvalidValue;
  const unsigned blocks = (unsigned)(((size_t)N * F + 255) / 256);
#define AKAS_ACT(TI, TO) activation_kernel<TI, TO><<<blocks, 256, 0, stream>>>((const TI*)z, ld, (TO*)out, N, F, act)
  if (in_dtype == AKAS_F32 && out_dtype == AKAS_F32) AKAS_ACT(float, float);
  else if (in_dtype == AKAS_F32) AKAS_ACT(float, bf16);
  else if (out_dtype == AKAS_F32) AKAS_ACT(bf16, float);
  else AKAS_ACT(bf16, bf16);
#undef AKAS_ACT
  return launch_status();
}

template <typename TO>
__global__ void gated_activation_kernel(const float* __restrict__ gu, long long ld, const float* __restrict__ bias,
                                        TO* __restrict__ out, int F, int act, float* __restrict__ res,
                                        const float* __restrict__ res_bias, int C) {
  const int n = blockIdx.x;
  const float* row = gu + (size_t)n * ld;
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    float g = row[f], u = row[F + f];
    if (bias != nullptr) { g += bias[f]; u += bias[F + f]; }
    const float a = act == 0 ? gelu_tanh_f32(g) : g / (1.f + expf(-g));
    out[(size_t)n * F + f] = from_f32<TO>(a * u);
  }
  if (res != nullptr)
    for (int c = threadIdx.x; c < C; c += blockDim.x) res[(size_t)n * C + c] += res_bias[c];
}

AKAS_API int akas_gated_activation(const float* gu, long long ld, const float* bias, void* out, int N, int F, int act,
                                   int out_dtype, float* res, const float* res_bias, int C, cudaStream_t stream) {
  if (N <= 0 || F <= 0) return 0;
  if (act != 0 && act != 1) return (int)cudaErrorInvalidValue;
  const int threads = F >= 1024 ? 256 : 128;
  if (out_dtype == AKAS_F32)
    gated_activation_kernel<float><<<N, threads, 0, stream>>>(gu, ld, bias, (float*)out, F, act, res, res_bias, C);
  else
    gated_activation_kernel<bf16><<<N, threads, 0, stream>>>(gu, ld, bias, (bf16*)out, F, act, res, res_bias, C);
  return launch_status();
}
