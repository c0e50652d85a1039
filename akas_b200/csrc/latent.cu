// Kernels of attention through low-rank latents (parts/latent.py), around the general attention kernels.
//
// latent_norm_store: from the stacked input product of a token (float32), the query latent over its root mean square
// times its weight (to the compute dtype), and the token's cache row: the key/value latent over ITS root mean square
// times its weight, followed by the shared key part rotated by the token's angles. Everything in float32, rounded once.
//
// head_linear: one small matrix per head, out[n, h, :O] = w[h] x[n, h, :K] (float32 sums, one ascending chain of
// fused multiply-adds per output whatever the batch), optionally times sigmoid(gate), and a tail of T channels per
// head carried over, rotated where angles are given. A block takes a head and a tile of tokens: the head's matrix is
// read once per tile, the tokens' rows wait in shared memory.
#include <math.h>

#include "common.cuh"

using namespace akas;

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
latent_norm_store_kernel(const float* __restrict__ proj, long long ld, int QR, int KR, int rot,
                         const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                         const float* __restrict__ cos_t, const float* __restrict__ sin_t, int interleaved,
                         T* __restrict__ q_out, T* __restrict__ pool, const int* __restrict__ block_table, int max_blocks,
                         const int* __restrict__ seq_of_token, const int* __restrict__ positions, int page_size, int write) {
  __shared__ float scratch[32];
  const int n = blockIdx.x;
  const int req = seq_of_token[n];
  if (req < 0) return;
  const float* row = proj + (size_t)n * ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < QR; i += blockDim.x) { const float x = row[i]; ss = fmaf(x, x, ss); }
  ss = block_sum(ss, scratch);
  const float inv_q = 1.f / sqrtf(ss / (float)QR + eps);
  for (int i = threadIdx.x; i < QR; i += blockDim.x) q_out[(size_t)n * QR + i] = from_f32<T>(row[i] * inv_q * qw[i]);
  if (!write) return;
  const float* c = row + QR;
  float sc = 0.f;
  for (int i = threadIdx.x; i < KR; i += blockDim.x) { const float x = c[i]; sc = fmaf(x, x, sc); }
  sc = block_sum(sc, scratch);
  const float inv_c = 1.f / sqrtf(sc / (float)KR + eps);
  const int pos = positions[n];
  const int page = block_table[(size_t)req * max_blocks + pos / page_size];
  T* dst = pool + ((size_t)page * page_size + pos % page_size) * (size_t)(KR + rot);
  for (int i = threadIdx.x; i < KR; i += blockDim.x) dst[i] = from_f32<T>(c[i] * inv_c * kw[i]);
  const float* tail = c + KR;
  if (cos_t == nullptr) {
    for (int i = threadIdx.x; i < rot; i += blockDim.x) dst[KR + i] = from_f32<T>(tail[i]);
    return;
  }
  const int half = rot / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
    const float u = tail[a], x = tail[b];
    const float cs = cos_t[(size_t)n * half + i], sn = sin_t[(size_t)n * half + i];
    dst[KR + a] = from_f32<T>(fmaf(u, cs, -x * sn));
    dst[KR + b] = from_f32<T>(fmaf(x, cs, u * sn));
  }
}

constexpr int kRows = 16;    // tokens of a block's tile
constexpr int kChunk = 256;  // inner channels staged at a time
constexpr int kPitch = kChunk + 4;

template <typename T, typename TG>
__global__ void __launch_bounds__(128)
head_linear_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w, T* __restrict__ out, long long ldo,
                   const TG* __restrict__ gate, long long ldg, const float* __restrict__ cos_t,
                   const float* __restrict__ sin_t, int interleaved, int N, int H, int O, int K, int Tt) {
  __shared__ __align__(16) float xs[kRows * kPitch];
  constexpr int VN = Vec<T>::N;
  const int h = blockIdx.y, n0 = blockIdx.x * kRows;
  const int rows = min(kRows, N - n0);
  const int tid = threadIdx.x;
  const T* xh = x + (size_t)n0 * ldx + (size_t)h * (K + Tt);
  const bool wide = K % VN == 0;  // a row of the matrix starts on a 16-byte boundary
  // every thread owns outputs o = tid, tid + 128, ...: passes over them, each a walk over the chunks of K
  for (int o0 = 0; o0 < O; o0 += blockDim.x) {
    const int o = o0 + tid;
    float acc[kRows];
#pragma unroll
    for (int t = 0; t < kRows; ++t) acc[t] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kChunk) {
      const int kc = min(kChunk, K - k0);
      __syncthreads();
      for (int i = tid; i < kRows * kc; i += blockDim.x) {
        const int t = i / kc, k = i % kc;
        xs[t * kPitch + k] = t < rows ? to_f32(xh[(size_t)t * ldx + k0 + k]) : 0.f;
      }
      __syncthreads();
      if (o < O) {
        const T* wr = w + ((size_t)h * O + o) * K + k0;
        int k = 0;
        if (wide) {
          for (; k + VN <= kc; k += VN) {
            float wv[VN];
            load_vec(wr + k, wv);
#pragma unroll
            for (int t = 0; t < kRows; ++t) {
#pragma unroll
              for (int e = 0; e < VN; e += 4) {
                const float4 xv = *reinterpret_cast<const float4*>(xs + t * kPitch + k + e);
                acc[t] = fmaf(xv.x, wv[e], acc[t]);
                acc[t] = fmaf(xv.y, wv[e + 1], acc[t]);
                acc[t] = fmaf(xv.z, wv[e + 2], acc[t]);
                acc[t] = fmaf(xv.w, wv[e + 3], acc[t]);
              }
            }
          }
        }
        for (; k < kc; ++k) {
          const float wv = to_f32(wr[k]);
#pragma unroll
          for (int t = 0; t < kRows; ++t) acc[t] = fmaf(xs[t * kPitch + k], wv, acc[t]);
        }
      }
    }
    if (o < O) {
#pragma unroll
      for (int t = 0; t < kRows; ++t) {
        if (t < rows) {
          float y = acc[t];
          if (gate != nullptr) y *= 1.f / (1.f + expf(-to_f32(gate[(size_t)(n0 + t) * ldg + (size_t)h * O + o])));
          out[(size_t)(n0 + t) * ldo + (size_t)h * (O + Tt) + o] = from_f32<T>(y);
        }
      }
    }
  }
  if (Tt <= 0) return;
  // the head's further channels: carried over, turned by the token's angles where there are any
  if (cos_t == nullptr) {
    for (int i = tid; i < rows * Tt; i += blockDim.x) {
      const int t = i / Tt, c = i % Tt;
      out[(size_t)(n0 + t) * ldo + (size_t)h * (O + Tt) + O + c] = xh[(size_t)t * ldx + K + c];
    }
    return;
  }
  const int half = Tt / 2;
  for (int i = tid; i < rows * half; i += blockDim.x) {
    const int t = i / half, p = i % half;
    const int a = interleaved ? 2 * p : p, b = interleaved ? 2 * p + 1 : p + half;
    const float u = to_f32(xh[(size_t)t * ldx + K + a]), v = to_f32(xh[(size_t)t * ldx + K + b]);
    const float cs = cos_t[(size_t)(n0 + t) * half + p], sn = sin_t[(size_t)(n0 + t) * half + p];
    T* dst = out + (size_t)(n0 + t) * ldo + (size_t)h * (O + Tt) + O;
    dst[a] = from_f32<T>(fmaf(u, cs, -v * sn));
    dst[b] = from_f32<T>(fmaf(v, cs, u * sn));
  }
}

}  // namespace

AKAS_API int akas_latent_norm_store(const float* proj, long long ld, int QR, int KR, int rot, const float* qw, const float* kw,
                                    float eps, const float* cos_t, const float* sin_t, int interleaved, void* q_out, void* pool,
                                    const int* block_table, int max_blocks, const int* seq_of_token, const int* positions,
                                    int page_size, int N, int write, int dtype, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (QR <= 0 || KR <= 0 || rot < 0 || (cos_t != nullptr && rot % 2)) return (int)cudaErrorInvalidValue;
  if (dtype == AKAS_F32)
    return launch_ordinary(latent_norm_store_kernel<float>, dim3(N), dim3(128), 0, stream, proj, ld, QR, KR, rot, qw, kw, eps,
                           cos_t, sin_t, interleaved, (float*)q_out, (float*)pool, block_table, max_blocks, seq_of_token,
                           positions, page_size, write);
  return launch_ordinary(latent_norm_store_kernel<bf16>, dim3(N), dim3(128), 0, stream, proj, ld, QR, KR, rot, qw, kw, eps,
                         cos_t, sin_t, interleaved, (bf16*)q_out, (bf16*)pool, block_table, max_blocks, seq_of_token, positions,
                         page_size, write);
}

// x [N, H * (K + T)] with row pitch ldx, w [H, O, K], out [N, H * (O + T)] with row pitch ldo, all of `dtype`; gate
// (float32 or the same dtype, pitch ldg, [N, H * O]) and the angles (float32 [N, T / 2]) may be null.
AKAS_API int akas_head_linear(const void* x, long long ldx, const void* w, void* out, long long ldo, const void* gate,
                              long long ldg, int gate_dtype, const float* cos_t, const float* sin_t, int interleaved, int N,
                              int H, int O, int K, int T, int dtype, cudaStream_t stream) {
  if (N <= 0 || H <= 0) return 0;
  if (O <= 0 || K <= 0 || T < 0 || (cos_t != nullptr && T % 2) || H > 65535) return (int)cudaErrorInvalidValue;
  const dim3 grid((N + kRows - 1) / kRows, H), block(128);
#define AKAS_HL(TT, TG)                                                                                                  \
  return launch_ordinary(head_linear_kernel<TT, TG>, grid, block, 0, stream, (const TT*)x, ldx, (const TT*)w, (TT*)out, ldo, \
                         (const TG*)gate, ldg, cos_t, sin_t, interleaved, N, H, O, K, T)
  if (dtype == AKAS_F32) {
    if (gate != nullptr && gate_dtype != AKAS_F32) return (int)cudaErrorInvalidValue;
    AKAS_HL(float, float);
  }
  if (gate != nullptr && gate_dtype == AKAS_BF16) AKAS_HL(bf16, bf16);
  AKAS_HL(bf16, float);
#undef AKAS_HL
}
