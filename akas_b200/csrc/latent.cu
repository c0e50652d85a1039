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
#include "mma.cuh"

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
  // everything the block reads is asked for before the first sum meets: the token's place, its page, both latents
  const int pos = positions[n];
  const float* row = proj + (size_t)n * ld;
  const float* c = row + QR;
  float ss = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < QR; i += blockDim.x) { const float x = row[i]; ss = fmaf(x, x, ss); }
  int page = 0;
  if (write) {
    for (int i = threadIdx.x; i < KR; i += blockDim.x) { const float x = c[i]; sc = fmaf(x, x, sc); }
    page = block_table[(size_t)req * max_blocks + pos / page_size];
  }
  ss = block_sum(ss, scratch);
  if (write) sc = block_sum(sc, scratch);  // (`write` is the same for the whole launch)
  const float inv_q = 1.f / sqrtf(ss / (float)QR + eps);
  for (int i = threadIdx.x; i < QR; i += blockDim.x) q_out[(size_t)n * QR + i] = from_f32<T>(row[i] * inv_q * qw[i]);
  if (!write) return;
  const float inv_c = 1.f / sqrtf(sc / (float)KR + eps);
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

// A head's further channels for `rows` tokens from n0 on: carried over, turned by the token's angles where there are any.
template <typename T>
__device__ __forceinline__ void head_tail(const T* __restrict__ xh, long long ldx, T* __restrict__ out, long long ldo,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int interleaved,
                                          int n0, int rows, int h, int O, int K, int Tt) {
  const int tid = threadIdx.x;
  if (Tt <= 0) return;
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

constexpr int kRows = 16;   // tokens of a block's tile
constexpr int kChunk = 64;  // inner channels staged at a time
constexpr int kPitch = kChunk + 4;
constexpr int kOuts = 128;  // outputs of a pass: one per thread

template <typename T, typename TG>
__global__ void __launch_bounds__(kOuts)
head_linear_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w, T* __restrict__ out, long long ldo,
                   const TG* __restrict__ gate, long long ldg, const float* __restrict__ cos_t,
                   const float* __restrict__ sin_t, int interleaved, int N, int H, int O, int K, int Tt) {
  constexpr int VN = Vec<T>::N;
  constexpr int WP = kChunk + VN;  // a staged weight row's pitch: an odd number of 16-byte units, so rows do not collide
  __shared__ __align__(16) float xs[kRows * kPitch];
  __shared__ __align__(16) T ws[kOuts * WP];
  const int h = blockIdx.y, n0 = blockIdx.x * kRows;
  const int rows = min(kRows, N - n0);
  const int tid = threadIdx.x;
  const T* xh = x + (size_t)n0 * ldx + (size_t)h * (K + Tt);
  // rows of the matrix, and of the tokens, that start on 16-byte boundaries come in 16-byte loads
  const bool wide = K % VN == 0 && (uintptr_t)w % 16 == 0;
  const bool xwide = wide && ldx % VN == 0 && (K + Tt) % VN == 0 && (uintptr_t)x % 16 == 0;
  // every thread owns outputs o = tid, tid + blockDim, ...: passes over them, each a walk over the chunks of K. A
  // chunk of the tokens' rows (float32) and of the pass's matrix rows waits in shared memory: every thread fetches its
  // share of both with loads that do not wait for one another, where a walk along a matrix row in global memory
  // would pay a trip to memory per step.
  for (int o0 = 0; o0 < O; o0 += blockDim.x) {
    const int o = o0 + tid;
    const int outs = min((int)blockDim.x, O - o0);
    float acc[kRows];
#pragma unroll
    for (int t = 0; t < kRows; ++t) acc[t] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kChunk) {
      const int kc = min(kChunk, K - k0);
      const T* wt = w + ((size_t)h * O + o0) * K + k0;
      __syncthreads();
      if (xwide) {
        const int per = kc / VN;
        for (int i = tid; i < kRows * per; i += blockDim.x) {
          const int t = i / per, v = (i % per) * VN;
          float xv[VN];
#pragma unroll
          for (int e = 0; e < VN; ++e) xv[e] = 0.f;
          if (t < rows) load_vec(xh + (size_t)t * ldx + k0 + v, xv);
#pragma unroll
          for (int e = 0; e < VN; e += 4)
            *reinterpret_cast<float4*>(xs + t * kPitch + v + e) = make_float4(xv[e], xv[e + 1], xv[e + 2], xv[e + 3]);
        }
      } else {
        for (int i = tid; i < kRows * kc; i += blockDim.x) {
          const int t = i / kc, k = i % kc;
          xs[t * kPitch + k] = t < rows ? to_f32(xh[(size_t)t * ldx + k0 + k]) : 0.f;
        }
      }
      if (wide) {
        const int per = kc / VN;
        for (int i = tid; i < outs * per; i += blockDim.x) {
          const int r = i / per, v = (i % per) * VN;
          *reinterpret_cast<uint4*>(ws + r * WP + v) = *reinterpret_cast<const uint4*>(wt + (size_t)r * K + v);
        }
      } else {
        for (int i = tid; i < outs * kc; i += blockDim.x) {
          const int r = i / kc, k = i % kc;
          ws[r * WP + k] = wt[(size_t)r * K + k];
        }
      }
      __syncthreads();
      if (o < O) {
        const T* wr = ws + tid * WP;
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
  head_tail(xh, ldx, out, ldo, cos_t, sin_t, interleaved, n0, rows, h, O, K, Tt);
}

// The same on the tensor cores, for bfloat16 with K and O multiples of 16 and rows that start on 16-byte boundaries:
// a block of four warps takes a head, stages the head's matrix once ([O][K + 8]: rows 16 bytes apart from a multiple
// of 128, so the 8 x 8 matrix loads do not collide), and walks tiles of 64 tokens, 16 a warp. Per pair of 8-wide
// output tiles a warp runs K / 16 steps of two m16n8k16 products whose operands come by matrix loads; a token's sums
// run along K in the same order whatever the batch.
constexpr int kTcRows = 64;
constexpr int kTcSmemMax = 200 * 1024;

template <typename TG>
__global__ void __launch_bounds__(128)
head_linear_tc_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w, bf16* __restrict__ out,
                      long long ldo, const TG* __restrict__ gate, long long ldg, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int interleaved, int N, int H, int O, int K, int Tt) {
  extern __shared__ __align__(16) unsigned char head_smem[];
  const int P = K + 8;
  bf16* ws = reinterpret_cast<bf16*>(head_smem);  // [O][P]
  bf16* xs = ws + (size_t)O * P;                  // [kTcRows][P]
  const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int per = K / 8;
  for (int i = tid; i < O * per; i += blockDim.x) {
    const int r = i / per, v = (i % per) * 8;
    cp_async16(ws + (size_t)r * P + v, w + ((size_t)h * O + r) * K + v, 16);  // lands with the first tile of tokens
  }
  for (int n0 = blockIdx.x * kTcRows; n0 < N; n0 += gridDim.x * kTcRows) {
    const int rows = min(kTcRows, N - n0);
    const bf16* xh = x + (size_t)n0 * ldx + (size_t)h * (K + Tt);
    __syncthreads();  // the tile before has been read
    for (int i = tid; i < kTcRows * per; i += blockDim.x) {
      const int t = i / per, v = (i % per) * 8;
      cp_async16(xs + (size_t)t * P + v, xh + (size_t)(t < rows ? t : 0) * ldx + v, t < rows ? 16 : 0);  // zeros past the batch
    }
    cp_async_commit();
    // the further channels meanwhile: their loads travel beside the copies
    head_tail(xh, ldx, out, ldo, cos_t, sin_t, interleaved, n0, rows, h, O, K, Tt);
    cp_async_wait<0>();
    __syncthreads();
    const int r0 = warp * 16;
    if (r0 < rows) {
      for (int np = 0; np < O / 16; ++np) {
        float c[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
        for (int ks = 0; ks < K / 16; ++ks) {
          uint32_t a[4], b[4];
          ldmatrix_x4(a, xs + (size_t)(r0 + (lane & 15)) * P + ks * 16 + (lane >> 4) * 8);
          ldmatrix_x4(b, ws + (size_t)(np * 16 + (lane & 7) + (lane >> 4) * 8) * P + ks * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(c[0], a, b[0], b[1]);
          mma_bf16(c[1], a, b[2], b[3]);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int o = np * 16 + j * 8 + 2 * (lane & 3);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int t = r0 + (lane >> 2) + half * 8;
            if (t >= rows) continue;
            float y0 = c[j][2 * half], y1 = c[j][2 * half + 1];
            if (gate != nullptr) {
              const TG* gp = gate + (size_t)(n0 + t) * ldg + (size_t)h * O + o;
              y0 *= 1.f / (1.f + expf(-to_f32(gp[0])));
              y1 *= 1.f / (1.f + expf(-to_f32(gp[1])));
            }
            *reinterpret_cast<uint32_t*>(out + (size_t)(n0 + t) * ldo + (size_t)h * (O + Tt) + o) = pack_bf16(y0, y1);
          }
        }
      }
    }
  }
}

template <typename TG>
int launch_head_tc(const void* x, long long ldx, const void* w, void* out, long long ldo, const void* gate, long long ldg,
                   const float* cos_t, const float* sin_t, int interleaved, int N, int H, int O, int K, int T, size_t smem,
                   cudaStream_t stream) {
  static bool raised[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (!raised[device]) {
    const cudaError_t e = cudaFuncSetAttribute(head_linear_tc_kernel<TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemMax);
    if (e != cudaSuccess) return (int)e;
    raised[device] = true;
  }
  const int tiles = (N + kTcRows - 1) / kTcRows;
  const dim3 grid(min(tiles, max(1, 1184 / H)), H);  // a few blocks per SM at most: a block keeps its head's matrix
  return launch_ordinary(head_linear_tc_kernel<TG>, grid, dim3(128), smem, stream, (const bf16*)x, ldx, (const bf16*)w,
                         (bf16*)out, ldo, (const TG*)gate, ldg, cos_t, sin_t, interleaved, N, H, O, K, T);
}

}  // namespace

AKAS_API int akas_latent_norm_store(const float* proj, long long ld, int QR, int KR, int rot, const float* qw, const float* kw,
                                    float eps, const float* cos_t, const float* sin_t, int interleaved, void* q_out, void* pool,
                                    const int* block_table, int max_blocks, const int* seq_of_token, const int* positions,
                                    int page_size, int N, int write, int dtype, cudaStream_t stream) {
  if (N <= 0) return 0;
  // QR 0: there is no query latent (queries that are a projection of their own); only the cached row is made
  if (QR < 0 || (QR > 0 && qw == nullptr) || KR <= 0 || rot < 0 || (cos_t != nullptr && rot % 2)) return (int)cudaErrorInvalidValue;
  if (QR == 0 && !write) return 0;
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
  const size_t tc_smem = (size_t)(O + kTcRows) * (K + 8) * sizeof(bf16);
  if (dtype == AKAS_BF16 && K % 16 == 0 && O % 16 == 0 && ldx % 8 == 0 && (K + T) % 8 == 0 && ldo % 2 == 0 && (O + T) % 2 == 0 &&
      (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 4 == 0 && tc_smem <= (size_t)kTcSmemMax) {
    if (gate != nullptr && gate_dtype == AKAS_BF16)
      return launch_head_tc<bf16>(x, ldx, w, out, ldo, gate, ldg, cos_t, sin_t, interleaved, N, H, O, K, T, tc_smem, stream);
    return launch_head_tc<float>(x, ldx, w, out, ldo, gate, ldg, cos_t, sin_t, interleaved, N, H, O, K, T, tc_smem, stream);
  }
  const dim3 grid((N + kRows - 1) / kRows, H), block(O >= kOuts ? kOuts : (O + 31) / 32 * 32);  // a thread per output of a pass, in whole warps
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
