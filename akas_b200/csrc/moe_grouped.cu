// The experts of a routed feed-forward for prompt portions in bfloat16, on Blackwell's tensor cores: a grouped
// product. The step's (token, chosen real expert) pairs are sorted by expert into a buffer of rows in which every
// expert's rows start on a multiple of 128, so a tile of 128 rows belongs to one expert; a table on the device names
// each tile's expert. Nothing about the routing is known on the host: the grid is sized for the most tiles the step
// can need, and blocks walk the tiles that the plan kernel counted.
//
//   moe_plan     one block: counts the pairs of every expert, lays the experts' row ranges out (each rounded up to
//                128 rows), gives every pair its row (-1 for an identity expert) and every tile its expert.
//   moe_gather   copies each pair's token row of h into its row of the sorted buffer.
//   grouped product (the persistent, TMA-fed, tcgen05 kernel of gemm_tcgen05.cu with an expert per tile): B tiles
//                come from the stacked matrices [experts * rows, K] at the tile's expert;
//                  SWIGLU: act[row, F] = silu(gate) * up, bfloat16;   F32: y[row, C] = act . W_down^T, float32.
//   moe_combine  out[n] = sum_k weight[n, k] * (y[row of pair (n, k)], or h[n] for an identity expert), in the
//                order of the choice, float32; or, given the residual stream x, x += mult * (ls_a * a + ls_b * that sum).
// Every output is a sum over the inner size in the tile order of K, whatever the step holds beside the token, so a
// token's result does not depend on the batch. Waits are bounded as in gemm_tcgen05.cu (akas_moe_grouped_status).
#include <math.h>

#include "tcgen05.cuh"

using namespace akas;
using namespace akas::tc;

namespace {

constexpr int BM = 128, STAGES = 4;
constexpr int THREADS = 192;
enum { EPI_F32 = 1, EPI_SWIGLU = 2 };

__device__ int g_grouped_status = 0;  // 0, or which bounded wait ran out last (1 producer, 2 tensor cores, 3 epilogue)

constexpr int kPlanThreads = 1024;
constexpr int kMaxExperts = 1024;

// plan[0] = tiles of 128 rows in use; tile_expert[t] = expert of tile t; row_of_pair[p] = row of pair p in the sorted
// buffer, or -1. Rows inside an expert's range are handed out in the order the threads arrive: which row a pair
// gets does not change what is computed for it.
__global__ void __launch_bounds__(kPlanThreads)
moe_plan_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ row_of_pair,
                int* __restrict__ tile_expert, int* __restrict__ plan) {
  __shared__ int count[kMaxExperts], start[kMaxExperts];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = tiles * BM;
      const int t = (count[e] + BM - 1) / BM;
      for (int i = 0; i < t; ++i) tile_expert[tiles + i] = e;
      tiles += t;
      count[e] = 0;  // from here on: the rows handed out
    }
    plan[0] = tiles;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = chosen[p];
    row_of_pair[p] = e >= 0 && e < experts ? start[e] + atomicAdd(&count[e], 1) : -1;
  }
}

// in_weights (or null): the pair's weight multiplies its copy of the token's row (the weight on an expert's input),
// in float32, rounded once.
__global__ void moe_gather_kernel(const bf16* __restrict__ h, long long ldh, const int* __restrict__ row_of_pair,
                                  bf16* __restrict__ sorted, int top, int C, const float* __restrict__ in_weights) {
  const int pair = blockIdx.x;
  const int row = row_of_pair[pair];
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(pair / top) * ldh);
  uint4* dst = reinterpret_cast<uint4*>(sorted + (size_t)row * C);
  if (in_weights == nullptr) {
    for (int i = threadIdx.x; i < C / 8; i += blockDim.x) dst[i] = src[i];
    return;
  }
  const float g = in_weights[pair];
  for (int i = threadIdx.x; i < C / 8; i += blockDim.x) {
    float v[8];
    load_vec(reinterpret_cast<const bf16*>(src + i), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= g;
    store_vec(reinterpret_cast<bf16*>(dst + i), v);
  }
}

__global__ void moe_combine_kernel(const bf16* __restrict__ h, long long ldh, const float* __restrict__ y,
                                   const int* __restrict__ row_of_pair, const float* __restrict__ weights,
                                   float* __restrict__ out, int top, int C, float* __restrict__ x, const float* __restrict__ a_res,
                                   const float* __restrict__ ls_a, const float* __restrict__ ls_b, float mult,
                                   const float* __restrict__ shared, const float* __restrict__ shared_gate, long long ldsg) {
  // null weights: every weight is one. shared (or null): float32 [N, C] added to the sum, times shared_gate[n * ldsg]
  // where that is given.
  const int n = blockIdx.x;
  for (int c = threadIdx.x * 4; c < C; c += blockDim.x * 4) {
    float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
    if (shared != nullptr) {
      const float sg = shared_gate != nullptr ? shared_gate[(size_t)n * ldsg] : 1.f;
      const float4 sv = *reinterpret_cast<const float4*>(shared + (size_t)n * C + c);
      total = make_float4(sg * sv.x, sg * sv.y, sg * sv.z, sg * sv.w);
    }
    for (int k = 0; k < top; ++k) {
      const int row = row_of_pair[(size_t)n * top + k];
      const float g = weights != nullptr ? weights[(size_t)n * top + k] : 1.f;
      float4 v;
      if (row >= 0) {
        v = *reinterpret_cast<const float4*>(y + (size_t)row * C + c);
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(h + (size_t)n * ldh + c);
        v = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                        __uint_as_float(raw.y & 0xffff0000u));
      }
      total.x = fmaf(g, v.x, total.x); total.y = fmaf(g, v.y, total.y);
      total.z = fmaf(g, v.z, total.z); total.w = fmaf(g, v.w, total.w);
    }
    if (x != nullptr) {
      const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
      const float4 la = ls_a ? *reinterpret_cast<const float4*>(ls_a + c) : one, lb = ls_b ? *reinterpret_cast<const float4*>(ls_b + c) : one;
      const float4 av = *reinterpret_cast<const float4*>(a_res + (size_t)n * C + c);
      float4 xv = *reinterpret_cast<float4*>(x + (size_t)n * C + c);
      xv.x = fmaf(mult, fmaf(lb.x, total.x, la.x * av.x), xv.x); xv.y = fmaf(mult, fmaf(lb.y, total.y, la.y * av.y), xv.y);
      xv.z = fmaf(mult, fmaf(lb.z, total.z, la.z * av.z), xv.z); xv.w = fmaf(mult, fmaf(lb.w, total.w, la.w * av.w), xv.w);
      *reinterpret_cast<float4*>(x + (size_t)n * C + c) = xv;
    } else {
      *reinterpret_cast<float4*>(out + (size_t)n * C + c) = total;
    }
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS)
grouped_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               void* __restrict__ y_, const int* __restrict__ tile_expert, const int* __restrict__ plan, int N, int K, int F) {
  // A tile's B rows are those of its expert in the stacked matrix [experts * N, K]; M is what the plan kernel counted.
  // N: channels of the product (for SWIGLU the stacked height 2F); a tile covers BN of them (SWIGLU: BN/2 gate
  // rows f0.. and BN/2 up rows F + f0..).
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TILE_N = EPI == EPI_SWIGLU ? BN / 2 : BN;  // output columns a tile yields
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int out_cols = EPI == EPI_SWIGLU ? F : N;
  const int tiles_m = plan[0], tiles_n = (out_cols + TILE_N - 1) / TILE_N;
  const int M = tiles_m * BM;
  const int tiles = tiles_m * tiles_n, k_blocks = (K + BK - 1) / BK;

  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory: two accumulators of BN float32 columns, 128 lanes
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(2 * BN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_s;

  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) {
    if (*(volatile int*)&abort_s) return;
    if (!mbar_wait(bar, parity)) {
      *(volatile int*)&abort_s = 1;
      atomicExch(&g_grouped_status, code);
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      unsigned it = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * BM, n0 = tile_expert[tile / tiles_n] * N + (tile % tiles_n) * TILE_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          wait_for(&empty_bar[s], ((it / STAGES) & 1) ^ 1, 1);
          if (*(volatile int*)&abort_s) break;
          unsigned char* a = smem + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          tma_load_2d(a, &map_x, kb * BK, m0, &full_bar[s]);
          if (EPI == EPI_SWIGLU) {
            tma_load_2d(a + A_BYTES, &map_w, kb * BK, n0, &full_bar[s]);
            tma_load_2d(a + A_BYTES + B_BYTES / 2, &map_w, kb * BK, F + n0, &full_bar[s]);
          } else {
            tma_load_2d(a + A_BYTES, &map_w, kb * BK, n0, &full_bar[s]);
          }
        }
        if (*(volatile int*)&abort_s) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor cores
    if (lane == 0) {
      // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = BN, M = 128
      constexpr unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
      unsigned it = 0, t = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
        const unsigned acc = t & 1;
        wait_for(&acc_empty[acc], ((t >> 1) & 1) ^ 1, 2);  // the epilogue has drained this accumulator
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          wait_for(&full_bar[s], (it / STAGES) & 1, 2);
          if (*(volatile int*)&abort_s) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* a = smem + (size_t)s * STAGE_BYTES;
          const uint64_t a_desc = smem_desc(a), b_desc = smem_desc(a + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further along the swizzled row per step
            umma(d, a_desc + (uint64_t)(k * UMMA_K * 2 >> 4), b_desc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                 (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);  // the stage is free once these products have read it
        }
        if (*(volatile int*)&abort_s) break;
        umma_commit(&acc_full[acc]);  // the tile's sums are complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: warps 2..5
    const int sub = warp & 3;  // the tensor-memory sub-partition (32 lanes) this warp may read
    unsigned t = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
      const unsigned acc = t & 1;
      const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * TILE_N;
      wait_for(&acc_full[acc], (t >> 1) & 1, 3);
      if (*(volatile int*)&abort_s) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = m0 + sub * 32 + lane;
      const unsigned taddr = tmem_base + acc * BN + ((unsigned)(sub * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < TILE_N; c += 16) {
        float v[16];
        tmem_load16(taddr + c, v);
        if (EPI == EPI_SWIGLU) {
          float u[16];
          tmem_load16(taddr + BN / 2 + c, u);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __fdividef(v[i], 1.f + __expf(-v[i])) * u[i];  // the fast division: IEEE division cost more than the tile's loads
        }
        const int col = n0 + c;
        if (row < M && col < out_cols) {
          if (EPI == EPI_F32) {
            float* dst = (float*)y_ + (size_t)row * out_cols + col;
            if (col + 16 <= out_cols && out_cols % 4 == 0) {
#pragma unroll
              for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            } else {
              for (int i = 0; i < 16 && col + i < out_cols; ++i) dst[i] = v[i];
            }
          } else {
            bf16* dst = (bf16*)y_ + (size_t)row * out_cols + col;
            if (col + 16 <= out_cols && out_cols % 8 == 0) {
              float lo[8], hi[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
              store_vec(dst, lo);
              store_vec(dst + 8, hi);
            } else {
              for (int i = 0; i < 16 && col + i < out_cols; ++i) dst[i] = __float2bfloat16_rn(v[i]);
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
  }

  // wind down: everyone meets, then the allocating warp frees tensor memory
  if (*(volatile int*)&abort_s) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // a lost launch: let copies and products in flight finish
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN));
  }
}

// ------------------------------------------------------------------------------------------------ host side

template <int BN, int EPI>
int launch(const void* x, const void* w, void* y, const int* tile_expert, const int* plan, int rows_cap, int experts, int N,
           int K, cudaStream_t stream) {
  constexpr int smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
  static int sms_of[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (sms_of[device] == 0) {
    const cudaError_t e = cudaFuncSetAttribute(grouped_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cudaDeviceGetAttribute(&sms_of[device], cudaDevAttrMultiProcessorCount, device);
  }
  const int sms = sms_of[device];
  const int F = N / 2;
  CUtensorMap map_x, map_w;
  int err = cached_map(&map_x, x, rows_cap, K, BM, false);
  if (err) return err;
  err = cached_map(&map_w, w, experts * N, K, EPI == EPI_SWIGLU ? BN / 2 : BN, true);
  if (err) return err;
  const int out_cols = EPI == EPI_SWIGLU ? F : N, tile_n = EPI == EPI_SWIGLU ? BN / 2 : BN;
  const long long most = (long long)(rows_cap / BM) * ((out_cols + tile_n - 1) / tile_n);
  const int grid = most < sms ? (int)most : sms;
  grouped_kernel<BN, EPI><<<grid, THREADS, smem, stream>>>(map_x, map_w, y, tile_expert, plan, N, K, F);
  return launch_status();
}

}  // namespace

// Rows that the sorted buffer needs for `pairs` pairs over `experts` experts: every expert's range rounded up to 128.
AKAS_API int akas_moe_grouped_rows(int pairs, int experts) { return ((pairs + experts * (BM - 1)) / BM + 1) * BM; }

// Whether the grouped path takes these sizes (16-byte rows for TMA and for the 8-byte loads of the combine kernel).
AKAS_API int akas_moe_grouped_takes(int C, int F, int experts) { return C % 8 == 0 && F % 8 == 0 && experts > 0 && experts <= kMaxExperts; }

// chosen [N, top] int32 (an expert number >= experts: an identity expert); outputs row_of_pair [N * top], tile_expert
// [rows_cap / 128], plan [1], sorted [rows_cap, C] bfloat16.
AKAS_API int akas_moe_sort(const void* h, long long ldh, const int* chosen, int* row_of_pair, int* tile_expert, int* plan,
                           void* sorted, int N, int top, int C, int experts, const float* in_weights, cudaStream_t stream) {
  if (N <= 0 || top <= 0) return 0;
  if (!akas_moe_grouped_takes(C, 8, experts) || ldh % 8 || (uintptr_t)h % 16 || (uintptr_t)sorted % 16) return (int)cudaErrorInvalidValue;
  int err = launch_ordinary(moe_plan_kernel, dim3(1), dim3(kPlanThreads), 0, stream, chosen, N * top, experts, row_of_pair,
                            tile_expert, plan);
  if (err) return err;
  return launch_ordinary(moe_gather_kernel, dim3(N * top), dim3(128), 0, stream, (const bf16*)h, ldh, (const int*)row_of_pair,
                         (bf16*)sorted, top, C, in_weights);
}

// epilogue 2: x = sorted [rows_cap, K = C], w = [experts, 2F, C] (N = 2F), y = act [rows_cap, F] bfloat16;
// epilogue 1: x = act [rows_cap, K = F], w = [experts, C, F] (N = C), y float32 [rows_cap, C].
AKAS_API int akas_moe_grouped_gemm(const void* x, const void* w, void* y, const int* tile_expert, const int* plan, int rows_cap,
                                   int experts, int N, int K, int epilogue, cudaStream_t stream) {
  if (rows_cap <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || rows_cap % BM || (uintptr_t)x % 16 || (uintptr_t)w % 16 || (uintptr_t)y % 16) return (int)cudaErrorInvalidValue;
  if (epilogue == EPI_SWIGLU) {
    if (N % 2 || (N / 2) % 8) return (int)cudaErrorInvalidValue;
    return launch<256, EPI_SWIGLU>(x, w, y, tile_expert, plan, rows_cap, experts, N, K, stream);
  }
  if (epilogue != EPI_F32) return (int)cudaErrorInvalidValue;
  // (128 x 128 tiles for steps whose 128 x 256 tiles would leave SMs without one were measured and dropped: the down
  // product of 64 tokens over 14 experts took 48 us against 43 us)
  return N <= 128 ? launch<128, EPI_F32>(x, w, y, tile_expert, plan, rows_cap, experts, N, K, stream)
                  : launch<256, EPI_F32>(x, w, y, tile_expert, plan, rows_cap, experts, N, K, stream);
}

AKAS_API int akas_moe_combine(const void* h, long long ldh, const float* y, const int* row_of_pair, const float* weights,
                              float* out, int N, int top, int C, float* x, const float* a_res, const float* ls_a,
                              const float* ls_b, float mult, const float* shared, const float* shared_gate, long long ldsg,
                              cudaStream_t stream) {
  if (N <= 0) return 0;
  if (C % 8 || ldh % 4 || (uintptr_t)h % 8 || (uintptr_t)y % 16 || (uintptr_t)out % 16 || (uintptr_t)shared % 16)
    return (int)cudaErrorInvalidValue;
  if (((uintptr_t)x | (uintptr_t)a_res | (uintptr_t)ls_a | (uintptr_t)ls_b) % 16) return (int)cudaErrorInvalidValue;
  return launch_ordinary(moe_combine_kernel, dim3(N), dim3(C >= 1024 ? 256 : 128), 0, stream, (const bf16*)h, ldh, y, row_of_pair,
                         weights, out, top, C, x, a_res, ls_a, ls_b, mult, shared, shared_gate, ldsg);
}

AKAS_API int akas_moe_grouped_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_grouped_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}
