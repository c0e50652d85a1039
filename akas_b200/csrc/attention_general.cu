// Paged softmax attention with options that the specialised kernels do not take: value heads of another size than
// the keys', a capped score, a logarithmic distance penalty, first tokens that stay visible behind a sliding window,
// a sink in the softmax's denominator, and a sigmoid gate per head on the output. Prompt portions and decoded tokens
// run through the same kernel: one block per (token, key/value head) that serves the group's query heads.
//
// Token i of a request sees key j iff j <= i and (window == 0 or i - j < window or j < keep_first). For head h:
//   s_j = (q . k_j) * scale;  s_j <- cap * tanh(s_j / cap) if cap > 0;  s_j <- s_j - r1_h * ln(1 + r2_h * (i - j)) if r1;
//   p_j = exp(s_j) / (sink + sum_j' exp(s_j'));  out = out_scale * sigmoid(gate_h) * sum_j p_j v_j.
// The sink is exp(0), or exp(sinks[h]) where a learned logit per head is given. The output's rows have a pitch of
// their own (ldo elements), so a layer may write its heads into a part of a wider row.
// Scores, weights and sums are float32. The visible keys are walked in tiles of kTile keys whose borders are
// multiples of kTile counted from position 0 (the kept first tokens come first), so what a token computes, and in
// which order, depends on its position only: not on how the prompt was cut or on what else is in the batch.
#include "common.cuh"

using namespace akas;

namespace {

constexpr int kTile = 128;    // keys per tile = threads per block
constexpr int kMaxGroup = 16;  // query heads of a key/value head that one block serves at a time

// One block per token: RMSNorm of every head of q and k over D with a plain weight (or none), then (where tables are
// given) the rotation of the first `rot` channels of each head by the token's angles, channel 2i with 2i + 1
// (interleaved) or i with i + rot / 2; q to q_out [N, H * D], k and the untouched v into the pages at the token's
// (page, offset). v may be the very rows of k: the values are then the keys as projected, before the rotation.
// Where biases are given (float32, one per channel of q, k, v), they are added first, in float32; q, k and v may then
// be the float32 result of a product (TI) while the pages hold T, so product plus bias is rounded once.
template <typename TI, typename T>
__global__ void qk_norm_store_kernel(const TI* __restrict__ q, long long ldq, const TI* __restrict__ k, long long ldk,
                                     const TI* __restrict__ v, long long ldv, const float* __restrict__ qw,
                                     const float* __restrict__ kw, float eps, T* __restrict__ q_out,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool, const int* __restrict__ block_table,
                                     int max_blocks, const int* __restrict__ seq_of_token,
                                     const int* __restrict__ positions, int page_size, int H, int G, int D, int V, int write,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                                     int interleaved, const float* __restrict__ qb, const float* __restrict__ kb,
                                     const float* __restrict__ vb) {
  const int n = blockIdx.x;
  const int req = seq_of_token[n];
  if (req < 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int pos = positions[n];
  const int page = block_table[(size_t)req * max_blocks + pos / page_size];
  const int off = pos % page_size;
  for (int head = warp; head < H + G; head += warps) {
    const bool is_q = head < H;
    if (!is_q && !write) continue;
    const TI* src = is_q ? q + (size_t)n * ldq + (size_t)head * D : k + (size_t)n * ldk + (size_t)(head - H) * D;
    const float* w = is_q ? qw : kw;
    const float* bias = is_q ? (qb != nullptr ? qb + (size_t)head * D : nullptr) : (kb != nullptr ? kb + (size_t)(head - H) * D : nullptr);
    auto at = [&](int d) { return bias != nullptr ? to_f32(src[d]) + bias[d] : to_f32(src[d]); };
    float inv = 1.f;
    if (w != nullptr) {
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) { const float x = at(d); ss = fmaf(x, x, ss); }
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / (float)D + eps);
    }
    T* dst = is_q ? q_out + ((size_t)n * H + head) * D
                  : k_pool + (((size_t)page * G + (head - H)) * page_size + off) * D;
    if (cos_t == nullptr) {
      for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(w != nullptr ? at(d) * inv * w[d] : at(d));
      continue;
    }
    const int half = rot / 2;
    for (int i = lane; i < half; i += 32) {
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
      float u = at(a), x = at(b);
      if (w != nullptr) { u *= inv * w[a]; x *= inv * w[b]; }
      const float c = cos_t[(size_t)n * half + i], sn = sin_t[(size_t)n * half + i];
      dst[a] = from_f32<T>(fmaf(u, c, -x * sn));
      dst[b] = from_f32<T>(fmaf(x, c, u * sn));
    }
    for (int d = rot + lane; d < D; d += 32) dst[d] = from_f32<T>(w != nullptr ? at(d) * inv * w[d] : at(d));
  }
  if (write) {
    for (int i = threadIdx.x; i < G * V; i += blockDim.x) {
      const int g = i / V, j = i % V;
      const float x = to_f32(v[(size_t)n * ldv + i]);
      v_pool[(((size_t)page * G + g) * page_size + off) * V + j] = from_f32<T>(vb != nullptr ? x + vb[i] : x);
    }
  }
}

// Scores of one key row against `heads` query rows in shared memory: the row is read once, 16 bytes at a time where
// its size allows, and every head's sum is one ascending chain of fused multiply-adds.
template <typename T>
__device__ __forceinline__ void dot_rows(const T* __restrict__ krow, const float* __restrict__ qs, int D, int heads,
                                         float (&acc)[kMaxGroup]) {
  constexpr int N = Vec<T>::N;
#pragma unroll
  for (int a = 0; a < kMaxGroup; ++a) acc[a] = 0.f;
  int d = 0;
  if ((D * (int)sizeof(T)) % 16 == 0) {
    for (; d + N <= D; d += N) {
      float kv[N];
      load_vec(krow + d, kv);
#pragma unroll
      for (int a = 0; a < kMaxGroup; ++a) {
        if (a < heads) {
#pragma unroll
          for (int e = 0; e < N; ++e) acc[a] = fmaf(qs[a * D + d + e], kv[e], acc[a]);
        }
      }
    }
  }
  for (; d < D; ++d) {
    const float kv = to_f32(krow[d]);
#pragma unroll
    for (int a = 0; a < kMaxGroup; ++a)
      if (a < heads) acc[a] = fmaf(qs[a * D + d], kv, acc[a]);
  }
}

// One block of kTile threads per (token, key/value head). In a tile, thread t owns key t: it computes the scores
// of its key for the group's heads (the key row is read once), the block finds the tile's maxima, and then thread
// c owns value channel c (c, c + kTile, ...) and adds the tile's weighted values to its running sums.
template <typename T, typename TG>
__global__ void __launch_bounds__(kTile)
attention_general_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_of_token,
                         const int* __restrict__ positions, T* __restrict__ out, float scale, int window, int keep_first,
                         float cap, const float* __restrict__ r1, const float* __restrict__ r2, int sink,
                         const TG* __restrict__ gate, long long ldg, int page_size, int H, int G, int D, int V, int row_words,
                         const float* __restrict__ sinks, float out_scale, long long ldo, long long vpitch, int gate_channels) {
  extern __shared__ __align__(16) float smem[];
  const int n = blockIdx.x, g = blockIdx.y;
  const int req = seq_of_token[n];
  if (req < 0) return;
  const int group = H / G;
  const int pos = positions[n];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;  // first key of the window
  const int kept = window > 0 ? min(keep_first, lo) : 0;      // keys [0, kept) stay visible behind it
  const int* table = block_table + (size_t)req * max_blocks;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  for (int h0 = 0; h0 < group; h0 += kMaxGroup) {
    const int heads = min(kMaxGroup, group - h0);
    float* qs = smem;                        // [heads][D]
    float* pw = qs + kMaxGroup * D;          // [heads][kTile] weights of the tile
    float* red = pw + kMaxGroup * kTile;     // [kMaxGroup][4] maxima / sums of the warps
    float* stat = red + kMaxGroup * 4;       // [kMaxGroup][2]: running maximum, correction of this tile
    long long* rowbase = reinterpret_cast<long long*>(smem + row_words);  // [kTile] row of each key of the tile in the pools
    __syncthreads();
    for (int i = tid; i < heads * D; i += kTile)
      qs[i] = to_f32(q[((size_t)n * H + (size_t)g * group + h0) * D + i]);
    float m_run[kMaxGroup], l_run[kMaxGroup];
#pragma unroll
    for (int a = 0; a < kMaxGroup; ++a) {
      m_run[a] = sinks != nullptr ? sinks[g * group + h0 + min(a, heads - 1)] : sink ? 0.f : -INFINITY;
      l_run[a] = sinks != nullptr || sink ? 1.f : 0.f;
    }
    // running sums of value channel c = tid + kTile * i for every head: kept in shared memory (any V), thread-private
    float* acc = stat + kMaxGroup * 2;  // [kMaxGroup][Vp], Vp = V rounded up to kTile
    const int Vp = (V + kTile - 1) / kTile * kTile;
    for (int i = tid; i < heads * Vp; i += kTile) acc[i] = 0.f;
    __syncthreads();

    // the two runs of visible keys: [0, kept) and [lo, pos]; tiles start at multiples of kTile
    for (int run = 0; run < 2; ++run) {
      const int first = run == 0 ? 0 : lo, last = run == 0 ? kept : pos + 1;  // [first, last)
      if (first >= last) continue;
      for (int t0 = first / kTile * kTile; t0 < last; t0 += kTile) {
        const int key = t0 + tid;
        const bool seen = key >= first && key < last;
        float sc[kMaxGroup];
        if (seen) {
          const int page = table[key / page_size];
          const long long base = ((long long)page * G + g) * page_size + key % page_size;
          rowbase[tid] = base;
          const float dist = (float)(pos - key);
          dot_rows(k_pool + (size_t)base * D, qs, D, heads, sc);
#pragma unroll
          for (int a = 0; a < kMaxGroup; ++a) {
            if (a < heads) {
              float s = sc[a] * scale;
              if (cap > 0.f) s = cap * tanhf(s / cap);
              if (r1 != nullptr) {
                const int h = g * group + h0 + a;
                s -= r1[h] * log1pf(r2[h] * dist);
              }
              sc[a] = s;
            }
          }
        }
        // maxima of the tile, per head
#pragma unroll
        for (int a = 0; a < kMaxGroup; ++a) {
          if (a < heads) {
            const float mx = warp_max(seen ? sc[a] : -INFINITY);
            if (lane == 0) red[a * 4 + warp] = mx;
          }
        }
        __syncthreads();
#pragma unroll
        for (int a = 0; a < kMaxGroup; ++a) {
          if (a < heads) {
            const float tile_max = fmaxf(fmaxf(red[a * 4], red[a * 4 + 1]), fmaxf(red[a * 4 + 2], red[a * 4 + 3]));
            const float m_new = fmaxf(m_run[a], tile_max);
            const float corr = m_run[a] == -INFINITY ? 0.f : expf(m_run[a] - m_new);
            const float p = seen ? expf(sc[a] - m_new) : 0.f;
            pw[a * kTile + tid] = p;
            m_run[a] = m_new;
            l_run[a] *= corr;
            if (tid == 0) stat[a * 2 + 1] = corr;
            sc[a] = p;
          }
        }
        __syncthreads();  // weights written, maxima read
        // sums of the weights: every thread adds the tile's weights in the same order, so all agree
#pragma unroll
        for (int a = 0; a < kMaxGroup; ++a) {
          if (a < heads) {
            const float part = warp_sum(sc[a]);
            if (lane == 0) red[a * 4 + warp] = part;
          }
        }
        // weighted values: thread c walks the tile's keys
        const int count = min(kTile, last - t0);
        const int begin = max(0, first - t0);
        for (int c = tid; c < V; c += kTile) {
          float add[kMaxGroup];
#pragma unroll
          for (int a = 0; a < kMaxGroup; ++a) add[a] = 0.f;
#pragma unroll 8
          for (int t = begin; t < count; ++t) {  // (the rows' places were found with the scores: these loads do not wait on one another)
            const float vv = to_f32(v_pool[(size_t)rowbase[t] * vpitch + c]);
#pragma unroll
            for (int a = 0; a < kMaxGroup; ++a)
              if (a < heads) add[a] = fmaf(pw[a * kTile + t], vv, add[a]);
          }
#pragma unroll
          for (int a = 0; a < kMaxGroup; ++a)
            if (a < heads) acc[a * Vp + c] = fmaf(acc[a * Vp + c], stat[a * 2 + 1], add[a]);
        }
        __syncthreads();  // sums of the warps written; weights and corrections read
#pragma unroll
        for (int a = 0; a < kMaxGroup; ++a)
          if (a < heads) l_run[a] += (red[a * 4] + red[a * 4 + 1]) + (red[a * 4 + 2] + red[a * 4 + 3]);
        __syncthreads();
      }
    }
    for (int c = tid; c < V; c += kTile) {
#pragma unroll
      for (int a = 0; a < kMaxGroup; ++a) {
        if (a < heads) {
          const int h = g * group + h0 + a;
          float o = l_run[a] > 0.f ? acc[a * Vp + c] / l_run[a] : 0.f;
          // one logit per head, or (gate_channels) one per channel of the token's output row
          if (gate != nullptr) o *= 1.f / (1.f + expf(-to_f32(gate[(size_t)n * ldg + (gate_channels ? (size_t)h * V + c : (size_t)h)])));
          out[(size_t)n * ldo + (size_t)h * V + c] = from_f32<T>(o * out_scale);
        }
      }
    }
  }
}

}  // namespace

AKAS_API int akas_qk_norm_store(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                                const float* qw, const float* kw, float eps, void* q_out, void* k_pool, void* v_pool,
                                const int* block_table, int max_blocks, const int* seq_of_token, const int* positions,
                                int page_size, int N, int H, int G, int D, int V, int write, int dtype, const float* cos_t,
                                const float* sin_t, int rot, int interleaved, int in_dtype, const float* qb, const float* kb,
                                const float* vb, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (cos_t != nullptr && (rot <= 0 || rot % 2 || rot > D)) return (int)cudaErrorInvalidValue;
  if (dtype == AKAS_F32 && in_dtype != AKAS_F32) return (int)cudaErrorInvalidValue;
  if (dtype == AKAS_F32)
    return launch_ordinary(qk_norm_store_kernel<float, float>, dim3(N), dim3(128), 0, stream, (const float*)q, ldq, (const float*)k, ldk,
                          (const float*)v, ldv, qw, kw, eps, (float*)q_out, (float*)k_pool, (float*)v_pool, block_table,
                          max_blocks, seq_of_token, positions, page_size, H, G, D, V, write, cos_t, sin_t, rot, interleaved, qb, kb, vb);
  if (in_dtype == AKAS_F32)
    return launch_ordinary(qk_norm_store_kernel<float, bf16>, dim3(N), dim3(128), 0, stream, (const float*)q, ldq, (const float*)k, ldk,
                          (const float*)v, ldv, qw, kw, eps, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, block_table, max_blocks,
                          seq_of_token, positions, page_size, H, G, D, V, write, cos_t, sin_t, rot, interleaved, qb, kb, vb);
  return launch_ordinary(qk_norm_store_kernel<bf16, bf16>, dim3(N), dim3(128), 0, stream, (const bf16*)q, ldq, (const bf16*)k, ldk,
                        (const bf16*)v, ldv, qw, kw, eps, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, block_table, max_blocks,
                        seq_of_token, positions, page_size, H, G, D, V, write, cos_t, sin_t, rot, interleaved, qb, kb, vb);
}

template <typename T, typename TG>
static int launch_general(const void* q, const void* k_pool, const void* v_pool, const int* block_table, int max_blocks,
                          const int* seq_of_token, const int* positions, void* out, float scale, int window, int keep_first,
                          float cap, const float* r1, const float* r2, int sink, const void* gate, long long ldg,
                          int page_size, int N, int H, int G, int D, int V, const float* sinks, float out_scale,
                          long long ldo, long long vpitch, int gate_channels, cudaStream_t stream) {
  const int Vp = (V + kTile - 1) / kTile * kTile;
  const int row_words = (kMaxGroup * D + kMaxGroup * kTile + kMaxGroup * 4 + kMaxGroup * 2 + kMaxGroup * Vp + 1) / 2 * 2;
  const size_t smem = sizeof(float) * (size_t)row_words + sizeof(long long) * kTile;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  static size_t allowed[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (smem > 48 * 1024 && device < 64 && allowed[device] < smem) {
    const cudaError_t e = cudaFuncSetAttribute(attention_general_kernel<T, TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed[device] = smem;
  }
  return launch_ordinary(attention_general_kernel<T, TG>, dim3(N, G), dim3(kTile), smem, stream, (const T*)q, (const T*)k_pool,
                        (const T*)v_pool, block_table, max_blocks, seq_of_token, positions, (T*)out, scale, window, keep_first,
                        cap, r1, r2, sink, (const TG*)gate, ldg, page_size, H, G, D, V, row_words, sinks, out_scale, ldo, vpitch, gate_channels);
}

AKAS_API int akas_attention_general(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                    int max_blocks, const int* seq_of_token, const int* positions, void* out, float scale,
                                    int window, int keep_first, float cap, const float* r1, const float* r2, int sink,
                                    const void* gate, long long ldg, int page_size, int N, int H, int G, int D, int V,
                                    int dtype, const float* sinks, float out_scale, long long ldo, long long vpitch,
                                    int gate_channels, int gate_dtype, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (G <= 0 || H % G || vpitch < V) return (int)cudaErrorInvalidValue;
  if (dtype == AKAS_BF16 && gate != nullptr && gate_dtype == AKAS_F32)  // the gate's logits as a float32 product left them
    return launch_general<bf16, float>(q, k_pool, v_pool, block_table, max_blocks, seq_of_token, positions, out, scale, window,
                                       keep_first, cap, r1, r2, sink, gate, ldg, page_size, N, H, G, D, V, sinks, out_scale, ldo, vpitch, gate_channels, stream);
  if (dtype == AKAS_F32 && gate != nullptr && gate_dtype != AKAS_F32) return (int)cudaErrorInvalidValue;
  if (dtype == AKAS_F32)
    return launch_general<float, float>(q, k_pool, v_pool, block_table, max_blocks, seq_of_token, positions, out, scale, window,
                                        keep_first, cap, r1, r2, sink, gate, ldg, page_size, N, H, G, D, V, sinks, out_scale, ldo, vpitch, gate_channels, stream);
  return launch_general<bf16, bf16>(q, k_pool, v_pool, block_table, max_blocks, seq_of_token, positions, out, scale, window,
                                    keep_first, cap, r1, r2, sink, gate, ldg, page_size, N, H, G, D, V, sinks, out_scale, ldo, vpitch, gate_channels, stream);
}
