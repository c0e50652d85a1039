// The general attention (see attention_general.cu for what it computes) for prompt portions in bfloat16 on the
// tensor cores, flash-attention style: the walk of attention_prefill.cu with the options as arguments.
//
// One block per (tile of 64 consecutive query tokens of one request, query head); 4 warps of 16 query rows. The block
// walks 64-key tiles aligned to absolute position 0: first the tiles of the kept first tokens that lie before its
// window, then from the first key its window reaches to its last query's own position. K rows [DK] and V rows [DV]
// come from the pages by 16-byte cp.async copies, two tiles in flight; columns beyond the real head sizes (which need
// only be multiples of 8) are zero in shared memory. S = Q.K^T and O += P.V are mma.sync m16n8k16; between them, in
// float32 registers: scale, cap * tanh(s / cap), minus r1 * ln(1 + r2 * distance), the mask by absolute positions,
// and the running maximum and sum, which start at the sink's logit (0, or a learned number per head) and 1 where the
// softmax has a sink. The head's output is multiplied by sigmoid(gate) and by a constant on its way out, into rows
// whose pitch is the caller's.
//
// Packed launches serve steps of single tokens (decoding): a block's rows are then the query heads that share one
// key/value head, all at the token's position, so its keys and values are read once for the whole group; warps
// without a live row only help with the copies. A packed launch may cut every request's key tiles into `splits`
// parts (gridDim.z): a block then walks its part only and leaves its unnormalised sums, its maximum and its sum of
// weights in a scratch buffer, and general_merge_kernel adds the parts (and the sink's term, once) in the order of
// their numbers: a decode step of a few requests with thousands of keys each fills the GPU that way.
#include <math.h>

#include "common.cuh"
#include "mma.cuh"

using namespace akas;

namespace {

constexpr int BQ = 64, BK = 64, WARPS = 4;
constexpr float kLog2e = 1.4426950408889634f;

// tanh(x) = 1 - 2 / (e^(2x) + 1) from the special-function unit's exp2 and reciprocal: an absolute error of a few
// 1e-7. (tanh.approx.f32 is good to about 5e-4 only, which the cap in front of it, often 20 to 50, would turn into
// errors of the scores as large as the rounding of bfloat16.)
__device__ __forceinline__ float fast_tanh(float x) {
  const float e = fast_exp2(fminf(x * (2.f * kLog2e), 80.f));
  return 1.f - __fdividef(2.f, e + 1.f);
}
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Options {
  float scale, cap;
  const float* r1;
  const float* r2;
  int window, keep_first, sink;
  const void* gate;    // logits of the output gate, bfloat16 or (gate_f32) float32, or null
  long long ldg;
  const float* sinks;  // a learned sink logit per head, or null
  float out_scale;
  long long ldo;       // elements between the output rows of two tokens
  long long vpitch;    // elements between two value rows in the pages (V, or more where a row holds more than the value)
  int gate_channels;   // the gate has one logit per output channel [H * V] of a token, not one per head [H]
  int gate_f32;        // the gate's logits are float32 (the rows of a product that left float32)
};

__device__ __forceinline__ float gate_at(const Options& opt, size_t at) {  // sigmoid of the logit at an element offset
  const float z = opt.gate_f32 ? reinterpret_cast<const float*>(opt.gate)[at] : to_f32(reinterpret_cast<const bf16*>(opt.gate)[at]);
  return 1.f / (1.f + __expf(-z));
}

__device__ __forceinline__ float gate_of(const Options& opt, size_t token, int head, int V, int c) {
  return gate_at(opt, token * opt.ldg + (size_t)head * V + c);
}

constexpr int kTableBefore = 128, kTableAfter = 192;  // entries of the penalty table on either side of the window's distances

template <int DKP, int DVP>  // head sizes rounded up to multiples of 32
__global__ void __launch_bounds__(WARPS * 32, (DKP + DVP <= 192) ? 3 : 2)
general_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                       const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ positions, bf16* __restrict__ out, Options opt, int page_size, int H, int KH,
                       int D, int V, int R, int packed, int table, float* __restrict__ partial, int splits) {
  constexpr int KSTRIDE = DKP + 8, VSTRIDE = DVP + 8;  // 16 bytes of padding keep ldmatrix conflict-free
  constexpr int KCH = DKP / 8, VCH = DVP / 8;          // 16-byte chunks per row
  constexpr int KS = DKP / 16;                         // k-steps of Q.K^T
  constexpr int NB = DVP / 8;                          // 8-wide output blocks of P.V
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* k_s = reinterpret_cast<bf16*>(smem_raw);  // [2][BK][KSTRIDE]; stage 0 first holds Q
  bf16* v_s = k_s + 2 * BK * KSTRIDE;             // [2][BK][VSTRIDE]
  // [table + kTableBefore + kTableAfter] the head's distance penalty r1 lg2(1 + r2 d), made once by the block, for
  // every distance that a tile without kept first tokens can hold: d from -126 (a key ahead of the query, masked) to
  // window + 125 (a key of the window's first tile that lies before the window, masked). A score then costs a
  // shared-memory read instead of a conversion and a logarithm, and the read needs no bounds.
  float* penalty = reinterpret_cast<float*>(v_s + 2 * BK * VSTRIDE) + kTableBefore;

  int tile = (int)gridDim.y - 1 - (int)blockIdx.y, r = 0, n = 0;  // long walks first
  for (; r < R; ++r) {
    n = cu_seqlens[r + 1] - cu_seqlens[r];
    const int tiles = (n + BQ - 1) / BQ;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (r >= R) return;
  const int group = H / KH;
  const int kvh = packed ? blockIdx.x : blockIdx.x / group;
  const int q0 = cu_seqlens[r] + tile * BQ;
  const int rows = packed ? group : min(BQ, n - tile * BQ);  // packed: row i is head kvh * group + i of token q0
  const int pos0 = positions[q0];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int window = opt.window, keep = opt.window > 0 ? opt.keep_first : 0;

  for (int c = tid; c < BQ * KCH; c += WARPS * 32) {
    const int row = c / KCH, col = (c % KCH) * 8;
    const int live = min(row, rows - 1);
    const bf16* src = q + (packed ? (size_t)q0 * H + kvh * group + live : (size_t)(q0 + live) * H + blockIdx.x) * D + min(col, D - 8);
    cp_async16(k_s + row * KSTRIDE + col, src, row < rows && col < D ? 16 : 0);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
    ldmatrix_x4(qf[ks], k_s + (warp * 16 + (lane & 15)) * KSTRIDE + ks * 16 + (lane >> 4) * 8);
  __syncthreads();

  const int last_key = packed ? pos0 : pos0 + rows - 1;
  const bool active = warp * 16 < rows;  // a warp without live rows copies tiles and computes nothing
  const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kt0 = first_key / BK, kt1 = last_key / BK;
  const int kept_tiles = min((keep + BK - 1) / BK, kt0);  // tiles of kept tokens that lie wholly before the window's first
  const int total = kept_tiles + (kt1 - kt0 + 1);
  int i_begin = 0, i_end = total;  // the tiles this block walks: all, or its part of them
  if (splits > 1) {
    const int per = (total + splits - 1) / splits;
    i_begin = min(total, (int)blockIdx.z * per);
    i_end = min(total, i_begin + per);
  }
  auto tile_of = [&](int i) { return i < kept_tiles ? i : kt0 + (i - kept_tiles); };

  auto load_tile = [&](int kt, int stage) {
    bf16* ks_ = k_s + stage * BK * KSTRIDE;
    bf16* vs_ = v_s + stage * BK * VSTRIDE;
    for (int c = tid; c < BK * (KCH + VCH); c += WARPS * 32) {
      const int row = c / (KCH + VCH), ch = c % (KCH + VCH);
      const int key = kt * BK + row;
      int page = -1;
      if (key <= last_key && (key >= first_key || key < keep)) page = block_table[(size_t)r * max_blocks + key / page_size];
      const size_t base = page >= 0 ? ((size_t)page * KH + kvh) * page_size + key % page_size : 0;
      if (ch < KCH) {
        const int col = ch * 8;
        cp_async16(ks_ + row * KSTRIDE + col, k_pool + base * D + min(col, D - 8), page >= 0 && col < D ? 16 : 0);
      } else {
        const int col = (ch - KCH) * 8;
        cp_async16(vs_ + row * VSTRIDE + col, v_pool + base * opt.vpitch + min(col, V - 8), page >= 0 && col < V ? 16 : 0);
      }
    }
    cp_async_commit();
  };

  float o[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) { o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f; }
  // running maximum (in units of log2 e) and this thread's share of the running sum; the sink is a term exp(0)
  float m_run[2], l_run[2];
  const int row2[2] = {warp * 16 + g, warp * 16 + g + 8};
  const int qpos[2] = {packed ? pos0 : pos0 + row2[0], packed ? pos0 : pos0 + row2[1]};
  const int head2[2] = {packed ? kvh * group + min(row2[0], rows - 1) : (int)blockIdx.x,
                        packed ? kvh * group + min(row2[1], rows - 1) : (int)blockIdx.x};
  const bool sunk = splits <= 1 && (opt.sink || opt.sinks != nullptr);  // with parts, the merge adds the sink's term
  m_run[0] = !sunk ? -INFINITY : opt.sinks != nullptr ? opt.sinks[head2[0]] * kLog2e : 0.f;
  m_run[1] = !sunk ? -INFINITY : opt.sinks != nullptr ? opt.sinks[head2[1]] * kLog2e : 0.f;
  l_run[0] = l_run[1] = sunk && t == 0 ? 1.f : 0.f;
  const bool biased = opt.r1 != nullptr;
  // r1 ln(1 + r2 d) in units of log2 e is r1 lg2(1 + r2 d): the two factors ln 2 and log2 e cancel
  const float r1[2] = {biased ? opt.r1[head2[0]] : 0.f, biased ? opt.r1[head2[1]] : 0.f};
  const float r2[2] = {biased ? opt.r2[head2[0]] : 0.f, biased ? opt.r2[head2[1]] : 0.f};
  const float inv_cap = opt.cap > 0.f ? 1.f / opt.cap : 0.f;
  const float cap2 = opt.cap * kLog2e, scale2 = opt.scale * kLog2e;

  if (i_begin < i_end) load_tile(tile_of(i_begin), 0);
  if (table > 0) {
    for (int d = tid - kTableBefore; d < table + kTableAfter; d += WARPS * 32)
      penalty[d] = d > 0 ? r1[0] * fast_log2(fmaf(r2[0], (float)d, 1.f)) : 0.f;
    __syncthreads();
  }
  const int wlimit = window > 0 ? window : 0x7fffffff;
  const float scale_cap = opt.scale * inv_cap;
  for (int i = i_begin; i < i_end; ++i) {
    const int kt = tile_of(i);
    const int stage = (i - i_begin) & 1;
    if (i + 1 < i_end) {
      load_tile(tile_of(i + 1), stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* ks_ = k_s + stage * BK * KSTRIDE;
    const bf16* vs_ = v_s + stage * BK * VSTRIDE;
    if (!active) {
      __syncthreads();
      continue;
    }

    float s[BK / 8][4];
#pragma unroll
    for (int nb = 0; nb < BK / 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < BK / 16; ++np) {
        uint32_t b[4];
        ldmatrix_x4(b, ks_ + (np * 16 + (lane & 7) + (lane >> 4) * 8) * KSTRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
      }
    }

    float m_new[2] = {m_run[0], m_run[1]};
    // A tile without kept first tokens (all but a request's first few): a key is seen iff 0 <= distance < window, and
    // the penalty of every distance in it is in the table (where there is a penalty, there must be a table).
    const bool fast = kt * BK >= keep && (!biased || table > 0);
    if (fast) {
      const int dbase[2] = {qpos[0] - (kt * BK + 2 * t), qpos[1] - (kt * BK + 2 * t)};
#pragma unroll
      for (int nb = 0; nb < BK / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int dist = dbase[e >> 1] - (nb * 8 + (e & 1));
          float x = opt.cap > 0.f ? cap2 * fast_tanh(s[nb][e] * scale_cap) : s[nb][e] * scale2;
          if (biased) x -= penalty[dist];
          s[nb][e] = (unsigned)dist < (unsigned)wlimit ? x : -INFINITY;
          m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nb][e]);
        }
      }
    } else {
#pragma unroll
      for (int nb = 0; nb < BK / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kt * BK + nb * 8 + 2 * t + (e & 1);
          const int qp = qpos[e >> 1];
          const bool seen = key <= qp && (window <= 0 || key > qp - window || key < keep);
          float x = opt.cap > 0.f ? cap2 * fast_tanh(s[nb][e] * scale_cap) : s[nb][e] * scale2;
          if (biased) x -= r1[e >> 1] * fast_log2(fmaf(r2[e >> 1], (float)max(qp - key, 0), 1.f));
          s[nb][e] = seen ? x : -INFINITY;
          m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nb][e]);
        }
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      m_new[h2] = fmaxf(m_new[h2], __shfl_xor_sync(0xffffffffu, m_new[h2], 1));
      m_new[h2] = fmaxf(m_new[h2], __shfl_xor_sync(0xffffffffu, m_new[h2], 2));
      m_use[h2] = m_new[h2] == -INFINITY ? 0.f : m_new[h2];
      corr[h2] = fast_exp2(m_run[h2] - m_use[h2]);
      m_run[h2] = m_new[h2];
    }
    float l_add[2] = {0.f, 0.f};
    uint32_t pf[BK / 16][4];
#pragma unroll
    for (int nb = 0; nb < BK / 8; ++nb) {
      const float p0 = fast_exp2(s[nb][0] - m_use[0]), p1 = fast_exp2(s[nb][1] - m_use[0]);
      const float p2 = fast_exp2(s[nb][2] - m_use[1]), p3 = fast_exp2(s[nb][3] - m_use[1]);
      l_add[0] += p0 + p1;
      l_add[1] += p2 + p3;
      pf[nb >> 1][(nb & 1) * 2] = pack_bf16(p0, p1);
      pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) l_run[h2] = l_run[h2] * corr[h2] + l_add[h2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      o[nb][0] *= corr[0]; o[nb][1] *= corr[0];
      o[nb][2] *= corr[1]; o[nb][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < NB / 2; ++np) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vs_ + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VSTRIDE + np * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * np], pf[kk], b[0], b[1]);
        mma_bf16(o[2 * np + 1], pf[kk], b[2], b[3]);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
  }
  if (splits > 1) {
    // this part's sums as they stand, per (token, head, part): V unnormalised channels, the maximum, the sum of weights
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const int row = warp * 16 + g + h2 * 8;
      if (row >= rows) continue;
      float* dst = partial + (((size_t)q0 * H + head2[h2]) * splits + blockIdx.z) * (V + 2);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
        if (nb * 8 + 2 * t < V) {
          dst[nb * 8 + 2 * t] = o[nb][h2 * 2];
          dst[nb * 8 + 2 * t + 1] = o[nb][h2 * 2 + 1];
        }
      if (t == 0) {
        dst[V] = m_run[h2];
        dst[V + 1] = l_run[h2];
      }
    }
    return;
  }
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    const int row = warp * 16 + g + h2 * 8;
    if (row >= rows) continue;
    float inv = l_run[h2] > 0.f ? 1.f / l_run[h2] : 0.f;
    const size_t token = packed ? q0 : q0 + row;
    const bool by_channel = opt.gate != nullptr && opt.gate_channels;
    if (opt.gate != nullptr && !by_channel) inv *= gate_at(opt, token * opt.ldg + head2[h2]);
    inv *= opt.out_scale;
    bf16* dst = out + token * opt.ldo + (size_t)head2[h2] * V;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
      if (nb * 8 + 2 * t < V) {
        float a = o[nb][h2 * 2] * inv, b = o[nb][h2 * 2 + 1] * inv;
        if (by_channel) {
          a *= gate_of(opt, token, head2[h2], V, nb * 8 + 2 * t);
          b *= gate_of(opt, token, head2[h2], V, nb * 8 + 2 * t + 1);
        }
        *reinterpret_cast<uint32_t*>(dst + nb * 8 + 2 * t) = pack_bf16(a, b);
      }
  }
}

// One block per (request of one token, head): the parts' sums, rescaled to the common maximum (the sink's logit
// included) and added in the order of the parts; then the division, the gate and the constant. The first warp reads
// every part's maximum and weight sum at once (two parts a lane) and leaves a factor per part in shared memory.
__global__ void general_merge_kernel(const float* __restrict__ partial, const int* __restrict__ cu_seqlens, bf16* __restrict__ out,
                                     Options opt, int H, int V, int splits) {
  __shared__ float factor[64];
  __shared__ float inv_s;
  const int token = cu_seqlens[blockIdx.x], head = blockIdx.y;
  const float* src = partial + ((size_t)token * H + head) * splits * (V + 2);
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const bool sunk = opt.sink || opt.sinks != nullptr;
    const float sink2 = opt.sinks != nullptr ? opt.sinks[head] * kLog2e : 0.f;
    float m[2], l[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int z = lane + 32 * i;
      m[i] = z < splits ? src[(size_t)z * (V + 2) + V] : -INFINITY;
      l[i] = z < splits ? src[(size_t)z * (V + 2) + V + 1] : 0.f;
    }
    float top = fmaxf(m[0], m[1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    if (sunk) top = fmaxf(top, sink2);
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float f = m[i] == -INFINITY ? 0.f : exp2f(m[i] - top);
      factor[lane + 32 * i] = f;
      part = fmaf(l[i], f, part);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    const float denom = part + (sunk ? exp2f(sink2 - top) : 0.f);
    float inv = denom > 0.f ? opt.out_scale / denom : 0.f;
    if (opt.gate != nullptr && !opt.gate_channels) inv *= gate_at(opt, (size_t)token * opt.ldg + head);
    if (lane == 0) inv_s = inv;
  }
  __syncthreads();
  const float inv = inv_s;
  const bool by_channel = opt.gate != nullptr && opt.gate_channels;
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    float acc = 0.f;
#pragma unroll 8
    for (int z = 0; z < splits; ++z) acc = fmaf(src[(size_t)z * (V + 2) + c], factor[z], acc);
    if (by_channel) acc *= gate_of(opt, (size_t)token, head, V, c);
    out[(size_t)token * opt.ldo + (size_t)head * V + c] = __float2bfloat16_rn(acc * inv);
  }
}

template <int DKP, int DVP>
int launch(const void* q, const void* k_pool, const void* v_pool, const int* block_table, int max_blocks,
           const int* cu_seqlens, const int* positions, void* out, const Options& opt, int page_size, int tiles, int H,
           int KH, int D, int V, int R, int packed, float* partial, int splits, cudaStream_t stream) {
  // the table of distance penalties: for unpacked launches (one head a block) with a window of at most kTableMost keys
  constexpr int kTableMost = 8192;
  const int table = !packed && opt.r1 != nullptr && opt.window > 0 && opt.window <= kTableMost ? opt.window : 0;
  constexpr int tiles_bytes = 2 * BK * ((DKP + 8) + (DVP + 8)) * (int)sizeof(bf16);
  const int smem = tiles_bytes + (table ? table + kTableBefore + kTableAfter : 0) * (int)sizeof(float);
  static bool configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (!configured[device]) {
    const cudaError_t e = cudaFuncSetAttribute(general_prefill_kernel<DKP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               tiles_bytes + (kTableMost + kTableBefore + kTableAfter) * (int)sizeof(float));
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  const int err = launch_ordinary(general_prefill_kernel<DKP, DVP>, dim3(packed ? KH : H, tiles, splits), dim3(WARPS * 32), (size_t)smem,
                                  stream, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, max_blocks,
                                  cu_seqlens, positions, (bf16*)out, opt, page_size, H, KH, D, V, R, packed, table, partial, splits);
  if (err || splits <= 1) return err;
  return launch_ordinary(general_merge_kernel, dim3(R, H), dim3(V >= 128 ? 128 : 64), 0, stream, (const float*)partial, cu_seqlens,
                         (bf16*)out, opt, H, V, splits);
}

}  // namespace

// Whether the kernel takes these head sizes: multiples of 8 up to 128.
AKAS_API int akas_attention_general_tc_takes(int D, int V) { return D % 8 == 0 && V % 8 == 0 && D >= 8 && V >= 8 && D <= 128 && V <= 128; }

// tiles: sum over the requests (R of them, from cu_seqlens[0] on) of ceil(tokens / 64); block_table's row 0 is the
// first of these requests. packed: every one of the R requests brings one token (tiles = R), and the heads of a
// key/value head (at most 64) share a block. 3999: sizes the kernel does not take.
AKAS_API int akas_attention_general_tc(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                       int max_blocks, const int* cu_seqlens, const int* positions, void* out, float scale,
                                       int window, int keep_first, float cap, const float* r1, const float* r2, int sink,
                                       const void* gate, long long ldg, int page_size, int tiles, int H, int KH, int D, int V,
                                       int R, int packed, const float* sinks, float out_scale, long long ldo, float* partial,
                                       int splits, long long vpitch, int gate_channels, int gate_dtype, cudaStream_t stream) {
  if (!akas_attention_general_tc_takes(D, V)) return 3999;
  if (ldo % 2 || vpitch % 8 || vpitch < V) return 3999;
  // parts: packed launches only; partial holds (first token of the launch + R) * H * splits * (V + 2) floats
  if (splits < 1 || splits > 64 || (splits > 1 && (!packed || partial == nullptr))) return (int)cudaErrorInvalidValue;
  if (packed && (KH <= 0 || H / KH > BQ || tiles != R)) return 3999;
  if (KH <= 0 || H % KH || tiles > 65535 || R <= 0) return (int)cudaErrorInvalidValue;
  if (tiles <= 0) return 0;
  const Options opt = {scale, cap, r1, r2, window, keep_first, sink, gate, ldg, sinks, out_scale, ldo, vpitch, gate_channels, gate_dtype == AKAS_F32};
  const int dk = (D + 31) / 32, dv = (V + 31) / 32;
#define AKAS_TC(A, B)                                                                                                   \
  if (dk == A && dv == B)                                                                                               \
    return launch<A * 32, B * 32>(q, k_pool, v_pool, block_table, max_blocks, cu_seqlens, positions, out, opt, page_size, \
                                  tiles, H, KH, D, V, R, packed, partial, splits, stream);
  AKAS_TC(1, 1) AKAS_TC(1, 2) AKAS_TC(1, 3) AKAS_TC(1, 4)
  AKAS_TC(2, 1) AKAS_TC(2, 2) AKAS_TC(2, 3) AKAS_TC(2, 4)
  AKAS_TC(3, 1) AKAS_TC(3, 2) AKAS_TC(3, 3) AKAS_TC(3, 4)
  AKAS_TC(4, 1) AKAS_TC(4, 2) AKAS_TC(4, 3) AKAS_TC(4, 4)
#undef AKAS_TC
  return 3999;
}
