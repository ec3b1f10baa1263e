// Sliding-window attention over the paged cache with optional extras, SIMT version (float32 arithmetic
// throughout; the cache, q and out are float32 or bfloat16).
//
// Token t of request r at position p reads the keys [p - window + 1, p] of r's pages (window 0: [0, p]) and,
// when the layer keeps pooled blocks, one key and one value per block of `pool` tokens that lies wholly before
// the window (block b holds positions b*pool .. b*pool + pool - 1 and is read when b*pool + pool - 1 <= p -
// window).  Tokens and blocks share one softmax.  Per (query head h, key j):
//   s = (q_h . k_j) * scale
//   s = cap * tanh(s / cap)                         (cap > 0)
//   s += dist_bias[(p - j) * nq + h]                (dist_bias not null: a learned bias by distance, one row per
//                                                    distance below the window; tokens only)
//   w_h(j) = exp(s) / (sum_j' exp(s_j') + exp(sink_h))      (sink not null: a term of the denominator that has no
//                                                            key and no value)
// Without `talk`: out_h = sum_j w_h(j) v_kv(h)(j).  With `talk` [nq, nq]: the heads' weights are mixed after the
// softmax, w'_h(j) = sum_g talk[h, g] w_g(j), and head h applies w'_h to the values of its own kv head.  That is
// computed as out_h = sum_g talk[h, g] O[g][kv(h)] with O[g][m] = sum_j w_g(j) v_m(j): every head's weights are
// applied to the values of ALL kv heads (float32 scratch [T, nq, nkv, vd]) and a second kernel mixes.
//
// One warp per (token, q head): lanes own keys for the scores, then own dims for P V.
#include "common.cuh"

constexpr int WA_WARPS = 4;
constexpr int WA_MAX_HD = 256;

template <typename A> struct WaVec;
template <> struct WaVec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct WaVec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

struct WaParams {
  const int* tok_pos;
  const int* tok_req;
  const int* block_table;      // token pages of the step's requests
  int bt_stride;
  const int* pool_table;       // pages of the pooled rows (null: no pooled blocks)
  int pool_stride;
  int T, nq, nkv, hd, vd, page_size, num_pages, num_pool_pages;
  float scale, cap;
  int window, pool;
  const float* dist_bias;      // [window, nq] or null
  const float* sink;           // [nq] or null
  int all_values;              // 1: every head's weights on the values of all kv heads (scratch), 0: its own
  int vec;
  int* status;
};

// NV: value chunks of 32 a lane holds, ceil(vd / 32)
template <typename A, int NV>
__global__ void __launch_bounds__(WA_WARPS * 32)
window_attention_kernel(const A* __restrict__ q, const A* __restrict__ k_cache, const A* __restrict__ v_cache,
                        const A* __restrict__ kp_cache, const A* __restrict__ vp_cache, A* __restrict__ out,
                        float* __restrict__ scratch, const WaParams P) {
  extern __shared__ float wa_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long wid = (long)blockIdx.x * WA_WARPS + warp;
  if (wid >= (long)P.T * P.nq) return;
  const int t = (int)(wid / P.nq), h = (int)(wid % P.nq);
  const int nq = P.nq, nkv = P.nkv, hd = P.hd, vd = P.vd, ps = P.page_size;
  const int kvh = h / (nq / nkv);
  const int GV = P.all_values ? nkv : 1;
  float* qs = wa_smem + (size_t)warp * (hd + (P.all_values ? nkv * vd : 0));
  float* acc_sm = qs + hd;                                 // [nkv][vd], this warp's, when all_values
  const A* qrow = q + ((size_t)t * nq + h) * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = qb_to_float<A>(qrow[d]);
  if (P.all_values)
    for (int i = lane; i < nkv * vd; i += 32) acc_sm[i] = 0.f;
  __syncwarp();

  const int pos = P.tok_pos[t];
  const int req = P.tok_req[t];
  const int* bt = P.block_table + (size_t)req * P.bt_stride;
  const int* pt = P.pool_table ? P.pool_table + (size_t)req * P.pool_stride : nullptr;
  const int lo = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
  // pooled blocks that lie wholly before the window: b * pool + pool - 1 <= pos - window
  const int n_blocks = (pt != nullptr && P.window > 0 && pos - P.window + 1 >= P.pool) ? (pos - P.window + 1) / P.pool : 0;
  const int n_keys = n_blocks + (pos - lo + 1);

  float m = -INFINITY, l = 0.f;
  float acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;

  for (int k0 = 0; k0 < n_keys; k0 += 32) {
    const int idx = k0 + lane;
    float s = -INFINITY;
    long base = -1;       // row of this lane's key among all (page, kv head 0, slot) rows; + m * page_size for kv head m
    int pooled = 0;
    if (idx < n_keys) {
      pooled = idx < n_blocks;
      const int row = pooled ? idx : lo + (idx - n_blocks);       // pooled row or token position
      const int page = pooled ? pt[row / ps] : bt[row / ps];
      if (page < 0 || page >= (pooled ? P.num_pool_pages : P.num_pages)) {
        qb_set_status(P.status, QB_STATUS_BAD_PAGE, page, 3);
      } else {
        base = ((long)page * nkv) * ps + row % ps;
        const A* kp = (pooled ? kp_cache : k_cache) + (base + (long)kvh * ps) * hd;
        float dot = 0.f;
        if (P.vec) {
          for (int d = 0; d < hd; d += WaVec<A>::N) {
            float kv[WaVec<A>::N];
            WaVec<A>::load(kp + d, kv);
#pragma unroll
            for (int i = 0; i < WaVec<A>::N; ++i) dot += qs[d + i] * kv[i];
          }
        } else {
          for (int d = 0; d < hd; ++d) dot += qs[d] * qb_to_float<A>(kp[d]);
        }
        s = dot * P.scale;
        if (P.cap > 0.f) s = P.cap * tanhf(s / P.cap);
        if (P.dist_bias != nullptr && !pooled) s += P.dist_bias[(size_t)(pos - row) * nq + h];
      }
    }
    const float mb = qb_warp_max(s);
    if (mb == -INFINITY) continue;
    const float m_new = fmaxf(m, mb);
    const float p = (base >= 0) ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + qb_warp_sum(p);
    m = m_new;
    const int n_here = min(32, n_keys - k0);
    for (int g = 0; g < GV; ++g) {
      const int vh = P.all_values ? g : kvh;
      if (P.all_values) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int d = lane + 32 * i;
          acc[i] = d < vd ? acc_sm[g * vd + d] : 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[i] *= corr;
      for (int j = 0; j < n_here; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const long bj = __shfl_sync(0xffffffffu, base, j);
        const int pl = __shfl_sync(0xffffffffu, pooled, j);
        if (bj < 0) continue;
        const A* vp = (pl ? vp_cache : v_cache) + (bj + (long)vh * ps) * vd;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int d = lane + 32 * i;
          if (d < vd) acc[i] += pj * qb_to_float<A>(vp[d]);
        }
      }
      if (P.all_values) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int d = lane + 32 * i;
          if (d < vd) acc_sm[g * vd + d] = acc[i];
        }
      }
    }
  }
  float denom = l;
  if (P.sink != nullptr) denom += (m == -INFINITY) ? 1.f : expf(P.sink[h] - m);
  const float inv_l = denom > 0.f ? 1.f / denom : 0.f;
  if (P.all_values) {
    float* srow = scratch + ((size_t)t * nq + h) * nkv * vd;
    for (int i = lane; i < nkv * vd; i += 32) srow[i] = acc_sm[i] * inv_l;
  } else {
    A* orow = out + ((size_t)t * nq + h) * vd;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = lane + 32 * i;
      if (d < vd) orow[d] = qb_from_float<A>(acc[i] * inv_l);
    }
  }
}

// out[t, h, :] = sum_g talk[h, g] * scratch[t, g, kv(h), :], g ascending.  One block per token.
template <typename A>
__global__ void talk_mix_kernel(const float* __restrict__ scratch, const float* __restrict__ talk, A* __restrict__ out,
                                int T, int nq, int nkv, int vd) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const float* srow = scratch + (size_t)t * nq * nkv * vd;
  for (int i = threadIdx.x; i < nq * vd; i += blockDim.x) {
    const int h = i / vd, d = i % vd;
    const int kvh = h / (nq / nkv);
    float v = 0.f;
    for (int g = 0; g < nq; ++g) v = fmaf(talk[h * nq + g], srow[((size_t)g * nkv + kvh) * vd + d], v);
    out[((size_t)t * nq + h) * vd + d] = qb_from_float<A>(v);
  }
}

extern "C" int qb_window_attention(const void* q, int dtype, const void* k_cache, const void* v_cache,
                                   const void* kp_cache, const void* vp_cache, void* out, float* scratch,
                                   const float* talk, const int* tok_pos, const int* tok_req, const int* block_table,
                                   int bt_stride, const int* pool_table, int pool_stride, int T, int nq, int nkv,
                                   int hd, int vd, int page_size, int num_pages, int num_pool_pages, float scale,
                                   float cap, int window, int pool, const float* dist_bias, const float* sink,
                                   int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || vd <= 0 || hd > WA_MAX_HD || vd > WA_MAX_HD || nq % nkv || page_size <= 0) return QB_ERR_UNSUPPORTED;
  if (pool_table != nullptr && (pool <= 0 || window <= 0 || kp_cache == nullptr || vp_cache == nullptr)) return QB_ERR_BAD_ARG;
  if (dist_bias != nullptr && window <= 0) return QB_ERR_BAD_ARG;
  if (talk != nullptr && scratch == nullptr) return QB_ERR_BAD_ARG;
  WaParams P;
  P.tok_pos = tok_pos; P.tok_req = tok_req; P.block_table = block_table; P.bt_stride = bt_stride;
  P.pool_table = pool_table; P.pool_stride = pool_stride;
  P.T = T; P.nq = nq; P.nkv = nkv; P.hd = hd; P.vd = vd; P.page_size = page_size; P.num_pages = num_pages;
  P.num_pool_pages = num_pool_pages; P.scale = scale; P.cap = cap; P.window = window; P.pool = pool;
  P.dist_bias = dist_bias; P.sink = sink; P.all_values = talk != nullptr; P.status = status;
  P.vec = (hd % 8 == 0 && ((uintptr_t)k_cache & 15) == 0 && (kp_cache == nullptr || ((uintptr_t)kp_cache & 15) == 0)) ? 1 : 0;
  const long warps = (long)T * nq;
  const int blocks = (int)((warps + WA_WARPS - 1) / WA_WARPS);
  const size_t smem = (size_t)WA_WARPS * (hd + (P.all_values ? nkv * vd : 0)) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
  const int nv = (vd + 31) / 32;
#define QB_WA_LAUNCH(A, NV)                                                                                      \
  do {                                                                                                           \
    auto kern = window_attention_kernel<A, NV>;                                                                  \
    if (smem > 48 * 1024) {                                                                                      \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
      if (e != cudaSuccess) return (int)e;                                                                       \
    }                                                                                                            \
    kern<<<blocks, WA_WARPS * 32, smem, stream>>>((const A*)q, (const A*)k_cache, (const A*)v_cache,             \
                                                  (const A*)kp_cache, (const A*)vp_cache, (A*)out, scratch, P);  \
  } while (0)
  QB_DISPATCH_DTYPE(dtype, A, {
    if (nv <= 1) QB_WA_LAUNCH(A, 1);
    else if (nv <= 2) QB_WA_LAUNCH(A, 2);
    else if (nv <= 4) QB_WA_LAUNCH(A, 4);
    else QB_WA_LAUNCH(A, 8);
  });
#undef QB_WA_LAUNCH
  QB_LAUNCH_CHECK();
  if (talk != nullptr) {
    QB_DISPATCH_DTYPE(dtype, A, talk_mix_kernel<A><<<T, 256, 0, stream>>>(scratch, talk, (A*)out, T, nq, nkv, vd));
    QB_LAUNCH_CHECK();
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Pooled blocks: a token whose position ends a block of `pool` tokens (pos % pool == pool - 1) leaves the mean of
// the block's keys and the mean of its values, as the cache holds them, in row pos / pool of the pooled pages.
// The block's earlier tokens may have come in earlier steps: they are read from the pages.  One block per token;
// sums in position order, float32.
// ---------------------------------------------------------------------------------------------
template <typename A>
__global__ void pool_blocks_kernel(const A* __restrict__ k_cache, const A* __restrict__ v_cache,
                                   A* __restrict__ kp_cache, A* __restrict__ vp_cache, const int* __restrict__ tok_pos,
                                   const int* __restrict__ tok_req, const int* __restrict__ block_table, int bt_stride,
                                   const int* __restrict__ pool_table, int pool_stride, int T, int nkv, int hd, int vd,
                                   int page_size, int num_pages, int num_pool_pages, int pool, int* status) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const int pos = tok_pos[t];
  if (pos % pool != pool - 1) return;
  const int b = pos / pool, req = tok_req[t];
  const int* bt = block_table + (size_t)req * bt_stride;
  const int dst_page = pool_table[(size_t)req * pool_stride + b / page_size];
  if (dst_page < 0 || dst_page >= num_pool_pages) {
    if (threadIdx.x == 0) qb_set_status(status, QB_STATUS_BAD_PAGE, dst_page, 2);
    return;
  }
  const float inv = 1.f / (float)pool;
  const int kn = nkv * hd, vn = nkv * vd;
  for (int i = threadIdx.x; i < kn + vn; i += blockDim.x) {
    const bool is_k = i < kn;
    const int j = is_k ? i : i - kn, w = is_k ? hd : vd;
    const int head = j / w, d = j % w;
    const A* src = is_k ? k_cache : v_cache;
    float sum = 0.f;
    for (int p = pos - pool + 1; p <= pos; ++p) {
      const int page = bt[p / page_size];
      if (page < 0 || page >= num_pages) { qb_set_status(status, QB_STATUS_BAD_PAGE, page, 2); continue; }
      sum += qb_to_float<A>(src[(((size_t)page * nkv + head) * page_size + p % page_size) * w + d]);
    }
    A* dst = is_k ? kp_cache : vp_cache;
    dst[(((size_t)dst_page * nkv + head) * page_size + b % page_size) * w + d] = qb_from_float<A>(sum * inv);
  }
}

extern "C" int qb_pool_blocks(const void* k_cache, const void* v_cache, void* kp_cache, void* vp_cache, int dtype,
                              const int* tok_pos, const int* tok_req, const int* block_table, int bt_stride,
                              const int* pool_table, int pool_stride, int T, int nkv, int hd, int vd, int page_size,
                              int num_pages, int num_pool_pages, int pool, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (pool <= 0 || page_size <= 0 || nkv <= 0 || hd <= 0 || vd <= 0) return QB_ERR_BAD_ARG;
  QB_DISPATCH_DTYPE(dtype, A, pool_blocks_kernel<A><<<T, 128, 0, stream>>>(
      (const A*)k_cache, (const A*)v_cache, (A*)kp_cache, (A*)vp_cache, tok_pos, tok_req, block_table, bt_stride,
      pool_table, pool_stride, T, nkv, hd, vd, page_size, num_pages, num_pool_pages, pool, status));
  QB_LAUNCH_CHECK();
  return 0;
}
