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
// One warp per (token, q head), or per (token, q head, range of the keys) in steps of few tokens, whose ranges a
// second kernel joins: lanes own keys for the scores, then own dims for P V.  Long portions in bfloat16 take the
// tensor-core kernel at the end of this file.
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
  int n_split;                 // > 1 (the ranges kernel): a warp takes one of n_split ranges of the keys and leaves (max,
  float* part;                 // sum, sums of values) in `part` [T, nq, n_split, 2 + (all_values ? nkv : 1) * vd]
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

// NV consecutive elements from an address that is a multiple of NV elements
template <typename A, int NV>
__device__ __forceinline__ void wa_load_run(const A* p, float* o) {
  struct alignas(sizeof(A) * NV) Run { A v[NV]; };
  const Run r = *reinterpret_cast<const Run*>(p);
#pragma unroll
  for (int i = 0; i < NV; ++i) o[i] = qb_to_float<A>(r.v[i]);
}

// Steps of few tokens: a warp takes one of n_split ranges of a token's keys for up to GQ q heads that share a kv
// head: a key row is read once for all of them (lanes own keys), a value row once (lanes own NV neighbouring
// dims).  It leaves (max, sum, sums of values) per head in `part` [T, nq, n_split, 2 + GV * vd] for the join;
// with all_values one warp per kv head whose values the heads' weights are applied to (GV = nkv).
template <typename A, int NV, int GQ>
__global__ void __launch_bounds__(WA_WARPS * 32)
window_attention_ranges_kernel(const A* __restrict__ q, const A* __restrict__ k_cache, const A* __restrict__ v_cache,
                               const A* __restrict__ kp_cache, const A* __restrict__ vp_cache, const WaParams P) {
  extern __shared__ float wa_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nq = P.nq, nkv = P.nkv, hd = P.hd, vd = P.vd, ps = P.page_size;
  const int group = nq / nkv, n_chunks = (group + GQ - 1) / GQ, GV = P.all_values ? nkv : 1;
  long wid = (long)blockIdx.x * WA_WARPS + warp;
  if (wid >= (long)P.T * nkv * n_chunks * P.n_split * GV) return;
  const int vsel = (int)(wid % GV); wid /= GV;
  const int split = (int)(wid % P.n_split); wid /= P.n_split;
  const int chunk = (int)(wid % n_chunks); wid /= n_chunks;
  const int kvh = (int)(wid % nkv);
  const int t = (int)(wid / nkv);
  const int h0 = kvh * group + chunk * GQ;
  const int n_g = min(GQ, group - chunk * GQ);
  const int vh = P.all_values ? vsel : kvh;
  float* qs = wa_smem + (size_t)warp * GQ * hd;
  for (int i = lane; i < GQ * hd; i += 32) {
    const int g = i / hd, d = i % hd;
    qs[i] = g < n_g ? qb_to_float<A>(q[((size_t)t * nq + h0 + g) * hd + d]) : 0.f;
  }
  __syncwarp();

  const int pos = P.tok_pos[t];
  const int req = P.tok_req[t];
  const int* bt = P.block_table + (size_t)req * P.bt_stride;
  const int* pt = P.pool_table ? P.pool_table + (size_t)req * P.pool_stride : nullptr;
  const int lo = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
  const int n_blocks = (pt != nullptr && P.window > 0 && pos - P.window + 1 >= P.pool) ? (pos - P.window + 1) / P.pool : 0;
  const int n_keys = n_blocks + (pos - lo + 1);
  const int per_split = ((n_keys + P.n_split - 1) / P.n_split + 31) / 32 * 32;
  const int k_begin = split * per_split;
  const int k_end = min(n_keys, k_begin + per_split);
  const bool v_runs = vd == 32 * NV;

  float m[GQ], l[GQ], acc[GQ][NV];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[g][i] = 0.f;
  }
  for (int k0 = k_begin; k0 < k_end; k0 += 32) {
    const int idx = k0 + lane;
    float s[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) s[g] = -INFINITY;
    long base = -1;
    int pooled = 0;
    if (idx < k_end) {
      pooled = idx < n_blocks;
      const int row = pooled ? idx : lo + (idx - n_blocks);
      const int page = pooled ? pt[row / ps] : bt[row / ps];
      if (page < 0 || page >= (pooled ? P.num_pool_pages : P.num_pages)) {
        qb_set_status(P.status, QB_STATUS_BAD_PAGE, page, 3);
      } else {
        base = ((long)page * nkv) * ps + row % ps;
        const A* kp = (pooled ? kp_cache : k_cache) + (base + (long)kvh * ps) * hd;
        float dot[GQ];
#pragma unroll
        for (int g = 0; g < GQ; ++g) dot[g] = 0.f;
        if (P.vec) {
          for (int d = 0; d < hd; d += WaVec<A>::N) {
            float kv[WaVec<A>::N];
            WaVec<A>::load(kp + d, kv);
#pragma unroll
            for (int g = 0; g < GQ; ++g)
#pragma unroll
              for (int i = 0; i < WaVec<A>::N; ++i) dot[g] += qs[g * hd + d + i] * kv[i];
          }
        } else {
          for (int d = 0; d < hd; ++d) {
            const float kv = qb_to_float<A>(kp[d]);
#pragma unroll
            for (int g = 0; g < GQ; ++g) dot[g] += qs[g * hd + d] * kv;
          }
        }
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
          float x = dot[g] * P.scale;
          if (P.cap > 0.f) x = P.cap * tanhf(x / P.cap);
          if (P.dist_bias != nullptr && !pooled && g < n_g) x += P.dist_bias[(size_t)(pos - row) * nq + h0 + g];
          s[g] = x;
        }
      }
    }
    if (!__any_sync(0xffffffffu, base >= 0)) continue;
    float p[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      const float m_new = fmaxf(m[g], qb_warp_max(s[g]));
      p[g] = (base >= 0) ? expf(s[g] - m_new) : 0.f;
      const float corr = expf(m[g] - m_new);
      l[g] = l[g] * corr + qb_warp_sum(p[g]);
      m[g] = m_new;
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[g][i] *= corr;
    }
    const int n_here = min(32, k_end - k0);
    // eight value rows are asked for before the first is used: with few warps on the device nothing else hides
    // the time a row takes to arrive
    for (int j0 = 0; j0 < n_here; j0 += 8) {
      float v[8][NV];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const long bj = __shfl_sync(0xffffffffu, base, j0 + u);
        const int pl = __shfl_sync(0xffffffffu, pooled, j0 + u);
        const bool there = j0 + u < n_here && bj >= 0;
        const A* vp = (pl ? vp_cache : v_cache) + (there ? (bj + (long)vh * ps) * vd : 0) + lane * NV;
        if (v_runs) {
          wa_load_run<A, NV>(vp, v[u]);
#pragma unroll
          for (int i = 0; i < NV; ++i) v[u][i] = there ? v[u][i] : 0.f;
        } else {
#pragma unroll
          for (int i = 0; i < NV; ++i) v[u][i] = (there && lane * NV + i < vd) ? qb_to_float<A>(vp[i]) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
          const float pj = __shfl_sync(0xffffffffu, p[g], j0 + u);
#pragma unroll
          for (int i = 0; i < NV; ++i) acc[g][i] = fmaf(pj, v[u][i], acc[g][i]);
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    if (g >= n_g) continue;
    float* prow = P.part + (((size_t)t * nq + h0 + g) * P.n_split + split) * (2 + (size_t)GV * vd);
    if (lane == 0 && vsel == 0) { prow[0] = m[g]; prow[1] = l[g]; }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = lane * NV + i;
      if (d < vd) prow[2 + (size_t)vsel * vd + d] = acc[g][i];
    }
  }
}

// The ranges of a (token, head) joined: with M = max of the ranges' maxima, weight_r = exp(m_r - M) / (sum_r l_r
// exp(m_r - M) + exp(sink - M)); the normed sums of values go to `out` (own kv head) or, when the heads' weights
// are mixed afterwards, to scratch [T, nq, nkv, vd].  One block per (token, head); its shared memory holds the
// ranges' weights; eight ranges are read before the first is used.
template <typename A>
__global__ void __launch_bounds__(128)
wa_merge_kernel(const float* __restrict__ part, const float* __restrict__ sink, A* __restrict__ out,
                float* __restrict__ scratch, int T, int nq, int nkv, int vd, int n_split, int all_values) {
  extern __shared__ float wm_w[];                       // [n_split]
  const int t = blockIdx.x / nq, h = blockIdx.x % nq;
  if (t >= T) return;
  const int GV = all_values ? nkv : 1;
  const size_t stride = 2 + (size_t)GV * vd;
  const float* prow = part + ((size_t)t * nq + h) * n_split * stride;
  for (int r = threadIdx.x; r < n_split; r += blockDim.x) wm_w[r] = prow[r * stride];
  __syncthreads();
  float M = -INFINITY;
  for (int r = 0; r < n_split; ++r) M = fmaxf(M, wm_w[r]);
  __syncthreads();
  for (int r = threadIdx.x; r < n_split; r += blockDim.x) {
    const float mr = prow[r * stride];
    wm_w[r] = mr == -INFINITY ? 0.f : expf(mr - M);
  }
  __syncthreads();
  float denom = 0.f;
  for (int r = 0; r < n_split; ++r) denom = fmaf(prow[r * stride + 1], wm_w[r], denom);
  if (sink != nullptr) denom += (M == -INFINITY) ? 1.f : expf(sink[h] - M);
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  const int n = GV * vd;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = 0.f;
    for (int r0 = 0; r0 < n_split; r0 += 8) {
      float x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) x[u] = r0 + u < n_split ? prow[(size_t)(r0 + u) * stride + 2 + i] : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) v = r0 + u < n_split ? fmaf(wm_w[r0 + u], x[u], v) : v;
    }
    v *= inv;
    if (all_values) scratch[((size_t)t * nq + h) * n + i] = v;
    else out[((size_t)t * nq + h) * n + i] = qb_from_float<A>(v);
  }
}

// out[t, h, :] = sum_g talk[h, g] * scratch[t, g, kv(h), :], g ascending.  One block per (token, head).
template <typename A>
__global__ void __launch_bounds__(128)
talk_mix_kernel(const float* __restrict__ scratch, const float* __restrict__ talk, A* __restrict__ out, int T, int nq,
                int nkv, int vd) {
  const int t = blockIdx.x / nq, h = blockIdx.x % nq;
  if (t >= T) return;
  const int kvh = h / (nq / nkv);
  const float* srow = scratch + (size_t)t * nq * nkv * vd + (size_t)kvh * vd;
  const float* trow = talk + (size_t)h * nq;
  for (int d = threadIdx.x; d < vd; d += blockDim.x) {
    float v = 0.f;
    for (int g0 = 0; g0 < nq; g0 += 8) {
      float x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) x[u] = g0 + u < nq ? srow[(size_t)(g0 + u) * nkv * vd + d] : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) v = g0 + u < nq ? fmaf(trow[g0 + u], x[u], v) : v;
    }
    out[((size_t)t * nq + h) * vd + d] = qb_from_float<A>(v);
  }
}

extern "C" int qb_window_attention(const void* q, int dtype, const void* k_cache, const void* v_cache,
                                   const void* kp_cache, const void* vp_cache, void* out, float* scratch,
                                   const float* talk, const int* tok_pos, const int* tok_req, const int* block_table,
                                   int bt_stride, const int* pool_table, int pool_stride, int T, int nq, int nkv,
                                   int hd, int vd, int page_size, int num_pages, int num_pool_pages, float scale,
                                   float cap, int window, int pool, const float* dist_bias, const float* sink,
                                   float* part, int n_split, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_split < 1 || (n_split > 1 && part == nullptr)) return QB_ERR_BAD_ARG;
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
  P.n_split = n_split; P.part = part;
  const int nv = (vd + 31) / 32;
  if (n_split > 1) {
    const int group = nq / nkv;
    const int gq = group > 4 ? 8 : group > 2 ? 4 : group > 1 ? 2 : 1;
    const int n_chunks = (group + gq - 1) / gq;
    const long rw = (long)T * nkv * n_chunks * n_split * (P.all_values ? nkv : 1);
    const int rblocks = (int)((rw + WA_WARPS - 1) / WA_WARPS);
    const size_t rsmem = (size_t)WA_WARPS * gq * hd * sizeof(float);
#define QB_WR_LAUNCH(A, NV, GQ)                                                                                   \
    window_attention_ranges_kernel<A, NV, GQ><<<rblocks, WA_WARPS * 32, rsmem, stream>>>(                           \
        (const A*)q, (const A*)k_cache, (const A*)v_cache, (const A*)kp_cache, (const A*)vp_cache, P)
#define QB_WR_GROUP(A, NV)                                                                                        \
    do {                                                                                                          \
      if (gq == 1) QB_WR_LAUNCH(A, NV, 1);                                                                        \
      else if (gq == 2) QB_WR_LAUNCH(A, NV, 2);                                                                   \
      else if (gq == 4) QB_WR_LAUNCH(A, NV, 4);                                                                   \
      else QB_WR_LAUNCH(A, NV, 8);                                                                                \
    } while (0)
    QB_DISPATCH_DTYPE(dtype, A, {
      if (nv <= 1) QB_WR_GROUP(A, 1);
      else if (nv <= 2) QB_WR_GROUP(A, 2);
      else if (nv <= 4) QB_WR_GROUP(A, 4);
      else QB_WR_GROUP(A, 8);
    });
#undef QB_WR_GROUP
#undef QB_WR_LAUNCH
    QB_LAUNCH_CHECK();
    const size_t wsm = (size_t)n_split * sizeof(float);
    if (wsm > 48 * 1024 || (long)T * nq > 0x7fffffffL) return QB_ERR_UNSUPPORTED;
    QB_DISPATCH_DTYPE(dtype, A, wa_merge_kernel<A><<<T * nq, 128, wsm, stream>>>(part, sink, (A*)out, scratch, T, nq, nkv,
                                                                                vd, n_split, P.all_values));
    QB_LAUNCH_CHECK();
    if (talk != nullptr) {
      QB_DISPATCH_DTYPE(dtype, A, talk_mix_kernel<A><<<T * nq, 128, 0, stream>>>(scratch, talk, (A*)out, T, nq, nkv, vd));
      QB_LAUNCH_CHECK();
    }
    return 0;
  }
  const long warps = (long)T * nq;
  const int blocks = (int)((warps + WA_WARPS - 1) / WA_WARPS);
  const size_t smem = (size_t)WA_WARPS * (hd + (P.all_values ? nkv * vd : 0)) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
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
    QB_DISPATCH_DTYPE(dtype, A, talk_mix_kernel<A><<<T * nq, 128, 0, stream>>>(scratch, talk, (A*)out, T, nq, nkv, vd));
    QB_LAUNCH_CHECK();
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Pooled blocks: a token whose position ends a block of `pool` tokens (pos % pool == pool - 1) leaves the mean of
// the block's keys and the mean of its values, as the cache holds them, in row pos / pool of the pooled pages.
// The block's earlier tokens may have come in earlier steps: they are read from the pages.  Blocks of 128 elements
// per token; sums in position order, float32.
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
  // a thread an element; eight positions are asked for before the first is added (few blocks have work)
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= kn + vn) return;
  const bool is_k = i < kn;
  const int j = is_k ? i : i - kn, w = is_k ? hd : vd;
  const int head = j / w, d = j % w;
  const A* src = is_k ? k_cache : v_cache;
  float sum = 0.f;
  for (int p0 = pos - pool + 1; p0 <= pos; p0 += 8) {
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int p = p0 + u;
      x[u] = 0.f;
      if (p <= pos) {
        const int page = bt[p / page_size];
        if (page < 0 || page >= num_pages) qb_set_status(status, QB_STATUS_BAD_PAGE, page, 2);
        else x[u] = qb_to_float<A>(src[(((size_t)page * nkv + head) * page_size + p % page_size) * w + d]);
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) sum += x[u];
  }
  A* dst = is_k ? kp_cache : vp_cache;
  dst[(((size_t)dst_page * nkv + head) * page_size + b % page_size) * w + d] = qb_from_float<A>(sum * inv);
}

extern "C" int qb_pool_blocks(const void* k_cache, const void* v_cache, void* kp_cache, void* vp_cache, int dtype,
                              const int* tok_pos, const int* tok_req, const int* block_table, int bt_stride,
                              const int* pool_table, int pool_stride, int T, int nkv, int hd, int vd, int page_size,
                              int num_pages, int num_pool_pages, int pool, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (pool <= 0 || page_size <= 0 || nkv <= 0 || hd <= 0 || vd <= 0) return QB_ERR_BAD_ARG;
  const dim3 grid(T, (nkv * (hd + vd) + 127) / 128);
  QB_DISPATCH_DTYPE(dtype, A, pool_blocks_kernel<A><<<grid, 128, 0, stream>>>(
      (const A*)k_cache, (const A*)v_cache, (A*)kp_cache, (A*)vp_cache, tok_pos, tok_req, block_table, bt_stride,
      pool_table, pool_stride, T, nkv, hd, vd, page_size, num_pages, num_pool_pages, pool, status));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Tensor-core version for prompt portions (bfloat16 q and caches; head sizes that are multiples of 16, values of
// at most 128 a head).  A block owns 64 rows of the step's token list for one q head (four warps of 16 rows) and
// walks the keys in tiles of 64: S = Q K^T with mma.sync m16n8k16 (float32 accumulators), then scale, cap, bias
// and the mask per element in float32, the running maximum and sum per row, and O += P V with P split in two
// bfloat16 parts (p = hi + lo, two MMAs), so that the weights enter the sum with 16 bits of mantissa and not 8.
// The rows of a tile may belong to several requests: the keys are walked request by request (the step's tokens
// of a request are neighbours), rows of other requests are masked, warps without a row of the request idle.
// With mixed heads every (q head g, kv head m) pair is a block of its own that applies g's weights to m's values
// and leaves the normed sums in scratch [T, nq, nkv, vd] for the mixing kernel.
// ---------------------------------------------------------------------------------------------
constexpr int WM_BM = 64, WM_BN = 64;

__device__ __forceinline__ void wm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void wm_ldmatrix_x2(uint32_t (&r)[2], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void wm_ldmatrix_x2_trans(uint32_t (&r)[2], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void wm_mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// two floats -> their bfloat16 roundings (hi) and the roundings of what is left (lo), each packed low | high
__device__ __forceinline__ void wm_split_pair(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
  const __nv_bfloat16 xl = __float2bfloat16_rn(x - __bfloat162float(xh)), yl = __float2bfloat16_rn(y - __bfloat162float(yh));
  hi = (uint32_t)__bfloat16_as_ushort(xh) | ((uint32_t)__bfloat16_as_ushort(yh) << 16);
  lo = (uint32_t)__bfloat16_as_ushort(xl) | ((uint32_t)__bfloat16_as_ushort(yl) << 16);
}

// NTV: value tiles of 8 a warp accumulates, vd <= 8 * NTV
template <int NTV>
__global__ void __launch_bounds__(128)
window_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                            const __nv_bfloat16* __restrict__ v_cache, const __nv_bfloat16* __restrict__ kp_cache,
                            const __nv_bfloat16* __restrict__ vp_cache, __nv_bfloat16* __restrict__ out,
                            float* __restrict__ scratch, const WaParams P) {
  extern __shared__ __align__(16) unsigned char wm_smem[];
  const int hd = P.hd, vd = P.vd, nq = P.nq, nkv = P.nkv, ps = P.page_size;
  const int pq = hd + 8, pv = vd + 8;                                  // row pitches in elements (16-byte multiples)
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(wm_smem);      // [64][pq]
  __nv_bfloat16* Ks0 = Qs + WM_BM * pq;                                // [2][64][pq]
  __nv_bfloat16* Vs0 = Ks0 + 2 * WM_BN * pq;                           // [2][64][pv]
  long long* s_base = reinterpret_cast<long long*>(Vs0 + 2 * WM_BN * pv);   // [2][64] cache row of a key, * 2 + pooled
  float* s_bias0 = reinterpret_cast<float*>(s_base + 2 * WM_BN);       // [2][128] the biases by distance of a tile
  int* s_pos = reinterpret_cast<int*>(s_bias0 + 4 * WM_BN);            // [64]
  int* s_req = s_pos + WM_BM;                                          // [64]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int t0 = blockIdx.x * WM_BM;
  const int h = blockIdx.y;
  const int kvh_k = h / (nq / nkv);
  const int kvh_v = P.all_values ? (int)blockIdx.z : kvh_k;
  const int n_rows = min(WM_BM, P.T - t0);
  const int qc = hd / 8, vc = vd / 8;                                  // 16-byte pieces a row

  for (int i = tid; i < WM_BM; i += 128) {
    s_pos[i] = i < n_rows ? P.tok_pos[t0 + i] : 0;
    s_req[i] = i < n_rows ? P.tok_req[t0 + i] : -1;
  }
  for (int i = tid; i < WM_BM * qc; i += 128) {
    const int r = i / qc, c = i % qc;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + r) * nq + h) * hd + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * pq + c * 8) = v;
  }
  __syncthreads();

  // this thread's two rows: warp * 16 + g8 and + 8
  const int r_a = warp * 16 + g8, r_b = r_a + 8;
  const int pos_a = s_pos[r_a], pos_b = s_pos[r_b];
  const int req_a = s_req[r_a], req_b = s_req[r_b];
  const int lo_a = (P.window > 0 && pos_a - P.window + 1 > 0) ? pos_a - P.window + 1 : 0;
  const int lo_b = (P.window > 0 && pos_b - P.window + 1 > 0) ? pos_b - P.window + 1 : 0;
  const bool pooling = P.pool_table != nullptr && P.window > 0;
  const int nb_a = (pooling && pos_a - P.window + 1 >= P.pool) ? (pos_a - P.window + 1) / P.pool : 0;
  const int nb_b = (pooling && pos_b - P.window + 1 >= P.pool) ? (pos_b - P.window + 1) / P.pool : 0;

  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  float o[NTV][4];
#pragma unroll
  for (int i = 0; i < NTV; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  int ra = 0;
  while (ra < n_rows) {
    const int req = s_req[ra];
    int rb = ra + 1;
    while (rb < n_rows && s_req[rb] == req) ++rb;
    // the keys that any row of the request's rows [ra, rb) reads
    int lo_min = 0x7fffffff, pos_max = -1, nb_max = 0;
    for (int r = ra; r < rb; ++r) {
      const int p = s_pos[r];
      const int lo = (P.window > 0 && p - P.window + 1 > 0) ? p - P.window + 1 : 0;
      const int nb = (pooling && p - P.window + 1 >= P.pool) ? (p - P.window + 1) / P.pool : 0;
      lo_min = min(lo_min, lo); pos_max = max(pos_max, p); nb_max = max(nb_max, nb);
    }
    const int n_keys = nb_max + (pos_max - lo_min + 1);
    const bool warp_active = warp * 16 < rb && warp * 16 + 16 > ra;
    const bool mine_a = req_a == req && r_a >= ra && r_a < rb, mine_b = req_b == req && r_b >= ra && r_b < rb;
    const int* bt = P.block_table + (size_t)req * P.bt_stride;
    const int* pt = pooling ? P.pool_table + (size_t)req * P.pool_stride : nullptr;
    // what the warp's 16 rows have in common: a tile of token keys that every one of them sees in full needs no
    // mask, and with neighbouring positions its biases sit at fixed places of the tile's bias row
    const bool w_whole = __all_sync(0xffffffffu, mine_a && mine_b);
    const int w_lo_max = __reduce_max_sync(0xffffffffu, max(lo_a, lo_b));
    const int w_pos_min = __reduce_min_sync(0xffffffffu, min(pos_a, pos_b));

    // the rows of the request's tokens in this tile and the distances that a tile of keys can be away from them
    int pos_min = 0x7fffffff;
    for (int r = ra; r < rb; ++r) pos_min = min(pos_min, s_pos[r]);

    // a tile's keys: which cache row each is (one lookup a key), then 16-byte asynchronous copies of the rows'
    // pieces into one of two buffers; the next tile's copies run while this tile is computed
    auto find_rows = [&](int k0, int buf) {
      if (tid < WM_BN) {
        const int idx = k0 + tid;
        long long enc = -1;
        if (idx < n_keys) {
          const bool pooled = idx < nb_max;
          const int row = pooled ? idx : lo_min + (idx - nb_max);
          const int page = pooled ? pt[row / ps] : bt[row / ps];
          if (page < 0 || page >= (pooled ? P.num_pool_pages : P.num_pages)) qb_set_status(P.status, QB_STATUS_BAD_PAGE, page, 3);
          else enc = ((((long long)page * nkv) * ps + row % ps) << 1) | (pooled ? 1 : 0);
        }
        s_base[buf * WM_BN + tid] = enc;
      }
    };
    auto start_copies = [&](int buf) {
      __nv_bfloat16* Kd = Ks0 + buf * WM_BN * pq;
      __nv_bfloat16* Vd = Vs0 + buf * WM_BN * pv;
      for (int i = tid; i < WM_BN * (qc + vc); i += 128) {
        const bool is_k = i < WM_BN * qc;
        const int j = is_k ? i : i - WM_BN * qc;
        const int w = is_k ? qc : vc;
        const int r = j / w, c = j % w;
        const long long enc = s_base[buf * WM_BN + r];
        const bool pooled = enc >= 0 && (enc & 1);
        const size_t base = enc >= 0 ? (size_t)(enc >> 1) : 0;
        const __nv_bfloat16* src = is_k ? (pooled ? kp_cache : k_cache) + (base + (size_t)kvh_k * ps) * hd + c * 8
                                        : (pooled ? vp_cache : v_cache) + (base + (size_t)kvh_v * ps) * vd + c * 8;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(is_k ? Kd + r * pq + c * 8 : Vd + r * pv + c * 8);
        const int n = enc >= 0 ? 16 : 0;                               // 0: the 16 bytes are filled with zeros
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(dst), "l"(src), "r"(n));
      }
      asm volatile("cp.async.commit_group;\n" ::);
    };

    __syncthreads();                                                   // the last request's tiles have been read
    find_rows(0, 0);
    __syncthreads();
    start_copies(0);
    int buf = 0;
    for (int k0 = 0; k0 < n_keys; k0 += WM_BN, buf ^= 1) {
      const bool more = k0 + WM_BN < n_keys;
      if (more) find_rows(k0 + WM_BN, buf ^ 1);
      // this tile's biases: distances d0 .. d0 + 127 cover every (row, key) pair when the request's positions in
      // the tile are neighbours; pairs outside read the table itself
      const int j_last = lo_min + (k0 + WM_BN - 1 - nb_max);
      const int d0 = pos_min - j_last;
      float* s_bias = s_bias0 + buf * 2 * WM_BN;                       // the other one may still be read
      if (P.dist_bias != nullptr) {
        const int d = d0 + tid;
        s_bias[tid] = (d >= 0 && d < P.window) ? P.dist_bias[(size_t)d * nq + h] : 0.f;
      }
      __syncthreads();                                                 // the rows of the next tile are known, and
      if (more) {                                                      // its buffer has been read by all warps
        start_copies(buf ^ 1);
        asm volatile("cp.async.wait_group 1;\n" ::);
      } else {
        asm volatile("cp.async.wait_group 0;\n" ::);
      }
      __syncthreads();                                                 // this tile's copies of all threads are there
      const __nv_bfloat16* Ks = Ks0 + buf * WM_BN * pq;
      const __nv_bfloat16* Vs = Vs0 + buf * WM_BN * pv;
      if (!warp_active) continue;

      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
      for (int kk = 0; kk < hd; kk += 16) {
        uint32_t a[4];
        wm_ldmatrix_x4(a, Qs + (warp * 16 + (lane & 15)) * pq + kk + (lane >> 4) * 8);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          uint32_t b[2];
          wm_ldmatrix_x2(b, Ks + (nt * 8 + (lane & 7)) * pq + kk + ((lane >> 3) & 1) * 8);
          wm_mma(s[nt], a, b);
        }
      }
      // scale, cap, bias, mask
      float mx_a = -INFINITY, mx_b = -INFINITY;
      const int j_first = lo_min + (k0 - nb_max);
      const bool open_tile = w_whole && k0 >= nb_max && k0 + WM_BN <= n_keys && j_first >= w_lo_max &&
                             j_first + WM_BN - 1 <= w_pos_min && pos_max - pos_min < WM_BM;
      if (open_tile) {
        const float* bias_a = s_bias + (pos_a - pos_min + WM_BN - 1 - 2 * t4);
        const float* bias_b = s_bias + (pos_b - pos_min + WM_BN - 1 - 2 * t4);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float x = s[nt][e] * P.scale;
            if (P.cap > 0.f) x = P.cap * tanhf(x / P.cap);
            if (P.dist_bias != nullptr) x += (e >= 2 ? bias_b : bias_a)[-(nt * 8 + (e & 1))];
            s[nt][e] = x;
            if (e >= 2) mx_b = fmaxf(mx_b, x); else mx_a = fmaxf(mx_a, x);
          }
        }
      } else {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const bool second = e >= 2;
          const int idx = k0 + nt * 8 + 2 * t4 + (e & 1);
          const bool mine = second ? mine_b : mine_a;
          const int pos = second ? pos_b : pos_a;
          float x = -INFINITY;
          if (mine && idx < n_keys) {
            if (idx < nb_max) {
              if (idx < (second ? nb_b : nb_a)) {
                x = s[nt][e] * P.scale;
                if (P.cap > 0.f) x = P.cap * tanhf(x / P.cap);
              }
            } else {
              const int j = lo_min + (idx - nb_max);
              if (j >= (second ? lo_b : lo_a) && j <= pos) {
                x = s[nt][e] * P.scale;
                if (P.cap > 0.f) x = P.cap * tanhf(x / P.cap);
                if (P.dist_bias != nullptr) {
                  const int dd = pos - j - d0;
                  x += (dd >= 0 && dd < 2 * WM_BN) ? s_bias[dd] : __ldg(P.dist_bias + (size_t)(pos - j) * nq + h);
                }
              }
            }
          }
          s[nt][e] = x;
          if (second) mx_b = fmaxf(mx_b, x); else mx_a = fmaxf(mx_a, x);
        }
      }
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      if (!__any_sync(0xffffffffu, mx_a > -INFINITY || mx_b > -INFINITY)) continue;     // no row of the warp sees the tile
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      const float corr_a = mn_a == -INFINITY ? 1.f : expf(m_a - mn_a), corr_b = mn_b == -INFINITY ? 1.f : expf(m_b - mn_b);
      m_a = mn_a; m_b = mn_b;
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = s[nt][0] == -INFINITY ? 0.f : expf(s[nt][0] - mn_a);
        s[nt][1] = s[nt][1] == -INFINITY ? 0.f : expf(s[nt][1] - mn_a);
        s[nt][2] = s[nt][2] == -INFINITY ? 0.f : expf(s[nt][2] - mn_b);
        s[nt][3] = s[nt][3] == -INFINITY ? 0.f : expf(s[nt][3] - mn_b);
        sum_a += s[nt][0] + s[nt][1];
        sum_b += s[nt][2] + s[nt][3];
      }
      l_a = l_a * corr_a + sum_a;
      l_b = l_b * corr_b + sum_b;
#pragma unroll
      for (int i = 0; i < NTV; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t ah[4], al[4];
        wm_split_pair(s[2 * ks][0], s[2 * ks][1], ah[0], al[0]);
        wm_split_pair(s[2 * ks][2], s[2 * ks][3], ah[1], al[1]);
        wm_split_pair(s[2 * ks + 1][0], s[2 * ks + 1][1], ah[2], al[2]);
        wm_split_pair(s[2 * ks + 1][2], s[2 * ks + 1][3], ah[3], al[3]);
#pragma unroll
        for (int nt = 0; nt < NTV; ++nt) {
          if (nt * 8 < vd) {
            uint32_t b[2];
            wm_ldmatrix_x2_trans(b, Vs + (ks * 16 + (lane & 15)) * pv + nt * 8);
            wm_mma(o[nt], ah, b);
            wm_mma(o[nt], al, b);
          }
        }
      }
    }
    ra = rb;
  }

  // the rows' sums over the four lanes that share them, the sink, and the division
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  if (P.sink != nullptr) {
    l_a += m_a == -INFINITY ? 1.f : expf(P.sink[h] - m_a);
    l_b += m_b == -INFINITY ? 1.f : expf(P.sink[h] - m_b);
  }
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
#pragma unroll
  for (int nt = 0; nt < NTV; ++nt) {
    const int d = nt * 8 + 2 * t4;
    if (d >= vd) continue;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = half ? r_b : r_a;
      if (r >= n_rows) continue;
      const float x = o[nt][2 * half] * (half ? inv_b : inv_a), y = o[nt][2 * half + 1] * (half ? inv_b : inv_a);
      if (P.all_values) {
        float* dst = scratch + (((size_t)(t0 + r) * nq + h) * nkv + kvh_v) * vd + d;
        dst[0] = x; dst[1] = y;
      } else {
        __nv_bfloat16* dst = out + ((size_t)(t0 + r) * nq + h) * vd + d;
        dst[0] = __float2bfloat16_rn(x); dst[1] = __float2bfloat16_rn(y);
      }
    }
  }
}

extern "C" int qb_window_attention_mma_supported(int dtype, int hd, int vd) {
  return dtype == QB_BF16 && hd > 0 && hd <= WA_MAX_HD && hd % 16 == 0 && vd > 0 && vd <= 128 && vd % 16 == 0;
}

extern "C" int qb_window_attention_mma(const void* q, int dtype, const void* k_cache, const void* v_cache,
                                       const void* kp_cache, const void* vp_cache, void* out, float* scratch,
                                       const float* talk, const int* tok_pos, const int* tok_req, const int* block_table,
                                       int bt_stride, const int* pool_table, int pool_stride, int T, int nq, int nkv,
                                       int hd, int vd, int page_size, int num_pages, int num_pool_pages, float scale,
                                       float cap, int window, int pool, const float* dist_bias, const float* sink,
                                       int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!qb_window_attention_mma_supported(dtype, hd, vd) || nq % nkv || page_size <= 0 || nq > 65535 || nkv > 65535)
    return QB_ERR_UNSUPPORTED;
  if (pool_table != nullptr && (pool <= 0 || window <= 0 || kp_cache == nullptr || vp_cache == nullptr)) return QB_ERR_BAD_ARG;
  if (dist_bias != nullptr && window <= 0) return QB_ERR_BAD_ARG;
  if (talk != nullptr && scratch == nullptr) return QB_ERR_BAD_ARG;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)kp_cache | (uintptr_t)vp_cache) & 15) return QB_ERR_BAD_ARG;
  WaParams P;
  P.tok_pos = tok_pos; P.tok_req = tok_req; P.block_table = block_table; P.bt_stride = bt_stride;
  P.pool_table = pool_table; P.pool_stride = pool_stride;
  P.T = T; P.nq = nq; P.nkv = nkv; P.hd = hd; P.vd = vd; P.page_size = page_size; P.num_pages = num_pages;
  P.num_pool_pages = num_pool_pages; P.scale = scale; P.cap = cap; P.window = window; P.pool = pool;
  P.dist_bias = dist_bias; P.sink = sink; P.all_values = talk != nullptr; P.status = status; P.vec = 1;
  P.n_split = 1; P.part = nullptr;
  const size_t smem = ((size_t)(WM_BM + 2 * WM_BN) * (hd + 8) + (size_t)2 * WM_BN * (vd + 8)) * 2 + 2 * WM_BN * sizeof(long long)
                      + 4 * WM_BN * sizeof(float) + 2 * WM_BM * sizeof(int);
  dim3 grid((T + WM_BM - 1) / WM_BM, nq, P.all_values ? nkv : 1);
#define QB_WM_LAUNCH(NTV)                                                                                         \
  do {                                                                                                            \
    auto kern = window_attention_mma_kernel<NTV>;                                                                 \
    if (smem > 48 * 1024) {                                                                                       \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
      if (e != cudaSuccess) return (int)e;                                                                        \
    }                                                                                                             \
    kern<<<grid, 128, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,                     \
                                      (const __nv_bfloat16*)v_cache, (const __nv_bfloat16*)kp_cache,              \
                                      (const __nv_bfloat16*)vp_cache, (__nv_bfloat16*)out, scratch, P);           \
  } while (0)
  if (vd <= 64) QB_WM_LAUNCH(8);
  else QB_WM_LAUNCH(16);
#undef QB_WM_LAUNCH
  QB_LAUNCH_CHECK();
  if (talk != nullptr) {
    talk_mix_kernel<__nv_bfloat16><<<T * nq, 128, 0, stream>>>(scratch, talk, (__nv_bfloat16*)out, T, nq, nkv, vd);
    QB_LAUNCH_CHECK();
  }
  return 0;
}
