// q/k RMSNorm + partial rotary position encoding + query temperature + write of K and V into the paged cache,
// one kernel.
//
// Input is a row of a fused projection, [q | k | v | anything else] (row_stride elements), of every token of the
// step; a layer that reads another layer's cache has rows [q | anything else] (has_kv = 0).  For each token:
//   q, k  <- RMSNorm (none | over all heads of the row | per head), float32
//            (src/quanta/minimax/model_m3.py:15-17 / src/quanta/minimax/attention.py:172-182)
//   q, k  <- rotate-half on the first `rd` dims of each head, pair j using position axis
//            pair_axis[j] and angle float(pos) * inv_freq[j]  (src/quanta/minimax/model_m3.py:83-96)
//   q     <- q * (1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1))     (temp_every > 0: a query
//            temperature that grows with the position, float32)
//   q     <- q * head_scale[head]          (head_scale: a float32 number per q head that multiplies the head's
//            scores; null for none)
//   v     <- (1 - lambda) v + lambda v_first      (v_first: float32 values [T, nkv * vd] that an earlier layer left for
//            the same tokens, lambda one number on the device; v_export: this layer leaves its own values there)
//   q     -> q_out [T, nq, hd];  k -> pages [page, kv_head, slot, hd], v -> pages [page, kv_head, slot, vd]
//            through the block table (keys and values may have different head sizes)
// The rows may be float32 accumulators of the projection while q and the cache are in the activation dtype, and a
// bias (float32, laid out like the row's [q | k | v]) may be added first.  A per-head norm may have no gains.
// One rounding to the activation dtype, at the store.  One block per token.
#include "common.cuh"

#define NORM_NONE 0
#define NORM_PER_LAYER 1
#define NORM_PER_HEAD 2

template <typename IN, typename A>
__global__ void qknorm_rope_write_kernel(
    const IN* __restrict__ qkv, int row_stride, A* __restrict__ q_out, A* __restrict__ k_cache, A* __restrict__ v_cache,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, int norm_kind, float eps,
    const float* __restrict__ inv_freq, const int* __restrict__ pair_axis,
    const int* __restrict__ positions, int n_axes, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_req, const int* __restrict__ block_table, int bt_stride, int T, int nq,
    int nkv_all, int hd, int vd, int has_kv, int rd, float temp_coef, int temp_every, int page_size, int num_pages,
    int vec, const float* __restrict__ bias, const float* __restrict__ v_first, const float* __restrict__ v_lambda,
    float* __restrict__ v_export, const float* __restrict__ head_scale, int* status) {
  extern __shared__ float smem[];
  const int t = blockIdx.x;
  if (t >= T) return;
  const int nkv = has_kv ? nkv_all : 0;
  const int qn = nq * hd, kn = nkv * hd, vn = nkv * vd;
  float* buf = smem;                 // [qn + kn]  q then k
  float* cs = buf + qn + kn;         // [rd/2] cos, [rd/2] sin
  float* scratch = cs + rd;          // 32 + (nq + nkv) head statistics
  float* head_r = scratch + 32;
  const IN* row = qkv + (size_t)t * row_stride;
  const int half = rd / 2;
  // Where this token's K and V go is a chain of three dependent loads (position, request, page id), and the
  // norm gains come from memory that the layer's expert weights have pushed out of L2: both are asked for
  // now, so that their latency passes under the phases below instead of after them.
  int pos = 0, page = -1;
  if (k_cache != nullptr || temp_every > 0) pos = tok_pos[t];
  if (k_cache != nullptr) page = block_table[(size_t)tok_req[t] * bt_stride + pos / page_size];
  const int n_chunks = vec ? (qn + kn) / 8 : 0;
  float w_first[8];                  // the gains of this thread's first chunk (NORM_PER_LAYER)
  if (norm_kind == NORM_PER_LAYER && (int)threadIdx.x < n_chunks) {
    const int i = threadIdx.x * 8;
    QbVec8<float>::load(i < qn ? q_norm_w + i : k_norm_w + (i - qn), w_first);
  }

  if (vec) {
    // 16-byte loads, all of a thread's loads issued before their first use
#pragma unroll 4
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
      float v[8];
      QbVec8<IN>::load(row + c * 8, v);
      if (bias != nullptr) {
        float b[8];
        QbVec8<float>::load(bias + c * 8, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += b[e];
      }
      QbVec8<float>::store(buf + c * 8, v);
    }
  } else {
    for (int i = threadIdx.x; i < qn + kn; i += blockDim.x)
      buf[i] = qb_to_float<IN>(row[i]) + (bias != nullptr ? bias[i] : 0.f);
  }
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const int ax = pair_axis ? pair_axis[j] : 0;
    const float ang = (float)positions[(size_t)t * n_axes + ax] * inv_freq[j];
    float s, c;
    sincosf(ang, &s, &c);
    cs[j] = c;
    cs[half + j] = s;
  }
  __syncthreads();

  if (norm_kind == NORM_PER_LAYER) {
    // a warp per head, then the heads' sums in head order: the same additions whatever the block size
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < nq + nkv; h += nwarps) {
      float sh = 0.f;
      for (int d = lane; d < hd; d += 32) sh += buf[h * hd + d] * buf[h * hd + d];
      sh = qb_warp_sum(sh);
      if (lane == 0) head_r[h] = sh;
    }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
    for (int h = 0; h < nq; ++h) tq += head_r[h];
    for (int h = 0; h < nkv; ++h) tk += head_r[nq + h];
    const float rq = rsqrtf(tq / (float)qn + eps), rk = rsqrtf(tk / (float)max(kn, 1) + eps);
    if (vec) {
#pragma unroll 4
      for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
        const int i = c * 8;
        float w[8], v[8];
        if (c == (int)threadIdx.x) {
#pragma unroll
          for (int e = 0; e < 8; ++e) w[e] = w_first[e];
        } else {
          QbVec8<float>::load(i < qn ? q_norm_w + i : k_norm_w + (i - qn), w);
        }
        QbVec8<float>::load(buf + i, v);
        const float r = i < qn ? rq : rk;
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = w[e] * (v[e] * r);
        QbVec8<float>::store(buf + i, v);
      }
    } else {
      for (int i = threadIdx.x; i < qn + kn; i += blockDim.x)
        buf[i] = (i < qn ? q_norm_w[i] : k_norm_w[i - qn]) * (buf[i] * (i < qn ? rq : rk));
    }
    __syncthreads();
  } else if (norm_kind == NORM_PER_HEAD) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < nq + nkv; h += nwarps) {
      float s = 0.f;
      for (int d = lane; d < hd; d += 32) s += buf[h * hd + d] * buf[h * hd + d];
      s = qb_warp_sum(s);
      if (lane == 0) head_r[h] = rsqrtf(s / (float)hd + eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < qn + kn; i += blockDim.x) {
      const int h = i / hd, d = i % hd;
      const float w = q_norm_w == nullptr ? 1.f : h < nq ? q_norm_w[d] : k_norm_w[d];
      buf[i] = w * (buf[i] * head_r[h]);
    }
    __syncthreads();
  }

  // rotation: each (head, pair) is owned by one thread
  for (int i = threadIdx.x; i < (nq + nkv) * half; i += blockDim.x) {
    const int h = i / half, j = i % half;
    const float a = buf[h * hd + j], b = buf[h * hd + half + j];
    const float c = cs[j], s = cs[half + j];
    buf[h * hd + j] = a * c - b * s;
    buf[h * hd + half + j] = b * c + a * s;
  }
  if (half > 0) __syncthreads();

  const float temp = temp_every > 0 ? 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f) : 1.f;
  A* qo = q_out + (size_t)t * qn;
  if (vec) {
    for (int c = threadIdx.x; c < qn / 8; c += blockDim.x) {
      float v[8];
      QbVec8<float>::load(buf + c * 8, v);
      const float m = head_scale != nullptr ? temp * head_scale[c * 8 / hd] : temp;     // hd % 8 == 0 here
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= m;
      QbVec8<A>::store(qo + c * 8, v);
    }
  } else {
    for (int i = threadIdx.x; i < qn; i += blockDim.x)
      qo[i] = qb_from_float<A>(buf[i] * (head_scale != nullptr ? temp * head_scale[i / hd] : temp));
  }

  if (k_cache == nullptr) return;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) qb_set_status(status, QB_STATUS_BAD_PAGE, page, 2);
    return;
  }
  const int slot = pos % page_size;
  const IN* vrow = row + qn + kn;
  const float* vbias = bias != nullptr ? bias + qn + kn : nullptr;
  const float lam = v_first != nullptr ? v_lambda[0] : 0.f;
  const float* vf = v_first != nullptr ? v_first + (size_t)t * vn : nullptr;
  float* vx = v_export != nullptr ? v_export + (size_t)t * vn : nullptr;
  if (vec) {
    for (int c = threadIdx.x; c < kn / 8; c += blockDim.x) {
      const int i = c * 8, h = i / hd, d = i % hd;
      float kv[8];
      QbVec8<float>::load(buf + qn + i, kv);
      QbVec8<A>::store(k_cache + (((size_t)page * nkv + h) * page_size + slot) * hd + d, kv);
    }
    for (int c = threadIdx.x; c < vn / 8; c += blockDim.x) {
      const int i = c * 8, h = i / vd, d = i % vd;
      float vv[8];
      QbVec8<IN>::load(vrow + i, vv);
      if (vbias != nullptr) {
        float b[8];
        QbVec8<float>::load(vbias + i, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) vv[e] += b[e];
      }
      if (vx != nullptr) QbVec8<float>::store(vx + i, vv);
      if (vf != nullptr) {
        float f[8];
        QbVec8<float>::load(vf + i, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) vv[e] = (1.f - lam) * vv[e] + lam * f[e];
      }
      QbVec8<A>::store(v_cache + (((size_t)page * nkv + h) * page_size + slot) * vd + d, vv);
    }
  } else {
    for (int i = threadIdx.x; i < kn; i += blockDim.x)
      k_cache[(((size_t)page * nkv + i / hd) * page_size + slot) * hd + i % hd] = qb_from_float<A>(buf[qn + i]);
    for (int i = threadIdx.x; i < vn; i += blockDim.x) {
      float v = qb_to_float<IN>(vrow[i]) + (vbias != nullptr ? vbias[i] : 0.f);
      if (vx != nullptr) vx[i] = v;
      if (vf != nullptr) v = (1.f - lam) * v + lam * vf[i];
      v_cache[(((size_t)page * nkv + i / vd) * page_size + slot) * vd + i % vd] = qb_from_float<A>(v);
    }
  }
}

extern "C" int qb_qknorm_rope_write(
    const void* qkv, int in_dtype, int dtype, int row_stride, void* q_out, void* k_cache, void* v_cache, const float* q_norm_w,
    const float* k_norm_w, int norm_kind, float eps, const float* inv_freq, const int* pair_axis,
    const int* positions, int n_axes, const int* tok_pos, const int* tok_req, const int* block_table,
    int bt_stride, int T, int nq, int nkv, int hd, int vd, int has_kv, int rd, float temp_coef, int temp_every,
    int page_size, int num_pages, const float* bias, const float* v_first, const float* v_lambda, float* v_export,
    const float* head_scale, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rd % 2 || rd > hd || rd < 0 || nq <= 0 || nkv <= 0 || page_size <= 0 || hd <= 0 || vd <= 0) return QB_ERR_BAD_ARG;
  // a norm over the whole row needs gains; a per-head norm may have none (both null)
  if (norm_kind == NORM_PER_LAYER && (q_norm_w == nullptr || (has_kv && k_norm_w == nullptr))) return QB_ERR_BAD_ARG;
  if (norm_kind == NORM_PER_HEAD && q_norm_w != nullptr && has_kv && k_norm_w == nullptr) return QB_ERR_BAD_ARG;
  if (norm_kind == NORM_PER_HEAD && q_norm_w == nullptr && k_norm_w != nullptr) return QB_ERR_BAD_ARG;
  if ((v_first != nullptr && v_lambda == nullptr) || ((v_first != nullptr || v_export != nullptr) && !has_kv)) return QB_ERR_BAD_ARG;
  if (in_dtype != dtype && in_dtype != QB_F32) return QB_ERR_BAD_ARG;
  if (!has_kv && k_cache != nullptr) return QB_ERR_BAD_ARG;
  const int nk = has_kv ? nkv : 0;
  if (row_stride < nq * hd + nk * (hd + vd)) return QB_ERR_BAD_ARG;
  // rows are moved in 16-byte pieces where every piece starts on such a boundary; else element by element
  const int vec = (hd % 8 == 0 && vd % 8 == 0 && row_stride % 8 == 0 && ((uintptr_t)qkv & 15) == 0) ? 1 : 0;
  const size_t smem = (size_t)((nq + nk) * hd + rd + 32 + nq + nk) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
#define QB_ROPE_LAUNCH(IN, A)                                                                                   \
  do {                                                                                                          \
    auto kern = qknorm_rope_write_kernel<IN, A>;                                                                \
    if (smem > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      if (e != cudaSuccess) return (int)e;                                                                      \
    }                                                                                                           \
    kern<<<T, threads, smem, stream>>>((const IN*)qkv, row_stride, (A*)q_out, (A*)k_cache, (A*)v_cache, q_norm_w, \
                                       k_norm_w, norm_kind, eps, inv_freq, pair_axis, positions, n_axes, tok_pos, \
                                       tok_req, block_table, bt_stride, T, nq, nkv, hd, vd, has_kv, rd, temp_coef, \
                                       temp_every, page_size, num_pages, vec, bias, v_first, v_lambda, v_export,  \
                                       head_scale, status);                                                              \
  } while (0)
  // steps of few tokens: more threads a token, so that each of the kernel's phases is short
  const int threads = T <= 64 ? 1024 : 256;
  if (dtype == QB_F32) QB_ROPE_LAUNCH(float, float);
  else if (dtype == QB_BF16 && in_dtype == QB_F32) QB_ROPE_LAUNCH(float, __nv_bfloat16);
  else if (dtype == QB_BF16) QB_ROPE_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return QB_ERR_BAD_ARG;
#undef QB_ROPE_LAUNCH
  QB_LAUNCH_CHECK();
  return 0;
}
