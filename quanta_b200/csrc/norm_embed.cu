// Embedding gather and RMSNorm fused with the residual sum.
//
// The residual stream h is float32 in both precisions.  A layer's output ("delta") is not added to h
// by the layer itself: the next norm adds it (in float32, slots in index order) while it reads the
// row anyway, writes the new h and the normed row.  One thread block owns one token row, so a row's
// numbers never depend on the rest of the batch.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// h[t,c,:] = float(table[ids[t],:]) * scale (+ float(pos_table[tok_pos[t],:]))   for every copy c
// (reference: src/quanta/minimax/model.py:91).  pos_table: a learned vector per position (not scaled), null for
// none; copies: how many equal residual streams the model keeps (1 for the usual single stream).
// ---------------------------------------------------------------------------------------------
template <typename W>
__global__ void embedding_kernel(float* __restrict__ h, const W* __restrict__ table,
                                 const int* __restrict__ ids, int T, int H, int V, float scale,
                                 const W* __restrict__ pos_table, const int* __restrict__ tok_pos, int n_pos,
                                 int copies, int* status) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const int id = ids[t];
  float* out = h + (size_t)t * copies * H;
  const int p = pos_table != nullptr ? tok_pos[t] : 0;
  const bool bad_id = id < 0 || id >= V, bad_pos = pos_table != nullptr && (p < 0 || p >= n_pos);
  if (bad_id || bad_pos) {
    if (threadIdx.x == 0) {
      if (bad_id) qb_set_status(status, QB_STATUS_BAD_TOKEN, id, 1);
      else qb_set_status(status, QB_STATUS_BAD_POSITION, p, 1);
    }
    for (int i = threadIdx.x; i < copies * H; i += blockDim.x) out[i] = 0.f;
    return;
  }
  const W* row = table + (size_t)id * H;
  const W* prow = pos_table != nullptr ? pos_table + (size_t)p * H : nullptr;
  if (H % 8 == 0) {
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float v[8];
      QbVec8<W>::load(row + i, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= scale;
      if (prow != nullptr) {
        float pv[8];
        QbVec8<W>::load(prow + i, pv);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += pv[e];
      }
      for (int c = 0; c < copies; ++c) QbVec8<float>::store(out + (size_t)c * H + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = qb_to_float<W>(row[i]) * scale;
      if (prow != nullptr) v += qb_to_float<W>(prow[i]);
      for (int c = 0; c < copies; ++c) out[(size_t)c * H + i] = v;
    }
  }
}

extern "C" int qb_embedding(float* h, const void* table, int table_dtype, const int* ids, int T, int H,
                            int V, float scale, const void* pos_table, const int* tok_pos, int n_pos, int copies,
                            int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (copies < 1 || (pos_table != nullptr && (tok_pos == nullptr || n_pos <= 0))) return QB_ERR_BAD_ARG;
  QB_DISPATCH_DTYPE(table_dtype, W,
                    embedding_kernel<W><<<T, 256, 0, stream>>>(h, (const W*)table, ids, T, H, V, scale,
                                                               (const W*)pos_table, tok_pos, n_pos, copies, status));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// row r (token rows[r] if rows != null, else r):
//   x = h[tok,:] + sum_s delta[tok,s,:]          (float32, s ascending)
//   if store_h: h[tok,:] = x
//   out[r,:] = w * (x * rsqrt(mean(x^2) + eps))  (reference: src/quanta/minimax/model_m3.py:60-65)
// out may be null (only fold the delta into h).  The row is held in shared memory between the passes.
// ---------------------------------------------------------------------------------------------
template <typename D, typename O>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const D* __restrict__ delta, int S,
                                   const float* __restrict__ w, O* __restrict__ out,
                                   const int* __restrict__ rows, int n_rows, int H, float eps,
                                   int store_h) {
  extern __shared__ float row_buf[];      // H floats + 32 scratch
  float* scratch = row_buf + H;
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const int tok = rows ? rows[r] : r;
  float* hrow = h + (size_t)tok * H;
  const D* drow = delta ? delta + (size_t)tok * S * H : nullptr;
  float ss = 0.f;
  // the gains of this thread's first chunk are asked for now: they come from memory that the layer's weights
  // have pushed out of L2, and would else be waited for after the row's sum
  float w_first[8];
  if (H % 8 == 0 && out != nullptr && (int)threadIdx.x * 8 < H) QbVec8<float>::load(w + threadIdx.x * 8, w_first);
  if (H % 8 == 0) {
    // 8 elements a thread and step, vector loads; the slots of the delta are still added in index order
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float x[8];
      QbVec8<float>::load(hrow + i, x);
      if (drow) {
#pragma unroll 8
        for (int s = 0; s < S; ++s) {
          float dv[8];
          QbVec8<D>::load(drow + (size_t)s * H + i, dv);
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] += dv[e];
        }
        if (store_h) QbVec8<float>::store(hrow + i, x);
      }
      QbVec8<float>::store(row_buf + i, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float x = hrow[i];
      if (drow) {
        for (int s = 0; s < S; ++s) x += qb_to_float<D>(drow[(size_t)s * H + i]);
      }
      row_buf[i] = x;
      if (store_h && drow) hrow[i] = x;
      ss += x * x;
    }
  }
  const float total = qb_block_sum(ss, scratch);
  if (out == nullptr) return;
  const float r_inv = rsqrtf(total / (float)H + eps);
  O* orow = out + (size_t)r * H;
  if (H % 8 == 0) {
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float x[8], wv[8];
      QbVec8<float>::load(row_buf + i, x);
      if (i == (int)threadIdx.x * 8) {
#pragma unroll
        for (int e = 0; e < 8; ++e) wv[e] = w_first[e];
      } else {
        QbVec8<float>::load(w + i, wv);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = wv[e] * (x[e] * r_inv);
      QbVec8<O>::store(orow + i, x);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      orow[i] = qb_from_float<O>(w[i] * (row_buf[i] * r_inv));
  }
}

extern "C" int qb_add_rmsnorm(float* h, const void* delta, int delta_dtype, int S, const float* w,
                              void* out, int out_dtype, const int* rows, int n_rows, int H, float eps,
                              int store_h, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
  const int threads = H >= 2048 ? 512 : 256;
  QB_DISPATCH_DTYPE(delta_dtype, D, QB_DISPATCH_DTYPE(out_dtype, O, {
    auto kern = add_rmsnorm_kernel<D, O>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    kern<<<n_rows, threads, smem, stream>>>(h, (const D*)delta, S, w, (O*)out, rows, n_rows, H, eps,
                                            store_h);
  }));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A sublayer's output that is RMS-normed (gain g, eps_y) BEFORE it joins the residual stream, fused with
// what follows.  The output may still be a sum that nobody has taken:
//   z = y_scale * (sum_s y[tok, s, :] + y_bias) + x2_scale * (y2[tok, :] + y2_bias)      (slots in order; y2 and
//                                                                                        the biases may be null)
// Row r (token rows[r] if rows != null, else r):
//   d = g * (z * rsqrt(mean(z^2) + eps_y));  x = h[tok,:] + d;  if store_h: h[tok,:] = x
//   out[r,:] = w * (x * rsqrt(mean(x^2) + eps))        (w null: out[r,:] = x, the stream itself for a sublayer
//                                                        that reads it without a norm)
// y null: nothing joins (d = 0).  A row's sums are added in a fixed order that depends on H alone.  The row is
// held in shared memory between the passes.
// ---------------------------------------------------------------------------------------------
template <typename O>
__global__ void normed_add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ y, int S, float y_scale,
                                          const float* __restrict__ y_bias, const float* __restrict__ y2,
                                          float y2_scale, const float* __restrict__ y2_bias,
                                          const float* __restrict__ g, float eps_y,
                                          const float* __restrict__ w, O* __restrict__ out,
                                          const int* __restrict__ rows, int n_rows, int H, float eps, int store_h) {
  extern __shared__ float row_buf[];      // H floats + 32 scratch
  float* scratch = row_buf + H;
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const int tok = rows ? rows[r] : r;
  float* hrow = h + (size_t)tok * H;
  const float* yrow = y ? y + (size_t)tok * S * H : nullptr;
  const float* y2row = y2 ? y2 + (size_t)tok * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; yrow != nullptr && i < H; i += blockDim.x) {
    float v = yrow[i];
    for (int s = 1; s < S; ++s) v += yrow[(size_t)s * H + i];
    if (y_bias) v += y_bias[i];
    v *= y_scale;
    if (y2row) v = fmaf(y2_scale, y2row[i] + (y2_bias ? y2_bias[i] : 0.f), v);
    row_buf[i] = v;
    ss += v * v;
  }
  const float y_inv = rsqrtf(qb_block_sum(ss, scratch) / (float)H + eps_y);
  ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float x = yrow != nullptr ? hrow[i] + g[i] * (row_buf[i] * y_inv) : hrow[i];
    row_buf[i] = x;
    if (store_h && yrow != nullptr) hrow[i] = x;
    ss += x * x;
  }
  if (out == nullptr) return;
  O* orow = out + (size_t)r * H;
  if (w == nullptr) {
    __syncthreads();
    for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = qb_from_float<O>(row_buf[i]);
    return;
  }
  const float total = qb_block_sum(ss, scratch);
  const float r_inv = rsqrtf(total / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = qb_from_float<O>(w[i] * (row_buf[i] * r_inv));
}

extern "C" int qb_normed_add_rmsnorm(float* h, const float* y, int S, float y_scale, const float* y_bias,
                                     const float* y2, float y2_scale, const float* y2_bias, const float* g,
                                     float eps_y, const float* w, void* out,
                                     int out_dtype, const int* rows, int n_rows, int H, float eps, int store_h,
                                     cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (S < 1 || (y != nullptr && g == nullptr)) return QB_ERR_BAD_ARG;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
  const int threads = H >= 2048 ? 512 : 256;
  QB_DISPATCH_DTYPE(out_dtype, O, {
    auto kern = normed_add_rmsnorm_kernel<O>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    kern<<<n_rows, threads, smem, stream>>>(h, y, S, y_scale, y_bias, y2, y2_scale, y2_bias, g, eps_y, w,
                                            (O*)out, rows, n_rows, H, eps, store_h);
  });
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// out[r,:] = silu(gu[r, 0:I]) * gu[r, I:2I]     (dense SwiGLU feed-forward; float32 inside)
// ---------------------------------------------------------------------------------------------
template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gu, A* __restrict__ out, int n_rows, int I) {
  const size_t n = (size_t)n_rows * I;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / I, c = i % I;
    const float g = qb_to_float<A>(gu[r * 2 * I + c]);
    const float u = qb_to_float<A>(gu[r * 2 * I + I + c]);
    out[i] = qb_from_float<A>(g / (1.f + expf(-g)) * u);
  }
}

extern "C" int qb_silu_mul(const void* gu, void* out, int dtype, int n_rows, int I, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t n = (size_t)n_rows * I;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  QB_DISPATCH_DTYPE(dtype, A, silu_mul_kernel<A><<<blocks, 256, 0, stream>>>((const A*)gu, (A*)out, n_rows, I));
  QB_LAUNCH_CHECK();
  return 0;
}


// ---------------------------------------------------------------------------------------------
// Several residual streams per token (x [T, S, H] float32), read by each sublayer as a weighted sum and written
// back through a mixing matrix.  One launch does what lies between two sublayers: the write-back of the
// sublayer that has just run, the read of the next one, and its RMS norm.  Row r (token rows[r] or r):
//   y      = sum_k delta[tok, k, :]                               (the sublayer's output, slots in order; may be null)
//   x'_t   = sum_s mix[s, t] * x_s + mult * out_w[t] * y          (all streams from the old ones; skipped without delta)
//   if store: x[tok] = x'
//   u      = sum_t read_w[t] * x'_t                               (read_w null: the plain sum of the streams)
//   out[r] = w * (u * rsqrt(mean(u^2) + eps))                     (out null: only the write-back; w null: u itself)
// Everything is float32 and every sum has a fixed order, so a row's numbers never depend on the batch.
// ---------------------------------------------------------------------------------------------
constexpr int QB_MAX_STREAMS = 16;

// SS: the number of streams when it is known at compile time (1 to 4: the streams' values stay in registers and rows
// whose width is a multiple of 8 move in 16- and 32-byte pieces), 0: any number up to QB_MAX_STREAMS.
template <typename D, typename O, int SS>
__global__ void streams_mix_rmsnorm_kernel(float* __restrict__ x, int S_rt, const D* __restrict__ delta, int K,
                                           const float* __restrict__ mix, const float* __restrict__ out_w, float mult,
                                           const float* __restrict__ read_w, const float* __restrict__ w,
                                           O* __restrict__ out, const int* __restrict__ rows, int n_rows, int H,
                                           float eps, int store) {
  extern __shared__ float sm_u[];          // H floats (u) + 32 scratch
  float* scratch = sm_u + H;
  __shared__ float s_mix[QB_MAX_STREAMS * QB_MAX_STREAMS], s_out[QB_MAX_STREAMS], s_read[QB_MAX_STREAMS];
  const int S = SS > 0 ? SS : S_rt;
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const int tok = rows ? rows[r] : r;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = mix ? mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    s_out[i] = out_w ? mult * out_w[i] : 0.f;
    s_read[i] = read_w ? read_w[i] : 1.f;
  }
  __syncthreads();
  float* xrow = x + (size_t)tok * S * H;
  const D* drow = delta ? delta + (size_t)tok * K * H : nullptr;
  float ss = 0.f;
  if (SS > 0 && H % 8 == 0) {
    constexpr int SC = SS > 0 ? SS : 1;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float xs[SC][8], u[8];
#pragma unroll
      for (int s = 0; s < SC; ++s) QbVec8<float>::load(xrow + (size_t)s * H + i, xs[s]);
#pragma unroll
      for (int e = 0; e < 8; ++e) u[e] = 0.f;
      if (drow != nullptr) {
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = 0.f;
        for (int k = 0; k < K; ++k) {
          float dv[8];
          QbVec8<D>::load(drow + (size_t)k * H + i, dv);
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] += dv[e];
        }
#pragma unroll
        for (int t = 0; t < SC; ++t) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < SC; ++s) acc = fmaf(s_mix[s * SC + t], xs[s][e], acc);
            v[e] = fmaf(s_out[t], y[e], acc);
            u[e] = fmaf(s_read[t], v[e], u[e]);
          }
          if (store) QbVec8<float>::store(xrow + (size_t)t * H + i, v);
        }
      } else {
#pragma unroll
        for (int t = 0; t < SC; ++t)
#pragma unroll
          for (int e = 0; e < 8; ++e) u[e] = fmaf(s_read[t], xs[t][e], u[e]);
      }
      QbVec8<float>::store(sm_u + i, u);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += u[e] * u[e];
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float xs[QB_MAX_STREAMS];
      for (int s = 0; s < S; ++s) xs[s] = xrow[(size_t)s * H + i];
      float u = 0.f;
      if (drow != nullptr) {
        float y = 0.f;
        for (int k = 0; k < K; ++k) y += qb_to_float<D>(drow[(size_t)k * H + i]);
        for (int t = 0; t < S; ++t) {
          float v = 0.f;
          for (int s = 0; s < S; ++s) v = fmaf(s_mix[s * S + t], xs[s], v);
          v = fmaf(s_out[t], y, v);
          if (store) xrow[(size_t)t * H + i] = v;
          u = fmaf(s_read[t], v, u);
        }
      } else {
        for (int t = 0; t < S; ++t) u = fmaf(s_read[t], xs[t], u);
      }
      sm_u[i] = u;
      ss += u * u;
    }
  }
  if (out == nullptr) return;
  const float total = qb_block_sum(ss, scratch);
  const float r_inv = w != nullptr ? rsqrtf(total / (float)H + eps) : 1.f;
  O* orow = out + (size_t)r * H;
  if (H % 8 == 0) {
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float u[8], wv[8];
      QbVec8<float>::load(sm_u + i, u);
      if (w != nullptr) {
        QbVec8<float>::load(w + i, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) u[e] = wv[e] * (u[e] * r_inv);
      }
      QbVec8<O>::store(orow + i, u);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      orow[i] = qb_from_float<O>(w != nullptr ? w[i] * (sm_u[i] * r_inv) : sm_u[i]);
  }
}

extern "C" int qb_streams_mix_rmsnorm(float* x, int S, const void* delta, int delta_dtype, int K, const float* mix,
                                      const float* out_w, float mult, const float* read_w, const float* w, void* out,
                                      int out_dtype, const int* rows, int n_rows, int H, float eps, int store,
                                      cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (S < 1 || S > QB_MAX_STREAMS) return QB_ERR_UNSUPPORTED;
  if (delta != nullptr && (mix == nullptr || out_w == nullptr || K < 1)) return QB_ERR_BAD_ARG;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
  const int threads = H >= 4096 ? 512 : 256;
#define QB_STREAMS(SS_)                                                                                          \
  do {                                                                                                           \
    auto kern = streams_mix_rmsnorm_kernel<D, O, SS_>;                                                           \
    if (smem > 48 * 1024) {                                                                                      \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
      if (e != cudaSuccess) return (int)e;                                                                       \
    }                                                                                                            \
    kern<<<n_rows, threads, smem, stream>>>(x, S, (const D*)delta, K, mix, out_w, mult, read_w, w, (O*)out, rows, \
                                            n_rows, H, eps, store);                                              \
  } while (0)
  QB_DISPATCH_DTYPE(delta_dtype, D, QB_DISPATCH_DTYPE(out_dtype, O, {
    if (S == 1) QB_STREAMS(1);
    else if (S == 2) QB_STREAMS(2);
    else if (S == 3) QB_STREAMS(3);
    else if (S == 4) QB_STREAMS(4);
    else QB_STREAMS(0);
  }));
#undef QB_STREAMS
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// out[r, c] = relu(x[r, c])^2     (the activation of an ungated feed-forward; float32 inside)
// ---------------------------------------------------------------------------------------------
template <typename A>
__global__ void relu_squared_kernel(const A* __restrict__ x, A* __restrict__ out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = fmaxf(qb_to_float<A>(x[i]), 0.f);
    out[i] = qb_from_float<A>(v * v);
  }
}

extern "C" int qb_relu_squared(const void* x, void* out, int dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  QB_DISPATCH_DTYPE(dtype, A, relu_squared_kernel<A><<<blocks, 256, 0, stream>>>((const A*)x, (A*)out, (size_t)n));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Per-head RMS norm with a gain and an elementwise gate, for mixers whose heads are normed before the output
// projection:  out[t, h*D + i] = o[t,h,i] / sqrt(mean_i(o[t,h,:]^2) + eps) * gain[..] * act(gate[t, h*D + i])
// gain: [H*D] (gain_shared 0) or [D], the same for every head (gain_shared 1); act: sigmoid (gate_kind 0) or
// silu (gate_kind 1).  One warp a (token, head); the sum is a warp reduction in a fixed order.
// ---------------------------------------------------------------------------------------------
template <typename O>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                      int gate_stride, const float* __restrict__ gain, O* __restrict__ out,
                                      int T, int H, int D, float eps, int gain_shared, int gate_kind) {
  constexpr int MAXR = 8;          // elements a lane keeps in registers: heads of up to 256 are read once
  const int lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long)T * H) return;
  const int t = (int)(wid / H), h = (int)(wid % H);
  const float* row = o + ((size_t)t * H + h) * D;
  const float* g = gate + (size_t)t * gate_stride + (size_t)h * D;
  const float* gn = gain + (gain_shared ? 0 : h * D);
  O* orow = out + ((size_t)t * H + h) * D;
  if (D <= 32 * MAXR) {
    // everything the lane needs is asked for at once, before the sum across lanes
    float rv[MAXR], gv[MAXR], nv[MAXR];
#pragma unroll
    for (int u = 0; u < MAXR; ++u) {
      const int i = lane + 32 * u;
      const bool in = i < D;
      rv[u] = in ? row[i] : 0.f;
      gv[u] = in ? g[i] : 0.f;
      nv[u] = in ? gn[i] : 0.f;
    }
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < MAXR; ++u) ss += rv[u] * rv[u];
    ss = qb_warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int u = 0; u < MAXR; ++u) {
      const int i = lane + 32 * u;
      if (i < D) {
        const float sg = 1.f / (1.f + expf(-gv[u]));
        orow[i] = qb_from_float<O>(rv[u] * inv * nv[u] * (gate_kind == 1 ? gv[u] * sg : sg));
      }
    }
    return;
  }
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) ss += row[i] * row[i];
  ss = qb_warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)D + eps);
  for (int i = lane; i < D; i += 32) {
    const float sg = 1.f / (1.f + expf(-g[i]));
    const float a = gate_kind == 1 ? g[i] * sg : sg;
    orow[i] = qb_from_float<O>(row[i] * inv * gn[i] * a);
  }
}

extern "C" int qb_head_norm_gate(const float* o, const float* gate, int gate_stride, const float* gain,
                                 void* out, int out_dtype, int T, int H, int D, float eps, int gain_shared,
                                 int gate_kind, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (gate_kind != 0 && gate_kind != 1) return QB_ERR_BAD_ARG;
  const long warps = (long)T * H;
  const int blocks = (int)((warps + 3) / 4);
  QB_DISPATCH_DTYPE(out_dtype, O, head_norm_gate_kernel<O><<<blocks, 128, 0, stream>>>(
      o, gate, gate_stride, gain, (O*)out, T, H, D, eps, gain_shared, gate_kind));
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// One gate per (token, head): x[t, h, :] *= sigmoid(gate[t, h]) in place (float32 inside, one rounding).
// gate: rows of gate_stride elements of the activation dtype (columns of a wider fused projection).
// ---------------------------------------------------------------------------------------------
template <typename A>
__global__ void head_sigmoid_gate_kernel(A* __restrict__ x, const A* __restrict__ gate, int gate_stride, int T,
                                         int H, int D, int vec) {
  if (vec) {        // D a multiple of 8: eight elements of one head a thread, 16-byte moves
    const size_t n8 = (size_t)T * H * D / 8;
    const int d8 = D / 8;
    for (size_t c = blockIdx.x * (size_t)blockDim.x + threadIdx.x; c < n8; c += (size_t)gridDim.x * blockDim.x) {
      const size_t th = c / d8, t = th / H, h = th % H;
      const float g = qb_to_float<A>(gate[t * gate_stride + h]);
      const float sg = 1.f / (1.f + expf(-g));
      float v[8];
      QbVec8<A>::load(x + c * 8, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= sg;
      QbVec8<A>::store(x + c * 8, v);
    }
    return;
  }
  const size_t n = (size_t)T * H * D;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t th = i / D, t = th / H, h = th % H;
    const float g = qb_to_float<A>(gate[t * gate_stride + h]);
    x[i] = qb_from_float<A>(qb_to_float<A>(x[i]) / (1.f + expf(-g)));
  }
}

extern "C" int qb_head_sigmoid_gate(void* x, const void* gate, int gate_stride, int dtype, int T, int H, int D,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  const int vec = (D % 8 == 0 && ((uintptr_t)x & 31) == 0) ? 1 : 0;
  const size_t n = (size_t)T * H * D / (vec ? 8 : 1);
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  QB_DISPATCH_DTYPE(dtype, A, head_sigmoid_gate_kernel<A><<<blocks, 256, 0, stream>>>((A*)x, (const A*)gate,
                                                                                      gate_stride, T, H, D, vec));
  QB_LAUNCH_CHECK();
  return 0;
}
