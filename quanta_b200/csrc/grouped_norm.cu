// What lies between two sublayers of a model whose sublayer OUTPUTS are normed in groups before they join the
// residual stream, whose branches may each be normed first, and whose stream may be replaced after a layer by a
// weighted sum of the results of all layers so far.  One block a token row, float32 throughout, every sum in an
// order that depends on the sizes alone.  Row r (token rows[r] if rows != null, else r):
//
//   a  = sum_s y[tok, s, :] + y_bias                      b  = y2[tok, :] + y2_bias
//   a' = y_gain * a * rsqrt(mean(a^2) + eps_branch)       b' likewise with y2_gain       (a gain that is null: a' = a)
//   z  = y_scale * a' + y2_scale * b'                     (y2 null: the first term alone)
//   d  = g * z * rsqrt(mean over the group (z^2) + eps_y) (the row in g_groups equal consecutive parts, each divided
//                                                          by its own root mean square; g null: d = z)
//   x  = h[tok, :] + d                                    (y null: x = h[tok, :])
//   hist[n_hist][tok, :] = x;  x = sum_{j <= n_hist} dwa[j] * hist[j][tok, :]            (hist null: skipped)
//   if store_h: h[tok, :] = x
//   out[r, :] = w * x * rsqrt(mean over the group (x^2) + eps)    (w_groups parts; w null: out[r, :] = x; out null: none)
//
// Also here: the tanh cap of logits and the activations of gated dense feed-forwards with biases or clamps.
#include "common.cuh"

#define GN_MAX_GROUPS 64
#define GN_CHUNK 256
#define GN_MAX_CHUNKS 512

// V consecutive floats (V = 4: one 16-byte move from an address that is a multiple of 16 bytes; V = 1: one float)
template <int V> __device__ __forceinline__ void gn_ld(const float* p, float (&v)[V]) {
  if constexpr (V == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    v[0] = *p;
  }
}
template <int V> __device__ __forceinline__ void gn_st(float* p, const float (&v)[V]) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else *p = v[0];
}
template <typename O, int V> __device__ __forceinline__ void gn_st_out(O* p, const float (&v)[V]) {
  if constexpr (V == 4 && sizeof(O) == 2) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  } else if constexpr (V == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
    *p = qb_from_float<O>(v[0]);
  }
}

// 1 / sqrt(mean(buf[group]^2) + eps) of every group into ginv.  One group: the block's fixed-order sum.  Several:
// a warp a chunk of up to GN_CHUNK elements of a group, then a group's chunks added in order.
template <int V>
__device__ __forceinline__ void gn_group_inv(const float* buf, int H, int G, float eps, float* scratch, float* psum,
                                             float* ginv) {
  if (G == 1) {
    float ss = 0.f;
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
      float v[V];
      gn_ld<V>(buf + i, v);
#pragma unroll
      for (int e = 0; e < V; ++e) ss += v[e] * v[e];
    }
    const float total = qb_block_sum(ss, scratch);
    if (threadIdx.x == 0) ginv[0] = rsqrtf(total / (float)H + eps);
    __syncthreads();
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gw = H / G;
  const int nc = (gw + GN_CHUNK - 1) / GN_CHUNK;
  __syncthreads();
  for (int c = warp; c < G * nc; c += nwarps) {
    const int g = c / nc, lo = (c % nc) * GN_CHUNK, hi = min(gw, lo + GN_CHUNK);
    float s = 0.f;
    for (int i = lo + lane * V; i < hi; i += 32 * V) {
      float v[V];
      gn_ld<V>(buf + g * gw + i, v);
#pragma unroll
      for (int e = 0; e < V; ++e) s += v[e] * v[e];
    }
    s = qb_warp_sum(s);
    if (lane == 0) psum[c] = s;
  }
  __syncthreads();
  if ((int)threadIdx.x < G) {
    float s = 0.f;
    for (int c = 0; c < nc; ++c) s += psum[threadIdx.x * nc + c];
    ginv[threadIdx.x] = rsqrtf(s / (float)gw + eps);
  }
  __syncthreads();
}

// Two block-wide sums at once, each in the fixed order of qb_block_sum.  `scratch` holds >= 64 floats.
__device__ __forceinline__ void gn_block_sum2(float& a, float& b, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  a = qb_warp_sum(a);
  b = qb_warp_sum(b);
  __syncthreads();
  if (lane == 0) { scratch[warp] = a; scratch[32 + warp] = b; }
  __syncthreads();
  float ta = 0.f, tb = 0.f;
  for (int w = 0; w < nwarps; ++w) { ta += scratch[w]; tb += scratch[32 + w]; }
  a = ta;
  b = tb;
}

// V = 4: the row moves in 16-byte pieces (the width and both group widths are multiples of 4 and every pointer is a
// multiple of 16 bytes); V = 1: element by element.  A thread touches the same elements of the row in every pass.
template <typename O, int V>
__global__ void grouped_normed_add_kernel(
    float* __restrict__ h, const float* __restrict__ y, int S, float y_scale, const float* __restrict__ y_bias,
    const float* __restrict__ y_gain, const float* __restrict__ y2, float y2_scale, const float* __restrict__ y2_bias,
    const float* __restrict__ y2_gain, float eps_branch, const float* __restrict__ g, int g_groups, float eps_y,
    float* __restrict__ hist, size_t hist_stride, int n_hist, const float* __restrict__ dwa,
    const float* __restrict__ w, int w_groups, float eps, O* __restrict__ out, const int* __restrict__ rows,
    int n_rows, int H, int store_h) {
  extern __shared__ __align__(16) float gn_smem[];
  float* buf = gn_smem;                  // H
  float* buf2 = buf + H;                 // H
  float* scratch = buf2 + H;             // 64
  float* psum = scratch + 64;            // GN_MAX_CHUNKS
  float* ginv = psum + GN_MAX_CHUNKS;    // GN_MAX_GROUPS
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const int tok = rows ? rows[r] : r;
  float* hrow = h + (size_t)tok * H;
  const int i0 = threadIdx.x * V, di = blockDim.x * V;
  if (y != nullptr) {
    const float* yrow = y + (size_t)tok * S * H;
    const float* y2row = y2 ? y2 + (size_t)tok * H : nullptr;
    float ss1 = 0.f, ss2 = 0.f;
#pragma unroll 2
    for (int i = i0; i < H; i += di) {
      float v[V], t[V];
      gn_ld<V>(yrow + i, v);
      for (int s = 1; s < S; ++s) {
        gn_ld<V>(yrow + (size_t)s * H + i, t);
#pragma unroll
        for (int e = 0; e < V; ++e) v[e] += t[e];
      }
      if (y_bias) {
        gn_ld<V>(y_bias + i, t);
#pragma unroll
        for (int e = 0; e < V; ++e) v[e] += t[e];
      }
      gn_st<V>(buf + i, v);
#pragma unroll
      for (int e = 0; e < V; ++e) ss1 += v[e] * v[e];
      if (y2row) {
        gn_ld<V>(y2row + i, v);
        if (y2_bias) {
          gn_ld<V>(y2_bias + i, t);
#pragma unroll
          for (int e = 0; e < V; ++e) v[e] += t[e];
        }
        gn_st<V>(buf2 + i, v);
#pragma unroll
        for (int e = 0; e < V; ++e) ss2 += v[e] * v[e];
      }
    }
    float inv1 = 1.f, inv2 = 1.f;
    if (y_gain != nullptr || (y2row != nullptr && y2_gain != nullptr)) {
      gn_block_sum2(ss1, ss2, scratch);
      if (y_gain) inv1 = rsqrtf(ss1 / (float)H + eps_branch);
      if (y2row && y2_gain) inv2 = rsqrtf(ss2 / (float)H + eps_branch);
    }
    for (int i = i0; i < H; i += di) {
      float a[V], b[V], t[V];
      gn_ld<V>(buf + i, a);
      if (y_gain) {
        gn_ld<V>(y_gain + i, t);
#pragma unroll
        for (int e = 0; e < V; ++e) a[e] = t[e] * (a[e] * inv1);
      }
#pragma unroll
      for (int e = 0; e < V; ++e) a[e] *= y_scale;
      if (y2row) {
        gn_ld<V>(buf2 + i, b);
        if (y2_gain) {
          gn_ld<V>(y2_gain + i, t);
#pragma unroll
          for (int e = 0; e < V; ++e) b[e] = t[e] * (b[e] * inv2);
        }
#pragma unroll
        for (int e = 0; e < V; ++e) a[e] += y2_scale * b[e];
      }
      gn_st<V>(buf + i, a);
    }
    if (g != nullptr) {
      gn_group_inv<V>(buf, H, g_groups, eps_y, scratch, psum, ginv);
      const int gw = H / g_groups;
      for (int i = i0; i < H; i += di) {
        float z[V], x[V], t[V];
        gn_ld<V>(buf + i, z);
        gn_ld<V>(hrow + i, x);
        gn_ld<V>(g + i, t);
        const float inv = ginv[i / gw];            // the V elements lie in one group
#pragma unroll
        for (int e = 0; e < V; ++e) x[e] += t[e] * (z[e] * inv);
        gn_st<V>(buf + i, x);
      }
    } else {
      for (int i = i0; i < H; i += di) {
        float z[V], x[V];
        gn_ld<V>(buf + i, z);
        gn_ld<V>(hrow + i, x);
#pragma unroll
        for (int e = 0; e < V; ++e) x[e] += z[e];
        gn_st<V>(buf + i, x);
      }
    }
  } else {
    for (int i = i0; i < H; i += di) {
      float x[V];
      gn_ld<V>(hrow + i, x);
      gn_st<V>(buf + i, x);
    }
  }
  if (hist != nullptr) {
    // the weights of the sum once into shared memory; the earlier results of an element are asked for several at a
    // time before any of them is used (the additions stay in the order j = 0, 1, ...)
    __syncthreads();
    for (int j = threadIdx.x; j <= n_hist; j += blockDim.x) psum[j] = dwa[j];
    __syncthreads();
    constexpr int AHEAD = V == 4 ? 4 : 8;
    for (int i = i0; i < H; i += di) {
      float x[V], acc[V];
      gn_ld<V>(buf + i, x);
      float* hp = hist + (size_t)tok * H + i;
      gn_st<V>(hp + (size_t)n_hist * hist_stride, x);
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] = 0.f;
      for (int j0 = 0; j0 < n_hist; j0 += AHEAD) {
        float v[AHEAD][V];
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
          if (j0 + u < n_hist) gn_ld<V>(hp + (size_t)(j0 + u) * hist_stride, v[u]);
        }
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
          if (j0 + u < n_hist) {
            const float wj = psum[j0 + u];
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] += wj * v[u][e];
          }
        }
      }
      const float wl = psum[n_hist];
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] += wl * x[e];
      gn_st<V>(buf + i, acc);
    }
  }
  if (store_h && (y != nullptr || hist != nullptr)) {
    for (int i = i0; i < H; i += di) {
      float x[V];
      gn_ld<V>(buf + i, x);
      gn_st<V>(hrow + i, x);
    }
  }
  if (out == nullptr) return;
  O* orow = out + (size_t)r * H;
  if (w == nullptr) {
    for (int i = i0; i < H; i += di) {
      float x[V];
      gn_ld<V>(buf + i, x);
      gn_st_out<O, V>(orow + i, x);
    }
    return;
  }
  gn_group_inv<V>(buf, H, w_groups, eps, scratch, psum, ginv);
  const int gw = H / w_groups;
  for (int i = i0; i < H; i += di) {
    float x[V], t[V];
    gn_ld<V>(buf + i, x);
    gn_ld<V>(w + i, t);
    const float inv = ginv[i / gw];
#pragma unroll
    for (int e = 0; e < V; ++e) x[e] = t[e] * (x[e] * inv);
    gn_st_out<O, V>(orow + i, x);
  }
}

static bool gn_groups_ok(int H, int G) {
  return G >= 1 && G <= GN_MAX_GROUPS && H % G == 0 && (G == 1 || (long)G * ((H / G + GN_CHUNK - 1) / GN_CHUNK) <= GN_MAX_CHUNKS);
}

extern "C" int qb_grouped_normed_add(
    float* h, const float* y, int S, float y_scale, const float* y_bias, const float* y_gain, const float* y2,
    float y2_scale, const float* y2_bias, const float* y2_gain, float eps_branch, const float* g, int g_groups,
    float eps_y, float* hist, long long hist_stride, int n_hist, const float* dwa, const float* w, int w_groups,
    float eps, void* out, int out_dtype, const int* rows, int n_rows, int H, int store_h, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (S < 1 || H <= 0 || (y == nullptr && (y2 != nullptr || g != nullptr))) return QB_ERR_BAD_ARG;
  if (hist != nullptr && (dwa == nullptr || n_hist < 0 || n_hist >= GN_MAX_CHUNKS || rows != nullptr)) return QB_ERR_BAD_ARG;
  if ((g != nullptr && !gn_groups_ok(H, g_groups)) || (w != nullptr && !gn_groups_ok(H, w_groups))) return QB_ERR_UNSUPPORTED;
  const size_t smem = (size_t)(2 * H + 64 + GN_MAX_CHUNKS + GN_MAX_GROUPS) * sizeof(float);
  if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
  // 16-byte moves where every piece starts on such a boundary and lies within one group
  auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = H % 4 == 0 && (g == nullptr || (H / g_groups) % 4 == 0) && (w == nullptr || (H / w_groups) % 4 == 0) &&
                   al16(h) && al16(y) && al16(y_bias) && al16(y_gain) && al16(y2) && al16(y2_bias) && al16(y2_gain) && al16(g) &&
                   al16(hist) && al16(w) && al16(out) && (hist == nullptr || hist_stride % 4 == 0);
  const int per = vec ? 4 : 1;
  const int threads = H >= 2048 * per ? 512 : 256;
#define GN_LAUNCH(O, V)                                                                                              \
  do {                                                                                                               \
    auto kern = grouped_normed_add_kernel<O, V>;                                                                     \
    if (smem > 48 * 1024) {                                                                                          \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
      if (e != cudaSuccess) return (int)e;                                                                           \
    }                                                                                                                \
    kern<<<n_rows, threads, smem, stream>>>(h, y, S, y_scale, y_bias, y_gain, y2, y2_scale, y2_bias, y2_gain, eps_branch, \
                                            g, g_groups, eps_y, hist, (size_t)hist_stride, n_hist, dwa, w, w_groups, eps, \
                                            (O*)out, rows, n_rows, H, store_h);                                      \
  } while (0)
  QB_DISPATCH_DTYPE(out_dtype, O, {
    if (vec) GN_LAUNCH(O, 4);
    else GN_LAUNCH(O, 1);
  });
#undef GN_LAUNCH
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// x <- cap * tanh(x / cap) in place (float32 logits).
// ---------------------------------------------------------------------------------------------
__global__ void tanh_cap_kernel(float* __restrict__ x, size_t n, float cap) {
  const float inv = 1.f / cap;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv);
}

extern "C" int qb_tanh_cap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.f)) return QB_ERR_BAD_ARG;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  tanh_cap_kernel<<<blocks, 256, 0, stream>>>(x, (size_t)n, cap);
  QB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// The activation of a gated dense feed-forward from the fused product gu [rows, 2 I] = [gate | up], float32 inside,
// one rounding.  With a = gu[r, c] + bias[c] and b = gu[r, I + c] + bias[I + c] (bias float32 [2 I] or null):
//   kind 0:  out = silu(a) * b
//   kind 1:  a' = min(a, limit), b' = clamp(b, -limit, limit);  out = a' * sigmoid(alpha * a') * (b' + 1)
// gu may hold the product's float32 accumulators while out is in the activation dtype.
// ---------------------------------------------------------------------------------------------
template <typename IN, typename A>
__global__ void glu_act_kernel(const IN* __restrict__ gu, const float* __restrict__ bias, A* __restrict__ out,
                               int n_rows, int I, int kind, float limit, float alpha) {
  const size_t n = (size_t)n_rows * I;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / I, c = i % I;
    float a = qb_to_float<IN>(gu[r * 2 * I + c]);
    float b = qb_to_float<IN>(gu[r * 2 * I + I + c]);
    if (bias != nullptr) { a += bias[c]; b += bias[I + c]; }
    float v;
    if (kind == 1) {
      a = fminf(a, limit);
      b = fminf(fmaxf(b, -limit), limit);
      v = a / (1.f + expf(-alpha * a)) * (b + 1.f);
    } else {
      v = a / (1.f + expf(-a)) * b;
    }
    out[i] = qb_from_float<A>(v);
  }
}

extern "C" int qb_glu_act(const void* gu, int in_dtype, const float* bias, void* out, int dtype, int n_rows, int I,
                          int kind, float limit, float alpha, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (I <= 0 || kind < 0 || kind > 1) return QB_ERR_BAD_ARG;
  if (in_dtype != dtype && in_dtype != QB_F32) return QB_ERR_BAD_ARG;
  const size_t n = (size_t)n_rows * I;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (dtype == QB_F32)
    glu_act_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)gu, bias, (float*)out, n_rows, I, kind, limit, alpha);
  else if (dtype == QB_BF16 && in_dtype == QB_F32)
    glu_act_kernel<float, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const float*)gu, bias, (__nv_bfloat16*)out, n_rows, I, kind, limit, alpha);
  else if (dtype == QB_BF16)
    glu_act_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, bias, (__nv_bfloat16*)out, n_rows, I, kind, limit, alpha);
  else return QB_ERR_BAD_ARG;
  QB_LAUNCH_CHECK();
  return 0;
}
