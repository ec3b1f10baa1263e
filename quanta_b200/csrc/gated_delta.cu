// Gated delta rule: a recurrence over time whose state is a matrix S [key channel i, value channel j] per
// (request, head), float32, kept in the request's state slot.  With one decay g and one write strength beta per
// (token, head), unit keys k and scaled unit queries q (shared by the heads of a group) and values v:
//
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (in this order)
//
// A first kernel turns the step's projections into what the chain reads: q and k of every (token, group) divided
// by sqrt(sum of squares + unit_eps), q also times q_scale; beta = sigmoid(b); g = exp(-exp(A_log) * softplus(a +
// dt_bias)); all float32.  The recurrence is a chain in time.  A column j of S never meets another column, so
// eight neighbouring lanes own one column (lane p the rows 4 (p + 8 j) .. + 3) in registers for the whole step, and a
// block owns some columns of one (request, head).  Tokens are taken in chunks whose k, q, v, g and beta come into
// shared memory by asynchronous copies while the chunk before is walked.  One token or a portion of a prompt is
// the same code, and a column's numbers do not depend on which block owns it, so a position's numbers depend
// neither on the cut nor on the batch.
#include "common.cuh"

constexpr int GD_MAX_THREADS = 512;

// One block a token.  qk: float32 rows [q (G x D) | k (G x D) | ...] (row stride qk_stride); ab: float32 rows whose
// columns a_off + h and b_off + h hold the pre-activations of the decay and of beta (row stride ab_stride).
__global__ void gated_delta_prep_kernel(const float* __restrict__ qk, int qk_stride, const float* __restrict__ ab,
                                        int ab_stride, int a_off, int b_off, const float* __restrict__ A_log,
                                        const float* __restrict__ dt_bias, float* __restrict__ q_out,
                                        float* __restrict__ k_out, float* __restrict__ g_out,
                                        float* __restrict__ beta_out, int T, int H, int G, int D, float q_scale,
                                        float unit_eps) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float* row = qk + (size_t)t * qk_stride;
  for (int v = warp; v < 2 * G; v += nwarps) {          // v < G: the queries of group v; else the keys of group v - G
    const float* src = row + (size_t)v * D;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) ss += src[i] * src[i];
    ss = qb_warp_sum(ss);
    const float inv = (v < G ? q_scale : 1.f) / sqrtf(ss + unit_eps);
    float* dst = (v < G ? q_out + ((size_t)t * G + v) * D : k_out + ((size_t)t * G + (v - G)) * D);
    for (int i = lane; i < D; i += 32) dst[i] = src[i] * inv;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float a = ab[(size_t)t * ab_stride + a_off + h] + dt_bias[h];
    const float sp = a > 20.f ? a : log1pf(expf(a));
    g_out[(size_t)t * H + h] = expf(-expf(A_log[h]) * sp);
    beta_out[(size_t)t * H + h] = 1.f / (1.f + expf(-ab[(size_t)t * ab_stride + b_off + h]));
  }
}

__device__ __forceinline__ void gd_copy4(float* dst_smem, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

__device__ __forceinline__ void gd_copy16(float* dst_smem, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// GD_LANES neighbouring lanes own a column; RPT rows of it a lane: D <= GD_LANES * RPT
template <int RPT, int GD_LANES>
__global__ void __launch_bounds__(GD_MAX_THREADS, 1)
gated_delta_kernel(const float* __restrict__ q_in, const float* __restrict__ k_in, const float* __restrict__ v_in,
                   int v_stride, const float* __restrict__ g_in, const float* __restrict__ beta_in,
                   float* __restrict__ state, float* __restrict__ out, const int* __restrict__ req_start,
                   const int* __restrict__ req_slot, int H, int G, int D, int DV, int cols_per_block, int chunk) {
  extern __shared__ __align__(16) float sm[];
  constexpr int DP = GD_LANES * RPT;       // padded key channels
  const int r = blockIdx.x, h = blockIdx.y;
  const int grp = h / (H / G);
  const int col0 = blockIdx.z * cols_per_block;
  const int tid = threadIdx.x;
  const int p = tid % GD_LANES;
  const int jl = tid / GD_LANES;
  const int j = col0 + jl;
  const bool owns = jl < cols_per_block && j < DV;
  // a buffer: k [chunk, DP], q [chunk, DP], v [chunk, cols], g [chunk], beta [chunk]
  const size_t plane = (size_t)chunk * DP;
  const size_t buf_floats = 2 * plane + (size_t)chunk * cols_per_block + 2 * chunk;
  // the padding rows (i >= D) are read as zeros and never written
  for (size_t i = tid; i < 2 * buf_floats; i += blockDim.x) sm[i] = 0.f;

  const int t0 = req_start[r], t1 = req_start[r + 1];
  float* S = state + ((size_t)req_slot[r] * H + h) * D * DV;
  // a lane's rows: groups of four consecutive rows, 4 (p + 8 jj) .. + 3, so that it reads its k and q of a token as
  // 16-byte pieces and the eight lanes of a column read 128 consecutive bytes
  float col[RPT];
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = 4 * (p + GD_LANES * (ii >> 2)) + (ii & 3);
    col[ii] = (owns && i < D) ? S[(size_t)i * DV + j] : 0.f;
  }
  __syncthreads();

  const bool wide = D % 4 == 0 && (((uintptr_t)k_in | (uintptr_t)q_in) & 15) == 0;
  auto fetch = [&](int c0, int buf) {
    const int n = min(chunk, t1 - c0);
    float* b = sm + (size_t)buf * buf_floats;
    if (wide) {
      // rows of a multiple of four channels from 16-byte aligned arrays: four channels a copy
      for (int idx = tid; idx < n * (DP / 4); idx += blockDim.x) {
        const int tt = idx / (DP / 4), i = (idx % (DP / 4)) * 4;
        if (i < D) {
          const size_t gsrc = ((size_t)(c0 + tt) * G + grp) * D + i;
          gd_copy16(b + (size_t)tt * DP + i, k_in + gsrc);
          gd_copy16(b + plane + (size_t)tt * DP + i, q_in + gsrc);
        }
      }
    } else {
      for (int idx = tid; idx < n * DP; idx += blockDim.x) {
        const int tt = idx / DP, i = idx % DP;
        if (i < D) {
          const size_t gsrc = ((size_t)(c0 + tt) * G + grp) * D + i;
          gd_copy4(b + idx, k_in + gsrc);
          gd_copy4(b + plane + idx, q_in + gsrc);
        }
      }
    }
    float* bv = b + 2 * plane;
    for (int idx = tid; idx < n * cols_per_block; idx += blockDim.x) {
      const int tt = idx / cols_per_block, c = idx % cols_per_block;
      if (col0 + c < DV) gd_copy4(bv + idx, v_in + (size_t)(c0 + tt) * v_stride + (size_t)h * DV + col0 + c);
    }
    float* bg = bv + (size_t)chunk * cols_per_block;
    for (int tt = tid; tt < n; tt += blockDim.x) {
      gd_copy4(bg + tt, g_in + (size_t)(c0 + tt) * H + h);
      gd_copy4(bg + chunk + tt, beta_in + (size_t)(c0 + tt) * H + h);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (t0 < t1) fetch(t0, 0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += chunk, buf ^= 1) {
    const int n = min(chunk, t1 - c0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                        // this chunk has landed, and everyone is done with the other buffer
    if (c0 + chunk < t1) fetch(c0 + chunk, buf ^ 1);
    const float* s_k = sm + (size_t)buf * buf_floats;
    const float* s_q = s_k + plane;
    const float* s_v = s_q + plane;
    const float* s_g = s_v + (size_t)chunk * cols_per_block;
    const float* s_b = s_g + chunk;
    for (int tt = 0; tt < n; ++tt) {
      const size_t o = (size_t)tt * DP;
      const float g = s_g[tt], beta = s_b[tt];
      // four partial sums a dot product: the chain of dependent additions is a quarter as long
      float d4[4] = {0.f, 0.f, 0.f, 0.f};
      float4 k4[RPT / 4];
#pragma unroll
      for (int jj = 0; jj < RPT / 4; ++jj) {
        k4[jj] = *reinterpret_cast<const float4*>(s_k + o + 4 * (p + GD_LANES * jj));
        col[4 * jj + 0] *= g; col[4 * jj + 1] *= g; col[4 * jj + 2] *= g; col[4 * jj + 3] *= g;
        d4[0] += k4[jj].x * col[4 * jj + 0];
        d4[1] += k4[jj].y * col[4 * jj + 1];
        d4[2] += k4[jj].z * col[4 * jj + 2];
        d4[3] += k4[jj].w * col[4 * jj + 3];
      }
      float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      dot += __shfl_xor_sync(0xffffffffu, dot, 4);
      if (GD_LANES == 16) dot += __shfl_xor_sync(0xffffffffu, dot, 8);
      const float vj = owns ? s_v[(size_t)tt * cols_per_block + jl] : 0.f;
      const float u = beta * (vj - dot);
      float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int jj = 0; jj < RPT / 4; ++jj) {
        const float4 q4 = *reinterpret_cast<const float4*>(s_q + o + 4 * (p + GD_LANES * jj));
        col[4 * jj + 0] += k4[jj].x * u; col[4 * jj + 1] += k4[jj].y * u;
        col[4 * jj + 2] += k4[jj].z * u; col[4 * jj + 3] += k4[jj].w * u;
        a4[0] += q4.x * col[4 * jj + 0];
        a4[1] += q4.y * col[4 * jj + 1];
        a4[2] += q4.z * col[4 * jj + 2];
        a4[3] += q4.w * col[4 * jj + 3];
      }
      float acc = (a4[0] + a4[1]) + (a4[2] + a4[3]);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (GD_LANES == 16) acc += __shfl_xor_sync(0xffffffffu, acc, 8);
      if (owns && p == 0) out[((size_t)(c0 + tt) * H + h) * DV + j] = acc;
    }
  }
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = 4 * (p + GD_LANES * (ii >> 2)) + (ii & 3);
    if (owns && i < D) S[(size_t)i * DV + j] = col[ii];
  }
}

// qkv: float32 rows [q (G x D) | k (G x D) | v (H x DV)] after convolution and activation (row stride qkv_stride);
// ab: float32 rows with the pre-activations of decay (a_off + h) and beta (b_off + h); scratch: T * (2 G D + 2 H)
// floats; out: float32 [T, H, DV].
extern "C" int qb_gated_delta(const float* qkv, int qkv_stride, const float* ab, int ab_stride, int a_off, int b_off,
                              const float* A_log, const float* dt_bias, float* state, float* out, float* scratch,
                              const int* req_start, const int* req_slot, int R, int T, int H, int G, int D, int DV,
                              float q_scale, float unit_eps, cudaStream_t stream) {
  if (R <= 0 || T <= 0) return 0;
  if (D <= 0 || D > 256 || DV <= 0 || DV > 256 || H <= 0 || G <= 0 || H % G) return QB_ERR_UNSUPPORTED;
  const size_t n = (size_t)T * G * D;
  float *q_s = scratch, *k_s = scratch + n, *g_s = scratch + 2 * n, *b_s = g_s + (size_t)T * H;
  gated_delta_prep_kernel<<<T, 128, 0, stream>>>(qkv, qkv_stride, ab, ab_stride, a_off, b_off, A_log, dt_bias, q_s, k_s,
                                                 g_s, b_s, T, H, G, D, q_scale, unit_eps);
  QB_LAUNCH_CHECK();
  // eight lanes a column.  Sixteen (half the multiply-adds a lane and token for one more step of the sums) were
  // measured: no faster on a prompt (637 against 631 us for 2,048 tokens, 16 heads of 128 x 128) and slower for single
  // tokens (22 against 14 us for 8 requests), whose state rows then come in shorter pieces
  const int lanes = 8;
  const int max_cols = GD_MAX_THREADS / lanes;
  // columns a block: all of them (at most max_cols) unless that leaves most SMs idle; then fewer, down to 16
  // where requests bring portions and down to 4 where every request brings one token; a multiple of 4: whole warps
  const int min_cols = T > R ? 16 : 4;
  int splits = (DV + max_cols - 1) / max_cols;
  while ((long)R * H * splits < 132 && (DV + 2 * splits - 1) / (2 * splits) >= min_cols) splits *= 2;
  int cols = (DV + splits - 1) / splits;
  cols = (cols + 3) / 4 * 4;
  splits = (DV + cols - 1) / cols;
  const int threads = cols * lanes;
  const int per_lane = (D + lanes - 1) / lanes;
  const int rpt = per_lane <= 4 ? 4 : per_lane <= 8 ? 8 : per_lane <= 16 ? 16 : 32;
  const int dp = rpt * lanes;
  const int chunk = dp <= 128 ? 16 : 8;
  const size_t smem = (size_t)2 * (2 * chunk * dp + chunk * cols + 2 * chunk) * sizeof(float);
  dim3 grid(R, H, splits);
  const float* v_in = qkv + (size_t)2 * G * D;
#define GD_LAUNCH(N, L)                                                                                    \
  do {                                                                                                     \
    auto kern = gated_delta_kernel<N, L>;                                                                  \
    if (smem > 48 * 1024) {                                                                                \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      if (e != cudaSuccess) return (int)e;                                                                 \
    }                                                                                                      \
    kern<<<grid, threads, smem, stream>>>(q_s, k_s, v_in, qkv_stride, g_s, b_s, state, out, req_start,     \
                                          req_slot, H, G, D, DV, cols, chunk);                             \
  } while (0)
  if (rpt == 4) GD_LAUNCH(4, 8);
  else if (rpt == 8) GD_LAUNCH(8, 8);
  else if (rpt == 16) GD_LAUNCH(16, 8);
  else GD_LAUNCH(32, 8);
#undef GD_LAUNCH
  QB_LAUNCH_CHECK();
  return 0;
}
