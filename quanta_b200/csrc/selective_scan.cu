// Selective state-space scan: a linear recurrence per channel whose decay and input depend on the token.
//
// Per channel c (of `inner`) and state index n (of N), with u the channel's input, dt its step size, B and C the
// token's input and output vectors (shared by all channels), A = -exp(A_log) and D per channel:
//   dt[t, c] = softplus(sum_r W_dt[c, r] * low[t, r] + dt_bias[c])                 (low: R numbers a token)
//   S[c, n] <- exp(dt[t, c] * A[c, n]) * S[c, n] + dt[t, c] * u[t, c] * B[t, n]
//   y[t, c]  = sum_n S[c, n] * C[t, n] + D[c] * u[t, c]
//   out[t, c] = y[t, c] * silu(z[t, c])
// S is float32, one [inner, N] matrix per request in its state slot, zero at admission.  Step sizes, decays,
// exponentials, the state and the gate are float32; u is read in the activation dtype (it is the rounded output
// of the convolution that also feeds the projection of low, B and C), `proj` holds that projection's float32
// accumulators [low | B | C] and z comes from the float32 rows of the input projection.
//
// The step projection W_dt low is a library product (float32) that the caller hands in; its bias and softplus are
// applied as the chain reads it.  The chain in time: eight lanes own a channel (each a stride-8 share of its N
// states, in registers), a block owns 16 channels of one request and walks the request's rows of this step in
// order, a chunk of tokens at a time through shared memory.  Single tokens and portions are the same code and a
// channel's arithmetic does not depend on which block owns it, so cut and batch change nothing.
#include "common.cuh"

constexpr int SS_LANES = 8;            // lanes that share a channel
constexpr int SS_CH = 16;              // channels a block
constexpr int SS_MAX_STATE = 256;

__device__ __forceinline__ float ss_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ void ss_copy4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

// NPL: states a lane holds, N <= 8 * NPL.  The request's rows are walked in chunks of `tok` tokens: the block first
// brings the chunk's step sizes, inputs, gates and B / C vectors into shared memory (asynchronous copies that run
// while the chunk before is computed), then every lane runs the chunk's steps from there (nothing in the chain
// waits for global memory), then the block gates and writes the chunk's outputs.
template <typename U, typename O, int NPL>
__global__ void __launch_bounds__(SS_CH * SS_LANES)
scan_chain_kernel(const U* __restrict__ u, const float* __restrict__ dt_pre, const float* __restrict__ dt_bias,
                  const float* __restrict__ proj,
                  int proj_stride, int b_off, int c_off, const float* __restrict__ z, int z_stride,
                  const float* __restrict__ A, const float* __restrict__ D, float* __restrict__ state,
                  O* __restrict__ out, const int* __restrict__ req_start, const int* __restrict__ req_slot, int inner,
                  int N, int tok) {
  extern __shared__ float ss_smem[];
  // two buffers of what the copies bring (step projections -> step sizes, gates, B and C vectors), one of the
  // inputs and one of the sums
  const int buf_floats = tok * (2 * SS_CH + 2 * N);
  float* s_u = ss_smem + 2 * buf_floats;        // [tok][SS_CH]
  float* s_y = s_u + tok * SS_CH;               // [tok][SS_CH]
  const int r = blockIdx.y;
  const int first = req_start[r], last = req_start[r + 1];
  if (last <= first) return;
  const int sub = threadIdx.x % SS_LANES, ch = threadIdx.x / SS_LANES;
  const int c0 = blockIdx.x * SS_CH;
  const int c = c0 + ch;
  const bool live = c < inner;
  const int cc = live ? c : inner - 1;                       // idle lanes walk along (the shuffles want whole groups)
  float* Srow = state + ((size_t)req_slot[r] * inner + cc) * N;
  float S[NPL], a[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int n = sub + SS_LANES * i;
    S[i] = n < N ? Srow[n] : 0.f;
    a[i] = n < N ? A[(size_t)cc * N + n] : 0.f;
  }
  const float d_c = D[cc];
  // a chunk's rows travel by 4-byte asynchronous copies while the chunk before it is computed and written
  auto start_copies = [&](int t0, int nt, int buf) {
    float* b_dt = ss_smem + buf * buf_floats;
    float* b_z = b_dt + tok * SS_CH;
    float* b_B = b_z + tok * SS_CH;
    float* b_C = b_B + tok * N;
    for (int i = threadIdx.x; i < nt * SS_CH; i += blockDim.x) {
      const int tt = i / SS_CH, k = min(c0 + i % SS_CH, inner - 1);
      ss_copy4(b_dt + i, dt_pre + (size_t)(t0 + tt) * inner + k);
      ss_copy4(b_z + i, z + (size_t)(t0 + tt) * z_stride + k);
    }
    for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
      const int tt = i / N, n = i % N;
      const float* row = proj + (size_t)(t0 + tt) * proj_stride;
      ss_copy4(b_B + i, row + b_off + n);
      ss_copy4(b_C + i, row + c_off + n);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  constexpr int UR = 32 * SS_CH / (SS_CH * SS_LANES);       // inputs of a chunk a thread carries (tok <= 32)
  float ur[UR];
  auto fetch_inputs = [&](int t0, int nt) {
#pragma unroll
    for (int j = 0; j < UR; ++j) {
      const int i = threadIdx.x + j * SS_CH * SS_LANES;
      ur[j] = i < nt * SS_CH ? qb_to_float<U>(u[(size_t)(t0 + i / SS_CH) * inner + min(c0 + i % SS_CH, inner - 1)]) : 0.f;
    }
  };
  start_copies(first, min(tok, last - first), 0);
  fetch_inputs(first, min(tok, last - first));
  int buf = 0;
  for (int t0 = first; t0 < last; t0 += tok, buf ^= 1) {
    const int nt = min(tok, last - t0);
    float* s_dt = ss_smem + buf * buf_floats;
    const float* s_z = s_dt + tok * SS_CH;
    const float* s_B = s_z + tok * SS_CH;
    const float* s_C = s_B + tok * N;
#pragma unroll
    for (int j = 0; j < UR; ++j) {
      const int i = threadIdx.x + j * SS_CH * SS_LANES;
      if (i < nt * SS_CH) s_u[i] = ur[j];
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    for (int i = threadIdx.x; i < nt * SS_CH; i += blockDim.x)      // the thread's own copies: step sizes from them
      s_dt[i] = ss_softplus(s_dt[i] + dt_bias[min(c0 + i % SS_CH, inner - 1)]);
    __syncthreads();                  // the chunk is there, and the chunk before it has been written out by all
    if (t0 + tok < last) {
      start_copies(t0 + tok, min(tok, last - t0 - tok), buf ^ 1);
      fetch_inputs(t0 + tok, min(tok, last - t0 - tok));
    }
    // U steps at a time: their decays, inputs and output vectors are formed first (nothing of that waits for the
    // state), then the state walks through them, then the U sums are added up across the lanes side by side
    constexpr int U = NPL <= 4 ? 4 : NPL <= 8 ? 2 : 1;
    for (int tt = 0; tt < nt; tt += U) {
      float dec[U][NPL], inb[U][NPL], cv[U][NPL], uvs[U], y[U];
#pragma unroll
      for (int s = 0; s < U; ++s) {
        const int row = min(tt + s, nt - 1);
        const float dtv = s_dt[row * SS_CH + ch];
        uvs[s] = s_u[row * SS_CH + ch];
        const float du = dtv * uvs[s];
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          const int n = sub + SS_LANES * i;
          dec[s][i] = n < N ? expf(dtv * a[i]) : 0.f;
          inb[s][i] = n < N ? du * s_B[row * N + n] : 0.f;
          cv[s][i] = n < N ? s_C[row * N + n] : 0.f;
        }
      }
#pragma unroll
      for (int s = 0; s < U; ++s) {
        y[s] = 0.f;
        if (tt + s < nt) {
#pragma unroll
          for (int i = 0; i < NPL; ++i) {
            S[i] = fmaf(dec[s][i], S[i], inb[s][i]);
            y[s] = fmaf(S[i], cv[s][i], y[s]);
          }
        }
      }
#pragma unroll
      for (int o = SS_LANES / 2; o > 0; o >>= 1) {
#pragma unroll
        for (int s = 0; s < U; ++s) y[s] += __shfl_xor_sync(0xffffffffu, y[s], o);
      }
#pragma unroll
      for (int s = 0; s < U; ++s)
        if (sub == 0 && tt + s < nt) s_y[(tt + s) * SS_CH + ch] = fmaf(d_c, uvs[s], y[s]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt * SS_CH; i += blockDim.x) {
      const int tt = i / SS_CH, k = c0 + i % SS_CH;
      if (k < inner) {
        const float zv = s_z[i];
        out[(size_t)(t0 + tt) * inner + k] = qb_from_float<O>(s_y[i] * (zv / (1.f + expf(-zv))));
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = sub + SS_LANES * i;
      if (n < N) Srow[n] = S[i];
    }
  }
}

// u [T, inner] in the activation dtype; proj float32 rows [low (R) | B (N) | C (N) | ...]; z float32 rows of
// z_stride; dt_pre float32 [T, inner], the step projection of `low` (a library product) before its bias and
// softplus; A float32 [inner, N] (already -exp(A_log)); state float32 [slots, inner, N]; out [T, inner] in the
// activation dtype.
extern "C" int qb_selective_scan(const void* u, int dtype, const float* proj, int proj_stride, const float* z,
                                 int z_stride, const float* dt_pre, const float* dt_bias, const float* A, const float* D,
                                 float* state, void* out, const int* req_start, const int* req_slot, int T,
                                 int R_req, int inner, int N, int rank, cudaStream_t stream) {
  if (T <= 0 || R_req <= 0) return 0;
  if (inner <= 0 || N <= 0 || rank <= 0 || proj_stride < rank + 2 * N || z_stride < inner) return QB_ERR_BAD_ARG;
  if (N > SS_MAX_STATE || R_req > 65535) return QB_ERR_UNSUPPORTED;
  dim3 grid((inner + SS_CH - 1) / SS_CH, R_req);
  // tokens a chunk: at most 32, at most the longest portion can be, and what 44 KB of shared memory hold
  const int per_tok = (2 * (2 * SS_CH + 2 * N) + 2 * SS_CH) * (int)sizeof(float);      // two buffers, inputs, sums
  int tok = 44 * 1024 / per_tok;
  tok = tok > 32 ? 32 : tok;
  tok = tok > T ? T : tok;
  const size_t smem = (size_t)tok * per_tok;
#define QB_SS_LAUNCH(NPL)                                                                                             \
  QB_DISPATCH_DTYPE(dtype, U, (scan_chain_kernel<U, U, NPL><<<grid, SS_CH * SS_LANES, smem, stream>>>(                \
      (const U*)u, dt_pre, dt_bias, proj, proj_stride, rank, rank + N, z, z_stride, A, D, state, (U*)out, req_start,  \
      req_slot, inner, N,                                                                                             \
      tok)))
  if (N <= 8 * 2) QB_SS_LAUNCH(2);
  else if (N <= 8 * 4) QB_SS_LAUNCH(4);
  else if (N <= 8 * 8) QB_SS_LAUNCH(8);
  else if (N <= 8 * 16) QB_SS_LAUNCH(16);
  else QB_SS_LAUNCH(32);
#undef QB_SS_LAUNCH
  QB_LAUNCH_CHECK();
  return 0;
}
