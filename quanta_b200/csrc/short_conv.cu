// Short causal convolution over time on every channel, and its state.  Two forms:
//
//   y_t = x_t + sum_{j < taps} w[:, j] * x_{t - taps + 1 + j}          (act 0: the input added back)
//   y_t = silu(b + sum_{j < taps} w[:, j] * x_{t - taps + 1 + j})      (act 1: a bias and silu, nothing added back)
//   y_t = sum_{j < taps} w[:, j] * x_{t - taps + 1 + j}                (act 2: the sum alone)
//
// with zeros before a sequence's start.  The rows of x may be a column range of wider rows (x_stride).
//
// x are the step's rows (float32, e.g. the output of a norm), all requests one after the other; the
// taps-1 rows that precede a request's first row of this step come from the request's state slot,
// which holds the last taps-1 inputs it has seen (zeros after admission).  Everything is float32; the
// result is written in the activation dtype.  A row's numbers depend only on its own request's
// inputs, in a fixed order of additions (j ascending), whatever the cut into steps.
//
// Two launches: the rows (which read the state), then the state (one block a request: the last taps-1
// inputs after this step, taken from the step's rows or, for a portion shorter than taps-1, shifted
// down from the old state).  A step of single tokens (at most two rows a request on average) is ONE launch:
// a thread owns a channel of a request, writes its rows in order and then its state rows, which nobody else
// reads; the additions are the same in the same order.
#include "common.cuh"

template <typename O>
__global__ void short_conv_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                       const float* __restrict__ state, O* __restrict__ out,
                                       const int* __restrict__ tok_req, const int* __restrict__ req_start,
                                       const int* __restrict__ req_slot, int T, int C, int taps, int x_stride,
                                       const float* __restrict__ bias, int act) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const int r = tok_req[t];
  const int first = req_start[r];
  const int hist = taps - 1;
  const float* st = state + (size_t)req_slot[r] * hist * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += blockDim.x * gridDim.y) {
    const float cur = x[(size_t)t * x_stride + c];
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = hist - j;          // how many rows before t
      float v;
      if (back == 0) v = cur;
      else if (t - back >= first) v = x[(size_t)(t - back) * x_stride + c];
      else v = st[(size_t)(hist - (first - (t - back))) * C + c];   // state row hist-1 is the newest
      acc += w[(size_t)c * taps + j] * v;
    }
    if (act == 1) {
      acc += bias != nullptr ? bias[c] : 0.f;
      out[(size_t)t * C + c] = qb_from_float<O>(acc / (1.f + expf(-acc)));
    } else if (act == 2) {
      out[(size_t)t * C + c] = qb_from_float<O>(acc);
    } else {
      out[(size_t)t * C + c] = qb_from_float<O>(cur + acc);
    }
  }
}

__global__ void short_conv_state_kernel(const float* __restrict__ x, float* __restrict__ state,
                                        const int* __restrict__ req_start, const int* __restrict__ req_slot,
                                        int R, int C, int taps, int x_stride) {
  const int r = blockIdx.x;
  if (r >= R) return;
  const int first = req_start[r], n = req_start[r + 1] - first;
  const int hist = taps - 1;
  if (n <= 0 || hist <= 0) return;
  float* st = state + (size_t)req_slot[r] * hist * C;
  // a thread owns its channels in every state row, so the shift needs no barrier: new row i is the input
  // n - hist + i of the step when that is >= 0, else old row i + n
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += blockDim.x * gridDim.y) {
    for (int i = 0; i < hist; ++i) {
      const int src = n - hist + i;
      st[(size_t)i * C + c] = src >= 0 ? x[(size_t)(first + src) * x_stride + c] : st[(size_t)(i + n) * C + c];
    }
  }
}

template <typename O>
__global__ void short_conv_step_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ state,
                                       O* __restrict__ out, const int* __restrict__ req_start,
                                       const int* __restrict__ req_slot, int R, int C, int taps, int x_stride,
                                       const float* __restrict__ bias, int act) {
  const int r = blockIdx.x;
  if (r >= R) return;
  const int first = req_start[r], n = req_start[r + 1] - first;
  const int hist = taps - 1;
  if (n <= 0) return;
  float* st = state + (size_t)req_slot[r] * hist * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += blockDim.x * gridDim.y) {
    for (int i = 0; i < n; ++i) {
      const int t = first + i;
      const float cur = x[(size_t)t * x_stride + c];
      float acc = 0.f;
      for (int j = 0; j < taps; ++j) {
        const int back = hist - j;
        float v;
        if (back == 0) v = cur;
        else if (i - back >= 0) v = x[(size_t)(t - back) * x_stride + c];
        else v = st[(size_t)(hist - (back - i)) * C + c];
        acc += w[(size_t)c * taps + j] * v;
      }
      if (act == 1) {
        acc += bias != nullptr ? bias[c] : 0.f;
        out[(size_t)t * C + c] = qb_from_float<O>(acc / (1.f + expf(-acc)));
      } else if (act == 2) {
        out[(size_t)t * C + c] = qb_from_float<O>(acc);
      } else {
        out[(size_t)t * C + c] = qb_from_float<O>(cur + acc);
      }
    }
    for (int i = 0; i < hist; ++i) {
      const int src = n - hist + i;
      st[(size_t)i * C + c] = src >= 0 ? x[(size_t)(first + src) * x_stride + c] : st[(size_t)(i + n) * C + c];
    }
  }
}

// whether a step of T rows in R requests runs as the one launch
extern "C" int qb_short_conv_one_launch(int T, int R) { return R > 0 && T <= 2 * R ? 1 : 0; }

extern "C" int qb_short_conv(const float* x, const float* w, float* state, void* out, int out_dtype,
                             const int* tok_req, const int* req_start, const int* req_slot, int T, int R,
                             int C, int taps, int x_stride, const float* bias, int act, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps < 1 || C <= 0 || x_stride < C || act < 0 || act > 2) return QB_ERR_BAD_ARG;
  const int threads = C >= 1024 ? 256 : 128;
  if (qb_short_conv_one_launch(T, R)) {
    QB_DISPATCH_DTYPE(out_dtype, O, short_conv_step_kernel<O><<<dim3(R, min(64, (C + threads - 1) / threads)), threads, 0, stream>>>(
        x, w, state, (O*)out, req_start, req_slot, R, C, taps, x_stride, bias, act));
    QB_LAUNCH_CHECK();
    return 0;
  }
  // a step of few rows spreads a row's channels over several blocks (a thread a channel): with one block a row
  // such a step is as long as its longest chain of loads
  const int parts = T >= 512 ? 1 : min(64, (C + threads - 1) / threads);
  QB_DISPATCH_DTYPE(out_dtype, O, short_conv_rows_kernel<O><<<dim3(T, parts), threads, 0, stream>>>(
      x, w, state, (O*)out, tok_req, req_start, req_slot, T, C, taps, x_stride, bias, act));
  QB_LAUNCH_CHECK();
  if (taps > 1) {
    short_conv_state_kernel<<<dim3(R, min(64, (C + threads - 1) / threads)), threads, 0, stream>>>(x, state, req_start, req_slot,
                                                                                                 R, C, taps, x_stride);
    QB_LAUNCH_CHECK();
  }
  return 0;
}
