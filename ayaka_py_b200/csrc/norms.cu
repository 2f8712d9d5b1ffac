// Root-mean-square norms and what rides on them: plain RMS norm of float32 rows (optionally
// gathered, optionally rows of a wider matrix), RMS norm fused with a short causal convolution
// over time whose last inputs live in a request's state slot, the RMS-normed sublayer output
// added to the residual stream, and the PolyNorm activation.  Statistics, weights and sums are
// 32-bit throughout; only the stored result may be bfloat16.
//
// "RMS norm" is x / sqrt(mean(x^2) + eps), eps inside the root.
#include "common.cuh"

namespace {

constexpr int THREADS = 128;

__device__ __forceinline__ float block_sum_128(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return (red[0] + red[1]) + (red[2] + red[3]);      // the same order in every thread
}

// Three sums at once (PolyNorm's three powers, or the statistics of several rows).
template <int N>
__device__ __forceinline__ void block_sums_128(float (&v)[N], float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = warp_sum(v[i]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) red[i * 4 + warp] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = (red[i * 4] + red[i * 4 + 1]) + (red[i * 4 + 2] + red[i * 4 + 3]);
}

// The same for a block of any number of whole warps (red: N x 32 floats).
template <int N>
__device__ __forceinline__ void block_sums_any(float (&v)[N], float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = warp_sum(v[i]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) red[i * 32 + warp] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float total = 0.f;
    for (int w = 0; w < nwarp; ++w) total += red[i * 32 + w];      // the same order in every thread
    v[i] = total;
  }
}

// The first n of N sums only (the rest are left as they are).
template <int N>
__device__ __forceinline__ void block_sums_upto(float (&v)[N], float* red, int n) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i)
    if (i < n) v[i] = warp_sum(v[i]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (i < n) red[i * 32 + warp] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    if (i < n) {
      float total = 0.f;
      for (int w = 0; w < nwarp; ++w) total += red[i * 32 + w];      // the same order in every thread
      v[i] = total;
    }
  }
}

// ----------------------------------------------------------------- rmsnorm --
// out[r, :] = x[src(r), :d] / rms * w.  One block per row and group: with several groups (grid y) a row
// is that many runs of d numbers side by side, each divided by its own root mean square.
template <typename O>
__global__ void __launch_bounds__(THREADS)
rmsnorm_kernel(O* __restrict__ out, long long out_stride, const float* __restrict__ x, long long x_stride,
               const float* __restrict__ w, const int* __restrict__ rows, int d, float eps) {
  __shared__ float red[4];
  pdl_trigger();
  const int r = blockIdx.x;
  const int src_row = rows ? rows[r] : r;
  const size_t group_at = (size_t)blockIdx.y * d;
  if (w) w += group_at;
  pdl_wait();
  const float* src = x + (size_t)src_row * x_stride + group_at;
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) {
    const float v = src[i];
    s = fmaf(v, v, s);
  }
  const float inv = 1.0f / sqrtf(block_sum_128(s, red) / (float)d + eps);
  O* dst = out + (size_t)r * out_stride + group_at;
  for (int i = threadIdx.x; i < d; i += THREADS) dst[i] = from_float<O>(src[i] * inv * (w ? w[i] : 1.0f));
}

// ------------------------------------------------- rmsnorm + time convolution --
// h_t = rmsnorm(x_t) * w;  out_t = h_t + sum_j c[:, j] * h_(t - taps + 1 + j), where inputs from
// before the row's portion come from the request's state (the last taps - 1 inputs h of earlier
// steps, oldest first; zeros for a new request) and inputs inside the portion are normed again
// from x.  One block per row.  ``inline_state``: every request of the step brings one row, and the
// block shifts the request's state itself (each thread owns its channels, so nothing races);
// otherwise conv_state_kernel runs afterwards.
constexpr int MAX_TAPS = 16;     // the general kernels; the float4 kernel keeps rows in registers and takes up to VEC_TAPS
constexpr int VEC_TAPS = 8;

template <typename O>
__global__ void __launch_bounds__(1024)
rmsnorm_conv_kernel(O* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                    const float* __restrict__ taps_w, float* __restrict__ state, const int* __restrict__ row_req,
                    const int* __restrict__ req_q_start, const int* __restrict__ req_slot, int d, int taps, float eps,
                    int inline_state) {
  __shared__ float red[32 * MAX_TAPS];
  pdl_trigger();
  const int t = blockIdx.x;
  const int req = row_req[t];
  const int first = req_q_start[req];
  const int slot = req_slot[req];
  pdl_wait();
  const int back = taps - 1;
  // statistics of this row and of the earlier rows of the portion that the taps reach
  float sums[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) sums[j] = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) {
      const int s = t - j;                       // j rows back
      if (j <= back && s >= first) {
        const float v = x[(size_t)s * d + i];
        sums[j] = fmaf(v, v, sums[j]);
      }
    }
  }
  block_sums_any<MAX_TAPS>(sums, red);
  float inv[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) inv[j] = 1.0f / sqrtf(sums[j] / (float)d + eps);
  float* st = state + (size_t)slot * back * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float wi = w[i];
    const float h0 = x[(size_t)t * d + i] * inv[0] * wi;
    float acc = h0 * (1.0f + taps_w[(size_t)back * d + i]);
    float held[MAX_TAPS];                        // the state's values of this channel (inline update)
#pragma unroll
    for (int j = 1; j < MAX_TAPS; ++j) {
      if (j <= back) {
        const int s = t - j;
        float hv;
        if (s >= first) hv = x[(size_t)s * d + i] * inv[j] * wi;
        else hv = st[(size_t)(back + (s - first)) * d + i];      // s - first in [-back, -1]
        held[j] = hv;
        acc = fmaf(taps_w[(size_t)(back - j) * d + i], hv, acc);
      }
    }
    out[(size_t)t * d + i] = from_float<O>(acc);
    if (inline_state) {
      // one row per request: the new state is the old one shifted by one, this row's h last
#pragma unroll
      for (int j = MAX_TAPS - 1; j >= 2; --j)
        if (j <= back) st[(size_t)(back - j) * d + i] = held[j - 1];
      if (back >= 1) st[(size_t)(back - 1) * d + i] = h0;
    }
  }
}

// The same for rows of whole float4s up to 4,096 wide: a thread keeps its (up to two) float4 columns
// of the row and of the earlier rows in registers between the two passes, so every row is read once
// per block, 16 bytes at a time.
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 w;
  w.x = *reinterpret_cast<uint32_t*>(&lo);
  w.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = w;
}

template <typename O, int VT>      // VT: the most taps this instance holds rows for
__global__ void __launch_bounds__(512, 2)
rmsnorm_conv_vec_kernel(O* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                        const float* __restrict__ taps_w, float* __restrict__ state, const int* __restrict__ row_req,
                        const int* __restrict__ req_q_start, const int* __restrict__ req_slot, int d, int taps, float eps,
                        int inline_state) {
  __shared__ float red[32 * VT];
  constexpr int V = 2;
  pdl_trigger();
  const int t = blockIdx.x;
  const int req = row_req[t];
  const int first = req_q_start[req];
  const int slot = req_slot[req];
  const int nv = d >> 2, back = taps - 1;
  pdl_wait();
  const float4* x4 = reinterpret_cast<const float4*>(x);
  float4* st4 = reinterpret_cast<float4*>(state + (size_t)slot * back * d);
  float4 xv[VT][V];
  float sums[VT];
#pragma unroll
  for (int j = 0; j < VT; ++j) {
    sums[j] = 0.f;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int idx = threadIdx.x + v * blockDim.x;
      xv[j][v] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j <= back && idx < nv) {
        if (t - j >= first) {
          xv[j][v] = x4[(size_t)(t - j) * nv + idx];
          sums[j] += (xv[j][v].x * xv[j][v].x + xv[j][v].y * xv[j][v].y) + (xv[j][v].z * xv[j][v].z + xv[j][v].w * xv[j][v].w);
        } else {
          xv[j][v] = st4[(size_t)(back + (t - j - first)) * nv + idx];     // an input of an earlier step: normed already
        }
      }
    }
  }
  block_sums_upto<VT>(sums, red, taps);
  float inv[VT];
#pragma unroll
  for (int j = 0; j < VT; ++j) inv[j] = j <= back ? 1.0f / sqrtf(sums[j] / (float)d + eps) : 0.f;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int idx = threadIdx.x + v * blockDim.x;
    if (idx >= nv) continue;
    const float4 wi = reinterpret_cast<const float4*>(w)[idx];
    float4 h[VT];
    h[0] = make_float4(xv[0][v].x * inv[0] * wi.x, xv[0][v].y * inv[0] * wi.y, xv[0][v].z * inv[0] * wi.z, xv[0][v].w * inv[0] * wi.w);
#pragma unroll
    for (int j = 1; j < VT; ++j) {
      if (j <= back) {
        const int s = t - j;
        if (s >= first) h[j] = make_float4(xv[j][v].x * inv[j] * wi.x, xv[j][v].y * inv[j] * wi.y, xv[j][v].z * inv[j] * wi.z, xv[j][v].w * inv[j] * wi.w);
        else h[j] = xv[j][v];
      }
    }
    float acc[4];
    const float4* tw4 = reinterpret_cast<const float4*>(taps_w);   // [taps][d]: a tap of four neighbouring channels is one float4
    const float4 t0 = tw4[(size_t)back * nv + idx];
    acc[0] = h[0].x * (1.0f + t0.x); acc[1] = h[0].y * (1.0f + t0.y);
    acc[2] = h[0].z * (1.0f + t0.z); acc[3] = h[0].w * (1.0f + t0.w);
#pragma unroll
    for (int j = 1; j < VT; ++j) {
      if (j <= back) {
        const float4 tj = tw4[(size_t)(back - j) * nv + idx];
        acc[0] = fmaf(tj.x, h[j].x, acc[0]); acc[1] = fmaf(tj.y, h[j].y, acc[1]);
        acc[2] = fmaf(tj.z, h[j].z, acc[2]); acc[3] = fmaf(tj.w, h[j].w, acc[3]);
      }
    }
    store4(out + (size_t)t * d + 4 * idx, acc[0], acc[1], acc[2], acc[3]);
    if (inline_state) {
#pragma unroll
      for (int j = VT - 1; j >= 2; --j)
        if (j <= back) st4[(size_t)(back - j) * nv + idx] = h[j - 1];
      if (back >= 1) st4[(size_t)(back - 1) * nv + idx] = h[0];
    }
  }
}

// The state after a step: the last taps - 1 of (old state, the portion's inputs h).  One block
// per request; a thread reads what it needs of its channels before it writes them.
__global__ void __launch_bounds__(1024)
conv_state_kernel(float* __restrict__ state, const float* __restrict__ x, const float* __restrict__ w,
                  const int* __restrict__ req_q_start, const int* __restrict__ req_slot, int d, int taps, float eps) {
  __shared__ float red[32 * MAX_TAPS];
  pdl_trigger();
  const int req = blockIdx.x;
  const int first = req_q_start[req], n = req_q_start[req + 1] - first;
  const int slot = req_slot[req];
  pdl_wait();
  const int back = taps - 1;
  float sums[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) sums[j] = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) {
      const int k = n - 1 - j;                   // j rows before the portion's end
      if (j < back && k >= 0) {
        const float v = x[(size_t)(first + k) * d + i];
        sums[j] = fmaf(v, v, sums[j]);
      }
    }
  }
  block_sums_upto<MAX_TAPS>(sums, red, back);
  float* st = state + (size_t)slot * back * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float fresh[MAX_TAPS];
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) {
      if (j < back) {
        const int k = n - 1 - j;
        if (k >= 0) fresh[j] = x[(size_t)(first + k) * d + i] * (1.0f / sqrtf(sums[j] / (float)d + eps)) * w[i];
        else fresh[j] = st[(size_t)(back - 1 - j + n) * d + i];     // still an old input: index back + k
      }
    }
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j)
      if (j < back) st[(size_t)(back - 1 - j) * d + i] = fresh[j];
  }
}

// ------------------------------------------------------ normed residual sum --
// x[t, :] += mult * y[t, :] / rms(y[t, :]) * w; with several groups (grid y) a row is that many runs of d
// numbers, each with its own root mean square.
__global__ void __launch_bounds__(THREADS)
rmsnorm_residual_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, int d,
                        float eps, float mult) {
  __shared__ float red[4];
  pdl_trigger();
  const size_t at = ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * d;
  w += (size_t)blockIdx.y * d;
  pdl_wait();
  const float* src = y + at;
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) {
    const float v = src[i];
    s = fmaf(v, v, s);
  }
  const float inv = 1.0f / sqrtf(block_sum_128(s, red) / (float)d + eps);
  float* dst = x + at;
  for (int i = threadIdx.x; i < d; i += THREADS) dst[i] += mult * (src[i] * inv * w[i]);
}

// The same, and the next norm of the updated stream in the same pass: out[t, :] = x[t, :] / rms(x[t, :]) * w2
// with x as just updated (same runs, each with its own root mean square; eps2 under the root).
template <typename O>
__global__ void __launch_bounds__(THREADS)
rmsnorm_residual_norm_kernel(float* __restrict__ x, O* __restrict__ out, const float* __restrict__ y,
                             const float* __restrict__ w, const float* __restrict__ w2, int d, float eps, float mult,
                             float eps2) {
  __shared__ float red[4], red2[4];
  pdl_trigger();
  const size_t at = ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * d;
  w += (size_t)blockIdx.y * d;
  w2 += (size_t)blockIdx.y * d;
  pdl_wait();
  const float* src = y + at;
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) {
    const float v = src[i];
    s = fmaf(v, v, s);
  }
  const float inv = 1.0f / sqrtf(block_sum_128(s, red) / (float)d + eps);
  float* dst = x + at;
  float s2 = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) {
    const float v = dst[i] + mult * (src[i] * inv * w[i]);
    dst[i] = v;
    s2 = fmaf(v, v, s2);
  }
  const float inv2 = 1.0f / sqrtf(block_sum_128(s2, red2) / (float)d + eps2);
  O* o = out + at;
  for (int i = threadIdx.x; i < d; i += THREADS) o[i] = from_float<O>(dst[i] * inv2 * w2[i]);     // each thread reads back its own stores
}

// ---------------------------------------------- layer-normed residual sum --
// x[t, :] += (y - mean(y)) / sqrt(var(y) + eps) * w + b over a row of d numbers (var: the mean of the squared
// deviations, made in a second pass over the row); b may be null.  With ``out``: the next layer norm of the
// updated stream in the same kernel, out[t, :] = (x - mean(x)) / sqrt(var(x) + eps2) * w2 + b2.
template <typename O>
__global__ void __launch_bounds__(THREADS)
layernorm_residual_kernel(float* __restrict__ x, O* __restrict__ out, const float* __restrict__ y,
                          const float* __restrict__ w, const float* __restrict__ b, const float* __restrict__ w2,
                          const float* __restrict__ b2, int d, float eps, float eps2) {
  __shared__ float red[4], red2[4], red3[4], red4[4];
  pdl_trigger();
  const size_t at = (size_t)blockIdx.x * d;
  pdl_wait();
  const float* src = y + at;
  const float inv_d = 1.0f / (float)d;
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) s += src[i];
  const float mean = block_sum_128(s, red) * inv_d;
  float q = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) {
    const float c = src[i] - mean;
    q = fmaf(c, c, q);
  }
  const float inv = 1.0f / sqrtf(block_sum_128(q, red2) * inv_d + eps);
  float* dst = x + at;
  float s2 = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) {
    const float v = dst[i] + fmaf((src[i] - mean) * inv, w[i], b ? b[i] : 0.f);
    dst[i] = v;
    s2 += v;
  }
  if (!out) return;
  const float mean2 = block_sum_128(s2, red3) * inv_d;
  float q2 = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) {         // each thread reads back its own stores
    const float c = dst[i] - mean2;
    q2 = fmaf(c, c, q2);
  }
  const float inv2 = 1.0f / sqrtf(block_sum_128(q2, red4) * inv_d + eps2);
  O* o = out + at;
  for (int i = threadIdx.x; i < d; i += THREADS) o[i] = from_float<O>(fmaf((dst[i] - mean2) * inv2, w2[i], b2 ? b2[i] : 0.f));
}

// ------------------------------------------------- short groups: a warp each --
// The three norms above for rows cut into groups of at most 1,024 numbers: a warp takes one (row, group), four
// to a block, and no barrier is needed.  ``units`` = rows * groups; taken from 2,048 units on (fewer rows keep a
// block per unit: more threads on each).
template <typename O>
__global__ void __launch_bounds__(THREADS)
rmsnorm_warp_kernel(O* __restrict__ out, long long out_stride, const float* __restrict__ x, long long x_stride,
                    const float* __restrict__ w, const int* __restrict__ rows, int d, int groups, int units, float eps) {
  pdl_trigger();
  const int u = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (u >= units) return;
  const int r = u / groups, grp = u - r * groups;
  const int src_row = rows ? rows[r] : r;
  pdl_wait();
  const size_t group_at = (size_t)grp * d;
  const float* src = x + (size_t)src_row * x_stride + group_at;
  float s = 0.f;
  for (int i = lane; i < d; i += 32) s = fmaf(src[i], src[i], s);
  const float inv = 1.0f / sqrtf(warp_sum(s) / (float)d + eps);
  O* dst = out + (size_t)r * out_stride + group_at;
  for (int i = lane; i < d; i += 32) dst[i] = from_float<O>(src[i] * inv * (w ? w[group_at + i] : 1.0f));
}

// x += mult * norm(y) * w; with ``out`` also out = norm(x) * w2 of the updated rows.
template <typename O>
__global__ void __launch_bounds__(THREADS)
rmsnorm_residual_warp_kernel(float* __restrict__ x, O* __restrict__ out, const float* __restrict__ y,
                             const float* __restrict__ w, const float* __restrict__ w2, int d, int groups, int units,
                             float eps, float mult, float eps2) {
  pdl_trigger();
  const int u = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (u >= units) return;
  pdl_wait();
  const size_t at = (size_t)u * d;              // rows are dense: unit u starts at u * d
  const int grp_at = (u % groups) * d;
  const float* src = y + at;
  float s = 0.f;
  for (int i = lane; i < d; i += 32) s = fmaf(src[i], src[i], s);
  const float inv = 1.0f / sqrtf(warp_sum(s) / (float)d + eps);
  float* dst = x + at;
  float s2 = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float v = dst[i] + mult * (src[i] * inv * w[grp_at + i]);
    dst[i] = v;
    s2 = fmaf(v, v, s2);
  }
  if (!out) return;
  const float inv2 = 1.0f / sqrtf(warp_sum(s2) / (float)d + eps2);
  O* o = out + at;
  for (int i = lane; i < d; i += 32) o[i] = from_float<O>(dst[i] * inv2 * w2[grp_at + i]);     // each lane reads back its own stores
}

// ---------------------------------------------------------------- polynorm --
// out = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e over a row of width n.
template <typename I, typename O>
__global__ void __launch_bounds__(THREADS)
polynorm_kernel(O* __restrict__ out, const I* __restrict__ z, const float* __restrict__ coeff, int n, float eps) {
  __shared__ float red[12];
  pdl_trigger();
  const float a = coeff[0], b = coeff[1], c = coeff[2], e = coeff[3];
  pdl_wait();
  const I* src = z + (size_t)blockIdx.x * n;
  float s[3] = {0.f, 0.f, 0.f};
  for (int i = threadIdx.x; i < n; i += THREADS) {
    const float v = to_float<I>(src[i]);
    const float v2 = v * v, v3 = v2 * v;
    s[0] += v2;
    s[1] = fmaf(v2, v2, s[1]);
    s[2] = fmaf(v3, v3, s[2]);
  }
  block_sums_128<3>(s, red);
  const float i1 = a / sqrtf(s[0] / (float)n + eps);
  const float i2 = b / sqrtf(s[1] / (float)n + eps);
  const float i3 = c / sqrtf(s[2] / (float)n + eps);
  O* dst = out + (size_t)blockIdx.x * n;
  for (int i = threadIdx.x; i < n; i += THREADS) {
    const float v = to_float<I>(src[i]);
    const float v2 = v * v;
    dst[i] = from_float<O>(fmaf(v, i1, fmaf(v2, i2, fmaf(v2 * v, i3, e))));
  }
}

// ------------------------------------------------------------ scaled embed --
template <typename W>
__global__ void embed_scaled_kernel(float* __restrict__ out, const int* __restrict__ tok, const W* __restrict__ table,
                                    int d, float scale) {
  pdl_trigger();
  pdl_wait();
  const W* e = table + (size_t)tok[blockIdx.x] * d;
  float* o = out + (size_t)blockIdx.x * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_float<W>(e[i]) * scale;
}

}  // namespace

// out[r, :d] = rmsnorm(x[rows ? rows[r] : r, :d]) * w (w null: no weight).  x rows lie x_stride
// floats apart, out rows out_stride elements.
// ``groups`` > 1: the d numbers are that many equal runs, each with a root mean square of its own.
AYK_EXPORT int ayk_rmsnorm_grouped(void* out, long long out_stride, const float* x, long long x_stride, const float* w,
                                   const int* rows, int n_rows, int d, int groups, float eps, int out_dtype,
                                   cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AYK_REQUIRE(d >= 1 && groups >= 1 && groups <= 65535 && d % groups == 0, "ayk_rmsnorm: width %d in %d groups", d, groups);
  if (groups > 1 && d / groups <= 1024 && (long long)n_rows * groups >= 2048 && (long long)n_rows * groups < (1ll << 30)) {       // short groups: a warp each
    const int units = n_rows * groups, blocks = (units + THREADS / 32 - 1) / (THREADS / 32);
    if (out_dtype == AYK_DTYPE_F32)
      ayk_launch(rmsnorm_warp_kernel<float>, dim3(blocks), dim3(THREADS), 0, stream, (float*)out, out_stride, x, x_stride, w, rows,
                 d / groups, groups, units, eps);
    else if (out_dtype == AYK_DTYPE_BF16)
      ayk_launch(rmsnorm_warp_kernel<__nv_bfloat16>, dim3(blocks), dim3(THREADS), 0, stream, (__nv_bfloat16*)out, out_stride, x,
                 x_stride, w, rows, d / groups, groups, units, eps);
    else
      return ayk_fail("ayk_rmsnorm: unknown dtype %d", out_dtype);
    return ayk_check_launch("ayk_rmsnorm");
  }
  const dim3 grid(n_rows, groups);
  if (out_dtype == AYK_DTYPE_F32)
    ayk_launch(rmsnorm_kernel<float>, grid, dim3(THREADS), 0, stream, (float*)out, out_stride, x, x_stride, w, rows, d / groups, eps);
  else if (out_dtype == AYK_DTYPE_BF16)
    ayk_launch(rmsnorm_kernel<__nv_bfloat16>, grid, dim3(THREADS), 0, stream, (__nv_bfloat16*)out, out_stride, x,
               x_stride, w, rows, d / groups, eps);
  else
    return ayk_fail("ayk_rmsnorm: unknown dtype %d", out_dtype);
  return ayk_check_launch("ayk_rmsnorm");
}

AYK_EXPORT int ayk_rmsnorm(void* out, long long out_stride, const float* x, long long x_stride, const float* w,
                           const int* rows, int n_rows, int d, float eps, int out_dtype, cudaStream_t stream) {
  return ayk_rmsnorm_grouped(out, out_stride, x, x_stride, w, rows, n_rows, d, 1, eps, out_dtype, stream);
}

// out[t] = h_t + conv(h)_t with h = rmsnorm(x) * w, taps_w [taps, d] (tap-major); state [slots, taps - 1, d]
// float32.  max_q_len == 1 lets the kernel shift the state itself; else a second kernel does.
AYK_EXPORT int ayk_rmsnorm_conv(void* out, const float* x, const float* w, const float* taps_w, float* state,
                                const int* row_req, const int* req_q_start, const int* req_slot, int T, int R, int d,
                                int taps, float eps, int max_q_len, int out_dtype, int* launched, cudaStream_t stream) {
  if (launched) *launched = 0;
  if (T == 0) return 0;
  AYK_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "ayk_rmsnorm_conv: %d taps, the kernel holds up to %d", taps, MAX_TAPS);
  const int inline_state = max_q_len == 1 ? 1 : 0;
  const bool vec = taps <= VEC_TAPS && d % 4 == 0 && d <= 4096 && (uintptr_t)taps_w % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)state % 16 == 0 &&
                   (uintptr_t)out % 16 == 0 && (out_dtype == AYK_DTYPE_F32 || out_dtype == AYK_DTYPE_BF16);
  if (vec) {
    // two float4 columns per thread; few rows (a decode step): one, so that a row's loads are all in flight together
    const int nv = d / 4;
    int threads = (((T <= 256 ? nv : (nv + 1) / 2) + 31) / 32) * 32;
    threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
#define AYK_CONV(OT, VT)                                                                                                  \
  ayk_launch(rmsnorm_conv_vec_kernel<OT, VT>, dim3(T), dim3(threads), 0, stream, (OT*)out, x, w, taps_w, state, row_req, \
             req_q_start, req_slot, d, taps, eps, inline_state)
    if (out_dtype == AYK_DTYPE_F32) {
      if (taps <= 4) AYK_CONV(float, 4); else AYK_CONV(float, VEC_TAPS);
    } else {
      if (taps <= 4) AYK_CONV(__nv_bfloat16, 4); else AYK_CONV(__nv_bfloat16, VEC_TAPS);
    }
#undef AYK_CONV
  } else {
    // few rows (a decode step): many threads per row, so that a row's loads are in flight together
    int threads = THREADS;
    if (T <= 256) threads = min(1024, max(THREADS, (d / 2 + 31) / 32 * 32));
    else if (d >= 2048) threads = 256;
    if (out_dtype == AYK_DTYPE_F32)
      ayk_launch(rmsnorm_conv_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)out, x, w, taps_w, state, row_req,
                 req_q_start, req_slot, d, taps, eps, inline_state);
    else if (out_dtype == AYK_DTYPE_BF16)
      ayk_launch(rmsnorm_conv_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (__nv_bfloat16*)out, x, w, taps_w,
                 state, row_req, req_q_start, req_slot, d, taps, eps, inline_state);
    else
      return ayk_fail("ayk_rmsnorm_conv: unknown dtype %d", out_dtype);
  }
  if (launched) *launched = 1;
  if (ayk_check_launch("ayk_rmsnorm_conv") != 0) return -1;
  if (!inline_state && taps > 1) {
    // one block per request: as many threads as channels (up to 1,024), so that its few loads are in flight together
    const int st_threads = d >= 1024 ? 1024 : (d + 31) / 32 * 32;
    ayk_launch(conv_state_kernel, dim3(R), dim3(st_threads), 0, stream, state, x, w, req_q_start, req_slot, d, taps, eps);
    if (launched) *launched = 2;
    return ayk_check_launch("ayk_rmsnorm_conv (state)");
  }
  return 0;
}

AYK_EXPORT int ayk_rmsnorm_residual(float* x, const float* y, const float* w, int T, int d, float eps, float mult,
                                    cudaStream_t stream) {
  if (T == 0) return 0;
  ayk_launch(rmsnorm_residual_kernel, dim3(T), dim3(THREADS), 0, stream, x, y, w, d, eps, mult);
  return ayk_check_launch("ayk_rmsnorm_residual");
}

// The same with the row cut into ``groups`` equal runs, each divided by its own root mean square.
AYK_EXPORT int ayk_rmsnorm_residual_grouped(float* x, const float* y, const float* w, int T, int d, int groups, float eps,
                                            float mult, cudaStream_t stream) {
  if (T == 0) return 0;
  AYK_REQUIRE(groups >= 1 && groups <= 65535 && d % groups == 0, "ayk_rmsnorm_residual: width %d in %d groups", d, groups);
  if (groups > 1 && d / groups <= 1024 && (long long)T * groups >= 2048 && (long long)T * groups < (1ll << 30)) {
    const int units = T * groups, blocks = (units + THREADS / 32 - 1) / (THREADS / 32);
    ayk_launch(rmsnorm_residual_warp_kernel<float>, dim3(blocks), dim3(THREADS), 0, stream, x, (float*)nullptr, y, w,
               (const float*)nullptr, d / groups, groups, units, eps, mult, 0.0f);
    return ayk_check_launch("ayk_rmsnorm_residual");
  }
  ayk_launch(rmsnorm_residual_kernel, dim3(T, groups), dim3(THREADS), 0, stream, x, y, w, d / groups, eps, mult);
  return ayk_check_launch("ayk_rmsnorm_residual");
}

// x += mult * norm(y) * w and out = norm(x) * w2 of the updated rows, in ``groups`` runs.
AYK_EXPORT int ayk_rmsnorm_residual_norm(float* x, void* out, const float* y, const float* w, const float* w2, int T, int d,
                                         int groups, float eps, float mult, float eps2, int out_dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  AYK_REQUIRE(groups >= 1 && groups <= 65535 && d % groups == 0, "ayk_rmsnorm_residual_norm: width %d in %d groups", d, groups);
  if (groups > 1 && d / groups <= 1024 && (long long)T * groups >= 2048 && (long long)T * groups < (1ll << 30) && (out_dtype == AYK_DTYPE_F32 || out_dtype == AYK_DTYPE_BF16)) {
    const int units = T * groups, blocks = (units + THREADS / 32 - 1) / (THREADS / 32);
    if (out_dtype == AYK_DTYPE_F32)
      ayk_launch(rmsnorm_residual_warp_kernel<float>, dim3(blocks), dim3(THREADS), 0, stream, x, (float*)out, y, w, w2, d / groups,
                 groups, units, eps, mult, eps2);
    else
      ayk_launch(rmsnorm_residual_warp_kernel<__nv_bfloat16>, dim3(blocks), dim3(THREADS), 0, stream, x, (__nv_bfloat16*)out, y, w,
                 w2, d / groups, groups, units, eps, mult, eps2);
    return ayk_check_launch("ayk_rmsnorm_residual_norm");
  }
  if (out_dtype == AYK_DTYPE_F32)
    ayk_launch(rmsnorm_residual_norm_kernel<float>, dim3(T, groups), dim3(THREADS), 0, stream, x, (float*)out, y, w, w2,
               d / groups, eps, mult, eps2);
  else if (out_dtype == AYK_DTYPE_BF16)
    ayk_launch(rmsnorm_residual_norm_kernel<__nv_bfloat16>, dim3(T, groups), dim3(THREADS), 0, stream, x, (__nv_bfloat16*)out,
               y, w, w2, d / groups, eps, mult, eps2);
  else
    return ayk_fail("ayk_rmsnorm_residual_norm: unknown dtype %d", out_dtype);
  return ayk_check_launch("ayk_rmsnorm_residual_norm");
}

AYK_EXPORT int ayk_polynorm(void* out, const void* z, const float* coeff, int T, int n, float eps, int in_dtype,
                            int out_dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  if (in_dtype == AYK_DTYPE_F32 && out_dtype == AYK_DTYPE_F32)
    ayk_launch(polynorm_kernel<float, float>, dim3(T), dim3(THREADS), 0, stream, (float*)out, (const float*)z, coeff, n, eps);
  else if (in_dtype == AYK_DTYPE_F32 && out_dtype == AYK_DTYPE_BF16)
    ayk_launch(polynorm_kernel<float, __nv_bfloat16>, dim3(T), dim3(THREADS), 0, stream, (__nv_bfloat16*)out,
               (const float*)z, coeff, n, eps);
  else if (in_dtype == AYK_DTYPE_BF16 && out_dtype == AYK_DTYPE_BF16)
    ayk_launch(polynorm_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(THREADS), 0, stream, (__nv_bfloat16*)out,
               (const __nv_bfloat16*)z, coeff, n, eps);
  else
    return ayk_fail("ayk_polynorm: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
  return ayk_check_launch("ayk_polynorm");
}

// out[t, :] = table[tok[t], :] * scale as float32.
AYK_EXPORT int ayk_embed_scaled(float* out, const int* tok, const void* table, int T, int d, float scale, int dtype,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  const int threads = d >= 256 ? 256 : 128;
  if (dtype == AYK_DTYPE_F32)
    ayk_launch(embed_scaled_kernel<float>, dim3(T), dim3(threads), 0, stream, out, tok, (const float*)table, d, scale);
  else if (dtype == AYK_DTYPE_BF16)
    ayk_launch(embed_scaled_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out, tok, (const __nv_bfloat16*)table, d, scale);
  else
    return ayk_fail("ayk_embed_scaled: unknown dtype %d", dtype);
  return ayk_check_launch("ayk_embed_scaled");
}

// x += layernorm(y) * w + b in place; with ``out`` also out = layernorm(x) * w2 + b2 of the updated rows.
AYK_EXPORT int ayk_layernorm_residual(float* x, void* out, const float* y, const float* w, const float* b, const float* w2,
                                      const float* b2, int T, int d, float eps, float eps2, int out_dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  AYK_REQUIRE(!out || w2, "ayk_layernorm_residual: the following norm needs its weight");
  if (!out || out_dtype == AYK_DTYPE_F32)
    ayk_launch(layernorm_residual_kernel<float>, dim3(T), dim3(THREADS), 0, stream, x, (float*)out, y, w, b, w2, b2, d, eps, eps2);
  else if (out_dtype == AYK_DTYPE_BF16)
    ayk_launch(layernorm_residual_kernel<__nv_bfloat16>, dim3(T), dim3(THREADS), 0, stream, x, (__nv_bfloat16*)out, y, w, b, w2,
               b2, d, eps, eps2);
  else
    return ayk_fail("ayk_layernorm_residual: unknown dtype %d", out_dtype);
  return ayk_check_launch("ayk_layernorm_residual");
}
