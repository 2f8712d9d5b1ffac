// mLSTM: a matrix memory per head with exponential gates and a running maximum that keeps them finite.
// Per head, with q (already times dim^-1/2), k of D numbers, v of DV numbers, a log input gate
// i = cap tanh(z_i / cap) and a log forget gate f = logsigmoid(cap tanh(z_f / cap)):
//   m_t = max(f_t + m_(t-1), i_t)
//   S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T         [D x DV]
//   n_t = the same with k_t alone                                              [D]
//   o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)
// A new request has S = 0, n = 0 and m = 0 (a finite m: the first tokens' denominators see e^(-m) = 1); all three live,
// 32-bit, in the request's state slot
// as [heads][D * DV + D + 4] floats (S row-major, then n, then m).  Each head's o is then divided by its
// root mean square, multiplied by a weight per channel and by sigmoid of a gate column, and stored in the
// compute dtype.  z_q, z_k, v, z_i, z_f and the gate are columns of one projection row:
// [q (H D) | k (H D) | v (H DV) | z_i (H) | z_f (H) | gate (H DV)].  Everything here is 32-bit.
//
// Two forms.  mlstm_walk_kernel takes the tokens one by one, a block per (request, head): the step of a
// request that brings one token reads and writes its state once, and the head's norm and gate are applied
// in the same kernel.  mlstm_chunk_kernel takes CT tokens at a time (prompt portions).  Inside a chunk, with
// b_t = sum_(r<=t) f_r, a_s = i_s - b_s and g_t = max(m_0, max_(s<=t) a_s), the recurrence of m unrolls to
// m_t = b_t + g_t, and
//   S_t^T q_t = e^(m_0 - g_t) S_0^T q_t + sum_(s<=t) e^(a_s - g_t) (k_s . q_t) v_s
//   n_t . q_t = e^(m_0 - g_t) n_0 . q_t + sum_(s<=t) e^(a_s - g_t) (k_s . q_t)
//   S_C = e^(m_0 - g_C) S_0 + sum_s e^(a_s - g_C) k_s v_s^T,   n_C likewise,   m_C = b_C + g_C,
// every exponent <= 0.  The columns of S do not depend on one another, so a block owns 32 value columns of
// one (request, head) and the grid has DV / 32 times as many blocks (the next chunk's rows arrive by cp.async
// while this one is worked on; the products are register tiles on the FP32 pipes); n and m are recomputed by every block of
// a head and left in a scratch buffer, which mlstm_finish_kernel (the head's norm and gate) files into the
// state: a block that finished early must not change what a later one still reads.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int HEAD_EXTRA = 4;          // floats after n: m and padding that keeps heads 16-byte aligned

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

struct MlstmCols {
  int q, k, v, i, f, g;
  __host__ __device__ MlstmCols(int H, int D, int DV) : q(0), k(H * D), v(2 * H * D), i(2 * H * D + H * DV), f(2 * H * D + H * DV + H),
                                                     g(2 * H * D + H * DV + 2 * H) {}
};

// Sum over a block of whole warps, the same order in every thread (red: 32 floats).
__device__ __forceinline__ float block_sum_any(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarp; ++w) total += red[w];
  return total;
}

// -------------------------------------------------------------------- walk --
// Block (request, head), WALK_THREADS threads as RG row groups x VP columns (VP = DV rounded up to 32): with a
// memory of 128 x 128 a thread owns 16 cells of one column, whose loads do not wait for one another.
constexpr int WALK_THREADS = 1024;

template <typename C>
__global__ void __launch_bounds__(WALK_THREADS)
mlstm_walk_kernel(C* __restrict__ out, float* __restrict__ state, const float* __restrict__ proj, long long stride,
                  const float* __restrict__ norm_w, const int* __restrict__ req_q_start, const int* __restrict__ req_slot,
                  int H, int D, int DV, float cap, float eps) {
  extern __shared__ float sh[];
  __shared__ float red[32];
  float* qs = sh;              // [D]
  float* ks = qs + D;          // [D]
  float* ns = ks + D;          // [D]
  float* part = ns + D;        // [RG][VP]
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int row0 = req_q_start[r], rows = req_q_start[r + 1] - row0, slot = req_slot[r];
  const MlstmCols col(H, D, DV);
  const int VP = (DV + 31) & ~31, RG = blockDim.x / VP;
  const int v = tid % VP, rg = tid / VP;
  const bool owner = rg < RG && v < DV;
  const float qscale = rsqrtf((float)D);
  const size_t head_floats = (size_t)D * DV + D + HEAD_EXTRA;
  float* S = state + ((size_t)slot * H + h) * head_floats;
  float* n_g = S + (size_t)D * DV;
  pdl_wait();
  if (rows <= 0) return;
  // The first token's cells of S are asked for before anything else, so that they travel while the row's gates,
  // q and k are fetched (a decode step is one token: three round trips become one).
  constexpr int PRE = 16;
  const bool ahead = (D + RG - 1) / RG <= PRE;
  float sreg[PRE];
  if (ahead && owner) {
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const int d = rg + i * RG;
      sreg[i] = d < D ? S[(size_t)d * DV + v] : 0.f;
    }
  }
  for (int d = tid; d < D; d += blockDim.x) ns[d] = n_g[d];
  float m = n_g[D];
  for (int t = 0; t < rows; ++t) {
    const float* row = proj + (size_t)(row0 + t) * stride;
    const float ig = cap * tanhf(row[col.i + h] / cap);
    const float fg = log_sigmoid(cap * tanhf(row[col.f + h] / cap));
    const float m_new = fmaxf(fg + m, ig);
    const float keep = expf(fg + m - m_new), wr = expf(ig - m_new);
    __syncthreads();                     // the last token's readers of qs, ks and part are through
    for (int d = tid; d < D; d += blockDim.x) {
      qs[d] = row[col.q + h * D + d] * qscale;
      ks[d] = row[col.k + h * D + d];
    }
    __syncthreads();
    float dot = 0.f;
    for (int d = tid; d < D; d += blockDim.x) {
      const float nd = fmaf(keep, ns[d], wr * ks[d]);
      ns[d] = nd;
      dot = fmaf(nd, qs[d], dot);
    }
    float acc = 0.f;
    if (owner && ahead && t == 0) {
      const float vv = row[col.v + h * DV + v] * wr;
#pragma unroll
      for (int i = 0; i < PRE; ++i) {
        const int d = rg + i * RG;
        if (d < D) {
          const float s = fmaf(keep, sreg[i], ks[d] * vv);
          S[(size_t)d * DV + v] = s;
          acc = fmaf(s, qs[d], acc);
        }
      }
    } else if (owner) {
      const float vv = row[col.v + h * DV + v] * wr;
#pragma unroll 8
      for (int d = rg; d < D; d += RG) {
        const float s = fmaf(keep, S[(size_t)d * DV + v], ks[d] * vv);
        S[(size_t)d * DV + v] = s;
        acc = fmaf(s, qs[d], acc);
      }
    }
    if (rg < RG) part[rg * VP + v] = acc;
    dot = block_sum_any(dot, red);       // its barriers also publish part
    float o = 0.f;
    if (tid < DV) {
      for (int g = 0; g < RG; ++g) o += part[g * VP + tid];
      o /= fmaxf(fabsf(dot), expf(-m_new)) + 1e-6f;
    }
    const float ss = block_sum_any(o * o, red);
    if (tid < DV) {
      const int c = h * DV + tid;
      const float inv = 1.0f / sqrtf(ss / (float)DV + eps);
      out[(size_t)(row0 + t) * H * DV + c] = from_float<C>(o * inv * norm_w[c] / (1.0f + expf(-row[col.g + c])));
    }
    m = m_new;
  }
  __syncthreads();
  for (int d = tid; d < D; d += blockDim.x) n_g[d] = ns[d];
  if (tid == 0) n_g[D] = m;
}

// ------------------------------------------------------------------- chunk --
constexpr int CWARPS = 8, CTHREADS = CWARPS * 32;

__device__ __forceinline__ void cp_async_4(float* dst, const float* src, bool live) {
  const uint32_t to = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = live ? 4 : 0;                    // 0: nothing is read and the four bytes are zeros
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(to), "l"(src), "r"(bytes) : "memory");
}

// Shared memory of the chunked kernel, in floats; D4 = D rounded up to 4, LD = D4 + 4 (rows of q and k stay
// 16-byte aligned and neighbouring rows start four banks apart).
__host__ __device__ inline size_t chunk_floats(int D, int CT, int COLS) {
  const int D4 = (D + 3) & ~3, LD = D4 + 4;
  return (size_t)D4 * COLS + 4 * (size_t)CT * LD + 2 * CT * COLS + 4 * CT + CT * (CT + 1) + D4 + 8 * CT + 8;
}

// Block (slice of COLS value columns, head, request), 256 threads; COLS is 32, or 16 where slices of 32 would leave
// most SMs without a block (a warp's lanes are then two groups of 16 columns that take different tokens and rows).
// raw [T, H * DV] float32 receives o before the head's
// norm; nm [requests, H, D + 1] the head's n and m after the portion (written by the first slice's block).
// The rows of the next chunk (q, k, the slice of v, the gates' inputs) arrive by cp.async into the other half of
// two buffers while this chunk is worked on.  q stays unscaled in shared memory; D^-1/2 multiplies the sums.
template <int CT, int COLS>
__global__ void __launch_bounds__(CTHREADS)
mlstm_chunk_kernel(float* __restrict__ raw, float* __restrict__ nm, float* __restrict__ state, const float* __restrict__ proj,
                   long long stride, const int* __restrict__ req_q_start, const int* __restrict__ req_slot, int H, int D,
                   int DV, float cap) {
  extern __shared__ __align__(16) float sh[];
  const int D4 = (D + 3) & ~3, LD = D4 + 4;
  float* Ss = sh;                          // [D4][COLS]
  float* Qb = Ss + D4 * COLS;              // [2][CT][LD]
  float* Kb = Qb + 2 * CT * LD;            // [2][CT][LD]
  float* Vb = Kb + 2 * CT * LD;            // [2][CT][COLS]
  float* Zb = Vb + 2 * CT * COLS;          // [2][2][CT]: z_i and z_f
  float* P = Zb + 4 * CT;                  // [CT][CT + 1]
  float* ns = P + CT * (CT + 1);           // [D4]
  float* av = ns + D4;                     // [CT] a_s
  float* gv = av + CT;                     // [CT] g_t
  float* mv = gv + CT;                     // [CT] m_t
  float* eg = mv + CT;                     // [CT] e^(m_0 - g_t)
  float* wv = eg + CT;                     // [CT] e^(a_s - g_C)
  float* den = wv + CT;                    // [CT]
  float* nq0 = den + CT;                   // [CT] n_0 . q_t (unscaled)
  float* carry = nq0 + CT;                 // [2] g_C and b_C
  pdl_trigger();
  const int c0 = blockIdx.x * COLS, h = blockIdx.y, r = blockIdx.z, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  constexpr int SUB = 32 / COLS;                     // groups of COLS lanes in a warp
  const int cl = lane % COLS, sg = lane / COLS;
  const int row0 = req_q_start[r], rows = req_q_start[r + 1] - row0, slot = req_slot[r];
  const MlstmCols col(H, D, DV);
  const int vcol = c0 + cl;
  const bool col_ok = vcol < DV;
  const float qscale = rsqrtf((float)D);
  const size_t head_floats = (size_t)D * DV + D + HEAD_EXTRA;
  float* S = state + ((size_t)slot * H + h) * head_floats;
  const float* n_g = S + (size_t)D * DV;
  pdl_wait();
  if (rows <= 0) return;

  // one chunk's rows on their way into buffer b: one group of copies per chunk
  auto fetch = [&](int t0, int b) {
    const int L = min(CT, rows - t0);
    float* Qd = Qb + b * CT * LD;
    float* Kd = Kb + b * CT * LD;
    for (int t = warp; t < CT; t += CWARPS) {          // a warp per row: no division by a size known only at run time
      const float* row = proj + (size_t)(row0 + t0 + min(t, L - 1)) * stride;
      const float* qsrc = row + col.q + h * D;
      const float* ksrc = row + col.k + h * D;
      for (int d = lane; d < D; d += 32) {
        cp_async_4(Qd + t * LD + d, qsrc + d, t < L);
        cp_async_4(Kd + t * LD + d, ksrc + d, t < L);
      }
    }
    for (int i = tid; i < CT * COLS; i += CTHREADS) {
      const int t = i / COLS, c = i - t * COLS;
      const bool live = t < L && c0 + c < DV;
      const float* row = proj + (size_t)(row0 + t0 + min(t, L - 1)) * stride;
      cp_async_4(Vb + b * CT * COLS + i, row + col.v + h * DV + (live ? c0 + c : 0), live);
    }
    if (tid < 2 * CT) {
      const int t = tid % CT, which = tid / CT;
      const float* row = proj + (size_t)(row0 + t0 + min(t, L - 1)) * stride;
      cp_async_4(Zb + b * 2 * CT + tid, row + (which ? col.f : col.i) + h, t < L);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(0, 0);
  for (int i = tid; i < D4 * COLS; i += CTHREADS) {
    const int d = i / COLS, c = i - d * COLS;
    Ss[i] = (d < D && c0 + c < DV) ? S[(size_t)d * DV + c0 + c] : 0.f;
  }
  for (int d = tid; d < D4; d += CTHREADS) ns[d] = d < D ? n_g[d] : 0.f;
  for (int i = tid; i < 2 * CT * (LD - D); i += CTHREADS) {        // the rows' padding is zero for good (the copies never touch it)
    const int t = i / (LD - D), d = D + i % (LD - D);
    Qb[t * LD + d] = 0.f;
    Kb[t * LD + d] = 0.f;
  }
  float m0 = n_g[D];
  int b = 0;
  for (int t0 = 0; t0 < rows; t0 += CT, b ^= 1) {
    const int L = min(CT, rows - t0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                    // this chunk's rows are there; the last chunk's readers are through; Ss and ns are up to date
    if (t0 + CT < rows) fetch(t0 + CT, b ^ 1);
    const float* Qs = Qb + b * CT * LD;
    const float* Ks = Kb + b * CT * LD;
    const float* Vs = Vb + b * CT * COLS;
    // The dot products q_t . k_s of the chunk (a thread per pair, kept in a register) do not wait for the gates:
    // warp 0 walks the gates meanwhile, the other warps also make n_0 . q_t.
    float pr[(CT * CT + CTHREADS - 1) / CTHREADS];
    if (warp == 0) {
      // lane t: the gates of token t; a prefix sum of f and a prefix maximum of a, in token order
      float ig = -INFINITY, fg = 0.f;
      if (lane < L) {
        ig = cap * tanhf(Zb[b * 2 * CT + lane] / cap);
        fg = log_sigmoid(cap * tanhf(Zb[b * 2 * CT + CT + lane] / cap));
      }
      float bsum = fg;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, bsum, o);
        if (lane >= o) bsum += up;
      }
      const float a = ig - bsum;                       // minus infinity past the portion's end
      float g = fmaxf(a, m0);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, g, o);
        if (lane >= o) g = fmaxf(g, up);
      }
      const float gC = __shfl_sync(0xffffffffu, g, CT - 1), bC = __shfl_sync(0xffffffffu, bsum, CT - 1);
      if (lane < CT) {
        av[lane] = a; gv[lane] = g; mv[lane] = bsum + g;
        eg[lane] = expf(m0 - g);
        wv[lane] = expf(a - gC);
      }
      if (lane == 0) { carry[0] = gC; carry[1] = bC; }
    }
#pragma unroll
    for (int k = 0; k < (CT * CT + CTHREADS - 1) / CTHREADS; ++k) {
      const int i = tid + k * CTHREADS, t = i / CT, s = i - t * CT;
      float dotp = 0.f;
      if (i < CT * CT && s <= t && t < L) {
        const float4* qr = reinterpret_cast<const float4*>(Qs + t * LD);
        const float4* kr = reinterpret_cast<const float4*>(Ks + s * LD);
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll 4
        for (int d = 0; d < D4 / 4; ++d) {
          const float4 x = qr[d], y = kr[d];
          d0 = fmaf(x.x, y.x, d0); d1 = fmaf(x.y, y.y, d1); d2 = fmaf(x.z, y.z, d2); d3 = fmaf(x.w, y.w, d3);
        }
        dotp = ((d0 + d1) + (d2 + d3)) * qscale;
      }
      pr[k] = dotp;
    }
    if (warp > 0) {
      for (int t = warp - 1; t < CT; t += CWARPS - 1) {          // n_0 . q_t
        float dotp = 0.f;
        for (int d = lane; d < D; d += 32) dotp = fmaf(ns[d], Qs[t * LD + d], dotp);
        dotp = warp_sum(dotp);
        if (lane == 0) nq0[t] = dotp;
      }
    }
    __syncthreads();
    // the pairs' weights, and each token's denominator from the sum of its row (CT lanes side by side hold a row)
#pragma unroll
    for (int k = 0; k < (CT * CT + CTHREADS - 1) / CTHREADS; ++k) {
      const int i = tid + k * CTHREADS, t = i / CT, s = i - t * CT;
      const bool live = i < CT * CT && s <= t && t < L;
      const float p = live ? pr[k] * expf(av[s] - gv[t]) : 0.f;
      if (i < CT * CT) P[t * (CT + 1) + s] = p;
      float sum = p;
#pragma unroll
      for (int o = CT / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (i < CT * CT && s == 0) den[t] = fmaxf(fabsf(fmaf(eg[t] * qscale, nq0[t], sum)), expf(-mv[t])) + 1e-6f;
    }
    __syncthreads();
    // o_t for the tokens of this group of lanes, a lane per value column: four rows of S and the tokens' q four at a
    // time, a sum of its own for each of the four so that no product waits for the one before it
    constexpr int TPW = CT / CWARPS, TPS = TPW / SUB;
    static_assert(TPS >= 1, "a chunk has at least one token per group of lanes");
    const int tok0 = warp * TPW + sg * TPS;
    float acc[TPS][4];
#pragma unroll
    for (int j = 0; j < TPS; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll 2
    for (int d = 0; d < D4; d += 4) {
      const float s0 = Ss[d * COLS + cl], s1 = Ss[(d + 1) * COLS + cl], s2 = Ss[(d + 2) * COLS + cl], s3 = Ss[(d + 3) * COLS + cl];
#pragma unroll
      for (int j = 0; j < TPS; ++j) {
        const float4 q4 = *reinterpret_cast<const float4*>(Qs + (tok0 + j) * LD + d);
        acc[j][0] = fmaf(q4.x, s0, acc[j][0]); acc[j][1] = fmaf(q4.y, s1, acc[j][1]);
        acc[j][2] = fmaf(q4.z, s2, acc[j][2]); acc[j][3] = fmaf(q4.w, s3, acc[j][3]);
      }
    }
    float o_t[TPS];
#pragma unroll
    for (int j = 0; j < TPS; ++j) {
      const int t = tok0 + j;
      float o = eg[t] * qscale * ((acc[j][0] + acc[j][1]) + (acc[j][2] + acc[j][3]));
      for (int s = 0; s <= t; ++s) o = fmaf(P[t * (CT + 1) + s], Vs[s * COLS + cl], o);
      o_t[j] = o;
    }
    float vw[CT];                                      // this column's values, each times what its token writes
#pragma unroll
    for (int u = 0; u < CT; ++u) vw[u] = wv[u] * Vs[u * COLS + cl];
#pragma unroll
    for (int j = 0; j < TPS; ++j) {
      const int t = tok0 + j;
      if (t < L && col_ok) raw[(size_t)(row0 + t0 + t) * H * DV + h * DV + vcol] = o_t[j] / den[t];
    }
    __syncthreads();                                   // every read of Ss and ns is done
    const float gC = carry[0], bC = carry[1];
    const float keep = expf(m0 - gC);
    for (int d = (warp * SUB + sg) * 4; d < D4; d += CWARPS * SUB * 4) {  // four rows of S at a time
      float s0 = keep * Ss[d * COLS + cl], s1 = keep * Ss[(d + 1) * COLS + cl];
      float s2 = keep * Ss[(d + 2) * COLS + cl], s3 = keep * Ss[(d + 3) * COLS + cl];
#pragma unroll
      for (int u = 0; u < CT; ++u) {
        const float4 k4 = *reinterpret_cast<const float4*>(Ks + u * LD + d);
        s0 = fmaf(k4.x, vw[u], s0); s1 = fmaf(k4.y, vw[u], s1); s2 = fmaf(k4.z, vw[u], s2); s3 = fmaf(k4.w, vw[u], s3);
      }
      Ss[d * COLS + cl] = s0; Ss[(d + 1) * COLS + cl] = s1; Ss[(d + 2) * COLS + cl] = s2; Ss[(d + 3) * COLS + cl] = s3;
    }
    for (int d = tid; d < D; d += CTHREADS) {
      float nd = keep * ns[d];
#pragma unroll
      for (int u = 0; u < CT; ++u) nd = fmaf(wv[u], Ks[u * LD + d], nd);
      ns[d] = nd;
    }
    m0 = bC + gC;
  }
  __syncthreads();
  for (int i = tid; i < D * COLS; i += CTHREADS) {
    const int d = i / COLS, c = i - d * COLS;
    if (c0 + c < DV) S[(size_t)d * DV + c0 + c] = Ss[i];
  }
  if (blockIdx.x == 0) {
    float* dst = nm + ((size_t)r * H + h) * (D + 1);
    for (int d = tid; d < D; d += CTHREADS) dst[d] = ns[d];
    if (tid == 0) dst[D] = m0;
  }
}

// Block (row, head): out = raw / rms(raw) * w * sigmoid(gate) over the head's DV numbers; the block of a
// request's first row also files the head's n and m from the scratch buffer into the state.
template <typename C>
__global__ void __launch_bounds__(128)
mlstm_finish_kernel(C* __restrict__ out, float* __restrict__ state, const float* __restrict__ raw, const float* __restrict__ nm,
                    const float* __restrict__ proj, long long stride, const float* __restrict__ norm_w,
                    const int* __restrict__ row_req, const int* __restrict__ req_q_start, const int* __restrict__ req_slot,
                    int H, int D, int DV, float eps) {
  __shared__ float red[32];
  pdl_trigger();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int r = row_req[t];
  const bool first = req_q_start[r] == t;
  const int slot = req_slot[r];
  const MlstmCols col(H, D, DV);
  pdl_wait();
  const float* src = raw + (size_t)t * H * DV + h * DV;
  float ss = 0.f;
  for (int c = tid; c < DV; c += blockDim.x) ss = fmaf(src[c], src[c], ss);
  const float inv = 1.0f / sqrtf(block_sum_any(ss, red) / (float)DV + eps);
  const float* gate = proj + (size_t)t * stride + col.g + h * DV;
  for (int c = tid; c < DV; c += blockDim.x)
    out[(size_t)t * H * DV + h * DV + c] = from_float<C>(src[c] * inv * norm_w[h * DV + c] / (1.0f + expf(-gate[c])));
  if (first) {
    const size_t head_floats = (size_t)D * DV + D + HEAD_EXTRA;
    float* n_g = state + ((size_t)slot * H + h) * head_floats + (size_t)D * DV;
    const float* from = nm + ((size_t)r * H + h) * (D + 1);
    for (int d = tid; d <= D; d += blockDim.x) n_g[d] = from[d];
  }
}

constexpr int CHUNK_TOKENS = 16;

size_t chunk_smem(int D) { return chunk_floats(D, CHUNK_TOKENS, 32) * sizeof(float); }

}  // namespace

static int g_slice_cols = 0;
// Value columns per block of the chunked form: 0 the library decides per launch (default), 16 or 32 always.
AYK_EXPORT void ayk_mlstm_slice_cols(int cols) { g_slice_cols = (cols == 16 || cols == 32) ? cols : 0; }

// Floats of one head's state (S, n, m and padding) and of the whole per-request state [H][...].
AYK_EXPORT int ayk_mlstm_head_floats(int D, int DV) { return D * DV + D + HEAD_EXTRA; }

// Whether the chunked form takes these sizes (its shared memory holds 32 columns of S and a chunk's q and k).
AYK_EXPORT int ayk_mlstm_chunk_takes(int D) { return chunk_smem(D) <= 200 * 1024; }

// Floats of the scratch that the chunked form needs: raw [T, H * DV] and nm [requests, H, D + 1].
AYK_EXPORT long long ayk_mlstm_scratch_floats(int T, int num_req, int H, int D, int DV) {
  return (long long)T * H * DV + (long long)num_req * H * (D + 1);
}

// out [T, H * DV] in out_dtype; state [slots, H, D * DV + D + 4] float32; proj float32 rows of ``stride``
// [q | k | v | z_i | z_f | gate]; norm_w [H * DV] float32.  scratch null: the walk, token by token (one
// launch; values of up to 256 numbers); else the chunked form and its finishing kernel (two launches; any vdim).
AYK_EXPORT int ayk_mlstm(void* out, float* state, const float* proj, long long stride, const float* norm_w, const int* row_req,
                         const int* req_q_start, const int* req_slot, int num_req, int T, int H, int D, int DV, float cap,
                         float eps, float* scratch, int out_dtype, cudaStream_t stream) {
  if (T == 0 || num_req == 0) return 0;
  AYK_REQUIRE(D >= 1 && DV >= 1 && H >= 1 && H <= 65535, "ayk_mlstm: %d heads of %d x %d", H, D, DV);
  AYK_REQUIRE(scratch || DV <= 256, "ayk_mlstm: the token-by-token kernel takes values of up to 256 numbers, not %d", DV);
  AYK_REQUIRE(cap > 0.f, "ayk_mlstm: the gates' cap must be positive");
  AYK_REQUIRE(out_dtype == AYK_DTYPE_F32 || out_dtype == AYK_DTYPE_BF16, "ayk_mlstm: unknown dtype %d", out_dtype);
  if (!scratch) {
    const int VP = (DV + 31) & ~31;
    const size_t smem = ((size_t)3 * D + (size_t)(WALK_THREADS / VP) * VP) * sizeof(float);
    AYK_REQUIRE(smem <= 200 * 1024, "ayk_mlstm: heads of %d numbers do not fit shared memory", D);
    cudaError_t err = cudaSuccess;
    static AykPerDevice configured[2];
    if (out_dtype == AYK_DTYPE_F32) {
      if (smem > 48 * 1024 && !configured[0].here()) {
        err = cudaFuncSetAttribute(mlstm_walk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        configured[0].here() = true;
      }
      if (err != cudaSuccess) return ayk_fail("ayk_mlstm: shared memory: %s", cudaGetErrorString(err));
      ayk_launch(mlstm_walk_kernel<float>, dim3(num_req, H), dim3(WALK_THREADS), smem, stream, (float*)out, state, proj, stride, norm_w,
                 req_q_start, req_slot, H, D, DV, cap, eps);
    } else {
      if (smem > 48 * 1024 && !configured[1].here()) {
        err = cudaFuncSetAttribute(mlstm_walk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        configured[1].here() = true;
      }
      if (err != cudaSuccess) return ayk_fail("ayk_mlstm: shared memory: %s", cudaGetErrorString(err));
      ayk_launch(mlstm_walk_kernel<__nv_bfloat16>, dim3(num_req, H), dim3(WALK_THREADS), smem, stream, (__nv_bfloat16*)out, state, proj,
                 stride, norm_w, req_q_start, req_slot, H, D, DV, cap, eps);
    }
    return ayk_check_launch("ayk_mlstm");
  }
  AYK_REQUIRE(ayk_mlstm_chunk_takes(D), "ayk_mlstm: the chunked form does not take heads of %d numbers", D);
  AYK_REQUIRE(num_req <= 65535, "ayk_mlstm: %d requests", num_req);
  float* raw = scratch;
  float* nm = scratch + (size_t)T * H * DV;
  // slices of 32 value columns, or of 16 where those would leave most SMs without a block
  const bool narrow = g_slice_cols ? g_slice_cols == 16
                                   : ((long long)((DV + 31) / 32) * H * num_req * 4 < (long long)ayk_sm_count() * 3 && DV > 16);
  const size_t smem = chunk_floats(D, CHUNK_TOKENS, narrow ? 16 : 32) * sizeof(float);
  static AykPerDevice chunk_configured[2];
  if (smem > 48 * 1024 && !chunk_configured[narrow].here()) {
    cudaError_t err = narrow ? cudaFuncSetAttribute(mlstm_chunk_kernel<CHUNK_TOKENS, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                             : cudaFuncSetAttribute(mlstm_chunk_kernel<CHUNK_TOKENS, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (err != cudaSuccess) return ayk_fail("ayk_mlstm: shared memory: %s", cudaGetErrorString(err));
    chunk_configured[narrow].here() = true;
  }
  if (narrow)
    ayk_launch(mlstm_chunk_kernel<CHUNK_TOKENS, 16>, dim3((DV + 15) / 16, H, num_req), dim3(CTHREADS), smem, stream, raw, nm,
               state, proj, stride, req_q_start, req_slot, H, D, DV, cap);
  else
    ayk_launch(mlstm_chunk_kernel<CHUNK_TOKENS, 32>, dim3((DV + 31) / 32, H, num_req), dim3(CTHREADS), smem, stream, raw, nm,
               state, proj, stride, req_q_start, req_slot, H, D, DV, cap);
  if (out_dtype == AYK_DTYPE_F32)
    ayk_launch(mlstm_finish_kernel<float>, dim3(T, H), dim3(128), 0, stream, (float*)out, state, (const float*)raw, (const float*)nm,
               proj, stride, norm_w, row_req, req_q_start, req_slot, H, D, DV, eps);
  else
    ayk_launch(mlstm_finish_kernel<__nv_bfloat16>, dim3(T, H), dim3(128), 0, stream, (__nv_bfloat16*)out, state, (const float*)raw,
               (const float*)nm, proj, stride, norm_w, row_req, req_q_start, req_slot, H, D, DV, eps);
  return ayk_check_launch("ayk_mlstm");
}
