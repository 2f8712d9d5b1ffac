// Mixture of experts: routing, the plan of a step's (token, choice) pairs sorted by expert, the
// grouped products over the sorted rows, the gated activation and the weighted sum.
//
// Routing: the ``top`` largest of a token's router logits (the lower index wins a tie), weights =
// softmax over the chosen logits only; all 32-bit.  Nothing of the routing goes to the host: the
// plan kernel counts the pairs of every expert, lays them out expert by expert (``sorted``: place
// -> pair), and cuts them into tiles of TILE_ROWS rows of one expert each; the grouped product is
// launched with the largest number of tiles that the pair count allows and its surplus blocks leave.
//
// An expert's activation: g = min(gate, limit), u = clamp(up, -limit, limit),
// y = g * sigmoid(slope * g) * (u + plus).  An infinite limit clamps nothing; slope 1 and plus 0 make it
// silu(gate) * up.
//
// Routing by sigmoid scores in groups (moe_route_scored_kernel): s = sigmoid(z); experts are ranked by
// s + correction[e]; the experts are ``groups`` equal runs of consecutive experts, a run's score is the sum of its
// two largest ranking scores, and only experts of the ``keep`` best runs can be chosen; the weights are
// the chosen s divided by their sum, times a factor.
#include <math.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }

__device__ __forceinline__ float glu_limited(float g, float u, float limit, float slope, float plus) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoidf(slope * g) * (u + plus);
}

constexpr int MAX_TOP = 16;
constexpr int TILE_ROWS = 32;

// ------------------------------------------------------------------- route --
// A warp per token.
__global__ void __launch_bounds__(128)
moe_route_kernel(int* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ logits, long long stride,
                 int T, int E, int top) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* z = logits + (size_t)t * stride;
  int chosen[MAX_TOP];
  float value[MAX_TOP];
#pragma unroll
  for (int k = 0; k < MAX_TOP; ++k) {
    if (k >= top) break;
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = false;
#pragma unroll
      for (int j = 0; j < MAX_TOP; ++j) taken |= (j < k && chosen[j] == e);
      const float v = z[e];
      if (!taken && (v > best || (v == best && e < at) || at == 0x7fffffff)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
    }
    chosen[k] = at;
    value[k] = best;
  }
  if (lane == 0) {
    float sum = 0.f, w[MAX_TOP];
#pragma unroll
    for (int k = 0; k < MAX_TOP; ++k) {
      if (k >= top) break;
      w[k] = expf(value[k] - value[0]);          // value[0] is the largest
      sum += w[k];
    }
#pragma unroll
    for (int k = 0; k < MAX_TOP; ++k) {
      if (k >= top) break;
      ids[(size_t)t * top + k] = chosen[k];
      weights[(size_t)t * top + k] = w[k] / sum;
    }
  }
}

// A warp per token.  Lane g holds the score of run g (at most 32 runs); the runs that may be chosen are a
// bit mask that every lane holds; then the same repeated arg-max as above over the allowed experts' ranking
// scores (the lower index wins a tie).
__global__ void __launch_bounds__(128)
moe_route_scored_kernel(int* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ logits, long long stride,
                        const float* __restrict__ correction, int T, int E, int top, int groups, int keep, float factor) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* z = logits + (size_t)t * stride;
  const int per = E / groups;
  unsigned allowed = 0xffffffffu;
  if (keep < groups) {
    float mine = -INFINITY;                    // lane g: the sum of run g's two largest ranking scores
    for (int g = 0; g < groups; ++g) {
      float best = -INFINITY, second = -INFINITY;
      for (int e = g * per + lane; e < (g + 1) * per; e += 32) {
        const float v = sigmoidf(z[e]) + (correction ? correction[e] : 0.f);
        if (v > best) { second = best; best = v; } else if (v > second) second = v;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, second, o);
        const float hi = fmaxf(best, ob), lo = fminf(best, ob);
        second = fmaxf(lo, fmaxf(second, os));
        best = hi;
      }
      const float score = per > 1 ? best + second : best;
      if (lane == g) mine = score;
    }
    int rank = 0;                              // runs that come before mine: a larger score, or the same and a lower index
    for (int g = 0; g < groups; ++g) {
      const float other = __shfl_sync(0xffffffffu, mine, g);
      rank += (other > mine || (other == mine && g < lane)) ? 1 : 0;
    }
    allowed = __ballot_sync(0xffffffffu, lane < groups && rank < keep);
  }
  int chosen[MAX_TOP];
  float value[MAX_TOP];
#pragma unroll
  for (int k = 0; k < MAX_TOP; ++k) {
    if (k >= top) break;
    float best = -INFINITY, best_s = 0.f;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = !((allowed >> (e / per)) & 1u);
#pragma unroll
      for (int j = 0; j < MAX_TOP; ++j) taken |= (j < k && chosen[j] == e);
      const float sc = sigmoidf(z[e]);
      const float v = sc + (correction ? correction[e] : 0.f);
      if (!taken && (v > best || (v == best && e < at) || at == 0x7fffffff)) { best = v; at = e; best_s = sc; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const float osc = __shfl_xor_sync(0xffffffffu, best_s, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; best_s = osc; }
    }
    chosen[k] = at;
    value[k] = best_s;
  }
  if (lane == 0) {
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < MAX_TOP; ++k) {
      if (k >= top) break;
      sum += value[k];
    }
    const float inv = factor / (sum + 1e-20f);
#pragma unroll
    for (int k = 0; k < MAX_TOP; ++k) {
      if (k >= top) break;
      ids[(size_t)t * top + k] = chosen[k];
      weights[(size_t)t * top + k] = value[k] * inv;
    }
  }
}

// -------------------------------------------------------------------- plan --
// One block.  tiles[0] = number of tiles; tile i: expert tiles[1 + 3 i], first sorted row
// tiles[2 + 3 i], rows tiles[3 + 3 i].
__global__ void __launch_bounds__(1024)
moe_plan_kernel(int* __restrict__ sorted, int* __restrict__ tiles, const int* __restrict__ ids, int P, int E) {
  extern __shared__ int sh[];
  int* count = sh;          // [E]
  int* start = sh + E;      // [E]
  int* cursor = sh + 2 * E; // [E]
  pdl_trigger();
  for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
  pdl_wait();
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&count[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, n = 0;
    for (int e = 0; e < E; ++e) {
      const int c = count[e];
      start[e] = off;
      for (int r = 0; r < c; r += TILE_ROWS) {
        tiles[1 + 3 * n] = e;
        tiles[2 + 3 * n] = off + r;
        tiles[3 + 3 * n] = min(TILE_ROWS, c - r);
        ++n;
      }
      off += c;
    }
    tiles[0] = n;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = ids[p];
    sorted[start[e] + atomicAdd(&cursor[e], 1)] = p;     // a row's result does not depend on its place
  }
}

// The plan for the product that runs on tcgen05 (gemm_tc_prefill, grouped form): every expert's pairs
// start at a multiple of PAD_ROWS rows, so that each 128-row tile of the gathered rows belongs to one
// expert.  row_of_pair[p]: the pair's row in that layout; w_rows1 / w_rows2 [max_tiles]: per tile the first
// weight row of its expert in the two stacked weights (n1 and n2 rows per expert; 0 for tiles past the end).
constexpr int PAD_ROWS = 128;

__global__ void __launch_bounds__(1024)
moe_plan_padded_kernel(int* __restrict__ row_of_pair, int* __restrict__ w_rows1, int* __restrict__ w_rows2,
                       const int* __restrict__ ids, int P, int E, int n1, int n2, int max_tiles) {
  extern __shared__ int sh[];
  int* count = sh;          // [E]
  int* start = sh + E;      // [E]
  int* cursor = sh + 2 * E; // [E]
  pdl_trigger();
  for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
  pdl_wait();
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&count[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = n * PAD_ROWS;
      for (int r = 0; r < count[e]; r += PAD_ROWS) {
        if (n < max_tiles) { w_rows1[n] = e * n1; w_rows2[n] = e * n2; }
        ++n;
      }
    }
    for (; n < max_tiles; ++n) { w_rows1[n] = 0; w_rows2[n] = 0; }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = ids[p];
    row_of_pair[p] = start[e] + atomicAdd(&cursor[e], 1);     // a row's result does not depend on its place
  }
}

// out[row_of_pair[p], :] = in[p / top, :], bfloat16 rows of d elements (d a multiple of 8); a warp per pair.
__global__ void __launch_bounds__(256)
moe_gather_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ in, long long in_stride,
                  const int* __restrict__ row_of_pair, int P, int top, int d) {
  pdl_trigger();
  pdl_wait();
  const int p = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (p >= P) return;
  const uint4* src = reinterpret_cast<const uint4*>(in + (size_t)(p / top) * in_stride);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row_of_pair[p] * d);
  for (int i = lane; i < d / 8; i += 32) dst[i] = src[i];
}

// --------------------------------------------------------- grouped product --
// out[o(s), n] = sum_k a[r(s), k] * w[expert, n, k] over the sorted rows s of a tile; w holds N_w
// rows per expert.  GLU: w rows [0, N) are the gate, [N, 2N) the up projection, and the output is
// the activation of the pair.  gather: r(s) = sorted[s] / top (rows of tokens), else s.  scatter:
// o(s) = sorted[s] (the pair's own row), else s.  On the FP32 pipes with 32-bit sums.
constexpr int BN = 64, BK = 32;

template <typename T, typename O, bool GLU>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(O* __restrict__ out, const T* __restrict__ a, long long a_stride, const T* __restrict__ w,
                const int* __restrict__ sorted, const int* __restrict__ tiles, int top, int gather, int scatter, int N,
                int N_w, int Kd, float limit, float slope, float plus) {
  __shared__ float As[BK][TILE_ROWS + 1];
  __shared__ float Bs[GLU ? 2 : 1][BK][BN + 1];
  __shared__ int a_row[TILE_ROWS], o_row[TILE_ROWS];
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.x >= tiles[0]) return;
  const int e = tiles[1 + 3 * blockIdx.x], s0 = tiles[2 + 3 * blockIdx.x], rows = tiles[3 + 3 * blockIdx.x];
  const int n0 = blockIdx.y * BN;
  const int tid = threadIdx.x;
  if (tid < TILE_ROWS) {
    const int pair = tid < rows ? sorted[s0 + tid] : -1;
    a_row[tid] = tid < rows ? (gather ? pair / top : s0 + tid) : -1;
    o_row[tid] = tid < rows ? (scatter ? pair : s0 + tid) : -1;
  }
  __syncthreads();
  const T* we = w + (size_t)e * N_w * Kd;
  const int ty = tid >> 4, tx = tid & 15;        // rows ty * 2 + {0, 1}; columns tx + 16 * {0 .. 3}
  float acc[GLU ? 2 : 1][2][4];
#pragma unroll
  for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;

  for (int k0 = 0; k0 < Kd; k0 += BK) {
    {   // A: 32 rows x 32 k
      const int kk = tid & 31;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = (tid >> 5) + 8 * i;
        const int src = a_row[r];
        As[kk][r] = (src >= 0 && k0 + kk < Kd) ? to_float<T>(a[(size_t)src * a_stride + k0 + kk]) : 0.f;
      }
    }
#pragma unroll
    for (int g = 0; g < (GLU ? 2 : 1); ++g) {   // B: 64 n x 32 k
      const int kk = tid & 31;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int n = (tid >> 5) + 8 * i;
        Bs[g][kk][n] = (n0 + n < N && k0 + kk < Kd) ? to_float<T>(we[(size_t)(g * N + n0 + n) * Kd + k0 + kk]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < BK; ++kk) {
      const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
#pragma unroll
      for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float b = Bs[g][kk][tx + 16 * j];
          acc[g][0][j] = fmaf(a0, b, acc[g][0][j]);
          acc[g][1][j] = fmaf(a1, b, acc[g][1][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int dst = o_row[ty * 2 + i];
    if (dst < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= N) continue;
      const float v = GLU ? glu_limited(acc[0][i][j], acc[GLU ? 1 : 0][i][j], limit, slope, plus) : acc[0][i][j];
      out[(size_t)dst * N + n] = from_float<O>(v);
    }
  }
}

// ------------------------------------- grouped product on the tensor cores --
// The same for bfloat16 operands: a tile of 32 sorted rows x 64 columns per block of four warps, each
// warp 32 rows x 16 columns as 2 x 2 fragments of mma.sync m16n8k16 with float32 sums; operands pass
// through shared memory as they lie in global memory (k innermost, rows padded by 8 elements so that
// a fragment's loads fall into different banks).
constexpr int TK = 64;                 // k per stage
constexpr int TLD = TK + 8;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename O, bool GLU>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(O* __restrict__ out, const __nv_bfloat16* __restrict__ a, long long a_stride,
                    const __nv_bfloat16* __restrict__ w, const int* __restrict__ sorted, const int* __restrict__ tiles,
                    int top, int gather, int scatter, int N, int N_w, int Kd, float limit, float slope, float plus) {
  __shared__ __align__(16) __nv_bfloat16 As[TILE_ROWS][TLD];
  __shared__ __align__(16) __nv_bfloat16 Bs[GLU ? 2 : 1][BN][TLD];
  __shared__ int a_row[TILE_ROWS], o_row[TILE_ROWS];
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.x >= tiles[0]) return;
  const int e = tiles[1 + 3 * blockIdx.x], s0 = tiles[2 + 3 * blockIdx.x], rows = tiles[3 + 3 * blockIdx.x];
  const int n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < TILE_ROWS) {
    const int pair = tid < rows ? sorted[s0 + tid] : -1;
    a_row[tid] = tid < rows ? (gather ? pair / top : s0 + tid) : -1;
    o_row[tid] = tid < rows ? (scatter ? pair : s0 + tid) : -1;
  }
  __syncthreads();
  const __nv_bfloat16* we = w + (size_t)e * N_w * Kd;
  float acc[GLU ? 2 : 1][2][2][4];
#pragma unroll
  for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[g][i][j][c] = 0.f;
  const int gid = lane >> 2, tig = lane & 3;
  const uint4 zero = make_uint4(0, 0, 0, 0);

  for (int k0 = 0; k0 < Kd; k0 += TK) {
    // 16-byte pieces: a row of TK elements is 8 pieces (Kd is a multiple of 8)
    for (int i = tid; i < TILE_ROWS * (TK / 8); i += 128) {
      const int r = i >> 3, piece = i & 7;
      const int src = a_row[r], k = k0 + piece * 8;
      uint4 v = zero;
      if (src >= 0 && k < Kd) v = *reinterpret_cast<const uint4*>(a + (size_t)src * a_stride + k);
      *reinterpret_cast<uint4*>(&As[r][piece * 8]) = v;
    }
#pragma unroll
    for (int g = 0; g < (GLU ? 2 : 1); ++g)
      for (int i = tid; i < BN * (TK / 8); i += 128) {
        const int n = i >> 3, piece = i & 7;
        const int k = k0 + piece * 8;
        uint4 v = zero;
        if (n0 + n < N && k < Kd) v = *reinterpret_cast<const uint4*>(we + (size_t)(g * N + n0 + n) * Kd + k);
        *reinterpret_cast<uint4*>(&Bs[g][n][piece * 8]) = v;
      }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const __nv_bfloat16* base = &As[i * 16 + gid][kk + tig * 2];
        af[i][0] = *reinterpret_cast<const uint32_t*>(base);
        af[i][1] = *reinterpret_cast<const uint32_t*>(base + 8 * TLD);
        af[i][2] = *reinterpret_cast<const uint32_t*>(base + 8);
        af[i][3] = *reinterpret_cast<const uint32_t*>(base + 8 * TLD + 8);
      }
#pragma unroll
      for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const __nv_bfloat16* base = &Bs[g][warp * 16 + j * 8 + gid][kk + tig * 2];
          uint32_t bf[2];
          bf[0] = *reinterpret_cast<const uint32_t*>(base);
          bf[1] = *reinterpret_cast<const uint32_t*>(base + 8);
#pragma unroll
          for (int i = 0; i < 2; ++i) mma_bf16(acc[g][i][j], af[i], bf);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int dst = o_row[i * 16 + gid + half * 8];
      if (dst < 0) continue;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + warp * 16 + j * 8 + tig * 2 + c;
          if (n >= N) continue;
          const float v0 = acc[0][i][j][half * 2 + c];
          const float v = GLU ? glu_limited(v0, acc[GLU ? 1 : 0][i][j][half * 2 + c], limit, slope, plus) : v0;
          out[(size_t)dst * N + n] = from_float<O>(v);
        }
    }
}

// --------------------------------------------- few pairs: matrix times vector --
// A step of single tokens has a handful of (token, choice) pairs, most on experts of their own: each pair
// then streams its expert's matrix once, and the product is bound by that stream.  A block takes one pair and
// 64 output features; the pair's activation row waits in shared memory as float32; a warp takes 8 features, two
// at a time, its lanes striding along K in 16-byte pieces of the weight rows (with the activation, both the gate
// row and the up row of a feature).  No sorting: pair p reads row p / top (gather) or p, and writes row p.
constexpr int GV_COLS = 64;

__device__ __forceinline__ float dot8(const uint4& w, const float4& x0, const float4& x1) {
  // a bfloat16 is the upper half of a float
  float s = __uint_as_float(w.x << 16) * x0.x;
  s = fmaf(__uint_as_float(w.x & 0xffff0000u), x0.y, s);
  s = fmaf(__uint_as_float(w.y << 16), x0.z, s);
  s = fmaf(__uint_as_float(w.y & 0xffff0000u), x0.w, s);
  s = fmaf(__uint_as_float(w.z << 16), x1.x, s);
  s = fmaf(__uint_as_float(w.z & 0xffff0000u), x1.y, s);
  s = fmaf(__uint_as_float(w.w << 16), x1.z, s);
  return fmaf(__uint_as_float(w.w & 0xffff0000u), x1.w, s);
}

template <typename O, bool GLU>
__global__ void __launch_bounds__(256)
moe_gemv_kernel(O* __restrict__ out, const __nv_bfloat16* __restrict__ a, long long a_stride,
                const __nv_bfloat16* __restrict__ w, const int* __restrict__ ids, int top, int gather, int N, int N_w,
                int Kd, float limit, float slope, float plus) {
  extern __shared__ __align__(16) float act[];          // [Kd]
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const __nv_bfloat16* arow = a + (size_t)(gather ? pair / top : pair) * a_stride;
  for (int i = tid; i < Kd / 8; i += 256) {
    const uint4 v = *reinterpret_cast<const uint4*>(arow + i * 8);
    float4 lo, hi;
    lo.x = __uint_as_float(v.x << 16); lo.y = __uint_as_float(v.x & 0xffff0000u);
    lo.z = __uint_as_float(v.y << 16); lo.w = __uint_as_float(v.y & 0xffff0000u);
    hi.x = __uint_as_float(v.z << 16); hi.y = __uint_as_float(v.z & 0xffff0000u);
    hi.z = __uint_as_float(v.w << 16); hi.w = __uint_as_float(v.w & 0xffff0000u);
    *reinterpret_cast<float4*>(act + i * 8) = lo;
    *reinterpret_cast<float4*>(act + i * 8 + 4) = hi;
  }
  __syncthreads();
  const __nv_bfloat16* we = w + (size_t)ids[pair] * N_w * Kd;
  const int first = blockIdx.y * GV_COLS + warp * 8;
#pragma unroll 1
  for (int j = 0; j < 8; j += 2) {
    const int n0 = first + j, n1 = n0 + 1;               // warp-uniform
    if (n0 >= N) break;
    const bool two = n1 < N;
    float g0 = 0.f, g1 = 0.f, u0 = 0.f, u1 = 0.f;
    const __nv_bfloat16* r0 = we + (size_t)n0 * Kd;
    const __nv_bfloat16* r1 = we + (size_t)(two ? n1 : n0) * Kd;
    for (int k = lane * 8; k < Kd; k += 256) {
      const float4 x0 = *reinterpret_cast<const float4*>(act + k), x1 = *reinterpret_cast<const float4*>(act + k + 4);
      const uint4 wa = *reinterpret_cast<const uint4*>(r0 + k), wb = *reinterpret_cast<const uint4*>(r1 + k);
      if (GLU) {
        const uint4 wc = *reinterpret_cast<const uint4*>(r0 + (size_t)N * Kd + k), wd = *reinterpret_cast<const uint4*>(r1 + (size_t)N * Kd + k);
        u0 += dot8(wc, x0, x1);
        u1 += dot8(wd, x0, x1);
      }
      g0 += dot8(wa, x0, x1);
      g1 += dot8(wb, x0, x1);
    }
    g0 = warp_sum(g0); g1 = warp_sum(g1);
    if (GLU) { u0 = warp_sum(u0); u1 = warp_sum(u1); }
    if (lane == 0) {
      out[(size_t)pair * N + n0] = from_float<O>(GLU ? glu_limited(g0, u0, limit, slope, plus) : g0);
      if (two) out[(size_t)pair * N + n1] = from_float<O>(GLU ? glu_limited(g1, u1, limit, slope, plus) : g1);
    }
  }
}

// ------------------------------------------------- activation and weighted sum --
// out[t, c] = act(in[t, c], in[t, n + c]) for the dense (shared) expert.
template <typename I, typename O>
__global__ void __launch_bounds__(256)
glu_limited_kernel(O* __restrict__ out, const I* __restrict__ in, long long stride, int n, float limit, float slope, float plus) {
  pdl_trigger();
  pdl_wait();
  const I* row = in + (size_t)blockIdx.x * stride;
  for (int c = threadIdx.x; c < n; c += blockDim.x)
    out[(size_t)blockIdx.x * n + c] = from_float<O>(glu_limited(to_float<I>(row[c]), to_float<I>(row[n + c]), limit, slope, plus));
}

// shared[t, :] = sum_k weights[t, k] * picked[row of pair t * top + k, :] + sigmoid(mix[t]) * shared[t, :], the
// chosen experts in the order of their choice; row_of_pair null: the pair's own number.
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ shared, const float* __restrict__ picked, const int* __restrict__ row_of_pair,
                   const float* __restrict__ weights, const float* __restrict__ mix, long long mix_stride, int top, int d) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float gate = mix ? sigmoidf(mix[(size_t)t * mix_stride]) : 1.0f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
      const size_t pair = (size_t)t * top + k;
      s = fmaf(weights[pair], picked[(size_t)(row_of_pair ? row_of_pair[pair] : pair) * d + c], s);
    }
    shared[(size_t)t * d + c] = fmaf(gate, shared[(size_t)t * d + c], s);
  }
}

}  // namespace

AYK_EXPORT int ayk_moe_tile_rows() { return TILE_ROWS; }

// ids, weights [T, top]; sorted [T * top]; tiles [1 + 3 * (T * top / TILE_ROWS + E)].  Two launches.
AYK_EXPORT int ayk_moe_route(int* ids, float* weights, int* sorted, int* tiles, const float* logits, long long stride,
                             int T, int E, int top, cudaStream_t stream) {
  if (T == 0) return 0;
  AYK_REQUIRE(top >= 1 && top <= MAX_TOP && top <= E, "ayk_moe_route: top %d of %d experts (at most %d)", top, E, MAX_TOP);
  AYK_REQUIRE(E <= 4096, "ayk_moe_route: %d experts (at most 4096)", E);
  ayk_launch(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, ids, weights, logits, stride, T, E, top);
  ayk_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), stream, sorted, tiles, (const int*)ids,
             T * top, E);
  return ayk_check_launch("ayk_moe_route");
}

// The same plan after routing by sigmoid scores in groups (see the head of the file).  correction [E] float32
// or null; groups equal runs of consecutive experts (at most 32) of which keep may be chosen from.
AYK_EXPORT int ayk_moe_route_scored(int* ids, float* weights, int* sorted, int* tiles, const float* logits, long long stride,
                                    const float* correction, int T, int E, int top, int groups, int keep, float factor,
                                    cudaStream_t stream) {
  if (T == 0) return 0;
  AYK_REQUIRE(top >= 1 && top <= MAX_TOP && top <= E, "ayk_moe_route_scored: top %d of %d experts (at most %d)", top, E, MAX_TOP);
  AYK_REQUIRE(E <= 4096, "ayk_moe_route_scored: %d experts (at most 4096)", E);
  AYK_REQUIRE(groups >= 1 && groups <= 32 && E % groups == 0 && keep >= 1 && keep <= groups && keep * (E / groups) >= top,
              "ayk_moe_route_scored: %d experts in %d groups of which %d are kept cannot give %d choices", E, groups, keep, top);
  ayk_launch(moe_route_scored_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, ids, weights, logits, stride, correction, T, E,
             top, groups, keep, factor);
  ayk_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), stream, sorted, tiles, (const int*)ids,
             T * top, E);
  return ayk_check_launch("ayk_moe_route_scored");
}

// See moe_gemm_kernel.  dtype: of a and w; out_dtype: of out (the activation's rows may be bfloat16,
// plain products are float32).  max_tiles: the grid's first dimension.
AYK_EXPORT int ayk_moe_gemm(void* out, const void* a, long long a_stride, const void* w, const int* sorted,
                            const int* tiles, int max_tiles, int top, int gather, int scatter, int N, int N_w, int Kd,
                            int glu, float limit, float slope, float plus, int dtype, int out_dtype, cudaStream_t stream) {
  if (max_tiles == 0 || N == 0) return 0;
  dim3 grid(max_tiles, (N + BN - 1) / BN);
#define AYK_MOE(T, O, G)                                                                                              \
  ayk_launch(moe_gemm_kernel<T, O, G>, grid, dim3(256), 0, stream, (O*)out, (const T*)a, a_stride, (const T*)w, sorted, \
             tiles, top, gather, scatter, N, N_w, Kd, limit, slope, plus)
#define AYK_MOE_MMA(O, G)                                                                                        \
  ayk_launch(moe_gemm_mma_kernel<O, G>, grid, dim3(128), 0, stream, (O*)out, (const __nv_bfloat16*)a, a_stride, \
             (const __nv_bfloat16*)w, sorted, tiles, top, gather, scatter, N, N_w, Kd, limit, slope, plus)
  if (dtype == AYK_DTYPE_F32) {
    AYK_REQUIRE(out_dtype == AYK_DTYPE_F32, "ayk_moe_gemm: float32 operands give float32 rows");
    if (glu) AYK_MOE(float, float, true); else AYK_MOE(float, float, false);
  } else if (dtype == AYK_DTYPE_BF16) {
    const bool tensor = Kd % 8 == 0 && a_stride % 8 == 0 && ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0);
    if (glu) {
      AYK_REQUIRE(out_dtype == AYK_DTYPE_BF16, "ayk_moe_gemm: the activation's rows are bfloat16 here");
      if (tensor) AYK_MOE_MMA(__nv_bfloat16, true); else AYK_MOE(__nv_bfloat16, __nv_bfloat16, true);
    } else {
      AYK_REQUIRE(out_dtype == AYK_DTYPE_F32, "ayk_moe_gemm: plain products give float32 rows");
      if (tensor) AYK_MOE_MMA(float, false); else AYK_MOE(__nv_bfloat16, float, false);
    }
  } else {
    return ayk_fail("ayk_moe_gemm: unknown dtype %d", dtype);
  }
#undef AYK_MOE
#undef AYK_MOE_MMA
  return ayk_check_launch("ayk_moe_gemm");
}

AYK_EXPORT int ayk_glu_limited(void* out, const void* in, long long stride, int T, int n, float limit, float slope, float plus,
                               int in_dtype, int out_dtype, cudaStream_t stream) {
  if (T == 0 || n == 0) return 0;
  if (in_dtype == AYK_DTYPE_F32 && out_dtype == AYK_DTYPE_F32)
    ayk_launch(glu_limited_kernel<float, float>, dim3(T), dim3(256), 0, stream, (float*)out, (const float*)in, stride, n, limit, slope, plus);
  else if (in_dtype == AYK_DTYPE_F32 && out_dtype == AYK_DTYPE_BF16)
    ayk_launch(glu_limited_kernel<float, __nv_bfloat16>, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)out, (const float*)in,
               stride, n, limit, slope, plus);
  else if (in_dtype == AYK_DTYPE_BF16 && out_dtype == AYK_DTYPE_BF16)
    ayk_launch(glu_limited_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)out,
               (const __nv_bfloat16*)in, stride, n, limit, slope, plus);
  else
    return ayk_fail("ayk_glu_limited: dtypes %d -> %d", in_dtype, out_dtype);
  return ayk_check_launch("ayk_glu_limited");
}

AYK_EXPORT int ayk_moe_pad_rows() { return PAD_ROWS; }

// The padded plan (see moe_plan_padded_kernel) and the gathered rows: gathered [max_tiles * 128, d] bfloat16 gets
// row p / top of ``in`` at row_of_pair[p].  Two launches.
AYK_EXPORT int ayk_moe_plan_padded(int* row_of_pair, int* w_rows1, int* w_rows2, void* gathered, const int* ids,
                                   const void* in, long long in_stride, int T, int E, int top, int d, int n1, int n2,
                                   int max_tiles, cudaStream_t stream) {
  if (T == 0) return 0;
  AYK_REQUIRE(E <= 4096 && d % 8 == 0 && in_stride % 8 == 0, "ayk_moe_plan_padded: %d experts, rows of %d", E, d);
  ayk_launch(moe_plan_padded_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), stream, row_of_pair, w_rows1, w_rows2, ids,
             T * top, E, n1, n2, max_tiles);
  ayk_launch(moe_gather_kernel, dim3((T * top + 7) / 8), dim3(256), 0, stream, (__nv_bfloat16*)gathered, (const __nv_bfloat16*)in,
             in_stride, (const int*)row_of_pair, T * top, top, d);
  return ayk_check_launch("ayk_moe_plan_padded");
}

AYK_EXPORT int ayk_moe_combine(float* shared, const float* picked, const int* row_of_pair, const float* weights,
                               const float* mix, long long mix_stride, int T, int top, int d, cudaStream_t stream) {
  if (T == 0 || d == 0) return 0;
  ayk_launch(moe_combine_kernel, dim3(T), dim3(256), 0, stream, shared, picked, row_of_pair, weights, mix, mix_stride, top, d);
  return ayk_check_launch("ayk_moe_combine");
}

// The products of a few pairs, pair by pair (see moe_gemv_kernel): bfloat16 a and w, K a multiple of 8 and at most
// 12,288.  glu: out [pairs, N] bfloat16 = activation of (gate, up) rows of w [E, 2 N, K], a row p / top; else
// out [pairs, N] float32 = a row p times w [E, N, K].
AYK_EXPORT int ayk_moe_gemv_takes(int Kd, long long a_stride) { return Kd % 8 == 0 && a_stride % 8 == 0 && Kd <= 12288; }

AYK_EXPORT int ayk_moe_gemv(void* out, const void* a, long long a_stride, const void* w, const int* ids, int pairs, int top,
                            int N, int N_w, int Kd, int glu, float limit, float slope, float plus, cudaStream_t stream) {
  if (pairs == 0 || N == 0) return 0;
  AYK_REQUIRE(ayk_moe_gemv_takes(Kd, a_stride), "ayk_moe_gemv: rows of %d elements (stride %lld)", Kd, a_stride);
  dim3 grid(pairs, (N + GV_COLS - 1) / GV_COLS);
  const size_t smem = (size_t)Kd * sizeof(float);
  if (glu)
    ayk_launch(moe_gemv_kernel<__nv_bfloat16, true>, grid, dim3(256), smem, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)a,
               a_stride, (const __nv_bfloat16*)w, ids, top, 1, N, N_w, Kd, limit, slope, plus);
  else
    ayk_launch(moe_gemv_kernel<float, false>, grid, dim3(256), smem, stream, (float*)out, (const __nv_bfloat16*)a, a_stride,
               (const __nv_bfloat16*)w, ids, top, 0, N, N_w, Kd, limit, slope, plus);
  return ayk_check_launch("ayk_moe_gemv");
}
