// Latent attention and rotary positions.
//
// Latent attention keeps, per token, one small normed latent c (kv_rank numbers) and one rotated
// key part k_r (rot_dim numbers) that all heads share; a head's unrotated key is U_k c and its
// value U_v c.  Since (q_n . U_k c) = (U_k^T q_n) . c and sum_j p_j U_v c_j = U_v (sum_j p_j c_j),
// the kernels work on the cached pair directly: the query of a head is [U_k^T q_n ; q_r], a key
// is [c ; k_r], the weighted sum runs over c, and U_v is applied once per row afterwards.  All
// heads read the same keys, so one block serves several heads from one tile of the cache.
//
// Rotation: dimension 2i is paired with 2i+1; the pair at position p turns by p * f_i, with
// cos and sin multiplied by a gain (1 unless frequency scaling asks for more).  Positions,
// angles, scores, weights and sums are 32-bit.
#include <math.h>

#include "common.cuh"

namespace {

// v[0 .. dims) of one head turned in place by position * freq[i]; v beyond dims passes.
__device__ __forceinline__ void turn_pair(float& u, float& v, float angle, float gain) {
  float s, c;
  sincosf(angle, &s, &c);
  s *= gain;
  c *= gain;
  const float a = u * c - v * s, b = v * c + u * s;
  u = a;
  v = b;
}

// ------------------------------------------------------------------ rotary --
// x[t, head * head_stride + offset + (0 .. dims)) turned in place; x rows lie x_stride apart.
// ``halves``: dimension i is paired with i + dims/2 instead of neighbours (2i, 2i + 1).
template <typename T>
__global__ void rotary_kernel(T* __restrict__ x, long long x_stride, const int* __restrict__ positions,
                              const float* __restrict__ freq, float gain, int heads, int head_stride, int offset,
                              int dims, int halves) {
  pdl_trigger();
  const float pos = (float)positions[blockIdx.x];
  pdl_wait();
  T* row = x + (size_t)blockIdx.x * x_stride;
  const int half = dims >> 1;
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int h = i / half, p = i - h * half;
    // pairs of neighbours (2p, 2p + 1), or dimension p with p + dims/2
    T* at = row + (size_t)h * head_stride + offset + (halves ? p : 2 * p);
    const int gap = halves ? half : 1;
    float u = to_float<T>(at[0]), v = to_float<T>(at[gap]);
    turn_pair(u, v, pos * freq[p], gain);
    at[0] = from_float<T>(u);
    at[gap] = from_float<T>(v);
  }
}

// ---------------------------------------------------------- latent prepare --
// Per row of the step, from the float32 projection row [q (H x (dim + rot)) | down (rank + rot) | ...]:
//   latent  = rmsnorm(down[:rank]) * w            -> latent pages (cache dtype)
//   k_r     = turn(down[rank:])                   -> rotated-key pages
//   q_r     = turn(q[h, dim:]) for every head     -> query[t, h, rank:]  (float32)
// The unrotated query parts are projected into query[t, h, :rank] by the per-head product.
template <typename C>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(C* __restrict__ latent_pages, C* __restrict__ rope_pages, float* __restrict__ query,
                      const float* __restrict__ proj, int proj_stride, const float* __restrict__ norm_w,
                      const float* __restrict__ freq, float gain, int rot_dims, const int* __restrict__ row_req,
                      const int* __restrict__ positions, const int* __restrict__ table, int table_stride, int page_size,
                      int H, int dim, int rot, int rank, float eps, int writes) {
  __shared__ float red[4];
  pdl_trigger();
  const int t = blockIdx.x;
  const int p = positions[t];
  const int page = table[(size_t)row_req[t] * table_stride + p / page_size];
  pdl_wait();
  const float* row = proj + (size_t)t * proj_stride;
  const float* down = row + (size_t)H * (dim + rot);
  const float pos = (float)p;
  const int half = rot_dims >> 1;
  const int Dk = rank + rot;
  // rotated query parts
  for (int i = threadIdx.x; i < H * rot; i += blockDim.x) {
    const int h = i / rot, e = i - h * rot;
    const float* src = row + (size_t)h * (dim + rot) + dim;
    float val;
    if (e < rot_dims) {
      const int pr = e >> 1;
      float u = src[2 * pr], v = src[2 * pr + 1];
      turn_pair(u, v, pos * freq[pr], gain);
      val = (e & 1) ? v : u;
    } else {
      val = src[e];
    }
    query[((size_t)t * H + h) * Dk + rank + e] = val;
  }
  if (!writes || page <= 0) return;      // a run step that reads another's cache; a padding lane
  const size_t at = (size_t)page * page_size + (p % page_size);
  for (int e = threadIdx.x; e < rot; e += blockDim.x) {
    float val;
    if (e < rot_dims) {
      const int pr = e >> 1;
      float u = down[rank + 2 * pr], v = down[rank + 2 * pr + 1];
      turn_pair(u, v, pos * freq[pr], gain);
      val = (e & 1) ? v : u;
    } else {
      val = down[rank + e];
    }
    rope_pages[at * rot + e] = from_float<C>(val);
  }
  float s = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) s = fmaf(down[i], down[i], s);
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  const float inv = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) latent_pages[at * rank + i] = from_float<C>(down[i] * inv * norm_w[i]);
}

// ------------------------------------------------------- per-head products --
// out[t, h, n] = (sum_k a[t, h, k] * w[h, n, k]) (* sigmoid(gate[t, h * gate_head + n * gate_col]): gate_head 1 and gate_col 0 for a number per head, gate_head N and gate_col 1 for a number per output): a small product per head
// with the head's own matrix.  Tile: 16 rows x 64 columns of one head, K in chunks of 32.
constexpr int HM_ROWS = 16, HM_COLS = 64, HM_K = 32;

template <typename W, typename O>
__global__ void __launch_bounds__(128)
head_matmul_kernel(O* __restrict__ out, long long out_row, int out_head, const float* __restrict__ a, long long a_row,
                   int a_head, const W* __restrict__ w, const float* __restrict__ gate, long long gate_row, int gate_head, int gate_col, int T, int N,
                   int K) {
  __shared__ float As[HM_ROWS][HM_K + 1];
  __shared__ float Ws[HM_COLS][HM_K + 1];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, t0 = blockIdx.x * HM_ROWS, n0 = blockIdx.z * HM_COLS;
  const int tn = threadIdx.x & 63, tr = (threadIdx.x >> 6) * 8;
  float acc[8] = {};
  const W* wh = w + (size_t)h * N * K;
  for (int k0 = 0; k0 < K; k0 += HM_K) {
    __syncthreads();
    for (int i = threadIdx.x; i < HM_ROWS * HM_K; i += 128) {
      const int r = i / HM_K, k = i - r * HM_K;
      As[r][k] = (t0 + r < T && k0 + k < K) ? a[(size_t)(t0 + r) * a_row + (size_t)h * a_head + k0 + k] : 0.f;
    }
    for (int i = threadIdx.x; i < HM_COLS * HM_K; i += 128) {
      const int n = i / HM_K, k = i - n * HM_K;
      Ws[n][k] = (n0 + n < N && k0 + k < K) ? to_float<W>(wh[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HM_K; ++k) {
      const float wv = Ws[tn][k];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(As[tr + i][k], wv, acc[i]);
    }
  }
  if (n0 + tn >= N) return;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int t = t0 + tr + i;
    if (t >= T) continue;
    float v = acc[i];
    if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_row + (size_t)h * gate_head + (size_t)(n0 + tn) * gate_col]));
    out[(size_t)t * out_row + (size_t)h * out_head + n0 + tn] = from_float<O>(v);
  }
}


// The same product for a handful of rows (a decode step): a block takes one head and eight output
// columns, one per warp; the rows' operand of that head sits in shared memory, a warp streams its
// weight row once (eight elements per lane and step) and keeps one sum per row.
constexpr int MV_ROWS = 16, MV_WARPS = 8;

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __bfloat162float(h[i].x); v[2 * i + 1] = __bfloat162float(h[i].y); }
}

template <typename W, typename O>
__global__ void __launch_bounds__(MV_WARPS * 32)
head_matvec_kernel(O* __restrict__ out, long long out_row, int out_head, const float* __restrict__ a, long long a_row,
                   int a_head, const W* __restrict__ w, const float* __restrict__ gate, long long gate_row, int gate_head, int gate_col, int T, int N,
                   int K) {
  extern __shared__ __align__(16) float rows[];          // [T][K]
  pdl_trigger();
  const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.y * MV_WARPS + warp;
  // the weight row does not depend on the kernel before: its first piece is asked for ahead of the wait
  const W* wr = w + ((size_t)h * N + (n < N ? n : 0)) * K;
  float w8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (lane * 8 < K) load8(wr + lane * 8, w8);
  pdl_wait();
  for (int i = threadIdx.x; i < T * (K / 4); i += blockDim.x) {
    const int t = i / (K / 4), c = (i - t * (K / 4)) * 4;
    *reinterpret_cast<float4*>(rows + t * K + c) = *reinterpret_cast<const float4*>(a + (size_t)t * a_row + (size_t)h * a_head + c);
  }
  __syncthreads();
  if (n >= N) return;
  float acc[MV_ROWS];
#pragma unroll
  for (int t = 0; t < MV_ROWS; ++t) acc[t] = 0.f;
  for (int k0 = lane * 8; k0 < K; k0 += 256) {
    if (k0 != lane * 8) load8(wr + k0, w8);
#pragma unroll
    for (int t = 0; t < MV_ROWS; ++t) {
      if (t < T) {
        float a8[8];
        load8(rows + t * K + k0, a8);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[t] = fmaf(a8[e], w8[e], acc[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < MV_ROWS; ++t) {
    if (t < T) {
      float v = warp_sum(acc[t]);
      if (lane == 0) {
        if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_row + (size_t)h * gate_head + (size_t)n * gate_col]));
        out[(size_t)t * out_row + (size_t)h * out_head + n] = from_float<O>(v);
      }
    }
  }
}

// --------------------------------------------------------------- attention --
// One block: up to 32 (row, head) pairs of one request: BR consecutive rows x HG heads.  Keys are
// taken 32 at a time; lane j scores key j; for the weighted sum lane l owns latent columns l, l+32...
constexpr int AQ = 32, AKEYS = 32, AWARPS = 4, ARQ = AQ / AWARPS;

template <typename C, int NC>
__global__ void __launch_bounds__(AWARPS * 32)
latent_attention_kernel(float* __restrict__ out, const float* __restrict__ query, const C* __restrict__ latent_pages,
                        const C* __restrict__ rope_pages, const int* __restrict__ table, int table_stride,
                        const int* __restrict__ req_q_start, const int* __restrict__ req_pos0, int num_req, int H, int HG,
                        int BR, int rank, int rot, int page_size, float scale) {
  pdl_trigger();
  pdl_wait();
  int tile = blockIdx.x, req = -1, q0 = 0, q_len = 0;
  for (int r = 0; r < num_req; ++r) {
    const int len = req_q_start[r + 1] - req_q_start[r];
    const int tiles = (len + BR - 1) / BR;
    if (tile < tiles) { req = r; q0 = tile * BR; q_len = len; break; }
    tile -= tiles;
  }
  if (req < 0) return;
  const int h0 = blockIdx.y * HG;
  const int heads = min(HG, H - h0);
  const int rows = min(BR, q_len - q0);
  const int row0 = req_q_start[req] + q0;
  const int pos0 = req_pos0[req] + q0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Dk = rank + rot;
  const int ldq = (Dk + 3) & ~3, ldk = Dk + 1;

  extern __shared__ float smem[];
  float* Qs = smem;                       // [AQ][ldq]
  float* Ks = Qs + AQ * ldq;              // [AKEYS][ldk]: latent then rotated part
  float* Ps = Ks + AKEYS * ldk;           // [AQ][AKEYS]

  // pair i of the block: row i / HG of the tile, head h0 + i % HG
  for (int i = threadIdx.x; i < AQ * Dk; i += blockDim.x) {
    const int pr = i / Dk, d = i - pr * Dk;
    const int r = pr / HG, hh = pr - r * HG;
    const bool live = r < rows && hh < heads && pr < BR * HG;
    Qs[pr * ldq + d] = live ? query[((size_t)(row0 + r) * H + h0 + hh) * Dk + d] : 0.f;
  }

  float acc[ARQ][NC];
  float m_run[ARQ], l_run[ARQ];
#pragma unroll
  for (int r = 0; r < ARQ; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
  }
  const int last_pos = pos0 + rows - 1;
  const int* my_table = table + (size_t)req * table_stride;

  for (int k0 = 0; k0 <= last_pos; k0 += AKEYS) {
    __syncthreads();
    for (int i = threadIdx.x; i < AKEYS * Dk; i += blockDim.x) {
      const int j = i / Dk, d = i - j * Dk;
      const int kp = k0 + j;
      float v = 0.f;
      if (kp <= last_pos) {
        const int page = my_table[kp / page_size];
        if (page > 0) {
          const size_t at = (size_t)page * page_size + (kp % page_size);
          v = d < rank ? to_float<C>(latent_pages[at * rank + d]) : to_float<C>(rope_pages[at * rot + (d - rank)]);
        }
      }
      Ks[j * ldk + d] = v;
    }
    __syncthreads();
    const int kp = k0 + lane;
    const bool page_ok = kp <= last_pos && my_table[kp / page_size] > 0;
#pragma unroll
    for (int r = 0; r < ARQ; ++r) {
      const int pr = warp * ARQ + r;                 // warp-uniform
      const int row = pr / HG;
      const bool live = row < rows && (pr - row * HG) < heads && pr < BR * HG;
      if (!live) continue;
      const int qpos = pos0 + row;
      const float* qr = Qs + pr * ldq;
      const float* kr = Ks + lane * ldk;
      float s = 0.f;
      int d = 0;
      for (; d + 4 <= Dk; d += 4) {
        const float4 qv = *reinterpret_cast<const float4*>(qr + d);
        s = fmaf(qv.x, kr[d], s);
        s = fmaf(qv.y, kr[d + 1], s);
        s = fmaf(qv.z, kr[d + 2], s);
        s = fmaf(qv.w, kr[d + 3], s);
      }
      for (; d < Dk; ++d) s = fmaf(qr[d], kr[d], s);
      const bool valid = page_ok && kp <= qpos;
      s = valid ? s * scale : -INFINITY;
      const float m_new = fmaxf(m_run[r], warp_max(s));
      float p = 0.f, alpha = 1.f;
      if (m_new > -INFINITY) {
        p = valid ? expf(s - m_new) : 0.f;
        alpha = expf(m_run[r] - m_new);
      }
      l_run[r] = l_run[r] * alpha + warp_sum(p);
      m_run[r] = m_new;
      Ps[pr * AKEYS + lane] = p;
#pragma unroll
      for (int c = 0; c < NC; ++c) acc[r][c] *= alpha;
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < ARQ; ++r) {
      const int pr = warp * ARQ + r;
      const int row = pr / HG;
      const bool live = row < rows && (pr - row * HG) < heads && pr < BR * HG;
      if (!live) continue;
      const float* prow = Ps + pr * AKEYS;
      for (int j = 0; j < AKEYS; ++j) {
        const float p = prow[j];
        const float* vr = Ks + j * ldk;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int d = lane + 32 * c;
          if (d < rank) acc[r][c] = fmaf(p, vr[d], acc[r][c]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < ARQ; ++r) {
    const int pr = warp * ARQ + r;
    const int row = pr / HG, hh = pr - row * HG;
    const bool live = row < rows && hh < heads && pr < BR * HG;
    if (!live) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    float* o = out + ((size_t)(row0 + row) * H + h0 + hh) * rank;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int d = lane + 32 * c;
      if (d < rank) o[d] = acc[r][c] * inv;
    }
  }
}

template <typename C, int NC>
int launch_latent_attention(float* out, const float* query, const void* latent_pages, const void* rope_pages,
                            const int* table, int table_stride, const int* req_q_start, const int* req_pos0, int num_req,
                            int total_rows, int H, int rank, int rot, int page_size, float scale, cudaStream_t stream) {
  const int HG = H < AQ ? H : AQ;
  const int BR = AQ / HG;
  const int Dk = rank + rot;
  const size_t smem = ((size_t)AQ * ((Dk + 3) & ~3) + (size_t)AKEYS * (Dk + 1) + (size_t)AQ * AKEYS) * sizeof(float);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(latent_attention_kernel<C, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return ayk_fail("ayk_latent_attention: shared memory %zu: %s", smem, cudaGetErrorString(err));
    configured = smem;
  }
  dim3 grid(total_rows / BR + num_req, (H + HG - 1) / HG);
  ayk_launch(latent_attention_kernel<C, NC>, grid, dim3(AWARPS * 32), smem, stream, out, query, (const C*)latent_pages,
             (const C*)rope_pages, table, table_stride, req_q_start, req_pos0, num_req, H, HG, BR, rank, rot, page_size, scale);
  return ayk_check_launch("ayk_latent_attention");
}

template <typename C>
int pick_latent_attention(float* out, const float* query, const void* latent_pages, const void* rope_pages, const int* table,
                          int table_stride, const int* req_q_start, const int* req_pos0, int num_req, int total_rows, int H,
                          int rank, int rot, int page_size, float scale, cudaStream_t stream) {
#define AYK_LATENT(NC)                                                                                                   \
  return launch_latent_attention<C, NC>(out, query, latent_pages, rope_pages, table, table_stride, req_q_start, req_pos0, \
                                        num_req, total_rows, H, rank, rot, page_size, scale, stream)
  if (rank <= 64) AYK_LATENT(2);
  if (rank <= 128) AYK_LATENT(4);
  if (rank <= 256) AYK_LATENT(8);
  AYK_LATENT(16);
#undef AYK_LATENT
}

}  // namespace

// x[t, head * head_stride + offset + (0 .. dims)) turned in place by positions[t] * freq[i].
AYK_EXPORT int ayk_rotary(void* x, long long x_stride, const int* positions, const float* freq, float gain, int T,
                          int heads, int head_stride, int offset, int dims, int halves, int dtype, cudaStream_t stream) {
  if (T == 0 || heads == 0 || dims == 0) return 0;
  AYK_REQUIRE(dims % 2 == 0, "ayk_rotary: %d rotated dimensions cannot be paired", dims);
  if (dtype == AYK_DTYPE_F32)
    ayk_launch(rotary_kernel<float>, dim3(T), dim3(128), 0, stream, (float*)x, x_stride, positions, freq, gain, heads,
               head_stride, offset, dims, halves);
  else if (dtype == AYK_DTYPE_BF16)
    ayk_launch(rotary_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (__nv_bfloat16*)x, x_stride, positions, freq,
               gain, heads, head_stride, offset, dims, halves);
  else
    return ayk_fail("ayk_rotary: unknown dtype %d", dtype);
  return ayk_check_launch("ayk_rotary");
}

AYK_EXPORT int ayk_latent_prepare(void* latent_pages, void* rope_pages, float* query, const float* proj, int proj_stride,
                                  const float* norm_w, const float* freq, float gain, int rot_dims, const int* row_req,
                                  const int* positions, const int* table, int table_stride, int page_size, int T, int H,
                                  int dim, int rot, int rank, float eps, int writes, int cache_dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  AYK_REQUIRE(rot_dims % 2 == 0 && rot_dims <= rot, "ayk_latent_prepare: %d rotated dimensions of %d", rot_dims, rot);
  if (cache_dtype == AYK_DTYPE_F32)
    ayk_launch(latent_prepare_kernel<float>, dim3(T), dim3(128), 0, stream, (float*)latent_pages, (float*)rope_pages, query,
               proj, proj_stride, norm_w, freq, gain, rot_dims, row_req, positions, table, table_stride, page_size, H, dim,
               rot, rank, eps, writes);
  else if (cache_dtype == AYK_DTYPE_BF16)
    ayk_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (__nv_bfloat16*)latent_pages,
               (__nv_bfloat16*)rope_pages, query, proj, proj_stride, norm_w, freq, gain, rot_dims, row_req, positions, table,
               table_stride, page_size, H, dim, rot, rank, eps, writes);
  else
    return ayk_fail("ayk_latent_prepare: unknown dtype %d", cache_dtype);
  return ayk_check_launch("ayk_latent_prepare");
}

// out[t, h, n] = sum_k a[t, h, k] w[h, n, k] (times sigmoid(gate[t, h * gate_head + n * gate_col]) when gate is given).  a is
// float32 with row and head strides; w [H, N, K] in w_dtype; out in out_dtype with its strides.
AYK_EXPORT int ayk_head_matmul(void* out, long long out_row, int out_head, const float* a, long long a_row, int a_head,
                               const void* w, const float* gate, long long gate_row, int gate_head, int gate_col, int T, int H, int N, int K, int w_dtype,
                               int out_dtype, cudaStream_t stream) {
  if (T == 0 || H == 0 || N == 0) return 0;
  dim3 grid((T + HM_ROWS - 1) / HM_ROWS, H, (N + HM_COLS - 1) / HM_COLS);
  AYK_REQUIRE(H <= 65535 && grid.z <= 65535, "ayk_head_matmul: too many heads or columns");
#define AYK_HM(WT, OT)                                                                                               \
  ayk_launch(head_matmul_kernel<WT, OT>, grid, dim3(128), 0, stream, (OT*)out, out_row, out_head, a, a_row, a_head, \
             (const WT*)w, gate, gate_row, gate_head, gate_col, T, N, K)
  if (w_dtype == AYK_DTYPE_F32 && out_dtype == AYK_DTYPE_F32) AYK_HM(float, float);
  else if (w_dtype == AYK_DTYPE_BF16 && out_dtype == AYK_DTYPE_F32) AYK_HM(__nv_bfloat16, float);
  else if (w_dtype == AYK_DTYPE_BF16 && out_dtype == AYK_DTYPE_BF16) AYK_HM(__nv_bfloat16, __nv_bfloat16);
  else return ayk_fail("ayk_head_matmul: unsupported dtypes w=%d out=%d", w_dtype, out_dtype);
#undef AYK_HM
  return ayk_check_launch("ayk_head_matmul");
}

// out[t, h, :rank] = softmax_j(query[t, h] . [latent_j ; rope_j] * scale) latent_j over the cached
// positions j <= position(t) of the row's request.  query [T, H, rank + rot] and out [T, H, rank]
// float32; pages [pages, page_size, rank] and [pages, page_size, rot] in cache_dtype.
AYK_EXPORT int ayk_latent_attention(float* out, const float* query, const void* latent_pages, const void* rope_pages,
                                    const int* table, int table_stride, const int* req_q_start, const int* req_pos0,
                                    int num_req, int total_rows, int H, int rank, int rot, int page_size, float scale,
                                    int cache_dtype, cudaStream_t stream) {
  if (num_req == 0 || total_rows == 0) return 0;
  AYK_REQUIRE(rank >= 1 && rank <= 512, "ayk_latent_attention: latent size %d is not in [1, 512]", rank);
  AYK_REQUIRE(rot >= 0 && rank + rot <= 640, "ayk_latent_attention: key size %d exceeds 640", rank + rot);
  if (cache_dtype == AYK_DTYPE_F32)
    return pick_latent_attention<float>(out, query, latent_pages, rope_pages, table, table_stride, req_q_start, req_pos0,
                                        num_req, total_rows, H, rank, rot, page_size, scale, stream);
  if (cache_dtype == AYK_DTYPE_BF16)
    return pick_latent_attention<__nv_bfloat16>(out, query, latent_pages, rope_pages, table, table_stride, req_q_start,
                                                req_pos0, num_req, total_rows, H, rank, rot, page_size, scale, stream);
  return ayk_fail("ayk_latent_attention: unknown dtype %d", cache_dtype);
}

// The per-head product for up to 16 rows (ayk_head_matvec_takes): K a multiple of 8, 16-byte aligned operands.
AYK_EXPORT int ayk_head_matvec_takes(const void* a, long long a_row, int a_head, const void* w, int T, int K) {
  return T >= 1 && T <= MV_ROWS && K % 8 == 0 && (size_t)T * K * 4 <= 96 * 1024 && a_row % 4 == 0 && a_head % 4 == 0 &&
         (uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0;
}

AYK_EXPORT int ayk_head_matvec(void* out, long long out_row, int out_head, const float* a, long long a_row, int a_head,
                               const void* w, const float* gate, long long gate_row, int gate_head, int gate_col, int T, int H, int N, int K, int w_dtype,
                               int out_dtype, cudaStream_t stream) {
  if (T == 0 || H == 0 || N == 0) return 0;
  AYK_REQUIRE(ayk_head_matvec_takes(a, a_row, a_head, w, T, K), "ayk_head_matvec: %d rows of %d are not taken", T, K);
  dim3 grid(H, (N + MV_WARPS - 1) / MV_WARPS);
  AYK_REQUIRE(grid.y <= 65535, "ayk_head_matvec: too many columns");
  const size_t smem = (size_t)T * K * sizeof(float);
#define AYK_MV(WT, OT)                                                                                                         \
  do {                                                                                                                         \
    static size_t configured = 48 * 1024;                                                                                      \
    if (smem > configured) {                                                                                                   \
      cudaError_t err = cudaFuncSetAttribute(head_matvec_kernel<WT, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (err != cudaSuccess) return ayk_fail("ayk_head_matvec: shared memory %zu: %s", smem, cudaGetErrorString(err));        \
      configured = smem;                                                                                                       \
    }                                                                                                                          \
    ayk_launch(head_matvec_kernel<WT, OT>, grid, dim3(MV_WARPS * 32), smem, stream, (OT*)out, out_row, out_head, a, a_row,     \
               a_head, (const WT*)w, gate, gate_row, gate_head, gate_col, T, N, K);                                                                 \
  } while (0)
  if (w_dtype == AYK_DTYPE_F32 && out_dtype == AYK_DTYPE_F32) AYK_MV(float, float);
  else if (w_dtype == AYK_DTYPE_BF16 && out_dtype == AYK_DTYPE_F32) AYK_MV(__nv_bfloat16, float);
  else if (w_dtype == AYK_DTYPE_BF16 && out_dtype == AYK_DTYPE_BF16) AYK_MV(__nv_bfloat16, __nv_bfloat16);
  else return ayk_fail("ayk_head_matvec: unsupported dtypes w=%d out=%d", w_dtype, out_dtype);
#undef AYK_MV
  return ayk_check_launch("ayk_head_matvec");
}
