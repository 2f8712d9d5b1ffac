// Softmax attention over the paged cache whose keys and values are grouped separately, with a
// distance bias per head, a window, and first tokens that the window never drops.
//
// QH query heads read KH key heads of size DK (query head h reads key head h / (QH / KH)) and VH
// value heads of size DV (value head h / (QH / VH)).  For the query at absolute position i of a
// request and a cached position j <= i of that request,
//     s_j = (q . k_j) * scale - slope[h] * (i - j)            (slope null: no distance bias)
// and j is visible when i - j < window (window <= 0: always) or j < keep_first, and, with chunk > 0, only when
// j lies in i's own run of ``chunk`` positions (floor(i / chunk) = floor(j / chunk)).  The weights are
// the softmax of s over the visible keys; scores, weights and sums are 32-bit.
//
// Two designs of attention reduce to this:
//  * scores that are mixed across heads before the softmax, s'_h = sum_g M[h, g] s_g.  The mix is
//    linear, so it moves to the queries: with q~_h = [sum over the heads g of key head c of
//    M[h, g] q_g] for c = 0 .. G-1 (one piece per key head, side by side) and the G key heads of a
//    token side by side as one key of size G * D, s'_h = q~_h . k - (sum_g M[h, g] slope_g) (i - j).
//    The attention then has KH = 1, DK = G * D, VH = G; ayk_head_norm_prepare makes q~.
//  * two score maps per head over the same values (the second map's output is taken off the
//    first's afterwards): QH = 2 H query heads laid out [key/value group][map][head of the group],
//    KH = 2 G key heads [group][map], VH = G; ayk_grouped_finish combines the maps.
//
// ayk_head_norm_prepare turns float32 projection rows into queries, cached keys and cached values:
// RMS norm per head over the head's D numbers with one weight of size D shared by all heads.
// ayk_grouped_attention runs the attention (FP32 pipes here; bfloat16 on the tensor cores in
// attention_grouped_mma.cu); when the context is cut into parts, or the maps are to be combined,
// it leaves float32 partial sums that ayk_grouped_finish merges.
#include <math.h>

#include "attention_grouped.cuh"

namespace {

// ----------------------------------------------------------------- prepare --
// One block per (row, key/value group c).  It norms the query heads of its group (head n = h * maps + m, h of H,
// m of maps, lands at head ((h / hpg) * maps + m) * hpg + h % hpg of the output, hpg = H / G: the heads that
// share a key head become neighbours), the group's key heads, and files the group's slice of the values.
// With ``mix`` (maps == 1) it writes piece c of every mixed query q~ as described above: a warp per query head,
// the group's normed queries in shared memory.
template <typename C>
__global__ void __launch_bounds__(256)
head_norm_prepare_kernel(C* __restrict__ qout, C* __restrict__ kpages, C* __restrict__ vpages,
                         const float* __restrict__ proj, long long stride, const float* __restrict__ qw,
                         const float* __restrict__ kw, const float* __restrict__ mix, const int* __restrict__ row_req,
                         const int* __restrict__ positions, const int* __restrict__ table, int table_stride,
                         int page_size, int H, int G, int D, int maps, int v_col0, int v_width, float eps, int writes) {
  extern __shared__ float qn[];              // [hpg][D] normed queries of the group, only with ``mix``
  pdl_trigger();
  const int t = blockIdx.x, c = blockIdx.y;
  const int p = positions[t];
  const int page = table[(size_t)row_req[t] * table_stride + p / page_size];
  pdl_wait();
  const float* row = proj + (size_t)t * stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int hpg = H / G;
  const int nq = H * maps, nk = G * maps;
  const float inv_d = 1.0f / (float)D;
  C* qdst = qout + (size_t)t * ((size_t)nq * D) * (mix ? G : 1);
  for (int j = warp; j < hpg * maps; j += nwarp) {
    const int n = c * hpg * maps + j;
    const float* src = row + (size_t)n * D;
    float s = 0.f;
    for (int d = lane; d < D; d += 32) s = fmaf(src[d], src[d], s);
    const float inv = 1.0f / sqrtf(warp_sum(s) * inv_d + eps);
    if (mix) {
      for (int d = lane; d < D; d += 32) qn[j * D + d] = src[d] * inv * qw[d];
    } else {
      const int h = n / maps, m = n - h * maps;
      C* dst = qdst + (size_t)(((h / hpg) * maps + m) * hpg + h % hpg) * D;
      for (int d = lane; d < D; d += 32) dst[d] = from_float<C>(src[d] * inv * qw[d]);
    }
  }
  if (writes && page > 0) {
    const size_t cell = (size_t)page * page_size + (p % page_size);
    const float* ksrc = row + (size_t)nq * D;
    C* kdst = kpages + cell * ((size_t)nk * D);
    for (int n = c * maps + warp; n < (c + 1) * maps; n += nwarp) {
      const float* src = ksrc + (size_t)n * D;
      float s = 0.f;
      for (int d = lane; d < D; d += 32) s = fmaf(src[d], src[d], s);
      const float inv = 1.0f / sqrtf(warp_sum(s) * inv_d + eps);
      for (int d = lane; d < D; d += 32) kdst[(size_t)n * D + d] = from_float<C>(src[d] * inv * kw[d]);
    }
    const int vpart = v_width / G;
    C* vdst = vpages + cell * (size_t)v_width + (size_t)c * vpart;
    for (int i = threadIdx.x; i < vpart; i += blockDim.x) vdst[i] = from_float<C>(row[v_col0 + c * vpart + i]);
  }
  if (mix) {
    __syncthreads();
    for (int h = warp; h < H; h += nwarp) {
      const float* coeff = mix + (size_t)h * H + c * hpg;
      C* dst = qdst + ((size_t)h * G + c) * D;
      for (int d = lane; d < D; d += 32) {
        float s = 0.f;
        for (int j = 0; j < hpg; ++j) s = fmaf(coeff[j], qn[j * D + d], s);
        dst[d] = from_float<C>(s);
      }
    }
  }
}

// The same with four numbers to a lane (16-byte loads, 8- or 16-byte stores): head sizes, the row stride, the
// values' first column and a group's slice of the values are multiples of 4 and the tensors 16-byte aligned.
__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t*>(&lo);
  packed.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}

template <typename C>
__global__ void __launch_bounds__(256)
head_norm_prepare_vec_kernel(C* __restrict__ qout, C* __restrict__ kpages, C* __restrict__ vpages,
                             const float* __restrict__ proj, long long stride, const float* __restrict__ qw,
                             const float* __restrict__ kw, const float* __restrict__ mix, const int* __restrict__ row_req,
                             const int* __restrict__ positions, const int* __restrict__ table, int table_stride,
                             int page_size, int H, int G, int D, int maps, int v_col0, int v_width, float eps, int writes) {
  extern __shared__ __align__(16) float qn[];              // [hpg][D] normed queries of the group, only with ``mix``
  pdl_trigger();
  const int t = blockIdx.x, c = blockIdx.y;
  const int p = positions[t];
  const int page = table[(size_t)row_req[t] * table_stride + p / page_size];
  pdl_wait();
  const float* row = proj + (size_t)t * stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int hpg = H / G;
  const int nq = H * maps, nk = G * maps;
  const float inv_d = 1.0f / (float)D;
  C* qdst = qout + (size_t)t * ((size_t)nq * D) * (mix ? G : 1);
  // one head: its sum of squares, then the normed numbers to ``to`` (a float4 at a time)
  auto normed = [&](const float* src, const float* w, auto&& to) {
    float s = 0.f;
    for (int d = lane * 4; d < D; d += 128) {
      const float4 v = *reinterpret_cast<const float4*>(src + d);
      s = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s))));
    }
    const float inv = 1.0f / sqrtf(warp_sum(s) * inv_d + eps);
    for (int d = lane * 4; d < D; d += 128) {
      const float4 v = *reinterpret_cast<const float4*>(src + d);
      const float4 g = *reinterpret_cast<const float4*>(w + d);
      to(d, v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
    }
  };
  for (int j = warp; j < hpg * maps; j += nwarp) {
    const int n = c * hpg * maps + j;
    if (mix) {
      float* dst = qn + j * D;
      normed(row + (size_t)n * D, qw, [&](int d, float a, float b, float e, float f) { store4(dst + d, a, b, e, f); });
    } else {
      const int h = n / maps, m = n - h * maps;
      C* dst = qdst + (size_t)(((h / hpg) * maps + m) * hpg + h % hpg) * D;
      normed(row + (size_t)n * D, qw, [&](int d, float a, float b, float e, float f) { store4(dst + d, a, b, e, f); });
    }
  }
  if (writes && page > 0) {
    const size_t cell = (size_t)page * page_size + (p % page_size);
    const float* ksrc = row + (size_t)nq * D;
    C* kdst = kpages + cell * ((size_t)nk * D);
    for (int n = c * maps + warp; n < (c + 1) * maps; n += nwarp) {
      C* dst = kdst + (size_t)n * D;
      normed(ksrc + (size_t)n * D, kw, [&](int d, float a, float b, float e, float f) { store4(dst + d, a, b, e, f); });
    }
    const int vpart = v_width / G;
    C* vdst = vpages + cell * (size_t)v_width + (size_t)c * vpart;
    const float* vsrc = row + v_col0 + c * vpart;
    for (int i = threadIdx.x * 4; i < vpart; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(vsrc + i);
      store4(vdst + i, v.x, v.y, v.z, v.w);
    }
  }
  if (mix) {
    __syncthreads();
    for (int h = warp; h < H; h += nwarp) {
      const float* coeff = mix + (size_t)h * H + c * hpg;
      C* dst = qdst + ((size_t)h * G + c) * D;
      for (int d = lane * 4; d < D; d += 128) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < hpg; ++j) {
          const float cj = coeff[j];
          const float4 v = *reinterpret_cast<const float4*>(qn + j * D + d);
          acc.x = fmaf(cj, v.x, acc.x); acc.y = fmaf(cj, v.y, acc.y); acc.z = fmaf(cj, v.z, acc.z); acc.w = fmaf(cj, v.w, acc.w);
        }
        store4(dst + d, acc.x, acc.y, acc.z, acc.w);
      }
    }
  }
}

// ------------------------------------------------------- the general kernel --
// One block works on up to 32 consecutive rows of one request, one query head and one part of the
// context: 4 warps x 8 rows.  Keys are taken 32 at a time (one per lane for the scores, one value
// column per lane for the weighted sum).
constexpr int BQ = 32;
constexpr int BKEYS = 32;
constexpr int WARPS = 4;
constexpr int RQ = BQ / WARPS;
constexpr int MAX_DV = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
grouped_attention_kernel(GroupedArgs a) {
  pdl_trigger();
  pdl_wait();
  int tile = blockIdx.x, req = -1, q0 = 0, q_len = 0;
  for (int r = 0; r < a.num_req; ++r) {
    int len = a.req_q_start[r + 1] - a.req_q_start[r];
    int tiles = (len + BQ - 1) / BQ;
    if (tile < tiles) { req = r; q0 = tile * BQ; q_len = len; break; }
    tile -= tiles;
  }
  if (req < 0) return;
  const int QH = a.QH, DK = a.DK, DV = a.DV;
  const int h = blockIdx.y, kh = h / (QH / a.KH), vh = h / (QH / a.VH);
  const int rows = min(BQ, q_len - q0);
  const int row0 = a.req_q_start[req] + q0;
  const int pos0 = a.req_pos0[req] + q0;
  const int last_pos = pos0 + rows - 1;
  const int part = blockIdx.z;
  const int k_first = a.part_keys > 0 ? part * a.part_keys : 0;
  const int k_last = a.part_keys > 0 ? min(last_pos, k_first + a.part_keys - 1) : last_pos;
  if (k_first > last_pos) return;                 // the merge does not read parts beyond the context
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ldk = DK + 1;
  const int ldq = (DK + 3) & ~3;
  const T* q = reinterpret_cast<const T*>(a.q);
  const T* kcache = reinterpret_cast<const T*>(a.kcache);
  const T* vcache = reinterpret_cast<const T*>(a.vcache);

  extern __shared__ float smem[];
  float* Qs = smem;                    // [BQ][ldq]
  float* Ks = Qs + BQ * ldq;           // [BKEYS][DK + 1]
  float* Vs = Ks + BKEYS * ldk;        // [BKEYS][DV]
  float* Ps = Vs + BKEYS * DV;         // [BQ][BKEYS]

  for (int i = threadIdx.x; i < BQ * DK; i += blockDim.x) {
    int r = i / DK, d = i - r * DK;
    Qs[r * ldq + d] = r < rows ? to_float<T>(q[(size_t)(row0 + r) * ((size_t)QH * DK) + (size_t)h * DK + d]) : 0.f;
  }
  const int NC = (DV + 31) / 32;
  float acc[RQ][MAX_DV / 32];
  float m_run[RQ], l_run[RQ];
#pragma unroll
  for (int r = 0; r < RQ; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int c = 0; c < MAX_DV / 32; ++c) acc[r][c] = 0.f;
  }
  const float slope = a.slopes ? a.slopes[h] : 0.f;
  const int* my_table = a.table + (size_t)req * a.table_stride;
  const GroupedTiles walk(k_first, k_last, pos0, a.window, a.keep_first, BKEYS, a.chunk);

  for (int k0 = walk.first(); k0 <= k_last; k0 = walk.next(k0)) {
    __syncthreads();
    for (int i = threadIdx.x; i < BKEYS * DK; i += blockDim.x) {
      int j = i / DK, d = i - j * DK;
      int kp = k0 + j;
      float kv = 0.f;
      if (kp <= k_last) {
        int page = my_table[kp / a.page_size];
        if (page > 0) kv = to_float<T>(kcache[(((size_t)page * a.page_size + (kp % a.page_size)) * a.KH + kh) * DK + d]);
      }
      Ks[j * ldk + d] = kv;
    }
    for (int i = threadIdx.x; i < BKEYS * DV; i += blockDim.x) {
      int j = i / DV, d = i - j * DV;
      int kp = k0 + j;
      float vv = 0.f;
      if (kp <= k_last) {
        int page = my_table[kp / a.page_size];
        if (page > 0) vv = to_float<T>(vcache[(((size_t)page * a.page_size + (kp % a.page_size)) * a.VH + vh) * DV + d]);
      }
      Vs[j * DV + d] = vv;
    }
    __syncthreads();

    const int kp = k0 + lane;
    const bool page_ok = kp <= k_last && my_table[kp / a.page_size] > 0;
#pragma unroll
    for (int r = 0; r < RQ; ++r) {
      const int row = warp * RQ + r;
      if (row >= rows) break;
      const int qpos = pos0 + row;
      const float* qr = Qs + row * ldq;
      const float* kr = Ks + lane * ldk;
      float s = 0.f;
      int d = 0;
      for (; d + 4 <= DK; d += 4) {
        float4 qv = *reinterpret_cast<const float4*>(qr + d);
        s = fmaf(qv.x, kr[d], s);
        s = fmaf(qv.y, kr[d + 1], s);
        s = fmaf(qv.z, kr[d + 2], s);
        s = fmaf(qv.w, kr[d + 3], s);
      }
      for (; d < DK; ++d) s = fmaf(qr[d], kr[d], s);
      const bool valid = page_ok && grouped_visible(qpos, kp, a.window, a.keep_first, a.chunk);
      s = valid ? fmaf(-slope, (float)(qpos - kp), s * a.scale) : -INFINITY;
      const float m_new = fmaxf(m_run[r], warp_max(s));
      float p = 0.f, alpha = 1.f;
      if (m_new > -INFINITY) {
        p = valid ? expf(s - m_new) : 0.f;
        alpha = expf(m_run[r] - m_new);    // exp(-inf) = 0 on the first visible tile
      }
      l_run[r] = l_run[r] * alpha + warp_sum(p);
      m_run[r] = m_new;
      Ps[row * BKEYS + lane] = p;
#pragma unroll
      for (int c = 0; c < MAX_DV / 32; ++c) acc[r][c] *= alpha;
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < RQ; ++r) {
      const int row = warp * RQ + r;
      if (row >= rows) break;
      const float* pr = Ps + row * BKEYS;
      for (int j = 0; j < BKEYS; ++j) {
        float p = pr[j];
        const float* vr = Vs + j * DV;
#pragma unroll
        for (int c = 0; c < MAX_DV / 32; ++c) {
          int d = lane + 32 * c;
          if (c < NC && d < DV) acc[r][c] = fmaf(p, vr[d], acc[r][c]);
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < RQ; ++r) {
    const int row = warp * RQ + r;
    if (row >= rows) break;
    const size_t head_at = (size_t)(row0 + row) * QH + h;
    if (a.partial_o) {
      // unnormalized sums with their maximum and denominator: ayk_grouped_finish merges the parts
      float* po = a.partial_o + ((size_t)part * a.total_rows * QH + head_at) * DV;
#pragma unroll
      for (int c = 0; c < MAX_DV / 32; ++c) {
        int d = lane + 32 * c;
        if (c < NC && d < DV) po[d] = acc[r][c];
      }
      if (lane == 0) {
        float* pml = a.partial_ml + ((size_t)part * a.total_rows * QH + head_at) * 2;
        pml[0] = m_run[r];
        pml[1] = l_run[r];
      }
    } else {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      T* o = reinterpret_cast<T*>(a.out) + head_at * DV;
      const float* gate = a.gate ? a.gate + (size_t)(row0 + row) * a.gate_stride + (size_t)h * DV : nullptr;
#pragma unroll
      for (int c = 0; c < MAX_DV / 32; ++c) {
        int d = lane + 32 * c;
        if (c < NC && d < DV) {
          float v = acc[r][c] * inv;
          if (gate) v *= 1.0f / (1.0f + expf(-gate[d]));
          o[d] = from_float<T>(v);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ finish --
// One block per (row, output head), one warp per map.  The parts that the row's context reaches are merged:
// the lanes take a part each for the maxima and the parts' factors exp(m_p - M), then the sums are added up
// four parts at a time (loads that do not wait for one another); then
//   maps == 1: out = o * sigmoid(gate) (gate null: o);
//   maps == 2: the partial heads lie [group][map][head of the group]; for output head h = g * hpg + i,
//              o = o1 - lambda * o2, divided by its root mean square over the head's DV numbers (eps
//              under the root), times post_scale, times sigmoid(gate[t, h]) when a gate is given (one
//              number per head).
template <typename C>
__global__ void __launch_bounds__(64)
grouped_finish_kernel(C* __restrict__ out, const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                      const int* __restrict__ positions, int total_rows, int QH, int DV, int parts, int part_keys,
                      int maps, int hpg, const float* __restrict__ gate, long long gate_stride, float lambda,
                      float post_scale, float eps) {
  __shared__ float other[MAX_DV];
  pdl_trigger();
  const int t = blockIdx.x, h = blockIdx.y;
  const int used = part_keys > 0 ? min(parts, positions[t] / part_keys + 1) : 1;
  pdl_wait();
  const int lane = threadIdx.x & 31, m = threadIdx.x >> 5;
  const int H = QH / maps;
  const int NC = (DV + 31) / 32;
  const int qh = maps == 1 ? h : ((h / hpg) * maps + m) * hpg + h % hpg;
  const size_t head_at = (size_t)t * QH + qh;
  const size_t part_stride = (size_t)total_rows * QH;
  float o[MAX_DV / 32];
#pragma unroll
  for (int c = 0; c < MAX_DV / 32; ++c) o[c] = 0.f;
  float L = 0.f, M = -INFINITY;
  if (used == 1) {                                       // an uncut context: the one part as it is
    if (lane == 0) L = partial_ml[head_at * 2 + 1];
    const float* po = partial_o + head_at * DV;
#pragma unroll
    for (int c = 0; c < MAX_DV / 32; ++c) {
      const int d = lane + 32 * c;
      if (c < NC && d < DV) o[c] = po[d];
    }
  } else {
    for (int p = lane; p < used; p += 32) M = fmaxf(M, partial_ml[(p * part_stride + head_at) * 2]);
    M = warp_max(M);
  }
  for (int p0 = 0; p0 < used && used > 1; p0 += 32) {
    const int p = p0 + lane;
    float w = 0.f;
    if (p < used) {
      const float2 ml = *reinterpret_cast<const float2*>(partial_ml + (p * part_stride + head_at) * 2);
      if (ml.y > 0.f) {                                  // else a part in which the row saw no key
        w = expf(ml.x - M);
        L = fmaf(ml.y, w, L);
      }
    }
    const int n = min(32, used - p0);
    for (int j0 = 0; j0 < n; j0 += 4) {
      float wj[4], v[4][MAX_DV / 32];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        wj[j] = __shfl_sync(0xffffffffu, w, (j0 + j) & 31);
        if (j0 + j >= n) wj[j] = 0.f;
        const float* po = partial_o + ((p0 + j0 + j) * part_stride + head_at) * DV;
#pragma unroll
        for (int c = 0; c < MAX_DV / 32; ++c) {
          const int d = lane + 32 * c;
          v[j][c] = (c < NC && d < DV && wj[j] != 0.f) ? po[d] : 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < MAX_DV / 32; ++c) o[c] = fmaf(v[j][c], wj[j], o[c]);
    }
  }
  L = warp_sum(L);
  const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
  for (int c = 0; c < MAX_DV / 32; ++c) o[c] *= inv;
  C* dst = out + ((size_t)t * H + h) * DV;
  if (maps == 1) {
    const float* g = gate ? gate + (size_t)t * gate_stride + (size_t)h * DV : nullptr;
#pragma unroll
    for (int c = 0; c < MAX_DV / 32; ++c) {
      const int d = lane + 32 * c;
      if (c < NC && d < DV) dst[d] = from_float<C>(g ? o[c] / (1.0f + expf(-g[d])) : o[c]);
    }
    return;
  }
  if (m == 1) {
#pragma unroll
    for (int c = 0; c < MAX_DV / 32; ++c) {
      const int d = lane + 32 * c;
      if (c < NC && d < DV) other[d] = o[c];
    }
  }
  __syncthreads();
  if (m != 0) return;
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < MAX_DV / 32; ++c) {
    const int d = lane + 32 * c;
    if (c < NC && d < DV) {
      o[c] = fmaf(-lambda, other[d], o[c]);
      ss = fmaf(o[c], o[c], ss);
    }
  }
  float scale = post_scale / sqrtf(warp_sum(ss) / (float)DV + eps);
  if (gate) scale /= 1.0f + expf(-gate[(size_t)t * gate_stride + h]);
#pragma unroll
  for (int c = 0; c < MAX_DV / 32; ++c) {
    const int d = lane + 32 * c;
    if (c < NC && d < DV) dst[d] = from_float<C>(o[c] * scale);
  }
}

}  // namespace

AYK_EXPORT int ayk_head_norm_prepare(void* qout, void* kpages, void* vpages, const float* proj, long long stride,
                                     const float* qw, const float* kw, const float* mix, const int* row_req,
                                     const int* positions, const int* table, int table_stride, int page_size, int T,
                                     int H, int G, int D, int maps, int v_col0, int v_width, float eps, int writes,
                                     int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  AYK_REQUIRE(G >= 1 && H % G == 0 && maps >= 1 && D >= 1, "ayk_head_norm_prepare: %d heads, %d key heads, %d maps", H, G, maps);
  AYK_REQUIRE(!mix || maps == 1, "ayk_head_norm_prepare: mixed queries take one map");
  AYK_REQUIRE(v_width % G == 0 && G <= 65535, "ayk_head_norm_prepare: values of %d numbers in %d groups", v_width, G);
  const size_t smem = mix ? (size_t)(H / G) * D * sizeof(float) : 0;
  AYK_REQUIRE(smem <= 48 * 1024, "ayk_head_norm_prepare: %d heads of %d do not fit the mixing buffer", H / G, D);
  const int threads = (mix ? H : (H / G) * maps) * D >= 2048 ? 256 : 128;
  const bool vec = D % 4 == 0 && stride % 4 == 0 && v_col0 % 4 == 0 && (v_width / G) % 4 == 0 &&
                   (((uintptr_t)proj | (uintptr_t)qout | (uintptr_t)kpages | (uintptr_t)vpages | (uintptr_t)qw | (uintptr_t)kw) & 15) == 0;
  const int vthreads = 128;                      // four numbers to a lane: four warps cover a group's heads, and more blocks share an SM
  if (vec && dtype == AYK_DTYPE_F32) {
    ayk_launch(head_norm_prepare_vec_kernel<float>, dim3(T, G), dim3(vthreads), smem, stream, (float*)qout, (float*)kpages,
               (float*)vpages, proj, stride, qw, kw, mix, row_req, positions, table, table_stride, page_size, H, G, D, maps,
               v_col0, v_width, eps, writes);
    return ayk_check_launch("ayk_head_norm_prepare");
  }
  if (vec && dtype == AYK_DTYPE_BF16) {
    ayk_launch(head_norm_prepare_vec_kernel<__nv_bfloat16>, dim3(T, G), dim3(vthreads), smem, stream, (__nv_bfloat16*)qout,
               (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages, proj, stride, qw, kw, mix, row_req, positions, table,
               table_stride, page_size, H, G, D, maps, v_col0, v_width, eps, writes);
    return ayk_check_launch("ayk_head_norm_prepare");
  }
  if (dtype == AYK_DTYPE_F32)
    ayk_launch(head_norm_prepare_kernel<float>, dim3(T, G), dim3(threads), smem, stream, (float*)qout, (float*)kpages,
               (float*)vpages, proj, stride, qw, kw, mix, row_req, positions, table, table_stride, page_size, H, G, D, maps,
               v_col0, v_width, eps, writes);
  else if (dtype == AYK_DTYPE_BF16)
    ayk_launch(head_norm_prepare_kernel<__nv_bfloat16>, dim3(T, G), dim3(threads), smem, stream, (__nv_bfloat16*)qout,
               (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages, proj, stride, qw, kw, mix, row_req, positions, table,
               table_stride, page_size, H, G, D, maps, v_col0, v_width, eps, writes);
  else
    return ayk_fail("ayk_head_norm_prepare: unknown dtype %d", dtype);
  return ayk_check_launch("ayk_head_norm_prepare");
}

int ayk_grouped_attention_mma(const GroupedArgs& a, cudaStream_t stream);      // attention_grouped_mma.cu; 1: not taken

static int g_tensor_cores = 1;
// 0: bfloat16 steps run on the FP32 pipes too (for comparing the two kernels).
AYK_EXPORT void ayk_grouped_attention_tensor_cores(int on) { g_tensor_cores = on ? 1 : 0; }

// q [T, QH * DK] dense, of the cache's dtype; keys [pages, page_size, KH, DK], values [pages, page_size, VH,
// DV].  parts > 1: the context is cut into parts of part_keys keys (grid z).  With ``partial_o`` (float32
// [parts, T, QH, DV]) and ``partial_ml`` ([parts, T, QH, 2]) the kernel leaves unnormalized sums, maxima
// and denominators for ayk_grouped_finish; without, it writes out [T, QH * DV] itself (parts must be 1),
// times sigmoid(gate) when ``gate`` (float32 rows of gate_stride, QH * DV used) is given.
AYK_EXPORT int ayk_grouped_attention(void* out, float* partial_o, float* partial_ml, const void* q, const void* kcache,
                                     const void* vcache, const int* table, int table_stride, const int* req_q_start,
                                     const int* req_pos0, int num_req, int total_rows, int QH, int KH, int VH, int DK,
                                     int DV, int page_size, float scale, const float* slopes, int window, int keep_first,
                                     int chunk, const float* gate, long long gate_stride, int parts, int part_keys, int dtype,
                                     cudaStream_t stream) {
  if (num_req == 0 || total_rows == 0) return 0;
  AYK_REQUIRE(DK >= 1 && DK <= 1024 && DV >= 1 && DV <= MAX_DV, "ayk_grouped_attention: head sizes %d / %d (keys up to 1024, values up to %d)", DK, DV, MAX_DV);
  AYK_REQUIRE(KH >= 1 && VH >= 1 && QH % KH == 0 && QH % VH == 0 && QH <= 65535,
              "ayk_grouped_attention: %d query heads cannot share %d key heads and %d value heads", QH, KH, VH);
  AYK_REQUIRE(parts >= 1 && parts <= 65535 && (parts == 1 || (partial_o && partial_ml && part_keys > 0)), "ayk_grouped_attention: bad partition");
  AYK_REQUIRE(!partial_o == !partial_ml, "ayk_grouped_attention: partial sums need both buffers");
  GroupedArgs a;
  a.out = out; a.partial_o = partial_o; a.partial_ml = partial_ml; a.q = q; a.kcache = kcache; a.vcache = vcache;
  a.table = table; a.table_stride = table_stride; a.req_q_start = req_q_start; a.req_pos0 = req_pos0;
  a.num_req = num_req; a.total_rows = total_rows; a.QH = QH; a.KH = KH; a.VH = VH; a.DK = DK; a.DV = DV;
  a.page_size = page_size; a.scale = scale; a.slopes = slopes; a.window = window; a.keep_first = keep_first; a.chunk = chunk;
  a.gate = gate; a.gate_stride = gate_stride; a.part_keys = parts > 1 ? part_keys : 0; a.parts = parts;
  if (dtype == AYK_DTYPE_BF16 && g_tensor_cores) {
    const int rc = ayk_grouped_attention_mma(a, stream);
    if (rc <= 0) return rc;
  }
  const int max_tiles = total_rows / BQ + num_req;
  const size_t smem = ((size_t)BQ * ((DK + 3) & ~3) + (size_t)BKEYS * (DK + 1) + (size_t)BKEYS * DV + (size_t)BQ * BKEYS) * sizeof(float);
  AYK_REQUIRE(smem <= 227 * 1024, "ayk_grouped_attention: keys of %d numbers do not fit shared memory", DK);
  dim3 grid(max_tiles, QH, parts);
  static size_t configured[2] = {0, 0};
  cudaError_t err;
  if (dtype == AYK_DTYPE_F32) {
    if (smem > configured[0]) {
      err = cudaFuncSetAttribute(grouped_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return ayk_fail("ayk_grouped_attention: shared memory %zu: %s", smem, cudaGetErrorString(err));
      configured[0] = smem;
    }
    ayk_launch(grouped_attention_kernel<float>, grid, dim3(WARPS * 32), smem, stream, a);
  } else if (dtype == AYK_DTYPE_BF16) {
    if (smem > configured[1]) {
      err = cudaFuncSetAttribute(grouped_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return ayk_fail("ayk_grouped_attention: shared memory %zu: %s", smem, cudaGetErrorString(err));
      configured[1] = smem;
    }
    ayk_launch(grouped_attention_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), smem, stream, a);
  } else {
    return ayk_fail("ayk_grouped_attention: unknown dtype %d", dtype);
  }
  return ayk_check_launch("ayk_grouped_attention");
}

AYK_EXPORT int ayk_grouped_finish(void* out, const float* partial_o, const float* partial_ml, const int* positions,
                                  int total_rows, int QH, int DV, int parts, int part_keys, int maps, int hpg,
                                  const float* gate, long long gate_stride, float lambda, float post_scale, float eps,
                                  int dtype, cudaStream_t stream) {
  if (total_rows == 0) return 0;
  AYK_REQUIRE(maps == 1 || maps == 2, "ayk_grouped_finish: %d maps", maps);
  AYK_REQUIRE(QH % maps == 0 && hpg >= 1 && (QH / maps) % hpg == 0 && DV <= MAX_DV, "ayk_grouped_finish: heads do not fit");
  const int pk = parts > 1 ? part_keys : 0;
  const int H = QH / maps;
  AYK_REQUIRE(H <= 65535, "ayk_grouped_finish: %d heads", H);
  const dim3 grid(total_rows, H), threads(32 * maps);
  if (dtype == AYK_DTYPE_F32)
    ayk_launch(grouped_finish_kernel<float>, grid, threads, 0, stream, (float*)out, partial_o, partial_ml,
               positions, total_rows, QH, DV, parts, pk, maps, hpg, gate, gate_stride, lambda, post_scale, eps);
  else if (dtype == AYK_DTYPE_BF16)
    ayk_launch(grouped_finish_kernel<__nv_bfloat16>, grid, threads, 0, stream, (__nv_bfloat16*)out,
               partial_o, partial_ml, positions, total_rows, QH, DV, parts, pk, maps, hpg, gate, gate_stride, lambda,
               post_scale, eps);
  else
    return ayk_fail("ayk_grouped_finish: unknown dtype %d", dtype);
  return ayk_check_launch("ayk_grouped_finish");
}
