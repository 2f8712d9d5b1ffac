// Latent attention on the tensor cores (bfloat16 operands, 32-bit scores, weights and sums), and the
// small per-head matrix products in front of and behind it.
//
// The same arithmetic as latent.cu: a head's query is [U_k^T q_n ; q_r] (rank + rot numbers), a key
// is the cached pair [c ; k_r], the weighted sum runs over c.  All heads share the keys, so a block
// takes 16 x WM (row, head) pairs of one request -- BR consecutive rows times HG heads -- against one
// tile of 32 cached positions at a time:
//   S = Q K^T      mma.sync m16n8k16, Q [pairs, rank + rot] and the key tile in shared memory
//   online softmax in registers (exp2, running maximum and sum per pair)
//   O += P C       the key tile's first rank columns are the values
// A warp owns 16 pairs and RPW columns of O (accumulators in registers); when the latent is wider
// than RPW, two warps share the pairs: each computes S for half of the tile's positions and hands it to the other.  With one row per
// request (decoding) a block has WM = 1 and the context is cut into partitions of PART positions
// (grid.z) whose partial results (maximum, sum, unnormalised O) a second kernel merges.
//
// tcgen05 is not used here: O for 128 pairs x 512 columns would fill tensor memory alone, and
// the score tile's K extent (rank + rot up to 576) wants operands staged in more shared memory
// than one SM has beside it; the warp-level form keeps O in registers and works for every latent
// size that is a multiple of 8.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int NK = 32;          // cached positions per tile

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async_16(void* smem_ptr, const void* gmem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(gmem_ptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// partial: [pairs of the step = T * H][parts][2 + rank] floats (maximum in the log2 domain, sum, O).
template <int RPW, int CG, int WM>
__global__ void __launch_bounds__(32 * WM * CG)
latent_attention_mma_kernel(float* __restrict__ out, float* __restrict__ partial, const float* __restrict__ query,
                            const __nv_bfloat16* __restrict__ latent_pages, const __nv_bfloat16* __restrict__ rope_pages,
                            const int* __restrict__ table, int table_stride, const int* __restrict__ req_q_start,
                            const int* __restrict__ req_pos0, int num_req, int H, int HG, int BR, int rank, int rot,
                            int page_size, float scale_log2, int parts, int part_keys) {
  constexpr int AQ = 16 * WM;
  pdl_trigger();
  // the last tiles of a request see the most keys: they start first (blocks are handed out in order)
  int tile = gridDim.x - 1 - blockIdx.x, req = -1, q0 = 0, q_len = 0;
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
  const int last_pos = pos0 + rows - 1;
  const int part = blockIdx.z;
  const int key_lo = part * part_keys;
  const int key_hi = parts > 1 ? min(last_pos, key_lo + part_keys - 1) : last_pos;      // inclusive
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp % WM, cg = warp / WM;
  const int g = lane >> 2, t4 = lane & 3;
  const int Dk = rank + rot;
  const int Dp = (Dk + 15) & ~15;
  const int ld = Dp + 8;                     // bf16 elements per row of the tiles: rows shift by 16 bytes

  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [AQ][ld]
  __nv_bfloat16* Ks = Qs + AQ * ld;                                    // two buffers of [NK][ld]
  int* there = reinterpret_cast<int*>(Ks + 2 * NK * ld);                // per buffer and position: is it cached (a page, inside the range)
  float* shared_scores = reinterpret_cast<float*>(there + 2 * NK);      // CG = 2: per warp 2 x 4 x 32 scores for its partner
  const int* my_table = table + (size_t)req * table_stride;

  pdl_wait();
  if (parts > 1 && key_lo > key_hi) {        // a partition beyond the context: nothing seen
    for (int pr = threadIdx.x; pr < AQ; pr += blockDim.x) {
      const int r = pr / HG, hh = pr - r * HG;
      if (r < rows && hh < heads && pr < BR * HG) {
        float* dst = partial + (((size_t)(row0 + r) * H + h0 + hh) * parts + part) * (size_t)(rank + 2);
        dst[0] = -INFINITY;
        dst[1] = 0.f;
      }
    }
    return;
  }
  // the pairs' queries as bfloat16 (rank and rot are multiples of 8, so a pair's row is whole float4s;
  // the padding columns are zeros)
  const int quads = Dp / 4;
#pragma unroll 4
  for (int i = threadIdx.x; i < AQ * quads; i += blockDim.x) {
    const int pr = i / quads, d = (i - pr * quads) * 4;
    const int r = pr / HG, hh = pr - r * HG;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows && hh < heads && pr < BR * HG && d < Dk)
      v = *reinterpret_cast<const float4*>(query + ((size_t)(row0 + r) * H + h0 + hh) * Dk + d);
    uint2 packed;
    packed.x = pack_bf16(v.x, v.y);
    packed.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(Qs + pr * ld + d) = packed;
  }

  // this thread's two pairs: rows g and g + 8 of the warp's 16
  int qpos[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int pr = wm * 16 + g + 8 * e;
    const int r = pr / HG, hh = pr - r * HG;
    qpos[e] = (r < rows && hh < heads && pr < BR * HG) ? pos0 + r : -1;
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[RPW / 8][4];
#pragma unroll
  for (int j = 0; j < RPW / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  const int col0 = cg * RPW;                 // first column of O that this warp owns

  // A tile of 32 cached positions: a warp copies whole rows (16-byte pieces, asynchronously); rows that
  // are not there (beyond the range, the padding page) and the padding columns are zeros.  Two
  // buffers: tile i + 1 is on its way while tile i is used.
  const int chunks_lat = rank / 8, chunks_rot = rot / 8, chunks = Dp / 8;
  const int nwarps = WM * CG;
  auto fetch = [&](int k0, __nv_bfloat16* dst, int* flags) {
    for (int j = warp; j < NK; j += nwarps) {
      const int kp = k0 + j;
      int page = 0;
      if (kp <= key_hi) page = my_table[kp / page_size];
      const size_t at = (size_t)page * page_size + (kp % page_size);
      if (lane == 0) flags[j] = page > 0;
      for (int c = lane; c < chunks; c += 32) {
        __nv_bfloat16* to = dst + j * ld + c * 8;
        if (page > 0 && c < chunks_lat) cp_async_16(to, latent_pages + at * rank + c * 8);
        else if (page > 0 && c < chunks_lat + chunks_rot) cp_async_16(to, rope_pages + at * rot + (c - chunks_lat) * 8);
        else *reinterpret_cast<uint4*>(to) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    cp_async_commit();
  };
  __nv_bfloat16* Kbuf[2] = {Ks, Ks + NK * ld};
  if (key_lo <= key_hi) fetch(key_lo, Kbuf[0], there);
  int it = 0;
  for (int k0 = key_lo; k0 <= key_hi; k0 += NK, ++it) {
    const bool more = k0 + NK <= key_hi;
    if (more) fetch(k0 + NK, Kbuf[(it + 1) & 1], there + ((it + 1) & 1) * NK);
    if (more) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    const __nv_bfloat16* Kt = Kbuf[it & 1];
    const int* cached = there + (it & 1) * NK;

    // S = Q K^T for the warp's 16 pairs and the tile's 32 positions.  Two warps that share their pairs
    // (CG = 2) each take 16 of the positions and hand the other its scores through shared memory.
    float s[NK / 8][4];
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    if (CG == 2) {
      float own[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, other[2][4];
#pragma unroll 4
      for (int ks = 0; ks < Dp; ks += 16) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, Qs + (wm * 16 + (lane & 15)) * ld + ks + (lane >> 4) * 8);
        ldmatrix_x4(b, Kt + (cg * 16 + (lane & 7) + ((lane >> 4) << 3)) * ld + ks + ((lane >> 3) & 1) * 8);
        mma_bf16(own[0], a, b[0], b[1]);
        mma_bf16(own[1], a, b[2], b[3]);
      }
      float* mine = shared_scores + ((wm * 2 + cg) * 2) * 128;          // [2 tiles of 8 positions][4 values][32 lanes]
      const float* theirs = shared_scores + ((wm * 2 + (1 - cg)) * 2) * 128;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) mine[(j * 4 + e) * 32 + lane] = own[j][e];
      asm volatile("bar.sync %0, 64;" ::"r"(1 + wm) : "memory");      // the two warps of this group of pairs
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) other[j][e] = theirs[(j * 4 + e) * 32 + lane];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[j][e] = cg == 0 ? own[j][e] : other[j][e];
          s[2 + j][e] = cg == 0 ? other[j][e] : own[j][e];
        }
    } else {
#pragma unroll 4
      for (int ks = 0; ks < Dp; ks += 16) {
        uint32_t a[4];
        ldmatrix_x4(a, Qs + (wm * 16 + (lane & 15)) * ld + ks + (lane >> 4) * 8);
#pragma unroll
        for (int jp = 0; jp < NK / 16; ++jp) {
          uint32_t b[4];
          ldmatrix_x4(b, Kt + (jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * ld + ks + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * jp], a, b[0], b[1]);
          mma_bf16(s[2 * jp + 1], a, b[2], b[3]);
        }
      }
    }
    // scale, mask, running maximum
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kj = j * 8 + 2 * t4 + (e & 1);
        const int which = e >> 1;
        const bool valid = k0 + kj <= qpos[which] && cached[kj];
        s[j][e] = valid ? s[j][e] * scale_log2 : -INFINITY;
        m_new[which] = fmaxf(m_new[which], s[j][e]);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 1));
      m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 2));
      m_use[e] = m_new[e] == -INFINITY ? 0.f : m_new[e];
      alpha[e] = exp2f(m_run[e] - m_use[e]);        // exp2(-inf) = 0 before the first visible key
      m_run[e] = m_new[e];
      l_run[e] *= alpha[e];
    }
    uint32_t p[NK / 16][4];
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) {
      const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
      const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      p[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
      p[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int j = 0; j < RPW / 8; ++j) {
      o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
      o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
    }
    // O += P C over the warp's columns
#pragma unroll
    for (int kk = 0; kk < NK / 16; ++kk) {
#pragma unroll
      for (int jp = 0; jp < RPW / 16; ++jp) {
        const int d0 = col0 + jp * 16;
        if (d0 < rank) {                       // warp-uniform
          uint32_t b[4];
          ldmatrix_x4_trans(b, Kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + d0 + (lane >> 4) * 8);
          mma_bf16(o[2 * jp], p[kk], b[0], b[1]);
          mma_bf16(o[2 * jp + 1], p[kk], b[2], b[3]);
        }
      }
    }
    __syncthreads();        // the buffer is free for the tile after the next
  }

  // the sums of a pair are spread over the four threads of its quad
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    if (qpos[e] < 0) continue;
    const int pr = wm * 16 + g + 8 * e;
    const int r = pr / HG, hh = pr - r * HG;
    const size_t pair = (size_t)(row0 + r) * H + h0 + hh;
    if (parts > 1) {
      float* dst = partial + (pair * parts + part) * (size_t)(rank + 2);
      if (cg == 0 && t4 == 0) { dst[0] = m_run[e]; dst[1] = l_run[e]; }
#pragma unroll
      for (int j = 0; j < RPW / 8; ++j) {
        const int d = col0 + j * 8 + 2 * t4;
        if (d < rank) { dst[2 + d] = o[j][2 * e]; dst[2 + d + 1] = o[j][2 * e + 1]; }
      }
    } else {
      const float inv = l_run[e] > 0.f ? 1.f / l_run[e] : 0.f;
      float* dst = out + pair * rank;
#pragma unroll
      for (int j = 0; j < RPW / 8; ++j) {
        const int d = col0 + j * 8 + 2 * t4;
        if (d < rank) *reinterpret_cast<float2*>(dst + d) = make_float2(o[j][2 * e] * inv, o[j][2 * e + 1] * inv);
      }
    }
  }
}

// out[pair, :] = sum_p exp2(m_p - m) O_p / sum_p exp2(m_p - m) l_p, partitions in order.  The
// partitions' maxima and sums are fetched side by side first; a partition that saw nothing is skipped.
constexpr int MERGE_PARTS = 1024;
__global__ void latent_merge_kernel(float* __restrict__ out, const float* __restrict__ partial, int rank, int parts) {
  __shared__ float weight[MERGE_PARTS];
  __shared__ float total[2];
  pdl_trigger();
  pdl_wait();
  const float* src = partial + (size_t)blockIdx.x * parts * (rank + 2);
  for (int p = threadIdx.x; p < parts; p += blockDim.x) weight[p] = src[(size_t)p * (rank + 2)];
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = -INFINITY;
    for (int p = 0; p < parts; ++p) m = fmaxf(m, weight[p]);
    total[0] = m;
  }
  __syncthreads();
  const float m = total[0];
  for (int p = threadIdx.x; p < parts; p += blockDim.x) {
    const float mp = weight[p];
    weight[p] = mp > -INFINITY ? exp2f(mp - m) : 0.f;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float l = 0.f;
    for (int p = 0; p < parts; ++p)
      if (weight[p] > 0.f) l = fmaf(weight[p], src[(size_t)p * (rank + 2) + 1], l);
    total[1] = l > 0.f ? 1.f / l : 0.f;
  }
  __syncthreads();
  const float inv = total[1];
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float acc = 0.f;
    for (int p = 0; p < parts; ++p) {
      const float wp = weight[p];
      if (wp > 0.f) acc = fmaf(wp, src[(size_t)p * (rank + 2) + 2 + d], acc);
    }
    out[(size_t)blockIdx.x * rank + d] = acc * inv;
  }
}

// ------------------------------------------------------- per-head products --
// out[t, h, n] = (sum_k a[t, h, k] w[h, n, k]) (* sigmoid(gate[t, h * gate_head + n * gate_col]): gate_head 1 and gate_col 0 for a number per head, gate_head N and gate_col 1 for a number per output) with bfloat16 weights on the
// tensor cores: a block takes 64 rows x 64 columns of one head, K in chunks of 64.  The float32
// operand goes into shared memory as two bfloat16 parts (its rounding and what the rounding left
// over), each multiplied with the weights, so that it keeps 16 bits of mantissa; sums are 32-bit.
constexpr int PM = 64, PN = 64, PK = 64, PLD = PK + 8;

template <typename O>
__global__ void __launch_bounds__(128)
head_matmul_mma_kernel(O* __restrict__ out, long long out_row, int out_head, const float* __restrict__ a, long long a_row,
                       int a_head, const __nv_bfloat16* __restrict__ w, const float* __restrict__ gate, long long gate_row, int gate_head, int gate_col,
                       int T, int N, int K) {
  __shared__ __align__(16) __nv_bfloat16 As[PM * PLD];
  __shared__ __align__(16) __nv_bfloat16 Al[PM * PLD];       // what rounding to bfloat16 left over
  __shared__ __align__(16) __nv_bfloat16 Ws[PN * PLD];
  pdl_trigger();
  const int h = blockIdx.y, t0 = blockIdx.x * PM, n0 = blockIdx.z * PN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const __nv_bfloat16* wh = w + (size_t)h * N * K;
  float acc[PN / 8][4];
#pragma unroll
  for (int j = 0; j < PN / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  pdl_wait();
  for (int k0 = 0; k0 < K; k0 += PK) {
    __syncthreads();
    for (int i = threadIdx.x; i < PM * (PK / 4); i += 128) {        // four floats of a at a time
      const int r = i / (PK / 4), c = (i - r * (PK / 4)) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t0 + r < T && k0 + c < K) v = *reinterpret_cast<const float4*>(a + (size_t)(t0 + r) * a_row + (size_t)h * a_head + k0 + c);
      const __nv_bfloat162 h01 = __floats2bfloat162_rn(v.x, v.y), h23 = __floats2bfloat162_rn(v.z, v.w);
      uint2 hi, lo;
      hi.x = *reinterpret_cast<const uint32_t*>(&h01);
      hi.y = *reinterpret_cast<const uint32_t*>(&h23);
      lo.x = pack_bf16(v.x - __bfloat162float(h01.x), v.y - __bfloat162float(h01.y));
      lo.y = pack_bf16(v.z - __bfloat162float(h23.x), v.w - __bfloat162float(h23.y));
      *reinterpret_cast<uint2*>(As + r * PLD + c) = hi;
      *reinterpret_cast<uint2*>(Al + r * PLD + c) = lo;
    }
    for (int i = threadIdx.x; i < PN * (PK / 8); i += 128) {        // eight weights at a time
      const int r = i / (PK / 8), c = (i - r * (PK / 8)) * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (n0 + r < N && k0 + c < K) v = *reinterpret_cast<const uint4*>(wh + (size_t)(n0 + r) * K + k0 + c);
      *reinterpret_cast<uint4*>(Ws + r * PLD + c) = v;
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < PK; ks += 16) {
      uint32_t af[4], al[4];
      ldmatrix_x4(af, As + (warp * 16 + (lane & 15)) * PLD + ks + (lane >> 4) * 8);
      ldmatrix_x4(al, Al + (warp * 16 + (lane & 15)) * PLD + ks + (lane >> 4) * 8);
#pragma unroll
      for (int jp = 0; jp < PN / 16; ++jp) {
        uint32_t b[4];
        ldmatrix_x4(b, Ws + (jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * PLD + ks + ((lane >> 3) & 1) * 8);
        mma_bf16(acc[2 * jp], al, b[0], b[1]);
        mma_bf16(acc[2 * jp + 1], al, b[2], b[3]);
        mma_bf16(acc[2 * jp], af, b[0], b[1]);
        mma_bf16(acc[2 * jp + 1], af, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int t = t0 + warp * 16 + g + 8 * e;
    if (t >= T) continue;
    const float* grow = gate ? gate + (size_t)t * gate_row + (size_t)h * gate_head : nullptr;
    const float scale = (gate && gate_col == 0) ? 1.0f / (1.0f + expf(-grow[0])) : 1.0f;
    O* dst = out + (size_t)t * out_row + (size_t)h * out_head;
#pragma unroll
    for (int j = 0; j < PN / 8; ++j) {
      const int n = n0 + j * 8 + 2 * t4;
      float s0 = scale, s1 = scale;
      if (gate && gate_col != 0) {                    // a gate per output number
        if (n < N) s0 = 1.0f / (1.0f + expf(-grow[(size_t)n * gate_col]));
        if (n + 1 < N) s1 = 1.0f / (1.0f + expf(-grow[(size_t)(n + 1) * gate_col]));
      }
      if (n < N) dst[n] = from_float<O>(acc[j][2 * e] * s0);
      if (n + 1 < N) dst[n + 1] = from_float<O>(acc[j][2 * e + 1] * s1);
    }
  }
}

template <int RPW, int CG, int WM>
int launch(float* out, float* partial, const float* query, const void* latent_pages, const void* rope_pages, const int* table,
           int table_stride, const int* req_q_start, const int* req_pos0, int num_req, int total_rows, int H, int rank, int rot,
           int page_size, float scale, int parts, int part_keys, cudaStream_t stream) {
  constexpr int AQ = 16 * WM;
  const int HG = H < AQ ? H : AQ;
  const int BR = AQ / HG;
  const int Dp = (rank + rot + 15) & ~15;
  const size_t smem = (size_t)(AQ + 2 * NK) * (Dp + 8) * sizeof(__nv_bfloat16) + 2 * NK * sizeof(int) + (CG == 2 ? (size_t)WM * 2 * 2 * 128 * sizeof(float) : 0);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(latent_attention_mma_kernel<RPW, CG, WM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return ayk_fail("ayk_latent_attention_mma: shared memory %zu: %s", smem, cudaGetErrorString(err));
    configured = smem;
  }
  dim3 grid(total_rows / BR + num_req, (H + HG - 1) / HG, parts);
  ayk_launch(latent_attention_mma_kernel<RPW, CG, WM>, grid, dim3(32 * WM * CG), smem, stream, out, partial, query,
             (const __nv_bfloat16*)latent_pages, (const __nv_bfloat16*)rope_pages, table, table_stride, req_q_start, req_pos0,
             num_req, H, HG, BR, rank, rot, page_size, scale * 1.4426950408889634f, parts, part_keys);
  return ayk_check_launch("ayk_latent_attention_mma");
}

}  // namespace

// Whether the tensor-core kernel takes these sizes: 16-byte pieces of the cached rows, O within the registers.
AYK_EXPORT int ayk_latent_attention_mma_takes(int rank, int rot) {
  return rank >= 8 && rank % 8 == 0 && rot % 8 == 0 && rank <= 512 && rank + rot <= 1024;
}

// As ayk_latent_attention, bfloat16 pages.  parts > 1 (only with one row per request): the context
// is cut into partitions of part_keys positions; partial holds T * H * parts * (rank + 2) floats.
AYK_EXPORT int ayk_latent_attention_mma(float* out, float* partial, const float* query, const void* latent_pages,
                                        const void* rope_pages, const int* table, int table_stride, const int* req_q_start,
                                        const int* req_pos0, int num_req, int total_rows, int max_q_len, int H, int rank,
                                        int rot, int page_size, float scale, int parts, int part_keys, int* launched,
                                        cudaStream_t stream) {
  if (launched) *launched = 0;
  if (num_req == 0 || total_rows == 0) return 0;
  AYK_REQUIRE(ayk_latent_attention_mma_takes(rank, rot), "ayk_latent_attention_mma: latent %d + %d is not taken", rank, rot);
  AYK_REQUIRE(parts == 1 || max_q_len == 1, "ayk_latent_attention_mma: the context is cut only for single rows");
  AYK_REQUIRE(parts >= 1 && parts <= MERGE_PARTS && (parts == 1 || part_keys % NK == 0), "ayk_latent_attention_mma: %d partitions of %d", parts, part_keys);
  const bool single = max_q_len == 1 && H <= 16;
  int rc;
#define AYK_LM(RPW, CG)                                                                                                     \
  rc = single ? launch<RPW, CG, 1>(out, partial, query, latent_pages, rope_pages, table, table_stride, req_q_start, req_pos0, \
                                   num_req, total_rows, H, rank, rot, page_size, scale, parts, part_keys, stream)             \
              : launch<RPW, CG, 4>(out, partial, query, latent_pages, rope_pages, table, table_stride, req_q_start, req_pos0, \
                                   num_req, total_rows, H, rank, rot, page_size, scale, parts, part_keys, stream)
  if (rank <= 64) { AYK_LM(64, 1); }
  else if (rank <= 128) { AYK_LM(128, 1); }
  else if (rank <= 256) { AYK_LM(256, 1); }
  else { AYK_LM(256, 2); }
#undef AYK_LM
  if (rc != 0) return rc;
  if (launched) *launched = 1;
  if (parts > 1) {
    ayk_launch(latent_merge_kernel, dim3(total_rows * H), dim3(rank >= 256 ? 128 : 64), 0, stream, out, (const float*)partial, rank, parts);
    if (launched) *launched = 2;
    return ayk_check_launch("ayk_latent_attention_mma (merge)");
  }
  return 0;
}

// As ayk_head_matmul for bfloat16 weights, on the tensor cores.  K a multiple of 8, the float32
// operand's rows and heads on 16-byte boundaries (the caller checks with ayk_head_matmul_mma_takes).
AYK_EXPORT int ayk_head_matmul_mma_takes(const void* a, long long a_row, int a_head, int K) {
  return K % 8 == 0 && a_row % 4 == 0 && a_head % 4 == 0 && (uintptr_t)a % 16 == 0;
}

AYK_EXPORT int ayk_head_matmul_mma(void* out, long long out_row, int out_head, const float* a, long long a_row, int a_head,
                                   const void* w, const float* gate, long long gate_row, int gate_head, int gate_col, int T, int H, int N, int K,
                                   int out_dtype, cudaStream_t stream) {
  if (T == 0 || H == 0 || N == 0) return 0;
  AYK_REQUIRE(ayk_head_matmul_mma_takes(a, a_row, a_head, K), "ayk_head_matmul_mma: operand layout is not taken (K %d)", K);
  dim3 grid((T + PM - 1) / PM, H, (N + PN - 1) / PN);
  AYK_REQUIRE(H <= 65535 && grid.z <= 65535, "ayk_head_matmul_mma: too many heads or columns");
  if (out_dtype == AYK_DTYPE_F32)
    ayk_launch(head_matmul_mma_kernel<float>, grid, dim3(128), 0, stream, (float*)out, out_row, out_head, a, a_row, a_head,
               (const __nv_bfloat16*)w, gate, gate_row, gate_head, gate_col, T, N, K);
  else if (out_dtype == AYK_DTYPE_BF16)
    ayk_launch(head_matmul_mma_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (__nv_bfloat16*)out, out_row, out_head, a,
               a_row, a_head, (const __nv_bfloat16*)w, gate, gate_row, gate_head, gate_col, T, N, K);
  else
    return ayk_fail("ayk_head_matmul_mma: unknown dtype %d", out_dtype);
  return ayk_check_launch("ayk_head_matmul_mma");
}
