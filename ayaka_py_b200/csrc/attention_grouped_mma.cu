// The grouped softmax attention (attention_grouped.cu) in bfloat16 on the tensor cores.
//
// The query heads fall into NG = max(KH, VH) groups whose heads read the same key head and the same
// value head.  The rows of a tile are (token, head of one group) pairs, token-major: a block of four
// warps holds 64 of them (16 per warp), so the heads of a group share its loads in prompts and in
// single-token steps alike.  The queries stay in shared memory (a key may be up to 1024 numbers wide,
// too many for registers); keys and values come KT at a time through three buffers, the next two tiles copied
// asynchronously under the products of this one, and only the tiles that the window and the kept first
// tokens leave are visited.  S = Q K^T with mma.sync m16n8k16 (float32 sums); scale, distance bias,
// mask and the running softmax (maximum, denominator, base 2) are 32-bit in the registers of S's
// fragments; the weights enter the second product rounded to bfloat16, as the cached values are; O
// stays in float32 registers and is written either normalized (times the sigmoid of a gate) or, when
// the context is cut into parts or two maps are to be combined, as partial sums for ayk_grouped_finish.
#include <math.h>

#include "attention_grouped.cuh"

namespace {

constexpr int TC_ROWS = 64;
constexpr int NBUF = 3;          // tiles of keys and values in shared memory: the one in use and two on their way
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;                    // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

// DVT: the value width rounded up to 32, 64 or 128 (O's registers); KT: keys per tile; DKP: the key
// width rounded up to a multiple of 16 (the padding is zeros in shared memory).
template <int DVT, int KT>
__global__ void __launch_bounds__(128, DVT > 64 && KT == 64 ? 2 : 3)
grouped_attention_mma_kernel(GroupedArgs a, int page_shift, int tq, int DKP, int qrows) {
  const int LDK = DKP + 8;
  constexpr int LDV = DVT + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [qrows][LDK], qrows = the most live rows of a tile in 16s
  __nv_bfloat16* tiles = Qs + qrows * LDK;                              // NBUF buffers: keys [KT][LDK], values [KT][LDV]
  const int TILE = KT * (LDK + LDV);
  unsigned char* okflag = reinterpret_cast<unsigned char*>(tiles + NBUF * TILE);   // [NBUF][KT]: the key lies on a page
  pdl_trigger();
  pdl_wait();
  const int QH = a.QH, DK = a.DK, DV = a.DV;
  const int NG = max(a.KH, a.VH), hpg = QH / NG;
  int tile = blockIdx.x, req = -1, q0 = 0, q_len = 0;
  if (a.total_rows == a.num_req) {                  // every request brings one row: the tile is the request
    if (tile < a.num_req) { req = tile; q_len = 1; }
  } else {
    for (int r = 0; r < a.num_req; ++r) {
      int len = a.req_q_start[r + 1] - a.req_q_start[r];
      int n = (len + tq - 1) / tq;
      if (tile < n) { req = r; q0 = tile * tq; q_len = len; break; }
      tile -= n;
    }
  }
  if (req < 0) return;
  const int g = blockIdx.y, kh = g / (NG / a.KH), vh = g / (NG / a.VH);
  const int tokens = min(tq, q_len - q0);
  const int rows = tokens * hpg;                    // live rows of the tile, <= 64
  const int row0 = a.req_q_start[req] + q0;
  const int pos0 = a.req_pos0[req] + q0;
  const int last_pos = pos0 + tokens - 1;
  const int part = blockIdx.z;
  const int k_first = a.part_keys > 0 ? part * a.part_keys : 0;
  const int k_last = a.part_keys > 0 ? min(last_pos, k_first + a.part_keys - 1) : last_pos;
  if (k_first > last_pos) return;                   // the merge does not read parts beyond the context
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int* my_table = a.table + (size_t)req * a.table_stride;
  const int page_mask = (1 << page_shift) - 1;
  const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  const __nv_bfloat16* kcache = reinterpret_cast<const __nv_bfloat16*>(a.kcache);
  const __nv_bfloat16* vcache = reinterpret_cast<const __nv_bfloat16*>(a.vcache);
  const int kpieces = DKP / 8, vpieces = DVT / 8;

  // A tile of KT keys and their values in 16-byte pieces; pieces beyond the part, on no page, or in the
  // padding of a head are filled with zeros.  128 / KT threads share a key: one look at the table each, made a
  // tile ahead of the copies that need it (the blocks' shared memory leaves the L1 little room for the table).
  constexpr int TPK = 128 / KT;
  const int fj = tid / TPK, fsub = tid - fj * TPK;
  auto lookup = [&](int k0) {
    const int kp = k0 + fj;
    return (k0 <= k_last && kp <= k_last) ? my_table[kp >> page_shift] : 0;
  };
  auto fetch = [&](int k0, int buf, int page) {
    __nv_bfloat16* Kd = tiles + buf * TILE + fj * LDK;
    __nv_bfloat16* Vd = tiles + buf * TILE + KT * LDK + fj * LDV;
    const int kp = k0 + fj;
    const bool on = page > 0;
    const size_t cell = on ? ((size_t)page << page_shift) + (kp & page_mask) : 0;
    const __nv_bfloat16* ksrc = kcache + (cell * a.KH + kh) * DK;
    const __nv_bfloat16* vsrc = vcache + (cell * a.VH + vh) * DV;
    for (int piece = fsub; piece < kpieces; piece += TPK) {
      const bool live = on && piece * 8 < DK;
      cp_async_16(Kd + piece * 8, live ? ksrc + piece * 8 : kcache, live);
    }
#pragma unroll
    for (int piece = fsub; piece < vpieces; piece += TPK) {
      const bool live = on && piece * 8 < DV;
      cp_async_16(Vd + piece * 8, live ? vsrc + piece * 8 : vcache, live);
    }
    if (fsub == 0) okflag[buf * KT + fj] = on ? 1 : 0;
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const GroupedTiles walk(k_first, k_last, pos0, a.window, a.keep_first, KT, a.chunk);
  // the queries, copied asynchronously as part of the first group (8 threads to a row; dead rows and padding are zeros)
  for (int m = tid >> 3; m < qrows; m += 16) {
    const int tok = m / hpg, head = g * hpg + (m - tok * hpg);
    const bool live_row = m < rows;
    const __nv_bfloat16* src = live_row ? q + ((size_t)(row0 + tok) * QH + head) * DK : q;
    for (int piece = tid & 7; piece < kpieces; piece += 8) {
      const bool live = live_row && piece * 8 < DK;
      cp_async_16(Qs + m * LDK + piece * 8, live ? src + piece * 8 : q, live);
    }
  }
  // every fetch (or its absence) is one group of copies, so that "all but the last two" always means this tile
  int k0 = walk.first();
  int k1 = k0 <= k_last ? walk.next(k0) : k0;
  int k2 = k1 <= k_last ? walk.next(k1) : k1;
  {
    const int page0 = lookup(k0), page1 = lookup(k1);
    if (k0 <= k_last) fetch(k0, 0, page0);
    if (k0 <= k_last && k1 <= k_last) fetch(k1, 1, page1);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  int page2 = lookup(k2);                               // read by the first iteration's fetch, after the queries are staged

  // this thread's two rows: their positions and their heads' slopes (base 2)
  int qpos[2], cstart[2];
  float slope2[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = warp * 16 + gid + half * 8;
    const int tok = m / hpg;
    qpos[half] = m < rows ? pos0 + tok : -1;                       // a dead row sees nothing
    cstart[half] = (a.chunk > 0 && m < rows) ? (pos0 + tok) / a.chunk * a.chunk : 0;      // first key of the row's own chunk
    slope2[half] = (a.slopes && m < rows) ? a.slopes[g * hpg + (m - tok * hpg)] * LOG2E : 0.f;
  }
  const float scale2 = a.scale * LOG2E;
  float o[DVT / 8][4];
#pragma unroll
  for (int nt = 0; nt < DVT / 8; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[nt][c] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};     // l: this thread's share of the row's denominator
  const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (lane >> 4) * 8);
  const int ksteps = DKP / 16;

  int buf = 0;
  for (; k0 <= k_last; buf = buf + 1 == NBUF ? 0 : buf + 1) {
    // the tile after the next streams into the buffer that was read an iteration ago (behind the barrier below)
    if (k2 <= k_last) fetch(k2, buf + 2 >= NBUF ? buf + 2 - NBUF : buf + 2, page2);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const int k3 = k2 <= k_last ? walk.next(k2) : k2;
    page2 = lookup(k3);                                 // for the next iteration's fetch
    asm volatile("cp.async.wait_group 2;" ::: "memory");
    __syncthreads();
    const __nv_bfloat16* Ks = tiles + buf * TILE;
    const __nv_bfloat16* Vs = Ks + KT * LDK;
    if (warp * 16 < rows) {                            // a warp without live rows only helps with the loads
      // S = Q K^T: KT / 8 tiles of 8 keys
      float sc[KT / 8][4];
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[nt][c] = 0.f;
      // key fragments four 8x8 matrices at a time: (keys 0-7 | 8-15 of a pair of tiles) x (dimensions 0-7 | 8-15)
      const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(Ks + ((lane >> 4) * 8 + (lane & 7)) * LDK + ((lane >> 3) & 1) * 8);
#pragma unroll 2
      for (int ks = 0; ks < ksteps; ++ks) {
        uint32_t qf[4];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(qf[0]), "=r"(qf[1]), "=r"(qf[2]), "=r"(qf[3]) : "r"(q_addr + ks * 32));
#pragma unroll
        for (int np = 0; np < KT / 16; ++np) {
          uint32_t b0, b1, b2, b3;
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(k_addr + (uint32_t)(np * 16 * LDK + ks * 16) * 2u));
          mma_bf16(sc[2 * np], qf, b0, b1);
          mma_bf16(sc[2 * np + 1], qf, b2, b3);
        }
      }
      // scores in base 2, masked; fragment element c of tile nt: row gid + 8 (c / 2), key k0 + 8 nt + 2 tig + (c & 1)
      const bool inside = k0 + KT - 1 <= min(pos0, k_last) && (a.window <= 0 || last_pos - k0 < a.window) &&
                          (a.chunk <= 0 || k0 >= last_pos / a.chunk * a.chunk);   // dead rows are never written
      const unsigned char* ok = okflag + buf * KT + tig * 2;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int key = k0 + nt * 8 + tig * 2 + (c & 1), i = qpos[c >> 1];
          float s = fmaf(-slope2[c >> 1], (float)(i - key), sc[nt][c] * scale2);
          if (!inside) {
            const bool seen = key <= min(i, k_last) && (a.window <= 0 || i - key < a.window || key < a.keep_first) &&
                              key >= cstart[c >> 1] && ok[nt * 8 + (c & 1)] != 0;
            s = seen ? s : -INFINITY;
          }
          sc[nt][c] = s;
          mx[c >> 1] = fmaxf(mx[c >> 1], s);
        }
      float alpha[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float m = mx[half];
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        const float m_new = fmaxf(m_run[half], m);
        alpha[half] = m_new > -INFINITY ? fast_exp2(m_run[half] - m_new) : 1.f;     // 2^(-inf) = 0 on the first visible tile
        m_run[half] = m_new;
        mx[half] = m_new > -INFINITY ? m_new : 0.f;                                 // nothing seen yet: every weight is 2^(-inf) = 0
      }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float p = fast_exp2(sc[nt][c] - mx[c >> 1]);
          sc[nt][c] = p;
          sum[c >> 1] += p;
        }
#pragma unroll
      for (int half = 0; half < 2; ++half) l_run[half] = fmaf(l_run[half], alpha[half], sum[half]);
#pragma unroll
      for (int nt = 0; nt < DVT / 8; ++nt) {
        o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0];
        o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
      }
      // O += P V: the 32-bit weights enter the product rounded to bfloat16, as the values they multiply are
#pragma unroll
      for (int ks = 0; ks < KT / 16; ++ks) {
        uint32_t pf[4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
          pf[r] = pack_bf16(sc[2 * ks + (r >> 1)][(r & 1) * 2], sc[2 * ks + (r >> 1)][(r & 1) * 2 + 1]);
#pragma unroll
        for (int np = 0; np < DVT / 16; ++np) {
          // two value tiles (16 columns) at a time: four 8x8 matrices, transposed on the way in
          uint32_t b0, b1, b2, b3;
          const __nv_bfloat16* at = Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + np * 16 + (lane >> 4) * 8;
          const uint32_t addr = (uint32_t)__cvta_generic_to_shared(at);
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
          mma_bf16(o[2 * np], pf, b0, b1);
          mma_bf16(o[2 * np + 1], pf, b2, b3);
        }
      }
    }
    __syncthreads();                                   // this buffer is refilled by the next iteration's fetch
    k0 = k1;
    k1 = k2;
    k2 = k3;
  }

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float l = l_run[half];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int m = warp * 16 + gid + half * 8;
    if (m >= rows) continue;
    const int tok = m / hpg, head = g * hpg + (m - tok * hpg);
    const size_t head_at = (size_t)(row0 + tok) * QH + head;
    if (a.partial_o) {
      float* po = a.partial_o + ((size_t)part * a.total_rows * QH + head_at) * DV;
#pragma unroll
      for (int nt = 0; nt < DVT / 8; ++nt) {
        const int col = nt * 8 + tig * 2;
        if (col < DV) *reinterpret_cast<float2*>(po + col) = make_float2(o[nt][half * 2], o[nt][half * 2 + 1]);
      }
      if (tig == 0) {
        float* pml = a.partial_ml + ((size_t)part * a.total_rows * QH + head_at) * 2;
        pml[0] = m_run[half] * LN2;                    // the merge works in base e
        pml[1] = l;
      }
    } else {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.out) + head_at * DV;
      const float* gate = a.gate ? a.gate + (size_t)(row0 + tok) * a.gate_stride + (size_t)head * DV : nullptr;
      float gv[DVT / 8][2];                            // all the gates first: loads that do not wait for the stores
#pragma unroll
      for (int nt = 0; nt < DVT / 8; ++nt) {
        const int col = nt * 8 + tig * 2;
        const bool on = gate != nullptr && col < DV;
        gv[nt][0] = on ? __ldg(gate + col) : 0.f;
        gv[nt][1] = on ? __ldg(gate + col + 1) : 0.f;
      }
#pragma unroll
      for (int nt = 0; nt < DVT / 8; ++nt) {
        const int col = nt * 8 + tig * 2;
        if (col >= DV) continue;
        float v0 = o[nt][half * 2] * inv, v1 = o[nt][half * 2 + 1] * inv;
        if (gate) {
          v0 = __fdividef(v0, 1.0f + __expf(-gv[nt][0]));
          v1 = __fdividef(v1, 1.0f + __expf(-gv[nt][1]));
        }
        *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(v0, v1);
      }
    }
  }
}

template <int DVT, int KT>
int launch(const GroupedArgs& a, int page_shift, int tq, int DKP, int qrows, size_t smem, dim3 grid, cudaStream_t stream) {
  static AykPerDevice granted;
  static size_t most = 0;
  if (!granted.here() || smem > most) {
    cudaError_t e = cudaFuncSetAttribute(grouped_attention_mma_kernel<DVT, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(227 * 1024));
    if (e != cudaSuccess) return ayk_fail("ayk_grouped_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
    granted.here() = true;
    most = 227 * 1024;
  }
  ayk_launch(grouped_attention_mma_kernel<DVT, KT>, grid, dim3(128), smem, stream, a, page_shift, tq, DKP, qrows);
  return ayk_check_launch("ayk_grouped_attention (tensor cores)");
}

size_t smem_bytes(int DKP, int DVT, int KT, int qrows) {
  return ((size_t)qrows * (DKP + 8) + (size_t)NBUF * KT * (DKP + 8 + DVT + 8)) * sizeof(__nv_bfloat16) + NBUF * KT;
}

}  // namespace

// 0: launched; 1: this geometry is left to the kernel on the FP32 pipes; < 0: an error.
int ayk_grouped_attention_mma(const GroupedArgs& a, cudaStream_t stream) {
  const int NG = a.KH > a.VH ? a.KH : a.VH;
  if (NG % a.KH || NG % a.VH || a.QH % NG) return 1;
  const int hpg = a.QH / NG;
  if (hpg > TC_ROWS || a.DK % 8 || a.DV % 8 || a.DV > 128) return 1;
  int page_shift = 0;
  while ((1 << page_shift) < a.page_size) ++page_shift;
  if ((1 << page_shift) != a.page_size) return 1;
  const int DKP = (a.DK + 15) & ~15;
  const int DVT = a.DV <= 32 ? 32 : (a.DV <= 64 ? 64 : 128);
  // every request brings one row: a tile holds the heads of one token, and only their rows are staged
  const bool single = a.total_rows == a.num_req;
  const int tq = single ? 1 : TC_ROWS / hpg;
  const int qrows = (tq * hpg + 15) & ~15;
  // 64 keys a tile while two blocks still fit a multiprocessor, else 32
  // (values of 128 leave registers for two blocks of 64-key tiles, or three of 32-key tiles when those fit)
  int KT = 64;
  if (smem_bytes(DKP, DVT, 64, qrows) > 112 * 1024) KT = 32;
  else if (DVT == 128 && !single && smem_bytes(DKP, DVT, 32, qrows) <= 74 * 1024) KT = 32;
  const size_t smem = smem_bytes(DKP, DVT, KT, qrows);
  if (smem > 227 * 1024) return 1;
  dim3 grid(single ? a.total_rows : a.total_rows / tq + a.num_req, NG, a.parts);
#define AYK_GROUPED(V, K) \
  if (DVT == V && KT == K) return launch<V, K>(a, page_shift, tq, DKP, qrows, smem, grid, stream);
  AYK_GROUPED(32, 64) AYK_GROUPED(64, 64) AYK_GROUPED(128, 64) AYK_GROUPED(32, 32) AYK_GROUPED(64, 32) AYK_GROUPED(128, 32)
#undef AYK_GROUPED
  return 1;
}
