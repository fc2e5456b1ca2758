// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, 32-bit accumulation) with the options a
// design may combine, for prompt portions and for decoding; keys of 64 or 128 entries and, separately, values of 64 or 128.
//
//   score = scale q.k, optionally capped (c tanh(score / c)); the row at position i sees key j <= i when there is no
//   window, or i - j < window, or j < keep_first; softmax in 32-bit; o = a v; the output optionally turned back by the
//   row's own position (halves layout: entry m with entry m + VD / 2, by -i f_m), optionally times sigmoid(gate) entry by
//   entry, times `out_scale`; written to rows of `ld_out` entries (a column slice of a wider tensor will do)
//
// One CTA of four warps takes a tile of query rows of one request and one KV head. The G query heads of that KV head are
// packed into the tile's 64 M rows (M row m = query row m / G, head m % G), so keys and values are read once for the whole
// group. Keys and values come in tiles of 64 aligned to absolute positions through a ring of cp.async stages into swizzled
// shared memory: first the tiles of the kept first tokens that lie before the window's tiles, then the window's. Scores,
// the running maximum, the sum and the output stay in registers. When every tile of the launch has at most 16 M rows in use
// (decoding), the four warps share those rows and split each key tile among themselves, 16 keys a warp, and are merged in
// warp order at the end. The order of a row's additions depends on its position only.
#include "common.cuh"

namespace tl {
namespace fx {

constexpr int KT = 64;            // keys a tile

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;          // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold N bf16 (N >= 64): chunks are XOR-swizzled by
// the row so that the eight rows an ldmatrix reads fall into different banks.
template <int N> __device__ __forceinline__ int swz(int row, int chunk) { return row * (N * 2) + ((chunk ^ (row & 7)) << 4); }

// The CTAs of a thread-block cluster (a launch without one is a cluster of one CTA): how many, which one this is, the
// barrier of all their threads, and a 32-bit float read from the same shared-memory place of another CTA.
__device__ __forceinline__ uint32_t cluster_ctas() { uint32_t n; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n)); return n; }
__device__ __forceinline__ uint32_t cluster_cta() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster(const float* mine, uint32_t cta) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(mine)), "r"(cta));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// c tanh(x / c) from one exponential: tanh(y) = 1 - 2 / (e^(2y) + 1), right at both ends (e^(2y) = inf gives 1, 0 gives -1)
__device__ __forceinline__ float capped(float x, float cap, float inv_cap) {
  const float t = __expf(2.f * x * inv_cap);
  return cap * (1.f - __fdividef(2.f, t + 1.f));
}

struct Options {
  float scale, softcap, out_scale;
  int window, keep_first;
  const float* inv_freq_out;      // [VD / 2] or null
  const bf16* gate;               // [rows, ld_gate], entry h * VD + i, or null
  long long ld_gate, ld_out;
};

template <int D, int VD, bool KEYSPLIT, int STAGES>
__global__ void __launch_bounds__(128) attention_flex_mma_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    const int* __restrict__ block_table, int max_pages, int page_size, int page_shift, int num_pages,
    const int* __restrict__ tiles, const int* __restrict__ positions, const Options opt, bf16* __restrict__ out, int Hq, int Hk,
    int* __restrict__ status) {
  constexpr int CHK = D / 8, CHV = VD / 8;        // 16-byte chunks a row
  constexpr int K_BYTES = KT * D * 2, V_BYTES = KT * VD * 2;
  constexpr int QROWS = KEYSPLIT ? 16 : 64;
  constexpr int NS = KEYSPLIT ? 2 : 8;            // 8-key score tiles a warp computes per key tile
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sq = smem;                             // [QROWS][D]
  uint8_t* sk = sq + QROWS * D * 2;               // [STAGES][64][D]
  uint8_t* sv = sk + STAGES * K_BYTES;            // [STAGES][64][VD]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t = blockIdx.x, g = blockIdx.y;
  const int b = tiles[3 * t], row0 = tiles[3 * t + 1], nq = tiles[3 * t + 2];
  const int G = Hq / Hk;
  if (KEYSPLIT && nq * G > 16) {                  // the caller promised small tiles
    if (tid == 0) atomicExch(status, 4);
    return;
  }
  const int window = opt.window, keep_first = opt.keep_first;
  const int pos0 = positions[row0];
  const int* table = block_table + (long long)b * max_pages;
  // keys any row of the tile may see: the window's k_lo .. k_hi, and the kept first ones below k_lo
  const int k_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int k_hi = pos0 + nq - 1;
  const int first_end = min(keep_first, k_lo);
  const int kt_first = k_lo / KT, kt_last = k_hi / KT;
  const int n_a = min(kt_first, (first_end + KT - 1) / KT);        // tiles of kept first tokens before the window's tiles
  const int n_tiles = n_a + kt_last - kt_first + 1;
  auto tile_of = [&](int it) { return it < n_a ? it : kt_first + (it - n_a); };
  // a cluster shares the key tiles of its (request, KV head): CTA c takes the c-th stretch of them (decoding form only)
  int it0 = 0, n_mine = n_tiles;
  uint32_t n_cta = 1, cta = 0;
  if constexpr (KEYSPLIT) {
    n_cta = cluster_ctas();
    cta = cluster_cta();
    if (n_cta > 1) {
      const int per = (n_tiles + (int)n_cta - 1) / (int)n_cta;
      it0 = min(n_tiles, (int)cta * per);
      n_mine = min(n_tiles, it0 + per) - it0;
    }
  }

  // ---- Q tile: M row m = (query row m / G, head m % G); rows past the tile's queries are zero ----
  for (int i = tid; i < QROWS * CHK; i += 128) {
    const int m = i / CHK, c = i % CHK;
    const int qi = m / G, hj = m % G;
    const bool valid = qi < nq;
    const bf16* src = q + ((long long)(row0 + (valid ? qi : 0)) * Hq + g * G + hj) * D + c * 8;
    cp_async16(sq + swz<D>(m, c), src, valid);
  }
  // Two threads copy one key's row and its value's: one page lookup a thread and tile.
  const int my_key = tid >> 1;
  auto load_kv = [&](int kt, int stage) {
    const int kp = kt * KT + my_key;
    bool valid = kp <= k_hi && (kp >= k_lo || kp < first_end);
    long long off = 0;
    if (valid) {
      const int pg = page_shift >= 0 ? kp >> page_shift : kp / page_size;
      const int page = table_page(table, pg, max_pages, num_pages);
      if (page < 0) {
        atomicExch(status, 3);
        valid = false;
      } else {
        off = ((long long)page * Hk + g) * page_size + (kp - pg * page_size);
      }
    }
    uint8_t* dk = sk + stage * K_BYTES;
    uint8_t* dv = sv + stage * V_BYTES;
#pragma unroll
    for (int j = 0; j < CHK / 2; ++j) {
      const int c = (tid & 1) + 2 * j;
      cp_async16(dk + swz<D>(my_key, c), k_cache + off * D + c * 8, valid);
    }
#pragma unroll
    for (int j = 0; j < CHV / 2; ++j) {
      const int c = (tid & 1) + 2 * j;
      cp_async16(dv + swz<VD>(my_key, c), v_cache + off * VD + c * 8, valid);
    }
  };
#pragma unroll
  for (int s0 = 0; s0 < STAGES - 1; ++s0) {
    if (s0 < n_mine) load_kv(tile_of(it0 + s0), s0);
    cp_async_commit();
  }

  // this thread's two M rows and their query positions
  const int wrow = KEYSPLIT ? 0 : warp * 16;
  const int r_lo = wrow + (lane >> 2), r_hi = r_lo + 8;
  const int q_lo = r_lo / G, q_hi = r_hi / G;
  const bool v_lo = q_lo < nq, v_hi = q_hi < nq;
  const int p_lo = pos0 + q_lo, p_hi = pos0 + q_hi;
  const int w_lo = window > 0 ? max(0, p_lo - window + 1) : 0, w_hi = window > 0 ? max(0, p_hi - window + 1) : 0;
  const int n_base = KEYSPLIT ? warp * 2 : 0;      // first 8-key score tile of this warp
  constexpr float LOG2E = 1.4426950408889634f;
  const float scale = opt.scale, cap = opt.softcap, inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  const bool active = wrow < nq * G;
  float o[VD / 8][4];
#pragma unroll
  for (int n = 0; n < VD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  uint32_t qf[D / 16][4];

  for (int it = 0; it < n_mine; ++it) {
    const int kt = tile_of(it0 + it), stage = it % STAGES;
    cp_async_wait<STAGES - 2>();      // this thread's copies of tile `it` have landed
    __syncthreads();                  // everybody's have, and everybody is done with the tile before
    if (it + STAGES - 1 < n_mine) load_kv(tile_of(it0 + it + STAGES - 1), (it + STAGES - 1) % STAGES);
    cp_async_commit();
    if (!active) continue;            // a warp whose 16 M rows lie past the tile's queries only helps with the loads
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int row = wrow + (lane & 15), c = kk * 2 + (lane >> 4);
        ldmatrix_x4(smem_addr(sq + swz<D>(row, c)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
      }
    }
    const uint8_t* ks = sk + stage * K_BYTES;
    const uint8_t* vs = sv + stage * V_BYTES;
    // ---- scores of this warp's 16 rows against its keys of the tile ----
    float s[NS][4];
#pragma unroll
    for (int n = 0; n < NS; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int n = 0; n < NS; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int row = (n_base + n + (lane >> 4)) * 8 + (lane & 7), c = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(smem_addr(ks + swz<D>(row, c)), b0, b1, b2, b3);
        mma_bf16(s[n], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
        mma_bf16(s[n + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
      }
    }
    // ---- scale, cap, mask (in units of log 2: the exponentials are exp2), running maximum ----
    const int key0 = kt * KT + n_base * 8 + (lane & 3) * 2;
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < NS; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int kp = key0 + n * 8 + e;
        float a0 = s[n][e] * scale, a1 = s[n][2 + e] * scale;
        if (cap > 0.f) {
          a0 = capped(a0, cap, inv_cap);
          a1 = capped(a1, cap, inv_cap);
        }
        const bool kept = kp < keep_first;
        s[n][e] = (v_lo && kp <= p_lo && (kp >= w_lo || kept)) ? a0 * LOG2E : -INFINITY;
        s[n][2 + e] = (v_hi && kp <= p_hi && (kp >= w_hi || kept)) ? a1 * LOG2E : -INFINITY;
        mx_lo = fmaxf(mx_lo, s[n][e]);
        mx_hi = fmaxf(mx_hi, s[n][2 + e]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float n_lo = fmaxf(m_lo, mx_lo), n_hi = fmaxf(m_hi, mx_hi);
    // a row that has seen no key yet keeps 0 as its reference, so that exp2(-inf - reference) is 0, not NaN
    const float c_lo = n_lo == -INFINITY ? 0.f : n_lo, c_hi = n_hi == -INFINITY ? 0.f : n_hi;
    const float a_lo = exp2f(m_lo - c_lo), a_hi = exp2f(m_hi - c_hi);      // 0 where the row had no key before
    m_lo = n_lo;
    m_hi = n_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pf[NS / 2][4];                   // P as A fragments: k-step j covers 16 of the warp's keys
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const float p0 = exp2f(s[n][0] - c_lo), p1 = exp2f(s[n][1] - c_lo);
      const float p2 = exp2f(s[n][2] - c_hi), p3 = exp2f(s[n][3] - c_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l_lo = l_lo * a_lo + sum_lo;
    l_hi = l_hi * a_hi + sum_hi;
    if (__any_sync(0xffffffffu, a_lo != 1.f || a_hi != 1.f)) {      // most tiles leave the maxima as they are
#pragma unroll
      for (int n = 0; n < VD / 8; ++n) {
        o[n][0] *= a_lo;
        o[n][1] *= a_lo;
        o[n][2] *= a_hi;
        o[n][3] *= a_hi;
      }
    }
    // ---- o += P V ----
#pragma unroll
    for (int j = 0; j < NS / 2; ++j) {
#pragma unroll
      for (int n = 0; n < VD / 8; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int row = (n_base / 2 + j) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = n + (lane >> 4);
        ldmatrix_x4_trans(smem_addr(vs + swz<VD>(row, c)), b0, b1, b2, b3);
        mma_bf16(o[n], pf[j][0], pf[j][1], pf[j][2], pf[j][3], b0, b1);
        mma_bf16(o[n + 1], pf[j][0], pf[j][1], pf[j][2], pf[j][3], b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  // the row sums live in the four lanes of a quad
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  // Four finished entries of M row r (entries c, c + 1 and their partners VD / 2 further on; c < VD / 2, even): divided by
  // the row's sum, turned back, gated, scaled, written.
  auto emit = [&](int r, int c, float a0, float a1, float b0, float b1, float l) {
    const int qi = r / G, head = g * G + r % G;
    const long long row = row0 + qi;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    a0 *= inv;
    a1 *= inv;
    b0 *= inv;
    b1 *= inv;
    if (opt.inv_freq_out) {
      const float p = (float)(pos0 + qi);
      float sn0, cs0, sn1, cs1;
      sincosf(p * opt.inv_freq_out[c], &sn0, &cs0);
      sincosf(p * opt.inv_freq_out[c + 1], &sn1, &cs1);
      const float x0 = a0 * cs0 + b0 * sn0, y0 = b0 * cs0 - a0 * sn0;
      const float x1 = a1 * cs1 + b1 * sn1, y1 = b1 * cs1 - a1 * sn1;
      a0 = x0;
      b0 = y0;
      a1 = x1;
      b1 = y1;
    }
    if (opt.gate) {
      const bf16* gr = opt.gate + row * opt.ld_gate + (long long)head * VD;
      a0 *= 1.f / (1.f + expf(-to_f32(gr[c])));
      a1 *= 1.f / (1.f + expf(-to_f32(gr[c + 1])));
      b0 *= 1.f / (1.f + expf(-to_f32(gr[c + VD / 2])));
      b1 *= 1.f / (1.f + expf(-to_f32(gr[c + VD / 2 + 1])));
    }
    bf16* dst = out + row * opt.ld_out + (long long)head * VD;
    *reinterpret_cast<uint32_t*>(dst + c) = pack_bf16(a0 * opt.out_scale, a1 * opt.out_scale);
    *reinterpret_cast<uint32_t*>(dst + c + VD / 2) = pack_bf16(b0 * opt.out_scale, b1 * opt.out_scale);
  };

  if constexpr (!KEYSPLIT) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (!(half ? v_hi : v_lo)) continue;
      const int r = half ? r_hi : r_lo;
      const float l = half ? l_hi : l_lo;
#pragma unroll
      for (int n = 0; n < VD / 16; ++n)
        emit(r, n * 8 + (lane & 3) * 2, o[n][half * 2], o[n][half * 2 + 1], o[n + VD / 16][half * 2],
             o[n + VD / 16][half * 2 + 1], l);
    }
  } else {
    // ---- merge the four warps' shares of the keys, in warp order ----
    float* mo = reinterpret_cast<float*>(sk);              // [4][16][VD]
    float* mml = mo + 4 * 16 * VD;                         // [4][16][2]
    float* co = mml + 4 * 16 * 2;                          // [16][VD]: this CTA's share, for the cluster's first CTA
    float* cml = co + 16 * VD;                             // [16][2]
    __syncthreads();                                       // every warp is done with the key/value stages
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = (lane >> 2) + half * 8;
      float* dst = mo + (warp * 16 + r) * VD + (lane & 3) * 2;
#pragma unroll
      for (int n = 0; n < VD / 8; ++n) {
        dst[n * 8] = o[n][half * 2];
        dst[n * 8 + 1] = o[n][half * 2 + 1];
      }
      if ((lane & 3) == 0) {
        mml[(warp * 16 + r) * 2] = half ? m_hi : m_lo;
        mml[(warp * 16 + r) * 2 + 1] = half ? l_hi : l_lo;
      }
    }
    __syncthreads();
    for (int i = tid; i < 16 * (VD / 4); i += 128) {
      const int r = i / (VD / 4), c = (i % (VD / 4)) * 2;
      if (r >= nq * G) continue;
      float mrow = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mrow = fmaxf(mrow, mml[(w * 16 + r) * 2]);
      float l = 0.f, a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = mml[(w * 16 + r) * 2];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - mrow);
        const float* src = mo + (w * 16 + r) * VD;
        l += f * mml[(w * 16 + r) * 2 + 1];
        a0 += f * src[c];
        a1 += f * src[c + 1];
        b0 += f * src[c + VD / 2];
        b1 += f * src[c + VD / 2 + 1];
      }
      if (n_cta == 1) {
        emit(r, c, a0, a1, b0, b1, l);
      } else {
        co[r * VD + c] = a0;
        co[r * VD + c + 1] = a1;
        co[r * VD + c + VD / 2] = b0;
        co[r * VD + c + VD / 2 + 1] = b1;
        if (c == 0) {
          cml[r * 2] = mrow;
          cml[r * 2 + 1] = l;
        }
      }
    }
    if (n_cta > 1) {
      // ---- the cluster's CTAs' shares, in their order, by its first CTA out of the others' shared memory ----
      cluster_sync();
      if (cta == 0) {
        for (int i = tid; i < 16 * (VD / 4); i += 128) {
          const int r = i / (VD / 4), c = (i % (VD / 4)) * 2;
          if (r >= nq * G) continue;
          float mrow = -INFINITY;
          for (uint32_t w = 0; w < n_cta; ++w) mrow = fmaxf(mrow, ld_cluster(cml + r * 2, w));
          float l = 0.f, a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
          for (uint32_t w = 0; w < n_cta; ++w) {
            const float mw = ld_cluster(cml + r * 2, w);
            if (mw == -INFINITY) continue;
            const float f = exp2f(mw - mrow);
            l += f * ld_cluster(cml + r * 2 + 1, w);
            a0 += f * ld_cluster(co + r * VD + c, w);
            a1 += f * ld_cluster(co + r * VD + c + 1, w);
            b0 += f * ld_cluster(co + r * VD + c + VD / 2, w);
            b1 += f * ld_cluster(co + r * VD + c + VD / 2 + 1, w);
          }
          emit(r, c, a0, a1, b0, b1, l);
        }
      }
      cluster_sync();        // nobody leaves while its shared memory may still be read
    }
  }
}

template <int D, int VD, bool KEYSPLIT, int STAGES>
static int launch(const void* q, const void* k_cache, const void* v_cache, const int* block_table, int max_pages, int page_size,
                  int num_pages, const int* tiles, int n_tiles, const int* positions, const Options& opt, void* out, int Hq,
                  int Hk, int cluster, int* status, cudaStream_t stream) {
  constexpr int SMEM = (KEYSPLIT ? 16 : 64) * D * 2 + STAGES * KT * (D + VD) * 2;
  static_assert(!KEYSPLIT || 5 * 16 * (VD + 2) * 4 <= STAGES * KT * (D + VD) * 2, "the merge buffer reuses the stages");
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(attention_flex_mma_kernel<D, VD, KEYSPLIT, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size;) ++page_shift;
  dim3 grid(n_tiles, Hk);
  if (KEYSPLIT && cluster > 1) {
    // a cluster of `cluster` CTAs along z shares a (request, KV head)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, Hk, cluster);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = cluster;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_flex_mma_kernel<D, VD, KEYSPLIT, STAGES>, (const bf16*)q,
                                       (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_pages, page_size, page_shift,
                                       num_pages, tiles, positions, opt, (bf16*)out, Hq, Hk, status);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
  }
  attention_flex_mma_kernel<D, VD, KEYSPLIT, STAGES><<<grid, 128, SMEM, stream>>>(
      (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_pages, page_size, page_shift, num_pages, tiles,
      positions, opt, (bf16*)out, Hq, Hk, status);
  return (int)cudaGetLastError();
}

}  // namespace fx
}  // namespace tl

using namespace tl;

extern "C" int tl_attention_flex_mma_supported(int Hq, int Hk, int D, int VD) {
  return (D == 64 || D == 128) && (VD == 64 || VD == 128) && Hk > 0 && Hq % Hk == 0 && Hq / Hk <= 64;
}

// Query rows of one request that fit a tile: 64 M rows hold 64 / G query rows of the G heads of a KV head.
extern "C" int tl_attention_flex_mma_tile_rows(int Hq, int Hk) {
  const int G = Hk > 0 ? Hq / Hk : 0;
  return (G >= 1 && G <= 64) ? 64 / G : 0;
}

// tiles: int32 [n_tiles, 3] = (request index, first row, query rows <= tile rows), rows of a tile consecutive in position.
// max_tile_rows: the most query rows any tile holds; when they and their heads fit 16 M rows, the form that splits the
// keys among the warps runs; there, with few tiles and `max_context` keys to go through, clusters of up to 8 CTAs share a
// (request, KV head)'s key tiles until the grid has a CTA an SM (`sm_count`), and the cluster's first CTA merges their shares
// out of their shared memory. out: rows of ld_out bf16, 4-byte aligned; gate: rows of ld_gate bf16 or null.
extern "C" int tl_attention_flex_mma(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                     int max_pages, int page_size, int num_pages, const int* tiles, int n_tiles,
                                     int max_tile_rows, const int* positions, float scale, float softcap, int window,
                                     int keep_first, const float* inv_freq_out, const void* gate, long long ld_gate,
                                     float out_scale, void* out, long long ld_out, int rows, int Hq, int Hk, int D, int VD,
                                     int max_context, int sm_count, int* status, cudaStream_t stream) {
  if (rows == 0 || n_tiles == 0) return 0;
  TL_REQUIRE(tl_attention_flex_mma_supported(Hq, Hk, D, VD), "attention (tensor cores): %d heads over %d KV heads, keys of %d, values of %d",
             Hq, Hk, D, VD);
  TL_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0 && keep_first >= 0,
             "attention: page size %d, table width %d, window %d, kept first tokens %d", page_size, max_pages, window, keep_first);
  TL_REQUIRE(Hk <= 65535, "attention: %d KV heads exceed the grid limit", Hk);
  TL_REQUIRE(max_tile_rows >= 1 && max_tile_rows <= tl_attention_flex_mma_tile_rows(Hq, Hk),
             "attention: tiles of %d query rows, at most %d fit", max_tile_rows, tl_attention_flex_mma_tile_rows(Hq, Hk));
  TL_REQUIRE(((uintptr_t)out % 4) == 0 && ld_out % 2 == 0, "attention: output rows of %lld entries must start on 4 bytes", ld_out);
  fx::Options opt{scale, softcap, out_scale, window, keep_first, inv_freq_out, (const bf16*)gate, ld_gate, ld_out};
  const bool keysplit = max_tile_rows * (Hq / Hk) <= 16;
  int cluster = 1;
  if (keysplit) {
    const int reach = window > 0 ? (max_context < window + keep_first + fx::KT ? max_context : window + keep_first + fx::KT) : max_context;
    const int key_tiles = (reach + fx::KT - 1) / fx::KT;
    const long long ctas = (long long)n_tiles * Hk;
    while (cluster < 8 && 2 * cluster <= key_tiles && ctas * cluster < (sm_count > 0 ? sm_count : 148)) cluster *= 2;
  }
#define TL_FX(D_, VD_, KS_, ST_)                                                                                              \
  fx::launch<D_, VD_, KS_, ST_>(q, k_cache, v_cache, block_table, max_pages, page_size, num_pages, tiles, n_tiles, positions, \
                                opt, out, Hq, Hk, cluster, status, stream)
  if (D == 64 && VD == 64) return keysplit ? TL_FX(64, 64, true, 4) : TL_FX(64, 64, false, 3);
  if (D == 64) return keysplit ? TL_FX(64, 128, true, 3) : TL_FX(64, 128, false, 2);
  if (VD == 64) return keysplit ? TL_FX(128, 64, true, 3) : TL_FX(128, 64, false, 2);
  return keysplit ? TL_FX(128, 128, true, 3) : TL_FX(128, 128, false, 2);
#undef TL_FX
}
