// Latent attention on the tensor cores (bfloat16): every head of a row attends over the same cached rows (the latent and
// the shared rotated key part), so the heads of a few neighbouring rows are the M rows of one tile and a tile of keys is
// read once for all of them. The arithmetic is that of csrc/attention_latent.cu: scores = scale * q' . key in 32-bit
// accumulators, softmax in 32-bit with a running maximum, the weights rounded to bfloat16 as the operand of the second
// product, out = sum_j p_j c_j over the latent part of the keys.
//
// A CTA of four warps takes 64 consecutive (row, head) pairs of one request (a warp 16 of them) and walks the visible keys
// in tiles of 32 aligned to absolute positions. A key tile is copied as it lies into one of two buffers in shared memory
// (cp.async, 16 bytes a copy) while the tile before it is computed on; it is the B operand of Q K^T as it lies (plain
// 32-bit loads) and, through ldmatrix with .trans, the B operand of P C. `mma.sync` m16n8k16; rows padded so that the
// eight rows a load touches fall into different banks. The latent's
// columns are taken in chunks of up to 256 (a CTA a chunk: the accumulators of one chunk are all a thread can hold), and,
// for steps of few rows, the keys in spans aligned to absolute positions, each span a CTA of its own; a second kernel
// joins the spans in order. One CTA finds its tile from the step's row_start by itself, so the launch needs no host list.
#include "common.cuh"

namespace tl {

constexpr int LM_ROWS = 64;     // (row, head) pairs a CTA
constexpr int LM_KEYS = 32;     // keys a tile

struct LatentMmaParams {
  const float* q;            // [rows, H, Dk] 32-bit
  const bf16* cache;         // [pages, 1, page_size, Dk]
  const int* table;
  int max_pages, page_size, num_pages;
  const int* req_of_row;     // [rows]: the row of the block table a row's request has
  const int* row_start;      // [requests + 1]
  const int* positions;
  float scale;
  int window;
  bf16* out;                 // [rows, H, L]
  float* part_o;             // [rows * H, n_spans, L] when n_spans > 1
  float* part_ml;            // [rows * H, n_spans, 2]
  int requests, H, L, Dk, Dkp, qs;      // Dkp: Dk rounded up to 16; qs: elements of a staged row (Dkp + 8)
  int n_spans, span_keys;
  int* status;
  const float* sinks;        // [H] or null: a head's softmax denominator also holds exp(sink), which has no key and no value
};

// What a row's sums are multiplied by and the reciprocal of its denominator, from its maximum m and sum l and the head's sink.
__device__ __forceinline__ void latent_finish(float m, float l, const float* sinks, int h, float* keep, float* inv) {
  *keep = 1.f;
  if (sinks) {
    const float sk = sinks[h], top = fmaxf(m, sk);
    *keep = m == -INFINITY ? 0.f : expf(m - top);
    l = l * *keep + expf(sk - top);
  }
  *inv = l > 0.f ? 1.f / l : 0.f;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (tiles upper bound, chunks of the latent / CPB, spans), 128 CPB threads. NT: 8-column tiles of the latent chunk.
// CPB: chunks a CTA takes (1 or 2): a second group of four warps runs the same 64 pairs for the next chunk of columns, on
// the same staged queries and keys.
template <int NT, int CPB>
__global__ void __launch_bounds__(128 * CPB) latent_mma_kernel(LatentMmaParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);                 // [64][qs]
  bf16* sK = sQ + LM_ROWS * p.qs;                                // two buffers of [32][qs], then some slack (see the launcher)
  __shared__ int s_pos[LM_ROWS], s_lo[LM_ROWS], s_page[2][LM_KEYS];
  __shared__ int s_tile[4];                                      // request, its first row, its rows, first pair of the tile
  const int H = p.H, L = p.L, Dk = p.Dk, qs = p.qs;
  const int warp = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int chunk_index = blockIdx.y * CPB + (threadIdx.x >> 7);
  const int chunk0 = chunk_index * NT * 8;
  if (threadIdx.x == 0) {
    int left = blockIdx.x, found = -1;
    for (int b = 0; b < p.requests && found < 0; ++b) {
      const int n = p.row_start[b + 1] - p.row_start[b];
      const int tiles = ceil_div(n * H, LM_ROWS);
      if (left < tiles) found = b;
      else left -= tiles;
    }
    s_tile[0] = found;
    if (found >= 0) {
      s_tile[1] = p.row_start[found];
      s_tile[2] = p.row_start[found + 1] - p.row_start[found];
      s_tile[3] = left * LM_ROWS;
    }
  }
  __syncthreads();
  const int b = s_tile[0];
  if (b < 0) return;
  const int row_base = s_tile[1], pairs = s_tile[2] * H, f0 = s_tile[3];
  // the tile's rows: positions, first visible keys, and the query rows (rounded to bfloat16; zero beyond the pairs and Dk)
  for (int m = threadIdx.x; m < LM_ROWS; m += blockDim.x) {
    const int f = f0 + m;
    int pos = -1, lo = 0;
    if (f < pairs) {
      pos = p.positions[row_base + f / H];
      lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    }
    s_pos[m] = pos;
    s_lo[m] = lo;
  }
  __syncthreads();
  // the keys this CTA walks: from the first row's first visible key to the last row's own position, within its span
  const int last = min(f0 + LM_ROWS, pairs) - 1;
  int key_lo = s_lo[0], key_hi = s_pos[last - f0];
  if (p.n_spans > 1) {
    key_lo = max(key_lo, (int)blockIdx.z * p.span_keys);
    key_hi = min(key_hi, ((int)blockIdx.z + 1) * p.span_keys - 1);
  }
  if (key_lo > key_hi) return;          // none of the tile's rows sees a key of this span: the join never asks for it
  for (int i = threadIdx.x; i < LM_ROWS * (qs / 2); i += blockDim.x) {
    const int m = i / (qs / 2), c = 2 * (i - m * (qs / 2));
    const int f = f0 + m;
    float x = 0.f, y = 0.f;
    if (f < pairs) {
      const float* src = p.q + ((long long)row_base * H + f) * Dk;
      if (c < Dk) x = src[c];
      if (c + 1 < Dk) y = src[c + 1];
    }
    reinterpret_cast<uint32_t*>(sQ + (size_t)m * qs)[c >> 1] = pack_bf16(x, y);
  }
  __syncthreads();
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int my_pos[2] = {s_pos[warp * 16 + g], s_pos[warp * 16 + g + 8]};
  const int my_lo[2] = {s_lo[warp * 16 + g], s_lo[warp * 16 + g + 8]};
  const int* tab = p.table + (long long)p.req_of_row[row_base] * p.max_pages;
  const bool vec = (Dk & 7) == 0 && ((uintptr_t)p.cache & 15) == 0;
  const int ksteps = p.Dkp >> 4;
  // Both key buffers' padding (the entries behind Dk that no copy touches) is zeroed once: the products read it.
  for (int i = threadIdx.x; i < 2 * LM_KEYS * (qs - (Dk & ~7)); i += blockDim.x) {
    const int per = qs - (Dk & ~7), rowi = i / per, c = (Dk & ~7) + (i - rowi * per);
    if (c >= Dk) sK[(size_t)rowi * qs + c] = __float2bfloat16_rn(0.f);
  }
  // A tile's pages are looked up (lookup), then its rows are sent on their way into one of the two buffers (fetch: 16-byte
  // cp.async copies where the rows allow them); the tile before it is computed on meanwhile.
  auto lookup = [&](int j0, int which) {
    if (threadIdx.x < LM_KEYS) {
      const int j = j0 + threadIdx.x;
      int page = -1;
      if (j >= key_lo && j <= key_hi) {
        page = table_page(tab, j / p.page_size, p.max_pages, p.num_pages);
        if (page < 0) atomicExch(p.status, 3);
      }
      s_page[which][threadIdx.x] = page;
    }
  };
  auto fetch = [&](int j0, int which) {
    bf16* dst = sK + (size_t)which * LM_KEYS * qs;
    if (vec) {
      const int per_row = Dk >> 3;                               // 16-byte pieces of a cached row
      for (int i = threadIdx.x; i < LM_KEYS * per_row; i += blockDim.x) {
        const int kk = i / per_row, c = (i - kk * per_row) << 3;
        const int page = s_page[which][kk];
        bf16* to = dst + (size_t)kk * qs + c;
        if (page >= 0) {
          const bf16* from = p.cache + ((long long)page * p.page_size + (j0 + kk) % p.page_size) * Dk + c;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(to)), "l"(from) : "memory");
        } else {
          *reinterpret_cast<uint4*>(to) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    } else {
      for (int i = threadIdx.x; i < LM_KEYS * Dk; i += blockDim.x) {
        const int kk = i / Dk, c = i - kk * Dk;
        const int page = s_page[which][kk];
        dst[(size_t)kk * qs + c] = page >= 0 ? p.cache[((long long)page * p.page_size + (j0 + kk) % p.page_size) * Dk + c]
                                             : __float2bfloat16_rn(0.f);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int j_first = (key_lo / LM_KEYS) * LM_KEYS;
  lookup(j_first, 0);
  __syncthreads();
  fetch(j_first, 0);
  int which = 0;
  for (int j0 = j_first; j0 <= key_hi; j0 += LM_KEYS, which ^= 1) {
    const bool more = j0 + LM_KEYS <= key_hi;
    if (more) lookup(j0 + LM_KEYS, which ^ 1);
    __syncthreads();
    if (more) {
      fetch(j0 + LM_KEYS, which ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();            // this tile's rows have landed, for every thread
    const bf16* tK = sK + (size_t)which * LM_KEYS * qs;
    const int* t_page = s_page[which];
    // S = Q K^T for the warp's 16 pairs and the tile's 32 keys
    float s[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    const uint32_t* q_lo = reinterpret_cast<const uint32_t*>(sQ + (size_t)(warp * 16 + g) * qs);
    const uint32_t* q_hi = reinterpret_cast<const uint32_t*>(sQ + (size_t)(warp * 16 + g + 8) * qs);
    for (int ks = 0; ks < ksteps; ++ks) {
      uint32_t a[4];
      a[0] = q_lo[ks * 8 + t];
      a[1] = q_hi[ks * 8 + t];
      a[2] = q_lo[ks * 8 + 4 + t];
      a[3] = q_hi[ks * 8 + 4 + t];
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const uint32_t* kr = reinterpret_cast<const uint32_t*>(tK + (size_t)(n * 8 + g) * qs);
        mma_bf16(s[n], a, kr[ks * 8 + t], kr[ks * 8 + 4 + t]);
      }
    }
    // scale, mask, running maximum and sum; thread (g, t) holds rows g and g + 8, keys 8 n + 2 t + {0, 1}
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1, kk = n * 8 + 2 * t + (e & 1), j = j0 + kk;
        const bool seen = t_page[kk] >= 0 && j >= my_lo[r] && j <= my_pos[r];
        s[n][e] = seen ? s[n][e] * p.scale : -INFINITY;
        tile_max[r] = fmaxf(tile_max[r], s[n][e]);
      }
    float fix[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float m_new = fmaxf(m_run[r], tile_max[r]);
      fix[r] = (m_run[r] == -INFINITY) ? 0.f : expf(m_run[r] - m_new);
      m_run[r] = m_new;
    }
    float tile_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float pe = s[n][e] == -INFINITY ? 0.f : expf(s[n][e] - m_run[r]);
        s[n][e] = pe;
        tile_sum[r] += pe;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_sum[r] += __shfl_xor_sync(0xffffffffu, tile_sum[r], 1);
      tile_sum[r] += __shfl_xor_sync(0xffffffffu, tile_sum[r], 2);
      l_run[r] = l_run[r] * fix[r] + tile_sum[r];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= fix[0]; o[n][1] *= fix[0];
      o[n][2] *= fix[1]; o[n][3] *= fix[1];
    }
    // O += P C: the weights go from the accumulators' layout straight into the A operand's; the latents are read as they
    // lie, [key][entry], and turned into the B operand's layout by ldmatrix (.trans), two 8-column tiles a load
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
      a[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
      a[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
      a[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
      // lane i gives the address of row (i % 8) of matrix i / 8: keys 0..7 and 8..15 of the block, for tile n and n + 1
      const bf16* rowp = tK + (size_t)(kb * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * qs + chunk0 + (lane >> 4) * 8;
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"((uint32_t)__cvta_generic_to_shared(rowp + n * 8)));
        mma_bf16(o[n], a, b0, b1);
        mma_bf16(o[n + 1], a, b2, b3);
      }
    }
    __syncthreads();            // the buffer may be filled again
  }
  // results: thread (g, t) holds pairs g and g + 8 of the warp, latent columns chunk0 + 8 n + 2 t + {0, 1}
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int f = f0 + warp * 16 + g + 8 * r;
    if (f >= pairs) continue;
    const long long pair = (long long)row_base * H + f;
    if (p.n_spans == 1) {
      float keep, inv;
      latent_finish(m_run[r], l_run[r], p.sinks, (int)(pair % H), &keep, &inv);
      inv *= keep;
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = chunk0 + n * 8 + 2 * t + e;
          if (c < L) p.out[pair * L + c] = __float2bfloat16_rn(o[n][2 * r + e] * inv);
        }
    } else {
      const long long at = pair * p.n_spans + blockIdx.z;
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = chunk0 + n * 8 + 2 * t + e;
          if (c < L) p.part_o[at * L + c] = o[n][2 * r + e];
        }
      if (chunk_index == 0 && t == 0) {
        p.part_ml[at * 2] = m_run[r];
        p.part_ml[at * 2 + 1] = l_run[r];
      }
    }
  }
}

// grid (rows * H), 128 threads: the spans of a pair joined in ascending order
__global__ void __launch_bounds__(128) latent_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                          const int* __restrict__ positions, int window, bf16* __restrict__ out,
                                                          int H, int L, int n_spans, int span_keys,
                                                          const float* __restrict__ sinks) {
  const long long pair = blockIdx.x;
  const int pos = positions[pair / H];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int s0 = lo / span_keys, s1 = min(pos / span_keys, n_spans - 1);
  float m = -INFINITY;
  for (int s = s0; s <= s1; ++s) m = fmaxf(m, part_ml[(pair * n_spans + s) * 2]);
  float sum = 0.f;
  for (int s = s0; s <= s1; ++s) {
    const float ms = part_ml[(pair * n_spans + s) * 2];
    if (ms != -INFINITY) sum += expf(ms - m) * part_ml[(pair * n_spans + s) * 2 + 1];
  }
  float keep, inv;
  latent_finish(m, sum, sinks, (int)(pair % H), &keep, &inv);
  inv *= keep;
  for (int c = threadIdx.x; c < L; c += blockDim.x) {
    float acc = 0.f;
    for (int s = s0; s <= s1; ++s) {
      const float ms = part_ml[(pair * n_spans + s) * 2];
      if (ms != -INFINITY) acc += expf(ms - m) * part_o[(pair * n_spans + s) * L + c];
    }
    out[pair * L + c] = __float2bfloat16_rn(acc * inv);
  }
}

}  // namespace tl

using namespace tl;

// Floats of scratch for `rows` rows of H heads cut into n_spans spans of keys.
extern "C" long long tl_attention_latent_mma_scratch(int rows, int H, int L, int n_spans) {
  return n_spans > 1 ? (long long)rows * H * n_spans * (L + 2) : 0;
}

// q float [rows, H, Dk]; cache bfloat16 [pages, 1, page_size, Dk]; out bfloat16 [rows, H, L]; row_start [requests + 1] cuts
// the rows into requests (a request's rows use table row req_of_row[its first row]); `tiles`: an upper bound of the (row, head) tiles of 64 of
// all requests. n_spans > 1: the keys are taken in spans of span_keys (a multiple of 32) positions, `scratch` holds
// tl_attention_latent_mma_scratch floats.
extern "C" int tl_attention_latent_mma(const float* q, const void* cache, const int* table, int max_pages, int page_size,
                                       int num_pages, const int* req_of_row, const int* row_start, const int* positions,
                                       float scale, int window,
                                       void* out, float* scratch, int rows, int requests, int tiles, int H, int L, int Dk,
                                       int n_spans, int span_keys, int* status, const float* sinks, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && requests > 0 && tiles > 0 && H > 0 && L > 0 && Dk >= L, "latent attention: %d rows of %d requests, %d "
             "heads, latent %d of %d", rows, requests, H, L, Dk);
  TL_REQUIRE(n_spans >= 1 && n_spans <= 65535 && (n_spans == 1 || (span_keys > 0 && span_keys % LM_KEYS == 0 && scratch)),
             "latent attention: %d spans of %d keys", n_spans, span_keys);
  TL_REQUIRE(window >= 0 && page_size > 0 && max_pages > 0, "latent attention: window %d, pages of %d", window, page_size);
  LatentMmaParams p;
  p.q = q; p.cache = (const bf16*)cache; p.table = table; p.max_pages = max_pages; p.page_size = page_size; p.num_pages = num_pages;
  p.req_of_row = req_of_row; p.row_start = row_start; p.positions = positions; p.scale = scale; p.window = window; p.out = (bf16*)out;
  p.part_o = scratch; p.part_ml = scratch ? scratch + (long long)rows * H * n_spans * L : nullptr;
  p.requests = requests; p.H = H; p.L = L; p.Dk = Dk; p.Dkp = ceil_div(Dk, 16) * 16; p.qs = p.Dkp + 8;
  p.n_spans = n_spans; p.span_keys = span_keys; p.status = status; p.sinks = sinks;
  const int nt_all = ceil_div(L, 8);
  const int nt = nt_all <= 4 ? 4 : nt_all <= 8 ? 8 : nt_all <= 16 ? 16 : 32;
  const int chunks = ceil_div(nt_all, nt);
  // (the second product reads whole 8-column tiles of a chunk, which may reach past a row's end into the next row or, behind
  // the last row, into the slack: those columns of the result are never stored)
  const size_t smem = ((size_t)(LM_ROWS + 2 * LM_KEYS) * p.qs + 8 * 32 + 256) * sizeof(bf16);
  TL_REQUIRE(smem <= 200 * 1024, "latent attention: keys of %d entries need %zu bytes of shared memory", Dk, smem);
#define TL_LM(NT_, CPB_)                                                                                                \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(latent_mma_kernel<NT_, CPB_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    latent_mma_kernel<NT_, CPB_><<<dim3(tiles, chunks / CPB_, n_spans), 128 * CPB_, smem, stream>>>(p);                 \
  } while (0)
  if (nt == 4) TL_LM(4, 1);
  else if (nt == 8) TL_LM(8, 1);
  else if (nt == 16) TL_LM(16, 1);
  else if (chunks == 2) TL_LM(32, 2);
  else TL_LM(32, 1);
#undef TL_LM
  TL_LAUNCH_CHECK();
  if (n_spans > 1) {
    latent_join_kernel<<<rows * H, 128, 0, stream>>>(p.part_o, p.part_ml, positions, window, (bf16*)out, H, L, n_spans, span_keys, sinks);
    TL_LAUNCH_CHECK();
  }
  return 0;
}
