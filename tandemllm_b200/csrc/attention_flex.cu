// Attention over the paged cache with the options a design may combine, on the CUDA cores, in 32-bit or bfloat16 storage
// with 32-bit arithmetic; any head size up to 256 for keys and, separately, for values.
//
//   tl_qkv_rotate_store   one row a block: q, k (first `rot` entries of a head turned by the row's position, halves
//                         layout: entry i with entry i + rot / 2) and v (optionally turned over all its entries with
//                         frequencies of its own) from one fused product; q to a plain tensor, k and v into their pages.
//                         The sines and cosines of q and k may carry a common factor (a stretched rotation's magnitude);
//                         v may first be blended with another tensor's values of the same row, (1 - l) v + l v_other, l a
//                         number on the device (values carried over from an earlier layer)
//   tl_attention_flex     one warp a (row, query head): score = scale q.k, optionally capped (c tanh(score / c)); row at
//                         position i sees key j <= i when there is no window, or i - j < window, or j < keep_first;
//                         softmax in 32-bit; the output optionally turned back by the row's own position (the inverse of
//                         the values' turn), optionally times sigmoid(gate) entry by entry, times `out_scale`
//
// Cache layout per site: K [pages, kv heads, page_size, D], V [pages, kv heads, page_size, VD]. Keys are visited in
// chunks of 32 aligned to absolute positions (first the kept first tokens that lie before the window, then the window)
// with an online softmax, so the order of additions for a row depends on its position only: never on the batch, the
// portion or the pages.
#include "common.cuh"

namespace tl {

constexpr int FLEX_MAX_DIM = 256;

template <typename T>
__device__ __forceinline__ float rotated_entry(const T* __restrict__ x, int i, int half, const float* __restrict__ sn,
                                               const float* __restrict__ cs) {
  if (i < half) return to_f32(x[i]) * cs[i] - to_f32(x[i + half]) * sn[i];
  if (i < 2 * half) return to_f32(x[i]) * cs[i - half] + to_f32(x[i - half]) * sn[i - half];
  return to_f32(x[i]);
}

template <typename T>
__global__ void __launch_bounds__(128) qkv_rotate_store_kernel(
    const T* __restrict__ qkv, long long ld, int q_col, int k_col, int v_col, const float* __restrict__ inv_freq, int rot,
    const float* __restrict__ inv_freq_v, const int* __restrict__ positions, const int* __restrict__ req_of_row,
    const int* __restrict__ block_table, int max_pages, int page_size, int num_pages, T* __restrict__ q_out,
    T* __restrict__ k_cache, T* __restrict__ v_cache, int Hq, int Hk, int D, int VD, int* __restrict__ status,
    float rot_magnitude, const T* __restrict__ v_other, long long ld_other, const float* __restrict__ v_blend) {
  __shared__ float sn[FLEX_MAX_DIM / 2], cs[FLEX_MAX_DIM / 2], snv[FLEX_MAX_DIM / 2], csv[FLEX_MAX_DIM / 2];
  const int r = blockIdx.x;
  const int pos = positions[r];
  const int half = inv_freq ? rot / 2 : 0, vhalf = inv_freq_v ? VD / 2 : 0;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    sincosf((float)pos * inv_freq[i], &sn[i], &cs[i]);
    sn[i] *= rot_magnitude;
    cs[i] *= rot_magnitude;
  }
  for (int i = threadIdx.x; i < vhalf; i += blockDim.x) sincosf((float)pos * inv_freq_v[i], &snv[i], &csv[i]);
  __syncthreads();
  const T* row = qkv + (long long)r * ld;
  for (int e = threadIdx.x; e < Hq * D; e += blockDim.x) {
    const int h = e / D, i = e - h * D;
    q_out[(long long)r * Hq * D + e] = from_f32<T>(rotated_entry(row + q_col + h * D, i, half, sn, cs));
  }
  if (k_col < 0) return;
  const int b = req_of_row[r];
  const int page = table_page(block_table + (long long)b * max_pages, pos / page_size, max_pages, num_pages);
  if (page < 0) {
    if (threadIdx.x == 0) atomicExch(status, 2);
    return;
  }
  const long long at = (long long)page * Hk * page_size + pos % page_size;
  for (int e = threadIdx.x; e < Hk * D; e += blockDim.x) {
    const int h = e / D, i = e - h * D;
    k_cache[(at + (long long)h * page_size) * D + i] = from_f32<T>(rotated_entry(row + k_col + h * D, i, half, sn, cs));
  }
  if (v_other) {
    // blended in 32-bit from the two stored values, rounded once; a blended value is not turned as well
    const float l = *v_blend;
    const T* other = v_other + (long long)r * ld_other;
    for (int e = threadIdx.x; e < Hk * VD; e += blockDim.x) {
      const int h = e / VD, i = e - h * VD;
      v_cache[(at + (long long)h * page_size) * VD + i] = from_f32<T>((1.f - l) * to_f32(row[v_col + e]) + l * to_f32(other[e]));
    }
    return;
  }
  for (int e = threadIdx.x; e < Hk * VD; e += blockDim.x) {
    const int h = e / VD, i = e - h * VD;
    v_cache[(at + (long long)h * page_size) * VD + i] = from_f32<T>(rotated_entry(row + v_col + h * VD, i, vhalf, snv, csv));
  }
}

template <typename T>
__global__ void __launch_bounds__(128) attention_flex_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ block_table, int max_pages, int page_size, int num_pages, const int* __restrict__ req_of_row,
    const int* __restrict__ positions, float scale, float softcap, int window, int keep_first,
    const float* __restrict__ inv_freq_out, const T* __restrict__ gate, long long ld_gate, float out_scale,
    T* __restrict__ out, long long ld_out, int Hq, int Hk, int D, int VD, int* __restrict__ status) {
  __shared__ float qs[4][FLEX_MAX_DIM];
  __shared__ float os[4][FLEX_MAX_DIM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * 4 + warp, r = blockIdx.x;
  if (h >= Hq) return;
  const int kvh = h / (Hq / Hk);
  const int b = req_of_row[r], pos = positions[r];
  const int* table = block_table + (long long)b * max_pages;
  const T* qrow = q + ((long long)r * Hq + h) * D;
  float* qv = qs[warp];
  for (int i = lane; i < D; i += 32) qv[i] = to_f32(qrow[i]) * scale;
  __syncwarp();

  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int first_end = min(keep_first, lo);        // the kept first tokens that the window does not hold anyway
  constexpr int NACC = FLEX_MAX_DIM / 32;
  float acc[NACC];
#pragma unroll
  for (int t = 0; t < NACC; ++t) acc[t] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int part = 0; part < 2; ++part) {
    const int from = part == 0 ? 0 : lo, to = part == 0 ? first_end - 1 : pos;     // positions from .. to, both included
    if (to < from) continue;
    for (int base = (from / 32) * 32; base <= to; base += 32) {
      const int kp = base + lane;
      const bool valid = kp >= from && kp <= to;
      long long off = -1;
      float s = -INFINITY;
      if (valid) {
        const int page = table_page(table, kp / page_size, max_pages, num_pages);
        if (page < 0) {
          atomicExch(status, 3);      // a visible key without a page: recorded, the key is skipped
        } else {
          off = ((long long)page * Hk + kvh) * page_size + kp % page_size;
          const T* kr = k_cache + off * D;
          float d = 0.f;
          for (int i = 0; i < D; ++i) d = fmaf(qv[i], to_f32(kr[i]), d);
          s = softcap > 0.f ? softcap * tanhf(d / softcap) : d;
        }
      }
      const float m_new = fmaxf(m, warp_max(s));
      if (m_new == -INFINITY) continue;
      const float p = off >= 0 ? expf(s - m_new) : 0.f;
      const float alpha = expf(m - m_new);
      l = l * alpha + warp_sum(p);
#pragma unroll
      for (int t = 0; t < NACC; ++t) acc[t] *= alpha;
      const int n_here = min(32, to - base + 1);
      for (int j = 0; j < n_here; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const long long oj = __shfl_sync(0xffffffffu, off, j);
        if (oj < 0) continue;
        const T* vr = v_cache + oj * VD;
#pragma unroll
        for (int t = 0; t < NACC; ++t) {
          const int i = lane + 32 * t;
          if (i < VD) acc[t] = fmaf(pj, to_f32(vr[i]), acc[t]);
        }
      }
      m = m_new;
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  float* ov = os[warp];
#pragma unroll
  for (int t = 0; t < NACC; ++t) {
    const int i = lane + 32 * t;
    if (i < VD) ov[i] = acc[t] * inv;
  }
  __syncwarp();
  T* o = out + (long long)r * ld_out + (long long)h * VD;
  const T* g = gate ? gate + (long long)r * ld_gate + (long long)h * VD : nullptr;
  const int vhalf = inv_freq_out ? VD / 2 : 0;
  for (int i = lane; i < VD; i += 32) {
    float y = ov[i];
    if (i < 2 * vhalf) {       // turned back: the angle of the values' turn with the row's own position, negated
      const int f = i < vhalf ? i : i - vhalf;
      float sn, c;
      sincosf((float)pos * inv_freq_out[f], &sn, &c);
      y = i < vhalf ? ov[i] * c + ov[i + vhalf] * sn : ov[i] * c - ov[i - vhalf] * sn;
    }
    if (g) y *= 1.f / (1.f + expf(-to_f32(g[i])));
    o[i] = from_f32<T>(y * out_scale);
  }
}

}  // namespace tl

using namespace tl;

extern "C" int tl_qkv_rotate_store(const void* qkv, long long ld, int q_col, int k_col, int v_col, const float* inv_freq,
                                   int rot, const float* inv_freq_v, const int* positions, const int* req_of_row,
                                   const int* block_table, int max_pages, int page_size, int num_pages, void* q_out,
                                   void* k_cache, void* v_cache, int rows, int Hq, int Hk, int D, int VD, int dtype,
                                   int* status, float rot_magnitude, const void* v_other, long long ld_other,
                                   const float* v_blend, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(!v_other || (v_blend && !inv_freq_v), "qkv_rotate_store: blended values want their weight and are not turned");
  TL_REQUIRE(Hq > 0 && Hk > 0 && D >= 1 && D <= FLEX_MAX_DIM && VD >= 1 && VD <= FLEX_MAX_DIM,
             "qkv_rotate_store: %d query heads, %d KV heads, key size %d, value size %d (sizes up to %d)", Hq, Hk, D, VD,
             FLEX_MAX_DIM);
  TL_REQUIRE(!inv_freq || (rot > 0 && rot <= D && rot % 2 == 0), "qkv_rotate_store: rotary size %d for head size %d", rot, D);
  TL_REQUIRE(!inv_freq_v || VD % 2 == 0, "qkv_rotate_store: values of odd size %d cannot be turned in pairs", VD);
  TL_REQUIRE(k_col < 0 || (k_cache && v_cache && block_table && page_size > 0 && max_pages > 0),
             "qkv_rotate_store: keys and values without pages to go to");
#define TL_QRS(T_)                                                                                                         \
  qkv_rotate_store_kernel<T_><<<rows, 128, 0, stream>>>((const T_*)qkv, ld, q_col, k_col, v_col, inv_freq, rot, inv_freq_v,  \
                                                        positions, req_of_row, block_table, max_pages, page_size, num_pages, \
                                                        (T_*)q_out, (T_*)k_cache, (T_*)v_cache, Hq, Hk, D, VD, status,    \
                                                        rot_magnitude, (const T_*)v_other, ld_other, v_blend)
  if (dtype == TL_FP32) TL_QRS(float);
  else TL_QRS(bf16);
#undef TL_QRS
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_attention_flex(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                 int max_pages, int page_size, int num_pages, const int* req_of_row, const int* positions,
                                 float scale, float softcap, int window, int keep_first, const float* inv_freq_out,
                                 const void* gate, long long ld_gate, float out_scale, void* out, long long ld_out, int rows,
                                 int Hq, int Hk, int D, int VD, int dtype, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(Hq > 0 && Hk > 0 && Hq % Hk == 0, "attention_flex: %d query heads over %d KV heads", Hq, Hk);
  TL_REQUIRE(D >= 1 && D <= FLEX_MAX_DIM && VD >= 1 && VD <= FLEX_MAX_DIM, "attention_flex: key size %d, value size %d (up to %d)",
             D, VD, FLEX_MAX_DIM);
  TL_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0 && keep_first >= 0,
             "attention_flex: page size %d, table width %d, window %d, kept first tokens %d", page_size, max_pages, window,
             keep_first);
  TL_REQUIRE(!inv_freq_out || VD % 2 == 0, "attention_flex: outputs of odd size %d cannot be turned in pairs", VD);
  dim3 grid(rows, ceil_div(Hq, 4));
  TL_REQUIRE(grid.y <= 65535, "attention_flex: %d heads exceed the grid limit", Hq);
#define TL_AF(T_)                                                                                                          \
  attention_flex_kernel<T_><<<grid, 128, 0, stream>>>((const T_*)q, (const T_*)k_cache, (const T_*)v_cache, block_table,     \
                                                      max_pages, page_size, num_pages, req_of_row, positions, scale, softcap, \
                                                      window, keep_first, inv_freq_out, (const T_*)gate, ld_gate, out_scale,   \
                                                      (T_*)out, ld_out, Hq, Hk, D, VD, status)
  if (dtype == TL_FP32) TL_AF(float);
  else TL_AF(bf16);
#undef TL_AF
  TL_LAUNCH_CHECK();
  return 0;
}
