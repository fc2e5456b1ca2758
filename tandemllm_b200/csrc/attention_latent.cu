// Latent attention: every head attends over ONE cached row a token, the normed latent c [L] followed by a rotated key
// part [Rr] that all heads share. A head's unrotated key would be W_uk c and its value W_uv c; instead the query is taken
// through W_uk once (q' = W_uk^T q_unrotated, a row of L numbers a head), the scores are q' . c + q_rotated . k_rotated, the
// softmax weights are applied to the latents themselves, and W_uv is applied to that sum afterwards: the same numbers in
// another order, and only c and the rotated part are ever stored.
//
//   latent_prepare    per row: c = w * kv[:L] / rms(kv[:L]) and rot(kv[L:]) go to the request's page at the row's position;
//                     rot(q_rotated) of every head goes to the query rows q' [rows, H, L + Rr] (32-bit) behind the L
//                     numbers that head_linear fills. rot: pairs (2i, 2i + 1) of the first `rot_dims` entries turn by
//                     position * inv_freq[i]; angles, sines and cosines in 32-bit.
//   head_linear       out[r, h, n] = sum_k a[r, h, k] w[h, n, k]: a product a head (q' from q, and the heads' outputs from
//                     the weighted latents), 32-bit accumulation in a fixed order
//   attention_latent  per (row, head): softmax over the visible keys j (0 <= pos - j < window, or all) of scale * q' . key_j,
//                     in 32-bit with a running maximum; out[r, h, :L] = sum_j p_j c_j. Keys are taken in tiles of 32 aligned
//                     to absolute positions, so the order of additions does not depend on how the sequence was cut into
//                     steps, what else is in the batch or which pages hold the keys. With `sinks` (a number a head) the
//                     softmax denominator also holds exp(sink): a share of the weight that has no key and no value.
//                     head_linear may multiply its result entry by entry by sigmoid(gate) (an output gate).
#include "common.cuh"

namespace tl {

// grid (rows), 128 threads
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(
    const T* __restrict__ q, long long ld_q, const T* __restrict__ kv, long long ld_kv, const float* __restrict__ c_weight,
    float eps, const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
    const int* __restrict__ req_of_row, const int* __restrict__ table, int max_pages, int page_size, int num_pages,
    T* __restrict__ cache, float* __restrict__ q_out, int H, int D, int L, int Rr, int* __restrict__ status) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int pos = positions[r], b = req_of_row[r];
  const int Dk = L + Rr;
  const T* kvr = kv + (long long)r * ld_kv;
  float ss = 0.f;
  for (int c = threadIdx.x; c < L; c += blockDim.x) {
    const float v = to_f32(kvr[c]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)L + eps);
  const int page = table_page(table + (long long)b * max_pages, pos / page_size, max_pages, num_pages);
  T* dst = nullptr;
  if (page < 0) {
    if (threadIdx.x == 0) atomicExch(status, 2);
  } else {
    dst = cache + ((long long)page * page_size + pos % page_size) * Dk;
  }
  if (dst)
    for (int c = threadIdx.x; c < L; c += blockDim.x) dst[c] = from_f32<T>(to_f32(kvr[c]) * inv * c_weight[c]);
  // the shared key part: pairs of the first rot_dims entries turn, the rest pass
  if (dst)
    for (int i = threadIdx.x; i < Rr; i += blockDim.x) {
      float v;
      if (i < rot_dims) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i >> 1], &sn, &cs);
        const float u = to_f32(kvr[L + (i & ~1)]), w = to_f32(kvr[L + (i | 1)]);
        v = (i & 1) ? w * cs + u * sn : u * cs - w * sn;
      } else {
        v = to_f32(kvr[L + i]);
      }
      dst[L + i] = from_f32<T>(v);
    }
  // the heads' rotated query parts
  const T* qr = q + (long long)r * ld_q;
  float* qo = q_out + (long long)r * H * Dk;
  for (int i = threadIdx.x; i < H * Rr; i += blockDim.x) {
    const int h = i / Rr, e = i - h * Rr;
    const T* src = qr + (long long)h * (D + Rr) + D;
    float v;
    if (e < rot_dims) {
      float sn, cs;
      sincosf((float)pos * inv_freq[e >> 1], &sn, &cs);
      const float u = to_f32(src[e & ~1]), w = to_f32(src[e | 1]);
      v = (e & 1) ? w * cs + u * sn : u * cs - w * sn;
    } else {
      v = to_f32(src[e]);
    }
    qo[(long long)h * Dk + L + e] = v;
  }
}

// out[r, :n] = w * in[r, :n] / rms(in[r, :n]); grid (rows), 128 threads. The rows are read in their own type, normed in
// 32-bit and rounded once.
template <typename T>
__global__ void __launch_bounds__(128) rmsnorm_rows_kernel(const T* __restrict__ in, long long ld_in, const float* __restrict__ w,
                                                           float eps, T* __restrict__ out, long long ld_out, int n) {
  __shared__ float scratch[33];
  const T* src = in + (long long)blockIdx.x * ld_in;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = to_f32(src[c]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)n + eps);
  T* dst = out + (long long)blockIdx.x * ld_out;
  for (int c = threadIdx.x; c < n; c += blockDim.x) dst[c] = from_f32<T>(to_f32(src[c]) * inv * w[c]);
}

// out[r, h, n] = sum_k a[r * ld_a + h * a_head + k] * w[(h * N + n) * K + k]; grid (ceil(N / 64), ceil(rows / 16), H), 256 threads:
// a block makes 16 rows x 64 outputs of one head, a thread 4 rows of one output; k in blocks of 32 through shared memory.
constexpr int HL_ROWS = 16, HL_COLS = 64, HL_K = 32;

template <typename T, typename TO>
__global__ void __launch_bounds__(256) head_linear_kernel(const T* __restrict__ a, long long ld_a, long long a_head,
                                                          const T* __restrict__ w, TO* __restrict__ out, long long ld_out,
                                                          long long out_head, int rows, int N, int K,
                                                          const T* __restrict__ gate, long long ld_gate) {
  __shared__ float sA[HL_ROWS][HL_K];
  __shared__ float sW[HL_COLS][HL_K + 1];
  const int h = blockIdx.z, r0 = blockIdx.y * HL_ROWS, n0 = blockIdx.x * HL_COLS;
  const int tn = threadIdx.x % HL_COLS, tr = (threadIdx.x / HL_COLS) * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += HL_K) {
    __syncthreads();
    for (int i = threadIdx.x; i < HL_ROWS * HL_K; i += blockDim.x) {
      const int rr = i / HL_K, kk = i - rr * HL_K;
      sA[rr][kk] = (r0 + rr < rows && k0 + kk < K) ? to_f32(a[(long long)(r0 + rr) * ld_a + (long long)h * a_head + k0 + kk]) : 0.f;
    }
    for (int i = threadIdx.x; i < HL_COLS * HL_K; i += blockDim.x) {
      const int nn = i / HL_K, kk = i - nn * HL_K;
      sW[nn][kk] = (n0 + nn < N && k0 + kk < K) ? to_f32(w[((long long)h * N + n0 + nn) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HL_K; ++kk) {
      const float wv = sW[tn][kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(sA[tr + i][kk], wv, acc[i]);
    }
  }
  if (n0 + tn < N)
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (r0 + tr + i < rows) {
        float v = acc[i];
        // (gate [rows, H * N] logits, rows ld_gate apart: the result times their sigmoid)
        if (gate) v *= 1.f / (1.f + expf(-to_f32(gate[(long long)(r0 + tr + i) * ld_gate + (long long)h * N + n0 + tn])));
        out[(long long)(r0 + tr + i) * ld_out + (long long)h * out_head + n0 + tn] = from_f32<TO>(v);
      }
}

constexpr int LA_WARPS = 8;     // heads a block: a warp a head
constexpr int LA_TILE = 32;     // keys a tile

// grid (rows, ceil(H / 8)), 256 threads. LPER: 32-number pieces of a latent a lane accumulates (L <= 32 LPER).
template <typename T, int LPER>
__global__ void __launch_bounds__(LA_WARPS * 32) attention_latent_kernel(
    const float* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ table, int max_pages, int page_size,
    int num_pages, const int* __restrict__ req_of_row, const int* __restrict__ positions, float scale, int window,
    T* __restrict__ out, int H, int L, int Dk, int* __restrict__ status, const float* __restrict__ sinks) {
  extern __shared__ __align__(16) float sm[];
  const int ldk = Dk + 1;                             // a key's row in shared memory, padded against bank conflicts
  float* sK = sm;                                     // [TILE][ldk]
  float* sQ = sK + LA_TILE * ldk;                     // [WARPS][Dk]
  __shared__ int s_page[LA_TILE];
  const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * LA_WARPS + warp;
  const bool head = h < H;
  const int pos = positions[r], b = req_of_row[r];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  if (head)
    for (int c = lane; c < Dk; c += 32) sQ[warp * Dk + c] = q[((long long)r * H + h) * Dk + c];
  float m = -INFINITY, l = 0.f;
  float acc[LPER];
#pragma unroll
  for (int i = 0; i < LPER; ++i) acc[i] = 0.f;
  const int* tab = table + (long long)b * max_pages;
  for (int j0 = (lo / LA_TILE) * LA_TILE; j0 <= pos; j0 += LA_TILE) {
    __syncthreads();
    if (threadIdx.x < LA_TILE) {
      const int j = j0 + threadIdx.x;
      int page = -1;
      if (j >= lo && j <= pos) {
        page = table_page(tab, j / page_size, max_pages, num_pages);
        if (page < 0) atomicExch(status, 3);
      }
      s_page[threadIdx.x] = page;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < LA_TILE * Dk; i += blockDim.x) {
      const int kk = i / Dk, c = i - kk * Dk;
      const int page = s_page[kk];
      sK[kk * ldk + c] = page >= 0 ? to_f32(cache[((long long)page * page_size + (j0 + kk) % page_size) * Dk + c]) : 0.f;
    }
    __syncthreads();
    if (head) {
      // lane = key: its score
      const float* kr = sK + lane * ldk;
      const float* qh = sQ + warp * Dk;
      float s = 0.f;
      for (int c = 0; c < Dk; ++c) s = fmaf(qh[c], kr[c], s);
      s = s_page[lane] < 0 ? -INFINITY : s * scale;
      const float tile_max = warp_max(s);
      const float m_new = fmaxf(m, tile_max);
      // the first tile holds the row's first visible key, so m_new is finite from the first tile on
      const float fix = m == -INFINITY ? 0.f : expf(m - m_new);
      const float pj = s == -INFINITY ? 0.f : expf(s - m_new);
      l = l * fix + warp_sum(pj);
#pragma unroll
      for (int i = 0; i < LPER; ++i) acc[i] *= fix;
      m = m_new;
      // lane = entry of the latent: add the tile's keys in order
      for (int kk = 0; kk < LA_TILE; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, pj, kk);
        if (pk != 0.f) {
          const float* cr = sK + kk * ldk;
#pragma unroll
          for (int i = 0; i < LPER; ++i) {
            const int c = lane + 32 * i;
            if (c < L) acc[i] = fmaf(pk, cr[c], acc[i]);
          }
        }
      }
    }
  }
  if (head) {
    float keep = 1.f;
    if (sinks) {
      const float sk = sinks[h], top = fmaxf(m, sk);
      keep = m == -INFINITY ? 0.f : expf(m - top);
      l = l * keep + expf(sk - top);
    }
    const float inv = (l > 0.f ? 1.f / l : 0.f) * keep;
    T* o = out + ((long long)r * H + h) * L;
#pragma unroll
    for (int i = 0; i < LPER; ++i) {
      const int c = lane + 32 * i;
      if (c < L) o[c] = from_f32<T>(acc[i] * inv);
    }
  }
}

template <typename T>
static int launch_latent(const float* q, const void* cache, const int* table, int max_pages, int page_size, int num_pages,
                         const int* req_of_row, const int* positions, float scale, int window, void* out, int rows, int H, int L,
                         int Dk, int* status, const float* sinks, cudaStream_t stream) {
  const dim3 grid(rows, ceil_div(H, LA_WARPS)), block(LA_WARPS * 32);
  const size_t smem = (size_t)(LA_TILE * (Dk + 1) + LA_WARPS * Dk) * sizeof(float);
  const int per = ceil_div(L, 32);
#define TL_LATENT(LPER_)                                                                                                         \
  do {                                                                                                                           \
    if (smem > 48 * 1024)                                                                                                        \
      cudaFuncSetAttribute(attention_latent_kernel<T, LPER_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
    attention_latent_kernel<T, LPER_><<<grid, block, smem, stream>>>(q, (const T*)cache, table, max_pages, page_size, num_pages, \
                                                                     req_of_row, positions, scale, window, (T*)out, H, L, Dk,    \
                                                                     status, sinks);                                             \
  } while (0)
  if (per <= 1) TL_LATENT(1);
  else if (per <= 2) TL_LATENT(2);
  else if (per <= 4) TL_LATENT(4);
  else if (per <= 8) TL_LATENT(8);
  else TL_LATENT(16);
#undef TL_LATENT
  TL_LAUNCH_CHECK();
  return 0;
}

}  // namespace tl

using namespace tl;

// q [rows, ld_q]: H heads of D unrotated then Rr rotated entries; kv [rows, ld_kv]: L latent entries then Rr; cache
// [pages, 1, page_size, L + Rr]; q_out float [rows, H, L + Rr] (only the last Rr entries of every head are written here).
extern "C" int tl_latent_prepare(const void* q, long long ld_q, const void* kv, long long ld_kv, const float* c_weight, float eps,
                                 const float* inv_freq, int rot_dims, const int* positions, const int* req_of_row,
                                 const int* table, int max_pages, int page_size, int num_pages, void* cache, float* q_out,
                                 int rows, int H, int D, int L, int Rr, int dtype, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && H > 0 && D >= 0 && L > 0 && Rr >= 0, "latent prepare: %d rows, %d heads of %d + %d, latent %d", rows, H, D,
             Rr, L);
  TL_REQUIRE(rot_dims >= 0 && rot_dims <= Rr && rot_dims % 2 == 0, "latent prepare: %d rotated entries of %d", rot_dims, Rr);
  TL_REQUIRE(table && cache && q_out && page_size > 0 && (rot_dims == 0 || inv_freq), "latent prepare: a cache, a table and "
             "frequencies are needed");
  if (dtype == TL_FP32)
    latent_prepare_kernel<float><<<rows, 128, 0, stream>>>((const float*)q, ld_q, (const float*)kv, ld_kv, c_weight, eps, inv_freq,
                                                           rot_dims, positions, req_of_row, table, max_pages, page_size,
                                                           num_pages, (float*)cache, q_out, H, D, L, Rr, status);
  else
    latent_prepare_kernel<bf16><<<rows, 128, 0, stream>>>((const bf16*)q, ld_q, (const bf16*)kv, ld_kv, c_weight, eps, inv_freq,
                                                          rot_dims, positions, req_of_row, table, max_pages, page_size, num_pages,
                                                          (bf16*)cache, q_out, H, D, L, Rr, status);
  TL_LAUNCH_CHECK();
  return 0;
}

// out[r, :n] = w * in[r, :n] / rms(in[r, :n]) for rows of `dtype` with strides ld_in and ld_out (elements).
extern "C" int tl_rmsnorm_rows(const void* in, long long ld_in, const float* w, float eps, void* out, long long ld_out, int rows,
                               int n, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && n > 0 && in && out && w, "rmsnorm rows: %d rows of %d", rows, n);
  if (dtype == TL_FP32)
    rmsnorm_rows_kernel<float><<<rows, 128, 0, stream>>>((const float*)in, ld_in, w, eps, (float*)out, ld_out, n);
  else
    rmsnorm_rows_kernel<bf16><<<rows, 128, 0, stream>>>((const bf16*)in, ld_in, w, eps, (bf16*)out, ld_out, n);
  TL_LAUNCH_CHECK();
  return 0;
}

// out[r * ld_out + h * out_head + n] = sum_k a[r * ld_a + h * a_head + k] * w[(h * N + n) * K + k]; a and w of `dtype`, out of
// `out_dtype`.
extern "C" int tl_head_linear(const void* a, long long ld_a, long long a_head, const void* w, void* out, long long ld_out,
                              long long out_head, int rows, int H, int N, int K, int dtype, int out_dtype, const void* gate,
                              long long ld_gate, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && H > 0 && H <= 65535 && N > 0 && K > 0, "head product: %d rows, %d heads, %d x %d", rows, H, N, K);
  TL_REQUIRE(ceil_div(rows, HL_ROWS) <= 65535, "head product: %d rows in one launch", rows);
  const dim3 grid(ceil_div(N, HL_COLS), ceil_div(rows, HL_ROWS), H);
#define TL_HL(T_, TO_)                                                                                                      \
  head_linear_kernel<T_, TO_><<<grid, 256, 0, stream>>>((const T_*)a, ld_a, a_head, (const T_*)w, (TO_*)out, ld_out, out_head, \
                                                        rows, N, K, (const T_*)gate, ld_gate)
  if (dtype == TL_FP32) {
    TL_REQUIRE(out_dtype == TL_FP32, "head product: 32-bit operands give a 32-bit result");
    TL_HL(float, float);
  } else if (out_dtype == TL_FP32) {
    TL_HL(bf16, float);
  } else {
    TL_HL(bf16, bf16);
  }
#undef TL_HL
  TL_LAUNCH_CHECK();
  return 0;
}

// q float [rows, H, Dk] (Dk = L + the rotated part); cache [pages, 1, page_size, Dk]; out [rows, H, L] of the cache's type.
extern "C" int tl_attention_latent(const float* q, const void* cache, const int* table, int max_pages, int page_size,
                                   int num_pages, const int* req_of_row, const int* positions, float scale, int window, void* out,
                                   int rows, int H, int L, int Dk, int dtype, int* status, const float* sinks, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && H > 0 && H <= 65535 * LA_WARPS && L > 0 && Dk >= L, "latent attention: %d rows, %d heads, latent %d of %d",
             rows, H, L, Dk);
  TL_REQUIRE(L <= 512, "latent attention: a latent of %d; up to 512 are implemented", L);
  TL_REQUIRE((size_t)(LA_TILE * (Dk + 1) + LA_WARPS * Dk) * sizeof(float) <= 200 * 1024, "latent attention: keys of %d entries", Dk);
  TL_REQUIRE(window >= 0 && page_size > 0, "latent attention: window %d, pages of %d", window, page_size);
  if (dtype == TL_FP32)
    return launch_latent<float>(q, cache, table, max_pages, page_size, num_pages, req_of_row, positions, scale, window, out, rows,
                                H, L, Dk, status, sinks, stream);
  return launch_latent<bf16>(q, cache, table, max_pages, page_size, num_pages, req_of_row, positions, scale, window, out, rows, H,
                             L, Dk, status, sinks, stream);
}
