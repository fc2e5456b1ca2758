// A product a head on the tensor cores (bfloat16): out[r, h, n] = sum_k a[r, h, k] w[h, n, k], the two regrouped products
// of latent attention (the query's unrotated part through a head's key matrix, the weighted latents through its value
// matrix). A CTA of four warps makes 64 rows x 64 outputs of one head; k comes in blocks of 64 through shared memory
// (16-byte loads where rows and heads are aligned for them, else element by element), rows padded so that the eight rows
// an operand load touches fall into different banks; `mma.sync` m16n8k16 with 32-bit accumulators, k in ascending order,
// so a row's result does not depend on the rows beside it. A decode step's few rows leave most of a tile's rows empty;
// the kernel is then bound by the heads' weights, which it reads once.
#include "common.cuh"

namespace tl {

constexpr int HM_TILE = 64, HM_K = 64, HM_LD = HM_K + 8;

__device__ __forceinline__ void hm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (ceil(N / 64), ceil(rows / 64), H), 128 threads
template <typename TO>
__global__ void __launch_bounds__(128) head_linear_mma_kernel(const bf16* __restrict__ a, long long ld_a, long long a_head,
                                                              const bf16* __restrict__ w, TO* __restrict__ out, long long ld_out,
                                                              long long out_head, int rows, int N, int K, int vec,
                                                              const bf16* __restrict__ gate, long long ld_gate) {
  __shared__ __align__(16) bf16 sA[HM_TILE][HM_LD];
  __shared__ __align__(16) bf16 sW[HM_TILE][HM_LD];
  const int h = blockIdx.z, r0 = blockIdx.y * HM_TILE, n0 = blockIdx.x * HM_TILE;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const bf16* ah = a + (long long)h * a_head;
  const bf16* wh = w + (long long)h * N * K;
  float acc[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HM_K) {
    __syncthreads();
    if (vec) {
      for (int i = threadIdx.x; i < HM_TILE * (HM_K / 8); i += blockDim.x) {
        const int rr = i / (HM_K / 8), c = (i - rr * (HM_K / 8)) * 8;
        uint4 va = make_uint4(0u, 0u, 0u, 0u), vw = make_uint4(0u, 0u, 0u, 0u);
        if (k0 + c < K) {
          if (r0 + rr < rows) va = *reinterpret_cast<const uint4*>(ah + (long long)(r0 + rr) * ld_a + k0 + c);
          if (n0 + rr < N) vw = *reinterpret_cast<const uint4*>(wh + (long long)(n0 + rr) * K + k0 + c);
        }
        *reinterpret_cast<uint4*>(&sA[rr][c]) = va;
        *reinterpret_cast<uint4*>(&sW[rr][c]) = vw;
      }
    } else {
      for (int i = threadIdx.x; i < HM_TILE * HM_K; i += blockDim.x) {
        const int rr = i / HM_K, c = i - rr * HM_K;
        const bool in = k0 + c < K;
        sA[rr][c] = (in && r0 + rr < rows) ? ah[(long long)(r0 + rr) * ld_a + k0 + c] : __float2bfloat16_rn(0.f);
        sW[rr][c] = (in && n0 + rr < N) ? wh[(long long)(n0 + rr) * K + k0 + c] : __float2bfloat16_rn(0.f);
      }
    }
    __syncthreads();
    const uint32_t* a_lo = reinterpret_cast<const uint32_t*>(&sA[warp * 16 + g][0]);
    const uint32_t* a_hi = reinterpret_cast<const uint32_t*>(&sA[warp * 16 + g + 8][0]);
#pragma unroll
    for (int ks = 0; ks < HM_K / 16; ++ks) {
      uint32_t fa[4];
      fa[0] = a_lo[ks * 8 + t];
      fa[1] = a_hi[ks * 8 + t];
      fa[2] = a_lo[ks * 8 + 4 + t];
      fa[3] = a_hi[ks * 8 + 4 + t];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const uint32_t* wr = reinterpret_cast<const uint32_t*>(&sW[n * 8 + g][0]);
        hm_mma(acc[n], fa, wr[ks * 8 + t], wr[ks * 8 + 4 + t]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r0 + warp * 16 + g + 8 * r;
    if (row >= rows) continue;
    TO* o = out + (long long)row * ld_out + (long long)h * out_head;
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = n0 + n * 8 + 2 * t + e;
        if (col < N) {
          float v = acc[n][2 * r + e];
          // (gate [rows, H * N] logits, rows ld_gate apart: the result times their sigmoid)
          if (gate) v *= 1.f / (1.f + expf(-to_f32(gate[(long long)row * ld_gate + (long long)h * N + col])));
          o[col] = from_f32<TO>(v);
        }
      }
  }
}

}  // namespace tl

using namespace tl;

// out[r * ld_out + h * out_head + n] = sum_k a[r * ld_a + h * a_head + k] * w[(h * N + n) * K + k]; a, w bfloat16; out bfloat16
// or float32 (`out_dtype`). `gate` (bfloat16 logits [rows, H * N], rows ld_gate apart; may be null): out times sigmoid(gate).
extern "C" int tl_head_linear_mma(const void* a, long long ld_a, long long a_head, const void* w, void* out, long long ld_out,
                                  long long out_head, int rows, int H, int N, int K, int out_dtype, const void* gate,
                                  long long ld_gate, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && H > 0 && H <= 65535 && N > 0 && K > 0, "head product: %d rows, %d heads, %d x %d", rows, H, N, K);
  TL_REQUIRE(ceil_div(rows, HM_TILE) <= 65535, "head product: %d rows in one launch", rows);
  const int vec = (K % 8 == 0 && ld_a % 8 == 0 && a_head % 8 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0) ? 1 : 0;
  const dim3 grid(ceil_div(N, HM_TILE), ceil_div(rows, HM_TILE), H);
  if (out_dtype == TL_FP32)
    head_linear_mma_kernel<float><<<grid, 128, 0, stream>>>((const bf16*)a, ld_a, a_head, (const bf16*)w, (float*)out, ld_out,
                                                            out_head, rows, N, K, vec, (const bf16*)gate, ld_gate);
  else
    head_linear_mma_kernel<bf16><<<grid, 128, 0, stream>>>((const bf16*)a, ld_a, a_head, (const bf16*)w, (bf16*)out, ld_out,
                                                           out_head, rows, N, K, vec, (const bf16*)gate, ld_gate);
  TL_LAUNCH_CHECK();
  return 0;
}
