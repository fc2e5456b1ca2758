// Linear recurrences over a matrix state a head, S [D keys, VD values] in 32-bit, carried in a request's slot:
//
//   decayed outer products   S <- c_h S + k v^T                                   (a fixed decay a head)
//   generalized delta rule   S <- diag(d) S - (a * u) (u^T S) + k v^T             (both terms read the old S)
//                            d = exp(-rate * sigmoid(w + w0)), a = sigmoid(a' + a_b), u = k / sqrt(sum k^2 + key_eps)
//   output                   o = S^T q   with the new S
//
// and the norm behind them: out = y / rms(y) over each of `groups` equal parts of a row, times a weight, times
// sigmoid(gate), times a constant.
//
// The scan: a block takes one (request, head, tile of value columns) and walks the request's rows of the step in
// order, starting from the slot's state and leaving the slot as the next portion needs it. Column j of S is held in
// registers by P neighbouring lanes, 16 keys each (key 4 (part + P m) + c, m, c < 4), so the two sums over keys are
// shuffles among P lanes and no thread waits for another inside a token. Eight tokens at a time are staged in shared
// memory: a warp a token forms the activations, decays and the unit key once (never once a thread). Everything is
// 32-bit. A row's result depends on its request's earlier rows only, added in a fixed order.
#include "common.cuh"

namespace tl {

constexpr int REC_TOKENS = 8;       // tokens staged at a time: one a warp
constexpr int REC_THREADS = 256;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }

// Dp = 16 P: D rounded up to what P lanes of 16 keys hold. Shared memory: REC_TOKENS x 5 (or 3) arrays of Dp floats, then
// REC_TOKENS x VD_tile values.
template <bool DELTA>
__global__ void __launch_bounds__(REC_THREADS) recurrence_scan_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int a_col,
    const float* __restrict__ wl, long long ld_w, const float* __restrict__ w0, const float* __restrict__ a_bias,
    const float* __restrict__ head_decay, float rate, float key_eps, int silu_inputs, float* __restrict__ state,
    long long slot_floats, const int* __restrict__ state_slot, const int* __restrict__ row_start, float* __restrict__ y,
    int H, int D, int VD, int P, int cols_per_block, int write_state) {
  extern __shared__ __align__(16) float sm[];
  const int Dp = 16 * P;
  constexpr int NARR = DELTA ? 5 : 2;
  // arrays a token: q, k, and for the delta rule d, u, au
  float* s_q = sm;
  float* s_k = s_q + REC_TOKENS * Dp;
  float* s_d = s_k + REC_TOKENS * Dp;
  float* s_u = s_d + (DELTA ? REC_TOKENS * Dp : 0);
  float* s_au = s_u + (DELTA ? REC_TOKENS * Dp : 0);
  float* s_v = sm + NARR * REC_TOKENS * Dp;          // [REC_TOKENS][cols_per_block]

  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cols_per_block;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int part = tid % P, jl = tid / P, j = col0 + jl;
  const bool owns = jl < cols_per_block && j < VD;
  const int r0 = row_start[b], r1 = row_start[b + 1];
  if (r1 <= r0) return;
  float* S = state + (long long)state_slot[b] * slot_floats + (long long)h * D * VD;
  const float c_h = DELTA ? 0.f : head_decay[h];

  float s[16];
#pragma unroll
  for (int m = 0; m < 4; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int i = 4 * (part + P * m) + c;
      s[4 * m + c] = (owns && i < D) ? S[(long long)i * VD + j] : 0.f;
    }

  for (int t0 = r0; t0 < r1; t0 += REC_TOKENS) {
    const int nt = min(REC_TOKENS, r1 - t0);
    __syncthreads();                      // the chunk before has been read
    if (warp < nt) {
      const float* row = proj + (long long)(t0 + warp) * ld + (long long)h * D;
      const float* vrow = proj + (long long)(t0 + warp) * ld + v_col + (long long)h * VD;
      float* tq = s_q + warp * Dp;
      float* tk = s_k + warp * Dp;
      float ss = 0.f;
      for (int i = lane; i < Dp; i += 32) {
        float qv = 0.f, kv = 0.f;
        if (i < D) {
          qv = row[q_col + i];
          kv = row[k_col + i];
          if (silu_inputs) {
            qv = siluf_(qv);
            kv = siluf_(kv);
          }
        }
        tq[i] = qv;
        tk[i] = kv;
        ss = fmaf(kv, kv, ss);
      }
      if (DELTA) {
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss + key_eps);
        const float* wrow = wl + (long long)(t0 + warp) * ld_w + (long long)h * D;
        for (int i = lane; i < Dp; i += 32) {
          float d = 0.f, u = 0.f, au = 0.f;
          if (i < D) {
            d = expf(-rate * sigmoidf_(wrow[i] + w0[h * D + i]));
            u = tk[i] * inv;
            au = sigmoidf_(row[a_col + i] + a_bias[h * D + i]) * u;
          }
          s_d[warp * Dp + i] = d;
          s_u[warp * Dp + i] = u;
          s_au[warp * Dp + i] = au;
        }
      }
      for (int c = lane; c < cols_per_block; c += 32) {
        float vv = col0 + c < VD ? vrow[col0 + c] : 0.f;
        if (silu_inputs) vv = siluf_(vv);
        s_v[warp * cols_per_block + c] = vv;
      }
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float4* q4 = reinterpret_cast<const float4*>(s_q + t * Dp);
      const float4* k4 = reinterpret_cast<const float4*>(s_k + t * Dp);
      const float vj = jl < cols_per_block ? s_v[t * cols_per_block + jl] : 0.f;
      float o = 0.f;
      if (DELTA) {
        const float4* d4 = reinterpret_cast<const float4*>(s_d + t * Dp);
        const float4* u4 = reinterpret_cast<const float4*>(s_u + t * Dp);
        const float4* au4 = reinterpret_cast<const float4*>(s_au + t * Dp);
        float us = 0.f;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float4 u = u4[part + P * m];
          us = fmaf(u.x, s[4 * m], us);
          us = fmaf(u.y, s[4 * m + 1], us);
          us = fmaf(u.z, s[4 * m + 2], us);
          us = fmaf(u.w, s[4 * m + 3], us);
        }
        for (int off = P >> 1; off > 0; off >>= 1) us += __shfl_xor_sync(0xffffffffu, us, off);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float4 d = d4[part + P * m], au = au4[part + P * m], k = k4[part + P * m], q = q4[part + P * m];
          s[4 * m] = fmaf(d.x, s[4 * m], fmaf(-au.x, us, k.x * vj));
          s[4 * m + 1] = fmaf(d.y, s[4 * m + 1], fmaf(-au.y, us, k.y * vj));
          s[4 * m + 2] = fmaf(d.z, s[4 * m + 2], fmaf(-au.z, us, k.z * vj));
          s[4 * m + 3] = fmaf(d.w, s[4 * m + 3], fmaf(-au.w, us, k.w * vj));
          o = fmaf(s[4 * m], q.x, o);
          o = fmaf(s[4 * m + 1], q.y, o);
          o = fmaf(s[4 * m + 2], q.z, o);
          o = fmaf(s[4 * m + 3], q.w, o);
        }
      } else {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float4 k = k4[part + P * m], q = q4[part + P * m];
          s[4 * m] = fmaf(c_h, s[4 * m], k.x * vj);
          s[4 * m + 1] = fmaf(c_h, s[4 * m + 1], k.y * vj);
          s[4 * m + 2] = fmaf(c_h, s[4 * m + 2], k.z * vj);
          s[4 * m + 3] = fmaf(c_h, s[4 * m + 3], k.w * vj);
          o = fmaf(s[4 * m], q.x, o);
          o = fmaf(s[4 * m + 1], q.y, o);
          o = fmaf(s[4 * m + 2], q.z, o);
          o = fmaf(s[4 * m + 3], q.w, o);
        }
      }
      for (int off = P >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (part == 0 && owns) y[(long long)(t0 + t) * H * VD + (long long)h * VD + j] = o;
    }
  }
  if (write_state && owns) {
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = 4 * (part + P * m) + c;
        if (i < D) S[(long long)i * VD + j] = s[4 * m + c];
      }
  }
}

// grid (rows, groups): out[r, c] = y[r, c] / sqrt(mean over the group of y^2 + eps) * weight[c] * sigmoid(gate[r, c]) * scale
template <typename T, typename G>
__global__ void group_norm_gate_kernel(const float* __restrict__ y, const G* __restrict__ gate, long long ld_gate,
                                       const float* __restrict__ weight, float eps, float scale, T* __restrict__ out,
                                       long long ld_out, int width, int group) {
  __shared__ float red[33];
  const int r = blockIdx.x, c0 = blockIdx.y * group;
  const float* yr = y + (long long)r * width + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < group; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)group + eps);
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    const float g = to_f32(gate[(long long)r * ld_gate + c0 + i]);
    out[(long long)r * ld_out + c0 + i] = from_f32<T>(yr[i] * inv * weight[c0 + i] * (1.f / (1.f + expf(-g))) * scale);
  }
}

}  // namespace tl

using namespace tl;

extern "C" int tl_recurrence_scan(const float* proj, long long ld, int q_col, int k_col, int v_col, int a_col, const float* wl,
                                  long long ld_w, const float* w0, const float* a_bias, const float* head_decay, float rate,
                                  float key_eps, int silu_inputs, float* state, long long slot_floats, const int* state_slot,
                                  const int* row_start, int requests, float* y, int H, int D, int VD, int write_state,
                                  cudaStream_t stream) {
  if (requests == 0) return 0;
  const bool delta = wl != nullptr;
  TL_REQUIRE(H > 0 && D >= 1 && D <= 512 && VD >= 1, "recurrence_scan: %d heads, %d keys (up to 512), %d values", H, D, VD);
  TL_REQUIRE(delta ? (w0 && a_bias && a_col >= 0) : head_decay != nullptr,
             "recurrence_scan: the delta rule wants w, w0, a and its bias; the fixed decay wants a number a head");
  TL_REQUIRE(H <= 65535, "recurrence_scan: %d heads exceed the grid limit", H);
  int P = 1;
  while (16 * P < D) P <<= 1;
  const int cols_per_block = min(REC_THREADS / P, ((VD + 7) / 8) * 8);
  const int tiles = ceil_div(VD, cols_per_block);
  const size_t smem = (size_t)((delta ? 5 : 2) * REC_TOKENS * 16 * P + REC_TOKENS * cols_per_block) * sizeof(float);
  dim3 grid(requests, H, tiles);
  if (delta) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(recurrence_scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    recurrence_scan_kernel<true><<<grid, REC_THREADS, smem, stream>>>(proj, ld, q_col, k_col, v_col, a_col, wl, ld_w, w0, a_bias,
                                                                      head_decay, rate, key_eps, silu_inputs, state, slot_floats,
                                                                      state_slot, row_start, y, H, D, VD, P, cols_per_block,
                                                                      write_state);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(recurrence_scan_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    recurrence_scan_kernel<false><<<grid, REC_THREADS, smem, stream>>>(proj, ld, q_col, k_col, v_col, a_col, wl, ld_w, w0, a_bias,
                                                                       head_decay, rate, key_eps, silu_inputs, state, slot_floats,
                                                                       state_slot, row_start, y, H, D, VD, P, cols_per_block,
                                                                       write_state);
  }
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_group_norm_gate(const float* y, const void* gate, long long ld_gate, int gate_dtype, const float* weight,
                                  float eps, float scale, void* out, long long ld_out, int rows, int width, int groups,
                                  int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(width > 0 && groups > 0 && width % groups == 0 && groups <= 65535, "group_norm_gate: rows of %d in %d parts", width,
             groups);
  const int group = width / groups;
  const int threads = group >= 1024 ? 256 : (group >= 256 ? 128 : (group > 32 ? 64 : 32));
  dim3 grid(rows, groups);
#define TL_GNG(T_, G_)                                                                                                   \
  group_norm_gate_kernel<T_, G_><<<grid, threads, 0, stream>>>(y, (const G_*)gate, ld_gate, weight, eps, scale, (T_*)out, \
                                                               ld_out, width, group)
  if (dtype == TL_FP32) {
    if (gate_dtype == TL_FP32) TL_GNG(float, float);
    else TL_GNG(float, bf16);
  } else {
    if (gate_dtype == TL_FP32) TL_GNG(bf16, float);
    else TL_GNG(bf16, bf16);
  }
#undef TL_GNG
  TL_LAUNCH_CHECK();
  return 0;
}
