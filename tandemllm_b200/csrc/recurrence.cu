// Linear recurrences over a matrix state a head, S [D keys, VD values] in 32-bit, carried in a request's slot:
//
//   decayed outer products   S <- c_h S + k v^T                                   (a fixed decay a head)
//   generalized delta rule   S <- diag(d) S - (a * u) (u^T S) + k v^T             (both terms read the old S)
//                            d = exp(-rate * sigmoid(w + w0)), a = sigmoid(a' + a_b), u = k / sqrt(sum k^2 + key_eps)
//   gated outer products     S <- diag(d) S + k v^T                               (a decay a key channel and token)
//                            d = sigmoid(w + w0)^rate = exp(-rate * softplus(-(w + w0)))
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
//
// Steps that bring long portions run two kernels instead: one warp a (row, head) forms the activations, decays and unit
// keys of all rows side by side into a scratch tensor, and the scan fetches them (and the values) a few tokens ahead
// through a ring of cp.async stages that a warp of its own keeps filled, so that nothing but the state's own chain of
// additions is left in the computing warps' loop. The
// blocks shrink (down to a warp of a few value columns) until the grid fills the GPU: the chain's length in time is the
// same for every block size, so more and smaller blocks only shorten the step. The arithmetic of a token is the same in
// both forms.
#include "common.cuh"

namespace tl {

constexpr int REC_TOKENS = 8;       // tokens staged at a time: one a warp
constexpr int REC_THREADS = 256;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
// sigmoid(z)^rate without forming the sigmoid: exp(-rate * log(1 + e^-z)), the logarithm split so that neither e^-z nor e^z overflows
__device__ __forceinline__ float sigmoid_powf_(float z, float rate) {
  return expf(-rate * (fmaxf(-z, 0.f) + log1pf(expf(-fabsf(z)))));
}

constexpr int RULE_FIXED = 0, RULE_DELTA = 1, RULE_GATED = 2;
__host__ __device__ constexpr int rec_arrays(int rule) { return rule == RULE_DELTA ? 5 : (rule == RULE_GATED ? 3 : 2); }

// Dp = 16 P: D rounded up to what P lanes of 16 keys hold. Shared memory: REC_TOKENS x 5 (or 3) arrays of Dp floats, then
// REC_TOKENS x VD_tile values.
template <int RULE>
__global__ void __launch_bounds__(REC_THREADS) recurrence_scan_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int a_col,
    const float* __restrict__ wl, long long ld_w, const float* __restrict__ w0, const float* __restrict__ a_bias,
    const float* __restrict__ head_decay, float rate, float key_eps, int silu_inputs, float q_scale, float* __restrict__ state,
    long long slot_floats, const int* __restrict__ state_slot, const int* __restrict__ row_start, float* __restrict__ y,
    int H, int D, int VD, int P, int cols_per_block, int write_state) {
  extern __shared__ __align__(16) float sm[];
  const int Dp = 16 * P;
  constexpr bool DELTA = RULE == RULE_DELTA, GATED = RULE == RULE_GATED;
  constexpr int NARR = rec_arrays(RULE);
  // arrays a token: q, k, a decay a channel d (delta rule, gated), and for the delta rule u, au
  float* s_q = sm;
  float* s_k = s_q + REC_TOKENS * Dp;
  float* s_d = s_k + REC_TOKENS * Dp;
  float* s_u = s_d + (DELTA || GATED ? REC_TOKENS * Dp : 0);
  float* s_au = s_u + (DELTA ? REC_TOKENS * Dp : 0);
  float* s_v = sm + NARR * REC_TOKENS * Dp;          // [REC_TOKENS][cols_per_block]

  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cols_per_block;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int part = tid % P, jl = tid / P, j = col0 + jl;
  const bool owns = jl < cols_per_block && j < VD;
  const int r0 = row_start[b], r1 = row_start[b + 1];
  if (r1 <= r0) return;
  float* S = state + (long long)state_slot[b] * slot_floats + (long long)h * D * VD;
  const float c_h = RULE != RULE_FIXED ? 0.f : head_decay[h];

  float s[16];
#pragma unroll
  for (int m = 0; m < 4; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int i = 4 * (part + P * m) + c;
      s[4 * m + c] = (owns && i < D) ? S[(long long)i * VD + j] : 0.f;
    }

  const int chunk_tokens = min(REC_TOKENS, (int)(blockDim.x >> 5));      // a warp a token
  for (int t0 = r0; t0 < r1; t0 += chunk_tokens) {
    const int nt = min(chunk_tokens, r1 - t0);
    __syncthreads();                      // the chunk before has been read
    if (warp < nt) {
      const int tw = warp;
      const float* row = proj + (long long)(t0 + tw) * ld + (long long)h * D;
      const float* vrow = proj + (long long)(t0 + tw) * ld + v_col + (long long)h * VD;
      float* tq = s_q + tw * Dp;
      float* tk = s_k + tw * Dp;
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
        tq[i] = qv * q_scale;
        tk[i] = kv;
        ss = fmaf(kv, kv, ss);
      }
      if (DELTA) {
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss + key_eps);
        const float* wrow = wl + (long long)(t0 + tw) * ld_w + (long long)h * D;
        for (int i = lane; i < Dp; i += 32) {
          float d = 0.f, u = 0.f, au = 0.f;
          if (i < D) {
            d = expf(-rate * sigmoidf_(wrow[i] + w0[h * D + i]));
            u = tk[i] * inv;
            au = sigmoidf_(row[a_col + i] + a_bias[h * D + i]) * u;
          }
          s_d[tw * Dp + i] = d;
          s_u[tw * Dp + i] = u;
          s_au[tw * Dp + i] = au;
        }
      }
      if (GATED) {
        const float* wrow = wl + (long long)(t0 + tw) * ld_w + (long long)h * D;
        for (int i = lane; i < Dp; i += 32) s_d[tw * Dp + i] = i < D ? sigmoid_powf_(wrow[i] + w0[h * D + i], rate) : 0.f;
      }
      for (int c = lane; c < cols_per_block; c += 32) {
        float vv = col0 + c < VD ? vrow[col0 + c] : 0.f;
        if (silu_inputs) vv = siluf_(vv);
        s_v[tw * cols_per_block + c] = vv;
      }
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float4* q4 = reinterpret_cast<const float4*>(s_q + t * Dp);
      const float4* k4 = reinterpret_cast<const float4*>(s_k + t * Dp);
      const float vj = jl < cols_per_block ? s_v[t * cols_per_block + jl] : 0.f;
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
      if (DELTA) {
        const float4* d4 = reinterpret_cast<const float4*>(s_d + t * Dp);
        const float4* u4 = reinterpret_cast<const float4*>(s_u + t * Dp);
        const float4* au4 = reinterpret_cast<const float4*>(s_au + t * Dp);
        float us0 = 0.f, us1 = 0.f, us2 = 0.f, us3 = 0.f;      // four short chains of additions instead of one long one
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float4 u = u4[part + P * m];
          us0 = fmaf(u.x, s[4 * m], us0);
          us1 = fmaf(u.y, s[4 * m + 1], us1);
          us2 = fmaf(u.z, s[4 * m + 2], us2);
          us3 = fmaf(u.w, s[4 * m + 3], us3);
        }
        float us = (us0 + us1) + (us2 + us3);
        for (int off = P >> 1; off > 0; off >>= 1) us += __shfl_xor_sync(0xffffffffu, us, off);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float4 d = d4[part + P * m], au = au4[part + P * m], k = k4[part + P * m], q = q4[part + P * m];
          s[4 * m] = fmaf(d.x, s[4 * m], fmaf(-au.x, us, k.x * vj));
          s[4 * m + 1] = fmaf(d.y, s[4 * m + 1], fmaf(-au.y, us, k.y * vj));
          s[4 * m + 2] = fmaf(d.z, s[4 * m + 2], fmaf(-au.z, us, k.z * vj));
          s[4 * m + 3] = fmaf(d.w, s[4 * m + 3], fmaf(-au.w, us, k.w * vj));
          o0 = fmaf(s[4 * m], q.x, o0);
          o1 = fmaf(s[4 * m + 1], q.y, o1);
          o2 = fmaf(s[4 * m + 2], q.z, o2);
          o3 = fmaf(s[4 * m + 3], q.w, o3);
        }
      } else if (GATED) {
        const float4* d4 = reinterpret_cast<const float4*>(s_d + t * Dp);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float4 d = d4[part + P * m], k = k4[part + P * m], q = q4[part + P * m];
          s[4 * m] = fmaf(d.x, s[4 * m], k.x * vj);
          s[4 * m + 1] = fmaf(d.y, s[4 * m + 1], k.y * vj);
          s[4 * m + 2] = fmaf(d.z, s[4 * m + 2], k.z * vj);
          s[4 * m + 3] = fmaf(d.w, s[4 * m + 3], k.w * vj);
          o0 = fmaf(s[4 * m], q.x, o0);
          o1 = fmaf(s[4 * m + 1], q.y, o1);
          o2 = fmaf(s[4 * m + 2], q.z, o2);
          o3 = fmaf(s[4 * m + 3], q.w, o3);
        }
      } else {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float4 k = k4[part + P * m], q = q4[part + P * m];
          s[4 * m] = fmaf(c_h, s[4 * m], k.x * vj);
          s[4 * m + 1] = fmaf(c_h, s[4 * m + 1], k.y * vj);
          s[4 * m + 2] = fmaf(c_h, s[4 * m + 2], k.z * vj);
          s[4 * m + 3] = fmaf(c_h, s[4 * m + 3], k.w * vj);
          o0 = fmaf(s[4 * m], q.x, o0);
          o1 = fmaf(s[4 * m + 1], q.y, o1);
          o2 = fmaf(s[4 * m + 2], q.z, o2);
          o3 = fmaf(s[4 * m + 3], q.w, o3);
        }
      }
      float o = (o0 + o1) + (o2 + o3);
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

// One warp a (row, head): what the scan needs of a token, [H][rows][NARR][Dp] = q, k (activated), a decay a channel d (delta rule,
// gated), and for the delta rule u, a * u; entries past D are zero (a head's tokens lie together, so a chunk of them is one stretch of memory). With `vact`, the activated values [rows][H * VD] as well.
template <int RULE>
__global__ void __launch_bounds__(128) recurrence_prepare_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int a_col, const float* __restrict__ wl,
    long long ld_w, const float* __restrict__ w0, const float* __restrict__ a_bias, float rate, float key_eps, int silu_inputs,
    float q_scale, float* __restrict__ prep, float* __restrict__ vact, int H, int D, int VD, int Dp, long long pairs) {
  constexpr bool DELTA = RULE == RULE_DELTA, GATED = RULE == RULE_GATED;
  constexpr int NARR = rec_arrays(RULE);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long idx = (long long)blockIdx.x * 4 + warp;
  if (idx >= pairs) return;
  const long long r = idx / H;
  const int h = (int)(idx - r * H);
  const float* row = proj + r * ld + (long long)h * D;
  float* tq = prep + ((long long)h * (pairs / H) + r) * NARR * Dp;
  float* tk = tq + Dp;
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
    tq[i] = qv * q_scale;
    tk[i] = kv;
    ss = fmaf(kv, kv, ss);
  }
  if (GATED) {
    const float* wrow = wl + r * ld_w + (long long)h * D;
    for (int i = lane; i < Dp; i += 32) tq[2 * Dp + i] = i < D ? sigmoid_powf_(wrow[i] + w0[h * D + i], rate) : 0.f;
  }
  if (DELTA) {
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss + key_eps);
    const float* wrow = wl + r * ld_w + (long long)h * D;
    for (int i = lane; i < Dp; i += 32) {
      float d = 0.f, u = 0.f, au = 0.f;
      if (i < D) {
        d = expf(-rate * sigmoidf_(wrow[i] + w0[h * D + i]));
        u = tk[i] * inv;                  // (this lane wrote it)
        au = sigmoidf_(row[a_col + i] + a_bias[h * D + i]) * u;
      }
      tq[2 * Dp + i] = d;
      tq[3 * Dp + i] = u;
      tq[4 * Dp + i] = au;
    }
  }
  if (vact) {
    const float* vrow = proj + r * ld + v_col + (long long)h * VD;
    for (int c = lane; c < VD; c += 32) vact[idx * VD + c] = silu_inputs ? siluf_(vrow[c]) : vrow[c];
  }
}

__device__ __forceinline__ void rec_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void rec_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Sums v[0..T) over the P neighbouring lanes that share a column (`part` = the lane's place among them; P divides 32). Each
// crossing halves what a lane still holds: afterwards v[i], i < T / P, of lane `part` are the whole sums of tokens
// part * (T / P) + i; with more lanes than tokens, v[0] of the P / T lanes from part = token * (P / T) on is that token's sum.
constexpr int REC_GROUP = 8;
constexpr int REC_CHUNK = 16;     // the most tokens a stage holds; a column's values of a stage lie this far apart
template <int T, int P>
__device__ __forceinline__ void rec_reduce_scatter(float (&v)[T], int part) {
#pragma unroll
  for (int step = 0; (P >> 1 >> step) > 0; ++step) {
    const int off = P >> 1 >> step;
    const int cnt = (T >> step) > 1 ? (T >> step) : 1;
    if (cnt > 1) {
      const int half = cnt / 2;
      const bool up = (part & off) != 0;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const float send = up ? v[i] : v[i + half];
        const float keep = up ? v[i + half] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
    }
  }
}

// REC_GROUP tokens (FULL) or the first n of them for one lane: the lane's KPL keys of its column go through the tokens, the
// outputs wait in registers and cross the lanes together. Everything a token needs lies at offsets the compiler knows
// (`tok`: the lane's first four floats of the group's first prepared token; `vcol`: the column's values, a token a float),
// so the group is straight-line code whose loads the compiler moves ahead of the chain.
template <int RULE, int KPL, int DP, bool FULL>
__device__ __forceinline__ void rec_group(float (&s)[KPL], const float* __restrict__ tok, const float* __restrict__ vcol,
                                          float* __restrict__ yg, long long ldy, int n, int part, bool owns, float c_h) {
  constexpr bool DELTA = RULE == RULE_DELTA, GATED = RULE == RULE_GATED;
  constexpr int P = DP / KPL, M = KPL / 4, tok_floats = rec_arrays(RULE) * DP, Q = DP / 4;
  float o[REC_GROUP];
#pragma unroll
  for (int tt = 0; tt < REC_GROUP; ++tt) {
    o[tt] = 0.f;
    if (FULL || tt < n) {
      const float4* a = reinterpret_cast<const float4*>(tok + tt * tok_floats);
      const float vj = vcol[tt];
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
      if (DELTA) {
        float us0 = 0.f, us1 = 0.f, us2 = 0.f, us3 = 0.f;      // four short chains of additions instead of one long one
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4 u = a[3 * Q + P * m];
          us0 = fmaf(u.x, s[4 * m], us0);
          us1 = fmaf(u.y, s[4 * m + 1], us1);
          us2 = fmaf(u.z, s[4 * m + 2], us2);
          us3 = fmaf(u.w, s[4 * m + 3], us3);
        }
        float us = (us0 + us1) + (us2 + us3);
#pragma unroll
        for (int off = P >> 1; off > 0; off >>= 1) us += __shfl_xor_sync(0xffffffffu, us, off);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4 q = a[P * m], k = a[Q + P * m], d = a[2 * Q + P * m], au = a[4 * Q + P * m];
          s[4 * m] = fmaf(d.x, s[4 * m], fmaf(-au.x, us, k.x * vj));
          s[4 * m + 1] = fmaf(d.y, s[4 * m + 1], fmaf(-au.y, us, k.y * vj));
          s[4 * m + 2] = fmaf(d.z, s[4 * m + 2], fmaf(-au.z, us, k.z * vj));
          s[4 * m + 3] = fmaf(d.w, s[4 * m + 3], fmaf(-au.w, us, k.w * vj));
          o0 = fmaf(s[4 * m], q.x, o0);
          o1 = fmaf(s[4 * m + 1], q.y, o1);
          o2 = fmaf(s[4 * m + 2], q.z, o2);
          o3 = fmaf(s[4 * m + 3], q.w, o3);
        }
      } else if (GATED) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4 q = a[P * m], k = a[Q + P * m], d = a[2 * Q + P * m];
          s[4 * m] = fmaf(d.x, s[4 * m], k.x * vj);
          s[4 * m + 1] = fmaf(d.y, s[4 * m + 1], k.y * vj);
          s[4 * m + 2] = fmaf(d.z, s[4 * m + 2], k.z * vj);
          s[4 * m + 3] = fmaf(d.w, s[4 * m + 3], k.w * vj);
          o0 = fmaf(s[4 * m], q.x, o0);
          o1 = fmaf(s[4 * m + 1], q.y, o1);
          o2 = fmaf(s[4 * m + 2], q.z, o2);
          o3 = fmaf(s[4 * m + 3], q.w, o3);
        }
      } else {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4 q = a[P * m], k = a[Q + P * m];
          s[4 * m] = fmaf(c_h, s[4 * m], k.x * vj);
          s[4 * m + 1] = fmaf(c_h, s[4 * m + 1], k.y * vj);
          s[4 * m + 2] = fmaf(c_h, s[4 * m + 2], k.z * vj);
          s[4 * m + 3] = fmaf(c_h, s[4 * m + 3], k.w * vj);
          o0 = fmaf(s[4 * m], q.x, o0);
          o1 = fmaf(s[4 * m + 1], q.y, o1);
          o2 = fmaf(s[4 * m + 2], q.z, o2);
          o3 = fmaf(s[4 * m + 3], q.w, o3);
        }
      }
      o[tt] = (o0 + o1) + (o2 + o3);
    }
  }
  rec_reduce_scatter<REC_GROUP, P>(o, part);
  if (!owns) return;
  if (P <= REC_GROUP) {
    constexpr int each = P <= REC_GROUP ? REC_GROUP / P : 1;
#pragma unroll
    for (int i = 0; i < each; ++i) {
      const int t = part * each + i;
      if (FULL || t < n) yg[t * ldy] = o[i];
    }
  } else {
    constexpr int share = P > REC_GROUP ? P / REC_GROUP : 1;
    const int t = part / share;
    if (part % share == 0 && (FULL || t < n)) yg[t * ldy] = o[0];
  }
}

// The scan over prepared tokens. Block: cols_per_block * P computing threads (a multiple of 32) and one more warp, the
// producer, which does nothing but fetch: it keeps STAGES - 1 chunks of TC tokens in flight (each token's NARR * Dp prepared
// floats, then the chunk's values, a column's REC_CHUNK apart) and meets the computing warps at one barrier a chunk, when the next
// chunk has landed and the last one has been read.
// KPL keys of a column a lane (16 or 4): with 4, four times as many lanes share a column and a token takes a warp a
// third of the instructions, at the price of two more lane crossings a sum; the launcher takes 4 where the GPU would
// otherwise stand idle. DP: the keys a head, filled up to a power of two (16 at least); sizes known to the compiler keep
// the loop free of address arithmetic.
constexpr int REC_STAGES = 3;
template <int RULE, int KPL, int DP>
__global__ void __launch_bounds__(REC_THREADS + 32) recurrence_scan_staged_kernel(
    const float* __restrict__ prep, const float* __restrict__ vsrc, long long ld_v, int v_col, const float* __restrict__ head_decay,
    float* __restrict__ state, long long slot_floats, const int* __restrict__ state_slot, const int* __restrict__ row_start,
    float* __restrict__ y, long long rows, int H, int D, int VD, int cols_per_block, int TC, int write_state) {
  constexpr int STAGES = REC_STAGES, P = DP / KPL, Dp = DP;
  extern __shared__ __align__(16) float sm[];
  constexpr int NARR = rec_arrays(RULE);
  constexpr int M = KPL / 4, tok_floats = NARR * Dp;
  const int stage_floats = TC * tok_floats + REC_CHUNK * cols_per_block;
  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cols_per_block;
  const int tid = threadIdx.x, nth = blockDim.x - 32;
  const bool producer = tid >= nth;
  const int part = tid % P, jl = tid / P, j = col0 + jl;
  const bool owns = !producer && j < VD;
  const int r0 = row_start[b], r1 = row_start[b + 1];
  if (r1 <= r0) return;
  float* S = state + (long long)state_slot[b] * slot_floats + (long long)h * D * VD;
  const float c_h = RULE != RULE_FIXED ? 0.f : head_decay[h];
  const int n_chunks = (r1 - r0 + TC - 1) / TC;

  // (the producer's lanes only)
  auto load = [&](int chunk) {
    const int lane = tid - nth;
    const int t0 = r0 + chunk * TC, nt = min(TC, r1 - t0);
    float* base = sm + (chunk % STAGES) * stage_floats;
    const float* src = prep + ((long long)h * rows + t0) * tok_floats;
    const int pieces = nt * (tok_floats / 4);
#pragma unroll 4
    for (int i = lane; i < pieces; i += 32) rec_cp16(base + 4 * i, src + 4 * i);
    float* vb = base + TC * tok_floats;
    const float* vs = vsrc + (long long)t0 * ld_v + v_col + (long long)h * VD + col0;
    for (int e = lane; e < nt * cols_per_block; e += 32) {
      const int t = e / cols_per_block, c = e - t * cols_per_block;
      if (col0 + c < VD) rec_cp4(vb + c * REC_CHUNK + t, vs + (long long)t * ld_v + c);
      else vb[c * REC_CHUNK + t] = 0.f;
    }
  };
  float s[KPL];
  if (producer) {
#pragma unroll
    for (int s0 = 0; s0 < STAGES - 1; ++s0) {
      if (s0 < n_chunks) load(s0);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");       // chunk 0 has landed
  } else {
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = 4 * (part + P * m) + c;
        s[4 * m + c] = (owns && i < D) ? S[(long long)i * VD + j] : 0.f;
      }
  }
  __syncthreads();

  for (int chunk = 0; chunk < n_chunks; ++chunk) {
    if (producer) {
      // the stage of chunk - 1 is free (everybody passed the barrier behind it): refill it, then wait for chunk + 1
      if (chunk + STAGES - 1 < n_chunks) load(chunk + STAGES - 1);
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    } else {
      const int t0 = r0 + chunk * TC, nt = min(TC, r1 - t0);
      const float* base = sm + (chunk % STAGES) * stage_floats;
      const float* tok = base + 4 * part;
      const float* vcol = base + TC * tok_floats + jl * REC_CHUNK;
      const long long ldy = (long long)H * VD;
      float* yg = y + (long long)t0 * ldy + (long long)h * VD + j;
      int g = 0;
      for (; g + REC_GROUP <= nt; g += REC_GROUP)
        rec_group<RULE, KPL, DP, true>(s, tok + g * tok_floats, vcol + g, yg + g * ldy, ldy, REC_GROUP, part, owns, c_h);
      if (g < nt) rec_group<RULE, KPL, DP, false>(s, tok + g * tok_floats, vcol + g, yg + g * ldy, ldy, nt - g, part, owns, c_h);
    }
    __syncthreads();
  }
  if (write_state && owns) {
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = 4 * (part + P * m) + c;
        if (i < D) S[(long long)i * VD + j] = s[4 * m + c];
      }
  }
}

// grid (rows, groups): out[r, c] = y[r, c] / sqrt(mean over the group of y^2 + eps) * weight[c] * act(gate[r, c]) * scale, act the
// sigmoid or (silu_gate) g sigmoid(g); with shared_weight the weight has one group's entries, which every group uses
template <typename T, typename G>
__global__ void group_norm_gate_kernel(const float* __restrict__ y, const G* __restrict__ gate, long long ld_gate,
                                       const float* __restrict__ weight, float eps, float scale, T* __restrict__ out,
                                       long long ld_out, int width, int group, int silu_gate, int shared_weight) {
  __shared__ float red[33];
  const int r = blockIdx.x, c0 = blockIdx.y * group;
  const float* yr = y + (long long)r * width + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < group; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)group + eps);
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    const float g = to_f32(gate[(long long)r * ld_gate + c0 + i]);
    const float a = silu_gate ? g / (1.f + expf(-g)) : 1.f / (1.f + expf(-g));
    out[(long long)r * ld_out + c0 + i] = from_f32<T>(yr[i] * inv * weight[(shared_weight ? 0 : c0) + i] * a * scale);
  }
}

}  // namespace tl

using namespace tl;

// Threads a block (a multiple of 32, at least P) and the value columns it takes: the largest block that still gives the GPU
// `want_blocks` blocks, else a single warp; never more columns than there are. (Steps of a few rows want many blocks in
// flight for the states they read and write; the staged form's blocks each fetch every prepared token of their head, so
// they stay as large as fills three SMs in four.)
static void recurrence_block(int requests, int H, int VD, int P, long long want_blocks, int* threads, int* cols) {
  const int needed = ((VD * P + 31) / 32) * 32;
  int th = REC_THREADS;
  while (th > 32 && th / 2 >= P && (long long)requests * H * ceil_div(VD, th / P) < want_blocks) th >>= 1;
  if (th > needed) th = needed;
  if (th < P) th = P;
  *threads = th;
  *cols = th / P;
}

// floats of scratch the staged form wants for `rows` rows: the prepared tokens, then (fixed decays) the activated values
// (rule: 0 a fixed decay a head, 1 the delta rule, 2 a decay a key channel and token)
extern "C" long long tl_recurrence_scratch_floats(long long rows, int H, int D, int VD, int rule) {
  int P = 1;
  while (16 * P < D) P <<= 1;
  return rows * H * (rec_arrays(rule) * 16LL * P + (rule == RULE_FIXED ? VD : 0));
}

// scratch: null runs the one-kernel form (steps of a few rows a request); else tl_recurrence_scratch_floats(rows, ...) floats.
extern "C" int tl_recurrence_scan(const float* proj, long long ld, int q_col, int k_col, int v_col, int a_col, const float* wl,
                                  long long ld_w, const float* w0, const float* a_bias, const float* head_decay, float rate,
                                  float key_eps, int silu_inputs, float* state, long long slot_floats, const int* state_slot,
                                  const int* row_start, int requests, float* y, int H, int D, int VD, int write_state,
                                  float* scratch, long long rows, int sm_count, int rule, float q_scale, cudaStream_t stream) {
  if (requests == 0) return 0;
  TL_REQUIRE(rule >= RULE_FIXED && rule <= RULE_GATED, "recurrence_scan: rule %d is not one of 0..2", rule);
  const bool delta = rule == RULE_DELTA, fixed = rule == RULE_FIXED;
  TL_REQUIRE(H > 0 && D >= 1 && D <= 512 && VD >= 1, "recurrence_scan: %d heads, %d keys (up to 512), %d values", H, D, VD);
  TL_REQUIRE(delta ? (wl && w0 && a_bias && a_col >= 0) : (fixed ? head_decay != nullptr : (wl && w0)),
             "recurrence_scan: the delta rule wants w, w0, a and its bias; the gated rule w and w0; the fixed decay a number a head");
  TL_REQUIRE(H <= 65535, "recurrence_scan: %d heads exceed the grid limit", H);
  int P = 1;
  while (16 * P < D) P <<= 1;
  const int P16 = P;
  const int sms = sm_count > 0 ? sm_count : 148;
  // the staged form gives a column to four times as many lanes (4 keys a lane) until the GPU has two warps a scheduler
  int kpl = 16;
  if (scratch && 4 * P <= 32 && (long long)requests * H * VD * P < 256LL * sms) {
    kpl = 4;
    P *= 4;
  }
  int threads, cols_per_block;
  recurrence_block(requests, H, VD, P, scratch ? (3LL * sms) / 4 : 2LL * sms, &threads, &cols_per_block);
  const int tiles = ceil_div(VD, cols_per_block);
  TL_REQUIRE(tiles <= 65535, "recurrence_scan: %d tiles of value columns exceed the grid limit", tiles);
  dim3 grid(requests, H, tiles);
  const int narr = rec_arrays(rule), Dp = 16 * P16;
  if (scratch) {
    const long long pairs = rows * H;
    float* prep = scratch;
    float* vact = fixed ? scratch + pairs * narr * Dp : nullptr;
    const unsigned pblocks = (unsigned)((pairs + 3) / 4);
#define TL_RPREP(RULE_)                                                                                                          \
  recurrence_prepare_kernel<RULE_><<<pblocks, 128, 0, stream>>>(proj, ld, q_col, k_col, v_col, a_col, wl, ld_w, w0, a_bias, rate, \
                                                                key_eps, silu_inputs, q_scale, prep, vact, H, D, VD, Dp, pairs)
    if (delta) TL_RPREP(RULE_DELTA);
    else if (fixed) TL_RPREP(RULE_FIXED);
    else TL_RPREP(RULE_GATED);
#undef TL_RPREP
    TL_LAUNCH_CHECK();
    // tokens a stage: as many (16 at most) as 96 KB hold in three stages
    int TC = REC_CHUNK;
    auto bytes = [&](int tc) { return (size_t)REC_STAGES * (tc * narr * Dp + REC_CHUNK * cols_per_block) * sizeof(float); };
    while (TC > 1 && bytes(TC) > 96 * 1024) TC >>= 1;
    const size_t smem = bytes(TC);
    const float* vsrc = fixed ? vact : proj;
    const long long ld_v = fixed ? (long long)H * VD : ld;
    const int vc = fixed ? 0 : v_col;
#define TL_RSS(DELTA_, KPL_, DP_)                                                                                               \
  do {                                                                                                                          \
    if (smem > 48 * 1024)                                                                                                       \
      cudaFuncSetAttribute(recurrence_scan_staged_kernel<DELTA_, KPL_, DP_>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                           96 * 1024);                                                                                          \
    recurrence_scan_staged_kernel<DELTA_, KPL_, DP_><<<grid, threads + 32, smem, stream>>>(                                     \
        prep, vsrc, ld_v, vc, head_decay, state, slot_floats, state_slot, row_start, y, rows, H, D, VD, cols_per_block, TC,           \
        write_state);                                                                                                           \
  } while (0)
#define TL_RSS_D(DELTA_, DP_)                   \
  do {                                          \
    if (kpl == 16) TL_RSS(DELTA_, 16, DP_);     \
    else if (DP_ <= 128) TL_RSS(DELTA_, 4, (DP_ <= 128 ? DP_ : 128)); \
  } while (0)
#define TL_RSS_ALL(DELTA_)                      \
  do {                                          \
    switch (Dp) {                               \
      case 16: TL_RSS_D(DELTA_, 16); break;     \
      case 32: TL_RSS_D(DELTA_, 32); break;     \
      case 64: TL_RSS_D(DELTA_, 64); break;     \
      case 128: TL_RSS_D(DELTA_, 128); break;   \
      case 256: TL_RSS_D(DELTA_, 256); break;   \
      default: TL_RSS_D(DELTA_, 512); break;    \
    }                                           \
  } while (0)
    if (delta) TL_RSS_ALL(RULE_DELTA);
    else if (fixed) TL_RSS_ALL(RULE_FIXED);
    else TL_RSS_ALL(RULE_GATED);
#undef TL_RSS_ALL
#undef TL_RSS_D
#undef TL_RSS
    TL_LAUNCH_CHECK();
    return 0;
  }
  const size_t smem = (size_t)(narr * REC_TOKENS * Dp + REC_TOKENS * cols_per_block) * sizeof(float);
#define TL_RSCAN(RULE_)                                                                                                        \
  do {                                                                                                                         \
    if (smem > 48 * 1024)                                                                                                      \
      cudaFuncSetAttribute(recurrence_scan_kernel<RULE_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
    recurrence_scan_kernel<RULE_><<<grid, threads, smem, stream>>>(proj, ld, q_col, k_col, v_col, a_col, wl, ld_w, w0, a_bias, \
                                                                   head_decay, rate, key_eps, silu_inputs, q_scale, state,     \
                                                                   slot_floats, state_slot, row_start, y, H, D, VD, P,         \
                                                                   cols_per_block, write_state);                               \
  } while (0)
  if (delta) TL_RSCAN(RULE_DELTA);
  else if (fixed) TL_RSCAN(RULE_FIXED);
  else TL_RSCAN(RULE_GATED);
#undef TL_RSCAN
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_group_norm_gate(const float* y, const void* gate, long long ld_gate, int gate_dtype, const float* weight,
                                  float eps, float scale, void* out, long long ld_out, int rows, int width, int groups,
                                  int dtype, int silu_gate, int shared_weight, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(width > 0 && groups > 0 && width % groups == 0 && groups <= 65535, "group_norm_gate: rows of %d in %d parts", width,
             groups);
  const int group = width / groups;
  const int threads = group >= 1024 ? 256 : (group >= 256 ? 128 : (group > 32 ? 64 : 32));
  dim3 grid(rows, groups);
#define TL_GNG(T_, G_)                                                                                                   \
  group_norm_gate_kernel<T_, G_><<<grid, threads, 0, stream>>>(y, (const G_*)gate, ld_gate, weight, eps, scale, (T_*)out, \
                                                               ld_out, width, group, silu_gate, shared_weight)
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
