// Layer norm with weight and bias, fused with the residual add in front of it.
//
//   residual += delta;  out = (residual - mean) / sqrt(var + eps) * w + b,  var = mean((residual - mean)^2)
//
// `delta` is a 32-bit tensor [rows, hidden], or `parts` partial sums [parts, rows, hidden] of a product split along k
// that are added in order. Mean and variance are taken in two passes over the row held in shared memory, in 32-bit,
// with a fixed order of additions, so a row's result never depends on the batch. With `gather` output row i is made
// from row gather[i] and the residual stays as it was (the last norm, for the rows whose logits are wanted).
#include "common.cuh"

namespace tl {

template <typename T>
__global__ void __launch_bounds__(256) add_layernorm_kernel(float* __restrict__ residual, const float* __restrict__ delta,
                                                            int parts, long long part_stride, const float* __restrict__ weight,
                                                            const float* __restrict__ bias, float eps, T* __restrict__ out,
                                                            const int* __restrict__ gather, int hidden) {
  extern __shared__ float row[];            // [hidden] + 33 for the reductions
  float* red = row + hidden;
  const int i = blockIdx.x;
  const int r = gather ? gather[i] : i;
  float* res = residual + (size_t)r * hidden;
  float sum = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float x = res[c];
    for (int p = 0; p < parts; ++p) x += delta[(size_t)p * part_stride + (size_t)r * hidden + c];
    if (!gather && parts) res[c] = x;
    row[c] = x;
    sum += x;
  }
  const float mean = block_sum(sum, red) / (float)hidden;
  float sq = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float d = row[c] - mean;
    sq = fmaf(d, d, sq);
  }
  const float var = block_sum(sq, red) / (float)hidden;
  const float inv = 1.f / sqrtf(var + eps);
  T* o = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = from_f32<T>(fmaf((row[c] - mean) * inv, weight[c], bias[c]));
}

}  // namespace tl

using namespace tl;

extern "C" int tl_add_layernorm(float* residual, const float* delta, int parts, long long part_stride, const float* weight,
                                const float* bias, float eps, void* out, const int* gather, int out_rows, int hidden,
                                int dtype, cudaStream_t stream) {
  if (out_rows == 0) return 0;
  TL_REQUIRE(hidden > 0 && hidden <= 11264 && parts >= 0 && (parts == 0 || delta), "add_layernorm: hidden %d (up to 11264), %d parts",
             hidden, parts);
  const int threads = hidden >= 1024 ? 256 : 128;
  const size_t smem = (size_t)(hidden + 40) * sizeof(float);
  if (dtype == TL_FP32)
    add_layernorm_kernel<float><<<out_rows, threads, smem, stream>>>(residual, delta, parts, part_stride, weight, bias, eps,
                                                                     (float*)out, gather, hidden);
  else
    add_layernorm_kernel<bf16><<<out_rows, threads, smem, stream>>>(residual, delta, parts, part_stride, weight, bias, eps,
                                                                    (bf16*)out, gather, hidden);
  TL_LAUNCH_CHECK();
  return 0;
}
