// Random weights on the device: the counter-based generator of
// weights/random_init.py evaluated by one thread per element, so that a model
// made on the device holds the very values that the random-weights folder of
// the same configuration and seed holds.
//
// Element i of a tensor with stream word s:
//   z = splitmix64 finaliser of (s + (i + 1) * 0x9E3779B97F4A7C15)
//   a = z >> 48 (16 bits), f = ((z >> 32) & 0xffff) / 65536
//   x = q[a] + (q[a + 1] - q[a]) * f        q: 65537 quantiles of N(0, 1), float32
//   value = mean + std * x, rounded to the storage type, then widened to the output type
// Every floating-point step is one correctly rounded float32 operation (no
// fused multiply-add), which is what makes host and device agree to the bit.
// The reference has only an offline script for random weights
// (scripts/make-tiny-qwen35.py:96-102).
#include "common.cuh"

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename TO>
__global__ void fill_normal_kernel(TO* __restrict__ out, long long n, unsigned long long stream,
                                   const float* __restrict__ quantiles, float mean, float std_dev,
                                   int round_bf16) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long z = mix64(stream + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull);
    const unsigned int a = (unsigned int)(z >> 48);
    const float f = (float)((unsigned int)(z >> 32) & 0xffffu) * (1.0f / 65536.0f);
    const float q0 = quantiles[a], q1 = quantiles[a + 1];
    const float x = __fadd_rn(q0, __fmul_rn(__fsub_rn(q1, q0), f));
    float v = __fadd_rn(mean, __fmul_rn(std_dev, x));
    if (round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
    out[i] = from_f32<TO>(v);
  }
}

// out: n elements of out_dtype; quantiles: 65537 float32 on the device; storage_dtype: the type the value is
// rounded to before it is widened to out_dtype (what a checkpoint of that storage type would hold).
LLMX_API int llmx_fill_normal(void* out, int out_dtype, long long n, unsigned long long stream,
                              const float* quantiles, float mean, float std_dev, int storage_dtype,
                              cudaStream_t cuda_stream) {
  if (n <= 0) return 0;
  if (!quantiles || (storage_dtype != LLMX_F32 && storage_dtype != LLMX_BF16)) return LLMX_REFUSED(1);
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
  if (out_dtype == LLMX_F32)
    fill_normal_kernel<float><<<blocks, threads, 0, cuda_stream>>>((float*)out, n, stream, quantiles, mean, std_dev,
                                                                    storage_dtype == LLMX_BF16);
  else if (out_dtype == LLMX_BF16)
    fill_normal_kernel<bf16><<<blocks, threads, 0, cuda_stream>>>((bf16*)out, n, stream, quantiles, mean, std_dev, 1);
  else
    return LLMX_REFUSED(2);
  return LLMX_LAUNCH_STATUS();
}
