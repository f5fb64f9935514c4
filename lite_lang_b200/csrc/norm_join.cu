// Two mixers side by side, joined: out = (rms(a + bias_a) * wa + rms(b) * wb) / 2, each RMS norm over the whole
// row (x / sqrt(mean(x^2) + eps), float32).  One block per token; the rows are read twice (the second time
// from L1/L2).  `bias_a` (float32, optional) is the first mixer's output bias, added here instead of in a
// pass of its own.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
rms_pair_mean_kernel(T* __restrict__ out, const T* __restrict__ a, long a_stride, const float* __restrict__ bias_a,
                     const float* __restrict__ wa, const T* __restrict__ b, long b_stride, const float* __restrict__ wb,
                     float eps, int width) {
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const T* ar = a + (size_t)t * a_stride;
  const T* br = b + (size_t)t * b_stride;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float x = to_f32<T>(ar[i]) + (bias_a ? bias_a[i] : 0.f);
    const float y = to_f32<T>(br[i]);
    sa = fmaf(x, x, sa);
    sb = fmaf(y, y, sb);
  }
  sa = block_sum(sa, scratch);
  sb = block_sum(sb, scratch);
  const float ia = 1.0f / sqrtf(sa / (float)width + eps);
  const float ib = 1.0f / sqrtf(sb / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float x = to_f32<T>(ar[i]) + (bias_a ? bias_a[i] : 0.f);
    const float y = to_f32<T>(br[i]);
    out[(size_t)t * width + i] = from_f32<T>(0.5f * (x * ia * wa[i] + y * ib * wb[i]));
  }
}

extern "C" int ll_rms_pair_mean(int dtype, void* out, const void* a, long a_stride, const float* bias_a,
                                const float* wa, const void* b, long b_stride, const float* wb, float eps,
                                int num_tokens, int width, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  LL_DISPATCH_DTYPE(dtype, ll_launch(rms_pair_mean_kernel<T>, dim3(num_tokens), dim3(256), 0, stream, (T*)out,
                                     (const T*)a, a_stride, bias_a, wa, (const T*)b, b_stride, wb, eps, width));
  return LL_LAUNCH_RESULT();
}
