// Two mixers side by side, joined: out = (rms(a + bias_a) * wa + rms(b) * wb) / 2, each RMS norm over the whole
// row (x / sqrt(mean(x^2) + eps), float32).  `bias_a` (float32, optional) is the first mixer's output bias, added
// here instead of in a pass of its own.
//
// One block per token; a thread keeps its pieces of both rows in registers between the sums of squares and the
// output (rows of up to 256 x PIECES x VEC numbers; longer rows are read a second time).  (A variant with one to
// eight warps a row, sums by shuffles and all loads asked for at once, was measured slower: 12.5 against 15.4 us for
// 2,048 rows of 1,536, but 9.3 against 3.8 us for 8 rows, and slower at 3,584 columns in both.)
#include "common.cuh"

#define NJ_THREADS 256
#define NJ_PIECES 4

// N float32 numbers from p + c (zeros if p is null); N a multiple of 4 goes in 16-byte pieces (c is a multiple of N then)
template <int N>
__device__ __forceinline__ void load_f32(float* dst, const float* __restrict__ p, int c) {
  if (p == nullptr) {
#pragma unroll
    for (int k = 0; k < N; ++k) dst[k] = 0.f;
  } else if (N % 4 == 0) {
#pragma unroll
    for (int k = 0; k < N; k += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + c + k);
      dst[k] = v.x; dst[k + 1] = v.y; dst[k + 2] = v.z; dst[k + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int k = 0; k < N; ++k) dst[k] = p[c + k];
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(NJ_THREADS)
rms_pair_mean_kernel(T* __restrict__ out, const T* __restrict__ a, long a_stride, const float* __restrict__ bias_a,
                     const float* __restrict__ wa, const T* __restrict__ b, long b_stride, const float* __restrict__ wb,
                     float eps, int width) {
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const T* ar = a + (size_t)t * a_stride;
  const T* br = b + (size_t)t * b_stride;
  const bool resident = width <= NJ_THREADS * NJ_PIECES * VEC;
  float xa[NJ_PIECES][VEC], xb[NJ_PIECES][VEC];
  float sa = 0.f, sb = 0.f;
  auto load = [&](int c, float* x, float* y) {
    T va[VEC], vb[VEC];
    if (VEC > 1) {
      *reinterpret_cast<uint4*>(va) = *reinterpret_cast<const uint4*>(ar + c);
      *reinterpret_cast<uint4*>(vb) = *reinterpret_cast<const uint4*>(br + c);
    } else {
      va[0] = ar[c];
      vb[0] = br[c];
    }
    float ba[VEC];
    load_f32<VEC>(ba, bias_a, c);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      x[k] = to_f32<T>(va[k]) + ba[k];
      y[k] = to_f32<T>(vb[k]);
    }
  };
  if (resident) {
#pragma unroll
    for (int p = 0; p < NJ_PIECES; ++p) {
      const int c = (threadIdx.x + p * NJ_THREADS) * VEC;
      if (c < width) {
        load(c, xa[p], xb[p]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          sa = fmaf(xa[p][k], xa[p][k], sa);
          sb = fmaf(xb[p][k], xb[p][k], sb);
        }
      }
    }
  } else {
    for (int c = threadIdx.x * VEC; c < width; c += NJ_THREADS * VEC) {
      load(c, xa[0], xb[0]);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        sa = fmaf(xa[0][k], xa[0][k], sa);
        sb = fmaf(xb[0][k], xb[0][k], sb);
      }
    }
  }
  {     // both sums over the block at once: one pair of barriers
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    sa = warp_sum(sa);
    sb = warp_sum(sb);
    if (lane == 0) {
      scratch[warp] = sa;
      scratch[8 + warp] = sb;
    }
    __syncthreads();
    sa = warp_sum(lane < NJ_THREADS / 32 ? scratch[lane] : 0.f);
    sb = warp_sum(lane < NJ_THREADS / 32 ? scratch[8 + lane] : 0.f);
  }
  const float ia = 1.0f / sqrtf(sa / (float)width + eps);
  const float ib = 1.0f / sqrtf(sb / (float)width + eps);
  auto store = [&](int c, const float* x, const float* y) {
    T vo[VEC];
    float fa[VEC], fb[VEC];
    load_f32<VEC>(fa, wa, c);
    load_f32<VEC>(fb, wb, c);
#pragma unroll
    for (int k = 0; k < VEC; ++k) vo[k] = from_f32<T>(0.5f * (x[k] * ia * fa[k] + y[k] * ib * fb[k]));
    if (VEC > 1) *reinterpret_cast<uint4*>(out + (size_t)t * width + c) = *reinterpret_cast<const uint4*>(vo);
    else out[(size_t)t * width + c] = vo[0];
  };
  if (resident) {
#pragma unroll
    for (int p = 0; p < NJ_PIECES; ++p) {
      const int c = (threadIdx.x + p * NJ_THREADS) * VEC;
      if (c < width) store(c, xa[p], xb[p]);
    }
  } else {
    for (int c = threadIdx.x * VEC; c < width; c += NJ_THREADS * VEC) {
      load(c, xa[0], xb[0]);
      store(c, xa[0], xb[0]);
    }
  }
}

extern "C" int ll_rms_pair_mean(int dtype, void* out, const void* a, long a_stride, const float* bias_a,
                                const float* wa, const void* b, long b_stride, const float* wb, float eps,
                                int num_tokens, int width, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  LL_DISPATCH_DTYPE(dtype, {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool wide = (width % VEC) == 0 && (a_stride % VEC) == 0 && (b_stride % VEC) == 0 &&
                      ((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
                      ((uintptr_t)bias_a % 16) == 0 && ((uintptr_t)wa % 16) == 0 && ((uintptr_t)wb % 16) == 0;
    if (wide)
      ll_launch(rms_pair_mean_kernel<T, VEC>, dim3(num_tokens), dim3(NJ_THREADS), 0, stream, (T*)out, (const T*)a,
                a_stride, bias_a, wa, (const T*)b, b_stride, wb, eps, width);
    else
      ll_launch(rms_pair_mean_kernel<T, 1>, dim3(num_tokens), dim3(NJ_THREADS), 0, stream, (T*)out, (const T*)a,
                a_stride, bias_a, wa, (const T*)b, b_stride, wb, eps, width);
  });
  return LL_LAUNCH_RESULT();
}
