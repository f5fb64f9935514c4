// A residual that is several streams wide (hyper-connections), with the norm that reads it.
//
// The residual of a token is S rows X[0..S-1] of `hidden` float32 numbers, laid out [tokens, S, hidden].
// A sublayer reads u = sum_s read[s] X[s] through a norm and writes its output y back as
//     X[t] <- sum_s mix[s, t] X[s] + write[t] * y          (all t from the old rows)
// The write of one sublayer and the read of the next are one pass over the rows here, as the residual sum and
// the norm are one pass for a single stream: `stream_tanh_norm` applies a pending write (if one is given),
// stores the new rows, and returns norm(sum_s read[s] X_new[s]) in the engine's dtype.  The norm is the
// "dynamic tanh" tanh(alpha * u) * w + b, which needs no statistics of the row, so the whole pass is
// elementwise over the columns.  Everything is float32 but y and the result.
#include "common.cuh"

#define ST_MAX 8   // most streams

// out [tokens, S, hidden] float32: every stream starts as the token's table row.
template <typename T>
__global__ void embed_streams_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                     int hidden, int vocab, int S, int* status) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = (id >= 0 && id < vocab);
  if (!ok && threadIdx.x == 0) set_status(status, LL_ERR_TOKEN_RANGE);
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  float* dst = out + (size_t)t * S * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = ok ? to_f32<T>(src[i]) : 0.f;
    for (int s = 0; s < S; ++s) dst[(size_t)s * hidden + i] = v;
  }
}

// Blocks (i, j): output row i (token r = rows ? rows[i] : i), the j-th 128 x VEC columns.  A thread takes VEC
// neighbouring columns.
// y: T [tokens, hidden] or null; y_parts: float32 [parts, tokens, hidden] partial sums of a split product, or null;
// mix [S, S] (from, to), write [S], read [S] (null: all ones), alpha [1], w, b [hidden] (b null: none): float32.
template <typename T, int VEC, int SM>      // SM: the most streams this instance takes (its register arrays)
__global__ void __launch_bounds__(128)
stream_tanh_norm_kernel(T* __restrict__ out, float* __restrict__ X, const T* __restrict__ y,
                        const float* __restrict__ y_parts, int parts, long part_stride, const float* __restrict__ mix,
                        const float* __restrict__ write, const float* __restrict__ read,
                        const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b,
                        const int* __restrict__ rows, int write_back, int S, int hidden) {
  __shared__ float s_mix[ST_MAX * ST_MAX], s_write[ST_MAX], s_read[ST_MAX];
  LL_PDL_TRIGGER();
  const bool pending = (mix != nullptr);
  if (threadIdx.x < S * S && pending) s_mix[threadIdx.x] = mix[threadIdx.x];     // (weights: not a predecessor's output)
  if (threadIdx.x < S) {
    s_write[threadIdx.x] = pending ? write[threadIdx.x] : 0.f;
    s_read[threadIdx.x] = read ? read[threadIdx.x] : 1.f;
  }
  const float a = alpha[0];
  LL_PDL_WAIT();
  __syncthreads();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* xr = X + (size_t)r * S * hidden;
  // (elementwise over the columns: a row's columns are shared out over the blocks along y)
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; c < hidden; c += gridDim.y * blockDim.x * VEC) {
    float xs[SM][VEC];
#pragma unroll
    for (int s = 0; s < SM; ++s) {
      if (s < S) {
        if (VEC == 4) {
          const float4 v = *reinterpret_cast<const float4*>(xr + (size_t)s * hidden + c);
          xs[s][0] = v.x; xs[s][1 % VEC] = v.y; xs[s][2 % VEC] = v.z; xs[s][3 % VEC] = v.w;
        } else {
          xs[s][0] = xr[(size_t)s * hidden + c];
        }
      }
    }
    if (pending) {
      float yv[VEC];
      if (y) {       // (VEC numbers of y in one access: the launcher checked its alignment)
        T raw[VEC];
        if (VEC == 4 && sizeof(T) == 2) *reinterpret_cast<uint2*>(raw) = *reinterpret_cast<const uint2*>(y + (size_t)r * hidden + c);
        else if (VEC == 4) *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(y + (size_t)r * hidden + c);
        else raw[0] = y[(size_t)r * hidden + c];
#pragma unroll
        for (int k = 0; k < VEC; ++k) yv[k] = to_f32<T>(raw[k]);
      } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) yv[k] = 0.f;
      }
      for (int p = 0; p < parts; ++p)
#pragma unroll
        for (int k = 0; k < VEC; ++k) yv[k] += y_parts[(size_t)p * part_stride + (size_t)r * hidden + c + k];
      float nx[SM][VEC];
#pragma unroll
      for (int t = 0; t < SM; ++t) {
        if (t < S) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            float v = 0.f;
#pragma unroll
            for (int s = 0; s < SM; ++s)
              if (s < S) v = fmaf(s_mix[s * S + t], xs[s][k], v);
            nx[t][k] = fmaf(s_write[t], yv[k], v);
          }
        }
      }
#pragma unroll
      for (int t = 0; t < SM; ++t) {
        if (t < S) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) xs[t][k] = nx[t][k];
          if (write_back) {
            if (VEC == 4)
              *reinterpret_cast<float4*>(xr + (size_t)t * hidden + c) =
                  make_float4(nx[t][0], nx[t][1 % VEC], nx[t][2 % VEC], nx[t][3 % VEC]);
            else
              xr[(size_t)t * hidden + c] = nx[t][0];
          }
        }
      }
    }
    T res[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < SM; ++s)
        if (s < S) u = fmaf(s_read[s], xs[s][k], u);
      res[k] = from_f32<T>(tanhf(a * u) * w[c + k] + (b ? b[c + k] : 0.f));
    }
    if (VEC == 4 && sizeof(T) == 2) *reinterpret_cast<uint2*>(out + (size_t)i * hidden + c) = *reinterpret_cast<const uint2*>(res);
    else if (VEC == 4) *reinterpret_cast<uint4*>(out + (size_t)i * hidden + c) = *reinterpret_cast<const uint4*>(res);
    else out[(size_t)i * hidden + c] = res[0];
  }
}

// total [tokens, hidden] float32 = sum_s X[s] (after a pending write, which is not stored): what a reader
// outside the layers (a probe of the residual) sees.
__global__ void stream_sum_kernel(float* __restrict__ total, const float* __restrict__ X, int S, int hidden) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int r = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < S; ++s) v += X[((size_t)r * S + s) * hidden + c];
    total[(size_t)r * hidden + c] = v;
  }
}

extern "C" int ll_embed_streams(int dtype, float* out, const void* table, const int* ids, int num_tokens, int hidden,
                                int vocab, int S, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (S <= 0 || S > ST_MAX) return (int)cudaErrorInvalidValue;
  LL_DISPATCH_DTYPE(dtype, ll_launch(embed_streams_kernel<T>, dim3(num_tokens), dim3(128), 0, stream, out,
                                     (const T*)table, ids, hidden, vocab, S, status));
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_stream_tanh_norm(int dtype, void* out, float* X, const void* y, const float* y_parts, int parts,
                                   long part_stride, const float* mix, const float* write, const float* read,
                                   const float* alpha, const float* w, const float* b, const int* rows, int write_back,
                                   int S, int hidden, int n_out, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (S <= 0 || S > ST_MAX || hidden <= 0) return (int)cudaErrorInvalidValue;
  const bool wide = (hidden % 4) == 0 && ((uintptr_t)X % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
                    ((uintptr_t)y % 16) == 0;
#define ST_LAUNCH(VV, MM)                                                                                            \
  ll_launch(stream_tanh_norm_kernel<T, VV, MM>, dim3(n_out, (hidden / VV + 127) / 128), dim3(128), 0, stream, (T*)out, X, (const T*)y, y_parts, \
            parts, part_stride, mix, write, read, alpha, w, b, rows, write_back, S, hidden)
  LL_DISPATCH_DTYPE(dtype, {
    if (wide) {
      if (S <= 2) ST_LAUNCH(4, 2);
      else if (S <= 4) ST_LAUNCH(4, 4);
      else ST_LAUNCH(4, ST_MAX);
    } else {
      if (S <= 2) ST_LAUNCH(1, 2);
      else if (S <= 4) ST_LAUNCH(1, 4);
      else ST_LAUNCH(1, ST_MAX);
    }
  });
#undef ST_LAUNCH
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_stream_sum(float* total, const float* X, int num_tokens, int S, int hidden, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  ll_launch(stream_sum_kernel, dim3(num_tokens), dim3(128), 0, stream, total, X, S, hidden);
  return LL_LAUNCH_RESULT();
}
