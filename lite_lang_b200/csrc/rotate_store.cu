// Bias, rotary position encoding with angles made in the kernel, and the write into the paged cache, for a
// q|k|v projection whose value heads may be wider or narrower than its key heads.
//
// Row t of `qkv` holds nh query heads and nkv key heads of hd values, then nkv value heads of vd values.
//   * bias (float32, optional) is added in float32;
//   * the first rot_dim values of every q and k head are rotated by angle = float(position) * freq[i], with
//     freq float32 [rot_dim / 2] (made on the host in float64 and rounded once; any scaling of the positions is
//     already inside it).  Pair i is (2i, 2i+1) when `interleaved`, (i, i + rot_dim/2) otherwise:
//     (u, v) -> (u cos a - v sin a, v cos a + u sin a).  cosf and sinf are the accurate ones (no fast math);
//   * q (and k, v) are written back in place, rounded once; k and v also go to the token's cache slot.
// No table of positions, so no position is out of range.
//
// With interleaved pairs and even sizes a pair is one access (two neighbouring values of the storage type), and
// so are two neighbouring values of a head's unrotated tail and of v.
//
// Cache plane: K [num_pages, nkv, page_size, hd], V [num_pages, nkv, page_size, vd].
#include "common.cuh"

#define RS_MAX_PAIRS 128      // (the pairs kernel takes heads of up to 256 rotated channels)

template <typename T> struct Pair;
template <> struct Pair<float> { typedef float2 type; };
template <> struct Pair<bf16> { typedef __nv_bfloat162 type; };
template <typename T> __device__ __forceinline__ float2 pair_to_f32(typename Pair<T>::type v);
template <> __device__ __forceinline__ float2 pair_to_f32<float>(float2 v) { return v; }
template <> __device__ __forceinline__ float2 pair_to_f32<bf16>(__nv_bfloat162 v) { return __bfloat1622float2(v); }
template <typename T> __device__ __forceinline__ typename Pair<T>::type pair_from_f32(float x, float y);
template <> __device__ __forceinline__ float2 pair_from_f32<float>(float x, float y) { return make_float2(x, y); }
template <> __device__ __forceinline__ __nv_bfloat162 pair_from_f32<bf16>(float x, float y) {
  return __floats2bfloat162_rn(x, y);
}

// interleaved pairs; hd, vd, rot_dim, the row stride and all offsets even, so every pair of neighbours is aligned
template <typename T>
__global__ void __launch_bounds__(256)
bias_rotate_store_pairs_kernel(T* __restrict__ qkv, long qkv_stride, const float* __restrict__ bias,
                               const int* __restrict__ positions, const float* __restrict__ freq, int rot_dim, int nh,
                               int nkv, int hd, int vd, const int* __restrict__ slot_map, T* __restrict__ k_cache,
                               T* __restrict__ v_cache, int page_size, long num_slots, int* status) {
  typedef typename Pair<T>::type P2;
  __shared__ float cs[RS_MAX_PAIRS], sn[RS_MAX_PAIRS];      // the token's cos and sin, made once for all heads
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  T* row = qkv + (size_t)t * qkv_stride;
  const float pos = (float)(positions ? positions[t] : 0);
  for (int i = threadIdx.x; i < (rot_dim >> 1); i += blockDim.x) {
    const float a = pos * freq[i];
    cs[i] = cosf(a);
    sn[i] = sinf(a);
  }
  __syncthreads();
  long slot = slot_map ? (long)slot_map[t] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) set_status(status, LL_ERR_SLOT_RANGE);
    slot = -1;
  }
  const long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  const int half = rot_dim >> 1, hp = hd >> 1, vp = vd >> 1;
  const int qk_pairs = (nh + nkv) * hp;
  for (int w = threadIdx.x; w < qk_pairs + nkv * vp; w += blockDim.x) {
    if (w < qk_pairs) {
      const int h = w / hp, i = w - h * hp;
      const size_t at = (size_t)h * hd + 2 * i;
      float2 x = pair_to_f32<T>(*reinterpret_cast<const P2*>(row + at));
      if (bias) {
        const float2 b2 = *reinterpret_cast<const float2*>(bias + at);
        x.x += b2.x;
        x.y += b2.y;
      }
      if (i < half) {
        const float c = cs[i], s = sn[i];
        x = make_float2(x.x * c - x.y * s, x.y * c + x.x * s);
      }
      const P2 r = pair_from_f32<T>(x.x, x.y);
      *reinterpret_cast<P2*>(row + at) = r;
      if (h >= nh && slot >= 0)
        *reinterpret_cast<P2*>(k_cache + (((size_t)page * nkv + (h - nh)) * page_size + off) * hd + 2 * i) = r;
    } else {
      const int u = w - qk_pairs;
      const int h = u / vp, j = 2 * (u - h * vp);
      const size_t at = (size_t)(nh + nkv) * hd + (size_t)h * vd + j;
      float2 x = pair_to_f32<T>(*reinterpret_cast<const P2*>(row + at));
      if (bias) {
        const float2 b2 = *reinterpret_cast<const float2*>(bias + at);
        x.x += b2.x;
        x.y += b2.y;
      }
      const P2 r = pair_from_f32<T>(x.x, x.y);
      if (bias) *reinterpret_cast<P2*>(row + at) = r;
      if (slot >= 0) *reinterpret_cast<P2*>(v_cache + (((size_t)page * nkv + h) * page_size + off) * vd + j) = r;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
bias_rotate_store_kernel(T* __restrict__ qkv, long qkv_stride, const float* __restrict__ bias,
                         const int* __restrict__ positions, const float* __restrict__ freq, int rot_dim,
                         int interleaved, int nh, int nkv, int hd, int vd, const int* __restrict__ slot_map,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, long num_slots, int* status) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  T* row = qkv + (size_t)t * qkv_stride;
  const float pos = (float)(positions ? positions[t] : 0);
  long slot = slot_map ? (long)slot_map[t] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) set_status(status, LL_ERR_SLOT_RANGE);
    slot = -1;
  }
  const long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  const int half = rot_dim >> 1;
  const int per_head = hd - half;      // work items of a head: `half` pairs + (hd - rot_dim) singles
  for (int w = threadIdx.x; w < (nh + nkv) * per_head; w += blockDim.x) {
    const int h = w / per_head;
    const int i = w - h * per_head;
    T* head = row + (size_t)h * hd;
    const float* b = bias ? bias + (size_t)h * hd : nullptr;
    T* dst = nullptr;
    if (h >= nh && slot >= 0) dst = k_cache + (((size_t)page * nkv + (h - nh)) * page_size + off) * hd;
    if (i < half) {
      const int j0 = interleaved ? 2 * i : i;
      const int j1 = interleaved ? 2 * i + 1 : i + half;
      float x0 = to_f32<T>(head[j0]);
      float x1 = to_f32<T>(head[j1]);
      if (b) {
        x0 += b[j0];
        x1 += b[j1];
      }
      const float a = pos * freq[i];
      const float c = cosf(a), s = sinf(a);
      const float o0 = x0 * c - x1 * s;
      const float o1 = x1 * c + x0 * s;
      head[j0] = from_f32<T>(o0);
      head[j1] = from_f32<T>(o1);
      if (dst) {
        dst[j0] = from_f32<T>(o0);
        dst[j1] = from_f32<T>(o1);
      }
    } else {
      const int j = rot_dim + (i - half);
      float x = to_f32<T>(head[j]);
      if (b) x += b[j];
      head[j] = from_f32<T>(x);
      if (dst) dst[j] = from_f32<T>(x);
    }
  }
  const size_t v0 = (size_t)(nh + nkv) * hd;
  for (int w = threadIdx.x; w < nkv * vd; w += blockDim.x) {
    const int h = w / vd;
    const int j = w - h * vd;
    float x = to_f32<T>(row[v0 + w]);
    if (bias) {
      x += bias[v0 + w];
      row[v0 + w] = from_f32<T>(x);
    }
    if (slot >= 0) v_cache[(((size_t)page * nkv + h) * page_size + off) * vd + j] = from_f32<T>(x);
  }
}

extern "C" int ll_bias_rotate_store(int dtype, void* qkv, long qkv_stride, const float* bias, const int* positions,
                                    const float* freq, int rot_dim, int interleaved, int nh, int nkv, int hd, int vd,
                                    const int* slot_map, void* k_cache, void* v_cache, int page_size, long num_slots,
                                    int num_tokens, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || hd <= 0 || vd <= 0) return (int)cudaErrorInvalidValue;
  const int esz = dtype == LL_DTYPE_F32 ? 4 : 2;
  const bool pairs = (interleaved || rot_dim == 0) && rot_dim <= 2 * RS_MAX_PAIRS && (hd % 2) == 0 && (vd % 2) == 0 && (qkv_stride % 2) == 0 &&
                     ((uintptr_t)qkv % (2 * esz)) == 0 && ((uintptr_t)bias % 8) == 0 &&
                     ((uintptr_t)k_cache % (2 * esz)) == 0 && ((uintptr_t)v_cache % (2 * esz)) == 0;
  LL_DISPATCH_DTYPE(dtype, {
    if (pairs)
      ll_launch(bias_rotate_store_pairs_kernel<T>, dim3(num_tokens), dim3(256), 0, stream, (T*)qkv, qkv_stride, bias,
                positions, freq, rot_dim, nh, nkv, hd, vd, slot_map, (T*)k_cache, (T*)v_cache, page_size, num_slots,
                status);
    else
      ll_launch(bias_rotate_store_kernel<T>, dim3(num_tokens), dim3(256), 0, stream, (T*)qkv, qkv_stride, bias,
                positions, freq, rot_dim, interleaved, nh, nkv, hd, vd, slot_map, (T*)k_cache, (T*)v_cache, page_size,
                num_slots, status);
  });
  return LL_LAUNCH_RESULT();
}
