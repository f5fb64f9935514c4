// Linear attention with a decay per head ("lightning attention"): a matrix state per head and request,
//     S_t = d_h * S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t,
// with q, k (heads x dk) and v (heads x dv) = SiLU of the projections.  The state is float32 and lives in
// the request's record [heads][dv][dk] (a value column's key channels side by side); everything here but the
// projections' storage is float32.
//
// `decay_scan`: one block per (entry, head, 16 value columns).  Every value column of S evolves on its own, so
// the scan is spread over them; a column's dk channels are held in registers by 8 lanes (channel = lane + 8 r).
// The entry's tokens are walked in order, 16 at a time through shared memory (SiLU applied on the way in); a
// token's arithmetic does not depend on where a step's portion began, so a position's result is the same bits
// however the tokens were cut into steps.  The only chain from token to token is one multiply-add a channel;
// the read-outs' lane reductions of different tokens are independent of each other.
//
// `linear_attn_out`: y = o / rms(o over all heads) * weight * sigmoid(gate), in the engine's dtype.
#include "common.cuh"

#define LA_COLS 16
#define LA_LANES 8
#define LA_THREADS (LA_COLS * LA_LANES)
#define LA_CHUNK 16

__device__ __forceinline__ float la_silu(float z) { return z / (1.0f + expf(-z)); }

// proj: T [tokens, stride]: q heads at q_off, k heads at k_off (dk each), v heads at v_off (dv each).
// state: float32 [slots][H][dv][dk]; o: float32 [tokens, H * dv].  R = ceil(dk / 8) rounded up to 4, 8, 16 or 32.
template <typename T, int R>
__global__ void __launch_bounds__(LA_THREADS)
decay_scan_kernel(const T* __restrict__ proj, long stride, int q_off, int k_off, int v_off,
                  const float* __restrict__ decay, float* __restrict__ state, long slot_stride, int num_slots,
                  const int* __restrict__ cu_q, const int* __restrict__ req_slot, float* __restrict__ o, int H, int dk,
                  int dv, int write_state, int* status) {
  extern __shared__ float smem[];
  const int dkp = R * LA_LANES;
  float* qs = smem;                           // [LA_CHUNK][dkp]
  float* ks = qs + LA_CHUNK * dkp;            // [LA_CHUNK][dkp]
  float* vs = ks + LA_CHUNK * dkp;            // [LA_CHUNK][LA_COLS]
  LL_PDL_TRIGGER();
  const int cg = blockIdx.x, h = blockIdx.y, e = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & (LA_LANES - 1), cl = tid / LA_LANES;
  const int col = cg * LA_COLS + cl;
  const float d = decay[h];
  LL_PDL_WAIT();
  const int t0 = cu_q[e], t1 = cu_q[e + 1];
  const int slot = req_slot[e];
  if (slot < 0 || slot >= num_slots) {       // a padding entry: defined output, nothing read
    if (slot >= num_slots && tid == 0) set_status(status, LL_ERR_SLOT_RANGE);
    if (lane == 0 && col < dv)
      for (int t = t0; t < t1; ++t) o[(size_t)t * H * dv + (size_t)h * dv + col] = 0.f;
    return;
  }
  float* srow = state + (size_t)slot * slot_stride + ((size_t)h * dv + (col < dv ? col : 0)) * dk;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int c = lane + LA_LANES * r;
    S[r] = (col < dv && c < dk) ? srow[c] : 0.f;
  }
  for (int base = t0; base < t1; base += LA_CHUNK) {
    const int n = min(LA_CHUNK, t1 - base);
    __syncthreads();
    for (int i = tid; i < n * dkp; i += LA_THREADS) {
      const int t = i / dkp, c = i - t * dkp;
      const T* row = proj + (size_t)(base + t) * stride;
      qs[i] = c < dk ? la_silu(to_f32<T>(row[q_off + h * dk + c])) : 0.f;
      ks[i] = c < dk ? la_silu(to_f32<T>(row[k_off + h * dk + c])) : 0.f;
    }
    for (int i = tid; i < n * LA_COLS; i += LA_THREADS) {
      const int t = i / LA_COLS, c = cg * LA_COLS + (i - t * LA_COLS);
      vs[i] = c < dv ? la_silu(to_f32<T>(proj[(size_t)(base + t) * stride + v_off + h * dv + c])) : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < n; ++t) {
      const float v = vs[t * LA_COLS + cl];
      const float* qt = qs + t * dkp + lane;
      const float* kt = ks + t * dkp + lane;
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        S[r] = fmaf(d, S[r], kt[LA_LANES * r] * v);
        acc = fmaf(S[r], qt[LA_LANES * r], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (lane == 0 && col < dv) o[(size_t)(base + t) * H * dv + (size_t)h * dv + col] = acc;
    }
  }
  if (write_state && col < dv) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int c = lane + LA_LANES * r;
      if (c < dk) srow[c] = S[r];
    }
  }
}

// y[t, :] = o[t, :] / sqrt(mean(o[t, :]^2) + eps) * weight * sigmoid(gate[t, :]); one block per token.
template <typename T>
__global__ void __launch_bounds__(256)
linear_attn_out_kernel(T* __restrict__ y, const float* __restrict__ o, const float* __restrict__ weight,
                       const T* __restrict__ gate, long gate_stride, float eps, int width) {
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const float* orow = o + (size_t)t * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(orow[i], orow[i], ss);
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  const T* g = gate + (size_t)t * gate_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float z = to_f32<T>(g[i]);
    y[(size_t)t * width + i] = from_f32<T>(orow[i] * inv * weight[i] / (1.0f + expf(-z)));
  }
}

extern "C" int ll_decay_scan(int dtype, const void* proj, long stride, int q_off, int k_off, int v_off,
                             const float* decay, float* state, long slot_stride, int num_slots, const int* cu_q,
                             const int* req_slot, float* o, int num_entries, int H, int dk, int dv, int write_state,
                             int* status, cudaStream_t stream) {
  if (num_entries <= 0) return 0;
  if (H <= 0 || dk <= 0 || dk > 256 || dv <= 0) return (int)cudaErrorInvalidValue;
  const int need = (dk + LA_LANES - 1) / LA_LANES;
  const int R = need <= 4 ? 4 : need <= 8 ? 8 : need <= 16 ? 16 : 32;
  const size_t smem = sizeof(float) * ((size_t)2 * LA_CHUNK * R * LA_LANES + LA_CHUNK * LA_COLS);
  dim3 grid((dv + LA_COLS - 1) / LA_COLS, H, num_entries);
#define LA_LAUNCH(RR)                                                                                              \
  ll_launch(decay_scan_kernel<T, RR>, grid, dim3(LA_THREADS), smem, stream, (const T*)proj, stride, q_off, k_off,  \
            v_off, decay, state, slot_stride, num_slots, cu_q, req_slot, o, H, dk, dv, write_state, status)
  LL_DISPATCH_DTYPE(dtype, {
    if (R == 4) LA_LAUNCH(4);
    else if (R == 8) LA_LAUNCH(8);
    else if (R == 16) LA_LAUNCH(16);
    else LA_LAUNCH(32);
  });
#undef LA_LAUNCH
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_linear_attn_out(int dtype, void* y, const float* o, const float* weight, const void* gate,
                                  long gate_stride, float eps, int num_tokens, int width, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  LL_DISPATCH_DTYPE(dtype, ll_launch(linear_attn_out_kernel<T>, dim3(num_tokens), dim3(256), 0, stream, (T*)y, o,
                                     weight, (const T*)gate, gate_stride, eps, width));
  return LL_LAUNCH_RESULT();
}
