// Gated delta rule: a linear recurrence with a matrix state per head.
//
// Per request and head the state S [dk, dv] (float32) evolves token by token:
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with q, k unit vectors (q also times dk^-1/2), beta in (0, 1) and a decay g in (0, 1] that is
// one number per head or one per head and key channel.  q, k and v come out of a short causal
// convolution over time (per channel, `taps` taps, the last one the current token's) and SiLU.
// A request's record in the state pool is float32 [heads][dv][dk] for S (a value column's key channels side by
// side, as the lanes of the scan hold them) followed by
// [(taps - 1), channels] for the last taps - 1 inputs of the convolutions (oldest first;
// channels = q | k | v), so that a request can go on in a later step from where it stopped.
//
// Four kernels, all reading the step's device arrays only (so that a step of single tokens can
// be captured and replayed):
//   delta_prepare      per token: convolution + SiLU, unit vectors, beta, decay -> float32 buffers
//   delta_conv_update  per entry: the new last taps - 1 inputs of the record
//   delta_recurrence   per (entry, head, 16 value columns): the scan over the entry's tokens
//   delta_out          per (token, head): o / rms(o) * weight * gate -> storage type
// Every value column of S evolves on its own (S^T k and S^T q are per column), so the scan is
// spread over value columns as well as over requests and heads; the order of every sum depends
// on the sizes only, never on how tokens were cut into steps or batched.
#include "common.cuh"

__device__ __forceinline__ float dr_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float dr_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float dr_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct DeltaShape {
  int H, Hk, dk, dv, taps;
  int per_channel;   // decay: 0 one per head, 1 one per head and key channel
};

// proj: the step's projections, row t at proj + t * proj_stride, with q at column q_off (Hk*dk wide), k at k_off
// (Hk*dk), v at v_off (H*dv), b at b_off (H).  a_in: the decay's input, [tokens, H] or [tokens, H*dk].
template <typename T>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const T* __restrict__ proj, long proj_stride, int q_off, int k_off, int v_off, int b_off,
                     const T* __restrict__ a_in, long a_stride, const float* __restrict__ conv_q,
                     const float* __restrict__ conv_k, const float* __restrict__ conv_v,
                     const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                     const float* __restrict__ state, long state_stride, long tail_off,
                     const int* __restrict__ token_req, const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                     const int* __restrict__ req_slot, const int* __restrict__ positions, float* __restrict__ qn,
                     float* __restrict__ kn, float* __restrict__ vc, float* __restrict__ beta, float* __restrict__ g,
                     DeltaShape s) {
  extern __shared__ float y[];   // [Cq + Ck + Cv] convolution outputs after SiLU
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const int e = token_req[t];
  const int slot = e >= 0 ? req_slot[e] : -1;
  if (slot < 0) return;   // padding entry: the scan writes its (zero) output
  const int Cq = s.Hk * s.dk, Cv = s.H * s.dv, C = 2 * Cq + Cv, K = s.taps;
  const int first = cu_q[e], ctx = ctx_len[e], p = positions[t];
  const float* tail = state + (size_t)slot * state_stride + tail_off;
  const int tid = threadIdx.x;
  for (int c = tid; c < C; c += blockDim.x) {
    const float* w;
    int col;
    if (c < Cq) {
      w = conv_q + (size_t)c * K;
      col = q_off + c;
    } else if (c < 2 * Cq) {
      w = conv_k + (size_t)(c - Cq) * K;
      col = k_off + c - Cq;
    } else {
      w = conv_v + (size_t)(c - 2 * Cq) * K;
      col = v_off + c - 2 * Cq;
    }
    float acc = 0.f;
    for (int j = K - 1; j >= 0; --j) {   // oldest input first
      float x = 0.f;
      if (t - j >= first) {
        x = to_f32<T>(proj[(size_t)(t - j) * proj_stride + col]);
      } else if (p - j >= 0) {
        x = tail[(size_t)(p - j - ctx + K - 1) * C + c];   // an input of an earlier step
      }
      acc = fmaf(w[K - 1 - j], x, acc);
    }
    y[c] = dr_silu(acc);
  }
  __syncthreads();
  const int lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  for (int hh = warp; hh < 2 * s.Hk; hh += nwarps) {   // unit vectors: q heads, then k heads
    const float* src = y + (size_t)hh * s.dk;
    float ss = 0.f;
    for (int i = lane; i < s.dk; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss + 1e-6f);
    const bool is_q = hh < s.Hk;
    if (is_q) inv *= 1.0f / sqrtf((float)s.dk);
    float* dst = (is_q ? qn + (size_t)t * Cq : kn + (size_t)t * Cq - Cq) + (size_t)hh * s.dk;
    for (int i = lane; i < s.dk; i += 32) dst[i] = src[i] * inv;
  }
  for (int i = tid; i < Cv; i += blockDim.x) vc[(size_t)t * Cv + i] = y[2 * Cq + i];
  for (int h = tid; h < s.H; h += blockDim.x)
    beta[(size_t)t * s.H + h] = dr_sigmoid(to_f32<T>(proj[(size_t)t * proj_stride + b_off + h]));
  const int ng = s.per_channel ? s.H * s.dk : s.H;
  for (int i = tid; i < ng; i += blockDim.x) {
    const int h = s.per_channel ? i / s.dk : i;
    const float a = to_f32<T>(a_in[(size_t)t * a_stride + i]) + dt_bias[i];
    g[(size_t)t * ng + i] = expf(-expf(A_log[h]) * dr_softplus(a));
  }
}

// The record's last taps - 1 inputs after the step: inputs of this step where it brought enough tokens,
// else what the record held, moved up.  A thread owns a channel and goes from the oldest place to the
// newest, reading only places above the one it writes.
template <typename T>
__global__ void delta_conv_update_kernel(const T* __restrict__ proj, long proj_stride, int q_off, int k_off, int v_off,
                                         float* __restrict__ state, long state_stride, long tail_off,
                                         const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                                         const int* __restrict__ req_slot, DeltaShape s) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int e = blockIdx.x;
  const int slot = req_slot[e];
  if (slot < 0) return;
  const int Cq = s.Hk * s.dk, Cv = s.H * s.dv, C = 2 * Cq + Cv, K = s.taps;
  const int first = cu_q[e], L = cu_q[e + 1] - first, ctx = ctx_len[e];
  float* tail = state + (size_t)slot * state_stride + tail_off;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    const int col = c < Cq ? q_off + c : c < 2 * Cq ? k_off + c - Cq : v_off + c - 2 * Cq;
    for (int i = 0; i < K - 1; ++i) {
      const int pos = ctx + L - (K - 1) + i;   // the position whose input place i holds afterwards
      float x = 0.f;
      if (pos >= ctx) x = to_f32<T>(proj[(size_t)(first + pos - ctx) * proj_stride + col]);
      else if (pos >= 0) x = tail[(size_t)(i + L) * C + c];
      tail[(size_t)i * C + c] = x;
    }
  }
}

// The scan.  What bounds it is the chain of dependent operations from one token to the next of a value column, so
// a column is spread over as many lanes as leave each lane DR_NR = 4 key channels (8 for heads of more than 128
// channels): two short multiply-add chains and log2(LANES) shuffle steps a sum, all columns of all heads resident
// at once, and enough warps a scheduler to fill the gaps that one warp's dependent instructions leave (a capture
// of the 8-channel version showed 0.27 instructions issued a cycle and scheduler with 1.3 warps each).  A block of 128 threads owns 128 / LANES value columns of one (entry, head); lane l holds
// channels l, l + LANES, ....  The tokens' q, k, decay, v and beta come through shared memory in chunks of DR_CH
// tokens, copied asynchronously (cp.async) a chunk ahead, so that the scan waits for memory once a chunk and meets
// no barrier between the tokens of a chunk; rows are padded with zeros to LANES * DR_NR channels so that the inner
// loops carry no bounds checks.  Sums run in two interleaved chains and then over the lanes, in a fixed order.
// The read-out is taken from the state before the token's write plus the write's own share (see the loop), which
// is the same number as reading the state after the write.
#define DR_THREADS 128
#define DR_CH 16
__device__ __forceinline__ void dr_copy4(float* dst_smem, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_copy16(float* dst_smem, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
template <int DR_LANES, int DR_NR>
__global__ void __launch_bounds__(DR_THREADS)
delta_recurrence_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vc,
                        const float* __restrict__ beta, const float* __restrict__ g, float* __restrict__ state,
                        long state_stride, const int* __restrict__ cu_q, const int* __restrict__ req_slot,
                        float* __restrict__ o, DeltaShape s) {
  extern __shared__ float sm[];   // two buffers of [q | k | decay][DR_CH][dkp], v [DR_CH][DR_COLS], beta, head decay [DR_CH]
  constexpr int DR_COLS = DR_THREADS / DR_LANES;
  constexpr int dkp = DR_LANES * DR_NR;
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int e = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, l = tid % DR_LANES, cl = tid / DR_LANES;
  const int col0 = blockIdx.z * DR_COLS, col = col0 + cl;
  const bool live_col = col < s.dv;
  const int first = cu_q[e], last = cu_q[e + 1];
  const int slot = req_slot[e];
  const int Cq = s.Hk * s.dk, Cv = s.H * s.dv, dk = s.dk;
  if (slot < 0) {
    if (live_col && l == 0)
      for (int t = first; t < last; ++t) o[(size_t)t * Cv + (size_t)h * s.dv + col] = 0.f;
    return;
  }
  const int hk = h / (s.H / s.Hk);
  const int ng = s.per_channel ? s.H * dk : s.H;
  const bool pc = s.per_channel != 0;
  constexpr int buf_floats = DR_CH * (3 * dkp + DR_COLS + 2);
  const bool wide = (dk % 4) == 0 && (Cq % 4) == 0 && (ng % 4 == 0 || !pc) &&
                    (((uintptr_t)qn | (uintptr_t)kn | (uintptr_t)g) % 16) == 0;
  float* S_ptr = state + (size_t)slot * state_stride + (size_t)h * dk * s.dv;
  float S[DR_NR];
#pragma unroll
  for (int i = 0; i < DR_NR; ++i) {
    const int c = l + DR_LANES * i;
    S[i] = (live_col && c < dk) ? S_ptr[(size_t)col * dk + c] : 0.f;
  }
  // the padding channels dk .. dkp - 1 of every row: zeros, written once (the copies never touch them)
  for (int idx = tid; idx < 2 * 3 * DR_CH * (dkp - dk); idx += DR_THREADS) {
    const int row = idx / (dkp - dk), c = dk + idx % (dkp - dk);
    const int buf = row / (3 * DR_CH), rr = row % (3 * DR_CH);
    sm[(size_t)buf * buf_floats + rr * dkp + c] = 0.f;
  }
  auto load_chunk = [&](int t0, int buf) {
    float* b = sm + (size_t)buf * buf_floats;
    const int nt = min(DR_CH, last - t0);
    for (int i = 0; i < nt; ++i) {
      const float* qs = qn + (size_t)(t0 + i) * Cq + (size_t)hk * dk;
      const float* ks = kn + (size_t)(t0 + i) * Cq + (size_t)hk * dk;
      const float* gs = g + (size_t)(t0 + i) * ng + (size_t)h * dk;
      if (wide) {     // rows of a multiple of four channels at 16-byte addresses: four numbers a copy
        for (int c = tid * 4; c < dk; c += DR_THREADS * 4) {
          dr_copy16(b + i * dkp + c, qs + c);
          dr_copy16(b + (DR_CH + i) * dkp + c, ks + c);
          if (pc) dr_copy16(b + (2 * DR_CH + i) * dkp + c, gs + c);
        }
      } else {
        for (int c = tid; c < dk; c += DR_THREADS) {
          dr_copy4(b + i * dkp + c, qs + c);
          dr_copy4(b + (DR_CH + i) * dkp + c, ks + c);
          if (pc) dr_copy4(b + (2 * DR_CH + i) * dkp + c, gs + c);
        }
      }
    }
    float* bv = b + 3 * DR_CH * dkp;
    for (int idx = tid; idx < nt * DR_COLS; idx += DR_THREADS) {
      const int i = idx / DR_COLS, cc = idx % DR_COLS;
      if (col0 + cc < s.dv) dr_copy4(bv + idx, vc + (size_t)(t0 + i) * Cv + (size_t)h * s.dv + col0 + cc);
      else bv[idx] = 0.f;
    }
    if (tid < nt) {
      dr_copy4(bv + DR_CH * DR_COLS + tid, beta + (size_t)(t0 + tid) * s.H + h);
      if (!pc) dr_copy4(bv + DR_CH * DR_COLS + DR_CH + tid, g + (size_t)(t0 + tid) * ng + h);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (first < last) load_chunk(first, 0);
  for (int t0 = first; t0 < last; t0 += DR_CH) {
    const int buf = ((t0 - first) / DR_CH) & 1;
    const bool more = t0 + DR_CH < last;
    if (more) {
      load_chunk(t0 + DR_CH, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* b = sm + (size_t)buf * buf_floats;
    const float* bv = b + 3 * DR_CH * dkp;
    const int nt = min(DR_CH, last - t0);
    for (int i = 0; i < nt; ++i) {
      const float* sq = b + i * dkp + l;
      const float* sk = b + (DR_CH + i) * dkp + l;
      const float* sg = b + (2 * DR_CH + i) * dkp + l;
      const float v = bv[i * DR_COLS + cl];
      const float bt = bv[DR_CH * DR_COLS + i];
      const float gh = pc ? 1.f : bv[DR_CH * DR_COLS + DR_CH + i];
      // Both sums of a token read the state as the token before left it: with S' = diag(g) S + k u^T,
      //   S^T (g . k) is what u needs, and o = S'^T q = S^T (g . q) + u (k . q),
      // so the two reductions over the lanes (and the one of k . q, which does not touch the state) run side
      // by side, and the chain from token to token is one reduction, not two.
      float kr[DR_NR], dec[DR_NR];
      float d0 = 0.f, d1 = 0.f, o0 = 0.f, o1 = 0.f, kq = 0.f;
#pragma unroll
      for (int j = 0; j < DR_NR; ++j) {
        kr[j] = sk[DR_LANES * j];
        dec[j] = pc ? sg[DR_LANES * j] : gh;
        const float qv = sq[DR_LANES * j];
        const float gk = dec[j] * kr[j], gq = dec[j] * qv;
        kq = fmaf(kr[j], qv, kq);
        if (j & 1) {
          d1 = fmaf(S[j], gk, d1);
          o1 = fmaf(S[j], gq, o1);
        } else {
          d0 = fmaf(S[j], gk, d0);
          o0 = fmaf(S[j], gq, o0);
        }
      }
      float dot = d0 + d1, oq = o0 + o1;
#pragma unroll
      for (int x = 1; x < DR_LANES; x <<= 1) {
        dot += __shfl_xor_sync(0xffffffffu, dot, x);
        oq += __shfl_xor_sync(0xffffffffu, oq, x);
        kq += __shfl_xor_sync(0xffffffffu, kq, x);
      }
      const float u = bt * (v - dot);
      oq = fmaf(u, kq, oq);
#pragma unroll
      for (int j = 0; j < DR_NR; ++j) S[j] = fmaf(dec[j], S[j], kr[j] * u);
      if (live_col && l == 0) o[(size_t)(t0 + i) * Cv + (size_t)h * s.dv + col] = oq;
    }
    __syncthreads();   // everyone is done with this buffer before the chunk after the next is copied into it
  }
#pragma unroll
  for (int i = 0; i < DR_NR; ++i) {
    const int c = l + DR_LANES * i;
    if (live_col && c < dk) S_ptr[(size_t)col * dk + c] = S[i];
  }
}

// out[t, h*dv + j] = o / sqrt(mean_j(o^2) + eps) * w[j] * act(gate[t, h*dv + j]); act: 0 SiLU, 1 sigmoid.
template <typename T>
__global__ void delta_out_kernel(T* __restrict__ out, const float* __restrict__ o, const float* __restrict__ w,
                                 const T* __restrict__ gate, long gate_stride, float eps, int num_pairs, int H, int dv,
                                 int gate_act) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= num_pairs) return;
  const int lane = threadIdx.x & 31;
  const int t = pair / H, h = pair % H;
  const float* src = o + (size_t)pair * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(src[j], src[j], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  const T* gt = gate + (size_t)t * gate_stride + (size_t)h * dv;
  T* dst = out + (size_t)pair * dv;
  for (int j = lane; j < dv; j += 32) {
    const float z = to_f32<T>(gt[j]);
    const float a = gate_act == 0 ? dr_silu(z) : dr_sigmoid(z);
    dst[j] = from_f32<T>(src[j] * inv * w[j] * a);
  }
}

extern "C" int ll_delta_prepare(int dtype, const void* proj, long proj_stride, int q_off, int k_off, int v_off,
                                int b_off, const void* a_in, long a_stride, const float* conv_q, const float* conv_k,
                                const float* conv_v, const float* A_log, const float* dt_bias, float* state,
                                long state_stride, long tail_off, const int* token_req, const int* cu_q,
                                const int* ctx_len, const int* req_slot, const int* positions, float* qn, float* kn,
                                float* vc, float* beta, float* g, int num_tokens, int num_entries, int H, int Hk, int dk,
                                int dv, int taps, int per_channel, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || Hk <= 0 || H % Hk || dk <= 0 || dv <= 0 || taps < 1) return (int)cudaErrorInvalidValue;
  DeltaShape s{H, Hk, dk, dv, taps, per_channel};
  const int C = 2 * Hk * dk + H * dv;
  const size_t smem = sizeof(float) * (size_t)C;
  LL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(delta_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(delta_prepare_kernel<T>, dim3(num_tokens), dim3(256), smem, stream, (const T*)proj, proj_stride, q_off,
              k_off, v_off, b_off, (const T*)a_in, a_stride, conv_q, conv_k, conv_v, A_log, dt_bias,
              (const float*)state, state_stride, tail_off, token_req, cu_q, ctx_len, req_slot, positions, qn, kn, vc,
              beta, g, s);
    if (taps > 1) {
      const int by = (C + 255) / 256;
      ll_launch(delta_conv_update_kernel<T>, dim3(num_entries, by < 8 ? by : 8), dim3(256), 0, stream, (const T*)proj,
                proj_stride, q_off, k_off, v_off, state, state_stride, tail_off, cu_q, ctx_len, req_slot, s);
    }
  });
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_delta_recurrence(const float* qn, const float* kn, const float* vc, const float* beta,
                                   const float* g, float* state, long state_stride, const int* cu_q,
                                   const int* req_slot, float* o, int num_entries, int H, int Hk, int dk, int dv,
                                   int per_channel, cudaStream_t stream) {
  if (num_entries <= 0) return 0;
  if (H <= 0 || Hk <= 0 || H % Hk || dk <= 0 || dk > 256 || dv <= 0) return (int)cudaErrorInvalidValue;
  DeltaShape s{H, Hk, dk, dv, 0, per_channel};
#define DR_LAUNCH(LANES, NR)                                                                                        \
  do {                                                                                                              \
    constexpr int cols = DR_THREADS / LANES;                                                                        \
    dim3 grid(num_entries, H, (dv + cols - 1) / cols), block(DR_THREADS);                                           \
    const size_t smem = sizeof(float) * 2 * DR_CH * (3 * (size_t)LANES * NR + cols + 2);                            \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(delta_recurrence_kernel<LANES, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                           (int)smem);                                                                              \
    ll_launch(delta_recurrence_kernel<LANES, NR>, grid, block, smem, stream, qn, kn, vc, beta, g, state,            \
              state_stride, cu_q, req_slot, o, s);                                                                  \
  } while (0)
  if (dk <= 4) DR_LAUNCH(1, 4);
  else if (dk <= 8) DR_LAUNCH(2, 4);
  else if (dk <= 16) DR_LAUNCH(4, 4);
  else if (dk <= 32) DR_LAUNCH(8, 4);
  else if (dk <= 64) DR_LAUNCH(16, 4);
  else if (dk <= 128) DR_LAUNCH(32, 4);
  else DR_LAUNCH(32, 8);
#undef DR_LAUNCH
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_delta_out(int dtype, void* out, const float* o, const float* w, const void* gate, long gate_stride,
                            float eps, int num_tokens, int H, int dv, int gate_act, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int pairs = num_tokens * H;
  LL_DISPATCH_DTYPE(dtype, ll_launch(delta_out_kernel<T>, dim3((pairs + 3) / 4), dim3(128), 0, stream, (T*)out, o, w,
                                     (const T*)gate, gate_stride, eps, pairs, H, dv, gate_act));
  return LL_LAUNCH_RESULT();
}
