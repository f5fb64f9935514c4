// Latent attention: softmax attention whose keys and values are expansions of one latent vector per token.
//
// Per token the cache holds one row [R + r]: the normed latent c (R numbers) and a rotated key part k_r (r
// numbers) that all heads share.  With per-head expansions k_h = Uk_h c and v_h = Uv_h c the score of query
// head h against a token is (q_h . Uk_h c + q_r,h . k_r) * scale = ((Uk_h^T q_h) . c + q_r,h . k_r) * scale, and
// the head's output is Uv_h (sum_j p_j c_j).  So the kernel here works in the latent space: its queries are
// a_h = Uk_h^T q_h (R numbers, made by a batched product before it) and the rotated part, its keys are the
// cached rows, its values the first R numbers of the same rows, and what it returns is sum_j p_j c_j per head
// (expanded by a batched product after it).  Nothing per head is ever cached or re-expanded.
//
// Rotation (interleaved pairs): numbers 2i and 2i+1 of a rotated part, for 2i < rot_dims, turn by the angle
// position * freq[i]; (u, v) -> (u cos - v sin, v cos + u sin); the rest passes unchanged.  Angles, the
// latent's norm, scores and softmax are float32.
//
//   latent_prepare    per token: RMS norm of the latent, rotation of k_r and of every head's q_r, cache write
//   latent_attention  per (token, 8 heads): online softmax over the visible rows of the request, i.e.
//                     positions lo..p with lo = max(0, p - window + 1) (window <= 0: all)
// Keys are walked in tiles of 32 positions that start at multiples of 32, so the order of every sum depends
// on the position only, not on how the tokens were cut into steps or batched.
#include "common.cuh"

// proj row t: q heads at q_off, head h's rotated part at q_off + h * (d + r) + d; the latent at kv_off (R wide),
// then the rotated key part (r wide).
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ proj, long proj_stride, int q_off, int kv_off, const float* __restrict__ norm_w,
                      float eps, const float* __restrict__ freq, int rot_dims, const int* __restrict__ positions,
                      const int* __restrict__ slot_map, T* __restrict__ cache, long num_slots,
                      float* __restrict__ q_rot, int H, int d, int r, int R, int* status) {
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x, tid = threadIdx.x;
  const T* row = proj + (size_t)t * proj_stride;
  const float p = (float)positions[t];
  // every head's rotated query part -> float32 [tokens, H, r]
  const int half = rot_dims / 2;
  for (int i = tid; i < H * r; i += blockDim.x) {
    const int h = i / r, j = i % r;
    const T* src = row + q_off + (size_t)h * (d + r) + d;
    float out;
    if (j < 2 * half) {
      float sn, cs;
      sincosf(p * freq[j >> 1], &sn, &cs);
      const float u = to_f32<T>(src[j & ~1]), v = to_f32<T>(src[j | 1]);
      out = (j & 1) ? v * cs + u * sn : u * cs - v * sn;
    } else {
      out = to_f32<T>(src[j]);
    }
    q_rot[((size_t)t * H + h) * r + j] = out;
  }
  const long slot = slot_map ? slot_map[t] : -1;
  if (slot < 0) return;     // padding token, or a run-step that only reads this plane
  if (slot >= num_slots) {
    if (tid == 0) set_status(status, LL_ERR_SLOT_RANGE);
    return;
  }
  const T* lat = row + kv_off;
  float ss = 0.f;
  for (int i = tid; i < R; i += blockDim.x) {
    const float x = to_f32<T>(lat[i]);
    ss = fmaf(x, x, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)R + eps);
  T* dst = cache + (size_t)slot * (R + r);
  for (int i = tid; i < R; i += blockDim.x) dst[i] = from_f32<T>(to_f32<T>(lat[i]) * inv * norm_w[i]);
  for (int j = tid; j < r; j += blockDim.x) {
    float out;
    if (j < 2 * half) {
      float sn, cs;
      sincosf(p * freq[j >> 1], &sn, &cs);
      const float u = to_f32<T>(lat[R + (j & ~1)]), v = to_f32<T>(lat[R + (j | 1)]);
      out = (j & 1) ? v * cs + u * sn : u * cs - v * sn;
    } else {
      out = to_f32<T>(lat[R + j]);
    }
    dst[R + j] = from_f32<T>(out);
  }
}

#define LA_TK 32
#define LA_THREADS 128
#define LA_WARPS 4
#define LA_GH 8
#define LA_MAX_R 512

// qa: float32 latent-space queries, head h of token t at qa + h * qa_hstride + t * qa_tstride (R numbers);
// q_rot: float32 [tokens, H, r]; cache: one plane [pages, 1, page_size, R + r]; out: T, head h of token t at
// out + h * out_hstride + t * out_tstride (R numbers).
template <typename T>
__global__ void __launch_bounds__(LA_THREADS)
latent_attention_kernel(T* __restrict__ out, long out_hstride, long out_tstride, const float* __restrict__ qa,
                        long qa_hstride, long qa_tstride, const float* __restrict__ q_rot,
                        const T* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
                        const int* __restrict__ token_req, const int* __restrict__ req_slot,
                        const int* __restrict__ positions, int H, int R, int r, int page_size, int num_pages,
                        int window, float scale, int* status) {
  extern __shared__ float smem[];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const int h0 = blockIdx.y * LA_GH;
  const int hc = min(LA_GH, H - h0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int KD = R + r;
  float* qs = smem;                         // [LA_GH][KD]
  float* ks = qs + LA_GH * KD;              // [LA_TK][KD + 1]
  float* ps = ks + LA_TK * (KD + 1);        // [LA_GH][LA_TK]
  float* alpha_s = ps + LA_GH * LA_TK;      // [LA_GH]
  float* l_s = alpha_s + LA_GH;             // [LA_GH]

  const int entry = token_req[t];
  const int slot = entry >= 0 ? req_slot[entry] : -1;
  const int p = positions[t];
  if (slot < 0 || p < 0) {
    for (int i = tid; i < hc * R; i += LA_THREADS)
      out[(size_t)(h0 + i / R) * out_hstride + (size_t)t * out_tstride + i % R] = from_f32<T>(0.f);
    return;
  }
  const int* bt = block_table + (size_t)slot * bt_stride;
  const int lo = (window > 0) ? max(0, p - window + 1) : 0;
  for (int i = tid; i < hc * KD; i += LA_THREADS) {
    const int g = i / KD, j = i % KD;
    qs[i] = j < R ? qa[(size_t)(h0 + g) * qa_hstride + (size_t)t * qa_tstride + j]
                  : q_rot[((size_t)t * H + h0 + g) * r + (j - R)];
  }
  float m_run[LA_GH / LA_WARPS], l_run[LA_GH / LA_WARPS];
#pragma unroll
  for (int i = 0; i < LA_GH / LA_WARPS; ++i) {
    m_run[i] = -INFINITY;
    l_run[i] = 0.f;
  }
  float acc[LA_GH][LA_MAX_R / LA_THREADS];
#pragma unroll
  for (int g = 0; g < LA_GH; ++g)
#pragma unroll
    for (int c = 0; c < LA_MAX_R / LA_THREADS; ++c) acc[g][c] = 0.f;

  for (int tile0 = (lo / LA_TK) * LA_TK; tile0 <= p; tile0 += LA_TK) {
    __syncthreads();
    for (int j = warp; j < LA_TK; j += LA_WARPS) {
      const int pos = tile0 + j;
      const bool valid = (pos >= lo && pos <= p);
      long base = -1;
      if (valid) {
        const int page = bt[pos / page_size];
        if (page < 0 || page >= num_pages) {
          if (lane == 0) set_status(status, LL_ERR_PAGE_RANGE);
        } else {
          base = ((long)page * page_size + (pos % page_size)) * KD;
        }
      }
      for (int c = lane; c < KD; c += 32) ks[j * (KD + 1) + c] = base >= 0 ? to_f32<T>(cache[base + c]) : 0.f;
    }
    __syncthreads();
    {
      const int pos = tile0 + lane;
      const bool valid = (pos >= lo && pos <= p);
#pragma unroll
      for (int i = 0; i < LA_GH / LA_WARPS; ++i) {
        const int g = warp + i * LA_WARPS;
        if (g < hc) {
          float s = 0.f;
          const float* qg = qs + g * KD;
          const float* kj = ks + lane * (KD + 1);
          for (int c = 0; c < KD; ++c) s = fmaf(qg[c], kj[c], s);
          s = valid ? s * scale : -INFINITY;
          const float m_new = fmaxf(m_run[i], warp_max(s));
          const float pj = valid ? expf(s - m_new) : 0.f;
          const float alpha = expf(m_run[i] - m_new);
          l_run[i] = l_run[i] * alpha + warp_sum(pj);
          m_run[i] = m_new;
          ps[g * LA_TK + lane] = pj;
          if (lane == 0) alpha_s[g] = alpha;
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < LA_MAX_R / LA_THREADS; ++c) {
      const int dd = tid + c * LA_THREADS;
      if (dd < R) {
#pragma unroll
        for (int g = 0; g < LA_GH; ++g) {
          if (g < hc) {
            float a = acc[g][c] * alpha_s[g];
            const float* pg = ps + g * LA_TK;
#pragma unroll 8
            for (int j = 0; j < LA_TK; ++j) a = fmaf(pg[j], ks[j * (KD + 1) + dd], a);
            acc[g][c] = a;
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < LA_GH / LA_WARPS; ++i) {
    const int g = warp + i * LA_WARPS;
    if (g < hc && lane == 0) l_s[g] = l_run[i];
  }
  __syncthreads();
#pragma unroll
  for (int c = 0; c < LA_MAX_R / LA_THREADS; ++c) {
    const int dd = tid + c * LA_THREADS;
    if (dd < R) {
#pragma unroll
      for (int g = 0; g < LA_GH; ++g)
        if (g < hc)
          out[(size_t)(h0 + g) * out_hstride + (size_t)t * out_tstride + dd] = from_f32<T>(acc[g][c] / l_s[g]);
    }
  }
}

extern "C" int ll_latent_prepare(int dtype, const void* proj, long proj_stride, int q_off, int kv_off,
                                 const float* norm_w, float eps, const float* freq, int rot_dims, const int* positions,
                                 const int* slot_map, void* cache, long num_slots, float* q_rot, int num_tokens, int H,
                                 int d, int r, int R, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || d < 0 || r < 0 || R <= 0 || rot_dims < 0 || rot_dims > r) return (int)cudaErrorInvalidValue;
  LL_DISPATCH_DTYPE(dtype, ll_launch(latent_prepare_kernel<T>, dim3(num_tokens), dim3(128), 0, stream, (const T*)proj,
                                     proj_stride, q_off, kv_off, norm_w, eps, freq, rot_dims, positions, slot_map,
                                     (T*)cache, num_slots, q_rot, H, d, r, R, status));
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_latent_attention(int dtype, void* out, long out_hstride, long out_tstride, const float* qa,
                                   long qa_hstride, long qa_tstride, const float* q_rot, const void* cache,
                                   const int* block_table, int bt_stride, const int* token_req, const int* req_slot,
                                   const int* positions, int num_tokens, int H, int R, int r, int page_size,
                                   int num_pages, int window, float scale, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || R <= 0 || R > LA_MAX_R || r < 0 || page_size <= 0) return (int)cudaErrorInvalidValue;
  const int KD = R + r;
  const size_t smem = sizeof(float) * ((size_t)LA_GH * KD + (size_t)LA_TK * (KD + 1) + LA_GH * LA_TK + 2 * LA_GH);
  dim3 grid(num_tokens, (H + LA_GH - 1) / LA_GH);
  LL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(latent_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(latent_attention_kernel<T>, grid, dim3(LA_THREADS), smem, stream, (T*)out, out_hstride, out_tstride, qa,
              qa_hstride, qa_tstride, q_rot, (const T*)cache, block_table, bt_stride, token_req, req_slot, positions, H,
              R, r, page_size, num_pages, window, scale, status);
  });
  return LL_LAUNCH_RESULT();
}
