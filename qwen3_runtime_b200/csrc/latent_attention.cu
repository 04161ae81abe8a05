// Attention through a low-rank latent: the cache holds one row [latent (rank) | rotated key part
// (rot)] per token for all heads; queries arrive already moved into the latent space, so every head
// scores against the same rows and the value of a row is its first `dv` elements.
//
//   latent_norm_rope_store  per token: RMSNorm of the query latent, RMSNorm of the key latent,
//                           rotation of the shared key part, write of the row into its page
//   rotate_heads            rotation of the queries' rotated part into the latent-space query
//   latent_attention        causal attention of every token over its sequence's rows, with an
//                           optional window and an optional per-head sink in the denominator
//
// Rotation: pair i = elements (2i, 2i + 1) (pairing 1) or (i, i + pairs) (pairing 0), angle =
// float(position) * inv_freq[i] in fp32, exact cosf/sinf, both multiplied by `magnitude`; elements beyond
// 2 * pairs pass unchanged.  All norms, scores and softmax are fp32.
#include "common.cuh"

// ---- query latent norm, key latent norm, key rotation, cache write -------------------------------
// in: [T, *] rows of [q_rank | kv_rank | rot_dim] (row stride in elements).  q_out: [T, q_rank].
// pages: [num_pages, ps, kv_rank + rot_dim].
template <typename T>
__global__ void latent_norm_rope_store_kernel(const T* __restrict__ in, long in_stride, int q_rank, int kv_rank,
                                              int rot_dim, const float* __restrict__ q_w,
                                              const float* __restrict__ kv_w, float eps,
                                              const float* __restrict__ inv_freq, int pairs,
                                              const int* __restrict__ positions, const int* __restrict__ token_seq,
                                              const int* __restrict__ block_table, int max_pages,
                                              T* __restrict__ pages, int ps, int write, T* __restrict__ q_out,
                                              int pairing, float magnitude) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const T* row = in + (long)t * in_stride;
  float sq = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float a = to_f32(row[i]);
    sq += a * a;
  }
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const float c = to_f32(row[q_rank + i]);
    sc += c * c;
  }
  const float rq = q_rank ? rsqrtf(block_sum(sq, red) / (float)q_rank + eps) : 0.f;
  const float rc = rsqrtf(block_sum(sc, red) / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    q_out[(long)t * q_rank + i] = from_f32<T>((to_f32(row[i]) * rq) * q_w[i]);
  if (!write) return;
  const int p = positions[t];
  const int page = block_table[(long)token_seq[t] * max_pages + p / ps];
  if (page < 0) return;
  T* dst = pages + ((long)page * ps + (p % ps)) * (kv_rank + rot_dim);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
    dst[i] = from_f32<T>((to_f32(row[q_rank + i]) * rc) * kv_w[i]);
  const T* k = row + q_rank + kv_rank;
  if (!pairing) {  // halves: pair i = (i, i + pairs); the rest is copied
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) {
      float y = to_f32(k[i]);
      if (i < 2 * pairs) {
        const bool first = i < pairs;
        const int pi = first ? i : i - pairs;
        const float other = to_f32(k[first ? i + pairs : i - pairs]);
        const float ang = (float)p * inv_freq[pi];
        const float cs = cosf(ang) * magnitude, sn = sinf(ang) * magnitude;
        y = first ? y * cs - other * sn : y * cs + other * sn;
      }
      dst[kv_rank + i] = from_f32<T>(y);
    }
    return;
  }
  for (int i = threadIdx.x; i < (rot_dim + 1) / 2; i += blockDim.x) {
    const float u = to_f32(k[2 * i]);
    if (2 * i + 1 >= rot_dim) {
      dst[kv_rank + 2 * i] = from_f32<T>(u);
    } else {
      const float v = to_f32(k[2 * i + 1]);
      if (i < pairs) {
        const float ang = (float)p * inv_freq[i];
        const float cs = cosf(ang) * magnitude, sn = sinf(ang) * magnitude;
        dst[kv_rank + 2 * i] = from_f32<T>(u * cs - v * sn);
        dst[kv_rank + 2 * i + 1] = from_f32<T>(v * cs + u * sn);
      } else {
        dst[kv_rank + 2 * i] = from_f32<T>(u);
        dst[kv_rank + 2 * i + 1] = from_f32<T>(v);
      }
    }
  }
}

Q3_EXPORT int q3_latent_norm_rope_store(int dtype, const void* in, long in_stride, int q_rank, int kv_rank, int rot_dim,
                                        const float* q_w, const float* kv_w, float eps, const float* inv_freq,
                                        int pairs, const int* positions, const int* token_seq,
                                        const int* block_table, int max_pages, void* pages, int ps, int num_tokens,
                                        int write, void* q_out, int pairing, float magnitude,
                                        cudaStream_t stream) {
  if (!in || !kv_w || q_rank < 0 || kv_rank < 1 || rot_dim < 0 || ps < 1) return Q3_ERR_ARGUMENT;
  if ((q_rank && (!q_w || !q_out)) || pairing < 0 || pairing > 1) return Q3_ERR_ARGUMENT;
  if (write && (!positions || !token_seq || !block_table || !pages)) return Q3_ERR_ARGUMENT;
  if (pairs < 0 || 2 * pairs > rot_dim || (pairs && !inv_freq)) return Q3_ERR_ARGUMENT;
  if (num_tokens == 0) return Q3_OK;
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(latent_norm_rope_store_kernel<float>, dim3(num_tokens), dim3(128), 0, stream, (const float*)in,
                   in_stride, q_rank, kv_rank, rot_dim, q_w, kv_w, eps, inv_freq, pairs, positions, token_seq,
                   block_table, max_pages, (float*)pages, ps, write, (float*)q_out, pairing, magnitude);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(latent_norm_rope_store_kernel<bf16>, dim3(num_tokens), dim3(128), 0, stream, (const bf16*)in,
                   in_stride, q_rank, kv_rank, rot_dim, q_w, kv_w, eps, inv_freq, pairs, positions, token_seq,
                   block_table, max_pages, (bf16*)pages, ps, write, (bf16*)q_out, pairing, magnitude);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// ---- rotation of [T, H, n] (strided) into [T, H, n] (strided) -------------------------------------
template <typename T>
__global__ void rotate_heads_kernel(const T* __restrict__ x, long xs_t, long xs_h, T* __restrict__ out, long os_t,
                                    long os_h, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int pairs, int n, int H, long total,
                                    int pairing, float magnitude) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  if (!pairing) {  // halves: one thread per element, pair i = (i, i + pairs)
    const int i = (int)(idx % n);
    const long th = idx / n;
    const int h = (int)(th % H);
    const long t = th / H;
    const T* src = x + t * xs_t + h * xs_h;
    float y = to_f32(src[i]);
    if (i < 2 * pairs) {
      const bool first = i < pairs;
      const int pi = first ? i : i - pairs;
      const float other = to_f32(src[first ? i + pairs : i - pairs]);
      const float ang = (float)positions[t] * inv_freq[pi];
      const float cs = cosf(ang) * magnitude, sn = sinf(ang) * magnitude;
      y = first ? y * cs - other * sn : y * cs + other * sn;
    }
    out[t * os_t + h * os_h + i] = from_f32<T>(y);
    return;
  }
  const int half = (n + 1) / 2;
  const int i = (int)(idx % half);
  const long th = idx / half;
  const int h = (int)(th % H);
  const long t = th / H;
  const T* src = x + t * xs_t + h * xs_h;
  T* dst = out + t * os_t + h * os_h;
  const float u = to_f32(src[2 * i]);
  if (2 * i + 1 >= n) {
    dst[2 * i] = from_f32<T>(u);
    return;
  }
  const float v = to_f32(src[2 * i + 1]);
  if (i < pairs) {
    const float ang = (float)positions[t] * inv_freq[i];
    const float cs = cosf(ang) * magnitude, sn = sinf(ang) * magnitude;
    dst[2 * i] = from_f32<T>(u * cs - v * sn);
    dst[2 * i + 1] = from_f32<T>(v * cs + u * sn);
  } else {
    dst[2 * i] = from_f32<T>(u);
    dst[2 * i + 1] = from_f32<T>(v);
  }
}

Q3_EXPORT int q3_rotate_heads(int dtype, const void* x, long xs_t, long xs_h, void* out, long os_t, long os_h,
                              const int* positions, const float* inv_freq, int pairs, int n, int H, int num_tokens,
                              int pairing, float magnitude, cudaStream_t stream) {
  if (!x || !out || n < 1 || H < 1 || pairs < 0 || 2 * pairs > n) return Q3_ERR_ARGUMENT;
  if (pairs && (!positions || !inv_freq)) return Q3_ERR_ARGUMENT;
  if (pairing < 0 || pairing > 1 || (!pairing && x == out)) return Q3_ERR_ARGUMENT;  // halves read their partner: not in place
  const long total = (long)num_tokens * H * (pairing ? (n + 1) / 2 : n);
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == Q3_DTYPE_F32)
    rotate_heads_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, xs_t, xs_h, (float*)out, os_t, os_h,
                                                            positions, inv_freq, pairs, n, H, total, pairing, magnitude);
  else if (dtype == Q3_DTYPE_BF16)
    rotate_heads_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)x, xs_t, xs_h, (bf16*)out, os_t, os_h,
                                                           positions, inv_freq, pairs, n, H, total, pairing, magnitude);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}

// ---- attention over latent rows, any sizes -------------------------------------------------------
// One block per (token, group of up to WARPS heads); one warp per head.  The query at absolute
// position p sees rows lo..p of its sequence (lo = p - window + 1 with a window, else 0).  Rows are
// visited in tiles of 32 aligned to absolute positions; a tile is brought into shared memory once
// for all the block's heads, each lane scores one row, and the softmax runs online in fp32 with
// exact expf.  A sink starts the running maximum at sink_h with a denominator of 1 and no value.
// The order of every reduction depends on (p, window) only, so a token's result does not depend on
// how the sequence was cut into steps or on what else is in the batch.
constexpr int LATENT_MAX_ACC = 32;  // value width up to 32 * 32

template <typename T, int WARPS>
__global__ void latent_attention_kernel(const T* __restrict__ q, long qs_t, long qs_h, const T* __restrict__ pages,
                                        int dk, int dv, const int* __restrict__ block_table, int max_pages,
                                        const int* __restrict__ token_seq, const int* __restrict__ positions,
                                        const float* __restrict__ sink, T* __restrict__ out, long os_t, long os_h,
                                        int H, int ps, float scale, int window) {
  extern __shared__ float smem[];
  float* qs = smem;                    // [WARPS][dk]
  float* ks = smem + WARPS * dk;       // [32][dk + 1]
  __shared__ long row_of[32];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * WARPS + warp;
  const bool live = h < H;
  const int p = positions[t];
  const int* bt = block_table + (long)token_seq[t] * max_pages;
  const int kst = dk + 1;
  if (live) {
    const T* qrow = q + (long)t * qs_t + (long)h * qs_h;
    for (int d = lane; d < dk; d += 32) qs[warp * dk + d] = to_f32(qrow[d]);
  }
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  float m = -INFINITY, l = 0.f;
  if (live && sink) {
    m = sink[h];
    l = 1.f;
  }
  float acc[LATENT_MAX_ACC];
#pragma unroll
  for (int c = 0; c < LATENT_MAX_ACC; ++c) acc[c] = 0.f;
  const float* myq = qs + warp * dk;
  for (int j0 = lo & ~31; j0 <= p; j0 += 32) {
    __syncthreads();  // the last tile has been read by every warp (and qs is written)
    if (threadIdx.x < 32) {
      const int j = j0 + threadIdx.x;
      long r = -1;
      if (j >= lo && j <= p) {
        const int page = bt[j / ps];
        if (page >= 0) r = ((long)page * ps + (j % ps)) * dk;
      }
      row_of[threadIdx.x] = r;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 32 * dk; idx += WARPS * 32) {
      const int jj = idx / dk, d = idx - jj * dk;
      const long r = row_of[jj];
      ks[jj * kst + d] = r >= 0 ? to_f32(pages[r + d]) : 0.f;
    }
    __syncthreads();
    if (!live) continue;
    const bool valid = row_of[lane] >= 0;
    float s = -INFINITY;
    if (valid) {
      const float* kr = ks + lane * kst;
      float dot = 0.f;
      for (int d = 0; d < dk; ++d) dot = fmaf(myq[d], kr[d], dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pl = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(pl);
#pragma unroll
    for (int c = 0; c < LATENT_MAX_ACC; ++c) acc[c] *= corr;
    const int count = min(32, p - j0 + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, pl, jj);
      if (pj == 0.f) continue;
      const float* vr = ks + jj * kst;
#pragma unroll
      for (int c = 0; c < LATENT_MAX_ACC; ++c) {
        const int d = lane + 32 * c;
        if (d < dv) acc[c] = fmaf(pj, vr[d], acc[c]);
      }
    }
    m = m_new;
  }
  if (!live) return;
  T* orow = out + (long)t * os_t + (long)h * os_h;
  const float inv = 1.f / l;
#pragma unroll
  for (int c = 0; c < LATENT_MAX_ACC; ++c) {
    const int d = lane + 32 * c;
    if (d < dv) orow[d] = from_f32<T>(acc[c] * inv);
  }
}

template <typename T, int WARPS>
static int launch_latent_attention(const void* q, long qs_t, long qs_h, const void* pages, int dk, int dv,
                                   const int* block_table, int max_pages, const int* token_seq,
                                   const int* positions, const float* sink, void* out, long os_t, long os_h,
                                   int num_tokens, int H, int ps, float scale, int window, cudaStream_t stream) {
  const size_t smem = ((size_t)WARPS * dk + 32 * (size_t)(dk + 1)) * sizeof(float);
  if (smem > 200 * 1024) return Q3_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_attention_kernel<T, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const dim3 grid(num_tokens, (H + WARPS - 1) / WARPS);
  return launch_pdl(latent_attention_kernel<T, WARPS>, grid, dim3(WARPS * 32), smem, stream, (const T*)q, qs_t, qs_h,
                    (const T*)pages, dk, dv, block_table, max_pages, token_seq, positions, sink, (T*)out, os_t, os_h,
                    H, ps, scale, window) == cudaSuccess
             ? Q3_OK
             : Q3_ERR_LAUNCH;
}

// q: (t, h, d) at q + t*qs_t + h*qs_h + d, d < dk.  pages: [num_pages, ps, dk].  out: (t, h, d) at
// out + t*os_t + h*os_h + d, d < dv <= dk.  sink: fp32 [H] or null.  window <= 0: none.
Q3_EXPORT int q3_latent_attention(int dtype, const void* q, long qs_t, long qs_h, const void* pages, int dk, int dv,
                                  const int* block_table, int max_pages, const int* token_seq, const int* positions,
                                  const float* sink, void* out, long os_t, long os_h, int num_tokens, int H, int ps,
                                  float scale, int window, cudaStream_t stream) {
  if (!q || !pages || !block_table || !token_seq || !positions || !out) return Q3_ERR_ARGUMENT;
  if (H < 1 || ps < 1 || dk < 1 || dv < 1 || dv > dk) return Q3_ERR_ARGUMENT;
  if (dv > 32 * LATENT_MAX_ACC) return Q3_ERR_UNSUPPORTED;
  if (num_tokens == 0) return Q3_OK;
  if (H > 65535) return Q3_ERR_UNSUPPORTED;
#define LAUNCH(TYPE, W)                                                                                              \
  return launch_latent_attention<TYPE, W>(q, qs_t, qs_h, pages, dk, dv, block_table, max_pages, token_seq, positions, \
                                          sink, out, os_t, os_h, num_tokens, H, ps, scale, window, stream)
  if (dtype == Q3_DTYPE_F32) {
    if (H >= 8) LAUNCH(float, 8);
    if (H >= 4) LAUNCH(float, 4);
    if (H >= 2) LAUNCH(float, 2);
    LAUNCH(float, 1);
  }
  if (dtype == Q3_DTYPE_BF16) {
    if (H >= 8) LAUNCH(bf16, 8);
    if (H >= 4) LAUNCH(bf16, 4);
    if (H >= 2) LAUNCH(bf16, 2);
    LAUNCH(bf16, 1);
  }
#undef LAUNCH
  return Q3_ERR_ARGUMENT;
}
