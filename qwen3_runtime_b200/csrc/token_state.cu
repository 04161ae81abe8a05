// What a layer carries from a sequence's previous token in a state slot: its id (an embedding that
// hashes pairs of tokens) or its input row (a mixer that blends every token's input with its
// predecessor's).
//
//   bigram_embed     x[t] = embed[id_t] * scale + bigram[row_t]     (fp32 rows; optionally a copy in the
//                    activation type)   row_t = (id_(t-1) * mul_prev + id_t * mul_cur) mod buckets, and
//                    row `buckets` for a sequence's first token (position 0)
//   token_shift_mix  y[s][t] = h[t] + (h[t-1] - h[t]) * mu[s]       for each of `n` blends s, fp32 math
//                    (h[-1] = 0 for a sequence's first token)
//
// The token before a step's first token of a sequence comes from the sequence's slot; a second small
// kernel stores the step's last token (its id, or its row as fp32) there afterwards.  A kernel starts
// with griddepcontrol.wait, so the store never overtakes the reads of the kernel before it.
#include "common.cuh"

template <typename T>
__global__ void bigram_embed_kernel(const int* __restrict__ ids, const T* __restrict__ embed, float scale,
                                    const T* __restrict__ bigram, int buckets, long mul_prev, long mul_cur,
                                    const int* __restrict__ prev_state, const int* __restrict__ positions,
                                    const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                                    const int* __restrict__ state_slots, float* __restrict__ out,
                                    T* __restrict__ copy, long copy_stride, int W, int vocab, int wide) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* erow = embed + (long)id * W;
  const T* brow = nullptr;
  if (bigram) {
    long row = buckets;
    if (positions[t] > 0) {
      const int b = token_seq[t];
      const long prev = t > cu_seqlens[b] ? ids[t - 1] : prev_state[state_slots[b]];
      row = (prev * mul_prev + (long)id * mul_cur) % buckets;
      if (row < 0) row += buckets;
    }
    brow = bigram + row * W;
  }
  if (wide) {  // rows of a multiple of 8 values, 16-byte aligned: eight values a thread
    for (int i = threadIdx.x * 8; i < W; i += blockDim.x * 8) {
      float v[8], b[8];
      load8(erow + i, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= scale;
      if (brow) {
        load8(brow + i, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += b[e];
      }
      store8(out + (long)t * W + i, v);
      if (copy) store8(copy + (long)t * copy_stride + i, v);
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = to_f32(erow[i]) * scale;
    if (brow) v += to_f32(brow[i]);
    out[(long)t * W + i] = v;
    if (copy) copy[(long)t * copy_stride + i] = from_f32<T>(v);
  }
}

__global__ void prev_token_update_kernel(const int* __restrict__ ids, const int* __restrict__ cu_seqlens,
                                         const int* __restrict__ state_slots, int* __restrict__ prev_state,
                                         int num_seqs) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= num_seqs) return;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  if (t1 > t0) prev_state[state_slots[b]] = ids[t1 - 1];
}

// ids: [T]; embed: [vocab, W]; bigram: [buckets + 1, W] or null; prev_state: int32 [slots] (one id per
// slot) or null without a bigram table; out: fp32 [T, W]; copy: [T, *] rows copy_stride apart, or null.
Q3_EXPORT int q3_bigram_embed(int dtype, const int* ids, const void* embed, float scale, const void* bigram,
                              int buckets, long mul_prev, long mul_cur, int* prev_state, const int* positions,
                              const int* token_seq, const int* cu_seqlens, const int* state_slots, float* out,
                              void* copy, long copy_stride, int num_tokens, int num_seqs, int W, int vocab,
                              cudaStream_t stream) {
  if (!ids || !embed || !out || W < 1 || vocab < 1) return Q3_ERR_ARGUMENT;
  if (bigram && (buckets < 1 || !prev_state || !positions || !token_seq || !cu_seqlens || !state_slots))
    return Q3_ERR_ARGUMENT;
  if (num_tokens == 0) return Q3_OK;
  const uintptr_t bits = (uintptr_t)embed | (uintptr_t)bigram | (uintptr_t)out | (uintptr_t)copy;
  const int wide = W % 8 == 0 && copy_stride % 8 == 0 && !(bits & 15);
  const int threads = wide ? (W >= 2048 ? 256 : (W >= 512 ? 64 : 32)) : (W >= 1024 ? 256 : 128);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(bigram_embed_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, ids, (const float*)embed,
                   scale, (const float*)bigram, buckets, mul_prev, mul_cur, (const int*)prev_state, positions,
                   token_seq, cu_seqlens, state_slots, out, (float*)copy, copy_stride, W, vocab, wide);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(bigram_embed_kernel<bf16>, dim3(num_tokens), dim3(threads), 0, stream, ids, (const bf16*)embed,
                   scale, (const bf16*)bigram, buckets, mul_prev, mul_cur, (const int*)prev_state, positions,
                   token_seq, cu_seqlens, state_slots, out, (bf16*)copy, copy_stride, W, vocab, wide);
  else
    return Q3_ERR_ARGUMENT;
  if (e != cudaSuccess) return Q3_ERR_LAUNCH;
  if (bigram) {
    e = launch_pdl(prev_token_update_kernel, dim3((num_seqs + 127) / 128), dim3(128), 0, stream, ids, cu_seqlens,
                   state_slots, prev_state, num_seqs);
    if (e != cudaSuccess) return Q3_ERR_LAUNCH;
  }
  return Q3_OK;
}

template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ h, long h_stride, const float* __restrict__ mu, int n,
                                       const float* __restrict__ state, const int* __restrict__ positions,
                                       const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                                       const int* __restrict__ state_slots, T* __restrict__ out, long plane, int W,
                                       int wide) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const bool first = positions[t] <= 0;
  const bool inside = t > cu_seqlens[b];
  const T* cur = h + (long)t * h_stride;
  const T* before = h + (long)(t - 1) * h_stride;
  const float* kept = state + (long)state_slots[b] * W;
  if (wide) {  // rows of a multiple of 8 values, 16-byte aligned: eight values a thread
    for (int i = threadIdx.x * 8; i < W; i += blockDim.x * 8) {
      float x[8], p[8], m[8], y[8];
      load8(cur + i, x);
      if (first) {
#pragma unroll
        for (int e = 0; e < 8; ++e) p[e] = 0.f;
      } else if (inside) {
        load8(before + i, p);
      } else {
        load8(kept + i, p);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) p[e] -= x[e];
      for (int s = 0; s < n; ++s) {
        load8(mu + (long)s * W + i, m);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = fmaf(p[e], m[e], x[e]);
        store8(out + s * plane + (long)t * W + i, y);
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float x = to_f32(cur[i]);
    const float p = first ? 0.f : (inside ? to_f32(before[i]) : kept[i]);
    const float d = p - x;
    for (int s = 0; s < n; ++s) out[s * plane + (long)t * W + i] = from_f32<T>(fmaf(d, mu[(long)s * W + i], x));
  }
}

template <typename T>
__global__ void token_shift_update_kernel(const T* __restrict__ h, long h_stride, const int* __restrict__ cu_seqlens,
                                          const int* __restrict__ state_slots, float* __restrict__ state, int W) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  if (t1 <= t0) return;
  const T* row = h + (long)(t1 - 1) * h_stride;
  float* kept = state + (long)state_slots[b] * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) kept[i] = to_f32(row[i]);
}

// h: [T, W] rows h_stride apart; mu: fp32 [n, W]; state: fp32 [slots, W]; out: [n, T, W] dense.
Q3_EXPORT int q3_token_shift_mix(int dtype, const void* h, long h_stride, const float* mu, int n, float* state,
                                 const int* positions, const int* token_seq, const int* cu_seqlens,
                                 const int* state_slots, void* out, int num_tokens, int num_seqs, int W,
                                 cudaStream_t stream) {
  if (!h || !mu || !state || !positions || !token_seq || !cu_seqlens || !state_slots || !out || n < 1 || W < 1)
    return Q3_ERR_ARGUMENT;
  if (num_tokens == 0) return Q3_OK;
  const uintptr_t bits = (uintptr_t)h | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)out;
  const int wide = W % 8 == 0 && h_stride % 8 == 0 && !(bits & 15);
  const int threads = W >= 1024 ? 256 : 128;
  const int mix_threads = wide ? (W >= 2048 ? 256 : (W >= 512 ? 64 : 32)) : threads;
  const long plane = (long)num_tokens * W;
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32) {
    e = launch_pdl(token_shift_mix_kernel<float>, dim3(num_tokens), dim3(mix_threads), 0, stream, (const float*)h,
                   h_stride, mu, n, (const float*)state, positions, token_seq, cu_seqlens, state_slots, (float*)out,
                   plane, W, wide);
    if (e == cudaSuccess)
      e = launch_pdl(token_shift_update_kernel<float>, dim3(num_seqs), dim3(threads), 0, stream, (const float*)h,
                     h_stride, cu_seqlens, state_slots, state, W);
  } else if (dtype == Q3_DTYPE_BF16) {
    e = launch_pdl(token_shift_mix_kernel<bf16>, dim3(num_tokens), dim3(mix_threads), 0, stream, (const bf16*)h,
                   h_stride, mu, n, (const float*)state, positions, token_seq, cu_seqlens, state_slots, (bf16*)out,
                   plane, W, wide);
    if (e == cudaSuccess)
      e = launch_pdl(token_shift_update_kernel<bf16>, dim3(num_seqs), dim3(threads), 0, stream, (const bf16*)h,
                     h_stride, cu_seqlens, state_slots, state, W);
  } else {
    return Q3_ERR_ARGUMENT;
  }
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}
