// Causal attention over the paged cache for any mix of prompt portions and single
// decoded tokens: the general kernel (any head_dim up to 256 (multiples of 8 with
// 16-byte loads), a value size of its own up to 256, any head counts, any page size, optional
// window), used by the fp32 path and wherever a specialised kernel refuses a size.  Options: a
// window that leaves the sequence's first `keep_first` keys readable (they are visited first, in
// tiles of their own, then the window's); a sink, one more score without a value in the softmax's
// denominator, p_j = exp(s_j) / (exp(sink) + sum exp(s_j')); a gate, the result times
// sigmoid(gate[t, h, d]) before the one rounding; a chunked mask (`chunk` > 0: position p reads keys from
// floor(p / chunk) * chunk on, chunks counted from the sequence's position 0); capped scores
// (`softcap` > 0: s <- softcap * tanh(s / softcap) after the scale).  A second kernel is differential
// attention: two score maps per head over the same values, combined and normed in the epilogue.
//
// One warp per (token, query head).  The query at absolute position p attends to
// keys lo..p of its own sequence (lo = p - window + 1 with a window, else 0), which
// the cache holds already because keys are stored before attention runs
// (attention/pytorch.py:12-47).  Keys are visited in tiles of 32 aligned to
// absolute positions, each lane scoring one key, with an online softmax in fp32
// and exact expf.  The order of every reduction depends only on (p, window), so
// the result of a token does not depend on how the work was cut into steps or on
// what else is in the batch.
#include "common.cuh"

template <typename T, int WARPS>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, int q_stride,
                                               const T* __restrict__ kpages, const T* __restrict__ vpages,
                                               const int* __restrict__ block_table, int max_pages,
                                               const int* __restrict__ token_seq,
                                               const int* __restrict__ positions, T* __restrict__ out,
                                               long out_stride, int num_tokens, int nq, int nkv, int D, int Dv, int ps, float scale,
                                               int window, int keep_first, int has_sink, float sink,
                                               const T* __restrict__ gate, long gate_stride, int chunk,
                                               float softcap) {
  extern __shared__ float qs_all[];  // WARPS * D
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * WARPS + warp;
  if (item >= (long)num_tokens * nq) return;
  const int t = (int)(item / nq);
  const int h = (int)(item - (long)t * nq);
  const int kvh = h / (nq / nkv);
  const int p = positions[t];
  const int* bt = block_table + (long)token_seq[t] * max_pages;
  float* qs = qs_all + warp * D;
  const T* qrow = q + (long)t * q_stride + (long)h * D;
  for (int d = lane; d < D; d += 32) qs[d] = to_f32(qrow[d]);
  __syncwarp();
  int lo = window > 0 ? max(0, p - window + 1) : 0;
  if (chunk > 0) lo = max(lo, p / chunk * chunk);
  float m = -INFINITY, l = 0.f;
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  // keys first..last (inclusive) of this range; tiles start at multiples of 32
  const int kept_last = min(keep_first, lo) - 1;  // the kept first keys that the window does not hold
  for (int range = kept_last >= 0 ? 0 : 1; range < 2; ++range) {
    const int first = range ? lo : 0, last = range ? p : kept_last;
    for (int j0 = first & ~31; j0 <= last; j0 += 32) {
      const int j = j0 + lane;
      const bool valid = j >= first && j <= last;
      long row = 0;  // the key's row among all (page, head, place) rows; keys have D, values Dv elements
      float s = -INFINITY;
      if (valid) {
        const int page = bt[j / ps];
        row = ((long)page * nkv + kvh) * ps + (j % ps);
        const T* kr = kpages + row * D;
        float dot = 0.f;
        if ((D & 7) == 0) {
          for (int d = 0; d < D; d += 8) {
            float kv[8];
            load8(kr + d, kv);
#pragma unroll
            for (int e = 0; e < 8; ++e) dot = fmaf(qs[d + e], kv[e], dot);
          }
        } else {  // rows that are not 16-byte multiples: one element at a time
          for (int d = 0; d < D; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
        }
        s = dot * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      }
      const float m_new = fmaxf(m, warp_max(s));
      const float pl = valid ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);
      l = l * corr + warp_sum(pl);
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] *= corr;
      const int count = min(32, last - j0 + 1);
      for (int jj = 0; jj < count; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pl, jj);
        const long rj = __shfl_sync(0xffffffffu, row, jj);
        if (pj == 0.f) continue;  // keys before the window, or fully underflowed
        const T* vr = vpages + rj * Dv;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int d = lane + 32 * c;
          if (d < Dv) acc[c] = fmaf(pj, to_f32(vr[d]), acc[c]);
        }
      }
      m = m_new;
    }
  }
  T* orow = out + (long)t * out_stride + (long)h * Dv;
  if (has_sink) {  // one more score in the denominator
    const float m_all = fmaxf(m, sink), corr = expf(m - m_all);
    l = l * corr + expf(sink - m_all);
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] *= corr;
  }
  const float inv = 1.f / l;
  const T* grow = gate ? gate + (long)t * gate_stride + (long)h * Dv : nullptr;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int d = lane + 32 * c;
    if (d < Dv) {
      float val = acc[c] * inv;
      if (grow) val *= 1.f / (1.f + expf(-to_f32(grow[d])));
      orow[d] = from_f32<T>(val);
    }
  }
}

// q: [num_tokens, *] with row stride q_stride (elements), head h at column h*D.  Keys are
// [pages, nkv, ps, D], values [pages, nkv, ps, Dv].  out: rows out_stride elements apart, head h at
// column h*Dv.  window <= 0: none; keep_first counts only with a window; gate: rows gate_stride elements
// apart, head h at column h*Dv, or null.  chunk <= 0: no chunked mask; softcap <= 0: scores as they are.
Q3_EXPORT int q3_paged_attention_generic(int dtype, const void* q, int q_stride, const void* kpages,
                                         const void* vpages, const int* block_table, int max_pages,
                                         const int* token_seq, const int* positions, void* out,
                                         long out_stride, int num_tokens, int nq, int nkv, int D, int Dv, int ps,
                                         float scale, int window, int keep_first, int has_sink, float sink,
                                         const void* gate, long gate_stride, int chunk, float softcap,
                                         cudaStream_t stream) {
  if (!q || !kpages || !vpages || !block_table || !token_seq || !positions || !out) return Q3_ERR_ARGUMENT;
  if (nq < 1 || nkv < 1 || nq % nkv || ps < 1) return Q3_ERR_ARGUMENT;
  if (D < 1 || D > 256 || Dv < 1 || Dv > 256 || out_stride < (long)nq * Dv) return Q3_ERR_UNSUPPORTED;
  if (keep_first < 0 || (gate && gate_stride < (long)nq * Dv)) return Q3_ERR_ARGUMENT;
  if (chunk < 0 || softcap < 0.f || (chunk > 0 && keep_first > 0)) return Q3_ERR_ARGUMENT;
  if (window <= 0) keep_first = 0;
  if (num_tokens == 0) return Q3_OK;
  constexpr int WARPS = 4;
  const size_t smem = (size_t)WARPS * D * sizeof(float);
  const long items = (long)num_tokens * nq;
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  if (dtype == Q3_DTYPE_F32)
    paged_attention_generic_kernel<float, WARPS><<<blocks, WARPS * 32, smem, stream>>>(
        (const float*)q, q_stride, (const float*)kpages, (const float*)vpages, block_table, max_pages,
        token_seq, positions, (float*)out, out_stride, num_tokens, nq, nkv, D, Dv, ps, scale, window, keep_first,
        has_sink, sink, (const float*)gate, gate_stride, chunk, softcap);
  else if (dtype == Q3_DTYPE_BF16)
    paged_attention_generic_kernel<bf16, WARPS><<<blocks, WARPS * 32, smem, stream>>>(
        (const bf16*)q, q_stride, (const bf16*)kpages, (const bf16*)vpages, block_table, max_pages,
        token_seq, positions, (bf16*)out, out_stride, num_tokens, nq, nkv, D, Dv, ps, scale, window, keep_first,
        has_sink, sink, (const bf16*)gate, gate_stride, chunk, softcap);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}


// ---- differential attention ------------------------------------------------------------------------
// A query head is two maps [q1 | q2] of D elements each, a key head [k1 | k2] likewise (key pages
// [pages, nkv, ps, 2 * D]); both maps attend over the same values (value pages [pages, nkv, ps, Dv]):
//   a_m = softmax_j(scale * q_m . k_m(j)) V        o = a_1 - lambda * a_2
//   out = o * rsqrt(mean(o^2) + eps) * out_scale   (over the head's Dv values, no weight)
// One warp per (token, query head); a key's row is read once for both scores and a value's row once for
// both sums.  Keys in tiles of 32 aligned to absolute positions, two online softmaxes in fp32 with exact
// expf: the order of every reduction depends only on the token's position and the masks.  window and
// chunk as in the kernel above.
template <typename T, int WARPS>
__global__ void paged_attention_diff_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ kpages,
                                            const T* __restrict__ vpages, const int* __restrict__ block_table,
                                            int max_pages, const int* __restrict__ token_seq,
                                            const int* __restrict__ positions, T* __restrict__ out, long out_stride,
                                            int num_tokens, int nq, int nkv, int D, int Dv, int ps, float scale,
                                            int window, int chunk, float lambda, float eps, float out_scale) {
  extern __shared__ float qs_all[];  // WARPS * 2 * D
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * WARPS + warp;
  if (item >= (long)num_tokens * nq) return;
  const int t = (int)(item / nq);
  const int h = (int)(item - (long)t * nq);
  const int kvh = h / (nq / nkv);
  const int p = positions[t];
  const int* bt = block_table + (long)token_seq[t] * max_pages;
  float* qs = qs_all + warp * 2 * D;
  const T* qrow = q + (long)t * q_stride + (long)h * 2 * D;
  for (int d = lane; d < 2 * D; d += 32) qs[d] = to_f32(qrow[d]);
  __syncwarp();
  int lo = window > 0 ? max(0, p - window + 1) : 0;
  if (chunk > 0) lo = max(lo, p / chunk * chunk);
  float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
  float acc1[8], acc2[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc1[c] = acc2[c] = 0.f;
  for (int j0 = lo & ~31; j0 <= p; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j >= lo && j <= p;
    long row = 0;
    float s1 = -INFINITY, s2 = -INFINITY;
    if (valid) {
      const int page = bt[j / ps];
      row = ((long)page * nkv + kvh) * ps + (j % ps);
      const T* kr = kpages + row * 2 * D;
      float d1 = 0.f, d2 = 0.f;
      if ((D & 7) == 0) {
        for (int d = 0; d < D; d += 8) {
          float ka[8], kb[8];
          load8(kr + d, ka);
          load8(kr + D + d, kb);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            d1 = fmaf(qs[d + e], ka[e], d1);
            d2 = fmaf(qs[D + d + e], kb[e], d2);
          }
        }
      } else {
        for (int d = 0; d < D; ++d) {
          d1 = fmaf(qs[d], to_f32(kr[d]), d1);
          d2 = fmaf(qs[D + d], to_f32(kr[D + d]), d2);
        }
      }
      s1 = d1 * scale;
      s2 = d2 * scale;
    }
    const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
    const float p1 = valid ? expf(s1 - n1) : 0.f, p2 = valid ? expf(s2 - n2) : 0.f;
    const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);
    l1 = l1 * c1 + warp_sum(p1);
    l2 = l2 * c2 + warp_sum(p2);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      acc1[c] *= c1;
      acc2[c] *= c2;
    }
    const int count = min(32, p - j0 + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float w1 = __shfl_sync(0xffffffffu, p1, jj);
      const float w2 = __shfl_sync(0xffffffffu, p2, jj);
      const long rj = __shfl_sync(0xffffffffu, row, jj);
      if (w1 == 0.f && w2 == 0.f) continue;  // keys before the mask's start, or fully underflowed
      const T* vr = vpages + rj * Dv;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int d = lane + 32 * c;
        if (d < Dv) {
          const float v = to_f32(vr[d]);
          acc1[c] = fmaf(w1, v, acc1[c]);
          acc2[c] = fmaf(w2, v, acc2[c]);
        }
      }
    }
    m1 = n1;
    m2 = n2;
  }
  const float i1 = 1.f / l1, i2 = 1.f / l2;
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int d = lane + 32 * c;
    if (d < Dv) {
      acc1[c] = acc1[c] * i1 - lambda * (acc2[c] * i2);
      ss += acc1[c] * acc1[c];
    }
  }
  const float rstd = rsqrtf(warp_sum(ss) / (float)Dv + eps) * out_scale;
  T* orow = out + (long)t * out_stride + (long)h * Dv;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int d = lane + 32 * c;
    if (d < Dv) orow[d] = from_f32<T>(acc1[c] * rstd);
  }
}

// q: rows q_stride elements apart, head h's two maps at columns h * 2D .. h * 2D + 2D.  D is one map's size.
Q3_EXPORT int q3_paged_attention_diff(int dtype, const void* q, int q_stride, const void* kpages, const void* vpages,
                                      const int* block_table, int max_pages, const int* token_seq,
                                      const int* positions, void* out, long out_stride, int num_tokens, int nq,
                                      int nkv, int D, int Dv, int ps, float scale, int window, int chunk,
                                      float lambda, float eps, float out_scale, cudaStream_t stream) {
  if (!q || !kpages || !vpages || !block_table || !token_seq || !positions || !out) return Q3_ERR_ARGUMENT;
  if (nq < 1 || nkv < 1 || nq % nkv || ps < 1 || chunk < 0) return Q3_ERR_ARGUMENT;
  if (D < 1 || D > 256 || Dv < 1 || Dv > 256 || out_stride < (long)nq * Dv) return Q3_ERR_UNSUPPORTED;
  if (num_tokens == 0) return Q3_OK;
  constexpr int WARPS = 4;
  const size_t smem = (size_t)WARPS * 2 * D * sizeof(float);
  const long items = (long)num_tokens * nq;
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  if (dtype == Q3_DTYPE_F32)
    paged_attention_diff_kernel<float, WARPS><<<blocks, WARPS * 32, smem, stream>>>(
        (const float*)q, q_stride, (const float*)kpages, (const float*)vpages, block_table, max_pages, token_seq,
        positions, (float*)out, out_stride, num_tokens, nq, nkv, D, Dv, ps, scale, window, chunk, lambda, eps,
        out_scale);
  else if (dtype == Q3_DTYPE_BF16)
    paged_attention_diff_kernel<bf16, WARPS><<<blocks, WARPS * 32, smem, stream>>>(
        (const bf16*)q, q_stride, (const bf16*)kpages, (const bf16*)vpages, block_table, max_pages, token_seq,
        positions, (bf16*)out, out_stride, num_tokens, nq, nkv, D, Dv, ps, scale, window, chunk, lambda, eps,
        out_scale);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}
