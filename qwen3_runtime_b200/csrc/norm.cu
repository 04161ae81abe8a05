// RMSNorm fused with what feeds it: the residual add, the embedding lookup and a
// row gather.  All arithmetic is fp32; one rounding at the store.
//
//   v   = (ids ? table[ids[r]] : resid[r]) + (pending ? pending[r] : 0)      (fp32)
//         pending is either [rows, H] of the output's type or, with parts > 0, fp32
//         [parts, rows, H] (planes `part_stride` elements apart) whose planes are the
//         partial sums of a product over ranges of its inner dimension
//         (csrc/gemm_stream.cu); they are added in plane order, then to the residual
//   resid[r] = v                                  (when write_resid)
//   out[i]  = (v * rsqrt(mean(v^2) + eps)) * w    (qwen3_runtime/layers/ops.py:17-37)
//
// `rows` (optional) selects which source rows are processed; output row i then
// comes from source row rows[i] (used for the final norm, which only runs on the
// rows whose logits are wanted, qwen3_runtime/models/qwen3.py:263-264).
#include "common.cuh"

template <typename T>
__global__ void fused_norm_kernel(const void* __restrict__ pending, int parts, long part_stride,
                                  float* __restrict__ resid, const int* __restrict__ ids,
                                  const T* __restrict__ table, const int* __restrict__ rows,
                                  const float* __restrict__ w, T* __restrict__ out, int H, float eps,
                                  int write_resid, int vocab) {
  extern __shared__ float vals[];  // H floats, then 33 for the reduction
  float* red = vals + H;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const long src = rows ? rows[r] : r;
  const T* trow = nullptr;
  if (ids) {
    int id = ids[src];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    trow = table + (long)id * H;
  }
  const T* prow = pending && !parts ? static_cast<const T*>(pending) + src * H : nullptr;
  const float* frow = pending && parts ? static_cast<const float*>(pending) + src * H : nullptr;
  float* rrow = resid ? resid + src * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = trow ? to_f32(trow[i]) : rrow[i];
    if (prow) v += to_f32(prow[i]);
    if (frow) {
      float sum = frow[i];
      for (int p = 1; p < parts; ++p) sum += frow[p * part_stride + i];
      v += sum;
    }
    if (write_resid) rrow[i] = v;
    vals[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, red);
  const float rstd = rsqrtf(total / (float)H + eps);
  T* orow = out + (long)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = from_f32<T>((vals[i] * rstd) * w[i]);
}

// The same with 16-byte accesses: H a multiple of 8 and every row 16-byte aligned.
// REGS: the block has a thread for every 8 elements of a row, so a thread's 8 values stay in
// registers between the two passes (no staging through shared memory).
// PLANES: what is pending may be partial-sum planes (a variant of its own, so that the common one
// keeps its registers).
template <typename T, bool REGS, bool PLANES>
__global__ void __launch_bounds__(512) fused_norm_vec_kernel(const void* __restrict__ pending, int parts, long part_stride,
                                      float* __restrict__ resid, const int* __restrict__ ids,
                                      const T* __restrict__ table, const int* __restrict__ rows,
                                      const float* __restrict__ w, T* __restrict__ out, int H, float eps,
                                      int write_resid, int vocab) {
  extern __shared__ float vals[];
  float* red = REGS ? vals : vals + H;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const long src = rows ? rows[r] : r;
  const T* trow = nullptr;
  if (ids) {
    int id = ids[src];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    trow = table + (long)id * H;
  }
  const T* prow = pending && !parts ? static_cast<const T*>(pending) + src * H : nullptr;
  const float* frow = PLANES && pending && parts ? static_cast<const float*>(pending) + src * H : nullptr;
  float* rrow = resid ? resid + src * H : nullptr;
  float ss = 0.f;
  float mine[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8];
    if (trow) load8(trow + i, v); else load8(rrow + i, v);
    if (prow) {
      float pv[8];
      load8(prow + i, pv);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += pv[e];
    }
    if (PLANES && frow) {  // four planes' loads in flight at a time; added in plane order
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int p0 = 0; p0 < parts; p0 += 4) {
        float pv[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (p0 + j < parts) load8(frow + (p0 + j) * part_stride + i, pv[j]);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (p0 + j < parts) {
#pragma unroll
            for (int e = 0; e < 8; ++e) sum[e] += pv[j][e];
          }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += sum[e];
    }
    if (write_resid) store8(rrow + i, v);
    if (REGS) {
#pragma unroll
      for (int e = 0; e < 8; ++e) mine[e] = v[e];
    } else {
      store8(vals + i, v);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
  }
  const float total = block_sum(ss, red);
  const float rstd = rsqrtf(total / (float)H + eps);
  T* orow = out + (long)r * H;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8], wv[8];
    if (REGS) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = mine[e];
    } else {
      load8(vals + i, v);
    }
    load8(w + i, wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = (v[e] * rstd) * wv[e];
    store8(orow + i, v);
  }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static int launch_fused_norm(const void* pending, int parts, long part_stride, float* resid, const int* ids,
                             const void* table, const int* rows, const float* w, void* out, int num_rows, int H,
                             float eps, int write_resid, int vocab, cudaStream_t stream) {
  if (num_rows == 0) return Q3_OK;
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  if (smem > 200 * 1024) return Q3_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(fused_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const bool vec = H % 8 == 0 && part_stride % 4 == 0 && aligned16(pending) && aligned16(resid) &&
                   aligned16(table) && aligned16(w) && aligned16(out);
  if (vec) {
    int threads = ((H / 8 + 31) / 32) * 32;
    threads = threads > 512 ? 512 : threads;
    const bool regs = threads * 8 >= H;  // one chunk per thread: the values stay in registers
    const size_t vec_smem = regs ? 33 * sizeof(float) : smem;
    void (*kernel)(const void*, int, long, float*, const int*, const T*, const int*, const float*, T*, int, float, int,
                   int);
    if (parts)
      kernel = regs ? fused_norm_vec_kernel<T, true, true> : fused_norm_vec_kernel<T, false, true>;
    else
      kernel = regs ? fused_norm_vec_kernel<T, true, false> : fused_norm_vec_kernel<T, false, false>;
    if (vec_smem > 48 * 1024)
      cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)vec_smem);
    return launch_pdl(kernel, dim3(num_rows), dim3(threads), vec_smem, stream, pending, parts, part_stride, resid, ids,
                      (const T*)table, rows, w, (T*)out, H, eps, write_resid, vocab) == cudaSuccess
               ? Q3_OK
               : Q3_ERR_LAUNCH;
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  fused_norm_kernel<T><<<num_rows, threads, smem, stream>>>(
      pending, parts, part_stride, resid, ids, (const T*)table, rows, w, (T*)out, H, eps, write_resid, vocab);
  return q3_launch_status();
}

// out[num_rows, H]; resid fp32 [*, H] (may be null only when ids is given and
// write_resid is 0); table/out have `dtype`; w is fp32 [H].  pending has `dtype` when
// pending_parts is 0, else it is fp32 with pending_parts planes, part_stride elements apart.
Q3_EXPORT int q3_fused_norm(int dtype, const void* pending, int pending_parts, long part_stride, float* resid,
                            const int* ids, const void* table,
                            const int* rows, const float* w, void* out, int num_rows, int H, float eps,
                            int write_resid, int vocab, cudaStream_t stream) {
  if (!w || !out || H < 1) return Q3_ERR_ARGUMENT;
  if (!ids && !resid) return Q3_ERR_ARGUMENT;
  if (ids && !table) return Q3_ERR_ARGUMENT;
  if (write_resid && !resid) return Q3_ERR_ARGUMENT;
  if (pending_parts < 0 || (pending_parts && (!pending || part_stride < 0))) return Q3_ERR_ARGUMENT;
  if (dtype == Q3_DTYPE_F32)
    return launch_fused_norm<float>(pending, pending_parts, part_stride, resid, ids, table, rows, w, out, num_rows, H, eps, write_resid,
                                    vocab, stream);
  if (dtype == Q3_DTYPE_BF16)
    return launch_fused_norm<bf16>(pending, pending_parts, part_stride, resid, ids, table, rows, w, out, num_rows, H, eps, write_resid,
                                   vocab, stream);
  return Q3_ERR_ARGUMENT;
}

// ---- SwiGLU product: out[t, i] = silu(gu[t, i]) * gu[t, I + i]  (layers/ops.py:23-25) ----
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long total, int I) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long t = idx / I;
  const int i = (int)(idx - t * I);
  const float g = to_f32(gu[t * 2 * I + i]);
  const float u = to_f32(gu[t * 2 * I + I + i]);
  out[idx] = from_f32<T>((g / (1.f + expf(-g))) * u);
}

template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, long chunks, int I) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= chunks) return;
  const int per_row = I / 8;
  const long t = idx / per_row;
  const int i = (int)(idx - t * per_row) * 8;
  float g[8], u[8];
  load8(gu + t * 2 * I + i, g);
  load8(gu + t * 2 * I + I + i, u);
#pragma unroll
  for (int e = 0; e < 8; ++e) g[e] = (g[e] / (1.f + expf(-g[e]))) * u[e];
  store8(out + t * I + i, g);
}

Q3_EXPORT int q3_silu_mul(int dtype, const void* gu, void* out, int num_rows, int I, cudaStream_t stream) {
  if (!gu || !out || I < 1) return Q3_ERR_ARGUMENT;
  const long total = (long)num_rows * I;
  if (total == 0) return Q3_OK;
  const int threads = 256;
  if (I % 8 == 0 && aligned16(gu) && aligned16(out)) {
    const long chunks = total / 8;
    const unsigned vblocks = (unsigned)((chunks + threads - 1) / threads);
    if (dtype == Q3_DTYPE_F32)
      silu_mul_vec_kernel<float><<<vblocks, threads, 0, stream>>>((const float*)gu, (float*)out, chunks, I);
    else if (dtype == Q3_DTYPE_BF16)
      silu_mul_vec_kernel<bf16><<<vblocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, chunks, I);
    else
      return Q3_ERR_ARGUMENT;
    return q3_launch_status();
  }
  const long blocks = (total + threads - 1) / threads;
  if (dtype == Q3_DTYPE_F32)
    silu_mul_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>((const float*)gu, (float*)out, total, I);
  else if (dtype == Q3_DTYPE_BF16)
    silu_mul_kernel<bf16><<<(unsigned)blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, total, I);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}

// ---- small epilogues that an architecture may ask for (Qwen3 dense uses neither) ---------------------
// out[r][c] += bias[c]: the bias of a projection, added in fp32 to the product's rounded value.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, long ld, const float* __restrict__ bias, long total, int N) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long r = idx / N;
  const int c = (int)(idx - r * N);
  out[r * ld + c] = from_f32<T>(to_f32(out[r * ld + c]) + bias[c]);
}

Q3_EXPORT int q3_add_bias(int dtype, void* out, long ld, const float* bias, int num_rows, int N, cudaStream_t stream) {
  if (!out || !bias || N < 1 || ld < N) return Q3_ERR_ARGUMENT;
  const long total = (long)num_rows * N;
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == Q3_DTYPE_F32)
    add_bias_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, ld, bias, total, N);
  else if (dtype == Q3_DTYPE_BF16)
    add_bias_kernel<bf16><<<blocks, 256, 0, stream>>>((bf16*)out, ld, bias, total, N);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}

// logits = logits * scale, then (cap > 0) cap * tanh(logits / cap), in place on fp32 logits.
__global__ void logit_scale_cap_kernel(float* __restrict__ logits, long total, float scale, float cap) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  float v = logits[idx] * scale;
  if (cap > 0.f) v = cap * tanhf(v / cap);
  logits[idx] = v;
}

Q3_EXPORT int q3_logit_scale_cap(float* logits, long total, float scale, float cap, cudaStream_t stream) {
  if (!logits || total < 0 || cap < 0.f) return Q3_ERR_ARGUMENT;
  if (total == 0) return Q3_OK;
  logit_scale_cap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(logits, total, scale, cap);
  return q3_launch_status();
}

// ---- x[r, i] *= sigmoid(g[r, i]): a gate on a sublayer's inner rows.  x dense [rows, n]; g rows g_stride
//      elements apart (a slice of a wider product).  fp32 math, one rounding. ----
template <typename T>
__global__ void sigmoid_mul_kernel(T* __restrict__ x, const T* __restrict__ g, long g_stride, long total, int n) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long r = idx / n;
  const int i = (int)(idx - r * n);
  const float gate = to_f32(g[r * g_stride + i]);
  x[idx] = from_f32<T>(to_f32(x[idx]) / (1.f + expf(-gate)));
}

Q3_EXPORT int q3_sigmoid_mul(int dtype, void* x, const void* g, long g_stride, int num_rows, int n,
                             cudaStream_t stream) {
  if (!x || !g || n < 1 || g_stride < n) return Q3_ERR_ARGUMENT;
  const long total = (long)num_rows * n;
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == Q3_DTYPE_F32)
    sigmoid_mul_kernel<float><<<blocks, 256, 0, stream>>>((float*)x, (const float*)g, g_stride, total, n);
  else if (dtype == Q3_DTYPE_BF16)
    sigmoid_mul_kernel<bf16><<<blocks, 256, 0, stream>>>((bf16*)x, (const bf16*)g, g_stride, total, n);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}

// ---- RMSNorm of the sum, with what is pending normalised before it is added -----------------------
// For blocks that norm a sublayer's output as well as its input:
//   y   = pending[r]                                              (the sublayer's output, fp32 math)
//   y'  = post_w ? (y * rsqrt(mean(y^2) + post_eps)) * post_w : y
//   v   = (ids ? table[ids[r]] : resid[r]) + y' + (add_ids ? add_table[add_ids[r]] : 0)
//   resid[r] = v (when write_resid);   out[i] = (v * rsqrt(mean(v^2) + eps)) * w
// `add_ids/add_table` add embedding rows to the sum once more (a looped stack fed its input again);
// `add_vec` (fp32 [H]) is added to every row's sum (a learned offset per pass of a loop).  Without `w`
// nothing is normalised: out = v, rounded (the stream itself as the input of a product).
// `center` bit 0: what is pending is layer-normed, (y - mean(y)) * rsqrt(mean((y - mean(y))^2) + post_eps) * post_w;
// bit 1: so is the sum, out = (v - mean(v)) * rsqrt(mean((v - mean(v))^2) + eps) * w.
// One block per row; the row's y and v stay in shared memory between the passes.
template <typename T>
__global__ void fused_post_norm_kernel(const void* __restrict__ pending_any, int parts, long part_stride,
                                       const float* __restrict__ post_w, float post_eps,
                                       float* __restrict__ resid, const int* __restrict__ ids,
                                       const T* __restrict__ table, const int* __restrict__ add_ids,
                                       const T* __restrict__ add_table, const float* __restrict__ add_vec,
                                       const int* __restrict__ rows,
                                       const float* __restrict__ w, T* __restrict__ out, int H, float eps,
                                       int write_resid, int vocab, int center) {
  extern __shared__ float vals[];  // y[H], v[H], 33 for the reductions
  float* ys = vals;
  float* vs = vals + H;
  float* red = vals + 2 * H;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const long src = rows ? rows[r] : r;
  float post_rstd = 1.f, post_mean = 0.f;
  const bool pending = pending_any != nullptr;
  if (pending) {
    const T* prow = static_cast<const T*>(pending_any) + src * H;
    const float* frow = static_cast<const float*>(pending_any) + src * H;  // with parts: fp32 planes, added in order
    float ss = 0.f, s1 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float y;
      if (parts) {
        y = frow[i];
        for (int p = 1; p < parts; ++p) y += frow[p * part_stride + i];
      } else {
        y = to_f32(prow[i]);
      }
      ys[i] = y;
      ss += y * y;
      s1 += y;
    }
    if (post_w && (center & 1)) {  // layer norm: the mean first, then the mean of the squared deviations
      post_mean = block_sum(s1, red) / (float)H;
      float sd = 0.f;
      for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = ys[i] - post_mean;
        sd += d * d;
      }
      post_rstd = rsqrtf(block_sum(sd, red) / (float)H + post_eps);
    } else if (post_w) {
      post_rstd = rsqrtf(block_sum(ss, red) / (float)H + post_eps);
    }
  }
  const T* trow = nullptr;
  if (ids) {
    int id = ids[src];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    trow = table + (long)id * H;
  }
  const T* arow = nullptr;
  if (add_ids) {
    int id = add_ids[src];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    arow = add_table + (long)id * H;
  }
  float* rrow = resid ? resid + src * H : nullptr;
  float ss = 0.f, s1 = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = trow ? to_f32(trow[i]) : rrow[i];
    if (pending) v += post_w ? ((ys[i] - post_mean) * post_rstd) * post_w[i] : ys[i];
    if (arow) v += to_f32(arow[i]);
    if (add_vec) v += add_vec[i];
    if (write_resid) rrow[i] = v;
    vs[i] = v;
    ss += v * v;
    s1 += v;
  }
  T* orow = out + (long)r * H;
  if (!w) {  // the sum itself, rounded to the output's type
    for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = from_f32<T>(vs[i]);
    return;
  }
  if (center & 2) {
    const float mean = block_sum(s1, red) / (float)H;
    float sd = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float d = vs[i] - mean;
      sd += d * d;
    }
    const float rstd = rsqrtf(block_sum(sd, red) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = from_f32<T>(((vs[i] - mean) * rstd) * w[i]);
    return;
  }
  const float rstd = rsqrtf(block_sum(ss, red) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = from_f32<T>((vs[i] * rstd) * w[i]);
}

// The same with 16-byte accesses: H a multiple of 8 and every row 16-byte aligned (plane strides
// multiples of 4 elements).
template <typename T>
__global__ void fused_post_norm_vec_kernel(const void* __restrict__ pending_any, int parts, long part_stride,
                                           const float* __restrict__ post_w, float post_eps,
                                           float* __restrict__ resid, const int* __restrict__ ids,
                                           const T* __restrict__ table, const int* __restrict__ add_ids,
                                           const T* __restrict__ add_table, const float* __restrict__ add_vec,
                                           const int* __restrict__ rows, const float* __restrict__ w,
                                           T* __restrict__ out, int H, float eps, int write_resid, int vocab,
                                           int center) {
  extern __shared__ __align__(16) float vals[];  // y[H], v[H], 33 for the reductions
  float* ys = vals;
  float* vs = vals + H;
  float* red = vals + 2 * H;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const long src = rows ? rows[r] : r;
  float post_rstd = 1.f, post_mean = 0.f;
  const bool pending = pending_any != nullptr;
  if (pending) {
    const T* prow = static_cast<const T*>(pending_any) + src * H;
    const float* frow = static_cast<const float*>(pending_any) + src * H;
    float ss = 0.f, s1 = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float y[8];
      if (parts) {
        load8(frow + i, y);
        for (int p = 1; p < parts; ++p) {
          float pv[8];
          load8(frow + p * part_stride + i, pv);
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] += pv[e];
        }
      } else {
        load8(prow + i, y);
      }
      store8(ys + i, y);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        ss += y[e] * y[e];
        s1 += y[e];
      }
    }
    if (post_w && (center & 1)) {  // layer norm: the mean first, then the mean of the squared deviations
      post_mean = block_sum(s1, red) / (float)H;
      float sd = 0.f;
      for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
        float y[8];
        load8(ys + i, y);
#pragma unroll
        for (int e = 0; e < 8; ++e) sd += (y[e] - post_mean) * (y[e] - post_mean);
      }
      post_rstd = rsqrtf(block_sum(sd, red) / (float)H + post_eps);
    } else if (post_w) {
      post_rstd = rsqrtf(block_sum(ss, red) / (float)H + post_eps);
    }
  }
  const T* trow = nullptr;
  if (ids) {
    int id = ids[src];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    trow = table + (long)id * H;
  }
  const T* arow = nullptr;
  if (add_ids) {
    int id = add_ids[src];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    arow = add_table + (long)id * H;
  }
  float* rrow = resid ? resid + src * H : nullptr;
  T* orow = out + (long)r * H;
  float ss = 0.f, s1 = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8], x[8];
    if (trow) load8(trow + i, v); else load8(rrow + i, v);
    if (pending) {
      load8(ys + i, x);
      if (post_w) {
        float pw[8];
        load8(post_w + i, pw);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += ((x[e] - post_mean) * post_rstd) * pw[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += x[e];
      }
    }
    if (arow) {
      load8(arow + i, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += x[e];
    }
    if (add_vec) {
      load8(add_vec + i, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += x[e];
    }
    if (write_resid) store8(rrow + i, v);
    if (!w) {
      store8(orow + i, v);  // the sum itself, rounded to the output's type
      continue;
    }
    store8(vs + i, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      ss += v[e] * v[e];
      s1 += v[e];
    }
  }
  if (!w) return;
  float mean = 0.f, rstd;
  if (center & 2) {
    mean = block_sum(s1, red) / (float)H;
    float sd = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float v[8];
      load8(vs + i, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) sd += (v[e] - mean) * (v[e] - mean);
    }
    rstd = rsqrtf(block_sum(sd, red) / (float)H + eps);
  } else {
    rstd = rsqrtf(block_sum(ss, red) / (float)H + eps);
  }
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8], wv[8];
    load8(vs + i, v);
    load8(w + i, wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = ((v[e] - mean) * rstd) * wv[e];
    store8(orow + i, v);
  }
}

template <typename T>
static int launch_fused_post_norm(const void* pending, int parts, long part_stride, const float* post_w, float post_eps,
                                  float* resid,
                                  const int* ids, const void* table, const int* add_ids, const void* add_table,
                                  const float* add_vec, const int* rows, const float* w, void* out, int num_rows,
                                  int H, float eps, int write_resid, int vocab, int center, cudaStream_t stream) {
  if (num_rows == 0) return Q3_OK;
  const size_t smem = (size_t)(2 * H + 33) * sizeof(float);
  if (smem > 200 * 1024) return Q3_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(fused_post_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (H % 8 == 0 && part_stride % 4 == 0 && aligned16(pending) && aligned16(post_w) && aligned16(resid) &&
      aligned16(table) && aligned16(add_table) && aligned16(add_vec) && aligned16(w) && aligned16(out)) {
    int vthreads = ((H / 8 + 31) / 32) * 32;  // eight elements a thread
    vthreads = vthreads > 512 ? 512 : vthreads;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(fused_post_norm_vec_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_pdl(fused_post_norm_vec_kernel<T>, dim3(num_rows), dim3(vthreads), smem, stream, pending, parts,
                      part_stride, post_w, post_eps, resid, ids, (const T*)table, add_ids, (const T*)add_table, add_vec,
                      rows, w, (T*)out, H, eps, write_resid, vocab, center) == cudaSuccess
               ? Q3_OK
               : Q3_ERR_LAUNCH;
  }
  int threads = ((H / 4 + 31) / 32) * 32;  // about four elements a thread: the row's loads are all in flight at once
  threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
  return launch_pdl(fused_post_norm_kernel<T>, dim3(num_rows), dim3(threads), smem, stream, pending, parts, part_stride,
                    post_w, post_eps, resid, ids, (const T*)table, add_ids, (const T*)add_table, add_vec, rows, w, (T*)out, H,
                    eps, write_resid, vocab, center) == cudaSuccess
             ? Q3_OK
             : Q3_ERR_LAUNCH;
}

// pending (pending_parts = 0), table, add_table and out have `dtype`; with pending_parts > 0 pending is
// fp32 [pending_parts, rows, H], planes part_stride elements apart; post_w and w are fp32 [H]; resid is fp32.
Q3_EXPORT int q3_fused_post_norm(int dtype, const void* pending, int pending_parts, long part_stride,
                                 const float* post_w, float post_eps, float* resid,
                                 const int* ids, const void* table, const int* add_ids, const void* add_table,
                                 const float* add_vec, const int* rows, const float* w, void* out, int num_rows,
                                 int H, float eps, int write_resid, int vocab, int center, cudaStream_t stream) {
  if (!out || H < 1 || center < 0 || center > 3) return Q3_ERR_ARGUMENT;
  if (!ids && !resid) return Q3_ERR_ARGUMENT;
  if ((ids && !table) || (add_ids && !add_table)) return Q3_ERR_ARGUMENT;
  if (write_resid && !resid) return Q3_ERR_ARGUMENT;
  if (post_w && !pending) return Q3_ERR_ARGUMENT;
  if (pending_parts < 0 || (pending_parts && (!pending || part_stride < 0))) return Q3_ERR_ARGUMENT;
  if (dtype == Q3_DTYPE_F32)
    return launch_fused_post_norm<float>(pending, pending_parts, part_stride, post_w, post_eps, resid, ids, table, add_ids, add_table, add_vec, rows,
                                         w, out, num_rows, H, eps, write_resid, vocab, center, stream);
  if (dtype == Q3_DTYPE_BF16)
    return launch_fused_post_norm<bf16>(pending, pending_parts, part_stride, post_w, post_eps, resid, ids, table, add_ids, add_table, add_vec, rows,
                                        w, out, num_rows, H, eps, write_resid, vocab, center, stream);
  return Q3_ERR_ARGUMENT;
}

// ---- clamped gated unit: g = min(gate, limit), u = clamp(up, -limit, limit),
//      out = g * sigmoid(alpha * g) * (u + up_offset); gu rows are [gate (F) | up (F)] ----
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, long total, int F, float limit,
                                   float alpha, float up_offset) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long t = idx / F;
  const int i = (int)(idx - t * F);
  const float g = fminf(to_f32(gu[t * 2 * F + i]), limit);
  const float u = fminf(fmaxf(to_f32(gu[t * 2 * F + F + i]), -limit), limit);
  out[idx] = from_f32<T>((g / (1.f + expf(-alpha * g))) * (u + up_offset));
}

Q3_EXPORT int q3_clamped_glu(int dtype, const void* gu, void* out, int num_rows, int F, float limit, float alpha,
                             float up_offset, cudaStream_t stream) {
  if (!gu || !out || F < 1) return Q3_ERR_ARGUMENT;
  const long total = (long)num_rows * F;
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == Q3_DTYPE_F32)
    clamped_glu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, (float*)out, total, F, limit, alpha, up_offset);
  else if (dtype == Q3_DTYPE_BF16)
    clamped_glu_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)gu, (bf16*)out, total, F, limit, alpha, up_offset);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}

// ---- gated slice of a second embedding: out[t, i] = gelu_tanh(gate[t, i]) * table[ids[t], offset + i] ----
// gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))), in fp32.
template <typename T>
__global__ void gelu_gate_rows_kernel(const T* __restrict__ gate, const int* __restrict__ ids,
                                      const T* __restrict__ table, long table_stride, int offset, int vocab,
                                      T* __restrict__ out, long total, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long t = idx / n;
  const int i = (int)(idx - t * n);
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const float z = to_f32(gate[idx]);
  const float g = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  out[idx] = from_f32<T>(g * to_f32(table[(long)id * table_stride + offset + i]));
}

// gate, out: dense [num_rows, n]; table: [vocab, table_stride] of which columns offset .. offset + n - 1 are read.
Q3_EXPORT int q3_gelu_gate_rows(int dtype, const void* gate, const int* ids, const void* table, long table_stride,
                                int offset, int vocab, void* out, int num_rows, int n, cudaStream_t stream) {
  if (!gate || !ids || !table || !out || n < 1 || offset < 0 || offset + n > table_stride || vocab < 1)
    return Q3_ERR_ARGUMENT;
  const long total = (long)num_rows * n;
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(gelu_gate_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate, ids,
                   (const float*)table, table_stride, offset, vocab, (float*)out, total, n);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(gelu_gate_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gate, ids,
                   (const bf16*)table, table_stride, offset, vocab, (bf16*)out, total, n);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// ---- squared ReLU over the leading columns of a product: out[t, i] = max(x[t, i], 0)^2, i < n ----
// x rows are x_stride apart (a product may carry further columns behind the n, e.g. a gate's logit).
template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ x, long x_stride, T* __restrict__ out, long total, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long t = idx / n;
  const int i = (int)(idx - t * n);
  const float v = fmaxf(to_f32(x[t * x_stride + i]), 0.f);
  out[idx] = from_f32<T>(v * v);
}

// The same with 16-byte accesses: n and x_stride multiples of 8, both pointers 16-byte aligned.
template <typename T>
__global__ void relu_squared_vec_kernel(const T* __restrict__ x, long x_stride, T* __restrict__ out, long chunks,
                                        int n) {
  pdl_wait();
  pdl_launch_dependents();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= chunks) return;
  const int per_row = n / 8;
  const long t = idx / per_row;
  const int i = (int)(idx - t * per_row) * 8;
  float v[8];
  load8(x + t * x_stride + i, v);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float r = fmaxf(v[e], 0.f);
    v[e] = r * r;
  }
  store8(out + t * n + i, v);
}

Q3_EXPORT int q3_relu_squared(int dtype, const void* x, long x_stride, void* out, int num_rows, int n,
                              cudaStream_t stream) {
  if (!x || !out || n < 1 || x_stride < n) return Q3_ERR_ARGUMENT;
  const long total = (long)num_rows * n;
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaError_t e;
  if (n % 8 == 0 && x_stride % 8 == 0 && aligned16(x) && aligned16(out) &&
      (dtype == Q3_DTYPE_F32 || dtype == Q3_DTYPE_BF16)) {
    const long chunks = total / 8;
    const unsigned vblocks = (unsigned)((chunks + 255) / 256);
    if (dtype == Q3_DTYPE_F32)
      e = launch_pdl(relu_squared_vec_kernel<float>, dim3(vblocks), dim3(256), 0, stream, (const float*)x, x_stride,
                     (float*)out, chunks, n);
    else
      e = launch_pdl(relu_squared_vec_kernel<bf16>, dim3(vblocks), dim3(256), 0, stream, (const bf16*)x, x_stride,
                     (bf16*)out, chunks, n);
    return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
  }
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(relu_squared_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, x_stride,
                   (float*)out, total, n);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(relu_squared_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)x, x_stride, (bf16*)out,
                   total, n);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// ---- grouped RMSNorm of a sum with up to two pending outputs and up to two weights ------------------
//   add = (planes summed in order | pending) + more          v = resid[r] + add        (fp32)
//   resid[r] = v                                              (when write_resid)
//   a row is cut into `groups` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps):
//   out[i] = unit(v) * w        out2[i] = unit(v) * w2        (w null: out[i] = v rounded, nothing normalised)
// One block per row; the values wait in shared memory, the groups' mean squares are taken by whole
// warps in turn (a fixed tree per group), so a row's bits do not depend on the rows around it.
template <typename T>
__global__ void grouped_norm_kernel(const void* __restrict__ pending, int parts, long part_stride,
                                    const T* __restrict__ more, float* __restrict__ resid,
                                    const int* __restrict__ rows, const float* __restrict__ w,
                                    const float* __restrict__ w2, T* __restrict__ out, long out_stride,
                                    T* __restrict__ out2, int H, int groups, float eps, int write_resid) {
  extern __shared__ float gvals[];  // H values, then one reciprocal root per group
  float* rstd = gvals + H;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const long src = rows ? rows[r] : r;
  const T* prow = pending && !parts ? static_cast<const T*>(pending) + src * H : nullptr;
  const float* frow = pending && parts ? static_cast<const float*>(pending) + src * H : nullptr;
  const T* mrow = more ? more + src * H : nullptr;
  float* rrow = resid + src * H;
  T* orow = out + (long)r * out_stride;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float add = 0.f;
    bool any = false;
    if (frow) {
      add = frow[i];
      for (int p = 1; p < parts; ++p) add += frow[p * part_stride + i];
      any = true;
    } else if (prow) {
      add = to_f32(prow[i]);
      any = true;
    }
    if (mrow) add = any ? add + to_f32(mrow[i]) : to_f32(mrow[i]);
    const float v = (any || mrow) ? rrow[i] + add : rrow[i];
    if (write_resid) rrow[i] = v;
    if (w) gvals[i] = v; else orow[i] = from_f32<T>(v);
  }
  if (!w) return;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int Hg = H / groups;
  for (int g = warp; g < groups; g += nwarp) {
    float ss = 0.f;
    for (int i = lane; i < Hg; i += 32) {
      const float v = gvals[g * Hg + i];
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) rstd[g] = rsqrtf(ss / (float)Hg + eps);
  }
  __syncthreads();
  T* orow2 = out2 ? out2 + (long)r * H : nullptr;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float u = gvals[i] * rstd[i / Hg];
    orow[i] = from_f32<T>(u * w[i]);
    if (orow2) orow2[i] = from_f32<T>(u * w2[i]);
  }
}

// The same with eight consecutive values a thread and 16-byte accesses (H and a group's size multiples of 8,
// every row 16-byte aligned).  The arithmetic per value and the groups' sums are those of the kernel above.
template <typename T>
__global__ void grouped_norm_kernel_v8(const void* __restrict__ pending, int parts, long part_stride,
                                       const T* __restrict__ more, float* __restrict__ resid,
                                       const int* __restrict__ rows, const float* __restrict__ w,
                                       const float* __restrict__ w2, T* __restrict__ out, long out_stride,
                                       T* __restrict__ out2, int H, int groups, float eps, int write_resid) {
  extern __shared__ __align__(16) float gvals[];
  float* rstd = gvals + H;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const long src = rows ? rows[r] : r;
  const T* prow = pending && !parts ? static_cast<const T*>(pending) + src * H : nullptr;
  const float* frow = pending && parts ? static_cast<const float*>(pending) + src * H : nullptr;
  const T* mrow = more ? more + src * H : nullptr;
  float* rrow = resid + src * H;
  T* orow = out + (long)r * out_stride;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8], a[8];
    load8(rrow + i, v);
    bool any = false;
    if (frow) {
      load8(frow + i, a);
      for (int p = 1; p < parts; ++p) {
        float b[8];
        load8(frow + p * part_stride + i, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] += b[e];
      }
      any = true;
    } else if (prow) {
      load8(prow + i, a);
      any = true;
    }
    if (mrow) {
      float b[8];
      load8(mrow + i, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = any ? a[e] + b[e] : b[e];
      any = true;
    }
    if (any) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = v[e] + a[e];
    }
    if (write_resid) store8(rrow + i, v);
    if (w) store8(gvals + i, v); else store8(orow + i, v);
  }
  if (!w) return;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int Hg = H / groups;
  for (int g = warp; g < groups; g += nwarp) {
    float ss = 0.f;
    for (int i = lane; i < Hg; i += 32) {
      const float v = gvals[g * Hg + i];
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) rstd[g] = rsqrtf(ss / (float)Hg + eps);
  }
  __syncthreads();
  T* orow2 = out2 ? out2 + (long)r * H : nullptr;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8], ww[8], y[8];
    load8(gvals + i, v);
    const float rs = rstd[i / Hg];
    load8(w + i, ww);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[e] = v[e] * rs;
      y[e] = v[e] * ww[e];
    }
    store8(orow + i, y);
    if (orow2) {
      load8(w2 + i, ww);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = v[e] * ww[e];
      store8(orow2 + i, y);
    }
  }
}

// pending: `dtype` [*, H] when pending_parts is 0, else fp32 planes part_stride elements apart (or null);
// more: `dtype` [*, H] or null; resid fp32 [*, H]; out rows out_stride elements apart; out2 dense or null
// (needs w2); w null: out gets the sum itself.
Q3_EXPORT int q3_grouped_norm(int dtype, const void* pending, int pending_parts, long part_stride, const void* more,
                              float* resid, const int* rows, const float* w, const float* w2, void* out,
                              long out_stride, void* out2, int num_rows, int H, int groups, float eps,
                              int write_resid, cudaStream_t stream) {
  if (!resid || !out || H < 1 || groups < 1 || H % groups || out_stride < H) return Q3_ERR_ARGUMENT;
  if ((out2 && !w2) || (w2 && !w) || pending_parts < 0 || (pending_parts && !pending)) return Q3_ERR_ARGUMENT;
  if (num_rows == 0) return Q3_OK;
  const size_t smem = (size_t)(H + groups) * sizeof(float);
  if (smem > 200 * 1024) return Q3_ERR_UNSUPPORTED;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  cudaError_t e;
  const uintptr_t bits = (uintptr_t)pending | (uintptr_t)more | (uintptr_t)resid | (uintptr_t)w | (uintptr_t)w2 |
                         (uintptr_t)out | (uintptr_t)out2;
  const bool wide = H % 8 == 0 && (H / groups) % 8 == 0 && out_stride % 8 == 0 && part_stride % 8 == 0 && !(bits & 15) &&
                    (dtype == Q3_DTYPE_F32 || dtype == Q3_DTYPE_BF16);
  if (wide) {
    const int vthreads = H >= 2048 ? 256 : (H >= 512 ? 64 : 32);
    if (dtype == Q3_DTYPE_F32) {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(grouped_norm_kernel_v8<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      e = launch_pdl(grouped_norm_kernel_v8<float>, dim3(num_rows), dim3(vthreads), smem, stream, pending,
                     pending_parts, part_stride, (const float*)more, resid, rows, w, w2, (float*)out, out_stride,
                     (float*)out2, H, groups, eps, write_resid);
    } else {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(grouped_norm_kernel_v8<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      e = launch_pdl(grouped_norm_kernel_v8<bf16>, dim3(num_rows), dim3(vthreads), smem, stream, pending,
                     pending_parts, part_stride, (const bf16*)more, resid, rows, w, w2, (bf16*)out, out_stride,
                     (bf16*)out2, H, groups, eps, write_resid);
    }
    return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
  }
  if (dtype == Q3_DTYPE_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(grouped_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = launch_pdl(grouped_norm_kernel<float>, dim3(num_rows), dim3(threads), smem, stream, pending, pending_parts,
                   part_stride, (const float*)more, resid, rows, w, w2, (float*)out, out_stride, (float*)out2, H, groups,
                   eps, write_resid);
  } else if (dtype == Q3_DTYPE_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(grouped_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = launch_pdl(grouped_norm_kernel<bf16>, dim3(num_rows), dim3(threads), smem, stream, pending, pending_parts,
                   part_stride, (const bf16*)more, resid, rows, w, w2, (bf16*)out, out_stride, (bf16*)out2, H, groups,
                   eps, write_resid);
  } else {
    return Q3_ERR_ARGUMENT;
  }
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// ---- tanh in place ------------------------------------------------------------------------------------
template <typename T>
__global__ void tanh_rows_kernel(T* __restrict__ x, long total) {
  pdl_wait();
  pdl_launch_dependents();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) x[i] = from_f32<T>(tanhf(to_f32(x[i])));
}

Q3_EXPORT int q3_tanh_rows(int dtype, void* x, long total, cudaStream_t stream) {
  if (!x || total < 0) return Q3_ERR_ARGUMENT;
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32) e = launch_pdl(tanh_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, total);
  else if (dtype == Q3_DTYPE_BF16) e = launch_pdl(tanh_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, total);
  else return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}
