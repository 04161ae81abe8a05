// Routed experts: router scores and choice, grouping of (token, choice) slots by expert on the
// device, the experts' two products over their own slots, and the per-token sum.
//
//   route_top      z = W_router h in fp32, the `top` largest z (the order of their sigmoids; lowest
//                  index on a tie) with sigmoid(z) as weights (optionally divided by their sum), or
//                  with the softmax over the chosen z as weights
//   group_slots    slots sorted by expert: offsets[E + 1], order[S], and for the products the
//                  first row tile of each expert, tile_offsets[E + 1] (tiles of `bm` slots)
//   expert_gate_up mid[slot] = glu(W_gate_e x, W_up_e x), x = h[token] * weight (rounded to the
//                  operand type) when the weight multiplies the expert's input
//                  glu: g = min(g, limit), u = clamp(u, -limit, limit), g * sigmoid(alpha g) * (u + off)
//   expert_up      mid[slot] = relu(W_up_e h[token])^2: the first product of an expert without a gate
//   expert_down    y[slot] = W_down_e mid[slot]
//   combine        out[t] = sum over the token's slots of y (times the weight when it multiplies
//                  the output), plus the shared expert's result (times the sigmoid of a gate logit, if
//                  one is given), summed in fp32 in slot order
//
// Products accumulate in fp32 on the FMA pipes, each output one accumulator over ascending k, so a
// token's result does not depend on which other tokens chose the same expert.  Nothing here reads
// a count back on the host: grids are sized for the worst case and surplus blocks leave at once.
#include "mma_tiles.cuh"

constexpr int EXPERT_BM = 32;  // slots per row tile of the FMA products

// ---- router ------------------------------------------------------------------------------------
// Two kernels.  route_logits: a block stages ROUTE_TT tokens' rows in shared memory as fp32 and each
// of its eight warps streams one expert's router row once for all of them (a step of a few tokens
// still spreads the router over E / 8 blocks).  route_pick: one warp per token takes the `top`
// largest logits -- the choice is made on the logits, which order the experts as their sigmoids do
// but do not collapse into ties where the sigmoid saturates; lowest index on an exact tie -- and
// writes sigmoid(logit) as the weight.
constexpr int ROUTE_TT = 8;

template <typename T>
__global__ void __launch_bounds__(256)
route_logits_kernel(const T* __restrict__ h, long h_stride, const float* __restrict__ router, int num_tokens, int E,
                    int W, int tt, float* __restrict__ logits) {
  extern __shared__ float route_rows[];  // [tt][W], tt <= ROUTE_TT tokens per block
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * tt;
  const int nt = min(tt, num_tokens - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < nt * W; i += 256) {
    const int t = i / W, k = i - t * W;
    route_rows[i] = to_f32(h[(long)(t0 + t) * h_stride + k]);
  }
  __syncthreads();
  const int e = blockIdx.y * 8 + warp;
  if (e >= E) return;
  const float* wr = router + (long)e * W;
  float acc[ROUTE_TT];
#pragma unroll
  for (int t = 0; t < ROUTE_TT; ++t) acc[t] = 0.f;
  if ((W & 3) == 0) {
#pragma unroll 2
    for (int i = lane * 4; i < W; i += 128) {
      const float4 w4 = *reinterpret_cast<const float4*>(wr + i);
#pragma unroll
      for (int t = 0; t < ROUTE_TT; ++t) {
        if (t < nt) {
          const float4 x4 = *reinterpret_cast<const float4*>(route_rows + t * W + i);
          acc[t] = fmaf(x4.x, w4.x, fmaf(x4.y, w4.y, fmaf(x4.z, w4.z, fmaf(x4.w, w4.w, acc[t]))));
        }
      }
    }
  } else {
    for (int i = lane; i < W; i += 32) {
      const float w1 = wr[i];
#pragma unroll
      for (int t = 0; t < ROUTE_TT; ++t)
        if (t < nt) acc[t] = fmaf(route_rows[t * W + i], w1, acc[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < ROUTE_TT; ++t) {
    if (t < nt) {
      const float v = warp_sum(acc[t]);
      if (lane == 0) logits[(long)(t0 + t) * E + e] = v;
    }
  }
}

// mode 0: weights are the chosen logits' sigmoids; 1: those divided by their sum; 2: the softmax over
// the chosen logits only.
__global__ void route_pick_kernel(float* __restrict__ logits, int num_tokens, int E, int top, int mode,
                                  int* __restrict__ chosen, float* __restrict__ weights) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= num_tokens) return;
  float* z = logits + (long)t * E;
  float total = 0.f, first = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < at)) {
        best = v;
        at = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) {
        best = ob;
        at = oa;
      }
    }
    if (k == 0) first = best;  // the largest logit: the softmax's reference point
    const float score = mode == 2 ? expf(best - first) : 1.f / (1.f + expf(-best));
    if (lane == 0) {
      chosen[(long)t * top + k] = at;
      weights[(long)t * top + k] = score;
      z[at] = -INFINITY;  // taken
    }
    total += score;
    __syncwarp();
  }
  if (mode)
    for (int k = lane; k < top; k += 32) weights[(long)t * top + k] /= total;
}

// mode 3: s = softmax over all E logits; the choice is made on c = s + correction (correction null: on s)
// among the outputs of the `keep` best of `count` equal groups of neighbours (a group's score: its largest
// c; count <= 1: no groups), lowest index on a tie; the weights are the chosen s, divided by their sum +
// 1e-20 when `renorm`.  One warp per token; c and the groups' scores wait in shared memory.
__global__ void route_pick_softmax_all_kernel(const float* __restrict__ logits, int num_tokens, int E, int top,
                                              const float* __restrict__ correction, int count, int keep, int renorm,
                                              int* __restrict__ chosen, float* __restrict__ weights) {
  extern __shared__ float pick_smem[];  // per warp: c[E], group scores[count]
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= num_tokens) return;
  const int groups = count > 1 ? count : 0;
  float* c = pick_smem + (long)warp * (E + groups);
  float* gs = c + E;
  const float* z = logits + (long)t * E;
  float zmax = -INFINITY;
  for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
  zmax = warp_max(zmax);
  float den = 0.f;
  for (int e = lane; e < E; e += 32) den += expf(z[e] - zmax);
  den = warp_sum(den);
  for (int e = lane; e < E; e += 32) c[e] = expf(z[e] - zmax) / den + (correction ? correction[e] : 0.f);
  __syncwarp();
  if (groups) {
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, c[e]);
      gs[g] = best;
    }
    __syncwarp();
    // a group stays if fewer than `keep` groups come before it (larger score, or equal and lower index)
    for (int g = lane; g < groups; g += 32) {
      const float mine = gs[g];
      int before = 0;
      for (int o = 0; o < groups; ++o) before += gs[o] > mine || (gs[o] == mine && o < g);
      if (before >= keep)
        for (int e = g * per; e < (g + 1) * per; ++e) c[e] = -INFINITY;
    }
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = c[e];
      if (v > best || (v == best && e < at)) {
        best = v;
        at = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) {
        best = ob;
        at = oa;
      }
    }
    if (at >= E) at = k;  // nothing left to choose from (more choices than open outputs): never read
    const float score = expf(z[at] - zmax) / den;
    if (lane == 0) {
      chosen[(long)t * top + k] = at;
      weights[(long)t * top + k] = score;
      c[at] = NAN;  // taken: compares false with everything
    }
    total += score;
    __syncwarp();
  }
  if (renorm)
    for (int k = lane; k < top; k += 32) weights[(long)t * top + k] /= total + 1e-20f;
}

// logits: fp32 scratch [num_tokens, E] (left with the chosen entries at -inf).
// mode 3 takes correction (fp32 [E] or null), count and keep (groups) and renorm; the other modes ignore them.
Q3_EXPORT int q3_route_top(int dtype, const void* h, long h_stride, const float* router, int num_tokens, int E, int W,
                           int top, int mode, float* logits, int* chosen, float* weights, const float* correction,
                           int count, int keep, int renorm, cudaStream_t stream) {
  if (!h || !router || !logits || !chosen || !weights || E < 1 || W < 1 || top < 1 || top > E) return Q3_ERR_ARGUMENT;
  if (mode == 3 && count > 1 && (E % count || keep < 1 || keep > count || top > keep * (E / count)))
    return Q3_ERR_ARGUMENT;
  if (num_tokens == 0) return Q3_OK;
  int tt = ROUTE_TT;  // fewer tokens per block when their rows would not fit in shared memory
  while (tt > 1 && (size_t)tt * W * sizeof(float) > 128 * 1024) tt >>= 1;
  const size_t smem = (size_t)tt * W * sizeof(float);
  if (smem > 200 * 1024 || (reinterpret_cast<uintptr_t>(router) & 15) || (E + 7) / 8 > 65535) return Q3_ERR_UNSUPPORTED;
  const dim3 grid((num_tokens + tt - 1) / tt, (E + 7) / 8);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(route_logits_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = launch_pdl(route_logits_kernel<float>, grid, dim3(256), smem, stream, (const float*)h, h_stride, router,
                   num_tokens, E, W, tt, logits);
  } else if (dtype == Q3_DTYPE_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(route_logits_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = launch_pdl(route_logits_kernel<bf16>, grid, dim3(256), smem, stream, (const bf16*)h, h_stride, router,
                   num_tokens, E, W, tt, logits);
  } else {
    return Q3_ERR_ARGUMENT;
  }
  if (e != cudaSuccess) return Q3_ERR_LAUNCH;
  if (mode == 3) {
    const size_t pick = (size_t)4 * (E + (count > 1 ? count : 0)) * sizeof(float);
    if (pick > 48 * 1024) return Q3_ERR_UNSUPPORTED;
    e = launch_pdl(route_pick_softmax_all_kernel, dim3((num_tokens + 3) / 4), dim3(128), pick, stream,
                   (const float*)logits, num_tokens, E, top, correction, count, keep, renorm, chosen, weights);
    return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
  }
  e = launch_pdl(route_pick_kernel, dim3((num_tokens + 3) / 4), dim3(128), 0, stream, logits, num_tokens, E, top,
                 mode, chosen, weights);
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// ---- slots grouped by expert ----------------------------------------------------------------------
// One block, for a few hundred slots.  Slots of one expert keep their order (slot s before slot
// s' > s), so the grouping is the same on every run.
__global__ void group_slots_kernel(const int* __restrict__ chosen, int S, int E, int bm, int* __restrict__ offsets,
                                   int* __restrict__ tile_offsets, int* __restrict__ order) {
  extern __shared__ int sm[];  // counts[E], cursor[E]
  int* counts = sm;
  int* cursor = sm + E;
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int s = threadIdx.x; s < S; s += blockDim.x) atomicAdd(&counts[chosen[s]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      tile_offsets[e] = tiles;
      cursor[e] = at;
      at += counts[e];
      tiles += (counts[e] + bm - 1) / bm;
    }
    offsets[E] = at;
    tile_offsets[E] = tiles;
  }
  __syncthreads();
  // a slot's place in its expert's group is the number of earlier slots with the same expert
  for (int s = threadIdx.x; s < S; s += blockDim.x) {
    const int e = chosen[s];
    int rank = 0;
    for (int r = 0; r < s; ++r) rank += chosen[r] == e;
    order[cursor[e] + rank] = s;
  }
}

// The same for many slots: placement by atomic cursor (the order inside an expert's group may then
// differ from run to run; every slot's result is computed on its own, so the outputs do not).
__global__ void group_slots_atomic_kernel(const int* __restrict__ chosen, int S, int E, int bm,
                                          int* __restrict__ offsets, int* __restrict__ tile_offsets,
                                          int* __restrict__ order) {
  extern __shared__ int sm[];
  int* counts = sm;
  int* cursor = sm + E;
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int s = threadIdx.x; s < S; s += blockDim.x) atomicAdd(&counts[chosen[s]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      tile_offsets[e] = tiles;
      cursor[e] = at;
      at += counts[e];
      tiles += (counts[e] + bm - 1) / bm;
    }
    offsets[E] = at;
    tile_offsets[E] = tiles;
  }
  __syncthreads();
  for (int s = threadIdx.x; s < S; s += blockDim.x) order[atomicAdd(&cursor[chosen[s]], 1)] = s;
}

// bm: slots per row tile of the products that will use tile_offsets (EXPERT_BM for the FMA kernels).
Q3_EXPORT int q3_group_slots(const int* chosen, int S, int E, int bm, int* offsets, int* tile_offsets, int* order,
                             cudaStream_t stream) {
  if (!chosen || !offsets || !tile_offsets || !order || E < 1 || S < 0 || bm < 1) return Q3_ERR_ARGUMENT;
  if (E > 8192) return Q3_ERR_UNSUPPORTED;
  const size_t smem = 2 * (size_t)E * sizeof(int);
  cudaError_t e;
  if (S <= 512)
    e = launch_pdl(group_slots_kernel, dim3(1), dim3(512), smem, stream, chosen, S, E, bm, offsets, tile_offsets,
                   order);
  else
    e = launch_pdl(group_slots_atomic_kernel, dim3(1), dim3(1024), smem, stream, chosen, S, E, bm, offsets,
                   tile_offsets, order);
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// ---- the experts' products ------------------------------------------------------------------------
__device__ __forceinline__ int expert_of_tile(const int* __restrict__ tile_offsets, int E, int tile) {
  int lo = 0, hi = E;  // the last e with tile_offsets[e] <= tile
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_offsets[mid] <= tile) lo = mid; else hi = mid;
  }
  return lo;
}

// GATE_UP: A rows are h[token(slot)] (times the slot's weight when scale_input), B is the expert's
// [2F, W] (gate rows, then up rows), the result mid[slot, F].  Else: A rows are A[slot / top] (top = 1:
// a row per slot, the second product; top = the choices per token: the token's row, a first product
// without a gate), B is the expert's [N, K], the result C[slot, N]; scale_input then stands for the
// activation: 0 none, 1 the squared ReLU of the rounded product.
template <typename T, bool GATE_UP>
__global__ void __launch_bounds__(256)
expert_gemm_kernel(const T* __restrict__ A, long a_stride, const T* __restrict__ B, T* __restrict__ C, int N, int K,
                   const int* __restrict__ offsets, const int* __restrict__ tile_offsets,
                   const int* __restrict__ order, const float* __restrict__ weights, int E, int top,
                   int scale_input, float limit, float alpha, float up_offset) {
  constexpr int BM = EXPERT_BM, BN = 64, BK = 16, TM = 2, TN = 4, THREADS = 256;
  constexpr int NB = GATE_UP ? 2 : 1;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[NB][BK][BN + 4];
  __shared__ int slot_of[BM];
  __shared__ float scale_of[BM];
  pdl_wait();
  pdl_launch_dependents();
  const int tile = blockIdx.y;
  if (tile >= tile_offsets[E]) return;
  const int e = expert_of_tile(tile_offsets, E, tile);
  const int row0 = offsets[e] + (tile - tile_offsets[e]) * BM;
  const int rows = min(BM, offsets[e + 1] - row0);
  const int tid = threadIdx.x;
  if (tid < BM) {
    const int slot = tid < rows ? order[row0 + tid] : -1;
    slot_of[tid] = slot;
    scale_of[tid] = (slot >= 0 && GATE_UP && scale_input) ? weights[slot] : 1.f;
  }
  __syncthreads();
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int n0 = blockIdx.x * BN;
  const T* Be = B + (long)e * (GATE_UP ? 2 : 1) * N * K;
  float acc[NB][TM][TN];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[b][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int x = tid; x < BM * BK; x += THREADS) {
      const int r = x / BK, c = x % BK;
      const int slot = slot_of[r], gk = k0 + c;
      float a = 0.f;
      if (slot >= 0 && gk < K) {
        const long arow = slot / top;
        a = to_f32(A[arow * a_stride + gk]);
        if (GATE_UP && scale_input) a = to_f32(from_f32<T>(a * scale_of[r]));
      }
      As[c][r] = a;
    }
    for (int x = tid; x < NB * BN * BK; x += THREADS) {
      const int b = x / (BN * BK), y = x % (BN * BK);
      const int r = y / BK, c = y % BK;
      const int gn = n0 + r, gk = k0 + c;
      Ws[b][c][r] = (gn < N && gk < K) ? to_f32(Be[((long)b * N + gn) * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float w[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j) w[j] = Ws[b][kk][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[b][i][j] = fmaf(a[i], w[j], acc[b][i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int slot = slot_of[ty * TM + i];
    if (slot < 0) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      if (GATE_UP) {
        // both products are rounded to the operand type before the gated unit, as two separate
        // products followed by an activation kernel would
        const float g = fminf(to_f32(from_f32<T>(acc[0][i][j])), limit);
        const float u = fminf(fmaxf(to_f32(from_f32<T>(acc[NB - 1][i][j])), -limit), limit);
        C[(long)slot * N + gn] = from_f32<T>((g / (1.f + expf(-alpha * g))) * (u + up_offset));
      } else if (scale_input) {
        const float r = fmaxf(to_f32(from_f32<T>(acc[0][i][j])), 0.f);
        C[(long)slot * N + gn] = from_f32<T>(r * r);
      } else {
        C[(long)slot * N + gn] = from_f32<T>(acc[0][i][j]);
      }
    }
  }
}

// h: [T, W] rows h_stride apart; gate_up: [E, 2F, W]; mid: [S, F]; S = T * top slots.
Q3_EXPORT int q3_expert_gate_up(int dtype, const void* h, long h_stride, const void* gate_up, void* mid, int S, int E,
                                int F, int W, int top, const int* offsets, const int* tile_offsets, const int* order,
                                const float* weights, int scale_input, float limit, float alpha, float up_offset,
                                cudaStream_t stream) {
  if (!h || !gate_up || !mid || !offsets || !tile_offsets || !order || !weights) return Q3_ERR_ARGUMENT;
  if (E < 1 || F < 1 || W < 1 || top < 1) return Q3_ERR_ARGUMENT;
  if (S == 0) return Q3_OK;
  const int tiles = S / EXPERT_BM + (E < S ? E : S);
  if (tiles > 65535) return Q3_ERR_UNSUPPORTED;
  const dim3 grid((F + 63) / 64, tiles);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(expert_gemm_kernel<float, true>, grid, dim3(256), 0, stream, (const float*)h, h_stride,
                   (const float*)gate_up, (float*)mid, F, W, offsets, tile_offsets, order, weights, E, top, scale_input,
                   limit, alpha, up_offset);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(expert_gemm_kernel<bf16, true>, grid, dim3(256), 0, stream, (const bf16*)h, h_stride,
                   (const bf16*)gate_up, (bf16*)mid, F, W, offsets, tile_offsets, order, weights, E, top, scale_input,
                   limit, alpha, up_offset);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// mid: [S, F]; down: [E, W, F]; y: [S, W].
Q3_EXPORT int q3_expert_down(int dtype, const void* mid, const void* down, void* y, int S, int E, int F, int W,
                             const int* offsets, const int* tile_offsets, const int* order, cudaStream_t stream) {
  if (!mid || !down || !y || !offsets || !tile_offsets || !order || E < 1 || F < 1 || W < 1) return Q3_ERR_ARGUMENT;
  if (S == 0) return Q3_OK;
  const int tiles = S / EXPERT_BM + (E < S ? E : S);
  if (tiles > 65535) return Q3_ERR_UNSUPPORTED;
  const dim3 grid((W + 63) / 64, tiles);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(expert_gemm_kernel<float, false>, grid, dim3(256), 0, stream, (const float*)mid, (long)F,
                   (const float*)down, (float*)y, W, F, offsets, tile_offsets, order, (const float*)nullptr, E, 1, 0,
                   0.f, 0.f, 0.f);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(expert_gemm_kernel<bf16, false>, grid, dim3(256), 0, stream, (const bf16*)mid, (long)F,
                   (const bf16*)down, (bf16*)y, W, F, offsets, tile_offsets, order, (const float*)nullptr, E, 1, 0, 0.f,
                   0.f, 0.f);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// An expert's first product without a gate: mid[slot] = act(W_up_e h[token(slot)]); up: [E, F, W].
// act 1: the squared ReLU.
Q3_EXPORT int q3_expert_up(int dtype, const void* h, long h_stride, const void* up, void* mid, int S, int E, int F,
                           int W, int top, const int* offsets, const int* tile_offsets, const int* order, int act,
                           cudaStream_t stream) {
  if (!h || !up || !mid || !offsets || !tile_offsets || !order || E < 1 || F < 1 || W < 1 || top < 1)
    return Q3_ERR_ARGUMENT;
  if (S == 0) return Q3_OK;
  const int tiles = S / EXPERT_BM + (E < S ? E : S);
  if (tiles > 65535) return Q3_ERR_UNSUPPORTED;
  const dim3 grid((F + 63) / 64, tiles);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(expert_gemm_kernel<float, false>, grid, dim3(256), 0, stream, (const float*)h, h_stride,
                   (const float*)up, (float*)mid, F, W, offsets, tile_offsets, order, (const float*)nullptr, E, top,
                   act, 0.f, 0.f, 0.f);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(expert_gemm_kernel<bf16, false>, grid, dim3(256), 0, stream, (const bf16*)h, h_stride,
                   (const bf16*)up, (bf16*)mid, F, W, offsets, tile_offsets, order, (const float*)nullptr, E, top, act,
                   0.f, 0.f, 0.f);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// ---- the same products on the tensor cores (bfloat16, mma.sync m16n8k16) ---------------------------
// A block owns BM slots of one expert and 64 output columns (of gate and of up for GATE_UP); four
// warps, WM = BM / 32 of them along the slots.  The slots' rows are gathered (and, for GATE_UP with
// the weight on the input, multiplied by it and rounded to bfloat16) into shared memory, the
// expert's rows come by cp.async through a ring of three stages, 32 of the inner dimension at a
// time, while the slots' rows of the step after next are already in registers.  K is a multiple of 8
// and all rows are 16-byte aligned.
template <bool GATE_UP, int BM>
__global__ void __launch_bounds__(128)
expert_gemm_tc_kernel(const bf16* __restrict__ A, long a_stride, const bf16* __restrict__ B, bf16* __restrict__ C,
                      int N, int K, const int* __restrict__ offsets, const int* __restrict__ tile_offsets,
                      const int* __restrict__ order, const float* __restrict__ weights, int E, int top,
                      int scale_input, float limit, float alpha, float up_offset) {
  constexpr int BN = 64, BK = 32, KS = BK + 8, NB = GATE_UP ? 2 : 1, STAGES = 3;
  constexpr int WM = BM / 32, WN = 4 / WM, COLS = BN / WN, NTW = COLS / 8;
  constexpr int A_CHUNKS = BM * (BK / 8) / 128;  // 16-byte chunks of the slots' rows per thread and step
  extern __shared__ __align__(16) unsigned char expert_smem[];
  typedef bf16 (*WTile)[BN][KS];
  typedef bf16 (*ATile)[KS];
  bf16* w_base = reinterpret_cast<bf16*>(expert_smem);             // [STAGES][NB][BN][KS]
  bf16* a_base = w_base + STAGES * NB * BN * KS;                   // [2][BM][KS]
  __shared__ int slot_of[BM];
  __shared__ float scale_of[BM];
  pdl_wait();
  pdl_launch_dependents();
  const int tile = blockIdx.y;
  if (tile >= tile_offsets[E]) return;
  const int e = expert_of_tile(tile_offsets, E, tile);
  const int row0 = offsets[e] + (tile - tile_offsets[e]) * BM;
  const int rows = min(BM, offsets[e + 1] - row0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int r = tid; r < BM; r += 128) {
    const int slot = r < rows ? order[row0 + r] : -1;
    slot_of[r] = slot;
    scale_of[r] = (slot >= 0 && GATE_UP && scale_input) ? weights[slot] : 1.f;
  }
  __syncthreads();
  const int wm = warp / WN, wn = warp % WN;
  const int n0 = blockIdx.x * BN;
  const bf16* Be = B + (long)e * NB * N * K;
  const int steps = (K + BK - 1) / BK;

  // the expert's rows of step s into ring stage s % STAGES (one commit group per call, also when empty)
  auto load_w = [&](int s) {
    if (s < steps) {
      WTile Ws = reinterpret_cast<WTile>(w_base + (s % STAGES) * NB * BN * KS);
      const int k0 = s * BK;
      for (int c = tid; c < NB * BN * (BK / 8); c += 128) {
        const int b = c / (BN * (BK / 8)), y = c % (BN * (BK / 8));
        const int r = y / (BK / 8), ch = y % (BK / 8);
        const int gn = n0 + r, gk = k0 + ch * 8;
        const bool in = gn < N && gk < K;
        cp_async16(smem_u32(&Ws[b][r][ch * 8]), in ? Be + ((long)b * N + gn) * K + gk : Be, in ? 16 : 0);
      }
    }
    cp_async_commit();
  };
  // the slots' rows of step s into registers (gathered, and scaled where the weight is on the input)
  uint4 a_regs[A_CHUNKS];
  auto fetch_a = [&](int s) {
#pragma unroll
    for (int i = 0; i < A_CHUNKS; ++i) {
      const int c = tid + i * 128;
      const int r = c / (BK / 8), ch = c % (BK / 8);
      const int slot = slot_of[r], gk = s * BK + ch * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (s < steps && slot >= 0 && gk < K) {
        const long arow = slot / top;
        v = *reinterpret_cast<const uint4*>(A + arow * a_stride + gk);
        if (GATE_UP && scale_input) {
          __nv_bfloat162* hv = reinterpret_cast<__nv_bfloat162*>(&v);
          const float w = scale_of[r];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const float2 f = __bfloat1622float2(hv[x]);
            hv[x] = __floats2bfloat162_rn(f.x * w, f.y * w);
          }
        }
      }
      a_regs[i] = v;
    }
  };
  auto store_a = [&](int s) {
    ATile As = reinterpret_cast<ATile>(a_base + (s & 1) * BM * KS);
#pragma unroll
    for (int i = 0; i < A_CHUNKS; ++i) {
      const int c = tid + i * 128;
      *reinterpret_cast<uint4*>(&As[c / (BK / 8)][(c % (BK / 8)) * 8]) = a_regs[i];
    }
  };

  float acc[NB][2][NTW][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[b][mt][nt][x] = 0.f;
  load_w(0);
  load_w(1);
  fetch_a(0);
  store_a(0);
  fetch_a(1);
  for (int s = 0; s < steps; ++s) {
    cp_async_wait<1>();  // the weights of step s have landed (those of s + 1 may still be on their way)
    __syncthreads();     // ... for every thread; rows of step s are stored; step s - 1 has been used up
    load_w(s + 2);       // into the stage step s - 1 used
    store_a(s + 1);      // into the buffer step s - 1 used
    fetch_a(s + 2);
    WTile Ws = reinterpret_cast<WTile>(w_base + (s % STAGES) * NB * BN * KS);
    ATile As = reinterpret_cast<ATile>(a_base + (s & 1) * BM * KS);
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        ldmatrix_x4(a[mt], smem_u32(&As[wm * 32 + mt * 16 + (lane & 15)][kk + (lane >> 4) * 8]));
#pragma unroll
      for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int np = 0; np < NTW / 2; ++np) {
          uint32_t bb[4];
          ldmatrix_x4(bb, smem_u32(&Ws[b][wn * COLS + np * 16 + (lane >> 4) * 8 + (lane & 7)][kk + ((lane >> 3) & 1) * 8]));
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            mma_bf16(acc[b][mt][2 * np], a[mt], bb[0], bb[1]);
            mma_bf16(acc[b][mt][2 * np + 1], a[mt], bb[2], bb[3]);
          }
        }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int slot = slot_of[wm * 32 + mt * 16 + half * 8 + (lane >> 2)];
      if (slot < 0) continue;
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int gn = n0 + wn * COLS + nt * 8 + 2 * (lane & 3) + x;
          if (gn >= N) continue;
          if (GATE_UP) {
            const float g = fminf(to_f32(from_f32<bf16>(acc[0][mt][nt][2 * half + x])), limit);
            const float u = fminf(fmaxf(to_f32(from_f32<bf16>(acc[NB - 1][mt][nt][2 * half + x])), -limit), limit);
            C[(long)slot * N + gn] = from_f32<bf16>((g / (1.f + expf(-alpha * g))) * (u + up_offset));
          } else if (scale_input) {
            const float r = fmaxf(to_f32(from_f32<bf16>(acc[0][mt][nt][2 * half + x])), 0.f);
            C[(long)slot * N + gn] = from_f32<bf16>(r * r);
          } else {
            C[(long)slot * N + gn] = from_f32<bf16>(acc[0][mt][nt][2 * half + x]);
          }
        }
    }
}

template <bool GATE_UP, int BM>
static constexpr size_t expert_tc_smem() {
  return (size_t)(3 * (GATE_UP ? 2 : 1) * 64 * 40 + 2 * BM * 40) * sizeof(bf16);
}

// The two products as above for bfloat16 with rows of 16-byte multiples; bm (32 or 64) is the row
// tile that group_slots was given.
Q3_EXPORT int q3_expert_gate_up_tc(const void* h, long h_stride, const void* gate_up, void* mid, int S, int E, int F,
                                   int W, int top, int bm, const int* offsets, const int* tile_offsets,
                                   const int* order, const float* weights, int scale_input, float limit, float alpha,
                                   float up_offset, cudaStream_t stream) {
  if (!h || !gate_up || !mid || !offsets || !tile_offsets || !order || !weights) return Q3_ERR_ARGUMENT;
  if (E < 1 || F < 1 || W < 1 || top < 1 || (bm != 32 && bm != 64)) return Q3_ERR_ARGUMENT;
  if (W % 8 || h_stride % 8 || (reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(gate_up) & 15))
    return Q3_ERR_UNSUPPORTED;
  if (S == 0) return Q3_OK;
  const int tiles = S / bm + (E < S ? E : S);
  if (tiles > 65535) return Q3_ERR_UNSUPPORTED;
  const dim3 grid((F + 63) / 64, tiles);
  auto kernel = bm == 64 ? expert_gemm_tc_kernel<true, 64> : expert_gemm_tc_kernel<true, 32>;
  const size_t smem = bm == 64 ? expert_tc_smem<true, 64>() : expert_tc_smem<true, 32>();
  return launch_pdl(kernel, grid, dim3(128), smem, stream, (const bf16*)h, h_stride, (const bf16*)gate_up, (bf16*)mid, F,
                    W, offsets, tile_offsets, order, weights, E, top, scale_input, limit, alpha, up_offset) == cudaSuccess
             ? Q3_OK
             : Q3_ERR_LAUNCH;
}

Q3_EXPORT int q3_expert_down_tc(const void* mid, const void* down, void* y, int S, int E, int F, int W, int bm,
                                const int* offsets, const int* tile_offsets, const int* order, cudaStream_t stream) {
  if (!mid || !down || !y || !offsets || !tile_offsets || !order || E < 1 || F < 1 || W < 1) return Q3_ERR_ARGUMENT;
  if (bm != 32 && bm != 64) return Q3_ERR_ARGUMENT;
  if (F % 8 || (reinterpret_cast<uintptr_t>(mid) & 15) || (reinterpret_cast<uintptr_t>(down) & 15))
    return Q3_ERR_UNSUPPORTED;
  if (S == 0) return Q3_OK;
  const int tiles = S / bm + (E < S ? E : S);
  if (tiles > 65535) return Q3_ERR_UNSUPPORTED;
  const dim3 grid((W + 63) / 64, tiles);
  auto kernel = bm == 64 ? expert_gemm_tc_kernel<false, 64> : expert_gemm_tc_kernel<false, 32>;
  const size_t smem = bm == 64 ? expert_tc_smem<false, 64>() : expert_tc_smem<false, 32>();
  return launch_pdl(kernel, grid, dim3(128), smem, stream, (const bf16*)mid, (long)F, (const bf16*)down, (bf16*)y, W, F,
                    offsets, tile_offsets, order, (const float*)nullptr, E, 1, 0, 0.f, 0.f, 0.f) == cudaSuccess
             ? Q3_OK
             : Q3_ERR_LAUNCH;
}

Q3_EXPORT int q3_expert_up_tc(const void* h, long h_stride, const void* up, void* mid, int S, int E, int F, int W,
                              int top, int bm, const int* offsets, const int* tile_offsets, const int* order, int act,
                              cudaStream_t stream) {
  if (!h || !up || !mid || !offsets || !tile_offsets || !order || E < 1 || F < 1 || W < 1 || top < 1)
    return Q3_ERR_ARGUMENT;
  if (bm != 32 && bm != 64) return Q3_ERR_ARGUMENT;
  if (W % 8 || h_stride % 8 || (reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(up) & 15))
    return Q3_ERR_UNSUPPORTED;
  if (S == 0) return Q3_OK;
  const int tiles = S / bm + (E < S ? E : S);
  if (tiles > 65535) return Q3_ERR_UNSUPPORTED;
  const dim3 grid((F + 63) / 64, tiles);
  auto kernel = bm == 64 ? expert_gemm_tc_kernel<false, 64> : expert_gemm_tc_kernel<false, 32>;
  const size_t smem = bm == 64 ? expert_tc_smem<false, 64>() : expert_tc_smem<false, 32>();
  return launch_pdl(kernel, grid, dim3(128), smem, stream, (const bf16*)h, h_stride, (const bf16*)up, (bf16*)mid, F, W,
                    offsets, tile_offsets, order, (const float*)nullptr, E, top, act, 0.f, 0.f, 0.f) == cudaSuccess
             ? Q3_OK
             : Q3_ERR_LAUNCH;
}

// ---- per-token sum ----------------------------------------------------------------------------------
template <typename T>
__global__ void combine_kernel(const T* __restrict__ y, const float* __restrict__ weights, const T* __restrict__ shared,
                               const T* __restrict__ shared_gate, long gate_stride, T* __restrict__ out, long total,
                               int W, int top, const int* __restrict__ chosen, int stored, const T* __restrict__ h,
                               long h_stride) {
  pdl_wait();
  pdl_launch_dependents();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long t = idx / W;
  const int i = (int)(idx - t * W);
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    // a choice beyond the stored experts stands for an expert that returns its input
    const bool same = chosen && chosen[t * top + k] >= stored;
    const float v = same ? to_f32(h[t * h_stride + i]) : to_f32(y[(t * top + k) * W + i]);
    sum += weights ? v * weights[t * top + k] : v;
  }
  if (shared) {
    const float v = to_f32(shared[idx]);
    sum += shared_gate ? v / (1.f + expf(-to_f32(shared_gate[t * gate_stride]))) : v;
  }
  out[idx] = from_f32<T>(sum);
}

// y: [T * top, W]; weights: fp32 [T * top] or null (the weight was applied to the input);
// shared: [T, W] or null; shared_gate: one logit per token, gate_stride elements apart, or null: the
// shared expert's result is multiplied by the logit's sigmoid; out: [T, W].  chosen (int32 [T * top], with
// h [T, W] rows h_stride apart, or null): a slot whose choice is >= `stored` takes the token's row of h in
// place of y.
Q3_EXPORT int q3_expert_combine(int dtype, const void* y, const float* weights, const void* shared,
                                const void* shared_gate, long gate_stride, void* out, int num_tokens, int W, int top,
                                const int* chosen, int stored, const void* h, long h_stride, cudaStream_t stream) {
  if (!y || !out || W < 1 || top < 1 || (chosen && !h)) return Q3_ERR_ARGUMENT;
  const long total = (long)num_tokens * W;
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(combine_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)y, weights,
                   (const float*)shared, (const float*)shared_gate, gate_stride, (float*)out, total, W, top, chosen,
                   stored, (const float*)h, h_stride);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(combine_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)y, weights,
                   (const bf16*)shared, (const bf16*)shared_gate, gate_stride, (bf16*)out, total, W, top, chosen,
                   stored, (const bf16*)h, h_stride);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}
