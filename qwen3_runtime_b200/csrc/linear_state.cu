// Linear attention with a decayed matrix state per (sequence, head), kept in fp32 in a state slot:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t        S: [D, Dv]
//
// a_t is a decay per key channel.  It comes either from logits, a_t[i] = sigmoid(z_t[i] + b[i])^(1 / tau)
// (gated linear attention), or is one constant per head (retention).  q and k may be rotated first
// (pairs (i, i + pairs) of a head turn by position * inv_freq[i]) and are multiplied by q_scale and
// k_scale; decays, angles, the state and the products with it are fp32, q, k, v and z arrive in the
// activation type.  Further forms of the same recurrence: the decay exp(-exp(z_t[i] + b[i])) per key
// channel (decay_mode 1); a decay and a factor on k given per (token, head) as fp32 numbers (gates worked
// out beforehand); a last value column whose value is 1 for every token (ones_col: the state then also
// carries the decayed sum of the keys, and o's last column is that sum times q); and a bonus u per key
// channel with which the present token counts while the state is read before its update,
//   o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t        S_t = diag(a_t) S_(t-1) + k_t v_t^T.
//
// stabilised_gates: the gates of a matrix memory with exponential input and forget gates, kept in range
// by a running maximum m per (sequence, head) (fp32, in a state slot, 0 at the start):
//   li = cap tanh((zi + bi) / cap)   lf = logsigmoid(cap tanh((zf + bf) / cap))   m_t = max(lf + m_(t-1), li)
//   decay_t = exp(lf + m_(t-1) - m_t)        k_scale_t = exp(li - m_t)
//
// decayed_state_scan: one block per (32 value columns, head, sequence).  A thread owns eight key
// rows of one value column of the state and keeps them in registers from the sequence's first token
// of the step to its last; the row groups of a column are neighbouring lanes of one warp, so a
// token's output is a shuffle sum over them (a fixed tree) and warps never wait for one another
// inside a chunk.  Tokens come 16 at a time: while the threads run the updates of one chunk from
// shared memory (q, k and decay rows as fp32, already rotated and scaled), the next chunk's raw
// values are already on their way into registers; they are turned into fp32 rows in the other half
// of the double buffer afterwards.  A token's arithmetic does not depend on where the step's portion
// starts or ends, so the result has the same bits however a prompt is cut.
//
// head_norm_gate: y[t, h, :] = o / sqrt(mean(o^2) + eps) * w * silu(g[t, h, :]) * out_scale, one warp
// per (token, head); w may be absent.
#include "common.cuh"

#define SCAN_CT 16  // tokens per chunk

// SCAN_R key rows per thread, SCAN_VT value columns per block; RGP2: row groups per value column (a
// power of two, 4..32): the block holds RGP2 * SCAN_R >= D key rows.  Four rows a thread and 16
// columns a block (key sizes up to 128) make four times as many warps as eight and 32 do: a single
// prompt's scan is a chain of dependent steps whose latencies only other warps can fill.
template <typename T, int RGP2, int SCAN_R, int SCAN_VT, bool BONUS>
__global__ void __launch_bounds__(SCAN_VT * RGP2)
decayed_state_scan_kernel(const T* __restrict__ q, long q_stride, const T* __restrict__ k, long k_stride,
                          const T* __restrict__ v, long v_stride, const T* __restrict__ z, long z_stride,
                          const float* __restrict__ z_bias, float inv_tau, const float* __restrict__ head_decay,
                          const float* __restrict__ inv_freq, int rot_pairs, const int* __restrict__ positions,
                          float q_scale, float k_scale, float* __restrict__ state,
                          const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                          float* __restrict__ out, int H, int D, int Dv, int decay_mode,
                          const float* __restrict__ tok_decay, const float* __restrict__ tok_kscale, int ones_col,
                          const float* __restrict__ bonus) {
  constexpr int THREADS = SCAN_VT * RGP2, DP = RGP2 * SCAN_R, CPW = 32 / RGP2;  // columns per warp
  constexpr int EPT = SCAN_CT * DP / THREADS;                              // row elements per thread and chunk: 4
  constexpr int VPT = (SCAN_CT * SCAN_VT + THREADS - 1) / THREADS;         // value elements per thread and chunk
  extern __shared__ __align__(16) float scan_smem[];
  typedef float (*Rows)[SCAN_CT][DP];
  typedef float (*Vals)[SCAN_CT][SCAN_VT];
  Rows qs = reinterpret_cast<Rows>(scan_smem);                    // [2][CT][DP]
  Rows ks = reinterpret_cast<Rows>(scan_smem + 2 * SCAN_CT * DP);
  Rows as = reinterpret_cast<Rows>(scan_smem + 4 * SCAN_CT * DP);
  Vals vs = reinterpret_cast<Vals>(scan_smem + 6 * SCAN_CT * DP);  // [2][CT][VT]
  float (*os)[SCAN_VT] = reinterpret_cast<float (*)[SCAN_VT]>(scan_smem + 6 * SCAN_CT * DP + 2 * SCAN_CT * SCAN_VT);
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = lane % RGP2, col = warp * CPW + lane / RGP2;
  const int h = blockIdx.y, b = blockIdx.z;
  const int j = blockIdx.x * SCAN_VT + col;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const long slot = state_slots[b];
  float* Sg = state + ((slot * H + h) * (long)D) * Dv;
  float S[SCAN_R];
#pragma unroll
  for (int r = 0; r < SCAN_R; ++r) {
    const int i = rg * SCAN_R + r;
    S[r] = (i < D && j < Dv) ? Sg[(long)i * Dv + j] : 0.f;
  }
  const float decay_h = head_decay ? head_decay[h] : 1.f;
  const int Dvin = Dv - ones_col;  // value columns that v brings; the column after them holds ones
  float U[SCAN_R];
#pragma unroll
  for (int r = 0; r < SCAN_R; ++r) {
    const int i = rg * SCAN_R + r;
    U[r] = (BONUS && i < D) ? bonus[h * D + i] : 0.f;
  }

  // what a thread fetches of a chunk: EPT elements of the q, k (and logit) rows, their rotation
  // partners, VPT values
  T qr[EPT], kr[EPT], zr[EPT], qo[EPT], ko[EPT], vr[VPT];
  auto fetch = [&](int c0) {
#pragma unroll
    for (int m = 0; m < EPT; ++m) {
      const int x = tid + m * THREADS, c = x / DP, i = x - c * DP;
      const long t = c0 + c;
      const bool live = t < t1 && i < D;
      qr[m] = live ? q[t * q_stride + h * D + i] : from_f32<T>(0.f);
      kr[m] = live ? k[t * k_stride + h * D + i] : from_f32<T>(0.f);
      zr[m] = (live && z) ? z[t * z_stride + h * D + i] : from_f32<T>(0.f);
      if (live && i < 2 * rot_pairs) {
        const int other = i < rot_pairs ? i + rot_pairs : i - rot_pairs;
        qo[m] = q[t * q_stride + h * D + other];
        ko[m] = k[t * k_stride + h * D + other];
      }
    }
#pragma unroll
    for (int m = 0; m < VPT; ++m) {
      const int x = tid + m * THREADS, c = x / SCAN_VT, jj = blockIdx.x * SCAN_VT + (x % SCAN_VT);
      const long t = c0 + c;
      vr[m] = (x < SCAN_CT * SCAN_VT && t < t1 && jj < Dvin) ? v[t * v_stride + h * Dvin + jj]
                                                            : from_f32<T>((t < t1 && jj < Dv) ? 1.f : 0.f);
    }
  };
  // turn what was fetched into the fp32 rows of buffer `buf`: rows beyond D and tokens beyond the
  // portion are zero (their state stays zero and adds nothing)
  auto stage = [&](int c0, int buf) {
#pragma unroll
    for (int m = 0; m < EPT; ++m) {
      const int x = tid + m * THREADS, c = x / DP, i = x - c * DP;
      const long t = c0 + c;
      float qv = 0.f, kv = 0.f, av = 0.f;
      if (t < t1 && i < D) {
        qv = to_f32(qr[m]);
        kv = to_f32(kr[m]);
        if (i < 2 * rot_pairs) {
          const int pair = i < rot_pairs ? i : i - rot_pairs;
          float sn, cs;
          sincosf((float)positions[t] * inv_freq[pair], &sn, &cs);
          const float qp = to_f32(qo[m]), kp = to_f32(ko[m]);
          // first of a pair: u cos - v sin; second: v cos + u sin
          qv = i < rot_pairs ? qv * cs - qp * sn : qv * cs + qp * sn;
          kv = i < rot_pairs ? kv * cs - kp * sn : kv * cs + kp * sn;
        }
        qv *= q_scale;
        kv *= k_scale;
        if (tok_kscale) kv *= tok_kscale[t * H + h];
        if (z) {
          const float zz = to_f32(zr[m]) + (z_bias ? z_bias[h * D + i] : 0.f);
          if (decay_mode == 1) {
            av = expf(-expf(zz));
          } else {
            const float log_sig = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));
            av = expf(log_sig * inv_tau);
          }
        } else {
          av = tok_decay ? tok_decay[t * H + h] : decay_h;
        }
      }
      qs[buf][c][i] = qv;
      ks[buf][c][i] = kv;
      as[buf][c][i] = av;
    }
#pragma unroll
    for (int m = 0; m < VPT; ++m) {
      const int x = tid + m * THREADS;
      if (x < SCAN_CT * SCAN_VT) vs[buf][x / SCAN_VT][x % SCAN_VT] = to_f32(vr[m]);
    }
  };

  fetch(t0);
  stage(t0, 0);
  __syncthreads();
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += SCAN_CT, buf ^= 1) {
    const int n = min(SCAN_CT, t1 - c0);
    const bool more = c0 + SCAN_CT < t1;
    if (more) fetch(c0 + SCAN_CT);  // in flight while this chunk is computed
    const int i0 = rg * SCAN_R;
    // one token's update of this thread's rows; returns its share of the token's output
    auto update = [&](int c) -> float {
      const float vj = vs[buf][c][col];
      const float4* a4 = reinterpret_cast<const float4*>(&as[buf][c][i0]);
      const float4* k4 = reinterpret_cast<const float4*>(&ks[buf][c][i0]);
      const float4* q4 = reinterpret_cast<const float4*>(&qs[buf][c][i0]);
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int g = 0; g < SCAN_R / 4; ++g) {
        const float4 a = a4[g], kk = k4[g], qq = q4[g];
        if (BONUS) {  // the output reads the state before its update, the present token through the bonus
          const float p0 = kk.x * vj, p1 = kk.y * vj, p2 = kk.z * vj, p3 = kk.w * vj;
          acc0 = fmaf(fmaf(U[4 * g + 0], p0, S[4 * g + 0]), qq.x, acc0);
          acc1 = fmaf(fmaf(U[4 * g + 1], p1, S[4 * g + 1]), qq.y, acc1);
          acc0 = fmaf(fmaf(U[4 * g + 2], p2, S[4 * g + 2]), qq.z, acc0);
          acc1 = fmaf(fmaf(U[4 * g + 3], p3, S[4 * g + 3]), qq.w, acc1);
          S[4 * g + 0] = fmaf(a.x, S[4 * g + 0], p0);
          S[4 * g + 1] = fmaf(a.y, S[4 * g + 1], p1);
          S[4 * g + 2] = fmaf(a.z, S[4 * g + 2], p2);
          S[4 * g + 3] = fmaf(a.w, S[4 * g + 3], p3);
          continue;
        }
        S[4 * g + 0] = fmaf(a.x, S[4 * g + 0], kk.x * vj);
        S[4 * g + 1] = fmaf(a.y, S[4 * g + 1], kk.y * vj);
        S[4 * g + 2] = fmaf(a.z, S[4 * g + 2], kk.z * vj);
        S[4 * g + 3] = fmaf(a.w, S[4 * g + 3], kk.w * vj);
        acc0 = fmaf(S[4 * g + 0], qq.x, acc0);
        acc1 = fmaf(S[4 * g + 1], qq.y, acc1);
        acc0 = fmaf(S[4 * g + 2], qq.z, acc0);
        acc1 = fmaf(S[4 * g + 3], qq.w, acc1);
      }
      return acc0 + acc1;
    };
    int c = 0;
    for (; c + 4 <= n; c += 4) {  // four tokens' sums over the row groups side by side: their shuffles overlap
      float acc[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = update(c + u);
#pragma unroll
      for (int o = 1; o < RGP2; o <<= 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
      }
      if (rg == 0) {
#pragma unroll
        for (int u = 0; u < 4; ++u) os[c + u][col] = acc[u];
      }
    }
    for (; c < n; ++c) {
      float acc = update(c);
#pragma unroll
      for (int o = 1; o < RGP2; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (rg == 0) os[c][col] = acc;
    }
    __syncthreads();  // the chunk's outputs are complete; nobody reads this half of the buffers any more
    for (int x = tid; x < n * SCAN_VT; x += THREADS) {
      const int c = x / SCAN_VT, jj = blockIdx.x * SCAN_VT + (x % SCAN_VT);
      if (jj < Dv) out[((long)(c0 + c) * H + h) * Dv + jj] = os[c][x % SCAN_VT];
    }
    if (more) stage(c0 + SCAN_CT, buf ^ 1);
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < SCAN_R; ++r) {
    const int i = rg * SCAN_R + r;
    if (i < D && j < Dv) Sg[(long)i * Dv + j] = S[r];
  }
}

template <typename T, int RGP2, int SCAN_R, int SCAN_VT, bool BONUS>
static cudaError_t launch_scan(cudaStream_t stream, int num_seqs, const void* q, long q_stride, const void* k,
                               long k_stride, const void* v, long v_stride, const void* z, long z_stride,
                               const float* z_bias, float inv_tau, const float* head_decay, const float* inv_freq,
                               int rot_pairs, const int* positions, float q_scale, float k_scale, float* state,
                               const int* cu_seqlens, const int* state_slots, float* out, int H, int D, int Dv,
                               int decay_mode, const float* tok_decay, const float* tok_kscale, int ones_col,
                               const float* bonus) {
  constexpr size_t smem = (size_t)(6 * SCAN_CT * RGP2 * SCAN_R + 3 * SCAN_CT * SCAN_VT) * sizeof(float);
  auto kernel = decayed_state_scan_kernel<T, RGP2, SCAN_R, SCAN_VT, BONUS>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const dim3 grid((Dv + SCAN_VT - 1) / SCAN_VT, H, num_seqs);
  return launch_pdl(kernel, grid, dim3(SCAN_VT * RGP2), smem, stream, (const T*)q, q_stride,
                    (const T*)k, k_stride, (const T*)v, v_stride, (const T*)z, z_stride, z_bias, inv_tau, head_decay,
                    inv_freq, rot_pairs, positions, q_scale, k_scale, state, cu_seqlens, state_slots, out, H, D, Dv,
                    decay_mode, tok_decay, tok_kscale, ones_col, bonus);
}

// q, k: head h of token t at [t * stride + h * D]; v at [t * v_stride + h * (Dv - ones_col)]; z (decay
// logits, or null) like q, z_bias fp32 [H * D] or null; decay_mode 0: exp(logsigmoid(z + b) * inv_tau), 1:
// exp(-exp(z + b)); head_decay fp32 [H] or tok_decay fp32 [T, H] (one of them when z is null); tok_kscale
// fp32 [T, H] or null; bonus fp32 [H * D] or null; inv_freq fp32 [rot_pairs] with positions, or
// rot_pairs = 0; state fp32 [slots, H, D, Dv]; out fp32 [T, H, Dv]; Dv counts the column of ones.
Q3_EXPORT int q3_decayed_state_scan(int dtype, const void* q, long q_stride, const void* k, long k_stride,
                                    const void* v, long v_stride, const void* z, long z_stride, const float* z_bias,
                                    float inv_tau, const float* head_decay, const float* inv_freq, int rot_pairs,
                                    const int* positions, float q_scale, float k_scale, float* state,
                                    const int* cu_seqlens, const int* state_slots, float* out, int num_seqs, int H,
                                    int D, int Dv, int decay_mode, const float* tok_decay, const float* tok_kscale,
                                    int ones_col, const float* bonus, cudaStream_t stream) {
  if (!q || !k || !v || !state || !cu_seqlens || !state_slots || !out) return Q3_ERR_ARGUMENT;
  if (!z && !head_decay && !tok_decay) return Q3_ERR_ARGUMENT;
  if (decay_mode < 0 || decay_mode > 1 || ones_col < 0 || ones_col > 1 || Dv - ones_col < 1) return Q3_ERR_ARGUMENT;
  if (rot_pairs < 0 || 2 * rot_pairs > D || (rot_pairs && (!inv_freq || !positions))) return Q3_ERR_ARGUMENT;
  if (H < 1 || D < 1 || Dv < 1 || H > 65535 || num_seqs > 65535) return Q3_ERR_ARGUMENT;
  if (D > 256 || (dtype != Q3_DTYPE_F32 && dtype != Q3_DTYPE_BF16)) return Q3_ERR_UNSUPPORTED;
  if (num_seqs == 0) return Q3_OK;
  cudaError_t e;
#define Q3_SCAN_B(T, RGP2, R, VT, B)                                                                                 \
  e = launch_scan<T, RGP2, R, VT, B>(stream, num_seqs, q, q_stride, k, k_stride, v, v_stride, z, z_stride, z_bias,   \
                                     inv_tau, head_decay, inv_freq, rot_pairs, positions, q_scale, k_scale, state,   \
                                     cu_seqlens, state_slots, out, H, D, Dv, decay_mode, tok_decay, tok_kscale,      \
                                     ones_col, bonus)
#define Q3_SCAN(T, RGP2, R, VT)                                                                                      \
  do { if (bonus) Q3_SCAN_B(T, RGP2, R, VT, true); else Q3_SCAN_B(T, RGP2, R, VT, false); } while (0)
#define Q3_SCAN_SIZES(T)                                                                                             \
  if (D <= 16) Q3_SCAN(T, 4, 4, 16); else if (D <= 32) Q3_SCAN(T, 8, 4, 16); else if (D <= 64) Q3_SCAN(T, 16, 4, 16); \
  else if (D <= 128) Q3_SCAN(T, 32, 4, 16); else Q3_SCAN(T, 32, 8, 32)
  if (dtype == Q3_DTYPE_F32) { Q3_SCAN_SIZES(float); } else { Q3_SCAN_SIZES(bf16); }
#undef Q3_SCAN_SIZES
#undef Q3_SCAN
#undef Q3_SCAN_B
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// ---- gates of a matrix memory with a running maximum ---------------------------------------------------
// One warp per (sequence, head), 32 tokens at a time: every lane works out its token's two log gates, the
// running maximum then goes through the 32 tokens in order (an add and a max per token, on values handed
// round by shuffles, so the chain is exactly the sequential one wherever a portion starts), and every
// lane turns its token's maximum and its predecessor's into the decay and the key factor.
template <typename T>
__global__ void stabilised_gates_kernel(const T* __restrict__ zi, const T* __restrict__ zf, long z_stride,
                                        const float* __restrict__ bi, const float* __restrict__ bf, float cap,
                                        float* __restrict__ m_state, const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ state_slots, float* __restrict__ decay,
                                        float* __restrict__ kscale, float* __restrict__ m_run, int H, int pairs) {
  pdl_wait();
  pdl_launch_dependents();
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= pairs) return;
  const int b = item / H, h = item - b * H;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  if (t1 <= t0) return;
  float* mslot = m_state + (long)state_slots[b] * H + h;
  float m = *mslot;
  const float bih = bi ? bi[h] : 0.f, bfh = bf ? bf[h] : 0.f, inv_cap = 1.f / cap;
  for (int c0 = t0; c0 < t1; c0 += 32) {
    const int t = c0 + lane, n = min(32, t1 - c0);
    float li = 0.f, lf = 0.f;
    if (t < t1) {
      li = cap * tanhf((to_f32(zi[t * z_stride + h]) + bih) * inv_cap);
      const float x = cap * tanhf((to_f32(zf[t * z_stride + h]) + bfh) * inv_cap);
      lf = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
    }
    float m_before = 0.f, m_after = 0.f;
    for (int s = 0; s < n; ++s) {
      const float lis = __shfl_sync(0xffffffffu, li, s), lfs = __shfl_sync(0xffffffffu, lf, s);
      const float next = fmaxf(lfs + m, lis);
      if (lane == s) { m_before = m; m_after = next; }
      m = next;
    }
    if (t < t1) {
      decay[(long)t * H + h] = expf(lf + m_before - m_after);
      kscale[(long)t * H + h] = expf(li - m_after);
      m_run[(long)t * H + h] = m_after;
    }
  }
  if (lane == 0) *mslot = m;
}

// zi, zf: [T, H] rows z_stride apart (the two gates' pre-activations); bi, bf: fp32 [H] or null; m_state:
// fp32 [slots, H]; decay, kscale, m_run: fp32 [T, H].
Q3_EXPORT int q3_stabilised_gates(int dtype, const void* zi, const void* zf, long z_stride, const float* bi,
                                  const float* bf, float cap, float* m_state, const int* cu_seqlens,
                                  const int* state_slots, float* decay, float* kscale, float* m_run, int num_seqs,
                                  int H, cudaStream_t stream) {
  if (!zi || !zf || !m_state || !cu_seqlens || !state_slots || !decay || !kscale || !m_run || H < 1 || !(cap > 0.f))
    return Q3_ERR_ARGUMENT;
  if (num_seqs == 0) return Q3_OK;
  const int pairs = num_seqs * H;
  const unsigned blocks = (unsigned)((pairs + 3) / 4);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(stabilised_gates_kernel<float>, dim3(blocks), dim3(128), 0, stream, (const float*)zi,
                   (const float*)zf, z_stride, bi, bf, cap, m_state, cu_seqlens, state_slots, decay, kscale, m_run, H,
                   pairs);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(stabilised_gates_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, (const bf16*)zi, (const bf16*)zf,
                   z_stride, bi, bf, cap, m_state, cu_seqlens, state_slots, decay, kscale, m_run, H, pairs);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// head_norm_gate: every head's fp32 output divided by its root mean square, times a weight (one per value
// channel, shared by the heads or one per head and channel), times act(gate) and out_scale, rounded once.
// gate_act 0: silu, 1: sigmoid.  With m_run (fp32 [T, H]) a row of o has one more column, c = o[Dv], and the
// values are first divided by max(|c|, exp(-m_run)) + 1e-6 (the normaliser of a memory whose gates are kept
// in range by a running maximum).
__device__ __forceinline__ float gate_value(float g, int gate_act) {
  const float sg = 1.f / (1.f + expf(-g));
  return gate_act == 1 ? sg : g * sg;
}

template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ m_run,
                                      const float* __restrict__ w, int w_per_head, float eps,
                                      const T* __restrict__ g, long g_stride, T* __restrict__ y, long y_stride,
                                      float out_scale, int gate_act, long items, int H, int Dv) {
  pdl_wait();
  pdl_launch_dependents();
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const long t = item / H;
  const int h = (int)(item - t * H);
  const float* orow = o + item * o_stride;
  const float den = m_run ? fmaxf(fabsf(orow[Dv]), expf(-m_run[item])) + 1e-6f : 1.f;
  float ss = 0.f;
  for (int d = lane; d < Dv; d += 32) {
    const float x = m_run ? orow[d] / den : orow[d];
    ss += x * x;
  }
  const float rstd = rsqrtf(warp_sum(ss) / (float)Dv + eps);
  const T* grow = g + t * g_stride + (long)h * Dv;
  T* yrow = y + t * y_stride + (long)h * Dv;
  const float* wrow = w ? (w_per_head ? w + (long)h * Dv : w) : nullptr;
  for (int d = lane; d < Dv; d += 32) {
    float val = (m_run ? orow[d] / den : orow[d]) * rstd;
    if (wrow) val *= wrow[d];
    yrow[d] = from_f32<T>(val * gate_value(to_f32(grow[d]), gate_act) * out_scale);
  }
}

// The same with 16-byte accesses for value sizes up to 256 that are multiples of 8 (rows 16-byte
// aligned): a lane keeps its eight values in registers between the sum of squares and the store, and a
// warp takes as many (token, head) items as fit (`lph` lanes per item, a power of two >= Dv / 8).  Rows of
// o with the extra column are not aligned and are read value by value.
template <typename T>
__global__ void head_norm_gate_vec_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ m_run,
                                          const float* __restrict__ w, int w_per_head, float eps,
                                          const T* __restrict__ g, long g_stride, T* __restrict__ y, long y_stride,
                                          float out_scale, int gate_act, long items, int H, int Dv, int lph) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, per_warp = 32 / lph;
  const long item = ((long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * per_warp + lane / lph;
  const int d = (lane % lph) * 8;
  const bool live = item < items && d < Dv;
  const long t = live ? item / H : 0;
  const int h = live ? (int)(item - t * H) : 0;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, gate[8];
  float ss = 0.f;
  if (live) {
    const float* orow = o + item * o_stride;
    if (m_run) {
      const float den = fmaxf(fabsf(orow[Dv]), expf(-m_run[item])) + 1e-6f;
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = orow[d + e] / den;
    } else {
      load8(orow + d, v);
    }
    load8(g + t * g_stride + (long)h * Dv + d, gate);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
  }
  for (int off = lph >> 1; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if (!live) return;
  const float rstd = rsqrtf(ss / (float)Dv + eps);
  float wv[8];
  if (w) load8(w + (w_per_head ? (long)h * Dv : 0) + d, wv);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float val = v[e] * rstd;
    if (w) val *= wv[e];
    v[e] = val * gate_value(gate[e], gate_act) * out_scale;
  }
  store8(y + t * y_stride + (long)h * Dv + d, v);
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// o: fp32 [T, H, Dv] (with m_run: [T, H, Dv + 1] and m_run fp32 [T, H]); w: fp32 [Dv] shared by the heads
// or [H, Dv] (w_per_head), or null; g, y: head h of token t at [t * stride + h * Dv].
Q3_EXPORT int q3_head_norm_gate(int dtype, const float* o, const float* m_run, const float* w, int w_per_head,
                                float eps, const void* g, long g_stride, void* y, long y_stride, float out_scale,
                                int gate_act, int num_tokens, int H, int Dv, cudaStream_t stream) {
  if (!o || !g || !y || H < 1 || Dv < 1 || gate_act < 0 || gate_act > 1) return Q3_ERR_ARGUMENT;
  const long items = (long)num_tokens * H;
  if (items == 0) return Q3_OK;
  const int o_stride = Dv + (m_run ? 1 : 0);
  const unsigned blocks = (unsigned)((items + 7) / 8);
  cudaError_t e;
  const bool vec = Dv % 8 == 0 && Dv <= 256 && g_stride % 8 == 0 && y_stride % 8 == 0 && (m_run || aligned16(o)) &&
                   aligned16(g) && aligned16(y) && (!w || aligned16(w));
  int lph = 1;  // lanes per (token, head) item
  while (lph * 8 < Dv) lph <<= 1;
  const long per_block = 8 * (32 / (lph > 32 ? 32 : lph));
  const unsigned vblocks = (unsigned)((items + per_block - 1) / per_block);
  if (vec && dtype == Q3_DTYPE_F32)
    e = launch_pdl(head_norm_gate_vec_kernel<float>, dim3(vblocks), dim3(256), 0, stream, o, o_stride, m_run, w,
                   w_per_head, eps, (const float*)g, g_stride, (float*)y, y_stride, out_scale, gate_act, items, H, Dv,
                   lph);
  else if (vec && dtype == Q3_DTYPE_BF16)
    e = launch_pdl(head_norm_gate_vec_kernel<bf16>, dim3(vblocks), dim3(256), 0, stream, o, o_stride, m_run, w,
                   w_per_head, eps, (const bf16*)g, g_stride, (bf16*)y, y_stride, out_scale, gate_act, items, H, Dv,
                   lph);
  else if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, o_stride, m_run, w, w_per_head,
                   eps, (const float*)g, g_stride, (float*)y, y_stride, out_scale, gate_act, items, H, Dv);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, o, o_stride, m_run, w, w_per_head,
                   eps, (const bf16*)g, g_stride, (bf16*)y, y_stride, out_scale, gate_act, items, H, Dv);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}
