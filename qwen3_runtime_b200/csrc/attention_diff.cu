// Differential attention over the paged cache in bfloat16: two softmax maps per head over the same values,
//   a_m = softmax_j(scale * q_m . k_m(j)) V  (m = 1, 2),   o = a_1 - lambda * a_2,
//   out = o * rsqrt(mean(o^2) + eps) * out_scale            (over the head's DV values, no weight).
// A query head is [q1 | q2] (D each), a key row [k1 | k2] (key pages [pages, nkv, ps, 2 D]), values
// [pages, nkv, ps, DV].  What a token at position p sees: keys max(lo_window, lo_chunk) .. p with
// lo_window = p - window + 1 (window > 0) and lo_chunk = floor(p / chunk) * chunk (chunk > 0).
//
//   diff_prefill   prompt portions (and whatever else a step holds) on the tensor cores: a work item is
//                  (sequence, kv head, block of 128 (token, head of the group) rows); keys and values in
//                  tiles of 64 through a 3-stage cp.async pipeline into XOR-swizzled shared memory; per map
//                  S = Q_m K_m^T and O_m += P_m V as m16n8k16 MMAs with fp32 accumulators and an online
//                  softmax of its own in fp32 (exp2 with the scale folded in); a value tile is loaded once
//                  for both maps; the subtraction and the head's norm are the epilogue.
//   diff_decode    steps in which every sequence brings one token: a block per (sequence, kv head, slice of
//                  the keys), 8 warps taking tiles of 32 keys in turn, a lane scoring one key for all heads
//                  of the group and both maps (the key row is read once) while the tile's value rows,
//                  requested before, wait in registers; fp32 throughout; the warps' partial results (running
//                  maximum, sum, weighted values) are merged in shared memory and written per slice;
//                  diff_merge adds the slices, subtracts, norms and stores.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace {

__device__ __forceinline__ int first_visible(int p, int window, int chunk) {
  int lo = window > 0 ? max(0, p - window + 1) : 0;
  if (chunk > 0) lo = max(lo, p / chunk * chunk);
  return lo;
}

// ---- prompt portions on the tensor cores -----------------------------------------------------------
constexpr int BLOCK_M = 128;
constexpr int TILE = 64;
constexpr int WARPS = BLOCK_M / 16;
constexpr int THREADS = WARPS * 32;
constexpr int STAGES = 3;

template <int D, int DV>
__global__ void __launch_bounds__(THREADS, 1)
diff_prefill_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kpages,
                    const bf16* __restrict__ vpages, const int* __restrict__ block_table, int max_pages,
                    const int* __restrict__ kv_lens, const int* __restrict__ cu_seqlens, bf16* __restrict__ out,
                    long out_stride, int num_seqs, int nq, int nkv, int ps, float scale_log2, int window, int chunk,
                    float lambda, float eps, float out_scale) {
  constexpr int KW = 2 * D;            // a key row: both maps
  constexpr int KCH = KW / 8, VCH = DV / 8;
  constexpr int K_BYTES = TILE * KW * 2, V_BYTES = TILE * DV * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                      // [BLOCK_M][KW]
  unsigned char* kv_s = smem + BLOCK_M * KW * 2;  // STAGES x (K tile, V tile)
  __shared__ int s_item[2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y;
  const int G = nq / nkv;

  if (tid == 0) {
    int acc = 0, found = -1, rb = 0;
    const int w = blockIdx.x;
    for (int s = 0; s < num_seqs; ++s) {
      const int ql = cu_seqlens[s + 1] - cu_seqlens[s];
      if (ql <= 0) continue;
      const int nb = (ql * G + BLOCK_M - 1) / BLOCK_M;
      if (w < acc + nb) {
        found = s;
        rb = w - acc;
        break;
      }
      acc += nb;
    }
    s_item[0] = found;
    s_item[1] = rb;
  }
  __syncthreads();
  const int seq = s_item[0];
  if (seq < 0) return;
  const int row0 = s_item[1] * BLOCK_M;
  const int tok0 = cu_seqlens[seq];
  const int q_len = cu_seqlens[seq + 1] - tok0;
  const int kv_len = kv_lens[seq];
  const int rows = q_len * G;
  const int base_pos = kv_len - q_len;
  const int* bt = block_table + (long)seq * max_pages;

  for (int c = tid; c < BLOCK_M * KCH; c += THREADS) {
    const int r = c / KCH, ch = c % KCH;
    const int R = row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < rows) {
      const int tk = R / G, hd = kvh * G + (R - tk * G);
      v = *reinterpret_cast<const uint4*>(q + (long)(tok0 + tk) * q_stride + (long)hd * KW + ch * 8);
    }
    *reinterpret_cast<uint4*>(q_s + swz<KW>(r, ch)) = v;
  }

  const int last_row = min(rows, row0 + BLOCK_M) - 1;
  const int p_min = base_pos + row0 / G, p_max = base_pos + last_row / G;
  const int k_lo = first_visible(p_min, window, chunk);  // the first key any row of the block sees
  const int t_begin = k_lo / TILE, t_end = p_max / TILE;  // inclusive
  const int num_tiles = t_end - t_begin + 1;

  auto load_tile = [&](int tile, int stage) {
    unsigned char* k_dst = kv_s + (size_t)stage * (K_BYTES + V_BYTES);
    unsigned char* v_dst = k_dst + K_BYTES;
    const int base = (t_begin + tile) * TILE;
    for (int c = tid; c < TILE * KCH; c += THREADS) {
      const int r = c / KCH, ch = c % KCH;
      const int j = base + r;
      const bool valid = j >= k_lo && j <= p_max;
      long src = 0;
      if (valid) src = (((long)bt[j / ps] * nkv + kvh) * ps + (j % ps)) * KW + ch * 8;
      cp_async16(smem_u32(k_dst + swz<KW>(r, ch)), kpages + src, valid ? 16 : 0);
    }
    for (int c = tid; c < TILE * VCH; c += THREADS) {
      const int r = c / VCH, ch = c % VCH;
      const int j = base + r;
      const bool valid = j >= k_lo && j <= p_max;
      long src = 0;
      if (valid) src = (((long)bt[j / ps] * nkv + kvh) * ps + (j % ps)) * DV + ch * 8;
      cp_async16(smem_u32(v_dst + swz<DV>(r, ch)), vpages + src, valid ? 16 : 0);
    }
  };

  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_tiles) load_tile(s, s);
    cp_async_commit();
  }
  __syncthreads();  // q_s complete

  int pos[2], lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int R = row0 + warp * 16 + (lane >> 2) + r * 8;
    pos[r] = R < rows ? base_pos + R / G : -1;
    lo[r] = pos[r] >= 0 ? first_visible(pos[r], window, chunk) : 0;
  }
  const int Rw0 = row0 + warp * 16, Rw1 = min(rows, Rw0 + 16) - 1;
  const bool warp_live = Rw0 < rows;
  const int wp_min = base_pos + Rw0 / G, wp_max = warp_live ? base_pos + Rw1 / G : -1;
  const int wlo_min = first_visible(wp_min, window, chunk);
  const int wlo_max = warp_live ? first_visible(wp_max, window, chunk) : 0;

  float o[2][DV / 8][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.f;
  float m_run[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}};
  float l_run[2][2] = {{0.f, 0.f}, {0.f, 0.f}};

  for (int tile = 0; tile < num_tiles; ++tile) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nxt = tile + STAGES - 1;
      if (nxt < num_tiles) load_tile(nxt, nxt % STAGES);
      cp_async_commit();
    }
    const int key0 = (t_begin + tile) * TILE;
    if (!warp_live || key0 > wp_max || key0 + TILE - 1 < wlo_min) continue;  // nothing for this warp
    const unsigned char* k_t = kv_s + (size_t)(tile % STAGES) * (K_BYTES + V_BYTES);
    const unsigned char* v_t = k_t + K_BYTES;
    const bool edge = key0 + TILE - 1 > wp_min || key0 < wlo_max;

#pragma unroll
    for (int m = 0; m < 2; ++m) {
      float s[TILE / 8][4];
#pragma unroll
      for (int n = 0; n < TILE / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t qa[4];
        ldmatrix_x4(qa, smem_u32(q_s + swz<KW>(warp * 16 + (lane & 15), m * (D / 8) + 2 * ks + (lane >> 4))));
#pragma unroll
        for (int nn = 0; nn < TILE / 16; ++nn) {
          uint32_t kb[4];
          const int row = nn * 16 + (lane & 7) + ((lane >> 4) << 3);
          ldmatrix_x4(kb, smem_u32(k_t + swz<KW>(row, m * (D / 8) + 2 * ks + ((lane >> 3) & 1))));
          mma_bf16(s[2 * nn], qa, kb[0], kb[1]);
          mma_bf16(s[2 * nn + 1], qa, kb[2], kb[3]);
        }
      }
      if (edge) {
#pragma unroll
        for (int n = 0; n < TILE / 8; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = key0 + n * 8 + 2 * (lane & 3) + (e & 1);
            if (j > pos[e >> 1] || j < lo[e >> 1]) s[n][e] = -INFINITY;
          }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < TILE / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[m][r], mx[r]);
        m_use[r] = m_new == -INFINITY ? 0.f : m_new;
        corr[r] = exp2f((m_run[m][r] - m_use[r]) * scale_log2);
        m_run[m][r] = m_new;
        l_run[m][r] *= corr[r];
      }
#pragma unroll
      for (int n = 0; n < TILE / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[n][e] = exp2f((s[n][e] - m_use[e >> 1]) * scale_log2);
          l_run[m][e >> 1] += s[n][e];
        }
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
          o[m][i][0] *= corr[0]; o[m][i][1] *= corr[0];
          o[m][i][2] *= corr[1]; o[m][i][3] *= corr[1];
        }
      }
#pragma unroll
      for (int kk = 0; kk < TILE / 16; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int i = 0; i < DV / 16; ++i) {
          uint32_t vb[4];
          const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          ldmatrix_x4_trans(vb, smem_u32(v_t + swz<DV>(row, 2 * i + (lane >> 4))));
          mma_bf16(o[m][2 * i], pa, vb[0], vb[1]);
          mma_bf16(o[m][2 * i + 1], pa, vb[2], vb[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

  // ---- o = a1 - lambda a2, divided by its root mean square, times out_scale ----------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float inv[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      float l = l_run[m][r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      inv[m] = 1.f / l;
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float v = o[0][i][2 * r + e] * inv[0] - lambda * (o[1][i][2 * r + e] * inv[1]);
        o[0][i][2 * r + e] = v;
        ss += v * v;
      }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    const int R = row0 + warp * 16 + (lane >> 2) + r * 8;
    if (R >= rows) continue;
    const float rstd = rsqrtf(ss / (float)DV + eps) * out_scale;
    const int tk = R / G, hd = kvh * G + (R - tk * G);
    bf16* dst = out + (long)(tok0 + tk) * out_stride + (long)hd * DV + 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < DV / 8; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[0][i][2 * r] * rstd, o[0][i][2 * r + 1] * rstd);
  }
}

template <int D, int DV>
int launch_diff_prefill(const bf16* q, int q_stride, const bf16* kpages, const bf16* vpages, const int* block_table,
                        int max_pages, const int* kv_lens, const int* cu_seqlens, bf16* out, long out_stride,
                        int num_seqs, int num_work, int nq, int nkv, int ps, float scale, int window, int chunk,
                        float lambda, float eps, float out_scale, cudaStream_t stream) {
  const size_t smem = (size_t)BLOCK_M * 2 * D * 2 + (size_t)STAGES * TILE * (2 * D + DV) * 2;
  static bool configured_on[Q3_MAX_DEVICES];
  bool& configured = configured_on[q3_current_device()];
  if (!configured) {
    if (cudaFuncSetAttribute(diff_prefill_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return Q3_ERR_LAUNCH;
    configured = true;
  }
  dim3 grid(num_work, nkv);
  diff_prefill_kernel<D, DV><<<grid, THREADS, smem, stream>>>(q, q_stride, kpages, vpages, block_table, max_pages,
                                                              kv_lens, cu_seqlens, out, out_stride, num_seqs, nq, nkv,
                                                              ps, scale * 1.4426950408889634f, window, chunk, lambda,
                                                              eps, out_scale);
  return q3_launch_status();
}

// ---- one token per sequence: slices of the keys on the FMA pipes ------------------------------------
constexpr int DEC_WARPS = 8;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int MAX_VC = 4;  // values of up to 128 (the merge kernel: 4 per lane)

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    v[2 * e] = f.x;
    v[2 * e + 1] = f.y;
  }
}

// mid: [num_seqs, nq, splits, 2 maps, DV + 2] floats: the weighted values, then the running maximum and sum.
// A tile is 32 keys.  Its value rows are requested first, 16 bytes a lane (DV / 8 lanes a row, so 256 / DV rows
// an instruction), and wait in registers while the lanes score one key each (all heads of the group, both
// maps, the key row in rounds of 32 elements a map); so a tile costs about three memory round trips, not one
// per key.  A warp serves GS heads of the group's G: the G / GS warps of a tile read the same rows (the second
// from cache) and each carries a short instruction stream and few accumulators, so that two blocks fit an SM.
// VB: value-row instructions in flight at a time.
template <int G, int GS, int VB>
__global__ void __launch_bounds__(DEC_THREADS, 2)
diff_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kpages,
                   const bf16* __restrict__ vpages, const int* __restrict__ block_table, int max_pages,
                   const int* __restrict__ kv_lens, const int* __restrict__ cu_seqlens, float* __restrict__ mid,
                   int nq, int nkv, int D, int DV, int ps, float scale, int window, int chunk, int splits) {
  extern __shared__ float dec_smem[];
  float* qs = dec_smem;                       // [G][2 D], scaled
  float* part = dec_smem + G * 2 * D;         // [NTS][G * 2][DV + 2]
  constexpr int WPT = G / GS;                 // warps a tile
  constexpr int NTS = DEC_WARPS / WPT;        // tiles the block works on at a time
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ts = warp / WPT, g0 = (warp % WPT) * GS;
  const int seq = blockIdx.x / nkv, kvh = blockIdx.x - seq * nkv;
  const int split = blockIdx.y;
  const int tok = cu_seqlens[seq];
  const int p = kv_lens[seq] - 1;
  const int lo = first_visible(p, window, chunk);
  const int n = p + 1 - lo;
  const int slice = (((n + splits - 1) / splits) + 31) & ~31;
  const int k_begin = lo + split * slice, k_end = min(p + 1, k_begin + slice);
  const int* bt = block_table + (long)seq * max_pages;
  const int KW = 2 * D;
  const int lpr = DV / 8;          // lanes a value row: 4, 8 or 16
  const int rpi = 32 / lpr;        // value rows an instruction
  const int col = (lane % lpr) * 8, sub = lane / lpr;
  const bf16* qrow = q + (long)tok * q_stride + (long)kvh * G * KW;
  for (int i = threadIdx.x; i < G * KW; i += DEC_THREADS) qs[i] = to_f32(qrow[i]) * scale;
  __syncthreads();

  float m[GS][2], l[GS][2], acc[GS][2][8];
#pragma unroll
  for (int g = 0; g < GS; ++g)
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      m[g][w] = -INFINITY;
      l[g][w] = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[g][w][c] = 0.f;
    }
  for (int j0 = k_begin + ts * 32; j0 < k_end; j0 += NTS * 32) {
    const int j = j0 + lane;
    const bool valid = j < k_end;
    const int count = min(32, k_end - j0);
    const long row = valid ? ((long)bt[j / ps] * nkv + kvh) * ps + (j % ps) : 0;
    float pw[GS][2];
#pragma unroll
    for (int vb = 0; vb < 16; vb += VB) {  // (one pass when all of a tile's value rows fit in registers)
      uint4 vreg[VB];
#pragma unroll
      for (int i = 0; i < VB; ++i) {
        const int key = (vb + i) * rpi + sub;
        const long rj = __shfl_sync(0xffffffffu, row, key & 31);
        vreg[i] = (vb + i) * rpi < 32 && key < count ? *reinterpret_cast<const uint4*>(vpages + rj * DV + col)
                                                      : make_uint4(0, 0, 0, 0);
      }
      if (vb == 0) {
        float s[GS][2];
#pragma unroll
        for (int g = 0; g < GS; ++g) s[g][0] = s[g][1] = 0.f;
        if (valid) {
          const bf16* kr = kpages + row * KW;
          for (int d0 = 0; d0 < D; d0 += 32) {  // 32 elements of each map a round, its eight loads in flight together
            uint4 ra[4], rb[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const bool in = d0 + 8 * u < D;
              ra[u] = in ? *reinterpret_cast<const uint4*>(kr + d0 + 8 * u) : make_uint4(0, 0, 0, 0);
              rb[u] = in ? *reinterpret_cast<const uint4*>(kr + D + d0 + 8 * u) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int d = d0 + 8 * u;
              if (d >= D) break;
              float ka[8], kb[8];
              unpack8(ra[u], ka);
              unpack8(rb[u], kb);
#pragma unroll
              for (int g = 0; g < GS; ++g) {
                const float* qg = qs + (g0 + g) * KW;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  s[g][0] = fmaf(qg[d + e], ka[e], s[g][0]);
                  s[g][1] = fmaf(qg[D + d + e], kb[e], s[g][1]);
                }
              }
            }
          }
        }
#pragma unroll
        for (int g = 0; g < GS; ++g)
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            const float sv = valid ? s[g][w] : -INFINITY;
            const float m_new = fmaxf(m[g][w], warp_max(sv));
            pw[g][w] = valid ? expf(sv - m_new) : 0.f;
            const float corr = expf(m[g][w] - m_new);
            l[g][w] = l[g][w] * corr + warp_sum(pw[g][w]);
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[g][w][c] *= corr;
            m[g][w] = m_new;
          }
      }
#pragma unroll
      for (int i = 0; i < VB; ++i) {
        const int key = ((vb + i) * rpi + sub) & 31;  // (rows past the tile were not loaded: zeros)
        float v[8];
        unpack8(vreg[i], v);
#pragma unroll
        for (int g = 0; g < GS; ++g)
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            const float pj = __shfl_sync(0xffffffffu, pw[g][w], key);
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[g][w][c] = fmaf(pj, v[c], acc[g][w][c]);
          }
      }
    }
  }
  // the lanes that hold the same columns added up, the tiles' results side by side, then one warp per
  // (head, map) merges them in order
  const int PW = DV + 2;
#pragma unroll
  for (int g = 0; g < GS; ++g)
#pragma unroll
    for (int w = 0; w < 2; ++w) {
#pragma unroll
      for (int c = 0; c < 8; ++c)
        for (int o = lpr; o < 32; o <<= 1) acc[g][w][c] += __shfl_xor_sync(0xffffffffu, acc[g][w][c], o);
      float* dst = part + ((long)ts * G * 2 + (g0 + g) * 2 + w) * PW;
      if (lane < lpr) {
#pragma unroll
        for (int c = 0; c < 8; ++c) dst[col + c] = acc[g][w][c];
      }
      if (lane == 0) {
        dst[DV] = m[g][w];
        dst[DV + 1] = l[g][w];
      }
    }
  __syncthreads();
  const int vc = DV / 32;
  for (int item = warp; item < G * 2; item += DEC_WARPS) {
    float mm = -INFINITY;
    for (int w = 0; w < NTS; ++w) mm = fmaxf(mm, part[((long)w * G * 2 + item) * PW + DV]);
    float ll = 0.f, a[MAX_VC];
#pragma unroll
    for (int c = 0; c < MAX_VC; ++c) a[c] = 0.f;
    for (int w = 0; w < NTS; ++w) {
      const float* src = part + ((long)w * G * 2 + item) * PW;
      const float f = src[DV] == -INFINITY ? 0.f : expf(src[DV] - mm);
      ll += f * src[DV + 1];
#pragma unroll
      for (int c = 0; c < MAX_VC; ++c)
        if (c < vc) a[c] += f * src[lane + 32 * c];
    }
    const int g = item >> 1, w = item & 1;
    float* dst = mid + ((((long)seq * nq + kvh * G + g) * splits + split) * 2 + w) * PW;
#pragma unroll
    for (int c = 0; c < MAX_VC; ++c)
      if (c < vc) dst[lane + 32 * c] = a[c];
    if (lane == 0) {
      dst[DV] = mm;
      dst[DV + 1] = ll;
    }
  }
}

// One warp per (sequence, head): the slices of both maps added up, the subtraction, the norm, the store.  A
// lane fetches one slice's maximum and sum (so all slices' are in flight at once) and the warp agrees on the
// weights; the value loads of four slices are in flight together.  splits <= 64.
__global__ void diff_merge_kernel(const float* __restrict__ mid, const int* __restrict__ cu_seqlens,
                                  bf16* __restrict__ out, long out_stride, int num_seqs, int nq, int DV, int splits,
                                  float lambda, float eps, float out_scale) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long)num_seqs * nq) return;
  const int seq = (int)(item / nq), h = (int)(item - (long)seq * nq);
  const int PW = DV + 2, vc = DV / 32;
  const float* base = mid + item * splits * 2 * PW;  // [splits][2 maps][PW]
  float f[2][2], inv[2];                               // weights of slices lane and lane + 32, per map
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    float ms[2], ls[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int sl = lane + 32 * k;
      ms[k] = sl < splits ? base[((long)sl * 2 + w) * PW + DV] : -INFINITY;
      ls[k] = sl < splits ? base[((long)sl * 2 + w) * PW + DV + 1] : 0.f;
    }
    const float mm = warp_max(fmaxf(ms[0], ms[1]));
#pragma unroll
    for (int k = 0; k < 2; ++k) f[w][k] = ms[k] == -INFINITY ? 0.f : expf(ms[k] - mm);
    inv[w] = 1.f / warp_sum(f[w][0] * ls[0] + f[w][1] * ls[1]);
  }
  float a[2][MAX_VC];
#pragma unroll
  for (int w = 0; w < 2; ++w)
#pragma unroll
    for (int c = 0; c < MAX_VC; ++c) a[w][c] = 0.f;
#pragma unroll 4
  for (int sl = 0; sl < splits; ++sl) {
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      const float fs = __shfl_sync(0xffffffffu, sl < 32 ? f[w][0] : f[w][1], sl & 31);
      const float* src = base + ((long)sl * 2 + w) * PW;
#pragma unroll
      for (int c = 0; c < MAX_VC; ++c)
        if (c < vc) a[w][c] = fmaf(fs, src[lane + 32 * c], a[w][c]);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < MAX_VC; ++c) {
    a[0][c] = c < vc ? a[0][c] * inv[0] - lambda * (a[1][c] * inv[1]) : 0.f;
    ss += a[0][c] * a[0][c];
  }
  const float rstd = rsqrtf(warp_sum(ss) / (float)DV + eps) * out_scale;
  bf16* dst = out + (long)cu_seqlens[seq] * out_stride + (long)h * DV;
#pragma unroll
  for (int c = 0; c < MAX_VC; ++c)
    if (c < vc) dst[lane + 32 * c] = __float2bfloat16_rn(a[0][c] * rstd);
}

template <int G>
int launch_diff_decode(const bf16* q, int q_stride, const bf16* kpages, const bf16* vpages, const int* block_table,
                       int max_pages, const int* kv_lens, const int* cu_seqlens, float* mid, int num_seqs, int nq,
                       int nkv, int D, int DV, int ps, float scale, int window, int chunk, int splits,
                       cudaStream_t stream) {
  const size_t smem = ((size_t)G * 2 * D + (size_t)DEC_WARPS * G * 2 * (DV + 2)) * sizeof(float);
  if (smem > 200 * 1024) return Q3_ERR_UNSUPPORTED;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(diff_decode_kernel<G, (G > 2 ? 2 : G), 8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess)
    return Q3_ERR_LAUNCH;
  dim3 grid(num_seqs * nkv, splits);
  diff_decode_kernel<G, (G > 2 ? 2 : G), 8><<<grid, DEC_THREADS, smem, stream>>>(
      q, q_stride, kpages, vpages, block_table, max_pages, kv_lens, cu_seqlens, mid, nq, nkv, D, DV, ps, scale, window,
      chunk, splits);
  return q3_launch_status();
}

}  // namespace

// Prompt portions (any mix of sequences): num_work = sum over the sequences of ceil(q_len * (nq / nkv) / 128).
// Map sizes D of 32, 64 or 128 with value sizes DV of 64 or 128; anything else answers
// "unsupported" and belongs on the general kernel.  out: rows out_stride elements apart, head h at column h * DV.
Q3_EXPORT int q3_diff_attention_prefill(const void* q, int q_stride, const void* kpages, const void* vpages,
                                        const int* block_table, int max_pages, const int* kv_lens,
                                        const int* cu_seqlens, void* out, long out_stride, int num_seqs, int num_work,
                                        int nq, int nkv, int D, int DV, int ps, float scale, int window, int chunk,
                                        float lambda, float eps, float out_scale, cudaStream_t stream) {
  if (!q || !kpages || !vpages || !block_table || !kv_lens || !cu_seqlens || !out) return Q3_ERR_ARGUMENT;
  if (nq < 1 || nkv < 1 || nq % nkv || ps < 1 || num_seqs < 0 || num_work < 0 || chunk < 0) return Q3_ERR_ARGUMENT;
  if (q_stride % 8 || out_stride % 2 || nkv > 65535 || out_stride < (long)nq * DV) return Q3_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)kpages | (uintptr_t)vpages) & 15 || ((uintptr_t)out & 3)) return Q3_ERR_UNSUPPORTED;
  if (num_work == 0) return Q3_OK;
#define Q3_DIFF_CASE(d, dv)                                                                                        \
  if (D == d && DV == dv)                                                                                          \
    return launch_diff_prefill<d, dv>((const bf16*)q, q_stride, (const bf16*)kpages, (const bf16*)vpages,          \
                                      block_table, max_pages, kv_lens, cu_seqlens, (bf16*)out, out_stride,         \
                                      num_seqs, num_work, nq, nkv, ps, scale, window, chunk, lambda, eps,          \
                                      out_scale, stream);
  Q3_DIFF_CASE(32, 64)
  Q3_DIFF_CASE(32, 128)
  Q3_DIFF_CASE(64, 64)
  Q3_DIFF_CASE(64, 128)
  Q3_DIFF_CASE(128, 64)
  Q3_DIFF_CASE(128, 128)
#undef Q3_DIFF_CASE
  return Q3_ERR_UNSUPPORTED;
}

// One token per sequence (token row of sequence b: cu_seqlens[b], its position kv_lens[b] - 1).  D a multiple of
// 8, DV 32, 64 or 128, groups of 1, 2, 4 or 8 heads; mid: num_seqs * nq * splits * 2 * (DV + 2) floats.
Q3_EXPORT int q3_diff_attention_decode(const void* q, int q_stride, const void* kpages, const void* vpages,
                                       const int* block_table, int max_pages, const int* kv_lens,
                                       const int* cu_seqlens, void* out, long out_stride, float* mid, int num_seqs,
                                       int nq, int nkv, int D, int DV, int ps, float scale, int window, int chunk,
                                       int splits, float lambda, float eps, float out_scale, cudaStream_t stream) {
  if (!q || !kpages || !vpages || !block_table || !kv_lens || !cu_seqlens || !out || !mid) return Q3_ERR_ARGUMENT;
  if (nq < 1 || nkv < 1 || nq % nkv || ps < 1 || num_seqs < 0 || splits < 1 || chunk < 0) return Q3_ERR_ARGUMENT;
  if (D < 8 || D % 8 || (DV != 32 && DV != 64 && DV != 128) || out_stride < (long)nq * DV) return Q3_ERR_UNSUPPORTED;
  if (((uintptr_t)kpages & 15) || ((uintptr_t)vpages & 15) || splits > 64) return Q3_ERR_UNSUPPORTED;
  if (num_seqs == 0) return Q3_OK;
  const int G = nq / nkv;
  int code = Q3_ERR_UNSUPPORTED;
#define Q3_DIFF_GROUP(g)                                                                                           \
  if (G == g)                                                                                                      \
    code = launch_diff_decode<g>((const bf16*)q, q_stride, (const bf16*)kpages, (const bf16*)vpages, block_table,  \
                                 max_pages, kv_lens, cu_seqlens, mid, num_seqs, nq, nkv, D, DV, ps, scale, window, \
                                 chunk, splits, stream);
  Q3_DIFF_GROUP(1)
  Q3_DIFF_GROUP(2)
  Q3_DIFF_GROUP(4)
  Q3_DIFF_GROUP(8)
#undef Q3_DIFF_GROUP
  if (code != Q3_OK) return code;
  const long items = (long)num_seqs * nq;
  diff_merge_kernel<<<(unsigned)((items + 3) / 4), 128, 0, stream>>>(mid, cu_seqlens, (bf16*)out, out_stride, num_seqs,
                                                                     nq, DV, splits, lambda, eps, out_scale);
  return q3_launch_status();
}
