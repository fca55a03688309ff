// chunk_attn.cu — chunked grouped-query attention over a paged cache of raw keys that are also the values:
// per-head RMS norm of queries and keys (the key norm's weight carried by the query, its 1/rms applied to the
// score), soft cap, a logarithmic distance penalty per head, visibility limited to the query's own chunk of
// positions, a softmax with a silent zero-score sink, a sigmoid output gate.  A scalar kernel (fp32 model, any
// head size) and two tensor-core kernels for bf16 caches: 16-token tiles of prompt portions, and single decoded
// tokens whose tile rows are the heads of a group.  Scores, softmax state and accumulators are fp32 in all.
#include <stdlib.h>

#include <algorithm>

#include "layered_common.cuh"

namespace b200q {

// seq_desc[4*s + ...] = {first batch row, tokens this step, position of the first of them, state slot}
struct SeqView {
  int row0, n, pos0, slot;
};
__device__ __forceinline__ SeqView seq_view(const int32_t* __restrict__ seq_desc, int s) {
  const int4 v = *reinterpret_cast<const int4*>(seq_desc + 4 * s);
  return {v.x, v.y, v.z, v.w};
}

// ------------------------------------------------------------------------------------------------
// chunk attention, step 1 (CTA per token): per-head RMS norm of the queries with BOTH norm weights folded
// in (q / rms(q) * w_q * w_k: the key norm's weight moves to the query side, its 1/rms is applied to the
// score), and the raw keys into the paged cache row of the token.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) chunk_attn_prep_kernel(const T* __restrict__ proj, int ldp, int heads,
                                                              int kv_heads, int dim, const float* __restrict__ w_qn,
                                                              const float* __restrict__ w_kn,
                                                              const int32_t* __restrict__ slot_mapping,
                                                              float* __restrict__ qs, T* __restrict__ cache, float eps) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* pr = proj + (long long)t * ldp;
  for (int h = warp; h < heads; h += 4) {
    const T* q = pr + (long long)h * dim;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) {
      const float v = ldf(q + d);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dim + eps);
    float* o = qs + ((long long)t * heads + h) * dim;
    for (int d = lane; d < dim; d += 32) o[d] = ldf(q + d) * inv * w_qn[d] * w_kn[d];
  }
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int GD = kv_heads * dim;
  const T* k = pr + (long long)heads * dim;
  T* row = cache + (long long)slot * GD;
  for (int e = threadIdx.x; e < GD; e += blockDim.x) row[e] = k[e];
}

// step 2: one CTA per (token, key/value head, group of 8 query heads that share it).  Tiles of 32 cached
// keys are staged in shared memory once and used by up to 8 query heads (warp = head; lane = key for the
// scores, lane = output dims for the weighted sum).  The sink enters as the initial state of the online
// softmax: running maximum 0, denominator 1, no value.  Tiles start at the first key of the token's chunk.
template <typename T, int ACC>
__global__ void __launch_bounds__(256) chunk_attn_kernel(const float* __restrict__ qs, const T* __restrict__ cache,
                                                         const int32_t* __restrict__ block_table, int bt_stride,
                                                         const int32_t* __restrict__ row_seq,
                                                         const int32_t* __restrict__ positions, int heads,
                                                         int kv_heads, int dim, int block_size, int chunk, float scale,
                                                         float softcap, const float* __restrict__ r1,
                                                         const float* __restrict__ r2, const T* __restrict__ gate,
                                                         int ld_gate, float eps, T* __restrict__ out) {
  extern __shared__ float sm[];
  const int KS = dim + 1;
  float* qsm = sm;              // [8][dim]
  float* ksm = sm + 8 * dim;    // [32][dim+1]
  float* kinv = ksm + 32 * KS;  // [32]
  const int t = blockIdx.x, g = blockIdx.y, rep = heads / kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hg = blockIdx.z * 8 + warp;  // head within the group
  const bool live = hg < rep;
  const int h = g * rep + hg;
  const int p = positions[t];
  const int32_t* bt = block_table + (long long)row_seq[t] * bt_stride;
  const int lo = chunk > 0 ? p - p % chunk : 0;
  const int GD = kv_heads * dim;
  for (int e = threadIdx.x; e < 8 * dim; e += blockDim.x) {
    const int hh = blockIdx.z * 8 + e / dim;
    qsm[e] = hh < rep ? qs[((long long)t * heads + g * rep + hh) * dim + e % dim] : 0.f;
  }
  const float c1 = live ? r1[h] : 0.f, c2 = live ? r2[h] : 0.f;
  float m = 0.f, l = 1.f;  // the sink: a score of zero without a value
  float acc[ACC];
#pragma unroll
  for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
  const float* qh = qsm + warp * dim;
  for (int j0 = lo; j0 <= p; j0 += 32) {
    const int n = min(32, p + 1 - j0);
    __syncthreads();
    for (int e = threadIdx.x; e < n * dim; e += blockDim.x) {
      const int j = e / dim, d = e % dim, pos = j0 + j;
      const long long row = (long long)bt[pos / block_size] * block_size + pos % block_size;
      ksm[j * KS + d] = ldf(cache + row * GD + (long long)g * dim + d);
    }
    __syncthreads();
    for (int j = warp; j < n; j += 8) {
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss = fmaf(ksm[j * KS + d], ksm[j * KS + d], ss);
      ss = warp_sum(ss);
      if (lane == 0) kinv[j] = 1.f / sqrtf(ss / (float)dim + eps);
    }
    __syncthreads();
    if (!live) continue;
    float s = -INFINITY;
    if (lane < n) {
      const float* kr = ksm + lane * KS;
      float dot = 0.f;
      for (int d = 0; d < dim; ++d) dot = fmaf(qh[d], kr[d], dot);
      s = dot * kinv[lane] * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      s -= c1 * log1pf(c2 * (float)(p - (j0 + lane)));
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float pl = lane < n ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pl);
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] *= corr;
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pl, j);
      const float* kr = ksm + j * KS;
#pragma unroll
      for (int i = 0; i < ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dim) acc[i] = fmaf(pj, kr[d], acc[i]);
      }
    }
    m = m_new;
  }
  if (!live) return;
  const float inv = 1.f / l;
  const T* gr = gate + (long long)t * ld_gate + (long long)h * dim;
  T* o = out + ((long long)t * heads + h) * dim;
#pragma unroll
  for (int i = 0; i < ACC; ++i) {
    const int d = lane + 32 * i;
    if (d < dim) stf(o + d, acc[i] * inv * sigmoidf_(ldf(gr + d)));
  }
}

// ------------------------------------------------------------------------------------------------
// chunk attention on the tensor cores (bf16 cache, head size 64 or 128).  One CTA per (sequence of the step,
// key/value head, tile of 16 consecutive tokens of the sequence's portion); warp w serves query head w of the
// group, the 16 tokens are the M rows of mma.sync.m16n8k16 tiles.  Key tiles of 64 cached rows arrive by
// cp.async into a double-buffered shared-memory tile that all heads of the group read twice: as keys
// (S = Q K^T, then times 1/rms(k) per key, scale, soft cap, distance penalty, chunk and causal mask) and, through
// ldmatrix.trans, as values (O += P K).  Online softmax in fp32 registers starting from the sink's state
// (maximum 0, denominator 1); the weights are rounded to bf16 before they are summed, as the value product
// sees them.  A decoded token is a tile with one live row.  Key tiles start at the chunk start of the tile's
// first token.
// ------------------------------------------------------------------------------------------------
constexpr int CATT_KEYS = 64;
// The tensor-core kernels serve the bf16 model only: their softmax weights are rounded to bf16 (2^-9), so the
// hardware exponential / logarithm (about 2^-21 relative) replace the full-precision library routines, which
// were the larger part of the instruction stream.  tanh(x) = 1 - 2 / (e^2x + 1), exact in both limits.
__device__ __forceinline__ float fast_tanh(float x) { return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f); }
// 1/rms of a cached key row of D bf16 values (one thread, 16-byte shared-memory loads, fixed order)
template <int D>
__device__ __forceinline__ float key_inv_rms(const bf16* row, float eps) {
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int c = 0; c < D / 8; ++c) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + c * 8);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      s0 = fmaf(bf16_lo(w[e]), bf16_lo(w[e]), s0);
      s1 = fmaf(bf16_hi(w[e]), bf16_hi(w[e]), s1);
    }
  }
  return rsqrtf((s0 + s1) / (float)D + eps);
}
template <int D>
__global__ void __launch_bounds__(256) chunk_attn_mma_kernel(const float* __restrict__ qs, const bf16* __restrict__ cache,
                                                             const int32_t* __restrict__ block_table, int bt_stride,
                                                             const int32_t* __restrict__ seq_desc, int heads,
                                                             int kv_heads, int block_size, int chunk, float scale,
                                                             float softcap, const float* __restrict__ r1,
                                                             const float* __restrict__ r2, const bf16* __restrict__ gate,
                                                             int ld_gate, float eps, bf16* __restrict__ out,
                                                             int skip_single) {
  constexpr int LDS = D + 8;  // padded row (bf16 elements): ldmatrix rows fall on different banks
  extern __shared__ __align__(16) uint8_t smraw[];
  const int nw = blockDim.x >> 5;
  bf16* qsm = reinterpret_cast<bf16*>(smraw);                 // [nw][16][LDS]
  bf16* kbuf = qsm + (long long)nw * 16 * LDS;                // [2][64][LDS]
  float* kinv = reinterpret_cast<float*>(kbuf + 2 * CATT_KEYS * LDS);  // [2][64]
  const SeqView sq = seq_view(seq_desc, blockIdx.x);
  const int r0 = blockIdx.z * 16;
  if (r0 >= sq.n || (skip_single && sq.n == 1)) return;  // single tokens: the decode kernel's
  const int nrows = min(16, sq.n - r0);
  const int rep = heads / kv_heads, parts = (rep + nw - 1) / nw;
  const int g = blockIdx.y / parts, part = blockIdx.y % parts;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, q4 = lane & 3;
  const int hg = part * nw + warp;
  const bool live = hg < rep;
  const int h = g * rep + (live ? hg : 0);
  const int p_first = sq.pos0 + r0, p_last = p_first + nrows - 1;
  const int lo_first = chunk > 0 ? p_first - p_first % chunk : 0;
  const int32_t* bt = block_table + (long long)blockIdx.x * bt_stride;
  const int GD = kv_heads * D;
  const int ntiles = (p_last - lo_first) / CATT_KEYS + 1;

  auto load_tile = [&](int c, int buf) {
    const int j0 = lo_first + c * CATT_KEYS;
    bf16* kb = kbuf + (long long)buf * CATT_KEYS * LDS;
    constexpr int CPR = D / 8;  // 16-byte pieces of a key row
    for (int e = tid; e < CATT_KEYS * CPR; e += blockDim.x) {
      const int j = e / CPR, ck = e % CPR, pos = j0 + j;
      bf16* dst = kb + j * LDS + ck * 8;
      if (pos <= p_last) {
        const long long row = (long long)bt[pos / block_size] * block_size + pos % block_size;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)),
                     "l"(cache + row * GD + (long long)g * D + ck * 8)
                     : "memory");
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_tile(0, 0);
  // the queries of this CTA's heads (norm weights folded in), bf16, rows past the portion are zeros
  for (int e = tid; e < nw * 16 * D; e += blockDim.x) {
    const int w = e / (16 * D), r = (e / D) % 16, d = e % D, hh = part * nw + w;
    const float v = (hh < rep && r < nrows) ? qs[((long long)(sq.row0 + r0 + r) * heads + g * rep + hh) * D + d] : 0.f;
    qsm[((long long)w * 16 + r) * LDS + d] = __float2bfloat16_rn(v);
  }
  const uint32_t q_s = smem_u32(qsm + (long long)warp * 16 * LDS);
  const uint32_t a_off = (uint32_t)(((lane & 15) * LDS + (lane >> 4) * 8) * 2);
  const uint32_t kq_off = (uint32_t)((((lane & 7) + 8 * (lane >> 4)) * LDS + 8 * ((lane >> 3) & 1)) * 2);
  const float c1 = r1[h], c2 = r2[h], inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  // rows gq and gq + 8 of the tile belong to this thread
  int p_row[2], lo_row[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = gq + 8 * r;
    p_row[r] = i < nrows ? p_first + i : -1;  // a dead row sees no key
    lo_row[r] = (chunk > 0 && i < nrows) ? p_row[r] - p_row[r] % chunk : 0;
  }
  float m_[2] = {0.f, 0.f}, l_[2] = {q4 == 0 ? 1.f : 0.f, q4 == 0 ? 1.f : 0.f};  // the sink, counted once per row
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int c = 0; c < ntiles; ++c) {
    const int buf = c & 1, j0 = lo_first + c * CATT_KEYS;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // tile c (and, first time, the queries) is in shared memory; tile c-1 is done with
    if (c + 1 < ntiles) load_tile(c + 1, buf ^ 1);
    const bf16* kb = kbuf + (long long)buf * CATT_KEYS * LDS;
    float* kiv = kinv + buf * CATT_KEYS;
    for (int j = tid; j < CATT_KEYS; j += blockDim.x) kiv[j] = key_inv_rms<D>(kb + j * LDS, eps);  // thread per key
    __syncthreads();
    if (!live) continue;
    const uint32_t kb_s = smem_u32(kb);
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(q_s + a_off + ks * 32, a0, a1, a2, a3);
#pragma unroll
      for (int nt2 = 0; nt2 < 4; ++nt2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kb_s + kq_off + (uint32_t)(nt2 * 16 * LDS * 2 + ks * 32), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * nt2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s[2 * nt2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // ---- scores -> capped, penalised, masked; online softmax over the tile ----
    float rmax[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kk = nt * 8 + 2 * q4 + (e & 1), j = j0 + kk, r = e >> 1;
        float v = -INFINITY;
        if (j <= p_row[r] && j >= lo_row[r]) {
          v = s[nt][e] * kiv[kk] * scale;
          if (softcap > 0.f) v = softcap * fast_tanh(v * inv_cap);
          v -= c1 * __logf(fmaf(c2, (float)(p_row[r] - j), 1.f));
        }
        s[nt][e] = v;
        rmax[r] = fmaxf(rmax[r], v);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 1));
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 2));
      const float mn = fmaxf(m_[r], rmax[r]);
      corr[r] = __expf(m_[r] - mn);
      m_[r] = mn;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = round_bf16(__expf(s[nt][e] - m_[e >> 1]));  // masked: exp(-inf) = 0
        s[nt][e] = pv;
        psum[e >> 1] += pv;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_[r] = l_[r] * corr[r] + psum[r];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    // ---- O += P V, the values being the raw keys of the same tile ----
#pragma unroll
    for (int kk2 = 0; kk2 < CATT_KEYS / 16; ++kk2) {
      const uint32_t a0 = pack_bf16x2(s[2 * kk2][0], s[2 * kk2][1]), a1 = pack_bf16x2(s[2 * kk2][2], s[2 * kk2][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kk2 + 1][0], s[2 * kk2 + 1][1]),
                     a3 = pack_bf16x2(s[2 * kk2 + 1][2], s[2 * kk2 + 1][3]);
      const int key = kk2 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const uint32_t v_row = kb_s + (uint32_t)((key * LDS + 8 * (lane >> 4)) * 2);
#pragma unroll
      for (int nd2 = 0; nd2 < D / 16; ++nd2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(v_row + nd2 * 32, b0, b1, b2, b3);
        mma_bf16_16816(o[2 * nd2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(o[2 * nd2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  if (!live) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 1);
    l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = gq + 8 * r;
    if (i >= nrows) continue;
    const long long t = sq.row0 + r0 + i;
    const float inv = 1.f / l_[r];
    const bf16* gr = gate + t * ld_gate + (long long)h * D;
    bf16* orow = out + (t * heads + h) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      const int d = nt * 8 + 2 * q4;
      const float g0 = sigmoidf_(__bfloat162float(gr[d])), g1 = sigmoidf_(__bfloat162float(gr[d + 1]));
      *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16x2(o[nt][2 * r] * inv * g0, o[nt][2 * r + 1] * inv * g1);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// The same for a single decoded token of a sequence: one CTA (4 warps) per (sequence, key/value head).  The M
// rows of the tiles are the query heads of the group (<= 16), so one pass over the cached keys serves all of
// them; warp w takes the 32-key tiles w, w+4, ... of the token's chunk through its own double-buffered
// cp.async ring (no CTA barrier inside the loop) and keeps its own softmax state; the four states are merged
// through shared memory in a fixed order at the end.  The sink is counted by warp 0.
// ------------------------------------------------------------------------------------------------
constexpr int CDEC_KEYS = 32, CDEC_WARPS = 4;
template <int D>
__global__ void __launch_bounds__(128) chunk_attn_decode_mma_kernel(const float* __restrict__ qs,
                                                                    const bf16* __restrict__ cache,
                                                                    const int32_t* __restrict__ block_table,
                                                                    int bt_stride, const int32_t* __restrict__ seq_desc,
                                                                    int heads, int kv_heads, int block_size, int chunk,
                                                                    float scale, float softcap,
                                                                    const float* __restrict__ r1,
                                                                    const float* __restrict__ r2,
                                                                    const bf16* __restrict__ gate, int ld_gate, float eps,
                                                                    bf16* __restrict__ out) {
  constexpr int LDS = D + 8;
  extern __shared__ __align__(16) uint8_t smraw[];
  bf16* qsm = reinterpret_cast<bf16*>(smraw);                              // [16][LDS]
  bf16* kbuf = qsm + 16 * LDS;                                             // [4 warps][2][32][LDS]
  float* kinv = reinterpret_cast<float*>(kbuf + CDEC_WARPS * 2 * CDEC_KEYS * LDS);  // [4][32]
  float* mrg = reinterpret_cast<float*>(kbuf);                             // after the loop: [4][16][D + 2]
  const SeqView sq = seq_view(seq_desc, blockIdx.x);
  if (sq.n != 1) return;  // portions of prompts take the tile kernel
  const int g = blockIdx.y, rep = heads / kv_heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, q4 = lane & 3;
  const int p = sq.pos0, lo = chunk > 0 ? p - p % chunk : 0;
  const long long t = sq.row0;
  const int32_t* bt = block_table + (long long)blockIdx.x * bt_stride;
  const int GD = kv_heads * D;
  const int ntiles = (p - lo) / CDEC_KEYS + 1;
  bf16* kw = kbuf + (long long)warp * 2 * CDEC_KEYS * LDS;
  float* kiv = kinv + warp * CDEC_KEYS;

  auto load_tile = [&](int c, int buf) {  // by this warp alone
    const int j0 = lo + c * CDEC_KEYS;
    bf16* kb = kw + (long long)buf * CDEC_KEYS * LDS;
    constexpr int CPR = D / 8;
    for (int e = lane; e < CDEC_KEYS * CPR; e += 32) {
      const int j = e / CPR, ck = e % CPR, pos = j0 + j;
      bf16* dst = kb + j * LDS + ck * 8;
      if (pos <= p) {
        const long long row = (long long)bt[pos / block_size] * block_size + pos % block_size;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)),
                     "l"(cache + row * GD + (long long)g * D + ck * 8)
                     : "memory");
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (warp < ntiles) load_tile(warp, 0);
  for (int e = tid; e < 16 * D; e += blockDim.x) {
    const int r = e / D, d = e % D;
    qsm[r * LDS + d] = __float2bfloat16_rn(r < rep ? qs[(t * heads + g * rep + r) * D + d] : 0.f);
  }
  __syncthreads();
  const uint32_t q_s = smem_u32(qsm);
  const uint32_t a_off = (uint32_t)(((lane & 15) * LDS + (lane >> 4) * 8) * 2);
  const uint32_t kq_off = (uint32_t)((((lane & 7) + 8 * (lane >> 4)) * LDS + 8 * ((lane >> 3) & 1)) * 2);
  float c1[2], c2[2];
  bool row_on[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int hr = gq + 8 * r;
    row_on[r] = hr < rep;
    c1[r] = row_on[r] ? r1[g * rep + hr] : 0.f;
    c2[r] = row_on[r] ? r2[g * rep + hr] : 0.f;
  }
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const float l0 = (warp == 0 && q4 == 0) ? 1.f : 0.f;  // the sink, counted once per row
  float m_[2] = {0.f, 0.f}, l_[2] = {l0, l0};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int c = warp, it = 0; c < ntiles; c += CDEC_WARPS, ++it) {
    const int buf = it & 1, j0 = lo + c * CDEC_KEYS;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    if (c + CDEC_WARPS < ntiles) load_tile(c + CDEC_WARPS, buf ^ 1);
    const bf16* kb = kw + (long long)buf * CDEC_KEYS * LDS;
    kiv[lane] = key_inv_rms<D>(kb + lane * LDS, eps);  // lane per key
    __syncwarp();
    const uint32_t kb_s = smem_u32(kb);
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(q_s + a_off + ks * 32, a0, a1, a2, a3);
#pragma unroll
      for (int nt2 = 0; nt2 < 2; ++nt2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kb_s + kq_off + (uint32_t)(nt2 * 16 * LDS * 2 + ks * 32), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * nt2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s[2 * nt2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    float rmax[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kk = nt * 8 + 2 * q4 + (e & 1), j = j0 + kk, r = e >> 1;
        float v = -INFINITY;
        if (row_on[r] && j <= p) {
          v = s[nt][e] * kiv[kk] * scale;
          if (softcap > 0.f) v = softcap * fast_tanh(v * inv_cap);
          v -= c1[r] * __logf(fmaf(c2[r], (float)(p - j), 1.f));
        }
        s[nt][e] = v;
        rmax[r] = fmaxf(rmax[r], v);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 1));
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 2));
      const float mn = fmaxf(m_[r], rmax[r]);
      corr[r] = __expf(m_[r] - mn);
      m_[r] = mn;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = round_bf16(__expf(s[nt][e] - m_[e >> 1]));
        s[nt][e] = pv;
        psum[e >> 1] += pv;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_[r] = l_[r] * corr[r] + psum[r];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk2 = 0; kk2 < CDEC_KEYS / 16; ++kk2) {
      const uint32_t a0 = pack_bf16x2(s[2 * kk2][0], s[2 * kk2][1]), a1 = pack_bf16x2(s[2 * kk2][2], s[2 * kk2][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kk2 + 1][0], s[2 * kk2 + 1][1]),
                     a3 = pack_bf16x2(s[2 * kk2 + 1][2], s[2 * kk2 + 1][3]);
      const int key = kk2 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const uint32_t v_row = kb_s + (uint32_t)((key * LDS + 8 * (lane >> 4)) * 2);
#pragma unroll
      for (int nd2 = 0; nd2 < D / 16; ++nd2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(v_row + nd2 * 32, b0, b1, b2, b3);
        mma_bf16_16816(o[2 * nd2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(o[2 * nd2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  // ---- merge the four warps' states: [warp][row][D + 2] = (o..., m, l) ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 1);
    l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 2);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();  // every warp is done with its key buffers: they become the merge area
  constexpr int MS = D + 2;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float* dst = mrg + ((long long)warp * 16 + gq + 8 * r) * MS;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      dst[nt * 8 + 2 * q4] = o[nt][2 * r];
      dst[nt * 8 + 2 * q4 + 1] = o[nt][2 * r + 1];
    }
    if (q4 == 0) {
      dst[D] = m_[r];
      dst[D + 1] = l_[r];
    }
  }
  __syncthreads();
  for (int e = tid; e < rep * D; e += blockDim.x) {
    const int r = e / D, d = e % D;
    float mx = 0.f;
#pragma unroll
    for (int w = 0; w < CDEC_WARPS; ++w) mx = fmaxf(mx, mrg[((long long)w * 16 + r) * MS + D]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < CDEC_WARPS; ++w) {
      const float* src = mrg + ((long long)w * 16 + r) * MS;
      const float f = expf(src[D] - mx);
      num = fmaf(src[d], f, num);
      den = fmaf(src[D + 1], f, den);
    }
    const int h = g * rep + r;
    const float gv = sigmoidf_(__bfloat162float(gate[t * ld_gate + (long long)h * D + d]));
    out[(t * heads + h) * D + d] = __float2bfloat16_rn(num / den * gv);
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_chunk_attn_prep(const void* proj, int ldp, int heads, int kv_heads, int dim, const float* w_qn,
                          const float* w_kn, const int32_t* slot_mapping, float* qs, void* cache, int T_, float eps,
                          int dtype, void* stream) {
  B200Q_CHECK_ARG(proj && w_qn && w_kn && slot_mapping && qs && cache && heads > 0 && kv_heads > 0 && dim > 0 &&
                      ldp >= (heads + kv_heads) * dim && T_ >= 0 && is_dtype(dtype),
                  "chunk_attn_prep: bad argument");
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (chunk_attn_prep_kernel<T><<<T_, 128, 0, as_stream(stream)>>>(
                        (const T*)proj, ldp, heads, kv_heads, dim, w_qn, w_kn, slot_mapping, qs, (T*)cache, eps)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

static int chunk_attn_mma_mode() {  // B200Q_CHUNK_ATTN_MMA=0: the scalar kernel everywhere
  static const int mode = [] {
    const char* v = getenv("B200Q_CHUNK_ATTN_MMA");
    return v ? atoi(v) : 1;
  }();
  return mode;
}

int b200q_chunk_attn(const float* qs, const void* cache, const int32_t* block_table, int bt_stride,
                     const int32_t* row_seq, const int32_t* positions, int T_, int heads, int kv_heads, int dim,
                     int block_size, int chunk, float scale, float softcap, const float* r1, const float* r2,
                     const void* gate, int ld_gate, float eps, void* out, int dtype, void* stream) {
  return b200q_chunk_attn_seq(qs, cache, block_table, bt_stride, row_seq, positions, nullptr, 0, T_, heads, kv_heads, dim,
                              block_size, chunk, scale, softcap, r1, r2, gate, ld_gate, eps, out, dtype, stream);
}

int b200q_chunk_attn_seq(const float* qs, const void* cache, const int32_t* block_table, int bt_stride,
                         const int32_t* row_seq, const int32_t* positions, const int32_t* seq_desc, int n_seqs, int T_,
                         int heads, int kv_heads, int dim, int block_size, int chunk, float scale, float softcap,
                         const float* r1, const float* r2, const void* gate, int ld_gate, float eps, void* out,
                         int dtype, void* stream) {
  B200Q_CHECK_ARG(qs && cache && block_table && row_seq && positions && r1 && r2 && gate && out && heads > 0 &&
                      kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && dim <= 512 && block_size > 0 && chunk >= 0 &&
                      T_ >= 0 && is_dtype(dtype),
                  "chunk_attn: bad argument (heads=%d kv_heads=%d dim=%d (<= 512))", heads, kv_heads, dim);
  if (T_ == 0) return B200Q_OK;
  const int rep = heads / kv_heads;
  // bf16 caches with head sizes the tensor-core tiles take, when the caller gives the per-sequence view
  if (seq_desc && n_seqs > 0 && dtype == B200Q_DTYPE_BF16 && (dim == 64 || dim == 128) && chunk_attn_mma_mode() &&
      ((reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 && (ld_gate & 1) == 0 &&
      (reinterpret_cast<uintptr_t>(gate) & 3) == 0) {
    const int nw = rep < 8 ? rep : 8, parts = (rep + nw - 1) / nw;
    const int ztiles = (T_ - n_seqs + 1 + 15) / 16;  // no portion of this step is longer than T - (n_seqs - 1)
    dim3 mgrid(n_seqs, kv_heads * parts, ztiles);
    B200Q_CHECK_ARG(mgrid.y <= 65535 && mgrid.z <= 65535, "chunk_attn: step too large (%d tokens)", T_);
    const size_t msm = ((size_t)nw * 16 + 2 * CATT_KEYS) * (dim + 8) * 2 + 2 * CATT_KEYS * sizeof(float);
    // single decoded tokens go to the kernel whose rows are the heads of a group (groups of up to 16 heads);
    // a step of single tokens only (T == n_seqs) needs no tile kernel, and the other way round is not known
    // here, so the decode kernel is launched whenever it can serve (sequences with portions leave it at once)
    const bool dec = rep <= 16, tiles = !dec || T_ > n_seqs;
    const size_t dsm = std::max((size_t)(16 + CDEC_WARPS * 2 * CDEC_KEYS) * (dim + 8) * 2 + CDEC_WARPS * CDEC_KEYS * 4,
                                (size_t)16 * (dim + 8) * 2 + (size_t)CDEC_WARPS * 16 * (dim + 2) * 4);
    dim3 dgrid(n_seqs, kv_heads);
#define MMA_ATTN(DD)                                                                                                 \
  do {                                                                                                               \
    if (tiles) {                                                                                                     \
      if (msm > 48 * 1024)                                                                                           \
        B200Q_CUDA(cudaFuncSetAttribute(chunk_attn_mma_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                        (int)msm));                                                                  \
      chunk_attn_mma_kernel<DD><<<mgrid, nw * 32, msm, as_stream(stream)>>>(                                         \
          qs, (const bf16*)cache, block_table, bt_stride, seq_desc, heads, kv_heads, block_size, chunk, scale,       \
          softcap, r1, r2, (const bf16*)gate, ld_gate, eps, (bf16*)out, dec ? 1 : 0);                                \
      B200Q_LAUNCH_CHECK();                                                                                          \
    }                                                                                                                \
    if (dec) {                                                                                                       \
      if (dsm > 48 * 1024)                                                                                           \
        B200Q_CUDA(cudaFuncSetAttribute(chunk_attn_decode_mma_kernel<DD>,                                            \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsm));                     \
      chunk_attn_decode_mma_kernel<DD><<<dgrid, 128, dsm, as_stream(stream)>>>(                                      \
          qs, (const bf16*)cache, block_table, bt_stride, seq_desc, heads, kv_heads, block_size, chunk, scale,       \
          softcap, r1, r2, (const bf16*)gate, ld_gate, eps, (bf16*)out);                                             \
      B200Q_LAUNCH_CHECK();                                                                                          \
    }                                                                                                                \
  } while (0)
    if (dim == 64) MMA_ATTN(64);
    else MMA_ATTN(128);
#undef MMA_ATTN
    return B200Q_OK;
  }
  dim3 grid(T_, kv_heads, (rep + 7) / 8);
  const size_t smem = (size_t)(8 * dim + 32 * (dim + 1) + 32) * sizeof(float);
#define ATTN(TT, ACC)                                                                                               \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      B200Q_CUDA(cudaFuncSetAttribute(chunk_attn_kernel<TT, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                      (int)smem));                                                                  \
    chunk_attn_kernel<TT, ACC><<<grid, 256, smem, as_stream(stream)>>>(                                             \
        qs, (const TT*)cache, block_table, bt_stride, row_seq, positions, heads, kv_heads, dim, block_size, chunk, \
        scale, softcap, r1, r2, (const TT*)gate, ld_gate, eps, (TT*)out);                                           \
  } while (0)
#define ATTN_BY_DIM(TT)                    \
  do {                                     \
    if (dim <= 64) ATTN(TT, 2);            \
    else if (dim <= 128) ATTN(TT, 4);      \
    else if (dim <= 256) ATTN(TT, 8);      \
    else ATTN(TT, 16);                     \
  } while (0)
  if (dtype == B200Q_DTYPE_F32) ATTN_BY_DIM(float);
  else ATTN_BY_DIM(bf16);
#undef ATTN_BY_DIM
#undef ATTN
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"
