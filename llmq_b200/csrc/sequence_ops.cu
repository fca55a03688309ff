// sequence_ops.cu — kernels of the post-norm layered form and of the mixers that carry per-sequence state:
// grouped RMS norm over the scaled residual sum, per-channel causal convolutions continued from the inputs a
// sequence left in its state slot, the gated delta rule, the selective scan, and the pieces of a
// sigmoid-routed mixture whose weight scales the expert's input.  (The attention of the same designs:
// chunk_attn.cu.)
//
// As in layered_ops.cu every kernel is a template over the element type of matrices, activations and cache
// (bf16 or fp32), and what has to be exact is fp32 in both: the residual sum and its norms, scores and
// softmax weights, unit norms, decays, step sizes, gates of the recurrences and the recurrent states.
// Every reduction has a fixed order per row and every loop over keys or tokens starts at a place that
// depends only on the token's position in its sequence (chunk start, sequence start), so a token's result
// does not depend on how its prompt was cut into steps, on its batch-mates, or on pages and slots.
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
// embedding + learned position vector into the fp32 residual
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) embed_pos_kernel(const int32_t* __restrict__ ids,
                                                        const int32_t* __restrict__ prev_out,
                                                        const T* __restrict__ table, const T* __restrict__ pos_table,
                                                        const int32_t* __restrict__ positions,
                                                        float* __restrict__ out, int Tn, int W) {
  const long long total = (long long)Tn * W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / W), c = (int)(i % W);
    int id = __ldg(ids + t);
    if (id < 0) id = prev_out[-1 - id];
    float v = ldf(table + (long long)id * W + c);
    if (pos_table) v += ldf(pos_table + (long long)positions[t] * W + c);
    out[i] = v;
  }
}

// ------------------------------------------------------------------------------------------------
// grouped RMS norm of v = alpha * x + scale * add (one CTA per row; v is kept in shared memory between
// the sums and the scaling, so x may be overwritten in place).  add: the row itself, or the sum of the
// `top` rows pair_pos[r*top + k] (outputs of the routed experts, in ascending k).
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) group_norm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                                         const T* __restrict__ add,
                                                         const int32_t* __restrict__ pair_pos, int top,
                                                         const float* __restrict__ scale, float alpha,
                                                         const float* __restrict__ w, int groups, float eps,
                                                         float* yf, T* __restrict__ yt, int W) {
  extern __shared__ float sm[];
  float* v = sm;        // [W]
  float* inv = sm + W;  // [groups]
  const int r = blockIdx.x;
  const long long src = rows ? rows[r] : r;
  const float* xr = x + src * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float a = 0.f;
    if (add) {
      if (pair_pos) {
        for (int k = 0; k < top; ++k) a += ldf(add + (long long)pair_pos[src * top + k] * W + c);
      } else {
        a = ldf(add + src * W + c);
      }
      if (scale) a *= scale[c];
    }
    v[c] = fmaf(alpha, xr[c], a);
  }
  __syncthreads();
  const int gs = W / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int g = warp; g < groups; g += nw) {
    float ss = 0.f;
    for (int c = lane; c < gs; c += 32) ss = fmaf(v[g * gs + c], v[g * gs + c], ss);
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float y = v[c] * inv[c / gs] * w[c];
    if (yf) yf[(long long)r * W + c] = y;
    if (yt) stf(yt + (long long)r * W + c, y);
  }
}

// ------------------------------------------------------------------------------------------------
// per-channel causal convolution over time, continued across steps.  A sequence's state region holds the
// last taps-1 inputs of the channel, oldest first: entry e is the input at position pos0 - (taps-1) + e.
// Inputs before position 0 are zeros, whatever the slot holds.  One thread per (token, channel).
// ------------------------------------------------------------------------------------------------
constexpr int CONV_MAX_TAPS = 16;
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) causal_conv_kernel(const TI* __restrict__ in, int ld_in,
                                                          const float* __restrict__ w,
                                                          const float* __restrict__ bias, int C, int taps, int act,
                                                          int add_input, const float* __restrict__ state,
                                                          long long slot_stride, const int32_t* __restrict__ seq_desc,
                                                          const int32_t* __restrict__ row_seq, TO* __restrict__ out,
                                                          int ld_out) {
  const int t = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
  if (c >= C) return;
  const SeqView s = seq_view(seq_desc, row_seq[t]);
  const int tt = t - s.row0;
  const float* st = state + (long long)s.slot * slot_stride;
  float acc = bias ? bias[c] : 0.f, cur = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int idx = tt - (taps - 1) + j;  // source token, relative to the first token of this portion
    float xv = 0.f;
    if (idx >= 0) xv = ldf(in + (long long)(s.row0 + idx) * ld_in + c);
    else if (s.pos0 + idx >= 0) xv = st[(long long)(taps - 1 + idx) * C + c];
    acc = fmaf(w[(long long)c * taps + j], xv, acc);
    cur = xv;
  }
  if (act == 1) acc = siluf_(acc);
  if (add_input) acc += cur;
  stf(out + (long long)t * ld_out + c, acc);
}

// the state after the portion: the last taps-1 inputs, taken from the portion and, where it is shorter,
// from the old state (read completely before anything is written)
template <typename TI>
__global__ void __launch_bounds__(256) conv_state_kernel(const TI* __restrict__ in, int ld_in, int C, int taps,
                                                         float* __restrict__ state, long long slot_stride,
                                                         const int32_t* __restrict__ seq_desc) {
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (c >= C) return;
  const SeqView s = seq_view(seq_desc, blockIdx.x);
  float* st = state + (long long)s.slot * slot_stride;
  float keep[CONV_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i) {
    if (i < taps - 1) {
      const int idx = s.n - (taps - 1) + i;
      float xv = 0.f;
      if (idx >= 0) xv = ldf(in + (long long)(s.row0 + idx) * ld_in + c);
      else if (s.pos0 + idx >= 0) xv = st[(long long)(taps - 1 + idx) * C + c];
      keep[i] = xv;
    }
  }
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i)
    if (i < taps - 1) st[(long long)i * C + c] = keep[i];
}

// ------------------------------------------------------------------------------------------------
// gated delta rule, three launches.
//   prepare (CTA per token): q, k -> unit vectors per head (q also times dim^-1/2), in place in the fp32
//           qkv rows; ba row (beta logits | decay inputs) -> (beta | g) in place
//   recur   (one warp per sequence x head x 8 value columns, 4 lanes per column, a quarter of S[0..dim) each):
//           S <- g S;  u = beta (v_j - k.S);  S <- S + k u;  o_j = q.S   -> raw [T, heads*vdim] (fp32)
//   finish  (CTA per token x head): out = raw / rms(raw) * out_norm * silu(gate)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) gdelta_prepare_kernel(float* __restrict__ qkv, float* __restrict__ ba,
                                                             const float* __restrict__ a_log,
                                                             const float* __restrict__ dt_bias, int heads,
                                                             int kv_heads, int dim, int vdim) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ldq = 2 * kv_heads * dim + heads * vdim;
  float* row = qkv + (long long)t * ldq;
  const float qs = 1.f / sqrtf((float)dim);
  for (int vh = warp; vh < 2 * kv_heads; vh += 4) {  // vectors 0..G-1: q heads, G..2G-1: k heads
    float* p = row + (long long)vh * dim;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss = fmaf(p[d], p[d], ss);
    ss = warp_sum(ss);
    const float inv = (vh < kv_heads ? qs : 1.f) / sqrtf(ss + 1e-6f);
    for (int d = lane; d < dim; d += 32) p[d] *= inv;
  }
  float* b = ba + (long long)t * 2 * heads;
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    const float beta = sigmoidf_(b[h]);
    // the decay constant is the same for every token of a head: an error in exp(a_log) would add up over a
    // sequence instead of averaging out, so this handful of values per token is evaluated in fp64
    const double sp = (double)b[heads + h] + (double)dt_bias[h];
    const float g = (float)exp(-exp((double)a_log[h]) * (sp > 30.0 ? sp : log1p(exp(sp))));
    b[h] = beta;
    b[heads + h] = g;
  }
}

// One warp per (sequence, head, 8 value columns): columns are independent, so a head's state is spread over
// vdim/8 CTAs, and inside the warp every column is shared by 4 lanes that each keep a quarter of the column
// (dim/4 values, zero-padded) in registers and sum their partial dot products by two butterfly shuffles — a
// single warp is bound by its own instruction stream, and there are far more SMs than (sequence, head) pairs
// in a prompt step.  k and q of 8 tokens at a time arrive in shared memory by cp.async one group ahead of the
// one being consumed, v of the group is prefetched into registers.
constexpr int GDELTA_G = 8, GDELTA_COLS = 8;
__device__ __forceinline__ void cp_async16_(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
template <int DT>
__global__ void __launch_bounds__(32) gdelta_recur_kernel(const float* __restrict__ qkv, const float* __restrict__ bg,
                                                          float* __restrict__ state, long long slot_stride,
                                                          const int32_t* __restrict__ seq_desc, int heads, int kv_heads,
                                                          int dim, int vdim, float* __restrict__ raw) {
  constexpr int QL = DT / 4;  // state values per lane
  extern __shared__ __align__(16) float sm[];  // [2][G][2*DT]: k (padded to DT) then q (padded to DT)
  const SeqView s = seq_view(seq_desc, blockIdx.x);
  const int h = blockIdx.y, lane = threadIdx.x, sub = lane >> 3, j = blockIdx.z * GDELTA_COLS + (lane & 7);
  const int kvh = h / (heads / kv_heads), q0 = sub * QL;
  const int GD = kv_heads * dim, ldq = 2 * GD + heads * vdim, HV = heads * vdim;
  const bool on = j < vdim;
  // 16-byte copies need every k and q vector to start on a 16-byte boundary: head size, row stride and base
  const bool vec = (dim & 3) == 0 && (ldq & 3) == 0 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0;
  float* st = state + (long long)s.slot * slot_stride + (long long)h * dim * vdim;
  for (int e = lane; e < 2 * GDELTA_G * 2 * DT; e += 32) sm[e] = 0.f;  // the padding stays zero
  __syncwarp();
  auto fetch = [&](int g0, int buf) {
    const int cnt = min(GDELTA_G, s.n - g0);
    float* dst0 = sm + (long long)buf * GDELTA_G * 2 * DT;
    if (vec) {
      const int per = dim / 2;  // 16-byte pieces of one token: dim/4 of k, dim/4 of q
      for (int e = lane; e < cnt * per; e += 32) {
        const int tk = e / per, pc = e % per;
        const float* r = qkv + (long long)(s.row0 + g0 + tk) * ldq + kvh * dim;
        const bool isq = pc >= dim / 4;
        const int off = (isq ? pc - dim / 4 : pc) * 4;
        cp_async16_(dst0 + tk * 2 * DT + (isq ? DT : 0) + off, r + (isq ? 0 : GD) + off);
      }
    } else {
      for (int e = lane; e < cnt * 2 * dim; e += 32) {
        const int tk = e / (2 * dim), i = e % (2 * dim);
        const float* r = qkv + (long long)(s.row0 + g0 + tk) * ldq + kvh * dim;
        dst0[tk * 2 * DT + (i < dim ? i : DT + i - dim)] = i < dim ? r[GD + i] : r[i - dim];
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(0, 0);
  float S[QL];
#pragma unroll
  for (int q = 0; q < QL; ++q) S[q] = (on && q0 + q < dim && s.pos0 > 0) ? st[(long long)(q0 + q) * vdim + j] : 0.f;
  for (int g0 = 0, buf = 0; g0 < s.n; g0 += GDELTA_G, buf ^= 1) {
    const int cnt = min(GDELTA_G, s.n - g0);
    float vj[GDELTA_G];
#pragma unroll
    for (int tk = 0; tk < GDELTA_G; ++tk)
      vj[tk] = (on && tk < cnt) ? qkv[(long long)(s.row0 + g0 + tk) * ldq + 2 * GD + h * vdim + j] : 0.f;
    // lane tk holds (beta, g) of token tk of the group
    float my_b = 0.f, my_g = 1.f;
    if (lane < cnt) {
      const float* b = bg + (long long)(s.row0 + g0 + lane) * 2 * heads;
      my_b = b[h];
      my_g = b[heads + h];
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();  // this group has landed; the other buffer is no longer read
    if (g0 + GDELTA_G < s.n) fetch(g0 + GDELTA_G, buf ^ 1);
    const float* base = sm + (long long)buf * GDELTA_G * 2 * DT + q0;
#pragma unroll
    for (int tk = 0; tk < GDELTA_G; ++tk) {
      if (tk < cnt) {
        const float beta = __shfl_sync(0xffffffffu, my_b, tk), g = __shfl_sync(0xffffffffu, my_g, tk);
        const float4* k4 = reinterpret_cast<const float4*>(base + tk * 2 * DT);
        const float4* q4 = reinterpret_cast<const float4*>(base + tk * 2 * DT + DT);
        float u0 = 0.f, u1 = 0.f, u2 = 0.f, u3 = 0.f;
#pragma unroll
        for (int q = 0; q < QL / 4; ++q) {
          const float4 k = k4[q];
          S[4 * q] *= g;
          S[4 * q + 1] *= g;
          S[4 * q + 2] *= g;
          S[4 * q + 3] *= g;
          u0 = fmaf(k.x, S[4 * q], u0);
          u1 = fmaf(k.y, S[4 * q + 1], u1);
          u2 = fmaf(k.z, S[4 * q + 2], u2);
          u3 = fmaf(k.w, S[4 * q + 3], u3);
        }
        float kS = (u0 + u1) + (u2 + u3);  // this lane's quarter; the column's sum over its four lanes
        kS += __shfl_xor_sync(0xffffffffu, kS, 8);
        kS += __shfl_xor_sync(0xffffffffu, kS, 16);
        const float u = beta * (vj[tk] - kS);
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int q = 0; q < QL / 4; ++q) {
          const float4 k = k4[q], qq = q4[q];
          S[4 * q] = fmaf(k.x, u, S[4 * q]);
          S[4 * q + 1] = fmaf(k.y, u, S[4 * q + 1]);
          S[4 * q + 2] = fmaf(k.z, u, S[4 * q + 2]);
          S[4 * q + 3] = fmaf(k.w, u, S[4 * q + 3]);
          o0 = fmaf(S[4 * q], qq.x, o0);
          o1 = fmaf(S[4 * q + 1], qq.y, o1);
          o2 = fmaf(S[4 * q + 2], qq.z, o2);
          o3 = fmaf(S[4 * q + 3], qq.w, o3);
        }
        float o = (o0 + o1) + (o2 + o3);
        o += __shfl_xor_sync(0xffffffffu, o, 8);
        o += __shfl_xor_sync(0xffffffffu, o, 16);
        if (on && sub == 0) raw[(long long)(s.row0 + g0 + tk) * HV + h * vdim + j] = o;
      }
    }
  }
  if (on) {
#pragma unroll
    for (int q = 0; q < QL; ++q)
      if (q0 + q < dim) st[(long long)(q0 + q) * vdim + j] = S[q];
  }
}

template <typename T>
__global__ void gdelta_finish_kernel(const float* __restrict__ raw, const T* __restrict__ gate, int ld_gate,
                                     const float* __restrict__ out_norm, int heads, int vdim, float eps,
                                     T* __restrict__ out) {
  __shared__ float red[32];
  const int t = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const bool on = j < vdim;
  const long long at = (long long)t * heads * vdim + h * vdim + j;
  const float o = on ? raw[at] : 0.f;
  const float sso = block_sum(o * o, red);
  if (on) {
    const float gv = siluf_(ldf(gate + (long long)t * ld_gate + h * vdim + j));
    stf(out + at, o / sqrtf(sso / (float)vdim + eps) * out_norm[j] * gv);
  }
}

// ------------------------------------------------------------------------------------------------
// selective scan: one CTA per (sequence, 32 channels); four lanes share a channel, each with a quarter of its
// state S[0..N) and of its decay rates A[n] = -exp(a_log) in registers, their partial outputs summed by two
// butterfly shuffles (a prompt step has few sequences and a warp is bound by its own instruction stream, so
// the channel's chain is cut in four).  B and C of 8 tokens at a time are staged in shared memory (they are
// shared by all channels), the channel's own inputs of the group are prefetched into registers.  State layout
// in the slot: [N][inner].
// ------------------------------------------------------------------------------------------------
constexpr int SCAN_G = 8, SCAN_CH = 32;  // tokens staged per barrier pair; channels per CTA (8 per warp)
// exp of a decay exponent: correctly rounded (through fp64) in the fp32 model, where a thousand decays of one
// state entry multiply up; the fast fp32 exponential in the bf16 model
template <typename T> __device__ __forceinline__ float decay_of(float x);
template <> __device__ __forceinline__ float decay_of<float>(float x) { return (float)exp((double)x); }
template <> __device__ __forceinline__ float decay_of<bf16>(float x) { return expf(x); }
template <typename T, int NT, int LPC>
__global__ void __launch_bounds__(128) selective_scan_kernel(const T* __restrict__ x, const float* __restrict__ dt_raw,
                                                             const float* __restrict__ dt_bias,
                                                             const T* __restrict__ bc, int ld_bc, int b_off,
                                                             const T* __restrict__ z, int ld_z,
                                                             const float* __restrict__ a_log,
                                                             const float* __restrict__ dvec, float* __restrict__ state,
                                                             long long slot_stride,
                                                             const int32_t* __restrict__ seq_desc, int inner, int N,
                                                             T* __restrict__ out) {
  // LPC lanes share a channel: 4 in steps that hold prompt portions (few sequences, long chains), 1 in steps
  // of single tokens (the state traffic is what counts there, and whole-warp rows of it are read at once)
  constexpr int NL = NT / LPC;   // states per lane
  extern __shared__ float sm[];  // [G][2N]
  const SeqView s = seq_view(seq_desc, blockIdx.x);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = LPC == 4 ? lane >> 3 : 0;
  const int c = LPC == 4 ? blockIdx.y * SCAN_CH + warp * 8 + (lane & 7) : blockIdx.y * 128 + (int)threadIdx.x;
  const int n0 = sub * NL;
  const bool on = c < inner;
  float* st = state + (long long)s.slot * slot_stride;
  float S[NL], A[NL];
#pragma unroll
  for (int i = 0; i < NL; ++i) {
    const int n = n0 + i;
    const bool in = on && n < N;
    S[i] = (in && s.pos0 > 0) ? st[(long long)n * inner + c] : 0.f;
    // a rate is used at every token: its error would add up over a sequence, so it is rounded once, from fp64
    A[i] = in ? -(float)exp((double)a_log[(long long)c * N + n]) : 0.f;
  }
  const float dc = on ? dvec[c] : 0.f, dtb = (on && dt_bias) ? dt_bias[c] : 0.f;
  for (int g0 = 0; g0 < s.n; g0 += SCAN_G) {
    const int cnt = min(SCAN_G, s.n - g0);
    // this channel's inputs of the whole group are fetched before the chain starts
    float dtv[SCAN_G], xs[SCAN_G], zs[SCAN_G];
#pragma unroll
    for (int tk = 0; tk < SCAN_G; ++tk) {
      const bool ok = on && tk < cnt;
      const long long r = s.row0 + g0 + tk;
      dtv[tk] = ok ? dt_raw[r * inner + c] : 0.f;
      xs[tk] = ok ? ldf(x + r * inner + c) : 0.f;
      zs[tk] = ok ? ldf(z + r * ld_z + c) : 0.f;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < cnt * 2 * N; e += blockDim.x) {
      const int tk = e / (2 * N), i = e % (2 * N);
      sm[e] = ldf(bc + (long long)(s.row0 + g0 + tk) * ld_bc + b_off + i);
    }
    __syncthreads();
#pragma unroll
    for (int tk = 0; tk < SCAN_G; ++tk) {
      if (tk < cnt) {
        const long long r = s.row0 + g0 + tk;
        const float* Bv = sm + tk * 2 * N + n0;
        const float* Cv = Bv + N;
        const float dt = softplusf_(dtv[tk] + dtb), xv = xs[tk], dx = dt * xv;
        float y = 0.f;
#pragma unroll
        for (int i = 0; i < NL; ++i)
          if (n0 + i < N) {
            S[i] = fmaf(decay_of<T>(dt * A[i]), S[i], dx * Bv[i]);
            y = fmaf(S[i], Cv[i], y);
          }
        if constexpr (LPC == 4) {  // the channel's sum over its four lanes
          y += __shfl_xor_sync(0xffffffffu, y, 8);
          y += __shfl_xor_sync(0xffffffffu, y, 16);
        }
        y = fmaf(dc, xv, y);
        if (on && sub == 0) stf(out + r * inner + c, y * siluf_(zs[tk]));
      }
    }
  }
  if (on) {
#pragma unroll
    for (int i = 0; i < NL; ++i)
      if (n0 + i < N) st[(long long)(n0 + i) * inner + c] = S[i];
  }
}

// ------------------------------------------------------------------------------------------------
// pieces of a mixture whose routing weight scales the expert's input
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) scatter_scaled_rows_kernel(const T* __restrict__ src,
                                                                  const int32_t* __restrict__ pair_pos,
                                                                  const float* __restrict__ wts, int top,
                                                                  T* __restrict__ dst, long long pairs, int W) {
  const long long total = pairs * W;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long p = e / W;
    const int c = (int)(e % W);
    stf(dst + (long long)pair_pos[p] * W + c, ldf(src + (p / top) * W + c) * wts[p]);
  }
}
// bf16 rows of a multiple of 8 values, 16-byte aligned: 8 values per thread
__global__ void __launch_bounds__(256) scatter_scaled_rows_v8_kernel(const bf16* __restrict__ src,
                                                                     const int32_t* __restrict__ pair_pos,
                                                                     const float* __restrict__ wts, int top,
                                                                     bf16* __restrict__ dst, long long pairs, int W) {
  const int per = W / 8;
  const long long total = pairs * per;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long p = e / per;
    const int c = (int)(e % per) * 8;
    const float w = wts[p];
    const uint4 v = ld_v4(src + (p / top) * W + c);
    const uint32_t in[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = pack_bf16x2(bf16_lo(in[i]) * w, bf16_hi(in[i]) * w);
    st_v4(dst + (long long)pair_pos[p] * W + c, make_uint4(o[0], o[1], o[2], o[3]));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) silu_glu_kernel(const T* __restrict__ gu, T* __restrict__ y, long long rows,
                                                       int F) {
  const long long total = rows * F;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / F;
    const int c = (int)(e % F);
    stf(y + e, siluf_(ldf(gu + r * 2 * F + c)) * ldf(gu + r * 2 * F + F + c));
  }
}
__global__ void __launch_bounds__(256) silu_glu_v8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ y,
                                                          long long rows, int F) {
  const int per = F / 8;
  const long long total = rows * per;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / per;
    const int c = (int)(e % per) * 8;
    const uint4 g = ld_v4(gu + r * 2 * F + c), u = ld_v4(gu + r * 2 * F + F + c);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      o[i] = pack_bf16x2(siluf_(bf16_lo(gw[i])) * bf16_lo(uw[i]), siluf_(bf16_hi(gw[i])) * bf16_hi(uw[i]));
    st_v4(y + r * F + c, make_uint4(o[0], o[1], o[2], o[3]));
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_embed_pos_f32(const int32_t* ids, const int32_t* prev_out, const void* table, const void* pos_table,
                        const int32_t* positions, float* out, int T_, int W, int dtype, void* stream) {
  B200Q_CHECK_ARG(ids && table && out && T_ >= 0 && W > 0 && is_dtype(dtype) && (!pos_table || positions),
                  "embed_pos_f32: bad argument");
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (embed_pos_kernel<T><<<grid_for((long long)T_ * W), 256, 0, as_stream(stream)>>>(
                        ids, prev_out, (const T*)table, (const T*)pos_table, positions, out, T_, W)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_group_rmsnorm(const float* x, const int32_t* rows, const void* add, const int32_t* pair_pos, int top,
                        const float* scale, float alpha, const float* w, int groups, float eps, float* y_f32,
                        void* y_t, int n, int W, int dtype, void* stream) {
  if (groups <= 0) groups = 1;
  B200Q_CHECK_ARG(x && w && (y_f32 || y_t) && n >= 0 && W > 0 && is_dtype(dtype) && W % groups == 0 &&
                      (!pair_pos || (add && top > 0)) && (!rows || !add),
                  "group_rmsnorm: bad argument (W=%d groups=%d)", W, groups);
  if (n == 0) return B200Q_OK;
  const size_t smem = (size_t)(W + groups) * sizeof(float);
  B200Q_CHECK_ARG(smem <= 200 * 1024, "group_rmsnorm: a row of %d does not fit shared memory", W);
  DISPATCH_T(dtype, {
    if (smem > 48 * 1024)
      B200Q_CUDA(cudaFuncSetAttribute(group_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    group_norm_kernel<T><<<n, 256, smem, as_stream(stream)>>>(x, rows, (const T*)add, pair_pos, top, scale, alpha, w,
                                                              groups, eps, y_f32, (T*)y_t, W);
  });
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_causal_conv(const void* in, int ld_in, int in_f32, const float* w, const float* bias, int C, int taps,
                      int act, int add_input, float* state, long long slot_stride, const int32_t* seq_desc,
                      const int32_t* row_seq, int n_seqs, void* out, int ld_out, int out_f32, int T_, int dtype,
                      void* stream) {
  B200Q_CHECK_ARG(in && w && (state || taps == 1) && seq_desc && row_seq && out && C > 0 && taps >= 1 &&
                      taps <= CONV_MAX_TAPS &&
                      ld_in >= C && ld_out >= C && n_seqs >= 0 && T_ >= 0 && is_dtype(dtype) && (act == 0 || act == 1),
                  "causal_conv: bad argument (C=%d taps=%d, at most %d taps)", C, taps, CONV_MAX_TAPS);
  if (T_ == 0 || n_seqs == 0) return B200Q_OK;
  const bool fi = in_f32 || dtype == B200Q_DTYPE_F32, fo = out_f32 || dtype == B200Q_DTYPE_F32;
  cudaStream_t st = as_stream(stream);
  dim3 grid(T_, (C + 255) / 256), sgrid(n_seqs, (C + 255) / 256);
#define CONV(TI, TO)                                                                                              \
  do {                                                                                                            \
    causal_conv_kernel<TI, TO><<<grid, 256, 0, st>>>((const TI*)in, ld_in, w, bias, C, taps, act, add_input, state, \
                                                     slot_stride, seq_desc, row_seq, (TO*)out, ld_out);           \
    B200Q_LAUNCH_CHECK();                                                                                         \
    if (taps > 1) {                                                                                               \
      conv_state_kernel<TI><<<sgrid, 256, 0, st>>>((const TI*)in, ld_in, C, taps, state, slot_stride, seq_desc);  \
      B200Q_LAUNCH_CHECK();                                                                                       \
    }                                                                                                             \
  } while (0)
  if (fi && fo) CONV(float, float);
  else if (fi) CONV(float, bf16);
  else if (fo) CONV(bf16, float);
  else CONV(bf16, bf16);
#undef CONV
  return B200Q_OK;
}

int b200q_gated_delta(float* qkv, float* ba, float* raw, const void* gate, int ld_gate, const float* a_log,
                      const float* dt_bias, const float* out_norm, float* state, long long slot_stride,
                      const int32_t* seq_desc, int n_seqs, int heads, int kv_heads, int dim, int vdim, float eps,
                      void* out, int T_, int dtype, void* stream) {
  B200Q_CHECK_ARG(qkv && ba && raw && gate && a_log && dt_bias && out_norm && state && seq_desc && out && heads > 0 &&
                      kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && dim <= 256 && vdim > 0 && vdim <= 1024 &&
                      n_seqs >= 0 && T_ >= 0 && is_dtype(dtype),
                  "gated_delta: bad argument (heads=%d kv_heads=%d dim=%d (<= 256) vdim=%d (<= 1024))", heads,
                  kv_heads, dim, vdim);
  if (n_seqs == 0 || T_ == 0) return B200Q_OK;
  cudaStream_t st = as_stream(stream);
  float* q = qkv;
  float* b = ba;
  gdelta_prepare_kernel<<<T_, 128, 0, st>>>(q, b, a_log, dt_bias, heads, kv_heads, dim, vdim);
  B200Q_LAUNCH_CHECK();
  const int threads = (vdim + 31) & ~31;
  dim3 grid(n_seqs, heads, (vdim + GDELTA_COLS - 1) / GDELTA_COLS);
  B200Q_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "gated_delta: too many heads or value columns");
#define RECUR(DT)                                                                                                  \
  do {                                                                                                             \
    const size_t smem = (size_t)2 * GDELTA_G * 2 * DT * sizeof(float);                                             \
    gdelta_recur_kernel<DT><<<grid, 32, smem, st>>>(q, b, state, slot_stride, seq_desc, heads, kv_heads, dim, vdim, \
                                                    raw);                                                          \
  } while (0)
  if (dim <= 32) RECUR(32);
  else if (dim <= 64) RECUR(64);
  else if (dim <= 128) RECUR(128);
  else RECUR(256);
#undef RECUR
  B200Q_LAUNCH_CHECK();
  dim3 fgrid(T_, heads);
  DISPATCH_T(dtype, (gdelta_finish_kernel<T><<<fgrid, threads, 0, st>>>(raw, (const T*)gate, ld_gate, out_norm, heads,
                                                                        vdim, eps, (T*)out)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_selective_scan(const void* x, const float* dt_raw, const float* dt_bias, const void* bc, int ld_bc, int b_off,
                         const void* z,
                         int ld_z, const float* a_log, const float* d, float* state, long long slot_stride,
                         const int32_t* seq_desc, int n_seqs, int inner, int N, void* out, int T_, int dtype,
                         void* stream) {
  B200Q_CHECK_ARG(x && dt_raw && bc && z && a_log && d && state && seq_desc && out && inner > 0 && N > 0 && N <= 256 &&
                      b_off >= 0 && ld_bc >= b_off + 2 * N && ld_z >= inner && n_seqs >= 0 && is_dtype(dtype),
                  "selective_scan: bad argument (inner=%d state=%d (<= 256))", inner, N);
  if (n_seqs == 0) return B200Q_OK;
  // a step with prompt portions: four lanes per channel; so are states too large for one lane's registers
  const bool split = T_ > n_seqs || N > 64;
  dim3 grid(n_seqs, split ? (inner + SCAN_CH - 1) / SCAN_CH : (inner + 127) / 128);
  B200Q_CHECK_ARG(grid.y <= 65535, "selective_scan: too many channels (%d)", inner);
  const size_t smem = (size_t)SCAN_G * 2 * N * sizeof(float);
#define SCAN(TT, NT, LPC)                                                                                         \
  selective_scan_kernel<TT, NT, LPC><<<grid, 128, smem, as_stream(stream)>>>(                                     \
      (const TT*)x, dt_raw, dt_bias, (const TT*)bc, ld_bc, b_off, (const TT*)z, ld_z, a_log, d, state, slot_stride, \
      seq_desc, inner, N, (TT*)out)
#define SCAN_BY_N(TT)                      \
  do {                                     \
    if (!split) {                          \
      if (N <= 16) SCAN(TT, 16, 1);        \
      else if (N <= 32) SCAN(TT, 32, 1);   \
      else SCAN(TT, 64, 1);                \
    } else if (N <= 16) SCAN(TT, 16, 4);   \
    else if (N <= 32) SCAN(TT, 32, 4);     \
    else if (N <= 64) SCAN(TT, 64, 4);     \
    else if (N <= 128) SCAN(TT, 128, 4);   \
    else SCAN(TT, 256, 4);                 \
  } while (0)
  if (dtype == B200Q_DTYPE_F32) SCAN_BY_N(float);
  else SCAN_BY_N(bf16);
#undef SCAN_BY_N
#undef SCAN
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_scatter_scaled_rows(const void* src, const int32_t* pair_pos, const float* wts, int top, void* dst, int T_,
                              int W, int dtype, void* stream) {
  B200Q_CHECK_ARG(src && pair_pos && wts && dst && top > 0 && T_ >= 0 && W > 0 && is_dtype(dtype),
                  "scatter_scaled_rows: bad argument");
  if (T_ == 0) return B200Q_OK;
  const long long pairs = (long long)T_ * top;
  if (dtype == B200Q_DTYPE_BF16 && W % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    scatter_scaled_rows_v8_kernel<<<grid_for(pairs * (W / 8)), 256, 0, as_stream(stream)>>>(
        (const bf16*)src, pair_pos, wts, top, (bf16*)dst, pairs, W);
    B200Q_LAUNCH_CHECK();
    return B200Q_OK;
  }
  DISPATCH_T(dtype, (scatter_scaled_rows_kernel<T><<<grid_for(pairs * W), 256, 0, as_stream(stream)>>>(
                        (const T*)src, pair_pos, wts, top, (T*)dst, pairs, W)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_silu_glu(const void* gate_up, void* y, int64_t rows, int F, int dtype, void* stream) {
  B200Q_CHECK_ARG(gate_up && y && rows >= 0 && F > 0 && is_dtype(dtype), "silu_glu: bad argument");
  if (rows == 0) return B200Q_OK;
  if (dtype == B200Q_DTYPE_BF16 && F % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    silu_glu_v8_kernel<<<grid_for(rows * (F / 8)), 256, 0, as_stream(stream)>>>((const bf16*)gate_up, (bf16*)y, rows, F);
    B200Q_LAUNCH_CHECK();
    return B200Q_OK;
  }
  DISPATCH_T(dtype, (silu_glu_kernel<T><<<grid_for(rows * F), 256, 0, as_stream(stream)>>>((const T*)gate_up, (T*)y,
                                                                                         rows, F)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"
