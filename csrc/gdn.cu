// Gated DeltaNet: token-parallel prep + per-head recurrent scan.
//
// Input is the fused projection row [q nk*dk ; k nk*dk ; v nv*dv ; z nv*dv ; a nv ; b nv]
// (bf16).  D = dk = dv in {64, 128}.
//
//   gdn_prep  (grid = tokens x heads): depthwise causal conv (taps read from this tick's rows
//             or, before the tick's first token, from the per-slot ring of raw rows
//             indexed by position % 16) + SiLU, L2-norm of q (with 1/sqrt(dk)) and k,
//             g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b).
//   gdn_recur (grid = (value head, sequence)): the decay-first delta rule
//                 S <- e^g S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q
//             with S[dk, dv] held in registers (thread = (column, k-quarter)), one
//             block-level reduction per token, raw o to an fp32 scratch; then a
//             token-parallel epilogue: RMSNorm over dv, * weight, * silu(z) -> bf16.
//             Also refreshes the ring with the tick's last raw rows, and in "keep"
//             mode stores the state after each token in planes 0..T-1 (speculative
//             verify); otherwise the final state goes back to the live plane.
//
// State pool: [slots, layers, planes, nv, D, D] fp32; cur[slot] = live plane.
// Reference parity: kernels_gdn.py:21-126 (prep), :539-744 (fused decode), :746-939
// (serial-scan prefill) of packages/tilerl-kernels/src/tilerl_kernels; maths
// reference.py:1142-1277.
#include <stdlib.h>

#include "common.cuh"

namespace {

constexpr int RING = 16;

// grid = (tokens, 2*nk + nv): one CTA of D threads per (token, head); q/k heads also
// L2-normalise, the first CTA of a token also emits the gates.
__global__ void __launch_bounds__(128)
gdn_prep_kernel(const bf16* inp, int ld, const float* __restrict__ conv_w,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                const bf16* ring, const int* positions,
                const int* seq_ids, const int* q_start,
                const int* state_slots, long ring_slot_stride,
                float* qn, float* kn, float* vc,
                float* gout, float* bout, int nk, int nv, int D, int KW) {
  __shared__ float red[32];
  pdl_launch_dependents(12);
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  const int C = 2 * nk * D + nv * D;
  const int pos = positions[t];
  const int seq = seq_ids[t];
  const int t0 = q_start[seq];
  const bf16* rg = ring + (size_t)state_slots[seq] * ring_slot_stride;
  const int d = threadIdx.x;
  const int c = head * D + d;
  float acc = 0.f;
  for (int j = 0; j < KW; ++j) {  // tap KW-1 multiplies the newest row
    const int back = KW - 1 - j;
    const int pj = pos - back;
    float v = 0.f;
    if (pj >= 0) {
      if (t - back >= t0)
        v = __bfloat162float(inp[(size_t)(t - back) * ld + c]);
      else
        v = __bfloat162float(rg[(size_t)(pj % RING) * C + c]);
    }
    acc = fmaf(v, conv_w[(size_t)c * KW + j], acc);
  }
  const float val = silu_f(acc);
  if (head < 2 * nk) {
    const float ss = block_sum(val * val, red);
    const float nrm = rsqrtf(ss + 1e-12f) * (head < nk ? rsqrtf((float)D) : 1.f);
    if (head < nk)
      qn[((size_t)t * nk + head) * D + d] = val * nrm;
    else
      kn[((size_t)t * nk + (head - nk)) * D + d] = val * nrm;
  } else {
    vc[((size_t)t * nv + (head - 2 * nk)) * D + d] = val;
  }
  if (head == 0) {
    const bf16* ab = inp + (size_t)t * ld + C + nv * D;
    for (int h = threadIdx.x; h < nv; h += blockDim.x) {
      const float a = __bfloat162float(ab[h]), b = __bfloat162float(ab[nv + h]);
      gout[(size_t)t * nv + h] = -__expf(a_log[h]) * softplus_f(a + dt_bias[h]);
      bout[(size_t)t * nv + h] = sigmoid_f(b);
    }
  }
}

// Thread (col, kq): col = tid % D, kq = tid / D in 0..3 owns S[kq*D/4 .. +D/4][col].
template <int D>
__global__ void __launch_bounds__(D * 4)
gdn_recur_kernel(const float* qn, const float* kn,
                 const float* vc, const float* gin,
                 const float* bin, const bf16* inp, int ld,
                 float* states, int* cur, bf16* ring,
                 const int* q_start, const int* q_len,
                 const int* positions, const int* state_slots,
                 const int* keep_flags, long state_slot_stride, long plane_stride,
                 long ring_slot_stride, const float* __restrict__ norm_w, float eps,
                 float* o_scratch, bf16* out, int nk, int nv, int planes) {
  constexpr int KQ = D / 4;
  __shared__ float s_q[2][D], s_k[2][D];
  __shared__ float s_part[4][2][D];
  __shared__ float s_sc[2][4];  // v unused; [buf][g, beta, qk]
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int col = threadIdx.x % D, kq = threadIdx.x / D;
  const int T = q_len[seq], t0 = q_start[seq];
  if (T == 0) return;
  const int slot = state_slots[seq];
  const int keep = keep_flags ? keep_flags[seq] : 0;
  const int kh = h * nk / nv;
  const int live = cur[slot];
  float* sbase = states + (size_t)slot * state_slot_stride + (size_t)h * D * D;
  const float* sin_ = sbase + (size_t)live * plane_stride;
  float S[KQ];
#pragma unroll
  for (int i = 0; i < KQ; ++i) S[i] = sin_[(size_t)(kq * KQ + i) * D + col];

  // prefetch token 0
  auto load_tok = [&](int i, int b) {
    const int t = t0 + i;
    if (threadIdx.x < D) s_q[b][threadIdx.x] = qn[((size_t)t * nk + kh) * D + threadIdx.x];
    else if (threadIdx.x < 2 * D) s_k[b][threadIdx.x - D] = kn[((size_t)t * nk + kh) * D + threadIdx.x - D];
  };
  load_tok(0, 0);
  __syncthreads();
  for (int i = 0; i < T; ++i) {
    const int b = i & 1;
    const int t = t0 + i;
    if (i + 1 < T) load_tok(i + 1, b ^ 1);
    const float g = gin[(size_t)t * nv + h], beta = bin[(size_t)t * nv + h];
    const float v = vc[((size_t)t * nv + h) * D + col];
    const float eg = __expf(g);
    float ks = 0.f, qs = 0.f, qk = 0.f;
#pragma unroll
    for (int j = 0; j < KQ; ++j) {
      const float kk = s_k[b][kq * KQ + j], qq = s_q[b][kq * KQ + j];
      ks = fmaf(kk, S[j], ks);
      qs = fmaf(qq, S[j], qs);
      qk = fmaf(qq, kk, qk);
    }
    s_part[kq][0][col] = ks;
    s_part[kq][1][col] = qs;
    if (col == 0) s_sc[b][kq] = qk;
    __syncthreads();
    const float ksum = s_part[0][0][col] + s_part[1][0][col] + s_part[2][0][col] + s_part[3][0][col];
    const float qsum = s_part[0][1][col] + s_part[1][1][col] + s_part[2][1][col] + s_part[3][1][col];
    const float qkd = s_sc[b][0] + s_sc[b][1] + s_sc[b][2] + s_sc[b][3];
    const float d = beta * (v - eg * ksum);
#pragma unroll
    for (int j = 0; j < KQ; ++j) S[j] = fmaf(s_k[b][kq * KQ + j], d, eg * S[j]);
    if (kq == 0) o_scratch[((size_t)t * nv + h) * D + col] = fmaf(eg, qsum, qkd * d);
    if (keep && i < planes) {
      float* sp = sbase + (size_t)i * plane_stride;
#pragma unroll
      for (int j = 0; j < KQ; ++j) sp[(size_t)(kq * KQ + j) * D + col] = S[j];
    }
    __syncthreads();  // s_part / next token buffers
  }
  if (!keep) {
    float* sp = sbase + (size_t)live * plane_stride;
#pragma unroll
    for (int j = 0; j < KQ; ++j) sp[(size_t)(kq * KQ + j) * D + col] = S[j];
  }
  // ring refresh: raw q/k rows by the first value head of each key head, v rows by
  // every head, for the last min(T, RING) tokens of the tick
  {
    bf16* rg = ring + (size_t)slot * ring_slot_stride;
    const int C = 2 * nk * D + nv * D;
    const int first = max(0, T - RING);
    const int rep = nv / nk;
    for (int i = first; i < T; ++i) {
      const int t = t0 + i;
      const int rrow = positions[t] % RING;
      const bf16* src = inp + (size_t)t * ld;
      bf16* dst = rg + (size_t)rrow * C;
      if (h % rep == 0) {
        for (int c = threadIdx.x; c < 2 * D; c += blockDim.x) {
          const int cc = (c < D) ? kh * D + c : nk * D + kh * D + (c - D);
          dst[cc] = src[cc];
        }
      }
      for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const int cc = 2 * nk * D + h * D + c;
        dst[cc] = src[cc];
      }
    }
  }
  __syncthreads();
  __threadfence_block();
  // epilogue: gated RMSNorm per token, one warp per token
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int C = 2 * nk * D + nv * D;
  for (int i = warp; i < T; i += nw) {
    const int t = t0 + i;
    const float* o = o_scratch + ((size_t)t * nv + h) * D;
    float ov[D / 32], ss = 0.f;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      ov[j] = o[lane + 32 * j];
      ss += ov[j] * ov[j];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
    const bf16* z = inp + (size_t)t * ld + C + (size_t)h * D;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      const int c = lane + 32 * j;
      out[((size_t)t * nv + h) * D + c] =
          __float2bfloat16(ov[j] * rstd * norm_w[c] * silu_f(__bfloat162float(z[c])));
    }
  }
}


// ---------------------------------------------------------------------------------------
// Column-sliced scan.  The delta rule never mixes state columns, so one (sequence, value
// head) is cut into D/32 CTAs of 32 columns each; a warp owns 4 columns and its lanes split
// the dk rows in eight groups (lane = group * 4 + column), so a step needs two 3-level
// shuffles and no block barrier; eight warps per CTA keep every scheduler busy while each
// warp waits on its own dependent FMA chain.  q / k / v / gates of 16 tokens at a time are staged in
// shared memory with cp.async one chunk ahead, so no step waits on global memory.  The raw
// outputs of a chunk go out coalesced; the last CTA of a head to finish (device counter)
// runs the gated RMSNorm over the whole head.
constexpr int SCAN_TC = 16;
constexpr int GDN_DONE_CAP = 16384;
__device__ int g_gdn_done[GDN_DONE_CAP];   // [seq * nv + head] arrival counters, self-resetting

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D>
__global__ void __launch_bounds__(256)
gdn_scan_kernel(const float* qn, const float* kn,
                const float* vc, const float* gin,
                const float* bin, const bf16* inp, int ld,
                float* states, int* cur, bf16* ring,
                const int* q_start, const int* q_len,
                const int* positions, const int* state_slots,
                const int* keep_flags, long state_slot_stride, long plane_stride,
                long ring_slot_stride, const float* __restrict__ norm_w, float eps,
                float* o_scratch, bf16* out, int nk, int nv, int planes) {
  constexpr int Q = 8;            // row groups (lanes that share a column)
  constexpr int R = D / Q;        // state rows per thread
  constexpr int NS = D / 32;      // column slices (CTAs) per head
  constexpr int KP = R + 4;       // padded group stride: the eight groups hit different banks
  constexpr int NT = 256, NW = NT / 32, CW = 32 / Q;   // threads, warps, columns per warp
  constexpr int TC = SCAN_TC;
  __shared__ __align__(16) float s_q[2][TC][Q * KP];
  __shared__ __align__(16) float s_k[2][TC][Q * KP];
  __shared__ __align__(16) float s_v[2][TC][32];
  __shared__ float s_g[2][TC], s_b[2][TC], s_qk[2][TC];
  __shared__ __align__(16) float s_o[TC][32];
  __shared__ int s_last;
  pdl_launch_dependents(2);
  pdl_wait();
  const int h = blockIdx.x / NS, slice = blockIdx.x % NS, seq = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = lane / CW, cl = warp * CW + (lane % CW), col = slice * 32 + cl;
  const int T = q_len[seq], t0 = q_start[seq];
  if (T == 0) return;
  const int slot = state_slots[seq];
  const int keep = keep_flags ? keep_flags[seq] : 0;
  const int kh = h * nk / nv;
  const int live = cur[slot];
  float* sbase = states + (size_t)slot * state_slot_stride + (size_t)h * D * D;
  const float* sin_ = sbase + (size_t)live * plane_stride;
  float S[R];
#pragma unroll
  for (int j = 0; j < R; ++j) S[j] = sin_[(size_t)(r * R + j) * D + col];

  auto stage = [&](int i0, int b) {
    const int n = min(TC, T - i0);
    // q and k rows: D/4 pieces of 16 B per token each; v: 8 pieces; gates: scalars
    for (int x = tid; x < n * (D / 4); x += NT) {
      const int tt = x / (D / 4), pc = x % (D / 4);
      const int e = pc * 4, dst = (e / R) * KP + (e % R);
      const size_t src = ((size_t)(t0 + i0 + tt) * nk + kh) * D + e;
      cp_async16(&s_q[b][tt][dst], qn + src);
      cp_async16(&s_k[b][tt][dst], kn + src);
    }
    for (int x = tid; x < n * 8; x += NT) {
      const int tt = x >> 3, pc = x & 7;
      cp_async16(&s_v[b][tt][pc * 4], vc + ((size_t)(t0 + i0 + tt) * nv + h) * D + slice * 32 + pc * 4);
    }
    if (tid < n) {
      s_g[b][tid] = gin[(size_t)(t0 + i0 + tid) * nv + h];
      s_b[b][tid] = bin[(size_t)(t0 + i0 + tid) * nv + h];
    }
    cp_async_commit();
  };

  stage(0, 0);
  int b = 0;
  for (int i0 = 0; i0 < T; i0 += TC, b ^= 1) {
    const int n = min(TC, T - i0);
    cp_async_wait<0>();
    __syncthreads();                       // chunk b landed; every thread left the previous chunk
    if (i0 > 0) {                          // raw outputs of the previous chunk, 128 B rows
      const int pn = TC;
      for (int x = tid; x < pn * 32; x += NT)
        o_scratch[((size_t)(t0 + i0 - TC + (x >> 5)) * nv + h) * D + slice * 32 + (x & 31)] = s_o[x >> 5][x & 31];
    }
    if (i0 + TC < T) stage(i0 + TC, b ^ 1);
    for (int tt = warp; tt < n; tt += NW) { // q.k of this chunk's tokens
      float a = 0.f;
      for (int e = lane; e < D; e += 32) {
        const int o = (e / R) * KP + (e % R);
        a = fmaf(s_q[b][tt][o], s_k[b][tt][o], a);
      }
      a = warp_sum(a);
      if (lane == 0) s_qk[b][tt] = a;
    }
    __syncthreads();                       // s_qk visible, s_o flushed
    for (int tt = 0; tt < n; ++tt) {
      const float eg = __expf(s_g[b][tt]), beta = s_b[b][tt], v = s_v[b][tt][cl], qk = s_qk[b][tt];
      const float4* k4 = reinterpret_cast<const float4*>(&s_k[b][tt][r * KP]);
      const float4* q4 = reinterpret_cast<const float4*>(&s_q[b][tt][r * KP]);
      float kreg[R];
      float ks0 = 0.f, ks1 = 0.f, qs0 = 0.f, qs1 = 0.f;
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const float4 kk = k4[j], qq = q4[j];
        kreg[4 * j] = kk.x, kreg[4 * j + 1] = kk.y, kreg[4 * j + 2] = kk.z, kreg[4 * j + 3] = kk.w;
        ks0 = fmaf(kk.x, S[4 * j], ks0), ks1 = fmaf(kk.y, S[4 * j + 1], ks1);
        ks0 = fmaf(kk.z, S[4 * j + 2], ks0), ks1 = fmaf(kk.w, S[4 * j + 3], ks1);
        qs0 = fmaf(qq.x, S[4 * j], qs0), qs1 = fmaf(qq.y, S[4 * j + 1], qs1);
        qs0 = fmaf(qq.z, S[4 * j + 2], qs0), qs1 = fmaf(qq.w, S[4 * j + 3], qs1);
      }
      float ks = ks0 + ks1, qs = qs0 + qs1;
#pragma unroll
      for (int m = CW; m < 32; m <<= 1) {
        ks += __shfl_xor_sync(0xffffffffu, ks, m);
        qs += __shfl_xor_sync(0xffffffffu, qs, m);
      }
      const float d = beta * (v - eg * ks);
#pragma unroll
      for (int j = 0; j < R; ++j) S[j] = fmaf(kreg[j], d, eg * S[j]);
      if (r == 0) s_o[tt][cl] = fmaf(eg, qs, qk * d);
      if (keep && i0 + tt < planes) {
        float* sp = sbase + (size_t)(i0 + tt) * plane_stride;
#pragma unroll
        for (int j = 0; j < R; ++j) sp[(size_t)(r * R + j) * D + col] = S[j];
      }
    }
  }
  __syncthreads();
  {                                        // raw outputs of the last chunk
    const int i0 = ((T - 1) / TC) * TC, n = T - i0;
    for (int x = tid; x < n * 32; x += NT)
      o_scratch[((size_t)(t0 + i0 + (x >> 5)) * nv + h) * D + slice * 32 + (x & 31)] = s_o[x >> 5][x & 31];
  }
  if (!keep) {
    float* sp = sbase + (size_t)live * plane_stride;
#pragma unroll
    for (int j = 0; j < R; ++j) sp[(size_t)(r * R + j) * D + col] = S[j];
  }
  const int C = 2 * nk * D + nv * D;
  if (slice == 0) {
    // ring refresh: raw q/k rows by the first value head of each key head, v rows by every
    // head, for the last min(T, RING) tokens of the tick
    bf16* rg = ring + (size_t)slot * ring_slot_stride;
    const int first = max(0, T - RING);
    const int rep = nv / nk;
    for (int i = first; i < T; ++i) {
      const int t = t0 + i;
      const int rrow = positions[t] % RING;
      const bf16* src = inp + (size_t)t * ld;
      bf16* dst = rg + (size_t)rrow * C;
      if (h % rep == 0) {
        for (int c = tid; c < 2 * D; c += NT) {
          const int cc = (c < D) ? kh * D + c : nk * D + kh * D + (c - D);
          dst[cc] = src[cc];
        }
      }
      for (int c = tid; c < D; c += NT) {
        const int cc = 2 * nk * D + h * D + c;
        dst[cc] = src[cc];
      }
    }
  }
  // the last slice of this head to get here normalises the head
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* ctr = g_gdn_done + (size_t)seq * nv + h;
    const int prev = atomicAdd(ctr, 1);
    s_last = (prev == NS - 1);
    if (prev == NS - 1) *ctr = 0;
  }
  __syncthreads();
  trl_trace_end();
  if (!s_last) return;
  __threadfence();
  for (int i = warp; i < T; i += NW) {     // gated RMSNorm per token, one warp per token
    const int t = t0 + i;
    const float* o = o_scratch + ((size_t)t * nv + h) * D;
    float ov[D / 32], ss = 0.f;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      ov[j] = __ldcg(o + lane + 32 * j);
      ss += ov[j] * ov[j];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
    const bf16* z = inp + (size_t)t * ld + C + (size_t)h * D;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      const int c = lane + 32 * j;
      out[((size_t)t * nv + h) * D + c] =
          __float2bfloat16(ov[j] * rstd * norm_w[c] * silu_f(__bfloat162float(z[c])));
    }
  }
}


// ---------------------------------------------------------------------------------------
// Chunk-parallel scan for prefill: the same column slicing and thread mapping as the scan
// above, but the 16 tokens of a chunk are not walked one after the other.  With the chunk's
// cumulative log-decay G_i, the chunk-start state S0 and, per state column,
//   p_i = k_i . S0,  r_i = q_i . S0                        (all tokens at once, no chain)
//   M_ij = beta_i e^{G_i-G_j} (k_i . k_j)  (j < i),   N_ij = e^{G_i-G_j} (q_i . k_j)  (j <= i)
// the delta rule unrolls to
//   d_i = beta_i (v_i - e^{G_i} p_i) - sum_{j<i} M_ij d_j     (16 x 16 forward substitution)
//   o_i = e^{G_i} r_i + sum_{j<=i} N_ij d_j
//   S   = e^{G_15} S0 + sum_i e^{G_15-G_i} k_i (x) d_i
// so a token no longer waits for the state update of the one before it: the only serial part
// is the small triangular solve.  M and N do not depend on the column and are built once per
// chunk by the CTA.  Tokens past the end of a sequence enter as beta = 0, g = 0, zero rows.
// Chunks of fewer than WY_MIN tokens run the serial step (identical to gdn_scan_kernel), so a
// prompt gives the same bits whether it is prefilled in one tick or in 16-aligned pieces.
// Parity: the chunkwise pipeline of tilerl_kernels/kernels_gdn.py:127-745 (cumsum, kkt,
// solve_tril, wu, state scan, chunk_o), here in one kernel per layer.
constexpr int WY_MIN = 4;
template <int D>
struct alignas(16) WySmem {
  static constexpr int Q = 8, R = D / Q, KP = R + 4, RS = Q * KP + 4, TC = SCAN_TC;
  float q[2][TC][RS];
  float k[2][TC][RS];
  float v[2][TC][32];
  float g[2][TC];
  float b[2][TC];
  float o[TC][32];
  float M[TC][TC];
  float N[TC][TC];
  float eG[TC];
  float w[TC];
  float Gc[TC];
  float qk[TC];
  int last;
};

template <int D>
__global__ void __launch_bounds__(256)
gdn_scan_wy_kernel(const float* qn, const float* kn,
                   const float* vc, const float* gin,
                   const float* bin, const bf16* inp, int ld,
                   float* states, int* cur, bf16* ring,
                   const int* q_start, const int* q_len,
                   const int* positions, const int* state_slots,
                   long state_slot_stride, long plane_stride, long ring_slot_stride,
                   const float* __restrict__ norm_w, float eps, float* o_scratch,
                   bf16* out, int nk, int nv) {
  using SM = WySmem<D>;
  constexpr int Q = SM::Q, R = SM::R, KP = SM::KP, TC = SM::TC;
  constexpr int NS = D / 32, NT = 256, NW = NT / 32, CW = 32 / Q;
  extern __shared__ __align__(16) unsigned char wy_raw[];
  SM& sm = *reinterpret_cast<SM*>(wy_raw);
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.x / NS, slice = blockIdx.x % NS, seq = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = lane / CW, cl = warp * CW + (lane % CW), col = slice * 32 + cl;
  const int T = q_len[seq], t0 = q_start[seq];
  if (T == 0) return;
  const int slot = state_slots[seq];
  const int kh = h * nk / nv;
  const int live = cur[slot];
  float* sbase = states + (size_t)slot * state_slot_stride + (size_t)h * D * D;
  float* splane = sbase + (size_t)live * plane_stride;
  float S[R];
#pragma unroll
  for (int j = 0; j < R; ++j) S[j] = splane[(size_t)(r * R + j) * D + col];

  auto stage = [&](int i0, int b) {
    const int n = min(TC, T - i0);
    for (int x = tid; x < TC * (D / 4); x += NT) {
      const int tt = x / (D / 4), pc = x % (D / 4);
      const int e = pc * 4, dst = (e / R) * KP + (e % R);
      if (tt < n) {
        const size_t src = ((size_t)(t0 + i0 + tt) * nk + kh) * D + e;
        cp_async16(&sm.q[b][tt][dst], qn + src);
        cp_async16(&sm.k[b][tt][dst], kn + src);
      } else {   // rows past the end: zeros, so they drop out of every product
        *reinterpret_cast<float4*>(&sm.q[b][tt][dst]) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(&sm.k[b][tt][dst]) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    for (int x = tid; x < TC * 8; x += NT) {
      const int tt = x >> 3, pc = x & 7;
      if (tt < n) cp_async16(&sm.v[b][tt][pc * 4], vc + ((size_t)(t0 + i0 + tt) * nv + h) * D + slice * 32 + pc * 4);
      else *reinterpret_cast<float4*>(&sm.v[b][tt][pc * 4]) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (tid < TC) {
      sm.g[b][tid] = tid < n ? gin[(size_t)(t0 + i0 + tid) * nv + h] : 0.f;
      sm.b[b][tid] = tid < n ? bin[(size_t)(t0 + i0 + tid) * nv + h] : 0.f;
    }
    cp_async_commit();
  };

  stage(0, 0);
  int b = 0;
  for (int i0 = 0; i0 < T; i0 += TC, b ^= 1) {
    const int n = min(TC, T - i0);
    const bool wy = n >= WY_MIN;
    cp_async_wait<0>();
    __syncthreads();                       // chunk b landed; every thread left the previous chunk
    if (i0 > 0) {                          // raw outputs of the previous chunk, 128 B rows
      for (int x = tid; x < TC * 32; x += NT)
        o_scratch[((size_t)(t0 + i0 - TC + (x >> 5)) * nv + h) * D + slice * 32 + (x & 31)] = sm.o[x >> 5][x & 31];
    }
    if (i0 + TC < T) stage(i0 + TC, b ^ 1);
    if (wy) {
      if (warp == 0) {                     // cumulative log-decay of the chunk and its exponentials
        float gc = lane < TC ? sm.g[b][lane] : 0.f;
#pragma unroll
        for (int o = 1; o < TC; o <<= 1) {
          const float nb = __shfl_up_sync(0xffffffffu, gc, o);
          if (lane >= o) gc += nb;
        }
        const float glast = __shfl_sync(0xffffffffu, gc, TC - 1);
        if (lane < TC) {
          sm.Gc[lane] = gc;
          sm.eG[lane] = __expf(gc);
          sm.w[lane] = __expf(glast - gc);
        }
      }
      __syncthreads();
      {                                    // M and N: one (i, j) pair per thread, j <= i
        const int i = tid >> 4, j = tid & 15;
        float mv = 0.f, nv_ = 0.f;
        if (j <= i) {
          float kk = 0.f, qk = 0.f;
#pragma unroll
          for (int grp = 0; grp < Q; ++grp) {
            const float4* ki = reinterpret_cast<const float4*>(&sm.k[b][i][grp * KP]);
            const float4* kj = reinterpret_cast<const float4*>(&sm.k[b][j][grp * KP]);
            const float4* qi = reinterpret_cast<const float4*>(&sm.q[b][i][grp * KP]);
#pragma unroll
            for (int f = 0; f < R / 4; ++f) {
              const float4 a = ki[f], c = kj[f], e = qi[f];
              kk = fmaf(a.x, c.x, kk), kk = fmaf(a.y, c.y, kk), kk = fmaf(a.z, c.z, kk), kk = fmaf(a.w, c.w, kk);
              qk = fmaf(e.x, c.x, qk), qk = fmaf(e.y, c.y, qk), qk = fmaf(e.z, c.z, qk), qk = fmaf(e.w, c.w, qk);
            }
          }
          const float dec = __expf(sm.Gc[i] - sm.Gc[j]);
          mv = j < i ? sm.b[b][i] * dec * kk : 0.f;
          nv_ = dec * qk;
        }
        sm.M[i][j] = mv;
        sm.N[i][j] = nv_;
      }
      __syncthreads();                     // M, N visible; s_o flushed
      float ks[TC], qs[TC];
#pragma unroll
      for (int tt = 0; tt < TC; ++tt) {    // p and r of every token against the chunk-start state
        const float4* k4 = reinterpret_cast<const float4*>(&sm.k[b][tt][r * KP]);
        const float4* q4 = reinterpret_cast<const float4*>(&sm.q[b][tt][r * KP]);
        float a0 = 0.f, a1 = 0.f, c0 = 0.f, c1 = 0.f;
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          const float4 kk = k4[j], qq = q4[j];
          a0 = fmaf(kk.x, S[4 * j], a0), a1 = fmaf(kk.y, S[4 * j + 1], a1);
          a0 = fmaf(kk.z, S[4 * j + 2], a0), a1 = fmaf(kk.w, S[4 * j + 3], a1);
          c0 = fmaf(qq.x, S[4 * j], c0), c1 = fmaf(qq.y, S[4 * j + 1], c1);
          c0 = fmaf(qq.z, S[4 * j + 2], c0), c1 = fmaf(qq.w, S[4 * j + 3], c1);
        }
        ks[tt] = a0 + a1, qs[tt] = c0 + c1;
      }
#pragma unroll
      for (int m = CW; m < 32; m <<= 1) {
#pragma unroll
        for (int tt = 0; tt < TC; ++tt) {
          ks[tt] += __shfl_xor_sync(0xffffffffu, ks[tt], m);
          qs[tt] += __shfl_xor_sync(0xffffffffu, qs[tt], m);
        }
      }
      float d[TC];
#pragma unroll
      for (int i = 0; i < TC; ++i) {       // forward substitution, the only chain of the chunk
        float acc = sm.b[b][i] * (sm.v[b][i][cl] - sm.eG[i] * ks[i]);
#pragma unroll
        for (int j = 0; j < i; ++j) acc = fmaf(-sm.M[i][j], d[j], acc);
        d[i] = acc;
      }
#pragma unroll
      for (int i = 0; i < TC; ++i) {       // outputs: row group r writes tokens r and r + 8
        if ((i & (Q - 1)) == r) {
          float acc = sm.eG[i] * qs[i];
#pragma unroll
          for (int j = 0; j <= i; ++j) acc = fmaf(sm.N[i][j], d[j], acc);
          sm.o[i][cl] = acc;
        }
      }
      const float glast = sm.eG[TC - 1];
#pragma unroll
      for (int j = 0; j < R; ++j) S[j] *= glast;
#pragma unroll
      for (int tt = 0; tt < TC; ++tt) {    // state update: all tokens' rank-1 terms at once
        const float c = sm.w[tt] * d[tt];
        const float4* k4 = reinterpret_cast<const float4*>(&sm.k[b][tt][r * KP]);
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          const float4 kk = k4[j];
          S[4 * j] = fmaf(kk.x, c, S[4 * j]), S[4 * j + 1] = fmaf(kk.y, c, S[4 * j + 1]);
          S[4 * j + 2] = fmaf(kk.z, c, S[4 * j + 2]), S[4 * j + 3] = fmaf(kk.w, c, S[4 * j + 3]);
        }
      }
    } else {
      for (int tt = warp; tt < n; tt += NW) {   // q.k of this chunk's tokens
        float a = 0.f;
        for (int e = lane; e < D; e += 32) {
          const int o = (e / R) * KP + (e % R);
          a = fmaf(sm.q[b][tt][o], sm.k[b][tt][o], a);
        }
        a = warp_sum(a);
        if (lane == 0) sm.qk[tt] = a;
      }
      __syncthreads();                     // q.k visible, s_o flushed
      for (int tt = 0; tt < n; ++tt) {     // the serial step of gdn_scan_kernel, operation for operation
        const float eg = __expf(sm.g[b][tt]), beta = sm.b[b][tt], v = sm.v[b][tt][cl], qk = sm.qk[tt];
        const float4* k4 = reinterpret_cast<const float4*>(&sm.k[b][tt][r * KP]);
        const float4* q4 = reinterpret_cast<const float4*>(&sm.q[b][tt][r * KP]);
        float kreg[R];
        float ks0 = 0.f, ks1 = 0.f, qs0 = 0.f, qs1 = 0.f;
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          const float4 kk = k4[j], qq = q4[j];
          kreg[4 * j] = kk.x, kreg[4 * j + 1] = kk.y, kreg[4 * j + 2] = kk.z, kreg[4 * j + 3] = kk.w;
          ks0 = fmaf(kk.x, S[4 * j], ks0), ks1 = fmaf(kk.y, S[4 * j + 1], ks1);
          ks0 = fmaf(kk.z, S[4 * j + 2], ks0), ks1 = fmaf(kk.w, S[4 * j + 3], ks1);
          qs0 = fmaf(qq.x, S[4 * j], qs0), qs1 = fmaf(qq.y, S[4 * j + 1], qs1);
          qs0 = fmaf(qq.z, S[4 * j + 2], qs0), qs1 = fmaf(qq.w, S[4 * j + 3], qs1);
        }
        float ks = ks0 + ks1, qs = qs0 + qs1;
#pragma unroll
        for (int m = CW; m < 32; m <<= 1) {
          ks += __shfl_xor_sync(0xffffffffu, ks, m);
          qs += __shfl_xor_sync(0xffffffffu, qs, m);
        }
        const float dd = beta * (v - eg * ks);
#pragma unroll
        for (int j = 0; j < R; ++j) S[j] = fmaf(kreg[j], dd, eg * S[j]);
        if (r == 0) sm.o[tt][cl] = fmaf(eg, qs, qk * dd);
      }
    }
  }
  __syncthreads();
  {                                        // raw outputs of the last chunk
    const int i0 = ((T - 1) / TC) * TC, n = T - i0;
    for (int x = tid; x < n * 32; x += NT)
      o_scratch[((size_t)(t0 + i0 + (x >> 5)) * nv + h) * D + slice * 32 + (x & 31)] = sm.o[x >> 5][x & 31];
  }
#pragma unroll
  for (int j = 0; j < R; ++j) splane[(size_t)(r * R + j) * D + col] = S[j];
  const int C = 2 * nk * D + nv * D;
  if (slice == 0) {
    // ring refresh: raw q/k rows by the first value head of each key head, v rows by every
    // head, for the last min(T, RING) tokens of the tick
    bf16* rg = ring + (size_t)slot * ring_slot_stride;
    const int first = max(0, T - RING);
    const int rep = nv / nk;
    for (int i = first; i < T; ++i) {
      const int t = t0 + i;
      const int rrow = positions[t] % RING;
      const bf16* src = inp + (size_t)t * ld;
      bf16* dst = rg + (size_t)rrow * C;
      if (h % rep == 0) {
        for (int c = tid; c < 2 * D; c += NT) {
          const int cc = (c < D) ? kh * D + c : nk * D + kh * D + (c - D);
          dst[cc] = src[cc];
        }
      }
      for (int c = tid; c < D; c += NT) {
        const int cc = 2 * nk * D + h * D + c;
        dst[cc] = src[cc];
      }
    }
  }
  // the last slice of this head to get here normalises the head
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* ctr = g_gdn_done + (size_t)seq * nv + h;
    const int prev = atomicAdd(ctr, 1);
    sm.last = (prev == NS - 1);
    if (prev == NS - 1) *ctr = 0;
  }
  __syncthreads();
  if (!sm.last) return;
  __threadfence();
  for (int i = warp; i < T; i += NW) {     // gated RMSNorm per token, one warp per token
    const int t = t0 + i;
    const float* o = o_scratch + ((size_t)t * nv + h) * D;
    float ov[D / 32], ss = 0.f;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      ov[j] = __ldcg(o + lane + 32 * j);
      ss += ov[j] * ov[j];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
    const bf16* z = inp + (size_t)t * ld + C + (size_t)h * D;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      const int c = lane + 32 * j;
      out[((size_t)t * nv + h) * D + c] =
          __float2bfloat16(ov[j] * rstd * norm_w[c] * silu_f(__bfloat162float(z[c])));
    }
  }
}

}  // namespace

static int g_gdn_wy = -1;   // -1: read TRL_GDN_WY at the first launch

// ---------------------------------------------------------------------------------------
// Decode tick (exactly one token per sequence, no kept planes) of a layer in ONE launch.
// One CTA of 4 * D threads owns a whole (sequence, value head): thread (col, kq) holds the D / 4
// state rows [kq * D / 4, ...) of column col, so every state load and store of a warp is one
// contiguous 128-byte row segment.
//   * before the dependency wait: the state (written by the previous tick) is loaded into
//     registers -- the slot and the live plane of a sequence are written by the host before a
//     tick and never by a kernel of a decode tick -- so the 2 x D x D x 4 bytes of the head are
//     already on their way while the in-projection GEMV still runs;
//   * after it: the prep of the token (conv + SiLU of the q / k / v channels of this head, L2
//     norms, gates) in three thread groups, the delta-rule step with one shared-memory reduction
//     over the four row groups, the gated RMSNorm of the head's output row and the ring refresh.
// No scratch buffer, no cross-CTA counter.
template <int D>
__global__ void __launch_bounds__(D * 4)
gdn_decode_kernel(const bf16* inp, int ld, const float* __restrict__ conv_w,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                  const float* __restrict__ norm_w, float* states, const int* cur, bf16* ring,
                  const int* positions, const int* q_start, const int* state_slots, long state_slot_stride,
                  long plane_stride, long ring_slot_stride, float eps, bf16* out, int nk, int nv, int KW) {
  constexpr int KQ = D / 4, WG = D / 32;      // state rows per thread, warps per thread group
  __shared__ float s_q[D], s_k[D], s_v[D];
  __shared__ float s_part[4][2][D];
  __shared__ float s_ss[3][WG], s_qk[4], s_gb[2];
  const int h = blockIdx.x, seq = blockIdx.y;
  const int tid = threadIdx.x, col = tid % D, kq = tid / D, lane = tid & 31;
  const int kh = h * nk / nv;
  const int slot = state_slots[seq];
  float* sp = states + (size_t)slot * state_slot_stride + (size_t)cur[slot] * plane_stride + (size_t)h * D * D;
  float S[KQ];
#pragma unroll
  for (int i = 0; i < KQ; ++i) S[i] = sp[(size_t)(kq * KQ + i) * D + col];
  pdl_launch_dependents(2);
  pdl_wait();
  const int t = q_start[seq], pos = positions[t];
  const int C = 2 * nk * D + nv * D;
  const bf16* row = inp + (size_t)t * ld;
  bf16* rg = ring + (size_t)slot * ring_slot_stride;
  // prep: thread group kq = 0 / 1 / 2 -> the q / k / v channel `col` of this head
  float val = 0.f;
  int ch = 0;
  if (kq < 3) {
    ch = (kq == 0 ? kh * D : kq == 1 ? nk * D + kh * D : 2 * nk * D + h * D) + col;
    float acc = 0.f;
    for (int j = 0; j < KW; ++j) {  // tap KW-1 multiplies the newest row
      const int back = KW - 1 - j, pj = pos - back;
      float v = 0.f;
      if (pj >= 0) v = __bfloat162float(back == 0 ? row[ch] : rg[(size_t)(pj % RING) * C + ch]);
      acc = fmaf(v, conv_w[(size_t)ch * KW + j], acc);
    }
    val = silu_f(acc);
    if (kq < 2) {
      const float w_ = warp_sum(val * val);
      if (lane == 0) s_ss[kq][col >> 5] = w_;
    }
  } else if (col == 0) {
    const bf16* ab = row + C + nv * D;
    s_gb[0] = -__expf(a_log[h]) * softplus_f(__bfloat162float(ab[h]) + dt_bias[h]);
    s_gb[1] = sigmoid_f(__bfloat162float(ab[nv + h]));
  }
  __syncthreads();
  if (kq < 2) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < WG; ++i) ss += s_ss[kq][i];
    const float nrm = rsqrtf(ss + 1e-12f) * (kq == 0 ? rsqrtf((float)D) : 1.f);
    (kq == 0 ? s_q : s_k)[col] = val * nrm;
  } else if (kq == 2) {
    s_v[col] = val;
  }
  __syncthreads();
  // the step: S <- e^g S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q
  const float eg = __expf(s_gb[0]), beta = s_gb[1], v = s_v[col];
  float kreg[KQ];
  float ks = 0.f, qs = 0.f, qk = 0.f;
#pragma unroll
  for (int j = 0; j < KQ; ++j) {
    const float kk = s_k[kq * KQ + j], qq = s_q[kq * KQ + j];
    kreg[j] = kk;
    ks = fmaf(kk, S[j], ks);
    qs = fmaf(qq, S[j], qs);
    qk = fmaf(qq, kk, qk);
  }
  s_part[kq][0][col] = ks;
  s_part[kq][1][col] = qs;
  if (col == 0) s_qk[kq] = qk;
  __syncthreads();
  const float ksum = (s_part[0][0][col] + s_part[1][0][col]) + (s_part[2][0][col] + s_part[3][0][col]);
  const float qsum = (s_part[0][1][col] + s_part[1][1][col]) + (s_part[2][1][col] + s_part[3][1][col]);
  const float qkd = (s_qk[0] + s_qk[1]) + (s_qk[2] + s_qk[3]);
  const float d = beta * (v - eg * ksum);
#pragma unroll
  for (int j = 0; j < KQ; ++j) sp[(size_t)(kq * KQ + j) * D + col] = fmaf(kreg[j], d, eg * S[j]);
  float o = 0.f;
  if (kq == 0) {
    o = fmaf(eg, qsum, qkd * d);
    const float w_ = warp_sum(o * o);
    if (lane == 0) s_ss[2][col >> 5] = w_;
  }
  // ring refresh: the raw q / k rows by the first value head of each key head, the v row by every head
  {
    bf16* dst = rg + (size_t)(pos % RING) * C;
    if (kq < 2 && h % (nv / nk) == 0) dst[ch] = row[ch];
    if (kq == 2) dst[ch] = row[ch];
  }
  __syncthreads();
  if (kq == 0) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < WG; ++i) ss += s_ss[2][i];
    const float rstd = rsqrtf(ss / (float)D + eps);
    const float z = __bfloat162float(row[C + (size_t)h * D + col]);
    out[((size_t)t * nv + h) * D + col] = __float2bfloat16(o * rstd * norm_w[col] * silu_f(z));
  }
  trl_trace_end();
}

// Turns the chunk-parallel prefill scan on or off at run time (tests compare the two paths).
TRL_API void trl_gdn_set_wy(int on) { g_gdn_wy = on ? 1 : 0; }

// Scratch (fp32): qn, kn [T*nk*D]; vc, o_scratch [T*nv*D]; g, beta [T*nv].
TRL_API int trl_gdn(const void* inp, int ld, const void* conv_w, const void* dt_bias, const void* a_log,
                    const void* norm_w, void* states, void* cur, void* ring, const void* positions,
                    const void* seq_ids, const void* q_start, const void* q_len,
                    const void* state_slots, const void* keep_flags, long state_slot_stride,
                    long plane_stride, long ring_slot_stride, void* qn, void* kn, void* vc, void* g,
                    void* beta, void* o_scratch, void* out, int T, int B, int nk, int nv, int D, int KW,
                    int planes, float eps, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = trl_launch(gdn_prep_kernel, dim3(T, 2 * nk + nv), dim3(D), 0, st, (const bf16*)inp, ld,
                             (const float*)conv_w, (const float*)dt_bias, (const float*)a_log,
                             (const bf16*)ring, (const int*)positions, (const int*)seq_ids,
                             (const int*)q_start, (const int*)state_slots, ring_slot_stride,
                             (float*)qn, (float*)kn, (float*)vc, (float*)g, (float*)beta, nk, nv, D, KW);
  if (e != cudaSuccess) return (int)e;
#define RECUR(DD)                                                                                   \
  e = trl_launch(gdn_recur_kernel<DD>, dim3(nv, B), dim3(DD * 4), 0, st, (const float*)qn,          \
                 (const float*)kn, (const float*)vc, (const float*)g, (const float*)beta,           \
                 (const bf16*)inp, ld, (float*)states, (int*)cur, (bf16*)ring, (const int*)q_start, \
                 (const int*)q_len, (const int*)positions, (const int*)state_slots,                 \
                 (const int*)keep_flags, state_slot_stride, plane_stride, ring_slot_stride,         \
                 (const float*)norm_w, eps, (float*)o_scratch, (bf16*)out, nk, nv, planes)
#define SCAN(DD)                                                                                    \
  e = trl_launch(gdn_scan_kernel<DD>, dim3(nv * (DD / 32), B), dim3(256), 0, st, (const float*)qn,  \
                 (const float*)kn, (const float*)vc, (const float*)g, (const float*)beta,           \
                 (const bf16*)inp, ld, (float*)states, (int*)cur, (bf16*)ring, (const int*)q_start, \
                 (const int*)q_len, (const int*)positions, (const int*)state_slots,                 \
                 (const int*)keep_flags, state_slot_stride, plane_stride, ring_slot_stride,         \
                 (const float*)norm_w, eps, (float*)o_scratch, (bf16*)out, nk, nv, planes)
#define SCANWY(DD)                                                                                  \
  {                                                                                                 \
    auto kern = gdn_scan_wy_kernel<DD>;                                                             \
    static bool configured = false;                                                                 \
    if (!configured) {                                                                              \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                   \
                               (int)sizeof(WySmem<DD>)) != cudaSuccess) return 3;                   \
      configured = true;                                                                            \
    }                                                                                               \
    e = trl_launch(kern, dim3(nv * (DD / 32), B), dim3(256), sizeof(WySmem<DD>), st,                \
                   (const float*)qn, (const float*)kn, (const float*)vc, (const float*)g,           \
                   (const float*)beta, (const bf16*)inp, ld, (float*)states, (int*)cur,             \
                   (bf16*)ring, (const int*)q_start, (const int*)q_len, (const int*)positions,      \
                   (const int*)state_slots, state_slot_stride, plane_stride, ring_slot_stride,      \
                   (const float*)norm_w, eps, (float*)o_scratch, (bf16*)out, nk, nv);               \
  }
  static const bool legacy = getenv("TRL_GDN_LEGACY") != nullptr;
  // chunk-parallel scan for ticks that carry prompt tokens (more tokens than sequences) and keep
  // no per-token states.  Off unless TRL_GDN_WY=1: with 8 row groups per column it issues more
  // instructions per token than the token-by-token scan and measured slower (577 vs 412 us per
  // 512-token layer); it needs more row groups per column to pay off.
  if (g_gdn_wy < 0) g_gdn_wy = (getenv("TRL_GDN_WY") && atoi(getenv("TRL_GDN_WY")) != 0) ? 1 : 0;
  const bool wy_on = g_gdn_wy != 0;
  const bool scan = !legacy && (long)B * nv <= GDN_DONE_CAP;
  const bool wy = scan && wy_on && T > B && keep_flags == nullptr;
  if (D == 128) { if (wy) SCANWY(128) else if (scan) SCAN(128); else RECUR(128); }
  else if (D == 64) { if (wy) SCANWY(64) else if (scan) SCAN(64); else RECUR(64); }
  else return (int)cudaErrorInvalidValue;
#undef RECUR
#undef SCAN
#undef SCANWY
  return (int)e;
}

// Decode tick of a Gated-DeltaNet layer in ONE launch: every sequence carries exactly one token
// (its row in `inp` is q_start[seq]), no per-token planes are kept.
TRL_API int trl_gdn_decode(const void* inp, int ld, const void* conv_w, const void* dt_bias, const void* a_log,
                           const void* norm_w, void* states, const void* cur, void* ring, const void* positions,
                           const void* q_start, const void* state_slots, long state_slot_stride,
                           long plane_stride, long ring_slot_stride, void* out, int B, int nk, int nv, int D,
                           int KW, float eps, void* stream) {
  if ((D != 128 && D != 64) || nk <= 0 || nv % nk != 0 || B <= 0 || B > 65535) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
#define DECODE(DD)                                                                                          \
  return (int)trl_launch(gdn_decode_kernel<DD>, dim3(nv, B), dim3(DD * 4), 0, st, (const bf16*)inp, ld,     \
                         (const float*)conv_w, (const float*)dt_bias, (const float*)a_log,                  \
                         (const float*)norm_w, (float*)states, (const int*)cur, (bf16*)ring,                \
                         (const int*)positions, (const int*)q_start, (const int*)state_slots,               \
                         state_slot_stride, plane_stride, ring_slot_stride, eps, (bf16*)out, nk, nv, KW)
  if (D == 128) DECODE(128);
  DECODE(64);
#undef DECODE
}
