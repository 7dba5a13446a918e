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

// grid = (ceil(tokens / TPC), 2*nk + nv), 128 threads: a thread owns 8 adjacent channels of one token
// (D / 8 threads per token, TPC = 1024 / D tokens per CTA): four 16-byte row loads (the conv window), depthwise
// causal conv + SiLU; q/k heads L2-normalise with shuffles inside the token's thread group; the head-0
// CTA of a tile also emits the gates.  No shared memory, no block barrier.
__global__ void __launch_bounds__(128)
gdn_prep_kernel(const bf16* inp, int ld, const float* __restrict__ conv_w,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                const bf16* ring, const int* positions,
                const int* seq_ids, const int* q_start,
                const int* state_slots, long ring_slot_stride,
                float* qn, float* kn, float* vc,
                float* gout, float* bout, int nk, int nv, int D, int KW, int T) {
  pdl_launch_dependents(12);
  pdl_wait();
  const int tpt = D >> 3;                       // threads per token
  const int tpc = 128 / tpt;                    // tokens per CTA
  const int t = blockIdx.x * tpc + threadIdx.x / tpt, head = blockIdx.y;
  const int d = (threadIdx.x % tpt) * 8;
  const int C = 2 * nk * D + nv * D;
  const int c = head * D + d;
  float val[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) val[e] = 0.f;
  if (t < T) {
    const int pos = positions[t];
    const int seq = seq_ids[t];
    const int t0 = q_start[seq];
    const bf16* rg = ring + (size_t)state_slots[seq] * ring_slot_stride;
    uint4 rows[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {               // tap KW-1 multiplies the newest row
      rows[j] = make_uint4(0u, 0u, 0u, 0u);
      if (j < KW) {
        const int back = KW - 1 - j;
        const int pj = pos - back;
        if (pj >= 0) {
          const bf16* src = t - back >= t0 ? inp + (size_t)(t - back) * ld + c : rg + (size_t)(pj % RING) * C + c;
          if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            rows[j] = *reinterpret_cast<const uint4*>(src);
          } else {                              // row width not a multiple of 8 (odd head counts of a TP shard): 4-byte pieces
            const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src);
            rows[j] = make_uint4(s32[0], s32[1], s32[2], s32[3]);
          }
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float wt[4] = {0.f, 0.f, 0.f, 0.f};
      if (KW == 4) {
        const float4 w4 = *reinterpret_cast<const float4*>(conv_w + (size_t)(c + e) * 4);
        wt[0] = w4.x, wt[1] = w4.y, wt[2] = w4.z, wt[3] = w4.w;
      } else {
        for (int j = 0; j < KW; ++j) wt[j] = conv_w[(size_t)(c + e) * KW + j];
      }
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t wd = e < 2 ? rows[j].x : e < 4 ? rows[j].y : e < 6 ? rows[j].z : rows[j].w;
        const float2 f = bf162_bits_to_f2(wd);
        acc = fmaf((e & 1) ? f.y : f.x, wt[j], acc);
      }
      val[e] = silu_f(acc);
    }
  }
  if (head < 2 * nk) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += val[e] * val[e];
    for (int m = 1; m < tpt; m <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);   // the token's threads are lane-aligned
    const float nrm = rsqrtf(ss + 1e-12f) * (head < nk ? rsqrtf((float)D) : 1.f);
    if (t < T) {
      float* dst = (head < nk ? qn + ((size_t)t * nk + head) * D : kn + ((size_t)t * nk + (head - nk)) * D) + d;
      *reinterpret_cast<float4*>(dst) = make_float4(val[0] * nrm, val[1] * nrm, val[2] * nrm, val[3] * nrm);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(val[4] * nrm, val[5] * nrm, val[6] * nrm, val[7] * nrm);
    }
  } else if (t < T) {
    float* dst = vc + ((size_t)t * nv + (head - 2 * nk)) * D + d;
    *reinterpret_cast<float4*>(dst) = make_float4(val[0], val[1], val[2], val[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(val[4], val[5], val[6], val[7]);
  }
  if (head == 0) {
    const int tb = blockIdx.x * tpc;
    for (int x = threadIdx.x; x < tpc * nv; x += blockDim.x) {
      const int tt = tb + x / nv, h = x % nv;
      if (tt >= T) break;
      const bf16* ab = inp + (size_t)tt * ld + C + nv * D;
      const float a = __bfloat162float(ab[h]), b = __bfloat162float(ab[nv + h]);
      gout[(size_t)tt * nv + h] = -__expf(a_log[h]) * softplus_f(a + dt_bias[h]);
      bout[(size_t)tt * nv + h] = sigmoid_f(b);
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


// ---------------------------------------------------------------------------------------
// Chunk-parallel prefill scan on the tensor cores (mma.sync m16n8k16 bf16, fp32 accumulate;
// dk = dv = 128).  One CTA of 8 warps per (sequence, value head) walks the sequence in chunks of
// 16 tokens; the fp32 state lives in accumulator fragments (warp w owns state rows 16 w .. 16 w + 15)
// with a bf16 copy in shared memory as the B operand of the products that read it.  Per chunk
// (G_i = running sum of the log-decays, all decays applied in fp32):
//   KK = K K^T, QK = Q K^T                       (16 x 16 x 128, warps 0 and 1)
//   A = beta_i KK_ij e^{G_i - G_j} (j < i),  T = (I + A)^-1   (forward substitution, one warp; bf16 hi + lo)
//   W = T (K beta e^G),  U = T (V beta)          (16 x 128 x 16 each)
//   V' = U - W S                                 (16 x 128 x 128)
//   O = (Q e^G) S + (QK e^{G_i - G_j}, j <= i) V'
//   S <- e^{G_last} S + (K e^{G_last - G})^T V'  (128 x 128 x 16)
// followed by the gated RMSNorm of the 16 output rows.  Operands are bf16 (the state's bf16 copy
// included), accumulation and the state itself fp32: the precision of chunked delta-rule kernels
// on tensor cores in general.  Reference parity: the six-stage chunk pipeline of
// packages/tilerl-kernels/src/tilerl_kernels/kernels_gdn.py:128-537 (cumsum, kkt, solve_tril, wu,
// state scan, chunk output), here one kernel.
constexpr int GC_C = 16, GC_D = 128, GC_ROW = GC_D * 2;     // chunk, head dim, bytes of a bf16 row over dk
constexpr int GC_NS = 2, GC_DV = GC_D / GC_NS, GC_VROW = GC_DV * 2;   // value columns per CTA, bytes of such a row
struct GcSmem {
  float sq[2][GC_C][GC_D], sk[2][GC_C][GC_D];    // fp32 q, k of the current and the next chunk
  float sv[2][GC_C][GC_DV];                      // fp32 v, this CTA's columns
  float sg[2][GC_C], sb[2][GC_C];
  __align__(128) unsigned char qraw[GC_C * GC_ROW], kraw[GC_C * GC_ROW], qe[GC_C * GC_ROW], kb[GC_C * GC_ROW],
      ws[GC_C * GC_ROW];                                                 // bf16 [16][128 dk], 16-byte chunks XOR-swizzled
  __align__(128) unsigned char vb[GC_C * GC_VROW], vn[GC_C * GC_VROW];   // bf16 [16][64 dv]
  __align__(128) unsigned char sbf[GC_D * GC_VROW];                      // bf16 copy of the state [dk][64 dv], swizzled
  __align__(16) unsigned char kdt[GC_D * 32];                            // (K e^{G_last - G})^T  bf16 [128][16]
  __align__(16) unsigned char t_hi[GC_C * 32], t_lo[GC_C * 32], qkm[GC_C * 32];   // bf16 [16][16]
  float a[GC_C][GC_C + 1];                       // fp32 A
};
__device__ __forceinline__ void gc_cp4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ uint32_t gc_off(int r, int c) { return (uint32_t)(r * GC_ROW + ((c ^ (r & 7)) << 4)); }
__device__ __forceinline__ uint32_t gc_offv(int r, int c) { return (uint32_t)(r * GC_VROW + ((c ^ (r & 7)) << 4)); }
__device__ __forceinline__ void gc_ldsm(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void gc_ldsm_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void gc_ldsm2_t(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void gc_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (2 nv, B): CTA = (value head, half of its value columns, sequence).  The delta rule never mixes
// value columns, so the two halves of a head are independent scans; what depends only on q, k and
// the gates (KK, QK, T, W) is computed by both.  Raw outputs go to o_scratch (fp32); the gated
// RMSNorm, which needs whole rows, is the small kernel below.
__global__ void __launch_bounds__(256, 2)
gdn_chunk_mma_kernel(const float* qn, const float* kn, const float* vc, const float* gin, const float* bin,
                     float* states, int* cur, bf16* ring, const bf16* inp, int ld, const int* q_start,
                     const int* q_len, const int* positions, const int* state_slots, long state_slot_stride,
                     long plane_stride, long ring_slot_stride, float* o_scratch, int nk, int nv) {
  constexpr int D = GC_D, C = GC_C, DV = GC_DV;
  extern __shared__ __align__(128) unsigned char gc_raw[];
  GcSmem& sm = *reinterpret_cast<GcSmem*>(gc_raw);
  pdl_launch_dependents(2);
  pdl_wait();
  const int h = blockIdx.x / GC_NS, c0 = (blockIdx.x % GC_NS) * DV, seq = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = q_len[seq], t0 = q_start[seq];
  if (T == 0) return;
  const int slot = state_slots[seq];
  const int kh = h * nk / nv;
  const int live = cur[slot];
  float* sp = states + (size_t)slot * state_slot_stride + (size_t)h * D * D + (size_t)live * plane_stride + c0;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;      // ldmatrix row of this lane (both x4 layouts used here)

  auto u32 = [](const void* p) { return (uint32_t)__cvta_generic_to_shared(p); };
  const uint32_t a_qraw = u32(sm.qraw), a_kraw = u32(sm.kraw), a_qe = u32(sm.qe), a_kb = u32(sm.kb), a_vb = u32(sm.vb),
                 a_ws = u32(sm.ws), a_vn = u32(sm.vn), a_sbf = u32(sm.sbf), a_kdt = u32(sm.kdt), a_thi = u32(sm.t_hi),
                 a_tlo = u32(sm.t_lo), a_qkm = u32(sm.qkm);

  // state rows 16 warp .. 16 warp + 15, this CTA's 64 columns, as accumulator fragments
  float S[DV / 8][4];
#pragma unroll
  for (int nt = 0; nt < DV / 8; ++nt) {
    const float2 lo = *reinterpret_cast<const float2*>(sp + (size_t)(16 * warp + g8) * D + nt * 8 + t4 * 2);
    const float2 hi = *reinterpret_cast<const float2*>(sp + (size_t)(16 * warp + g8 + 8) * D + nt * 8 + t4 * 2);
    S[nt][0] = lo.x, S[nt][1] = lo.y, S[nt][2] = hi.x, S[nt][3] = hi.y;
  }
  auto store_sbf = [&]() {
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
      *reinterpret_cast<uint32_t*>(sm.sbf + gc_offv(16 * warp + g8, nt) + t4 * 4) = f2_to_bf162_bits(S[nt][0], S[nt][1]);
      *reinterpret_cast<uint32_t*>(sm.sbf + gc_offv(16 * warp + g8 + 8, nt) + t4 * 4) = f2_to_bf162_bits(S[nt][2], S[nt][3]);
    }
  };
  store_sbf();

  auto stage = [&](int i0, int b) {      // fp32 q, k, v rows and the gates of chunk i0 .. i0 + 15 (rows past T: zeros)
    for (int x = tid; x < C * (D / 4); x += 256) {
      const int tt = x / (D / 4), e = (x % (D / 4)) * 4;
      if (i0 + tt < T) {
        const size_t src = ((size_t)(t0 + i0 + tt) * nk + kh) * D + e;
        cp_async16(&sm.sq[b][tt][e], qn + src);
        cp_async16(&sm.sk[b][tt][e], kn + src);
      } else {
        *reinterpret_cast<float4*>(&sm.sq[b][tt][e]) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(&sm.sk[b][tt][e]) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    {
      const int tt = tid >> 4, e = (tid & 15) * 4;
      if (i0 + tt < T) cp_async16(&sm.sv[b][tt][e], vc + ((size_t)(t0 + i0 + tt) * nv + h) * D + c0 + e);
      else *reinterpret_cast<float4*>(&sm.sv[b][tt][e]) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (tid < C) {                       // gates: asynchronous too, nothing of the next chunk is waited for here
      if (i0 + tid < T) {
        gc_cp4(&sm.sg[b][tid], gin + (size_t)(t0 + i0 + tid) * nv + h);
        gc_cp4(&sm.sb[b][tid], bin + (size_t)(t0 + i0 + tid) * nv + h);
      } else {
        sm.sg[b][tid] = 0.f, sm.sb[b][tid] = 0.f;                           // padding rows: no decay, no update
      }
    }
    cp_async_commit();
  };

  stage(0, 0);
  int b = 0;
  for (int i0 = 0; i0 < T; i0 += C, b ^= 1) {
    cp_async_wait<0>();
    __syncthreads();                       // chunk b landed; the previous chunk's tiles are free
    if (i0 + C < T) stage(i0 + C, b ^ 1);
    // running sums of the log-decays, recomputed where they are needed (16 broadcast reads)
    float g_last = 0.f;
#pragma unroll
    for (int j = 0; j < C; ++j) g_last += sm.sg[b][j];
    // ---- operand tiles (bf16) from the staged fp32 rows: thread = (token, 8 columns)
    {
      const int tt = tid >> 4, ch = tid & 15, e = ch * 8;
      float gi = 0.f;
      for (int j = 0; j <= tt; ++j) gi += sm.sg[b][j];
      const float eg = __expf(gi), beta = sm.sb[b][tt], kbs = beta * eg;
      const float4 q0 = *reinterpret_cast<const float4*>(&sm.sq[b][tt][e]), q1 = *reinterpret_cast<const float4*>(&sm.sq[b][tt][e + 4]);
      const float4 k0 = *reinterpret_cast<const float4*>(&sm.sk[b][tt][e]), k1 = *reinterpret_cast<const float4*>(&sm.sk[b][tt][e + 4]);
      const float qv[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      const float kv[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
      uint32_t oq[4], ok_[4], oqe[4], okb[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        oq[j] = f2_to_bf162_bits(qv[2 * j], qv[2 * j + 1]);
        ok_[j] = f2_to_bf162_bits(kv[2 * j], kv[2 * j + 1]);
        oqe[j] = f2_to_bf162_bits(qv[2 * j] * eg, qv[2 * j + 1] * eg);
        okb[j] = f2_to_bf162_bits(kv[2 * j] * kbs, kv[2 * j + 1] * kbs);
      }
      const uint32_t off = gc_off(tt, ch);
      *reinterpret_cast<uint4*>(sm.qraw + off) = make_uint4(oq[0], oq[1], oq[2], oq[3]);
      *reinterpret_cast<uint4*>(sm.kraw + off) = make_uint4(ok_[0], ok_[1], ok_[2], ok_[3]);
      *reinterpret_cast<uint4*>(sm.qe + off) = make_uint4(oqe[0], oqe[1], oqe[2], oqe[3]);
      *reinterpret_cast<uint4*>(sm.kb + off) = make_uint4(okb[0], okb[1], okb[2], okb[3]);
      if (ch < DV / 8) {
        const float4 v0 = *reinterpret_cast<const float4*>(&sm.sv[b][tt][e]), v1 = *reinterpret_cast<const float4*>(&sm.sv[b][tt][e + 4]);
        *reinterpret_cast<uint4*>(sm.vb + gc_offv(tt, ch)) =
            make_uint4(f2_to_bf162_bits(v0.x * beta, v0.y * beta), f2_to_bf162_bits(v0.z * beta, v0.w * beta),
                       f2_to_bf162_bits(v1.x * beta, v1.y * beta), f2_to_bf162_bits(v1.z * beta, v1.w * beta));
      }
    }
    {
      // transposed decayed keys [dk][token]: thread = (dk row, 8 tokens), one 16-byte store
      const int r = tid & 127, half = tid >> 7;
      float gi = 0.f;
      for (int j = 0; j < half * 8; ++j) gi += sm.sg[b][j];
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        gi += sm.sg[b][half * 8 + 2 * j];
        const float x0 = sm.sk[b][half * 8 + 2 * j][r] * __expf(g_last - gi);
        gi += sm.sg[b][half * 8 + 2 * j + 1];
        const float x1 = sm.sk[b][half * 8 + 2 * j + 1][r] * __expf(g_last - gi);
        o[j] = f2_to_bf162_bits(x0, x1);
      }
      *reinterpret_cast<uint4*>(sm.kdt + (size_t)r * 32 + half * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    __syncthreads();
    // ---- warp 0: KK -> A -> T = (I + A)^-1;  warp 1: QK';  warps 2..7 meanwhile start O = (Q e^G) S
    float O[4] = {0.f, 0.f, 0.f, 0.f};     // this warp's 8 value columns
    auto qs_product = [&]() {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t af[4], bs[2];
        gc_ldsm(af, a_qe + gc_off(lrow, kk * 2 + (lane >> 4)));
        gc_ldsm2_t(bs, a_sbf + gc_offv(kk * 16 + lrow, warp));
        gc_mma(O, af, bs[0], bs[1]);
      }
    };
    if (warp < 2) {
      float gc[C];                         // inclusive running sums
      {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < C; ++j) acc += sm.sg[b][j], gc[j] = acc;
      }
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const uint32_t a_base = warp == 0 ? a_kraw : a_qraw;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t af[4], bfr[4];
        gc_ldsm(af, a_base + gc_off(lrow, kk * 2 + (lane >> 4)));
        gc_ldsm(bfr, a_kraw + gc_off((lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1)));
        gc_mma(acc[0], af, bfr[0], bfr[1]);
        gc_mma(acc[1], af, bfr[2], bfr[3]);
      }
#pragma unroll
      for (int n8 = 0; n8 < 2; ++n8)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = g8 + (e >> 1) * 8, j = n8 * 8 + t4 * 2 + (e & 1);
          float gi_ = 0.f, gj_ = 0.f;
#pragma unroll
          for (int q = 0; q < C; ++q) gi_ = q == i ? gc[q] : gi_, gj_ = q == j ? gc[q] : gj_;
          const float dec = j <= i ? __expf(gi_ - gj_) : 0.f;
          if (warp == 0) sm.a[i][j] = j < i ? sm.sb[b][i] * acc[n8][e] * dec : 0.f;
          else *reinterpret_cast<bf16*>(sm.qkm + i * 32 + j * 2) = __float2bfloat16(acc[n8][e] * dec);
        }
      if (warp == 0) {
        __syncwarp();
        if (lane < C) {                    // lane j solves column j of T by forward substitution
          float tcol[C];
#pragma unroll
          for (int i = 0; i < C; ++i) {
            float v = i == lane ? 1.f : 0.f;
#pragma unroll
            for (int m = 0; m < i; ++m) v -= sm.a[i][m] * tcol[m];
            tcol[i] = i < lane ? 0.f : v;
          }
#pragma unroll
          for (int i = 0; i < C; ++i) {
            const bf16 hi = __float2bfloat16(tcol[i]);
            *reinterpret_cast<bf16*>(sm.t_hi + i * 32 + lane * 2) = hi;
            *reinterpret_cast<bf16*>(sm.t_lo + i * 32 + lane * 2) = __float2bfloat16(tcol[i] - __bfloat162float(hi));
          }
        }
      }
    } else {
      qs_product();
    }
    __syncthreads();
    // ---- W = T (K beta e^G) over all of dk (16 columns per warp); U = T (V beta), this warp's 8 value columns
    if (warp < 2) qs_product();
    float U[4] = {0.f, 0.f, 0.f, 0.f};
    {
      float Wf[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      uint32_t thi[4], tlo[4], bk[4], bv[2];
      const uint32_t trow = (uint32_t)(lrow * 32 + (lane >> 4) * 16);
      gc_ldsm(thi, a_thi + trow);
      gc_ldsm(tlo, a_tlo + trow);
      gc_ldsm_t(bk, a_kb + gc_off(lrow, 2 * warp + (lane >> 4)));
      gc_ldsm2_t(bv, a_vb + gc_offv(lrow, warp));
      gc_mma(Wf[0], thi, bk[0], bk[1]), gc_mma(Wf[1], thi, bk[2], bk[3]);
      gc_mma(Wf[0], tlo, bk[0], bk[1]), gc_mma(Wf[1], tlo, bk[2], bk[3]);
      gc_mma(U, thi, bv[0], bv[1]);
      gc_mma(U, tlo, bv[0], bv[1]);
#pragma unroll
      for (int n8 = 0; n8 < 2; ++n8) {
        *reinterpret_cast<uint32_t*>(sm.ws + gc_off(g8, 2 * warp + n8) + t4 * 4) = f2_to_bf162_bits(Wf[n8][0], Wf[n8][1]);
        *reinterpret_cast<uint32_t*>(sm.ws + gc_off(g8 + 8, 2 * warp + n8) + t4 * 4) = f2_to_bf162_bits(Wf[n8][2], Wf[n8][3]);
      }
    }
    __syncthreads();
    // ---- V' = U - W S (this warp's 8 columns), kept as the bf16 B operand of the next two products
    {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t af[4], bs[2];
        gc_ldsm(af, a_ws + gc_off(lrow, kk * 2 + (lane >> 4)));
        gc_ldsm2_t(bs, a_sbf + gc_offv(kk * 16 + lrow, warp));
        gc_mma(acc, af, bs[0], bs[1]);
      }
      *reinterpret_cast<uint32_t*>(sm.vn + gc_offv(g8, warp) + t4 * 4) = f2_to_bf162_bits(U[0] - acc[0], U[1] - acc[1]);
      *reinterpret_cast<uint32_t*>(sm.vn + gc_offv(g8 + 8, warp) + t4 * 4) = f2_to_bf162_bits(U[2] - acc[2], U[3] - acc[3]);
    }
    __syncthreads();
    // ---- O += QK' V' (this warp's 8 columns) -> raw rows; state rows of this warp: S <- e^{G_last} S + Kd^T V'
    {
      uint32_t aq[4], bvn[2];
      gc_ldsm(aq, a_qkm + (uint32_t)(lrow * 32 + (lane >> 4) * 16));
      gc_ldsm2_t(bvn, a_vn + gc_offv(lrow, warp));
      gc_mma(O, aq, bvn[0], bvn[1]);
      float* orow = o_scratch + ((size_t)(t0 + i0) * nv + h) * D + c0 + 8 * warp + t4 * 2;
      if (i0 + g8 < T) *reinterpret_cast<float2*>(orow + (size_t)g8 * nv * D) = make_float2(O[0], O[1]);
      if (i0 + g8 + 8 < T) *reinterpret_cast<float2*>(orow + (size_t)(g8 + 8) * nv * D) = make_float2(O[2], O[3]);
      const float el = __expf(g_last);
      uint32_t ak[4];
      gc_ldsm(ak, a_kdt + (uint32_t)((16 * warp + lrow) * 32 + (lane >> 4) * 16));
#pragma unroll
      for (int nt = 0; nt < DV / 8; nt += 2) {
        uint32_t bvv[4];
        gc_ldsm_t(bvv, a_vn + gc_offv(lrow, nt + (lane >> 4)));
#pragma unroll
        for (int e = 0; e < 4; ++e) S[nt][e] *= el, S[nt + 1][e] *= el;
        gc_mma(S[nt], ak, bvv[0], bvv[1]);
        gc_mma(S[nt + 1], ak, bvv[2], bvv[3]);
      }
    }
    __syncthreads();                       // every warp has read the old state copy
    store_sbf();
  }
  // ---- state back to its plane; conv ring refresh for the last tokens (as the token-serial scan does)
#pragma unroll
  for (int nt = 0; nt < DV / 8; ++nt) {
    *reinterpret_cast<float2*>(sp + (size_t)(16 * warp + g8) * D + nt * 8 + t4 * 2) = make_float2(S[nt][0], S[nt][1]);
    *reinterpret_cast<float2*>(sp + (size_t)(16 * warp + g8 + 8) * D + nt * 8 + t4 * 2) = make_float2(S[nt][2], S[nt][3]);
  }
  if (c0 == 0) {
    const int cw = 2 * nk * D + nv * D;
    bf16* rg = ring + (size_t)slot * ring_slot_stride;
    const int first = max(0, T - RING);
    const int rep = nv / nk;
    for (int i = first; i < T; ++i) {
      const int t = t0 + i;
      const int rrow = positions[t] % RING;
      const bf16* src = inp + (size_t)t * ld;
      bf16* dst = rg + (size_t)rrow * cw;
      if (h % rep == 0) {
        for (int c = tid; c < 2 * D; c += 256) {
          const int cc = (c < D) ? kh * D + c : nk * D + kh * D + (c - D);
          dst[cc] = src[cc];
        }
      }
      for (int c = tid; c < D; c += 256) {
        const int cc = 2 * nk * D + h * D + c;
        dst[cc] = src[cc];
      }
    }
  }
  trl_trace_end();
}

// Gated RMSNorm of raw GDN output rows: out[t, h, :] = o * rsqrt(mean(o^2) + eps) * w * silu(z); one warp per row.
__global__ void __launch_bounds__(256)
gdn_gated_norm_kernel(const float* o_scratch, const bf16* inp, int ld, const float* __restrict__ norm_w, float eps,
                      bf16* out, int rows, int nk, int nv) {
  constexpr int D = GC_D;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int t = row / nv, h = row % nv;
  const float4 ov = __ldcg(reinterpret_cast<const float4*>(o_scratch + (size_t)row * D) + lane);
  const uint2 zr = *reinterpret_cast<const uint2*>(inp + (size_t)t * ld + (2 * nk * D + nv * D) + (size_t)h * D + lane * 4);
  const float4 w = *reinterpret_cast<const float4*>(norm_w + lane * 4);
  const float ss = warp_sum(ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w);
  const float rstd = rsqrtf(ss / (float)D + eps);
  const float2 z0 = bf162_bits_to_f2(zr.x), z1 = bf162_bits_to_f2(zr.y);
  uint2 o;
  o.x = f2_to_bf162_bits(ov.x * rstd * w.x * silu_f(z0.x), ov.y * rstd * w.y * silu_f(z0.y));
  o.y = f2_to_bf162_bits(ov.z * rstd * w.z * silu_f(z1.x), ov.w * rstd * w.w * silu_f(z1.y));
  *reinterpret_cast<uint2*>(out + (size_t)row * D + lane * 4) = o;
}

}  // namespace

static int g_gdn_wy = -1;   // -1: read TRL_GDN_WY at the first launch
static int g_gdn_mma = -1;  // -1: on unless TRL_GDN_MMA=0 (read at the first launch)

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
// Prefill scan on the tensor cores (gdn_chunk_mma_kernel): 1 on, 0 off (token-serial scan), -1 = the environment's choice.
TRL_API void trl_gdn_set_mma(int on) { g_gdn_mma = on; }

// Scratch (fp32): qn, kn [T*nk*D]; vc, o_scratch [T*nv*D]; g, beta [T*nv].
TRL_API int trl_gdn(const void* inp, int ld, const void* conv_w, const void* dt_bias, const void* a_log,
                    const void* norm_w, void* states, void* cur, void* ring, const void* positions,
                    const void* seq_ids, const void* q_start, const void* q_len,
                    const void* state_slots, const void* keep_flags, long state_slot_stride,
                    long plane_stride, long ring_slot_stride, void* qn, void* kn, void* vc, void* g,
                    void* beta, void* o_scratch, void* out, int T, int B, int nk, int nv, int D, int KW,
                    int planes, float eps, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (KW > 4) return (int)cudaErrorInvalidValue;
  if ((D != 64 && D != 128) || (ld % 2) != 0) return (int)cudaErrorInvalidValue;
  const int prep_tpc = 1024 / D;
  cudaError_t e = trl_launch(gdn_prep_kernel, dim3((T + prep_tpc - 1) / prep_tpc, 2 * nk + nv), dim3(128), 0, st,
                             (const bf16*)inp, ld, (const float*)conv_w, (const float*)dt_bias, (const float*)a_log,
                             (const bf16*)ring, (const int*)positions, (const int*)seq_ids,
                             (const int*)q_start, (const int*)state_slots, ring_slot_stride,
                             (float*)qn, (float*)kn, (float*)vc, (float*)g, (float*)beta, nk, nv, D, KW, T);
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
  // prefill ticks (more tokens than sequences, no per-token state planes) with dk = dv = 128 take the
  // tensor-core chunk kernel; TRL_GDN_MMA=0 (or trl_gdn_set_mma(0)) falls back to the token-serial scan
  if (g_gdn_mma < 0) g_gdn_mma = (getenv("TRL_GDN_MMA") && atoi(getenv("TRL_GDN_MMA")) == 0) ? 0 : 1;
  if (g_gdn_mma != 0 && D == 128 && T > B && keep_flags == nullptr) {
    static bool configured = false;
    if (!configured) {
      if (cudaFuncSetAttribute(gdn_chunk_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(GcSmem)) != cudaSuccess)
        return 3;
      configured = true;
    }
    e = trl_launch(gdn_chunk_mma_kernel, dim3(nv * GC_NS, B), dim3(256), sizeof(GcSmem), st, (const float*)qn,
                   (const float*)kn, (const float*)vc, (const float*)g, (const float*)beta, (float*)states, (int*)cur,
                   (bf16*)ring, (const bf16*)inp, ld, (const int*)q_start, (const int*)q_len, (const int*)positions,
                   (const int*)state_slots, state_slot_stride, plane_stride, ring_slot_stride, (float*)o_scratch, nk, nv);
    if (e != cudaSuccess) return (int)e;
    return (int)trl_launch(gdn_gated_norm_kernel, dim3((T * nv + 7) / 8), dim3(256), 0, st, (const float*)o_scratch,
                           (const bf16*)inp, ld, (const float*)norm_w, eps, (bf16*)out, T * nv, nk, nv);
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
