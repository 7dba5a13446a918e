// Skinny (M <= 4 rows per pass) weight-streaming linears for the decode tick.
//
//   y[m, n] = epi( tscale * sum_k x'[m, k] * W[n, k] )
//
// * W is NVFP4 in the checkpoint layout: e2m1 nibbles [N, K/2] (low nibble = even
//   k), one e4m3 scale per 16 k [N, K/16], one fp32 tensor scale -- or bf16 [N, K].
// * x' = x, or RMSNorm(x) * norm_w when norm_w != nullptr: the norm is folded into
//   the prologue, every CTA recomputes it from the (L2-resident) activation row.
// * epi: plain store | + residual | SwiGLU on interleaved (gate, up) row pairs.
//
// The kernel is HBM-bound by construction: each warp owns R consecutive weight
// rows and walks K in 32-weight chunks with 128-bit streaming loads (R*U loads
// in flight per lane).  The activation lives in shared memory as f16, pre-scaled
// by a per-row power of two so that a 16-element block sum cannot overflow, in a
// chunk-interleaved layout that makes the four 16-byte reads per chunk
// bank-conflict free.  e2m1 -> f16x2 uses the native cvt; products accumulate in
// f16x2 within one 16-element scale block (exact products: 2-bit x 8-bit
// mantissas), then promote to fp32 with the block scale.
//
// Reference parity: `linear_fp4_gemv` / `linear_bf16_gemv` of
// packages/tilerl-kernels/src/tilerl_kernels/kernels_linear.py:924-1097.
#include <stdlib.h>

#include "common.cuh"

__device__ TrlError g_trl_error = {0, 0, 0, 0};
int g_trl_use_pdl = 1;
#ifdef TRL_TRACE
__device__ TrlTraceRec g_trl_trace[TRL_TRACE_CAP];
__device__ unsigned int g_trl_trace_n = 0;
__device__ unsigned int g_trl_trace_cur = 0;
__device__ unsigned long long g_trl_last_exit = 0;
#endif

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_STORE_F32 = 3, EPI_PUSH = 4 };

namespace {

constexpr int GEMV_THREADS = 512;

// Stage x (bf16 [M, K], optional RMSNorm) into shared memory as scaled f16.
// Layout per row m: piece p (8 halves) of 32-element chunk c sits at
// ((p * nchunks + c) * 8) halves.  Returns nothing; xs_inv[m] = 1 / applied scale.
template <int M>
__device__ __forceinline__ void stage_x(const bf16* x, int ldx, int K,
                                        const float* __restrict__ norm_w, float eps,
                                        __half* xs, float* xs_inv, float* red) {
  const int nchunks = K >> 5;
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const bf16* xr = x + (size_t)m * ldx;
    // one pass: sum of squares and max |x * w| together (the max of the normalised row is
    // rstd times the latter), one block reduction for both
    float rstd = 1.f;
    float ss = 0.f, amax = 0.f;
    for (int k = threadIdx.x * 2; k < K; k += blockDim.x * 2) {
      float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + k));
      ss += v.x * v.x + v.y * v.y;
      if (norm_w != nullptr) v.x *= norm_w[k], v.y *= norm_w[k + 1];
      amax = fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y)));
    }
    {
      const int lane_ = threadIdx.x & 31, w_ = threadIdx.x >> 5, nw_ = (blockDim.x + 31) >> 5;
      ss = warp_sum(ss);
      amax = warp_max(amax);
      __syncthreads();
      if (lane_ == 0) red[w_] = ss, red[32 + w_] = amax;
      __syncthreads();
      ss = warp_sum(lane_ < nw_ ? red[lane_] : 0.f);
      amax = warp_max(lane_ < nw_ ? red[32 + lane_] : 0.f);
    }
    if (norm_w != nullptr) {
      rstd = rsqrtf(ss / (float)K + eps);
      amax *= rstd * 1.01f;   // bf16 rounding of the normalised values can add < 0.4 %
    }
    // power-of-two scale s with amax * s <= 256: 16 products of |w| <= 6 stay < 65504
    int e = 0;
    if (amax > 0.f) {
      frexpf(amax, &e);  // amax = f * 2^e, f in [0.5, 1)
    }
    const float s = exp2f((float)(8 - e));
    if (threadIdx.x == 0) xs_inv[m] = exp2f((float)(e - 8));
    __half* dst = xs + (size_t)m * K;
    for (int k = threadIdx.x * 2; k < K; k += blockDim.x * 2) {
      float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + k));
      if (norm_w != nullptr) {
        v.x = __bfloat162float(__float2bfloat16(v.x * rstd * norm_w[k]));
        v.y = __bfloat162float(__float2bfloat16(v.y * rstd * norm_w[k + 1]));
      }
      const int c = k >> 5, p = (k >> 3) & 3, o = k & 7;
      *reinterpret_cast<__half2*>(dst + ((size_t)(p * nchunks + c) << 3) + o) =
          __floats2half2_rn(v.x * s, v.y * s);
    }
  }
  __syncthreads();
}

template <int M, int R, int EPI>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
gemv_nvfp4_kernel(const bf16* x, int ldx, const uint8_t* __restrict__ wq,
                  const uint8_t* __restrict__ wscale, const float* __restrict__ tscale,
                  const float* __restrict__ norm_w, float eps, const bf16* residual,
                  int ldr, void* yout, int ldy, int N, int K, const TrlPushArgs push) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  float* xs_inv = reinterpret_cast<float*>(smem_raw + (size_t)M * K * sizeof(__half));
  float* red = xs_inv + 8;
  // a pushing kernel lets the next kernel in only after its pushes (see allreduce_finish_kernel)
  pdl_enter();
  if (EPI != EPI_PUSH) pdl_trigger();
  pdl_wait();
  stage_x<M>(x, ldx, K, norm_w, eps, xs, xs_inv, red);

  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (GEMV_THREADS / 32) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (GEMV_THREADS / 32);
  const int nchunks = K >> 5;
  const size_t row_bytes = (size_t)K >> 1, srow_bytes = (size_t)K >> 4;
  const float ts = *tscale;

  for (int r0 = warp * R; r0 < N; r0 += nwarps * R) {
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
    const uint8_t* wrow[R];
    const uint8_t* srow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int rr = min(r0 + r, N - 1);
      wrow[r] = wq + (size_t)rr * row_bytes;
      srow[r] = wscale + (size_t)rr * srow_bytes;
    }
    // D-deep register ring: while chunk c is consumed, the loads of the next D-1 chunks of
    // every row are in flight (the loop is bound by memory latency / D, not by latency)
    constexpr int D = (R * M <= 4) ? 4 : 2;
    uint4 wv[D][R];
    uint16_t sv[D][R];
#pragma unroll
    for (int d = 0; d < D; ++d) {
      const int c = lane + 32 * d;
      if (c < nchunks) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          wv[d][r] = ldg_stream_16(wrow[r] + ((size_t)c << 4));
          sv[d][r] = ldg_stream_2(srow[r] + ((size_t)c << 1));
        }
      }
    }
    for (int base = lane; base < nchunks; base += 32 * D) {
#pragma unroll
      for (int d = 0; d < D; ++d) {
        const int c = base + 32 * d;
        if (c < nchunks) {
#pragma unroll
          for (int m = 0; m < M; ++m) {
            uint32_t xh[16];
            const __half* xm = xs + (size_t)m * K;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              uint4 t = *reinterpret_cast<const uint4*>(xm + ((size_t)(p * nchunks + c) << 3));
              xh[p * 4 + 0] = t.x, xh[p * 4 + 1] = t.y, xh[p * 4 + 2] = t.z, xh[p * 4 + 3] = t.w;
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const float2 sc = h2_to_f2(cvt_e4m3x2_to_h2(sv[d][r]));
              const uint32_t w4[4] = {wv[d][r].x, wv[d][r].y, wv[d][r].z, wv[d][r].w};
#pragma unroll
              for (int blk = 0; blk < 2; ++blk) {
                uint32_t a = 0u;  // f16x2 zero
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  uint32_t h[4];
                  cvt_e2m1x8_to_h2x4(w4[blk * 2 + q], h);
#pragma unroll
                  for (int i = 0; i < 4; ++i) a = hfma2_u(h[i], xh[(blk * 2 + q) * 4 + i], a);
                }
                const float2 af = h2_to_f2(a);
                acc[r][m] = fmaf(blk == 0 ? sc.x : sc.y, af.x + af.y, acc[r][m]);
              }
            }
          }
          const int cn = c + 32 * D;
          if (cn < nchunks) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
              wv[d][r] = ldg_stream_16(wrow[r] + ((size_t)cn << 4));
              sv[d][r] = ldg_stream_2(srow[r] + ((size_t)cn << 1));
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]) * ts * xs_inv[m];

    if (EPI == EPI_SWIGLU) {
      // rows (2j, 2j+1) = (gate_j, up_j); R is even and r0 is a multiple of R
      if (lane < (R / 2) * M) {
        const int j = lane / M, m = lane % M;
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int r = 0; r < R; r += 2)
#pragma unroll
          for (int mm = 0; mm < M; ++mm)
            if (r / 2 == j && mm == m) g = acc[r][mm], u = acc[r + 1][mm];
        const int n = r0 + 2 * j;
        if (n + 1 < N)
          reinterpret_cast<bf16*>(yout)[(size_t)m * ldy + (n >> 1)] = __float2bfloat16(silu_f(g) * u);
      }
    } else {
      if (lane < R * M) {
        const int r = lane / M, m = lane % M;
        float v = 0.f;
#pragma unroll
        for (int rr = 0; rr < R; ++rr)
#pragma unroll
          for (int mm = 0; mm < M; ++mm)
            if (rr == r && mm == m) v = acc[rr][mm];
        const int n = r0 + r;
        if (n < N) {
          if (EPI == EPI_PUSH) {
            // fp32 partial row straight into every rank's all-reduce slot (NVLink stores)
            // {value, epoch} in ONE 8-byte store per peer: the receiver polls the epoch half of
            // the word it needs, so no fence, counter or separate flag sits between the last
            // weight byte and the peer's sum
            const uint32_t epoch = *reinterpret_cast<const uint32_t*>(push.ws[push.rank]) + 1;
            const size_t off = 65536 + ((size_t)(((epoch & 1) * 8 + push.rank) * 8 + push.row0 + m) * push.hmax + n) * 8;
            const uint2 word = make_uint2(__float_as_uint(v), epoch);
            for (int p = 0; p < push.world; ++p) st_relaxed_sys_v2(push.ws[p] + off, word);
          } else {
            if (EPI == EPI_RESIDUAL) v += __bfloat162float(residual[(size_t)m * ldr + n]);
            if (EPI == EPI_STORE_F32)
              reinterpret_cast<float*>(yout)[(size_t)m * ldy + n] = v;
            else
              reinterpret_cast<bf16*>(yout)[(size_t)m * ldy + n] = __float2bfloat16(v);
          }
        }
      }
    }
  }
  if (EPI == EPI_PUSH) pdl_trigger();
}

// Balanced variant.  A CTA owns a contiguous block of row PAIRS and its 16 warps split that
// block's (pair, 32-chunk step) units evenly, whatever the row count: a 5120-row projection
// on 148 x 16 warps no longer runs two rounds with the second almost empty.  A pair that is
// cut between warps is summed through shared-memory slots in a fixed order (bitwise
// reproducible); the epilogue then runs block-wide with coalesced stores.
__device__ __forceinline__ int sk_owner(int unit, int U, int W) {
  int w = (int)(((long long)unit * W) / U);
  while (w + 1 < W && (int)(((long long)(w + 1) * U) / W) <= unit) ++w;
  while (w > 0 && (int)(((long long)w * U) / W) > unit) --w;
  return w;
}

template <int M, int EPI>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
gemv_nvfp4_sk_kernel(const bf16* x, int ldx, const uint8_t* __restrict__ wq,
                     const uint8_t* __restrict__ wscale, const float* __restrict__ tscale,
                     const float* __restrict__ norm_w, float eps, const bf16* residual,
                     int ldr, void* yout, int ldy, int N, int K, int nslot,
                     const TrlPushArgs push) {
  constexpr int W = GEMV_THREADS / 32;
  constexpr int D = 4;   // units in flight per lane: 4 x 2 rows x 16 B
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  float* xs_inv = reinterpret_cast<float*>(smem_raw + (size_t)M * K * sizeof(__half));
  float* red = xs_inv + 8;
  float* slots = red + 64;   // [pairs_local][2 rows][nslot][M]
  pdl_enter();
  if (EPI != EPI_PUSH) pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int npairs = N >> 1;
  const int p_lo = (int)(((long long)blockIdx.x * npairs) / gridDim.x);
  const int p_hi = (int)(((long long)(blockIdx.x + 1) * npairs) / gridDim.x);
  const int pl = p_hi - p_lo;
  for (int i = threadIdx.x; i < pl * 2 * nslot * M; i += GEMV_THREADS) slots[i] = 0.f;
  pdl_wait();
  stage_x<M>(x, ldx, K, norm_w, eps, xs, xs_inv, red);   // ends with a block barrier

  const int nchunks = K >> 5;
  const int nsteps = (nchunks + 31) >> 5;
  const size_t row_bytes = (size_t)K >> 1, srow_bytes = (size_t)K >> 4;
  const int U = pl * nsteps;
  const int u0 = (int)(((long long)warp * U) / W), u1 = (int)(((long long)(warp + 1) * U) / W);

  if (u0 < u1) {
    uint4 wv[D][2];
    uint16_t sv[D][2];
    // loader cursor
    // byte offsets from this CTA's first row (32-bit: a CTA's block is a few MB), advanced
    // incrementally: 32 chunks per step, two rows per pair
    int ls = u0 % nsteps;
    const uint8_t* wbase = wq + (size_t)p_lo * 2 * row_bytes;
    const uint8_t* sbase = wscale + (size_t)p_lo * 2 * srow_bytes;
    uint32_t woff = (uint32_t)(u0 / nsteps) * 2u * (uint32_t)row_bytes + (uint32_t)(ls * 32 + lane) * 16u;
    uint32_t soff = (uint32_t)(u0 / nsteps) * 2u * (uint32_t)srow_bytes + (uint32_t)(ls * 32 + lane) * 2u;
    const uint32_t wwrap = 2u * (uint32_t)row_bytes - (uint32_t)nsteps * 512u;
    const uint32_t swrap = 2u * (uint32_t)srow_bytes - (uint32_t)nsteps * 64u;
    auto load = [&](int d) {
      if (ls * 32 + lane < nchunks) {
        wv[d][0] = ldg_stream_16(wbase + woff);
        wv[d][1] = ldg_stream_16(wbase + woff + (uint32_t)row_bytes);
        sv[d][0] = ldg_stream_2(sbase + soff);
        sv[d][1] = ldg_stream_2(sbase + soff + (uint32_t)srow_bytes);
      }
      woff += 512u, soff += 64u;
      if (++ls == nsteps) ls = 0, woff += wwrap, soff += swrap;
    };
#pragma unroll
    for (int d = 0; d < D; ++d)
      if (u0 + d < u1) load(d);
    // consumer cursor
    int cp = u0 / nsteps, cs = u0 % nsteps;
    float acc[2][M];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
    auto flush = [&](int pair_local) {
      // two-slot mode: slot 0 belongs to the warp that holds the pair's first unit
      const int slot = nslot == 2 ? (pair_local * nsteps >= u0 ? 0 : 1) : warp - sk_owner(pair_local * nsteps, U, W);
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float v = warp_sum(acc[r][m]);
          if (lane == 0) slots[((size_t)(pair_local * 2 + r) * nslot + slot) * M + m] = v;
          acc[r][m] = 0.f;
        }
    };
    for (int ub = u0; ub < u1; ub += D) {
#pragma unroll
      for (int d = 0; d < D; ++d) {
        const int uc = ub + d;
        if (uc < u1) {
          const int c = cs * 32 + lane;
          if (c < nchunks) {
#pragma unroll
            for (int m = 0; m < M; ++m) {
              uint32_t xh[16];
              const __half* xm = xs + (size_t)m * K;
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                uint4 t = *reinterpret_cast<const uint4*>(xm + ((size_t)(p * nchunks + c) << 3));
                xh[p * 4 + 0] = t.x, xh[p * 4 + 1] = t.y, xh[p * 4 + 2] = t.z, xh[p * 4 + 3] = t.w;
              }
#pragma unroll
              for (int r = 0; r < 2; ++r) {
                const float2 sc = h2_to_f2(cvt_e4m3x2_to_h2(sv[d][r]));
                const uint32_t w4[4] = {wv[d][r].x, wv[d][r].y, wv[d][r].z, wv[d][r].w};
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                  uint32_t a = 0u;  // f16x2 zero
#pragma unroll
                  for (int q = 0; q < 2; ++q) {
                    uint32_t h[4];
                    cvt_e2m1x8_to_h2x4(w4[blk * 2 + q], h);
#pragma unroll
                    for (int i = 0; i < 4; ++i) a = hfma2_u(h[i], xh[(blk * 2 + q) * 4 + i], a);
                  }
                  const float2 af = h2_to_f2(a);
                  acc[r][m] = fmaf(blk == 0 ? sc.x : sc.y, af.x + af.y, acc[r][m]);
                }
              }
            }
          }
          if (uc + D < u1) load(d);
          if (++cs == nsteps) {
            flush(cp);
            cs = 0, ++cp;
          }
        }
      }
    }
    if (cs != 0) flush(cp);   // range ended inside a pair
  }
  __syncthreads();

  // block-wide epilogue over this CTA's rows
  const float ts = *tscale;
  if (EPI == EPI_SWIGLU) {
    for (int i = threadIdx.x; i < pl * M; i += GEMV_THREADS) {
      const int pr = i / M, m = i % M;
      float g = 0.f, u = 0.f;
      for (int sl = 0; sl < nslot; ++sl) {
        g += slots[((size_t)(pr * 2) * nslot + sl) * M + m];
        u += slots[((size_t)(pr * 2 + 1) * nslot + sl) * M + m];
      }
      const float sc = ts * xs_inv[m];
      const int n = (p_lo + pr) * 2;
      if (n + 1 < N)
        reinterpret_cast<bf16*>(yout)[(size_t)m * ldy + (n >> 1)] = __float2bfloat16(silu_f(g * sc) * (u * sc));
    }
  } else {
    for (int i = threadIdx.x; i < pl * 2 * M; i += GEMV_THREADS) {
      const int rl = i / M, m = i % M;
      const int n = p_lo * 2 + rl;
      if (n >= N) continue;
      float v = 0.f;
      for (int sl = 0; sl < nslot; ++sl) v += slots[((size_t)rl * nslot + sl) * M + m];
      v *= ts * xs_inv[m];
      if (EPI == EPI_PUSH) {
        const uint32_t epoch = *reinterpret_cast<const uint32_t*>(push.ws[push.rank]) + 1;
        const size_t off = 65536 + ((size_t)(((epoch & 1) * 8 + push.rank) * 8 + push.row0 + m) * push.hmax + n) * 8;
        const uint2 word = make_uint2(__float_as_uint(v), epoch);
        for (int p = 0; p < push.world; ++p) st_relaxed_sys_v2(push.ws[p] + off, word);
      } else {
        if (EPI == EPI_RESIDUAL) v += __bfloat162float(residual[(size_t)m * ldr + n]);
        if (EPI == EPI_STORE_F32)
          reinterpret_cast<float*>(yout)[(size_t)m * ldy + n] = v;
        else
          reinterpret_cast<bf16*>(yout)[(size_t)m * ldy + n] = __float2bfloat16(v);
      }
    }
  }
  if (EPI == EPI_PUSH) pdl_trigger();
}

// bf16 weights [N, K]: fp32 FMA, 8 weights per 16-byte load.  x staged as fp32.
template <int M, int R, int EPI>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
gemv_bf16_kernel(const bf16* x, int ldx, const bf16* __restrict__ w,
                 const float* __restrict__ norm_w, float eps, const bf16* residual,
                 int ldr, void* yout, int ldy, int N, int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* xs = reinterpret_cast<float*>(smem_raw);
  float* red = xs + (size_t)M * K;
  pdl_launch_dependents(6);
  pdl_wait();
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const bf16* xr = x + (size_t)m * ldx;
    float rstd = 1.f;
    if (norm_w != nullptr) {
      float ss = 0.f;
      for (int k = threadIdx.x; k < K; k += blockDim.x) {
        float v = __bfloat162float(xr[k]);
        ss += v * v;
      }
      ss = block_sum(ss, red);
      rstd = rsqrtf(ss / (float)K + eps);
    }
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      float v = __bfloat162float(xr[k]);
      if (norm_w != nullptr) v = __bfloat162float(__float2bfloat16(v * rstd * norm_w[k]));
      xs[(size_t)m * K + k] = v;
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (GEMV_THREADS / 32) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (GEMV_THREADS / 32);
  const int nvec = K >> 3;
  for (int r0 = warp * R; r0 < N; r0 += nwarps * R) {
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
    for (int c = lane; c < nvec; c += 32) {
      uint4 wv[R];
#pragma unroll
      for (int r = 0; r < R; ++r)
        wv[r] = ldg_stream_16(w + (size_t)min(r0 + r, N - 1) * K + ((size_t)c << 3));
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4 x0 = *reinterpret_cast<const float4*>(xs + (size_t)m * K + (c << 3));
        const float4 x1 = *reinterpret_cast<const float4*>(xs + (size_t)m * K + (c << 3) + 4);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float2 a = bf162_bits_to_f2(wv[r].x), b = bf162_bits_to_f2(wv[r].y);
          float2 cc = bf162_bits_to_f2(wv[r].z), d = bf162_bits_to_f2(wv[r].w);
          float s = acc[r][m];
          s = fmaf(a.x, x0.x, s), s = fmaf(a.y, x0.y, s), s = fmaf(b.x, x0.z, s), s = fmaf(b.y, x0.w, s);
          s = fmaf(cc.x, x1.x, s), s = fmaf(cc.y, x1.y, s), s = fmaf(d.x, x1.z, s), s = fmaf(d.y, x1.w, s);
          acc[r][m] = s;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]);
    if (lane < R * M) {
      const int r = lane / M, m = lane % M;
      float v = 0.f;
#pragma unroll
      for (int rr = 0; rr < R; ++rr)
#pragma unroll
        for (int mm = 0; mm < M; ++mm)
          if (rr == r && mm == m) v = acc[rr][mm];
      const int n = r0 + r;
      if (n < N) {
        if (EPI == EPI_RESIDUAL) v += __bfloat162float(residual[(size_t)m * ldr + n]);
        if (EPI == EPI_STORE_F32)
          reinterpret_cast<float*>(yout)[(size_t)m * ldy + n] = v;
        else
          reinterpret_cast<bf16*>(yout)[(size_t)m * ldy + n] = __float2bfloat16(v);
      }
    }
  }
}

// bf16 weights [N, K] for 3..16 activation rows on the tensor cores (mma.sync m16n8k16, fp32
// accumulation): the weight matrix is streamed ONCE for all rows (the kernel above handles four rows
// per pass).  A warp owns 16 weight rows; lane (g, t) = (lane / 4, lane % 4) loads 16 bytes (8
// consecutive k) of rows g and g + 8 per 32-wide k step straight into A fragments.  A dot product
// does not care in which order k is summed, so the 8 loaded values serve two MMAs under a fixed
// permutation of k: fragment slots {2t, 2t+1, 2t+8, 2t+9} of the first MMA are elements 0..3 of the
// lane's chunk, of the second elements 4..7; the B fragment (activation row g, staged as normalised
// bf16 in shared memory) is the same 16-byte chunk of the activation row, split the same way.
constexpr int BM_THREADS = 512, BM_PAD = 32;     // activation row stride K + 32 elements: 64 bytes off a bank cycle
template <int NT, int EPI>                       // NT tiles of 8 activation rows
__global__ void __launch_bounds__(BM_THREADS, 1)
gemv_bf16_mma_kernel(const bf16* x, int ldx, const bf16* __restrict__ w, const float* __restrict__ norm_w, float eps,
                     const bf16* residual, int ldr, void* yout, int ldy, int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);                 // [NT * 8][K + BM_PAD]
  __shared__ float red[32];
  const int ldxs = K + BM_PAD;
  pdl_launch_dependents(6);
  pdl_wait();
  for (int m = 0; m < NT * 8; ++m) {
    bf16* dst = xs + (size_t)m * ldxs;
    if (m >= M) {
      for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = __float2bfloat16(0.f);
      continue;
    }
    const bf16* xr = x + (size_t)m * ldx;
    float rstd = 1.f;
    if (norm_w != nullptr) {
      float ss = 0.f;
      for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = __bfloat162float(xr[k]);
        ss += v * v;
      }
      ss = block_sum(ss, red);
      rstd = rsqrtf(ss / (float)K + eps);
    }
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      float v = __bfloat162float(xr[k]);
      if (norm_w != nullptr) v = v * rstd * norm_w[k];
      dst[k] = __float2bfloat16(v);
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int warp = blockIdx.x * (BM_THREADS / 32) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (BM_THREADS / 32);
  const int steps = K >> 5;                                    // 32 k per step
  constexpr int U = NT == 1 ? 8 : 4;                           // steps whose weight loads are in flight together
  for (int r0 = warp * 16; r0 < N; r0 += nwarps * 16) {
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const bf16* wa = w + (size_t)min(r0 + g, N - 1) * K + (t << 3);
    const bf16* wb = w + (size_t)min(r0 + g + 8, N - 1) * K + (t << 3);
    const bf16* xb = xs + (size_t)g * ldxs + (t << 3);
    for (int j0 = 0; j0 < steps; j0 += U) {
      uint4 va[U], vb[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int j = min(j0 + u, steps - 1);
        va[u] = ldg_stream_16(wa + ((size_t)j << 5));
        vb[u] = ldg_stream_16(wb + ((size_t)j << 5));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (j0 + u < steps) {
          const uint32_t a1[4] = {va[u].x, vb[u].x, va[u].y, vb[u].y};
          const uint32_t a2[4] = {va[u].z, vb[u].z, va[u].w, vb[u].w};
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xb + (size_t)i * 8 * ldxs + ((j0 + u) << 5));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(acc[i][0]), "+f"(acc[i][1]), "+f"(acc[i][2]), "+f"(acc[i][3])
                         : "r"(a1[0]), "r"(a1[1]), "r"(a1[2]), "r"(a1[3]), "r"(xv.x), "r"(xv.y));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(acc[i][0]), "+f"(acc[i][1]), "+f"(acc[i][2]), "+f"(acc[i][3])
                         : "r"(a2[0]), "r"(a2[1]), "r"(a2[2]), "r"(a2[3]), "r"(xv.z), "r"(xv.w));
          }
        }
      }
    }
    // accumulator (row g | g + 8 of the warp's 16, activation rows 2t | 2t + 1 of tile i)
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = r0 + g + (e >> 1) * 8, m = i * 8 + 2 * t + (e & 1);
        if (n < N && m < M) {
          float v = acc[i][e];
          if (EPI == EPI_RESIDUAL) v += __bfloat162float(residual[(size_t)m * ldr + n]);
          if (EPI == EPI_STORE_F32)
            reinterpret_cast<float*>(yout)[(size_t)m * ldy + n] = v;
          else
            reinterpret_cast<bf16*>(yout)[(size_t)m * ldy + n] = __float2bfloat16(v);
        }
      }
  }
}

int g_num_sms = 0;
int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <int M, int R, int EPI>
cudaError_t launch_nvfp4(const bf16* x, int ldx, const uint8_t* wq, const uint8_t* ws, const float* ts,
                         const float* norm_w, float eps, const bf16* res, int ldr, void* y, int ldy,
                         int N, int K, cudaStream_t st, const TrlPushArgs& push) {
  const size_t smem = (size_t)M * K * sizeof(__half) + 8 * sizeof(float) + 64 * sizeof(float);
  auto kern = gemv_nvfp4_kernel<M, R, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  const int warps_needed = (N + R - 1) / R;
  int grid = min(num_sms(), (warps_needed + GEMV_THREADS / 32 - 1) / (GEMV_THREADS / 32));
  return trl_launch(kern, dim3(grid), dim3(GEMV_THREADS), smem, st, x, ldx, wq, ws, ts, norm_w, eps,
                    res, ldr, y, ldy, N, K, push);
}

template <int M, int EPI>
cudaError_t launch_nvfp4_sk(const bf16* x, int ldx, const uint8_t* wq, const uint8_t* ws, const float* ts,
                            const float* norm_w, float eps, const bf16* res, int ldr, void* y, int ldy,
                            int N, int K, cudaStream_t st, const TrlPushArgs& push) {
  constexpr int W = GEMV_THREADS / 32;
  if (N % 2 != 0) return cudaErrorInvalidValue;   // the older kernel handles odd row counts
  const int npairs = N / 2;
  const int grid = min(num_sms(), npairs);
  const int pl_max = (npairs + grid - 1) / grid;
  // a pair is shared by at most two warps once every CTA's warp share is at least one pair
  const int nslot = (npairs / grid) >= W ? 2 : W;
  const size_t smem = (size_t)M * K * sizeof(__half) + 8 * sizeof(float) + 64 * sizeof(float) +
                      (size_t)pl_max * 2 * nslot * M * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  auto kern = gemv_nvfp4_sk_kernel<M, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  return trl_launch(kern, dim3(grid), dim3(GEMV_THREADS), smem, st, x, ldx, wq, ws, ts, norm_w, eps,
                    res, ldr, y, ldy, N, K, nslot, push);
}

template <int M, int EPI>
cudaError_t dispatch_r(const bf16* x, int ldx, const uint8_t* wq, const uint8_t* ws, const float* ts,
                       const float* norm_w, float eps, const bf16* res, int ldr, void* y, int ldy,
                       int N, int K, cudaStream_t st, const TrlPushArgs& push) {
  // The balanced kernel pays a block-wide epilogue; it wins where whole-row rounds leave warps
  // idle: rounds * R row-times against the ideal N / warps.
  static const char* mode = getenv("TRL_GEMV_BALANCED");   // "0" never, "1" always, unset: by shape
  const int all_warps = num_sms() * (GEMV_THREADS / 32);
  const int R0 = (M > 2 && N >= all_warps * 4 * 2) ? 4 : 2;
  const float ideal = (float)N / (float)all_warps;
  const float rounds = (float)(((N + R0 - 1) / R0 + all_warps - 1) / all_warps) * (float)R0;
  const bool balanced = mode ? (mode[0] == '1') : (ideal / rounds < 0.7f);
  if (balanced) {
    const cudaError_t e = launch_nvfp4_sk<M, EPI>(x, ldx, wq, ws, ts, norm_w, eps, res, ldr, y, ldy, N, K, st, push);
    if (e != cudaErrorInvalidValue) return e;
  }
  // enough row blocks to give every warp of a full grid at least two -> R = 4
  const int full_warps = num_sms() * (GEMV_THREADS / 32);
  if (M > 2 && N >= full_warps * 4 * 2)
    return launch_nvfp4<M, 4, EPI>(x, ldx, wq, ws, ts, norm_w, eps, res, ldr, y, ldy, N, K, st, push);
  return launch_nvfp4<M, 2, EPI>(x, ldx, wq, ws, ts, norm_w, eps, res, ldr, y, ldy, N, K, st, push);
}

template <int EPI>
cudaError_t dispatch_m(int M, const bf16* x, int ldx, const uint8_t* wq, const uint8_t* ws,
                       const float* ts, const float* norm_w, float eps, const bf16* res, int ldr,
                       void* y, int ldy, int N, int K, cudaStream_t st, const TrlPushArgs& push = TrlPushArgs()) {
  switch (M) {
    case 1: return dispatch_r<1, EPI>(x, ldx, wq, ws, ts, norm_w, eps, res, ldr, y, ldy, N, K, st, push);
    case 2: return dispatch_r<2, EPI>(x, ldx, wq, ws, ts, norm_w, eps, res, ldr, y, ldy, N, K, st, push);
    case 3: return dispatch_r<3, EPI>(x, ldx, wq, ws, ts, norm_w, eps, res, ldr, y, ldy, N, K, st, push);
    case 4: return dispatch_r<4, EPI>(x, ldx, wq, ws, ts, norm_w, eps, res, ldr, y, ldy, N, K, st, push);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

// y: bf16 (or fp32 for EPI_STORE_F32).  M up to 4 per pass; larger M is looped.
// K must be a multiple of 32 and M*K*2 bytes must fit in shared memory (<= ~190 KB).
TRL_API int trl_gemv_nvfp4(const void* x, int ldx, const void* wq, const void* wscale, const void* tscale,
                           const void* norm_w, float eps, const void* residual, int ldr, void* y, int ldy,
                           int M, int N, int K, int epi, void* stream) {
  if (K % 32 != 0 || N <= 0 || M <= 0) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t ysz = (epi == EPI_STORE_F32) ? 4 : 2;
  int per = 4;
  while (per > 1 && (size_t)per * K * 2 > 190 * 1024) --per;
  for (int m0 = 0; m0 < M; m0 += per) {
    const int mm = min(per, M - m0);
    const bf16* xp = (const bf16*)x + (size_t)m0 * ldx;
    const bf16* rp = residual ? (const bf16*)residual + (size_t)m0 * ldr : nullptr;
    void* yp = (char*)y + (size_t)m0 * ldy * ysz;
    cudaError_t e;
    switch (epi) {
      case EPI_STORE: e = dispatch_m<EPI_STORE>(mm, xp, ldx, (const uint8_t*)wq, (const uint8_t*)wscale, (const float*)tscale, (const float*)norm_w, eps, rp, ldr, yp, ldy, N, K, st); break;
      case EPI_RESIDUAL: e = dispatch_m<EPI_RESIDUAL>(mm, xp, ldx, (const uint8_t*)wq, (const uint8_t*)wscale, (const float*)tscale, (const float*)norm_w, eps, rp, ldr, yp, ldy, N, K, st); break;
      case EPI_SWIGLU: e = dispatch_m<EPI_SWIGLU>(mm, xp, ldx, (const uint8_t*)wq, (const uint8_t*)wscale, (const float*)tscale, (const float*)norm_w, eps, rp, ldr, yp, ldy, N, K, st); break;
      case EPI_STORE_F32: e = dispatch_m<EPI_STORE_F32>(mm, xp, ldx, (const uint8_t*)wq, (const uint8_t*)wscale, (const float*)tscale, (const float*)norm_w, eps, rp, ldr, yp, ldy, N, K, st); break;
      default: return (int)cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

TRL_API int trl_gemv_bf16(const void* x, int ldx, const void* w, const void* norm_w, float eps,
                          const void* residual, int ldr, void* y, int ldy, int M, int N, int K, int epi,
                          void* stream) {
  if (K % 8 != 0 || N <= 0 || M <= 0) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t ysz = (epi == EPI_STORE_F32) ? 4 : 2;
  if (M > 2 && M <= 16 && K % 32 == 0 && (epi == EPI_STORE || epi == EPI_STORE_F32 || epi == EPI_RESIDUAL)) {
    // 3..16 rows: one pass over the weights on the tensor cores, if the activation rows fit shared memory
    // (measured on the 248 320 x 5120 head: 4 rows 762 us with the FMA kernel below, 8 rows 421 us here)
    const int nt = M <= 8 ? 1 : 2;
    const size_t smem = (size_t)nt * 8 * (K + BM_PAD) * sizeof(bf16);
    if (smem <= 200 * 1024) {
      const int grid = min(num_sms(), (N + 16 * (BM_THREADS / 32) - 1) / (16 * (BM_THREADS / 32)));
      cudaError_t e = cudaErrorInvalidValue;
#define BM_CASE(NTT, EP)                                                                           \
  if (nt == NTT && epi == EP) {                                                                    \
    auto kern = gemv_bf16_mma_kernel<NTT, EP>;                                                     \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
    e = trl_launch(kern, dim3(grid), dim3(BM_THREADS), smem, st, (const bf16*)x, ldx, (const bf16*)w, \
                   (const float*)norm_w, eps, (const bf16*)residual, ldr, y, ldy, M, N, K);        \
  }
      BM_CASE(1, EPI_STORE) BM_CASE(1, EPI_STORE_F32) BM_CASE(1, EPI_RESIDUAL)
      BM_CASE(2, EPI_STORE) BM_CASE(2, EPI_STORE_F32) BM_CASE(2, EPI_RESIDUAL)
#undef BM_CASE
      return (int)e;
    }
  }
  int per = 4;
  while (per > 1 && (size_t)per * K * 4 > 190 * 1024) --per;
  for (int m0 = 0; m0 < M; m0 += per) {
    const int mm = min(per, M - m0);
    const bf16* xp = (const bf16*)x + (size_t)m0 * ldx;
    const bf16* rp = residual ? (const bf16*)residual + (size_t)m0 * ldr : nullptr;
    void* yp = (char*)y + (size_t)m0 * ldy * ysz;
    const size_t smem = (size_t)mm * K * 4 + 32 * 4;
    const int grid = min(num_sms(), (N / 2 + GEMV_THREADS / 32 - 1) / (GEMV_THREADS / 32) + 1);
    cudaError_t e = cudaErrorInvalidValue;
#define BF16_CASE(MM, EP)                                                                          \
  if (mm == MM && epi == EP) {                                                                     \
    auto kern = gemv_bf16_kernel<MM, 2, EP>;                                                       \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
    e = trl_launch(kern, dim3(grid), dim3(GEMV_THREADS), smem, st, xp, ldx, (const bf16*)w,        \
                   (const float*)norm_w, eps, rp, ldr, yp, ldy, N, K);                             \
  }
    BF16_CASE(1, EPI_STORE) BF16_CASE(2, EPI_STORE) BF16_CASE(3, EPI_STORE) BF16_CASE(4, EPI_STORE)
    BF16_CASE(1, EPI_STORE_F32) BF16_CASE(2, EPI_STORE_F32) BF16_CASE(3, EPI_STORE_F32) BF16_CASE(4, EPI_STORE_F32)
    BF16_CASE(1, EPI_RESIDUAL) BF16_CASE(2, EPI_RESIDUAL) BF16_CASE(3, EPI_RESIDUAL) BF16_CASE(4, EPI_RESIDUAL)
#undef BF16_CASE
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

TRL_API void trl_set_pdl(int on) { g_trl_use_pdl = on; }

TRL_API int trl_error_read(int* out4, int clear) {
  TrlError h;
  cudaError_t e = cudaMemcpyFromSymbol(&h, g_trl_error, sizeof(h));
  if (e != cudaSuccess) return (int)e;
  out4[0] = h.code, out4[1] = h.a, out4[2] = h.b, out4[3] = h.c;
  if (clear && h.code != 0) {
    TrlError z = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_trl_error, &z, sizeof(z));
  }
  return 0;
}

// Row-parallel GEMV whose epilogue pushes fp32 partial rows into every rank's one-shot
// all-reduce slot (see comm.cu); trl_allreduce_finish completes the sum on each rank.
TRL_API int trl_gemv_nvfp4_push(const void* x, int ldx, const void* wq, const void* wscale, const void* tscale,
                                void* const* ws, int rank, int world, int hmax, int M, int N, int K, void* stream) {
  if (K % 32 != 0 || N <= 0 || M <= 0 || M > 8 || N > hmax) return (int)cudaErrorInvalidValue;
  int per = 4;
  while (per > 1 && (size_t)per * K * 2 > 190 * 1024) --per;
  for (int m0 = 0; m0 < M; m0 += per) {
    const int mm = min(per, M - m0);
    TrlPushArgs push;
    for (int i = 0; i < 8; ++i) push.ws[i] = i < world ? (unsigned char*)ws[i] : nullptr;
    push.rank = rank, push.world = world, push.hmax = hmax, push.row0 = m0;
    const int last = (m0 + mm >= M) ? 1 : 0;
    cudaError_t e = dispatch_m<EPI_PUSH>(mm, (const bf16*)x + (size_t)m0 * ldx, ldx, (const uint8_t*)wq,
                                         (const uint8_t*)wscale, (const float*)tscale, nullptr, 0.f, nullptr, 0,
                                         nullptr, last, N, K, (cudaStream_t)stream, push);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

// Timeline records of the launches since the last reset (builds with -DTRL_TRACE; otherwise
// returns 0 records).  out: n x 16 uint64 {kind, entry, dependency wait done, exit, mark 0, mark 1,
// latest exit of any CTA of the launches before, unused, marks 2..9} in ns.
TRL_API int trl_trace_read(void* out, int cap, int reset) {
#ifdef TRL_TRACE
  unsigned int n = 0;
  if (cudaMemcpyFromSymbol(&n, g_trl_trace_n, sizeof(n)) != cudaSuccess) return -1;
  if ((int)n > cap) n = cap;
  if (n > TRL_TRACE_CAP) n = TRL_TRACE_CAP;
  if (n && cudaMemcpyFromSymbol(out, g_trl_trace, (size_t)n * sizeof(TrlTraceRec)) != cudaSuccess) return -1;
  if (reset) {
    const unsigned int z = 0;
    cudaMemcpyToSymbol(g_trl_trace_n, &z, sizeof(z));
  }
  return (int)n;
#else
  (void)out, (void)cap, (void)reset;
  return 0;
#endif
}
