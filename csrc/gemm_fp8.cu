// Block-scaled FP8 GEMM on tcgen05 (kind::f8f6f4) and the FP8 weight-streaming GEMV.
//
//   Y[tok, n] = epi( sum_kb  ws[n/128, kb] * as[tok, kb] * sum_{k in kb} X8[tok, k] * W8[n, k] )
//
// W8: e4m3 [N, K] with one fp32 scale per 128 x 128 block (the FP8 checkpoint format);
// X8: e4m3 [T, K] with one fp32 scale per (token, 128 consecutive k), produced by
// quant_act_fp8_kernel (optional RMSNorm / SwiGLU folded in).  K % 128 == 0.
//
// The tensor core multiplies raw e4m3 and accumulates in fp32, but the scales change every 128
// k, so one k-block (4 MMAs of K = 32) is accumulated into a fresh TMEM tile and then *promoted*:
// the eight epilogue warps read the tile from TMEM, multiply by ws * as and add into fp32
// registers, while the MMA warp already fills the second TMEM tile with the next k-block (two
// accumulator tiles ping-pong).  The weight is the MMA "A" operand (128 rows -> TMEM lanes, one
// epilogue thread per output feature), 128 tokens are the "B" operand (TMEM columns).
//
// Warp roles (320 threads): warp 0 = TMA producer (both operands, 128B-swizzled boxes of
// 128 rows x 128 bytes, no cluster multicast), warp 1 = TMEM owner + MMA issuer, warps 2-9 =
// promotion + epilogue (two warps per TMEM lane quadrant, 64 token columns each).  Every mbarrier wait is bounded (error word, abort flag, TMEM freed).
//
// Reference parity: `linear_fp8` (DeepGEMM-style 2x accumulation on WGMMA),
// `linear_fp8_gemv` and `quant_fp8` of
// packages/tilerl-kernels/src/tilerl_kernels/kernels_linear.py:1777-1813, :1442-1494, :1547-1590;
// the reference quantises activations per token, here per 1 x 128 block.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int F8_TILE = 128;          // output features per tile (TMEM lanes)
constexpr int F8_BN = 128;            // tokens per tile (TMEM columns)
constexpr int F8_KB = 128;            // k per block = bytes per operand row per stage
constexpr int F8_THREADS = 320;          // 2 role warps + 8 promotion / epilogue warps
constexpr int F8_EPI_THREADS = F8_THREADS - 64;
constexpr int F8_COLS = F8_BN / 2;        // token columns per epilogue thread (two warps share a TMEM lane quadrant)
constexpr int F8_STAGES = 6;
constexpr int F8_STAGE_BYTES = 2 * F8_TILE * F8_KB;   // A + B tile
enum { F8_EPI_STORE = 0, F8_EPI_RESIDUAL = 1, F8_EPI_SWIGLU = 2, F8_EPI_STORE_F32 = 3 };

struct Fp8Params {
  const float* ws;       // [ceil(N/128), K/128]
  const float* as;       // [T, K/128]
  const bf16* residual;
  void* out;
  int N, K, T, nkb;
  int ldr, ldo, epi;
  int n_tiles, t_tiles;
};

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                const Fp8Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)F8_STAGES * F8_STAGE_BYTES);
  // bars: [0,S) full, [S,2S) empty, 2S+{0,1} accum_full, 2S+{2,3} accum_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * F8_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* sc_s = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + 256);   // [2][F8_BN] ws * as of a k-block

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (F8_STAGES + s); };
  auto acc_full = [&](int b) { return bar0 + 8u * (2 * F8_STAGES + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * (2 * F8_STAGES + 2 + b); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) mbar_init(full(s), 1), mbar_init(empty(s), 1);
    for (int b = 0; b < 2; ++b) mbar_init(acc_full(b), 1), mbar_init(acc_empty(b), F8_EPI_THREADS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  const int n_work = p.n_tiles * p.t_tiles;
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int st = 0;
      uint32_t ph = 0;
      long issued = 0;
      bool ok = true;
      bool waited = false;
      for (int tile = blockIdx.x; ok && tile < n_work; tile += gridDim.x) {
        const int nt = tile / p.t_tiles, tt = tile % p.t_tiles;
        for (int kb = 0; ok && kb < p.nkb; ++kb, ++issued) {
          if (issued >= F8_STAGES) {
            ok = mbar_wait(empty(st), ph ^ 1u, abort_flag);
            if (!ok) break;
          }
          const uint32_t dst = smem_u32(smem) + (uint32_t)st * F8_STAGE_BYTES;
          mbar_expect_tx(full(st), F8_STAGE_BYTES);
          tma_load_2d(dst, &map_w, kb * F8_KB, nt * F8_TILE, full(st));       // weights: independent of earlier kernels
          if (!waited) {                                                          // activations: after the quantiser
            pdl_wait();
            waited = true;
          }
          tma_load_2d(dst + F8_TILE * F8_KB, &map_x, kb * F8_KB, tt * F8_BN, full(st));
          if (++st == F8_STAGES) st = 0, ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    pdl_wait();
    if (lane == 0) {
      // dense f8f6f4: fp32 accumulator, e4m3 x e4m3, both K-major, N = F8_BN, M = 128
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(F8_BN >> 3) << 17) | ((uint32_t)(F8_TILE >> 4) << 24);
      const uint64_t d0 = desc_sw128(smem_u32(smem));
      const uint32_t lo0 = (uint32_t)d0, hi = (uint32_t)(d0 >> 32);
      int st = 0;
      uint32_t ph = 0;
      long blk = 0;                 // running k-block count: accumulator buffer = blk & 1
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_work; tile += gridDim.x) {
        for (int kb = 0; ok && kb < p.nkb; ++kb, ++blk) {
          const int buf = (int)(blk & 1);
          if (blk >= 2) {
            ok = mbar_wait(acc_empty(buf), (uint32_t)((blk >> 1) - 1) & 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
          }
          ok = mbar_wait(full(st), ph, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t aoff = (uint32_t)st * (uint32_t)(F8_STAGE_BYTES >> 4);
          const uint32_t boff = aoff + (uint32_t)((F8_TILE * F8_KB) >> 4);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            tc_mma_f8_lh(tmem_base + (uint32_t)buf * F8_BN, lo0 + aoff + i * 2, lo0 + boff + i * 2, hi, idesc, i ? 1u : 0u);
          tc_commit(empty(st));
          tc_commit(acc_full(buf));
          if (++st == F8_STAGES) st = 0, ph ^= 1u;
        }
      }
    }
  } else {
    // ---------------- promotion + epilogue (warps 2..9) ----------------
    pdl_wait();
    const int quad = warp & 3;                 // a warp may read only the TMEM lanes of its quadrant
    const int half = (warp - 2) >> 2;          // which 64 token columns of the tile
    const int row = quad * 32 + lane;         // TMEM lane = output feature within the tile
    const int e = (int)threadIdx.x - 64;      // 0..255 among the epilogue threads
    long blk = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_work; tile += gridDim.x) {
      const int nt = tile / p.t_tiles, tt = tile % p.t_tiles;
      const int n = nt * F8_TILE + row;
      const int tok0 = tt * F8_BN;
      float acc[F8_COLS];
#pragma unroll
      for (int c = 0; c < F8_COLS; ++c) acc[c] = 0.f;
      // ws (one value per tile and k-block) * as[token, k-block], fetched by the first 128 threads
      auto load_scale = [&](int kb) -> float {
        const int tok = tok0 + e;
        if (e >= F8_BN || kb >= p.nkb || tok >= p.T) return 0.f;
        return __ldcg(p.as + (size_t)tok * p.nkb + kb) * p.ws[(size_t)nt * p.nkb + kb];
      };
      float a_cur = load_scale(0), a_nxt = load_scale(1);
      for (int kb = 0; ok && kb < p.nkb; ++kb, ++blk) {
        const int buf = (int)(blk & 1);
        // scale of this k-block for every token column: ws (one value for the tile) * as[token]
        if (e < F8_BN) {
          sc_s[buf * F8_BN + e] = a_cur;
          a_cur = a_nxt;                        // the loads run two k-blocks ahead of their use
          a_nxt = load_scale(kb + 2);
        }
        ok = mbar_wait(acc_full(buf), (uint32_t)(blk >> 1) & 1u, abort_flag);
        {
          uint32_t all;   // one decision for the four warps; also publishes sc_s
          asm volatile(
              "{ .reg .pred p, q;\n"
              "  setp.ne.u32 q, %1, 0;\n"
              "  bar.red.and.pred p, 1, 256, q;\n"
              "  selp.u32 %0, 1, 0, p; }\n"
              : "=r"(all) : "r"((uint32_t)ok) : "memory");
          ok = all != 0;
        }
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * F8_BN + half * F8_COLS);
        const float* sc = sc_s + buf * F8_BN + half * F8_COLS;
        {
          uint32_t r[F8_COLS];     // both 32-column reads in flight before the one wait
          tc_ld32(taddr, *reinterpret_cast<uint32_t(*)[32]>(r));
          tc_ld32(taddr + 32u, *reinterpret_cast<uint32_t(*)[32]>(r + 32));
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < F8_COLS; c += 4) {
            const float4 s4 = *reinterpret_cast<const float4*>(sc + c);
            acc[c + 0] = fmaf(__uint_as_float(r[c + 0]), s4.x, acc[c + 0]);
            acc[c + 1] = fmaf(__uint_as_float(r[c + 1]), s4.y, acc[c + 1]);
            acc[c + 2] = fmaf(__uint_as_float(r[c + 2]), s4.z, acc[c + 2]);
            acc[c + 3] = fmaf(__uint_as_float(r[c + 3]), s4.w, acc[c + 3]);
          }
        }
        tc_fence_before();
        mbar_arrive(acc_empty(buf));
      }
      if (!ok) break;
      // epilogue of the tile: thread `row` holds feature n for the tile's 128 tokens
#pragma unroll
      for (int c = 0; c < F8_COLS; ++c) {   // fully unrolled: acc[] stays in registers
        const int tok = tok0 + half * F8_COLS + c;
        float v = acc[c];
        if (p.epi == F8_EPI_SWIGLU) {
          const float other = __shfl_xor_sync(0xffffffffu, v, 1);
          const float y = __fdividef(v, 1.f + __expf(-v)) * other;
          if ((lane & 1) == 0 && tok < p.T && n + 1 < p.N)
            reinterpret_cast<bf16*>(p.out)[(size_t)tok * p.ldo + (n >> 1)] = __float2bfloat16(y);
        } else if (tok < p.T && n < p.N) {
          if (p.epi == F8_EPI_RESIDUAL) v += __bfloat162float(__ldcg(p.residual + (size_t)tok * p.ldr + n));
          if (p.epi == F8_EPI_STORE_F32)
            reinterpret_cast<float*>(p.out)[(size_t)tok * p.ldo + n] = v;
          else
            reinterpret_cast<bf16*>(p.out)[(size_t)tok * p.ldo + n] = __float2bfloat16(v);
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    const long long t0 = clock64();   // copies still in flight must land before the CTA's memory goes away
    while (clock64() - t0 < 2000000LL) {
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
  }
}


// ---------------------------------------------------------------------------------------
// Activation quantiser: optional RMSNorm (or SwiGLU of an interleaved gate/up row), then e4m3
// with one fp32 scale per (token, 128 consecutive k): scale = amax / 448.  One CTA per token,
// one warp per 128-block at a time (4 elements per lane).
__global__ void __launch_bounds__(256)
quant_act_fp8_kernel(const bf16* x, int ldx, const float* __restrict__ norm_w, float eps, uint8_t* x8, float* as,
                     int K, int swiglu_in) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x;
  const bf16* xr = x + (size_t)tok * ldx;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  auto load4 = [&](int k, float (&v)[4]) {
    if (swiglu_in) {   // interleaved (gate, up) pairs: K outputs from 2K inputs
      const uint4 u = __ldcg(reinterpret_cast<const uint4*>(xr + 2 * k));
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 gu = bf162_bits_to_f2(w[i]);
        v[i] = __bfloat162float(__float2bfloat16(silu_f(gu.x) * gu.y));
      }
    } else {
      const uint2 u = __ldcg(reinterpret_cast<const uint2*>(xr + k));
      const float2 a = bf162_bits_to_f2(u.x), b = bf162_bits_to_f2(u.y);
      v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
    }
  };
  float rstd = 1.f;
  if (norm_w != nullptr) {
    float ss = 0.f;
    for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
      float v[4];
      load4(k, v);
      ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    }
    ss = block_sum(ss, red);
    rstd = rsqrtf(ss / (float)K + eps);
  }
  const int nkb = K >> 7;
  for (int kb = warp; kb < nkb; kb += nw) {
    const int k = kb * 128 + lane * 4;
    float v[4];
    load4(k, v);
    if (norm_w != nullptr) {
      const float4 w = *reinterpret_cast<const float4*>(norm_w + k);
      v[0] = __bfloat162float(__float2bfloat16(v[0] * rstd * w.x));
      v[1] = __bfloat162float(__float2bfloat16(v[1] * rstd * w.y));
      v[2] = __bfloat162float(__float2bfloat16(v[2] * rstd * w.z));
      v[3] = __bfloat162float(__float2bfloat16(v[3] * rstd * w.w));
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const float sc = fmaxf(amax, 1e-30f) * (1.f / 448.f);
    const float inv = __frcp_rn(sc);
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(v[1] * inv), "f"(v[0] * inv));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(v[3] * inv), "f"(v[2] * inv));
    *reinterpret_cast<uint32_t*>(x8 + (size_t)tok * K + k) = (uint32_t)lo | ((uint32_t)hi << 16);
    if (lane == 0) as[(size_t)tok * nkb + kb] = sc;
  }
}

// ---------------------------------------------------------------------------------------
// FP8 weight-streaming GEMV for M <= 4 rows: e4m3 [N, K] rows streamed with 128-bit loads (16
// weights per lane and step), converted two at a time to f16x2 (e4m3 is exact in f16) and
// multiplied with the activation held as f16x2 in shared memory (optional RMSNorm in the
// prologue; values clamped to the f16 range).  The 16 products of a lane are summed in f16x2,
// everything above that (the 8 lanes of a 128-k block, the block scale, the blocks) in fp32.
constexpr int GV8_THREADS = 512;
template <int M, int EPI>
__global__ void __launch_bounds__(GV8_THREADS, 2)
gemv_fp8_kernel(const bf16* x, int ldx, const uint8_t* __restrict__ w8, const float* __restrict__ ws,
                const float* __restrict__ norm_w, float eps, const bf16* residual, int ldr, void* yout,
                int ldy, int N, int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);                       // [M][K]
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)M * K * 2);
  pdl_launch_dependents();
  pdl_wait();
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const bf16* xr = x + (size_t)m * ldx;
    float rstd = 1.f;
    if (norm_w != nullptr) {
      float ss = 0.f;
      for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = __bfloat162float(__ldcg(xr + k));
        ss += v * v;
      }
      ss = block_sum(ss, red);
      rstd = rsqrtf(ss / (float)K + eps);
    }
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      float v = __bfloat162float(__ldcg(xr + k));
      if (norm_w != nullptr) v = __bfloat162float(__float2bfloat16(v * rstd * norm_w[k]));
      xs[(size_t)m * K + k] = __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (GV8_THREADS / 32) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (GV8_THREADS / 32);
  const int nkb = K >> 7;
  for (int n = warp; n < N; n += nwarps) {
    const uint8_t* wr = w8 + (size_t)n * K;
    const float* sr = ws + (size_t)(n >> 7) * nkb;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    // a lane owns 16 consecutive k of every 512: 8 lanes cover one 128-k scale block.  Four steps
    // (2048 k) of loads are issued before the first is used.
    for (int k0 = 0; k0 < K; k0 += 2048) {
      uint4 wv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + u * 512 + lane * 16;
        wv[u] = k < K ? ldg_stream_16(wr + k) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + u * 512 + lane * 16;
        if (k0 + u * 512 >= K) break;
        float part[M];
#pragma unroll
        for (int m = 0; m < M; ++m) part[m] = 0.f;
        if (k < K) {
          const uint32_t w4[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
          uint32_t wh[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            wh[2 * i] = cvt_e4m3x2_to_h2((uint16_t)(w4[i] & 0xFFFFu));
            wh[2 * i + 1] = cvt_e4m3x2_to_h2((uint16_t)(w4[i] >> 16));
          }
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)m * K + k);
            const uint4 xa = xp[0], xb = xp[1];
            uint32_t s0 = 0u, s1 = 0u;     // two chains of four
            s0 = hfma2_u(wh[0], xa.x, s0), s1 = hfma2_u(wh[1], xa.y, s1);
            s0 = hfma2_u(wh[2], xa.z, s0), s1 = hfma2_u(wh[3], xa.w, s1);
            s0 = hfma2_u(wh[4], xb.x, s0), s1 = hfma2_u(wh[5], xb.y, s1);
            s0 = hfma2_u(wh[6], xb.z, s0), s1 = hfma2_u(wh[7], xb.w, s1);
            const float2 f0 = h2_to_f2(s0), f1 = h2_to_f2(s1);
            part[m] = (f0.x + f0.y) + (f1.x + f1.y);
          }
        }
        // the 8 lanes of a 128-k block sum their pieces, then the block scale is applied once
        const int kb = ((k0 + u * 512) >> 7) + (lane >> 3);
        const float bs = ((lane & 7) == 0 && kb < nkb) ? sr[kb] : 0.f;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float sum = part[m];
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          sum += __shfl_xor_sync(0xffffffffu, sum, 4);
          acc[m] = fmaf(sum, bs, acc[m]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = acc[m];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      if (lane == 0) {
        if (EPI == F8_EPI_RESIDUAL) v += __bfloat162float(__ldcg(residual + (size_t)m * ldr + n));
        if (EPI == F8_EPI_STORE_F32) reinterpret_cast<float*>(yout)[(size_t)m * ldy + n] = v;
        else reinterpret_cast<bf16*>(yout)[(size_t)m * ldy + n] = __float2bfloat16(v);
      }
    }
  }
}

typedef CUresult (*EncodeTiledFn8)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn8 g_encode8 = nullptr;

// [rows, row_bytes] bytes, box = 128 bytes x 128 rows, 128B swizzle; rows beyond the tensor read as zero
int make_map8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t row_bytes) {
  if (!g_encode8) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return 1;
    g_encode8 = (EncodeTiledFn8)fn;
  }
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)F8_KB, (cuuint32_t)F8_TILE};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode8(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

}  // namespace

// x [T, K] bf16 (or [T, 2K] interleaved gate/up when swiglu_in) -> x8 [T, K] e4m3, as [T, K/128] fp32.
TRL_API int trl_quant_act_fp8(const void* x, int ldx, const void* norm_w, float eps, void* x8, void* as, int T, int K,
                              int swiglu_in, void* stream) {
  if (K % 128 != 0 || T <= 0) return (int)cudaErrorInvalidValue;
  return (int)trl_launch(quant_act_fp8_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x, ldx,
                         (const float*)norm_w, eps, (uint8_t*)x8, (float*)as, K, swiglu_in);
}

// out[tok, n] = epi(block-scaled x8 @ w8^T).  w8 [N, K] e4m3, ws [ceil(N/128), K/128] fp32; x8 / as from
// trl_quant_act_fp8.  K % 128 == 0; the activation buffer must hold whole 16-byte rows (K % 16 == 0).
TRL_API int trl_gemm_fp8(const void* w8, const void* ws, const void* x8, const void* as, const void* residual, int ldr,
                         void* out, int ldo, int T, int N, int K, int epi, void* stream) {
  if (K % 128 != 0 || T <= 0 || N <= 0 || epi < 0 || epi > 3) return (int)cudaErrorInvalidValue;
  CUtensorMap mw, mx;
  if (make_map8(&mw, w8, (uint64_t)N, (uint64_t)K) || make_map8(&mx, x8, (uint64_t)T, (uint64_t)K))
    return (int)cudaErrorInvalidValue;
  Fp8Params p;
  p.ws = (const float*)ws, p.as = (const float*)as, p.residual = (const bf16*)residual, p.out = out;
  p.N = N, p.K = K, p.T = T, p.nkb = K / 128, p.ldr = ldr, p.ldo = ldo, p.epi = epi;
  p.n_tiles = (N + F8_TILE - 1) / F8_TILE, p.t_tiles = (T + F8_BN - 1) / F8_BN;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = min(sms, p.n_tiles * p.t_tiles);
  const int smem = F8_STAGES * F8_STAGE_BYTES + 1024 + 256 + 2 * F8_BN * 4 + 64;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return 3;
    configured = true;
  }
  return (int)trl_launch(gemm_fp8_kernel, dim3(grid), dim3(F8_THREADS), (size_t)smem, (cudaStream_t)stream, mw, mx, p);
}

// y = epi(norm(x) @ dequant(W8)^T) for M <= 8 rows (looped 4 at a time).  epi: 0 store, 1 + residual, 3 fp32 store.
TRL_API int trl_gemv_fp8(const void* x, int ldx, const void* w8, const void* ws, const void* norm_w, float eps,
                         const void* residual, int ldr, void* y, int ldy, int M, int N, int K, int epi, void* stream) {
  if (K % 128 != 0 || N <= 0 || M <= 0 || (epi != 0 && epi != 1 && epi != 3)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t ysz = epi == 3 ? 4 : 2;
  int per = 4;
  while (per > 1 && (size_t)per * K * 2 > 180 * 1024) --per;
  for (int m0 = 0; m0 < M; m0 += per) {
    const int mm = min(per, M - m0);
    const bf16* xp = (const bf16*)x + (size_t)m0 * ldx;
    const bf16* rp = residual ? (const bf16*)residual + (size_t)m0 * ldr : nullptr;
    void* yp = (char*)y + (size_t)m0 * ldy * ysz;
    const size_t smem = (size_t)mm * K * 2 + 32 * 4;
    const int per_sm = smem <= 100 * 1024 ? 2 : 1;
    const int grid = min(per_sm * sms, (N + GV8_THREADS / 32 - 1) / (GV8_THREADS / 32));
    cudaError_t e = cudaErrorInvalidValue;
#define GV8_CASE(MM, EP)                                                                                    \
  if (mm == MM && epi == EP) {                                                                              \
    auto kern = gemv_fp8_kernel<MM, EP>;                                                                    \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);                    \
    e = trl_launch(kern, dim3(grid), dim3(GV8_THREADS), smem, st, xp, ldx, (const uint8_t*)w8,              \
                   (const float*)ws, (const float*)norm_w, eps, rp, ldr, yp, ldy, N, K);                    \
  }
    GV8_CASE(1, 0) GV8_CASE(2, 0) GV8_CASE(3, 0) GV8_CASE(4, 0)
    GV8_CASE(1, 1) GV8_CASE(2, 1) GV8_CASE(3, 1) GV8_CASE(4, 1)
    GV8_CASE(1, 3) GV8_CASE(2, 3) GV8_CASE(3, 3) GV8_CASE(4, 3)
#undef GV8_CASE
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
