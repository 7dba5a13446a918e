// Streamed NVFP4 GEMV for the decode tick (M <= 2 rows): the weights arrive through a
// shared-memory ring filled by bulk asynchronous copies, so that
//
//   * the first ring fill is issued BEFORE griddepcontrol.wait -- weights do not depend on
//     the previous kernel -- and DRAM keeps streaming while the predecessor drains and
//     while this kernel stages its activation row;
//   * the bytes in flight per SM (CTAs x 8 warps x NS stages of 2304 B) do not cost
//     registers: the kernel runs at <= 80 registers and 256 threads, three CTAs fit on an
//     SM, and a grid of two CTAs per SM leaves the third slot to the NEXT kernel of the
//     stream, whose CTAs start under programmatic dependent launch, fill their rings and
//     wait.  The fixed cost between two projections of a tick (launch, prologue, first-byte
//     latency, tail) then overlaps with the neighbours instead of adding to them.
//
// The kernel reads a *stream layout* copy of the weight (built once per weight by
// trl_gemv_stream_pack): rows are taken in pairs and K in steps of 32 chunks of 32
// weights; one unit = (row pair, step) holds
//     [n x 16 B row 0][n x 16 B row 1][n x 2 B scales row 0][n x 2 B scales row 1]
// (n = 32 chunks, fewer in the last step of a row), units of a pair and pairs follow each
// other without gaps.  A CTA owns a contiguous block of row pairs and its warps split the
// block's units evenly (the balanced split of gemv_nvfp4_sk_kernel), so every warp streams
// ONE contiguous byte range, two units (2304 B) per bulk copy: measured on a B200, copies of
// 1152 B reach 4-5 TB/s of HBM reads, 2304 B and more reach 6 TB/s.
//
// Tensor parallelism.  A row-parallel projection pushes its fp32 partial rows into every rank's
// one-shot slots (EPI2_PUSH, protocol of comm.cu).  The projection that consumes the reduced
// residual stream finishes the all-reduce in ITS prologue (COOP): after the dependency wait every
// CTA sums a small slice of the row from the slots of all ranks (bounded polls of the epoch half
// of each word), adds the residual and stores the slice; one arrival counter plus a release word
// in the workspace form a grid barrier, after which every CTA stages the whole row as usual.  No
// separate finishing launch sits between the two projections.
//
// Arithmetic is that of gemv.cu: e2m1 -> f16x2 by the native cvt, f16x2 FMA inside a
// 16-element scale block, fp32 across blocks, per-row power-of-two activation scale.
//
// Reference parity: `linear_fp4_gemv` of
// packages/tilerl-kernels/src/tilerl_kernels/kernels_linear.py:924-978 (register-streamed,
// twiddled layout); the ring, the layout and the overlap with the neighbouring kernels have
// no counterpart there.
#include <stdlib.h>

#include "common.cuh"

enum { EPI2_STORE = 0, EPI2_RESIDUAL = 1, EPI2_SWIGLU = 2, EPI2_STORE_F32 = 3, EPI2_PUSH = 4 };

// One projection of a chained launch (trl_gemv2_chain), as the host passes it.
struct TrlChainOp {
  const void* x;          // [M, K] bf16 activation rows (for coop = 1: the residual stream, updated in place)
  const void* wst;        // stream layout of the [N, K] NVFP4 weight
  const void* tscale;
  const void* norm_w;     // fp32 [K] or null
  const void* residual;   // EPI2_RESIDUAL: [M, N] bf16
  void* out;
  int ldx, ldr, ldy, N, K, epi, coop;
  float eps;
};

namespace {

constexpr int G2_THREADS = 256;
constexpr int G2_WARPS = G2_THREADS / 32;
constexpr int G2_MAX_NS = 8;
constexpr int UNIT_BYTES = 1152;              // full unit: 32 chunks x (16 + 16 + 2 + 2) bytes
constexpr int STAGE_UNITS = 2;                // units per bulk copy / ring stage
constexpr int STAGE_BYTES = STAGE_UNITS * UNIT_BYTES;
constexpr long long G2_WAIT_CYCLES = 4000000000LL;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void g2_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void g2_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t g2_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p;\n"
      "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "  selp.u32 %0, 1, 0, p; }\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ void g2_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ uint4 g2_lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint16_t g2_lds16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}

// x (bf16 [M, K], optional RMSNorm weight) -> shared memory as f16.  Piece p (8 halves) of
// 32-element chunk c sits at ((p * nchunks + c) * 8) halves: the four 16-byte reads of a chunk are
// conflict-free across lanes.  One pass: a thread holds up to XV 8-element vectors of the row.
constexpr int G2_XV = 9;   // K <= 9 * 256 * 8 = 18432
// The activation row is staged as f16 (x * norm weight * 2^-4, clamped to the f16 range): no
// reduction sits between the dependency and the first product.  The row's 1 / rms is a scalar and
// multiplies the finished dot product instead (g2_row_scale); its sum of squares is collected here.
constexpr float G2_X_PRESCALE = 0.0625f;
template <int M>
__device__ __forceinline__ void g2_stage_x(const bf16* __restrict__ x, int ldx, int K,
                                           const float* __restrict__ norm_w, __half* xs, float* red) {
  const int nchunks = K >> 5, nvec = K >> 3;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const bf16* xr = x + (size_t)m * ldx;
    uint4 xv[G2_XV];
#pragma unroll
    for (int i = 0; i < G2_XV; ++i) {
      const int v = threadIdx.x + i * G2_THREADS;
      xv[i] = make_uint4(0u, 0u, 0u, 0u);
      // through L2: under programmatic dependent launch this CTA can share its SM (and L1) with
      // CTAs of earlier kernels that read the previous contents of these rows
      if (v < nvec) xv[i] = __ldcg(reinterpret_cast<const uint4*>(xr + (size_t)v * 8));
    }
    float ss = 0.f;
    __half* dst = xs + (size_t)m * K;
#pragma unroll
    for (int i = 0; i < G2_XV; ++i) {
      const int v = threadIdx.x + i * G2_THREADS;
      if (v < nvec) {
        const uint32_t u4[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
        uint32_t o[4];
        float nw[8];
        if (norm_w != nullptr) {
          const float4 a = *reinterpret_cast<const float4*>(norm_w + (size_t)v * 8);
          const float4 b = *reinterpret_cast<const float4*>(norm_w + (size_t)v * 8 + 4);
          nw[0] = a.x, nw[1] = a.y, nw[2] = a.z, nw[3] = a.w, nw[4] = b.x, nw[5] = b.y, nw[6] = b.z, nw[7] = b.w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = bf162_bits_to_f2(u4[j]);
          if (norm_w != nullptr) {
            ss += f.x * f.x + f.y * f.y;
            f.x *= nw[2 * j], f.y *= nw[2 * j + 1];
          }
          // saturating conversion: values beyond the f16 range become +-65504, never inf
          asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(o[j]) : "f"(f.y * G2_X_PRESCALE), "f"(f.x * G2_X_PRESCALE));
        }
        // vector v = piece (v & 3) of chunk (v >> 2)
        *reinterpret_cast<uint4*>(dst + ((size_t)((v & 3) * nchunks + (v >> 2)) << 3)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[m * G2_WARPS + w] = ss;     // summed by g2_row_scale after the main loop
  }
  __syncthreads();
}

// 1 / rms of activation row m (1 without a norm) times the inverse of the staging prescale.
__device__ __forceinline__ float g2_row_scale(const float* red, int m, int K, bool norm, float eps) {
  float ss = 0.f;
#pragma unroll
  for (int w = 0; w < G2_WARPS; ++w) ss += red[m * G2_WARPS + w];
  return (norm ? rsqrtf(ss / (float)K + eps) : 1.f) * (1.f / G2_X_PRESCALE);
}

// Finish of the one-shot all-reduce inside the consumer (see the header).  Returns false when a
// bounded wait ran out (the error word is set; the caller still runs to completion on whatever
// the row holds, so no barrier of the CTA is skipped).
constexpr size_t G2_OFF_SLOTS = 65536;     // comm.cu: one-shot slots {fp32, epoch} [2][8 src][8 rows][hmax]
constexpr int G2_CTRL_EPOCH = 0, G2_CTRL_ARRIVE = 17, G2_CTRL_RELEASE = 64;   // the polled word has a 128-byte line of its own
__device__ __forceinline__ bool g2_coop_finish(bf16* __restrict__ x, int ldx, int M, int N, unsigned char* ws,
                                               int world, int hmax, int* s_flag) {
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(ws);
  if (threadIdx.x == 0) s_flag[0] = (int)(__ldcg(ctrl + G2_CTRL_EPOCH) + 1u), s_flag[1] = 1;
  __syncthreads();
  const uint32_t epoch = (uint32_t)s_flag[0];
  const int buf = epoch & 1;
  const int total = M * N;
  const int per = (total + (int)gridDim.x - 1) / (int)gridDim.x;
  const int e = (int)blockIdx.x * per + (int)threadIdx.x;
  bool ok = true;
  // threads beyond `per` idle: a CTA's slice is a handful of elements (5120 / 444 = 12)
  for (int i = e; i < min(total, ((int)blockIdx.x + 1) * per); i += G2_THREADS) {
    const int m = i / N, n = i % N;
    float v = __bfloat162float(__ldcg(x + (size_t)m * ldx + n));
    for (int sr = 0; ok && sr < world; ++sr) {
      const uint2* w = reinterpret_cast<const uint2*>(ws + G2_OFF_SLOTS) +
                       ((size_t)(buf * 8 + sr) * 8 + m) * hmax + n;
      uint2 xw = ld_relaxed_sys_v2(w);
      if (xw.y != epoch) {
        const long long t0 = clock64();
        for (uint32_t it = 0; xw.y != epoch; ++it) {
          xw = ld_relaxed_sys_v2(w);
          if ((it & 15) == 15 && clock64() - t0 > G2_WAIT_CYCLES) {
            // a = 5, b = source rank | epoch found in the slot << 8, c = epoch waited for
            trl_set_error(TRL_ERR_WAIT_TIMEOUT, 5, sr | (int)(xw.y << 8), (int)epoch);
            ok = false;
            break;
          }
        }
      }
      v += __uint_as_float(xw.x);
    }
    if (ok) x[(size_t)m * ldx + n] = __float2bfloat16(v);
  }
  if (!ok) s_flag[1] = 0;
  __syncthreads();                         // this CTA's slice is stored
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(ctrl + G2_CTRL_ARRIVE, 1u);
    if (prev == gridDim.x - 1) {           // every CTA has read the epoch and stored its slice
      ctrl[G2_CTRL_ARRIVE] = 0;
      ctrl[G2_CTRL_EPOCH] = epoch;
      __threadfence();
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ctrl + G2_CTRL_RELEASE), "r"(epoch) : "memory");
    } else {
      uint32_t seen;
      const long long t0 = clock64();
      for (uint32_t it = 0;; ++it) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(ctrl + G2_CTRL_RELEASE) : "memory");
        if (seen == epoch) break;
        __nanosleep(32);
        if ((it & 15) == 15 && clock64() - t0 > G2_WAIT_CYCLES) {
          // a = 6, b = arrivals counted so far | CTA << 16, c = epoch waited for
          trl_set_error(TRL_ERR_WAIT_TIMEOUT, 6, (int)(__ldcg(ctrl + G2_CTRL_ARRIVE) | (blockIdx.x << 16)), (int)epoch);
          s_flag[1] = 0;
          break;
        }
      }
    }
  }
  __syncthreads();
  return s_flag[1] != 0;
}

// Warp w of W owns units [w * U / W, (w + 1) * U / W): the owner of `unit` (U * W < 2^31).
__device__ __forceinline__ int g2_owner(int unit, int U, int W) {
  return ((unit + 1) * W - 1) / U;
}

template <int M, int EPI, bool FULL, bool COOP>
__global__ void __launch_bounds__(G2_THREADS, 3)
gemv2_kernel(const bf16* __restrict__ x, int ldx, const uint8_t* __restrict__ wst,
             const float* __restrict__ tscale, const float* __restrict__ norm_w, float eps,
             const bf16* __restrict__ residual, int ldr, void* __restrict__ yout, int ldy, int N, int K,
             int nslot, int NS, const TrlPushArgs push, int trig) {
  constexpr int W = G2_WARPS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // ring [W][NS][STAGE_BYTES] | bars [W][NS] | xs [M][K] f16 | 8 spare floats | red[64] | slots
  unsigned char* ring = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)W * NS * STAGE_BYTES);
  __half* xs = reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(bars) + W * G2_MAX_NS * 8);
  float* xs_inv = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xs) + (size_t)M * K * sizeof(__half));
  float* red = xs_inv + 8;
  float* slots = red + 64;   // [pairs_local][2 rows][nslot][M]

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int npairs = N >> 1;
  const int p_lo = (int)(((long long)blockIdx.x * npairs) / gridDim.x);
  const int p_hi = (int)(((long long)(blockIdx.x + 1) * npairs) / gridDim.x);
  const int pl = p_hi - p_lo;
  const int nchunks = K >> 5;
  const int nsteps = (nchunks + 31) >> 5;
  const int nlast = nchunks - 32 * (nsteps - 1);
  const uint32_t pair_bytes = (uint32_t)nchunks * 36u;
  const int U = pl * nsteps;
  const int u0 = (int)(((long long)warp * U) / W), u1 = (int)(((long long)(warp + 1) * U) / W);

  const uint32_t ring_w = smem_addr(ring + (size_t)warp * NS * STAGE_BYTES);
  const uint32_t bar_w = smem_addr(bars + warp * G2_MAX_NS);
  // producer cursor (lane 0): byte offset of the next unit and its step index
  const uint8_t* src = wst + (size_t)p_lo * pair_bytes;
  uint32_t p_off = (uint32_t)(u0 / nsteps) * pair_bytes + (uint32_t)(u0 % nsteps) * (uint32_t)UNIT_BYTES;
  int p_step = u0 % nsteps, p_unit = u0, p_slot = 0;
  auto issue = [&]() {   // one stage: the next STAGE_UNITS units of this warp's range (fewer at its end)
    uint32_t bytes = 0;
#pragma unroll
    for (int g = 0; g < STAGE_UNITS; ++g) {
      if (p_unit < u1) {
        bytes += (p_step == nsteps - 1) ? (uint32_t)nlast * 36u : (uint32_t)UNIT_BYTES;
        if (++p_step == nsteps) p_step = 0;
        ++p_unit;
      }
    }
    const uint32_t bar = bar_w + 8u * p_slot;
    g2_expect_tx(bar, bytes);
    g2_bulk_load(ring_w + (uint32_t)p_slot * STAGE_BYTES, src + p_off, bytes, bar);
    p_off += bytes;
    if (++p_slot == NS) p_slot = 0;
  };
  if (lane == 0) {
    for (int s = 0; s < NS; ++s) g2_mbar_init(bar_w + 8u * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // first ring fill: independent of the previous kernel
    for (int s = 0; s < NS && p_unit < u1; ++s) issue();
  }
  for (int i = threadIdx.x; i < pl * 2 * nslot * M; i += G2_THREADS) slots[i] = 0.f;
  // the norm weights are a constant parameter: bring this thread's lines into L1 while waiting
  if (norm_w != nullptr) {
#pragma unroll
    for (int i = 0; i < G2_XV; ++i) {
      const int v = threadIdx.x + i * G2_THREADS;
      if (v < (K >> 3)) asm volatile("prefetch.global.L1 [%0];" ::"l"(norm_w + (size_t)v * 8));
    }
  }
  // When the next kernel may come in (trig): 0 = at entry for every kernel; 1 = a kernel with the grid
  // barrier of the cooperative finish lets it in only behind that barrier; 2 = in addition a pushing
  // kernel lets it in only after its pushes.
  const bool late = (COOP && trig >= 1) || (EPI == EPI2_PUSH && trig >= 2);
  pdl_enter(100 + EPI * 2 + (COOP ? 1 : 0));
  if (!late) pdl_trigger();
  pdl_wait();
  // epilogue operands that do not depend on this kernel's own work: requested now, used at the end
  float res0 = 0.f;
  uint32_t push_epoch = 0;
  if (EPI == EPI2_RESIDUAL && (int)threadIdx.x < pl * 2 * M)
    res0 = __bfloat162float(__ldcg(residual + (size_t)(threadIdx.x % M) * ldr + p_lo * 2 + threadIdx.x / M));
  if (EPI == EPI2_PUSH) push_epoch = __ldcg(reinterpret_cast<const uint32_t*>(push.ws[push.rank])) + 1;
  if (COOP)   // x is the residual stream: complete the pending all-reduce into it first
    g2_coop_finish(const_cast<bf16*>(x), ldx, M, K, push.ws[push.rank], push.world, push.hmax,
                   reinterpret_cast<int*>(red));
  if (COOP && late) pdl_trigger();
  g2_stage_x<M>(x, ldx, K, norm_w, xs, red);   // ends with a block barrier
  trl_trace_mark(0);

  bool ok = true;
  const uint32_t xs_a = smem_addr(xs) + (uint32_t)lane * 16u;
  const uint32_t pstride = (uint32_t)nchunks * 16u, xrow_bytes = (uint32_t)K * 2u;
  if (u0 < u1) {
    int cp = u0 / nsteps, cs = u0 % nsteps, slot = 0;
    uint32_t parity = 0;
    float acc[2][M];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
    auto flush = [&](int pair_local) {
      // two-slot mode: slot 0 belongs to the warp that holds the pair's first unit
      const int sl = nslot == 2 ? (pair_local * nsteps >= u0 ? 0 : 1) : warp - g2_owner(pair_local * nsteps, U, W);
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float v = warp_sum(acc[r][m]);
          if (lane == 0) slots[((size_t)(pair_local * 2 + r) * nslot + sl) * M + m] = v;
          acc[r][m] = 0.f;
        }
    };
    // one 32-chunk unit at shared address `ua` (already offset by lane * 16), step `st` of its row pair
    auto unit_full = [&](uint32_t ua, int st) {
      const uint4 wv0 = g2_lds128(ua), wv1 = g2_lds128(ua + 512u);
      const uint16_t sv[2] = {g2_lds16(ua + 1024u - (uint32_t)lane * 14u), g2_lds16(ua + 1088u - (uint32_t)lane * 14u)};
      const uint32_t w4[2][4] = {{wv0.x, wv0.y, wv0.z, wv0.w}, {wv1.x, wv1.y, wv1.z, wv1.w}};
      const uint32_t xa = xs_a + (uint32_t)st * 512u;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        uint32_t xh[16];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const uint4 t = g2_lds128(xa + (uint32_t)m * xrow_bytes + (uint32_t)p * pstride);
          xh[p * 4 + 0] = t.x, xh[p * 4 + 1] = t.y, xh[p * 4 + 2] = t.z, xh[p * 4 + 3] = t.w;
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float2 sc = h2_to_f2(cvt_e4m3x2_to_h2(sv[r]));
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            uint32_t a = 0u;  // f16x2 zero
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              uint32_t h[4];
              cvt_e2m1x8_to_h2x4(w4[r][blk * 2 + q], h);
#pragma unroll
              for (int i = 0; i < 4; ++i) a = hfma2_u(h[i], xh[(blk * 2 + q) * 4 + i], a);
            }
            const float2 af = h2_to_f2(a);
            acc[r][m] = fmaf(blk == 0 ? sc.x : sc.y, af.x + af.y, acc[r][m]);
          }
        }
      }
    };
    auto wait_stage = [&](uint32_t bar, uint32_t par, int u) {
      if (g2_try_wait(bar, par)) return true;
      const long long t0 = clock64();
      bool fine = true;
      for (uint32_t it = 1; !g2_try_wait(bar, par); ++it) {
        if ((it & 63) == 0 && clock64() - t0 > G2_WAIT_CYCLES) {
          trl_set_error(TRL_ERR_MBAR_TIMEOUT, (int)blockIdx.x, 200 + warp, u);
          fine = false;
          break;
        }
      }
      return (bool)__all_sync(0xffffffffu, fine);
    };
    if (FULL) {
      // every unit holds 32 chunks: constant offsets, two units per stage, no per-lane predicate
      const int n_units = u1 - u0;
      int p_left = u1 - p_unit;                    // units the producer has not requested yet
      for (int base = 0; base < n_units; base += STAGE_UNITS) {
        ok = wait_stage(bar_w + 8u * slot, parity, u0 + base);
        if (!ok) break;
        const uint32_t ua = ring_w + (uint32_t)slot * STAGE_BYTES + (uint32_t)lane * 16u;
        unit_full(ua, cs);
        if (++cs == nsteps) {
          flush(cp);
          cs = 0, ++cp;
        }
        if (base + 1 < n_units) {
          unit_full(ua + UNIT_BYTES, cs);
          if (++cs == nsteps) {
            flush(cp);
            cs = 0, ++cp;
          }
        }
        __syncwarp();
        if (lane == 0 && p_left > 0) {             // refill the stage just consumed
          const uint32_t bytes = (uint32_t)min(p_left, STAGE_UNITS) * UNIT_BYTES;
          const uint32_t bar = bar_w + 8u * slot;
          g2_expect_tx(bar, bytes);
          g2_bulk_load(ring_w + (uint32_t)slot * STAGE_BYTES, src + p_off, bytes, bar);
          p_off += bytes;
          p_left -= STAGE_UNITS;
        }
        if (++slot == NS) slot = 0, parity ^= 1u;
      }
    } else {
    for (int u = u0; u < u1;) {
      ok = wait_stage(bar_w + 8u * slot, parity, u);
      if (!ok) break;
      uint32_t ua = ring_w + (uint32_t)slot * STAGE_BYTES;   // shared address of the current unit
#pragma unroll
      for (int g = 0; g < STAGE_UNITS; ++g) {
        if (u >= u1) break;
        const int n = (cs == nsteps - 1) ? nlast : 32;
        if (lane < n) {
          const uint4 wv0 = g2_lds128(ua + lane * 16);
          const uint4 wv1 = g2_lds128(ua + n * 16 + lane * 16);
          const uint16_t sv[2] = {g2_lds16(ua + n * 32 + lane * 2), g2_lds16(ua + n * 34 + lane * 2)};
          const uint32_t w4[2][4] = {{wv0.x, wv0.y, wv0.z, wv0.w}, {wv1.x, wv1.y, wv1.z, wv1.w}};
          const uint32_t xa = xs_a + (uint32_t)cs * 512u;    // chunk cs * 32 + lane, piece 0
#pragma unroll
          for (int m = 0; m < M; ++m) {
            uint32_t xh[16];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              const uint4 t = g2_lds128(xa + (uint32_t)m * xrow_bytes + (uint32_t)p * pstride);
              xh[p * 4 + 0] = t.x, xh[p * 4 + 1] = t.y, xh[p * 4 + 2] = t.z, xh[p * 4 + 3] = t.w;
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const float2 sc = h2_to_f2(cvt_e4m3x2_to_h2(sv[r]));
#pragma unroll
              for (int blk = 0; blk < 2; ++blk) {
                uint32_t a = 0u;  // f16x2 zero
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  uint32_t h[4];
                  cvt_e2m1x8_to_h2x4(w4[r][blk * 2 + q], h);
#pragma unroll
                  for (int i = 0; i < 4; ++i) a = hfma2_u(h[i], xh[(blk * 2 + q) * 4 + i], a);
                }
                const float2 af = h2_to_f2(a);
                acc[r][m] = fmaf(blk == 0 ? sc.x : sc.y, af.x + af.y, acc[r][m]);
              }
            }
          }
        }
        ua += (uint32_t)n * 36u;
        ++u;
        if (++cs == nsteps) {
          flush(cp);
          cs = 0, ++cp;
        }
      }
      __syncwarp();
      if (lane == 0 && p_unit < u1) issue();   // refill the stage just consumed
      if (++slot == NS) slot = 0, parity ^= 1u;
    }
    }
    if (ok && cs != 0) flush(cp);   // range ended inside a pair
    if (!ok) {
      // copies may still be in flight towards this CTA's shared memory: let them land
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) {
      }
    }
  }
  trl_trace_mark(1);
  __syncthreads();

  // block-wide epilogue over this CTA's rows
  const float ts = *tscale;
  float rsc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) rsc[m] = ts * g2_row_scale(red, m, K, norm_w != nullptr, eps);
  if (EPI == EPI2_SWIGLU) {
    for (int i = threadIdx.x; i < pl * M; i += G2_THREADS) {
      const int pr = i / M, m = i % M;
      float g = 0.f, u = 0.f;
      for (int sl = 0; sl < nslot; ++sl) {
        g += slots[((size_t)(pr * 2) * nslot + sl) * M + m];
        u += slots[((size_t)(pr * 2 + 1) * nslot + sl) * M + m];
      }
      const float sc = rsc[m];
      const int n = (p_lo + pr) * 2;
      reinterpret_cast<bf16*>(yout)[(size_t)m * ldy + (n >> 1)] = __float2bfloat16(silu_f(g * sc) * (u * sc));
    }
  } else {
    for (int i = threadIdx.x; i < pl * 2 * M; i += G2_THREADS) {
      const int rl = i / M, m = i % M;
      const int n = p_lo * 2 + rl;
      float v = 0.f;
      for (int sl = 0; sl < nslot; ++sl) v += slots[((size_t)rl * nslot + sl) * M + m];
      v *= rsc[m];
      if (EPI == EPI2_PUSH) {
        const uint32_t epoch = push_epoch;
        const size_t off = 65536 + ((size_t)(((epoch & 1) * 8 + push.rank) * 8 + push.row0 + m) * push.hmax + n) * 8;
        const uint2 word = make_uint2(__float_as_uint(v), epoch);
        for (int p = 0; p < push.world; ++p) st_relaxed_sys_v2(push.ws[p] + off, word);
      } else {
        if (EPI == EPI2_RESIDUAL) v += i < G2_THREADS ? res0 : __bfloat162float(__ldcg(residual + (size_t)m * ldr + n));
        if (EPI == EPI2_STORE_F32)
          reinterpret_cast<float*>(yout)[(size_t)m * ldy + n] = v;
        else
          reinterpret_cast<bf16*>(yout)[(size_t)m * ldy + n] = __float2bfloat16(v);
      }
    }
  }
  if (EPI == EPI2_PUSH && late) pdl_trigger();
  trl_trace_end();
}

// (wq [N, K/2], scale [N, K/16]) -> stream layout.  One thread per (row, chunk).
__global__ void __launch_bounds__(256)
gemv_stream_pack_kernel(const uint8_t* __restrict__ wq, const uint8_t* __restrict__ scale,
                        uint8_t* __restrict__ out, int N, int K) {
  const int nchunks = K >> 5;
  const long long total = (long long)N * nchunks;
  const int nsteps = (nchunks + 31) >> 5;
  const int nlast = nchunks - 32 * (nsteps - 1);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / nchunks), c = (int)(i % nchunks);
    const int p = row >> 1, r = row & 1, s = c >> 5, j = c & 31;
    const int n = (s == nsteps - 1) ? nlast : 32;
    uint8_t* ub = out + (size_t)p * nchunks * 36 + (size_t)s * UNIT_BYTES;
    *reinterpret_cast<uint4*>(ub + (size_t)(r * n + j) * 16) =
        *reinterpret_cast<const uint4*>(wq + (size_t)row * (K >> 1) + (size_t)c * 16);
    *reinterpret_cast<uint16_t*>(ub + (size_t)n * 32 + (size_t)(r * n + j) * 2) =
        *reinterpret_cast<const uint16_t*>(scale + (size_t)row * (K >> 4) + (size_t)c * 2);
  }
}

// ---------------------------------------------------------------------------------------
// Chain of up to four projections in ONE launch.  Consecutive decode projections depend on each
// other through a full activation row, so between two of them every CTA must have stored its
// rows: here that is a grid barrier (arrival counter + release generation, bounded waits)
// instead of a kernel boundary.  What the chain buys is the weight stream: a warp's producer
// simply continues with its share of the NEXT projection when the current one is exhausted, so
// the rings refill across the barrier and the activation staging, where separate launches can
// only prefetch once their CTAs have found room on an SM.  Ops: plain / residual / SwiGLU / fp32
// store, tensor-parallel push, and the cooperative all-reduce finish in front of an op.
struct G2Op {
  const bf16* x;
  const uint8_t* wst;
  const float* tscale;
  const float* norm_w;
  const bf16* residual;
  void* out;
  int ldx, ldr, ldy, N, K, nslot, epi, coop;
  float eps;
};
constexpr int G2_CHAIN_MAX = 4;
struct G2Chain {
  G2Op op[G2_CHAIN_MAX];
  int n_ops;
  int xs_bytes;          // bytes reserved for the staged activation rows (max over the ops)
  uint32_t* bar;         // [0] arrival counter, [32] release generation (separate 128-byte lines)
};
constexpr int G2_BAR_RELEASE = 32;

struct G2Range {
  int p_lo, pl, nchunks, nsteps, nlast, U, u0, u1;
  uint32_t pair_bytes;
};
__device__ __forceinline__ G2Range g2_range(const G2Op& o, int warp) {
  G2Range r;
  const int npairs = o.N >> 1;
  r.p_lo = (int)(((long long)blockIdx.x * npairs) / gridDim.x);
  r.pl = (int)(((long long)(blockIdx.x + 1) * npairs) / gridDim.x) - r.p_lo;
  r.nchunks = o.K >> 5;
  r.nsteps = (r.nchunks + 31) >> 5;
  r.nlast = r.nchunks - 32 * (r.nsteps - 1);
  r.pair_bytes = (uint32_t)r.nchunks * 36u;
  r.U = r.pl * r.nsteps;
  r.u0 = (int)(((long long)warp * r.U) / G2_WARPS);
  r.u1 = (int)(((long long)(warp + 1) * r.U) / G2_WARPS);
  return r;
}

// Grid barrier of the chain: generation `target` is released by the last CTA to arrive.
__device__ __forceinline__ bool g2_grid_barrier(uint32_t* bar, uint32_t target, int* s_flag) {
  __syncthreads();                       // this CTA's stores of the finished op are issued
  if (threadIdx.x == 0) {
    s_flag[2] = 1;
    __threadfence();
    const uint32_t prev = atomicAdd(bar, 1u);
    if (prev == gridDim.x - 1) {
      bar[0] = 0;
      __threadfence();
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(bar + G2_BAR_RELEASE), "r"(target) : "memory");
    } else {
      uint32_t seen;
      const long long t0 = clock64();
      for (uint32_t it = 0;; ++it) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(bar + G2_BAR_RELEASE) : "memory");
        if (seen == target) break;
        __nanosleep(32);                  // hundreds of CTAs poll one word: leave the L2 slice room for the arrivals
        if ((it & 15) == 15 && clock64() - t0 > G2_WAIT_CYCLES) {
          trl_set_error(TRL_ERR_WAIT_TIMEOUT, 7, (int)blockIdx.x, (int)target);
          s_flag[2] = 0;
          break;
        }
      }
    }
  }
  __syncthreads();
  return s_flag[2] != 0;
}

template <int M>
__global__ void __launch_bounds__(G2_THREADS, 3)
gemv2_chain_kernel(const __grid_constant__ G2Chain ch, int NS, const TrlPushArgs push) {
  constexpr int W = G2_WARPS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // ring [W][NS][STAGE_BYTES] | bars [W][MAX_NS] | xs (xs_bytes) | 8 spare floats | red[64] | slots
  unsigned char* ring = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)W * NS * STAGE_BYTES);
  __half* xs = reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(bars) + W * G2_MAX_NS * 8);
  float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xs) + ch.xs_bytes) + 8;
  float* slots = red + 64;
  int* s_flag = reinterpret_cast<int*>(red + 48);      // [0..1] cooperative finish, [2] chain barrier, [3] generation

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t ring_w = smem_addr(ring + (size_t)warp * NS * STAGE_BYTES);
  const uint32_t bar_w = smem_addr(bars + warp * G2_MAX_NS);

  // ---- producer (lane 0 of each warp): walks this warp's unit ranges of op 0, 1, ... in order
  int pj = 0, p_unit = 0, p_step = 0, p_slot = 0;
  uint32_t p_off = 0;
  G2Range pr = g2_range(ch.op[0], warp);
  const uint8_t* p_src = ch.op[0].wst + (size_t)pr.p_lo * pr.pair_bytes;
  auto p_enter = [&]() {                 // position the cursor at the start of op pj's range
    p_unit = pr.u0, p_step = pr.u0 % pr.nsteps;
    p_off = (uint32_t)(pr.u0 / pr.nsteps) * pr.pair_bytes + (uint32_t)(pr.u0 % pr.nsteps) * (uint32_t)UNIT_BYTES;
  };
  p_enter();
  auto issue = [&]() {   // one stage: the next STAGE_UNITS units of the producer's current op
    while (pj < ch.n_ops && p_unit >= pr.u1) {
      if (++pj < ch.n_ops) {
        pr = g2_range(ch.op[pj], warp);
        p_src = ch.op[pj].wst + (size_t)pr.p_lo * pr.pair_bytes;
        p_enter();
      }
    }
    if (pj >= ch.n_ops) return;
    uint32_t bytes = 0;
#pragma unroll
    for (int g = 0; g < STAGE_UNITS; ++g) {
      if (p_unit < pr.u1) {
        bytes += (p_step == pr.nsteps - 1) ? (uint32_t)pr.nlast * 36u : (uint32_t)UNIT_BYTES;
        if (++p_step == pr.nsteps) p_step = 0;
        ++p_unit;
      }
    }
    const uint32_t bar = bar_w + 8u * p_slot;
    g2_expect_tx(bar, bytes);
    g2_bulk_load(ring_w + (uint32_t)p_slot * STAGE_BYTES, p_src + p_off, bytes, bar);
    p_off += bytes;
    if (++p_slot == NS) p_slot = 0;
  };
  if (lane == 0) {
    for (int s = 0; s < NS; ++s) g2_mbar_init(bar_w + 8u * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int s = 0; s < NS; ++s) issue();     // weights never depend on the previous kernel
  }
  pdl_enter(120);                        // the next kernel is let in behind this launch's last grid barrier
  if (ch.n_ops == 1 && !ch.op[0].coop) pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) s_flag[3] = (int)__ldcg(ch.bar + G2_BAR_RELEASE);
  __syncthreads();
  const uint32_t gen0 = (uint32_t)s_flag[3];
  uint32_t n_bar = 0;

  int slot = 0;
  uint32_t parity = 0;
  bool ok = true;
  for (int j = 0; j < ch.n_ops; ++j) {
    const G2Op& o = ch.op[j];
    const G2Range cr = g2_range(o, warp);
    const int K = o.K, nslot = o.nslot, nsteps = cr.nsteps, pl = cr.pl, p_lo = cr.p_lo;
    const bool full = (K & 1023) == 0;
    // the cooperative finish has a grid barrier of its own after which every CTA is past op j - 1
    if (j > 0 && !o.coop) ok = g2_grid_barrier(ch.bar, gen0 + (++n_bar), s_flag) && ok;
    else __syncthreads();                 // slots and red of the previous op are free
    trl_trace_mark(3 * j);                // past the barrier in front of op j
    for (int i = threadIdx.x; i < pl * 2 * nslot * M; i += G2_THREADS) slots[i] = 0.f;
    float res0 = 0.f;
    uint32_t push_epoch = 0;
    if (o.epi == EPI2_RESIDUAL && (int)threadIdx.x < pl * 2 * M)
      res0 = __bfloat162float(__ldcg(o.residual + (size_t)(threadIdx.x % M) * o.ldr + p_lo * 2 + threadIdx.x / M));
    if (o.epi == EPI2_PUSH) push_epoch = __ldcg(reinterpret_cast<const uint32_t*>(push.ws[push.rank])) + 1;
    if (o.coop)
      ok = g2_coop_finish(const_cast<bf16*>(o.x), o.ldx, M, K, push.ws[push.rank], push.world, push.hmax, s_flag) && ok;
    if (j == ch.n_ops - 1 && (ch.n_ops > 1 || o.coop)) pdl_trigger();
    g2_stage_x<M>(o.x, o.ldx, K, o.norm_w, xs, red);   // ends with a block barrier
    trl_trace_mark(3 * j + 1);

    const uint32_t xs_a = smem_addr(xs) + (uint32_t)lane * 16u;
    const uint32_t pstride = (uint32_t)cr.nchunks * 16u, xrow_bytes = (uint32_t)K * 2u;
    if (cr.u0 < cr.u1 && ok) {
      int cp = cr.u0 / nsteps, cs = cr.u0 % nsteps;
      float acc[2][M];
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
      auto flush = [&](int pair_local) {
        const int sl = nslot == 2 ? (pair_local * nsteps >= cr.u0 ? 0 : 1) : warp - g2_owner(pair_local * nsteps, cr.U, W);
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const float v = warp_sum(acc[r][m]);
            if (lane == 0) slots[((size_t)(pair_local * 2 + r) * nslot + sl) * M + m] = v;
            acc[r][m] = 0.f;
          }
      };
      // one unit of n chunks at shared address `ua`, step `st` of its row pair (n = 32: every lane works)
      auto unit = [&](uint32_t ua, int st, int n) {
        if (lane < n) {
          const uint4 wv0 = g2_lds128(ua + lane * 16);
          const uint4 wv1 = g2_lds128(ua + n * 16 + lane * 16);
          const uint16_t sv[2] = {g2_lds16(ua + n * 32 + lane * 2), g2_lds16(ua + n * 34 + lane * 2)};
          const uint32_t w4[2][4] = {{wv0.x, wv0.y, wv0.z, wv0.w}, {wv1.x, wv1.y, wv1.z, wv1.w}};
          const uint32_t xa = xs_a + (uint32_t)st * 512u;
#pragma unroll
          for (int m = 0; m < M; ++m) {
            uint32_t xh[16];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              const uint4 t = g2_lds128(xa + (uint32_t)m * xrow_bytes + (uint32_t)p * pstride);
              xh[p * 4 + 0] = t.x, xh[p * 4 + 1] = t.y, xh[p * 4 + 2] = t.z, xh[p * 4 + 3] = t.w;
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const float2 sc = h2_to_f2(cvt_e4m3x2_to_h2(sv[r]));
#pragma unroll
              for (int blk = 0; blk < 2; ++blk) {
                uint32_t a = 0u;  // f16x2 zero
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  uint32_t h[4];
                  cvt_e2m1x8_to_h2x4(w4[r][blk * 2 + q], h);
#pragma unroll
                  for (int i = 0; i < 4; ++i) a = hfma2_u(h[i], xh[(blk * 2 + q) * 4 + i], a);
                }
                const float2 af = h2_to_f2(a);
                acc[r][m] = fmaf(blk == 0 ? sc.x : sc.y, af.x + af.y, acc[r][m]);
              }
            }
          }
        }
      };
      // the same with 32 chunks (K % 1024 == 0): constant offsets, no per-lane predicate
      auto unit_full = [&](uint32_t ua, int st) {
        const uint4 wv0 = g2_lds128(ua), wv1 = g2_lds128(ua + 512u);
        const uint16_t sv[2] = {g2_lds16(ua + 1024u - (uint32_t)lane * 14u), g2_lds16(ua + 1088u - (uint32_t)lane * 14u)};
        const uint32_t w4[2][4] = {{wv0.x, wv0.y, wv0.z, wv0.w}, {wv1.x, wv1.y, wv1.z, wv1.w}};
        const uint32_t xa = xs_a + (uint32_t)st * 512u;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          uint32_t xh[16];
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const uint4 t = g2_lds128(xa + (uint32_t)m * xrow_bytes + (uint32_t)p * pstride);
            xh[p * 4 + 0] = t.x, xh[p * 4 + 1] = t.y, xh[p * 4 + 2] = t.z, xh[p * 4 + 3] = t.w;
          }
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const float2 sc = h2_to_f2(cvt_e4m3x2_to_h2(sv[r]));
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              uint32_t a = 0u;  // f16x2 zero
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                uint32_t h[4];
                cvt_e2m1x8_to_h2x4(w4[r][blk * 2 + q], h);
#pragma unroll
                for (int i = 0; i < 4; ++i) a = hfma2_u(h[i], xh[(blk * 2 + q) * 4 + i], a);
              }
              const float2 af = h2_to_f2(a);
              acc[r][m] = fmaf(blk == 0 ? sc.x : sc.y, af.x + af.y, acc[r][m]);
            }
          }
        }
      };
      auto wait_stage = [&](uint32_t bar, uint32_t par, int u) {
        if (g2_try_wait(bar, par)) return true;
        const long long t0 = clock64();
        bool fine = true;
        for (uint32_t it = 1; !g2_try_wait(bar, par); ++it) {
          if ((it & 63) == 0 && clock64() - t0 > G2_WAIT_CYCLES) {
            trl_set_error(TRL_ERR_MBAR_TIMEOUT, (int)blockIdx.x, 300 + warp, u);
            fine = false;
            break;
          }
        }
        return (bool)__all_sync(0xffffffffu, fine);
      };
      if (full) {
        for (int u = cr.u0; u < cr.u1; u += STAGE_UNITS) {
          ok = wait_stage(bar_w + 8u * slot, parity, u);
          if (!ok) break;
          const uint32_t ua = ring_w + (uint32_t)slot * STAGE_BYTES + (uint32_t)lane * 16u;
          unit_full(ua, cs);
          if (++cs == nsteps) {
            flush(cp);
            cs = 0, ++cp;
          }
          if (u + 1 < cr.u1) {
            unit_full(ua + UNIT_BYTES, cs);
            if (++cs == nsteps) {
              flush(cp);
              cs = 0, ++cp;
            }
          }
          __syncwarp();
          if (lane == 0) issue();          // refill the stage just consumed (this op's or a later op's bytes)
          if (++slot == NS) slot = 0, parity ^= 1u;
        }
      } else {
        for (int u = cr.u0; u < cr.u1;) {
          ok = wait_stage(bar_w + 8u * slot, parity, u);
          if (!ok) break;
          uint32_t ua = ring_w + (uint32_t)slot * STAGE_BYTES;
#pragma unroll
          for (int g = 0; g < STAGE_UNITS; ++g) {
            if (u >= cr.u1) break;
            const int n = (cs != nsteps - 1) ? 32 : cr.nlast;
            unit(ua, cs, n);
            ua += (uint32_t)n * 36u;
            ++u;
            if (++cs == nsteps) {
              flush(cp);
              cs = 0, ++cp;
            }
          }
          __syncwarp();
          if (lane == 0) issue();
          if (++slot == NS) slot = 0, parity ^= 1u;
        }
      }
      if (ok && cs != 0) flush(cp);        // range ended inside a pair
    }
    trl_trace_mark(3 * j + 2);
    __syncthreads();

    // block-wide epilogue over this CTA's rows of op j
    const float ts = *o.tscale;
    float rsc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) rsc[m] = ts * g2_row_scale(red, m, K, o.norm_w != nullptr, o.eps);
    if (o.epi == EPI2_SWIGLU) {
      for (int i = threadIdx.x; i < pl * M; i += G2_THREADS) {
        const int pr_ = i / M, m = i % M;
        float g = 0.f, u = 0.f;
        for (int sl = 0; sl < nslot; ++sl) {
          g += slots[((size_t)(pr_ * 2) * nslot + sl) * M + m];
          u += slots[((size_t)(pr_ * 2 + 1) * nslot + sl) * M + m];
        }
        const float sc = rsc[m];
        const int n = (p_lo + pr_) * 2;
        reinterpret_cast<bf16*>(o.out)[(size_t)m * o.ldy + (n >> 1)] = __float2bfloat16(silu_f(g * sc) * (u * sc));
      }
    } else {
      for (int i = threadIdx.x; i < pl * 2 * M; i += G2_THREADS) {
        const int rl = i / M, m = i % M;
        const int n = p_lo * 2 + rl;
        float v = 0.f;
        for (int sl = 0; sl < nslot; ++sl) v += slots[((size_t)rl * nslot + sl) * M + m];
        v *= rsc[m];
        if (o.epi == EPI2_PUSH) {
          const size_t off = 65536 + ((size_t)(((push_epoch & 1) * 8 + push.rank) * 8 + push.row0 + m) * push.hmax + n) * 8;
          const uint2 word = make_uint2(__float_as_uint(v), push_epoch);
          for (int p = 0; p < push.world; ++p) st_relaxed_sys_v2(push.ws[p] + off, word);
        } else {
          if (o.epi == EPI2_RESIDUAL) v += i < G2_THREADS ? res0 : __bfloat162float(__ldcg(o.residual + (size_t)m * o.ldr + n));
          if (o.epi == EPI2_STORE_F32)
            reinterpret_cast<float*>(o.out)[(size_t)m * o.ldy + n] = v;
          else
            reinterpret_cast<bf16*>(o.out)[(size_t)m * o.ldy + n] = __float2bfloat16(v);
        }
      }
    }
  }
  if (!ok) {
    // copies may still be in flight towards this CTA's shared memory: let them land
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
  trl_trace_end();
}

int g_g2_trigger = -1;
int g2_trigger_mode() {
  if (g_g2_trigger < 0) g_g2_trigger = getenv("TRL_TP_TRIGGER") ? atoi(getenv("TRL_TP_TRIGGER")) : 2;
  return g_g2_trigger;
}

int g2_num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

template <int M, int EPI, bool COOP>
cudaError_t launch_gemv2(const bf16* x, int ldx, const uint8_t* wst, const float* ts, const float* norm_w,
                         float eps, const bf16* res, int ldr, void* y, int ldy, int N, int K, cudaStream_t st,
                         const TrlPushArgs& push) {
  constexpr int W = G2_WARPS;
  const int npairs = N / 2;
  static const int ctas_per_sm = getenv("TRL_GEMV2_CTAS") ? atoi(getenv("TRL_GEMV2_CTAS")) : 3;
  const int grid = min(g2_num_sms() * ctas_per_sm, npairs);
  const int pl_max = (npairs + grid - 1) / grid;
  const int nslot = (npairs / grid) >= W ? 2 : W;
  const size_t fixed = (size_t)W * G2_MAX_NS * 8 + (size_t)M * K * sizeof(__half) + 8 * sizeof(float) +
                       64 * sizeof(float) + (size_t)pl_max * 2 * nslot * M * sizeof(float);
  // three CTAs per SM when the activation row leaves room for a useful ring, else two
  static const int ns_env = getenv("TRL_GEMV2_NS") ? atoi(getenv("TRL_GEMV2_NS")) : 0;
  int ns = (int)((74 * 1024 - (long)fixed) / (W * STAGE_BYTES));
  if (ns < 2) ns = (int)((112 * 1024 - (long)fixed) / (W * STAGE_BYTES));
  if (ns_env > 0) ns = ns_env;
  ns = min(ns, G2_MAX_NS);
  if (ns < 2) return cudaErrorInvalidValue;
  const size_t smem = (size_t)W * ns * STAGE_BYTES + fixed;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(gemv2_kernel<M, EPI, true, COOP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(gemv2_kernel<M, EPI, true, COOP>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    cudaFuncSetAttribute(gemv2_kernel<M, EPI, false, COOP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(gemv2_kernel<M, EPI, false, COOP>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    configured = true;
  }
  if (COOP) {
    // the grid barrier of the cooperative finish needs every CTA resident at once
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv2_kernel<M, EPI, true, COOP>, G2_THREADS, smem) != cudaSuccess ||
        per_sm * g2_num_sms() < grid)
      return cudaErrorInvalidValue;
  }
  if ((K % 1024) == 0)   // every step of a row is full: 32 chunks
    return trl_launch(gemv2_kernel<M, EPI, true, COOP>, dim3(grid), dim3(G2_THREADS), smem, st, x, ldx, wst, ts,
                      norm_w, eps, res, ldr, y, ldy, N, K, nslot, ns, push, g2_trigger_mode());
  return trl_launch(gemv2_kernel<M, EPI, false, COOP>, dim3(grid), dim3(G2_THREADS), smem, st, x, ldx, wst, ts,
                    norm_w, eps, res, ldr, y, ldy, N, K, nslot, ns, push, g2_trigger_mode());
}

template <int EPI, bool COOP = false>
cudaError_t dispatch2(int M, const bf16* x, int ldx, const uint8_t* wst, const float* ts, const float* norm_w,
                      float eps, const bf16* res, int ldr, void* y, int ldy, int N, int K, cudaStream_t st,
                      const TrlPushArgs& push = TrlPushArgs()) {
  if (M == 1) return launch_gemv2<1, EPI, COOP>(x, ldx, wst, ts, norm_w, eps, res, ldr, y, ldy, N, K, st, push);
  if (M == 2) return launch_gemv2<2, EPI, COOP>(x, ldx, wst, ts, norm_w, eps, res, ldr, y, ldy, N, K, st, push);
  return cudaErrorInvalidValue;
}


template <int M>
cudaError_t launch_chain(const TrlChainOp* ops, int n_ops, uint32_t* bar, const TrlPushArgs& push, cudaStream_t st) {
  constexpr int W = G2_WARPS;
  static const int ctas_per_sm = getenv("TRL_GEMV2_CTAS") ? atoi(getenv("TRL_GEMV2_CTAS")) : 3;
  int grid = g2_num_sms() * ctas_per_sm;
  int kmax = 0;
  for (int j = 0; j < n_ops; ++j) grid = min(grid, ops[j].N / 2), kmax = max(kmax, ops[j].K);
  G2Chain ch;
  ch.n_ops = n_ops, ch.bar = bar, ch.xs_bytes = M * kmax * (int)sizeof(__half);
  size_t slot_bytes = 0;
  for (int j = 0; j < n_ops; ++j) {
    const TrlChainOp& a = ops[j];
    G2Op& o = ch.op[j];
    const int npairs = a.N / 2;
    o.x = (const bf16*)a.x, o.wst = (const uint8_t*)a.wst, o.tscale = (const float*)a.tscale;
    o.norm_w = (const float*)a.norm_w, o.residual = (const bf16*)a.residual, o.out = a.out;
    o.ldx = a.ldx, o.ldr = a.ldr, o.ldy = a.ldy, o.N = a.N, o.K = a.K, o.epi = a.epi, o.coop = a.coop, o.eps = a.eps;
    o.nslot = (npairs / grid) >= W ? 2 : W;
    const int pl_max = (npairs + grid - 1) / grid;
    slot_bytes = max(slot_bytes, (size_t)pl_max * 2 * o.nslot * M * sizeof(float));
  }
  for (int j = n_ops; j < G2_CHAIN_MAX; ++j) ch.op[j] = ch.op[0];
  const size_t fixed = (size_t)W * G2_MAX_NS * 8 + (size_t)ch.xs_bytes + 8 * sizeof(float) + 64 * sizeof(float) + slot_bytes;
  int ns = (int)((74 * 1024 - (long)fixed) / (W * STAGE_BYTES));
  if (ns < 2) ns = (int)((112 * 1024 - (long)fixed) / (W * STAGE_BYTES));
  ns = min(ns, G2_MAX_NS);
  if (ns < 2) return cudaErrorInvalidValue;
  const size_t smem = (size_t)W * ns * STAGE_BYTES + fixed;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(gemv2_chain_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(gemv2_chain_kernel<M>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    configured = true;
  }
  // the grid barriers need every CTA resident at once
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv2_chain_kernel<M>, G2_THREADS, smem) != cudaSuccess ||
      per_sm * g2_num_sms() < grid)
    return cudaErrorInvalidValue;
  return trl_launch(gemv2_chain_kernel<M>, dim3(grid), dim3(G2_THREADS), smem, st, ch, ns, push);
}

}  // namespace

// Bytes of the stream layout of an [N, K] NVFP4 weight (N even, K % 128 == 0).
TRL_API long trl_gemv_stream_bytes(int N, int K) {
  if (N <= 0 || (N & 1) || K <= 0 || (K % 128) != 0) return -1;
  return (long)(N / 2) * (K / 32) * 36;
}

TRL_API int trl_gemv_stream_pack(const void* wq, const void* scale, void* out, int N, int K, void* stream) {
  if (trl_gemv_stream_bytes(N, K) < 0) return (int)cudaErrorInvalidValue;
  const long long total = (long long)N * (K / 32);
  const int grid = (int)min((long long)4096, (total + 255) / 256);
  gemv_stream_pack_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)wq, (const uint8_t*)scale,
                                                                 (uint8_t*)out, N, K);
  return (int)cudaGetLastError();
}

// y = epi(tscale * norm(x) @ W^T) for M <= 2 rows from the stream layout of W.
TRL_API int trl_gemv2_nvfp4(const void* x, int ldx, const void* wst, const void* tscale, const void* norm_w, float eps,
                            const void* residual, int ldr, void* y, int ldy, int M, int N, int K, int epi,
                            void* stream) {
  if (trl_gemv_stream_bytes(N, K) < 0 || M < 1 || M > 2 || K > G2_XV * G2_THREADS * 8) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  const bf16* xp = (const bf16*)x;
  const bf16* rp = (const bf16*)residual;
  const uint8_t* wp = (const uint8_t*)wst;
  const float* tp = (const float*)tscale;
  const float* np_ = (const float*)norm_w;
  switch (epi) {
    case EPI2_STORE: return (int)dispatch2<EPI2_STORE>(M, xp, ldx, wp, tp, np_, eps, rp, ldr, y, ldy, N, K, st);
    case EPI2_RESIDUAL: return (int)dispatch2<EPI2_RESIDUAL>(M, xp, ldx, wp, tp, np_, eps, rp, ldr, y, ldy, N, K, st);
    case EPI2_SWIGLU: return (int)dispatch2<EPI2_SWIGLU>(M, xp, ldx, wp, tp, np_, eps, rp, ldr, y, ldy, N, K, st);
    case EPI2_STORE_F32: return (int)dispatch2<EPI2_STORE_F32>(M, xp, ldx, wp, tp, np_, eps, rp, ldr, y, ldy, N, K, st);
  }
  return (int)cudaErrorInvalidValue;
}

// Row-parallel variant: fp32 partial rows go into every rank's one-shot all-reduce slot.
TRL_API int trl_gemv2_nvfp4_push(const void* x, int ldx, const void* wst, const void* tscale, void* const* ws,
                                 int rank, int world, int hmax, int M, int N, int K, void* stream) {
  if (trl_gemv_stream_bytes(N, K) < 0 || M < 1 || M > 2 || N > hmax || K > G2_XV * G2_THREADS * 8)
    return (int)cudaErrorInvalidValue;
  TrlPushArgs push;
  for (int i = 0; i < 8; ++i) push.ws[i] = i < world ? (unsigned char*)ws[i] : nullptr;
  push.rank = rank, push.world = world, push.hmax = hmax, push.row0 = 0;
  return (int)dispatch2<EPI2_PUSH>(M, (const bf16*)x, ldx, (const uint8_t*)wst, (const float*)tscale, nullptr, 0.f,
                                   nullptr, 0, nullptr, 0, N, K, (cudaStream_t)stream, push);
}

// Consumer of a pending one-shot all-reduce: x (the residual stream, [M, K] bf16 in this rank's
// memory) first receives residual + sum of all ranks' partial rows, then y = epi(norm(x) @ W^T)
// (epi: plain store or SwiGLU).  ws: table of all ranks' workspaces (comm.cu layout).
TRL_API int trl_gemv2_nvfp4_coop(void* x, int ldx, const void* wst, const void* tscale, const void* norm_w,
                                 float eps, void* y, int ldy, int M, int N, int K, int epi, void* const* ws,
                                 int rank, int world, int hmax, void* stream) {
  if (trl_gemv_stream_bytes(N, K) < 0 || M < 1 || M > 2 || K > hmax || K > G2_XV * G2_THREADS * 8 || world > 8)
    return (int)cudaErrorInvalidValue;
  TrlPushArgs push;
  for (int i = 0; i < 8; ++i) push.ws[i] = i < world ? (unsigned char*)ws[i] : nullptr;
  push.rank = rank, push.world = world, push.hmax = hmax, push.row0 = 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (epi == EPI2_STORE)
    return (int)dispatch2<EPI2_STORE, true>(M, (const bf16*)x, ldx, (const uint8_t*)wst, (const float*)tscale,
                                            (const float*)norm_w, eps, nullptr, 0, y, ldy, N, K, st, push);
  if (epi == EPI2_SWIGLU)
    return (int)dispatch2<EPI2_SWIGLU, true>(M, (const bf16*)x, ldx, (const uint8_t*)wst, (const float*)tscale,
                                             (const float*)norm_w, eps, nullptr, 0, y, ldy, N, K, st, push);
  return (int)cudaErrorInvalidValue;
}

// Up to four dependent projections (M <= 2 rows) in one launch: op j + 1 may read what op j stored.
// `bar`: 64 zero-initialised uint32 words in device memory that belong to this stream of launches.
// ws / rank / world / hmax: the tensor-parallel workspace table for EPI2_PUSH and coop ops (null / 0 without).
TRL_API int trl_gemv2_chain(const void* ops, int n_ops, int M, void* bar, void* const* ws, int rank, int world,
                            int hmax, void* stream) {
  const TrlChainOp* a = (const TrlChainOp*)ops;
  if (n_ops < 1 || n_ops > G2_CHAIN_MAX || M < 1 || M > 2 || bar == nullptr) return (int)cudaErrorInvalidValue;
  for (int j = 0; j < n_ops; ++j) {
    if (trl_gemv_stream_bytes(a[j].N, a[j].K) < 0 || a[j].K > G2_XV * G2_THREADS * 8) return (int)cudaErrorInvalidValue;
    if (a[j].epi < EPI2_STORE || a[j].epi > EPI2_PUSH) return (int)cudaErrorInvalidValue;
    if ((a[j].epi == EPI2_PUSH || a[j].coop) && (ws == nullptr || world < 1 || world > 8)) return (int)cudaErrorInvalidValue;
    if (a[j].epi == EPI2_PUSH && a[j].N > hmax) return (int)cudaErrorInvalidValue;
    if (a[j].coop && (a[j].K > hmax || (a[j].epi != EPI2_STORE && a[j].epi != EPI2_SWIGLU))) return (int)cudaErrorInvalidValue;
  }
  TrlPushArgs push;
  for (int i = 0; i < 8; ++i) push.ws[i] = (ws != nullptr && i < world) ? (unsigned char*)ws[i] : nullptr;
  push.rank = rank, push.world = world, push.hmax = hmax, push.row0 = 0;
  if (M == 1) return (int)launch_chain<1>(a, n_ops, (uint32_t*)bar, push, (cudaStream_t)stream);
  return (int)launch_chain<2>(a, n_ops, (uint32_t*)bar, push, (cudaStream_t)stream);
}

// When tensor-parallel projections let the next kernel in (see gemv2_kernel): 0, 1 or 2; -1 = the environment's choice.
TRL_API void trl_gemv2_set_trigger(int mode) { g_g2_trigger = mode; }
