// NVFP4 projection for 3..16 activation rows on the tensor cores (batched decode, speculative
// verify windows): y = epi(norm(x) @ dequant(W)^T) with the weights streamed ONCE for all rows and
// the activations kept in f16 -- no activation quantiser launch, no NVFP4 rounding of x.
//
// mma.sync m16n8k16 (f16 inputs, fp32 accumulation) with the WEIGHTS as the A operand: a warp
// tile is 16 weight rows, decoded e2m1 -> f16 by the native cvt and multiplied by their e4m3
// block scale in f16 (exact: 2 + 4 significant bits), the B operand is 8 activation rows from
// shared memory (two n-tiles for 9..16 rows).  Lane (g, t) = (lane / 4, lane % 4) streams 64
// contiguous bytes (128 k) of weight rows `2g` and `2g + 1` of the tile per 512-k unit, plus their
// eight scale bytes; a dot product does not care in which order k is summed, so those 128 values
// feed 32 MMAs under a fixed permutation of k, and the activation rows are written to shared memory
// in exactly that permuted order, so that the B fragments are plain ldmatrix loads.  Rows 2g / 2g+1
// share a lane: the gate / up pair of the SwiGLU epilogue needs no exchange.
//
// A CTA owns a contiguous run of 8-row half tiles; its (tile, unit) pairs are split evenly over
// the 12 warps (a warp's share spans at most three tiles), partial tiles meet in shared memory in
// warp order (fixed summation order: run twice, same bits).  Activations that do not fit shared
// memory (K = 17408) are staged in phases; a warp meets the same tiles in every phase, so its
// accumulators stay in registers.  Weight loads are double buffered in registers and the first
// unit is fetched before the dependency wait.
//
// Reference parity: linear_fp4_mma8 (packages/tilerl-kernels/src/tilerl_kernels/kernels_linear.py:1494)
// serves the same row counts with the weights as the MMA's A operand.
#include "common.cuh"

namespace {

enum { ME_STORE = 0, ME_RESIDUAL = 1, ME_SWIGLU = 2, ME_STORE_F32 = 3 };
constexpr int MM_THREADS = 384, MM_WARPS = MM_THREADS / 32, MM_SLOTS = 3;
constexpr int MM_UNIT = 512;                        // k per unit: 4 lanes x 128 values
constexpr int MM_XPAD = 8;                          // f16 elements of padding per activation row (16 bytes)
constexpr float MM_PRESCALE = 0.0625f;              // activations are staged as f16(x / 16), saturating
constexpr int MM_XS_BYTES = 150 * 1024;

struct MmParams {
  const bf16* x;
  const uint8_t* wq;
  const uint8_t* wscale;
  const float* tscale;
  const float* norm_w;
  const bf16* residual;
  void* y;
  float eps;
  int ldx, ldr, ldy, M, N, K;
  int phases, units_per_phase;                      // K = phases * units_per_phase * 512
};

struct MmBuf {                                      // one unit of one lane: 128 values of two rows + their scales
  uint4 a[4], b[4];
  uint2 sa, sb;
};

__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint2 ldg_stream_8b(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

template <int NT, int EPI>
__global__ void __launch_bounds__(MM_THREADS, 1)
gemv_nvfp4_mma_kernel(const MmParams p) {
  extern __shared__ __align__(16) unsigned char mm_smem[];
  __shared__ float s_rstd[16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int Sp = p.units_per_phase, Kp = Sp * MM_UNIT;
  const int ldxs = Kp + MM_XPAD;                              // f16 elements per staged activation row
  __half* xs = reinterpret_cast<__half*>(mm_smem);            // [NT * 8][ldxs], k permuted inside each 512-block
  float* part = reinterpret_cast<float*>(mm_smem + (size_t)NT * 8 * ldxs * sizeof(__half));   // [warp][slot][lane][NT * 4]
  const uint32_t xs_a = (uint32_t)__cvta_generic_to_shared(xs);
  pdl_launch_dependents(130);

  // this CTA's rows: a contiguous run of 8-row half tiles, walked as 16-row tiles from R0
  const int H = (p.N + 7) >> 3;
  const int h0 = (int)((long long)H * blockIdx.x / gridDim.x), h1 = (int)((long long)H * (blockIdx.x + 1) / gridDim.x);
  const int R0 = h0 * 8, R1 = min(p.N, h1 * 8);
  const int T = (R1 - R0 + 15) >> 4;
  const int tot = T * Sp;                                     // (tile, unit) pairs per phase
  const int ua = tot * warp / MM_WARPS, ub = tot * (warp + 1) / MM_WARPS;
  const int tile_first = ua / Sp;
  const size_t row_bytes = (size_t)p.K >> 1, srow_bytes = (size_t)p.K >> 4;

  auto load = [&](MmBuf& b, int phase, int u) {
    const int tile = u / Sp, ss = phase * Sp + (u - tile * Sp);
    const int ra = R0 + tile * 16 + 2 * g, rb = ra + 1;
    const size_t off = (size_t)ss * (MM_UNIT / 2) + t * 64, soff = (size_t)ss * (MM_UNIT / 16) + t * 8;
    if (ra < R1) {
      const uint8_t* w = p.wq + (size_t)ra * row_bytes + off;
#pragma unroll
      for (int q = 0; q < 4; ++q) b.a[q] = ldg_stream_16(w + 16 * q);
      b.sa = ldg_stream_8b(p.wscale + (size_t)ra * srow_bytes + soff);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) b.a[q] = make_uint4(0u, 0u, 0u, 0u);
      b.sa = make_uint2(0u, 0u);
    }
    if (rb < R1) {
      const uint8_t* w = p.wq + (size_t)rb * row_bytes + off;
#pragma unroll
      for (int q = 0; q < 4; ++q) b.b[q] = ldg_stream_16(w + 16 * q);
      b.sb = ldg_stream_8b(p.wscale + (size_t)rb * srow_bytes + soff);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) b.b[q] = make_uint4(0u, 0u, 0u, 0u);
      b.sb = make_uint2(0u, 0u);
    }
  };

  // ldmatrix row address of this lane inside a staged 512-block: lanes 0-7 rows of matrix 0 (chunk c),
  // 8-15 matrix 1 (chunk c + 1), 16-31 the same for activation rows 8..15 (second n-tile)
  const uint32_t x_lane = xs_a + (uint32_t)((((lane & 7) + (NT == 2 ? (lane >> 4) * 8 : 0)) * ldxs) * 2 + ((lane >> 3) & 1) * 16);

  // B fragments of one 16-byte weight piece: 8 MMAs x (2 | 4) registers, fetched one piece ahead of
  // their use so that the ldmatrix latency hides behind the decode and the MMAs of the piece before
  auto load_b = [&](uint32_t (&bf)[8][2 * NT], uint32_t xb, int u) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t addr = xb + (uint32_t)((u * 8 + i) * 2) * 16;
      if (NT == 1)
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(bf[i][0]), "=r"(bf[i][1]) : "r"(addr));
      else
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(bf[i][0]), "=r"(bf[i][1]), "=r"(bf[i][2 * NT - 2]), "=r"(bf[i][2 * NT - 1]) : "r"(addr));
    }
  };
  auto process = [&](const MmBuf& b, int ssl, float (&acc)[NT][4]) {
    const uint32_t sa2[4] = {cvt_e4m3x2_to_h2((uint16_t)(b.sa.x & 0xffffu)), cvt_e4m3x2_to_h2((uint16_t)(b.sa.x >> 16)),
                             cvt_e4m3x2_to_h2((uint16_t)(b.sa.y & 0xffffu)), cvt_e4m3x2_to_h2((uint16_t)(b.sa.y >> 16))};
    const uint32_t sb2[4] = {cvt_e4m3x2_to_h2((uint16_t)(b.sb.x & 0xffffu)), cvt_e4m3x2_to_h2((uint16_t)(b.sb.x >> 16)),
                             cvt_e4m3x2_to_h2((uint16_t)(b.sb.y & 0xffffu)), cvt_e4m3x2_to_h2((uint16_t)(b.sb.y >> 16))};
    const uint32_t xb = x_lane + (uint32_t)ssl * (MM_UNIT * 2);
    // four accumulators in rotation: consecutive MMAs do not wait for one another
    float a4[4][NT][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int i = 0; i < NT; ++i) a4[r][i][0] = a4[r][i][1] = a4[r][i][2] = a4[r][i][3] = 0.f;
    uint32_t bf[2][8][2 * NT];
    load_b(bf[0], xb, 0);
#pragma unroll
    for (int u = 0; u < 4; ++u) {                             // 16-byte piece u: values 32u .. 32u + 31, scales 2u, 2u + 1
      if (u + 1 < 4) load_b(bf[(u + 1) & 1], xb, u + 1);
      const uint32_t wa[4] = {b.a[u].x, b.a[u].y, b.a[u].z, b.a[u].w};
      const uint32_t wb[4] = {b.b[u].x, b.b[u].y, b.b[u].z, b.b[u].w};
      const uint32_t sal = __byte_perm(sa2[u], sa2[u], 0x1010), sah = __byte_perm(sa2[u], sa2[u], 0x3232);
      const uint32_t sbl = __byte_perm(sb2[u], sb2[u], 0x1010), sbh = __byte_perm(sb2[u], sb2[u], 0x3232);
#pragma unroll
      for (int j = 0; j < 4; ++j) {                           // word j: values 8j .. 8j + 7 of the piece
        uint32_t ha[4], hb[4];
        cvt_e2m1x8_to_h2x4(wa[j], ha);
        cvt_e2m1x8_to_h2x4(wb[j], hb);
        const uint32_t s_a = j < 2 ? sal : sah, s_b = j < 2 ? sbl : sbh;
#pragma unroll
        for (int q = 0; q < 4; ++q) ha[q] = hmul2_u(ha[q], s_a), hb[q] = hmul2_u(hb[q], s_b);
#pragma unroll
        for (int ii = 0; ii < 2; ++ii) {                      // MMA i = 2j + ii of the piece: values 4i .. 4i + 3
          const int i = j * 2 + ii;
          mma_f16(a4[i & 3][0], ha[2 * ii], hb[2 * ii], ha[2 * ii + 1], hb[2 * ii + 1], bf[u & 1][i][0], bf[u & 1][i][1]);
          if (NT == 2)
            mma_f16(a4[i & 3][NT - 1], ha[2 * ii], hb[2 * ii], ha[2 * ii + 1], hb[2 * ii + 1], bf[u & 1][i][2 * NT - 2],
                    bf[u & 1][i][2 * NT - 1]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][e] += (a4[0][i][e] + a4[1][i][e]) + (a4[2][i][e] + a4[3][i][e]);
  };

  // the first unit's weights do not depend on the previous kernel
  MmBuf nxt;
  if (ua < ub) load(nxt, 0, ua);
  pdl_wait();

  // 1 / rms of every activation row (warp per row)
  for (int m = warp; m < NT * 8; m += MM_WARPS) {
    float rstd = 1.f;
    if (m < p.M && p.norm_w != nullptr) {
      float ss = 0.f;
      const bf16* xr = p.x + (size_t)m * p.ldx;
      for (int k = lane * 8; k < p.K; k += 256) {
        const uint4 v = *reinterpret_cast<const uint4*>(xr + k);
        const float2 a = bf162_bits_to_f2(v.x), b2 = bf162_bits_to_f2(v.y), c = bf162_bits_to_f2(v.z), d = bf162_bits_to_f2(v.w);
        ss += a.x * a.x + a.y * a.y + b2.x * b2.x + b2.y * b2.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
      }
      ss = warp_sum(ss);
      rstd = rsqrtf(ss / (float)p.K + p.eps);
    }
    if (lane == 0) s_rstd[m] = rstd;
  }
  __syncthreads();

  float acc[MM_SLOTS][NT][4];
#pragma unroll
  for (int s = 0; s < MM_SLOTS; ++s)
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[s][i][0] = acc[s][i][1] = acc[s][i][2] = acc[s][i][3] = 0.f;

  for (int phase = 0; phase < p.phases; ++phase) {
    if (phase > 0) __syncthreads();                            // every warp is done with the staged rows of the phase before
    // stage rows [k0, k0 + Kp) of the activations: normalised, rounded to bf16 like the oracle's rows,
    // scaled by 1/16 into f16 (saturating), k permuted inside each 512-block
    const int k0 = phase * Kp, oct = Kp >> 3;
#pragma unroll 2
    for (int idx = threadIdx.x; idx < NT * 8 * oct; idx += MM_THREADS) {
      const int m = idx / oct, kk = (idx - m * oct) * 8;          // 8 consecutive k: MMAs i, i + 1 of one (lane, piece)
      uint32_t packed[4] = {0u, 0u, 0u, 0u};
      if (m < p.M) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + k0 + kk);
        const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
        float nwv[8];
        float r = 1.f;
        if (p.norm_w != nullptr) {
          const float4 n0 = *reinterpret_cast<const float4*>(p.norm_w + k0 + kk);
          const float4 n1 = *reinterpret_cast<const float4*>(p.norm_w + k0 + kk + 4);
          nwv[0] = n0.x, nwv[1] = n0.y, nwv[2] = n0.z, nwv[3] = n0.w, nwv[4] = n1.x, nwv[5] = n1.y, nwv[6] = n1.z, nwv[7] = n1.w;
          r = s_rstd[m];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 v = bf162_bits_to_f2(rw[q]);
          if (p.norm_w != nullptr) v = bf162_bits_to_f2(f2_to_bf162_bits(v.x * r * nwv[2 * q], v.y * r * nwv[2 * q + 1]));
          asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(packed[q]) : "f"(v.y * MM_PRESCALE), "f"(v.x * MM_PRESCALE));
        }
      }
      const int blk = kk >> 9, r5 = kk & 511;
      const int pt = r5 >> 7, pu = (r5 >> 5) & 3, pi = (r5 >> 2) & 7;     // pi is even: this thread fills MMAs pi and pi + 1
      __half* dst = xs + (size_t)m * ldxs + (blk << 9) + (pt << 1);
#pragma unroll
      for (int q = 0; q < 4; ++q)                                  // q = 2 * (MMA within the pair) + h
        *reinterpret_cast<uint32_t*>(dst + ((((pu * 8 + pi + (q >> 1)) * 2 + (q & 1)) * 4) << 1)) = packed[q];
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < MM_SLOTS; ++s) {
      const int tile = tile_first + s;
      const int lo = max(ua, tile * Sp), hi = min(ub, (tile + 1) * Sp);
      for (int u = lo; u < hi; ++u) {
        const MmBuf cur = nxt;
        if (u + 1 < ub) load(nxt, phase, u + 1);
        else if (phase + 1 < p.phases) load(nxt, phase + 1, ua);
        process(cur, u - tile * Sp, acc[s]);
      }
    }
  }

  // partial tiles meet in shared memory, summed in warp order by the warp that owns the tile
#pragma unroll
  for (int s = 0; s < MM_SLOTS; ++s) {
    const int tile = tile_first + s;
    if (max(ua, tile * Sp) < min(ub, (tile + 1) * Sp)) {
      float* dst = part + ((size_t)(warp * MM_SLOTS + s) * 32 + lane) * (NT * 4);
#pragma unroll
      for (int i = 0; i < NT; ++i)
        *reinterpret_cast<float4*>(dst + i * 4) = make_float4(acc[s][i][0], acc[s][i][1], acc[s][i][2], acc[s][i][3]);
    }
  }
  __syncthreads();
  const float fs = (1.f / MM_PRESCALE) * p.tscale[0];
  for (int tile = warp; tile < T; tile += MM_WARPS) {
    float sum[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) sum[i][0] = sum[i][1] = sum[i][2] = sum[i][3] = 0.f;
    for (int w2 = 0; w2 < MM_WARPS; ++w2) {
      const int ua2 = tot * w2 / MM_WARPS, ub2 = tot * (w2 + 1) / MM_WARPS;
      const int s2 = tile - ua2 / Sp;
      if (s2 < 0 || s2 >= MM_SLOTS || max(ua2, tile * Sp) >= min(ub2, (tile + 1) * Sp)) continue;
      const float* src = part + ((size_t)(w2 * MM_SLOTS + s2) * 32 + lane) * (NT * 4);
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(src + i * 4);
        sum[i][0] += v.x, sum[i][1] += v.y, sum[i][2] += v.z, sum[i][3] += v.w;
      }
    }
    // fragment: (weight row 2g | 2g + 1 of the tile) x (activation rows 2t, 2t + 1 of n-tile i)
    const int ra = R0 + tile * 16 + 2 * g, rb = ra + 1;
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = i * 8 + 2 * t + e;
        if (tok >= p.M || ra >= R1) continue;
        float va = sum[i][e] * fs, vb = sum[i][2 + e] * fs;
        if (EPI == ME_SWIGLU) {
          if (rb < R1) reinterpret_cast<bf16*>(p.y)[(size_t)tok * p.ldy + (ra >> 1)] = __float2bfloat16(silu_f(va) * vb);
          continue;
        }
        if (EPI == ME_RESIDUAL) {
          va += __bfloat162float(p.residual[(size_t)tok * p.ldr + ra]);
          if (rb < R1) vb += __bfloat162float(p.residual[(size_t)tok * p.ldr + rb]);
        }
        if (EPI == ME_STORE_F32) {
          reinterpret_cast<float*>(p.y)[(size_t)tok * p.ldy + ra] = va;
          if (rb < R1) reinterpret_cast<float*>(p.y)[(size_t)tok * p.ldy + rb] = vb;
        } else {
          reinterpret_cast<bf16*>(p.y)[(size_t)tok * p.ldy + ra] = __float2bfloat16(va);
          if (rb < R1) reinterpret_cast<bf16*>(p.y)[(size_t)tok * p.ldy + rb] = __float2bfloat16(vb);
        }
      }
  }
}

}  // namespace

// y = epi(norm(x) @ dequant(W)^T) for 3..16 rows.  x [M, K] bf16 (16-byte aligned rows), wq [N, K/2] packed e2m1,
// wscale [N, K/16] e4m3, tscale fp32[1].  epi: 0 store bf16, 1 + residual, 2 SwiGLU over interleaved (gate, up)
// rows -> y [M, N/2], 3 store fp32.  K % 512 == 0.  Returns cudaErrorNotSupported for shapes it does not
// take (the caller then uses the quantiser + tcgen05 GEMM).
TRL_API int trl_gemv_nvfp4_mma(const void* x, int ldx, const void* wq, const void* wscale, const void* tscale,
                               const void* norm_w, float eps, const void* residual, int ldr, void* y, int ldy, int M,
                               int N, int K, int epi, void* stream) {
  if (M < 1 || M > 16 || N <= 0 || K <= 0 || epi < 0 || epi > 3) return (int)cudaErrorInvalidValue;
  if (K % MM_UNIT != 0 || ldx % 8 != 0 || ((uintptr_t)x & 15) || (epi == ME_SWIGLU && N % 2 != 0))
    return (int)cudaErrorNotSupported;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int nt = M <= 8 ? 1 : 2;
  const int H = (N + 7) / 8, grid = H < sms ? H : sms;
  const int max_rows = 8 * ((H + grid - 1) / grid);
  if ((max_rows + 15) / 16 > 16) return (int)cudaErrorNotSupported;     // a warp's share must span at most three tiles
  const int units = K / MM_UNIT;
  int phases = 0;
  for (int d = 1; d <= units; ++d)
    if (units % d == 0 && (size_t)nt * 8 * (K / d + MM_XPAD) * 2 <= (size_t)MM_XS_BYTES) {
      phases = d;
      break;
    }
  if (phases == 0) return (int)cudaErrorNotSupported;
  MmParams p;
  p.x = (const bf16*)x, p.wq = (const uint8_t*)wq, p.wscale = (const uint8_t*)wscale, p.tscale = (const float*)tscale;
  p.norm_w = (const float*)norm_w, p.residual = (const bf16*)residual, p.y = y, p.eps = eps;
  p.ldx = ldx, p.ldr = ldr, p.ldy = ldy, p.M = M, p.N = N, p.K = K, p.phases = phases, p.units_per_phase = units / phases;
  const size_t smem = (size_t)nt * 8 * (K / phases + MM_XPAD) * 2 + (size_t)MM_WARPS * MM_SLOTS * 32 * nt * 4 * sizeof(float);
  cudaError_t e = cudaErrorInvalidValue;
#define MM_CASE(NTT, EP)                                                                           \
  if (nt == NTT && epi == EP) {                                                                    \
    auto kern = gemv_nvfp4_mma_kernel<NTT, EP>;                                                    \
    static bool configured = false;                                                                \
    if (!configured) {                                                                             \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return 3; \
      configured = true;                                                                           \
    }                                                                                              \
    e = trl_launch(kern, dim3(grid), dim3(MM_THREADS), smem, (cudaStream_t)stream, p);             \
  }
  MM_CASE(1, ME_STORE) MM_CASE(1, ME_RESIDUAL) MM_CASE(1, ME_SWIGLU) MM_CASE(1, ME_STORE_F32)
  MM_CASE(2, ME_STORE) MM_CASE(2, ME_RESIDUAL) MM_CASE(2, ME_SWIGLU) MM_CASE(2, ME_STORE_F32)
#undef MM_CASE
  return (int)e;
}
