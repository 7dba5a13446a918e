// Gated GQA attention over an fp8 (e4m3) paged KV pool.
//
// Pool layout per layer: values [blocks, hkv, 16, D] e4m3, scales [blocks, hkv, 16] fp32 with
// scale = amax(|row|) / 448 over the head dim of one (token, kv head); K is quantised after
// RoPE.  The pool holds half the bytes of the bf16 pool, so a decode tick at long context reads
// half as much and twice the context fits.
//
//   attn_prep_fp8  : q/k per-head RMSNorm + partial RoPE, normalised Q out in bf16, K / V rows
//                    quantised and scattered with their scales (one warp per head).
//   attn_split_fp8 : the split-KV kernel of attn.cu reading e4m3 rows (one 8-byte load per lane
//                    at D = 256) and folding the row scales into the score and into p * V.
//   attn_combine   : merge of the split partials + sigmoid gate (same maths as the bf16 path).
//
// Reference parity: kernels_mma.py:89-166,247-366 (fp8 write / attn_prep_fp8) and the `_fp8`
// variants of kernels_attn.py:151-334 of packages/tilerl-kernels/src/tilerl_kernels; format
// definition reference.py:382-402.
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

constexpr int KVB = 16;
constexpr int MAXG = 8;
constexpr float E4M3_MAX = 448.f;

__device__ __forceinline__ unsigned char to_e4m3(float v) {
  return (unsigned char)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

__global__ void __launch_bounds__(256)
attn_prep_fp8_kernel(const bf16* qkv, int ld, const float* __restrict__ qw,
                     const float* __restrict__ kw, const int* positions,
                     const int* slot_mapping, bf16* q_out,
                     unsigned char* kcache, unsigned char* vcache,
                     float* kscale, float* vscale, int n_q, int n_kv, int D,
                     int rotary, float log2_theta, float eps, int gated) {
  extern __shared__ float sm[];
  float* cs = sm;                 // [rotary/2] cos
  float* sn = sm + rotary / 2;    // [rotary/2] sin
  float* buf = sn + rotary / 2;   // [warps][D]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int pos = positions[t];
  const int half = rotary >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const double inv = exp2(-(double)(2 * i) / (double)rotary * (double)log2_theta);
    double s, c;
    sincos((double)pos * inv, &s, &c);
    cs[i] = (float)c, sn[i] = (float)s;
  }
  __syncthreads();
  const bf16* row = qkv + (size_t)t * ld;
  const int per_q = gated ? 2 * D : D;
  const int slot = slot_mapping[t];
  float* hb = buf + (size_t)warp * D;
  for (int h = warp; h < n_q + 2 * n_kv; h += nw) {
    const bool is_q = h < n_q, is_k = !is_q && h < n_q + n_kv;
    const bf16* src = is_q ? row + (size_t)h * per_q
                           : row + (size_t)n_q * per_q + (size_t)(h - n_q) * D;
    if (!is_q && slot < 0) continue;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float v = __bfloat162float(src[d]);
      hb[d] = v;
      ss += v * v;
    }
    __syncwarp();
    if (is_q || is_k) {
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / (float)D + eps);
      const float* w = is_q ? qw : kw;
      for (int d = lane; d < D; d += 32) hb[d] = hb[d] * rstd * w[d];
      __syncwarp();
      // rotate in place: each lane reads the pair it needs before anyone overwrites it
      for (int d = lane; d < half; d += 32) {
        const float a = hb[d], b = hb[d + half];
        hb[d] = a * cs[d] - b * sn[d];
        hb[d + half] = b * cs[d] + a * sn[d];
      }
      __syncwarp();
    }
    if (is_q) {
      bf16* dst = q_out + ((size_t)t * n_q + h) * D;
      for (int d = lane; d < D; d += 32) dst[d] = __float2bfloat16(hb[d]);
    } else {
      const int kvh = is_k ? h - n_q : h - n_q - n_kv;
      const size_t ridx = ((size_t)(slot / KVB) * n_kv + kvh) * KVB + (slot % KVB);
      float amax = 0.f;
      for (int d = lane; d < D; d += 32) amax = fmaxf(amax, fabsf(hb[d]));
      amax = warp_max(amax);
      const float sc = fmaxf(amax, 1e-30f) / E4M3_MAX;
      unsigned char* dst = (is_k ? kcache : vcache) + ridx * D;
      for (int d = lane; d < D; d += 32) dst[d] = to_e4m3(hb[d] / sc);
      if (lane == 0) (is_k ? kscale : vscale)[ridx] = sc;
    }
    __syncwarp();
  }
}

template <int VEC>
__device__ __forceinline__ void load_e4m3_row(const unsigned char* p, float (&f)[VEC]) {
  if constexpr (VEC == 8) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    const uint32_t u[2] = {w.x, w.y};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 a = h2_to_f2(cvt_e4m3x2_to_h2((uint16_t)(u[i] & 0xFFFFu)));
      const float2 b = h2_to_f2(cvt_e4m3x2_to_h2((uint16_t)(u[i] >> 16)));
      f[4 * i] = a.x, f[4 * i + 1] = a.y, f[4 * i + 2] = b.x, f[4 * i + 3] = b.y;
    }
  } else if constexpr (VEC == 4) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(p);
    const float2 a = h2_to_f2(cvt_e4m3x2_to_h2((uint16_t)(u & 0xFFFFu)));
    const float2 b = h2_to_f2(cvt_e4m3x2_to_h2((uint16_t)(u >> 16)));
    f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
  } else {
    static_assert(VEC == 2, "head dim must be 64, 128 or 256");
    const float2 a = h2_to_f2(cvt_e4m3x2_to_h2(*reinterpret_cast<const uint16_t*>(p)));
    f[0] = a.x, f[1] = a.y;
  }
}

// One CTA per (split, kv head, token).  VEC = D / 32 elements per lane.
template <int VEC>
__global__ void __launch_bounds__(256)
attn_split_fp8_kernel(const bf16* q, const bf16* gate_src, int gate_ld,
                      const unsigned char* kcache, const unsigned char* vcache,
                      const float* kscale, const float* vscale,
                      const int* block_table, int max_blocks,
                      const int* seq_ids, const int* positions,
                      float* po, float* pm, float* pl,
                      bf16* out, int n_q, int n_kv, int n_splits, float scale_log2e,
                      int gated) {
  constexpr int D = VEC * 32;
  __shared__ float s_m[8][MAXG], s_l[8][MAXG];
  extern __shared__ float s_acc[];  // [8 warps][MAXG][D]
  pdl_launch_dependents();
  pdl_wait();
  const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = n_q / n_kv;
  const int pos = positions[t];
  const int kv_len = pos + 1;
  const int* table = block_table + (size_t)seq_ids[t] * max_blocks;
  const int pages = (kv_len + KVB - 1) / KVB;
  const int pps = (pages + n_splits - 1) / n_splits;
  const int lo = split * pps * KVB, hi = min(kv_len, (split + 1) * pps * KVB);

  float qr[MAXG][VEC];
#pragma unroll
  for (int g = 0; g < MAXG; ++g) {
    if (g < G) {
      const bf16* qp = q + ((size_t)t * n_q + kvh * G + g) * D + lane * VEC;
#pragma unroll
      for (int v = 0; v < VEC; ++v) qr[g][v] = __bfloat162float(qp[v]) * scale_log2e;
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) qr[g][v] = 0.f;
    }
  }
  float m[MAXG], l[MAXG], acc[MAXG][VEC];
#pragma unroll
  for (int g = 0; g < MAXG; ++g) {
    m[g] = -INFINITY, l[g] = 0.f;
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[g][v] = 0.f;
  }
  for (int j = lo + warp; j < hi; j += 8) {
    const int blk = table[j / KVB];
    const size_t ridx = ((size_t)blk * n_kv + kvh) * KVB + (j % KVB);
    const size_t off = ridx * D + lane * VEC;
    float kf[VEC], vf[VEC];
    load_e4m3_row<VEC>(kcache + off, kf);
    load_e4m3_row<VEC>(vcache + off, vf);
    const float ks = kscale[ridx], vs = vscale[ridx];
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
      if (g < G) {
        float s = 0.f;
#pragma unroll
        for (int v = 0; v < VEC; ++v) s = fmaf(qr[g][v], kf[v], s);
        s = warp_sum(s) * ks;
        const float mn = fmaxf(m[g], s);
        const float corr = exp2f(m[g] - mn), p = exp2f(s - mn);
        l[g] = l[g] * corr + p;
        const float pv = p * vs;
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[g][v] = fmaf(acc[g][v], corr, pv * vf[v]);
        m[g] = mn;
      }
    }
  }
  // merge the 8 warps
#pragma unroll
  for (int g = 0; g < MAXG; ++g) {
    if (g < G) {
      if (lane == 0) s_m[warp][g] = m[g], s_l[warp][g] = l[g];
#pragma unroll
      for (int v = 0; v < VEC; ++v) s_acc[((size_t)warp * MAXG + g) * D + lane * VEC + v] = acc[g][v];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float c = (s_m[w][g] == -INFINITY) ? 0.f : exp2f(s_m[w][g] - mm);
      ll += s_l[w][g] * c;
      a += s_acc[((size_t)w * MAXG + g) * D + d] * c;
    }
    const int h = kvh * G + g;
    if (n_splits == 1) {
      float o = ll > 0.f ? a / ll : 0.f;
      if (gated) o *= sigmoid_f(__bfloat162float(gate_src[(size_t)t * gate_ld + (size_t)h * 2 * D + D + d]));
      out[((size_t)t * n_q + h) * D + d] = __float2bfloat16(o);
    } else {
      const size_t base = ((size_t)t * n_q + h) * n_splits + split;
      po[base * D + d] = a;
      if (d == 0) pm[base] = mm, pl[base] = ll;
    }
  }
}

__global__ void __launch_bounds__(256)
attn_combine_fp8_kernel(const float* po, const float* pm,
                        const float* pl, const bf16* gate_src, int gate_ld,
                        bf16* out, int n_q, int D, int n_splits, int gated) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const size_t base = ((size_t)t * n_q + h) * n_splits;
  float mm = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, pm[base + s]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float ll = 0.f, a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = pm[base + s];
      const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
      ll += pl[base + s] * c;
      a += po[(base + s) * D + d] * c;
    }
    float o = ll > 0.f ? a / ll : 0.f;
    if (gated) o *= sigmoid_f(__bfloat162float(gate_src[(size_t)t * gate_ld + (size_t)h * 2 * D + D + d]));
    out[((size_t)t * n_q + h) * D + d] = __float2bfloat16(o);
  }
}

}  // namespace

// kcache / vcache: e4m3 bytes of one layer; kscale / vscale: its fp32 row scales.
TRL_API int trl_attn_prep_fp8(const void* qkv, int ld, const void* q_norm, const void* k_norm,
                              const void* positions, const void* slot_mapping, void* q_out, void* kcache,
                              void* vcache, void* kscale, void* vscale, int T, int n_q, int n_kv, int D,
                              int rotary, float theta, float eps, int gated, void* stream) {
  const int threads = 256;
  if (rotary > D || (rotary & 1)) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)(rotary + (threads / 32) * D) * sizeof(float);
  return (int)trl_launch(attn_prep_fp8_kernel, dim3(T), dim3(threads), smem, (cudaStream_t)stream,
                         (const bf16*)qkv, ld, (const float*)q_norm, (const float*)k_norm,
                         (const int*)positions, (const int*)slot_mapping, (bf16*)q_out,
                         (unsigned char*)kcache, (unsigned char*)vcache, (float*)kscale, (float*)vscale, n_q,
                         n_kv, D, rotary, log2f(theta), eps, gated);
}

// Scratch as for the bf16 split kernel: po [T*n_q*n_splits*D] fp32, pm/pl [T*n_q*n_splits] fp32.
TRL_API int trl_attn_paged_fp8(const void* q, const void* gate_src, int gate_ld, const void* kcache,
                               const void* vcache, const void* kscale, const void* vscale,
                               const void* block_table, int max_blocks, const void* seq_ids,
                               const void* positions, void* po, void* pm, void* pl, void* out, int T, int n_q,
                               int n_kv, int D, int n_splits, float scale, int gated, void* stream) {
  if (n_q % n_kv != 0 || n_q / n_kv > MAXG) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  const float sl2 = scale * 1.4426950408889634f;
  const dim3 grid(n_splits, n_kv, T);
  const size_t smem = (size_t)8 * MAXG * D * sizeof(float);
  cudaError_t e;
#define SPLIT_CASE(V)                                                                                 \
  {                                                                                                   \
    auto kern = attn_split_fp8_kernel<V>;                                                             \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);               \
    e = trl_launch(kern, grid, dim3(256), smem, st, (const bf16*)q, (const bf16*)gate_src, gate_ld,   \
                   (const unsigned char*)kcache, (const unsigned char*)vcache, (const float*)kscale,  \
                   (const float*)vscale, (const int*)block_table, max_blocks, (const int*)seq_ids,    \
                   (const int*)positions, (float*)po, (float*)pm, (float*)pl, (bf16*)out, n_q, n_kv,  \
                   n_splits, sl2, gated);                                                             \
  }
  if (D == 256) SPLIT_CASE(8)
  else if (D == 128) SPLIT_CASE(4)
  else if (D == 64) SPLIT_CASE(2)
  else return (int)cudaErrorInvalidValue;
#undef SPLIT_CASE
  if (e != cudaSuccess) return (int)e;
  if (n_splits > 1)
    e = trl_launch(attn_combine_fp8_kernel, dim3(T, n_q), dim3(min(D, 256)), 0, st, (const float*)po,
                   (const float*)pm, (const float*)pl, (const bf16*)gate_src, gate_ld, (bf16*)out, n_q, D,
                   n_splits, gated);
  return (int)e;
}
