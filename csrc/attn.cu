// Gated GQA attention over the paged KV pool.
//
//   attn_prep   : fused q/k per-head RMSNorm (fp32) + partial RoPE + paged K/V write,
//                 straight off the fused qkv projection row
//                 [hq x (query D ; gate D)] ++ [hkv x D] ++ [hkv x D].
//   attn_split  : flash-decoding style split-KV attention.  One CTA = (kv split,
//                 kv head, token); its warps walk the keys of the split, each key's
//                 row is one coalesced 16-byte-per-lane load, the G query heads of
//                 the group share every K/V load.  Causal by absolute position, so
//                 the same kernel serves decode (1 token), speculative verify
//                 (W tokens of one sequence) and prefill chunks.
//   attn_combine: merges the split partials, applies the sigmoid output gate and
//                 writes bf16 [T, hq*D].  With one split the split kernel writes
//                 the final output itself.
//
// Pool layout: [blocks, hkv, 16, D] bf16 per layer; block_table [B, max_blocks].
// Reference parity: kernels_mma.py:168-366 (attn_prep), kernels_attn.py:151-334
// (split decode + combine) of packages/tilerl-kernels/src/tilerl_kernels.
#include "common.cuh"

namespace {

constexpr int KVB = 16;
constexpr int MAXG = 8;

__global__ void __launch_bounds__(256)
attn_prep_kernel(const bf16* __restrict__ qkv, int ld, const float* __restrict__ qw,
                 const float* __restrict__ kw, const int* __restrict__ positions,
                 const int* __restrict__ slot_mapping, bf16* __restrict__ q_out,
                 bf16* __restrict__ kcache, bf16* __restrict__ vcache, int n_q, int n_kv, int D,
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
  // heads 0..n_q-1 = q, n_q..n_q+n_kv-1 = k, then v
  for (int h = warp; h < n_q + 2 * n_kv; h += nw) {
    const bool is_q = h < n_q, is_k = !is_q && h < n_q + n_kv;
    const bf16* src = is_q ? row + (size_t)h * per_q
                           : row + (size_t)n_q * per_q + (size_t)(h - n_q) * D;
    bf16* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * n_q + h) * D;
    } else {
      if (slot < 0) continue;
      const int kvh = is_k ? h - n_q : h - n_q - n_kv;
      bf16* cache = is_k ? kcache : vcache;
      dst = cache + (((size_t)(slot / KVB) * n_kv + kvh) * KVB + (slot % KVB)) * D;
    }
    if (!is_q && !is_k) {  // v: plain copy
      for (int d = lane; d < D; d += 32) dst[d] = src[d];
      continue;
    }
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float v = __bfloat162float(src[d]);
      hb[d] = v;
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
    const float* w = is_q ? qw : kw;
    __syncwarp();
    for (int d = lane; d < D; d += 32) hb[d] = hb[d] * rstd * w[d];
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
      float v = hb[d];
      if (d < half)
        v = hb[d] * cs[d] - hb[d + half] * sn[d];
      else if (d < rotary)
        v = hb[d] * cs[d - half] + hb[d - half] * sn[d - half];
      dst[d] = __float2bfloat16(v);
    }
    __syncwarp();
  }
}

// One CTA per (split, kv head, token).  VEC = D / 32 elements per lane.
template <int VEC>
__global__ void __launch_bounds__(256)
attn_split_kernel(const bf16* __restrict__ q, const bf16* __restrict__ gate_src, int gate_ld,
                  const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                  const int* __restrict__ block_table, int max_blocks,
                  const int* __restrict__ seq_ids, const int* __restrict__ positions,
                  float* __restrict__ po, float* __restrict__ pm, float* __restrict__ pl,
                  bf16* __restrict__ out, int n_q, int n_kv, int n_splits, float scale_log2e,
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
  // split boundaries on page granularity
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
    const size_t off = (((size_t)blk * n_kv + kvh) * KVB + (j % KVB)) * D + lane * VEC;
    float kf[VEC], vf[VEC];
    if (VEC == 8) {
      const uint4 kk = *reinterpret_cast<const uint4*>(kcache + off);
      const uint4 vv = *reinterpret_cast<const uint4*>(vcache + off);
      const uint32_t ku[4] = {kk.x, kk.y, kk.z, kk.w}, vu[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 a = bf162_bits_to_f2(ku[i]), b = bf162_bits_to_f2(vu[i]);
        kf[2 * i] = a.x, kf[2 * i + 1] = a.y, vf[2 * i] = b.x, vf[2 * i + 1] = b.y;
      }
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        kf[v] = __bfloat162float(kcache[off + v]);
        vf[v] = __bfloat162float(vcache[off + v]);
      }
    }
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
      if (g < G) {
        float s = 0.f;
#pragma unroll
        for (int v = 0; v < VEC; ++v) s = fmaf(qr[g][v], kf[v], s);
        s = warp_sum(s);
        const float mn = fmaxf(m[g], s);
        const float corr = exp2f(m[g] - mn), p = exp2f(s - mn);
        l[g] = l[g] * corr + p;
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[g][v] = fmaf(acc[g][v], corr, p * vf[v]);
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
attn_combine_kernel(const float* __restrict__ po, const float* __restrict__ pm,
                    const float* __restrict__ pl, const bf16* __restrict__ gate_src, int gate_ld,
                    bf16* __restrict__ out, int n_q, int D, int n_splits, int gated) {
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

TRL_API int trl_attn_prep(const void* qkv, int ld, const void* q_norm, const void* k_norm,
                          const void* positions, const void* slot_mapping, void* q_out, void* kcache,
                          void* vcache, int T, int n_q, int n_kv, int D, int rotary, float theta,
                          float eps, int gated, void* stream) {
  const int threads = 256;
  const size_t smem = (size_t)(rotary + (threads / 32) * D) * sizeof(float);
  return (int)trl_launch(attn_prep_kernel, dim3(T), dim3(threads), smem, (cudaStream_t)stream,
                         (const bf16*)qkv, ld, (const float*)q_norm, (const float*)k_norm,
                         (const int*)positions, (const int*)slot_mapping, (bf16*)q_out, (bf16*)kcache,
                         (bf16*)vcache, n_q, n_kv, D, rotary, log2f(theta), eps, gated);
}

// Scratch: po [T*n_q*n_splits*D] fp32, pm/pl [T*n_q*n_splits] fp32 (unused when n_splits == 1).
TRL_API int trl_attn_paged(const void* q, const void* gate_src, int gate_ld, const void* kcache,
                           const void* vcache, const void* block_table, int max_blocks,
                           const void* seq_ids, const void* positions, void* po, void* pm, void* pl,
                           void* out, int T, int n_q, int n_kv, int D, int n_splits, float scale,
                           int gated, void* stream) {
  if (n_q % n_kv != 0 || n_q / n_kv > MAXG) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  const float sl2 = scale * 1.4426950408889634f;
  const dim3 grid(n_splits, n_kv, T);
  const size_t smem = (size_t)8 * MAXG * D * sizeof(float);
  cudaError_t e;
#define SPLIT_CASE(V)                                                                              \
  {                                                                                                \
    auto kern = attn_split_kernel<V>;                                                              \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    e = trl_launch(kern, grid, dim3(256), smem, st, (const bf16*)q, (const bf16*)gate_src, gate_ld, \
                   (const bf16*)kcache, (const bf16*)vcache, (const int*)block_table, max_blocks,  \
                   (const int*)seq_ids, (const int*)positions, (float*)po, (float*)pm, (float*)pl, \
                   (bf16*)out, n_q, n_kv, n_splits, sl2, gated);                                   \
  }
  if (D == 256) SPLIT_CASE(8)
  else if (D == 128) SPLIT_CASE(4)
  else if (D == 64) SPLIT_CASE(2)
  else return (int)cudaErrorInvalidValue;
#undef SPLIT_CASE
  if (e != cudaSuccess) return (int)e;
  if (n_splits > 1)
    e = trl_launch(attn_combine_kernel, dim3(T, n_q), dim3(min(D, 256)), 0, st, (const float*)po,
                   (const float*)pm, (const float*)pl, (const bf16*)gate_src, gate_ld, (bf16*)out, n_q,
                   D, n_splits, gated);
  return (int)e;
}

// ---- allocation-free variant (declared in attn_static.h) --------------------------------------
#include "attn_static.h"

// Scratch for the split partials of trl_attn_paged_static.  In host code this name is only a
// stand-in for the symbol, not a device address: the address is fetched per device below.
static __device__ __align__(256) unsigned char g_attn_static_scratch[TRL_ATTN_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {nullptr};
}  // namespace

TRL_API size_t trl_attn_static_scratch_needed(int T, int n_q, int D, int n_splits) {
  return (size_t)T * n_q * n_splits * ((size_t)D + 2) * sizeof(float);
}

TRL_API int trl_attn_paged_static(const void* q, const void* gate_src, int gate_ld, const void* kcache,
                                  const void* vcache, const void* block_table, int max_blocks,
                                  const void* seq_ids, const void* positions, void* out, int T, int n_q,
                                  int n_kv, int D, int n_splits, float scale, int gated, void* stream) {
  if (T <= 0 || n_q <= 0 || n_splits <= 0 || D <= 0) return (int)cudaErrorInvalidValue;
  const size_t need = trl_attn_static_scratch_needed(T, n_q, D, n_splits);
  if (need > (size_t)TRL_ATTN_STATIC_SCRATCH_BYTES) return (int)cudaErrorInvalidValue;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  if (g_static_scratch_ptr[dev] == nullptr) {
    // once per device, with that device current: the symbol's address on THIS device
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
    if (e != cudaSuccess) return (int)e;
    g_static_scratch_ptr[dev] = p;
  }
  float* po = reinterpret_cast<float*>(g_static_scratch_ptr[dev]);
  float* pm = po + (size_t)T * n_q * n_splits * D;
  float* pl = pm + (size_t)T * n_q * n_splits;
  return trl_attn_paged(q, gate_src, gate_ld, kcache, vcache, block_table, max_blocks, seq_ids, positions, po,
                        pm, pl, out, T, n_q, n_kv, D, n_splits, scale, gated, stream);
}
