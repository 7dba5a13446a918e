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
#include <cuda.h>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace {

constexpr int KVB = 16;
constexpr int MAXG = 8;
constexpr int COMBINE_SPLITS = 64;     // splits whose (max, denominator) the combine kernel stages in shared memory

__global__ void __launch_bounds__(256)
attn_prep_kernel(const bf16* qkv, int ld, const float* __restrict__ qw,
                 const float* __restrict__ kw, const int* positions,
                 const int* slot_mapping, bf16* q_out,
                 bf16* kcache, bf16* vcache, int n_q, int n_kv, int D,
                 int rotary, float log2_theta, float eps, int gated, int n_slots) {
  extern __shared__ float sm[];
  float* cs = sm;                 // [rotary/2] cos
  float* sn = sm + rotary / 2;    // [rotary/2] sin
  float* buf = sn + rotary / 2;   // [warps][D]
  pdl_launch_dependents(3);
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
  int slot = slot_mapping[t];
  if (slot >= 0) slot = trl_checked(slot, n_slots, 1);
  float* hb = buf + (size_t)warp * D;
  // heads 0..n_q-1 = q, n_q..n_q+n_kv-1 = k, then v; CTA blockIdx.y takes heads [y * nw, (y + 1) * nw):
  // a decode tick's single token is spread over several CTAs instead of one walking 32 heads
  for (int h = blockIdx.y * nw + warp; h < min(n_q + 2 * n_kv, ((int)blockIdx.y + 1) * nw); h += nw) {
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
attn_split_kernel(const bf16* q, const bf16* gate_src, int gate_ld,
                  const bf16* kcache, const bf16* vcache,
                  const int* block_table, int max_blocks,
                  const int* seq_ids, const int* positions,
                  float* po, float* pm, float* pl,
                  bf16* out, int n_q, int n_kv, int n_splits, float scale_log2e,
                  int gated) {
  constexpr int D = VEC * 32;
  __shared__ float s_m[8][MAXG], s_l[8][MAXG];
  extern __shared__ float s_acc[];  // [8 warps][MAXG][D]
  pdl_launch_dependents(4);
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
  // K / V rows of this warp's next key are requested while the current key is processed
  auto row_off = [&](int j) {
    const int blk = table[j / KVB];
    return (((size_t)blk * n_kv + kvh) * KVB + (j % KVB)) * D + lane * VEC;
  };
  uint4 kk_n = make_uint4(0u, 0u, 0u, 0u), vv_n = kk_n;
  if (VEC == 8 && lo + warp < hi) {
    const size_t o0 = row_off(lo + warp);
    kk_n = *reinterpret_cast<const uint4*>(kcache + o0);
    vv_n = *reinterpret_cast<const uint4*>(vcache + o0);
  }
  for (int j = lo + warp; j < hi; j += 8) {
    const size_t off = row_off(j);
    float kf[VEC], vf[VEC];
    if (VEC == 8) {
      const uint4 kk = kk_n, vv = vv_n;
      if (j + 8 < hi) {
        const size_t o1 = row_off(j + 8);
        kk_n = *reinterpret_cast<const uint4*>(kcache + o1);
        vv_n = *reinterpret_cast<const uint4*>(vcache + o1);
      }
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
attn_combine_kernel(const float* po, const float* pm,
                    const float* pl, const bf16* gate_src, int gate_ld,
                    bf16* out, int n_q, int D, int n_splits, int gated) {
  __shared__ float s_pm[COMBINE_SPLITS], s_pl[COMBINE_SPLITS];
  pdl_launch_dependents(5);
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const size_t base = ((size_t)t * n_q + h) * n_splits;
  // (max, denominator) of every split once per CTA; the partial rows then come eight loads at a
  // time, and splits that saw no key (max = -inf) are not read at all
  const bool staged = n_splits <= COMBINE_SPLITS;
  if (staged) {
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) s_pm[s] = pm[base + s], s_pl[s] = pl[base + s];
    __syncthreads();
  }
  float mm = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, staged ? s_pm[s] : pm[base + s]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float ll = 0.f, a = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {
      float pv[8], ms[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        ms[k] = (s0 + k < n_splits) ? (staged ? s_pm[s0 + k] : pm[base + s0 + k]) : -INFINITY;
        pv[k] = (ms[k] != -INFINITY) ? po[(base + s0 + k) * D + d] : 0.f;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (ms[k] != -INFINITY) {      // ascending split order, as before
          const float c = exp2f(ms[k] - mm);
          ll += (staged ? s_pl[s0 + k] : pl[base + s0 + k]) * c;
          a += pv[k] * c;
        }
      }
    }
    float o = ll > 0.f ? a / ll : 0.f;
    if (gated) o *= sigmoid_f(__bfloat162float(gate_src[(size_t)t * gate_ld + (size_t)h * 2 * D + D + d]));
    out[((size_t)t * n_q + h) * D + d] = __float2bfloat16(o);
  }
}


// ---------------------------------------------------------------------------------------
// Tiled prefill attention (legacy tensor-core path: mma.sync m16n8k16 bf16, fp32 accumulate).
// One CTA = (16-token tile of one sequence, kv head); warp g of the CTA owns query head
// kvh * G + g, so the G heads of a group share every K / V tile.  K and V tiles of 32 keys
// (two 16-token pages) are gathered through the block table with cp.async into 128-bit-chunk
// XOR-swizzled shared memory, double buffered; QK^T and PV run on mma.sync with the usual
// register reuse of the score fragment as the A operand of PV; online softmax in the exp2
// domain; causal by absolute position; sigmoid output gate fused.  D = 256.
// The split-KV kernel above re-reads K / V for every query token; this one reads them once per
// 16 tokens, which is what makes long prompts tractable.
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

constexpr int PF_D = 256, PF_TQ = 16, PF_BC = 32, PF_ROW = PF_D * 2 /*bytes*/, PF_CHUNKS = PF_ROW / 16;

// byte offset of 16-byte chunk `c` of row `r` in a swizzled [rows][512 B] tile
__device__ __forceinline__ uint32_t pf_off(int r, int c) { return (uint32_t)(r * PF_ROW + ((c ^ (r & 7)) << 4)); }
// bf16 pool: a K / V tile of 32 keys is two pages, each brought by one tiled copy as four slabs
// [16 keys][128 B] under the tensor map's 128-byte swizzle (see attn_decode_mma_kernel below)
__device__ __forceinline__ uint32_t pt_off(int r, int c) {
  return (uint32_t)((r >> 4) * (KVB * PF_ROW) + (c >> 3) * (KVB * 128) + (r & 15) * 128 + (((c & 7) ^ (r & 7)) << 4));
}
__device__ __forceinline__ uint32_t dm_try_wait(uint32_t bar, uint32_t parity);
constexpr long long PF_WAIT_CYCLES = 4000000000LL;

// FP8: the pool holds e4m3 rows with one fp32 scale per (token, kv head).  The raw bytes of the
// next tile are staged with cp.async (double buffered) while this tile is computed; a conversion
// pass then expands the staged tile into the (single) swizzled bf16 tile the mma path reads.
__device__ __forceinline__ void cp4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void e4m3x16_to_bf16(const uint4& raw, float s, uint4& o0, uint4& o1) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t r[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = h2_to_f2(cvt_e4m3x2_to_h2((uint16_t)(w[i] & 0xFFFFu)));
    const float2 b = h2_to_f2(cvt_e4m3x2_to_h2((uint16_t)(w[i] >> 16)));
    r[2 * i] = f2_to_bf162_bits(a.x * s, a.y * s);
    r[2 * i + 1] = f2_to_bf162_bits(b.x * s, b.y * s);
  }
  o0 = make_uint4(r[0], r[1], r[2], r[3]);
  o1 = make_uint4(r[4], r[5], r[6], r[7]);
}

template <bool FP8>
__global__ void __launch_bounds__(256)
attn_prefill_kernel(const bf16* q, const bf16* gate_src, int gate_ld,
                    const bf16* kcache, const bf16* vcache,
                    const float* kscale, const float* vscale,
                    const int* block_table, int max_blocks, const int* q_start,
                    const int* q_len, const int* positions, bf16* out,
                    int n_q, int n_kv, float scale_log2e, int gated,
                    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, int map3d,
                    int n_blocks) {
  extern __shared__ unsigned char pf_smem_raw[];
  __shared__ uint64_t pf_full[2];
  __shared__ volatile int pf_ok;
  const uint32_t pf_raw_a = (uint32_t)__cvta_generic_to_shared(pf_smem_raw);
  unsigned char* pf_smem = pf_smem_raw + (((pf_raw_a + 1023u) & ~1023u) - pf_raw_a);    // swizzle atoms are 1024-byte aligned
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int G = n_q / n_kv;
  const int T = q_len[seq];
  if (tile * PF_TQ >= T) return;
  const int t0 = q_start[seq] + tile * PF_TQ;
  const int rows = min(PF_TQ, T - tile * PF_TQ);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = kvh * G + warp;
  unsigned char* qs = pf_smem + (size_t)warp * PF_TQ * PF_ROW;                 // [G][16][512 B]
  unsigned char* ks = pf_smem + (size_t)G * PF_TQ * PF_ROW;                    // [2][32][512 B] ([1] when FP8)
  unsigned char* vs = ks + (FP8 ? 1 : 2) * PF_BC * PF_ROW;                     // [2][32][512 B] ([1] when FP8)
  unsigned char* raw_k = vs + PF_BC * PF_ROW;                                  // FP8: [2][32][256 B] staged e4m3 rows
  unsigned char* raw_v = raw_k + 2 * PF_BC * PF_D;                             // FP8: [2][32][256 B]
  float* s_sc = reinterpret_cast<float*>(raw_v + 2 * PF_BC * PF_D);            // FP8: [2][K, V][32] row scales
  const uint32_t qs_a = (uint32_t)__cvta_generic_to_shared(qs);
  const uint32_t ks_a = (uint32_t)__cvta_generic_to_shared(ks), vs_a = (uint32_t)__cvta_generic_to_shared(vs);
  const int* table = block_table + (size_t)seq * max_blocks;
  // causal bound of the tile: keys 0 .. position of its last token
  const int n_keys = positions[t0 + rows - 1] + 1;
  const int n_tiles = (n_keys + PF_BC - 1) / PF_BC;

  // this warp's 16 query rows (zero rows past the end of the sequence)
  for (int x = lane; x < PF_TQ * PF_CHUNKS; x += 32) {
    const int r = x / PF_CHUNKS, c = x % PF_CHUNKS;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + r) * n_q + h) * PF_D + c * 8);
    *reinterpret_cast<uint4*>(qs + pf_off(r, c)) = v;
  }
  auto load_kv = [&](int kt, int buf) {
    const int j0 = kt * PF_BC;
    for (int x = threadIdx.x; x < PF_BC * PF_CHUNKS; x += blockDim.x) {
      const int r = x / PF_CHUNKS, c = x % PF_CHUNKS;
      const int j = j0 + r;
      const uint32_t dk = ks_a + buf * PF_BC * PF_ROW + pf_off(r, c);
      const uint32_t dv = vs_a + buf * PF_BC * PF_ROW + pf_off(r, c);
      if (j < n_keys) {
        const size_t off = (((size_t)table[j / KVB] * n_kv + kvh) * KVB + (j % KVB)) * PF_D + c * 8;
        cp16(dk, kcache + off);
        cp16(dv, vcache + off);
      } else {                      // rows past the bound: zeros (they are masked, but must not be NaN)
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dk), "r"(0u) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dv), "r"(0u) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // bf16 pool: thread 0 issues one tiled copy per K / V page of the tile (two pages), counted on full[buf]
  const uint32_t full_a = (uint32_t)__cvta_generic_to_shared(pf_full);
  auto load_kv_tma = [&](int kt, int buf) {
    const int j0 = kt * PF_BC;
    const int n_pg = min(PF_BC / KVB, (n_keys - j0 + KVB - 1) / KVB);
    const uint32_t bar = full_a + 8u * buf;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(n_pg * 2 * KVB * PF_ROW)) : "memory");
    for (int pg = 0; pg < n_pg; ++pg) {
      const int y = (trl_checked(table[j0 / KVB + pg], n_blocks, 3) * n_kv + kvh) * KVB;
      const uint32_t dk = ks_a + buf * PF_BC * PF_ROW + pg * (KVB * PF_ROW), dv = vs_a + buf * PF_BC * PF_ROW + pg * (KVB * PF_ROW);
      if (map3d) {
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                     ::"r"(dk), "l"(&map_k), "r"(0), "r"(y), "r"(0), "r"(bar) : "memory");
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                     ::"r"(dv), "l"(&map_v), "r"(0), "r"(y), "r"(0), "r"(bar) : "memory");
      } else {
        for (int sl = 0; sl < 4; ++sl) {
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(dk + sl * (KVB * 128)), "l"(&map_k), "r"(sl * 64), "r"(y), "r"(bar) : "memory");
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(dv + sl * (KVB * 128)), "l"(&map_v), "r"(sl * 64), "r"(y), "r"(bar) : "memory");
        }
      }
    }
  };
  auto stage_fp8 = [&](int kt, int sb) {
    const int j0 = kt * PF_BC;
    const unsigned char* k8 = reinterpret_cast<const unsigned char*>(kcache);
    const unsigned char* v8 = reinterpret_cast<const unsigned char*>(vcache);
    const uint32_t rk_a = (uint32_t)__cvta_generic_to_shared(raw_k), rv_a = (uint32_t)__cvta_generic_to_shared(raw_v);
    const uint32_t sc_a = (uint32_t)__cvta_generic_to_shared(s_sc);
    for (int x = threadIdx.x; x < PF_BC * 16; x += blockDim.x) {
      const int r = x >> 4, c = x & 15;
      const int j = j0 + r;
      if (j < n_keys) {
        const size_t ridx = ((size_t)table[j / KVB] * n_kv + kvh) * KVB + (j % KVB);
        cp16(rk_a + (sb * PF_BC + r) * PF_D + c * 16, k8 + ridx * PF_D + c * 16);
        cp16(rv_a + (sb * PF_BC + r) * PF_D + c * 16, v8 + ridx * PF_D + c * 16);
        if (c == 0) {
          cp4(sc_a + ((sb * 2 + 0) * PF_BC + r) * 4, kscale + ridx);
          cp4(sc_a + ((sb * 2 + 1) * PF_BC + r) * 4, vscale + ridx);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto convert_fp8 = [&](int kt, int sb) {
    const int j0 = kt * PF_BC;
    for (int x = threadIdx.x; x < PF_BC * 16; x += blockDim.x) {
      const int r = x >> 4, c = x & 15;
      uint4 k0 = make_uint4(0u, 0u, 0u, 0u), k1 = k0, v0 = k0, v1 = k0;   // rows past the bound: zeros
      if (j0 + r < n_keys) {
        const uint4 rk = *reinterpret_cast<const uint4*>(raw_k + (sb * PF_BC + r) * PF_D + c * 16);
        const uint4 rv = *reinterpret_cast<const uint4*>(raw_v + (sb * PF_BC + r) * PF_D + c * 16);
        e4m3x16_to_bf16(rk, s_sc[(sb * 2 + 0) * PF_BC + r], k0, k1);
        e4m3x16_to_bf16(rv, s_sc[(sb * 2 + 1) * PF_BC + r], v0, v1);
      }
      *reinterpret_cast<uint4*>(ks + pf_off(r, 2 * c)) = k0;
      *reinterpret_cast<uint4*>(ks + pf_off(r, 2 * c + 1)) = k1;
      *reinterpret_cast<uint4*>(vs + pf_off(r, 2 * c)) = v0;
      *reinterpret_cast<uint4*>(vs + pf_off(r, 2 * c + 1)) = v1;
    }
  };

  const int r_lo = lane >> 2;                      // fragment rows r_lo and r_lo + 8
  const int pos_lo = r_lo < rows ? positions[t0 + r_lo] : -1;
  const int pos_hi = r_lo + 8 < rows ? positions[t0 + r_lo + 8] : -1;
  float o[PF_D / 8][4];
#pragma unroll
  for (int i = 0; i < PF_D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  auto kv_off = [](int r, int c) { return FP8 ? pf_off(r, c) : pt_off(r, c); };
  if constexpr (!FP8) {
    // barriers; the V buffers start as zeros (a tile whose second page lies past the bound is not copied
    // there, and 0 x whatever shared memory held must be 0)
    if (threadIdx.x == 0) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full_a));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full_a + 8u));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      pf_ok = 1;
    }
    for (int x = threadIdx.x; x < 2 * PF_BC * PF_CHUNKS; x += blockDim.x)
      *reinterpret_cast<uint4*>(vs + (size_t)x * 16) = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) load_kv_tma(0, 0);
  } else {
    (void)load_kv;
    stage_fp8(0, 0);
  }
  for (int kt = 0; kt < n_tiles; ++kt) {
    const int buf = FP8 ? 0 : (kt & 1);
    bool have = true;
    if constexpr (FP8) {
      if (kt + 1 < n_tiles) {
        stage_fp8(kt + 1, (kt + 1) & 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();
      convert_fp8(kt, kt & 1);
      __syncthreads();
    } else {
      if (kt + 1 < n_tiles && threadIdx.x == 0) load_kv_tma(kt + 1, buf ^ 1);
      const uint32_t bar = full_a + 8u * buf, parity = (uint32_t)(kt >> 1) & 1u;
      if (!dm_try_wait(bar, parity)) {
        const long long t_begin = clock64();
        for (uint32_t it = 1; !dm_try_wait(bar, parity); ++it) {
          if ((it & 63) == 0 && (!pf_ok || clock64() - t_begin > PF_WAIT_CYCLES)) {
            if (pf_ok) trl_set_error(TRL_ERR_MBAR_TIMEOUT, (int)blockIdx.x, 420 + buf, kt);
            pf_ok = 0;
            have = false;
            break;
          }
        }
      }
    }
    const uint32_t kb = ks_a + buf * PF_BC * PF_ROW, vb = vs_a + buf * PF_BC * PF_ROW;
    if (have) {
    // ---- S = Q K^T for 32 keys: 4 n-tiles of 8 keys
    float sc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < PF_D / 16; ++kk) {
      uint32_t a[4];
      ldsm_x4(a, qs_a + pf_off((lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4)));
#pragma unroll
      for (int np = 0; np < 2; ++np) {             // two n-tiles per ldmatrix.x4
        uint32_t b[4];
        ldsm_x4(b, kb + kv_off(np * 16 + (lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1)));
        mma_bf16(sc[np * 2], a, b[0], b[1]);
        mma_bf16(sc[np * 2 + 1], a, b[2], b[3]);
      }
    }
    // ---- mask, scale, online softmax
    const int j0 = kt * PF_BC;
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int j = j0 + nt * 8 + (lane & 3) * 2;
      sc[nt][0] = (j <= pos_lo) ? sc[nt][0] * scale_log2e : -INFINITY;
      sc[nt][1] = (j + 1 <= pos_lo) ? sc[nt][1] * scale_log2e : -INFINITY;
      sc[nt][2] = (j <= pos_hi) ? sc[nt][2] * scale_log2e : -INFINITY;
      sc[nt][3] = (j + 1 <= pos_hi) ? sc[nt][3] * scale_log2e : -INFINITY;
      mx_lo = fmaxf(mx_lo, fmaxf(sc[nt][0], sc[nt][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(sc[nt][2], sc[nt][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo, base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
    const float al_lo = exp2f(m_lo - base_lo), al_hi = exp2f(m_hi - base_hi);   // exp2(-inf) = 0 on the first tile
    m_lo = mn_lo, m_hi = mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pa[2][4];                             // P as the A operand of PV: two k-steps of 16 keys
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float p0 = exp2f(sc[nt][0] - base_lo), p1 = exp2f(sc[nt][1] - base_lo);
      const float p2 = exp2f(sc[nt][2] - base_hi), p3 = exp2f(sc[nt][3] - base_hi);
      sum_lo += p0 + p1, sum_hi += p2 + p3;
      pa[nt >> 1][(nt & 1) * 2] = f2_to_bf162_bits(p0, p1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = f2_to_bf162_bits(p2, p3);
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    l_lo = l_lo * al_lo + sum_lo, l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
    for (int i = 0; i < PF_D / 8; ++i) o[i][0] *= al_lo, o[i][1] *= al_lo, o[i][2] *= al_hi, o[i][3] *= al_hi;
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int nd = 0; nd < PF_D / 8; nd += 2) {
        uint32_t b[4];
        ldsm_x4_t(b, vb + kv_off(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, nd + (lane >> 4)));
        mma_bf16(o[nd], pa[kk], b[0], b[1]);
        mma_bf16(o[nd + 1], pa[kk], b[2], b[3]);
      }
    }
    }
    __syncthreads();                               // the other buffer may be overwritten next round
    if constexpr (!FP8) {
      if (!pf_ok) break;                           // a wait ran out (error word set): every thread leaves together
    }
  }
  // ---- epilogue: normalise, gate, store
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
  for (int nd = 0; nd < PF_D / 8; ++nd) {
    const int d = nd * 8 + (lane & 3) * 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = r_lo + half * 8;
      if (r >= rows) continue;
      const int t = t0 + r;
      float v0 = o[nd][half * 2] * (half ? inv_hi : inv_lo), v1 = o[nd][half * 2 + 1] * (half ? inv_hi : inv_lo);
      if (gated) {
        const bf16* gp = gate_src + (size_t)t * gate_ld + (size_t)h * 2 * PF_D + PF_D + d;
        v0 *= sigmoid_f(__bfloat162float(gp[0])), v1 *= sigmoid_f(__bfloat162float(gp[1]));
      }
      *reinterpret_cast<uint32_t*>(out + ((size_t)t * n_q + h) * PF_D + d) = f2_to_bf162_bits(v0, v1);
    }
  }
}


// ---------------------------------------------------------------------------------------
// Split-KV decode / verify attention on the tensor cores (mma.sync m16n8k16 bf16, fp32
// accumulate; D = 256).  One CTA = (key split, kv head, group of `tpg` consecutive tokens of one
// sequence): the G query heads of the kv head times the group's tokens are the (up to 16) rows
// of ONE M tile, so a K / V row is read once for all of them -- the scalar kernel above reads
// it once per token and spends 2 G D fp32 FMAs per key on it.  The CTA walks its key range in
// tiles of 64 keys gathered through the block table with cp.async (double buffered, 128-bit
// chunk XOR swizzle); warp w owns keys [16 w, 16 w + 16) of every tile with its own online
// softmax state, and the four warps are merged through shared memory at the end.  Output:
// the same split partials (unnormalised row, running max in the exp2 domain, denominator) the
// combine kernel reads, or the finished gated row when there is one split.
constexpr int DM_KEYS = 64, DM_WARPS = 4, DM_ROWS = 16, DM_STAGES = 3, DM_TAB = 512;
constexpr int DM_RS = PF_ROW + 16;                 // Q row stride in shared memory: 512 B of data + 16 B, so that the
                                                   // eight rows of an ldmatrix fall into different banks without a swizzle
constexpr int DM_QBYTES = 9216;                    // 16 Q rows (8448 B) rounded up to the 1024-byte alignment of the stages
constexpr int DM_PAGE = KVB * PF_ROW;              // one page of one kv head: 16 keys x 512 B, contiguous in the pool
constexpr int DM_SLAB = KVB * 128;                 // 128-byte column slab of a page: the unit of the 128-byte swizzle
constexpr int DM_TILE = (DM_KEYS / KVB) * DM_PAGE;
constexpr int DM_SMEM = 1024 + DM_QBYTES + 2 * DM_STAGES * DM_TILE + 64;    // alignment slack, Q tile, K and V rings, barriers
constexpr long long DM_WAIT_CYCLES = 4000000000LL;
static_assert(DM_WARPS * 16 == DM_KEYS && KVB == 16, "a consumer warp owns one page of every tile");

__device__ __forceinline__ uint32_t dm_off(int r, int c) { return (uint32_t)(r * DM_RS + c * 16); }
// 16-byte chunk c (0..31) of key `key` (0..63) of a stage.  A page arrives as four slabs [16 keys][128 B] under the
// tensor map's 128-byte swizzle: within a slab the chunk index is XORed with the key's low three bits.
__device__ __forceinline__ uint32_t dm_kv_off(int key, int c) {
  const int r = key & 15;
  return (uint32_t)((key >> 4) * DM_PAGE + (c >> 3) * DM_SLAB + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}
__device__ __forceinline__ uint32_t dm_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p;\n"
      "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "  selp.u32 %0, 1, 0, p; }\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}

// Warps 0-3 compute, warp 4 produces.  The pool is described to the copy engine as a tensor
// {64 elements, rows of 512 B, 4 column slabs of 128 B}: ONE tiled copy brings a whole page of a kv head
// (16 keys, 8 KB) as four swizzled slabs, so a 64-key tile is eight copies (K and V of four pages)
// into a three-stage ring.  A stage's "full" mbarrier counts the bytes, its "empty" mbarrier the four
// consumer warps.  The block-table entries of the CTA's key range are read into shared memory once,
// so no global load sits in the loop.  map3d == 0: the same layout from 2-D copies, one per slab.
//
// FUSED (decode ticks: one new token per sequence, rotary width 64): the kernel is the whole attention
// layer.  `q` is then the raw fused projection row [hq x (query ; gate)] ++ [hkv x D] ++ [hkv x D] (leading
// dimension gate_ld): every CTA normalises and rotates the six query rows of its kv head itself, the CTA
// whose key range holds the new position does the same for the new K row, copies the V row, writes both
// to the pool and patches them into its shared-memory tile (the tile copy may have fetched the page before
// the write landed); the last CTA of a (token, kv head) to finish merges the split partials and writes the
// gated output rows, so neither the prep nor the combine kernel is launched.
struct DmFused {
  const float *q_norm, *k_norm;
  const int* slot_mapping;
  bf16 *kcache, *vcache;
  int* counters;                                   // [T * n_kv], zero between launches
  float log2_theta, eps;
  int rotary;
};
constexpr int DM_ROT_HALF = 32;                    // the fused form takes rotary == 64

// One head row of the fused projection: RMSNorm (fp32), rotation of the first 64 dims by the position's
// angles, bf16.  Lane l owns dims 8l .. 8l + 7; lanes 0-3 pair with lanes 4-7 for the rotation.
__device__ __forceinline__ uint4 dm_prep_row(const bf16* src, const float* __restrict__ w, float eps, const float* cs,
                                             const float* sn, int lane) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src + lane * 8);
  const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
  float v[8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = bf162_bits_to_f2(rw[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
    ss += f.x * f.x + f.y * f.y;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)PF_D + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd * w[lane * 8 + i];
  float o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float other = __shfl_xor_sync(0xffffffffu, v[i], 4);
    const int d = lane * 8 + i;
    if (lane < 4) o[i] = v[i] * cs[d] - other * sn[d];
    else if (lane < 8) o[i] = v[i] * cs[d - DM_ROT_HALF] + other * sn[d - DM_ROT_HALF];
    else o[i] = v[i];
  }
  return make_uint4(f2_to_bf162_bits(o[0], o[1]), f2_to_bf162_bits(o[2], o[3]), f2_to_bf162_bits(o[4], o[5]),
                    f2_to_bf162_bits(o[6], o[7]));
}

template <bool FUSED>
__global__ void __launch_bounds__((DM_WARPS + 1) * 32)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, int map3d,
                       const bf16* q, const bf16* gate_src, int gate_ld,
                       const int* block_table, int max_blocks, const int* seq_ids, const int* positions,
                       float* po, float* pm, float* pl, bf16* out, int T, int n_q, int n_kv, int n_splits,
                       int tpg, float scale_log2e, int gated, const DmFused fz, int n_blocks) {
  extern __shared__ unsigned char dm_smem_raw[];
  __shared__ float s_m[DM_WARPS][DM_ROWS], s_l[DM_WARPS][DM_ROWS];
  __shared__ int s_tab[DM_TAB];
  __shared__ volatile int s_ok;
  __shared__ float s_cs[DM_ROT_HALF], s_sn[DM_ROT_HALF];
  __shared__ __align__(16) uint4 s_knew[32], s_vnew[32];      // the new token's K and V rows (bf16 x 256)
  __shared__ int s_last;
  const int split = blockIdx.x, kvh = blockIdx.y, t0 = blockIdx.z * tpg;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t raw_a = (uint32_t)__cvta_generic_to_shared(dm_smem_raw);
  unsigned char* dm_smem = dm_smem_raw + (((raw_a + 1023u) & ~1023u) - raw_a);
  unsigned char* qs = dm_smem;                               // [16][528 B]
  unsigned char* ks = dm_smem + DM_QBYTES;                   // [stages][4 pages][4 slabs][16 keys][128 B]
  unsigned char* vs = ks + DM_STAGES * DM_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(vs + DM_STAGES * DM_TILE);   // full[stages], empty[stages]
  const uint32_t qs_a = (uint32_t)__cvta_generic_to_shared(qs);
  const uint32_t ks_a = (uint32_t)__cvta_generic_to_shared(ks), vs_a = (uint32_t)__cvta_generic_to_shared(vs);
  const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(bars);
  auto full = [&](int st) { return bar_a + 8u * st; };
  auto empty = [&](int st) { return bar_a + 8u * (DM_STAGES + st); };
  if (threadIdx.x == 0) {
    for (int st = 0; st < DM_STAGES; ++st) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full(st)));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty(st)), "r"(DM_WARPS));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_ok = 1;
  }
  pdl_launch_dependents(4);
  pdl_wait();
  const int G = n_q / n_kv;
  const int nt = min(tpg, T - t0);
  const int rows = nt * G;
  int kv_len = 0;                                           // keys the group's furthest row sees (rows of a
  for (int i = 0; i < nt; ++i) kv_len = max(kv_len, positions[t0 + i] + 1);   // padded window need not ascend)
  const int* table = block_table + (size_t)seq_ids[t0] * max_blocks;
  const int pages = (kv_len + KVB - 1) / KVB;
  // the grid's split count is fixed when a graph is captured, the context is not: a short context is cut
  // into splits of at least 128 keys, the CTAs past them find an empty range and write a neutral partial
  const int n_eff = max(1, min(n_splits, (kv_len + 127) / 128));
  const int pps = (pages + n_eff - 1) / n_eff;
  const int lo = split * pps * KVB, hi = min(kv_len, (split + 1) * pps * KVB);
  const int n_tiles = hi > lo ? (hi - lo + DM_KEYS - 1) / DM_KEYS : 0;
  const int page0 = lo / KVB, n_pages = hi > lo ? (hi - lo + KVB - 1) / KVB : 0;
  const bool tab_cached = n_pages <= DM_TAB;
  if (tab_cached)
    for (int i = threadIdx.x; i < n_pages; i += blockDim.x) s_tab[i] = table[page0 + i];

  // row r of the tile = (token r / G of the group, head r % G of the kv head); unused rows are zero
  const int new_pos = kv_len - 1;                  // FUSED: the position of the tick's token
  if (FUSED) {
    if (threadIdx.x < DM_ROT_HALF) {               // the position's rotation angles, in double like the prep kernel
      const double inv = exp2(-(double)(2 * threadIdx.x) / (double)fz.rotary * (double)fz.log2_theta);
      double sd, cd;
      sincos((double)new_pos * inv, &sd, &cd);
      s_cs[threadIdx.x] = (float)cd, s_sn[threadIdx.x] = (float)sd;
    }
    for (int x = threadIdx.x; x < (DM_ROWS - rows) * PF_CHUNKS; x += blockDim.x)
      *reinterpret_cast<uint4*>(qs + dm_off(rows + x / PF_CHUNKS, x % PF_CHUNKS)) = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const bf16* row = q + (size_t)t0 * gate_ld;
    const int per_q = gated ? 2 * PF_D : PF_D;
    // the G query rows, then the new K row and the new V row, dealt round the five warps
    for (int job = warp; job < rows + 2; job += DM_WARPS + 1) {
      if (job < rows) {
        const uint4 v = dm_prep_row(row + (size_t)(kvh * G + job) * per_q, fz.q_norm, fz.eps, s_cs, s_sn, lane);
        *reinterpret_cast<uint4*>(qs + dm_off(job, lane)) = v;
      } else if (new_pos >= lo && new_pos < hi) {
        int slot = fz.slot_mapping[t0];
        if (slot >= 0) slot = trl_checked(slot, n_blocks * KVB, 4);
        const size_t dst = (((size_t)(slot / KVB) * n_kv + kvh) * KVB + (slot % KVB)) * PF_D + lane * 8;
        if (job == rows) {
          const uint4 v = dm_prep_row(row + (size_t)n_q * per_q + (size_t)kvh * PF_D, fz.k_norm, fz.eps, s_cs, s_sn, lane);
          s_knew[lane] = v;
          if (slot >= 0) *reinterpret_cast<uint4*>(fz.kcache + dst) = v;
        } else {
          const uint4 v = *reinterpret_cast<const uint4*>(row + (size_t)n_q * per_q + (size_t)(n_kv + kvh) * PF_D + lane * 8);
          s_vnew[lane] = v;
          if (slot >= 0) *reinterpret_cast<uint4*>(fz.vcache + dst) = v;
        }
      }
    }
  } else {
    for (int x = threadIdx.x; x < DM_ROWS * PF_CHUNKS; x += blockDim.x) {
      const int r = x / PF_CHUNKS, c = x % PF_CHUNKS;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + r / G) * n_q + kvh * G + r % G) * PF_D + c * 8);
      *reinterpret_cast<uint4*>(qs + dm_off(r, c)) = v;
    }
  }
  __syncthreads();                                 // barriers initialised, table and Q rows in place
  auto bounded_wait = [&](uint32_t bar, uint32_t parity, int what) {
    if (dm_try_wait(bar, parity)) return true;
    const long long t_begin = clock64();
    for (uint32_t it = 1; !dm_try_wait(bar, parity); ++it) {
      if ((it & 63) == 0) {
        if (!s_ok) return false;
        if (clock64() - t_begin > DM_WAIT_CYCLES) {
          trl_set_error(TRL_ERR_MBAR_TIMEOUT, (int)blockIdx.x, what, (int)parity);
          s_ok = 0;
          return false;
        }
      }
    }
    return true;
  };

  if (warp == DM_WARPS) {
    // ---------------- producer ----------------
    for (int kt = 0; kt < n_tiles; ++kt) {
      const int st = kt % DM_STAGES;
      if (kt >= DM_STAGES && !bounded_wait(empty(st), (uint32_t)(kt / DM_STAGES - 1) & 1u, 410 + st)) break;
      const int j0 = lo + kt * DM_KEYS;
      const int n_pg = min(DM_KEYS / KVB, (hi - j0 + KVB - 1) / KVB);     // whole pages: keys past `hi` are masked
      if (lane == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full(st)), "r"((uint32_t)(n_pg * 2 * DM_PAGE)) : "memory");
      __syncwarp();
      // lane -> (K or V, page of the tile, slab); with the 3-D map the lanes of slab 0 copy the whole page
      const int is_v = lane >> 4, pg = (lane >> 2) & 3, sl = lane & 3;
      if (pg < n_pg && (!map3d || sl == 0)) {
        const int pi = j0 / KVB + pg;
        const int blk = trl_checked(tab_cached ? s_tab[pi - page0] : table[pi], n_blocks, 2);
        const int y = (blk * n_kv + kvh) * KVB;
        const uint32_t dst = (is_v ? vs_a : ks_a) + st * DM_TILE + pg * DM_PAGE + sl * DM_SLAB;
        const CUtensorMap* mp = is_v ? &map_v : &map_k;
        if (map3d)
          asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                       ::"r"(dst), "l"(mp), "r"(0), "r"(y), "r"(0), "r"(full(st)) : "memory");
        else
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(dst), "l"(mp), "r"(sl * 64), "r"(y), "r"(full(st)) : "memory");
      }
    }
  }

  const int r_lo = lane >> 2;                      // fragment rows r_lo and r_lo + 8
  const int pos_lo = r_lo < rows ? positions[t0 + r_lo / G] : -1;
  const int pos_hi = r_lo + 8 < rows ? positions[t0 + (r_lo + 8) / G] : -1;
  float o[PF_D / 8][4];
#pragma unroll
  for (int i = 0; i < PF_D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int kt = 0; kt < n_tiles && warp < DM_WARPS; ++kt) {
    const int buf = kt % DM_STAGES;
    if (!bounded_wait(full(buf), (uint32_t)(kt / DM_STAGES) & 1u, 400 + buf)) break;
    const int jw = lo + kt * DM_KEYS + warp * 16;     // this warp's first key of the tile
    if (jw < hi && s_ok) {
      const uint32_t kb = ks_a + buf * DM_TILE, vb = vs_a + buf * DM_TILE;
      if (FUSED && new_pos >= jw && new_pos < jw + 16) {
        // this tick's token: its rows come from this CTA's registers, not from the page copy
        const int key = warp * 16 + (new_pos - jw);
        const uint4 kn = s_knew[lane], vn = s_vnew[lane];
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(kb + dm_kv_off(key, lane)), "r"(kn.x), "r"(kn.y), "r"(kn.z), "r"(kn.w) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(vb + dm_kv_off(key, lane)), "r"(vn.x), "r"(vn.y), "r"(vn.z), "r"(vn.w) : "memory");
        __syncwarp();
      }
      if (jw + 16 > hi) {
        // the page's keys past the range hold whatever the pool holds: their scores are masked by a
        // select, but 0 x V must be 0, so their V rows are cleared (only this warp reads them)
        for (int x = lane; x < (jw + 16 - hi) * PF_CHUNKS; x += 32) {
          const int key = warp * 16 + (hi - jw) + x / PF_CHUNKS;
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(vb + dm_kv_off(key, x % PF_CHUNKS)), "r"(0u) : "memory");
        }
        __syncwarp();
      }
      // ---- S = Q K^T for this warp's 16 keys: two n-tiles of 8
      float sc[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < PF_D / 16; ++kk) {
        uint32_t a[4], b[4];
        ldsm_x4(a, qs_a + dm_off((lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4)));
        ldsm_x4(b, kb + dm_kv_off(warp * 16 + (lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1)));
        mma_bf16(sc[0], a, b[0], b[1]);
        mma_bf16(sc[1], a, b[2], b[3]);
      }
      // ---- mask (causal per row, and the end of the split's range), scale, online softmax
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int n8 = 0; n8 < 2; ++n8) {
        const int j = jw + n8 * 8 + (lane & 3) * 2;
        const bool in0 = j < hi, in1 = j + 1 < hi;
        sc[n8][0] = (in0 && j <= pos_lo) ? sc[n8][0] * scale_log2e : -INFINITY;
        sc[n8][1] = (in1 && j + 1 <= pos_lo) ? sc[n8][1] * scale_log2e : -INFINITY;
        sc[n8][2] = (in0 && j <= pos_hi) ? sc[n8][2] * scale_log2e : -INFINITY;
        sc[n8][3] = (in1 && j + 1 <= pos_hi) ? sc[n8][3] * scale_log2e : -INFINITY;
        mx_lo = fmaxf(mx_lo, fmaxf(sc[n8][0], sc[n8][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(sc[n8][2], sc[n8][3]));
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo, base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float al_lo = exp2f(m_lo - base_lo), al_hi = exp2f(m_hi - base_hi);
      m_lo = mn_lo, m_hi = mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
      uint32_t pa[4];                                // P as the A operand of PV: one k-step of 16 keys
#pragma unroll
      for (int n8 = 0; n8 < 2; ++n8) {
        const float p0 = exp2f(sc[n8][0] - base_lo), p1 = exp2f(sc[n8][1] - base_lo);
        const float p2 = exp2f(sc[n8][2] - base_hi), p3 = exp2f(sc[n8][3] - base_hi);
        sum_lo += p0 + p1, sum_hi += p2 + p3;
        pa[n8 * 2] = f2_to_bf162_bits(p0, p1);
        pa[n8 * 2 + 1] = f2_to_bf162_bits(p2, p3);
      }
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
      l_lo = l_lo * al_lo + sum_lo, l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < PF_D / 8; ++i) o[i][0] *= al_lo, o[i][1] *= al_lo, o[i][2] *= al_hi, o[i][3] *= al_hi;
      // ---- O += P V
#pragma unroll
      for (int nd = 0; nd < PF_D / 8; nd += 2) {
        uint32_t b[4];
        ldsm_x4_t(b, vb + dm_kv_off(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, nd + (lane >> 4)));
        mma_bf16(o[nd], pa, b[0], b[1]);
        mma_bf16(o[nd + 1], pa, b[2], b[3]);
      }
    }
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty(buf)) : "memory");   // this warp is done with the stage
  }
  __syncthreads();                                 // every warp is out of its loop: the K ring becomes the merge buffer
  if (!s_ok) {                                     // copies may still be in flight towards this CTA's shared memory
    const long long t_begin = clock64();
    while (clock64() - t_begin < 2000000LL) {
    }
  }

  // ---- merge the four warps (each saw different keys) through shared memory
  float* so = reinterpret_cast<float*>(ks);        // [4 warps][16 rows][256] fp32, inside the K buffers
  if (warp < DM_WARPS) {
    if ((lane & 3) == 0) {
      s_m[warp][r_lo] = m_lo, s_m[warp][r_lo + 8] = m_hi;
      s_l[warp][r_lo] = l_lo, s_l[warp][r_lo + 8] = l_hi;
    }
#pragma unroll
    for (int nd = 0; nd < PF_D / 8; ++nd) {
      const int d = nd * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(so + ((size_t)warp * DM_ROWS + r_lo) * PF_D + d) = make_float2(o[nd][0], o[nd][1]);
      *reinterpret_cast<float2*>(so + ((size_t)warp * DM_ROWS + r_lo + 8) * PF_D + d) = make_float2(o[nd][2], o[nd][3]);
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows * PF_D; idx += blockDim.x) {
    const int r = idx / PF_D, d = idx % PF_D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) mm = fmaxf(mm, s_m[w][r]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) {
      const float c = (s_m[w][r] == -INFINITY) ? 0.f : exp2f(s_m[w][r] - mm);
      ll += s_l[w][r] * c;
      a += so[((size_t)w * DM_ROWS + r) * PF_D + d] * c;
    }
    const int t = t0 + r / G, h = kvh * G + r % G;
    if (n_splits == 1) {
      float ov = ll > 0.f ? a / ll : 0.f;
      if (gated) ov *= sigmoid_f(__bfloat162float(gate_src[(size_t)t * gate_ld + (size_t)h * 2 * PF_D + PF_D + d]));
      out[((size_t)t * n_q + h) * PF_D + d] = __float2bfloat16(ov);
    } else if (!FUSED || split < n_eff) {          // FUSED: the merge below reads the first n_eff splits only
      const size_t base = ((size_t)t * n_q + h) * n_splits + split;
      po[base * PF_D + d] = a;
      if (d == 0) pm[base] = mm, pl[base] = ll;
    }
  }
  if (FUSED && n_splits > 1) {
    // the last CTA of this (token, kv head) to get here merges the splits: what the combine kernel does
    // for a head, here for the G heads of the group
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int old = atomicAdd(fz.counters + (size_t)t0 * n_kv + kvh, 1);
      s_last = old == n_splits - 1;
      if (s_last) fz.counters[(size_t)t0 * n_kv + kvh] = 0;     // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float* wgt = so;                               // [G][n_eff] weights exp2(m_s - m) / l, in the (idle) K ring
    for (int x = threadIdx.x; x < rows * n_eff; x += blockDim.x) {
      const int r = x / n_eff;
      const size_t base = ((size_t)t0 * n_q + kvh * G + r) * n_splits;
      float mm = -INFINITY, ll = 0.f;
      for (int s2 = 0; s2 < n_eff; ++s2) mm = fmaxf(mm, __ldcg(pm + base + s2));
      for (int s2 = 0; s2 < n_eff; ++s2) {
        const float ms = __ldcg(pm + base + s2);
        if (ms != -INFINITY) ll += __ldcg(pl + base + s2) * exp2f(ms - mm);
      }
      const float ms = __ldcg(pm + base + x % n_eff);
      wgt[x] = (ms != -INFINITY && ll > 0.f) ? exp2f(ms - mm) / ll : 0.f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows * PF_D; idx += blockDim.x) {
      const int r = idx / PF_D, d = idx % PF_D, h = kvh * G + r;
      const size_t base = ((size_t)t0 * n_q + h) * n_splits;
      float a = 0.f;
      for (int s0 = 0; s0 < n_eff; s0 += 8) {
        float pv[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) pv[k] = (s0 + k < n_eff) ? __ldcg(po + (base + s0 + k) * PF_D + d) : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (s0 + k < n_eff) a += pv[k] * wgt[r * n_eff + s0 + k];
      }
      if (gated) a *= sigmoid_f(__bfloat162float(gate_src[(size_t)t0 * gate_ld + (size_t)h * 2 * PF_D + PF_D + d]));
      out[((size_t)t0 * n_q + h) * PF_D + d] = __float2bfloat16(a);
    }
  }
}

}  // namespace

// n_blocks: pages of the pool (the checked build compares every KV slot against n_blocks * 16).
TRL_API int trl_attn_prep(const void* qkv, int ld, const void* q_norm, const void* k_norm,
                          const void* positions, const void* slot_mapping, void* q_out, void* kcache,
                          void* vcache, int T, int n_q, int n_kv, int D, int rotary, float theta,
                          float eps, int gated, int n_blocks, void* stream) {
  const int threads = 256;
  const size_t smem = (size_t)(rotary + (threads / 32) * D) * sizeof(float);
  const int chunks = (n_q + 2 * n_kv + threads / 32 - 1) / (threads / 32);   // one warp per head
  return (int)trl_launch(attn_prep_kernel, dim3(T, chunks), dim3(threads), smem, (cudaStream_t)stream,
                         (const bf16*)qkv, ld, (const float*)q_norm, (const float*)k_norm,
                         (const int*)positions, (const int*)slot_mapping, (bf16*)q_out, (bf16*)kcache,
                         (bf16*)vcache, n_q, n_kv, D, rotary, log2f(theta), eps, gated, n_blocks * KVB);
}

// Scratch: po [T*n_q*n_splits*D] fp32, pm/pl [T*n_q*n_splits] fp32 (unused when n_splits == 1).
TRL_API int trl_attn_paged(const void* q, const void* gate_src, int gate_ld, const void* kcache,
                           const void* vcache, const void* block_table, int max_blocks,
                           const void* seq_ids, const void* positions, void* po, void* pm, void* pl,
                           void* out, int T, int n_q, int n_kv, int D, int n_splits, float scale,
                           int gated, void* stream) {
  if (n_kv <= 0 || n_q <= 0 || n_q % n_kv != 0 || n_q / n_kv > MAXG) return (int)cudaErrorInvalidValue;
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

namespace {

// Tensor maps of a layer's K and V pools for attn_decode_mma_kernel, cached by (pointers, blocks, heads).
// Preferred form: {64 elements, rows (512 B apart), 4 column slabs (128 B apart)} with a box of a whole
// page {64, 16, 4} under the 128-byte swizzle; if the driver refuses that encoding, a 2-D map
// {256 elements, rows} with a box of one slab {64, 16}.
struct DmMaps {
  const void *k, *v;
  int n_blocks, n_kv, mode3d;
  CUtensorMap mk, mv;
};
typedef CUresult (*DmEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::mutex g_dm_mu;
std::vector<DmMaps> g_dm_maps;
DmEncodeFn g_dm_encode = nullptr;

int dm_encode(CUtensorMap* m, const void* base, uint64_t rows, int mode3d) {
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r;
  if (mode3d) {
    const cuuint64_t dims[3] = {64, rows, 4};
    const cuuint64_t strides[2] = {(cuuint64_t)PF_ROW, 128};
    const cuuint32_t box[3] = {64, (cuuint32_t)KVB, 4};
    r = g_dm_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    const cuuint64_t dims[2] = {(cuuint64_t)PF_D, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)PF_ROW};
    const cuuint32_t box[2] = {64, (cuuint32_t)KVB};
    r = g_dm_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? 0 : 1;
}

// 0 on success; fills `out`.  force2d: environment TRL_ATTN_MAP2D=1 selects the per-slab form.
int dm_get_maps(const void* k, const void* v, int n_blocks, int n_kv, DmMaps* out) {
  std::lock_guard<std::mutex> lock(g_dm_mu);
  for (const DmMaps& e : g_dm_maps)
    if (e.k == k && e.v == v && e.n_blocks == n_blocks && e.n_kv == n_kv) {
      *out = e;
      return 0;
    }
  if (!g_dm_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return 1;
    g_dm_encode = (DmEncodeFn)fn;
  }
  static const bool force2d = [] { const char* e = getenv("TRL_ATTN_MAP2D"); return e && e[0] == '1'; }();
  DmMaps m;
  m.k = k, m.v = v, m.n_blocks = n_blocks, m.n_kv = n_kv;
  const uint64_t rows = (uint64_t)n_blocks * n_kv * KVB;
  m.mode3d = force2d ? 0 : 1;
  if (m.mode3d && (dm_encode(&m.mk, k, rows, 1) || dm_encode(&m.mv, v, rows, 1))) m.mode3d = 0;
  if (!m.mode3d && (dm_encode(&m.mk, k, rows, 0) || dm_encode(&m.mv, v, rows, 0))) return 2;
  if (g_dm_maps.size() >= 1024) g_dm_maps.erase(g_dm_maps.begin(), g_dm_maps.begin() + 512);
  g_dm_maps.push_back(m);
  *out = m;
  return 0;
}

}  // namespace

// Tensor-core variant of trl_attn_paged for the bf16 pool (D = 256): `tpg` consecutive tokens of the
// batch that belong to one sequence (1 for decode; a divisor of the verify width) share a CTA, with
// tpg * (n_q / n_kv) <= 16 rows.  Same scratch and combine as trl_attn_paged.  The pools are
// [n_blocks, n_kv, 16, D] bf16 at 16-byte aligned addresses.
TRL_API int trl_attn_decode_mma(const void* q, const void* gate_src, int gate_ld, const void* kcache,
                                const void* vcache, const void* block_table, int max_blocks, int n_blocks,
                                const void* seq_ids, const void* positions, void* po, void* pm, void* pl,
                                void* out, int T, int n_q, int n_kv, int D, int n_splits, int tpg, float scale,
                                int gated, void* stream) {
  if (D != PF_D || n_kv <= 0 || n_q <= 0 || n_q % n_kv != 0 || tpg < 1 || tpg * (n_q / n_kv) > DM_ROWS || T <= 0 ||
      n_splits < 1 || n_blocks <= 0 || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15))
    return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_decode_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DM_SMEM) != cudaSuccess)
      return 3;
    configured = true;
  }
  DmMaps maps;
  if (dm_get_maps(kcache, vcache, n_blocks, n_kv, &maps)) return (int)cudaErrorInvalidValue;
  const dim3 grid(n_splits, n_kv, (T + tpg - 1) / tpg);
  DmFused none = {};
  cudaError_t e = trl_launch(attn_decode_mma_kernel<false>, grid, dim3((DM_WARPS + 1) * 32), (size_t)DM_SMEM, st, maps.mk, maps.mv,
                             maps.mode3d, (const bf16*)q, (const bf16*)gate_src, gate_ld,
                             (const int*)block_table, max_blocks, (const int*)seq_ids, (const int*)positions,
                             (float*)po, (float*)pm, (float*)pl, (bf16*)out, T, n_q, n_kv, n_splits, tpg,
                             scale * 1.4426950408889634f, gated, none, n_blocks);
  if (e != cudaSuccess) return (int)e;
  if (n_splits > 1)
    e = trl_launch(attn_combine_kernel, dim3(T, n_q), dim3(min(D, 256)), 0, st, (const float*)po,
                   (const float*)pm, (const float*)pl, (const bf16*)gate_src, gate_ld, (bf16*)out, n_q,
                   D, n_splits, gated);
  return (int)e;
}

// The whole attention layer of a decode tick in ONE launch (bf16 pool, D = 256, rotary width 64, one new
// token per sequence): q / k RMSNorm + rotation + KV write, split-KV attention on the tensor cores, merge of
// the splits by the last CTA of each (token, kv head) and the sigmoid gate.  qkv: the fused projection rows
// [T, ld]; counters: T * n_kv ints, zero on entry and zero again on exit.  Scratch as trl_attn_paged.
TRL_API int trl_attn_decode_fused(const void* qkv, int ld, const void* q_norm, const void* k_norm, const void* positions,
                                  const void* slot_mapping, void* kcache, void* vcache, const void* block_table,
                                  int max_blocks, int n_blocks, const void* seq_ids, void* po, void* pm, void* pl,
                                  void* counters, void* out, int T, int n_q, int n_kv, int D, int rotary, float theta,
                                  float eps, int n_splits, float scale, int gated, void* stream) {
  if (D != PF_D || rotary != 2 * DM_ROT_HALF || n_kv <= 0 || n_q <= 0 || n_q % n_kv != 0 || n_q / n_kv > DM_ROWS ||
      T <= 0 || n_splits < 1 || n_splits > COMBINE_SPLITS || n_blocks <= 0 || ((uintptr_t)kcache & 15) ||
      ((uintptr_t)vcache & 15) || ((uintptr_t)qkv & 15) || ld % 8 != 0)
    return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_decode_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DM_SMEM) != cudaSuccess)
      return 3;
    configured = true;
  }
  DmMaps maps;
  if (dm_get_maps(kcache, vcache, n_blocks, n_kv, &maps)) return (int)cudaErrorInvalidValue;
  DmFused fz;
  fz.q_norm = (const float*)q_norm, fz.k_norm = (const float*)k_norm, fz.slot_mapping = (const int*)slot_mapping;
  fz.kcache = (bf16*)kcache, fz.vcache = (bf16*)vcache, fz.counters = (int*)counters;
  fz.log2_theta = log2f(theta), fz.eps = eps, fz.rotary = rotary;
  return (int)trl_launch(attn_decode_mma_kernel<true>, dim3(n_splits, n_kv, T), dim3((DM_WARPS + 1) * 32), (size_t)DM_SMEM,
                         (cudaStream_t)stream, maps.mk, maps.mv, maps.mode3d, (const bf16*)qkv, (const bf16*)qkv, ld,
                         (const int*)block_table, max_blocks, (const int*)seq_ids, (const int*)positions, (float*)po,
                         (float*)pm, (float*)pl, (bf16*)out, T, n_q, n_kv, n_splits, 1, scale * 1.4426950408889634f, gated,
                         fz, n_blocks);
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

// Tiled prefill attention over whole sequences of the batch (D = 256, G = n_q / n_kv <= 8):
// q_start / q_len give each sequence's token range in the flat batch; `out` [T, n_q * D].
TRL_API int trl_attn_prefill(const void* q, const void* gate_src, int gate_ld, const void* kcache, const void* vcache,
                             const void* block_table, int max_blocks, int n_blocks, const void* q_start, const void* q_len,
                             const void* positions, void* out, int B, int max_q_len, int n_q, int n_kv, int D,
                             float scale, int gated, void* stream) {
  const int G = n_kv > 0 ? n_q / n_kv : 0;
  if (D != PF_D || G < 1 || G > 8 || n_q % n_kv != 0 || B <= 0 || max_q_len <= 0) return (int)cudaErrorInvalidValue;
  if (n_blocks <= 0 || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15)) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)G * PF_TQ * PF_ROW + (size_t)4 * PF_BC * PF_ROW + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * PF_TQ * PF_ROW + 4 * PF_BC * PF_ROW + 1024) != cudaSuccess)
      return 3;
    configured = true;
  }
  DmMaps maps;
  if (dm_get_maps(kcache, vcache, n_blocks, n_kv, &maps)) return (int)cudaErrorInvalidValue;
  const dim3 grid((max_q_len + PF_TQ - 1) / PF_TQ, n_kv, B);
  return (int)trl_launch(attn_prefill_kernel<false>, grid, dim3(G * 32), smem, (cudaStream_t)stream, (const bf16*)q,
                         (const bf16*)gate_src, gate_ld, (const bf16*)kcache, (const bf16*)vcache,
                         (const float*)nullptr, (const float*)nullptr,
                         (const int*)block_table, max_blocks, (const int*)q_start, (const int*)q_len,
                         (const int*)positions, (bf16*)out, n_q, n_kv, scale * 1.4426950408889634f, gated, maps.mk, maps.mv,
                         maps.mode3d, n_blocks);
}

// The same over an e4m3 pool: kcache / vcache are the e4m3 bytes of one layer, kscale / vscale its
// fp32 row scales [blocks, hkv, 16].
TRL_API int trl_attn_prefill_fp8(const void* q, const void* gate_src, int gate_ld, const void* kcache,
                                 const void* vcache, const void* kscale, const void* vscale,
                                 const void* block_table, int max_blocks, const void* q_start, const void* q_len,
                                 const void* positions, void* out, int B, int max_q_len, int n_q, int n_kv, int D,
                                 float scale, int gated, void* stream) {
  const int G = n_kv > 0 ? n_q / n_kv : 0;
  if (D != PF_D || G < 1 || G > 8 || n_q % n_kv != 0 || B <= 0 || max_q_len <= 0) return (int)cudaErrorInvalidValue;
  constexpr size_t kv_bytes = (size_t)2 * PF_BC * PF_ROW + (size_t)4 * PF_BC * PF_D + (size_t)4 * PF_BC * sizeof(float) + 1024;
  const size_t smem = (size_t)G * PF_TQ * PF_ROW + kv_bytes;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(8 * PF_TQ * PF_ROW + kv_bytes)) != cudaSuccess)
      return 3;
    configured = true;
  }
  const dim3 grid((max_q_len + PF_TQ - 1) / PF_TQ, n_kv, B);
  return (int)trl_launch(attn_prefill_kernel<true>, grid, dim3(G * 32), smem, (cudaStream_t)stream, (const bf16*)q,
                         (const bf16*)gate_src, gate_ld, (const bf16*)kcache, (const bf16*)vcache,
                         (const float*)kscale, (const float*)vscale,
                         (const int*)block_table, max_blocks, (const int*)q_start, (const int*)q_len,
                         (const int*)positions, (bf16*)out, n_q, n_kv, scale * 1.4426950408889634f, gated, CUtensorMap{},
                         CUtensorMap{}, 0, 0);
}

TRL_API int trl_attn_paged_static(const void* q, const void* gate_src, int gate_ld, const void* kcache,
                                  const void* vcache, const void* block_table, int max_blocks,
                                  const void* seq_ids, const void* positions, void* out, int T, int n_q,
                                  int n_kv, int D, int n_splits, float scale, int gated, void* stream) {
  if (T <= 0 || n_q <= 0 || n_kv <= 0 || n_splits <= 0 || D <= 0) return (int)cudaErrorInvalidValue;
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
