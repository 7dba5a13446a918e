// Small memory-bound ops: embedding gather, standalone RMSNorm, SwiGLU on interleaved
// (gate, up) columns, row argmax, gather of rows, fused AdamW, NVFP4 (re)quantisation.
// Reference parity: kernels.py:30-200 (rmsnorm), :361-403 (silu_mul), :464-509
// (embedding) of packages/tilerl-kernels/src/tilerl_kernels; AdamW src/tilerl/autograd.py:466;
// requantize_fp4 src/tilerl/model.py:1255-1296.
#include "common.cuh"

namespace {

__global__ void embedding_kernel(const bf16* __restrict__ table, const int* ids,
                                 bf16* out, int H, int V) {
  pdl_launch_dependents(7);
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * H);
  if (id < 0 || id >= V) {   // never read outside the table: zero row + error word {BOUNDS, 1, token, id}
    if (threadIdx.x == 0) trl_set_error(TRL_ERR_BOUNDS, 1, t, id);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void gather_rows_kernel(const bf16* x, const int* idx,
                                   bf16* out, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)idx[t] * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void __launch_bounds__(256)
rmsnorm_kernel(const bf16* x, const float* __restrict__ w, bf16* out, int H,
               float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const bf16* xr = x + (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + i));
    ss += v.x * v.x + v.y * v.y;
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)H + eps);
  bf16* o = out + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + i));
    *reinterpret_cast<bf162*>(o + i) = __floats2bfloat162_rn(v.x * rstd * w[i], v.y * rstd * w[i + 1]);
  }
}

__global__ void swiglu_kernel(const bf16* gu, bf16* out, long n_out) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n_out; i += (long)gridDim.x * blockDim.x) {
    float2 v = __bfloat1622float2(reinterpret_cast<const bf162*>(gu)[i]);
    out[i] = __float2bfloat16(silu_f(v.x) * v.y);
  }
}

// Row argmax in two stages: (row, chunk) partial maxima, then one warp-level merge per row.
// Ties resolve to the lowest index.
constexpr int ARGMAX_CHUNKS = 64;
__device__ __forceinline__ void argmax_merge(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) best = ov, bi = oi;
}
__global__ void __launch_bounds__(256)
argmax_stage1_kernel(const float* logits, int ld, int V, float* pv,
                     int* pi) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, chunk = blockIdx.y;
  const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
  const int lo = chunk * per, hi = min(V, lo + per);
  const float* r = logits + (size_t)row * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) argmax_merge(best, bi, r[i], i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) sv[w] = best, si[w] = bi;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < 8; ++k) argmax_merge(best, bi, sv[k], si[k]);
    pv[row * ARGMAX_CHUNKS + chunk] = best;
    pi[row * ARGMAX_CHUNKS + chunk] = bi;
  }
}
__global__ void __launch_bounds__(64)
argmax_stage2_kernel(const float* pv, const int* pi, int* out) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  float best = pv[row * ARGMAX_CHUNKS + threadIdx.x];
  int bi = pi[row * ARGMAX_CHUNKS + threadIdx.x];
  __shared__ float sv[2];
  __shared__ int si[2];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = best, si[threadIdx.x >> 5] = bi;
  __syncthreads();
  if (threadIdx.x == 0) {
    argmax_merge(best, bi, sv[1], si[1]);
    // a row of NaN compares false everywhere and keeps the sentinel: it yields token 0, never a
    // wild index (the captured decode tick feeds this token to the next tick's embedding gather)
    out[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

// Fused AdamW on fp32 master + moments; optionally refreshes a bf16 copy.
__global__ void adamw_kernel(float* p, float* m, float* v,
                             const float* g, bf16* p_bf16, long n, float lr,
                             float b1, float b2, float eps, float wd, float c1, float c2, float gscale) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float gi = g[i] * gscale;
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi, v[i] = vi;
    float w = p[i] * (1.f - lr * wd);
    w -= lr * (mi / c1) / (sqrtf(vi / c2) + eps);
    p[i] = w;
    if (p_bf16) p_bf16[i] = __float2bfloat16(w);
  }
}

// NVFP4 quantisation of a dense [N, K] matrix with a given tensor scale: one thread
// per 16-element block; writes 8 packed bytes + 1 e4m3 scale.
template <typename T>
__global__ void quant_nvfp4_kernel(const T* __restrict__ w, const float* __restrict__ tscale,
                                   uint8_t* __restrict__ wq, uint8_t* sc, long nblocks) {
  const float ts = *tscale;
  for (long b = blockIdx.x * (long)blockDim.x + threadIdx.x; b < nblocks; b += (long)gridDim.x * blockDim.x) {
    float x[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      x[i] = (float)w[b * 16 + i];
      amax = fmaxf(amax, fabsf(x[i]));
    }
    float s = fminf(amax / 6.f / ts, 448.f);
    // round the block scale to e4m3 and read it back
    uint16_t s8;
    asm("{ .reg .b16 t; cvt.rn.satfinite.e4m3x2.f32 t, %1, %2; mov.b16 %0, t; }" : "=h"(s8) : "f"(0.f), "f"(s));
    const float sf = h2_to_f2(cvt_e4m3x2_to_h2(s8)).x;
    const float denom = sf * ts;
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const float a = denom > 0.f ? x[i] / denom : 0.f, c = denom > 0.f ? x[i + 1] / denom : 0.f;
      uint16_t byte;
      asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(byte) : "f"(c), "f"(a));
      packed[i / 8] |= ((uint32_t)(byte & 0xff)) << ((i % 8) * 4);
    }
    reinterpret_cast<uint2*>(wq)[b] = make_uint2(packed[0], packed[1]);
    sc[b] = (uint8_t)(s8 & 0xff);
  }
}

// NVFP4 -> bf16 dense matrix (8 elements per thread).
__global__ void dequant_nvfp4_kernel(const uint8_t* __restrict__ wq, const uint8_t* sc,
                                     const float* __restrict__ tscale, bf16* out, long n8) {
  const float ts = *tscale;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(wq)[i];
    const uint16_t s2 = (uint16_t)sc[i >> 1];
    const float s = h2_to_f2(cvt_e4m3x2_to_h2(s2)).x * ts;
    uint32_t h[4];
    cvt_e2m1x8_to_h2x4(w, h);
    uint4 o;
    float2 f;
    f = h2_to_f2(h[0]); o.x = f2_to_bf162_bits(f.x * s, f.y * s);
    f = h2_to_f2(h[1]); o.y = f2_to_bf162_bits(f.x * s, f.y * s);
    f = h2_to_f2(h[2]); o.z = f2_to_bf162_bits(f.x * s, f.y * s);
    f = h2_to_f2(h[3]); o.w = f2_to_bf162_bits(f.x * s, f.y * s);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// out[i] = a[i] + b[i] (bf16), used by the large-M path where the residual add is
// not folded into a GEMV epilogue.
__global__ void add_kernel(const bf16* a, const bf16* b, bf16* out, long n2) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n2; i += (long)gridDim.x * blockDim.x) {
    float2 x = __bfloat1622float2(reinterpret_cast<const bf162*>(a)[i]);
    float2 y = __bfloat1622float2(reinterpret_cast<const bf162*>(b)[i]);
    reinterpret_cast<bf162*>(out)[i] = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
  }
}

// Device-side tick advance: feed each row's sampled token back as the next input,
// bump position / KV length, recompute the KV write slot from the block table and
// append the token to a history row.  Lets a captured decode tick be replayed
// back to back with no host round trip.
__global__ void decode_advance_kernel(const int* tok, int* ids,
                                      int* pos, int* smap,
                                      int* kvlen, const int* __restrict__ table, int B,
                                      int max_blocks, int* hist, int hist_cap,
                                      int* hist_n) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < B) {
    const int p = pos[r] + 1;
    ids[r] = tok[r];
    pos[r] = p;
    kvlen[r] = p + 1;
    const int pg = min(p / 16, max_blocks - 1);
    smap[r] = table[(size_t)r * max_blocks + pg] * 16 + (p % 16);
    const int n = *hist_n;
    if (hist && n < hist_cap) hist[(size_t)r * hist_cap + n] = tok[r];
  }
  __syncthreads();
  if (r == 0) *hist_n = min(*hist_n + 1, hist_cap);
}

template <typename T>
__global__ void absmax_kernel(const T* __restrict__ w, long n, float* out) {
  __shared__ float red[32];
  float a = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    a = fmaxf(a, fabsf((float)w[i]));
  a = block_max(a, red);
  if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(out), __float_as_int(a));  // a >= 0
}

__global__ void tscale_kernel(const float* amax, float* ts) { *ts = fmaxf(*amax, 1e-30f) / (6.f * 448.f); }


// ---------------------------------------------------------------------------------------
// Seeded temperature sampling of whole rows (top_p = 1, top_k = 0: the RL rollout setting):
// softmax(logits / T) by two block reductions, then the inverse CDF at u = hash(seed).  Each
// of the 1024 threads owns one contiguous chunk of the vocabulary; a block scan over the chunk
// sums finds the chunk that holds u * total and its owner walks it.  One CTA per row, no host
// round trip per row; the same (seed, logits) always give the same token.  Also returns the
// log-probability of the token under the sampled distribution.
// Parity: `sample_batch` of tilerl_kernels/reference.py:1656-1720 (there a torch multinomial
// on the host generator); per-position seeds as in engine.py:206 of the reference.
__device__ __forceinline__ float sample_u01(unsigned long long seed) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(1024)
sample_softmax_kernel(const float* logits, int ld, const int* rows,
                      const long long* seeds, const float* inv_temp,
                      int* out_tok, float* out_lp, int V) {
  __shared__ float s_red[32];
  __shared__ float s_sum[1024];
  __shared__ float s_bcast[2];
  __shared__ int s_pick;
  const int b = blockIdx.x, tid = threadIdx.x;
  pdl_wait();
  const float* lg = logits + (size_t)rows[b] * ld;
  const float it = inv_temp[b];
  const int C = (V + 1023) / 1024;
  const int lo = min(V, tid * C), hi = min(V, lo + C);
  float mx = -INFINITY;
  for (int i = lo; i < hi; ++i) mx = fmaxf(mx, lg[i] * it);
  mx = warp_max(mx);
  if ((tid & 31) == 0) s_red[tid >> 5] = mx;
  __syncthreads();
  if (tid < 32) {
    float v = warp_max(s_red[tid]);
    if (tid == 0) s_bcast[0] = v;
  }
  __syncthreads();
  mx = s_bcast[0];
  float sum = 0.f;
  for (int i = lo; i < hi; ++i) sum += __expf(lg[i] * it - mx);
  s_sum[tid] = sum;
  __syncthreads();
  // inclusive scan of the 1024 chunk sums by the first warp (32 values per lane)
  if (tid < 32) {
    float run = 0.f;
    for (int j = 0; j < 32; ++j) run += s_sum[tid * 32 + j];
    float incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, incl, o);
      if (tid >= o) incl += n;
    }
    float acc = incl - run;   // exclusive prefix of this lane's 32 chunks
    for (int j = 0; j < 32; ++j) {
      const float v = s_sum[tid * 32 + j];
      s_sum[tid * 32 + j] = acc;   // becomes the exclusive prefix of chunk tid*32+j
      acc += v;
    }
    if (tid == 31) s_bcast[1] = acc;   // total
  }
  if (tid == 0) s_pick = -1;
  __syncthreads();
  const float total = s_bcast[1];
  const float target = sample_u01((unsigned long long)seeds[b]) * total;
  const float begin = s_sum[tid];
  const float end = (tid == 1023) ? total : s_sum[tid + 1];
  // the chunk whose [begin, end) holds the target; the last non-empty chunk takes rounding spill
  if (hi > lo && target >= begin && (target < end || end >= total)) atomicMax(&s_pick, tid);
  __syncthreads();
  if (tid == max(s_pick, 0) && (s_pick >= 0 || tid == 0)) {
    float acc = begin;
    int tok = hi > lo ? hi - 1 : 0;
    float e_tok = 0.f;
    for (int i = lo; i < hi; ++i) {
      const float e = __expf(lg[i] * it - mx);
      acc += e;
      if (acc > target && e > 0.f) {
        tok = i, e_tok = e;
        break;
      }
      if (e > 0.f) tok = i, e_tok = e;
    }
    out_tok[b] = tok;
    out_lp[b] = logf(fmaxf(e_tok, 1e-45f)) - logf(total);
  }
}


// ---------------------------------------------------------------------------------------
// Top-k / top-p (nucleus) sampling on the device, one CTA per row, no sort.
//
// Every logit is keyed by its distance below the row maximum in units of 2^-19 nat
// (q = (max - s) * 2^19, clamped to 24 bits: anything more than 32 nats down has probability
// < 2e-14 and is never drawn) and weighted by an integer mass m = exp(-(max - s)) * 2^40, so all
// sums are exact integers and the result does not depend on the order of the atomics.
//   top-k : the k-th smallest key by a 3-digit radix select over counts; keys equal to it are kept.
//   top-p : the smallest key whose cumulative mass (in descending probability) reaches top_p * Z,
//           by the same radix select over masses; the token that crosses the bound is kept.
//   draw  : inverse CDF at u = hash(seed) over the kept masses in (thread, stride) order.
// The order of the inverse CDF does not change the distribution, only which token a given u maps to.
__device__ __forceinline__ unsigned nuc_key(float d) {
  const float q = d * 524288.f;
  return (q >= 16777215.f || !(q == q)) ? 0xFFFFFFu : (unsigned)q;
}
__device__ __forceinline__ unsigned long long nuc_mass(float d, unsigned q) {
  return q == 0xFFFFFFu ? 0ull : (unsigned long long)(__expf(-d) * 1099511627776.f);
}

struct NucShared {
  unsigned long long hist[256];
  unsigned long long part[1024];
  float red[32];
  float mx;
  unsigned sel;
  unsigned long long need;
  unsigned long long total;
  int pick;
  int ncand;
  float cd[1024];                 // candidates of the small path: distance below the maximum,
  int ci[1024];                   // vocabulary index,
  unsigned long long cm[1024];    // integer mass
};
constexpr int NUC_CAP = 1024;
constexpr int NUC_U = 8;   // vocabulary loads in flight per thread in every pass (the passes are latency-bound otherwise)

// Sum of one value per thread over the CTA (all threads get the result).
__device__ __forceinline__ unsigned long long nuc_block_sum(NucShared& sh, unsigned long long v, int tid) {
  __syncthreads();
  sh.part[tid] = v;
  __syncthreads();
  if (tid < 32) {
    unsigned long long a = 0;
    for (int j = 0; j < 32; ++j) a += sh.part[tid * 32 + j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (tid == 0) sh.total = a;
  }
  __syncthreads();
  return sh.total;
}

// Smallest 24-bit key t such that the weight (count or mass) of {q <= t, q <= qcap} reaches `need`
// (0xFFFFFF when the whole row does not reach it).
// Warp 0 scans the 256-bin histogram for the bin where the running weight reaches `need` and
// leaves the extended prefix in sh.sel and the weight still wanted inside that bin in sh.need.
__device__ __forceinline__ void nuc_pick(NucShared& sh, unsigned prefix, unsigned long long need, int tid) {
  if (tid < 32) {
    unsigned long long loc[8], run = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      loc[j] = sh.hist[tid * 8 + j];
      run += loc[j];
    }
    unsigned long long incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
      if (tid >= o) incl += n;
    }
    const unsigned long long excl = incl - run;
    const bool has = excl < need && incl >= need;
    const unsigned ball = __ballot_sync(0xffffffffu, has);
    if (ball == 0u) {
      if (tid == 0) {
        sh.sel = (prefix << 8) | 255u;
        sh.need = need;
      }
    } else if (has) {
      unsigned long long cum = excl;
      int b = 7;
      bool found = false;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (!found) {
          if (j == 7 || cum + loc[j] >= need) b = j, found = true;
          else cum += loc[j];
        }
      }
      sh.sel = (prefix << 8) | (unsigned)(tid * 8 + b);
      sh.need = need - cum;
    }
  }
}

__device__ unsigned nuc_select(NucShared& sh, const float* lg, float it, float mx, int V, bool by_mass,
                               unsigned long long need, unsigned qcap, int tid) {
  unsigned prefix = 0;
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = 16 - 8 * pass;
    __syncthreads();
    if (tid < 256) sh.hist[tid] = 0ull;
    __syncthreads();
    for (int i0 = tid; i0 < V; i0 += NUC_U * 1024) {   // NUC_U loads in flight per thread
      float x[NUC_U];
#pragma unroll
      for (int u = 0; u < NUC_U; ++u) x[u] = i0 + u * 1024 < V ? lg[i0 + u * 1024] : 0.f;
#pragma unroll
      for (int u = 0; u < NUC_U; ++u) {
        if (i0 + u * 1024 >= V) continue;
        const float d = mx - x[u] * it;
        const unsigned q = nuc_key(d);
        if (q > qcap) continue;
        if (pass > 0 && (q >> (shift + 8)) != prefix) continue;
        const unsigned long long w = by_mass ? nuc_mass(d, q) : 1ull;
        if (w) atomicAdd(&sh.hist[(q >> shift) & 255u], w);
      }
    }
    __syncthreads();
    nuc_pick(sh, prefix, need, tid);
    __syncthreads();
    prefix = sh.sel;
    need = sh.need;
  }
  return prefix;
}

__global__ void __launch_bounds__(1024)
sample_nucleus_kernel(const float* logits, int ld, const int* rows,
                      const long long* seeds, const float* inv_temp,
                      const int* top_k, const float* top_p, int* out_tok,
                      float* out_lp, int V) {
  __shared__ NucShared sh;
  const int b = blockIdx.x, tid = threadIdx.x;
  pdl_wait();
  const float* lg = logits + (size_t)rows[b] * ld;
  const float it = inv_temp[b];
  float mx = -INFINITY;
  for (int i0 = tid; i0 < V; i0 += NUC_U * 1024) {
    float x[NUC_U];
#pragma unroll
    for (int u = 0; u < NUC_U; ++u) x[u] = i0 + u * 1024 < V ? lg[i0 + u * 1024] * it : -INFINITY;
#pragma unroll
    for (int u = 0; u < NUC_U; ++u) mx = fmaxf(mx, x[u]);
  }
  mx = warp_max(mx);
  if ((tid & 31) == 0) sh.red[tid >> 5] = mx;
  __syncthreads();
  if (tid < 32) {
    const float v = warp_max(sh.red[tid]);
    if (tid == 0) sh.mx = v;
  }
  __syncthreads();
  mx = sh.mx;
  if (!(mx > -INFINITY)) {   // nothing to draw from (all masked): token 0, logprob 0
    if (tid == 0) out_tok[b] = 0, out_lp[b] = 0.f;
    return;
  }
  const int k = top_k[b];
  const float p = top_p[b];
  unsigned qcut = 0xFFFFFFu;
  if (k > 0 && k < V) qcut = nuc_select(sh, lg, it, mx, V, false, (unsigned long long)k, 0xFFFFFFu, tid);
  if (k > 0 && k < V && k <= NUC_CAP / 2) {
    // Small path (the served default, top_k of a few tens): the tokens that survive top-k are
    // compacted into shared memory in one pass and everything after that (normaliser, nucleus
    // bound, draw) runs over those few entries instead of over the vocabulary again.  The
    // compaction order is not deterministic, so nothing below depends on it: sums are integer,
    // and the inverse CDF runs in vocabulary-index order.
    if (tid == 0) sh.ncand = 0;
    __syncthreads();
    for (int i0 = tid; i0 < V; i0 += NUC_U * 1024) {
      float x[NUC_U];
#pragma unroll
      for (int u = 0; u < NUC_U; ++u) x[u] = i0 + u * 1024 < V ? lg[i0 + u * 1024] : 0.f;
#pragma unroll
      for (int u = 0; u < NUC_U; ++u) {
        const float d = mx - x[u] * it;
        if (i0 + u * 1024 < V && nuc_key(d) <= qcut) {
          const int pos = atomicAdd(&sh.ncand, 1);
          if (pos < NUC_CAP) sh.cd[pos] = d, sh.ci[pos] = i0 + u * 1024;
        }
      }
    }
    __syncthreads();
    const int n = sh.ncand;
    if (n <= NUC_CAP) {
      const bool valid = tid < n;
      const float my_d = valid ? sh.cd[tid] : 0.f;
      const unsigned my_q = valid ? nuc_key(my_d) : 0xFFFFFFu;
      const unsigned long long my_m = valid ? nuc_mass(my_d, my_q) : 0ull;
      const int my_i = valid ? sh.ci[tid] : 0x7fffffff;
      unsigned qp = 0xFFFFFFu;
      if (p < 1.f) {
        const unsigned long long z = nuc_block_sum(sh, my_m, tid);
        unsigned long long want = (unsigned long long)((double)fmaxf(p, 0.f) * (double)z);
        if (want < 1ull) want = 1ull;
        unsigned prefix = 0;
        for (int pass = 0; pass < 3; ++pass) {   // the same radix select, over the candidates
          const int shift = 16 - 8 * pass;
          __syncthreads();
          if (tid < 256) sh.hist[tid] = 0ull;
          __syncthreads();
          if (my_m && (pass == 0 || (my_q >> (shift + 8)) == prefix)) atomicAdd(&sh.hist[(my_q >> shift) & 255u], my_m);
          __syncthreads();
          nuc_pick(sh, prefix, want, tid);
          __syncthreads();
          prefix = sh.sel;
          want = sh.need;
        }
        qp = prefix;
      }
      const bool kept = valid && my_m > 0ull && my_q <= qp;
      const unsigned long long total = nuc_block_sum(sh, kept ? my_m : 0ull, tid);
      __syncthreads();
      sh.cm[tid] = kept ? my_m : 0ull;
      if (!valid) sh.ci[tid] = 0x7fffffff;
      if (tid == 0) sh.pick = -1;
      __syncthreads();
      if (total == 0ull) {
        if (tid == 0) out_tok[b] = 0, out_lp[b] = 0.f;
        return;
      }
      unsigned long long target = (unsigned long long)((double)sample_u01((unsigned long long)seeds[b]) * (double)total);
      if (target >= total) target = total - 1ull;
      if (kept) {
        unsigned long long before = 0ull;      // mass of the kept candidates with a smaller index
        for (int c = 0; c < n; ++c) before += sh.ci[c] < my_i ? sh.cm[c] : 0ull;
        if (target >= before && target < before + my_m) {   // exactly one candidate
          out_tok[b] = my_i;
          out_lp[b] = logf((float)my_m) - logf((float)total);
        }
      }
      return;
    }
  }
  if (p < 1.f) {
    unsigned long long z = 0;
    for (int i0 = tid; i0 < V; i0 += NUC_U * 1024) {
      float x[NUC_U];
#pragma unroll
      for (int u = 0; u < NUC_U; ++u) x[u] = i0 + u * 1024 < V ? lg[i0 + u * 1024] : 0.f;
#pragma unroll
      for (int u = 0; u < NUC_U; ++u) {
        const float d = mx - x[u] * it;
        const unsigned q = nuc_key(d);
        if (i0 + u * 1024 < V && q <= qcut) z += nuc_mass(d, q);
      }
    }
    z = nuc_block_sum(sh, z, tid);
    unsigned long long want = (unsigned long long)((double)fmaxf(p, 0.f) * (double)z);
    if (want < 1ull) want = 1ull;
    const unsigned qp = nuc_select(sh, lg, it, mx, V, true, want, qcut, tid);
    qcut = min(qcut, qp);
  }
  // kept mass per thread over its strided elements, exclusive prefix over threads
  unsigned long long mine = 0;
  for (int i0 = tid; i0 < V; i0 += NUC_U * 1024) {
    float x[NUC_U];
#pragma unroll
    for (int u = 0; u < NUC_U; ++u) x[u] = i0 + u * 1024 < V ? lg[i0 + u * 1024] : 0.f;
#pragma unroll
    for (int u = 0; u < NUC_U; ++u) {
      const float d = mx - x[u] * it;
      const unsigned q = nuc_key(d);
      if (i0 + u * 1024 < V && q <= qcut) mine += nuc_mass(d, q);
    }
  }
  __syncthreads();
  sh.part[tid] = mine;
  if (tid == 0) sh.pick = -1;
  __syncthreads();
  if (tid < 32) {
    unsigned long long run = 0;
    for (int j = 0; j < 32; ++j) run += sh.part[tid * 32 + j];
    unsigned long long incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
      if (tid >= o) incl += n;
    }
    unsigned long long acc = incl - run;
    for (int j = 0; j < 32; ++j) {
      const unsigned long long v = sh.part[tid * 32 + j];
      sh.part[tid * 32 + j] = acc;
      acc += v;
    }
    if (tid == 31) sh.total = acc;
  }
  __syncthreads();
  const unsigned long long total = sh.total;
  if (total == 0ull) {   // cannot happen (the maximum has mass 2^40); keep the output defined
    if (tid == 0) out_tok[b] = 0, out_lp[b] = 0.f;
    return;
  }
  unsigned long long target = (unsigned long long)((double)sample_u01((unsigned long long)seeds[b]) * (double)total);
  if (target >= total) target = total - 1ull;
  const unsigned long long begin = sh.part[tid];
  if (mine > 0ull && target >= begin && target < begin + mine) sh.pick = tid;   // exactly one thread
  __syncthreads();
  if (tid == sh.pick) {
    unsigned long long acc = begin, m_tok = 0ull;
    int tok = -1;
    for (int i0 = tid; i0 < V && tok < 0; i0 += 8 * 1024) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + j * 1024;
        v[j] = i < V ? lg[i] * it : -INFINITY;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = mx - v[j];
        const unsigned q = nuc_key(d);
        const unsigned long long m = q <= qcut ? nuc_mass(d, q) : 0ull;
        if (tok < 0 && m > 0ull) {
          if (target < acc + m) tok = i0 + j * 1024, m_tok = m;
          acc += m;
        }
      }
    }
    out_tok[b] = max(tok, 0);
    out_lp[b] = logf(fmaxf((float)m_tok, 1.f)) - logf((float)total);
  }
}

// ---------------------------------------------------------------------------------------
// LoRA delta of a served projection, two small kernels instead of a chain of library calls:
//   lora_a: t[tok, r] = sum_k xn[tok, k] * A[r, k]   (xn = x, or RMSNorm(x) * norm_w)
//   lora_b: y[tok, n] += s * sum_r t[tok, r] * B[n, r]
// grid (tokens, rank) and (tokens, ceil(N / 256)).  A, B are the fp32 trainable tensors.
// Parity: `_linear` of src/tilerl/model.py:379-385 (two `linear` calls there).
__global__ void __launch_bounds__(256)
lora_a_kernel(const bf16* x, int ldx, const float* __restrict__ norm_w, float eps,
              const float* __restrict__ A, float* t, int K, int R) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x, r = blockIdx.y;
  const bf16* xr = x + (size_t)tok * ldx;
  const float* ar = A + (size_t)r * K;
  float acc = 0.f, ss = 0.f;
  for (int k = threadIdx.x * 2; k < K; k += blockDim.x * 2) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + k));
    ss += v.x * v.x + v.y * v.y;
    if (norm_w != nullptr)
      acc += v.x * norm_w[k] * ar[k] + v.y * norm_w[k + 1] * ar[k + 1];
    else
      acc += v.x * ar[k] + v.y * ar[k + 1];
  }
  acc = block_sum(acc, red);
  __syncthreads();
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) t[(size_t)tok * R + r] = norm_w != nullptr ? acc * rsqrtf(ss / (float)K + eps) : acc;
}

__global__ void __launch_bounds__(256)
lora_b_kernel(const float* t, const float* __restrict__ B, bf16* y, int ldy, int N,
              int R, float s) {
  __shared__ float ts[64];
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x;
  if (threadIdx.x < R) ts[threadIdx.x] = t[(size_t)tok * R + threadIdx.x];
  __syncthreads();
  const int n = blockIdx.y * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const float* br = B + (size_t)n * R;
  float acc = 0.f;
  for (int r = 0; r < R; ++r) acc = fmaf(br[r], ts[r], acc);
  bf16* yp = y + (size_t)tok * ldy + n;
  *yp = __float2bfloat16(__bfloat162float(*yp) + s * acc);
}

// Speculative verify tick, greedy acceptance on the device.  Sequence b owns rows b*W .. b*W + q_len[b] - 1
// of the tick: row k carried the chain token c_k (c_0 the last committed token, c_1.. the drafts) and
// `tok[b*W + k]` is the trunk's argmax after it.  accept[b] = number of leading drafts the trunk
// reproduced (c_{k+1} == tok[k]); the GDN state plane stored after chain token accept[b] becomes the
// sequence's current one (cur[state_slots[b]], the index write of GdnStatePool.select_step).
// pack: [B*W argmax tokens ; B accept counts], one buffer for the host to fetch.
// Reference parity: the accept walk of spec.py:1071-1146 (src/tilerl), which the reference runs on the host.
__global__ void spec_accept_kernel(const int* tok, const int* chain, const int* q_len, const int* state_slots,
                                   int* cur, int* pack, int B, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = B * W;
  for (int i = threadIdx.x; i < t; i += blockDim.x) pack[i] = tok[i];
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const int n = q_len[b];
    int ok = 0;
    while (ok + 1 < n && tok[b * W + ok] == chain[b * W + ok + 1]) ++ok;
    pack[t + b] = ok;
    if (n > 0) cur[state_slots[b]] = ok;
  }
}

}  // namespace

TRL_API int trl_embedding(const void* table, const void* ids, void* out, int T, int H, int V, void* stream) {
  return (int)trl_launch(embedding_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream,
                         (const bf16*)table, (const int*)ids, (bf16*)out, H, V);
}
TRL_API int trl_gather_rows(const void* x, const void* idx, void* out, int T, int H, void* stream) {
  return (int)trl_launch(gather_rows_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream,
                         (const bf16*)x, (const int*)idx, (bf16*)out, H);
}
TRL_API int trl_rmsnorm(const void* x, const void* w, void* out, int T, int H, float eps, void* stream) {
  return (int)trl_launch(rmsnorm_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x,
                         (const float*)w, (bf16*)out, H, eps);
}
TRL_API int trl_swiglu(const void* gu, void* out, long n_out, void* stream) {
  const int grid = (int)min((n_out + 255) / 256, (long)148 * 8);
  return (int)trl_launch(swiglu_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const bf16*)gu,
                         (bf16*)out, n_out);
}
// scratch: M * 64 floats followed by M * 64 ints.
TRL_API int trl_spec_accept(const void* tok, const void* chain, const void* q_len, const void* state_slots, void* cur,
                            void* pack, int B, int W, void* stream) {
  if (B <= 0 || W <= 0) return (int)cudaErrorInvalidValue;
  return (int)trl_launch(spec_accept_kernel, dim3(1), dim3(128), 0, (cudaStream_t)stream, (const int*)tok,
                         (const int*)chain, (const int*)q_len, (const int*)state_slots, (int*)cur, (int*)pack, B, W);
}

TRL_API int trl_argmax(const void* logits, int ld, int M, int V, void* out, void* scratch, void* stream) {
  float* pv = (float*)scratch;
  int* pi = (int*)(pv + (size_t)M * ARGMAX_CHUNKS);
  cudaError_t e = trl_launch(argmax_stage1_kernel, dim3(M, ARGMAX_CHUNKS), dim3(256), 0, (cudaStream_t)stream,
                             (const float*)logits, ld, V, pv, pi);
  if (e != cudaSuccess) return (int)e;
  return (int)trl_launch(argmax_stage2_kernel, dim3(M), dim3(64), 0, (cudaStream_t)stream, (const float*)pv,
                         (const int*)pi, (int*)out);
}
// Stage 1 only (per-row chunk maxima) for the vocab-parallel argmax: pv/pi are [M, 64].
TRL_API int trl_argmax_stage1(const void* logits, int ld, int M, int V, void* pv, void* pi, void* stream) {
  return (int)trl_launch(argmax_stage1_kernel, dim3(M, ARGMAX_CHUNKS), dim3(256), 0, (cudaStream_t)stream,
                         (const float*)logits, ld, V, (float*)pv, (int*)pi);
}
TRL_API int trl_adamw(void* p, void* m, void* v, const void* g, void* p_bf16, long n, float lr, float b1,
                      float b2, float eps, float wd, int step, float gscale, void* stream) {
  const float c1 = 1.f - powf(b1, (float)step), c2 = 1.f - powf(b2, (float)step);
  const int grid = (int)min((n + 255) / 256, (long)148 * 16);
  adamw_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((float*)p, (float*)m, (float*)v, (const float*)g,
                                                       (bf16*)p_bf16, n, lr, b1, b2, eps, wd, c1, c2, gscale);
  return (int)cudaGetLastError();
}
// dtype: 0 = fp32, 1 = bf16.  amax_tmp: one fp32 of scratch (zeroed here).  If
// fixed_tscale != 0 the tensor scale in `tscale` is kept, else it is recomputed.
TRL_API int trl_quant_nvfp4(const void* w, int dtype, long N, long K, void* wq, void* scale, void* tscale,
                            void* amax_tmp, int fixed_tscale, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const long n = N * K, nb = n / 16;
  const int grid = (int)min((nb + 255) / 256, (long)148 * 16);
  if (!fixed_tscale) {
    cudaMemsetAsync(amax_tmp, 0, 4, st);
    if (dtype == 0) absmax_kernel<float><<<grid, 256, 0, st>>>((const float*)w, n, (float*)amax_tmp);
    else absmax_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)w, n, (float*)amax_tmp);
    tscale_kernel<<<1, 1, 0, st>>>((const float*)amax_tmp, (float*)tscale);
  }
  if (dtype == 0)
    quant_nvfp4_kernel<float><<<grid, 256, 0, st>>>((const float*)w, (const float*)tscale, (uint8_t*)wq, (uint8_t*)scale, nb);
  else
    quant_nvfp4_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)w, (const float*)tscale, (uint8_t*)wq, (uint8_t*)scale, nb);
  return (int)cudaGetLastError();
}

TRL_API int trl_dequant_nvfp4(const void* wq, const void* scale, const void* tscale, void* out, long N,
                              long K, void* stream) {
  const long n8 = N * K / 8;
  const int grid = (int)min((n8 + 255) / 256, (long)148 * 32);
  dequant_nvfp4_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)wq, (const uint8_t*)scale,
                                                               (const float*)tscale, (bf16*)out, n8);
  return (int)cudaGetLastError();
}
TRL_API int trl_add(const void* a, const void* b, void* out, long n, void* stream) {
  const long n2 = n / 2;
  const int grid = (int)min((n2 + 255) / 256, (long)148 * 16);
  return (int)trl_launch(add_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const bf16*)a,
                         (const bf16*)b, (bf16*)out, n2);
}

TRL_API int trl_decode_advance(const void* tok, void* ids, void* pos, void* smap, void* kvlen,
                               const void* table, int B, int max_blocks, void* hist, int hist_cap,
                               void* hist_n, void* stream) {
  return (int)trl_launch(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, (cudaStream_t)stream,
                         (const int*)tok, (int*)ids, (int*)pos, (int*)smap, (int*)kvlen, (const int*)table,
                         B, max_blocks, (int*)hist, hist_cap, (int*)hist_n);
}

// rows[b]: logits row to sample; seeds[b]; inv_temp[b] = 1 / temperature.  One CTA per entry.
TRL_API int trl_sample_softmax(const void* logits, int ld, const void* rows, const void* seeds,
                               const void* inv_temp, void* out_tok, void* out_lp, int B, int V, void* stream) {
  if (B <= 0) return 0;
  return (int)trl_launch(sample_softmax_kernel, dim3(B), dim3(1024), 0, (cudaStream_t)stream, (const float*)logits,
                         ld, (const int*)rows, (const long long*)seeds, (const float*)inv_temp, (int*)out_tok,
                         (float*)out_lp, V);
}

// As trl_sample_softmax, with a per-entry top_k (0 = off) and top_p (>= 1 = off) restriction.
TRL_API int trl_sample_nucleus(const void* logits, int ld, const void* rows, const void* seeds,
                               const void* inv_temp, const void* top_k, const void* top_p, void* out_tok,
                               void* out_lp, int B, int V, void* stream) {
  if (B <= 0) return 0;
  return (int)trl_launch(sample_nucleus_kernel, dim3(B), dim3(1024), 0, (cudaStream_t)stream,
                         (const float*)logits, ld, (const int*)rows, (const long long*)seeds,
                         (const float*)inv_temp, (const int*)top_k, (const float*)top_p, (int*)out_tok,
                         (float*)out_lp, V);
}

// y[T, N] (bf16, in place) += s * (norm(x) A^T) B^T.  t: fp32 scratch [T, R]; R <= 64; K even.
TRL_API int trl_lora_add(const void* x, int ldx, const void* norm_w, float eps, const void* A, const void* B,
                         void* t, void* y, int ldy, int T, int N, int K, int R, float s, void* stream) {
  if (R > 64 || R < 1 || (K & 1)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = trl_launch(lora_a_kernel, dim3(T, R), dim3(256), 0, st, (const bf16*)x, ldx, (const float*)norm_w,
                             eps, (const float*)A, (float*)t, K, R);
  if (e != cudaSuccess) return (int)e;
  return (int)trl_launch(lora_b_kernel, dim3(T, (N + 255) / 256), dim3(256), 0, st, (const float*)t,
                         (const float*)B, (bf16*)y, ldy, N, R, s);
}
