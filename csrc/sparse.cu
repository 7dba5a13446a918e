// Page selection for sparse-KV decode attention on the device.
//
//   quest_score_kernel : one CTA per early page of a sequence.  Reads the page's K rows
//                        ([hkv, 16, D] bf16) once, forms the per-dimension min / max over its 16
//                        tokens in registers and scores the page with the Quest upper bound
//                        sum_{kv head} sum_{query head of the group} sum_d max(q_d min_d, q_d max_d).
//                        No bounds tensor is materialised.
//   page_mean_kernel   : mean key of a page per kv head (input of the learned indexer's projection);
//   index_score_kernel : the learned indexer's page score, sum over index heads of relu(q . k) / sqrt(d).
//   topk_pages_kernel  : one CTA per sequence.  k-th largest score by a 4-pass radix select over
//                        order-preserving keys, then the kept page indices in ascending order
//                        (all scores above the k-th, and the first equals in page order until k).
//
// The sums run in a fixed order (dims inside a lane, lanes by shuffle tree, query heads, kv heads),
// so a selection does not depend on scheduling.
//
// Reference parity: page_bounds kernels of packages/tilerl-kernels/src/tilerl_kernels/kernels.py:558-622 and
// the device selection of src/tilerl/sparse_engine.py:768; the reference keeps a bounds cache, here
// a refresh re-reads the K pages (64 MB per layer at 32k context, a few microseconds of HBM time).
#include "common.cuh"

namespace {

constexpr int QS_D = 256;                          // head dim served (8 dims per lane)
constexpr int QS_PAGE = 16;
constexpr int TK_THREADS = 1024;

__global__ void __launch_bounds__(128)
quest_score_kernel(const bf16* q, const bf16* kcache, const int* table, float* scores, int n_q, int n_kv) {
  __shared__ float s_part[32];
  pdl_launch_dependents();
  pdl_wait();
  const int page = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int G = n_q / n_kv;
  const int blk = table[page];
  float mine = 0.f;                                // this warp's kv heads, in ascending order
  for (int kvh = warp; kvh < n_kv; kvh += nw) {
    const bf16* rows = kcache + ((size_t)blk * n_kv + kvh) * QS_PAGE * QS_D + lane * 8;
    float lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) lo[i] = INFINITY, hi[i] = -INFINITY;
#pragma unroll 4
    for (int r = 0; r < QS_PAGE; ++r) {
      const uint4 v = *reinterpret_cast<const uint4*>(rows + (size_t)r * QS_D);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = bf162_bits_to_f2(w[i]);
        lo[2 * i] = fminf(lo[2 * i], f.x), hi[2 * i] = fmaxf(hi[2 * i], f.x);
        lo[2 * i + 1] = fminf(lo[2 * i + 1], f.y), hi[2 * i + 1] = fmaxf(hi[2 * i + 1], f.y);
      }
    }
    for (int g = 0; g < G; ++g) {
      const uint4 v = *reinterpret_cast<const uint4*>(q + ((size_t)(kvh * G + g)) * QS_D + lane * 8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = bf162_bits_to_f2(w[i]);
        s += fmaxf(f.x * lo[2 * i], f.x * hi[2 * i]);
        s += fmaxf(f.y * lo[2 * i + 1], f.y * hi[2 * i + 1]);
      }
      mine += warp_sum(s);
    }
  }
  if (lane == 0) s_part[warp] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w2 = 0; w2 < nw; ++w2) tot += s_part[w2];
    scores[page] = tot;
  }
}

// Mean key of a page per kv head: pooled[page][kvh * D + d] = mean over the page's 16 tokens (fp32).  The learned
// indexer projects these rows with its own small matrix (a library GEMM) before scoring.
__global__ void __launch_bounds__(128)
page_mean_kernel(const bf16* kcache, const int* table, float* pooled, int n_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int page = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int blk = table[page];
  for (int kvh = warp; kvh < n_kv; kvh += nw) {
    const bf16* rows = kcache + ((size_t)blk * n_kv + kvh) * QS_PAGE * QS_D + lane * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 4
    for (int r = 0; r < QS_PAGE; ++r) {
      const uint4 v = *reinterpret_cast<const uint4*>(rows + (size_t)r * QS_D);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = bf162_bits_to_f2(w[i]);
        acc[2 * i] += f.x, acc[2 * i + 1] += f.y;
      }
    }
    float* dst = pooled + ((size_t)page * n_kv + kvh) * QS_D + lane * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0] * 0.0625f, acc[1] * 0.0625f, acc[2] * 0.0625f, acc[3] * 0.0625f);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4] * 0.0625f, acc[5] * 0.0625f, acc[6] * 0.0625f, acc[7] * 0.0625f);
  }
}

// Learned-indexer score of a page: sum over index heads of relu(q_idx[h] . k_idx[page][h]) / sqrt(d).
// q_idx [H, d], k_idx [pages, H, d] fp32; one warp per head, heads summed in ascending order.
__global__ void __launch_bounds__(128)
index_score_kernel(const float* q_idx, const float* k_idx, float* scores, int H, int d) {
  __shared__ float s_part[32];
  pdl_launch_dependents();
  pdl_wait();
  const int page = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float mine = 0.f;
  for (int h = warp; h < H; h += nw) {
    const float* kr = k_idx + ((size_t)page * H + h) * d;
    const float* qr = q_idx + (size_t)h * d;
    float s = 0.f;
    for (int i = lane; i < d; i += 32) s = fmaf(qr[i], kr[i], s);
    s = warp_sum(s);
    mine += fmaxf(s, 0.f);
  }
  if (lane == 0) s_part[warp] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w2 = 0; w2 < nw; ++w2) tot += s_part[w2];
    scores[page] = tot * rsqrtf((float)d);
  }
}

// larger float <=> larger key
__device__ __forceinline__ uint32_t tk_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(TK_THREADS)
topk_pages_kernel(const float* scores, int n, int k, long long* sel) {
  __shared__ unsigned int s_hist[256];
  __shared__ unsigned int s_prefix, s_need;
  __shared__ int s_gt[TK_THREADS], s_eq[TK_THREADS];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  if (k >= n) {                                    // everything is kept
    for (int i = tid; i < n; i += TK_THREADS) sel[i] = i;
    return;
  }
  // ---- the k-th largest key, eight bits at a time from the top
  if (tid == 0) s_prefix = 0u, s_need = (unsigned int)k;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += TK_THREADS) s_hist[i] = 0u;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < n; i += TK_THREADS) {
      const uint32_t key = tk_key(scores[i]);
      if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned int need = s_need;
      int b = 255;
      for (; b > 0; --b) {                         // buckets from the largest digit down
        if (s_hist[b] >= need) break;
        need -= s_hist[b];
      }
      s_prefix = prefix | ((uint32_t)b << shift);
      s_need = need;                               // how many of this bucket (at the last pass: of the equals) are kept
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;
  const int need_eq = (int)s_need;
  // ---- ascending compaction: thread t owns the contiguous pages [t * seg, (t + 1) * seg)
  const int seg = (n + TK_THREADS - 1) / TK_THREADS;
  const int p0 = min(n, tid * seg), p1 = min(n, p0 + seg);
  int gt = 0, eq = 0;
  for (int i = p0; i < p1; ++i) {
    const uint32_t key = tk_key(scores[i]);
    gt += key > kth, eq += key == kth;
  }
  s_gt[tid] = gt, s_eq[tid] = eq;
  __syncthreads();
  if (tid == 0) {                                  // exclusive prefix sums (1024 entries, once per refresh)
    int ag = 0, ae = 0;
    for (int i = 0; i < TK_THREADS; ++i) {
      const int g2 = s_gt[i], e2 = s_eq[i];
      s_gt[i] = ag, s_eq[i] = ae;
      ag += g2, ae += e2;
    }
  }
  __syncthreads();
  int eq_before = s_eq[tid];
  int out = s_gt[tid] + min(eq_before, need_eq);
  for (int i = p0; i < p1; ++i) {
    const uint32_t key = tk_key(scores[i]);
    if (key > kth) {
      sel[out++] = i;
    } else if (key == kth) {
      if (eq_before < need_eq) sel[out++] = i;
      ++eq_before;
    }
  }
}

}  // namespace

// scores[p] = Quest upper bound of page table[p] for the token whose prepared query rows are q [n_q, 256] bf16.
// kcache: [blocks, n_kv, 16, 256] bf16.
TRL_API int trl_quest_scores(const void* q, const void* kcache, const void* table, void* scores, int n_pages, int n_q,
                             int n_kv, int D, void* stream) {
  if (D != QS_D || n_pages <= 0 || n_kv <= 0 || n_q % n_kv != 0) return (int)cudaErrorInvalidValue;
  return (int)trl_launch(quest_score_kernel, dim3(n_pages), dim3(128), 0, (cudaStream_t)stream, (const bf16*)q,
                         (const bf16*)kcache, (const int*)table, (float*)scores, n_q, n_kv);
}

// sel[0 .. min(k, n)) = indices of the k largest scores, ascending (ties at the k-th score: lowest indices first).
TRL_API int trl_topk_pages(const void* scores, int n, int k, void* sel, void* stream) {
  if (n <= 0 || k <= 0) return (int)cudaErrorInvalidValue;
  return (int)trl_launch(topk_pages_kernel, dim3(1), dim3(TK_THREADS), 0, (cudaStream_t)stream, (const float*)scores, n, k,
                         (long long*)sel);
}

// pooled[p] = mean K row of page table[p] per kv head: [n_pages, n_kv * 256] fp32.
TRL_API int trl_page_mean(const void* kcache, const void* table, void* pooled, int n_pages, int n_kv, int D, void* stream) {
  if (D != QS_D || n_pages <= 0 || n_kv <= 0) return (int)cudaErrorInvalidValue;
  return (int)trl_launch(page_mean_kernel, dim3(n_pages), dim3(128), 0, (cudaStream_t)stream, (const bf16*)kcache,
                         (const int*)table, (float*)pooled, n_kv);
}

// scores[p] = sum_h relu(q_idx[h] . k_idx[p][h]) / sqrt(d); q_idx [H, d], k_idx [n_pages, H, d], fp32.
TRL_API int trl_index_scores(const void* q_idx, const void* k_idx, void* scores, int n_pages, int H, int d, void* stream) {
  if (n_pages <= 0 || H <= 0 || d <= 0) return (int)cudaErrorInvalidValue;
  return (int)trl_launch(index_score_kernel, dim3(n_pages), dim3(128), 0, (cudaStream_t)stream, (const float*)q_idx,
                         (const float*)k_idx, (float*)scores, H, d);
}
