// tcgen05 block-scaled NVFP4 GEMM (and its activation quantiser).
//
//   Y[tok, n] = epi( tscale * sum_j rs[col] * sum_k Xq[col, k] sfx[col, k/16] * Wq[n, k] sfw[n, k/16] )
//
// The *weight* is the MMA "A" operand (128 rows per tile -> TMEM lanes), the
// activation columns are the "B" operand (BN in {16..256} -> TMEM columns): a decode
// tick with a handful of tokens still fills the 128-lane datapath, and the weight
// stream -- the only large operand -- is read exactly once by TMA straight into
// 128B-swizzled shared memory with no ALU decode at all.
//
// Activation precision is a *column count* here: token t occupies J consecutive
// columns holding successive NVFP4 residual terms x ~= x1 + x2 + ... (each with its
// own per-16 e4m3 scales and fp32 row scale), summed in the epilogue.  J = 1 is plain
// W4A4; J = 4 reproduces a bf16 activation to ~2^-9 while still running entirely on
// the FP4 tensor cores -- that is how the B = 1 decode tick reads its weights at
// HBM speed with bf16-accurate activations.
//
// Schedule: stream-K.  The (tile, k-tile) units are split evenly over one CTA per
// SM; a CTA whose range covers a whole tile finishes it from TMEM, otherwise it stores its
// partial tile into its own fp32 slot of a scratch buffer, and the last CTA of the tile to
// arrive (atomic counter, reset by that CTA) sums the slots in segment order -- bitwise
// reproducible, nothing to zero -- and runs the epilogue.  Small-N / large-K projections
// (down_proj, o_proj) therefore use every SM.
//
// Warp roles (192 threads): warp 0 = TMA producer (weight tiles are prefetched
// *before* griddepcontrol.wait, since they do not depend on the previous kernel),
// warp 1 = TMEM owner + MMA issuer (one elected lane), warps 2-5 = epilogue
// (tcgen05.ld, scale, residual / SwiGLU, store).  Every mbarrier wait is bounded: on
// expiry the CTA records an error word, raises a shared abort flag, frees its TMEM
// and returns.
//
// Scale factors use the 128x4 tiled layout the tensor core reads:
//   byte offset = ((row/128) * KT4 + k64) * 512 + (row%32)*16 + ((row%128)/32)*4 + (k16%4)
// so that one k-tile of a 128-row atom is 2 KB contiguous.
//
// No counterpart exists in the reference: its Blackwell kernel cell is empty
// (packages/tilerl-kernels/src/tilerl_kernels/registry.py:188-189); functionally this
// replaces linear_fp4_fp8 / linear_fp4_gemv / linear_fp4_mma8 (kernels_linear.py:924-1687).
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int TILE_N = 128;
constexpr int KT_BYTES = 128;   // bytes of K per row per k-tile (= 256 e2m1)
constexpr int KT_ELEMS = 256;
constexpr int GEMM_THREADS = 192;
constexpr int SF_ATOM = TC_SF_ATOM;    // bytes: 128 rows x 4 scales

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_STORE_F32 = 3 };

struct GemmParams {
  const uint8_t* sfw;    // weight scales, tiled
  const uint8_t* sfx;    // activation scales, tiled
  const float* tscale;   // weight tensor scale
  const float* rs;       // per-column activation scale [cols]
  const bf16* residual;  // [tokens, ldr]
  void* out;
  float* partial;        // [tiles, max_seg, BN/J, 128] fp32 split-K slots (no init needed)
  int* counters;         // [tiles], zero on entry, zero on exit
  int N, K, cols, tokens, J;
  int ldr, ldo;
  int n_tiles, c_tiles, nk, kt4;
  int max_seg;
  int w_tiled; // weights stored tile-contiguous [n_tiles, nk, 128 rows, 128 B]
  int split;   // 1: stream-K over (tile, k-tile) units; 0: whole tiles per CTA
  int sa, sb;  // stages of the weight ring and of the activation ring
  int epi;
};

__device__ __forceinline__ int owner_of(long long unit, long long U, int G) {
  int i = (int)((unit * G) / U);
  while ((long long)(i + 1) * U / G <= unit) ++i;
  while ((long long)i * U / G > unit) --i;
  return i;
}


// One finished (token, row) value of a whole tile.  Compile-time epilogue kind: the caller's
// unrolled loops stay free of branches, so the few epilogue warps overlap the tokens of a chunk.
template <int EPI>
__device__ __forceinline__ void epi_store(const GemmParams& p, int tok, int n, int lane, float v, float res) {
  if (EPI == EPI_SWIGLU) {
    const float other = __shfl_xor_sync(0xffffffffu, v, 1);
    const float y = __fdividef(v, 1.f + __expf(-v)) * other;
    if ((lane & 1) == 0 && tok < p.tokens && n + 1 < p.N)
      reinterpret_cast<bf16*>(p.out)[(size_t)tok * p.ldo + (n >> 1)] = __float2bfloat16(y);
  } else {
    v += res;
    if (tok < p.tokens && n < p.N) {
      if (EPI == EPI_STORE_F32)
        reinterpret_cast<float*>(p.out)[(size_t)tok * p.ldo + n] = v;
      else
        reinterpret_cast<bf16*>(p.out)[(size_t)tok * p.ldo + n] = __float2bfloat16(v);
    }
  }
}

// Epilogue of one accumulator tile: TMEM -> registers in chunks of CH columns, J columns summed
// per token with their activation scales, then either the final store (WHOLE) or this CTA's
// split-K slot.  tok_first = first token of the tile; slot_row = slot + row.
template <int BN, int J, int EPI, bool WHOLE>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t taddr0, const float* rs_s, float ts,
                                              int tok_first, int n, int lane, float* slot_row) {
  constexpr int CH = BN >= 32 ? 32 : 16;
  constexpr int TPC = CH / J;
#pragma unroll 1
  for (int c = 0; c < BN / CH; ++c) {
    uint32_t r[32];
    if (CH == 32) tc_ld32(taddr0 + (uint32_t)(c * CH), r); else tc_ld16(taddr0 + (uint32_t)(c * CH), r);
    const int tokc = tok_first + c * TPC;
    float res[TPC];
#pragma unroll
    for (int t = 0; t < TPC; ++t)   // issued before the wait and before any store of this chunk
      res[t] = (WHOLE && EPI == EPI_RESIDUAL && tokc + t < p.tokens && n < p.N)
                   ? __bfloat162float(p.residual[(size_t)(tokc + t) * p.ldr + n]) : 0.f;
    tc_wait_ld();
    float v[TPC];
#pragma unroll
    for (int t = 0; t < TPC; ++t) {
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < J; ++j) a = fmaf(__uint_as_float(r[t * J + j]), rs_s[c * CH + t * J + j], a);
      v[t] = a * ts;
    }
#pragma unroll
    for (int t = 0; t < TPC; ++t) {
      if (WHOLE) epi_store<EPI>(p, tokc + t, n, lane, v[t], res[t]);
      else slot_row[(size_t)(c * TPC + t) * TILE_N] = v[t];
    }
  }
}

template <int BN, int J>
__device__ __forceinline__ void epilogue_dispatch(const GemmParams& p, bool whole, uint32_t taddr0, const float* rs_s,
                                                  float ts, int tok_first, int n, int lane, float* slot_row) {
  if (!whole) epilogue_tile<BN, J, EPI_STORE, false>(p, taddr0, rs_s, ts, tok_first, n, lane, slot_row);
  else if (p.epi == EPI_SWIGLU) epilogue_tile<BN, J, EPI_SWIGLU, true>(p, taddr0, rs_s, ts, tok_first, n, lane, slot_row);
  else if (p.epi == EPI_RESIDUAL) epilogue_tile<BN, J, EPI_RESIDUAL, true>(p, taddr0, rs_s, ts, tok_first, n, lane, slot_row);
  else if (p.epi == EPI_STORE_F32) epilogue_tile<BN, J, EPI_STORE_F32, true>(p, taddr0, rs_s, ts, tok_first, n, lane, slot_row);
  else epilogue_tile<BN, J, EPI_STORE, true>(p, taddr0, rs_s, ts, tok_first, n, lane, slot_row);
}

template <int BN>
struct Cfg {
  static constexpr int SFB_ATOMS = BN > 128 ? 2 : 1;
  static constexpr int A_BYTES = TILE_N * KT_BYTES;
  static constexpr int B_BYTES = BN * KT_BYTES;
  static constexpr int B_ALLOC = (B_BYTES + 1023) / 1024 * 1024;
  static constexpr int SFA_BYTES = 4 * SF_ATOM;
  static constexpr int SFB_BYTES = SFB_ATOMS * 4 * SF_ATOM;
  // Two rings: the weight tile + its scales (A stage) and the activation tile + its scales
  // (B stage).  The weight stream needs many loads in flight (load latency ~2 us), so it gets
  // most of the shared memory; the stage counts are launch parameters.
  static constexpr int A_STAGE = A_BYTES + SFA_BYTES;
  static constexpr int B_STAGE = B_ALLOC + SFB_BYTES;
  static constexpr int MAX_STAGES = 8;
  static constexpr int RING_BYTES = 216 * 1024;
  static constexpr int BAR_BYTES = 512;
  static constexpr int TMEM_COLS = BN <= 64 ? 256 : 512;
  static constexpr int SF_COL0 = BN <= 64 ? 128 : 256;
  static constexpr int smem_bytes(int sa, int sb) {
    return sa * A_STAGE + sb * B_STAGE + 1024 /*align*/ + BAR_BYTES + 1024 /*column scales*/;
  }
};

// Phase timestamps of one launch (builds with -DTRL_TRACE only): [CTA][slot] = globaltimer in ns.
//   0 entry, 1 set-up done, 2 producer past the dependency wait, 3 first operands landed,
//   4 last MMA issued, 5 first accumulator complete, 6 last TMEM read-out done,
//   7 split-tile finishing done, 8 teardown, 9 segment counted, 10 reduction starts,
//   11 first reduction batch stored.
constexpr int TRACE_SLOTS = 16, TRACE_CTAS = 256;
__device__ unsigned long long g_gemm_trace[TRACE_CTAS * TRACE_SLOTS];
__device__ __forceinline__ void trace_stamp(int slot) {
#ifdef TRL_TRACE
  if (blockIdx.x < TRACE_CTAS) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    g_gemm_trace[blockIdx.x * TRACE_SLOTS + slot] = t;
  }
#else
  (void)slot;
#endif
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                  const GemmParams p) {
  using C = Cfg<BN>;
  constexpr int MS = C::MAX_STAGES;
  const int SA = p.sa, SB = p.sb;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* smem_b = smem + (size_t)SA * C::A_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_b + (size_t)SB * C::B_STAGE);
  // bars: [0,MS) full_a, [MS,2MS) empty_a, [2MS,3MS) full_b, [3MS,4MS) empty_b, accum_full, accum_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * MS + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;
  float* rs_s = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + C::BAR_BYTES);  // [BN] column scales

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) trace_stamp(0);
  const uint32_t bar0 = smem_u32(bars);
  auto full_a = [&](int s) { return bar0 + 8u * s; };
  auto empty_a = [&](int s) { return bar0 + 8u * (MS + s); };
  auto full_b = [&](int s) { return bar0 + 8u * (2 * MS + s); };
  auto empty_b = [&](int s) { return bar0 + 8u * (3 * MS + s); };
  const uint32_t accum_full = bar0 + 8u * (4 * MS), accum_empty = bar0 + 8u * (4 * MS + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < MS; ++s) {
      mbar_init(full_a(s), 1), mbar_init(empty_a(s), 1);
      mbar_init(full_b(s), 1), mbar_init(empty_b(s), 1);
    }
    mbar_init(accum_full, 1);
    mbar_init(accum_empty, 128);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  if (threadIdx.x == 0) trace_stamp(1);

  const long long U = (long long)p.n_tiles * p.c_tiles * p.nk;
  const int G = gridDim.x;
  long long u0 = (long long)blockIdx.x * U / G, u1 = (long long)(blockIdx.x + 1) * U / G;
  if (!p.split) {
    const long long T = (long long)p.n_tiles * p.c_tiles;
    u0 = ((long long)blockIdx.x * T / G) * p.nk, u1 = ((long long)(blockIdx.x + 1) * T / G) * p.nk;
  }
  const uint32_t a_tx = C::A_BYTES + C::SFA_BYTES, b_tx = C::B_BYTES + C::SFB_BYTES;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int n_units = (int)(u1 - u0);
      const uint32_t smem_a0 = smem_u32(smem), smem_b0 = smem_u32(smem_b);
      // two cursors over the same unit sequence: weights run up to SA units ahead of the MMA,
      // activations up to SB; running (tile, k-tile) coordinates, no division per unit
      struct Cur { int nt, ct, kt, st; uint32_t ph; };
      auto advance = [&](Cur& c, int ring) {
        if (++c.kt == p.nk) {
          c.kt = 0;
          if (++c.ct == p.c_tiles) c.ct = 0, ++c.nt;
        }
        if (++c.st == ring) c.st = 0, c.ph ^= 1u;
      };
      const int tile0 = (int)(u0 / p.nk);
      Cur ca{tile0 / p.c_tiles, tile0 % p.c_tiles, (int)(u0 % p.nk), 0, 0u};
      Cur cb = ca;
      auto load_a = [&](const Cur& c) {
        const uint32_t st = smem_a0 + (uint32_t)c.st * C::A_STAGE;
        mbar_expect_tx(full_a(c.st), a_tx);
        tma_load_2d(st, &map_w, p.w_tiled ? 0 : c.kt * KT_BYTES,
                    p.w_tiled ? (c.nt * p.nk + c.kt) * TILE_N : c.nt * TILE_N, full_a(c.st));
        bulk_load(st + C::A_BYTES, p.sfw + ((size_t)(c.nt * p.kt4 + c.kt * 4)) * SF_ATOM, C::SFA_BYTES, full_a(c.st));
      };
      auto load_b = [&](const Cur& c) {
        const uint32_t st = smem_b0 + (uint32_t)c.st * C::B_STAGE;
        mbar_expect_tx(full_b(c.st), b_tx);
        tma_load_2d(st, &map_x, c.kt * KT_BYTES, c.ct * BN, full_b(c.st));
#pragma unroll
        for (int j = 0; j < C::SFB_ATOMS; ++j) {
          const int atom_row = (c.ct * BN) / 128 + j;
          bulk_load(st + C::B_ALLOC + j * 4 * SF_ATOM, p.sfx + ((size_t)(atom_row * p.kt4 + c.kt * 4)) * SF_ATOM,
                    4 * SF_ATOM, full_b(c.st));
        }
      };
      // prologue: the first SA weight tiles do not depend on the previous kernel
      int a_issued = 0, b_issued = 0;
      const bool lockstep = SA == SB;   // equal rings: one barrier pair per stage serves both operands
      if (lockstep) {
        // both operands of a stage complete on full_a; the stage is free again on empty_a
        auto load_ab_b = [&](const Cur& c) {   // activation half of stage c.st, onto full_a
          const uint32_t st = smem_b0 + (uint32_t)c.st * C::B_STAGE;
          tma_load_2d(st, &map_x, c.kt * KT_BYTES, c.ct * BN, full_a(c.st));
#pragma unroll
          for (int j = 0; j < C::SFB_ATOMS; ++j) {
            const int atom_row = (c.ct * BN) / 128 + j;
            bulk_load(st + C::B_ALLOC + j * 4 * SF_ATOM, p.sfx + ((size_t)(atom_row * p.kt4 + c.kt * 4)) * SF_ATOM,
                      4 * SF_ATOM, full_a(c.st));
          }
        };
        auto load_a_ls = [&](const Cur& c) {   // weight half, expecting the bytes of both halves
          const uint32_t st = smem_a0 + (uint32_t)c.st * C::A_STAGE;
          mbar_expect_tx(full_a(c.st), a_tx + b_tx);
          tma_load_2d(st, &map_w, p.w_tiled ? 0 : c.kt * KT_BYTES,
                      p.w_tiled ? (c.nt * p.nk + c.kt) * TILE_N : c.nt * TILE_N, full_a(c.st));
          bulk_load(st + C::A_BYTES, p.sfw + ((size_t)(c.nt * p.kt4 + c.kt * 4)) * SF_ATOM, C::SFA_BYTES, full_a(c.st));
        };
        const int pre = min(SA, n_units);
        for (; a_issued < pre; ++a_issued) load_a_ls(ca), advance(ca, SA);
        pdl_wait();
        trace_stamp(2);
        bool ok = true;
        for (; ok && b_issued < n_units; ++b_issued) {
          if (b_issued >= pre) {
            ok = mbar_wait(empty_a(cb.st), cb.ph ^ 1u, abort_flag);
            if (!ok) break;
            load_a_ls(ca), advance(ca, SA), ++a_issued;
          }
          load_ab_b(cb), advance(cb, SB);
        }
      } else {
      for (; a_issued < min(SA, n_units); ++a_issued) load_a(ca), advance(ca, SA);
      pdl_wait();
      bool ok = true;
      while (ok && b_issued < n_units) {
        if (b_issued >= SB) ok = mbar_wait(empty_b(cb.st), cb.ph ^ 1u, abort_flag);
        if (!ok) break;
        load_b(cb), advance(cb, SB), ++b_issued;
        // weight unit (b_issued - 1 + SA) may go once the MMA of unit (b_issued - 1) has retired
        if (a_issued < n_units && a_issued < b_issued + SA - 1) {
          ok = mbar_wait(empty_a(ca.st), ca.ph ^ 1u, abort_flag);
          if (!ok) break;
          load_a(ca), advance(ca, SA), ++a_issued;
        }
      }
      while (ok && a_issued < n_units) {   // not reached when SA <= n_units bookkeeping holds; kept for safety
        ok = mbar_wait(empty_a(ca.st), ca.ph ^ 1u, abort_flag);
        if (!ok) break;
        load_a(ca), advance(ca, SA), ++a_issued;
      }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    pdl_wait();
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);
      long long u = u0;
      int it = 0, seg = 0, sa_i = 0, sb_i = 0;
      uint32_t sa_ph = 0, sb_ph = 0;
      bool ok = true;
      // descriptor words of stage 0 / k-block 0; everything else is an affine offset
      const uint64_t d_a = desc_sw128(smem_u32(smem)), d_b = desc_sw128(smem_u32(smem_b));
      const uint64_t d_sfa = desc_sf(smem_u32(smem + C::A_BYTES)), d_sfb = desc_sf(smem_u32(smem_b + C::B_ALLOC));
      const uint32_t a_lo = (uint32_t)d_a, b_lo = (uint32_t)d_b, op_hi = (uint32_t)(d_a >> 32);
      const uint32_t sfa_lo = (uint32_t)d_sfa, sfb_lo = (uint32_t)d_sfb, sf_hi = (uint32_t)(d_sfa >> 32);
      while (ok && u < u1) {
        const int k0 = (int)(u % p.nk);
        const int len = (int)min((long long)(p.nk - k0), u1 - u);
        if (seg > 0) {
          ok = mbar_wait(accum_empty, (uint32_t)(seg - 1) & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
        }
        for (int i = 0; ok && i < len; ++i, ++it) {
          ok = mbar_wait(full_a(sa_i), sa_ph, abort_flag) && (SA == SB || mbar_wait(full_b(sb_i), sb_ph, abort_flag));
          if (!ok) break;
          tc_fence_after();
          if (it == 0) trace_stamp(3);
          const uint32_t aoff = (uint32_t)sa_i * (uint32_t)(C::A_STAGE >> 4);
          const uint32_t boff = (uint32_t)sb_i * (uint32_t)(C::B_STAGE >> 4);
          const uint32_t sf_cols = tmem_base + C::SF_COL0 + (uint32_t)(it & 1) * 64;  // double-buffered by parity
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            tc_cp_sf_lh(sf_cols + kb * 4, sfa_lo + aoff + kb * (SF_ATOM >> 4), sf_hi);
#pragma unroll
            for (int j = 0; j < C::SFB_ATOMS; ++j)
              tc_cp_sf_lh(sf_cols + 16 + kb * 8 + j * 4, sfb_lo + boff + (j * 4 + kb) * (SF_ATOM >> 4), sf_hi);
          }
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            tc_mma_nvfp4_lh(tmem_base, a_lo + aoff + kb * 2, b_lo + boff + kb * 2, op_hi, idesc, sf_cols + kb * 4,
                            sf_cols + 16 + kb * 8, (i | kb) ? 1u : 0u);
          tc_commit(empty_a(sa_i));
          if (SA != SB) tc_commit(empty_b(sb_i));
          if (++sa_i == SA) sa_i = 0, sa_ph ^= 1u;
          if (++sb_i == SB) sb_i = 0, sb_ph ^= 1u;
        }
        if (ok) tc_commit(accum_full);
        u += len;
        ++seg;
      }
      trace_stamp(4);
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    pdl_wait();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const float ts = *p.tscale;
    const int J = p.J;
    long long u = u0;
    int seg = 0;
    bool ok = true;
    while (ok && u < u1) {
      const int tile = (int)(u / p.nk);
      const int k0 = (int)(u % p.nk);
      const int len = (int)min((long long)(p.nk - k0), u1 - u);
      const bool whole = (k0 == 0 && len == p.nk);
      const int nt = tile / p.c_tiles, ct = tile % p.c_tiles;
      const int n = nt * TILE_N + row;
      const int tok0 = (ct * BN) / J;
      // split tiles: this CTA's private slot (deterministic, order-independent reduction)
      const long long t_lo = (long long)tile * p.nk;
      const int first_owner = whole ? 0 : owner_of(t_lo, U, G);
      float* tile_slots = p.partial + (size_t)tile * p.max_seg * (BN / J) * TILE_N;
      float* slot = tile_slots + (size_t)((int)blockIdx.x - first_owner) * (BN / J) * TILE_N;
      // per-column activation scales of this tile: staged once in shared memory (while the
      // mainloop still runs), so the value loop below has no global load between its stores
      asm volatile("bar.sync 1, 128;" ::: "memory");   // previous tile's readers are done
      for (int i = threadIdx.x - 64; i < BN; i += 128) {
        const int col = ct * BN + i;
        rs_s[i] = col < p.cols ? __ldcg(p.rs + col) : 0.f;   // written by the quantiser kernel just before: read through L2
      }
      ok = mbar_wait(accum_full, (uint32_t)seg & 1u, abort_flag);
      {
        // one decision for all four epilogue warps (they meet at named barriers below), which
        // also publishes the staged scales
        uint32_t all;
        asm volatile(
            "{ .reg .pred p, q;\n"
            "  setp.ne.u32 q, %1, 0;\n"
            "  bar.red.and.pred p, 1, 128, q;\n"
            "  selp.u32 %0, 1, 0, p; }\n"
            : "=r"(all) : "r"((uint32_t)ok) : "memory");
        ok = all != 0;
      }
      if (!ok) break;
      tc_fence_after();
      if (seg == 0 && threadIdx.x == 64) trace_stamp(5);
      // finishing one (token, row) value of a split tile (run-time epilogue kind)
      auto finish = [&](int tok, float v, float res) {
        if (p.epi == EPI_SWIGLU) epi_store<EPI_SWIGLU>(p, tok, n, lane, v, res);
        else if (p.epi == EPI_STORE_F32) epi_store<EPI_STORE_F32>(p, tok, n, lane, v, res);
        else epi_store<EPI_STORE>(p, tok, n, lane, v, res);
      };
      auto load_res = [&](int tok) -> float {
        return (p.epi == EPI_RESIDUAL && tok < p.tokens && n < p.N)
                   ? __bfloat162float(p.residual[(size_t)tok * p.ldr + n]) : 0.f;
      };
      {
        const uint32_t taddr0 = tmem_base + ((uint32_t)(quad * 32) << 16);
        if (J == 4) epilogue_dispatch<BN, 4>(p, whole, taddr0, rs_s, ts, tok0, n, lane, slot + row);
        else if (J == 2) epilogue_dispatch<BN, 2>(p, whole, taddr0, rs_s, ts, tok0, n, lane, slot + row);
        else epilogue_dispatch<BN, 1>(p, whole, taddr0, rs_s, ts, tok0, n, lane, slot + row);
      }
      tc_fence_before();
      mbar_arrive(accum_empty);
      if (threadIdx.x == 64) trace_stamp(6);
      if (!whole) {
        // split tile: the last CTA to arrive finishes it from the per-segment slots
        asm volatile("bar.sync 1, 128;" ::: "memory");   // all slot stores of this CTA issued
        const int nseg = owner_of(t_lo + p.nk - 1, U, G) - first_owner + 1;
        if (threadIdx.x == 64) {
          __threadfence();                                // publish them (cumulative over the barrier)
          const int prev = atomicAdd(p.counters + tile, 1);
          *last_flag = (prev == nseg - 1);
          if (prev == nseg - 1) p.counters[tile] = 0;
          trace_stamp(9);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag) {
          __threadfence();
          if (threadIdx.x == 64) trace_stamp(10);
          const int ntok = BN / J;
          const bool vec_ok = (p.N & 3) == 0 && (p.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 &&
                              (p.epi != EPI_RESIDUAL ||
                               ((p.ldr & 3) == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 7) == 0));
          if (vec_ok) {
            // a thread owns 4 consecutive rows of 4 tokens per pass: 128-bit slot loads, one 64-bit
            // (bf16) or 128-bit (fp32) store per token, a quarter of the memory instructions of the
            // row-per-thread mapping; segments are summed in ascending order (bitwise reproducible)
            constexpr int TQ = 4, SGB = 4;
            const int e = (int)threadIdx.x - 64;
            const int rg = e & 31, tsub = e >> 5;
            const int n4 = nt * TILE_N + rg * 4;
            for (int g0 = 0; g0 < ntok; g0 += 4 * TQ) {
              float4 acc[TQ];
              uint2 res[TQ];
#pragma unroll
              for (int q = 0; q < TQ; ++q) {
                const int g = g0 + q * 4 + tsub, tok = tok0 + g;
                acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                res[q] = make_uint2(0u, 0u);
                if (p.epi == EPI_RESIDUAL && g < ntok && tok < p.tokens && n4 < p.N)
                  res[q] = *reinterpret_cast<const uint2*>(p.residual + (size_t)tok * p.ldr + n4);
              }
              for (int sg0 = 0; sg0 < nseg; sg0 += SGB) {
                float4 part[TQ][SGB];
#pragma unroll
                for (int q = 0; q < TQ; ++q)
#pragma unroll
                  for (int sj = 0; sj < SGB; ++sj) {
                    const int g = g0 + q * 4 + tsub;
                    part[q][sj] = (sg0 + sj < nseg && g < ntok)
                                      ? __ldcg(reinterpret_cast<const float4*>(
                                            tile_slots + ((size_t)(sg0 + sj) * ntok + g) * TILE_N + rg * 4))
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
                  }
#pragma unroll
                for (int q = 0; q < TQ; ++q)
#pragma unroll
                  for (int sj = 0; sj < SGB; ++sj) {
                    acc[q].x += part[q][sj].x, acc[q].y += part[q][sj].y;
                    acc[q].z += part[q][sj].z, acc[q].w += part[q][sj].w;
                  }
              }
#pragma unroll
              for (int q = 0; q < TQ; ++q) {
                const int g = g0 + q * 4 + tsub, tok = tok0 + g;
                if (g >= ntok || tok >= p.tokens || n4 >= p.N) continue;
                float4 a = acc[q];
                if (p.epi == EPI_SWIGLU) {
                  const float y0 = __fdividef(a.x, 1.f + __expf(-a.x)) * a.y;
                  const float y1 = __fdividef(a.z, 1.f + __expf(-a.z)) * a.w;
                  *reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(p.out) + (size_t)tok * p.ldo + (n4 >> 1)) =
                      f2_to_bf162_bits(y0, y1);
                } else if (p.epi == EPI_STORE_F32) {
                  *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)tok * p.ldo + n4) = a;
                } else {
                  const float2 r0 = bf162_bits_to_f2(res[q].x), r1 = bf162_bits_to_f2(res[q].y);
                  a.x += r0.x, a.y += r0.y, a.z += r1.x, a.w += r1.y;
                  *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p.out) + (size_t)tok * p.ldo + n4) =
                      make_uint2(f2_to_bf162_bits(a.x, a.y), f2_to_bf162_bits(a.z, a.w));
                }
              }
              if (g0 == 0 && threadIdx.x == 64) trace_stamp(11);
            }
          } else {
          // row-per-thread fallback for outputs that do not allow vector stores
          constexpr int GB = 16, SGB = 4;
          for (int g0 = 0; g0 < ntok; g0 += GB) {
            float acc[GB], res[GB];
#pragma unroll
            for (int gi = 0; gi < GB; ++gi) {
              acc[gi] = 0.f;
              res[gi] = g0 + gi < ntok ? load_res(tok0 + g0 + gi) : 0.f;
            }
            for (int sg0 = 0; sg0 < nseg; sg0 += SGB) {
              float part[GB][SGB];
#pragma unroll
              for (int gi = 0; gi < GB; ++gi)
#pragma unroll
                for (int sj = 0; sj < SGB; ++sj)
                  part[gi][sj] = (sg0 + sj < nseg && g0 + gi < ntok)
                                     ? __ldcg(tile_slots + ((size_t)(sg0 + sj) * ntok + g0 + gi) * TILE_N + row) : 0.f;
#pragma unroll
              for (int gi = 0; gi < GB; ++gi)
#pragma unroll
                for (int sj = 0; sj < SGB; ++sj) acc[gi] += part[gi][sj];   // ascending segment order: bitwise reproducible
            }
#pragma unroll
            for (int gi = 0; gi < GB; ++gi)
              if (g0 + gi < ntok) finish(tok0 + g0 + gi, acc[gi], res[gi]);
          }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (threadIdx.x == 64) trace_stamp(7);
      u += len;
      ++seg;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    // give copies that are still in flight time to land before the CTA's memory goes away
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0) trace_stamp(8);
}

// ---------------------------------------------------------------------------------------
// Activation quantiser: optional RMSNorm (or SwiGLU of an interleaved gate/up row), then
// J NVFP4 residual terms per token.  column (tok*J + j): xq [cols, K/2], sf tiled (see
// header), rs[col] fp32.
//
// Grid = (tokens, slices): every CTA first reduces the whole (L2-resident) row for the
// norm statistics and the row maximum, then each thread owns one 16-element block and
// runs all J terms in registers.  The row scale of term j is rs_0 / 4^j -- a bound, not a
// reduction: one e2m1 term leaves a remainder of at most 1/4 of the block maximum it
// encoded (worst gap 4..6 of 6 plus the e4m3 scale rounding) -- so no second pass over
// the row is needed.
__global__ void __launch_bounds__(256)
quant_act_kernel(const bf16* x, int ldx, const float* __restrict__ norm_w, float eps,
                 uint8_t* xq, uint8_t* sf, float* rs, int K, int J,
                 int kt4, int swiglu_in) {
  __shared__ float red[32];
  // one CTA per row (gridDim.y == 1): the pass that finds the row maximum leaves the (normalised) row in
  // shared memory as bf16, and the quantising pass reads it from there -- read from L2 again, that pass
  // is a chain of dependent loads, one per 1024 elements of the row
  extern __shared__ __align__(16) uint2 qa_row[];
  const bool staged = gridDim.y == 1;
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x;
  const bf16* xr = x + (size_t)tok * ldx;
  // four consecutive elements starting at k (k % 4 == 0)
  auto load4 = [&](int k, float (&v)[4]) {
    if (swiglu_in) {  // interleaved (gate, up) pairs: K outputs from 2K inputs
      const uint4 u = *reinterpret_cast<const uint4*>(xr + 2 * k);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 gu = bf162_bits_to_f2(w[i]);
        v[i] = __bfloat162float(__float2bfloat16(silu_f(gu.x) * gu.y));
      }
    } else {
      const uint2 u = *reinterpret_cast<const uint2*>(xr + k);
      const float2 a = bf162_bits_to_f2(u.x), b = bf162_bits_to_f2(u.y);
      v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
    }
  };
  float rstd = 1.f;
  if (norm_w != nullptr) {
    float ss = 0.f;
#pragma unroll 4
    for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
      float v[4];
      load4(k, v);
      ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    }
    ss = block_sum(ss, red);
    rstd = rsqrtf(ss / (float)K + eps);
  }
  float amax = 0.f;
#pragma unroll 4
  for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
    float v[4];
    load4(k, v);
    if (norm_w != nullptr) {
      const float4 w = *reinterpret_cast<const float4*>(norm_w + k);
      v[0] = __bfloat162float(__float2bfloat16(v[0] * rstd * w.x));
      v[1] = __bfloat162float(__float2bfloat16(v[1] * rstd * w.y));
      v[2] = __bfloat162float(__float2bfloat16(v[2] * rstd * w.z));
      v[3] = __bfloat162float(__float2bfloat16(v[3] * rstd * w.w));
    }
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
    if (staged) qa_row[k >> 2] = make_uint2(f2_to_bf162_bits(v[0], v[1]), f2_to_bf162_bits(v[2], v[3]));   // exact: v is bf16-valued
  }
  amax = block_max(amax, red);
  const float rs0 = fmaxf(amax, 1e-30f) * (1.f / (6.f * 448.f));
  if (blockIdx.y == 0 && threadIdx.x < J) rs[tok * J + threadIdx.x] = rs0 * exp2f(-2.f * (float)threadIdx.x);
  if (staged) {
    // one CTA per row: a thread takes whole 16-element blocks out of the staged row (the scale arithmetic
    // is paid once per block, no shuffles; 8 bytes of e2m1 per term and block in one store).  Same
    // arithmetic per element as the quarter-block form below, so the same bits.
    const int n_blk = kt4 * 4;                            // 16-element blocks of the padded row
    for (int b = threadIdx.x; b < n_blk; b += blockDim.x) {
      const int k = b * 16;                               // K % 16 == 0: a block is whole or padding
      float r[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) r[i] = 0.f;
      if (k < K) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint2 u = qa_row[b * 4 + i];
          const float2 a = bf162_bits_to_f2(u.x), b2 = bf162_bits_to_f2(u.y);
          r[4 * i] = a.x, r[4 * i + 1] = a.y, r[4 * i + 2] = b2.x, r[4 * i + 3] = b2.y;
        }
      }
      float rscale = rs0;
      for (int j = 0; j < J; ++j, rscale *= 0.25f) {
        const int col = tok * J + j;
        float bm = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) bm = fmaxf(bm, fabsf(r[i]));
        const float s = fminf(__fdividef(bm, 6.f * rscale), 448.f);
        uint16_t s16;
        asm("{ .reg .b16 t; cvt.rn.satfinite.e4m3x2.f32 t, %1, %2; mov.b16 %0, t; }" : "=h"(s16) : "f"(0.f), "f"(s));
        const float sfv = h2_to_f2(cvt_e4m3x2_to_h2(s16)).x;
        const float denom = sfv * rscale;
        const float inv = denom > 0.f ? __frcp_rn(denom) : 0.f;
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; ++i) {                     // byte i: elements 2i (low nibble), 2i + 1
          uint16_t by;
          asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(by) : "f"(r[2 * i + 1] * inv), "f"(r[2 * i] * inv));
          packed[i >> 2] |= (uint32_t)(by & 0xff) << (8 * (i & 3));
          if (j + 1 < J) {                                // the next term encodes the remainder
            uint32_t h;
            asm("{ .reg .b8 t; cvt.u8.u16 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h) : "h"(by));
            const float2 d = h2_to_f2(h);
            r[2 * i] = fmaf(-d.x, denom, r[2 * i]);
            r[2 * i + 1] = fmaf(-d.y, denom, r[2 * i + 1]);
          }
        }
        if (k < K) *reinterpret_cast<uint2*>(xq + (size_t)col * (K >> 1) + (size_t)b * 8) = make_uint2(packed[0], packed[1]);
        sf[((size_t)(col >> 7) * kt4 + (b >> 2)) * SF_ATOM + (col & 31) * 16 + ((col & 127) >> 5) * 4 + (b & 3)] =
            (k < K) ? (uint8_t)(s16 & 0xff) : (uint8_t)0;
      }
    }
    return;
  }
  // this thread's quarter blocks: one per slice; gridDim.y slices run in parallel, the rest in
  // a loop (one CTA per row when there are enough rows to fill the GPU: the row is then read
  // from L2 by one CTA instead of by every slice's CTA)
  const int n_slices = (kt4 * 16 + (int)blockDim.x - 1) / (int)blockDim.x;
  for (int sl = blockIdx.y; sl < n_slices; sl += gridDim.y) {
  const int q4 = sl * blockDim.x + threadIdx.x;          // index of the 4-element group
  const int k = q4 * 4;
  const int b = q4 >> 2;                                  // 16-element block
  const bool valid = b < kt4 * 4;                         // whole 4-lane groups are valid or not
  float r[4] = {0.f, 0.f, 0.f, 0.f};
  if (k < K) {
    load4(k, r);
    if (norm_w != nullptr) {
      const float4 w = *reinterpret_cast<const float4*>(norm_w + k);
      r[0] = __bfloat162float(__float2bfloat16(r[0] * rstd * w.x));
      r[1] = __bfloat162float(__float2bfloat16(r[1] * rstd * w.y));
      r[2] = __bfloat162float(__float2bfloat16(r[2] * rstd * w.z));
      r[3] = __bfloat162float(__float2bfloat16(r[3] * rstd * w.w));
    }
  }
  float rscale = rs0;
  for (int j = 0; j < J; ++j, rscale *= 0.25f) {
    const int col = tok * J + j;
    float bm = fmaxf(fmaxf(fabsf(r[0]), fabsf(r[1])), fmaxf(fabsf(r[2]), fabsf(r[3])));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
    const float s = fminf(__fdividef(bm, 6.f * rscale), 448.f);
    uint16_t s16;
    asm("{ .reg .b16 t; cvt.rn.satfinite.e4m3x2.f32 t, %1, %2; mov.b16 %0, t; }" : "=h"(s16) : "f"(0.f), "f"(s));
    const float sfv = h2_to_f2(cvt_e4m3x2_to_h2(s16)).x;
    const float denom = sfv * rscale;
    const float inv = denom > 0.f ? __frcp_rn(denom) : 0.f;
    uint16_t lo, hi;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(lo) : "f"(r[1] * inv), "f"(r[0] * inv));
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(hi) : "f"(r[3] * inv), "f"(r[2] * inv));
    uint32_t h0, h1;
    asm("{ .reg .b8 t; cvt.u8.u16 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h0) : "h"(lo));
    asm("{ .reg .b8 t; cvt.u8.u16 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h1) : "h"(hi));
    const float2 d0 = h2_to_f2(h0), d1 = h2_to_f2(h1);
    r[0] = fmaf(-d0.x, denom, r[0]);   // the next term encodes the remainder
    r[1] = fmaf(-d0.y, denom, r[1]);
    r[2] = fmaf(-d1.x, denom, r[2]);
    r[3] = fmaf(-d1.y, denom, r[3]);
    if (k < K)
      reinterpret_cast<uint16_t*>(xq + (size_t)col * (K >> 1))[q4] = (uint16_t)((lo & 0xff) | ((hi & 0xff) << 8));
    if (valid && (threadIdx.x & 3) == 0)  // scale byte (zero for the K padding)
      sf[((size_t)(col >> 7) * kt4 + (b >> 2)) * SF_ATOM + (col & 31) * 16 + ((col & 127) >> 5) * 4 + (b & 3)] =
          (k < K) ? (uint8_t)(s16 & 0xff) : (uint8_t)0;
  }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return 1;
    g_encode = (EncodeTiledFn)fn;
  }
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)KT_BYTES, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

template <int BN>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, GemmParams p, int grid, cudaStream_t st) {
  using C = Cfg<BN>;
  auto kern = gemm_nvfp4_kernel<BN>;
  // default: equal rings (one barrier pair per stage); unequal rings are an experiment knob --
  // measured on the 27B shapes they did not pay for their second wait / commit per unit
  int sa = C::RING_BYTES / (C::A_STAGE + C::B_STAGE);
  sa = sa > C::MAX_STAGES ? C::MAX_STAGES : sa;
  int sb = sa;
  if (const char* e = getenv("TRL_GEMM_SA")) sa = atoi(e);
  if (const char* e = getenv("TRL_GEMM_SB")) sb = atoi(e);
  if (sa < 1 || sb < 1 || sa > C::MAX_STAGES || sb > C::MAX_STAGES || C::smem_bytes(sa, sb) > 227 * 1024)
    return (int)cudaErrorInvalidValue;
  p.sa = sa, p.sb = sb;
  static int configured = 0;
  const int smem = C::smem_bytes(sa, sb);
  if (configured < smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return 3;
    configured = smem;
  }
  return (int)trl_launch(kern, dim3(grid), dim3(GEMM_THREADS), (size_t)smem, st, mw, mx, p);
}

}  // namespace

// Quantise activations for the GEMM.  xq: [tokens*J, K/2]; sf: tiled, (ceil(tokens*J/256)*2) atoms
// of rows x kt4 atoms of K; rs: [tokens*J].  K % 16 == 0.
TRL_API int trl_quant_act_nvfp4(const void* x, int ldx, const void* norm_w, float eps, void* xq, void* sf,
                                void* rs, int tokens, int K, int J, int swiglu_in, void* stream) {
  if (K % 16 != 0 || J < 1 || J > 16) return (int)cudaErrorInvalidValue;
  const int nk = (K + KT_ELEMS - 1) / KT_ELEMS;
  int slices = (nk * KT_ELEMS / 4 + 255) / 256;  // 4 elements per thread
  if (tokens >= 128) slices = 1;                        // enough rows to fill the GPU: one CTA per row
  const size_t smem = slices == 1 ? (size_t)((K + 3) / 4) * sizeof(uint2) : 0;      // the staged row, bf16
  if (smem > 48 * 1024) {
    static size_t configured = 0;
    if (configured < smem) {
      if (cudaFuncSetAttribute(quant_act_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 3;
      configured = smem;
    }
  }
  return (int)trl_launch(quant_act_kernel, dim3(tokens, slices), dim3(256), smem, (cudaStream_t)stream, (const bf16*)x,
                         ldx, (const float*)norm_w, eps, (uint8_t*)xq, (uint8_t*)sf, (float*)rs, K, J, nk * 4,
                         swiglu_in);
}

// Largest number of CTAs that share one output tile under the even stream-K split.
static int max_segments(long long U, int G, int nk) {
  // a tile spans nk consecutive units; CTA ranges are ~U/G long
  const long long per = U / G;
  if (per >= nk && U % G == 0 && per % nk == 0) return 1;
  return (int)min((long long)G, (long long)nk / (per > 0 ? per : 1) + 2);
}

static int pick_bn(int cols) {
  int bn = 16;
  while (bn < cols && bn < 256) bn <<= 1;
  return bn;
}

// Bytes of split-K scratch trl_gemm_nvfp4 needs for this problem (0 if no tile is split).
// Copies the phase timestamps of the last launch of a -DTRL_TRACE build: n_ctas x 16 values (zeros otherwise).
TRL_API int trl_gemm_trace_read(void* out, int n_ctas) {
  if (n_ctas < 0 || n_ctas > TRACE_CTAS) return (int)cudaErrorInvalidValue;
  return (int)cudaMemcpyFromSymbol(out, g_gemm_trace, (size_t)n_ctas * TRACE_SLOTS * sizeof(unsigned long long));
}

TRL_API long trl_gemm_nvfp4_scratch_bytes(int tokens, int J, int N, int K, int max_ctas) {
  const int cols = tokens * J, BN = pick_bn(cols);
  const int n_tiles = (N + TILE_N - 1) / TILE_N, c_tiles = (cols + BN - 1) / BN, nk = (K + KT_ELEMS - 1) / KT_ELEMS;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (max_ctas > 0) sms = min(sms, max_ctas);
  const long long U = (long long)n_tiles * c_tiles * nk;
  const int grid = (int)min((long long)sms, U);
  return (long)n_tiles * c_tiles * max_segments(U, grid, nk) * (BN / J) * TILE_N * (long)sizeof(float);
}

// out[tok, n] = epi(...).  wq [N, K/2] packed e2m1; sfw / sfx tiled scales; partial: fp32
// split-K slots of at least trl_gemm_nvfp4_scratch_bytes() bytes (contents irrelevant);
// counters: int32 [n_tiles * c_tiles], zero on entry and zero again on exit.
TRL_API int trl_gemm_nvfp4(const void* wq, const void* sfw, const void* tscale, const void* xq, const void* sfx,
                           const void* rs, const void* residual, int ldr, void* out, int ldo, void* partial,
                           void* counters, long partial_bytes, int tokens, int J, int N, int K, int epi, int max_ctas,
                           int split, int w_tiled, void* stream) {
  if (K % 32 != 0 || J < 1 || (32 % J) != 0 || J > 16) return (int)cudaErrorInvalidValue;
  const int cols = tokens * J;
  const int BN = pick_bn(cols);
  CUtensorMap mw, mx;
  {
    const uint64_t nt = (N + TILE_N - 1) / TILE_N, nkk = (K + KT_ELEMS - 1) / KT_ELEMS;
    const int rc = w_tiled ? make_map(&mw, wq, nt * nkk * TILE_N, KT_BYTES, TILE_N)
                           : make_map(&mw, wq, (uint64_t)N, (uint64_t)K / 2, TILE_N);
    if (rc) return (int)cudaErrorInvalidValue;
  }
  if (make_map(&mx, xq, (uint64_t)cols, (uint64_t)K / 2, (uint32_t)BN)) return (int)cudaErrorInvalidValue;
  GemmParams p;
  p.sfw = (const uint8_t*)sfw, p.sfx = (const uint8_t*)sfx, p.tscale = (const float*)tscale, p.rs = (const float*)rs;
  p.residual = (const bf16*)residual, p.out = out, p.partial = (float*)partial, p.counters = (int*)counters;
  p.N = N, p.K = K, p.cols = cols, p.tokens = tokens, p.J = J, p.ldr = ldr, p.ldo = ldo;
  p.n_tiles = (N + TILE_N - 1) / TILE_N;
  p.c_tiles = (cols + BN - 1) / BN;
  p.nk = (K + KT_ELEMS - 1) / KT_ELEMS;
  p.kt4 = p.nk * 4;
  p.epi = epi;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (max_ctas > 0) sms = min(sms, max_ctas);
  const long long U = (long long)p.n_tiles * p.c_tiles * p.nk;
  p.split = split;
  p.w_tiled = w_tiled;
  const int grid = split ? (int)min((long long)sms, U) : min(sms, p.n_tiles * p.c_tiles);
  p.max_seg = split ? max_segments(U, grid, p.nk) : 1;
  if (split && (size_t)p.n_tiles * p.c_tiles * p.max_seg * (BN / J) * TILE_N * sizeof(float) > (size_t)partial_bytes)
    return (int)cudaErrorMemoryAllocation;
  cudaStream_t st = (cudaStream_t)stream;
  switch (BN) {
    case 16: return launch<16>(mw, mx, p, grid, st);
    case 32: return launch<32>(mw, mx, p, grid, st);
    case 64: return launch<64>(mw, mx, p, grid, st);
    case 128: return launch<128>(mw, mx, p, grid, st);
    default: return launch<256>(mw, mx, p, grid, st);
  }
}
