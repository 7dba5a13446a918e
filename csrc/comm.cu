// Tensor-parallel collectives as kernels over NVLink peer memory (no library collective).
//
// Every rank owns one symmetric workspace (cudaMalloc, exported with CUDA IPC); each rank
// holds a table of all peers' workspace pointers.  Layout of a workspace:
//
//   ctrl   [0, 4 KiB)      u32 words: [0] one-shot epoch, [16] CTA-done counter,
//                          [32] two-shot epoch, [48] argmax epoch
//   flags  [4 KiB, 8 KiB)  u32: oneshot[2 bufs][8 src] @0, ready[8] @64, done[8] @96, amax[8] @128
//   amax   [8 KiB, 64 KiB) per source rank: (value, index) pairs for up to 256 rows
//   slots  [64 KiB, ...)   one-shot partials  {fp32, epoch} [2 bufs][8 src][8 rows][hmax]
//   big    [...]           two-shot operand   bf16 [tmax][hmax]
//
// * One-shot all-reduce (decode sizes): the row-parallel GEMV pushes its fp32 partial rows
//   straight into slot [buf][my_rank] of EVERY peer from its epilogue as {value, epoch} pairs,
//   one 8-byte store each over NVLink (overlapping the weight stream; no fence, counter or
//   flag stage), and `allreduce_finish` on each rank polls the epoch half of the words it
//   needs, sums the partials in rank order (bitwise identical on every rank), adds the
//   residual and writes the residual stream.  Two buffers alternate by epoch parity; the epoch lives in device
//   memory and is advanced by the finish kernel, so the sequence is CUDA-graph replayable.
// * Two-shot all-reduce (prefill sizes): every rank reduces its 1/tp slice of the rows by
//   reading all peers' partials (reduce-scatter), adds the residual and writes the slice
//   into every peer's residual stream (all-gather), bracketed by ready / done flags.
// * Vocab-parallel argmax: each rank pushes its (max, index) per row to all peers; every
//   rank picks the same winner.
//
// All waits are bounded (~2 s): on expiry the kernel records an error word and returns.
// Only plain peer loads and stores are used (no in-switch reduction).
//
// The reference has no counterpart: its collectives are torch.distributed calls
// (packages/tilerl-kernels/src/tilerl_kernels/backend.py:165-364).
#include "common.cuh"

namespace {

constexpr int MAX_RANKS = 8;
constexpr int ONESHOT_ROWS = 8;
// limit of every device-side wait, in SM clock cycles (~2 s by default; settable for tests)
__device__ long long g_comm_wait_cycles = 4000000000LL;
constexpr size_t OFF_FLAGS = 4096, OFF_AMAX = 8192, OFF_SLOTS = 65536;

struct Peers {
  unsigned char* ws[MAX_RANKS];
  int rank, world, hmax;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until *p >= want (epochs only grow).  False on timeout.
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t want, int code_a, int code_b) {
  if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0;; ++it) {
    if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
    if ((it & 15) == 15 && clock64() - t0 > g_comm_wait_cycles) {
      trl_set_error(TRL_ERR_WAIT_TIMEOUT, code_a, code_b, (int)want);
      return false;
    }
  }
}

// One-shot slots hold {fp32 value, epoch} pairs (8 bytes, written by one store).
__device__ __forceinline__ uint2* oneshot_slot(unsigned char* ws, int buf, int src, int hmax) {
  return reinterpret_cast<uint2*>(ws + OFF_SLOTS) + ((size_t)(buf * MAX_RANKS + src) * ONESHOT_ROWS) * hmax;
}

// x[m, n] = residual[m, n] + sum_src partial[src][m][n]; advances the epoch.  Every thread
// polls the epoch half of exactly the words it sums (bounded), so the sum of an element starts
// as soon as its last partial has landed.
__global__ void __launch_bounds__(256)
allreduce_finish_kernel(const Peers P, const bf16* residual, int ldr, bf16* out,
                        int ldo, int M, int N) {
  // a kernel that spins on peers' stores lets the next kernel in only after its last poll: an early
  // dependent's CTAs would sit on SM slots while this grid (or a peer's) still waits for CTAs to run
  pdl_enter(10);
  pdl_wait();
  unsigned char* me = P.ws[P.rank];
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(me);
  const uint32_t epoch = ctrl[0] + 1;
  const int buf = epoch & 1;
  const int total = M * N;
  bool ok = true;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; ok && i < total; i += gridDim.x * blockDim.x) {
    const int m = i / N, n = i % N;
    float v = __bfloat162float(residual[(size_t)m * ldr + n]);
    for (int s = 0; ok && s < P.world; ++s) {
      const uint2* w = oneshot_slot(me, buf, s, P.hmax) + (size_t)m * P.hmax + n;
      uint2 x = ld_relaxed_sys_v2(w);
      if (x.y != epoch) {
        const long long t0 = clock64();
        for (uint32_t it = 0; x.y != epoch; ++it) {
          x = ld_relaxed_sys_v2(w);
          if ((it & 15) == 15 && clock64() - t0 > g_comm_wait_cycles) {
            trl_set_error(TRL_ERR_WAIT_TIMEOUT, 1, s, (int)epoch);
            ok = false;
            break;
          }
        }
      }
      v += __uint_as_float(x.x);
    }
    if (ok) out[(size_t)m * ldo + n] = __float2bfloat16(v);
  }
  // the last CTA to finish advances the epoch
  __syncthreads();
  pdl_trigger();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(ctrl + 17, 1u);
    if (prev == gridDim.x - 1) {
      ctrl[17] = 0;
      __threadfence();
      ctrl[0] = epoch;
    }
  }
}

// Two-shot all-reduce of `big` [T, N] bf16 partials + residual -> every rank's `out`.
__global__ void __launch_bounds__(512)
allreduce_twoshot_kernel(const Peers P, size_t off_big, size_t off_out, const bf16* residual,
                         int ldr, int ldo, int T, int N) {
  unsigned char* me = P.ws[P.rank];
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(me);
  const uint32_t epoch = ctrl[32] + 1;
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(me + OFF_FLAGS);
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  // phase 0: my partial is complete (stream order) -> tell every peer, wait for theirs
  if (blockIdx.x == 0 && threadIdx.x < P.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(P.ws[threadIdx.x] + OFF_FLAGS) + 64 + P.rank, epoch);
  }
  if (threadIdx.x < P.world) {
    if (!wait_flag(my_flags + 64 + threadIdx.x, epoch, 2, threadIdx.x)) ok_s = 0;
  }
  __syncthreads();
  if (ok_s) {
    // my slice of the rows
    const int per = (T + P.world - 1) / P.world;
    const int r0 = min(T, P.rank * per), r1 = min(T, r0 + per);
    const int nvec = N / 8;
    const long total = (long)(r1 - r0) * nvec;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
      const int r = r0 + (int)(i / nvec), c = (int)(i % nvec) * 8;
      float acc[8];
      {
        const uint4 v = *reinterpret_cast<const uint4*>(residual + (size_t)r * ldr + c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = bf162_bits_to_f2(w[k]);
          acc[2 * k] = f.x, acc[2 * k + 1] = f.y;
        }
      }
      for (int s = 0; s < P.world; ++s) {
        const bf16* src = reinterpret_cast<const bf16*>(P.ws[s] + off_big) + (size_t)r * N + c;
        const uint4 v = *reinterpret_cast<const uint4*>(src);   // plain peer load over NVLink
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = bf162_bits_to_f2(w[k]);
          acc[2 * k] += f.x, acc[2 * k + 1] += f.y;
        }
      }
      uint4 o;
      o.x = f2_to_bf162_bits(acc[0], acc[1]), o.y = f2_to_bf162_bits(acc[2], acc[3]);
      o.z = f2_to_bf162_bits(acc[4], acc[5]), o.w = f2_to_bf162_bits(acc[6], acc[7]);
      for (int d = 0; d < P.world; ++d)
        *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(P.ws[d] + off_out) + (size_t)r * ldo + c) = o;   // all-gather by peer stores
    }
  }
  // phase 1: everyone's slice has landed everywhere
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t prev = atomicAdd(ctrl + 33, 1u);
    last_s = (prev == gridDim.x - 1);
  }
  __syncthreads();
  if (last_s) {
    if (threadIdx.x < P.world)
      st_release_sys(reinterpret_cast<uint32_t*>(P.ws[threadIdx.x] + OFF_FLAGS) + 96 + P.rank, epoch);
    if (threadIdx.x < P.world) wait_flag(my_flags + 96 + threadIdx.x, epoch, 3, threadIdx.x);
    __syncthreads();
    if (threadIdx.x == 0) {
      ctrl[33] = 0;
      __threadfence();
      ctrl[32] = epoch;
    }
  }
}

// Vocab-parallel argmax: local (value, index) per row -> all peers -> same winner everywhere.
__global__ void __launch_bounds__(256)
argmax_tp_kernel(const Peers P, const float* pv, const int* pi, int chunks,
                 int v_local, int* out, int M) {
  pdl_enter();
  pdl_wait();
  unsigned char* me = P.ws[P.rank];
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(me);
  const uint32_t epoch = ctrl[48] + 1;
  const int row = threadIdx.x;
  if (row < M) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = 0; c < chunks; ++c) {
      const float v = pv[row * chunks + c];
      const int i = pi[row * chunks + c];
      if (v > best || (v == best && i < bi)) best = v, bi = i;
    }
    const int gi = bi == 0x7fffffff ? bi : bi + P.rank * v_local;   // no comparable value (all NaN): keep the sentinel
    for (int p = 0; p < P.world; ++p) {
      float2* slot = reinterpret_cast<float2*>(P.ws[p] + OFF_AMAX) + ((size_t)((epoch & 1) * MAX_RANKS + P.rank) * 256 + row);
      *slot = make_float2(best, __int_as_float(gi));
    }
  }
  __syncthreads();
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < P.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(P.ws[threadIdx.x] + OFF_FLAGS) + 128 + (epoch & 1) * MAX_RANKS + P.rank, epoch);
  }
  if (threadIdx.x < P.world) {
    if (!wait_flag(reinterpret_cast<const uint32_t*>(me + OFF_FLAGS) + 128 + (epoch & 1) * MAX_RANKS + threadIdx.x, epoch, 4, threadIdx.x))
      ok_s = 0;
  }
  __syncthreads();
  if (ok_s && row < M) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int s = 0; s < P.world; ++s) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(me + OFF_AMAX) + ((size_t)((epoch & 1) * MAX_RANKS + s) * 256 + row));
      const int i = __float_as_int(v.y);
      if (v.x > best || (v.x == best && i < bi)) best = v.x, bi = i;
    }
    out[row] = bi == 0x7fffffff ? 0 : bi;   // a row without any comparable logit yields token 0, never a wild index
  }
  __syncthreads();
  pdl_trigger();
  if (threadIdx.x == 0) ctrl[48] = epoch;
}

Peers make_peers(void* const* ws, int rank, int world, int hmax) {
  Peers P;
  for (int i = 0; i < MAX_RANKS; ++i) P.ws[i] = i < world ? (unsigned char*)ws[i] : nullptr;
  P.rank = rank, P.world = world, P.hmax = hmax;
  return P;
}

}  // namespace

TRL_API size_t trl_symm_out_offset(int hmax, int tmax) {
  return OFF_SLOTS + (size_t)2 * MAX_RANKS * ONESHOT_ROWS * hmax * sizeof(uint2) + (size_t)tmax * hmax * sizeof(bf16);
}
TRL_API size_t trl_symm_bytes(int hmax, int tmax) {
  return OFF_SLOTS + (size_t)2 * MAX_RANKS * ONESHOT_ROWS * hmax * sizeof(uint2) + (size_t)2 * tmax * hmax * sizeof(bf16);
}
TRL_API size_t trl_symm_big_offset(int hmax) {
  return OFF_SLOTS + (size_t)2 * MAX_RANKS * ONESHOT_ROWS * hmax * sizeof(uint2);
}
TRL_API int trl_symm_alloc(size_t bytes, void** out) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, bytes);
}
TRL_API int trl_symm_free(void* p) { return (int)cudaFree(p); }
TRL_API int trl_ipc_get(void* p, void* handle64) {
  return (int)cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), p);
}
TRL_API int trl_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
TRL_API int trl_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

TRL_API int trl_allreduce_finish(void* const* ws, int rank, int world, int hmax, const void* residual, int ldr,
                                 void* out, int ldo, int M, int N, void* stream) {
  if (M > ONESHOT_ROWS || N > hmax || world > MAX_RANKS) return (int)cudaErrorInvalidValue;
  const int grid = max(1, min(16, (M * N + 2047) / 2048));
  return (int)trl_launch(allreduce_finish_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                         make_peers(ws, rank, world, hmax), (const bf16*)residual, ldr, (bf16*)out, ldo, M, N);
}

// This rank's [T, N] bf16 partial must already be in its `big` region; the reduced rows
// (+ residual) are written into every rank's `out` region (the residual stream lives there).
TRL_API int trl_allreduce_twoshot(void* const* ws, int rank, int world, int hmax, int tmax, const void* residual,
                                  int ldr, int ldo, int T, int N, void* stream) {
  if (N % 8 != 0 || world > MAX_RANKS) return (int)cudaErrorInvalidValue;
  const long work = (long)((T + world - 1) / world) * (N / 8);
  const int grid = (int)max(1L, min(64L, (work + 511) / 512));
  allreduce_twoshot_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(
      make_peers(ws, rank, world, hmax), trl_symm_big_offset(hmax), trl_symm_out_offset(hmax, tmax),
      (const bf16*)residual, ldr, ldo, T, N);
  return (int)cudaGetLastError();
}

TRL_API int trl_argmax_tp(void* const* ws, int rank, int world, int hmax, const void* pv, const void* pi,
                          int chunks, int v_local, void* out, int M, void* stream) {
  if (M > 256) return (int)cudaErrorInvalidValue;
  return (int)trl_launch(argmax_tp_kernel, dim3(1), dim3(256), 0, (cudaStream_t)stream,
                         make_peers(ws, rank, world, hmax), (const float*)pv, (const int*)pi, chunks, v_local,
                         (int*)out, M);
}

// Limit of the bounded waits of the kernels in this file, in milliseconds at 2 GHz.
TRL_API int trl_comm_set_wait_ms(int ms) {
  const long long cycles = (long long)ms * 2000000LL;
  return (int)cudaMemcpyToSymbol(g_comm_wait_cycles, &cycles, sizeof(cycles));
}
