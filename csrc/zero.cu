// ZeRO-3 collectives as kernels over NVLink peer memory: parameter all-gather and gradient
// reduce-scatter with the 1/world scale and the cast to fp32 fused.
//
// Every rank owns one symmetric region (cudaMalloc + CUDA IPC, same mechanism as the tensor-
// parallel workspace):
//
//   ctrl   [0, 4 KiB)   u32: [0] epoch, [1] CTA-done counter; flags ready[8] @256, done[8] @288
//   data   [4 KiB, ..)  staging areas (byte offsets are call arguments): the rank's parameter
//                       shard in the working dtype (all-gather) and its full flat gradient of the
//                       current unit (reduce-scatter)
//
// * all-gather: after a ready handshake every rank copies each peer's shard out of that peer's
//   staging area into its own full buffer with 16-byte peer loads.
// * reduce-scatter: after the handshake rank r reads slice r of every peer's gradient, adds the
//   slices in rank order in fp32 (the same order on every rank: reproducible), multiplies by
//   `scale` and writes or accumulates its fp32 gradient shard.
// Both end with a done handshake so the staging area may be overwritten by the next call.
// Every wait is bounded (~2 s): on expiry the kernel records an error word and returns.
// Only plain peer loads are used (no in-switch reduction, no bulk-tensor copies).
//
// The reference has no counterpart (no ZeRO/FSDP; gradients are all-reduced per tensor through
// torch.distributed: packages/tilerl-kernels/src/tilerl_kernels/backend.py:216-247).
#include "common.cuh"

namespace {

constexpr int Z_MAX_RANKS = 8;
constexpr long long Z_WAIT_CYCLES = 4000000000LL;
constexpr size_t Z_OFF_DATA = 4096;

struct ZPeers {
  unsigned char* ws[Z_MAX_RANKS];
  int rank, world;
};

__device__ __forceinline__ uint32_t z_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void z_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool z_wait(const uint32_t* p, uint32_t want, int a, int b) {
  if ((int32_t)(z_ld_acquire(p) - want) >= 0) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0;; ++it) {
    if ((int32_t)(z_ld_acquire(p) - want) >= 0) return true;
    if ((it & 15) == 15 && clock64() - t0 > Z_WAIT_CYCLES) {
      trl_set_error(TRL_ERR_WAIT_TIMEOUT, a, b, (int)want);
      return false;
    }
  }
}

// Phase 0: my staging area is complete (stream order) -> tell every peer; wait for theirs.
__device__ __forceinline__ bool z_ready(const ZPeers& P, uint32_t epoch, int* ok_s) {
  unsigned char* me = P.ws[P.rank];
  if (threadIdx.x == 0) *ok_s = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < P.world) {
    __threadfence_system();
    z_st_release(reinterpret_cast<uint32_t*>(P.ws[threadIdx.x]) + 256 + P.rank, epoch);
  }
  if (threadIdx.x < P.world) {
    if (!z_wait(reinterpret_cast<const uint32_t*>(me) + 256 + threadIdx.x, epoch, 10, threadIdx.x)) *ok_s = 0;
  }
  __syncthreads();
  return *ok_s != 0;
}

// Phase 1: the last CTA tells every peer that this rank no longer reads their staging areas,
// waits for the same from them and advances the epoch.
__device__ __forceinline__ void z_done(const ZPeers& P, uint32_t epoch, int* last_s) {
  unsigned char* me = P.ws[P.rank];
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(me);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t prev = atomicAdd(ctrl + 1, 1u);
    *last_s = (prev == gridDim.x - 1);
  }
  __syncthreads();
  if (*last_s) {
    if (threadIdx.x < P.world) z_st_release(reinterpret_cast<uint32_t*>(P.ws[threadIdx.x]) + 288 + P.rank, epoch);
    if (threadIdx.x < P.world) z_wait(reinterpret_cast<const uint32_t*>(me) + 288 + threadIdx.x, epoch, 11, threadIdx.x);
    __syncthreads();
    if (threadIdx.x == 0) {
      ctrl[1] = 0;
      __threadfence();
      ctrl[0] = epoch;
    }
  }
}

// Four independent 16-byte peer loads per thread and pass: NVLink latency is ~2 us, so the
// bytes in flight, not the instruction count, set the rate.
__global__ void __launch_bounds__(512)
zero_allgather_kernel(const ZPeers P, size_t off, long shard_vecs, uint4* dst) {
  __shared__ int ok_s, last_s;
  const uint32_t epoch = reinterpret_cast<const uint32_t*>(P.ws[P.rank])[0] + 1;
  if (z_ready(P, epoch, &ok_s)) {
    const long stride = (long)gridDim.x * blockDim.x;
    for (int k = 0; k < P.world; ++k) {
      // source order rotated by rank and by CTA: at any moment a rank reads every peer at once and no
      // source serves all readers at once (in rank order every rank queued on the same source: 224 GB/s
      // received at 8 GPUs where the reduce-scatter, which reads all peers per element, reached 498)
      const int p = (P.rank + k + (int)blockIdx.x) % P.world;
      const uint4* src = reinterpret_cast<const uint4*>(P.ws[p] + off);
      uint4* d = dst + (long)p * shard_vecs;
      long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
      for (; i + 3 * stride < shard_vecs; i += 4 * stride) {
        const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], e = src[i + 3 * stride];
        d[i] = a, d[i + stride] = b, d[i + 2 * stride] = c, d[i + 3 * stride] = e;
      }
      for (; i < shard_vecs; i += stride) d[i] = src[i];
    }
  }
  z_done(P, epoch, &last_s);
}

template <bool BF16>
__global__ void __launch_bounds__(512)
zero_reduce_scatter_kernel(const ZPeers P, size_t off, long shard_elems, float scale, float* out,
                           int accumulate) {
  __shared__ int ok_s, last_s;
  const uint32_t epoch = reinterpret_cast<const uint32_t*>(P.ws[P.rank])[0] + 1;
  if (z_ready(P, epoch, &ok_s)) {
    constexpr int EPV = BF16 ? 8 : 4;   // elements per 16-byte load
    const long nvec = shard_elems / EPV;
    const size_t slice_bytes = (size_t)shard_elems * (BF16 ? 2 : 4);
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
      uint4 vs[Z_MAX_RANKS];
#pragma unroll
      for (int s = 0; s < Z_MAX_RANKS; ++s)   // every peer's load is issued before the first use
        if (s < P.world) vs[s] = reinterpret_cast<const uint4*>(P.ws[s] + off + (size_t)P.rank * slice_bytes)[i];
#pragma unroll
      for (int s = 0; s < Z_MAX_RANKS; ++s) {
        if (s >= P.world) break;
        const uint4 v = vs[s];
        if (BF16) {
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f = bf162_bits_to_f2(w[k]);
            acc[2 * k] += f.x, acc[2 * k + 1] += f.y;
          }
        } else {
          acc[0] += __uint_as_float(v.x), acc[1] += __uint_as_float(v.y);
          acc[2] += __uint_as_float(v.z), acc[3] += __uint_as_float(v.w);
        }
      }
      float* o = out + i * EPV;
#pragma unroll
      for (int k = 0; k < EPV; ++k) o[k] = (accumulate ? o[k] : 0.f) + acc[k] * scale;
    }
  }
  z_done(P, epoch, &last_s);
}

ZPeers z_peers(void* const* ws, int rank, int world) {
  ZPeers P;
  for (int i = 0; i < Z_MAX_RANKS; ++i) P.ws[i] = i < world ? (unsigned char*)ws[i] : nullptr;
  P.rank = rank, P.world = world;
  return P;
}

int z_grid(long work_items) {
  // a modest grid: these kernels run beside the layer's compute and their CTAs spin while a
  // peer is late; 64 CTAs of 16-byte loads are enough to fill one NVLink direction
  return (int)max(1L, min(128L, (work_items + 511) / 512));
}

}  // namespace

TRL_API size_t trl_zero_data_offset() { return Z_OFF_DATA; }

// dst (local, 16-byte aligned) receives world * shard_bytes: the shards found at byte offset
// `off` (16-byte aligned, >= trl_zero_data_offset()) of the regions of ranks 0..world-1.
TRL_API int trl_zero_allgather(void* const* ws, int rank, int world, long off, long shard_bytes, void* dst,
                               void* stream) {
  if (shard_bytes % 16 != 0 || off % 16 != 0 || world > Z_MAX_RANKS || world < 1) return (int)cudaErrorInvalidValue;
  const long vecs = shard_bytes / 16;
  zero_allgather_kernel<<<z_grid(vecs), 512, 0, (cudaStream_t)stream>>>(z_peers(ws, rank, world), (size_t)off, vecs,
                                                                        (uint4*)dst);
  return (int)cudaGetLastError();
}

// At byte offset `off` every rank's region holds its full flat gradient (world * shard_elems
// elements, bf16 or fp32); out (fp32, shard_elems) = [out +] scale * sum over ranks of slice `rank`.
TRL_API int trl_zero_reduce_scatter(void* const* ws, int rank, int world, long off, long shard_elems, int is_bf16,
                                    float scale, void* out, int accumulate, void* stream) {
  if (shard_elems % 8 != 0 || off % 16 != 0 || world > Z_MAX_RANKS || world < 1) return (int)cudaErrorInvalidValue;
  const ZPeers P = z_peers(ws, rank, world);
  const int grid = z_grid(shard_elems / (is_bf16 ? 8 : 4));
  if (is_bf16)
    zero_reduce_scatter_kernel<true><<<grid, 512, 0, (cudaStream_t)stream>>>(P, (size_t)off, shard_elems, scale, (float*)out, accumulate);
  else
    zero_reduce_scatter_kernel<false><<<grid, 512, 0, (cudaStream_t)stream>>>(P, (size_t)off, shard_elems, scale, (float*)out, accumulate);
  return (int)cudaGetLastError();
}
