// Shared device helpers for the sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TRL_API extern "C" __attribute__((visibility("default")))

// ---- global loads and programmatic dependent launch -----------------------------------------
// Every kernel of a tick calls griddepcontrol.launch_dependents first, so CTAs of several
// consecutive kernels sit on one SM at the same time and share its L1.  A line that an older,
// still resident kernel read (the residual stream before this layer's update, a projection
// buffer of the previous layer) can stay in that L1 and be hit by a younger kernel after its
// griddepcontrol.wait: measured on a B200 as a stale activation row in a two-row decode tick.
// Data that another kernel of the stream writes is therefore never read through L1: the
// extension is compiled with `-Xptxas -dlcm=cg` (plain global loads go to L2), and only pointers
// to constants of a tick (weights, norm and conv vectors, tables) carry `__restrict__`, so the
// compiler cannot route a load of an activation, a state or a batch descriptor through the
// read-only (L1) path either.  Streaming weight loads name their cache policy explicitly
// (ldg_stream_*).

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// ---- error word ------------------------------------------------------------------
// Kernels never trap.  A bounded wait that runs out (or a debug bounds check that
// fails) records {code, a, b, c} in this device-global word set and returns; the
// host reads it with trl_error_read() after the step.
struct TrlError {
  int code;
  int a, b, c;
};
enum { TRL_OK = 0, TRL_ERR_WAIT_TIMEOUT = 1, TRL_ERR_BOUNDS = 2, TRL_ERR_MBAR_TIMEOUT = 3 };
extern __device__ TrlError g_trl_error;

__device__ __forceinline__ void trl_set_error(int code, int a, int b, int c) {
  if (atomicCAS(&g_trl_error.code, 0, code) == 0) {
    g_trl_error.a = a;
    g_trl_error.b = b;
    g_trl_error.c = c;
  }
}

// Checked table index.  Builds with -DTRL_DEBUG_BOUNDS only (python -m tilerl_b200.build --bounds): an index
// outside [0, n) records the error word {TRL_ERR_BOUNDS, site, index, n} and comes back clamped into range,
// so the access that follows stays inside the buffer and the context stays usable; the normal build
// compiles to the bare index.  Sites: 1 KV slot of a token (attn_prep), 2 block-table entry in decode
// attention, 3 block-table entry in prefill attention, 4 KV slot in the one-launch decode attention.
#ifdef TRL_DEBUG_BOUNDS
__device__ __forceinline__ int trl_checked(int i, int n, int site) {
  if ((unsigned)i >= (unsigned)n) {
    trl_set_error(TRL_ERR_BOUNDS, site, i, n);
    return n > 0 ? min(max(i, 0), n - 1) : 0;
  }
  return i;
}
#else
__device__ __forceinline__ int trl_checked(int i, int, int) { return i; }
#endif

// ---- tensor-parallel push target (see comm.cu) --------------------------------------------
// Peer workspace pointers for the row-parallel GEMV epilogue that writes its fp32 partial
// rows into every rank's one-shot all-reduce slot.
struct TrlPushArgs {
  unsigned char* ws[8];
  int rank, world, hmax, row0;
};

// ---- tick timeline (builds with -DTRL_TRACE only) ----------------------------------------------
// Per launch: {kind, entry of CTA 0, end of its dependency wait, its exit, two phase marks of CTA 0
// (trl_trace_mark), the latest exit of any CTA of the launches before it, unused, eight more marks} in
// nanoseconds of %globaltimer, recorded from pdl_launch_dependents(kind) / pdl_wait() /
// trl_trace_end(); trl_trace_read copies the records out.  Without the flag nothing is compiled in.
#ifdef TRL_TRACE
constexpr int TRL_TRACE_CAP = 8192;
struct TrlTraceRec { unsigned long long kind, t_entry, t_dep, t_exit, t_mark[2], t_prev_last_exit, pad, t_more[8]; };
extern __device__ unsigned long long g_trl_last_exit;
extern __device__ TrlTraceRec g_trl_trace[TRL_TRACE_CAP];
extern __device__ unsigned int g_trl_trace_n;
__device__ __forceinline__ unsigned long long trl_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned int& trl_trace_slot() {
  __shared__ unsigned int s;
  return s;
}
__device__ __forceinline__ bool trl_trace_lead() {
  return threadIdx.x == 0 && threadIdx.y == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
}
__device__ __forceinline__ void trl_trace_begin(int kind) {
  if (trl_trace_lead()) {
    const unsigned int i = atomicAdd(&g_trl_trace_n, 1u);
    trl_trace_slot() = i;
    if (i < TRL_TRACE_CAP) {
      g_trl_trace[i].kind = (unsigned long long)kind, g_trl_trace[i].t_entry = trl_now();
      g_trl_trace[i].t_dep = 0, g_trl_trace[i].t_exit = 0;
      g_trl_trace[i].t_mark[0] = 0, g_trl_trace[i].t_mark[1] = 0, g_trl_trace[i].t_prev_last_exit = 0;
      for (int k = 0; k < 8; ++k) g_trl_trace[i].t_more[k] = 0;
    }
  }
}
__device__ __forceinline__ void trl_trace_dep() {
  if (trl_trace_lead() && trl_trace_slot() < TRL_TRACE_CAP) {
    g_trl_trace[trl_trace_slot()].t_dep = trl_now();
    // every CTA of the launches this one depends on has exited: take their latest exit
    g_trl_trace[trl_trace_slot()].t_prev_last_exit = atomicExch(&g_trl_last_exit, 0ull);
  }
}
__device__ __forceinline__ void trl_trace_mark(int which) {
  if (trl_trace_lead() && trl_trace_slot() < TRL_TRACE_CAP) {
    if (which < 2) g_trl_trace[trl_trace_slot()].t_mark[which] = trl_now();
    else if (which < 10) g_trl_trace[trl_trace_slot()].t_more[which - 2] = trl_now();
  }
}
__device__ __forceinline__ void trl_trace_end() {
  if (threadIdx.x == 0 && threadIdx.y == 0) atomicMax(&g_trl_last_exit, trl_now());
  if (trl_trace_lead() && trl_trace_slot() < TRL_TRACE_CAP) g_trl_trace[trl_trace_slot()].t_exit = trl_now();
}
#else
__device__ __forceinline__ void trl_trace_begin(int) {}
__device__ __forceinline__ void trl_trace_dep() {}
__device__ __forceinline__ void trl_trace_mark(int) {}
__device__ __forceinline__ void trl_trace_end() {}
#endif

// ---- programmatic dependent launch ----------------------------------------------------
// Every kernel calls pdl_launch_dependents() first (the next kernel in the stream
// may begin its own prologue) and pdl_wait() before touching anything a
// predecessor wrote.  Without the launch attribute both are no-ops.  `kind` names the kernel in
// the timeline of a -DTRL_TRACE build.
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  trl_trace_dep();
}
__device__ __forceinline__ void pdl_launch_dependents(int kind = 0) {
  trl_trace_begin(kind);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// The same in two steps, for kernels that let their dependents in later than at entry.
__device__ __forceinline__ void pdl_enter(int kind = 0) { trl_trace_begin(kind); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- small math --------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum / max through `red` (>= 32 floats of shared memory).  All threads
// must call; result is broadcast.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(r);
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// 8-byte store visible system-wide as one unit (value + epoch pairs of the one-shot all-reduce)
// (a single 64-bit scalar access: single-copy atomic by the PTX memory model)
__device__ __forceinline__ void st_relaxed_sys_v2(void* p, uint2 v) {
  const unsigned long long w = ((unsigned long long)v.y << 32) | (unsigned long long)v.x;
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_relaxed_sys_v2(const void* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return make_uint2((uint32_t)w, (uint32_t)(w >> 32));
}

// ---- streaming loads -----------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream_8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_4(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint16_t ldg_stream_2(const void* p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

// ---- narrow float decode --------------------------------------------------------------------
// Four bytes of packed e2m1 (low nibble = even element) -> four f16x2 registers.
__device__ __forceinline__ void cvt_e2m1x8_to_h2x4(uint32_t w, uint32_t (&h)[4]) {
  asm("{ .reg .b8 b0, b1, b2, b3;\n"
      "  mov.b32 {b0, b1, b2, b3}, %4;\n"
      "  cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "  cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "  cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "  cvt.rn.f16x2.e2m1x2 %3, b3; }\n"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}
// Two e4m3 bytes -> f16x2.
__device__ __forceinline__ uint32_t cvt_e4m3x2_to_h2(uint16_t s) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(s));
  return r;
}
__device__ __forceinline__ float2 h2_to_f2(uint32_t h) {
  __half2 v = *reinterpret_cast<__half2*>(&h);
  return __half22float2(v);
}
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float bf16_bits_to_f(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
__device__ __forceinline__ float2 bf162_bits_to_f2(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
__device__ __forceinline__ uint32_t f2_to_bf162_bits(float a, float b) {
  bf162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---- launch helper (host) ---------------------------------------------------------------------
// Launch with the programmatic-stream-serialization attribute so consecutive
// kernels of a tick overlap their tails/prologues (also inside CUDA graphs).
extern int g_trl_use_pdl;
template <typename... KArgs, typename... Args>
static inline cudaError_t trl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_trl_use_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
