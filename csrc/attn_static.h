// Allocation-free entry point for the split-KV paged attention.
//
// This entry point has no counterpart in the reference: it exists for embedders of this
// library that are not allowed to allocate device memory at call time -- a host process
// that has reserved the whole GPU for its own pools, a plug-in running under a fixed
// memory budget, or a latency-critical serving loop in which a cudaMalloc (which
// synchronises the device and may fail) is unacceptable.  Such callers still pass every
// input and output buffer; only the kernel's scratch (the per-split partial outputs,
// maxima and sums that the combine step reads) is provided by the library, from a
// file-scope device array of fixed size.
//
// Limits and rules:
//   * scratch need = T * n_q * n_splits * (D + 2) * 4 bytes must not exceed
//     TRL_ATTN_STATIC_SCRATCH_BYTES (8 MiB); larger problems are rejected with
//     cudaErrorInvalidValue and nothing is launched.
//   * The array exists once per GPU that loads the library and is held until the process
//     exits, whether or not this entry point is ever called.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current).  Make that first call before any
//     stream capture begins on the device.
//   * Every call uses the same array, so two calls whose kernels may overlap on the GPU
//     (different streams without an ordering between them) race; order them.  The array
//     keeps the previous call's contents; nothing in it has to start at zero, because every
//     (token, head, split) entry is written before the combine step reads it.
//   * No cudaMalloc / cudaFree / allocating library routine is called.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRL_ATTN_STATIC_SCRATCH_BYTES (8u << 20)

// Same contract as trl_attn_paged (csrc/attn.cu) minus the three scratch pointers.
// Returns 0 on success, otherwise a cudaError_t value.
int trl_attn_paged_static(const void* q, const void* gate_src, int gate_ld, const void* kcache,
                          const void* vcache, const void* block_table, int max_blocks, const void* seq_ids,
                          const void* positions, void* out, int T, int n_q, int n_kv, int D, int n_splits,
                          float scale, int gated, void* stream);

// Bytes of the static scratch a problem of this size needs (for callers that want to check first).
size_t trl_attn_static_scratch_needed(int T, int n_q, int D, int n_splits);

#ifdef __cplusplus
}
#endif
