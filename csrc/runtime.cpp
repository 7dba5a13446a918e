// Host-side runtime of the serving loop (no device code): the paged-KV block allocator and the
// builder of a tick's flat-token batch descriptor.  Both sit on the per-tick host path between
// two launches, where an interpreter loop over tokens costs more than the kernels it feeds at
// large batch; here they are plain C++ behind the same C ABI as the kernels.
//
//   pager      : free list + reference counts over the blocks of one KV pool (block 0 is the pad
//                page and is never handed out).  A block returns to the free list when its count
//                reaches zero; prefix-cache entries and running requests hold counts.
//   batch_fill : writes, for the scheduled sequences of a tick, every int32 array of the batch
//                descriptor into ONE staging block (the caller passes pinned memory, so the whole
//                descriptor goes to the device in a single copy):
//                [ids T][positions T][seq_ids T][slot_mapping T]
//                [q_start B][q_len B][kv_len B][state_slot B][last_idx B][keep B][block_table B x max_blocks]
//
// Reference parity: the allocator of src/tilerl/kv_cache.py:53-245 (PagedKvPool.alloc_block,
// refcounts, sentinel block) and the per-forward view of kv_cache.py:954-1015 (BatchKv) of the
// reference, both Python there.
#include <cstdint>
#include <cstring>
#include <new>
#include <vector>

#define TRL_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

struct Pager {
  std::vector<int32_t> ref;
  std::vector<int32_t> free_list;   // stack: the back is handed out next
};

inline bool valid(const Pager* p, int b) { return p != nullptr && b >= 0 && b < (int)p->ref.size(); }

}  // namespace

// A pool of `num_blocks` blocks; block 0 is reserved.  Blocks are handed out in ascending order.
TRL_HOST_API void* trl_pager_create(int num_blocks) {
  if (num_blocks < 1) return nullptr;
  Pager* p = new (std::nothrow) Pager();
  if (p == nullptr) return nullptr;
  p->ref.assign((size_t)num_blocks, 0);
  p->ref[0] = 1;
  p->free_list.reserve((size_t)num_blocks);
  for (int b = num_blocks - 1; b >= 1; --b) p->free_list.push_back(b);
  return p;
}

TRL_HOST_API void trl_pager_destroy(void* h) { delete static_cast<Pager*>(h); }

// One block with count 1, or -1 when the pool is exhausted.
TRL_HOST_API int trl_pager_alloc(void* h) {
  Pager* p = static_cast<Pager*>(h);
  if (p == nullptr || p->free_list.empty()) return -1;
  const int b = p->free_list.back();
  p->free_list.pop_back();
  p->ref[(size_t)b] = 1;
  return b;
}

// `n` blocks or none: returns n and fills `out`, or -1 (nothing taken) when fewer are free.
TRL_HOST_API int trl_pager_alloc_many(void* h, int n, int32_t* out) {
  Pager* p = static_cast<Pager*>(h);
  if (p == nullptr || n < 0 || (size_t)n > p->free_list.size()) return -1;
  for (int i = 0; i < n; ++i) {
    const int b = p->free_list.back();
    p->free_list.pop_back();
    p->ref[(size_t)b] = 1;
    out[i] = b;
  }
  return n;
}

// New count of a live block, or -1 for a free / out-of-range block (nothing changes).
TRL_HOST_API int trl_pager_incref(void* h, int b) {
  Pager* p = static_cast<Pager*>(h);
  if (!valid(p, b) || p->ref[(size_t)b] <= 0) return -1;
  return ++p->ref[(size_t)b];
}

// New count; at zero the block is free again.  -1 for block 0, a free or an out-of-range block.
TRL_HOST_API int trl_pager_release(void* h, int b) {
  Pager* p = static_cast<Pager*>(h);
  if (!valid(p, b) || b == 0 || p->ref[(size_t)b] <= 0) return -1;
  const int c = --p->ref[(size_t)b];
  if (c == 0) p->free_list.push_back(b);
  return c;
}

TRL_HOST_API int trl_pager_free_count(void* h) {
  Pager* p = static_cast<Pager*>(h);
  return p == nullptr ? 0 : (int)p->free_list.size();
}

TRL_HOST_API int trl_pager_refcount(void* h, int b) {
  Pager* p = static_cast<Pager*>(h);
  return valid(p, b) ? p->ref[(size_t)b] : -1;
}

// Copies the first min(n, num_blocks) counts; returns how many.
TRL_HOST_API int trl_pager_refs(void* h, int32_t* out, int n) {
  Pager* p = static_cast<Pager*>(h);
  if (p == nullptr || n <= 0) return 0;
  const int m = n < (int)p->ref.size() ? n : (int)p->ref.size();
  std::memcpy(out, p->ref.data(), (size_t)m * sizeof(int32_t));
  return m;
}

// Number of int32 values trl_batch_fill writes for T tokens of B sequences.
TRL_HOST_API long long trl_batch_ints(long long T, int B, int max_blocks) {
  return 4 * T + 6 * (long long)B + (long long)B * max_blocks;
}

// tokens [T] with tok_off [B+1] delimiting each sequence's tokens of this tick; starts [B] the
// absolute position of each sequence's first token; blocks with blk_off [B+1] its physical block
// list; keep [B] may be null.  Returns the number of int32 values written, -1 when `out` is too
// small or an argument is malformed, -2 when a token lies beyond its sequence's block list or a
// block list is longer than max_blocks.
TRL_HOST_API long long trl_batch_fill(int B, const int32_t* tokens, const int32_t* tok_off, const int32_t* starts,
                                      const int32_t* slots, const int32_t* keep, const int32_t* blocks,
                                      const int32_t* blk_off, int max_blocks, int kv_block, int32_t* out,
                                      long long out_cap) {
  if (B < 0 || max_blocks < 1 || kv_block < 1 || tok_off == nullptr || blk_off == nullptr) return -1;
  const long long T = B > 0 ? tok_off[B] : 0;
  const long long need = trl_batch_ints(T, B, max_blocks);
  if (T < 0 || need > out_cap) return -1;
  int32_t* ids = out;
  int32_t* pos = ids + T;
  int32_t* sid = pos + T;
  int32_t* smap = sid + T;
  int32_t* q_start = smap + T;
  int32_t* q_len = q_start + B;
  int32_t* kv_len = q_len + B;
  int32_t* slot = kv_len + B;
  int32_t* last = slot + B;
  int32_t* kp = last + B;
  int32_t* table = kp + B;
  std::memset(table, 0, (size_t)B * (size_t)max_blocks * sizeof(int32_t));
  for (int r = 0; r < B; ++r) {
    const int t0 = tok_off[r], n = tok_off[r + 1] - t0;
    const int nb = blk_off[r + 1] - blk_off[r];
    const int32_t* bl = blocks + blk_off[r];
    if (n < 0 || nb < 0 || nb > max_blocks) return -2;
    const int start = starts[r];
    q_start[r] = t0;
    q_len[r] = n;
    kv_len[r] = start + n;
    slot[r] = slots[r];
    last[r] = t0 + n - 1;
    kp[r] = keep != nullptr ? (keep[r] != 0) : 0;
    std::memcpy(table + (size_t)r * max_blocks, bl, (size_t)nb * sizeof(int32_t));
    for (int j = 0; j < n; ++j) {
      const int p = start + j;
      const int page = p / kv_block;
      if (p < 0 || page >= nb) return -2;
      ids[t0 + j] = tokens[t0 + j];
      pos[t0 + j] = p;
      sid[t0 + j] = r;
      smap[t0 + j] = bl[page] * kv_block + p % kv_block;
    }
  }
  return need;
}
