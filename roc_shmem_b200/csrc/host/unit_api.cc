// unit_api.cc — C entry points that expose internal building blocks (allocator,
// address records, team arithmetic) to the unit tests, the way the reference's
// gtest suite includes library-internal headers (clients/unit_tests/CMakeLists.txt:61-66).
#include <cstring>

#include "../include/bshmem_types.h"
#include "allocator.h"
#include "team.h"

using namespace bshmem;

extern "C" {

void* bshmem_unit_alloc_create(uint64_t heap_bytes, uint64_t reserved, uint64_t min_block) {
  return new Pow2BuddyAllocator(heap_bytes, reserved, min_block ? min_block : BSHMEM_ALIGNMENT);
}
void bshmem_unit_alloc_destroy(void* a) { delete static_cast<Pow2BuddyAllocator*>(a); }
uint64_t bshmem_unit_alloc(void* a, uint64_t bytes, uint64_t align) {
  return static_cast<Pow2BuddyAllocator*>(a)->alloc_aligned(bytes, align ? align : BSHMEM_ALIGNMENT);
}
int bshmem_unit_free(void* a, uint64_t off) { return static_cast<Pow2BuddyAllocator*>(a)->free(off) ? 1 : 0; }
uint64_t bshmem_unit_block_size(void* a, uint64_t off) { return static_cast<Pow2BuddyAllocator*>(a)->block_size(off); }
void bshmem_unit_usage(void* a, uint64_t out[9]) {
  HeapUsage u = static_cast<Pow2BuddyAllocator*>(a)->usage();
  out[0] = u.heap_bytes; out[1] = u.reserved_bytes; out[2] = u.allocated_bytes; out[3] = u.requested_bytes;
  out[4] = u.live_blocks; out[5] = u.largest_free; out[6] = u.n_allocs; out[7] = u.n_frees; out[8] = u.n_failed;
}
int bshmem_unit_roots(void* a, uint64_t* offsets, uint64_t* sizes, int max) {
  auto r = static_cast<Pow2BuddyAllocator*>(a)->roots();
  int n = 0;
  for (auto& x : r) { if (n >= max) break; offsets[n] = x.offset; sizes[n] = x.size; ++n; }
  return (int)r.size();
}
uint64_t bshmem_unit_round_up_pow2(uint64_t v, uint64_t min_block) { return Pow2BuddyAllocator::round_up_pow2(v, min_block); }

// AddressRecord: split returns the upper half in out[2..3], the shrunk record in out[0..1]
void bshmem_unit_record_split(uint64_t off, uint64_t size, uint64_t out[4]) {
  AddressRecord r{off, size};
  AddressRecord up = r.split();
  out[0] = r.offset; out[1] = r.size; out[2] = up.offset; out[3] = up.size;
}
int bshmem_unit_record_combine(uint64_t off_a, uint64_t size_a, uint64_t off_b, uint64_t size_b, uint64_t out[2]) {
  AddressRecord a{off_a, size_a};
  bool ok = a.combine(AddressRecord{off_b, size_b});
  out[0] = a.offset; out[1] = a.size;
  return ok ? 1 : 0;
}

void* bshmem_unit_mono_create(uint64_t base, uint64_t bytes, uint64_t align) { return new MonoLinearAllocator(base, bytes, align ? align : 128); }
uint64_t bshmem_unit_mono_alloc(void* m, uint64_t bytes) { return static_cast<MonoLinearAllocator*>(m)->alloc(bytes); }
void bshmem_unit_mono_reset(void* m) { static_cast<MonoLinearAllocator*>(m)->reset(); }
void bshmem_unit_mono_destroy(void* m) { delete static_cast<MonoLinearAllocator*>(m); }

// Team arithmetic on plain triplets: index of `pe` in (start, stride, size), or -1.
int bshmem_unit_team_index(int start, int stride, int size, int pe) { return TeamInfo{start, stride, size}.index_of(pe); }
int bshmem_unit_pick_slot(uint64_t mask) { return TeamTracker::pick_slot(mask); }

}  // extern "C"
