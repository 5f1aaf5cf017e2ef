// allocator.h — symmetric-heap allocation strategies (host-side metadata only).
//
// The heap itself may live in GPU memory (CUDA VMM) or in a shared-memory
// segment (CPU backend); these classes only hand out *offsets*, so the same
// code serves both.  Every PE runs its own instance and performs the same
// sequence of collective malloc/free calls, therefore every PE computes the
// same offsets and a symmetric address is "base[pe] + offset".
//
// Parity: library/src/memory/pow2_bins.hpp (power-of-two bins, split a larger
// bin on demand), binner.hpp (carve the heap into largest-first chunks),
// address_record.hpp, bin.hpp, dev_mono_linear.hpp (bump pointer).  Unlike the
// reference, free() coalesces buddies, so a long-running job does not
// fragment the heap into small bins for ever.
#pragma once
#include <cstdint>
#include <map>
#include <mutex>
#include <set>
#include <vector>

namespace bshmem {

constexpr uint64_t kNoOffset = ~0ull;

// One (offset, size) pair; split() / combine() mirror the buddy operations.
struct AddressRecord {
  uint64_t offset = 0;
  uint64_t size = 0;
  bool operator==(const AddressRecord& o) const { return offset == o.offset && size == o.size; }
  // Halve the record; returns the upper half and shrinks *this to the lower.
  AddressRecord split();
  // Merge with an adjacent record of the same size (either side).
  bool combine(const AddressRecord& other);
};

// A bin holds free blocks of one size, lowest address first (deterministic).
class Bin {
 public:
  bool empty() const { return free_.empty(); }
  size_t size() const { return free_.size(); }
  void put(uint64_t offset) { free_.insert(offset); }
  uint64_t take_lowest();
  bool take(uint64_t offset);
  bool contains(uint64_t offset) const { return free_.count(offset) != 0; }
 private:
  std::set<uint64_t> free_;
};

struct HeapUsage {
  uint64_t heap_bytes;
  uint64_t reserved_bytes;   // internal region at the start of the heap
  uint64_t allocated_bytes;  // sum of rounded block sizes currently live
  uint64_t requested_bytes;  // sum of the sizes the callers asked for
  uint64_t live_blocks;
  uint64_t largest_free;     // largest block a malloc could get right now
  uint64_t n_allocs, n_frees, n_failed;
};

// Power-of-two buddy allocator over [reserved, heap_bytes).
class Pow2BuddyAllocator {
 public:
  Pow2BuddyAllocator(uint64_t heap_bytes, uint64_t reserved_bytes, uint64_t min_block = 128);

  // Returns an offset from the heap base, or kNoOffset (size 0 or exhausted).
  uint64_t alloc(uint64_t bytes);
  // Aligned variant: alignment must be a power of two (blocks are naturally
  // aligned to their own size relative to their root chunk, roots are aligned
  // to min(block size, 2 MiB) so any alignment <= block size holds).
  uint64_t alloc_aligned(uint64_t bytes, uint64_t alignment);
  // Returns false when the offset is not the start of a live block.
  bool free(uint64_t offset);
  // Size of the live block starting at offset (0 if none).
  uint64_t block_size(uint64_t offset) const;
  HeapUsage usage() const;
  static uint64_t round_up_pow2(uint64_t v, uint64_t min_block);
  // Sizes of the root chunks the binner carved, largest first.
  std::vector<AddressRecord> roots() const { return roots_; }

 private:
  int order_of(uint64_t block) const;  // log2(block / min_block)
  const AddressRecord* root_of(uint64_t offset) const;

  uint64_t heap_bytes_, reserved_, min_block_;
  std::vector<AddressRecord> roots_;            // sorted by offset
  std::vector<Bin> bins_;                       // index = order
  std::map<uint64_t, std::pair<uint64_t, uint64_t>> live_;  // off -> (block, requested)
  uint64_t allocated_ = 0, requested_ = 0, n_allocs_ = 0, n_frees_ = 0, n_failed_ = 0;
  mutable std::mutex mu_;
};

// Monotonic bump allocator (host mirror of the device-callable slab): never
// frees individual blocks, reset() releases everything.
class MonoLinearAllocator {
 public:
  MonoLinearAllocator(uint64_t base, uint64_t bytes, uint64_t align = 128)
      : base_(base), end_(base + bytes), cur_(base), align_(align) {}
  uint64_t alloc(uint64_t bytes);
  void reset() { cur_ = base_; }
  uint64_t used() const { return cur_ - base_; }
 private:
  uint64_t base_, end_, cur_, align_;
};

}  // namespace bshmem
