// allocator.cc — buddy allocator over heap offsets.  See allocator.h.
#include "allocator.h"

#include <algorithm>

namespace bshmem {

AddressRecord AddressRecord::split() {
  size /= 2;
  return AddressRecord{offset + size, size};
}

bool AddressRecord::combine(const AddressRecord& o) {
  if (o.size != size) return false;
  if (o.offset == offset + size) { size *= 2; return true; }
  if (offset == o.offset + o.size) { offset = o.offset; size *= 2; return true; }
  return false;
}

uint64_t Bin::take_lowest() {
  auto it = free_.begin();
  uint64_t off = *it;
  free_.erase(it);
  return off;
}

bool Bin::take(uint64_t offset) { return free_.erase(offset) != 0; }

uint64_t Pow2BuddyAllocator::round_up_pow2(uint64_t v, uint64_t min_block) {
  uint64_t b = min_block;
  // stop at the top bit: a request above 2^63 has no power of two to round up to (the caller's size check rejects it)
  while (b < v && b < (1ull << 63)) b <<= 1;
  return b;
}

Pow2BuddyAllocator::Pow2BuddyAllocator(uint64_t heap_bytes, uint64_t reserved, uint64_t min_block)
    : heap_bytes_(heap_bytes), reserved_(reserved), min_block_(min_block) {
  // Round the start of the user region up to the minimum block.
  uint64_t p = (reserved_ + min_block_ - 1) / min_block_ * min_block_;
  reserved_ = p;
  // Carve [p, heap) into naturally aligned power-of-two roots: at each
  // position take the largest block that is both aligned there and fits.
  while (p + min_block_ <= heap_bytes_) {
    uint64_t s = min_block_;
    while (true) {
      uint64_t n = s << 1;
      if (n == 0 || p % n != 0 || p + n > heap_bytes_) break;
      s = n;
    }
    roots_.push_back({p, s});
    p += s;
  }
  uint64_t largest = min_block_;
  for (auto& r : roots_) largest = std::max(largest, r.size);
  bins_.resize(order_of(largest) + 1);
  for (auto& r : roots_) bins_[order_of(r.size)].put(r.offset);
}

int Pow2BuddyAllocator::order_of(uint64_t block) const {
  int o = 0;
  uint64_t b = min_block_;
  while (b < block) { b <<= 1; ++o; }
  return o;
}

const AddressRecord* Pow2BuddyAllocator::root_of(uint64_t offset) const {
  // roots_ is sorted by offset; find the last root starting at or below.
  auto it = std::upper_bound(roots_.begin(), roots_.end(), offset,
                             [](uint64_t v, const AddressRecord& r) { return v < r.offset; });
  if (it == roots_.begin()) return nullptr;
  --it;
  if (offset >= it->offset + it->size) return nullptr;
  return &*it;
}

uint64_t Pow2BuddyAllocator::alloc(uint64_t bytes) { return alloc_aligned(bytes, min_block_); }

uint64_t Pow2BuddyAllocator::alloc_aligned(uint64_t bytes, uint64_t alignment) {
  std::lock_guard<std::mutex> g(mu_);
  if (bytes == 0) return kNoOffset;
  if (alignment == 0 || (alignment & (alignment - 1)) != 0) return kNoOffset;
  if (std::max(bytes, alignment) > heap_bytes_) { ++n_failed_; return kNoOffset; }   // can never fit (and bounds the rounding)
  // A block is aligned to its own size, so asking for max(bytes, alignment)
  // rounded to a power of two satisfies the alignment.
  uint64_t block = round_up_pow2(std::max(bytes, alignment), min_block_);
  if (block < bytes) { ++n_failed_; return kNoOffset; }  // overflow
  int want = order_of(block);
  int have = -1;
  for (int o = want; o < (int)bins_.size(); ++o) {
    if (!bins_[o].empty()) { have = o; break; }
  }
  if (have < 0) { ++n_failed_; return kNoOffset; }
  AddressRecord rec{bins_[have].take_lowest(), min_block_ << have};
  while (have > want) {  // split down, keep the lower half, bin the upper
    AddressRecord upper = rec.split();
    --have;
    bins_[have].put(upper.offset);
  }
  live_[rec.offset] = {rec.size, bytes};
  allocated_ += rec.size;
  requested_ += bytes;
  ++n_allocs_;
  return rec.offset;
}

bool Pow2BuddyAllocator::free(uint64_t offset) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = live_.find(offset);
  if (it == live_.end()) return false;
  AddressRecord rec{offset, it->second.first};
  allocated_ -= it->second.first;
  requested_ -= it->second.second;
  live_.erase(it);
  ++n_frees_;
  const AddressRecord* root = root_of(offset);
  // Coalesce with the buddy while it is free and we stay inside the root.
  while (root && rec.size < root->size) {
    uint64_t buddy = rec.offset ^ rec.size;
    int o = order_of(rec.size);
    if (!bins_[o].take(buddy)) break;
    rec.combine(AddressRecord{buddy, rec.size});
  }
  bins_[order_of(rec.size)].put(rec.offset);
  return true;
}

uint64_t Pow2BuddyAllocator::block_size(uint64_t offset) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = live_.find(offset);
  return it == live_.end() ? 0 : it->second.first;
}

HeapUsage Pow2BuddyAllocator::usage() const {
  std::lock_guard<std::mutex> g(mu_);
  HeapUsage u{};
  u.heap_bytes = heap_bytes_;
  u.reserved_bytes = reserved_;
  u.allocated_bytes = allocated_;
  u.requested_bytes = requested_;
  u.live_blocks = live_.size();
  u.largest_free = 0;
  for (int o = (int)bins_.size() - 1; o >= 0; --o) {
    if (!bins_[o].empty()) { u.largest_free = min_block_ << o; break; }
  }
  u.n_allocs = n_allocs_;
  u.n_frees = n_frees_;
  u.n_failed = n_failed_;
  return u;
}

uint64_t MonoLinearAllocator::alloc(uint64_t bytes) {
  if (bytes == 0) return kNoOffset;
  uint64_t p = (cur_ + align_ - 1) / align_ * align_;
  if (p + bytes > end_ || p + bytes < p) return kNoOffset;
  cur_ = p + bytes;
  return p;
}

}  // namespace bshmem
