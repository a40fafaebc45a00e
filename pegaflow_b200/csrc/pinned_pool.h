// Pinned, GPU-mapped host memory and the allocator that hands out block storage from it.
// Replaces pegaflow-core/src/pinned_mem.rs (backing strategies), allocator.rs (offset
// allocator wrapper) and pinned_pool.rs (pool, shards, per-NUMA pools).
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <unordered_map>
#include <vector>

#include "common.h"

namespace pf {

// A pinned region with both of its addresses: the CPU's and the one kernels / DMA use.
// (Registered memory may map at a different device address, transfer/mod.rs:30-35.)
class PinnedMemory {
 public:
  enum class Strategy { CudaHostAlloc, MmapRegister, HugePages, MmapTransparentHuge };
  PinnedMemory(size_t bytes, Strategy strategy, int numa_node);
  ~PinnedMemory();
  PinnedMemory(const PinnedMemory &) = delete;
  PinnedMemory &operator=(const PinnedMemory &) = delete;
  char *host() const { return host_; }
  uint64_t device() const { return device_; }
  size_t size() const { return size_; }

 private:
  char *host_ = nullptr;
  uint64_t device_ = 0;
  size_t size_ = 0;
  Strategy strategy_;
};

// Workers used to pre-touch a mapping of `bytes` bytes, and the kernel's huge page size (0 when
// unknown): pinned_mem.rs:378-391 and `read_hugepage_size_from_proc`.
size_t pre_touch_threads(size_t bytes);
size_t huge_page_size();

// Best-fit offset allocator with neighbour coalescing, in units of `unit` bytes.
// Same observable rules as the reference's wrapper (allocator.rs:66-141): sizes round up to
// the unit, capacity rounds down, the first allocation of a fresh range sits at offset 0,
// freed neighbours merge.
class OffsetAllocator {
 public:
  OffsetAllocator(uint64_t total_bytes, uint64_t unit);
  // Returns false when no free range is large enough.
  bool allocate(uint64_t bytes, uint64_t *offset, uint64_t *granted);
  void release(uint64_t offset, uint64_t granted);
  uint64_t unit() const { return unit_; }
  uint64_t total_bytes() const { return total_; }
  uint64_t free_bytes() const { return free_; }
  uint64_t largest_free() const { return by_size_.empty() ? 0 : by_size_.rbegin()->first; }

 private:
  uint64_t unit_, total_, free_;
  std::map<uint64_t, uint64_t> by_offset_;              // offset -> length
  std::set<std::pair<uint64_t, uint64_t>> by_size_;     // (length, offset)
};

class PinnedPool;

// RAII allocation (pinned_pool.rs:57-115): returns its bytes to the pool when the last
// reference goes away.
class PinnedAllocation {
 public:
  PinnedAllocation(std::shared_ptr<PinnedPool> pool, uint64_t offset, uint64_t size);
  ~PinnedAllocation();
  char *host() const { return host_; }
  uint64_t device() const { return device_; }
  uint64_t size() const { return size_; }
  uint64_t offset() const { return offset_; }

 private:
  std::shared_ptr<PinnedPool> pool_;
  uint64_t offset_, size_;
  char *host_;
  uint64_t device_;
};

class PinnedPool : public std::enable_shared_from_this<PinnedPool> {
 public:
  PinnedPool(size_t bytes, PinnedMemory::Strategy strategy, uint64_t unit_hint, int numa_node);
  std::shared_ptr<PinnedAllocation> allocate(uint64_t bytes);  // nullptr when exhausted
  void usage(uint64_t *used, uint64_t *total, uint64_t *largest_free);
  const PinnedMemory &backing() const { return backing_; }

 private:
  friend class PinnedAllocation;
  void release(uint64_t offset, uint64_t size);
  PinnedMemory backing_;
  std::mutex mu_;
  OffsetAllocator alloc_;
};

// Shards (round-robin, fall through to the others) and optional per-NUMA-node pools
// (pinned_pool.rs:349-715).
class PinnedAllocator {
 public:
  // numa_nodes empty: one global (sharded) pool; otherwise capacity is split evenly and each
  // node's pool is created on a thread pinned to that node.
  PinnedAllocator(size_t capacity, const std::vector<int> &numa_nodes, int shards, PinnedMemory::Strategy strategy,
                  uint64_t unit_hint);
  std::shared_ptr<PinnedAllocation> allocate(uint64_t bytes, int numa_node);
  void usage(uint64_t *used, uint64_t *total);
  uint64_t largest_free(int numa_node);
  bool is_numa() const { return !by_node_.empty(); }

 private:
  struct Sharded {
    std::vector<std::shared_ptr<PinnedPool>> shards;
    std::atomic<size_t> cursor{0};
  };
  std::shared_ptr<PinnedAllocation> allocate_from(Sharded &s, uint64_t bytes);
  std::unique_ptr<Sharded> global_;
  std::unordered_map<int, std::unique_ptr<Sharded>> by_node_;
};

}  // namespace pf
