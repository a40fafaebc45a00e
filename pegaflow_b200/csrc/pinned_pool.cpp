#include "pinned_pool.h"

#include <cuda_runtime.h>
#include <sched.h>
#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <fstream>
#include <string>
#include <thread>

#include "layout.h"
#include "numa.h"

namespace pf {

namespace {
std::string cuda_msg(const char *what, cudaError_t e) {
  return strf("%s failed: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

// Touch one byte per page (and the last byte) from several threads bound to `node`, so that the
// kernel places the pages there before cudaHostRegister pins them (pinned_mem.rs:343-391).
void parallel_pre_touch(char *ptr, size_t bytes, size_t page, int node) {
  const size_t n_threads = pre_touch_threads(bytes);
  const size_t chunk = (bytes + n_threads - 1) / n_threads;
  std::vector<std::thread> threads;
  for (size_t t = 0; t < n_threads; ++t) {
    const size_t off = t * chunk;
    if (off >= bytes) break;
    const size_t len = std::min(chunk, bytes - off);
    threads.emplace_back([=] {
      if (node >= 0) numa::pin_thread_to_node(node);
      volatile char *p = ptr + off;
      for (size_t o = 0; o < len; o += page) p[o] = 0;
      p[len - 1] = 0;
    });
  }
  for (auto &t : threads) t.join();
}
}  // namespace

// pinned_mem.rs:378-391 `touch_threads`: one worker per GiB (rounded up), never more than the
// CPUs this process may run on.
size_t pre_touch_threads(size_t bytes) {
  const size_t by_size = std::max<size_t>(1, (bytes + (1ull << 30) - 1) >> 30);
  cpu_set_t set;
  size_t by_cpu = 0;
  if (sched_getaffinity(0, sizeof set, &set) == 0) by_cpu = (size_t)CPU_COUNT(&set);
  if (by_cpu == 0) by_cpu = 8;
  return std::min(by_size, by_cpu);
}

// `Hugepagesize:    2048 kB` of /proc/meminfo in bytes, 0 when the line is absent
// (pinned_mem.rs `read_hugepage_size_from_proc`).
size_t huge_page_size() {
  std::ifstream f("/proc/meminfo");
  std::string line;
  while (std::getline(f, line)) {
    if (line.rfind("Hugepagesize:", 0) != 0) continue;
    unsigned long long kb = 0;
    if (sscanf(line.c_str() + 13, "%llu", &kb) == 1 && kb) return (size_t)kb << 10;
  }
  return 0;
}

PinnedMemory::PinnedMemory(size_t bytes, Strategy strategy, int numa_node) : size_(bytes), strategy_(strategy) {
  if (bytes == 0) throw Error::storage("pinned memory size must be greater than zero");
  if (strategy == Strategy::CudaHostAlloc) {
    // The driver places the pages by the calling thread's memory policy, so a known node is
    // honoured by allocating from a thread pinned to it (pinned_mem.rs:149-185 does the same
    // through its per-node allocation threads).  The helper thread keeps the caller's device.
    void *p = nullptr;
    cudaError_t e = cudaSuccess;
    int device = 0;
    cudaGetDevice(&device);
    auto alloc = [&] {
      cudaSetDevice(device);
      e = cudaHostAlloc(&p, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
    };
    if (numa_node >= 0) numa::run_on_node(numa_node, alloc);
    else alloc();
    if (e != cudaSuccess) throw Error::storage(cuda_msg("cudaHostAlloc", e));
    host_ = static_cast<char *>(p);
  } else {
    const bool huge = strategy == Strategy::HugePages;
    const bool thp = strategy == Strategy::MmapTransparentHuge;
    const size_t page = huge || thp ? huge_page_size() : (size_t)sysconf(_SC_PAGESIZE);
    if (page == 0) throw Error::storage("huge page size is not available from /proc/meminfo");
    size_ = (bytes + page - 1) / page * page;
    int flags = MAP_PRIVATE | MAP_ANONYMOUS | (huge ? MAP_HUGETLB : 0);
    void *p = mmap(nullptr, size_, PROT_READ | PROT_WRITE, flags, -1, 0);
    if (p == MAP_FAILED)
      throw Error::storage(strf("mmap of %zu bytes failed%s", size_, huge ? " (are huge pages reserved?)" : ""));
    host_ = static_cast<char *>(p);
    // Advice only: a kernel whose transparent huge pages are off ignores it and the pool is backed by
    // ordinary pages.  (The mapping is not 2 MiB aligned; the kernel uses huge pages for the aligned part.)
    if (thp) madvise(host_, size_, MADV_HUGEPAGE);
    parallel_pre_touch(host_, size_, (size_t)sysconf(_SC_PAGESIZE), numa_node);
    cudaError_t e = cudaHostRegister(host_, size_, cudaHostRegisterMapped | cudaHostRegisterPortable);
    if (e != cudaSuccess) {
      munmap(host_, size_);
      host_ = nullptr;
      throw Error::storage(cuda_msg("cudaHostRegister", e));
    }
  }
  void *dev = nullptr;
  cudaError_t e = cudaHostGetDevicePointer(&dev, host_, 0);
  if (e != cudaSuccess) throw Error::storage(cuda_msg("cudaHostGetDevicePointer", e));
  device_ = (uint64_t)(uintptr_t)dev;
}

PinnedMemory::~PinnedMemory() {
  if (!host_) return;
  if (strategy_ == Strategy::CudaHostAlloc) {
    cudaFreeHost(host_);
  } else {
    cudaHostUnregister(host_);
    munmap(host_, size_);
  }
}

OffsetAllocator::OffsetAllocator(uint64_t total_bytes, uint64_t unit) : unit_(unit) {
  if (unit == 0) throw Error::storage("unit size must be greater than zero");
  total_ = total_bytes / unit * unit;
  free_ = total_;
  if (total_) {
    by_offset_[0] = total_;
    by_size_.insert({total_, 0});
  }
}

bool OffsetAllocator::allocate(uint64_t bytes, uint64_t *offset, uint64_t *granted) {
  if (bytes == 0) return false;
  const uint64_t need = (bytes + unit_ - 1) / unit_ * unit_;
  auto it = by_size_.lower_bound({need, 0});  // smallest sufficient range, lowest offset first
  if (it == by_size_.end()) return false;
  const uint64_t len = it->first, off = it->second;
  by_size_.erase(it);
  by_offset_.erase(off);
  if (len > need) {
    by_offset_[off + need] = len - need;
    by_size_.insert({len - need, off + need});
  }
  free_ -= need;
  *offset = off;
  *granted = need;
  return true;
}

void OffsetAllocator::release(uint64_t offset, uint64_t granted) {
  uint64_t off = offset, len = granted;
  auto next = by_offset_.lower_bound(off);
  if (next != by_offset_.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == off) {
      off = prev->first;
      len += prev->second;
      by_size_.erase({prev->second, prev->first});
      by_offset_.erase(prev);
    }
  }
  if (next != by_offset_.end() && offset + granted == next->first) {
    len += next->second;
    by_size_.erase({next->second, next->first});
    by_offset_.erase(next);
  }
  by_offset_[off] = len;
  by_size_.insert({len, off});
  free_ += granted;
}

PinnedAllocation::PinnedAllocation(std::shared_ptr<PinnedPool> pool, uint64_t offset, uint64_t size)
    : pool_(std::move(pool)), offset_(offset), size_(size) {
  host_ = pool_->backing().host() + offset;
  device_ = pool_->backing().device() + offset;
}

PinnedAllocation::~PinnedAllocation() { pool_->release(offset_, size_); }

PinnedPool::PinnedPool(size_t bytes, PinnedMemory::Strategy strategy, uint64_t unit_hint, int numa_node)
    : backing_(bytes, strategy, numa_node), alloc_(backing_.size(), pool_unit_size(backing_.size(), unit_hint)) {}

std::shared_ptr<PinnedAllocation> PinnedPool::allocate(uint64_t bytes) {
  uint64_t off, granted;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (!alloc_.allocate(bytes, &off, &granted)) return nullptr;
  }
  return std::make_shared<PinnedAllocation>(shared_from_this(), off, granted);
}

void PinnedPool::release(uint64_t offset, uint64_t size) {
  std::lock_guard<std::mutex> g(mu_);
  alloc_.release(offset, size);
}

void PinnedPool::usage(uint64_t *used, uint64_t *total, uint64_t *largest_free) {
  std::lock_guard<std::mutex> g(mu_);
  if (total) *total = alloc_.total_bytes();
  if (used) *used = alloc_.total_bytes() - alloc_.free_bytes();
  if (largest_free) *largest_free = alloc_.largest_free();
}

PinnedAllocator::PinnedAllocator(size_t capacity, const std::vector<int> &numa_nodes, int shards,
                                 PinnedMemory::Strategy strategy, uint64_t unit_hint) {
  const size_t n_shards = (size_t)std::max(1, shards);
  auto make = [&](size_t bytes, int node) {
    auto s = std::make_unique<Sharded>();
    const size_t per = bytes / n_shards;
    for (size_t i = 0; i < n_shards; ++i) s->shards.push_back(std::make_shared<PinnedPool>(per, strategy, unit_hint, node));
    return s;
  };
  if (numa_nodes.empty()) {
    global_ = make(capacity, numa::kUnknown);
    return;
  }
  const size_t per_node = capacity / numa_nodes.size();
  for (int node : numa_nodes) {
    if (node < 0) continue;
    std::unique_ptr<Sharded> made;
    numa::run_on_node(node, [&] { made = make(per_node, node); });
    by_node_[node] = std::move(made);
  }
}

std::shared_ptr<PinnedAllocation> PinnedAllocator::allocate_from(Sharded &s, uint64_t bytes) {
  const size_t n = s.shards.size();
  const size_t start = s.cursor.fetch_add(1, std::memory_order_relaxed) % n;
  for (size_t i = 0; i < n; ++i)
    if (auto a = s.shards[(start + i) % n]->allocate(bytes)) return a;
  return nullptr;
}

std::shared_ptr<PinnedAllocation> PinnedAllocator::allocate(uint64_t bytes, int numa_node) {
  if (global_) return allocate_from(*global_, bytes);
  auto it = by_node_.find(numa_node);
  if (it == by_node_.end()) return nullptr;
  return allocate_from(*it->second, bytes);
}

void PinnedAllocator::usage(uint64_t *used, uint64_t *total) {
  uint64_t u = 0, t = 0;
  auto add = [&](Sharded &s) {
    for (auto &p : s.shards) {
      uint64_t pu, pt;
      p->usage(&pu, &pt, nullptr);
      u += pu;
      t += pt;
    }
  };
  if (global_) add(*global_);
  for (auto &kv : by_node_) add(*kv.second);
  *used = u;
  *total = t;
}

uint64_t PinnedAllocator::largest_free(int numa_node) {
  uint64_t best = 0;
  auto scan = [&](Sharded &s) {
    for (auto &p : s.shards) {
      uint64_t lf;
      p->usage(nullptr, nullptr, &lf);
      best = std::max(best, lf);
    }
  };
  if (global_) {
    scan(*global_);
  } else {
    auto it = by_node_.find(numa_node);
    if (it != by_node_.end()) scan(*it->second);
  }
  return best;
}

}  // namespace pf
