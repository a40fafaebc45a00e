// The transfer backend: every byte the engine moves between HBM and the pinned host pool (or
// a peer GPU) goes through this class.  It replaces the reference's two backends
// (pegaflow-core/src/transfer/memcpy.rs, kernel.rs) with one path that has two routes:
//
//   staged    scattered KV blocks are gathered by a kernel into a contiguous HBM staging ring
//             at HBM speed, and the copy engine moves each slot to/from the pool in one large
//             DMA (256-byte PCIe payloads).  Gather of slot i+1 overlaps the DMA of slot i.
//   zero-copy a TMA ring kernel (a handful of CTAs, one issuing thread each) moves blocks
//             directly between HBM and mapped pinned memory; used where the host side is
//             irregular or the batch is too small to amortise the staging hand-off.
//
// All calls only enqueue work (transfer/mod.rs:51-52 contract): nothing here synchronises the
// caller's stream.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <deque>
#include <vector>

#include "common.h"

namespace pf {

// One side of a batch of equally sized items: item i lives at table[i], or at
// base + (ids ? ids[i] : i) * stride.  `ids` / `table` are device pointers.
struct Side {
  uint64_t base;
  uint64_t stride;
  const uint32_t *ids;
  const uint64_t *table;
};

class TransferBackend {
 public:
  TransferBackend(int device, const pf_backend_config *config);
  ~TransferBackend();
  TransferBackend(const TransferBackend &) = delete;
  TransferBackend &operator=(const TransferBackend &) = delete;

  int device() const { return device_; }
  const char *name() const { return "b200"; }

  void copy_descs(const pf_copy_desc *copies, size_t n, bool host_is_src, cudaStream_t stream);
  void move_layers(const pf_layer_xfer *layers, size_t n_layers, bool host_is_src, cudaStream_t stream,
                   void *const *layer_done);
  // The HBM half of a staged save on its own: the gather kernels fill the staging ring exactly
  // as move_layers(.., host_is_src = false, ..) would, and no DMA leaves the ring.  For timing the
  // kernel alone; runs that do not take the staged route are rejected.
  void gather_layers(const pf_layer_xfer *layers, size_t n_layers, cudaStream_t stream);
  void peer_copy(const pf_device_layout &src, const uint32_t *src_ids, const pf_device_layout &dst,
                 const uint32_t *dst_ids, size_t n_blocks, cudaStream_t stream);
  // The same for several layers that share the block ids: one upload of the ids, a few launches.
  void peer_copy_layers(const pf_device_layout *src, const pf_device_layout *dst, size_t n_layers,
                        const uint32_t *src_ids, const uint32_t *dst_ids, size_t n_blocks, cudaStream_t stream);
  void stats(pf_backend_stats *out);

 private:
  struct Slot {
    char *ptr = nullptr;
    cudaEvent_t filled = nullptr;   // staging slot holds data (gather done / DMA-in done)
    cudaEvent_t drained = nullptr;  // staging slot may be overwritten (DMA-out done / scatter done)
    bool used = false;
  };
  struct MetaRegion {
    size_t begin, end;
    cudaEvent_t done;
  };
  struct TimedLaunch {
    cudaEvent_t start, stop;
    uint64_t bytes;
    bool link;
    int stamp_idx;  // slot of the kernel's own {start, end} stamps, -1 if none
  };

  // Meta ring: pinned host bytes + device mirror for block ids, address tables and descriptors.
  size_t meta_alloc(size_t bytes);
  void meta_upload(size_t off, size_t bytes, cudaStream_t stream);
  void meta_grow(size_t need);
  cudaEvent_t take_event();

  Slot &next_slot();
  void ensure_staging();

  // Kernel launchers (transfer.cu).
  struct StagedUnit;
  struct HeldGroup;
  void launch_group(const StagedUnit *units, char *const *slot_ptrs, size_t count, bool to_staging, cudaStream_t s);
  void launch_held(const std::vector<HeldGroup> &held, bool to_staging, cudaStream_t s);
  void launch_link(const Side &src, const Side &dst, size_t n_items, size_t item_bytes, cudaStream_t s,
                   bool peer);
  void launch_descs(const uint64_t *triples_dev, size_t n, bool aligned, cudaStream_t s);

  // One run of one range of one layer through the staged route.
  void staged_run(const Side &dev_side, const pf_host_run &run, size_t item_bytes, bool host_is_src,
                  cudaStream_t stream);
  void flush_group(bool may_hold);
  void emit_held();
  int next_aux();
  void join_copy_streams(cudaStream_t target, std::vector<char> &dirty, int skip);

  int device_;
  pf_backend_config cfg_;
  int sm_count_ = 0;
  // The open group of the staged route: units that will share one staging slot and one DMA.
  struct StagedUnit {
    Side dev;
    size_t n_items, item_bytes, slot_offset;
    char *host;
    size_t host_stride;
  };
  std::vector<StagedUnit> group_;
  // Closed save groups whose gather has not been launched yet (see flush_group).
  struct HeldGroup {
    Slot *slot = nullptr;
    int copy_index = -1;       // copy stream of the group's DMA; -1: no DMA (gather_layers)
    std::vector<StagedUnit> units;
    size_t bytes = 0;
    bool dense = true;
    char *host_begin = nullptr;
    cudaStream_t stream = nullptr;
  };
  std::vector<HeldGroup> held_;
  size_t group_bytes_ = 0;
  size_t group_limit_ = ~(size_t)0;  // current size limit of a group (ramps up within a call)
  char *group_host_begin_ = nullptr, *group_host_end_ = nullptr;
  bool group_dense_ = true, group_host_is_src_ = false;
  bool gather_only_ = false;             // set for the duration of gather_layers
  cudaStream_t group_stream_ = nullptr;

  std::vector<cudaStream_t> aux_;      // copy-engine streams of the staged route
  std::vector<cudaEvent_t> aux_join_;  // one per copy stream, for joining it into another stream
  cudaEvent_t fork_ = nullptr;         // caller's stream position at the start of a load call
  std::vector<char> aux_forked_;       // copy streams that already wait for fork_ in this call
  std::vector<char> aux_layer_dirty_, aux_task_dirty_;  // copy streams used by the current layer / call
  size_t aux_cursor_ = 0;
  int aux_last_ = 0;
  std::vector<Slot> slots_;
  char *staging_ = nullptr;
  size_t slot_cursor_ = 0;

  char *meta_host_ = nullptr;
  char *meta_dev_ = nullptr;
  size_t meta_cap_ = 0, meta_head_ = 0;
  std::deque<MetaRegion> meta_inflight_;
  std::vector<cudaEvent_t> event_pool_;

  unsigned int *status_host_ = nullptr;  // mapped pinned word kernels write when a wait expires
  unsigned int *status_dev_ = nullptr;
  // Kernel timing (cfg_.time_kernels): event pairs of launches not yet folded into stats_.
  void time_begin(cudaStream_t s, cudaEvent_t *start);
  void time_end(cudaStream_t s, cudaEvent_t start, uint64_t bytes, bool link, int stamp_idx);
  void fold_timings(bool wait);
  std::deque<TimedLaunch> timed_;
  std::vector<cudaEvent_t> timing_event_pool_;
  // Device-clock stamps written by the gather/scatter kernel itself (first CTA start, last CTA
  // end): up to kStampRing launches per backend are stamped.
  static constexpr int kStampRing = 1 << 16;
  unsigned long long *stamps_dev_ = nullptr;
  std::vector<unsigned long long> stamps_host_;
  size_t stamps_used_ = 0;

  bool tables_aligned_ = true;           // set while an address table is filled
  pf_backend_stats stats_{};
};

void enable_peer_access(int device, int peer);

// Makes `device` current for the calling thread and restores the previous one on scope exit,
// so a call through the C ABI never changes the caller's current device.
class DeviceGuard {
 public:
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev_) != cudaSuccess) prev_ = -1;
    if (prev_ != device) cudaSetDevice(device);
    else prev_ = -1;
  }
  ~DeviceGuard() {
    if (prev_ >= 0) cudaSetDevice(prev_);
  }
  DeviceGuard(const DeviceGuard &) = delete;
  DeviceGuard &operator=(const DeviceGuard &) = delete;

 private:
  int prev_ = -1;
};

}  // namespace pf
