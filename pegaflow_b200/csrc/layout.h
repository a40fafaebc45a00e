// Per-layer KV-cache addressing: one affine formula
//   addr(block, range) = data_ptr + block * block_stride + range * kv_stride
// covers dense, fused-buffer strided, MLA single-segment and K/V-split caches.
// Behaviour follows pegaflow-core/src/layout.rs:43-285; validation happens once, at
// construction, so the copy paths never produce an out-of-bounds range.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "common.h"

namespace pf {

struct DeviceRange {
  uint64_t addr;
  size_t bytes;
};

class KVCacheLayout {
 public:
  KVCacheLayout() = default;
  // Throws std::invalid_argument-like pf::LayoutError (plain message, no prefix) on bad input.
  KVCacheLayout(uint64_t data_ptr, size_t size_bytes, size_t num_blocks, size_t segment_bytes,
                size_t kv_stride_bytes, size_t segments);

  void set_block_stride(size_t stride);        // layout.rs:140-153
  void set_host_alignment(size_t alignment);   // layout.rs:157-160

  // layout.rs:231-255; returns 1 or 2 ranges.
  int block_copies(size_t block_idx, DeviceRange out[2]) const;

  uint64_t data_ptr() const { return data_ptr_; }
  size_t size_bytes() const { return size_bytes_; }
  size_t num_blocks() const { return num_blocks_; }
  size_t block_stride_bytes() const { return block_stride_; }
  size_t segment_bytes() const { return segment_bytes_; }
  size_t segments() const { return segments_; }
  bool is_split() const { return split_; }
  size_t kv_stride_bytes() const { return split_ ? kv_stride_ : 0; }
  size_t block_bytes() const { return segment_bytes_ * segments_; }
  size_t padded_segment_bytes() const { return padded_segment_; }
  size_t padded_block_bytes() const { return padded_segment_ * segments_; }
  // Device ranges per block and their size: (1, block_bytes) or (2, segment_bytes).
  uint32_t n_ranges() const { return split_ ? 2u : 1u; }
  size_t range_bytes() const { return split_ ? segment_bytes_ : block_bytes(); }

  void fill(pf_layout *out) const;

 private:
  void check_bounds() const;
  void check_split_disjoint() const;

  uint64_t data_ptr_ = 0;
  size_t size_bytes_ = 0, num_blocks_ = 0, block_stride_ = 0, segment_bytes_ = 0, segments_ = 0;
  size_t padded_segment_ = 0, kv_stride_ = 0;
  bool split_ = false;
};

// Plain-message error thrown by layout / page-layout validation; callers wrap it into
// Error::invalid("layer <name>: <message>") as the reference does (lib.rs:361-377).
struct LayoutError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// Page-first placement (instance.rs:79-162): a shard is the set of layers one writer holds;
// each shard is one storage slot whose page concatenates its layers in layer-id order.
struct PageLayout {
  std::vector<size_t> layer_shard, layer_offsets, layer_bytes, shard_page_sizes;
};
PageLayout build_page_layout(const std::vector<std::vector<size_t>> &worker_layer_sets, size_t n_layers,
                             const std::vector<size_t> &padded_bytes,
                             const std::vector<std::string> *names = nullptr);

uint64_t pool_unit_size(uint64_t pool_bytes, uint64_t hint);  // pinned_pool.rs:135-141

}  // namespace pf
