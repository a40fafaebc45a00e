#include "layout.h"

#include <algorithm>
#include <cstring>
#include <mutex>
#include <set>

namespace pf {

std::string strf(const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  return std::string(buf);
}

static thread_local std::string g_last_error;
void set_last_error(const std::string &msg) { g_last_error = msg; }
const char *last_error() { return g_last_error.c_str(); }

namespace {
bool mul_overflows(size_t a, size_t b, size_t *out) { return __builtin_mul_overflow(a, b, out); }
bool add_overflows(size_t a, size_t b, size_t *out) { return __builtin_add_overflow(a, b, out); }
}  // namespace

KVCacheLayout::KVCacheLayout(uint64_t data_ptr, size_t size_bytes, size_t num_blocks, size_t segment_bytes,
                             size_t kv_stride_bytes, size_t segments) {
  if (data_ptr == 0) throw LayoutError("data_ptr must not be null");
  if (size_bytes == 0) throw LayoutError("size_bytes must be > 0");
  if (segment_bytes == 0 || num_blocks == 0 || segments == 0)
    throw LayoutError("segment_bytes, num_blocks, and segments must be non-zero");
  uint64_t end_ptr;
  if (__builtin_add_overflow(data_ptr, (uint64_t)size_bytes, &end_ptr))
    throw LayoutError("data_ptr + size_bytes overflows the address space");
  size_t block_bytes;
  if (mul_overflows(segment_bytes, segments, &block_bytes)) throw LayoutError("block size overflow");

  // Which shape is it: one range per block, or K and V kv_stride apart?
  if (segments > 1) {
    if (kv_stride_bytes == 0) throw LayoutError("kv_stride_bytes must be > 0 when segments > 1");
    if (kv_stride_bytes < segment_bytes)
      throw LayoutError(strf("kv_stride_bytes %zu < segment_bytes %zu: segments would overlap", kv_stride_bytes,
                             segment_bytes));
    if (kv_stride_bytes > segment_bytes) {
      if (segments != 2)
        throw LayoutError(strf("split layout (kv_stride_bytes %zu > segment_bytes %zu) supports exactly 2 "
                               "segments, got %zu",
                               kv_stride_bytes, segment_bytes, segments));
      split_ = true;
    }
  }
  data_ptr_ = data_ptr;
  size_bytes_ = size_bytes;
  num_blocks_ = num_blocks;
  segment_bytes_ = segment_bytes;
  segments_ = segments;
  padded_segment_ = segment_bytes;
  kv_stride_ = split_ ? kv_stride_bytes : 0;
  block_stride_ = split_ ? segment_bytes : block_bytes;
  check_bounds();
}

void KVCacheLayout::set_block_stride(size_t stride) {
  size_t min_stride = split_ ? segment_bytes_ : block_bytes();
  if (stride < min_stride)
    throw LayoutError(strf("block_stride %zu must be >= %zu: blocks would overlap", stride, min_stride));
  block_stride_ = stride;
  check_bounds();
}

void KVCacheLayout::set_host_alignment(size_t alignment) {
  if (alignment > 1) padded_segment_ = (segment_bytes_ + alignment - 1) / alignment * alignment;
}

void KVCacheLayout::check_split_disjoint() const {
  // The V region starts kv_stride after K.  It may only alias a K segment of a block whose
  // distance (in strides) brackets kv_stride, so two candidates are enough.
  const size_t farthest = num_blocks_ - 1;
  const size_t below = kv_stride_ / block_stride_;
  for (int k = 0; k < 2; ++k) {
    size_t dist = below + (size_t)k;
    if (dist < below) dist = SIZE_MAX;  // saturate
    if (dist == 0 || dist > farthest) continue;
    size_t dist_bytes;
    if (mul_overflows(dist, block_stride_, &dist_bytes)) throw LayoutError("memory layout overflow");
    size_t gap = kv_stride_ > dist_bytes ? kv_stride_ - dist_bytes : dist_bytes - kv_stride_;
    if (gap < segment_bytes_)
      throw LayoutError(strf("kv_stride_bytes %zu overlaps blocks %zu apart", kv_stride_, dist));
  }
}

void KVCacheLayout::check_bounds() const {
  size_t span, tmp;
  if (!split_) {
    const size_t bb = block_bytes();
    if (block_stride_ < bb)
      throw LayoutError(strf("block_stride %zu must be >= block_bytes %zu: blocks would overlap", block_stride_, bb));
    if (mul_overflows(num_blocks_ - 1, block_stride_, &tmp) || add_overflows(tmp, bb, &span))
      throw LayoutError("memory layout overflow");
  } else {
    if (block_stride_ < segment_bytes_)
      throw LayoutError(strf("block_stride %zu must be >= segment_bytes %zu: blocks would overlap", block_stride_,
                             segment_bytes_));
    check_split_disjoint();
    size_t k_span;
    if (mul_overflows(num_blocks_ - 1, block_stride_, &tmp) || add_overflows(tmp, segment_bytes_, &k_span) ||
        add_overflows(kv_stride_, k_span, &span))
      throw LayoutError("memory layout overflow");
  }
  if (span > size_bytes_)
    throw LayoutError(strf("registered memory too small: need %zu bytes, got %zu", span, size_bytes_));
}

int KVCacheLayout::block_copies(size_t block_idx, DeviceRange out[2]) const {
  if (block_idx >= num_blocks_)
    throw LayoutError(strf("block %zu out of range (%zu blocks)", block_idx, num_blocks_));
  const uint64_t first = data_ptr_ + (uint64_t)block_idx * block_stride_;
  if (!split_) {
    out[0] = {first, block_bytes()};
    return 1;
  }
  out[0] = {first, segment_bytes_};
  out[1] = {first + kv_stride_, segment_bytes_};
  return 2;
}

void KVCacheLayout::fill(pf_layout *out) const {
  out->data_ptr = data_ptr_;
  out->size_bytes = size_bytes_;
  out->num_blocks = num_blocks_;
  out->block_stride_bytes = block_stride_;
  out->segment_bytes = segment_bytes_;
  out->segments = segments_;
  out->padded_segment_bytes = padded_segment_;
  out->split = split_ ? 1 : 0;
  out->kv_stride_bytes = kv_stride_;
}

PageLayout build_page_layout(const std::vector<std::vector<size_t>> &worker_layer_sets, size_t n_layers,
                             const std::vector<size_t> &padded_bytes, const std::vector<std::string> *names) {
  auto label = [&](size_t layer) { return names ? (*names)[layer] : std::to_string(layer); };
  // Identical sets are replicas of one shard; order shards by their smallest layer id.
  std::vector<std::set<size_t>> shards;
  for (const auto &raw : worker_layer_sets) {
    std::set<size_t> s(raw.begin(), raw.end());
    if (std::find(shards.begin(), shards.end(), s) == shards.end()) shards.push_back(std::move(s));
  }
  std::stable_sort(shards.begin(), shards.end(), [](const std::set<size_t> &a, const std::set<size_t> &b) {
    size_t ka = a.empty() ? SIZE_MAX : *a.begin(), kb = b.empty() ? SIZE_MAX : *b.begin();
    return ka < kb;
  });
  PageLayout p;
  p.layer_shard.assign(n_layers, SIZE_MAX);
  for (size_t sid = 0; sid < shards.size(); ++sid) {
    for (size_t layer : shards[sid]) {
      if (layer >= n_layers) throw LayoutError(strf("page-first layer id %zu out of range", layer));
      if (p.layer_shard[layer] != SIZE_MAX)
        throw LayoutError(strf("page-first layer %s claimed by shards %zu and %zu: registered layer sets must be "
                               "identical (replica) or disjoint (split)",
                               label(layer).c_str(), p.layer_shard[layer], sid));
      p.layer_shard[layer] = sid;
    }
  }
  for (size_t layer = 0; layer < n_layers; ++layer)
    if (p.layer_shard[layer] == SIZE_MAX)
      throw LayoutError(strf("page-first layer %s has no shard owner after sealing", label(layer).c_str()));
  p.layer_offsets.assign(n_layers, 0);
  p.layer_bytes.assign(n_layers, 0);
  p.shard_page_sizes.assign(shards.size(), 0);
  for (size_t layer = 0; layer < n_layers; ++layer) {
    size_t &page = p.shard_page_sizes[p.layer_shard[layer]];
    p.layer_offsets[layer] = page;
    p.layer_bytes[layer] = padded_bytes[layer];
    page += padded_bytes[layer];
  }
  return p;
}

uint64_t pool_unit_size(uint64_t pool_bytes, uint64_t hint) {
  const uint64_t kAlign = 512, kMaxUnits = 0xFFFFFFFFull;
  uint64_t floor_unit = (pool_bytes + kMaxUnits - 1) / kMaxUnits;
  uint64_t unit = std::max<uint64_t>(hint ? hint : kAlign, floor_unit);
  return (unit + kAlign - 1) / kAlign * kAlign;
}

}  // namespace pf
