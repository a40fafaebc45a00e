// extern "C" surface of the layout arithmetic and the transfer backend (include/pegaflow_b200.h,
// sections 0 and 1).
#include <cuda_runtime.h>

#include <vector>

#include "common.h"
#include "layout.h"
#include "transfer.h"

using namespace pf;

struct pf_backend {
  TransferBackend impl;
  pf_backend(int device, const pf_backend_config *cfg) : impl(device, cfg) {}
};

extern "C" {

int pf_abi_version(void) { return PF_ABI_VERSION; }
const char *pf_last_error(void) { return last_error(); }

int pf_layout_init(pf_layout *out, uint64_t data_ptr, size_t size_bytes, size_t num_blocks, size_t segment_bytes,
                   size_t kv_stride_bytes, size_t segments, size_t block_stride_bytes, size_t host_alignment) {
  return guarded([&] {
    if (!out) throw Error::invalid("out is null");
    try {
      KVCacheLayout l(data_ptr, size_bytes, num_blocks, segment_bytes, kv_stride_bytes, segments);
      if (block_stride_bytes) l.set_block_stride(block_stride_bytes);
      l.set_host_alignment(host_alignment);
      l.fill(out);
    } catch (const LayoutError &e) {
      throw Error::invalid(e.what());
    }
  });
}

int pf_layout_block_copies(const pf_layout *layout, size_t block_idx, uint64_t addr[2], size_t bytes[2],
                           int *n_ranges) {
  return guarded([&] {
    if (!layout || !addr || !bytes || !n_ranges) throw Error::invalid("null argument");
    if (block_idx >= layout->num_blocks)
      throw Error::invalid(strf("block %zu out of range (%zu blocks)", block_idx, layout->num_blocks));
    const uint64_t first = layout->data_ptr + (uint64_t)block_idx * layout->block_stride_bytes;
    addr[0] = first;
    if (layout->split) {
      bytes[0] = bytes[1] = layout->segment_bytes;
      addr[1] = first + layout->kv_stride_bytes;
      *n_ranges = 2;
    } else {
      bytes[0] = layout->segment_bytes * layout->segments;
      *n_ranges = 1;
    }
  });
}

int pf_build_page_layout(const size_t *set_offsets, const size_t *set_items, size_t n_sets, size_t n_layers,
                         const size_t *padded_bytes, size_t *layer_shard, size_t *layer_offsets, size_t *layer_bytes,
                         size_t *shard_page_sizes, size_t *n_shards) {
  return guarded([&] {
    std::vector<std::vector<size_t>> sets(n_sets);
    for (size_t s = 0; s < n_sets; ++s) sets[s].assign(set_items + set_offsets[s], set_items + set_offsets[s + 1]);
    std::vector<size_t> padded(padded_bytes, padded_bytes + n_layers);
    PageLayout p;
    try {
      p = build_page_layout(sets, n_layers, padded);
    } catch (const LayoutError &e) {
      throw Error::invalid(e.what());
    }
    for (size_t l = 0; l < n_layers; ++l) {
      layer_shard[l] = p.layer_shard[l];
      layer_offsets[l] = p.layer_offsets[l];
      layer_bytes[l] = p.layer_bytes[l];
    }
    for (size_t s = 0; s < p.shard_page_sizes.size(); ++s) shard_page_sizes[s] = p.shard_page_sizes[s];
    *n_shards = p.shard_page_sizes.size();
  });
}

uint64_t pf_pool_unit_size(uint64_t pool_bytes, uint64_t hint) { return pool_unit_size(pool_bytes, hint); }

int pf_backend_new(int device_id, const pf_backend_config *config, pf_backend **out) {
  return guarded([&] {
    if (!out) throw Error::invalid("out is null");
    *out = new pf_backend(device_id, config);
  });
}

void pf_backend_free(pf_backend *backend) { delete backend; }

const char *pf_backend_name(const pf_backend *backend) { return backend ? backend->impl.name() : ""; }

int pf_backend_h2d(pf_backend *backend, const pf_copy_desc *copies, size_t n, void *stream) {
  return guarded([&] {
    if (!backend) throw Error::invalid("backend is null");
    backend->impl.copy_descs(copies, n, true, (cudaStream_t)stream);
  });
}

int pf_backend_d2h(pf_backend *backend, const pf_copy_desc *copies, size_t n, void *stream) {
  return guarded([&] {
    if (!backend) throw Error::invalid("backend is null");
    backend->impl.copy_descs(copies, n, false, (cudaStream_t)stream);
  });
}

int pf_backend_save_layers(pf_backend *backend, const pf_layer_xfer *layers, size_t n_layers, void *stream,
                           void *const *layer_done) {
  return guarded([&] {
    if (!backend) throw Error::invalid("backend is null");
    backend->impl.move_layers(layers, n_layers, false, (cudaStream_t)stream, layer_done);
  });
}

int pf_backend_load_layers(pf_backend *backend, const pf_layer_xfer *layers, size_t n_layers, void *stream,
                           void *const *layer_done) {
  return guarded([&] {
    if (!backend) throw Error::invalid("backend is null");
    backend->impl.move_layers(layers, n_layers, true, (cudaStream_t)stream, layer_done);
  });
}

int pf_backend_gather_layers(pf_backend *backend, const pf_layer_xfer *layers, size_t n_layers, void *stream) {
  return guarded([&] {
    if (!backend) throw Error::invalid("backend is null");
    if (!layers && n_layers) throw Error::invalid("layers is null");
    backend->impl.gather_layers(layers, n_layers, (cudaStream_t)stream);
  });
}

int pf_backend_peer_copy(pf_backend *backend, const pf_device_layout *src, const uint32_t *src_ids,
                         const pf_device_layout *dst, const uint32_t *dst_ids, size_t n_blocks, void *stream) {
  return guarded([&] {
    if (!backend || !src || !dst) throw Error::invalid("null argument");
    backend->impl.peer_copy(*src, src_ids, *dst, dst_ids, n_blocks, (cudaStream_t)stream);
  });
}

int pf_backend_peer_copy_layers(pf_backend *backend, const pf_device_layout *src, const pf_device_layout *dst,
                                size_t n_layers, const uint32_t *src_ids, const uint32_t *dst_ids, size_t n_blocks,
                                void *stream) {
  return guarded([&] {
    if (!backend) throw Error::invalid("peer copy: null backend");
    if (n_layers && (!src || !dst)) throw Error::invalid("peer copy: null layout array");
    if (n_blocks && (!src_ids || !dst_ids)) throw Error::invalid("peer copy: null block id array");
    backend->impl.peer_copy_layers(src, dst, n_layers, src_ids, dst_ids, n_blocks, (cudaStream_t)stream);
  });
}

int pf_enable_peer_access(int device_id, int peer_device) {
  return guarded([&] { enable_peer_access(device_id, peer_device); });
}

int pf_backend_get_stats(pf_backend *backend, pf_backend_stats *out) {
  return guarded([&] {
    if (!backend || !out) throw Error::invalid("null argument");
    backend->impl.stats(out);
  });
}

}  // extern "C"
