/* CPU oracle for the PegaFlow KV-block save/load path: test infrastructure only, never part
 * of the product.  See pf_oracle.c for the reference citations of each function. */
#ifndef PF_ORACLE_H
#define PF_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct pfo_layout {
  uint64_t data_ptr;
  size_t size_bytes;
  size_t num_blocks;
  size_t block_stride_bytes;
  size_t segment_bytes;
  size_t segments;
  size_t padded_segment_bytes;
  int split;              /* 1: K and V are separate ranges kv_stride_bytes apart */
  size_t kv_stride_bytes; /* meaningful when split */
} pfo_layout;

typedef struct pfo_copy_desc {
  uint64_t device;
  uint64_t host;
  uint64_t host_device;
  size_t size;
  size_t device_allocation;
  size_t host_allocation;
} pfo_copy_desc;

/* Host image of one block for one layer: one or two segments plus a byte offset into them
 * (the offset is non-zero only for page-first storage). */
typedef struct pfo_host_block {
  size_t block_idx;
  size_t n_segments;
  uint64_t seg_host[2];
  uint64_t seg_host_device[2];
  size_t seg_allocation[2];
  size_t host_offset;
} pfo_host_block;

typedef struct pfo_layer_task {
  pfo_layout layout;
  size_t n_blocks;
  const pfo_host_block *blocks;
} pfo_layer_task;

int pfo_layout_new(pfo_layout *out, uint64_t data_ptr, size_t size_bytes, size_t num_blocks, size_t segment_bytes,
                   size_t kv_stride_bytes, size_t segments, char *err, size_t errlen);
int pfo_layout_with_block_stride(pfo_layout *l, size_t stride, char *err, size_t errlen);
void pfo_layout_with_ssd_padding(pfo_layout *l, size_t alignment);
size_t pfo_layout_padded_block_bytes(const pfo_layout *l);
int pfo_layout_block_copies(const pfo_layout *l, size_t block_idx, uint64_t addr[2], size_t bytes[2], char *err,
                            size_t errlen);
int pfo_build_page_layout(const size_t *set_offsets, const size_t *set_items, size_t n_sets, size_t n_layers,
                          const size_t *padded_bytes, size_t *layer_shard, size_t *layer_offsets,
                          size_t *layer_bytes, size_t *shard_page_sizes, size_t *n_shards_out, char *err,
                          size_t errlen);
long pfo_build_copy_descs(const pfo_layer_task *layers, size_t n_layers, pfo_copy_desc *out, size_t out_cap,
                          size_t *total_bytes, char *err, size_t errlen);
size_t pfo_merge(const pfo_copy_desc *in, size_t n, pfo_copy_desc *out);
void pfo_execute(const pfo_copy_desc *d, size_t n, int host_is_src);
double pfo_execute_mt(const pfo_copy_desc *d, size_t n, int host_is_src, int threads);
uint64_t pfo_pool_unit_size(uint64_t pool_size, uint64_t hint);

#ifdef __cplusplus
}
#endif
#endif
