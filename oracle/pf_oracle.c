/*
 * CPU oracle for the PegaFlow KV-block save/load path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of the
 * reference's transfer path so that the CUDA product can be checked against it.  It is
 * never linked into, imported by, or called from the product library; only the test-suite,
 * the smoke check and the benchmark's CPU-baseline / reference legs use it.
 *
 * Parity pins: the known-answer tests of the reference's own unit tests
 * (pegaflow-core/src/layout.rs:299-474, instance/tests.rs:160-215, transfer/memcpy.rs:124-138,
 * transfer/kernel.rs:205-267) are replayed against these functions by the CPU test-suite.
 *
 * "Device memory" in the oracle is ordinary host memory: a descriptor's `device` field holds
 * the address of a byte buffer that stands in for the GPU KV cache.
 *
 * Each function names the reference file:line it follows.
 */
#define _GNU_SOURCE
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "pf_oracle.h"

static int fail(char *err, size_t errlen, const char *fmt, ...) __attribute__((format(printf, 3, 4)));
#include <stdarg.h>
static int fail(char *err, size_t errlen, const char *fmt, ...) {
  if (err && errlen) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, errlen, fmt, ap);
    va_end(ap);
  }
  return -1;
}

static int mul_ovf(size_t a, size_t b, size_t *out) { return __builtin_mul_overflow(a, b, out); }
static int add_ovf(size_t a, size_t b, size_t *out) { return __builtin_add_overflow(a, b, out); }

static size_t block_bytes(const pfo_layout *l) { return l->segment_bytes * l->segments; }

/* layout.rs:205-225 — a split layout is valid only when the V region cannot alias a K
 * segment of any other block: test the two block distances nearest to kv_stride. */
static int check_split_disjoint(const pfo_layout *l, char *err, size_t errlen) {
  size_t max_dist = l->num_blocks - 1;
  size_t nearest = l->kv_stride_bytes / l->block_stride_bytes;
  size_t cand[2];
  cand[0] = nearest;
  cand[1] = nearest == SIZE_MAX ? SIZE_MAX : nearest + 1;
  for (int k = 0; k < 2; ++k) {
    size_t d = cand[k];
    if (d == 0 || d > max_dist) continue;
    size_t dist_bytes;
    if (mul_ovf(d, l->block_stride_bytes, &dist_bytes)) return fail(err, errlen, "memory layout overflow");
    size_t gap = l->kv_stride_bytes > dist_bytes ? l->kv_stride_bytes - dist_bytes : dist_bytes - l->kv_stride_bytes;
    if (gap < l->segment_bytes)
      return fail(err, errlen, "kv_stride_bytes %zu overlaps blocks %zu apart", l->kv_stride_bytes, d);
  }
  return 0;
}

/* layout.rs:164-203 — every addressed byte must lie inside the registered region. */
static int check_bounds(const pfo_layout *l, char *err, size_t errlen) {
  size_t end, t;
  if (!l->split) {
    size_t bb = block_bytes(l);
    if (l->block_stride_bytes < bb)
      return fail(err, errlen, "block_stride %zu must be >= block_bytes %zu: blocks would overlap",
                  l->block_stride_bytes, bb);
    if (mul_ovf(l->num_blocks - 1, l->block_stride_bytes, &t) || add_ovf(t, bb, &end))
      return fail(err, errlen, "memory layout overflow");
  } else {
    if (l->block_stride_bytes < l->segment_bytes)
      return fail(err, errlen, "block_stride %zu must be >= segment_bytes %zu: blocks would overlap",
                  l->block_stride_bytes, l->segment_bytes);
    if (check_split_disjoint(l, err, errlen)) return -1;
    size_t last_end;
    if (mul_ovf(l->num_blocks - 1, l->block_stride_bytes, &t) || add_ovf(t, l->segment_bytes, &last_end) ||
        add_ovf(l->kv_stride_bytes, last_end, &end))
      return fail(err, errlen, "memory layout overflow");
  }
  if (end > l->size_bytes)
    return fail(err, errlen, "registered memory too small: need %zu bytes, got %zu", end, l->size_bytes);
  return 0;
}

/* layout.rs:73-131 — KVCacheLayout::new. */
int pfo_layout_new(pfo_layout *out, uint64_t data_ptr, size_t size_bytes, size_t num_blocks, size_t segment_bytes,
                   size_t kv_stride_bytes, size_t segments, char *err, size_t errlen) {
  if (data_ptr == 0) return fail(err, errlen, "data_ptr must not be null");
  if (size_bytes == 0) return fail(err, errlen, "size_bytes must be > 0");
  if (segment_bytes == 0 || num_blocks == 0 || segments == 0)
    return fail(err, errlen, "segment_bytes, num_blocks, and segments must be non-zero");
  uint64_t endp;
  if (__builtin_add_overflow(data_ptr, (uint64_t)size_bytes, &endp))
    return fail(err, errlen, "data_ptr + size_bytes overflows the address space");
  size_t bb;
  if (mul_ovf(segment_bytes, segments, &bb)) return fail(err, errlen, "block size overflow");

  int split = 0;
  if (segments == 1) {
    split = 0;
  } else if (kv_stride_bytes == 0) {
    return fail(err, errlen, "kv_stride_bytes must be > 0 when segments > 1");
  } else if (kv_stride_bytes < segment_bytes) {
    return fail(err, errlen, "kv_stride_bytes %zu < segment_bytes %zu: segments would overlap", kv_stride_bytes,
                segment_bytes);
  } else if (kv_stride_bytes == segment_bytes) {
    split = 0;
  } else if (segments == 2) {
    split = 1;
  } else {
    return fail(err, errlen,
                "split layout (kv_stride_bytes %zu > segment_bytes %zu) supports exactly 2 segments, got %zu",
                kv_stride_bytes, segment_bytes, segments);
  }
  memset(out, 0, sizeof *out);
  out->data_ptr = data_ptr;
  out->size_bytes = size_bytes;
  out->num_blocks = num_blocks;
  out->segment_bytes = segment_bytes;
  out->segments = segments;
  out->padded_segment_bytes = segment_bytes;
  out->split = split;
  out->kv_stride_bytes = split ? kv_stride_bytes : 0;
  out->block_stride_bytes = split ? segment_bytes : bb;
  return check_bounds(out, err, errlen);
}

/* layout.rs:140-153 — with_block_stride. */
int pfo_layout_with_block_stride(pfo_layout *l, size_t stride, char *err, size_t errlen) {
  size_t min_stride = l->split ? l->segment_bytes : block_bytes(l);
  if (stride < min_stride)
    return fail(err, errlen, "block_stride %zu must be >= %zu: blocks would overlap", stride, min_stride);
  l->block_stride_bytes = stride;
  return check_bounds(l, err, errlen);
}

/* layout.rs:157-160 — with_ssd_padding: host stride of a segment rounded up. */
void pfo_layout_with_ssd_padding(pfo_layout *l, size_t alignment) {
  l->padded_segment_bytes = (l->segment_bytes + alignment - 1) / alignment * alignment;
}

size_t pfo_layout_padded_block_bytes(const pfo_layout *l) { return l->padded_segment_bytes * l->segments; }

/* layout.rs:231-255 — block_copies: one range (contiguous) or K and V ranges (split). */
int pfo_layout_block_copies(const pfo_layout *l, size_t block_idx, uint64_t addr[2], size_t bytes[2], char *err,
                            size_t errlen) {
  if (block_idx >= l->num_blocks)
    return fail(err, errlen, "block %zu out of range (%zu blocks)", block_idx, l->num_blocks);
  uint64_t base = l->data_ptr + (uint64_t)(block_idx * l->block_stride_bytes);
  if (!l->split) {
    addr[0] = base;
    bytes[0] = block_bytes(l);
    return 1;
  }
  addr[0] = base;
  bytes[0] = l->segment_bytes;
  addr[1] = base + l->kv_stride_bytes;
  bytes[1] = l->segment_bytes;
  return 2;
}

/* instance.rs:107-162 — build_page_layout.  Worker layer-id sets arrive CSR-style:
 * set s owns set_items[set_offsets[s] .. set_offsets[s+1]) (ascending). */
int pfo_build_page_layout(const size_t *set_offsets, const size_t *set_items, size_t n_sets, size_t n_layers,
                          const size_t *padded_bytes, size_t *layer_shard, size_t *layer_offsets,
                          size_t *layer_bytes, size_t *shard_page_sizes, size_t *n_shards_out, char *err,
                          size_t errlen) {
  /* distinct sets, in first-seen order */
  size_t *distinct = malloc((n_sets ? n_sets : 1) * sizeof(size_t));
  size_t nd = 0;
  for (size_t s = 0; s < n_sets; ++s) {
    size_t len = set_offsets[s + 1] - set_offsets[s];
    int seen = 0;
    for (size_t d = 0; d < nd && !seen; ++d) {
      size_t o = distinct[d];
      size_t olen = set_offsets[o + 1] - set_offsets[o];
      if (olen == len && memcmp(set_items + set_offsets[o], set_items + set_offsets[s], len * sizeof(size_t)) == 0)
        seen = 1;
    }
    if (!seen) distinct[nd++] = s;
  }
  /* stable order by minimum layer id (empty set sorts last) */
  for (size_t i = 1; i < nd; ++i) {
    size_t cur = distinct[i];
    size_t curkey = set_offsets[cur + 1] > set_offsets[cur] ? set_items[set_offsets[cur]] : SIZE_MAX;
    size_t j = i;
    while (j > 0) {
      size_t p = distinct[j - 1];
      size_t pkey = set_offsets[p + 1] > set_offsets[p] ? set_items[set_offsets[p]] : SIZE_MAX;
      if (pkey <= curkey) break;
      distinct[j] = p;
      --j;
    }
    distinct[j] = cur;
  }
  for (size_t l = 0; l < n_layers; ++l) layer_shard[l] = SIZE_MAX;
  for (size_t d = 0; d < nd; ++d) {
    size_t s = distinct[d];
    for (size_t k = set_offsets[s]; k < set_offsets[s + 1]; ++k) {
      size_t layer = set_items[k];
      if (layer_shard[layer] != SIZE_MAX) {
        int rc = fail(err, errlen,
                      "page-first layer %zu claimed by shards %zu and %zu: registered layer sets must be "
                      "identical (replica) or disjoint (split)",
                      layer, layer_shard[layer], d);
        free(distinct);
        return rc;
      }
      layer_shard[layer] = d;
    }
  }
  for (size_t l = 0; l < n_layers; ++l) {
    if (layer_shard[l] == SIZE_MAX) {
      free(distinct);
      return fail(err, errlen, "page-first layer %zu has no shard owner after sealing", l);
    }
  }
  for (size_t d = 0; d < nd; ++d) shard_page_sizes[d] = 0;
  for (size_t l = 0; l < n_layers; ++l) {
    size_t sh = layer_shard[l];
    layer_offsets[l] = shard_page_sizes[sh];
    layer_bytes[l] = padded_bytes[l];
    shard_page_sizes[sh] += padded_bytes[l];
  }
  *n_shards_out = nd;
  free(distinct);
  return 0;
}

/* gpu_worker.rs:353-423 — build_copy_descs: one descriptor per GPU range of every block of
 * every layer, in (layer, block, K-then-V) order; a split GPU block whose host image has a
 * single segment places V directly after K. */
long pfo_build_copy_descs(const pfo_layer_task *layers, size_t n_layers, pfo_copy_desc *out, size_t out_cap,
                          size_t *total_bytes, char *err, size_t errlen) {
  size_t n = 0, total = 0;
  for (size_t li = 0; li < n_layers; ++li) {
    const pfo_layer_task *L = &layers[li];
    for (size_t b = 0; b < L->n_blocks; ++b) {
      const pfo_host_block *hb = &L->blocks[b];
      uint64_t addr[2];
      size_t bytes[2];
      int nr = pfo_layout_block_copies(&L->layout, hb->block_idx, addr, bytes, err, errlen);
      if (nr < 0) return -1;
      if (n + (size_t)nr > out_cap) return fail(err, errlen, "descriptor buffer too small");
      if (nr == 2) {
        uint64_t k_host = hb->seg_host[0] + hb->host_offset;
        uint64_t k_dev = hb->seg_host_device[0] + hb->host_offset;
        uint64_t v_host, v_dev;
        size_t v_alloc;
        if (hb->n_segments >= 2) {
          v_host = hb->seg_host[1] + hb->host_offset;
          v_dev = hb->seg_host_device[1] + hb->host_offset;
          v_alloc = hb->seg_allocation[1];
        } else {
          v_host = k_host + bytes[0];
          v_dev = k_dev + bytes[0];
          v_alloc = hb->seg_allocation[0];
        }
        out[n++] = (pfo_copy_desc){addr[0], k_host, k_dev, bytes[0], li, hb->seg_allocation[0]};
        out[n++] = (pfo_copy_desc){addr[1], v_host, v_dev, bytes[1], li, v_alloc};
        total += bytes[0] + bytes[1];
      } else {
        out[n++] = (pfo_copy_desc){addr[0], hb->seg_host[0] + hb->host_offset,
                                   hb->seg_host_device[0] + hb->host_offset, bytes[0], li, hb->seg_allocation[0]};
        total += bytes[0];
      }
    }
  }
  if (total_bytes) *total_bytes = total;
  return (long)n;
}

/* transfer/memcpy.rs:25-55 — merge: join neighbours that are adjacent on BOTH sides and
 * belong to the same device and host allocations. */
size_t pfo_merge(const pfo_copy_desc *in, size_t n, pfo_copy_desc *out) {
  size_t m = 0, i = 0;
  while (i < n) {
    pfo_copy_desc cur = in[i];
    size_t j = i + 1;
    while (j < n) {
      const pfo_copy_desc *nx = &in[j];
      int same = cur.device_allocation == nx->device_allocation && cur.host_allocation == nx->host_allocation;
      if (same && cur.device + cur.size == nx->device && cur.host + cur.size == nx->host) {
        cur.size += nx->size;
        ++j;
      } else {
        break;
      }
    }
    out[m++] = cur;
    i = j;
  }
  return m;
}

/* transfer/kernel.rs:25-46 and transfer/memcpy.rs:61-97 — both backends move exactly `size`
 * bytes per descriptor, nothing else.  host_is_src != 0 is the load direction (h2d). */
void pfo_execute(const pfo_copy_desc *d, size_t n, int host_is_src) {
  for (size_t i = 0; i < n; ++i) {
    if (host_is_src)
      memcpy((void *)(uintptr_t)d[i].device, (const void *)(uintptr_t)d[i].host, d[i].size);
    else
      memcpy((void *)(uintptr_t)d[i].host, (const void *)(uintptr_t)d[i].device, d[i].size);
  }
}

typedef struct {
  const pfo_copy_desc *d;
  size_t begin, end;
  int host_is_src;
} mt_arg;

static void *mt_worker(void *p) {
  mt_arg *a = p;
  pfo_execute(a->d + a->begin, a->end - a->begin, a->host_is_src);
  return NULL;
}

/* Host-core pool packing: the same descriptor batch executed by `threads` host threads
 * (contiguous slices).  Returns elapsed seconds (CLOCK_MONOTONIC). */
double pfo_execute_mt(const pfo_copy_desc *d, size_t n, int host_is_src, int threads) {
  if (threads < 1) threads = 1;
  if ((size_t)threads > n && n > 0) threads = (int)n;
  struct timespec t0, t1;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  if (threads == 1 || n == 0) {
    pfo_execute(d, n, host_is_src);
  } else {
    pthread_t *th = malloc(sizeof(pthread_t) * threads);
    mt_arg *args = malloc(sizeof(mt_arg) * threads);
    for (int t = 0; t < threads; ++t) {
      args[t].d = d;
      args[t].begin = n * (size_t)t / threads;
      args[t].end = n * (size_t)(t + 1) / threads;
      args[t].host_is_src = host_is_src;
      pthread_create(&th[t], NULL, mt_worker, &args[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(th[t], NULL);
    free(th);
    free(args);
  }
  clock_gettime(CLOCK_MONOTONIC, &t1);
  return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}

/* pinned_pool.rs:135-141 — allocator unit: at least the hint (default 512), large enough that
 * the pool fits in 2^32-1 units, rounded up to a multiple of 512. */
uint64_t pfo_pool_unit_size(uint64_t pool_size, uint64_t hint) {
  const uint64_t align = 512, max_units = 0xFFFFFFFFull;
  uint64_t min_unit = (pool_size + max_units - 1) / max_units;
  uint64_t base = hint ? hint : align;
  uint64_t unit = base > min_unit ? base : min_unit;
  return (unit + align - 1) / align * align;
}
