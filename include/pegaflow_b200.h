/*
 * pegaflow_b200 — C ABI of the B200-native KV-cache save/load path.
 *
 * The library is a drop-in for one path of PegaFlow: moving paged KV-cache blocks between GPU
 * memory and a pinned host pool (and between two GPUs of one box).  Three nested boundaries are
 * exported, innermost first; each entry point names the reference interface it replaces
 * (paths are relative to the reference repository).
 *
 *   1. backend  — a batch of copies enqueued on a caller's CUDA stream
 *                 (pegaflow-core/src/transfer/mod.rs:36-60, `CopyDesc` / `trait TransferBackend`)
 *   2. engine   — registration, save, prefix query, lease, load
 *                 (pegaflow-core/src/lib.rs, offload.rs: `PegaEngine`)
 *   3. LoadState — the shared-memory completion word a vLLM worker polls
 *                 (pegaflow-core/src/sync_state.rs)
 *
 * Conventions: every function returns a status (0 = ok) unless stated; on failure a
 * thread-local message is available from pf_last_error().  Status values 1..7 are the
 * reference's `EngineError` variants in declaration order (pegaflow-core/src/lib.rs:72-87).
 * No function takes or returns a torch type; `stream` / `event` arguments are `cudaStream_t` /
 * `cudaEvent_t` passed as `void*`.  There is no CPU fallback: without a CUDA device every call
 * that would move bytes fails with PF_CUDA_INIT.
 */
#ifndef PEGAFLOW_B200_H
#define PEGAFLOW_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PF_ABI_VERSION 1

enum pf_status {
  PF_OK = 0,
  PF_INSTANCE_MISSING = 1,  /* EngineError::InstanceMissing   */
  PF_WORKER_MISSING = 2,    /* EngineError::WorkerMissing     */
  PF_INVALID_ARGUMENT = 3,  /* EngineError::InvalidArgument   */
  PF_CUDA_INIT = 4,         /* EngineError::CudaInit          */
  PF_STORAGE = 5,           /* EngineError::Storage           */
  PF_POISONED = 6,          /* EngineError::Poisoned          */
  PF_TOPOLOGY_MISMATCH = 7  /* EngineError::TopologyMismatch  */
};

int pf_abi_version(void);
/* Message of the last failure on the calling thread ("" when none).  Text follows the
 * reference's Display strings, e.g. "invalid argument: layer l0: data_ptr must not be null". */
const char *pf_last_error(void);

/* ------------------------------------------------------------------------------------------
 * 0. Layout arithmetic (pure host code, usable without a GPU).
 *    Replaces `KVCacheLayout` (pegaflow-core/src/layout.rs:43-285).
 * ---------------------------------------------------------------------------------------- */
typedef struct pf_layout {
  uint64_t data_ptr;
  size_t size_bytes;
  size_t num_blocks;
  size_t block_stride_bytes;
  size_t segment_bytes;        /* one of K or V */
  size_t segments;             /* 1 or 2 */
  size_t padded_segment_bytes; /* host-side stride of a segment */
  int split;                   /* K and V are separate device ranges */
  size_t kv_stride_bytes;      /* distance K -> V when split */
} pf_layout;

/* layout.rs:73-131 `KVCacheLayout::new`; block_stride_bytes == 0 keeps the dense default,
 * otherwise layout.rs:140-153 `with_block_stride`; host_alignment > 1 applies
 * layout.rs:157-160 `with_ssd_padding`. */
int pf_layout_init(pf_layout *out, uint64_t data_ptr, size_t size_bytes, size_t num_blocks,
                   size_t segment_bytes, size_t kv_stride_bytes, size_t segments,
                   size_t block_stride_bytes, size_t host_alignment);
/* layout.rs:231-255 `block_copies`: writes 1 or 2 (addr, bytes) pairs, returns their count in
 * *n_ranges. */
int pf_layout_block_copies(const pf_layout *layout, size_t block_idx, uint64_t addr[2],
                           size_t bytes[2], int *n_ranges);
/* instance.rs:107-162 `build_page_layout`.  Worker w registered the layer ids
 * set_items[set_offsets[w] .. set_offsets[w+1]).  Outputs have n_layers entries, except
 * shard_page_sizes (n_sets entries, *n_shards used). */
int pf_build_page_layout(const size_t *set_offsets, const size_t *set_items, size_t n_sets,
                         size_t n_layers, const size_t *padded_bytes, size_t *layer_shard,
                         size_t *layer_offsets, size_t *layer_bytes, size_t *shard_page_sizes,
                         size_t *n_shards);
/* pinned_pool.rs:135-141 `compute_unit_size` (hint 0 = none). */
uint64_t pf_pool_unit_size(uint64_t pool_bytes, uint64_t hint);

/* ------------------------------------------------------------------------------------------
 * 1. Backend boundary.
 * ---------------------------------------------------------------------------------------- */

/* transfer/mod.rs:36-44 `CopyDesc`. */
typedef struct pf_copy_desc {
  uint64_t device;          /* absolute device address */
  void *host;               /* host virtual address of the pinned bytes */
  uint64_t host_device;     /* device-visible address of the same bytes (mapped pinned memory) */
  size_t size;
  size_t device_allocation; /* ids used only to decide which neighbours may be coalesced */
  size_t host_allocation;
} pf_copy_desc;

typedef struct pf_backend pf_backend;

enum pf_route {
  PF_ROUTE_AUTO = 0,     /* staged DMA for host-regular runs >= min_dma_bytes, zero-copy otherwise */
  PF_ROUTE_STAGED = 1,   /* always gather/scatter through the HBM staging ring + copy engine */
  PF_ROUTE_ZEROCOPY = 2  /* always the zero-copy kernel over mapped pinned memory */
};

typedef struct pf_backend_config {
  size_t staging_slot_bytes; /* bytes per HBM staging slot (0 = 32 MiB) */
  int staging_slots;         /* ring depth (0 = 6) */
  int pack_ctas;             /* CTAs of the HBM gather/scatter kernel (0 = 8 per SM) */
  int link_ctas;             /* CTAs of the zero-copy / peer kernel (0 = 16 for PCIe, 8 per SM for NVLink) */
  size_t min_dma_bytes;      /* smallest host-contiguous run sent through the copy engine (0 = 256 KiB) */
  int route;                 /* enum pf_route */
  int time_kernels;          /* 1: bracket every kernel launch with CUDA events (see pf_backend_stats) */
  int copy_streams;          /* copy-engine streams the staged route alternates between (0 = 1) */
  int gather_slots;          /* staging slots one gather launch of a save may fill (0 = 3, at most half the ring;
                                1 = one launch per slot) */
} pf_backend_config;

/* Replaces `KernelBackend::new` (transfer/kernel.rs:63-77) / `build_backend`
 * (gpu_worker.rs:264-276).  One backend per worker thread; calls on one backend are serial. */
int pf_backend_new(int device_id, const pf_backend_config *config, pf_backend **out);
void pf_backend_free(pf_backend *backend);
/* `TransferBackend::name` (transfer/mod.rs:59). */
const char *pf_backend_name(const pf_backend *backend);
/* `TransferBackend::h2d` / `d2h` (transfer/mod.rs:53-58): enqueue only, never synchronise.
 * The caller keeps every address valid until it has synchronised `stream`. */
int pf_backend_h2d(pf_backend *backend, const pf_copy_desc *copies, size_t n, void *stream);
int pf_backend_d2h(pf_backend *backend, const pf_copy_desc *copies, size_t n, void *stream);

/* Descriptor-free, layer-wise form of the same boundary.  It carries what
 * `build_copy_descs` (gpu_worker.rs:353-423) would expand: the layer's affine device layout,
 * the block ids, and where the blocks' host images lie.  The host side of range r (0 = K or
 * the whole block, 1 = V) is a list of runs; run j covers blocks
 * [first_block, first_block + n_blocks) of `block_ids`, block first_block + i living at
 * host + i * stride_bytes. */
typedef struct pf_host_run {
  size_t first_block;
  size_t n_blocks;
  void *host;
  uint64_t host_device;
  size_t stride_bytes;
} pf_host_run;

typedef struct pf_layer_xfer {
  uint64_t data_ptr;         /* layout.rs: data_ptr */
  size_t block_stride_bytes; /* layout.rs: block_stride_bytes */
  size_t kv_stride_bytes;    /* distance range 0 -> range 1 on the device (0 when n_ranges == 1) */
  size_t range_bytes;        /* bytes of one device range: block bytes, or segment bytes when split */
  uint32_t n_ranges;         /* 1 or 2 */
  size_t n_blocks;
  const uint32_t *block_ids; /* GPU block index of each moved block */
  size_t n_runs[2];
  const pf_host_run *runs[2];
} pf_layer_xfer;

/* Save (device -> host) / load (host -> device) of whole layers, in order.  When
 * `layer_done` is non-NULL it holds one cudaEvent_t per layer (entries may be NULL); event i
 * is recorded when layer i's bytes have landed, so layer i+1 moves while layer i is consumed.
 * Replaces `process_save_task` / `process_load_task` minus their single trailing
 * synchronisation (gpu_worker.rs:428-523). */
int pf_backend_save_layers(pf_backend *backend, const pf_layer_xfer *layers, size_t n_layers,
                           void *stream, void *const *layer_done);
int pf_backend_load_layers(pf_backend *backend, const pf_layer_xfer *layers, size_t n_layers,
                           void *stream, void *const *layer_done);
/* Measurement aid without a counterpart in the reference: the device half of a staged save on
 * its own.  The gather kernels pack the blocks into the backend's HBM staging ring exactly as
 * pf_backend_save_layers would, but no DMA leaves the ring and nothing reaches the host, so the
 * kernel can be timed back to back (bench.py's roofline figure).  Every run must be one the
 * staged route gathers (scattered block ids, at least `min_dma_bytes`, a block no larger than a
 * staging slot); anything else is PF_INVALID_ARGUMENT.  Synchronise `stream` before the next
 * real transfer on this backend. */
int pf_backend_gather_layers(pf_backend *backend, const pf_layer_xfer *layers, size_t n_layers, void *stream);

/* GPU -> GPU block copy over NVLink for same-box prefix hits: block src_ids[i] of the source
 * layout (memory of a peer GPU, reachable from this backend's device) lands in block
 * dst_ids[i] of the destination layout.  Has no counterpart in the reference, whose
 * cross-instance sharing goes through the host pool. */
typedef struct pf_device_layout {
  uint64_t data_ptr;
  size_t block_stride_bytes;
  size_t kv_stride_bytes;
  size_t range_bytes;
  uint32_t n_ranges;
  size_t num_blocks; /* blocks in the cache; when non-zero every block id is checked against it
                        before anything is launched, 0 = the caller vouches for the ids */
} pf_device_layout;
int pf_backend_peer_copy(pf_backend *backend, const pf_device_layout *src, const uint32_t *src_ids,
                         const pf_device_layout *dst, const uint32_t *dst_ids, size_t n_blocks,
                         void *stream);
/* The same for `n_layers` layers that share the block ids (a whole model's prefix hit): the ids
 * are uploaded once and up to 96 (layer, range) units of equal block size go into one launch. */
int pf_backend_peer_copy_layers(pf_backend *backend, const pf_device_layout *src, const pf_device_layout *dst,
                                size_t n_layers, const uint32_t *src_ids, const uint32_t *dst_ids,
                                size_t n_blocks, void *stream);
/* Cross-process registration (python/pegaflow/ipc_wrapper.py:101-163 + pegaflow-server/src/registry.rs:172-203):
 * the process that owns a KV-cache tensor exports the region, the process that runs the engine
 * opens it and registers the returned pointer.  The region travels as these 96 plain bytes.
 * Devices are matched by UUID, so the two processes may number their GPUs differently.  A region
 * cannot be opened by the process that exported it (a CUDA IPC rule).  Mappings are shared: regions
 * of one allocation open it once; pf_ipc_close drops one use. */
typedef struct pf_ipc_region {
  uint8_t handle[64];      /* cudaIpcMemHandle_t of the allocation that contains the region */
  uint64_t offset;         /* of the region inside that allocation */
  uint64_t nbytes;
  uint8_t device_uuid[16];
} pf_ipc_region;
int pf_ipc_export(uint64_t device_ptr, size_t nbytes, pf_ipc_region *out);
int pf_ipc_open(const pf_ipc_region *region, uint64_t *device_ptr, int *device_id);
int pf_ipc_close(const pf_ipc_region *region);
/* The same for a reader on another GPU: another instance's KV cache, opened so that kernels and
 * copies of `accessing_device` can read it over NVLink (the source side of pf_backend_peer_copy_layers
 * when the two instances are different processes).  The driver binds an imported allocation to the
 * device that was current when it was opened, so the pointer pf_ipc_open returns (opened on the owning
 * GPU, for an engine that works on that GPU) is not usable from a peer device; this one is, and only
 * from `accessing_device`.  *owner_device receives the GPU the memory lives on.  Has no counterpart
 * in the reference, which has no GPU-to-GPU path. */
int pf_ipc_open_for(const pf_ipc_region *region, int accessing_device, uint64_t *device_ptr, int *owner_device);
int pf_ipc_close_for(const pf_ipc_region *region, int accessing_device);

/* Make `peer_device`'s memory addressable from `device_id` (cudaDeviceEnablePeerAccess). */
int pf_enable_peer_access(int device_id, int peer_device);

/* Allocation-free save of a small batch of blocks.  It has no counterpart in the reference.
 *
 * Meant for callers that cannot allocate device memory when they need blocks copied out: a
 * serving process whose free HBM has all gone to the KV cache, a thread that cannot afford the
 * device-wide synchronisation of cudaMalloc/cudaFree, or code running while a stream is being
 * captured elsewhere in the process.  Blocks block_ids[0..n_blocks) of `layout` (memory of
 * `device_id`) are gathered into a staging area that is part of the library image and copied to
 * host_dst: range 0 of every block back to back, then range 1 of every block (the image
 * pf_backend_save_layers writes for one dense host run per range).  The work is enqueued on
 * `stream` and the call does not wait for it.  It is fully asynchronous only when both
 * `block_ids` and `host_dst` are page-locked: from ordinary pageable memory the runtime stages
 * the id upload itself and may hold the call until earlier work on the stream has finished.
 * With layout->num_blocks set, an id outside the cache is PF_INVALID_ARGUMENT and nothing is
 * launched; with 0 the ids are not checked and an id outside the cache reads outside it.
 *
 * No cudaMalloc, cudaFree, stream, event or other allocating call is made.  Limits: at most
 * PF_NOALLOC_MAX_BLOCKS blocks and PF_NOALLOC_MAX_PAYLOAD_BYTES bytes per call, otherwise
 * PF_INVALID_ARGUMENT.  The staging area (PF_NOALLOC_MAX_PAYLOAD_BYTES plus 4 bytes per block
 * id) is static device memory: each GPU that loads the library holds it until the process
 * ends.  The first call on a device (an empty batch counts) looks the area's address up
 * (cudaGetSymbolAddress with that device current), so make that first call before any stream
 * capture starts.  All calls
 * on one device share the area and it keeps the previous call's bytes; nothing in it needs
 * clearing between calls, but two calls whose GPU work overlaps (different streams) race. */
#define PF_NOALLOC_MAX_PAYLOAD_BYTES (8u << 20)
#define PF_NOALLOC_MAX_BLOCKS 16384
int pf_save_blocks_noalloc(int device_id, const pf_device_layout *layout, const uint32_t *block_ids,
                           size_t n_blocks, void *host_dst, size_t host_dst_bytes, void *stream);

/* Counters of one backend since creation (what was launched, which route bytes took). */
typedef struct pf_backend_stats {
  uint64_t kernel_launches;
  uint64_t dma_copies;
  uint64_t bytes_staged;
  uint64_t bytes_zero_copy;
  uint64_t bytes_peer;
  uint32_t device_status; /* 0, or the code a kernel wrote when a bounded wait expired */
  /* Filled when time_kernels is set; only launches that have finished are counted.
   * "pack" = the HBM gather/scatter kernel of the staged route (bytes = read + written),
   * "link" = the zero-copy / peer kernel (bytes = payload). */
  double pack_kernel_ms;
  uint64_t pack_kernel_launches;
  uint64_t pack_kernel_bytes;
  double link_kernel_ms;
  uint64_t link_kernel_launches;
  uint64_t link_kernel_bytes;
  /* The gather/scatter kernel's own clock (%globaltimer, first CTA start to last CTA end) for the
   * first 65536 timed launches: an event pair around a ~10 us kernel measures mostly the pair. */
  double pack_kernel_device_ms;
  uint64_t pack_kernel_device_launches;
} pf_backend_stats;
int pf_backend_get_stats(pf_backend *backend, pf_backend_stats *out);

/* ------------------------------------------------------------------------------------------
 * 2. Pinned host pool.  Replaces `PinnedAllocator` (pinned_pool.rs:616-715) and
 *    `PinnedMemory` (pinned_mem.rs:149-301).
 * ---------------------------------------------------------------------------------------- */
typedef struct pf_pool pf_pool;
typedef struct pf_pool_config {
  int use_hugepages;      /* mmap(MAP_HUGETLB) + pre-touch + cudaHostRegister */
  int use_mmap;           /* mmap + NUMA pre-touch + cudaHostRegister instead of cudaHostAlloc */
  int numa_node;          /* first-touch node for the mmap strategies; -1 = caller's affinity */
  uint64_t unit_hint;     /* allocator granularity hint (0 = 512 B) */
  int shards;             /* independent allocators (0/1 = one) */
  int transparent_huge;   /* with use_mmap: madvise(MADV_HUGEPAGE) before the pre-touch, so that a kernel with
                             transparent huge pages in "madvise" or "always" mode backs the pool with 2 MiB pages */
} pf_pool_config;
int pf_pool_new(size_t bytes, const pf_pool_config *config, pf_pool **out);
void pf_pool_free(pf_pool *pool);
/* pinned_pool.rs:228-275 `allocate`: returns PF_STORAGE when the pool cannot satisfy it. */
int pf_pool_alloc(pf_pool *pool, size_t bytes, void **host, uint64_t *host_device, uint64_t *handle);
int pf_pool_release(pf_pool *pool, uint64_t handle);
/* pinned_pool.rs:293-299 `usage`. */
int pf_pool_usage(pf_pool *pool, uint64_t *used, uint64_t *total, uint64_t *largest_free);

/* pinned_mem.rs:378-391 `touch_threads`: workers that pre-touch an mmap-backed pool of `bytes`
 * bytes (one per GiB, rounded up, at most the CPUs the process may run on); and the kernel's
 * huge page size in bytes from /proc/meminfo, 0 when unknown (`read_hugepage_size_from_proc`). */
size_t pf_pool_pre_touch_threads(size_t bytes);
size_t pf_huge_page_size(void);

/* NUMA helpers (pegaflow-common/src/numa.rs).  Node ids are plain ints, -1 = unknown
 * (`NumaNode::UNKNOWN`).  The topology is read from sysfs; the tree's root is /sys unless the
 * environment variable PEGAFLOW_SYSFS_ROOT or pf_numa_set_sysfs_root names another one (NULL or
 * "" restores /sys) - for containers that mount it elsewhere and for tests. */
int pf_numa_set_sysfs_root(const char *root);
/* numa.rs:344-411 `NumaTopology::numa_for_gpu` / `num_nodes`. */
int pf_numa_node_of_device(int device_id);
int pf_numa_num_nodes(void);
/* numa.rs:129-168 `parse_cpulist`: "0-2,8,16-17" -> 0,1,2,8,16,17 (sorted, each once).  *n is
 * always the number of CPUs; PF_INVALID_ARGUMENT for malformed text or when they do not fit. */
int pf_numa_parse_cpulist(const char *text, int *cpus_out, size_t capacity, size_t *n);
/* numa.rs:88-126 `read_cpu_topology_from_sysfs`, one node: empty when the node is unknown. */
int pf_numa_cpus_of_node(int node, int *cpus_out, size_t capacity, size_t *n);
/* numa.rs:178-218 `pin_thread_to_numa_node`: restricts the calling thread to the node's CPUs;
 * PF_INVALID_ARGUMENT with the reference's message ("Cannot pin to unknown NUMA node", "No CPUs
 * found for NUMA node N", ...) otherwise. */
int pf_numa_pin_thread_to_node(int node);
/* Node of a PCI device ("0000:1b:00.0") from <root>/bus/pci/devices/<id>/numa_node; the
 * reference asks the driver's tool instead (numa.rs:266-291), whose answer this parses
 * (numa.rs:293-302 `parse_closest_cpu_numa_node`: the first id listed). */
int pf_numa_node_of_pci_device(const char *bus_id);
int pf_numa_parse_closest_cpu_node(const char *text);
/* numa.rs:392-402 `gpu_numa_nodes`: the known entries of a device -> node list, sorted, each
 * once.  nodes_out needs room for n_devices entries. */
int pf_numa_distinct_valid_nodes(const int *device_nodes, size_t n_devices, int *nodes_out, size_t *n);
/* numa.rs:441-497 `query_pages_numa`: node on which the page of each address lives (-1 when it
 * is not resident or the query fails). */
int pf_numa_query_pages(const void *const *addrs, size_t n, int *nodes_out);

/* ------------------------------------------------------------------------------------------
 * 3. Engine boundary.  Replaces `PegaEngine` (pegaflow-core/src/lib.rs:113-126).
 * ---------------------------------------------------------------------------------------- */
typedef struct pf_engine pf_engine;
typedef struct pf_block pf_block; /* a sealed, fully saved block (`Arc<SealedBlock>`) */

/* `StorageConfig` (storage/mod.rs:43-92), fields on the transfer path only. */
typedef struct pf_storage_config {
  int enable_numa_affinity;     /* per-NUMA-node pools, workers pinned to the GPU's node */
  int blockwise_alloc;          /* one pool allocation per block instead of per layer batch */
  uint64_t hint_value_size;     /* allocator unit hint (0 = none) */
  int pool_shards;              /* allocator shards (0/1 = one) */
  size_t host_alignment;        /* pad host segment strides to this many bytes (0/1 = none; the
                                   reference pads to 512 when its SSD tier is on, lib.rs:379-388) */
  int use_mmap_pool;            /* pool backing: 0 cudaHostAlloc, 1 mmap+register */
  pf_backend_config backend;    /* transfer tuning; zero-initialised = defaults */
} pf_storage_config;

/* lib.rs:138-142 `PegaEngine::new_with_config`. */
int pf_engine_new(size_t pool_bytes, int use_hugepages, const pf_storage_config *config, pf_engine **out);
void pf_engine_free(pf_engine *engine);

enum pf_transfer_mode { PF_TRANSFER_DIRECT = 0, PF_TRANSFER_KERNEL = 1 }; /* transfer/mod.rs:66-76 */

/* lib.rs:302-322 `register_context_layer_batch_strided`; argument order and meaning are the
 * reference's.  block_stride_bytes and layer_group_ids may be NULL. */
int pf_engine_register_context_layer_batch_strided(
    pf_engine *engine, const char *instance_id, const char *namespace_, int device_id, size_t tp_rank,
    size_t pp_rank, size_t tp_size, size_t world_size, size_t n_layers, const char *const *layer_names,
    const uint64_t *data_ptrs, const size_t *size_bytes, const size_t *num_blocks,
    const size_t *bytes_per_block, const size_t *kv_stride_bytes, const size_t *segments,
    const size_t *block_stride_bytes, const uint32_t *layer_group_ids, int transfer_mode, int page_first);
/* lib.rs:443-460 `unregister_instance`. */
int pf_engine_unregister_instance(pf_engine *engine, const char *instance_id);
/* lib.rs:459-489 `unregister_all_instances`, `list_instance_ids`, `instance_namespace`.  Text results
 * are written NUL-terminated into buf when cap suffices (an empty string otherwise); *needed is the
 * size that does, terminator included.  Instance ids come one per line, sorted; the first of the
 * three returns the ids it removed. */
int pf_engine_unregister_all_instances(pf_engine *engine, char *buf, size_t cap, size_t *needed);
int pf_engine_list_instances(pf_engine *engine, char *buf, size_t cap, size_t *needed);
int pf_engine_instance_namespace(pf_engine *engine, const char *instance_id, char *buf, size_t cap, size_t *needed);

/* block.rs:22-26 `LayerSave`: hashes are passed as one byte string per block. */
typedef struct pf_layer_save {
  const char *layer_name;
  size_t n_blocks;
  const size_t *block_ids;
  const uint8_t *const *block_hashes;
  const size_t *block_hash_lens;
} pf_layer_save;
/* offload.rs:293-300 `batch_save_kv_blocks_from_ipc` (blocks until the bytes are in the pool). */
int pf_engine_batch_save(pf_engine *engine, const char *instance_id, size_t tp_rank, size_t pp_rank,
                         int device_id, size_t n_layers, const pf_layer_save *saves);
/* lib.rs:903 `flush_saves`. */
int pf_engine_flush_saves(pf_engine *engine);

/* lib.rs:506-533 `count_prefix_hit_blocks_with_prefetch` (always terminal: there is no SSD
 * tier to wait for).  Writes up to `n` owned block handles into blocks_out and their count
 * into *n_hit; *n_missing = n - *n_hit.  Release each handle with pf_block_release. */
int pf_engine_query_prefix(pf_engine *engine, const char *instance_id, const char *req_id, size_t n,
                           const uint8_t *const *hashes, const size_t *hash_lens, pf_block **blocks_out,
                           size_t *n_hit, size_t *n_missing);
/* lib.rs:592-612 `query_group_membership`: blocks_out[i] is NULL on a miss. */
int pf_engine_query_group_membership(pf_engine *engine, const char *instance_id, uint32_t group_id,
                                     size_t n, const uint8_t *const *hashes, const size_t *hash_lens,
                                     pf_block **blocks_out);
void pf_block_release(pf_block *block);
/* Releases n handles in one call (entries may be NULL): what a caller does with the array
 * pf_engine_query_prefix filled once it holds a lease. */
void pf_blocks_release(pf_block *const *blocks, size_t n);
/* `SealedBlock::slots().len()` and a copy of one slot's segment bytes (`get_slot` +
 * `RawBlock` segments, block.rs): what a host-side consumer (SSD/RDMA tier, a test) reads. */
size_t pf_block_num_slots(const pf_block *block);
int pf_block_slot_info(const pf_block *block, size_t slot, size_t *n_segments, size_t seg_bytes[2]);
int pf_block_slot_read(const pf_block *block, size_t slot, size_t segment, void *out, size_t out_bytes);

/* lib.rs:614-628 `create_query_lease`, lib.rs:631-633 `release_query_lease` (*released = 0
 * when the lease was unknown or expired). */
int pf_engine_create_query_lease(pf_engine *engine, const char *instance_id, size_t n_blocks,
                                 pf_block *const *blocks, uint8_t lease_out[16]);
int pf_engine_release_query_lease(pf_engine *engine, const uint8_t lease[16], int *released);

/* One `(QueryLeaseId, Vec<Vec<Option<usize>>>)` of lib.rs:660: for each load group, one
 * destination per leased block; PF_NO_BLOCK stands for `None`. */
#define PF_NO_BLOCK ((size_t)-1)
typedef struct pf_lease_load {
  uint8_t lease[16];
  size_t n_blocks;             /* blocks held by the lease */
  const size_t *const *dst_ids; /* [n_groups][n_blocks] */
} pf_lease_load;
typedef struct pf_layer_groups {
  size_t n_groups;
  const size_t *group_sizes;        /* layers per group */
  const char *const *layer_names;   /* concatenated, group after group */
} pf_layer_groups;

/* lib.rs:654-680 `batch_load_kv_blocks_multi_layer`: returns after enqueueing; completion is
 * written to the LoadState segment named load_state_shm. */
int pf_engine_batch_load_shm(pf_engine *engine, const char *instance_id, size_t tp_rank, int device_id,
                             const char *load_state_shm, const pf_layer_groups *groups,
                             size_t n_loads, const pf_lease_load *loads);
/* lib.rs:691-709 `batch_load_kv_blocks_multi_layer_inproc`: completion is polled or awaited on
 * the returned handle instead. */
typedef struct pf_completion pf_completion;
int pf_engine_batch_load_inproc(pf_engine *engine, const char *instance_id, size_t tp_rank, int device_id,
                                const pf_layer_groups *groups, size_t n_loads, const pf_lease_load *loads,
                                pf_completion **out);
/* *state: 0 pending, 1 success, -1 error (message via pf_completion_error). */
int pf_completion_poll(pf_completion *completion, int *state);
int pf_completion_wait(pf_completion *completion, double timeout_seconds, int *state);
const char *pf_completion_error(pf_completion *completion);
void pf_completion_free(pf_completion *completion);

/* Layer-wise overlap (new, additive).  The event of `layer_name` on `device_id` is recorded
 * when that layer's bytes of the most recent load have reached the GPU; a compute stream
 * waits on it before running the layer (the body of vLLM's `wait_for_layer_load`, which the
 * reference leaves empty: python/pegaflow/connector/worker.py:712-713). */
int pf_engine_layer_load_event(pf_engine *engine, const char *instance_id, int device_id,
                               const char *layer_name, void **event_out);
/* Make `stream` wait for `event` (cudaStreamWaitEvent), for callers that hold stream and event
 * as plain handles, e.g. a Python connector ordering vLLM's compute stream after a layer's
 * load event. */
int pf_stream_wait_event(void *stream, void *event);
/* Save one or more layers as soon as `ready_event` (recorded by the caller on its compute
 * stream after the layers were written; may be NULL) has fired, without blocking the caller:
 * the body of vLLM's `save_kv_layer` (worker.py:755-765 is a stub in the reference).  The
 * saved slots become visible like those of pf_engine_batch_save once pf_engine_flush_saves
 * returns; a failure of the copy is reported by that pf_engine_flush_saves call.  The caller
 * keeps `ready_event` and the KV memory alive until then. */
int pf_engine_save_layers_async(pf_engine *engine, const char *instance_id, size_t tp_rank, size_t pp_rank,
                                int device_id, size_t n_layers, const pf_layer_save *saves,
                                void *ready_event);

/* Same-box prefix hit without a host round trip (new, additive): copy blocks src_block_ids of
 * every layer both instances registered from src_instance/src_device into dst_block_ids of
 * dst_instance/dst_device over NVLink.  Layers are matched by name and must have the same
 * geometry.  Blocks until the copy has finished. */
int pf_engine_peer_load(pf_engine *engine, const char *src_instance, int src_device,
                        const char *dst_instance, int dst_device, size_t n_blocks,
                        const size_t *src_block_ids, const size_t *dst_block_ids);

/* Transfer metrics with the reference's names (pegaflow-core/src/metrics.rs:325-349). */
typedef struct pf_engine_metrics {
  uint64_t save_bytes;          /* pegaflow_save_bytes */
  double save_duration_seconds; /* sum of pegaflow_save_duration */
  uint64_t save_batches;
  uint64_t load_bytes;          /* pegaflow_load_bytes */
  double load_duration_seconds; /* sum of pegaflow_load_duration */
  uint64_t load_tasks;
  uint64_t load_failures;       /* pegaflow_load_failures */
  uint64_t pool_capacity_bytes; /* pegaflow_pool_capacity_bytes */
  uint64_t pool_used_bytes;     /* pegaflow_pool_used_bytes */
  uint64_t pool_alloc_failures; /* pool_alloc_failures */
  uint64_t cache_blocks;        /* sealed blocks resident */
  uint64_t evicted_blocks;
  pf_backend_stats transfer;    /* sum over the backends of all GPU workers, as of their last task */
} pf_engine_metrics;
int pf_engine_get_metrics(pf_engine *engine, pf_engine_metrics *out);

/* Drop every block from the resident cache (PegaEngine::cleanup_memory_cache, lib.rs:636-639,
 * storage/mod.rs:395-445).  Blocks that a lease, a load in flight or a caller's handle still holds
 * leave the cache too but keep their pool memory until the holder lets go: evicted_bytes is the
 * footprint that left the cache, reclaimed_bytes what the pool got back at once. */
typedef struct pf_cache_cleanup_stats {
  uint64_t evicted_blocks;
  uint64_t evicted_bytes;
  uint64_t reclaimed_bytes;
  uint64_t still_referenced_blocks;
} pf_cache_cleanup_stats;
int pf_engine_cleanup_memory_cache(pf_engine *engine, pf_cache_cleanup_stats *out);

/* `gc_stale_inflight` (lib.rs:938-948; the server calls it every 60 s with 300 s,
 * pegaflow-server/src/lib.rs:612-648): drop the blocks that have been waiting longer than
 * max_age_seconds for slots that never came (a TP rank or a layer that did not save) and give their
 * pool memory back.  *cleaned = number of blocks dropped. */
int pf_engine_gc_stale_inflight(pf_engine *engine, double max_age_seconds, size_t *cleaned);

/* Where a save and a load spend their time on the host side, accumulated since the engine was
 * created: seconds and number of samples per phase.  Phases that the reference traces carry its
 * span names (pf_engine_phase_name: "save.resolve_metadata", "save.hash_filter",
 * "save.pinned_alloc", "save.gpu_copy", "gpu.save_task", "load.cache_lookup", "load.build_tasks",
 * "gpu.load_task"; offload.rs:311,391,428,532, lib.rs:775,835, gpu_worker.rs:433,488); the others
 * split those further.  The same names mark NVTX ranges on the calling and worker threads. */
#define PF_PHASE_COUNT 17
typedef struct pf_engine_phase_times {
  double seconds[PF_PHASE_COUNT];
  uint64_t calls[PF_PHASE_COUNT];
} pf_engine_phase_times;
int pf_engine_get_phase_times(pf_engine *engine, pf_engine_phase_times *out);
const char *pf_engine_phase_name(int phase); /* NULL when out of range */

/* ------------------------------------------------------------------------------------------
 * 4. LoadState.  Replaces `LoadState` (pegaflow-core/src/sync_state.rs:104-188); the segment
 *    layout is bit-compatible, so either side may be the reference's.
 * ---------------------------------------------------------------------------------------- */
typedef struct pf_load_state pf_load_state;
int pf_load_state_new(pf_load_state **out);                      /* sync_state.rs:129-147 `new` */
int pf_load_state_attach(const char *shm_name, pf_load_state **out); /* :150-160 `attach` */
const char *pf_load_state_shm_name(const pf_load_state *state);  /* :163-165 */
int64_t pf_load_state_get(const pf_load_state *state);           /* :168-170; 0 / 1 / -1 */
void pf_load_state_set_completed(pf_load_state *state);          /* :173-177 */
void pf_load_state_set_error(pf_load_state *state);              /* :180-182 */
void pf_load_state_free(pf_load_state *state);                   /* unlinks when it created it */

#ifdef __cplusplus
}
#endif
#endif /* PEGAFLOW_B200_H */
