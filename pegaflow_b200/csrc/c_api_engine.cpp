// extern "C" surface of the pinned pool, the engine and LoadState (include/pegaflow_b200.h,
// sections 2-4).
#include <chrono>
#include <cstring>
#include <map>

#include "common.h"
#include "engine.h"
#include "load_state.h"
#include "numa.h"
#include "pinned_pool.h"

using namespace pf;

struct pf_pool {
  std::unique_ptr<PinnedAllocator> impl;
  std::mutex mu;
  uint64_t next_handle = 1;
  std::unordered_map<uint64_t, std::shared_ptr<PinnedAllocation>> live;
  int node = -1;
};
struct pf_engine {
  Engine impl;
  pf_engine(size_t pool, bool huge, const pf_storage_config *cfg) : impl(pool, huge, cfg) {}
};
struct pf_block {
  BlockRef ref;
};
struct pf_completion {
  std::shared_ptr<Completion> impl;
  std::string error_copy;
};
struct pf_load_state {
  std::unique_ptr<LoadState> impl;
};

namespace {
std::vector<std::string> to_hashes(size_t n, const uint8_t *const *hashes, const size_t *lens) {
  std::vector<std::string> out;
  out.reserve(n);
  for (size_t i = 0; i < n; ++i) out.emplace_back(reinterpret_cast<const char *>(hashes[i]), lens[i]);
  return out;
}

std::vector<LayerSaveIn> to_saves(size_t n_layers, const pf_layer_save *saves) {
  std::vector<LayerSaveIn> out(n_layers);
  // Layers that point at the same hash array share one copy of it.
  std::map<std::pair<const void *, size_t>, HashList> seen;
  for (size_t i = 0; i < n_layers; ++i) {
    const pf_layer_save &s = saves[i];
    if (!s.layer_name) throw Error::invalid("layer_name is null");
    out[i].layer_name = s.layer_name;
    out[i].block_ids.assign(s.block_ids, s.block_ids + s.n_blocks);
    auto key = std::make_pair((const void *)s.block_hashes, s.n_blocks);
    auto it = seen.find(key);
    if (it == seen.end())
      it = seen.emplace(key, std::make_shared<const std::vector<std::string>>(
                                 to_hashes(s.n_blocks, s.block_hashes, s.block_hash_lens))).first;
    out[i].block_hashes = it->second;
  }
  return out;
}

void to_load_args(const pf_layer_groups *groups, size_t n_loads, const pf_lease_load *loads,
                  std::vector<std::vector<std::string>> *layer_groups, std::vector<LeaseLoadIn> *lease_loads) {
  if (!groups) throw Error::invalid("layer groups are null");
  size_t cursor = 0;
  for (size_t g = 0; g < groups->n_groups; ++g) {
    std::vector<std::string> names;
    for (size_t i = 0; i < groups->group_sizes[g]; ++i) names.emplace_back(groups->layer_names[cursor++]);
    layer_groups->push_back(std::move(names));
  }
  for (size_t l = 0; l < n_loads; ++l) {
    LeaseLoadIn in;
    memcpy(in.lease.data(), loads[l].lease, 16);
    for (size_t g = 0; g < groups->n_groups; ++g)
      in.dst_ids.emplace_back(loads[l].dst_ids[g], loads[l].dst_ids[g] + loads[l].n_blocks);
    lease_loads->push_back(std::move(in));
  }
}
}  // namespace

extern "C" {

// ---- pool ----------------------------------------------------------------------------------------
int pf_pool_new(size_t bytes, const pf_pool_config *config, pf_pool **out) {
  return guarded([&] {
    if (!out) throw Error::invalid("out is null");
    if (bytes == 0) throw Error::storage("Pinned memory pool size must be greater than zero");
    pf_pool_config c = config ? *config : pf_pool_config{0, 0, -1, 0, 1, 0};
    PinnedMemory::Strategy st = c.use_hugepages      ? PinnedMemory::Strategy::HugePages
                                : c.transparent_huge ? PinnedMemory::Strategy::MmapTransparentHuge
                                : c.use_mmap         ? PinnedMemory::Strategy::MmapRegister
                                                     : PinnedMemory::Strategy::CudaHostAlloc;
    auto pool = std::make_unique<pf_pool>();
    std::vector<int> nodes;
    if (c.numa_node >= 0) nodes.push_back(c.numa_node);
    pool->node = c.numa_node;
    pool->impl = std::make_unique<PinnedAllocator>(bytes, nodes, c.shards, st, c.unit_hint);
    *out = pool.release();
  });
}

void pf_pool_free(pf_pool *pool) { delete pool; }

int pf_pool_alloc(pf_pool *pool, size_t bytes, void **host, uint64_t *host_device, uint64_t *handle) {
  return guarded([&] {
    if (!pool || !host || !host_device || !handle) throw Error::invalid("null argument");
    auto a = pool->impl->allocate(bytes, pool->node);
    if (!a) throw Error::storage("pinned pool exhausted");
    *host = a->host();
    *host_device = a->device();
    std::lock_guard<std::mutex> g(pool->mu);
    *handle = pool->next_handle++;
    pool->live[*handle] = std::move(a);
  });
}

int pf_pool_release(pf_pool *pool, uint64_t handle) {
  return guarded([&] {
    if (!pool) throw Error::invalid("pool is null");
    std::lock_guard<std::mutex> g(pool->mu);
    if (!pool->live.erase(handle)) throw Error::invalid("unknown pool allocation handle");
  });
}

int pf_pool_usage(pf_pool *pool, uint64_t *used, uint64_t *total, uint64_t *largest_free) {
  return guarded([&] {
    if (!pool) throw Error::invalid("pool is null");
    uint64_t u, t;
    pool->impl->usage(&u, &t);
    if (used) *used = u;
    if (total) *total = t;
    if (largest_free) *largest_free = pool->impl->largest_free(pool->node);
  });
}

size_t pf_pool_pre_touch_threads(size_t bytes) { return pre_touch_threads(bytes); }
size_t pf_huge_page_size(void) { return huge_page_size(); }

// ---- NUMA ----------------------------------------------------------------------------------------
namespace {
void copy_ints(const std::vector<int> &v, int *out, size_t capacity, size_t *n) {
  if (!n) throw Error::invalid("n is null");
  *n = v.size();
  if (v.size() > capacity) throw Error::invalid(strf("%zu entries do not fit a buffer of %zu", v.size(), capacity));
  for (size_t i = 0; i < v.size(); ++i) out[i] = v[i];
}
}  // namespace

int pf_numa_node_of_device(int device_id) { return numa::node_of_device(device_id); }
int pf_numa_num_nodes(void) { return (int)numa::online_nodes().size(); }
int pf_numa_set_sysfs_root(const char *root) {
  return guarded([&] { numa::set_sysfs_root(root ? root : ""); });
}
int pf_numa_parse_cpulist(const char *text, int *cpus_out, size_t capacity, size_t *n) {
  return guarded([&] {
    if (!text) throw Error::invalid("text is null");
    try {
      copy_ints(numa::parse_cpulist(text), cpus_out, capacity, n);
    } catch (const std::invalid_argument &e) {
      throw Error::invalid(e.what());
    }
  });
}
int pf_numa_cpus_of_node(int node, int *cpus_out, size_t capacity, size_t *n) {
  return guarded([&] { copy_ints(numa::cpus_of_node(node), cpus_out, capacity, n); });
}
int pf_numa_pin_thread_to_node(int node) {
  return guarded([&] {
    const std::string why = numa::pin_thread_to_node_why(node);
    if (!why.empty()) throw Error::invalid(why);
  });
}
int pf_numa_node_of_pci_device(const char *bus_id) { return bus_id ? numa::node_of_pci_device(bus_id) : numa::kUnknown; }
int pf_numa_parse_closest_cpu_node(const char *text) { return text ? numa::parse_closest_cpu_node(text) : numa::kUnknown; }
int pf_numa_distinct_valid_nodes(const int *device_nodes, size_t n_devices, int *nodes_out, size_t *n) {
  return guarded([&] {
    if (n_devices && !device_nodes) throw Error::invalid("device_nodes is null");
    copy_ints(numa::distinct_valid_nodes(std::vector<int>(device_nodes, device_nodes + n_devices)), nodes_out, n_devices, n);
  });
}
int pf_numa_query_pages(const void *const *addrs, size_t n, int *nodes_out) {
  return guarded([&] {
    if (n && (!addrs || !nodes_out)) throw Error::invalid("null argument");
    const std::vector<int> nodes = numa::query_pages(std::vector<const void *>(addrs, addrs + n));
    for (size_t i = 0; i < n; ++i) nodes_out[i] = nodes[i];
  });
}

// ---- engine --------------------------------------------------------------------------------------
int pf_engine_new(size_t pool_bytes, int use_hugepages, const pf_storage_config *config, pf_engine **out) {
  return guarded([&] {
    if (!out) throw Error::invalid("out is null");
    *out = new pf_engine(pool_bytes, use_hugepages != 0, config);
  });
}

void pf_engine_free(pf_engine *engine) { delete engine; }

int pf_engine_register_context_layer_batch_strided(
    pf_engine *engine, const char *instance_id, const char *namespace_, int device_id, size_t tp_rank, size_t pp_rank,
    size_t tp_size, size_t world_size, size_t n_layers, const char *const *layer_names, const uint64_t *data_ptrs,
    const size_t *size_bytes, const size_t *num_blocks, const size_t *bytes_per_block, const size_t *kv_stride_bytes,
    const size_t *segments, const size_t *block_stride_bytes, const uint32_t *layer_group_ids, int transfer_mode,
    int page_first) {
  return guarded([&] {
    if (!engine || !instance_id || !namespace_) throw Error::invalid("null argument");
    std::vector<std::string> names;
    for (size_t i = 0; i < n_layers; ++i) names.emplace_back(layer_names[i]);
    engine->impl.register_context_layer_batch_strided(instance_id, namespace_, device_id, tp_rank, pp_rank, tp_size,
                                                      world_size, names, data_ptrs, size_bytes, num_blocks,
                                                      bytes_per_block, kv_stride_bytes, segments, block_stride_bytes,
                                                      layer_group_ids, transfer_mode, page_first != 0);
  });
}

int pf_engine_unregister_instance(pf_engine *engine, const char *instance_id) {
  return guarded([&] {
    if (!engine || !instance_id) throw Error::invalid("null argument");
    engine->impl.unregister_instance(instance_id);
  });
}

namespace {
// Writes `text` (NUL-terminated) into buf when it fits; *needed is its size with the terminator.
void copy_out(const std::string &text, char *buf, size_t cap, size_t *needed) {
  if (needed) *needed = text.size() + 1;
  if (buf && cap > text.size()) memcpy(buf, text.c_str(), text.size() + 1);
  else if (buf && cap) buf[0] = 0;
}
std::string join_lines(const std::vector<std::string> &ids) {
  std::string out;
  for (size_t i = 0; i < ids.size(); ++i) out += (i ? "\n" : "") + ids[i];
  return out;
}
}  // namespace

int pf_engine_list_instances(pf_engine *engine, char *buf, size_t cap, size_t *needed) {
  return guarded([&] {
    if (!engine) throw Error::invalid("null argument");
    copy_out(join_lines(engine->impl.list_instance_ids()), buf, cap, needed);
  });
}

int pf_engine_unregister_all_instances(pf_engine *engine, char *buf, size_t cap, size_t *needed) {
  return guarded([&] {
    if (!engine) throw Error::invalid("null argument");
    copy_out(join_lines(engine->impl.unregister_all_instances()), buf, cap, needed);
  });
}

int pf_engine_instance_namespace(pf_engine *engine, const char *instance_id, char *buf, size_t cap, size_t *needed) {
  return guarded([&] {
    if (!engine || !instance_id) throw Error::invalid("null argument");
    copy_out(engine->impl.instance_namespace(instance_id), buf, cap, needed);
  });
}

int pf_engine_batch_save(pf_engine *engine, const char *instance_id, size_t tp_rank, size_t pp_rank, int device_id,
                         size_t n_layers, const pf_layer_save *saves) {
  return guarded([&] {
    if (!engine || !instance_id) throw Error::invalid("null argument");
    engine->impl.batch_save(instance_id, tp_rank, pp_rank, device_id, to_saves(n_layers, saves), false, nullptr);
  });
}

int pf_engine_save_layers_async(pf_engine *engine, const char *instance_id, size_t tp_rank, size_t pp_rank,
                                int device_id, size_t n_layers, const pf_layer_save *saves, void *ready_event) {
  return guarded([&] {
    if (!engine || !instance_id) throw Error::invalid("null argument");
    engine->impl.batch_save(instance_id, tp_rank, pp_rank, device_id, to_saves(n_layers, saves), true,
                            (cudaEvent_t)ready_event);
  });
}

int pf_engine_flush_saves(pf_engine *engine) {
  return guarded([&] {
    if (!engine) throw Error::invalid("engine is null");
    engine->impl.flush_saves();
  });
}

int pf_engine_query_prefix(pf_engine *engine, const char *instance_id, const char *req_id, size_t n,
                           const uint8_t *const *hashes, const size_t *hash_lens, pf_block **blocks_out, size_t *n_hit,
                           size_t *n_missing) {
  (void)req_id;  // only tags SSD prefetch state in the reference; there is no SSD tier here
  return guarded([&] {
    if (!engine || !instance_id || !n_hit || !n_missing) throw Error::invalid("null argument");
    std::vector<BlockRef> blocks;
    size_t missing = 0;
    engine->impl.query_prefix(instance_id, to_hashes(n, hashes, hash_lens), &blocks, &missing);
    for (size_t i = 0; i < blocks.size(); ++i) blocks_out[i] = new pf_block{std::move(blocks[i])};
    *n_hit = blocks.size();
    *n_missing = missing;
  });
}

int pf_engine_query_group_membership(pf_engine *engine, const char *instance_id, uint32_t group_id, size_t n,
                                     const uint8_t *const *hashes, const size_t *hash_lens, pf_block **blocks_out) {
  return guarded([&] {
    if (!engine || !instance_id) throw Error::invalid("null argument");
    auto blocks = engine->impl.query_group_membership(instance_id, group_id, to_hashes(n, hashes, hash_lens));
    for (size_t i = 0; i < blocks.size(); ++i) blocks_out[i] = blocks[i] ? new pf_block{std::move(blocks[i])} : nullptr;
  });
}

void pf_block_release(pf_block *block) { delete block; }

void pf_blocks_release(pf_block *const *blocks, size_t n) {
  for (size_t i = 0; blocks && i < n; ++i) delete blocks[i];
}

size_t pf_block_num_slots(const pf_block *block) { return block ? block->ref->slots.size() : 0; }

int pf_block_slot_info(const pf_block *block, size_t slot, size_t *n_segments, size_t seg_bytes[2]) {
  return guarded([&] {
    if (!block || slot >= block->ref->slots.size()) throw Error::invalid("slot out of range");
    const RawBlock &raw = block->ref->slots[slot];
    *n_segments = (size_t)raw.n_segments;
    seg_bytes[0] = raw.seg[0].size;
    seg_bytes[1] = raw.n_segments > 1 ? raw.seg[1].size : 0;
  });
}

int pf_block_slot_read(const pf_block *block, size_t slot, size_t segment, void *out, size_t out_bytes) {
  return guarded([&] {
    if (!block || slot >= block->ref->slots.size()) throw Error::invalid("slot out of range");
    const RawBlock &raw = block->ref->slots[slot];
    if (segment >= (size_t)raw.n_segments) throw Error::invalid("segment out of range");
    if (out_bytes > raw.seg[segment].size) throw Error::invalid("read exceeds the segment");
    memcpy(out, raw.seg[segment].host, out_bytes);
  });
}

int pf_engine_create_query_lease(pf_engine *engine, const char *instance_id, size_t n_blocks, pf_block *const *blocks,
                                 uint8_t lease_out[16]) {
  return guarded([&] {
    if (!engine || !instance_id || !lease_out) throw Error::invalid("null argument");
    std::vector<BlockRef> refs;
    for (size_t i = 0; i < n_blocks; ++i) {
      if (!blocks[i]) throw Error::invalid("null block handle");
      refs.push_back(blocks[i]->ref);
    }
    auto token = engine->impl.create_query_lease(instance_id, std::move(refs));
    memcpy(lease_out, token.data(), 16);
  });
}

int pf_engine_release_query_lease(pf_engine *engine, const uint8_t lease[16], int *released) {
  return guarded([&] {
    if (!engine || !lease) throw Error::invalid("null argument");
    std::array<uint8_t, 16> token;
    memcpy(token.data(), lease, 16);
    const bool ok = engine->impl.release_query_lease(token);
    if (released) *released = ok ? 1 : 0;
  });
}

int pf_engine_batch_load_shm(pf_engine *engine, const char *instance_id, size_t tp_rank, int device_id,
                             const char *load_state_shm, const pf_layer_groups *groups, size_t n_loads,
                             const pf_lease_load *loads) {
  return guarded([&] {
    if (!engine || !instance_id || !load_state_shm) throw Error::invalid("null argument");
    std::vector<std::vector<std::string>> layer_groups;
    std::vector<LeaseLoadIn> lease_loads;
    to_load_args(groups, n_loads, loads, &layer_groups, &lease_loads);
    engine->impl.batch_load(instance_id, tp_rank, device_id, layer_groups, lease_loads, load_state_shm, nullptr);
  });
}

int pf_engine_batch_load_inproc(pf_engine *engine, const char *instance_id, size_t tp_rank, int device_id,
                                const pf_layer_groups *groups, size_t n_loads, const pf_lease_load *loads,
                                pf_completion **out) {
  return guarded([&] {
    if (!engine || !instance_id || !out) throw Error::invalid("null argument");
    std::vector<std::vector<std::string>> layer_groups;
    std::vector<LeaseLoadIn> lease_loads;
    to_load_args(groups, n_loads, loads, &layer_groups, &lease_loads);
    auto completion = std::make_shared<Completion>();
    engine->impl.batch_load(instance_id, tp_rank, device_id, layer_groups, lease_loads, "", completion);
    *out = new pf_completion{completion, ""};
  });
}

int pf_completion_poll(pf_completion *completion, int *state) {
  return guarded([&] {
    if (!completion || !state) throw Error::invalid("null argument");
    std::lock_guard<std::mutex> g(completion->impl->mu);
    *state = completion->impl->state;
  });
}

int pf_completion_wait(pf_completion *completion, double timeout_seconds, int *state) {
  return guarded([&] {
    if (!completion || !state) throw Error::invalid("null argument");
    std::unique_lock<std::mutex> g(completion->impl->mu);
    completion->impl->cv.wait_for(g, std::chrono::duration<double>(timeout_seconds),
                                  [&] { return completion->impl->state != 0; });
    *state = completion->impl->state;
  });
}

const char *pf_completion_error(pf_completion *completion) {
  if (!completion) return "";
  std::lock_guard<std::mutex> g(completion->impl->mu);
  completion->error_copy = completion->impl->error;
  return completion->error_copy.c_str();
}

void pf_completion_free(pf_completion *completion) { delete completion; }

int pf_engine_layer_load_event(pf_engine *engine, const char *instance_id, int device_id, const char *layer_name,
                               void **event_out) {
  return guarded([&] {
    if (!engine || !instance_id || !layer_name || !event_out) throw Error::invalid("null argument");
    *event_out = engine->impl.layer_load_event(instance_id, device_id, layer_name);
  });
}

int pf_stream_wait_event(void *stream, void *event) {
  return guarded([&] {
    if (!event) throw Error::invalid("event is null");
    cudaError_t e = cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0);
    if (e != cudaSuccess) throw Error::storage(strf("cudaStreamWaitEvent failed: %s", cudaGetErrorString(e)));
  });
}

int pf_engine_peer_load(pf_engine *engine, const char *src_instance, int src_device, const char *dst_instance,
                        int dst_device, size_t n_blocks, const size_t *src_block_ids, const size_t *dst_block_ids) {
  return guarded([&] {
    if (!engine || !src_instance || !dst_instance) throw Error::invalid("null argument");
    engine->impl.peer_load(src_instance, src_device, dst_instance, dst_device,
                           std::vector<size_t>(src_block_ids, src_block_ids + n_blocks),
                           std::vector<size_t>(dst_block_ids, dst_block_ids + n_blocks));
  });
}

int pf_engine_get_phase_times(pf_engine *engine, pf_engine_phase_times *out) {
  return guarded([&] {
    if (!engine || !out) throw Error::invalid("null argument");
    engine->impl.phase_times(out);
  });
}

const char *pf_engine_phase_name(int phase) { return phase_name(phase); }

int pf_engine_get_metrics(pf_engine *engine, pf_engine_metrics *out) {
  return guarded([&] {
    if (!engine || !out) throw Error::invalid("null argument");
    engine->impl.metrics(out);
  });
}

int pf_engine_gc_stale_inflight(pf_engine *engine, double max_age_seconds, size_t *cleaned) {
  return guarded([&] {
    if (!engine || !cleaned) throw Error::invalid("null argument");
    if (!(max_age_seconds >= 0)) throw Error::invalid("max_age_seconds must be >= 0");
    *cleaned = engine->impl.gc_stale_inflight(max_age_seconds);
  });
}

int pf_engine_cleanup_memory_cache(pf_engine *engine, pf_cache_cleanup_stats *out) {
  return guarded([&] {
    if (!engine || !out) throw Error::invalid("null argument");
    engine->impl.cleanup_memory_cache(out);
  });
}

// ---- LoadState -------------------------------------------------------------------------------------
int pf_load_state_new(pf_load_state **out) {
  return guarded([&] {
    if (!out) throw Error::invalid("out is null");
    auto ls = std::make_unique<pf_load_state>();
    ls->impl.reset(LoadState::create());
    *out = ls.release();
  });
}

int pf_load_state_attach(const char *shm_name, pf_load_state **out) {
  return guarded([&] {
    if (!out || !shm_name) throw Error::invalid("null argument");
    auto ls = std::make_unique<pf_load_state>();
    ls->impl.reset(LoadState::attach(shm_name));
    *out = ls.release();
  });
}

const char *pf_load_state_shm_name(const pf_load_state *state) { return state ? state->impl->shm_name().c_str() : ""; }
int64_t pf_load_state_get(const pf_load_state *state) { return state ? state->impl->get() : LoadState::kError; }
void pf_load_state_set_completed(pf_load_state *state) {
  if (state) state->impl->set_completed();
}
void pf_load_state_set_error(pf_load_state *state) {
  if (state) state->impl->set_error();
}
void pf_load_state_free(pf_load_state *state) { delete state; }

}  // extern "C"
