// Host-side engine: instance registration and topology sealing, the save scheduler
// (validate -> dedupe -> pinned allocation -> one GPU batch -> deferred cache insert), prefix
// query + leases, and the load path.  It mirrors `PegaEngine` of the reference
// (pegaflow-core/src/lib.rs, offload.rs, instance.rs, gpu_worker.rs) on the transfer path and
// keeps a minimal resident block cache in place of the reference's storage tiers.
#pragma once

#include <cuda_runtime.h>

#include <array>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <future>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "common.h"
#include "layout.h"
#include "load_state.h"
#include "pinned_pool.h"
#include "transfer.h"

namespace pf {

// Phases of a save and a load whose time the engine accumulates (pf_engine_get_phase_times).  Where
// the reference has a trace span for the same stretch, the phase carries its name (offload.rs:311,
// 391,428,532; lib.rs:775,835; gpu_worker.rs:433,488), and the same names mark NVTX ranges.
enum Phase {
  kSaveResolve = 0,   // save.resolve_metadata
  kSaveHashFilter,    // save.hash_filter
  kSavePinnedAlloc,   // save.pinned_alloc
  kSaveGpuCopy,       // save.gpu_copy: caller's wait from submit until the worker reports the copy done
  kSaveQueueWait,     //   of which: the task sat in the save worker's queue
  kSaveTask,          // gpu.save_task: the worker's time in the task (enqueue + wait for the GPU)
  kSaveEnqueue,       //   of which: building and enqueueing the transfers
  kSaveInsertBuild,   // per-block bookkeeping for the cache, built on the caller while the copy runs
  kSaveInsert,        // sealing and inserting blocks on the insert thread
  kFlushWait,         // flush_saves: waiting for the insert thread
  kQueryPrefix,       // prefix lookup
  kCreateLease,
  kLoadCacheLookup,   // load.cache_lookup: leases consumed, targets mapped
  kLoadBuildTasks,    // load.build_tasks
  kLoadQueueWait,     // the task sat in the load worker's queue
  kLoadTask,          // gpu.load_task
  kLoadEnqueue,       //   of which: building and enqueueing the transfers
  kPhaseCount
};
static_assert(kPhaseCount == PF_PHASE_COUNT, "phase list and C ABI disagree");
const char *phase_name(int phase);

// ---- stored blocks (block.rs) --------------------------------------------------------------
struct Segment {
  char *host = nullptr;
  uint64_t device = 0;
  size_t size = 0;
};

// Keeps pool memory alive: a pinned allocation, or the set of allocations of one save call.
using Owner = std::shared_ptr<const void>;

// One slot of a block: one segment (contiguous / page) or two (K and V).  The reference ties
// every segment to its allocation (`Arc<PinnedAllocation>` per Segment, block.rs:64-71); a layer
// batch allocation is shared by all blocks of the save, so here the owner is kept once per save
// where possible (on the sealed block, else on the slot) instead of twice per slot.
struct RawBlock {
  Segment seg[2];
  int n_segments = 0;
  Owner owner;  // null when the enclosing SealedBlock / RawSaveBatch owns the memory
  size_t total_size() const { return seg[0].size + (n_segments > 1 ? seg[1].size : 0); }
};

struct SealedBlock {
  std::vector<RawBlock> slots;
  Owner owner;  // covers every slot whose own owner is null
  size_t footprint = 0;
};
using BlockRef = std::shared_ptr<SealedBlock>;

struct BlockKey {
  std::string ns, hash;
  bool operator==(const BlockKey &o) const { return ns == o.ns && hash == o.hash; }
};
struct BlockKeyHash {
  size_t operator()(const BlockKey &k) const {
    return std::hash<std::string>()(k.hash) * 1000003u ^ std::hash<std::string>()(k.ns);
  }
};

// group 0 keeps the raw hash, other groups append the big-endian group id
// (pegaflow-common/src/block.rs:35-43).
std::string group_hash(const std::string &hash, uint32_t group);

// ---- resident cache with LRU eviction (storage/read_cache.rs, storage/mod.rs:482-554) -------
class ReadCache {
 public:
  bool contains(const BlockKey &key);
  void contains_many(const std::string &ns, const std::vector<std::string> &hashes, std::vector<char> *out);
  BlockRef get(const BlockKey &key, bool touch);
  // Returns false (and drops `block`) when the key is already resident.
  bool insert(const BlockKey &key, BlockRef block);
  // Drops up to n least recently used blocks; returns how many were dropped.
  size_t evict_lru(size_t n);
  // Takes every resident block out of the cache, held by someone else or not.
  std::vector<BlockRef> remove_all();
  size_t size();

 private:
  struct Entry {
    BlockRef block;
    std::list<BlockKey>::iterator pos;
  };
  std::mutex mu_;
  std::unordered_map<BlockKey, Entry, BlockKeyHash> map_;
  std::list<BlockKey> lru_;  // front = most recent
};

// ---- per-layer work item shared by save and load -----------------------------------------------
// Owns what a pf_layer_xfer points at.
struct LayerWork {
  std::string layer_name;
  KVCacheLayout layout;
  std::vector<uint32_t> block_ids;
  std::vector<pf_host_run> runs[2];
  size_t payload_bytes() const { return block_ids.size() * layout.range_bytes() * layout.n_ranges(); }
};

// Merges consecutive host addresses into runs of constant stride.
class RunBuilder {
 public:
  explicit RunBuilder(size_t item_bytes) : item_bytes_(item_bytes) {}
  void add(char *host, uint64_t device);
  std::vector<pf_host_run> take() { return std::move(runs_); }

 private:
  size_t item_bytes_;
  size_t next_index_ = 0;
  std::vector<pf_host_run> runs_;
};

// ---- topology (instance.rs:48-269) -----------------------------------------------------------
struct LayerTopology {
  std::unordered_map<std::string, size_t> name_to_id;
  std::vector<std::string> names;
  size_t tp_size = 1;
  std::vector<uint32_t> layer_group;
  std::vector<size_t> group_layer_count, layer_group_rank;
  std::optional<PageLayout> page;

  size_t layer_id(const std::string &name) const;
  size_t num_layers() const { return names.size(); }
  size_t num_groups() const { return group_layer_count.size(); }
  size_t total_slots() const { return page ? page->shard_page_sizes.size() : num_layers() * tp_size; }
  size_t group_total_slots(uint32_t group) const;
  size_t slot_index(size_t layer_id, size_t tp_rank) const;
  size_t shard_layer_count(size_t shard) const;
};

// ---- GPU workers (gpu_worker.rs:118-345) ---------------------------------------------------
// A dedicated thread with its own stream and transfer backend, pinned to the GPU's NUMA node.
class GpuWorker {
 public:
  using Task = std::function<void(TransferBackend &, cudaStream_t)>;
  GpuWorker(const std::string &name, int device, int numa_node, const pf_backend_config &cfg);
  ~GpuWorker();
  void submit(Task task);
  // A task is about to be submitted: have the thread awake and polling for it (for a bounded
  // time) by then, so that its wake-up overlaps the caller's preparation instead of following it.
  void expect_task();
  // Number of tasks submitted so far; task k (1-based) carries ticket k.
  uint64_t submitted() const { return submitted_.load(); }
  // Ticket of the task the worker thread is running (valid inside a task only).
  uint64_t current_ticket() const { return current_ticket_; }
  // Blocks until the task with this ticket has enqueued its GPU work (it calls mark_enqueued)
  // or has finished.
  void wait_enqueued(uint64_t ticket);
  void mark_enqueued(uint64_t ticket);
  // Counters of the worker's backend as of the end of its last task.
  pf_backend_stats last_stats();

 private:
  void loop(int device, int numa_node, pf_backend_config cfg, std::promise<void> ready);
  std::string name_;
  std::thread thread_;
  std::mutex mu_;
  std::condition_variable cv_, enq_cv_;
  std::deque<Task> queue_;
  bool stop_ = false;
  bool expected_ = false;
  std::atomic<uint64_t> submitted_{0};
  uint64_t enqueued_ = 0;
  uint64_t current_ticket_ = 0;
  pf_backend_stats last_stats_{};
};

struct GpuContext {
  int device_id = 0;
  size_t tp_rank = 0, pp_rank = 0;
  int numa_node = -1;
  std::unordered_map<std::string, KVCacheLayout> layouts;
  std::unordered_map<std::string, uint32_t> groups;
  std::unordered_map<std::string, cudaEvent_t> load_events;  // one per layer, see layer_load_event
  std::unique_ptr<GpuWorker> load_worker, save_worker;
  uint32_t group_of(const std::string &layer) const {
    auto it = groups.find(layer);
    return it == groups.end() ? 0 : it->second;
  }
  ~GpuContext();
};

struct InstanceContext {
  std::string id, ns;
  size_t tp_size = 1, world_size = 1;
  bool page_first = false;
  std::mutex mu;
  std::map<int, std::shared_ptr<GpuContext>> gpus;
  std::shared_ptr<LayerTopology> topology;
};

// Completion of an in-process load (LoadCompletion::Channel, gpu_worker.rs:29-52).
struct Completion {
  std::mutex mu;
  std::condition_variable cv;
  int state = 0;  // 0 pending, 1 ok, -1 error
  std::string error;
  void signal(bool ok, const std::string &msg);
};

// A list of block hashes, shared between the layers of a save that carry the same list.
using HashList = std::shared_ptr<const std::vector<std::string>>;

struct LayerSaveIn {
  std::string layer_name;
  std::vector<size_t> block_ids;
  HashList block_hashes;
};

struct LeaseLoadIn {
  std::array<uint8_t, 16> lease;
  std::vector<std::vector<size_t>> dst_ids;  // [group][block], PF_NO_BLOCK = none
};

class Engine {
 public:
  Engine(size_t pool_bytes, bool use_hugepages, const pf_storage_config *config);
  ~Engine();

  void register_context_layer_batch_strided(const std::string &instance_id, const std::string &ns, int device_id,
                                            size_t tp_rank, size_t pp_rank, size_t tp_size, size_t world_size,
                                            const std::vector<std::string> &layer_names, const uint64_t *data_ptrs,
                                            const size_t *size_bytes, const size_t *num_blocks,
                                            const size_t *bytes_per_block, const size_t *kv_stride_bytes,
                                            const size_t *segments, const size_t *block_stride_bytes,
                                            const uint32_t *layer_group_ids, int transfer_mode, bool page_first);
  void unregister_instance(const std::string &instance_id);
  std::vector<std::string> unregister_all_instances();
  std::vector<std::string> list_instance_ids();
  std::string instance_namespace(const std::string &instance_id);

  // ready_event == nullptr && !async: blocking save (offload.rs:293).  async: returns after the
  // pinned allocation; the copy, its completion wait and the cache insert run on the save worker.
  void batch_save(const std::string &instance_id, size_t tp_rank, size_t pp_rank, int device_id,
                  std::vector<LayerSaveIn> saves, bool async, cudaEvent_t ready_event);
  void flush_saves();

  void query_prefix(const std::string &instance_id, const std::vector<std::string> &hashes,
                    std::vector<BlockRef> *blocks, size_t *missing);
  std::vector<BlockRef> query_group_membership(const std::string &instance_id, uint32_t group,
                                               const std::vector<std::string> &hashes);
  std::array<uint8_t, 16> create_query_lease(const std::string &instance_id, std::vector<BlockRef> blocks);
  bool release_query_lease(const std::array<uint8_t, 16> &lease);

  // Exactly one of shm_name / completion is used (LoadCompletion, gpu_worker.rs:29-52).
  void batch_load(const std::string &instance_id, size_t tp_rank, int device_id,
                  const std::vector<std::vector<std::string>> &layer_groups, const std::vector<LeaseLoadIn> &loads,
                  const std::string &shm_name, std::shared_ptr<Completion> completion);
  cudaEvent_t layer_load_event(const std::string &instance_id, int device_id, const std::string &layer);
  void peer_load(const std::string &src_instance, int src_device, const std::string &dst_instance, int dst_device,
                 const std::vector<size_t> &src_ids, const std::vector<size_t> &dst_ids);
  void metrics(pf_engine_metrics *out);
  void cleanup_memory_cache(pf_cache_cleanup_stats *out);
  // Drops blocks that have waited for their missing slots longer than max_age_seconds (a rank or a
  // layer that never saved); returns how many.  Their pool memory goes back.
  size_t gc_stale_inflight(double max_age_seconds);
  void phase_times(pf_engine_phase_times *out);

 private:
  // Adds the time since `since` to a phase and returns now.
  std::chrono::steady_clock::time_point lap(Phase p, std::chrono::steady_clock::time_point since);
  std::atomic<uint64_t> phase_nanos_[kPhaseCount] = {}, phase_calls_[kPhaseCount] = {};

  struct RawSaveLayer {
    size_t slot_id;
    std::vector<RawBlock> blocks;
    std::shared_ptr<const std::vector<std::string>> hashes;  // already group-encoded
  };
  struct RawSaveBatch {
    std::string ns;
    size_t total_slots;
    std::vector<RawSaveLayer> layers;
    Owner owner;  // all pool allocations of the save call (null when the slots carry their own)
    // A save that fills every slot of its blocks by itself (one rank, all layers, one hash list) is
    // sealed while its copy runs: block b of `sealed` belongs under (*sealed_hashes)[b], `layers` is empty.
    std::vector<BlockRef> sealed;
    HashList sealed_hashes;
  };
  struct Inflight {
    size_t total_slots;
    size_t filled = 0;
    std::vector<std::optional<RawBlock>> slots;
    std::chrono::steady_clock::time_point created = std::chrono::steady_clock::now();
  };
  struct Lease {
    std::string instance_id;
    std::vector<BlockRef> blocks;
    size_t remaining;
    std::chrono::steady_clock::time_point expires;
  };
  struct LeaseKeyHash {
    size_t operator()(const std::array<uint8_t, 16> &k) const {
      uint64_t a, b;
      memcpy(&a, k.data(), 8);
      memcpy(&b, k.data() + 8, 8);
      return (size_t)(a ^ (b * 0x9E3779B97F4A7C15ull));
    }
  };

  std::shared_ptr<InstanceContext> get_instance(const std::string &id);
  std::shared_ptr<LayerTopology> sealed_topology(InstanceContext &inst);
  std::shared_ptr<LayerTopology> seal(InstanceContext &inst, const std::vector<std::shared_ptr<GpuContext>> &gpus);
  std::shared_ptr<PinnedAllocation> allocate(uint64_t bytes, int numa_node, const char *what);
  void send_raw_insert(RawSaveBatch batch);
  void insert_loop();
  void process_insert(RawSaveBatch &batch);
  void insert_slot(const BlockKey &key, size_t slot, RawBlock block, size_t total_slots, const Owner &batch_owner);
  std::vector<BlockRef> consume_lease(const std::string &instance_id, const std::array<uint8_t, 16> &lease);
  void sweep_leases();

  pf_storage_config cfg_{};
  std::unique_ptr<PinnedAllocator> allocator_;
  ReadCache cache_;
  std::mutex instances_mu_;
  std::unordered_map<std::string, std::shared_ptr<InstanceContext>> instances_;

  std::mutex leases_mu_;
  std::unordered_map<std::array<uint8_t, 16>, Lease, LeaseKeyHash> leases_;

  // deferred insert worker (storage/write_path.rs:74-103)
  std::thread insert_thread_;
  std::mutex insert_mu_;
  std::condition_variable insert_cv_, insert_idle_cv_;
  std::deque<RawSaveBatch> insert_queue_;
  size_t insert_pending_ = 0;  // queued + in progress + async saves not yet handed over
  bool insert_stop_ = false;
  bool trace_ = false;       // PEGAFLOW_B200_TRACE=1: per-save phase timings on stderr
  std::string async_error_;  // first failure of an asynchronous save since the last flush
  std::mutex inflight_mu_;  // the insert thread and gc_stale_inflight
  std::unordered_map<BlockKey, Inflight, BlockKeyHash> inflight_;

  // metrics (metrics.rs:325-349)
  std::atomic<uint64_t> save_bytes_{0}, save_batches_{0}, load_bytes_{0}, load_tasks_{0}, load_failures_{0},
      alloc_failures_{0}, evicted_{0};
  std::atomic<uint64_t> save_nanos_{0}, load_nanos_{0};
};

}  // namespace pf
