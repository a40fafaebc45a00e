#include "engine.h"

#include <algorithm>
#include <cstring>
#include <random>
#include <set>

#include <nvtx3/nvToolsExt.h>

#include "numa.h"

namespace pf {

namespace {
// NVTX range named like the reference's trace span for the same stretch of work.
struct Range {
  explicit Range(const char *name) { nvtxRangePushA(name); }
  ~Range() { nvtxRangePop(); }
  Range(const Range &) = delete;
  Range &operator=(const Range &) = delete;
};
using Clock = std::chrono::steady_clock;

constexpr size_t kReclaimBatch = 512;                      // blocks evicted per reclaim step (storage/mod.rs:32)
constexpr auto kLeaseTtl = std::chrono::seconds(600);      // lease.rs:11
constexpr uint64_t kMaxRunStride = 1ull << 30;             // 2D DMA pitch stays far below its limit

const char *bool_str(bool b) { return b ? "true" : "false"; }

void cuda_or_storage(cudaError_t e, const char *what) {
  if (e != cudaSuccess) throw Error::storage(strf("%s failed: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e)));
}
}  // namespace

const char *phase_name(int phase) {
  static const char *const names[kPhaseCount] = {
      "save.resolve_metadata", "save.hash_filter", "save.pinned_alloc", "save.gpu_copy", "save.queue_wait",
      "gpu.save_task", "gpu.save_task.enqueue", "save.insert_build", "save.insert", "save.flush_wait",
      "query.prefix", "query.create_lease", "load.cache_lookup", "load.build_tasks", "load.queue_wait",
      "gpu.load_task", "gpu.load_task.enqueue"};
  return phase >= 0 && phase < kPhaseCount ? names[phase] : nullptr;
}

Clock::time_point Engine::lap(Phase p, Clock::time_point since) {
  const auto now = Clock::now();
  phase_nanos_[p].fetch_add((uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(now - since).count(),
                            std::memory_order_relaxed);
  phase_calls_[p].fetch_add(1, std::memory_order_relaxed);
  return now;
}

void Engine::phase_times(pf_engine_phase_times *out) {
  for (int i = 0; i < kPhaseCount; ++i) {
    out->seconds[i] = phase_nanos_[i].load() * 1e-9;
    out->calls[i] = phase_calls_[i].load();
  }
}

std::string group_hash(const std::string &hash, uint32_t group) {
  if (group == 0) return hash;
  std::string out = hash;
  for (int shift = 24; shift >= 0; shift -= 8) out.push_back((char)((group >> shift) & 0xFF));
  return out;
}

// ---- ReadCache ---------------------------------------------------------------------------------
bool ReadCache::contains(const BlockKey &key) {
  std::lock_guard<std::mutex> g(mu_);
  return map_.count(key) != 0;
}

BlockRef ReadCache::get(const BlockKey &key, bool touch) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = map_.find(key);
  if (it == map_.end()) return nullptr;
  if (touch) lru_.splice(lru_.begin(), lru_, it->second.pos);
  return it->second.block;
}

bool ReadCache::insert(const BlockKey &key, BlockRef block) {
  std::lock_guard<std::mutex> g(mu_);
  if (map_.count(key)) return false;
  lru_.push_front(key);
  map_.emplace(key, Entry{std::move(block), lru_.begin()});
  return true;
}

void ReadCache::contains_many(const std::string &ns, const std::vector<std::string> &hashes, std::vector<char> *out) {
  out->assign(hashes.size(), 0);
  BlockKey key{ns, ""};
  std::lock_guard<std::mutex> g(mu_);
  for (size_t i = 0; i < hashes.size(); ++i) {
    key.hash = hashes[i];
    (*out)[i] = map_.count(key) ? 1 : 0;
  }
}

size_t ReadCache::evict_lru(size_t n) {
  std::vector<BlockRef> dropped;  // destroyed outside the lock (frees pool memory)
  {
    std::lock_guard<std::mutex> g(mu_);
    // Every resident block is looked at once at most.  A block that someone else still holds (a
    // lease, a load in flight, a handle given to the caller) frees nothing when dropped and must
    // stay findable: it is skipped and its recency refreshed (storage/read_cache.rs:362-389).
    for (size_t candidates = lru_.size(); candidates > 0 && dropped.size() < n; --candidates) {
      auto it = map_.find(lru_.back());
      if (it->second.block.use_count() == 1) {
        dropped.push_back(std::move(it->second.block));
        map_.erase(it);
        lru_.pop_back();
      } else {
        lru_.splice(lru_.begin(), lru_, it->second.pos);
      }
    }
  }
  return dropped.size();
}

std::vector<BlockRef> ReadCache::remove_all() {
  std::vector<BlockRef> out;
  std::lock_guard<std::mutex> g(mu_);
  out.reserve(map_.size());
  for (auto &kv : map_) out.push_back(std::move(kv.second.block));
  map_.clear();
  lru_.clear();
  return out;
}

size_t ReadCache::size() {
  std::lock_guard<std::mutex> g(mu_);
  return map_.size();
}

// ---- RunBuilder --------------------------------------------------------------------------------
void RunBuilder::add(char *host, uint64_t device) {
  const size_t index = next_index_++;
  if (!runs_.empty()) {
    pf_host_run &r = runs_.back();
    char *base = static_cast<char *>(r.host);
    if (r.n_blocks == 1) {
      // The second block fixes the run's stride.
      if (host > base) {
        const uint64_t stride = (uint64_t)(host - base);
        if (stride >= item_bytes_ && stride <= kMaxRunStride && device == r.host_device + stride) {
          r.stride_bytes = stride;
          r.n_blocks = 2;
          return;
        }
      }
    } else if (host == base + r.n_blocks * r.stride_bytes && device == r.host_device + r.n_blocks * r.stride_bytes) {
      ++r.n_blocks;
      return;
    }
  }
  runs_.push_back(pf_host_run{index, 1, host, device, item_bytes_});
}

// ---- topology ----------------------------------------------------------------------------------
size_t LayerTopology::layer_id(const std::string &name) const {
  auto it = name_to_id.find(name);
  if (it == name_to_id.end()) throw Error::invalid("layer " + name + " is not registered");
  return it->second;
}

size_t LayerTopology::group_total_slots(uint32_t group) const {
  if (group >= num_groups())
    throw Error::invalid(strf("storage group %u out of range (%zu groups)", group, num_groups()));
  return page ? page->shard_page_sizes.size() : group_layer_count[group] * tp_size;
}

size_t LayerTopology::slot_index(size_t layer, size_t tp_rank) const {
  if (layer >= num_layers()) throw Error::invalid(strf("layer_id %zu out of range (%zu layers)", layer, num_layers()));
  if (tp_rank >= tp_size) throw Error::invalid(strf("tp_rank %zu out of range (tp_size %zu)", tp_rank, tp_size));
  return page ? page->layer_shard[layer] : layer_group_rank[layer] * tp_size + tp_rank;
}

size_t LayerTopology::shard_layer_count(size_t shard) const {
  return (size_t)std::count(page->layer_shard.begin(), page->layer_shard.end(), shard);
}

// ---- GpuWorker ---------------------------------------------------------------------------------
GpuWorker::GpuWorker(const std::string &name, int device, int numa_node, const pf_backend_config &cfg) : name_(name) {
  std::promise<void> ready;
  std::future<void> ok = ready.get_future();
  thread_ = std::thread(&GpuWorker::loop, this, device, numa_node, cfg, std::move(ready));
  try {
    ok.get();  // rethrows a CudaInit failure from the worker thread
  } catch (...) {
    thread_.join();
    throw;
  }
}

GpuWorker::~GpuWorker() {
  {
    std::lock_guard<std::mutex> g(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
}

void GpuWorker::submit(Task task) {
  {
    std::lock_guard<std::mutex> g(mu_);
    queue_.push_back(std::move(task));
    submitted_.fetch_add(1);
  }
  cv_.notify_one();
}

void GpuWorker::expect_task() {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (!queue_.empty() || expected_) return;  // awake already, or about to be
    expected_ = true;
  }
  cv_.notify_one();
}

void GpuWorker::mark_enqueued(uint64_t ticket) {
  {
    std::lock_guard<std::mutex> g(mu_);
    enqueued_ = std::max(enqueued_, ticket);
  }
  enq_cv_.notify_all();
}

pf_backend_stats GpuWorker::last_stats() {
  std::lock_guard<std::mutex> g(mu_);
  return last_stats_;
}

void GpuWorker::wait_enqueued(uint64_t ticket) {
  std::unique_lock<std::mutex> g(mu_);
  enq_cv_.wait(g, [&] { return enqueued_ >= ticket || stop_; });
}

void GpuWorker::loop(int device, int numa_node, pf_backend_config cfg, std::promise<void> ready) {
  pthread_setname_np(pthread_self(), name_.substr(0, 15).c_str());
  if (numa_node >= 0) numa::pin_thread_to_node(numa_node);  // before any allocation (gpu_worker.rs:148-152)
  std::unique_ptr<TransferBackend> backend;
  cudaStream_t stream = nullptr;
  try {
    // This thread works on one device for its whole life (gpu_worker.rs:278-283).
    if (cudaSetDevice(device) != cudaSuccess)
      throw Error::cuda_init(strf("Failed to create CUDA context: cudaSetDevice(%d) failed", device));
    backend = std::make_unique<TransferBackend>(device, &cfg);
    if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess)
      throw Error::cuda_init("Failed to create CUDA stream");
    ready.set_value();
  } catch (...) {
    ready.set_exception(std::current_exception());
    return;
  }
  uint64_t ticket = 0;
  for (;;) {
    Task task;
    {
      std::unique_lock<std::mutex> g(mu_);
      cv_.wait(g, [&] { return stop_ || !queue_.empty() || expected_; });
      if (queue_.empty() && expected_ && !stop_) {
        // Woken ahead of a task: poll for it without the lock, for half a millisecond at most.
        expected_ = false;
        g.unlock();
        const auto until = std::chrono::steady_clock::now() + std::chrono::microseconds(500);
        while (submitted_.load(std::memory_order_acquire) == ticket && std::chrono::steady_clock::now() < until)
          __builtin_ia32_pause();
        continue;
      }
      expected_ = false;
      if (queue_.empty()) break;
      task = std::move(queue_.front());
      queue_.pop_front();
    }
    current_ticket_ = ++ticket;
    task(*backend, stream);
    pf_backend_stats snap;
    backend->stats(&snap);
    {
      std::lock_guard<std::mutex> g(mu_);
      last_stats_ = snap;
    }
    mark_enqueued(ticket);
  }
  cudaStreamSynchronize(stream);
  backend.reset();
  cudaStreamDestroy(stream);
}

GpuContext::~GpuContext() {
  load_worker.reset();
  save_worker.reset();
  for (auto &kv : load_events) cudaEventDestroy(kv.second);
}

void Completion::signal(bool ok, const std::string &msg) {
  {
    std::lock_guard<std::mutex> g(mu);
    state = ok ? 1 : -1;
    error = msg;
  }
  cv.notify_all();
}

// ---- Engine ------------------------------------------------------------------------------------
Engine::Engine(size_t pool_bytes, bool use_hugepages, const pf_storage_config *config) {
  if (config) cfg_ = *config;
  if (pool_bytes == 0) throw Error::storage("Pinned memory pool size must be greater than zero");
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    throw Error::cuda_init(strf("no CUDA device available (%s)", cudaGetErrorString(e)));
  // lib.rs:144-166: per-node pools only when asked for and the host really has several nodes.
  std::vector<int> nodes;
  if (cfg_.enable_numa_affinity && numa::online_nodes().size() > 1) {
    nodes = numa::gpu_nodes();
    if (nodes.empty()) nodes = numa::online_nodes();
  }
  PinnedMemory::Strategy strategy = use_hugepages     ? PinnedMemory::Strategy::HugePages
                                    : cfg_.use_mmap_pool ? PinnedMemory::Strategy::MmapRegister
                                                         : PinnedMemory::Strategy::CudaHostAlloc;
  allocator_ = std::make_unique<PinnedAllocator>(pool_bytes, nodes, cfg_.pool_shards, strategy, cfg_.hint_value_size);
  if (const char *e = getenv("PEGAFLOW_B200_TRACE")) trace_ = atoi(e) != 0;
  insert_thread_ = std::thread(&Engine::insert_loop, this);
}

Engine::~Engine() {
  {
    std::lock_guard<std::mutex> g(instances_mu_);
    instances_.clear();  // joins the GPU workers (pending async saves hand their batches over first)
  }
  {
    std::lock_guard<std::mutex> g(insert_mu_);
    insert_stop_ = true;
  }
  insert_cv_.notify_all();
  if (insert_thread_.joinable()) insert_thread_.join();
}

std::shared_ptr<InstanceContext> Engine::get_instance(const std::string &id) {
  std::lock_guard<std::mutex> g(instances_mu_);
  auto it = instances_.find(id);
  if (it == instances_.end()) throw Error::instance_missing(id);
  return it->second;
}

std::shared_ptr<LayerTopology> Engine::sealed_topology(InstanceContext &inst) {
  std::lock_guard<std::mutex> g(inst.mu);
  if (!inst.topology)
    throw Error::invalid(strf("instance %s registration incomplete: %zu/%zu workers registered", inst.id.c_str(),
                              inst.gpus.size(), inst.world_size));
  return inst.topology;
}

void Engine::register_context_layer_batch_strided(
    const std::string &instance_id, const std::string &ns, int device_id, size_t tp_rank, size_t pp_rank,
    size_t tp_size, size_t world_size, const std::vector<std::string> &layer_names, const uint64_t *data_ptrs,
    const size_t *size_bytes, const size_t *num_blocks, const size_t *bytes_per_block, const size_t *kv_stride_bytes,
    const size_t *segments, const size_t *block_stride_bytes, const uint32_t *layer_group_ids, int transfer_mode,
    bool page_first) {
  if (transfer_mode != PF_TRANSFER_DIRECT && transfer_mode != PF_TRANSFER_KERNEL)
    throw Error::invalid(strf("unknown transfer mode %d", transfer_mode));
  // Both of the reference's modes map onto the one backend this library has.
  auto gpu = std::make_shared<GpuContext>();
  for (size_t i = 0; i < layer_names.size(); ++i) {
    const std::string &name = layer_names[i];
    try {
      KVCacheLayout layout(data_ptrs[i], size_bytes[i], num_blocks[i], bytes_per_block[i], kv_stride_bytes[i],
                           segments[i]);
      if (block_stride_bytes) layout.set_block_stride(block_stride_bytes[i]);
      layout.set_host_alignment(cfg_.host_alignment);
      if (!gpu->layouts.emplace(name, layout).second)
        throw Error::invalid("duplicate layer name in registration batch: " + name);
    } catch (const LayoutError &e) {
      throw Error::invalid("layer " + name + ": " + e.what());
    }
    if (layer_group_ids) gpu->groups[name] = layer_group_ids[i];
  }

  // lib.rs:193-236 get_or_create_instance
  std::shared_ptr<InstanceContext> inst;
  {
    std::lock_guard<std::mutex> g(instances_mu_);
    auto it = instances_.find(instance_id);
    if (it != instances_.end()) {
      inst = it->second;
      if (inst->tp_size != tp_size || inst->world_size != world_size || inst->page_first != page_first)
        throw Error::topology(strf("instance %s exists with tp=%zu, world=%zu, page_first=%s; requested tp=%zu, "
                                   "world=%zu, page_first=%s",
                                   instance_id.c_str(), inst->tp_size, inst->world_size, bool_str(inst->page_first),
                                   tp_size, world_size, bool_str(page_first)));
    } else {
      if (tp_size == 0 || world_size == 0) throw Error::invalid("tp_size and world_size must be > 0");
      inst = std::make_shared<InstanceContext>();
      inst->id = instance_id;
      inst->ns = ns;
      inst->tp_size = tp_size;
      inst->world_size = world_size;
      inst->page_first = page_first;
      instances_[instance_id] = inst;
    }
  }

  const int numa_node = numa::node_of_device(device_id);
  if (allocator_->is_numa() && numa_node < 0)
    throw Error::invalid(strf("NUMA-aware allocation is enabled, but GPU %d NUMA affinity is unknown. Please ensure "
                              "GPU NUMA topology is detectable, or disable NUMA-aware allocation.",
                              device_id));

  // instance.rs:757-825 register_new_gpu
  if (tp_rank >= inst->tp_size)
    throw Error::invalid(strf("tp_rank %zu out of range (tp_size %zu)", tp_rank, inst->tp_size));
  if (gpu->layouts.empty()) throw Error::invalid(strf("device %d registered no KV cache layers", device_id));
  auto ensure_accepting = [&] {
    if (inst->gpus.count(device_id)) throw Error::invalid(strf("GPU context for device %d already exists", device_id));
    if (inst->topology)
      throw Error::invalid(strf("instance %s is already fully registered (%zu workers); device %d cannot join",
                                inst->id.c_str(), inst->world_size, device_id));
  };
  {
    std::lock_guard<std::mutex> g(inst->mu);
    ensure_accepting();
  }
  if (device_id < 0) throw Error::invalid(strf("device_id %d must be >= 0", device_id));
  gpu->device_id = device_id;
  gpu->tp_rank = tp_rank;
  gpu->pp_rank = pp_rank;
  gpu->numa_node = numa_node;
  const int worker_node = cfg_.enable_numa_affinity ? numa_node : numa::kUnknown;
  gpu->load_worker = std::make_unique<GpuWorker>(strf("gpu%d-load", device_id), device_id, worker_node, cfg_.backend);
  gpu->save_worker = std::make_unique<GpuWorker>(strf("gpu%d-save", device_id), device_id, worker_node, cfg_.backend);
  DeviceGuard on_device(device_id);
  for (auto &kv : gpu->layouts) {
    cudaEvent_t ev;
    cuda_or_storage(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
    gpu->load_events[kv.first] = ev;
  }
  {
    std::lock_guard<std::mutex> g(inst->mu);
    ensure_accepting();
    if (inst->gpus.size() + 1 == inst->world_size) {
      std::vector<std::shared_ptr<GpuContext>> all;
      for (auto &kv : inst->gpus) all.push_back(kv.second);
      all.push_back(gpu);
      inst->topology = seal(*inst, all);
    }
    inst->gpus[device_id] = gpu;
  }
}

// instance.rs:500-672: seal the layer-id space from everything the workers registered.
std::shared_ptr<LayerTopology> Engine::seal(InstanceContext &inst, const std::vector<std::shared_ptr<GpuContext>> &gpus) {
  struct Geometry {
    size_t segment_bytes;
    bool split;
    size_t padded_block_bytes;
    bool operator==(const Geometry &o) const {
      return segment_bytes == o.segment_bytes && split == o.split && padded_block_bytes == o.padded_block_bytes;
    }
  };
  std::map<std::string, Geometry> geometry;  // std::map orders names byte-wise, as the reference sorts them
  for (auto &gpu : gpus) {
    for (auto &kv : gpu->layouts) {
      Geometry g{kv.second.segment_bytes(), kv.second.is_split(), kv.second.padded_block_bytes()};
      auto it = geometry.find(kv.first);
      if (it == geometry.end()) {
        geometry.emplace(kv.first, g);
      } else if (!(it->second == g)) {
        throw Error::invalid(strf(
            "layer %s registered with inconsistent geometry: segment_bytes=%zu split=%s padded_block_bytes=%zu vs "
            "segment_bytes=%zu split=%s padded_block_bytes=%zu on device %d",
            kv.first.c_str(), it->second.segment_bytes, bool_str(it->second.split), it->second.padded_block_bytes,
            g.segment_bytes, bool_str(g.split), g.padded_block_bytes, gpu->device_id));
      }
    }
  }
  auto topo = std::make_shared<LayerTopology>();
  topo->tp_size = inst.tp_size;
  for (auto &kv : geometry) {
    topo->name_to_id[kv.first] = topo->names.size();
    topo->names.push_back(kv.first);
  }
  std::map<std::string, uint32_t> group_by_name;
  for (auto &gpu : gpus) {
    for (auto &kv : gpu->layouts) {
      const uint32_t group = gpu->group_of(kv.first);
      auto it = group_by_name.find(kv.first);
      if (it == group_by_name.end()) {
        group_by_name[kv.first] = group;
      } else if (it->second != group) {
        throw Error::invalid(strf("layer %s registered in storage group %u on one device but group %u on device %d",
                                  kv.first.c_str(), it->second, group, gpu->device_id));
      }
    }
  }
  uint32_t max_group = 0;
  std::set<uint32_t> distinct;
  for (auto &kv : group_by_name) {
    max_group = std::max(max_group, kv.second);
    distinct.insert(kv.second);
  }
  const size_t num_groups = (size_t)max_group + 1;
  if (distinct.size() != num_groups)
    throw Error::invalid(strf("storage groups must be dense 0..%zu: an unregistered group would never seal its blocks",
                              num_groups));
  const size_t n = topo->names.size();
  topo->layer_group.assign(n, 0);
  topo->layer_group_rank.assign(n, 0);
  topo->group_layer_count.assign(num_groups, 0);
  for (size_t id = 0; id < n; ++id) {
    const uint32_t group = group_by_name[topo->names[id]];
    topo->layer_group[id] = group;
    topo->layer_group_rank[id] = topo->group_layer_count[group]++;
  }
  if (inst.page_first && num_groups > 1)
    throw Error::invalid(strf("page-first storage does not support multiple storage groups (%zu registered)", num_groups));

  // Every (layer, tp_rank) needs an owner; replicas may only differ in device.
  struct Owner {
    bool set = false;
    int device = 0;
    size_t pp_rank = 0;
  };
  std::vector<Owner> owners(n * inst.tp_size);
  for (auto &gpu : gpus) {
    for (auto &kv : gpu->layouts) {
      Owner &o = owners[topo->name_to_id[kv.first] * inst.tp_size + gpu->tp_rank];
      if (!o.set) {
        o = Owner{true, gpu->device_id, gpu->pp_rank};
      } else if (o.pp_rank != gpu->pp_rank) {
        throw Error::invalid(strf("layer %s claimed by different pipeline stages: device=%d pp_rank=%zu; device=%d "
                                  "pp_rank=%zu tp_rank=%zu",
                                  kv.first.c_str(), o.device, o.pp_rank, gpu->device_id, gpu->pp_rank, gpu->tp_rank));
      }
    }
  }
  for (size_t i = 0; i < owners.size(); ++i)
    if (!owners[i].set)
      throw Error::invalid(strf("instance %s has incomplete KV registration: layer %s has no owner for tp_rank %zu "
                                "after all %zu workers registered",
                                inst.id.c_str(), topo->names[i / inst.tp_size].c_str(), i % inst.tp_size,
                                inst.world_size));
  if (inst.page_first) {
    std::vector<std::vector<size_t>> sets;
    for (auto &gpu : gpus) {
      std::vector<size_t> ids;
      for (auto &kv : gpu->layouts) ids.push_back(topo->name_to_id[kv.first]);
      sets.push_back(std::move(ids));
    }
    std::vector<size_t> padded;
    for (auto &name : topo->names) padded.push_back(geometry[name].padded_block_bytes);
    try {
      topo->page = build_page_layout(sets, n, padded, &topo->names);
    } catch (const LayoutError &e) {
      throw Error::invalid(e.what());
    }
  }
  return topo;
}

void Engine::unregister_instance(const std::string &instance_id) {
  std::shared_ptr<InstanceContext> inst;
  {
    std::lock_guard<std::mutex> g(instances_mu_);
    auto it = instances_.find(instance_id);
    if (it == instances_.end()) throw Error::instance_missing(instance_id);
    inst = it->second;
    instances_.erase(it);
  }
  {
    std::lock_guard<std::mutex> g(leases_mu_);
    for (auto it = leases_.begin(); it != leases_.end();)
      it = it->second.instance_id == instance_id ? leases_.erase(it) : std::next(it);
  }
  inst.reset();  // last reference: joins the instance's GPU workers
}

// lib.rs:938-948, storage/write_path.rs: the background sweep of blocks that never got all their slots.
size_t Engine::gc_stale_inflight(double max_age_seconds) {
  std::vector<Inflight> stale;  // destroyed outside the lock (frees pool memory)
  {
    const auto now = std::chrono::steady_clock::now();
    std::lock_guard<std::mutex> g(inflight_mu_);
    for (auto it = inflight_.begin(); it != inflight_.end();) {
      if (std::chrono::duration<double>(now - it->second.created).count() > max_age_seconds) {
        stale.push_back(std::move(it->second));
        it = inflight_.erase(it);
      } else {
        ++it;
      }
    }
  }
  return stale.size();
}

// lib.rs:459-475
std::vector<std::string> Engine::unregister_all_instances() {
  std::vector<std::shared_ptr<InstanceContext>> gone;
  std::vector<std::string> ids;
  {
    std::lock_guard<std::mutex> g(instances_mu_);
    for (auto &kv : instances_) {
      ids.push_back(kv.first);
      gone.push_back(std::move(kv.second));
    }
    instances_.clear();
  }
  {
    std::lock_guard<std::mutex> g(leases_mu_);
    leases_.clear();  // every lease belongs to an instance that is gone now
  }
  gone.clear();  // last references: joins the instances' GPU workers
  std::sort(ids.begin(), ids.end());
  return ids;
}

// lib.rs:477-484
std::vector<std::string> Engine::list_instance_ids() {
  std::vector<std::string> ids;
  {
    std::lock_guard<std::mutex> g(instances_mu_);
    for (auto &kv : instances_) ids.push_back(kv.first);
  }
  std::sort(ids.begin(), ids.end());
  return ids;
}

// lib.rs:487-489
std::string Engine::instance_namespace(const std::string &instance_id) { return get_instance(instance_id)->ns; }

// storage/mod.rs:294-330: allocate, evicting least recently used blocks until it fits.
std::shared_ptr<PinnedAllocation> Engine::allocate(uint64_t bytes, int numa_node, const char *what) {
  for (;;) {
    if (auto a = allocator_->allocate(bytes, numa_node)) return a;
    const size_t dropped = cache_.evict_lru(kReclaimBatch);
    if (dropped == 0) break;
    evicted_.fetch_add(dropped);
  }
  alloc_failures_.fetch_add(1);
  throw Error::storage(std::string("pinned pool exhausted while allocating ") + what);
}

void Engine::batch_save(const std::string &instance_id, size_t tp_rank, size_t pp_rank, int device_id,
                        std::vector<LayerSaveIn> saves, bool async, cudaEvent_t ready_event) {
  sweep_leases();
  const auto t0 = std::chrono::steady_clock::now();
  auto inst = get_instance(instance_id);
  auto topo = sealed_topology(*inst);

  // ---- phase 0: resolve layout / slot / group, validate ids (offload.rs:313-378)
  nvtxRangePushA("save.resolve_metadata");
  std::shared_ptr<GpuContext> gpu;
  {
    std::lock_guard<std::mutex> g(inst->mu);
    auto it = inst->gpus.find(device_id);
    if (it == inst->gpus.end()) throw Error::worker_missing(instance_id, device_id);
    gpu = it->second;
  }
  gpu->save_worker->expect_task();
  if (gpu->tp_rank != tp_rank || gpu->pp_rank != pp_rank)
    throw Error::invalid(strf("device_id %d is registered for tp_rank %zu, pp_rank %zu, but save requested tp_rank "
                              "%zu, pp_rank %zu",
                              device_id, gpu->tp_rank, gpu->pp_rank, tp_rank, pp_rank));
  struct Ctx {
    std::string name;
    const KVCacheLayout *layout;
    size_t slot;
    uint32_t group;
    std::vector<size_t> ids;
    HashList hashes;  // phase 0: as given; after phase 1: group-encoded and filtered
    std::vector<RawBlock> raw;
  };
  std::vector<Ctx> ctxs;
  for (auto &s : saves) {
    const size_t n_hashes = s.block_hashes ? s.block_hashes->size() : 0;
    if (s.block_ids.size() != n_hashes)
      throw Error::invalid(strf("block_ids length %zu does not match block_hashes %zu for layer %s", s.block_ids.size(),
                                n_hashes, s.layer_name.c_str()));
    const size_t layer_id = topo->layer_id(s.layer_name);
    auto lit = gpu->layouts.find(s.layer_name);
    if (lit == gpu->layouts.end()) throw Error::invalid("layer " + s.layer_name + " not registered on device");
    const size_t slot = topo->slot_index(layer_id, tp_rank);
    const uint32_t group = topo->layer_group[layer_id];
    for (size_t id : s.block_ids)
      if (id >= lit->second.num_blocks())
        throw Error::invalid(strf("block_id %zu out of range (num_blocks=%zu) for layer %s", id,
                                  lit->second.num_blocks(), s.layer_name.c_str()));
    if (s.block_ids.empty()) continue;
    ctxs.push_back(Ctx{s.layer_name, &lit->second, slot, group, std::move(s.block_ids), s.block_hashes, {}});
  }
  nvtxRangePop();
  if (ctxs.empty()) return;
  const auto t1 = lap(kSaveResolve, t0);

  // ---- phase 1: drop blocks whose (group, hash) is already resident (offload.rs:393-424).
  // Layers of one save normally share one hash list: each distinct (list, group) is encoded and
  // looked up once and the result is shared.
  {
    Range nvtx("save.hash_filter");
    struct Filtered {
      HashList hashes;                 // group-encoded, resident ones removed
      std::vector<uint32_t> kept;      // positions that survive (empty + all_kept: every position)
      bool all_kept = false;
    };
    std::map<std::pair<const void *, uint32_t>, Filtered> memo;
    size_t total = 0;
    for (auto &c : ctxs) {
      auto key = std::make_pair((const void *)c.hashes.get(), c.group);
      auto it = memo.find(key);
      if (it == memo.end()) {
        auto encoded = std::make_shared<std::vector<std::string>>();
        encoded->reserve(c.hashes->size());
        for (auto &h : *c.hashes) encoded->push_back(group_hash(h, c.group));
        std::vector<char> resident;
        cache_.contains_many(inst->ns, *encoded, &resident);
        Filtered f;
        if (std::find(resident.begin(), resident.end(), 1) == resident.end()) {
          f.all_kept = true;
          f.hashes = std::move(encoded);
        } else {
          auto survivors = std::make_shared<std::vector<std::string>>();
          for (size_t i = 0; i < encoded->size(); ++i)
            if (!resident[i]) {
              f.kept.push_back((uint32_t)i);
              survivors->push_back(std::move((*encoded)[i]));
            }
          f.hashes = std::move(survivors);
        }
        it = memo.emplace(key, std::move(f)).first;
      }
      const Filtered &f = it->second;
      if (!f.all_kept) {
        std::vector<size_t> ids;
        ids.reserve(f.kept.size());
        for (uint32_t i : f.kept) ids.push_back(c.ids[i]);
        c.ids.swap(ids);
      }
      c.hashes = f.hashes;
      total += c.ids.size();
    }
    ctxs.erase(std::remove_if(ctxs.begin(), ctxs.end(), [](const Ctx &c) { return c.ids.empty(); }), ctxs.end());
    if (total == 0 || ctxs.empty()) return;
  }
  const auto t2 = lap(kSaveHashFilter, t1);

  // ---- phase 2: host placement (offload.rs:428-527, 182-282).  Only what the GPU copy needs is
  // built here (allocations, block ids, host runs); the per-block bookkeeping for the cache is
  // built after the copy has been submitted, while it runs.
  nvtxRangePushA("save.pinned_alloc");
  struct PopRange {
    bool armed = true;
    ~PopRange() {
      if (armed) nvtxRangePop();
    }
  } alloc_range;
  const int numa_node = gpu->numa_node;
  const bool page_first = topo->page.has_value();
  const bool blockwise = cfg_.blockwise_alloc != 0 && !page_first;
  auto work = std::make_shared<std::vector<LayerWork>>();
  auto all_allocs = std::make_shared<std::vector<std::shared_ptr<PinnedAllocation>>>();
  // Everything the GPU copy writes into: the worker's task holds it, so the pool ranges outlive the
  // copy even when this call unwinds early.
  auto copy_targets = std::make_shared<std::vector<std::shared_ptr<PinnedAllocation>>>();
  std::vector<std::shared_ptr<PinnedAllocation>> pages;
  // allocs[c][a] = (K-or-whole, V) allocation a of layer context c
  std::vector<std::vector<std::array<std::shared_ptr<PinnedAllocation>, 2>>> layer_allocs(ctxs.size());
  size_t padded_total = 0;
  work->reserve(ctxs.size());
  if (page_first) {
    const size_t shard = ctxs[0].slot;
    const size_t page_size = topo->page->shard_page_sizes[shard];
    std::set<size_t> layer_ids;
    for (auto &c : ctxs) {
      if (c.layout->is_split())
        throw Error::invalid("page-first save does not support split K/V (layer " + c.name + ")");
      if (c.slot != shard)
        throw Error::invalid("page-first save spans multiple shards (one writer must save one shard)");
      if (c.ids != ctxs[0].ids || (c.hashes != ctxs[0].hashes && *c.hashes != *ctxs[0].hashes))
        throw Error::invalid("page-first save requires the same block set across all layers");
      layer_ids.insert(topo->layer_id(c.name));
    }
    const size_t shard_layers = topo->shard_layer_count(shard);
    if (layer_ids.size() != shard_layers)
      throw Error::invalid(strf("page-first save must cover all %zu layers of shard %zu, got %zu distinct (one worker "
                                "must write a shard's entire page)",
                                shard_layers, shard, layer_ids.size()));
    if (page_size == 0) throw Error::storage("page size is zero");
    pages.reserve(ctxs[0].ids.size());
    for (size_t i = 0; i < ctxs[0].ids.size(); ++i) pages.push_back(allocate(page_size, numa_node, "page"));
    *copy_targets = pages;
    for (auto &c : ctxs) {
      const size_t layer_id = topo->layer_id(c.name);
      const size_t offset = topo->page->layer_offsets[layer_id];
      LayerWork w;
      w.layer_name = c.name;
      w.layout = *c.layout;
      w.block_ids.reserve(c.ids.size());
      RunBuilder rb(c.layout->range_bytes());
      for (size_t i = 0; i < c.ids.size(); ++i) {
        w.block_ids.push_back((uint32_t)c.ids[i]);
        rb.add(pages[i]->host() + offset, pages[i]->device() + offset);
      }
      w.runs[0] = rb.take();
      work->push_back(std::move(w));
    }
    padded_total = page_size * pages.size();
  } else {
    for (size_t ci = 0; ci < ctxs.size(); ++ci) {
      Ctx &c = ctxs[ci];
      const KVCacheLayout &layout = *c.layout;
      const size_t n = c.ids.size();
      const size_t n_allocs = blockwise ? n : 1, per = blockwise ? 1 : n;
      LayerWork w;
      w.layer_name = c.name;
      w.layout = layout;
      w.block_ids.reserve(n);
      for (size_t id : c.ids) w.block_ids.push_back((uint32_t)id);
      const bool split = layout.is_split();
      const size_t stride = split ? layout.padded_segment_bytes() : layout.padded_block_bytes();
      layer_allocs[ci].reserve(n_allocs);
      for (size_t a = 0; a < n_allocs; ++a) {
        std::array<std::shared_ptr<PinnedAllocation>, 2> pair;
        pair[0] = allocate(stride * per, numa_node, split ? "K segment buffer" : "block buffer");
        if (split) pair[1] = allocate(stride * per, numa_node, "V segment buffer");
        for (int r = 0; r < (split ? 2 : 1); ++r) {
          // one run per allocation; neighbouring allocations that happen to continue it are merged
          auto &runs = w.runs[r];
          if (!runs.empty() && (char *)runs.back().host + runs.back().n_blocks * runs.back().stride_bytes == pair[r]->host() &&
              runs.back().host_device + runs.back().n_blocks * runs.back().stride_bytes == pair[r]->device() &&
              runs.back().stride_bytes == stride)
            runs.back().n_blocks += per;
          else
            runs.push_back(pf_host_run{a * per, per, pair[r]->host(), pair[r]->device(), stride});
        }
        copy_targets->push_back(pair[0]);
        if (split) copy_targets->push_back(pair[1]);
        if (!blockwise) {
          all_allocs->push_back(pair[0]);
          if (split) all_allocs->push_back(pair[1]);
        }
        layer_allocs[ci].push_back(std::move(pair));
      }
      padded_total += layout.padded_block_bytes() * n;
      work->push_back(std::move(w));
    }
  }
  nvtxRangePop();
  alloc_range.armed = false;
  const auto t3 = lap(kSavePinnedAlloc, t2);

  // ---- phase 3: one GPU batch (offload.rs:532-536 -> gpu_worker.rs:482-523)
  auto done = std::make_shared<std::promise<void>>();
  std::future<void> finished = done->get_future();
  auto batches_ready = std::make_shared<std::promise<std::shared_ptr<std::vector<RawSaveBatch>>>>();
  auto batches_future = batches_ready->get_future().share();
  {
    std::lock_guard<std::mutex> g(insert_mu_);
    ++insert_pending_;  // until the batches have been handed to the insert worker
  }
  auto hand_over = [this, batches_future] {
    auto batches = batches_future.get();
    std::lock_guard<std::mutex> g(insert_mu_);
    if (batches)
      for (auto &b : *batches) {
        insert_queue_.push_back(std::move(b));
        ++insert_pending_;
      }
    --insert_pending_;
    insert_cv_.notify_all();
    insert_idle_cv_.notify_all();
  };
  auto abandon = [this] {
    std::lock_guard<std::mutex> g(insert_mu_);
    --insert_pending_;
    insert_idle_cv_.notify_all();
  };
  gpu->save_worker->submit([=](TransferBackend &backend, cudaStream_t stream) {
    Range nvtx("gpu.save_task");
    const auto w0 = lap(kSaveQueueWait, t3);
    try {
      std::vector<pf_layer_xfer> xf(work->size());
      for (size_t i = 0; i < work->size(); ++i) {
        LayerWork &w = (*work)[i];
        xf[i] = pf_layer_xfer{w.layout.data_ptr(), w.layout.block_stride_bytes(), w.layout.kv_stride_bytes(),
                              w.layout.range_bytes(), w.layout.n_ranges(), w.block_ids.size(), w.block_ids.data(),
                              {w.runs[0].size(), w.runs[1].size()}, {w.runs[0].data(), w.runs[1].data()}};
      }
      if (ready_event) cuda_or_storage(cudaStreamWaitEvent(stream, ready_event, 0), "cudaStreamWaitEvent");
      backend.move_layers(xf.data(), xf.size(), false, stream, nullptr);
      lap(kSaveEnqueue, w0);
      cuda_or_storage(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
      lap(kSaveTask, w0);
      (void)copy_targets;
      if (async) hand_over();
      done->set_value();
    } catch (const std::exception &e) {
      if (async) {
        // Nobody waits on an asynchronous save: keep the failure for the next flush_saves().
        {
          std::lock_guard<std::mutex> g(insert_mu_);
          if (async_error_.empty()) async_error_ = e.what();
        }
        abandon();
      }
      done->set_exception(std::current_exception());
    }
  });

  // ---- phase 4 input, built while the copy runs: one RawBlock per (layer, block) and the
  // batches the insert worker will seal (offload.rs:594-656).
  try {
    Range nvtx("save.insert_build");
    auto batches = std::make_shared<std::vector<RawSaveBatch>>();
    if (page_first) {
      const size_t slot = ctxs[0].slot;
      const size_t page_size = topo->page->shard_page_sizes[slot];
      RawSaveLayer layer;
      layer.slot_id = slot;
      layer.hashes = ctxs[0].hashes;
      layer.blocks.reserve(pages.size());
      for (auto &page : pages) {
        RawBlock rbk;
        rbk.n_segments = 1;
        rbk.seg[0] = Segment{page->host(), page->device(), page_size};
        rbk.owner = page;  // a page lives and dies with its block
        layer.blocks.push_back(std::move(rbk));
      }
      RawSaveBatch b{inst->ns, topo->total_slots(), {}, nullptr, {}, nullptr};
      b.layers.push_back(std::move(layer));
      batches->push_back(std::move(b));
    } else {
      std::map<uint32_t, RawSaveBatch> by_group;
      const Owner batch_owner = blockwise ? Owner() : Owner(all_allocs);
      // Which groups this save seals on its own: it brings every slot of the group exactly once and
      // all its layers carry one hash list.
      std::map<uint32_t, std::vector<size_t>> ctx_of_group;
      for (size_t ci = 0; ci < ctxs.size(); ++ci) ctx_of_group[ctxs[ci].group].push_back(ci);
      std::set<uint32_t> seals_alone;
      for (auto &kv : ctx_of_group) {
        const size_t total = topo->group_total_slots(kv.first);
        std::vector<char> seen(total, 0);
        bool ok = kv.second.size() == total;
        for (size_t ci : kv.second) {
          const Ctx &c = ctxs[ci];
          ok = ok && c.hashes.get() == ctxs[kv.second[0]].hashes.get() && c.slot < total && !seen[c.slot];
          if (ok) seen[c.slot] = 1;
        }
        if (ok) seals_alone.insert(kv.first);
      }
      for (size_t ci = 0; ci < ctxs.size(); ++ci) {
        Ctx &c = ctxs[ci];
        auto it = by_group.find(c.group);
        if (it == by_group.end())
          it = by_group.emplace(c.group, RawSaveBatch{inst->ns, topo->group_total_slots(c.group), {}, batch_owner, {}, nullptr}).first;
        RawSaveBatch &batch = it->second;
        const bool split = c.layout->is_split();
        const size_t stride = split ? c.layout->padded_segment_bytes() : c.layout->padded_block_bytes();
        const size_t per = blockwise ? 1 : c.ids.size();
        const bool presealed = seals_alone.count(c.group) != 0;
        RawSaveLayer layer;
        if (presealed) {
          if (batch.sealed.empty()) {
            batch.sealed_hashes = c.hashes;  // already group-encoded
            batch.sealed.resize(c.ids.size());
            for (auto &sb : batch.sealed) {
              sb = std::make_shared<SealedBlock>();
              sb->owner = batch_owner;
              sb->slots.resize(batch.total_slots);
            }
          }
        } else {
          layer.slot_id = c.slot;
          layer.hashes = c.hashes;  // already group-encoded
          layer.blocks.resize(c.ids.size());
        }
        for (size_t a = 0; a < layer_allocs[ci].size(); ++a) {
          auto &pair = layer_allocs[ci][a];
          Owner own;
          if (blockwise) own = split ? Owner(std::make_shared<std::array<std::shared_ptr<PinnedAllocation>, 2>>(pair))
                                     : Owner(pair[0]);
          for (size_t i = 0; i < per; ++i) {
            RawBlock &rbk = presealed ? batch.sealed[a * per + i]->slots[c.slot] : layer.blocks[a * per + i];
            rbk.n_segments = split ? 2 : 1;
            rbk.seg[0] = Segment{pair[0]->host() + i * stride, pair[0]->device() + i * stride, stride};
            if (split) rbk.seg[1] = Segment{pair[1]->host() + i * stride, pair[1]->device() + i * stride, stride};
            rbk.owner = own;
            if (presealed) batch.sealed[a * per + i]->footprint += rbk.total_size();
          }
        }
        if (!presealed) batch.layers.push_back(std::move(layer));
      }
      for (auto &kv : by_group) batches->push_back(std::move(kv.second));
    }
    batches_ready->set_value(std::move(batches));
    lap(kSaveInsertBuild, t3);
  } catch (...) {
    batches_ready->set_value(nullptr);
    if (!async) {
      try {
        finished.get();
      } catch (...) {
      }
      abandon();
    }
    throw;
  }
  if (async) {
    save_bytes_.fetch_add(padded_total);
    save_batches_.fetch_add(1);
    return;
  }
  try {
    Range nvtx("save.gpu_copy");
    finished.get();
  } catch (...) {
    abandon();
    throw;
  }
  save_bytes_.fetch_add(padded_total);
  save_batches_.fetch_add(1);
  const auto t4 = lap(kSaveGpuCopy, t3);
  save_nanos_.fetch_add((uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(t4 - t0).count());
  hand_over();
  if (trace_) {
    auto ms = [](auto a, auto b) { return std::chrono::duration<double, std::milli>(b - a).count(); };
    fprintf(stderr, "[pegaflow_b200] save %s: resolve %.2f ms, hash_filter %.2f ms, pinned_alloc %.2f ms, gpu_copy %.2f ms\n",
            instance_id.c_str(), ms(t0, t1), ms(t1, t2), ms(t2, t3), ms(t3, t4));
  }
}

void Engine::flush_saves() {
  const auto t0 = Clock::now();
  std::unique_lock<std::mutex> g(insert_mu_);
  insert_idle_cv_.wait(g, [&] { return insert_pending_ == 0; });
  lap(kFlushWait, t0);
  if (!async_error_.empty()) {
    std::string msg;
    msg.swap(async_error_);
    throw Error(PF_STORAGE, msg.rfind("storage error: ", 0) == 0 ? msg : "storage error: asynchronous save failed: " + msg);
  }
}

void Engine::insert_loop() {
  pthread_setname_np(pthread_self(), "pf-insert");
  for (;;) {
    RawSaveBatch batch;
    {
      std::unique_lock<std::mutex> g(insert_mu_);
      insert_cv_.wait(g, [&] { return insert_stop_ || !insert_queue_.empty(); });
      if (insert_queue_.empty()) return;
      batch = std::move(insert_queue_.front());
      insert_queue_.pop_front();
    }
    {
      const auto t0 = Clock::now();
      process_insert(batch);
      lap(kSaveInsert, t0);
    }
    {
      std::lock_guard<std::mutex> g(insert_mu_);
      --insert_pending_;
    }
    insert_idle_cv_.notify_all();
  }
}

// storage/write_path.rs:119-254 + offload.rs:70-151.
void Engine::process_insert(RawSaveBatch &batch) {
  std::lock_guard<std::mutex> inflight_guard(inflight_mu_);
  if (!batch.sealed.empty()) {
    // sealed by the save itself while its copy ran: publish
    const auto &hashes = *batch.sealed_hashes;
    for (size_t b = 0; b < batch.sealed.size(); ++b) {
      BlockKey key{batch.ns, hashes[b]};
      if (cache_.contains(key) || inflight_.count(key)) {
        // someone else is filling or has filled this block: slot by slot, first writer wins
        for (size_t slot = 0; slot < batch.sealed[b]->slots.size(); ++slot)
          insert_slot(key, slot, std::move(batch.sealed[b]->slots[slot]), batch.total_slots, batch.owner);
        continue;
      }
      cache_.insert(key, std::move(batch.sealed[b]));
    }
    return;
  }
  if (batch.layers.empty()) return;
  bool same_order = true;
  for (auto &l : batch.layers)
    if (l.hashes != batch.layers[0].hashes && *l.hashes != *batch.layers[0].hashes) same_order = false;
  if (same_order && batch.layers.size() == batch.total_slots) {
    // Every layer carries the same hashes in the same order and together they fill every
    // slot: seal block by block without touching the inflight map.
    std::vector<size_t> slot_of(batch.layers.size());
    std::vector<char> seen(batch.total_slots, 0);
    bool distinct = true;
    for (size_t l = 0; l < batch.layers.size(); ++l) {
      slot_of[l] = batch.layers[l].slot_id;
      if (slot_of[l] >= batch.total_slots || seen[slot_of[l]]) distinct = false;
      else seen[slot_of[l]] = 1;
    }
    if (distinct) {
      const auto &hashes = *batch.layers[0].hashes;
      for (size_t b = 0; b < hashes.size(); ++b) {
        BlockKey key{batch.ns, hashes[b]};
        if (cache_.contains(key) || inflight_.count(key)) {
          for (size_t l = 0; l < batch.layers.size(); ++l)
            insert_slot(key, slot_of[l], std::move(batch.layers[l].blocks[b]), batch.total_slots, batch.owner);
          continue;
        }
        auto sealed = std::make_shared<SealedBlock>();
        sealed->owner = batch.owner;
        sealed->slots.resize(batch.total_slots);
        for (size_t l = 0; l < batch.layers.size(); ++l) {
          sealed->footprint += batch.layers[l].blocks[b].total_size();
          sealed->slots[slot_of[l]] = std::move(batch.layers[l].blocks[b]);
        }
        cache_.insert(key, std::move(sealed));
      }
      return;
    }
  }
  for (auto &l : batch.layers)
    for (size_t b = 0; b < l.hashes->size(); ++b)
      insert_slot(BlockKey{batch.ns, (*l.hashes)[b]}, l.slot_id, std::move(l.blocks[b]), batch.total_slots, batch.owner);
}

void Engine::insert_slot(const BlockKey &key, size_t slot, RawBlock block, size_t total_slots,
                         const Owner &batch_owner) {
  if (cache_.contains(key)) return;  // late duplicate of a resident block
  if (!block.owner) block.owner = batch_owner;  // slots of one block may come from different saves
  auto it = inflight_.find(key);
  if (it == inflight_.end()) {
    Inflight fresh;
    fresh.total_slots = total_slots;
    fresh.slots.resize(total_slots);
    it = inflight_.emplace(key, std::move(fresh)).first;
  }
  Inflight &inf = it->second;
  if (inf.total_slots != total_slots || slot >= total_slots) return;  // incompatible writer: ignored
  if (inf.slots[slot].has_value()) return;                           // duplicate slot: first one wins
  inf.slots[slot] = std::move(block);
  if (++inf.filled == inf.total_slots) {
    auto sealed = std::make_shared<SealedBlock>();
    sealed->slots.reserve(total_slots);
    for (auto &s : inf.slots) {
      sealed->footprint += s->total_size();
      sealed->slots.push_back(std::move(*s));
    }
    inflight_.erase(it);
    cache_.insert(key, std::move(sealed));
  }
}

void Engine::query_prefix(const std::string &instance_id, const std::vector<std::string> &hashes,
                          std::vector<BlockRef> *blocks, size_t *missing) {
  const auto t0 = Clock::now();
  auto inst = get_instance(instance_id);
  blocks->clear();
  for (auto &h : hashes) {
    BlockRef b = cache_.get(BlockKey{inst->ns, h}, true);
    if (!b) break;
    blocks->push_back(std::move(b));
  }
  *missing = hashes.size() - blocks->size();
  lap(kQueryPrefix, t0);
}

std::vector<BlockRef> Engine::query_group_membership(const std::string &instance_id, uint32_t group,
                                                     const std::vector<std::string> &hashes) {
  auto inst = get_instance(instance_id);
  auto topo = sealed_topology(*inst);
  topo->group_total_slots(group);  // unknown group is a caller bug, not "all miss"
  std::vector<BlockRef> out;
  for (auto &h : hashes) out.push_back(cache_.get(BlockKey{inst->ns, group_hash(h, group)}, true));
  return out;
}

void Engine::sweep_leases() {
  const auto now = std::chrono::steady_clock::now();
  std::lock_guard<std::mutex> g(leases_mu_);
  for (auto it = leases_.begin(); it != leases_.end();) it = it->second.expires <= now ? leases_.erase(it) : std::next(it);
}

std::array<uint8_t, 16> Engine::create_query_lease(const std::string &instance_id, std::vector<BlockRef> blocks) {
  const auto t0 = Clock::now();
  auto inst = get_instance(instance_id);
  if (blocks.empty()) throw Error::invalid("query lease requires at least one block");
  sweep_leases();
  std::array<uint8_t, 16> token;
  std::random_device rd;
  for (int i = 0; i < 16; i += 4) {
    uint32_t v = rd();
    memcpy(token.data() + i, &v, 4);
  }
  std::lock_guard<std::mutex> g(leases_mu_);
  leases_[token] = Lease{instance_id, std::move(blocks), std::max<size_t>(1, inst->world_size),
                         std::chrono::steady_clock::now() + kLeaseTtl};
  lap(kCreateLease, t0);
  return token;
}

bool Engine::release_query_lease(const std::array<uint8_t, 16> &lease) {
  sweep_leases();
  std::lock_guard<std::mutex> g(leases_mu_);
  return leases_.erase(lease) != 0;
}

// lease.rs:98-133: every worker of the instance consumes the lease once.
std::vector<BlockRef> Engine::consume_lease(const std::string &instance_id, const std::array<uint8_t, 16> &lease) {
  sweep_leases();
  std::lock_guard<std::mutex> g(leases_mu_);
  auto it = leases_.find(lease);
  if (it == leases_.end()) throw Error::storage("query lease is unknown or expired");
  if (it->second.instance_id != instance_id)
    throw Error::storage("query lease belongs to instance " + it->second.instance_id + ", got " + instance_id);
  if (it->second.remaining > 1) {
    --it->second.remaining;
    return it->second.blocks;
  }
  std::vector<BlockRef> blocks = std::move(it->second.blocks);
  leases_.erase(it);
  return blocks;
}

void Engine::batch_load(const std::string &instance_id, size_t tp_rank, int device_id,
                        const std::vector<std::vector<std::string>> &layer_groups,
                        const std::vector<LeaseLoadIn> &loads, const std::string &shm_name,
                        std::shared_ptr<Completion> completion) {
  // lib.rs:654-680: the LoadState must be attachable before anything else happens, and a
  // failure before submission flips it to ERROR.
  std::shared_ptr<LoadState> shm_state;
  if (!completion) shm_state.reset(LoadState::attach(shm_name));
  auto signal = [shm_state, completion](bool ok, const std::string &msg) {
    if (completion) completion->signal(ok, msg);
    else if (ok) shm_state->set_completed();
    else shm_state->set_error();
  };
  const auto t_begin = std::chrono::steady_clock::now();
  try {
    auto inst = get_instance(instance_id);
    auto topo = sealed_topology(*inst);
    std::shared_ptr<GpuContext> gpu;
    {
      std::lock_guard<std::mutex> g(inst->mu);
      auto it = inst->gpus.find(device_id);
      if (it == inst->gpus.end()) throw Error::worker_missing(instance_id, device_id);
      gpu = it->second;
    }
    gpu->load_worker->expect_task();
    if (layer_groups.empty()) throw Error::invalid("load requires at least one layer group");
    {
      std::unordered_set<std::string> unique;
      size_t count = 0;
      for (auto &g : layer_groups)
        for (auto &n : g) {
          unique.insert(n);
          ++count;
        }
      if (unique.size() != count) throw Error::invalid("load layer names must be unique across groups");
    }
    std::vector<std::optional<uint32_t>> storage_group;
    for (auto &names : layer_groups) {
      std::optional<uint32_t> group;
      for (auto &name : names) {
        const uint32_t lg = topo->layer_group[topo->layer_id(name)];
        if (!group) group = lg;
        else if (*group != lg)
          throw Error::invalid(strf("load group mixes storage groups %u and %u (layer %s)", *group, lg, name.c_str()));
      }
      storage_group.push_back(group);
    }
    // consume the leases; targets per group are (destination block, index into block_cache)
    std::vector<std::vector<std::pair<size_t, size_t>>> targets(layer_groups.size());
    std::vector<BlockRef> block_cache;
    for (auto &ld : loads) {
      std::vector<BlockRef> blocks = consume_lease(instance_id, ld.lease);
      if (ld.dst_ids.size() != layer_groups.size())
        throw Error::invalid(strf("load group count %zu does not match layer group count %zu", ld.dst_ids.size(),
                                  layer_groups.size()));
      const size_t start = block_cache.size();
      for (size_t gi = 0; gi < ld.dst_ids.size(); ++gi) {
        const auto &dst = ld.dst_ids[gi];
        if (blocks.size() != dst.size())
          throw Error::invalid(strf("query lease block count %zu does not match destination block count %zu for "
                                    "group %zu",
                                    blocks.size(), dst.size(), gi));
        if (storage_group[gi]) {
          const size_t expected = topo->group_total_slots(*storage_group[gi]);
          for (size_t si = 0; si < dst.size(); ++si)
            if (dst[si] != PF_NO_BLOCK && blocks[si]->slots.size() != expected)
              throw Error::invalid(strf("stored block has %zu slots but storage group %u of instance %s expects "
                                        "%zu: namespace is shared by incompatible KV layouts",
                                        blocks[si]->slots.size(), *storage_group[gi], instance_id.c_str(), expected));
        }
        for (size_t si = 0; si < dst.size(); ++si)
          if (dst[si] != PF_NO_BLOCK) targets[gi].emplace_back(dst[si], start + si);
      }
      for (auto &b : blocks) block_cache.push_back(std::move(b));
    }
    const auto t_lookup = lap(kLoadCacheLookup, t_begin);
    // per layer work (lib.rs:836-888 + gpu_worker.rs:353-423 pairing)
    Range nvtx_build("load.build_tasks");
    auto work = std::make_shared<std::vector<LayerWork>>();
    for (size_t gi = 0; gi < layer_groups.size(); ++gi) {
      if (targets[gi].empty()) continue;
      // what each layer of the group needs from a stored block
      struct PerLayer {
        const std::string *name;
        const KVCacheLayout *layout;
        size_t slot, offset;
      };
      std::vector<PerLayer> per;
      for (auto &name : layer_groups[gi]) {
        const size_t layer_id = topo->layer_id(name);
        auto lit = gpu->layouts.find(name);
        if (lit == gpu->layouts.end())
          throw Error::invalid(strf("layer %s not registered on device %d", name.c_str(), device_id));
        per.push_back(PerLayer{&name, &lit->second, topo->slot_index(layer_id, tp_rank),
                               topo->page ? topo->page->layer_offsets[layer_id] : 0});
      }
      std::vector<uint32_t> ids;
      ids.reserve(targets[gi].size());
      for (auto &t : targets[gi]) ids.push_back((uint32_t)t.first);
      std::vector<RunBuilder> rb0, rb1;
      for (auto &p : per) {
        rb0.emplace_back(p.layout->range_bytes());
        rb1.emplace_back(p.layout->range_bytes());
      }
      // Block by block, every layer of the block in turn: a stored block's slots lie next to each
      // other in memory, a layer's slots of different blocks do not.
      for (auto &t : targets[gi]) {
        const SealedBlock &sb = *block_cache[t.second];
        for (size_t k = 0; k < per.size(); ++k) {
          const PerLayer &p = per[k];
          if (p.slot >= sb.slots.size() || sb.slots[p.slot].n_segments == 0)
            throw Error::invalid(strf("stored block is missing slot %zu for layer %s", p.slot, p.name->c_str()));
          if (t.first >= p.layout->num_blocks())
            throw Error::storage(strf("layer %s: block %zu out of range (%zu blocks)", p.name->c_str(), t.first,
                                      p.layout->num_blocks()));
          const RawBlock &raw = sb.slots[p.slot];
          char *k_host = raw.seg[0].host + p.offset;
          const uint64_t k_dev = raw.seg[0].device + p.offset;
          rb0[k].add(k_host, k_dev);
          if (p.layout->is_split()) {
            // V comes from the second host segment, or directly after K when the stored
            // block has a single segment (gpu_worker.rs:376-379).
            if (raw.n_segments > 1) rb1[k].add(raw.seg[1].host + p.offset, raw.seg[1].device + p.offset);
            else rb1[k].add(k_host + p.layout->segment_bytes(), k_dev + p.layout->segment_bytes());
          }
        }
      }
      for (size_t k = 0; k < per.size(); ++k) {
        LayerWork w;
        w.layer_name = *per[k].name;
        w.layout = *per[k].layout;
        w.block_ids = ids;
        w.runs[0] = rb0[k].take();
        if (per[k].layout->is_split()) w.runs[1] = rb1[k].take();
        work->push_back(std::move(w));
      }
    }
    if (work->empty()) {
      signal(true, "");
      return;
    }
    auto keep_alive = std::make_shared<std::vector<BlockRef>>(std::move(block_cache));
    GpuContext *gpu_raw = gpu.get();
    if (trace_)
      fprintf(stderr, "[pegaflow_b200] load %s: build_tasks %.2f ms\n", instance_id.c_str(),
              std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_begin).count());
    const auto t_submit = lap(kLoadBuildTasks, t_lookup);
    gpu->load_worker->submit([=](TransferBackend &backend, cudaStream_t stream) {
      Range nvtx("gpu.load_task");
      const auto t0 = lap(kLoadQueueWait, t_submit);
      try {
        std::vector<pf_layer_xfer> xf(work->size());
        std::vector<void *> events(work->size(), nullptr);
        size_t bytes = 0;
        for (size_t i = 0; i < work->size(); ++i) {
          LayerWork &w = (*work)[i];
          xf[i] = pf_layer_xfer{w.layout.data_ptr(), w.layout.block_stride_bytes(), w.layout.kv_stride_bytes(),
                                w.layout.range_bytes(), w.layout.n_ranges(), w.block_ids.size(), w.block_ids.data(),
                                {w.runs[0].size(), w.runs[1].size()}, {w.runs[0].data(), w.runs[1].data()}};
          auto ev = gpu_raw->load_events.find(w.layer_name);
          if (ev != gpu_raw->load_events.end()) events[i] = ev->second;
          bytes += w.payload_bytes();
        }
        backend.move_layers(xf.data(), xf.size(), true, stream, events.data());
        lap(kLoadEnqueue, t0);
        gpu_raw->load_worker->mark_enqueued(gpu_raw->load_worker->current_ticket());
        cuda_or_storage(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        lap(kLoadTask, t0);
        load_bytes_.fetch_add(bytes);
        load_tasks_.fetch_add(1);
        load_nanos_.fetch_add((uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
                                  std::chrono::steady_clock::now() - t0).count());
        (void)keep_alive;
        signal(true, "");
      } catch (const std::exception &e) {
        load_failures_.fetch_add(1);
        signal(false, e.what());
      }
    });
    (void)gpu;
  } catch (const Error &e) {
    signal(false, e.what());
    throw;
  }
}

cudaEvent_t Engine::layer_load_event(const std::string &instance_id, int device_id, const std::string &layer) {
  auto inst = get_instance(instance_id);
  std::shared_ptr<GpuContext> gpu;
  {
    std::lock_guard<std::mutex> g(inst->mu);
    auto it = inst->gpus.find(device_id);
    if (it == inst->gpus.end()) throw Error::worker_missing(instance_id, device_id);
    gpu = it->second;
  }
  auto ev = gpu->load_events.find(layer);
  if (ev == gpu->load_events.end()) throw Error::invalid("layer " + layer + " is not registered");
  // The event only means something once the load that records it has been enqueued.
  gpu->load_worker->wait_enqueued(gpu->load_worker->submitted());
  return ev->second;
}

void Engine::peer_load(const std::string &src_instance, int src_device, const std::string &dst_instance,
                       int dst_device, const std::vector<size_t> &src_ids, const std::vector<size_t> &dst_ids) {
  if (src_ids.size() != dst_ids.size()) throw Error::invalid("peer load needs one destination per source block");
  auto find_gpu = [&](const std::string &id, int device) {
    auto inst = get_instance(id);
    sealed_topology(*inst);
    std::lock_guard<std::mutex> g(inst->mu);
    auto it = inst->gpus.find(device);
    if (it == inst->gpus.end()) throw Error::worker_missing(id, device);
    return it->second;
  };
  auto src = find_gpu(src_instance, src_device);
  auto dst = find_gpu(dst_instance, dst_device);
  struct Pair {
    pf_device_layout s, d;
  };
  auto pairs = std::make_shared<std::vector<Pair>>();
  auto sids = std::make_shared<std::vector<uint32_t>>(), dids = std::make_shared<std::vector<uint32_t>>();
  for (auto &kv : dst->layouts) {
    auto sit = src->layouts.find(kv.first);
    if (sit == src->layouts.end()) continue;
    const KVCacheLayout &a = sit->second, &b = kv.second;
    if (a.range_bytes() != b.range_bytes() || a.n_ranges() != b.n_ranges())
      throw Error::invalid("layer " + kv.first + " has different block geometry on the two instances");
    for (size_t i = 0; i < src_ids.size(); ++i) {
      if (src_ids[i] >= a.num_blocks())
        throw Error::invalid(strf("block_id %zu out of range (num_blocks=%zu) for layer %s", src_ids[i], a.num_blocks(),
                                  kv.first.c_str()));
      if (dst_ids[i] >= b.num_blocks())
        throw Error::invalid(strf("block_id %zu out of range (num_blocks=%zu) for layer %s", dst_ids[i], b.num_blocks(),
                                  kv.first.c_str()));
    }
    pairs->push_back(Pair{{a.data_ptr(), a.block_stride_bytes(), a.kv_stride_bytes(), a.range_bytes(), a.n_ranges(),
                           a.num_blocks()},
                          {b.data_ptr(), b.block_stride_bytes(), b.kv_stride_bytes(), b.range_bytes(), b.n_ranges(),
                           b.num_blocks()}});
  }
  if (pairs->empty()) throw Error::invalid("the two instances share no layer name");
  for (size_t v : src_ids) sids->push_back((uint32_t)v);
  for (size_t v : dst_ids) dids->push_back((uint32_t)v);
  if (src_device != dst_device) enable_peer_access(dst_device, src_device);
  auto done = std::make_shared<std::promise<void>>();
  auto finished = done->get_future();
  dst->load_worker->submit([=](TransferBackend &backend, cudaStream_t stream) {
    try {
      std::vector<pf_device_layout> from, to;
      for (auto &p : *pairs) {
        from.push_back(p.s);
        to.push_back(p.d);
      }
      backend.peer_copy_layers(from.data(), to.data(), from.size(), sids->data(), dids->data(), sids->size(), stream);
      cuda_or_storage(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
      done->set_value();
    } catch (...) {
      done->set_exception(std::current_exception());
    }
  });
  finished.get();
}

// storage/mod.rs:395-445: every resident block leaves the cache; one that a lease, a load in
// flight or a caller's handle still holds keeps its pool memory until that holder lets go.
void Engine::cleanup_memory_cache(pf_cache_cleanup_stats *out) {
  memset(out, 0, sizeof *out);
  uint64_t used_before = 0, used_after = 0, total = 0;
  allocator_->usage(&used_before, &total);
  std::vector<BlockRef> removed = cache_.remove_all();
  if (removed.empty()) return;
  for (const BlockRef &b : removed) {
    out->evicted_bytes += b->footprint;
    if (b.use_count() > 1) ++out->still_referenced_blocks;
  }
  out->evicted_blocks = removed.size();
  evicted_.fetch_add(removed.size());
  removed.clear();  // frees the pool memory of the blocks nobody else holds
  allocator_->usage(&used_after, &total);
  out->reclaimed_bytes = used_before > used_after ? used_before - used_after : 0;
}

void Engine::metrics(pf_engine_metrics *out) {
  memset(out, 0, sizeof *out);
  out->save_bytes = save_bytes_.load();
  out->save_duration_seconds = save_nanos_.load() * 1e-9;
  out->save_batches = save_batches_.load();
  out->load_bytes = load_bytes_.load();
  out->load_duration_seconds = load_nanos_.load() * 1e-9;
  out->load_tasks = load_tasks_.load();
  out->load_failures = load_failures_.load();
  uint64_t used = 0, total = 0;
  allocator_->usage(&used, &total);
  out->pool_capacity_bytes = total;
  out->pool_used_bytes = used;
  out->pool_alloc_failures = alloc_failures_.load();
  out->cache_blocks = cache_.size();
  out->evicted_blocks = evicted_.load();
  std::vector<std::shared_ptr<InstanceContext>> all;
  {
    std::lock_guard<std::mutex> g(instances_mu_);
    for (auto &kv : instances_) all.push_back(kv.second);
  }
  pf_backend_stats &t = out->transfer;
  for (auto &inst : all) {
    std::lock_guard<std::mutex> g(inst->mu);
    for (auto &kv : inst->gpus) {
      for (GpuWorker *w : {kv.second->load_worker.get(), kv.second->save_worker.get()}) {
        const pf_backend_stats s = w->last_stats();
        t.kernel_launches += s.kernel_launches;
        t.dma_copies += s.dma_copies;
        t.bytes_staged += s.bytes_staged;
        t.bytes_zero_copy += s.bytes_zero_copy;
        t.bytes_peer += s.bytes_peer;
        t.device_status |= s.device_status;
        t.pack_kernel_ms += s.pack_kernel_ms;
        t.pack_kernel_launches += s.pack_kernel_launches;
        t.pack_kernel_bytes += s.pack_kernel_bytes;
        t.link_kernel_ms += s.link_kernel_ms;
        t.link_kernel_launches += s.link_kernel_launches;
        t.link_kernel_bytes += s.link_kernel_bytes;
        t.pack_kernel_device_ms += s.pack_kernel_device_ms;
        t.pack_kernel_device_launches += s.pack_kernel_device_launches;
      }
    }
  }
}

}  // namespace pf
