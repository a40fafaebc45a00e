// sm_100a kernels and host-side sequencing of the transfer backend (see transfer.h).
//
// Kernels
//   copy_items_ldst / copy_descs_ldst : CTA-wide 16-byte vector copy, any alignment.  Used as
//       the HBM<->HBM gather/scatter of the staged route (bound by HBM bandwidth: every payload
//       byte is read once and written once) and as the fallback when an address or size is
//       not a multiple of 16.
//   copy_items_tma / copy_descs_tma   : one thread per CTA drives a ring of bulk async copies
//       (cp.async.bulk global->shared, then shared->global).  Used where the other side is
//       behind PCIe or NVLink: a few CTAs keep hundreds of KiB in flight, which hides link
//       latency without occupying the SMs a model is computing on.
//
// Every device-side wait is bounded; on expiry the kernel writes a code to a mapped status
// word, drains its own stores and returns, so the context stays usable.
#include "transfer.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace pf {

#define PF_CUDA(expr)                                                                                   \
  do {                                                                                                  \
    cudaError_t err__ = (expr);                                                                         \
    if (err__ != cudaSuccess)                                                                           \
      throw Error::storage(strf("%s failed: %s (%s)", #expr, cudaGetErrorName(err__), cudaGetErrorString(err__))); \
  } while (0)

namespace {

constexpr int kLdstThreads = 256;
constexpr int kLdstUnroll = 4;
// Full occupancy (2048 threads per SM, so at most 32 registers per thread): with 4 KiB items a
// thread has a single 16-byte load in flight per iteration, and the number of resident threads is
// what keeps HBM busy (measured on 4 KiB items: 4 CTAs per SM 4.3 TB/s, 8 CTAs per SM 5.7 TB/s).
constexpr int kLdstCtasPerSm = 8;
constexpr uint32_t kPackChunk = 16384;   // bytes one CTA iteration of the ld/st kernel moves
constexpr int kStages = 4;               // ring depth of the TMA kernels
constexpr uint32_t kStageBytes = 32768;  // bytes per ring stage
constexpr unsigned kStatusWaitExpired = 0x57A17u;
constexpr size_t kSmallTaskBytes = 2u << 20;      // multi-layer tasks up to this size take one zero-copy launch
constexpr size_t kFirstGroupBytes = 4u << 20;     // size limit of a call's first staging group, doubled per group
constexpr size_t kMinEventGroupBytes = 8u << 20;  // a layer with fewer staged bytes shares the DMA of the next ones
constexpr size_t kMinPairBytes = 8u << 20;        // a save group at least this large waits for a partner to share a launch
constexpr int kHeldGroupsDefault = 3;             // staging slots one gather launch of a save fills
constexpr size_t kMinLinkLaunchBytes = 32u << 20; // ... and one with fewer zero-copy bytes the launch of the next ones

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint64_t side_addr(const Side &s, uint32_t i) {
  if (s.table) return s.table[i];
  uint64_t idx = s.ids ? (uint64_t)s.ids[i] : (uint64_t)i;
  return s.base + idx * s.stride;
}

// Chunk generators: both yield (src, dst, len) triples for the calling CTA.
struct ItemGen {
  Side src, dst;
  uint32_t item_bytes, chunk_bytes, chunks_per_item;
  uint64_t cursor, total, step;
  __device__ ItemGen(const Side &s, const Side &d, uint32_t n_items, uint32_t ib, uint32_t cb)
      : src(s), dst(d), item_bytes(ib), chunk_bytes(cb) {
    chunks_per_item = (ib + cb - 1) / cb;
    total = (uint64_t)n_items * chunks_per_item;
    cursor = blockIdx.x;
    step = gridDim.x;
  }
  __device__ bool next(uint64_t &s, uint64_t &d, uint32_t &len) {
    if (cursor >= total) return false;
    uint32_t item = (uint32_t)(cursor / chunks_per_item);
    uint32_t off = (uint32_t)(cursor % chunks_per_item) * chunk_bytes;
    len = min(chunk_bytes, item_bytes - off);
    s = side_addr(src, item) + off;
    d = side_addr(dst, item) + off;
    cursor += step;
    return true;
  }
};

// Descriptor triples [dst, src, size] as in the reference's kernel backend
// (pegaflow-core/src/transfer/kernel.rs:21-24), sizes may differ per descriptor.
struct DescGen {
  const uint64_t *triples;
  uint32_t n, chunk_bytes, i, step;
  uint64_t off;
  __device__ DescGen(const uint64_t *t, uint32_t n_, uint32_t cb)
      : triples(t), n(n_), chunk_bytes(cb), i(blockIdx.x), step(gridDim.x), off(0) {}
  __device__ bool next(uint64_t &s, uint64_t &d, uint32_t &len) {
    while (i < n) {
      uint64_t size = triples[3 * (uint64_t)i + 2];
      if (off < size) {
        uint64_t left = size - off;
        len = left < chunk_bytes ? (uint32_t)left : chunk_bytes;
        d = triples[3 * (uint64_t)i] + off;
        s = triples[3 * (uint64_t)i + 1] + off;
        off += len;
        return true;
      }
      i += step;
      off = 0;
    }
    return false;
  }
};

// CTA-wide copy of one span, any alignment: 16-byte vectors when source and destination share
// their misalignment (head bytes are peeled), plain bytes otherwise.  Kept out of line so that its
// registers do not count against the aligned fast path below.
__device__ __noinline__ void copy_span_any(uint64_t dst, uint64_t src, uint32_t len) {
  const uint32_t tid = threadIdx.x, nthr = blockDim.x;
  if (((dst ^ src) & 15ull) != 0) {
    char *d = reinterpret_cast<char *>(dst);
    const char *s = reinterpret_cast<const char *>(src);
    for (uint32_t j = tid; j < len; j += nthr) d[j] = s[j];
    return;
  }
  uint32_t head = (uint32_t)((16 - (src & 15ull)) & 15ull);
  if (head > len) head = len;
  if (tid < head) reinterpret_cast<char *>(dst)[tid] = reinterpret_cast<const char *>(src)[tid];
  const int4 *s16 = reinterpret_cast<const int4 *>(src + head);
  int4 *d16 = reinterpret_cast<int4 *>(dst + head);
  const uint32_t n16 = (len - head) >> 4;
  for (uint32_t j = tid; j < n16; j += nthr) d16[j] = s16[j];
  for (uint32_t j = head + (n16 << 4) + tid; j < len; j += nthr)
    reinterpret_cast<char *>(dst)[j] = reinterpret_cast<const char *>(src)[j];
}

// CTA-wide copy of one span.  Fast path: both addresses and the length are multiples of 16, every
// thread keeps kLdstUnroll independent 16-byte loads in flight (streamed past L1).  (L2
// eviction-priority hints on either side were measured and changed nothing: the staging slot
// stays in L2 without them.)
template <bool kAligned = false>
__device__ __forceinline__ void copy_span(uint64_t dst, uint64_t src, uint32_t len) {
  if (!kAligned && ((dst | src | len) & 15ull) != 0) {
    copy_span_any(dst, src, len);
    return;
  }
  const int4 *s16 = reinterpret_cast<const int4 *>(src);
  int4 *d16 = reinterpret_cast<int4 *>(dst);
  const uint32_t n16 = len >> 4;
  for (uint32_t j = threadIdx.x; j < n16; j += kLdstThreads * kLdstUnroll) {
    int4 v[kLdstUnroll];
#pragma unroll
    for (int u = 0; u < kLdstUnroll; ++u) {
      const uint32_t jj = j + u * kLdstThreads;
      if (jj < n16)
        asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                     : "l"(s16 + jj));
    }
#pragma unroll
    for (int u = 0; u < kLdstUnroll; ++u) {
      const uint32_t jj = j + u * kLdstThreads;
      if (jj < n16) d16[jj] = v[u];
    }
  }
}

// `stamp` (optional) points at {first start, last end} in %globaltimer nanoseconds, pre-set to
// {UINT64_MAX, 0}: a device-side measure of the launch that needs no event around it.
__global__ void __launch_bounds__(kLdstThreads, kLdstCtasPerSm)
copy_items_ldst(Side src, Side dst, uint32_t n_items, uint32_t item_bytes, uint32_t chunk_bytes,
                unsigned long long *stamp) {
  if (stamp && threadIdx.x == 0) atomicMin(&stamp[0], (unsigned long long)global_timer_ns());
  ItemGen gen(src, dst, n_items, item_bytes, chunk_bytes);
  uint64_t s, d;
  uint32_t len;
  while (gen.next(s, d, len)) copy_span(d, s, len);
  if (stamp) {
    __syncthreads();
    if (threadIdx.x == 0) atomicMax(&stamp[1], (unsigned long long)global_timer_ns());
  }
}

// The NVLink peer path.  Warp-granular copy of equally sized, 16-byte aligned blocks between two
// scattered sides: every warp moves pieces of kWarpPiece bytes on its own (no CTA-wide step), 4
// independent 16-byte loads per lane.  The reads cross the link (the kernel runs on the
// destination GPU), and with 2048 resident threads per SM there are enough of them in flight to
// cover its latency whatever the block size.  Measured on scattered 4 / 8 / 32 KiB blocks between
// two B200s: 676 / 670 / 677 GB/s, against 525 / 637 / 653 for a bulk-copy (TMA) ring and 775 for
// one large cudaMemcpy; running on the source GPU (stores across the link) gave 625.
// One launch covers up to kMaxPeerUnits (layer, range) units that share block ids and size, so a
// whole model's layers take a handful of launches and one upload of the ids.
constexpr uint32_t kWarpPiece = 32 * 16 * kLdstUnroll;
constexpr int kMaxPeerUnits = 96;
struct PeerUnit {
  uint64_t src_base, src_stride, dst_base, dst_stride;
};
struct PeerParams {
  const uint32_t *src_ids, *dst_ids;
  uint32_t n_units, n_items, item_bytes, pieces_per_item;
  PeerUnit unit[kMaxPeerUnits];
};
__global__ void __launch_bounds__(kLdstThreads, kLdstCtasPerSm)
copy_peer_warp(const __grid_constant__ PeerParams p) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t per_unit = p.n_items * p.pieces_per_item;  // the host keeps this below 2^32
  const uint64_t total = (uint64_t)p.n_units * per_unit;
  const uint64_t n_warps = (uint64_t)gridDim.x * (kLdstThreads / 32);
  for (uint64_t c = (uint64_t)blockIdx.x * (kLdstThreads / 32) + (threadIdx.x >> 5); c < total; c += n_warps) {
    const uint32_t k = (uint32_t)(c / per_unit);
    const uint32_t r = (uint32_t)(c - (uint64_t)k * per_unit);
    const uint32_t item = r / p.pieces_per_item;
    const uint32_t off = (r - item * p.pieces_per_item) * kWarpPiece;
    const uint32_t n16 = min(kWarpPiece, p.item_bytes - off) >> 4;
    const int4 *s16 =
        reinterpret_cast<const int4 *>(p.unit[k].src_base + (uint64_t)p.src_ids[item] * p.unit[k].src_stride + off);
    int4 *d16 = reinterpret_cast<int4 *>(p.unit[k].dst_base + (uint64_t)p.dst_ids[item] * p.unit[k].dst_stride + off);
    int4 v[kLdstUnroll];
#pragma unroll
    for (int u = 0; u < kLdstUnroll; ++u) {
      const uint32_t jj = lane + u * 32;
      if (jj < n16)
        asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                     : "l"(s16 + jj));
    }
#pragma unroll
    for (int u = 0; u < kLdstUnroll; ++u) {
      const uint32_t jj = lane + u * 32;
      if (jj < n16) d16[jj] = v[u];
    }
  }
}

// One launch for a whole staging group: up to kMaxGroupUnits runs of equally sized items, each
// with its own KV-side addressing, laid back to back in the staging slot.  `to_staging` selects
// the direction.  The unit table travels in the kernel parameters (no upload).
constexpr int kMaxGroupUnits = 40;
struct GroupUnit {
  Side kv;               // the scattered side (KV cache blocks)
  uint64_t slot_addr;    // where the unit starts in the staging slot
  uint32_t item_bytes;
  uint32_t chunks_per_item;
  uint64_t chunk_end;    // exclusive prefix sum of chunks over the units
};
struct GroupParams {
  uint32_t n_units;
  uint32_t chunk_bytes;
  GroupUnit unit[kMaxGroupUnits];
};

// kAligned: the host has checked that every address and size in the group is a multiple of 16
// (the usual case), so the kernel carries no byte path and fits 32 registers without spilling.
template <bool kAligned>
__global__ void __launch_bounds__(kLdstThreads, kLdstCtasPerSm)
copy_group_ldst(const __grid_constant__ GroupParams p, int to_staging, unsigned long long *stamp) {
  // Programmatic dependent launch: the next kernel of the stream may be scheduled onto the SMs as
  // this one's CTAs leave them, and this one touches memory only when everything enqueued before it
  // has completed and is visible.  Both instructions do nothing in a launch without the attribute.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (stamp && threadIdx.x == 0) atomicMin(&stamp[0], (unsigned long long)global_timer_ns());
  // 32-bit chunk arithmetic: a group holds at most one staging slot of bytes
  const uint32_t total = (uint32_t)p.unit[p.n_units - 1].chunk_end;
  uint32_t k = 0, unit_begin = 0, unit_end = (uint32_t)p.unit[0].chunk_end;
  for (uint32_t c = blockIdx.x; c < total; c += gridDim.x) {
    while (c >= unit_end) {  // chunks are visited in ascending order
      ++k;
      unit_begin = unit_end;
      unit_end = (uint32_t)p.unit[k].chunk_end;
    }
    const uint32_t local = c - unit_begin;
    const uint32_t cpi = p.unit[k].chunks_per_item, item_bytes = p.unit[k].item_bytes;
    const uint32_t item = local / cpi;
    const uint32_t off = (local - item * cpi) * p.chunk_bytes;
    const uint32_t len = min(p.chunk_bytes, item_bytes - off);
    const uint32_t *ids = p.unit[k].kv.ids;
    const uint64_t *table = p.unit[k].kv.table;
    const uint64_t kv = (table ? table[item] : p.unit[k].kv.base + (uint64_t)(ids ? ids[item] : item) * p.unit[k].kv.stride) + off;
    const uint64_t st = p.unit[k].slot_addr + (uint64_t)item * item_bytes + off;
    copy_span<kAligned>(to_staging ? st : kv, to_staging ? kv : st, len);
  }
  if (stamp) {
    __syncthreads();
    if (threadIdx.x == 0) atomicMax(&stamp[1], (unsigned long long)global_timer_ns());
  }
}

__global__ void __launch_bounds__(kLdstThreads)
copy_descs_ldst(const uint64_t *__restrict__ triples, uint32_t n, uint32_t chunk_bytes) {
  DescGen gen(triples, n, chunk_bytes);
  uint64_t s, d;
  uint32_t len;
  while (gen.next(s, d, len)) copy_span(d, s, len);
}

// ---- bulk async copy (TMA) primitives ------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0,1,0,p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(void *smem_dst, uint64_t gsrc, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(uint64_t gdst, const void *smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Waits for a ring stage to fill.  Gives up after ~2 s (a link read normally takes microseconds).
__device__ __forceinline__ bool wait_stage(uint64_t *bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t start = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 1023u) == 0 && global_timer_ns() - start > 2000000000ull) return false;
  }
  return true;
}

// One thread runs the ring.  Prologue: loads 0..kStages-1 fill every stage.  Steady state, for
// chunk k: wait for its load, issue its store, then (from k = 1 on) wait until every store but
// the newest has finished reading shared memory and issue load k-1+kStages into the stage of
// chunk k-1.  So kStages-1 loads are in flight while one store drains.
template <class Gen>
__device__ __forceinline__ void tma_ring(Gen &gen, char *ring, uint64_t *bars, uint32_t stage_bytes,
                                         unsigned int *status) {
  uint64_t dsts[kStages];
  uint32_t lens[kStages];
  for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");

  uint64_t produced = 0, consumed = 0;
  bool more = true;
  auto produce = [&]() -> bool {
    uint64_t s, d;
    uint32_t len;
    if (!gen.next(s, d, len)) return false;
    int st = (int)(produced % kStages);
    dsts[st] = d;
    lens[st] = len;
    mbar_expect_tx(&bars[st], len);
    bulk_g2s(ring + (size_t)st * stage_bytes, s, len, &bars[st]);
    ++produced;
    return true;
  };
  for (int s = 0; s < kStages && more; ++s) more = produce();
  while (consumed < produced) {
    const int st = (int)(consumed % kStages);
    const uint32_t parity = (uint32_t)((consumed / kStages) & 1);
    if (!wait_stage(&bars[st], parity)) {
      *status = kStatusWaitExpired;
      bulk_wait_all();
      return;
    }
    bulk_s2g(dsts[st], ring + (size_t)st * stage_bytes, lens[st]);
    bulk_commit();
    ++consumed;
    if (more && consumed >= 2) {
      bulk_wait_read_1();  // every store but the newest has finished reading shared memory
      more = produce();    // lands in the stage of chunk consumed-2
    }
  }
  bulk_wait_all();
}

__global__ void __launch_bounds__(32)
copy_items_tma(Side src, Side dst, uint32_t n_items, uint32_t item_bytes, uint32_t stage_bytes,
               unsigned int *status) {
  extern __shared__ __align__(128) char ring[];
  __shared__ uint64_t bars[kStages];
  if (threadIdx.x != 0) return;
  ItemGen gen(src, dst, n_items, item_bytes, stage_bytes);
  tma_ring(gen, ring, bars, stage_bytes, status);
}

__global__ void __launch_bounds__(32)
copy_descs_tma(const uint64_t *__restrict__ triples, uint32_t n, uint32_t stage_bytes, unsigned int *status) {
  extern __shared__ __align__(128) char ring[];
  __shared__ uint64_t bars[kStages];
  if (threadIdx.x != 0) return;
  DescGen gen(triples, n, stage_bytes);
  tma_ring(gen, ring, bars, stage_bytes, status);
}


// ---- zero-copy over PCIe, one launch for a whole task ---------------------------------------------
// A unit is one host run of one device range of one layer: item i lives at
// kv_base + ids[i] * kv_stride on the GPU and at host_base + i * host_stride in the (mapped) pool.
// The unit table and the ids lie in device memory, so a launch covers any number of layers.  One
// thread per CTA drives a ring of bulk copies; the PCIe side of a ring stage is one large bulk copy
// whenever the host side of the chunk is dense, whatever the block size: blocks of 2-16 KiB are
// batched kLinkItemsMax to a stage (several bulk loads from scattered HBM blocks fill the stage, one
// bulk store drains it to the pool; the mirror image for a load).
constexpr uint32_t kLinkItemsMax = 16;
struct LinkUnit {
  uint64_t kv_base, kv_stride;
  uint64_t host_base, host_stride;   // pool side when host_table is null
  const uint64_t *host_table;        // else: the pool address of every item (host runs that do not line up)
  const uint32_t *ids;
  uint64_t chunk_end;        // exclusive prefix sum of chunks over the units of the call
  uint32_t n_items, item_bytes;
  uint32_t items_per_chunk;  // >= 2: a chunk is that many whole items; otherwise an item is cut
  uint32_t chunks_per_item;  //      into this many chunks of chunk_bytes (the last one may be shorter)
  uint32_t chunk_bytes;
  uint32_t pad_;
};

__global__ void __launch_bounds__(32)
copy_units_tma(const LinkUnit *__restrict__ units, uint32_t n_units, uint64_t chunk_begin, int to_host,
               unsigned int *status) {
  extern __shared__ __align__(128) char ring[];
  __shared__ uint64_t bars[kStages];
  if (threadIdx.x != 0) return;
  for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");

  // what each ring stage holds: `count` pieces of `len` bytes, piece j = bytes [off, off + len) of item item0 + j
  uint32_t st_unit[kStages], st_item0[kStages], st_count[kStages], st_off[kStages], st_len[kStages];
  const uint64_t total_end = units[n_units - 1].chunk_end;
  uint64_t cursor = chunk_begin + blockIdx.x, unit_begin = chunk_begin;
  uint32_t k = 0;
  uint64_t produced = 0, consumed = 0;

  auto host_addr = [](const LinkUnit &u, uint32_t item) -> uint64_t {
    return u.host_table ? u.host_table[item] : u.host_base + (uint64_t)item * u.host_stride;
  };
  // whole items that lie back to back in the pool cross the link as one bulk copy
  auto host_dense = [](const LinkUnit &u, uint32_t len) -> bool { return !u.host_table && u.host_stride == len; };

  auto produce = [&]() -> bool {
    if (cursor >= total_end) return false;
    while (cursor >= units[k].chunk_end) {  // chunks are visited in ascending order
      unit_begin = units[k].chunk_end;
      ++k;
    }
    const LinkUnit &u = units[k];
    const uint64_t local = cursor - unit_begin;
    uint32_t item0, count, off, len;
    if (u.items_per_chunk >= 2) {
      item0 = (uint32_t)local * u.items_per_chunk;
      count = min(u.items_per_chunk, u.n_items - item0);
      off = 0;
      len = u.item_bytes;
    } else {
      item0 = (uint32_t)(local / u.chunks_per_item);
      count = 1;
      off = (uint32_t)(local - (uint64_t)item0 * u.chunks_per_item) * u.chunk_bytes;
      len = min(u.chunk_bytes, u.item_bytes - off);
    }
    const int st = (int)(produced % kStages);
    st_unit[st] = k, st_item0[st] = item0, st_count[st] = count, st_off[st] = off, st_len[st] = len;
    char *stage = ring + (size_t)st * kStageBytes;
    mbar_expect_tx(&bars[st], count * len);
    if (to_host) {
      for (uint32_t j = 0; j < count; ++j)
        bulk_g2s(stage + (size_t)j * len, u.kv_base + (uint64_t)u.ids[item0 + j] * u.kv_stride + off, len, &bars[st]);
    } else if (host_dense(u, len)) {
      bulk_g2s(stage, u.host_base + (uint64_t)item0 * u.host_stride, count * len, &bars[st]);
    } else {
      for (uint32_t j = 0; j < count; ++j) bulk_g2s(stage + (size_t)j * len, host_addr(u, item0 + j) + off, len, &bars[st]);
    }
    ++produced;
    cursor += gridDim.x;
    return true;
  };

  bool more = true;
  for (int s = 0; s < kStages && more; ++s) more = produce();
  while (consumed < produced) {
    const int st = (int)(consumed % kStages);
    if (!wait_stage(&bars[st], (uint32_t)((consumed / kStages) & 1))) {
      *status = kStatusWaitExpired;
      bulk_wait_all();
      return;
    }
    const LinkUnit &u = units[st_unit[st]];
    const uint32_t item0 = st_item0[st], count = st_count[st], off = st_off[st], len = st_len[st];
    const char *stage = ring + (size_t)st * kStageBytes;
    if (!to_host) {
      for (uint32_t j = 0; j < count; ++j)
        bulk_s2g(u.kv_base + (uint64_t)u.ids[item0 + j] * u.kv_stride + off, stage + (size_t)j * len, len);
    } else if (host_dense(u, len)) {
      bulk_s2g(u.host_base + (uint64_t)item0 * u.host_stride, stage, count * len);
    } else {
      for (uint32_t j = 0; j < count; ++j) bulk_s2g(host_addr(u, item0 + j) + off, stage + (size_t)j * len, len);
    }
    bulk_commit();
    ++consumed;
    if (more && consumed >= 2) {
      bulk_wait_read_1();  // every store group but the newest has finished reading shared memory
      more = produce();    // lands in the stage of chunk consumed-2
    }
  }
  bulk_wait_all();
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

static_assert(kStages >= 2, "ring needs two stages");

// ------------------------------------------------------------------------------------------------

TransferBackend::TransferBackend(int device, const pf_backend_config *config) : device_(device) {
  cfg_ = config ? *config : pf_backend_config{};
  if (cfg_.staging_slot_bytes == 0) cfg_.staging_slot_bytes = 32u << 20;
  if (cfg_.staging_slots <= 0) cfg_.staging_slots = 6;
  // One copy stream: DMAs of consecutive slots run back to back.  Two streams let two DMAs share the
  // link; measured, that is never faster, spreads more from step to step and doubles the time until
  // the first layer of a save is in the pool.
  if (cfg_.copy_streams <= 0) cfg_.copy_streams = 1;
  if (cfg_.copy_streams > 8) cfg_.copy_streams = 8;
  if (cfg_.gather_slots <= 0) cfg_.gather_slots = kHeldGroupsDefault;
  cfg_.gather_slots = std::min(cfg_.gather_slots, std::max(1, cfg_.staging_slots / 2));
  if (cfg_.min_dma_bytes == 0) cfg_.min_dma_bytes = 256u << 10;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    throw Error::cuda_init(strf("no CUDA device available (%s)", cudaGetErrorString(e)));
  if (device < 0 || device >= count) throw Error::cuda_init(strf("device %d out of range (%d devices)", device, count));
  DeviceGuard on_device(device);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) throw Error::cuda_init("cudaGetDeviceProperties failed");
  if (prop.major < 10)
    throw Error::cuda_init(strf("device %d is sm_%d%d; this library carries sm_100a code only", device, prop.major,
                                prop.minor));
  sm_count_ = prop.multiProcessorCount;
  if (cfg_.pack_ctas <= 0) cfg_.pack_ctas = sm_count_ * 8;
  aux_.resize(cfg_.copy_streams, nullptr);
  aux_join_.resize(cfg_.copy_streams, nullptr);
  aux_layer_dirty_.assign(cfg_.copy_streams, 0);
  aux_task_dirty_.assign(cfg_.copy_streams, 0);
  aux_forked_.assign(cfg_.copy_streams, 0);
  PF_CUDA(cudaEventCreateWithFlags(&fork_, cudaEventDisableTiming));
  for (int i = 0; i < cfg_.copy_streams; ++i) {
    if (cudaStreamCreateWithFlags(&aux_[i], cudaStreamNonBlocking) != cudaSuccess)
      throw Error::cuda_init("failed to create a copy stream");
    PF_CUDA(cudaEventCreateWithFlags(&aux_join_[i], cudaEventDisableTiming));
  }
  PF_CUDA(cudaHostAlloc(&status_host_, sizeof(unsigned int), cudaHostAllocMapped));
  *status_host_ = 0;
  PF_CUDA(cudaHostGetDevicePointer(&status_dev_, status_host_, 0));
  PF_CUDA(cudaFuncSetAttribute(copy_items_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, kStages * kStageBytes));
  PF_CUDA(cudaFuncSetAttribute(copy_descs_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, kStages * kStageBytes));
  PF_CUDA(cudaFuncSetAttribute(copy_units_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, kStages * kStageBytes));
  meta_grow(1u << 20);
  if (cfg_.time_kernels) {
    stamps_host_.assign(2 * (size_t)kStampRing, 0);
    for (size_t i = 0; i < (size_t)kStampRing; ++i) stamps_host_[2 * i] = ~0ull;
    PF_CUDA(cudaMalloc(&stamps_dev_, stamps_host_.size() * sizeof(unsigned long long)));
    PF_CUDA(cudaMemcpy(stamps_dev_, stamps_host_.data(), stamps_host_.size() * sizeof(unsigned long long),
                       cudaMemcpyHostToDevice));
  }
}

TransferBackend::~TransferBackend() {
  DeviceGuard on_device(device_);
  for (auto st : aux_)
    if (st) cudaStreamSynchronize(st);
  for (auto &r : meta_inflight_) cudaEventSynchronize(r.done);
  for (auto &s : slots_) {
    if (s.filled) cudaEventDestroy(s.filled);
    if (s.drained) cudaEventDestroy(s.drained);
  }
  for (auto &r : meta_inflight_) cudaEventDestroy(r.done);
  for (auto ev : event_pool_) cudaEventDestroy(ev);
  for (auto &t : timed_) {
    cudaEventDestroy(t.start);
    cudaEventDestroy(t.stop);
  }
  for (auto ev : timing_event_pool_) cudaEventDestroy(ev);
  if (staging_) cudaFree(staging_);
  if (stamps_dev_) cudaFree(stamps_dev_);
  if (meta_dev_) cudaFree(meta_dev_);
  if (meta_host_) cudaFreeHost(meta_host_);
  if (status_host_) cudaFreeHost(status_host_);
  if (fork_) cudaEventDestroy(fork_);
  for (auto ev : aux_join_)
    if (ev) cudaEventDestroy(ev);
  for (auto st : aux_)
    if (st) cudaStreamDestroy(st);
}

void TransferBackend::time_begin(cudaStream_t s, cudaEvent_t *start) {
  *start = nullptr;
  if (!cfg_.time_kernels) return;
  if (timed_.size() > 8192) fold_timings(false);
  auto take = [&]() {
    if (!timing_event_pool_.empty()) {
      cudaEvent_t ev = timing_event_pool_.back();
      timing_event_pool_.pop_back();
      return ev;
    }
    cudaEvent_t ev;
    PF_CUDA(cudaEventCreate(&ev));
    return ev;
  };
  *start = take();
  PF_CUDA(cudaEventRecord(*start, s));
}

void TransferBackend::time_end(cudaStream_t s, cudaEvent_t start, uint64_t bytes, bool link, int stamp_idx) {
  if (!start) return;
  cudaEvent_t stop;
  if (!timing_event_pool_.empty()) {
    stop = timing_event_pool_.back();
    timing_event_pool_.pop_back();
  } else {
    PF_CUDA(cudaEventCreate(&stop));
  }
  PF_CUDA(cudaEventRecord(stop, s));
  timed_.push_back({start, stop, bytes, link, stamp_idx});
}

void TransferBackend::fold_timings(bool wait) {
  bool stamps_fetched = false;
  while (!timed_.empty()) {
    TimedLaunch &t = timed_.front();
    cudaError_t q = wait ? cudaEventSynchronize(t.stop) : cudaEventQuery(t.stop);
    if (q != cudaSuccess) {
      cudaGetLastError();
      break;
    }
    float ms = 0;
    if (cudaEventElapsedTime(&ms, t.start, t.stop) == cudaSuccess) {
      if (t.link) {
        stats_.link_kernel_ms += ms;
        ++stats_.link_kernel_launches;
        stats_.link_kernel_bytes += t.bytes;
      } else {
        stats_.pack_kernel_ms += ms;
        ++stats_.pack_kernel_launches;
        stats_.pack_kernel_bytes += t.bytes;
        if (t.stamp_idx >= 0) {
          if (!stamps_fetched) {
            // finished launches have written their stamps; one copy serves the whole fold
            if (cudaMemcpy(stamps_host_.data(), stamps_dev_, stamps_used_ * 2 * sizeof(unsigned long long),
                           cudaMemcpyDeviceToHost) == cudaSuccess)
              stamps_fetched = true;
          }
          const unsigned long long a = stamps_host_[2 * (size_t)t.stamp_idx], b = stamps_host_[2 * (size_t)t.stamp_idx + 1];
          if (stamps_fetched && b > a && a != ~0ull) {
            stats_.pack_kernel_device_ms += (double)(b - a) * 1e-6;
            ++stats_.pack_kernel_device_launches;
          }
        }
      }
    }
    timing_event_pool_.push_back(t.start);
    timing_event_pool_.push_back(t.stop);
    timed_.pop_front();
  }
}

void TransferBackend::stats(pf_backend_stats *out) {
  if (cfg_.time_kernels) {
    DeviceGuard on_device(device_);
    fold_timings(false);
  }
  *out = stats_;
  out->device_status = status_host_ ? *(volatile unsigned int *)status_host_ : 0;
}

cudaEvent_t TransferBackend::take_event() {
  if (!event_pool_.empty()) {
    cudaEvent_t ev = event_pool_.back();
    event_pool_.pop_back();
    return ev;
  }
  cudaEvent_t ev;
  PF_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  return ev;
}

void TransferBackend::meta_grow(size_t need) {
  // Everything in flight still reads the old buffers: wait for it, then replace them.
  for (auto &r : meta_inflight_) {
    PF_CUDA(cudaEventSynchronize(r.done));
    event_pool_.push_back(r.done);
  }
  meta_inflight_.clear();
  size_t cap = meta_cap_ ? meta_cap_ : (1u << 20);
  while (cap < need) cap *= 2;
  if (meta_dev_) PF_CUDA(cudaFree(meta_dev_));
  if (meta_host_) PF_CUDA(cudaFreeHost(meta_host_));
  meta_dev_ = nullptr;
  meta_host_ = nullptr;
  PF_CUDA(cudaHostAlloc(&meta_host_, cap, cudaHostAllocDefault));
  PF_CUDA(cudaMalloc(&meta_dev_, cap));
  meta_cap_ = cap;
  meta_head_ = 0;
}

size_t TransferBackend::meta_alloc(size_t bytes) {
  bytes = align_up(std::max<size_t>(bytes, 16), 256);
  // Drop regions whose work has already finished.
  while (!meta_inflight_.empty() && cudaEventQuery(meta_inflight_.front().done) == cudaSuccess) {
    event_pool_.push_back(meta_inflight_.front().done);
    meta_inflight_.pop_front();
  }
  cudaGetLastError();  // cudaEventQuery reports "not ready" as an error code
  if (bytes > meta_cap_ / 2) meta_grow(bytes * 2);
  if (meta_head_ + bytes > meta_cap_) meta_head_ = 0;
  const size_t begin = meta_head_, end = meta_head_ + bytes;
  // Reclaim regions the new one overlaps (oldest first; they complete in order).
  while (!meta_inflight_.empty()) {
    bool overlaps = false;
    for (auto &r : meta_inflight_)
      if (r.begin < end && begin < r.end) overlaps = true;
    if (!overlaps) break;
    MetaRegion r = meta_inflight_.front();
    meta_inflight_.pop_front();
    PF_CUDA(cudaEventSynchronize(r.done));
    event_pool_.push_back(r.done);
  }
  meta_head_ = end;
  return begin;
}

void TransferBackend::meta_upload(size_t off, size_t bytes, cudaStream_t stream) {
  PF_CUDA(cudaMemcpyAsync(meta_dev_ + off, meta_host_ + off, bytes, cudaMemcpyHostToDevice, stream));
}

void TransferBackend::ensure_staging() {
  if (staging_) return;
  PF_CUDA(cudaMalloc(&staging_, cfg_.staging_slot_bytes * (size_t)cfg_.staging_slots));
  slots_.resize(cfg_.staging_slots);
  for (int i = 0; i < cfg_.staging_slots; ++i) {
    slots_[i].ptr = staging_ + (size_t)i * cfg_.staging_slot_bytes;
    PF_CUDA(cudaEventCreateWithFlags(&slots_[i].filled, cudaEventDisableTiming));
    PF_CUDA(cudaEventCreateWithFlags(&slots_[i].drained, cudaEventDisableTiming));
  }
}

TransferBackend::Slot &TransferBackend::next_slot() {
  Slot &s = slots_[slot_cursor_];
  slot_cursor_ = (slot_cursor_ + 1) % slots_.size();
  return s;
}

// Gathers (to_staging) or scatters `count` staged units in one launch; unit i lies at
// slot_ptrs[i] + units[i].slot_offset of the staging ring (the units may sit in different slots).
void TransferBackend::launch_group(const StagedUnit *units, char *const *slot_ptrs, size_t count, bool to_staging,
                                   cudaStream_t s) {
  GroupParams p;
  p.n_units = (uint32_t)count;
  p.chunk_bytes = kPackChunk;
  uint64_t chunks = 0, payload = 0;
  bool aligned = true;
  for (size_t i = 0; i < count; ++i) {
    const StagedUnit &u = units[i];
    GroupUnit &g = p.unit[i];
    g.kv = u.dev;
    g.slot_addr = (uint64_t)(uintptr_t)(slot_ptrs[i] + u.slot_offset);
    g.item_bytes = (uint32_t)u.item_bytes;
    g.chunks_per_item = (uint32_t)((u.item_bytes + kPackChunk - 1) / kPackChunk);
    aligned = aligned && !u.dev.table && (u.dev.base | u.dev.stride | g.slot_addr | u.item_bytes) % 16 == 0;
    chunks += (uint64_t)u.n_items * g.chunks_per_item;
    g.chunk_end = chunks;
    payload += (uint64_t)u.n_items * u.item_bytes;
  }
  const int grid = (int)std::min<uint64_t>(chunks, (uint64_t)cfg_.pack_ctas);
  cudaEvent_t t0;
  time_begin(s, &t0);
  unsigned long long *stamp = nullptr;
  int stamp_idx = -1;
  if (t0 && stamps_dev_ && stamps_used_ < kStampRing) {
    stamp_idx = (int)stamps_used_++;
    stamp = stamps_dev_ + 2 * (size_t)stamp_idx;
  }
  // Back-to-back launches overlap their launch latency with the tail of the kernel before them
  // (PEGAFLOW_B200_PDL=0 turns the attribute off).
  static const bool dependent_launch = [] {
    const char *e = getenv("PEGAFLOW_B200_PDL");
    return !e || atoi(e) != 0;
  }();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3((unsigned)grid);
  lc.blockDim = dim3(kLdstThreads);
  lc.stream = s;
  lc.attrs = attr;
  lc.numAttrs = dependent_launch ? 1 : 0;
  const int dir = to_staging ? 1 : 0;
  if (aligned) PF_CUDA(cudaLaunchKernelEx(&lc, copy_group_ldst<true>, p, dir, stamp));
  else PF_CUDA(cudaLaunchKernelEx(&lc, copy_group_ldst<false>, p, dir, stamp));
  PF_CUDA(cudaGetLastError());
  time_end(s, t0, 2 * payload, false, stamp_idx);
  ++stats_.kernel_launches;
}

// All units of the groups in `held` (each in its own staging slot), kMaxGroupUnits per launch.
void TransferBackend::launch_held(const std::vector<HeldGroup> &held, bool to_staging, cudaStream_t s) {
  std::vector<StagedUnit> units;
  std::vector<char *> ptrs;
  for (const HeldGroup &h : held)
    for (const StagedUnit &u : h.units) {
      units.push_back(u);
      ptrs.push_back(h.slot->ptr);
    }
  for (size_t i = 0; i < units.size(); i += kMaxGroupUnits)
    launch_group(units.data() + i, ptrs.data() + i, std::min<size_t>(kMaxGroupUnits, units.size() - i), to_staging, s);
}

void TransferBackend::launch_link(const Side &src, const Side &dst, size_t n_items, size_t item_bytes,
                                  cudaStream_t s, bool peer) {
  if (n_items == 0) return;
  // Bulk async copies and the vector kernels need 16-byte aligned addresses and sizes.  Affine sides are checked here;
  // whoever fills an address table clears tables_aligned_ when an entry is not aligned.
  auto aligned16 = [](const Side &x) { return x.table != nullptr || ((x.base | x.stride) & 15ull) == 0; };
  const bool all16 = aligned16(src) && aligned16(dst) && (item_bytes & 15u) == 0 && tables_aligned_;
  int ctas = cfg_.link_ctas > 0 ? cfg_.link_ctas : 16;
  cudaEvent_t t0;
  time_begin(s, &t0);
  if (all16 && !peer) {
    const uint32_t stage = (uint32_t)std::min<size_t>(kStageBytes, item_bytes);
    const uint64_t chunks = (uint64_t)n_items * ((item_bytes + stage - 1) / stage);
    const int grid = (int)std::min<uint64_t>(chunks, (uint64_t)ctas);
    copy_items_tma<<<grid, 32, (size_t)kStages * stage, s>>>(src, dst, (uint32_t)n_items, (uint32_t)item_bytes, stage,
                                                             status_dev_);
  } else {
    // unaligned geometry (and, over NVLink, the rare unit that copy_peer_warp cannot take)
    const uint64_t chunks = (uint64_t)n_items * ((item_bytes + kPackChunk - 1) / kPackChunk);
    const int grid = (int)std::min<uint64_t>(chunks, (uint64_t)(peer ? std::max(ctas, cfg_.pack_ctas) : std::max(ctas, sm_count_)));
    copy_items_ldst<<<grid, kLdstThreads, 0, s>>>(src, dst, (uint32_t)n_items, (uint32_t)item_bytes, kPackChunk,
                                                     nullptr);
  }
  PF_CUDA(cudaGetLastError());
  time_end(s, t0, (uint64_t)n_items * item_bytes, true, -1);
  ++stats_.kernel_launches;
}

void TransferBackend::launch_descs(const uint64_t *triples_dev, size_t n, bool aligned, cudaStream_t s) {
  if (n == 0) return;
  int ctas = cfg_.link_ctas > 0 ? cfg_.link_ctas : 16;
  if (aligned) {
    const int grid = (int)std::min<size_t>(n, (size_t)ctas);
    copy_descs_tma<<<grid, 32, (size_t)kStages * kStageBytes, s>>>(triples_dev, (uint32_t)n, kStageBytes, status_dev_);
  } else {
    const int grid = (int)std::min<size_t>(n, (size_t)std::max(ctas, sm_count_));
    copy_descs_ldst<<<grid, kLdstThreads, 0, s>>>(triples_dev, (uint32_t)n, kPackChunk);
  }
  PF_CUDA(cudaGetLastError());
  ++stats_.kernel_launches;
}

// With more than one copy stream configured, the streams take the DMAs of consecutive staging slots in turn.
int TransferBackend::next_aux() {
  const int i = (int)(aux_cursor_++ % aux_.size());
  aux_layer_dirty_[i] = 1;
  aux_task_dirty_[i] = 1;
  aux_last_ = i;
  return i;
}

// Makes `target` wait for everything enqueued so far on the copy streams flagged in `dirty`
// (except `skip`, for the case where target is that copy stream itself).
void TransferBackend::join_copy_streams(cudaStream_t target, std::vector<char> &dirty, int skip) {
  for (size_t i = 0; i < aux_.size(); ++i) {
    if (!dirty[i] || (int)i == skip) continue;
    PF_CUDA(cudaEventRecord(aux_join_[i], aux_[i]));
    PF_CUDA(cudaStreamWaitEvent(target, aux_join_[i], 0));
  }
}

// Adds run.n_blocks items (`item_bytes` each) to the staged route.  `dev_side.ids` / `.table`
// already point at the run's first item.  A run is cut into equal chunks that fit a staging
// slot; chunks whose host bytes follow each other without a gap share a slot and one DMA (the
// group), so many small (layer, K-or-V) runs in neighbouring pool allocations still reach the
// copy engine as one large transfer.  Nothing is enqueued until the group is flushed.
void TransferBackend::staged_run(const Side &dev_side, const pf_host_run &run, size_t item_bytes, bool host_is_src,
                                 cudaStream_t stream) {
  const size_t cap = cfg_.staging_slot_bytes / item_bytes;
  const size_t n_chunks = (run.n_blocks + cap - 1) / cap;
  const size_t per_chunk = (run.n_blocks + n_chunks - 1) / n_chunks;
  char *host = static_cast<char *>(run.host);
  const bool dense = run.stride_bytes == item_bytes || run.n_blocks == 1;
  for (size_t b0 = 0; b0 < run.n_blocks; b0 += per_chunk) {
    const size_t nb = std::min(per_chunk, run.n_blocks - b0);
    StagedUnit u;
    u.dev = dev_side;
    if (u.dev.table) u.dev.table += b0;
    if (u.dev.ids) u.dev.ids += b0;
    if (!u.dev.table && !u.dev.ids) u.dev.base += (uint64_t)b0 * u.dev.stride;
    u.n_items = nb;
    u.item_bytes = item_bytes;
    u.host = host + b0 * run.stride_bytes;
    u.host_stride = run.stride_bytes;
    const size_t bytes = nb * item_bytes;
    const bool joins = !group_.empty() && group_dense_ && dense && group_host_is_src_ == host_is_src &&
                       group_stream_ == stream && group_host_end_ == u.host &&
                       group_bytes_ + bytes <= std::min(cfg_.staging_slot_bytes, group_limit_) &&
                       (group_bytes_ & 15u) == 0;
    if (!joins) {
      flush_group(true);
      group_dense_ = dense;
      group_host_is_src_ = host_is_src;
      group_stream_ = stream;
      group_host_begin_ = u.host;
      group_bytes_ = 0;
    }
    u.slot_offset = group_bytes_;
    group_bytes_ += bytes;
    group_host_end_ = u.host + bytes;
    group_.push_back(u);
  }
}

// Closes the open group.  Load: one DMA into a staging slot, then the scatter kernel.  Save: the
// group gets its slot and waits in `held_`; emit_held() gathers every held group with ONE launch and
// sends one DMA per slot after it.  With `may_hold` a full-size group waits for its successor, so that
// in the steady state a launch fills two slots (K and V of a layer): half the launches for the same
// DMAs.  Call sites that need the bytes on their way (a layer's event, the end of a call) pass false.
void TransferBackend::flush_group(bool may_hold) {
  if (group_.empty()) {
    if (!may_hold) emit_held();
    return;
  }
  ensure_staging();
  cudaStream_t stream = group_stream_;
  if (!group_host_is_src_ || gather_only_) {
    if (!held_.empty() && held_.front().stream != stream) emit_held();
    HeldGroup h;
    h.slot = &next_slot();
    h.copy_index = gather_only_ ? -1 : next_aux();
    h.units.swap(group_);
    h.bytes = group_bytes_;
    h.dense = group_dense_;
    h.host_begin = group_host_begin_;
    h.stream = stream;
    held_.push_back(std::move(h));
    const bool hold = may_hold && held_.size() < (size_t)cfg_.gather_slots && held_.back().bytes >= kMinPairBytes;
    if (!hold) emit_held();
  } else {
    Slot &slot = next_slot();
    const int copy_index = next_aux();
    cudaStream_t copy = aux_[copy_index];
    const StagedUnit &first = group_.front();
    // The DMA reads host memory that earlier work on the caller's stream may still be writing
    // (a save enqueued just before): each copy stream joins the caller's stream once per call.
    if (!aux_forked_[copy_index]) {
      PF_CUDA(cudaStreamWaitEvent(copy, fork_, 0));
      aux_forked_[copy_index] = 1;
    }
    if (slot.used) PF_CUDA(cudaStreamWaitEvent(copy, slot.drained, 0));
    if (group_dense_)
      PF_CUDA(cudaMemcpyAsync(slot.ptr, group_host_begin_, group_bytes_, cudaMemcpyHostToDevice, copy));
    else
      PF_CUDA(cudaMemcpy2DAsync(slot.ptr, first.item_bytes, first.host, first.host_stride, first.item_bytes,
                                first.n_items, cudaMemcpyHostToDevice, copy));
    PF_CUDA(cudaEventRecord(slot.filled, copy));
    PF_CUDA(cudaStreamWaitEvent(stream, slot.filled, 0));
    std::vector<char *> ptrs(group_.size(), slot.ptr);
    for (size_t i = 0; i < group_.size(); i += kMaxGroupUnits)
      launch_group(group_.data() + i, ptrs.data() + i, std::min<size_t>(kMaxGroupUnits, group_.size() - i), false, stream);
    PF_CUDA(cudaEventRecord(slot.drained, stream));
    slot.used = true;
    ++stats_.dma_copies;
    stats_.bytes_staged += group_bytes_;
    group_.clear();
  }
  group_bytes_ = 0;
  group_limit_ = std::min(group_limit_ * 2, cfg_.staging_slot_bytes);  // ramp up: the first DMAs start early
}

// One gather launch for every held save group, then one DMA per group on its copy stream.
void TransferBackend::emit_held() {
  if (held_.empty()) return;
  cudaStream_t stream = held_.front().stream;
  // A slot that an earlier save still drains is waited for first.
  for (const HeldGroup &h : held_)
    if (h.slot->used) PF_CUDA(cudaStreamWaitEvent(stream, h.slot->drained, 0));
  launch_held(held_, true, stream);
  if (held_.front().copy_index >= 0) {   // (gather_layers: the kernels alone, nothing leaves the ring)
    cudaEvent_t filled = held_.front().slot->filled;
    PF_CUDA(cudaEventRecord(filled, stream));
    for (const HeldGroup &h : held_) {
      cudaStream_t copy = aux_[h.copy_index];
      const StagedUnit &first = h.units.front();
      PF_CUDA(cudaStreamWaitEvent(copy, filled, 0));
      if (h.dense)
        PF_CUDA(cudaMemcpyAsync(h.host_begin, h.slot->ptr, h.bytes, cudaMemcpyDeviceToHost, copy));
      else
        PF_CUDA(cudaMemcpy2DAsync(first.host, first.host_stride, h.slot->ptr, first.item_bytes, first.item_bytes,
                                  first.n_items, cudaMemcpyDeviceToHost, copy));
      PF_CUDA(cudaEventRecord(h.slot->drained, copy));
      h.slot->used = true;
      ++stats_.dma_copies;
      stats_.bytes_staged += h.bytes;
    }
  }
  held_.clear();
}

void TransferBackend::gather_layers(const pf_layer_xfer *layers, size_t n_layers, cudaStream_t stream) {
  // Every run must be one the staged route gathers: anything else would move bytes to the host.
  for (size_t li = 0; li < n_layers; ++li) {
    const pf_layer_xfer &L = layers[li];
    if (L.n_blocks == 0) continue;
    if (!L.block_ids || L.n_ranges < 1 || L.n_ranges > 2 || L.range_bytes == 0 ||
        L.range_bytes > cfg_.staging_slot_bytes)
      throw Error::invalid(strf("layer %zu: not a staged transfer", li));
    for (uint32_t r = 0; r < L.n_ranges; ++r)
      for (size_t j = 0; j < L.n_runs[r]; ++j) {
        const pf_host_run &run = L.runs[r][j];
        if (run.n_blocks == 0) continue;
        if (run.first_block + run.n_blocks > L.n_blocks)
          throw Error::invalid(strf("layer %zu range %u: host run outside the block list", li, r));
        const bool staged = cfg_.route == PF_ROUTE_STAGED ||
                            (cfg_.route == PF_ROUTE_AUTO && run.n_blocks * L.range_bytes >= cfg_.min_dma_bytes);
        bool consecutive = run.n_blocks >= 2;
        for (size_t k = 1; k < run.n_blocks && consecutive; ++k)
          consecutive = L.block_ids[run.first_block + k] == L.block_ids[run.first_block + k - 1] + 1;
        if (!staged || consecutive)
          throw Error::invalid(strf("layer %zu range %u run %zu: takes a route without a gather kernel", li, r, j));
      }
  }
  size_t total_bytes = 0;
  for (size_t li = 0; li < n_layers; ++li) total_bytes += layers[li].n_blocks * layers[li].range_bytes * layers[li].n_ranges;
  if (cfg_.route != PF_ROUTE_STAGED && n_layers > 1 && total_bytes <= kSmallTaskBytes)
    throw Error::invalid("task small enough for the single zero-copy launch: no gather kernel");
  struct Reset {
    bool &flag;
    ~Reset() { flag = false; }
  } reset{gather_only_};
  gather_only_ = true;
  move_layers(layers, n_layers, false, stream, nullptr);
}

void TransferBackend::move_layers(const pf_layer_xfer *layers, size_t n_layers, bool host_is_src,
                                  cudaStream_t stream, void *const *layer_done) {
  DeviceGuard on_device(device_);
  size_t total_bytes = 0;
  for (size_t li = 0; li < n_layers; ++li) total_bytes += layers[li].n_blocks * layers[li].range_bytes * layers[li].n_ranges;
  // Small tasks (a few blocks of every layer, e.g. the tail blocks saved while decoding): launches,
  // not bytes, are what they cost, so everything goes into the one zero-copy launch.
  const bool small_task = cfg_.route != PF_ROUTE_STAGED && n_layers > 1 && total_bytes <= kSmallTaskBytes;
  // Every host run takes one of three routes: staged (gather kernel + copy engine; consecutive block
  // ids: one pitched DMA instead) or zero-copy.
  auto takes_staged_route = [&](const pf_layer_xfer &L, const pf_host_run &run) {
    if (L.range_bytes > cfg_.staging_slot_bytes || small_task) return false;
    return cfg_.route == PF_ROUTE_STAGED ||
           (cfg_.route == PF_ROUTE_AUTO && run.n_blocks * L.range_bytes >= cfg_.min_dma_bytes);
  };

  // ---- validate everything before anything is enqueued, and size the meta region: the block ids of
  // every layer, one zero-copy unit per device range, and for ranges whose zero-copy runs do not form
  // one strided sequence a table of their blocks' pool addresses (8 B) and ids (4 B).
  size_t ids_bytes = 0, table_items = 0;
  std::vector<size_t> ids_off(n_layers, 0);
  for (size_t li = 0; li < n_layers; ++li) {
    const pf_layer_xfer &L = layers[li];
    if (L.n_blocks == 0) continue;
    if (L.n_ranges < 1 || L.n_ranges > 2) throw Error::invalid(strf("layer %zu: n_ranges must be 1 or 2", li));
    if (L.range_bytes == 0 || L.range_bytes > 0xFFFFFFFFull)
      throw Error::invalid(strf("layer %zu: range_bytes %zu unsupported", li, L.range_bytes));
    if (L.n_blocks > 0xFFFFFFFFull) throw Error::invalid("too many blocks in one layer transfer");
    if (!L.block_ids) throw Error::invalid(strf("layer %zu: block_ids is null", li));
    ids_off[li] = ids_bytes;
    ids_bytes += align_up(L.n_blocks * sizeof(uint32_t), 256);
    for (uint32_t r = 0; r < L.n_ranges; ++r) {
      size_t covered = 0, zc_runs = 0, zc_items = 0;
      const pf_host_run *runs = L.runs[r];
      for (size_t j = 0; j < L.n_runs[r]; ++j) {
        const pf_host_run &run = runs[j];
        if (run.first_block != covered)
          throw Error::invalid(strf("layer %zu range %u: host runs must cover the blocks in order", li, r));
        if (run.n_blocks && (!run.host || !run.host_device))
          throw Error::invalid(strf("layer %zu range %u: host run without an address", li, r));
        if (run.n_blocks > 1 && run.stride_bytes < L.range_bytes)
          throw Error::invalid(strf("layer %zu range %u: host stride smaller than the range", li, r));
        covered += run.n_blocks;
        if (run.n_blocks && !takes_staged_route(L, run)) {
          ++zc_runs;
          zc_items += run.n_blocks;
        }
      }
      if (covered != L.n_blocks)
        throw Error::invalid(strf("layer %zu range %u: host runs cover %zu of %zu blocks", li, r, covered, L.n_blocks));
      if (zc_runs > 1) table_items += zc_items;
    }
  }
  if (ids_bytes == 0) {
    if (layer_done)
      for (size_t li = 0; li < n_layers; ++li)
        if (layer_done[li]) PF_CUDA(cudaEventRecord((cudaEvent_t)layer_done[li], stream));
    return;
  }

  // The ids go up now; units and tables are filled layer by layer and uploaded just before the launch
  // that reads them, so the first transfer is on its way after one layer has been planned.
  const size_t units_off = ids_bytes;
  const size_t tables_off = units_off + align_up(2 * n_layers * sizeof(LinkUnit), 256);
  const size_t zids_off = tables_off + align_up(table_items * sizeof(uint64_t), 256);
  const size_t meta_bytes = zids_off + align_up(table_items * sizeof(uint32_t), 256);
  const size_t base = meta_alloc(meta_bytes);
  for (size_t li = 0; li < n_layers; ++li)
    if (layers[li].n_blocks)
      std::memcpy(meta_host_ + base + ids_off[li], layers[li].block_ids, layers[li].n_blocks * sizeof(uint32_t));
  meta_upload(base, ids_bytes, stream);
  LinkUnit *units = reinterpret_cast<LinkUnit *>(meta_host_ + base + units_off);
  uint64_t *table = reinterpret_cast<uint64_t *>(meta_host_ + base + tables_off);
  uint32_t *zids = reinterpret_cast<uint32_t *>(meta_host_ + base + zids_off);
  const LinkUnit *units_dev = reinterpret_cast<const LinkUnit *>(meta_dev_ + base + units_off);
  const uint64_t *table_dev = reinterpret_cast<const uint64_t *>(meta_dev_ + base + tables_off);
  const uint32_t *zids_dev = reinterpret_cast<const uint32_t *>(meta_dev_ + base + zids_off);
  size_t n_units = 0, n_table = 0, table_uploaded = 0;
  uint64_t chunk_total = 0;

  group_limit_ = kFirstGroupBytes;
  std::fill(aux_task_dirty_.begin(), aux_task_dirty_.end(), 0);
  std::fill(aux_forked_.begin(), aux_forked_.end(), 0);
  if (host_is_src) PF_CUDA(cudaEventRecord(fork_, stream));
  // Zero-copy units not launched yet: [link_first, n_units) of the table.
  size_t link_first = 0;
  uint64_t link_bytes = 0;
  auto flush_link = [&]() {
    if (n_units == link_first) return;
    const uint64_t chunk_begin = link_first ? units[link_first - 1].chunk_end : 0;
    const uint64_t chunks = units[n_units - 1].chunk_end - chunk_begin;
    const int ctas = cfg_.link_ctas > 0 ? cfg_.link_ctas : 16;
    meta_upload(base + units_off + link_first * sizeof(LinkUnit), (n_units - link_first) * sizeof(LinkUnit), stream);
    if (n_table > table_uploaded) {
      meta_upload(base + tables_off + table_uploaded * sizeof(uint64_t), (n_table - table_uploaded) * sizeof(uint64_t), stream);
      meta_upload(base + zids_off + table_uploaded * sizeof(uint32_t), (n_table - table_uploaded) * sizeof(uint32_t), stream);
      table_uploaded = n_table;
    }
    cudaEvent_t t0;
    time_begin(stream, &t0);
    copy_units_tma<<<(int)std::min<uint64_t>(chunks, (uint64_t)ctas), 32, (size_t)kStages * kStageBytes, stream>>>(
        units_dev + link_first, (uint32_t)(n_units - link_first), chunk_begin, host_is_src ? 0 : 1, status_dev_);
    PF_CUDA(cudaGetLastError());
    time_end(stream, t0, link_bytes, true, -1);
    ++stats_.kernel_launches;
    stats_.bytes_zero_copy += link_bytes;
    link_first = n_units;
    link_bytes = 0;
  };
  // Appends the unit of one device range; `n_items` items of `item_bytes`.
  auto add_unit = [&](uint64_t dev_base, uint64_t dev_stride, const uint32_t *ids_dev_ptr, size_t n_items, size_t item_bytes,
                      uint64_t host_base, uint64_t host_stride, const uint64_t *host_table_dev) {
    LinkUnit &u = units[n_units++];
    u.kv_base = dev_base;
    u.kv_stride = dev_stride;
    u.host_base = host_base;
    u.host_stride = host_stride;
    u.host_table = host_table_dev;
    u.ids = ids_dev_ptr;
    u.n_items = (uint32_t)n_items;
    u.item_bytes = (uint32_t)item_bytes;
    u.items_per_chunk = (uint32_t)std::min<size_t>(kLinkItemsMax, kStageBytes / item_bytes);
    u.chunks_per_item = (uint32_t)((item_bytes + kStageBytes - 1) / kStageBytes);
    // an item larger than a ring stage is cut into equal chunks (a multiple of 128 bytes each)
    u.chunk_bytes = (uint32_t)std::min<size_t>(kStageBytes, align_up((item_bytes + u.chunks_per_item - 1) / u.chunks_per_item, 128));
    u.pad_ = 0;
    chunk_total += u.items_per_chunk >= 2 ? (n_items + u.items_per_chunk - 1) / u.items_per_chunk
                                          : (uint64_t)n_items * u.chunks_per_item;
    u.chunk_end = chunk_total;
    link_bytes += n_items * item_bytes;
  };
  // Events of layers whose bytes are still in an open (small) group or launch wait here until it is flushed.
  std::vector<cudaEvent_t> deferred;
  bool layer_stream = false;
  for (size_t li = 0; li < n_layers; ++li) {
    const pf_layer_xfer &L = layers[li];
    if (deferred.empty()) {
      layer_stream = false;
      std::fill(aux_layer_dirty_.begin(), aux_layer_dirty_.end(), 0);
    }
    if (L.n_blocks) {
      const uint32_t *ids_dev = reinterpret_cast<const uint32_t *>(meta_dev_ + base + ids_off[li]);
      for (uint32_t r = 0; r < L.n_ranges; ++r) {
        const uint64_t dev_base = L.data_ptr + (uint64_t)r * L.kv_stride_bytes;
        // how this range's zero-copy runs travel: one strided unit, one table-driven unit, or (an
        // address or size that is not a multiple of 16) the ld/st kernel run by run
        size_t zc_runs = 0;
        bool zc_aligned = ((dev_base | L.block_stride_bytes | L.range_bytes) & 15ull) == 0;
        for (size_t j = 0; j < L.n_runs[r]; ++j) {
          const pf_host_run &run = L.runs[r][j];
          if (run.n_blocks == 0 || takes_staged_route(L, run)) continue;
          ++zc_runs;
          if ((run.host_device | (run.n_blocks > 1 ? run.stride_bytes : 0)) & 15ull) zc_aligned = false;
        }
        const size_t table_first = n_table;
        for (size_t j = 0; j < L.n_runs[r]; ++j) {
          const pf_host_run &run = L.runs[r][j];
          if (run.n_blocks == 0) continue;
          const size_t bytes = run.n_blocks * L.range_bytes;
          if (!takes_staged_route(L, run)) {
            if (!zc_aligned) {
              const Side dev{dev_base, L.block_stride_bytes, ids_dev + run.first_block, nullptr};
              const Side host{run.host_device, run.stride_bytes, nullptr, nullptr};
              if (host_is_src) launch_link(host, dev, run.n_blocks, L.range_bytes, stream, false);
              else launch_link(dev, host, run.n_blocks, L.range_bytes, stream, false);
              stats_.bytes_zero_copy += bytes;
            } else if (zc_runs == 1) {
              add_unit(dev_base, L.block_stride_bytes, ids_dev + run.first_block, run.n_blocks, L.range_bytes,
                       run.host_device, run.n_blocks > 1 ? run.stride_bytes : L.range_bytes, nullptr);
            } else {
              for (size_t i = 0; i < run.n_blocks; ++i, ++n_table) {
                table[n_table] = run.host_device + (uint64_t)i * run.stride_bytes;
                zids[n_table] = L.block_ids[run.first_block + i];
              }
            }
            layer_stream = true;
            continue;
          }
          // Consecutive block ids (a fresh prompt usually gets them from an ordered free list) are
          // one strided region on the device as well: a single pitched DMA, nothing to gather.  It
          // runs on the caller's stream like the zero-copy launches, which keeps the layer's event
          // and the ordering rules unchanged.
          const uint32_t *ids = L.block_ids + run.first_block;
          const bool linear = L.block_stride_bytes == L.range_bytes && run.stride_bytes == L.range_bytes;
          // (pitched rows are only worth a DMA of their own when they are long: the staged route
          // already turns short padded rows into large linear copies)
          bool consecutive = run.n_blocks >= 2 && L.block_stride_bytes >= L.range_bytes &&
                             run.stride_bytes >= L.range_bytes && (linear || L.range_bytes >= (32u << 10));
          for (size_t k = 1; k < run.n_blocks && consecutive; ++k) consecutive = ids[k] == ids[k - 1] + 1;
          if (consecutive) {
            char *device_first = reinterpret_cast<char *>(dev_base + (uint64_t)ids[0] * L.block_stride_bytes);
            if (host_is_src)
              PF_CUDA(cudaMemcpy2DAsync(device_first, L.block_stride_bytes, run.host, run.stride_bytes, L.range_bytes,
                                        run.n_blocks, cudaMemcpyHostToDevice, stream));
            else
              PF_CUDA(cudaMemcpy2DAsync(run.host, run.stride_bytes, device_first, L.block_stride_bytes, L.range_bytes,
                                        run.n_blocks, cudaMemcpyDeviceToHost, stream));
            ++stats_.dma_copies;
            stats_.bytes_staged += bytes;
            layer_stream = true;
            continue;
          }
          const Side dev{dev_base, L.block_stride_bytes, ids_dev + run.first_block, nullptr};
          staged_run(dev, run, L.range_bytes, host_is_src, stream);
        }
        if (n_table > table_first)
          add_unit(dev_base, L.block_stride_bytes, zids_dev + table_first, n_table - table_first, L.range_bytes, 0, 0,
                   table_dev + table_first);
      }
    }
    cudaEvent_t done = layer_done ? (cudaEvent_t)layer_done[li] : nullptr;
    if (done) deferred.push_back(done);
    // A layer's event should not wait for later layers - unless its bytes are so few that a DMA or a
    // launch of its own would waste the link: then it shares the group, and the event, of its successors.
    const bool last = li + 1 == n_layers;
    const bool keep_open = !last && ((!group_.empty() && group_bytes_ < kMinEventGroupBytes) ||
                                     (n_units > link_first && link_bytes < kMinLinkLaunchBytes));
    if (!deferred.empty() && !keep_open) {
      flush_group(false);
      flush_link();
      // Saved layers are complete when their DMAs (copy streams) and zero-copy kernels (caller's
      // stream) are; loaded layers always end with a scatter on the caller's stream.
      const bool layer_aux = std::find(aux_layer_dirty_.begin(), aux_layer_dirty_.end(), 1) != aux_layer_dirty_.end();
      cudaStream_t where = stream;
      if (!host_is_src && layer_aux && !layer_stream) {
        // Signal from the copy stream that took the last DMA, after the others.
        join_copy_streams(aux_[aux_last_], aux_layer_dirty_, aux_last_);
        where = aux_[aux_last_];
      } else if (!host_is_src && layer_aux) {
        join_copy_streams(stream, aux_layer_dirty_, -1);
      }
      for (cudaEvent_t ev : deferred) PF_CUDA(cudaEventRecord(ev, where));
      deferred.clear();
    }
  }
  flush_group(false);
  flush_link();
  if (!host_is_src) join_copy_streams(stream, aux_task_dirty_, -1);
  // The meta region is free once everything enqueued above has run.
  cudaEvent_t ev = take_event();
  PF_CUDA(cudaEventRecord(ev, stream));
  meta_inflight_.push_back({base, base + align_up(std::max<size_t>(meta_bytes, 16), 256), ev});
}

void TransferBackend::copy_descs(const pf_copy_desc *copies, size_t n, bool host_is_src, cudaStream_t stream) {
  if (n == 0) return;
  DeviceGuard on_device(device_);
  if (n > 0xFFFFFFFFull) throw Error::invalid("too many copy descriptors in one batch");
  // Split the batch: maximal runs of equally sized descriptors whose host side is contiguous
  // go through the staging ring (the device side may be scattered); the rest become
  // [dst, src, size] triples for the zero-copy kernel.
  //
  // Fast path first: equally sized descriptors whose host sides tile one dense range - every slot
  // of the range hit exactly once, in whatever order they arrive - need no run detection at all.
  // The device addresses go straight into the table in slot order (a counting sort, O(n)) and the
  // whole batch is a single staged run, or one plain DMA when the device side is dense as well.
  // (The outcome of a batch does not depend on descriptor order: destinations do not overlap.)
  if (n >= 2 && cfg_.route != PF_ROUTE_ZEROCOPY && copies[0].size > 0 && copies[0].size <= cfg_.staging_slot_bytes &&
      copies[0].size <= 0xFFFFFFFFull && (cfg_.route == PF_ROUTE_STAGED || n * copies[0].size >= cfg_.min_dma_bytes)) {
    const size_t sz = copies[0].size;
    uintptr_t lo = (uintptr_t)copies[0].host;
    bool uniform = true, in_order = true;   // in_order: already ascending and dense on both sides
    for (size_t i = 0; i < n && uniform; ++i) {
      const uintptr_t h = (uintptr_t)copies[i].host;
      uniform = copies[i].size == sz && copies[i].device != 0 && h != 0 &&
                copies[i].host_device - copies[0].host_device == (uint64_t)(h - (uintptr_t)copies[0].host);
      if (i) in_order = in_order && h == (uintptr_t)copies[i - 1].host + sz && copies[i].device == copies[i - 1].device + sz;
      lo = std::min(lo, h);
    }
    if (uniform && in_order) {
      const size_t bytes = n * sz;
      if (host_is_src)
        PF_CUDA(cudaMemcpyAsync((void *)(uintptr_t)copies[0].device, copies[0].host, bytes, cudaMemcpyHostToDevice, stream));
      else
        PF_CUDA(cudaMemcpyAsync(copies[0].host, (const void *)(uintptr_t)copies[0].device, bytes, cudaMemcpyDeviceToHost, stream));
      ++stats_.dma_copies;
      stats_.bytes_staged += bytes;
      return;
    }
    if (uniform) {
      const size_t table_bytes = align_up(n * sizeof(uint64_t), 256);
      const size_t base = meta_alloc(table_bytes);
      uint64_t *table = reinterpret_cast<uint64_t *>(meta_host_ + base);
      std::memset(table, 0, n * sizeof(uint64_t));
      bool tiles = true;
      for (size_t i = 0; i < n && tiles; ++i) {
        const uintptr_t d = (uintptr_t)copies[i].host - lo;
        const size_t slot = d / sz;
        tiles = d % sz == 0 && slot < n && table[slot] == 0;
        if (tiles) table[slot] = copies[i].device;
      }
      if (tiles) {
        bool dense = true;
        for (size_t k = 1; k < n && dense; ++k) dense = table[k] == table[k - 1] + sz;
        char *host_lo = reinterpret_cast<char *>(lo);
        const uint64_t host_dev_lo = copies[0].host_device - (uint64_t)((uintptr_t)copies[0].host - lo);
        if (dense) {
          const size_t bytes = n * sz;
          if (host_is_src)
            PF_CUDA(cudaMemcpyAsync((void *)(uintptr_t)table[0], host_lo, bytes, cudaMemcpyHostToDevice, stream));
          else
            PF_CUDA(cudaMemcpyAsync(host_lo, (const void *)(uintptr_t)table[0], bytes, cudaMemcpyDeviceToHost, stream));
          ++stats_.dma_copies;
          stats_.bytes_staged += bytes;
          meta_head_ = base;  // nothing was uploaded: the region is handed out again
          return;
        }
        meta_upload(base, table_bytes, stream);
        std::fill(aux_task_dirty_.begin(), aux_task_dirty_.end(), 0);
        std::fill(aux_forked_.begin(), aux_forked_.end(), 0);
        group_limit_ = kFirstGroupBytes;
        if (host_is_src) PF_CUDA(cudaEventRecord(fork_, stream));
        const Side dev{0, 0, nullptr, reinterpret_cast<const uint64_t *>(meta_dev_ + base)};
        staged_run(dev, pf_host_run{0, n, host_lo, host_dev_lo, sz}, sz, host_is_src, stream);
        flush_group(false);
        if (!host_is_src) join_copy_streams(stream, aux_task_dirty_, -1);
        cudaEvent_t ev = take_event();
        PF_CUDA(cudaEventRecord(ev, stream));
        meta_inflight_.push_back({base, base + table_bytes, ev});
        return;
      }
      // not a tiling (gaps, duplicates, mixed strides): the general path below; the table region is
      // simply handed out again, nothing in flight refers to it
      meta_head_ = base;
    }
  }

  // A run whose device side is contiguous as well needs no gather at all: it is one plain DMA,
  // which is what the reference's merge rule produces for it (memcpy.rs:25-55).
  struct Run {
    size_t first, count;
    bool dense;
  };
  std::vector<Run> staged;
  std::vector<char> is_staged(n, 0);   // 0: zero-copy descriptor, 1: staged through the ring, 2: part of a dense run
  size_t n_staged = 0, n_dense = 0;
  if (cfg_.route != PF_ROUTE_ZEROCOPY) {
    size_t i = 0;
    while (i < n) {
      size_t j = i + 1;
      const size_t sz = copies[i].size;
      bool dense = true;
      while (j < n && copies[j].size == sz &&
             (char *)copies[j].host == (char *)copies[j - 1].host + sz &&
             copies[j].host_device == copies[j - 1].host_device + sz &&
             copies[j].host_allocation == copies[i].host_allocation) {
        dense = dense && copies[j].device == copies[j - 1].device + sz;
        ++j;
      }
      const size_t bytes = (j - i) * sz;
      const bool want = cfg_.route == PF_ROUTE_STAGED || bytes >= cfg_.min_dma_bytes;
      if (want && sz > 0 && dense && copies[i].device && copies[i].host) {
        staged.push_back({i, j - i, true});
        for (size_t k = i; k < j; ++k) is_staged[k] = 2;
        n_dense += j - i;
      } else if (want && sz > 0 && sz <= cfg_.staging_slot_bytes && sz <= 0xFFFFFFFFull) {
        staged.push_back({i, j - i, false});
        for (size_t k = i; k < j; ++k) is_staged[k] = 1;
        n_staged += j - i;
      }
      i = j;
    }
  }
  const size_t n_direct = n - n_staged - n_dense;
  const size_t table_bytes = align_up(n_staged * sizeof(uint64_t), 256);
  const size_t triple_bytes = align_up(n_direct * 3 * sizeof(uint64_t), 256);
  const size_t meta_bytes = table_bytes + triple_bytes;
  const size_t base = meta_alloc(meta_bytes);
  uint64_t *table = reinterpret_cast<uint64_t *>(meta_host_ + base);
  uint64_t *triples = reinterpret_cast<uint64_t *>(meta_host_ + base + table_bytes);
  bool aligned = true;
  size_t t = 0, q = 0;
  for (size_t i = 0; i < n; ++i) {
    const pf_copy_desc &c = copies[i];
    if (is_staged[i] == 2) continue;
    if (is_staged[i] == 1) {
      table[t++] = c.device;
    } else {
      if (c.size && (!c.device || !c.host_device)) throw Error::invalid(strf("copy descriptor %zu has a null address", i));
      triples[3 * q + 0] = host_is_src ? c.device : c.host_device;
      triples[3 * q + 1] = host_is_src ? c.host_device : c.device;
      triples[3 * q + 2] = c.size;
      if ((c.device | c.host_device | c.size) & 15ull) aligned = false;
      stats_.bytes_zero_copy += c.size;
      ++q;
    }
  }
  if (meta_bytes) meta_upload(base, meta_bytes, stream);
  std::fill(aux_task_dirty_.begin(), aux_task_dirty_.end(), 0);
  std::fill(aux_forked_.begin(), aux_forked_.end(), 0);
  group_limit_ = kFirstGroupBytes;
  if (host_is_src) PF_CUDA(cudaEventRecord(fork_, stream));
  size_t table_cursor = 0;
  for (auto &r : staged) {
    const pf_copy_desc &c0 = copies[r.first];
    if (r.dense) {
      const size_t bytes = r.count * c0.size;
      if (host_is_src)
        PF_CUDA(cudaMemcpyAsync((void *)(uintptr_t)c0.device, c0.host, bytes, cudaMemcpyHostToDevice, stream));
      else
        PF_CUDA(cudaMemcpyAsync(c0.host, (const void *)(uintptr_t)c0.device, bytes, cudaMemcpyDeviceToHost, stream));
      ++stats_.dma_copies;
      stats_.bytes_staged += bytes;
      continue;
    }
    const Side dev{0, 0, nullptr, reinterpret_cast<const uint64_t *>(meta_dev_ + base) + table_cursor};
    const pf_host_run run{0, r.count, c0.host, c0.host_device, c0.size};
    staged_run(dev, run, c0.size, host_is_src, stream);
    table_cursor += r.count;
  }
  flush_group(false);
  launch_descs(reinterpret_cast<const uint64_t *>(meta_dev_ + base + table_bytes), n_direct, aligned, stream);
  if (!host_is_src) join_copy_streams(stream, aux_task_dirty_, -1);
  cudaEvent_t ev = take_event();
  PF_CUDA(cudaEventRecord(ev, stream));
  meta_inflight_.push_back({base, base + align_up(std::max<size_t>(meta_bytes, 16), 256), ev});
}

void TransferBackend::peer_copy(const pf_device_layout &src, const uint32_t *src_ids, const pf_device_layout &dst,
                                const uint32_t *dst_ids, size_t n_blocks, cudaStream_t stream) {
  peer_copy_layers(&src, &dst, 1, src_ids, dst_ids, n_blocks, stream);
}

void TransferBackend::peer_copy_layers(const pf_device_layout *src, const pf_device_layout *dst, size_t n_layers,
                                       const uint32_t *src_ids, const uint32_t *dst_ids, size_t n_blocks,
                                       cudaStream_t stream) {
  if (n_blocks == 0 || n_layers == 0) return;
  DeviceGuard on_device(device_);
  for (size_t l = 0; l < n_layers; ++l) {
    if (src[l].n_ranges != dst[l].n_ranges || src[l].range_bytes != dst[l].range_bytes)
      throw Error::invalid("peer copy needs the same block geometry on both sides");
    if (src[l].n_ranges < 1 || src[l].n_ranges > 2 || src[l].range_bytes == 0 || src[l].range_bytes > 0xFFFFFFFFull)
      throw Error::invalid("peer copy: unsupported block geometry");
  }
  if (n_blocks > 0xFFFFFFFFull) throw Error::invalid("peer copy: too many blocks");
  for (size_t l = 0; l < n_layers; ++l)
    for (int side = 0; side < 2; ++side) {
      const pf_device_layout &lay = side ? dst[l] : src[l];
      const uint32_t *ids = side ? dst_ids : src_ids;
      if (!lay.num_blocks) continue;  // not stated: the ids are trusted
      for (size_t i = 0; i < n_blocks; ++i)
        if (ids[i] >= lay.num_blocks)
          throw Error::invalid(strf("peer copy: block_id %u out of range (num_blocks=%zu) for layer %zu", ids[i],
                                    lay.num_blocks, l));
    }
  // one upload of the ids serves every layer
  const size_t ids_bytes = align_up(n_blocks * sizeof(uint32_t), 256);
  const size_t base = meta_alloc(2 * ids_bytes);
  std::memcpy(meta_host_ + base, src_ids, n_blocks * sizeof(uint32_t));
  std::memcpy(meta_host_ + base + ids_bytes, dst_ids, n_blocks * sizeof(uint32_t));
  meta_upload(base, 2 * ids_bytes, stream);
  const uint32_t *sids_dev = reinterpret_cast<const uint32_t *>(meta_dev_ + base);
  const uint32_t *dids_dev = reinterpret_cast<const uint32_t *>(meta_dev_ + base + ids_bytes);
  tables_aligned_ = true;

  PeerParams p;
  p.src_ids = sids_dev;
  p.dst_ids = dids_dev;
  p.n_items = (uint32_t)n_blocks;
  p.n_units = 0;
  p.item_bytes = 0;
  auto flush = [&]() {
    if (p.n_units == 0) return;
    const uint64_t pieces = (uint64_t)p.n_units * p.n_items * p.pieces_per_item;
    const uint64_t want = (pieces + kLdstThreads / 32 - 1) / (kLdstThreads / 32);
    const int ctas = cfg_.link_ctas > 0 ? cfg_.link_ctas : cfg_.pack_ctas;
    cudaEvent_t t0;
    time_begin(stream, &t0);
    copy_peer_warp<<<(int)std::min<uint64_t>(want, (uint64_t)ctas), kLdstThreads, 0, stream>>>(p);
    PF_CUDA(cudaGetLastError());
    time_end(stream, t0, (uint64_t)p.n_units * p.n_items * p.item_bytes, true, -1);
    ++stats_.kernel_launches;
    p.n_units = 0;
  };
  for (size_t l = 0; l < n_layers; ++l) {
    const size_t bytes = src[l].range_bytes;
    const uint64_t pieces_per_item = (bytes + kWarpPiece - 1) / kWarpPiece;
    for (uint32_t r = 0; r < src[l].n_ranges; ++r) {
      const uint64_t sb = src[l].data_ptr + (uint64_t)r * src[l].kv_stride_bytes;
      const uint64_t db = dst[l].data_ptr + (uint64_t)r * dst[l].kv_stride_bytes;
      const bool fits = ((sb | db | src[l].block_stride_bytes | dst[l].block_stride_bytes | bytes) & 15ull) == 0 &&
                        n_blocks * pieces_per_item <= 0xFFFFFFFFull;
      if (!fits) {
        flush();
        launch_link(Side{sb, src[l].block_stride_bytes, sids_dev, nullptr},
                    Side{db, dst[l].block_stride_bytes, dids_dev, nullptr}, n_blocks, bytes, stream, true);
      } else {
        if (p.n_units == kMaxPeerUnits || (p.n_units && p.item_bytes != bytes)) flush();
        p.item_bytes = (uint32_t)bytes;
        p.pieces_per_item = (uint32_t)pieces_per_item;
        p.unit[p.n_units++] = PeerUnit{sb, src[l].block_stride_bytes, db, dst[l].block_stride_bytes};
      }
      stats_.bytes_peer += n_blocks * bytes;
    }
  }
  flush();
  cudaEvent_t ev = take_event();
  PF_CUDA(cudaEventRecord(ev, stream));
  meta_inflight_.push_back({base, base + 2 * ids_bytes, ev});
}

void enable_peer_access(int device, int peer) {
  DeviceGuard on_device(device);
  int can = 0;
  PF_CUDA(cudaDeviceCanAccessPeer(&can, device, peer));
  if (!can) throw Error::cuda_init(strf("device %d cannot access device %d", device, peer));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return;
  }
  if (e != cudaSuccess) throw Error::cuda_init(strf("cudaDeviceEnablePeerAccess(%d->%d): %s", device, peer, cudaGetErrorString(e)));
}

}  // namespace pf

// ------------------------------------------------------------------------------------------------
// Allocation-free save of a few blocks.
//
// Some callers of this library must not allocate device memory at the moment they want KV
// blocks copied out: a serving process that has handed all free HBM to its KV cache (a late
// cudaMalloc simply fails there), a latency-critical scheduler thread (cudaMalloc and cudaFree
// synchronise the whole device), or code that runs while another thread is capturing a stream.
// For them the gather -> staging -> DMA sequence of the staged route is offered with the
// staging area (and the block-id table) inside the library image instead of on the heap.
//
// The array below is file-scope device memory: every GPU that loads the library carries it
// until the process exits.  In host code its name is only a handle for the runtime, not an
// address a kernel could use, so each device's address is looked up once with
// cudaGetSymbolAddress while that device is current.
namespace pf {
namespace {
constexpr size_t kNoAllocPayload = PF_NOALLOC_MAX_PAYLOAD_BYTES;
constexpr size_t kNoAllocIds = (size_t)PF_NOALLOC_MAX_BLOCKS * sizeof(uint32_t);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocPayload + kNoAllocIds];

struct NoAllocDevice {
  unsigned char *scratch = nullptr;  // device address of g_noalloc_scratch on this GPU
  int sm_count = 0;
};
std::mutex g_noalloc_mu;
NoAllocDevice g_noalloc_devices[64];

// First use on a device: resolve the symbol with that device current.
const NoAllocDevice &noalloc_device(int device) {
  if (device < 0 || device >= 64) throw Error::invalid(strf("device %d out of range", device));
  std::lock_guard<std::mutex> g(g_noalloc_mu);
  NoAllocDevice &d = g_noalloc_devices[device];
  if (!d.scratch) {
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr)
      throw Error::cuda_init(strf("cudaGetSymbolAddress for the built-in staging area failed on device %d: %s", device,
                                  cudaGetErrorString(e)));
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess || sms <= 0) throw Error::cuda_init("cudaDeviceGetAttribute(multiProcessorCount) failed");
    d.sm_count = sms;
    d.scratch = static_cast<unsigned char *>(ptr);
  }
  return d;
}
}  // namespace
}  // namespace pf

extern "C" int pf_save_blocks_noalloc(int device_id, const pf_device_layout *layout, const uint32_t *block_ids,
                                      size_t n_blocks, void *host_dst, size_t host_dst_bytes, void *stream) {
  using namespace pf;
  return guarded([&] {
    if (!layout || (!block_ids && n_blocks) || (!host_dst && n_blocks)) throw Error::invalid("null argument");
    if (layout->n_ranges < 1 || layout->n_ranges > 2 || layout->range_bytes == 0)
      throw Error::invalid("unsupported block geometry");
    // Any first call on a device, an empty one included, resolves the staging area's address there.
    DeviceGuard on_device(device_id);
    const NoAllocDevice &dev = noalloc_device(device_id);
    if (n_blocks == 0) return;
    if (n_blocks > PF_NOALLOC_MAX_BLOCKS)
      throw Error::invalid(strf("%zu blocks exceed the built-in staging area's limit of %d blocks; use "
                                "pf_backend_save_layers for larger batches",
                                n_blocks, PF_NOALLOC_MAX_BLOCKS));
    const size_t per_range = n_blocks * layout->range_bytes;
    const size_t total = per_range * layout->n_ranges;
    if (layout->range_bytes > 0xFFFFFFFFull || total > kNoAllocPayload)
      throw Error::invalid(strf("%zu bytes exceed the built-in staging area of %zu bytes; use pf_backend_save_layers "
                                "for larger batches",
                                total, kNoAllocPayload));
    if (host_dst_bytes < total)
      throw Error::invalid(strf("destination holds %zu bytes, the blocks need %zu", host_dst_bytes, total));
    // The kernel trusts the ids: a caller that states how many blocks the cache has gets them checked here.
    if (layout->num_blocks)
      for (size_t i = 0; i < n_blocks; ++i)
        if (block_ids[i] >= layout->num_blocks)
          throw Error::invalid(strf("block_id %u out of range (num_blocks=%zu)", block_ids[i], layout->num_blocks));
    cudaStream_t s = (cudaStream_t)stream;
    uint32_t *ids_dev = reinterpret_cast<uint32_t *>(dev.scratch + kNoAllocPayload);
    PF_CUDA(cudaMemcpyAsync(ids_dev, block_ids, n_blocks * sizeof(uint32_t), cudaMemcpyHostToDevice, s));
    for (uint32_t r = 0; r < layout->n_ranges; ++r) {
      const Side src{layout->data_ptr + (uint64_t)r * layout->kv_stride_bytes, layout->block_stride_bytes, ids_dev,
                     nullptr};
      const Side dst{(uint64_t)(uintptr_t)(dev.scratch + r * per_range), layout->range_bytes, nullptr, nullptr};
      const uint64_t chunks = (uint64_t)n_blocks * ((layout->range_bytes + kPackChunk - 1) / kPackChunk);
      const int grid = (int)std::min<uint64_t>(chunks, (uint64_t)dev.sm_count * 8);
      copy_items_ldst<<<grid, kLdstThreads, 0, s>>>(src, dst, (uint32_t)n_blocks, (uint32_t)layout->range_bytes,
                                                       kPackChunk, nullptr);
      PF_CUDA(cudaGetLastError());
    }
    PF_CUDA(cudaMemcpyAsync(host_dst, dev.scratch, total, cudaMemcpyDeviceToHost, s));
  });
}
