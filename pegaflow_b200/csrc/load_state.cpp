#include "load_state.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <random>

namespace pf {

namespace {
struct Header {
  std::atomic<uint32_t> magic;
  std::atomic<uint32_t> version;
  std::atomic<int64_t> state;
};
static_assert(sizeof(Header) == 16 && alignof(Header) == 8, "LoadState header layout");

std::string random_hex32() {
  std::random_device rd;
  static const char *digits = "0123456789abcdef";
  std::string s(32, '0');
  for (int i = 0; i < 32; i += 8) {
    uint32_t v = rd();
    for (int k = 0; k < 8; ++k) s[i + k] = digits[(v >> (4 * k)) & 15];
  }
  return s;
}

Error ls_error(const std::string &msg) { return Error::storage("LoadState: " + msg); }
}  // namespace

LoadState *LoadState::create() {
  std::string name = "pega_load_" + random_hex32();
  int fd = shm_open(("/" + name).c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) throw ls_error(strf("failed to create shared memory: %s", strerror(errno)));
  if (ftruncate(fd, kMappingBytes) != 0) {
    close(fd);
    shm_unlink(("/" + name).c_str());
    throw ls_error(strf("failed to create shared memory: %s", strerror(errno)));
  }
  void *map = mmap(nullptr, kMappingBytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (map == MAP_FAILED) {
    shm_unlink(("/" + name).c_str());
    throw ls_error(strf("failed to create shared memory: %s", strerror(errno)));
  }
  // The header sits at the first 8-byte aligned address past the offset word.
  const uintptr_t base = (uintptr_t)map;
  const uintptr_t aligned = (base + 8 + 7) & ~(uintptr_t)7;
  const uint64_t offset = aligned - base;
  std::memcpy(map, &offset, sizeof offset);
  Header *h = reinterpret_cast<Header *>(aligned);
  h->magic.store(kMagic, std::memory_order_release);
  h->version.store(kVersion, std::memory_order_release);
  h->state.store(kPending, std::memory_order_release);
  LoadState *ls = new LoadState();
  ls->name_ = name;
  ls->map_ = map;
  ls->map_len_ = kMappingBytes;
  ls->state_ = &h->state;
  ls->owner_ = true;
  return ls;
}

LoadState *LoadState::attach(const std::string &shm_name) {
  int fd = shm_open(("/" + shm_name).c_str(), O_RDWR, 0600);
  if (fd < 0) throw ls_error(strf("failed to open shared memory: %s", strerror(errno)));
  struct stat st;
  if (fstat(fd, &st) != 0) {
    close(fd);
    throw ls_error(strf("failed to open shared memory: %s", strerror(errno)));
  }
  const size_t len = (size_t)st.st_size;
  if (len < kMappingBytes) {
    close(fd);
    throw ls_error(strf("shared memory too small (actual=%zu bytes, required=%zu bytes)", len, kMappingBytes));
  }
  void *map = mmap(nullptr, len, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (map == MAP_FAILED) throw ls_error(strf("failed to open shared memory: %s", strerror(errno)));
  auto bail = [&](const std::string &msg) {
    munmap(map, len);
    return ls_error(msg);
  };
  uint64_t offset;
  std::memcpy(&offset, map, sizeof offset);
  if (offset < 8) throw bail(strf("invalid LoadState offset (offset=%llu, len=%zu) recorded in shared memory",
                                  (unsigned long long)offset, len));
  if (offset > len || len - offset < sizeof(Header))
    throw bail(strf("shared memory too small (actual=%zu bytes, required=%llu bytes)", len,
                    (unsigned long long)(offset + sizeof(Header))));
  const uintptr_t addr = (uintptr_t)map + offset;
  if (addr % alignof(Header) != 0) throw bail(strf("aligned pointer %#lx is not 8-byte aligned", (unsigned long)addr));
  Header *h = reinterpret_cast<Header *>(addr);
  const uint32_t magic = h->magic.load(std::memory_order_acquire), version = h->version.load(std::memory_order_acquire);
  if (magic != kMagic || version != kVersion)
    throw bail(strf("invalid LoadState header (magic=%#x, version=%u, expected magic=%#x, version=%u)", magic, version,
                    kMagic, kVersion));
  LoadState *ls = new LoadState();
  ls->name_ = shm_name;
  ls->map_ = map;
  ls->map_len_ = len;
  ls->state_ = &h->state;
  ls->owner_ = false;
  return ls;
}

LoadState::~LoadState() {
  if (map_) munmap(map_, map_len_);
  if (owner_) shm_unlink(("/" + name_).c_str());
}

}  // namespace pf
