// Shared-memory completion word a vLLM worker polls while its KV blocks are loaded.
// Bit-compatible with pegaflow-core/src/sync_state.rs:23-47,190-302: a POSIX shm segment
// "pega_load_<32 hex>" of 32 bytes holding an 8-byte offset word, then at that offset
// {u32 magic 'PFLD', u32 version 1, i64 state}; state is 0 pending, 1 success, -1 error.
#pragma once

#include <atomic>
#include <cstdint>
#include <string>

#include "common.h"

namespace pf {

class LoadState {
 public:
  static constexpr uint32_t kMagic = 0x50464c44;
  static constexpr uint32_t kVersion = 1;
  static constexpr int64_t kPending = 0, kSuccess = 1, kError = -1;
  static constexpr size_t kMappingBytes = 8 + 16 + 8;

  // Creates a fresh segment (state PENDING).  Throws Error::storage("LoadState: ...").
  static LoadState *create();
  // Attaches to an existing segment and validates size, offset and header.
  static LoadState *attach(const std::string &shm_name);
  ~LoadState();

  const std::string &shm_name() const { return name_; }
  int64_t get() const { return state_->load(std::memory_order_acquire); }
  void set_completed() { state_->store(kSuccess, std::memory_order_release); }
  void set_error() { state_->store(kError, std::memory_order_release); }

 private:
  LoadState() = default;
  std::string name_;
  void *map_ = nullptr;
  size_t map_len_ = 0;
  std::atomic<int64_t> *state_ = nullptr;
  bool owner_ = false;
};

}  // namespace pf
