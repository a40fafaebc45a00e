// Shared helpers of the host-side engine: the error type every layer throws and the
// thread-local message the C ABI hands out.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "../../include/pegaflow_b200.h"

namespace pf {

// Mirrors `EngineError` (pegaflow-core/src/lib.rs:72-103): a variant plus the text its
// Display impl would print.
class Error : public std::runtime_error {
 public:
  Error(pf_status status, const std::string &display) : std::runtime_error(display), status_(status) {}
  pf_status status() const { return status_; }

  static Error instance_missing(const std::string &id) {
    return Error(PF_INSTANCE_MISSING, "instance " + id + " not found");
  }
  static Error worker_missing(const std::string &id, int device) {
    return Error(PF_WORKER_MISSING, "device " + std::to_string(device) + " not found in instance " + id);
  }
  static Error invalid(const std::string &msg) { return Error(PF_INVALID_ARGUMENT, "invalid argument: " + msg); }
  static Error cuda_init(const std::string &msg) {
    return Error(PF_CUDA_INIT, "failed to initialize CUDA: " + msg);
  }
  static Error storage(const std::string &msg) { return Error(PF_STORAGE, "storage error: " + msg); }
  static Error topology(const std::string &msg) { return Error(PF_TOPOLOGY_MISMATCH, "topology mismatch: " + msg); }

 private:
  pf_status status_;
};

std::string strf(const char *fmt, ...) __attribute__((format(printf, 1, 2)));

// Thread-local last-error slot behind pf_last_error().
void set_last_error(const std::string &msg);
const char *last_error();

// Runs `fn`, translating exceptions into a status + thread-local message.
template <class F>
int guarded(F &&fn) {
  try {
    fn();
    set_last_error("");
    return PF_OK;
  } catch (const Error &e) {
    set_last_error(e.what());
    return e.status();
  } catch (const std::exception &e) {
    set_last_error(std::string("storage error: ") + e.what());
    return PF_STORAGE;
  }
}

}  // namespace pf
