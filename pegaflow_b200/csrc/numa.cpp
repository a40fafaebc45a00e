#include "numa.h"

#include <cuda_runtime.h>
#include <sched.h>

#include <algorithm>
#include <cctype>
#include <fstream>
#include <set>
#include <sstream>
#include <stdexcept>
#include <thread>

namespace pf {
namespace numa {

namespace {
bool read_text(const std::string &path, std::string *out) {
  std::ifstream f(path);
  if (!f) return false;
  std::stringstream ss;
  ss << f.rdbuf();
  *out = ss.str();
  while (!out->empty() && std::isspace((unsigned char)out->back())) out->pop_back();
  return true;
}
}  // namespace

std::vector<int> parse_cpulist(const std::string &text) {
  std::vector<int> cpus;
  std::stringstream ss(text);
  std::string part;
  auto to_int = [](const std::string &s) {
    if (s.empty() || !std::all_of(s.begin(), s.end(), [](unsigned char c) { return std::isdigit(c); }))
      throw std::invalid_argument("Invalid CPU ID: " + s);
    return std::stoi(s);
  };
  while (std::getline(ss, part, ',')) {
    if (part.empty()) continue;
    auto dash = part.find('-');
    if (dash == std::string::npos) {
      cpus.push_back(to_int(part));
    } else {
      if (part.find('-', dash + 1) != std::string::npos) throw std::invalid_argument("Invalid CPU range format: " + part);
      int lo = to_int(part.substr(0, dash)), hi = to_int(part.substr(dash + 1));
      for (int c = lo; c <= hi; ++c) cpus.push_back(c);
    }
  }
  std::sort(cpus.begin(), cpus.end());
  cpus.erase(std::unique(cpus.begin(), cpus.end()), cpus.end());
  return cpus;
}

std::vector<int> online_nodes() {
  std::string text;
  if (!read_text("/sys/devices/system/node/online", &text)) return {};
  try {
    return parse_cpulist(text);
  } catch (const std::invalid_argument &) {
    return {};
  }
}

std::vector<int> cpus_of_node(int node) {
  std::string text;
  if (node < 0 || !read_text("/sys/devices/system/node/node" + std::to_string(node) + "/cpulist", &text)) return {};
  try {
    return parse_cpulist(text);
  } catch (const std::invalid_argument &) {
    return {};
  }
}

bool pin_thread_to_node(int node) {
  std::vector<int> cpus = cpus_of_node(node);
  if (cpus.empty()) return false;
  cpu_set_t set;
  CPU_ZERO(&set);
  for (int c : cpus)
    if (c < CPU_SETSIZE) CPU_SET(c, &set);
  return sched_setaffinity(0, sizeof set, &set) == 0;
}

void run_on_node(int node, const std::function<void()> &fn) {
  std::exception_ptr failure;
  std::thread t([&] {
    if (node >= 0) pin_thread_to_node(node);
    try {
      fn();
    } catch (...) {
      failure = std::current_exception();
    }
  });
  t.join();
  if (failure) std::rethrow_exception(failure);
}

int node_of_device(int device) {
  char bdf[32] = {0};
  if (cudaDeviceGetPCIBusId(bdf, sizeof bdf, device) != cudaSuccess) {
    cudaGetLastError();
    return kUnknown;
  }
  std::string id(bdf);
  std::transform(id.begin(), id.end(), id.begin(), [](unsigned char c) { return std::tolower(c); });
  std::string text;
  int node = kUnknown;
  if (read_text("/sys/bus/pci/devices/" + id + "/numa_node", &text)) {
    try {
      node = std::stoi(text);
    } catch (...) {
      node = kUnknown;
    }
  }
  if (node < 0) {
    std::vector<int> nodes = online_nodes();
    node = nodes.size() == 1 ? nodes[0] : kUnknown;
  }
  return node;
}

std::vector<int> gpu_nodes() {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return {};
  }
  std::set<int> nodes;
  for (int d = 0; d < count; ++d) {
    int n = node_of_device(d);
    if (n >= 0) nodes.insert(n);
  }
  return std::vector<int>(nodes.begin(), nodes.end());
}

}  // namespace numa
}  // namespace pf
