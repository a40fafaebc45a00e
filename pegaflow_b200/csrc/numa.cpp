#include "numa.h"

#include <cuda_runtime.h>
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <cstring>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <mutex>
#include <set>
#include <sstream>
#include <stdexcept>
#include <thread>

namespace pf {
namespace numa {

namespace {
std::mutex g_root_mu;
std::string g_root;
bool g_root_set = false;

bool read_text(const std::string &path, std::string *out) {
  std::ifstream f(path);
  if (!f) return false;
  std::stringstream ss;
  ss << f.rdbuf();
  *out = ss.str();
  while (!out->empty() && std::isspace((unsigned char)out->back())) out->pop_back();
  return true;
}

std::string lower(std::string s) {
  std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return std::tolower(c); });
  return s;
}
}  // namespace

void set_sysfs_root(const std::string &root) {
  std::lock_guard<std::mutex> g(g_root_mu);
  g_root = root;
  g_root_set = true;
}

std::string sysfs_root() {
  std::lock_guard<std::mutex> g(g_root_mu);
  if (!g_root_set) {
    const char *env = getenv("PEGAFLOW_SYSFS_ROOT");
    g_root = env ? env : "";
    g_root_set = true;
  }
  return g_root.empty() ? "/sys" : g_root;
}

std::vector<int> parse_cpulist(const std::string &text) {
  std::vector<int> cpus;
  std::stringstream ss(text);
  std::string part;
  auto to_int = [](const std::string &s) {
    if (s.empty() || s.size() > 9 || !std::all_of(s.begin(), s.end(), [](unsigned char c) { return std::isdigit(c); }))
      throw std::invalid_argument("Invalid CPU ID: " + s);
    return std::stoi(s);
  };
  while (std::getline(ss, part, ',')) {
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
  if (!read_text(sysfs_root() + "/devices/system/node/online", &text)) return {};
  try {
    return parse_cpulist(text);
  } catch (const std::invalid_argument &) {
    return {};
  }
}

std::vector<int> cpus_of_node(int node) {
  std::string text;
  if (node < 0 || !read_text(sysfs_root() + "/devices/system/node/node" + std::to_string(node) + "/cpulist", &text))
    return {};
  try {
    return parse_cpulist(text);
  } catch (const std::invalid_argument &) {
    return {};
  }
}

std::string pin_thread_to_node_why(int node) {
  if (node < 0) return "Cannot pin to unknown NUMA node";
  std::string text;
  if (!read_text(sysfs_root() + "/devices/system/node/node" + std::to_string(node) + "/cpulist", &text))
    return "No CPUs found for NUMA node " + std::to_string(node);
  std::vector<int> cpus;
  try {
    cpus = parse_cpulist(text);
  } catch (const std::invalid_argument &e) {
    return std::string("Failed to get NUMA topology: ") + e.what();
  }
  if (cpus.empty()) return "CPU list is empty for NUMA node " + std::to_string(node);
  cpu_set_t set;
  CPU_ZERO(&set);
  for (int c : cpus)
    if (c < CPU_SETSIZE) CPU_SET(c, &set);
  if (sched_setaffinity(0, sizeof set, &set) != 0) return std::string("sched_setaffinity failed: ") + strerror(errno);
  return "";
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

int node_of_pci_device(const std::string &bus_id) {
  std::string text;
  if (!read_text(sysfs_root() + "/bus/pci/devices/" + lower(bus_id) + "/numa_node", &text)) return kUnknown;
  try {
    const int node = std::stoi(text);
    return node < 0 ? kUnknown : node;
  } catch (...) {
    return kUnknown;
  }
}

int parse_closest_cpu_node(const std::string &text) {
  const std::string line = text.substr(0, text.find('\n'));
  const auto colon = line.find(':');
  if (colon == std::string::npos) return kUnknown;
  std::string ids = line.substr(colon + 1);
  const auto next_colon = ids.find(':');
  if (next_colon != std::string::npos) ids = ids.substr(0, next_colon);
  std::string first = ids.substr(0, ids.find(','));
  first.erase(0, first.find_first_not_of(" \t\r"));
  first.erase(first.find_last_not_of(" \t\r") + 1);
  if (first.empty() || first.size() > 9 || !std::all_of(first.begin(), first.end(), [](unsigned char c) { return std::isdigit(c); }))
    return kUnknown;
  return std::stoi(first);
}

namespace {
// The reference's source for the map (numa.rs:266-291); used here only when sysfs has no answer
// on a host with several nodes.
int ask_driver_tool(int device) {
  char cmd[128];
  snprintf(cmd, sizeof cmd, "nvidia-smi topo --get-numa-id-of-nearby-cpu -i %d 2>/dev/null", device);
  FILE *p = popen(cmd, "r");
  if (!p) return kUnknown;
  std::string out;
  char buf[256];
  while (fgets(buf, sizeof buf, p)) out += buf;
  if (pclose(p) != 0) return kUnknown;
  return parse_closest_cpu_node(out);
}
}  // namespace

int node_of_device(int device) {
  char bdf[32] = {0};
  if (cudaDeviceGetPCIBusId(bdf, sizeof bdf, device) != cudaSuccess) {
    cudaGetLastError();
    return kUnknown;
  }
  int node = node_of_pci_device(bdf);
  if (node < 0) {
    std::vector<int> nodes = online_nodes();
    if (nodes.size() == 1) node = nodes[0];
    else if (nodes.size() > 1) node = ask_driver_tool(device);
  }
  return node;
}

std::vector<int> distinct_valid_nodes(const std::vector<int> &device_nodes) {
  std::set<int> nodes;
  for (int n : device_nodes)
    if (n >= 0) nodes.insert(n);
  return std::vector<int>(nodes.begin(), nodes.end());
}

std::vector<int> gpu_nodes() {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return {};
  }
  std::vector<int> all;
  for (int d = 0; d < count; ++d) all.push_back(node_of_device(d));
  return distinct_valid_nodes(all);
}

std::vector<int> query_pages(const std::vector<const void *> &addrs) {
  if (addrs.empty()) return {};
  const uintptr_t page = (uintptr_t)std::max<long>(1, sysconf(_SC_PAGESIZE));
  std::vector<void *> pages(addrs.size());
  for (size_t i = 0; i < addrs.size(); ++i) pages[i] = (void *)((uintptr_t)addrs[i] & ~(page - 1));
  std::vector<int> status(addrs.size(), kUnknown);
  const long rc = syscall(SYS_move_pages, 0, (unsigned long)addrs.size(), pages.data(), (const int *)nullptr, status.data(), 0);
  if (rc != 0) return std::vector<int>(addrs.size(), kUnknown);
  for (int &s : status)
    if (s < 0) s = kUnknown;
  return status;
}

}  // namespace numa
}  // namespace pf
