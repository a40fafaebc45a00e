// NUMA helpers: which node a GPU hangs off, and running host threads on that node so that
// pinned-pool pages are first-touched next to the GPU's PCIe root.
// Behaviour follows pegaflow-common/src/numa.rs:88-258,344-411; the GPU->node map is read from
// sysfs (/sys/bus/pci/devices/<bdf>/numa_node) instead of an external tool.
#pragma once

#include <functional>
#include <string>
#include <vector>

namespace pf {
namespace numa {

constexpr int kUnknown = -1;

// "0-3,8-11" -> {0,1,2,3,8,9,10,11}; throws std::invalid_argument on malformed input.
std::vector<int> parse_cpulist(const std::string &text);
// Online node ids (empty when the kernel exposes no NUMA information).
std::vector<int> online_nodes();
std::vector<int> cpus_of_node(int node);
// Restrict the calling thread to the CPUs of `node`; false when unknown or refused.
bool pin_thread_to_node(int node);
// Run fn on a temporary thread pinned to `node` (unpinned when node is unknown) and wait.
void run_on_node(int node, const std::function<void()> &fn);
// NUMA node of a CUDA device; kUnknown if it cannot be determined.  On a single-node host
// every device is on node 0.
int node_of_device(int device);
// Distinct known nodes of all visible GPUs.
std::vector<int> gpu_nodes();

}  // namespace numa
}  // namespace pf
