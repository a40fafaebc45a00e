// NUMA helpers: which node a GPU hangs off, and running host threads on that node so that
// pinned-pool pages are first-touched next to the GPU's PCIe root.
// Behaviour follows pegaflow-common/src/numa.rs:88-258,344-497; the GPU->node map is read from
// sysfs (<root>/bus/pci/devices/<bdf>/numa_node) first and from the driver's topology tool
// only where sysfs does not know.
#pragma once

#include <functional>
#include <string>
#include <vector>

namespace pf {
namespace numa {

constexpr int kUnknown = -1;

// Where the sysfs tree is read from: "/sys" unless the environment variable PEGAFLOW_SYSFS_ROOT
// (read once) or set_sysfs_root() says otherwise.  An empty string restores the default.
void set_sysfs_root(const std::string &root);
std::string sysfs_root();

// "0-3,8-11" -> {0,1,2,3,8,9,10,11}; throws std::invalid_argument on malformed input
// (numa.rs:129-168, same messages).
std::vector<int> parse_cpulist(const std::string &text);
// Online node ids (empty when the kernel exposes no NUMA information).
std::vector<int> online_nodes();
std::vector<int> cpus_of_node(int node);
// Restrict the calling thread to the CPUs of `node` (numa.rs:178-218).  Returns "" on success,
// otherwise the reason ("Cannot pin to unknown NUMA node", "No CPUs found for NUMA node 7", ...).
std::string pin_thread_to_node_why(int node);
inline bool pin_thread_to_node(int node) { return pin_thread_to_node_why(node).empty(); }
// Run fn on a temporary thread pinned to `node` (unpinned when node is unknown) and wait.
void run_on_node(int node, const std::function<void()> &fn);
// NUMA node of the PCI device "0000:1b:00.0" from sysfs; kUnknown when absent or negative.
int node_of_pci_device(const std::string &bus_id);
// First node id in the answer of `nvidia-smi topo --get-numa-id-of-nearby-cpu`
// ("NUMA IDs of closest CPU: 1,18-33" -> 1), kUnknown when it has none (numa.rs:293-302).
int parse_closest_cpu_node(const std::string &text);
// NUMA node of a CUDA device; kUnknown if it cannot be determined.  On a single-node host
// every device is on that node.
int node_of_device(int device);
// The valid entries of `device_nodes`, sorted, each once (numa.rs:392-402).
std::vector<int> distinct_valid_nodes(const std::vector<int> &device_nodes);
// Distinct known nodes of all visible GPUs.
std::vector<int> gpu_nodes();
// Node each address's page currently lives on, kUnknown for a page that is not resident or
// when the query fails (numa.rs:441-497, move_pages(2) in query mode).
std::vector<int> query_pages(const std::vector<const void *> &addrs);

}  // namespace numa
}  // namespace pf
