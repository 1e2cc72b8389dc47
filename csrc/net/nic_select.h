// NIC choice and NUMA affinity helpers for the verbs provider.  Policy kept
// from the reference (reference: src/transport/RDMATransport.h:402-458): an
// exact-name override (MINI_NCCL_NET_DEVICE; no match is an error), else
// "rxe0" (Soft-RoCE development setups), else the first device whose name
// contains "mlx5", else device 0.  NUMA: read the device's node from sysfs,
// read that node's cpulist, pin to it (reference: :460-502).  The reference
// pins the whole process; here only the calling thread is pinned and the
// sysfs root is a parameter so the logic is testable against a fake tree.
#pragma once
#include <string>
#include <vector>

namespace mnccl {

// Index into `names`.  Throws Error(SystemError) when `names` is empty or the
// override names a device that does not exist.
int select_nic(const std::vector<std::string>& names, const std::string& override_name);

// "0-3,8,10-11" -> {0,1,2,3,8,10,11}.  Malformed pieces are skipped.
std::vector<int> parse_cpu_list(const std::string& list);

// -1 when unknown / not NUMA.
int read_nic_numa_node(const std::string& sysfs_root, const std::string& device);
std::vector<int> read_numa_cpus(const std::string& sysfs_root, int node);

// Pins the calling thread.  False when the list is empty or the call fails.
bool bind_this_thread(const std::vector<int>& cpus);

// Whole sequence with logging ("[NUMA] ..."): returns the node or -1.
int bind_to_nic_numa_node(const std::string& sysfs_root, const std::string& device);

}  // namespace mnccl
