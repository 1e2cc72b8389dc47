#include "net/nic_select.h"

#include <cstdlib>
#include <fstream>
#include <pthread.h>
#include <sched.h>
#include <sstream>

#include "core/error.h"
#include "core/log.h"

namespace mnccl {

int select_nic(const std::vector<std::string>& names, const std::string& override_name) {
  if (names.empty()) fail(Result::SystemError, "No RDMA devices found");
  if (!override_name.empty()) {
    for (size_t i = 0; i < names.size(); ++i)
      if (names[i] == override_name) return static_cast<int>(i);
    fail(Result::SystemError, "MINI_NCCL_NET_DEVICE='" + override_name + "' matches no RDMA device");
  }
  for (size_t i = 0; i < names.size(); ++i)
    if (names[i] == "rxe0") return static_cast<int>(i);
  for (size_t i = 0; i < names.size(); ++i)
    if (names[i].find("mlx5") != std::string::npos) return static_cast<int>(i);
  return 0;
}

std::vector<int> parse_cpu_list(const std::string& list) {
  std::vector<int> cpus;
  std::stringstream ss(list);
  std::string piece;
  while (std::getline(ss, piece, ',')) {
    while (!piece.empty() && (piece.back() == '\n' || piece.back() == ' ')) piece.pop_back();
    if (piece.empty()) continue;
    size_t dash = piece.find('-');
    char* end = nullptr;
    if (dash == std::string::npos) {
      long v = std::strtol(piece.c_str(), &end, 10);
      if (end != piece.c_str() && v >= 0) cpus.push_back(static_cast<int>(v));
    } else {
      long a = std::strtol(piece.substr(0, dash).c_str(), &end, 10);
      long b = std::strtol(piece.substr(dash + 1).c_str(), &end, 10);
      if (a >= 0 && b >= a && b - a < 65536)
        for (long c = a; c <= b; ++c) cpus.push_back(static_cast<int>(c));
    }
  }
  return cpus;
}

int read_nic_numa_node(const std::string& sysfs_root, const std::string& device) {
  std::ifstream f(sysfs_root + "/class/infiniband/" + device + "/device/numa_node");
  int node = -1;
  if (!(f >> node)) return -1;
  return node;
}

std::vector<int> read_numa_cpus(const std::string& sysfs_root, int node) {
  if (node < 0) return {};
  std::ifstream f(sysfs_root + "/devices/system/node/node" + std::to_string(node) + "/cpulist");
  std::string line;
  if (!std::getline(f, line)) return {};
  return parse_cpu_list(line);
}

bool bind_this_thread(const std::vector<int>& cpus) {
  if (cpus.empty()) return false;
  cpu_set_t set;
  CPU_ZERO(&set);
  for (int c : cpus)
    if (c >= 0 && c < CPU_SETSIZE) CPU_SET(c, &set);
  return pthread_setaffinity_np(pthread_self(), sizeof(set), &set) == 0;
}

int bind_to_nic_numa_node(const std::string& sysfs_root, const std::string& device) {
  int node = read_nic_numa_node(sysfs_root, device);
  if (node < 0) {
    MNCCL_INFO("NUMA", "Device %s reports no NUMA node; affinity unchanged", device.c_str());
    return -1;
  }
  std::vector<int> cpus = read_numa_cpus(sysfs_root, node);
  if (cpus.empty()) {
    MNCCL_INFO("NUMA", "Node %d has no readable cpulist; affinity unchanged", node);
    return -1;
  }
  if (bind_this_thread(cpus)) {
    MNCCL_INFO("NUMA", "Device %s is on node %d; pinned the calling thread to %zu CPUs", device.c_str(), node, cpus.size());
    return node;
  }
  MNCCL_WARN("NUMA", "Could not set affinity for node %d", node);
  return -1;
}

}  // namespace mnccl
