#include "net/verbs_transport.h"

#include <chrono>
#include <cstdlib>
#include <cstring>

#include "bootstrap/store.h"
#include "core/config.h"
#include "core/error.h"
#include "core/log.h"
#include "net/nic_select.h"

namespace mnccl {
namespace {
// wr_id layout: bit 0 = 1 -> pointer to a Request; 0 -> internal forced signal, peer in the high bits.
inline uint64_t wrid_of(Request* r) { return reinterpret_cast<uint64_t>(r) | 1ull; }
inline uint64_t wrid_internal(int peer) { return static_cast<uint64_t>(peer) << 8; }
}  // namespace

VerbsTransport::VerbsRegion::~VerbsRegion() {
  if (mr) ibv_dereg_mr(mr);
}

VerbsTransport::VerbsTransport(int rank, int size) : rank_(rank), size_(size) {
  const Config& cfg = Config::get();
  timeout_ms_ = cfg.socket_timeout_ms;
  if (const char* e = std::getenv("MINI_NCCL_IB_GID_INDEX")) gid_index_ = atoi(e);
  if (const char* e = std::getenv("MINI_NCCL_IB_PORT")) port_ = static_cast<uint8_t>(atoi(e));
  int n = 0;
  ibv_device** list = ibv_get_device_list(&n);
  if (!list || n <= 0) {
    if (list) ibv_free_device_list(list);
    fail(Result::SystemError, "No RDMA devices found");
  }
  std::vector<std::string> names;
  for (int i = 0; i < n; ++i) names.push_back(ibv_get_device_name(list[i]));
  int pick = 0;
  try {
    pick = select_nic(names, cfg.net_device);
  } catch (...) {
    ibv_free_device_list(list);
    throw;
  }
  device_name_ = names[pick];
  log_always("Mini-NCCL", "Using RDMA Device: %s", device_name_.c_str());
  if (cfg.numa_bind) bind_to_nic_numa_node("/sys", device_name_);
  ctx_ = ibv_open_device(list[pick]);
  ibv_free_device_list(list);
  if (!ctx_) fail(Result::SystemError, "ibv_open_device failed for " + device_name_);
  pd_ = ibv_alloc_pd(ctx_);
  if (!pd_) fail(Result::SystemError, "ibv_alloc_pd failed");
  cq_ = ibv_create_cq(ctx_, kCqDepth, nullptr, nullptr, 0);
  if (!cq_) fail(Result::SystemError, "ibv_create_cq failed");
  if (posix_memalign(reinterpret_cast<void**>(&flags_), 4096, sizeof(uint32_t) * kNumFlags) != 0)
    fail(Result::SystemError, "cannot allocate the flag array");
  memset(flags_, 0, sizeof(uint32_t) * kNumFlags);
}

VerbsTransport::~VerbsTransport() {
  flags_mr_.reset();
  cache_.clear();
  for (ibv_qp* q : qps_)
    if (q) ibv_destroy_qp(q);
  if (cq_) ibv_destroy_cq(cq_);
  if (pd_) ibv_dealloc_pd(pd_);
  if (ctx_) ibv_close_device(ctx_);
  free(flags_);
}

void VerbsTransport::connect(BootstrapStore& store) {
  flags_mr_ = register_memory(flags_, sizeof(uint32_t) * kNumFlags);
  flags_remote_.addr = reinterpret_cast<uint64_t>(flags_);
  flags_remote_.rkey = flags_mr_->rkey;
  qps_.assign(size_, nullptr);
  unsignaled_.assign(size_, 0);
  posted_.assign(size_, 0);
  retired_.assign(size_, 0);
  signaled_at_.assign(size_, std::deque<uint64_t>());
  ibv_port_attr pattr;
  memset(&pattr, 0, sizeof(pattr));
  if (ibv_query_port(ctx_, port_, &pattr) != 0) fail(Result::SystemError, "ibv_query_port failed");
  ibv_gid gid;
  memset(&gid, 0, sizeof(gid));
  if (ibv_query_gid(ctx_, port_, gid_index_, &gid) != 0) fail(Result::SystemError, "ibv_query_gid failed");
  // One RC queue pair per peer (full mesh); my row of the N x N table of endpoints.
  std::vector<QpInfo> mine(size_);
  memset(mine.data(), 0, sizeof(QpInfo) * size_);
  for (int p = 0; p < size_; ++p) {
    if (p == rank_) continue;
    ibv_qp_init_attr ia;
    memset(&ia, 0, sizeof(ia));
    ia.send_cq = cq_;
    ia.recv_cq = cq_;
    ia.qp_type = IBV_QPT_RC;
    ia.cap.max_send_wr = kSendDepth;
    ia.cap.max_recv_wr = 16;
    ia.cap.max_send_sge = 1;
    ia.cap.max_recv_sge = 1;
    ia.cap.max_inline_data = 64;
    qps_[p] = ibv_create_qp(pd_, &ia);
    if (!qps_[p]) fail(Result::SystemError, "ibv_create_qp failed");
    to_init(qps_[p]);
    mine[p].qpn = qps_[p]->qp_num;
    mine[p].psn = 0;
    mine[p].lid = pattr.lid;
    memcpy(mine[p].gid, &gid, 16);
  }
  std::vector<QpInfo> all(size_t(size_) * size_);
  store.all_gather(mine.data(), all.data(), sizeof(QpInfo) * size_);
  for (int p = 0; p < size_; ++p) {
    if (p == rank_) continue;
    const QpInfo& remote = all[size_t(p) * size_ + rank_];  // the QP peer p created for me
    to_rtr(qps_[p], remote);
    to_rts(qps_[p]);
  }
  store.barrier();
}

void VerbsTransport::to_init(ibv_qp* qp) {
  ibv_qp_attr a;
  memset(&a, 0, sizeof(a));
  a.qp_state = IBV_QPS_INIT;
  a.pkey_index = 0;
  a.port_num = port_;
  a.qp_access_flags = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ;
  if (ibv_modify_qp(qp, &a, IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS) != 0)
    fail(Result::SystemError, "QP RESET->INIT failed");
}

void VerbsTransport::to_rtr(ibv_qp* qp, const QpInfo& remote) {
  ibv_qp_attr a;
  memset(&a, 0, sizeof(a));
  a.qp_state = IBV_QPS_RTR;
  a.path_mtu = IBV_MTU_1024;
  a.dest_qp_num = remote.qpn;
  a.rq_psn = remote.psn;
  a.max_dest_rd_atomic = 1;
  a.min_rnr_timer = 12;
  a.ah_attr.is_global = 1;
  a.ah_attr.dlid = remote.lid;
  a.ah_attr.sl = 0;
  a.ah_attr.src_path_bits = 0;
  a.ah_attr.port_num = port_;
  memcpy(&a.ah_attr.grh.dgid, remote.gid, 16);
  a.ah_attr.grh.sgid_index = static_cast<uint8_t>(gid_index_);
  a.ah_attr.grh.hop_limit = 1;
  if (ibv_modify_qp(qp, &a, IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN |
                                IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER) != 0)
    fail(Result::SystemError, "QP INIT->RTR failed");
}

void VerbsTransport::to_rts(ibv_qp* qp) {
  ibv_qp_attr a;
  memset(&a, 0, sizeof(a));
  a.qp_state = IBV_QPS_RTS;
  a.timeout = 14;
  a.retry_cnt = 7;
  a.rnr_retry = 7;
  a.sq_psn = 0;
  a.max_rd_atomic = 1;
  if (ibv_modify_qp(qp, &a, IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN |
                                IBV_QP_MAX_QP_RD_ATOMIC) != 0)
    fail(Result::SystemError, "QP RTR->RTS failed");
}

std::shared_ptr<MemoryRegion> VerbsTransport::register_memory(void* ptr, size_t size) {
  uint64_t before = cache_.misses();
  auto mr = cache_.get(ptr, size, [this](void* base, size_t sz) {
    auto r = std::make_shared<VerbsRegion>();
    r->mr = ibv_reg_mr(pd_, base, sz, IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ);
    if (!r->mr)
      fail(Result::SystemError, "ibv_reg_mr failed (for GPU memory this needs GPUDirect RDMA: nvidia-peermem)");
    r->ptr = base;
    r->size = sz;
    r->lkey = r->mr->lkey;
    r->rkey = r->mr->rkey;
    return std::static_pointer_cast<MemoryRegion>(r);
  });
  if (cache_.misses() != before) stats_.reg_misses++; else stats_.reg_hits++;
  return mr;
}

void VerbsTransport::invalidate(void* ptr, size_t size) { cache_.invalidate(ptr, size); }

void VerbsTransport::post(int peer, ibv_send_wr* wr, bool* signaled_out) {
  if (peer < 0 || peer >= size_ || peer == rank_ || !qps_[peer]) fail(Result::InvalidArgument, "verbs: bad peer");
  if (aborted()) fail(Result::InternalError, "transport aborted");
  std::lock_guard<std::mutex> lk(post_mu_);
  // Keep the send queue from overflowing: unsignalled work requests only retire when a later
  // signalled one completes, so signal one every kForceSignalEvery posts and wait when the
  // queue is nearly full.
  bool signaled = (wr->send_flags & IBV_SEND_SIGNALED) != 0;
  if (!signaled && ++unsignaled_[peer] >= kForceSignalEvery) {
    wr->send_flags |= IBV_SEND_SIGNALED;
    wr->wr_id = wrid_internal(peer);
    signaled = true;
  }
  if (signaled) unsignaled_[peer] = 0;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms_);
  while (posted_[peer] - retired_[peer] >= static_cast<uint64_t>(kSendDepth - 8)) {
    poll();
    if (std::chrono::steady_clock::now() > deadline) fail(Result::InternalError, "verbs: send queue stayed full");
  }
  ibv_send_wr* bad = nullptr;
  if (ibv_post_send(qps_[peer], wr, &bad) != 0) fail(Result::SystemError, "ibv_post_send failed");
  ++posted_[peer];
  if (signaled) signaled_at_[peer].push_back(posted_[peer]);
  if (signaled_out) *signaled_out = signaled;
}

Request* VerbsTransport::write(int peer, const void* local, const MemoryRegion& local_mr, RemoteBuffer remote,
                               size_t remote_offset, size_t len, bool signaled) {
  const uintptr_t l = reinterpret_cast<uintptr_t>(local), b = reinterpret_cast<uintptr_t>(local_mr.ptr);
  if (l < b || l + len > b + local_mr.size) fail(Result::InvalidArgument, "write: local range outside its registered region");
  Request* req = nullptr;
  if (signaled) {
    req = pool_.acquire(0);
    if (!req) fail(Result::InternalError, "request pool exhausted");
  }
  ibv_sge sge;
  sge.addr = l;
  sge.length = static_cast<uint32_t>(len);
  sge.lkey = local_mr.lkey;
  ibv_send_wr wr;
  memset(&wr, 0, sizeof(wr));
  wr.wr_id = req ? wrid_of(req) : 0;
  wr.sg_list = &sge;
  wr.num_sge = 1;
  wr.opcode = IBV_WR_RDMA_WRITE;
  wr.send_flags = signaled ? IBV_SEND_SIGNALED : 0;
  wr.wr.rdma.remote_addr = remote.addr + remote_offset;
  wr.wr.rdma.rkey = remote.rkey;
  try {
    post(peer, &wr, nullptr);
  } catch (...) {
    if (req) pool_.release(req);
    throw;
  }
  stats_.writes++;
  stats_.bytes_written += len;
  if (req) stats_.signaled++;
  return req;
}

Request* VerbsTransport::write_flag(int peer, RemoteBuffer remote_flags, uint32_t index, uint32_t value, bool signaled) {
  if (index >= kNumFlags) fail(Result::InvalidArgument, "flag index out of range");
  Request* req = nullptr;
  if (signaled) {
    req = pool_.acquire(0);
    if (!req) fail(Result::InternalError, "request pool exhausted");
  }
  uint32_t v = value;  // copied into the work request at post time (inline)
  ibv_sge sge;
  sge.addr = reinterpret_cast<uintptr_t>(&v);
  sge.length = 4;
  sge.lkey = 0;
  ibv_send_wr wr;
  memset(&wr, 0, sizeof(wr));
  wr.wr_id = req ? wrid_of(req) : 0;
  wr.sg_list = &sge;
  wr.num_sge = 1;
  wr.opcode = IBV_WR_RDMA_WRITE;
  wr.send_flags = IBV_SEND_INLINE | (signaled ? IBV_SEND_SIGNALED : 0);
  wr.wr.rdma.remote_addr = remote_flags.addr + 4ull * index;
  wr.wr.rdma.rkey = remote_flags.rkey;
  try {
    post(peer, &wr, nullptr);
  } catch (...) {
    if (req) pool_.release(req);
    throw;
  }
  stats_.flag_writes++;
  if (req) stats_.signaled++;
  return req;
}

int VerbsTransport::poll() {
  ibv_wc wc[16];
  int n = ibv_poll_cq(cq_, 16, wc);
  if (n < 0) fail(Result::SystemError, "ibv_poll_cq failed");
  for (int i = 0; i < n; ++i) {
    const int status = wc[i].status == IBV_WC_SUCCESS ? 0 : static_cast<int>(wc[i].status);
    if (status != 0) stats_.completion_errors++;
    // A signalled completion retires every earlier work request of its queue pair.
    for (int p = 0; p < size_; ++p)
      if (qps_[p] && qps_[p]->qp_num == wc[i].qp_num && !signaled_at_[p].empty()) {
        retired_[p] = signaled_at_[p].front();
        signaled_at_[p].pop_front();
      }
    if (wc[i].wr_id & 1ull) reinterpret_cast<Request*>(wc[i].wr_id & ~1ull)->complete(status);
    else if (status != 0) MNCCL_WARN("Mini-NCCL", "verbs: work request failed with status %d", status);
  }
  return n;
}

}  // namespace mnccl
