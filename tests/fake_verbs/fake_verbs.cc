// Test-only implementation of the verbs subset in infiniband/verbs.h (this directory).  Devices
// come from FAKE_VERBS_DEVICES (comma separated, default "mlx5_0,rxe0"); the GID of a port is
// the owning process id; an RDMA write is a process_vm_writev into that process.  Writes of a
// queue pair happen in post order, so "payload, then flag" holds as on a reliable connection.
#include <infiniband/verbs.h>
#include <sys/uio.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

namespace {
struct Completion {
  ibv_wc wc;
  ibv_qp* qp;        // the queue pair whose send queue this completion retires
  uint64_t upto;     // ... up to and including this request (1-based count of posts)
};
struct CqImpl {
  std::mutex mu;
  std::deque<Completion> q;
};
std::atomic<uint32_t> g_qpn{100}, g_key{0x5000};
std::vector<ibv_device> g_devs;
}  // namespace

extern "C" {

ibv_device** ibv_get_device_list(int* num) {
  if (g_devs.empty()) {
    const char* e = std::getenv("FAKE_VERBS_DEVICES");
    std::stringstream ss(e ? e : "mlx5_0,rxe0");
    std::string n;
    while (std::getline(ss, n, ',')) {
      if (n.empty()) continue;
      ibv_device d;
      memset(&d, 0, sizeof(d));
      strncpy(d.name, n.c_str(), sizeof(d.name) - 1);
      g_devs.push_back(d);
    }
  }
  ibv_device** list = static_cast<ibv_device**>(calloc(g_devs.size() + 1, sizeof(ibv_device*)));
  for (size_t i = 0; i < g_devs.size(); ++i) list[i] = &g_devs[i];
  if (num) *num = static_cast<int>(g_devs.size());
  return list;
}
void ibv_free_device_list(ibv_device** list) { free(list); }
const char* ibv_get_device_name(ibv_device* dev) { return dev->name; }
ibv_context* ibv_open_device(ibv_device* dev) { return new ibv_context{dev}; }
int ibv_close_device(ibv_context* ctx) { delete ctx; return 0; }
ibv_pd* ibv_alloc_pd(ibv_context* ctx) { return new ibv_pd{ctx}; }
int ibv_dealloc_pd(ibv_pd* pd) { delete pd; return 0; }
ibv_cq* ibv_create_cq(ibv_context* ctx, int, void*, void*, int) { return new ibv_cq{ctx, new CqImpl()}; }
int ibv_destroy_cq(ibv_cq* cq) { delete static_cast<CqImpl*>(cq->impl); delete cq; return 0; }
ibv_qp* ibv_create_qp(ibv_pd*, ibv_qp_init_attr* a) {
  if (a->qp_type != IBV_QPT_RC || a->cap.max_send_wr == 0) return nullptr;
  return new ibv_qp{g_qpn.fetch_add(1), a->send_cq, IBV_QPS_RESET, 0, 0, a->cap.max_send_wr, 0, 0};
}
int ibv_destroy_qp(ibv_qp* qp) { delete qp; return 0; }
int ibv_modify_qp(ibv_qp* qp, ibv_qp_attr* a, int mask) {
  if (!(mask & IBV_QP_STATE)) return EINVAL;
  // the state machine must be walked in order, as on real hardware
  if (a->qp_state == IBV_QPS_INIT && qp->state != IBV_QPS_RESET) return EINVAL;
  if (a->qp_state == IBV_QPS_RTR && qp->state != IBV_QPS_INIT) return EINVAL;
  if (a->qp_state == IBV_QPS_RTS && qp->state != IBV_QPS_RTR) return EINVAL;
  if (a->qp_state == IBV_QPS_RTR) {
    if (!(mask & IBV_QP_AV) || !(mask & IBV_QP_DEST_QPN)) return EINVAL;
    memcpy(&qp->dest_pid, a->ah_attr.grh.dgid.raw, sizeof(int));
    qp->dest_qpn = a->dest_qp_num;
  }
  qp->state = a->qp_state;
  return 0;
}
int ibv_query_port(ibv_context*, uint8_t, ibv_port_attr* attr) { attr->lid = 0; attr->state = 4; return 0; }
int ibv_query_gid(ibv_context*, uint8_t, int, ibv_gid* gid) {
  memset(gid, 0, sizeof(*gid));
  int pid = static_cast<int>(getpid());
  memcpy(gid->raw, &pid, sizeof(pid));
  return 0;
}
ibv_mr* ibv_reg_mr(ibv_pd*, void* addr, size_t length, int) {
  uint32_t k = g_key.fetch_add(1);
  return new ibv_mr{addr, length, k, k};
}
int ibv_dereg_mr(ibv_mr* mr) { delete mr; return 0; }

int ibv_post_send(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad) {
  for (; wr; wr = wr->next) {
    if (qp->state == IBV_QPS_ERR) {
      // as on real hardware: after a failed request the queue pair is in the error state and every
      // later request is flushed with an error completion; nothing reaches the peer any more
      CqImpl* cq = static_cast<CqImpl*>(qp->send_cq->impl);
      std::lock_guard<std::mutex> lk(cq->mu);
      cq->q.push_back(Completion{ibv_wc{wr->wr_id, IBV_WC_WR_FLUSH_ERR, qp->qp_num}, qp, ++qp->posted});
      continue;
    }
    if (qp->state != IBV_QPS_RTS || wr->opcode != IBV_WR_RDMA_WRITE || wr->num_sge != 1) {
      if (bad) *bad = wr;
      return EINVAL;
    }
    // A send-queue slot is free again only when a LATER signalled completion has been polled:
    // a poster that never signals (or never polls) overruns the queue, as on real hardware.
    // FAKE_VERBS_SQ_DEPTH_CHECK=0 switches the depth model off (used when a program that is known to
    // overrun its queue has to be run to completion anyway).
    static const bool depth_check = [] {
      const char* e = std::getenv("FAKE_VERBS_SQ_DEPTH_CHECK");
      return !(e && e[0] == '0');
    }();
    if (depth_check && qp->posted - qp->retired >= qp->max_send_wr) {
      if (bad) *bad = wr;
      return ENOMEM;
    }
    const uint64_t my_index = ++qp->posted;
    iovec l{reinterpret_cast<void*>(wr->sg_list[0].addr), wr->sg_list[0].length};
    iovec r{reinterpret_cast<void*>(wr->wr.rdma.remote_addr), wr->sg_list[0].length};
    ibv_wc_status st = IBV_WC_SUCCESS;
    // Fault injection for the tests, on the host: the n-th signalled work request of the process
    // (FAKE_VERBS_FAIL_SIGNALED_AT=n) moves nothing and completes with a remote access error.
    if (wr->send_flags & IBV_SEND_SIGNALED) {
      static std::atomic<long> signaled{0};
      static const long fail_at = [] {
        const char* e = std::getenv("FAKE_VERBS_FAIL_SIGNALED_AT");
        return e ? std::atol(e) : 0L;
      }();
      if (fail_at > 0 && ++signaled == fail_at) st = IBV_WC_REM_ACCESS_ERR;
    }
    size_t done = 0;
    while (st == IBV_WC_SUCCESS && done < l.iov_len) {
      iovec l2{static_cast<char*>(l.iov_base) + done, l.iov_len - done};
      iovec r2{static_cast<char*>(r.iov_base) + done, l.iov_len - done};
      ssize_t n = process_vm_writev(qp->dest_pid, &l2, 1, &r2, 1, 0);
      if (n <= 0) { st = IBV_WC_REM_ACCESS_ERR; break; }
      done += static_cast<size_t>(n);
    }
    if (st != IBV_WC_SUCCESS) qp->state = IBV_QPS_ERR;
    if ((wr->send_flags & IBV_SEND_SIGNALED) || st != IBV_WC_SUCCESS) {
      CqImpl* cq = static_cast<CqImpl*>(qp->send_cq->impl);
      std::lock_guard<std::mutex> lk(cq->mu);
      cq->q.push_back(Completion{ibv_wc{wr->wr_id, st, qp->qp_num}, qp, my_index});
    }
  }
  return 0;
}
int ibv_poll_cq(ibv_cq* cq, int n, ibv_wc* wc) {
  CqImpl* c = static_cast<CqImpl*>(cq->impl);
  std::lock_guard<std::mutex> lk(c->mu);
  int got = 0;
  while (got < n && !c->q.empty()) {
    const Completion& done = c->q.front();
    wc[got++] = done.wc;
    if (done.upto > done.qp->retired) done.qp->retired = done.upto;
    c->q.pop_front();
  }
  return got;
}

}  // extern "C"
