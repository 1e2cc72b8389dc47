/* A stand-in for <infiniband/verbs.h> used ONLY by the test-suite, so that the verbs provider
 * (csrc/net/verbs_transport.cc) can be compiled and exercised on machines without libibverbs or
 * an RDMA device.  It declares the small subset of the verbs API the provider uses; the
 * implementation (fake_verbs.cc) performs an RDMA write as a process_vm_writev into the peer
 * process, in order, which is all the ring protocol relies on.  Not part of the library. */
#ifndef MNCCL_FAKE_INFINIBAND_VERBS_H
#define MNCCL_FAKE_INFINIBAND_VERBS_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

struct ibv_device { char name[64]; };
struct ibv_context { struct ibv_device* device; };
struct ibv_pd { struct ibv_context* context; };
struct ibv_cq { struct ibv_context* context; void* impl; };
struct ibv_mr { void* addr; size_t length; uint32_t lkey; uint32_t rkey; };
struct ibv_qp {
  uint32_t qp_num; struct ibv_cq* send_cq; int state; int dest_pid; uint32_t dest_qpn;
  /* send-queue model of the stand-in: depth, requests posted, requests retired by a polled completion */
  uint32_t max_send_wr; uint64_t posted; uint64_t retired;
};
union ibv_gid { uint8_t raw[16]; };
struct ibv_port_attr { uint16_t lid; int state; };

enum ibv_qp_type { IBV_QPT_RC = 2 };
enum ibv_qp_state { IBV_QPS_RESET, IBV_QPS_INIT, IBV_QPS_RTR, IBV_QPS_RTS, IBV_QPS_ERR = 6 };
enum ibv_mtu { IBV_MTU_256 = 1, IBV_MTU_512, IBV_MTU_1024, IBV_MTU_2048, IBV_MTU_4096 };
enum ibv_access_flags { IBV_ACCESS_LOCAL_WRITE = 1, IBV_ACCESS_REMOTE_WRITE = 2, IBV_ACCESS_REMOTE_READ = 4 };
enum ibv_send_flags { IBV_SEND_FENCE = 1, IBV_SEND_SIGNALED = 2, IBV_SEND_SOLICITED = 4, IBV_SEND_INLINE = 8 };
enum ibv_wr_opcode { IBV_WR_RDMA_WRITE = 0, IBV_WR_SEND = 2 };
enum ibv_wc_status { IBV_WC_SUCCESS = 0, IBV_WC_WR_FLUSH_ERR = 5, IBV_WC_REM_ACCESS_ERR = 10, IBV_WC_GENERAL_ERR = 21 };
enum ibv_qp_attr_mask {
  IBV_QP_STATE = 1 << 0, IBV_QP_ACCESS_FLAGS = 1 << 3, IBV_QP_PKEY_INDEX = 1 << 4, IBV_QP_PORT = 1 << 5,
  IBV_QP_AV = 1 << 7, IBV_QP_PATH_MTU = 1 << 8, IBV_QP_TIMEOUT = 1 << 9, IBV_QP_RETRY_CNT = 1 << 10,
  IBV_QP_RNR_RETRY = 1 << 11, IBV_QP_RQ_PSN = 1 << 12, IBV_QP_MAX_QP_RD_ATOMIC = 1 << 13,
  IBV_QP_MIN_RNR_TIMER = 1 << 15, IBV_QP_SQ_PSN = 1 << 16, IBV_QP_MAX_DEST_RD_ATOMIC = 1 << 17,
  IBV_QP_DEST_QPN = 1 << 20
};

struct ibv_qp_cap { uint32_t max_send_wr, max_recv_wr, max_send_sge, max_recv_sge, max_inline_data; };
struct ibv_qp_init_attr {
  void* qp_context; struct ibv_cq* send_cq; struct ibv_cq* recv_cq; void* srq; struct ibv_qp_cap cap;
  enum ibv_qp_type qp_type; int sq_sig_all;
};
struct ibv_global_route { union ibv_gid dgid; uint32_t flow_label; uint8_t sgid_index, hop_limit, traffic_class; };
struct ibv_ah_attr { struct ibv_global_route grh; uint16_t dlid; uint8_t sl, src_path_bits, static_rate, is_global, port_num; };
struct ibv_qp_attr {
  enum ibv_qp_state qp_state; enum ibv_mtu path_mtu; uint32_t rq_psn, sq_psn, dest_qp_num; int qp_access_flags;
  struct ibv_ah_attr ah_attr; uint16_t pkey_index; uint8_t max_rd_atomic, max_dest_rd_atomic, min_rnr_timer, port_num,
      timeout, retry_cnt, rnr_retry;
};
struct ibv_sge { uint64_t addr; uint32_t length; uint32_t lkey; };
struct ibv_send_wr {
  uint64_t wr_id; struct ibv_send_wr* next; struct ibv_sge* sg_list; int num_sge; enum ibv_wr_opcode opcode;
  unsigned int send_flags;
  union { struct { uint64_t remote_addr; uint32_t rkey; } rdma; } wr;
};
struct ibv_wc { uint64_t wr_id; enum ibv_wc_status status; uint32_t qp_num; };

struct ibv_device** ibv_get_device_list(int* num);
void ibv_free_device_list(struct ibv_device** list);
const char* ibv_get_device_name(struct ibv_device* dev);
struct ibv_context* ibv_open_device(struct ibv_device* dev);
int ibv_close_device(struct ibv_context* ctx);
struct ibv_pd* ibv_alloc_pd(struct ibv_context* ctx);
int ibv_dealloc_pd(struct ibv_pd* pd);
struct ibv_cq* ibv_create_cq(struct ibv_context* ctx, int cqe, void* cq_context, void* channel, int comp_vector);
int ibv_destroy_cq(struct ibv_cq* cq);
struct ibv_qp* ibv_create_qp(struct ibv_pd* pd, struct ibv_qp_init_attr* attr);
int ibv_destroy_qp(struct ibv_qp* qp);
int ibv_modify_qp(struct ibv_qp* qp, struct ibv_qp_attr* attr, int mask);
int ibv_query_port(struct ibv_context* ctx, uint8_t port, struct ibv_port_attr* attr);
int ibv_query_gid(struct ibv_context* ctx, uint8_t port, int index, union ibv_gid* gid);
struct ibv_mr* ibv_reg_mr(struct ibv_pd* pd, void* addr, size_t length, int access);
int ibv_dereg_mr(struct ibv_mr* mr);
int ibv_post_send(struct ibv_qp* qp, struct ibv_send_wr* wr, struct ibv_send_wr** bad);
int ibv_poll_cq(struct ibv_cq* cq, int n, struct ibv_wc* wc);

#ifdef __cplusplus
}
#endif
#endif
