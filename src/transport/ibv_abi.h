// The part of the libibverbs binary interface that the InfiniBand backend uses, declared here because the verbs
// development headers are not a build requirement: the library is opened at run time (dlopen) and only these
// structures cross the boundary. Layouts follow the public rdma-core <infiniband/verbs.h> ABI (IBVERBS_1.x), which
// libibverbs keeps stable; records that newer versions extend at the end carry spare room here.
// The fast-path calls (post send / post receive / poll) are not exported symbols: the verbs headers define them as
// inline calls through the operations table inside the device context, and so does this file.
// Reference parity: src/include/ibvcore.h, src/include/ibvsymbols.h, src/misc/ibvwrap.cc.
#pragma once
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>

extern "C" {

union ibv_gid {
  uint8_t raw[16];
  struct { uint64_t subnet_prefix, interface_id; } global;
};

enum { IBV_MTU_256 = 1, IBV_MTU_512, IBV_MTU_1024, IBV_MTU_2048, IBV_MTU_4096 };
enum { IBV_PORT_DOWN = 1, IBV_PORT_INIT, IBV_PORT_ARMED, IBV_PORT_ACTIVE };
enum { IBV_LINK_LAYER_UNSPECIFIED = 0, IBV_LINK_LAYER_INFINIBAND = 1, IBV_LINK_LAYER_ETHERNET = 2 };
enum { IBV_ACCESS_LOCAL_WRITE = 1, IBV_ACCESS_REMOTE_WRITE = 2, IBV_ACCESS_REMOTE_READ = 4, IBV_ACCESS_RELAXED_ORDERING = 1 << 20 };
enum { IBV_QPT_RC = 2 };
enum { IBV_QPS_RESET = 0, IBV_QPS_INIT, IBV_QPS_RTR, IBV_QPS_RTS, IBV_QPS_SQD, IBV_QPS_SQE, IBV_QPS_ERR };
enum {
  IBV_QP_STATE = 1 << 0, IBV_QP_ACCESS_FLAGS = 1 << 3, IBV_QP_PKEY_INDEX = 1 << 4, IBV_QP_PORT = 1 << 5, IBV_QP_AV = 1 << 7,
  IBV_QP_PATH_MTU = 1 << 8, IBV_QP_TIMEOUT = 1 << 9, IBV_QP_RETRY_CNT = 1 << 10, IBV_QP_RNR_RETRY = 1 << 11, IBV_QP_RQ_PSN = 1 << 12,
  IBV_QP_MAX_QP_RD_ATOMIC = 1 << 13, IBV_QP_MIN_RNR_TIMER = 1 << 15, IBV_QP_SQ_PSN = 1 << 16, IBV_QP_MAX_DEST_RD_ATOMIC = 1 << 17,
  IBV_QP_DEST_QPN = 1 << 20
};
enum { IBV_WR_RDMA_WRITE = 0, IBV_WR_RDMA_WRITE_WITH_IMM, IBV_WR_SEND, IBV_WR_SEND_WITH_IMM, IBV_WR_RDMA_READ };
enum { IBV_SEND_FENCE = 1, IBV_SEND_SIGNALED = 2, IBV_SEND_SOLICITED = 4, IBV_SEND_INLINE = 8 };
enum { IBV_WC_SUCCESS = 0, IBV_WC_LOC_LEN_ERR = 1, IBV_WC_LOC_PROT_ERR = 4, IBV_WC_WR_FLUSH_ERR = 5, IBV_WC_REM_ACCESS_ERR = 10, IBV_WC_RETRY_EXC_ERR = 12,
       IBV_WC_RNR_RETRY_EXC_ERR = 13, IBV_WC_GENERAL_ERR = 21 };
enum { IBV_WC_SEND = 0, IBV_WC_RDMA_WRITE = 1, IBV_WC_RDMA_READ = 2, IBV_WC_RECV = 1 << 7, IBV_WC_RECV_RDMA_WITH_IMM = (1 << 7) + 1 };
enum { IBV_WC_WITH_IMM = 2 };

struct ibv_context;
struct ibv_cq;
struct ibv_qp;
struct ibv_wc;
struct ibv_send_wr;
struct ibv_recv_wr;

struct ibv_device {
  void* ops[2];
  int node_type, transport_type;
  char name[64], dev_name[64], dev_path[256], ibdev_path[256];
};

// Positions in the operations table of a context (one pointer each, 32 in all); only the fast-path ones are called.
enum { IBV_OP_POLL_CQ = 11, IBV_OP_POST_SEND = 25, IBV_OP_POST_RECV = 26, IBV_OP_COUNT = 32 };

struct ibv_context {
  ibv_device* device;
  void* ops[IBV_OP_COUNT];
  int cmd_fd, async_fd, num_comp_vectors;
  pthread_mutex_t mutex;
  void* abi_compat;
};

struct ibv_device_attr {
  char fw_ver[64];
  uint64_t node_guid, sys_image_guid, max_mr_size, page_size_cap;
  uint32_t vendor_id, vendor_part_id, hw_ver;
  int max_qp, max_qp_wr, device_cap_flags, max_sge, max_sge_rd, max_cq, max_cqe, max_mr, max_pd, max_qp_rd_atom, max_ee_rd_atom, max_res_rd_atom,
      max_qp_init_rd_atom, max_ee_init_rd_atom, atomic_cap, max_ee, max_rdd, max_mw, max_raw_ipv6_qp, max_raw_ethy_qp, max_mcast_grp,
      max_mcast_qp_attach, max_total_mcast_qp_attach, max_ah, max_fmr, max_map_per_fmr, max_srq, max_srq_wr, max_srq_sge;
  uint16_t max_pkeys;
  uint8_t local_ca_ack_delay, phys_port_cnt;
  uint8_t spare[64];
};

struct ibv_port_attr {
  int state, max_mtu, active_mtu, gid_tbl_len;
  uint32_t port_cap_flags, max_msg_sz, bad_pkey_cntr, qkey_viol_cntr;
  uint16_t pkey_tbl_len, lid, sm_lid;
  uint8_t lmc, max_vl_num, sm_sl, subnet_timeout, init_type_reply, active_width, active_speed, phys_state, link_layer, flags;
  uint16_t port_cap_flags2;
  uint32_t active_speed_ex;
  uint8_t spare[64];
};

struct ibv_pd { ibv_context* context; uint32_t handle; };
struct ibv_mr {
  ibv_context* context;
  ibv_pd* pd;
  void* addr;
  size_t length;
  uint32_t handle, lkey, rkey;
};

struct ibv_cq {
  ibv_context* context;
  void* channel;
  void* cq_context;
  uint32_t handle;
  int cqe;
  pthread_mutex_t mutex;
  pthread_cond_t cond;
  uint32_t comp_events_completed, async_events_completed;
};

struct ibv_qp {
  ibv_context* context;
  void* qp_context;
  ibv_pd* pd;
  ibv_cq* send_cq;
  ibv_cq* recv_cq;
  void* srq;
  uint32_t handle, qp_num;
  int state, qp_type;
  pthread_mutex_t mutex;
  pthread_cond_t cond;
  uint32_t events_completed;
};

struct ibv_qp_cap { uint32_t max_send_wr, max_recv_wr, max_send_sge, max_recv_sge, max_inline_data; };
struct ibv_qp_init_attr {
  void* qp_context;
  ibv_cq* send_cq;
  ibv_cq* recv_cq;
  void* srq;
  ibv_qp_cap cap;
  int qp_type, sq_sig_all;
  void* xrc_domain;
};

struct ibv_global_route {
  ibv_gid dgid;
  uint32_t flow_label;
  uint8_t sgid_index, hop_limit, traffic_class;
};
struct ibv_ah_attr {
  ibv_global_route grh;
  uint16_t dlid;
  uint8_t sl, src_path_bits, static_rate, is_global, port_num;
};
struct ibv_qp_attr {
  int qp_state, cur_qp_state, path_mtu, path_mig_state;
  uint32_t qkey, rq_psn, sq_psn, dest_qp_num;
  int qp_access_flags;
  ibv_qp_cap cap;
  ibv_ah_attr ah_attr, alt_ah_attr;
  uint16_t pkey_index, alt_pkey_index;
  uint8_t en_sqd_async_notify, sq_draining, max_rd_atomic, max_dest_rd_atomic, min_rnr_timer, port_num, timeout, retry_cnt, rnr_retry, alt_port_num,
      alt_timeout;
  uint8_t spare[32];
};

struct ibv_sge { uint64_t addr; uint32_t length, lkey; };
struct ibv_send_wr {
  uint64_t wr_id;
  ibv_send_wr* next;
  ibv_sge* sg_list;
  int num_sge, opcode, send_flags;
  uint32_t imm_data;   // network byte order
  union {
    struct { uint64_t remote_addr; uint32_t rkey; } rdma;
    struct { uint64_t remote_addr, compare_add, swap; uint32_t rkey; } atomic;
    struct { void* ah; uint32_t remote_qpn, remote_qkey; } ud;
  } wr;
  uint32_t xrc_remote_srq_num;
  uint8_t spare[64];   // later versions append memory-window and segmentation fields
};
struct ibv_recv_wr {
  uint64_t wr_id;
  ibv_recv_wr* next;
  ibv_sge* sg_list;
  int num_sge;
};
struct ibv_wc {
  uint64_t wr_id;
  int status, opcode;
  uint32_t vendor_err, byte_len, imm_data, qp_num, src_qp;
  int wc_flags;
  uint16_t pkey_index, slid;
  uint8_t sl, dlid_path_bits;
};

static inline int ibv_poll_cq(ibv_cq* cq, int n, ibv_wc* wc) {
  return ((int (*)(ibv_cq*, int, ibv_wc*))cq->context->ops[IBV_OP_POLL_CQ])(cq, n, wc);
}
static inline int ibv_post_send(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad) {
  return ((int (*)(ibv_qp*, ibv_send_wr*, ibv_send_wr**))qp->context->ops[IBV_OP_POST_SEND])(qp, wr, bad);
}
static inline int ibv_post_recv(ibv_qp* qp, ibv_recv_wr* wr, ibv_recv_wr** bad) {
  return ((int (*)(ibv_qp*, ibv_recv_wr*, ibv_recv_wr**))qp->context->ops[IBV_OP_POST_RECV])(qp, wr, bad);
}

}  // extern "C"

// Exported entry points, resolved with dlsym when the backend starts.
struct IbvApi {
  ibv_device** (*get_device_list)(int* n);
  void (*free_device_list)(ibv_device** list);
  const char* (*get_device_name)(ibv_device* d);
  ibv_context* (*open_device)(ibv_device* d);
  int (*close_device)(ibv_context* c);
  int (*query_device)(ibv_context* c, ibv_device_attr* a);
  int (*query_port)(ibv_context* c, uint8_t port, ibv_port_attr* a);
  int (*query_gid)(ibv_context* c, uint8_t port, int index, ibv_gid* gid);
  ibv_pd* (*alloc_pd)(ibv_context* c);
  int (*dealloc_pd)(ibv_pd* pd);
  ibv_mr* (*reg_mr)(ibv_pd* pd, void* addr, size_t len, int access);
  ibv_mr* (*reg_dmabuf_mr)(ibv_pd* pd, uint64_t offset, size_t len, uint64_t iova, int fd, int access);   // optional
  int (*dereg_mr)(ibv_mr* mr);
  ibv_cq* (*create_cq)(ibv_context* c, int cqe, void* cq_context, void* channel, int comp_vector);
  int (*destroy_cq)(ibv_cq* cq);
  ibv_qp* (*create_qp)(ibv_pd* pd, ibv_qp_init_attr* a);
  int (*modify_qp)(ibv_qp* qp, ibv_qp_attr* a, int mask);
  int (*destroy_qp)(ibv_qp* qp);
  int (*fork_init)();   // optional
};
