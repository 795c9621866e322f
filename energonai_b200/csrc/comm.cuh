// Tensor-parallel exchange context shared by the kernels that move partial sums between GPUs.
//
// Every rank owns a receive area in device memory that its peers can address over NVLink (a
// CUDA IPC mapping, or pointers the caller mapped itself).  Data travels in "flagged lines":
// 16 bytes = two 8-byte words, each holding 4 bytes of payload and the 4-byte sequence number of
// the exchange.  An aligned 8-byte store is delivered as a unit, so a reader that sees the
// expected sequence number in a word also sees its payload: no fence, no separate flag, no
// round trip before the flag may be written.  The price is twice the bytes, which is nothing at
// generation-step sizes (a [16, 5120] fp16 partial sum is 164 KB).
//
// The area is used as two halves by alternate exchanges: a rank can run at most one exchange
// ahead of the slowest rank (it cannot finish exchange e+1 before everybody has contributed to
// it, and a rank contributes to e+1 only after it consumed e), so when half (e & 1) is written
// again for e+2 nobody still reads e.  The sequence number lives in device memory (`epoch`,
// local to each rank and advanced by the kernels themselves), so a captured launch can be
// replayed; all ranks issue the same exchanges in the same order, hence the numbers agree.
#pragma once

#include "common.cuh"

struct eb_comm {
  int rank, world, device;
  size_t recv_bytes;                 // one rank's receive area (both halves)
  void *recv[8];                     // recv[r]: rank r's area as addressable from this process
  bool opened[8];                    // recv[r] came from cudaIpcOpenMemHandle (to be closed)
  bool owns_recv;                    // recv[rank] was allocated by the library
  unsigned int *ctl;                 // local control words (see CommDev)
  unsigned long long wait_budget_ns;
  bool connected;
};

namespace eb {

constexpr int kCtlEpoch = 0;         // exchanges completed on this rank
constexpr int kCtlBlocks = 1;        // arrival counter of eb_allreduce's blocks
constexpr int kCtlStatus = 4;        // [4..7]: code, where, block, detail of a wait that ran out
constexpr size_t kCtlBytes = 256;

// What a kernel needs of the context (passed by value).
struct CommDev {
  int rank, world;
  unsigned char *recv[8];
  unsigned int *ctl;
  unsigned long long half_bytes;
  unsigned long long wait_budget_ns;
};

inline CommDev comm_dev(const eb_comm *c) {
  CommDev d{};
  d.rank = c->rank;
  d.world = c->world;
  for (int r = 0; r < c->world; ++r) d.recv[r] = reinterpret_cast<unsigned char *>(c->recv[r]);
  d.ctl = c->ctl;
  d.half_bytes = c->recv_bytes / 2;
  d.wait_budget_ns = c->wait_budget_ns;
  return d;
}

// Bytes one exchange of a [rows, cols] 16-bit matrix occupies in one half of a receive area.
inline size_t comm_exchange_bytes(int world, long long rows, long long cols) {
  return (size_t)world * (size_t)rows * (size_t)cols * 4;
}

// ---- flagged lines ------------------------------------------------------------------------
__device__ __forceinline__ void ll_store(void *line, uint32_t d0, uint32_t d1, uint32_t seq) {
  const unsigned long long a = ((unsigned long long)seq << 32) | d0, b = ((unsigned long long)seq << 32) | d1;
  asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(line), "l"(a), "l"(b) : "memory");
}
// True when both words of the line carry `seq`; d0 / d1 are then the payload.
__device__ __forceinline__ bool ll_load(const void *line, uint32_t seq, uint32_t &d0, uint32_t &d1) {
  unsigned long long a, b;
  asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(line) : "memory");
  d0 = (uint32_t)a;
  d1 = (uint32_t)b;
  return (uint32_t)(a >> 32) == seq && (uint32_t)(b >> 32) == seq;
}

__device__ __forceinline__ unsigned long long comm_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Records a wait that ran out in the context's control words (first failure wins).
__device__ __forceinline__ void comm_record_timeout(const CommDev &c, int where, int detail) {
  int *st = reinterpret_cast<int *>(c.ctl + kCtlStatus);
  if (atomicCAS(st, 0, EB_ETIMEDOUT) == 0) {
    st[1] = where;
    st[2] = (int)blockIdx.x;
    st[3] = detail;
  }
}

}  // namespace eb
