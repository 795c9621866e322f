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
  size_t line_bytes;                 // flagged-line region of a receive area (both halves)
  size_t bulk_bytes;                 // bulk region behind it (prompt-sized tensors, plain data)
  size_t recv_bytes;                 // whole area: signals + line_bytes + bulk_bytes
  void *recv[8];                     // recv[r]: rank r's area as addressable from this process
  bool opened[8];                    // recv[r] came from cudaIpcOpenMemHandle (to be closed)
  bool owns_recv;                    // recv[rank] was allocated by the library
  unsigned int *ctl;                 // local control words (see CommDev)
  unsigned long long wait_budget_ns;
  bool connected;
};

namespace eb {

constexpr int kCtlEpoch = 0;         // flagged-line exchanges completed on this rank
constexpr int kCtlBlocks = 1;        // arrival counter of the blocks of the kernel in flight
constexpr int kCtlBarrier = 2;       // cross-rank barriers completed on this rank (bulk exchanges)
constexpr int kCtlStatus = 4;        // [4..7]: code, where, block, detail of a wait that ran out
constexpr size_t kCtlBytes = 256;

// Layout of a receive area: [4 KB of signal words][flagged-line region: two halves][bulk region].
// Signal words: u32 [2 slots][8 sources]; source s of a cross-rank barrier stores the barrier's
// sequence number into slot / s of every rank's area and waits until all sources' words in its
// own area have reached it.
constexpr size_t kSignalBytes = 4096;

// What a kernel needs of the context (passed by value).
struct CommDev {
  int rank, world;
  unsigned char *recv[8];            // flagged-line regions (recv[rank] is local)
  unsigned char *bulk[8];            // bulk regions
  unsigned int *sig[8];              // signal words
  unsigned int *ctl;                 // local control words (never touched by peers)
  unsigned long long half_bytes;     // one half of a flagged-line region
  unsigned long long wait_budget_ns;
};

inline CommDev comm_dev(const eb_comm *c) {
  CommDev d{};
  d.rank = c->rank;
  d.world = c->world;
  for (int r = 0; r < c->world; ++r) {
    unsigned char *base = reinterpret_cast<unsigned char *>(c->recv[r]);
    d.sig[r] = reinterpret_cast<unsigned int *>(base);
    d.recv[r] = base + kSignalBytes;
    d.bulk[r] = base + kSignalBytes + c->line_bytes;
  }
  d.ctl = c->ctl;
  d.half_bytes = c->line_bytes / 2;
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

// The same load without the test.  Polling code issues ALL the loads of a group first and looks
// at the sequence numbers afterwards: a test between two loads would make every load wait for
// the one before it (a full trip to L2 each).
struct LlLine {
  unsigned long long a, b;
  __device__ __forceinline__ bool valid(uint32_t seq) const { return (uint32_t)(a >> 32) == seq && (uint32_t)(b >> 32) == seq; }
  __device__ __forceinline__ uint32_t d0() const { return (uint32_t)a; }
  __device__ __forceinline__ uint32_t d1() const { return (uint32_t)b; }
};
__device__ __forceinline__ LlLine ll_fetch(const void *line) {
  LlLine l;
  asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(l.a), "=l"(l.b) : "l"(line) : "memory");
  return l;
}

__device__ __forceinline__ unsigned long long comm_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Sum over the ranks of a prompt-sized [M, N] 16-bit tensor, in two kernels over the bulk region:
// the row-parallel GEMM stores the tiles of its partial product straight into the staging area
// of the rank that owns those rows (rows are dealt out in `world` contiguous blocks of whole
// 128-row tiles; staging layout [source][row within the block][N]), and a second kernel, after a
// barrier over the ranks, adds the `world` partials of its own rows (+ bias + residual), stores
// the finished rows into the gather area [M][N] of every rank and ends with another barrier.
inline long long comm_rows_per_rank(long long M, int world) {
  const long long tiles = (M + 127) / 128;
  return ((tiles + world - 1) / world) * 128;
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
