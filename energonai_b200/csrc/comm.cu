// Host side of the tensor-parallel exchange context (eb_comm_*) and the stand-alone one-shot
// all-reduce (eb_allreduce).  The protocol is described in comm.cuh.
//
// The reference sets its tensor-parallel groups up through colossalai.launch
// (energonai/worker.py:27-28) and reduces with NCCL inside colossalai's Linear1D_Row; its own
// NCCL-id helper (energonai/kernel/cuda_native/csrc/get_ncclid.cpp:104-127) is not built.
#include <cstring>
#include <new>

#include "comm.cuh"

namespace eb {
namespace {

constexpr int kArThreads = 256;

template <typename T> struct Payload;          // 8 bytes of T <-> fp32
template <> struct Payload<float> {
  static constexpr int N = 2;
  __device__ static void add(float *acc, uint32_t d0, uint32_t d1) {
    acc[0] += __uint_as_float(d0);
    acc[1] += __uint_as_float(d1);
  }
  __device__ static uint2 pack(const float *acc) { return make_uint2(__float_as_uint(acc[0]), __float_as_uint(acc[1])); }
};
template <> struct Payload<__half> {
  static constexpr int N = 4;
  __device__ static void add(float *acc, uint32_t d0, uint32_t d1) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&d0));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&d1));
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  }
  __device__ static uint2 pack(const float *acc) {
    const __half2 a = __floats2half2_rn(acc[0], acc[1]), b = __floats2half2_rn(acc[2], acc[3]);
    return make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
  }
};
template <> struct Payload<__nv_bfloat16> {
  static constexpr int N = 4;
  __device__ static void add(float *acc, uint32_t d0, uint32_t d1) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&d0));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&d1));
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  }
  __device__ static uint2 pack(const float *acc) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(acc[0], acc[1]), b = __floats2bfloat162_rn(acc[2], acc[3]);
    return make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
  }
};

// In-place SUM of `lines` 8-byte groups of `buf` over the ranks.  Every thread first sends all
// its groups to every rank (itself included), then collects the same groups of every source
// from the local receive area and adds them in rank order (so all ranks hold bit-identical
// sums).  Blocks depend on remote ranks only, never on one another.
template <typename T>
__global__ void __launch_bounds__(kArThreads) allreduce_kernel(const CommDev c, T *buf, unsigned long long lines) {
  griddep_launch();
  griddep_wait();
  const uint32_t seq = *reinterpret_cast<volatile unsigned int *>(c.ctl + kCtlEpoch) + 1u;
  const unsigned long long half = (seq & 1u) * c.half_bytes;
  const unsigned long long stride = (unsigned long long)gridDim.x * kArThreads;
  const unsigned long long first = (unsigned long long)blockIdx.x * kArThreads + threadIdx.x;
  uint2 *data = reinterpret_cast<uint2 *>(buf);
  for (unsigned long long i = first; i < lines; i += stride) {
    const uint2 mine = data[i];
    const unsigned long long off = half + ((unsigned long long)c.rank * lines + i) * 16ull;
    for (int r = 0; r < c.world; ++r) ll_store(c.recv[r] + off, mine.x, mine.y, seq);
  }
  bool failed = false;
  for (unsigned long long i = first; i < lines; i += stride) {
    // all sources' lines are requested together and looked at afterwards
    LlLine got[8];
    const unsigned char *base = c.recv[c.rank] + half + i * 16ull;
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
      bool all = true;
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s < c.world) got[s] = ll_fetch(base + (unsigned long long)s * lines * 16ull);
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s < c.world) all = all && got[s].valid(seq);
      if (all || failed) break;
      if ((it & 63u) == 63u) {
        if (t0 == 0) t0 = comm_timer();
        else if (comm_timer() - t0 > c.wait_budget_ns) {
          int missing = 0;
#pragma unroll
          for (int s = 7; s >= 0; --s)
            if (s < c.world && !got[s].valid(seq)) missing = s;
          comm_record_timeout(c, 20, missing);
          failed = true;              // give up on this and every later line: the call has failed
        }
      }
    }
    float acc[Payload<T>::N];
#pragma unroll
    for (int e = 0; e < Payload<T>::N; ++e) acc[e] = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s)
      if (s < c.world) Payload<T>::add(acc, got[s].d0(), got[s].d1());
    data[i] = Payload<T>::pack(acc);
  }
  // the last block to finish advances the sequence number for the next exchange
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int arrived = atomicAdd(c.ctl + kCtlBlocks, 1u);
    if (arrived == gridDim.x - 1) {
      c.ctl[kCtlBlocks] = 0u;
      c.ctl[kCtlEpoch] = seq;
      __threadfence();
    }
  }
}

int check_comm(const eb_comm *c, const char *what) {
  if (!c) return fail(EB_EINVAL, "%s: null context", what);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != c->device) {
    cudaGetLastError();
    return fail(EB_EINVAL, "%s: the context belongs to device %d, which is not current", what, c->device);
  }
  return EB_OK;
}

}  // namespace
}  // namespace eb

using namespace eb;

extern "C" size_t eb_comm_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" size_t eb_comm_exchange_bytes(int world, int rows, int cols) {
  if (world <= 0 || rows <= 0 || cols <= 0) return 0;
  return comm_exchange_bytes(world, rows, cols);
}

extern "C" size_t eb_comm_area_bytes(size_t line_bytes, size_t bulk_bytes) { return kSignalBytes + line_bytes + bulk_bytes; }

extern "C" int eb_comm_create(int rank, int world, size_t line_bytes, size_t bulk_bytes, void *recv_local, eb_comm **out) {
  EB_REQUIRE(out, "comm_create: null result pointer");
  *out = nullptr;
  EB_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world, "comm_create: bad rank %d / world %d", rank, world);
  EB_REQUIRE(line_bytes >= 4096 && line_bytes % 512 == 0, "comm_create: the flagged-line region must be a multiple of 512 bytes (>= 4096)");
  EB_REQUIRE(bulk_bytes % 512 == 0, "comm_create: the bulk region must be a multiple of 512 bytes");
  EB_REQUIRE(!recv_local || (reinterpret_cast<uintptr_t>(recv_local) & 255u) == 0, "comm_create: recv_local must be 256-byte aligned");
  const size_t recv_bytes = kSignalBytes + line_bytes + bulk_bytes;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return fail(EB_ECUDA, "comm_create: no current device");
  }
  eb_comm *c = new (std::nothrow) eb_comm();
  if (!c) return fail(EB_ECUDA, "comm_create: out of host memory");
  c->rank = rank; c->world = world; c->device = dev; c->recv_bytes = recv_bytes;
  c->line_bytes = line_bytes; c->bulk_bytes = bulk_bytes;
  c->wait_budget_ns = 5ull * 1000ull * 1000ull * 1000ull;     // 5 s: ranks may be seconds apart while one of them loads code or captures a graph
  cudaError_t e = cudaSuccess;
  if (recv_local) {
    c->recv[rank] = recv_local;
  } else {
    e = cudaMalloc(&c->recv[rank], recv_bytes);
    c->owns_recv = e == cudaSuccess;
  }
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&c->ctl), kCtlBytes);
  // Sequence numbers start at 1, so a zeroed area holds no valid line.
  if (e == cudaSuccess) e = cudaMemset(c->recv[rank], 0, recv_bytes);
  if (e == cudaSuccess) e = cudaMemset(c->ctl, 0, kCtlBytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (c->owns_recv) cudaFree(c->recv[rank]);
    if (c->ctl) cudaFree(c->ctl);
    delete c;
    return fail(EB_ECUDA, "comm_create: %s", cudaGetErrorString(e));
  }
  c->connected = world == 1;
  *out = c;
  return EB_OK;
}

extern "C" int eb_comm_export_handle(const eb_comm *c, void *blob, size_t blob_bytes) {
  int rc = check_comm(c, "comm_export_handle");
  if (rc) return rc;
  EB_REQUIRE(blob && blob_bytes >= sizeof(cudaIpcMemHandle_t), "comm_export_handle: the blob must hold %zu bytes",
             sizeof(cudaIpcMemHandle_t));
  EB_REQUIRE(c->owns_recv, "comm_export_handle: the receive area was supplied by the caller, who also maps it (eb_comm_connect_pointers)");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, c->recv[c->rank]);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(EB_ECUDA, "comm_export_handle: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  memcpy(blob, &h, sizeof(h));
  return EB_OK;
}

extern "C" int eb_comm_connect(eb_comm *c, const void *blobs, size_t blobs_bytes) {
  int rc = check_comm(c, "comm_connect");
  if (rc) return rc;
  EB_REQUIRE(!c->connected || c->world == 1, "comm_connect: already connected");
  EB_REQUIRE(blobs && blobs_bytes == (size_t)c->world * sizeof(cudaIpcMemHandle_t),
             "comm_connect: expected %d handles of %zu bytes in rank order (got %zu bytes)", c->world,
             sizeof(cudaIpcMemHandle_t), blobs_bytes);
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, reinterpret_cast<const char *>(blobs) + (size_t)r * sizeof(h), sizeof(h));
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      for (int q = 0; q < r; ++q)
        if (c->opened[q]) { cudaIpcCloseMemHandle(c->recv[q]); c->opened[q] = false; c->recv[q] = nullptr; }
      return fail(EB_ECUDA, "comm_connect: cannot map the receive area of rank %d: %s", r, cudaGetErrorString(e));
    }
    c->recv[r] = p;
    c->opened[r] = true;
  }
  c->connected = true;
  return EB_OK;
}

extern "C" int eb_comm_connect_pointers(eb_comm *c, void *const *peer_recv) {
  int rc = check_comm(c, "comm_connect_pointers");
  if (rc) return rc;
  EB_REQUIRE(peer_recv, "comm_connect_pointers: null pointer table");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    EB_REQUIRE(peer_recv[r] && (reinterpret_cast<uintptr_t>(peer_recv[r]) & 255u) == 0,
               "comm_connect_pointers: rank %d's area is null or not 256-byte aligned", r);
  }
  for (int r = 0; r < c->world; ++r)
    if (r != c->rank) { c->recv[r] = peer_recv[r]; c->opened[r] = false; }
  c->connected = true;
  return EB_OK;
}

extern "C" int eb_comm_set_wait_budget(eb_comm *c, double seconds) {
  EB_REQUIRE(c, "comm_set_wait_budget: null context");
  EB_REQUIRE(seconds > 0.0 && seconds <= 60.0, "comm_set_wait_budget: between 0 and 60 seconds");
  c->wait_budget_ns = (unsigned long long)(seconds * 1e9);
  return EB_OK;
}

extern "C" int eb_comm_status(eb_comm *c, int *out4, int clear) {
  int rc = check_comm(c, "comm_status");
  if (rc) return rc;
  int host[4] = {0, 0, 0, 0};
  if (cudaMemcpy(host, c->ctl + kCtlStatus, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return fail(EB_ECUDA, "comm_status: cannot read the status words");
  }
  if (out4)
    for (int i = 0; i < 4; ++i) out4[i] = host[i];
  if (clear && host[0] != 0) cudaMemset(c->ctl + kCtlStatus, 0, sizeof(host));
  return EB_OK;
}

extern "C" int eb_comm_destroy(eb_comm *c) {
  if (!c) return EB_OK;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (c->opened[r]) cudaIpcCloseMemHandle(c->recv[r]);
  if (c->owns_recv) cudaFree(c->recv[c->rank]);
  cudaFree(c->ctl);
  cudaGetLastError();
  if (prev >= 0) cudaSetDevice(prev);
  delete c;
  return EB_OK;
}


namespace eb {
namespace {

constexpr int kRbThreads = 256;

// One lane per source: announces this rank at barrier `seq` (slot 0 or 1) to every rank.
__device__ __forceinline__ void barrier_signal(const CommDev &c, int slot, uint32_t seq) {
  if ((int)threadIdx.x < c.world)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(c.sig[threadIdx.x] + slot * 8 + c.rank), "r"(seq) : "memory");
}
// One lane per source: waits (bounded) until every rank has announced itself.  True on success.
__device__ __forceinline__ bool barrier_wait(const CommDev &c, int slot, uint32_t seq, int where) {
  bool ok = true;
  if ((int)threadIdx.x < c.world) {
    const unsigned int *w = c.sig[c.rank] + slot * 8 + threadIdx.x;
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(w) : "memory");
      if ((int)(v - seq) >= 0) break;
      if ((it & 63u) == 63u) {
        if (t0 == 0) t0 = comm_timer();
        else if (comm_timer() - t0 > c.wait_budget_ns) {
          comm_record_timeout(c, where, (int)threadIdx.x);
          ok = false;
          break;
        }
      }
    }
  }
  return ok;
}

// The second kernel of the bulk all-reduce (comm.cuh): rows [rank * rpr, (rank + 1) * rpr) of
// the [M, N] tensor are summed over the `world` staged partials (+ bias + residual), rounded to
// T and stored into every rank's gather area.  16-byte pieces, one per thread and step; a
// warp's stores cover 512 contiguous bytes of a row, locally and over NVLink.
template <typename T>
__global__ void __launch_bounds__(kRbThreads) reduce_broadcast_kernel(const CommDev c, long long M, int N, long long rpr,
                                                                      unsigned long long stage_off, unsigned long long gather_off,
                                                                      const T *bias, const T *residual, long long ldr) {
  griddep_launch();
  griddep_wait();
  __shared__ int s_ok;
  const uint32_t seq = *reinterpret_cast<volatile unsigned int *>(c.ctl + kCtlBarrier) + 1u;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // everybody's partial products are in place once every rank's GEMM has completed
  if (blockIdx.x == 0) {
    __threadfence_system();
    barrier_signal(c, 0, seq);
  }
  if (!barrier_wait(c, 0, seq, 21)) s_ok = 0;
  __syncthreads();
  const long long row0 = (long long)c.rank * rpr;
  const long long my_rows = s_ok ? (M - row0 < rpr ? (M - row0 > 0 ? M - row0 : 0) : rpr) : 0;
  const int packs = N / 8;
  const long long total = my_rows * packs;
  const T *stage = reinterpret_cast<const T *>(c.bulk[c.rank] + stage_off);
  for (long long i = (long long)blockIdx.x * kRbThreads + threadIdx.x; i < total; i += (long long)gridDim.x * kRbThreads) {
    const long long lr = i / packs;
    const int n = (int)(i - lr * packs) * 8;
    Vec16<T> part[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
      if (s < c.world) part[s].raw = __ldcg(reinterpret_cast<const uint4 *>(stage + ((long long)s * rpr + lr) * N + n));
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < c.world) {
        float f[8];
        part[s].unpack(f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += f[e];
      }
    }
    if (bias) {
      Vec16<T> b;
      b.load(bias + n);
      float f[8];
      b.unpack(f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    if (residual) {
      Vec16<T> r;
      r.load(residual + (row0 + lr) * ldr + n);
      float f[8];
      r.unpack(f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    Vec16<T> o;
    o.pack(acc);
    const unsigned long long off = gather_off + (unsigned long long)((row0 + lr) * N + n) * sizeof(T);
    for (int r = 0; r < c.world; ++r) *reinterpret_cast<uint4 *>(c.bulk[r] + off) = o.raw;
  }
  // every rank holds all rows once every rank's stores have landed
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(c.ctl + kCtlBlocks, 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    barrier_signal(c, 1, seq);
    barrier_wait(c, 1, seq, 22);
    __syncthreads();
    if (threadIdx.x == 0) {
      c.ctl[kCtlBlocks] = 0u;
      c.ctl[kCtlBarrier] = seq;
      __threadfence();
    }
  }
}

}  // namespace
}  // namespace eb

extern "C" int eb_comm_local_area(eb_comm *c, void **bulk_ptr, size_t *bulk_bytes) {
  EB_REQUIRE(c && bulk_ptr && bulk_bytes, "comm_local_area: null argument");
  *bulk_ptr = reinterpret_cast<unsigned char *>(c->recv[c->rank]) + kSignalBytes + c->line_bytes;
  *bulk_bytes = c->bulk_bytes;
  return EB_OK;
}

extern "C" size_t eb_reduce_broadcast_stage_bytes(int world, long long M, int N) {
  if (world <= 0 || M <= 0 || N <= 0) return 0;
  return (size_t)world * (size_t)comm_rows_per_rank(M, world) * (size_t)N * 2;
}

extern "C" int eb_reduce_broadcast(eb_comm *c, long long M, int N, int dtype, size_t stage_offset, size_t gather_offset,
                                   const void *bias, const void *residual, long long ldr, void *stream) {
  int rc = check_comm(c, "reduce_broadcast");
  if (rc) return rc;
  EB_REQUIRE(dtype == EB_F16 || dtype == EB_BF16, "reduce_broadcast: fp16 or bf16 only");
  EB_REQUIRE(M > 0 && N > 0 && N % 8 == 0, "reduce_broadcast: N must be a positive multiple of 8");
  EB_REQUIRE(c->connected, "reduce_broadcast: the context is not connected to its peers yet");
  const long long rpr = comm_rows_per_rank(M, c->world);
  const size_t stage = (size_t)c->world * rpr * N * 2, gather = (size_t)M * N * 2;
  EB_REQUIRE(stage_offset % 256 == 0 && gather_offset % 256 == 0, "reduce_broadcast: offsets must be multiples of 256");
  if (stage_offset + stage > c->bulk_bytes || gather_offset + gather > c->bulk_bytes)
    return fail(EB_ELIMIT, "reduce_broadcast: %lld x %d needs %zu + %zu bytes of the bulk region, which has %zu", M, N, stage,
                gather, c->bulk_bytes);
  EB_REQUIRE((stage_offset + stage <= gather_offset) || (gather_offset + gather <= stage_offset),
             "reduce_broadcast: the staging and gather areas overlap");
  EB_REQUIRE(aligned16(bias) && aligned16(residual) && (!residual || (ldr >= N && ldr % 8 == 0)), "reduce_broadcast: bad bias / residual");
  const CommDev d = comm_dev(c);
  const long long total = rpr * (N / 8);
  const long long want = (total + kRbThreads - 1) / kRbThreads;
  const int grid = (int)(want < sm_count() ? (want > 0 ? want : 1) : sm_count());
  cudaStream_t st = as_stream(stream);
  if (dtype == EB_F16)
    launch_pdl(reduce_broadcast_kernel<__half>, dim3(grid), dim3(kRbThreads), 0, st, d, M, N, rpr, (unsigned long long)stage_offset,
               (unsigned long long)gather_offset, reinterpret_cast<const __half *>(bias), reinterpret_cast<const __half *>(residual), ldr);
  else
    launch_pdl(reduce_broadcast_kernel<__nv_bfloat16>, dim3(grid), dim3(kRbThreads), 0, st, d, M, N, rpr,
               (unsigned long long)stage_offset, (unsigned long long)gather_offset, reinterpret_cast<const __nv_bfloat16 *>(bias),
               reinterpret_cast<const __nv_bfloat16 *>(residual), ldr);
  return check_launch("reduce_broadcast");
}

extern "C" int eb_allreduce(eb_comm *c, void *buf, size_t count, int dtype, void *stream) {
  int rc = check_comm(c, "allreduce");
  if (rc) return rc;
  EB_REQUIRE(dtype_ok(dtype), "allreduce: unknown dtype %d", dtype);
  if (count == 0) return EB_OK;
  EB_REQUIRE(c->connected, "allreduce: the context is not connected to its peers yet");
  const size_t bytes = count * dtype_size(dtype);
  EB_REQUIRE(buf && (reinterpret_cast<uintptr_t>(buf) & 7u) == 0 && bytes % 8 == 0,
             "allreduce: the buffer must be 8-byte aligned and a multiple of 8 bytes");
  const unsigned long long lines = bytes / 8;
  if ((unsigned long long)c->world * lines * 16ull > c->line_bytes / 2)
    return fail(EB_ELIMIT, "allreduce: %zu bytes from %d ranks need %llu bytes per half of the receive area, which has %zu",
                bytes, c->world, (unsigned long long)c->world * lines * 16ull, c->line_bytes / 2);
  const CommDev d = comm_dev(c);
  const long long want = (long long)((lines + kArThreads - 1) / kArThreads);
  const int grid = (int)(want < sm_count() ? want : sm_count());
  cudaStream_t st = as_stream(stream);
  if (dtype == EB_F32) launch_pdl(allreduce_kernel<float>, dim3(grid), dim3(kArThreads), 0, st, d, reinterpret_cast<float *>(buf), lines);
  else if (dtype == EB_F16) launch_pdl(allreduce_kernel<__half>, dim3(grid), dim3(kArThreads), 0, st, d, reinterpret_cast<__half *>(buf), lines);
  else launch_pdl(allreduce_kernel<__nv_bfloat16>, dim3(grid), dim3(kArThreads), 0, st, d, reinterpret_cast<__nv_bfloat16 *>(buf), lines);
  return check_launch("allreduce");
}
