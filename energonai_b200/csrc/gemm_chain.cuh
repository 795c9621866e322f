// One launch for a chain of dependent generation-step operations.
//
// A generation step is a sequence of small-batch GEMMs (weight streams) separated by LayerNorms:
//   out-proj -> LayerNorm -> FC1 -> FC2 -> LayerNorm(next layer) -> QKV(next layer)
// Launched one kernel per operation, every boundary costs a drain, a launch and a pipeline
// fill during which HBM idles.  Here the whole chain runs in one persistent kernel (one CTA per
// SM): the TMA producer keeps streaming the weights of the following GEMM into the shared-memory
// ring while the grid waits for the previous operation to complete, because weights never
// depend on it; only the (tiny) activation tiles wait.  Operations are separated by grid-wide
// barriers implemented as one arrival counter per operation in global memory; every wait on
// them is bounded like the mbarrier waits and ends in the same abort path.
//
// Included by gemm.cu inside namespace eb::(anonymous), after the single-GEMM kernel whose PTX
// wrappers, descriptors and status word it shares.
#pragma once

constexpr int kMaxOps = 8;
constexpr int kOpGemm = 0, kOpLayerNorm = 1, kOpReduceLn = 2;

struct ChainGemm {
  int N, K, kblocks, nsk;        // nsk = pipeline stages per 128-row tile
  int tiles;                     // 128-row tiles of W
  int units_per_cta;             // stream-K units (stages) per CTA; CTA b owns [b*u, min((b+1)*u, tiles*nsk))
  void *C;
  long long ldc;
  int c_rows_per_batch;
  long long c_batch_stride;
  const int *c_row_offset_dev;
  int c_row_limit;               // > 0: the device row offset must lie in [0, limit)
  const void *bias, *residual;
  long long ldr;
  int act, out_f32;
  float *partial;                // [grid][2][BN][128]
  int *counters;                 // [tiles], zero between launches
  // exchange >= 0: a row-parallel product of a tensor-parallel group.  Instead of being stored,
  // the finished tiles go to every rank's receive area as flagged lines [source][m][N / 4]
  // (comm.cuh), with sequence number epoch + 1 + exchange; the kReduceLn operation that follows
  // adds the ranks' contributions up.  -1: an ordinary GEMM.
  int exchange;
};

struct ChainLn {
  const void *x, *gamma, *beta;
  void *y;
  int n2;
  float eps;
  // kOpReduceLn only: x_sum = sum over ranks of the preceding exchange + bias + residual is
  // written to `sum_out` (rounded to the operand type) and normalised into y (gamma == null: no
  // normalisation, y unused).
  const void *bias, *residual;
  long long ldr;
  void *sum_out;
  long long ld_sum;
  int exchange;
  // kOpReduceLn: a row is cut into `split` column slices, one CTA each (CTA m * split + j takes
  // slice j of row m), so that the collection of the ranks' lines is one or two rounds of loads
  // per thread instead of ten; the slices' partial statistics meet in `stats` [row][slice] and
  // `rowdone` [row] counts the slices that have delivered theirs (zero between launches).
  int split;
  float2 *stats;
  int *rowdone;
};

struct ChainParams {
  int n_ops, M, stages, kpb;
  int prefetch;                  // weight stages requested into L2 beyond the ring while the producer waits
  int type[kMaxOps];
  ChainGemm g[kMaxOps];
  ChainLn l[kMaxOps];
  int *done;                     // [kMaxOps] arrival counters, zero between launches
  CommDev comm;                  // exchange context (world >= 1) when n_exchanges > 0
  int n_exchanges;               // exchanges this launch performs; the epoch advances by that much
  uint32_t xpose_off;            // shared-memory offset (from the tiles) of the push staging area
};

struct ChainMaps {
  CUtensorMap w[kMaxOps];        // weights  [N, K], box 64 x 128
  CUtensorMap x[kMaxOps];        // activations [M, K], box 64 x BN
};

__device__ __forceinline__ int ld_acquire_gpu(const int *p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Position of one CTA inside the stream-K range of one GEMM of the chain.
struct ChainCursor {
  int pos, end, nsk, tile, sk;           // pos = tile * nsk + sk
  __device__ void open(const ChainGemm &g) {
    const int total = g.tiles * g.nsk;
    nsk = g.nsk;
    pos = (int)blockIdx.x * g.units_per_cta;
    end = pos + g.units_per_cta < total ? pos + g.units_per_cta : total;
    if (pos > end) pos = end;
    tile = pos / nsk;
    sk = pos - tile * nsk;
  }
  __device__ bool empty() const { return pos >= end; }
  __device__ void step() {               // one stage forward
    ++pos;
    if (++sk == nsk) { sk = 0; ++tile; }
  }
};

// Bounded wait until `count` CTAs have arrived at done[op]; false when the CTA is aborting.
__device__ __noinline__ bool chain_wait_done(const int *done, int op, int count, volatile int *abort_flag) {
  if (ld_acquire_gpu(done + op) >= count) return true;
  const unsigned long long t0 = globaltimer();
  for (unsigned it = 1;; ++it) {
    if (ld_acquire_gpu(done + op) >= count) return true;
    if ((it & 15u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer() - t0 > kWaitBudgetNs) {
        *abort_flag = 1;
        if (atomicCAS(&g_status[0], 0, EB_ETIMEDOUT) == 0) {
          g_status[1] = 7; g_status[2] = blockIdx.x; g_status[3] = op;
        }
        return false;
      }
    }
  }
}


template <typename T, int BN>
__global__ void __launch_bounds__(kThreads, 1)
chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams p) {
  constexpr uint32_t kColBytes = BN * 128, lane_bytes = kLanes * 128u;
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  constexpr uint32_t kIdesc = make_idesc(BN, std::is_same<T, __nv_bfloat16>::value ? 1 : 0);
  constexpr uint32_t sub_bytes = lane_bytes + kColBytes;
  const uint32_t stage_bytes = sub_bytes * (uint32_t)p.kpb;
  const int stages = p.stages, kpb = p.kpb;
  const int grid = gridDim.x;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
  const uint32_t full_bar = smem_u32(bars), empty_bar = full_bar + 8 * kMaxStages;
  const uint32_t tfull_bar = empty_bar + 8 * kMaxStages, tempty_bar = tfull_bar + 16, epi_bar = tempty_bar + 16;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kMaxStages + 5);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile int *last_flag = reinterpret_cast<volatile int *>(tmem_slot + 2);   // two entries, alternating
  float *ln_scratch = reinterpret_cast<float *>(tmem_slot + 4);                // 8 floats
  const uint32_t tiles_addr = smem_u32(smem) + kBarrierBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar + 8 * a, 1);
      mbar_init(tempty_bar + 8 * a, 4);
    }
    mbar_init(epi_bar, 128);
    *abort_flag = 0;
    last_flag[0] = last_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  griddep_launch();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // Two cursors over the same sequence of pipeline stages: the weight cursor arms a stage and
    // requests its weight tiles as soon as the slot is free; the activation cursor follows and
    // requests the activation tiles of armed stages once the operation that produces them is
    // complete (grid-wide).  Lane j moves k-block j of a stage.
    const bool mover = lane < kpb;
    const uint32_t movers_mask = kpb >= 32 ? 0xffffffffu : ((1u << kpb) - 1u);
    if (mover) {
      int w_op = 0, x_op = 0, ahead = 0, ready_upto = -1;   // ahead: stages armed whose activations are
      int w_slot = 0, x_slot = 0;                           // not requested yet; ops [0, ready_upto] complete
      uint32_t w_par = 1;                                   // parity to wait for on empty_bar[w_slot]
      ChainCursor wc, xc, pc;                               // pc: L2 prefetch cursor, pf_ahead stages beyond wc
      int p_op = 0, pf_ahead = 0;
      auto seek = [&](int &op, ChainCursor &c) {           // next GEMM with work for this CTA, from `op` on
        while (op < p.n_ops) {
          if (p.type[op] == kOpGemm) {
            c.open(p.g[op]);
            if (!c.empty()) return;
          }
          ++op;
        }
      };
      seek(w_op, wc);
      seek(x_op, xc);
      seek(p_op, pc);
      // While the ring is full of weights whose activations are not available yet, HBM would
      // idle; keep it busy by pulling the following weight stages into L2, from where the ring
      // refills faster than from DRAM once the dependency is resolved.
      auto prefetch_one = [&]() {
        const ChainGemm &g = p.g[p_op];
        const int nvalid = g.kblocks - pc.sk * kpb < kpb ? g.kblocks - pc.sk * kpb : kpb;
        if (lane < nvalid) tma_prefetch_l2_2d(&maps.w[p_op], (pc.sk * kpb + lane) * kBlockK, pc.tile * kLanes);
        pc.step();
        if (pc.empty()) { ++p_op; seek(p_op, pc); }
        ++pf_ahead;
      };
      bool waited = false;                                 // griddepcontrol.wait done (inputs of op 0 valid)
      unsigned idle = 0;
      unsigned long long t0 = 0;
      while (x_op < p.n_ops) {
        int act = 0;
        if (lane == 0) {
          int pending = ahead;
          if (w_op < p.n_ops && ahead < stages) {
            // nothing else to do: a suspending wait is fine; activations outstanding: only probe
            const bool free_slot = ahead == 0 ? mbar_try_wait(empty_bar + 8 * w_slot, w_par)
                                              : mbar_test_wait(empty_bar + 8 * w_slot, w_par);
            if (free_slot) { act |= 1; ++pending; }
          }
          if (pending > 0) {
            if (!waited) {
              // the arrival counters may still hold the previous launch's values until the
              // preceding kernels have completed: never read them before griddepcontrol.wait
              act |= 4;
            } else {
              // the activation operand of op x_op is produced by op x_op-1 (or precedes the kernel)
              bool ok = x_op == 0 ? true : x_op - 1 <= ready_upto;
              if (!ok && ld_acquire_gpu(p.done + x_op - 1) >= grid) {
                ready_upto = x_op - 1; ok = true; act |= 8;
              }
              if (ok) act |= 2;
            }
          }
        }
        act = __shfl_sync(movers_mask, act, 0);
        if (act & 1) {
          const ChainGemm &g = p.g[w_op];
          const int tile = wc.tile, sk = wc.sk;
          const uint32_t fb = full_bar + 8 * w_slot;
          const int nvalid = g.kblocks - sk * kpb < kpb ? g.kblocks - sk * kpb : kpb;
          if (lane == 0) mbar_expect_tx(fb, (uint32_t)nvalid * sub_bytes);
          __syncwarp(movers_mask);
          if (lane < nvalid)
            tma_load_2d(tiles_addr + w_slot * stage_bytes + lane * sub_bytes, &maps.w[w_op], fb, (sk * kpb + lane) * kBlockK,
                        tile * kLanes);
          ++ahead;
          if (++w_slot == stages) { w_slot = 0; w_par ^= 1u; }
          wc.step();
          if (wc.empty()) { ++w_op; seek(w_op, wc); }
          if (pf_ahead > 0) --pf_ahead;
          else { p_op = w_op; pc = wc; }
        }
        if ((act & 5) == 4) {                              // ring full (or weights exhausted): now wait
          while (pf_ahead < p.prefetch && p_op < p.n_ops) prefetch_one();
          griddep_wait();
          waited = true;
        }
        // the activations were written by generic-proxy stores of other CTAs and the TMA reads
        // them through the async proxy: one proxy fence when an operation is first seen complete
        if (act & 8) asm volatile("fence.proxy.async;" ::: "memory");
        if (act & 2) {
          const ChainGemm &g = p.g[x_op];
          const int sk = xc.sk;
          const int nvalid = g.kblocks - sk * kpb < kpb ? g.kblocks - sk * kpb : kpb;
          if (lane < nvalid)
            tma_load_2d(tiles_addr + x_slot * stage_bytes + lane * sub_bytes + lane_bytes, &maps.x[x_op],
                        full_bar + 8 * x_slot, (sk * kpb + lane) * kBlockK, 0);
          --ahead;
          if (++x_slot == stages) x_slot = 0;
          xc.step();
          if (xc.empty()) { ++x_op; seek(x_op, xc); }
        }
        if (act) { idle = 0; continue; }
        if (ahead > 0 && pf_ahead < p.prefetch && p_op < p.n_ops) {   // waiting for an operation to complete
          prefetch_one();
          continue;
        }
        // nothing could be issued: bounded idle
        int stop = 0;
        if (lane == 0) {
          if (idle == 0) t0 = globaltimer();
          if ((idle & 63u) == 63u) {
            if (*abort_flag) stop = 1;
            else if (globaltimer() - t0 > kWaitBudgetNs) {
              *abort_flag = 1;
              if (atomicCAS(&g_status[0], 0, EB_ETIMEDOUT) == 0) { g_status[1] = 8; g_status[2] = blockIdx.x; g_status[3] = x_op; }
              stop = 1;
            }
          }
        }
        ++idle;
        stop = __shfl_sync(movers_mask, stop, 0);
        if (stop) break;
      }
      if (!waited) griddep_wait();
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    griddep_wait();
    if (lane == 0) {
      int slot = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int op = 0; op < p.n_ops && ok; ++op) {
        if (p.type[op] != kOpGemm) continue;
        const ChainGemm &g = p.g[op];
        ChainCursor c;
        c.open(g);
        while (ok && !c.empty()) {
          const int tile = c.pos / c.nsk, sk0 = c.pos - tile * c.nsk;
          const int left = c.end - c.pos;
          const int sk1 = sk0 + left < c.nsk ? sk0 + left : c.nsk;
          if (!mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, 2)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          for (int sk = sk0; sk < sk1; ++sk) {
            if (!mbar_wait(full_bar + 8 * slot, phase, abort_flag, 3)) { ok = false; break; }
            tcgen05_fence_after();
            for (int j = 0; j < kpb && sk * kpb + j < g.kblocks; ++j) {
              const uint32_t a_addr = tiles_addr + slot * stage_bytes + j * sub_bytes;
              const uint64_t a_desc = make_smem_desc(a_addr), b_desc = make_smem_desc(a_addr + lane_bytes);
#pragma unroll
              for (int k = 0; k < kBlockK / kUmmaK; ++k)
                tcgen05_mma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, kIdesc, (sk > sk0 || j > 0 || k > 0) ? 1u : 0u);
            }
            tcgen05_commit(empty_bar + 8 * slot);
            if (++slot == stages) { slot = 0; phase ^= 1u; }
          }
          if (!ok) break;
          tcgen05_commit(tfull_bar + 8 * acc);
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
          c.pos += sk1 - sk0;
        }
      }
    }
  } else {
#include "gemm_chain_epilogue.inc"
  }

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}
