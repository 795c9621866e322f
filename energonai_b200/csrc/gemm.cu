// Dense C = act(A · Wᵀ + bias) + residual on the 5th-generation tensor cores (tcgen05).
//
// Both operands are K-major 16-bit matrices (A [M,K], W [N,K]); accumulation is fp32 in
// tensor memory.  One kernel template serves two orientations:
//
//   normal (M > 128): TMEM lanes = 128 rows of A, TMEM columns = BN rows of W.  Persistent
//       CTAs walk 128 x BN output tiles in a grouped raster so that concurrently running CTAs
//       share A and W panels in L2.
//   swapped (M <= 128, generation steps): TMEM lanes = 128 rows of W, TMEM columns = the (padded)
//       M rows of A.  The work is one pass over W (HBM-bound).  An MMA over 128 lanes costs the
//       same however many lanes carry useful rows, so W is always taken in full 128-row tiles,
//       and the (tile, k) space is cut stream-K style into equal contiguous ranges, one per CTA:
//       every SM pulls the same number of weight bytes.  A tile shared by several CTAs is
//       reduced through fp32 partials in a caller-provided workspace by whichever CTA arrives
//       last, summing in a fixed order, so results are deterministic.
//
// Warp roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = TMEM allocation and
// tcgen05.mma issue (one lane), warps 2-5 = epilogue (tcgen05.ld -> bias / activation /
// residual -> global).  Shared-memory stages are handed over with mbarriers (full: TMA
// transaction bytes; empty: tcgen05.commit), and two TMEM accumulators are ping-ponged so the
// epilogue of one tile overlaps the main loop of the next.
//
// The kernel is launched with programmatic stream serialization: its prologue and the first
// weight tiles (which never depend on the preceding kernel) are issued before
// griddepcontrol.wait; only the activation tiles and the epilogue wait for the predecessor.
//
// Every mbarrier wait is bounded by a wall-clock budget.  When it expires the CTA records
// where it gave up in a device status word (eb_device_status), raises a CTA-wide abort flag so
// the other roles leave their loops, lets in-flight copies land, frees its tensor memory and
// returns; the context stays usable.
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "comm.cuh"

namespace eb {
namespace {

constexpr int kLanes = 128;      // rows of the lane-side operand per tile (UMMA M)
constexpr int kBlockK = 64;      // 64 x 16 bit = 128 bytes = one swizzle-128B row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kGroup = 16;       // raster group height (lane-side tiles) in normal mode
constexpr unsigned long long kWaitBudgetNs = 1000ull * 1000ull * 1000ull;
constexpr int kMaxStages = 32;
constexpr int kXposeMaxLines = 8;            // fused exchange: widest per-thread line count that is sent through shared memory
constexpr uint32_t kBarrierBytes = 1024;      // head of shared memory: mbarriers, TMEM slot, abort flag

__device__ int g_status[4];      // [0] code (0 = ok), [1] where, [2] block, [3] detail

struct GemmParams {
  int M, N, K;                   // logical problem: C[M,N] = A[M,K] W[N,K]^T
  int lane_rows, col_rows;       // rows of the lane-side / column-side operand (swap: N, M)
  int kblocks;                   // ceil(K / 64)
  void *C;
  long long ldc;
  int c_rows_per_batch;          // 0: row m of C is at m*ldc; else (m / rpb)*c_batch_stride + (m % rpb)*ldc
  long long c_batch_stride;
  const int *c_row_offset_dev;   // optional device scalar: extra row offset of C (rows of ldc), read at run time
  int c_row_limit;               // > 0: the device offset must lie in [0, limit); otherwise nothing is stored
  const void *bias;              // [N] or null
  const void *residual;          // [M, N] rows ldr apart, or null
  long long ldr;
  int act;
  int out_f32;                   // 1: C is fp32, else the input type
  float *partial;                // swap mode: stream-K partial sums [cta][2][BN][128]
  int *counters;                 // swap mode: one arrival counter per 128-row tile, zero between calls
  int units_per_cta;             // swap mode: stream-K units (one unit = one pipeline stage of one tile) per CTA
  int stages;                    // pipeline depth actually used (<= kMaxStages)
  int kpb;                       // k-blocks (64 columns each) per pipeline stage / barrier hand-over
  int static_w;                  // W may be read before the preceding kernel of the stream has finished
  int x3d;                       // swap mode: tm_col is a 3-D map [k-block][row][64] of the activations: one copy per stage
  // Fused all-reduce of the generation orientation (comm.world >= 1; a single rank exchanges with itself): the CTA that completes a
  // tile sends this rank's partial product to every rank as flagged lines and adds up what the
  // ranks sent it (see comm.cuh).  A thread's BN batch values of output column n are contiguous
  // in the receive area: lines [source][n][BN / 4].
  CommDev comm;
  // Normal orientation, reduce-scatter mode (rs != 0): the tile is this rank's partial product of
  // a row-parallel layer and goes, in the operand type, into the staging area of the rank that
  // owns its rows (comm.cuh): bulk[owner] + rs_stage_off, layout [source][row in block][N].
  int rs;
  long long rs_rpr;
  unsigned long long rs_stage_off;
  // swap mode, optional: the A operand is the un-normalised input of a LayerNorm whose scale
  // was multiplied into W beforehand.  The kernel computes each row's mean / inverse std over
  // K itself and the last epilogue of a tile evaluates
  //   y[m][n] = rstd[m] * (acc[m][n] - mean[m] * ln_colsum[n]) + ln_bias[n]
  // (ln_colsum[n] = sum_k W'[n][k], ln_bias[n] = bias[n] + sum_k W[n][k] * beta[k], both fp32).
  const float *ln_colsum, *ln_bias;
  const void *ln_x;
  long long ln_ldx;
  float ln_eps;
};

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking probe (try_wait may suspend the thread for a hardware-defined time).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (this or another role ran out of time).
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int where) {
  const unsigned long long t0 = globaltimer();
  for (unsigned it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer() - t0 > kWaitBudgetNs) {
        *abort_flag = 1;
        if (atomicCAS(&g_status[0], 0, EB_ETIMEDOUT) == 0) {
          g_status[1] = where;
          g_status[2] = blockIdx.x;
          g_status[3] = (int)parity;
        }
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, where);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// Asks for a weight tile to be brought into L2 (no shared-memory destination, no completion).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float *v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B): 8-row groups are 1024
// bytes apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulate, A/B format (0 f16, 1 bf16), both K-major.
__host__ __device__ constexpr uint32_t make_idesc(int n, int is_bf16) {
  return (1u << 4) | ((uint32_t)is_bf16 << 7) | ((uint32_t)is_bf16 << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kLanes >> 4) << 24);
}

// ---- work decomposition -----------------------------------------------------------------------
struct Segment {
  int lane_row0;             // first row of the lane-side operand
  int lane_tile;             // its tile index
  int col_tile;              // tile index of the column-side operand
  int sk0, sk1;              // range of pipeline stages (kpb k-blocks each) of this tile
  bool partial;              // covers only part of K (swap mode)
  int which;                 // 0: first segment of this CTA's range, 1: a later one
};

template <int BN, bool SWAP> struct Scheduler {
  const GemmParams &p;
  int lane_tiles, col_tiles, nsk;
  int pos, end;              // 32-bit on purpose: these feed divisions on the critical path
  int h0, h1;                // swap mode: the CTA's last, partial tile, which it processes FIRST
  bool first;
  __device__ Scheduler(const GemmParams &pp) : p(pp) {
    lane_tiles = (p.lane_rows + kLanes - 1) / kLanes;
    col_tiles = SWAP ? 1 : (p.col_rows + BN - 1) / BN;
    nsk = (p.kblocks + p.kpb - 1) / p.kpb;
    first = true;
    if (SWAP) {
      // The CTA owns the stage range [pos, end) of the tile-major sequence.  If the range ends
      // inside a tile (and started before it), that partial piece [h0, h1) goes first, then
      // the rest in order: partial pieces need the cross-CTA sum, whose round trips are hidden
      // while later stages stream in, and the pieces a CTA finishes with are complete tiles.
      const int total = lane_tiles * nsk;
      pos = (int)blockIdx.x * p.units_per_cta;
      end = pos + p.units_per_cta < total ? pos + p.units_per_cta : total;
      h0 = h1 = 0;
      if (end > pos) {
        const int tile_start = (end / nsk) * nsk;
        if (end > tile_start && tile_start > pos) { h0 = tile_start; h1 = end; end = tile_start; }
      }
    } else {
      pos = blockIdx.x;
      end = lane_tiles * col_tiles;
    }
  }
  __device__ bool next(Segment &s) {
    if (SWAP && h1 > h0) {
      s.lane_tile = h0 / nsk;
      s.col_tile = 0;
      s.sk0 = 0;
      s.sk1 = h1 - h0;
      s.partial = true;
      s.which = 1;             // not the first piece of the range in k order
      s.lane_row0 = s.lane_tile * kLanes;
      h1 = h0;
      return true;
    }
    if (pos >= end) return false;
    if (SWAP) {
      s.lane_tile = pos / nsk;
      s.col_tile = 0;
      s.sk0 = pos - s.lane_tile * nsk;
      const int left = end - pos;
      s.sk1 = s.sk0 + left < nsk ? s.sk0 + left : nsk;
      s.partial = !(s.sk0 == 0 && s.sk1 == nsk);
      s.which = first ? 0 : 1;
      pos += s.sk1 - s.sk0;
    } else {
      const int per_group = kGroup * col_tiles;
      const int group = pos / per_group, in_group = pos - group * per_group;
      const int first_lane = group * kGroup;
      const int gsz = lane_tiles - first_lane < kGroup ? lane_tiles - first_lane : kGroup;
      s.lane_tile = first_lane + in_group % gsz;
      s.col_tile = in_group / gsz;
      s.sk0 = 0;
      s.sk1 = nsk;
      s.partial = false;
      s.which = 0;
      pos += gridDim.x;
    }
    s.lane_row0 = s.lane_tile * kLanes;
    first = false;
    return true;
  }
};

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == EB_ACT_RELU) return fmaxf(v, 0.f);
  if (act == EB_ACT_GELU_TANH) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * v * (1.f + 0.044715f * v * v)));
  if (act == EB_ACT_GELU_ERF) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  return v;
}

// A run-time row offset outside [0, c_row_limit) would write past the caller's buffer (a cache
// that was not sized for the step): nothing is stored and the status word says so.
__device__ __forceinline__ bool row_in_limit(const GemmParams &p, int row) {
  if (!p.c_row_offset_dev || p.c_row_limit <= 0 || (row >= 0 && row < p.c_row_limit)) return true;
  if (atomicCAS(&g_status[0], 0, EB_ELIMIT) == 0) {
    g_status[1] = 9; g_status[2] = blockIdx.x; g_status[3] = row;
  }
  return false;
}

__device__ __forceinline__ long long c_row_offset(const GemmParams &p, int m) {
  const long long extra = p.c_row_offset_dev ? (long long)__ldg(p.c_row_offset_dev) * p.ldc : 0;
  if (p.c_rows_per_batch <= 0) return (long long)m * p.ldc + extra;
  return (long long)(m / p.c_rows_per_batch) * p.c_batch_stride + (long long)(m % p.c_rows_per_batch) * p.ldc + extra;
}

// ---- the kernel ---------------------------------------------------------------------------------
// Shared memory: [1 KB: mbarriers, TMEM slot, flags][stages x kpb x (lane tile | column tile)].
// (A form with two CTAs per SM, half the stages each, so that the next launch's CTAs could start
// their weight stream beside a running launch, was measured on the shard shapes of an 8-way
// group: 51 us per layer against 36 us.  One CTA per SM it is.)
template <typename T, int BN, bool SWAP>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_lane, const __grid_constant__ CUtensorMap tm_col, const GemmParams p) {
  constexpr uint32_t kColBytes = BN * 128;
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  constexpr uint32_t kIdesc = make_idesc(BN, std::is_same<T, __nv_bfloat16>::value ? 1 : 0);
  constexpr uint32_t lane_bytes = kLanes * 128u;
  const uint32_t sub_bytes = lane_bytes + kColBytes;      // one k-block: lane tile + column tile
  const uint32_t stage_bytes = sub_bytes * (uint32_t)p.kpb;   // a stage: [kpb lane tiles][kpb column tiles]
  const uint32_t col_base = lane_bytes * (uint32_t)p.kpb;    // offset of the column tiles inside a stage
  const int stages = p.stages, kpb = p.kpb;
  const int nsk = (p.kblocks + kpb - 1) / kpb;             // stages' worth of K per output tile

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
  const uint32_t full_bar = smem_u32(bars), empty_bar = full_bar + 8 * kMaxStages;
  const uint32_t tfull_bar = empty_bar + 8 * kMaxStages, tempty_bar = tfull_bar + 16;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kMaxStages + 5);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t epi_bar = tempty_bar + 16;
  const uint32_t tiles_addr = smem_u32(smem) + kBarrierBytes;
  // behind the stages: per epilogue warp, the lines of a fused exchange on their way out (see the epilogue)
  uint8_t *xpose = smem + kBarrierBytes + (size_t)p.stages * stage_bytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    // the descriptors are fetched now, not by the first copy that needs them
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_lane) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_col) : "memory");
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar + 8 * a, 1);
      mbar_init(tempty_bar + 8 * a, 4);   // one arrival per epilogue warp
    }
    mbar_init(epi_bar, 128);               // rendezvous of the four epilogue warps
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_lane) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_col) : "memory");
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
  griddep_launch();   // the next kernel of the stream may become resident and run its own prologue

  if (warp == 0) {
    // ---------------- TMA producer (whole warp; lane j moves k-block j of every stage) ----------------
    // A single thread issuing every copy was the bottleneck of the weight-streaming case (its
    // dependent instruction chain per stage took longer than the stage's bytes need at HBM
    // speed), so the k-blocks of a stage are spread over lanes and the per-stage bookkeeping
    // (barrier wait, expected byte count) is done once by lane 0.
    //
    // When the caller declares the weights static (they do not depend on the preceding kernel
    // of the stream), the weight tiles of the first `stages` stages are requested before
    // waiting for that kernel; activations always follow the wait.
    const CUtensorMap *tm_w = SWAP ? &tm_lane : &tm_col;
    const CUtensorMap *tm_x = SWAP ? &tm_col : &tm_lane;
    const uint32_t lane_off = lane * lane_bytes, colt_off = col_base + lane * kColBytes;
    const uint32_t w_off = SWAP ? lane_off : colt_off;
    const uint32_t x_off = SWAP ? colt_off : lane_off;
    // The activation tiles of the swapped orientation are small (batch rows x 128 bytes), and a
    // TMA copy of such a box costs about 0.3 us whatever its size: with one copy per k-block the
    // stages of a CTA became ready 0.6 us apart although their weights had long arrived.  With a
    // 3-D view [k-block][row][64 columns] of the activations one copy brings all kpb tiles of a stage.
    const bool x3d = SWAP && p.x3d;
    const bool mover = lane < kpb;
    const uint32_t movers_mask = kpb >= 32 ? 0xffffffffu : ((1u << kpb) - 1u);
    if (mover) {
    const int last_valid = p.kblocks - (nsk - 1) * kpb;                   // k-blocks in the last stage of a tile
    const uint32_t full_tx = stage_bytes;
    const uint32_t last_tx = x3d ? (uint32_t)last_valid * lane_bytes + (uint32_t)kpb * kColBytes : (uint32_t)last_valid * sub_bytes;
    int pre = 0;
    if (!p.static_w) griddep_wait();
    {
      Scheduler<BN, SWAP> sw(p);
      Segment s;
      while (pre < stages && sw.next(s)) {
        const int w_row = SWAP ? s.lane_row0 : s.col_tile * BN;
        for (int sk = s.sk0; sk < s.sk1 && pre < stages; ++sk, ++pre) {
          const uint32_t fb = full_bar + 8 * pre;
          if (lane == 0) mbar_expect_tx(fb, sk == nsk - 1 ? last_tx : full_tx);
          __syncwarp(movers_mask);
          const int kb = sk * kpb + lane;
          if (mover && kb < p.kblocks) tma_load_2d(tiles_addr + pre * stage_bytes + w_off, tm_w, fb, kb * kBlockK, w_row);
        }
      }
    }
    if (p.static_w) griddep_wait();
    Scheduler<BN, SWAP> sched(p);
    Segment s;
    int stage = 0, iter = 0;
    uint32_t phase = 0;
    bool ok = true;
    while (ok && sched.next(s)) {
      const int w_row = SWAP ? s.lane_row0 : s.col_tile * BN;
      const int x_row = SWAP ? s.col_tile * BN : s.lane_row0;
      for (int sk = s.sk0; sk < s.sk1; ++sk, ++iter) {
        const uint32_t fb = full_bar + 8 * stage;
        const uint32_t dst = tiles_addr + stage * stage_bytes;
        const bool fresh = iter >= pre;          // the weight tile was not requested before the wait
        if (fresh) {
          int good = 1;
          if (lane == 0) {
            good = mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, 1) ? 1 : 0;
            if (good) mbar_expect_tx(fb, sk == nsk - 1 ? last_tx : full_tx);
          }
          good = __shfl_sync(movers_mask, good, 0);
          if (!good) { ok = false; break; }
        }
        const int kb = sk * kpb + lane;
        if (mover && kb < p.kblocks) {
          if (fresh) tma_load_2d(dst + w_off, tm_w, fb, kb * kBlockK, w_row);
          if (!x3d) tma_load_2d(dst + x_off, tm_x, fb, kb * kBlockK, x_row);
        }
        if (x3d && lane == 0) tma_load_3d(dst + col_base, tm_x, fb, 0, x_row, sk * kpb);   // k-blocks beyond K read as zeros
        if (++stage == stages) { stage = 0; phase ^= 1u; }
      }
    }
    }   // mover lanes
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    griddep_wait();
    if (lane == 0) {
      Scheduler<BN, SWAP> sched(p);
      Segment s;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      while (ok && sched.next(s)) {
        if (!mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, 2)) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int sk = s.sk0; sk < s.sk1; ++sk) {
          if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, 3)) { ok = false; break; }
          tcgen05_fence_after();
          for (int j = 0; j < kpb && sk * kpb + j < p.kblocks; ++j) {
            const uint32_t st_addr = tiles_addr + stage * stage_bytes;
            const uint64_t a_desc = make_smem_desc(st_addr + j * lane_bytes), b_desc = make_smem_desc(st_addr + col_base + j * kColBytes);
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              // advancing 16 elements along K inside the swizzle atom = +32 bytes = +2 in the address field
              tcgen05_mma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, kIdesc, (sk > s.sk0 || j > 0 || k > 0) ? 1u : 0u);
            }
          }
          tcgen05_commit(empty_bar + 8 * stage);   // frees the stage once these MMAs have read it
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tcgen05_commit(tfull_bar + 8 * acc);        // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    griddep_wait();
    const int quarter = warp & 3;                   // TMEM lane quarter this warp may access
    const int lrow = quarter * 32 + lane;           // lane-side row inside the tile
    const T *bias = reinterpret_cast<const T *>(p.bias);
    const T *res = reinterpret_cast<const T *>(p.residual);
    // sequence number of this launch's exchange (the counter is advanced when the grid is done)
    const uint32_t comm_seq = (SWAP && p.comm.world >= 1) ? *reinterpret_cast<volatile unsigned int *>(p.comm.ctl + kCtlEpoch) + 1u : 0u;
    Scheduler<BN, SWAP> sched(p);
    Segment s;
    int acc = 0;
    uint32_t acc_phase = 0, epi_phase = 0;
    bool alive = true;
    // Rendezvous of the 128 epilogue threads with a bounded wait (a plain bar.sync could not
    // be abandoned if one warp had already left on an abort).
    // (Every give-up is made uniform over the warp with a vote before anybody acts on it: a
    // lane that left while the others went on to a warp-synchronous instruction, a shuffle or a
    // tensor-memory load, would leave them waiting for it for ever.)
    auto epi_sync = [&]() {
      mbar_arrive(epi_bar);
      const bool ok = mbar_wait(epi_bar, epi_phase, abort_flag, 5);
      epi_phase ^= 1u;
      return __all_sync(0xffffffffu, ok) != 0;
    };
    // Folded LayerNorm: row statistics of the activations, computed here while the first
    // weight stages are on their way (these warps have nothing else to do yet).  BN / 128 of
    // the epilogue threads share a row; shifted single-pass sums as in the LayerNorm kernel.
    constexpr bool kCanFold = SWAP && BN <= 32;
    float *ln_mean_s = reinterpret_cast<float *>(smem + 640), *ln_rstd_s = ln_mean_s + 32;
    const bool fold = kCanFold && p.ln_colsum != nullptr;
    if (kCanFold && fold) {
      constexpr int tpr = 128 / (kCanFold ? BN : 128);          // threads per row
      const int et = threadIdx.x - 64, r = et / tpr, j = et % tpr;
      float sum = 0.f, sq = 0.f, pivot = 0.f;
      if (r < p.M) {
        const T *xr = reinterpret_cast<const T *>(p.ln_x) + (long long)r * p.ln_ldx;
        pivot = to_f32<T>(__ldcg(xr));
        const int packs = p.K / 8;
#pragma unroll 8
        for (int pk = j; pk < packs; pk += tpr) {
          Vec16<T> a;
          a.raw = __ldcg(reinterpret_cast<const uint4 *>(xr) + pk);
          float f[8];
          a.unpack(f);
#pragma unroll
          for (int e = 0; e < 8; ++e) { const float d = f[e] - pivot; sum += d; sq += d * d; }
        }
      }
#pragma unroll
      for (int o = tpr / 2; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
      }
      if (j == 0) {
        const float inv_k = 1.f / (float)p.K, ms = sum * inv_k;
        ln_mean_s[r] = r < p.M ? pivot + ms : 0.f;
        ln_rstd_s[r] = r < p.M ? rsqrtf(fmaxf(sq * inv_k - ms * ms, 0.f) + p.ln_eps) : 0.f;
      }
      if (!epi_sync()) alive = false;
    }
    while (alive && sched.next(s)) {
      // Swapped orientation: the bias and the residual of this thread's outputs are requested
      // now, all rows at once, so that their latency passes while the tile is still being
      // multiplied; fetched inside the store loop at the end, every load would wait for the
      // store before it (the two may alias), 15 us per launch with a residual.
      constexpr bool kEarlyRes = SWAP && BN <= 32;
      T r_early[kEarlyRes ? BN : 1];
      float b = 0.f, colsum = 0.f;
      // run-time row offset of C (the cache row of a generation step): one load, up front
      const int c_row = (SWAP && p.c_row_offset_dev) ? __ldg(p.c_row_offset_dev) : 0;
      const long long c_extra = (long long)c_row * p.ldc;
      const bool row_ok = row_in_limit(p, c_row);
      if (SWAP) {
        const int n = s.lane_row0 + lrow;
        if (n < p.N) {
          b = fold ? __ldg(p.ln_bias + n) : bias ? to_f32<T>(bias[n]) : 0.f;
          colsum = fold ? __ldg(p.ln_colsum + n) : 0.f;
          if (kEarlyRes && res) {
#pragma unroll
            for (int m = 0; m < (kEarlyRes ? BN : 1); ++m)
              if (m < p.M) r_early[m] = __ldcg(res + (long long)m * p.ldr + n);
          }
        }
      }
      if (kEarlyRes && !res) {                 // always defined: the epilogue adds it unconditionally
#pragma unroll
        for (int m = 0; m < (kEarlyRes ? BN : 1); ++m) r_early[m] = from_f32<T>(0.f);
      }
      // CTAs whose unit range intersects this tile (two divisions: done while the tile is still
      // being multiplied, not between the accumulator and the hand-over)
      int t0 = 0, first_cta = 0, last_cta = 0;
      if (SWAP && s.partial) {
        t0 = s.lane_tile * sched.nsk;
        first_cta = t0 / p.units_per_cta;
        last_cta = (t0 + sched.nsk - 1) / p.units_per_cta;
      }
      if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar + 8 * acc, acc_phase, abort_flag, 4))) break;
      tcgen05_fence_after();
      const uint32_t t_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;

      if (!SWAP && p.rs) {
        // Reduce-scatter mode.  A thread holds one row of the tile, but a store instruction that
        // writes 32 different rows would cross NVLink as 32 small packets: each warp turns 64
        // columns of its 32 rows around in shared memory and writes them as 128-byte row
        // segments (8 lanes x 16 bytes per row, 4 rows per instruction).
        const long long rpr = p.rs_rpr;
        const int owner = (int)(s.lane_row0 / rpr);
        const long long local0 = s.lane_row0 - (long long)owner * rpr + quarter * 32;
        T *dst = reinterpret_cast<T *>(p.comm.bulk[owner] + p.rs_stage_off) + ((long long)p.comm.rank * rpr + local0) * p.N;
        constexpr int kPitch = 72;                           // 64 values + 8 of padding per staged row
        T *stage = reinterpret_cast<T *>(smem + kBarrierBytes + p.stages * ((size_t)kLanes * 128 + (size_t)BN * 128)) +
                   (size_t)quarter * 32 * kPitch;
        const int rows_left = p.M - (s.lane_row0 + quarter * 32);
        for (int c0 = 0; c0 < BN; c0 += 64) {
          const int n_base = s.col_tile * BN + c0;
          if (n_base >= p.N) break;                          // warp-uniform
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            float v[16];
            tmem_ld16(t_base + c0 + cc * 16, v);
            Vec16<T> lo, hi;
            float a[8], b[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { a[j] = v[j]; b[j] = v[8 + j]; }
            lo.pack(a);
            hi.pack(b);
            lo.store(stage + lane * kPitch + cc * 16);
            hi.store(stage + lane * kPitch + cc * 16 + 8);
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int row = it * 4 + (lane >> 3), col = (lane & 7) * 8;
            if (row < rows_left && n_base + col < p.N)
              *reinterpret_cast<uint4 *>(dst + (long long)row * p.N + n_base + col) =
                  *reinterpret_cast<const uint4 *>(stage + row * kPitch + col);
          }
          __syncwarp();
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar + 8 * acc);
      } else if (!SWAP) {
        // One output row per thread, 16 columns at a time.  The bias and residual of a chunk are
        // requested two chunks ahead (their L2 latency was exposed once per chunk, which made a
        // tile's epilogue as long as its main loop), absent operands are zeros, and the
        // activation is chosen once per chunk: these warps are alone on their schedulers.
        const int m = s.lane_row0 + lrow;
        const bool m_ok = m < p.M && row_in_limit(p, p.c_row_offset_dev ? __ldg(p.c_row_offset_dev) : 0);
        const long long c_off = m_ok ? c_row_offset(p, m) : 0;
        const int n_base = s.col_tile * BN;
        const int act = p.act;
        const bool out_f32 = p.out_f32 != 0;
        const T *res_row = (res && m_ok) ? res + (long long)m * p.ldr : nullptr;
        constexpr int kChunks = BN / 16;
        Vec16<T> bq[4][2], rq[4][2];
        auto fetch = [&](int c, int slot) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int n = n_base + c * 16 + h * 8;
            bq[slot][h].raw = make_uint4(0u, 0u, 0u, 0u);
            rq[slot][h].raw = make_uint4(0u, 0u, 0u, 0u);
            if (n < p.N) {
              if (bias) bq[slot][h].load(bias + n);
              if (res_row) rq[slot][h].load(res_row + n);
            }
          }
        };
        fetch(0, 0);
        if (kChunks > 1) fetch(1, 1);
#pragma unroll 1
        for (int c4 = 0; c4 < kChunks; c4 += 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int c = c4 + i;
            const int n0 = n_base + c * 16;
            if (c < kChunks && n0 < p.N) {            // warp-uniform
              if (c + 2 < kChunks) fetch(c + 2, (i + 2) & 3);
              float v[16];
              tmem_ld16(t_base + c * 16, v);
              if (m_ok) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {         // two groups of 8 columns (N is a multiple of 8)
                  const int n = n0 + h * 8;
                  if (n < p.N) {
                    float *vv = v + h * 8;
                    float bf[8], rf[8];
                    bq[i][h].unpack(bf);
                    rq[i][h].unpack(rf);
#pragma unroll
                    for (int j = 0; j < 8; ++j) vv[j] += bf[j];
                    if (act == EB_ACT_RELU) {
#pragma unroll
                      for (int j = 0; j < 8; ++j) vv[j] = fmaxf(vv[j], 0.f);
                    } else if (act != EB_ACT_NONE) {
#pragma unroll
                      for (int j = 0; j < 8; ++j) vv[j] = apply_act(vv[j], act);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) vv[j] += rf[j];
                    if (out_f32) {
                      float4 *o = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.C) + c_off + n);
                      o[0] = make_float4(vv[0], vv[1], vv[2], vv[3]);
                      o[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
                    } else {
                      Vec16<T> o;
                      float tmp[8];
#pragma unroll
                      for (int j = 0; j < 8; ++j) tmp[j] = vv[j];
                      o.pack(tmp);
                      o.store(reinterpret_cast<T *>(p.C) + c_off + n);
                    }
                  }
                }
              }
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar + 8 * acc);
      } else {
        // swapped: this thread owns weight row n, TMEM columns are the batch rows m
        const int n = s.lane_row0 + lrow;
        const bool n_ok = n < p.N;
        float v[BN];
#pragma unroll
        for (int c = 0; c < BN / 16; ++c) tmem_ld16(t_base + c * 16, v + c * 16);
        // the accumulator is in registers: release it before any global traffic
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar + 8 * acc);

        bool do_epilogue = true;
        if (s.partial) {
          float *mine = p.partial + ((size_t)(blockIdx.x * 2 + s.which) * BN) * kLanes;
#pragma unroll
          for (int m = 0; m < BN; ++m)
            if (m < p.M) __stcg(mine + (size_t)m * kLanes + lrow, v[m]);
          {
            // Each warp owns a quarter of the tile's rows in every CTA, so the hand-over is done
            // warp by warp (one counter per tile and quarter): no CTA-wide rendezvous, and the
            // release / acquire ride on the counter update itself.
            __syncwarp();
            int arrived = 0;
            int *counter = p.counters + 4 * s.lane_tile + quarter;
            if (lane == 0) {
              asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(arrived) : "l"(counter) : "memory");
              if (arrived == last_cta - first_cta) *counter = 0;   // ready for the next call
            }
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
            __syncwarp();
            do_epilogue = arrived == last_cta - first_cta;
          }
          if (do_epilogue) {
            // The contributions are added in CTA order, so the sum does not depend on which CTA
            // arrived last; this CTA's own comes from its registers, the others' are read up to
            // kBatch at a time with all their loads in flight together.
            constexpr int kBatch = BN <= 16 ? 4 : (BN <= 32 ? 2 : 1);
            // (for the widest tile the registers do not hold two accumulators: there the own
            // contribution is read back from memory like the others)
            constexpr bool kOwnRegs = BN <= 64;
            const int me = kOwnRegs ? (int)blockIdx.x : -1, n_others = last_cta - first_cta + (kOwnRegs ? 0 : 1);
            float sum_store[kOwnRegs ? BN : 1];
            float *sum = kOwnRegs ? sum_store : v;
            if (!kOwnRegs) {
#pragma unroll
              for (int m = 0; m < BN; ++m) v[m] = 0.f;
            }
#pragma unroll
            for (int m = 0; m < (kOwnRegs ? BN : 1); ++m) sum_store[m] = 0.f;
            bool own_added = !kOwnRegs;
            for (int o0 = 0; o0 < n_others || !own_added; o0 += kBatch) {
              float t[kBatch][BN];
#pragma unroll
              for (int j = 0; j < kBatch; ++j) {
                if (o0 + j < n_others) {
                  const int cta = first_cta + o0 + j + ((kOwnRegs && first_cta + o0 + j >= me) ? 1 : 0);
                  const int which = cta * p.units_per_cta >= t0 ? 0 : 1;   // its range starts inside this tile
                  const float *theirs = p.partial + ((size_t)(cta * 2 + which) * BN) * kLanes;
#pragma unroll
                  for (int m = 0; m < BN; ++m)
                    if (m < p.M) t[j][m] = __ldcg(theirs + (size_t)m * kLanes + lrow);
                }
              }
#pragma unroll
              for (int j = 0; j < kBatch; ++j) {
                if (o0 + j < n_others) {
                  const int cta = first_cta + o0 + j + ((kOwnRegs && first_cta + o0 + j >= me) ? 1 : 0);
                  if (!own_added && cta > me) {
#pragma unroll
                    for (int m = 0; m < BN; ++m) sum[m] += v[m];
                    own_added = true;
                  }
#pragma unroll
                  for (int m = 0; m < BN; ++m)
                    if (m < p.M) sum[m] += t[j][m];
                }
              }
              if (o0 + kBatch >= n_others && !own_added) {
#pragma unroll
                for (int m = 0; m < BN; ++m) sum[m] += v[m];
                own_added = true;
              }
            }
            if (kOwnRegs) {
#pragma unroll
              for (int m = 0; m < BN; ++m) v[m] = sum[m];
            }
          }
        }
        bool lost = false;
        if (do_epilogue && p.comm.world >= 1) {        // (warp-uniform: every lane of the warp is here or none)
          // Fused all-reduce: a thread holds the rank's complete partial products of output
          // column n for every batch row.  They go to every rank (this one included) as flagged
          // lines, rounded to the operand type (what an all-reduce of the product would carry);
          // then the lines of all sources are collected from the local area and added in rank
          // order, so every rank forms the bit-identical sum.  No fence and no rendezvous: a line
          // is valid when it carries this exchange's sequence number.
          const CommDev &cm = p.comm;
          constexpr int kLines = BN / 4;
          const unsigned long long per_src = (unsigned long long)p.N * kLines;            // lines per source
          const unsigned long long half = (comm_seq & 1u) * cm.half_bytes;
          {
            uint32_t packed[BN / 2];
#pragma unroll
            for (int q = 0; q < BN / 8; ++q) {
              Vec16<T> pk;
              float tmp[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) tmp[j] = v[q * 8 + j];
              pk.pack(tmp);
              packed[q * 4 + 0] = pk.raw.x; packed[q * 4 + 1] = pk.raw.y;
              packed[q * 4 + 2] = pk.raw.z; packed[q * 4 + 3] = pk.raw.w;
            }
            if (kLines <= kXposeMaxLines) {
              // The lines of a warp's 32 columns are one contiguous piece of every rank's area,
              // but a thread's own lines lie 16 * kLines bytes from its neighbour's: stored
              // straight from the registers, every 16-byte line was a transaction of its own on
              // NVLink (an exchange among 8 ranks took 16 us, several times what its bytes need).
              // The warp lays its lines out in shared memory and sends them with consecutive
              // lanes writing consecutive lines: 512 contiguous bytes per store instruction.
              unsigned long long *stage = reinterpret_cast<unsigned long long *>(xpose) + (size_t)quarter * (32 * kLines * 2);
              if (n_ok) {
#pragma unroll
                for (int q = 0; q < kLines; ++q) {
                  stage[(lane * kLines + q) * 2] = ((unsigned long long)comm_seq << 32) | packed[2 * q];
                  stage[(lane * kLines + q) * 2 + 1] = ((unsigned long long)comm_seq << 32) | packed[2 * q + 1];
                }
              }
              __syncwarp();
              const int n0 = s.lane_row0 + quarter * 32;                      // the warp's first column
              const int warp_lines = (p.N - n0 < 32 ? (p.N - n0 > 0 ? p.N - n0 : 0) : 32) * kLines;
              const unsigned long long piece = half + ((unsigned long long)cm.rank * per_src + (unsigned long long)n0 * kLines) * 16ull;
              for (int rr = 0; rr < cm.world; ++rr) {
                int r = cm.rank + rr;                                          // every rank starts with another peer
                if (r >= cm.world) r -= cm.world;
#pragma unroll
                for (int it = 0; it < kLines; ++it) {
                  const int c = it * 32 + lane;                                // line c of the warp's piece
                  if (c < warp_lines)
                    asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(cm.recv[r] + piece + (unsigned long long)c * 16ull),
                                 "l"(stage[c * 2]), "l"(stage[c * 2 + 1])
                                 : "memory");
                }
              }
              __syncwarp();
            } else if (n_ok) {
              const unsigned long long mine = half + ((unsigned long long)cm.rank * per_src + (unsigned long long)n * kLines) * 16ull;
              for (int r = 0; r < cm.world; ++r) {
#pragma unroll
                for (int q = 0; q < kLines; ++q) ll_store(cm.recv[r] + mine + q * 16, packed[2 * q], packed[2 * q + 1], comm_seq);
              }
            }
          }
          if (n_ok) {
#pragma unroll
          for (int m = 0; m < BN; ++m) v[m] = 0.f;
          // Collect: the lines of kSrc sources at a time are requested together and their
          // sequence numbers looked at afterwards (a test between two loads would serialise them).
          constexpr int kSrc = kLines <= 4 ? 4 : (kLines <= 8 ? 2 : 1);   // (register budget)
          for (int r0 = 0; r0 < cm.world && !lost; r0 += kSrc) {
            LlLine got[kSrc][kLines];
            const unsigned char *src = cm.recv[cm.rank] + half + ((unsigned long long)r0 * per_src + (unsigned long long)n * kLines) * 16ull;
            unsigned long long t0 = 0;
            for (unsigned it = 0;; ++it) {
              bool all = true;
#pragma unroll
              for (int j = 0; j < kSrc; ++j)
                if (r0 + j < cm.world) {
#pragma unroll
                  for (int q = 0; q < kLines; ++q) got[j][q] = ll_fetch(src + (unsigned long long)j * per_src * 16ull + q * 16);
                }
#pragma unroll
              for (int j = 0; j < kSrc; ++j)
                if (r0 + j < cm.world) {
#pragma unroll
                  for (int q = 0; q < kLines; ++q) all = all && got[j][q].valid(comm_seq);
                }
              if (all) break;
              if ((it & 63u) == 63u) {
                if (t0 == 0) t0 = globaltimer();
                if (*abort_flag || globaltimer() - t0 > cm.wait_budget_ns) {
                  *abort_flag = 1;
                  if (atomicCAS(&g_status[0], 0, EB_ETIMEDOUT) == 0) {
                    g_status[1] = 6; g_status[2] = blockIdx.x; g_status[3] = r0;
                  }
                  lost = true;
                  break;
                }
              }
            }
#pragma unroll
            for (int j = 0; j < kSrc; ++j)
              if (r0 + j < cm.world) {
#pragma unroll
                for (int q = 0; q < kLines; ++q) {
                  const float2 lo = unpack2<T>(got[j][q].d0()), hi = unpack2<T>(got[j][q].d1());
                  v[4 * q] += lo.x; v[4 * q + 1] += lo.y; v[4 * q + 2] += hi.x; v[4 * q + 3] += hi.y;
                }
              }
          }
          }
        }
        // a peer's lines never came: the whole warp leaves together (lanes without a column of
        // their own, beyond N, did not wait and must not be left behind at the next tile)
        if (p.comm.world >= 1 && __any_sync(0xffffffffu, lost)) { alive = false; continue; }
        if (do_epilogue && n_ok && row_ok) {
          // offset of row m of C, advanced row by row (a division per row by the run-time
          // rows-per-batch cost 0.1 us each: 2 us per tile)
          long long row_off = c_extra + n;
          const int rpb = p.c_rows_per_batch;
          const long long batch_step = rpb > 0 ? p.c_batch_stride - (long long)(rpb - 1) * p.ldc : p.ldc;
          int row_in_batch = 0;
          // Straight-line code, 16 rows at a time: all values, the activation chosen once per
          // chunk, the residual, then all stores.  With a single warp per scheduler nothing
          // hides a branch, and a handful of branches per row was a third of a short launch.
          const int rows = p.M;
          const long long ldc = p.ldc;
          const int act = p.act;
          const bool out_f32 = p.out_f32 != 0;
#pragma unroll
          for (int m0 = 0; m0 < BN; m0 += 16) {
            float r[16];
            if (kEarlyRes) {
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = to_f32<T>(r_early[kEarlyRes ? m0 + j : 0]);
            } else {
              T r_late[16];                          // 16 rows of residual in flight together
#pragma unroll
              for (int j = 0; j < 16; ++j) r_late[j] = from_f32<T>(0.f);
              if (res) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  if (m0 + j < rows) r_late[j] = __ldcg(res + (long long)(m0 + j) * p.ldr + n);
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = to_f32<T>(r_late[j]);
            }
            float y[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + j;
              const float rs = (kCanFold && fold) ? ln_rstd_s[m & 31] : 1.f;
              const float mc = (kCanFold && fold) ? ln_mean_s[m & 31] * colsum : 0.f;
              y[j] = rs * (v[m] - mc) + b;
            }
            if (act == EB_ACT_RELU) {
#pragma unroll
              for (int j = 0; j < 16; ++j) y[j] = fmaxf(y[j], 0.f);
            } else if (act != EB_ACT_NONE) {
#pragma unroll
              for (int j = 0; j < 16; ++j) y[j] = apply_act(y[j], act);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) y[j] += r[j];
            if (out_f32) {
              float *c = reinterpret_cast<float *>(p.C);
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (m0 + j < rows) c[row_off] = y[j];
                const bool wrap = ++row_in_batch == rpb;
                row_in_batch = wrap ? 0 : row_in_batch;
                row_off += wrap ? batch_step : ldc;
              }
            } else {
              T *c = reinterpret_cast<T *>(p.C);
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (m0 + j < rows) c[row_off] = from_f32<T>(y[j]);
                const bool wrap = ++row_in_batch == rpb;
                row_in_batch = wrap ? 0 : row_in_batch;
                row_off += wrap ? batch_step : ldc;
              }
            }
          }
        }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (SWAP && p.comm.world >= 1 && threadIdx.x == 0) {
    // the last CTA of the grid advances the exchange's sequence number for the next launch
    unsigned int *ctl = p.comm.ctl;
    const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(ctl + kCtlEpoch) + 1u;
    __threadfence();
    if (atomicAdd(ctl + kCtlBlocks, 1u) == gridDim.x - 1) {
      ctl[kCtlBlocks] = 0u;
      ctl[kCtlEpoch] = seq;
      __threadfence();
    }
  }
  if (*abort_flag) {
    // bounded grace period for copies that may still be in flight to this CTA's shared memory
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

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D map over a row-major [rows, K] 16-bit matrix (row stride ld elements), box 64 x box_rows,
// 128-byte swizzle, out-of-bounds elements read as zero.
int make_map(CUtensorMap *map, const void *base, int dtype, long long rows, long long K, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(EB_ECUDA, "gemm: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == EB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(EB_ECUDA, "gemm: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return EB_OK;
}

// 3-D view of a [rows][K] matrix, K a multiple of 64: (column in k-block, row, k-block); one box
// holds `blocks` consecutive k-blocks of `box_rows` rows, each written as a swizzled tile of
// 128-byte rows like make_map's, the tiles one after the other.
int make_map_blocks(CUtensorMap *map, const void *base, int dtype, long long rows, long long K, long long ld, int box_rows, int blocks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(EB_ECUDA, "gemm: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {(cuuint64_t)kBlockK, (cuuint64_t)rows, (cuuint64_t)(K / kBlockK)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)kBlockK * 2};
  cuuint32_t box[3] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows, (cuuint32_t)blocks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dtype == EB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(EB_ECUDA, "gemm: cuTensorMapEncodeTiled (3-D) failed with CUresult %d", (int)r);
  return EB_OK;
}

template <typename T, int BN, bool SWAP>
int launch(const CUtensorMap &tl, const CUtensorMap &tc, const GemmParams &p, int grid, size_t smem, cudaStream_t st) {
  auto kern = gemm_kernel<T, BN, SWAP>;
  static size_t configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && configured[dev] < smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return fail(EB_ECUDA, "gemm: cannot reserve shared memory");
    }
    configured[dev] = 227 * 1024;
  }
  launch_pdl(kern, dim3(grid), dim3(kThreads), smem, st, tl, tc, p);
  return check_launch("gemm");
}

inline int swap_bn(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128; }

// Stream-K split of the swapped orientation: grid and units (pipeline stages of a tile) per CTA.
// A short K (few stages per tile, the row-parallel GEMMs of a wide tensor-parallel group) is not
// worth cutting: one CTA streams a whole tile in a few microseconds, which is less than the
// partial-sum hand-over of a shared tile costs.
// (Dealing the units evenly over all SMs instead, 148 CTAs rather than the 120-134 that equal
// whole-unit ranges give on the shard shapes of an 8-way group, was measured slower, 2.75 ms per
// generation step against 2.63: more CTAs share a tile, and the last arriver's sum of their
// partial products is on the critical path.  So was a deeper pipeline, 225 KB instead of 200 KB
// of stages: no difference.)
constexpr long long kNoSplitStages = 10;

inline void swap_split(int N, int K, int kpb, int *grid, int *units) {
  const long long tiles = (N + kLanes - 1) / kLanes, kblocks = (K + kBlockK - 1) / kBlockK;
  const long long nsk = (kblocks + kpb - 1) / kpb;
  const long long total = tiles * nsk;
  long long g = sm_count();
  if (nsk <= kNoSplitStages && tiles <= g) {
    *units = (int)nsk;
    *grid = (int)tiles;
    return;
  }
  if (g > total / 2) g = total / 2 > 0 ? total / 2 : 1;   // at least two stages per CTA
  *units = (int)((total + g - 1) / g);
  *grid = (int)((total + *units - 1) / *units);
}

constexpr size_t kCounterBytes = 64 * 1024;   // workspace head: four ints per 128-row tile, zero between calls

#include "gemm_chain.cuh"

template <typename T, int BN>
int launch_chain(const ChainMaps &maps, const ChainParams &p, int grid, size_t smem, cudaStream_t st) {
  auto kern = chain_kernel<T, BN>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return fail(EB_ECUDA, "decode_chain: cannot reserve shared memory");
    }
    configured[dev] = true;
  }
  launch_pdl(kern, dim3(grid), dim3(kThreads), smem, st, maps, p);
  return check_launch("decode_chain");
}

// Workspace of a chain: [4 KB: arrival counters of the operations, then at byte 512 the per-row
// counters of the reductions][kMaxOps x 16 KB tile counters][per operation, in order: the
// stream-K partial sums of a GEMM, or the slice statistics of a reduction].  Every counter sits at an offset that
// does not depend on the operations, so chains of different make-up can share one zero-filled
// workspace: no chain's partial sums ever land on another chain's counters.
constexpr size_t kChainHeadBytes = 4096, kChainTileCounterBytes = 16384, kChainStatsBytes = 8192;
constexpr size_t kChainPartialOffset = kChainHeadBytes + kMaxOps * kChainTileCounterBytes;

inline size_t chain_op_bytes(int grid, int bn) { return (size_t)grid * 2 * bn * kLanes * sizeof(float); }

}  // namespace
}  // namespace eb

using namespace eb;

extern "C" size_t eb_decode_chain_workspace_bytes(const eb_chain_op *ops, int n_ops, int M) {
  if (!ops || n_ops <= 0 || n_ops > kMaxOps || M <= 0 || M > kLanes) return 0;
  size_t total = kChainPartialOffset;
  for (int i = 0; i < n_ops; ++i) {
    if (ops[i].type == EB_OP_GEMM) total += chain_op_bytes(sm_count(), swap_bn(M));
    if (ops[i].type == EB_OP_REDUCE_LAYERNORM) total += kChainStatsBytes;
  }
  return total;
}

extern "C" int eb_decode_chain(const eb_chain_op *ops, int n_ops, int M, int dtype, void *workspace,
                               size_t workspace_bytes, eb_comm *comm, void *stream) {
  EB_REQUIRE(ops && n_ops >= 1 && n_ops <= kMaxOps, "decode_chain: 1..%d operations", kMaxOps);
  EB_REQUIRE(dtype == EB_F16 || dtype == EB_BF16, "decode_chain: fp16 or bf16 only");
  EB_REQUIRE(M >= 1 && M <= kLanes, "decode_chain: M must be in [1, 128] (got %d)", M);
  const int grid = sm_count();
  EB_REQUIRE(M <= grid, "decode_chain: M exceeds the number of SMs");
  const size_t need = eb_decode_chain_workspace_bytes(ops, n_ops, M);
  EB_REQUIRE(workspace && aligned16(workspace) && workspace_bytes >= need,
             "decode_chain: needs a workspace of %zu bytes, zero-filled once", need);
  const int bn = swap_bn(M);
  ChainParams p{};
  ChainMaps maps;
  p.n_ops = n_ops; p.M = M;
  p.prefetch = 8;
  p.kpb = bn <= 32 ? 2 : 1;
  // shared memory: [1 KB barriers][ring of stages][staging area of the exchange: 4 warps x BN rows x 32 values]
  const size_t stage_bytes = ((size_t)kLanes * 128 + (size_t)bn * 128) * p.kpb;
  const size_t xpose_bytes = (size_t)bn * 256;
  int stages = (int)((200 * 1024 - kBarrierBytes - 1024 - xpose_bytes) / stage_bytes);
  p.stages = stages > kMaxStages ? kMaxStages : (stages < 2 ? 2 : stages);
  p.xpose_off = (uint32_t)(p.stages * stage_bytes);
  const size_t smem = kBarrierBytes + 1024 + (size_t)p.stages * stage_bytes + xpose_bytes;
  p.done = reinterpret_cast<int *>(workspace);
  char *cursor = reinterpret_cast<char *>(workspace) + kChainPartialOffset;
  int rc;
  bool any_gemm = false;
  int pending_exchange = -1;            // index of the exchange a kReduceLn must follow
  for (int i = 0; i < n_ops; ++i) {
    const eb_chain_op &o = ops[i];
    if (o.type == EB_OP_GEMM) {
      any_gemm = true;
      EB_REQUIRE(pending_exchange < 0, "decode_chain: op %d: the exchange of op %d must be followed by EB_OP_REDUCE_LAYERNORM", i, i - 1);
      EB_REQUIRE(o.A && o.W, "decode_chain: op %d: null GEMM operand", i);
      EB_REQUIRE(o.N > 0 && o.K >= 8 && o.K % 8 == 0, "decode_chain: op %d: K must be a positive multiple of 8", i);
      EB_REQUIRE(o.lda >= o.K && o.ldw >= o.K && o.lda % 8 == 0 && o.ldw % 8 == 0, "decode_chain: op %d: bad leading dimensions", i);
      EB_REQUIRE(aligned16(o.A) && aligned16(o.W), "decode_chain: op %d: pointers must be 16-byte aligned", i);
      ChainGemm &g = p.g[i];
      p.type[i] = kOpGemm;
      g.N = o.N; g.K = o.K;
      g.kblocks = (o.K + kBlockK - 1) / kBlockK;
      g.nsk = (g.kblocks + p.kpb - 1) / p.kpb;
      g.tiles = (o.N + kLanes - 1) / kLanes;
      const long long total = (long long)g.tiles * g.nsk;
      EB_REQUIRE(total < (1ll << 30), "decode_chain: op %d too large", i);
      g.units_per_cta = (g.nsk <= kNoSplitStages && g.tiles <= grid) ? g.nsk : (int)((total + grid - 1) / grid);
      g.exchange = -1;
      if (o.exchange) {
        EB_REQUIRE(comm, "decode_chain: op %d exchanges its product: a context is needed", i);
        EB_REQUIRE(!o.bias && !o.residual && o.act == EB_ACT_NONE, "decode_chain: op %d: bias, residual and activation belong to the reduction that follows an exchange", i);
        EB_REQUIRE(o.N % 8 == 0, "decode_chain: op %d: an exchanged product needs N to be a multiple of 8", i);
        EB_REQUIRE(comm_exchange_bytes(comm->world, M, o.N) <= comm->recv_bytes / 2,
                   "decode_chain: op %d: %d x %d from %d ranks does not fit half of the receive area (%zu bytes)", i, M, o.N,
                   comm->world, comm->recv_bytes / 2);
        g.exchange = p.n_exchanges++;
        pending_exchange = g.exchange;
      } else {
        EB_REQUIRE(o.C && aligned16(o.C) && o.ldc >= o.N, "decode_chain: op %d: bad output", i);
        EB_REQUIRE(!o.residual || (o.ldr >= o.N && o.ldr % 8 == 0), "decode_chain: op %d: bad residual stride", i);
        EB_REQUIRE(o.out_dtype == dtype || o.out_dtype == EB_F32, "decode_chain: op %d: bad output type", i);
        EB_REQUIRE(o.act >= EB_ACT_NONE && o.act <= EB_ACT_GELU_ERF, "decode_chain: op %d: unknown activation", i);
      }
      g.C = o.C; g.ldc = o.ldc; g.c_rows_per_batch = o.c_rows_per_batch; g.c_batch_stride = o.c_batch_stride;
      g.c_row_offset_dev = o.c_row_offset_device; g.c_row_limit = o.c_row_offset_limit;
      g.bias = o.bias; g.residual = o.residual; g.ldr = o.ldr; g.act = o.act; g.out_f32 = o.out_dtype == EB_F32;
      EB_REQUIRE((size_t)g.tiles * sizeof(int) <= kChainTileCounterBytes, "decode_chain: op %d: N too large", i);
      g.counters = reinterpret_cast<int *>(reinterpret_cast<char *>(workspace) + kChainHeadBytes + i * kChainTileCounterBytes);
      g.partial = reinterpret_cast<float *>(cursor);
      cursor += chain_op_bytes(grid, bn);
      if ((rc = make_map(&maps.w[i], o.W, dtype, o.N, o.K, o.ldw, kLanes))) return rc;
      if ((rc = make_map(&maps.x[i], o.A, dtype, M, o.K, o.lda, bn))) return rc;
    } else if (o.type == EB_OP_LAYERNORM) {
      EB_REQUIRE(pending_exchange < 0, "decode_chain: op %d: the exchange of op %d must be followed by EB_OP_REDUCE_LAYERNORM", i, i - 1);
      EB_REQUIRE(o.x && o.y && o.gamma && o.beta && o.n2 > 0 && o.n2 % 8 == 0, "decode_chain: op %d: bad LayerNorm operands", i);
      EB_REQUIRE(aligned16(o.x) && aligned16(o.y) && aligned16(o.gamma) && aligned16(o.beta),
                 "decode_chain: op %d: pointers must be 16-byte aligned", i);
      p.type[i] = kOpLayerNorm;
      ChainLn &l = p.l[i];
      l = ChainLn{};
      l.x = o.x; l.gamma = o.gamma; l.beta = o.beta; l.y = o.y; l.n2 = o.n2; l.eps = (float)o.eps;
    } else if (o.type == EB_OP_REDUCE_LAYERNORM) {
      EB_REQUIRE(pending_exchange >= 0 && i > 0 && ops[i - 1].type == EB_OP_GEMM && ops[i - 1].N == o.n2,
                 "decode_chain: op %d: a reduction follows the exchanged GEMM whose N equals its n2", i);
      EB_REQUIRE(o.C && aligned16(o.C) && o.ldc >= o.n2 && o.ldc % 8 == 0, "decode_chain: op %d: bad sum output", i);
      EB_REQUIRE(!o.residual || (aligned16(o.residual) && o.ldr >= o.n2 && o.ldr % 8 == 0), "decode_chain: op %d: bad residual", i);
      EB_REQUIRE(aligned16(o.bias), "decode_chain: op %d: misaligned bias", i);
      EB_REQUIRE(!o.gamma || (o.beta && o.y && aligned16(o.y) && aligned16(o.gamma) && aligned16(o.beta)),
                 "decode_chain: op %d: bad LayerNorm operands", i);
      p.type[i] = kOpReduceLn;
      ChainLn &l = p.l[i];
      l = ChainLn{};
      l.gamma = o.gamma; l.beta = o.beta; l.y = o.y; l.n2 = o.n2; l.eps = (float)o.eps;
      l.bias = o.bias; l.residual = o.residual; l.ldr = o.ldr; l.sum_out = o.C; l.ld_sum = o.ldc;
      l.exchange = pending_exchange;
      // column slices per row: as many CTAs as the grid spares, at most eight
      l.split = grid / M >= 8 ? 8 : grid / M >= 4 ? 4 : grid / M >= 2 ? 2 : 1;
      l.rowdone = reinterpret_cast<int *>(reinterpret_cast<char *>(workspace) + 512) + pending_exchange * kLanes;
      l.stats = reinterpret_cast<float2 *>(cursor);          // [128 rows][8 slices], needs no initialisation
      cursor += kChainStatsBytes;
      EB_REQUIRE(pending_exchange < 7, "decode_chain: too many exchanges in one chain");
      pending_exchange = -1;
    } else {
      return fail(EB_EINVAL, "decode_chain: op %d: unknown type %d", i, o.type);
    }
  }
  EB_REQUIRE(pending_exchange < 0, "decode_chain: the last operation exchanges its product but nothing reduces it");
  EB_REQUIRE(any_gemm, "decode_chain: a chain needs at least one GEMM");
  if (p.n_exchanges > 0) {
    int dev = -1;
    cudaGetDevice(&dev);
    EB_REQUIRE(comm->connected && comm->device == dev, "decode_chain: the context is not connected or belongs to another device");
    p.comm = comm_dev(comm);
  }
  cudaStream_t st = as_stream(stream);
#define EB_CHAIN(BN) (dtype == EB_F16 ? launch_chain<__half, BN>(maps, p, grid, smem, st) \
                                      : launch_chain<__nv_bfloat16, BN>(maps, p, grid, smem, st))
  if (bn == 16) return EB_CHAIN(16);
  if (bn == 32) return EB_CHAIN(32);
  if (bn == 64) return EB_CHAIN(64);
  return EB_CHAIN(128);
#undef EB_CHAIN
}

extern "C" size_t eb_gemm_workspace_bytes(int M, int N, int K) {
  if (M > kLanes || M <= 0 || N <= 0 || K <= 0) return 0;
  // the partials are sized for the largest grid (one CTA per SM)
  return kCounterBytes + (size_t)sm_count() * 2 * swap_bn(M) * kLanes * sizeof(float);
}

namespace eb {
int attention_tc_status(int *out4, bool clear);   // attention_tc.cu
}

extern "C" int eb_device_status(int *out4, int clear) {
  int host[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(host, g_status, sizeof(host)) != cudaSuccess) {
    cudaGetLastError();
    return fail(EB_ECUDA, "device_status: cannot read the status word");
  }
  // the tensor-core attention kernel keeps its own words; "where" codes 100+ are its waits
  int attn[4] = {0, 0, 0, 0};
  if (eb::attention_tc_status(attn, clear != 0) != EB_OK) return fail(EB_ECUDA, "device_status: cannot read the status word");
  if (clear && host[0] != 0) {
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_status, zero, sizeof(zero));
  }
  if (host[0] == 0 && attn[0] != 0) {
    for (int i = 0; i < 4; ++i) host[i] = attn[i];
    host[1] += 100;
  }
  if (out4)
    for (int i = 0; i < 4; ++i) out4[i] = host[i];
  return EB_OK;
}

static int gemm_impl(const void *A, long long lda, const void *W, long long ldw, void *C, long long ldc,
                     const void *bias, const void *residual, long long ldr, int M, int N, int K, int dtype,
                     int out_dtype, int act, int c_rows_per_batch, long long c_batch_stride,
                     const int32_t *c_row_offset_device, int c_row_offset_limit, int flags, void *workspace,
                     size_t workspace_bytes, void *stream, const eb_comm *comm, const float *ln_colsum = nullptr,
                     const float *ln_bias = nullptr, double ln_eps = 0.0, bool reduce_scatter = false,
                     size_t rs_stage_offset = 0) {
  EB_REQUIRE(dtype == EB_F16 || dtype == EB_BF16, "gemm: operands must be fp16 or bf16 (got dtype %d)", dtype);
  if (ln_colsum || ln_bias) {
    EB_REQUIRE(ln_colsum && ln_bias, "gemm_ln: ln_colsum and ln_bias go together");
    EB_REQUIRE(M <= 32, "gemm_ln: the folded LayerNorm serves M <= 32 rows (got %d)", M);
    EB_REQUIRE(!bias, "gemm_ln: the bias is part of ln_bias");
    EB_REQUIRE(ln_eps > 0.0, "gemm_ln: eps must be positive");
    EB_REQUIRE(((uintptr_t)ln_colsum % 4 == 0) && ((uintptr_t)ln_bias % 4 == 0), "gemm_ln: misaligned fp32 vectors");
  }
  EB_REQUIRE(out_dtype == dtype || out_dtype == EB_F32, "gemm: output must be the input type or fp32");
  EB_REQUIRE(M >= 0 && N >= 0 && K >= 0, "gemm: negative size");
  EB_REQUIRE(act >= EB_ACT_NONE && act <= EB_ACT_GELU_ERF, "gemm: unknown activation %d", act);
  EB_REQUIRE((flags & ~EB_GEMM_STATIC_W) == 0, "gemm: unknown flag bits 0x%x", flags);
  if (M == 0 || N == 0) return EB_OK;
  EB_REQUIRE(A && W && (C || reduce_scatter), "gemm: null operand");
  // the generation orientation (M <= 128) writes C one element at a time: any N will do there
  EB_REQUIRE(K >= 8 && K % 8 == 0 && (N % 8 == 0 || M <= kLanes), "gemm: K, and N for M > 128, must be positive multiples of 8 (K=%d N=%d)", K, N);
  EB_REQUIRE(lda >= K && ldw >= K && lda % 8 == 0 && ldw % 8 == 0, "gemm: lda/ldw must be multiples of 8 and >= K");
  EB_REQUIRE(ldc >= N && (ldc % 8 == 0 || M <= kLanes) && (!residual || (ldr >= N && (ldr % 8 == 0 || M <= kLanes))),
             "gemm: ldc/ldr must be >= N (and multiples of 8 for M > 128)");
  EB_REQUIRE(c_rows_per_batch >= 0 && (c_rows_per_batch == 0 || c_batch_stride % 8 == 0 || M <= kLanes), "gemm: bad batch mapping of C");
  EB_REQUIRE(c_row_offset_limit >= 0, "gemm: negative row-offset limit");
  EB_REQUIRE(aligned16(A) && aligned16(W) && aligned16(C) && aligned16(bias) && aligned16(residual),
             "gemm: pointers must be 16-byte aligned");
  cudaStream_t st = as_stream(stream);

  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.kblocks = (K + kBlockK - 1) / kBlockK;
  p.C = C; p.ldc = ldc; p.c_rows_per_batch = c_rows_per_batch; p.c_batch_stride = c_batch_stride;
  p.c_row_offset_dev = c_row_offset_device; p.c_row_limit = c_row_offset_limit;
  p.static_w = (flags & EB_GEMM_STATIC_W) ? 1 : 0;
  p.ln_colsum = ln_colsum; p.ln_bias = ln_bias; p.ln_x = A; p.ln_ldx = lda; p.ln_eps = (float)ln_eps;
  if (reduce_scatter) {
    int dev = -1;
    cudaGetDevice(&dev);
    EB_REQUIRE(comm && comm->connected && comm->device == dev, "gemm_reduce_scatter: the context is not connected or belongs to another device");
    EB_REQUIRE(M > kLanes, "gemm_reduce_scatter: serves M > 128 (smaller products use eb_gemm_allreduce)");
    EB_REQUIRE(!bias && !residual && act == EB_ACT_NONE && out_dtype == dtype,
               "gemm_reduce_scatter: bias, residual and activation belong to eb_reduce_broadcast");
    p.rs = 1;
    p.rs_rpr = comm_rows_per_rank(M, comm->world);
    p.rs_stage_off = rs_stage_offset;
    const size_t need = (size_t)comm->world * p.rs_rpr * N * 2;
    EB_REQUIRE(rs_stage_offset % 256 == 0, "gemm_reduce_scatter: the staging offset must be a multiple of 256");
    if (rs_stage_offset + need > comm->bulk_bytes)
      return fail(EB_ELIMIT, "gemm_reduce_scatter: %d x %d from %d ranks needs %zu bytes of the bulk region at offset %zu, which has %zu",
                  M, N, comm->world, need, rs_stage_offset, comm->bulk_bytes);
    p.comm = comm_dev(comm);
  } else if (comm) {
    int dev = -1;
    cudaGetDevice(&dev);
    EB_REQUIRE(comm->connected && comm->device == dev, "gemm_allreduce: the context is not connected or belongs to another device");
    EB_REQUIRE(M <= kLanes, "gemm_allreduce: the fused exchange serves M <= 128 only (M=%d)", M);
    EB_REQUIRE(N % 4 == 0, "gemm_allreduce: N must be a multiple of 4");
    EB_REQUIRE(comm_exchange_bytes(comm->world, swap_bn(M), N) <= comm->recv_bytes / 2,
               "gemm_allreduce: %d x %d from %d ranks does not fit half of the receive area (%zu bytes)", swap_bn(M), N,
               comm->world, comm->recv_bytes / 2);
    p.comm = comm_dev(comm);
  }
  p.bias = bias; p.residual = residual; p.ldr = ldr; p.act = act; p.out_f32 = out_dtype == EB_F32 && dtype != EB_F32;

  CUtensorMap tl, tc;
  int rc;
  if (M <= kLanes) {
    // swapped orientation: lanes = rows of W, columns = rows of A
    const int bn = swap_bn(M);
    int grid;
    // k-blocks per stage: stages of about 36 KB keep the hand-over count per byte low
    const size_t sub_bytes = (size_t)kLanes * 128 + (size_t)bn * 128;
    p.kpb = bn <= 32 ? 2 : 1;
    const size_t stage_bytes = sub_bytes * p.kpb;
    EB_REQUIRE((long long)((N + kLanes - 1) / kLanes) * ((K + kBlockK - 1) / kBlockK) < (1ll << 30), "gemm: N*K too large");
    swap_split(N, K, p.kpb, &grid, &p.units_per_cta);
    const size_t budget = (size_t)200 * 1024;
    // a fused exchange of up to 32 batch rows stages its outgoing lines per epilogue warp: 4 x 32 x (bn / 4) x 16 bytes
    const size_t xpose_bytes = (p.comm.world >= 1 && bn / 4 <= kXposeMaxLines) ? (size_t)512 * bn : 0;
    const size_t fixed = kBarrierBytes + 1024 + xpose_bytes;        // barriers, alignment, exchange staging
    int stages = (int)((budget - fixed) / stage_bytes);
    stages = stages > kMaxStages ? kMaxStages : (stages < 2 ? 2 : stages);
    p.stages = stages;
    const size_t smem = fixed + (size_t)stages * stage_bytes;
    const size_t tiles = (N + kLanes - 1) / kLanes;
    EB_REQUIRE(tiles * 4 * sizeof(int) <= kCounterBytes, "gemm: N=%d exceeds the decode path's tile-counter capacity", N);
    // The counters sit at a fixed place (the head of the workspace) so that calls of any
    // shape find them zero; the partials behind them need no initialisation.
    const size_t need = kCounterBytes + (size_t)grid * 2 * bn * kLanes * sizeof(float);
    EB_REQUIRE(workspace && workspace_bytes >= need && aligned16(workspace),
               "gemm: M=%d needs a workspace of %zu bytes, zero-filled once (eb_gemm_workspace_bytes)", M, need);
    p.counters = reinterpret_cast<int *>(workspace);
    p.partial = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + kCounterBytes);
    p.lane_rows = N; p.col_rows = M;
    if ((rc = make_map(&tl, W, dtype, N, K, ldw, kLanes))) return rc;
    p.x3d = (K % kBlockK == 0 && p.kpb > 1) ? 1 : 0;
    if (p.x3d) {
      if ((rc = make_map_blocks(&tc, A, dtype, M, K, lda, bn, p.kpb))) return rc;
    } else if ((rc = make_map(&tc, A, dtype, M, K, lda, bn))) {
      return rc;
    }
#define EB_SWAP(BN)                                                                             \
  (dtype == EB_F16 ? launch<__half, BN, true>(tl, tc, p, grid, smem, st)                        \
                   : launch<__nv_bfloat16, BN, true>(tl, tc, p, grid, smem, st))
    if (bn == 16) return EB_SWAP(16);
    if (bn == 32) return EB_SWAP(32);
    if (bn == 64) return EB_SWAP(64);
    return EB_SWAP(128);
#undef EB_SWAP
  }
  p.lane_rows = M; p.col_rows = N;
  const long long lane_tiles = (M + kLanes - 1) / kLanes;
  const bool wide = lane_tiles * ((N + 255) / 256) >= sm_count();   // enough 128x256 tiles to fill the machine
  const int bn = wide ? 256 : 128;
  const long long tiles = lane_tiles * ((N + bn - 1) / bn);
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  p.stages = wide ? 4 : 6;
  p.kpb = 1;
  // (+ 18 KB behind the stages: the staging rows of the reduce-scatter epilogue)
  const size_t smem = kBarrierBytes + 1024 + (size_t)p.stages * (kLanes * 128 + bn * 128) + (p.rs ? 4 * 32 * 72 * 2 : 0);
  if ((rc = make_map(&tl, A, dtype, M, K, lda, kLanes))) return rc;
  if ((rc = make_map(&tc, W, dtype, N, K, ldw, bn))) return rc;
  if (bn == 256)
    return dtype == EB_F16 ? launch<__half, 256, false>(tl, tc, p, grid, smem, st)
                           : launch<__nv_bfloat16, 256, false>(tl, tc, p, grid, smem, st);
  return dtype == EB_F16 ? launch<__half, 128, false>(tl, tc, p, grid, smem, st)
                         : launch<__nv_bfloat16, 128, false>(tl, tc, p, grid, smem, st);
}

extern "C" int eb_gemm(const void *A, long long lda, const void *W, long long ldw, void *C, long long ldc,
                       const void *bias, const void *residual, long long ldr, int M, int N, int K, int dtype,
                       int out_dtype, int act, int c_rows_per_batch, long long c_batch_stride,
                       const int32_t *c_row_offset_device, int c_row_offset_limit, int flags, void *workspace,
                       size_t workspace_bytes, void *stream) {
  return gemm_impl(A, lda, W, ldw, C, ldc, bias, residual, ldr, M, N, K, dtype, out_dtype, act, c_rows_per_batch,
                   c_batch_stride, c_row_offset_device, c_row_offset_limit, flags, workspace, workspace_bytes, stream,
                   nullptr);
}

extern "C" int eb_gemm_ln(const void *A, long long lda, const void *W, long long ldw, void *C, long long ldc,
                          const float *ln_colsum, const float *ln_bias, double eps, const void *residual,
                          long long ldr, int M, int N, int K, int dtype, int out_dtype, int act,
                          int c_rows_per_batch, long long c_batch_stride, const int32_t *c_row_offset_device,
                          int c_row_offset_limit, int flags, void *workspace, size_t workspace_bytes, void *stream) {
  EB_REQUIRE(ln_colsum && ln_bias, "gemm_ln: ln_colsum and ln_bias are required");
  return gemm_impl(A, lda, W, ldw, C, ldc, nullptr, residual, ldr, M, N, K, dtype, out_dtype, act, c_rows_per_batch,
                   c_batch_stride, c_row_offset_device, c_row_offset_limit, flags, workspace, workspace_bytes, stream,
                   nullptr, ln_colsum, ln_bias, eps);
}

extern "C" int eb_gemm_allreduce(const void *A, long long lda, const void *W, long long ldw, void *C, long long ldc,
                                 const void *bias, const void *residual, long long ldr, int M, int N, int K,
                                 int dtype, int out_dtype, int act, int c_rows_per_batch, long long c_batch_stride,
                                 const int32_t *c_row_offset_device, int c_row_offset_limit, int flags,
                                 void *workspace, size_t workspace_bytes, eb_comm *comm, void *stream) {
  EB_REQUIRE(comm, "gemm_allreduce: null context");
  return gemm_impl(A, lda, W, ldw, C, ldc, bias, residual, ldr, M, N, K, dtype, out_dtype, act, c_rows_per_batch,
                   c_batch_stride, c_row_offset_device, c_row_offset_limit, flags, workspace, workspace_bytes, stream,
                   comm);
}

extern "C" int eb_gemm_reduce_scatter(const void *A, long long lda, const void *W, long long ldw, int M, int N, int K,
                                      int dtype, int flags, eb_comm *comm, size_t stage_offset, void *stream) {
  EB_REQUIRE(comm, "gemm_reduce_scatter: null context");
  return gemm_impl(A, lda, W, ldw, nullptr, N, nullptr, nullptr, 0, M, N, K, dtype, dtype, EB_ACT_NONE, 0, 0, nullptr, 0,
                   flags, nullptr, 0, stream, comm, nullptr, nullptr, 0.0, true, stage_offset);
}
