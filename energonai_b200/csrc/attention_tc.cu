// Prompt-pass attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
//   out[b,i,h,:] = softmax_j( scale * q[b,i,h,:].k[b,j,h,:] + mask[b,j] ; causal ) . v[b,j,h,:]
// (energonai/model/attention.py:105-124, without materialising the score tensor).
//
// One CTA owns 128 query rows of one (sequence, head) and walks the visible keys in tiles of
// 128.  Both products run on tcgen05.mma with fp32 accumulators in tensor memory:
//   S  = Q . K_tile^T    (128 x 128, K = head_dim)   TMEM columns [0, 128) and [128, 256), alternating
//   PV = P . V_tile      (128 x head_dim, K = 128)    TMEM columns [256, 256 + head_dim)
// Q and the K tiles arrive by TMA (3-D maps over the [batch][row][head*dim] views, 128-byte
// swizzle, rows beyond the sequence read as zeros).  The second product needs its B operand with
// the contraction index (keys) contiguous, i.e. V transposed: a small kernel writes
// vT[b][h][d][key] once per call into caller-provided scratch, and the V tiles are TMA boxes of
// that.  Warp roles (192 threads): warp 0 issues TMA, warp 1 issues the MMAs, warps 2-5 are
// the softmax: thread r owns query row r, reads its score row from TMEM (tcgen05.ld), keeps the
// running maximum / sum (fp32, log2 domain), writes the probabilities as the 16-bit, swizzled A
// operand of the second product into shared memory, and accumulates the output row in
// registers (O = O * alpha + PV, PV read back from TMEM), so nothing in TMEM needs rescaling.
// The score accumulator is double-buffered: S of tile j+1 is computed while the softmax warps
// still work on tile j, so they never wait for the first product.
//
// Every mbarrier wait is bounded; a wait that runs out is recorded, the CTA's roles leave (each
// decision made uniform over the warp first), copies in flight are given time to land, TMEM is
// freed and the kernel returns.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"

namespace eb {
namespace {

constexpr int kRows = 128;                 // query rows per CTA = UMMA M = TMEM lanes
constexpr int kKeys = 128;                 // keys per tile
constexpr int kTcThreads = 192;
constexpr float kLog2eTc = 1.4426950408889634f;
constexpr unsigned long long kTcWaitNs = 1000ull * 1000ull * 1000ull;

__device__ int g_tc_status[4];             // [0] code, [1] where, [2] block, [3] detail

struct TcParams {
  int B, H, Sq, Sk, causal;
  int mask_vec;                            // mask rows start on 16-byte boundaries
  float scale_log2;                        // scale * log2(e)
  const void *mask;                        // additive [B][>= Sk] in T, or null
  long long mask_bs;
  void *o;
  long long o_bs, o_rs;
};

// ---- PTX wrappers (the same forms the GEMM uses) ----------------------------------------------
__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
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
__device__ __noinline__ bool bar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int where) {
  const unsigned long long t0 = gtimer();
  for (unsigned it = 1;; ++it) {
    if (bar_try(bar, parity)) return true;
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      if (gtimer() - t0 > kTcWaitNs) {
        *abort_flag = 1;
        if (atomicCAS(&g_tc_status[0], 0, EB_ETIMEDOUT) == 0) {
          g_tc_status[1] = where;
          g_tc_status[2] = blockIdx.x;
          g_tc_status[3] = (int)parity;
        }
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int where) {
  if (bar_try(bar, parity)) return true;
  return bar_wait_slow(bar, parity, abort_flag, where);
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float *v) {
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
// K-major tile of 128-byte rows with the 128-byte swizzle; 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// kind::f16, fp32 accumulate, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t tc_idesc(int n, int is_bf16) {
  return (1u << 4) | ((uint32_t)is_bf16 << 7) | ((uint32_t)is_bf16 << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
}

// Scores of 16 consecutive keys -> logits in the log2 domain: scale, additive mask, -inf for
// keys this row does not see (behind the diagonal or beyond the sequence).
template <typename T>
__device__ __forceinline__ void tile_logits(float (&x)[16], const T *mrow, bool vec, int kbase, int Sk, int vis_end, float scale_log2) {
  float mf[16];
  if (mrow && vec && kbase + 16 <= Sk) {
    Vec16<T> m0, m1;
    m0.load(mrow + kbase);
    m1.load(mrow + kbase + 8);
    float t0[8], t1[8];
    m0.unpack(t0);
    m1.unpack(t1);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      mf[e] = t0[e];
      mf[8 + e] = t1[e];
    }
  } else {
#pragma unroll
    for (int e = 0; e < 16; ++e) mf[e] = (mrow && kbase + e < Sk) ? to_f32<T>(mrow[kbase + e]) : 0.f;
  }
#pragma unroll
  for (int e = 0; e < 16; ++e) x[e] = kbase + e < vis_end ? x[e] * scale_log2 + mf[e] * kLog2eTc : -INFINITY;
}

// ---- V transposed: vT[b][h][d][key] --------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) transpose_v_kernel(const T *__restrict__ v, T *__restrict__ vt, long long v_bs, long long v_rs,
                                                          int H, int D, int Sk, int Skp) {
  __shared__ T tile[64][66];
  griddep_wait();
  griddep_launch();
  const int b = blockIdx.z, col0 = blockIdx.y * 64, key0 = blockIdx.x * 64;     // col = h*D + d
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int r = ty; r < 64; r += 4) {
    const int key = key0 + r;
    tile[r][tx] = key < Sk ? v[b * v_bs + (long long)key * v_rs + col0 + tx] : from_f32<T>(0.f);
  }
  __syncthreads();
  for (int r = ty; r < 64; r += 4) {
    const int col = col0 + r, key = key0 + tx;
    if (key < Skp) vt[((long long)b * H * D + col) * Skp + key] = tile[tx][r];
  }
}

// ---- the attention kernel ----------------------------------------------------------------------
// Shared memory (1024-aligned): [1 KB barriers, TMEM slot, abort flag][Q: D/64 sub-tiles of
// 128 rows x 128 B][2 stages x (K: D/64 sub-tiles | VT: 2 sub-tiles of D rows x 128 B)]
// [P: 2 sub-tiles of 128 rows x 128 B].
template <typename T, int D>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                            const __grid_constant__ CUtensorMap tm_vt, const TcParams p) {
  constexpr int kSub = D / 64;                                   // 64-column sub-tiles of Q / K
  constexpr uint32_t kQBytes = kSub * kRows * 128, kKBytes = kSub * kKeys * 128, kVBytes = 2 * D * 128;
  constexpr uint32_t kStageBytes = kKBytes + kVBytes;
  constexpr uint32_t kTmemCols = 512, kPvCol = 2 * kKeys;
  constexpr int kBf16 = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t kIdescS = tc_idesc(kKeys, kBf16), kIdescPV = tc_idesc(D, kBf16);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = s32(smem_raw);
  uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
  const uint32_t bar0 = s32(bars);
  const uint32_t q_full = bar0, kv_full = bar0 + 8, kv_empty = bar0 + 24, s_full = bar0 + 40, s_free = bar0 + 56,
                 p_full = bar0 + 72, pv_full = bar0 + 80, pv_free = bar0 + 88;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 128);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 136);
  const uint32_t q_addr = s32(smem) + 1024, kv_addr = q_addr + kQBytes, p_addr = kv_addr + 2 * kStageBytes;
  uint8_t *p_ptr = smem + 1024 + kQBytes + 2 * kStageBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;   // longest (latest, under the causal mask) tiles first
  const int q0 = qt * kRows, shift = p.Sk - p.Sq;
  // keys any row of this CTA may see: all of them, or up to the last row's diagonal
  const int last_key = p.causal ? min(p.Sk - 1, q0 + kRows - 1 + shift) : p.Sk - 1;
  const int ntiles = last_key >= 0 ? last_key / kKeys + 1 : 0;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_vt) : "memory");
    bar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      bar_init(kv_full + 8 * s, 1);
      bar_init(kv_empty + 8 * s, 1);
      bar_init(s_full + 8 * s, 1);
      bar_init(s_free + 8 * s, 4);
    }
    bar_init(p_full, 4);
    bar_init(pv_full, 1);
    bar_init(pv_free, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  griddep_launch();
  griddep_wait();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && ntiles > 0) {
      bar_expect_tx(q_full, kQBytes);
#pragma unroll
      for (int kb = 0; kb < kSub; ++kb) tma_load_3d(q_addr + kb * kRows * 128, &tm_q, q_full, h * D + kb * 64, q0, b);
      for (int j = 0; j < ntiles; ++j) {
        const int s = j & 1;
        if (j >= 2 && !bar_wait(kv_empty + 8 * s, ((j >> 1) - 1) & 1, abort_flag, 1)) break;
        const uint32_t dst = kv_addr + s * kStageBytes;
        bar_expect_tx(kv_full + 8 * s, kStageBytes);
#pragma unroll
        for (int kb = 0; kb < kSub; ++kb) tma_load_3d(dst + kb * kKeys * 128, &tm_k, kv_full + 8 * s, h * D + kb * 64, j * kKeys, b);
#pragma unroll
        for (int a = 0; a < 2; ++a) tma_load_3d(dst + kKBytes + a * D * 128, &tm_vt, kv_full + 8 * s, j * kKeys + a * 64, 0, b * p.H + h);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && ntiles > 0) {
      // scores of tile t into S buffer t & 1 (its previous occupant, tile t - 2, must have been read)
      auto issue_scores = [&](int t) -> bool {
        const int s = t & 1;
        const uint32_t k_tile = kv_addr + s * kStageBytes;
        if (!bar_wait(kv_full + 8 * s, (t >> 1) & 1, abort_flag, 3)) return false;
        if (t >= 2 && !bar_wait(s_free + 8 * s, ((t >> 1) - 1) & 1, abort_flag, 4)) return false;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < kSub; ++kb) {
          const uint64_t a = tc_desc(q_addr + kb * kRows * 128), bd = tc_desc(k_tile + kb * kKeys * 128);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma(tmem + s * kKeys, a + 2 * k, bd + 2 * k, kIdescS, (kb > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(s_full + 8 * s);
        return true;
      };
      bool ok = bar_wait(q_full, 0, abort_flag, 2) && issue_scores(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j & 1;
        const uint32_t v_tile = kv_addr + s * kStageBytes + kKBytes;
        if (j + 1 < ntiles && !issue_scores(j + 1)) break;
        if (!bar_wait(p_full, j & 1, abort_flag, 5)) break;                      // P of this tile is in shared memory
        if (j > 0 && !bar_wait(pv_free, (j - 1) & 1, abort_flag, 6)) break;      // PV of the previous tile has been read
        tc_fence_after();
#pragma unroll
        for (int a2 = 0; a2 < 2; ++a2) {
          const uint64_t a = tc_desc(p_addr + a2 * kRows * 128), bd = tc_desc(v_tile + a2 * D * 128);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma(tmem + kPvCol, a + 2 * k, bd + 2 * k, kIdescPV, (a2 > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(pv_full);
        tc_commit(kv_empty + 8 * s);
      }
    }
  } else {
    // ---------------- softmax warps (2..5): thread = query row ----------------
    const int quarter = warp & 3, row = quarter * 32 + lane, qi = q0 + row;
    const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16), t_pv = t_lane + kPvCol;
    const T *mrow = p.mask ? reinterpret_cast<const T *>(p.mask) + (long long)b * p.mask_bs : nullptr;
    const int vis_end = p.causal ? min(p.Sk, qi + shift + 1) : p.Sk;               // keys [0, vis_end) are visible to this row
    float o[D];
#pragma unroll
    for (int d = 0; d < D; ++d) o[d] = 0.f;
    float m_run = -1e30f, l_run = 0.f;
    bool alive = ntiles > 0;
    for (int j = 0; j < ntiles && alive; ++j) {
      const int key0 = j * kKeys;
      const uint32_t t_s = t_lane + (j & 1) * kKeys;
      if (!__all_sync(0xffffffffu, bar_wait(s_full + 8 * (j & 1), (j >> 1) & 1, abort_flag, 7))) { alive = false; break; }
      tc_fence_after();
      // pass 1: the row maximum of this tile (log2 domain, masks applied)
      float m_tile = -1e30f;
#pragma unroll 1
      for (int c = 0; c < kKeys / 16; ++c) {
        float x[16];
        tc_ld16(t_s + c * 16, x);
        tile_logits<T>(x, mrow, p.mask_vec != 0, key0 + c * 16, p.Sk, vis_end, p.scale_log2);
#pragma unroll
        for (int e = 0; e < 16; ++e) m_tile = fmaxf(m_tile, x[e]);
      }
      const float m_new = fmaxf(m_run, m_tile);
      const float alpha = exp2f(m_run - m_new);
      // pass 2: probabilities -> the 16-bit A operand of the second product (swizzled rows of 128 bytes)
      float l_tile = 0.f;
#pragma unroll 1
      for (int c = 0; c < kKeys / 16; ++c) {
        float x[16];
        tc_ld16(t_s + c * 16, x);
        tile_logits<T>(x, mrow, p.mask_vec != 0, key0 + c * 16, p.Sk, vis_end, p.scale_log2);
        Vec16<T> lo, hi;
        float a8[8], b8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          a8[e] = exp2f(x[e] - m_new);
          b8[e] = exp2f(x[8 + e] - m_new);
        }
        lo.pack(a8);
        hi.pack(b8);
        // the sum runs over the ROUNDED probabilities, the values the second product multiplies
        lo.unpack(a8);
        hi.unpack(b8);
#pragma unroll
        for (int e = 0; e < 8; ++e) l_tile += a8[e] + b8[e];
        uint8_t *dst = p_ptr + (c >> 2) * (kRows * 128) + row * 128;
        const int u = (c & 3) * 2;
        *reinterpret_cast<uint4 *>(dst + ((u ^ (row & 7)) << 4)) = lo.raw;
        *reinterpret_cast<uint4 *>(dst + (((u + 1) ^ (row & 7)) << 4)) = hi.raw;
      }
      // S has been read (twice): the tensor core may overwrite it with the next tile's scores
      tc_fence_before();
      __syncwarp();
      if (lane == 0) bar_arrive(s_free + 8 * (j & 1));
      // P is complete for this warp's 32 rows: make it visible to the tensor core's reads
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive(p_full);
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      if (!__all_sync(0xffffffffu, bar_wait(pv_full, j & 1, abort_flag, 8))) { alive = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        float x[16];
        tc_ld16(t_pv + c * 16, x);
#pragma unroll
        for (int e = 0; e < 16; ++e) o[c * 16 + e] = o[c * 16 + e] * alpha + x[e];
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) bar_arrive(pv_free);
    }
    if (alive && qi < p.Sq) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      T *orow = reinterpret_cast<T *>(p.o) + (long long)b * p.o_bs + (long long)qi * p.o_rs + h * D;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        Vec16<T> pk;
        float t8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) t8[e] = o[c * 8 + e] * inv;
        pk.pack(t8);
        pk.store(orow + c * 8);
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = gtimer();
    while (gtimer() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                             const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn tc_encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  }
  return fn;
}

// 3-D map over [batch][rows][cols] (cols contiguous), box 64 x box_rows x 1, 128-byte swizzle,
// out-of-bounds elements read as zero.  Strides in elements.
int tc_map3(CUtensorMap *map, const void *base, int dtype, long long cols, long long rows, long long batch, long long row_stride,
            long long batch_stride, int box_rows) {
  EncodeFn fn = tc_encode_fn();
  if (!fn) return fail(EB_ECUDA, "attention_prefill: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)batch_stride * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dtype == EB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base),
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(EB_ECUDA, "attention_prefill: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return EB_OK;
}

template <typename T, int D>
int launch_tc(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const TcParams &p, cudaStream_t st) {
  constexpr size_t smem = 1024 + 1024 + (size_t)(D / 64) * kRows * 128 + 2 * ((size_t)(D / 64) * kKeys * 128 + 2 * D * 128) + 2 * kRows * 128;
  auto kern = attention_prefill_tc_kernel<T, D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return fail(EB_ECUDA, "attention_prefill: cannot reserve %zu bytes of shared memory", smem);
    }
    configured[dev] = true;
  }
  dim3 grid((p.Sq + kRows - 1) / kRows, p.H, p.B);
  launch_pdl(kern, grid, dim3(kTcThreads), smem, st, mq, mk, mv, p);
  return check_launch("attention_prefill");
}

}  // namespace

// Status words of this file's kernels, for eb_device_status.
int attention_tc_status(int *out4, bool clear) {
  int host[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(host, g_tc_status, sizeof(host)) != cudaSuccess) {
    cudaGetLastError();
    return EB_ECUDA;
  }
  for (int i = 0; i < 4; ++i) out4[i] = host[i];
  if (clear && host[0] != 0) {
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_tc_status, zero, sizeof(zero));
  }
  return EB_OK;
}

}  // namespace eb

using namespace eb;

extern "C" size_t eb_attention_prefill_scratch_bytes(int batch, int heads, int kv_len, int head_dim) {
  if (batch <= 0 || heads <= 0 || kv_len <= 0 || head_dim <= 0) return 0;
  const size_t skp = ((size_t)kv_len + 63) / 64 * 64;
  return (size_t)batch * heads * head_dim * skp * 2;
}

extern "C" int eb_attention_prefill_tc(const void *q, const void *k, const void *v, void *out, const void *mask,
                                       long long q_batch_stride, long long q_row_stride, long long k_batch_stride,
                                       long long k_row_stride, long long v_batch_stride, long long v_row_stride,
                                       long long o_batch_stride, long long o_row_stride, long long mask_batch_stride, int batch,
                                       int heads, int q_len, int kv_len, int head_dim, int causal, float scale, int dtype,
                                       void *scratch, size_t scratch_bytes, void *stream) {
  if (batch == 0 || heads == 0 || q_len == 0) return EB_OK;
  EB_REQUIRE(dtype == EB_F16 || dtype == EB_BF16, "attention_prefill: fp16 or bf16 only (dtype %d)", dtype);
  EB_REQUIRE(head_dim == 64 || head_dim == 128, "attention_prefill: head_dim %d not supported (64 or 128)", head_dim);
  EB_REQUIRE(batch > 0 && heads > 0 && q_len > 0 && kv_len > 0, "attention_prefill: negative or zero size");
  EB_REQUIRE(heads <= 65535 && batch <= 65535, "attention_prefill: batch and heads are limited to 65535");
  EB_REQUIRE(q && k && v && out, "attention_prefill: null pointer");
  EB_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), "attention_prefill: pointers must be 16-byte aligned");
  const long long strides[] = {q_batch_stride, q_row_stride, k_batch_stride, k_row_stride, v_batch_stride, v_row_stride,
                               o_batch_stride, o_row_stride};
  for (long long s : strides) EB_REQUIRE(s % 8 == 0, "attention_prefill: strides must be multiples of 8 elements");
  EB_REQUIRE(kv_len >= q_len || !causal, "attention_prefill: causal attention needs kv_len >= q_len");
  const size_t need = eb_attention_prefill_scratch_bytes(batch, heads, kv_len, head_dim);
  EB_REQUIRE(scratch && aligned16(scratch) && scratch_bytes >= need, "attention_prefill: needs a scratch of %zu bytes (eb_attention_prefill_scratch_bytes)", need);
  const int skp = (kv_len + 63) / 64 * 64;
  cudaStream_t st = as_stream(stream);
  const long long hd = (long long)heads * head_dim;
  {
    dim3 grid(skp / 64, (unsigned)(hd / 64), batch);
    if (dtype == EB_F16)
      launch_pdl(transpose_v_kernel<__half>, grid, dim3(256), 0, st, reinterpret_cast<const __half *>(v), reinterpret_cast<__half *>(scratch),
                 v_batch_stride, v_row_stride, heads, head_dim, kv_len, skp);
    else
      launch_pdl(transpose_v_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, reinterpret_cast<const __nv_bfloat16 *>(v),
                 reinterpret_cast<__nv_bfloat16 *>(scratch), v_batch_stride, v_row_stride, heads, head_dim, kv_len, skp);
    int rc = check_launch("attention_prefill (transpose)");
    if (rc) return rc;
  }
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = tc_map3(&mq, q, dtype, hd, q_len, batch, q_row_stride, q_batch_stride, kRows))) return rc;
  if ((rc = tc_map3(&mk, k, dtype, hd, kv_len, batch, k_row_stride, k_batch_stride, kKeys))) return rc;
  if ((rc = tc_map3(&mv, scratch, dtype, kv_len, head_dim, (long long)batch * heads, skp, (long long)head_dim * skp, head_dim))) return rc;
  TcParams p{};
  p.B = batch; p.H = heads; p.Sq = q_len; p.Sk = kv_len; p.causal = causal;
  p.scale_log2 = scale * kLog2eTc;
  p.mask = mask; p.mask_bs = mask_batch_stride;
  p.mask_vec = mask && aligned16(mask) && mask_batch_stride % 8 == 0;
  p.o = out; p.o_bs = o_batch_stride; p.o_rs = o_row_stride;
  if (dtype == EB_F16) return head_dim == 64 ? launch_tc<__half, 64>(mq, mk, mv, p, st) : launch_tc<__half, 128>(mq, mk, mv, p, st);
  return head_dim == 64 ? launch_tc<__nv_bfloat16, 64>(mq, mk, mv, p, st) : launch_tc<__nv_bfloat16, 128>(mq, mk, mv, p, st);
}
