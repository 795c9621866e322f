// Prompt-pass attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
//   out[b,i,h,:] = softmax_j( scale * q[b,i,h,:].k[b,j,h,:] + mask[b,j] ; causal ) . v[b,j,h,:]
// (energonai/model/attention.py:105-124, without materialising the score tensor).
//
// One CTA owns 128 query rows of one (sequence, head) and walks the visible keys in tiles of
// 128.  Both products run on tcgen05.mma with fp32 accumulators in tensor memory:
//   S  = Q . K_tile^T    (128 x 128, K = head_dim)   TMEM columns [t*128, +128) for row tile t
//   O += P . V_tile      (128 x head_dim, K = 128)    TMEM columns [256 + t*128, +head_dim)
// Q, K and V tiles arrive by TMA (3-D maps over the [batch][row][head*dim] views, 128-byte
// swizzle, rows beyond the sequence read as zeros).  V is used as it lies in memory: for the
// second product the contraction index (keys) runs down the rows of the tile, which the shared-
// memory descriptor expresses as an N-major B operand, so nothing is transposed.
// A CTA serves two row tiles (256 query rows).  Warp roles (320 threads): warp 0 issues
// TMA, warp 1 issues the MMAs, warps 2-5 and 6-9 are the softmax of row tile 0 and 1: thread r
// owns query row r, reads its score row from TMEM (tcgen05.ld), keeps the running maximum / sum
// (fp32, log2 domain) and writes the probabilities as the 16-bit, swizzled A operand of the second
// product into shared memory.  The output row accumulates in TMEM across the key tiles (the
// second product adds to it).  Its scale is the maximum the row had when it was last rescaled:
// only when a new tile raises the row maximum by more than 2^8 do the softmax warps read the row
// back, multiply it and store it again (tcgen05.ld / st), so that in the common case they never
// wait for the second product and the probabilities stay below 2^8 (fine in fp16 and bf16, the
// sum is fp32).  The two row tiles alternate on the tensor core: while the softmax warps of one
// work on their scores, it serves the other.
//
// Every mbarrier wait is bounded; a wait that runs out is recorded, the CTA's roles leave (each
// decision made uniform over the warp first), copies in flight are given time to land, TMEM is
// freed and the kernel returns.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"

namespace eb {
namespace {

constexpr int kRows = 128;                 // query rows per row tile = UMMA M = TMEM lanes
constexpr int kTiles = 2;                  // row tiles per CTA, each with its own four softmax warps
constexpr int kKeys = 128;                 // keys per tile
constexpr int kTcThreads = 64 + kTiles * 128;

// Shared-memory plan per head_dim.  With head_dim 128 everything but a second V stage fits.
template <int D> struct TcSmem {
  static constexpr uint32_t kQBytes = (D / 64) * kRows * 128, kKBytes = (D / 64) * kKeys * 128, kVBytes = (D / 64) * kKeys * 128,
                            kPBytes = 2 * kRows * 128;
  static constexpr int kVStages = D > 64 ? 1 : 2;
  static constexpr size_t kTotal = 1024 + 1024 + (size_t)kTiles * kQBytes + 2 * kKBytes + (size_t)kVStages * kVBytes + (size_t)kTiles * kPBytes;
};
constexpr float kLog2eTc = 1.4426950408889634f;
constexpr float kRescaleLog2 = 8.f;         // the accumulated row is rescaled when its maximum grows by more than 2^8
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
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float *v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
      "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const float *v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
      "%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// K-major tile of 128-byte rows with the 128-byte swizzle; 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// N-major B operand (the contraction index runs down the rows of the tile): 64-column atoms of
// 8 rows x 128 bytes, swizzled; atoms along N lie atom_stride bytes apart (leading offset), 8-row
// groups along K 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_desc_nmajor(uint32_t addr, uint32_t atom_stride) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(atom_stride >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// kind::f16, fp32 accumulate, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t tc_idesc(int n, int is_bf16) {
  return (1u << 4) | ((uint32_t)is_bf16 << 7) | ((uint32_t)is_bf16 << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
}

// ---- the attention kernel ----------------------------------------------------------------------
// Shared memory (1024-aligned): [1 KB barriers, TMEM slot, abort flag][Q: 2 row tiles x D/64
// sub-tiles of 128 rows x 128 B][K ring: 2 x D/64 sub-tiles][V ring: kVStages x D/64 sub-tiles
// of 128 key rows x 128 B][P: 2 row tiles x 2 sub-tiles of 128 rows x 128 B].
template <typename T, int D>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                            const __grid_constant__ CUtensorMap tm_v, const TcParams p) {
  constexpr int kSub = D / 64;                                   // 64-column sub-tiles of Q / K
  constexpr int kVStages = TcSmem<D>::kVStages;
  constexpr uint32_t kQBytes = TcSmem<D>::kQBytes, kKBytes = TcSmem<D>::kKBytes, kVBytes = TcSmem<D>::kVBytes,
                     kPBytes = TcSmem<D>::kPBytes;
  constexpr uint32_t kTmemCols = 512, kPvCol = 2 * kKeys;
  constexpr int kBf16 = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t kIdescS = tc_idesc(kKeys, kBf16), kIdescPV = tc_idesc(D, kBf16) | (1u << 16);   // bit 16: B is N-major

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = s32(smem_raw);
  uint8_t *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
  const uint32_t bar0 = s32(bars);
  // per-ring barriers are indexed by stage, per-row-tile barriers by tile (8 bytes apart)
  const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = bar0 + 24, v_full = bar0 + 40, v_empty = bar0 + 56,
                 s_full = bar0 + 72, p_full = bar0 + 88, pv_full = bar0 + 104;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 256);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 264);
  const uint32_t q_addr = s32(smem) + 1024, k_addr = q_addr + kTiles * kQBytes, v_addr = k_addr + 2 * kKBytes,
                 p_addr = v_addr + kVStages * kVBytes;
  uint8_t *p_ptr = smem + 1024 + kTiles * kQBytes + 2 * kKBytes + kVStages * kVBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;   // longest (latest, under the causal mask) blocks first
  const int q0 = qb * (kTiles * kRows), shift = p.Sk - p.Sq;
  // key tiles each row tile walks: all of them, or up to its last row's diagonal; none for a
  // row tile that lies wholly behind the end of the sequence
  int nt[kTiles], nmax = 0;
#pragma unroll
  for (int t = 0; t < kTiles; ++t) {
    const int qt0 = q0 + t * kRows;
    const int last_key = p.causal ? min(p.Sk - 1, qt0 + kRows - 1 + shift) : p.Sk - 1;
    nt[t] = (qt0 < p.Sq && last_key >= 0) ? last_key / kKeys + 1 : 0;
    nmax = max(nmax, nt[t]);
  }

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_v) : "memory");
    bar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      bar_init(k_full + 8 * s, 1);
      bar_init(k_empty + 8 * s, 1);
      bar_init(v_full + 8 * s, 1);
      bar_init(v_empty + 8 * s, 1);
      bar_init(s_full + 8 * s, 1);
      bar_init(p_full + 8 * s, 4);
      bar_init(pv_full + 8 * s, 1);
    }
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
    if (lane == 0 && nmax > 0) {
      bar_expect_tx(q_full, kTiles * kQBytes);
#pragma unroll
      for (int t = 0; t < kTiles; ++t)
#pragma unroll
        for (int kb = 0; kb < kSub; ++kb)
          tma_load_3d(q_addr + t * kQBytes + kb * kRows * 128, &tm_q, q_full, h * D + kb * 64, q0 + t * kRows, b);
      // K runs one tile ahead of V: its stage is released earlier (after the scores, not after
      // the value product), and the next scores are what the softmax warps wait for
      auto load_k = [&](int j) -> bool {
        const int ks = j & 1;
        if (j >= 2 && !bar_wait(k_empty + 8 * ks, ((j >> 1) - 1) & 1, abort_flag, 1)) return false;
        bar_expect_tx(k_full + 8 * ks, kKBytes);
#pragma unroll
        for (int kb = 0; kb < kSub; ++kb)
          tma_load_3d(k_addr + ks * kKBytes + kb * kKeys * 128, &tm_k, k_full + 8 * ks, h * D + kb * 64, j * kKeys, b);
        return true;
      };
      bool ok = load_k(0);
      for (int j = 0; j < nmax && ok; ++j) {
        const int vs = j % kVStages, vu = j / kVStages;
        if (j + 1 < nmax && !load_k(j + 1)) break;
        if (j >= kVStages && !bar_wait(v_empty + 8 * vs, (vu - 1) & 1, abort_flag, 9)) break;
        bar_expect_tx(v_full + 8 * vs, kVBytes);
#pragma unroll
        for (int kb = 0; kb < kSub; ++kb)
          tma_load_3d(v_addr + vs * kVBytes + kb * kKeys * 128, &tm_v, v_full + 8 * vs, h * D + kb * 64, j * kKeys, b);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // Per row tile the order is S(0), then for every key tile j, as soon as P(j) is written
    // (which also says that S(j) has been read): S(j+1) first, so the softmax warps get their
    // next scores as early as possible, then O += P(j) . V(j).
    if (lane == 0 && nmax > 0) {
      auto last_reader = [&](int j) { return (kTiles > 1 && j < nt[kTiles - 1]) ? kTiles - 1 : 0; };
      auto issue_scores = [&](int t, int j) -> bool {
        const int ks = j & 1;
        if (!bar_wait(k_full + 8 * ks, (j >> 1) & 1, abort_flag, 3)) return false;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < kSub; ++kb) {
          const uint64_t a = tc_desc(q_addr + t * kQBytes + kb * kRows * 128), bd = tc_desc(k_addr + ks * kKBytes + kb * kKeys * 128);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma(tmem + t * kKeys, a + 2 * k, bd + 2 * k, kIdescS, (kb > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(s_full + 8 * t);
        if (t == last_reader(j)) tc_commit(k_empty + 8 * ks);
        return true;
      };
      bool ok = bar_wait(q_full, 0, abort_flag, 2);
      for (int t = 0; t < kTiles && ok; ++t)
        if (nt[t] > 0) ok = issue_scores(t, 0);
      for (int j = 0; j < nmax && ok; ++j) {
        const int vs = j % kVStages, vu = j / kVStages;
        for (int t = 0; t < kTiles && ok; ++t) {
          if (j >= nt[t]) continue;
          ok = bar_wait(p_full + 8 * t, j & 1, abort_flag, 5);
          if (ok && j + 1 < nt[t]) ok = issue_scores(t, j + 1);
          ok = ok && bar_wait(v_full + 8 * vs, vu & 1, abort_flag, 10);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int a2 = 0; a2 < 2; ++a2) {
            const uint64_t a = tc_desc(p_addr + t * kPBytes + a2 * kRows * 128);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              // 16 keys per instruction: two 8-row groups (2048 bytes) down the V tile
              const uint64_t bd = tc_desc_nmajor(v_addr + vs * kVBytes + (a2 * 4 + k) * 2048, kKeys * 128);
              tc_mma(tmem + kPvCol + t * kKeys, a + 2 * k, bd, kIdescPV, (j > 0 || a2 > 0 || k > 0) ? 1u : 0u);
            }
          }
          tc_commit(pv_full + 8 * t);
          if (t == last_reader(j)) tc_commit(v_empty + 8 * vs);
        }
      }
    }
  } else {
    // ---------------- softmax warps: 4 per row tile, thread = query row ----------------
    const int t = (warp - 2) >> 2, quarter = warp & 3, row = quarter * 32 + lane, qi = q0 + t * kRows + row;
    const int ntiles = nt[t];
    const uint32_t t_s = tmem + ((uint32_t)(quarter * 32) << 16) + t * kKeys, t_pv = t_s + kPvCol;
    const uint32_t my_s_full = s_full + 8 * t, my_p_full = p_full + 8 * t, my_pv_full = pv_full + 8 * t;
    uint8_t *p_row = p_ptr + t * kPBytes + row * 128;
    const T *mrow = p.mask ? reinterpret_cast<const T *>(p.mask) + (long long)b * p.mask_bs : nullptr;
    const int vis_end = p.causal ? min(p.Sk, qi + shift + 1) : p.Sk;               // keys [0, vis_end) are visible to this row
    float m_ref = -1e30f, l_run = 0.f;      // m_ref: the maximum the accumulated row and l_run are scaled by
    bool alive = ntiles > 0;
    for (int j = 0; j < ntiles && alive; ++j) {
      const int key0 = j * kKeys;
      // Work per chunk of 32 keys, decided for the warp as a whole (tensor-memory loads are
      // warp-wide): 0 = hidden from every row of the warp (behind the diagonal or the end of the
      // sequence): nothing to read, P = 0; 1 = visible to every row and no mask value set: one
      // multiply-add and one exponential per key, most chunks of a long prompt; 2 = per-key
      // work (the chunk the diagonal crosses, chunks with mask values).  Lane l keeps the mask
      // value of key l of each chunk, in the log2 domain.
      int cls[kKeys / 32];
      float mval[kKeys / 32];
#pragma unroll
      for (int c = 0; c < kKeys / 32; ++c) {
        const int kb = key0 + c * 32;
        float mv = 0.f;
        if (mrow && kb + lane < p.Sk) mv = to_f32<T>(mrow[kb + lane]) * kLog2eTc;
        mval[c] = mv;
        const bool hidden = __all_sync(0xffffffffu, kb >= vis_end);
        const bool simple = __all_sync(0xffffffffu, kb + 32 <= vis_end && mv == 0.f);
        cls[c] = hidden ? 0 : (simple ? 1 : 2);
      }
      if (!__all_sync(0xffffffffu, bar_wait(my_s_full, j & 1, abort_flag, 7))) { alive = false; break; }
      tc_fence_after();
      // pass 1: the row maximum of this tile (log2 domain, masks applied)
      float r0 = -INFINITY, r1 = -INFINITY, r2 = -INFINITY, r3 = -INFINITY, m_tile = -1e30f;
#pragma unroll
      for (int c = 0; c < kKeys / 32; ++c) {
        if (cls[c] == 0) continue;
        float x[32];
        tc_ld32(t_s + c * 32, x);
        if (cls[c] == 1) {
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            r0 = fmaxf(r0, x[e]);
            r1 = fmaxf(r1, x[e + 1]);
            r2 = fmaxf(r2, x[e + 2]);
            r3 = fmaxf(r3, x[e + 3]);
          }
        } else {
          const int nvis = vis_end - (key0 + c * 32);
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float v = fmaf(x[e], p.scale_log2, __shfl_sync(0xffffffffu, mval[c], e));
            m_tile = fmaxf(m_tile, e < nvis ? v : -INFINITY);
          }
        }
      }
      r0 = fmaxf(fmaxf(r0, r1), fmaxf(r2, r3));
      if (r0 > -INFINITY) m_tile = fmaxf(m_tile, r0 * p.scale_log2);   // the scale is positive: the maximum commutes with it
      // The previous tile's value product must be complete before P is overwritten (it reads P)
      // and before the accumulated row is rescaled; it was issued right behind the scores just
      // read, so this wait is normally over already.
      if (j > 0 && !__all_sync(0xffffffffu, bar_wait(my_pv_full, (j - 1) & 1, abort_flag, 8))) { alive = false; break; }
      // rescale only when some row of the warp gained more than 2^8 (the loads and stores of
      // tensor memory are warp-wide, so the warp decides together)
      if (__any_sync(0xffffffffu, m_tile > m_ref + kRescaleLog2)) {
        const float m_new = fmaxf(m_ref, m_tile);
        const float alpha = ex2(m_ref - m_new);
        m_ref = m_new;
        l_run *= alpha;
        if (j > 0) {
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            float x[32];
            tc_ld32(t_pv + c * 32, x);
#pragma unroll
            for (int e = 0; e < 32; ++e) x[e] *= alpha;
            tc_st32(t_pv + c * 32, x);
          }
          tc_st_wait();
        }
      }
      // pass 2: probabilities -> the 16-bit A operand of the second product (swizzled rows of 128 bytes)
      float l0 = 0.f, l1 = 0.f;
      const float neg_m = -m_ref;
#pragma unroll
      for (int c = 0; c < kKeys / 32; ++c) {
        uint8_t *dst = p_row + (c >> 1) * (kRows * 128);
        if (cls[c] == 0) {
#pragma unroll
          for (int g = 0; g < 4; ++g) *reinterpret_cast<uint4 *>(dst + ((((c & 1) * 4 + g) ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
          continue;
        }
        float x[32];
        tc_ld32(t_s + c * 32, x);
        if (cls[c] == 1) {
#pragma unroll
          for (int e = 0; e < 32; ++e) x[e] = ex2(fmaf(x[e], p.scale_log2, neg_m));
        } else {
          const int nvis = vis_end - (key0 + c * 32);
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float v = fmaf(x[e], p.scale_log2, __shfl_sync(0xffffffffu, mval[c], e));
            x[e] = e < nvis ? ex2(v + neg_m) : 0.f;
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = pack2<T>(x[g * 8 + 0], x[g * 8 + 1]);
          w.y = pack2<T>(x[g * 8 + 2], x[g * 8 + 3]);
          w.z = pack2<T>(x[g * 8 + 4], x[g * 8 + 5]);
          w.w = pack2<T>(x[g * 8 + 6], x[g * 8 + 7]);
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            l0 += x[g * 8 + e];
            l1 += x[g * 8 + e + 1];
          }
          *reinterpret_cast<uint4 *>(dst + ((((c & 1) * 4 + g) ^ (row & 7)) << 4)) = w;
        }
      }
      l_run += l0 + l1;
      // P is complete for this warp's 32 rows: make it visible to the tensor core's reads.  The
      // same arrival tells the issuer that S has been read and that the row has been rescaled.
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive(my_p_full);
    }
    if (alive && !__all_sync(0xffffffffu, bar_wait(my_pv_full, (ntiles - 1) & 1, abort_flag, 11))) alive = false;
    if (alive) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      T *orow = reinterpret_cast<T *>(p.o) + (long long)b * p.o_bs + (long long)qi * p.o_rs + h * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        float x[32];
        tc_ld32(t_pv + c * 32, x);                 // warp-wide: rows behind the end of the sequence read too, and store nothing
        if (qi < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack2<T>(x[g * 8 + 0] * inv, x[g * 8 + 1] * inv);
            w.y = pack2<T>(x[g * 8 + 2] * inv, x[g * 8 + 3] * inv);
            w.z = pack2<T>(x[g * 8 + 4] * inv, x[g * 8 + 5] * inv);
            w.w = pack2<T>(x[g * 8 + 6] * inv, x[g * 8 + 7] * inv);
            *reinterpret_cast<uint4 *>(orow + c * 32 + g * 8) = w;
          }
        }
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
  constexpr size_t smem = TcSmem<D>::kTotal;
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
  dim3 grid((p.Sq + kTiles * kRows - 1) / (kTiles * kRows), p.H, p.B);
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

extern "C" int eb_attention_prefill_tc(const void *q, const void *k, const void *v, void *out, const void *mask,
                                       long long q_batch_stride, long long q_row_stride, long long k_batch_stride,
                                       long long k_row_stride, long long v_batch_stride, long long v_row_stride,
                                       long long o_batch_stride, long long o_row_stride, long long mask_batch_stride, int batch,
                                       int heads, int q_len, int kv_len, int head_dim, int causal, float scale, int dtype,
                                       void *stream) {
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
  EB_REQUIRE(scale > 0.f, "attention_prefill: the scale must be positive");
  cudaStream_t st = as_stream(stream);
  const long long hd = (long long)heads * head_dim;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = tc_map3(&mv, v, dtype, hd, kv_len, batch, v_row_stride, v_batch_stride, kKeys))) return rc;
  if ((rc = tc_map3(&mq, q, dtype, hd, q_len, batch, q_row_stride, q_batch_stride, kRows))) return rc;
  if ((rc = tc_map3(&mk, k, dtype, hd, kv_len, batch, k_row_stride, k_batch_stride, kKeys))) return rc;
  TcParams p{};
  p.B = batch; p.H = heads; p.Sq = q_len; p.Sk = kv_len; p.causal = causal;
  p.scale_log2 = scale * kLog2eTc;
  p.mask = mask; p.mask_bs = mask_batch_stride;
  p.mask_vec = mask && aligned16(mask) && mask_batch_stride % 8 == 0;
  p.o = out; p.o_bs = o_batch_stride; p.o_rs = o_row_stride;
  if (dtype == EB_F16) return head_dim == 64 ? launch_tc<__half, 64>(mq, mk, mv, p, st) : launch_tc<__half, 128>(mq, mk, mv, p, st);
  return head_dim == 64 ? launch_tc<__nv_bfloat16, 64>(mq, mk, mv, p, st) : launch_tc<__nv_bfloat16, 128>(mq, mk, mv, p, st);
}
