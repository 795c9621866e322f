// Fused attention for the layer forward: scores, mask, softmax and the value product in one
// pass, never materialising the [batch, heads, S, S] score tensor.
//
//   attention_prefill : all query rows of a prompt against all keys (flash-style: 64-query x
//       64-key tiles, fp32 online softmax, tensor-core products).
//   attention_decode  : one new query row per sequence against the cached keys/values.  The
//       work is one pass over the cache (HBM-bound), so the key range of each (sequence,
//       head) is split over several CTAs; partial (max, sum, output) triples go through a
//       caller-provided fp32 scratch and the CTA that arrives last merges them.
//
// Masking follows energonai/model/attention.py:105-116: scores are scaled by head_dim^-0.5,
// keys after the query are hidden when `causal`, and an optional additive per-key mask row
// (0 / -10000 from the padding mask) is added before an fp32 softmax.  Hidden keys get weight
// exactly 0 (the reference reaches the same through exp(-1e4) underflow).
//
// Q, K and V are addressed as [batch][row][head*D + d] with independent batch and row strides,
// so they may be column slices of one fused projection / cache buffer.
#include <mutex>

#include "common.cuh"

namespace eb {
namespace {

constexpr int kBM = 64, kBN = 64, kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kDecodeStages = 2;   // key/value tiles in flight per CTA of the generation-step kernel

struct AttnParams {
  const void *q, *k, *v;
  void *o;
  const void *mask;            // additive per-key mask [batch][kv_len] in the tensor dtype, or null
  long long q_bs, q_rs, k_bs, k_rs, v_bs, v_rs, o_bs, o_rs, mask_bs;   // strides in elements
  int B, H, Sq, Sk;            // Sk = kv length when kv_len_ptr is null
  const int *kv_len_ptr;       // decode: device scalar with the current kv length (overrides Sk)
  int causal;
  float scale;
  // decode split-KV
  int nsplit;
  float *scratch;              // [B*H][nsplit][D + 2]
  int *counters;               // [B*H], zero between calls
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
  const int bytes = valid ? 16 : 0;   // src-size 0 zero-fills the destination
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <typename T> __device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&h);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] 16-bit tile whose chunks are
// XOR-swizzled with the row index (conflict-free ldmatrix and cp.async).
template <int D> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// Load `kBN` rows starting at `row0` of a [*, D] slice (row stride rs elements) into a tile;
// rows >= row_end are zero-filled.  Thread t always moves 16-byte chunk (t % (D/8)) of rows
// t / (D/8) + k * (kThreads / (D/8)); the row step is a multiple of 8, so the swizzle term is the
// same for all of a thread's chunks and both addresses advance by constants.
template <typename T, int D>
__device__ __forceinline__ void load_tile(uint32_t tile, const T *base, long long rs, int row0, int row_end) {
  constexpr int kChunks = D / 8, kRowStep = kThreads / kChunks, kIters = kBN / kRowStep;
  static_assert(kRowStep % 8 == 0 && kBN % kRowStep == 0, "tile shape must keep the swizzle term constant per thread");
  const int r0 = threadIdx.x / kChunks, c = threadIdx.x % kChunks;
  uint32_t dst = tile + tile_off<D>(r0, c);
  const T *src = base + (long long)(row0 + r0) * rs + c * 8;
  const long long src_step = (long long)kRowStep * rs;
  int row = row0 + r0;
#pragma unroll
  for (int k = 0; k < kIters; ++k) {
    const bool ok = row < row_end;
    cp_async16(dst, ok ? src : base, ok);
    dst += kRowStep * D * 2;
    src += src_step;
    row += kRowStep;
  }
}

// The 16 rows [warp*16, warp*16+16) of a tile, loaded by that warp alone: the generation-step
// kernel gives every warp its own slice of each tile, so the warps need no CTA-wide barrier
// inside the key loop.  Lane l moves chunk l % (D/8) of rows l / (D/8) + k * (32 / (D/8)).
template <typename T, int D>
__device__ __forceinline__ void load_warp_rows(uint32_t tile, const T *base, long long rs, int row0, int row_end,
                                               int warp, int lane) {
  constexpr int kChunks = D / 8, kRowStep = 32 / kChunks, kIters = 16 / kRowStep;
  const int c = lane % kChunks, rl = lane / kChunks;
  int row = row0 + warp * 16 + rl;
  const T *src = base + (long long)row * rs + c * 8;
  const long long src_step = (long long)kRowStep * rs;
  const uint32_t dst0 = tile + (uint32_t)((warp * 16 + rl) * D * 2);
#pragma unroll
  for (int k = 0; k < kIters; ++k) {
    const bool ok = row < row_end;
    // swizzle term of row warp*16 + rl + k*kRowStep (warp*16 is a multiple of 8)
    const uint32_t dst = dst0 + (uint32_t)(k * kRowStep * D * 2) + (uint32_t)((c ^ ((rl + k * kRowStep) & 7)) << 4);
    cp_async16(dst, ok ? src : base, ok);
    src += src_step;
    row += kRowStep;
  }
}

// ------------------------------------------------------------------------------------------------
// prefill
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
attention_prefill_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kTileBytes = kBN * D * 2;
  const uint32_t q_s = smem_u32(smem), k_s = q_s + kTileBytes, v_s = k_s + 2 * kTileBytes;
  float *mask_s = reinterpret_cast<float *>(smem + 5 * kTileBytes);   // [2][kBN]

  griddep_wait();
  griddep_launch();
  const int qt = gridDim.x - 1 - blockIdx.x;   // heavy (late) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int Sq = p.Sq, Sk = p.Sk;
  const int i0 = qt * kBM;
  const int shift = Sk - Sq;                   // query i sees keys j <= i + shift under the causal mask

  const T *qb = reinterpret_cast<const T *>(p.q) + b * p.q_bs + h * D;
  const T *kb = reinterpret_cast<const T *>(p.k) + b * p.k_bs + h * D;
  const T *vb = reinterpret_cast<const T *>(p.v) + b * p.v_bs + h * D;
  const T *mb = p.mask ? reinterpret_cast<const T *>(p.mask) + b * p.mask_bs : nullptr;

  int ntiles = (Sk + kBN - 1) / kBN;
  if (p.causal) {
    const int last_key = min(Sk - 1, i0 + kBM - 1 + shift);
    ntiles = last_key < 0 ? 0 : last_key / kBN + 1;
  }

  load_tile<T, D>(q_s, qb, p.q_rs, i0, Sq);
  auto load_kv = [&](int n, int buf) {
    load_tile<T, D>(k_s + buf * kTileBytes, kb, p.k_rs, n * kBN, Sk);
    load_tile<T, D>(v_s + buf * kTileBytes, vb, p.v_rs, n * kBN, Sk);
    if (threadIdx.x < kBN) {
      const int j = n * kBN + threadIdx.x;
      mask_s[buf * kBN + threadIdx.x] = (mb && j < Sk) ? to_f32<T>(mb[j]) * kLog2e : 0.f;
    }
  };
  if (ntiles > 0) load_kv(0, 0);
  cp_async_commit();

  uint32_t qf[D / 16][4];
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sc = p.scale * kLog2e;
  const int row_lo = i0 + warp * 16 + g;       // this thread's two query rows: row_lo, row_lo + 8

  for (int n = 0; n < ntiles; ++n) {
    const int buf = n & 1;
    if (n + 1 < ntiles) load_kv(n + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (n == 0) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(qf[kk], q_s + tile_off<D>(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), kk * 2 + (lane >> 4)));
    }
    // S = Q K^T for 16 query rows x 64 keys
    float s[kBN / 8][4];
#pragma unroll
    for (int i = 0; i < kBN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    const uint32_t kt = k_s + buf * kTileBytes, vt = v_s + buf * kTileBytes;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int nb = 0; nb < kBN / 16; ++nb) {
        uint32_t kf[4];
        ldmatrix_x4(kf, kt + tile_off<D>(nb * 16 + (lane & 7) + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
        mma16816<T>(s[2 * nb], qf[kk], kf[0], kf[1]);
        mma16816<T>(s[2 * nb + 1], qf[kk], kf[2], kf[3]);
      }
    }
    // scale, mask
    const int j0 = n * kBN;
    const bool edge = (p.causal && j0 + kBN - 1 > i0 + warp * 16 + shift) || j0 + kBN > Sk;
#pragma unroll
    for (int i = 0; i < kBN / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int jl = i * 8 + 2 * t + (e & 1);
        float x = s[i][e] * sc + mask_s[buf * kBN + jl];
        if (edge) {
          const int j = j0 + jl, row = row_lo + (e >> 1) * 8;
          if (j >= Sk || (p.causal && j > row + shift)) x = -INFINITY;
        }
        s[i][e] = x;
      }
    }
    // online softmax for rows row_lo (e = 0,1) and row_lo + 8 (e = 2,3)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < kBN / 8; ++i) mx = fmaxf(mx, fmaxf(s[i][2 * r], s[i][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float corr = exp2f(m_run[r] - m_use);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < kBN / 8; ++i) {
        s[i][2 * r] = exp2f(s[i][2 * r] - m_use);
        s[i][2 * r + 1] = exp2f(s[i][2 * r + 1] - m_use);
        sum += s[i][2 * r] + s[i][2 * r + 1];
      }
      l_run[r] = l_run[r] * corr + sum;
      m_run[r] = m_new;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) { o[i][2 * r] *= corr; o[i][2 * r + 1] *= corr; }
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) {
      uint32_t pf[4];
      pf[0] = pack2<T>(s[2 * kk][0], s[2 * kk][1]);
      pf[1] = pack2<T>(s[2 * kk][2], s[2 * kk][3]);
      pf[2] = pack2<T>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pf[3] = pack2<T>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int db = 0; db < D / 16; ++db) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vt + tile_off<D>(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), db * 2 + (lane >> 4)));
        mma16816<T>(o[2 * db], pf, vf[0], vf[1]);
        mma16816<T>(o[2 * db + 1], pf, vf[2], vf[3]);
      }
    }
    __syncthreads();   // this buffer is refilled by the prefetch of the next iteration
  }
  cp_async_wait<0>();

  // normalise, stage the 64 x D output tile through shared memory (Q's tile), store 16-byte rows
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int row = warp * 16 + g + r * 8;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const uint32_t val = pack2<T>(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
      *reinterpret_cast<uint32_t *>(smem + tile_off<D>(row, i) + t * 4) = val;
    }
  }
  __syncthreads();
  T *ob = reinterpret_cast<T *>(p.o) + b * p.o_bs + h * D;
  constexpr int kChunks = D / 8;
  for (int i = threadIdx.x; i < kBM * kChunks; i += kThreads) {
    const int r = i / kChunks, c = i % kChunks;
    if (i0 + r < Sq)
      *reinterpret_cast<uint4 *>(ob + (long long)(i0 + r) * p.o_rs + c * 8) =
          *reinterpret_cast<const uint4 *>(smem + tile_off<D>(r, c));
  }
}

// ------------------------------------------------------------------------------------------------
// decode: one query row per (sequence, head); keys split over gridDim.x CTAs
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
attention_decode_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kTileBytes = kBN * D * 2;
  // Three tiles of keys and values in flight per CTA: a CTA usually owns three tiles in all
  // (see pick of nsplit on the host), so its whole key range is requested up front and the
  // HBM latency is paid once instead of once per tile.
  const uint32_t k_s = smem_u32(smem), v_s = k_s + kDecodeStages * kTileBytes;
  float *mask_s = reinterpret_cast<float *>(smem + 2 * kDecodeStages * kTileBytes);   // [stages][kBN]
  float *red = mask_s + kDecodeStages * kBN;                                   // [4][D + 2] warp partials
  __shared__ int s_last;

  griddep_wait();
  griddep_launch();
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // a device-side length is clamped to the capacity the host stated (p.Sk, when positive)
  const int Sk = p.kv_len_ptr ? max(1, p.Sk > 0 ? min(*p.kv_len_ptr, p.Sk) : *p.kv_len_ptr) : p.Sk;
  const int tiles_total = (Sk + kBN - 1) / kBN;
  const int tiles_per = (tiles_total + p.nsplit - 1) / p.nsplit;
  const int tile0 = split * tiles_per, tile1 = min(tiles_total, tile0 + tiles_per);

  const T *qrow = reinterpret_cast<const T *>(p.q) + b * p.q_bs + (long long)(Sk - 1) * p.q_rs + h * D;
  const T *kb = reinterpret_cast<const T *>(p.k) + b * p.k_bs + h * D;
  const T *vb = reinterpret_cast<const T *>(p.v) + b * p.v_bs + h * D;
  const T *mb = p.mask ? reinterpret_cast<const T *>(p.mask) + b * p.mask_bs : nullptr;

  // every warp loads, waits for and consumes only its own 16 keys of each tile
  auto load_kv = [&](int n, int buf) {
    load_warp_rows<T, D>(k_s + buf * kTileBytes, kb, p.k_rs, n * kBN, Sk, warp, lane);
    load_warp_rows<T, D>(v_s + buf * kTileBytes, vb, p.v_rs, n * kBN, Sk, warp, lane);
    if (lane < 16) {
      const int jl = warp * 16 + lane, j = n * kBN + jl;
      mask_s[buf * kBN + jl] = (mb && j < Sk) ? to_f32<T>(mb[j]) * kLog2e : 0.f;
    }
  };
  for (int i = 0; i < kDecodeStages - 1; ++i) {
    if (tile0 + i < tile1) load_kv(tile0 + i, i);
    cp_async_commit();
  }

  // A fragments of the single query row (row 0 of the 16-row MMA tile; the other rows are zero)
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    qf[kk][0] = qf[kk][1] = qf[kk][2] = qf[kk][3] = 0u;
    if (g == 0) {
      qf[kk][0] = *reinterpret_cast<const uint32_t *>(qrow + kk * 16 + 2 * t);
      qf[kk][2] = *reinterpret_cast<const uint32_t *>(qrow + kk * 16 + 8 + 2 * t);
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const float sc = p.scale * kLog2e;

  for (int n = tile0; n < tile1; ++n) {
    const int buf = (n - tile0) % kDecodeStages;
    if (n + kDecodeStages - 1 < tile1) load_kv(n + kDecodeStages - 1, (buf + kDecodeStages - 1) % kDecodeStages);
    cp_async_commit();
    cp_async_wait<kDecodeStages - 1>();
    __syncwarp();
    const uint32_t kt = k_s + buf * kTileBytes, vt = v_s + buf * kTileBytes;
    // this warp's 16 keys of the tile: two 8-key n-tiles
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t kf[4];
      ldmatrix_x4(kf, kt + tile_off<D>(warp * 16 + (lane & 7) + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
      mma16816<T>(s[0], qf[kk], kf[0], kf[1]);
      mma16816<T>(s[1], qf[kk], kf[2], kf[3]);
    }
    // row 0 lives in elements 0,1 of lanes with g == 0; other rows are ignored (kept finite)
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int jl = warp * 16 + i * 8 + 2 * t + e, j = n * kBN + jl;
        float x = s[i][e] * sc + mask_s[buf * kBN + jl];
        if (j >= Sk) x = -INFINITY;
        s[i][e] = x;
        mx = fmaxf(mx, x);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx = __shfl_sync(0xffffffffu, mx, t);            // broadcast row 0's value (lanes 0..3 hold it)
    const float m_new = fmaxf(m_run, mx);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    const float corr = exp2f(m_run - m_use);
    float pr[2][2];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pr[i][e] = g == 0 ? exp2f(s[i][e] - m_use) : 0.f;
        sum += pr[i][e];
      }
    l_run = l_run * corr + sum;
    m_run = m_new;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr; o[i][1] *= corr; }
    uint32_t pf[4] = {pack2<T>(pr[0][0], pr[0][1]), 0u, pack2<T>(pr[1][0], pr[1][1]), 0u};
#pragma unroll
    for (int db = 0; db < D / 16; ++db) {
      uint32_t vf[4];
      ldmatrix_x4_trans(vf, vt + tile_off<D>(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), db * 2 + (lane >> 4)));
      mma16816<T>(o[2 * db], pf, vf[0], vf[1]);
      mma16816<T>(o[2 * db + 1], pf, vf[2], vf[3]);
    }
    __syncwarp();                // the buffer is refilled by this warp's next request
  }
  cp_async_wait<0>();

  // merge the four warps (each saw a quarter of every tile) -> one (m, l, o[D]) for this split
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  float *mine = red + warp * (D + 2);
  if (g == 0) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { mine[i * 8 + 2 * t] = o[i][0]; mine[i * 8 + 2 * t + 1] = o[i][1]; }
    if (t == 0) { mine[D] = m_run; mine[D + 1] = l_run; }
  }
  __syncthreads();
  float m_all = -INFINITY;
#pragma unroll
  for (int w = 0; w < 4; ++w) m_all = fmaxf(m_all, red[w * (D + 2) + D]);
  const float m_ref = m_all == -INFINITY ? 0.f : m_all;
  float l_all = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) l_all += red[w * (D + 2) + D + 1] * exp2f(red[w * (D + 2) + D] - m_ref);
  float acc = 0.f;   // thread d < D owns output dimension d
  if (threadIdx.x < D) {
#pragma unroll
    for (int w = 0; w < 4; ++w) acc += red[w * (D + 2) + threadIdx.x] * exp2f(red[w * (D + 2) + D] - m_ref);
  }
  T *out = reinterpret_cast<T *>(p.o) + b * p.o_bs + h * D;
  if (p.nsplit == 1) {
    if (threadIdx.x < D) out[threadIdx.x] = from_f32<T>(l_all > 0.f ? acc / l_all : 0.f);
    return;
  }
  const int bh = b * p.H + h;
  float *slot = p.scratch + ((size_t)bh * p.nsplit + split) * (D + 2);
  if (threadIdx.x < D) slot[threadIdx.x] = acc;
  if (threadIdx.x == 0) { slot[D] = m_all; slot[D + 1] = l_all; }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(p.counters + bh, 1);
    s_last = arrived == p.nsplit - 1;
    if (s_last) p.counters[bh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float *all = p.scratch + (size_t)bh * p.nsplit * (D + 2);
  float mm = -INFINITY;
  for (int sidx = 0; sidx < p.nsplit; ++sidx) mm = fmaxf(mm, __ldcg(all + sidx * (D + 2) + D));
  const float mref = mm == -INFINITY ? 0.f : mm;
  float ll = 0.f, oo = 0.f;
  for (int sidx = 0; sidx < p.nsplit; ++sidx) {
    const float w = exp2f(__ldcg(all + sidx * (D + 2) + D) - mref);
    ll += __ldcg(all + sidx * (D + 2) + D + 1) * w;
    if (threadIdx.x < D) oo += __ldcg(all + sidx * (D + 2) + threadIdx.x) * w;
  }
  if (threadIdx.x < D) out[threadIdx.x] = from_f32<T>(ll > 0.f ? oo / ll : 0.f);
}

template <typename T, int D> int launch_prefill(const AttnParams &p, cudaStream_t st) {
  constexpr size_t smem = 5 * (size_t)kBN * D * 2 + 2 * kBN * sizeof(float);
  auto kern = attention_prefill_kernel<T, D>;
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
  dim3 grid((p.Sq + kBM - 1) / kBM, p.H, p.B);
  launch_pdl(kern, grid, dim3(kThreads), smem, st, p);
  return check_launch("attention_prefill");
}

template <typename T, int D> int launch_decode(const AttnParams &p, cudaStream_t st) {
  constexpr size_t smem = 2 * kDecodeStages * (size_t)kBN * D * 2 + kDecodeStages * kBN * sizeof(float) +
                          4 * (D + 2) * sizeof(float);
  auto kern = attention_decode_kernel<T, D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return fail(EB_ECUDA, "attention_decode: cannot reserve %zu bytes of shared memory", smem);
    }
    configured[dev] = true;
  }
  dim3 grid(p.nsplit, p.H, p.B);
  launch_pdl(kern, grid, dim3(kThreads), smem, st, p);
  return check_launch("attention_decode");
}

int check_common(const char *name, const AttnParams &p, int head_dim, int dtype) {
  if (dtype != EB_F16 && dtype != EB_BF16) return fail(EB_EINVAL, "%s: fp16 or bf16 only (dtype %d)", name, dtype);
  if (head_dim != 64 && head_dim != 128) return fail(EB_EUNSUPPORTED, "%s: head_dim %d not supported (64 or 128)", name, head_dim);
  if (p.B < 0 || p.H < 0 || p.Sq < 0 || p.Sk < 0) return fail(EB_EINVAL, "%s: negative size", name);
  if (p.H > 65535 || p.B > 65535) return fail(EB_ELIMIT, "%s: batch and heads are limited to 65535", name);
  if (!p.q || !p.k || !p.v || !p.o) return fail(EB_EINVAL, "%s: null pointer", name);
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.o))
    return fail(EB_EINVAL, "%s: pointers must be 16-byte aligned", name);
  const long long strides[] = {p.q_bs, p.q_rs, p.k_bs, p.k_rs, p.v_bs, p.v_rs, p.o_bs, p.o_rs};
  for (long long s : strides)
    if (s % 8 != 0) return fail(EB_EINVAL, "%s: strides must be multiples of 8 elements", name);
  return EB_OK;
}

}  // namespace
}  // namespace eb

using namespace eb;

extern "C" int eb_attention_prefill(const void *q, const void *k, const void *v, void *out, const void *mask,
                                    long long q_batch_stride, long long q_row_stride, long long k_batch_stride,
                                    long long k_row_stride, long long v_batch_stride, long long v_row_stride,
                                    long long o_batch_stride, long long o_row_stride, long long mask_batch_stride,
                                    int batch, int heads, int q_len, int kv_len, int head_dim, int causal, float scale,
                                    int dtype, void *stream) {
  AttnParams p{};
  p.q = q; p.k = k; p.v = v; p.o = out; p.mask = mask;
  p.q_bs = q_batch_stride; p.q_rs = q_row_stride; p.k_bs = k_batch_stride; p.k_rs = k_row_stride;
  p.v_bs = v_batch_stride; p.v_rs = v_row_stride; p.o_bs = o_batch_stride; p.o_rs = o_row_stride;
  p.mask_bs = mask_batch_stride;
  p.B = batch; p.H = heads; p.Sq = q_len; p.Sk = kv_len; p.causal = causal; p.scale = scale; p.nsplit = 1;
  if (batch == 0 || heads == 0 || q_len == 0) return EB_OK;
  int rc = check_common("attention_prefill", p, head_dim, dtype);
  if (rc) return rc;
  EB_REQUIRE(kv_len >= q_len || !causal, "attention_prefill: causal attention needs kv_len >= q_len");
  EB_REQUIRE(kv_len > 0, "attention_prefill: kv_len must be positive");
  cudaStream_t st = as_stream(stream);
  if (dtype == EB_F16) return head_dim == 64 ? launch_prefill<__half, 64>(p, st) : launch_prefill<__half, 128>(p, st);
  return head_dim == 64 ? launch_prefill<__nv_bfloat16, 64>(p, st) : launch_prefill<__nv_bfloat16, 128>(p, st);
}

extern "C" size_t eb_attention_decode_scratch_bytes(int batch, int heads, int head_dim, int nsplit) {
  if (batch <= 0 || heads <= 0 || nsplit <= 1) return 0;
  return 64 * 1024 + (size_t)batch * heads * nsplit * (head_dim + 2) * sizeof(float);
}

extern "C" int eb_attention_decode(const void *q, const void *k, const void *v, void *out, const void *mask,
                                   long long q_batch_stride, long long q_row_stride, long long k_batch_stride,
                                   long long k_row_stride,
                                   long long v_batch_stride, long long v_row_stride, long long o_batch_stride,
                                   long long mask_batch_stride, int batch, int heads, int kv_len,
                                   const int32_t *kv_len_device, int head_dim, float scale, int dtype, int nsplit,
                                   void *scratch, size_t scratch_bytes, void *stream) {
  AttnParams p{};
  p.q = q; p.k = k; p.v = v; p.o = out; p.mask = mask;
  p.q_bs = q_batch_stride; p.q_rs = q_row_stride; p.k_bs = k_batch_stride; p.k_rs = k_row_stride;
  p.v_bs = v_batch_stride; p.v_rs = v_row_stride; p.o_bs = o_batch_stride; p.o_rs = 0;
  p.mask_bs = mask_batch_stride;
  p.B = batch; p.H = heads; p.Sq = 1; p.Sk = kv_len; p.kv_len_ptr = kv_len_device; p.causal = 0; p.scale = scale;
  p.nsplit = nsplit;
  if (batch == 0 || heads == 0) return EB_OK;
  int rc = check_common("attention_decode", p, head_dim, dtype);
  if (rc) return rc;
  EB_REQUIRE(nsplit >= 1 && nsplit <= 1024, "attention_decode: nsplit must be in [1, 1024]");
  EB_REQUIRE(kv_len > 0 || kv_len_device, "attention_decode: kv_len must be positive");
  if (nsplit > 1) {
    const size_t need = eb_attention_decode_scratch_bytes(batch, heads, head_dim, nsplit);
    EB_REQUIRE((size_t)batch * heads * sizeof(int) <= 64 * 1024, "attention_decode: batch*heads exceeds the counter capacity (16384)");
    EB_REQUIRE(scratch && scratch_bytes >= need && aligned16(scratch),
               "attention_decode: nsplit=%d needs a scratch of %zu bytes, zero-filled once", nsplit, need);
    p.counters = reinterpret_cast<int *>(scratch);
    p.scratch = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + 64 * 1024);
  }
  cudaStream_t st = as_stream(stream);
  if (dtype == EB_F16) return head_dim == 64 ? launch_decode<__half, 64>(p, st) : launch_decode<__half, 128>(p, st);
  return head_dim == 64 ? launch_decode<__nv_bfloat16, 64>(p, st) : launch_decode<__nv_bfloat16, 128>(p, st);
}

// ------------------------------------------------------------------------------------------------
// Generation-step attention for callers that must not allocate device memory
// ------------------------------------------------------------------------------------------------
// Some hosts of this library cannot call cudaMalloc on the serving path: a worker whose memory
// pool was sized and handed out once at start-up, code running inside a region where the
// allocator is locked, or an embedding that is only given raw pointers to tensors somebody
// else owns.  For them the split-KV scratch lives in the library image itself: a fixed array
// in device memory that every GPU loading the library carries until the process exits.
constexpr size_t kStaticScratchBytes = 8u << 20;   // 64 KB of counters + ~7.9 MB of partial results
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticScratchBytes];

extern "C" int eb_attention_decode_noalloc(const void *q, const void *k, const void *v, void *out, const void *mask,
                                           long long q_batch_stride, long long q_row_stride,
                                           long long k_batch_stride, long long k_row_stride,
                                           long long v_batch_stride, long long v_row_stride,
                                           long long o_batch_stride, long long mask_batch_stride, int batch,
                                           int heads, int kv_len, const int32_t *kv_len_device, int head_dim,
                                           float scale, int dtype, int nsplit, void *stream) {
  // In host code the array's name is only a handle for the runtime, not a device address; the
  // address is looked up once per device, with that device current, and remembered.  The
  // look-up and the one-time clearing of the counters run under a lock, so two host threads
  // making their first call on a device cannot both enqueue the clearing (the later one could
  // otherwise zero counters under the other thread's kernel).
  static void *device_ptr[64] = {};
  static std::mutex setup_lock;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return fail(EB_ECUDA, "attention_decode_noalloc: no usable current device");
  }
  const size_t need = eb_attention_decode_scratch_bytes(batch, heads, head_dim, nsplit);
  if (need > kStaticScratchBytes)
    return fail(EB_ELIMIT,
                "attention_decode_noalloc: batch %d x heads %d x nsplit %d needs %zu bytes of scratch, the built-in "
                "array holds %zu; lower nsplit or use eb_attention_decode with a caller-provided scratch",
                batch, heads, nsplit, need, (size_t)kStaticScratchBytes);
  if (need == 0)   // a single split uses no scratch: nothing to look up or clear
    return eb_attention_decode(q, k, v, out, mask, q_batch_stride, q_row_stride, k_batch_stride, k_row_stride,
                               v_batch_stride, v_row_stride, o_batch_stride, mask_batch_stride, batch, heads, kv_len,
                               kv_len_device, head_dim, scale, dtype, nsplit, nullptr, 0, stream);
  {
    std::lock_guard<std::mutex> guard(setup_lock);
    if (device_ptr[dev] == nullptr) {
      void *ptr = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_decode_scratch);
      if (e != cudaSuccess || ptr == nullptr) {
        cudaGetLastError();
        return fail(EB_ECUDA, "attention_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      }
      // The arrival counters at the head of the array must start at zero.  A freshly loaded image
      // is zero already; clearing them here also covers a process that reuses the device after an
      // aborted call.  (Stream-ordered, so this first call should not be inside a stream capture.)
      e = cudaMemsetAsync(ptr, 0, 64 * 1024, as_stream(stream));
      if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(EB_ECUDA, "attention_decode_noalloc: clearing the counters failed: %s", cudaGetErrorString(e));
      }
      device_ptr[dev] = ptr;
    }
  }
  return eb_attention_decode(q, k, v, out, mask, q_batch_stride, q_row_stride, k_batch_stride, k_row_stride,
                             v_batch_stride, v_row_stride, o_batch_stride, mask_batch_stride, batch, heads, kv_len,
                             kv_len_device, head_dim, scale, dtype, nsplit, device_ptr[dev], kStaticScratchBytes,
                             stream);
}
