// In-place masked softmax over attention scores [batch, heads, S, S].
//
// One warp per query row.  The visible prefix of the row (keys j <= i under the causal
// mask, j < real_len under the key-length mask) is loaded once in 16-byte vectors and kept
// in registers, reduced with warp shuffles (max, then sum of exp), and the whole row is
// written back once: probabilities for visible keys, exact zeros for masked keys.  Only
// the visible prefix is ever read, so a causal row i costs (i+1) reads + S writes.
// Rows longer than the register budget take a variant that re-reads the row from memory.
#include <cfloat>

#include "common.cuh"

namespace eb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <typename T, int VEC> struct alignas(sizeof(T) * VEC > 16 ? 16 : sizeof(T) * VEC) Pack { T e[VEC]; };

// VPL = packs cached per lane (0: no caching, re-read).
template <typename T, int VEC, int VPL>
__global__ void __launch_bounds__(kThreads, (VPL * VEC <= 16 ? 4 : (VPL * VEC <= 32 ? 3 : 2)))
softmax_kernel(T *__restrict__ scores, const int32_t *__restrict__ real_len, int B, int S, int H, int flags,
               float scale) {
  using P = Pack<T, VEC>;
  const int lane = threadIdx.x & 31;
  // blockIdx.y = batch entry; rows of one batch entry (head, query) are walked with 32-bit
  // arithmetic (64-bit divisions per row were a visible part of the row's latency chain)
  const int b = blockIdx.y;
  const unsigned rows_b = (unsigned)H * (unsigned)S;
  const unsigned warp0 = blockIdx.x * kWarps + (threadIdx.x >> 5), nwarps = gridDim.x * kWarps;
  const int packs_row = S / VEC;   // S % VEC == 0 on this path
  int len = real_len[b];
  len = len < 0 ? 0 : (len > S ? S : len);
  if constexpr (VPL > 0) {
    // Only rows that are rewritten are walked (query i < real_len unless ALLROWS): live row r of
    // this batch entry is (head r / live_q, query r % live_q).  With one row at a time the
    // load -> max -> exp -> sum -> store chain left each warp with memory traffic in flight only
    // about half of the time, and the kernel ran at half of the copy bandwidth: rows are
    // pipelined (see the loop below).
    const unsigned live_q = (flags & EB_SM_ALLROWS) ? (unsigned)S : (unsigned)len;
    const unsigned live = (unsigned)H * live_q;
    struct Row { P *rp; int nvis, packs_vis; bool on; };
    auto locate = [&](unsigned r) {
      Row w;
      w.on = r < live;
      const unsigned rr = w.on ? r : 0u;
      const unsigned h = live_q ? rr / live_q : 0u;
      const int i = (int)(rr - h * live_q);
      int nvis = S;
      if (flags & EB_SM_CAUSAL) nvis = min(nvis, i + 1);
      if (flags & EB_SM_KEYLEN) nvis = min(nvis, len);
      w.nvis = w.on ? nvis : 0;
      w.packs_vis = (w.nvis + VEC - 1) / VEC;
      w.rp = reinterpret_cast<P *>(scores + ((long long)b * rows_b + (long long)h * S + i) * S);
      return w;
    };
    // The kernel is bound by instruction issue, not by memory, unless the per-element work is
    // kept minimal: a pack is converted and scaled once, the keys of the one pack that
    // straddles the end of the visible prefix are set to -inf there (so the later phases need
    // no comparisons: exp(-inf - max) is an exact 0), every exponential is evaluated once and
    // kept in its register, and packs that lie wholly behind the prefix are stored as zeros
    // without any arithmetic.
    auto finish = [&](const Row &w, const P (&raw)[VPL > 0 ? VPL : 1]) {
      float x[VPL > 0 ? VPL : 1][VEC];
      float mx = -FLT_MAX;
#pragma unroll
      for (int t = 0; t < VPL; ++t) {
        const int v = lane + 32 * t;
        if (v < w.packs_vis) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) x[t][e] = to_f32<T>(raw[t].e[e]) * scale;
          if ((v + 1) * VEC > w.nvis) {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              if (v * VEC + e >= w.nvis) x[t][e] = -INFINITY;
          }
#pragma unroll
          for (int e = 0; e < VEC; ++e) mx = fmaxf(mx, x[t][e]);
        }
      }
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int t = 0; t < VPL; ++t) {
        if (lane + 32 * t < w.packs_vis) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            x[t][e] = __expf(x[t][e] - mx);
            sum += x[t][e];
          }
        }
      }
      sum = warp_sum(sum);
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
      for (int t = 0; t < VPL; ++t) {
        const int v = lane + 32 * t;
        if (v < packs_row) {
          P out;
          if (v < w.packs_vis) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) out.e[e] = from_f32<T>(x[t][e] * inv);
          } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) out.e[e] = from_f32<T>(0.f);
          }
          w.rp[v] = out;
        }
      }
    };
    // software pipeline: the packs of the warp's NEXT row are requested before the current row
    // is reduced, so every warp has loads in flight all the time
    Row cur = locate(warp0);
    P raw_cur[VPL > 0 ? VPL : 1];
#pragma unroll
    for (int t = 0; t < VPL; ++t)
      if (lane + 32 * t < cur.packs_vis) raw_cur[t] = cur.rp[lane + 32 * t];
    for (unsigned r = warp0; r < live; r += nwarps) {
      const Row nxt = locate(r + nwarps);
      P raw_nxt[VPL > 0 ? VPL : 1];
#pragma unroll
      for (int t = 0; t < VPL; ++t)
        if (lane + 32 * t < nxt.packs_vis) raw_nxt[t] = nxt.rp[lane + 32 * t];
      finish(cur, raw_cur);
      cur = nxt;
#pragma unroll
      for (int t = 0; t < VPL; ++t) raw_cur[t] = raw_nxt[t];
    }
  } else {
  for (unsigned rb = warp0; rb < rows_b; rb += nwarps) {
    const int i = (int)(rb % (unsigned)S);
    const long long row = (long long)b * rows_b + rb;
    if (i >= len && !(flags & EB_SM_ALLROWS)) continue;
    int nvis = S;
    if (flags & EB_SM_CAUSAL) nvis = min(nvis, i + 1);
    if (flags & EB_SM_KEYLEN) nvis = min(nvis, len);
    P *rp = reinterpret_cast<P *>(scores + row * S);
    const int packs_vis = (nvis + VEC - 1) / VEC;
    {
      float mx = -FLT_MAX;
      for (int v = lane; v < packs_vis; v += 32) {
        P c = rp[v];
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          if (v * VEC + e < nvis) mx = fmaxf(mx, to_f32<T>(c.e[e]) * scale);
      }
      mx = warp_max(mx);
      float sum = 0.f;
      for (int v = lane; v < packs_vis; v += 32) {
        P c = rp[v];
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          if (v * VEC + e < nvis) sum += __expf(to_f32<T>(c.e[e]) * scale - mx);
      }
      sum = warp_sum(sum);
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      for (int v = lane; v < packs_row; v += 32) {
        P c, out;
        if (v < packs_vis) c = rp[v];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float p = 0.f;
          if (v < packs_vis && v * VEC + e < nvis) p = __expf(to_f32<T>(c.e[e]) * scale - mx) * inv;
          out.e[e] = from_f32<T>(p);
        }
        rp[v] = out;
      }
    }
  }
  }
}

template <typename T>
int launch_softmax(void *scores, const int32_t *real_len, int B, int S, int H, int flags, float scale,
                   cudaStream_t st) {
  const long long rows_b = (long long)H * S;
  long long gx = (rows_b + kWarps - 1) / kWarps;
  const long long cap = ((long long)sm_count() * 32 + B - 1) / B;
  if (gx > cap) gx = cap;
  if (gx < 1) gx = 1;
  const dim3 grid((unsigned)gx, (unsigned)B);
  constexpr int N = 16 / sizeof(T);
  T *p = reinterpret_cast<T *>(scores);
#define EB_SM_LAUNCH(VEC, VPL) \
  softmax_kernel<T, VEC, VPL><<<grid, kThreads, 0, st>>>(p, real_len, B, S, H, flags, scale)
  if (S % N == 0 && aligned16(scores)) {
    const int packs = S / N;
    if (packs <= 32) EB_SM_LAUNCH(N, 1);
    else if (packs <= 64) EB_SM_LAUNCH(N, 2);
    else if (packs <= 128) EB_SM_LAUNCH(N, 4);
    else if (packs <= 256) EB_SM_LAUNCH(N, 8);
    else EB_SM_LAUNCH(N, 0);
  } else {
    if (S <= 32) EB_SM_LAUNCH(1, 1);
    else if (S <= 128) EB_SM_LAUNCH(1, 4);
    else if (S <= 512) EB_SM_LAUNCH(1, 16);
    else EB_SM_LAUNCH(1, 0);
  }
#undef EB_SM_LAUNCH
  return check_launch("scale_mask_softmax");
}

}  // namespace
}  // namespace eb

extern "C" int eb_scale_mask_softmax(void *scores, const int32_t *real_seq_len, int batch, int seq_len, int head_num,
                                     int dtype, int flags, float scale, void *stream) {
  using namespace eb;
  EB_REQUIRE(dtype_ok(dtype), "scale_mask_softmax: bad dtype %d", dtype);
  EB_REQUIRE(batch >= 0 && seq_len >= 0 && head_num >= 0, "scale_mask_softmax: negative size");
  EB_REQUIRE(batch <= 65535 && (long long)head_num * seq_len < (1ll << 31), "scale_mask_softmax: batch > 65535 or heads*seq too large");
  EB_REQUIRE((flags & ~7) == 0, "scale_mask_softmax: unknown flag bits 0x%x", flags);
  if ((long long)batch * seq_len * head_num == 0) return EB_OK;
  EB_REQUIRE(scores && real_seq_len, "scale_mask_softmax: null pointer");
  cudaStream_t st = as_stream(stream);
  if (dtype == EB_F32) return launch_softmax<float>(scores, real_seq_len, batch, seq_len, head_num, flags, scale, st);
  if (dtype == EB_F16) return launch_softmax<__half>(scores, real_seq_len, batch, seq_len, head_num, flags, scale, st);
  return launch_softmax<__nv_bfloat16>(scores, real_seq_len, batch, seq_len, head_num, flags, scale, st);
}
