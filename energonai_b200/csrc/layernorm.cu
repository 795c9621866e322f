// LayerNorm forward with optional fused residual / bias add.
//
// One CTA of 128 threads per row.  The row (after the optional adds) is loaded once in
// 16-byte vectors into fp32 registers; mean and the centred second moment are each one
// block reduction over the register copy (two-pass, so no cancellation), and the output is
// written once (statistics: one reduction of the sum and the sum of squares of the row shifted
// by its first element).  HBM traffic is therefore the algorithmic minimum: one read of every input
// operand and one write of every output.  Rows that do not fit the register budget, or that
// are not 16-byte aligned, take a three-pass variant that re-reads the operands.
#include "common.cuh"

namespace eb {
namespace {

constexpr int kThreads = 128;

template <typename T, int VEC> struct alignas(sizeof(T) * VEC > 16 ? 16 : sizeof(T) * VEC) Pack { T e[VEC]; };

// The row is kept in registers as the raw 16-byte packs that were loaded (half the registers of
// an fp32 copy for 16-bit inputs), and unpacked again in each of the three passes: more rows are
// in flight per SM, which is what a bandwidth-bound kernel with a two-reduction latency chain
// per row needs.  With fused operands the sum is formed once, rounded to the input type (that is
// what the residual stream stores) and kept as the pack.
// G threads cooperate on one row: G = 128 (the whole CTA, long rows) or G = 32 (one warp per row,
// four rows per CTA and no block-wide synchronisation, for rows that fit 32 lanes x MAXV packs).
// Mean and variance come from one reduction of (sum, sum of squares) of the row shifted by its
// first element, which keeps the single pass free of cancellation for the value ranges a
// residual stream has.
template <typename Tin, typename Tout, int MAXV, int G>
__global__ void __launch_bounds__(kThreads)
ln_cached_kernel(Tout *__restrict__ y, float *__restrict__ mean, float *__restrict__ invvar,
                 const Tin *__restrict__ x, const Tin *__restrict__ residual, const Tin *__restrict__ bias,
                 Tin *__restrict__ sum_out, const Tout *__restrict__ gamma, const Tout *__restrict__ beta,
                 long long n1, int n2, float eps) {
  constexpr int VEC = 16 / sizeof(Tin);
  using PI = Pack<Tin, VEC>;
  using PO = Pack<Tout, VEC>;
  __shared__ float scratch[2 * (kThreads / 32)];
  griddep_wait();
  griddep_launch();
  const int packs = n2 / VEC;
  const float inv_n = 1.f / (float)n2;
  const bool fused = residual != nullptr || bias != nullptr;
  constexpr int kRowsPerCta = kThreads / G;
  const int gtid = threadIdx.x % G;
  // every thread of a CTA runs the same number of iterations (the block reduction synchronises)
  for (long long row0 = (long long)blockIdx.x * kRowsPerCta; row0 < n1; row0 += (long long)gridDim.x * kRowsPerCta) {
    const long long row = row0 + threadIdx.x / G;
    const bool live = row < n1;
    const long long rsafe = live ? row : 0;
    const PI *xr = reinterpret_cast<const PI *>(x + rsafe * n2);
    const PI *rr = residual ? reinterpret_cast<const PI *>(residual + rsafe * n2) : nullptr;
    PI v[MAXV];
#pragma unroll
    for (int t = 0; t < MAXV; ++t) {
      const int p = gtid + t * G;
      if (p < packs) v[t] = xr[p];
    }
    if (fused) {
#pragma unroll
      for (int t = 0; t < MAXV; ++t) {
        const int p = gtid + t * G;
        if (p < packs) {
          float f[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) f[e] = to_f32<Tin>(v[t].e[e]);
          if (rr) {
            const PI r = rr[p];
#pragma unroll
            for (int e = 0; e < VEC; ++e) f[e] += to_f32<Tin>(r.e[e]);
          }
          if (bias) {
            const PI bb = reinterpret_cast<const PI *>(bias)[p];
#pragma unroll
            for (int e = 0; e < VEC; ++e) f[e] += to_f32<Tin>(bb.e[e]);
          }
#pragma unroll
          for (int e = 0; e < VEC; ++e) v[t].e[e] = from_f32<Tin>(f[e]);
          if (sum_out && live) reinterpret_cast<PI *>(sum_out + row * n2)[p] = v[t];
        }
      }
    } else if (sum_out) {
#pragma unroll
      for (int t = 0; t < MAXV; ++t) {
        const int p = gtid + t * G;
        if (p < packs && live) reinterpret_cast<PI *>(sum_out + row * n2)[p] = v[t];
      }
    }
    // shift by the row's first element (same value in every thread of the group)
    float pivot = to_f32<Tin>(v[0].e[0]);
    if (G == 32) {
      pivot = __shfl_sync(0xffffffffu, pivot, 0);
    } else {
      __syncthreads();
      if (threadIdx.x == 0) scratch[0] = pivot;
      __syncthreads();
      pivot = scratch[0];
    }
    float s = 0.f, q = 0.f;
#pragma unroll
    for (int t = 0; t < MAXV; ++t) {
      if (gtid + t * G < packs) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) { const float d = to_f32<Tin>(v[t].e[e]) - pivot; s += d; q += d * d; }
      }
    }
    if (G == 32) {
      s = warp_sum(s);
      q = warp_sum(q);
    } else {
      s = warp_sum(s);
      q = warp_sum(q);
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
      __syncthreads();
      if (lane == 0) { scratch[warp] = s; scratch[kThreads / 32 + warp] = q; }
      __syncthreads();
      s = lane < kThreads / 32 ? scratch[lane] : 0.f;
      q = lane < kThreads / 32 ? scratch[kThreads / 32 + lane] : 0.f;
      s = warp_sum(s);
      q = warp_sum(q);
    }
    const float ms = s * inv_n;                       // mean of the shifted row
    const float mu = pivot + ms;
    const float var = fmaxf(q * inv_n - ms * ms, 0.f);
    const float iv = rsqrtf(var + eps);
    PO *yr = reinterpret_cast<PO *>(y + row * n2);
#pragma unroll
    for (int t = 0; t < MAXV; ++t) {
      const int p = gtid + t * G;
      if (p < packs && live) {
        PO o;
        if (gamma) {
          const PO g = reinterpret_cast<const PO *>(gamma)[p], bt = reinterpret_cast<const PO *>(beta)[p];
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            o.e[e] = from_f32<Tout>(to_f32<Tout>(g.e[e]) * ((to_f32<Tin>(v[t].e[e]) - mu) * iv) + to_f32<Tout>(bt.e[e]));
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) o.e[e] = from_f32<Tout>((to_f32<Tin>(v[t].e[e]) - mu) * iv);
        }
        yr[p] = o;
      }
    }
    if (gtid == 0 && live) {
      if (mean) mean[row] = mu;
      if (invvar) invvar[row] = iv;
    }
  }
}

// Any n2 / alignment: element-wise, operands re-read in each of the three passes.
template <typename Tin, typename Tout>
__global__ void __launch_bounds__(kThreads)
ln_generic_kernel(Tout *__restrict__ y, float *__restrict__ mean, float *__restrict__ invvar,
                  const Tin *__restrict__ x, const Tin *__restrict__ residual, const Tin *__restrict__ bias,
                  Tin *__restrict__ sum_out, const Tout *__restrict__ gamma, const Tout *__restrict__ beta,
                  long long n1, int n2, float eps) {
  __shared__ float scratch[kThreads / 32];
  griddep_wait();
  griddep_launch();
  const float inv_n = 1.f / (float)n2;
  for (long long row = blockIdx.x; row < n1; row += gridDim.x) {
    const Tin *xr = x + row * n2;
    const Tin *rr = residual ? residual + row * n2 : nullptr;
    auto value = [&](int i) {
      float t = to_f32<Tin>(xr[i]);
      if (rr) t += to_f32<Tin>(rr[i]);
      if (bias) t += to_f32<Tin>(bias[i]);
      return sum_out ? to_f32<Tin>(from_f32<Tin>(t)) : t;
    };
    float s = 0.f;
    for (int i = threadIdx.x; i < n2; i += kThreads) s += value(i);
    const float mu = block_sum<kThreads>(s, scratch) * inv_n;
    float q = 0.f;
    for (int i = threadIdx.x; i < n2; i += kThreads) { const float d = value(i) - mu; q += d * d; }
    const float iv = rsqrtf(block_sum<kThreads>(q, scratch) * inv_n + eps);
    for (int i = threadIdx.x; i < n2; i += kThreads) {
      const float t = value(i);
      float o = (t - mu) * iv;
      if (gamma) o = to_f32<Tout>(gamma[i]) * o + to_f32<Tout>(beta[i]);
      y[row * n2 + i] = from_f32<Tout>(o);
    }
    if (sum_out) {
      __syncthreads();   // all reads of x/residual for this row are done (sum_out may alias them)
      for (int i = threadIdx.x; i < n2; i += kThreads) {
        float t = to_f32<Tin>(xr[i]);
        if (rr) t += to_f32<Tin>(rr[i]);
        if (bias) t += to_f32<Tin>(bias[i]);
        sum_out[row * n2 + i] = from_f32<Tin>(t);
      }
    }
    if (threadIdx.x == 0) {
      if (mean) mean[row] = mu;
      if (invvar) invvar[row] = iv;
    }
  }
}

template <typename Tin, typename Tout>
int launch_ln(void *y, float *mean, float *invvar, const void *x, const void *residual, const void *bias,
              void *sum_out, const void *gamma, const void *beta, long long n1, int n2, float eps, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(Tin);
  const long long cap = (long long)sm_count() * 32;
  const int grid = (int)(n1 < cap ? n1 : cap);
  const bool vec_ok = n2 % VEC == 0 && aligned16(x) && aligned16(y) && aligned16(residual) && aligned16(bias) &&
                      aligned16(sum_out) && aligned16(gamma) && aligned16(beta) &&
                      ((size_t)n2 * sizeof(Tout)) % 16 == 0;
  const int packs = n2 / VEC;
#define EB_LN_ARGS (Tout *)y, mean, invvar, (const Tin *)x, (const Tin *)residual, (const Tin *)bias, (Tin *)sum_out, \
                   (const Tout *)gamma, (const Tout *)beta, n1, n2, eps
  if (vec_ok && packs <= 32 * 8 && n1 >= 64) {
    // short rows, many of them: one warp per row
    const int need = (packs + 31) / 32;
    const long long ctas = (n1 + 3) / 4;
    const int g4 = (int)(ctas < cap ? ctas : cap);
    if (need <= 1) launch_pdl(ln_cached_kernel<Tin, Tout, 1, 32>, dim3(g4), dim3(kThreads), 0, st, EB_LN_ARGS);
    else if (need <= 2) launch_pdl(ln_cached_kernel<Tin, Tout, 2, 32>, dim3(g4), dim3(kThreads), 0, st, EB_LN_ARGS);
    else if (need <= 4) launch_pdl(ln_cached_kernel<Tin, Tout, 4, 32>, dim3(g4), dim3(kThreads), 0, st, EB_LN_ARGS);
    else launch_pdl(ln_cached_kernel<Tin, Tout, 8, 32>, dim3(g4), dim3(kThreads), 0, st, EB_LN_ARGS);
  } else if (vec_ok && packs <= kThreads * 16) {
    const int need = (packs + kThreads - 1) / kThreads;
    if (need <= 1) launch_pdl(ln_cached_kernel<Tin, Tout, 1, kThreads>, dim3(grid), dim3(kThreads), 0, st, EB_LN_ARGS);
    else if (need <= 2) launch_pdl(ln_cached_kernel<Tin, Tout, 2, kThreads>, dim3(grid), dim3(kThreads), 0, st, EB_LN_ARGS);
    else if (need <= 4) launch_pdl(ln_cached_kernel<Tin, Tout, 4, kThreads>, dim3(grid), dim3(kThreads), 0, st, EB_LN_ARGS);
    else if (need <= 6) launch_pdl(ln_cached_kernel<Tin, Tout, 6, kThreads>, dim3(grid), dim3(kThreads), 0, st, EB_LN_ARGS);
    else if (need <= 8) launch_pdl(ln_cached_kernel<Tin, Tout, 8, kThreads>, dim3(grid), dim3(kThreads), 0, st, EB_LN_ARGS);
    else launch_pdl(ln_cached_kernel<Tin, Tout, 16, kThreads>, dim3(grid), dim3(kThreads), 0, st, EB_LN_ARGS);
  } else {
    launch_pdl(ln_generic_kernel<Tin, Tout>, dim3(grid), dim3(kThreads), 0, st, EB_LN_ARGS);
  }
#undef EB_LN_ARGS
  return check_launch("layer_norm_fwd");
}

template <typename Tin>
int dispatch_out(int out_dtype, void *y, float *mean, float *invvar, const void *x, const void *residual,
                 const void *bias, void *sum_out, const void *gamma, const void *beta, long long n1, int n2, float eps,
                 cudaStream_t st) {
  if (out_dtype == EB_F32) return launch_ln<Tin, float>(y, mean, invvar, x, residual, bias, sum_out, gamma, beta, n1, n2, eps, st);
  if (out_dtype == EB_F16) return launch_ln<Tin, __half>(y, mean, invvar, x, residual, bias, sum_out, gamma, beta, n1, n2, eps, st);
  return launch_ln<Tin, __nv_bfloat16>(y, mean, invvar, x, residual, bias, sum_out, gamma, beta, n1, n2, eps, st);
}

}  // namespace
}  // namespace eb

extern "C" int eb_layer_norm_fwd(void *y, float *mean, float *invvar, const void *x, const void *residual,
                                 const void *bias, void *sum_out, const void *gamma, const void *beta, int64_t n1,
                                 int n2, double eps, int in_dtype, int out_dtype, void *stream) {
  using namespace eb;
  EB_REQUIRE(dtype_ok(in_dtype) && dtype_ok(out_dtype), "layer_norm_fwd: bad dtype %d/%d", in_dtype, out_dtype);
  EB_REQUIRE(n1 >= 0 && n2 >= 0, "layer_norm_fwd: negative size");
  if (n1 == 0 || n2 == 0) return EB_OK;
  EB_REQUIRE(y && x, "layer_norm_fwd: null input or output");
  EB_REQUIRE((gamma == nullptr) == (beta == nullptr), "layer_norm_fwd: gamma and beta must both be given or both be NULL");
  cudaStream_t st = as_stream(stream);
  const float e = (float)eps;
  if (in_dtype == EB_F32) return dispatch_out<float>(out_dtype, y, mean, invvar, x, residual, bias, sum_out, gamma, beta, n1, n2, e, st);
  if (in_dtype == EB_F16) return dispatch_out<__half>(out_dtype, y, mean, invvar, x, residual, bias, sum_out, gamma, beta, n1, n2, e, st);
  return dispatch_out<__nv_bfloat16>(out_dtype, y, mean, invvar, x, residual, bias, sum_out, gamma, beta, n1, n2, e, st);
}
