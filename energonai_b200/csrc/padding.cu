// Padding-offset construction and the (un)padding / head-transpose copies.
//
// All copies are organised as one warp per token row: the warp resolves the row's
// source/destination once (a prefix sum or a binary search that every lane performs on
// the same addresses, i.e. one broadcast load per step), then streams the row in 16-byte
// units, lanes striding across the row so that every warp-level access is a run of
// consecutive 16-byte vectors.  Rows whose byte length or base alignment is not a multiple
// of 16 take the same kernels instantiated on a 4- or 2-byte unit.  Zero rows of padded
// outputs are written by the same kernel, so no separate memset pass exists.
#include "common.cuh"

namespace eb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ int clamp_len(int v, int hi) { return v < 0 ? 0 : (v > hi ? hi : v); }

template <typename U> __device__ __forceinline__ U zero_unit();
template <> __device__ __forceinline__ uint4 zero_unit<uint4>() { return make_uint4(0, 0, 0, 0); }
template <> __device__ __forceinline__ uint32_t zero_unit<uint32_t>() { return 0u; }
template <> __device__ __forceinline__ uint16_t zero_unit<uint16_t>() { return 0; }

// Copy (or zero, when src == nullptr) `units` units of one row; whole warp participates.
template <typename U>
__device__ __forceinline__ void warp_copy_row(U *__restrict__ dst, const U *__restrict__ src, int units, int lane) {
  if (src != nullptr) {
    int i = lane;
    for (; i + 96 < units; i += 128) {   // four independent loads in flight per lane
      U a = src[i], b = src[i + 32], c = src[i + 64], d = src[i + 96];
      dst[i] = a; dst[i + 32] = b; dst[i + 64] = c; dst[i + 96] = d;
    }
    for (; i < units; i += 32) dst[i] = src[i];
  } else {
    for (int i = lane; i < units; i += 32) dst[i] = zero_unit<U>();
  }
}

// Largest k in [0, valid) with k + off[k] <= pos, or -1.  k + off[k] is strictly increasing.
__device__ __forceinline__ int find_packed(const int32_t *__restrict__ off, int valid, int pos) {
  int lo = 0, hi = valid;   // invariant: answer in [lo-1, hi-1]
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (mid + __ldg(off + mid) <= pos) lo = mid + 1; else hi = mid;
  }
  return lo - 1;
}

// ---- build_padding_offsets --------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
build_offsets_kernel(const int32_t *__restrict__ lens, int batch, int max_len, int32_t *__restrict__ valid_word_num,
                     int32_t *__restrict__ off) {
  __shared__ int warp_part[kWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int b = blockIdx.x; b <= batch; b += gridDim.x) {
    // start = sum of lens[0..b): block-wide integer reduction
    int part = 0;
    for (int j = threadIdx.x; j < b; j += kThreads) part += clamp_len(lens[j], max_len);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    __syncthreads();
    if (lane == 0) warp_part[warp] = part;
    __syncthreads();
    int start = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) start += warp_part[w];
    if (b == batch) {   // the extra iteration b == batch yields the total
      if (threadIdx.x == 0) valid_word_num[0] = start;
    } else {
      const int len = clamp_len(lens[b], max_len);
      const int pads_before = b * max_len - start;
      for (int j = threadIdx.x; j < len; j += kThreads) off[start + j] = pads_before;
    }
  }
}

// ---- remove / rebuild padding -------------------------------------------------------------
template <typename U>
__global__ void __launch_bounds__(kThreads)
remove_padding_kernel(const U *__restrict__ src, U *__restrict__ tgt, const int32_t *__restrict__ tmp_off,
                      int32_t *__restrict__ off_out, int valid, int units) {
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * kWarps + (threadIdx.x >> 5), nwarps = gridDim.x * kWarps;
  for (int k = warp0; k < valid; k += nwarps) {
    const int o = __ldg(tmp_off + k);
    if (lane == 0) off_out[k] = o;
    warp_copy_row(tgt + (size_t)k * units, src + (size_t)(k + o) * units, units, lane);
  }
}

template <typename U, bool kZeroFill>
__global__ void __launch_bounds__(kThreads)
rebuild_padding_kernel(const U *__restrict__ src, U *__restrict__ tgt, const int32_t *__restrict__ off, int valid,
                       int units, int total_rows) {
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * kWarps + (threadIdx.x >> 5), nwarps = gridDim.x * kWarps;
  if (kZeroFill) {
    for (int p = warp0; p < total_rows; p += nwarps) {
      const int k = find_packed(off, valid, p);
      const bool hit = k >= 0 && k + __ldg(off + k) == p;
      warp_copy_row(tgt + (size_t)p * units, hit ? src + (size_t)k * units : (const U *)nullptr, units, lane);
    }
  } else {
    for (int k = warp0; k < valid; k += nwarps) {
      const int p = k + __ldg(off + k);
      if (p < total_rows) warp_copy_row(tgt + (size_t)p * units, src + (size_t)k * units, units, lane);
    }
  }
}

// ---- [valid, H, D] <-> [B, H, S, D] -------------------------------------------------------
// One warp per token; the token's H chunks of `du` units go to / come from H places.
template <typename U>
__device__ __forceinline__ void warp_scatter_heads(U *__restrict__ buf, const U *__restrict__ packed_row, int b, int s,
                                                   int H, int S, int du, int lane) {
  const int row_units = H * du;
  for (int i = lane; i < row_units; i += 32) {
    const int h = i / du, d = i - h * du;
    const U v = packed_row ? packed_row[i] : zero_unit<U>();
    buf[((size_t)(b * H + h) * S + s) * du + d] = v;
  }
}

template <typename U, bool kZeroFill>
__global__ void __launch_bounds__(kThreads)
transpose_rebuild_kernel(const U *__restrict__ Q, const U *__restrict__ K, const U *__restrict__ V,
                         U *__restrict__ qb, U *__restrict__ kb, U *__restrict__ vb, int B, int S, int H, int du,
                         int valid, const int32_t *__restrict__ off) {
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * kWarps + (threadIdx.x >> 5), nwarps = gridDim.x * kWarps;
  const U *in = blockIdx.y == 0 ? Q : (blockIdx.y == 1 ? K : V);
  U *out = blockIdx.y == 0 ? qb : (blockIdx.y == 1 ? kb : vb);
  const size_t row_units = (size_t)H * du;
  if (kZeroFill) {
    const int total = B * S;
    for (int p = warp0; p < total; p += nwarps) {
      const int k = find_packed(off, valid, p);
      const bool hit = k >= 0 && k + __ldg(off + k) == p;
      warp_scatter_heads(out, hit ? in + k * row_units : (const U *)nullptr, p / S, p % S, H, S, du, lane);
    }
  } else {
    for (int k = warp0; k < valid; k += nwarps) {
      const int p = k + __ldg(off + k);
      if (p < B * S) warp_scatter_heads(out, in + k * row_units, p / S, p % S, H, S, du, lane);
    }
  }
}

template <typename U>
__global__ void __launch_bounds__(kThreads)
transpose_remove_kernel(const U *__restrict__ src, U *__restrict__ dst, int valid, int B, int S, int H, int du,
                        const int32_t *__restrict__ off) {
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * kWarps + (threadIdx.x >> 5), nwarps = gridDim.x * kWarps;
  const int row_units = H * du;
  for (int k = warp0; k < valid; k += nwarps) {
    const int p = k + __ldg(off + k);
    if (p >= B * S) continue;
    const int b = p / S, s = p % S;
    U *out = dst + (size_t)k * row_units;
    for (int i = lane; i < row_units; i += 32) {
      const int h = i / du, d = i - h * du;
      out[i] = src[((size_t)(b * H + h) * S + s) * du + d];
    }
  }
}

// ---- Turbo-style transposes driven by seq_lens ---------------------------------------------
// Exclusive prefix sums of the (clamped) lengths into shared memory; prefix[B] = total.
__device__ __forceinline__ void block_prefix_lens(const int32_t *__restrict__ lens, int B, int max_len, int *prefix) {
  // B is small (a batch); a single thread walks it after a cooperative load.
  for (int j = threadIdx.x; j < B; j += blockDim.x) prefix[j + 1] = clamp_len(lens[j], max_len);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    prefix[0] = 0;
    for (int j = 1; j <= B; ++j) { run += prefix[j]; prefix[j] = run; }
  }
  __syncthreads();
}

template <typename U>
__global__ void __launch_bounds__(kThreads)
transpose_pad_kernel(const U *__restrict__ src, U *__restrict__ dst, int B, int S, const int32_t *__restrict__ lens,
                     int H, int du) {
  extern __shared__ int prefix[];
  block_prefix_lens(lens, B, S, prefix);
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * kWarps + (threadIdx.x >> 5), nwarps = gridDim.x * kWarps;
  const size_t row_units = (size_t)H * du;
  for (int p = warp0; p < B * S; p += nwarps) {
    const int b = p / S, s = p % S;
    const int len = prefix[b + 1] - prefix[b];
    warp_scatter_heads(dst, s < len ? src + (size_t)(prefix[b] + s) * row_units : (const U *)nullptr, b, s, H, S, du,
                       lane);
  }
}

template <typename U>
__global__ void __launch_bounds__(kThreads)
transpose_depad_kernel(const U *__restrict__ src, U *__restrict__ dst, int B, int sum_seq, int S,
                       const int32_t *__restrict__ lens, int H, int du) {
  extern __shared__ int prefix[];
  block_prefix_lens(lens, B, S, prefix);
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * kWarps + (threadIdx.x >> 5), nwarps = gridDim.x * kWarps;
  const int row_units = H * du;
  const int total = prefix[B];
  for (int r = warp0; r < sum_seq; r += nwarps) {
    U *out = dst + (size_t)r * row_units;
    if (r >= total) {
      warp_copy_row(out, (const U *)nullptr, row_units, lane);
      continue;
    }
    int lo = 0, hi = B;   // largest b with prefix[b] <= r (skips empty sequences correctly)
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (prefix[mid] <= r) lo = mid; else hi = mid;
    }
    const int b = lo, s = r - prefix[b];
    for (int i = lane; i < row_units; i += 32) {
      const int h = i / du, d = i - h * du;
      out[i] = src[((size_t)(b * H + h) * S + s) * du + d];
    }
  }
}

// ---- host side ------------------------------------------------------------------------------
inline int grid_for_rows(long long rows) {
  long long g = (rows + kWarps - 1) / kWarps;
  long long cap = (long long)sm_count() * 16;   // 16 CTAs of 256 threads cover 2 full waves per SM
  if (g > cap) g = cap;
  return g < 1 ? 1 : (int)g;
}

// Unit size in bytes usable for rows of `row_bytes` bytes at these pointers.
inline int pick_unit(size_t row_bytes, int esize, std::initializer_list<const void *> ptrs) {
  bool ok = row_bytes % 16 == 0;
  for (const void *p : ptrs) ok = ok && aligned16(p);
  return ok ? 16 : esize;
}

#define EB_DISPATCH_UNIT(unit, ...)                                     \
  do {                                                                  \
    if ((unit) == 16) { using U = uint4; __VA_ARGS__; }                 \
    else if ((unit) == 4) { using U = uint32_t; __VA_ARGS__; }          \
    else { using U = uint16_t; __VA_ARGS__; }                           \
  } while (0)

}  // namespace
}  // namespace eb

using namespace eb;

extern "C" int eb_build_padding_offsets(const int32_t *seq_lens, int batch, int max_seq_len, int32_t *valid_word_num,
                                        int32_t *tmp_mask_offset, void *stream) {
  EB_REQUIRE(seq_lens && valid_word_num && tmp_mask_offset, "build_padding_offsets: null pointer");
  EB_REQUIRE(batch >= 0 && max_seq_len >= 0, "build_padding_offsets: negative size");
  EB_REQUIRE((long long)batch * max_seq_len < (1ll << 31), "build_padding_offsets: batch*max_seq_len overflows int32");
  int grid = batch + 1 < sm_count() * 8 ? batch + 1 : sm_count() * 8;
  build_offsets_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(seq_lens, batch, max_seq_len, valid_word_num,
                                                                 tmp_mask_offset);
  return check_launch("build_padding_offsets");
}

extern "C" int eb_remove_padding(const void *src, void *tgt, const int32_t *tmp_mask_offset, int32_t *mask_offset,
                                 int valid, int n, int dtype, void *stream) {
  EB_REQUIRE(dtype_ok(dtype), "remove_padding: bad dtype %d", dtype);
  EB_REQUIRE(valid >= 0 && n >= 0, "remove_padding: negative size");
  if (valid == 0) return EB_OK;
  EB_REQUIRE(src && tgt && tmp_mask_offset && mask_offset, "remove_padding: null pointer");
  const int e = dtype_size(dtype);
  const int unit = pick_unit((size_t)n * e, e, {src, tgt});
  const int units = n * e / unit;
  EB_DISPATCH_UNIT(unit, (remove_padding_kernel<U><<<grid_for_rows(valid), kThreads, 0, as_stream(stream)>>>(
                             (const U *)src, (U *)tgt, tmp_mask_offset, mask_offset, valid, units)));
  return check_launch("remove_padding");
}

extern "C" int eb_rebuild_padding(const void *src, void *tgt, const int32_t *mask_offset, int valid, int n, int batch,
                                  int max_seq_len, int dtype, int zero_fill, void *stream) {
  EB_REQUIRE(dtype_ok(dtype), "rebuild_padding: bad dtype %d", dtype);
  EB_REQUIRE(valid >= 0 && n >= 0 && batch >= 0 && max_seq_len >= 0, "rebuild_padding: negative size");
  const long long total = (long long)batch * max_seq_len;
  EB_REQUIRE(total < (1ll << 31) && valid <= total, "rebuild_padding: valid=%d exceeds batch*max_seq_len=%lld", valid, total);
  if (total == 0 || n == 0 || (valid == 0 && !zero_fill)) return EB_OK;
  EB_REQUIRE(tgt && (valid == 0 || (src && mask_offset)), "rebuild_padding: null pointer");
  const int e = dtype_size(dtype);
  const int unit = pick_unit((size_t)n * e, e, {src, tgt});
  const int units = n * e / unit;
  if (zero_fill) {
    EB_DISPATCH_UNIT(unit, (rebuild_padding_kernel<U, true><<<grid_for_rows(total), kThreads, 0, as_stream(stream)>>>(
                               (const U *)src, (U *)tgt, mask_offset, valid, units, (int)total)));
  } else {
    EB_DISPATCH_UNIT(unit, (rebuild_padding_kernel<U, false><<<grid_for_rows(valid), kThreads, 0, as_stream(stream)>>>(
                               (const U *)src, (U *)tgt, mask_offset, valid, units, (int)total)));
  }
  return check_launch("rebuild_padding");
}

extern "C" int eb_transpose_rebuild_padding(const void *Q, const void *K, const void *V, void *q_buf, void *k_buf,
                                            void *v_buf, int batch, int seq_len, int head_num, int size_per_head,
                                            int valid, const int32_t *mask_offset, int dtype, int zero_fill,
                                            void *stream) {
  EB_REQUIRE(dtype_ok(dtype), "transpose_rebuild_padding: bad dtype %d", dtype);
  EB_REQUIRE(batch >= 0 && seq_len >= 0 && head_num >= 0 && size_per_head >= 0 && valid >= 0,
             "transpose_rebuild_padding: negative size");
  const long long total = (long long)batch * seq_len;
  EB_REQUIRE(total * head_num < (1ll << 31) && valid <= total, "transpose_rebuild_padding: sizes out of range");
  if (total == 0 || head_num == 0 || size_per_head == 0 || (valid == 0 && !zero_fill)) return EB_OK;
  EB_REQUIRE(q_buf && k_buf && v_buf && (valid == 0 || (Q && K && V && mask_offset)),
             "transpose_rebuild_padding: null pointer");
  const int e = dtype_size(dtype);
  const int unit = pick_unit((size_t)size_per_head * e, e, {Q, K, V, q_buf, k_buf, v_buf});
  const int du = size_per_head * e / unit;
  dim3 grid(grid_for_rows(zero_fill ? total : valid), 3);
  if (zero_fill) {
    EB_DISPATCH_UNIT(unit, (transpose_rebuild_kernel<U, true><<<grid, kThreads, 0, as_stream(stream)>>>(
                               (const U *)Q, (const U *)K, (const U *)V, (U *)q_buf, (U *)k_buf, (U *)v_buf, batch,
                               seq_len, head_num, du, valid, mask_offset)));
  } else {
    EB_DISPATCH_UNIT(unit, (transpose_rebuild_kernel<U, false><<<grid, kThreads, 0, as_stream(stream)>>>(
                               (const U *)Q, (const U *)K, (const U *)V, (U *)q_buf, (U *)k_buf, (U *)v_buf, batch,
                               seq_len, head_num, du, valid, mask_offset)));
  }
  return check_launch("transpose_rebuild_padding");
}

extern "C" int eb_transpose_remove_padding(const void *src, void *dst, int valid, int batch, int seq_len, int head_num,
                                           int size_per_head, const int32_t *mask_offset, int dtype, void *stream) {
  EB_REQUIRE(dtype_ok(dtype), "transpose_remove_padding: bad dtype %d", dtype);
  EB_REQUIRE(batch >= 0 && seq_len >= 0 && head_num >= 0 && size_per_head >= 0 && valid >= 0,
             "transpose_remove_padding: negative size");
  const long long total = (long long)batch * seq_len;
  EB_REQUIRE(total * head_num < (1ll << 31) && valid <= total, "transpose_remove_padding: sizes out of range");
  if (valid == 0 || head_num == 0 || size_per_head == 0) return EB_OK;
  EB_REQUIRE(src && dst && mask_offset, "transpose_remove_padding: null pointer");
  const int e = dtype_size(dtype);
  const int unit = pick_unit((size_t)size_per_head * e, e, {src, dst});
  const int du = size_per_head * e / unit;
  EB_DISPATCH_UNIT(unit, (transpose_remove_kernel<U><<<grid_for_rows(valid), kThreads, 0, as_stream(stream)>>>(
                             (const U *)src, (U *)dst, valid, batch, seq_len, head_num, du, mask_offset)));
  return check_launch("transpose_remove_padding");
}

static int check_turbo(const char *name, int batch, int max_seq_len, int head_num, int size_per_head, int dtype) {
  if (!dtype_ok(dtype)) return fail(EB_EINVAL, "%s: bad dtype %d", name, dtype);
  if (batch < 0 || max_seq_len < 0 || head_num < 0 || size_per_head < 0) return fail(EB_EINVAL, "%s: negative size", name);
  if ((long long)batch * max_seq_len * head_num >= (1ll << 31)) return fail(EB_EINVAL, "%s: sizes out of range", name);
  if (batch > 12000) return fail(EB_ELIMIT, "%s: batch %d exceeds the supported maximum 12000", name, batch);
  return EB_OK;
}

extern "C" int eb_transpose_pad(const void *src, void *dst, int batch, int max_seq_len, const int32_t *seq_lens,
                                int head_num, int size_per_head, int dtype, void *stream) {
  int rc = check_turbo("transpose_pad", batch, max_seq_len, head_num, size_per_head, dtype);
  if (rc) return rc;
  const long long total = (long long)batch * max_seq_len;
  if (total == 0 || head_num == 0 || size_per_head == 0) return EB_OK;
  EB_REQUIRE(dst && seq_lens, "transpose_pad: null pointer");   // src may be empty when every length is 0
  const int e = dtype_size(dtype);
  const int unit = pick_unit((size_t)size_per_head * e, e, {src, dst});
  const int du = size_per_head * e / unit;
  const size_t smem = (size_t)(batch + 1) * sizeof(int);
  EB_DISPATCH_UNIT(unit, (transpose_pad_kernel<U><<<grid_for_rows(total), kThreads, smem, as_stream(stream)>>>(
                             (const U *)src, (U *)dst, batch, max_seq_len, seq_lens, head_num, du)));
  return check_launch("transpose_pad");
}

extern "C" int eb_transpose_depad(const void *src, void *dst, int batch, int sum_seq, int max_seq_len,
                                  const int32_t *seq_lens, int head_num, int size_per_head, int dtype, void *stream) {
  int rc = check_turbo("transpose_depad", batch, max_seq_len, head_num, size_per_head, dtype);
  if (rc) return rc;
  EB_REQUIRE(sum_seq >= 0, "transpose_depad: negative sum_seq");
  if (sum_seq == 0 || head_num == 0 || size_per_head == 0) return EB_OK;
  EB_REQUIRE(dst && seq_lens, "transpose_depad: null pointer");   // src may be empty when every length is 0
  const int e = dtype_size(dtype);
  const int unit = pick_unit((size_t)size_per_head * e, e, {src, dst});
  const int du = size_per_head * e / unit;
  const size_t smem = (size_t)(batch + 1) * sizeof(int);
  EB_DISPATCH_UNIT(unit, (transpose_depad_kernel<U><<<grid_for_rows(sum_seq), kThreads, smem, as_stream(stream)>>>(
                             (const U *)src, (U *)dst, batch, sum_seq, max_seq_len, seq_lens, head_num, du)));
  return check_launch("transpose_depad");
}
