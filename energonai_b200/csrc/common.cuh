// Shared helpers for the energon_b200 kernels: error reporting for the C ABI, dtype traits,
// 16-byte vector access, warp/block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/energon_b200.h"

namespace eb {

// ---- error reporting (thread-local message behind eb_last_error) -----------------------
int fail(int code, const char *fmt, ...);
int check_launch(const char *what);   // cudaPeekAtLastError -> EB_ECUDA

#define EB_REQUIRE(cond, ...)                         \
  do {                                                \
    if (!(cond)) return ::eb::fail(EB_EINVAL, __VA_ARGS__); \
  } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int dtype_size(int dtype) { return dtype == EB_F32 ? 4 : 2; }
inline bool dtype_ok(int dtype) { return dtype == EB_F32 || dtype == EB_F16 || dtype == EB_BF16; }
inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

int sm_count();   // multiprocessors of the current device (cached per device)
bool pdl_enabled();   // programmatic dependent launch (on unless the environment sets EB_PDL=0)

// Launch with programmatic stream serialization: the kernel may start while its predecessor
// in the stream is still draining, and must execute griddep_wait() before it touches anything
// the predecessor wrote.  Work that only reads constants (weights) can be issued before that.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// Wait for the preceding kernel of the stream (complete and visible); no-op for a plain launch.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Allow the following kernel of the stream to begin launching.
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- dtype conversion ---------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Two packed 16-bit values -> fp32.
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2 *>(&w));
}
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// A 16-byte vector of T (4 floats or 8 halves) with fp32 unpack/pack.
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ void load(const T *p) { raw = *reinterpret_cast<const uint4 *>(p); }
  __device__ __forceinline__ void store(T *p) const { *reinterpret_cast<uint4 *>(p) = raw; }
  __device__ __forceinline__ void unpack(float (&f)[N]) const {
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = to_f32<T>(e[i]);
  }
  __device__ __forceinline__ void pack(const float (&f)[N]) {
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) e[i] = from_f32<T>(f[i]);
  }
};

// ---- reductions ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a CTA of THREADS threads (multiple of 32); every thread gets the result.
// `scratch` must hold THREADS/32 floats; safe to call repeatedly with the same scratch.
template <int THREADS> __device__ __forceinline__ float block_sum(float v, float *scratch) {
  if (THREADS == 32) return warp_sum(v);
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();   // previous use of scratch is complete
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < THREADS / 32 ? scratch[lane] : 0.f;
  return warp_sum(r);
}

}  // namespace eb
