// Shared host/device helpers for the Fourier KV-cache kernels (sm_100a).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "fourier_b200.h"

namespace fa {

// ---- error reporting ---------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define FA_REQUIRE(cond, code, ...)        \
  do {                                     \
    if (!(cond)) {                         \
      ::fa::set_error(__VA_ARGS__);        \
      return (code);                       \
    }                                      \
  } while (0)

#define FA_CHECK_LAUNCH(what)                                   \
  do {                                                          \
    cudaError_t e__ = cudaGetLastError();                       \
    if (e__ != cudaSuccess) return ::fa::cuda_fail(e__, what);  \
  } while (0)

// ---- dtype helpers -----------------------------------------------------------------------
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
struct Pack2;
template <>
struct Pack2<__half> {
  using type = __half2;
  __device__ static __forceinline__ float2 cvt(__half2 v) { return __half22float2(v); }
};
template <>
struct Pack2<__nv_bfloat16> {
  using type = __nv_bfloat162;
  __device__ static __forceinline__ float2 cvt(__nv_bfloat162 v) { return __bfloat1622float2(v); }
};

// eight 16-bit values (one 128-bit load) -> eight floats
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  using P = typename Pack2<T>::type;
  const P* p = reinterpret_cast<const P*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = Pack2<T>::cvt(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// ---- phases ------------------------------------------------------------------------------
// (pos * n) mod T without overflow; the 32-bit path covers every shape in practice.
__device__ __forceinline__ uint32_t phase_mod(uint64_t pos, uint32_t n, uint32_t T) {
  uint64_t p = pos * (uint64_t)n;
  if (p < 0xFFFFFFFFull) return (uint32_t)p % T;
  return (uint32_t)(p % (uint64_t)T);
}

// cos/sin(2*pi*ph/T), 0 <= ph < T
__device__ __forceinline__ void sincos_phase(uint32_t ph, float inv_T, float* s, float* c) {
  // 2*ph/T in [0,2): sincospif keeps full accuracy over that range
  sincospif(2.0f * (float)ph * inv_T, s, c);
}

// The float32 angle of the reference projection kernel: fl(fl(fl(c*pos)*n)/T)
__device__ __forceinline__ float km57_angle(float pos, float n, float T) {
  const float c = (float)(2.0 * 3.14159265359);
  float a = __fmul_rn(c, pos);
  a = __fmul_rn(a, n);
  return __fdiv_rn(a, T);
}

// ---- warp reductions ---------------------------------------------------------------------
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

// ---- cp.async (16-byte, L2 only) ---------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

int sm_count();

// (cols x rows x B) tiled tensor map of a 16-bit tensor, 128-byte swizzle, out-of-range elements read as 0.
// box_cols * 2 bytes must not exceed 128.  Strides in elements.
int make_tensor_map_3d(CUtensorMap* m, const void* base, int dtype, int cols, int rows, int64_t row_stride, int B,
                       int64_t batch_stride, int box_cols, int box_rows);

// tensor-core projection (compress_tc.cu)
bool compress_tc_usable(const void* x, int B, int K, int64_t x_sb, int64_t x_sk, int x_cols, int N);
size_t compress_tc_scratch_bytes(int B, int K, int N, int x_cols);
int compress_tc_launch(const void* x, int dtype, int B, int K, int64_t x_sb, int64_t x_sk, int x_cols, const int32_t* idx,
                       int Mc, int N, int T_c, int64_t k_start, float* coef, int accumulate, void* scratch,
                       size_t scratch_bytes, cudaStream_t st);

}  // namespace fa
