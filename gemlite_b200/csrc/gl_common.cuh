// Shared host/device helpers for the gemlite_b200 sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include "../../include/gemlite_b200.h"

// ---- error reporting (thread-local message, C status codes) -----------------------------
void gl_set_error(const char* fmt, ...);
#define GL_FAIL(code, ...) do { gl_set_error(__VA_ARGS__); return (code); } while (0)
#define GL_CUDA_CHECK(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) { \
  gl_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
  return GL_E_CUDA; } } while (0)
#define GL_LAUNCH_CHECK(name) do { cudaError_t _e = cudaGetLastError(); if (_e != cudaSuccess) { \
  gl_set_error("launch of %s failed: %s", name, cudaGetErrorString(_e)); return GL_E_CUDA; } } while (0)

// Launch with the programmatic-stream-serialization attribute: the kernel may become resident while the previous
// kernel of the stream drains.  Such a kernel executes griddepcontrol.wait before it touches anything the previous
// kernel wrote or may still read (gl_grid_dependency_wait), and griddepcontrol.launch_dependents once its own
// successor may start.
#ifdef __CUDACC__
template <typename K, typename... A>
static inline cudaError_t gl_launch_pdl(K kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}
__device__ __forceinline__ void gl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void gl_grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

static inline int gl_dtype_size(int dt) {
  switch (dt) {
    case GL_FP32: case GL_INT32: case GL_UINT32: return 4;
    case GL_FP16: case GL_BF16: case GL_INT16: case GL_UINT16: case GL_MXFP16: case GL_MXBF16: return 2;
    case GL_FP8: case GL_FP8E5: case GL_INT8: case GL_UINT8: case GL_MXFP8: case GL_MXFP4:
    case GL_NVFP4: case GL_E8M0: return 1;
    case GL_INT64: return 8;
    default: return 0;
  }
}
static inline bool gl_is_mx(int dt) {
  return dt == GL_MXFP16 || dt == GL_MXBF16 || dt == GL_MXFP8 || dt == GL_MXFP4 || dt == GL_NVFP4;
}
static inline int64_t gl_cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// number of SMs of the current device (cached per device id)
int gl_num_sms();
// integer field of a tile-config cache entry, or dflt (gl_cfg.cpp)
uint64_t gl_cfg_generation();   // changes whenever the config cache changes
int gl_cfg_int(const char* family, const char* signature, const char* key, int dflt);

// ---- family launchers (each returns GL_OK / GL_E_*; GL_E_UNSUPPORTED = "not my case") -----
int gl_gemv_stream_supported(const gl_matmul_args* a);
uint64_t gl_gemv_stream_workspace(const gl_matmul_args* a);
const char* gl_gemv_stream_kernel_name(const gl_matmul_args* a);
int gl_gemv_stream_launch(const gl_matmul_args* a, cudaStream_t st);
int gl_gemv_split_rows_ok(const gl_matmul_args* a);   // 17..32 rows served by two launches of the warp-independent kernel
int gl_generic_launch(const gl_matmul_args* a, cudaStream_t st);
// weight-only 8-bit layers (unpacked INT8 / FP8 weights, one scale per channel) at decode sizes (gl_w8.cu)
bool gl_w8_gemv_supported(const gl_matmul_args* a);
int gl_w8_gemv_launch(const gl_matmul_args* a, cudaStream_t st);
// weight-only block-scaled fp4 (e2m1 + e8m0 / e4m3 group scales, 16-bit activations) at decode sizes (gl_w8.cu)
bool gl_w4mx_gemv_supported(const gl_matmul_args* a);
int gl_w4mx_gemv_launch(const gl_matmul_args* a, cudaStream_t st);
int gl_validate_matmul_args(const gl_matmul_args* a);
int gl_gemm_tc_supported(const gl_matmul_args* a);
uint64_t gl_gemm_tc_workspace(const gl_matmul_args* a);
int gl_gemm_tc_launch(const gl_matmul_args* a, cudaStream_t st);

#ifdef __CUDACC__
// ---- device-side scalar conversions -------------------------------------------------------
__device__ __forceinline__ float gl_e2m1_to_float(uint32_t code) {
  // E2M1: sign bit 3, magnitudes {0,.5,1,1.5,2,3,4,6} (gemlite/quant_utils.py:36-41)
  uint32_t m = code & 7u;
  float v = (m < 2u) ? 0.5f * (float)m : (float)(2u + (m & 1u)) * (float)(1u << ((m >> 1) - 1u)) * 0.5f;
  return (code & 8u) ? -v : v;
}
__device__ __forceinline__ float gl_e8m0_to_float(uint32_t b) {
  // 2^(b-127); b==0 -> 2^-127 (denormal bit pattern 0x00400000), b==255 -> NaN
  if (b == 0u) return __uint_as_float(0x00400000u);
  if (b == 255u) return __uint_as_float(0x7fc00000u);
  return __uint_as_float(b << 23);
}
__device__ __forceinline__ float gl_e4m3_to_float(uint32_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ float gl_e5m2_to_float(uint32_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E5M2);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
// load element i of a buffer with a runtime dtype code as fp32
__device__ __forceinline__ float gl_load_as_float(const void* p, int64_t i, int dt) {
  switch (dt) {
    case GL_FP32: return reinterpret_cast<const float*>(p)[i];
    case GL_FP16: case GL_MXFP16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    case GL_BF16: case GL_MXBF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    case GL_FP8: case GL_MXFP8: return gl_e4m3_to_float(reinterpret_cast<const uint8_t*>(p)[i]);
    case GL_FP8E5: return gl_e5m2_to_float(reinterpret_cast<const uint8_t*>(p)[i]);
    case GL_INT8: return (float)reinterpret_cast<const int8_t*>(p)[i];
    case GL_UINT8: return (float)reinterpret_cast<const uint8_t*>(p)[i];
    case GL_INT32: return (float)reinterpret_cast<const int32_t*>(p)[i];
    case GL_INT16: return (float)reinterpret_cast<const int16_t*>(p)[i];
    case GL_E8M0: return gl_e8m0_to_float(reinterpret_cast<const uint8_t*>(p)[i]);
    default: return 0.f;
  }
}
// round an fp32 value to the precision of dtype `dt` (fp16 / bf16 / fp32), keep as fp32
__device__ __forceinline__ float gl_round_to(float v, int dt) {
  if (dt == GL_BF16 || dt == GL_MXBF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (dt == GL_FP16 || dt == GL_MXFP16) return __half2float(__float2half_rn(v));
  return v;
}
__device__ __forceinline__ void gl_store_out(void* p, int64_t i, float v, int dt) {
  if (dt == GL_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else if (dt == GL_FP16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}
#endif
