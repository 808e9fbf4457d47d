// Dynamic activation quantisation kernels (HBM-bound elementwise + small reductions), sm_100a.
//
// Arithmetic follows the reference's active Triton kernels (aliases at
// gemlite/quant_utils.py:2680-2684), in fp32 with IEEE division so that the results are
// reproducible bit for bit:
//   per-token fp8/int8   quant_utils.py:467-508
//   mxfp8  (e8m0 per 32) quant_utils.py:1024-1093, power-of-two scale :697-705
//   mxfp4  (e8m0 per 32) quant_utils.py:2005-2105, e2m1 by thresholds :66-73, 2081-2090
//   nvfp4  (e4m3 per 16 + fp32 tensor scale) quant_utils.py:2161-2311, 2329-2431
// Loads are 128-bit; one lane owns 8 consecutive k, a group of 32 (16) values is 4 (2)
// adjacent lanes, so group maxima are one or two shuffles.  The NVFP4 tensor-wide amax is a
// separate pass (atomicMax on the fp32 bit pattern) instead of the reference's in-kernel spin
// barrier (quant_utils.py:2220-2231): nothing here waits on another CTA.
#include "gl_common.cuh"
#include <cuda_fp4.h>

namespace {

__device__ __forceinline__ void load8(const void* x, int64_t idx, int dt, float (&v)[8]) {
  if (dt == GL_FP32) {
    const float4 a = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + idx)[0];
    const float4 b = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + idx)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + idx);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (dt == GL_BF16) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        v[2 * i] = __half2float(__ushort_as_half((unsigned short)(w[i] & 0xffffu)));
        v[2 * i + 1] = __half2float(__ushort_as_half((unsigned short)(w[i] >> 16)));
      }
    }
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 2^ceil(log2(v)) by exponent bits, clamped to [2^-30, 2^127]; returns the biased exponent
__device__ __forceinline__ uint32_t pow2_ceil_exp(float v) {
  const uint32_t xi = __float_as_uint(v);
  uint32_t e = (xi >> 23) & 0xffu;
  if (xi & 0x7fffffu) e += 1u;
  e = min(e, 254u);
  e = max(e, 127u - 30u);
  return e;
}

// index of the scale of (row m, group kg): plain rows [*, G] or 128-row x 4-group atoms of 512 bytes
__device__ __forceinline__ int64_t scale_index(int m, int kg, int G, int layout) {
  if (layout == 0) return (int64_t)m * G + kg;
  return ((int64_t)(m >> 7) * (G >> 2) + (kg >> 2)) * 512 + (m & 31) * 16 + ((m & 127) >> 5) * 4 + (kg & 3);
}

// Two e2m1 codes (low nibble = a, high nibble = b) of values that came from 16-bit activations times a power of two.
// The reference's thresholds are strict (> 0.25, > 0.75, ...): a value exactly half way between two e2m1 numbers goes to
// the smaller magnitude, and -0.0 gets code 0.  The hardware conversion rounds half to even, so each value is first
// moved one fp32 ulp towards zero: a tie then lies below the midpoint, and nothing else changes, because a value with at
// most 11 significant bits is never one fp32 ulp above a midpoint (midpoints have 3 significant bits).  fp32
// activations do not have that guarantee and keep the threshold form.  (16384 x 16384 bf16: 0.459 -> 0.281 ms; the seven
// compares and adds per value had made the kernel issue-bound.  More units per thread and trip, or rows kept in registers
// by the per-token kernel, were 10-20 % slower: these kernels need their 32 registers per thread, 2048 threads per SM.)
__device__ __forceinline__ uint32_t e2m1x2_from16(float a, float b) {
  uint32_t ua = __float_as_uint(a), ub = __float_as_uint(b);
  ua = (ua << 1) ? ua - 1u : 0u;
  ub = (ub << 1) ? ub - 1u : 0u;
  return (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(__uint_as_float(ua), __uint_as_float(ub)), __NV_E2M1, cudaRoundNearest);
}

// Two e2m1 codes of arbitrary fp32 values (NVFP4, fp32 activations): the hardware conversion (round half to even) agrees
// with the reference's strict thresholds except on the three midpoints it rounds up, 0.75 / 1.75 / 3.5, where the code
// is one too high, and on -0.0, which the reference codes as +0 (`v >= 0`); both are put right here.  Seven compares
// and adds per value become three compares.
__device__ __forceinline__ uint32_t e2m1x2_exact(float a, float b) {
  a = __fadd_rn(a, 0.0f);                                  // -0.0 -> +0.0, everything else unchanged
  b = __fadd_rn(b, 0.0f);
  const uint32_t c = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(a, b), __NV_E2M1, cudaRoundNearest);
  const uint32_t ma = __float_as_uint(a) & 0x7fffffffu, mb = __float_as_uint(b) & 0x7fffffffu;
  const uint32_t ta = (ma == 0x3f400000u) | (ma == 0x3fe00000u) | (ma == 0x40600000u);
  const uint32_t tb = (mb == 0x3f400000u) | (mb == 0x3fe00000u) | (mb == 0x40600000u);
  return c - ta - (tb << 4);
}

// (row, first k) of unit u, units of 8 consecutive k: a shift and a mask when a row holds a power of two of them (`shift`
// >= 0; every benchmark shape), else the 64-bit division (a subroutine of about a hundred instructions)
__device__ __forceinline__ void unit_row_k(int64_t u, int64_t units_per_row, int shift, int& m, int& k) {
  if (shift >= 0) {
    m = (int)(u >> shift);
    k = (int)(u & (units_per_row - 1)) * 8;
  } else {
    m = (int)(u / units_per_row);
    k = (int)(u % units_per_row) * 8;
  }
}
__device__ __forceinline__ int pow2_shift(int64_t v) { return (v & (v - 1)) == 0 ? 63 - __clzll(v) : -1; }

// ---------------------------------------------------------------------------------------------
// per-token: one CTA per row (grid-stride), two passes over the row (second one hits L1/L2)
template <bool INT8>
__global__ void __launch_bounds__(256) per_token_kernel(const void* __restrict__ x, uint8_t* __restrict__ q,
                                                        float* __restrict__ scales, int M, int K, int x_dtype) {
  __shared__ float s_red[8];
  __shared__ float s_scale;
  gl_launch_dependents();          // the matmul that follows may set itself up and prefetch weights meanwhile
  gl_grid_dependency_wait();       // x comes from the previous kernel of the stream; q / scales may still be read by it
  const float qmax = INT8 ? 127.f : 448.f, qmin = INT8 ? -128.f : -448.f;
  for (int m = blockIdx.x; m < M; m += gridDim.x) {
    float amax = 0.f;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
      float v[8];
      load8(x, (int64_t)m * K + k, x_dtype, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) a = fmaxf(a, s_red[i]);
      const float s = fmaxf(a / qmax, 1e-6f);
      s_scale = s;
      scales[m] = s;
    }
    __syncthreads();
    const float s = s_scale;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
      float v[8];
      load8(x, (int64_t)m * K + k, x_dtype, v);
      uint32_t o[2] = {0u, 0u};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float t = fminf(fmaxf(v[i] / s, qmin), qmax);
        uint32_t b;
        if (INT8) b = (uint32_t)(uint8_t)(int8_t)(int)roundf(t);
        else b = (uint32_t)__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3);
        o[i >> 2] |= b << (8 * (i & 3));
      }
      *reinterpret_cast<uint2*>(q + (int64_t)m * K + k) = make_uint2(o[0], o[1]);
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// mxfp4 / mxfp8: thread = 8 consecutive k of one row; 4 lanes = one group of 32
template <bool FP4>
__global__ void __launch_bounds__(256) mx_quant_kernel(const void* __restrict__ x, uint8_t* __restrict__ q,
                                                       uint8_t* __restrict__ scales, int M, int Mpad, int K, int x_dtype, int layout) {
  gl_launch_dependents();
  gl_grid_dependency_wait();
  const int64_t units_per_row = K / 8;
  const int64_t total = (int64_t)Mpad * units_per_row;
  const int shift = pow2_shift(units_per_row);
  // the loop bound is warp-uniform so that every lane takes part in the group shuffles
  for (int64_t u0 = blockIdx.x * (int64_t)blockDim.x + (threadIdx.x & ~31); u0 < total; u0 += (int64_t)gridDim.x * blockDim.x) {
    const int64_t u = u0 + (threadIdx.x & 31);
    const bool valid = u < total;
    int m = Mpad, k = 0;
    if (valid) unit_row_k(u, units_per_row, shift, m, k);
    float v[8];
    const bool real = m < M;
    if (real) load8(x, (int64_t)m * K + k, x_dtype, v);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t e = pow2_ceil_exp(amax / (FP4 ? 6.f : 448.f));
    const float scale = __uint_as_float(e << 23);
    if (valid && (threadIdx.x & 3) == 0) scales[scale_index(m, k / 32, K / 32, layout)] = real ? (uint8_t)e : (uint8_t)127;
    if (!real) continue;
    const float inv = 1.0f / scale;                    // a power of two in [2^-127, 2^30]: multiplying by it is the division, exactly
    if (FP4) {
      uint32_t o = 0u;
      if (x_dtype == GL_FP32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) o |= e2m1x2_exact(v[2 * i] * inv, v[2 * i + 1] * inv) << (8 * i);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) o |= e2m1x2_from16(v[2 * i] * inv, v[2 * i + 1] * inv) << (8 * i);
      }
      *reinterpret_cast<uint32_t*>(q + (int64_t)m * (K / 2) + k / 2) = o;
    } else {
      uint32_t o[2] = {0u, 0u};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float t = fminf(fmaxf(v[i] * inv, -448.f), 448.f);
        o[i >> 2] |= (uint32_t)__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3) << (8 * (i & 3));
      }
      *reinterpret_cast<uint2*>(q + (int64_t)m * K + k) = make_uint2(o[0], o[1]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// nvfp4 pass 1: tensor-wide max |x| as an fp32 bit pattern (non-negative floats order as uints)
__global__ void __launch_bounds__(256) amax_kernel(const void* __restrict__ x, uint32_t* __restrict__ amax_bits,
                                                   int64_t total_units, int x_dtype) {
  float amax = 0.f;
  gl_launch_dependents();
  gl_grid_dependency_wait();
  for (int64_t u = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; u < total_units; u += (int64_t)gridDim.x * blockDim.x) {
    float v[8];
    load8(x, u * 8, x_dtype, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  __shared__ float s_red[8];
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) a = fmaxf(a, s_red[i]);
    atomicMax(amax_bits, __float_as_uint(a));
  }
}

// nvfp4 pass 2: thread = 8 consecutive k; 2 lanes = one group of 16
__global__ void __launch_bounds__(256) nvfp4_quant_kernel(const void* __restrict__ x, uint8_t* __restrict__ q,
                                                          uint8_t* __restrict__ scales, float* __restrict__ meta_out,
                                                          const float* __restrict__ meta_in,
                                                          const uint32_t* __restrict__ amax_bits, int M, int Mpad, int K,
                                                          int x_dtype, int layout) {
  float meta;
  gl_launch_dependents();
  gl_grid_dependency_wait();       // the tensor-wide amax comes from the previous kernel
  if (meta_in != nullptr) meta = *meta_in;
  else meta = (448.f * 6.0f) / fmaxf(__uint_as_float(*amax_bits), 1e-6f);
  if (blockIdx.x == 0 && threadIdx.x == 0) *meta_out = meta;
  const int64_t units_per_row = K / 8;
  const int64_t total = (int64_t)Mpad * units_per_row;
  const int shift = pow2_shift(units_per_row);
  // the loop bound is warp-uniform so that every lane takes part in the group shuffles
  for (int64_t u0 = blockIdx.x * (int64_t)blockDim.x + (threadIdx.x & ~31); u0 < total; u0 += (int64_t)gridDim.x * blockDim.x) {
    const int64_t u = u0 + (threadIdx.x & 31);
    const bool valid = u < total;
    int m = Mpad, k = 0;
    if (valid) unit_row_k(u, units_per_row, shift, m, k);
    const bool real = m < M;
    float v[8];
    if (real) load8(x, (int64_t)m * K + k, x_dtype, v);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const float sraw = fminf(amax * meta / 6.f, 448.f);
    const uint8_t s8 = (uint8_t)__nv_cvt_float_to_fp8(sraw, __NV_SATFINITE, __NV_E4M3);
    if (valid && (threadIdx.x & 1) == 0) scales[scale_index(m, k / 16, K / 16, layout)] = real ? s8 : (uint8_t)0x38;  // 0x38 = 1.0 e4m3
    if (!real) continue;
    const float sfull = fmaxf(gl_e4m3_to_float(s8) / meta, 1e-6f);
    uint32_t o = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) o |= e2m1x2_exact(v[2 * i] / sfull, v[2 * i + 1] / sfull) << (8 * i);
    *reinterpret_cast<uint32_t*>(q + (int64_t)m * (K / 2) + k / 2) = o;
  }
}

int check_x(const char* fn, const void* x, int M, int K, int x_dtype, int kmult) {
  if (M < 0 || K <= 0) { gl_set_error("%s: bad shape M=%d K=%d", fn, M, K); return GL_E_INVALID; }
  if (K % kmult != 0) { gl_set_error("%s: K=%d must be a multiple of %d", fn, K, kmult); return GL_E_INVALID; }
  if (!(x_dtype == GL_FP16 || x_dtype == GL_BF16 || x_dtype == GL_FP32)) { gl_set_error("%s: unsupported activation dtype %d", fn, x_dtype); return GL_E_INVALID; }
  if ((uintptr_t)x & 15) { gl_set_error("%s: x must be 16-byte aligned", fn); return GL_E_INVALID; }
  return GL_OK;
}
unsigned grid_units(int64_t total_threads) {
  int64_t b = gl_cdiv(total_threads, 256);
  const int64_t cap = (int64_t)gl_num_sms() * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}

}  // namespace

extern "C" int gl_scale_activations_per_token(const void* x, void* q, float* scales, int32_t M, int32_t K,
                                              int32_t x_dtype, int32_t q_dtype, void* stream) {
  if (int rc = check_x("gl_scale_activations_per_token", x, M, K, x_dtype, 8)) return rc;
  if (!(q_dtype == GL_FP8 || q_dtype == GL_INT8)) GL_FAIL(GL_E_INVALID, "gl_scale_activations_per_token: q_dtype must be FP8 (e4m3) or INT8, got %d", q_dtype);
  if (M == 0) return GL_OK;
  if (!q || !scales || ((uintptr_t)q & 7)) GL_FAIL(GL_E_INVALID, "gl_scale_activations_per_token: null or misaligned output");
  cudaStream_t st = (cudaStream_t)stream;
  const int cap = gl_num_sms() * 8;
  const unsigned grid = (unsigned)(M < cap ? M : cap);
  if (q_dtype == GL_INT8) GL_CUDA_CHECK(gl_launch_pdl(per_token_kernel<true>, dim3(grid), dim3(256), 0, st, x, (uint8_t*)q, scales, M, K, x_dtype));
  else GL_CUDA_CHECK(gl_launch_pdl(per_token_kernel<false>, dim3(grid), dim3(256), 0, st, x, (uint8_t*)q, scales, M, K, x_dtype));
  return GL_OK;
}

// ---------------------------------------------------------------------------------------------
// per block: one scale per (row, 128 consecutive k) -- the activation side of 128 x 128 block quantisation
// (gemlite/quant_utils.py:2504-2522).  Sixteen lanes own a block (8 elements each): amax by four shuffles inside the
// half warp, scale = max(amax / qmax, 1e-6), q = clamp(x / scale) cast (FP8) or rounded half away from zero (INT8, as
// the reference's active kernel does: quant_utils.py:2613-2675 with libdevice.round).
template <bool INT8>
__global__ void __launch_bounds__(256) per_block_kernel(const void* __restrict__ x, uint8_t* __restrict__ q,
                                                        float* __restrict__ scales, int64_t total_units, int K, int x_dtype) {
  gl_launch_dependents();
  gl_grid_dependency_wait();
  const float qmax = INT8 ? 127.f : 448.f, qmin = INT8 ? -128.f : -448.f;
  const int units_per_row = K / 8;
  const int shift = pow2_shift(units_per_row);
  // the loop bound is half-warp-uniform: a block's sixteen units are either all inside or all outside
  for (int64_t u0 = blockIdx.x * (int64_t)blockDim.x + (threadIdx.x & ~15); u0 < total_units; u0 += (int64_t)gridDim.x * blockDim.x) {
    const int64_t u = u0 + (threadIdx.x & 15);
    int m, k;
    unit_row_k(u, units_per_row, shift, m, k);
    float v[8];
    load8(x, (int64_t)m * K + k, x_dtype, v);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const unsigned half_mask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;     // the other half warp may be past the end
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(half_mask, amax, o));
    const float s = fmaxf(amax / qmax, 1e-6f);
    if ((threadIdx.x & 15) == 0) scales[(int64_t)m * (K / 128) + k / 128] = s;
    uint32_t o2[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float t = fminf(fmaxf(v[i] / s, qmin), qmax);
      uint32_t b;
      if (INT8) b = (uint32_t)(uint8_t)(int8_t)(int)roundf(t);                // libdevice.round: half away from zero
      else b = (uint32_t)__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3);
      o2[i >> 2] |= b << (8 * (i & 3));
    }
    *reinterpret_cast<uint2*>(q + (int64_t)m * K + k) = make_uint2(o2[0], o2[1]);
  }
}

extern "C" int gl_scale_activations_per_block(const void* x, void* q, float* scales, int32_t M, int32_t K,
                                              int32_t x_dtype, int32_t q_dtype, void* stream) {
  if (int rc = check_x("gl_scale_activations_per_block", x, M, K, x_dtype, 128)) return rc;
  if (!(q_dtype == GL_FP8 || q_dtype == GL_INT8)) GL_FAIL(GL_E_INVALID, "gl_scale_activations_per_block: q_dtype must be FP8 (e4m3) or INT8, got %d", q_dtype);
  if (M == 0) return GL_OK;
  if (!q || !scales || ((uintptr_t)q & 7)) GL_FAIL(GL_E_INVALID, "gl_scale_activations_per_block: null or misaligned output");
  const int64_t units = (int64_t)M * (K / 8);
  if (q_dtype == GL_INT8) GL_CUDA_CHECK(gl_launch_pdl(per_block_kernel<true>, dim3(grid_units(units)), dim3(256), 0, (cudaStream_t)stream, x, (uint8_t*)q, scales, units, K, x_dtype));
  else GL_CUDA_CHECK(gl_launch_pdl(per_block_kernel<false>, dim3(grid_units(units)), dim3(256), 0, (cudaStream_t)stream, x, (uint8_t*)q, scales, units, K, x_dtype));
  return GL_OK;
}

static int check_layout(const char* fn, int layout, int G) {
  if (layout != 0 && layout != 1) { gl_set_error("%s: scale_layout must be 0 or 1", fn); return GL_E_INVALID; }
  if (layout == 1 && G % 4 != 0) { gl_set_error("%s: scale atoms need K / group_size to be a multiple of 4", fn); return GL_E_INVALID; }
  return GL_OK;
}

extern "C" int gl_scale_activations_mxfp4(const void* x, uint8_t* q, uint8_t* scales, int32_t M, int32_t K,
                                          int32_t x_dtype, int32_t scale_layout, void* stream) {
  if (int rc = check_x("gl_scale_activations_mxfp4", x, M, K, x_dtype, 32)) return rc;
  if (M == 0) return GL_OK;
  if (!q || !scales || ((uintptr_t)q & 3)) GL_FAIL(GL_E_INVALID, "gl_scale_activations_mxfp4: null or misaligned output");
  if (int rc = check_layout("gl_scale_activations_mxfp4", scale_layout, K / 32)) return rc;
  const int Mpad = scale_layout ? (M + 127) / 128 * 128 : (M + 31) / 32 * 32;
  GL_CUDA_CHECK(gl_launch_pdl(mx_quant_kernel<true>, dim3(grid_units((int64_t)Mpad * (K / 8))), dim3(256), 0, (cudaStream_t)stream, x, q, scales, M, Mpad, K, x_dtype, scale_layout));
  return GL_OK;
}

extern "C" int gl_scale_activations_mxfp8(const void* x, uint8_t* q, uint8_t* scales, int32_t M, int32_t K,
                                          int32_t x_dtype, int32_t scale_layout, void* stream) {
  if (int rc = check_x("gl_scale_activations_mxfp8", x, M, K, x_dtype, 32)) return rc;
  if (M == 0) return GL_OK;
  if (!q || !scales || ((uintptr_t)q & 7)) GL_FAIL(GL_E_INVALID, "gl_scale_activations_mxfp8: null or misaligned output");
  if (int rc = check_layout("gl_scale_activations_mxfp8", scale_layout, K / 32)) return rc;
  const int Mpad = scale_layout ? (M + 127) / 128 * 128 : (M + 31) / 32 * 32;
  GL_CUDA_CHECK(gl_launch_pdl(mx_quant_kernel<false>, dim3(grid_units((int64_t)Mpad * (K / 8))), dim3(256), 0, (cudaStream_t)stream, x, q, scales, M, Mpad, K, x_dtype, scale_layout));
  return GL_OK;
}

extern "C" int gl_scale_activations_nvfp4(const void* x, uint8_t* q, uint8_t* scales, float* meta_scale,
                                          const float* meta_in, uint32_t* amax_scratch, int32_t M, int32_t K,
                                          int32_t x_dtype, int32_t scale_layout, void* stream) {
  if (int rc = check_x("gl_scale_activations_nvfp4", x, M, K, x_dtype, 16)) return rc;
  if (int rc = check_layout("gl_scale_activations_nvfp4", scale_layout, K / 16)) return rc;
  if (M == 0) return GL_OK;
  if (!q || !scales || !meta_scale || ((uintptr_t)q & 3)) GL_FAIL(GL_E_INVALID, "gl_scale_activations_nvfp4: null or misaligned output");
  if (meta_in == nullptr && amax_scratch == nullptr) GL_FAIL(GL_E_INVALID, "gl_scale_activations_nvfp4: amax_scratch needed for the dynamic tensor scale");
  cudaStream_t st = (cudaStream_t)stream;
  const int Mpad = scale_layout ? (M + 127) / 128 * 128 : (M + 15) / 16 * 16;
  if (meta_in == nullptr) {
    GL_CUDA_CHECK(cudaMemsetAsync(amax_scratch, 0, sizeof(uint32_t), st));
    const int64_t units = (int64_t)M * (K / 8);
    GL_CUDA_CHECK(gl_launch_pdl(amax_kernel, dim3(grid_units(units)), dim3(256), 0, st, x, amax_scratch, units, x_dtype));
  }
  GL_CUDA_CHECK(gl_launch_pdl(nvfp4_quant_kernel, dim3(grid_units((int64_t)Mpad * (K / 8))), dim3(256), 0, st, x, q, scales, meta_scale, meta_in, amax_scratch, M, Mpad, K, x_dtype, scale_layout));
  return GL_OK;
}
