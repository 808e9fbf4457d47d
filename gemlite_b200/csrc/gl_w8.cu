// Decode-size kernel for weight-only 8-bit layers: fp16 / bf16 activations, INT8 or FP8 (e4m3) weights stored
// unpacked [N, K] with K contiguous, one scale per output channel (the reference's A16W8 processors,
// gemlite/helper.py:89-171: W_group_mode 2 with one group = K, or channel_scale_mode 1; its kernels for them are the
// GEMV / GEMM families of gemlite/triton_kernels with W_nbits = 8, elements_per_sample = 1).
//
// HBM-bound: N * K weight bytes are read once.  A warp owns four output channels; a lane reads 16 weight bytes of each
// per step (a warp instruction covers 512 contiguous bytes of a row), keeps two steps in flight (4 KB per warp), and
// multiplies them with activations that were staged in shared memory as fp32 in the order the lanes consume them
// (conflict-free 16-byte reads).  INT8 weights become fp32 with a PRMT and an FADD each (0x4B0000bb = 2^23 + b for the
// biased byte b = w ^ 0x80, minus 2^23 + 128: exact); FP8 weights go through cvt.f16x2.e4m3x2.  fp32 accumulation, the channel scale and the bias are applied to the finished sum:
// out = scale[n] * sum_k x[m,k] * w[n,k] + bias[n]  (for W_group_mode 2 the reference rounds w * scale to the
// activation dtype per element first; the difference is below the output rounding).
#include "gl_common.cuh"
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>

namespace {

constexpr int kWarps = 8;             // warps per CTA
constexpr int kRows = 4;              // output channels per warp
constexpr int kMaxM = 4;
constexpr size_t kSmemLimit = 200 * 1024;

struct W8Params {
  const void* x; const uint8_t* w; const void* scales; const void* bias; void* out;
  int M, N, K, x_dtype, out_dtype, scales_dtype, is_fp8, has_scale;
  long long s_stride_g, s_stride_n;                    // grouped (MXFP8 weights): e8m0 scale of (group, channel)
};

__device__ __forceinline__ float x_as_float(const void* x, int64_t i, int dt) {
  return dt == GL_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]) : __half2float(reinterpret_cast<const __half*>(x)[i]);
}

// GROUPED: weight-only MXFP8 (e4m3 weights, one e8m0 scale per 32 weights, the reference's A16W8_MXFP processor): a
// lane's 16 weights are half a group, so the group scale multiplies the lane's partial sum of the step.
template <int MM, bool FP8, bool GROUPED = false>
__global__ void __launch_bounds__(kWarps * 32) gl_w8_gemv_kernel(const W8Params p) {
  extern __shared__ float xs[];                       // [MM][steps][4][32] float4-interleaved activations
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = p.K / 16;                         // 16-byte units per weight row
  const int steps = (units + 31) / 32;
  const int n0 = (blockIdx.x * kWarps + warp) * kRows;
  const uint4* wrow[kRows];
  int nrow[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    nrow[r] = min(n0 + r, p.N - 1);
    wrow[r] = reinterpret_cast<const uint4*>(p.w + (size_t)nrow[r] * p.K);
  }
  // the first two steps of weights are requested before the dependency wait: they do not depend on the previous kernel
  uint4 buf[2][kRows];
  uint32_t sbuf[2][kRows];                            // grouped: the unit's scale byte
  auto fetch = [&](int i, uint4 (&b)[kRows], uint32_t (&sb)[kRows]) {
    const int u = i * 32 + lane;
    const bool ok = i < steps && u < units;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      b[r] = ok ? __ldg(wrow[r] + u) : make_uint4(0u, 0u, 0u, 0u);
      if (GROUPED) sb[r] = ok ? (uint32_t)__ldg(reinterpret_cast<const uint8_t*>(p.scales) + (long long)(u >> 1) * p.s_stride_g + (long long)nrow[r] * p.s_stride_n) : 0u;
    }
  };
  fetch(0, buf[0], sbuf[0]);
  fetch(1, buf[1], sbuf[1]);
  gl_launch_dependents();
  gl_grid_dependency_wait();
  // stage x: unit u = 32 * i + l holds k = 16 u .. 16 u + 15; its four float4 go to xs[m][i][j][l]
  for (int m = 0; m < MM; ++m) {
    for (int idx = threadIdx.x; idx < steps * 128; idx += blockDim.x) {        // one float4 per index
      const int i = idx >> 7, j = (idx >> 5) & 3, l = idx & 31;
      const int k = 16 * (32 * i + l) + 4 * j;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < p.K) {
        const int64_t o = (int64_t)m * p.K + k;
        v = make_float4(x_as_float(p.x, o, p.x_dtype), x_as_float(p.x, o + 1, p.x_dtype), x_as_float(p.x, o + 2, p.x_dtype), x_as_float(p.x, o + 3, p.x_dtype));
      }
      reinterpret_cast<float4*>(xs)[(size_t)m * steps * 128 + idx] = v;
    }
  }
  __syncthreads();
  float acc[kRows][MM];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int m = 0; m < MM; ++m) acc[r][m] = 0.f;
  // one step: consume the 16 bytes per row held in `b`, then refill `b` with step i + 2
  auto step = [&](int i, uint4 (&b)[kRows], uint32_t (&sb)[kRows]) {
    uint4 wv[kRows];
    uint32_t sv[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) { wv[r] = b[r]; sv[r] = GROUPED ? sb[r] : 0u; }
    fetch(i + 2, b, sb);
    float part[kRows][MM];                             // grouped: the step's partial sums, scaled once below
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
      for (int m = 0; m < MM; ++m) part[r][m] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float4 xv[MM];
#pragma unroll
      for (int m = 0; m < MM; ++m) xv[m] = reinterpret_cast<const float4*>(xs)[((size_t)m * steps + i) * 128 + j * 32 + lane];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const uint32_t w4 = j == 0 ? wv[r].x : j == 1 ? wv[r].y : j == 2 ? wv[r].z : wv[r].w;
        float f0, f1, f2, f3;
        if (FP8) {
          const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w4 & 0xFFFFu), __NV_E4M3);
          const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w4 >> 16), __NV_E4M3);
          const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo)), c = __half22float2(*reinterpret_cast<const __half2*>(&hi));
          f0 = a.x; f1 = a.y; f2 = c.x; f3 = c.y;
        } else {
          const uint32_t u4 = w4 ^ 0x80808080u;        // signed byte -> byte + 128
          f0 = __uint_as_float(__byte_perm(u4, 0x4B000000u, 0x7540)) - 8388736.f;      // (2^23 + 128 + w) - (2^23 + 128)
          f1 = __uint_as_float(__byte_perm(u4, 0x4B000000u, 0x7541)) - 8388736.f;
          f2 = __uint_as_float(__byte_perm(u4, 0x4B000000u, 0x7542)) - 8388736.f;
          f3 = __uint_as_float(__byte_perm(u4, 0x4B000000u, 0x7543)) - 8388736.f;
        }
#pragma unroll
        for (int m = 0; m < MM; ++m) {
          if (GROUPED) part[r][m] = fmaf(xv[m].x, f0, fmaf(xv[m].y, f1, fmaf(xv[m].z, f2, fmaf(xv[m].w, f3, part[r][m]))));
          else acc[r][m] = fmaf(xv[m].x, f0, fmaf(xv[m].y, f1, fmaf(xv[m].z, f2, fmaf(xv[m].w, f3, acc[r][m]))));
        }
      }
    }
    if (GROUPED) {
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const float sc = gl_e8m0_to_float(sv[r]);
#pragma unroll
        for (int m = 0; m < MM; ++m) acc[r][m] = fmaf(part[r][m], sc, acc[r][m]);
      }
    }
  };
  for (int i = 0; i < steps; i += 2) {
    step(i, buf[0], sbuf[0]);
    if (i + 1 < steps) step(i + 1, buf[1], sbuf[1]);
  }
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int m = 0; m < MM; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[r][m] = v;
    }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int n = n0 + r;
      if (n >= p.N) break;
      const float sc = p.has_scale ? gl_load_as_float(p.scales, n, p.scales_dtype) : 1.f;
      const float bi = p.bias != nullptr ? gl_load_as_float(p.bias, n, p.out_dtype) : 0.f;
#pragma unroll
      for (int m = 0; m < MM; ++m) {
        gl_store_out(p.out, (int64_t)m * p.N + n, fmaf(acc[r][m], sc, bi), p.out_dtype);
      }
    }
  }
}

// Weight-only block-scaled fp4 (the reference's A16W4_MXFP / A16W4_NVFP processors, gemlite/helper.py:384-504: e2m1
// codes two per byte [N, K/2], K contiguous; one e8m0 scale per 32 weights or one e4m3 scale per 16 plus a tensor scale;
// 16-bit activations).  Same structure as above: a lane's 16 bytes are 32 weights = one MX group (two NV groups), so the
// group scale multiplies the lane's partial sum of the step once instead of every weight.
struct W4Params {
  const void* x; const uint8_t* w; const uint8_t* scales; const float* meta_scale; const void* bias; void* out;
  int M, N, K, x_dtype, out_dtype, group;
  long long s_stride_g, s_stride_n;
};

template <int MM, bool NV>
__global__ void __launch_bounds__(kWarps * 32) gl_w4mx_gemv_kernel(const W4Params p) {
  extern __shared__ float xs[];                       // [MM][steps][8][32] float4-interleaved activations
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = p.K / 32;                         // 16-byte units (32 weights) per row
  const int steps = (units + 31) / 32;
  const int n0 = (blockIdx.x * kWarps + warp) * kRows;
  const uint4* wrow[kRows];
  int nrow[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    nrow[r] = min(n0 + r, p.N - 1);
    wrow[r] = reinterpret_cast<const uint4*>(p.w + (size_t)nrow[r] * (p.K / 2));
  }
  uint4 buf[2][kRows];
  uint32_t sbuf[2][kRows];                            // the unit's scale byte (MX) or its two scale bytes (NV)
  auto fetch = [&](int i, uint4 (&b)[kRows], uint32_t (&sb)[kRows]) {
    const int u = i * 32 + lane;
    const bool ok = i < steps && u < units;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      b[r] = ok ? __ldg(wrow[r] + u) : make_uint4(0u, 0u, 0u, 0u);
      if (!ok) sb[r] = 0u;
      else if (NV) sb[r] = (uint32_t)__ldg(p.scales + (long long)(2 * u) * p.s_stride_g + (long long)nrow[r] * p.s_stride_n) |
                           ((uint32_t)__ldg(p.scales + (long long)(2 * u + 1) * p.s_stride_g + (long long)nrow[r] * p.s_stride_n) << 8);
      else sb[r] = (uint32_t)__ldg(p.scales + (long long)u * p.s_stride_g + (long long)nrow[r] * p.s_stride_n);
    }
  };
  fetch(0, buf[0], sbuf[0]);                          // weights and scales do not depend on the previous kernel
  fetch(1, buf[1], sbuf[1]);
  gl_launch_dependents();
  gl_grid_dependency_wait();
  // stage x: unit u = 32 * i + l holds k = 32 u .. 32 u + 31; its eight float4 go to xs[m][i][j][l]
  for (int m = 0; m < MM; ++m)
    for (int idx = threadIdx.x; idx < steps * 256; idx += blockDim.x) {
      const int i = idx >> 8, j = (idx >> 5) & 7, l = idx & 31;
      const int k = 32 * (32 * i + l) + 4 * j;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < p.K) {
        const int64_t o = (int64_t)m * p.K + k;
        v = make_float4(x_as_float(p.x, o, p.x_dtype), x_as_float(p.x, o + 1, p.x_dtype), x_as_float(p.x, o + 2, p.x_dtype), x_as_float(p.x, o + 3, p.x_dtype));
      }
      reinterpret_cast<float4*>(xs)[(size_t)m * steps * 256 + idx] = v;
    }
  __syncthreads();
  float acc[kRows][MM];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int m = 0; m < MM; ++m) acc[r][m] = 0.f;
  auto step = [&](int i, uint4 (&b)[kRows], uint32_t (&sb)[kRows]) {
    uint4 wv[kRows];
    uint32_t sv[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) { wv[r] = b[r]; sv[r] = sb[r]; }
    fetch(i + 2, b, sb);
    float part[kRows][MM][2];                         // partial sums of the unit's two halves (16 weights each)
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
      for (int m = 0; m < MM; ++m) part[r][m][0] = part[r][m][1] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {                     // float4 j of x <-> weights 4 j .. 4 j + 3 <-> 16 bits of word j / 2
      float4 xv[MM];
#pragma unroll
      for (int m = 0; m < MM; ++m) xv[m] = reinterpret_cast<const float4*>(xs)[((size_t)m * steps + i) * 256 + j * 32 + lane];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const uint32_t word = (j >> 1) == 0 ? wv[r].x : (j >> 1) == 1 ? wv[r].y : (j >> 1) == 2 ? wv[r].z : wv[r].w;
        const uint32_t h16 = (j & 1) ? (word >> 16) : (word & 0xFFFFu);         // two bytes = four codes, low nibble first
        const __half2_raw lo = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(h16 & 0xFFu), __NV_E2M1);
        const __half2_raw hi = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(h16 >> 8), __NV_E2M1);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo)), c = __half22float2(*reinterpret_cast<const __half2*>(&hi));
#pragma unroll
        for (int m = 0; m < MM; ++m)
          part[r][m][j >> 2] = fmaf(xv[m].x, a.x, fmaf(xv[m].y, a.y, fmaf(xv[m].z, c.x, fmaf(xv[m].w, c.y, part[r][m][j >> 2]))));
      }
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const float s0 = NV ? gl_e4m3_to_float(sv[r] & 0xFFu) : gl_e8m0_to_float(sv[r] & 0xFFu);
      const float s1 = NV ? gl_e4m3_to_float(sv[r] >> 8) : s0;
#pragma unroll
      for (int m = 0; m < MM; ++m) acc[r][m] = fmaf(part[r][m][1], s1, fmaf(part[r][m][0], s0, acc[r][m]));
    }
  };
  for (int i = 0; i < steps; i += 2) {
    step(i, buf[0], sbuf[0]);
    if (i + 1 < steps) step(i + 1, buf[1], sbuf[1]);
  }
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int m = 0; m < MM; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[r][m] = v;
    }
  if (lane == 0) {
    const float meta = (NV && p.meta_scale != nullptr) ? *p.meta_scale : 1.f;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int n = n0 + r;
      if (n >= p.N) break;
      const float bi = p.bias != nullptr ? gl_load_as_float(p.bias, n, p.out_dtype) : 0.f;
#pragma unroll
      for (int m = 0; m < MM; ++m) gl_store_out(p.out, (int64_t)m * p.N + n, fmaf(acc[r][m], meta, bi), p.out_dtype);
    }
  }
}

size_t smem_bytes(int M, int K) { return (size_t)M * ((K / 16 + 31) / 32) * 512 * sizeof(float); }

}  // namespace

static bool w8_grouped(const gl_matmul_args* a) {       // weight-only MXFP8: e4m3 weights, e8m0 scale per 32, 16-bit activations
  return gl_is_mx(a->input_dtype) && a->w_dtype == GL_FP8 && a->group_size == 32 && a->channel_scale_mode == 0 &&
         a->scales != nullptr && a->scales_x == nullptr && a->K % 32 == 0;
}

bool gl_w8_gemv_supported(const gl_matmul_args* a) {
  if (a->M < 1 || a->M > kMaxM || a->W_nbits != 8 || a->elements_per_sample != 1) return false;
  if (!(a->w_dtype == GL_INT8 || a->w_dtype == GL_FP8)) return false;
  if (!(a->x_dtype == GL_FP16 || a->x_dtype == GL_BF16)) return false;
  if (a->w_stride_k != 1 || a->w_stride_n != a->K || a->K % 16 != 0 || ((uintptr_t)a->w & 15)) return false;
  if (gl_is_mx(a->input_dtype)) return w8_grouped(a) && smem_bytes(a->M, a->K) <= kSmemLimit;
  if (a->input_dtype != a->x_dtype) return false;
  const bool pre = a->W_group_mode == 2 && a->channel_scale_mode == 0 && a->group_size == a->K;   // one scale per channel, applied to the weights
  const bool post = a->W_group_mode == 0 && a->channel_scale_mode == 1;
  const bool none = a->W_group_mode == 0 && a->channel_scale_mode == 0;
  if (!(pre || post || none)) return false;
  if ((pre || post) && a->scales == nullptr) return false;
  if (pre && a->s_stride_n != 1) return false;
  return smem_bytes(a->M, a->K) <= kSmemLimit;
}

int gl_w8_gemv_launch(const gl_matmul_args* a, cudaStream_t st) {
  W8Params p;
  p.x = a->x; p.w = reinterpret_cast<const uint8_t*>(a->w); p.scales = a->scales; p.bias = a->bias; p.out = a->out;
  p.M = a->M; p.N = a->N; p.K = a->K; p.x_dtype = a->x_dtype; p.out_dtype = a->out_dtype; p.scales_dtype = a->meta_dtype;
  const bool grouped = gl_is_mx(a->input_dtype);
  p.is_fp8 = a->w_dtype == GL_FP8; p.has_scale = (!grouped && (a->W_group_mode == 2 || a->channel_scale_mode == 1)) ? 1 : 0;
  p.s_stride_g = a->s_stride_g; p.s_stride_n = a->s_stride_n;
  const size_t smem = smem_bytes(a->M, a->K);
  const dim3 grid((unsigned)gl_cdiv(a->N, kWarps * kRows)), block(kWarps * 32);
#define GL_W8(MM)                                                                                                   \
  case MM: {                                                                                                        \
    if (grouped)  { GL_CUDA_CHECK(cudaFuncSetAttribute(gl_w8_gemv_kernel<MM, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit)); \
                    GL_CUDA_CHECK(gl_launch_pdl(gl_w8_gemv_kernel<MM, true, true>, grid, block, smem, st, p)); }    \
    else if (p.is_fp8) { GL_CUDA_CHECK(cudaFuncSetAttribute(gl_w8_gemv_kernel<MM, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit)); \
                    GL_CUDA_CHECK(gl_launch_pdl(gl_w8_gemv_kernel<MM, true>, grid, block, smem, st, p)); }          \
    else          { GL_CUDA_CHECK(cudaFuncSetAttribute(gl_w8_gemv_kernel<MM, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit)); \
                    GL_CUDA_CHECK(gl_launch_pdl(gl_w8_gemv_kernel<MM, false>, grid, block, smem, st, p)); }         \
    return GL_OK; }
  switch (a->M) { GL_W8(1) GL_W8(2) GL_W8(3) GL_W8(4) }
#undef GL_W8
  GL_FAIL(GL_E_UNSUPPORTED, "gl_matmul: weight-only 8-bit decode kernel takes 1..4 rows");
}

bool gl_w4mx_gemv_supported(const gl_matmul_args* a) {
  if (a->M < 1 || a->M > kMaxM || a->W_nbits != 4 || a->elements_per_sample != 2 || !gl_is_mx(a->input_dtype)) return false;
  if (a->w_dtype != GL_UINT8 || !(a->x_dtype == GL_FP16 || a->x_dtype == GL_BF16)) return false;       // weight-only: 16-bit activations
  if (a->channel_scale_mode != 0 || a->scales == nullptr || a->scales_x != nullptr) return false;
  if (!(a->group_size == 32 || a->group_size == 16) || a->K % 32 != 0) return false;
  if (a->w_stride_k != 1 || a->w_stride_n != a->K / 2 || ((uintptr_t)a->w & 15)) return false;
  return (size_t)a->M * ((a->K / 32 + 31) / 32) * 1024 * sizeof(float) <= kSmemLimit;
}

int gl_w4mx_gemv_launch(const gl_matmul_args* a, cudaStream_t st) {
  W4Params p;
  p.x = a->x; p.w = reinterpret_cast<const uint8_t*>(a->w); p.scales = reinterpret_cast<const uint8_t*>(a->scales);
  p.meta_scale = a->meta_scale; p.bias = a->bias; p.out = a->out;
  p.M = a->M; p.N = a->N; p.K = a->K; p.x_dtype = a->x_dtype; p.out_dtype = a->out_dtype; p.group = a->group_size;
  p.s_stride_g = a->s_stride_g; p.s_stride_n = a->s_stride_n;
  const size_t smem = (size_t)a->M * ((a->K / 32 + 31) / 32) * 1024 * sizeof(float);
  const dim3 grid((unsigned)gl_cdiv(a->N, kWarps * kRows)), block(kWarps * 32);
  const bool nv = a->group_size == 16;
#define GL_W4(MM)                                                                                                   \
  case MM: {                                                                                                        \
    if (nv) { GL_CUDA_CHECK(cudaFuncSetAttribute(gl_w4mx_gemv_kernel<MM, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit)); \
              GL_CUDA_CHECK(gl_launch_pdl(gl_w4mx_gemv_kernel<MM, true>, grid, block, smem, st, p)); }              \
    else    { GL_CUDA_CHECK(cudaFuncSetAttribute(gl_w4mx_gemv_kernel<MM, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit)); \
              GL_CUDA_CHECK(gl_launch_pdl(gl_w4mx_gemv_kernel<MM, false>, grid, block, smem, st, p)); }             \
    return GL_OK; }
  switch (a->M) { GL_W4(1) GL_W4(2) GL_W4(3) GL_W4(4) }
#undef GL_W4
  GL_FAIL(GL_E_UNSUPPORTED, "gl_matmul: weight-only fp4 decode kernel takes 1..4 rows");
}
