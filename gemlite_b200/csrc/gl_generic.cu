// General CUDA-core kernel: every (W_nbits, packing width, W_group_mode, channel_scale_mode,
// dtype, stride) combination the reference's five Triton families accept
// (gemlite/triton_kernels/gemm_kernels.py:285-496 for integer / fp8 / fp16 weights,
// :509-737 for MX / NV block-scaled weights), computed the way those kernels define it:
// unpack -> dequantise in the scale dtype (triton_kernels/utils.py:73-105) -> multiply with
// the activations -> fp32 (int32 for INT8 x INT8) accumulation -> channel scales -> bias.
// Eight threads share one output column (one K slice each, added in slice order) for up to MBG batch rows; it is the
// correctness-complete path for shapes and modes that the streaming and tensor-core kernels
// do not specialise, not a fast path.
#include "gl_common.cuh"

namespace {

constexpr int MBG = 4;

struct GenParams {
  gl_matmul_args a;
  int is_mx;        // block-scaled (e2m1 / e4m3 weights + e8m0 / e4m3 group scales)
  int int_acc;      // INT8 x integer weights: exact int32 accumulation
  int gx;           // activation scale group size (mode 4)
  int sx_stride;    // activation scale row stride (mode 4) = K / gx
};

__device__ __forceinline__ uint64_t load_word(const void* w, int64_t idx, int dt) {
  switch (dt) {
    case GL_UINT8: case GL_INT8: case GL_FP8: case GL_FP8E5: return reinterpret_cast<const uint8_t*>(w)[idx];
    case GL_INT16: case GL_UINT16: case GL_FP16: case GL_BF16: return reinterpret_cast<const uint16_t*>(w)[idx];
    case GL_INT32: case GL_UINT32: case GL_FP32: return reinterpret_cast<const uint32_t*>(w)[idx];
    default: return reinterpret_cast<const uint64_t*>(w)[idx];
  }
}

// A CTA is 32 columns x KS slices of K: thread (x, y) walks the packed words of slice y of column x, the slices are
// added in slice order through shared memory (deterministic), slice 0 finishes the column.
constexpr int KS = 8;

__global__ void __launch_bounds__(32 * KS) gl_generic_kernel(const GenParams p) {
  const gl_matmul_args& a = p.a;
  const int n = blockIdx.x * 32 + threadIdx.x;
  const int m0 = blockIdx.y * MBG;
  const bool valid = n < a.N;
  const int e = a.elements_per_sample;
  const uint64_t mask = (a.W_nbits >= 64) ? ~0ull : ((1ull << a.W_nbits) - 1ull);
  const int gs = a.group_size;
  const int wgm = a.W_group_mode;
  float acc[MBG];
  int iacc[MBG];
#pragma unroll
  for (int i = 0; i < MBG; ++i) { acc[i] = 0.f; iacc[i] = 0; }

  float zscalar = 0.f;
  if (a.zero_is_scalar && a.zeros) zscalar = gl_load_as_float(a.zeros, 0, a.zeros_dtype);
  const bool x_fp4 = p.is_mx && a.x_dtype == GL_UINT8;   // activations packed e2m1, two per byte

  // channel_scale_mode 5 (128 x 128 block quantisation, gemm_kernels.py:396-450): the sum over each block of 128 k is
  // multiplied by the activation scale of (row, block) and the weight scale of (block, n / 128) before it is added
  const bool block_quant = !p.is_mx && a.channel_scale_mode == 5;
  float bacc[MBG];
  int biacc[MBG];
#pragma unroll
  for (int i = 0; i < MBG; ++i) { bacc[i] = 0.f; biacc[i] = 0; }

  const int kwords = a.K / e, per = (kwords + KS - 1) / KS;
  const int kw_begin = min(kwords, (int)threadIdx.y * per), kw_end = valid ? min(kwords, kw_begin + per) : kw_begin;
  for (int kw = kw_begin; kw < kw_end; ++kw) {
    const uint64_t word = load_word(a.w, (int64_t)kw * a.w_stride_k + (int64_t)n * a.w_stride_n, a.w_dtype);
    for (int j = 0; j < e; ++j) {
      const int k = kw * e + j;
      const int g = k / gs;
      float b;
      int bi = 0;
      if (p.is_mx) {
        // weights: e2m1 nibbles (e == 2) or e4m3 bytes (e == 1); group scale e8m0 or e4m3
        const uint32_t q = (uint32_t)((word >> (j * a.W_nbits)) & mask);
        b = (e == 2) ? gl_e2m1_to_float(q) : gl_e4m3_to_float(q);
        const uint32_t sb = reinterpret_cast<const uint8_t*>(a.scales)[(int64_t)g * a.s_stride_g + (int64_t)n * a.s_stride_n];
        b *= (gs == 16) ? gl_e4m3_to_float(sb) : gl_e8m0_to_float(sb);
      } else {
        if (e > 1 || a.w_dtype == GL_UINT8) {
          bi = (int)((word >> (j * a.W_nbits)) & mask);
          b = (float)bi;
        } else if (a.w_dtype == GL_INT8) { bi = (int)(int8_t)word; b = (float)bi; }
        else if (a.w_dtype == GL_FP8) b = gl_e4m3_to_float((uint32_t)word);
        else if (a.w_dtype == GL_FP8E5) b = gl_e5m2_to_float((uint32_t)word);
        else if (a.w_dtype == GL_FP16) b = __half2float(__ushort_as_half((unsigned short)word));
        else if (a.w_dtype == GL_BF16) b = __uint_as_float((uint32_t)word << 16);
        else if (a.w_dtype == GL_FP32) b = __uint_as_float((uint32_t)word);
        else { bi = (int)word; b = (float)bi; }
        float s = 1.f, z = 0.f;
        if (wgm >= 2) s = gl_load_as_float(a.scales, (int64_t)g * a.s_stride_g + (int64_t)n * a.s_stride_n, a.meta_dtype);
        if (wgm == 1 || wgm >= 3)
          z = a.zero_is_scalar ? zscalar
                               : gl_load_as_float(a.zeros, (int64_t)g * a.s_stride_g + (int64_t)n * a.s_stride_n, a.zeros_dtype);
        // dequantize(): arithmetic in the scale dtype, one rounding per op as Triton does
        const int md = a.meta_dtype;
        if (wgm == 1) { b = gl_round_to(b - z, md); bi -= (int)z; }
        else if (wgm == 2) b = gl_round_to(b * s, md);
        else if (wgm == 3) b = a.zero_is_scalar ? gl_round_to((b - z) * s, md) : gl_round_to(gl_round_to(b - z, md) * s, md);
        else if (wgm == 4) b = gl_round_to(fmaf(b, s, z), md);
        // tl.dot(a, b.to(input_dtype)): weights are cast to the activation dtype
        if (a.x_dtype == GL_BF16 || a.x_dtype == GL_FP16) b = gl_round_to(b, a.x_dtype);
        else if (a.x_dtype == GL_FP8) b = gl_e4m3_to_float(__nv_cvt_float_to_fp8(b, __NV_SATFINITE, __NV_E4M3));
      }
#pragma unroll
      for (int i = 0; i < MBG; ++i) {
        const int m = m0 + i;
        if (m >= a.M) break;
        if (block_quant) {
          if (p.int_acc) biacc[i] += (int)reinterpret_cast<const int8_t*>(a.x)[(int64_t)m * a.K + k] * bi;
          else bacc[i] = fmaf(gl_load_as_float(a.x, (int64_t)m * a.K + k, a.x_dtype), b, bacc[i]);
          if ((k & 127) == 127 || kw == kw_end - 1) {        // end of the block, or of this thread's share of it
            const int kb = k >> 7;
            const float sc = reinterpret_cast<const float*>(a.scales_x)[(int64_t)m * (a.K / 128) + kb] *
                             gl_load_as_float(a.scales, (int64_t)kb * a.s_stride_g + (int64_t)(n >> 7) * a.s_stride_n, a.meta_dtype);
            acc[i] = fmaf(p.int_acc ? (float)biacc[i] : bacc[i], sc, acc[i]);
            bacc[i] = 0.f; biacc[i] = 0;
          }
        } else if (p.int_acc) {
          iacc[i] += (int)reinterpret_cast<const int8_t*>(a.x)[(int64_t)m * a.K + k] * bi;
        } else {
          float xv;
          if (x_fp4) {
            const uint32_t byte = reinterpret_cast<const uint8_t*>(a.x)[(int64_t)m * (a.K / 2) + (k >> 1)];
            xv = gl_e2m1_to_float((k & 1) ? (byte >> 4) : (byte & 15u));
          } else {
            xv = gl_load_as_float(a.x, (int64_t)m * a.K + k, a.x_dtype);
          }
          if (p.is_mx && a.channel_scale_mode == 4) {
            const int kg = k / p.gx;
            const int64_t si = a.sx_layout == 0 ? (int64_t)m * p.sx_stride + kg
                                                : ((int64_t)(m >> 7) * (p.sx_stride >> 2) + (kg >> 2)) * 512 + (m & 31) * 16 + ((m & 127) >> 5) * 4 + (kg & 3);
            const uint32_t sa = reinterpret_cast<const uint8_t*>(a.scales_x)[si];
            xv *= (p.gx == 16) ? gl_e4m3_to_float(sa) : gl_e8m0_to_float(sa);
          }
          acc[i] = fmaf(xv, b, acc[i]);
        }
      }
    }
  }

  __shared__ float s_acc[KS][MBG][32];
  __shared__ int s_iacc[KS][MBG][32];
#pragma unroll
  for (int i = 0; i < MBG; ++i) { s_acc[threadIdx.y][i][threadIdx.x] = acc[i]; s_iacc[threadIdx.y][i][threadIdx.x] = iacc[i]; }
  __syncthreads();
  if (threadIdx.y != 0 || !valid) return;
#pragma unroll
  for (int i = 0; i < MBG; ++i)
    for (int y = 1; y < KS; ++y) { acc[i] += s_acc[y][i][threadIdx.x]; iacc[i] += s_iacc[y][i][threadIdx.x]; }

  const int md = (a.meta_dtype == GL_FP16 || a.meta_dtype == GL_BF16 || a.meta_dtype == GL_FP32) ? a.meta_dtype : GL_FP32;
#pragma unroll
  for (int i = 0; i < MBG; ++i) {
    const int m = m0 + i;
    if (m >= a.M) break;
    float v = (p.int_acc && !block_quant) ? (float)iacc[i] : acc[i];
    if (p.is_mx) {
      if (gs == 16 && a.meta_scale) v *= *a.meta_scale;
      if (a.channel_scale_mode == 2) v *= reinterpret_cast<const float*>(a.scales_x)[m];
    } else {
      const int csm = a.channel_scale_mode;
      if (csm == 1) v = gl_round_to(gl_round_to(v, md) * gl_load_as_float(a.scales, n, a.meta_dtype), md);
      else if (csm == 2) v = gl_round_to(gl_round_to(v, md) * reinterpret_cast<const float*>(a.scales_x)[m], md);
      else if (csm == 3) v = gl_round_to(gl_round_to(v, md) * (reinterpret_cast<const float*>(a.scales_x)[m] * gl_load_as_float(a.scales, n, a.meta_dtype)), md);
    }
    if (a.bias) v += gl_load_as_float(a.bias, n, a.out_dtype);
    gl_store_out(a.out, (int64_t)m * a.N + n, v, a.out_dtype);
  }
}

}  // namespace

int gl_generic_launch(const gl_matmul_args* a, cudaStream_t st) {
  GenParams p;
  p.a = *a;
  p.is_mx = gl_is_mx(a->input_dtype) ? 1 : 0;
  p.gx = a->group_size;
  p.sx_stride = a->K / (a->group_size > 0 ? a->group_size : 1);
  p.int_acc = 0;
  if (a->channel_scale_mode == 5) {
    if (p.is_mx || a->W_nbits != 8 || a->elements_per_sample != 1 || a->W_group_mode != 0)
      GL_FAIL(GL_E_UNSUPPORTED, "gl_matmul: channel_scale_mode 5 (128x128 block quantisation) takes unpacked 8-bit weights without group modes");
    if (a->scales == nullptr || a->scales_x == nullptr || a->K % 128 != 0)
      GL_FAIL(GL_E_INVALID, "gl_matmul: channel_scale_mode 5 needs block scales, per-block activation scales and K %% 128 == 0");
  }
  if (!p.is_mx && a->input_dtype == GL_INT8 && a->x_dtype == GL_INT8) {
    if (a->W_group_mode == 0 || (a->W_group_mode == 1)) p.int_acc = 1;
  }
  if (p.is_mx) {
    if (!(a->elements_per_sample == 1 || a->elements_per_sample == 2)) GL_FAIL(GL_E_INVALID, "gl_matmul: MX weights need elements_per_sample 1 or 2");
    if (a->scales == nullptr) GL_FAIL(GL_E_INVALID, "gl_matmul: MX weights need group scales");
    if (a->channel_scale_mode == 4 && a->scales_x == nullptr) GL_FAIL(GL_E_INVALID, "gl_matmul: channel_scale_mode 4 needs activation scales");
  }
  if ((a->channel_scale_mode == 2 || a->channel_scale_mode == 3) && a->scales_x == nullptr)
    GL_FAIL(GL_E_INVALID, "gl_matmul: channel_scale_mode %d needs activation scales", a->channel_scale_mode);
  dim3 block(32, KS), grid((unsigned)gl_cdiv(a->N, 32), (unsigned)gl_cdiv(a->M, MBG));
  gl_generic_kernel<<<grid, block, 0, st>>>(p);
  GL_LAUNCH_CHECK("gl_generic_kernel");
  return GL_OK;
}
