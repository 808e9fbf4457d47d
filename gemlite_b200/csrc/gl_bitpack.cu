// Bit packing / unpacking kernels, bit-exact with gemlite/bitpack.py:
//   pack over cols  (bitpack.py:36-60, 78-144):  out[r, c] = OR_j in[r, c*e + j] << (j*nbits)
//   pack over rows  (bitpack.py:10-34, 254-318): out[r, c] = OR_j in[r*e + j, c] << (j*nbits)
//   unpack          (bitpack.py:146-251, 320-427): (word >> j*nbits) & (2^nbits - 1)
// e = packing_bitwidth / nbits, field 0 in the least significant bits.  Words are uint8 /
// int16 / int32 / int64 (gemlite/dtypes.py:95-100).  Pure byte traffic: one thread per output
// word (pack) or per input word (unpack), grid-stride, 64-bit index arithmetic.
#include "gl_common.cuh"

namespace {

template <typename WT>
__global__ void pack_cols_kernel(const uint8_t* __restrict__ in, WT* __restrict__ out, int64_t rows, int64_t cols_out,
                                 int nbits, int e) {
  const int64_t total = rows * cols_out;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const uint8_t* src = in + i * e;   // row-major: (r, c*e) == r*cols_in + c*e == i*e
    uint64_t w = 0;
    for (int j = 0; j < e; ++j) w |= (uint64_t)src[j] << (j * nbits);
    out[i] = (WT)w;
  }
}

template <typename WT>
__global__ void pack_rows_kernel(const uint8_t* __restrict__ in, WT* __restrict__ out, int64_t rows_out, int64_t cols,
                                 int nbits, int e) {
  const int64_t total = rows_out * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i % cols;
    uint64_t w = 0;
    for (int j = 0; j < e; ++j) w |= (uint64_t)in[(r * e + j) * cols + c] << (j * nbits);
    out[i] = (WT)w;
  }
}

__device__ __forceinline__ void store_val(void* out, int64_t idx, uint32_t v, int dt) {
  switch (dt) {
    case GL_UINT8: case GL_INT8: reinterpret_cast<uint8_t*>(out)[idx] = (uint8_t)v; break;
    case GL_INT16: case GL_UINT16: reinterpret_cast<uint16_t*>(out)[idx] = (uint16_t)v; break;
    case GL_INT32: case GL_UINT32: reinterpret_cast<uint32_t*>(out)[idx] = v; break;
    case GL_INT64: reinterpret_cast<int64_t*>(out)[idx] = (int64_t)v; break;
    case GL_FP16: reinterpret_cast<__half*>(out)[idx] = __float2half_rn((float)v); break;
    case GL_BF16: reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn((float)v); break;
    default: reinterpret_cast<float*>(out)[idx] = (float)v; break;
  }
}

template <typename WT>
__global__ void unpack_cols_kernel(const WT* __restrict__ in, void* __restrict__ out, int64_t total_words, int nbits,
                                   int e, int out_dtype) {
  const uint64_t mask = (1ull << nbits) - 1ull;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total_words; i += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t w = (uint64_t)in[i];
    for (int j = 0; j < e; ++j) store_val(out, i * e + j, (uint32_t)((w >> (j * nbits)) & mask), out_dtype);
  }
}

template <typename WT>
__global__ void unpack_rows_kernel(const WT* __restrict__ in, void* __restrict__ out, int64_t rows_packed, int64_t cols,
                                   int nbits, int e, int out_dtype) {
  const uint64_t mask = (1ull << nbits) - 1ull;
  const int64_t total = rows_packed * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i % cols;
    const uint64_t w = (uint64_t)in[i];
    for (int j = 0; j < e; ++j) store_val(out, (r * e + j) * cols + c, (uint32_t)((w >> (j * nbits)) & mask), out_dtype);
  }
}

int check_bits(int nbits, int pb) {
  if (!(pb == 8 || pb == 16 || pb == 32 || pb == 64)) { gl_set_error("Unsuported bitpacking width %d", pb); return GL_E_INVALID; }
  if (!(nbits == 8 || nbits == 4 || nbits == 2 || nbits == 1)) { gl_set_error("Unsuported nbits %d", nbits); return GL_E_INVALID; }
  if (nbits > pb) { gl_set_error("W_nbits %d larger than packing width %d", nbits, pb); return GL_E_INVALID; }
  return GL_OK;
}
unsigned grid_for(int64_t total) {
  int64_t b = gl_cdiv(total, 256);
  const int64_t cap = (int64_t)gl_num_sms() * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}
bool out_dtype_ok(int dt) {
  return dt == GL_UINT8 || dt == GL_INT8 || dt == GL_INT16 || dt == GL_UINT16 || dt == GL_INT32 || dt == GL_UINT32 ||
         dt == GL_INT64 || dt == GL_FP16 || dt == GL_BF16 || dt == GL_FP32;
}

}  // namespace


#define GL_PB_SWITCH(pb, CALL)                      \
  switch (pb) {                                     \
    case 8:  { using WT = uint8_t;  CALL; } break;  \
    case 16: { using WT = uint16_t; CALL; } break;  \
    case 32: { using WT = uint32_t; CALL; } break;  \
    default: { using WT = uint64_t; CALL; } break;  \
  }

extern "C" int gl_pack_over_cols(const uint8_t* in, void* out, int64_t rows, int64_t cols, int32_t W_nbits,
                                 int32_t packing_bitwidth, void* stream) {
  if (int rc = check_bits(W_nbits, packing_bitwidth)) return rc;
  const int e = packing_bitwidth / W_nbits;
  if (rows < 0 || cols < 0) GL_FAIL(GL_E_INVALID, "gl_pack_over_cols: negative shape");
  if (cols % e != 0) GL_FAIL(GL_E_INVALID, "gl_pack_over_cols: cols (%lld) not a multiple of %d", (long long)cols, e);
  const int64_t cols_out = cols / e;
  if (rows * cols_out == 0) return GL_OK;
  if (!in || !out) GL_FAIL(GL_E_INVALID, "gl_pack_over_cols: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = grid_for(rows * cols_out);
  GL_PB_SWITCH(packing_bitwidth, (pack_cols_kernel<WT><<<grid, 256, 0, st>>>(in, reinterpret_cast<WT*>(out), rows, cols_out, W_nbits, e)));
  GL_LAUNCH_CHECK("pack_cols_kernel");
  return GL_OK;
}

extern "C" int gl_pack_over_rows(const uint8_t* in, void* out, int64_t rows, int64_t cols, int32_t W_nbits,
                                 int32_t packing_bitwidth, void* stream) {
  if (int rc = check_bits(W_nbits, packing_bitwidth)) return rc;
  const int e = packing_bitwidth / W_nbits;
  if (rows < 0 || cols < 0) GL_FAIL(GL_E_INVALID, "gl_pack_over_rows: negative shape");
  if (rows % e != 0) GL_FAIL(GL_E_INVALID, "gl_pack_over_rows: rows (%lld) not a multiple of %d", (long long)rows, e);
  const int64_t rows_out = rows / e;
  if (rows_out * cols == 0) return GL_OK;
  if (!in || !out) GL_FAIL(GL_E_INVALID, "gl_pack_over_rows: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = grid_for(rows_out * cols);
  GL_PB_SWITCH(packing_bitwidth, (pack_rows_kernel<WT><<<grid, 256, 0, st>>>(in, reinterpret_cast<WT*>(out), rows_out, cols, W_nbits, e)));
  GL_LAUNCH_CHECK("pack_rows_kernel");
  return GL_OK;
}

extern "C" int gl_unpack_over_cols(const void* in, void* out, int64_t rows, int64_t cols_packed, int32_t W_nbits,
                                   int32_t packing_bitwidth, int32_t elements_per_sample, int32_t out_dtype, void* stream) {
  if (int rc = check_bits(W_nbits, packing_bitwidth)) return rc;
  if (!out_dtype_ok(out_dtype)) GL_FAIL(GL_E_INVALID, "gl_unpack_over_cols: unsupported output dtype %d", out_dtype);
  const int e = elements_per_sample;
  if (e < 1 || e * W_nbits > packing_bitwidth) GL_FAIL(GL_E_INVALID, "gl_unpack_over_cols: %d fields of %d bits do not fit a %d-bit word", e, W_nbits, packing_bitwidth);
  if (rows < 0 || cols_packed < 0) GL_FAIL(GL_E_INVALID, "gl_unpack_over_cols: negative shape");
  const int64_t total = rows * cols_packed;
  if (total == 0) return GL_OK;
  if (!in || !out) GL_FAIL(GL_E_INVALID, "gl_unpack_over_cols: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = grid_for(total);
  GL_PB_SWITCH(packing_bitwidth, (unpack_cols_kernel<WT><<<grid, 256, 0, st>>>(reinterpret_cast<const WT*>(in), out, total, W_nbits, e, out_dtype)));
  GL_LAUNCH_CHECK("unpack_cols_kernel");
  return GL_OK;
}

extern "C" int gl_unpack_over_rows(const void* in, void* out, int64_t rows_packed, int64_t cols, int32_t W_nbits,
                                   int32_t packing_bitwidth, int32_t elements_per_sample, int32_t out_dtype, void* stream) {
  if (int rc = check_bits(W_nbits, packing_bitwidth)) return rc;
  if (!out_dtype_ok(out_dtype)) GL_FAIL(GL_E_INVALID, "gl_unpack_over_rows: unsupported output dtype %d", out_dtype);
  const int e = elements_per_sample;
  if (e < 1 || e * W_nbits > packing_bitwidth) GL_FAIL(GL_E_INVALID, "gl_unpack_over_rows: %d fields of %d bits do not fit a %d-bit word", e, W_nbits, packing_bitwidth);
  if (rows_packed < 0 || cols < 0) GL_FAIL(GL_E_INVALID, "gl_unpack_over_rows: negative shape");
  if (rows_packed * cols == 0) return GL_OK;
  if (!in || !out) GL_FAIL(GL_E_INVALID, "gl_unpack_over_rows: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = grid_for(rows_packed * cols);
  GL_PB_SWITCH(packing_bitwidth, (unpack_rows_kernel<WT><<<grid, 256, 0, st>>>(reinterpret_cast<const WT*>(in), out, rows_packed, cols, W_nbits, e, out_dtype)));
  GL_LAUNCH_CHECK("unpack_rows_kernel");
  return GL_OK;
}
