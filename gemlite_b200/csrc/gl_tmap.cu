// Host helper: encode 2-D TMA tensor maps through the driver entry point (no link against libcuda).
#include "gl_tc_common.cuh"
#include <mutex>

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (PFN_encodeTiled)p;
    else
      cudaGetLastError();
  });
  return fn;
}

int gl_make_tmap_2d(CUtensorMap* out, const void* base, int elem_kind, uint64_t inner_elems, uint64_t rows,
                    uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows, bool swizzle128) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) GL_FAIL(GL_E_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  CUtensorMapDataType dt;
  switch (elem_kind) {
    case 0: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case 1: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case 2: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    default: dt = CU_TENSOR_MAP_DATA_TYPE_INT32; break;
  }
  if (((uintptr_t)base & 15) || (row_stride_bytes & 15)) GL_FAIL(GL_E_INVALID, "TMA operand must be 16-byte aligned with a 16-byte multiple row pitch");
  cuuint64_t dims[2] = {inner_elems, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) GL_FAIL(GL_E_CUDA, "cuTensorMapEncodeTiled failed with code %d (inner %llu rows %llu pitch %llu box %u x %u)", (int)r,
                                 (unsigned long long)inner_elems, (unsigned long long)rows, (unsigned long long)row_stride_bytes, box_inner, box_rows);
  return GL_OK;
}
