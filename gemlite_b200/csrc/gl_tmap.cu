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

int gl_make_tmap_sf_replicated(CUtensorMap* out, const void* base, uint64_t k_atoms, uint64_t blocks, uint32_t box_atoms) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) GL_FAIL(GL_E_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  if ((uintptr_t)base & 15) GL_FAIL(GL_E_INVALID, "TMA operand must be 16-byte aligned");
  cuuint64_t dims[4] = {128, 4, k_atoms, blocks};
  cuuint64_t strides[3] = {0, 512, 512 * k_atoms};      // the replica dimension re-reads the same 512 bytes
  cuuint32_t box[4] = {128, 4, box_atoms, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) GL_FAIL(GL_E_CUDA, "cuTensorMapEncodeTiled (scale atoms) failed with code %d (k atoms %llu blocks %llu)", (int)r,
                                 (unsigned long long)k_atoms, (unsigned long long)blocks);
  return GL_OK;
}
