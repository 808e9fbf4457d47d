// C-ABI entry points: error state, build info, kernel-family selection and gl_matmul dispatch.
#include "gl_common.cuh"
#include <string.h>
#include <mutex>

static thread_local char g_err[512] = "";

void gl_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int gl_num_sms() {
  static int cached[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 148; }
  std::lock_guard<std::mutex> lk(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 148; }
    cached[dev] = n;
  }
  return cached[dev];
}

extern "C" int gl_abi_version(void) { return GL_ABI_VERSION; }
extern "C" const char* gl_last_error(void) { return g_err; }
extern "C" const char* gl_build_info(void) {
#define GL_STR2(x) #x
#define GL_STR(x) GL_STR2(x)
  return "gemlite_b200 sm_100a nvcc " GL_STR(__CUDACC_VER_MAJOR__) "." GL_STR(__CUDACC_VER_MINOR__) "." GL_STR(__CUDACC_VER_BUILD__);
}

// gemlite/core.py:163-179
extern "C" int gl_get_matmul_type(int32_t M, int32_t W_nbits, int32_t is_mx_dtype) {
  if (M >= 64) return GL_MM_GEMM;
  const int gemv_limit = (W_nbits < 8 && !is_mx_dtype) ? 4 : 2;
  if (M > gemv_limit) return GL_MM_GEMM_SPLITK;
  if (is_mx_dtype) return GL_MM_GEMM_SPLITK;
  return (W_nbits < 8) ? GL_MM_GEMV_REVSPLITK : GL_MM_GEMV_SPLITK;
}

enum KernelId { K_INVALID = 0, K_STREAM, K_TC, K_W8, K_W4MX, K_GENERIC };

int gl_validate_matmul_args(const gl_matmul_args* a) {
  if (a == nullptr) GL_FAIL(GL_E_INVALID, "gl_matmul: null argument struct");
  if (a->M < 0 || a->N <= 0 || a->K <= 0) GL_FAIL(GL_E_INVALID, "gl_matmul: bad shape M=%d N=%d K=%d", a->M, a->N, a->K);
  if (a->x == nullptr || a->w == nullptr || a->out == nullptr) GL_FAIL(GL_E_INVALID, "gl_matmul: null x / w / out pointer");
  if (!(a->W_nbits == 1 || a->W_nbits == 2 || a->W_nbits == 4 || a->W_nbits == 8 || a->W_nbits == 16 || a->W_nbits == 32))
    GL_FAIL(GL_E_INVALID, "gl_matmul: unsupported W_nbits %d", a->W_nbits);
  if (a->elements_per_sample < 1 || a->K % a->elements_per_sample != 0)
    GL_FAIL(GL_E_INVALID, "gl_matmul: K=%d not a multiple of elements_per_sample=%d", a->K, a->elements_per_sample);
  if (a->group_size < 1 || a->K % a->group_size != 0)
    GL_FAIL(GL_E_INVALID, "gl_matmul: K=%d not a multiple of group_size=%d", a->K, a->group_size);
  if (a->matmul_type < GL_MM_AUTO || a->matmul_type > GL_MM_GEMM) GL_FAIL(GL_E_INVALID, "gl_matmul: bad matmul_type %d", a->matmul_type);
  if (a->W_group_mode < 0 || a->W_group_mode > 4) GL_FAIL(GL_E_INVALID, "gl_matmul: bad W_group_mode %d", a->W_group_mode);
  if (a->channel_scale_mode < 0 || a->channel_scale_mode > 5) GL_FAIL(GL_E_INVALID, "gl_matmul: bad channel_scale_mode %d", a->channel_scale_mode);
  if (!(a->out_dtype == GL_FP16 || a->out_dtype == GL_BF16 || a->out_dtype == GL_FP32))
    GL_FAIL(GL_E_INVALID, "gl_matmul: output dtype %d must be FP16 / BF16 / FP32", a->out_dtype);
  if (gl_dtype_size(a->x_dtype) == 0 || gl_dtype_size(a->w_dtype) == 0) GL_FAIL(GL_E_INVALID, "gl_matmul: unknown x / w dtype");
  if (a->W_group_mode >= 2 && a->scales == nullptr) GL_FAIL(GL_E_INVALID, "gl_matmul: W_group_mode %d needs scales", a->W_group_mode);
  if ((a->W_group_mode == 1 || a->W_group_mode >= 3) && a->zeros == nullptr) GL_FAIL(GL_E_INVALID, "gl_matmul: W_group_mode %d needs zeros", a->W_group_mode);
  if ((a->channel_scale_mode == 1 || a->channel_scale_mode == 3) && a->scales == nullptr) GL_FAIL(GL_E_INVALID, "gl_matmul: channel_scale_mode %d needs scales", a->channel_scale_mode);
  for (int i = 0; i < 2; ++i) if (a->reserved[i] != 0) GL_FAIL(GL_E_INVALID, "gl_matmul: reserved fields must be 0");
  return GL_OK;
}

namespace {

// which kernel serves (family, problem)
KernelId select(const gl_matmul_args* a, int* family_out) {
  const bool mx = gl_is_mx(a->input_dtype);
  int fam = a->matmul_type;
  if (fam == GL_MM_AUTO) fam = gl_get_matmul_type(a->M, a->W_nbits, mx ? 1 : 0);
  if (family_out) *family_out = fam;
  if (mx && (fam == GL_MM_GEMV_REVSPLITK || fam == GL_MM_GEMV_SPLITK)) return K_INVALID;  // as the reference: MX only on GEMV / GEMM*
  if (a->kernel_override == 1) return K_GENERIC;
  if (a->kernel_override == 2 && gl_gemm_tc_supported(a)) return K_TC;
  // decode sizes stream; from M = 17 the tensor-core kernel is faster (measured on 8192 x 8192 A16W4 at M = 32: 30 us
  // with the operands swapped, 44 us as two 16-row launches of the streaming kernel), and the streaming kernel only
  // covers what that kernel cannot take (17..32 rows as two launches of 16 rows where a plan exists)
  const bool stream_ok = !mx && gl_gemv_stream_supported(a);
  if (stream_ok && a->M <= 16) return K_STREAM;
  if (gl_gemm_tc_supported(a)) return K_TC;
  if (stream_ok) return K_STREAM;
  if (gl_w8_gemv_supported(a)) return K_W8;                // (also weight-only MXFP8)
  if (mx && gl_w4mx_gemv_supported(a)) return K_W4MX;
  return K_GENERIC;
}

}  // namespace

extern "C" uint64_t gl_matmul_workspace_bytes(const gl_matmul_args* a) {
  if (a == nullptr || a->M <= 0) return 0;
  int fam;
  const KernelId k = select(a, &fam);
  if (k == K_STREAM) return gl_gemv_stream_workspace(a);
  if (k == K_TC) return gl_gemm_tc_workspace(a);
  return 0;
}

extern "C" const char* gl_matmul_kernel_name(const gl_matmul_args* a) {
  if (a == nullptr) return "invalid";
  int fam;
  switch (select(a, &fam)) {
    case K_STREAM: return gl_gemv_stream_kernel_name(a);
    case K_TC: return "gl_gemm_tc_kernel";
    case K_W8: return "gl_w8_gemv_kernel";
    case K_W4MX: return "gl_w4mx_gemv_kernel";
    case K_GENERIC: return "gl_generic_kernel";
    default: return "invalid";
  }
}

extern "C" int gl_matmul(const gl_matmul_args* a, void* stream) {
  if (int rc = gl_validate_matmul_args(a)) return rc;
  if (a->M == 0) return GL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  int fam;
  switch (select(a, &fam)) {
    case K_STREAM: return gl_gemv_stream_launch(a, st);
    case K_TC: return gl_gemm_tc_launch(a, st);
    case K_W8: return gl_w8_gemv_launch(a, st);
    case K_W4MX: return gl_w4mx_gemv_launch(a, st);
    case K_GENERIC: return gl_generic_launch(a, st);
    default:
      GL_FAIL(GL_E_UNSUPPORTED, "gl_matmul: kernel family %d does not support MX / NV block-scaled dtypes", fam);
  }
}
