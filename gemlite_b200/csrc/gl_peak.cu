// Tensor-pipe ceiling of this GPU for the MMA kinds the GEMM kernels use: back-to-back tcgen05.mma on operand tiles
// that stay resident in shared memory (no loads, no epilogue), one CTA per SM.  MEASURED_PEAKS-style figures exist
// for bf16 only (a cuBLAS GEMM); the FP8 / FP4 roofline denominators come from here, measured in the same process and
// under the same power cap as the kernels they are compared with.  The operand bytes are pseudo-random (all-zero
// tiles would draw less power and clock higher than real data).
#include "gl_tc_common.cuh"
#include <string.h>

using namespace gltc;

namespace {

template <int KIND>
__global__ void __launch_bounds__(128, 1) gl_mma_peak_kernel(int iters, uint32_t idesc, int* status) {
  constexpr int BN = 256;
  constexpr bool MX = (KIND == KIND_MXF4 || KIND == KIND_NVF4);
  constexpr int SF_ATOMS = KIND == KIND_MXF4 ? 2 : (KIND == KIND_NVF4 ? 4 : 0);
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  unsigned char* a_tile = smem;                            // 128 rows x 128 B, 128-byte swizzle (content is arbitrary)
  unsigned char* b_tile = smem + 128 * 128;                // 256 rows x 128 B
  unsigned char* sf = b_tile + BN * 128;                   // scale-factor atoms, all 1.0
  uint64_t* bar = reinterpret_cast<uint64_t*>(sf + 8 * 512);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5;
  // finite operands for every kind: fp8 bytes without the all-ones exponent, fp4 nibbles are always finite
  uint32_t seed = 0x9E3779B9u * (blockIdx.x + 1) + threadIdx.x;
  for (int i = threadIdx.x; i < (128 + BN) * 128 / 4; i += blockDim.x) {
    seed = seed * 1664525u + 1013904223u;
    reinterpret_cast<uint32_t*>(smem)[i] = (seed >> 4) & 0xB7B7B7B7u;   // random sign, small exponent
  }
  for (int i = threadIdx.x; i < 8 * 512 / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(sf)[i] = KIND == KIND_MXF4 ? 0x7F7F7F7Fu : 0x38383838u;   // e8m0 1.0 / ue4m3 1.0
  if (threadIdx.x == 0) { s_abort = 0; mbar_init(bar, 1); fence_barrier_init(); }
  fence_proxy_async_smem();
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 32) {
    const uint32_t sa = smem_u32(a_tile), sb = smem_u32(b_tile), ss = smem_u32(sf);
    if (MX) {
      for (int a = 0; a < SF_ATOMS; ++a) {
        tmem_cp_sf(tmem_base + 256 + a * 4, smem_desc_sf(ss + a * 512));
        tmem_cp_sf(tmem_base + 256 + 16 + a * 8, smem_desc_sf(ss + a * 512));
        tmem_cp_sf(tmem_base + 256 + 16 + a * 8 + 4, smem_desc_sf(ss + a * 512));
      }
    }
    const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sb);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t accum = (it > 0 || j > 0) ? 1u : 0u;
        if constexpr (KIND == KIND_MXF4) {
          const uint32_t sfid = (uint32_t)(2 * (j & 1));
          mma_ss_block_scaled<KIND>(tmem_base, da + 2 * j, db + 2 * j, idesc | (sfid << 29) | (sfid << 4),
                                    tmem_base + 256 + (j >> 1) * 4, tmem_base + 256 + 16 + (j >> 1) * 8, accum);
        } else if constexpr (KIND == KIND_NVF4) {
          mma_ss_block_scaled<KIND>(tmem_base, da + 2 * j, db + 2 * j, idesc, tmem_base + 256 + j * 4, tmem_base + 256 + 16 + j * 8, accum);
        } else {
          mma_ss<KIND>(tmem_base, da + 2 * j, db + 2 * j, idesc, accum);
        }
      }
    }
    tc_commit(bar);
    mbar_wait(bar, 0u, &s_abort, status, 9);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

template <int KIND>
int launch_peak(int iters, uint32_t idesc, int* status, cudaStream_t st) {
  const size_t smem = 1024 + (128 + 256) * 128 + 8 * 512 + 64;
  auto kern = gl_mma_peak_kernel<KIND>;
  GL_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<gl_num_sms(), 128, smem, st>>>(iters, idesc, status);
  GL_LAUNCH_CHECK("gl_mma_peak_kernel");
  return GL_OK;
}

}  // namespace

// kind: GL_BF16, GL_FP8, GL_INT8, GL_MXFP4 or GL_NVFP4.  Enqueues one kernel in which every SM issues `iters` x 4
// MMAs of 128 x 256 x (32 bytes of K); *flops_out = the floating-point (or integer) operations of the whole launch.
// The caller times the launch with events.  `status_word` = 4 device bytes, zero (set if the final wait runs out).
extern "C" int gl_mma_peak(int32_t kind, int32_t iters, void* status_word, double* flops_out, void* stream) {
  if (iters < 1 || status_word == nullptr) GL_FAIL(GL_E_INVALID, "gl_mma_peak: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  int* status = reinterpret_cast<int*>(status_word);
  int k_per_mma = 0, rc = GL_E_INVALID;
  switch (kind) {
    case GL_BF16: k_per_mma = 16; rc = launch_peak<KIND_F16>(iters, gl_idesc(1, 1, 1, 128, 256), status, st); break;
    case GL_FP8: k_per_mma = 32; rc = launch_peak<KIND_F8F6F4>(iters, gl_idesc(1, 0, 0, 128, 256), status, st); break;
    case GL_INT8: k_per_mma = 32; rc = launch_peak<KIND_I8>(iters, gl_idesc(2, 1, 1, 128, 256), status, st); break;
    case GL_MXFP4: k_per_mma = 64; rc = launch_peak<KIND_MXF4>(iters, gl_idesc_block_scaled(1, 1, 128, 256), status, st); break;
    case GL_NVFP4: k_per_mma = 64; rc = launch_peak<KIND_NVF4>(iters, gl_idesc_block_scaled(1, 0, 128, 256), status, st); break;
    default: GL_FAIL(GL_E_INVALID, "gl_mma_peak: kind %d", kind);
  }
  if (flops_out) *flops_out = 2.0 * 128 * 256 * k_per_mma * 4.0 * iters * gl_num_sms();
  return rc;
}
