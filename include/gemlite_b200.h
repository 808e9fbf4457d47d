/*
 * gemlite_b200 — C ABI of the sm_100a low-bit matmul library.
 *
 * Every entry point is `extern "C"`, takes plain pointers / sizes / integer codes and a
 * CUDA stream handle (`void*` = cudaStream_t), never allocates or frees device memory
 * and never synchronises the stream: outputs and scratch are caller-owned.  All functions
 * return 0 on success or a negative GL_E* code; gl_last_error() gives the message of the
 * last failure on the calling thread.
 *
 * Dtype codes are the integer values of the reference's `DType` enum
 * (gemlite/dtypes.py:8-30) so that the `metadata` tensor of a checkpoint can be handed
 * through unchanged.
 *
 * Each declaration names the reference interface it replaces (path inside the
 * reference project : line).
 */
#ifndef GEMLITE_B200_H_
#define GEMLITE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GL_ABI_VERSION 1

#if defined(__GNUC__)
#define GL_API __attribute__((visibility("default")))
#else
#define GL_API
#endif

/* ---- status codes -------------------------------------------------------------------- */
enum {
  GL_OK            = 0,
  GL_E_INVALID     = -1, /* bad argument (shape, dtype, mode, alignment)                  */
  GL_E_UNSUPPORTED = -2, /* combination not implemented by the named kernel family        */
  GL_E_WORKSPACE   = -3, /* workspace too small (see gl_matmul_workspace_bytes)           */
  GL_E_CUDA        = -4, /* a CUDA runtime / driver call failed (launch, tensor map, ...) */
  GL_E_IO          = -5, /* config-cache file could not be read or written                */
  GL_E_NOTFOUND    = -6  /* config-cache lookup miss                                      */
};

/* ---- dtype codes = gemlite/dtypes.py:8-30 ------------------------------------------------ */
enum {
  GL_FP32 = 0, GL_FP16 = 1, GL_BF16 = 2, GL_FP8 = 3, GL_INT8 = 4, GL_UINT8 = 5,
  GL_INT32 = 6, GL_UINT32 = 7, GL_FP8E5 = 8, GL_INT16 = 9, GL_UINT16 = 10, GL_INT64 = 11,
  GL_MXFP16 = 14, GL_MXBF16 = 15, GL_MXFP8 = 16, GL_MXFP4 = 17, GL_NVFP4 = 18, GL_E8M0 = 19
};

/* ---- kernel families = GEMLITE_MATMUL_TYPES order, gemlite/core.py:57-67 ----------------- */
enum {
  GL_MM_AUTO           = -1,
  GL_MM_GEMV           = 0,
  GL_MM_GEMV_REVSPLITK = 1,
  GL_MM_GEMV_SPLITK    = 2,
  GL_MM_GEMM_SPLITK    = 3,
  GL_MM_GEMM           = 4
};

/* W_group_mode / channel_scale_mode: gemlite/core.py:646-703, triton_kernels/utils.py:73-105.
 *   W_group_mode       0 none | 1 b-z | 2 b*s | 3 (b-z)*s | 4 fma(b,s,z')
 *   channel_scale_mode 0 none | 1 *s_w[n] | 2 *s_x[m] | 3 both | 4 block-scaled (MX/NV)
 *                      activations | 5 128x128 block quant                               */

/*
 * One matmul problem  out[M,N] = x[M,K] . dequant(W)[K,N] (+ bias[N]).
 * Replaces the tensor/meta argument lists of gemlite::forward_functional
 * (gemlite/core.py:193-274, 798-817) and the per-family `forward` launchers
 * (e.g. gemlite/triton_kernels/gemm_kernels.py:740-799).
 *
 * Layouts (element strides, as the reference hands them to its kernels):
 *   x        [M,K] row-major, dtype x_dtype (FP16/BF16/FP32, or FP8/INT8/packed-fp4 UINT8
 *            when the activations were quantised by gl_scale_activations_*).
 *   w        packed integer weights: logical [K/e, N] words of w_dtype with strides
 *            (w_stride_k, w_stride_n); e = elements_per_sample k-values per word, value j
 *            of a word in bits [j*W_nbits, (j+1)*W_nbits)  (gemlite/bitpack.py:36-60).
 *            8/16-bit unpacked weights: logical [K,N] with strides (1, K) (the `.t()` view
 *            of [N,K], gemlite/core.py:598-610).  MX/NV fp4: bytes [K/2, N] with strides
 *            (1, K/2), even k in the low nibble.
 *   scales   group-wise: logical [G,N] strides (s_stride_g, s_stride_n), dtype meta_dtype;
 *            channel-wise: N contiguous values; MX/NV: logical [N,G] strides
 *            (s_stride_n, s_stride_g) given the same way (s_stride_g = distance between
 *            groups of one output column).
 *   zeros    same layout as scales, dtype zeros_dtype; or one scalar when zero_is_scalar.
 *            128x128 block quantisation (mode 5): fp32, logical [K/128, N/128] (both rounded up) with
 *            strides (s_stride_g, s_stride_n); unpacked 8-bit weights (gemlite/helper.py:517-617).
 *   scales_x activation scales: [M] fp32 (modes 2/3), [Mpad, K/gx] bytes (mode 4),
 *            [M, K/128] fp32 (mode 5, from gl_scale_activations_per_block).
 *   bias     [N] in out_dtype or NULL.  Fused into the kernel epilogue (the reference adds
 *            it with a separate torch op, gemlite/core.py:271-272).
 *   out      [M,N] row-major, out_dtype (FP16/BF16/FP32).
 */
typedef struct gl_matmul_args {
  const void*  x;
  const void*  w;
  const void*  scales;
  const void*  zeros;
  const void*  scales_x;
  const void*  bias;
  const float* meta_scale;     /* device fp32 scalar multiplied into the result (NVFP4), or NULL */
  void*        out;
  void*        workspace;      /* device scratch, >= gl_matmul_workspace_bytes(); may be NULL if 0 */
  uint64_t     workspace_bytes;
  int32_t      M, N, K;
  int32_t      W_nbits;
  int32_t      group_size;
  int32_t      elements_per_sample;
  int32_t      input_dtype;    /* layer input dtype code (meta_args[5])                     */
  int32_t      x_dtype;        /* dtype of the buffer `x` actually points to                */
  int32_t      w_dtype;        /* dtype of the words `w` points to                          */
  int32_t      out_dtype;
  int32_t      meta_dtype;     /* dtype of `scales`                                         */
  int32_t      zeros_dtype;    /* dtype of `zeros`                                          */
  int32_t      channel_scale_mode;
  int32_t      W_group_mode;
  int32_t      zero_is_scalar;
  int32_t      matmul_type;    /* GL_MM_* ; GL_MM_AUTO applies get_matmul_type()            */
  int64_t      w_stride_k, w_stride_n;
  int64_t      s_stride_g, s_stride_n;
  int32_t      kernel_override; /* 0 = library picks the kernel; 1 = the general CUDA-core kernel; 2 = the tensor-core kernel where it covers the problem (testing / tuning) */
  int32_t      sx_layout;      /* layout of block-scaled `scales_x`: 0 = [Mpad, K/g] rows, 1 = 128x4 scale atoms */
  int32_t      reserved[2];    /* must be 0 */
  const void*  w_scales_atoms; /* optional copy of the MX / NV weight scales as 128x4 scale atoms, or NULL   */
} gl_matmul_args;

/* "128x4 scale atoms": the scale-factor layout block-scaled tcgen05.mma reads, identical to the reference's 5-D
 * pre-shuffled scales [1, R/128, G/4, 2, 256] (gemlite/core.py:748-752): for row r (output column n for
 * weights, batch row m for activations) and group g,
 *   byte offset = ((r/128) * (G/4) + g/4) * 512 + (r%32) * 16 + ((r%128)/32) * 4 + g%4,   G = K / group_size.
 * Rows are padded to a multiple of 128 and G must be a multiple of 4.  The tensor-core kernels for MXFP4 /
 * NVFP4 need both operands' scales in this layout; the general kernel reads the row layouts. */

/* library / build info */
GL_API int         gl_abi_version(void);
GL_API const char* gl_last_error(void);
GL_API const char* gl_build_info(void);   /* "sm_100a nvcc <ver> ..." */

/* Family the automatic dispatcher picks.  Replaces get_matmul_type(), gemlite/core.py:163-179. */
GL_API int gl_get_matmul_type(int32_t M, int32_t W_nbits, int32_t is_mx_dtype);

/* Scratch bytes gl_matmul() needs for `a` (0 for most kernels; the split-K streaming kernel
 * keeps fp32 partial sums and arrival counters there).  The first
 * gl_matmul_counter_bytes() bytes of a workspace must be zero before its FIRST use; the
 * kernels restore them to zero before they finish, so a workspace can be reused by
 * successive calls on one stream without clearing.  Replaces the zero-filled output /
 * 256-slot output ring of the reference's atomics-based GEMV
 * (gemlite/triton_kernels/gemv_revsplitK_kernels.py:460-485). */
GL_API uint64_t gl_matmul_workspace_bytes(const gl_matmul_args* a);
GL_API uint64_t gl_matmul_counter_bytes(void);
/* Byte offset, inside a workspace, of the 32-bit status word of the tensor-core kernels: 0 after a clean launch; a
 * bounded wait that gave up leaves its code there (the launch's output is then undefined).  The library never reads
 * it (no synchronisation): a host that wants to check copies the word after it has synchronised the stream, and after
 * a non-zero status clears the first gl_matmul_counter_bytes() bytes before it uses the workspace again.  No
 * counterpart in the reference (its kernels have no bounded waits). */
GL_API uint64_t gl_matmul_status_offset(void);

/* Launch on `stream`.  Replaces GEMLITE_TRITON_MAPPING[type].forward(...) + the bias add,
 * gemlite/core.py:263-272. */
GL_API int gl_matmul(const gl_matmul_args* a, void* stream);

/* gl_matmul() for callers that cannot hand over a workspace because they cannot allocate one.
 * (No counterpart in the reference: its kernels get their scratch from torch, e.g. the zero-filled output of
 * gemv_revsplitK_forward; this entry point exists for hosts where that is not possible.)
 *
 * Who that is: a plug-in that only receives device pointers from a framework whose allocator it may not call;
 * code on a serving hot path where cudaMalloc / cudaFree would stall the device; a
 * binding from a language runtime that has no device allocator at all.  Such callers still pass x, weights,
 * meta data and `out`; `workspace` / `workspace_bytes` of `a` are ignored.
 *
 * What it runs: the streaming decode kernel (packed 4/2/1-bit weights, fp16/bf16 activations, M <= 32; anything
 * else returns GL_E_UNSUPPORTED) in its split-K-through-scratch form.  The scratch -- arrival counters, a status
 * word and the fp32 partial sums -- is a fixed array of GL_NOALLOC_SCRATCH_BYTES (4 MiB) inside the library.
 * Every GPU that loads the library holds those 4 MiB until the process exits.  A problem whose partial sums do
 * not fit (counter block + slices * M * N * 4 bytes > 4 MiB) is rejected with GL_E_WORKSPACE and a message giving
 * both sizes; use gl_matmul() with your own workspace for it.
 *
 * The call allocates and frees nothing (no cudaMalloc / cudaFree, no allocating library routine).  The first call
 * on each device looks up the array's device address (cudaGetSymbolAddress, with that device current) and caches
 * it: make that first call outside of any stream capture.  Every call clears the counter block on `stream`
 * before the kernel (the array keeps what the previous call left behind) and all calls share the one array, so
 * two calls that can overlap on the GPU (for example on different streams) race; keep the calls on one device
 * ordered on one stream.  Results equal gl_matmul()'s. */
#define GL_NOALLOC_SCRATCH_BYTES (4u << 20)
GL_API int gl_matmul_noalloc(const gl_matmul_args* a, void* stream);

/* Name of the CUDA kernel gl_matmul() would launch for `a` (for logs and the config cache). */
GL_API const char* gl_matmul_kernel_name(const gl_matmul_args* a);

/* ---- bit packing: gemlite/bitpack.py -------------------------------------------------- */
/* in: uint8 [rows, cols] row-major (one value per byte). out: [rows, cols/e] words of
 * packing_bitwidth bits, e = packing_bitwidth / W_nbits.
 * Replaces pack_weights_over_cols_{torch,triton}, gemlite/bitpack.py:36-60, 78-144. */
GL_API int gl_pack_over_cols(const uint8_t* in, void* out, int64_t rows, int64_t cols,
                      int32_t W_nbits, int32_t packing_bitwidth, void* stream);
/* in: uint8 [rows, cols]; out: [rows/e, cols] words.
 * Replaces pack_weights_over_rows_{torch,triton}, gemlite/bitpack.py:10-34, 254-318. */
GL_API int gl_pack_over_rows(const uint8_t* in, void* out, int64_t rows, int64_t cols,
                      int32_t W_nbits, int32_t packing_bitwidth, void* stream);
/* in: [rows, cols_packed] words; out: [rows, cols_packed*e] values of out_dtype
 * (GL_UINT8 / GL_INT32 / GL_FP16 / GL_BF16 / GL_FP32 ...).  e = elements_per_sample fields are
 * taken from each word, lowest bits first; the reference derives e from the requested output
 * width, not from the word width (gemlite/bitpack.py:154-155), so e may be smaller than
 * packing_bitwidth / W_nbits.
 * Replaces unpack_over_cols_{torch,triton}, gemlite/bitpack.py:146-251. */
GL_API int gl_unpack_over_cols(const void* in, void* out, int64_t rows, int64_t cols_packed,
                        int32_t W_nbits, int32_t packing_bitwidth, int32_t elements_per_sample,
                        int32_t out_dtype, void* stream);
/* in: [rows_packed, cols] words; out: [rows_packed*e, cols] values.
 * Replaces unpack_over_rows_{torch,triton}, gemlite/bitpack.py:320-427. */
GL_API int gl_unpack_over_rows(const void* in, void* out, int64_t rows_packed, int64_t cols,
                        int32_t W_nbits, int32_t packing_bitwidth, int32_t elements_per_sample,
                        int32_t out_dtype, void* stream);

/* ---- dynamic activation quantisation: gemlite/quant_utils.py --------------------------- */
/* x [M,K] -> q [M,K] (GL_FP8 e4m3 or GL_INT8) + fp32 scales [M, K/128]: one scale per row and 128 consecutive k,
 * scale = max(amax / qmax, 1e-6), q = clamp(x / scale) cast (FP8) or rounded half away from zero (INT8); K % 128 == 0.
 * The activation side of 128 x 128 block quantisation (channel_scale_mode 5).  Replaces
 * scale_activations_per_block, gemlite/quant_utils.py:2504-2590. */
GL_API int gl_scale_activations_per_block(const void* x, void* q, float* scales, int32_t M, int32_t K,
                                          int32_t x_dtype, int32_t q_dtype, void* stream);

/* x [M,K] (x_dtype FP16/BF16/FP32) -> q [M,K] (q_dtype GL_FP8 e4m3 or GL_INT8) + fp32
 * scales [M]; s = max(amax/qmax, 1e-6), q = clamp(x/s) (rounded for int8).
 * Replaces scale_activations_per_token (v3 kernel), gemlite/quant_utils.py:459-539. */
GL_API int gl_scale_activations_per_token(const void* x, void* q, float* scales, int32_t M, int32_t K,
                                   int32_t x_dtype, int32_t q_dtype, void* stream);
/* x [M,K] -> q uint8 [M,K/2] (e2m1 pairs, even k low nibble) + e8m0 bytes
 * scales [ceil32(M), K/32] (pad rows = 127); scale_layout 1 writes them as 128x4 scale atoms over
 * ceil128(M) rows instead (see gl_matmul_args).
 * Replaces scale_activations_mxfp4 (v5 kernel), gemlite/quant_utils.py:1993-2135. */
GL_API int gl_scale_activations_mxfp4(const void* x, uint8_t* q, uint8_t* scales, int32_t M, int32_t K,
                               int32_t x_dtype, int32_t scale_layout, void* stream);
/* x [M,K] -> q uint8 [M,K/2] + e4m3 bytes scales [ceil16(M), K/16] (pad rows = 1.0) and the
 * fp32 tensor scale meta_scale[0] = 448*6/max(amax,1e-6).  When meta_in != NULL that
 * device scalar is used instead of the dynamic amax (static / calibrated scale) and copied to
 * meta_scale.  `amax_scratch` = 4 device bytes (any content).
 * Replaces scale_activations_nvfp4 (fused v6 / v5 kernels), gemlite/quant_utils.py:2152-2493. */
GL_API int gl_scale_activations_nvfp4(const void* x, uint8_t* q, uint8_t* scales, float* meta_scale,
                               const float* meta_in, uint32_t* amax_scratch,
                               int32_t M, int32_t K, int32_t x_dtype, int32_t scale_layout, void* stream);
/* x [M,K] -> q fp8 e4m3 [M,K] + e8m0 bytes scales [ceil32(M), K/32] (pad rows = 127).
 * Replaces scale_activations_mxfp8 (v4 kernel), gemlite/quant_utils.py:1024-1124. */
GL_API int gl_scale_activations_mxfp8(const void* x, uint8_t* q, uint8_t* scales, int32_t M, int32_t K,
                               int32_t x_dtype, int32_t scale_layout, void* stream);

/* ---- tile-config cache: gemlite/core.py:80-89, 838-906 ---------------------------------- */
/* The cache maps  family name -> signature string "(Mb, N, K, group_size, e, type_id)" -> a
 * JSON object of launch parameters, with the reference's file format and merge rules. */
GL_API int         gl_cfg_load(const char* filename, int32_t overwrite);  /* load_config  core.py:879-901 */
GL_API int         gl_cfg_save(const char* filename);                     /* cache_config core.py:838-877 */
GL_API void        gl_cfg_reset(void);                                    /* reset_config core.py:903-906 */
GL_API int         gl_cfg_set(const char* family, const char* signature, const char* json_object);
/* Returns the JSON object text (valid until the next gl_cfg_* call on this thread) or NULL. */
GL_API const char* gl_cfg_get(const char* family, const char* signature);
GL_API int64_t     gl_cfg_size(const char* family);                       /* entries; family NULL = all */
/* M bucket used in signatures.  Replaces get_closest_m(), triton_kernels/utils.py:182-220. */
GL_API int32_t     gl_get_closest_m(int32_t M);

/* ---- tensor parallelism: one-shot all-reduce over peer memory ---------------------------------- */
/* The reference has no multi-GPU code: under vLLM the host shards the layers and calls
 * tensor_model_parallel_all_reduce after every row-parallel one (gemlite/vllm/onthefly.py:83-99).  These entry
 * points are that host role for decode-size results ([M, N] of a few KB to a few MB), where an NCCL ring is bound by
 * launch and hop latency: one kernel pushes the local partial result to every rank's receive area with plain stores
 * to peer memory (NVLink / NVSwitch), publishes a per-chunk flag, waits (bounded) for the other ranks' flags and adds
 * the received chunks in rank order, so every rank ends with bit-identical sums.
 *
 * Unlike the rest of the library, gl_tp_buffer_create / _destroy allocate and free device memory (cudaMalloc), once,
 * at set-up: the receive areas must be exportable to the other processes.  Every rank creates one buffer of
 * gl_tp_buffer_bytes(world, slot_bytes), sends its 64-byte handle to the other ranks by any host channel, opens
 * theirs, and fills a gl_tp_comm.  One process per GPU; at most GL_TP_MAX_RANKS ranks. */
#define GL_TP_MAX_RANKS 8
#define GL_TP_MAX_CTAS 512
#define GL_TP_HANDLE_BYTES 64
typedef struct gl_tp_comm {
  int32_t  rank, world;
  uint64_t slot_bytes;                 /* largest all-reduce input in bytes (what the buffers were sized for) */
  uint64_t wait_cycles;                /* SM cycles a flag wait may take before it gives up; 0 = about two seconds */
  void*    buffers[GL_TP_MAX_RANKS];   /* buffers[r] = rank r's buffer as mapped in this process (own: the created pointer) */
} gl_tp_comm;
GL_API uint64_t gl_tp_buffer_bytes(int32_t world, uint64_t slot_bytes);
GL_API int gl_tp_buffer_create(uint64_t bytes, void** ptr, uint8_t* handle /* GL_TP_HANDLE_BYTES */);  /* zero-filled, on the current device */
GL_API int gl_tp_buffer_open(const uint8_t* handle, void** ptr);     /* map another rank's buffer (enables peer access) */
GL_API int gl_tp_buffer_close(void* ptr);
GL_API int gl_tp_buffer_destroy(void* ptr);
/* out[i] = sum over ranks of in[i], i < count; `in` 16-byte aligned, count * sizeof(dtype) a multiple of 16 and
 * <= slot_bytes; every rank must call it with the same count and dtype, in the same order.  A wait that runs out sets
 * the communicator's status word (gl_tp_status) and leaves `out` of the affected chunks unwritten; nothing hangs. */
GL_API int gl_tp_allreduce(const gl_tp_comm* c, const void* in, void* out, int64_t count, int32_t in_dtype,
                           int32_t out_dtype, void* stream);
/* Reads the status word (0 = no wait ever gave up) and the number of completed all-reduces.  Synchronous copy. */
GL_API int gl_tp_status(const gl_tp_comm* c, int32_t* status, uint32_t* epoch);
/* act[m, j] = silu(gate_up[m, j]) * gate_up[m, inter + j]: the element-wise step between a fused gate/up projection
 * and the down projection of a decoder MLP (two torch ops in a host that runs the reference). fp16 / bf16. */
GL_API int gl_silu_mul(const void* gate_up, void* out, int32_t M, int32_t inter, int32_t dtype, void* stream);

/* ---- measurement: tensor-pipe ceiling ------------------------------------------------------------ */
/* Enqueues one kernel in which every SM issues iters x 4 tcgen05.mma of 128 x 256 x (32 bytes of K) on operand tiles
 * resident in shared memory: the MMA-issue ceiling for `kind` (GL_BF16, GL_FP8, GL_INT8, GL_MXFP4, GL_NVFP4) on this
 * GPU at its current clocks.  *flops_out receives the operations of the launch; the caller times it with events.
 * `status_word`: 4 zeroed device bytes (set if the kernel's final wait runs out).  No counterpart in the reference
 * (its benchmarks quote spec-sheet peaks); bench.py uses it as the FP8 / FP4 roofline denominator. */
GL_API int gl_mma_peak(int32_t kind, int32_t iters, void* status_word, double* flops_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GEMLITE_B200_H_ */
