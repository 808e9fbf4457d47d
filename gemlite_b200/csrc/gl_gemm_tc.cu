// Tensor-core GEMM for prefill sizes (M >= 64) on tcgen05 / TMEM, sm_100a.
//
// Replaces the reference's gemm / gemm_splitK Triton kernels for large batches
// (gemlite/triton_kernels/gemm_kernels.py:285-496 integer / fp8 weights, :509-737 MX / NV block-scaled).
//
// One CTA computes a 128 x BN output tile; the accumulator lives in TMEM (128 lanes x BN fp32 columns).
// Shared memory holds a ring of K stages; every operand row of a stage is 128 bytes of K (64 bf16 / 128 fp8 /
// 256 fp4 values) in the 128-byte-swizzled K-major layout tcgen05.mma reads through shared-memory descriptors.
// Warp roles (warp-specialised, mbarrier pipelines, every wait bounded):
//   warp 0        TMA producer: activations (always) and weights (fp8 / int8 / fp4: already K-major in memory);
//                 block-scaled formats also bulk-copy their scale-factor atoms
//   warp 1        allocates TMEM, issues tcgen05.mma (one elected lane), commits stages back to the producer
//   warps 2-5     epilogue: tcgen05.ld the accumulator, channel / tensor scales, bias, cast, store
//   warps 6-13    (A16Wn only) dequantisers: packed int32 words staged by TMA -> unpack -> (q - z) * s in
//                 bf16/fp16 exactly as the reference's dequantize() -> swizzled B tile in shared memory
// Formats:
//   A16Wn   kind::f16, B produced in shared memory by the dequant warps (the reference's packed [K/8, N] layout
//           is N-major, tcgen05 wants K-major: one packed word = one 16-byte swizzle chunk of a B row)
//   A8W8    kind::f8f6f4 (e4m3 x e4m3) or kind::i8, fp32 / int32 accumulate, epilogue acc * s_x[m] * s_w[n]
//   MXFP4   kind::mxf4.block_scale (e8m0 per 32), NVFP4 kind::mxf4nvf4.block_scale (ue4m3 per 16): scale
//           factors are copied shared -> TMEM with tcgen05.cp from 128-row x 4-scale atoms (512 bytes)
#include "gl_tc_common.cuh"
#include <string.h>
#include <type_traits>
#include <stdlib.h>

using namespace gltc;

namespace {

constexpr int kNumEpiWarps = 4;

struct TcParams {
  int M, N, K, nkt;
  uint32_t idesc;
  void* out; int out_dtype;
  const void* bias;
  const float* scales_x;                        // [M] per-token activation scales or null
  const void* scales_w; int scales_w_dtype;     // [N] channel scales or null
  const float* meta_scale;                      // tensor scale (NVFP4) or null
  int* status;
  int swap;                                     // operands swapped: kernel rows = output channels, columns = tokens
  // split-K (A16Wn, few tiles): fp32 partial tiles [splits][M][N] and one arrival counter per tile in the workspace
  int splits;
  // block-scaled formats: scale-factor atoms [rows/128][kblocks][512 B]
  const uint8_t* sfa; const uint8_t* sfb; int sf_kblocks;
  // A16Wn
  const void* gscales; const void* gzeros; int group_size; int W_group_mode; int zero_is_scalar;
  // 128 x 128 block quantisation: fp32 weight scales [K/128][N/128] with these strides (activation scales: scales_x [M][K/128])
  const float* bq_scales; long long bq_stride_g, bq_stride_n;
  int band;   // row tiles per band of the tile order (0: one band)
  // A16Wn, a launch over part of the tiles: grid_tiles CTAs along x (0: all tiles); tail = 1: CTA t is column half t & 1
  // of the twice as wide tile tile_base + t / 2 (the tiles that a last, partly filled wave would have run)
  int grid_tiles, tile_base, tail;
};

template <int KIND> struct KindTraits;
template <> struct KindTraits<KIND_F16>    { static constexpr int ELEMS_PER_ROW = 64;  static constexpr int SF_ATOMS = 0; };
template <> struct KindTraits<KIND_F8F6F4> { static constexpr int ELEMS_PER_ROW = 128; static constexpr int SF_ATOMS = 0; };
template <> struct KindTraits<KIND_I8>     { static constexpr int ELEMS_PER_ROW = 128; static constexpr int SF_ATOMS = 0; };
template <> struct KindTraits<KIND_MXF4>   { static constexpr int ELEMS_PER_ROW = 256; static constexpr int SF_ATOMS = 2; };
template <> struct KindTraits<KIND_NVF4>   { static constexpr int ELEMS_PER_ROW = 256; static constexpr int SF_ATOMS = 4; };
template <> struct KindTraits<KIND_MXF8>   { static constexpr int ELEMS_PER_ROW = 128; static constexpr int SF_ATOMS = 1; };   // 128 e4m3 per row and stage = 4 groups of 32 = one atom

constexpr uint32_t next_pow2_cols(uint32_t c) { return c <= 32 ? 32 : c <= 64 ? 64 : c <= 128 ? 128 : c <= 256 ? 256 : 512; }

// ---- tile order ---------------------------------------------------------------------------------------
// Tiles are numbered in bands of GM row tiles: inside a band the row tile changes fastest, then the column tile, then the
// next band.  The CTAs that run together (consecutive numbers) then share GM row tiles of the activations and a handful
// of weight column tiles, which fit the L2 together; with one band over all rows, a problem whose activations exceed the
// L2 (16384 x 16384 fp4: 134 MB) re-reads all of them from HBM for every column of tiles (2.61 -> 2.39 ms there).  The
// host turns it on (gm > 0) only for activations of 64 MB and more: below, one band was 1-3 % faster.
__device__ __forceinline__ void tile_origin(int GM, int tile, int tiles_m, int tiles_n, int& mt, int& nt) {
  if (GM <= 0 || tiles_m <= GM) { mt = tile % tiles_m; nt = tile / tiles_m; return; }
  const int band = tile / (GM * tiles_n);
  const int rows = min(GM, tiles_m - band * GM);        // the last band may be short
  const int r = tile - band * GM * tiles_n;
  mt = band * GM + r % rows;
  nt = r / rows;
}

// ---- epilogue shared by all formats ---------------------------------------------------------------
// per-column epilogue constants of the tile, staged once in shared memory (fp32): channel scale and bias
__device__ __forceinline__ void stage_epilogue_consts(const TcParams& p, float* sw_s, float* b_s, int n0, int BN) {
  for (int c = threadIdx.x; c < BN; c += blockDim.x) {
    const int n = n0 + c;
    sw_s[c] = (p.scales_w != nullptr && n < p.N) ? gl_load_as_float(p.scales_w, n, p.scales_w_dtype) : 1.f;
    b_s[c] = (p.bias != nullptr && n < p.N) ? gl_load_as_float(p.bias, n, p.out_dtype) : 0.f;
  }
}

// one row's 32-column chunk: out = v * rowscale * s_w + bias, cast and stored (vector stores when the chunk is whole)
__device__ __forceinline__ void finish_row_chunk(const TcParams& p, int m, int nb, float (&v)[32], float rowscale, const float* sw, const float* bs) {
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const float4 s4v = *reinterpret_cast<const float4*>(sw + 4 * q);
    const float4 b4v = *reinterpret_cast<const float4*>(bs + 4 * q);
    const float s4[4] = {s4v.x, s4v.y, s4v.z, s4v.w}, b4[4] = {b4v.x, b4v.y, b4v.z, b4v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) v[4 * q + j] = fmaf(v[4 * q + j] * rowscale, s4[j], b4[j]);
  }
  const size_t o = (size_t)m * p.N + nb;
  const bool full = (nb + 32 <= p.N);
  if (p.out_dtype == GL_BF16 || p.out_dtype == GL_FP16) {
    if (full && (p.N % 8 == 0)) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + o);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (p.out_dtype == GL_BF16) { __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * q + 2 * j], v[8 * q + 2 * j + 1]); w[j] = *reinterpret_cast<uint32_t*>(&h); }
          else { __half2 h = __floats2half2_rn(v[8 * q + 2 * j], v[8 * q + 2 * j + 1]); w[j] = *reinterpret_cast<uint32_t*>(&h); }
        }
        dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
      for (int i = 0; i < 32 && nb + i < p.N; ++i) gl_store_out(p.out, o + i, v[i], p.out_dtype);
    }
  } else {
    if (full && (p.N % 4 == 0)) {
      float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o);
#pragma unroll
      for (int q = 0; q < 8; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
      for (int i = 0; i < 32 && nb + i < p.N; ++i) reinterpret_cast<float*>(p.out)[o + i] = v[i];
    }
  }
}

template <bool INT_ACC>
__device__ __forceinline__ void epilogue_tile(const TcParams& p, uint32_t tmem_d, int m0, int n0, int BN, int epi_warp, int lane,
                                              const float* sw_s, const float* b_s) {
  const int quad = epi_warp & 3;                       // TMEM lane quadrant this warp may read
  const int m = m0 + quad * 32 + lane;
  float rowscale = (p.scales_x != nullptr && m < p.M) ? p.scales_x[m] : 1.f;
  if (p.meta_scale != nullptr) rowscale *= *p.meta_scale;
  for (int c0 = 0; c0 < BN; c0 += 32) {
    if (n0 + c0 >= p.N) break;                         // warp-uniform
    uint32_t rr[32];
    tmem_ld_32x32(tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, rr);
    if (m >= p.M) continue;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = INT_ACC ? (float)(int32_t)rr[i] : __uint_as_float(rr[i]);
    finish_row_chunk(p, m, n0 + c0, v, rowscale, sw_s + c0, b_s + c0);
  }
}

// Operands swapped (decode sizes): the kernel's rows are output channels and its columns are tokens.  p.M / p.N are
// the kernel's dimensions (channels / tokens); scales_w and bias go with the row, scales_x with the column.
template <bool INT_ACC>
__device__ __forceinline__ void epilogue_tile_swapped(const TcParams& p, uint32_t tmem_d, int m0, int n0, int BN, int epi_warp, int lane) {
  const int quad = epi_warp & 3;
  const int ch = m0 + quad * 32 + lane;                // output channel
  float rs = 1.f, bias = 0.f;
  if (ch < p.M) {
    if (p.scales_w != nullptr) rs = gl_load_as_float(p.scales_w, ch, p.scales_w_dtype);
    if (p.bias != nullptr) bias = gl_load_as_float(p.bias, ch, p.out_dtype);
  }
  if (p.meta_scale != nullptr) rs *= *p.meta_scale;
  for (int c0 = 0; c0 < BN; c0 += 32) {
    if (n0 + c0 >= p.N) break;                         // warp-uniform
    uint32_t rr[32];
    tmem_ld_32x32(tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, rr);
    if (ch >= p.M) continue;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int tok = n0 + c0 + i;
      if (c0 + i < BN && tok < p.N) {
        const float a = INT_ACC ? (float)(int32_t)rr[i] : __uint_as_float(rr[i]);
        const float cs = p.scales_x != nullptr ? p.scales_x[tok] : 1.f;
        gl_store_out(p.out, (int64_t)tok * p.M + ch, fmaf(a * cs, rs, bias), p.out_dtype);
      }
    }
  }
}

// Operands swapped (at most 64 rows of x): the accumulator's lanes are output channels and its columns are tokens.
// One block of 32 channels x 32 tokens: out[token][channel] = v * s_w[channel] + bias[channel]; the 32 lanes of a
// warp write 32 consecutive channels of one token.
__device__ __forceinline__ void finish_swapped_block(const TcParams& p, int ch, int ch_local, int tok0, const float (&v)[32], const float* sw_s,
                                                     const float* b_s) {
  if (ch >= p.N) return;
  const float sc = sw_s[ch_local], bi = b_s[ch_local];
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (tok0 + i < p.M) gl_store_out(p.out, (size_t)(tok0 + i) * p.N + ch, fmaf(v[i], sc, bi), p.out_dtype);
}

// split-K of the A16Wn kernel: the CTAs that share an output tile (one per K range) form a thread-block cluster.  Each
// leaves its fp32 partial tile in its own shared memory (the operand ring is free by then) as 4 KB blocks of
// 32 rows x 32 columns, [float4 index][row] so that a warp moves 512 contiguous bytes per instruction ...
__device__ __forceinline__ void epilogue_dump_partial(uint32_t tmem_d, unsigned char* dump, int block0, int BN, int epi_warp, int lane) {
  const int quad = epi_warp & 3;                       // TMEM lane quadrant this warp may read
  for (int c = 0; c < (BN + 31) / 32; ++c) {
    uint32_t rr[32];
    tmem_ld_32x32(tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), rr);
    float4* dst = reinterpret_cast<float4*>(dump + (size_t)(block0 + c * 4 + quad) * 4096) + lane;
#pragma unroll
    for (int q = 0; q < 8; ++q)
      dst[q * 32] = make_float4(__uint_as_float(rr[4 * q]), __uint_as_float(rr[4 * q + 1]), __uint_as_float(rr[4 * q + 2]), __uint_as_float(rr[4 * q + 3]));
  }
}
// ... and after a cluster barrier CTA r sums, in split order, every block b with b % splits == r out of all the CTAs'
// shared memories and finishes those rows.  Every warp of the CTA takes part.
// (swapped operands: BN is the number of token columns, a block's lanes are channels n0 + quad * 32 + lane)
__device__ __forceinline__ void cluster_reduce_partials(const TcParams& p, const unsigned char* dump, int m0, int n0, int BN, int AM, int warp,
                                                        int n_warps, int lane, const float* sw_s, const float* b_s, bool swapped) {
  const int CB = (BN + 31) / 32, blocks = AM * CB * 4, S = p.splits, r = blockIdx.y;
  for (int b = r + S * warp; b < blocks; b += S * n_warps) {
    const int am = b / (CB * 4), c = (b >> 2) % CB, quad = b & 3;
    const int mrow = swapped ? c * 32 : m0 + am * 128 + quad * 32, nb = swapped ? n0 + quad * 32 : n0 + c * 32;
    if (mrow >= p.M || nb >= p.N) continue;            // warp-uniform
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = 0.f;
    const uint32_t local = smem_u32(dump + (size_t)b * 4096) + (uint32_t)lane * 16u;
    for (int sidx = 0; sidx < S; ++sidx) {
      uint32_t ra;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local), "r"(sidx));
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 t;
        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w) : "r"(ra + (uint32_t)q * 512u) : "memory");
        v[4 * q] += t.x; v[4 * q + 1] += t.y; v[4 * q + 2] += t.z; v[4 * q + 3] += t.w;
      }
    }
    if (swapped) finish_swapped_block(p, nb + lane, quad * 32 + lane, mrow, v, sw_s, b_s);
    else if (mrow + lane < p.M) finish_row_chunk(p, mrow + lane, nb, v, 1.f, sw_s + c * 32, b_s + c * 32);
  }
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- both operands by TMA: fp8 / int8 / mxfp4 / nvfp4 ---------------------------------------------
// Decode sizes run with the operands swapped (p.swap): the weight rows are the MMA's 128-row side and the batch is its
// 16- or 32-column side, so an MMA costs a fraction of the 128 x 128 one and the kernel streams at memory speed.
// Persistent: the grid is one CTA per SM and CTA c computes tiles c, c + gridDim.x, ...  The shared-memory ring
// runs straight across tile boundaries, so the loads of the next tile are in flight while the current one
// finishes.  Without scale factors there is room in TMEM for two 256-column accumulators: the epilogue warps drain
// one while the MMAs fill the other.  (Block-scaled formats keep one accumulator: 256 columns + scale factors.)
template <int KIND, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1) gl_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA,
                                                            const __grid_constant__ CUtensorMap tmB,
                                                            const __grid_constant__ CUtensorMap tmSFA,
                                                            const __grid_constant__ CUtensorMap tmSFB, const TcParams p) {
  using KT = KindTraits<KIND>;
  constexpr bool MX = KT::SF_ATOMS > 0;
  // 256-column block-scaled tiles copy their scale factors to TMEM two atoms at a time (tcgen05.cp.128x256b: every
  // copy costs ~70 cycles in the MMA pipe whatever its size).  That shape wants the four lane quadrants spelled out
  // in shared memory, so the atoms arrive through 4-D tensor maps whose replica dimension has stride 0.
  // (measured at M = 4096, 16384²: NVFP4, 12 copies per K tile, 0.79 -> 0.75 ms; MXFP4, 6 copies, is better off with a
  // fourth pipeline stage than with the 9 KB of replicated atoms per stage: 0.59 ms against 0.62 ms)
  // MXFP4 copies only the A-side atoms this way: 5 copies per K tile instead of 6 with a fourth stage still fitting.
  constexpr bool WIDE_A = MX && BN == 256 && KT::SF_ATOMS >= 2;
  constexpr bool WIDE_B = KIND == KIND_NVF4 && BN == 256;
  constexpr int REP_A = WIDE_A ? 4 : 1, REP_B = WIDE_B ? 4 : 1;
  constexpr int A_BYTES = 128 * 128, B_BYTES = BN * 128;
  constexpr int NBLK = (BN + 127) / 128;               // 128-row scale-factor blocks of the B tile
  constexpr int ACC_STRIDE = BN < 32 ? 32 : BN;        // TMEM columns per accumulator (tcgen05.ld reads 32 at a time)
  constexpr int SFA_BYTES = KT::SF_ATOMS * 512 * REP_A, SFB_BYTES = KT::SF_ATOMS * 512 * REP_B * NBLK;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  constexpr int ACC_BUFS = MX ? 1 : 2;
  constexpr uint32_t SFA_COL = ACC_BUFS * ACC_STRIDE, SFB_COL = SFA_COL + KT::SF_ATOMS * 4;
  constexpr uint32_t TMEM_COLS = next_pow2_cols(ACC_BUFS * ACC_STRIDE + KT::SF_ATOMS * 4 * (1 + NBLK));

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;                 // [ACC_BUFS] accumulator complete
  uint64_t* tmem_empty = tmem_full + 2;                 // [ACC_BUFS] accumulator drained by the four epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  float* consts = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(tmem_slot + 1) + 15) & ~(uintptr_t)15);   // [4 warps][2][BN]
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + 127) / 128, tiles_n = (p.N + BN - 1) / BN;
  const int tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < ACC_BUFS; ++b) { mbar_init(tmem_full + b, 1); mbar_init(tmem_empty + b, kNumEpiWarps); }
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (MX && !(WIDE_A && WIDE_B)) {   // scale-factor atoms that a short last K tile does not overwrite must hold finite numbers
    for (int s = 0; s < STAGES; ++s)
      for (int i = threadIdx.x; i < (SFA_BYTES + SFB_BYTES) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(smem + s * STAGE_BYTES + A_BYTES + B_BYTES)[i] = 0u;
    fence_proxy_async_smem();
  }
  if (MX && (p.sfa == nullptr || p.sfb == nullptr)) {
    // an operand without block scales (activations quantised per token, their scale applied by the epilogue): its atoms
    // are never loaded and hold e8m0 1.0 in every stage
    __syncthreads();                                     // (after the zero fill above, which other threads did)
    for (int s = 0; s < STAGES; ++s) {
      uint32_t* sf = reinterpret_cast<uint32_t*>(smem + s * STAGE_BYTES + A_BYTES + B_BYTES);
      if (p.sfa == nullptr) for (int i = threadIdx.x; i < SFA_BYTES / 4; i += blockDim.x) sf[i] = 0x7f7f7f7fu;
      if (p.sfb == nullptr) for (int i = threadIdx.x; i < SFB_BYTES / 4; i += blockDim.x) sf[SFA_BYTES / 4 + i] = 0x7f7f7f7fu;
    }
    fence_proxy_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  gl_launch_dependents();
  if (warp >= 2) gl_grid_dependency_wait();            // the epilogue reads activation scales of, and overwrites buffers known to, the previous kernel

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;                                   // K tiles issued so far, over all tiles of this CTA
      bool ok = true;
      auto stage_bytes = [&](int kt, int valid_nb) {
        uint32_t bytes = A_BYTES + B_BYTES;
        if (MX) {
          const int atoms = min(KT::SF_ATOMS, p.sf_kblocks - kt * KT::SF_ATOMS);
          if (p.sfa != nullptr) bytes += WIDE_A ? (uint32_t)SFA_BYTES : (uint32_t)atoms * 512u;            // wide boxes are always whole
          if (p.sfb != nullptr) bytes += WIDE_B ? (uint32_t)SFB_BYTES : (uint32_t)atoms * 512u * valid_nb;
        }
        return bytes;
      };
      auto load_a = [&](int kt, int s, int m0) {           // operand A of the kernel and its scale atoms
        unsigned char* st = smem + s * STAGE_BYTES;
        tma_load_2d(st, &tmA, full + s, kt * 128, m0);
        if (MX && p.sfa != nullptr) {
          const int atoms = min(KT::SF_ATOMS, p.sf_kblocks - kt * KT::SF_ATOMS);
          const size_t koff = (size_t)kt * KT::SF_ATOMS;
          if (WIDE_A) tma_load_4d(st + A_BYTES + B_BYTES, &tmSFA, full + s, 0, 0, kt * KT::SF_ATOMS, m0 / 128);
          else bulk_load_1d(st + A_BYTES + B_BYTES, p.sfa + ((size_t)(m0 / 128) * p.sf_kblocks + koff) * 512, (uint32_t)atoms * 512u, full + s);
        }
      };
      auto load_b = [&](int kt, int s, int n0, int valid_nb) {
        unsigned char* st = smem + s * STAGE_BYTES;
        tma_load_2d(st + A_BYTES, &tmB, full + s, kt * 128, n0);
        if (MX && p.sfb != nullptr) {
          const int atoms = min(KT::SF_ATOMS, p.sf_kblocks - kt * KT::SF_ATOMS);
          const size_t koff = (size_t)kt * KT::SF_ATOMS;
          if (WIDE_B) {
#pragma unroll
            for (int nb = 0; nb < NBLK; ++nb)
              tma_load_4d(st + A_BYTES + B_BYTES + SFA_BYTES + nb * (SFB_BYTES / NBLK), &tmSFB, full + s, 0, 0, kt * KT::SF_ATOMS, n0 / 128 + nb);
          } else {
            for (int nb = 0; nb < valid_nb; ++nb)
              bulk_load_1d(st + A_BYTES + B_BYTES + SFA_BYTES + nb * KT::SF_ATOMS * 512,
                           p.sfb + ((size_t)(n0 / 128 + nb) * p.sf_kblocks + koff) * 512, (uint32_t)atoms * 512u, full + s);
          }
        }
      };
      // Decode sizes (operands swapped): operand A is the weights, which do not depend on the previous kernel of the
      // stream, so the first stages' weight tiles are requested before the dependency wait and overlap that kernel's tail.
      int pre = 0;
      if (p.swap && (int)blockIdx.x < tiles) {
        int mt, nt;
        tile_origin(p.band, (int)blockIdx.x, tiles_m, tiles_n, mt, nt);
        const int m0 = mt * 128, n0 = nt * BN;
        const int valid_nb = min(NBLK, (p.N - n0 + 127) / 128);
        pre = min(STAGES, p.nkt);
        for (int kt = 0; kt < pre; ++kt) {
          mbar_expect_tx(full + kt, stage_bytes(kt, valid_nb));
          load_a(kt, kt, m0);
        }
      }
      gl_grid_dependency_wait();
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int mt, nt;
        tile_origin(p.band, tile, tiles_m, tiles_n, mt, nt);
        const int m0 = mt * 128, n0 = nt * BN;
        const int valid_nb = min(NBLK, (p.N - n0 + 127) / 128);   // 128-column blocks of this tile that exist
        for (int kt = 0; kt < p.nkt; ++kt, ++it) {
          const int s = it % STAGES;
          if ((int)it < pre) { load_b(kt, s, n0, valid_nb); continue; }      // the other half of a stage opened above
          if (!mbar_wait_spin(empty + s, ((it / STAGES) & 1u) ^ 1u, &s_abort, p.status, 2)) { ok = false; break; }
          mbar_expect_tx(full + s, stage_bytes(kt, valid_nb));
          load_a(kt, s, m0);
          load_b(kt, s, n0, valid_nb);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, local = 0;                        // K tiles consumed; tiles of this CTA started
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
        const uint32_t ab = local % ACC_BUFS;
        // the epilogue must have drained this accumulator (first use of each passes at once)
        if (!mbar_wait(tmem_empty + ab, ((local / ACC_BUFS) & 1u) ^ 1u, &s_abort, p.status, 6)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * ACC_STRIDE;
        for (int kt = 0; kt < p.nkt; ++kt, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait_spin(full + s, (it / STAGES) & 1u, &s_abort, p.status, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + A_BYTES;
          if (MX) {
            const uint32_t sfa_s = sb + B_BYTES, sfb_s = sfa_s + SFA_BYTES;
            if (WIDE_A) {
#pragma unroll
              for (int a = 0; a < KT::SF_ATOMS; a += 2)      // atoms a, a + 1 of the A rows: adjacent in shared memory and TMEM
                tmem_cp_sf_pair2(tmem_base + SFA_COL + a * 4, smem_desc_sf2(sfa_s + a * 2048, 2048));
            } else {
#pragma unroll
              for (int a = 0; a < KT::SF_ATOMS; ++a) tmem_cp_sf(tmem_base + SFA_COL + a * 4, smem_desc_sf(sfa_s + a * 512));
            }
            if (WIDE_B) {
#pragma unroll
              for (int a = 0; a < KT::SF_ATOMS; ++a)         // atom a of both 128-column blocks of B
                tmem_cp_sf_pair2(tmem_base + SFB_COL + a * 8, smem_desc_sf2(sfb_s + a * 2048, SFB_BYTES / NBLK));
            } else {
#pragma unroll
              for (int a = 0; a < KT::SF_ATOMS; ++a)
#pragma unroll
                for (int nb = 0; nb < NBLK; ++nb)
                  tmem_cp_sf(tmem_base + SFB_COL + a * 4 * NBLK + nb * 4, smem_desc_sf(sfb_s + (nb * KT::SF_ATOMS + a) * 512));
            }
          }
          const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sb);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t accum = (kt > 0 || j > 0) ? 1u : 0u;
            if constexpr (KIND == KIND_MXF4) {
              const uint32_t sfid = (uint32_t)(2 * (j & 1));
              mma_ss_block_scaled<KIND>(d_tmem, da + 2 * j, db + 2 * j, p.idesc | (sfid << 29) | (sfid << 4),
                                        tmem_base + SFA_COL + (j >> 1) * 4, tmem_base + SFB_COL + (j >> 1) * 4 * NBLK, accum);
            } else if constexpr (KIND == KIND_NVF4) {
              mma_ss_block_scaled<KIND>(d_tmem, da + 2 * j, db + 2 * j, p.idesc,
                                        tmem_base + SFA_COL + j * 4, tmem_base + SFB_COL + j * 4 * NBLK, accum);
            } else if constexpr (KIND == KIND_MXF8) {      // MMA j covers k 32 j .. 32 j + 31: byte j of the atom's scale words
              mma_ss_block_scaled<KIND>(d_tmem, da + 2 * j, db + 2 * j, p.idesc | ((uint32_t)j << 29) | ((uint32_t)j << 4),
                                        tmem_base + SFA_COL, tmem_base + SFB_COL, accum);
            } else {
              mma_ss<KIND>(d_tmem, da + 2 * j, db + 2 * j, p.idesc, accum);
            }
          }
          tc_commit(empty + s);
        }
        if (ok) tc_commit(tmem_full + ab);
      }
    }
  } else {
    float* sw_s = consts + (warp - 2) * 2 * BN;          // this warp's copy of the tile's per-column constants
    float* b_s = sw_s + BN;
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      int mt, nt;
      tile_origin(p.band, tile, tiles_m, tiles_n, mt, nt);
      const int m0 = mt * 128, n0 = nt * BN;
      const uint32_t ab = local % ACC_BUFS;
      if (!p.swap) {
        for (int c = lane; c < BN; c += 32) {
          const int n = n0 + c;
          sw_s[c] = (p.scales_w != nullptr && n < p.N) ? gl_load_as_float(p.scales_w, n, p.scales_w_dtype) : 1.f;
          b_s[c] = (p.bias != nullptr && n < p.N) ? gl_load_as_float(p.bias, n, p.out_dtype) : 0.f;
        }
        __syncwarp();
      }
      if (!mbar_wait(tmem_full + ab, (local / ACC_BUFS) & 1u, &s_abort, p.status, 4)) break;
      tc_fence_after();
      if (p.swap) epilogue_tile_swapped<KIND == KIND_I8>(p, tmem_base + ab * ACC_STRIDE, m0, n0, BN, warp, lane);
      else epilogue_tile<KIND == KIND_I8>(p, tmem_base + ab * ACC_STRIDE, m0, n0, BN, warp, lane, sw_s, b_s);
      tc_fence_before();                                  // this warp's TMEM reads are complete (tcgen05.wait::ld inside)
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + ab);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- A16Wn: weights dequantised into the B tile by eight warps -------------------------------------
template <typename XT> struct H2;
template <> struct H2<__nv_bfloat16> {
  using T = __nv_bfloat162;
  static constexpr uint32_t MAGIC = 0x43004300u;
  __device__ static T from_float(float v) { return __float2bfloat162_rn(v); }
};
template <> struct H2<__half> {
  using T = __half2;
  static constexpr uint32_t MAGIC = 0x64006400u;
  __device__ static T from_float(float v) { return __float2half2_rn(v); }
};

// AM: 128-row activation tiles per CTA (1 or 2).  The kernel is bound by the dequantisation of the weight tile (unpack,
// HFMA2, swizzled stores: the same work whatever the batch), so with AM = 2 one dequantised tile feeds two 128-row
// accumulators (2 x BN TMEM columns): half the dequantisation per flop and half the re-reads of the packed weights.
// K tiles per stage of the A16Wn kernel: the swapped form groups them (fewer barrier round trips, commits and waits per
// tile for the single MMA-issuing thread): 2 with two CTAs per SM, GL_SW_KT with one
#ifndef GL_SW_KT
#define GL_SW_KT 2
#endif
constexpr int a16_tiles_per_stage(int SW, int DQW) { return SW ? (DQW == 8 ? GL_SW_KT : 2) : 1; }

// bytes of a slot of the A16Wn kernel's packed-word ring: the packed words of a 64-deep K tile, a row of scales and a row of zeros
constexpr int a16_wslot_bytes(int NB, int BN) { return ((64 / (32 / NB) * BN * 4 + 2 * BN * 2 + 255) / 256) * 256; }

// Profiling build (-DGL_TC_TRACE): the A16Wn kernel writes 16 counters per CTA (globaltimer stamps of its phases and
// clock64 sums of what its MMA, producer and first dequant warp waited for) to a buffer set with gl_debug_tc_trace.
#ifdef GL_TC_TRACE
__device__ unsigned long long* g_tc_trace = nullptr;
extern "C" __attribute__((visibility("default"))) void gl_debug_tc_trace(void* buf) {
  unsigned long long* b = reinterpret_cast<unsigned long long*>(buf);
  cudaMemcpyToSymbol(g_tc_trace, &b, sizeof(b));
}
#define TC_GT(i) do { if (g_tc_trace) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
    g_tc_trace[(size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 + (i)] = t_; } } while (0)
#if GL_TC_TRACE == 2   // light mode: no clock reads inside the loops, failed barrier polls are counted instead
#define TC_CK(v) const long long v = 0
#define TC_ACC(acc, a, b) do { } while (0)
__device__ __forceinline__ bool mbar_wait_counted(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code, long long& polls) {
  while (!mbar_try_wait(bar, parity)) {
    if (((++polls) & 0xFFFFF) == 0) { *abort_flag = 1; if (status) atomicCAS(status, 0, code); return false; }
    if (*abort_flag) return false;
  }
  return true;
}
#define TC_WAIT(bar, par, code, acc) mbar_wait_counted(bar, par, &s_abort, p.status, code, acc)
#else
#define TC_CK(v) const long long v = clock64()
#define TC_ACC(acc, a, b) acc += (b) - (a)
#define TC_WAIT(bar, par, code, acc) mbar_wait_spin(bar, par, &s_abort, p.status, code)
#endif
#define TC_PUT(i, acc) do { if (g_tc_trace) g_tc_trace[(size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 + (i)] = (unsigned long long)(acc); } while (0)
#else
#define TC_GT(i) do { } while (0)
#define TC_CK(v) do { } while (0)
#define TC_ACC(acc, a, b) do { } while (0)
#define TC_PUT(i, acc) do { } while (0)
#define TC_WAIT(bar, par, code, acc) mbar_wait_spin(bar, par, &s_abort, p.status, code)
#endif
// waits of the dequant warps (32 lanes each)
#ifdef GL_SPIN_DQ
#define TC_WAIT_DQ(bar, par, code, acc) TC_WAIT(bar, par, code, acc)
#else
#define TC_WAIT_DQ(bar, par, code, acc) mbar_wait(bar, par, &s_abort, p.status, code)
#endif

// WS: slots of the packed-word ring.  The packed weights come from DRAM (every other operand of a stage is L2- or
// SM-local), and a K tile of them is only a few KB, so they get a ring of their own that runs WS tiles ahead of the
// STAGES-deep activation / dequantised-tile ring: with both in one ring the DRAM latency was paid once per STAGES tiles.
// A slot of that ring also carries the tile's row of group scales and of group zeros (BN values each): a dequant warp
// that fetched them from global memory had the load's latency in its chain at every change of group, because the
// mbarrier arrive that publishes its tile orders all of the thread's earlier memory operations.
// SW > 0: operands swapped for at most SW (32 / 64) rows of x.  The dequantised tile (128 channels x 64 k) is the MMA's
// 128-row operand and is written straight to tensor memory (lane = channel, 32 columns of two k each) instead of
// shared memory; x is the SW-column operand in shared memory; the accumulator holds [channel lane][token column].
// Shared memory carries 128 bytes per clock: with both operands there, a 128 x 128 x 64 step moves 32 KB for the MMAs,
// 16 KB of dequantised stores and 20 KB of TMA writes, which takes longer than its arithmetic.  This form moves the
// x tile (SW x 128 bytes) in and out and the packed words, nothing else.
// DQW: dequant warps.  4 (one per 32 channels of a 128-channel tile, 10 warps in all, at most 102 registers) lets two
// CTAs share an SM: at decode sizes a CTA's pipeline is a chain of barrier round trips that leaves every unit of
// the SM mostly idle, and a second, independent chain on the same SM fills the gaps.
template <typename XT, int NB, int BN, int STAGES, int AM = 1, int WS = STAGES, int SW = 0, int DQW = 8>
__global__ void __launch_bounds__((6 + DQW) * 32, DQW == 4 ? 2 : 1) gl_gemm_tc_a16wn_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                  const __grid_constant__ CUtensorMap tmW,
                                                                  const __grid_constant__ CUtensorMap tmS,
                                                                  const __grid_constant__ CUtensorMap tmZ, const TcParams p) {
  constexpr int E = 32 / NB;                           // k values per packed word
  constexpr int WROWS = 64 / E;                        // packed rows per 64-wide K tile (8 for 4-bit)
  static_assert(SW == 0 || (BN == 128 && AM == 1), "swapped operands: one 128-channel tile");
  constexpr int A_TILE = (SW ? SW : 128) * 128;        // rows of x per tile x 64 k x 2 bytes
  // K tiles per stage: the swapped form pairs them, which halves the barrier round trips, commits and waits per tile
  // (its stage is small: KT x tiles and KT x 32 tensor-memory columns)
  constexpr int KT = a16_tiles_per_stage(SW, DQW);
  constexpr int A_BYTES = KT * AM * A_TILE, B_BYTES = SW ? 0 : BN * 128, W_BYTES = WROWS * BN * 4;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t WT_COL0 = SW;                     // swapped: dequantised tiles of the STAGES slots follow the accumulator
  constexpr int META_BYTES = BN * 2;                   // one row of scales or zeros
  constexpr int WSLOT_BYTES = a16_wslot_bytes(NB, BN);
  constexpr uint32_t TMEM_COLS = next_pow2_cols(SW ? SW + STAGES * KT * 32 : AM * BN);
  constexpr int HALF = 16 / NB;                        // field a shares a 32-bit extraction with field a + HALF
  constexpr uint32_t FMASK = ((1u << NB) - 1u) * 0x00010001u;
  using h2 = typename H2<XT>::T;

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  unsigned char* wring = smem + STAGES * STAGE_BYTES;                           // [WS] packed-word tiles
  // ready: the stage's operands are complete (the x tile landed and every dequant warp of the tile arrived)
  uint64_t* ready = reinterpret_cast<uint64_t*>(wring + WS * WSLOT_BYTES);
  uint64_t* empty = ready + STAGES;                                             // MMAs of the stage retired
  uint64_t* wfull = empty + STAGES;                                             // [WS] packed W landed
  uint64_t* wempty = wfull + WS;                                                // [WS] packed W read by every dequant warp
  uint64_t* tmem_full = wempty + WS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
  float* sw_s = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(tmem_slot + 1) + 15) & ~(uintptr_t)15);
  float* b_s = sw_s + BN;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = SW ? 1 : (p.M + 128 * AM - 1) / (128 * AM);
  int mt, nt;
  if (p.tail) {
    tile_origin(p.band, p.tile_base + ((int)blockIdx.x >> 1), tiles_m, (p.N + 2 * BN - 1) / (2 * BN), mt, nt);
    nt = nt * 2 + ((int)blockIdx.x & 1);
  } else {
    tile_origin(p.band, (int)blockIdx.x, tiles_m, (p.N + BN - 1) / BN, mt, nt);
  }
  const int m0 = mt * (128 * AM), n0 = nt * BN;
  if (n0 >= p.N) return;                               // (the right half of a ragged last tile: nothing to compute)
  // K tiles of this CTA: blockIdx.y picks one of p.splits equal ranges (the last one may be shorter)
  const int kt_per = (p.nkt + p.splits - 1) / p.splits;
  const int kt0 = blockIdx.y * kt_per;
  const int nloc = min(kt_per, p.nkt - kt0);
  const int nstages = (nloc + KT - 1) / KT;            // stages of KT K tiles
  if (threadIdx.x == 0) TC_GT(0);
  stage_epilogue_consts(p, sw_s, b_s, n0, BN);

  if (threadIdx.x == 0) {
    s_abort = 0;
    // a K tile is dequantised by BN / 32 warps (one per 32 columns)
    for (int s = 0; s < STAGES; ++s) { mbar_init(ready + s, 1 + BN / 32); mbar_init(empty + s, 1); }
    for (int s = 0; s < WS; ++s) { mbar_init(wfull + s, 1); mbar_init(wempty + s, BN / 32); }
    mbar_init(tmem_full, 1);
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmS);
    prefetch_tmap(&tmZ);
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool need_s = p.W_group_mode >= 2, need_z = (p.W_group_mode == 1 || p.W_group_mode >= 3) && !p.zero_is_scalar;
  if (threadIdx.x == 0) TC_GT(1);
#ifdef GL_TC_TRACE
  long long acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0;
#endif

  gl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      gl_grid_dependency_wait();                           // x is the previous kernel's output; the packed words (warp 2) are not
      for (int j = 0; j < nstages; ++j) {
        const int s = j % STAGES, kt = kt0 + j * KT;
        const int nt = min(KT, nloc - j * KT);             // K tiles of this stage (the last one may be short)
        TC_CK(c0);
        if (!TC_WAIT(empty + s, (uint32_t)(((j / STAGES) & 1) ^ 1), 2, acc0)) break;
        TC_CK(c1); TC_ACC(acc0, c0, c1);
        unsigned char* st = smem + s * STAGE_BYTES;
        mbar_expect_tx(ready + s, (uint32_t)(nt * AM * A_TILE));
        for (int t = 0; t < nt; ++t)
#pragma unroll
          for (int am = 0; am < AM; ++am) tma_load_2d(st + (t * AM + am) * A_TILE, &tmA, ready + s, (kt + t) * 64, m0 + am * 128);   // rows past M read as zeros
      }
      TC_PUT(12, acc0);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // The issuing thread's instruction count per stage is what this loop is written for: the stage index is a
      // compile-time constant (the loop over stages is unrolled inside a loop over ring revolutions), descriptors are
      // the ring base's low word plus constants, and only the very first MMA has a run-time accumulate flag.
      bool ok = true;
      TC_CK(cl0);
      const uint64_t d0 = smem_desc_sw128(smem_u32(smem));
      const uint32_t d_lo = (uint32_t)d0, d_hi = (uint32_t)(d0 >> 32);
      const uint32_t idesc = p.idesc;
      for (int i0 = 0; i0 < nstages && ok; i0 += STAGES) {
        const uint32_t ph = (uint32_t)((i0 / STAGES) & 1);
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
          const int i = i0 + s;
          if (i >= nstages) break;
          TC_CK(c0);
          if (!TC_WAIT(ready + s, ph, 3, acc0)) { ok = false; break; }
          TC_CK(c1); TC_ACC(acc0, c0, c1);
          TC_CK(c2); TC_ACC(acc1, c1, c2);
          tc_fence_after();
          const uint32_t st_lo = d_lo + (uint32_t)(s * STAGE_BYTES / 16);      // (the start-address field counts 16-byte units)
          if constexpr (SW > 0) {
#pragma unroll
            for (int t = 0; t < KT; ++t) {
              if (t > 0 && i * KT + t >= nloc) break;         // short last stage
#pragma unroll
              for (int j = 0; j < 4; ++j)                     // 16 k = 8 tensor-memory columns of the dequantised tile, 32 bytes of the x rows
                mma_ts_f16_lohi(tmem_base, tmem_base + WT_COL0 + (uint32_t)((s * KT + t) * 32 + j * 8), st_lo + (uint32_t)(t * A_TILE / 16 + 2 * j),
                                d_hi, idesc, (t > 0 || j > 0) ? 1u : (uint32_t)(i > 0));
            }
          } else {
#pragma unroll
            for (int am = 0; am < AM; ++am)
#pragma unroll
              for (int j = 0; j < 4; ++j)
                mma_ss_f16_lohi(tmem_base + am * BN, st_lo + (uint32_t)(am * A_TILE / 16 + 2 * j), st_lo + (uint32_t)(A_BYTES / 16 + 2 * j), d_hi, idesc,
                                j > 0 ? 1u : (uint32_t)(i > 0));
          }
          TC_CK(c2b); TC_ACC(acc3, c2, c2b);
          tc_commit(empty + s);
          TC_CK(c3); TC_ACC(acc2, c2, c3);
        }
      }
      if (ok) tc_commit(tmem_full);
      TC_CK(cl1);
      TC_GT(2); TC_PUT(5, acc0); TC_PUT(6, acc1); TC_PUT(7, acc2); TC_PUT(15, cl1 - cl0); TC_PUT(4, acc3);
    }
  } else if (warp < 2 + kNumEpiWarps) {
    if (warp == 2) {
      // the first epilogue warp has nothing to do until the accumulator is complete: it feeds the packed-word ring.
      // Lanes 0 / 1 / 2 issue the copies of the packed words / the scale row / the zero row in one warp instruction.
      if (lane < 3) {
        const CUtensorMap* tm = lane == 0 ? &tmW : lane == 1 ? &tmS : &tmZ;
        const bool active = lane == 0 || (lane == 1 && need_s) || (lane == 2 && need_z);
        const uint32_t off = lane == 0 ? 0u : lane == 1 ? (uint32_t)W_BYTES : (uint32_t)(W_BYTES + META_BYTES);
        const uint32_t tx = W_BYTES + (need_s ? META_BYTES : 0) + (need_z ? META_BYTES : 0);
        const int tiles_per_group = p.group_size / 64;
        int g = (kt0 * 64) / p.group_size, g_left = tiles_per_group - kt0 % tiles_per_group;
        for (int i = 0; i < nloc; ++i) {
          const int ws = i % WS;
          if (!TC_WAIT(wempty + ws, (uint32_t)(((i / WS) & 1) ^ 1), 7, acc0)) break;
          if (lane == 0) mbar_expect_tx(wfull + ws, tx);
          if (active) tma_load_2d(wring + ws * WSLOT_BYTES + off, tm, wfull + ws, n0, lane == 0 ? (kt0 + i) * WROWS : g);   // columns past N read as zeros
          if (--g_left == 0) { ++g; g_left = tiles_per_group; }
        }
        if (lane == 0) TC_PUT(3, acc0);
      }
      __syncwarp();
    }
    gl_grid_dependency_wait();
    if (mbar_wait(tmem_full, 0u, &s_abort, p.status, 4)) {
      tc_fence_after();
      if (p.splits == 1) {
        if constexpr (SW > 0) {
          const int quad = warp & 3;
          for (int c0 = 0; c0 < SW && c0 < p.M; c0 += 32) {
            uint32_t rr[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, rr);
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rr[i]);
            finish_swapped_block(p, n0 + quad * 32 + lane, quad * 32 + lane, c0, v, sw_s, b_s);
          }
        } else {
#pragma unroll
          for (int am = 0; am < AM; ++am) epilogue_tile<false>(p, tmem_base + am * BN, m0 + am * 128, n0, BN, warp, lane, sw_s, b_s);
        }
      } else {
        // every operand of the ring has been consumed (the accumulator is complete): the ring holds the partial tile now
        if constexpr (SW > 0) epilogue_dump_partial(tmem_base, smem, 0, SW, warp, lane);
        else {
#pragma unroll
          for (int am = 0; am < AM; ++am) epilogue_dump_partial(tmem_base + am * BN, smem, am * (BN / 32) * 4, BN, warp, lane);
        }
      }
    }
  } else {
    // dequant warps: warp dw owns 32 columns of a K tile
    const int dw = warp - 2 - kNumEpiWarps;
    constexpr int CBLOCKS = BN / 32;                       // 32-column blocks in the tile
    // With more warps than column blocks (BN = 128) the warps form groups that take the K tiles in turn: the chain of a
    // tile (wait, read, unpack, store, fence, arrive) is mostly latency, and two tiles in flight hide it.
    constexpr int TSPLIT = DQW / CBLOCKS;                  // warp groups (1 or 2)
    static_assert(DQW % CBLOCKS == 0 && TSPLIT >= 1, "dequant warps: a multiple of the 32-column blocks");
    constexpr int RPW = WROWS;                             // packed rows per warp: the whole K tile of its 32 columns
    // (swapped: the warp writes the lane quadrant of tensor memory it may access, so its 32 channels are that quadrant's)
    const int nl = (SW ? (warp & 3) : (dw % CBLOCKS)) * 32 + lane;             // column (channel) inside the tile
    constexpr int c_begin = 0;
    constexpr uint32_t kMagic = H2<XT>::MAGIC;
    uint32_t magic_bits = kMagic;
    const h2 magic = *reinterpret_cast<const h2*>(&magic_bits);
    h2 s2 = H2<XT>::from_float(1.f), z2 = H2<XT>::from_float(0.f);
    if (p.zero_is_scalar && p.gzeros) z2 = H2<XT>::from_float((float)(*reinterpret_cast<const int32_t*>(p.gzeros)));
    // the group's n-th K tile: stages (of KT tiles) go to the groups in turn
    for (int n = 0;; ++n) {
      const int j = dw / CBLOCKS + (n / KT) * TSPLIT, t = n % KT, i = j * KT + t;
      if (i >= nloc) break;
      const int s = j % STAGES, ws = i % WS;
      const bool first_of_stage = (t == 0), last_of_stage = (t == KT - 1) || (i + 1 >= nloc);
      TC_CK(c0);
      if (!TC_WAIT_DQ(wfull + ws, (uint32_t)((i / WS) & 1), 6, acc0)) break;
      TC_CK(c1); TC_ACC(acc0, c0, c1);
      unsigned char* st = smem + s * STAGE_BYTES;
      const uint32_t* wst = reinterpret_cast<const uint32_t*>(wring + ws * WSLOT_BYTES);
      // this column's scale and zero of the tile's group arrived with the packed words
      if (need_s) { const XT sv = reinterpret_cast<const XT*>(wring + ws * WSLOT_BYTES + W_BYTES)[nl]; s2 = h2(sv, sv); }
      if (need_z) { const XT zv = reinterpret_cast<const XT*>(wring + ws * WSLOT_BYTES + W_BYTES + META_BYTES)[nl]; z2 = h2(zv, zv); }
      unsigned char* brow = st + A_BYTES + nl * 128;
      // all packed words into registers first (the stores below may alias the words for the compiler)
      uint32_t wv[RPW];
#pragma unroll
      for (int cc = 0; cc < RPW; ++cc) wv[cc] = wst[(c_begin + cc) * BN + nl];
      TC_CK(c2);
      // the dequantised tile of K tile i - STAGES must have been consumed before its slot is overwritten (swapped: the
      // tile is built in registers first and the wait comes before the store to tensor memory)
      if constexpr (SW == 0) if (!TC_WAIT_DQ(empty + s, (uint32_t)(((j / STAGES) & 1) ^ 1), 8, acc1)) break;
      TC_CK(c3); TC_ACC(acc1, c2, c3);
      uint32_t outr[SW ? 32 : 1];                          // swapped: this channel's 64 k, two per register
      // 16-byte chunk `chunk` (8 consecutive k) of this channel's row
      auto emit = [&](int chunk, uint32_t e0, uint32_t e1, uint32_t e2, uint32_t e3) {
        if constexpr (SW > 0) { outr[4 * chunk] = e0; outr[4 * chunk + 1] = e1; outr[4 * chunk + 2] = e2; outr[4 * chunk + 3] = e3; }
        else *reinterpret_cast<uint4*>(brow + ((chunk ^ (nl & 7)) << 4)) = make_uint4(e0, e1, e2, e3);
      };
      // the mode is decided once per K tile, outside the unrolled loops: a branch per pair would serialise them
      auto unpack_tile = [&](auto fma_tag) {
        constexpr bool FMA = decltype(fma_tag)::value;
        const h2 zs2 = (p.W_group_mode == 1 || p.W_group_mode == 3) ? z2 : H2<XT>::from_float(0.f);
        const h2 ss2 = (p.W_group_mode >= 2) ? s2 : H2<XT>::from_float(1.f);
        uint32_t keep_lo = 0u, keep_hi = 0u;
#pragma unroll
        for (int cc = 0; cc < RPW; ++cc) {
          const int c = c_begin + cc;                        // packed row inside the K tile
          const uint32_t w = wv[cc];
          // pair a = (field a, field a + HALF), dequantised exactly as dequantize() does in the scale dtype
          uint32_t P[HALF];
#pragma unroll
          for (int a = 0; a < HALF; ++a) {
            h2 q;                                                            // exact integer code
            if constexpr (NB == 8 && sizeof(XT) == 2 && H2<XT>::MAGIC == 0x43004300u) {
              // bf16 has 7 mantissa bits: the byte goes in as its low 7 bits (128 + q7) and its top bit (128 or 256)
              const uint32_t v = w >> (8 * a);
              uint32_t lo7 = (v & 0x007F007Fu) | kMagic, top = (v & 0x00800080u) | kMagic;
              q = __hadd2(__hsub2(*reinterpret_cast<h2*>(&lo7), magic), __hsub2(*reinterpret_cast<h2*>(&top), magic));
            } else {
              uint32_t bits = ((w >> (NB * a)) & FMASK) | kMagic;
              q = __hsub2(*reinterpret_cast<h2*>(&bits), magic);
            }
            // mode 4: q*s + z' in one rounding; the other modes as (q - z) * s with z = 0 / s = 1 where absent:
            // the same roundings as the reference's dequantize() (triton_kernels/utils.py:73-105)
            if (FMA) q = __hfma2(q, s2, z2);
            else q = __hmul2(__hsub2(q, zs2), ss2);
            P[a] = *reinterpret_cast<uint32_t*>(&q);
          }
          // natural k order: low halves are fields 0..HALF-1, high halves fields HALF..2*HALF-1
          uint32_t L[HALF / 2], Hh[HALF / 2];
#pragma unroll
          for (int j = 0; j < HALF / 2; ++j) {
            L[j] = __byte_perm(P[2 * j], P[2 * j + 1], 0x5410);
            Hh[j] = __byte_perm(P[2 * j], P[2 * j + 1], 0x7632);
          }
          const int chunk0 = c * (E / 8);
          if constexpr (NB == 8) {                         // a word holds 4 k: two consecutive packed rows make one 16-byte chunk
            if ((cc & 1) == 0) { keep_lo = L[0]; keep_hi = Hh[0]; }
            else emit(c >> 1, keep_lo, keep_hi, L[0], Hh[0]);
          } else if constexpr (NB == 4) {
            emit(chunk0, L[0], L[1], Hh[0], Hh[1]);
          } else {
            constexpr int CH = HALF / 8;                     // chunks per half (1 for 2-bit, 2 for 1-bit)
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
              emit(chunk0 + ch, L[4 * ch], L[4 * ch + 1], L[4 * ch + 2], L[4 * ch + 3]);
              emit(chunk0 + CH + ch, Hh[4 * ch], Hh[4 * ch + 1], Hh[4 * ch + 2], Hh[4 * ch + 3]);
            }
          }
        }
      };
      if (p.W_group_mode == 4) unpack_tile(std::true_type{}); else unpack_tile(std::false_type{});
      // The ring slot goes back to its producer only now, after the tile has been unpacked.  Handing it back right after
      // the loads above (words, scale and zero already in registers) gave wrong values in 16-byte granules of a tile's
      // scale row (8 columns, all rows of the tile) in a few calls out of a hundred whenever the MMAs, not the dequant
      // warps, set the pace (two accumulators per CTA); neither volatile loads, nor an instruction consuming words, scale
      // and zero before the arrive, nor a warp barrier before the proxy fence, nor expect_tx ordered before the scale /
      // zero copies changed that, so the cause is not known.  Released here the same calls were bit-identical in some
      // 3000 calls out of 3000, at the same speed.
      __syncwarp();
      if (lane == 0) mbar_arrive(wempty + ws);
      TC_CK(c4); TC_ACC(acc2, c3, c4);
      if constexpr (SW > 0) {
        if (first_of_stage) {
          if (!TC_WAIT_DQ(empty + s, (uint32_t)(((j / STAGES) & 1) ^ 1), 8, acc1)) break;
          tc_fence_after();                                // the MMAs that read this slot have retired
        }
        tmem_st_32x32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + WT_COL0 + (uint32_t)((s * KT + t) * 32), outr);
        if (last_of_stage) tc_fence_before();
      } else {
        fence_proxy_async_smem();                          // generic-proxy stores -> visible to the tensor core
      }
      if (last_of_stage) {
        __syncwarp();
        if (lane == 0) mbar_arrive(ready + s);
      }
      TC_CK(c5); TC_ACC(acc3, c4, c5);
    }
    if (dw == 0 && lane == 0) { TC_GT(13); TC_PUT(8, acc0); TC_PUT(9, acc1); TC_PUT(10, acc2); TC_PUT(11, acc3); }
  }
  if (p.splits > 1) {
    // all threads of all the tile's CTAs: partial tiles complete -> reduce -> nobody leaves while its tile is being read
    __syncwarp();
    cluster_barrier();
    cluster_reduce_partials(p, smem, m0, n0, SW ? SW : BN, AM, warp, (int)(blockDim.x >> 5), lane, sw_s, b_s, SW > 0);
    __syncwarp();
    cluster_barrier();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TC_GT(14);
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}


// ---- 128 x 128 block quantisation (channel_scale_mode 5): FP8 x FP8 or INT8 x INT8 --------------------------
// out[m, n] = sum_kb (sum_{k in kb} x[m,k] w[n,k]) * s_x[m, kb] * s_w[kb, n / 128]  (gemm_kernels.py:396-450).  A K tile of
// 128 bytes is exactly one block, so every K tile's four MMAs start a fresh partial sum in one of the tensor-memory
// accumulators (512 / BN of them, used in turn); the epilogue warps drain it (tcgen05.ld), multiply by the two block scales and add it to the running
// sums they keep in registers while the MMAs of the next K tile fill the other accumulator.  Eight epilogue warps: a
// warp owns one 32-row quadrant and one half of the columns.
// One 128 x BN output tile per CTA (BN = 256: two weight blocks side by side, each column half with its own block scale;
// a K tile then moves 48 KB through shared memory for twice the arithmetic of the 32 KB of BN = 128); both operands by
// TMA (128-byte swizzle) through a STAGES-deep ring.
constexpr int kBlockqEpiWarps = 8;
template <bool INT8, int BN, int STAGES>
__global__ void __launch_bounds__(64 + 32 * kBlockqEpiWarps, 1) gl_gemm_tc_blockq_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                   const __grid_constant__ CUtensorMap tmB, const TcParams p) {
  constexpr int A_BYTES = 128 * 128, B_BYTES = BN * 128, STAGE_BYTES = A_BYTES + B_BYTES, HALF = BN / 2;
  constexpr int NBUF = 512 / BN;                        // accumulators: all of tensor memory, so that the MMAs run ahead of the drain
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;                  // [NBUF] the K tile's partial sum is complete
  uint64_t* acc_empty = acc_full + 8;                   // [NBUF] ... and has been drained by the eight epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 8);
  float* sw_s = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(tmem_slot + 1) + 15) & ~(uintptr_t)15);
  float* b_s = sw_s + BN;
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + 127) / 128;
  int mt, nt;
  tile_origin(p.band, (int)blockIdx.x, tiles_m, (p.N + BN - 1) / BN, mt, nt);
  const int m0 = mt * 128, n0 = nt * BN;
  stage_epilogue_consts(p, sw_s, b_s, n0, BN);          // bias (no channel scale in this mode: sw_s = 1)
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < NBUF; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, kBlockqEpiWarps); }
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) tmem_alloc(tmem_slot, NBUF * BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  gl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      gl_grid_dependency_wait();
      for (int kt = 0; kt < p.nkt; ++kt) {
        const int s = kt % STAGES;
        if (!mbar_wait_spin(empty + s, (uint32_t)(((kt / STAGES) & 1) ^ 1), &s_abort, p.status, 2)) break;
        unsigned char* st = smem + s * STAGE_BYTES;
        mbar_expect_tx(full + s, A_BYTES + B_BYTES);
        tma_load_2d(st, &tmA, full + s, kt * 128, m0);
        tma_load_2d(st + A_BYTES, &tmB, full + s, kt * 128, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kt = 0; kt < p.nkt && ok; ++kt) {
        const int s = kt % STAGES, ab = kt % NBUF;
        if (!mbar_wait_spin(acc_empty + ab, (uint32_t)(((kt / NBUF) & 1) ^ 1), &s_abort, p.status, 6) ||
            !mbar_wait_spin(full + s, (uint32_t)((kt / STAGES) & 1), &s_abort, p.status, 3)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_ss<INT8 ? KIND_I8 : KIND_F8F6F4>(tmem_base + (uint32_t)(ab * BN), da + 2 * j, db + 2 * j, p.idesc, j > 0 ? 1u : 0u);
        tc_commit(empty + s);
        tc_commit(acc_full + ab);
      }
    }
  } else {
    gl_grid_dependency_wait();
    const int quad = warp & 3, cb = ((warp - 2) >> 2) * HALF;   // TMEM lane quadrant and first column of this warp
    const int m = m0 + quad * 32 + lane;
    const int kblocks = p.K / 128;
    float acc[HALF];
#pragma unroll
    for (int i = 0; i < HALF; ++i) acc[i] = 0.f;
    bool ok = true;
    // the two block scales of a K tile are requested one K tile ahead: their latency is off the accumulator hand-over
    const float* sxp = p.scales_x + (size_t)(m < p.M ? m : 0) * kblocks;
    const int nblk = min((n0 + cb) >> 7, (p.N - 1) >> 7);           // (a column half past N computes and stores nothing)
    const float* swp = p.bq_scales + (long long)nblk * p.bq_stride_n;
    float sx_n = sxp[0], sw_n = swp[0];
    for (int kt = 0; kt < p.nkt && ok; ++kt) {
      const int ab = kt % NBUF;
      const float sc = (m < p.M ? sx_n : 0.f) * sw_n;
      if (kt + 1 < p.nkt) { sx_n = sxp[kt + 1]; sw_n = swp[(long long)(kt + 1) * p.bq_stride_g]; }
      if (!mbar_wait_spin(acc_full + ab, (uint32_t)((kt / NBUF) & 1), &s_abort, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ab * BN + cb);
      if constexpr (HALF == 64) {                            // both loads in flight, the buffer handed back before the arithmetic
        uint32_t r0[32], r1[32];
        tmem_ld_32x32_issue(taddr, r0);
        tmem_ld_32x32_issue(taddr + 32, r1);
        tmem_ld_wait();
        tmem_ld_fence(r0);
        tmem_ld_fence(r1);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + ab);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[i] = fmaf(INT8 ? (float)(int32_t)r0[i] : __uint_as_float(r0[i]), sc, acc[i]);
          acc[32 + i] = fmaf(INT8 ? (float)(int32_t)r1[i] : __uint_as_float(r1[i]), sc, acc[32 + i]);
        }
      } else {                                               // 128 columns: 32 at a time (registers)
#pragma unroll
        for (int c0 = 0; c0 < HALF; c0 += 32) {
          uint32_t rr[32];
          tmem_ld_32x32(taddr + c0, rr);
          if (c0 + 32 == HALF) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + ab);
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c0 + i] = fmaf(INT8 ? (float)(int32_t)rr[i] : __uint_as_float(rr[i]), sc, acc[c0 + i]);
        }
      }
    }
    if (ok && m < p.M) {
#pragma unroll
      for (int c0 = 0; c0 < HALF; c0 += 32) {
        if (n0 + cb + c0 >= p.N) break;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = acc[c0 + i];
        finish_row_chunk(p, m, n0 + cb + c0, v, 1.f, sw_s + cb + c0, b_s + cb + c0);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, NBUF * BN);
}

template <typename K>
static int set_smem(K kern, size_t smem) {
  GL_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  return GL_OK;
}

template <bool INT8, int BN, int STAGES>
static int launch_blockq_kernel(const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, cudaStream_t st) {
  const size_t smem = 1024 + STAGES * (128 * 128 + BN * 128) + (2 * STAGES + 16) * 8 + 32 + 2 * BN * 4 + 16;
  auto kern = gl_gemm_tc_blockq_kernel<INT8, BN, STAGES>;
  if (int rc = set_smem(kern, smem)) return rc;
  const int tiles = ((p.M + 127) / 128) * ((p.N + BN - 1) / BN);
  GL_CUDA_CHECK(gl_launch_pdl(kern, dim3(tiles), dim3(64 + 32 * kBlockqEpiWarps), smem, st, tmA, tmB, p));
  return GL_OK;
}


template <int KIND, int BN, int STAGES>
static int launch_tma_kernel(const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, cudaStream_t st,
                             const CUtensorMap* tmSFA = nullptr, const CUtensorMap* tmSFB = nullptr) {
  using KT = KindTraits<KIND>;
  constexpr int rep_a = (KT::SF_ATOMS >= 2 && BN == 256) ? 4 : 1, rep_b = (KIND == KIND_NVF4 && BN == 256) ? 4 : 1;
  constexpr size_t stage = 128 * 128 + BN * 128 + KT::SF_ATOMS * 512 * (rep_a + rep_b * ((BN + 127) / 128));
  const size_t smem = 1024 + STAGES * stage + (2 * STAGES + 4) * 8 + 32 + 4 * 2 * BN * 4 + 16;
  auto kern = gl_gemm_tc_kernel<KIND, BN, STAGES>;
  if (int rc = set_smem(kern, smem)) return rc;
  const int tiles = ((p.M + 127) / 128) * ((p.N + BN - 1) / BN);
  const int grid = tiles < gl_num_sms() ? tiles : gl_num_sms();
  GL_CUDA_CHECK(gl_launch_pdl(kern, dim3(grid), dim3(192), smem, st, tmA, tmB, tmSFA ? *tmSFA : tmA, tmSFB ? *tmSFB : tmB, p));
  return GL_OK;
}

// slots of the packed-word ring: what is left of the 227 KB after the activation / dequantised-tile stages, at most 16
constexpr int a16_wslots(int NB, int BN, int STAGES, int AM, int SW = 0, int ctas_per_sm = 1) {
  const int wslot = a16_wslot_bytes(NB, BN);
  const int left = (ctas_per_sm == 2 ? 113 * 1024 : 232448) - 1024 -
                   STAGES * (SW ? a16_tiles_per_stage(SW, ctas_per_sm == 2 ? 4 : 8) * SW * 128 : AM * 128 * 128 + BN * 128) - 4096;
  return left / wslot > 16 ? 16 : left / wslot;
}

template <typename XT, int NB, int BN, int STAGES, int AM = 1, int SW = 0, int DQW = 8>
static int launch_a16_kernel(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmS, const CUtensorMap& tmZ, const TcParams& p,
                             cudaStream_t st) {
  constexpr int WROWS = 64 / (32 / NB);
  constexpr int WS = a16_wslots(NB, BN, STAGES, AM, SW, DQW == 4 ? 2 : 1);
  static_assert(WS >= 2, "packed-word ring needs two slots");
  constexpr size_t stage = SW ? a16_tiles_per_stage(SW, DQW) * SW * 128 : AM * 128 * 128 + BN * 128, wslot = a16_wslot_bytes(NB, BN);
  constexpr size_t smem = 1024 + STAGES * stage + WS * wslot + (3 * STAGES + 2 * WS + 1) * 8 + 32 + 2 * BN * 4 + 16;
  static_assert(smem <= (DQW == 4 ? 113 * 1024 : 232448), "shared memory of the A16Wn kernel");
  auto kern = gl_gemm_tc_a16wn_kernel<XT, NB, BN, STAGES, AM, WS, SW, DQW>;
  if (int rc = set_smem(kern, smem)) return rc;
  const int tiles = p.grid_tiles > 0 ? p.grid_tiles : (SW ? 1 : (p.M + 128 * AM - 1) / (128 * AM)) * ((p.N + BN - 1) / BN);
  // K splits: the CTAs of a tile are one cluster along y and add their partial tiles through distributed shared memory
  if (p.splits > 1 && (p.splits > 8 || (size_t)AM * 128 * (SW ? 64 : BN) * 4 > STAGES * stage + WS * wslot))
    GL_FAIL(GL_E_INVALID, "gl_matmul: %d K splits of a %d x %d tile do not fit the cluster reduction", p.splits, AM * 128, BN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, p.splits);
  cfg.blockDim = dim3((6 + DQW) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)p.splits;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;       // the packed-word ring fills while the previous kernel drains
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  GL_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmA, tmW, tmS, tmZ, p));
  GL_LAUNCH_CHECK("gl_gemm_tc_a16wn_kernel");
  return GL_OK;
}

enum TcPath { TC_NONE = 0, TC_A16WN, TC_FP8, TC_INT8, TC_MXFP4, TC_NVFP4, TC_MXFP8, TC_BLOCKQ_FP8, TC_BLOCKQ_INT8 };

static TcPath classify(const gl_matmul_args* a) {
  if (a->M < 1) return TC_NONE;
  if (((uintptr_t)a->x & 15) || ((uintptr_t)a->w & 15) || ((uintptr_t)a->out & 15)) return TC_NONE;
  if (!(a->out_dtype == GL_BF16 || a->out_dtype == GL_FP16 || a->out_dtype == GL_FP32)) return TC_NONE;
  // 128 x 128 block quantisation: e4m3 x e4m3 or int8 x int8, fp32 block scales on both sides
  if (a->channel_scale_mode == 5) {
    if (a->elements_per_sample != 1 || a->W_nbits != 8 || a->W_group_mode != 0 || a->w_stride_k != 1 || a->w_stride_n != a->K ||
        a->K % 128 != 0 || a->scales == nullptr || a->scales_x == nullptr || a->meta_dtype != GL_FP32) return TC_NONE;
    if (a->x_dtype == GL_FP8 && a->w_dtype == GL_FP8 && a->input_dtype == GL_FP8) return TC_BLOCKQ_FP8;
    if (a->x_dtype == GL_INT8 && a->w_dtype == GL_INT8 && a->input_dtype == GL_INT8) return TC_BLOCKQ_INT8;
    return TC_NONE;
  }
  const int e = a->elements_per_sample;
  // A16Wn: fp16 / bf16 activations, 4- or 2-bit codes packed in int32 along K, group-wise meta data
  if ((a->x_dtype == GL_BF16 || a->x_dtype == GL_FP16) && a->input_dtype == a->x_dtype && a->w_dtype == GL_INT32 &&
      (a->W_nbits == 8 || a->W_nbits == 4 || a->W_nbits == 2 || a->W_nbits == 1) && e == 32 / a->W_nbits) {
    if (a->w_stride_n != 1 || a->w_stride_k != a->N || a->N % 4 != 0) return TC_NONE;
    if (a->group_size % 64 != 0) return TC_NONE;
    if (!(a->channel_scale_mode == 0 || a->channel_scale_mode == 1)) return TC_NONE;
    const bool need_s = a->W_group_mode >= 2, need_z = a->W_group_mode == 1 || a->W_group_mode >= 3;
    if ((need_s || a->channel_scale_mode == 1) && (a->scales == nullptr || a->meta_dtype != a->x_dtype)) return TC_NONE;
    if (need_s && (a->s_stride_n != 1 || a->s_stride_g != a->N)) return TC_NONE;
    if (need_z && a->zeros == nullptr) return TC_NONE;
    if (need_z && !a->zero_is_scalar && a->zeros_dtype != a->x_dtype) return TC_NONE;
    if (need_z && a->zero_is_scalar && a->zeros_dtype != GL_INT32) return TC_NONE;
    if (a->channel_scale_mode == 1 && a->W_group_mode >= 2) return TC_NONE;
    // the rows of group scales / zeros travel by TMA: 16-byte base and pitch
    if ((need_s || (need_z && !a->zero_is_scalar)) && a->N % 8 != 0) return TC_NONE;
    if (need_s && ((uintptr_t)a->scales & 15)) return TC_NONE;
    if (need_z && !a->zero_is_scalar && ((uintptr_t)a->zeros & 15)) return TC_NONE;
    return TC_A16WN;
  }
  // MXFP8 with block-scaled activations (A8W8_MXFP_dynamic): e4m3 x e4m3, e8m0 scale per 32 on both sides, given as atoms
  // ... or with activations quantised per token (A8W8_MXFP_dynamic(post_scale=True), channel_scale_mode 2): the same MMA kind
  // with unit activation scale atoms, the token's fp32 scale applied by the epilogue
  if (a->input_dtype == GL_MXFP8 && a->x_dtype == GL_FP8 && a->w_dtype == GL_FP8 && e == 1 && a->W_nbits == 8 &&
      (a->channel_scale_mode == 4 || a->channel_scale_mode == 2) &&
      a->w_stride_k == 1 && a->w_stride_n == a->K && a->K % 128 == 0 && a->group_size == 32) {
    if (a->w_scales_atoms == nullptr || a->scales_x == nullptr || (a->channel_scale_mode == 4 && a->sx_layout != 1)) return TC_NONE;
    if (((uintptr_t)a->w_scales_atoms & 15) || ((uintptr_t)a->scales_x & 15)) return TC_NONE;
    return TC_MXFP8;
  }
  // A8W8: e4m3 x e4m3 or int8 x int8, weights [N, K] with K contiguous, optional per-token / per-channel scales
  if (e == 1 && a->W_nbits == 8 && a->W_group_mode == 0 && a->w_stride_k == 1 && a->w_stride_n == a->K && a->K % 16 == 0) {
    if ((a->channel_scale_mode == 2 || a->channel_scale_mode == 3) && a->scales_x == nullptr) return TC_NONE;
    if ((a->channel_scale_mode == 1 || a->channel_scale_mode == 3) && a->scales == nullptr) return TC_NONE;
    if (a->x_dtype == GL_FP8 && a->w_dtype == GL_FP8 && a->input_dtype == GL_FP8) return TC_FP8;
    if (a->x_dtype == GL_INT8 && a->w_dtype == GL_INT8 && a->input_dtype == GL_INT8) return TC_INT8;
    return TC_NONE;
  }
  // MXFP4 / NVFP4 with block-scaled activations: both operands packed e2m1, scale factors given as atoms
  if ((a->input_dtype == GL_MXFP4 || a->input_dtype == GL_NVFP4) && a->x_dtype == GL_UINT8 && a->w_dtype == GL_UINT8 && e == 2 &&
      a->channel_scale_mode == 4 && a->w_stride_k == 1 && a->w_stride_n == a->K / 2 && a->K % 32 == 0) {
    const int gs = a->input_dtype == GL_MXFP4 ? 32 : 16;
    if (a->group_size != gs || a->w_scales_atoms == nullptr || a->scales_x == nullptr || a->sx_layout != 1) return TC_NONE;
    if ((a->K / gs) % 4 != 0) return TC_NONE;
    if (((uintptr_t)a->w_scales_atoms & 15) || ((uintptr_t)a->scales_x & 15)) return TC_NONE;
    return a->input_dtype == GL_MXFP4 ? TC_MXFP4 : TC_NVFP4;
  }
  return TC_NONE;
}

}  // namespace

int gl_gemm_tc_supported(const gl_matmul_args* a) { return classify(a) != TC_NONE; }

// Tile-config cache entry of this problem: family GEMM (M >= 64) / GEMM_SPLITK under the reference's signature
// "(Mb, N, K, group_size, e, type_id)"; the fields "tile_n" (128 / 256) and "splits" (A16Wn K splits) override the
// built-in choices below.
static int tc_cfg_int(const gl_matmul_args* a, const char* key, int dflt) {
  const int idt = (a->input_dtype == GL_BF16) ? GL_FP16 : a->input_dtype;
  char sig[128];
  snprintf(sig, sizeof(sig), "(%d, %d, %d, %d, %d, %d)", gl_get_closest_m(a->M), a->N, a->K, a->group_size, a->elements_per_sample, idt * 100 + a->W_nbits);
  return gl_cfg_int(a->M >= 64 ? "GEMM" : "GEMM_SPLITK", sig, key, dflt);
}

static int tc_tile_n(const gl_matmul_args* a) {
  const int dflt = (a->N >= 256 && ((int64_t)((a->M + 127) / 128) * ((a->N + 255) / 256) >= 96)) ? 256 : 128;
  const int req = tc_cfg_int(a, "tile_n", 0);
  return ((req == 128 || req == 256) && a->N >= req) ? req : dflt;
}

// Shape of an A16Wn launch: columns per tile (BN), 128-row activation tiles per CTA (AM) and K splits.
// More than 128 rows and words of at most 4 bits share one dequantised weight tile between two accumulators (AM = 2);
// 256-column tiles when that still gives 96 CTAs; when the tiles alone leave more than half of the SMs idle, the K range
// is divided so that about one CTA per SM runs (every split gets at least 8 K tiles and none is empty).
// Cache entry fields "tile_n", "am", "splits" override the three choices.
struct A16Plan { int BN, AM, splits, SW, ctas; };
static A16Plan a16_plan(const gl_matmul_args* a) {
  A16Plan pl;
  // at most 64 rows: operands swapped, the rows of x are the MMA's 32 or 64 columns ("swap": 0 in the cache entry turns it off)
  pl.SW = (a->M <= 64 && tc_cfg_int(a, "swap", 1) != 0) ? (a->M <= 32 ? 32 : 64) : 0;
  pl.AM = (a->M > 128 && a->W_nbits <= 4 && tc_cfg_int(a, "am", 2) == 2) ? 2 : 1;
  const int64_t tiles_m = (a->M + 128 * pl.AM - 1) / (128 * pl.AM);
  const int req_bn = tc_cfg_int(a, "tile_n", 0);
  pl.BN = (a->N >= 256 && tiles_m * ((a->N + 255) / 256) >= 96) ? 256 : 128;
  if ((req_bn == 128 || req_bn == 256) && a->N >= req_bn) pl.BN = req_bn;
  if (pl.SW) pl.BN = 128;
  // swapped form: two CTAs per SM (4 dequant warps each) unless the cache entry says "ctas": 1
  pl.ctas = (pl.SW && tc_cfg_int(a, "ctas", 2) == 2) ? 2 : 1;
  const int64_t tiles = tiles_m * ((a->N + pl.BN - 1) / pl.BN);
  const int nkt = (a->K + 63) / 64, sms = gl_num_sms();
  pl.splits = 1;
  if (tiles > 16384 || nkt < 16) return pl;
  if (pl.AM == 2 && pl.BN == 256) return pl;           // a 256 x 256 fp32 partial tile does not fit the CTA's shared memory
  auto trim = [&](int s) { while (s > 1 && (s - 1) * ((nkt + s - 1) / s) >= nkt) --s; return s; };
  const int req = tc_cfg_int(a, "splits", 0);
  if (req >= 1 && req <= 8 && req <= nkt / 8) { pl.splits = trim(req); return pl; }
  if (tiles * 2 > sms * pl.ctas) return pl;
  int s = (int)(sms * pl.ctas / tiles);
  if (s > 8) s = 8;
  if (s > nkt / 8) s = nkt / 8;
  if (s < 1) s = 1;
  pl.splits = trim(s);
  return pl;
}

uint64_t gl_gemm_tc_workspace(const gl_matmul_args* a) {
  uint64_t need = gl_matmul_counter_bytes();
  return need;
}

int gl_gemm_tc_launch(const gl_matmul_args* a, cudaStream_t st) {
  const TcPath path = classify(a);
  if (path == TC_NONE) GL_FAIL(GL_E_UNSUPPORTED, "gl_matmul: no tensor-core kernel for this problem");
  if (a->workspace == nullptr || a->workspace_bytes < gl_gemm_tc_workspace(a))
    GL_FAIL(GL_E_WORKSPACE, "gl_matmul: workspace of %llu bytes needed", (unsigned long long)gl_gemm_tc_workspace(a));
  if ((uintptr_t)a->workspace & 15) GL_FAIL(GL_E_INVALID, "gl_matmul: workspace must be 16-byte aligned");
  TcParams p;
  memset(&p, 0, sizeof(p));
  p.splits = 1;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.out = a->out; p.out_dtype = a->out_dtype; p.bias = a->bias;
  p.status = reinterpret_cast<int*>(reinterpret_cast<char*>(a->workspace) + gl_matmul_counter_bytes() - 256);
  p.meta_scale = nullptr;
  // activations of 64 MB and more: tiles in bands of 2048 rows (see tile_origin)
  const int64_t x_bytes = (int64_t)a->M * a->K * (a->x_dtype == GL_BF16 || a->x_dtype == GL_FP16 ? 4 : (a->x_dtype == GL_UINT8 ? 1 : 2)) / 2;
  const A16Plan a16 = path == TC_A16WN ? a16_plan(a) : A16Plan{0, 1, 1, 0, 1};
  const int BN = path == TC_A16WN ? a16.BN : tc_tile_n(a);
  // decode sizes of the TMA formats swap the operands (16 or 32 token columns)
  const int swap_bn = (path != TC_A16WN && a->M <= 32 && a->N >= 128) ? (a->M <= 16 ? 16 : 32) : 0;
  p.band = x_bytes >= (64ll << 20) ? (path == TC_A16WN ? 16 / a16.AM : 16) : 0;
  CUtensorMap tmA, tmB;
  if (path == TC_A16WN) {
    p.nkt = (a->K + 63) / 64;
    p.splits = a16.splits;
    p.idesc = gl_idesc(1, a->x_dtype == GL_BF16 ? 1 : 0, a->x_dtype == GL_BF16 ? 1 : 0, 128, a16.SW ? a16.SW : BN);
    if (a->channel_scale_mode == 1) { p.scales_w = a->scales; p.scales_w_dtype = a->meta_dtype; }
    p.gscales = a->scales; p.gzeros = a->zeros; p.group_size = a->group_size; p.W_group_mode = a->W_group_mode; p.zero_is_scalar = a->zero_is_scalar;
    const int wrows = 64 / a->elements_per_sample;
    if (int rc = gl_make_tmap_2d(&tmA, a->x, a->x_dtype == GL_BF16 ? 1 : 2, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->K * 2, 64, a16.SW ? (uint32_t)a16.SW : 128u, true)) return rc;
    if (int rc = gl_make_tmap_2d(&tmB, a->w, 3, (uint64_t)a->N, (uint64_t)(a->K / a->elements_per_sample), (uint64_t)a->N * 4, (uint32_t)BN, (uint32_t)wrows, false)) return rc;
    // rows of group scales / zeros [groups][N]; modes without them never touch their map
    CUtensorMap tmS = tmB, tmZ = tmB;
    const int xkind = a->x_dtype == GL_BF16 ? 1 : 2;
    const uint64_t n_groups = (uint64_t)(a->K / a->group_size);
    if (a->W_group_mode >= 2)
      if (int rc = gl_make_tmap_2d(&tmS, a->scales, xkind, (uint64_t)a->N, n_groups, (uint64_t)a->N * 2, (uint32_t)BN, 1, false)) return rc;
    if ((a->W_group_mode == 1 || a->W_group_mode >= 3) && !a->zero_is_scalar)
      if (int rc = gl_make_tmap_2d(&tmZ, a->zeros, xkind, (uint64_t)a->N, n_groups, (uint64_t)a->N * 2, (uint32_t)BN, 1, false)) return rc;
#define GL_A16(XT, NB)                                                                              \
    (BN == 256 ? launch_a16_kernel<XT, NB, 256, 3>(tmA, tmB, tmS, tmZ, p, st) : launch_a16_kernel<XT, NB, 128, 4>(tmA, tmB, tmS, tmZ, p, st))
    if (a16.SW) {
#ifndef GL_SW_STAGES
#define GL_SW_STAGES 4      // stages of the x / tensor-memory ring of the swapped form
#endif
#define GL_A16_SW(XT, NB) (a16.ctas == 2 ? (a16.SW == 32 ? launch_a16_kernel<XT, NB, 128, 2, 1, 32, 4>(tmA, tmB, tmS, tmZ, p, st) : launch_a16_kernel<XT, NB, 128, 2, 1, 64, 4>(tmA, tmB, tmS, tmZ, p, st)) \
                                         : (a16.SW == 32 ? launch_a16_kernel<XT, NB, 128, GL_SW_STAGES, 1, 32>(tmA, tmB, tmS, tmZ, p, st) : launch_a16_kernel<XT, NB, 128, GL_SW_STAGES, 1, 64>(tmA, tmB, tmS, tmZ, p, st)))
      if (a->x_dtype == GL_BF16) {
        if (a->W_nbits == 8) return GL_A16_SW(__nv_bfloat16, 8);
        if (a->W_nbits == 4) return GL_A16_SW(__nv_bfloat16, 4);
        if (a->W_nbits == 2) return GL_A16_SW(__nv_bfloat16, 2);
        return GL_A16_SW(__nv_bfloat16, 1);
      }
      if (a->W_nbits == 8) return GL_A16_SW(__half, 8);
      if (a->W_nbits == 4) return GL_A16_SW(__half, 4);
      if (a->W_nbits == 2) return GL_A16_SW(__half, 2);
      return GL_A16_SW(__half, 1);
#undef GL_A16_SW
    }
    if (a16.AM == 2) {      // (words of at most 4 bits: three 72 KB stages at BN = 256, four 52 KB stages at BN = 128)
      // 256 x 256 tiles whose last wave would fill at most half of the SMs: that wave's tiles run as 256 x 128 halves in
      // a second launch (one wave of about 0.6 of a wide tile's time instead of a whole one; "tail": 0 in the cache
      // entry turns it off).  8192 x 8192, M = 4096: 512 tiles = 3.46 waves -> 444 tiles + 136 halves.
      const int sms = gl_num_sms();
      const int wide_tiles = ((a->M + 255) / 256) * ((a->N + 255) / 256), rem = wide_tiles % sms;
      if (BN == 256 && p.splits == 1 && wide_tiles > sms && rem > 0 && 2 * rem <= sms && tc_cfg_int(a, "tail", 1) != 0) {
        TcParams p1 = p, p2 = p;
        p1.grid_tiles = wide_tiles - rem;
        p2.grid_tiles = 2 * rem; p2.tile_base = wide_tiles - rem; p2.tail = 1;
        p2.idesc = gl_idesc(1, a->x_dtype == GL_BF16 ? 1 : 0, a->x_dtype == GL_BF16 ? 1 : 0, 128, 128);
        CUtensorMap tmB2, tmS2, tmZ2;
        if (int rc = gl_make_tmap_2d(&tmB2, a->w, 3, (uint64_t)a->N, (uint64_t)(a->K / a->elements_per_sample), (uint64_t)a->N * 4, 128u, (uint32_t)wrows, false)) return rc;
        tmS2 = tmB2; tmZ2 = tmB2;
        if (a->W_group_mode >= 2)
          if (int rc = gl_make_tmap_2d(&tmS2, a->scales, xkind, (uint64_t)a->N, n_groups, (uint64_t)a->N * 2, 128u, 1, false)) return rc;
        if ((a->W_group_mode == 1 || a->W_group_mode >= 3) && !a->zero_is_scalar)
          if (int rc = gl_make_tmap_2d(&tmZ2, a->zeros, xkind, (uint64_t)a->N, n_groups, (uint64_t)a->N * 2, 128u, 1, false)) return rc;
#define GL_A16_TAIL(XT, NB)                                                                          \
        do {                                                                                        \
          if (int rc = launch_a16_kernel<XT, NB, 256, 3, 2>(tmA, tmB, tmS, tmZ, p1, st)) return rc;  \
          return launch_a16_kernel<XT, NB, 128, 4, 2>(tmA, tmB2, tmS2, tmZ2, p2, st);                \
        } while (0)
        if (a->x_dtype == GL_BF16) {
          if (a->W_nbits == 4) GL_A16_TAIL(__nv_bfloat16, 4);
          if (a->W_nbits == 2) GL_A16_TAIL(__nv_bfloat16, 2);
          GL_A16_TAIL(__nv_bfloat16, 1);
        }
        if (a->W_nbits == 4) GL_A16_TAIL(__half, 4);
        if (a->W_nbits == 2) GL_A16_TAIL(__half, 2);
        GL_A16_TAIL(__half, 1);
#undef GL_A16_TAIL
      }
#define GL_A16_2(XT, NB) (BN == 256 ? launch_a16_kernel<XT, NB, 256, 3, 2>(tmA, tmB, tmS, tmZ, p, st) : launch_a16_kernel<XT, NB, 128, 4, 2>(tmA, tmB, tmS, tmZ, p, st))
      if (a->x_dtype == GL_BF16) {
        if (a->W_nbits == 4) return GL_A16_2(__nv_bfloat16, 4);
        if (a->W_nbits == 2) return GL_A16_2(__nv_bfloat16, 2);
        return GL_A16_2(__nv_bfloat16, 1);
      }
      if (a->W_nbits == 4) return GL_A16_2(__half, 4);
      if (a->W_nbits == 2) return GL_A16_2(__half, 2);
      return GL_A16_2(__half, 1);
#undef GL_A16_2
    }
    if (a->x_dtype == GL_BF16) {
      if (a->W_nbits == 8) return GL_A16(__nv_bfloat16, 8);
      if (a->W_nbits == 4) return GL_A16(__nv_bfloat16, 4);
      if (a->W_nbits == 2) return GL_A16(__nv_bfloat16, 2);
      return GL_A16(__nv_bfloat16, 1);
    }
    if (a->W_nbits == 8) return GL_A16(__half, 8);
    if (a->W_nbits == 4) return GL_A16(__half, 4);
    if (a->W_nbits == 2) return GL_A16(__half, 2);
    return GL_A16(__half, 1);
#undef GL_A16
  }
  if (path == TC_BLOCKQ_FP8 || path == TC_BLOCKQ_INT8) {
    p.nkt = a->K / 128;
    // 256-column tiles when they still give every SM a tile ("tile_n" in the cache entry overrides).  Decode sizes: an MMA
    // reads its 128-row operand (here the mostly empty x tile) at 32 B/clk, 128 cycles per 32 bytes of K whatever the
    // number of weight columns, so a CTA streams 128-column weight tiles at 32 B/clk at best; 64-column tiles on twice
    // as many SMs measured the same total (8192 x 8192, M = 1: 37 against 32 us) and are not built.
    const int bq_req = tc_cfg_int(a, "tile_n", 0);
    const int64_t bq_tm = (a->M + 127) / 128;
    int bq_bn = (a->N >= 256 && bq_tm * ((a->N + 255) / 256) >= gl_num_sms()) ? 256 : 128;
    if ((bq_req == 128 || bq_req == 256) && a->N >= bq_req) bq_bn = bq_req;
    p.idesc = (path == TC_BLOCKQ_FP8) ? gl_idesc(1, 0, 0, 128, bq_bn) : gl_idesc(2, 1, 1, 128, bq_bn);
    p.scales_x = reinterpret_cast<const float*>(a->scales_x);
    p.bq_scales = reinterpret_cast<const float*>(a->scales);
    p.bq_stride_g = a->s_stride_g; p.bq_stride_n = a->s_stride_n;
    if (int rc = gl_make_tmap_2d(&tmA, a->x, 0, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->K, 128, 128, true)) return rc;
    if (int rc = gl_make_tmap_2d(&tmB, a->w, 0, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->K, 128, (uint32_t)bq_bn, true)) return rc;
    if (bq_bn == 256) return path == TC_BLOCKQ_FP8 ? launch_blockq_kernel<false, 256, 4>(tmA, tmB, p, st) : launch_blockq_kernel<true, 256, 4>(tmA, tmB, p, st);
    return path == TC_BLOCKQ_FP8 ? launch_blockq_kernel<false, 128, 6>(tmA, tmB, p, st) : launch_blockq_kernel<true, 128, 6>(tmA, tmB, p, st);
  }
  if (path == TC_FP8 || path == TC_INT8) {
    p.nkt = (a->K + 127) / 128;
    p.idesc = (path == TC_FP8) ? gl_idesc(1, 0, 0, 128, BN) : gl_idesc(2, 1, 1, 128, BN);
    if (a->channel_scale_mode == 2 || a->channel_scale_mode == 3) p.scales_x = reinterpret_cast<const float*>(a->scales_x);
    if (a->channel_scale_mode == 1 || a->channel_scale_mode == 3) { p.scales_w = a->scales; p.scales_w_dtype = a->meta_dtype; }
    if (swap_bn) {   // decode sizes: weights on the 128-row side, tokens on the narrow side
      p.M = a->N; p.N = a->M; p.swap = 1;
      p.idesc = (path == TC_FP8) ? gl_idesc(1, 0, 0, 128, swap_bn) : gl_idesc(2, 1, 1, 128, swap_bn);
      if (int rc = gl_make_tmap_2d(&tmA, a->w, 0, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->K, 128, 128, true)) return rc;
      if (int rc = gl_make_tmap_2d(&tmB, a->x, 0, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->K, 128, (uint32_t)swap_bn, true)) return rc;
#ifndef GL_SWAP_STAGES
#define GL_SWAP_STAGES 8     // ring depth of the swapped (decode) form: 8 x 18 KB
#endif
      if (path == TC_FP8) return swap_bn == 16 ? launch_tma_kernel<KIND_F8F6F4, 16, GL_SWAP_STAGES>(tmA, tmB, p, st) : launch_tma_kernel<KIND_F8F6F4, 32, GL_SWAP_STAGES>(tmA, tmB, p, st);
      return swap_bn == 16 ? launch_tma_kernel<KIND_I8, 16, GL_SWAP_STAGES>(tmA, tmB, p, st) : launch_tma_kernel<KIND_I8, 32, GL_SWAP_STAGES>(tmA, tmB, p, st);
    }
    if (int rc = gl_make_tmap_2d(&tmA, a->x, 0, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->K, 128, 128, true)) return rc;
    if (int rc = gl_make_tmap_2d(&tmB, a->w, 0, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->K, 128, (uint32_t)BN, true)) return rc;
    if (path == TC_FP8) return BN == 256 ? launch_tma_kernel<KIND_F8F6F4, 256, 4>(tmA, tmB, p, st) : launch_tma_kernel<KIND_F8F6F4, 128, 6>(tmA, tmB, p, st);
    return BN == 256 ? launch_tma_kernel<KIND_I8, 256, 4>(tmA, tmB, p, st) : launch_tma_kernel<KIND_I8, 128, 6>(tmA, tmB, p, st);
  }
  if (path == TC_MXFP8) {
    // block-scaled fp8: operands as in the FP8 path (128 bytes = 128 values of K per row and stage), one scale atom per stage
    p.nkt = a->K / 128;
    p.sf_kblocks = a->K / 32 / 4;
    p.meta_scale = nullptr;
    const int bn8 = swap_bn ? swap_bn : BN;              // (256-column tiles copy this kind's single atom per operand block one by one)
    p.idesc = gl_idesc_block_scaled(0, 1, 128, bn8);     // formats: e4m3 x e4m3, e8m0 scales
    const bool per_token = a->channel_scale_mode == 2;  // no activation atoms: fp32 scale per token in the epilogue
    if (per_token) p.scales_x = reinterpret_cast<const float*>(a->scales_x);
    if (swap_bn) {
      p.M = a->N; p.N = a->M; p.swap = 1;
      p.sfa = reinterpret_cast<const uint8_t*>(a->w_scales_atoms);
      p.sfb = per_token ? nullptr : reinterpret_cast<const uint8_t*>(a->scales_x);
      if (int rc = gl_make_tmap_2d(&tmA, a->w, 0, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->K, 128, 128, true)) return rc;
      if (int rc = gl_make_tmap_2d(&tmB, a->x, 0, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->K, 128, (uint32_t)swap_bn, true)) return rc;
      return swap_bn == 16 ? launch_tma_kernel<KIND_MXF8, 16, 8>(tmA, tmB, p, st) : launch_tma_kernel<KIND_MXF8, 32, 8>(tmA, tmB, p, st);
    }
    p.sfa = per_token ? nullptr : reinterpret_cast<const uint8_t*>(a->scales_x);
    p.sfb = reinterpret_cast<const uint8_t*>(a->w_scales_atoms);
    if (int rc = gl_make_tmap_2d(&tmA, a->x, 0, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->K, 128, 128, true)) return rc;
    if (int rc = gl_make_tmap_2d(&tmB, a->w, 0, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->K, 128, (uint32_t)BN, true)) return rc;
    return BN == 256 ? launch_tma_kernel<KIND_MXF8, 256, 4>(tmA, tmB, p, st) : launch_tma_kernel<KIND_MXF8, 128, 6>(tmA, tmB, p, st);
  }
  // block-scaled fp4
  const int gs = path == TC_MXFP4 ? 32 : 16;
  p.nkt = (a->K + 255) / 256;
  p.idesc = gl_idesc_block_scaled(1, path == TC_MXFP4 ? 1 : 0, 128, BN);
  p.sfa = reinterpret_cast<const uint8_t*>(a->scales_x);
  p.sfb = reinterpret_cast<const uint8_t*>(a->w_scales_atoms);
  p.sf_kblocks = a->K / gs / 4;
  p.meta_scale = (path == TC_NVFP4) ? a->meta_scale : nullptr;
  if (swap_bn) {
    p.M = a->N; p.N = a->M; p.swap = 1;
    p.idesc = gl_idesc_block_scaled(1, path == TC_MXFP4 ? 1 : 0, 128, swap_bn);
    p.sfa = reinterpret_cast<const uint8_t*>(a->w_scales_atoms);
    p.sfb = reinterpret_cast<const uint8_t*>(a->scales_x);
    if (int rc = gl_make_tmap_2d(&tmA, a->w, 0, (uint64_t)a->K / 2, (uint64_t)a->N, (uint64_t)a->K / 2, 128, 128, true)) return rc;
    if (int rc = gl_make_tmap_2d(&tmB, a->x, 0, (uint64_t)a->K / 2, (uint64_t)a->M, (uint64_t)a->K / 2, 128, (uint32_t)swap_bn, true)) return rc;
    if (path == TC_MXFP4) return swap_bn == 16 ? launch_tma_kernel<KIND_MXF4, 16, 8>(tmA, tmB, p, st) : launch_tma_kernel<KIND_MXF4, 32, 8>(tmA, tmB, p, st);
    return swap_bn == 16 ? launch_tma_kernel<KIND_NVF4, 16, 8>(tmA, tmB, p, st) : launch_tma_kernel<KIND_NVF4, 32, 8>(tmA, tmB, p, st);
  }
  if (int rc = gl_make_tmap_2d(&tmA, a->x, 0, (uint64_t)a->K / 2, (uint64_t)a->M, (uint64_t)a->K / 2, 128, 128, true)) return rc;
  if (int rc = gl_make_tmap_2d(&tmB, a->w, 0, (uint64_t)a->K / 2, (uint64_t)a->N, (uint64_t)a->K / 2, 128, (uint32_t)BN, true)) return rc;
  if (BN == 256) {
    // scale-factor atoms [128-row block][K atom][512 B] seen as [block][K atom][4 replicas, stride 0][128 words]
    CUtensorMap tmSFA, tmSFB;
    const uint32_t atoms = path == TC_MXFP4 ? 2 : 4;
    if (int rc = gl_make_tmap_sf_replicated(&tmSFA, a->scales_x, (uint64_t)p.sf_kblocks, (uint64_t)((a->M + 127) / 128), atoms)) return rc;
    if (int rc = gl_make_tmap_sf_replicated(&tmSFB, a->w_scales_atoms, (uint64_t)p.sf_kblocks, (uint64_t)((a->N + 127) / 128), atoms)) return rc;
    return path == TC_MXFP4 ? launch_tma_kernel<KIND_MXF4, 256, 4>(tmA, tmB, p, st, &tmSFA, &tmSFB)
                            : launch_tma_kernel<KIND_NVF4, 256, 3>(tmA, tmB, p, st, &tmSFA, &tmSFB);
  }
  if (path == TC_MXFP4) return launch_tma_kernel<KIND_MXF4, 128, 6>(tmA, tmB, p, st);
  return launch_tma_kernel<KIND_NVF4, 128, 6>(tmA, tmB, p, st);
}
