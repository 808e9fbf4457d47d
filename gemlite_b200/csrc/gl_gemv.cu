// Streaming low-bit GEMV / skinny GEMM for decode sizes (M <= 32), sm_100a.
//
// Replaces the reference's gemv / gemv_revsplitK / gemv_splitK Triton kernels
// (gemlite/triton_kernels/gemv_kernels.py:245-426, gemv_revsplitK_kernels.py:248-443,
// gemv_splitK_kernels.py:257-477) and its small-M gemm_splitK path
// (gemm_splitK_kernels.py:300-523) for packed integer weights.
//
// The kernel is HBM-bound, so it is organised around the weight stream:
//  * W_q is the reference's packed layout, int32 [K/e, N] row-major, e = 32/W_nbits values of
//    one output column per word (gemlite/bitpack.py:36-60, gemlite/core.py:623-637).  Every lane
//    issues 128-bit streaming loads of 4 adjacent columns (a warp instruction covers 4 packed rows x
//    128 bytes); two batches of U loads per lane are in flight (register double buffer).
//  * Fields are unpacked two at a time with one shift + one LOP3 into fp16/bf16 "magic number"
//    pairs (BIAS+q) and fed straight to mma.sync m16n8k16 as the A operand (16 output columns x
//    16 k); the activations are the B operand (8 batch rows per MMA), so M = 1..8 costs one MMA
//    per 256 weights and M <= 32 re-uses the same A fragments.  The k order inside a packed word
//    is permuted identically on both operands, which a dot product does not see.
//  * Dequantisation is applied per group to the fp32 accumulators, not per weight:
//        sum_k x_k*(q_k*s + z')  =  s * sum_k x_k*(BIAS+q_k)  +  (z' - BIAS*s) * sum_k x_k
//    with the group sums of x computed once per CTA while x is staged in shared memory.
//  * K is split over blockIdx.y.  Up to 8 slices form a thread-block cluster: each CTA parks its fp32
//    partial tile in shared memory and the ranks add disjoint column slices through distributed
//    shared memory in rank order (deterministic, no global scratch).  More slices go through an fp32
//    workspace: the last CTA to arrive for a column tile (arrival counter, no spinning) adds the
//    partials in slice order.  Channel scales / bias are applied once, in the final sum.
//  * Programmatic dependent launch: the first batch of weight loads and the scale / zero prefetch
//    are issued before griddepcontrol.wait, so in a chain of layers they overlap the tail of the
//    previous kernel; activations, workspace and output are only touched after the wait.
#include "gl_tc_common.cuh"
#include <stdlib.h>
#include <string.h>
#include <mutex>

namespace {

constexpr int kMaxTiles = 16384;                  // arrival counters at the head of the workspace
constexpr int kStatusBytes = 256;                 // device status word after the counters

struct GemvParams {
  const void* x; const int32_t* w; const void* scales; const void* zeros; const void* bias;
  void* out; float* partials; unsigned int* counters; int* status;
  int M, N, K;
  int T;            // iterations over K: one iteration = 4 packed rows = 4*e k-values
  int gi;           // iterations per quantisation group
  int splitK;
  int cluster;      // CTAs per thread-block cluster along K (1 = split-K through the global workspace)
  int W_group_mode, channel_scale_mode, zero_is_scalar;
  int out_dtype;
  int max_slice_iters, max_seg;
  int s_in, c_in;   // warp-independent kernel: K slices and 32-column groups inside a CTA
#ifdef GL_GEMV_TRACE
  unsigned long long* trace;   // profiling build: per-warp globaltimer stamps [cta][warp][8]
#endif
};
// Profiling build (-DGL_GEMV_TRACE): every warp of the warp-independent kernel records globaltimer stamps at its phase
// boundaries (start, constants ready, dependency resolved, activations staged, main loop done, end).
#ifdef GL_GEMV_TRACE
#define GL_STAMP(i) do { if (p.trace != nullptr && (threadIdx.x & 31) == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
  p.trace[(((size_t)blockIdx.y * gridDim.x + blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 8 + (i)] = t_; } } while (0)
#else
#define GL_STAMP(i) do { } while (0)
#endif

template <typename XT> struct XTraits;
template <> struct XTraits<__nv_bfloat16> {
  static constexpr uint32_t MAGIC = 0x43004300u;  // 128.0 | q, exact for q < 128
  static constexpr float BIAS = 128.f;
  __device__ static float to_float(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }
};
template <> struct XTraits<__half> {
  static constexpr uint32_t MAGIC = 0x64006400u;  // 1024.0 | q, exact for q < 1024
  static constexpr float BIAS = 1024.f;
  __device__ static float to_float(uint16_t v) { return __half2float(__ushort_as_half(v)); }
};

template <typename XT>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                 uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ int4 ldg_stream(const int32_t* p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// load 4 consecutive meta values (scales / zeros of this lane's 4 columns) as fp32
template <typename XT>
__device__ __forceinline__ void load_meta4(const void* base, int64_t idx, float (&o)[4]) {
  uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + idx);
  o[0] = XTraits<XT>::to_float((uint16_t)(v.x & 0xffffu)); o[1] = XTraits<XT>::to_float((uint16_t)(v.x >> 16));
  o[2] = XTraits<XT>::to_float((uint16_t)(v.y & 0xffffu)); o[3] = XTraits<XT>::to_float((uint16_t)(v.y >> 16));
}

// NB: bits per weight (4/2/1). XT: activation / scale dtype. MT: number of 8-row batch tiles (M <= 8*MT).
// U: packed-row loads per lane per batch; two batches are in flight (register double buffer).
template <int NB, typename XT, int MT, int U>
__global__ void __launch_bounds__(128) gl_gemv_stream_kernel(const GemvParams p) {
  constexpr int E = 32 / NB;        // k-values per packed word
  constexpr int H = E / 8;          // 16-byte pieces of x per packed row
  constexpr int HALF = E / 2;       // field i is paired with field i + HALF
  constexpr uint32_t FMASK = ((1u << NB) - 1u) * 0x00010001u;
  using XTr = XTraits<XT>;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int r = lane >> 2, t = lane & 3;

  // K slice of this CTA, in iterations
  const int split = blockIdx.y;
  const int it0 = (int)(((long long)p.T * split) / p.splitK);
  const int it1 = (int)(((long long)p.T * (split + 1)) / p.splitK);
  const int nit = it1 - it0;
  const int g0 = it0 / p.gi;                          // first group touched
  const int nseg = (it1 + p.gi - 1) / p.gi - g0;      // group segments in this slice

  // shared: xs | xsum | scales | zeros   (xs is re-used for the partial tile of the cluster reduction)
  uint4* xs = reinterpret_cast<uint4*>(smem_raw);                 // [iteration][piece][batch row][quad lane] 16-byte units
  const int xs_units = p.max_slice_iters * H * p.M * 4;
  const int cta_cols = nwarps * 32;
  const int part_units = (p.M * cta_cols + 3) / 4;                // fp32 partial tile, in 16-byte units
  float* xsum = reinterpret_cast<float*>(xs + max(xs_units, part_units));   // [segment][8*MT]
  uint16_t* ms = reinterpret_cast<uint16_t*>(xsum + (size_t)p.max_seg * 8 * MT);   // scales [segment][cta_cols]
  uint16_t* mz = ms + (size_t)p.max_seg * cta_cols;                                // zeros  [segment][cta_cols]

  // ---- before the dependency wait: everything that only touches weights ---------------------------
  const int n0 = (blockIdx.x * nwarps + warp) * 32 + 4 * r;      // this lane's first column
  const bool ncol_ok = n0 < p.N;
  const int32_t* wp = p.w + (size_t)(it0 * 4 + t) * p.N + n0;
  const size_t wstep = (size_t)4 * p.N;
  int4 cur[U], nxt[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    cur[u] = make_int4(0, 0, 0, 0);
    if (ncol_ok && u < nit) cur[u] = ldg_stream(wp + (size_t)u * wstep);
  }
  {
    const bool need_s = p.W_group_mode >= 2;
    const bool need_z = (p.W_group_mode == 1 || p.W_group_mode >= 3) && !p.zero_is_scalar;
    const int pieces_per_row = cta_cols / 4;                       // 8-byte pieces (4 columns)
    const int ccol0 = blockIdx.x * cta_cols;
    for (int i = threadIdx.x; i < nseg * pieces_per_row; i += blockDim.x) {
      const int sg = i / pieces_per_row, pc = i % pieces_per_row;
      const int n = ccol0 + pc * 4;
      if (n < p.N) {
        const size_t goff = (size_t)(g0 + sg) * p.N + n;
        if (need_s)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(gltc::smem_u32(ms + sg * cta_cols + pc * 4)),
                       "l"(reinterpret_cast<const uint16_t*>(p.scales) + goff) : "memory");
        if (need_z)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(gltc::smem_u32(mz + sg * cta_cols + pc * 4)),
                       "l"(reinterpret_cast<const uint16_t*>(p.zeros) + goff) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- stage x in fragment order and sum it per quantisation group ------------------------------------
  // One (segment, batch row) pair is handled by a group of GL lanes: each lane permutes 16-byte units of x
  // into the MMA B-fragment order, keeps a running sum, and a fixed shuffle tree adds the lanes (deterministic).
  {
    const uint16_t* xg = reinterpret_cast<const uint16_t*>(p.x);
    const int kbase = it0 * 4 * E;
    for (int i = threadIdx.x; i < nseg * 8 * MT; i += blockDim.x) xsum[i] = 0.f;
    const int seg_units = p.gi * 4 * H;                            // 16-byte units in a full segment
    int GL = 4;
    while (GL < 32 && GL < seg_units) GL <<= 1;
    const int pairs_per_warp = 32 / GL;
    const int sub = lane / GL, l = lane % GL;
    const int npairs = nseg * p.M;
    const int passes = (seg_units + GL - 1) / GL;
    __syncthreads();
    for (int pb = warp * pairs_per_warp; pb < npairs; pb += nwarps * pairs_per_warp) {   // warp-uniform
      const int pair = pb + sub;
      const bool pv = pair < npairs;
      const int sg = pv ? pair / p.M : 0, m = pv ? pair % p.M : 0;
      const int ua = (max((g0 + sg) * p.gi, it0) - it0) * 4 * H;
      const int ub = (min((g0 + sg + 1) * p.gi, it1) - it0) * 4 * H;
      float sum = 0.f;
      for (int ps = 0; ps < passes; ++ps) {
        const int u = ua + ps * GL + l;
        if (pv && u < ub) {
          const int row = u / H, hh = u % H;
          // piece hh holds, for pp = 2*hh, 2*hh+1: x[2pp], x[2pp+HALF], x[2pp+1], x[2pp+1+HALF]
          const uint16_t* xr = xg + (size_t)m * p.K + kbase + row * E;
          uint16_t v[8];
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int pp = 2 * hh + q;
            const uint32_t lo = *reinterpret_cast<const uint32_t*>(xr + 2 * pp);          // x[2pp], x[2pp+1]
            const uint32_t hi = *reinterpret_cast<const uint32_t*>(xr + 2 * pp + HALF);   // x[2pp+HALF], x[2pp+1+HALF]
            v[4 * q + 0] = (uint16_t)(lo & 0xffffu); v[4 * q + 1] = (uint16_t)(hi & 0xffffu);
            v[4 * q + 2] = (uint16_t)(lo >> 16);     v[4 * q + 3] = (uint16_t)(hi >> 16);
          }
          float s8 = 0.f;
#pragma unroll
          for (int q = 0; q < 8; ++q) s8 += XTr::to_float(v[q]);
          sum += s8;
          uint4 o;
          o.x = v[0] | ((uint32_t)v[1] << 16); o.y = v[2] | ((uint32_t)v[3] << 16);
          o.z = v[4] | ((uint32_t)v[5] << 16); o.w = v[6] | ((uint32_t)v[7] << 16);
          xs[((((row >> 2) * H + hh) * p.M + m) << 2) + (row & 3)] = o;
        }
      }
      for (int off = GL >> 1; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (pv && l == 0) xsum[sg * 8 * MT + m] = sum;
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();

  // ---- main loop ----------------------------------------------------------------------------
  // acc[q][a][mt]: separate accumulators for the two MMAs of a packed row (q) so that consecutive MMAs do not
  // depend on each other; they are added when a group is flushed
  float acc[2][2][MT][4], outv[2][MT][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < MT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) { acc[0][a][b][c] = 0.f; acc[1][a][b][c] = 0.f; outv[a][b][c] = 0.f; }

  int seg = 0;
  int seg_end = min((g0 + 1) * p.gi, it1) - it0;     // local iteration where the segment ends

  auto flush = [&](int sgi) {
    // out += alpha[col] * acc + beta[col] * xsum[m]
    float al[4], be[4];
    const int mcol = warp * 32 + 4 * r;                            // this lane's columns inside the CTA tile
    if (p.W_group_mode >= 2) {
      const uint2 v = *reinterpret_cast<const uint2*>(ms + sgi * cta_cols + mcol);
      al[0] = XTr::to_float((uint16_t)(v.x & 0xffffu)); al[1] = XTr::to_float((uint16_t)(v.x >> 16));
      al[2] = XTr::to_float((uint16_t)(v.y & 0xffffu)); al[3] = XTr::to_float((uint16_t)(v.y >> 16));
    } else { al[0] = al[1] = al[2] = al[3] = 1.f; }
    float z[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.W_group_mode == 1 || p.W_group_mode >= 3) {
      if (p.zero_is_scalar) { const float zz = (float)(*reinterpret_cast<const int32_t*>(p.zeros)); z[0] = z[1] = z[2] = z[3] = zz; }
      else {
        const uint2 v = *reinterpret_cast<const uint2*>(mz + sgi * cta_cols + mcol);
        z[0] = XTr::to_float((uint16_t)(v.x & 0xffffu)); z[1] = XTr::to_float((uint16_t)(v.x >> 16));
        z[2] = XTr::to_float((uint16_t)(v.y & 0xffffu)); z[3] = XTr::to_float((uint16_t)(v.y >> 16));
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (p.W_group_mode == 4)      be[c] = z[c] - XTr::BIAS * al[c];          // fma(b, s, z')
      else if (p.W_group_mode == 3) be[c] = -(XTr::BIAS + z[c]) * al[c];       // (b - z) * s
      else if (p.W_group_mode == 1) be[c] = -(XTr::BIAS + z[c]);               // b - z
      else                          be[c] = -XTr::BIAS * al[c];                // b * s | b
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const float xs0 = xsum[sgi * 8 * MT + mt * 8 + 2 * t], xs1 = xsum[sgi * 8 * MT + mt * 8 + 2 * t + 1];
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        outv[a][mt][0] += al[2 * a] * (acc[0][a][mt][0] + acc[1][a][mt][0]) + be[2 * a] * xs0;
        outv[a][mt][1] += al[2 * a] * (acc[0][a][mt][1] + acc[1][a][mt][1]) + be[2 * a] * xs1;
        outv[a][mt][2] += al[2 * a + 1] * (acc[0][a][mt][2] + acc[1][a][mt][2]) + be[2 * a + 1] * xs0;
        outv[a][mt][3] += al[2 * a + 1] * (acc[0][a][mt][3] + acc[1][a][mt][3]) + be[2 * a + 1] * xs1;
#pragma unroll
        for (int c = 0; c < 4; ++c) { acc[0][a][mt][c] = 0.f; acc[1][a][mt][c] = 0.f; }
      }
    }
  };

  for (int itb = 0; itb < nit; itb += U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      nxt[u] = make_int4(0, 0, 0, 0);
      if (ncol_ok && itb + U + u < nit) nxt[u] = ldg_stream(wp + (size_t)(itb + U + u) * wstep);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int it = itb + u;
      if (it < nit) {
        const uint32_t w[4] = {(uint32_t)cur[u].x, (uint32_t)cur[u].y, (uint32_t)cur[u].z, (uint32_t)cur[u].w};
#pragma unroll
        for (int hh = 0; hh < H; ++hh) {
          uint4 xb[MT];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {      // batch rows >= M contribute zeros (their outputs are never stored)
            const int m = mt * 8 + r;
            xb[mt] = (m < p.M) ? xs[(((it * H + hh) * p.M + m) << 2) + t] : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int pp = 2 * hh + q;               // MMA index inside the packed row
            uint32_t f0[4], f1[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              f0[c] = ((w[c] >> (NB * (2 * pp))) & FMASK) | XTr::MAGIC;       // fields 2pp, 2pp+HALF
              f1[c] = ((w[c] >> (NB * (2 * pp + 1))) & FMASK) | XTr::MAGIC;   // fields 2pp+1, 2pp+1+HALF
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint32_t b0 = q ? xb[mt].z : xb[mt].x, b1 = q ? xb[mt].w : xb[mt].y;
              mma16816<XT>(acc[q][0][mt], f0[0], f0[1], f1[0], f1[1], b0, b1);
              mma16816<XT>(acc[q][1][mt], f0[2], f0[3], f1[2], f1[3], b0, b1);
            }
          }
        }
        if (it + 1 == seg_end) {
          flush(seg);
          ++seg;
          seg_end = min((g0 + seg + 1) * p.gi, it1) - it0;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) cur[u] = nxt[u];
  }

  // ---- epilogue -------------------------------------------------------------------------------
  // lane owns columns n0..n0+3 and batch rows m = mt*8 + 2t, 2t+1:
  //   outv[a][mt][0] = (col 2a, m=2t)  [1] = (col 2a, 2t+1)  [2] = (col 2a+1, 2t)  [3] = (col 2a+1, 2t+1)
  if (p.cluster > 1) {
    // Split-K inside a thread-block cluster: every CTA parks its fp32 partial tile in its own shared memory,
    // then CTA `rank` adds a slice of the columns over all ranks (fixed order) through distributed shared memory.
    float* part = reinterpret_cast<float*>(xs);
    __syncthreads();                                 // xs is dead
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int m = mt * 8 + 2 * t + j;
        if (m < p.M)
          *reinterpret_cast<float4*>(part + m * cta_cols + warp * 32 + 4 * r) =
              make_float4(outv[0][mt][j], outv[0][mt][2 + j], outv[1][mt][j], outv[1][mt][2 + j]);
      }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int slice = cta_cols / p.cluster;          // columns reduced by this CTA
    const uint32_t part_s = gltc::smem_u32(part);
    for (int i = threadIdx.x; i < p.M * slice; i += blockDim.x) {
      const int m = i / slice, c = rank * slice + i % slice;
      const int n = blockIdx.x * cta_cols + c;
      float v = 0.f;
      for (int q = 0; q < p.cluster; ++q) {
        uint32_t ra;
        float pv;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(part_s + (uint32_t)(m * cta_cols + c) * 4u), "r"(q));
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv) : "r"(ra) : "memory");
        v += pv;
      }
      if (n < p.N) {
        if (p.channel_scale_mode == 1) v *= XTr::to_float(reinterpret_cast<const uint16_t*>(p.scales)[n]);
        if (p.bias != nullptr) v += gl_load_as_float(p.bias, n, p.out_dtype);
        gl_store_out(p.out, (int64_t)m * p.N + n, v, p.out_dtype);
      }
    }
    // nobody may leave while a peer still reads its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    return;
  }

  const bool multi = p.splitK > 1;
  if (multi) {
    if (ncol_ok) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int m = mt * 8 + 2 * t + j;
          if (m < p.M) {
            float4 v = make_float4(outv[0][mt][j], outv[0][mt][2 + j], outv[1][mt][j], outv[1][mt][2 + j]);
            __stcg(reinterpret_cast<float4*>(p.partials + ((size_t)split * p.M + m) * p.N + n0), v);
          }
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int prev = atomicAdd(p.counters + blockIdx.x, 1u);
      s_last = (prev == (unsigned int)(p.splitK - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) p.counters[blockIdx.x] = 0u;   // leave the counter clean for the next call
  }
  if (!ncol_ok) return;

  float chs[4] = {1.f, 1.f, 1.f, 1.f};
  if (p.channel_scale_mode == 1) load_meta4<XT>(p.scales, n0, chs);
  float bs[4] = {0.f, 0.f, 0.f, 0.f};
  if (p.bias != nullptr) {
    if (p.out_dtype == GL_FP32) { const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.bias) + n0); bs[0] = b.x; bs[1] = b.y; bs[2] = b.z; bs[3] = b.w; }
    else if (p.out_dtype == GL_BF16) load_meta4<__nv_bfloat16>(p.bias, n0, bs);
    else load_meta4<__half>(p.bias, n0, bs);
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int m = mt * 8 + 2 * t + j;
      if (m >= p.M) continue;
      float v[4];
      if (multi) {
        v[0] = v[1] = v[2] = v[3] = 0.f;
        for (int s = 0; s < p.splitK; ++s) {
          const float4 q = __ldcg(reinterpret_cast<const float4*>(p.partials + ((size_t)s * p.M + m) * p.N + n0));
          v[0] += q.x; v[1] += q.y; v[2] += q.z; v[3] += q.w;
        }
      } else {
        v[0] = outv[0][mt][j]; v[1] = outv[0][mt][2 + j]; v[2] = outv[1][mt][j]; v[3] = outv[1][mt][2 + j];
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) v[c] = v[c] * chs[c] + bs[c];
      const size_t o = (size_t)m * p.N + n0;
      if (p.out_dtype == GL_BF16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 pk; pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o) = pk;
      } else if (p.out_dtype == GL_FP16) {
        __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
        uint2 pk; pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + o) = pk;
      } else {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
}

// ---- warp-independent kernel ---------------------------------------------------------------------------
// The same arithmetic with every trip count fixed and no CTA-wide barrier before the final reduction.
// A CTA is s_in x c_in warps: c_in column groups of 32 columns times s_in consecutive K slices; the grid's y
// dimension adds `cluster` outer slices that are summed through distributed shared memory.  A warp owns one
// (slice, 32 columns) pair end to end: it issues its first weight loads and scale/zero copies before the
// dependency wait, converts its own per-group constants, and only shares the staged activations of its slice
// with the c_in - 1 warps beside it (named barrier).  The per-group sums of x come out of the tensor core as well
// (an all-ones A operand), so staging is a permuted copy.
// Preconditions (checked by the planner): N % (32 c_in) == 0; T % (s_in cluster) == 0; every slice is a whole
// number of 8-iteration batches and either holds whole groups or lies inside one group.
template <typename XT>
__device__ __forceinline__ void mma16816z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816z<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  const float z = 0.f;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}
template <>
__device__ __forceinline__ void mma16816z<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  const float z = 0.f;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}
template <typename XT> struct OnesPair;
template <> struct OnesPair<__nv_bfloat16> { static constexpr uint32_t V = 0x3F803F80u; };
template <> struct OnesPair<__half> { static constexpr uint32_t V = 0x3C003C00u; };

// (v & mask) | magic as one three-input logic op with both constants in registers
__device__ __forceinline__ uint32_t and_or(uint32_t v, uint32_t mask, uint32_t magic) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(v), "r"(mask), "r"(magic));
  return d;
}

// GI: iterations per quantisation group when it divides 8 (1, 2, 4); 0 = a multiple of 8 (p.gi), flushed at run time
template <int NB, typename XT, int MT, int GI>
__global__ void __launch_bounds__(MT == 1 ? 512 : 256, MT == 1 ? 1 : 2) gl_gemv_warp_kernel(const GemvParams p) {
  // 8-bit words hold 4 k: two iterations share one 16-byte unit of staged activations (W8 below)
  constexpr bool W8 = NB == 8;
  constexpr int E = 32 / NB, H = W8 ? 1 : E / 8, HALF = E / 2, U = 8;
  // bf16 has 7 mantissa bits: a byte enters as (128 + low 7 bits) and (128 + 128 * top bit) in two MMAs, bias 256 in all
  constexpr bool SPLIT8 = W8 && XTraits<XT>::MAGIC == 0x43004300u;
  constexpr float BIASV = SPLIT8 ? 256.f : XTraits<XT>::BIAS;
  constexpr uint32_t FMASK = SPLIT8 ? 0x007F007Fu : ((1u << NB) - 1u) * 0x00010001u;
  constexpr uint32_t ONES = OnesPair<XT>::V;
  using XTr = XTraits<XT>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane >> 2, t = lane & 3;
  const int s_in = p.s_in, c_in = p.c_in;
  const int sl = warp / c_in, wc = warp - sl * c_in;       // slice and column group of this warp inside the CTA
  const int nit = p.T / (s_in * p.cluster);                // iterations per slice (exact)
  const int it0 = (blockIdx.y * s_in + sl) * nit;
  const int g0 = it0 / p.gi;
  const int nseg = (nit + p.gi - 1) / p.gi;                // whole groups, or 1 when the slice lies inside a group
  const int ccols = c_in * 32;

  // shared: x fragments [slice] | per-warp {alpha, beta, raw scales, raw zeros, zero unit} | partial tiles [slice]
  const int xs_slice_units = (W8 ? nit / 2 : nit * H) * p.M * 4;
  uint4* xs = reinterpret_cast<uint4*>(smem_raw) + (size_t)sl * xs_slice_units;
  unsigned char* wbase = smem_raw + (size_t)s_in * xs_slice_units * 16 + (size_t)warp * (nseg * 32 * 12 + 16);
  float* alpha = reinterpret_cast<float*>(wbase);
  float* beta = alpha + nseg * 32;
  uint16_t* ms = reinterpret_cast<uint16_t*>(beta + nseg * 32);
  uint16_t* mz = ms + nseg * 32;
  uint4* zero_unit = reinterpret_cast<uint4*>(mz + nseg * 32);
  float* part = reinterpret_cast<float*>(smem_raw + (size_t)s_in * xs_slice_units * 16 +
                                         (size_t)s_in * c_in * (nseg * 32 * 12 + 16));     // [slice][M][ccols]

  GL_STAMP(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next layer may start its own weight loads
  // ---- before the dependency wait: first batch of weights, raw scales / zeros of this warp's groups -------
  const int n0 = blockIdx.x * ccols + wc * 32 + 4 * r;
  const int32_t* wp = p.w + (size_t)(it0 * 4 + t) * p.N + n0;
  const size_t wstep = (size_t)4 * p.N;
  int4 buf[U];
#pragma unroll
  for (int u = 0; u < U; ++u) buf[u] = ldg_stream(wp + (size_t)u * wstep);
  // Epilogue constants of the column this thread finishes after the last barrier (thread i finishes elements i,
  // i + blockDim.x, ... of the [M][ccols] tile, and blockDim.x is a multiple of ccols): requested now, so that their
  // DRAM latency is not paid by the last CTA at the very end of the kernel
  float epi_bias = 0.f, epi_scale = 1.f;
  {
    const int n = blockIdx.x * ccols + (int)(threadIdx.x % ccols);
    if (p.bias != nullptr) epi_bias = gl_load_as_float(p.bias, n, p.out_dtype);
    if (p.channel_scale_mode == 1) epi_scale = XTr::to_float(reinterpret_cast<const uint16_t*>(p.scales)[n]);
  }
  {
    const bool need_s = p.W_group_mode >= 2;
    const bool need_z = (p.W_group_mode == 1 || p.W_group_mode >= 3) && !p.zero_is_scalar;
    for (int i = lane; i < nseg * 8; i += 32) {                    // 8-byte pieces (4 columns)
      const int sg = i >> 3, pc = i & 7;
      const size_t goff = (size_t)(g0 + sg) * p.N + blockIdx.x * ccols + wc * 32 + pc * 4;
      if (need_s)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(gltc::smem_u32(ms + sg * 32 + pc * 4)),
                     "l"(reinterpret_cast<const uint16_t*>(p.scales) + goff) : "memory");
      if (need_z)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(gltc::smem_u32(mz + sg * 32 + pc * 4)),
                     "l"(reinterpret_cast<const uint16_t*>(p.zeros) + goff) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  if (lane == 0) *zero_unit = make_uint4(0u, 0u, 0u, 0u);
  // still before the dependency wait (this only touches the layer's own weights): convert the group constants
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncwarp();
  {                                                   // per-group fp32 constants: out += alpha * acc + beta * xsum
    // a lane converts 8 consecutive columns of one group at a time (two 16-byte loads, four 16-byte stores)
    const float zs = p.zero_is_scalar ? (float)(*reinterpret_cast<const int32_t*>(p.zeros)) : 0.f;
    const bool has_s = p.W_group_mode >= 2, has_z = (p.W_group_mode == 1 || p.W_group_mode >= 3) && !p.zero_is_scalar;
    for (int i = lane * 8; i < nseg * 32; i += 256) {
      uint4 sv = make_uint4(0u, 0u, 0u, 0u), zv = make_uint4(0u, 0u, 0u, 0u);
      if (has_s) sv = *reinterpret_cast<const uint4*>(ms + i);
      if (has_z) zv = *reinterpret_cast<const uint4*>(mz + i);
      const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w}, zw[4] = {zv.x, zv.y, zv.z, zv.w};
      float al[8], be[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a1 = has_s ? XTr::to_float((uint16_t)((sw[j >> 1] >> (16 * (j & 1))) & 0xffffu)) : 1.f;
        const float z1 = has_z ? XTr::to_float((uint16_t)((zw[j >> 1] >> (16 * (j & 1))) & 0xffffu)) : zs;
        float b1;
        if (p.W_group_mode == 4)      b1 = z1 - BIASV * a1;
        else if (p.W_group_mode == 3) b1 = -(BIASV + z1) * a1;
        else if (p.W_group_mode == 1) b1 = -(BIASV + z1);
        else                          b1 = -BIASV * a1;
        al[j] = a1; be[j] = b1;
      }
      *reinterpret_cast<float4*>(alpha + i) = make_float4(al[0], al[1], al[2], al[3]);
      *reinterpret_cast<float4*>(alpha + i + 4) = make_float4(al[4], al[5], al[6], al[7]);
      *reinterpret_cast<float4*>(beta + i) = make_float4(be[0], be[1], be[2], be[3]);
      *reinterpret_cast<float4*>(beta + i + 4) = make_float4(be[4], be[5], be[6], be[7]);
    }
    __syncwarp();
  }
  GL_STAMP(1);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  GL_STAMP(2);

  // ---- stage this slice of x in B-fragment order (shared by the c_in warps of the slice) -------------------
  {
    const uint16_t* xg = reinterpret_cast<const uint16_t*>(p.x) + (size_t)it0 * 4 * E;
    const int row_units = W8 ? nit * 2 : nit * 4 * H;              // 16-byte units per batch row
    const int tg = wc * 32 + lane, tgn = ccols;
    for (int m = 0; m < p.M; ++m) {
      const uint16_t* xr = xg + (size_t)m * p.K;
      if (W8) {
        // unit (iteration pair j, packed row t): {b0, b1} of iteration 2j then of 2j + 1, where b0 = (x0, x2) and
        // b1 = (x1, x3) of the row's four k (bytes 0 / 2 and 1 / 3 of the packed word share an extraction)
        for (int u = tg; u < row_units; u += tgn) {
          const int j = u >> 2, tt = u & 3;
          const uint2 ev = *reinterpret_cast<const uint2*>(xr + ((2 * j) * 4 + tt) * 4);
          const uint2 od = *reinterpret_cast<const uint2*>(xr + ((2 * j + 1) * 4 + tt) * 4);
          uint4 o;
          o.x = __byte_perm(ev.x, ev.y, 0x5410); o.y = __byte_perm(ev.x, ev.y, 0x7632);
          o.z = __byte_perm(od.x, od.y, 0x5410); o.w = __byte_perm(od.x, od.y, 0x7632);
          xs[((j * p.M + m) << 2) + tt] = o;
        }
        continue;
      }
      for (int u = tg; u < row_units; u += tgn) {
        const int row = u / H, hh = u - row * H;                   // packed row inside the slice, piece of the row
        const uint2 lo = *reinterpret_cast<const uint2*>(xr + row * E + 4 * hh);
        const uint2 hi = *reinterpret_cast<const uint2*>(xr + row * E + HALF + 4 * hh);
        uint4 o;
        o.x = __byte_perm(lo.x, hi.x, 0x5410); o.y = __byte_perm(lo.x, hi.x, 0x7632);
        o.z = __byte_perm(lo.y, hi.y, 0x5410); o.w = __byte_perm(lo.y, hi.y, 0x7632);
        xs[((((row >> 2) * H + hh) * p.M + m) << 2) + (row & 3)] = o;
      }
    }
  }
  if (c_in > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + sl), "r"(ccols) : "memory");
  else __syncwarp();
  GL_STAMP(3);

  // ---- main loop ----------------------------------------------------------------------------------------------
  const uint4* xcur[MT];
  int xstride[MT], pstride[MT];
  // constants kept in registers: the unpack mask / magic, and four separate copies of the all-ones A operand
  // (an MMA operand is a register quad; one shared register would be copied into a quad before every MMA)
  uint32_t fmask = FMASK, magic = XTr::MAGIC, ones0 = ONES, ones1 = ONES, ones2 = ONES, ones3 = ONES;
  asm volatile("" : "+r"(fmask), "+r"(magic), "+r"(ones0), "+r"(ones1), "+r"(ones2), "+r"(ones3));
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {                    // batch rows >= M read the zero unit with stride 0
    const int m = mt * 8 + r;
    const bool ok = m < p.M;
    xcur[mt] = ok ? xs + ((m << 2) + t) : zero_unit;
    xstride[mt] = ok ? H * p.M * 4 : 0;
    pstride[mt] = ok ? p.M * 4 : 0;
  }
  float acc[2][MT][4], accS[MT][4], outv[2][MT][4];
#pragma unroll
  for (int b = 0; b < MT; ++b)
#pragma unroll
    for (int c = 0; c < 4; ++c) { acc[0][b][c] = acc[1][b][c] = 0.f; accS[b][c] = 0.f; outv[0][b][c] = outv[1][b][c] = 0.f; }
  int seg = 0;

  auto flush = [&](int sgi, bool clear) {
    const float4 al4 = *reinterpret_cast<const float4*>(alpha + sgi * 32 + 4 * r);
    const float4 be4 = *reinterpret_cast<const float4*>(beta + sgi * 32 + 4 * r);
    const float al[4] = {al4.x, al4.y, al4.z, al4.w}, be[4] = {be4.x, be4.y, be4.z, be4.w};
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const float x0 = accS[mt][0], x1 = accS[mt][1];             // sums of x over the group, batch rows 2t, 2t+1
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        outv[a][mt][0] += al[2 * a] * acc[a][mt][0] + be[2 * a] * x0;
        outv[a][mt][1] += al[2 * a] * acc[a][mt][1] + be[2 * a] * x1;
        outv[a][mt][2] += al[2 * a + 1] * acc[a][mt][2] + be[2 * a + 1] * x0;
        outv[a][mt][3] += al[2 * a + 1] * acc[a][mt][3] + be[2 * a + 1] * x1;
        if (clear) { acc[a][mt][0] = acc[a][mt][1] = acc[a][mt][2] = acc[a][mt][3] = 0.f; }
      }
      if (clear) { accS[mt][0] = accS[mt][1] = accS[mt][2] = accS[mt][3] = 0.f; }
    }
  };

  // One rolling set of U loads per lane: as soon as an iteration's words have been unpacked, the same registers
  // are re-loaded with the words of iteration + U, so U x 512 bytes per warp stay in flight at all times.
  const int32_t* wnext = wp + (size_t)U * wstep;
  auto process = [&](int itb, bool reload) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t w[4] = {(uint32_t)buf[u].x, (uint32_t)buf[u].y, (uint32_t)buf[u].z, (uint32_t)buf[u].w};
      if constexpr (W8) {
        // one MMA K extent per iteration: bytes 0 / 2 of a word are k slots (2t, 2t+1), bytes 1 / 3 slots (2t+8, 2t+9)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint4 xv = xcur[mt][0];
          const uint32_t b0 = (u & 1) ? xv.z : xv.x, b1 = (u & 1) ? xv.w : xv.y;
          uint32_t lo[4], hi[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) { lo[c] = and_or(w[c], fmask, magic); hi[c] = and_or(w[c] >> 8, fmask, magic); }
          mma16816<XT>(acc[0][mt], lo[0], lo[1], hi[0], hi[1], b0, b1);
          mma16816<XT>(acc[1][mt], lo[2], lo[3], hi[2], hi[3], b0, b1);
          if constexpr (SPLIT8) {                        // the top bit of every byte: 128 + 128 * bit
#pragma unroll
            for (int c = 0; c < 4; ++c) { lo[c] = and_or(w[c], 0x00800080u, magic); hi[c] = and_or(w[c] >> 8, 0x00800080u, magic); }
            mma16816<XT>(acc[0][mt], lo[0], lo[1], hi[0], hi[1], b0, b1);
            mma16816<XT>(acc[1][mt], lo[2], lo[3], hi[2], hi[3], b0, b1);
          }
          mma16816<XT>(accS[mt], ones0, ones1, ones2, ones3, b0, b1);
        }
      }
#pragma unroll
      for (int hh = 0; hh < (W8 ? 0 : H); ++hh) {
        uint4 xb[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) xb[mt] = xcur[mt][hh * pstride[mt]];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int pp = 2 * hh + q;
          uint32_t f0[4], f1[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            f0[c] = and_or(w[c] >> (NB * (2 * pp)), fmask, magic);
            f1[c] = and_or(w[c] >> (NB * (2 * pp + 1)), fmask, magic);
          }
          const bool first = (GI > 0) && ((u % (GI > 0 ? GI : 1)) == 0) && hh == 0 && q == 0;   // compile-time
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint32_t b0 = q ? xb[mt].z : xb[mt].x, b1 = q ? xb[mt].w : xb[mt].y;
            if (first) {
              mma16816z<XT>(acc[0][mt], f0[0], f0[1], f1[0], f1[1], b0, b1);
              mma16816z<XT>(acc[1][mt], f0[2], f0[3], f1[2], f1[3], b0, b1);
              mma16816z<XT>(accS[mt], ones0, ones1, ones2, ones3, b0, b1);
            } else {
              mma16816<XT>(acc[0][mt], f0[0], f0[1], f1[0], f1[1], b0, b1);
              mma16816<XT>(acc[1][mt], f0[2], f0[3], f1[2], f1[3], b0, b1);
              mma16816<XT>(accS[mt], ones0, ones1, ones2, ones3, b0, b1);
            }
          }
        }
      }
      if (reload) { buf[u] = ldg_stream(wnext); wnext += wstep; }
      if (!W8 || (u & 1)) {                            // two 8-bit iterations share a unit
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) xcur[mt] += xstride[mt];
      }
      if (GI > 0) {
        if ((u % (GI > 0 ? GI : 1)) == (GI > 0 ? GI : 1) - 1) { flush(seg, false); ++seg; }
      }
    }
    if (GI == 0) {                                   // group = several whole batches (or the whole slice)
      const int done = itb + U;
      if (done % p.gi == 0 || done == nit) { flush(seg, true); ++seg; }
    }
  };

  const int nb = nit / U;
  for (int b = 0; b + 1 < nb; ++b) process(b * U, true);
  process((nb - 1) * U, false);

  GL_STAMP(4);
  // ---- reduction over the CTA's slices, then over the cluster ---------------------------------------------------
  {
    float* mine = part + (size_t)sl * p.M * ccols + wc * 32 + 4 * r;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int m = mt * 8 + 2 * t + j;
        if (m < p.M)
          *reinterpret_cast<float4*>(mine + m * ccols) = make_float4(outv[0][mt][j], outv[0][mt][2 + j], outv[1][mt][j], outv[1][mt][2 + j]);
      }
  }
  __syncthreads();
  const int tile_elems = p.M * ccols;
  if (p.cluster == 1) {
    for (int i = threadIdx.x; i < tile_elems; i += blockDim.x) {
      float v = part[i];
      for (int q = 1; q < s_in; ++q) v += part[q * tile_elems + i];
      const int m = i / ccols, n = blockIdx.x * ccols + (i - m * ccols);
      gl_store_out(p.out, (int64_t)m * p.N + n, v * epi_scale + epi_bias, p.out_dtype);
    }
    GL_STAMP(5);
    return;
  }
  for (int i = threadIdx.x; i < tile_elems; i += blockDim.x) {      // fold the CTA's slices into slice 0
    float v = part[i];
    for (int q = 1; q < s_in; ++q) v += part[q * tile_elems + i];
    part[i] = v;
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int slice = ccols / p.cluster;
    const uint32_t part_s = gltc::smem_u32(part);
    for (int i = threadIdx.x; i < p.M * slice; i += blockDim.x) {
      const int m = i / slice, c = rank * slice + (i - m * slice);
      const int n = blockIdx.x * ccols + c;
      float v = 0.f;
      for (int q = 0; q < p.cluster; ++q) {
        uint32_t ra;
        float pv;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(part_s + (uint32_t)(m * ccols + c) * 4u), "r"(q));
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv) : "r"(ra) : "memory");
        v += pv;
      }
      if (p.channel_scale_mode == 1) v *= XTr::to_float(reinterpret_cast<const uint16_t*>(p.scales)[n]);
      if (p.bias != nullptr) v += gl_load_as_float(p.bias, n, p.out_dtype);
      gl_store_out(p.out, (int64_t)m * p.N + n, v, p.out_dtype);
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

struct GemvPlan { int warps_n, splitK, cluster, MT, slice_iters, max_seg, tiles, warp_kernel, gi, s_in, c_in; size_t smem; };

// Tile parameters: built-in heuristic, overridden by a config-cache entry for the GEMV_REVSPLITK /
// GEMV_SPLITK / GEMV family under the reference's signature "(Mb, N, K, group_size, e, type_id)" with
// the integer fields "split_k", "warps_n", "stages".
static int json_int(const char* js, const char* key, int dflt) {
  if (!js) return dflt;
  char pat[64];
  snprintf(pat, sizeof(pat), "\"%s\"", key);
  const char* p = strstr(js, pat);
  if (!p) return dflt;
  p = strchr(p + strlen(pat), ':');
  if (!p) return dflt;
  return atoi(p + 1);
}

// One attempt at a plan for the warp-independent kernel with `c_in0` column groups per CTA and a shared-memory budget;
// returns false when the kernel's preconditions do not hold or the budget is exceeded.
static bool plan_warp_with(const gl_matmul_args* a, GemvPlan* pl, const char* js, int c_in0, size_t smem_limit) {
  const int e = a->elements_per_sample;
  if (!(a->W_nbits == 8 || a->W_nbits == 4 || a->W_nbits == 2) || a->M > 16 || a->N % 32 != 0 || a->K % (4 * e) != 0) return false;
  if (a->group_size % (4 * e) != 0) return false;
  const int T = a->K / (4 * e), H = e / 8, gi = a->group_size / (4 * e);
  const int colgroups = a->N / 32;
  if (!(gi == 1 || gi == 2 || gi == 4 || gi % 8 == 0)) return false;
  if (a->W_nbits == 8 && gi % 8 != 0) return false;               // 8-bit: only the run-time flush variant is built
  auto slice_ok = [&](int S) {
    if (S < 1 || T % S != 0) return false;
    const int nit = T / S;
    if (nit < 8 || nit % 8 != 0) return false;
    return gi <= 4 ? (nit % gi == 0) : (nit % gi == 0 || gi % nit == 0);
  };
  int c_in = c_in0;
  int s_in = 0, cluster = 0;
  if (js) {
    c_in = json_int(js, "c_in", c_in);
    s_in = json_int(js, "s_in", 0);
    cluster = json_int(js, "cluster_k", 0);
  }
  while (c_in > 1 && colgroups % c_in != 0) c_in >>= 1;
  if (c_in < 1 || c_in > 16 || colgroups % c_in != 0) return false;
  // staged activations + per-warp group constants + partial sums of a CTA of s slices x c column groups, nit iterations per slice
  auto smem_of = [&](int s, int c, int nit) {
    const int nseg = (nit + gi - 1) / gi;
    const size_t x_bytes = a->W_nbits == 8 ? (size_t)nit * a->M * 32 : (size_t)nit * H * a->M * 64;
    return (size_t)s * x_bytes + (size_t)s * c * (nseg * 32 * 12 + 16) + (size_t)s * a->M * c * 32 * 4 + 16;
  };
  if (s_in <= 0 || cluster <= 0) {
    // slices: fewest "waves x (iterations per warp + fixed per-warp cost)" over every split into equal slices that fit
    // the CTA shape rules and the shared-memory budget
    // (K = 3584 has 112 iterations: 7 slices of 16 fill the machine where the power-of-two choice, 2 of 56, cannot;
    //  a very wide layer must not fall back to one whole-K slice per CTA whose staged activations do not fit)
    const int64_t warp_slots = (int64_t)gl_num_sms() * 16;
    const int max_warps = a->M <= 8 ? 16 : 8;
    // CTA shape for S slices: prefer CTAs of at most 8 warps (two per SM), then up to max_warps
    auto shape_of = [&](int S, int* s_out, int* cl_out) {
      for (int lim = 8; lim <= max_warps; lim <<= 1)
        for (int cl = 1; cl <= 8; cl <<= 1)
          if (S % cl == 0 && (S / cl) * c_in <= lim && (32 * c_in) % cl == 0 && (c_in == 1 || S / cl <= 15) &&
              smem_of(S / cl, c_in, T / S) <= smem_limit) { *s_out = S / cl; *cl_out = cl; return true; }
      return false;
    };
    int S = 0;
    int64_t best_cost = 0;
    for (int cand = 1; cand <= 64; ++cand) {
      if (!slice_ok(cand)) continue;
      int s_c, cl_c;
      if (!shape_of(cand, &s_c, &cl_c)) continue;
      const int64_t waves = ((int64_t)colgroups * cand + warp_slots - 1) / warp_slots;
      const int64_t cost = waves * (T / cand + 12);
      if (S == 0 || cost < best_cost) { S = cand; best_cost = cost; }
    }
    if (S == 0) return false;
    if (!shape_of(S, &s_in, &cluster)) return false;
  }
  if (cluster < 1 || cluster > 8 || (cluster & (cluster - 1)) != 0 || s_in < 1 || s_in * c_in > (a->M <= 8 ? 16 : 8)) return false;
  if (c_in > 1 && s_in > 15) return false;                          // one named barrier per slice
  if (!slice_ok(s_in * cluster) || (32 * c_in) % cluster != 0) return false;
  const int nit = T / (s_in * cluster), nseg = (nit + gi - 1) / gi;
  const size_t smem = smem_of(s_in, c_in, nit);
  if (smem > smem_limit) return false;
  pl->warp_kernel = 1; pl->gi = gi; pl->s_in = s_in; pl->c_in = c_in; pl->cluster = cluster; pl->splitK = cluster;
  pl->MT = a->M <= 8 ? 1 : 2;
  pl->warps_n = s_in * c_in; pl->tiles = colgroups / c_in; pl->smem = smem;
  pl->slice_iters = nit; pl->max_seg = nseg;
  return true;
}

// Plan for the warp-independent kernel.  Without a cache entry the CTA shape starts from what was measured best on
// 8192 x 8192 (8 slices x 1 column group up to 4 batch rows: M = 4 runs 12.6 us that way against 13.4 us as 2 x 4 with a
// cluster of 4; 2 x 4 up to 8 rows; 1 x 8 above) and widens the column groups (which shrinks the staged activations per
// CTA) until two CTAs fit an SM's shared memory, then until one does.
static bool plan_warp(const gl_matmul_args* a, GemvPlan* pl, const char* js) {
  if (js && json_int(js, "s_in", 0) > 0) return plan_warp_with(a, pl, js, json_int(js, "c_in", 1), 200 * 1024);
  const int first = a->M <= 4 ? 1 : (a->M <= 8 ? 4 : 8);
  const size_t budgets[2] = {110 * 1024, 200 * 1024};
  for (int b = 0; b < 2; ++b)
    for (int c = first; c <= 8; c <<= 1)
      if (plan_warp_with(a, pl, js, c, budgets[b])) return true;
  // long K with many batch rows: narrower CTAs (more K slices per CTA, fewer column groups) keep the staged activations in budget
  for (int c = first >> 1; c >= 1; c >>= 1)
    if (plan_warp_with(a, pl, js, c, budgets[1])) return true;
  return false;
}

static void plan_for_uncached(const gl_matmul_args* a, GemvPlan* pl, bool force_workspace);

// The plan depends on the problem's shape and modes and on the config cache only; an eager forward asks for it two or
// three times per layer (workspace size, kernel choice, launch), so the last few are kept per thread.
static void plan_for(const gl_matmul_args* a, GemvPlan* pl, bool force_workspace = false) {
  struct Key { int M, N, K, gs, e, nbits, idt, force, dev; uint64_t gen; };
  struct Slot { Key k; GemvPlan pl; bool used; };
  static thread_local Slot slots[8] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); dev = 0; }
  const Key k = {a->M, a->N, a->K, a->group_size, a->elements_per_sample, a->W_nbits, a->input_dtype, force_workspace ? 1 : 0, dev, gl_cfg_generation()};
  const unsigned h = ((unsigned)k.M * 31u + (unsigned)k.N * 7u + (unsigned)k.K + (unsigned)k.nbits * 3u + (unsigned)k.force) & 7u;
  Slot& sl = slots[h];
  const Key& c = sl.k;
  if (sl.used && c.M == k.M && c.N == k.N && c.K == k.K && c.gs == k.gs && c.e == k.e && c.nbits == k.nbits && c.idt == k.idt &&
      c.force == k.force && c.dev == k.dev && c.gen == k.gen) { *pl = sl.pl; return; }
  plan_for_uncached(a, pl, force_workspace);
  sl.k = k; sl.pl = *pl; sl.used = true;
}

static void plan_for_uncached(const gl_matmul_args* a, GemvPlan* pl, bool force_workspace) {
  const int e = a->elements_per_sample;
  const int T = a->K / (4 * e);
  pl->MT = a->M <= 8 ? 1 : (a->M <= 16 ? 2 : 4);
  const int H = e >= 8 ? e / 8 : 1;   // (packed bytes, e = 4, never reach the general kernel; this keeps the sizes below defined)
  int warps_n = a->N <= 32 ? 1 : 2;
  int split_req = 0, cluster_req = -1;
  const char* cfg_js = nullptr;
  {
    const int idt = (a->input_dtype == GL_BF16) ? GL_FP16 : a->input_dtype;
    char sig[128];
    snprintf(sig, sizeof(sig), "(%d, %d, %d, %d, %d, %d)", gl_get_closest_m(a->M), a->N, a->K, a->group_size, e, idt * 100 + a->W_nbits);
    const char* fams[3] = {"GEMV_REVSPLITK", "GEMV_SPLITK", "GEMV"};
    for (int f = 0; f < 3; ++f) {
      const char* js = gl_cfg_get(fams[f], sig);
      if (js) {
        cfg_js = js;
        split_req = json_int(js, "split_k", 0);
        warps_n = json_int(js, "warps_n", warps_n);
        cluster_req = json_int(js, "cluster", -1);
        break;
      }
    }
  }
  pl->warp_kernel = 0; pl->s_in = pl->c_in = 1;
  // "kernel": 1 in a cache entry pins the general kernel; entries that carry split_k / warps_n tune that kernel
  const bool general_req = cfg_js && (json_int(cfg_js, "kernel", 0) == 1 || split_req > 0);
  if (!force_workspace && !general_req && plan_warp(a, pl, cfg_js)) return;
  if (warps_n < 1) warps_n = 1;
  if (warps_n > 4) warps_n = 4;
  pl->warps_n = warps_n;
  pl->tiles = (int)gl_cdiv(a->N, 32 * warps_n);
  const int per_iter_bytes = H * a->M * 4 * 16;       // x fragments per iteration of the slice
  const int max_iters_smem = (96 * 1024) / per_iter_bytes;
  int min_split = (int)gl_cdiv(T, max_iters_smem > 1 ? max_iters_smem : 1);
  int splitK;
  if (split_req > 0) splitK = split_req;
  else {
    // default: 8 slices (one thread-block cluster per column tile) when the machine is filled that way
    splitK = 8;
    while (splitK > 1 && (T / splitK < 4)) splitK >>= 1;
    const int sms = gl_num_sms();
    if ((int64_t)pl->tiles * splitK < (int64_t)sms * 2) splitK = (int)gl_cdiv((int64_t)sms * 4, pl->tiles);
  }
  if (splitK < min_split) splitK = min_split;
  if (splitK > T) splitK = T > 0 ? T : 1;
  if (splitK < 1) splitK = 1;
  pl->splitK = splitK;
  const bool pow2 = (splitK & (splitK - 1)) == 0;
  pl->cluster = (!force_workspace && cluster_req != 0 && pow2 && splitK <= 8 && splitK > 1 && (32 * warps_n) % splitK == 0) ? splitK : 1;
  pl->slice_iters = (int)gl_cdiv(T, splitK) + 1;
  const int gi = a->group_size / (4 * e);
  pl->max_seg = pl->slice_iters / (gi > 0 ? gi : 1) + 2;
  const size_t xs_bytes = (size_t)pl->slice_iters * per_iter_bytes;
  const size_t part_bytes = ((size_t)a->M * 32 * warps_n * 4 + 15) / 16 * 16;
  pl->smem = (xs_bytes > part_bytes ? xs_bytes : part_bytes) + (size_t)pl->max_seg * (8 * pl->MT * 4 + 2 * warps_n * 32 * 2) + 32;
  pl->gi = gi;
  pl->warp_kernel = 0;
}

template <int NB, typename XT, int MT>
static int launch_t(const GemvParams& p, dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  auto kern = gl_gemv_stream_kernel<NB, XT, MT, 8>;
  if (smem > 48 * 1024) GL_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  int na = 1;
  if (p.cluster > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1; attr[1].val.clusterDim.y = (unsigned)p.cluster; attr[1].val.clusterDim.z = 1;
    na = 2;
  }
  cfg.attrs = attr; cfg.numAttrs = na;
  GL_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, p));
  return GL_OK;
}
// cudaFuncSetAttribute costs about a microsecond of host time: the limit is raised once per (kernel, device) to the
// largest size any plan can ask for, not on every launch.  (All kernels here share one function-pointer type, so the
// record is keyed by the pointer value.)
static int raise_smem_limit(const void* kern) {
  static const void* seen[64][96];
  static int nseen[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); dev = -1; }
  if (dev >= 0) {
    std::lock_guard<std::mutex> lk(mu);
    for (int i = 0; i < nseen[dev]; ++i) if (seen[dev][i] == kern) return GL_OK;
  }
  GL_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  if (dev >= 0) {
    std::lock_guard<std::mutex> lk(mu);
    if (nseen[dev] < 96) seen[dev][nseen[dev]++] = kern;
  }
  return GL_OK;
}
template <typename K>
static int launch_kernel(K kern, const GemvParams& p, dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  if (smem > 48 * 1024) { if (int rc = raise_smem_limit(reinterpret_cast<const void*>(kern))) return rc; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  int na = 1;
  if (p.cluster > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1; attr[1].val.clusterDim.y = (unsigned)p.cluster; attr[1].val.clusterDim.z = 1;
    na = 2;
  }
  cfg.attrs = attr; cfg.numAttrs = na;
  GL_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, p));
  return GL_OK;
}
template <int NB, typename XT, int MT>
static int launch_warp_gi(int gi, const GemvParams& p, dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  if (gi == 1) return launch_kernel(gl_gemv_warp_kernel<NB, XT, MT, 1>, p, grid, block, smem, st);
  if (gi == 2) return launch_kernel(gl_gemv_warp_kernel<NB, XT, MT, 2>, p, grid, block, smem, st);
  if (gi == 4) return launch_kernel(gl_gemv_warp_kernel<NB, XT, MT, 4>, p, grid, block, smem, st);
  return launch_kernel(gl_gemv_warp_kernel<NB, XT, MT, 0>, p, grid, block, smem, st);
}
template <typename XT>
static int launch_warp(int NB, int MT, int gi, const GemvParams& p, dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  if (NB == 8) return MT == 1 ? launch_kernel(gl_gemv_warp_kernel<8, XT, 1, 0>, p, grid, block, smem, st)
                              : launch_kernel(gl_gemv_warp_kernel<8, XT, 2, 0>, p, grid, block, smem, st);
  if (NB == 4) return MT == 1 ? launch_warp_gi<4, XT, 1>(gi, p, grid, block, smem, st) : launch_warp_gi<4, XT, 2>(gi, p, grid, block, smem, st);
  return MT == 1 ? launch_warp_gi<2, XT, 1>(gi, p, grid, block, smem, st) : launch_warp_gi<2, XT, 2>(gi, p, grid, block, smem, st);
}

template <int NB, typename XT>
static int launch_mt(int MT, const GemvParams& p, dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  if (MT == 1) return launch_t<NB, XT, 1>(p, grid, block, smem, st);
  if (MT == 2) return launch_t<NB, XT, 2>(p, grid, block, smem, st);
  return launch_t<NB, XT, 4>(p, grid, block, smem, st);
}
template <typename XT>
static int launch_nb(int NB, int MT, const GemvParams& p, dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  if (NB == 4) return launch_mt<4, XT>(MT, p, grid, block, smem, st);
  if (NB == 2) return launch_mt<2, XT>(MT, p, grid, block, smem, st);
  return launch_mt<1, XT>(MT, p, grid, block, smem, st);
}

}  // namespace
int gl_gemv_stream_supported(const gl_matmul_args* a) {
  const int e = a->elements_per_sample;
  if (a->M < 1 || a->M > 32) return 0;
  if (!(a->W_nbits == 8 || a->W_nbits == 4 || a->W_nbits == 2 || a->W_nbits == 1)) return 0;
  if (a->w_dtype != GL_INT32 || e != 32 / a->W_nbits) return 0;
  if (!(a->x_dtype == GL_BF16 || a->x_dtype == GL_FP16) || a->input_dtype != a->x_dtype) return 0;
  if (a->w_stride_n != 1 || a->w_stride_k != a->N) return 0;
  if (a->N % 4 != 0 || a->K % (4 * e) != 0) return 0;
  if (a->W_group_mode < 0 || a->W_group_mode > 4) return 0;
  if (!(a->channel_scale_mode == 0 || a->channel_scale_mode == 1)) return 0;
  if (a->group_size % (4 * e) != 0 || a->K % a->group_size != 0) return 0;
  const bool need_s = a->W_group_mode >= 2 || a->channel_scale_mode == 1;
  const bool need_z = a->W_group_mode == 1 || a->W_group_mode >= 3;
  if (need_s && (a->scales == nullptr || a->meta_dtype != a->x_dtype)) return 0;
  if (a->W_group_mode >= 2 && (a->s_stride_n != 1 || a->s_stride_g != a->N)) return 0;
  if (need_z) {
    if (a->zeros == nullptr) return 0;
    if (a->zero_is_scalar) { if (a->zeros_dtype != GL_INT32) return 0; }
    else if (a->zeros_dtype != a->x_dtype) return 0;
  }
  if (a->channel_scale_mode == 1 && a->W_group_mode >= 2) return 0;
  if (!(a->out_dtype == GL_BF16 || a->out_dtype == GL_FP16 || a->out_dtype == GL_FP32)) return 0;
  if (((uintptr_t)a->w & 15) || ((uintptr_t)a->x & 15) || ((uintptr_t)a->out & 15)) return 0;
  if (need_s && ((uintptr_t)a->scales & 7)) return 0;
  if (need_z && !a->zero_is_scalar && ((uintptr_t)a->zeros & 7)) return 0;
  if (a->bias && ((uintptr_t)a->bias & 15)) return 0;
  GemvPlan pl;
  plan_for(a, &pl);
  if (a->W_nbits == 8 && !pl.warp_kernel) return 0;               // packed bytes: only the warp-independent kernel
  if (pl.tiles > kMaxTiles) return 0;
  if (pl.smem > 200 * 1024) return 0;
  return 1;
}

uint64_t gl_matmul_counter_bytes(void) { return (uint64_t)kMaxTiles * sizeof(unsigned int) + kStatusBytes; }
extern "C" uint64_t gl_matmul_status_offset(void) { return gl_matmul_counter_bytes() - 256; }

// 17 to 32 batch rows: two launches of the warp-independent kernel (rows 0..15, then the rest).  The packed weights of
// one layer are a fraction of the 126 MB L2, so the second launch reads them from there; together they take about half
// the time of the 128-row tensor-core tile (which pads the batch and dequantises through shared memory) at these sizes.
static bool split_rows_plans(const gl_matmul_args* a, gl_matmul_args* lo, gl_matmul_args* hi, GemvPlan* pl_lo, GemvPlan* pl_hi) {
  if (a->M <= 16 || a->M > 32) return false;
  *lo = *a; *hi = *a;
  lo->M = 16; hi->M = a->M - 16;
  hi->x = reinterpret_cast<const char*>(a->x) + (size_t)16 * a->K * gl_dtype_size(a->x_dtype);
  hi->out = reinterpret_cast<char*>(a->out) + (size_t)16 * a->N * gl_dtype_size(a->out_dtype);
  plan_for(lo, pl_lo);
  plan_for(hi, pl_hi);
  return pl_lo->warp_kernel && pl_hi->warp_kernel;
}

int gl_gemv_split_rows_ok(const gl_matmul_args* a) {
  gl_matmul_args lo, hi;
  GemvPlan p1, p2;
  return split_rows_plans(a, &lo, &hi, &p1, &p2) ? 1 : 0;
}

uint64_t gl_gemv_stream_workspace(const gl_matmul_args* a) {
  GemvPlan pl;
  {
    gl_matmul_args lo, hi;
    GemvPlan pl_hi;
    if (split_rows_plans(a, &lo, &hi, &pl, &pl_hi)) return gl_matmul_counter_bytes();   // both launches reduce inside CTAs / clusters
  }
  plan_for(a, &pl);
  return gl_matmul_counter_bytes() + ((pl.splitK > 1 && pl.cluster == 1) ? (uint64_t)pl.splitK * a->M * a->N * sizeof(float) : 0);
}


static uint64_t workspace_for_plan(const gl_matmul_args* a, const GemvPlan& pl) {
  return gl_matmul_counter_bytes() + ((pl.splitK > 1 && pl.cluster == 1) ? (uint64_t)pl.splitK * a->M * a->N * sizeof(float) : 0);
}

#ifdef GL_GEMV_TRACE
// profiling build only: a device buffer of 64 x 8192 x 8 stamps that successive launches fill round-robin
static unsigned long long* g_gemv_trace = nullptr;
static unsigned int g_gemv_trace_launch = 0;
extern "C" __attribute__((visibility("default"))) void gl_debug_gemv_trace(unsigned long long* buf) { g_gemv_trace = buf; g_gemv_trace_launch = 0; }
#endif

// launches the streaming kernel with `workspace` as its scratch (counters | status | partial sums)
static int gemv_launch_impl(const gl_matmul_args* a, cudaStream_t st, const GemvPlan& pl, void* workspace, uint64_t workspace_bytes) {
  const uint64_t need = workspace_for_plan(a, pl);
  if (workspace == nullptr || workspace_bytes < need)
    GL_FAIL(GL_E_WORKSPACE, "gl_matmul: workspace of %llu bytes needed, %llu given",
            (unsigned long long)need, (unsigned long long)workspace_bytes);
  if ((uintptr_t)workspace & 15) GL_FAIL(GL_E_INVALID, "gl_matmul: workspace must be 16-byte aligned");
  const int e = a->elements_per_sample;
  GemvParams p;
  memset(&p, 0, sizeof(p));
  p.x = a->x; p.w = reinterpret_cast<const int32_t*>(a->w); p.scales = a->scales; p.zeros = a->zeros; p.bias = a->bias;
  p.out = a->out;
  p.counters = reinterpret_cast<unsigned int*>(workspace);
  p.status = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + (size_t)kMaxTiles * sizeof(unsigned int));
  p.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + gl_matmul_counter_bytes());
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.T = a->K / (4 * e);
  p.gi = a->group_size / (4 * e);
  p.splitK = pl.splitK;
  p.cluster = pl.cluster;
  p.W_group_mode = a->W_group_mode; p.channel_scale_mode = a->channel_scale_mode; p.zero_is_scalar = a->zero_is_scalar;
  p.out_dtype = a->out_dtype;
  p.max_slice_iters = pl.slice_iters;
  p.max_seg = pl.max_seg;
  p.s_in = pl.s_in; p.c_in = pl.c_in;
#ifdef GL_GEMV_TRACE
  p.trace = g_gemv_trace ? g_gemv_trace + (size_t)(g_gemv_trace_launch++ % 64) * 8192 * 8 : nullptr;   // one 8192-warp record per launch
#endif
  dim3 grid(pl.tiles, pl.splitK), block(32 * pl.warps_n);
  if (pl.warp_kernel) {
    if (a->x_dtype == GL_BF16) return launch_warp<__nv_bfloat16>(a->W_nbits, pl.MT, pl.gi, p, grid, block, pl.smem, st);
    return launch_warp<__half>(a->W_nbits, pl.MT, pl.gi, p, grid, block, pl.smem, st);
  }
  if (a->W_nbits == 8) GL_FAIL(GL_E_UNSUPPORTED, "gl_matmul: packed 8-bit weights have no general streaming kernel for this shape");
  if (a->x_dtype == GL_BF16) return launch_nb<__nv_bfloat16>(a->W_nbits, pl.MT, p, grid, block, pl.smem, st);
  return launch_nb<__half>(a->W_nbits, pl.MT, p, grid, block, pl.smem, st);
}

const char* gl_gemv_stream_kernel_name(const gl_matmul_args* a) {
  GemvPlan pl;
  if (gl_gemv_split_rows_ok(a)) return "gl_gemv_warp_kernel";
  plan_for(a, &pl);
  return pl.warp_kernel ? "gl_gemv_warp_kernel" : "gl_gemv_stream_kernel";
}

int gl_gemv_stream_launch(const gl_matmul_args* a, cudaStream_t st) {
  GemvPlan pl;
  {
    gl_matmul_args lo, hi;
    GemvPlan pl_hi;
    if (split_rows_plans(a, &lo, &hi, &pl, &pl_hi)) {
      if (int rc = gemv_launch_impl(&lo, st, pl, a->workspace, a->workspace_bytes)) return rc;
      return gemv_launch_impl(&hi, st, pl_hi, a->workspace, a->workspace_bytes);
    }
  }
  plan_for(a, &pl);
  return gemv_launch_impl(a, st, pl, a->workspace, a->workspace_bytes);
}

// ---- gl_matmul_noalloc: the split-K streaming kernel on scratch that lives inside the library -------------
// For callers that must not (or cannot) allocate device memory around the call: plug-ins that only receive
// tensors from a host framework whose allocator they may not touch, code inside a memory-pool-managed serving
// loop where a cudaMalloc would synchronise the device, and hosts that bind the C ABI from a language runtime without a device allocator of their own.
//
// The scratch (arrival counters, status word, fp32 split-K partial sums) is this file-scope device array.  Every
// GPU that loads the library carries GL_NOALLOC_SCRATCH_BYTES of it until the process exits.  The name
// `g_noalloc_scratch` is only a host-side handle here: its device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and that pointer is what the kernel receives.
static __device__ __align__(256) unsigned char g_noalloc_scratch[GL_NOALLOC_SCRATCH_BYTES];

static int noalloc_scratch_ptr(void** out) {
  static void* ptrs[64];
  static std::mutex mu;
  int dev = 0;
  GL_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) GL_FAIL(GL_E_INVALID, "gl_matmul_noalloc: device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);   // address on the current device
    if (e != cudaSuccess || p == nullptr) {
      gl_set_error("gl_matmul_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return GL_E_CUDA;
    }
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return GL_OK;
}

extern "C" int gl_matmul_noalloc(const gl_matmul_args* a, void* stream) {
  if (int rc = gl_validate_matmul_args(a)) return rc;
  if (a->M == 0) return GL_OK;
  // packed 8-bit words only run on the warp-independent kernel, which has no split-K-through-scratch form
  if (gl_is_mx(a->input_dtype) || a->W_nbits == 8 || !gl_gemv_stream_supported(a))
    GL_FAIL(GL_E_UNSUPPORTED, "gl_matmul_noalloc: only the streaming decode kernel (packed 4/2/1-bit weights, fp16/bf16 "
                              "activations, M <= 32) has a built-in-scratch variant");
  GemvPlan pl;
  plan_for(a, &pl, /*force_workspace=*/true);
  // the limits are checked on the plan that is launched, before anything is enqueued
  if (pl.tiles > kMaxTiles || pl.smem > 200 * 1024)
    GL_FAIL(GL_E_UNSUPPORTED, "gl_matmul_noalloc: this shape (M=%d N=%d K=%d) exceeds the streaming kernel's tile or shared-memory limits",
            a->M, a->N, a->K);
  const uint64_t need = workspace_for_plan(a, pl);
  if (need > (uint64_t)GL_NOALLOC_SCRATCH_BYTES)
    GL_FAIL(GL_E_WORKSPACE, "gl_matmul_noalloc: this problem (M=%d N=%d, %d K slices) needs %llu bytes of scratch, the built-in "
                            "array holds %llu; use gl_matmul with a caller-provided workspace",
            a->M, a->N, pl.splitK, (unsigned long long)need, (unsigned long long)GL_NOALLOC_SCRATCH_BYTES);
  void* scratch = nullptr;
  if (int rc = noalloc_scratch_ptr(&scratch)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // the array keeps whatever the previous call left: the counters and the status word must start at zero
  GL_CUDA_CHECK(cudaMemsetAsync(scratch, 0, (size_t)gl_matmul_counter_bytes(), st));
  return gemv_launch_impl(a, st, pl, scratch, (uint64_t)GL_NOALLOC_SCRATCH_BYTES);
}
