// Tensor-parallel plumbing for the row-parallel layers: a one-shot all-reduce over peer memory (NVLink / NVSwitch)
// and the element-wise glue of a decoder's MLP.
//
// The reference has no multi-GPU code; under vLLM the host shards the weights and calls
// tensor_model_parallel_all_reduce after the row-parallel layers (gemlite/vllm/onthefly.py:83-99).  For the decode
// sizes of this path ([M, 8192] with M <= 64, i.e. 16 KB .. 2 MB) an NCCL ring is launch- and latency-bound, so the
// reduction here is a single kernel:
//   push   every CTA copies its chunk of the local partial result into the receive area of every rank
//          (plain 16-byte stores to peer memory: one NVLink crossing, no read round trip),
//   signal after a CTA-wide barrier, lane r publishes the epoch to rank r with a system-scope release store,
//   wait   the CTA polls its own (local) flags until all ranks have published the epoch (bounded: on time-out the
//          status word is set and the kernel returns),
//   sum    the CTA adds the `world` received chunks in rank order (the same order on every rank, so all ranks hold
//          bit-identical results) and writes the output.
// Synchronisation is per chunk: CTA c of every rank only depends on CTA c of the other ranks, so nothing spans the
// grid.  Two receive areas alternate with the epoch, which lives on the device (CUDA-graph replays advance it).
// No TMA is involved and no library kernel ever sees a peer pointer.
#include "gl_common.cuh"
#include <string.h>

namespace {

constexpr int kMaxRanks = GL_TP_MAX_RANKS;
constexpr int kMaxCtas = GL_TP_MAX_CTAS;
constexpr int kCtaThreads = 128;
constexpr unsigned long long kDefaultWaitCycles = 4000000000ull;

// control block at the head of every rank's buffer
struct TpCtrl {
  unsigned int epoch;          // all-reduces completed on this rank
  unsigned int done;           // CTAs of the running all-reduce that have finished
  int status;                  // 0, or the code of the first wait that gave up
  unsigned int pad[61];
  unsigned int flags[kMaxRanks * kMaxCtas];   // flags[src * kMaxCtas + cta] = epoch published by rank `src` for chunk `cta`
};

struct TpParams {
  unsigned char* peers[kMaxRanks];   // every rank's buffer as mapped into this process (peers[rank] = the local one)
  const void* in; void* out;
  long long count;                   // elements
  int in_dtype, out_dtype;
  int rank, world;
  unsigned long long slot_bytes;
  unsigned long long wait_cycles;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ size_t data_offset() { return (sizeof(TpCtrl) + 255) / 256 * 256; }

// 16 bytes of the input dtype -> fp32 accumulators (8 values for 16-bit types, 4 for fp32)
template <int DT>
__device__ __forceinline__ void accumulate16(const uint4& u, float (&acc)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  if constexpr (DT == GL_FP32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] += __uint_as_float(w[i]);
  } else if constexpr (DT == GL_BF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { acc[2 * i] += __uint_as_float(w[i] << 16); acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u); }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += __half2float(__ushort_as_half((unsigned short)(w[i] & 0xffffu)));
      acc[2 * i + 1] += __half2float(__ushort_as_half((unsigned short)(w[i] >> 16)));
    }
  }
}

template <int DT>
__global__ void __launch_bounds__(kCtaThreads) gl_tp_allreduce_kernel(const TpParams p) {
  constexpr int EPV = (DT == GL_FP32) ? 4 : 8;          // elements per 16-byte vector
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");    // the partial result comes from the previous kernel of the stream
  TpCtrl* ctrl = reinterpret_cast<TpCtrl*>(p.peers[p.rank]);
  __shared__ unsigned int s_epoch;
  __shared__ int s_fail;
  if (threadIdx.x == 0) { s_epoch = *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch); s_fail = 0; }
  __syncthreads();
  const unsigned int epoch = s_epoch, want = epoch + 1u;
  const size_t slot_off = data_offset() + (size_t)(epoch & 1u) * p.world * p.slot_bytes;
  const long long nvec = (p.count + EPV - 1) / EPV;      // count is a multiple of EPV (checked by the host)
  const long long per_cta = (nvec + gridDim.x - 1) / gridDim.x;
  const long long v0 = (long long)blockIdx.x * per_cta, v1 = min(nvec, v0 + per_cta);

  // ---- push this CTA's chunk into the receive area [rank] of every rank ----
  const uint4* src = reinterpret_cast<const uint4*>(p.in);
  for (long long v = v0 + threadIdx.x; v < v1; v += kCtaThreads) {
    const uint4 val = src[v];
    for (int r = 0; r < p.world; ++r)
      reinterpret_cast<uint4*>(p.peers[r] + slot_off + (size_t)p.rank * p.slot_bytes)[v] = val;
  }
  __syncthreads();
  if (threadIdx.x < p.world) {
    __threadfence_system();
    TpCtrl* peer = reinterpret_cast<TpCtrl*>(p.peers[threadIdx.x]);
    st_release_sys(&peer->flags[p.rank * kMaxCtas + blockIdx.x], want);
  }
  // ---- wait until every rank has published this chunk (bounded) ----
  if (threadIdx.x < p.world) {
    const unsigned int* f = &ctrl->flags[threadIdx.x * kMaxCtas + blockIdx.x];
    const long long t0 = clock64();
    unsigned int spins = 0;
    // epochs only grow; a flag that is ahead belongs to a later all-reduce of a faster rank and also proves arrival
    while ((int)(ld_acquire_sys(f) - want) < 0) {
      if ((++spins & 31u) == 0u && (unsigned long long)(clock64() - t0) > p.wait_cycles) {
        atomicCAS(&ctrl->status, 0, 100 + (int)threadIdx.x);
        s_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_fail) {
    // ---- sum the received chunks in rank order ----
    const unsigned char* mine = p.peers[p.rank] + slot_off;
    for (long long v = v0 + threadIdx.x; v < v1; v += kCtaThreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < p.world; ++r)
        accumulate16<DT>(ld_cg_v4(reinterpret_cast<const uint4*>(mine + (size_t)r * p.slot_bytes) + v), acc);
      const long long e0 = v * EPV;
      if (p.out_dtype == DT && DT != GL_FP32) {           // same 16-bit dtype in and out: one 16-byte store
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (DT == GL_BF16) { __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]); w[i] = *reinterpret_cast<uint32_t*>(&h); }
          else { __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]); w[i] = *reinterpret_cast<uint32_t*>(&h); }
        }
        reinterpret_cast<uint4*>(p.out)[v] = make_uint4(w[0], w[1], w[2], w[3]);
      } else {
#pragma unroll
        for (int i = 0; i < EPV; ++i) gl_store_out(p.out, e0 + i, acc[i], p.out_dtype);
      }
    }
  }
  // ---- the CTA that finishes last advances the epoch ----
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(&ctrl->done, 1u);
    if (prev == gridDim.x - 1) {
      ctrl->done = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch) = want;
    }
  }
}

// act[m, j] = silu(gu[m, j]) * gu[m, inter + j]   (gate and up projections fused in one column-parallel layer)
template <typename T>
__global__ void gl_silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ act, int M, int inter) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long total = (long long)M * inter;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i / inter), j = (int)(i - (long long)m * inter);
    const float g = (float)gu[(size_t)m * 2 * inter + j], u = (float)gu[(size_t)m * 2 * inter + inter + j];
    // silu in the activation dtype, then the product rounded once more: the roundings of the two torch ops it replaces
    const T s = (T)(g / (1.f + __expf(-g)));
    act[i] = (T)((float)s * u);
  }
}

template <typename K, typename... A>
int launch_pdl(K kern, dim3 grid, dim3 block, cudaStream_t st, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  GL_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, args...));
  return GL_OK;
}

}  // namespace

extern "C" uint64_t gl_tp_buffer_bytes(int32_t world, uint64_t slot_bytes) {
  return (sizeof(TpCtrl) + 255) / 256 * 256 + 2ull * (uint64_t)world * ((slot_bytes + 255) / 256 * 256);
}

extern "C" int gl_tp_buffer_create(uint64_t bytes, void** ptr, uint8_t* handle) {
  if (ptr == nullptr || handle == nullptr || bytes == 0) GL_FAIL(GL_E_INVALID, "gl_tp_buffer_create: null argument or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == GL_TP_HANDLE_BYTES, "IPC handle size");
  void* p = nullptr;
  GL_CUDA_CHECK(cudaMalloc(&p, bytes));
  GL_CUDA_CHECK(cudaMemset(p, 0, bytes));
  GL_CUDA_CHECK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    gl_set_error("gl_tp_buffer_create: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    return GL_E_CUDA;
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return GL_OK;
}

extern "C" int gl_tp_buffer_open(const uint8_t* handle, void** ptr) {
  if (ptr == nullptr || handle == nullptr) GL_FAIL(GL_E_INVALID, "gl_tp_buffer_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  GL_CUDA_CHECK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return GL_OK;
}

extern "C" int gl_tp_buffer_close(void* ptr) {
  if (ptr != nullptr) GL_CUDA_CHECK(cudaIpcCloseMemHandle(ptr));
  return GL_OK;
}

extern "C" int gl_tp_buffer_destroy(void* ptr) {
  if (ptr != nullptr) GL_CUDA_CHECK(cudaFree(ptr));
  return GL_OK;
}

extern "C" int gl_tp_status(const gl_tp_comm* c, int32_t* status, uint32_t* epoch) {
  if (c == nullptr || c->buffers[c->rank] == nullptr) GL_FAIL(GL_E_INVALID, "gl_tp_status: null communicator");
  TpCtrl h;
  GL_CUDA_CHECK(cudaMemcpy(&h, c->buffers[c->rank], 256, cudaMemcpyDeviceToHost));
  if (status) *status = h.status;
  if (epoch) *epoch = h.epoch;
  return GL_OK;
}

extern "C" int gl_tp_allreduce(const gl_tp_comm* c, const void* in, void* out, int64_t count, int32_t in_dtype,
                               int32_t out_dtype, void* stream) {
  if (c == nullptr || in == nullptr || out == nullptr) GL_FAIL(GL_E_INVALID, "gl_tp_allreduce: null argument");
  if (c->world < 1 || c->world > kMaxRanks || c->rank < 0 || c->rank >= c->world)
    GL_FAIL(GL_E_INVALID, "gl_tp_allreduce: bad rank %d / world %d (at most %d ranks)", c->rank, c->world, kMaxRanks);
  for (int r = 0; r < c->world; ++r)
    if (c->buffers[r] == nullptr) GL_FAIL(GL_E_INVALID, "gl_tp_allreduce: buffer of rank %d is not mapped", r);
  if (!(in_dtype == GL_BF16 || in_dtype == GL_FP16 || in_dtype == GL_FP32)) GL_FAIL(GL_E_INVALID, "gl_tp_allreduce: input dtype %d", in_dtype);
  if (!(out_dtype == GL_BF16 || out_dtype == GL_FP16 || out_dtype == GL_FP32)) GL_FAIL(GL_E_INVALID, "gl_tp_allreduce: output dtype %d", out_dtype);
  if (count <= 0) return GL_OK;
  const int epv = in_dtype == GL_FP32 ? 4 : 8;
  if (count % epv != 0 || ((uintptr_t)in & 15)) GL_FAIL(GL_E_INVALID, "gl_tp_allreduce: the input must be 16-byte aligned and a multiple of 16 bytes long");
  const uint64_t bytes = (uint64_t)count * gl_dtype_size(in_dtype);
  const uint64_t slot = (c->slot_bytes + 255) / 256 * 256;
  if (bytes > c->slot_bytes) GL_FAIL(GL_E_WORKSPACE, "gl_tp_allreduce: %llu bytes do not fit the %llu-byte receive slots", (unsigned long long)bytes, (unsigned long long)c->slot_bytes);
  TpParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < c->world; ++r) p.peers[r] = reinterpret_cast<unsigned char*>(c->buffers[r]);
  p.in = in; p.out = out; p.count = count; p.in_dtype = in_dtype; p.out_dtype = out_dtype;
  p.rank = c->rank; p.world = c->world; p.slot_bytes = slot;
  p.wait_cycles = c->wait_cycles ? c->wait_cycles : kDefaultWaitCycles;
  // 2 KB of input per CTA pass; all ranks must use the same grid (it only depends on the byte count)
  const long long nvec = bytes / 16;
  long long ctas = (nvec + kCtaThreads - 1) / kCtaThreads;
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (ctas < 1) ctas = 1;
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype == GL_BF16) return launch_pdl(gl_tp_allreduce_kernel<GL_BF16>, dim3((unsigned)ctas), dim3(kCtaThreads), st, p);
  if (in_dtype == GL_FP16) return launch_pdl(gl_tp_allreduce_kernel<GL_FP16>, dim3((unsigned)ctas), dim3(kCtaThreads), st, p);
  return launch_pdl(gl_tp_allreduce_kernel<GL_FP32>, dim3((unsigned)ctas), dim3(kCtaThreads), st, p);
}

extern "C" int gl_silu_mul(const void* gate_up, void* out, int32_t M, int32_t inter, int32_t dtype, void* stream) {
  if (gate_up == nullptr || out == nullptr || M < 0 || inter <= 0) GL_FAIL(GL_E_INVALID, "gl_silu_mul: bad argument");
  if (M == 0) return GL_OK;
  const long long total = (long long)M * inter;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == GL_BF16)
    return launch_pdl(gl_silu_mul_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), st, reinterpret_cast<const __nv_bfloat16*>(gate_up),
                      reinterpret_cast<__nv_bfloat16*>(out), (int)M, (int)inter);
  if (dtype == GL_FP16)
    return launch_pdl(gl_silu_mul_kernel<__half>, dim3((unsigned)blocks), dim3(256), st, reinterpret_cast<const __half*>(gate_up),
                      reinterpret_cast<__half*>(out), (int)M, (int)inter);
  GL_FAIL(GL_E_INVALID, "gl_silu_mul: dtype %d (fp16 / bf16 only)", dtype);
}
