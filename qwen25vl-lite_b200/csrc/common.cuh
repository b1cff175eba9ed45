// Shared device helpers for the sm_100a kernels of this engine.
//
// Conventions used by every kernel file:
//   * activations and weights come as T = float (the true 32-bit path) or __nv_bfloat16 (the
//     serving path); statistics, softmax state, angles and the residual stream are float in both;
//   * every exported function is `extern "C" int q25_<name>_<f32|bf16>(..., void* stream)` and
//     returns the cudaError_t of its launch (0 = success), so Python can call it through ctypes
//     with raw device pointers and the stream it is recording or capturing on;
//   * no kernel waits on another kernel: everything is stream-ordered.  Waits inside a kernel (on
//     an mbarrier, or on the grid barrier of gemm_chain.cu) are bounded and report through a flag.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

#define Q25_EXPORT extern "C" __attribute__((visibility("default")))

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a thread block in a fixed order (lanes by butterfly, then warps in index order),
// so the result for a row never depends on what else is in the batch.  `scratch` holds 32
// floats.  Every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}

// ---- shared memory addresses, mbarriers, bulk copies -------------------------------------------------
// Thin wrappers of the PTX that every kernel with asynchronous copies uses.  A wait on an mbarrier
// polls at most MBAR_WAIT_LIMIT times and says whether the phase completed: the caller records an
// error code and runs on to its end.  A parity wait cannot tell "not yet" from "two phases on" (nor
// from "a phase behind"), so a waiter must stay within one phase of its barrier.
#define MBAR_WAIT_LIMIT (1 << 22)

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
  for (int i = 0; i < MBAR_WAIT_LIMIT; ++i) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
// One contiguous piece of global memory into shared memory (both 16-byte aligned, a multiple of 16
// bytes); the bytes are counted on the mbarrier.
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// The same for data that is read once and never again (a stream of weights): the cache policy asks
// L2 to give these lines up first, so that what a step reads again and again (activations, partial
// sums, the rows of the cache just written) is not pushed out by gigabytes that pass through.
__device__ __forceinline__ unsigned long long l2_evict_first() {
  unsigned long long policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void bulk_copy_once(void* dst, const void* src, unsigned bytes, unsigned long long* bar,
                                               unsigned long long policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}

// ---- programmatic dependent launch -----------------------------------------------------------------
// Every kernel of the engine is launched with the attribute that lets it be scheduled while the
// kernel before it in the stream is still running; it calls pdl_trigger() at its top (the next one
// may be scheduled as soon as every CTA of this one has started) and pdl_wait() before it touches
// anything an earlier kernel wrote or still reads.  pdl_wait() returns when all earlier kernels have
// finished and their writes are visible, so the results are those of plain stream order; what is
// gained is the launch latency and whatever a kernel does before its wait (the weight-streaming
// GEMM starts fetching weights).  Before pdl_wait() a kernel may read only what no kernel ever
// writes: weights, constant tables, and the step's own lists, lengths and block tables, which come
// with the step's copy from the host, ahead of its first kernel.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static thread_local cudaError_t q25_launch_error = cudaSuccess;

// cluster: CTAs per thread-block cluster along x (1: none); the grid is then a multiple of it.
template <typename... KArgs, typename... Args>
static inline void launch_clusters(int cluster, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                   Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = (unsigned)cluster;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster > 1 ? 2 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  if (e != cudaSuccess && q25_launch_error == cudaSuccess) q25_launch_error = e;
}
template <typename... KArgs, typename... Args>
static inline void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  launch_clusters(1, kernel, grid, block, smem, stream, args...);
}

// ---- thread-block clusters --------------------------------------------------------------------------
// All threads of all CTAs of the cluster meet; what they wrote to shared memory before is visible to
// the others' ld.shared::cluster after.  A hardware barrier like __syncthreads: every thread must
// come, so it stands only where all waits before it are bounded.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The address, in the cluster's shared window, of this CTA's shared address in the CTA of that rank.
__device__ __forceinline__ unsigned cluster_map(unsigned smem_addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

// Streaming multiprocessors of the current device (asked once per device): persistent grids and
// split heuristics are sized from it.  148 on the B200 the kernels were tuned on.
static inline int device_sm_count() {
  static int known[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (known[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    known[dev] = n;
  }
  return known[dev];
}

// Error of the launches since the last call (0 = none).
static inline int launch_status() {
  cudaError_t e = q25_launch_error;
  q25_launch_error = cudaSuccess;
  if (e == cudaSuccess) e = cudaGetLastError();
  return (int)e;
}
