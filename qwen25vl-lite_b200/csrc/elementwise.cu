// Embedding gather, fused residual-add + RMSNorm, SiLU-mul.
//
// Formulas (reference: zhangjianbang-nb/qwen25vl-lite):
//   embedding   x[n,:] = E[token[n],:]                          src/qwen25vl_lite/text.py:213
//   RMSNorm     h = x * rsqrt(mean(x^2) + eps) * w              src/qwen25vl_lite/layers.py:27-31
//   SwiGLU act  f = silu(g) * u, silu(z) = z / (1 + exp(-z))    src/qwen25vl_lite/text.py:66
// The residual stream x is float in both dtypes; the norm fuses the pending residual update
// (x += delta) so that a block's output is read once.
#include "common.cuh"

template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ x, int hidden, int vocab) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // the host validates ids; never read outside
  const T* src = table + (size_t)id * hidden;
  float* dst = x + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32(src[c]);
}

// Four consecutive values as floats, and back (bf16: 8 bytes, float: 16 bytes at a time).
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const unsigned*>(&a);
  raw.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// x[row] += delta[row] (if delta), then out[r] = rmsnorm(x[row]) * w.
// rows == nullptr: row = r, x is updated in place.  rows != nullptr: row = rows[r], x is left
// untouched (used for the final norm, which only the wanted positions need).
// VEC: hidden is a multiple of 4 and every row starts on a 16-byte boundary, so a thread moves four
// values at a time.  The sum of squares is taken thread by thread, then lanes, then warps, in a fixed
// order that depends on hidden alone.
template <typename T, bool EXACT, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                   const float* __restrict__ w, float eps, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float row_cache[];  // hidden floats + 32 scratch
  float* scratch = row_cache + hidden;
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* xr = x + (size_t)row * hidden;
  const T* dr = delta ? delta + (size_t)row * hidden : nullptr;
  T* o = out + (size_t)r * hidden;
  float ss = 0.f;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + c);
      if (dr) {
        const float4 d = load4<T>(dr + c);
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        if (!rows) *reinterpret_cast<float4*>(xr + c) = v;
      }
      *reinterpret_cast<float4*>(row_cache + c) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float v = xr[c];
      if (dr) {
        v += to_f32(dr[c]);
        if (!rows) xr[c] = v;
      }
      row_cache[c] = v;
      ss += v * v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = EXACT ? 1.0f / sqrtf(total / (float)hidden + eps) : rsqrtf(total / (float)hidden + eps);
  if (VEC) {
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row_cache + c), ww = *reinterpret_cast<const float4*>(w + c);
      store4<T>(o + c, make_float4(v.x * inv * ww.x, v.y * inv * ww.y, v.z * inv * ww.z, v.w * inv * ww.w));
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = from_f32<T>(row_cache[c] * inv * w[c]);
  }
}

// gu is [n, 2*inter].  paired == 0: gate in the first half of a row, up in the second.
// paired == 1: groups of 16 columns hold 8 gate features followed by their 8 up features (the
// layout the skinny GEMM's SwiGLU epilogue wants of the weight rows).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int n, int inter, int paired) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n * inter;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / inter, c = i % inter;
    const size_t gc = paired ? (c >> 3) * 16 + (c & 7) : c;
    const size_t uc = paired ? gc + 8 : inter + c;
    const float g = to_f32(gu[row * 2 * inter + gc]);
    const float u = to_f32(gu[row * 2 * inter + uc]);
    out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

template <typename T>
static int embed_gather(const void* table, const int* ids, float* x, int n, int hidden, int vocab, void* stream) {
  if (n <= 0) return 0;
  launch(embed_gather_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, (const T*)table, ids, x, hidden, vocab);
  return launch_status();
}

template <typename T, bool EXACT>
static int add_rmsnorm(float* x, const void* delta, const float* w, float eps, void* out, const int* rows,
                       int n_out, int hidden, void* stream) {
  if (n_out <= 0) return 0;
  const size_t smem = (size_t)(hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T, EXACT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(add_rmsnorm_kernel<T, EXACT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = hidden >= 1024 ? 256 : 128;
  const bool vec = hidden % 4 == 0 && !(((uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15);
  if (vec) launch(add_rmsnorm_kernel<T, EXACT, true>, dim3(n_out), dim3(threads), smem, (cudaStream_t)stream, x, (const T*)delta, w, eps, (T*)out, rows, hidden);
  else launch(add_rmsnorm_kernel<T, EXACT, false>, dim3(n_out), dim3(threads), smem, (cudaStream_t)stream, x, (const T*)delta, w, eps, (T*)out, rows, hidden);
  return launch_status();
}

template <typename T>
static int silu_mul(const void* gu, void* out, int n, int inter, int paired, void* stream) {
  if (n <= 0) return 0;
  const size_t total = (size_t)n * inter;
  size_t blocks = (total + 255) / 256;
  const size_t most = (size_t)(device_sm_count() > 0 ? device_sm_count() : 148) * 16;
  if (blocks > most) blocks = most;
  launch(silu_mul_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)gu, (T*)out, n, inter, paired);
  return launch_status();
}

Q25_EXPORT int q25_embed_gather_f32(const void* t, const int* ids, float* x, int n, int h, int v, void* s) { return embed_gather<float>(t, ids, x, n, h, v, s); }
Q25_EXPORT int q25_embed_gather_bf16(const void* t, const int* ids, float* x, int n, int h, int v, void* s) { return embed_gather<bf16>(t, ids, x, n, h, v, s); }
Q25_EXPORT int q25_add_rmsnorm_f32(float* x, const void* d, const float* w, float eps, void* o, const int* rows, int n, int h, void* s) { return add_rmsnorm<float, true>(x, d, w, eps, o, rows, n, h, s); }
Q25_EXPORT int q25_add_rmsnorm_bf16(float* x, const void* d, const float* w, float eps, void* o, const int* rows, int n, int h, void* s) { return add_rmsnorm<bf16, false>(x, d, w, eps, o, rows, n, h, s); }
Q25_EXPORT int q25_silu_mul_f32(const void* gu, void* o, int n, int inter, int paired, void* s) { return silu_mul<float>(gu, o, n, inter, paired, s); }
Q25_EXPORT int q25_silu_mul_bf16(const void* gu, void* o, int n, int inter, int paired, void* s) { return silu_mul<bf16>(gu, o, n, inter, paired, s); }

// Streaming multiprocessors of the current device (0 if it cannot be read).
Q25_EXPORT int q25_sm_count(void) { return device_sm_count(); }
