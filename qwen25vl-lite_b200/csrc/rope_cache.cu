// Multimodal rotary position encoding applied to q and k, fused with the write of k and v into
// the paged cache.
//
// Formulas (reference: zhangjianbang-nb/qwen25vl-lite):
//   angle[j] = pos[axis(j)] * inv_freq[j], j in [0, D/2), computed in float
//                                                   src/qwen25vl_lite/rope.py:48-68
//   axis(j): the section list [s0,s1,s2] is repeated over the D table channels and its chunks
//            take axes 0,1,2,0,1,2, so channels j and j + D/2 share axis(j)
//                                                   src/qwen25vl_lite/rope.py:71-96
//   y[j]       = x[j] cos - x[j+D/2] sin
//   y[j + D/2] = x[j+D/2] cos + x[j] sin            (x*cos + rotate_half(x)*sin, rope.py:36-40,96)
//   the step's k (rotated) and v are written at slot = page * page_size + offset before the
//   attention reads them                            src/qwen25vl_lite/text.py:125-126
//
// qkv is [n, (nq + 2 nkv) * D]: q heads, then k heads, then v heads.  q is rotated in place.
// The pages of one cache layer are K: [num_pages, nkv, page_size, D] and V the same.
#include "common.cuh"

// Eight consecutive values as floats, and back (bf16: 16 bytes, float: 32 bytes).
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(h[i]); v[2 * i + 1] = __high2float(h[i]); }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<bf16>(bf16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// One block per token.  The token's D/2 (cos, sin) pairs are computed once into shared memory;
// then a thread takes 8 channels j .. j+7 of a head with their partners j + D/2 .. (D is a
// multiple of 16, so both runs are whole 16- or 32-byte vectors).
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ pos, int n_tokens,
                                  const float* __restrict__ inv_freq, const int* __restrict__ axis,
                                  T* __restrict__ kpages, T* __restrict__ vpages,
                                  const int* __restrict__ kv_slot, int nq, int nkv, int d, int page_size,
                                  int rotate, int store, const float2* __restrict__ angles) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float2 cs[];                       // [d / 2] (cos, sin)
  const int token = blockIdx.x;
  const int half = d >> 1;
  T* row = qkv + (size_t)token * (nq + 2 * nkv) * d;
  const int slot = store ? kv_slot[token] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot % page_size : 0;
  if (rotate) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      if (angles) {                                    // the step's (cos, sin), computed once for all its layers
        cs[j] = angles[(size_t)token * half + j];
        continue;
      }
      const float p = (float)pos[(size_t)axis[j] * n_tokens + token];
      float s, c;
      sincosf(p * inv_freq[j], &s, &c);
      cs[j] = make_float2(c, s);
    }
    __syncthreads();
  }
  const int chunks = half >> 3;                        // 8-channel runs in half a head
  for (int idx = threadIdx.x; idx < (nq + nkv) * chunks; idx += blockDim.x) {
    const int head = idx / chunks, j = (idx - head * chunks) << 3;
    if (head < nq && !rotate) continue;                // q is left as it is
    T* hp = row + (size_t)head * d;
    float x1[8], x2[8], y1[8], y2[8];
    load8<T>(hp + j, x1);
    load8<T>(hp + j + half, x2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 t = rotate ? cs[j + i] : make_float2(1.f, 0.f);
      y1[i] = x1[i] * t.x - x2[i] * t.y;
      y2[i] = x2[i] * t.x + x1[i] * t.y;
    }
    if (head < nq) {
      store8<T>(hp + j, y1);
      store8<T>(hp + j + half, y2);
    } else if (slot >= 0) {
      T* kr = kpages + (((size_t)page * nkv + (head - nq)) * page_size + off) * d;
      store8<T>(kr + j, y1);
      store8<T>(kr + j + half, y2);
    }
  }
  if (slot >= 0) {
    const T* vsrc = row + (size_t)(nq + nkv) * d;
    for (int idx = threadIdx.x * 8; idx < nkv * d; idx += blockDim.x * 8) {
      const int h = idx / d, c = idx - h * d;
      float v[8];
      load8<T>(vsrc + idx, v);
      store8<T>(vpages + (((size_t)page * nkv + h) * page_size + off) * d + c, v);
    }
  }
}

// The same with the step's angles given (float2 [n, D/2]: what rope_angles made of the positions):
// nothing is shared inside a token any more, so the work is flat: a thread takes one run of 8
// channels of one head of one token with its partner run, or 8 values of v.  With a block per token
// (144 runs for 128 threads, three trips to memory one after the other) 2,048 tokens of 16 + 2
// heads took 13 us for 22 MB; every thread busy once, its loads asked for together, is one trip.
template <typename T>
__global__ void rope_store_flat_kernel(T* __restrict__ qkv, int n_tokens, const float2* __restrict__ angles,
                                       T* __restrict__ kpages, T* __restrict__ vpages, const int* __restrict__ kv_slot,
                                       int nq, int nkv, int d, int page_size, int store) {
  pdl_trigger();
  pdl_wait();
  const int half = d >> 1, chunks = half >> 3;
  const int rot_items = (nq + nkv) * chunks, v_items = store ? nkv * (d >> 3) : 0, per_token = rot_items + v_items;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * per_token) return;
  const int token = (int)(idx / per_token), item = (int)(idx - (long long)token * per_token);
  T* row = qkv + (size_t)token * (nq + 2 * nkv) * d;
  const int slot = store ? kv_slot[token] : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  if (item >= rot_items) {                             // 8 values of v into their page
    if (slot < 0) return;
    const int e = (item - rot_items) << 3, h = e / d, c = e - h * d;
    float v[8];
    load8<T>(row + (size_t)(nq + nkv) * d + e, v);
    store8<T>(vpages + (((size_t)page * nkv + h) * page_size + off) * d + c, v);
    return;
  }
  const int head = item / chunks, j = (item - head * chunks) << 3;
  if (head >= nq && slot < 0) return;                  // a key that is stored nowhere
  T* hp = row + (size_t)head * d;
  float x1[8], x2[8], y1[8], y2[8];
  const float4* cs = reinterpret_cast<const float4*>(angles + (size_t)token * half + j);   // 8 (cos, sin) pairs: 64 bytes
  const float4 t0 = cs[0], t1 = cs[1], t2 = cs[2], t3 = cs[3];
  load8<T>(hp + j, x1);
  load8<T>(hp + j + half, x2);
  const float c[8] = {t0.x, t0.z, t1.x, t1.z, t2.x, t2.z, t3.x, t3.z}, sn[8] = {t0.y, t0.w, t1.y, t1.w, t2.y, t2.w, t3.y, t3.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    y1[i] = x1[i] * c[i] - x2[i] * sn[i];
    y2[i] = x2[i] * c[i] + x1[i] * sn[i];
  }
  if (head < nq) {
    store8<T>(hp + j, y1);
    store8<T>(hp + j + half, y2);
  } else {
    T* kr = kpages + (((size_t)page * nkv + (head - nq)) * page_size + off) * d;
    store8<T>(kr + j, y1);
    store8<T>(kr + j + half, y2);
  }
}

template <typename T>
static int rope_store(void* qkv, const int* pos, int n, const float* inv_freq, const int* axis, void* kpages,
                      void* vpages, const int* kv_slot, int nq, int nkv, int d, int page_size, int rotate, int store,
                      const void* angles, void* stream) {
  if (n <= 0) return 0;
  if (d % 16 || (((uintptr_t)qkv | (uintptr_t)kpages | (uintptr_t)vpages) & 15)) return (int)cudaErrorInvalidValue;
  if (angles && rotate && !((uintptr_t)angles & 15)) {
    const long long items = (long long)n * ((nq + nkv) * (d / 16) + (store ? nkv * (d / 8) : 0));
    launch(rope_store_flat_kernel<T>, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, (T*)qkv, n,
           (const float2*)angles, (T*)kpages, (T*)vpages, kv_slot, nq, nkv, d, page_size, store);
    return launch_status();
  }
  launch(rope_store_kernel<T>, dim3(n), dim3(128), (size_t)(d / 2) * sizeof(float2), (cudaStream_t)stream, (T*)qkv, pos, n, inv_freq, axis, (T*)kpages, (T*)vpages,
                                                            kv_slot, nq, nkv, d, page_size, rotate, store, (const float2*)angles);
  return launch_status();
}

// angles: float2 [n, d / 2] (cos, sin) of every token's rotary angles, or null to compute them here.
Q25_EXPORT int q25_rope_store_f32(void* qkv, const int* pos, int n, const float* inv, const int* axis, void* kp, void* vp,
                                  const int* slot, int nq, int nkv, int d, int ps, int rotate, int store, const void* angles,
                                  void* s) {
  return rope_store<float>(qkv, pos, n, inv, axis, kp, vp, slot, nq, nkv, d, ps, rotate, store, angles, s);
}
Q25_EXPORT int q25_rope_store_bf16(void* qkv, const int* pos, int n, const float* inv, const int* axis, void* kp, void* vp,
                                   const int* slot, int nq, int nkv, int d, int ps, int rotate, int store, const void* angles,
                                   void* s) {
  return rope_store<bf16>(qkv, pos, n, inv, axis, kp, vp, slot, nq, nkv, d, ps, rotate, store, angles, s);
}
