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

template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ pos, int n_tokens,
                                  const float* __restrict__ inv_freq, const int* __restrict__ axis,
                                  T* __restrict__ kpages, T* __restrict__ vpages,
                                  const int* __restrict__ kv_slot, int nq, int nkv, int d, int page_size,
                                  int rotate, int store) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const int half = d >> 1;
  T* row = qkv + (size_t)token * (nq + 2 * nkv) * d;
  const int slot = store ? kv_slot[token] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot % page_size : 0;

  for (int idx = threadIdx.x; idx < (nq + nkv) * half; idx += blockDim.x) {
    const int head = idx / half, j = idx - head * half;
    T* hp = row + (size_t)head * d;
    const float x1 = to_f32(hp[j]), x2 = to_f32(hp[j + half]);
    float y1 = x1, y2 = x2;
    if (rotate) {
      const float p = (float)pos[(size_t)axis[j] * n_tokens + token];
      float s, c;
      sincosf(p * inv_freq[j], &s, &c);
      y1 = x1 * c - x2 * s;
      y2 = x2 * c + x1 * s;
    }
    if (head < nq) {
      hp[j] = from_f32<T>(y1);
      hp[j + half] = from_f32<T>(y2);
    } else if (slot >= 0) {
      T* kr = kpages + (((size_t)page * nkv + (head - nq)) * page_size + off) * d;
      kr[j] = from_f32<T>(y1);
      kr[j + half] = from_f32<T>(y2);
    }
  }
  if (slot >= 0) {
    const T* vsrc = row + (size_t)(nq + nkv) * d;
    for (int idx = threadIdx.x; idx < nkv * d; idx += blockDim.x) {
      const int h = idx / d, c = idx - h * d;
      vpages[(((size_t)page * nkv + h) * page_size + off) * d + c] = vsrc[idx];
    }
  }
}

template <typename T>
static int rope_store(void* qkv, const int* pos, int n, const float* inv_freq, const int* axis, void* kpages,
                      void* vpages, const int* kv_slot, int nq, int nkv, int d, int page_size, int rotate, int store,
                      void* stream) {
  if (n <= 0) return 0;
  if (d % 2) return (int)cudaErrorInvalidValue;
  launch(rope_store_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, (T*)qkv, pos, n, inv_freq, axis, (T*)kpages, (T*)vpages,
                                                            kv_slot, nq, nkv, d, page_size, rotate, store);
  return launch_status();
}

Q25_EXPORT int q25_rope_store_f32(void* qkv, const int* pos, int n, const float* inv, const int* axis, void* kp, void* vp,
                                  const int* slot, int nq, int nkv, int d, int ps, int rotate, int store, void* s) {
  return rope_store<float>(qkv, pos, n, inv, axis, kp, vp, slot, nq, nkv, d, ps, rotate, store, s);
}
Q25_EXPORT int q25_rope_store_bf16(void* qkv, const int* pos, int n, const float* inv, const int* axis, void* kp, void* vp,
                                   const int* slot, int nq, int nkv, int d, int ps, int rotate, int store, void* s) {
  return rope_store<bf16>(qkv, pos, n, inv, axis, kp, vp, slot, nq, nkv, d, ps, rotate, store, s);
}
