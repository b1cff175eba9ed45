// Causal attention over the paged cache for a batch of (request, run of tokens): the general
// kernel.  It takes any head size that is a multiple of 16 up to 256, any number of heads and
// groups, any page size, a window or none, float or bfloat16, and any mixture of run lengths.
// It is the only attention of the 32-bit path and the fallback of the serving path for sizes the
// tensor-core kernels refuse.
//
// Formula (reference: zhangjianbang-nb/qwen25vl-lite): S = (q . k^T) * D^-1/2; the query at
// absolute index a = computed + i sees keys j <= a; softmax over keys; o = P v; query head h
// reads kv head h / (nq / nkv).   src/qwen25vl_lite/text.py:78,156-175;
// src/qwen25vl_lite/attention.py:143-148,366-372.  A window W (0 = none) also hides j <= a - W.
//
// One warp per (token, query head).  Keys are walked in tiles of 32 aligned to the absolute key
// index, lanes over keys for the scores and over channels for P.v, with a running maximum and
// sum in float.  The order of every sum depends only on the query's own position, never on how
// the tokens were cut into steps or on what else is in the batch.
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_D 256

template <typename T>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ qkv, int qkv_stride, T* __restrict__ out, const T* __restrict__ kpages,
    const T* __restrict__ vpages, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ token_seq, const int* __restrict__ cu_q, const int* __restrict__ q_start_pos,
    int n_tokens, int nq, int nkv, int d, int page_size, int window, float scale) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char att_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // per warp: q (d floats), probabilities (32 floats), V row offsets (32 x size_t)
  const size_t per_warp = (size_t)(d + 32) * sizeof(float) + 32 * sizeof(size_t);
  unsigned char* base = att_smem + warp * per_warp;
  size_t* voff = reinterpret_cast<size_t*>(base);
  float* qs = reinterpret_cast<float*>(base + 32 * sizeof(size_t));
  float* ps = qs + d;

  const long long item = (long long)blockIdx.x * ATT_WARPS + warp;
  if (item >= (long long)n_tokens * nq) return;
  const int token = (int)(item / nq), head = (int)(item % nq);
  const int kvh = head / (nq / nkv);
  const int seq = token_seq[token];
  if (seq < 0) return;  // a padding token of a fixed-shape batch
  const int p = q_start_pos[seq] + token - cu_q[seq];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;

  const T* q = qkv + (size_t)token * qkv_stride + (size_t)head * d;
  for (int c = lane; c < d; c += 32) qs[c] = to_f32(q[c]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < ATT_MAX_D / 32; ++i) acc[i] = 0.f;

  const int* table = block_table + (size_t)seq * table_width;
  for (int t0 = lo & ~31; t0 <= p; t0 += 32) {
    const int key = t0 + lane;
    const bool valid = key >= lo && key <= p;
    float s = -INFINITY;
    size_t off = 0;
    if (valid) {
      const int page = table[key / page_size];
      off = (((size_t)page * nkv + kvh) * page_size + (key % page_size)) * d;
      const T* kr = kpages + off;
      float dot = 0.f;
      for (int c = 0; c < d; ++c) dot = fmaf(qs[c], to_f32(kr[c]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));  // finite: every tile holds at least one valid key
    const float pexp = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);          // first tile: exp(-inf) = 0
    l = l * corr + warp_sum(pexp);
    m = m_new;
    ps[lane] = pexp;
    voff[lane] = off;
    __syncwarp();
    const int kmax = min(32, p - t0 + 1);
    const int kmin = max(0, lo - t0);
#pragma unroll
    for (int i = 0; i < ATT_MAX_D / 32; ++i) {
      const int c = lane + 32 * i;
      if (c < d) {
        float a = acc[i] * corr;
        for (int kk = kmin; kk < kmax; ++kk) a = fmaf(ps[kk], to_f32(vpages[voff[kk] + c]), a);
        acc[i] = a;
      }
    }
    __syncwarp();
  }
  T* o = out + (size_t)token * nq * d + (size_t)head * d;
  const float inv_l = 1.0f / l;
#pragma unroll
  for (int i = 0; i < ATT_MAX_D / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < d) o[c] = from_f32<T>(acc[i] * inv_l);
  }
}

template <typename T>
static int paged_attention_generic(const void* qkv, int qkv_stride, void* out, const void* kpages, const void* vpages,
                                   const int* block_table, int table_width, const int* token_seq, const int* cu_q,
                                   const int* q_start_pos, int n_tokens, int nq, int nkv, int d, int page_size,
                                   int window, float scale, void* stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || d > ATT_MAX_D || nkv <= 0 || nq % nkv) return (int)cudaErrorInvalidValue;
  const long long items = (long long)n_tokens * nq;
  const unsigned blocks = (unsigned)((items + ATT_WARPS - 1) / ATT_WARPS);
  const size_t smem = ATT_WARPS * ((size_t)(d + 32) * sizeof(float) + 32 * sizeof(size_t));
  launch(paged_attention_generic_kernel<T>, dim3(blocks), dim3(ATT_WARPS * 32), smem, (cudaStream_t)stream, 
      (const T*)qkv, qkv_stride, (T*)out, (const T*)kpages, (const T*)vpages, block_table, table_width, token_seq,
      cu_q, q_start_pos, n_tokens, nq, nkv, d, page_size, window, scale);
  return launch_status();
}

Q25_EXPORT int q25_paged_attention_generic_f32(const void* qkv, int qs, void* out, const void* kp, const void* vp,
                                               const int* bt, int tw, const int* ts, const int* cu, const int* sp, int n,
                                               int nq, int nkv, int d, int ps, int window, float scale, void* s) {
  return paged_attention_generic<float>(qkv, qs, out, kp, vp, bt, tw, ts, cu, sp, n, nq, nkv, d, ps, window, scale, s);
}
Q25_EXPORT int q25_paged_attention_generic_bf16(const void* qkv, int qs, void* out, const void* kp, const void* vp,
                                                const int* bt, int tw, const int* ts, const int* cu, const int* sp, int n,
                                                int nq, int nkv, int d, int ps, int window, float scale, void* s) {
  return paged_attention_generic<bf16>(qkv, qs, out, kp, vp, bt, tw, ts, cu, sp, n, nq, nkv, d, ps, window, scale, s);
}
