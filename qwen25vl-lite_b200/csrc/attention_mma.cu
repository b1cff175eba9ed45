// Tensor-core attention over the paged cache for the bfloat16 serving path.
//
// Same formula and masking as the general kernel (attention_generic.cu; reference
// src/qwen25vl_lite/text.py:78,156-175, src/qwen25vl_lite/attention.py:143-148,366-372), computed
// FlashAttention-style: S = Q K^T and O += P V on mma.sync m16n8k16 (bf16 in, float accumulate),
// running maximum and sum in float, scores in the exp2 domain.  The rows of a tile are (token,
// query head of one kv group) pairs, so one read of a kv head's keys and values serves the whole
// group (the reference's Triton kernel re-reads them per query head,
// src/qwen25vl_lite/paged_attn_triton.py:71-122).
//
// Two kernels:
//   decode   entries that bring one token: grid (entry, kv head, split).  The 4 warps of a CTA take
//            alternate 32-key tiles of the split through warp-private cp.async double buffers and
//            merge in shared memory; with more than one split the CTA writes an unnormalised
//            partial (O, m, l) to scratch memory and a combine kernel finishes
//            (flash-decoding; the reference's K1/K2, paged_attn_triton.py:71-148).
//   prefill  entries that bring runs of tokens: grid (64-row tile, kv head); the 4 warps share
//            64-key tiles through a CTA-wide cp.async double buffer; key tiles past the causal
//            edge are skipped.
// Head sizes: multiples of 16 up to 128.  Page sizes: powers of two.  Other sizes take the general
// kernel.
#include "attention_decode.cuh"


// ------------------------------------------------------------------------------------------------
// decode: one token per entry, rows = the G query heads of the kv group (G <= 16)
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(ATTN_THREADS) attention_decode_kernel(AttnArgs a) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int P = Tile<D>::PITCH;
  constexpr int TILE = DEC_BN * P;                 // bytes of one K (or V) tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int item = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int seq = a.items[item];
  const int G = a.nq / a.nkv;
  const int token = a.cu_q[seq];
  const int p = a.q_start_pos[seq];                // the token's own index = its last visible key
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  const int first_tile_key = lo & ~(DEC_BN - 1);
  const int n_tiles = (p - first_tile_key) / DEC_BN + 1;
  const int per_split = (n_tiles + a.n_splits - 1) / a.n_splits;
  const int t_begin = split * per_split, t_end = min(n_tiles, t_begin + per_split);
  const int* table = a.block_table + (size_t)seq * a.table_width;

  unsigned qf[D / 16][4];
  const bf16* qbase = a.qkv + (size_t)token * a.qkv_stride + (size_t)kvh * G * D;
  load_q<D>(qf, [&](int r) { return r < G ? qbase + (size_t)r * D : (const bf16*)nullptr; });

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int nb = 0; nb < D / 8; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;

  unsigned char* wbuf = smem + (size_t)warp * 4 * TILE;   // [stage][K,V]
  int tile = t_begin + warp;
  if (tile < t_end) {
    load_kv_tile<D, DEC_BN, 32>(wbuf, wbuf + TILE, a, table, kvh, first_tile_key + tile * DEC_BN, p, lane);
  }
  cp_async_commit();
  int stage = 0;
  for (; tile < t_end; tile += 4) {
    const int next = tile + 4;
    if (next < t_end) {
      unsigned char* nb = wbuf + (size_t)(stage ^ 1) * 2 * TILE;
      load_kv_tile<D, DEC_BN, 32>(nb, nb + TILE, a, table, kvh, first_tile_key + next * DEC_BN, p, lane);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncwarp();
    const int key0 = first_tile_key + tile * DEC_BN;
    const bool need_mask = key0 < lo || key0 + DEC_BN - 1 > p;
    unsigned char* cb = wbuf + (size_t)stage * 2 * TILE;
    attend_tile<D, DEC_BN>(qf, cb, cb + TILE, key0, lo, p, lo, p, need_mask, a.scale_log2, m, l, o);
    __syncwarp();
    stage ^= 1;
  }
  cp_async_wait<0>();
  l[0] = quad_sum(l[0]);
  l[1] = quad_sum(l[1]);

  // merge the 4 warps: maxima and sums through shared memory, O through per-warp slabs
  __syncthreads();
  float* ml = reinterpret_cast<float*>(smem);                 // [4 warps][16 rows][2]
  float* slab = ml + 4 * 16 * 2;                              // [4 warps][16 rows][D]
  if (t == 0) {
    ml[(warp * 16 + g) * 2] = m[0];
    ml[(warp * 16 + g) * 2 + 1] = l[0];
    ml[(warp * 16 + g + 8) * 2] = m[1];
    ml[(warp * 16 + g + 8) * 2 + 1] = l[1];
  }
  __syncthreads();
  float mall[2], f[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, ml[(w * 16 + r) * 2]);
    mall[h] = mm;
    f[h] = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - mm);
  }
#pragma unroll
  for (int nb = 0; nb < D / 8; ++nb) {
    float* r0 = slab + ((size_t)warp * 16 + g) * D + nb * 8 + 2 * t;
    float* r1 = slab + ((size_t)warp * 16 + g + 8) * D + nb * 8 + 2 * t;
    r0[0] = o[nb][0] * f[0];
    r0[1] = o[nb][1] * f[0];
    r1[0] = o[nb][2] * f[1];
    r1[1] = o[nb][3] * f[1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += ATTN_THREADS) {
    const int r = idx / D, c = idx - r * D;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, ml[(w * 16 + r) * 2]);
    float lsum = 0.f, acc = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float mw = ml[(w * 16 + r) * 2];
      lsum += mw == -INFINITY ? 0.f : ml[(w * 16 + r) * 2 + 1] * exp2f(mw - mm);
      acc += slab[((size_t)w * 16 + r) * D + c];
    }
    const int head = kvh * G + r;
    if (a.n_splits == 1) {
      a.out[(size_t)token * a.nq * D + (size_t)head * D + c] = __float2bfloat16_rn(acc / lsum);
    } else {
      const size_t pi = ((size_t)item * a.nq + head) * a.n_splits + split;
      a.part_o[pi * D + c] = acc;
      if (c == 0) {
        a.part_ml[pi * 2] = mm;
        a.part_ml[pi * 2 + 1] = lsum;
      }
    }
  }
}

// out = sum_i 2^(m_i - M) O_i / sum_i 2^(m_i - M) l_i over the splits; one warp per (entry, head).
// Any number of splits: the lanes stride over them for the maximum and the sum, and every lane
// walks all of them for its channels (the weight of a split is a broadcast load and one exp2).
template <int D>
__global__ void attention_combine_kernel(AttnArgs a, int n_items) {
  pdl_trigger();
  pdl_wait();
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= n_items * a.nq) return;
  const int item = w / a.nq, head = w - item * a.nq;
  const int token = a.cu_q[a.items[item]];
  const size_t base = ((size_t)item * a.nq + head) * a.n_splits;
  const float2* ml = reinterpret_cast<const float2*>(a.part_ml) + base;
  float mx = -INFINITY;
  for (int i = lane; i < a.n_splits; i += 32) mx = fmaxf(mx, ml[i].x);
  const float M = warp_max(mx);
  float lpart = 0.f;
  for (int i = lane; i < a.n_splits; i += 32) {
    const float2 v = ml[i];
    if (v.x != -INFINITY) lpart += v.y * exp2f(v.x - M);
  }
  const float inv = 1.0f / warp_sum(lpart);
  for (int c = lane; c < D; c += 32) {
    float acc = 0.f;
#pragma unroll 4
    for (int i = 0; i < a.n_splits; ++i) {
      const float mi = ml[i].x;
      const float wi = mi == -INFINITY ? 0.f : exp2f(mi - M);
      acc = fmaf(a.part_o[(base + i) * D + c], wi, acc);
    }
    a.out[(size_t)token * a.nq * D + (size_t)head * D + c] = __float2bfloat16_rn(acc * inv);
  }
}

// ------------------------------------------------------------------------------------------------
// prefill: runs of tokens; a tile is 64 rows = (token, head of the group) pairs of one entry
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(ATTN_THREADS) attention_prefill_kernel(AttnArgs a) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int P = Tile<D>::PITCH;
  constexpr int TILE = PRE_BN * P;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int seq = a.items[2 * blockIdx.x], row_tile = a.items[2 * blockIdx.x + 1], kvh = blockIdx.y;
  const int G = a.nq / a.nkv;
  const int q0 = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q0, start = a.q_start_pos[seq];
  const int n_rows = q_len * G;
  const int R0 = row_tile * 64;
  const int* table = a.block_table + (size_t)seq * a.table_width;

  // the rows of this thread: R0 + 16 warp + g and + 8
  int tok[2], hi[2], lo[2];
  bool live[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int R = R0 + warp * 16 + g + 8 * h;
    live[h] = R < n_rows;
    tok[h] = live[h] ? R / G : 0;
    hi[h] = live[h] ? start + tok[h] : -1;
    lo[h] = live[h] ? (a.window > 0 ? max(0, hi[h] - a.window + 1) : 0) : 0;
  }
  unsigned qf[D / 16][4];
  load_q<D>(qf, [&](int r) {
    const int R = R0 + warp * 16 + r;
    return R < n_rows ? a.qkv + (size_t)(q0 + R / G) * a.qkv_stride + (size_t)(kvh * G + R % G) * D : (const bf16*)nullptr;
  });
  // key range of the warp and of the CTA
  const int w_first = min(R0 + warp * 16, n_rows - 1) / G, w_last = min(R0 + warp * 16 + 15, n_rows - 1) / G;
  const bool warp_live = R0 + warp * 16 < n_rows;
  const int w_hi = start + w_last, w_hi_min = start + w_first;
  const int w_lo = a.window > 0 ? max(0, start + w_first - a.window + 1) : 0;
  const int w_lo_max = a.window > 0 ? max(0, start + w_last - a.window + 1) : 0;
  const int c_first = R0 / G, c_last = min(R0 + 63, n_rows - 1) / G;
  const int c_hi = start + c_last;
  const int c_lo = a.window > 0 ? max(0, start + c_first - a.window + 1) : 0;
  const int key_begin = c_lo & ~(PRE_BN - 1);
  const int n_tiles = (c_hi - key_begin) / PRE_BN + 1;

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int nb = 0; nb < D / 8; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;

  load_kv_tile<D, PRE_BN, ATTN_THREADS>(smem, smem + TILE, a, table, kvh, key_begin, c_hi, threadIdx.x);
  cp_async_commit();
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) {
      unsigned char* nb = smem + (size_t)(stage ^ 1) * 2 * TILE;
      load_kv_tile<D, PRE_BN, ATTN_THREADS>(nb, nb + TILE, a, table, kvh, key_begin + (tile + 1) * PRE_BN, c_hi, threadIdx.x);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int key0 = key_begin + tile * PRE_BN;
    if (warp_live && key0 <= w_hi && key0 + PRE_BN - 1 >= w_lo) {
      const bool need_mask = key0 + PRE_BN - 1 > w_hi_min || key0 < w_lo_max;
      unsigned char* cb = smem + (size_t)stage * 2 * TILE;
      attend_tile<D, PRE_BN>(qf, cb, cb + TILE, key0, lo[0], hi[0], lo[1], hi[1], need_mask, a.scale_log2, m, l, o);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  l[0] = quad_sum(l[0]);
  l[1] = quad_sum(l[1]);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!live[h]) continue;
    const int R = R0 + warp * 16 + g + 8 * h;
    const float inv = 1.0f / l[h];
    bf16* dst = a.out + (size_t)(q0 + tok[h]) * a.nq * D + (size_t)(kvh * G + R % G) * D + 2 * t;
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) {
      *reinterpret_cast<__nv_bfloat162*>(dst + nb * 8) = __floats2bfloat162_rn(o[nb][2 * h] * inv, o[nb][2 * h + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// decode, fused: position encoding of q and k, the write of the new key and value into the pages,
// the attention and the merge of the splits in one kernel.  Each split leaves its partial result in
// scratch memory and counts itself in; the CTA that comes last merges them (nobody waits).
// The CTA whose range holds the token's own key rotates that key, patches it (and the value) into
// the tile in shared memory and stores both to the pages for later steps, so no kernel has to
// run before this one.  Rotation as in rope_cache.cu (reference src/qwen25vl_lite/rope.py:48-96).
// ------------------------------------------------------------------------------------------------

// (cos, sin) of every token's D/2 angles: the same for every layer of a step, so a step computes
// them once (angle[j] = pos[axis(j)] * inv_freq[j] in float, reference src/qwen25vl_lite/rope.py:48-96).
__global__ void rope_angles_kernel(const int* __restrict__ positions, int n_tokens, const float* __restrict__ inv_freq,
                                   const int* __restrict__ axis, int half, float2* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_tokens * half) return;
  const int token = idx / half, j = idx - token * half;
  const float p = (float)positions[(size_t)axis[j] * n_tokens + token];
  float sn, c;
  sincosf(p * inv_freq[j], &sn, &c);
  out[idx] = make_float2(c, sn);
}

// The fused decode kernel: 8 warps (4 where that lets all CTAs run at once, see launch_decode_fused),
// a warp's tile is 16 keys = one page look-up, made an iteration ahead, 3 stages of tiles per warp
// (210 KB of shared memory at head size 128 with 8 warps).  A shape without a
// loop (a 32-key tile per warp, all asked for at once) was no faster where it applies (at most 256
// keys per CTA) and is not kept.
template <int D, int WARPS, int BN, int STAGES>
__global__ void __launch_bounds__(WARPS * 32) attention_decode_fused_kernel(AttnArgs a, RopeArgs r) {
  pdl_trigger();
  extern __shared__ __align__(16) unsigned char smem[];
  using Unit = DecodeUnit<D, WARPS, BN, STAGES>;
  // the look-ups and the first tiles' copies inside come before the wait for the kernel that made q
  Unit::run(a, r, blockIdx.x, blockIdx.y, blockIdx.z, smem, threadIdx.x, [] { __syncthreads(); }, [] { pdl_wait(); });
}


template <int D, int WARPS, int BN, int STAGES>
static int launch_decode_fused_shape(const AttnArgs& a, const RopeArgs& r, int n_items, cudaStream_t s) {
  constexpr size_t smem = DecodeUnit<D, WARPS, BN, STAGES>::SMEM;
  cudaError_t e = cudaFuncSetAttribute(attention_decode_fused_kernel<D, WARPS, BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  launch(attention_decode_fused_kernel<D, WARPS, BN, STAGES>, dim3(dim3(n_items, a.nkv, a.n_splits)), dim3(WARPS * 32), smem, s, a, r);
  return launch_status();
}

template <int D>
static int launch_decode_fused(const AttnArgs& a, const RopeArgs& r, int n_items, cudaStream_t s) {
  // A CTA of 8 warps has its SM to itself.  Between one and two CTAs per SM, CTAs of 4 warps (half
  // the shared memory, two to an SM) all run at once instead of in two waves: 128 requests on 2 kv
  // heads, 2,048 keys each: 57 -> 51 us.  With still more CTAs the waves of 8 warps are faster again
  // (96 requests on 4 kv heads, 2,560 keys: 98 against 104 us).
  const long long ctas = (long long)n_items * a.nkv * a.n_splits;
  const int sms = device_sm_count();
  if (ctas > sms && ctas <= 2 * sms) return launch_decode_fused_shape<D, 4, 16, 3>(a, r, n_items, s);
  return launch_decode_fused_shape<D, 8, 16, 3>(a, r, n_items, s);
}


// ------------------------------------------------------------------------------------------------
template <int D>
static int launch_decode(const AttnArgs& a, int n_items, cudaStream_t s) {
  constexpr size_t kv = (size_t)4 * 4 * DEC_BN * Tile<D>::PITCH;                       // 4 warps x 2 stages x (K,V)
  constexpr size_t merge = (size_t)(4 * 16 * 2 + 4 * 16 * D) * sizeof(float);
  constexpr size_t smem = kv > merge ? kv : merge;
  cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  launch(attention_decode_kernel<D>, dim3(dim3(n_items, a.nkv, a.n_splits)), dim3(ATTN_THREADS), smem, s, a);
  if (a.n_splits > 1) {
    const int warps = n_items * a.nq;
    launch(attention_combine_kernel<D>, dim3((warps * 32 + 127) / 128), dim3(128), 0, s, a, n_items);
  }
  return launch_status();
}

template <int D>
static int launch_prefill(const AttnArgs& a, int n_tiles, cudaStream_t s) {
  constexpr size_t smem = (size_t)4 * PRE_BN * Tile<D>::PITCH;                         // 2 stages x (K,V)
  cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  launch(attention_prefill_kernel<D>, dim3(dim3(n_tiles, a.nkv)), dim3(ATTN_THREADS), smem, s, a);
  return launch_status();
}

#define DISPATCH_D(FN, ...)                          \
  switch (d) {                                       \
    case 16: return FN<16>(__VA_ARGS__);             \
    case 32: return FN<32>(__VA_ARGS__);             \
    case 48: return FN<48>(__VA_ARGS__);             \
    case 64: return FN<64>(__VA_ARGS__);             \
    case 80: return FN<80>(__VA_ARGS__);             \
    case 96: return FN<96>(__VA_ARGS__);             \
    case 112: return FN<112>(__VA_ARGS__);           \
    case 128: return FN<128>(__VA_ARGS__);           \
    default: return (int)cudaErrorInvalidValue;      \
  }


// Scratch floats a decode launch needs: n_items * nq * n_splits * (D + 2); none for one split.
Q25_EXPORT long long q25_attention_decode_scratch_floats(int n_items, int nq, int d, int n_splits) {
  return n_splits <= 1 ? 0 : (long long)n_items * nq * n_splits * (d + 2);
}

// items: entry index of each decode entry (entries that bring exactly one token).
Q25_EXPORT int q25_attention_decode_bf16(const void* qkv, int qkv_stride, void* out, const void* kp, const void* vp,
                                         const int* bt, int tw, const int* cu_q, const int* q_start, const int* items,
                                         int n_items, int nq, int nkv, int d, int page_size, int window, float scale,
                                         int n_splits, float* scratch, void* stream) {
  if (n_items <= 0) return 0;
  AttnArgs a;
  int e = fill_args(a, qkv, qkv_stride, out, kp, vp, bt, tw, cu_q, q_start, items, nq, nkv, page_size, window, scale);
  if (e) return e;
  if (nq / nkv > 16 || n_splits < 1 || (n_splits > 1 && !scratch)) return (int)cudaErrorInvalidValue;
  a.n_splits = n_splits;
  a.part_o = scratch;
  a.part_ml = scratch ? scratch + (size_t)n_items * nq * n_splits * d : nullptr;
  cudaStream_t s = (cudaStream_t)stream;
  DISPATCH_D(launch_decode, a, n_items, s)
}

// items: (entry, row tile) pairs; a row tile is 64 consecutive (token, head-of-group) rows.
Q25_EXPORT int q25_attention_prefill_bf16(const void* qkv, int qkv_stride, void* out, const void* kp, const void* vp,
                                          const int* bt, int tw, const int* cu_q, const int* q_start, const int* items,
                                          int n_tiles, int nq, int nkv, int d, int page_size, int window, float scale,
                                          void* stream) {
  if (n_tiles <= 0) return 0;
  AttnArgs a;
  int e = fill_args(a, qkv, qkv_stride, out, kp, vp, bt, tw, cu_q, q_start, items, nq, nkv, page_size, window, scale);
  if (e) return e;
  cudaStream_t s = (cudaStream_t)stream;
  DISPATCH_D(launch_prefill, a, n_tiles, s)
}

// Fused decode step of attention: rotates q and the new k by the 3-axis rotary encoding, stores the new
// k and v at kv_slot, attends, merges the n_splits key ranges (scratch as for q25_attention_decode_bf16,
// counters: n_items * nkv ints that are zero and stay zero).  qkv holds the un-rotated projections
// and is not modified.  Head sizes 32, 64, 96, 128; groups of at most 16.  dense: the items are 0 .. n_items - 1 and every
// entry has one token (token i belongs to entry i): the kernel then reads neither items nor cu_q.
Q25_EXPORT int q25_attention_decode_fused_bf16(const void* qkv, int qkv_stride, void* out, void* kp, void* vp,
                                               const int* bt, int tw, const int* cu_q, const int* q_start,
                                               const int* items, int n_items, int nq, int nkv, int d, int page_size,
                                               int window, float scale, int n_splits, const int* positions,
                                               int n_tokens, const float* inv_freq, const int* axis,
                                               const int* kv_slot, float* scratch, int* counters, const void* angles,
                                               int dense, void* stream) {
  if (n_items <= 0) return 0;
  AttnArgs a;
  int e = fill_args(a, qkv, qkv_stride, out, kp, vp, bt, tw, cu_q, q_start, items, nq, nkv, page_size, window, scale);
  if (e) return e;
  if (nq / nkv > 16 || n_splits < 1 || n_splits > 64 || !positions || !inv_freq || !axis || !kv_slot || (n_splits > 1 && (!scratch || !counters)))
    return (int)cudaErrorInvalidValue;
  if (dense) a.items = nullptr;
  a.n_splits = n_splits;
  a.part_o = scratch;
  a.part_ml = scratch ? scratch + (size_t)n_items * nq * n_splits * d : nullptr;
  RopeArgs r;
  r.counters = counters;
  r.positions = positions; r.n_tokens = n_tokens; r.inv_freq = inv_freq; r.axis = axis; r.kv_slot = kv_slot;
  r.kpages_w = (bf16*)kp; r.vpages_w = (bf16*)vp;
  r.angles = (const float2*)angles;
  cudaStream_t s = (cudaStream_t)stream;
  switch (d) {
    case 32: return launch_decode_fused<32>(a, r, n_items, s);
    case 64: return launch_decode_fused<64>(a, r, n_items, s);
    case 96: return launch_decode_fused<96>(a, r, n_items, s);
    case 128: return launch_decode_fused<128>(a, r, n_items, s);
    default: return (int)cudaErrorInvalidValue;
  }
}

// out[token][j] = (cos, sin)(positions[axis[j]][token] * inv_freq[j]) for j < half.
Q25_EXPORT int q25_rope_angles(const int* positions, int n_tokens, const float* inv_freq, const int* axis, int half,
                               void* out, void* stream) {
  if (n_tokens <= 0 || half <= 0) return 0;
  const int total = n_tokens * half;
  launch(rope_angles_kernel, dim3((total + 127) / 128), dim3(128), 0, (cudaStream_t)stream, positions, n_tokens, inv_freq, axis,
         half, (float2*)out);
  return launch_status();
}

// ------------------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate: see attention_noalloc.h.
// ------------------------------------------------------------------------------------------------
#include <stdio.h>

#include "attention_noalloc.h"

// Scratch for the split partials.  In host code this name is only a stand-in for the symbol, not a
// device address: the address each device gave it is looked up once below and passed to the kernel.
static __device__ __align__(256) float q25_noalloc_scratch[Q25_NOALLOC_SCRATCH_FLOATS];

#define Q25_NOALLOC_MAX_DEVICES 64
static float* q25_noalloc_address[Q25_NOALLOC_MAX_DEVICES];
static thread_local char q25_noalloc_message[256] = "";

Q25_EXPORT const char* q25_attention_decode_noalloc_error(void) { return q25_noalloc_message; }

Q25_EXPORT int q25_attention_decode_bf16_noalloc(const void* qkv, int qkv_stride, void* out, const void* kp,
                                                 const void* vp, const int* bt, int tw, const int* cu_q,
                                                 const int* q_start, const int* items, int n_items, int nq, int nkv,
                                                 int d, int page_size, int window, float scale, int n_splits,
                                                 void* stream) {
  q25_noalloc_message[0] = 0;
  if (n_items <= 0) return 0;
  const long long need = q25_attention_decode_scratch_floats(n_items, nq, d, n_splits);
  if (need > (long long)Q25_NOALLOC_SCRATCH_FLOATS) {
    snprintf(q25_noalloc_message, sizeof(q25_noalloc_message),
             "attention_decode_noalloc: %d entries x %d heads x %d splits need %lld floats of scratch, the built-in "
             "array holds %d; use fewer splits or the entry point that takes a scratch buffer",
             n_items, nq, n_splits, need, Q25_NOALLOC_SCRATCH_FLOATS);
    return Q25_NOALLOC_TOO_LARGE;
  }
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e == cudaSuccess && (device < 0 || device >= Q25_NOALLOC_MAX_DEVICES)) e = cudaErrorInvalidDevice;
  if (e == cudaSuccess && !q25_noalloc_address[device]) {   // set-up: first call on this device
    void* address = nullptr;
    e = cudaGetSymbolAddress(&address, q25_noalloc_scratch);
    if (e == cudaSuccess) q25_noalloc_address[device] = static_cast<float*>(address);
  }
  if (e != cudaSuccess) {
    snprintf(q25_noalloc_message, sizeof(q25_noalloc_message), "attention_decode_noalloc: set-up failed: %s",
             cudaGetErrorString(e));
    return (int)e;
  }
  return q25_attention_decode_bf16(qkv, qkv_stride, out, kp, vp, bt, tw, cu_q, q_start, items, n_items, nq, nkv, d,
                                   page_size, window, scale, n_splits, n_splits > 1 ? q25_noalloc_address[device] : nullptr,
                                   stream);
}
