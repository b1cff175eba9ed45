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
#include "common.cuh"

#define ATTN_THREADS 128
#define DEC_BN 32
#define PRE_BN 64

struct AttnArgs {
  const bf16* qkv;
  int qkv_stride;
  bf16* out;
  const bf16* kpages;
  const bf16* vpages;
  const int* block_table;
  int table_width;
  const int* cu_q;
  const int* q_start_pos;
  const int* items;   // decode: entry index per blockIdx.x; prefill: (entry, row tile) pairs
  int nq, nkv, page_shift, window;
  float scale_log2;
  int n_splits;
  float* part_o;      // [items, nq, splits, D]
  float* part_ml;     // [items, nq, splits, 2]
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Row pitch of a key/value tile in shared memory: D bf16 plus 16 bytes, an odd number of 16-byte
// chunks, so the 8 row addresses of an ldmatrix fall into different banks.
template <int D> struct Tile { static constexpr int PITCH = D * 2 + 16; };

// The warp's 16 query rows as mma A fragments, D/16 k-steps.  row_ptr(r) gives row r or nullptr.
template <int D, typename RowPtr>
__device__ __forceinline__ void load_q(unsigned (&qf)[D / 16][4], RowPtr row_ptr) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const bf16* r0 = row_ptr(g);
  const bf16* r1 = row_ptr(g + 8);
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int c = ks * 16 + 2 * t;
    qf[ks][0] = r0 ? *reinterpret_cast<const unsigned*>(r0 + c) : 0u;
    qf[ks][1] = r1 ? *reinterpret_cast<const unsigned*>(r1 + c) : 0u;
    qf[ks][2] = r0 ? *reinterpret_cast<const unsigned*>(r0 + c + 8) : 0u;
    qf[ks][3] = r1 ? *reinterpret_cast<const unsigned*>(r1 + c + 8) : 0u;
  }
}

// Copies keys [key0, key0 + BN) of one kv head into a tile (zeros past last_key), by NT threads of
// which this is number `tid`.  The loop is unrolled and free of branches, so the block-table
// look-ups of all its iterations are in flight together instead of one after the other.
template <int D, int BN, int NT>
__device__ __forceinline__ void load_kv_tile(unsigned char* ks, unsigned char* vs, const AttnArgs& a, const int* table,
                                             int kvh, int key0, int last_key, int tid) {
  constexpr int CH = D / 8;  // 16-byte chunks in a row
  static_assert((BN * CH) % NT == 0, "the chunks of a tile divide evenly among the threads");
  const int ps_mask = (1 << a.page_shift) - 1;
#pragma unroll
  for (int i = 0; i < BN * CH / NT; ++i) {
    const int idx = tid + i * NT;
    const int key = idx / CH, ch = idx - key * CH;
    const int kidx = key0 + key;
    const bool valid = kidx <= last_key;
    const int kc = valid ? kidx : last_key;             // a readable address also for the zero-filled rows
    const int page = table[kc >> a.page_shift];
    const size_t off = ((((size_t)page * a.nkv + kvh) << a.page_shift) + (kc & ps_mask)) * D + ch * 8;
    cp_async16(ks + key * Tile<D>::PITCH + ch * 16, a.kpages + off, valid);
    cp_async16(vs + key * Tile<D>::PITCH + ch * 16, a.vpages + off, valid);
  }
}

// One tile of keys for the warp's 16 rows: scores, mask, running softmax, O += P V.
// hi0/hi1 (lo0/lo1): last (first) visible key of rows g and g+8; a row that sees nothing has hi < lo.
template <int D, int BN>
__device__ __forceinline__ void attend_tile(const unsigned (&qf)[D / 16][4], const unsigned char* ks,
                                            const unsigned char* vs, int key0, int lo0, int hi0, int lo1, int hi1,
                                            bool need_mask, float scale_log2, float (&m)[2], float (&l)[2],
                                            float (&o)[D / 8][4]) {
  constexpr int P = Tile<D>::PITCH;
  const int lane = threadIdx.x & 31, t = lane & 3;
  float s[BN / 8][4];
#pragma unroll
  for (int j = 0; j < BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
  // k-step outermost: the MMAs that follow one another go to different accumulators (one per block
  // of 8 keys), so they do not wait for each other
  if constexpr (D % 32 == 0) {
#pragma unroll
    for (int kp = 0; kp < D / 32; ++kp) {
      unsigned b[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) ldmatrix_x4(b[j], ks + (j * 8 + (lane & 7)) * P + (kp * 32 + 8 * (lane >> 3)) * 2);
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) mma_bf16(s[j], qf[2 * kp], b[j][0], b[j][1]);
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) mma_bf16(s[j], qf[2 * kp + 1], b[j][2], b[j][3]);
    }
  } else {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      unsigned b[BN / 8][2];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) ldmatrix_x2(b[j], ks + (j * 8 + (lane & 7)) * P + (kk * 16 + 8 * ((lane >> 3) & 1)) * 2);
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) mma_bf16(s[j], qf[kk], b[j][0], b[j][1]);
    }
  }
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float v = s[j][e] * scale_log2;
      if (need_mask) {
        const int kidx = key0 + j * 8 + 2 * t + (e & 1);
        const bool ok = e < 2 ? (kidx >= lo0 && kidx <= hi0) : (kidx >= lo1 && kidx <= hi1);
        v = ok ? v : -INFINITY;
      }
      s[j][e] = v;
    }
    mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
    mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
  const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;  // nothing seen yet
  const float c0 = exp2f(m[0] - ms0), c1 = exp2f(m[1] - ms1);
  m[0] = mn0;
  m[1] = mn1;
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int j = 0; j < BN / 8; ++j) {
    s[j][0] = exp2f(s[j][0] - ms0);
    s[j][1] = exp2f(s[j][1] - ms0);
    s[j][2] = exp2f(s[j][2] - ms1);
    s[j][3] = exp2f(s[j][3] - ms1);
    sum0 += s[j][0] + s[j][1];
    sum1 += s[j][2] + s[j][3];
  }
  l[0] = l[0] * c0 + sum0;  // per-thread partial sums; the quad is reduced once at the end
  l[1] = l[1] * c1 + sum1;
#pragma unroll
  for (int nb = 0; nb < D / 8; ++nb) {
    o[nb][0] *= c0;
    o[nb][1] *= c0;
    o[nb][2] *= c1;
    o[nb][3] *= c1;
  }
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk) {
    unsigned pa[4];
    pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    const unsigned char* vrow = vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * P;
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      unsigned b[4];
      ldmatrix_x4_trans(b, vrow + (np * 16 + 8 * (lane >> 4)) * 2);
      mma_bf16(o[2 * np], pa, b[0], b[1]);
      mma_bf16(o[2 * np + 1], pa, b[2], b[3]);
    }
  }
}

__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

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
template <int D>
__global__ void attention_combine_kernel(AttnArgs a, int n_items) {
  pdl_trigger();
  pdl_wait();
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= n_items * a.nq) return;
  const int item = w / a.nq, head = w - item * a.nq;
  const int token = a.cu_q[a.items[item]];
  const size_t base = ((size_t)item * a.nq + head) * a.n_splits;
  // lanes over the splits for the maximum and the sum (n_splits <= 64), then over the channels
  float m0 = lane < a.n_splits ? a.part_ml[(base + lane) * 2] : -INFINITY;
  float m1 = lane + 32 < a.n_splits ? a.part_ml[(base + lane + 32) * 2] : -INFINITY;
  const float M = warp_max(fmaxf(m0, m1));
  const float w0 = m0 == -INFINITY ? 0.f : exp2f(m0 - M), w1 = m1 == -INFINITY ? 0.f : exp2f(m1 - M);
  float lpart = 0.f;
  if (lane < a.n_splits) lpart += a.part_ml[(base + lane) * 2 + 1] * w0;
  if (lane + 32 < a.n_splits) lpart += a.part_ml[(base + lane + 32) * 2 + 1] * w1;
  const float inv = 1.0f / warp_sum(lpart);
  for (int c0 = 0; c0 < D; c0 += 32) {      // every lane takes part in the shuffles, also past D
    const int c = c0 + lane;
    float acc = 0.f;
#pragma unroll 4
    for (int i = 0; i < a.n_splits; ++i) {
      const float wi = __shfl_sync(0xffffffffu, i < 32 ? w0 : w1, i & 31);
      if (c < D) acc = fmaf(a.part_o[(base + i) * D + c], wi, acc);
    }
    if (c < D) a.out[(size_t)token * a.nq * D + (size_t)head * D + c] = __float2bfloat16_rn(acc * inv);
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
struct RopeArgs {
  const int* positions;   // [axes, n_tokens]
  int n_tokens;
  const float* inv_freq;  // [D/2]
  const int* axis;        // [D/2]
  const int* kv_slot;     // [n_tokens]: page * page_size + offset of each token's key
  bf16* kpages_w;
  bf16* vpages_w;
  int* counters;          // [n_items * nkv], zero before the first launch; the kernel leaves them zero
  const float2* angles;   // [n_tokens, D/2] (cos, sin) of every token's angles, or nullptr: computed here
};

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

__device__ __forceinline__ unsigned rotate_pair_lo(unsigned x1, unsigned x2, float c0, float s0, float c1, float s1) {
  const __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&x1), b = *reinterpret_cast<__nv_bfloat162*>(&x2);
  return pack_bf16(__low2float(a) * c0 - __low2float(b) * s0, __high2float(a) * c1 - __high2float(b) * s1);
}
__device__ __forceinline__ unsigned rotate_pair_hi(unsigned x1, unsigned x2, float c0, float s0, float c1, float s1) {
  const __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&x1), b = *reinterpret_cast<__nv_bfloat162*>(&x2);
  return pack_bf16(__low2float(b) * c0 + __low2float(a) * s0, __high2float(b) * c1 + __high2float(a) * s1);
}

template <int D>
__global__ void __launch_bounds__(ATTN_THREADS) attention_decode_fused_kernel(AttnArgs a, RopeArgs r) {
  pdl_trigger();
  pdl_wait();
  static_assert(D % 32 == 0, "the rotation pairs channel j with j + D/2 inside one thread");
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int P = Tile<D>::PITCH;
  constexpr int TILE = DEC_BN * P;
  constexpr int HALF = D / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int item = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int seq = a.items[item];
  const int G = a.nq / a.nkv;
  const int token = a.cu_q[seq];
  const int p = a.q_start_pos[seq];
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  const int first_tile_key = lo & ~(DEC_BN - 1);
  const int n_tiles = (p - first_tile_key) / DEC_BN + 1;
  const int per_split = (n_tiles + a.n_splits - 1) / a.n_splits;
  const int t_begin = split * per_split, t_end = min(n_tiles, t_begin + per_split);
  const int* table = a.block_table + (size_t)seq * a.table_width;

  // start the first tile's copies before the position-encoding arithmetic
  unsigned char* wbuf = smem + (size_t)warp * 4 * TILE;
  int tile = t_begin + warp;
  if (tile < t_end) load_kv_tile<D, DEC_BN, 32>(wbuf, wbuf + TILE, a, table, kvh, first_tile_key + tile * DEC_BN, p, lane);
  cp_async_commit();

  // q of the group's heads, rotated in registers: channels j and j + D/2 sit in k-steps ks and
  // ks + D/32 of the same thread
  unsigned qf[D / 16][4];
  const bf16* qbase = a.qkv + (size_t)token * a.qkv_stride + (size_t)kvh * G * D;
  load_q<D>(qf, [&](int row) { return row < G ? qbase + (size_t)row * D : (const bf16*)nullptr; });
  // the token has D/2 angles; one thread computes each (cos, sin) once for the whole CTA
  __shared__ float2 cs[HALF];
  if (threadIdx.x < HALF && r.angles) {
    cs[threadIdx.x] = r.angles[(size_t)token * HALF + threadIdx.x];
  } else if (threadIdx.x < HALF) {
    const int j = threadIdx.x;
    // all five loads are independent of one another, so they cost one memory latency, not two
    const int ax = r.axis[j];
    const float p0 = (float)r.positions[token], p1 = (float)r.positions[(size_t)r.n_tokens + token],
                p2 = (float)r.positions[(size_t)2 * r.n_tokens + token];
    const float pj = ax == 0 ? p0 : (ax == 1 ? p1 : p2);
    float sn, c;
    sincosf(pj * r.inv_freq[j], &sn, &c);
    cs[j] = make_float2(c, sn);
  }
  __syncthreads();
#pragma unroll
  for (int ks = 0; ks < D / 32; ++ks) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {       // registers 0,1 (columns 2t, 2t+1) and 2,3 (columns 2t+8, 2t+9)
      const int j = ks * 16 + 2 * t + 8 * half;
      const float c0 = cs[j].x, s0 = cs[j].y, c1 = cs[j + 1].x, s1 = cs[j + 1].y;
#pragma unroll
      for (int row = 0; row < 2; ++row) {         // rows g and g + 8
        const unsigned x1 = qf[ks][2 * half + row], x2 = qf[ks + D / 32][2 * half + row];
        qf[ks][2 * half + row] = rotate_pair_lo(x1, x2, c0, s0, c1, s1);
        qf[ks + D / 32][2 * half + row] = rotate_pair_hi(x1, x2, c0, s0, c1, s1);
      }
    }
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int nb = 0; nb < D / 8; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;

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
    unsigned char* cb = wbuf + (size_t)stage * 2 * TILE;
    if (tile == n_tiles - 1) {
      // the token's own key and value: rotate k, patch both into the tile, store both to the pages
      const bf16* kv_new = a.qkv + (size_t)token * a.qkv_stride + (size_t)(a.nq + kvh) * D;
      const bf16* v_new = kv_new + (size_t)a.nkv * D;
      const int slot = r.kv_slot[token];
      const size_t page_off = slot >= 0 ? ((((size_t)(slot >> a.page_shift) * a.nkv + kvh) << a.page_shift)
                                           + (slot & ((1 << a.page_shift) - 1))) * D : 0;
      bf16* krow = reinterpret_cast<bf16*>(cb + (p - key0) * P);
      bf16* vrow = reinterpret_cast<bf16*>(cb + TILE + (p - key0) * P);
      for (int j = lane; j < HALF; j += 32) {
        const float cj = cs[j].x, sn = cs[j].y;
        const float x1 = __bfloat162float(kv_new[j]), x2 = __bfloat162float(kv_new[j + HALF]);
        const bf16 y1 = __float2bfloat16_rn(x1 * cj - x2 * sn), y2 = __float2bfloat16_rn(x2 * cj + x1 * sn);
        krow[j] = y1;
        krow[j + HALF] = y2;
        if (slot >= 0) {
          r.kpages_w[page_off + j] = y1;
          r.kpages_w[page_off + j + HALF] = y2;
        }
      }
      for (int c = lane; c < D; c += 32) {
        const bf16 v = v_new[c];
        vrow[c] = v;
        if (slot >= 0) r.vpages_w[page_off + c] = v;
      }
      __syncwarp();
    }
    const bool need_mask = key0 < lo || key0 + DEC_BN - 1 > p;
    attend_tile<D, DEC_BN>(qf, cb, cb + TILE, key0, lo, p, lo, p, need_mask, a.scale_log2, m, l, o);
    __syncwarp();
    stage ^= 1;
  }
  cp_async_wait<0>();
  l[0] = quad_sum(l[0]);
  l[1] = quad_sum(l[1]);

  // merge the 4 warps of the CTA (as in attention_decode_kernel), keep the result in shared memory
  __syncthreads();
  float* ml = reinterpret_cast<float*>(smem);                 // [4 warps][16 rows][2]
  float* slab = ml + 4 * 16 * 2;                              // [4 warps][16 rows][D]
  __shared__ int is_last;
  if (t == 0) {
    ml[(warp * 16 + g) * 2] = m[0];
    ml[(warp * 16 + g) * 2 + 1] = l[0];
    ml[(warp * 16 + g + 8) * 2] = m[1];
    ml[(warp * 16 + g + 8) * 2 + 1] = l[1];
  }
  __syncthreads();
  float f[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = g + 8 * h;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, ml[(w * 16 + row) * 2]);
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
    const int row = idx / D, c = idx - row * D;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, ml[(w * 16 + row) * 2]);
    float lsum = 0.f, acc = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float mw = ml[(w * 16 + row) * 2];
      lsum += mw == -INFINITY ? 0.f : ml[(w * 16 + row) * 2 + 1] * exp2f(mw - mm);
      acc += slab[((size_t)w * 16 + row) * D + c];
    }
    const int head = kvh * G + row;
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
  if (a.n_splits == 1) return;

  // merge the splits: every CTA counts itself in after its partial is written; the one that finds
  // all the others already counted reads their partials and writes the output.  Nobody waits.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(r.counters + item * a.nkv + kvh, 1);
    is_last = done == a.n_splits - 1;
    if (is_last) r.counters[item * a.nkv + kvh] = 0;            // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // A thread merges four channels of one row over all splits.  The partials of 16 splits are asked
  // for together (one trip to L2 for all of them), then weighted by exp2(m_k - M) and added in split
  // order; with more than 16 splits the running maximum is carried as in the attention loop itself.
  const int n4 = G * (D / 4);
  for (int e = threadIdx.x; e < n4; e += ATTN_THREADS) {
    const int row = e / (D / 4), c4 = e - row * (D / 4);
    const size_t base = ((size_t)item * a.nq + kvh * G + row) * a.n_splits;
    const float2* ml_row = reinterpret_cast<const float2*>(a.part_ml) + base;
    float M = -INFINITY, L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < a.n_splits; k0 += 16) {
      float2 ml[16];
      float4 po[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int kk = min(k0 + j, a.n_splits - 1);                  // always a readable address
        ml[j] = __ldcg(ml_row + kk);
        po[j] = __ldcg(reinterpret_cast<const float4*>(a.part_o + (base + kk) * D) + c4);
      }
      float mb = -INFINITY;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (k0 + j < a.n_splits) mb = fmaxf(mb, ml[j].x);
      const float Mn = fmaxf(M, mb);
      const float keep = M == -INFINITY ? 0.f : exp2f(M - Mn);
      acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
      L *= keep;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (k0 + j >= a.n_splits || ml[j].x == -INFINITY) continue;
        const float w = exp2f(ml[j].x - Mn);
        L += ml[j].y * w;
        acc.x = fmaf(po[j].x, w, acc.x); acc.y = fmaf(po[j].y, w, acc.y);
        acc.z = fmaf(po[j].z, w, acc.z); acc.w = fmaf(po[j].w, w, acc.w);
      }
      M = Mn;
    }
    const float inv = 1.0f / L;
    uint2 packed;
    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(a.out + (size_t)token * a.nq * D + (size_t)(kvh * G + row) * D + c4 * 4) = packed;
  }
}

template <int D>
static int launch_decode_fused(const AttnArgs& a, const RopeArgs& r, int n_items, cudaStream_t s) {
  constexpr size_t kv = (size_t)4 * 4 * DEC_BN * Tile<D>::PITCH;
  constexpr size_t merge = (size_t)(4 * 16 * 2 + 4 * 16 * D) * sizeof(float);
  constexpr size_t smem = kv > merge ? kv : merge;
  cudaError_t e = cudaFuncSetAttribute(attention_decode_fused_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  launch(attention_decode_fused_kernel<D>, dim3(dim3(n_items, a.nkv, a.n_splits)), dim3(ATTN_THREADS), smem, s, a, r);
  return launch_status();
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

static int fill_args(AttnArgs& a, const void* qkv, int qkv_stride, void* out, const void* kp, const void* vp,
                     const int* bt, int tw, const int* cu_q, const int* q_start, const int* items, int nq, int nkv,
                     int page_size, int window, float scale) {
  if (page_size <= 0 || (page_size & (page_size - 1)) || nkv <= 0 || nq % nkv) return (int)cudaErrorInvalidValue;
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  a.qkv = (const bf16*)qkv; a.qkv_stride = qkv_stride; a.out = (bf16*)out; a.kpages = (const bf16*)kp;
  a.vpages = (const bf16*)vp; a.block_table = bt; a.table_width = tw; a.cu_q = cu_q; a.q_start_pos = q_start;
  a.items = items; a.nq = nq; a.nkv = nkv; a.page_shift = shift; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f; a.n_splits = 1; a.part_o = nullptr; a.part_ml = nullptr;
  return 0;
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
// and is not modified.  Head sizes 32, 64, 96, 128; groups of at most 16.
Q25_EXPORT int q25_attention_decode_fused_bf16(const void* qkv, int qkv_stride, void* out, void* kp, void* vp,
                                               const int* bt, int tw, const int* cu_q, const int* q_start,
                                               const int* items, int n_items, int nq, int nkv, int d, int page_size,
                                               int window, float scale, int n_splits, const int* positions,
                                               int n_tokens, const float* inv_freq, const int* axis,
                                               const int* kv_slot, float* scratch, int* counters, const void* angles,
                                               void* stream) {
  if (n_items <= 0) return 0;
  AttnArgs a;
  int e = fill_args(a, qkv, qkv_stride, out, kp, vp, bt, tw, cu_q, q_start, items, nq, nkv, page_size, window, scale);
  if (e) return e;
  if (nq / nkv > 16 || n_splits < 1 || n_splits > 64 || !positions || !inv_freq || !axis || !kv_slot || (n_splits > 1 && (!scratch || !counters)))
    return (int)cudaErrorInvalidValue;
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
