// Device code shared by the attention kernels (attention_mma.cu, attention_tcgen05.cu): the argument
// structs, the tensor-core helpers, one tile of FlashAttention-style attention, and the fused decode
// attention unit.
#pragma once

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
  const int* items;   // decode: entry index per blockIdx.x (null: entry i is token i, one token each); prefill: (entry, row tile) pairs
  int nq, nkv, page_shift, window;
  float scale_log2;
  int n_splits;
  float* part_o;      // [items, nq, splits, D]
  float* part_ml;     // [items, nq, splits, 2]
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async16_whole(void* dst, const void* src) {     // without the size operand
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src));
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
    // past L1: inside a chain of operations another SM may have written q since this SM last read it
    qf[ks][0] = r0 ? __ldcg(reinterpret_cast<const unsigned*>(r0 + c)) : 0u;
    qf[ks][1] = r1 ? __ldcg(reinterpret_cast<const unsigned*>(r1 + c)) : 0u;
    qf[ks][2] = r0 ? __ldcg(reinterpret_cast<const unsigned*>(r0 + c + 8)) : 0u;
    qf[ks][3] = r1 ? __ldcg(reinterpret_cast<const unsigned*>(r1 + c + 8)) : 0u;
  }
}

// Copies keys [key0, key0 + BN) of one kv head into a tile (zeros past last_key), by NT threads of
// which this is number `tid`.  key0 is a multiple of BN.
//
// With pages of 16 tokens or more, a block of 16 keys lies in one page in one piece of 16 rows: a
// thread's copies of a block then read block + (tid + i * NT) * 16, one 64-bit base and constants.
// (Copies whose source addresses each need a look-up and a 64-bit multiply-add take a warp about
// three times as long to issue, which is most of what a copy costs the warp.)  Smaller pages, or a
// block whose chunks do not divide among the threads, take the general loop; it is unrolled and
// free of branches, so the block-table look-ups of all its iterations are in flight together.
template <int D, int BN, int NT>
__device__ __forceinline__ void load_kv_tile(unsigned char* ks, unsigned char* vs, const AttnArgs& a, const int* table,
                                             int kvh, int key0, int last_key, int tid) {
  constexpr int CH = D / 8;  // 16-byte chunks in a row
  static_assert((BN * CH) % NT == 0, "the chunks of a tile divide evenly among the threads");
  const int ps_mask = (1 << a.page_shift) - 1;
  if constexpr (BN % 16 == 0 && (16 * CH) % NT == 0) {
    if (a.page_shift >= 4) {
      constexpr int NB = BN / 16, PER = 16 * CH / NT;
      const unsigned char* kb[NB];
      const unsigned char* vb[NB];
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int kf = key0 + 16 * b;                      // a multiple of 16: the block does not straddle pages
        const bool any = kf <= last_key;
        const int page = table[(any ? kf : last_key) >> a.page_shift];
        const size_t off = (((((size_t)page * a.nkv + kvh) << a.page_shift) + (any ? (kf & ps_mask) : 0)) * D + (size_t)tid * 8) * sizeof(bf16);
        kb[b] = reinterpret_cast<const unsigned char*>(a.kpages) + off;
        vb[b] = reinterpret_cast<const unsigned char*>(a.vpages) + off;
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          const int c = tid + i * NT;
          const int key = c / CH, ch = c - key * CH;
          const bool valid = key0 + 16 * b + key <= last_key;
          const int dst = (16 * b + key) * Tile<D>::PITCH + ch * 16;
          cp_async16(ks + dst, kb[b] + i * NT * 16, valid);
          cp_async16(vs + dst, vb[b] + i * NT * 16, valid);
        }
      }
      return;
    }
  }
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

// The copies of a block of 16 keys that starts at key kf (a multiple of 16) and lies in `page` (pages
// of 16 tokens or more), by the 32 lanes of a warp: D / 16 pairs (one piece of K, one of V) per lane.
// The caller has looked the page up, ahead of time if it can.  (The load/store unit of an SM takes one
// such copy of 32 x 16 bytes about every 4 cycles: with 8 warps copying, 16 pairs cost each of them
// about 700 cycles, whether issued in one go or spread over the tile's arithmetic.)
template <int D>
struct BlockCopy {
  static constexpr int CH = D / 8, PAIRS = 16 * CH / 32;
  unsigned char *ks, *vs;
  const unsigned char *kb, *vb;
  int n_valid, lane;

  __device__ __forceinline__ void set(unsigned char* ks_, unsigned char* vs_, const AttnArgs& a, int page, int kvh, int kf, int last_key,
                                      int lane_) {
    ks = ks_; vs = vs_; lane = lane_;
    n_valid = min(max(last_key - kf + 1, 0), 16);
    const size_t off = (((((size_t)page * a.nkv + kvh) << a.page_shift) + (n_valid > 0 ? (kf & ((1 << a.page_shift) - 1)) : 0)) * D
                        + (size_t)lane * 8) * sizeof(bf16);
    kb = reinterpret_cast<const unsigned char*>(a.kpages) + off;
    vb = reinterpret_cast<const unsigned char*>(a.vpages) + off;
  }
  __device__ __forceinline__ void pair(int i) const {       // i < PAIRS, a constant after unrolling
    const int c = lane + i * 32;
    const int key = c / CH, ch = c - key * CH;
    const int dst = key * Tile<D>::PITCH + ch * 16;
    if (n_valid == 16) {                                     // every key exists: copies without a size operand
      cp_async16_whole(ks + dst, kb + i * 512);
      cp_async16_whole(vs + dst, vb + i * 512);
    } else {
      cp_async16(ks + dst, kb + i * 512, key < n_valid);
      cp_async16(vs + dst, vb + i * 512, key < n_valid);
    }
  }
  __device__ __forceinline__ void all() const {
#pragma unroll
    for (int i = 0; i < PAIRS; ++i) pair(i);
  }
};

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

__device__ __forceinline__ unsigned rotate_pair_lo(unsigned x1, unsigned x2, float c0, float s0, float c1, float s1) {
  const __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&x1), b = *reinterpret_cast<__nv_bfloat162*>(&x2);
  return pack_bf16(__low2float(a) * c0 - __low2float(b) * s0, __high2float(a) * c1 - __high2float(b) * s1);
}
__device__ __forceinline__ unsigned rotate_pair_hi(unsigned x1, unsigned x2, float c0, float s0, float c1, float s1) {
  const __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&x1), b = *reinterpret_cast<__nv_bfloat162*>(&x2);
  return pack_bf16(__low2float(b) * c0 + __low2float(a) * s0, __high2float(b) * c1 + __high2float(a) * s1);
}

// ------------------------------------------------------------------------------------------------
// One (entry, kv head, key range) unit of the fused decode attention, run by WARPS warps whose
// threads are numbered tid = 0 .. WARPS*32-1 and meet at sync().  It is the body of
// attention_decode_fused_kernel (8 warps, or 4 where that lets all CTAs run at once; 16-key tiles,
// three stages per warp).  Position encoding of q and the new k, the write of the new key and
// value into the pages, attention over the unit's key range, the merge of the warps, and the merge
// of the ranges by the unit that counts itself in last (nobody waits).  Rotation as in
// rope_cache.cu (reference src/qwen25vl_lite/rope.py:48-96).
//
// Shared memory (decode_unit_smem bytes): (cos, sin) of the token's angles | a flag | the warps'
// tiles, reused for the merge of the warps.
// ------------------------------------------------------------------------------------------------
template <int D, int WARPS, int BN, int STAGES>
struct DecodeUnit {
  static constexpr int P = Tile<D>::PITCH;
  static constexpr int TILE = BN * P;
  static constexpr int HALF = D / 2;
  static constexpr int TILES_OFF = 1024;
  static constexpr int KV_BYTES = WARPS * STAGES * 2 * TILE;
  static constexpr int SLAB_P = D + 8;                 // floats per row of a warp's output in the merge: the rows of a quad's lanes fall into different banks
  static constexpr int MERGE_BYTES = (WARPS * 16 * 2 + WARPS * 16 * SLAB_P + 16 * 2) * (int)sizeof(float);
  static constexpr int SMEM = TILES_OFF + (KV_BYTES > MERGE_BYTES ? KV_BYTES : MERGE_BYTES);
  static_assert(D % 32 == 0, "the rotation pairs channel j with j + D/2 inside one thread");
  static_assert(HALF * 8 + 16 <= TILES_OFF, "the angles and the flag fit before the tiles");

  struct Range { int seq, token, p, lo, first_tile_key, n_tiles, t_begin, t_end; const int* table; };

  __device__ static __forceinline__ Range range(const AttnArgs& a, int item, int split) {
    Range R;
    R.seq = a.items ? a.items[item] : item;              // without the list: one trip to memory less
    R.token = a.items ? a.cu_q[R.seq] : item;
    R.p = a.q_start_pos[R.seq];
    R.lo = a.window > 0 ? max(0, R.p - a.window + 1) : 0;
    R.first_tile_key = R.lo & ~(BN - 1);
    R.n_tiles = (R.p - R.first_tile_key) / BN + 1;
    const int per_split = (R.n_tiles + a.n_splits - 1) / a.n_splits;
    R.t_begin = split * per_split;
    R.t_end = min(R.n_tiles, R.t_begin + per_split);
    R.table = a.block_table + (size_t)R.seq * a.table_width;
    return R;
  }

  // Starts the copies of each warp's first tiles (all stages but one; with one stage, that one).
  // They read only keys and values of earlier steps, so a caller may issue them before the kernel
  // (or operation) that produces q has finished.
  static constexpr int AHEAD = STAGES > 1 ? STAGES - 1 : 1;
  __device__ static __forceinline__ void prefetch(const AttnArgs& a, int item, int kvh, int split, unsigned char* smem, int tid) {
    prefetch(a, range(a, item, split), kvh, smem, tid);
  }
  __device__ static __forceinline__ void prefetch(const AttnArgs& a, const Range& R, int kvh, unsigned char* smem, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    unsigned char* wbuf = smem + TILES_OFF + (size_t)warp * STAGES * 2 * TILE;
    if (BN == 16 && a.page_shift >= 4) {               // one page per tile: all look-ups first, then all copies
      int page[AHEAD];
#pragma unroll
      for (int s = 0; s < AHEAD; ++s) {
        const int tile = R.t_begin + warp + s * WARPS;
        page[s] = tile < R.t_end ? R.table[min(R.first_tile_key + tile * BN, R.p) >> a.page_shift] : 0;
      }
#pragma unroll
      for (int s = 0; s < AHEAD; ++s) {
        const int tile = R.t_begin + warp + s * WARPS;
        unsigned char* sb = wbuf + (size_t)s * 2 * TILE;
        if (tile < R.t_end) {
          BlockCopy<D> bc;
          bc.set(sb, sb + TILE, a, page[s], kvh, R.first_tile_key + tile * BN, R.p, lane);
          bc.all();
        }
        cp_async_commit();
      }
      return;
    }
#pragma unroll
    for (int s = 0; s < AHEAD; ++s) {
      const int tile = R.t_begin + warp + s * WARPS;
      unsigned char* sb = wbuf + (size_t)s * 2 * TILE;
      if (tile < R.t_end) load_kv_tile<D, BN, 32>(sb, sb + TILE, a, R.table, kvh, R.first_tile_key + tile * BN, R.p, lane);
      cp_async_commit();
    }
  }

  // What does not depend on the kernel before this one comes first: the entry's position and block
  // table (step metadata, copied before any kernel of the step ran) and the copies of the first
  // tiles of keys and values (written by earlier steps).  wait() then waits for that kernel
  // (programmatic dependent launch: this prologue overlaps its tail), and q, the token's own key and
  // value and the angles are asked for together: one trip to memory.
  template <typename Sync, typename Wait>
  __device__ static __forceinline__ void run(const AttnArgs& a, const RopeArgs& r, int item, int kvh, int split,
                                             unsigned char* smem, int tid, Sync sync, Wait wait) {
    constexpr int NT = WARPS * 32;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int G = a.nq / a.nkv;
    const Range R = range(a, item, split);
    const int token = R.token;
    const int slot_new = r.kv_slot[token];
    prefetch(a, R, kvh, smem, tid);
    wait();
    // q of the group's heads, rotated in registers later: channels j and j + D/2 sit in k-steps ks and
    // ks + D/32 of the same thread
    unsigned qf[D / 16][4];
    const bf16* qbase = a.qkv + (size_t)token * a.qkv_stride + (size_t)kvh * G * D;
    load_q<D>(qf, [&](int row) { return row < G ? qbase + (size_t)row * D : (const bf16*)nullptr; });
    // the token's own key and value: the unit that holds the last tile patches them into it
    constexpr int KI = (HALF + 31) / 32, VI = (D + 31) / 32;
    const bf16* kv_new = a.qkv + (size_t)token * a.qkv_stride + (size_t)(a.nq + kvh) * D;
    const unsigned short* kraw = reinterpret_cast<const unsigned short*>(kv_new);
    const unsigned short* vraw = reinterpret_cast<const unsigned short*>(kv_new + (size_t)a.nkv * D);
    unsigned short k1_new[KI], k2_new[KI], v_newv[VI];
#pragma unroll
    for (int i = 0; i < KI; ++i) {
      const int j = lane + 32 * i;
      k1_new[i] = j < HALF ? __ldcg(kraw + j) : (unsigned short)0;
      k2_new[i] = j < HALF ? __ldcg(kraw + j + HALF) : (unsigned short)0;
    }
#pragma unroll
    for (int i = 0; i < VI; ++i) v_newv[i] = lane + 32 * i < D ? __ldcg(vraw + lane + 32 * i) : (unsigned short)0;
    // the token has D/2 angles; from the step's table, or computed below once for the whole unit
    float2 angle_of_tid = make_float2(1.f, 0.f);
    if (r.angles && tid < HALF) angle_of_tid = __ldcg(r.angles + (size_t)token * HALF + tid);

    const int p = R.p, lo = R.lo;
    float2* cs = reinterpret_cast<float2*>(smem);
    int* is_last = reinterpret_cast<int*>(smem + HALF * 8);
    unsigned char* wbuf = smem + TILES_OFF + (size_t)warp * STAGES * 2 * TILE;
    int tile = R.t_begin + warp;
    for (int j = tid; j < HALF; j += NT) {
      if (r.angles) {
        cs[j] = j == tid ? angle_of_tid : __ldcg(r.angles + (size_t)token * HALF + j);
      } else {
        // all five loads are independent of one another, so they cost one memory latency, not two
        const int ax = r.axis[j];
        const float p0 = (float)r.positions[token], p1 = (float)r.positions[(size_t)r.n_tokens + token],
                    p2 = (float)r.positions[(size_t)2 * r.n_tokens + token];
        const float pj = ax == 0 ? p0 : (ax == 1 ? p1 : p2);
        float sn, c;
        sincosf(pj * r.inv_freq[j], &sn, &c);
        cs[j] = make_float2(c, sn);
      }
    }
    sync();
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
    // With one page per tile the page of the tile to ask for next is looked up an iteration before
    // it is needed: asked for in the same iteration, the copies would wait for the trip to the table.
    const bool page_per_tile = STAGES >= 2 && BN == 16 && a.page_shift >= 4;
    int page_ahead = 0;
    if (page_per_tile && tile + AHEAD * WARPS < R.t_end)
      page_ahead = R.table[min(R.first_tile_key + (tile + AHEAD * WARPS) * BN, p) >> a.page_shift];
    for (; tile < R.t_end; tile += WARPS) {
      const int next = tile + AHEAD * WARPS;
      if constexpr (STAGES >= 2) {
        const int ns = stage + STAGES - 1 >= STAGES ? stage - 1 : stage + STAGES - 1;
        unsigned char* nb = wbuf + (size_t)ns * 2 * TILE;
        if (next < R.t_end) {
          if (page_per_tile) {
            BlockCopy<D> bc;
            bc.set(nb, nb + TILE, a, page_ahead, kvh, R.first_tile_key + next * BN, p, lane);
            bc.all();
          } else {
            load_kv_tile<D, BN, 32>(nb, nb + TILE, a, R.table, kvh, R.first_tile_key + next * BN, p, lane);
          }
        }
        cp_async_commit();
        if (page_per_tile && next + WARPS < R.t_end)
          page_ahead = R.table[min(R.first_tile_key + (next + WARPS) * BN, p) >> a.page_shift];
        cp_async_wait<STAGES - 1>();
      } else {
        cp_async_wait<0>();
      }
      __syncwarp();
      const int key0 = R.first_tile_key + tile * BN;
      unsigned char* cb = wbuf + (size_t)stage * 2 * TILE;
      if (tile == R.n_tiles - 1) {
        // the token's own key and value: rotate k, patch both into the tile, store both to the pages
        const int slot = slot_new;
        const size_t page_off = slot >= 0 ? ((((size_t)(slot >> a.page_shift) * a.nkv + kvh) << a.page_shift)
                                             + (slot & ((1 << a.page_shift) - 1))) * D : 0;
        bf16* krow = reinterpret_cast<bf16*>(cb + (p - key0) * P);
        bf16* vrow = reinterpret_cast<bf16*>(cb + TILE + (p - key0) * P);
#pragma unroll
        for (int i = 0; i < KI; ++i) {
          const int j = lane + 32 * i;
          if (j < HALF) {
            const float cj = cs[j].x, sn = cs[j].y;
            const float x1 = __bfloat162float(__ushort_as_bfloat16(k1_new[i]));
            const float x2 = __bfloat162float(__ushort_as_bfloat16(k2_new[i]));
            const bf16 y1 = __float2bfloat16_rn(x1 * cj - x2 * sn), y2 = __float2bfloat16_rn(x2 * cj + x1 * sn);
            krow[j] = y1;
            krow[j + HALF] = y2;
            if (slot >= 0) {
              r.kpages_w[page_off + j] = y1;
              r.kpages_w[page_off + j + HALF] = y2;
            }
          }
        }
#pragma unroll
        for (int i = 0; i < VI; ++i) {
          const int c = lane + 32 * i;
          if (c < D) {
            const bf16 v = __ushort_as_bfloat16(v_newv[i]);
            vrow[c] = v;
            if (slot >= 0) r.vpages_w[page_off + c] = v;
          }
        }
        __syncwarp();
      }
      const bool need_mask = key0 < lo || key0 + BN - 1 > p;
      attend_tile<D, BN>(qf, cb, cb + TILE, key0, lo, p, lo, p, need_mask, a.scale_log2, m, l, o);
      __syncwarp();
      if constexpr (STAGES >= 2) {
        stage = stage + 1 == STAGES ? 0 : stage + 1;
      } else {
        if (next < R.t_end) load_kv_tile<D, BN, 32>(wbuf, wbuf + TILE, a, R.table, kvh, R.first_tile_key + next * BN, p, lane);
        cp_async_commit();
      }
    }
    cp_async_wait<0>();
    l[0] = quad_sum(l[0]);
    l[1] = quad_sum(l[1]);

    // merge the warps of the unit, keep the result in shared memory
    sync();
    float* ml = reinterpret_cast<float*>(smem + TILES_OFF);     // [WARPS][16 rows][2]
    float* slab = ml + WARPS * 16 * 2;                          // [WARPS][16 rows][SLAB_P]
    if (t == 0) {
      ml[(warp * 16 + g) * 2] = m[0];
      ml[(warp * 16 + g) * 2 + 1] = l[0];
      ml[(warp * 16 + g + 8) * 2] = m[1];
      ml[(warp * 16 + g + 8) * 2 + 1] = l[1];
    }
    sync();
    float f[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = g + 8 * h;
      float mm = -INFINITY;
      for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, ml[(w * 16 + row) * 2]);
      f[h] = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - mm);
    }
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) {
      float* r0 = slab + ((size_t)warp * 16 + g) * SLAB_P + nb * 8 + 2 * t;
      float* r1 = slab + ((size_t)warp * 16 + g + 8) * SLAB_P + nb * 8 + 2 * t;
      r0[0] = o[nb][0] * f[0];
      r0[1] = o[nb][1] * f[0];
      r1[0] = o[nb][2] * f[1];
      r1[1] = o[nb][3] * f[1];
    }
    // the rows' maxima and sums over the warps, once per row
    float* rowstat = slab + WARPS * 16 * SLAB_P;                // [16 rows][2]
    if (tid < 16) {
      float mm = -INFINITY;
      for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, ml[(w * 16 + tid) * 2]);
      float lsum = 0.f;
      for (int w = 0; w < WARPS; ++w) {
        const float mw = ml[(w * 16 + tid) * 2];
        lsum += mw == -INFINITY ? 0.f : ml[(w * 16 + tid) * 2 + 1] * exp2f(mw - mm);
      }
      rowstat[2 * tid] = mm;
      rowstat[2 * tid + 1] = lsum;
    }
    sync();
    for (int idx = tid; idx < G * (D / 4); idx += NT) {         // four channels of a row
      const int row = idx / (D / 4), c = (idx - row * (D / 4)) * 4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int w = 0; w < WARPS; ++w) {
        const float4 v = *reinterpret_cast<const float4*>(slab + ((size_t)w * 16 + row) * SLAB_P + c);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      const float mm = rowstat[2 * row], lsum = rowstat[2 * row + 1];
      const int head = kvh * G + row;
      if (a.n_splits == 1) {
        const float inv = 1.0f / lsum;
        uint2 packed;
        packed.x = pack_bf16(acc.x * inv, acc.y * inv);
        packed.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(a.out + (size_t)token * a.nq * D + (size_t)head * D + c) = packed;
      } else {
        const size_t pi = ((size_t)item * a.nq + head) * a.n_splits + split;
        *reinterpret_cast<float4*>(a.part_o + pi * D + c) = acc;
        if (c == 0) {
          a.part_ml[pi * 2] = mm;
          a.part_ml[pi * 2 + 1] = lsum;
        }
      }
    }
    if (a.n_splits == 1) return;

    // merge the ranges: every unit counts itself in after its partial is written; the one that finds
    // all the others already counted reads their partials and writes the output.  Nobody waits.
    // One thread counts for the unit with an acquire-release add: the barrier before it puts the other
    // threads' partials before the add, the barrier after it puts their reads of the others' partials
    // after it (a fence by every thread on both sides cost half a microsecond more).
    sync();
    if (tid == 0) {
      int done;
      asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;\n" : "=r"(done) : "l"(r.counters + item * a.nkv + kvh) : "memory");
      *is_last = done == a.n_splits - 1;
      if (*is_last) r.counters[item * a.nkv + kvh] = 0;            // ready for the next launch
    }
    sync();
    if (!*is_last) return;
    // A thread merges four channels of one row over all ranges.  The partials of 16 ranges are asked
    // for together (one trip to L2 for all of them), then weighted by exp2(m_k - M) and added in
    // order; with more than 16 ranges the running maximum is carried as in the attention loop itself.
    const int n4 = G * (D / 4);
    for (int e = tid; e < n4; e += NT) {
      const int row = e / (D / 4), c4 = e - row * (D / 4);
      const size_t base = ((size_t)item * a.nq + kvh * G + row) * a.n_splits;
      const float2* ml_row = reinterpret_cast<const float2*>(a.part_ml) + base;
      float M = -INFINITY, L = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k0 = 0; k0 < a.n_splits; k0 += 16) {
        float2 mlk[16];
        float4 po[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int kk = min(k0 + j, a.n_splits - 1);                  // always a readable address
          mlk[j] = __ldcg(ml_row + kk);
          po[j] = __ldcg(reinterpret_cast<const float4*>(a.part_o + (base + kk) * D) + c4);
        }
        float mb = -INFINITY;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (k0 + j < a.n_splits) mb = fmaxf(mb, mlk[j].x);
        const float Mn = fmaxf(M, mb);
        const float keep = M == -INFINITY ? 0.f : exp2f(M - Mn);
        acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
        L *= keep;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (k0 + j >= a.n_splits || mlk[j].x == -INFINITY) continue;
          const float w = exp2f(mlk[j].x - Mn);
          L += mlk[j].y * w;
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
};

// Fills the arguments that every attention entry point shares; returns a cudaError_t.
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
