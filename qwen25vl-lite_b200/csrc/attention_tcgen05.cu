// Prefill attention over the paged cache on the 5th-generation tensor cores (tcgen05), head size 128.
//
// Same formula and masking as the other attention kernels (reference src/qwen25vl_lite/text.py:78,
// 156-175, src/qwen25vl_lite/attention.py:143-148): S = Q K^T * D^-1/2, a query at position a sees
// keys j <= a (and j > a - window), softmax over the keys in float, O = P V.
//
// A CTA takes 128 rows = (token, query head of one kv group) pairs of one entry, so one pass over a
// kv head's keys serves the whole group, and walks the keys in tiles of 64.  Its threads have two
// roles that meet only at mbarriers:
//   * the row threads, one per row (= one lane of tensor memory): they copy Q (once) and the K and V
//     tiles from their pages into shared memory by 16-byte cp.async, in the 128-byte-swizzled layout
//     the tensor core reads (rows of 64 values, 8 rows per 1 KB atom, chunk c of row r at c ^ (r % 8));
//     they read their 64 scores of a tile with tcgen05.ld, do the running softmax alone (no
//     shuffles), and write their row of P as bfloat16 pairs back into the tensor-memory columns the
//     scores came from;
//   * one thread of the warp after them issues tcgen05.mma: S[128 x 64] = Q . K^T (both operands
//     K-major in shared memory, 8 steps of 16 over the head size) into one of two score
//     buffers in tensor memory, and O[128 x 128] += P . V with P read from tensor memory and V read
//     as it lies (a row of 128 head-size values per key: the MN-major operand form, 64-value halves
//     8 KB apart, groups of 8 keys 1 KB apart).
// The scores of tile t + 1 are computed while the rows work on tile t; a row asks for K(t + 2) and
// V(t) when tile t begins and waits for them when its softmax of tile t is done, so in the steady
// state it waits for no product and no copy.  The output accumulates in tensor memory over all
// tiles; the exponentials use a lazy maximum (see below), so it is rescaled only rarely.
// A step takes as long as its longest walk, so where a step has few row tiles the host cuts their keys
// (ops/attention.py: cut_keys).  Either into parts: a CTA then walks one part and leaves its
// unnormalised output rows with their maxima and sums in scratch memory, and
// attention_prefill_merge_kernel adds the parts of a tile up, in the order of the parts.  Or between
// the two CTAs of a cluster, which take half of a tile's keys each and add up through the cluster's
// shared memory.
// Two CTAs fit an SM (99 KB of shared memory, 256 of the 512 tensor-memory columns each).  (Two row
// tiles to a CTA, which halve the key and value traffic per row, were slower at every length tried:
// 8,192 tokens 375 against 298 us.  So were two threads to a row, 32 keys of a tile each, their maxima
// exchanged through shared memory: 2,048 tokens 60 against 45 us, 8,192 tokens 575 against 291 us.)
//
// Every mbarrier wait is bounded; a wait that gives up records a code in *err, and the CTA runs to
// its end (freeing its tensor memory) with invalid output.  A parity wait cannot tell "not yet" from
// "two phases on", so every wait here is provably within one phase of its barrier.
#include "attention_decode.cuh"
#include "tcgen05.cuh"

#define A5_ROWS 128
#define A5_NROW 128                          // row threads
#define A5_THREADS (A5_NROW + 32)             // and the warp that issues the products
#define A5_BN 64
#define A5_D 128
#define A5_Q_BYTES (2 * A5_ROWS * 128)            // Q: two 64-value halves of 128 rows
#define A5_KV_BYTES (2 * A5_BN * 128)             // two halves of 64 keys
#define A5_SMEM (A5_Q_BYTES + 4 * A5_KV_BYTES + 2048 + 1024)  // Q, two K and two V tiles, barriers and key rows, room to align

// 2^x on the special-function unit (exact enough for probabilities that are rounded to bfloat16; 2^-inf = 0).
__device__ __forceinline__ float a5_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// The larger of three (one instruction on sm_100).
__device__ __forceinline__ float a5_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Byte offset of the 16-byte chunk c (0..7) of row r inside a swizzled block of 128-byte rows.
__device__ __forceinline__ int a5_swz(int r, int c) { return (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4); }

// Where key kidx of a kv head lies: its row in the pages seen as [rows, D]; -1 past last_key.
__device__ __forceinline__ int a5_key_row(const AttnArgs& a, const int* __restrict__ table, int kvh, int kidx, int last_key) {
  if (kidx > last_key) return -1;
  return (((__ldg(table + (kidx >> a.page_shift)) * a.nkv + kvh) << a.page_shift)) + (kidx & ((1 << a.page_shift) - 1));
}

// The same for pages of 16 tokens or more, where a block of 16 keys of a tile is 4 KB in one piece:
// warp w copies block w, every lane 8 pieces of 16 bytes at
// block + (lane + 32 j) * 16, so a copy's addresses are one base and constants (copies whose
// addresses each take a 64-bit multiply-add cost the warp three times as long to issue).
// block_row: the row of the block's first key in the pages seen as [rows, D]; n_valid: how many of
// its 16 keys exist (the others are filled with zeros).
__device__ __forceinline__ void a5_load_block(unsigned char* dst_tile, const bf16* __restrict__ pages, int block_row, int n_valid,
                                              int warp, int lane) {
  constexpr int PER = 8;                               // copies per lane
  const int blk = warp & 3, j0 = 0;
  const int h = lane >> 4, cc = lane & 15;
  const unsigned char* src = reinterpret_cast<const unsigned char*>(pages + (size_t)block_row * A5_D) + lane * 16;
  unsigned char* dst = dst_tile + (cc >> 3) * (A5_BN * 128) + blk * 2048 + h * 128;
  const int x = ((cc & 7) ^ h) << 4;
#pragma unroll
  for (int jj = 0; jj < PER; ++jj) {
    const int j = j0 + jj;                             // key of the block: h + 2 j; its row in the tile: 16 blk + h + 2 j
    const int r7 = (2 * jj) & 7;                       // (row % 8) without h
    cp_async16(dst + (j >> 2) * 1024 + r7 * 128 + (x ^ (r7 << 4)), src + j * 512, h + 2 * j < n_valid);
  }
}

// A tile of 64 keys from their pages into a swizzled tile (zeros for rows[key] < 0): 1,024 copies
// of 16 bytes shared among the row threads.  rows: the 64 keys' rows, in shared memory.
__device__ __forceinline__ void a5_load_tile(unsigned char* dst_tile, const bf16* __restrict__ pages, const int* rows, int tid) {
  constexpr int N = A5_BN * 16 / A5_NROW;
  // all rows first: the copies are volatile statements, and a read between two of them would wait for its turn
  int row[N];
#pragma unroll
  for (int i = 0; i < N; ++i) row[i] = rows[(tid + i * A5_NROW) >> 4];
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const int idx = tid + i * A5_NROW;
    const int key = idx >> 4, cc = idx & 15;
    cp_async16(dst_tile + (cc >> 3) * (A5_BN * 128) + a5_swz(key, cc & 7), pages + (size_t)max(row[i], 0) * A5_D + cc * 8, row[i] >= 0);
  }
}

struct A5Bars {
  unsigned long long s_full[2];   // scores of a tile are in their buffer (one arrival: tcgen05.commit)
  unsigned long long k_full[2];   // a K tile has landed (every row thread arrives for its copies)
  unsigned long long pv_ready[2]; // P of a tile is in tensor memory and its V tile has landed (every row thread); two, since
                                  // a row may be a tile ahead of another: the scores of the next tile are there early
  unsigned long long pv_done[2];  // the product P V of a tile is done (tcgen05.commit); two, so that a wait is never
                                  // two phases away from its barrier, where a parity wait would be wrong
  unsigned tmem;
};

__global__ void __launch_bounds__(A5_THREADS, 2) attention_prefill_tcgen05_kernel(AttnArgs a, int n_sms, int* __restrict__ err) {
  constexpr int NROW = A5_NROW, ROWS = A5_ROWS;         // one thread per row; the warp after them issues the products
  constexpr int TMEM_COLS = 256, O_COL = 128;           // two score buffers of 64 columns, then the outputs
  pdl_trigger();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + A5_Q_BYTES;                  // two K tiles
  unsigned char* v_s = k_s + 2 * A5_KV_BYTES;             // two V tiles
  A5Bars* bars = reinterpret_cast<A5Bars*>(v_s + 2 * A5_KV_BYTES);
  int* key_rows = reinterpret_cast<int*>(v_s + 2 * A5_KV_BYTES + 128);   // [4 tiles][64 keys]: see below

  const int tid = threadIdx.x, warp = tid >> 5;
  // Which (row tile, kv head) this CTA takes.  The list comes heaviest first.  Two CTAs share an SM
  // and its throughput, and the first 148 CTAs of a grid go one to each SM, the next 148 join them in
  // the same order: with 149 to 296 CTAs in all, CTA 148 + s therefore takes the s-th lightest piece
  // of work, so that every SM gets a heavy and a light one (2,048 tokens in 256 pieces: the busiest
  // SM has 34 key tiles instead of 61).  Larger grids are taken in order: CTAs start as others end.
  // Launched as clusters of two CTAs, a cluster takes a piece of work (in the list's order): a tile
  // of code 2 half of its keys each, the second CTA leaving its rows in its shared memory for the
  // first to add up; a whole tile (code 1) the first CTA alone.
  unsigned n_rank, rank;
  asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(n_rank));
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
  const bool pair = n_rank == 2;
  const int n_work = pair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int work = pair ? (int)(blockIdx.x >> 1)
                        : ((n_work > n_sms && n_work <= 2 * n_sms && (int)blockIdx.x >= n_sms)
                               ? n_work - 1 - ((int)blockIdx.x - n_sms) : (int)blockIdx.x);
  const int item = work / a.nkv, kvh = work - item * a.nkv;
  const int seq = a.items[3 * item], row_tile = a.items[3 * item + 1], code = a.items[3 * item + 2];
  const int n_parts = code & 15, first_part = code >> 8;                            // 1 part: the whole tile
  const int part = pair ? (int)rank : (code >> 4) & 15;
  if (pair && n_parts == 1 && rank == 1) return;                                    // nothing for the second CTA
  const int G = a.nq / a.nkv;
  const int q0 = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q0, start = a.q_start_pos[seq];
  const int n_rows = q_len * G;
  const int R0 = row_tile * ROWS;
  const int* table = a.block_table + (size_t)seq * a.table_width;
  // key range of the CTA
  const int c_first = R0 / G, c_last = min(R0 + ROWS - 1, n_rows - 1) / G;
  int c_hi = start + c_last;                               // the last key anybody of the CTA sees: nothing is loaded past it
  const int c_lo = a.window > 0 ? max(0, start + c_first - a.window + 1) : 0;
  int key_begin = c_lo & ~(A5_BN - 1);
  int n_tiles = (c_hi - key_begin) / A5_BN + 1;
  if (n_parts > 1) {                                       // this CTA's part of the key tiles
    const int per = (n_tiles + n_parts - 1) / n_parts;
    const int t0 = part * per, t1 = min(n_tiles, t0 + per);
    if (t1 < n_tiles) c_hi = key_begin + t1 * A5_BN - 1;
    key_begin += t0 * A5_BN;
    n_tiles = t1 - t0;
  }

  if (tid == 0) {
    mbar_init(bars->s_full, 1);
    mbar_init(bars->s_full + 1, 1);
    mbar_init(bars->k_full, NROW);
    mbar_init(bars->k_full + 1, NROW);
    mbar_init(bars->pv_ready, NROW);
    mbar_init(bars->pv_ready + 1, NROW);
    mbar_init(bars->pv_done, 1);
    mbar_init(bars->pv_done + 1, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == NROW / 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars->tmem)), "n"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }

  // this thread's row (threads of the last warp have none)
  const int R = R0 + tid;
  const bool live = tid < NROW && R < n_rows;
  const int tok = live ? R / G : 0, head = live ? R - tok * G : 0;
  const int hi = live ? start + tok : -1;
  const int lo = live ? (a.window > 0 ? max(0, hi - a.window + 1) : 0) : 0;

  // Where the keys lie.  The page lookup is a trip to the L2, so it runs three tiles ahead: the
  // lanes of a warp that stand first look up the rows of the keys that their warp copies (key
  // (tid + i * NROW) / 16 for copy i), when tile t begins for tile t + 3, and leave them in shared
  // memory when it ends; the warp reads them a tile later for K and three tiles later for V.
  // Writers and readers are lanes of one warp, so __syncwarp orders them.
  // With pages of 16 tokens or more a warp needs one row per tile, that of its block of 16 keys:
  // every lane keeps those of the tiles t, t + 1 and t + 2 in registers and asks for the page of t + 3.
  constexpr int N_COPIES = A5_BN * 16 / NROW;
  const int lane = tid & 31;
  const bool blocks = a.page_shift >= 4;
  const int block_key = key_begin + 16 * (warp & 3);                          // first key of this warp's block in tile 0
  auto block_row = [&](int page, int kfirst) { return ((page * a.nkv + kvh) << a.page_shift) + (kfirst & ((1 << a.page_shift) - 1)); };
  auto block_valid = [&](int kfirst) { return min(max(c_hi - kfirst + 1, 0), 16); };
  int rb0 = 0, rb1 = 0, rb2 = 0;
  if (blocks && tid < NROW) {
    const int k0 = block_key, k1 = block_key + A5_BN, k2 = block_key + 2 * A5_BN;
    const int p0 = k0 <= c_hi ? __ldg(table + (k0 >> a.page_shift)) : 0;
    const int p1 = k1 <= c_hi ? __ldg(table + (k1 >> a.page_shift)) : 0;
    const int p2 = k2 <= c_hi ? __ldg(table + (k2 >> a.page_shift)) : 0;
    rb0 = k0 <= c_hi ? block_row(p0, k0) : 0;
    rb1 = k1 <= c_hi ? block_row(p1, k1) : 0;
    rb2 = k2 <= c_hi ? block_row(p2, k2) : 0;
  }
  const int my_key = 2 * warp + (lane & 1) + (NROW / 16) * (lane >> 1);      // for lanes < 2 * N_COPIES
  const bool looks_up = !blocks && tid < NROW && lane < 2 * N_COPIES;
  if (looks_up) {
#pragma unroll
    for (int j = 0; j < 3; ++j)
      if (j < n_tiles) key_rows[j * A5_BN + my_key] = a5_key_row(a, table, kvh, key_begin + j * A5_BN + my_key, c_hi);
  }
  __syncwarp();
  // Up to here the kernel has read the step's work list, lengths and block tables only, which came
  // with the step's copy from the host before any of its kernels; q, and the keys and values of the
  // step's own tokens, are what the kernels before this one wrote.
  pdl_wait();
  // The first two K tiles, the first V tile and Q.  After that a row asks for K(t + 2) and V(t) when
  // tile t begins and waits for them when its part of tile t is done, a softmax later: at its fence
  // nothing of its own is in flight.
  if (tid < NROW) {
    if (blocks) {
      a5_load_block(k_s, a.kpages, rb0, block_valid(block_key), warp, lane);
      if (n_tiles > 1) a5_load_block(k_s + A5_KV_BYTES, a.kpages, rb1, block_valid(block_key + A5_BN), warp, lane);
      a5_load_block(v_s, a.vpages, rb0, block_valid(block_key), warp, lane);
    } else {
      a5_load_tile(k_s, a.kpages, key_rows, tid);
      if (n_tiles > 1) a5_load_tile(k_s + A5_KV_BYTES, a.kpages, key_rows + A5_BN, tid);
      a5_load_tile(v_s, a.vpages, key_rows, tid);
    }
    cp_async_commit();
    const uint4* src = reinterpret_cast<const uint4*>(a.qkv + (size_t)(q0 + tok) * a.qkv_stride + (size_t)(kvh * G + head) * A5_D);
#pragma unroll
    for (int cc = 0; cc < 16; ++cc) {
      const uint4 v = live ? __ldcg(src + cc) : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(q_s + (cc >> 3) * (A5_ROWS * 128) + a5_swz(tid, cc & 7)) = v;
    }
    cp_async_wait<0>();
    tc5_proxy_fence();                                    // Q and this thread's part of K and V, visible to the tensor core
  }
  tc5_fence_before();
  __syncthreads();                                       // barriers initialised, tensor memory allocated
  tc5_fence_after();
  const unsigned tmem_base = bars->tmem;
  const unsigned idesc_s = tc5_idesc(A5_BN, false), idesc_pv = tc5_idesc(A5_D, true);
  bool ok = true;
  // Running softmax with a lazy maximum: the exponentials use m_used, which follows the true maximum
  // only when that has grown by more than 8 (a factor 256, far inside the range of bfloat16 and of
  // the float sums), so the output rows in tensor memory are read, scaled and written back only
  // on those rare occasions, not once per tile.
  float m_used = -INFINITY, l = 0.f;
  const unsigned t_lane = tmem_base + ((unsigned)((warp & 3) * 32) << 16);      // this warp's lanes: the score buffers
  const unsigned t_o = t_lane + O_COL;                                         // and the outputs

  if (tid == NROW) {
    // ---- the thread that issues the products ----
    auto scores = [&](int t) {                            // S(t) = Q . K(t)^T into score buffer t % 2
      const unsigned char* kt = k_s + (size_t)(t & 1) * A5_KV_BYTES;
#pragma unroll
      for (int ks = 0; ks < A5_D / 16; ++ks) {            // 16 values of the head size per step: 32 bytes along a row
        const unsigned long long ad = tc5_desc(smem_u32(q_s) + (ks >> 2) * (A5_ROWS * 128) + (ks & 3) * 32, 16, 1024);
        const unsigned long long bd = tc5_desc(smem_u32(kt) + (ks >> 2) * (A5_BN * 128) + (ks & 3) * 32, 16, 1024);
        tc5_mma(tmem_base + (unsigned)(t & 1) * A5_BN, ad, bd, idesc_s, ks != 0);
      }
      tc5_commit(bars->s_full + (t & 1));
    };
    auto fail = [&](int code) { ok = false; atomicExch(err, code); };
    if (!mbar_wait(bars->k_full, 0)) fail(21);
    tc5_fence_after();
    scores(0);
    if (n_tiles > 1) {
      if (ok && !mbar_wait(bars->k_full + 1, 0)) fail(21);
      tc5_fence_after();
      scores(1);
    }
    for (int t = 0; t < n_tiles; ++t) {
      if (ok && !mbar_wait(bars->pv_ready + (t & 1), (unsigned)(t >> 1) & 1)) fail(22);
      tc5_fence_after();
      const unsigned char* vt = v_s + (size_t)(t & 1) * A5_KV_BYTES;
#pragma unroll
      for (int ks = 0; ks < A5_BN / 16; ++ks) {           // 16 keys per step: 8 columns of P, 2 KB down V
        const unsigned long long bd = tc5_desc(smem_u32(vt) + ks * 2048, A5_BN * 128, 1024);
        tc5_mma_ts(tmem_base + O_COL, tmem_base + (unsigned)(t & 1) * A5_BN + ks * 8, bd, idesc_pv, (t | ks) != 0);
      }
      tc5_commit(bars->pv_done + (t & 1));
      if (t + 2 < n_tiles) {
        // the score buffer holds P(t) until this product is done; K(t + 2) was asked for a tile ago
        if (ok && !mbar_wait(bars->pv_done + (t & 1), (unsigned)(t >> 1) & 1)) fail(23);
        if (ok && !mbar_wait(bars->k_full + (t & 1), (unsigned)((t + 2) >> 1) & 1)) fail(21);
        tc5_fence_after();
        scores(t + 2);
      }
    }
  } else if (tid < NROW) {
    // ---- the rows ----
    mbar_arrive(bars->k_full);                         // K(0) and K(1), after the fence above
    if (n_tiles > 1) mbar_arrive(bars->k_full + 1);
    const int min_hi = start + c_first;                                       // the least any live row of the CTA sees
    const int max_lo = a.window > 0 ? max(0, start + c_last - a.window + 1) : 0;
    const bool all_live = R0 + ROWS <= n_rows;

    for (int tile = 0; tile < n_tiles; ++tile) {
      const int stage = tile & 1;
      const int key0 = key_begin + tile * A5_BN;
      if (ok && !mbar_wait(bars->s_full + stage, (unsigned)(tile >> 1) & 1)) {
        ok = false;
        atomicExch(err, 24);
      }
      tc5_fence_after();
      // K(t + 2) goes where K(t) was, which the scores are done with; V(t) where V(t - 2) was, whose
      // product was done before the scores of this tile were asked for
      const int kb = block_key + tile * A5_BN;             // this warp's block in this tile
      int row_ahead = -1, page_ahead = 0;                  // asked for now, used when the tile ends
      if (blocks) {
        if (tile + 2 < n_tiles)
          a5_load_block(k_s + (size_t)stage * A5_KV_BYTES, a.kpages, rb2, block_valid(kb + 2 * A5_BN), warp, lane);
        if (tile > 0) a5_load_block(v_s + (size_t)stage * A5_KV_BYTES, a.vpages, rb0, block_valid(kb), warp, lane);
        cp_async_commit();
        if (kb + 3 * A5_BN <= c_hi) page_ahead = __ldg(table + ((kb + 3 * A5_BN) >> a.page_shift));
      } else {
        if (tile + 2 < n_tiles)
          a5_load_tile(k_s + (size_t)stage * A5_KV_BYTES, a.kpages, key_rows + ((tile + 2) & 3) * A5_BN, tid);
        if (tile > 0) a5_load_tile(v_s + (size_t)stage * A5_KV_BYTES, a.vpages, key_rows + (tile & 3) * A5_BN, tid);
        cp_async_commit();
        if (looks_up && tile + 3 < n_tiles) row_ahead = a5_key_row(a, table, kvh, key0 + 3 * A5_BN + my_key, c_hi);
      }

      // this row's 64 scores
      float s[A5_BN];
      {
        float part[32];
        tc5_ld32(t_lane + stage * A5_BN, part);
#pragma unroll
        for (int j = 0; j < 32; ++j) s[j] = part[j];
        tc5_ld32(t_lane + stage * A5_BN + 32, part);
#pragma unroll
        for (int j = 0; j < 32; ++j) s[32 + j] = part[j];
      }
      const bool need_mask = !all_live || key0 + A5_BN - 1 > min_hi || key0 < max_lo;      // the same for the whole CTA
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < A5_BN; ++j) {
          const int kidx = key0 + j;
          s[j] = (kidx >= lo && kidx <= hi) ? s[j] : -INFINITY;
        }
      }
      float mx0 = a5_max3(s[0], s[1], s[2]), mx1 = a5_max3(s[3], s[4], s[5]);   // two chains of three-input maxima
#pragma unroll
      for (int j = 6; j + 3 < A5_BN; j += 4) {
        mx0 = a5_max3(mx0, s[j], s[j + 1]);
        mx1 = a5_max3(mx1, s[j + 2], s[j + 3]);
      }
      float mx = a5_max3(mx0, mx1, fmaxf(s[A5_BN - 2], s[A5_BN - 1]));
      mx *= a.scale_log2;                                  // the scale is positive: the maximum of the scaled scores
      const bool grow = mx > m_used + 8.0f || (m_used == -INFINITY && mx != -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float factor = grow ? (m_used == -INFINITY ? 0.f : a5_ex2(m_used - mx)) : 1.0f;
        if (grow) m_used = mx;
        l *= factor;
        if (tile > 0) {                                    // the rows in tensor memory follow (warp-wide: lanes that keep theirs multiply by 1)
          if (ok && !mbar_wait(bars->pv_done + (stage ^ 1), (unsigned)((tile - 1) >> 1) & 1)) {   // nobody adds to them meanwhile
            ok = false;
            atomicExch(err, 25);
          }
          tc5_fence_after();
#pragma unroll
          for (int c = 0; c < A5_D / 32; ++c) {
            float part[32];
            tc5_ld32(t_o + c * 32, part);
#pragma unroll
            for (int j = 0; j < 32; ++j) part[j] *= factor;
            tc5_st32(t_o + c * 32, part);
          }
        }
      }
      const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
      float sum = 0.f;
      unsigned w[A5_BN / 2];
#pragma unroll
      for (int e = 0; e < A5_BN / 2; ++e) {
        const float p0 = a5_ex2(fmaf(s[2 * e], a.scale_log2, neg_m));
        const float p1 = a5_ex2(fmaf(s[2 * e + 1], a.scale_log2, neg_m));
        sum += p0 + p1;
        w[e] = pack_bf16(p0, p1);
      }
      l += sum;
      tc5_st32u(t_lane + stage * A5_BN, w);                 // P where the scores were: 64 bfloat16 in 32 columns
      if (blocks) {
        rb0 = rb1;
        rb1 = rb2;
        rb2 = kb + 3 * A5_BN <= c_hi ? block_row(page_ahead, kb + 3 * A5_BN) : 0;
      } else {
        if (looks_up && tile + 3 < n_tiles) key_rows[((tile + 3) & 3) * A5_BN + my_key] = row_ahead;
        __syncwarp();
      }
      // the copies asked for when the tile began have had a softmax's time to land
      cp_async_wait<0>();
      tc5_proxy_fence();
      tc5_fence_before();
      if (tile + 2 < n_tiles) mbar_arrive(bars->k_full + stage);
      mbar_arrive(bars->pv_ready + stage);
    }
    if (ok && !mbar_wait(bars->pv_done + ((n_tiles - 1) & 1), (unsigned)((n_tiles - 1) >> 1) & 1)) {
      ok = false;
      atomicExch(err, 27);
    }
    tc5_fence_after();
  }

  // ---- the results ----
  if (pair && n_parts > 1) {
    // Two CTAs of a cluster with half of the keys each.  The second leaves its rows as they are, with
    // their maxima and sums, in its own shared memory (the K and V tiles are done with: 64 KB, value
    // quads of all rows side by side; maxima and sums where Q was); the first adds them to its own:
    // out = (w0 O0 + w1 O1) / (w0 l0 + w1 l1), w_p = 2^(m_p - max(m0, m1)).  The second CTA stays until
    // the first has read.
    if (rank == 1 && tid < NROW) {
#pragma unroll
      for (int c = 0; c < A5_D / 32; ++c) {
        float vals[32];
        tc5_ld32(t_o + c * 32, vals);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(k_s + (size_t)((c * 8 + q) * NROW + tid) * 16) = make_float4(vals[q * 4], vals[q * 4 + 1], vals[q * 4 + 2], vals[q * 4 + 3]);
      }
      *reinterpret_cast<float2*>(q_s + tid * 8) = make_float2(m_used, l);
    }
    cluster_sync();
    if (rank == 0 && tid < NROW) {
      const unsigned peer_o = cluster_map(smem_u32(k_s), 1), peer_ml = cluster_map(smem_u32(q_s), 1);
      float m1, l1;
      asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];\n" : "=f"(m1), "=f"(l1) : "r"(peer_ml + tid * 8) : "memory");
      const float M = fmaxf(m_used, m1);
      const float w0 = m_used == -INFINITY ? 0.f : a5_ex2(m_used - M), w1 = m1 == -INFINITY ? 0.f : a5_ex2(m1 - M);
      const float L = l * w0 + l1 * w1;
      const float inv = live && L > 0.f ? 1.0f / L : 0.f;
      const float s0 = w0 * inv, s1 = w1 * inv;
      bf16* dst = a.out + (size_t)(q0 + tok) * a.nq * A5_D + (size_t)(kvh * G + head) * A5_D;
#pragma unroll
      for (int c = 0; c < A5_D / 32; ++c) {
        float mine[32], theirs[32];
        tc5_ld32(t_o + c * 32, mine);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                       : "=f"(theirs[q * 4]), "=f"(theirs[q * 4 + 1]), "=f"(theirs[q * 4 + 2]), "=f"(theirs[q * 4 + 3])
                       : "r"(peer_o + (unsigned)((c * 8 + q) * NROW + tid) * 16) : "memory");
        if (!live) continue;
#pragma unroll
        for (int j = 0; j < 32; ++j) mine[j] = mine[j] * s0 + theirs[j] * s1;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o;
          o.x = pack_bf16(mine[q * 8], mine[q * 8 + 1]);
          o.y = pack_bf16(mine[q * 8 + 2], mine[q * 8 + 3]);
          o.z = pack_bf16(mine[q * 8 + 4], mine[q * 8 + 5]);
          o.w = pack_bf16(mine[q * 8 + 6], mine[q * 8 + 7]);
          *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = o;
        }
      }
    }
    cluster_sync();
  } else if (tid < NROW) {
    if (n_parts > 1) {
      // a part of the keys: the sums as they are, with the maximum they were taken against and the
      // sum of the weights, for the merge kernel
      const size_t slot = ((size_t)(first_part + part) * a.nkv + kvh) * ROWS + tid;
      float* po = a.part_o + slot * A5_D;
#pragma unroll
      for (int c = 0; c < A5_D / 32; ++c) {
        float vals[32];
        tc5_ld32(t_o + c * 32, vals);
        if (!live) continue;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(po + c * 32 + q * 4) = make_float4(vals[q * 4], vals[q * 4 + 1], vals[q * 4 + 2], vals[q * 4 + 3]);
      }
      if (live) *reinterpret_cast<float2*>(a.part_ml + slot * 2) = make_float2(m_used, l);
    } else {
    const float inv = live && l > 0.f ? 1.0f / l : 0.f;
    bf16* dst = a.out + (size_t)(q0 + tok) * a.nq * A5_D + (size_t)(kvh * G + head) * A5_D;
#pragma unroll
    for (int c = 0; c < A5_D / 32; ++c) {                 // tcgen05.ld is warp-wide: dead rows read too, and store nothing
      float part[32];
      tc5_ld32(t_o + c * 32, part);
      if (!live) continue;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack_bf16(part[q * 8] * inv, part[q * 8 + 1] * inv);
        o.y = pack_bf16(part[q * 8 + 2] * inv, part[q * 8 + 3] * inv);
        o.z = pack_bf16(part[q * 8 + 4] * inv, part[q * 8 + 5] * inv);
        o.w = pack_bf16(part[q * 8 + 6] * inv, part[q * 8 + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = o;
      }
    }
    }
  }
  // every thread gets here (all waits are bounded); then the tensor memory goes back
  tc5_fence_before();
  __syncthreads();
  if (warp == NROW / 32) {
    tc5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
  }
}

// Adds up the parts of the row tiles whose keys were cut.  merges: (entry, row tile, first part,
// parts).  The parts' maxima m_p
// (in the units of the exponent: scaled scores times log2 e) and sums l_p give the weights
// 2^(m_p - M), M the largest, and out = sum_p w_p O_p / sum_p w_p l_p, parts in order.  A warp takes
// one row (a lane four of its 128 values), a block 8 rows.
constexpr int A5_MERGE_WARPS = 8;
__global__ void __launch_bounds__(A5_MERGE_WARPS * 32, 4) attention_prefill_merge_kernel(AttnArgs a, const int* __restrict__ merges) {
  pdl_trigger();
  pdl_wait();
  constexpr int BLOCKS_PER_TILE = A5_ROWS / A5_MERGE_WARPS;
  const int work = blockIdx.x / BLOCKS_PER_TILE;
  const int item = work / a.nkv, kvh = work - item * a.nkv;
  const int seq = merges[4 * item], row_tile = merges[4 * item + 1], first_part = merges[4 * item + 2], n_parts = merges[4 * item + 3];
  const int G = a.nq / a.nkv;
  const int q0 = a.cu_q[seq], n_rows = (a.cu_q[seq + 1] - q0) * G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = (blockIdx.x - work * BLOCKS_PER_TILE) * A5_MERGE_WARPS + warp;
  const int R = row_tile * A5_ROWS + r;
  if (R >= n_rows) return;
  const int tok = R / G, head = R - tok * G;
  const size_t slot0 = ((size_t)first_part * a.nkv + kvh) * A5_ROWS + r, slot_step = (size_t)a.nkv * A5_ROWS;
  // lane p holds part p's (maximum, sum); then every lane takes its four values of five parts at a
  // time (a tile has five parts or fewer unless its step had very few tiles)
  float2 ml = make_float2(-INFINITY, 0.f);
  if (lane < n_parts) ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml) + slot0 + lane * slot_step);
  float M = ml.x;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
  const float w_mine = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);      // a part whose keys the row does not see brings nothing
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float L = 0.f;
  for (int p0 = 0; p0 < n_parts; p0 += 5) {
    float4 o[5];
#pragma unroll
    for (int k = 0; k < 5; ++k)
      if (p0 + k < n_parts) o[k] = __ldcg(reinterpret_cast<const float4*>(a.part_o + (slot0 + (p0 + k) * slot_step) * A5_D) + lane);
#pragma unroll
    for (int k = 0; k < 5; ++k) {
      const float w = __shfl_sync(0xffffffffu, w_mine, (p0 + k) & 31), lp = __shfl_sync(0xffffffffu, ml.y, (p0 + k) & 31);
      if (p0 + k < n_parts && w > 0.f) {
        L = fmaf(lp, w, L);
        acc.x = fmaf(o[k].x, w, acc.x); acc.y = fmaf(o[k].y, w, acc.y); acc.z = fmaf(o[k].z, w, acc.z); acc.w = fmaf(o[k].w, w, acc.w);
      }
    }
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  uint2 packed;
  packed.x = pack_bf16(acc.x * inv, acc.y * inv);
  packed.y = pack_bf16(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(a.out + (size_t)(q0 + tok) * a.nq * A5_D + (size_t)(kvh * G + head) * A5_D + lane * 4) = packed;
}

// tiles: (entry, row tile, code) triples with row tiles of 128 rows (code 1: the whole tile; else
// first part << 8 | part << 4 | parts: one of up to 15 parts of its keys); merges: (entry, row tile,
// first part, parts) of the n_merges tiles that were cut, scratch: n_tiles * nkv * 128 * (D + 2)
// floats when there are any.  pairs != 0: every piece of work goes to a cluster of two CTAs, and the
// codes are 1 (the whole tile, one CTA) or 2 (half of the keys each).  Otherwise the arguments of
// q25_attention_prefill_bf16.  Head size 128 only.  err: one int that receives a nonzero code if a
// wait gave up.
Q25_EXPORT int q25_attention_prefill_tcgen05_bf16(const void* qkv, int qkv_stride, void* out, const void* kp, const void* vp,
                                                  const int* bt, int tw, const int* cu_q, const int* q_start,
                                                  const int* tiles, int n_tiles, int nq, int nkv, int d, int page_size,
                                                  int window, float scale, const int* merges, int n_merges, float* scratch,
                                                  int pairs, int* err, void* stream) {
  if (n_tiles <= 0) return 0;
  if (d != A5_D || !err || (n_merges > 0 && (!merges || !scratch || window > 0 || pairs)) || (pairs && window > 0))
    return (int)cudaErrorInvalidValue;
  AttnArgs a;
  int e = fill_args(a, qkv, qkv_stride, out, kp, vp, bt, tw, cu_q, q_start, tiles, nq, nkv, page_size, window, scale);
  if (e) return e;
  if (((uintptr_t)qkv & 15) || (qkv_stride % 8) || ((uintptr_t)out & 15)) return (int)cudaErrorInvalidValue;
  cudaError_t ce = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A5_SMEM);
  if (ce != cudaSuccess) return (int)ce;
  a.part_o = scratch;                                    // [part, kv head, row, D], then [part, kv head, row, (m, l)]
  a.part_ml = scratch ? scratch + (size_t)n_tiles * nkv * A5_ROWS * A5_D : nullptr;
  launch_clusters(pairs ? 2 : 1, attention_prefill_tcgen05_kernel, dim3(n_tiles * nkv * (pairs ? 2 : 1)), dim3(A5_THREADS),
                  (size_t)A5_SMEM, (cudaStream_t)stream, a, device_sm_count(), err);
  if (n_merges > 0)
    launch(attention_prefill_merge_kernel, dim3(n_merges * nkv * (A5_ROWS / A5_MERGE_WARPS)), dim3(A5_MERGE_WARPS * 32), 0,
           (cudaStream_t)stream, a, merges);
  return launch_status();
}
