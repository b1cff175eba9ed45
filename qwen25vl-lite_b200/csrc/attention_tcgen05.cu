// Prefill attention over the paged cache on the 5th-generation tensor cores (tcgen05), head size 128.
//
// Same formula and masking as the other attention kernels (reference src/qwen25vl_lite/text.py:78,
// 156-175, src/qwen25vl_lite/attention.py:143-148): S = Q K^T * D^-1/2, a query at position a sees
// keys j <= a (and j > a - window), softmax over the keys in float, O = P V.
//
// A CTA takes 128 rows = (token, query head of one kv group) pairs of one entry, so one pass over a
// kv head's keys serves the whole group, and walks the keys in tiles of 64:
//   * Q (once) and every K and V tile are written to shared memory in the 128-byte-swizzled layout
//     that the tensor core reads: rows of 64 values (128 bytes), 8 rows per 1 KB atom, the 16-byte
//     chunk c of row r at chunk c ^ (r % 8).  K and V come from their pages by 16-byte cp.async.
//   * thread 0 issues tcgen05.mma: S[128 x 64] = Q . K^T (both operands K-major, 8 steps of 16 over
//     the head size) into tensor memory; every thread owns one row (one lane of tensor memory),
//     reads its 64 scores with tcgen05.ld, does the running softmax alone (no shuffles), and writes
//     its row of P as bfloat16 into shared memory, again swizzled;
//   * thread 0 issues O_tile[128 x 128] = P . V (P K-major; V is read as it lies, a row of 128
//     head-size values per key: the MN-major operand form, 64-value halves 8 KB apart, groups of 8 keys
//     1 KB apart) into a second accumulator; every thread adds its row of it, scaled by the
//     softmax correction, to the output row it keeps in registers.
// Two CTAs fit an SM (98 KB of shared memory, 256 of the 512 tensor-memory columns each), so one
// CTA's softmax runs under the other's products.  K/V tiles are double-buffered; P is written where
// the K tile was, which the tensor core has finished with once S is there.
//
// Every mbarrier wait is bounded; a wait that gives up records a code in *err, and the CTA runs to
// its end (freeing its tensor memory) with invalid output.
#include "attention_decode.cuh"

#define A5_ROWS 128
#define A5_BN 64
#define A5_D 128
#define A5_THREADS 128
#define A5_WAIT_LIMIT (1 << 22)
#define A5_Q_BYTES (2 * A5_ROWS * 128)            // two 64-value halves of 128 rows
#define A5_KV_BYTES (2 * A5_BN * 128)             // two halves of 64 keys
#define A5_SMEM (A5_Q_BYTES + 4 * A5_KV_BYTES + 1024 + 1024)  // P (128 rows x 128 bytes) takes the place of the K tile it came from

__device__ __forceinline__ unsigned a5_s32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void a5_mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(a5_s32(bar)), "r"(count));
}
__device__ __forceinline__ bool a5_mbar_wait(unsigned long long* bar, unsigned parity) {
  for (int i = 0; i < A5_WAIT_LIMIT; ++i) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(a5_s32(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
// Shared-memory matrix descriptor, 128-byte swizzle.  lbo / sbo in bytes.
__device__ __forceinline__ unsigned long long a5_desc(unsigned smem_addr, unsigned lbo, unsigned sbo) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3FFFF) >> 4);
  d |= (unsigned long long)(lbo >> 4) << 16;
  d |= (unsigned long long)(sbo >> 4) << 32;
  d |= (unsigned long long)1 << 46;                         // descriptor version of sm_100
  d |= (unsigned long long)2 << 61;                         // 128-byte swizzle
  return d;
}
// bf16 x bf16 -> f32, M 128, N n; b_mn: the B operand is MN-major (else K-major); A is K-major.
__device__ __forceinline__ unsigned a5_idesc(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) | ((unsigned)(A5_ROWS >> 4) << 24);
}
__device__ __forceinline__ void a5_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void a5_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(a5_s32(bar)) : "memory");
}
__device__ __forceinline__ void a5_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void a5_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void a5_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
// 32 consecutive float columns of this thread's lane of tensor memory.
__device__ __forceinline__ void a5_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The same 32 columns written back.
__device__ __forceinline__ void a5_st32(unsigned taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
// 2^x on the special-function unit (exact enough for probabilities that are rounded to bfloat16; 2^-inf = 0).
__device__ __forceinline__ float a5_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of the 16-byte chunk c (0..7) of row r inside a swizzled block of 128-byte rows.
__device__ __forceinline__ int a5_swz(int r, int c) { return (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4); }

// Keys [key0, key0 + 64) of one kv head into a swizzled K tile and V tile (zeros past last_key).
__device__ __forceinline__ void a5_load_kv(unsigned char* ks, unsigned char* vs, const AttnArgs& a, const int* table, int kvh,
                                           int key0, int last_key, int tid) {
  const int ps_mask = (1 << a.page_shift) - 1;
#pragma unroll
  for (int i = 0; i < A5_BN * 16 / A5_THREADS; ++i) {
    const int idx = tid + i * A5_THREADS;
    const int key = idx >> 4, cc = idx & 15;
    const int kidx = key0 + key;
    const bool valid = kidx <= last_key;
    const int kc = valid ? kidx : last_key;             // a readable address also for the zero-filled rows
    const int page = table[kc >> a.page_shift];
    const size_t off = ((((size_t)page * a.nkv + kvh) << a.page_shift) + (kc & ps_mask)) * A5_D + cc * 8;
    const int dst = (cc >> 3) * (A5_BN * 128) + a5_swz(key, cc & 7);
    cp_async16(ks + dst, a.kpages + off, valid);
    cp_async16(vs + dst, a.vpages + off, valid);
  }
}

__global__ void __launch_bounds__(A5_THREADS, 2) attention_prefill_tcgen05_kernel(AttnArgs a, int* __restrict__ err) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = smem;
  unsigned char* kv_s = q_s + A5_Q_BYTES;                 // stage s: K at kv_s + s * 2 * KV, V right after it
  unsigned long long* s_bar = reinterpret_cast<unsigned long long*>(kv_s + 4 * A5_KV_BYTES);
  unsigned long long* pv_bar = s_bar + 1;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(pv_bar + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int seq = a.items[2 * blockIdx.x], row_tile = a.items[2 * blockIdx.x + 1], kvh = blockIdx.y;
  const int G = a.nq / a.nkv;
  const int q0 = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q0, start = a.q_start_pos[seq];
  const int n_rows = q_len * G;
  const int R0 = row_tile * A5_ROWS;
  const int* table = a.block_table + (size_t)seq * a.table_width;

  if (tid == 0) {
    a5_mbar_init(s_bar, 1);
    a5_mbar_init(pv_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(a5_s32(tmem_slot)), "n"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }

  // this thread's row
  const int R = R0 + tid;
  const bool live = R < n_rows;
  const int tok = live ? R / G : 0, head = live ? R - tok * G : 0;
  const int hi = live ? start + tok : -1;
  const int lo = live ? (a.window > 0 ? max(0, hi - a.window + 1) : 0) : 0;
  // key range of the CTA
  const int c_first = R0 / G, c_last = min(R0 + A5_ROWS - 1, n_rows - 1) / G;
  const int c_hi = start + c_last;
  const int c_lo = a.window > 0 ? max(0, start + c_first - a.window + 1) : 0;
  const int key_begin = c_lo & ~(A5_BN - 1);
  const int n_tiles = (c_hi - key_begin) / A5_BN + 1;

  // first K/V tile on its way, then Q
  a5_load_kv(kv_s, kv_s + A5_KV_BYTES, a, table, kvh, key_begin, c_hi, tid);
  cp_async_commit();
  {
    const uint4* src = reinterpret_cast<const uint4*>(a.qkv + (size_t)(q0 + tok) * a.qkv_stride + (size_t)(kvh * G + head) * A5_D);
#pragma unroll
    for (int cc = 0; cc < 16; ++cc) {
      const uint4 v = live ? __ldcg(src + cc) : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(q_s + (cc >> 3) * (A5_ROWS * 128) + a5_swz(tid, cc & 7)) = v;
    }
  }
  a5_proxy_fence();
  a5_fence_before();
  __syncthreads();
  a5_fence_after();
  const unsigned tmem_base = *tmem_slot;
  const unsigned t_s = tmem_base + ((unsigned)(warp * 32) << 16);           // this warp's lanes: scores
  const unsigned t_pv = t_s + 128;                                          // and the P V product

  // Running softmax with a lazy maximum: the exponentials use m_used, which follows the true maximum
  // only when that has grown by more than 8 (a factor 256, far inside the range of bfloat16 and of
  // the float sums).  The output rows then accumulate in tensor memory over all tiles and are read,
  // scaled and written back only on those rare occasions, not once per tile.
  float m_used = -INFINITY, l = 0.f;
  bool ok = true;
  const unsigned idesc_s = a5_idesc(A5_BN, false), idesc_pv = a5_idesc(A5_D, true);
  const int min_hi = start + c_first;                                       // the least any live row of the CTA sees
  const int max_lo = a.window > 0 ? max(0, start + c_last - a.window + 1) : 0;
  const bool all_live = R0 + A5_ROWS <= n_rows;

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    unsigned char* k_s = kv_s + (size_t)stage * 2 * A5_KV_BYTES;
    unsigned char* v_s = k_s + A5_KV_BYTES;
    // the product P V of the tile before: done before its shared memory is loaded into again and
    // before anybody rescales the output rows
    if (tile > 0 && ok) {
      ok = a5_mbar_wait(pv_bar, (unsigned)(tile - 1) & 1);
      if (!ok && (tid & 31) == 0) atomicExch(err, 22);
    }
    a5_fence_after();
    if (tile + 1 < n_tiles) {
      unsigned char* nk = kv_s + (size_t)(stage ^ 1) * 2 * A5_KV_BYTES;
      a5_load_kv(nk, nk + A5_KV_BYTES, a, table, kvh, key_begin + (tile + 1) * A5_BN, c_hi, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    a5_proxy_fence();                                  // the copies of this thread, visible to the tensor core
    a5_fence_before();
    __syncthreads();
    const int key0 = key_begin + tile * A5_BN;
    if (tid == 0) {
      a5_fence_after();
#pragma unroll
      for (int ks = 0; ks < A5_D / 16; ++ks) {          // 16 values of the head size per step: 32 bytes along a row
        const unsigned long long ad = a5_desc(a5_s32(q_s) + (ks >> 2) * (A5_ROWS * 128) + (ks & 3) * 32, 16, 1024);
        const unsigned long long bd = a5_desc(a5_s32(k_s) + (ks >> 2) * (A5_BN * 128) + (ks & 3) * 32, 16, 1024);
        a5_mma(tmem_base, ad, bd, idesc_s, ks != 0);
      }
      a5_commit(s_bar);
    }
    if (ok) {
      ok = a5_mbar_wait(s_bar, (unsigned)tile & 1);
      if (!ok && (tid & 31) == 0) atomicExch(err, 21);
    }
    a5_fence_after();

    // this row's 64 scores
    float s[A5_BN];
    {
      float part[32];
      a5_ld32(t_s, part);
#pragma unroll
      for (int j = 0; j < 32; ++j) s[j] = part[j];
      a5_ld32(t_s + 32, part);
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
    float mx = s[0];
#pragma unroll
    for (int j = 1; j < A5_BN; ++j) mx = fmaxf(mx, s[j]);
    mx *= a.scale_log2;                                  // the scale is positive: the maximum of the scaled scores
    const bool grow = mx > m_used + 8.0f || (m_used == -INFINITY && mx != -INFINITY);
    if (__any_sync(0xffffffffu, grow)) {
      const float factor = grow ? (m_used == -INFINITY ? 0.f : a5_ex2(m_used - mx)) : 1.0f;
      if (grow) m_used = mx;
      l *= factor;
      if (tile > 0) {                                    // the rows in tensor memory follow (warp-wide: lanes that keep theirs multiply by 1)
#pragma unroll
        for (int c = 0; c < A5_D / 32; ++c) {
          float part[32];
          a5_ld32(t_pv + c * 32, part);
#pragma unroll
          for (int j = 0; j < 32; ++j) part[j] *= factor;
          a5_st32(t_pv + c * 32, part);
        }
      }
    }
    const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      unsigned w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p0 = a5_ex2(fmaf(s[c * 8 + 2 * e], a.scale_log2, neg_m));
        const float p1 = a5_ex2(fmaf(s[c * 8 + 2 * e + 1], a.scale_log2, neg_m));
        sum += p0 + p1;
        w[e] = pack_bf16(p0, p1);
      }
      *reinterpret_cast<uint4*>(k_s + a5_swz(tid, c)) = make_uint4(w[0], w[1], w[2], w[3]);   // P where K was: S is done with it
    }
    l += sum;
    a5_proxy_fence();
    a5_fence_before();
    __syncthreads();
    if (tid == 0) {
      a5_fence_after();
#pragma unroll
      for (int ks = 0; ks < A5_BN / 16; ++ks) {          // 16 keys per step: 32 bytes along a row of P, 2 KB down V
        const unsigned long long ad = a5_desc(a5_s32(k_s) + ks * 32, 16, 1024);
        const unsigned long long bd = a5_desc(a5_s32(v_s) + ks * 2048, A5_BN * 128, 1024);
        a5_mma(tmem_base + 128, ad, bd, idesc_pv, (tile | ks) != 0);
      }
      a5_commit(pv_bar);
    }
  }
  cp_async_wait<0>();
  if (ok) {
    ok = a5_mbar_wait(pv_bar, (unsigned)(n_tiles - 1) & 1);
    if (!ok && (tid & 31) == 0) atomicExch(err, 23);
  }
  a5_fence_after();

  {
    const float inv = live && l > 0.f ? 1.0f / l : 0.f;
    bf16* dst = a.out + (size_t)(q0 + tok) * a.nq * A5_D + (size_t)(kvh * G + head) * A5_D;
#pragma unroll
    for (int c = 0; c < A5_D / 32; ++c) {                 // tcgen05.ld is warp-wide: dead rows read too, and store nothing
      float part[32];
      a5_ld32(t_pv + c * 32, part);
      if (!live) continue;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 w;
        w.x = pack_bf16(part[q * 8] * inv, part[q * 8 + 1] * inv);
        w.y = pack_bf16(part[q * 8 + 2] * inv, part[q * 8 + 3] * inv);
        w.z = pack_bf16(part[q * 8 + 4] * inv, part[q * 8 + 5] * inv);
        w.w = pack_bf16(part[q * 8 + 6] * inv, part[q * 8 + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = w;
      }
    }
  }
  // every thread gets here (all waits are bounded); then the tensor memory goes back
  a5_fence_before();
  __syncthreads();
  if (warp == 0) {
    a5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(256) : "memory");
  }
}

// items: (entry, 128-row tile) pairs; otherwise the arguments of q25_attention_prefill_bf16.  Head size
// 128 only.  err: one int that receives a nonzero code if a wait gave up.
Q25_EXPORT int q25_attention_prefill_tcgen05_bf16(const void* qkv, int qkv_stride, void* out, const void* kp, const void* vp,
                                                  const int* bt, int tw, const int* cu_q, const int* q_start,
                                                  const int* tiles, int n_tiles, int nq, int nkv, int d, int page_size,
                                                  int window, float scale, int* err, void* stream) {
  if (n_tiles <= 0) return 0;
  if (d != A5_D || !err) return (int)cudaErrorInvalidValue;
  AttnArgs a;
  int e = fill_args(a, qkv, qkv_stride, out, kp, vp, bt, tw, cu_q, q_start, tiles, nq, nkv, page_size, window, scale);
  if (e) return e;
  if (((uintptr_t)qkv & 15) || (qkv_stride % 8) || ((uintptr_t)out & 15)) return (int)cudaErrorInvalidValue;
  cudaError_t ce = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A5_SMEM);
  if (ce != cudaSuccess) return (int)ce;
  launch(attention_prefill_tcgen05_kernel, dim3(n_tiles, nkv), dim3(A5_THREADS), (size_t)A5_SMEM, (cudaStream_t)stream, a, err);
  return launch_status();
}
