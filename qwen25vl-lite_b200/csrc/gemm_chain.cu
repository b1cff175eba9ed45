// y[M,N] = x[M,K] . W[N,K]^T for a handful of rows (decode steps: M = live requests <= 8), bfloat16,
// as one operation or as a chain of up to eight in ONE persistent kernel.
//
// With so few rows a product is a stream of its weights: every byte of W is read once and used for M
// multiply-adds, so the kernel is built around keeping HBM busy, not the tensor cores.  And a decode
// step is a chain of such products, each of which needs the whole result of the one before it:
// o-projection -> gate/up -> down -> next layer's qkv ...  Launched one by one, every link pays
// for the end of one kernel and the start of the next: the stream of weights stops, the SMs drain,
// the next kernel's first bytes take a memory latency to arrive (measured in a step: 7 to 12 us
// for products whose weights pass in 1.5 us).  Here the links are operations of one kernel:
//
//   * One CTA per SM stays resident for the whole chain: the grid has as many CTAs as the device has
//     SMs and a CTA's shared memory leaves room for no second one, so every CTA finds an SM as soon
//     as the kernels before this one have left it, and all are resident together.  Between two
//     operations the CTAs meet at a barrier in global memory (a counter that only grows).
//   * The kernel is launched like every other kernel of the engine (programmatic dependent launch,
//     common.cuh): its CTAs start on the SMs that the kernel before it has already left, set up
//     their barriers and start the stream of weights, and only the warps that read x or write the
//     output wait for that kernel to finish.
//   * The producer warp does not meet anybody: weights depend on no activation, so it walks on
//     through the operations and fills the ring of stages with the next operation's weights while
//     the other warps are still finishing this one or stand at the barrier.  The stream from memory
//     does not stop at a link.
//   * Inside an operation: groups of 16 output features (16 rows of W), the weights on the 16-row
//     side of mma.sync m16n8k16 (the operands are swapped: W is "A", x^T is "B", 8 batch columns
//     per instruction; a thread reads 16 contiguous bytes of a row from shared memory and feeds
//     them to two MMAs, and since a dot product does not care about the order of its terms the 8
//     values take the MMA's k slots in memory order and x is read with the same assignment), eight
//     MMA warps taking alternate 32-wide
//     k blocks, an epilogue warp adding their partial sums in warp order, x resident in shared
//     memory (read past the L1 cache, which knows nothing of what other SMs wrote since the
//     launch), optional RMSNorm of the float residual stream on the way in (reference
//     src/qwen25vl_lite/layers.py:27-31), epilogues store / +bias / float / SwiGLU pairs
//     (src/qwen25vl_lite/text.py:66) / add into the residual stream.  One request brings one row
//     of a group, up to 4 KB (the copy engine takes a request about every 100 cycles whatever its
//     size).
//   * K longer than 2048 is cut into slices, so that a slice of x fits into shared memory.  With
//     few groups per CTA (a down projection: 128 groups) a CTA takes the slices of its group one
//     after the other: the sums stay in registers, and the next slice of x arrives (cp.async into the
//     other of two buffers) while this one is multiplied.  With many groups per CTA every CTA works
//     in one slice; the slices' partial sums go to scratch slots, and an owner CTA, when all slices
//     have counted themselves in, adds them in slice order and runs the epilogue.  Either way the
//     result does not depend on timing.  Up to 8 rows of a width that is cut but not long (3584,
//     5120) stay in shared memory whole, and a CTA walks the slices of its groups over them: no
//     scratch memory and nothing to finish afterwards (the owners' pass of a wide gate/up product,
//     sixteen groups a CTA, cost 13 to 23 us of a layer's 130).
//   * A stage of the ring is as long as the longest slice of the chain, and the host picks the cut
//     (chain_plan below): x whole where it fits, else the cut that leaves the most bytes in the ring.
//     At a width of 2048 that is two stages of 65 KB, at 3584 and 5120 four of 39 and 45 KB.  (How
//     deep the ring is matters little once it holds two stages: at the 7B and 32B sizes two, three
//     and four stages gave 99 / 105 / 101 and 186 / 181 / 178 us a layer.  What costs is what stands
//     between the operations.)
//
// Every wait (mbarrier or grid barrier) is bounded: when it gives up, the kernel records a code in
// *err, stops waiting anywhere and runs to its end (its output is then invalid).
#include "common.cuh"

enum { EPI_STORE = 0, EPI_BIAS = 1, EPI_F32 = 2, EPI_SWIGLU = 3, EPI_RESIDUAL = 4 };

#define GC_ROWS 16
#define GC_MAX_M 8                               // rows of x: one 8-column tile of the MMA (MT = 1).  A second tile
                                                 // (9 to 16 rows) was measured slower than the library's products
                                                 // at every size and is not instantiated.
#define GC_CONSUMERS 8
#define GC_RED_BUFS 2
#define GC_THREADS ((GC_CONSUMERS + 2) * 32)
#define GC_MAX_OPS 8
#define GC_SLICE_K 2048                          // most K elements of a slice
#define GC_SMEM_LIMIT (227 * 1024)
#define GC_GRID_WAIT_LIMIT (1 << 21)             // polls of global memory, about a second

struct ChainOp {
  const bf16* W;          // [N, K]
  const void* X;          // bf16 [M, K], or float [M, K] when norm
  const float* norm_w;    // [K] when norm
  const float* bias;      // [N] when epi == EPI_BIAS
  void* out;
  int ldx, ldo, M, N, K, epi, norm;
  float eps;
  int slices, slice_k, ctas, groups;   // K cut into `slices` of `slice_k` elements; `ctas` CTAs work in each slice
  int seq;                // the K slices of a group are taken one after the other by the same CTA (see below):
                          // 1 with the slices of x through two buffers, 2 with x whole in shared memory
  int xp;                 // bytes between the rows of x in shared memory
};

struct ChainArgs {
  int n_ops, n_stages;
  int pitch;              // bytes between rows in shared memory: the longest slice, padded so that pitch mod 128 = 64 (no bank conflicts)
  int slot;               // one stage: the 16 rows of a group, one slice long
  int x_off;              // where x begins in shared memory
  int stash_off;          // where a norm operation's weights wait in shared memory (-1: no room, they are read in place)
  int stash_bytes;
  float* scratch;         // slots of partial sums, [slice][group][MT * 128] floats, reused by every operation
  int* counters;          // one per group, zero before the launch and after it
  unsigned* barrier;      // arrivals at the barriers between operations; only grows
  unsigned barrier_base;  // its value when this launch begins
  int* err;
  ChainOp op[GC_MAX_OPS];
};

// cp.async of 16 bytes (zeros when !valid) and its group bookkeeping: x slices of the sequential K walk
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ uint4 gc_lds128(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}
__device__ __forceinline__ float4 gc_ldcg128(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned gc_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void gc_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The weights a CTA streams are a sequence of items, one stage of the ring each: for every operation
// in order the CTA's groups, and for an operation that walks K sequentially the slices of each
// group.  Advances (k, grp, j) = (operation, group, slice) to the next item; start with k = -1.
__device__ __forceinline__ bool item_next(const ChainArgs& A, int cta, int& k, int& grp, int& j) {
  if (k >= 0) {
    const ChainOp& op = A.op[k];
    if (op.seq) {
      if (++j < op.slices) return true;
      j = 0;
    }
    grp += op.ctas;
    if (grp < op.groups) return true;
  }
  for (++k; k < A.n_ops; ++k) {
    const ChainOp& op = A.op[k];
    if (op.seq) {
      grp = cta; j = 0;
    } else {
      j = cta / op.ctas;
      if (j >= op.slices) continue;
      grp = cta - j * op.ctas;
    }
    if (grp < op.groups) return true;
  }
  return false;
}

// accumulator (mt, e): output feature row0 + g + 8 * (e / 2), batch column mt * 8 + 2 t + (e & 1)
template <int MT>
__device__ __forceinline__ void gc_store_group(const float (&acc)[MT][4], int grp, const ChainOp& op, bool has_old = false) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int row0 = grp * GC_ROWS;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int m = mt * 8 + 2 * t + e;
      if (m >= op.M) continue;
      if (op.epi == EPI_SWIGLU) {
        // rows g of the group are gate features, rows g + 8 the matching up features
        if (row0 + g + 8 < op.N) {
          const float gate = acc[mt][e], up = acc[mt][e + 2];
          reinterpret_cast<bf16*>(op.out)[(size_t)m * op.ldo + (row0 >> 1) + g] =
              __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
        }
        continue;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int n = row0 + g + 8 * h;
        if (n >= op.N) continue;
        float v = acc[mt][e + 2 * h];
        if (op.epi == EPI_BIAS) v += op.bias[n];
        if (op.epi == EPI_F32) reinterpret_cast<float*>(op.out)[(size_t)m * op.ldo + n] = v;
        else if (op.epi == EPI_RESIDUAL) {
          float* dst = reinterpret_cast<float*>(op.out) + (size_t)m * op.ldo + n;
          *dst = has_old ? v : __ldcg(dst) + v;       // has_old: the old value is in v already
        }
        else reinterpret_cast<bf16*>(op.out)[(size_t)m * op.ldo + n] = __float2bfloat16_rn(v);
      }
    }
  }
}

// One copy of the store code for the owners' pass, which runs once per operation: inlined there
// for every group of a batch, it is a third of the kernel's code, fetched cold every time.
template <int MT>
__device__ __noinline__ void gc_store_group_once(float4 a, float4 b, int grp, const ChainOp& op, bool has_old) {
  float acc[MT][4];
  acc[0][0] = a.x; acc[0][1] = a.y; acc[0][2] = a.z; acc[0][3] = a.w;
  if (MT > 1) { acc[MT - 1][0] = b.x; acc[MT - 1][1] = b.y; acc[MT - 1][2] = b.z; acc[MT - 1][3] = b.w; }
  gc_store_group<MT>(acc, grp, op, has_old);
}

// The owners' pass of an operation whose slices were other CTAs'.  The i-th group of list r (the
// groups r, r + ctas, ...) is finished by the CTA of slice (i + r) mod slices, and there by MMA warp
// (i / slices) mod 8: the warp waits (bounded) until every slice has counted the group in, adds
// the slices' shares in slice order and runs the epilogue.  G groups at a time and J slices of each
// per trip to memory, and every load of a trip is asked for before any is used and depends on no
// condition (behind a branch each, they wait for one another): a place that is not wanted (past the
// last group of the batch, past the last slice, outside the output) reads a neighbour that is, and
// a select drops what it brought.  One warp doing this for all sixteen groups of a CTA, group by
// group, took 23 us after a wide gate/up product; eight warps with their loads batched take 4.
template <int MT, int G, int J>
__device__ __forceinline__ bool gc_finish_groups(const ChainArgs& A, const ChainOp& op, int r, int slice, int warp, bool ok) {
  const int lane = threadIdx.x & 31;
  const bool add_old = op.epi == EPI_RESIDUAL;
  const size_t slice_stride = (size_t)op.groups * (MT * 32);                         // in float4
  const int n_list = (op.groups - r + op.ctas - 1) / op.ctas;                        // groups in list r
  const int first = ((slice - r) % op.slices + op.slices) % op.slices + warp * op.slices, step = GC_CONSUMERS * op.slices;
  for (int i0 = first; i0 < n_list; i0 += G * step) {
    int grp[G], n = 0;
#pragma unroll
    for (int q = 0; q < G; ++q) {
      const bool in = i0 + q * step < n_list;
      grp[q] = in ? r + (i0 + q * step) * op.ctas : grp[0];
      n += in ? 1 : 0;
    }
    if (lane < n && ok) {                        // lane q waits for group q of the batch
      int mine = grp[0];
#pragma unroll
      for (int q = 1; q < G; ++q) mine = lane == q ? grp[q] : mine;
      int i = 0;
      while ((int)gc_ld_acquire(reinterpret_cast<const unsigned*>(A.counters + mine)) != op.slices && ++i < GC_GRID_WAIT_LIMIT) {}
      if (i >= GC_GRID_WAIT_LIMIT) { ok = false; atomicExch(A.err, 18); }
      A.counters[mine] = 0;                      // left as it was found, for the next operation and the next launch
    }
    ok = __all_sync(0xffffffffu, ok);
    float acc[G][MT][4];
    if (add_old) {                               // asked for together with the slices' shares: one trip, not two
#pragma unroll
      for (int q = 0; q < G; ++q)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int m = mt * 8 + 2 * (lane & 3) + (e & 1), f = grp[q] * GC_ROWS + (lane >> 2) + 8 * (e >> 1);
            const float old = __ldcg(reinterpret_cast<const float*>(op.out) + (size_t)min(m, op.M - 1) * op.ldo + min(f, op.N - 1));
            acc[q][mt][e] = (m < op.M && f < op.N) ? old : 0.f;
          }
    } else {
#pragma unroll
      for (int q = 0; q < G; ++q)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) acc[q][mt][0] = acc[q][mt][1] = acc[q][mt][2] = acc[q][mt][3] = 0.f;
    }
    for (int j0 = 0; j0 < op.slices; j0 += J) {
      float4 v[G][J][MT];
#pragma unroll
      for (int q = 0; q < G; ++q)
#pragma unroll
        for (int jj = 0; jj < J; ++jj)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            v[q][jj][mt] = __ldcg(reinterpret_cast<const float4*>(A.scratch + (size_t)grp[q] * (MT * 128)) + lane +
                                  (size_t)min(j0 + jj, op.slices - 1) * slice_stride + mt * 32);
#pragma unroll
      for (int q = 0; q < G; ++q)
#pragma unroll
        for (int jj = 0; jj < J; ++jj) {
          const bool in = j0 + jj < op.slices;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            acc[q][mt][0] += in ? v[q][jj][mt].x : 0.f; acc[q][mt][1] += in ? v[q][jj][mt].y : 0.f;
            acc[q][mt][2] += in ? v[q][jj][mt].z : 0.f; acc[q][mt][3] += in ? v[q][jj][mt].w : 0.f;
          }
        }
    }
#pragma unroll
    for (int q = 0; q < G; ++q)
      if (q < n)
        gc_store_group_once<MT>(make_float4(acc[q][0][0], acc[q][0][1], acc[q][0][2], acc[q][0][3]),
                                make_float4(acc[q][MT - 1][0], acc[q][MT - 1][1], acc[q][MT - 1][2], acc[q][MT - 1][3]),
                                grp[q], op, add_old);
  }
  return ok;
}

template <int MT>
__global__ void __launch_bounds__(GC_THREADS, 1) gemm_chain_kernel(const __grid_constant__ ChainArgs A) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int S = A.n_stages, P = A.pitch, SLOT = A.slot;
  unsigned char* xs = smem + A.x_off;             // x of a product
  const float4* stash = A.stash_off >= 0 ? reinterpret_cast<const float4*>(smem + A.stash_off) : nullptr;
  unsigned char* slots = smem;
  float* red = reinterpret_cast<float*>(slots + (size_t)S * SLOT);
  unsigned long long* full = reinterpret_cast<unsigned long long*>(red + GC_RED_BUFS * GC_CONSUMERS * 32 * MT * 4);
  unsigned long long* empty = full + S;
  unsigned long long* go = empty + S;             // the operation before this one is complete on every CTA
  unsigned long long* fixed = go + 1;             // the MMA warps have finished the groups this CTA owns (an operation cut across CTAs)
  unsigned long long* red_full = fixed + 1;
  unsigned long long* red_empty = red_full + GC_RED_BUFS;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int cta = blockIdx.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, GC_CONSUMERS);
    }
    mbar_init(go, 1);
    mbar_init(fixed, GC_CONSUMERS);
    for (int b = 0; b < GC_RED_BUFS; ++b) {
      mbar_init(red_full + b, GC_CONSUMERS);
      mbar_init(red_empty + b, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  pdl_trigger();

  if (warp == GC_CONSUMERS) {
    // ---- producer: the weights of every operation, one bulk copy per row, as stages come free ----
    // (Asking for the items further ahead to be brought into the L2 cache while the ring is full --
    // cp.async.bulk.prefetch.L2, two to eight items ahead, or the first megabytes of the next kernel's
    // weights at the end -- made a step slower by 5 to 30 % or changed nothing, measured on B200: the
    // operations wait at their barriers and for their rows of x, not for the weights.)
    bool ok = true;
    int s = 0, wrapped = 0;
    unsigned parity = 1;
    int ck = -1, cg = 0, cj = 0;
    const unsigned long long once = l2_evict_first();
    while (item_next(A, cta, ck, cg, cj)) {
      const ChainOp& op = A.op[ck];
      const int k0 = cj * op.slice_k;
      const unsigned bytes = (unsigned)min(op.slice_k, op.K - k0) * 2;
      if (wrapped && ok) {
        ok = mbar_wait(empty + s, parity);
        if (!ok && lane == 0) atomicExch(A.err, 11);
      }
      unsigned char* st = slots + (size_t)s * SLOT;
      if (lane == 0) mbar_expect_tx(full + s, bytes * GC_ROWS);
      __syncwarp();
      if (lane < GC_ROWS)
        bulk_copy_once(st + lane * P, op.W + (size_t)min(cg * GC_ROWS + lane, op.N - 1) * op.K + k0, bytes, full + s, once);
      if (++s == S) { s = 0; wrapped = 1; parity ^= 1; }
    }
    return;
  }

  if (warp == GC_CONSUMERS + 1) {
    // ---- epilogue warp: grid barrier, x, sums of the MMA warps' partial sums, stores ----
    pdl_wait();                 // the first operation's output may still be read (or be written) by the kernel before
    bool ok = true;
    int rb = 0;
    unsigned red_parity = 0;
    unsigned fixed_parity = 0;
    for (int k = 0; k < A.n_ops; ++k) {
      const ChainOp& op = A.op[k];
      if (k > 0) {
        if (A.op[k - 1].slices > 1 && !A.op[k - 1].seq) {
          // what this CTA's MMA warps stored for the groups it owns belongs to the operation before too
          if (ok) {
            ok = mbar_wait(fixed, fixed_parity);
            if (!ok && lane == 0) atomicExch(A.err, 19);
          }
          fixed_parity ^= 1;
        }
        // everything the operation before this one wrote, on every CTA, before anybody reads it: the
        // lanes' stores meet at __syncwarp, and the release of the first lane's add carries them all
        // (a fence by each of the 32 lanes first cost about a third of a microsecond per barrier)
        __syncwarp();
        if (lane == 0) {
          // The counter only grows: the k-th barrier of this launch is passed when it has reached
          // base + k * (number of CTAs).  The last arrival itself lets everybody go; nothing is
          // reset and no second flag is written (the caller zeroes the counter between steps).
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(A.barrier) : "memory");
          if (ok) {
            const unsigned target = A.barrier_base + (unsigned)k * gridDim.x;
            int i = 0;
            while ((int)(gc_ld_acquire(A.barrier) - target) < 0 && ++i < GC_GRID_WAIT_LIMIT) {}
            if (i >= GC_GRID_WAIT_LIMIT) { ok = false; atomicExch(A.err, 16); }
          }
          mbar_arrive(go);
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
      const bool sliced = op.slices > 1 && !op.seq;    // the slices are other CTAs' and meet in scratch memory
      const int slice = op.seq ? 0 : cta / op.ctas, r = op.seq ? cta : cta - slice * op.ctas;
      if (op.seq ? cta >= op.ctas : slice >= op.slices) continue;
      const bool add_old = op.epi == EPI_RESIDUAL && !sliced;
      for (int grp = r; grp < op.groups; grp += op.ctas) {
        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
        if (add_old) {
          // the residual stream's old values, fetched while the MMA warps still work on the group
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int m = mt * 8 + 2 * (lane & 3) + (e & 1), n = grp * GC_ROWS + (lane >> 2) + 8 * (e >> 1);
              if (m < op.M && n < op.N) acc[mt][e] = __ldcg(reinterpret_cast<const float*>(op.out) + (size_t)m * op.ldo + n);
            }
        }
        if (ok) {
          ok = mbar_wait(red_full + rb, red_parity);
          if (!ok && lane == 0) atomicExch(A.err, 15);
        }
#pragma unroll
        for (int w = 0; w < GC_CONSUMERS; ++w) {
          const float* src = red + (((size_t)rb * GC_CONSUMERS + w) * 32 + lane) * MT * 4;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const float4 v = *reinterpret_cast<const float4*>(src + mt * 4);
            acc[mt][0] += v.x; acc[mt][1] += v.y; acc[mt][2] += v.z; acc[mt][3] += v.w;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(red_empty + rb);
        if (++rb == GC_RED_BUFS) { rb = 0; red_parity ^= 1; }

        if (sliced) {
          // a slice's share of the group: into its scratch slot; who completes the group is settled
          // once for all groups, after the last one (one trip to memory, not one per group)
          float* mine = A.scratch + ((size_t)slice * op.groups + grp) * (MT * 128);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            *reinterpret_cast<float4*>(mine + mt * 128 + lane * 4) = make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
          continue;
        }
        gc_store_group<MT>(acc, grp, op, add_old);
      }
      if (sliced) {
        // This slice's shares of the CTA's groups are written: every group is counted in, and the
        // MMA warps of the CTA that owns it (gc_finish_groups) will see all slices there.
        __threadfence();
        __syncwarp();
        for (int grp = r + lane * op.ctas; grp < op.groups; grp += 32 * op.ctas) atomicAdd(A.counters + grp, 1);
      }
    }
    return;
  }

  // ---- MMA warps ----
  pdl_wait();                   // x of the first operation comes from the kernel before this one
  bool ok = true;
  int s = 0, rb = 0;
  unsigned parity = 0, red_parity = 1;
  bool red_wrapped = false;
  const int ctid = threadIdx.x;                     // 0 .. 255 in the MMA warps
  auto consumer_sync = [] { asm volatile("bar.sync 1, %0;\n" ::"n"(GC_CONSUMERS * 32) : "memory"); };
  for (int k = 0; k < A.n_ops; ++k) {
    const ChainOp& op = A.op[k];
    // The norm weights of this operation are asked for before the wait at the barrier (nothing
    // writes them): read after it, they cost a second trip to memory behind the one for x, and
    // they are cold, every layer having its own.
    const int slice = op.seq ? 0 : cta / op.ctas, r = cta - slice * op.ctas;
    const bool mine = op.seq ? cta < op.ctas : slice < op.slices;                // this CTA has a share of the operation
    const int k0 = op.seq ? 0 : slice * op.slice_k;                              // the columns of x it needs
    const int klen = op.seq ? op.K : min(op.slice_k, op.K - k0);
    const bool stashed = op.norm && stash != nullptr && mine && klen * 4 <= A.stash_bytes;
    if (stashed) {
      for (int i = ctid; i < klen / 4; i += GC_CONSUMERS * 32)
        cp_async16(smem + A.stash_off + (size_t)i * 16, op.norm_w + k0 + (size_t)i * 4, true);
      cp_async_commit();
    } else if (op.norm && mine) {
      // no room for them there: at least they are brought near (L1) meanwhile
      for (int i = ctid; i < (klen * 4 + 127) / 128; i += GC_CONSUMERS * 32)
        asm volatile("prefetch.global.L1 [%0];\n" ::"l"(reinterpret_cast<const char*>(op.norm_w + k0) + (size_t)i * 128));
    }
    if (k > 0 && ok) {
      ok = mbar_wait(go, (unsigned)(k - 1) & 1);
      if (!ok && lane == 0) atomicExch(A.err, 12);
    }
    if (op.seq == 1) {
      // ---- the K slices of a group one after the other; x slices through two buffers ----
      if (cta >= op.ctas) continue;
      const bf16* X = reinterpret_cast<const bf16*>(op.X);
      const int xbuf_bytes = (op.M * P + 127) / 128 * 128;
      const int my_groups = (op.groups - cta + op.ctas - 1) / op.ctas;
      const int n_items = my_groups * op.slices;
      auto fetch_x = [&](int item) {                  // the x slice of item (group, slice) into buffer item & 1
        const int j = item % op.slices;
        const int k0 = j * op.slice_k, chunks = min(op.slice_k, op.K - k0) / 8;     // 16-byte chunks of a row
        unsigned char* dst = xs + (size_t)(item & 1) * xbuf_bytes;
        for (int idx = ctid; idx < op.M * chunks; idx += GC_CONSUMERS * 32) {
          const int row = idx / chunks, c = idx - row * chunks;
          cp_async16(dst + (size_t)row * P + c * 16, X + (size_t)row * op.ldx + k0 + c * 8, true);
        }
        cp_async_commit();
      };
      fetch_x(0);
      float acc[2][MT][4];
      for (int item = 0; item < n_items; ++item) {
        const int j = item % op.slices;
        cp_async_wait<0>();
        consumer_sync();                              // this item's x is in, and nobody reads the other buffer any more
        if (item + 1 < n_items) fetch_x(item + 1);
        if (j == 0) {
#pragma unroll
          for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) acc[q][mt][0] = acc[q][mt][1] = acc[q][mt][2] = acc[q][mt][3] = 0.f;
        }
        const unsigned char* xb = xs + (size_t)(item & 1) * xbuf_bytes + t * 16;
        const int kblocks = min(op.slice_k, op.K - j * op.slice_k) / 32;
        if (ok) {
          ok = mbar_wait(full + s, parity);
          if (!ok && lane == 0) atomicExch(A.err, 14);
        }
        const unsigned char* st = slots + (size_t)s * SLOT + g * P + t * 16;
#pragma unroll 2
        for (int kb = warp; kb < kblocks; kb += GC_CONSUMERS) {
          const uint4 a0 = gc_lds128(st + kb * 64);
          const uint4 a1 = gc_lds128(st + 8 * P + kb * 64);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint4 b = gc_lds128(xb + (size_t)min(mt * 8 + g, op.M - 1) * P + kb * 64);
            gc_mma(acc[0][mt], a0.x, a1.x, a0.y, a1.y, b.x, b.y);
            gc_mma(acc[1][mt], a0.z, a1.z, a0.w, a1.w, b.z, b.w);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
        if (++s == S) { s = 0; parity ^= 1; }
        if (j + 1 < op.slices) continue;
        // the group is complete: hand the sums to the epilogue warp
        if (red_wrapped && ok) {
          ok = mbar_wait(red_empty + rb, red_parity);
          if (!ok && lane == 0) atomicExch(A.err, 17);
        }
        float* dst = red + (((size_t)rb * GC_CONSUMERS + warp) * 32 + lane) * MT * 4;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          *reinterpret_cast<float4*>(dst + mt * 4) = make_float4(acc[0][mt][0] + acc[1][mt][0], acc[0][mt][1] + acc[1][mt][1],
                                                                 acc[0][mt][2] + acc[1][mt][2], acc[0][mt][3] + acc[1][mt][3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(red_full + rb);
        if (++rb == GC_RED_BUFS) { rb = 0; red_wrapped = true; red_parity ^= 1; }
      }
      consumer_sync();                                // x of the next operation goes where these buffers are
      continue;
    }
    const bool sliced = op.slices > 1 && !op.seq;    // the slices are other CTAs' and meet in scratch memory
    if (!mine) {
      if (sliced && lane == 0) mbar_arrive(fixed);
      continue;
    }
    const int XP = op.xp;
    // x is read past L1 (__ldcg): other SMs wrote it since this kernel began.  The loads of a batch
    // are issued together (one by one, each would cost a trip to L2), and none of them depends on a
    // condition: a lane past the end of its row reads the row's last place and drops it.
    if (op.norm) {
      const float* Xf = reinterpret_cast<const float*>(op.X);
      if (stashed) {
        cp_async_wait<0>();
        asm volatile("bar.sync 1, %0;\n" ::"n"(GC_CONSUMERS * 32) : "memory");      // every thread's share of them is in
      }
      const int n4 = op.K / 4, a4 = k0 / 4, s4 = klen / 4;
      const float4* w4 = stashed ? stash : reinterpret_cast<const float4*>(op.norm_w + k0);
      const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
      auto sq = [](const float4& q) { return q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w; };
      auto put = [&](unsigned char* dst, int i, const float4& q, float inv) {        // normalised values i of the CTA's columns
        const float4 w = w4[i];
        __nv_bfloat162 lo = __floats2bfloat162_rn(q.x * inv * w.x, q.y * inv * w.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn(q.z * inv * w.z, q.w * inv * w.w);
        uint2 packed;
        packed.x = *reinterpret_cast<unsigned*>(&lo);
        packed.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(dst + (size_t)i * 8) = packed;
      };
      for (int m = warp; m < op.M; m += GC_CONSUMERS) {
        const float4* xr = reinterpret_cast<const float4*>(Xf + (size_t)m * op.ldx);
        unsigned char* dst = xs + (size_t)m * XP;
        if (s4 <= 32 * 16) {
          // The CTA's columns of the row (all of it, or a slice of at most 2048 values) stay in
          // registers, 16 float4 a lane; the rest of a longer row is read for the sum of squares
          // only, in batches of the same size.
          float4 v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int i = j * 32 + lane;
            const float4 q = __ldcg(xr + a4 + min(i, s4 - 1));
            v[j] = i < s4 ? q : zero4;
          }
          float ss = 0.f;
          const int rest = n4 - s4;
          for (int i0 = 0; i0 < rest; i0 += 32 * 16) {
            float4 u[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int i = min(i0 + j * 32 + lane, rest - 1);       // the i-th float4 of the row outside the slice
              u[j] = __ldcg(xr + (i < a4 ? i : i + s4));
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) ss += i0 + j * 32 + lane < rest ? sq(u[j]) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) ss += sq(v[j]);
          const float inv = rsqrtf(warp_sum(ss) / (float)op.K + op.eps);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j * 32 + lane < s4) put(dst, j * 32 + lane, v[j], inv);
          continue;
        }
        // All of a row that is longer than the registers hold: once for the sum of squares and once
        // more, from L2, for the values.
        float ss = 0.f;
        for (int i0 = 0; i0 < n4; i0 += 32 * 16) {
          float4 u[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) u[j] = __ldcg(xr + min(i0 + j * 32 + lane, n4 - 1));
#pragma unroll
          for (int j = 0; j < 16; ++j) ss += i0 + j * 32 + lane < n4 ? sq(u[j]) : 0.f;
        }
        const float inv = rsqrtf(warp_sum(ss) / (float)op.K + op.eps);
        for (int i0 = 0; i0 < s4; i0 += 32 * 16) {
          float4 u[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) u[j] = __ldcg(xr + a4 + min(i0 + j * 32 + lane, s4 - 1));
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (i0 + j * 32 + lane < s4) put(dst, i0 + j * 32 + lane, u[j], inv);
        }
      }
    } else {
      const bf16* X = reinterpret_cast<const bf16*>(op.X);
      for (int m = warp; m < op.M; m += GC_CONSUMERS) {
        const uint4* xr = reinterpret_cast<const uint4*>(X + (size_t)m * op.ldx + k0);
        const int n16 = klen / 8;
        for (int i0 = 0; i0 < n16; i0 += 32 * 8) {
          uint4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = __ldcg(xr + min(i0 + j * 32 + lane, n16 - 1));
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int i = i0 + j * 32 + lane;
            if (i < n16) *reinterpret_cast<uint4*>(xs + (size_t)m * XP + (size_t)i * 16) = v[j];
          }
        }
      }
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(GC_CONSUMERS * 32) : "memory");
    // rows of x this thread reads for each 8-column tile (rows past M repeat the last one; their
    // columns are never stored)
    const unsigned char* xrow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) xrow[mt] = xs + (size_t)min(mt * 8 + g, op.M - 1) * XP + t * 16;

    // The groups of this CTA; of each, the slice that is this CTA's, or, over x whole, all slices
    // one after the other with the sums staying in registers.
    const int walk = op.seq ? op.slices : 1;
    for (int grp = r; grp < op.groups; grp += op.ctas) {
      float acc[2][MT][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) acc[j][mt][0] = acc[j][mt][1] = acc[j][mt][2] = acc[j][mt][3] = 0.f;
      for (int j = 0; j < walk; ++j) {
        const int kj = op.seq ? j * op.slice_k : 0;                 // where in the resident x this stage begins
        const int kblocks = (op.seq ? min(op.slice_k, op.K - kj) : klen) / 32;
        if (ok) {
          ok = mbar_wait(full + s, parity);
          if (!ok && lane == 0) atomicExch(A.err, 14);
        }
        const unsigned char* st = slots + (size_t)s * SLOT + g * P + t * 16;
#pragma unroll 2
        for (int kb = warp; kb < kblocks; kb += GC_CONSUMERS) {
          const uint4 a0 = gc_lds128(st + kb * 64);
          const uint4 a1 = gc_lds128(st + 8 * P + kb * 64);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint4 b = gc_lds128(xrow[mt] + kj * 2 + kb * 64);
            gc_mma(acc[0][mt], a0.x, a1.x, a0.y, a1.y, b.x, b.y);
            gc_mma(acc[1][mt], a0.z, a1.z, a0.w, a1.w, b.z, b.w);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
        if (++s == S) { s = 0; parity ^= 1; }
      }

      // hand the partial sums to the epilogue warp
      if (red_wrapped && ok) {
        ok = mbar_wait(red_empty + rb, red_parity);
        if (!ok && lane == 0) atomicExch(A.err, 17);
      }
      float* dst = red + (((size_t)rb * GC_CONSUMERS + warp) * 32 + lane) * MT * 4;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
        *reinterpret_cast<float4*>(dst + mt * 4) = make_float4(acc[0][mt][0] + acc[1][mt][0], acc[0][mt][1] + acc[1][mt][1],
                                                               acc[0][mt][2] + acc[1][mt][2], acc[0][mt][3] + acc[1][mt][3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(red_full + rb);
      if (++rb == GC_RED_BUFS) { rb = 0; red_wrapped = true; red_parity ^= 1; }
    }
    if (sliced) {
      // few slices: a warp may own several groups; many: one or none, and all its slices in one trip
      ok = op.slices <= 2   ? gc_finish_groups<MT, 4 / MT, 2>(A, op, r, slice, warp, ok)
           : op.slices <= 4 ? gc_finish_groups<MT, 2, 4 / MT>(A, op, r, slice, warp, ok)
                            : gc_finish_groups<MT, 1, 16 / MT>(A, op, r, slice, warp, ok);
      __syncwarp();
      if (lane == 0) mbar_arrive(fixed);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// The description of one operation as the caller gives it (plain C layout, read through ctypes).
struct ChainOpDesc {
  const void* W;
  const void* X;
  const float* norm_w;
  const float* bias;
  void* out;
  int ldx, ldo, M, N, K, epi, norm;
  float eps;
  int reserved;
};

// Bytes between rows of a stage (and of x) for `k` elements a row: pitch mod 128 = 64 keeps the
// 16-byte shared loads of eight rows on different banks.
static int chain_pitch(int k) { return k * 2 + ((k * 2) % 128 == 0 ? 64 : 0); }

enum { CUT_ONLY = 0, CUT_OR_SEQ = 1, CUT_SEQ_OR_WALK = 2 };
#define GC_WALK_X_BYTES (96 * 1024)      // most shared memory that x whole may take

// Cuts one operation: K into slices of at most `limit` elements, the slices either to different
// CTAs (their shares meet in scratch memory) or, where `ways` allows and it pays, one after the
// other to the same CTA.  Leaves the pitch of x for the caller where x is a slice (op.xp = 0).
static bool chain_cut(const ChainOpDesc& d, ChainOp& op, int sms, int limit, int ways) {
  if (sms <= 0) return false;
  if (d.M <= 0 || d.M > GC_MAX_M || d.N <= 0 || d.K <= 0 || d.K % 32) return false;
  if (((unsigned long long)d.W & 15) || ((unsigned long long)d.X & 15)) return false;
  if (d.norm ? (d.ldx % 4 || !d.norm_w) : (d.ldx % 8 != 0)) return false;
  if ((d.epi == EPI_SWIGLU && d.N % 16) || (d.epi == EPI_BIAS && !d.bias) || d.epi < 0 || d.epi > EPI_RESIDUAL) return false;
  op.W = (const bf16*)d.W; op.X = d.X; op.norm_w = d.norm_w; op.bias = d.bias; op.out = d.out;
  op.ldx = d.ldx; op.ldo = d.ldo; op.M = d.M; op.N = d.N; op.K = d.K; op.epi = d.epi; op.norm = d.norm; op.eps = d.eps;
  op.groups = (d.N + GC_ROWS - 1) / GC_ROWS;
  // nearly equal slices of whole k blocks; sms / slices CTAs work in each
  auto cut = [&](int slices, int& slice_k, int& ctas, double& busy) {
    slice_k = ((d.K + slices - 1) / slices + 31) / 32 * 32;
    if (slices > sms || (long long)(slices - 1) * slice_k >= d.K) return false;
    ctas = sms / slices < op.groups ? sms / slices : op.groups;
    busy = (double)op.groups * slices / ((double)((op.groups + ctas - 1) / ctas) * sms);     // share of the CTAs' time that is work
    return true;
  };
  double busy_cut;
  op.slices = (d.K + limit - 1) / limit;
  if (!cut(op.slices, op.slice_k, op.ctas, busy_cut)) return false;
  op.seq = 0;
  op.xp = 0;
  if (op.slices == 1) return true;
  const int seq_ctas = op.groups < sms ? op.groups : sms;
  const double busy_seq = (double)op.groups / ((double)((op.groups + seq_ctas - 1) / seq_ctas) * sms);
  // A K that is cut but not long: x whole in shared memory and every CTA walks the
  // slices of its groups, unless the groups divide so badly among the CTAs that way that the cut
  // across CTAs, with its pass of finishing, keeps a fifth more of them busy.
  if (ways >= CUT_SEQ_OR_WALK && GC_MAX_M * chain_pitch(d.K) <= GC_WALK_X_BYTES && busy_cut <= 1.2 * busy_seq) {
    op.seq = 2; op.ctas = seq_ctas; op.xp = chain_pitch(d.K);
    return true;
  }
  // A few more slices, not much shorter, when the CTAs then divide the work better (15 slices
  // employ 135 of 148 CTAs, 16 employ 144).
  for (int s = op.slices + 1; s <= op.slices + 3; ++s) {
    int slice_k, ctas;
    double busy;
    if (!cut(s, slice_k, ctas, busy) || slice_k * 100 < op.slice_k * 85) break;
    if (busy > 1.03 * busy_cut) { op.slices = s; op.slice_k = slice_k; op.ctas = ctas; busy_cut = busy; break; }
  }
  // Few groups per CTA, no norm: the slices one after the other
  // with the slices of x following them, unless the groups divide so badly among the CTAs that way
  // (224 groups on 148 CTAs: half of them stream a second group alone) that the cut across CTAs
  // keeps a tenth more of them busy.
  if (ways >= CUT_OR_SEQ && !d.norm && op.groups <= 2 * sms && busy_cut <= 1.1 * busy_seq) {
    op.seq = 1; op.ctas = seq_ctas;
  }
  return true;
}

// Shared memory of the kernel: the ring of stages, the partial-sum buffers and the barriers, then
// `x_bytes` for x.
// `stash`: bytes for a norm operation's weights behind x, if that costs no stage of the ring.
static int chain_smem(int rows, int pitch, int x_bytes, int stash, int& n_stages, int& x_off, int& stash_off) {
  const int MT = (rows + 7) / 8;
  const int red = GC_RED_BUFS * GC_CONSUMERS * 32 * MT * 4 * (int)sizeof(float);
  const int bars = 1024;
  const int slot = GC_ROWS * pitch;
  x_bytes = (x_bytes + 127) / 128 * 128;
  n_stages = (GC_SMEM_LIMIT - x_bytes - red - bars) / slot;
  if (n_stages > 24) n_stages = 24;
  stash = (stash + 127) / 128 * 128;
  x_off = n_stages * slot + red + bars;
  const bool room = stash > 0 && x_off + x_bytes + stash <= GC_SMEM_LIMIT;
  stash_off = room ? x_off + x_bytes : -1;
  return x_off + x_bytes + (room ? stash : 0);
}

// One way of cutting a whole chain: the operations into A.op, the pitch of the stages, and what x
// needs (the most of: a slice's rows, two buffers of them, or the rows whole).
static bool chain_cut_all(const ChainOpDesc* ops, int n_ops, int sms, int rows, int limit, int ways, ChainArgs& A, int& x_bytes, int& stash) {
  int kmax = 0;
  for (int i = 0; i < n_ops; ++i) {
    if (!chain_cut(ops[i], A.op[i], sms, limit, ways) || A.op[i].groups > 65536) return false;
    if (A.op[i].slice_k > kmax) kmax = A.op[i].slice_k;
  }
  A.pitch = chain_pitch(kmax);
  A.slot = GC_ROWS * A.pitch;
  x_bytes = stash = 0;
  for (int i = 0; i < n_ops; ++i) {
    ChainOp& op = A.op[i];
    if (op.seq != 2) op.xp = A.pitch;
    const int need = op.seq == 1 ? 2 * ((rows * A.pitch + 127) / 128 * 128) : rows * op.xp;
    if (need > x_bytes) x_bytes = need;
    const int w_bytes = (op.seq == 2 ? op.K : op.slice_k) * 4;
    if (op.norm && w_bytes <= 8192 && w_bytes > stash) stash = w_bytes;     // longer ones are read in place
  }
  return true;
}

// Cuts every operation of a chain and lays out shared memory.  What a CTA can have on its way
// from memory is the ring: stages x slice length, less the half stage that is on average being
// handed over (a ring of two leaves the copy engine idle from the moment a stage is handed over
// until it is free again).  Every way of cutting (x whole where possible; operations that keep
// two buffers of x; slices to different CTAs only) is tried with slice limits from 2048 down
// (rows of 2.3 KB still keep the copy engine's request rate above the memory's; an operation
// that fits in one slice is never cut for it), and marked by that length averaged over the
// operations' weights.  The best mark wins, except that x whole is taken from three quarters of
// the best mark on: it has nothing to finish afterwards.  Returns the kernel's shared memory in
// bytes, 0 if the chain cannot run.
static int chain_plan(const ChainOpDesc* ops, int n_ops, int sms, ChainArgs& A) {
  if (n_ops <= 0 || n_ops > GC_MAX_OPS) return 0;
  int whole = 0;
  for (int i = 0; i < n_ops; ++i)
    if (ops[i].K <= GC_SLICE_K && ops[i].K > whole) whole = ops[i].K;
  const int rows = GC_MAX_M;                     // shared memory is laid out for a full tile of rows
  double mark[3] = {-1.0, -1.0, -1.0};
  int limit_of[3] = {0, 0, 0}, x_bytes, stash, x_off;
  // slices shorter than 1152 only when nothing else can be had (a K just above 2048 has to be cut
  // in two of little more than 1024)
  for (int shortest = 1152; shortest >= 1024 && mark[0] < 0.0 && mark[1] < 0.0 && mark[2] < 0.0; shortest -= 128)
    for (int ways = CUT_ONLY; ways <= CUT_SEQ_OR_WALK; ++ways)
      for (int limit = GC_SLICE_K; limit >= 1152 && limit >= whole; limit -= 32) {
        if (!chain_cut_all(ops, n_ops, sms, rows, limit, ways, A, x_bytes, stash)) continue;
        chain_smem(rows, A.pitch, x_bytes, 0, A.n_stages, x_off, A.stash_off);
        if (A.n_stages < 2) continue;
        bool short_rows = false;
        for (int i = 0; i < n_ops; ++i) short_rows |= A.op[i].slices > 1 && A.op[i].slice_k < shortest;
        if (short_rows) continue;
        double sum = 0.0, weights = 0.0;
        for (int i = 0; i < n_ops; ++i) {
          const double w = (double)ops[i].N * ops[i].K;
          sum += w * (A.n_stages - 0.5) * A.op[i].slice_k;
          weights += w;
        }
        if (sum / weights > mark[ways] * 1.0001) { mark[ways] = sum / weights; limit_of[ways] = limit; }
      }
  int ways = mark[CUT_OR_SEQ] >= mark[CUT_ONLY] ? CUT_OR_SEQ : CUT_ONLY;
  if (mark[CUT_SEQ_OR_WALK] >= 0.75 * mark[ways]) ways = CUT_SEQ_OR_WALK;
  if (mark[ways] < 0.0) return 0;
  A.n_ops = n_ops;
  if (!chain_cut_all(ops, n_ops, sms, rows, limit_of[ways], ways, A, x_bytes, stash)) return 0;
  A.stash_bytes = stash;
  return chain_smem(rows, A.pitch, x_bytes, stash, A.n_stages, A.x_off, A.stash_off);
}

// Floats of scratch that a chain needs (0: no operation's slices meet there; -1: it cannot run).
Q25_EXPORT long long q25_gemm_chain_scratch_floats(const ChainOpDesc* ops, int n_ops) {
  ChainArgs A;
  if (!chain_plan(ops, n_ops, device_sm_count(), A)) return -1;
  long long most = 0;
  for (int i = 0; i < n_ops; ++i) {
    const ChainOp& op = A.op[i];
    if (op.slices > 1 && !op.seq) {
      const long long need = (long long)op.slices * op.groups * 128;
      if (need > most) most = need;
    }
  }
  return most;
}

// How a chain would be cut on a device of `sms` SMs, without touching a device: for tests of the
// planner and for whoever wants to see it.  out[i]: slices, slice_k, ctas, groups, seq, x pitch of
// operation i; returns the kernel's shared memory in bytes (0: the chain cannot run).
struct ChainPlanOp { int slices, slice_k, ctas, groups, seq, xp; };
Q25_EXPORT int q25_gemm_chain_plan(const ChainOpDesc* ops, int n_ops, int sms, int* n_stages, int* pitch, int* x_off,
                                   ChainPlanOp* out) {
  ChainArgs A;
  const int total = chain_plan(ops, n_ops, sms, A);
  if (!total) return 0;
  if (n_stages) *n_stages = A.n_stages;
  if (pitch) *pitch = A.pitch;
  if (x_off) *x_off = A.x_off;
  for (int i = 0; out && i < n_ops; ++i) {
    out[i].slices = A.op[i].slices; out[i].slice_k = A.op[i].slice_k; out[i].ctas = A.op[i].ctas;
    out[i].groups = A.op[i].groups; out[i].seq = A.op[i].seq; out[i].xp = A.op[i].xp;
  }
  return total;
}

// Whether the device can hold the whole grid at once (one CTA per SM), which the barrier needs.
Q25_EXPORT int q25_gemm_chain_available(void) {
  static int known = -1;
  if (known >= 0) return known;
  int dev = 0, coop = 0, sms = 0, smem = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  known = (coop && sms > 0 && smem >= GC_SMEM_LIMIT) ? 1 : 0;
  return known;
}

// Size of the description struct, so that a caller that builds it elsewhere can check its layout.
Q25_EXPORT int q25_gemm_chain_desc_bytes(void) { return (int)sizeof(ChainOpDesc); }

// CTAs of the kernel: one per SM of the current device.
Q25_EXPORT int q25_gemm_chain_grid(void) { return device_sm_count(); }

// Runs ops[0 .. n_ops) (at most 8 products of at most 8 rows) as one kernel; every operation may
// read what the ones before it wrote.  scratch: q25_gemm_chain_scratch_floats() floats; counters:
// 65536 ints, zero; barrier: one unsigned int whose value when the launch begins is barrier_base
// (each launch adds (n_ops - 1) * q25_gemm_chain_grid() to it); err: one int that receives a
// nonzero code if a wait gave up.
Q25_EXPORT int q25_gemm_chain_bf16(const ChainOpDesc* ops, int n_ops, float* scratch, int* counters, unsigned* barrier,
                                   unsigned barrier_base, int* err, void* stream) {
  if (n_ops <= 0) return 0;
  if (n_ops > GC_MAX_OPS || !counters || !barrier || !err || !q25_gemm_chain_available()) return (int)cudaErrorInvalidValue;
  ChainArgs A;
  const int total = chain_plan(ops, n_ops, device_sm_count(), A);
  if (!total || A.n_stages < 2) return (int)cudaErrorInvalidValue;
  A.scratch = scratch; A.counters = counters; A.barrier = barrier; A.barrier_base = barrier_base; A.err = err;
  for (int i = 0; i < n_ops; ++i)
    if (A.op[i].slices > 1 && !A.op[i].seq && !scratch) return (int)cudaErrorInvalidValue;
  void (*kernel)(const ChainArgs) = gemm_chain_kernel<1>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, total);
  if (e != cudaSuccess) return (int)e;
  launch(kernel, dim3(device_sm_count()), dim3(GC_THREADS), (size_t)total, (cudaStream_t)stream, A);
  e = (cudaError_t)launch_status();
  return (int)e;
}
