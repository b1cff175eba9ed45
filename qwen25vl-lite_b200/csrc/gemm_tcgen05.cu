// y[M,N] = x[M,K] . W[N,K]^T in bfloat16 on the 5th-generation tensor cores (tcgen05), for the
// many-row products of prefill.  Both operands are K-major (x rows and W rows are contiguous in K),
// the accumulator lives in tensor memory.
//
// One persistent CTA per SM, 6 warps with fixed roles:
//   warp 0   TMA producer: one lane issues cp.async.bulk.tensor loads of a 128 x 64 tile of x and a
//            BN x 64 tile of W (128-byte swizzle; BN = 256, or what fills the SMs best, see pick_bn)
//            into a ring of 4 to 6 shared-memory stages; each stage has a "full" mbarrier that counts
//            the bytes;
//   warp 1   MMA issuer: allocates 512 columns of tensor memory (two 128 x BN float accumulators),
//            then one lane issues tcgen05.mma (M 128, N BN, K 16) four times per stage and commits
//            to the stage's "empty" mbarrier, and after the last K block to the accumulator's
//            "full" mbarrier; while the epilogue drains one accumulator the next tile fills the other;
//   warps 2-5  epilogue: each reads its quarter of the 128 accumulator rows with tcgen05.ld (a lane
//            owns one row), applies the epilogue and stores straight to global memory.
// Epilogues as in gemm_chain.cu: store, + float bias, float output, SwiGLU on paired rows (8 gate
// features followed by their 8 up features; reference formula src/qwen25vl_lite/text.py:66), and
// add into the float residual stream.
//
// Tiles are walked with the row block fastest, so the CTAs that run together share W tiles through
// L2.  Edges: rows past M and features past N are zero-filled by TMA and masked at the store.
// Every mbarrier wait is bounded; a wait that gives up records a code in *err and the CTA runs to
// its end (freeing its tensor memory) with invalid output.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

enum { T5_STORE = 0, T5_BIAS = 1, T5_F32 = 2, T5_SWIGLU = 3, T5_RESIDUAL = 4 };

#define T5_BM 128
#define T5_BK 64
#define T5_A_BYTES (T5_BM * T5_BK * 2)
#define T5_MAX_STAGES 6

// The feature tile is `bn` wide, a multiple of 32 up to 256 that the host picks (pick_bn): a stage
// of the ring is 16 KB of x and bn x 128 bytes of W, and as many stages as fit in 200 KB, six at most
// (4 stages of 48 KB at 256, 6 of 32 KB at 128).
#define T5_MAX_BN 256
static inline int t5_stage_bytes(int bn) { return T5_A_BYTES + bn * T5_BK * 2; }
static inline int t5_stages(int bn) {
  const int s = (200 * 1024) / t5_stage_bytes(bn);
  return s > T5_MAX_STAGES ? T5_MAX_STAGES : s;
}
#define T5_THREADS 192

// 2-D tiled TMA load (no multicast): box at element coordinates (x = K index, y = row).
__device__ __forceinline__ void t5_tma_load(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

struct T5Shared {
  unsigned long long full[T5_MAX_STAGES], empty[T5_MAX_STAGES], acc_full[2], acc_empty[2];
  unsigned tmem_base;
};

// The epilogue of 32 consecutive features n .. n + 31 of row m, from their float sums (m < M, n < N).
template <int EPI>
__device__ __forceinline__ void t5_emit32(const float (&v)[32], int m, int n, int N, const float* __restrict__ bias,
                                          void* __restrict__ out, int ldo) {
  if constexpr (EPI == T5_SWIGLU) {
    // columns come in groups of 16: 8 gate features, then their 8 up features
    bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)m * ldo + (n >> 1);
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
      if (n + grp * 16 + 16 > N) break;
      __align__(16) bf16 o8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gate = v[grp * 16 + j], up = v[grp * 16 + 8 + j];
        o8[j] = __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
      }
      *reinterpret_cast<uint4*>(dst + grp * 8) = *reinterpret_cast<const uint4*>(o8);
    }
  } else if constexpr (EPI == T5_F32 || EPI == T5_RESIDUAL) {
    float* dst = reinterpret_cast<float*>(out) + (size_t)m * ldo + n;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (n + j >= N) break;
      if constexpr (EPI == T5_RESIDUAL) dst[j] += v[j];
      else dst[j] = v[j];
    }
  } else {
    bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)m * ldo + n;
    if (n + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        __align__(16) bf16 o8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float y = v[q * 8 + j];
          if constexpr (EPI == T5_BIAS) y += bias[n + q * 8 + j];
          o8[j] = __float2bfloat16_rn(y);
        }
        *reinterpret_cast<uint4*>(dst + q * 8) = *reinterpret_cast<const uint4*>(o8);
      }
    } else {
      for (int j = 0; j < 32 && n + j < N; ++j) {
        float y = v[j];
        if constexpr (EPI == T5_BIAS) y += bias[n + j];
        dst[j] = __float2bfloat16_rn(y);
      }
    }
  }
}

template <int EPI>
__global__ void __launch_bounds__(T5_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, void* __restrict__ out, int ldo, int M, int N, int K,
                    int bn, int n_stages, int* __restrict__ err) {
  const int T5_BN = bn, T5_STAGES = n_stages, T5_STAGE_BYTES = T5_A_BYTES + bn * T5_BK * 2;
  extern __shared__ __align__(1024) unsigned char t5_smem[];
  // the dynamic shared memory starts with the stages (1024-byte aligned for the swizzle), the barriers follow
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(t5_smem) + 1023) & ~(uintptr_t)1023);
  T5Shared* sh = reinterpret_cast<T5Shared*>(stages + T5_STAGES * T5_STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (M + T5_BM - 1) / T5_BM, n_blocks = (N + T5_BN - 1) / T5_BN;
  const int n_tiles = m_blocks * n_blocks;
  const int k_blocks = (K + T5_BK - 1) / T5_BK;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < T5_STAGES; ++s) {
      mbar_init(sh->full + s, 1);
      mbar_init(sh->empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(sh->acc_full + b, 1);
      mbar_init(sh->acc_empty + b, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // x was written by the kernel before this one; the output may still be read by it.  The tensor
  // memory is asked for only after that kernel has finished: a CTA that held columns while it waited
  // could starve a CTA of the earlier kernel on the same SM that still has to allocate its own.
  pdl_wait();
  if (warp == 1) {   // tensor memory: two accumulators of up to 256 columns (the CTA has its SM to itself)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh->tmem_base)), "n"(2 * T5_MAX_BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc5_fence_before();
  __syncthreads();
  tc5_fence_after();
  const unsigned tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ---- producer ----
    if (lane == 0) {
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int m0 = (tile % m_blocks) * T5_BM, n0 = (tile / m_blocks) * T5_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % T5_STAGES;
          if (it >= T5_STAGES && ok) {
            ok = mbar_wait(sh->empty + s, ((it / T5_STAGES) - 1) & 1);
            if (!ok) atomicExch(err, 11);
          }
          unsigned char* st = stages + (size_t)s * T5_STAGE_BYTES;
          mbar_expect_tx(sh->full + s, (unsigned)T5_STAGE_BYTES);
          t5_tma_load(st, &map_x, kb * T5_BK, m0, sh->full + s);
          t5_tma_load(st + T5_A_BYTES, &map_w, kb * T5_BK, n0, sh->full + s);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      bool ok = true;
      const unsigned idesc = tc5_idesc(T5_BN, false);
      int it = 0, tile_it = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tile_it) {
        const int b = tile_it & 1;
        if (tile_it >= 2 && ok) {
          ok = mbar_wait(sh->acc_empty + b, ((tile_it >> 1) - 1) & 1);
          if (!ok) atomicExch(err, 12);
        }
        tc5_fence_after();
        const unsigned acc = tmem_base + (unsigned)b * T5_MAX_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % T5_STAGES;
          if (ok) {
            ok = mbar_wait(sh->full + s, (it / T5_STAGES) & 1);
            if (!ok) atomicExch(err, 13);
          }
          tc5_fence_after();
          const unsigned a_addr = smem_u32(stages + (size_t)s * T5_STAGE_BYTES);
          const unsigned long long adesc = tc5_desc(a_addr, 16, 1024), bdesc = tc5_desc(a_addr + T5_A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < T5_BK / 16; ++k)   // 32 bytes further along K inside the swizzle atom: + 2 in the address field
            tc5_mma(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
          tc5_commit(sh->empty + s);
        }
        tc5_commit(sh->acc_full + b);
      }
    }
  } else {
    // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) .. + 31 ----
    const int quarter = warp & 3;
    bool ok = true;
    int tile_it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tile_it) {
      const int m0 = (tile % m_blocks) * T5_BM, n0 = (tile / m_blocks) * T5_BN;
      const int b = tile_it & 1;
      if (ok) {
        ok = mbar_wait(sh->acc_full + b, (tile_it >> 1) & 1);
        if (!ok && lane == 0) atomicExch(err, 14);
      }
      tc5_fence_after();
      const int m = m0 + quarter * 32 + lane;
      const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)b * T5_MAX_BN;
#pragma unroll 1
      for (int c = 0; c < T5_BN; c += 32) {
        float v[32];
        tc5_ld32(taddr + c, v);
        const int n = n0 + c;
        if (m >= M || n >= N) continue;
        t5_emit32<EPI>(v, m, n, N, bias, out, ldo);
      }
      tc5_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sh->acc_empty + b);
    }
  }

  // every warp gets here (all waits are bounded); then the tensor memory goes back
  tc5_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(2 * T5_MAX_BN) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// The same product on PAIRS of CTAs (tcgen05 with cta_group::2), for 256 rows and more.
//
// A cluster of two CTAs (on the two SMs of a pair) takes a tile of 256 rows x 256 features.  Each
// CTA loads its own 128 rows of x and its own 128 of the tile's 256 rows of W, two K blocks of 64 to
// a stage (64 KB; three stages.  Measured at 2,048 rows: 151 / 147 / 159 us for gate/up and
// 76 / 67 / 76 us for down with one / two / three K blocks a stage: fewer, larger stages save
// barrier round trips until too few are left to hide the loads); one thread of the first CTA issues tcgen05.mma.cta_group::2 (M 256, N 256, K 16), which
// reads both CTAs' shared memory at the same offsets and leaves each CTA's 128 rows x 256 columns of
// sums in that CTA's tensor memory.  Per instruction an SM reads half as many bytes of W from its
// shared memory as in the one-CTA kernel, whose tensor pipe waits for shared memory 27 % of the time.
//
// Who signals whom: the TMA loads of both CTAs count their bytes on the FIRST CTA's "full" barrier
// (the barrier operand with the peer bit cleared; that CTA's producer expects the bytes of both);
// the MMA thread's commits arrive at the "empty" barrier of the stage and at the accumulator's
// "full" barrier in BOTH CTAs (tcgen05.commit with a CTA mask); the epilogue warps of both CTAs
// arrive at the first CTA's accumulator-"empty" barrier (the second CTA's with a remote arrive).
// The loads use no cluster multicast.  Every wait is bounded; the two CTAs meet at a cluster barrier
// after the barriers are set up and before the tensor memory goes back.
#define P2_KPS 2                                        // K blocks of 64 in a stage
#define P2_STAGES 3
#define P2_BN 256
#define P2_HALF_BYTES (128 * T5_BK * 2)                 // this CTA's 128 of the tile's 256 rows of W, 64 values of K
#define P2_STAGE_BYTES (P2_KPS * (T5_A_BYTES + P2_HALF_BYTES))
#define P2_PEER_MASK 0xFEFFFFFFu                        // a shared-memory address of either CTA -> the same place in the first

struct P2Shared {
  unsigned long long full[P2_STAGES], empty[P2_STAGES], acc_full[2], acc_empty[2];
  unsigned tmem_base;
};

__device__ __forceinline__ unsigned p2_cta_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void p2_tma_load(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar) & P2_PEER_MASK), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void p2_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                      unsigned accumulate) {
  const unsigned zero = 0;     // no output lane is switched off
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}
// The MMAs issued so far are done: an arrival at this barrier in both CTAs of the pair.
__device__ __forceinline__ void p2_commit(unsigned long long* bar) {
  const unsigned short both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
// An arrival at the first CTA's barrier, from either CTA.
__device__ __forceinline__ void p2_arrive_first(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(smem_u32(bar) & P2_PEER_MASK) : "memory");
}
// bf16 x bf16 -> f32, M 256 over the pair, N n, both operands K-major.
__device__ __forceinline__ unsigned p2_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(256 >> 4) << 24);
}

// The tiles a pair takes: whole waves of 256 x 256 tiles round-robin; if the tiles left over fill
// at most half of the pairs, each is cut into two halves of 128 features, so that the last wave
// takes half as long (a prefill's gate/up product has 688 tiles for 74 pairs: 9 waves and 22 tiles).
struct P2Units {
  int n_pairs, pair, waves, rest, first_rest, count;
  bool halves;
  __device__ __forceinline__ P2Units(int n_tiles, int n_pairs_, int pair_) : n_pairs(n_pairs_), pair(pair_) {
    waves = n_tiles / n_pairs;
    first_rest = waves * n_pairs;
    rest = n_tiles - first_rest;
    halves = rest > 0 && 2 * rest <= n_pairs;
    count = waves + ((halves ? pair < 2 * rest : pair < rest) ? 1 : 0);
  }
  // unit i of this pair: its tile, the first feature inside the tile, and how many features wide it is
  __device__ __forceinline__ void get(int i, int& tile, int& n_off, int& width) const {
    if (i < waves) { tile = pair + i * n_pairs; n_off = 0; width = P2_BN; return; }
    if (halves) { tile = first_rest + (pair >> 1); n_off = (pair & 1) * 128; width = 128; return; }
    tile = first_rest + pair; n_off = 0; width = P2_BN;
  }
};

template <int EPI>
__global__ void __launch_bounds__(T5_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_w64, const float* __restrict__ bias, void* __restrict__ out, int ldo, int M, int N, int K,
                         int* __restrict__ err) {
  extern __shared__ __align__(1024) unsigned char t5_smem[];
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(t5_smem) + 1023) & ~(uintptr_t)1023);
  P2Shared* sh = reinterpret_cast<P2Shared*>(stages + P2_STAGES * P2_STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)p2_cta_rank();                  // 0: issues the MMAs and owns the barriers both CTAs signal
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int m_blocks = (M + 255) / 256, n_blocks = (N + P2_BN - 1) / P2_BN;
  const int n_tiles = m_blocks * n_blocks;
  const int k_blocks = (K + P2_KPS * T5_BK - 1) / (P2_KPS * T5_BK);     // stages of P2_KPS blocks of 64
  const P2Units units(n_tiles, n_pairs, pair);

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < P2_STAGES; ++s) {
      mbar_init(sh->full + s, 1);
      mbar_init(sh->empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(sh->acc_full + b, 1);
      mbar_init(sh->acc_empty + b, 8);                  // four epilogue warps of each CTA
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // x was written by the kernel before this one, the output may still be read by it, and tensor
  // memory is asked for only when that kernel has gone (see the one-CTA kernel)
  pdl_wait();
  cluster_sync();                                    // the other CTA's barriers exist before anything signals them
  if (warp == 1) {   // tensor memory: two accumulators of 256 columns, in both CTAs (the same warp of each asks)
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh->tmem_base)), "n"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  tc5_fence_before();
  __syncthreads();
  tc5_fence_after();
  const unsigned tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ---- producer (each CTA for its own halves) ----
    if (lane == 0) {
      bool ok = true;
      int it = 0;
      for (int u = 0; u < units.count; ++u) {
        int tile, n_off, width;
        units.get(u, tile, n_off, width);
        const int m0 = (tile % m_blocks) * 256 + rank * 128, n0 = (tile / m_blocks) * P2_BN + n_off + rank * (width / 2);
        const CUtensorMap* mw = width == P2_BN ? &map_w : &map_w64;      // boxes of 128 or of 64 rows of W
        const unsigned bytes = 2 * P2_KPS * (T5_A_BYTES + (unsigned)(width / 2) * T5_BK * 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % P2_STAGES;
          if (it >= P2_STAGES && ok) {
            ok = mbar_wait(sh->empty + s, ((it / P2_STAGES) - 1) & 1);
            if (!ok) atomicExch(err, 31);
          }
          unsigned char* st = stages + (size_t)s * P2_STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(sh->full + s, bytes);
#pragma unroll
          for (int j = 0; j < P2_KPS; ++j) {             // (a box past K is filled with zeros and still counts its bytes)
            p2_tma_load(st + j * (T5_A_BYTES + P2_HALF_BYTES), &map_x, (kb * P2_KPS + j) * T5_BK, m0, sh->full + s);
            p2_tma_load(st + j * (T5_A_BYTES + P2_HALF_BYTES) + T5_A_BYTES, mw, (kb * P2_KPS + j) * T5_BK, n0, sh->full + s);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one thread of the first CTA, for the pair ----
    if (lane == 0 && rank == 0) {
      bool ok = true;
      int it = 0;
      for (int tile_it = 0; tile_it < units.count; ++tile_it) {
        int tile, n_off, width;
        units.get(tile_it, tile, n_off, width);
        const unsigned idesc = p2_idesc(width);
        const int b = tile_it & 1;
        if (tile_it >= 2 && ok) {
          ok = mbar_wait(sh->acc_empty + b, ((tile_it >> 1) - 1) & 1);
          if (!ok) atomicExch(err, 32);
        }
        tc5_fence_after();
        const unsigned acc = tmem_base + (unsigned)b * P2_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % P2_STAGES;
          if (ok) {
            ok = mbar_wait(sh->full + s, (it / P2_STAGES) & 1);
            if (!ok) atomicExch(err, 33);
          }
          tc5_fence_after();
#pragma unroll
          for (int j = 0; j < P2_KPS; ++j) {
            const unsigned a_addr = smem_u32(stages + (size_t)s * P2_STAGE_BYTES + j * (T5_A_BYTES + P2_HALF_BYTES));
            const unsigned long long adesc = tc5_desc(a_addr, 16, 1024), bdesc = tc5_desc(a_addr + T5_A_BYTES, 16, 1024);
#pragma unroll
            for (int k = 0; k < T5_BK / 16; ++k) p2_mma(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | j | k) != 0);
          }
          p2_commit(sh->empty + s);
        }
        p2_commit(sh->acc_full + b);
      }
    }
  } else {
    // ---- epilogue: each CTA its own 128 rows; warp w reads TMEM lanes 32 (w % 4) .. + 31 ----
    const int quarter = warp & 3;
    bool ok = true;
    for (int tile_it = 0; tile_it < units.count; ++tile_it) {
      int tile, n_off, width;
      units.get(tile_it, tile, n_off, width);
      const int m0 = (tile % m_blocks) * 256 + rank * 128, n0 = (tile / m_blocks) * P2_BN + n_off;
      const int b = tile_it & 1;
      if (ok) {
        ok = mbar_wait(sh->acc_full + b, (tile_it >> 1) & 1);
        if (!ok && lane == 0) atomicExch(err, 34);
      }
      tc5_fence_after();
      const int m = m0 + quarter * 32 + lane;
      const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)b * P2_BN;
#pragma unroll 1
      for (int c = 0; c < width; c += 32) {
        float v[32];
        tc5_ld32(taddr + c, v);
        const int n = n0 + c;
        if (m >= M || n >= N) continue;
        t5_emit32<EPI>(v, m, n, N, bias, out, ldo);
      }
      tc5_fence_before();
      __syncwarp();
      if (lane == 0) p2_arrive_first(sh->acc_empty + b);
    }
  }

  // all threads of both CTAs get here (all waits are bounded): neither CTA leaves, or gives its
  // tensor memory back, while the other may still signal it or compute into it
  tc5_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(512) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// A [rows, K] bfloat16 row-major matrix with row pitch ld (elements), boxes of box_rows x 64.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {T5_BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int EPI>
static int launch_t5(const CUtensorMap& mx, const CUtensorMap& mw, const float* bias, void* out, int ldo, int M, int N, int K,
                     int bn, int* err, cudaStream_t s) {
  const int stages = t5_stages(bn);
  // the kernel may take the most any width needs: the attribute is set once per kernel, not per width
  const size_t most = (size_t)200 * 1024 + 1024 + sizeof(T5Shared);
  const size_t smem = (size_t)stages * t5_stage_bytes(bn) + 1024 + sizeof(T5Shared);
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
  if (e != cudaSuccess) return (int)e;
  const int tiles = ((M + T5_BM - 1) / T5_BM) * ((N + bn - 1) / bn);
  const int sms = device_sm_count();
  if (sms <= 0) return (int)cudaErrorInvalidDevice;
  launch(gemm_tcgen05_kernel<EPI>, dim3(tiles < sms ? tiles : sms), dim3(T5_THREADS), smem, s, mx, mw, bias, out, ldo, M, N, K,
         bn, stages, err);
  return launch_status();
}

template <int EPI>
static int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mw64, const float* bias, void* out,
                       int ldo, int M, int N, int K, int* err, cudaStream_t s) {
  const size_t smem = (size_t)P2_STAGES * P2_STAGE_BYTES + 1024 + sizeof(P2Shared);
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int sms = device_sm_count();
  if (sms < 2) return (int)cudaErrorInvalidDevice;
  const int tiles = ((M + 255) / 256) * ((N + P2_BN - 1) / P2_BN);
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(T5_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<EPI>, mx, mw, mw64, bias, out, ldo, M, N, K, err);
  if (e == cudaSuccess) e = cudaGetLastError();
  return (int)e;
}

// Width of the feature tile.  Up to 128 rows (one tile of rows: a decode step of that many requests)
// the product is a stream of the weights, a tile's time is its width, and the width is the multiple
// of 32 for which (waves of tiles over the SMs) x (width) is least: 22,016 features are 86 tiles of
// 256 on 148 SMs but 138 of 160 (23 -> 15 us), 37,888 are 148 of 256.  With more rows the 256-wide
// MMA counts: the 128-wide one does half the arithmetic for the same traffic of the x operand out
// of shared memory and runs at about 0.7 of it (measured), so it is only used when 256-wide tiles
// would leave more than half of the SMs without a tile.
static int pick_bn(int M, int N) {
  const int sms = device_sm_count();
  if (M > T5_BM) {
    const long long t256 = (long long)((M + T5_BM - 1) / T5_BM) * ((N + 255) / 256);
    return 2 * t256 <= sms ? 128 : 256;
  }
  int best = T5_MAX_BN;
  long long best_cost = -1;
  for (int bn = T5_MAX_BN; bn >= 64; bn -= 32) {
    const long long tiles = (N + bn - 1) / bn, cost = ((tiles + sms - 1) / sms) * bn;
    if (best_cost < 0 || cost < best_cost) { best = bn; best_cost = cost; }
  }
  return best;
}

// x: [M, K] bfloat16 with row pitch ldx; W: [N, K] bfloat16 contiguous.  epi as in gemm_chain.cu
// (0 store, 1 + bias, 2 float out, 3 SwiGLU pairs, 4 add into float out).  Needs K % 8 == 0,
// ldx % 8 == 0 and 16-byte aligned bases (TMA).  err: device int that gets a code if a wait gave up.
Q25_EXPORT int q25_gemm_tcgen05_bf16(const void* W, const void* X, int ldx, const float* bias, void* out, int ldo, int M,
                                     int N, int K, int epi, int* err, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ((uintptr_t)W & 15) || ((uintptr_t)X & 15) || !err || (epi == T5_SWIGLU && N % 16) ||
      (epi == T5_BIAS && !bias))
    return (int)cudaErrorInvalidValue;
  CUtensorMap mx, mw;
  int r = make_map(&mx, X, M, K, ldx, T5_BM);
  if (r) return r;
  cudaStream_t s = (cudaStream_t)stream;
  if (M >= 256 && N >= 256) {      // CTA pairs, tiles of 256 x 256: each CTA loads boxes of 128 rows of x and of W
    CUtensorMap mw64;
    r = make_map(&mw, W, N, K, K, 128);
    if (!r) r = make_map(&mw64, W, N, K, K, 64);
    if (r) return r;
    switch (epi) {
      case T5_STORE: return launch_pair<T5_STORE>(mx, mw, mw64, bias, out, ldo, M, N, K, err, s);
      case T5_BIAS: return launch_pair<T5_BIAS>(mx, mw, mw64, bias, out, ldo, M, N, K, err, s);
      case T5_F32: return launch_pair<T5_F32>(mx, mw, mw64, bias, out, ldo, M, N, K, err, s);
      case T5_SWIGLU: return launch_pair<T5_SWIGLU>(mx, mw, mw64, bias, out, ldo, M, N, K, err, s);
      case T5_RESIDUAL: return launch_pair<T5_RESIDUAL>(mx, mw, mw64, bias, out, ldo, M, N, K, err, s);
      default: return (int)cudaErrorInvalidValue;
    }
  }
  const int bn = pick_bn(M, N);
  r = make_map(&mw, W, N, K, K, bn);
  if (r) return r;
#define T5_CASE(E) \
  case E: return launch_t5<E>(mx, mw, bias, out, ldo, M, N, K, bn, err, s);
  switch (epi) {
    T5_CASE(T5_STORE)
    T5_CASE(T5_BIAS)
    T5_CASE(T5_F32)
    T5_CASE(T5_SWIGLU)
    T5_CASE(T5_RESIDUAL)
    default: return (int)cudaErrorInvalidValue;
  }
#undef T5_CASE
}
