// y[M,N] = x[M,K] . W[N,K]^T for a handful of rows (decode steps: M = live requests <= 16), bf16.
//
// With so few rows the product is a stream of the weights: every byte of W is read once and used
// for M multiply-adds, so the kernel is built around keeping HBM busy, not the tensor cores.
//
//   * One persistent CTA per SM takes groups of 16 output features (16 rows of W) in turn and walks
//     K in chunks of 1024 or 2048.  A producer warp brings each chunk into shared memory with one bulk
//     asynchronous copy per row (cp.async.bulk, 2 or 4 KB contiguous in global memory each) that signals
//     an mbarrier; a ring of stages keeps several chunks in flight, across group borders too,
//     while the eight consumer warps work.  x is copied once and stays in shared memory when it
//     fits; otherwise its part of each chunk travels with the chunk.
//   * The weights take the 16-row side of mma.sync m16n8k16 (the operands are swapped: W is "A",
//     x^T is "B"), 8 batch columns per instruction.  A thread reads 16 contiguous bytes of a row
//     from shared memory and feeds them to two MMAs; a dot product does not care about the order
//     of its terms, so the 8 values take the MMA's k slots in memory order and x is read with the
//     same assignment.
//   * The eight MMA warps take alternate 32-wide k blocks of every chunk; at the end of a group
//     they leave their partial sums in shared memory for an epilogue warp, which adds them in warp
//     order (so the result does not depend on timing) and stores, while the MMA warps go on.
//   * Epilogues: plain store, + float bias, float output (logits), and SwiGLU: the 16 rows come as
//     8 gate features followed by their 8 up features, so silu(gate) * up is formed in registers
//     (reference formula src/qwen25vl_lite/text.py:66).
//
// Every wait on an mbarrier is bounded: after MBAR_WAIT_LIMIT polls the kernel records an error code in
// *err, stops waiting anywhere, and runs to its end (its output is then invalid).
#include "common.cuh"

enum { EPI_STORE = 0, EPI_BIAS = 1, EPI_F32 = 2, EPI_SWIGLU = 3, EPI_RESIDUAL = 4 };

#define GS_ROWS 16
#define GS_CONSUMERS 8
#define GS_RED_BUFS 2                    // buffers of partial sums between the MMA warps and the epilogue warp
#define GS_THREADS ((GS_CONSUMERS + 2) * 32)
#define GS_SMEM_BUDGET (220 * 1024)       // shared memory a CTA may take
#define GS_KC_DEFAULT 1024                // K elements per chunk of a small product (2 KB rows)

__device__ __forceinline__ uint4 lds128(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared memory of a CTA:  x (when it stays resident: M rows of K values, pitch xp)  |  the ring of
// stages, each 16 weight rows of one chunk (and, when x is not resident, the M rows of x for that
// chunk)  |  buffers of per-warp partial sums  |  mbarriers: full[S], empty[S], x, red_full[], red_empty[].
struct SkinnyLayout {
  int xp;            // pitch of a resident x row in bytes (0: x travels with the chunks)
  int kc;            // K elements per chunk (a multiple of 64)
  int pitch;         // bytes between the rows of a chunk: kc * 2 + 64, so pitch mod 128 = 64 keeps 16-byte shared loads conflict-free
  int stage_bytes;
  int n_stages;
  size_t stages_off, red_off, bar_off, total;
};

static SkinnyLayout skinny_layout_kc(int M, int K, int MT, int kc) {
  SkinnyLayout L;
  L.kc = kc;
  L.pitch = L.kc * 2 + 64;
  const int n_chunks = (K + L.kc - 1) / L.kc;
  const size_t red = (size_t)GS_RED_BUFS * GS_CONSUMERS * 32 * MT * 4 * sizeof(float);
  const size_t bars = 64 * sizeof(unsigned long long);
  const int xrow = K * 2 + ((K * 2) % 128 == 0 ? 64 : 0);
  const size_t resident = (size_t)M * xrow;
  const bool fits = resident + 2 * (size_t)GS_ROWS * L.pitch + red + bars <= (size_t)GS_SMEM_BUDGET;
  L.xp = fits ? xrow : 0;
  const size_t xbytes = fits ? (resident + 127) / 128 * 128 : 0;
  L.stage_bytes = (GS_ROWS + (fits ? 0 : M)) * L.pitch;
  int s = (int)((GS_SMEM_BUDGET - xbytes - red - bars) / L.stage_bytes);
  // more stages than the chunks of four row groups would never fill
  L.n_stages = s > 4 * n_chunks ? 4 * n_chunks : (s > 24 ? 24 : s);
  if (L.n_stages < 1) L.n_stages = 1;
  L.stages_off = xbytes;
  L.red_off = L.stages_off + (size_t)L.n_stages * L.stage_bytes;
  L.bar_off = L.red_off + red;
  L.total = L.bar_off + bars;
  return L;
}

// The copy engine of an SM takes a bulk copy about every 100 cycles whatever its size (measured on
// B200: the time of a chunk did not change from 512-byte to 2 KB rows), so with 2 KB per row the
// requests, not the memory, bound a long stream at about 5 TB/s.  Large products therefore move
// 4 KB per row and request (two stages of 64 KB are in flight); small ones keep 2 KB rows, whose
// finer ring starts and drains faster.  Whether x stays resident does not depend on the choice.
static SkinnyLayout skinny_layout(int M, int N, int K, int MT) {
  const SkinnyLayout small = skinny_layout_kc(M, K, MT, GS_KC_DEFAULT);
  if ((long long)N * K < (32ll << 20) && K < 4096) return small;
  const SkinnyLayout large = skinny_layout_kc(M, K, MT, 2048);
  if (large.n_stages < 2 || (large.xp == 0) != (small.xp == 0) || large.total > (size_t)GS_SMEM_BUDGET) return small;
  return large;
}

// The epilogue warp: adds the MMA warps' partial sums in warp order and stores the 16 features of
// the group for every batch row.
template <int MT, int EPI>
__device__ __forceinline__ void skinny_epilogue(const float* red, unsigned long long* red_full, unsigned long long* red_empty,
                                                const float* __restrict__ bias, void* __restrict__ out, int ldo, int M,
                                                int N, int groups, int* err) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  bool ok = true;
  int round = 0;
  for (int grp = blockIdx.x; grp < groups; grp += gridDim.x, ++round) {
    const int b = round % GS_RED_BUFS;
    if (ok) {
      ok = mbar_wait(red_full + b, (round / GS_RED_BUFS) & 1);
      if (!ok && lane == 0) atomicExch(err, 5);
    }
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
#pragma unroll
    for (int w = 0; w < GS_CONSUMERS; ++w) {
      const float* src = red + (((size_t)b * GS_CONSUMERS + w) * 32 + lane) * MT * 4;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const float4 v = *reinterpret_cast<const float4*>(src + mt * 4);
        acc[mt][0] += v.x; acc[mt][1] += v.y; acc[mt][2] += v.z; acc[mt][3] += v.w;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(red_empty + b);

    // accumulator (mt, e): output feature row0 + g + 8 * (e / 2), batch column mt * 8 + 2 t + (e & 1)
    const int row0 = grp * GS_ROWS;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = mt * 8 + 2 * t + e;
        if (m >= M) continue;
        if constexpr (EPI == EPI_SWIGLU) {
          // rows g of the group are gate features, rows g + 8 the matching up features
          const int f = (row0 >> 1) + g;
          if (row0 + g + 8 < N) {
            const float gate = acc[mt][e], up = acc[mt][e + 2];
            reinterpret_cast<bf16*>(out)[(size_t)m * ldo + f] = __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
          }
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int n = row0 + g + 8 * h;
            if (n >= N) continue;
            float v = acc[mt][e + 2 * h];
            if constexpr (EPI == EPI_BIAS) v += bias[n];
            if constexpr (EPI == EPI_F32) reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v;
            else if constexpr (EPI == EPI_RESIDUAL) reinterpret_cast<float*>(out)[(size_t)m * ldo + n] += v;
            else reinterpret_cast<bf16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(v);
          }
        }
      }
    }
  }
}

// NORM: X is the float residual stream; the rows are RMS-normalised (x * rsqrt(mean(x^2) + eps) *
// norm_w, reference src/qwen25vl_lite/layers.py:27-31) into shared memory by the MMA warps while
// the first weight chunks are already on their way, so the norm costs no launch and no time.
template <int MT, int EPI, bool NORM>
__global__ void __launch_bounds__(GS_THREADS)
gemm_skinny_kernel(const bf16* __restrict__ W, const void* __restrict__ Xv, int ldx, const float* __restrict__ norm_w,
                   float eps, const float* __restrict__ bias, void* __restrict__ out, int ldo, int M, int N, int K,
                   SkinnyLayout L, int* __restrict__ err) {
  const bf16* X = reinterpret_cast<const bf16*>(Xv);
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* xs = smem;
  unsigned char* stages = smem + L.stages_off;
  float* red = reinterpret_cast<float*>(smem + L.red_off);
  unsigned long long* full = reinterpret_cast<unsigned long long*>(smem + L.bar_off);
  unsigned long long* empty = full + L.n_stages;
  unsigned long long* xbar = empty + L.n_stages;
  unsigned long long* red_full = xbar + 1;
  unsigned long long* red_empty = red_full + GS_RED_BUFS;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int KC = L.kc, PITCH = L.pitch;
  const int n_chunks = (K + KC - 1) / KC;
  const int groups = (N + GS_ROWS - 1) / GS_ROWS;
  const bool resident = L.xp != 0;
  const int S = L.n_stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, GS_CONSUMERS);
    }
    mbar_init(xbar, 1);
    for (int b = 0; b < GS_RED_BUFS; ++b) {
      mbar_init(red_full + b, GS_CONSUMERS);
      mbar_init(red_empty + b, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  // The weights are never written by a kernel, so their copies start at once; everything that
  // reads x or writes the output first waits for the kernels before this one (see common.cuh).
  pdl_trigger();
  if (warp == GS_CONSUMERS) {
    // ---- producer: one bulk copy per row and chunk, running ahead through the ring ----
    if (!resident) pdl_wait();                     // x travels with the chunks
    bool ok = true;
    int it = 0;
    const unsigned long long once = l2_evict_first();      // the weights pass through L2 once; what the step reads again stays
    for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
      const bf16* src = W + (size_t)min(grp * GS_ROWS + (lane & 15), N - 1) * K;
      for (int c = 0; c < n_chunks; ++c, ++it) {
        const int s = it % S;
        if (it >= S && ok) {
          ok = mbar_wait(empty + s, ((it / S) - 1) & 1);
          if (!ok && lane == 0) atomicExch(err, 1);
        }
        const unsigned bytes = (unsigned)min(KC, K - c * KC) * 2;
        unsigned char* st = stages + (size_t)s * L.stage_bytes;
        if (lane == 0) mbar_expect_tx(full + s, bytes * (GS_ROWS + (resident ? 0 : M)));
        __syncwarp();
        if (lane < GS_ROWS) bulk_copy_once(st + lane * PITCH, src + (size_t)c * KC, bytes, full + s, once);
        if (!resident && lane < M)
          bulk_copy(st + (GS_ROWS + lane) * PITCH, X + (size_t)lane * ldx + (size_t)c * KC, bytes, full + s);
      }
    }
    return;
  }

  if (warp == GS_CONSUMERS + 1) {
    pdl_wait();
    if (resident && !NORM) {                       // x stays resident: one copy per row, once
      if (lane == 0) mbar_expect_tx(xbar, (unsigned)M * K * 2);
      __syncwarp();
      if (lane < M) bulk_copy(xs + (size_t)lane * L.xp, X + (size_t)lane * ldx, (unsigned)K * 2, xbar);
    }
    skinny_epilogue<MT, EPI>(red, red_full, red_empty, bias, out, ldo, M, N, groups, err);
    return;
  }

  // ---- consumers (MMA warps) ----
  bool ok = true;
  if constexpr (NORM) {
    pdl_wait();
    const float* Xf = reinterpret_cast<const float*>(Xv);
    for (int m = warp; m < M; m += GS_CONSUMERS) {
      const float* xr = Xf + (size_t)m * ldx;
      float ss = 0.f;
      for (int k = lane * 4; k < K; k += 128) {
        const float4 v = *reinterpret_cast<const float4*>(xr + k);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      const float inv = rsqrtf(warp_sum(ss) / (float)K + eps);
      for (int k = lane * 4; k < K; k += 128) {
        const float4 v = *reinterpret_cast<const float4*>(xr + k);
        const float4 w = *reinterpret_cast<const float4*>(norm_w + k);
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * inv * w.x, v.y * inv * w.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * inv * w.z, v.w * inv * w.w);
        uint2 packed;
        packed.x = *reinterpret_cast<unsigned*>(&lo);
        packed.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(xs + (size_t)m * L.xp + (size_t)k * 2) = packed;
      }
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(GS_CONSUMERS * 32) : "memory");
  } else if (resident) {
    ok = mbar_wait(xbar, 0);
    if (!ok && lane == 0) atomicExch(err, 3);
  }
  // rows of x this thread reads for each 8-column tile (rows past M repeat the last one; their
  // columns are never stored)
  int xrow[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) xrow[mt] = min(mt * 8 + g, M - 1);

  int it = 0, round = 0;
  for (int grp = blockIdx.x; grp < groups; grp += gridDim.x, ++round) {
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
    for (int c = 0; c < n_chunks; ++c, ++it) {
      const int s = it % S;
      if (ok) {
        ok = mbar_wait(full + s, (it / S) & 1);
        if (!ok && lane == 0) atomicExch(err, 2);
      }
      const unsigned char* st = stages + (size_t)s * L.stage_bytes;
      const unsigned char* xb = resident ? xs + (size_t)c * KC * 2 : st + GS_ROWS * PITCH;
      const int xpitch = resident ? L.xp : PITCH;
      const int kblocks = min(KC, K - c * KC) / 32;
#pragma unroll 2
      for (int kb = warp; kb < kblocks; kb += GS_CONSUMERS) {
        const uint4 a0 = lds128(st + g * PITCH + kb * 64 + t * 16);
        const uint4 a1 = lds128(st + (g + 8) * PITCH + kb * 64 + t * 16);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint4 b = lds128(xb + (size_t)xrow[mt] * xpitch + kb * 64 + t * 16);
          mma16816(acc[mt], a0.x, a1.x, a0.y, a1.y, b.x, b.y);
          mma16816(acc[mt], a0.z, a1.z, a0.w, a1.w, b.z, b.w);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + s);
    }

    // hand the partial sums to the epilogue warp
    const int b = round % GS_RED_BUFS;
    if (round >= GS_RED_BUFS && ok) {
      ok = mbar_wait(red_empty + b, ((round / GS_RED_BUFS) - 1) & 1);
      if (!ok && lane == 0) atomicExch(err, 4);
    }
    float* dst = red + (((size_t)b * GS_CONSUMERS + warp) * 32 + lane) * MT * 4;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
      *reinterpret_cast<float4*>(dst + mt * 4) = make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
    __syncwarp();
    if (lane == 0) mbar_arrive(red_full + b);
  }
}

template <int MT, int EPI, bool NORM>
static int launch_skinny(const bf16* W, const void* X, int ldx, const float* norm_w, float eps, const float* bias, void* out,
                  int ldo, int M, int N, int K, int* err, cudaStream_t s) {
  const SkinnyLayout L = skinny_layout(M, N, K, MT);
  if (L.total > (size_t)GS_SMEM_BUDGET || (L.n_stages < 2 && (K + L.kc - 1) / L.kc > 1)) return (int)cudaErrorInvalidValue;
  if (NORM && L.xp == 0) return (int)cudaErrorInvalidValue;      // the normalised rows must stay resident
  cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MT, EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)L.total);
  if (e != cudaSuccess) return (int)e;
  const int groups = (N + GS_ROWS - 1) / GS_ROWS;
  const int sms = device_sm_count();
  if (sms <= 0) return (int)cudaErrorInvalidDevice;
  const int grid = groups < sms ? groups : sms;          // one persistent CTA per SM
  launch(gemm_skinny_kernel<MT, EPI, NORM>, dim3(grid), dim3(GS_THREADS), L.total, s, W, X, ldx, norm_w, eps, bias, out, ldo, M, N, K, L, err);
  return launch_status();
}

template <int MT, bool NORM>
static int launch_epi(int epi, const bf16* W, const void* X, int ldx, const float* norm_w, float eps, const float* bias,
                      void* out, int ldo, int M, int N, int K, int* err, cudaStream_t s) {
  switch (epi) {
    case EPI_STORE: return launch_skinny<MT, EPI_STORE, NORM>(W, X, ldx, norm_w, eps, bias, out, ldo, M, N, K, err, s);
    case EPI_BIAS: return launch_skinny<MT, EPI_BIAS, NORM>(W, X, ldx, norm_w, eps, bias, out, ldo, M, N, K, err, s);
    case EPI_F32: return launch_skinny<MT, EPI_F32, NORM>(W, X, ldx, norm_w, eps, bias, out, ldo, M, N, K, err, s);
    case EPI_SWIGLU: return launch_skinny<MT, EPI_SWIGLU, NORM>(W, X, ldx, norm_w, eps, bias, out, ldo, M, N, K, err, s);
    case EPI_RESIDUAL: return launch_skinny<MT, EPI_RESIDUAL, NORM>(W, X, ldx, norm_w, eps, bias, out, ldo, M, N, K, err, s);
    default: return (int)cudaErrorInvalidValue;
  }
}

// Whether x of M rows and K columns stays resident in shared memory (what the norm-fused variant needs).
Q25_EXPORT int q25_gemm_skinny_resident(int M, int K) {
  if (M <= 0 || M > 16 || K <= 0 || K % 32) return 0;
  return skinny_layout(M, 0, K, M <= 8 ? 1 : 2).xp != 0;
}

// epi: 0 store bf16, 1 + bias then store bf16, 2 store float, 3 SwiGLU pairs (N counts gate and up
// rows together, the output has N / 2 columns), 4 add into a float matrix (out[m][n] += y[m][n], the
// residual stream).  Needs K % 32 == 0, 1 <= M <= 16, 16-byte aligned rows of W and x.
// err: one int in device memory that receives a nonzero code if a wait gave up.
Q25_EXPORT int q25_gemm_skinny_bf16(const void* W, const void* X, int ldx, const float* bias, void* out, int ldo, int M,
                                    int N, int K, int epi, int* err, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 || ldx % 8 || (epi == EPI_SWIGLU && N % 16) || (epi == EPI_BIAS && !bias) || !err)
    return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (M <= 8) return launch_epi<1, false>(epi, (const bf16*)W, X, ldx, nullptr, 0.f, bias, out, ldo, M, N, K, err, s);
  return launch_epi<2, false>(epi, (const bf16*)W, X, ldx, nullptr, 0.f, bias, out, ldo, M, N, K, err, s);
}

// The same product on rmsnorm(X) * norm_w, X being float rows (the residual stream); the
// normalisation happens inside the kernel.  Needs q25_gemm_skinny_resident(M, K).
Q25_EXPORT int q25_gemm_skinny_norm_bf16(const void* W, const float* X, int ldx, const float* norm_w, float eps,
                                         const float* bias, void* out, int ldo, int M, int N, int K, int epi, int* err,
                                         void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 || ldx % 4 || !norm_w || (epi == EPI_SWIGLU && N % 16) || (epi == EPI_BIAS && !bias) || !err)
    return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (M <= 8) return launch_epi<1, true>(epi, (const bf16*)W, X, ldx, norm_w, eps, bias, out, ldo, M, N, K, err, s);
  return launch_epi<2, true>(epi, (const bf16*)W, X, ldx, norm_w, eps, bias, out, ldo, M, N, K, err, s);
}
