// y[M,N] = x[M,K] . W[N,K]^T for a handful of rows (decode steps: M = live requests <= 64), bf16.
//
// With so few rows the product is a stream of the weights: every byte of W is read once and
// used for M multiply-adds, so the kernel is built around keeping HBM busy, not the tensor cores.
// The weights take the 16-row side of mma.sync m16n8k16 (the roles of the operands are swapped:
// W is "A", x^T is "B"), which gives 8 batch columns per instruction and M/8 instructions per
// weight fragment.  Each thread loads 16 contiguous bytes of a weight row straight from global
// memory (no shared-memory staging) and feeds them to two MMAs; because a dot product does not
// care about the order of its terms, the 8 values are assigned to the MMA's k slots in the order
// they lie in memory, and x is read with the same assignment.  x is small and stays in L1/L2.
//
// A CTA has WARPS_N x WARPS_K warps: WARPS_N groups of 16 output features, each summed over K by
// WARPS_K warps that take contiguous K ranges and add up through shared memory in a fixed order.
// Epilogues: plain store, + float bias, float output (logits), and SwiGLU (rows come as 8 gate
// rows followed by their 8 up rows, so silu(gate) * up is formed in registers; reference formula
// src/qwen25vl_lite/text.py:66).
#include "common.cuh"

enum { EPI_STORE = 0, EPI_BIAS = 1, EPI_F32 = 2, EPI_SWIGLU = 3 };

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, int WARPS_N, int WARPS_K, int EPI>
__global__ void __launch_bounds__(WARPS_N * WARPS_K * 32)
gemm_skinny_kernel(const bf16* __restrict__ W, const bf16* __restrict__ X, int ldx, const float* __restrict__ bias,
                   void* __restrict__ out, int ldo, int M, int N, int K) {
  constexpr int UNROLL = 4;                        // 32-wide K blocks whose weight loads are in flight together
  __shared__ float red[WARPS_K > 1 ? (WARPS_K - 1) * WARPS_N * 16 * MT * 8 : 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int wn = warp % WARPS_N, wk = warp / WARPS_N;
  const int row0 = (blockIdx.x * WARPS_N + wn) * 16;
  const int kblocks = K / 32;
  const int per = (kblocks + WARPS_K - 1) / WARPS_K;
  const int kb_begin = wk * per, kb_end = min(kblocks, kb_begin + per);

  const bf16* w0 = W + (size_t)min(row0 + g, N - 1) * K + 8 * t;
  const bf16* w1 = W + (size_t)min(row0 + g + 8, N - 1) * K + 8 * t;
  const bf16* xr[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) xr[mt] = X + (size_t)min(mt * 8 + g, M - 1) * ldx + 8 * t;

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;

  int kb = kb_begin;
  for (; kb + UNROLL <= kb_end; kb += UNROLL) {
    uint4 a0[UNROLL], a1[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      a0[u] = ldg_stream(w0 + (size_t)(kb + u) * 32);
      a1[u] = ldg_stream(w1 + (size_t)(kb + u) * 32);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint4 b = *reinterpret_cast<const uint4*>(xr[mt] + (size_t)(kb + u) * 32);
        mma16816(acc[mt], a0[u].x, a1[u].x, a0[u].y, a1[u].y, b.x, b.y);
        mma16816(acc[mt], a0[u].z, a1[u].z, a0[u].w, a1[u].w, b.z, b.w);
      }
    }
  }
  for (; kb < kb_end; ++kb) {
    const uint4 a0 = ldg_stream(w0 + (size_t)kb * 32), a1 = ldg_stream(w1 + (size_t)kb * 32);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const uint4 b = *reinterpret_cast<const uint4*>(xr[mt] + (size_t)kb * 32);
      mma16816(acc[mt], a0.x, a1.x, a0.y, a1.y, b.x, b.y);
      mma16816(acc[mt], a0.z, a1.z, a0.w, a1.w, b.z, b.w);
    }
  }

  if constexpr (WARPS_K > 1) {   // sum over the K ranges, in warp order
    if (wk > 0) {
      float* dst = red + (((size_t)(wk - 1) * WARPS_N + wn) * 32 + lane) * MT * 4;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) dst[mt * 4 + e] = acc[mt][e];
    }
    __syncthreads();
    if (wk > 0) return;
#pragma unroll
    for (int k2 = 1; k2 < WARPS_K; ++k2) {
      const float* src = red + (((size_t)(k2 - 1) * WARPS_N + wn) * 32 + lane) * MT * 4;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] += src[mt * 4 + e];
    }
  }

  // accumulator (mt, e): output feature row0 + g + 8 * (e / 2), batch column mt * 8 + 2 t + (e & 1)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int m = mt * 8 + 2 * t + e;
      if (m >= M) continue;
      if constexpr (EPI == EPI_SWIGLU) {
        // rows g of this 16-row group are gate features, rows g + 8 the matching up features
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
          else reinterpret_cast<bf16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

template <int MT, int WARPS_N, int WARPS_K>
static int launch_epi(int epi, const bf16* W, const bf16* X, int ldx, const float* bias, void* out, int ldo, int M, int N,
                      int K, cudaStream_t s) {
  const dim3 grid((N + WARPS_N * 16 - 1) / (WARPS_N * 16)), block(WARPS_N * WARPS_K * 32);
  switch (epi) {
    case EPI_STORE: gemm_skinny_kernel<MT, WARPS_N, WARPS_K, EPI_STORE><<<grid, block, 0, s>>>(W, X, ldx, bias, out, ldo, M, N, K); break;
    case EPI_BIAS: gemm_skinny_kernel<MT, WARPS_N, WARPS_K, EPI_BIAS><<<grid, block, 0, s>>>(W, X, ldx, bias, out, ldo, M, N, K); break;
    case EPI_F32: gemm_skinny_kernel<MT, WARPS_N, WARPS_K, EPI_F32><<<grid, block, 0, s>>>(W, X, ldx, bias, out, ldo, M, N, K); break;
    case EPI_SWIGLU: gemm_skinny_kernel<MT, WARPS_N, WARPS_K, EPI_SWIGLU><<<grid, block, 0, s>>>(W, X, ldx, bias, out, ldo, M, N, K); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return launch_status();
}

template <int MT>
static int launch_shape(int epi, const bf16* W, const bf16* X, int ldx, const float* bias, void* out, int ldo, int M, int N,
                        int K, cudaStream_t s) {
  // Wide outputs: 4 feature groups per CTA, each warp sums all of K.  Narrow outputs would leave
  // SMs idle that way, so a CTA takes one group of 16 features and its warps split K.
  const long long wide_ctas = (N + 63) / 64;
  if (wide_ctas >= 2 * 148) return launch_epi<MT, 4, 1>(epi, W, X, ldx, bias, out, ldo, M, N, K, s);
  if (K >= 8192) return launch_epi<MT, 1, 8>(epi, W, X, ldx, bias, out, ldo, M, N, K, s);
  return launch_epi<MT, 1, 4>(epi, W, X, ldx, bias, out, ldo, M, N, K, s);
}

// epi: 0 store bf16, 1 + bias then store bf16, 2 store float, 3 SwiGLU pairs (N counts gate and up
// rows together, the output has N / 2 columns).  Needs K % 32 == 0, 1 <= M <= 64, 16-byte aligned rows.
Q25_EXPORT int q25_gemm_skinny_bf16(const void* W, const void* X, int ldx, const float* bias, void* out, int ldo, int M,
                                    int N, int K, int epi, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % 32 || ldx % 8 || (epi == EPI_SWIGLU && N % 16) || (epi == EPI_BIAS && !bias))
    return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const bf16* w = (const bf16*)W;
  const bf16* x = (const bf16*)X;
  if (M <= 8) return launch_shape<1>(epi, w, x, ldx, bias, out, ldo, M, N, K, s);
  if (M <= 16) return launch_shape<2>(epi, w, x, ldx, bias, out, ldo, M, N, K, s);
  if (M <= 32) return launch_shape<4>(epi, w, x, ldx, bias, out, ldo, M, N, K, s);
  return launch_shape<8>(epi, w, x, ldx, bias, out, ldo, M, N, K, s);
}
