// Token selection on the device: argmax, temperature sampling, penalties.
//
// Reference (zhangjianbang-nb/qwen25vl-lite):
//   greedy       temperature <= 0 -> argmax (first maximum)      src/qwen25vl_lite/sampling.py:69-70
//   temperature  scores = float(logits) / T, softmax, one draw   src/qwen25vl_lite/sampling.py:72,103-106
//   keying       one random stream per (seed, index of the token being drawn)
//                                                                src/qwen25vl_lite/engine.py:823-829
//   penalties    seen tokens: positive logits / r, negative * r; minus presence; minus
//                frequency * count                               src/qwen25vl_lite/sampling.py:44-64
//
// The draw is Gumbel-max: argmax_i(score_i + g_i) with g_i = -log(-log(u_i)) is a sample of
// softmax(score).  u_i comes from a counter-based generator, so a row needs no scan and no
// state: key = mix(seed * GOLDEN + token_index), u_i = (top 23 bits of mix(key + i * ODD) + 0.5)
// / 2^23, mix = the splitmix64 finaliser.  This is not torch.multinomial's stream; the plain
// implementation of the test-suite restates it.
#include "common.cuh"

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

__device__ __forceinline__ float gumbel(unsigned long long key, int i) {
  const unsigned long long bits = mix64(key + (unsigned long long)i * 0xD1342543DE82EF95ull) >> 41;
  const float u = ((float)bits + 0.5f) * (1.0f / 8388608.0f);  // exact: 24-bit odd numerator
  return -logf(-logf(u));
}

// Value of candidate i of a row: the logit itself (greedy) or logit / T + Gumbel noise.
__device__ __forceinline__ float candidate(const float* lg, int i, bool draw, float t, unsigned long long key) {
  const float v = lg[i];
  return draw ? v / t + gumbel(key, i) : v;
}

__device__ __forceinline__ void better(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) { bv = v; bi = i; }
}

// Best (value, index) of the block's candidates; ties go to the lowest index.  Valid in thread 0.
__device__ __forceinline__ void block_best(float& bv, int& bi) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff) better(bv, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    for (int w = 1; w < nwarps; ++w)
      if (best_i[w] != 0x7fffffff) better(bv, bi, best_v[w], best_i[w]);
  }
}

// grid (chunks, rows): each block scans one chunk of a row's vocabulary.  With one chunk the
// winner is final; with more, partial winners go to `partial` and sample_final_kernel picks.
// temperature[row] <= 0: plain argmax.
__global__ void sample_rows_kernel(const float* __restrict__ logits, size_t ld, int vocab, int chunk,
                                   const float* __restrict__ temperature,
                                   const unsigned long long* __restrict__ seed,
                                   const int* __restrict__ token_index, int* __restrict__ out,
                                   float* __restrict__ partial_v, int* __restrict__ partial_i) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.y;
  const float* lg = logits + (size_t)row * ld;
  const float t = temperature ? temperature[row] : 0.f;
  const bool draw = t > 0.f;
  unsigned long long key = 0;
  if (draw) key = mix64(seed[row] * 0x9E3779B97F4A7C15ull + (unsigned long long)(long long)token_index[row]);
  const int begin = blockIdx.x * chunk, end = min(vocab, begin + chunk);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  // eight loads asked for together (a chunk of 4,096 is one such trip for 512 threads), then compared in order
  for (int i0 = begin + threadIdx.x; i0 < end; i0 += 8 * blockDim.x) {
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = i0 + k * blockDim.x;
      v[k] = i < end ? candidate(lg, i, draw, t, key) : -INFINITY;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = i0 + k * blockDim.x;
      if (i < end) better(bv, bi, v[k], i);
    }
  }
  block_best(bv, bi);
  if (threadIdx.x == 0) {
    if (gridDim.x == 1) {
      out[row] = bi == 0x7fffffff ? 0 : bi;
    } else {
      partial_v[(size_t)row * gridDim.x + blockIdx.x] = bv;
      partial_i[(size_t)row * gridDim.x + blockIdx.x] = bi;
    }
  }
}

__global__ void sample_final_kernel(const float* __restrict__ partial_v, const int* __restrict__ partial_i, int chunks,
                                    int* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const int i = partial_i[(size_t)row * chunks + c];
    if (i != 0x7fffffff) better(bv, bi, partial_v[(size_t)row * chunks + c], i);
  }
  block_best(bv, bi);
  if (threadIdx.x == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

// In place on logits[row]: ids/counts of row r are [offsets[r], offsets[r+1]).
__global__ void apply_penalties_kernel(float* __restrict__ logits, size_t ld, int vocab, const int* __restrict__ ids,
                                       const int* __restrict__ counts, const int* __restrict__ offsets,
                                       const float* __restrict__ repetition, const float* __restrict__ presence,
                                       const float* __restrict__ frequency) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  float* lg = logits + (size_t)row * ld;
  const float r = repetition[row], pr = presence[row], fr = frequency[row];
  for (int e = offsets[row] + threadIdx.x; e < offsets[row + 1]; e += blockDim.x) {
    const int id = ids[e];
    if (id < 0 || id >= vocab) continue;
    float v = lg[id];
    if (r != 1.0f) v = v > 0.f ? v / r : v * r;
    v -= pr;
    v -= fr * (float)counts[e];
    lg[id] = v;
  }
}

// Chunks a row is cut into: enough blocks to fill the GPU when there are few rows.
Q25_EXPORT int q25_sample_chunks(int rows, int vocab) {
  if (vocab < 16384) return 1;
  // chunks of 4,096: one trip to memory for a block, however many rows there are (64 rows in five
  // chunks each, 60 loads a thread one after the other, took 33 us for 39 MB)
  (void)rows;
  return (vocab + 4095) / 4096;
}

// scratch: 2 * rows * chunks 4-byte words when q25_sample_chunks(rows, vocab) > 1, else unused.
Q25_EXPORT int q25_sample_rows(const float* logits, long long ld, int rows, int vocab, const float* temperature,
                               const unsigned long long* seed, const int* token_index, int* out, void* scratch,
                               void* stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return (int)cudaErrorInvalidValue;
  const int chunks = q25_sample_chunks(rows, vocab);
  if (chunks > 1 && !scratch) return (int)cudaErrorInvalidValue;
  const int chunk = (vocab + chunks - 1) / chunks;
  const int threads = chunk > 2048 ? 512 : 256;
  float* pv = (float*)scratch;
  int* pi = (int*)scratch + (size_t)rows * chunks;
  launch(sample_rows_kernel, dim3(dim3(chunks, rows)), dim3(threads), 0, (cudaStream_t)stream, logits, (size_t)ld, vocab, chunk, temperature,
                                                                            seed, token_index, out, pv, pi);
  if (chunks > 1) launch(sample_final_kernel, dim3(rows), dim3(64), 0, (cudaStream_t)stream, pv, pi, chunks, out);
  return launch_status();
}

Q25_EXPORT int q25_apply_penalties(float* logits, long long ld, int rows, int vocab, const int* ids, const int* counts,
                                   const int* offsets, const float* repetition, const float* presence,
                                   const float* frequency, void* stream) {
  if (rows <= 0) return 0;
  launch(apply_penalties_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, logits, (size_t)ld, vocab, ids, counts, offsets,
                                                                 repetition, presence, frequency);
  return launch_status();
}
