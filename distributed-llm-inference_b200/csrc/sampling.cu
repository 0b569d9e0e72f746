// One token per row of float32 logits: argmax (lowest id on ties) for greedy rows; for the
// others temperature, top-k, top-p and one draw from the request's own counter-based stream.
//
// Stochastic rows, in the reference's order (divide by temperature, keep the k largest,
// softmax, drop a token once the mass of the strictly more likely ones reaches top_p, softmax
// again, draw) but without a sort: the k-th largest value and the top-p cut are found by
// bisection on the order-preserving integer image of the floats, and the draw inverts the
// cumulative distribution in ascending token id.  Ties at the k-th value are all kept.
// Every sum runs in an order fixed by the vocabulary size and the block size, so a row's
// token depends on its logits, its parameters and (seed, draw) only.
#include "common.cuh"
#include <math_constants.h>

using namespace dli;

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ uint32_t ordered_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

__device__ __forceinline__ unsigned block_sum_u32(unsigned v, unsigned* smem /* 33 */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned t = lane < (THREADS >> 5) ? smem[lane] : 0u;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) smem[32] = t;
  }
  __syncthreads();
  return smem[32];
}

__global__ void __launch_bounds__(THREADS) sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
                                                         long long row_stride, int V, const float* __restrict__ temperature,
                                                         const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                         const unsigned long long* __restrict__ seed,
                                                         unsigned long long* __restrict__ draw, const int* __restrict__ slots) {
  // With ``slots`` the five parameter arrays are tables indexed by the request's state slot (slots[row]) and a
  // stochastic row's draw count is advanced by one on the device; without it they are indexed by the row.
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float redf[33];
  __shared__ unsigned redu[33];
  __shared__ float wmax[32];
  __shared__ int widx[32];
  __shared__ float chunk_prefix[THREADS];
  __shared__ int found;

  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * row_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- argmax, lowest id on ties
  // (four logits a load where the row starts on a 16-byte boundary, several loads in flight: with one logit a load
  // the scan of 128 K logits by 1,024 threads waits for memory 125 times in a row and takes 10 us of the kernel's 12)
  float best = -CUDART_INF_F;
  int best_i = 0x7fffffff;
  int scanned = 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int n4 = V >> 2;
#pragma unroll 8
    for (int i = tid; i < n4; i += THREADS) {
      const float4 v = x4[i];
      if (v.x > best || best_i == 0x7fffffff) { best = v.x; best_i = 4 * i; }  // ids ascend within a thread
      if (v.y > best) { best = v.y; best_i = 4 * i + 1; }
      if (v.z > best) { best = v.z; best_i = 4 * i + 2; }
      if (v.w > best) { best = v.w; best_i = 4 * i + 3; }
    }
    scanned = n4 << 2;
  }
  for (int i = scanned + tid; i < V; i += THREADS) {
    const float v = x[i];
    if (v > best || best_i == 0x7fffffff) { best = v; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { wmax[warp] = best; widx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = wmax[lane]; best_i = widx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { wmax[0] = best; widx[0] = best_i; }
  }
  __syncthreads();
  const float xmax = wmax[0];
  const int arg = widx[0];

  const int at = slots ? slots[row] : row;
  const float T = temperature ? temperature[at] : 0.f;
  const int k = top_k ? top_k[at] : -1;
  if (T == 0.f || k == 1) {
    if (tid == 0) out[row] = arg;
    return;
  }
  const float P = top_p ? top_p[at] : 1.f;
  const float zmax = xmax / T;

  // ---- top-k: largest key K with count(key >= K) >= k
  uint32_t cut = 0u;  // keep tokens whose key >= cut
  if (k > 0 && k < V) {
    uint32_t lo = 0u, hi = ordered_key(zmax);  // count(key >= hi) >= 1, count(key >= 0) = V >= k
    // invariant: count(>= lo) >= k; find the largest such value
    while (lo < hi) {
      const uint32_t mid = lo + (uint32_t)(((unsigned long long)hi - lo + 1) >> 1);
      unsigned c = 0;
      for (int i = tid; i < V; i += THREADS) c += ordered_key(x[i] / T) >= mid;
      c = block_sum_u32(c, redu);
      if ((int)c >= k) lo = mid; else hi = mid - 1;
    }
    cut = lo;
  }

  // ---- softmax mass of the kept tokens
  float s = 0.f;
  for (int i = tid; i < V; i += THREADS) {
    const float z = x[i] / T;
    if (ordered_key(z) >= cut) s += expf(z - zmax);
  }
  const float mass_k = block_sum(s, redf);

  // ---- top-p: smallest key K with mass(key > K) < P * mass_k; keep key >= K
  if (P < 1.f) {
    const float limit = P * mass_k;
    uint32_t lo = cut, hi = ordered_key(zmax);  // mass(key > hi) = 0 < limit
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      float a = 0.f;
      for (int i = tid; i < V; i += THREADS) {
        const float z = x[i] / T;
        const uint32_t key = ordered_key(z);
        if (key > mid && key >= cut) a += expf(z - zmax);
      }
      a = block_sum(a, redf);
      if (a < limit) hi = mid; else lo = mid + 1;
    }
    cut = lo;
  }

  // ---- inverse CDF in ascending token id; thread t owns ids [t*per, (t+1)*per)
  const int per = (V + THREADS - 1) / THREADS;
  const int begin = min(V, tid * per), end = min(V, begin + per);
  float mine = 0.f;
  for (int i = begin; i < end; ++i) {
    const float z = x[i] / T;
    if (ordered_key(z) >= cut) mine += expf(z - zmax);
  }
  chunk_prefix[tid] = mine;
  if (tid == 0) found = 0x7fffffff;
  __syncthreads();
  if (tid == 0) {  // exclusive scan in id order (1024 additions, fixed order)
    float run = 0.f;
    for (int t = 0; t < THREADS; ++t) {
      const float c = chunk_prefix[t];
      chunk_prefix[t] = run;
      run += c;
    }
    redf[0] = run;
  }
  __syncthreads();
  const float total = redf[0];
  const unsigned long long this_draw = draw[at];
  uint32_t c[4] = {(uint32_t)this_draw, (uint32_t)(this_draw >> 32), 0u, 0u};
  philox4x32_10(c, (uint32_t)seed[at], (uint32_t)(seed[at] >> 32));
  const float u = (float)(c[0] >> 8) * (1.0f / 16777216.0f);
  const float target = u * total;
  const float before = chunk_prefix[tid];
  if (before <= target && target < before + mine) {
    float run = before;
    for (int i = begin; i < end; ++i) {
      const float z = x[i] / T;
      if (ordered_key(z) >= cut) {
        run += expf(z - zmax);
        if (run > target) { atomicMin(&found, i); break; }
      }
    }
  }
  __syncthreads();
  if (slots && tid == 0) draw[at] = this_draw + 1;  // every thread has read it; the request's next token is its next draw
  int result = found;
  if (result == 0x7fffffff) {  // rounding left the target at or past the end: last kept token
    if (tid == 0) widx[0] = -1;
    __syncthreads();
    for (int i = end - 1; i >= begin; --i)
      if (ordered_key(x[i] / T) >= cut) { atomicMax(&widx[0], i); break; }
    __syncthreads();
    result = widx[0];
  }
  if (tid == 0) out[row] = result;
}

}  // namespace

DLI_EXPORT int dli_sample(int* out, const float* logits, long long row_stride, int rows, int V, const float* temperature,
                          const int* top_k, const float* top_p, const unsigned long long* seed,
                          unsigned long long* draw, const int* slots, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (V < 1) return DLI_ERR_UNSUPPORTED;
  if (slots && !(temperature && top_k && top_p && seed && draw)) return DLI_ERR_UNSUPPORTED;
  launch_pdl((sample_kernel), dim3(rows), dim3(THREADS), 0, stream, 1, out, logits, row_stride, V, temperature, top_k, top_p, seed, draw, slots);
  return (int)cudaGetLastError();
}
