// One token per row of float32 logits: argmax (lowest id on ties) for greedy rows; for the
// others temperature, top-k, top-p and one draw from the request's own counter-based stream.
//
// Stochastic rows, in the reference's order (divide by temperature, keep the k largest,
// softmax, drop a token once the mass of the strictly more likely ones reaches top_p, softmax
// again, draw) but without a sort.  A cluster of up to 8 CTAs holds the row's logits / T in
// shared memory (one read of the row), so every later pass runs on chip:
//   * the k-th largest value and the top-p cut are found by radix selection on the
//     order-preserving integer image of the floats, eight bits a pass: a histogram of 256 bins
//     per CTA (counts for top-k, probability mass for top-p), exchanged through distributed
//     shared memory, four passes each.  Ties at the k-th value are all kept.
//   * probability mass is summed as integers: exp(z - zmax) in units of 2^-40.  Integer sums do
//     not depend on their order, so the histograms, the totals and the cumulative distribution
//     are the same whatever the number of CTAs, warps or rows; a row's token depends on its
//     logits, its parameters and (seed, draw) only.
//   * the draw inverts the cumulative distribution in ascending token id: per-warp totals of
//     contiguous ranges locate the CTA and the warp that hold the target, and that one warp
//     walks its range.
// A batch of greedy rows only takes the plain argmax kernel below.
#include "common.cuh"
#include <math_constants.h>

using namespace dli;

namespace {

constexpr int THREADS = 1024;
constexpr int MAX_CLUSTER = 8;        // CTAs that share a row
constexpr int BINS = 256;             // eight bits of the key a pass
constexpr int SLICE_MAX = 47 * 1024;  // logits of a row that one CTA keeps (188 KB beside 38 KB of static shared memory)
constexpr float MASS_ONE = 1099511627776.0f;  // 2^40: the integer that stands for a probability ratio of 1
typedef unsigned long long u64;

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

// (value, id) with the larger value, the lower id on ties
__device__ __forceinline__ void take_better(float& best, int& best_i, float ov, int oi) {
  if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
}

// Argmax of x[begin .. end) over the block, lowest id on ties; every thread gets it.  Four logits a load where
// the range starts on a 16-byte boundary, several loads in flight: with one logit a load the scan of 128 K
// logits by 1,024 threads waits for memory 125 times in a row.  `store` (or null) receives x[i] * 1 or x[i] / T.
template <bool STORE>
__device__ __forceinline__ void block_argmax(const float* __restrict__ x, int begin, int end, float* __restrict__ store, float T,
                                             float* wmax, int* widx, float& out_v, int& out_i) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float best = -CUDART_INF_F;
  int best_i = 0x7fffffff;
  const float* xs = x + begin;
  const int n = end - begin;
  int scanned = 0;
  if ((reinterpret_cast<uintptr_t>(xs) & 15) == 0) {
    const float4* x4 = reinterpret_cast<const float4*>(xs);
    const int n4 = n >> 2;
#pragma unroll 8
    for (int i = tid; i < n4; i += THREADS) {
      const float4 v = x4[i];
      const int id = begin + 4 * i;
      if (v.x > best || best_i == 0x7fffffff) { best = v.x; best_i = id; }  // ids ascend within a thread
      if (v.y > best) { best = v.y; best_i = id + 1; }
      if (v.z > best) { best = v.z; best_i = id + 2; }
      if (v.w > best) { best = v.w; best_i = id + 3; }
      if (STORE) reinterpret_cast<float4*>(store)[i] = make_float4(v.x / T, v.y / T, v.z / T, v.w / T);
    }
    scanned = n4 << 2;
  }
  for (int i = scanned + tid; i < n; i += THREADS) {
    const float v = xs[i];
    if (v > best || best_i == 0x7fffffff) { best = v; best_i = begin + i; }
    if (STORE) store[i] = v / T;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) take_better(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
  if (lane == 0) { wmax[warp] = best; widx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = wmax[lane]; best_i = widx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) take_better(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
    if (lane == 0) { wmax[0] = best; widx[0] = best_i; }
  }
  __syncthreads();
  out_v = wmax[0];
  out_i = widx[0];
  __syncthreads();  // wmax and widx may be written again
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, long long row_stride, int V) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float wmax[32];
  __shared__ int widx[32];
  float v;
  int i;
  block_argmax<false>(logits + (size_t)blockIdx.x * row_stride, 0, V, nullptr, 1.f, wmax, widx, v, i);
  if (threadIdx.x == 0) out[blockIdx.x] = i;
}

// ---- the stochastic kernel: a cluster of gridDim.y CTAs per row (blockIdx.y = rank in the cluster)

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_address(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  return remote;
}
__device__ __forceinline__ void st_peer(uint32_t addr, u64 v) { asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory"); }

// exp(z - zmax), a number in [0, 1], in units of 2^-40 (rounded down)
__device__ __forceinline__ u64 mass_of(float z, float zmax) { return __float2ull_rz(expf(z - zmax) * MASS_ONE); }

struct Exchange {
  u64 recv[2][MAX_CLUSTER][BINS];  // the histograms of every CTA of the cluster, two passes deep
  unsigned hist[3][BINS];          // this CTA's histogram: counts in [0]; mass in three pieces of 14, 14 and 13 bits
  u64 tot[BINS];
  u64 wtot[32];
  u64 ctot[MAX_CLUSTER];
  u64 above;
  float amax[MAX_CLUSTER];
  int aidx[MAX_CLUSTER];
  float wmax[32];
  int widx[32];
  int bin;
};

// One lane of every group of lanes with the same bin adds the group's sum: the 256 bins are few, and in the first
// pass nearly all keys share two or three of them.  The additions are 32-bit (64-bit additions in shared memory
// are compare-and-swap loops): a mass, below 2^41, goes in three pieces, each of whose sums over a CTA's part of
// the row (fewer than 2^16 logits) stays below 2^32.
template <bool MASS>
__device__ __forceinline__ void hist_add(unsigned (*hist)[BINS], int bin /* BINS: nothing to add */, u64 v) {
  const unsigned group = __match_any_sync(0xffffffffu, bin);
  const bool adds = bin < BINS && (int)(threadIdx.x & 31) == __ffs(group) - 1;
  if (MASS) {
    const unsigned p0 = __reduce_add_sync(group, (unsigned)v & 0x3FFFu);
    const unsigned p1 = __reduce_add_sync(group, (unsigned)(v >> 14) & 0x3FFFu);
    const unsigned p2 = __reduce_add_sync(group, (unsigned)(v >> 28));
    if (adds) {
      atomicAdd(&hist[0][bin], p0);
      atomicAdd(&hist[1][bin], p1);
      atomicAdd(&hist[2][bin], p2);
    }
  } else if (adds) {
    atomicAdd(&hist[0][bin], (unsigned)__popc(group));
  }
}

// Radix selection over the keys of zs[0 .. n) of every CTA of the cluster, most significant byte first.
//   counts (MASS false): the largest key K with  #(key >= K) >= need
//   mass   (MASS true):  among keys >= floor_key, the smallest K with  mass(key > K) < top_p * mass(all), which is
//                        the largest K with mass(key >= K) >= that bound, the bound being at least one unit
// Both walk the bins from the top until the running sum reaches the bound.  Every CTA computes the same answer.
template <bool MASS>
__device__ uint32_t radix_select(const float* zs, int n, float zmax, uint32_t floor_key, u64 need, float top_p, Exchange& ex, int cluster,
                                 int rank, int& parity) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t prefix = 0, mask = 0;
  u64 above = 0;  // what the bins above the chosen ones hold
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < BINS) ex.hist[0][tid] = ex.hist[1][tid] = ex.hist[2][tid] = 0;
    __syncthreads();
    // four logits a thread and turn: after the first pass few keys still match the chosen bytes, and a warp whose
    // 128 logits hold none of them goes on at once
    const float4* z4 = reinterpret_cast<const float4*>(zs);
    const int n4 = (n + 3) >> 2;
    for (int base = 0; base < n4; base += THREADS) {
      const int q = base + tid;
      const float4 v = q < n4 ? z4[q] : make_float4(0.f, 0.f, 0.f, 0.f);
      const int left = n - 4 * q;  // how many of the four are logits of the row (none when q >= n4)
      const float z[4] = {v.x, v.y, v.z, v.w};
      uint32_t key[4];
      bool active[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        key[j] = ordered_key(z[j]);
        active[j] = j < left && (key[j] & mask) == prefix && (!MASS || key[j] >= floor_key);
      }
      if (!__any_sync(0xffffffffu, active[0] || active[1] || active[2] || active[3])) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        hist_add<MASS>(ex.hist, active[j] ? (int)((key[j] >> shift) & 255u) : BINS, MASS && active[j] ? mass_of(z[j], zmax) : 0);
    }
    __syncthreads();
    for (int j = tid; j < BINS * cluster; j += THREADS) {
      const int b = j & (BINS - 1);
      const u64 v = MASS ? (u64)ex.hist[0][b] + ((u64)ex.hist[1][b] << 14) + ((u64)ex.hist[2][b] << 28) : (u64)ex.hist[0][b];
      st_peer(peer_address(&ex.recv[parity][rank][b], (uint32_t)(j >> 8)), v);
    }
    cluster_sync();
    if (tid < BINS) {
      u64 t = 0;
      for (int r = 0; r < cluster; ++r) t += ex.recv[parity][r][tid];
      ex.tot[tid] = t;
    }
    __syncthreads();
    if (warp == 0) {  // lane l owns bins 8 l .. 8 l + 7; `over` = what the lanes above it hold
      u64 s = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) s += ex.tot[8 * lane + j];
      u64 incl = s;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const u64 t = __shfl_down_sync(0xffffffffu, incl, o);
        if (lane + o < 32) incl += t;
      }
      if (MASS && shift == 24) {  // the first pass saw every kept token: its total sets the bound
        const u64 total = __shfl_sync(0xffffffffu, incl, 0);
        u64 bound = (u64)ceil((double)top_p * (double)total);
        need = bound < 1 ? 1 : (bound > total ? total : bound);
      }
      const u64 over = above + incl - s;
      const bool here = over < need && over + s >= need;
      const unsigned found = __ballot_sync(0xffffffffu, here);
      if (here) {
        u64 run = over;
        for (int b = 8 * lane + 7; b >= 8 * lane; --b) {
          if (run + ex.tot[b] >= need) { ex.bin = b; ex.above = run; break; }
          run += ex.tot[b];
        }
      }
      if (!found && lane == 0) { ex.bin = 0; ex.above = over + s - ex.tot[0]; }  // fewer than the bound in all: keep everything
    }
    __syncthreads();
    prefix |= (uint32_t)ex.bin << shift;
    mask |= 255u << shift;
    above = ex.above;
    parity ^= 1;
  }
  return prefix;
}

// PER_SM: CTAs that share an SM.  Two (32 registers a thread, a few of them spilled) when the rows' CTAs outnumber
// the SMs: 64 rows then take two thirds of the time; one when they do not, so that the CTAs spread over the SMs.
template <int PER_SM>
__global__ void __launch_bounds__(THREADS, PER_SM) sample_cluster_kernel(int* __restrict__ out, const float* __restrict__ logits,
                                                                         long long row_stride, int V, int slice,
                                                                         const float* __restrict__ temperature, const int* __restrict__ top_k,
                                                                         const float* __restrict__ top_p, const u64* __restrict__ seed,
                                                                         u64* __restrict__ draw, const int* __restrict__ slots) {
  // With ``slots`` the five parameter arrays are tables indexed by the request's state slot (slots[row]) and a
  // stochastic row's draw count is advanced by one on the device; without it they are indexed by the row.
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float zs[];  // this CTA's part of the row, divided by the temperature
  __shared__ Exchange ex;

  const int row = blockIdx.x, rank = blockIdx.y, cluster = gridDim.y;
  const float* x = logits + (size_t)row * row_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int begin = min(V, rank * slice), end = min(V, begin + slice), n = end - begin;

  const int at = slots ? slots[row] : row;
  const float T = temperature[at];
  const int k = top_k[at];
  const float P = top_p[at];
  const u64 this_draw = draw[at], this_seed = seed[at];
  const bool greedy = T == 0.f || k == 1;

  // ---- argmax over the cluster (lowest id on ties), and logits / T into shared memory
  float best;
  int best_i;
  if (greedy) block_argmax<false>(x, begin, end, nullptr, 1.f, ex.wmax, ex.widx, best, best_i);
  else block_argmax<true>(x, begin, end, zs, T, ex.wmax, ex.widx, best, best_i);
  if (tid < cluster) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(peer_address(&ex.amax[rank], tid)), "f"(best) : "memory");
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(peer_address(&ex.aidx[rank], tid)), "r"(best_i) : "memory");
  }
  cluster_sync();
  float xmax = ex.amax[0];
  int arg = ex.aidx[0];
  for (int r = 1; r < cluster; ++r) take_better(xmax, arg, ex.amax[r], ex.aidx[r]);
  if (greedy || !(xmax > -CUDART_INF_F)) {  // (a row without one finite logit has no distribution)
    if (rank == 0 && tid == 0) out[row] = arg;
    return;
  }
  if (slots && rank == 0 && tid == 0) draw[at] = this_draw + 1;  // every CTA has read it; the request's next token is its next draw
  const float zmax = xmax / T;
  int parity = 0;

  // ---- top-k: the largest key with at least k keys at or above it; top-p: see radix_select
  uint32_t cut = 0u;  // tokens whose key >= cut are kept
  if (k > 0 && k < V) cut = radix_select<false>(zs, n, zmax, 0u, (u64)k, 1.f, ex, cluster, rank, parity);
  if (P < 1.f) cut = radix_select<true>(zs, n, zmax, cut, 0, P, ex, cluster, rank, parity);

  // ---- the kept mass of contiguous ranges: a warp's, a CTA's, the row's
  const int chunk = (((n + 31) >> 5) + 31) & ~31;  // ids per warp, a multiple of 32
  const int w0 = min(n, warp * chunk), w1 = min(n, w0 + chunk);
  u64 mine = 0;
  for (int i = w0 + lane; i < w1; i += 32) {
    const float z = zs[i];
    if (ordered_key(z) >= cut) mine += mass_of(z, zmax);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  if (lane == 0) ex.wtot[warp] = mine;
  __syncthreads();
  if (warp == 0) {
    u64 t = ex.wtot[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane < cluster) st_peer(peer_address(&ex.ctot[rank], lane), t);
  }
  cluster_sync();  // the last exchange: from here on nobody touches a peer's memory, so CTAs leave as they finish
  u64 total = 0, before = 0;
  for (int r = 0; r < cluster; ++r) {
    if (r == rank) before = total;
    total += ex.ctot[r];
  }

  // ---- the draw: the first token, in ascending id, whose cumulative mass exceeds u * total (u a multiple of 2^-24)
  uint32_t c[4] = {(uint32_t)this_draw, (uint32_t)(this_draw >> 32), 0u, 0u};
  philox4x32_10(c, (uint32_t)this_seed, (uint32_t)(this_seed >> 32));
  const u64 u24 = c[0] >> 8;
  const u64 target = (__umul64hi(total, u24) << 40) | ((total * u24) >> 24);  // floor(total * u24 / 2^24) < total
  if (target < before || target >= before + ex.ctot[rank]) return;
  u64 run = before;
  for (int w = 0; w < warp; ++w) run += ex.wtot[w];
  if (target < run || target >= run + ex.wtot[warp]) return;
  for (int base = w0; base < w1; base += 32) {
    const int i = base + lane;
    const float z = i < w1 ? zs[i] : 0.f;
    u64 incl = (i < w1 && ordered_key(z) >= cut) ? mass_of(z, zmax) : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u64 t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, run + incl > target);
    if (hit) {
      if (lane == __ffs(hit) - 1) out[row] = begin + i;
      return;
    }
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
}

}  // namespace

DLI_EXPORT int dli_sample(int* out, const float* logits, long long row_stride, int rows, int V, const float* temperature,
                          const int* top_k, const float* top_p, const unsigned long long* seed,
                          unsigned long long* draw, const int* slots, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (V < 1) return DLI_ERR_UNSUPPORTED;
  if (slots && !(temperature && top_k && top_p && seed && draw)) return DLI_ERR_UNSUPPORTED;
  if (!temperature) {
    launch_pdl((argmax_kernel), dim3(rows), dim3(THREADS), 0, stream, 1, out, logits, row_stride, V);
    return (int)cudaGetLastError();
  }
  if (!(top_k && top_p && seed && draw)) return DLI_ERR_UNSUPPORTED;
  // 16 logits or fewer per thread and pass; a CTA's part is a multiple of four logits, so that it starts on a
  // 16-byte boundary where the row does
  int cluster = 1;
  while (cluster < MAX_CLUSTER && V > 8192 * cluster) cluster *= 2;
  const int slice = (((V + cluster - 1) / cluster) + 3) & ~3;
  if (slice > SLICE_MAX) return DLI_ERR_UNSUPPORTED;
  const size_t smem = (size_t)slice * sizeof(float);
  const bool two = rows * cluster > sm_count() && 2 * (smem + sizeof(Exchange) + 1024) <= 227 * 1024;
  auto kernel = two ? sample_cluster_kernel<2> : sample_cluster_kernel<1>;
  static MaxPerDevice set[2];
  if ((int)smem > set[two].here()) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return (int)cudaGetLastError();
    set[two].here() = (int)smem;
  }
  launch_pdl(kernel, dim3(rows, cluster), dim3(THREADS), smem, stream, cluster, out, logits, row_stride, V, slice, temperature, top_k, top_p, seed,
             draw, slots);
  return (int)cudaGetLastError();
}
