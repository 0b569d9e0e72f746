// Paged causal GQA attention for prompt portions on the fifth-generation tensor cores
// (bfloat16, head size 64 — and 128 in the kernel with a thread per row —, page sizes 8..128 that divide 128).
//
// A CTA owns 128 rows — (token, query head) pairs that share one KV head — and walks the keys
// of its sequence in tiles of 128:
//
//   * TMA brings the tile's pages of K and V, [page_size x 64] boxes with 128-byte swizzle, straight
//     from the cache pools through the block table into two-stage shared-memory buffers;
//   * S = Q K^T is one group of tcgen05.mma (M = 128 rows, N = 128 keys, K = 64) into tensor memory;
//   * two threads share a row: each reads 64 of its 128 scores with tcgen05.ld, masks by absolute
//     position, keeps running maximum and sum in float32 (the halves meet through shared memory
//     once per tile), and writes its probabilities as bfloat16 into a swizzled shared-memory tile;
//   * O += P V is a second group of tcgen05.mma (V is the MN-major operand, exactly as it lies in
//     the pages), accumulated in tensor memory over all tiles; the threads rescale it in place only
//     when a row's maximum has grown by more than 2^8, and read it once, at the end.
//
// One warp issues the copies, one the matrix products; they meet each other and the softmax threads on
// mbarriers only.  Keys, values, scores and probabilities are double-buffered, so the tensor cores work
// one tile ahead of the softmax (one CTA per SM, 512 columns of tensor memory).  Every mbarrier wait is
// bounded: after WAIT_LIMIT polls the kernel sets *error_flag, stops using the tensor cores, frees its
// tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include <math_constants.h>

using namespace dli;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int D = 64;
constexpr int ROWS = 128;      // (token, head) rows per CTA
constexpr int KEYS = 128;      // keys per tile
constexpr int TILE_BYTES = 128 * 128;  // 128 rows of 128 bytes (Q, K, V tiles and each half of P)
constexpr int SOFTMAX_THREADS = 256;
constexpr int THREADS = SOFTMAX_THREADS + 64;  // plus a warp that issues the matrix products and a warp that issues the copies
constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 + 2 + 4) + 4 * ROWS * 4 + 256 + 1024;  // Q, K x2, V x2, P x2 (two halves each), row maxima x2, barriers, alignment
constexpr int TMEM_COLS = 512;  // S: 2 x 128 columns, the output: 64 columns (320, rounded up to a power of two)
constexpr unsigned WAIT_LIMIT = 1u << 24;

struct Params {
  bf16* out;
  const bf16* q;
  long long q_stride;
  const int* block_tables;
  int max_blocks;
  const int* q_start;
  const int* kv_len;
  int seq0, nh, nkv, page_size, window;
  float scale_log2;
  int tokens_per_tile, heads_per_chunk, head_chunks;
  int* error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// 128-byte-swizzled tiles: 1024 bytes between groups of eight rows (both for K-major operands and,
// along K, for the MN-major V operand); layout code 2; descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16, float32 accumulator, bfloat16 operands; A K-major; B K-major or MN-major
__device__ __forceinline__ uint32_t instr_desc(int m, int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
      "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
      "%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait that also gives up as soon as another thread has recorded a failure
__device__ __forceinline__ bool wait_or_fail(uint32_t bar, uint32_t parity, volatile int* failed, int code, int* error_flag) {
  for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 1023) == 1023 && *failed) return false;
  }
  *failed = code;
  atomicExch(error_flag, code);
  return false;
}

// 320 threads, one CTA per SM.  Warps 0..7 do the softmax: thread t works on row (t & 127); its half
// (t >> 7) owns 64 of the tile's 128 key columns and 32 of the 64 output columns (warps w and w + 4
// read the same 32 lanes of tensor memory: the lane group is the warp index modulo 4).  Warp 8 issues
// every tcgen05.mma from its first lane; warp 9 issues every TMA copy, one page per lane.
//
// Keys, values, the scores S (tensor memory) and the probabilities P (shared memory) exist twice,
// indexed by the tile's parity, so the tensor cores run one tile ahead of the softmax: S(i + 1) =
// Q K(i + 1)^T is issued as soon as the threads have read S(i - 1).  The output accumulates in tensor
// memory over all tiles: O += P(i) V(i).  The probabilities of a row are scaled by a reference maximum
// that follows the row's running maximum only when that has grown by more than 2^8; only then the
// threads multiply their part of O by 2^(old - new) in place (tcgen05.ld / tcgen05.st), which after the
// first tiles is rare.  The sides meet on mbarriers only (two of each, by parity):
//   k_full, v_full   TMA -> products             s_done, o_done   products -> softmax threads and TMA
//   p_ready (256)    P written, output rescaled, S read
__global__ void __launch_bounds__(THREADS, 1) paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                      const __grid_constant__ CUtensorMap map_v, const Params p) {
  pdl_launch_dependents();
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem;
  unsigned char* sK = sQ + TILE_BYTES;          // two stages
  unsigned char* sV = sK + 2 * TILE_BYTES;      // two stages
  unsigned char* sP = sV + 2 * TILE_BYTES;      // two buffers of (keys 0..63 | keys 64..127)
  float* row_max = (float*)(sP + 4 * TILE_BYTES);   // [2 (tile parity)][2 (half)][128]: each half's maximum of the tile, at the end its sum
  uint64_t* bars = (uint64_t*)(row_max + 4 * ROWS);  // k_full[2], v_full[2], s_done[2], o_done[2], p_ready[2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 10);
  volatile int* failed = (volatile int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = tid & (ROWS - 1), half = (tid >> 7) & 1;
  const uint32_t k_full = smem_u32(bars), v_full = smem_u32(bars + 2), s_done = smem_u32(bars + 4), o_done = smem_u32(bars + 6),
                 p_ready = smem_u32(bars + 8);

  // CTAs are handed out x first, z last: the tile index is z, counted from the end, so that over ALL heads and
  // sequences the tiles of the last tokens, which see the most keys, start first (with the tile index in x the
  // first wave held every head's short tiles and the last heads' longest tiles began late: 2,048 tokens on
  // 148 SMs took 72 us instead of 61)
  const int s = p.seq0 + blockIdx.y;
  const int tile = gridDim.z - 1 - blockIdx.z;
  const int kvh = blockIdx.x / p.head_chunks, hc = blockIdx.x - kvh * p.head_chunks;
  const int q0 = p.q_start[s];
  const int qlen = p.q_start[s + 1] - q0;
  const int tok0 = tile * p.tokens_per_tile;
  if (tok0 >= qlen) return;  // the whole CTA: nothing was set up yet
  const int kvlen = p.kv_len[s];
  const int ntok = min(p.tokens_per_tile, qlen - tok0);
  const int G = p.nh / p.nkv, Gc = p.heads_per_chunk;
  const int head0 = kvh * G + hc * Gc;
  const int nheads = min(Gc, G - hc * Gc);
  const int pos0 = kvlen - qlen + tok0;
  const int rows_used = ntok * Gc;
  const int* table = p.block_tables + (size_t)s * p.max_blocks;
  const int hi = pos0 + ntok;
  const int lo = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int t_begin = lo / KEYS, t_end = (hi + KEYS - 1) / KEYS;
  const int num_tiles = t_end - t_begin;

  if (tid == 0) {
    for (int i = 0; i < 8; ++i) mbar_init(k_full + 8 * i, 1);  // k_full, v_full, s_done, o_done
    for (int i = 0; i < 2; ++i) mbar_init(p_ready + 8 * i, SOFTMAX_THREADS);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();  // queries and the cache are the work of the kernels before this one

  // ---- Q tile, swizzled by hand: 16-byte chunk c of row r lies at r * 128 + ((c ^ (r & 7)) * 16);
  //      rows beyond the used ones are zero.  Both value stages start as zeros: pages beyond the
  //      sequence are never fetched, and their (masked) columns must not multiply garbage.
  for (int idx = tid; idx < ROWS * 8; idx += THREADS) {
    const int rr = idx >> 3, c = idx & 7;
    const int tok = rr / Gc, hd = rr - tok * Gc;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rr < rows_used && hd < nheads)
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + tok0 + tok) * p.q_stride + (size_t)(head0 + hd) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + rr * 128 + ((c ^ (rr & 7)) << 4)) = v;
  }
  for (int idx = tid; idx < 2 * TILE_BYTES / 16; idx += THREADS) reinterpret_cast<uint4*>(sV)[idx] = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  // tensor memory: S of even tiles, S of odd tiles, the output
  const uint32_t tmem_s = tmem, tmem_o = tmem + 2 * KEYS;

  if (warp == SOFTMAX_THREADS / 32 + 1) {
    // ================================================================ the warp that copies
    // The copies of a tile are issued by the whole warp, one page per lane (lanes 0..15 keys, lanes
    // 16..31 values): a single thread would spend microseconds on sixteen table look-ups and
    // address computations per tile.  A tile's stage is free once the product that read the tile
    // two before it has finished; the table entry of the next tile is asked for a tile ahead.
    const int pages = KEYS / p.page_size;
    const int page_i = lane & 15;
    auto lookup = [&](int t) -> int {  // this lane's page of tile t (absolute tile index), or -1 if it is not needed
      const int first = t * KEYS + page_i * p.page_size;
      const bool need = t < t_end && page_i < pages && first < hi && first + p.page_size > lo;
      return need ? table[first / p.page_size] : -1;
    };
    auto issue = [&](bool keys, int stage, int page) {  // called by the sixteen lanes of one side
      const uint32_t bar = (keys ? k_full : v_full) + 8 * stage;
      unsigned char* dst = (keys ? sK : sV) + stage * TILE_BYTES;
      const unsigned side = keys ? 0x0000ffffu : 0xffff0000u;
      const int count = __popc(__ballot_sync(side, page >= 0));
      if (page_i == 0) mbar_expect_tx(bar, (uint32_t)(count * p.page_size * 128));
      __syncwarp(side);
      if (page >= 0) tma_load_2d(smem_u32(dst + page_i * p.page_size * 128), keys ? &map_k : &map_v, 0, (page * p.nkv + kvh) * p.page_size, bar);
    };
    int page = lookup(t_begin);
    for (int t = 0; t < num_tiles && !*failed; ++t) {
      const int st = t & 1, par = ((t - 2) >> 1) & 1;
      const int cur = page;
      page = lookup(t_begin + t + 1);  // used an iteration from now
      if (t >= 2) {
        if (lane == 0) wait_or_fail(s_done + 8 * st, par, failed, 12, p.error_flag);  // Q K(t - 2)^T has read the stage
        __syncwarp();
        if (*failed) break;
      }
      if (lane < 16) issue(true, st, cur);
      if (t >= 2) {
        if (lane == 0) wait_or_fail(o_done + 8 * st, par, failed, 13, p.error_flag);  // P V(t - 2) has read the stage
        __syncwarp();
        if (*failed) break;
      }
      if (lane >= 16) issue(false, st, cur);
    }
  } else if (warp == SOFTMAX_THREADS / 32) {
    // ================================================================ the warp that issues the matrix products (its first lane)
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(ROWS, KEYS, 0), idesc_o = instr_desc(ROWS, D, 1);
      auto qk = [&](int t) {  // S(t) = Q K(t)^T once the keys have arrived
        const int b = t & 1;
        if (!wait_or_fail(k_full + 8 * b, (t >> 1) & 1, failed, 11, p.error_flag)) return;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = smem_u32(sQ), k = smem_u32(sK + b * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) umma(tmem_s + b * KEYS, smem_desc_sw128(a + kk * 32), smem_desc_sw128(k + kk * 32), idesc_s, kk != 0);
        umma_commit(s_done + 8 * b);
      };
      qk(0);
      for (int it = 0; it < num_tiles && !*failed; ++it) {
        const int b = it & 1, par = (it >> 1) & 1;
        // S(it + 1): its buffer held S(it - 1), which every thread had read when p_ready(it - 1) was seen (last iteration)
        if (it + 1 < num_tiles) qk(it + 1);
        // O += P(it) V(it): the probabilities are written (and the output rescaled where a row's maximum grew),
        // the values have arrived.  The output stays in tensor memory over all tiles.
        if (wait_or_fail(p_ready + 8 * b, par, failed, 15, p.error_flag) && wait_or_fail(v_full + 8 * b, par, failed, 14, p.error_flag)) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a = smem_u32(sP + b * 2 * TILE_BYTES), v = smem_u32(sV + b * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < KEYS / 16; ++k)
            umma(tmem_o, smem_desc_sw128(a + (k >> 2) * TILE_BYTES + (k & 3) * 32), smem_desc_sw128(v + k * 2048), idesc_o, (it | k) != 0);
          umma_commit(o_done + 8 * b);
        }
      }
    }
    __syncwarp();
  } else {
    // ================================================================ softmax threads
    const int rtok = r / Gc;
    const bool rvalid = r < rows_used && (r - rtok * Gc) < nheads;
    const int rpos = pos0 + rtok;
    const uint32_t lane_bits = (uint32_t)((warp & 3) * 32) << 16;
    const int col0 = half * 64;
    // m: running maximum of the row's raw scores; m_ref: the maximum that the probabilities and the output
    // are scaled by at present; l: this half's share of the row sum (in that scale).  m_ref follows m only
    // when m has grown by more than RESCALE_STEP (in powers of two): the output, which accumulates in
    // tensor memory over all tiles, then has to be multiplied by 2^(old - new), and that is rare after the
    // first tiles.  Probabilities thus reach at most 2^RESCALE_STEP, which bfloat16 and the float32 sums hold
    // with the same relative precision.
    constexpr float RESCALE_STEP = 8.f;
    float m = -CUDART_INF_F, m_ref = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    const int group = r >> 6;  // rows 0..63 (warps 0, 1, 4, 5) and rows 64..127 (warps 2, 3, 6, 7)
    const uint32_t my_o = tmem_o + lane_bits + half * 32;  // output columns 32 * half .. 32 * half + 31 of the row

    for (int it = 0; it < num_tiles; ++it) {
      const int b = it & 1;
      const int base = (t_begin + it) * KEYS;
      ok = wait_or_fail(s_done + 8 * b, (it >> 1) & 1, failed, 12, p.error_flag) && ok;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // a tile that lies wholly at or before the first row's position, inside every row's window, needs no mask
      const bool full = base + KEYS - 1 <= pos0 && base >= lo && p.window <= 0;
      // ---- this thread's 64 raw scores, read once; masked ones become -inf.  Rows that hold no query
      //      (zeros in Q) are computed like the others and never written out.
      //      (Read also after a failed wait: nothing is stored then, and one way only for the scores to get their
      //      values saves a register move per score.)
      float sc[64];
      {
        uint32_t v0[32], v1[32];
        tmem_ld32_nowait(tmem_s + b * KEYS + lane_bits + col0, v0);
        tmem_ld32_nowait(tmem_s + b * KEYS + lane_bits + col0 + 32, v1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) { sc[j] = __uint_as_float(v0[j]); sc[32 + j] = __uint_as_float(v1[j]); }
      }
      if (!full) {
        const int first = base + col0;  // visible: first + j in (rpos - window, rpos]
        const int hi_j = rpos - first, lo_j = p.window > 0 ? rpos - p.window - first : -1;
#pragma unroll
        for (int j = 0; j < 64; ++j) sc[j] = (j <= hi_j && j > lo_j) ? sc[j] : -CUDART_INF_F;
      }
      float mx[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) mx[j] = sc[j];
#pragma unroll
      for (int j = 8; j < 64; ++j) mx[j & 7] = fmaxf(mx[j & 7], sc[j]);
      mx[0] = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      mx[4] = fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]));
      float* rm = row_max + b * 2 * ROWS;  // by parity: a fast thread's next tile writes the other buffer
      rm[half * ROWS + r] = fmaxf(mx[0], mx[4]);
      if (group == 0) asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_THREADS / 2) : "memory");  // the two halves of this row's 64-row group
      else asm volatile("bar.sync 2, %0;" ::"n"(SOFTMAX_THREADS / 2) : "memory");
      m = fmaxf(m, fmaxf(rm[r], rm[ROWS + r]));
      float corr = 1.f;
      const bool grown = (m - m_ref) * p.scale_log2 > RESCALE_STEP;  // also the first finite maximum (m_ref = -inf)
      if (grown) {
        corr = (m_ref == -CUDART_INF_F) ? 0.f : ex2((m_ref - m) * p.scale_log2);  // nothing finite was accumulated before
        m_ref = m;
      }
      const float neg = (m_ref == -CUDART_INF_F) ? 0.f : -m_ref * p.scale_log2;
      // P's buffer was read by the product of tile it - 2
      if (it >= 2) ok = wait_or_fail(o_done + 8 * b, ((it - 2) >> 1) & 1, failed, 13, p.error_flag) && ok;
      // the output so far, multiplied by 2^(old - new) in the rows whose reference moved (the whole warp
      // reads and writes tensor memory together, rows that did not move with factor 1)
      if (it > 0 && __any_sync(0xffffffffu, grown)) {
        ok = wait_or_fail(o_done + 8 * (b ^ 1), ((it - 1) >> 1) & 1, failed, 13, p.error_flag) && ok;  // the product of tile it - 1 has finished
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
          uint32_t v[32];
          tmem_ld32_nowait(my_o, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
          tmem_st32(my_o, v);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      // ---- probabilities, their sum, and the bfloat16 tile for the P V product
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      unsigned char* prow = sP + b * 2 * TILE_BYTES + half * TILE_BYTES + r * 128;
      // in three sweeps, so that the 64 exponentials follow each other without waiting for anything
#pragma unroll
      for (int j = 0; j < 64; ++j) sc[j] = fmaf(sc[j], p.scale_log2, neg);
#pragma unroll
      for (int j = 0; j < 64; ++j) sc[j] = ex2(sc[j]);  // masked: ex2(-inf) = 0
#pragma unroll
      for (int j = 0; j < 64; j += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          sum[(e >> 1) & 3] += sc[j + e] + sc[j + e + 1];
          __nv_bfloat162 b2 = __floats2bfloat162_rn(sc[j + e], sc[j + e + 1]);
          packed[e >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
        *reinterpret_cast<uint4*>(prow + (((j >> 3) ^ (r & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
      l = l * corr + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P is read by the tensor cores
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(p_ready + 8 * b);  // P is written, the output rescaled and S read: P V and the Q K^T of tile it + 2 may be issued

    }
    // ---- the finished output, once the last product is done
    float o[32];
    ok = wait_or_fail(o_done + 8 * ((num_tiles - 1) & 1), ((num_tiles - 1) >> 1) & 1, failed, 13, p.error_flag) && ok;
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      uint32_t v[32];
      tmem_ld32_nowait(my_o, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 0; j < 32; ++j) o[j] = __uint_as_float(v[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) o[j] = 0.f;
    }

    // ---- the row sum is the two halves' sums; each half writes its 32 output columns
    float* rl = row_max + (num_tiles & 1) * 2 * ROWS;  // not the buffer of the last tile's maxima
    rl[half * ROWS + r] = l;
    if (group == 0) asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_THREADS / 2) : "memory");
    else asm volatile("bar.sync 2, %0;" ::"n"(SOFTMAX_THREADS / 2) : "memory");
    if (!*failed && rvalid) {
      const float inv = 1.f / (rl[r] + rl[ROWS + r]);
      const size_t row = (size_t)(q0 + tok0 + rtok) * p.nh + head0 + (r - rtok * Gc);
      uint4* dst = reinterpret_cast<uint4*>(p.out + row * D + half * 32);
#pragma unroll
      for (int c = 0; c < 32; c += 8) {
        uint4 w;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
        for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(o[c + 2 * e] * inv, o[c + 2 * e + 1] * inv);
        dst[c >> 3] = w;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

// ================================================================ two query tiles per CTA
// The same products, arranged so that the special-function units (16 exponentials per clock per SM,
// a quarter of them per scheduler) never wait: a CTA owns two query tiles of 128 rows, A and B, that
// read the same keys and values.  A row belongs to one thread (warps 0..3: tile A, warps 4..7: tile B;
// a scheduler holds one warp of each), which reads its 128 scores into registers at once, so a
// tile's S is free for the next product at once, and needs no other thread for its maximum.  The two
// groups take turns at the exponentials (named barriers): while A computes its probabilities, B
// reads scores, takes maxima, rescales its output and hands in P, and the other way round.  The
// third warpgroup has a warp per job: the products of tile A, the copies of keys, the products of
// tile B, the copies of values.
//   k_full, v_full [2]     TMA -> products              k_free, v_free [2]   products done -> TMA
//   s_done [A, B]          S there                      s_read [A, B] (128)  S in registers
//   p_ready [A, B] (128)   P written, output rescaled   o_done [A, B]        O += P V finished
// Head size 64: two query tiles per CTA.  Head size 128: one (its Q, K and V tiles are twice as large), so the
// group has no partner; a row of keys or values is then two 128-byte slabs, each with its own TMA box, the
// score product runs over both, and the output product is one group of tcgen05.mma per slab of 64 columns.
template <int HD>
struct T2Cfg {
  static_assert(HD == 64 || HD == 128, "head sizes with whole 128-byte slabs");
  static constexpr int QT = HD == 64 ? 2 : 1;             // query tiles per CTA
  static constexpr int SLABS = HD / 64;
  static constexpr int THREADS = QT * ROWS + 128;         // softmax warpgroups and one whose warps issue the products (one per query tile) and the copies (keys, values)
  static constexpr int KV_BYTES = SLABS * TILE_BYTES;     // one stage of keys or of values; also one Q tile
  static constexpr int SMEM = QT * KV_BYTES + 4 * KV_BYTES + QT * 2 * TILE_BYTES + 256 + 1024;  // Q, K x2, V x2, P per query tile, barriers, alignment
  static constexpr int TMEM = QT * KEYS + QT * HD <= 256 ? 256 : 512;
};

// Pairs of float32 in a 64-bit register, for the instructions that work on both at once (sm_100).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// the largest of three (one instruction on sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <int HD>
__global__ void __launch_bounds__(T2Cfg<HD>::THREADS, 1) paged_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                                  const __grid_constant__ CUtensorMap map_v, const Params p) {
  using Cfg = T2Cfg<HD>;
  constexpr int QT = Cfg::QT, SLABS = Cfg::SLABS, KV_BYTES = Cfg::KV_BYTES, T2_THREADS = Cfg::THREADS;
  constexpr int D = HD;  // shadows the one-tile kernel's head size within this kernel
  pdl_launch_dependents();
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem;                     // tile A (, tile B); a tile is SLABS slabs of [128 rows x 128 bytes]
  unsigned char* sK = sQ + QT * KV_BYTES;       // two stages
  unsigned char* sV = sK + 2 * KV_BYTES;        // two stages
  unsigned char* sP = sV + 2 * KV_BYTES;        // per query tile (keys 0..63 | keys 64..127)
  uint64_t* bars = (uint64_t*)(sP + QT * 2 * TILE_BYTES);
  uint32_t* tmem_slot = (uint32_t*)(bars + 16);
  volatile int* failed = (volatile int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t k_full = smem_u32(bars), v_full = smem_u32(bars + 2), k_free = smem_u32(bars + 4), v_free = smem_u32(bars + 6),
                 s_done = smem_u32(bars + 8), s_read = smem_u32(bars + 10), p_ready = smem_u32(bars + 12), o_done = smem_u32(bars + 14);

  // CTAs are handed out x first, z last: the tile index is z, counted from the end, so that over ALL heads and
  // sequences the tiles of the last tokens, which see the most keys, start first (with the tile index in x the
  // first wave held every head's short tiles and the last heads' longest tiles began late: 2,048 tokens on
  // 148 SMs took 72 us instead of 61)
  const int s = p.seq0 + blockIdx.y;
  const int tile = gridDim.z - 1 - blockIdx.z;
  const int kvh = blockIdx.x / p.head_chunks, hc = blockIdx.x - kvh * p.head_chunks;
  const int q0 = p.q_start[s];
  const int qlen = p.q_start[s + 1] - q0;
  const int tpt = p.tokens_per_tile;
  const int tok0 = tile * QT * tpt;
  if (tok0 >= qlen) return;  // the whole CTA: nothing was set up yet
  const int kvlen = p.kv_len[s];
  const int ntok = min(QT * tpt, qlen - tok0);  // tokens of the CTA's tiles
  const int G = p.nh / p.nkv, Gc = p.heads_per_chunk;
  const int head0 = kvh * G + hc * Gc;
  const int nheads = min(Gc, G - hc * Gc);
  const int pos0 = kvlen - qlen + tok0;
  const int* table = p.block_tables + (size_t)s * p.max_blocks;
  const int hi = pos0 + ntok;
  const int lo = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int t_begin = lo / KEYS, t_end = (hi + KEYS - 1) / KEYS;
  const int num_tiles = t_end - t_begin;  // both query tiles walk all of them (the later tile sees at most one more)

  if (tid == 0) {
    for (int i = 0; i < 10; ++i) mbar_init(k_full + 8 * i, (i >= 4 && i < 8) ? QT : 1);  // k_full, v_full, k_free, v_free (one arrival per issuing thread), s_done
    for (int i = 10; i < 14; ++i) mbar_init(k_full + 8 * i, ROWS);  // s_read, p_ready
    for (int i = 14; i < 16; ++i) mbar_init(k_full + 8 * i, 1);  // o_done
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::TMEM) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();  // queries and the cache are the work of the kernels before this one

  // ---- both Q tiles, swizzled by hand (rows beyond the used ones are zero); the value stages start as zeros
  for (int idx = tid; idx < QT * ROWS * (D / 8); idx += T2_THREADS) {
    const int rr = idx / (D / 8), c = idx - rr * (D / 8);  // rr: row among those of all tiles; c: 16-byte chunk of the row
    const int rt = rr & (ROWS - 1), tok = (rr >> 7) * tpt + rt / Gc, hd = rt % Gc;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rt / Gc < tpt && tok < ntok && hd < nheads)
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + tok0 + tok) * p.q_stride + (size_t)(head0 + hd) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + (rr >> 7) * KV_BYTES + (c >> 3) * TILE_BYTES + rt * 128 + (((c & 7) ^ (rt & 7)) << 4)) = v;
  }
  for (int idx = tid; idx < 2 * KV_BYTES / 16; idx += T2_THREADS) reinterpret_cast<uint4*>(sV)[idx] = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_s = tmem, tmem_o = tmem + QT * KEYS;  // S of each query tile, then O of each

  // The softmax threads hold a row of 128 scores in registers; the third warpgroup needs few and gives its
  // share away (a scheduler then holds two warps of 224 registers and one of 40).
  if (warp >= QT * ROWS / 32) {
    // 384 threads start with 168 registers each; the two softmax warpgroups take 224, which leaves 56 for this one
    if (QT == 2) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == QT * ROWS / 32 + 1 || warp == QT * ROWS / 32 + 3) {
    // ================================================================ the warps that copy: one the keys, one the values
    // (a copy of a small page costs its issuing thread a few hundred clocks whatever its size; with one warp for both,
    // the keys of the next tile stood in line behind the values of this one, which wait for an older product)
    // a lane copies one page, all its slabs of 64 columns
    const bool keys = warp == QT * ROWS / 32 + 1;
    const int pages = KEYS / p.page_size;
    const int page_i = lane & 15;
    const uint32_t full = keys ? k_full : v_full, freed = keys ? k_free : v_free;
    unsigned char* stage0 = keys ? sK : sV;
    const CUtensorMap* map = keys ? &map_k : &map_v;
    auto lookup = [&](int t) -> int {
      const int first = t * KEYS + page_i * p.page_size;
      const bool need = lane < 16 && t < t_end && page_i < pages && first < hi && first + p.page_size > lo;
      return need ? table[first / p.page_size] : -1;
    };
    int page = lookup(t_begin);
    for (int t = 0; t < num_tiles && !*failed; ++t) {
      const int st = t & 1, par = ((t - 2) >> 1) & 1;
      const int cur = page;
      page = lookup(t_begin + t + 1);
      if (t >= 2) {
        if (lane == 0) wait_or_fail(freed + 8 * st, par, failed, keys ? 12 : 13, p.error_flag);
        __syncwarp();
        if (*failed) break;
      }
      const int count = __popc(__ballot_sync(0xffffffffu, cur >= 0));
      if (lane == 0) mbar_expect_tx(full + 8 * st, (uint32_t)(count * p.page_size * 128 * SLABS));
      __syncwarp();
      if (cur >= 0) {
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl)
          tma_load_2d(smem_u32(stage0 + st * KV_BYTES + sl * TILE_BYTES + page_i * p.page_size * 128), map, sl * 64, (cur * p.nkv + kvh) * p.page_size, full + 8 * st);
      }
    }
  } else if (warp == QT * ROWS / 32 || (QT == 2 && warp == QT * ROWS / 32 + 2)) {
    // ================================================================ the warps that issue the matrix products (their first lanes):
    // one per query tile.  A single thread that served both tiles spent its time on issuing and became what every
    // softmax group waited for.  A tile's products become possible in a fixed order, S(t + 1) (its threads have S(t) in
    // registers) before O += P(t) V(t) (the same threads have written P(t)), so the thread waits for each in turn and
    // sleeps in the barrier meanwhile: a polling loop takes issue slots from the softmax warps of its scheduler.  A stage
    // of keys or values is handed back to the copies when both threads have committed their products with it (those
    // barriers count QT arrivals).
    const int q = warp == QT * ROWS / 32 ? 0 : 1;  // this thread's query tile
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(ROWS, KEYS, 0), idesc_o = instr_desc(ROWS, 64, 1);
      const uint32_t qa = smem_u32(sQ + q * KV_BYTES), pa = smem_u32(sP + q * 2 * TILE_BYTES);
      auto scores = [&](int t) {  // S_q(t) = Q_q K(t)^T
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k = smem_u32(sK + (t & 1) * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma(tmem_s + q * KEYS, smem_desc_sw128(qa + (kk >> 2) * TILE_BYTES + (kk & 3) * 32), smem_desc_sw128(k + (kk >> 2) * TILE_BYTES + (kk & 3) * 32), idesc_s, kk != 0);
        umma_commit(s_done + 8 * q);
        umma_commit(k_free + 8 * (t & 1));  // this tile's product with K(t) is issued
      };
      bool ok = num_tiles > 0 && wait_or_fail(k_full, 0, failed, 17, p.error_flag);
      if (ok) scores(0);
      for (int t = 0; t < num_tiles && ok; ++t) {
        if (t + 1 < num_tiles) {  // the keys are there and the thread of every row has S_q(t) in registers
          ok = wait_or_fail(k_full + 8 * ((t + 1) & 1), ((t + 1) >> 1) & 1, failed, 17, p.error_flag) && wait_or_fail(s_read + 8 * q, t & 1, failed, 18, p.error_flag);
          if (!ok) break;
          scores(t + 1);
        }
        // O_q += P_q(t) V(t)
        ok = wait_or_fail(p_ready + 8 * q, t & 1, failed, 19, p.error_flag) && wait_or_fail(v_full + 8 * (t & 1), (t >> 1) & 1, failed, 20, p.error_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v = smem_u32(sV + (t & 1) * KV_BYTES);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl)  // 64 output columns at a time: the values' slab is the MN-major operand
#pragma unroll
          for (int k = 0; k < KEYS / 16; ++k)
            umma(tmem_o + q * D + sl * 64, smem_desc_sw128(pa + (k >> 2) * TILE_BYTES + (k & 3) * 32), smem_desc_sw128(v + sl * TILE_BYTES + k * 2048), idesc_o, (t | k) != 0);
        umma_commit(o_done + 8 * q);
        umma_commit(v_free + 8 * (t & 1));  // this tile's product with V(t) is issued
      }
    }
    __syncwarp();
  }
  } else {
    if (QT == 2) asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ================================================================ softmax threads: one per row
    const int q = warp >> 2;                 // query tile A or B
    const int r = tid & (ROWS - 1);          // row of the tile
    const int rtok = q * tpt + r / Gc;       // token among the CTA's
    const bool rvalid = rtok < ntok && (r % Gc) < nheads && r / Gc < tpt;
    const int rpos = pos0 + rtok;
    const uint32_t lane_bits = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t my_s = tmem_s + q * KEYS + lane_bits, my_o = tmem_o + q * D + lane_bits;
    const uint32_t my_s_done = s_done + 8 * q, my_s_read = s_read + 8 * q, my_p_ready = p_ready + 8 * q, my_o_done = o_done + 8 * q;
    constexpr float RESCALE_STEP = 8.f;
    float m = -CUDART_INF_F, m_ref = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    const int first_pos = pos0 + q * tpt;  // position of the tile's first row
    // where this row's eight 16-byte chunks of a 128-byte slab of P lie (the swizzle), as shared-memory addresses: a
    // store then needs no address arithmetic of its own (through a generic pointer each cost five instructions more;
    // 8,192 tokens: 455 -> 436 us)
    uint32_t pchunk[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) pchunk[c] = smem_u32(sP) + q * 2 * TILE_BYTES + r * 128 + ((c ^ (r & 7)) << 4);
    if (QT == 2 && q == 1 && num_tiles > 0) asm volatile("bar.arrive 1, %0;" ::"n"(2 * ROWS) : "memory");  // tile A takes the first turn

    for (int t = 0; t < num_tiles; ++t) {
      const int base = (t_begin + t) * KEYS;
      ok = wait_or_fail(my_s_done, t & 1, failed, 12, p.error_flag) && ok;
      ok = __all_sync(0xffffffffu, ok);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // (also after a failed wait: what is read then is never stored, and a second way for the scores to get their
      // values costs a register move per score on the way that counts: 8,192 tokens took 498 us with it, 455 without)
      float sc[128];
#pragma unroll
      for (int c = 0; c < 128; c += 64) {
        uint32_t v0[32], v1[32];
        tmem_ld32_nowait(my_s + c, v0);
        tmem_ld32_nowait(my_s + c + 32, v1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) { sc[c + j] = __uint_as_float(v0[j]); sc[c + 32 + j] = __uint_as_float(v1[j]); }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(my_s_read);  // S is in registers: the next product of this tile may overwrite it
      // a tile that lies wholly at or before the first row's position, inside every row's window, needs no mask
      const bool full = base + KEYS - 1 <= first_pos && base >= lo && p.window <= 0;
      if (!full) {
        const int hi_j = rpos - base, lo_j = p.window > 0 ? rpos - p.window - base : -1;
#pragma unroll
        for (int j = 0; j < 128; ++j) sc[j] = (j <= hi_j && j > lo_j) ? sc[j] : -CUDART_INF_F;
      }
      float mx[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) mx[j] = max3(sc[j], sc[j + 8], sc[j + 16]);
#pragma unroll
      for (int j = 24; j < 120; j += 16)
#pragma unroll
        for (int i = 0; i < 8; ++i) mx[i] = max3(mx[i], sc[j + i], sc[j + 8 + i]);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx[i] = fmaxf(mx[i], sc[120 + i]);
      m = max3(m, max3(mx[0], mx[1], mx[2]), max3(max3(mx[3], mx[4], mx[5]), mx[6], mx[7]));
      float corr = 1.f;
      const bool grown = (m - m_ref) * p.scale_log2 > RESCALE_STEP;  // also the first finite maximum (m_ref = -inf)
      if (grown) {
        corr = (m_ref == -CUDART_INF_F) ? 0.f : ex2((m_ref - m) * p.scale_log2);
        m_ref = m;
      }
      const float neg = (m_ref == -CUDART_INF_F) ? 0.f : -m_ref * p.scale_log2;
      // P and O of this tile are free once its product of the key tile before has finished
      if (t > 0) {
        ok = wait_or_fail(my_o_done, (t - 1) & 1, failed, 13, p.error_flag) && ok;
        ok = __all_sync(0xffffffffu, ok);
        if (__any_sync(0xffffffffu, grown)) {  // the output so far times 2^(old - new) in the rows whose reference moved
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (ok) {
#pragma unroll
            for (int c = 0; c < D; c += 32) {
              uint32_t v[32];
              tmem_ld32_nowait(my_o + c, v);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
              tmem_st32(my_o + c, v);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          }
        }
      }
      // ---- this group's turn at the exponentials (measured: 562 us at 8,192 tokens with turns, 694 without)
      if (QT == 2) {
        if (q == 0) asm volatile("bar.sync 1, %0;" ::"n"(2 * ROWS) : "memory");
        else asm volatile("bar.sync 2, %0;" ::"n"(2 * ROWS) : "memory");
      }
      // two elements per instruction where there is one for it (fma and add on pairs of float32): the loop is
      // bound by the number of instructions that one warp gets issued, not by the special-function units alone
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), neg2 = pack_f32x2(neg, neg);
#pragma unroll
      for (int j = 0; j < 128; j += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(sc[j + e], sc[j + e + 1]), scale2, neg2), x0, x1);
          const float p0 = ex2(x0), p1 = ex2(x1);  // masked: ex2(-inf) = 0
          sum2[(e >> 1) & 3] = add_f32x2(sum2[(e >> 1) & 3], pack_f32x2(p0, p1));
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
          packed[e >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
        st_shared_v4(pchunk[(j >> 3) & 7] + (j >> 6) * TILE_BYTES, packed[0], packed[1], packed[2], packed[3]);
      }
      float sum[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float lo_, hi_;
        unpack_f32x2(sum2[i], lo_, hi_);
        sum[i] = lo_ + hi_;
      }
      if (QT == 2) {
        if (q == 0) asm volatile("bar.arrive 2, %0;" ::"n"(2 * ROWS) : "memory");
        else if (t + 1 < num_tiles) asm volatile("bar.arrive 1, %0;" ::"n"(2 * ROWS) : "memory");
      }
      l = l * corr + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P is read by the tensor cores
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(my_p_ready);
    }
    // ---- the finished row, once the last product is done
    ok = wait_or_fail(my_o_done, (num_tiles - 1) & 1, failed, 13, p.error_flag) && ok;
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const float inv = 1.f / l;
    const size_t row = (size_t)(q0 + tok0 + rtok) * p.nh + head0 + (r % Gc);
#pragma unroll
    for (int c = 0; c < D; c += 32) {
      uint32_t v[32];
      if (ok) {
        tmem_ld32_nowait(my_o + c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
      if (ok && !*failed && rvalid) {
        uint4* dst = reinterpret_cast<uint4*>(p.out + row * D + c);
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 w;
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
          for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * e]) * inv, __uint_as_float(v[j + 2 * e + 1]) * inv);
          dst[j >> 3] = w;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::TMEM) : "memory");
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)ptr;
  }
  return fn;
}
// a pool [pages, nkv, page_size, d] seen as rows of d elements; boxes of one page of one head, 64 columns wide
bool make_pool_map(CUtensorMap* map, const void* base, long long rows, int page_size, int d = D) {
  EncodeTiled fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)d * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int* error_flag_device = nullptr;
int* error_flag_host = nullptr;

}  // namespace

// Sequences [seq0, seq0 + num_seqs) of a batch, each bringing at most max_q_len tokens.
// Head size 64 or 128; page_size must be 8, 16, 32, 64 or 128; num_pages is the pools' first extent.
// query_tiles (head size 64): 1 or 2 tiles of 128 rows per CTA, 0 to let the launcher choose.
DLI_EXPORT int dli_paged_prefill_tc(void* out, const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                                    long long num_pages, const int* block_tables, int max_blocks, const int* q_start,
                                    const int* kv_len, int seq0, int num_seqs, int max_q_len, int nh, int nkv, int head_dim,
                                    int page_size, int window, float scale, int query_tiles, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (head_dim != 64 && head_dim != 128) return DLI_ERR_UNSUPPORTED;
  if (nkv < 1 || nh % nkv || page_size < 8 || page_size > 128 || (KEYS % page_size) != 0) return DLI_ERR_UNSUPPORTED;
  if (((uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)q) & 15) return DLI_ERR_UNSUPPORTED;
  if (!error_flag_host) {
    if (cudaHostAlloc((void**)&error_flag_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) return (int)cudaGetLastError();
    *error_flag_host = 0;
    if (cudaHostGetDevicePointer((void**)&error_flag_device, error_flag_host, 0) != cudaSuccess) return (int)cudaGetLastError();
  }
  static OncePerDevice configured;
  if (!configured.here()) {
    cudaError_t e = cudaFuncSetAttribute(paged_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured.here() = true;
  }
  CUtensorMap map_k, map_v;
  const long long rows = num_pages * nkv * page_size;
  if (!make_pool_map(&map_k, k_pool, rows, page_size, head_dim) || !make_pool_map(&map_v, v_pool, rows, page_size, head_dim)) return DLI_ERR_UNSUPPORTED;
  Params p;
  p.out = (bf16*)out; p.q = (const bf16*)q; p.q_stride = q_stride;
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.q_start = q_start; p.kv_len = kv_len; p.seq0 = seq0;
  p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int G = nh / nkv;
  p.heads_per_chunk = G < ROWS ? G : ROWS;
  p.head_chunks = (G + p.heads_per_chunk - 1) / p.heads_per_chunk;
  p.tokens_per_tile = ROWS / p.heads_per_chunk;
  p.error_flag = error_flag_device;
  if (head_dim == 128) {  // one query tile per CTA, a thread per row
    static OncePerDevice configured128;
    if (!configured128.here()) {
      cudaError_t e = cudaFuncSetAttribute(paged_prefill_tc2_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, T2Cfg<128>::SMEM);
      if (e != cudaSuccess) return (int)e;
      configured128.here() = true;
    }
    const int tiles = (max_q_len + p.tokens_per_tile - 1) / p.tokens_per_tile;
    if (tiles > 65535 || num_seqs > 65535) return DLI_ERR_UNSUPPORTED;  // the grid's y and z
    return (int)launch_pdl(paged_prefill_tc2_kernel<128>, dim3(nkv * p.head_chunks, num_seqs, tiles), dim3(T2Cfg<128>::THREADS),
                           (size_t)T2Cfg<128>::SMEM, stream, 1, map_k, map_v, p);
  }
  // two query tiles per CTA when a sequence brings more tokens than one tile holds, unless the caller chose
  const bool two = query_tiles == 2 || (query_tiles != 1 && max_q_len > p.tokens_per_tile);
  if (two) {
    static OncePerDevice configured2;
    if (!configured2.here()) {
      cudaError_t e = cudaFuncSetAttribute(paged_prefill_tc2_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, T2Cfg<64>::SMEM);
      if (e != cudaSuccess) return (int)e;
      configured2.here() = true;
    }
    const int tiles = (max_q_len + 2 * p.tokens_per_tile - 1) / (2 * p.tokens_per_tile);
    if (tiles > 65535 || num_seqs > 65535) return DLI_ERR_UNSUPPORTED;
    return (int)launch_pdl(paged_prefill_tc2_kernel<64>, dim3(nkv * p.head_chunks, num_seqs, tiles), dim3(T2Cfg<64>::THREADS),
                           (size_t)T2Cfg<64>::SMEM, stream, 1, map_k, map_v, p);
  }
  const int tiles = (max_q_len + p.tokens_per_tile - 1) / p.tokens_per_tile;
  if (tiles > 65535 || num_seqs > 65535) return DLI_ERR_UNSUPPORTED;
  cudaError_t e = launch_pdl(paged_prefill_tc_kernel, dim3(nkv * p.head_chunks, num_seqs, tiles), dim3(THREADS), (size_t)SMEM_BYTES, stream, 1,
                             map_k, map_v, p);
  return (int)e;
}


// ================================================================ single-token sequences, TMA-fed
namespace {

constexpr int DN = 16;                 // keys per tile of one warp
constexpr int CLUSTER_SPLITS_MAX = 16;  // the largest cluster of this GPU (more than 8 is the kernel's opt-in)
constexpr int CLUSTER_ROWS_MAX = 23;    // rows of partial results that may arrive at one CTA

// Sizes that depend on the head size HD (64 or 128).  A row of keys or values is HD * 2 bytes; the
// 128-byte swizzle covers 64 elements, so a tile of 16 rows lies in shared memory as HD / 64 slabs of
// [16 rows x 128 bytes], each filled by its own TMA box (the columns 64 s .. 64 s + 63 of the rows).
// DWARPS: warps of a CTA, each with its own tiles and stages.  Four, so that four CTAs (two at head size 128) share an
// SM when the grid is large; eight when the grid has fewer CTAs than two per SM (one or two long sequences), where
// nothing else would hide a warp's latencies.
template <int HD, int DWARPS>
struct DecodeCfg {
  static_assert(HD == 64 || HD == 128, "head sizes with whole 128-byte slabs");
  static_assert(DWARPS == 4 || DWARPS == 8, "four or eight warps");
  static constexpr int SLABS = HD / 64;
  static constexpr int SLAB = DN * 128;                 // bytes of one slab
  static constexpr int TILE = SLABS * SLAB;             // one K or V tile
  static constexpr int STAGES = HD == 64 ? 3 : 2;
  static constexpr int QROW = HD * 2 + 16;              // padded query rows (read once)
  // Splits merged inside a cluster: row r of the 16 belongs to CTA (r mod splits); every CTA pushes its
  // partial (sums[HD], maximum, denominator) of a row into the owner's memory: splits * ceil(rows / splits)
  // rows arrive at one CTA, and the launcher merges in the cluster only if that is at most
  // CLUSTER_ROWS_MAX.  The region starts where the query rows lay: they are in registers by then.
  static constexpr int RECV_ROW = HD + 2;
  static constexpr int RECV_BYTES = CLUSTER_ROWS_MAX * RECV_ROW * 4;
  static constexpr int SMEM = 1024 + DWARPS * STAGES * 2 * TILE + RECV_BYTES + DWARPS * STAGES * 8 + 64;
  static_assert(RECV_BYTES >= 16 * QROW, "the received partial results lie over the query rows");
  static_assert(DWARPS * 16 * (HD + 2) * 4 <= DWARPS * STAGES * 2 * TILE, "the merge buffer reuses the key/value stages");
  static_assert((DWARPS == 8 ? 1 : HD == 64 ? 4 : 2) * (SMEM + 1024) <= 227 * 1024, "four CTAs per SM at head size 64, two at 128 (four warps)");
};

struct DecodeParams {
  bf16* out;
  const bf16* q;
  long long q_stride;
  const int* block_tables;
  int max_blocks;
  const int* q_start;
  const int* kv_len;
  int seq0, nh, nkv, page_size, window, splits;
  int cluster_merge;  // the splits of a (sequence, head group) are one cluster and merge through shared memory
  float scale_log2;
  float* part_acc;
  float* part_ml;
  int* error_flag;
};

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// as wait_or_fail, for a barrier whose bytes other CTAs of the cluster send (st.async)
__device__ __forceinline__ bool wait_cluster_or_fail(uint32_t bar, uint32_t parity, volatile int* failed, int code, int* error_flag) {
  for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  *failed = code;
  atomicExch(error_flag, code);
  return false;
}
// store into the same shared-memory offset of another CTA of the cluster; the four bytes are counted on that CTA's
// mbarrier at `local_bar` when they have landed
__device__ __forceinline__ void st_async_peer(uint32_t local_addr, uint32_t local_bar, uint32_t cta_rank, float v) {
  uint32_t remote, remote_bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta_rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(local_bar), "r"(cta_rank));
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
               ::"r"(remote), "r"(__float_as_uint(v)), "r"(remote_bar) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// grid (sequences, splits, kv heads * chunks of 16 query heads).  The 16 rows of a warp's MMA tile
// are the query heads of one KV head; each warp walks its own share of the 16-key tiles.  A tile's
// keys and values arrive by TMA (one box per page piece, 128-byte swizzle), four tiles ahead, on the
// warp's own mbarriers: no thread spends instructions on addresses of individual 16-byte copies.
template <int HD, int DWARPS>
__global__ void __launch_bounds__(DWARPS * 32) paged_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                       const __grid_constant__ CUtensorMap map_v, const DecodeParams p) {
  using Cfg = DecodeCfg<HD, DWARPS>;
  constexpr int DSTAGES = Cfg::STAGES, DTILE = Cfg::TILE, QROW = Cfg::QROW, RECV_BYTES = Cfg::RECV_BYTES, RECV_ROW = Cfg::RECV_ROW;
  constexpr int D = HD;  // shadows the prefill kernel's head size within this kernel
  pdl_launch_dependents();
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sKV = smem;                                   // [warp][stage][K | V]
  unsigned char* sQ = sKV + DWARPS * DSTAGES * 2 * DTILE;      // 16 padded rows
  uint64_t* bars = (uint64_t*)(sQ + RECV_BYTES);               // [warp][stage]
  volatile int* failed = (volatile int*)(bars + DWARPS * DSTAGES);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int s = p.seq0 + blockIdx.x;
  const int split = blockIdx.y;
  const int G = p.nh / p.nkv;
  const int chunks = (G + 15) / 16;
  const int kvh = blockIdx.z / chunks, hc = blockIdx.z - kvh * chunks;
  const int head0 = kvh * G + hc * 16;
  const int nheads = min(16, G - hc * 16);
  const int token = p.q_start[s];
  const int kvlen = p.kv_len[s];
  const int pos = kvlen - 1;
  const int* table = p.block_tables + (size_t)s * p.max_blocks;
  const int hi = kvlen;
  const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  const int first_tile = lo / DN;
  const int tiles_total = (hi + DN - 1) / DN - first_tile;
  const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
  const int t_begin = first_tile + split * tiles_per_split;
  const int t_end = min(first_tile + tiles_total, t_begin + tiles_per_split);

  // rows r = split, split + splits, .. of the head group are merged by this CTA
  const int mine = split < nheads ? (nheads - split + p.splits - 1) / p.splits : 0;
  const uint32_t merged = smem_u32(bars + DWARPS * DSTAGES + 1);  // completes when every split's partial results of those rows have landed
  if (tid == 0) {
    *failed = 0;
    mbar_init(merged, 1);
    if (p.cluster_merge && mine > 0) mbar_expect_tx(merged, (uint32_t)(p.splits * mine * RECV_ROW * 4));
  }
  if (lane == 0) {
    for (int st = 0; st < DSTAGES; ++st) mbar_init(smem_u32(bars + warp * DSTAGES + st), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();  // this warp's barriers are set up

  unsigned char* wbuf = sKV + warp * DSTAGES * 2 * DTILE;
  const uint32_t wbar = smem_u32(bars + warp * DSTAGES);
  const int my_tiles = (t_end - t_begin - warp + DWARPS - 1) / DWARPS;
  const int box_rows = p.page_size < DN ? p.page_size : DN;  // a tile is one piece of a page, or two whole pages of 8
  const int boxes = DN / box_rows;

  // Where the boxes lie is worked out 32 boxes at a time, one per lane (block-table entry, row in the pools), and
  // handed to lane 0 by shuffle: lane 0 must never wait for a global load, or divide, between two copies.
  int cached_first = 0;
  auto box_row = [&](int e) -> int {  // first pool row of this warp's e-th box (box = tile piece of box_rows keys)
    const int key = (t_begin + warp + (boxes == 2 ? e >> 1 : e) * DWARPS) * DN + (boxes == 2 ? e & 1 : 0) * box_rows;
    if (key >= hi || key + box_rows <= lo) return 0x3fffff00;  // no key of the box is visible: a row beyond the pool makes the copy fill the box with zeros
    const int entry = key / p.page_size;
    return (table[entry] * p.nkv + kvh) * p.page_size + (key - entry * p.page_size);
  };
  int cached = box_row(lane);
  // every lane calls this (the shuffles need them all); lane 0 issues the copies of the warp's i-th tile into stage st
  auto issue = [&](int i, int st) {
    const uint32_t bar = wbar + 8 * st;
    if (lane == 0) mbar_expect_tx(bar, 2 * DTILE);
    for (int b = 0; b < boxes; ++b) {
      const int e = i * boxes + b;
      if (e >= cached_first + 32) {
        cached_first = e;
        cached = box_row(e + lane);
      }
      const int row = __shfl_sync(0xffffffffu, cached, e - cached_first);
      if (lane == 0) {
#pragma unroll
        for (int sl = 0; sl < Cfg::SLABS; ++sl) {
          tma_load_2d(smem_u32(wbuf + st * 2 * DTILE + sl * Cfg::SLAB + b * box_rows * 128), &map_k, sl * 64, row, bar);
          tma_load_2d(smem_u32(wbuf + st * 2 * DTILE + DTILE + sl * Cfg::SLAB + b * box_rows * 128), &map_v, sl * 64, row, bar);
        }
      }
    }
  };

  const int r0 = lane >> 2, r1 = r0 + 8;
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F};
  float l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

  // Keys and values of earlier steps do not depend on the kernel before this one (it wrote this
  // step's token only), nor do the tables and lengths: the first tiles are requested before the wait
  // on that kernel, all but the tile that holds the new token.
  const int newest_tile = pos / DN;
  int deferred = -1;
  for (int i = 0; i < DSTAGES - 1 && i < my_tiles; ++i) {
    if (t_begin + warp + i * DWARPS == newest_tile) deferred = i;  // the last of this warp's tiles, if any
    else issue(i, i);
  }
  pdl_wait();
  if (deferred >= 0) issue(deferred, deferred);

  for (int idx = tid; idx < 16 * (D / 8); idx += DWARPS * 32) {
    const int r = idx / (D / 8), c = idx - r * (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nheads) v = *reinterpret_cast<const uint4*>(p.q + (size_t)token * p.q_stride + (size_t)(head0 + r) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + r * QROW + c * 16) = v;
  }
  __syncthreads();

  // the query fragments stay in registers
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) ldsm_x4(qf[kk], smem_u32(sQ + (lane & 15) * QROW + (kk * 16 + (lane >> 4) * 8) * 2));
  if (p.cluster_merge) cluster_arrive();  // this thread is done with the query rows; waited for before the first push

  // The running maximum m of a row is a reference, not the exact maximum: it moves only when a tile's maximum
  // exceeds it by more than 2^RESCALE_STEP (or is the first finite one), and only then are the sums rescaled; the
  // probabilities are 2^(s - m) <= 2^RESCALE_STEP meanwhile, which bfloat16 and float32 hold as well as values <= 1.
  // Scores stay raw; the scale goes into the exponent's multiply-add.  Tiles that lie wholly inside the visible
  // range, all but the last and a window's first, skip the mask.
  constexpr float RESCALE_STEP = 8.f;
  bool ok = true;
  int st = 0, phase = 0;
  for (int i = 0; i < my_tiles; ++i) {
    if (i + DSTAGES - 1 < my_tiles) issue(i + DSTAGES - 1, st == 0 ? DSTAGES - 1 : st - 1);  // into the stage finished an iteration ago
    if (ok && !wait_or_fail(wbar + 8 * st, phase, failed, 21, p.error_flag)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const uint32_t tK = smem_u32(wbuf + st * 2 * DTILE), tV = tK + DTILE;
      const int base = (t_begin + warp + i * DWARPS) * DN;
      // ---- S = Q K^T for 16 keys: two 8-key column tiles
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t b[4];
        const int key = (lane & 7) + (lane >> 4) * 8;
        const int chunk = (kk & 3) * 2 + ((lane >> 3) & 1);
        ldsm_x4(b, tK + (kk >> 2) * Cfg::SLAB + key * 128 + ((chunk ^ (key & 7)) << 4));
        mma16816(sc[0], qf[kk], b[0], b[1]);
        mma16816(sc[1], qf[kk], b[2], b[3]);
      }
      // ---- mask (only a tile that reaches beyond the visible keys) and online softmax
      if (base < lo || base + DN - 1 > pos) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = base + j * 8 + (lane & 3) * 2 + (e & 1);
            if (key > pos || key < lo) sc[j][e] = -CUDART_INF_F;
          }
      }
      float tmax[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        tmax[rr] = fmaxf(fmaxf(sc[0][2 * rr], sc[0][2 * rr + 1]), fmaxf(sc[1][2 * rr], sc[1][2 * rr + 1]));
        tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 1));
        tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 2)) * p.scale_log2;  // the scale is positive
      }
      const bool grown0 = tmax[0] - m[0] > RESCALE_STEP, grown1 = tmax[1] - m[1] > RESCALE_STEP;  // also the first finite maximum; never a NaN's turn
      if (__any_sync(0xffffffffu, grown0 || grown1)) {
        const float c0 = grown0 ? ((m[0] == -CUDART_INF_F) ? 0.f : ex2(m[0] - tmax[0])) : 1.f;
        const float c1 = grown1 ? ((m[1] == -CUDART_INF_F) ? 0.f : ex2(m[1] - tmax[1])) : 1.f;
        if (grown0) m[0] = tmax[0];
        if (grown1) m[1] = tmax[1];
        l[0] *= c0;
        l[1] *= c1;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          o[j][0] *= c0; o[j][1] *= c0;
          o[j][2] *= c1; o[j][3] *= c1;
        }
      }
      const float neg0 = (m[0] == -CUDART_INF_F) ? 0.f : -m[0], neg1 = (m[1] == -CUDART_INF_F) ? 0.f : -m[1];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = ex2(fmaf(sc[j][e], p.scale_log2, (e >> 1) ? neg1 : neg0));  // masked: ex2(-inf) = 0
          sc[j][e] = pv;
          l[e >> 1] += pv;
        }
      // ---- O += P V (16 keys = one k step)
      uint32_t a[4] = {pack2(sc[0][0], sc[0][1]), pack2(sc[0][2], sc[0][3]), pack2(sc[1][0], sc[1][1]), pack2(sc[1][2], sc[1][3])};
#pragma unroll
      for (int jp = 0; jp < D / 16; ++jp) {
        uint32_t b[4];
        const int key = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int chunk = (jp & 3) * 2 + (lane >> 4);
        ldsm_x4_trans(b, tV + (jp >> 2) * Cfg::SLAB + key * 128 + ((chunk ^ (key & 7)) << 4));
        mma16816(o[2 * jp], a, b[0], b[1]);
        mma16816(o[2 * jp + 1], a, b[2], b[3]);
      }
    }
    __syncwarp();  // every lane has read the stage before lane 0 refills it
    if (++st == DSTAGES) { st = 0; phase ^= 1; }
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
    l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
  }

  // ---- merge the four warps' partial results in shared memory (the key/value stages are free)
  __syncthreads();
  float* mo = reinterpret_cast<float*>(sKV);   // [DWARPS][16][D]
  float* mm = mo + DWARPS * 16 * D;            // [DWARPS][16]
  float* ml = mm + DWARPS * 16;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = rr ? r1 : r0;
    float* dst = mo + (warp * 16 + row) * D;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) *reinterpret_cast<float2*>(dst + j * 8 + (lane & 3) * 2) = make_float2(o[j][2 * rr], o[j][2 * rr + 1]);
    if ((lane & 3) == 0) {
      mm[warp * 16 + row] = m[rr];
      ml[warp * 16 + row] = l[rr];
    }
  }
  __syncthreads();
  const bool bad = *failed != 0;
  if (bad && !p.cluster_merge) return;
  float* recv = reinterpret_cast<float*>(sQ);  // [split][owned row][sums | maximum | denominator]
  const int owned_max = (nheads + p.splits - 1) / p.splits;
  if (p.cluster_merge) cluster_wait();  // every CTA of the cluster has its query in registers: the region may be written
  for (int idx = tid; idx < nheads * D; idx += DWARPS * 32) {
    const int r = idx / D, dcol = idx - r * D;
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < DWARPS; ++w) mx = fmaxf(mx, mm[w * 16 + r]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < DWARPS; ++w) {
      const float mw = mm[w * 16 + r];
      const float f = (mw == -CUDART_INF_F) ? 0.f : ex2(mw - mx);
      L += ml[w * 16 + r] * f;
      acc += mo[(w * 16 + r) * D + dcol] * f;
    }
    const size_t row = (size_t)token * p.nh + head0 + r;
    if (p.splits == 1) {
      p.out[row * D + dcol] = __float2bfloat16_rn(acc / L);
    } else if (p.cluster_merge) {
      const uint32_t dst = smem_u32(recv + (split * owned_max + r / p.splits) * RECV_ROW);
      const int owner = r % p.splits;
      st_async_peer(dst + dcol * 4, merged, owner, acc);
      if (dcol == 0) {
        st_async_peer(dst + D * 4, merged, owner, mx);
        st_async_peer(dst + (D + 1) * 4, merged, owner, L);
      }
    } else {
      p.part_acc[(row * p.splits + split) * D + dcol] = acc;
      if (dcol == 0) {
        p.part_ml[(row * p.splits + split) * 2] = mx;
        p.part_ml[(row * p.splits + split) * 2 + 1] = L;
      }
    }
  }
  if (!p.cluster_merge || mine == 0) return;
  // every split's partial result of my rows has arrived (each store counted its bytes on this CTA's barrier: no
  // cluster barrier, which would also hold the CTAs that merge nothing); nobody reads a peer's memory, and a CTA
  // leaves only after what was sent to it has landed
  if (!wait_cluster_or_fail(merged, 0, failed, 22, p.error_flag) || bad) return;
  for (int idx = tid; idx < mine * D; idx += DWARPS * 32) {
    const int ri = idx / D, dcol = idx - ri * D;
    const int r = split + ri * p.splits;
    float mx = -CUDART_INF_F;
    for (int i = 0; i < p.splits; ++i) mx = fmaxf(mx, recv[(i * owned_max + ri) * RECV_ROW + D]);
    float L = 0.f, acc = 0.f;
    for (int i = 0; i < p.splits; ++i) {  // split 0 first: a fixed order
      const float* part = recv + (i * owned_max + ri) * RECV_ROW;
      const float mi = part[D];
      if (mi != -CUDART_INF_F) {
        const float f = ex2(mi - mx);
        L += part[D + 1] * f;
        acc += part[dcol] * f;
      }
    }
    p.out[((size_t)token * p.nh + head0 + r) * D + dcol] = __float2bfloat16_rn(acc / L);
  }
}

// out[row] = sum_i acc_i 2^(m_i - max m) / sum_i l_i 2^(m_i - max m); one block per (token, head) row.
__global__ void merge_decode_splits_kernel(bf16* __restrict__ out, const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                           int row0, int splits, int d) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = (size_t)row0 + blockIdx.x;
  const float* ml = part_ml + row * splits * 2;
  float mmax = -CUDART_INF_F;
  for (int i = 0; i < splits; ++i) mmax = fmaxf(mmax, ml[2 * i]);
  float L = 0.f;
  for (int i = 0; i < splits; ++i) {
    const float mi = ml[2 * i];
    if (mi != -CUDART_INF_F) L += ml[2 * i + 1] * exp2f(mi - mmax);
  }
  const float inv = 1.f / L;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < splits; ++i) {
      const float mi = ml[2 * i];
      if (mi != -CUDART_INF_F) acc += part_acc[(row * splits + i) * d + c] * exp2f(mi - mmax);
    }
    out[row * d + c] = __float2bfloat16_rn(acc * inv);
  }
}

// a pool [pages, nkv, page_size, d] seen as rows of d elements; boxes of box_rows rows x 64 elements
bool make_decode_map(CUtensorMap* map, const void* base, long long rows, int box_rows, int d) {
  EncodeTiled fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)d * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// whether the key splits of these sizes merge inside one cluster (else: scratch and the merge kernel)
bool merges_in_cluster(int nh, int nkv, int splits) {
  const int G = nh / nkv, rows = G < 16 ? G : 16;
  // (clusters of 9 to 15 CTAs were measured slower than 8 splits, or than more splits and the merge kernel)
  return splits > 1 && (splits <= 8 || splits == CLUSTER_SPLITS_MAX) && splits * ((rows + splits - 1) / splits) <= CLUSTER_ROWS_MAX;
}

template <int HD, int DWARPS>
int launch_decode_warps(const CUtensorMap& map_k, const CUtensorMap& map_v, const DecodeParams& p, int num_seqs, int first_row, cudaStream_t stream) {
  static OncePerDevice configured;
  if (!configured.here()) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_tma_kernel<HD, DWARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<HD, DWARPS>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(paged_decode_tma_kernel<HD, DWARPS>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
    configured.here() = true;
  }
  const int G = p.nh / p.nkv;
  cudaError_t e = launch_pdl(paged_decode_tma_kernel<HD, DWARPS>, dim3(num_seqs, p.splits, p.nkv * ((G + 15) / 16)), dim3(DWARPS * 32),
                             (size_t)DecodeCfg<HD, DWARPS>::SMEM, stream, p.cluster_merge ? p.splits : 1, map_k, map_v, p);
  if (e != cudaSuccess) return (int)e;
  if (p.splits > 1 && !p.cluster_merge)
    e = launch_pdl(merge_decode_splits_kernel, dim3(num_seqs * p.nh), dim3(64), 0, stream, 1, p.out, (const float*)p.part_acc,
                   (const float*)p.part_ml, first_row * p.nh, p.splits, HD);
  return (int)e;
}


// Eight warps a CTA at head size 64 when the grid leaves SMs with one CTA at most and every warp still gets four tiles
// or more: one sequence of 32 K keys in 16 splits takes 33 us with four warps and 27 with eight.  (Measured slower
// with eight: two CTAs on an SM, 39 -> 48 us for two such sequences, and head size 128, 44 -> 58 us.)
template <int HD>
int launch_decode(const CUtensorMap& map_k, const CUtensorMap& map_v, const DecodeParams& p, int num_seqs, int first_row, int max_kv_len,
                  cudaStream_t stream) {
  const int G = p.nh / p.nkv;
  const long long ctas = (long long)num_seqs * p.splits * p.nkv * ((G + 15) / 16);
  const int tiles_per_split = (max_kv_len + DN - 1) / DN / p.splits;
  if (HD == 64 && ctas <= sm_count() && tiles_per_split >= 32) return launch_decode_warps<HD, 8>(map_k, map_v, p, num_seqs, first_row, stream);
  return launch_decode_warps<HD, 4>(map_k, map_v, p, num_seqs, first_row, stream);
}
}  // namespace

// Attention of num_seqs single-token sequences (head size 64 or 128; page size a multiple of 8, and
// of 16 if larger than 8).  Up to 16 splits are one cluster and merge on the chip; more go through
// part_acc / part_ml (scratch, as for dli_paged_attention_mma) and a second kernel.
DLI_EXPORT int dli_paged_decode_tma(void* out, const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                                    long long num_pages, const int* block_tables, int max_blocks, const int* q_start,
                                    const int* kv_len, int seq0, int num_seqs, int first_row, int nh, int nkv, int head_dim,
                                    int page_size, int window, float scale, int splits, float* part_acc, float* part_ml,
                                    int max_kv_len, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (head_dim != 64 && head_dim != 128) return DLI_ERR_UNSUPPORTED;
  if (nkv < 1 || nh % nkv || splits < 1 || (splits > 1 && (!part_acc || !part_ml))) return DLI_ERR_UNSUPPORTED;
  if (page_size < 8 || (page_size % 8) || (page_size > 8 && (page_size % 16)) || page_size > 256) return DLI_ERR_UNSUPPORTED;
  if (((uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)q) & 15) return DLI_ERR_UNSUPPORTED;
  if (!error_flag_host) {
    if (cudaHostAlloc((void**)&error_flag_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) return (int)cudaGetLastError();
    *error_flag_host = 0;
    if (cudaHostGetDevicePointer((void**)&error_flag_device, error_flag_host, 0) != cudaSuccess) return (int)cudaGetLastError();
  }
  CUtensorMap map_k, map_v;
  const long long rows = num_pages * nkv * page_size;
  const int box_rows = page_size < DN ? page_size : DN;
  if (!make_decode_map(&map_k, k_pool, rows, box_rows, head_dim) || !make_decode_map(&map_v, v_pool, rows, box_rows, head_dim))
    return DLI_ERR_UNSUPPORTED;
  DecodeParams p;
  p.out = (bf16*)out; p.q = (const bf16*)q; p.q_stride = q_stride;
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.q_start = q_start; p.kv_len = kv_len; p.seq0 = seq0;
  p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.window = window; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.part_acc = part_acc; p.part_ml = part_ml; p.error_flag = error_flag_device;
  p.cluster_merge = merges_in_cluster(nh, nkv, splits);
  return head_dim == 64 ? launch_decode<64>(map_k, map_v, p, num_seqs, first_row, max_kv_len, stream)
                        : launch_decode<128>(map_k, map_v, p, num_seqs, first_row, max_kv_len, stream);
}

DLI_EXPORT int dli_decode_tma_merges_in_cluster(int nh, int nkv, int splits) { return merges_in_cluster(nh, nkv, splits) ? 1 : 0; }

// 0, or the code of the first bounded wait that ran out (11 keys, 12 scores or a key stage, 13 an output product or a
// value stage, 14 values, 15 probabilities, 17 the product warp found nothing to issue; 21: a decode warp's keys and values)
DLI_EXPORT int dli_paged_prefill_tc_error() { return error_flag_host ? *error_flag_host : 0; }
// Forget a recorded code (the host has read it); call with no launch of this library in flight.
DLI_EXPORT int dli_paged_prefill_tc_clear_error() { if (error_flag_host) *error_flag_host = 0; return 0; }
