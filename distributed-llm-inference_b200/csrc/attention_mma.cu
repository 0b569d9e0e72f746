// Paged causal GQA attention in bfloat16 on tensor cores, for one head size (-DHEAD_DIM=...,
// a multiple of 16 up to 256).  One kernel serves prompt portions and single decoded tokens:
//
//   * a CTA owns a tile of up to 64 rows; a row is one (token, query head) pair, and all rows
//     of a tile share one KV head, so a key/value tile fetched once serves the whole GQA group;
//   * keys and values are read in place from the cache pages, 64 keys at a time, by cp.async
//     through the sequence's block table (any page size), double buffered in shared memory;
//   * scores, running maximum, sum and output accumulate in float32 (online softmax); the
//     probabilities are rounded to bfloat16 only as the operand of the P V product;
//   * causality is by absolute position (a portion that starts at position `start` sees keys
//     0 .. its own position), with an optional window;
//   * sequences that bring a single token (decoding) have their own kernel: the 16 rows of a
//     tile are the query heads of one KV head; each of the four warps walks its own share of
//     the key tiles with its own cp.async pipeline (no CTA-wide barrier in the loop), and the
//     four partial results are merged in shared memory;
//   * with splits > 1 (single-token sequences, long contexts) each CTA takes a slice of the
//     keys and writes an unnormalised partial result; a second kernel merges the slices.
//
// Shared-memory rows are padded by 16 bytes: for every head size that is a multiple of 16 the
// eight rows an ldmatrix reads then fall into eight different 16-byte bank groups.
#include "common.cuh"
#include <math_constants.h>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 16>"
#endif

using namespace dli;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int D = HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");
constexpr int BLOCK_N = 64;             // keys per tile
constexpr int NWARPS = 4;
constexpr int BLOCK_M = 16 * NWARPS;    // rows per tile
constexpr int THREADS = 32 * NWARPS;
constexpr int CHUNKS = D / 8;           // 16-byte chunks per row
constexpr int ROW_BYTES = D * 2 + 16;   // padded row
constexpr int TILE_BYTES = BLOCK_N * ROW_BYTES;
constexpr int STAGES = 2;
constexpr int SMEM_BYTES = BLOCK_M * ROW_BYTES + 2 * STAGES * TILE_BYTES;

struct Params {
  bf16* out;                 // [n, nh * D]
  const bf16* q;             // rows of q_stride elements; head h at column h * D
  long long q_stride;
  const bf16* k_pool;        // [pages, nkv, page_size, D]
  const bf16* v_pool;
  const int* block_tables;   // [seqs, max_blocks]
  int max_blocks;
  const int* q_start;        // [seqs + 1]
  const int* kv_len;         // [seqs]
  int seq0;                  // first sequence of this launch
  int nh, nkv, page_size, window;
  float scale_log2;          // softmax scale times log2(e)
  int tokens_per_tile, heads_per_chunk, head_chunks, splits;
  float* part_acc;           // [n * nh, splits, D]   (splits > 1)
  float* part_ml;            // [n * nh, splits, 2]
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copies `rows` consecutive keys (from position `base`) of one KV head into a shared-memory
// tile, keys and values, 16 bytes per cp.async; keys outside [lo, hi) become zero rows.
// `nthreads` threads take part, thread `t` of them.  When the 16-byte chunks of a row divide
// the thread count, a thread keeps its chunk column and walks down the rows, stepping through
// the block table without a division per copy.
template <int ROWS>
__device__ __forceinline__ void load_kv_tile(unsigned char* dK, unsigned char* dV, const bf16* __restrict__ k_pool,
                                             const bf16* __restrict__ v_pool, const int* __restrict__ table, int base, int lo, int hi,
                                             int nkv, int kvh, int page_size, int t, int nthreads) {
  if ((nthreads % CHUNKS) == 0) {
    const int step = nthreads / CHUNKS;
    const int c = t % CHUNKS;
    int r = t / CHUNKS;
    int key = base + r;
    int blk = key / page_size, off = key - blk * page_size;
    for (; r < ROWS; r += step) {
      const bool ok = key >= lo && key < hi;
      size_t src = 0;
      if (ok) src = (((size_t)table[blk] * nkv + kvh) * page_size + off) * D + c * 8;
      cp_async16(smem_u32(dK + r * ROW_BYTES + c * 16), k_pool + src, ok ? 16 : 0);
      cp_async16(smem_u32(dV + r * ROW_BYTES + c * 16), v_pool + src, ok ? 16 : 0);
      key += step;
      off += step;
      while (off >= page_size) { off -= page_size; ++blk; }
    }
  } else {
    for (int idx = t; idx < ROWS * CHUNKS; idx += nthreads) {
      const int r = idx / CHUNKS, c = idx - r * CHUNKS;
      const int key = base + r;
      const bool ok = key >= lo && key < hi;
      size_t src = 0;
      if (ok) {
        const int blk = key / page_size;
        src = (((size_t)table[blk] * nkv + kvh) * page_size + (key - blk * page_size)) * D + c * 8;
      }
      cp_async16(smem_u32(dK + r * ROW_BYTES + c * 16), k_pool + src, ok ? 16 : 0);
      cp_async16(smem_u32(dV + r * ROW_BYTES + c * 16), v_pool + src, ok ? 16 : 0);
    }
  }
}

// One tile of NK keys for the 16 rows of a warp: S = Q K^T, mask, online softmax, O += P V.
// q16: the warp's 16 query rows; tK, tV: the tile's keys and values (rows of ROW_BYTES);
// base: position of the tile's first key; rvalid / rpos: validity and position of the two
// rows this thread holds (lane / 4 and lane / 4 + 8).
template <int NK>
__device__ __forceinline__ void tile_update(const unsigned char* sQ, const unsigned char* tK, const unsigned char* tV, int base,
                                            const bool (&rvalid)[2], const int (&rpos)[2], int window, float scale_log2,
                                            float (&m)[2], float (&l)[2], float (&o)[D / 8][4], int lane) {
  // ---- S = Q K^T
  float sc[NK / 8][4];
#pragma unroll
  for (int j = 0; j < NK / 8; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, smem_u32(sQ + ((lane & 15)) * ROW_BYTES + (kk * 16 + (lane >> 4) * 8) * 2));
#pragma unroll
    for (int jp = 0; jp < NK / 16; ++jp) {
      uint32_t b[4];
      const int key = jp * 16 + (lane & 7) + (lane >> 4) * 8;
      const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
      ldmatrix_x4(b, smem_u32(tK + key * ROW_BYTES + dim * 2));
      mma_bf16(sc[2 * jp], a, b[0], b[1]);
      mma_bf16(sc[2 * jp + 1], a, b[2], b[3]);
    }
  }

  // ---- mask, online softmax (float32)
  float tmax[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
  for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int rr = e >> 1;
      const int key = base + j * 8 + (lane & 3) * 2 + (e & 1);
      bool ok = rvalid[rr] && key <= rpos[rr];
      if (window > 0) ok = ok && key > rpos[rr] - window;
      const float t = ok ? sc[j][e] * scale_log2 : -CUDART_INF_F;
      sc[j][e] = t;
      tmax[rr] = fmaxf(tmax[rr], t);
    }
  }
  float corr[2], msafe[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 1));
    tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 2));
    const float mnew = fmaxf(m[rr], tmax[rr]);
    msafe[rr] = (mnew == -CUDART_INF_F) ? 0.f : mnew;
    corr[rr] = exp2f(m[rr] - msafe[rr]);  // 0 while m is still -inf
    m[rr] = mnew;
    l[rr] *= corr[rr];
  }
#pragma unroll
  for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float pv = exp2f(sc[j][e] - msafe[e >> 1]);
      sc[j][e] = pv;
      l[e >> 1] += pv;
    }
  }
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    o[j][0] *= corr[0]; o[j][1] *= corr[0];
    o[j][2] *= corr[1]; o[j][3] *= corr[1];
  }

  // ---- O += P V
#pragma unroll
  for (int kk = 0; kk < NK / 16; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
    a[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
    a[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
    a[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
    for (int jp = 0; jp < D / 16; ++jp) {
      uint32_t b[4];
      const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int dim = jp * 16 + (lane >> 4) * 8;
      ldmatrix_x4_trans(b, smem_u32(tV + key * ROW_BYTES + dim * 2));
      mma_bf16(o[2 * jp], a, b[0], b[1]);
      mma_bf16(o[2 * jp + 1], a, b[2], b[3]);
    }
  }
}

__global__ void __launch_bounds__(THREADS) paged_attention_mma_kernel(const Params p) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sQ = smem;
  unsigned char* sK = smem + BLOCK_M * ROW_BYTES;
  unsigned char* sV = sK + STAGES * TILE_BYTES;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int s = p.seq0 + blockIdx.y;
  const int tile = blockIdx.x / p.splits, split = blockIdx.x - tile * p.splits;
  const int kvh = blockIdx.z / p.head_chunks, hc = blockIdx.z - kvh * p.head_chunks;
  const int q0 = p.q_start[s];
  const int qlen = p.q_start[s + 1] - q0;
  const int kvlen = p.kv_len[s];
  const int tok0 = tile * p.tokens_per_tile;
  if (tok0 >= qlen) return;
  const int ntok = min(p.tokens_per_tile, qlen - tok0);
  const int G = p.nh / p.nkv, Gc = p.heads_per_chunk;
  const int head0 = kvh * G + hc * Gc;
  const int nheads = min(Gc, G - hc * Gc);
  const int pos0 = kvlen - qlen + tok0;  // position of the tile's first token
  const int rows_used = ntok * Gc;
  const int* table = p.block_tables + (size_t)s * p.max_blocks;

  // key range of the tile: [lo, hi), cut into `splits` runs of whole key tiles
  const int hi = pos0 + ntok;
  const int lo = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int first_tile = lo / BLOCK_N;
  const int tiles_total = (hi + BLOCK_N - 1) / BLOCK_N - first_tile;
  const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
  const int t_begin = first_tile + split * tiles_per_split;
  const int t_end = min(first_tile + tiles_total, t_begin + tiles_per_split);
  const int num_tiles = max(0, t_end - t_begin);

  // ---- Q tile to shared memory (rows beyond the used ones are zero)
  for (int idx = tid; idx < BLOCK_M * CHUNKS; idx += THREADS) {
    const int r = idx / CHUNKS, c = idx - r * CHUNKS;
    const int tok = r / Gc, hd = r - tok * Gc;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows_used && hd < nheads)
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + tok0 + tok) * p.q_stride + (size_t)(head0 + hd) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + r * ROW_BYTES + c * 16) = v;
  }

  auto load_tile = [&](int stage, int t) {
    load_kv_tile<BLOCK_N>(sK + stage * TILE_BYTES, sV + stage * TILE_BYTES, p.k_pool, p.v_pool, table, t * BLOCK_N, lo, hi, p.nkv, kvh,
                          p.page_size, tid, THREADS);
  };


  // per-thread rows: lane/4 and lane/4 + 8 of the warp's 16 rows
  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
  const bool warp_active = warp * 16 < rows_used;
  int rpos[2];
  bool rvalid[2];
  {
    const int t0 = r0 / Gc, t1 = r1 / Gc;
    rvalid[0] = r0 < rows_used && (r0 - t0 * Gc) < nheads;
    rvalid[1] = r1 < rows_used && (r1 - t1 * Gc) < nheads;
    rpos[0] = pos0 + t0;
    rpos[1] = pos0 + t1;
  }

  float m[2] = {-CUDART_INF_F, -CUDART_INF_F};
  float l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

  if (num_tiles > 0) load_tile(0, t_begin);
  cp_async_commit();

  for (int it = 0; it < num_tiles; ++it) {
    const int stage = it & 1;
    if (it + 1 < num_tiles) load_tile(stage ^ 1, t_begin + it + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    if (warp_active)
      tile_update<BLOCK_N>(sQ + warp * 16 * ROW_BYTES, sK + stage * TILE_BYTES, sV + stage * TILE_BYTES, (t_begin + it) * BLOCK_N,
                           rvalid, rpos, p.window, p.scale_log2, m, l, o, lane);
    __syncthreads();  // the stage is overwritten by the load issued next iteration
  }
  cp_async_wait<0>();

  if (!warp_active) return;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
    l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    if (!rvalid[rr]) continue;
    const int r = rr ? r1 : r0;
    const int tok = r / Gc, hd = r - tok * Gc;
    const size_t row = (size_t)(q0 + tok0 + tok) * p.nh + head0 + hd;  // (token, head) row of the batch
    if (p.splits == 1) {
      const float inv = 1.f / l[rr];
      bf16* dst = p.out + row * D;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        const int dim = j * 8 + (lane & 3) * 2;
        *reinterpret_cast<__nv_bfloat162*>(dst + dim) = __floats2bfloat162_rn(o[j][2 * rr] * inv, o[j][2 * rr + 1] * inv);
      }
    } else {
      float* dst = p.part_acc + (row * p.splits + split) * D;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        const int dim = j * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(dst + dim) = make_float2(o[j][2 * rr], o[j][2 * rr + 1]);
      }
      if ((lane & 3) == 0) {
        p.part_ml[(row * p.splits + split) * 2] = m[rr];
        p.part_ml[(row * p.splits + split) * 2 + 1] = l[rr];
      }
    }
  }
}


// ---------------------------------------------------------------- single-token sequences
// Two shapes of the decode kernel.  The loop is bound by instruction latency, not by tensor
// throughput, so occupancy decides: with many (sequence, KV head) pairs small tiles and a
// short pipeline leave room for five CTAs per SM; with few pairs a deeper pipeline of larger
// tiles keeps more bytes in flight per CTA.
template <int KEYS, int PIPE>
struct DecodeShape {
  static constexpr int N = KEYS;                      // keys per tile of one warp
  static constexpr int STAGES = PIPE;
  static constexpr int TILE = KEYS * ROW_BYTES;
  static constexpr int WARP = 2 * PIPE * TILE;        // K and V stages of one warp
  static constexpr int MERGE = NWARPS * 16 * (D + 2) * 4;  // per warp: o[16][D], m[16], l[16]
  static constexpr int SMEM = 16 * ROW_BYTES + (NWARPS * WARP > MERGE ? NWARPS * WARP : MERGE);
};
typedef DecodeShape<16, 2> DecodeMany;
typedef DecodeShape<(D <= 128 ? 32 : 16), (D <= 64 ? 3 : 2)> DecodeFew;

// grid (splits, sequences, kv heads * chunks of 16 query heads); every sequence brings one token.
template <typename Shape>
__global__ void __launch_bounds__(THREADS) paged_decode_mma_kernel(const Params p) {
  constexpr int DEC_N = Shape::N, DEC_STAGES = Shape::STAGES, DEC_TILE_BYTES = Shape::TILE, DEC_WARP_BYTES = Shape::WARP;
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sQ = smem;
  unsigned char* sKV = smem + 16 * ROW_BYTES;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int s = p.seq0 + blockIdx.y;
  const int split = blockIdx.x;
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
  const int first_tile = lo / DEC_N;
  const int tiles_total = (hi + DEC_N - 1) / DEC_N - first_tile;
  const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
  const int t_begin = first_tile + split * tiles_per_split;
  const int t_end = min(first_tile + tiles_total, t_begin + tiles_per_split);

  for (int idx = tid; idx < 16 * CHUNKS; idx += THREADS) {
    const int r = idx / CHUNKS, c = idx - r * CHUNKS;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nheads) v = *reinterpret_cast<const uint4*>(p.q + (size_t)token * p.q_stride + (size_t)(head0 + r) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + r * ROW_BYTES + c * 16) = v;
  }
  __syncthreads();

  unsigned char* wK = sKV + warp * DEC_WARP_BYTES;
  unsigned char* wV = wK + DEC_STAGES * DEC_TILE_BYTES;
  auto load_tile = [&](int stage, int t) {
    load_kv_tile<DEC_N>(wK + stage * DEC_TILE_BYTES, wV + stage * DEC_TILE_BYTES, p.k_pool, p.v_pool, table, t * DEC_N, lo, hi, p.nkv,
                        kvh, p.page_size, lane, 32);
  };


  const int rows[2] = {lane >> 2, (lane >> 2) + 8};
  const bool rvalid[2] = {rows[0] < nheads, rows[1] < nheads};
  const int rpos[2] = {pos, pos};
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F};
  float l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

  // this warp's tiles: t_begin + warp, + NWARPS, ...
  const int my_tiles = (t_end - t_begin - warp + NWARPS - 1) / NWARPS;
#pragma unroll
  for (int i = 0; i < DEC_STAGES - 1; ++i) {
    if (i < my_tiles) load_tile(i, t_begin + warp + i * NWARPS);
    cp_async_commit();
  }
  for (int it = 0; it < my_tiles; ++it) {
    const int stage = it % DEC_STAGES;
    if (it + DEC_STAGES - 1 < my_tiles) load_tile((it + DEC_STAGES - 1) % DEC_STAGES, t_begin + warp + (it + DEC_STAGES - 1) * NWARPS);
    cp_async_commit();
    cp_async_wait<DEC_STAGES - 1>();
    __syncwarp();
    tile_update<DEC_N>(sQ, wK + stage * DEC_TILE_BYTES, wV + stage * DEC_TILE_BYTES, (t_begin + warp + it * NWARPS) * DEC_N, rvalid,
                       rpos, p.window, p.scale_log2, m, l, o, lane);
    __syncwarp();  // the stage is overwritten by the load issued next iteration
  }
  cp_async_wait<0>();
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
    l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
  }

  // ---- merge the four warps' partial results in shared memory
  __syncthreads();  // every warp is done with its key and value stages
  float* mo = reinterpret_cast<float*>(sKV);          // [NWARPS][16][D]
  float* mm = mo + NWARPS * 16 * D;                    // [NWARPS][16]
  float* ml = mm + NWARPS * 16;                        // [NWARPS][16]
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    float* dst = mo + (warp * 16 + rows[rr]) * D;
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
      *reinterpret_cast<float2*>(dst + j * 8 + (lane & 3) * 2) = make_float2(o[j][2 * rr], o[j][2 * rr + 1]);
    if ((lane & 3) == 0) {
      mm[warp * 16 + rows[rr]] = m[rr];
      ml[warp * 16 + rows[rr]] = l[rr];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < nheads * D; idx += THREADS) {
    const int r = idx / D, dcol = idx - r * D;
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) mx = fmaxf(mx, mm[w * 16 + r]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float mw = mm[w * 16 + r];
      const float f = (mw == -CUDART_INF_F) ? 0.f : exp2f(mw - mx);
      L += ml[w * 16 + r] * f;
      acc += mo[(w * 16 + r) * D + dcol] * f;
    }
    const size_t row = (size_t)token * p.nh + head0 + r;
    if (p.splits == 1) {
      p.out[row * D + dcol] = __float2bfloat16_rn(acc / L);
    } else {
      p.part_acc[(row * p.splits + split) * D + dcol] = acc;
      if (dcol == 0) {
        p.part_ml[(row * p.splits + split) * 2] = mx;
        p.part_ml[(row * p.splits + split) * 2 + 1] = L;
      }
    }
  }
}

// out[row] = sum_i acc_i 2^(m_i - max m) / sum_i l_i 2^(m_i - max m); one block per (token, head) row.
__global__ void merge_splits_kernel(bf16* __restrict__ out, const float* __restrict__ part_acc,
                                    const float* __restrict__ part_ml, int row0, int splits) {
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
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < splits; ++i) {
      const float mi = ml[2 * i];
      if (mi != -CUDART_INF_F) acc += part_acc[(row * splits + i) * D + d] * exp2f(mi - mmax);
    }
    out[row * D + d] = __float2bfloat16_rn(acc * inv);
  }
}

}  // namespace

// One launch for the sequences [seq0, seq0 + num_seqs) of a batch, each of which brings at most
// max_q_len tokens.  With splits > 1 every one of them must bring exactly one token; part_acc and
// part_ml are scratch of (rows * splits * D) and (rows * splits * 2) floats, rows counted from
// token 0 of the batch up to the last token of these sequences.
DLI_EXPORT int dli_paged_attention_mma(void* out, const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                                       const int* block_tables, int max_blocks, const int* q_start, const int* kv_len,
                                       int seq0, int num_seqs, int max_q_len, int first_row, int nh, int nkv, int page_size,
                                       int window, float scale, int splits, float* part_acc, float* part_ml,
                                       cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (nkv < 1 || nh % nkv || splits < 1 || (splits > 1 && (max_q_len != 1 || !part_acc || !part_ml))) return DLI_ERR_UNSUPPORTED;
  static OncePerDevice configured;
  if (!configured.here()) {
    cudaError_t e = cudaFuncSetAttribute(paged_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(paged_decode_mma_kernel<DecodeMany>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeMany::SMEM);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(paged_decode_mma_kernel<DecodeFew>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeFew::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured.here() = true;
  }
  Params p;
  p.out = (bf16*)out; p.q = (const bf16*)q; p.q_stride = q_stride;
  p.k_pool = (const bf16*)k_pool; p.v_pool = (const bf16*)v_pool;
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.q_start = q_start; p.kv_len = kv_len; p.seq0 = seq0;
  p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int G = nh / nkv;
  p.heads_per_chunk = G < BLOCK_M ? G : BLOCK_M;
  p.head_chunks = (G + p.heads_per_chunk - 1) / p.heads_per_chunk;
  p.tokens_per_tile = BLOCK_M / p.heads_per_chunk;
  p.splits = splits; p.part_acc = part_acc; p.part_ml = part_ml;
  if (max_q_len == 1) {
    const dim3 grid(splits, num_seqs, nkv * ((G + 15) / 16));
    if ((long long)num_seqs * grid.z >= 2 * sm_count())
      launch_pdl((paged_decode_mma_kernel<DecodeMany>), grid, dim3(THREADS), DecodeMany::SMEM, stream, 1, p);
    else
      launch_pdl((paged_decode_mma_kernel<DecodeFew>), grid, dim3(THREADS), DecodeFew::SMEM, stream, 1, p);
  } else {
    const int tiles = (max_q_len + p.tokens_per_tile - 1) / p.tokens_per_tile;
    dim3 grid(tiles * splits, num_seqs, nkv * p.head_chunks);
    launch_pdl((paged_attention_mma_kernel), dim3(grid), dim3(THREADS), SMEM_BYTES, stream, 1, p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (splits > 1) {
    launch_pdl((merge_splits_kernel), dim3(num_seqs * nh), dim3(D < 128 ? 64 : 128), 0, stream, 1, (bf16*)out, part_acc, part_ml, first_row * nh, splits);
    e = cudaGetLastError();
  }
  return (int)e;
}

DLI_EXPORT int dli_paged_attention_mma_head_dim() { return D; }

// ---------------------------------------------------------------- entry point without allocation
#include "no_alloc_entry.h"

namespace {
// Scratch of the no-allocation entry point: part of the library's device image, one copy per
// GPU that loads the library.  In host code this name is only a handle for the runtime; the
// address a kernel can use comes from cudaGetSymbolAddress.
static __device__ __align__(256) float noalloc_scratch[DLI_NOALLOC_SCRATCH_FLOATS];
constexpr int NOALLOC_MAX_DEVICES = 64;
}  // namespace

DLI_EXPORT int dli_paged_decode_attention_noalloc(void* out, const void* q, long long q_stride, const void* k_pool,
                                                  const void* v_pool, const int* block_tables, int max_blocks, const int* q_start,
                                                  const int* kv_len, int seq0, int num_seqs, int first_row, int nh, int nkv,
                                                  int page_size, int window, float scale, int splits, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (splits < 1 || nh < 1 || first_row < 0) return DLI_ERR_UNSUPPORTED;
  // rows are counted from token 0 of the batch, as the ordinary entry point indexes its scratch
  const unsigned long long rows = (unsigned long long)(first_row + num_seqs) * (unsigned long long)nh;
  const unsigned long long need = rows * (unsigned long long)splits * (unsigned long long)(D + 2);
  if (need > DLI_NOALLOC_SCRATCH_FLOATS) return DLI_ERR_SCRATCH_TOO_SMALL;

  // set-up, once per device: the device address of the array, looked up with that device current
  static float* base[NOALLOC_MAX_DEVICES] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return DLI_ERR_UNSUPPORTED;
  if (!base[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    base[dev] = p;
  }
  float* part_acc = base[dev];
  float* part_ml = part_acc + rows * (unsigned long long)splits * (unsigned long long)D;
  if (splits == 1) part_acc = part_ml = nullptr;  // no partial results: the kernel writes the output itself
  return dli_paged_attention_mma(out, q, q_stride, k_pool, v_pool, block_tables, max_blocks, q_start, kv_len, seq0, num_seqs, 1,
                                 first_row, nh, nkv, page_size, window, scale, splits, part_acc, part_ml, stream);
}
