// out[t, f] = sum over k of x[t, k] * W[f, k]      (bfloat16 in, bfloat16 out; float32 sums)
//
// The matrix product of a step that brings many tokens (a prompt's portion): tokens take the 128-row side of
// the tensor-core instruction, features its 256 columns, so a thread of the epilogue holds one token's row of
// a tile and the elementwise step that follows a product in the layer (SiLU(gate) * up; the rotary embedding
// with the cache write) can be done on the sums before they are stored: the product's raw output is then never
// written and re-read by a kernel of its own.
//
// Two CTAs, the two SMs of a cluster, work as one (tcgen05 cta_group::2): a pair owns a tile of 256 tokens x 256
// features, each CTA its 128 tokens of it in its own tensor memory, and each CTA loads only HALF of the weight tile
// (128 of its 256 rows); the instruction, issued by the pair's first CTA, reads both halves.
//
//   * A pair is persistent: it walks the tiles pair, pair + pairs, ... (token tile first: the pairs that run together
//     share few weight tiles).
//   * One thread of each CTA issues its TMA copies (cp.async.bulk.tensor, 128-byte swizzle) of a [128 x 64] tile of
//     x and a [128 x 64] half tile of W per k step, six steps ahead; rows beyond the matrices arrive as zeros.
//   * One thread of the first CTA issues tcgen05.mma (M = 2 x 128, N = 256, K = 16; four per k step) into one of TWO
//     accumulators in tensor memory (2 x 256 columns in each CTA), so the products of the next tile run while
//   * four warps of each CTA read the finished accumulator with tcgen05.ld (lane = token, column = feature), apply
//     the epilogue and store.
//
// Measured with one CTA to a tile of 128 x 256 first (48 KB a k step, four stages, the copies 2,048 tensor-core clocks
// ahead of the products): the tensor pipe stood idle a third of the time waiting for operands and the plain product
// took 1.12 of the library's time at 2,048 x 16,384 x 2,048; with the pair (32 KB a k step and CTA, six stages, 3,072
// clocks ahead) it takes 1.00.
//
//   full[s]      (first CTA)  both CTAs' copies of stage s have landed: their bytes are counted on the first CTA's barrier
//   empty[s]     (each CTA)   the products have read stage s: the commit arrives in both CTAs
//   acc_full[b]  (each CTA)   accumulator b is finished: the commit arrives in both CTAs
//   acc_empty[b] (first CTA)  the epilogue threads of both CTAs (256) have read accumulator b
//
// Every wait on an mbarrier is bounded: after `wait_limit` polls the kernel records a code in *error_flag,
// stops issuing work, frees its tensor memory and returns.  Neither CTA leaves before the other has reached the end.
#include <cuda.h>

#include "common.cuh"

using namespace dli;

namespace {

constexpr int BM = 128;   // tokens per CTA of a tile (a pair's tile has 256)
constexpr int BN = 256;   // features per tile
constexpr int BK = 64;    // k per stage: 128 bytes of bfloat16, one swizzle row
constexpr int A_BYTES = BM * BK * 2;
constexpr int THREADS = 192;  // warp 0: copies; warp 1: products (first CTA); warps 2..5: epilogue
constexpr unsigned WAIT_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// true when the phase with this parity has completed; false after `limit` polls or once another thread has failed
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned limit, volatile int* failed) {
  for (unsigned i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 1023) == 1023 && *failed) return false;
  }
  return false;
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, swizzled in 128-byte mode:
// start address, 1024 bytes between groups of eight rows, layout code 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor of kind::f16: float32 accumulator, bfloat16 A and B, both K-major.
__device__ __forceinline__ uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
        "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
        "=r"(v[31])
      : "r"(taddr));
}

// What happens to a token's finished sums of a tile (as in the decode product):
//   EP_STORE     out[t, f] = sum
//   EP_SWIGLU    the weight rows are interleaved in blocks of 64 (64 gate rows, then the 64 up rows of the same
//                features): out[t, 64 * block + i] = silu(gate_i) * up_i, out being [tokens, features / 2]
//   EP_ROTARY    the features are q | k | v heads of size d (64 or 128: a head never straddles tiles).  q and k are
//                rotated by the token's position (rotate-half pairing over the first `rot` elements, rot 0, 64 or
//                128; cosines and sines from the step's table [tokens, rot]: cos | sin); q goes to
//                out[t, nh * d], k and v into the cache pages at the token's slot
enum { EP_STORE = 0, EP_SWIGLU = 1, EP_ROTARY = 2 };
struct DenseParams {
  __nv_bfloat16* out;
  int tokens, features, k_tiles, m_tiles, n_tiles;
  int* error_flag;
  unsigned wait_limit;
  int mode;
  const float* trig;   // EP_ROTARY: [tokens, rot]
  const int* slots;
  __nv_bfloat16* k_pool;
  __nv_bfloat16* v_pool;
  int nh, nkv, d, rot, page_size, write_kv;
  int skip_tile;  // -1 in every launch of the engine: the k step whose copies a test leaves out (dli_dense_gemm_wait_test)
};

// 32 consecutive columns of this thread's row of the accumulator.  `rounded`: as bfloat16 would hold them.  The
// epilogues that go on computing take the sums so: a portion's activations are then what the library's product,
// which stores bfloat16, and the separate kernel behind it would have made of them, and a prompt's keys, values
// and activations do not depend on which of the two ways its portion took.
__device__ __forceinline__ void load_chunk(uint32_t taddr, float (&f)[32], bool rounded = false) {
  uint32_t v[32];
  tmem_ld32(taddr, v);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int j = 0; j < 32; ++j) f[j] = rounded ? __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[j]))) : __uint_as_float(v[j]);
}

__device__ __forceinline__ void store8(__nv_bfloat16* dst, const float* v) {
  uint4 w;
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
  for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  *reinterpret_cast<uint4*>(dst) = w;
}
// 32 floats from global memory, eight 16-byte loads issued together (nothing between them that could alias)
__device__ __forceinline__ void load32(const float* src, float (&f)[32]) {
  float4 v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = *reinterpret_cast<const float4*>(src + 4 * j);
#pragma unroll
  for (int j = 0; j < 8; ++j) { f[4 * j] = v[j].x; f[4 * j + 1] = v[j].y; f[4 * j + 2] = v[j].z; f[4 * j + 3] = v[j].w; }
}

// The epilogue of one tile for the thread that holds token `row`: acc is the tensor-memory address of column 0 of
// its row.  Every thread of the warp runs through the same tensor-memory loads (they are warp-wide); global memory is
// per thread, a row each, in runs of 64 or 128 bytes.  (Tried: handing the rows round through shared memory so that
// a warp touches one row per instruction; the extra passes cost more than the scattered sectors: q|k|v with rotary
// 41 -> 74 us at 2,048 tokens.)  What an epilogue reads from global memory (cosines and sines) is asked for before
// the accumulator's chunk is waited for, all loads of a chunk together.
__device__ __forceinline__ void epilogue_row(const DenseParams& p, uint32_t acc, int row, int n) {
  const bool live = row < p.tokens;
  const int f0 = n * BN;  // first feature of the tile
  if (p.mode == EP_STORE) {
    __nv_bfloat16* dst = p.out + (size_t)row * p.features + f0;
#pragma unroll 1
    for (int c = 0; c < BN && f0 + c < p.features; c += 32) {
      float f[32];
      load_chunk(acc + c, f);
      if (live) {
#pragma unroll
        for (int j = 0; j < 32; j += 8)
          if (f0 + c + j < p.features) store8(dst + c + j, f + j);  // features are a multiple of 8
      }
    }
    return;
  }
  if (p.mode == EP_SWIGLU) {
    const int I = p.features >> 1;
#pragma unroll 1
    for (int b = 0; b < BN / 128; ++b)
#pragma unroll 1
      for (int j = 0; j < 64; j += 32) {
        const int col = (n * (BN / 128) + b) * 64 + j;
        if (col >= I) break;
        float g[32], u[32];
        load_chunk(acc + b * 128 + j, g, true);
        load_chunk(acc + b * 128 + 64 + j, u, true);
        if (live) {
#pragma unroll
          for (int e = 0; e < 32; ++e) g[e] = g[e] / (1.f + expf(-g[e])) * u[e];
#pragma unroll
          for (int e = 0; e < 32; e += 8)
            if (col + e < I) store8(p.out + (size_t)row * I + col + e, g + e);
        }
      }
    return;
  }
  if (p.mode == EP_ROTARY) {
    const int half = p.rot >> 1;
    const float* trig = p.trig + (size_t)row * p.rot;  // cos [half] | sin [half]
    const int slot = (live && p.write_kv) ? p.slots[row] : -1;
    const int page = slot >= 0 ? slot / p.page_size : 0, off = slot >= 0 ? slot - page * p.page_size : 0;
#pragma unroll 1
    for (int hd = 0; hd < BN / 64 && f0 + hd * 64 < p.features; hd += p.d / 64) {  // heads of the tile (a head is 64 or 128 columns)
      const int head = (f0 + hd * 64) / p.d;
      __nv_bfloat16* dst = nullptr;  // where this head's d elements of the token go
      if (live) {
        if (head < p.nh) dst = p.out + ((size_t)row * p.nh + head) * p.d;
        else if (slot >= 0 && head < p.nh + p.nkv) dst = p.k_pool + (((size_t)page * p.nkv + (head - p.nh)) * p.page_size + off) * p.d;
        else if (slot >= 0) dst = p.v_pool + (((size_t)page * p.nkv + (head - p.nh - p.nkv)) * p.page_size + off) * p.d;
      }
      const bool rotated = head < p.nh + p.nkv;
      const uint32_t hacc = acc + hd * 64;
      int i = 0;
      if (rotated) {
#pragma unroll 1
        for (; i < half; i += 32) {  // pairs (i + e, i + half + e)
          float cs[32], sn[32];
          if (dst) {
            load32(trig + i, cs);
            load32(trig + half + i, sn);
          }
          float lo[32], hi[32];
          load_chunk(hacc + i, lo, true);
          load_chunk(hacc + half + i, hi, true);
          if (dst) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float a = lo[e], bb = hi[e];
              lo[e] = a * cs[e] - bb * sn[e];
              hi[e] = bb * cs[e] + a * sn[e];
            }
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              store8(dst + i + e, lo + e);
              store8(dst + half + i + e, hi + e);
            }
          }
        }
        i = p.rot;
      }
#pragma unroll 1
      for (; i < p.d; i += 32) {  // elements that pass through (beyond rot; every element of a value head)
        float f[32];
        load_chunk(hacc + i, f);
        if (dst) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) store8(dst + i + e, f + e);
        }
      }
    }
  }
}

constexpr int PAIR_STAGES = 6;  // of a [128 x 64] tile of x and a [128 x 64] half tile of W
constexpr int PAIR_B_BYTES = (BN / 2) * BK * 2;
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 256 + 1024;
static_assert(PAIR_SMEM_BYTES <= 227 * 1024, "one CTA per SM");
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;  // a shared-memory address with this bit cleared names the pair's first CTA

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a copy whose bytes are counted on the barrier of the pair's first CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar & PEER_BIT_MASK), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the products issued so far have finished, on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_at(uint32_t bar, uint32_t cta) {
  asm volatile("{\n\t.reg .b32 remote;\n\tmapa.shared::cluster.u32 remote, %0, %1;\n\tmbarrier.arrive.shared::cluster.b64 _, [remote];\n\t}"
               ::"r"(bar), "r"(cta) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1) dense_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                     const __grid_constant__ CUtensorMap map_w, const DenseParams p) {
  pdl_launch_dependents();
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + PAIR_STAGES * PAIR_STAGE_BYTES);  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * PAIR_STAGES + 4);
  volatile int* failed = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: the CTA that issues the products
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + PAIR_STAGES), acc_full0 = smem_u32(bars + 2 * PAIR_STAGES),
                 acc_empty0 = smem_u32(bars + 2 * PAIR_STAGES + 2);
  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 256);  // every epilogue thread of both CTAs has read its row
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // the other CTA's barriers are set up before anything is sent to them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  const int m_pairs = (p.m_tiles + 1) / 2;  // tiles of 256 tokens
  const int tiles = m_pairs * p.n_tiles;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ---- copies: this CTA's 128 tokens and its half of the weight tile's rows
    if (lane == 0) {
      pdl_wait();  // the activations are the work of the kernel before this one
      int it = 0;
      for (int tile = pair; tile < tiles && !*failed; tile += pairs) {
        const int m = tile % m_pairs, n = tile / m_pairs;
        for (int kt = 0; kt < p.k_tiles; ++kt, ++it) {
          const int s = it % PAIR_STAGES;
          if (it >= PAIR_STAGES && !mbar_wait(empty0 + 8 * s, ((it / PAIR_STAGES) - 1) & 1, p.wait_limit, failed)) {
            if (!*failed) { *failed = 1; atomicCAS(p.error_flag, 0, 1); }
            break;
          }
          if (kt == p.skip_tile) continue;
          const uint32_t a = smem_u32(smem + (size_t)s * PAIR_STAGE_BYTES);
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * PAIR_STAGE_BYTES);
          tma_load_2d_pair(a, &map_x, kt * BK, m * 2 * BM + (int)rank * BM, full0 + 8 * s);
          tma_load_2d_pair(a + A_BYTES, &map_w, kt * BK, n * BN + (int)rank * (BN / 2), full0 + 8 * s);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- products: the first CTA's thread issues them for both
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = instr_desc(2 * BM, BN);
      int it = 0, local = 0;
      for (int tile = pair; tile < tiles && !*failed; tile += pairs, ++local) {
        const int buf = local & 1;
        if (local >= 2 && !mbar_wait(acc_empty0 + 8 * buf, ((local >> 1) - 1) & 1, p.wait_limit, failed)) {
          if (!*failed) { *failed = 2; atomicCAS(p.error_flag, 0, 2); }
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        bool ok = true;
        for (int kt = 0; kt < p.k_tiles; ++kt, ++it) {
          const int s = it % PAIR_STAGES;
          if (!mbar_wait(full0 + 8 * s, (it / PAIR_STAGES) & 1, p.wait_limit, failed)) {
            if (!*failed) { *failed = 3; atomicCAS(p.error_flag, 0, 3); }
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a = smem_u32(smem + (size_t)s * PAIR_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_pair(tmem + buf * BN, smem_desc_sw128(a + k * 32), smem_desc_sw128(a + A_BYTES + k * 32), idesc, (kt | k) != 0);
          umma_commit_pair(empty0 + 8 * s);  // arrives in both CTAs once these products have read the stage
        }
        if (!ok) break;
        umma_commit_pair(acc_full0 + 8 * buf);  // arrives in both CTAs once every product of the tile has finished
      }
    }
    __syncwarp();
  } else {
    // ---- epilogue: this CTA's 128 tokens of the tile
    const int quad = warp & 3;
    const uint32_t lane_bits = (uint32_t)(quad * 32) << 16;
    pdl_wait();  // the output may alias memory that the kernel before this one still reads
    int local = 0;
    for (int tile = pair; tile < tiles; tile += pairs, ++local) {
      const int m = tile % m_pairs, n = tile / m_pairs;
      const int buf = local & 1;
      bool ok = mbar_wait(acc_full0 + 8 * buf, (local >> 1) & 1, p.wait_limit, failed);
      if (!ok && !*failed) { *failed = 4; atomicCAS(p.error_flag, 0, 4); }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      epilogue_row(p, tmem + buf * BN + lane_bits, m * 2 * BM + (int)rank * BM + quad * 32 + lane, n);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive_at(acc_empty0 + 8 * buf, 0);
    }
  }

  // ---- teardown: neither CTA leaves while the other may still send to its barriers or read its shared memory
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
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
// [rows, K] bfloat16 row-major, boxes of [box_rows x 64 k], 128-byte swizzle, zeros outside
bool make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
  EncodeTiled fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int* error_flag_device = nullptr;
int* error_flag_host = nullptr;

}  // namespace

// launch_pdl with the cluster along x
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl_x(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  attr[n].id = cudaLaunchAttributeClusterDimension;
  attr[n].val.clusterDim.x = cluster_x;
  attr[n].val.clusterDim.y = 1;
  attr[n].val.clusterDim.z = 1;
  ++n;
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

static int launch_dense(DenseParams p, const void* x, const void* w, int tokens, int features, int K, cudaStream_t stream) {
  if (tokens < 1 || features < 8 || features % 8 || K < 8 || K % 8) return DLI_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)p.out) & 15) return DLI_ERR_UNSUPPORTED;
  if (!error_flag_host) {
    if (cudaHostAlloc((void**)&error_flag_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) return (int)cudaGetLastError();
    *error_flag_host = 0;
    if (cudaHostGetDevicePointer((void**)&error_flag_device, error_flag_host, 0) != cudaSuccess) return (int)cudaGetLastError();
  }
  CUtensorMap map_x, map_w;
  if (!make_map(&map_x, x, tokens, K, BM) || !make_map(&map_w, w, features, K, BN / 2)) return DLI_ERR_UNSUPPORTED;  // W in boxes of half a tile's rows
  p.tokens = tokens; p.features = features;
  p.k_tiles = (K + BK - 1) / BK;
  p.m_tiles = (tokens + BM - 1) / BM;
  p.n_tiles = (features + BN - 1) / BN;
  p.error_flag = error_flag_device;
  if (p.wait_limit == 0) {
    p.wait_limit = WAIT_LIMIT;
    p.skip_tile = -1;
  }
  static OncePerDevice configured;
  if (!configured.here()) {
    cudaError_t e = cudaFuncSetAttribute(dense_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured.here() = true;
  }
  const long long tiles = (long long)((p.m_tiles + 1) / 2) * p.n_tiles;
  const long long pairs = sm_count() / 2;
  const int grid = 2 * (int)(tiles < pairs ? tiles : pairs);
  cudaError_t e = launch_pdl_x(dense_gemm_pair_kernel, dim3(grid), dim3(THREADS), (size_t)PAIR_SMEM_BYTES, stream, 2, map_x, map_w, p);
  return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// out [tokens, features] = x [tokens, K] times w [features, K] transposed.  K and features multiples of 8.
DLI_EXPORT int dli_dense_gemm(void* out, const void* x, const void* w, int tokens, int features, int K, cudaStream_t stream) {
  DenseParams p = {};
  p.out = (__nv_bfloat16*)out;
  p.mode = EP_STORE;
  return launch_dense(p, x, w, tokens, features, K, stream);
}

// act [tokens, features / 2] = silu(gate) * up, for weights whose rows are interleaved in blocks of 64.
DLI_EXPORT int dli_dense_gemm_swiglu(void* act, const void* x, const void* w, int tokens, int features, int K, cudaStream_t stream) {
  if (features % 128) return DLI_ERR_UNSUPPORTED;
  DenseParams p = {};
  p.out = (__nv_bfloat16*)act;
  p.mode = EP_SWIGLU;
  return launch_dense(p, x, w, tokens, features, K, stream);
}

// q | k | v projection with the rotary embedding and the cache write in the epilogue: q_out [tokens, nh * d] receives
// the rotated queries; keys (rotated) and values go to the pools [pages, nkv, page_size, d] at slots[t].  trig
// [tokens, rot] float32: the cosines, then the sines, of every token's angles.  d 64 or 128; rot 0, 64 or 128, <= d.
DLI_EXPORT int dli_dense_gemm_rotary(void* q_out, const void* x, const void* w, int tokens, int K, const float* trig, const int* slots,
                                     void* k_pool, void* v_pool, int nh, int nkv, int d, int rot, int page_size, int write_kv,
                                     cudaStream_t stream) {
  if ((d != 64 && d != 128) || (rot != 0 && rot != 64 && rot != 128) || rot > d || (rot > 0 && !trig)) return DLI_ERR_UNSUPPORTED;
  if (write_kv && (!slots || !k_pool || !v_pool || page_size < 1)) return DLI_ERR_UNSUPPORTED;
  if (((uintptr_t)trig | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return DLI_ERR_UNSUPPORTED;
  DenseParams p = {};
  p.out = (__nv_bfloat16*)q_out;
  p.mode = EP_ROTARY;
  p.trig = trig; p.slots = slots; p.k_pool = (__nv_bfloat16*)k_pool; p.v_pool = (__nv_bfloat16*)v_pool;
  p.nh = nh; p.nkv = nkv; p.d = d; p.rot = rot; p.page_size = page_size; p.write_kv = write_kv;
  return launch_dense(p, x, w, tokens, (nh + 2 * nkv) * d, K, stream);
}

// For the test of the bounded waits only.  The plain product of ONE tile (tokens <= 256, features <= 256) whose k
// steps all have a stage of their own (K <= 384), but neither CTA issues the copies of the last k step and every wait
// gives up after `wait_limit` polls: the waits for those operands, and for the accumulator that depends on them, run
// out; the kernel records the first one's code, both CTAs reach the end together, free their tensor memory and
// return.  No copy is in flight then: every copy that was issued has been waited for.  The engine never calls this.
DLI_EXPORT int dli_dense_gemm_wait_test(void* out, const void* x, const void* w, int tokens, int features, int K, unsigned wait_limit,
                                        cudaStream_t stream) {
  const int k_tiles = (K + BK - 1) / BK;
  if (wait_limit < 1 || wait_limit > WAIT_LIMIT || tokens > 2 * BM || features > BN || k_tiles > PAIR_STAGES || k_tiles < 1) return DLI_ERR_UNSUPPORTED;
  DenseParams p = {};
  p.out = (__nv_bfloat16*)out;
  p.mode = EP_STORE;
  p.wait_limit = wait_limit;
  p.skip_tile = k_tiles - 1;
  return launch_dense(p, x, w, tokens, features, K, stream);
}

// 0, or the code of the first wait that ran out (1 copies, 2 and 3 products, 4 epilogue)
DLI_EXPORT int dli_dense_gemm_error() { return error_flag_host ? *error_flag_host : 0; }
DLI_EXPORT int dli_dense_gemm_clear_error() { if (error_flag_host) *error_flag_host = 0; return 0; }
