// out[t, f] = sum over k of x[t, k] * W[f, k]      (bfloat16 in; bfloat16 or float32 out)
//
// The matrix product of the decode step: a few tokens (t < 256) against a large weight matrix
// that is read once from HBM.  Weights take the 128-row side of the tensor-core instruction
// (features are the MMA's M, tokens its N), so a tile of 128 features x 64 k is one
// tcgen05.mma group whatever the number of tokens:
//
//   * TMA (cp.async.bulk.tensor, 128-byte swizzle) brings a [128 x 64] weight tile and the
//     [tokens x 64] activation tile of the same k range into shared memory, several stages ahead;
//     rows or columns beyond the matrices are filled with zeros by the copy itself;
//   * one thread issues tcgen05.mma (M = 128, N = tokens rounded up to 16, K = 16, four per
//     stage) into an accumulator in tensor memory; tcgen05.commit frees the stage and, at the
//     end, signals the epilogue;
//   * four warps read the accumulator with tcgen05.ld (lane = feature, column = token) and
//     store, coalesced along features — or finish the layer's next elementwise step in place:
//     SiLU(gate) * up, the rotary embedding with the write of keys and values into the cache, or
//     the residual addition with the first half of the next RMS norm (see Epilogue).
//
// The grid is (feature tiles, K slices).  Slices exist to fill the GPU when a matrix has few
// feature tiles.  The CTAs of one tile's slices form a thread-block cluster (up to 16, the largest this
// GPU takes; more than 8 is the kernel's opt-in): each
// pushes its partial sums of a token into the shared memory of the CTA that owns the token
// (distributed shared memory; st.async, which counts the bytes on the owner's mbarrier), and when
// its bytes are complete the owner adds them, slice 0 first, so the order is fixed, and writes the
// output.  No partial sum ever leaves the chip,
// and no scratch memory is needed.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the kernel records an error
// code in *error_flag (1 copies, 2 products, 3 accumulator, 5 the slices' partial sums), stops
// issuing work, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

using namespace dli;

namespace {

constexpr int BM = 128;       // features per CTA
constexpr int BK = 64;        // k per stage: 128 bytes of bfloat16, one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int BARRIER_BYTES = 512;  // behind the stages: mbarriers (at most 17), the TMEM address, the failure flag,
constexpr int WSUM_OFFSET = 192;    // four warp sums,
constexpr int RSTD_OFFSET = 256;    // and the row factors of up to RSTD_MAX_TOKENS tokens
constexpr int RSTD_MAX_TOKENS = 64;
constexpr unsigned WAIT_LIMIT = 1u << 24;
constexpr int MAX_SLICES = 16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// true when the phase with this parity has completed; false after `limit` polls
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned limit) {
  for (unsigned i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, swizzled in
// 128-byte mode: start address, 1024 bytes between groups of eight rows, layout code 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);          // bits 0-13: start address / 16
  d |= (uint64_t)0 << 16;                           // bits 16-29: leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                 // bits 32-45: stride byte offset / 16
  d |= (uint64_t)1 << 46;                           // bits 46-47: descriptor version of sm_100
  d |= (uint64_t)2 << 61;                           // bits 61-63: 128-byte swizzle
  return d;
}

// Instruction descriptor of kind::f16: float32 accumulator, bfloat16 A and B, both K-major.
__device__ __forceinline__ uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void store_out(void* out, int out_f32, size_t idx, float v) {
  if (out_f32) ((float*)out)[idx] = v;
  else ((__nv_bfloat16*)out)[idx] = __float2bfloat16_rn(v);
}

// What happens to the finished sums of a tile.
//   EP_STORE     out[t, f] = sum                                   (bfloat16 or float32)
//   EP_SWIGLU    the weight rows were interleaved in blocks of 64 (64 gate rows, then the 64 up rows of the
//                same features), so a tile holds both: out[t, 64 * tile + i] = silu(gate_i) * up_i
//   EP_ROTARY    the features are q | k | v heads of size d (d divides 128, so a head never straddles tiles):
//                q and k are rotated by the token's position (rotate-half pairing over the first `rot`
//                elements), q goes to out[t, nh * d], k and v into the cache pages at the token's slot
//   EP_RESIDUAL  the product is the delta of a residual stream: h[t, f] += sum (float32, in place),
//                out[t, f] = bfloat16(h[t, f] * gain[f]), the input of the next RMS norm's consumer, and
//                out_ssq[t, tile] = the tile's sum of h[t, f]^2.  The division by the row's RMS is left to
//                the product that reads `out` (row scaling, below): it is a factor per token, so it
//                commutes with the product and is applied to the float32 sums.
// Row scaling of the input (in_ssq != null): the activations are h * gain of EP_RESIDUAL; every sum of
// token t is multiplied by rsqrt(sum over in_tiles of in_ssq[t, .] * in_inv_size + in_eps).
enum { EP_STORE = 0, EP_SWIGLU = 1, EP_ROTARY = 2, EP_RESIDUAL = 3 };
struct Epilogue {
  int mode;
  const int* positions;
  const float* inv_freq;
  const int* slots;
  __nv_bfloat16* k_pool;
  __nv_bfloat16* v_pool;
  int nh, nkv, d, rot, page_size, write_kv;
  float* h;
  const float* gain;
  float* out_ssq;
  const float* in_ssq;
  int in_tiles;
  float in_eps, in_inv_size;
};

// fin: this token's 128 finished sums of the tile; fl: the feature of this thread; h_pre: h[t, f] if the
// caller loaded it ahead (have_h); gain: the next norm's weight of this feature (EP_RESIDUAL).  Called by all threads of the CTA together.
__device__ __forceinline__ void fused_epilogue(const Epilogue& ep, void* out, const float* fin, int t, int tile, int fl, int features,
                                               float* wsum, float h_pre, bool have_h, float gain) {
  if (ep.mode == EP_RESIDUAL) {
    const int f = tile * BM + fl;
    float hn = 0.f;
    if (f < features) {
      const size_t idx = (size_t)t * features + f;
      hn = (have_h ? h_pre : ep.h[idx]) + fin[fl];
      ep.h[idx] = hn;
      ((__nv_bfloat16*)out)[idx] = __float2bfloat16_rn(hn * gain);
    }
    const float sq = warp_sum(hn * hn);
    if ((fl & 31) == 0) wsum[fl >> 5] = sq;
    __syncthreads();
    if (fl == 0) ep.out_ssq[(size_t)t * gridDim.x + tile] = (wsum[0] + wsum[1]) + (wsum[2] + wsum[3]);
    __syncthreads();  // the warp sums are free for the next token
    return;
  }
  if (ep.mode == EP_SWIGLU) {
    const int I = features >> 1, col = tile * 64 + fl;
    if (fl < 64 && col < I) {
      const float g = fin[fl], u = fin[fl + 64];
      ((__nv_bfloat16*)out)[(size_t)t * I + col] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
    }
    return;
  }
  const int f = tile * BM + fl;
  if (f >= features) return;
  const int head = f / ep.d, i = f - head * ep.d;
  float val = fin[fl];
  if (head < ep.nh + ep.nkv && i < ep.rot) {
    const int half = ep.rot >> 1;
    const bool low = i < half;
    const float other = fin[low ? fl + half : fl - half];
    float sn, cs;
    sincosf((float)ep.positions[t] * ep.inv_freq[low ? i : i - half], &sn, &cs);
    val = low ? val * cs - other * sn : val * cs + other * sn;
  }
  const __nv_bfloat16 b = __float2bfloat16_rn(val);
  if (head < ep.nh) {
    ((__nv_bfloat16*)out)[((size_t)t * ep.nh + head) * ep.d + i] = b;
    return;
  }
  const int slot = ep.write_kv ? ep.slots[t] : -1;
  if (slot < 0) return;
  const int page = slot / ep.page_size, off = slot - page * ep.page_size;
  const int kvh = head - ep.nh;
  if (kvh < ep.nkv) ep.k_pool[(((size_t)page * ep.nkv + kvh) * ep.page_size + off) * ep.d + i] = b;
  else ep.v_pool[(((size_t)page * ep.nkv + (kvh - ep.nkv)) * ep.page_size + off) * ep.d + i] = b;
}

// (relaxed: the barrier only tells that every CTA of the cluster runs and has set up its mbarriers, which
// fence.mbarrier_init.release.cluster has made visible; no data is handed over through it)
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Store into the same shared-memory offset of another CTA of the cluster, and count the four bytes on that CTA's
// mbarrier at `local_bar` when they have landed: the receiver waits for its bytes and nobody for a cluster barrier.
__device__ __forceinline__ void st_async_peer(uint32_t local_addr, uint32_t local_bar, uint32_t cta_rank, float v) {
  uint32_t remote, remote_bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta_rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(local_bar), "r"(cta_rank));
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
               ::"r"(remote), "r"(__float_as_uint(v)), "r"(remote_bar) : "memory");
}
// as mbar_wait, for a barrier that other CTAs of the cluster complete
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, unsigned limit) {
  for (unsigned i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

__global__ void __launch_bounds__(128) skinny_gemm_kernel(const __grid_constant__ CUtensorMap map_w,
                                                          const __grid_constant__ CUtensorMap map_x, void* __restrict__ out,
                                                          int out_f32, int tokens, int features, int k_tiles, int tiles_per_slice,
                                                          int npad, int stages, int tmem_cols, int* error_flag, const Epilogue ep,
                                                          unsigned wait_limit, int skip_tile) {
  pdl_launch_dependents();
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int b_bytes = npad * BK * 2;
  const int stage_bytes = A_BYTES + b_bytes;
  uint64_t* bars = (uint64_t*)(smem + (size_t)stages * stage_bytes);  // full[stages], empty[stages], accum, reduced
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * stages + 2);
  volatile int* failed = (volatile int*)(tmem_slot + 1);
  float* wsum = (float*)((unsigned char*)bars + WSUM_OFFSET);
  float* rstd = (float*)((unsigned char*)bars + RSTD_OFFSET);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + stages), accum = smem_u32(bars + 2 * stages);
  const uint32_t reduced = accum + 8;  // completes when every slice's partial sums of this CTA's tokens have landed
  // tokens t = rank, rank + slices, .. of the cluster belong to this CTA
  const int owned = (int)blockIdx.y < tokens ? (tokens - (int)blockIdx.y + (int)gridDim.y - 1) / (int)gridDim.y : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(accum, 1);
    mbar_init(reduced, 1);
    if (gridDim.y > 1 && owned > 0) mbar_expect_tx(reduced, (uint32_t)(gridDim.y * owned * BM * 4));
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  if (gridDim.y > 1) cluster_arrive();  // waited for just before the first store into a peer's memory

  const int tile = blockIdx.x, slice = blockIdx.y;
  const int kt0 = slice * tiles_per_slice;
  const int nkt = max(0, min(k_tiles, kt0 + tiles_per_slice) - kt0);

  // The other lanes of the two role warps park at __syncwarp: if they polled the accumulator
  // barrier meanwhile, their warp would alternate between the poll and the role loop.
  if (warp == 0) {
    // ---- producer: TMA loads, `stages` ahead of the MMAs.  Weights do not depend on the
    // kernel that runs before this one, so the first stages' weight tiles are requested before
    // the wait on that kernel; the activations only after it.
    if (lane == 0) {
    // (skip_tile, -1 in every launch of the engine: the k tile whose copies a test leaves out, so that the wait
    // for them runs out; see dli_skinny_gemm_wait_test)
    const int pre = min(nkt, stages);
    for (int i = 0; i < pre; ++i) {
      if (kt0 + i == skip_tile) continue;
      mbar_expect_tx(full0 + 8 * i, (uint32_t)stage_bytes);
      tma_load_2d(smem_u32(smem + (size_t)i * stage_bytes), &map_w, (kt0 + i) * BK, tile * BM, full0 + 8 * i);
    }
    pdl_wait();
    for (int i = 0; i < pre; ++i)
      if (kt0 + i != skip_tile) tma_load_2d(smem_u32(smem + (size_t)i * stage_bytes) + A_BYTES, &map_x, (kt0 + i) * BK, 0, full0 + 8 * i);
    for (int i = pre; i < nkt; ++i) {
      const int s = i % stages;
      if (!mbar_wait(empty0 + 8 * s, ((i / stages) - 1) & 1, wait_limit)) {
        *failed = 1;
        atomicExch(error_flag, 1);
        break;
      }
      if (*failed) break;
      if (kt0 + i == skip_tile) continue;
      const uint32_t a = smem_u32(smem + (size_t)s * stage_bytes);
      mbar_expect_tx(full0 + 8 * s, (uint32_t)stage_bytes);
      tma_load_2d(a, &map_w, (kt0 + i) * BK, tile * BM, full0 + 8 * s);
      tma_load_2d(a + A_BYTES, &map_x, (kt0 + i) * BK, 0, full0 + 8 * s);
    }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- MMA issuer
    const uint32_t idesc = instr_desc(BM, npad);
    if (lane == 0) {
    for (int i = 0; i < nkt; ++i) {
      const int s = i % stages;
      if (!mbar_wait(full0 + 8 * s, (i / stages) & 1, wait_limit)) {
        *failed = 2;
        atomicExch(error_flag, 2);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a = smem_u32(smem + (size_t)s * stage_bytes);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k)
        umma(tmem, smem_desc_sw128(a + k * UMMA_K * 2), smem_desc_sw128(a + A_BYTES + k * UMMA_K * 2), idesc, (i | k) != 0);
      umma_commit(empty0 + 8 * s);  // arrives once these MMAs have read the stage
    }
    umma_commit(accum);  // arrives once every MMA issued so far has finished
    }
    __syncwarp();
  } else if (ep.in_ssq) {
    // ---- the other two warps: the factor of every token's row, while the products run
    // (a warp per token, a lane per tile's sum of squares: the loads of a token are in flight together, and
    // the order of the additions depends on the number of tiles alone)
    pdl_wait();
#pragma unroll 4
    for (int t = warp - 2; t < tokens; t += 2) {
      float sum = 0.f;
      for (int i = lane; i < ep.in_tiles; i += 32) sum += ep.in_ssq[(size_t)t * ep.in_tiles + i];
      sum = warp_sum(sum);
      if (lane == 0) rstd[t] = rsqrtf(sum * ep.in_inv_size + ep.in_eps);
    }
  }

  // ---- epilogue: all four warps; lane = feature row of the tile, column = token
  // (the norm's gain is a weight: asked for before anything is waited for)
  const int f_own = blockIdx.x * BM + (int)threadIdx.x;
  const float gain_pre = (ep.mode == EP_RESIDUAL && f_own < features) ? ep.gain[f_own] : 0.f;
  bool ok = true;
  if (nkt > 0) {
    ok = mbar_wait(accum, 0, wait_limit);
    if (!ok) atomicExch(error_flag, 3);
  }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  pdl_wait();  // the output may alias memory the kernel before this one still reads
  ok = ok && !*failed;
  const int fl = warp * 32 + lane, f = tile * BM + fl;
  const int slices = gridDim.y;  // the cluster spans the grid's y dimension: slice = rank in the cluster
  const bool scaled = ep.in_ssq != nullptr;
  if (scaled) __syncthreads();  // the row factors are in place
  // the residual of this CTA's first token is asked for now and used after the reduction
  const bool have_h = ep.mode == EP_RESIDUAL && slice < tokens && f < features;
  const float h_pre = have_h ? ep.h[(size_t)slice * features + f] : 0.f;
  const bool fused = ep.mode != EP_STORE;
  // With several slices, token t belongs to CTA (t mod slices) of the cluster.  Every CTA pushes its
  // partial sums of a token straight into the owner's shared memory (remote stores need no answer); each
  // store counts its bytes on the owner's mbarrier, the owner waits until all of them have landed (0.3 us
  // less than a cluster barrier, which also holds back the CTAs that own nothing) and adds them from its
  // own memory, slice 0 first.  Nobody reads a peer's memory, and a CTA leaves only after what was sent
  // to it has arrived, so CTAs may leave as they finish.
  //   recv[slice][owned token][feature of the tile], a region of its own behind the barriers: a peer
  // may push while this CTA's pipeline stages are still in use
  float* recv = reinterpret_cast<float*>(smem + (size_t)stages * stage_bytes + BARRIER_BYTES);
  const int owned_max = (tokens + slices - 1) / slices;
  const uint32_t recv_addr = smem_u32(recv);
  const int tok8 = (tokens + 7) & ~7;
  if (slices > 1) cluster_wait();  // every CTA of the cluster runs (they arrived during setup): its memory may be written
  for (int c = 0; c < npad && c < tok8; c += 8) {
    uint32_t r[8];
    if (nkt > 0 && ok) {
      const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c;
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                   : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) r[j] = 0u;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int t = c + j;
      if (t >= tokens) continue;
      if (slices > 1) {
        const int owner = t % slices, ti = t / slices;
        st_async_peer(recv_addr + (uint32_t)(((slice * owned_max + ti) * BM + fl) * 4), reduced, owner, __uint_as_float(r[j]));
      } else if (fused) {
        recv[t * BM + fl] = __uint_as_float(r[j]) * (scaled ? rstd[t] : 1.f);
      } else if (f < features) {
        store_out(out, out_f32, (size_t)t * features + f, __uint_as_float(r[j]) * (scaled ? rstd[t] : 1.f));
      }
    }
  }
  // finished sums of the owned tokens for the fused epilogues (they combine features of a tile)
  float* fin = slices > 1 ? recv + slices * owned_max * BM : recv;
  if (slices > 1) {
    if (owned > 0 && !mbar_wait_cluster(reduced, 0, wait_limit)) {  // every slice's partial sums of my tokens have arrived
      atomicExch(error_flag, 5);
      ok = false;
    }
    for (int t = slice, ti = 0; t < tokens && ok; t += slices, ++ti) {
      float acc = 0.f;
#pragma unroll 8
      for (int s2 = 0; s2 < slices; ++s2) acc += recv[(s2 * owned_max + ti) * BM + fl];  // slice 0 first
      if (scaled) acc *= rstd[t];
      if (fused) fin[ti * BM + fl] = acc;
      else if (f < features) store_out(out, out_f32, (size_t)t * features + f, acc);
    }
  }
  if (fused) {
    __syncthreads();  // the finished sums of every feature of the tile are in place
    for (int t = slice, ti = 0; t < tokens; t += slices, ++ti)
      fused_epilogue(ep, out, fin + ti * BM, t, tile, fl, features, wsum, h_pre, have_h && ti == 0, gain_pre);
  }

  // ---- teardown: nobody touches tensor memory after this barrier; warp 0 frees it
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
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

int* error_flag_device = nullptr;  // mapped pinned host memory: the host reads it without a copy
int* error_flag_host = nullptr;

}  // namespace

// Number of K slices recommended for the given sizes: enough CTAs to fill the GPU, no slice
// shorter than four k-tiles, at most 16 (the largest cluster of this GPU; 8 is the portable size).
DLI_EXPORT int dli_skinny_gemm_slices(int tokens, int features, int K) {
  const int tiles = (features + BM - 1) / BM;
  const int k_tiles = (K + BK - 1) / BK;
  int want = (sm_count() * 2 + tiles - 1) / tiles;
  int most = k_tiles / 4;
  if (most < 1) most = 1;
  if (most > MAX_SLICES) most = MAX_SLICES;
  int slices = want < most ? want : most;
  if (slices < 1) slices = 1;
  const int per = (k_tiles + slices - 1) / slices;
  return (k_tiles + per - 1) / per;  // no empty slice
}

static int launch_skinny(void* out, int out_f32, const void* x, const void* w, int tokens, int features, int K, int slices,
                         int max_stages, const Epilogue& ep, cudaStream_t stream, unsigned wait_limit = WAIT_LIMIT, int skip_tile = -1) {
  if (tokens < 1 || tokens > 256 || features < 1 || K < 8 || K % 8 || slices < 1 || slices > MAX_SLICES) return DLI_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return DLI_ERR_UNSUPPORTED;
  if (!error_flag_host) {
    if (cudaHostAlloc((void**)&error_flag_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) return (int)cudaGetLastError();
    *error_flag_host = 0;
    if (cudaHostGetDevicePointer((void**)&error_flag_device, error_flag_host, 0) != cudaSuccess) return (int)cudaGetLastError();
  }
  const int npad = (tokens + 15) & ~15;
  CUtensorMap map_w, map_x;
  if (!make_map(&map_w, w, features, K, BM) || !make_map(&map_x, x, tokens, K, npad)) return DLI_ERR_UNSUPPORTED;
  const int k_tiles = (K + BK - 1) / BK;
  const int per = (k_tiles + slices - 1) / slices;
  const int stage_bytes = A_BYTES + npad * BK * 2;
  int stages = per < 8 ? per : 8;
  // room for the partial sums pushed by every slice [slices][owned][128] and, for a fused epilogue, the
  // finished sums of the owned tokens (one slice: the tile's sums [tokens][128])
  const int owned = (tokens + slices - 1) / slices;
  const int scratch = slices > 1 ? (slices + (ep.mode != EP_STORE ? 1 : 0)) * owned * BM * 4 : (ep.mode != EP_STORE ? tokens * BM * 4 : 0);
  // A grid of more than one CTA per SM fits three per SM, all told; a smaller one takes 72 KB of stages
  // beside its scratch (two per SM, this kernel's and the next one's; measured: deeper pipelines were
  // slower in a chain of such kernels).  A caller that launches one CTA per SM and nothing behind it may ask for more.
  const int ctas = ((features + BM - 1) / BM) * slices;
  const int budget = max_stages > 0 ? 200 * 1024 : ctas > sm_count() ? 73 * 1024 - scratch : 72 * 1024;
  if (max_stages > 0 && stages > max_stages) stages = max_stages;
  const int fixed = BARRIER_BYTES + scratch + 1024;
  while (stages > 1 && (stages * stage_bytes > budget || stages * stage_bytes + fixed > 227 * 1024)) --stages;
  if (stages < 1) stages = 1;
  const int smem = stages * stage_bytes + fixed;
  if (smem > 227 * 1024) return DLI_ERR_UNSUPPORTED;
  int tmem_cols = 32;
  while (tmem_cols < npad) tmem_cols <<= 1;
  static OncePerDevice big_clusters;
  if (slices > 8 && !big_clusters.here()) {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
    big_clusters.here() = true;
  }
  static MaxPerDevice configured;
  if (smem > configured.here()) {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured.here() = smem;
  }
  cudaError_t e = launch_pdl(skinny_gemm_kernel, dim3((features + BM - 1) / BM, slices), dim3(128), (size_t)smem, stream, slices, map_w,
                             map_x, out, out_f32, tokens, features, k_tiles, per, npad, stages, tmem_cols, error_flag_device, ep, wait_limit, skip_tile);
  return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// Row scaling of the input (see Epilogue): in_ssq [tokens, in_tiles] or null.
static bool set_row_scale(Epilogue& ep, int tokens, const float* in_ssq, int in_tiles, float in_eps, int in_size) {
  ep.in_ssq = in_ssq;
  if (!in_ssq) return true;
  if (tokens > RSTD_MAX_TOKENS || in_tiles < 1 || in_size < 1) return false;
  ep.in_tiles = in_tiles; ep.in_eps = in_eps; ep.in_inv_size = 1.f / (float)in_size;
  return true;
}

DLI_EXPORT int dli_skinny_gemm(void* out, int out_f32, const void* x, const void* w, int tokens, int features, int K,
                               int slices, int max_stages, const float* in_ssq, int in_tiles, float in_eps, int in_size,
                               cudaStream_t stream) {
  Epilogue ep = {};
  ep.mode = EP_STORE;
  if (!set_row_scale(ep, tokens, in_ssq, in_tiles, in_eps, in_size)) return DLI_ERR_UNSUPPORTED;
  return launch_skinny(out, out_f32, x, w, tokens, features, K, slices, max_stages, ep, stream);
}

// act[tokens, features / 2] = silu(gate) * up, for weights whose rows are interleaved in blocks of 64
// (rows 128 j .. 128 j + 63: gate features 64 j .., rows 128 j + 64 .. 128 j + 127: the same up features).
DLI_EXPORT int dli_skinny_gemm_swiglu(void* act, const void* x, const void* w, int tokens, int features, int K, int slices,
                                      const float* in_ssq, int in_tiles, float in_eps, int in_size, cudaStream_t stream) {
  if (features % 128) return DLI_ERR_UNSUPPORTED;
  Epilogue ep = {};
  ep.mode = EP_SWIGLU;
  if (!set_row_scale(ep, tokens, in_ssq, in_tiles, in_eps, in_size)) return DLI_ERR_UNSUPPORTED;
  return launch_skinny(act, 0, x, w, tokens, features, K, slices, 0, ep, stream);
}

// q | k | v projection with the rotary embedding and the cache write in the epilogue: q_out [tokens, nh * d]
// receives the rotated queries; keys (rotated) and values go to the pools [pages, nkv, page_size, d] at slots[t].
DLI_EXPORT int dli_skinny_gemm_rotary(void* q_out, const void* x, const void* w, int tokens, int K, int slices, const int* positions,
                                      const float* inv_freq, const int* slots, void* k_pool, void* v_pool, int nh, int nkv, int d,
                                      int rot, int page_size, int write_kv, const float* in_ssq, int in_tiles, float in_eps,
                                      int in_size, cudaStream_t stream) {
  if (d < 2 || (BM % d) != 0 || rot < 0 || rot > d || (rot & 1) || (rot > 0 && !inv_freq)) return DLI_ERR_UNSUPPORTED;
  if (write_kv && (!slots || !k_pool || !v_pool)) return DLI_ERR_UNSUPPORTED;
  Epilogue ep = {};
  ep.mode = EP_ROTARY;
  if (!set_row_scale(ep, tokens, in_ssq, in_tiles, in_eps, in_size)) return DLI_ERR_UNSUPPORTED;
  ep.positions = positions; ep.inv_freq = inv_freq; ep.slots = slots;
  ep.k_pool = (__nv_bfloat16*)k_pool; ep.v_pool = (__nv_bfloat16*)v_pool;
  ep.nh = nh; ep.nkv = nkv; ep.d = d; ep.rot = rot; ep.page_size = page_size; ep.write_kv = write_kv;
  return launch_skinny(q_out, 0, x, w, tokens, (nh + 2 * nkv) * d, K, slices, 0, ep, stream);
}

// The delta of a residual stream with the first half of the next RMS norm (EP_RESIDUAL): h [tokens, features]
// float32 is updated in place, x_out [tokens, features] receives bfloat16(h * gain), out_ssq
// [tokens, ceil(features / 128)] the sums of squares per tile of 128 features.
DLI_EXPORT int dli_skinny_gemm_residual(void* x_out, float* h, const float* gain, float* out_ssq, const void* x, const void* w,
                                        int tokens, int features, int K, int slices, const float* in_ssq, int in_tiles, float in_eps,
                                        int in_size, cudaStream_t stream) {
  if (!h || !gain || !out_ssq) return DLI_ERR_UNSUPPORTED;
  Epilogue ep = {};
  ep.mode = EP_RESIDUAL;
  ep.h = h; ep.gain = gain; ep.out_ssq = out_ssq;
  if (!set_row_scale(ep, tokens, in_ssq, in_tiles, in_eps, in_size)) return DLI_ERR_UNSUPPORTED;
  return launch_skinny(x_out, 0, x, w, tokens, features, K, slices, 0, ep, stream);
}

// 0, or the code of the first wait that ran out (1 producer, 2 MMA issuer, 3 epilogue)
DLI_EXPORT int dli_skinny_gemm_error() { return error_flag_host ? *error_flag_host : 0; }
// Forget a recorded code (the host has read it); call with no launch of this library in flight.
DLI_EXPORT int dli_skinny_gemm_clear_error() { if (error_flag_host) *error_flag_host = 0; return 0; }

// For the test of the bounded waits only.  The plain product (float32 out, `slices` K slices), but the copies of
// k tile `skip_tile` are never issued and every wait gives up after `wait_limit` polls: the tensor-core warp's wait
// for that tile runs out, the kernel records code 2, stores whatever it has, completes its cluster barriers, frees
// its tensor memory and returns.  With skip_tile the last tile of a slice, and no more tiles in a slice than the
// pipeline has stages, no copy is in flight when the CTA leaves.  The engine never calls this.
DLI_EXPORT int dli_skinny_gemm_wait_test(void* out, const void* x, const void* w, int tokens, int features, int K, int slices,
                                         unsigned wait_limit, int skip_tile, cudaStream_t stream) {
  if (wait_limit < 1 || wait_limit > WAIT_LIMIT) return DLI_ERR_UNSUPPORTED;
  const int k_tiles = (K + BK - 1) / BK, per = (k_tiles + slices - 1) / (slices > 0 ? slices : 1);
  if (per > 8) return DLI_ERR_UNSUPPORTED;  // every tile of a slice has a stage of its own
  Epilogue ep = {};
  ep.mode = EP_STORE;
  return launch_skinny(out, 1, x, w, tokens, features, K, slices, 0, ep, stream, wait_limit, skip_tile);
}
