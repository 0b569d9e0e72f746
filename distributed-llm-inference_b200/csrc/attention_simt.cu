// Paged causal attention on CUDA cores, any head size that is a multiple of 2 up to 256.
// It is the float32 path's attention (true 32-bit dot products and expf) and takes any mix
// of prompt portions and single decoded tokens: one warp per (token, query head) walks that
// token's keys 0..position through the block table in chunks of 32, so the order of every
// sum depends only on the token's own position, never on the batch or on how a prompt was cut.
#include "common.cuh"
#include <math_constants.h>

using namespace dli;

template <typename T>
__global__ void paged_attention_simt_kernel(T* __restrict__ out, const T* __restrict__ q, int q_stride,
                                            const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                            const int* __restrict__ block_tables, int max_blocks,
                                            const int* __restrict__ seq_of_token, const int* __restrict__ positions, int n,
                                            int nh, int nkv, int d, int page_size, int window, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31;
  const int warp_in_block = threadIdx.x >> 5;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + warp_in_block;
  if (warp >= (long long)n * nh) return;
  const int t = (int)(warp / nh), h = (int)(warp % nh);
  const int kvh = h / (nh / nkv);
  const int p = positions[t];
  const int* table = block_tables + (size_t)seq_of_token[t] * max_blocks;
  float* qs = smem + warp_in_block * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_float(q[(size_t)t * q_stride + (size_t)h * d + i]);
  __syncwarp();

  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  float m = -CUDART_INF_F, l = 0.f;
  float acc[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) acc[r] = 0.f;

  for (int base = lo; base <= p; base += 32) {
    const int key = base + lane;
    const bool valid = key <= p;
    float sc = -CUDART_INF_F;
    long long row = 0;  // element offset of this lane's key row in the pools
    if (valid) {
      const int page = table[key / page_size];
      row = (((long long)page * nkv + kvh) * page_size + key % page_size) * d;
      const T* kr = k_pool + row;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_float(kr[i]), dot);
      sc = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float pj = valid ? expf(sc - m_new) : 0.f;
    const float corr = expf(m - m_new);  // 0 on the first chunk (m = -inf, m_new finite)
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] *= corr;
    const int count = min(32, p - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pb = __shfl_sync(0xffffffffu, pj, j);
      const long long vrow = __shfl_sync(0xffffffffu, row, j);
      const T* vr = v_pool + vrow;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int i = lane + 32 * r;
        if (i < d) acc[r] = fmaf(pb, to_float(vr[i]), acc[r]);
      }
    }
    m = m_new;
  }
  const float inv = 1.f / l;
  T* o = out + (size_t)t * nh * d + (size_t)h * d;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int i = lane + 32 * r;
    if (i < d) o[i] = from_float<T>(acc[r] * inv);
  }
}

DLI_EXPORT int dli_paged_attention_simt(void* out, const void* q, int q_stride, const void* k_pool, const void* v_pool,
                                        const int* block_tables, int max_blocks, const int* seq_of_token,
                                        const int* positions, int n, int nh, int nkv, int d, int page_size, int window,
                                        float scale, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (d < 1 || d > 256 || nkv < 1 || nh % nkv) return DLI_ERR_UNSUPPORTED;
  const int warps = 4;
  const long long total = (long long)n * nh;
  const int blocks = (int)((total + warps - 1) / warps);
  const size_t smem = (size_t)warps * d * sizeof(float);
  if (dtype == DLI_F32)
    launch_pdl((paged_attention_simt_kernel<float>), dim3(blocks), dim3(warps * 32), smem, stream, 1, 
        (float*)out, (const float*)q, q_stride, (const float*)k_pool, (const float*)v_pool, block_tables, max_blocks,
        seq_of_token, positions, n, nh, nkv, d, page_size, window, scale);
  else
    launch_pdl((paged_attention_simt_kernel<__nv_bfloat16>), dim3(blocks), dim3(warps * 32), smem, stream, 1, 
        (__nv_bfloat16*)out, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
        block_tables, max_blocks, seq_of_token, positions, n, nh, nkv, d, page_size, window, scale);
  return (int)cudaGetLastError();
}
