// Shared device helpers for the engine's kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DLI_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python wrappers
#define DLI_F32 0
#define DLI_BF16 1

// error codes a launcher returns besides cudaError_t values (those are < 1000)
#define DLI_ERR_UNSUPPORTED 1001

#include <cstdlib>

namespace dli {

// Programmatic dependent launch.  Every kernel of the engine lets its successor start early
// (launch_dependents at its top) and waits for its predecessor's memory before it reads or
// writes anything the predecessor may touch (wait).  A launch then overlaps the tail of the
// kernel before it; a kernel that follows a library kernel simply starts when that one ends.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = std::getenv("DLI_B200_NO_PDL");
    on = (e && e[0] == '1') ? 0 : 1;
  }
  return on == 1;
}

// The current device (indices wrap at 64) and its number of SMs, asked once per device.
inline int current_device() {
  int d = 0;
  cudaGetDevice(&d);
  return d & 63;
}
inline int sm_count() {
  static int count[64] = {};
  const int d = current_device();
  if (!count[d]) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d);
    count[d] = v > 0 ? v : 1;
  }
  return count[d];
}
// Attributes of a kernel (dynamic shared memory, cluster size) are set per device: each device has its own
// copy of the kernel.  `here()` is the current device's flag (or largest value set so far).
struct OncePerDevice {
  bool done[64] = {};
  bool& here() { return done[current_device()]; }
};
struct MaxPerDevice {
  int value[64] = {};
  int& here() { return value[current_device()]; }
};

// Launch with the programmatic-serialization attribute (and, if cluster_y > 1, a cluster of
// that many CTAs along y).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_y,
                              Args... args) {
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
  if (cluster_y > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = cluster_y;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  return e != cudaSuccess ? e : cudaGetLastError();
}

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// The order of the additions depends only on blockDim, never on the data or the batch.
__device__ __forceinline__ float block_sum(float v, float* smem /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = (lane < (int)((blockDim.x + 31) >> 5)) ? smem[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) smem[32] = t;
  }
  __syncthreads();
  return smem[32];
}

}  // namespace dli
