// Shared device helpers: storage-type conversion, warp and block reductions.
// Every kernel in this folder computes in float and rounds once on store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace b200 {

constexpr int kWarp = 32;

// Storage types are selected at run time by an integer tag so that the C entry
// points need no templates in their signatures.
enum DType : int { kF32 = 0, kBF16 = 1 };

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// 16-byte vectors of the storage type: 4 floats or 8 bfloat16.
template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int n = 4;
  using type = float4;
  __device__ static void unpack(const type& v, float* f) { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
  __device__ static type pack(const float* f) { return make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int n = 8;
  using type = uint4;
  __device__ static void unpack(const type& v, float* f) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __bfloat1622float2(p[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static type pack(const float* f) {
    type v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
};

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

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  The order
// of additions depends only on blockDim, never on the data or on other blocks.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float total = (lane < nwarps) ? scratch[lane] : 0.f;
  total = warp_sum(total);
  return total;
}

// Launch status for the C entry points: 0 on success, else the cudaError value.
inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel started through launch() may begin while the
// kernel before it in the stream is still draining: everything it does before pdl_wait()
// (index arithmetic, fetching weights, which no kernel ever writes) overlaps that tail.
// pdl_wait() returns once the preceding kernels have completed and their writes are
// visible, so every read of an activation and every write must come after it.
// Every kernel started through launch() must call pdl_wait() on all paths that touch memory.
// LLM_RUNTIME_STUDY_B200_PDL=0 turns the overlap off (plain stream order).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
// The next kernel is released when a CTA exits (the implicit trigger).  Releasing it
// earlier, at the top of every CTA, was measured slower on the decode step: the
// dependent's CTAs then take SM slots while they wait.
__device__ __forceinline__ void pdl_trigger() {
#ifdef B200_PDL_EARLY_TRIGGER
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
#endif
}

// Unconditional release of the next kernel, for small kernels whose CTAs are all resident at once
// and whose successor does useful work before its own pdl_wait() (fetching weights, asking for
// cache pages of earlier steps).  What the successor does before its wait must not depend on this
// kernel or on any kernel before it.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// True in exactly one lane of a converged warp.  Code that every lane runs and that only issues its
// asynchronous instructions under this predicate keeps descriptors, addresses and counters in uniform
// registers, where the copy, barrier and MMA instructions take them from.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}

inline bool pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("LLM_RUNTIME_STUDY_B200_PDL");
    enabled = e ? (atoi(e) != 0 ? 1 : 0) : 1;
  }
  return enabled == 1;
}

template <typename... Params, typename... Args>
inline void launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// The opt-in to more than 48 KB of dynamic shared memory is an attribute of (kernel, device), and the
// number of SMs is the device's: a launcher keeps one of these per kernel and sets a device up the
// first time it launches there, whichever device is current.
constexpr int kMaxDevices = 64;
struct DeviceOnce {
  bool done[kMaxDevices] = {};
  int sm_count[kMaxDevices] = {};
};
// 0, or a cudaError_t / 10007 (device index out of range); *sm_count receives the current device's SM count.
template <typename Kernel>
inline int configure_once(DeviceOnce& once, Kernel kernel, size_t smem_bytes, int* sm_count = nullptr) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 10007;
  if (!once.done[device]) {
    if (smem_bytes > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    if (cudaDeviceGetAttribute(&once.sm_count[device], cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 10007;
    once.done[device] = true;
  }
  if (sm_count) *sm_count = once.sm_count[device];
  return 0;
}

}  // namespace b200

// Error codes of our own, above the CUDA range, for refused sizes.
#define B200_ERR_BAD_SIZE 10001
#define B200_ERR_BAD_DTYPE 10002
#define B200_ERR_TOO_LARGE 10003

#define B200_DISPATCH_DTYPE(tag, T, ...)                                  \
  switch (tag) {                                                          \
    case b200::kF32: { using T = float; __VA_ARGS__; break; }             \
    case b200::kBF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }    \
    default: return B200_ERR_BAD_DTYPE;                                   \
  }
