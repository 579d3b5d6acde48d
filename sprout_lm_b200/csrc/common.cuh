// Shared helpers of the sm_100a kernel library: error reporting to the host,
// element conversion, small reductions.  Every exported function is
// `extern "C"`, takes raw device pointers and a stream, validates its
// arguments on the host and returns 0 or a non-zero code whose text
// sprout_last_error() gives.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <utility>

#define SPROUT_API extern "C" __attribute__((visibility("default")))

enum SproutDtype : int { SPROUT_F32 = 0, SPROUT_BF16 = 1 };

// Bits of the device status word that kernels set instead of faulting.
enum SproutStatus : int {
  SPROUT_STATUS_BAD_PAGE = 1,       // a block-table entry outside the pool
  SPROUT_STATUS_BAD_TOKEN = 2,      // a token id outside the vocabulary
  SPROUT_STATUS_NONFINITE = 4,      // non-finite logits met while sampling
  SPROUT_STATUS_WAIT_TIMEOUT = 8,   // a bounded mbarrier wait ran out
  SPROUT_STATUS_BAD_POSITION = 16,  // a position outside the rotary table
  SPROUT_STATUS_BAD_LAYOUT = 32,    // a kernel's shared memory did not start where its tiles need it
};

int sprout_fail(const char* fmt, ...);   // records the message, returns 1
int sprout_check_launch(const char* what);
// Streaming multiprocessors of the current device (queried once per device; 148, the B200's count, where no
// device can be asked, which only host-side plan inspection meets).
extern "C" int sprout_sm_count();

// Programmatic dependent launch.  Every kernel of the library is launched so that it may start
// while the kernel before it in the stream still runs: it calls pdl_launch_dependents() at entry
// (its successor may be scheduled), does what does not depend on earlier kernels (set-up,
// loads of weights and tables) and calls pdl_wait() before it reads or writes anything an
// earlier kernel may have written.  pdl_wait() returns once all earlier kernels have completed
// and their writes are visible; every block executes it, so a kernel never completes before its
// predecessors.  sprout_set_pdl(0) turns the launch attribute off (the calls then do nothing).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

int sprout_pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t sprout_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = sprout_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

// With -DSPROUT_TIMELINE the kernels of a decode layer record when they ran (%globaltimer, ns): per
// file up to four kernels, each with the entry of its first CTA, the latest return of any CTA's
// wait for the earlier kernels, and the latest exit of any CTA's first thread.  Time only grows, so
// after a step the records are those of its last layer.  sprout_timeline_<file>(out) copies them out.
#ifdef SPROUT_TIMELINE
static __device__ unsigned long long g_sprout_tl[8][4];
__device__ __forceinline__ unsigned long long sprout_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define SPROUT_TL_ENTRY(slot) do { if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) g_sprout_tl[slot][0] = sprout_now_ns(); } while (0)
#define SPROUT_TL_WAITED(slot) do { if (threadIdx.x == 0) atomicMax(&g_sprout_tl[slot][1], sprout_now_ns()); } while (0)
#define SPROUT_TL_EXIT(slot) do { if (threadIdx.x == 0) atomicMax(&g_sprout_tl[slot][2], sprout_now_ns()); } while (0)
#define SPROUT_TL_READER(name) extern "C" __attribute__((visibility("default"))) void sprout_timeline_##name(unsigned long long* out) { cudaMemcpyFromSymbol(out, g_sprout_tl, sizeof(g_sprout_tl)); }
#else
#define SPROUT_TL_ENTRY(slot) do { } while (0)
#define SPROUT_TL_WAITED(slot) do { } while (0)
#define SPROUT_TL_EXIT(slot) do { } while (0)
#define SPROUT_TL_READER(name)
#endif

#define SPROUT_REQUIRE(cond, ...) \
  do { if (!(cond)) return sprout_fail(__VA_ARGS__); } while (0)

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Block-wide sum / max for blocks of up to 1024 threads; `scratch` holds 33 floats.
// Every thread gets the result.  The order of the additions is fixed by the
// block size alone.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < warps ? scratch[lane] : 0.f;
    w = warp_sum(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < warps ? scratch[lane] : -INFINITY;
    w = warp_max(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}
