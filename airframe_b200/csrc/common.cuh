// Shared helpers of the sm_100a kernel library: dtype codes, conversions,
// reductions and the error channel of the C entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define AF_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes of the C interface
enum AfDtype { AF_F32 = 0, AF_BF16 = 1 };

// activation codes of the gated feed-forward
enum AfAct { AF_ACT_GELU_TANH = 0, AF_ACT_SILU = 1 };

// rotary pairings
enum AfPairing { AF_PAIR_HALF = 0, AF_PAIR_ADJACENT = 1 };

// The fused arg-max keeps one 64-bit key per token; keys lie this many words apart (a cache line each:
// every block of the head joins its best into every token's key, and keys in one line would queue up
// behind one another in the L2).
#define AF_KEY_STRIDE 16

// Tokens per cache page.  A sequence holds whole pages.
#define AF_PAGE 64

// The order in which the blocks of a tensor-core product walk its tiles (weight tiles x token tiles).
// group == 0: a weight tile's token tiles one after the other (a prompt of few token tiles: the blocks that work at
// the same time hold all of them).  Else the weight tiles in groups of `group`, within a group the weight tile
// fastest: the blocks at work share `group` weight tiles and about SMs / group token tiles, so that both
// operands come out of L2 (with thousands of token tiles the other order streams all activations from memory
// once for every weight tile).
#ifdef __CUDACC__
__host__ __device__ __forceinline__ void af_tile_of(int t, int tiles_w, int tiles_m, int group, int* wt, int* mt) {
  if (group <= 0) {
    *wt = t / tiles_m;
    *mt = t % tiles_m;
    return;
  }
  const int per_group = group * tiles_m;
  const int g = t / per_group, r = t - g * per_group;
  const int width = min(group, tiles_w - g * group);      // (the last group may hold fewer weight tiles)
  *wt = g * group + r % width;
  *mt = r / width;
}
// The group for these many token tiles on `sms` blocks.
__host__ __device__ __forceinline__ int af_tile_group(int tiles_m, int sms) {
  if (tiles_m <= 16) return 0;
  int g = 1;
  while ((g + 1) * (g + 1) <= sms) ++g;
  return g;
}
#endif

// Records a message that af_last_error() returns and yields the error code.
int af_fail(int code, const char* fmt, ...);

#define AF_REQUIRE(cond, ...)                     \
  do {                                            \
    if (!(cond)) return af_fail(-1, __VA_ARGS__); \
  } while (0)

// Kernels launched by this library since it was loaded (af_launch_count()).
extern unsigned long long g_af_launches;

#define AF_COUNT_LAUNCH(name)                                                    \
  do {                                                                           \
    cudaError_t e__ = cudaGetLastError();                                        \
    if (e__ != cudaSuccess)                                                      \
      return af_fail((int)e__, "%s: launch failed: %s", name, cudaGetErrorString(e__)); \
    ++g_af_launches;                                                             \
  } while (0)

#define AF_CHECK_LAUNCH(name) \
  do {                        \
    AF_COUNT_LAUNCH(name);    \
    return 0;                 \
  } while (0)

// ---- the checked build (-DAF_BOUNDS_CHECK)
// Indices that kernels take from data (a page of the page table, a row of a page table, a token id) are
// checked before they are used: a bad one is recorded (a word per translation unit: failed, the index) and
// its access is skipped; nothing traps.  af_bounds_failures() (elementwise.cu) reads and clears the words.
// In the normal build AF_INDEX_OK(cond, index) is `true` and costs nothing.
#ifdef AF_BOUNDS_CHECK
static __device__ int af_bounds_word[2];
typedef int (*AfBoundsReader)(int*);
void af_register_bounds_reader(AfBoundsReader reader);
static int af_bounds_read_here(int* out) {
  int zero[2] = {0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(out, af_bounds_word, sizeof(zero));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(af_bounds_word, zero, sizeof(zero));
  return (int)e;
}
static struct AfBoundsRegistration {
  AfBoundsRegistration() { af_register_bounds_reader(&af_bounds_read_here); }
} af_bounds_registration;
#define AF_INDEX_OK(cond, index) \
  ((cond) ? true : (atomicExch(&af_bounds_word[1], (int)(index)), atomicExch(&af_bounds_word[0], 1), false))
#else
#define AF_INDEX_OK(cond, index) true
#endif

// ---- the current device
// Limits and attributes belong to a device, not to the process: what is learnt or set once is
// kept per device ordinal.
constexpr int AF_MAX_DEVICES = 64;
// Ordinal of the current device, or -1 (with the error recorded) when it cannot be had or lies beyond AF_MAX_DEVICES.
int af_current_device();
// Streaming multiprocessors of the current device, asked of the driver once per device; <= 0 with the error recorded.
int af_sm_count();
// True the first time it is called for (flags, current device): the caller then sets what must be set once per device.
inline bool af_first_on_device(bool* flags, int dev) {
  if (dev < 0 || dev >= AF_MAX_DEVICES || flags[dev]) return false;
  flags[dev] = true;
  return true;
}

// ---- programmatic dependent launch
// Kernels are launched so that a kernel's blocks may become resident while the
// kernel before it in the stream still runs.  Every kernel calls
// pdl_launch_dependents() at its start and pdl_wait() before it reads or writes
// global memory that earlier kernels touch; pdl_wait() returns once every
// earlier kernel has finished and its memory is visible.  What a kernel does
// before the wait (barrier set-up, TMEM allocation, loads of weights) overlaps
// the tail of its predecessor.  af_set_pdl(0) turns the launch attribute off;
// the two instructions are then no-ops.
extern int g_af_pdl;

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// A kernel that does work before pdl_wait() passes every pointer to memory that earlier kernels
// write through this after the wait.  Loads through a `const __restrict__` pointer may be moved by
// the compiler across the wait (it takes the memory for unchanging while the kernel runs); it
// cannot move them across the point where the pointer's value becomes known.
template <typename T>
__device__ __forceinline__ T* pdl_fresh(T* p) {
  asm volatile("" : "+l"(p)::"memory");
  return p;
}

template <typename... KArgs, typename... Args>
inline cudaError_t af_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_af_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// cap * tanh(x / cap) for cap > 0, x otherwise (exact tanhf).
__device__ __forceinline__ float softcap_f32(float x, float cap) {
  return cap > 0.f ? cap * tanhf(x / cap) : x;
}

// Dispatch on a dtype code: DT becomes float or __nv_bfloat16.
#define AF_DISPATCH_DTYPE(code, DT, ...)                      \
  do {                                                        \
    if ((code) == AF_F32) {                                   \
      using DT = float;                                       \
      __VA_ARGS__;                                            \
    } else if ((code) == AF_BF16) {                           \
      using DT = __nv_bfloat16;                               \
      __VA_ARGS__;                                            \
    } else {                                                  \
      return af_fail(-1, "unsupported dtype code %d", (code)); \
    }                                                         \
  } while (0)
