// Embedding gather, RMS norms (plain and fused with the residual sum), the
// gated activation, logit softcap, and the library's error channel.
//
// All statistics, the residual sum and the (offset + w) factor are 32-bit.
// The residual stream is float in both precisions; the normalised rows that
// feed matrix products are in the compute dtype.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

int af_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code == 0 ? -1 : code;
}

AF_EXPORT const char* af_last_error() { return g_error; }

AF_EXPORT int af_abi_version() { return 1; }

int af_current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    af_fail((int)e, "cudaGetDevice: %s", cudaGetErrorString(e));
    return -1;
  }
  if (dev < 0 || dev >= AF_MAX_DEVICES) {
    af_fail(-1, "device ordinal %d beyond the %d this library keeps state for", dev, AF_MAX_DEVICES);
    return -1;
  }
  return dev;
}

int af_sm_count() {
  static int sms[AF_MAX_DEVICES] = {};
  const int dev = af_current_device();
  if (dev < 0) return -1;
  if (sms[dev] == 0) {
    int n = 0;
    cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || n <= 0) {
      af_fail(e != cudaSuccess ? (int)e : -1, "the multiprocessor count of device %d: %s", dev, cudaGetErrorString(e));
      return -1;
    }
    sms[dev] = n;
  }
  return sms[dev];
}

// Streaming multiprocessors of the current device (the policies that cut work into blocks ask for it).
AF_EXPORT int af_device_sm_count() { return af_sm_count(); }

// The checked build's record: how many translation units saw a bad index since the last call (0: none),
// *index one of the bad values.  The normal build checks nothing and answers -1.
#ifdef AF_BOUNDS_CHECK
static AfBoundsReader g_bounds_readers[32];
static int g_n_bounds_readers = 0;
void af_register_bounds_reader(AfBoundsReader reader) {
  if (g_n_bounds_readers < 32) g_bounds_readers[g_n_bounds_readers++] = reader;
}
AF_EXPORT int af_bounds_failures(int* index) {
  cudaDeviceSynchronize();
  int failed = 0;
  for (int i = 0; i < g_n_bounds_readers; ++i) {
    int w[2] = {0, 0};
    if (g_bounds_readers[i](w) != 0) return af_fail(-1, "af_bounds_failures: cannot read a record");
    if (w[0]) {
      ++failed;
      if (index) *index = w[1];
    }
  }
  return failed;
}
#else
AF_EXPORT int af_bounds_failures(int* index) {
  (void)index;
  return -1;
}
#endif

unsigned long long g_af_launches = 0;
int g_af_pdl = 1;

// 1 (default): kernels may start while their predecessor in the stream is finishing; 0: plain stream order.
AF_EXPORT void af_set_pdl(int on) { g_af_pdl = on ? 1 : 0; }

AF_EXPORT unsigned long long af_launch_count() { return g_af_launches; }

// ---------------------------------------------------------------- embedding

template <typename TW>
__global__ void embed_kernel(float* __restrict__ out, const TW* __restrict__ table,
                             const int* __restrict__ ids, int hidden, int vocab, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  // ids are validated on the host; a bad one yields zeros rather than a wild read
  const bool ok = id >= 0 && id < vocab;
  (void)AF_INDEX_OK(ok, id);
  const TW* row = table + (size_t)(ok ? id : 0) * hidden;
  float* o = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = ok ? to_f32(row[i]) * scale : 0.f;
}

AF_EXPORT int af_embed(float* out, const void* table, int table_dtype, const int* ids, int n_tokens,
                       int hidden, int vocab, float scale, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0, "af_embed: bad sizes");
  AF_DISPATCH_DTYPE(table_dtype, TW,
                    af_launch(embed_kernel<TW>, dim3(n_tokens), dim3(256), 0, stream, out, (const TW*)table, ids, hidden,
                                                                  vocab, scale));
  AF_CHECK_LAUNCH("af_embed");
}

// ---------------------------------------------------------------- RMS norm

// y[r] = x[src(r)] * rsqrt(mean(x^2) + eps) * (offset + w); rows gathered by
// `rows` when given (the final norm runs at the wanted positions only).
template <typename TY>
__global__ void rmsnorm_kernel(TY* __restrict__ y, const float* __restrict__ x,
                               const float* __restrict__ w, const int* __restrict__ rows, int hidden,
                               float eps, float offset) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = xr[i];
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TY* yr = y + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    yr[i] = from_f32<TY>(xr[i] * inv * (offset + w[i]));
}

// The same for rows of up to 8192 elements with hidden % 4 == 0: a thread keeps its NV groups of
// four elements in registers (one pass over the row, 16-byte loads all issued at once).
template <typename TY, int NV>
__global__ void __launch_bounds__(1024)
rmsnorm_row_kernel(TY* __restrict__ y, const float* __restrict__ x, const float* __restrict__ w,
                   const int* __restrict__ rows, int hidden, float eps, float offset) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * hidden;
  float4 xv[NV], wv[NV];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (threadIdx.x + v * blockDim.x) * 4;
    xv[v] = wv[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < hidden) {
      xv[v] = *reinterpret_cast<const float4*>(xr + i);
      wv[v] = *reinterpret_cast<const float4*>(w + i);
    }
    ss += xv[v].x * xv[v].x + xv[v].y * xv[v].y + xv[v].z * xv[v].z + xv[v].w * xv[v].w;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (threadIdx.x + v * blockDim.x) * 4;
    if (i >= hidden) continue;
    TY* yr = y + (size_t)r * hidden + i;
    yr[0] = from_f32<TY>(xv[v].x * inv * (offset + wv[v].x));
    yr[1] = from_f32<TY>(xv[v].y * inv * (offset + wv[v].y));
    yr[2] = from_f32<TY>(xv[v].z * inv * (offset + wv[v].z));
    yr[3] = from_f32<TY>(xv[v].w * inv * (offset + wv[v].w));
  }
}

AF_EXPORT int af_rmsnorm(void* y, int y_dtype, const float* x, const float* w, const int* rows,
                         int n_rows, int hidden, float eps, float offset, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && hidden > 0, "af_rmsnorm: bad sizes");
  if (hidden % 4 == 0 && hidden <= 8192 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0) {
    const int nv = hidden > 4096 ? 2 : 1;
    const int threads = ((hidden / (4 * nv) + 31) / 32) * 32;
    if (nv == 2) {
      AF_DISPATCH_DTYPE(y_dtype, TY,
                        af_launch(rmsnorm_row_kernel<TY, 2>, dim3(n_rows), dim3(threads), 0, stream, (TY*)y, x, w,
                                  rows, hidden, eps, offset));
    } else {
      AF_DISPATCH_DTYPE(y_dtype, TY,
                        af_launch(rmsnorm_row_kernel<TY, 1>, dim3(n_rows), dim3(threads), 0, stream, (TY*)y, x, w,
                                  rows, hidden, eps, offset));
    }
    AF_CHECK_LAUNCH("af_rmsnorm");
  }
  AF_DISPATCH_DTYPE(y_dtype, TY,
                    af_launch(rmsnorm_kernel<TY>, dim3(n_rows), dim3(256), 0, stream, (TY*)y, x, w, rows, hidden, eps,
                                                                  offset));
  AF_CHECK_LAUNCH("af_rmsnorm");
}

// x += norm(a) * (offset + w_post); then, when y is given,
// y = norm(x) * (offset + w_next).  `a` may come as `n_parts` partial sums
// (float, [n_parts, rows, hidden]) that are added in index order first.
template <typename TA, typename TY>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TA* __restrict__ a, int n_parts,
                                   size_t part_stride, const float* __restrict__ w_post,
                                   TY* __restrict__ y, const float* __restrict__ w_next, int hidden,
                                   float eps_post, float eps_next, float offset) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];  // hidden floats: a, then the new x
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const TA* ar = a + (size_t)r * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f32(ar[i]);
    for (int p = 1; p < n_parts; ++p) v += to_f32(ar[(size_t)p * part_stride + i]);
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps_post);
  float* xr = x + (size_t)r * hidden;
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = xr[i] + row[i] * inv * (offset + w_post[i]);
    xr[i] = v;
    row[i] = v;
    ss2 += v * v;
  }
  if (y == nullptr) return;
  ss2 = block_sum(ss2, scratch);
  const float inv2 = rsqrtf(ss2 / (float)hidden + eps_next);
  TY* yr = y + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    yr[i] = from_f32<TY>(row[i] * inv2 * (offset + w_next[i]));
}

// The same for rows of up to 8192 elements with hidden % 4 == 0: a thread owns NV groups of four
// elements (group v of thread t at element 4 (t + v * threads)), every load issued before the first
// reduction.  Few rows (decode): NV = 1, many threads per row, what costs is the chain of memory
// latencies; many rows (prefill): NV = 2, smaller blocks, more rows in flight on an SM.
// MANY (the rows of a prompt): the kernel is bound by how many rows an SM holds at a time, so it keeps to 32
// registers (seven blocks of a 2304-wide row per SM instead of four) and reads the norms' weights, which
// every row shares and the L1 holds, where it uses them instead of keeping them from the start.
template <typename TA, typename TY, int NV, bool MANY = false>
__global__ void __launch_bounds__(MANY ? 512 : 1024, MANY ? 4 : 1)
add_rmsnorm_row_kernel(float* __restrict__ x, const TA* __restrict__ a, int n_parts, size_t part_stride,
                       const float* __restrict__ w_post, TY* __restrict__ y, const float* __restrict__ w_next,
                       int hidden, float eps_post, float eps_next, float offset) {
  pdl_launch_dependents();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  float av[NV][4], xv[NV][4], wp[NV][4], wn[NV][4];
  bool on[NV];
  // the norms' weights do not depend on the kernel in front (and are cold: the step's other
  // weights have pushed them out of L2): they are asked for before the wait
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (threadIdx.x + v * blockDim.x) * 4;
    on[v] = i < hidden;
#pragma unroll
    for (int u = 0; u < 4; ++u) av[v][u] = xv[v][u] = wp[v][u] = wn[v][u] = 0.f;
    if (!on[v] || MANY) continue;
    const float4 pt = *reinterpret_cast<const float4*>(w_post + i);
    wp[v][0] = pt.x, wp[v][1] = pt.y, wp[v][2] = pt.z, wp[v][3] = pt.w;
    if (y != nullptr) {
      const float4 nt = *reinterpret_cast<const float4*>(w_next + i);
      wn[v][0] = nt.x, wn[v][1] = nt.y, wn[v][2] = nt.z, wn[v][3] = nt.w;
    }
  }
  pdl_wait();
  a = pdl_fresh(a);
  x = pdl_fresh(x);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (threadIdx.x + v * blockDim.x) * 4;
    if (!on[v]) continue;
    const size_t at = (size_t)r * hidden + i;
    if constexpr (sizeof(TA) == 4) {
      const float* ap = reinterpret_cast<const float*>(a) + at;
      for (int p0 = 0; p0 < n_parts; p0 += 8) {
        float4 t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          t[u] = p0 + u < n_parts ? *reinterpret_cast<const float4*>(ap + (size_t)(p0 + u) * part_stride)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          av[v][0] += t[u].x;
          av[v][1] += t[u].y;
          av[v][2] += t[u].z;
          av[v][3] += t[u].w;
        }
      }
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(a + at);
      av[v][0] = __uint_as_float(raw.x << 16);
      av[v][1] = __uint_as_float(raw.x & 0xffff0000u);
      av[v][2] = __uint_as_float(raw.y << 16);
      av[v][3] = __uint_as_float(raw.y & 0xffff0000u);
    }
    const float4 xt = *reinterpret_cast<const float4*>(x + at);
    xv[v][0] = xt.x, xv[v][1] = xt.y, xv[v][2] = xt.z, xv[v][3] = xt.w;
  }
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) ss += av[v][0] * av[v][0] + av[v][1] * av[v][1] + av[v][2] * av[v][2] + av[v][3] * av[v][3];
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps_post);
  float ss2 = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    if (MANY && on[v]) {
      const float4 pt = *reinterpret_cast<const float4*>(w_post + (threadIdx.x + v * blockDim.x) * 4);
      wp[v][0] = pt.x, wp[v][1] = pt.y, wp[v][2] = pt.z, wp[v][3] = pt.w;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      xv[v][u] = xv[v][u] + av[v][u] * inv * (offset + wp[v][u]);
      ss2 += on[v] ? xv[v][u] * xv[v][u] : 0.f;
    }
    if (on[v])
      *reinterpret_cast<float4*>(x + (size_t)r * hidden + (threadIdx.x + v * blockDim.x) * 4) =
          make_float4(xv[v][0], xv[v][1], xv[v][2], xv[v][3]);
  }
  if (y == nullptr) return;
  ss2 = block_sum(ss2, scratch);
  const float inv2 = rsqrtf(ss2 / (float)hidden + eps_next);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    if (!on[v]) continue;
    if (MANY) {
      const float4 nt = *reinterpret_cast<const float4*>(w_next + (threadIdx.x + v * blockDim.x) * 4);
      wn[v][0] = nt.x, wn[v][1] = nt.y, wn[v][2] = nt.z, wn[v][3] = nt.w;
    }
    TY* yr = y + (size_t)r * hidden + (threadIdx.x + v * blockDim.x) * 4;
    if constexpr (sizeof(TY) == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(xv[v][0] * inv2 * (offset + wn[v][0]), xv[v][1] * inv2 * (offset + wn[v][1]));
      __nv_bfloat162 hi = __floats2bfloat162_rn(xv[v][2] * inv2 * (offset + wn[v][2]), xv[v][3] * inv2 * (offset + wn[v][3]));
      *reinterpret_cast<uint2*>(yr) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else {
#pragma unroll
      for (int u = 0; u < 4; ++u) yr[u] = from_f32<TY>(xv[v][u] * inv2 * (offset + wn[v][u]));
    }
  }
}

AF_EXPORT int af_add_rmsnorm(float* x, const void* a, int a_dtype, int n_parts, long long part_stride,
                             const float* w_post, void* y, int y_dtype, const float* w_next,
                             int n_rows, int hidden, float eps_post, float eps_next, float offset,
                             cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && hidden > 0 && n_parts >= 1, "af_add_rmsnorm: bad sizes");
  AF_REQUIRE(hidden * sizeof(float) <= 160 * 1024, "af_add_rmsnorm: hidden %d too wide", hidden);
  AF_REQUIRE(n_parts == 1 || a_dtype == AF_F32, "af_add_rmsnorm: partial sums must be float");
  const bool aligned = (((uintptr_t)x | (uintptr_t)a | (uintptr_t)w_post | (uintptr_t)w_next) & 15) == 0 &&
                       (part_stride % 4 == 0);
  if (hidden % 4 == 0 && hidden <= 8192 && aligned && ((uintptr_t)y & 7) == 0) {
    const int nv = (n_rows >= 256 && hidden >= 1024) || hidden > 4096 ? 2 : 1;
    const int threads = ((hidden / (4 * nv) + 31) / 32) * 32;
#define LAUNCH_ROW(TA, TY)                                                                                  \
  do {                                                                                                      \
    if (nv == 2 && n_rows >= 256 && threads <= 512)                                                         \
      af_launch(add_rmsnorm_row_kernel<TA, TY, 2, true>, dim3(n_rows), dim3(threads), 0, stream, x, (const TA*)a, \
                n_parts, (size_t)part_stride, w_post, (TY*)y, w_next, hidden, eps_post, eps_next, offset);  \
    else if (nv == 2)                                                                                       \
      af_launch(add_rmsnorm_row_kernel<TA, TY, 2>, dim3(n_rows), dim3(threads), 0, stream, x, (const TA*)a, \
                n_parts, (size_t)part_stride, w_post, (TY*)y, w_next, hidden, eps_post, eps_next, offset);  \
    else                                                                                                    \
      af_launch(add_rmsnorm_row_kernel<TA, TY, 1>, dim3(n_rows), dim3(threads), 0, stream, x, (const TA*)a, \
                n_parts, (size_t)part_stride, w_post, (TY*)y, w_next, hidden, eps_post, eps_next, offset);  \
  } while (0)
    AF_DISPATCH_DTYPE(a_dtype, TA, AF_DISPATCH_DTYPE(y_dtype, TY, LAUNCH_ROW(TA, TY)));
#undef LAUNCH_ROW
    AF_CHECK_LAUNCH("af_add_rmsnorm");
  }
  const size_t smem = (size_t)hidden * sizeof(float);
#define LAUNCH(TA, TY)                                                                          \
  do {                                                                                          \
    if (smem > 48 * 1024)                                                                       \
      cudaFuncSetAttribute(add_rmsnorm_kernel<TA, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                          \
    af_launch(add_rmsnorm_kernel<TA, TY>, dim3(n_rows), dim3(256), smem, stream,                                   \
        x, (const TA*)a, n_parts, (size_t)part_stride, w_post, (TY*)y, w_next, hidden, eps_post, \
        eps_next, offset);                                                                      \
  } while (0)
  AF_DISPATCH_DTYPE(a_dtype, TA, AF_DISPATCH_DTYPE(y_dtype, TY, LAUNCH(TA, TY)));
#undef LAUNCH
  AF_CHECK_LAUNCH("af_add_rmsnorm");
}

// ---------------------------------------------------------------- gated activation

__device__ __forceinline__ float act_f32(float g, int act) {
  if (act == AF_ACT_GELU_TANH) {
    const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.f + tanhf(u));
  }
  return g / (1.f + expf(-g));
}

// out[m, i] = act(gu[m, i]) * gu[m, inter + i]
template <typename T>
__global__ void gated_act_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int m = blockIdx.x;
  const T* g = gu + (size_t)m * 2 * inter;
  const T* u = g + inter;
  T* o = out + (size_t)m * inter;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x)
    o[i] = from_f32<T>(act_f32(to_f32(g[i]), act) * to_f32(u[i]));
}

AF_EXPORT int af_gated_act(void* out, const void* gu, int dtype, int n_rows, int inter, int act,
                           cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && inter > 0, "af_gated_act: bad sizes");
  AF_REQUIRE(act == AF_ACT_GELU_TANH || act == AF_ACT_SILU, "af_gated_act: unknown activation %d", act);
  dim3 grid(n_rows, (inter + 255) / 256 < 64 ? (inter + 255) / 256 : 64);
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(gated_act_kernel<T>, dim3(grid), dim3(256), 0, stream, (T*)out, (const T*)gu, inter, act));
  AF_CHECK_LAUNCH("af_gated_act");
}

// ---------------------------------------------------------------- residual sum

template <typename T>
__global__ void add_kernel(float* __restrict__ x, const T* __restrict__ a, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    x[i] += to_f32(a[i]);
}

AF_EXPORT int af_add(float* x, const void* a, int a_dtype, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  const int sms = af_sm_count();
  if (sms <= 0) return -1;
  long long blocks = (n + 255) / 256;
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  AF_DISPATCH_DTYPE(a_dtype, T, af_launch(add_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, x, (const T*)a, (size_t)n));
  AF_CHECK_LAUNCH("af_add");
}

// ---------------------------------------------------------------- softcap

__global__ void softcap_kernel(float* __restrict__ z, size_t n, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    z[i] = softcap_f32(z[i], cap);
}

AF_EXPORT int af_softcap(float* z, long long n, float cap, cudaStream_t stream) {
  if (n == 0 || cap <= 0.f) return 0;
  const int sms = af_sm_count();
  if (sms <= 0) return -1;
  long long blocks = (n + 255) / 256;
  if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
  af_launch(softcap_kernel, dim3((int)blocks), dim3(256), 0, stream, z, (size_t)n, cap);
  AF_CHECK_LAUNCH("af_softcap");
}
