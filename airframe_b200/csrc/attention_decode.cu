// Decode attention over the paged bfloat16 cache, split over the keys so that
// a step of few sequences still fills the GPU (it is bound by the bytes of K
// and V it reads; every byte is read once).
//
// Pass 1, grid (sequence, kv head x head tile, split): a block of 256 threads
// walks its share of the sequence's cache pages.  A page of one kv head is
// contiguous, so one thread brings K and V pages in with bulk copies
// (cp.async.bulk, mbarrier-tracked) through a ring of shared-memory stages.
// Eight lanes own one key: each holds head_dim / 8 elements of the K row, dots
// them with GT query heads of the group, reduces over the eight lanes, and
// keeps an online softmax (32-bit max, sum, output) per head.  The 32 key
// groups of a block are merged through shared memory and leave (max, sum,
// output) in scratch memory.  Waits on the copies are bounded in time.
// Pass 2, grid (sequence, head): merges the splits and writes bfloat16.
//
// Scores are 32-bit; softcap uses tanh.approx and the softmax ex2.approx, which
// is what the bfloat16 path allows; the 32-bit path uses the plain kernel.
#include <mutex>

#include "airframe_b200.h"
#include "common.cuh"

namespace {

constexpr int DA_THREADS = 256;
constexpr int DA_KEY_GROUPS = DA_THREADS / 8;

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// E bfloat16 values (E even) from p into f[]: 16-byte loads when E % 8 == 0, else 4-byte loads.
template <int E>
__device__ __forceinline__ void load_bf16(const __nv_bfloat16* p, float* f) {
  if constexpr (E % 8 == 0) {
#pragma unroll
    for (int i = 0; i < E / 8; ++i) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p + 8 * i);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
        f[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < E / 2; ++i) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(p + 2 * i);
      f[2 * i] = __uint_as_float(w << 16);
      f[2 * i + 1] = __uint_as_float(w & 0xffff0000u);
    }
  }
}

struct DecodeArgs {
  const __nv_bfloat16* q;
  long long q_stride;
  const __nv_bfloat16* kcache;
  const __nv_bfloat16* vcache;
  const int* page_table;
  int max_pages;
  const int* slots;
  const int* lens;
  int nq, nkv;
  float scale, cap;
  int window, ring_rows;
  int n_splits;
  float* part_o;   // [batch, nq, splits, HD]
  float* part_ml;  // [batch, nq, splits, 2]
  int* err;        // set to 1 when a bounded wait ran out
};

__device__ __forceinline__ uint32_t da_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long da_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool da_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(da_smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when two seconds pass or another thread gave up.
__device__ __forceinline__ bool da_wait(uint64_t* bar, uint32_t parity, volatile int* give_up) {
  if (da_try_wait(bar, parity)) return true;
  const unsigned long long t0 = da_now_ns();
  for (;;) {
    if (da_try_wait(bar, parity)) return true;
    if (*give_up) return false;
    if (da_now_ns() - t0 > 2000000000ull) {
      *give_up = 1;
      return false;
    }
  }
}
// One page of one kv head is contiguous in the cache: a single bulk copy brings it in.
__device__ __forceinline__ void da_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(da_smem_u32(dst)), "l"(src), "r"(bytes), "r"(da_smem_u32(bar))
               : "memory");
}

template <int HD>
__host__ __device__ constexpr int da_stages() { return HD >= 256 ? 3 : 4; }

// 8 bfloat16 (one 16-byte piece) -> floats
__device__ __forceinline__ void da_unpack8(const uint4& raw, float* f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(w[j] << 16);
    f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}

template <int HD, int GT>
__global__ void __launch_bounds__(DA_THREADS, 1)
attn_decode_split_kernel(DecodeArgs a) {
  // A row of HD elements is HD / 8 pieces of 16 bytes; lane `sub` of a key's 8
  // lanes owns the pieces sub, sub + 8, ...: the 8 lanes read 128 contiguous bytes.
  constexpr int U = HD / 64;               // pieces per lane
  constexpr int E = U * 8;                 // elements per lane
  constexpr int STAGES = da_stages<HD>();
  constexpr uint32_t PAGE_BYTES = AF_PAGE * HD * 2;
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ __align__(128) unsigned char da_smem[];  // STAGES x (K page, V page); later the merge buffer
  __shared__ __align__(16) float q_s[GT * HD];               // [h][u][half][sub][4]
  __shared__ float m_s[DA_KEY_GROUPS * GT], l_s[DA_KEY_GROUPS * GT];
  __shared__ uint64_t full[STAGES];
  __shared__ int give_up_s;
  volatile int* give_up = &give_up_s;

  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const int group = a.nq / a.nkv;
  const int tiles = group / GT;
  const int kvh = blockIdx.y / tiles;
  const int head0 = kvh * group + (blockIdx.y % tiles) * GT;
  const int z = blockIdx.z;
  const int tid = threadIdx.x, kg = tid >> 3, sub = tid & 7;
  const int slot = a.slots[b];
  const int len = slot >= 0 ? a.lens[b] : 0;
  const int pos = len - 1;
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;

  int pp_begin = 0, pp_end = 0;
  if (len > 0) {
    const int first_pp = lo / AF_PAGE, last_pp = pos / AF_PAGE;
    const int n_pp = last_pp - first_pp + 1;
    const int per = (n_pp + a.n_splits - 1) / a.n_splits;
    pp_begin = first_pp + z * per;
    pp_end = min(pp_begin + per, last_pp + 1);
  }
  const int n_pages = max(pp_end - pp_begin, 0);
  const int ring_pages = a.ring_rows / AF_PAGE;
  const int* pt = a.page_table + (size_t)max(slot, 0) * a.max_pages;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(da_smem_u32(&full[s])), "r"(1));
    give_up_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < GT * HD; i += DA_THREADS) {
    const int h = i / HD, d = i - h * HD;
    const int c = d >> 3, w = d & 7;
    const int idx = (((h * U + (c >> 3)) * 2 + (w >> 2)) * 8 + (c & 7)) * 4 + (w & 3);
    q_s[idx] = len > 0 ? __bfloat162float(a.q[(size_t)b * a.q_stride + (size_t)(head0 + h) * HD + d]) * a.scale : 0.f;
  }
  __syncthreads();

  auto issue = [&](int i) {  // page i of this block's share into stage i % STAGES
    const int pp = pp_begin + i;
    const int page = pt[ring_pages > 0 ? pp % ring_pages : pp];
    const size_t off = ((size_t)page * a.nkv + kvh) * AF_PAGE * HD;
    unsigned char* st = da_smem + (size_t)(i % STAGES) * 2 * PAGE_BYTES;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(da_smem_u32(&full[i % STAGES])),
                 "r"(2 * PAGE_BYTES)
                 : "memory");
    da_bulk_load(st, a.kcache + off, PAGE_BYTES, &full[i % STAGES]);
    da_bulk_load(st + PAGE_BYTES, a.vcache + off, PAGE_BYTES, &full[i % STAGES]);
  };
  if (tid == 0)
    for (int i = 0; i < STAGES && i < n_pages; ++i) issue(i);

  float m[GT], l[GT], o[GT][E];
#pragma unroll
  for (int h = 0; h < GT; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) o[h][e] = 0.f;
  }
  const float inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;

  int landed = 0;  // pages whose copies are known to be complete (for the exit path)
  for (int i = 0; i < n_pages; ++i) {
    const int s = i % STAGES;
    if (!da_wait(&full[s], (i / STAGES) & 1, give_up)) break;
    landed = i + 1;
    const unsigned char* kst = da_smem + (size_t)s * 2 * PAGE_BYTES;
    const unsigned char* vst = kst + PAGE_BYTES;
    const int pp = pp_begin + i;
#pragma unroll 1
    for (int jj = kg; jj < AF_PAGE; jj += DA_KEY_GROUPS) {
      const int j = pp * AF_PAGE + jj;
      const bool valid = j >= lo && j <= pos;  // uniform over the 8 lanes of a key
      float kf[E];
#pragma unroll
      for (int u = 0; u < U; ++u)
        da_unpack8(*reinterpret_cast<const uint4*>(kst + ((size_t)jj * HD + (u * 8 + sub) * 8) * 2), kf + 8 * u);
      float sc[GT];
#pragma unroll
      for (int h = 0; h < GT; ++h) {
        float dot = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float4 q0 = *reinterpret_cast<const float4*>(q_s + (((h * U + u) * 2 + 0) * 8 + sub) * 4);
          const float4 q1 = *reinterpret_cast<const float4*>(q_s + (((h * U + u) * 2 + 1) * 8 + sub) * 4);
          dot = fmaf(q0.x, kf[8 * u + 0], dot);
          dot = fmaf(q0.y, kf[8 * u + 1], dot);
          dot = fmaf(q0.z, kf[8 * u + 2], dot);
          dot = fmaf(q0.w, kf[8 * u + 3], dot);
          dot = fmaf(q1.x, kf[8 * u + 4], dot);
          dot = fmaf(q1.y, kf[8 * u + 5], dot);
          dot = fmaf(q1.z, kf[8 * u + 6], dot);
          dot = fmaf(q1.w, kf[8 * u + 7], dot);
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        const float t = a.cap > 0.f ? a.cap * fast_tanh(dot * inv_cap) : dot;
        sc[h] = valid ? t * LOG2E : -INFINITY;  // softmax in base 2
      }
      float vf[E];
#pragma unroll
      for (int u = 0; u < U; ++u)
        da_unpack8(*reinterpret_cast<const uint4*>(vst + ((size_t)jj * HD + (u * 8 + sub) * 8) * 2), vf + 8 * u);
#pragma unroll
      for (int h = 0; h < GT; ++h) {
        const float m_new = fmaxf(m[h], sc[h]);
        const float ref = m_new == -INFINITY ? 0.f : m_new;
        const float corr = fast_exp2(m[h] - ref);
        const float p = fast_exp2(sc[h] - ref);
        l[h] = l[h] * corr + p;
#pragma unroll
        for (int e = 0; e < E; ++e) o[h][e] = fmaf(p, vf[e], o[h][e] * corr);
        m[h] = m_new;
      }
    }
    __syncthreads();  // everyone is done with stage s
    if (tid == 0 && i + STAGES < n_pages && !*give_up) issue(i + STAGES);
  }
  if (*give_up) {
    // copies that were issued must land before the stage memory is reused below
    if (tid == 0) {
      const unsigned long long t0 = da_now_ns();
      while (da_now_ns() - t0 < 1000000ull) {
      }
    }
    (void)landed;
  }
  __syncthreads();

  // merge the key groups of the block; the stage memory serves as the buffer
  float* o_s = reinterpret_cast<float*>(da_smem);  // [key group][GT][HD]
#pragma unroll
  for (int h = 0; h < GT; ++h) {
    if (sub == 0) {
      m_s[kg * GT + h] = m[h];
      l_s[kg * GT + h] = l[h];
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int w = 0; w < 8; ++w) o_s[((size_t)kg * GT + h) * HD + (u * 8 + sub) * 8 + w] = o[h][8 * u + w];
  }
  __syncthreads();
  for (int i = tid; i < GT * HD; i += DA_THREADS) {
    const int h = i / HD, d = i - h * HD;
    float M = -INFINITY;
#pragma unroll
    for (int g = 0; g < DA_KEY_GROUPS; ++g) M = fmaxf(M, m_s[g * GT + h]);
    const float ref = M == -INFINITY ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll 8
    for (int g = 0; g < DA_KEY_GROUPS; ++g) {
      const float w = fast_exp2(m_s[g * GT + h] - ref);
      L += l_s[g * GT + h] * w;
      O += o_s[((size_t)g * GT + h) * HD + d] * w;
    }
    const size_t pidx = ((size_t)b * a.nq + head0 + h) * a.n_splits + z;
    a.part_o[pidx * HD + d] = O;
    if (d == 0) {
      a.part_ml[pidx * 2] = M;
      a.part_ml[pidx * 2 + 1] = L;
    }
  }
  if (tid == 0 && give_up_s && a.err) atomicExch(a.err, 1);
}

template <int HD>
__global__ void attn_decode_merge_kernel(__nv_bfloat16* __restrict__ out, long long out_stride,
                                         const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         int nq, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const size_t p0 = ((size_t)b * nq + h) * n_splits;
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(p0 + s) * 2]);
  const float ref = M == -INFINITY ? 0.f : M;
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) L += part_ml[(p0 + s) * 2 + 1] * fast_exp2(part_ml[(p0 + s) * 2] - ref);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float O = 0.f;
    for (int s = 0; s < n_splits; ++s) O += part_o[(p0 + s) * HD + d] * fast_exp2(part_ml[(p0 + s) * 2] - ref);
    out[(size_t)b * out_stride + (size_t)h * HD + d] = __float2bfloat16_rn(O * inv);
  }
}

template <int HD, int GT>
int launch_decode(const DecodeArgs& a, __nv_bfloat16* out, long long out_stride, int batch, cudaStream_t stream) {
  const size_t stage_bytes = (size_t)da_stages<HD>() * 2 * AF_PAGE * HD * 2;
  const size_t merge_bytes = (size_t)DA_KEY_GROUPS * GT * HD * sizeof(float);
  const size_t smem = stage_bytes > merge_bytes ? stage_bytes : merge_bytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_split_kernel<HD, GT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return af_fail((int)e, "af_attn_decode: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int group = a.nq / a.nkv;
  dim3 grid(batch, a.nkv * (group / GT), a.n_splits);
  af_launch(attn_decode_split_kernel<HD, GT>, dim3(grid), dim3(DA_THREADS), smem, stream, a);
  AF_COUNT_LAUNCH("af_attn_decode (split)");
  af_launch(attn_decode_merge_kernel<HD>, dim3(dim3(batch, a.nq)), dim3(HD < 128 ? HD : 128), 0, stream, 
      out, out_stride, a.part_o, a.part_ml, a.nq, a.n_splits);
  AF_CHECK_LAUNCH("af_attn_decode (merge)");
}

template <int HD>
int launch_decode_hd(const DecodeArgs& a, __nv_bfloat16* out, long long out_stride, int batch, cudaStream_t s) {
  // the widest head tile that divides the group and keeps the output in registers
  constexpr int LIMIT = 512 / HD;  // 2 heads of 256, 4 of 128, 8 of 64
  const int group = a.nq / a.nkv;
  if (LIMIT >= 8 && group % 8 == 0) return launch_decode<HD, (LIMIT >= 8 ? 8 : 1)>(a, out, out_stride, batch, s);
  if (LIMIT >= 4 && group % 4 == 0) return launch_decode<HD, (LIMIT >= 4 ? 4 : 1)>(a, out, out_stride, batch, s);
  if (LIMIT >= 2 && group % 2 == 0) return launch_decode<HD, (LIMIT >= 2 ? 2 : 1)>(a, out, out_stride, batch, s);
  return launch_decode<HD, 1>(a, out, out_stride, batch, s);
}

}  // namespace

// 1 when the split kernel takes this head size (else the plain kernel serves).
AF_EXPORT int af_attn_decode_supported(int hd) { return hd == 64 || hd == 128 || hd == 256 ? 1 : 0; }

// Floats of scratch memory that af_attn_decode needs: outputs, then (max, sum).
AF_EXPORT long long af_attn_decode_scratch(int batch, int nq, int hd, int n_splits) {
  return (long long)batch * nq * n_splits * (hd + 2);
}

// out [batch, nq * hd] bfloat16 = attention of one new token per sequence over
// its cache (lens[b] counts the new token, which the cache holds already).
// scratch: af_attn_decode_scratch(...) floats.  Sequences with slot < 0 give zeros.
AF_EXPORT int af_attn_decode(void* out, long long out_stride, const void* q, long long q_stride,
                             const void* kcache, const void* vcache, const int* page_table, int max_pages,
                             const int* slots, const int* lens, int batch, int nq, int nkv, int hd, float scale,
                             float cap, int window, int ring_rows, int n_splits, float* scratch, int* err,
                             cudaStream_t stream) {
  if (batch == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "af_attn_decode: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(af_attn_decode_supported(hd), "af_attn_decode: head_dim %d (takes 64, 128, 256)", hd);
  AF_REQUIRE(ring_rows % AF_PAGE == 0 && (ring_rows == 0 || (window > 0 && window <= ring_rows)),
             "af_attn_decode: window %d, ring rows %d", window, ring_rows);
  AF_REQUIRE(n_splits >= 1 && n_splits <= 65535 && scratch != nullptr, "af_attn_decode: splits %d", n_splits);
  AF_REQUIRE(((uintptr_t)kcache & 15) == 0 && ((uintptr_t)vcache & 15) == 0, "af_attn_decode: cache alignment");
  DecodeArgs a;
  a.q = (const __nv_bfloat16*)q;
  a.q_stride = q_stride;
  a.kcache = (const __nv_bfloat16*)kcache;
  a.vcache = (const __nv_bfloat16*)vcache;
  a.page_table = page_table;
  a.max_pages = max_pages;
  a.slots = slots;
  a.lens = lens;
  a.nq = nq;
  a.nkv = nkv;
  a.scale = scale;
  a.cap = cap;
  a.window = window;
  a.ring_rows = ring_rows;
  a.n_splits = n_splits;
  a.part_o = scratch;
  a.part_ml = scratch + (size_t)batch * nq * n_splits * hd;
  a.err = err;
  __nv_bfloat16* o = (__nv_bfloat16*)out;
  if (hd == 64) return launch_decode_hd<64>(a, o, out_stride, batch, stream);
  if (hd == 128) return launch_decode_hd<128>(a, o, out_stride, batch, stream);
  return launch_decode_hd<256>(a, o, out_stride, batch, stream);
}

// ---------------------------------------------------------------- no allocation

// Scratch of af_attn_decode_static: the split pass's partial results.  It lives
// in the library image, so every GPU that loads the library holds these 4 MiB
// until the process exits.
static __device__ __align__(256) float g_decode_scratch[AF_ATTN_DECODE_STATIC_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// The array's address on the current device.  In host code the array's name
// stands for a host-side shadow, not for device memory, so the address comes
// from cudaGetSymbolAddress, once per device, with that device current.
int decode_scratch_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return af_fail((int)e, "af_attn_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return af_fail(-1, "af_attn_decode_static: device ordinal %d beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr)
      return af_fail(e != cudaSuccess ? (int)e : -1, "af_attn_decode_static: cudaGetSymbolAddress: %s",
                     cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}
}  // namespace

AF_EXPORT long long af_attn_decode_static_capacity() { return AF_ATTN_DECODE_STATIC_FLOATS; }

AF_EXPORT int af_attn_decode_static(void* out, long long out_stride, const void* q, long long q_stride,
                                    const void* kcache, const void* vcache, const int* page_table, int max_pages,
                                    const int* slots, const int* lens, int batch, int nq, int nkv, int hd,
                                    float scale, float cap, int window, int ring_rows, int n_splits, int* err,
                                    cudaStream_t stream) {
  if (batch == 0) return 0;
  AF_REQUIRE(batch > 0 && nq > 0 && hd > 0 && n_splits >= 1, "af_attn_decode_static: bad sizes");
  const long long need = af_attn_decode_scratch(batch, nq, hd, n_splits);
  AF_REQUIRE(need <= AF_ATTN_DECODE_STATIC_FLOATS,
             "af_attn_decode_static: batch %d x heads %d x splits %d x (head_dim %d + 2) = %lld floats of scratch, "
             "the built-in array holds %d; use fewer splits or af_attn_decode with scratch of your own",
             batch, nq, n_splits, hd, need, AF_ATTN_DECODE_STATIC_FLOATS);
  float* scratch = nullptr;
  const int rc = decode_scratch_address(&scratch);
  if (rc) return rc;
  return af_attn_decode(out, out_stride, q, q_stride, kcache, vcache, page_table, max_pages, slots, lens, batch, nq,
                        nkv, hd, scale, cap, window, ring_rows, n_splits, scratch, err, stream);
}
