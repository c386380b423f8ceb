// Decode attention over the paged bfloat16 cache, split over the keys so that
// a step of few sequences still fills the GPU (it is bound by the bytes of K
// and V it reads; every byte is read once).
//
// The sequences of a batch may differ much in length: a sequence's keys are cut into as many splits
// (up to the grid's) as give every block about the same number of pages; blocks beyond a sequence's
// splits leave at once.
// Pass 1, grid (sequence, kv head, split): a block of two groups of 4 warps
// walks its share of the sequence's cache pages, the groups taking alternate
// pages (one warp per scheduler cannot hide the latency of its own chain of
// shared-memory loads and mma).  One thread brings the K and V tiles of a page
// in by TMA (128-byte swizzled boxes, mbarrier-tracked) through a ring of
// shared-memory stages.  The query heads of the kv group are the rows of an
// m16n8k16 tile (mma.sync, 32-bit accumulators): Q K^T, online softmax in
// registers (32-bit max, sum, output), P V.  Each warp takes 16 of a page's 64
// keys; all warps are merged through shared memory and leave (max, sum,
// output) in scratch memory.  Waits on the copies are bounded in time.
// Pass 2, grid (sequence, head): merges the splits and writes bfloat16.
//
// The cache rows of earlier tokens do not depend on the kernels before this
// one in the stream, nor do slots, lengths and page table (they are step
// inputs), so a block starts its first page copies before it waits for its
// predecessor; only the page that holds the new token waits.
//
// Scores are 32-bit; softcap uses tanh.approx and the softmax ex2.approx, which
// is what the bfloat16 path allows; the 32-bit path uses the plain kernel.
#include <mutex>

#include "airframe_b200.h"
#include "tma.cuh"

namespace {

constexpr int DA_GROUPS = 2;    // warp groups of a block; a group of four warps works on one page at a time
constexpr int DA_THREADS = DA_GROUPS * 128;
constexpr int DA_WARPS = DA_THREADS / 32;
constexpr int DA_SCH = 2;  // chains of score accumulators

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
  int n_splits;    // at most this many splits of a sequence's keys (the stride of the partial results)
  int batch, n_sms;
  float* part_o;   // [batch, nq, splits, HD]
  float* part_ml;  // [batch, nq, splits, 2]
  int* err;        // set to 1 when a bounded wait ran out
  __nv_bfloat16* out;  // [batch, nq * HD], rows out_stride apart
  long long out_stride;
};

__device__ __forceinline__ void da_ldm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void da_ldm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void da_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t da_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Pages of the cache that sequence b's new token attends to: [first, last].
__device__ __forceinline__ int da_pages(const int* slots, const int* lens, int b, int window, int* first_pp, int* last_pp) {
  const int len = slots[b] >= 0 ? lens[b] : 0;
  if (len <= 0) {
    *first_pp = 0;
    *last_pp = -1;
    return 0;
  }
  const int pos = len - 1;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  *first_pp = lo / AF_PAGE;
  *last_pp = pos / AF_PAGE;
  return *last_pp - *first_pp + 1;
}

// Into how many splits sequence b's pages are cut (1..max_splits).  The sequences of a batch may differ
// much in length: every block gets about the same number of pages, total pages / (SMs per row of the
// grid), so a long sequence among short ones is cut into many splits and the short ones into one,
// instead of the same number for all.  (The split and the merge kernel compute it alike.)
__device__ __forceinline__ int da_splits_of(int total, int mine, int rows_of_grid, int n_sms, int max_splits) {
  const int blocks = max(1, n_sms / max(1, rows_of_grid));       // blocks there are for one kv head of all sequences
  const int target = max(1, (total + blocks - 1) / blocks);      // pages a block should get
  return max(1, min(max_splits, (mine + target / 2) / target));
}
// The pages of all sequences of the batch, summed by the block's first warp into *total_s (shared memory);
// the caller synchronises the block before it reads it.
__device__ __forceinline__ void da_total_pages(const int* slots, const int* lens, int batch, int window, int* total_s) {
  if (threadIdx.x < 32) {
    int t = 0, f, l;
    for (int i = threadIdx.x; i < batch; i += 32) t += da_pages(slots, lens, i, window, &f, &l);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) *total_s = t;
  }
}

template <int HD>
__host__ __device__ constexpr int da_stages() { return HD >= 256 ? 3 : 4; }

// Address of the 16-byte piece `c` (of HD / 8) of key row `r` in a page tile:
// HD / 64 sub-tiles of [64 rows][128 bytes], each swizzled as TMA writes it.
__device__ __forceinline__ uint32_t da_piece(uint32_t tile, int r, int c) {
  return tile + (uint32_t)((c >> 3) * 8192 + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

// The heads of one kv group are the (up to 16) rows of an m16n8k16 tile; the
// four warps of a block share each page's 64 keys, 16 keys a warp.
template <int HD>
__global__ void __launch_bounds__(DA_THREADS, 1)
attn_decode_split_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         DecodeArgs a) {
  constexpr int KSTEPS = HD / 16;
  constexpr int ONT = HD / 8;
  constexpr int STAGES = da_stages<HD>();
  constexpr int SCH = DA_SCH;
  constexpr uint32_t TILE_BYTES = AF_PAGE * HD * 2;
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ unsigned char da_smem_raw[];
  unsigned char* da_smem = (unsigned char*)(((uintptr_t)da_smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ float m_s[DA_WARPS * 16], l_s[DA_WARPS * 16];
  // a barrier per page modulo 2 * STAGES: the two groups run ahead of one another, and a page and the
  // page STAGES later (the other group's, in the same stage) must not share a barrier's phases
  constexpr int NBAR = 2 * STAGES;
  __shared__ uint64_t full[NBAR];
  __shared__ int give_up_s, total_pages_s;
  volatile int* give_up = &give_up_s;

  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int group = a.nq / a.nkv;
  const int tiles = (group + 15) / 16;
  const int kvh = blockIdx.y / tiles;
  const int row_head0 = kvh * group + (blockIdx.y % tiles) * 16;        // head of tile row 0
  const int n_rows = min(16, kvh * group + group - row_head0);           // heads in this tile
  const int z = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = warp >> 2, wq = warp & 3;   // warp group; this warp's quarter of a page's keys
  const int g = lane >> 2, t = lane & 3;
  if (tid == 0) {
    for (int s = 0; s < NBAR; ++s) mbar_init(&full[s], 1);
    give_up_s = 0;
    mbar_fence_init();
  }
  const int slot = a.slots[b];
  const int len = slot >= 0 ? a.lens[b] : 0;
  const int pos = len - 1;
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;

  int pp_begin = 0, pp_end = 0, first_pp, last_pp;  // last_pp: the page of the new token, which the kernel before wrote
  const int my_pages = da_pages(a.slots, a.lens, b, a.window, &first_pp, &last_pp);
  int splits = 1;
  if (a.n_splits > 1) {
    da_total_pages(a.slots, a.lens, a.batch, a.window, &total_pages_s);
    __syncthreads();
    splits = da_splits_of(total_pages_s, my_pages, gridDim.y, a.n_sms, a.n_splits);
  }
  if (z >= splits) return;                          // (nothing of the block's is in flight yet)
  if (len > 0) {
    const int n_pp = last_pp - first_pp + 1;
    const int per = (n_pp + splits - 1) / splits;
    pp_begin = first_pp + z * per;
    pp_end = min(pp_begin + per, last_pp + 1);
  }
  const int n_pages = max(pp_end - pp_begin, 0);
  const int ring_pages = a.ring_rows / AF_PAGE;
  const int* pt = a.page_table + (size_t)max(slot, 0) * a.max_pages;
  __syncthreads();

  auto issue = [&](int i) {  // page i of this block's share into stage i % STAGES
    const int pp = pp_begin + i;
    const int entry = ring_pages > 0 ? pp % ring_pages : pp;
    int page = AF_INDEX_OK(entry < a.max_pages, entry) ? pt[entry] : 0;
    if (!AF_INDEX_OK(page >= 0, page)) page = 0;     // (the copy must still be made: the stage's barrier expects its bytes)
    const int row = (page * a.nkv + kvh) * AF_PAGE;
    unsigned char* st = da_smem + (size_t)(i % STAGES) * 2 * TILE_BYTES;
    uint64_t* bar = &full[i % NBAR];
    mbar_expect_tx(bar, 2 * TILE_BYTES);
#pragma unroll
    for (int c = 0; c < HD / 64; ++c) {
      tma_load_2d(st + c * 8192, &map_k, c * 64, row, bar);
      tma_load_2d(st + TILE_BYTES + c * 8192, &map_v, c * 64, row, bar);
    }
  };
  int issued = 0;
  if (tid == 0)
    for (; issued < STAGES && issued < n_pages && pp_begin + issued != last_pp; ++issued) issue(issued);
  pdl_wait();
  if (tid == 0)
    for (; issued < STAGES && issued < n_pages; ++issued) issue(issued);

  // the query heads as A fragments: rows g and g + 8 of the tile
  uint32_t qf[KSTEPS][4];
  {
    const __nv_bfloat16* q0 = a.q + (size_t)b * a.q_stride + (size_t)(row_head0 + g) * HD;
    const __nv_bfloat16* q1 = q0 + (size_t)8 * HD;
    const bool on0 = len > 0 && g < n_rows, on1 = len > 0 && g + 8 < n_rows;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int d = ks * 16 + 2 * t;
      qf[ks][0] = on0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
      qf[ks][1] = on1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
      qf[ks][2] = on0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
      qf[ks][3] = on1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
    }
  }
  float o[ONT][4];
#pragma unroll
  for (int n = 0; n < ONT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f};
  const float cs = a.cap > 0.f ? a.scale / a.cap : a.scale * LOG2E;
  const float cap2 = a.cap * LOG2E;
  for (int i = grp; i < n_pages; i += DA_GROUPS) {
    const int s = i % STAGES;
    const int ok = mbar_wait(&full[i % NBAR], (i / NBAR) & 1, give_up) ? 1 : 0;
    // the four warps of the group go on or give up together
    int all_ok;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "barrier.red.and.pred.aligned p, %2, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(all_ok)
        : "r"(ok), "r"(1 + grp)
        : "memory");
    if (!all_ok) break;
    const uint32_t k_t = smem_u32(da_smem + (size_t)s * 2 * TILE_BYTES);
    const uint32_t v_t = k_t + TILE_BYTES;
    // ---- S = Q K^T for this warp's 16 keys
    // (SCH chains of accumulators: an mma waits for the one before it on the same accumulator)
    float scp[SCH][2][4];
#pragma unroll
    for (int c = 0; c < SCH; ++c)
#pragma unroll
      for (int n = 0; n < 2; ++n) scp[c][n][0] = scp[c][n][1] = scp[c][n][2] = scp[c][n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t b0, b1, b2, b3;
      da_ldm4(da_piece(k_t, wq * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
      da_mma(scp[ks % SCH][0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
      da_mma(scp[ks % SCH][1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
    }
    float sc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = scp[0][n][e];
#pragma unroll
        for (int c = 1; c < SCH; ++c) v += scp[c][n][e];
        sc[n][e] = v;
      }
    // ---- scale, softcap, mask, online softmax (base 2)
    const int j0 = (pp_begin + i) * AF_PAGE + wq * 16;
    float new_max[2] = {mx[0], mx[1]};
    // (the test on the cap stands outside the loops: inside it stays a branch per score)
    if (a.cap > 0.f) {
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[n][e] = cap2 * fast_tanh(sc[n][e] * cs);
    } else {
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[n][e] *= cs;
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + n * 8 + 2 * t + (e & 1);
        const float v = (j >= lo && j <= pos) ? sc[n][e] : -INFINITY;
        sc[n][e] = v;
        new_max[e >> 1] = fmaxf(new_max[e >> 1], v);
      }
    }
    float corr[2], ref[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      new_max[r] = fmaxf(new_max[r], __shfl_xor_sync(0xffffffffu, new_max[r], 1));
      new_max[r] = fmaxf(new_max[r], __shfl_xor_sync(0xffffffffu, new_max[r], 2));
      ref[r] = new_max[r] == -INFINITY ? 0.f : new_max[r];
      corr[r] = fast_exp2(mx[r] - ref[r]);
      mx[r] = new_max[r];
      sum[r] *= corr[r];
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = fast_exp2(sc[n][e] - ref[e >> 1]);
        sc[n][e] = p;
        sum[e >> 1] += p;
      }
    }
    if (corr[0] != 1.f || corr[1] != 1.f) {
#pragma unroll
      for (int n = 0; n < ONT; ++n) {
        o[n][0] *= corr[0];
        o[n][1] *= corr[0];
        o[n][2] *= corr[1];
        o[n][3] *= corr[1];
      }
    }
    // ---- O += P V over this warp's 16 keys
    {
      const uint32_t a0 = da_pack(sc[0][0], sc[0][1]), a1 = da_pack(sc[0][2], sc[0][3]);
      const uint32_t a2 = da_pack(sc[1][0], sc[1][1]), a3 = da_pack(sc[1][2], sc[1][3]);
#pragma unroll
      for (int np = 0; np < ONT / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        da_ldm4t(da_piece(v_t, wq * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, np * 2 + (lane >> 4)), b0, b1, b2, b3);
        da_mma(o[2 * np], a0, a1, a2, a3, b0, b1);
        da_mma(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // the group is done with stage s (a barrier of its own four warps): its first thread refills it
    asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
    if ((tid & 127) == 0 && i + STAGES < n_pages && !*give_up) issue(i + STAGES);
  }
  if (*give_up && tid == 0) grace_period();
  __syncthreads();

  // ---- merge the four warps (each saw a quarter of the keys); the stage memory is the buffer
  float* o_s = reinterpret_cast<float*>(da_smem);  // [warp][rows of real heads][HD]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
    const int row = g + 8 * r;
    if (t == 0) {
      m_s[warp * 16 + row] = mx[r];
      l_s[warp * 16 + row] = sum[r];
    }
    if (row < n_rows) {
#pragma unroll
      for (int n = 0; n < ONT; ++n) {
        float* dst = o_s + ((size_t)(warp * n_rows + row)) * HD + n * 8 + 2 * t;
        dst[0] = o[n][2 * r];
        dst[1] = o[n][2 * r + 1];
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < n_rows * HD; i += DA_THREADS) {
    const int row = i / HD, d = i - row * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DA_WARPS; ++w) M = fmaxf(M, m_s[w * 16 + row]);
    const float ref = M == -INFINITY ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < DA_WARPS; ++w) {
      const float f = fast_exp2(m_s[w * 16 + row] - ref);
      L += l_s[w * 16 + row] * f;
      O += o_s[((size_t)(w * n_rows + row)) * HD + d] * f;
    }
    const size_t pidx = ((size_t)b * a.nq + row_head0 + row) * a.n_splits + z;
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
                                         int nq, int max_splits, const int* __restrict__ slots,
                                         const int* __restrict__ lens, int window, int rows_of_grid, int n_sms) {
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.y;
  const size_t p0 = ((size_t)b * nq + h) * max_splits;
  // (slots and lengths are inputs of the step: the number of splits is worked out before the wait)
  __shared__ int total_pages_s;
  int first_pp, last_pp, n_splits = 1;
  if (max_splits > 1) {
    const int my_pages = da_pages(slots, lens, b, window, &first_pp, &last_pp);
    da_total_pages(slots, lens, gridDim.x, window, &total_pages_s);
    __syncthreads();
    n_splits = da_splits_of(total_pages_s, my_pages, rows_of_grid, n_sms, max_splits);
  }
  pdl_wait();
  // (the number of splits is known before the wait and the loads below depend on nothing else: without
  // this the compiler may move them, through the const __restrict__ pointers, above the wait)
  part_o = pdl_fresh(part_o);
  part_ml = pdl_fresh(part_ml);
  constexpr int FEW = 8;
  const int d = threadIdx.x;   // HD >= 128: threads 0..127 take d and d + 128 (HD 256)
  if (n_splits <= FEW) {
    // few splits: every load (outputs, maxima, sums) is issued before the first use, one round trip
    constexpr int PER = HD > 128 ? HD / 128 : 1;
    float o[FEW][PER], m[FEW], l[FEW];
#pragma unroll
    for (int s = 0; s < FEW; ++s) {
      const bool on = s < n_splits;
      m[s] = on ? part_ml[(p0 + s) * 2] : -INFINITY;
      l[s] = on ? part_ml[(p0 + s) * 2 + 1] : 0.f;
#pragma unroll
      for (int e = 0; e < PER; ++e) o[s][e] = on && d + e * 128 < HD ? part_o[(p0 + s) * HD + d + e * 128] : 0.f;
    }
    float M = -INFINITY;
#pragma unroll
    for (int s = 0; s < FEW; ++s) M = fmaxf(M, m[s]);
    const float ref = M == -INFINITY ? 0.f : M;
    float L = 0.f, O[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) O[e] = 0.f;
#pragma unroll
    for (int s = 0; s < FEW; ++s) {
      const float f = fast_exp2(m[s] - ref);
      L += l[s] * f;
#pragma unroll
      for (int e = 0; e < PER; ++e) O[e] += o[s][e] * f;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int e = 0; e < PER; ++e)
      if (d + e * 128 < HD) out[(size_t)b * out_stride + (size_t)h * HD + d + e * 128] = __float2bfloat16_rn(O[e] * inv);
    return;
  }
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(p0 + s) * 2]);
  const float ref = M == -INFINITY ? 0.f : M;
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) L += part_ml[(p0 + s) * 2 + 1] * fast_exp2(part_ml[(p0 + s) * 2] - ref);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int dd = threadIdx.x; dd < HD; dd += blockDim.x) {
    float O = 0.f;
    for (int s = 0; s < n_splits; ++s) O += part_o[(p0 + s) * HD + dd] * fast_exp2(part_ml[(p0 + s) * 2] - ref);
    out[(size_t)b * out_stride + (size_t)h * HD + dd] = __float2bfloat16_rn(O * inv);
  }
}

template <int HD>
int launch_decode(DecodeArgs a, int batch, long long n_pages, cudaStream_t stream) {
  const size_t stage_bytes = (size_t)da_stages<HD>() * 2 * AF_PAGE * HD * 2;
  const size_t merge_bytes = (size_t)DA_WARPS * 16 * HD * sizeof(float);
  const size_t smem = (stage_bytes > merge_bytes ? stage_bytes : merge_bytes) + 1024;
  // (the limit on dynamic shared memory is a device's: set once on each)
  static bool configured[AF_MAX_DEVICES] = {};
  const int dev__ = af_current_device();
  if (dev__ < 0) return -1;
  if (!configured[dev__]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_split_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return af_fail((int)e, "af_attn_decode: %s", cudaGetErrorString(e));
    configured[dev__] = true;
  }
  // the cache of one layer as a matrix [pages * kv heads * 64 rows, HD]; boxes of 64 rows x 64 columns
  CUtensorMap mk, mv;
  int rc = af_make_map_bf16(&mk, a.kcache, n_pages * a.nkv * AF_PAGE, HD, HD, AF_PAGE);
  if (rc) return rc;
  rc = af_make_map_bf16(&mv, a.vcache, n_pages * a.nkv * AF_PAGE, HD, HD, AF_PAGE);
  if (rc) return rc;
  const int group = a.nq / a.nkv;
  dim3 grid(batch, a.nkv * ((group + 15) / 16), a.n_splits);
  af_launch(attn_decode_split_kernel<HD>, grid, dim3(DA_THREADS), smem, stream, mk, mv, a);
  AF_COUNT_LAUNCH("af_attn_decode (split)");
  af_launch(attn_decode_merge_kernel<HD>, dim3(batch, a.nq), dim3(HD < 128 ? HD : 128), 0, stream, a.out,
            a.out_stride, (const float*)a.part_o, (const float*)a.part_ml, a.nq, a.n_splits, a.slots, a.lens, a.window,
            (int)grid.y, a.n_sms);
  AF_CHECK_LAUNCH("af_attn_decode (merge)");
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
// The cache of the layer holds n_pages pages [kv heads][64][hd].  scratch:
// af_attn_decode_scratch(...) floats.  Sequences with slot < 0 give zeros.  n_splits: the most splits
// of a sequence's keys (the third extent of the grid).
AF_EXPORT int af_attn_decode(void* out, long long out_stride, const void* q, long long q_stride,
                             const void* kcache, const void* vcache, long long n_pages, const int* page_table,
                             int max_pages, const int* slots, const int* lens, int batch, int nq, int nkv, int hd,
                             float scale, float cap, int window, int ring_rows, int n_splits, float* scratch,
                             int* err, cudaStream_t stream) {
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
  a.batch = batch;
  a.n_sms = af_sm_count();
  if (a.n_sms <= 0) return -1;
  a.part_o = scratch;
  a.part_ml = scratch + (size_t)batch * nq * n_splits * hd;
  a.err = err;
  a.out = (__nv_bfloat16*)out;
  a.out_stride = out_stride;
  AF_REQUIRE(n_pages > 0 && n_pages * nkv * AF_PAGE < (1ll << 31), "af_attn_decode: %lld cache pages", n_pages);
  if (hd == 64) return launch_decode<64>(a, batch, n_pages, stream);
  if (hd == 128) return launch_decode<128>(a, batch, n_pages, stream);
  return launch_decode<256>(a, batch, n_pages, stream);
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
                                    const void* kcache, const void* vcache, long long n_pages,
                                    const int* page_table, int max_pages, const int* slots, const int* lens,
                                    int batch, int nq, int nkv, int hd, float scale, float cap, int window,
                                    int ring_rows, int n_splits, int* err, cudaStream_t stream) {
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
  return af_attn_decode(out, out_stride, q, q_stride, kcache, vcache, n_pages, page_table, max_pages, slots, lens,
                        batch, nq, nkv, hd, scale, cap, window, ring_rows, n_splits, scratch, err, stream);
}
