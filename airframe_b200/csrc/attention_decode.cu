// Decode attention over the paged bfloat16 cache, split over the keys so that
// a step of few sequences still fills the GPU (it is bound by the bytes of K
// and V it reads; every byte is read once).
//
// How the work is cut.  The grid is one block an SM.  A unit is a (sequence, kv head) pair (a tile of 16
// heads of it, if the group is larger) with the cache pages its sequence's new token attends to; the pages
// of all units, divided by the blocks, are a block's share.  The cut follows from the lengths alone
// (da_plan); a small kernel works it out once a step for all layers that read their caches alike and leaves
// every block what it begins with (af_attn_decode_plan), or, without such a plan, every block works it out:
//  * the even cut: every unit into about pages / share splits of equal size, one split a block.  No block
//    meets the end of a unit; taken when the splits are no more than the blocks and none is more than two
//    pages above the share (sequences of equal or of mixed lengths, one long one among short ones);
//  * else the run cut: all units' pages end to end, each block an equal run of them.  A run may end one unit
//    and begin the next: the block works them as segments, one after the other, and leaves a partial result
//    for each (many short sequences; more units than blocks).
// Pass 1: a block of two groups of 4 warps
// walks its pages, the groups taking alternate
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
  const int* plan; // the step's plan (attn_decode_plan_kernel), or null: every block works the cut out itself
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
  const int slot = slots[b], len_b = lens[b];   // (both loads at once: neither waits for the other)
  const int len = slot >= 0 ? len_b : 0;
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

template <int HD>
__host__ __device__ constexpr int da_stages() { return HD >= 256 ? 3 : 4; }

// Address of the 16-byte piece `c` (of HD / 8) of key row `r` in a page tile:
// HD / 64 sub-tiles of [64 rows][128 bytes], each swizzled as TMA writes it.
__device__ __forceinline__ uint32_t da_piece(uint32_t tile, int r, int c) {
  return tile + (uint32_t)((c >> 3) * 8192 + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}


// ---------------------------------------------------------------- how the work is cut

constexpr int DA_MAX_BATCH = 2048;   // sequences whose page counts a block keeps in shared memory

// The blocks that share the work in the run cut.  A unit of P pages lies in at most P + 1 runs and in at most
// n_blocks / units_per_seq + 2 (a run is at least total / n_blocks pages, and the unit's sequence alone has
// units_per_seq * P): if the room for partial results, `room` a unit, is below both, fewer blocks work, so that
// no unit is cut more often than it has room for.
__device__ __forceinline__ int da_blocks_used(int n_blocks, int room, int units_per_seq, int most_pages) {
  if (room >= most_pages + 1 || room >= n_blocks / units_per_seq + 2) return n_blocks;
  return max(1, min(n_blocks, (room - 2) * units_per_seq));
}

// Splits of a unit of P pages in the even cut: pages / share, rounded to the nearest (how 1) or down (how 2).
__device__ __forceinline__ int da_even_splits(int P, int share, int room, int how) {
  return P > 0 ? max(1, min(room, (P + (how == 1 ? share / 2 : 0)) / share)) : 0;
}

// What a block loses at the end of a unit inside its run (merging, the next unit's queries, the first page's
// wait), in pages: the even cut is taken if its largest split is no more than this above the share.
constexpr int DA_BREAK_PAGES = 2;

struct DaPlan {
  int share;        // pages a block should get
  int n_blocks;     // blocks that work in the run cut
  int even;         // 0: the run cut; else the even cut, and how it rounds (da_even_splits)
  int pages_before; // pages of the sequences before `b_query` (each counted once, not per unit)
};

// The plan, by one whole warp (every lane returns the same).  32-bit arithmetic all through: the launcher has
// checked that batch x pages x units stays below 2^31.  If `pages_s` is given it gets the pages of the sequences
// before b, and `splits_s` their splits in the even cut (b = 0 .. batch).
__device__ __forceinline__ DaPlan da_plan(const int* slots, const int* lens, int batch, int window, int units_per_seq,
                                          int grid_blocks, int room, int b_query, int* pages_s, int* splits_s) {
  const int lane = threadIdx.x & 31;
  int carry = 0, most = 0, before = 0, f, l, P_first = 0;
  if (pages_s && lane == 0) pages_s[0] = 0;
  for (int base = 0; base < batch; base += 32) {
    const int i = base + lane;
    const int P = i < batch ? da_pages(slots, lens, i, window, &f, &l) : 0;
    if (base == 0) P_first = P;
    most = max(most, P);
    if (i < b_query) before += P;
    int v = P;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += up;
    }
    if (pages_s && i < batch) pages_s[i + 1] = carry + v;
    carry += __shfl_sync(0xffffffffu, v, 31);
  }
  most = __reduce_max_sync(0xffffffffu, most);
  DaPlan pl;
  pl.pages_before = __reduce_add_sync(0xffffffffu, before);
  const int total = carry * units_per_seq;
  pl.n_blocks = da_blocks_used(grid_blocks, room, units_per_seq, most);
  pl.share = max(1, (total + pl.n_blocks - 1) / pl.n_blocks);
  // the even cut, rounding either way: how many splits in all, and the most pages of one
  int items1 = 0, worst1 = 0, items2 = 0, worst2 = 0;
  for (int base = 0; base < batch; base += 32) {
    const int i = base + lane;
    const int P = base == 0 ? P_first : (i < batch ? da_pages(slots, lens, i, window, &f, &l) : 0);
    const int sp1 = da_even_splits(P, pl.share, room, 1), sp2 = da_even_splits(P, pl.share, room, 2);
    if (P > 0) {
      worst1 = max(worst1, (P + sp1 - 1) / sp1);
      worst2 = max(worst2, (P + sp2 - 1) / sp2);
    }
    items1 += sp1;
    items2 += sp2;
  }
  items1 = __reduce_add_sync(0xffffffffu, items1);
  items2 = __reduce_add_sync(0xffffffffu, items2);
  worst1 = __reduce_max_sync(0xffffffffu, worst1);
  worst2 = __reduce_max_sync(0xffffffffu, worst2);
  const bool fits1 = items1 * units_per_seq <= grid_blocks, fits2 = items2 * units_per_seq <= grid_blocks;
  int how = 0, worst = 0;
  if (fits1 && (!fits2 || worst1 <= worst2)) how = 1, worst = worst1;
  else if (fits2) how = 2, worst = worst2;
  pl.even = (how != 0 && worst <= pl.share + DA_BREAK_PAGES) ? how : 0;
  if (splits_s && pl.even) {
    int items = 0;
    if (lane == 0) splits_s[0] = 0;
    for (int base = 0; base < batch; base += 32) {
      const int i = base + lane;
      const int P = base == 0 ? P_first : (i < batch ? da_pages(slots, lens, i, window, &f, &l) : 0);
      int v = da_even_splits(P, pl.share, room, pl.even);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += up;
      }
      if (i < batch) splits_s[i + 1] = items + v;
      items += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  return pl;
}

// The largest b in [0, n) with arr[b] * scale <= x (arr ascends, arr[0] = 0).
__device__ __forceinline__ int da_find(const int* arr, int n, int scale, int x) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (arr[mid] * scale <= x) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// What block w begins with: pages [p_in, p_in + n_pages) of unit y of sequence b, the unit's split z; run_pages is
// all the block works (in the run cut it goes on with the units that follow).  n_pages < 0: the block has no work.
struct DaFirst {
  int n_pages, b, y, z, p_in, run_pages;
};

__device__ __forceinline__ DaFirst da_first_segment(const DaPlan& pl, const int* pages_s, const int* splits_s, int batch,
                                                    int units_per_seq, int w) {
  DaFirst fs;
  fs.n_pages = -1;
  fs.b = fs.y = fs.z = fs.p_in = fs.run_pages = 0;
  if (pl.even) {
    // split z of unit y of sequence b, one of da_even_splits(...) equal parts of its pages
    if (w >= splits_s[batch] * units_per_seq) return fs;
    const int b = da_find(splits_s, batch, units_per_seq, w);
    const int sp = splits_s[b + 1] - splits_s[b], P = pages_s[b + 1] - pages_s[b];
    const int r = w - splits_s[b] * units_per_seq;
    const int per = (P + sp - 1) / sp;
    fs.b = b;
    fs.y = r / sp;
    fs.z = r - fs.y * sp;
    fs.p_in = fs.z * per;
    fs.n_pages = max(0, min(per, P - fs.p_in));   // (0: the unit has fewer pages than splits; an empty partial result)
    fs.run_pages = fs.n_pages;
    return fs;
  }
  // the run cut: pages [gpos, gend) of all units' pages end to end
  const int total = pages_s[batch] * units_per_seq;
  const int gpos = w * pl.share, gend = min(total, gpos + pl.share);
  if (w >= pl.n_blocks || gpos >= gend) return fs;
  const int b = da_find(pages_s, batch, units_per_seq, gpos);
  const int P = pages_s[b + 1] - pages_s[b];
  const int seq0 = pages_s[b] * units_per_seq;
  fs.b = b;
  fs.y = (gpos - seq0) / P;
  fs.p_in = (gpos - seq0) - fs.y * P;
  fs.run_pages = gend - gpos;
  fs.n_pages = min(P - fs.p_in, fs.run_pages);
  fs.z = w - (seq0 + fs.y * P) / pl.share;   // (the run may begin inside a unit: then it is not the unit's first split)
  return fs;
}

// ---------------------------------------------------------------- the plan of a step
//
// The cut depends on the step's lengths alone, so the layers that read the same caches the same way (one group of
// layers) can share it: a small kernel works it out once, and each layer's blocks read their first segment from
// it with one load, where otherwise each block loads slots and lengths, works out the cut and loads page ids,
// one after the other, before its first copy can start.  The plan, 32-bit integers:
//   [0, 8)                    room (splits a unit may have), grid blocks, sequences, units a sequence, how cut
//   [8, 8 + sequences*units)  the splits of every unit, for the merge
//   then 16 a block           n_pages (< 0: no work), b, y, z, p_in, run_pages, position of the new token, slot,
//                             the cache pages of the segment's first four pages
constexpr int DA_PLAN_HEAD = 8;
constexpr int DA_PLAN_REC = 16;

__host__ __device__ inline long long da_plan_records_at(int batch, int units_per_seq) {
  return DA_PLAN_HEAD + (((long long)batch * units_per_seq + 3) / 4) * 4;
}

// One block.  It does not release its dependents early: the kernel behind it starts when the plan is complete, and
// so does every kernel after that one, so all of them may read the plan before they wait for anything.
__global__ void __launch_bounds__(256)
attn_decode_plan_kernel(int* __restrict__ plan, const int* __restrict__ slots, const int* __restrict__ lens,
                        const int* __restrict__ page_table, int max_pages, int batch, int nq, int nkv, int window,
                        int ring_rows, int room, int grid_blocks) {
  extern __shared__ int dp_smem[];
  int* pages_s = dp_smem;                 // [batch + 1]
  int* splits_s = dp_smem + batch + 1;    // [batch + 1]
  __shared__ DaPlan plan_s;
  pdl_wait();
  const int group = nq / nkv, tiles = (group + 15) / 16, units_per_seq = nkv * tiles;
  if (threadIdx.x < 32) {
    const DaPlan pl = da_plan(slots, lens, batch, window, units_per_seq, grid_blocks, room, 0, pages_s, splits_s);
    if (threadIdx.x == 0) plan_s = pl;
  }
  __syncthreads();
  const DaPlan pl = plan_s;
  if (threadIdx.x == 0) {
    plan[0] = room;
    plan[1] = grid_blocks;
    plan[2] = batch;
    plan[3] = units_per_seq;
    plan[4] = pl.even;
    plan[5] = pl.share;
    plan[6] = pl.n_blocks;
    plan[7] = 0;
  }
  for (int u = threadIdx.x; u < batch * units_per_seq; u += blockDim.x) {
    const int b = u / units_per_seq, y = u - b * units_per_seq;
    const int P = pages_s[b + 1] - pages_s[b];
    int n = 0;
    if (pl.even) {
      n = da_even_splits(P, pl.share, room, pl.even);
    } else if (P > 0) {
      const int unit0 = pages_s[b] * units_per_seq + y * P;
      n = (unit0 + P - 1) / pl.share - unit0 / pl.share + 1;
    }
    plan[DA_PLAN_HEAD + u] = n;
  }
  int* recs = plan + da_plan_records_at(batch, units_per_seq);
  const int ring_pages = ring_rows / AF_PAGE;
  for (int w = threadIdx.x; w < grid_blocks; w += blockDim.x) {
    const DaFirst fs = da_first_segment(pl, pages_s, splits_s, batch, units_per_seq, w);
    int* r = recs + (size_t)w * DA_PLAN_REC;
    int pos = 0, slot = 0, ids[4] = {0, 0, 0, 0};
    if (fs.n_pages >= 0) {
      pos = lens[fs.b] - 1;
      slot = slots[fs.b];
      const int lo = window > 0 ? max(0, pos - window + 1) : 0;
      for (int i = 0; i < 4 && i < fs.n_pages; ++i) {
        const int pp = lo / AF_PAGE + fs.p_in + i;
        const int entry = ring_pages > 0 ? pp % ring_pages : pp;
        int page = AF_INDEX_OK(entry < max_pages, entry) ? page_table[(size_t)slot * max_pages + entry] : 0;
        if (!AF_INDEX_OK(page >= 0, page)) page = 0;
        ids[i] = page;
      }
    }
    reinterpret_cast<int4*>(r)[0] = make_int4(fs.n_pages, fs.b, fs.y, fs.z);
    reinterpret_cast<int4*>(r)[1] = make_int4(fs.p_in, fs.run_pages, pos, slot);
    reinterpret_cast<int4*>(r)[2] = make_int4(ids[0], ids[1], ids[2], ids[3]);
    reinterpret_cast<int4*>(r)[3] = make_int4(0, 0, 0, 0);
  }
}

// The heads of one kv group are the (up to 16) rows of an m16n8k16 tile; the
// four warps of a group share each page's 64 keys, 16 keys a warp.
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
  // a stage's two uses in a row (a page and the page STAGES later, the other group's) must not share a
  // barrier's phases
  constexpr int NBAR = 2 * STAGES;
  __shared__ uint64_t full[NBAR];
  __shared__ int give_up_s;
  __shared__ int pages_s[DA_MAX_BATCH + 1], splits_s[DA_MAX_BATCH + 1];
  __shared__ DaPlan plan_s;
  volatile int* give_up = &give_up_s;

  pdl_launch_dependents();
  const int group = a.nq / a.nkv;
  const int tiles = (group + 15) / 16;
  const int units_per_seq = a.nkv * tiles;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = warp >> 2, wq = warp & 3;   // warp group; this warp's quarter of a page's keys
  const int g = lane >> 2, t = lane & 3;
  if (tid == 0) {
    for (int s = 0; s < NBAR; ++s) mbar_init(&full[s], 1);
    give_up_s = 0;
    mbar_fence_init();
  }
  // What the block begins with: from the step's plan with one load, or worked out here (slots and lengths are
  // inputs of the step, not results of the kernel in front).
  DaFirst fs;
  int pos0 = 0, slot0 = 0, ids0[4] = {0, 0, 0, 0};
  if (a.plan != nullptr) {
    const int4* rec = reinterpret_cast<const int4*>(a.plan + da_plan_records_at(a.batch, units_per_seq)) +
                      (size_t)blockIdx.x * (DA_PLAN_REC / 4);
    const uint64_t keep = l2_policy_keep();   // (every layer of the group reads the plan: it should stay in L2)
    const int4 head = ld_keep_int4(reinterpret_cast<const int4*>(a.plan), keep);
    const int4 r0 = ld_keep_int4(rec, keep), r1 = ld_keep_int4(rec + 1, keep), r2 = ld_keep_int4(rec + 2, keep);
    fs.n_pages = r0.x, fs.b = r0.y, fs.y = r0.z, fs.z = r0.w;
    fs.p_in = r1.x, fs.run_pages = r1.y, pos0 = r1.z, slot0 = r1.w;
    ids0[0] = r2.x, ids0[1] = r2.y, ids0[2] = r2.z, ids0[3] = r2.w;
    if (head.x != a.n_splits || head.y != (int)gridDim.x || head.z != a.batch || head.w != units_per_seq) {
      // (a plan made for another launch: nothing is read or written by it)
      if (tid == 0 && a.err) atomicExch(a.err, 1);
      return;
    }
    __syncthreads();     // (the barriers are set up)
  } else {
    if (warp == 0) {
      const DaPlan pl = da_plan(a.slots, a.lens, a.batch, a.window, units_per_seq, (int)gridDim.x, a.n_splits, 0,
                                pages_s, splits_s);
      if (lane == 0) plan_s = pl;
    }
    __syncthreads();
    fs = da_first_segment(plan_s, pages_s, splits_s, a.batch, units_per_seq, (int)blockIdx.x);
    if (fs.n_pages >= 0) {
      pos0 = a.lens[fs.b] - 1;
      slot0 = a.slots[fs.b];
    }
  }
  if (fs.n_pages < 0) return;                          // (nothing of the block's is in flight yet)
  int left = fs.run_pages;                             // pages the block has still to work
  const int ring_pages = a.ring_rows / AF_PAGE;
  const float cs = a.cap > 0.f ? a.scale / a.cap : a.scale * LOG2E;
  const float cap2 = a.cap * LOG2E;

  // A segment: some of the pages of one unit.
  struct Segment {
    int b, y, kvh, row_head0, n_rows, z, n_pages, pp_begin, last_pp, lo, pos;
    const int* pt;
  };
  auto of_unit = [&](Segment& sg, int b, int y, int p_in, int pos, int slot) {
    sg.b = b;
    sg.y = y;
    sg.kvh = y / tiles;
    sg.row_head0 = sg.kvh * group + (y % tiles) * 16;             // head of tile row 0
    sg.n_rows = min(16, sg.kvh * group + group - sg.row_head0);    // heads in this tile
    sg.pos = pos;
    sg.lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    sg.last_pp = pos / AF_PAGE;        // the page of the new token, which the kernel in front wrote
    sg.pp_begin = sg.lo / AF_PAGE + p_in;
    sg.pt = a.page_table + (size_t)slot * a.max_pages;
  };
  // the run cut goes on with the unit behind sg's: the same sequence's next, or the first of the next sequence
  // that has pages (one there is: pages are left)
  auto next_unit = [&](const Segment& sg) {
    Segment nx;
    int b = sg.b, y = sg.y + 1;
    if (y >= units_per_seq) {
      y = 0;
      int f, l;
      do ++b; while (b < a.batch - 1 && da_pages(a.slots, a.lens, b, a.window, &f, &l) == 0);
    }
    int f, l;
    const int P = da_pages(a.slots, a.lens, b, a.window, &f, &l);
    nx.z = 0;
    nx.n_pages = min(P, left);
    of_unit(nx, b, y, 0, a.lens[b] - 1, a.slots[b]);
    return nx;
  };
  // the cache page that holds page i of segment sg (a load from the page table: asked for ahead of its use)
  auto page_id = [&](const Segment& sg, int i) {
    const int pp = sg.pp_begin + i;
    const int entry = ring_pages > 0 ? pp % ring_pages : pp;
    int page = AF_INDEX_OK(entry < a.max_pages, entry) ? sg.pt[entry] : 0;
    if (!AF_INDEX_OK(page >= 0, page)) page = 0;   // (the copy must still be made: the stage's barrier expects its bytes)
    return page;
  };
  const uint64_t read_once = l2_policy_read_once();   // (a step reads every cache page once)
  // cache page `page` of kv head kvh, the block's page number ii, into stage ii % STAGES
  auto issue = [&](int kvh, int page, int ii) {
    const int row = (page * a.nkv + kvh) * AF_PAGE;
    unsigned char* st = da_smem + (size_t)(ii % STAGES) * 2 * TILE_BYTES;
    uint64_t* bar = &full[ii % NBAR];
    mbar_expect_tx(bar, 2 * TILE_BYTES);
#pragma unroll
    for (int c = 0; c < HD / 64; ++c) {
      tma_load_2d_once(st + c * 8192, &map_k, c * 64, row, bar, read_once);
      tma_load_2d_once(st + TILE_BYTES + c * 8192, &map_v, c * 64, row, bar, read_once);
    }
  };
  // the first pages of a segment: their page ids are loaded together, then the copies go out
  auto issue_first = [&](const Segment& sg, int from, int to, int ii0, bool skip_last) {
    int ids[STAGES];
#pragma unroll
    for (int i = 0; i < STAGES; ++i) ids[i] = (i >= from && i < to) ? page_id(sg, i) : 0;
    int i = from;
#pragma unroll
    for (int k = 0; k < STAGES; ++k)
      if (k == i && k < to && !(skip_last && sg.pp_begin + k == sg.last_pp)) {
        issue(sg.kvh, ids[k], ii0 + k);
        ++i;
      }
    return i;
  };

  int i_base = 0;          // pages this block has worked before the segment: barriers and stages count on
  Segment sg;
  sg.z = fs.z;
  sg.n_pages = fs.n_pages;
  of_unit(sg, fs.b, fs.y, fs.p_in, pos0, slot0);
  int issued = 0;          // pages of the segment that are on their way already
  // the cache rows of earlier tokens do not depend on the kernel in front: the first pages are on their way
  // before the wait for it; only the page that holds the new token waits
  if (tid == 0) {
    if (a.plan != nullptr) {
      // (the plan holds the first pages' ids: no load from the page table stands before the copies)
#pragma unroll
      for (int k = 0; k < STAGES; ++k)
        if (k == issued && k < sg.n_pages && sg.pp_begin + k != sg.last_pp) {
          issue(sg.kvh, ids0[k], k);
          ++issued;
        }
    } else {
      issued = issue_first(sg, 0, min(STAGES, sg.n_pages), 0, true);
    }
  }
  pdl_wait();
  while (true) {
    const int b = sg.b, n_pages = sg.n_pages, n_rows = sg.n_rows, row_head0 = sg.row_head0, z = sg.z;
    const int pp_begin = sg.pp_begin, lo = sg.lo, pos = sg.pos;
    if (tid == 0) issued = issue_first(sg, issued, min(STAGES, n_pages), i_base, false);

    // the query heads as A fragments: rows g and g + 8 of the tile
    uint32_t qf[KSTEPS][4];
    {
      const __nv_bfloat16* q0 = a.q + (size_t)b * a.q_stride + (size_t)(row_head0 + g) * HD;
      const __nv_bfloat16* q1 = q0 + (size_t)8 * HD;
      const bool on0 = g < n_rows, on1 = g + 8 < n_rows;
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
    // group `grp` takes the pages whose count since the block began is grp modulo 2
    for (int i = (grp - i_base) & 1; i < n_pages; i += DA_GROUPS) {
      const int ii = i_base + i;
      const int s = ii % STAGES;
      // (the group's first thread refills the stage when the group is done with it: the page's id is asked for now)
      const bool refill = (tid & 127) == 0 && i + STAGES < n_pages;
      const int refill_page = refill ? page_id(sg, i + STAGES) : 0;
      const int ok = mbar_wait(&full[ii % NBAR], (ii / NBAR) & 1, give_up) ? 1 : 0;
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
      // the group is done with the stage (a barrier of its own four warps): its first thread refills it
      asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
      if (refill && !*give_up) issue(sg.kvh, refill_page, ii + STAGES);
    }
    if (*give_up && tid == 0) grace_period();
    __syncthreads();
    const bool gave_up = *give_up != 0;      // (the same for all threads: nobody waits on a barrier any more)

    // ---- merge the eight warps (each saw a part of the keys); a stage is the buffer.  Where the buffer fits one
    // stage (up to 8 heads in the tile), the next segment's first pages go into the other stages before the
    // merge, so that the block's stream of pages does not stop at a unit's end.
    i_base += n_pages;
    left -= n_pages;
    const bool more = left > 0 && !gave_up;          // (the even cut: one segment)
    Segment nx = sg;
    issued = 0;
    if (more) {
      nx = next_unit(sg);
      if (tid == 0 && n_rows <= 8) issued = issue_first(nx, 0, min(STAGES - 1, nx.n_pages), i_base, false);
      // the next unit's queries: asked into L1 now, read when the merge is done
      if (tid < nx.n_rows * (HD / 64))
        asm volatile("prefetch.global.L1 [%0];" ::"l"(a.q + (size_t)nx.b * a.q_stride +
                                                       (size_t)(nx.row_head0 + tid / (HD / 64)) * HD + (tid % (HD / 64)) * 64));
    }
    // [warp][rows of real heads][HD], in the stage that the next pages reach last (thread 0 alone issues on)
    float* o_s = reinterpret_cast<float*>(da_smem + (n_rows <= 8 ? (size_t)((i_base + STAGES - 1) % STAGES) * 2 * TILE_BYTES : 0));
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
    if (!more) break;
    __syncthreads();       // (the buffer is one of the next segment's stages)
    sg = nx;
  }
  if (tid == 0 && give_up_s && a.err) atomicExch(a.err, 1);
}

// ---------------------------------------------------------------- pass 2

constexpr int DA_MERGE_FEW = 8;        // up to this many splits: 128 threads, every load at once
constexpr int DA_MERGE_THREADS = 512;  // more, and few (sequence, head) pairs: groups of threads take the splits in turn
constexpr int DA_MERGE_MOST = 512;     // splits whose (max, sum) the block keeps in shared memory

// Merges the splits of (sequence, head), cut as the split kernel cut them (da_plan with that kernel's grid).
template <int HD>
__global__ void attn_decode_merge_kernel(__nv_bfloat16* __restrict__ out, long long out_stride,
                                         const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         int nq, int nkv, int max_splits, const int* __restrict__ slots,
                                         const int* __restrict__ lens, int window, int grid_blocks,
                                         const int* __restrict__ plan) {
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.y, batch = gridDim.x;
  const size_t p0 = ((size_t)b * nq + h) * max_splits;
  __shared__ DaPlan plan_s;
  __shared__ float m_sh[DA_MERGE_MOST], l_sh[DA_MERGE_MOST];
  __shared__ float red_s[DA_MERGE_THREADS * 2];
  const int group = nq / nkv, tiles = (group + 15) / 16, units_per_seq = nkv * tiles;
  // (the plan, or slots and lengths, are inputs of the step: the cut is known before the wait)
  int n_splits;
  if (plan != nullptr) {
    n_splits = ld_keep_int(plan + DA_PLAN_HEAD + b * units_per_seq + (h / group) * tiles + (h % group) / 16, l2_policy_keep());
  } else {
    if (threadIdx.x < 32) {
      const DaPlan pl = da_plan(slots, lens, batch, window, units_per_seq, grid_blocks, max_splits, b, nullptr, nullptr);
      if (threadIdx.x == 0) plan_s = pl;
    }
    __syncthreads();
    int first_pp, last_pp;
    const int P = da_pages(slots, lens, b, window, &first_pp, &last_pp);
    if (plan_s.even) {
      n_splits = da_even_splits(P, plan_s.share, max_splits, plan_s.even);
    } else {
      const int y = (h / group) * tiles + (h % group) / 16;
      const int unit0 = plan_s.pages_before * units_per_seq + y * P;
      n_splits = P > 0 ? (unit0 + P - 1) / plan_s.share - unit0 / plan_s.share + 1 : 0;
    }
  }
  pdl_wait();
  // (the number of splits is known before the wait and the loads below depend on nothing else: without
  // this the compiler may move them, through the const __restrict__ pointers, above the wait)
  part_o = pdl_fresh(part_o);
  part_ml = pdl_fresh(part_ml);
  __nv_bfloat16* dst = out + (size_t)b * out_stride + (size_t)h * HD;
  if (n_splits <= DA_MERGE_FEW) {
    // few splits: every load (outputs, maxima, sums) is issued before the first use, one round trip
    constexpr int FEW = DA_MERGE_FEW;
    constexpr int PER = HD > 128 ? HD / 128 : 1;
    const int d = threadIdx.x;   // HD >= 128: threads 0..127 take d and d + 128 (HD 256)
    if (d >= 128 || d >= HD) return;
    float o[FEW][PER], m[FEW], l[FEW];
#pragma unroll
    for (int s = 0; s < FEW; ++s) {
      const bool on = s < n_splits;
      m[s] = on ? part_ml[(p0 + s) * 2] : -INFINITY;
      l[s] = on ? part_ml[(p0 + s) * 2 + 1] : 0.f;
#pragma unroll
      for (int e = 0; e < PER; ++e) o[s][e] = on ? part_o[(p0 + s) * HD + d + e * 128] : 0.f;
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
    for (int e = 0; e < PER; ++e) dst[d + e * 128] = __float2bfloat16_rn(O[e] * inv);
    return;
  }
  if (n_splits <= DA_MERGE_MOST && blockDim.x % (HD / 2) == 0) {
    // many splits, three round trips: (max, sum) of every split at once; the outputs, the splits dealt to
    // groups of HD / 2 threads (two dims a thread), eight loads in flight each; the groups' sums through shared memory
    const int tid = threadIdx.x;
    for (int s = tid; s < n_splits; s += (int)blockDim.x) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (p0 + s) * 2));
      m_sh[s] = ml.x;
      l_sh[s] = ml.y;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int s = tid & 31; s < n_splits; s += 32) M = fmaxf(M, m_sh[s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float ref = M == -INFINITY ? 0.f : M;
    float L = 0.f;
    for (int s = tid & 31; s < n_splits; s += 32) L += l_sh[s] * fast_exp2(m_sh[s] - ref);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    constexpr int ROW = HD / 2;                       // threads of a group
    const int GROUPS = (int)blockDim.x / ROW;         // (1 .. 16)
    const int grp = tid / ROW, dp = tid - grp * ROW;
    float2 acc = make_float2(0.f, 0.f);
    int s = grp;
    for (; s + 7 * GROUPS < n_splits; s += 8 * GROUPS) {
      float2 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcg(reinterpret_cast<const float2*>(part_o + (p0 + s + u * GROUPS) * HD) + dp);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float f = fast_exp2(m_sh[s + u * GROUPS] - ref);
        acc.x += v[u].x * f;
        acc.y += v[u].y * f;
      }
    }
    {
      float2 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = s + u * GROUPS < n_splits ? __ldcg(reinterpret_cast<const float2*>(part_o + (p0 + s + u * GROUPS) * HD) + dp)
                                         : make_float2(0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float f = s + u * GROUPS < n_splits ? fast_exp2(m_sh[s + u * GROUPS] - ref) : 0.f;
        acc.x += v[u].x * f;
        acc.y += v[u].y * f;
      }
    }
    red_s[tid * 2] = acc.x;
    red_s[tid * 2 + 1] = acc.y;
    __syncthreads();
    if (tid < ROW) {
      float2 O = make_float2(0.f, 0.f);
      for (int gq = 0; gq < GROUPS; ++gq) {
        O.x += red_s[(gq * ROW + tid) * 2];
        O.y += red_s[(gq * ROW + tid) * 2 + 1];
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      *reinterpret_cast<__nv_bfloat162*>(dst + 2 * tid) = __floats2bfloat162_rn(O.x * inv, O.y * inv);
    }
    return;
  }
  // (more splits than the block keeps: one after the other)
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(p0 + s) * 2]);
  const float ref = M == -INFINITY ? 0.f : M;
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) L += part_ml[(p0 + s) * 2 + 1] * fast_exp2(part_ml[(p0 + s) * 2] - ref);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int dd = threadIdx.x; dd < HD; dd += blockDim.x) {
    float O = 0.f;
    for (int s = 0; s < n_splits; ++s) O += part_o[(p0 + s) * HD + dd] * fast_exp2(part_ml[(p0 + s) * 2] - ref);
    dst[dd] = __float2bfloat16_rn(O * inv);
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
  const int units_per_seq = a.nkv * ((group + 15) / 16);
  // (a sequence attends to at most max_pages + 1 pages: a window's first and last page may be the same of the ring)
  AF_REQUIRE(batch <= DA_MAX_BATCH && (long long)batch * (a.max_pages + 1) * units_per_seq < (1ll << 31),
             "af_attn_decode: %d sequences of up to %d pages (takes %d sequences)", batch, a.max_pages, DA_MAX_BATCH);
  const int n_blocks = a.n_sms;   // one block an SM; the blocks work out among themselves which of them work
  af_launch(attn_decode_split_kernel<HD>, dim3(n_blocks), dim3(DA_THREADS), smem, stream, mk, mv, a);
  AF_COUNT_LAUNCH("af_attn_decode (split)");
  // The large block only where the merge's blocks are few: the split kernel's blocks fill their SMs' registers, so
  // the merge's blocks wait (their part before the wait done) on the SMs that the split kernel left idle, and
  // those hold few large blocks.  Many (sequence, head) pairs have few splits each, unless one long sequence stands
  // among short ones: then one group of threads takes its splits eight at a time.
  const int merge_threads = a.n_splits > DA_MERGE_FEW && batch * a.nq <= 32 ? DA_MERGE_THREADS : (HD < 128 ? HD : 128);
  af_launch(attn_decode_merge_kernel<HD>, dim3(batch, a.nq), dim3(merge_threads), 0, stream, a.out, a.out_stride,
            (const float*)a.part_o, (const float*)a.part_ml, a.nq, a.nkv, a.n_splits, a.slots, a.lens, a.window,
            n_blocks, a.plan);
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
                             const int* plan, int* err, cudaStream_t stream) {
  if (batch == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "af_attn_decode: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(af_attn_decode_supported(hd), "af_attn_decode: head_dim %d (takes 64, 128, 256)", hd);
  AF_REQUIRE(ring_rows % AF_PAGE == 0 && (ring_rows == 0 || (window > 0 && window <= ring_rows)),
             "af_attn_decode: window %d, ring rows %d", window, ring_rows);
  AF_REQUIRE(n_splits >= 1 && n_splits <= 65535 && scratch != nullptr, "af_attn_decode: splits %d", n_splits);
  AF_REQUIRE(((uintptr_t)kcache & 15) == 0 && ((uintptr_t)vcache & 15) == 0 && ((uintptr_t)plan & 15) == 0,
             "af_attn_decode: cache and plan alignment");
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
  a.plan = plan;
  a.out = (__nv_bfloat16*)out;
  a.out_stride = out_stride;
  AF_REQUIRE(n_pages > 0 && n_pages * nkv * AF_PAGE < (1ll << 31), "af_attn_decode: %lld cache pages", n_pages);
  if (hd == 64) return launch_decode<64>(a, batch, n_pages, stream);
  if (hd == 128) return launch_decode<128>(a, batch, n_pages, stream);
  return launch_decode<256>(a, batch, n_pages, stream);
}

// ---------------------------------------------------------------- the plan of a step

// 32-bit integers of a plan for af_attn_decode.
AF_EXPORT long long af_attn_decode_plan_ints(int batch, int nq, int nkv) {
  if (batch <= 0 || nq <= 0 || nkv <= 0 || nq % nkv) return 0;
  const int units_per_seq = nkv * ((nq / nkv + 15) / 16);
  int sms = af_sm_count();
  if (sms <= 0) return 0;
  return da_plan_records_at(batch, units_per_seq) + (long long)sms * DA_PLAN_REC;
}

// Works out, once for a step, how af_attn_decode cuts the work of the layers that read the same caches the same
// way (the same slots, lengths, page table, heads, window, ring and n_splits): pass `plan` to each of their calls.
// It holds for these lengths alone: a step later it is made again.
AF_EXPORT int af_attn_decode_plan(int* plan, long long plan_ints, const int* page_table, int max_pages,
                                  const int* slots, const int* lens, int batch, int nq, int nkv, int window,
                                  int ring_rows, int n_splits, cudaStream_t stream) {
  if (batch == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "af_attn_decode_plan: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(plan != nullptr && ((uintptr_t)plan & 15) == 0 && plan_ints >= af_attn_decode_plan_ints(batch, nq, nkv),
             "af_attn_decode_plan: a plan of %lld integers, 16-byte aligned, wanted", af_attn_decode_plan_ints(batch, nq, nkv));
  AF_REQUIRE(n_splits >= 1 && ring_rows % AF_PAGE == 0, "af_attn_decode_plan: splits %d, ring rows %d", n_splits, ring_rows);
  const int units_per_seq = nkv * ((nq / nkv + 15) / 16);
  AF_REQUIRE(batch <= DA_MAX_BATCH && (long long)batch * (max_pages + 1) * units_per_seq < (1ll << 31),
             "af_attn_decode_plan: %d sequences of up to %d pages (takes %d sequences)", batch, max_pages, DA_MAX_BATCH);
  const int sms = af_sm_count();
  if (sms <= 0) return -1;
  af_launch(attn_decode_plan_kernel, dim3(1), dim3(256), (size_t)2 * (batch + 1) * sizeof(int), stream, plan, slots,
            lens, page_table, max_pages, batch, nq, nkv, window, ring_rows, n_splits, sms);
  AF_CHECK_LAUNCH("af_attn_decode_plan");
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
                        batch, nq, nkv, hd, scale, cap, window, ring_rows, n_splits, scratch, nullptr, err, stream);
}
