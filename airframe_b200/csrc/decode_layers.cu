// The layers of one decode step (at most 8 tokens, bfloat16) as ONE persistent
// kernel: a block per SM walks a list of phases, with a barrier over the grid
// between two phases.
//
// A step of few tokens is bound by the bytes it streams (weights, cache
// pages).  As a chain of kernels, each of the nine short kernels of a layer
// pays its own fill and drain and its own dependent memory round trips.  Here
// one thread of every block (the producer) copies the tiles of ALL phases, in
// order, by TMA through one ring of shared-memory stages, and runs ahead of
// the eight consumer warps by the depth of the ring: while the consumers wait
// at a grid barrier, or do a phase's short dependent work, the weights of the
// next phases keep arriving.
//
// Phases (each an entry of 32 words, made by the host from the layers' parts):
//   GEMV   y[t, n] = sum_k W[n, k] a[t, k] for the step's tokens.  A unit is a
//          pair of 16-row tiles of W times a part of K; the token rows are the
//          n = 8 of mma.sync m16n8k16 (32-bit accumulators), the eight warps
//          split a stage's 512 columns and are summed through shared memory.
//          The two tiles of a unit hold the two rows that an epilogue joins:
//          a rotary pair (row i and i + head_dim / 2: rotation, then q to its
//          buffer and k, v to their cache rows), gate and up (activation times
//          up), or nothing (32-bit partial sums per K part).
//   ATTN   a unit is (sequence, kv head, split of the keys): cache pages come
//          in through the ring (K in one stage, V in the next), each warp
//          takes 8 of a page's 64 keys: Q K^T (m16n8k16), softcap, online
//          softmax in 32 bits, P V (m16n8k8); the warps are merged and leave
//          (max, sum, output) per split.
//   MERGE  joins the splits, writes bfloat16.
//   NORM   x += norm(sum of partial sums) and the next norm of x as bfloat16
//          (one block per token).
// What a phase writes, a later phase reads after the grid barrier between
// them; the one cache page that holds the new token is copied only after the
// barrier of the phase that wrote it.
//
// Every wait (copies, ring, grid barrier) is bounded in time; a block that
// gives up raises a flag that ends the others, and the error word is set.
#include <cstring>

#include "airframe_b200.h"
#include "tma.cuh"

namespace {

constexpr int MK_T = 8;                // token rows of a step at most
constexpr int MK_WARPS = 8;            // consumer warps
constexpr int MK_CONSUMERS = MK_WARPS * 32;
constexpr int MK_THREADS = MK_CONSUMERS + 32;   // + the producer's warp
constexpr int MK_STAGES = 5;
constexpr int MK_STAGE_BYTES = 32768;  // 32 weight rows x 512 columns, or a page's K (or V) tile of 64 x 256
constexpr int MK_KC = 512;             // weight columns of a stage
constexpr int MK_KP_MAX = 3584;        // columns of the token operand that a block keeps
constexpr int MK_ACT_BYTES = MK_T * (MK_KP_MAX + 8) * 2;
constexpr int MK_RED_BYTES = MK_WARPS * 2 * 16 * MK_T * 4;
constexpr int MK_SMEM = MK_STAGES * MK_STAGE_BYTES + MK_ACT_BYTES + MK_RED_BYTES + 1024;
constexpr int MK_WORDS = 32;           // words of a phase entry and of an attention entry

enum MkKind { MK_GEMV = 0, MK_ATTN = 1, MK_MERGE = 2, MK_NORM = 3 };
enum MkEpilogue { MK_EP_PART = 0, MK_EP_ROPE = 1, MK_EP_GATED = 2 };

// words of a phase entry
enum {
  PH_KIND = 0, PH_MAP = 2, PH_TILES = 3, PH_KPARTS = 4, PH_KPART = 5, PH_EP = 6, PH_HEADS = 7, PH_IN = 8, PH_IN_LD = 9,
  PH_ROWS = 10, PH_ACT = 11, PH_ATTN = 12, PH_ROT = 13, PH_NPARTS = 14, PH_DEP = 15, PH_WPOST = 16, PH_WNEXT = 18,
  PH_EPS_POST = 20, PH_EPS_NEXT = 21, PH_OFFSET = 22
};
// words of an attention entry
enum {
  AT_NQ = 0, AT_NKV = 1, AT_WINDOW = 2, AT_RING = 3, AT_MAXPAGES = 4, AT_SPLITS = 5, AT_SCALE = 6, AT_CAP = 7,
  AT_KCACHE = 8, AT_VCACHE = 10, AT_TABLE = 12, AT_FREQ = 14, AT_MAPK = 16
};

struct MkArgs {
  const int* phases;
  const int* attn;
  const CUtensorMap* maps;
  int n_phases, n_tok, hidden, n_ctas;
  float* x;                 // [n_tok, hidden] residual stream
  __nv_bfloat16* buf[4];    // 0: normed x [n_tok, hidden]; 1: attention output; 2: gated activation; 3: q
  float* parts;             // [K parts][n_tok][hidden] partial sums of the O and down products
  float* part_o;            // [n_tok, nq, splits, HD]
  float* part_ml;           // [n_tok, nq, splits, 2]
  const int* positions;
  const int* slots;
  const int* len_after;
  unsigned* sync;           // [0]: arrivals at the grid barrier, [1]: a block gave up
  int* err;
  unsigned long long* trace;  // optional [blocks][phases][8] times (ns): 0 phase begun, 1 its work done, 2.. marks inside
};

template <typename T>
__device__ __forceinline__ T* word_ptr(const int* w) {
  return reinterpret_cast<T*>((unsigned long long)(unsigned)w[0] | ((unsigned long long)(unsigned)w[1] << 32));
}

__device__ __forceinline__ void mk_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mk_ldm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mk_ldm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mk_mma16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mk_mma8(float* c, uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t mk_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float mk_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float mk_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// rows of global memory into shared memory by the copy engine; `bytes` a multiple of 16, both ends 16-byte aligned
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(MK_CONSUMERS) : "memory"); }
// generic-proxy writes to global memory before, copies by TMA (the async proxy) after
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Waits until `target` blocks have arrived at sync[0] (sync[1] != 0: a block gave up; both words are
// read with one load).  False when the time ran out, another block gave up, or this block gave up.
__device__ __forceinline__ bool wait_arrivals(unsigned* sync, unsigned target, volatile int* give_up) {
  const unsigned long long t0 = now_ns();
  for (int spin = 0;; ++spin) {
    // relaxed polls, one acquire fence once the count is there (an acquire load per poll is slower)
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(sync) : "memory");
    if ((v >> 32) == 0 && (unsigned)v >= target) {
      asm volatile("fence.acq_rel.gpu;" ::: "memory");
      return true;
    }
    if ((v >> 32) != 0 || *give_up || ((spin & 63) == 63 && now_ns() - t0 > AF_WAIT_LIMIT_NS)) {
      *give_up = 1;
      atomicExch(sync + 1, 1u);
      return false;
    }
  }
}

// The barrier over the grid after phase `done` (0-based), called by the consumer warps.  The
// block's writes are ordered before its first thread's arrival by the block barrier, and the
// arrival is a release; the wait reads with acquire.
__device__ __forceinline__ bool grid_barrier(const MkArgs& a, int done, volatile int* give_up, int tid) {
  consumers_sync();
  if (tid == 0) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(a.sync), "r"(1u) : "memory");
    wait_arrivals(a.sync, (unsigned)(done + 1) * (unsigned)a.n_ctas, give_up);
  }
  consumers_sync();
  return *give_up == 0;
}

// Sum over the consumer threads; every one of them gets the result.
__device__ __forceinline__ float consumers_sum(float v, float* scratch, int warp, int lane) {
  v = warp_sum(v);
  consumers_sync();
  if (lane == 0) scratch[warp] = v;
  consumers_sync();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < MK_WARPS; ++w) t += scratch[w];
  return t;
}

__device__ __forceinline__ void mark(const MkArgs& a, int phase, int k, int tid) {
  if (a.trace != nullptr && tid == 0) a.trace[((size_t)blockIdx.x * a.n_phases + phase) * 8 + k] = now_ns();
}

// ---- the units of a block in a phase (the producer and the consumers enumerate alike)

// GEMV: with P parts of K, block c works on part c % P and on the row tiles c / P, c / P + per, ...
struct GemvWork {
  int p, first, step, n_tiles, n_stages, kp;
};
__device__ __forceinline__ GemvWork gemv_work(const int* ph, int c, int n_ctas) {
  GemvWork w;
  const int P = ph[PH_KPARTS];
  w.kp = ph[PH_KPART];
  w.step = n_ctas / P;
  w.p = c % P;
  w.first = c / P;
  w.n_tiles = c < w.step * P ? ph[PH_TILES] : 0;
  w.n_stages = (w.kp + MK_KC - 1) / MK_KC;
  return w;
}
// rows of the two 16-row tiles of unit j
__device__ __forceinline__ void gemv_rows(const int* ph, int j, int hd, int& row_a, int& row_b) {
  if (ph[PH_HEADS]) {              // heads of the packed [q | k | v] rows: features i and i + hd / 2
    const int per = hd / 32;
    row_a = (j / per) * hd + (j % per) * 16;
    row_b = row_a + hd / 2;
  } else {
    row_a = j * 32;
    row_b = row_a + 16;
  }
}

// ATTN: the pages of unit u = (b * nkv + kvh) * splits + z
struct AttnWork {
  int b, kvh, z, slot, len, pos, lo, pp_begin, n_pages, last_pp;
};
__device__ __forceinline__ AttnWork attn_work(const MkArgs& a, const int* at, int u) {
  AttnWork w;
  const int splits = at[AT_SPLITS], nkv = at[AT_NKV], window = at[AT_WINDOW];
  w.z = u % splits;
  w.kvh = (u / splits) % nkv;
  w.b = u / (splits * nkv);
  w.slot = a.slots[w.b];
  w.len = w.slot >= 0 ? a.len_after[w.b] : 0;
  w.pos = w.len - 1;
  w.lo = window > 0 ? max(0, w.pos - window + 1) : 0;
  w.last_pp = w.pos / AF_PAGE;
  w.pp_begin = 0;
  w.n_pages = 0;
  if (w.len > 0) {
    const int first_pp = w.lo / AF_PAGE;
    const int n_pp = w.last_pp - first_pp + 1;
    const int per = (n_pp + splits - 1) / splits;
    w.pp_begin = first_pp + w.z * per;
    w.n_pages = max(min(w.pp_begin + per, w.last_pp + 1) - w.pp_begin, 0);
  }
  return w;
}

// ------------------------------------------------------------------ the producer (one thread)

template <int HD>
__device__ void producer(const MkArgs& a, unsigned char* ring, uint64_t* full, uint64_t* empty, volatile int* give_up) {
  const int cta = blockIdx.x;
  uint32_t n = 0;   // stages filled so far
  for (int i = 0; i < a.n_phases; ++i) {
    const int* ph = a.phases + (size_t)i * MK_WORDS;
    const int kind = ph[PH_KIND];
    const int c = (cta + ph[PH_ROT]) % a.n_ctas;
    if (kind == MK_GEMV) {
      const GemvWork w = gemv_work(ph, c, a.n_ctas);
      const CUtensorMap* map = a.maps + ph[PH_MAP];
      for (int j = w.first; j < w.n_tiles; j += w.step) {
        int row_a, row_b;
        gemv_rows(ph, j, HD, row_a, row_b);
        for (int s = 0; s < w.n_stages; ++s, ++n) {
          const int slot = n % MK_STAGES;
          if (!mbar_wait(&empty[slot], ((n / MK_STAGES) & 1) ^ 1, give_up)) return;
          const int cols = min(MK_KC, w.kp - s * MK_KC);
          unsigned char* st = ring + (size_t)slot * MK_STAGE_BYTES;
          mbar_expect_tx(&full[slot], (uint32_t)(cols / 64) * 4096u);
          const int col0 = w.p * w.kp + s * MK_KC;
          for (int cc = 0; cc < cols / 64; ++cc) {
            tma_load_2d(st + cc * 4096, map, col0 + cc * 64, row_a, &full[slot]);
            tma_load_2d(st + cc * 4096 + 2048, map, col0 + cc * 64, row_b, &full[slot]);
          }
        }
      }
    } else if (kind == MK_ATTN) {
      const int* at = a.attn + (size_t)ph[PH_ATTN] * MK_WORDS;
      const int nkv = at[AT_NKV], ring_pages = at[AT_RING] / AF_PAGE;
      const int units = a.n_tok * nkv * at[AT_SPLITS];
      const CUtensorMap* map_k = a.maps + at[AT_MAPK];
      const CUtensorMap* map_v = map_k + 1;
      const int* table = word_ptr<const int>(at + AT_TABLE);
      bool written = false;   // the phase that wrote the new token's cache row is over
      for (int u = c; u < units; u += a.n_ctas) {
        const AttnWork w = attn_work(a, at, u);
        const int* pt = table + (size_t)max(w.slot, 0) * at[AT_MAXPAGES];
        for (int pg = 0; pg < w.n_pages; ++pg) {
          const int pp = w.pp_begin + pg;
          if (pp == w.last_pp && !written) {
            if (!wait_arrivals(a.sync, (unsigned)(ph[PH_DEP] + 1) * (unsigned)a.n_ctas, give_up)) return;
            proxy_fence();
            written = true;
          }
          const int page = pt[ring_pages > 0 ? pp % ring_pages : pp];
          const int row = (page * nkv + w.kvh) * AF_PAGE;
#pragma unroll
          for (int kv = 0; kv < 2; ++kv, ++n) {
            const int slot = n % MK_STAGES;
            if (!mbar_wait(&empty[slot], ((n / MK_STAGES) & 1) ^ 1, give_up)) return;
            unsigned char* st = ring + (size_t)slot * MK_STAGE_BYTES;
            mbar_expect_tx(&full[slot], (uint32_t)(AF_PAGE * HD * 2));
#pragma unroll
            for (int cc = 0; cc < HD / 64; ++cc) tma_load_2d(st + cc * 8192, kv ? map_v : map_k, cc * 64, row, &full[slot]);
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------ the consumers' phases

template <int HD>
__device__ bool gemv_phase(const MkArgs& a, int phase, const int* ph, int c, unsigned char* ring, __nv_bfloat16* acts, float* red,
                           uint64_t* full, uint64_t* empty, uint64_t* act_bar, uint32_t& act_uses, uint32_t& n,
                           volatile int* give_up, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  const GemvWork w = gemv_work(ph, c, a.n_ctas);
  if (w.first >= w.n_tiles) return true;
  const int SA = w.kp + 8;   // elements between token rows in shared memory (16 bytes off a multiple of 128)
  {
    // the token operand of this block's K part: one bulk copy per token row (the copy engine moves it in one
    // round trip; plain loads are held back by the few misses an SM keeps in flight).  The rows were
    // written by other blocks' plain stores before the grid barrier: this thread passed the barrier's
    // acquire, the proxy fence orders the copies after it.
    const __nv_bfloat16* src = a.buf[ph[PH_IN]] + (size_t)w.p * w.kp;
    const int ld = ph[PH_IN_LD];
    if (tid == 0) {
      proxy_fence();
      mbar_expect_tx(act_bar, (uint32_t)(a.n_tok * w.kp * 2));
      for (int t = 0; t < a.n_tok; ++t) bulk_load(acts + (size_t)t * SA, src + (size_t)t * ld, (uint32_t)(w.kp * 2), act_bar);
    }
    const int pieces = w.kp / 8;
    for (int idx = a.n_tok * pieces + tid; idx < MK_T * pieces; idx += MK_CONSUMERS) {   // rows without a token
      const int t = idx / pieces, c8 = idx - t * pieces;
      *reinterpret_cast<uint4*>(acts + (size_t)t * SA + c8 * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  const uint32_t acts_u = smem_u32(acts);
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;   // ldmatrix row of the weight tiles
  const int ep = ph[PH_EP];
  const int e_tk = tid >> 4, e_r = tid & 15;   // the (token, row of the tile) that this thread finishes
  for (int j = w.first; j < w.n_tiles; j += w.step) {
    int row_a, row_b;
    gemv_rows(ph, j, HD, row_a, row_b);
    // the rotary epilogue's inputs are the step's own (positions, slots, page table): the pair's sine and
    // cosine and its place in the q buffer or in the cache are worked out while the operand and the unit's
    // tiles arrive
    float sn = 0.f, cs = 1.f;
    __nv_bfloat16* pair_dst = nullptr;
    bool to_cache = false;
    if (ep == MK_EP_ROPE && tid < MK_T * 16 && e_tk < a.n_tok) {
      const int* at = a.attn + (size_t)ph[PH_ATTN] * MK_WORDS;
      const int nq = at[AT_NQ], nkv = at[AT_NKV];
      const int head = row_a / HD, i0 = row_a - head * HD + e_r;
      const int pos = a.positions[e_tk];
      if (head < nq + nkv) sincosf((float)pos * word_ptr<const float>(at + AT_FREQ)[i0], &sn, &cs);
      if (head < nq) {
        pair_dst = a.buf[3] + (size_t)e_tk * nq * HD + (size_t)head * HD + i0;
      } else {
        const int slot = a.slots[e_tk];
        if (slot >= 0) {
          const int ring_rows = at[AT_RING];
          const int rr = ring_rows > 0 ? pos % ring_rows : pos;
          const int page = word_ptr<const int>(at + AT_TABLE)[(size_t)slot * at[AT_MAXPAGES] + rr / AF_PAGE];
          const bool is_v = head >= nq + nkv;
          const int h = head - nq - (is_v ? nkv : 0);
          pair_dst = word_ptr<__nv_bfloat16>(at + (is_v ? AT_VCACHE : AT_KCACHE)) +
                     (((size_t)page * nkv + h) * AF_PAGE + rr % AF_PAGE) * HD + i0;
          to_cache = true;
        }
      }
    }
    if (j == w.first) {
      const bool ok = mbar_wait(act_bar, act_uses & 1, give_up);
      ++act_uses;
      if (!ok) return false;
      consumers_sync();   // (the zeroed rows)
      mark(a, phase, 2, tid);
    }
    float acc[2][4];
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[0][e] = acc[1][e] = 0.f;
    for (int s = 0; s < w.n_stages; ++s, ++n) {
      const int slot = n % MK_STAGES;
      if (!mbar_wait(&full[slot], (n / MK_STAGES) & 1, give_up)) return false;
      if (j == w.first && s == 0) mark(a, phase, 3, tid);
      const int cols = min(MK_KC, w.kp - s * MK_KC);
      if (warp * 64 < cols) {
        const uint32_t st = smem_u32(ring + (size_t)slot * MK_STAGE_BYTES + warp * 4096);
        const int col0 = s * MK_KC + warp * 64;
#pragma unroll
        for (int kk = 0; kk < 4; kk += 2) {
          uint32_t b0, b1, b2, b3;   // the tokens' k 0-7, 8-15 of step kk and of step kk + 1
          mk_ldm4(acts_u + (uint32_t)(((lane & 7) * SA + col0 + kk * 16 + (lane >> 3) * 8) * 2), b0, b1, b2, b3);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int piece = (kk + h) * 2 + (lane >> 4);
            const uint32_t off = (uint32_t)(a_row * 128 + ((piece ^ (a_row & 7)) << 4));
            uint32_t x0, x1, x2, x3, y0, y1, y2, y3;
            mk_ldm4(st + off, x0, x1, x2, x3);
            mk_ldm4(st + 2048 + off, y0, y1, y2, y3);
            mk_mma16(acc[0], x0, x1, x2, x3, h ? b2 : b0, h ? b3 : b1);
            mk_mma16(acc[1], y0, y1, y2, y3, h ? b2 : b0, h ? b3 : b1);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mk_arrive(&empty[slot]);
    }
    // ---- the eight warps' sums of the unit: red[warp][tile][token][row]
    if (j + w.step >= w.n_tiles) mark(a, phase, 4, tid);
    consumers_sync();   // (the unit before has been read)
    {
      const int g = lane >> 2, t = lane & 3;
#pragma unroll
      for (int tile = 0; tile < 2; ++tile) {
        float* r = red + ((warp * 2 + tile) * MK_T) * 16;
        r[(2 * t) * 16 + g] = acc[tile][0];
        r[(2 * t + 1) * 16 + g] = acc[tile][1];
        r[(2 * t) * 16 + g + 8] = acc[tile][2];
        r[(2 * t + 1) * 16 + g + 8] = acc[tile][3];
      }
    }
    consumers_sync();
    if (tid < MK_T * 16) {
      const int tk = e_tk, r = e_r;
      float v0 = 0.f, v1 = 0.f;
#pragma unroll
      for (int ww = 0; ww < MK_WARPS; ++ww) {
        v0 += red[((ww * 2 + 0) * MK_T + tk) * 16 + r];
        v1 += red[((ww * 2 + 1) * MK_T + tk) * 16 + r];
      }
      if (tk < a.n_tok) {
        if (ep == MK_EP_PART) {
          const int rows = ph[PH_ROWS];
          float* dst = a.parts + ((size_t)w.p * a.n_tok + tk) * rows;
          if (row_a + r < rows) dst[row_a + r] = v0;
          if (row_b + r < rows) dst[row_b + r] = v1;
        } else if (ep == MK_EP_GATED) {
          // rows 32 j + r: gate of feature 16 j + r; rows 32 j + 16 + r: its up
          const int f = j * 16 + r;
          if (f < ph[PH_ROWS]) {
            float act;
            if (ph[PH_ACT] == AF_ACT_GELU_TANH) {
              const float uu = 0.7978845608028654f * (v0 + 0.044715f * v0 * v0 * v0);
              act = 0.5f * v0 * (1.f + mk_tanh(uu));
            } else {
              act = v0 / (1.f + __expf(-v0));
            }
            a.buf[2][(size_t)tk * ph[PH_ROWS] + f] = __float2bfloat16_rn(act * v1);
          }
        } else if (pair_dst != nullptr) {
          // a rotary pair: features i0 and i0 + HD / 2 of a head (v heads: sine 0, cosine 1)
          pair_dst[0] = __float2bfloat16_rn(v0 * cs - v1 * sn);
          pair_dst[HD / 2] = __float2bfloat16_rn(v1 * cs + v0 * sn);
          if (to_cache) proxy_fence();   // the attention phase copies this row by TMA
        }
      }
    }
  }
  mark(a, phase, 5, tid);
  return true;
}

// Address of the 16-byte piece `c` (of HD / 8) of key row `r` in a K or V tile: HD / 64 sub-tiles of
// [64 rows][128 bytes], each swizzled as TMA writes it.
__device__ __forceinline__ uint32_t mk_piece(uint32_t tile, int r, int c) {
  return tile + (uint32_t)((c >> 3) * 8192 + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

template <int HD>
__device__ bool attn_phase(const MkArgs& a, const int* ph, int c, unsigned char* ring, unsigned char* work, float* red,
                           uint64_t* full, uint64_t* empty, uint32_t& n, volatile int* give_up, int tid) {
  constexpr int KSTEPS = HD / 16, ONT = HD / 8, QLD = HD + 8;
  constexpr float LOG2E = 1.4426950408889634f;
  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;   // ldmatrix row of the query tile
  const int* at = a.attn + (size_t)ph[PH_ATTN] * MK_WORDS;
  const int nq = at[AT_NQ], nkv = at[AT_NKV], splits = at[AT_SPLITS];
  const int group = nq / nkv;   // the host checked: at most 16, and the merge buffer holds them
  const float scale = __int_as_float(at[AT_SCALE]), cap = __int_as_float(at[AT_CAP]);
  const float cs = cap > 0.f ? scale / cap : scale * LOG2E;
  const float cap2 = cap * LOG2E;
  const int units = a.n_tok * nkv * splits;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(work);              // [16][HD + 8]
  float* o_s = reinterpret_cast<float*>(work + 16 * QLD * 2);               // [warp][group][HD]
  float* m_s = red;                                                         // [warp][16]
  float* l_s = red + MK_WARPS * 16;
  for (int u = c; u < units; u += a.n_ctas) {
    const AttnWork w = attn_work(a, at, u);
    consumers_sync();   // (the unit before has been merged)
    {
      const __nv_bfloat16* q = a.buf[3] + (size_t)w.b * nq * HD + (size_t)w.kvh * group * HD;
      for (int idx = tid; idx < 16 * (HD / 8); idx += MK_CONSUMERS) {
        const int r = idx / (HD / 8), c8 = idx - r * (HD / 8);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < group && w.len > 0) v = *reinterpret_cast<const uint4*>(q + (size_t)r * HD + c8 * 8);
        *reinterpret_cast<uint4*>(q_s + r * QLD + c8 * 8) = v;
      }
    }
    consumers_sync();
    const uint32_t q_u = smem_u32(q_s);
    float o[ONT][4];
#pragma unroll
    for (int nn = 0; nn < ONT; ++nn) o[nn][0] = o[nn][1] = o[nn][2] = o[nn][3] = 0.f;
    float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f};
    for (int pg = 0; pg < w.n_pages; ++pg) {
      // ---- S = Q K^T for this warp's 8 keys of the page
      const int slot_k = n % MK_STAGES;
      if (!mbar_wait(&full[slot_k], (n / MK_STAGES) & 1, give_up)) return false;
      const uint32_t k_t = smem_u32(ring + (size_t)slot_k * MK_STAGE_BYTES);
      float sc2[2][4];
#pragma unroll
      for (int e = 0; e < 4; ++e) sc2[0][e] = sc2[1][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ks += 2) {
        uint32_t b0, b1, b2, b3;   // the keys' d 0-7, 8-15 of step ks and of step ks + 1
        mk_ldm4(mk_piece(k_t, warp * 8 + (lane & 7), ks * 2 + (lane >> 3)), b0, b1, b2, b3);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t q0, q1, q2, q3;
          mk_ldm4(q_u + (uint32_t)((a_row * QLD + (ks + h) * 16 + (lane >> 4) * 8) * 2), q0, q1, q2, q3);
          mk_mma16(sc2[h], q0, q1, q2, q3, h ? b2 : b0, h ? b3 : b1);
        }
      }
      __syncwarp();
      if (lane == 0) mk_arrive(&empty[slot_k]);
      ++n;
      float sc[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[e] = sc2[0][e] + sc2[1][e];
      // ---- scale, softcap, mask, online softmax (base 2)
      if (cap > 0.f) {
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[e] = cap2 * mk_tanh(sc[e] * cs);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[e] *= cs;
      }
      const int j0 = (w.pp_begin + pg) * AF_PAGE + warp * 8 + 2 * t;
      float new_max[2] = {mx[0], mx[1]};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int jj = j0 + (e & 1);
        const float v = (jj >= w.lo && jj <= w.pos) ? sc[e] : -INFINITY;
        sc[e] = v;
        new_max[e >> 1] = fmaxf(new_max[e >> 1], v);
      }
      float corr[2], ref[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        new_max[r] = fmaxf(new_max[r], __shfl_xor_sync(0xffffffffu, new_max[r], 1));
        new_max[r] = fmaxf(new_max[r], __shfl_xor_sync(0xffffffffu, new_max[r], 2));
        ref[r] = new_max[r] == -INFINITY ? 0.f : new_max[r];
        corr[r] = mk_exp2(mx[r] - ref[r]);
        mx[r] = new_max[r];
        sum[r] *= corr[r];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = mk_exp2(sc[e] - ref[e >> 1]);
        sc[e] = p;
        sum[e >> 1] += p;
      }
      if (corr[0] != 1.f || corr[1] != 1.f) {
#pragma unroll
        for (int nn = 0; nn < ONT; ++nn) {
          o[nn][0] *= corr[0];
          o[nn][1] *= corr[0];
          o[nn][2] *= corr[1];
          o[nn][3] *= corr[1];
        }
      }
      // ---- O += P V over this warp's 8 keys
      const int slot_v = n % MK_STAGES;
      if (!mbar_wait(&full[slot_v], (n / MK_STAGES) & 1, give_up)) return false;
      const uint32_t v_t = smem_u32(ring + (size_t)slot_v * MK_STAGE_BYTES);
      const uint32_t a0 = mk_pack(sc[0], sc[1]), a1 = mk_pack(sc[2], sc[3]);
#pragma unroll
      for (int np = 0; np < ONT / 4; ++np) {
        uint32_t b0, b1, b2, b3;   // d 32 np + 8 m .. + 7 of the warp's keys, m = 0..3
        mk_ldm4t(mk_piece(v_t, warp * 8 + (lane & 7), np * 4 + (lane >> 3)), b0, b1, b2, b3);
        mk_mma8(o[4 * np], a0, a1, b0);
        mk_mma8(o[4 * np + 1], a0, a1, b1);
        mk_mma8(o[4 * np + 2], a0, a1, b2);
        mk_mma8(o[4 * np + 3], a0, a1, b3);
      }
      __syncwarp();
      if (lane == 0) mk_arrive(&empty[slot_v]);
      ++n;
    }
    // ---- merge the eight warps (each saw an eighth of the keys)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
      const int row = g + 8 * r;
      if (t == 0) {
        m_s[warp * 16 + row] = mx[r];
        l_s[warp * 16 + row] = sum[r];
      }
      if (row < group) {
#pragma unroll
        for (int nn = 0; nn < ONT; ++nn) {
          float* dst = o_s + ((size_t)(warp * group + row)) * HD + nn * 8 + 2 * t;
          dst[0] = o[nn][2 * r];
          dst[1] = o[nn][2 * r + 1];
        }
      }
    }
    consumers_sync();
    for (int i = tid; i < group * HD; i += MK_CONSUMERS) {
      const int row = i / HD, d = i - row * HD;
      float M = -INFINITY;
#pragma unroll
      for (int ww = 0; ww < MK_WARPS; ++ww) M = fmaxf(M, m_s[ww * 16 + row]);
      const float ref = M == -INFINITY ? 0.f : M;
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int ww = 0; ww < MK_WARPS; ++ww) {
        const float f = mk_exp2(m_s[ww * 16 + row] - ref);
        L += l_s[ww * 16 + row] * f;
        O += o_s[((size_t)(ww * group + row)) * HD + d] * f;
      }
      const size_t pidx = ((size_t)w.b * nq + w.kvh * group + row) * splits + w.z;
      a.part_o[pidx * HD + d] = O;
      if (d == 0) {
        a.part_ml[pidx * 2] = M;
        a.part_ml[pidx * 2 + 1] = L;
      }
    }
  }
  return true;
}

template <int HD>
__device__ void merge_phase(const MkArgs& a, const int* ph, int c, int tid) {
  constexpr int FEW = 8;
  const int* at = a.attn + (size_t)ph[PH_ATTN] * MK_WORDS;
  const int nq = at[AT_NQ], splits = at[AT_SPLITS];
  const int units = a.n_tok * nq;
  for (int u = c; u < units; u += a.n_ctas) {
    const size_t p0 = (size_t)u * splits;
    if (splits <= FEW) {
      // every load (outputs, maxima, sums) is issued before the first use: one round trip
      const int d = tid;
      float o[FEW], m[FEW], l[FEW];
#pragma unroll
      for (int s = 0; s < FEW; ++s) {
        const bool on = s < splits;
        m[s] = on ? a.part_ml[(p0 + s) * 2] : -INFINITY;
        l[s] = on ? a.part_ml[(p0 + s) * 2 + 1] : 0.f;
        o[s] = on && d < HD ? a.part_o[(p0 + s) * HD + d] : 0.f;
      }
      float M = -INFINITY;
#pragma unroll
      for (int s = 0; s < FEW; ++s) M = fmaxf(M, m[s]);
      const float ref = M == -INFINITY ? 0.f : M;
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int s = 0; s < FEW; ++s) {
        const float f = mk_exp2(m[s] - ref);
        L += l[s] * f;
        O += o[s] * f;
      }
      if (d < HD) a.buf[1][(size_t)u * HD + d] = __float2bfloat16_rn(O * (L > 0.f ? 1.f / L : 0.f));
      continue;
    }
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, a.part_ml[(p0 + s) * 2]);
    const float ref = M == -INFINITY ? 0.f : M;
    float L = 0.f;
    for (int s = 0; s < splits; ++s) L += a.part_ml[(p0 + s) * 2 + 1] * mk_exp2(a.part_ml[(p0 + s) * 2] - ref);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = tid; d < HD; d += MK_CONSUMERS) {
      float O = 0.f;
      for (int s = 0; s < splits; ++s) O += a.part_o[(p0 + s) * HD + d] * mk_exp2(a.part_ml[(p0 + s) * 2] - ref);
      a.buf[1][(size_t)u * HD + d] = __float2bfloat16_rn(O * inv);
    }
  }
}

__device__ void norm_phase(const MkArgs& a, const int* ph, int c, float* scratch, int tid) {
  constexpr int NV = (MK_KP_MAX / 4 + MK_CONSUMERS - 1) / MK_CONSUMERS;   // groups of 4 elements a thread holds
  const int warp = tid >> 5, lane = tid & 31;
  const int H = a.hidden, H4 = H / 4, n_parts = ph[PH_NPARTS];
  const float4* w_post = word_ptr<const float4>(ph + PH_WPOST);
  const float4* w_next = word_ptr<const float4>(ph + PH_WNEXT);
  const float offset = __int_as_float(ph[PH_OFFSET]);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int tk = c; tk < a.n_tok; tk += a.n_ctas) {
    // every load (x, the norms' weights, the partial sums) is issued before the first use: one round trip
    float4 av[NV], xv[NV], wp[NV], wn[NV];
    float4* x = reinterpret_cast<float4*>(a.x + (size_t)tk * H);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int i = tid + v * MK_CONSUMERS;
      const bool on = i < H4;
      xv[v] = on ? x[i] : zero;
      wp[v] = on && n_parts > 0 ? w_post[i] : zero;
      wn[v] = on && w_next != nullptr ? w_next[i] : zero;
      av[v] = zero;
    }
    for (int p0 = 0; p0 < n_parts; p0 += 4) {
      float4 t[4][NV];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          const int i = tid + v * MK_CONSUMERS;
          t[u][v] = (p0 + u < n_parts && i < H4)
                        ? reinterpret_cast<const float4*>(a.parts + ((size_t)(p0 + u) * a.n_tok + tk) * H)[i]
                        : zero;
        }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          av[v].x += t[u][v].x;
          av[v].y += t[u][v].y;
          av[v].z += t[u][v].z;
          av[v].w += t[u][v].w;
        }
    }
    if (n_parts > 0) {
      float ss = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v) ss += av[v].x * av[v].x + av[v].y * av[v].y + av[v].z * av[v].z + av[v].w * av[v].w;
      ss = consumers_sum(ss, scratch, warp, lane);
      const float inv = rsqrtf(ss / (float)H + __int_as_float(ph[PH_EPS_POST]));
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int i = tid + v * MK_CONSUMERS;
        xv[v].x += av[v].x * inv * (offset + wp[v].x);
        xv[v].y += av[v].y * inv * (offset + wp[v].y);
        xv[v].z += av[v].z * inv * (offset + wp[v].z);
        xv[v].w += av[v].w * inv * (offset + wp[v].w);
        if (i < H4) x[i] = xv[v];
      }
    }
    if (w_next != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v) ss += xv[v].x * xv[v].x + xv[v].y * xv[v].y + xv[v].z * xv[v].z + xv[v].w * xv[v].w;
      ss = consumers_sum(ss, scratch, warp, lane);
      const float inv = rsqrtf(ss / (float)H + __int_as_float(ph[PH_EPS_NEXT]));
      uint2* y = reinterpret_cast<uint2*>(a.buf[0] + (size_t)tk * H);
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int i = tid + v * MK_CONSUMERS;
        if (i < H4)
          y[i] = make_uint2(mk_pack(xv[v].x * inv * (offset + wn[v].x), xv[v].y * inv * (offset + wn[v].y)),
                            mk_pack(xv[v].z * inv * (offset + wn[v].z), xv[v].w * inv * (offset + wn[v].w)));
      }
    }
  }
}

template <int HD>
__global__ void __launch_bounds__(MK_THREADS, 1) decode_layers_kernel(const __grid_constant__ MkArgs a) {
  extern __shared__ unsigned char mk_raw[];
  unsigned char* base = (unsigned char*)(((uintptr_t)mk_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* ring = base;
  unsigned char* work = base + MK_STAGES * MK_STAGE_BYTES;          // token operand; q and the warps' outputs
  float* red = reinterpret_cast<float*>(work + MK_ACT_BYTES);
  __shared__ uint64_t full[MK_STAGES], empty[MK_STAGES], act_bar;
  __shared__ float scratch[MK_WARPS];
  __shared__ int give_up_s;
  volatile int* give_up = &give_up_s;
  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int s = 0; s < MK_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], MK_WARPS);
    }
    mbar_init(&act_bar, 1);
    give_up_s = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (tid >= MK_CONSUMERS) {
    if (tid == MK_CONSUMERS) {
      producer<HD>(a, ring, full, empty, give_up);
      if (*give_up) grace_period();
    }
    return;
  }
  uint32_t n = 0;          // stages taken so far
  uint32_t act_uses = 0;   // token operands copied so far
  for (int i = 0; i < a.n_phases; ++i) {
    const int* ph = a.phases + (size_t)i * MK_WORDS;
    const int kind = ph[PH_KIND];
    const int c = (blockIdx.x + ph[PH_ROT]) % a.n_ctas;
    bool ok = true;
    if (a.trace != nullptr && tid == 0) a.trace[((size_t)blockIdx.x * a.n_phases + i) * 8] = now_ns();
    if (kind == MK_GEMV)
      ok = gemv_phase<HD>(a, i, ph, c, ring, reinterpret_cast<__nv_bfloat16*>(work), red, full, empty, &act_bar, act_uses, n,
                          give_up, tid);
    else if (kind == MK_ATTN)
      ok = attn_phase<HD>(a, ph, c, ring, work, red, full, empty, n, give_up, tid);
    else if (kind == MK_MERGE)
      merge_phase<HD>(a, ph, c, tid);
    else
      norm_phase(a, ph, c, scratch, tid);
    if (!ok) break;
    if (a.trace != nullptr && tid == 0) a.trace[((size_t)blockIdx.x * a.n_phases + i) * 8 + 1] = now_ns();
    if (i + 1 < a.n_phases && !grid_barrier(a, i, give_up, tid)) break;
  }
  if (*give_up && tid == 0) {
    atomicExch(a.sync + 1, 1u);
    grace_period();
    if (a.err) atomicExch(a.err, 1);
  }
}

template <int HD>
int launch_layers(const MkArgs& a, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_layers_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, MK_SMEM);
    if (e != cudaSuccess) return af_fail((int)e, "af_decode_layers: %s", cudaGetErrorString(e));
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel<HD>, MK_THREADS, MK_SMEM);
    if (e != cudaSuccess || per_sm < 1)
      return af_fail(e != cudaSuccess ? (int)e : -1, "af_decode_layers: the kernel does not fit an SM");
    configured = true;
  }
  cudaError_t e = cudaMemsetAsync(a.sync, 0, 2 * sizeof(unsigned), stream);
  if (e != cudaSuccess) return af_fail((int)e, "af_decode_layers: %s", cudaGetErrorString(e));
  // all blocks wait for one another: the launch is cooperative (it fails rather than run a part of the grid)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.n_ctas);
  cfg.blockDim = dim3(MK_THREADS);
  cfg.dynamicSmemBytes = MK_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, decode_layers_kernel<HD>, a);
  if (e != cudaSuccess) return af_fail((int)e, "af_decode_layers: launch failed: %s", cudaGetErrorString(e));
  AF_CHECK_LAUNCH("af_decode_layers");
}

}  // namespace

// What the kernel is built for: the numbers that the host needs to lay out phases.
AF_EXPORT int af_decode_layers_limit(int what) {
  switch (what) {
    case 0: return MK_T;          // tokens of a step
    case 1: return MK_KP_MAX;     // columns of a K part
    case 2: return MK_KC;         // columns of a stage
    case 3: return MK_ACT_BYTES;  // bytes for q and the warps' outputs of an attention unit
    case 4: return MK_WORDS;
    default: return -1;
  }
}

// Writes the 128-byte tensor map of a bfloat16 matrix [rows, cols] (dense rows `ld` elements apart,
// boxes of 64 columns x box_rows rows) to host memory at `out`.
AF_EXPORT int af_tensor_map_bf16(void* out, const void* base, long long rows, long long cols, long long ld,
                                 int box_rows) {
  static_assert(sizeof(CUtensorMap) == 128, "tensor maps are 128 bytes");
  AF_REQUIRE(((uintptr_t)base & 15) == 0 && ld % 8 == 0 && cols % 8 == 0, "af_tensor_map_bf16: alignment");
  CUtensorMap m;
  const int rc = af_make_map_bf16(&m, base, rows, cols, ld, box_rows);
  if (rc) return rc;
  memcpy(out, &m, sizeof(m));
  return 0;
}

// Runs the phases (see the head of this file).  `maps`: tensor maps in device memory (64-byte aligned).
// `trace` (optional): [n_ctas][n_phases][8] times in nanoseconds, per block and phase: begin, end of its work,
// then marks inside the phase (product: operand loaded, first tile arrived, last tile used, epilogue done).
AF_EXPORT int af_decode_layers(const int* phases, int n_phases, const int* attn, const void* maps, int n_tok,
                               int hidden, int hd, int n_ctas, float* x, void* normed, void* attn_out, void* gated,
                               void* q, float* parts, float* part_o, float* part_ml, const int* positions,
                               const int* slots, const int* len_after, unsigned* sync, int* err,
                               unsigned long long* trace, cudaStream_t stream) {
  AF_REQUIRE(n_phases > 0 && n_tok > 0 && n_tok <= MK_T, "af_decode_layers: %d tokens (takes 1 to %d)", n_tok, MK_T);
  AF_REQUIRE(hidden > 0 && hidden <= MK_KP_MAX, "af_decode_layers: width %d (takes up to %d)", hidden, MK_KP_MAX);
  AF_REQUIRE(hd == 128 || hd == 256, "af_decode_layers: head_dim %d (takes 128, 256)", hd);
  AF_REQUIRE(((uintptr_t)maps & 63) == 0, "af_decode_layers: tensor maps must be 64-byte aligned");
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  AF_REQUIRE(n_ctas >= 1 && n_ctas <= sms, "af_decode_layers: %d blocks on %d SMs", n_ctas, sms);
  MkArgs a;
  a.phases = phases;
  a.attn = attn;
  a.maps = (const CUtensorMap*)maps;
  a.n_phases = n_phases;
  a.n_tok = n_tok;
  a.hidden = hidden;
  a.n_ctas = n_ctas;
  a.x = x;
  a.buf[0] = (__nv_bfloat16*)normed;
  a.buf[1] = (__nv_bfloat16*)attn_out;
  a.buf[2] = (__nv_bfloat16*)gated;
  a.buf[3] = (__nv_bfloat16*)q;
  a.parts = parts;
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.positions = positions;
  a.slots = slots;
  a.len_after = len_after;
  a.sync = sync;
  a.err = err;
  a.trace = trace;
  if (hd == 128) return launch_layers<128>(a, stream);
  return launch_layers<256>(a, stream);
}
