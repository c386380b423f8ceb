// bfloat16 matrix product on the 5th-generation tensor cores:
//   out[M, N] = x[M, K] * w[N, K]^T      (tokens x features, weights [out, in])
//
// The weight is the tcgen05 "A" operand: a tile is 128 output features (the
// 128 TMEM lanes) by BN tokens (TMEM columns), so the same kernel serves
// decode (BN = 16 .. 64, bandwidth bound: the weights stream through once, a
// block per tile) and prefill (BN = 256: one block per SM walks the tiles,
// token tile fastest so that blocks running together share weight tiles in L2,
// and fetches the next tile's operands while this tile's accumulators are read back).  Both operands are K-major, staged by TMA into 128-byte
// swizzled shared memory; one elected thread issues tcgen05.mma with the
// accumulator in TMEM; four warps read it back with tcgen05.ld for the epilogue.
//
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM allocation, MMA issue (one lane), TMEM release
//   warps 2..5  epilogue: TMEM -> registers -> global
//
// Variants: NACC = 2 keeps two accumulators (two consecutive 128-feature tiles
// share one token tile: fewer bytes per flop for prefill); GATED expects a
// weight whose 32-row groups hold 16 gate rows then the 16 up rows of the same
// features, and writes act(g) * u (the halves meet by warp shuffles in the
// epilogue); split-K (gridDim.z > 1) writes float partial sums [split, M, N]
// that the consumer adds in order; `cap` > 0 applies cap * tanh(v / cap).
//
// ARGMAX (ACT == -3) is the head of greedy decoding: instead of writing logits it keeps, per token, the largest
// (capped) value and its row: every epilogue warp reduces its 32 rows and joins the result into a 64-bit key per
// token with one atomicMax (value in order-preserving bits above, ~row below: equal values go to the lowest row),
// so [tokens, vocabulary] never goes to memory.  Only finite values take part.
//
// ROPE (ACT == -2) is the projection of a mixer's packed [q | k | v] rows with the rotary
// position encoding and the cache write in its epilogue.  The weight's rows are permuted within
// each head into groups of 32: 16 rows of the head's first half, then the 16 rows they are
// rotated with (element i pairs with i + head_dim / 2), so that a pair meets inside a warp by
// one shuffle, as gate and up do.  Cosines and sines come from a table made once per step
// ([token][pair] of (cos, sin), 32-bit); rotated q, k and plain v go to the output rows in the
// unpermuted order, and k and v also to each token's row of its cache page.  With split-K the
// partial tiles go to scratch memory and the last block of a tile to finish (a ticket per tile
// and epilogue warp) adds them in index order and runs the epilogue: the sum does not depend on
// who was last.
//
// Every wait on an mbarrier is bounded in time.  A wait that runs out sets an
// error word that the host reads after the launch; the CTA then lets its
// copies in flight land, releases its TMEM and returns.
#include "umma.cuh"

namespace {

constexpr int TC_BM = 128;  // features per CTA = UMMA M
constexpr int TC_BK = 64;   // K per stage: 128 bytes of bfloat16 = one swizzle row
constexpr int TC_THREADS = 192;
constexpr int TC_SMEM_BUDGET = 192 * 1024;    // of one block alone on its SM
constexpr int TC_SMEM_BUDGET_2 = 108 * 1024;  // of each of two blocks that share an SM

__host__ __device__ constexpr int tc_stage_bytes(int bn, int nacc) {
  return nacc * TC_BM * TC_BK * 2 + bn * TC_BK * 2;
}
__host__ __device__ constexpr int tc_stages(int bn, int nacc, int per_sm) {
  int s = (per_sm == 2 ? TC_SMEM_BUDGET_2 : TC_SMEM_BUDGET) / tc_stage_bytes(bn, nacc);
  return s > 8 ? 8 : s;
}
__host__ __device__ constexpr int tc_tmem_cols(int bn, int nacc) {
  int c = nacc * bn;
  return c < 32 ? 32 : c;  // bn is a power of two
}

// The activation of the gated epilogue.  Its result is rounded to bfloat16, so
// tanh.approx (relative error 2^-11) and ex2.approx serve.
__device__ __forceinline__ float tc_act(float g, int act) {
  if (act == AF_ACT_GELU_TANH) {
    const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    return 0.5f * g * (1.f + t);
  }
  return g / (1.f + __expf(-g));
}

struct TcArgs {
  void* out;
  long long ldo;          // row stride of out in elements
  long long part_stride;  // elements between split-K partial results
  int M, N, K;            // N: output features (GATED: half the weight's rows)
  int kb_per_split;       // K blocks handled by one z-slice
  int tiles_w, tiles_m;   // tiles along the weight rows and along the tokens; a block walks the tiles
                          // blockIdx.x, blockIdx.x + gridDim.x, ... (token tile fastest)
  float cap;
  int* err;
  // ROPE only
  const float2* rope_table;  // [M][hd / 2] (cos, sin) of each token's position
  const int* kv_rows;        // [M] row of the token in the cache for kv head 0 (-1: not stored), or null
  __nv_bfloat16* kcache;     // pages [.., kv heads, AF_PAGE, hd]
  __nv_bfloat16* vcache;
  int hd, nq, nkv;
  float* parts;              // split-K: [splits][M][N] partial sums
  int* tickets;              // split-K: a counter per tile, zero between launches
  // ARGMAX only
  unsigned long long* keys;  // [M * AF_KEY_STRIDE] best (value, row) per token, zero before the launch
  int group;                 // the order in which the blocks walk the tiles (af_tile_of)
};

// Float bits whose unsigned order is the floats' order.
__device__ __forceinline__ uint32_t tc_ordered_bits(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// ACT: -1 plain product, else the gated epilogue's activation.  PER_SM: 2 halves the stages so that
// two blocks share an SM (grids of several waves: one block's fill and drain hide behind the other).
template <int BN, int NACC, int ACT, typename TO, int PER_SM>
__global__ void __launch_bounds__(TC_THREADS, PER_SM)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcArgs a) {
  constexpr bool GATED = ACT >= 0;
  constexpr bool ROPE = ACT == -2;
  constexpr bool ARGMAX = ACT == -3;
  constexpr int STAGES = tc_stages(BN, NACC, PER_SM);
  constexpr int A_BYTES = TC_BM * TC_BK * 2;
  constexpr int STAGE_BYTES = tc_stage_bytes(BN, NACC);
  constexpr int COLS = tc_tmem_cols(BN, NACC);
  constexpr uint32_t IDESC = umma_idesc(BN);

  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[STAGES], empty[STAGES], acc_full, acc_empty;
  __shared__ uint32_t tmem_base_s;
  __shared__ int give_up_s;
  volatile int* give_up = &give_up_s;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (a.K + TC_BK - 1) / TC_BK;
  const int kb0 = blockIdx.z * a.kb_per_split;
  const int kb_count = min(a.kb_per_split, total_kb - kb0);
  const int n_tiles = a.tiles_w * a.tiles_m;
  // with one tile of tokens every weight is read once: it is marked first to leave L2 (many tiles of tokens
  // come back to the same weights, which should stay)
  const bool w_once = a.tiles_m == 1;
  const uint64_t read_once = l2_policy_read_once();

  // The producer thread sets the barriers up and sends the first stages' weight tiles on their way at once,
  // before the block meets at its first barrier and before the wait for the kernel in front: the weights
  // depend on nothing, and what a short kernel loses is the time until its first bytes arrive.
  const int early = (blockIdx.x < n_tiles) ? min(STAGES, kb_count) : 0;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_full, 1);
    mbar_init(&acc_empty, 4);   // one arrival an epilogue warp
    give_up_s = 0;
    mbar_fence_init();
    int wt_first, mt_first;
    af_tile_of((int)blockIdx.x, a.tiles_w, a.tiles_m, a.group, &wt_first, &mt_first);
    const int n0 = wt_first * (TC_BM * NACC);
    for (int kb = 0; kb < early; ++kb) {
      unsigned char* st = tiles + (size_t)kb * STAGE_BYTES;
      mbar_expect_tx(&full[kb], STAGE_BYTES);
      const int k = (kb0 + kb) * TC_BK;
#pragma unroll
      for (int acc = 0; acc < NACC; ++acc) {
        if (w_once) tma_load_2d_once(st + acc * A_BYTES, &map_w, k, n0 + acc * TC_BM, &full[kb], read_once);
        else tma_load_2d(st + acc * A_BYTES, &map_w, k, n0 + acc * TC_BM, &full[kb]);
      }
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  // A block walks its tiles one after another; the K blocks of all its tiles form one sequence
  // (`it`) through the ring of stages, so the producer is already fetching the next tile while
  // the accumulators of this one are read back.
  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool first = true;
      for (int tile = blockIdx.x; tile < n_tiles && !*give_up; tile += gridDim.x) {
        int wt, mt;
        af_tile_of(tile, a.tiles_w, a.tiles_m, a.group, &wt, &mt);
        const int n0 = wt * (TC_BM * NACC), m0 = mt * BN;
        int kb = 0;
        if (first) {
          // (the weight tiles of these stages are on their way since the kernel began) the activations follow
          // once the kernel in front is done
          kb = early;
          pdl_wait();
          for (int e = 0; e < early; ++e)
            tma_load_2d(tiles + (size_t)e * STAGE_BYTES + NACC * A_BYTES, &map_x, (kb0 + e) * TC_BK, m0, &full[e]);
          it = early;
          first = false;
        }
        for (; kb < kb_count; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (it >= STAGES && !mbar_wait(&empty[s], ph ^ 1, give_up)) break;
          unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          const int k = (kb0 + kb) * TC_BK;
#pragma unroll
          for (int acc = 0; acc < NACC; ++acc) {
            if (w_once) tma_load_2d_once(st + acc * A_BYTES, &map_w, k, n0 + acc * TC_BM, &full[s], read_once);
            else tma_load_2d(st + acc * A_BYTES, &map_w, k, n0 + acc * TC_BM, &full[s]);
          }
          tma_load_2d(st + NACC * A_BYTES, &map_x, k, m0, &full[s]);
        }
      }
      if (first) pdl_wait();
      if (*give_up) grace_period();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      int it = 0, round = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++round) {
        // the accumulators are free once the epilogue warps have read the tile before out of them
        if (round > 0 && !mbar_wait(&acc_empty, (round - 1) & 1, give_up)) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kb = 0; kb < kb_count; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, give_up)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t db = umma_desc(st + NACC * A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
#pragma unroll
            for (int acc = 0; acc < NACC; ++acc)  // 32 bytes of K per step
              umma_f16(tmem_base + acc * BN, umma_desc(st + acc * A_BYTES) + 2 * k, db + 2 * k, IDESC, accum);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full);
      }
    }
  } else {
    // epilogue: warp w reads TMEM lanes [32 * (w % 4), + 32)
    const int quarter = warp & 3;
    pdl_wait();
    int round = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++round) {
      int tile_w, mt;
      af_tile_of(tile, a.tiles_w, a.tiles_m, a.group, &tile_w, &mt);
      const int m0 = mt * BN;
      if (!mbar_wait(&acc_full, round & 1, give_up)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      TO* out = reinterpret_cast<TO*>(a.out) + (size_t)blockIdx.z * a.part_stride;
      const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
      // CW columns (tokens) per round: the TMEM loads of a round are issued
      // together and waited for once
      constexpr int CW = BN >= 64 ? 64 : BN;
#pragma unroll 1
      for (int acc = 0; acc < NACC; ++acc) {
        // the output feature of this lane: a weight row, or for GATED the feature whose gate row it is
        const int wt = tile_w * NACC + acc;
        const int f = GATED ? wt * 64 + quarter * 16 + (lane & 15) : wt * TC_BM + quarter * 32 + lane;
        // ROPE: this warp's 32 weight rows are one group of a head: pairs p .. p + 15, low lanes the first half
        const int g_row0 = (wt * 4 + quarter) * 32;
        const int rp_head = ROPE ? g_row0 / a.hd : 0;
        const int rp_pair = ROPE ? ((g_row0 % a.hd) >> 5) * 16 + (lane & 15) : 0;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CW) {
          float v[CW];
          if constexpr (CW >= 32) {
#pragma unroll
            for (int c = 0; c < CW; c += 32) tmem_ld32(lane_base + acc * BN + c0 + c, v + c);
          } else {
            tmem_ld16(lane_base + acc * BN + c0, v);
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (acc == NACC - 1 && c0 + CW >= BN) {
            // everything of this tile is in registers: the next tile's products may start
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty);
          }
          if constexpr (ROPE) {
            const int half = a.hd >> 1;
            const bool live = g_row0 < a.N;              // (whole groups: N is a multiple of 32)
            if constexpr (BN <= 64 && NACC == 1) {
              if (gridDim.z > 1) {
                // split-K: leave this warp's part of the partial tile and take a ticket for its 32 rows; the
                // last of the tile's blocks to come adds all parts in index order.  (A ticket per warp, so that
                // no block-wide barrier stands behind a wait that may give up.)
                float* part = a.parts + (size_t)blockIdx.z * a.part_stride;
                if (live) {
#pragma unroll
                  for (int j = 0; j < CW; ++j)
                    if (m0 + j < a.M) part[(size_t)(m0 + j) * a.N + g_row0 + lane] = v[j];
                }
                __threadfence();
                __syncwarp();
                int ticket = 0;
                if (lane == 0) ticket = atomicAdd(a.tickets + tile * 4 + quarter, 1);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket != (int)gridDim.z - 1) continue;          // (not the last: done)
                __threadfence();
                if (lane == 0) a.tickets[tile * 4 + quarter] = 0;    // every block of the tile has taken its ticket
#pragma unroll
                for (int j = 0; j < CW; ++j) v[j] = 0.f;
                if (live) {
                  for (int sp = 0; sp < (int)gridDim.z; ++sp) {
                    const float* ps = a.parts + (size_t)sp * a.part_stride + g_row0 + lane;
#pragma unroll
                    for (int j = 0; j < CW; ++j)
                      if (m0 + j < a.M) v[j] += __ldcg(ps + (size_t)(m0 + j) * a.N);
                  }
                }
              }
            }
            const bool hi = lane >= 16;
            const bool rotate = rp_head < a.nq + a.nkv;
            const int d = rp_pair + (hi ? half : 0);
            const bool is_kv = rp_head >= a.nq && a.kv_rows != nullptr;
            const bool is_v = rp_head >= a.nq + a.nkv;
            __nv_bfloat16* cache = is_v ? a.vcache : a.kcache;
            const int kvh = rp_head - a.nq - (is_v ? a.nkv : 0);
            // Cosines, sines and cache rows of 16 tokens are fetched together before the first store: a load
            // that stands behind a store in the program is not moved before it by the compiler, and the loads
            // of a loop that stores as it goes would pay the memory's latency one after the other.
#pragma unroll
            for (int j0 = 0; j0 < CW; j0 += 16) {
              float2 cs[16];
              int crow[16];
#pragma unroll
              for (int u = 0; u < 16; ++u) {
                const int tok = m0 + c0 + j0 + u;
                const bool on = live && tok < a.M;
                cs[u] = on && rotate ? __ldg(a.rope_table + (size_t)tok * half + rp_pair) : make_float2(1.f, 0.f);
                crow[u] = on && is_kv ? __ldg(a.kv_rows + tok) : -1;
              }
#pragma unroll
              for (int u = 0; u < 16; ++u) {
                const int j = j0 + u;
                const int tok = m0 + c0 + j;
                const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
                if (!live || tok >= a.M) continue;
                const float r = hi ? v[j] * cs[u].x + other * cs[u].y : v[j] * cs[u].x - other * cs[u].y;
                const __nv_bfloat16 rb = __float2bfloat16_rn(r);
                reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)tok * a.ldo + (size_t)rp_head * a.hd + d] = rb;
                if (crow[u] >= 0) cache[((size_t)crow[u] + (size_t)kvh * AF_PAGE) * a.hd + d] = rb;
              }
            }
            continue;
          }
          if (GATED) {
            // Within a warp lanes 0..15 hold gate rows and lanes 16..31 the up rows of the
            // same 16 features.  Each half keeps one half of the round's tokens and gets
            // the partner's values for them with one shuffle per token.
            const int low = lane < 16 ? 1 : 0;
#pragma unroll
            for (int j = 0; j < CW / 2; ++j) {
              const float got = __shfl_xor_sync(0xffffffffu, pick(low, v[j + CW / 2], v[j]), 16);
              // low lanes: g(own) * u(partner) for tokens [0, CW/2); high lanes: g(partner) * u(own) for [CW/2, CW)
              const float g = pick(low, v[j], got), u = pick(low, got, v[j + CW / 2]);
              v[j] = tc_act(g, ACT) * u;
            }
          }
          if (a.cap > 0.f) {  // (fully unrolled: v stays in registers)
#pragma unroll
            for (int j = 0; j < CW; ++j) v[j] = a.cap * tanhf(v[j] / a.cap);
          }
          if constexpr (ARGMAX) {
            // per token: the warp's largest value (one redux on the order-preserving bits), then the lowest
            // row among the lanes that hold it (a second one)
#pragma unroll
            for (int j = 0; j < CW; ++j) {
              const bool has = f < a.N && isfinite(v[j]);
              const uint32_t bits = has ? tc_ordered_bits(v[j]) : 0u;        // (finite values never map to 0)
              const uint32_t best = __reduce_max_sync(0xffffffffu, bits);
              const uint32_t row = __reduce_min_sync(0xffffffffu, has && bits == best ? (uint32_t)f : 0xffffffffu);
              if (lane == 0 && best != 0u && m0 + c0 + j < a.M)
                atomicMax(a.keys + (size_t)(m0 + c0 + j) * AF_KEY_STRIDE,
                          ((unsigned long long)best << 32) | (unsigned long long)(0xffffffffu - row));
            }
            continue;
          }
          if (GATED) {
            // lane l and lane l + 16 write the same feature, for the first and the second half of the tokens
            const int tok0 = m0 + c0 + (lane < 16 ? 0 : CW / 2);
            if (f < a.N) {
              TO* o = out + (size_t)tok0 * a.ldo + f;
              if (tok0 + CW / 2 <= a.M) {
#pragma unroll
                for (int j = 0; j < CW / 2; ++j) o[(size_t)j * a.ldo] = from_f32<TO>(v[j]);
              } else {
#pragma unroll
                for (int j = 0; j < CW / 2; ++j)
                  if (tok0 + j < a.M) o[(size_t)j * a.ldo] = from_f32<TO>(v[j]);
              }
            }
          } else if (f < a.N) {
            TO* o = out + (size_t)(m0 + c0) * a.ldo + f;
            if (m0 + c0 + CW <= a.M) {
#pragma unroll
              for (int j = 0; j < CW; ++j) o[(size_t)j * a.ldo] = from_f32<TO>(v[j]);
            } else {
#pragma unroll
              for (int j = 0; j < CW; ++j)
                if (m0 + c0 + j < a.M) o[(size_t)j * a.ldo] = from_f32<TO>(v[j]);
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)COLS));
  }
  if (threadIdx.x == 0 && give_up_s && a.err) atomicExch(a.err, 1);
}

// ---------------------------------------------------------------- host side

template <int BN, int NACC, int ACT, typename TO, int PER_SM>
int launch_on(dim3 grid, const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, cudaStream_t stream) {
  constexpr int smem = tc_stages(BN, NACC, PER_SM) * tc_stage_bytes(BN, NACC) + 1024;
  // (the limit on dynamic shared memory is a device's: set once on each)
  static bool configured[AF_MAX_DEVICES] = {};
  const int dev__ = af_current_device();
  if (dev__ < 0) return -1;
  if (!configured[dev__]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, NACC, ACT, TO, PER_SM>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return af_fail((int)e, "gemm_tc: %s", cudaGetErrorString(e));
    configured[dev__] = true;
  }
  af_launch(gemm_tc_kernel<BN, NACC, ACT, TO, PER_SM>, grid, dim3(TC_THREADS), smem, stream, mw, mx, a);
  AF_CHECK_LAUNCH("af_gemm_tc");
}

template <int BN, int NACC, int ACT, typename TO>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, TcArgs a, long long n_w_rows, int splits, int per_sm,
           cudaStream_t stream) {
  const long long w_tiles = (n_w_rows + TC_BM - 1) / TC_BM;
  a.tiles_w = (int)((w_tiles + NACC - 1) / NACC);
  a.tiles_m = (a.M + BN - 1) / BN;
  const long long tiles = (long long)a.tiles_w * a.tiles_m;
  const int sms = af_sm_count();
  if (sms <= 0) return -1;
  a.group = af_tile_group(a.tiles_m, sms);
  if constexpr (BN <= 64 && NACC == 1) {
    // bound by the weight stream: a block per tile; many waves of them run two to an SM
    dim3 grid((unsigned)tiles, 1, splits);
    // Half an SM's shared memory a block for grids of more than one wave: one block's fill and drain hide
    // behind the other's stream, and a grid of one and a half waves (the gated product of 9B sizes: 224 tiles)
    // streams all its tiles at once instead of 148 and then 76 (the decode step of 9B sizes, batch 8: 4.72 ms
    // against 5.08).  (For grids that fit one wave, whose next kernel's blocks would then fit beside these, it
    // measured the same or worse inside the step: 1.68 ms against 1.66 at batch 1 of 2B sizes.)
    if (per_sm == 2 || (per_sm == 0 && tiles * splits > sms))
      return launch_on<BN, NACC, ACT, TO, 2>(grid, mw, mx, a, stream);
    return launch_on<BN, NACC, ACT, TO, 1>(grid, mw, mx, a, stream);
  }
  // bound by the products: one block per SM walks the tiles
  dim3 grid((unsigned)(tiles < sms ? tiles : sms), 1, splits);
  return launch_on<BN, NACC, ACT, TO, 1>(grid, mw, mx, a, stream);
}

template <int NACC, int ACT, typename TO>
int launch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, long long rows, int splits,
              int per_sm, cudaStream_t s) {
  switch (bn) {
    case 16: return launch<16, NACC, ACT, TO>(mw, mx, a, rows, splits, per_sm, s);
    case 32: return launch<32, NACC, ACT, TO>(mw, mx, a, rows, splits, per_sm, s);
    case 64: return launch<64, NACC, ACT, TO>(mw, mx, a, rows, splits, per_sm, s);
    case 128: return launch<128, NACC, ACT, TO>(mw, mx, a, rows, splits, per_sm, s);
    case 256: return launch<256, NACC, ACT, TO>(mw, mx, a, rows, splits, per_sm, s);
  }
  return af_fail(-1, "gemm_tc: token tile %d", bn);
}

template <typename TO>
int launch_variant(int nacc, int gated, int act, int bn, const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a,
                   long long rows, int splits, int per_sm, cudaStream_t s) {
  if (gated && act == AF_ACT_GELU_TANH) {
    if (nacc == 2) return launch_bn<2, AF_ACT_GELU_TANH, TO>(bn, mw, mx, a, rows, 1, per_sm, s);
    return launch_bn<1, AF_ACT_GELU_TANH, TO>(bn, mw, mx, a, rows, 1, per_sm, s);
  }
  if (gated) {
    if (nacc == 2) return launch_bn<2, AF_ACT_SILU, TO>(bn, mw, mx, a, rows, 1, per_sm, s);
    return launch_bn<1, AF_ACT_SILU, TO>(bn, mw, mx, a, rows, 1, per_sm, s);
  }
  if (nacc == 2) return launch_bn<2, -1, TO>(bn, mw, mx, a, rows, splits, per_sm, s);
  return launch_bn<1, -1, TO>(bn, mw, mx, a, rows, splits, per_sm, s);
}

// Tensor maps of the two operands and the checks both entry points share.
int prepare(CUtensorMap* mw, CUtensorMap* mx, const char* who, const void* x, long long ldx, const void* w, long long ldw,
            long long n_w_rows, int M, int K, int splits, int* kb_per_split, int* bn) {
  AF_REQUIRE(M > 0 && n_w_rows > 0 && K > 0, "%s: bad sizes %d %lld %d", who, M, n_w_rows, K);
  AF_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "%s: K %d and row strides must be multiples of 8", who, K);
  AF_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "%s: operands must be 16-byte aligned", who);
  const int total_kb = (K + TC_BK - 1) / TC_BK;
  AF_REQUIRE(splits >= 1 && splits <= total_kb, "%s: %d splits of %d K blocks", who, splits, total_kb);
  *kb_per_split = (total_kb + splits - 1) / splits;
  AF_REQUIRE((splits - 1) * *kb_per_split < total_kb, "%s: an empty K split", who);
  *bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  int rc = af_make_map_bf16(mw, w, n_w_rows, K, ldw, TC_BM);
  if (rc) return rc;
  return af_make_map_bf16(mx, x, M, K, ldx, *bn);
}

}  // namespace

// The token tile the kernel uses for M rows.
AF_EXPORT int af_gemm_tc_token_tile(int M) {
  return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
}

// out = x w^T on the tensor cores.  x [M, K] and w [n_w_rows, K] bfloat16 with
// dense rows (strides ldx, ldw elements, multiples of 8; bases 16-byte
// aligned).  gated == 0: N = n_w_rows output features.  gated != 0: w holds,
// in every group of 32 rows, 16 gate rows followed by the up rows of the same
// 16 features, N = n_w_rows / 2, and out[m, f] = act(x . gate_f) * (x . up_f).
// n_acc: 1 or 2 weight tiles per block.  splits > 1: out is float [splits, M,
// N] partial sums (part_stride elements apart) and out_dtype must be AF_F32.
// per_sm (weight-bound products of up to 64 tokens only): 2 gives a block half an SM's shared memory, so that the
// blocks of the next product in the stream fit beside it and fetch their first weight tiles while this one still
// runs; 1 gives it the whole SM; 0 chooses (2 for grids of more than one wave).
// err: device word set to 1 when a wait inside the kernel ran out of time.
AF_EXPORT int af_gemm_tc(void* out, int out_dtype, long long ldo, long long part_stride, const void* x,
                         long long ldx, const void* w, long long ldw, long long n_w_rows, int M, int K, int gated,
                         int act, int n_acc, float cap, int splits, int per_sm, int* err, cudaStream_t stream) {
  if (M == 0 || n_w_rows == 0) return 0;
  AF_REQUIRE(M > 0 && n_w_rows > 0 && K > 0, "af_gemm_tc: bad sizes %d %lld %d", M, n_w_rows, K);
  AF_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "af_gemm_tc: K %d and row strides must be multiples of 8", K);
  AF_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "af_gemm_tc: operands must be 16-byte aligned");
  AF_REQUIRE(splits >= 1 && (splits == 1 || out_dtype == AF_F32), "af_gemm_tc: split-K partial sums are float");
  AF_REQUIRE(!(gated && splits > 1), "af_gemm_tc: the gated variant does not split K");
  AF_REQUIRE(!gated || n_w_rows % 32 == 0, "af_gemm_tc: a gated weight holds whole groups of 16 + 16 rows");
  AF_REQUIRE(n_acc == 1 || n_acc == 2, "af_gemm_tc: %d accumulators", n_acc);
  AF_REQUIRE(per_sm >= 0 && per_sm <= 2, "af_gemm_tc: %d blocks per SM", per_sm);
  AF_REQUIRE(!gated || act == AF_ACT_GELU_TANH || act == AF_ACT_SILU, "af_gemm_tc: unknown activation %d", act);
  int kb_per_split = 0, bn = 0;
  CUtensorMap mw, mx;
  const int rc = prepare(&mw, &mx, "af_gemm_tc", x, ldx, w, ldw, n_w_rows, M, K, splits, &kb_per_split, &bn);
  if (rc) return rc;
  const int N = gated ? (int)(n_w_rows / 2) : (int)n_w_rows;
  TcArgs a{out, ldo, part_stride, M, N, K, kb_per_split, 0, 0, cap, err};
  if (out_dtype == AF_BF16)
    return launch_variant<__nv_bfloat16>(n_acc, gated, act, bn, mw, mx, a, n_w_rows, splits, per_sm, stream);
  return launch_variant<float>(n_acc, gated, act, bn, mw, mx, a, n_w_rows, splits, per_sm, stream);
}


// The projection of a mixer's packed rows with rotary encoding and cache write in its epilogue:
// out[M, n_w_rows] bfloat16 = rotated q heads | rotated k heads | v heads, where w [(nq + 2 nkv) hd, K] holds
// the heads' rows permuted into groups of 32 (16 rows of a head's first half, then the 16 rows hd / 2 further on;
// head_dim a multiple of 32), and out is written in the unpermuted order.  rope_table: float [M][hd / 2][2]
// (cos, sin).  kv_rows (or null: nothing is stored): int [M], the row of each token in the cache for kv head 0
// (page * nkv * 64 + row in page; -1: skip), kcache / vcache the layer's pages.  splits > 1 (up to 64 tokens
// only): parts is float [splits][M][n_w_rows] scratch, tickets int [4 * tiles] that are zero between launches.
AF_EXPORT int af_gemm_tc_rope(void* out, long long ldo, const void* x, long long ldx, const void* w, long long ldw,
                              long long n_w_rows, int M, int K, int n_acc, int splits, float* parts, int* tickets,
                              const float* rope_table, const int* kv_rows, void* kcache, void* vcache, int hd,
                              int nq, int nkv, int per_sm, int* err, cudaStream_t stream) {
  if (M == 0) return 0;
  AF_REQUIRE(hd > 0 && hd % 32 == 0 && nq > 0 && nkv > 0 && n_w_rows == (long long)(nq + 2 * nkv) * hd,
             "af_gemm_tc_rope: %lld rows are not (%d + 2 x %d) heads of %d (a multiple of 32)", n_w_rows, nq, nkv, hd);
  AF_REQUIRE(rope_table != nullptr && ((uintptr_t)rope_table & 7) == 0, "af_gemm_tc_rope: the table of cosines and sines");
  AF_REQUIRE(kv_rows == nullptr || (kcache != nullptr && vcache != nullptr), "af_gemm_tc_rope: cache pages");
  AF_REQUIRE(n_acc == 1 || n_acc == 2, "af_gemm_tc_rope: %d accumulators", n_acc);
  AF_REQUIRE(per_sm >= 0 && per_sm <= 2, "af_gemm_tc_rope: %d blocks per SM", per_sm);
  AF_REQUIRE(splits == 1 || (M <= 64 && n_acc == 1 && parts != nullptr && tickets != nullptr),
             "af_gemm_tc_rope: split-K serves up to 64 tokens and needs scratch and tickets");
  int kb_per_split = 0, bn = 0;
  CUtensorMap mw, mx;
  const int rc = prepare(&mw, &mx, "af_gemm_tc_rope", x, ldx, w, ldw, n_w_rows, M, K, splits, &kb_per_split, &bn);
  if (rc) return rc;
  TcArgs a{out, ldo, (long long)M * n_w_rows, M, (int)n_w_rows, K, kb_per_split, 0, 0, 0.f, err};
  a.rope_table = reinterpret_cast<const float2*>(rope_table);
  a.kv_rows = kv_rows;
  a.kcache = (__nv_bfloat16*)kcache;
  a.vcache = (__nv_bfloat16*)vcache;
  a.hd = hd;
  a.nq = nq;
  a.nkv = nkv;
  a.parts = parts;
  a.tickets = tickets;
  if (n_acc == 2) return launch_bn<2, -2, __nv_bfloat16>(bn, mw, mx, a, n_w_rows, splits, per_sm, stream);
  return launch_bn<1, -2, __nv_bfloat16>(bn, mw, mx, a, n_w_rows, splits, per_sm, stream);
}

// The head of greedy decoding: keys[m * AF_KEY_STRIDE] = max over the rows n of (softcap(x[m] . w[n]), n) as a 64-bit key (see
// the ARGMAX epilogue); keys must be zero before the call; af_argmax_finish turns them into token ids and
// zeroes them again.
AF_EXPORT int af_gemm_tc_argmax(unsigned long long* keys, const void* x, long long ldx, const void* w, long long ldw,
                                long long n_w_rows, int M, int K, float cap, int per_sm, int* err,
                                cudaStream_t stream) {
  if (M == 0) return 0;
  AF_REQUIRE(keys != nullptr && ((uintptr_t)keys & 7) == 0, "af_gemm_tc_argmax: keys");
  AF_REQUIRE(n_w_rows < 0xffffffffll, "af_gemm_tc_argmax: %lld rows", n_w_rows);
  AF_REQUIRE(per_sm >= 0 && per_sm <= 2, "af_gemm_tc_argmax: %d blocks per SM", per_sm);
  int kb_per_split = 0, bn = 0;
  CUtensorMap mw, mx;
  const int rc = prepare(&mw, &mx, "af_gemm_tc_argmax", x, ldx, w, ldw, n_w_rows, M, K, 1, &kb_per_split, &bn);
  if (rc) return rc;
  TcArgs a{nullptr, 0, 0, M, (int)n_w_rows, K, kb_per_split, 0, 0, cap, err};
  a.keys = keys;
  return launch_bn<1, -3, float>(bn, mw, mx, a, n_w_rows, 1, per_sm, stream);
}

// How many tickets af_gemm_tc_rope needs for these sizes.
AF_EXPORT int af_gemm_tc_rope_tickets(int M, long long n_w_rows) {
  const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  return (int)(4 * ((n_w_rows + TC_BM - 1) / TC_BM) * ((M + bn - 1) / bn));
}
