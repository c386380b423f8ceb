// The prefill matrix product on pairs of SMs:  out[M, N] = x[M, K] * w[N, K]^T  (bfloat16, 32-bit sums).
//
// Two blocks (a cluster of two, on neighbouring SMs) work on one tile of 256 weight rows by 256 tokens
// with tcgen05.mma.cta_group::2: each block loads its own 128 weight rows (the "A" operand, the TMEM
// lanes of its own accumulator) and its own 128 of the 256 tokens (half of the "B" operand); the tensor
// cores of both SMs read both halves.  Against one block that does 256 x 256 alone this halves the
// operand bytes a block stages per product and leaves each SM an accumulator of 256 TMEM columns, so
// there is room for two: while the epilogue warps read one tile's accumulator back and store it, the
// products of the next tile already run into the other.
//
//   warp 0      TMA producer (one lane), in both blocks: own weight rows, own tokens
//   warp 1      TMEM allocation (both blocks); MMA issue by one lane of the leader (rank 0) for the pair
//   warps 2..5  epilogue of the block's own 128 rows: TMEM -> registers -> global
//
// Barriers.  full[s] lives in the leader: its producer expects the bytes of both blocks, both blocks'
// copies complete on it.  empty[s] and acc_full[b] are signalled in both blocks at once by the leader's
// tcgen05.commit (multicast to the pair).  acc_empty[b] lives in the leader and counts the epilogue
// warps of both blocks.  No copy is multicast.  Every wait is bounded in time (a wait that runs out
// sets the error word); the two blocks meet at a cluster barrier before they release TMEM and leave,
// so neither signals into the shared memory of a block that is gone.
//
// Epilogues: plain (bfloat16 or float out, optional cap), or gated (weight rows in groups of 16 gate +
// 16 up rows, out = act(g) * u), as in gemm_tc.cu.
#include "umma.cuh"

namespace {

constexpr int TP_BM = 128;        // weight rows per block
constexpr int TP_BN = 256;        // tokens per pair
constexpr int TP_BK = 64;
constexpr int TP_THREADS = 192;
constexpr int TP_A_BYTES = TP_BM * TP_BK * 2;
constexpr int TP_B_BYTES = (TP_BN / 2) * TP_BK * 2;
constexpr int TP_STAGE_BYTES = TP_A_BYTES + TP_B_BYTES;
constexpr int TP_STAGES = 6;
constexpr int TP_SMEM = TP_STAGES * TP_STAGE_BYTES + 1024;

struct TpArgs {
  void* out;
  long long ldo;
  int M, N, K;
  int tiles_w, tiles_m;   // tiles of 256 weight rows and of 256 tokens; pair p walks p, p + pairs, ... (token tile fastest)
  float cap;
  int* err;
  int group;              // the order in which the pairs walk the tiles (af_tile_of)
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared window, of the variable at `addr` of this block in the block of rank `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tiled copy whose completion is counted on a barrier that may lie in the other block of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrives, once the pair's earlier products are done, on the barrier at this offset in both blocks.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// M = 256 over the pair, N = bn; both operands K-major
__host__ __device__ constexpr uint32_t umma_idesc_pair(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

__device__ __forceinline__ float tp_act(float g, int act) {
  if (act == AF_ACT_GELU_TANH) {
    const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    return 0.5f * g * (1.f + t);
  }
  return g / (1.f + __expf(-g));
}

template <int ACT, typename TO>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TP_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TpArgs a) {
  constexpr bool GATED = ACT >= 0;
  constexpr uint32_t IDESC = umma_idesc_pair(TP_BN);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[TP_STAGES], empty[TP_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int give_up_s;
  volatile int* give_up = &give_up_s;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int kb_count = (a.K + TP_BK - 1) / TP_BK;
  const int n_tiles = a.tiles_w * a.tiles_m;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TP_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);   // four epilogue warps in each of the two blocks
    }
    give_up_s = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // the other block's barriers exist before anything is signalled into them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      // the K blocks of all tiles of this pair form one sequence `it` through the ring of stages
      const int my_tiles = pair < n_tiles ? (n_tiles - pair + n_pairs - 1) / n_pairs : 0;
      const int total = my_tiles * kb_count;
      // The two streams of copies (weights, activations) each walk the tiles' K blocks in order; where a stream
      // is in its walk is counted on, not divided out stage by stage (this thread has a stage's copies to send
      // in the time its products take).
      struct Walk {
        int kb, tile, wt, mt;
      };
      auto begin = [&](Walk& w) {
        w.kb = 0;
        w.tile = pair;
        w.wt = w.mt = 0;
        if (w.tile < n_tiles) af_tile_of(w.tile, a.tiles_w, a.tiles_m, a.group, &w.wt, &w.mt);
      };
      auto step = [&](Walk& w) {
        if (++w.kb == kb_count) {
          w.kb = 0;
          w.tile += n_pairs;
          if (w.tile < n_tiles) af_tile_of(w.tile, a.tiles_w, a.tiles_m, a.group, &w.wt, &w.mt);
        }
      };
      Walk ww, wx;
      begin(ww);
      begin(wx);
      auto load_w = [&](int it) {
        const int n0 = ww.wt * (2 * TP_BM) + (int)rank * TP_BM;
        tma_load_2d_pair(tiles + (size_t)(it % TP_STAGES) * TP_STAGE_BYTES, &map_w, ww.kb * TP_BK, n0,
                         map_to_rank(smem_u32(&full[it % TP_STAGES]), 0));
        step(ww);
      };
      auto load_x = [&](int it) {
        const int m0 = wx.mt * TP_BN + (int)rank * (TP_BN / 2);
        tma_load_2d_pair(tiles + (size_t)(it % TP_STAGES) * TP_STAGE_BYTES + TP_A_BYTES, &map_x, wx.kb * TP_BK,
                         m0, map_to_rank(smem_u32(&full[it % TP_STAGES]), 0));
        step(wx);
      };
      // The weights do not depend on the kernel in front: the first stages' weight tiles go out before the
      // wait for it, the activations after it.
      const int early = total < TP_STAGES ? total : TP_STAGES;
      for (int it = 0; it < early; ++it) {
        if (leader) mbar_expect_tx(&full[it], 2 * TP_STAGE_BYTES);
        load_w(it);
      }
      pdl_wait();
      for (int it = 0; it < early; ++it) load_x(it);
      for (int it = early; it < total; ++it) {
        const int s = it % TP_STAGES;
        const uint32_t ph = (it / TP_STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, give_up)) break;
        if (leader) mbar_expect_tx(&full[s], 2 * TP_STAGE_BYTES);
        load_w(it);
        load_x(it);
      }
      if (*give_up) grace_period();
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      bool ok = true;
      int it = 0, round = 0;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++round) {
        const int buf = round & 1;
        // the accumulator is free once the epilogue warps of both blocks have read the tile two rounds back
        if (round >= 2 && !mbar_wait(&acc_empty[buf], ((round >> 1) - 1) & 1, give_up)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < kb_count; ++kb, ++it) {
          const int s = it % TP_STAGES;
          const uint32_t ph = (it / TP_STAGES) & 1;
          if (!mbar_wait(&full[s], ph, give_up)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t st = smem_u32(tiles + (size_t)s * TP_STAGE_BYTES);
          const uint64_t da = umma_desc(st), db = umma_desc(st + TP_A_BYTES);
#pragma unroll
          for (int k = 0; k < TP_BK / 16; ++k)
            umma_f16_pair(tmem_base + buf * TP_BN, da + 2 * k, db + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s]);
        }
        if (ok) umma_commit_pair(&acc_full[buf]);
      }
    }
  } else {
    const int quarter = warp & 3;
    pdl_wait();
    const uint32_t acc_empty_leader[2] = {map_to_rank(smem_u32(&acc_empty[0]), 0), map_to_rank(smem_u32(&acc_empty[1]), 0)};
    int round = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++round) {
      const int buf = round & 1;
      int wt2, mt;
      af_tile_of(tile, a.tiles_w, a.tiles_m, a.group, &wt2, &mt);
      const int wt = wt2 * 2 + (int)rank;                      // this block's tile of 128 weight rows
      const int m0 = mt * TP_BN;
      if (!mbar_wait(&acc_full[buf], (round >> 1) & 1, give_up)) break;
      tc_fence_after();
      TO* out = reinterpret_cast<TO*>(a.out);
      const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TP_BN;
      const int f = GATED ? wt * 64 + quarter * 16 + (lane & 15) : wt * TP_BM + quarter * 32 + lane;
      constexpr int CW = 64;
#pragma unroll 1
      for (int c0 = 0; c0 < TP_BN; c0 += CW) {
        float v[CW];
        tmem_ld32(lane_base + c0, v);
        tmem_ld32(lane_base + c0 + 32, v + 32);
        tmem_wait_ld();
        if (c0 + CW >= TP_BN) {
          // all of this tile is in registers: its accumulator may be written again
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc_empty_leader[buf]);
        }
        if (GATED) {
          // lanes 0..15 hold gate rows, lanes 16..31 the up rows of the same 16 features: each half keeps one
          // half of the round's tokens and gets the partner's values for them with one shuffle per token
          const int low = lane < 16 ? 1 : 0;
#pragma unroll
          for (int j = 0; j < CW / 2; ++j) {
            const float got = __shfl_xor_sync(0xffffffffu, pick(low, v[j + CW / 2], v[j]), 16);
            const float g = pick(low, v[j], got), u = pick(low, got, v[j + CW / 2]);
            v[j] = tp_act(g, ACT) * u;
          }
          const int tok0 = m0 + c0 + (lane < 16 ? 0 : CW / 2);
          if (f < a.N) {
            TO* o = out + (size_t)tok0 * a.ldo + f;
#pragma unroll
            for (int j = 0; j < CW / 2; ++j)
              if (tok0 + j < a.M) o[(size_t)j * a.ldo] = from_f32<TO>(v[j]);
          }
        } else {
          if (a.cap > 0.f) {
#pragma unroll
            for (int j = 0; j < CW; ++j) v[j] = a.cap * tanhf(v[j] / a.cap);
          }
          if (f < a.N) {
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
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // nothing of either block is in flight towards the other any more
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u));
  }
  if (threadIdx.x == 0 && give_up_s && a.err) atomicExch(a.err, 1);
}

template <int ACT, typename TO>
int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, TpArgs a, long long n_w_rows, cudaStream_t stream) {
  static bool configured[AF_MAX_DEVICES] = {};
  const int dev = af_current_device();
  if (dev < 0) return -1;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<ACT, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM);
    if (e != cudaSuccess) return af_fail((int)e, "af_gemm_tc_pair: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  a.tiles_w = (int)((n_w_rows + 2 * TP_BM - 1) / (2 * TP_BM));
  a.tiles_m = (a.M + TP_BN - 1) / TP_BN;
  const long long tiles = (long long)a.tiles_w * a.tiles_m;
  const int sms = af_sm_count();
  if (sms <= 0) return -1;
  const long long pairs = tiles < sms / 2 ? tiles : sms / 2;
  a.group = af_tile_group(a.tiles_m, sms / 2);
  af_launch(gemm_tc_pair_kernel<ACT, TO>, dim3((unsigned)(2 * pairs)), dim3(TP_THREADS), TP_SMEM, stream, mw, mx, a);
  AF_CHECK_LAUNCH("af_gemm_tc_pair");
}

}  // namespace

// out = x w^T on pairs of SMs (see the top of the file); meant for many tokens (prompts).  x [M, K] and
// w [n_w_rows, K] bfloat16 with dense rows (strides multiples of 8, bases 16-byte aligned).  gated != 0: w holds
// groups of 16 gate rows + 16 up rows, N = n_w_rows / 2, out = act(x . gate) * (x . up).  out: bfloat16 or float
// [M, N], rows ldo apart.  err: device word set to 1 when a wait inside the kernel ran out of time.
AF_EXPORT int af_gemm_tc_pair(void* out, int out_dtype, long long ldo, const void* x, long long ldx, const void* w,
                              long long ldw, long long n_w_rows, int M, int K, int gated, int act, float cap,
                              int* err, cudaStream_t stream) {
  if (M == 0 || n_w_rows == 0) return 0;
  AF_REQUIRE(M > 0 && n_w_rows > 0 && K > 0, "af_gemm_tc_pair: bad sizes %d %lld %d", M, n_w_rows, K);
  AF_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "af_gemm_tc_pair: K %d and row strides must be multiples of 8", K);
  AF_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "af_gemm_tc_pair: operands must be 16-byte aligned");
  AF_REQUIRE(!gated || n_w_rows % 32 == 0, "af_gemm_tc_pair: a gated weight holds whole groups of 16 + 16 rows");
  AF_REQUIRE(!gated || act == AF_ACT_GELU_TANH || act == AF_ACT_SILU, "af_gemm_tc_pair: unknown activation %d", act);
  AF_REQUIRE(!(gated && cap > 0.f), "af_gemm_tc_pair: the gated variant takes no cap");
  CUtensorMap mw, mx;
  int rc = af_make_map_bf16(&mw, w, n_w_rows, K, ldw, TP_BM);
  if (rc) return rc;
  rc = af_make_map_bf16(&mx, x, M, K, ldx, TP_BN / 2);
  if (rc) return rc;
  const int N = gated ? (int)(n_w_rows / 2) : (int)n_w_rows;
  TpArgs a{out, ldo, M, N, K, 0, 0, cap, err};
  const bool bf = out_dtype == AF_BF16;
  AF_REQUIRE(bf || out_dtype == AF_F32, "af_gemm_tc_pair: out dtype %d", out_dtype);
  if (gated && act == AF_ACT_GELU_TANH)
    return bf ? launch_pair<AF_ACT_GELU_TANH, __nv_bfloat16>(mw, mx, a, n_w_rows, stream)
              : launch_pair<AF_ACT_GELU_TANH, float>(mw, mx, a, n_w_rows, stream);
  if (gated)
    return bf ? launch_pair<AF_ACT_SILU, __nv_bfloat16>(mw, mx, a, n_w_rows, stream)
              : launch_pair<AF_ACT_SILU, float>(mw, mx, a, n_w_rows, stream);
  return bf ? launch_pair<-1, __nv_bfloat16>(mw, mx, a, n_w_rows, stream) : launch_pair<-1, float>(mw, mx, a, n_w_rows, stream);
}
