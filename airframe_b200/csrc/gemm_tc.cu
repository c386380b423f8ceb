// bfloat16 matrix product on the 5th-generation tensor cores:
//   out[M, N] = x[M, K] * w[N, K]^T      (tokens x features, weights [out, in])
//
// The weight is the tcgen05 "A" operand: a CTA owns 128 output features (the
// 128 TMEM lanes) and BN tokens (TMEM columns), so the same kernel serves
// decode (BN = 16 .. 64, bandwidth bound: the weights stream through once) and
// prefill (BN = 256).  Both operands are K-major, staged by TMA into 128-byte
// swizzled shared memory; one elected thread issues tcgen05.mma with the
// accumulator in TMEM; four warps read it back with tcgen05.ld for the epilogue.
//
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM allocation, MMA issue (one lane), TMEM release
//   warps 2..5  epilogue: TMEM -> registers -> global
//
// Variants: DUAL keeps two accumulators (rows n and up_offset + n of the weight,
// the gate and up halves of a gated feed-forward) and writes act(g) * u;
// split-K (gridDim.z > 1) writes float partial sums [split, M, N] that the
// consumer adds in order; `cap` > 0 applies cap * tanh(v / cap).
//
// Every wait on an mbarrier is bounded in time.  A wait that runs out sets an
// error word that the host reads after the launch; the CTA then lets its
// copies in flight land, releases its TMEM and returns.
#include "tma.cuh"

namespace {

constexpr int TC_BM = 128;  // features per CTA = UMMA M
constexpr int TC_BK = 64;   // K per stage: 128 bytes of bfloat16 = one swizzle row
constexpr int TC_THREADS = 192;
constexpr int TC_SMEM_BUDGET = 200 * 1024;

__host__ __device__ constexpr int tc_stage_bytes(int bn, bool dual) {
  return (dual ? 2 : 1) * TC_BM * TC_BK * 2 + bn * TC_BK * 2;
}
__host__ __device__ constexpr int tc_stages(int bn, bool dual) {
  int s = TC_SMEM_BUDGET / tc_stage_bytes(bn, dual);
  return s > 8 ? 8 : s;
}
__host__ __device__ constexpr int tc_tmem_cols(int bn, bool dual) {
  int c = dual ? 2 * bn : bn;
  return c < 32 ? 32 : c;  // bn is a power of two
}

// K-major operand tile in 128-byte swizzled rows: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// bf16 x bf16 -> f32, A and B K-major, M = 128, N = bn
__host__ __device__ constexpr uint32_t umma_idesc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

__device__ __forceinline__ float tc_act(float g, int act) {
  if (act == AF_ACT_GELU_TANH) {
    const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.f + tanhf(u));
  }
  return g / (1.f + expf(-g));
}

struct TcArgs {
  void* out;
  long long ldo;          // row stride of out in elements
  long long part_stride;  // elements between split-K partial results
  int M, N, K;
  int kb_per_split;       // K blocks handled by one z-slice
  int up_offset;          // DUAL: weight row of feature 0's second operand
  int act;
  float cap;
  int* err;
};

template <int BN, bool DUAL, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcArgs a) {
  constexpr int STAGES = tc_stages(BN, DUAL);
  constexpr int A_BYTES = TC_BM * TC_BK * 2;
  constexpr int B_BYTES = BN * TC_BK * 2;
  constexpr int STAGE_BYTES = tc_stage_bytes(BN, DUAL);
  constexpr int COLS = tc_tmem_cols(BN, DUAL);
  constexpr uint32_t IDESC = umma_idesc(BN);

  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[STAGES], empty[STAGES], acc_full;
  __shared__ uint32_t tmem_base_s;
  __shared__ int give_up_s;
  volatile int* give_up = &give_up_s;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TC_BM, m0 = blockIdx.y * BN;
  const int total_kb = (a.K + TC_BK - 1) / TC_BK;
  const int kb0 = blockIdx.z * a.kb_per_split;
  const int kb_count = min(a.kb_per_split, total_kb - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_full, 1);
    give_up_s = 0;
    mbar_fence_init();
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

  if (warp == 0) {
    if (lane == 0) {
      // The weights do not depend on earlier kernels: the first stages' weight
      // tiles are fetched before the wait for them, the activations after it.
      const int early = min(STAGES, kb_count);
      for (int kb = 0; kb < early; ++kb) {
        unsigned char* st = tiles + (size_t)kb * STAGE_BYTES;
        mbar_expect_tx(&full[kb], STAGE_BYTES);
        const int k = (kb0 + kb) * TC_BK;
        tma_load_2d(st, &map_w, k, n0, &full[kb]);
        if (DUAL) tma_load_2d(st + A_BYTES, &map_w, k, a.up_offset + n0, &full[kb]);
      }
      pdl_wait();
      for (int kb = 0; kb < early; ++kb)
        tma_load_2d(tiles + (size_t)kb * STAGE_BYTES + (DUAL ? 2 : 1) * A_BYTES, &map_x, (kb0 + kb) * TC_BK, m0,
                    &full[kb]);
      for (int kb = early; kb < kb_count; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, give_up)) break;
        unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        const int k = (kb0 + kb) * TC_BK;
        tma_load_2d(st, &map_w, k, n0, &full[s]);
        if (DUAL) tma_load_2d(st + A_BYTES, &map_w, k, a.up_offset + n0, &full[s]);
        tma_load_2d(st + (DUAL ? 2 : 1) * A_BYTES, &map_x, k, m0, &full[s]);
      }
      if (*give_up) grace_period();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < kb_count && ok; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&full[s], ph, give_up)) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t st = smem_u32(tiles + (size_t)s * STAGE_BYTES);
        const uint64_t da = umma_desc(st);
        const uint64_t db = umma_desc(st + (DUAL ? 2 : 1) * A_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k) {
          const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
          umma_f16(tmem_base, da + 2 * k, db + 2 * k, IDESC, acc);  // 32 bytes of K per step
          if (DUAL) umma_f16(tmem_base + BN, umma_desc(st + A_BYTES) + 2 * k, db + 2 * k, IDESC, acc);
        }
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(&acc_full);
    }
  } else {
    // epilogue: warp w reads TMEM lanes [32 * (w % 4), + 32)
    const int quarter = warp & 3;
    const int f = n0 + quarter * 32 + lane;
    pdl_wait();
    const bool done = mbar_wait(&acc_full, 0, give_up);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (done) {
      TO* out = reinterpret_cast<TO*>(a.out) + (size_t)blockIdx.z * a.part_stride;
      const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16], u[16];
        tmem_ld16(lane_base + c0, v);
        if (DUAL) tmem_ld16(lane_base + BN + c0, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (f < a.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m < a.M) {
              float r = v[j];
              if (DUAL) r = tc_act(r, a.act) * u[j];
              r = softcap_f32(r, a.cap);
              out[(size_t)m * a.ldo + f] = from_f32<TO>(r);
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

template <int BN, bool DUAL, typename TO>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, int splits, cudaStream_t stream) {
  constexpr int smem = tc_stages(BN, DUAL) * tc_stage_bytes(BN, DUAL) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, DUAL, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return af_fail((int)e, "gemm_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((a.N + TC_BM - 1) / TC_BM, (a.M + BN - 1) / BN, splits);
  af_launch(gemm_tc_kernel<BN, DUAL, TO>, dim3(grid), dim3(TC_THREADS), smem, stream, mw, mx, a);
  AF_CHECK_LAUNCH("af_gemm_tc");
}

template <bool DUAL, typename TO>
int launch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, int splits, cudaStream_t s) {
  switch (bn) {
    case 16: return launch<16, DUAL, TO>(mw, mx, a, splits, s);
    case 32: return launch<32, DUAL, TO>(mw, mx, a, splits, s);
    case 64: return launch<64, DUAL, TO>(mw, mx, a, splits, s);
    case 128: return launch<128, DUAL, TO>(mw, mx, a, splits, s);
    case 256: return launch<256, DUAL, TO>(mw, mx, a, splits, s);
  }
  return af_fail(-1, "gemm_tc: token tile %d", bn);
}

}  // namespace

// The token tile the kernel uses for M rows.
AF_EXPORT int af_gemm_tc_token_tile(int M) {
  return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
}

// out = x w^T on the tensor cores.  x [M, K] and w [n_w_rows, K] bfloat16 with
// dense rows (strides ldx, ldw elements, multiples of 8; bases 16-byte
// aligned).  N output features.  dual != 0: w holds 2 operands per feature,
// rows f and up_offset + f, and out = act(x w_f) * (x w_{up_offset + f}).
// splits > 1: out is float [splits, M, N] partial sums (part_stride elements
// apart) and out_dtype must be AF_F32.  err: device word set to 1 when a wait
// inside the kernel ran out of time.
AF_EXPORT int af_gemm_tc(void* out, int out_dtype, long long ldo, long long part_stride, const void* x,
                         long long ldx, const void* w, long long ldw, long long n_w_rows, int M, int N, int K,
                         int dual, int up_offset, int act, float cap, int splits, int* err,
                         cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  AF_REQUIRE(M > 0 && N > 0 && K > 0, "af_gemm_tc: bad sizes %d %d %d", M, N, K);
  AF_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "af_gemm_tc: K %d and row strides must be multiples of 8", K);
  AF_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "af_gemm_tc: operands must be 16-byte aligned");
  AF_REQUIRE(splits >= 1 && (splits == 1 || out_dtype == AF_F32), "af_gemm_tc: split-K partial sums are float");
  AF_REQUIRE(!(dual && splits > 1), "af_gemm_tc: the gated variant does not split K");
  const int total_kb = (K + TC_BK - 1) / TC_BK;
  AF_REQUIRE(splits <= total_kb, "af_gemm_tc: %d splits of %d K blocks", splits, total_kb);
  const int kb_per_split = (total_kb + splits - 1) / splits;
  AF_REQUIRE((splits - 1) * kb_per_split < total_kb, "af_gemm_tc: an empty K split");
  const int bn = af_gemm_tc_token_tile(M);
  CUtensorMap mw, mx;
  int rc = af_make_map_bf16(&mw, w, n_w_rows, K, ldw, TC_BM);
  if (rc) return rc;
  rc = af_make_map_bf16(&mx, x, M, K, ldx, bn);
  if (rc) return rc;
  TcArgs a{out, ldo, part_stride, M, N, K, kb_per_split, up_offset, act, cap, err};
  if (dual) {
    if (out_dtype == AF_BF16) return launch_bn<true, __nv_bfloat16>(bn, mw, mx, a, 1, stream);
    return launch_bn<true, float>(bn, mw, mx, a, 1, stream);
  }
  if (out_dtype == AF_BF16) return launch_bn<false, __nv_bfloat16>(bn, mw, mx, a, splits, stream);
  return launch_bn<false, float>(bn, mw, mx, a, splits, stream);
}
