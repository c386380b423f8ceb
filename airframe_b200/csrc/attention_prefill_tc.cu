// Prefill attention on tcgen05: prompts that start at position 0, bfloat16,
// causal with an optional window, softcapped scores, grouped heads, sequences
// of unequal lengths packed row after row.
//
// A block owns 128 query rows of one head of one sequence (the 128 TMEM lanes).
//   S = Q K^T   tcgen05.mma, Q and the K tile K-major in 128-byte swizzled shared
//               memory (TMA), S (128 x 64, float) in TMEM, two S buffers so that
//               the next tile's scores are computed while this tile's softmax runs
//   softmax     eight warps, two threads a query row (32 keys each): tcgen05.ld of
//               their part of the S row, scale, softcap, mask, running maximum
//               (shared through shared memory) and sum in 32 bits; P is rounded
//               to bfloat16 and written to swizzled shared memory
//   O += P V    tcgen05.mma, P K-major, the V tile MN-major as TMA wrote it,
//               O (128 x head_dim, float) in TMEM for the whole block
// The running maximum only moves when it grows by more than 8 (in base-2
// exponent units): then O is rescaled in TMEM; otherwise P is computed against
// the older maximum (bounded by 2^8), which changes no result.
//
//   warp 0      TMA producer of Q and K    warp 1      MMA issue, TMEM allocation
//   warps 2..9  softmax, O rescale, epilogue   warp 10  TMA producer of V
// Every mbarrier wait is bounded in time; a wait that runs out sets the error
// word, and the block releases its TMEM and returns.
#include "umma.cuh"

namespace {

constexpr int TA_BM = 128;  // query rows per block
constexpr int TA_BN = 64;   // keys per tile
constexpr int TA_PARTS = 4;      // threads per query row in the softmax (16 keys each)
constexpr int TA_THREADS = (2 + 4 * TA_PARTS + 1) * 32;  // Q/K producer, MMA, softmax warps, V producer
constexpr float TA_LOG2E = 1.4426950408889634f;
constexpr float TA_RESCALE = 8.f;  // the maximum moves only when it grows by more than this

__device__ __forceinline__ float ta_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ta_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct TaArgs {
  __nv_bfloat16* out;
  long long out_stride;
  const int* seq_starts;
  int nq, nkv;
  float scale, cap;
  int window;
  int* err;
};

template <int HD>
__global__ void __launch_bounds__(TA_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, TaArgs a) {
  constexpr int SUB = HD / 64;                       // 64-column sub-tiles of a head
  constexpr int Q_SUB = TA_BM * 128;                 // bytes of one Q sub-tile [128 rows][128 B]
  constexpr int KV_SUB = TA_BN * 128;                // bytes of one K or V sub-tile [64 rows][128 B]
  constexpr int Q_BYTES = SUB * Q_SUB, KV_BYTES = SUB * KV_SUB;
  constexpr int P_BYTES = TA_BM * TA_BN * 2;         // [128 rows][64 keys] bfloat16 = one swizzled sub-tile
  constexpr int O_COL = 2 * TA_BN;                   // TMEM columns: S0 [0,64) S1 [64,128) O [128, 128 + HD)
  constexpr int COLS = 512;
  constexpr uint32_t IDESC_S = umma_idesc(TA_BN, false);
  constexpr uint32_t IDESC_O = umma_idesc(HD, true);

  extern __shared__ unsigned char ta_raw[];
  unsigned char* sm = (unsigned char*)(((uintptr_t)ta_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = sm;
  unsigned char* kv_s = sm + Q_BYTES;                // [stage][K tile | V tile]
  unsigned char* p_s = kv_s + 4 * KV_BYTES;
  __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full, p_empty, o_full, x_full;
  __shared__ float mx_s[2][TA_PARTS][TA_BM], l_s[TA_PARTS][TA_BM];
  __shared__ uint32_t tmem_base_s;
  __shared__ int give_up_s;
  volatile int* give_up = &give_up_s;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.y, head = blockIdx.z;
  const int kvh = head / (a.nq / a.nkv);

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 128 * TA_PARTS);
    }
    mbar_init(&p_full, 128 * TA_PARTS);
    mbar_init(&x_full, 128 * TA_PARTS);
    mbar_init(&p_empty, 1);
    mbar_init(&o_full, 1);
    give_up_s = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  pdl_wait();
  const int row0 = a.seq_starts[seq];
  const int len = a.seq_starts[seq + 1] - row0;
  // heavy tiles (late queries see many keys) are scheduled first
  const int m0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * TA_BM;
  const bool active = m0 < len;
  const int m_last = min(m0 + TA_BM, len) - 1;
  const int j_lo = a.window > 0 ? max(0, m0 - a.window + 1) : 0;
  const int kb_lo = j_lo / TA_BN, kb_hi = active ? m_last / TA_BN : -1;
  const int nb = active ? kb_hi - kb_lo + 1 : 0;     // key tiles of this block

  if (warp == 0) {
    // Q, then the K tiles: a K slot is free as soon as its scores are computed,
    // well before the tile's V slot, so K and V have producers of their own
    if (lane == 0 && active) {
      mbar_expect_tx(&q_full, Q_BYTES);
#pragma unroll
      for (int c = 0; c < SUB; ++c) tma_load_2d(q_s + c * Q_SUB, &map_q, head * HD + c * 64, row0 + m0, &q_full);
      for (int j = 0; j < nb; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&k_empty[s], ((j >> 1) & 1) ^ 1, give_up)) break;
        unsigned char* st = kv_s + (size_t)s * 2 * KV_BYTES;
        mbar_expect_tx(&k_full[s], KV_BYTES);
        const int r = row0 + (kb_lo + j) * TA_BN;
#pragma unroll
        for (int c = 0; c < SUB; ++c) tma_load_2d(st + c * KV_SUB, &map_k, kvh * HD + c * 64, r, &k_full[s]);
      }
      if (*give_up) grace_period();
    }
  } else if (warp == 2 + 4 * TA_PARTS) {
    if (lane == 0 && active) {
      for (int j = 0; j < nb; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&v_empty[s], ((j >> 1) & 1) ^ 1, give_up)) break;
        unsigned char* st = kv_s + (size_t)s * 2 * KV_BYTES + KV_BYTES;
        mbar_expect_tx(&v_full[s], KV_BYTES);
        const int r = row0 + (kb_lo + j) * TA_BN;
#pragma unroll
        for (int c = 0; c < SUB; ++c) tma_load_2d(st + c * KV_SUB, &map_v, kvh * HD + c * 64, r, &v_full[s]);
      }
      if (*give_up) grace_period();
    }
  } else if (warp == 1) {
    if (lane == 0 && active) {
      bool ok = mbar_wait(&q_full, 0, give_up);
      auto issue_s = [&](int j) {  // S(j) = Q K(j)^T into S buffer j % 2
        const uint32_t kt = smem_u32(kv_s + (size_t)(j & 1) * 2 * KV_BYTES);
        const uint32_t qt = smem_u32(q_s);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_f16(tmem + (j & 1) * TA_BN, umma_desc(qt + (ks >> 2) * Q_SUB) + 2 * (ks & 3),
                   umma_desc(kt + (ks >> 2) * KV_SUB) + 2 * (ks & 3), IDESC_S, ks > 0 ? 1u : 0u);
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[j & 1]);    // the K tile is consumed
      };
      if (ok && nb > 0) {
        ok = mbar_wait(&k_full[0], 0, give_up);
        if (ok) {
          tc_fence_after();
          issue_s(0);
        }
      }
      for (int j = 0; j < nb && ok; ++j) {
        if (j + 1 < nb) {  // the next tile's scores, while this tile's softmax runs
          const int s = (j + 1) & 1;
          ok = mbar_wait(&k_full[s], ((j + 1) >> 1) & 1, give_up);
          if (ok && j + 1 >= 2) ok = mbar_wait(&s_empty[s], (((j + 1) >> 1) & 1) ^ 1, give_up);
          if (!ok) break;
          tc_fence_after();
          issue_s(j + 1);
        }
        ok = mbar_wait(&v_full[j & 1], (j >> 1) & 1, give_up) && mbar_wait(&p_full, j & 1, give_up);
        if (!ok) break;
        tc_fence_after();
        // O += P(j) V(j): P K-major [128 x 64 keys], V MN-major [64 keys x HD]
        const uint32_t vt = smem_u32(kv_s + (size_t)(j & 1) * 2 * KV_BYTES + KV_BYTES);
        const uint32_t pt = smem_u32(p_s);
#pragma unroll
        for (int kk = 0; kk < TA_BN / 16; ++kk)
          umma_f16(tmem + O_COL, umma_desc(pt) + 2 * kk, umma_desc_mn(vt + kk * 2048, KV_SUB), IDESC_O,
                   (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&p_empty);           // P consumed, O updated
        umma_commit(&v_empty[j & 1]);    // the V tile is consumed
      }
      if (ok) umma_commit(&o_full);
    }
  } else if (active && warp < 2 + 4 * TA_PARTS) {
    // ---- softmax warps: a thread owns a part (16 keys) of a query row's scores; the warps
    // w, w + 4, ... share the rows of TMEM lane quarter w % 4
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int i = m0 + row;                                   // this thread's query position
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const float cs = a.cap > 0.f ? a.scale / a.cap : a.scale * TA_LOG2E;
    const float cap2 = a.cap * TA_LOG2E;
    constexpr int W = TA_BN / TA_PARTS;                       // scores per thread and tile
    constexpr int OW = HD / TA_PARTS;                         // O columns per thread
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nb; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, give_up)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float s[W];
      tmem_ld16(lane_addr + (j & 1) * TA_BN + half * W, s);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&s_empty[j & 1]);                           // the S buffer may be overwritten
      const int j0 = (kb_lo + j) * TA_BN + half * W;
      const bool edge = (j0 + W - 1 > i) || (j0 + W > len) || (a.window > 0 && i - j0 >= a.window);
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < W; ++c) {
        float v = s[c] * cs;
        if (a.cap > 0.f) v = cap2 * ta_tanh(v);
        if (edge) {
          const int jj = j0 + c;
          v = (jj <= i && jj < len && (a.window <= 0 || i - jj < a.window)) ? v : -INFINITY;
        }
        s[c] = v;
        mx4[c & 3] = fmaxf(mx4[c & 3], v);
      }
      // the row's maximum over both halves
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx_s[j & 1][half][row] = mx;
      mbar_arrive(&x_full);
      if (!mbar_wait(&x_full, j & 1, give_up)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int h = 0; h < TA_PARTS; ++h) mx = fmaxf(mx, mx_s[j & 1][h][row]);
      // the reference maximum moves only when it has to
      float corr = 1.f;
      if (mx > m_ref + TA_RESCALE || m_ref == -INFINITY) {
        const float m_new = fmaxf(m_ref, mx);
        corr = m_ref == -INFINITY ? 0.f : ta_exp2(m_ref - m_new);
        m_ref = m_new;
      }
      const float ref = m_ref == -INFINITY ? 0.f : m_ref;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[W / 2];
#pragma unroll
      for (int c = 0; c < W; c += 2) {
        const float p0 = ta_exp2(s[c] - ref), p1 = ta_exp2(s[c + 1] - ref);
        __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        // the sum uses the rounded values that the product will see
        sum4[(c >> 1) & 3] += __low2float(pb) + __high2float(pb);
        packed[c / 2] = *reinterpret_cast<uint32_t*>(&pb);
      }
      l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      // P(j-1) V(j-1) must be done before O is rescaled and P's memory reused
      if (j > 0 && !mbar_wait(&p_empty, (j - 1) & 1, give_up)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll 1
        for (int c0 = 0; c0 < OW; c0 += 32) {
          float o[32];
          tmem_ld32(lane_addr + O_COL + half * OW + c0, o);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] *= corr;
          tmem_st32(lane_addr + O_COL + half * OW + c0, o);
        }
        tmem_wait_st();
      }
      // P half row into the swizzled [128 x 128 B] tile: 16-byte piece c lands at piece c ^ (row & 7)
      unsigned char* prow = p_s + row * 128;
#pragma unroll
      for (int c = 0; c < W / 8; ++c)
        *reinterpret_cast<uint4*>(prow + (((half * (W / 8) + c) ^ (row & 7)) << 4)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    // ---- epilogue: O / l -> bfloat16 (l is the sum of both halves' sums)
    if (ok && nb > 0) ok = mbar_wait(&o_full, 0, give_up);
    l_s[half][row] = l;
    if (ok && nb > 0) {
      mbar_arrive(&x_full);
      ok = mbar_wait(&x_full, nb & 1, give_up);
    }
    if (ok && nb > 0) {
      tc_fence_after();
      float lt = 0.f;
#pragma unroll
      for (int h = 0; h < TA_PARTS; ++h) lt += l_s[h][row];
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      __nv_bfloat16* dst = a.out + (size_t)(row0 + i) * a.out_stride + (size_t)head * HD + half * OW;
#pragma unroll 1
      for (int c0 = 0; c0 < OW; c0 += 32) {
        float o[32];
        tmem_ld32(lane_addr + O_COL + half * OW + c0, o);
        tmem_wait_ld();
        if (i < len) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 pb = __floats2bfloat162_rn(o[c + 2 * e] * inv, o[c + 2 * e + 1] * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&pb);
            }
            *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)COLS));
  }
  if (threadIdx.x == 0 && give_up_s && a.err) atomicExch(a.err, 1);
}

template <int HD>
int launch_ta(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TaArgs& a, int n_seqs,
              int max_len, cudaStream_t stream) {
  constexpr int smem = TA_BM * HD * 2 + 4 * TA_BN * HD * 2 + TA_BM * TA_BN * 2 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return af_fail((int)e, "af_attn_prefill_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((max_len + TA_BM - 1) / TA_BM, n_seqs, a.nq);
  af_launch(attn_prefill_tc_kernel<HD>, grid, dim3(TA_THREADS), smem, stream, mq, mk, mv, a);
  AF_CHECK_LAUNCH("af_attn_prefill_tc");
}

}  // namespace

// 1 when the tcgen05 prefill attention takes this head size.
AF_EXPORT int af_attn_prefill_tc_supported(int hd) { return hd == 128 || hd == 256 ? 1 : 0; }

// out [T, nq * hd] = attention of sequences that start at position 0 over
// their own keys, on tcgen05.  q [T, nq * hd], k and v [T, nkv * hd]:
// bfloat16 rows with the given strides (elements, multiples of 8; bases
// 16-byte aligned); n_tokens rows in all; seq_starts [n_seqs + 1].
AF_EXPORT int af_attn_prefill_tc(void* out, long long out_stride, const void* q, long long q_stride, const void* k,
                                 long long k_stride, const void* v, long long v_stride, const int* seq_starts,
                                 int n_seqs, int n_tokens, int max_len, int nq, int nkv, int hd, float scale,
                                 float cap, int window, int* err, cudaStream_t stream) {
  if (n_seqs == 0 || max_len == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "af_attn_prefill_tc: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(af_attn_prefill_tc_supported(hd), "af_attn_prefill_tc: head_dim %d (takes 128, 256)", hd);
  AF_REQUIRE(q_stride % 8 == 0 && k_stride % 8 == 0 && v_stride % 8 == 0 && out_stride % 8 == 0,
             "af_attn_prefill_tc: row strides must be multiples of 8");
  AF_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) == 0,
             "af_attn_prefill_tc: operands must be 16-byte aligned");
  AF_REQUIRE(n_seqs <= 65535 && nq <= 65535, "af_attn_prefill_tc: too many sequences or heads");
  CUtensorMap mq, mk, mv;
  int rc = af_make_map_bf16(&mq, q, n_tokens, (long long)nq * hd, q_stride, TA_BM);
  if (rc) return rc;
  rc = af_make_map_bf16(&mk, k, n_tokens, (long long)nkv * hd, k_stride, TA_BN);
  if (rc) return rc;
  rc = af_make_map_bf16(&mv, v, n_tokens, (long long)nkv * hd, v_stride, TA_BN);
  if (rc) return rc;
  TaArgs a{(__nv_bfloat16*)out, out_stride, seq_starts, nq, nkv, scale, cap, window, err};
  if (hd == 128) return launch_ta<128>(mq, mk, mv, a, n_seqs, max_len, stream);
  return launch_ta<256>(mq, mk, mv, a, n_seqs, max_len, stream);
}
