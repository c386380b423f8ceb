// Prefill attention on tcgen05: prompts that start at position 0, bfloat16,
// causal with an optional window, softcapped scores, grouped heads, sequences
// of unequal lengths packed row after row.
//
// A block owns 128 query rows of one head of one sequence (the 128 TMEM lanes)
// and walks the keys 128 at a time (two TMA tiles of 64 keys).
//   S = Q K^T   tcgen05.mma with N = 128.  Q is copied once from shared memory
//               into TMEM and is the product's A operand there (operands in
//               shared memory are fetched at some 64 bytes a cycle, and Q would
//               be half of the score product's operand bytes, step after
//               step); the pair of K tiles is K-major in 128-byte swizzled
//               shared memory, two buffers (the second is where Q arrived); S
//               (128 x 128, float) in TMEM.  The next pair's scores are computed
//               as soon as the softmax warps hold this pair's in registers.
//   softmax     two groups of eight warps, one for each 64-key half of a step,
//               two threads a query row in each (32 keys a thread): tcgen05.ld
//               of their part of the S row, scale, softcap, mask, maximum and
//               sum in 32 bits; P is rounded to bfloat16 and written to
//               swizzled shared memory.  The halves are steps of the online
//               softmax in turn: a group takes the running maximum that the
//               other group published for the half before, so that one
//               group's exponentials and stores overlap the other's maxima.
//   O += P V    tcgen05.mma, P K-major, the V tiles MN-major as TMA wrote them,
//               O (128 x head_dim, float) in TMEM for the whole block
// The running maximum only moves when it grows by more than 8 (in base-2
// exponent units): then O is rescaled in TMEM; otherwise P is computed against
// the older maximum (bounded by 2^8), which changes no result.
//
//   warp 0       TMA producer of Q and K      warp 1    issue of S = Q K^T, TMEM allocation
//   warps 2..17  softmax, O rescale, epilogue
//   warp 18      TMA producer of V            warp 19   issue of O += P V
// Every mbarrier wait is bounded in time; a wait that runs out sets the error
// word, and the block releases its TMEM and returns.
#include "umma.cuh"

namespace {

constexpr int TA_BM = 128;  // query rows per block
constexpr int TA_KT = 64;   // keys per TMA tile (a 128-byte swizzled row holds 64 of P's keys, too)
constexpr int TA_BN = 128;  // keys per step: one S product, two tiles
constexpr int TA_PARTS = 2;      // threads per query row in a softmax group (32 keys each)
constexpr int TA_SM_WARPS = 2 * 4 * TA_PARTS;   // softmax warps: two groups
constexpr int TA_THREADS = (2 + TA_SM_WARPS + 2) * 32;
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
  constexpr int K_SUB = TA_BN * 128;                 // one K sub-tile of a pair [128 keys][128 B]
  constexpr int V_SUB = TA_KT * 128;                 // one V sub-tile [64 keys][128 B]
  constexpr int Q_BYTES = SUB * Q_SUB, K_BYTES = SUB * K_SUB, V_BYTES = SUB * V_SUB;
  constexpr int P_SUB = TA_BM * 128;                 // P of 64 keys [128 rows][128 B]
  constexpr int Q_COL = TA_BN;                       // TMEM columns: S [0,128) Q [128, 128 + HD/2) O [256, 256 + HD)
  constexpr int O_COL = 256;
  constexpr int COLS = 512;
  constexpr uint32_t IDESC_S = umma_idesc(TA_BN, false);
  constexpr uint32_t IDESC_O = umma_idesc(HD, true);

  extern __shared__ __align__(1024) unsigned char sm[];
  static_assert(Q_BYTES == K_BYTES, "Q's memory becomes the second K buffer");
  unsigned char* q_s = sm;                           // Q until it is in TMEM, then K buffer 0
  unsigned char* k_s = sm;                           // [buffer][sub-tile][128 keys of the pair][128 B]: pair j in buffer (j + 1) % 2
  unsigned char* v_s = k_s + 2 * K_BYTES;            // [tile slot 0, 1][sub-tile][64 keys][128 B]
  unsigned char* p_s = v_s + 2 * V_BYTES;            // [64-key half][128 rows][128 B]
  __shared__ uint64_t q_full, q_moved, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full, s_empty, p_full[2],
      p_empty[2], o_full, x_full[2], m_ready[2], l_full;
  // the parts' maxima of a row [group][step parity][part][row] and the running maximum that a group
  // publishes [group][row]; rounded up to bfloat16 (the reference maximum may sit a little above the true one)
  __shared__ __nv_bfloat16 mx_s[2][2][TA_PARTS][TA_BM];
  __shared__ __nv_bfloat16 mref_s[2][TA_BM];
  __shared__ uint32_t tmem_base_s;
  __shared__ int give_up_s;
  volatile int* give_up = &give_up_s;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.y, head = blockIdx.z;
  const int kvh = head / (a.nq / a.nkv);

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    mbar_init(&q_moved, TA_SM_WARPS);        // one arrival a softmax warp
    mbar_init(&s_full, 1);
    mbar_init(&s_empty, TA_SM_WARPS);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&p_full[s], 4 * TA_PARTS);   // the warps of one group
      mbar_init(&x_full[s], 4 * TA_PARTS);
      mbar_init(&m_ready[s], 4 * TA_PARTS);
      mbar_init(&p_empty[s], 1);
    }
    mbar_init(&l_full, TA_SM_WARPS);
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
  const int kt_lo = j_lo / TA_KT, kt_hi = active ? m_last / TA_KT : -1;
  const int n_tiles = active ? kt_hi - kt_lo + 1 : 0;   // 64-key tiles this block needs
  const int np = (n_tiles + 1) / 2;                     // steps: pairs of tiles (the last may hold one masked tile)

  if (warp == 0) {
    // Q, then the pairs of K tiles (one buffer: the next pair is fetched as soon as this pair's scores are computed)
    if (lane == 0 && active) {
      mbar_expect_tx(&q_full, Q_BYTES);
#pragma unroll
      for (int c = 0; c < SUB; ++c) tma_load_2d(q_s + c * Q_SUB, &map_q, head * HD + c * 64, row0 + m0, &q_full);
      for (int j = 0; j < np; ++j) {
        const int b = (j + 1) & 1;           // pair 0 goes beside Q, pair 1 where Q was
        if (j == 1 && !mbar_wait(&q_moved, 0, give_up)) break;
        if (j >= 2 && !mbar_wait(&k_empty[b], ((j >> 1) & 1) ^ 1, give_up)) break;
        unsigned char* kb = k_s + (size_t)b * K_BYTES;
        mbar_expect_tx(&k_full[b], K_BYTES);
        const int r = row0 + (kt_lo + 2 * j) * TA_KT;
#pragma unroll
        for (int c = 0; c < SUB; ++c) {
          // rows past the packed rows read as zeros; rows of the next sequence are masked by position
          tma_load_2d(kb + c * K_SUB, &map_k, kvh * HD + c * 64, r, &k_full[b]);
          tma_load_2d(kb + c * K_SUB + TA_KT * 128, &map_k, kvh * HD + c * 64, r + TA_KT, &k_full[b]);
        }
      }
      if (*give_up) grace_period();
    }
  } else if (warp == 2 + TA_SM_WARPS) {
    if (lane == 0 && active) {
      for (int t = 0; t < 2 * np; ++t) {
        const int s = t & 1;
        if (!mbar_wait(&v_empty[s], ((t >> 1) & 1) ^ 1, give_up)) break;
        unsigned char* st = v_s + (size_t)s * V_BYTES;
        mbar_expect_tx(&v_full[s], V_BYTES);
        const int r = row0 + (kt_lo + t) * TA_KT;
#pragma unroll
        for (int c = 0; c < SUB; ++c) tma_load_2d(st + c * V_SUB, &map_v, kvh * HD + c * 64, r, &v_full[s]);
      }
      if (*give_up) grace_period();
    }
  } else if (warp == 1) {
    if (lane == 0 && active) {
      bool ok = mbar_wait(&q_moved, 0, give_up);
      for (int j = 0; j < np && ok; ++j) {  // S(j) = Q K(j)^T
        const int b = (j + 1) & 1;
        ok = mbar_wait(&k_full[b], (j >> 1) & 1, give_up);
        // once the softmax warps hold the scores of the step before in registers
        if (ok && j >= 1) ok = mbar_wait(&s_empty, (j - 1) & 1, give_up);
        if (!ok) break;
        tc_fence_after();
        const uint32_t kt = smem_u32(k_s + (size_t)b * K_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_f16_ts(tmem, tmem + Q_COL + ks * 8, umma_desc(kt + (ks >> 2) * K_SUB) + 2 * (ks & 3), IDESC_S,
                      ks > 0 ? 1u : 0u);
        umma_commit(&s_full);
        umma_commit(&k_empty[b]);          // the pair of K tiles is consumed
      }
    }
  } else if (warp == 3 + TA_SM_WARPS) {
    // ---- O += P(j) V(j), issued by a thread of its own: the tensor pipe takes the
    // instructions of both issuing threads as they come
    if (lane == 0 && active) {
      bool ok = true;
      for (int j = 0; j < np && ok; ++j) {
#pragma unroll
        for (int h = 0; h < 2 && ok; ++h) {
          const int t = 2 * j + h;
          ok = mbar_wait(&p_full[h], j & 1, give_up) && mbar_wait(&v_full[t & 1], (t >> 1) & 1, give_up);
          if (!ok) break;
          tc_fence_after();
          // P K-major [128 x 64 keys], V MN-major [64 keys x HD]
          const uint32_t vt = smem_u32(v_s + (size_t)(t & 1) * V_BYTES);
          const uint32_t pt = smem_u32(p_s + h * P_SUB);
#pragma unroll
          for (int kk = 0; kk < TA_KT / 16; ++kk)
            umma_f16(tmem + O_COL, umma_desc(pt) + 2 * kk, umma_desc_mn(vt + kk * 2048, V_SUB), IDESC_O,
                     (t > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&v_empty[t & 1]);    // the V tile is consumed
          umma_commit(&p_empty[h]);        // this half's P is consumed, O updated
        }
      }
      if (ok) umma_commit(&o_full);
    }
  } else if (active && warp < 2 + TA_SM_WARPS) {
    // ---- softmax warps.  Group g (warps 2 + 8 g ..) owns the keys [64 g, 64 g + 64) of every step; in a
    // group a thread owns 32 keys of a query row; the warps w, w + 4, ... share the rows of TMEM lane
    // quarter w % 4.  The half-steps (j, 0), (j, 1), (j + 1, 0), ... are the steps of the online softmax.
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 3;
    const int part = ((warp - 2) >> 2) & 1;
    const int row = quarter * 32 + lane;
    const int i = m0 + row;                                   // this thread's query position
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const float cs = a.cap > 0.f ? a.scale / a.cap : a.scale * TA_LOG2E;
    const float cap2 = a.cap * TA_LOG2E;
    constexpr int W = TA_KT / TA_PARTS;                       // scores per thread and step
    static_assert(W == 32, "a thread reads its scores with one 32-column load");
    constexpr int RW = HD / TA_PARTS;                         // O columns a thread rescales (its group alone)
    float m_known = -INFINITY, l = 0.f;                       // this thread's sum is relative to m_known
    const int quad = grp * TA_PARTS + part;                   // this thread among the row's four
    bool ok = mbar_wait(&q_full, 0, give_up);
    if (ok) {
      // ---- Q from shared memory into TMEM: this thread's quarter of its row, 16-byte pieces
      // un-swizzled, two elements a column
      constexpr int QW = HD / 8;                              // 32-bit columns per thread
      const int e0 = quad * (HD / 4);                         // first element of this thread's share
      const unsigned char* qrow = q_s + (e0 >> 6) * Q_SUB + row * 128;
      const int p0 = (e0 & 63) >> 3;                          // first 16-byte piece within the 128-byte row
      uint32_t w[QW];
#pragma unroll
      for (int c = 0; c < QW / 4; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(qrow + (((p0 + c) ^ (row & 7)) << 4));
        w[4 * c] = v.x, w[4 * c + 1] = v.y, w[4 * c + 2] = v.z, w[4 * c + 3] = v.w;
      }
      if constexpr (QW == 32) {
        tmem_st32(lane_addr + Q_COL + quad * QW, reinterpret_cast<const float*>(w));
      } else {
        tmem_st16(lane_addr + Q_COL + quad * QW, reinterpret_cast<const float*>(w));
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_moved);
    }
    for (int j = 0; j < np && ok; ++j) {
      if (!mbar_wait(&s_full, j & 1, give_up)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float s[W];
      tmem_ld32(lane_addr + grp * TA_KT + part * W, s);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty);                   // the S buffer may be overwritten
      const int j0 = (kt_lo + 2 * j + grp) * TA_KT + part * W;
      const bool edge = (j0 + W - 1 > i) || (j0 + W > len) || (a.window > 0 && i - j0 >= a.window);
      // (the tests on the cap and on the edge stand outside the loops: inside, the compiler kept
      // them as a branch per element)
      if (a.cap > 0.f) {
#pragma unroll
        for (int c = 0; c < W; ++c) s[c] = cap2 * ta_tanh(s[c] * cs);
      } else {
#pragma unroll
        for (int c = 0; c < W; ++c) s[c] *= cs;
      }
      if (edge) {
        const int hi = min(i, len - 1) - j0;                       // last visible key of this part
        const int lo = a.window > 0 ? i - a.window + 1 - j0 : -1;  // first visible key
#pragma unroll
        for (int c = 0; c < W; ++c) s[c] = (c <= hi && c >= lo) ? s[c] : -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < W; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
      // the row's maximum over this half's parts
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx_s[grp][j & 1][part][row] = __float2bfloat16_ru(mx);
      __syncwarp();
      if (lane == 0) mbar_arrive(&x_full[grp]);
      if (!mbar_wait(&x_full[grp], j & 1, give_up)) {
        ok = false;
        break;
      }
      mx = fmaxf(__bfloat162float(mx_s[grp][j & 1][0][row]), __bfloat162float(mx_s[grp][j & 1][1][row]));
      // the running maximum after the half-step before this one, published by the other group
      float m_prev = -INFINITY;
      if (grp == 1 || j > 0) {
        if (!mbar_wait(&m_ready[grp ^ 1], grp == 1 ? (j & 1) : ((j - 1) & 1), give_up)) {
          ok = false;
          break;
        }
        m_prev = __bfloat162float(mref_s[grp ^ 1][row]);
      }
      // it moves only when it has to
      float m_new = m_prev;
      if (mx > m_prev + TA_RESCALE || m_prev == -INFINITY) m_new = fmaxf(m_prev, mx);
      if (part == 0) mref_s[grp][row] = __float2bfloat16_ru(m_new);   // (exact: both are bfloat16 values)
      __syncwarp();
      if (lane == 0) mbar_arrive(&m_ready[grp]);              // read the other group's, wrote ours
      const float ref = m_new == -INFINITY ? 0.f : m_new;
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
      l = l * (m_known == -INFINITY ? 0.f : ta_exp2(m_known - ref)) + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      m_known = m_new;
      // This group's P of the step before must be consumed before its memory is reused.  (Waited for
      // here, ahead of the wait below: it also pins the phase that wait looks at.)
      if (j > 0 && !mbar_wait(&p_empty[grp], (j - 1) & 1, give_up)) {
        ok = false;
        break;
      }
      const bool first = j == 0 && grp == 0;                  // no product has been issued yet
      if (!first && __any_sync(0xffffffffu, m_new != m_prev)) {
        // O is rescaled by this group alone, once the product of the half-step before is complete
        // (products complete in order; the next one waits for this group's P)
        if (!mbar_wait(&p_empty[grp ^ 1], grp == 1 ? (j & 1) : ((j - 1) & 1), give_up)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const float corr = m_prev == -INFINITY ? 0.f : ta_exp2(m_prev - ref);
#pragma unroll 1
        for (int c0 = 0; c0 < RW; c0 += 32) {
          float o[32];
          tmem_ld32(lane_addr + O_COL + part * RW + c0, o);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] *= corr;
          tmem_st32(lane_addr + O_COL + part * RW + c0, o);
        }
        tmem_wait_st();
      }
      // The thread's 32 keys are half a row of the swizzled [128 x 128 B] tile of its group's 64 keys:
      // 16-byte piece c of the row lands at piece c ^ (row & 7)
      unsigned char* prow = p_s + grp * P_SUB + row * 128;
#pragma unroll
      for (int c = 0; c < W / 8; ++c)
        *reinterpret_cast<uint4*>(prow + (((part * (W / 8) + c) ^ (row & 7)) << 4)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[grp]);
    }
    // ---- epilogue: O / l -> bfloat16; l is the sum of the four threads' sums, brought to the last maximum
    if (ok && np > 0) ok = mbar_wait(&m_ready[1], (np - 1) & 1, give_up);
    if (ok && np > 0) ok = mbar_wait(&o_full, 0, give_up);
    float* l_s = reinterpret_cast<float*>(p_s);               // [thread of the row][row]: P is free once O is complete
    if (ok && np > 0) {
      const float m_fin = __bfloat162float(mref_s[1][row]);
      l_s[quad * TA_BM + row] =
          (m_known == -INFINITY || m_fin == -INFINITY) ? 0.f : l * ta_exp2(m_known - m_fin);
      __syncwarp();
      if (lane == 0) mbar_arrive(&l_full);
      ok = mbar_wait(&l_full, 0, give_up);
    }
    if (ok && np > 0) {
      tc_fence_after();
      constexpr int OW = HD / (2 * TA_PARTS);                 // O columns a thread writes out
      float lt = 0.f;
#pragma unroll
      for (int h = 0; h < 2 * TA_PARTS; ++h) lt += l_s[h * TA_BM + row];
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      __nv_bfloat16* dst = a.out + (size_t)(row0 + i) * a.out_stride + (size_t)head * HD + quad * OW;
#pragma unroll 1
      for (int c0 = 0; c0 < OW; c0 += 32) {
        float o[32];
        tmem_ld32(lane_addr + O_COL + quad * OW + c0, o);
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
  constexpr int smem = 2 * TA_BN * HD * 2 + 2 * TA_KT * HD * 2 + TA_BM * TA_BN * 2;  // two K pairs (Q arrives in one), two V tiles, P
  // (the limit on dynamic shared memory is a device's: set once on each)
  static bool configured[AF_MAX_DEVICES] = {};
  const int dev__ = af_current_device();
  if (dev__ < 0) return -1;
  if (!configured[dev__]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return af_fail((int)e, "af_attn_prefill_tc: %s", cudaGetErrorString(e));
    configured[dev__] = true;
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
  rc = af_make_map_bf16(&mk, k, n_tokens, (long long)nkv * hd, k_stride, TA_KT);
  if (rc) return rc;
  rc = af_make_map_bf16(&mv, v, n_tokens, (long long)nkv * hd, v_stride, TA_KT);
  if (rc) return rc;
  TaArgs a{(__nv_bfloat16*)out, out_stride, seq_starts, nq, nkv, scale, cap, window, err};
  if (hd == 128) return launch_ta<128>(mq, mk, mv, a, n_seqs, max_len, stream);
  return launch_ta<256>(mq, mk, mv, a, n_seqs, max_len, stream);
}
