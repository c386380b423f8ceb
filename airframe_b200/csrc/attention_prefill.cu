// Prefill attention for prompts that start at position 0, bfloat16, on the
// tensor cores (mma.sync m16n8k16, 32-bit accumulators): causal with an
// optional window, softcapped scores, grouped heads, sequences of unequal
// lengths packed row after row.
//
// A block owns 64 or 128 query rows of one head of one sequence; a warp owns
// 16 of them.  K and V tiles of 32 or 64 keys come through two shared-memory
// stages (cp.async, 16-byte pieces, XOR-swizzled so that ldmatrix is free of
// bank conflicts).  Scores, the running maximum, the running sum and the output
// stay in 32-bit registers (online softmax); P is rounded to bfloat16 for the
// P V product.  tanh.approx and ex2.approx serve the softcap and the softmax.
#include "common.cuh"

namespace {

// Tile shapes per head size: query rows per block (16 a warp) and keys per
// tile.  Smaller tiles for head size 256 let two blocks share an SM and spread
// the triangular work of a causal mask over more blocks.
template <int HD> struct PfShape { static constexpr int BM = 128, BN = 64; };
template <> struct PfShape<256> { static constexpr int BM = 64, BN = 32; };

__device__ __forceinline__ float pf_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float pf_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pf_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void pf_cp16(uint32_t dst, const void* src, bool on) {
  const int n = on ? 16 : 0;  // 0 bytes read: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void pf_ldm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void pf_ldm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void pf_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct PrefillArgs {
  __nv_bfloat16* out;
  long long out_stride;
  const __nv_bfloat16* q;
  long long q_stride;
  const __nv_bfloat16* k;
  long long k_stride;
  const __nv_bfloat16* v;
  long long v_stride;
  const int* seq_starts;  // [n_seqs + 1] first row of each sequence
  int nq, nkv;
  float scale, cap;
  int window;
};

// Byte offset of the 16-byte piece `c` of row `r` in a tile whose rows hold HD bfloat16.
template <int HD>
__device__ __forceinline__ uint32_t pf_off(int r, int c) {
  return (uint32_t)(r * (HD * 2) + ((c ^ (r & 7)) << 4));
}

// rows [row0, row0 + ROWS) of a [*, stride] matrix -> swizzled tile; rows >= row_end are zero
template <int HD, int ROWS>
__device__ __forceinline__ void pf_load_tile(unsigned char* tile, const __nv_bfloat16* base, long long stride,
                                             int row0, int row_end) {
  constexpr int PIECES = HD / 8;
  for (int i = threadIdx.x; i < ROWS * PIECES; i += blockDim.x) {
    const int r = i / PIECES, c = i - r * PIECES;
    const bool on = row0 + r < row_end;
    const __nv_bfloat16* src = base + (size_t)(on ? row0 + r : row0) * stride + c * 8;
    pf_cp16(pf_smem(tile) + pf_off<HD>(r, c), src, on);
  }
}

template <int HD>
__global__ void __launch_bounds__(PfShape<HD>::BM * 2)
attn_prefill_mma_kernel(PrefillArgs a) {
  constexpr int PF_BM = PfShape<HD>::BM, PF_BN = PfShape<HD>::BN;
  pdl_launch_dependents();
  pdl_wait();
  constexpr int KSTEPS = HD / 16;      // k-steps of Q K^T
  constexpr int ONT = HD / 8;          // n-tiles of the output
  constexpr int SNT = PF_BN / 8;       // n-tiles of the scores
  constexpr int TILE_Q = PF_BM * HD * 2;
  constexpr int TILE_KV = PF_BN * HD * 2;
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ __align__(128) unsigned char pf_smem_raw[];
  unsigned char* q_s = pf_smem_raw;
  unsigned char* kv_s = pf_smem_raw + TILE_Q;  // [stage][K tile, V tile]

  const int seq = blockIdx.y, head = blockIdx.z;
  const int row0 = a.seq_starts[seq];
  const int len = a.seq_starts[seq + 1] - row0;
  // heavy tiles (late queries see many keys) are scheduled first
  const int m0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * PF_BM;
  if (m0 >= len) return;
  const int kvh = head / (a.nq / a.nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  const __nv_bfloat16* qb = a.q + (size_t)row0 * a.q_stride + (size_t)head * HD;
  const __nv_bfloat16* kb = a.k + (size_t)row0 * a.k_stride + (size_t)kvh * HD;
  const __nv_bfloat16* vb = a.v + (size_t)row0 * a.v_stride + (size_t)kvh * HD;

  const int m_last = min(m0 + PF_BM, len) - 1;                               // last query row of the block
  const int j_lo = a.window > 0 ? max(0, m0 - a.window + 1) : 0;             // first key any row sees
  const int kb_lo = j_lo / PF_BN, kb_hi = m_last / PF_BN;                    // key tiles [kb_lo, kb_hi]

  pf_load_tile<HD, PF_BM>(q_s, qb, a.q_stride, m0, len);
  pf_load_tile<HD, PF_BN>(kv_s, kb, a.k_stride, kb_lo * PF_BN, len);
  pf_load_tile<HD, PF_BN>(kv_s + TILE_KV, vb, a.v_stride, kb_lo * PF_BN, len);
  asm volatile("cp.async.commit_group;" ::: "memory");

  float o[ONT][4];
#pragma unroll
  for (int n = 0; n < ONT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f};
  const int qrow[2] = {m0 + warp * 16 + g, m0 + warp * 16 + g + 8};          // this thread's two query positions
  const float cs = a.cap > 0.f ? a.scale / a.cap : a.scale * LOG2E;           // scale into tanh, or straight to base 2
  const float cap2 = a.cap * LOG2E;

  for (int kt = kb_lo; kt <= kb_hi; ++kt) {
    const int st = (kt - kb_lo) & 1;
    unsigned char* k_s = kv_s + (size_t)st * 2 * TILE_KV;
    unsigned char* v_s = k_s + TILE_KV;
    if (kt < kb_hi) {  // next tile into the other stage
      unsigned char* nk = kv_s + (size_t)(st ^ 1) * 2 * TILE_KV;
      pf_load_tile<HD, PF_BN>(nk, kb, a.k_stride, (kt + 1) * PF_BN, len);
      pf_load_tile<HD, PF_BN>(nk + TILE_KV, vb, a.v_stride, (kt + 1) * PF_BN, len);
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();

    // ---- S = Q K^T for this warp's 16 rows and the tile's 64 keys
    float s[SNT][4];
#pragma unroll
    for (int n = 0; n < SNT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t a0, a1, a2, a3;
      pf_ldm4(pf_smem(q_s) + pf_off<HD>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a0, a1,
              a2, a3);
#pragma unroll
      for (int np = 0; np < SNT / 2; ++np) {  // two n-tiles (16 keys) per ldmatrix
        uint32_t b0, b1, b2, b3;
        pf_ldm4(pf_smem(k_s) + pf_off<HD>(np * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)), b0, b1,
                b2, b3);
        pf_mma(s[2 * np], a0, a1, a2, a3, b0, b1);
        pf_mma(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }

    // ---- scale, softcap, mask, online softmax (base 2)
    const int j0 = kt * PF_BN;
    const bool edge = (j0 + PF_BN - 1 > m0 + warp * 16) || (j0 + PF_BN > len) ||
                      (a.window > 0 && (m0 + warp * 16 + 15) - j0 >= a.window);
    float new_max[2] = {mx[0], mx[1]};
    // (the tests on the cap and on the edge stand outside the loops: inside they stay a branch per score)
    if (a.cap > 0.f) {
#pragma unroll
      for (int n = 0; n < SNT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] = cap2 * pf_tanh(s[n][e] * cs);
    } else {
#pragma unroll
      for (int n = 0; n < SNT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] *= cs;
    }
    if (edge) {
#pragma unroll
      for (int n = 0; n < SNT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + n * 8 + 2 * t + (e & 1);
          const int i = qrow[e >> 1];
          const bool ok = j <= i && j < len && (a.window <= 0 || i - j < a.window);
          s[n][e] = ok ? s[n][e] : -INFINITY;
        }
      }
    }
#pragma unroll
    for (int n = 0; n < SNT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) new_max[e >> 1] = fmaxf(new_max[e >> 1], s[n][e]);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      new_max[r] = fmaxf(new_max[r], __shfl_xor_sync(0xffffffffu, new_max[r], 1));
      new_max[r] = fmaxf(new_max[r], __shfl_xor_sync(0xffffffffu, new_max[r], 2));
    }
    float corr[2], ref[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      ref[r] = new_max[r] == -INFINITY ? 0.f : new_max[r];
      corr[r] = pf_exp2(mx[r] - ref[r]);
      mx[r] = new_max[r];
      sum[r] *= corr[r];
    }
#pragma unroll
    for (int n = 0; n < SNT; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = pf_exp2(s[n][e] - ref[e >> 1]);
        s[n][e] = p;
        sum[e >> 1] += p;
      }
    }
#pragma unroll
    for (int n = 0; n < ONT; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }

    // ---- O += P V
#pragma unroll
    for (int ks = 0; ks < PF_BN / 16; ++ks) {
      const uint32_t a0 = pf_pack(s[2 * ks][0], s[2 * ks][1]), a1 = pf_pack(s[2 * ks][2], s[2 * ks][3]);
      const uint32_t a2 = pf_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), a3 = pf_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int np = 0; np < ONT / 2; ++np) {  // two n-tiles (16 output columns) per ldmatrix
        uint32_t b0, b1, b2, b3;
        pf_ldm4t(pf_smem(v_s) + pf_off<HD>(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, np * 2 + (lane >> 4)), b0, b1,
                 b2, b3);
        pf_mma(o[2 * np], a0, a1, a2, a3, b0, b1);
        pf_mma(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();  // the stage is free for the tile after next
  }

  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = qrow[r];
    if (i >= len) continue;
    const float inv = sum[r] > 0.f ? 1.f / sum[r] : 0.f;
    __nv_bfloat16* dst = a.out + (size_t)(row0 + i) * a.out_stride + (size_t)head * HD;
#pragma unroll
    for (int n = 0; n < ONT; ++n)
      *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = pf_pack(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
  }
}

template <int HD>
int launch_prefill(const PrefillArgs& a, int n_seqs, int max_len, cudaStream_t stream) {
  constexpr int PF_BM = PfShape<HD>::BM, PF_BN = PfShape<HD>::BN;
  const int smem = PF_BM * HD * 2 + 4 * PF_BN * HD * 2;
  // (the limit on dynamic shared memory is a device's: set once on each)
  static bool configured[AF_MAX_DEVICES] = {};
  const int dev__ = af_current_device();
  if (dev__ < 0) return -1;
  if (!configured[dev__]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return af_fail((int)e, "af_attn_prefill: %s", cudaGetErrorString(e));
    configured[dev__] = true;
  }
  dim3 grid((max_len + PF_BM - 1) / PF_BM, n_seqs, a.nq);
  af_launch(attn_prefill_mma_kernel<HD>, dim3(grid), dim3(PF_BM * 2), smem, stream, a);
  AF_CHECK_LAUNCH("af_attn_prefill");
}

}  // namespace

// 1 when the tensor-core kernel takes this head size (else the plain kernel serves).
AF_EXPORT int af_attn_prefill_supported(int hd) { return hd == 64 || hd == 128 || hd == 256 ? 1 : 0; }

// out [T, nq * hd] = attention of sequences that start at position 0 over
// their own keys.  q, k, v, out: bfloat16 rows with the given strides
// (elements, multiples of 8; bases 16-byte aligned); seq_starts [n_seqs + 1].
AF_EXPORT int af_attn_prefill(void* out, long long out_stride, const void* q, long long q_stride, const void* k,
                              long long k_stride, const void* v, long long v_stride, const int* seq_starts,
                              int n_seqs, int max_len, int nq, int nkv, int hd, float scale, float cap, int window,
                              cudaStream_t stream) {
  if (n_seqs == 0 || max_len == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "af_attn_prefill: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(af_attn_prefill_supported(hd), "af_attn_prefill: head_dim %d (takes 64, 128, 256)", hd);
  AF_REQUIRE(q_stride % 8 == 0 && k_stride % 8 == 0 && v_stride % 8 == 0 && out_stride % 2 == 0,
             "af_attn_prefill: row strides must be multiples of 8");
  AF_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0 && ((uintptr_t)out & 3) == 0,
             "af_attn_prefill: operands must be 16-byte aligned");
  AF_REQUIRE(n_seqs <= 65535 && nq <= 65535, "af_attn_prefill: too many sequences or heads");
  PrefillArgs a{(__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k,
                k_stride, (const __nv_bfloat16*)v, v_stride, seq_starts, nq, nkv, scale, cap, window};
  if (hd == 64) return launch_prefill<64>(a, n_seqs, max_len, stream);
  if (hd == 128) return launch_prefill<128>(a, n_seqs, max_len, stream);
  return launch_prefill<256>(a, n_seqs, max_len, stream);
}
