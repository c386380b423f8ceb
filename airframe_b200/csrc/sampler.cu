// Token sampling on the device: repetition penalty, greedy arg-max, and
// temperature sampling inside the top-p nucleus.  One block per row of logits.
//
// Meaning of the options (as in the reference's sample_token,
// src/runtime/gpu.rs:880-962): the penalty divides a positive logit and
// multiplies a negative one, once per occurrence among the recent tokens;
// temperature < 1e-7 is arg-max over finite logits; otherwise logits / T,
// softmax, the nucleus is the smallest set of most probable tokens whose mass
// reaches top_p, and one token is drawn from it with the uniform number u.
//
// Arithmetic.  Weights are fixed point: q_i = trunc(exp(z_i - max z) * 2^40) as
// 64-bit integers, so sums do not depend on the order of addition and a row
// gives the same token whatever else is in the batch.  The nucleus holds every
// token with q above the cutoff value and, of the tokens equal to it, as many
// (lowest index first) as the mass asks for.  The draw walks the nucleus in
// index order: the token i with prefix(i) <= r < prefix(i) + q_i,
// r = trunc(u * nucleus mass).  (The reference walks in order of descending
// probability with ties in unspecified order; the distribution is the same.)
// Ties in arg-max go to the lowest index.
#include "common.cuh"

#define SM_THREADS 1024
#define SM_BITS 14
#define SM_BINS (1 << SM_BITS)
#define SM_LEVELS 3
#define SM_KEY_BITS (SM_BITS * SM_LEVELS)  // 42 >= 41 bits of q

typedef unsigned long long u64;

__device__ __forceinline__ u64 warp_scan_u64(u64 v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    u64 t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

// Inclusive scan over the block; `total` gets the block's sum.  scratch: 33 u64.
__device__ __forceinline__ u64 block_scan_u64(u64 v, u64* scratch, u64* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  u64 inc = warp_scan_u64(v, lane);
  __syncthreads();
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    u64 t = scratch[lane];
    u64 s = warp_scan_u64(t, lane);
    scratch[lane] = s - t;  // exclusive offset of each warp
    if (lane == 31) scratch[32] = s;
  }
  __syncthreads();
  *total = scratch[32];
  return inc + scratch[warp];
}

__device__ __forceinline__ u64 block_sum_u64(u64 v, u64* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    u64 t = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ u64 weight_of(float logit, float inv_t, float zmax) {
  if (!isfinite(logit)) return 0ull;
  const float e = expf(logit * inv_t - zmax);
  return (u64)(e * 1099511627776.0f);  // 2^40
}

__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(float* __restrict__ logits, int ld, int V, const int* __restrict__ recent,
              const int* __restrict__ n_recent, int recent_stride, float temperature, float top_p,
              float penalty, const float* __restrict__ uniform, int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ u64 bins[];  // SM_BINS
  __shared__ u64 scratch[33];
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ int s_recent[64];
  __shared__ u64 s_a, s_b;
  __shared__ int s_i, s_found;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x;
  float* z = logits + (size_t)row * ld;

  // ---- repetition penalty, in place, once per occurrence
  const int nr = n_recent ? min(n_recent[row], 64) : 0;
  if (penalty != 1.0f && nr > 0) {
    if (tid < nr) s_recent[tid] = recent[(size_t)row * recent_stride + tid];
    __syncthreads();
    if (tid < nr) {
      const int tok = s_recent[tid];
      int count = 0;
      bool first = true;
      for (int j = 0; j < nr; ++j) {
        if (s_recent[j] == tok) {
          ++count;
          if (j < tid) first = false;
        }
      }
      if (first && tok >= 0 && tok < V) {
        float v = z[tok];
        for (int c = 0; c < count; ++c) v = v > 0.f ? v / penalty : v * penalty;
        z[tok] = v;
      }
    }
    __syncthreads();
  }

  // ---- maximum over finite logits, lowest index on ties
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  int done = 0;
  if ((((uintptr_t)z) & 15) == 0) {
    // 16-byte loads, four in flight a thread (indices still rise within a thread: the first maximum stays)
    const float4* z4 = reinterpret_cast<const float4*>(z);
    const int n4 = V / 4;
    for (int i0 = tid; i0 < n4; i0 += 4 * SM_THREADS) {
      float4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        q[u] = i0 + u * SM_THREADS < n4 ? z4[i0 + u * SM_THREADS] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = (i0 + u * SM_THREADS) * 4;
        const float e[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (isfinite(e[c]) && e[c] > best) {
            best = e[c];
            best_i = i + c;
          }
        }
      }
    }
    done = n4 * 4;
  }
  for (int i = done + tid; i < V; i += SM_THREADS) {
    const float v = z[i];
    if (isfinite(v) && v > best) {  // indices rise within a thread: first maximum stays
      best = v;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    best = s_val[lane];
    best_i = s_idx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (lane == 0) {
      s_val[0] = best;
      s_idx[0] = best_i;
    }
  }
  __syncthreads();
  best = s_val[0];
  best_i = s_idx[0];
  if (best_i == 0x7fffffff) {  // nothing finite
    if (tid == 0) out[row] = 0;
    return;
  }
  if (temperature < 1e-7f) {
    if (tid == 0) out[row] = best_i;
    return;
  }

  const float inv_t = 1.0f / temperature;
  const float zmax = best * inv_t;

  // ---- nucleus cutoff: the largest key x with sum(q >= x) >= tau
  u64 prefix = 0;      // key digits settled so far
  u64 above = 0;       // mass of keys above the settled prefix's range
  u64 set_total = 0;   // mass of keys that match the settled prefix
  u64 total = 0, cut_key = 0, n_cut = 0, mass = 0;
  const bool whole = top_p >= 1.0f;
  for (int level = 0; level < SM_LEVELS; ++level) {
    const int shift = SM_KEY_BITS - SM_BITS * (level + 1);
    for (int b = tid; b < SM_BINS; b += SM_THREADS) bins[b] = 0ull;
    __syncthreads();
    u64 mine = 0;
    for (int i0 = 0; i0 < V; i0 += SM_THREADS) {
      const int i = i0 + tid;
      u64 q = i < V ? weight_of(z[i], inv_t, zmax) : 0ull;
      if (level == 0) mine += q;
      const bool in_set = level == 0 || (q >> (shift + SM_BITS)) == prefix;
      const unsigned digit = (unsigned)((q >> shift) & (SM_BINS - 1));
      // digit 0 is left out: its mass follows from the set's total
      const bool add = !whole && in_set && digit != 0 && q != 0;
      const unsigned active = __ballot_sync(0xffffffffu, add);
      if (add) {
        const unsigned peers = __match_any_sync(active, digit);
        const unsigned lo = __reduce_add_sync(peers, (unsigned)(q & 0xfffffu));
        const unsigned hi = __reduce_add_sync(peers, (unsigned)(q >> 20));
        if (lane == __ffs(peers) - 1) atomicAdd(&bins[digit], (u64)lo + ((u64)hi << 20));
      }
    }
    if (level == 0) {
      total = block_sum_u64(mine, scratch);
      set_total = total;
      if (whole) break;
    }
    __syncthreads();
    // mass of the bins above each bin, top down; thread t owns bins [t*16, t*16+16)
    const int per = SM_BINS / SM_THREADS;
    const int b0 = (SM_THREADS - 1 - tid) * per;  // thread 0 owns the top bins
    u64 local = 0;
    for (int j = per - 1; j >= 0; --j) local += (b0 + j == 0) ? 0ull : bins[b0 + j];
    u64 tot_nz;
    const u64 inc = block_scan_u64(local, scratch, &tot_nz);
    if (tid == SM_THREADS - 1) bins[0] = set_total - tot_nz;  // digit 0's mass
    __syncthreads();
    if (level == 0) {
      const double tau_d = ceil((double)top_p * (double)total);
      if (tid == 0) s_a = tau_d < 1.0 ? 1ull : (u64)tau_d;
      __syncthreads();
    }
    const u64 tau = s_a;
    // find the bin where above + cumulative reaches tau
    u64 run = above + (inc - local);
    for (int j = per - 1; j >= 0; --j) {
      const u64 m = bins[b0 + j];
      if (run < tau && run + m >= tau) {
        s_i = b0 + j;
        s_b = run;
      }
      run += m;
    }
    __syncthreads();
    const int digit = s_i;
    above = s_b;
    set_total = bins[digit];
    prefix = (prefix << SM_BITS) | (u64)digit;
    __syncthreads();
  }
  if (whole) {
    cut_key = 0;
    n_cut = 0;
    mass = total;
  } else {
    cut_key = prefix;  // > 0: a bin with no mass never reaches tau
    const u64 tau = s_a;
    const u64 need = tau - above;                     // 1 .. set_total
    n_cut = (need + cut_key - 1) / cut_key;           // tokens equal to the cutoff that belong
    mass = above + n_cut * cut_key;
  }
#ifdef AF_SAMPLER_DEBUG
  if (tid == 0) printf("row %d total %llu tau %llu cut_key %llu n_cut %llu above %llu mass %llu prefix %llu\n", row, total, s_a, cut_key, n_cut, above, mass, prefix);
#endif
  if (mass == 0) {
    if (tid == 0) out[row] = best_i;
    return;
  }

  // ---- the draw: index order over the nucleus
  const double rd = (double)uniform[row] * (double)mass;
  u64 r = rd <= 0.0 ? 0ull : (u64)rd;
  if (r >= mass) r = mass - 1;
  u64 before = 0;     // nucleus mass in earlier tiles
  u64 eq_before = 0;  // tokens equal to the cutoff in earlier tiles
  if (tid == 0) s_found = -1;
  __syncthreads();
  for (int i0 = 0; i0 < V; i0 += SM_THREADS) {
    const int i = i0 + tid;
    const u64 q = i < V ? weight_of(z[i], inv_t, zmax) : 0ull;
    const bool eq = q == cut_key && q > 0;
    u64 eq_total;
    const u64 eq_inc = block_scan_u64(eq ? 1ull : 0ull, scratch, &eq_total);
    // with top_p >= 1 the cutoff is 0: every token with weight belongs
    const u64 rank = eq_before + eq_inc;
    u64 w = 0ull;
    if (q > cut_key) w = q;
    if (eq && rank <= n_cut) w = q;
    const bool in = w != 0ull;
    u64 w_total;
    const u64 w_inc = block_scan_u64(w, scratch, &w_total);
    const u64 start = before + w_inc - w;
#ifdef AF_SAMPLER_DEBUG
    if (tid < 5) printf("tid %d q %llu eq %d eq_inc %llu in %d w_inc %llu start %llu r %llu\n", tid, q, (int)eq, eq_inc, (int)in, w_inc, start, r);
#endif
    if (in && start <= r && r < start + w) s_found = i;
    __syncthreads();
    if (s_found >= 0) break;
    before += w_total;
    eq_before += eq_total;
  }
  if (tid == 0) out[row] = s_found >= 0 ? s_found : best_i;
}

// logits [rows, ld] float (changed in place by the penalty), recent [rows,
// recent_stride] token ids with n_recent[rows] valid (newest 64 at most),
// uniform [rows] in [0, 1), out [rows].
AF_EXPORT int af_sample(float* logits, int ld, int rows, int vocab, const int* recent,
                        const int* n_recent, int recent_stride, float temperature, float top_p,
                        float penalty, const float* uniform, int* out, cudaStream_t stream) {
  if (rows == 0) return 0;
  AF_REQUIRE(rows > 0 && vocab > 0 && ld >= vocab, "af_sample: bad sizes");
  AF_REQUIRE(temperature >= 0.f && top_p > 0.f && penalty > 0.f, "af_sample: bad options");
  AF_REQUIRE(temperature < 1e-7f || uniform != nullptr, "af_sample: uniform numbers are required");
  const size_t smem = SM_BINS * sizeof(u64);
  // (the limit on dynamic shared memory is a device's: set once on each)
  static bool configured[AF_MAX_DEVICES] = {};
  const int dev__ = af_current_device();
  if (dev__ < 0) return -1;
  if (!configured[dev__]) {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return af_fail((int)e, "af_sample: %s", cudaGetErrorString(e));
    configured[dev__] = true;
  }
  af_launch(sample_kernel, dim3(rows), dim3(SM_THREADS), smem, stream, logits, ld, vocab, recent, n_recent, recent_stride,
                                                    temperature, top_p, penalty, uniform, out);
  AF_CHECK_LAUNCH("af_sample");
}


// ---------------------------------------------------------------- arg-max keys of the fused head

// tokens[r] = the row held in keys[r * AF_KEY_STRIDE] (see af_gemm_tc_argmax), 0 when no finite value took part (as the
// arg-max over finite logits of an all-non-finite row); the keys are zeroed for the next use.
__global__ void argmax_finish_kernel(int* __restrict__ tokens, unsigned long long* __restrict__ keys, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const unsigned long long k = keys[(size_t)r * AF_KEY_STRIDE];
  tokens[r] = k ? (int)(0xffffffffu - (uint32_t)k) : 0;
  keys[(size_t)r * AF_KEY_STRIDE] = 0ull;
}

AF_EXPORT int af_argmax_finish(int* tokens, unsigned long long* keys, int n, cudaStream_t stream) {
  if (n == 0) return 0;
  AF_REQUIRE(n > 0 && tokens != nullptr && keys != nullptr, "af_argmax_finish: bad arguments");
  af_launch(argmax_finish_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens, keys, n);
  AF_CHECK_LAUNCH("af_argmax_finish");
}

// Words between the keys of two tokens.
AF_EXPORT int af_argmax_key_stride() { return AF_KEY_STRIDE; }
