// Rotary position encoding with the cache write, and the plain attention
// kernels (one warp per query row and head, keys in order).  They serve the
// 32-bit path and stand beside the faster bfloat16 kernels as their twins.
//
// Cache of one layer: pages [n_pages][n_kv_heads][AF_PAGE][head_dim] for K and
// for V.  A sequence's page table maps row / AF_PAGE to a page.  A layer with
// a window keeps rows modulo `ring_rows` (a multiple of AF_PAGE, >= window).
#include "common.cuh"

#define AF_MAX_HD 512
#define AF_HD_SLICES (AF_MAX_HD / 32)

// ---------------------------------------------------------------- rope + cache write

// One block per (token, head) of the packed row [q heads | k heads | v heads].
// Rotates q and k heads in place (32-bit angles and arithmetic) and, when a
// cache is given, stores the rotated k and the v in the row's page.  The row
// may arrive as split-K partial sums (float), added in index order first.
template <typename T>
__device__ __forceinline__ float rope_src(const T* row, const float* parts, int n_parts, size_t part_stride,
                                          int i) {
  if (parts == nullptr) return to_f32(row[i]);
  // (16 loads in flight: a product of up to 16 splits costs one round trip; the sums go on in index order)
  float acc[16];
  float v = 0.f;
  for (int p0 = 0; p0 < n_parts; p0 += 16) {
#pragma unroll
    for (int u = 0; u < 16; ++u) acc[u] = p0 + u < n_parts ? parts[(size_t)(p0 + u) * part_stride + i] : 0.f;
#pragma unroll
    for (int u = 0; u < 16; ++u) v += acc[u];
  }
  return v;
}

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, int row_stride, const float* __restrict__ parts,
                                  int n_parts, size_t part_stride, const int* __restrict__ positions,
                                  const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                  const int* __restrict__ len_after, const float* __restrict__ inv_freq,
                                  int nq, int nkv, int hd, int rot_dim, int pairing,
                                  T* __restrict__ kcache, T* __restrict__ vcache,
                                  const int* __restrict__ page_table, int max_pages, int ring_rows) {
  pdl_launch_dependents();
  // Positions, slots, lengths, the page table and the frequencies are inputs of the step, not
  // results of the kernel before: the row's place in the cache and the first pair's sine and
  // cosine are worked out before the wait for that kernel.
  const int t = blockIdx.x, head = blockIdx.y;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * row_stride + (size_t)head * hd;
  const float* pr = parts ? parts + (size_t)t * (nq + 2 * nkv) * hd + (size_t)head * hd : nullptr;  // (read after the wait)
  const int half = rot_dim / 2;
  // where this head's row goes in the cache (k and v heads only)
  T* dst = nullptr;
  if (kcache != nullptr && head >= nq) {
    const int seq = seq_of_token[t];
    const int slot = slots[seq];
    // of the tokens of this step that share a ring row only the last is kept; padding rows are skipped
    if (slot >= 0 && !(ring_rows > 0 && pos + ring_rows < len_after[seq])) {
      const int r = ring_rows > 0 ? pos % ring_rows : pos;
      if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < max_pages, r)) {
        const int page = page_table[(size_t)slot * max_pages + r / AF_PAGE];
        const bool is_v = head >= nq + nkv;
        const int h = head - nq - (is_v ? nkv : 0);
        if (AF_INDEX_OK(page >= 0, page))
          dst = (is_v ? vcache : kcache) + (((size_t)page * nkv + h) * AF_PAGE + r % AF_PAGE) * hd;
      }
    }
  }
  const bool rotate = head < nq + nkv;
  float s0 = 0.f, c0 = 1.f;
  if (rotate && threadIdx.x < half) sincosf((float)pos * inv_freq[threadIdx.x], &s0, &c0);
  pdl_wait();
  pr = pdl_fresh(pr);
  row = pdl_fresh(row);
  // rotary pairs
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    const int i0 = pairing == AF_PAIR_HALF ? p : 2 * p;
    const int i1 = pairing == AF_PAIR_HALF ? p + half : 2 * p + 1;
    float a = rope_src(row, pr, n_parts, part_stride, i0);
    float b = rope_src(row, pr, n_parts, part_stride, i1);
    if (rotate) {
      float s = s0, c = c0;
      if (p != threadIdx.x) sincosf((float)pos * inv_freq[p], &s, &c);
      const float ra = a * c - b * s, rb = b * c + a * s;
      a = ra;
      b = rb;
    }
    const T ta = from_f32<T>(a), tb = from_f32<T>(b);
    if (rotate || pr != nullptr) {
      row[i0] = ta;
      row[i1] = tb;
    }
    if (dst != nullptr) {
      dst[i0] = ta;
      dst[i1] = tb;
    }
  }
  // elements beyond the rotary part
  for (int i = rot_dim + threadIdx.x; i < hd; i += blockDim.x) {
    const T v = from_f32<T>(rope_src(row, pr, n_parts, part_stride, i));
    if (pr != nullptr) row[i] = v;
    if (dst != nullptr) dst[i] = v;
  }
}

// The same for bfloat16 rows without partial sums, half-split pairs over the
// whole head and head_dim % 16 == 0: one block per token, 16-byte loads and
// stores, eight pairs a thread.
__global__ void __launch_bounds__(256)
rope_cache_vec_kernel(__nv_bfloat16* __restrict__ qkv, long long row_stride, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                      const int* __restrict__ len_after, const float* __restrict__ inv_freq,
                      const float2* __restrict__ table, int nq, int nkv, int hd,
                      __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                      const int* __restrict__ page_table, int max_pages, int ring_rows) {
  pdl_launch_dependents();
  // (positions, slots, lengths, page table and frequencies are inputs of the step: the row's place in
  // the cache and the sines and cosines are worked out before the wait for the kernel in front)
  const int t = blockIdx.x;
  const int pos = positions[t];
  __nv_bfloat16* row = qkv + (size_t)t * row_stride;
  const int half = hd / 2;
  const int per_head = half / 8;                 // 16-byte pieces of a half head
  const int n_heads = nq + 2 * nkv;
  // where this token's k and v rows go in the cache
  size_t dst_row = 0;
  bool store = false;
  if (kcache != nullptr) {
    const int seq = seq_of_token[t];
    const int slot = slots[seq];
    if (slot >= 0 && !(ring_rows > 0 && pos + ring_rows < len_after[seq])) {
      const int r = ring_rows > 0 ? pos % ring_rows : pos;
      if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < max_pages, r)) {
        const int page = page_table[(size_t)slot * max_pages + r / AF_PAGE];
        dst_row = ((size_t)page * nkv) * AF_PAGE + r % AF_PAGE;   // + h * AF_PAGE rows for kv head h
        store = AF_INDEX_OK(page >= 0, page);
      }
    }
  }
  // a thread's pieces all have the same place in their heads when the block's size is a multiple of
  // the pieces of a head (it is for head sizes up to 512 that divide so): its 8 pairs' angles are fixed
  const bool fixed_c = blockDim.x % per_head == 0;
  float sn0[8], cs0[8];
  if (fixed_c && table == nullptr) {
    const int c = threadIdx.x % per_head;
#pragma unroll
    for (int e = 0; e < 8; ++e) sincosf((float)pos * inv_freq[c * 8 + e], &sn0[e], &cs0[e]);
  }
  pdl_wait();
  row = pdl_fresh(row);
  if (fixed_c && table != nullptr) {
    // the step's table of (cos, sin), made once for all layers by the same arithmetic (a kernel of this step
    // wrote it: read after the wait)
    const float4* tp = reinterpret_cast<const float4*>(pdl_fresh(table) + (size_t)t * half + (threadIdx.x % per_head) * 8);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 v = tp[e];
      cs0[2 * e] = v.x, sn0[2 * e] = v.y, cs0[2 * e + 1] = v.z, sn0[2 * e + 1] = v.w;
    }
  }
  for (int i = threadIdx.x; i < n_heads * per_head; i += blockDim.x) {
    const int head = i / per_head, c = i - head * per_head;
    __nv_bfloat16* x = row + (size_t)head * hd + c * 8;
    uint4 lo = *reinterpret_cast<const uint4*>(x);
    uint4 hi = *reinterpret_cast<const uint4*>(x + half);
    if (head < nq + nkv) {
      uint32_t* lw = reinterpret_cast<uint32_t*>(&lo);
      uint32_t* hw = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a[2] = {__uint_as_float(lw[j] << 16), __uint_as_float(lw[j] & 0xffff0000u)};
        float b[2] = {__uint_as_float(hw[j] << 16), __uint_as_float(hw[j] & 0xffff0000u)};
        float ra[2], rb[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float sn = sn0[2 * j + e], cs = cs0[2 * j + e];
          if (!fixed_c) sincosf((float)pos * inv_freq[c * 8 + 2 * j + e], &sn, &cs);
          ra[e] = a[e] * cs - b[e] * sn;
          rb[e] = b[e] * cs + a[e] * sn;
        }
        __nv_bfloat162 pa = __floats2bfloat162_rn(ra[0], ra[1]), pb = __floats2bfloat162_rn(rb[0], rb[1]);
        lw[j] = *reinterpret_cast<uint32_t*>(&pa);
        hw[j] = *reinterpret_cast<uint32_t*>(&pb);
      }
      *reinterpret_cast<uint4*>(x) = lo;
      *reinterpret_cast<uint4*>(x + half) = hi;
    }
    if (store && head >= nq) {
      const bool is_v = head >= nq + nkv;
      const int h = head - nq - (is_v ? nkv : 0);
      __nv_bfloat16* d = (is_v ? vcache : kcache) + (dst_row + (size_t)h * AF_PAGE) * hd + c * 8;
      *reinterpret_cast<uint4*>(d) = lo;
      *reinterpret_cast<uint4*>(d + half) = hi;
    }
  }
}

// `parts` (optional): float [n_parts, n_tokens, row width] partial sums of the
// rows, part_stride elements apart; they are added in order into qkv first.
AF_EXPORT int af_rope_cache_write(void* qkv, int dtype, int row_stride, const float* parts, int n_parts,
                                  long long part_stride, const int* positions,
                                  const int* seq_of_token, const int* slots, const int* len_after,
                                  const float* inv_freq, const float* table, int n_tokens, int nq, int nkv, int hd,
                                  int rot_dim, int pairing, void* kcache, void* vcache,
                                  const int* page_table, int max_pages, int ring_rows,
                                  cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && hd > 0, "af_rope_cache_write: bad sizes");
  AF_REQUIRE(rot_dim >= 0 && rot_dim <= hd && rot_dim % 2 == 0,
             "af_rope_cache_write: rotary dim %d must be even and <= head_dim %d", rot_dim, hd);
  AF_REQUIRE(pairing == AF_PAIR_HALF || pairing == AF_PAIR_ADJACENT, "af_rope_cache_write: pairing");
  AF_REQUIRE(ring_rows % AF_PAGE == 0, "af_rope_cache_write: ring rows %d not whole pages", ring_rows);
  AF_REQUIRE((kcache == nullptr) == (vcache == nullptr), "af_rope_cache_write: k and v cache");
  if (dtype == AF_BF16 && parts == nullptr && pairing == AF_PAIR_HALF && rot_dim == hd && hd % 16 == 0 &&
      row_stride % 8 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)kcache & 15) == 0 &&
      ((uintptr_t)vcache & 15) == 0 && n_tokens >= 64) {
    af_launch(rope_cache_vec_kernel, dim3(n_tokens), dim3(256), 0, stream, (__nv_bfloat16*)qkv, (long long)row_stride,
              positions, seq_of_token, slots, len_after, inv_freq,
              ((uintptr_t)table & 15) == 0 ? reinterpret_cast<const float2*>(table) : nullptr, nq, nkv, hd, (__nv_bfloat16*)kcache,
              (__nv_bfloat16*)vcache, page_table, max_pages, ring_rows);
    AF_CHECK_LAUNCH("af_rope_cache_write");
  }
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(rope_cache_kernel<T>, dim3(dim3(n_tokens, nq + 2 * nkv)), dim3(hd / 2 < 32 ? 32 : (hd / 2 > 256 ? 256 : hd / 2)), 0, stream, 
                        (T*)qkv, row_stride, parts, n_parts, (size_t)part_stride, positions, seq_of_token,
                        slots, len_after, inv_freq, nq,
                        nkv, hd, rot_dim, pairing, (T*)kcache, (T*)vcache, page_table, max_pages,
                        ring_rows));
  AF_CHECK_LAUNCH("af_rope_cache_write");
}

// ---------------------------------------------------------------- tables of a step

// (cos, sin) of position * frequency for every token and rotary pair: float [n_tokens][half][2].  Made once
// per step for all layers that rotate by the same frequencies; 32-bit angles as in the rotary kernels.
__global__ void rope_table_kernel(float2* __restrict__ table, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[p], &s, &c);
    table[(size_t)t * half + p] = make_float2(c, s);
  }
}

AF_EXPORT int af_rope_table(float* table, const int* positions, const float* inv_freq, int n_tokens, int half,
                            cudaStream_t stream) {
  if (n_tokens == 0 || half == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && half > 0 && ((uintptr_t)table & 7) == 0, "af_rope_table: bad sizes");
  af_launch(rope_table_kernel, dim3(n_tokens), dim3(half < 32 ? 32 : (half > 256 ? 256 : half)), 0, stream,
            reinterpret_cast<float2*>(table), positions, inv_freq, half);
  AF_CHECK_LAUNCH("af_rope_table");
}

// Where each token's keys and values go in the cache of one group of layers: rows[t] = page * nkv * AF_PAGE +
// row in page (the row of kv head 0; head h lies h * AF_PAGE rows further), or -1 when the token is not stored
// (a padding row; a token of a long prompt whose ring row a later token of the same step takes).
__global__ void kv_rows_kernel(int* __restrict__ rows, const int* __restrict__ positions,
                               const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                               const int* __restrict__ len_after, const int* __restrict__ page_table, int max_pages,
                               int ring_rows, int nkv, int n_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  const int pos = positions[t], seq = seq_of_token[t], slot = slots[seq];
  int row = -1;
  if (slot >= 0 && !(ring_rows > 0 && pos + ring_rows < len_after[seq])) {
    const int r = ring_rows > 0 ? pos % ring_rows : pos;
    if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < max_pages, r)) {
      const int page = page_table[(size_t)slot * max_pages + r / AF_PAGE];
      if (AF_INDEX_OK(page >= 0, page)) row = page * nkv * AF_PAGE + r % AF_PAGE;
    }
  }
  rows[t] = row;
}

AF_EXPORT int af_kv_rows(int* rows, const int* positions, const int* seq_of_token, const int* slots,
                         const int* len_after, const int* page_table, int max_pages, int ring_rows, int nkv,
                         int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && nkv > 0 && ring_rows % AF_PAGE == 0, "af_kv_rows: bad sizes");
  af_launch(kv_rows_kernel, dim3((n_tokens + 127) / 128), dim3(128), 0, stream, rows, positions, seq_of_token, slots,
            len_after, page_table, max_pages, ring_rows, nkv, n_tokens);
  AF_CHECK_LAUNCH("af_kv_rows");
}

// ---------------------------------------------------------------- plain attention

// Online-softmax state of one (query, head) held by a warp: lane l owns the
// elements l, l + 32, ... of the head.
struct WarpAttn {
  float q[AF_HD_SLICES];
  float o[AF_HD_SLICES];
  float m, l;
};

template <typename T>
__device__ __forceinline__ void attn_load_q(WarpAttn& st, const T* q, int hd, int lane) {
#pragma unroll
  for (int e = 0; e < AF_HD_SLICES; ++e) {
    const int d = lane + 32 * e;
    st.q[e] = d < hd ? to_f32(q[d]) : 0.f;
    st.o[e] = 0.f;
  }
  st.m = -INFINITY;
  st.l = 0.f;
}

template <typename T>
__device__ __forceinline__ void attn_key(WarpAttn& st, const T* k, const T* v, int hd, int lane,
                                         float scale, float cap, float bias) {
  float dot = 0.f;
#pragma unroll
  for (int e = 0; e < AF_HD_SLICES; ++e) {
    const int d = lane + 32 * e;
    if (d < hd) dot += st.q[e] * to_f32(k[d]);
  }
  dot = warp_sum(dot);
  const float s = softcap_f32(dot * scale, cap) + bias;   // bias: a position encoding's slope * (key - query)
  const float m_new = fmaxf(st.m, s);
  const float corr = expf(st.m - m_new);  // exp(-inf) = 0 on the first key
  const float p = expf(s - m_new);
  st.l = st.l * corr + p;
#pragma unroll
  for (int e = 0; e < AF_HD_SLICES; ++e) {
    const int d = lane + 32 * e;
    if (d < hd) st.o[e] = st.o[e] * corr + p * to_f32(v[d]);
  }
  st.m = m_new;
}

template <typename T>
__device__ __forceinline__ void attn_store(const WarpAttn& st, T* out, int hd, int lane) {
  const float inv = st.l > 0.f ? 1.f / st.l : 0.f;
#pragma unroll
  for (int e = 0; e < AF_HD_SLICES; ++e) {
    const int d = lane + 32 * e;
    if (d < hd) out[d] = from_f32<T>(st.o[e] * inv);
  }
}

// Prompts that start at position 0: keys and values are the step's own rows.
// Warp w of the grid handles (token, head) = (w / nq, w % nq).
template <typename T>
__global__ void attn_prefill_plain_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ q,
                                          int q_stride, const T* __restrict__ k, int k_stride,
                                          const T* __restrict__ v, int v_stride,
                                          const int* __restrict__ positions,
                                          int n_tokens, int nq, int nkv, int hd, float scale, float cap,
                                          int window, const float* __restrict__ slopes) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * nq) return;
  const int t = (int)(w / nq), h = (int)(w % nq);
  const int g = h / (nq / nkv);
  const int pos = positions[t];          // position inside its sequence
  const int first_row = t - pos;         // row of the sequence's position 0
  WarpAttn st;
  attn_load_q(st, q + (size_t)t * q_stride + (size_t)h * hd, hd, lane);
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const float slope = slopes ? slopes[h] : 0.f;
  for (int j = lo; j <= pos; ++j) {
    const size_t r = (size_t)(first_row + j);
    attn_key(st, k + r * k_stride + (size_t)g * hd, v + r * v_stride + (size_t)g * hd, hd, lane, scale,
             cap, slope * (float)(j - pos));
  }
  attn_store(st, out + (size_t)t * out_stride + (size_t)h * hd, hd, lane);
}

AF_EXPORT int af_attn_prefill_plain(void* out, int out_stride, const void* q, int q_stride,
                                    const void* k, int k_stride, const void* v, int v_stride, int dtype,
                                    const int* positions, int n_tokens, int nq, int nkv, int hd,
                                    float scale, float cap, int window, const float* slopes,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "af_attn_prefill_plain: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(hd > 0 && hd <= AF_MAX_HD, "af_attn_prefill_plain: head_dim %d beyond %d", hd, AF_MAX_HD);
  const long long warps = (long long)n_tokens * nq;
  const int wpb = 4;
  const long long blocks = (warps + wpb - 1) / wpb;
  AF_REQUIRE(blocks < (1ll << 31), "af_attn_prefill_plain: too many rows");
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(attn_prefill_plain_kernel<T>, dim3((unsigned)blocks), dim3(wpb * 32), 0, stream, 
                        (T*)out, out_stride, (const T*)q, q_stride, (const T*)k, k_stride, (const T*)v,
                        v_stride, positions, n_tokens, nq, nkv, hd, scale, cap, window, slopes));
  AF_CHECK_LAUNCH("af_attn_prefill_plain");
}

// One new token per sequence: keys and values come from the cache pages.
// `lens[b]` counts the new token, which the cache holds already.
template <typename T>
__global__ void attn_decode_plain_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ q,
                                         int q_stride, const T* __restrict__ kcache,
                                         const T* __restrict__ vcache, const int* __restrict__ page_table,
                                         int max_pages, const int* __restrict__ slots,
                                         const int* __restrict__ lens, int batch, int nq, int nkv, int hd,
                                         float scale, float cap, int window, int ring_rows,
                                         const float* __restrict__ slopes) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)batch * nq) return;
  const int b = (int)(w / nq), h = (int)(w % nq);
  const int g = h / (nq / nkv);
  const int slot = slots[b];
  T* o = out + (size_t)b * out_stride + (size_t)h * hd;
  if (slot < 0) {  // padding row
    for (int d = lane; d < hd; d += 32) o[d] = from_f32<T>(0.f);
    return;
  }
  const int len = lens[b];
  const int pos = len - 1;
  WarpAttn st;
  attn_load_q(st, q + (size_t)b * q_stride + (size_t)h * hd, hd, lane);
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int* pt = page_table + (size_t)slot * max_pages;
  const float slope = slopes ? slopes[h] : 0.f;
  for (int j = lo; j <= pos; ++j) {
    const int r = ring_rows > 0 ? j % ring_rows : j;
    if (!AF_INDEX_OK(r / AF_PAGE < max_pages && pt[r / AF_PAGE] >= 0, r)) continue;
    const size_t base = (((size_t)pt[r / AF_PAGE] * nkv + g) * AF_PAGE + r % AF_PAGE) * hd;
    attn_key(st, kcache + base, vcache + base, hd, lane, scale, cap, slope * (float)(j - pos));
  }
  attn_store(st, o, hd, lane);
}

AF_EXPORT int af_attn_decode_plain(void* out, int out_stride, const void* q, int q_stride,
                                   const void* kcache, const void* vcache, int dtype,
                                   const int* page_table, int max_pages, const int* slots,
                                   const int* lens, int batch, int nq, int nkv, int hd, float scale,
                                   float cap, int window, int ring_rows, const float* slopes,
                                   cudaStream_t stream) {
  if (batch == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "af_attn_decode_plain: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(hd > 0 && hd <= AF_MAX_HD, "af_attn_decode_plain: head_dim %d beyond %d", hd, AF_MAX_HD);
  AF_REQUIRE(ring_rows % AF_PAGE == 0 && (ring_rows == 0 || window > 0) && (window <= ring_rows || ring_rows == 0),
             "af_attn_decode_plain: window %d, ring rows %d", window, ring_rows);
  const long long warps = (long long)batch * nq;
  const int wpb = 4;
  const long long blocks = (warps + wpb - 1) / wpb;
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(attn_decode_plain_kernel<T>, dim3((unsigned)blocks), dim3(wpb * 32), 0, stream, 
                        (T*)out, out_stride, (const T*)q, q_stride, (const T*)kcache, (const T*)vcache,
                        page_table, max_pages, slots, lens, batch, nq, nkv, hd, scale, cap, window,
                        ring_rows, slopes));
  AF_CHECK_LAUNCH("af_attn_decode_plain");
}
