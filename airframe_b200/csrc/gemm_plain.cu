// Plain matrix product out[M, N] = x[M, K] * w[N, K]^T on the CUDA cores with
// 32-bit multiply-adds and 32-bit accumulators (no tensor cores, no reduced
// precision mode).  Every output element adds its K products in index order,
// whatever M and N are, so a row's result does not depend on the batch it is
// in.  It is the matrix product of the 32-bit path and the twin of the
// tensor-core kernels.
#include "common.cuh"

#define GP_BM 64
#define GP_BN 64
#define GP_BK 16

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(TO* __restrict__ out, int ldo, const T* __restrict__ x, int ldx,
                  const T* __restrict__ w, int ldw, int M, int N, int K, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float xs[GP_BK][GP_BM + 1];
  __shared__ float ws[GP_BK][GP_BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * GP_BM, n0 = blockIdx.x * GP_BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GP_BK) {
    // 64 rows x 16 k per operand = 1024 elements, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      const int m = m0 + r, n = n0 + r;
      xs[kk][r] = (m < M && k < K) ? to_f32(x[(size_t)m * ldx + k]) : 0.f;
      ws[kk][r] = (n < N && k < K) ? to_f32(w[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GP_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)m * ldo + n] = from_f32<TO>(softcap_f32(acc[i][j], cap));
    }
  }
}

// `cap` > 0 applies cap * tanh(v / cap) to every output (the head's softcap).
AF_EXPORT int af_gemm_plain(void* out, int out_dtype, int ldo, const void* x, int ldx, const void* w,
                            int ldw, int dtype, int M, int N, int K, float cap, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  AF_REQUIRE(M > 0 && N > 0 && K > 0, "af_gemm_plain: bad sizes %d %d %d", M, N, K);
  dim3 grid((N + GP_BN - 1) / GP_BN, (M + GP_BM - 1) / GP_BM);
  AF_REQUIRE(grid.y <= 65535, "af_gemm_plain: M %d too large", M);
  AF_DISPATCH_DTYPE(dtype, T,
                    AF_DISPATCH_DTYPE(out_dtype, TO,
                                      af_launch(gemm_plain_kernel<T, TO>, dim3(grid), dim3(256), 0, stream, 
                                          (TO*)out, ldo, (const T*)x, ldx, (const T*)w, ldw, M, N, K,
                                          cap)));
  AF_CHECK_LAUNCH("af_gemm_plain");
}
