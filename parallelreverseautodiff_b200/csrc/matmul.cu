// Matrix-multiply entry points of the C ABI: the general GEMM, MatrixMultiplyOperation
// forward / backward (plain, fused with an activation derivative, batched), the
// MultiplyAndSum pair and the host-buffer form of the MatMul->activation node.
#include "act_math.cuh"
#include "common.cuh"
#include "reduce.cuh"

namespace prad {

template <typename T>
prad_status gemm_simt(prad_ctx* ctx, bool exact, bool tA, bool tB, int M, int N, int K,
                      double alpha, const void* A, int lda, const void* B, int ldb, double beta,
                      void* C, int ldc, int batch, int64_t sA, int64_t sB, int64_t sC,
                      const GemmEpilogue& e);

// tensor-core variants (return PRAD_ERR_UNSUPPORTED when a shape does not fit them)
prad_status gemm_tf32x3(prad_ctx* ctx, bool tA, bool tB, int M, int N, int K, double alpha,
                        const void* A, int lda, const void* B, int ldb, double beta, void* C,
                        int ldc, int batch, int64_t sA, int64_t sB, int64_t sC,
                        const GemmEpilogue& e, bool probe_only);
prad_status gemm_f64_dmma(prad_ctx* ctx, bool tA, bool tB, int M, int N, int K, double alpha,
                          const void* A, int lda, const void* B, int ldb, double beta, void* C,
                          int ldc, int batch, int64_t sA, int64_t sB, int64_t sC,
                          const GemmEpilogue& e, bool probe_only);

prad_status gemm_dispatch(prad_ctx* ctx, prad_dtype dt, bool tA, bool tB, int M, int N, int K,
                          double alpha, const void* A, int lda, const void* B, int ldb,
                          double beta, void* C, int ldc, int batch, int64_t sA, int64_t sB,
                          int64_t sC, const GemmEpilogue& epi) {
  if (M == 0 || N == 0 || batch == 0) return PRAD_OK;
  if (dt == PRAD_F32) {
    const bool want_tc = ctx->gemm_f32 == GemmF32::Auto || ctx->gemm_f32 == GemmF32::Tf32x3 ||
                         ctx->gemm_f32 == GemmF32::Tf32B16 || ctx->gemm_f32 == GemmF32::Bf16x3 ||
                         ctx->gemm_f32 == GemmF32::Fp16x3;
    if (want_tc) {
      prad_status p = gemm_tf32x3(ctx, tA, tB, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc,
                                  batch, sA, sB, sC, epi, true);
      if (p == PRAD_OK)
        return gemm_tf32x3(ctx, tA, tB, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, batch, sA,
                           sB, sC, epi, false);
    }
    return gemm_simt<float>(ctx, ctx->gemm_f32 != GemmF32::SimtFma, tA, tB, M, N, K, alpha, A, lda,
                            B, ldb, beta, C, ldc, batch, sA, sB, sC, epi);
  }
  const bool want_dmma = ctx->gemm_f64 == GemmF64::Auto || ctx->gemm_f64 == GemmF64::Dmma;
  if (want_dmma) {
    prad_status p = gemm_f64_dmma(ctx, tA, tB, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc,
                                  batch, sA, sB, sC, epi, true);
    if (p == PRAD_OK)
      return gemm_f64_dmma(ctx, tA, tB, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, batch, sA,
                           sB, sC, epi, false);
  }
  return gemm_simt<double>(ctx, ctx->gemm_f64 != GemmF64::SimtFma, tA, tB, M, N, K, alpha, A, lda,
                           B, ldb, beta, C, ldc, batch, sA, sB, sC, epi);
}

// ---- MultiplyAndSum ------------------------------------------------------------------------
// forward: out[q] = sum_ij (A*B_q)_ij  =  sum_k (sum_i A[i][k]) * (sum_j B_q[k][j]).
// The reference multiplies first and sums afterwards (MatrixMultiplyAndSumOperation.cs:
// 58-66); here the product is formed by the GEMM into scratch and reduced per slice by one
// CTA with a fixed-order block sum.
template <typename T>
__global__ void __launch_bounds__(256)
slice_sum_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t per_slice) {
  const T* xs = x + (int64_t)blockIdx.x * per_slice;
  double acc = 0.0;
  for (int64_t i = threadIdx.x; i < per_slice; i += 256) acc += (double)xs[i];
  double s = block_sum_d<256>(acc);
  if (threadIdx.x == 0) out[blockIdx.x] = (T)s;
}

// backward (MatrixMultiplyAndSumOperation.cs:70-89): dB_q = A^T * dOut[q] ;
// dA = sum_q B_q^T * dOut[q], q ascending, starting from a zero matrix.
template <typename T>
__global__ void __launch_bounds__(256)
mas_backward_dB_kernel(const T* __restrict__ A, const T* __restrict__ dOut, T* __restrict__ dB,
                       int R, int C, int P) {
  const int64_t per = (int64_t)C * R, total = per * P;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    int q = (int)(e / per);
    int64_t r = e % per;
    int i = (int)(r / R), j = (int)(r % R);  // dB_q[i][j] = A[j][i] * s
    dB[e] = mul_rn(A[(int64_t)j * C + i], dOut[q]);
  }
}
template <typename T>
__global__ void __launch_bounds__(256)
mas_backward_dA_kernel(const T* __restrict__ B, const T* __restrict__ dOut, T* __restrict__ dA,
                       int C, int N, int P) {
  const int64_t total = (int64_t)N * C;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    int i = (int)(e / C), j = (int)(e % C);  // dA[i][j] += B_q[j][i] * s
    T acc = (T)0;
    for (int q = 0; q < P; ++q)
      acc = add_rn(acc, mul_rn(B[(int64_t)q * C * N + (int64_t)j * N + i], dOut[q]));
    dA[e] = acc;
  }
}

static prad_status matmul_backward_impl(prad_ctx* ctx, prad_dtype dt, const void* A,
                                        const void* B, const void* dC, void* dA, void* dB, int M,
                                        int K, int N, int accumulate_dB, double dB_scale,
                                        prad_act act_below, const void* saved_below,
                                        double act_alpha) {
  prad_status s;
  if (dA) {
    GemmEpilogue e;
    e.dact = act_below;
    e.saved = saved_below;
    e.act_alpha = act_alpha;
    // dA (MxK) = dC (MxN) * B^T  (B is KxN)
    s = gemm_dispatch(ctx, dt, false, true, M, K, N, 1.0, dC, N, B, N, 0.0, dA, K, 1, 0, 0, 0, e);
    if (s) return s;
  }
  if (dB) {
    GemmEpilogue e;
    // dB (KxN) = A^T (A is MxK) * dC (MxN)
    s = gemm_dispatch(ctx, dt, true, false, K, N, M, dB_scale, A, K, dC, N,
                      accumulate_dB ? 1.0 : 0.0, dB, N, 1, 0, 0, 0, e);
    if (s) return s;
  }
  return PRAD_OK;
}

}  // namespace prad

using namespace prad;

#define CHECK_DIMS(who, M, K, N)                                                          \
  PRAD_REQUIRE((M) >= 0 && (K) >= 0 && (N) >= 0, PRAD_ERR_SHAPE, who ": negative dimension")

extern "C" {

prad_status prad_gemm(prad_ctx* ctx, prad_dtype dt, int transA, int transB, int M, int N, int K,
                      double alpha, const void* A, int lda, const void* B, int ldb, double beta,
                      void* C, int ldc, int batch, int64_t strideA, int64_t strideB,
                      int64_t strideC) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_gemm: bad dtype");
  PRAD_REQUIRE(M >= 0 && N >= 0 && K >= 0 && batch >= 0, PRAD_ERR_SHAPE, "prad_gemm: negative dimension");
  if (M == 0 || N == 0 || batch == 0) return PRAD_OK;
  PRAD_REQUIRE(C && (K == 0 || (A && B)), PRAD_ERR_INVALID, "prad_gemm: null pointer");
  PRAD_REQUIRE(lda >= (transA ? M : K) && ldb >= (transB ? K : N) && ldc >= N, PRAD_ERR_SHAPE,
               "prad_gemm: leading dimension smaller than the row length");
  GemmEpilogue e;
  return gemm_dispatch(ctx, dt, transA != 0, transB != 0, M, N, K, alpha, A, lda, B, ldb, beta, C,
                       ldc, batch, strideA, strideB, strideC, e);
}

prad_status prad_matmul_forward(prad_ctx* ctx, prad_dtype dt, const void* A, const void* B,
                                void* Y, int M, int K, int N, const void* bias, void* Z_out,
                                prad_act act, double act_alpha) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_matmul_forward: bad dtype");
  CHECK_DIMS("prad_matmul_forward", M, K, N);
  if (M == 0 || N == 0) return PRAD_OK;
  PRAD_REQUIRE(Y && (K == 0 || (A && B)), PRAD_ERR_INVALID, "prad_matmul_forward: null pointer");
  GemmEpilogue e;
  e.bias = bias;
  e.z_out = Z_out;
  e.act = act;
  e.act_alpha = act_alpha;
  return gemm_dispatch(ctx, dt, false, false, M, N, K, 1.0, A, K, B, N, 0.0, Y, N, 1, 0, 0, 0, e);
}

prad_status prad_matmul_backward(prad_ctx* ctx, prad_dtype dt, const void* A, const void* B,
                                 const void* dC, void* dA, void* dB, int M, int K, int N,
                                 int accumulate_dB, double dB_scale, prad_act act_below,
                                 const void* saved_below, double act_alpha) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_matmul_backward: bad dtype");
  CHECK_DIMS("prad_matmul_backward", M, K, N);
  PRAD_REQUIRE(dC || M == 0 || N == 0, PRAD_ERR_INVALID, "prad_matmul_backward: dC is null");
  PRAD_REQUIRE(!dA || B || K == 0 || N == 0, PRAD_ERR_INVALID, "prad_matmul_backward: dA needs B");
  PRAD_REQUIRE(!dB || A || K == 0 || M == 0, PRAD_ERR_INVALID, "prad_matmul_backward: dB needs A");
  PRAD_REQUIRE(act_below == PRAD_ACT_NONE || saved_below, PRAD_ERR_INVALID,
               "prad_matmul_backward: activation given without its saved tensor");
  return matmul_backward_impl(ctx, dt, A, B, dC, dA, dB, M, K, N, accumulate_dB, dB_scale,
                              act_below, saved_below, act_alpha);
}

prad_status prad_matmul_act_backward(prad_ctx* ctx, prad_dtype dt, const void* A, const void* B,
                                     const void* dOut, prad_act act, const void* saved,
                                     double act_alpha, void* dPre, void* dA, void* dB, int M,
                                     int K, int N) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_matmul_act_backward: bad dtype");
  CHECK_DIMS("prad_matmul_act_backward", M, K, N);
  PRAD_REQUIRE(dPre && dOut && (saved || act == PRAD_ACT_NONE), PRAD_ERR_INVALID,
               "prad_matmul_act_backward: null pointer");
  prad_status s = prad_act_backward(ctx, dt, act, saved ? saved : dOut, dOut, dPre, (int64_t)M * N, act_alpha);
  if (s) return s;
  return matmul_backward_impl(ctx, dt, A, B, dPre, dA, dB, M, K, N, 0, 1.0, PRAD_ACT_NONE, nullptr, 0.0);
}

prad_status prad_matmul_act_backward_host(prad_ctx* ctx, prad_dtype dt, const void* A_host,
                                          const void* B_host, const void* dOut_host,
                                          prad_act act, const void* saved_host, double act_alpha,
                                          void* dPre_host, void* dA_host, void* dB_host, int M,
                                          int K, int N) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_matmul_act_backward_host: bad dtype");
  CHECK_DIMS("prad_matmul_act_backward_host", M, K, N);
  PRAD_NOT_CAPTURING(ctx, "prad_matmul_act_backward_host");
  PRAD_REQUIRE(A_host && B_host && dOut_host && dPre_host && dA_host && dB_host &&
                   (saved_host || act == PRAD_ACT_NONE),
               PRAD_ERR_INVALID, "prad_matmul_act_backward_host: null pointer");
  const size_t es = dtype_size(dt);
  auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
  const size_t bA = al((size_t)M * K * es), bB = al((size_t)K * N * es), bC = al((size_t)M * N * es);
  prad_status s = ensure_stage(ctx, 2 * bA + 2 * bB + 3 * bC);
  if (s) return s;
  char* p = (char*)ctx->stage;
  void* dA_in = p; p += bA;
  void* dB_in = p; p += bB;
  void* dO = p; p += bC;
  void* dS = p; p += bC;
  void* dP = p; p += bC;
  void* dA_out = p; p += bA;
  void* dB_out = p;
  cudaStream_t st = ctx->stream;
  PRAD_CUDA(cudaMemcpyAsync(dA_in, A_host, (size_t)M * K * es, cudaMemcpyHostToDevice, st));
  PRAD_CUDA(cudaMemcpyAsync(dB_in, B_host, (size_t)K * N * es, cudaMemcpyHostToDevice, st));
  PRAD_CUDA(cudaMemcpyAsync(dO, dOut_host, (size_t)M * N * es, cudaMemcpyHostToDevice, st));
  if (saved_host) PRAD_CUDA(cudaMemcpyAsync(dS, saved_host, (size_t)M * N * es, cudaMemcpyHostToDevice, st));
  s = prad_matmul_act_backward(ctx, dt, dA_in, dB_in, dO, act, saved_host ? dS : nullptr, act_alpha, dP, dA_out, dB_out, M, K, N);
  if (s) return s;
  PRAD_CUDA(cudaMemcpyAsync(dPre_host, dP, (size_t)M * N * es, cudaMemcpyDeviceToHost, st));
  PRAD_CUDA(cudaMemcpyAsync(dA_host, dA_out, (size_t)M * K * es, cudaMemcpyDeviceToHost, st));
  PRAD_CUDA(cudaMemcpyAsync(dB_host, dB_out, (size_t)K * N * es, cudaMemcpyDeviceToHost, st));
  PRAD_CUDA(cudaStreamSynchronize(st));
  return PRAD_OK;
}

prad_status prad_batch_matmul_forward(prad_ctx* ctx, prad_dtype dt, const void* A, const void* B,
                                      void* C, int depth, int M, int K, int N, int b_shared) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_batch_matmul_forward: bad dtype");
  CHECK_DIMS("prad_batch_matmul_forward", M, K, N);
  PRAD_REQUIRE(depth >= 0, PRAD_ERR_SHAPE, "prad_batch_matmul_forward: negative depth");
  if (depth == 0 || M == 0 || N == 0) return PRAD_OK;
  PRAD_REQUIRE(C && (K == 0 || (A && B)), PRAD_ERR_INVALID, "prad_batch_matmul_forward: null pointer");
  GemmEpilogue e;
  if (b_shared)  // every slice multiplies the same B: one tall product
    return gemm_dispatch(ctx, dt, false, false, depth * M, N, K, 1.0, A, K, B, N, 0.0, C, N, 1, 0, 0, 0, e);
  return gemm_dispatch(ctx, dt, false, false, M, N, K, 1.0, A, K, B, N, 0.0, C, N, depth,
                       (int64_t)M * K, (int64_t)K * N, (int64_t)M * N, e);
}

prad_status prad_batch_matmul_backward(prad_ctx* ctx, prad_dtype dt, const void* A,
                                       const void* B, const void* dC, void* dA, void* dB,
                                       void* dB_mean, int depth, int M, int K, int N,
                                       int b_shared) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_batch_matmul_backward: bad dtype");
  CHECK_DIMS("prad_batch_matmul_backward", M, K, N);
  PRAD_REQUIRE(depth >= 0, PRAD_ERR_SHAPE, "prad_batch_matmul_backward: negative depth");
  PRAD_REQUIRE(!dB_mean || b_shared, PRAD_ERR_INVALID,
               "prad_batch_matmul_backward: dB_mean only exists for a shared B");
  if (depth == 0) return PRAD_OK;
  PRAD_REQUIRE(dC && A && B, PRAD_ERR_INVALID, "prad_batch_matmul_backward: null pointer");
  GemmEpilogue e;
  prad_status s;
  if (dA) {
    if (b_shared)
      s = gemm_dispatch(ctx, dt, false, true, depth * M, K, N, 1.0, dC, N, B, N, 0.0, dA, K, 1, 0, 0, 0, e);
    else
      s = gemm_dispatch(ctx, dt, false, true, M, K, N, 1.0, dC, N, B, N, 0.0, dA, K, depth,
                        (int64_t)M * N, (int64_t)K * N, (int64_t)M * K, e);
    if (s) return s;
  }
  if (dB) {
    s = gemm_dispatch(ctx, dt, true, false, K, N, M, 1.0, A, K, dC, N, 0.0, dB, N, depth,
                      (int64_t)M * K, (int64_t)M * N, (int64_t)K * N, e);
    if (s) return s;
  }
  if (dB_mean) {  // (1/depth) * sum_d A_d^T dC_d  ==  one product with K' = depth*M
    s = gemm_dispatch(ctx, dt, true, false, K, N, depth * M, 1.0 / (double)depth, A, K, dC, N, 0.0,
                      dB_mean, N, 1, 0, 0, 0, e);
    if (s) return s;
  }
  return PRAD_OK;
}

prad_status prad_matmul_and_sum_forward(prad_ctx* ctx, prad_dtype dt, const void* A,
                                        const void* B, void* out, int R, int C, int N, int P) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_matmul_and_sum_forward: bad dtype");
  PRAD_REQUIRE(R > 0 && C > 0 && N > 0 && P > 0, PRAD_ERR_SHAPE, "prad_matmul_and_sum_forward: empty operand");
  PRAD_REQUIRE(A && B && out, PRAD_ERR_INVALID, "prad_matmul_and_sum_forward: null pointer");
  const size_t es = dtype_size(dt);
  prad_status s = ensure_stage(ctx, (size_t)P * R * N * es);
  if (s) return s;
  GemmEpilogue e;
  s = gemm_dispatch(ctx, dt, false, false, R, N, C, 1.0, A, C, B, N, 0.0, ctx->stage, N, P, 0,
                    (int64_t)C * N, (int64_t)R * N, e);
  if (s) return s;
  if (dt == PRAD_F32) slice_sum_kernel<float><<<P, 256, 0, ctx->stream>>>((const float*)ctx->stage, (float*)out, (int64_t)R * N);
  else slice_sum_kernel<double><<<P, 256, 0, ctx->stream>>>((const double*)ctx->stage, (double*)out, (int64_t)R * N);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_matmul_and_sum_backward(prad_ctx* ctx, prad_dtype dt, const void* A,
                                         const void* B, const void* dOut, void* dA, void* dB,
                                         int R, int C, int N, int P) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_matmul_and_sum_backward: bad dtype");
  PRAD_REQUIRE(R > 0 && C > 0 && N > 0 && P > 0, PRAD_ERR_SHAPE, "prad_matmul_and_sum_backward: empty operand");
  PRAD_REQUIRE(A && B && dOut && dA && dB, PRAD_ERR_INVALID, "prad_matmul_and_sum_backward: null pointer");
  int g1 = stream_grid(ctx, (int64_t)P * C * R, 256, 8), g2 = stream_grid(ctx, (int64_t)N * C, 256, 8);
  if (dt == PRAD_F32) {
    mas_backward_dB_kernel<float><<<g1, 256, 0, ctx->stream>>>((const float*)A, (const float*)dOut, (float*)dB, R, C, P);
    PRAD_LAUNCHED(ctx);
    mas_backward_dA_kernel<float><<<g2, 256, 0, ctx->stream>>>((const float*)B, (const float*)dOut, (float*)dA, C, N, P);
  } else {
    mas_backward_dB_kernel<double><<<g1, 256, 0, ctx->stream>>>((const double*)A, (const double*)dOut, (double*)dB, R, C, P);
    PRAD_LAUNCHED(ctx);
    mas_backward_dA_kernel<double><<<g2, 256, 0, ctx->stream>>>((const double*)B, (const double*)dOut, (double*)dA, C, N, P);
  }
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

}  // extern "C"
