// FP64 GEMM on the tensor cores (DMMA): C = alpha*op(A)*op(B) + beta*C with
// mma.sync.aligned.m8n8k4.row.col.f64 tiles.  tcgen05.mma has no FP64 kind, so double
// precision stays on the warp-level MMA path.
//
// A CTA owns a 64 x 64 tile, its 8 warps a 32 x 16 sub-tile each (4 x 2 MMA tiles, 16
// accumulator doubles per thread); k advances in blocks of 16 staged through shared memory
// as [k][m] / [k][n] panels whose row pitch (72 doubles) puts the four k-rows a fragment
// load touches into two bank groups, i.e. the minimum two wavefronts per 256-byte load.
// Operand tiles are read with 128-bit global loads into registers one k-block ahead.
// (No TMA here: arbitrary double matrices rarely meet TMA's 16-byte pitch rule, and the
// transposed forms would need sub-tiled boxes; the loader below handles every shape.)
//
// The summation order inside a DMMA differs from the managed code's sequential loop, so this
// variant is held to the tolerance, not to bit equality; "auto" uses it only for large
// products and keeps the bit-exact FMA-free kernel for everything else.
#include "gemm_tiles.cuh"

namespace prad {

__device__ __forceinline__ void dmma_m8n8k4(double& d0, double& d1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
               : "+d"(d0), "+d"(d1) : "d"(a), "d"(b));
}

template <bool TA, bool TB>
__global__ void __launch_bounds__(256)
gemm_dmma_kernel(int M, int N, int K, double alpha, const double* __restrict__ A, int64_t lda,
                 const double* __restrict__ B, int64_t ldb, double beta, double* __restrict__ C,
                 int64_t ldc, int64_t sA, int64_t sB, int64_t sC, bool vecA, bool vecB, bool vecC,
                 EpiParams<double> epi) {
  constexpr int BM = 64, BN = 64, BK = 16, NT = 256, PAD = 8;
  __shared__ __align__(16) double As[2][BK][BM + PAD];
  __shared__ __align__(16) double Bs[2][BK][BN + PAD];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = (warp >> 2) * 32, wn = (warp & 3) * 16;   // warp tile origin inside the CTA tile
  const int g = lane >> 2, q = lane & 3;                    // fragment row group / k index
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int64_t bz = blockIdx.z;
  A += bz * sA;
  B += bz * sB;
  C += bz * sC;
  const double* saved = epi.saved ? epi.saved + bz * sC : nullptr;
  double* z_out = epi.z_out ? epi.z_out + bz * sC : nullptr;

  TileLoader<double, BM, BK, NT, !TA> la;
  TileLoader<double, BN, BK, NT, TB> lb;

  double acc[4][2][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

  const int ktiles = (K + BK - 1) / BK;
  la.load(A, lda, m0, 0, M, K, vecA, tid);
  lb.load(B, ldb, n0, 0, N, K, vecB, tid);
  la.store(As[0], tid);
  lb.store(Bs[0], tid);
  __syncthreads();

  for (int kt = 0; kt < ktiles; ++kt) {
    const int cur = kt & 1;
    if (kt + 1 < ktiles) {
      la.load(A, lda, m0, (kt + 1) * BK, M, K, vecA, tid);
      lb.load(B, ldb, n0, (kt + 1) * BK, N, K, vecB, tid);
    }
#pragma unroll
    for (int k4 = 0; k4 < BK; k4 += 4) {
      double a[4], b[2];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[cur][k4 + q][wm + i * 8 + g];
#pragma unroll
      for (int j = 0; j < 2; ++j) b[j] = Bs[cur][k4 + q][wn + j * 8 + g];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) dmma_m8n8k4(acc[i][j][0], acc[i][j][1], a[i], b[j]);
    }
    if (kt + 1 < ktiles) {
      la.store(As[cur ^ 1], tid);
      lb.store(Bs[cur ^ 1], tid);
    }
    __syncthreads();
  }

  // epilogue: thread holds rows wm + i*8 + g, columns wn + j*8 + 2q + {0,1}
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + wm + i * 8 + g;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int n = n0 + wn + j * 8 + 2 * q;
      if (n >= N) continue;
      const int64_t off = (int64_t)m * ldc + n;
      const bool pair = vecC && (n + 2 <= N);
      double out[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        double v = alpha * acc[i][j][e];
        if (n + e < N) {
          if (beta != 0.0) v = fma(beta, C[off + e], v);
          if (epi.bias) v += epi.bias[n + e];
          if (z_out) z_out[off + e] = v;
          if (epi.act != PRAD_ACT_NONE) v = act_value<double>((prad_act)epi.act, v, epi.act_alpha);
          if (epi.dact != PRAD_ACT_NONE)
            v = mul_rn(v, act_derivative<double>((prad_act)epi.dact, saved[off + e], epi.act_alpha));
        }
        out[e] = v;
      }
      if (pair) {
        *reinterpret_cast<double2*>(C + off) = make_double2(out[0], out[1]);
      } else {
        C[off] = out[0];
        if (n + 1 < N) C[off + 1] = out[1];
      }
    }
  }
}

prad_status gemm_f64_dmma(prad_ctx* ctx, bool tA, bool tB, int M, int N, int K, double alpha,
                          const void* A, int lda, const void* B, int ldb, double beta, void* C,
                          int ldc, int batch, int64_t sA, int64_t sB, int64_t sC,
                          const GemmEpilogue& e, bool probe_only) {
  const bool forced = ctx->gemm_f64 == GemmF64::Dmma;
  const bool big = (int64_t)M * N * K * batch >= ((int64_t)1 << 27) && M >= 32 && N >= 32;
  if (!(forced || big) || K < 1) return PRAD_ERR_UNSUPPORTED;
  if (probe_only) return PRAD_OK;
  dim3 grid((unsigned)ceil_div(N, 64), (unsigned)ceil_div(M, 64), (unsigned)batch);
  PRAD_REQUIRE(grid.y <= 65535 && grid.z <= 65535, PRAD_ERR_UNSUPPORTED,
               "gemm dmma: grid too large (M tiles %u, batch %u)", grid.y, grid.z);
  EpiParams<double> epi{(const double*)e.bias, (double*)e.z_out, (int)e.act, (int)e.dact,
                        (const double*)e.saved, e.act_alpha};
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  bool vA = al(A) && lda % 2 == 0 && sA % 2 == 0;
  bool vB = al(B) && ldb % 2 == 0 && sB % 2 == 0;
  bool vC = al(C) && ldc % 2 == 0 && sC % 2 == 0;
  const double* Ad = (const double*)A;
  const double* Bd = (const double*)B;
  double* Cd = (double*)C;
#define PRAD_DMMA_LAUNCH(TA_, TB_)                                                          \
  gemm_dmma_kernel<TA_, TB_><<<grid, 256, 0, ctx->stream>>>(M, N, K, alpha, Ad, lda, Bd, ldb, \
                                                            beta, Cd, ldc, sA, sB, sC, vA, vB, vC, epi)
  if (!tA && !tB) PRAD_DMMA_LAUNCH(false, false);
  else if (!tA && tB) PRAD_DMMA_LAUNCH(false, true);
  else if (tA && !tB) PRAD_DMMA_LAUNCH(true, false);
  else PRAD_DMMA_LAUNCH(true, true);
#undef PRAD_DMMA_LAUNCH
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

}  // namespace prad
