// FP64 GEMM on the tensor cores (DMMA): C = alpha*op(A)*op(B) + beta*C with
// mma.sync.aligned.m8n8k4.row.col.f64 tiles.  tcgen05.mma has no FP64 kind, so double
// precision stays on the warp-level MMA path.
//
// Two kernels.
//   gemm_dmma_async_kernel (large products): a CTA owns a 128 x 128 tile, its 8 warps a 64 x 32 sub-tile
//   each (8 x 4 MMA tiles, 64 accumulator doubles per thread, 12 fragment loads per 32 MMAs); k advances
//   in blocks of 16 through a three-stage ring of shared-memory tiles filled with cp.async (16-byte
//   copies, zero-filled outside the matrix; 8-byte copies when a pitch or pointer is not 16-byte
//   aligned), so two blocks are in flight while one is multiplied and no thread ever holds operand data
//   in registers on its way to shared memory.  Each operand keeps the orientation it has in global
//   memory -- [mn][k] with pitch 20 doubles when k is contiguous, [k][mn] with pitch 136 when mn is --
//   and both pitches put the 32 lanes of a fragment load into the minimum two wavefronts.
//   (cp.async rather than TMA: a double matrix with an odd pitch cannot be described by a tensor map,
//   and the k-contiguous form would need 16 x 8-byte boxes; cp.async serves every shape with one code
//   path and the copies overlap the MMAs just the same.)
//   gemm_dmma_kernel (small M or N): 64 x 64 tiles, 32 x 16 per warp, register-prefetch double buffer.
//
// The summation order inside a DMMA differs from the managed code's sequential loop, so this
// variant is held to the tolerance, not to bit equality; "auto" uses it only for large
// products and keeps the bit-exact FMA-free kernel for everything else.
#include <atomic>

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
                 EpiParams<double> epi, int kslices = 1, int64_t kA = 0, int64_t kB = 0) {
  // kslices > 1: blockIdx.z = batch * kslices + slice; slice s multiplies k range [s K, (s + 1) K) (operands kA / kB
  // elements further on) into its own dense M x N block of C (sC apart, slices of a batch consecutive)
  constexpr int BM = 64, BN = 64, BK = 16, NT = 256, PAD = 8;
  __shared__ __align__(16) double As[2][BK][BM + PAD];
  __shared__ __align__(16) double Bs[2][BK][BN + PAD];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = (warp >> 2) * 32, wn = (warp & 3) * 16;   // warp tile origin inside the CTA tile
  const int g = lane >> 2, q = lane & 3;                    // fragment row group / k index
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int64_t bz = blockIdx.z;
  if (kslices > 1) {
    const int64_t b = bz / kslices, sl = bz - b * kslices;
    A += b * sA + sl * kA;
    B += b * sB + sl * kB;
  } else {
    A += bz * sA;
    B += bz * sB;
  }
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

// ---------------------------------------------------------------- 128 x 128 tiles, cp.async ring
namespace dm {
constexpr int BM = 128, BN = 128, BK = 16, STAGES = 3, NT = 256;
constexpr int LDK = BK + 4;        // pitch of a [mn][k] tile (k contiguous in memory)
constexpr int LDM = BM + 8;        // pitch of a [k][mn] tile (mn contiguous in memory)
constexpr int TILE_DOUBLES = (BM * LDK > BK * LDM) ? BM * LDK : BK * LDM;     // either layout fits
constexpr int SMEM_BYTES = STAGES * 2 * TILE_DOUBLES * (int)sizeof(double);

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async8(void* dst, const void* src, int src_bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Copies the (128 x 16) operand tile at (mn0, k0) into `tile`.  K_CONTIG: memory is [mn][k] (k contiguous),
// shared layout [mn][LDK]; otherwise memory is [k][mn], shared layout [k][LDM].  Out-of-range elements
// become zero (src-size 0 keeps the address unread; it is clamped to the matrix anyway).
template <bool K_CONTIG>
__device__ __forceinline__ void load_tile(double* tile, const double* __restrict__ p, int64_t ld, int mn0, int k0, int MN,
                                          int K, bool vec, int tid) {
  constexpr int FAST = K_CONTIG ? BK : BM;       // contiguous extent of the tile
  constexpr int SLOW = K_CONTIG ? BM : BK;
  constexpr int PITCH = K_CONTIG ? LDK : LDM;
  const int fast0 = K_CONTIG ? k0 : mn0, slow0 = K_CONTIG ? mn0 : k0;
  const int fast_lim = K_CONTIG ? K : MN, slow_lim = K_CONTIG ? MN : K;
  constexpr int CHUNKS = SLOW * FAST / 2;        // 16-byte chunks
#pragma unroll
  for (int it = 0; it < CHUNKS / NT; ++it) {
    const int idx = tid + it * NT;
    const int s = idx / (FAST / 2), f = (idx % (FAST / 2)) * 2;
    const int gs = slow0 + s, gf = fast0 + f;
    double* dst = tile + s * PITCH + f;
    const bool row_ok = gs < slow_lim;
    const double* src = p + (int64_t)(row_ok ? gs : 0) * ld + (gf < fast_lim ? gf : 0);
    if (vec) {
      const int bytes = !row_ok ? 0 : (gf + 2 <= fast_lim ? 16 : (gf < fast_lim ? 8 : 0));
      cp_async16(dst, src, bytes);
    } else {
      cp_async8(dst, src, (row_ok && gf < fast_lim) ? 8 : 0);
      const double* src1 = p + (int64_t)(row_ok ? gs : 0) * ld + (gf + 1 < fast_lim ? gf + 1 : 0);
      cp_async8(dst + 1, src1, (row_ok && gf + 1 < fast_lim) ? 8 : 0);
    }
  }
}
// fragment element (mn, k) of a tile in either layout
template <bool K_CONTIG>
__device__ __forceinline__ double frag(const double* tile, int mn, int k) {
  return K_CONTIG ? tile[mn * LDK + k] : tile[k * LDM + mn];
}
}  // namespace dm

template <bool TA, bool TB>
__global__ void __launch_bounds__(dm::NT, 1)
gemm_dmma_async_kernel(int M, int N, int K, double alpha, const double* __restrict__ A, int64_t lda,
                       const double* __restrict__ B, int64_t ldb, double beta, double* __restrict__ C,
                       int64_t ldc, int64_t sA, int64_t sB, int64_t sC, bool vecA, bool vecB, bool vecC,
                       EpiParams<double> epi) {
  using namespace dm;
  extern __shared__ __align__(16) double dsm[];
  // op(A) is M x K: k is contiguous in memory unless TA.  op(B) is K x N: n is contiguous unless TB.
  constexpr bool A_KC = !TA, B_KC = TB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
  const int g = lane >> 2, q = lane & 3;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int64_t bz = blockIdx.z;
  A += bz * sA;
  B += bz * sB;
  C += bz * sC;
  const double* saved = epi.saved ? epi.saved + bz * sC : nullptr;
  double* z_out = epi.z_out ? epi.z_out + bz * sC : nullptr;
  auto a_tile = [&](int s) { return dsm + (size_t)s * 2 * TILE_DOUBLES; };
  auto b_tile = [&](int s) { return dsm + (size_t)s * 2 * TILE_DOUBLES + TILE_DOUBLES; };

  double acc[8][4][2];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

  const int ktiles = (K + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {        // prologue: two blocks in flight
    if (s < ktiles) {
      load_tile<A_KC>(a_tile(s), A, lda, m0, s * BK, M, K, vecA, tid);
      load_tile<B_KC>(b_tile(s), B, ldb, n0, s * BK, N, K, vecB, tid);
    }
    cp_async_commit();
  }
  for (int kt = 0; kt < ktiles; ++kt) {
    cp_async_wait<STAGES - 2>();                // block kt has landed (for this thread's copies)
    __syncthreads();                            // ... and for everybody's; block kt-1's stage is free
    const int nxt = kt + STAGES - 1;
    if (nxt < ktiles) {
      load_tile<A_KC>(a_tile(nxt % STAGES), A, lda, m0, nxt * BK, M, K, vecA, tid);
      load_tile<B_KC>(b_tile(nxt % STAGES), B, ldb, n0, nxt * BK, N, K, vecB, tid);
    }
    cp_async_commit();
    const double* as = a_tile(kt % STAGES);
    const double* bs = b_tile(kt % STAGES);
#pragma unroll
    for (int k4 = 0; k4 < BK; k4 += 4) {
      double a[8], b[4];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = frag<A_KC>(as, wm + i * 8 + g, k4 + q);
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = frag<B_KC>(bs, wn + j * 8 + g, k4 + q);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dmma_m8n8k4(acc[i][j][0], acc[i][j][1], a[i], b[j]);
    }
  }
  cp_async_wait<0>();

  // epilogue: thread holds rows wm + i*8 + g, columns wn + j*8 + 2q + {0,1}
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + wm + i * 8 + g;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
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

// C = alpha * (P_0 + P_1 + ...) + beta * C, slices added in order; P_s are dense M x N.
__global__ void __launch_bounds__(256)
splitk_combine_f64_kernel(const double* __restrict__ part, int splits, int64_t mn, int N, double* __restrict__ C,
                          int64_t ldc, int64_t sC, double alpha, double beta) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  part += (int64_t)blockIdx.y * splits * mn;      // blockIdx.y = batch
  C += (int64_t)blockIdx.y * sC;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < mn; i += stride) {
    double acc = part[i];
    for (int s = 1; s < splits; ++s) acc = __dadd_rn(acc, part[(int64_t)s * mn + i]);
    const int64_t off = (i / N) * ldc + (i % N);
    double v = __dmul_rn(alpha, acc);
    if (beta != 0.0) v = (beta == 1.0) ? __dadd_rn(C[off], v) : fma(beta, C[off], v);
    C[off] = v;
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
  // large tiles when both extents fill them and there are enough of them to occupy the machine
  const bool large = M >= 128 && N >= 128 &&
                     (int64_t)ceil_div(M, dm::BM) * ceil_div(N, dm::BN) * batch >= ctx->sm_count;
  if (large) {
    dim3 g2((unsigned)ceil_div(N, dm::BN), (unsigned)ceil_div(M, dm::BM), (unsigned)batch);
    PRAD_REQUIRE(g2.y <= 65535, PRAD_ERR_UNSUPPORTED, "gemm dmma: too many row tiles (%u)", g2.y);
#define PRAD_DMMA_ASYNC(TA_, TB_)                                                                              \
  do {                                                                                                          \
    static std::atomic<uint64_t> done{0};                                                                       \
    const uint64_t bit = 1ull << (ctx->device & 63);                                                            \
    if (!(done.load(std::memory_order_acquire) & bit)) {                                                        \
      const cudaError_t ae = cudaFuncSetAttribute(gemm_dmma_async_kernel<TA_, TB_>,                             \
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, dm::SMEM_BYTES); \
      PRAD_REQUIRE(ae == cudaSuccess, PRAD_ERR_CUDA, "gemm dmma: cannot reserve %d bytes of shared memory: %s", \
                   dm::SMEM_BYTES, cudaGetErrorString(ae));                                                     \
      done.fetch_or(bit, std::memory_order_release);                                                            \
    }                                                                                                           \
    gemm_dmma_async_kernel<TA_, TB_><<<g2, dm::NT, dm::SMEM_BYTES, ctx->stream>>>(                              \
        M, N, K, alpha, Ad, lda, Bd, ldb, beta, Cd, ldc, sA, sB, sC, vA, vB, vC, epi);                          \
  } while (0)
    if (!tA && !tB) PRAD_DMMA_ASYNC(false, false);
    else if (!tA && tB) PRAD_DMMA_ASYNC(false, true);
    else if (tA && !tB) PRAD_DMMA_ASYNC(true, false);
    else PRAD_DMMA_ASYNC(true, true);
#undef PRAD_DMMA_ASYNC
    PRAD_LAUNCHED(ctx);
    return PRAD_OK;
  }
  // Few output tiles and a long k (the time-batched weight gradients of an LSTM: 128 x 1024 outputs over k = 2048 run on
  // 32 CTAs): k is cut into slices that run as the "batch" dimension into scratch, and an ordered pass adds them.
  const int64_t tiles = (int64_t)grid.x * grid.y * batch;
  const bool plain = !e.bias && !e.z_out && e.act == PRAD_ACT_NONE && e.dact == PRAD_ACT_NONE;
  if (plain && tiles * 2 <= ctx->sm_count && K >= 1024 && batch <= 65535) {
    int S = (int)(ctx->sm_count / tiles);
    if (S > K / 256) S = K / 256;
    while (S > 1 && K % S != 0) --S;
    if (S >= 2 && (int64_t)batch * S <= 65535) {
      const int Ks = K / S;
      const int64_t mn = (int64_t)M * N;
      prad_status st = ensure_stage(ctx, (size_t)batch * S * mn * sizeof(double));
      if (st) return st;
      double* part = (double*)ctx->stage;
      const int64_t zA = tA ? (int64_t)Ks * lda : Ks, zB = tB ? Ks : (int64_t)Ks * ldb;
      const bool wA = vA && zA % 2 == 0, wB = vB && zB % 2 == 0;
      const bool wC = N % 2 == 0;
      dim3 gs(grid.x, grid.y, (unsigned)(batch * S));
      EpiParams<double> none{nullptr, nullptr, 0, 0, nullptr, 0.0};
#define PRAD_DMMA_SLICES(TA_, TB_)                                                                                 \
  gemm_dmma_kernel<TA_, TB_><<<gs, 256, 0, ctx->stream>>>(M, N, Ks, 1.0, Ad, lda, Bd, ldb, 0.0, part, N, sA, sB, mn, \
                                                          wA, wB, wC, none, S, zA, zB)
      if (!tA && !tB) PRAD_DMMA_SLICES(false, false);
      else if (!tA && tB) PRAD_DMMA_SLICES(false, true);
      else if (tA && !tB) PRAD_DMMA_SLICES(true, false);
      else PRAD_DMMA_SLICES(true, true);
#undef PRAD_DMMA_SLICES
      PRAD_LAUNCHED(ctx);
      const int cg = stream_grid(ctx, mn, 256, 8);
      splitk_combine_f64_kernel<<<dim3((unsigned)cg, (unsigned)batch), 256, 0, ctx->stream>>>(part, S, mn, N, Cd, ldc, sC,
                                                                                           alpha, beta);
      PRAD_LAUNCHED(ctx);
      return PRAD_OK;
    }
  }
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
