// SIMT GEMM family (FP32 FMA / FP64 DFMA): C = alpha*op(A)*op(B) + beta*C, row-major,
// any M/N/K, strided-batched, with the fused epilogues of the backward path.
//
// This is the always-available variant: every product in the storage precision, k ascending,
// either with separately rounded multiply and add (EXACT: bit-identical to the managed
// code's sequential `+=` loop, the default) or with FMA accumulation (twice the rate), for
// all transpose forms the backward needs
//   NN  C = A*B          MatrixMultiplyOperation.Forward   (MatrixMultiplyOperation.cs:50-80)
//   NT  dA = dC*B^T      MatrixMultiplyOperation.Backward  (:94-104)
//   TN  dB = A^T*dC      MatrixMultiplyOperation.Backward  (:110-120)
// Register-tiled: a CTA owns a BM x BN tile, every thread a TM x TN sub-tile made of
// VEC-wide chunks so that shared-memory reads are 128-bit and conflict free; operand
// tiles are staged through registers (global -> reg -> smem) so the next tile's loads
// are in flight while the current one is multiplied.
#include "gemm_tiles.cuh"

namespace prad {

template <typename T, int BM, int BN, int BK, int TM, int TN, bool TA, bool TB, bool EXACT>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(int M, int N, int K, T alpha, const T* __restrict__ A, int64_t lda,
                 const T* __restrict__ B, int64_t ldb, T beta, T* __restrict__ C, int64_t ldc,
                 int64_t sA, int64_t sB, int64_t sC, bool vecA, bool vecB, bool vecC,
                 EpiParams<T> epi) {
  constexpr int VEC = VecOf<T>::N;
  using V = typename VecOf<T>::type;
  constexpr int NT = (BM / TM) * (BN / TN);
  constexpr int TX = BN / TN;  // threads along n
  constexpr int CM = TM / VEC, CN = TN / VEC;  // chunks per thread
  constexpr int PAD = VEC;                     // keeps rows 16-byte aligned
  static_assert(TM % VEC == 0 && TN % VEC == 0, "thread tile must be made of vectors");

  __shared__ __align__(16) T As[2][BK][BM + PAD];
  __shared__ __align__(16) T Bs[2][BK][BN + PAD];

  const int tid = threadIdx.x;
  const int tx = tid % TX, ty = tid / TX;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int64_t bz = blockIdx.z;
  A += bz * sA;
  B += bz * sB;
  C += bz * sC;
  const T* saved = epi.saved ? epi.saved + bz * sC : nullptr;
  T* z_out = epi.z_out ? epi.z_out + bz * sC : nullptr;

  // op(A) is M x K: memory has k contiguous when !TA.  op(B) is K x N: memory has k
  // contiguous when TB.
  TileLoader<T, BM, BK, NT, !TA> la;
  TileLoader<T, BN, BK, NT, TB> lb;

  T acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = (T)0;

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
    for (int k = 0; k < BK; ++k) {
      T a[TM], b[TN];
#pragma unroll
      for (int c = 0; c < CM; ++c) {
        V v = *reinterpret_cast<const V*>(&As[cur][k][c * (BM / CM) + ty * VEC]);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int q = 0; q < VEC; ++q) a[c * VEC + q] = e[q];
      }
#pragma unroll
      for (int c = 0; c < CN; ++c) {
        V v = *reinterpret_cast<const V*>(&Bs[cur][k][c * (BN / CN) + tx * VEC]);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int q = 0; q < VEC; ++q) b[c * VEC + q] = e[q];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          // EXACT: round the product, then the sum, as `Output[i][j] += a * b` does in the
          // managed code (k ascending), so the result is bit-identical to that loop
          if (EXACT) acc[i][j] = add_rn(acc[i][j], mul_rn(a[i], b[j]));
          else acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
    }
    if (kt + 1 < ktiles) {
      la.store(As[cur ^ 1], tid);
      lb.store(Bs[cur ^ 1], tid);
    }
    __syncthreads();
  }

  // epilogue
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + (i / VEC) * (BM / CM) + ty * VEC + (i % VEC);
    if (m >= M) continue;
#pragma unroll
    for (int c = 0; c < CN; ++c) {
      const int n = n0 + c * (BN / CN) + tx * VEC;
      if (n >= N) continue;
      T out[VEC];
      const int64_t off = (int64_t)m * ldc + n;
      const bool full = vecC && (n + VEC <= N);
      T old[VEC];
      if (beta != (T)0) {
        if (full) {
          V v = *reinterpret_cast<const V*>(C + off);
          const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
          for (int q = 0; q < VEC; ++q) old[q] = e[q];
        } else {
#pragma unroll
          for (int q = 0; q < VEC; ++q) old[q] = (n + q < N) ? C[off + q] : (T)0;
        }
      }
#pragma unroll
      for (int q = 0; q < VEC; ++q) {
        T v = mul_rn(alpha, acc[i][c * VEC + q]);
        if (beta != (T)0) v = (beta == (T)1) ? add_rn(old[q], v) : fma(beta, old[q], v);
        if (n + q < N) {
          if (epi.bias) v += epi.bias[n + q];
          if (z_out) z_out[off + q] = v;
          if (epi.act != PRAD_ACT_NONE) v = act_value<T>((prad_act)epi.act, v, epi.act_alpha);
          if (epi.dact != PRAD_ACT_NONE)
            v = mul_rn(v, act_derivative<T>((prad_act)epi.dact, saved[off + q], epi.act_alpha));
        }
        out[q] = v;
      }
      if (full) {
        V v;
        T* e = reinterpret_cast<T*>(&v);
#pragma unroll
        for (int q = 0; q < VEC; ++q) e[q] = out[q];
        *reinterpret_cast<V*>(C + off) = v;
      } else {
#pragma unroll
        for (int q = 0; q < VEC; ++q)
          if (n + q < N) C[off + q] = out[q];
      }
    }
  }
}

// ---- many small products ----------------------------------------------------------------------
// A strided batch of products whose whole output is at most 64 x 64 (the per-window, per-head
// attention products Q K^T, P V and their four backward forms: 49 x 49 x 32 and 49 x 32 x 49).  The
// 64 x 64 tile of the kernel above would spend more than half of its multiply-adds on rows, columns
// and k beyond the matrices, and at these sizes the arithmetic, not the memory, is what takes the
// time.  Here a CTA owns one product and has just the threads its output needs (4 x 4 outputs per
// thread, rounded up to whole warps); both operands of up to KC values of k sit in shared memory in
// k-major order, so a thread reads one 4-vector of each per k.  Same arithmetic per output element
// as above (k ascending, one accumulator), hence bit-identical results.
template <typename T> __device__ __forceinline__ void load4(const T* p, T (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load4<double>(const double* p, double (&v)[4]) {
  const double2 t = *reinterpret_cast<const double2*>(p), u = *reinterpret_cast<const double2*>(p + 2);
  v[0] = t.x; v[1] = t.y; v[2] = u.x; v[3] = u.y;
}

// one operand chunk into shared memory as [k][XP]: X operand rows (M or N; columns X..XP-1 are zero-filled),
// kc values of k starting at k0.  KMAJOR: memory is [K][X] (x contiguous), otherwise [X][K].  A warp takes
// every nw-th memory row, its lanes consecutive elements of it (at most 64: two trips); the loads of eight rows
// are issued before the first of them is stored, so that a thread has up to sixteen loads in flight.
template <typename T, bool KMAJOR>
__device__ __forceinline__ void load_small_operand(T* __restrict__ s, int XP, const T* __restrict__ g, int64_t ld, int X,
                                                   int k0, int kc, int warp, int lane, int nw) {
  constexpr int U = 8;
  const int rows = KMAJOR ? kc : XP;          // memory rows of the chunk (rows X..XP-1 of the [X][K] form are zeros)
  const int cols = KMAJOR ? XP : kc;          // elements taken from each
  const int rows_valid = KMAJOR ? kc : X, cols_valid = KMAJOR ? X : kc;
  const T* base = KMAJOR ? g + (int64_t)k0 * ld : g + k0;
  for (int r0 = warp; r0 < rows; r0 += nw * U) {
    T v[U][2];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * nw;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int c = lane + 32 * t;
        v[u][t] = (r < rows_valid && c < cols_valid) ? base[(int64_t)r * ld + c] : (T)0;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * nw;
      if (r >= rows) break;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int c = lane + 32 * t;
        if (c < cols) s[KMAJOR ? r * XP + c : c * XP + r] = v[u][t];
      }
    }
  }
}

template <typename T, bool TA, bool TB, bool EXACT>
__global__ void __launch_bounds__(256)
gemm_small_kernel(int M, int N, int K, int KC, int MP, int NP, T alpha, const T* __restrict__ A, int64_t lda,
                  const T* __restrict__ B, int64_t ldb, T beta, T* __restrict__ C, int64_t ldc, int64_t sA, int64_t sB,
                  int64_t sC, bool vecC) {
  extern __shared__ __align__(16) unsigned char small_smem[];
  T* As = reinterpret_cast<T*>(small_smem);   // [KC][MP]
  T* Bs = As + KC * MP;                        // [KC][NP]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  const int txn = NP >> 2;
  const int tx = tid % txn, ty = tid / txn;
  const bool active = ty < (MP >> 2);
  const int64_t bz = blockIdx.x;
  A += bz * sA;
  B += bz * sB;
  C += bz * sC;

  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = (T)0;

  for (int k0 = 0; k0 < K; k0 += KC) {
    const int kc = K - k0 < KC ? K - k0 : KC;
    if (k0) __syncthreads();
    load_small_operand<T, TA>(As, MP, A, lda, M, k0, kc, warp, lane, nw);     // op(A) is M x K: k-major memory when TA
    load_small_operand<T, !TB>(Bs, NP, B, ldb, N, k0, kc, warp, lane, nw);    // op(B) is K x N: k-major memory unless TB
    __syncthreads();
    if (active) {
      const T* ap = As + 4 * ty;
      const T* bp = Bs + 4 * tx;
#pragma unroll 4
      for (int k = 0; k < kc; ++k) {
        T a[4], b[4];
        load4<T>(ap + k * MP, a);
        load4<T>(bp + k * NP, b);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (EXACT) acc[i][j] = add_rn(acc[i][j], mul_rn(a[i], b[j]));
            else acc[i][j] = fma(a[i], b[j], acc[i][j]);
          }
      }
    }
  }
  if (!active) return;
  const int n = 4 * tx;
  const bool full = vecC && n + 4 <= N;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = 4 * ty + i;
    if (m >= M) continue;
    const int64_t off = (int64_t)m * ldc + n;
    T out[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      T v = mul_rn(alpha, acc[i][q]);
      if (beta != (T)0 && n + q < N) {
        const T old = C[off + q];
        v = (beta == (T)1) ? add_rn(old, v) : fma(beta, old, v);
      }
      out[q] = v;
    }
    if (full) {
      if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(C + off) = make_float4(out[0], out[1], out[2], out[3]);
      } else {
        *reinterpret_cast<double2*>(C + off) = make_double2(out[0], out[1]);
        *reinterpret_cast<double2*>(C + off + 2) = make_double2(out[2], out[3]);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (n + q < N) C[off + q] = out[q];
    }
  }
}

template <typename T>
static prad_status launch_small(prad_ctx* ctx, bool exact, bool tA, bool tB, int M, int N, int K, T alpha, const T* A,
                                int64_t lda, const T* B, int64_t ldb, T beta, T* C, int64_t ldc, int batch, int64_t sA,
                                int64_t sB, int64_t sC) {
  const int MP = (M + 3) & ~3, NP = (N + 3) & ~3;
  const int kc_max = sizeof(T) == 4 ? 64 : 32;                  // at most 32 KB of shared memory
  const int KC = K < kc_max ? K : kc_max;
  int nt = (MP / 4) * (NP / 4);
  nt = (nt + 31) & ~31;
  if (nt < 64) nt = 64;
  const size_t smem = (size_t)KC * (MP + NP) * sizeof(T);
  const bool vC = (((uintptr_t)C & 15) == 0) && ldc % 4 == 0 && sC % 4 == 0;
#define PRAD_SMALL_LAUNCH(TA_, TB_)                                                                          \
  do {                                                                                                       \
    if (exact)                                                                                               \
      gemm_small_kernel<T, TA_, TB_, true><<<(unsigned)batch, nt, smem, ctx->stream>>>(                     \
          M, N, K, KC, MP, NP, alpha, A, lda, B, ldb, beta, C, ldc, sA, sB, sC, vC);                         \
    else                                                                                                     \
      gemm_small_kernel<T, TA_, TB_, false><<<(unsigned)batch, nt, smem, ctx->stream>>>(                    \
          M, N, K, KC, MP, NP, alpha, A, lda, B, ldb, beta, C, ldc, sA, sB, sC, vC);                         \
  } while (0)
  if (!tA && !tB) PRAD_SMALL_LAUNCH(false, false);
  else if (!tA && tB) PRAD_SMALL_LAUNCH(false, true);
  else if (tA && !tB) PRAD_SMALL_LAUNCH(true, false);
  else PRAD_SMALL_LAUNCH(true, true);
#undef PRAD_SMALL_LAUNCH
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

template <typename T> static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <typename T, int BM, int BN, int BK, int TM, int TN>
static prad_status launch_cfg(prad_ctx* ctx, bool exact, bool tA, bool tB, int M, int N, int K, T alpha,
                              const T* A, int64_t lda, const T* B, int64_t ldb, T beta, T* C,
                              int64_t ldc, int batch, int64_t sA, int64_t sB, int64_t sC,
                              const EpiParams<T>& epi) {
  constexpr int VEC = VecOf<T>::N;
  constexpr int NT = (BM / TM) * (BN / TN);
  dim3 grid((unsigned)ceil_div(N, BN), (unsigned)ceil_div(M, BM), (unsigned)batch);
  PRAD_REQUIRE(grid.y <= 65535 && grid.z <= 65535, PRAD_ERR_UNSUPPORTED,
               "gemm: grid too large (M tiles %u, batch %u)", grid.y, grid.z);
  bool vA = aligned16<T>(A) && lda % VEC == 0 && sA % VEC == 0;
  bool vB = aligned16<T>(B) && ldb % VEC == 0 && sB % VEC == 0;
  bool vC = aligned16<T>(C) && ldc % VEC == 0 && sC % VEC == 0;
#define PRAD_GEMM_LAUNCH(TA_, TB_)                                                           \
  do {                                                                                       \
    if (exact)                                                                               \
      gemm_simt_kernel<T, BM, BN, BK, TM, TN, TA_, TB_, true><<<grid, NT, 0, ctx->stream>>>( \
          M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, sA, sB, sC, vA, vB, vC, epi);        \
    else                                                                                     \
      gemm_simt_kernel<T, BM, BN, BK, TM, TN, TA_, TB_, false><<<grid, NT, 0, ctx->stream>>>(\
          M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, sA, sB, sC, vA, vB, vC, epi);        \
  } while (0)
  if (!tA && !tB) PRAD_GEMM_LAUNCH(false, false);
  else if (!tA && tB) PRAD_GEMM_LAUNCH(false, true);
  else if (tA && !tB) PRAD_GEMM_LAUNCH(true, false);
  else PRAD_GEMM_LAUNCH(true, true);
#undef PRAD_GEMM_LAUNCH
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

template <typename T>
prad_status gemm_simt(prad_ctx* ctx, bool exact, bool tA, bool tB, int M, int N, int K,
                      double alpha, const void* A, int lda, const void* B, int ldb, double beta,
                      void* C, int ldc, int batch, int64_t sA, int64_t sB, int64_t sC,
                      const GemmEpilogue& e) {
  EpiParams<T> epi{(const T*)e.bias, (T*)e.z_out, (int)e.act, (int)e.dact, (const T*)e.saved,
                   (T)e.act_alpha};
  // a batch of products no larger than one small tile each, enough of them to fill the machine by themselves
  const bool plain = !e.bias && !e.z_out && e.act == PRAD_ACT_NONE && e.dact == PRAD_ACT_NONE;
  if (plain && M <= 64 && N <= 64 && K >= 1 && batch >= ctx->sm_count && ctx->gemm_small)
    return launch_small<T>(ctx, exact, tA, tB, M, N, K, (T)alpha, (const T*)A, lda, (const T*)B, ldb, (T)beta, (T*)C, ldc,
                           batch, sA, sB, sC);
  // tile choice: big tiles when the output fills the machine, small ones otherwise
  int64_t big_tiles = ceil_div(M, 128) * ceil_div(N, 128) * batch;
  const bool use_big = big_tiles >= ctx->sm_count && M >= 96 && N >= 96;
  if constexpr (sizeof(T) == 4) {
    if (use_big)
      return launch_cfg<T, 128, 128, 16, 8, 8>(ctx, exact, tA, tB, M, N, K, (T)alpha, (const T*)A, lda,
                                               (const T*)B, ldb, (T)beta, (T*)C, ldc, batch, sA,
                                               sB, sC, epi);
    // fewer 64 x 64 tiles than SMs (the products of a small MLP: 256 x 512 outputs over k = 512 are 32 tiles): such a
    // CTA has an SM to itself; 32 x 32 tiles put the same arithmetic on four times as many SMs (measured on that MLP's
    // backward pass: 0.190 -> 0.184 ms with 32 k per stage, 0.221 ms with 64)
    const int64_t t64 = ceil_div(M, 64) * ceil_div(N, 64) * batch;
    if (t64 < ctx->sm_count && K >= 64)
      return launch_cfg<T, 32, 32, 32, 4, 4>(ctx, exact, tA, tB, M, N, K, (T)alpha, (const T*)A, lda,
                                             (const T*)B, ldb, (T)beta, (T*)C, ldc, batch, sA, sB,
                                             sC, epi);
    return launch_cfg<T, 64, 64, 16, 4, 4>(ctx, exact, tA, tB, M, N, K, (T)alpha, (const T*)A, lda,
                                           (const T*)B, ldb, (T)beta, (T*)C, ldc, batch, sA, sB,
                                           sC, epi);
  } else {
    int64_t t64 = ceil_div(M, 64) * ceil_div(N, 64) * batch;
    if (t64 >= ctx->sm_count && M >= 48 && N >= 48)
      return launch_cfg<T, 64, 64, 16, 4, 4>(ctx, exact, tA, tB, M, N, K, (T)alpha, (const T*)A, lda,
                                             (const T*)B, ldb, (T)beta, (T*)C, ldc, batch, sA,
                                             sB, sC, epi);
    // the recurrent products of an LSTM time step (32 x 256 outputs per gate over k = 256) would occupy 32 SMs with
    // 32 x 32 tiles: 16 x 16 tiles spread the same work over four times as many, and 64 k per stage leave four
    // dependent round trips to L2 instead of sixteen (what such a product waits for; measured 1.15 -> 0.91 ms per
    // backward pass of the 64-step LSTM)
    int64_t t32 = ceil_div(M, 32) * ceil_div(N, 32) * batch;
    if (t32 * 2 <= ctx->sm_count && K >= 64)
      return launch_cfg<T, 16, 16, 64, 2, 2>(ctx, exact, tA, tB, M, N, K, (T)alpha, (const T*)A, lda,
                                             (const T*)B, ldb, (T)beta, (T*)C, ldc, batch, sA, sB,
                                             sC, epi);
    return launch_cfg<T, 32, 32, 16, 2, 2>(ctx, exact, tA, tB, M, N, K, (T)alpha, (const T*)A, lda,
                                           (const T*)B, ldb, (T)beta, (T*)C, ldc, batch, sA, sB,
                                           sC, epi);
  }
}

template prad_status gemm_simt<float>(prad_ctx*, bool, bool, bool, int, int, int, double,
                                      const void*, int, const void*, int, double, void*, int, int,
                                      int64_t, int64_t, int64_t, const GemmEpilogue&);
template prad_status gemm_simt<double>(prad_ctx*, bool, bool, bool, int, int, int, double,
                                       const void*, int, const void*, int, double, void*, int,
                                       int, int64_t, int64_t, int64_t, const GemmEpilogue&);

}  // namespace prad
