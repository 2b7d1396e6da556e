// Pieces shared by the register-tiled GEMM kernels (FMA and DMMA): 128-bit vector types, the
// epilogue parameter block and the global -> register -> shared-memory tile loader.
#pragma once

#include "act_math.cuh"
#include "common.cuh"

namespace prad {

template <typename T> struct VecOf;
template <> struct VecOf<float> { using type = float4; static constexpr int N = 4; };
template <> struct VecOf<double> { using type = double2; static constexpr int N = 2; };

template <typename T> struct EpiParams {
  const T* bias;
  T* z_out;
  int act;
  int dact;
  const T* saved;
  T act_alpha;
};

// Tile loader.  The logical operand tile is ROWS(mn) x BK(k); in memory either the k index
// is contiguous (K_CONTIG) or the mn index is.  Shared layout is always [BK][ROWS + PAD].
template <typename T, int ROWS, int BK, int NT, bool K_CONTIG>
struct TileLoader {
  static constexpr int VEC = VecOf<T>::N;
  using V = typename VecOf<T>::type;
  static constexpr int VECS = ROWS * BK / VEC;
  static constexpr int PER_THREAD = (VECS + NT - 1) / NT;
  T regs[PER_THREAD][VEC];

  // mn0: first mn index of the tile, k0: first k index; MN, K: operand extents
  __device__ __forceinline__ void load(const T* __restrict__ p, int64_t ld, int mn0, int k0,
                                       int MN, int K, bool vec_ok, int tid) {
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      int idx = tid + it * NT;
      if (VECS % NT != 0 && idx >= VECS) break;
      int r, c;  // r: slow index in memory, c: fast (contiguous) index, both tile-local
      if (K_CONTIG) {
        r = idx / (BK / VEC);
        c = (idx % (BK / VEC)) * VEC;
      } else {
        r = idx / (ROWS / VEC);
        c = (idx % (ROWS / VEC)) * VEC;
      }
      int mn = K_CONTIG ? mn0 + r : mn0 + c;
      int k = K_CONTIG ? k0 + c : k0 + r;
      int slow = K_CONTIG ? mn : k, fast = K_CONTIG ? k : mn;
      int slow_lim = K_CONTIG ? MN : K, fast_lim = K_CONTIG ? K : MN;
      const T* src = p + (int64_t)slow * ld + fast;
      if (slow < slow_lim && fast + VEC <= fast_lim && vec_ok) {
        V v = *reinterpret_cast<const V*>(src);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int q = 0; q < VEC; ++q) regs[it][q] = e[q];
      } else {
#pragma unroll
        for (int q = 0; q < VEC; ++q)
          regs[it][q] = (slow < slow_lim && fast + q < fast_lim) ? src[q] : (T)0;
      }
    }
  }

  template <int LDS>
  __device__ __forceinline__ void store(T (*sm)[LDS], int tid) {
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      int idx = tid + it * NT;
      if (VECS % NT != 0 && idx >= VECS) break;
      if (K_CONTIG) {
        int r = idx / (BK / VEC);
        int c = (idx % (BK / VEC)) * VEC;
#pragma unroll
        for (int q = 0; q < VEC; ++q) sm[c + q][r] = regs[it][q];
      } else {
        int r = idx / (ROWS / VEC);
        int c = (idx % (ROWS / VEC)) * VEC;
        V v;
        T* e = reinterpret_cast<T*>(&v);
#pragma unroll
        for (int q = 0; q < VEC; ++q) e[q] = regs[it][q];
        *reinterpret_cast<V*>(&sm[r][c]) = v;
      }
    }
  }
};

}  // namespace prad
