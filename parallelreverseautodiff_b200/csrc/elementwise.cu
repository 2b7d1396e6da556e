// Stand-alone elementwise kernels of the backward path: HBM-bound streams with 128-bit
// loads and stores, grid sized as a multiple of the SM count, grid-stride loop.
// (Compiled with -fmad=false so that products and sums round as the managed code's do.)
#include <mutex>

#include "act_math.cuh"
#include "common.cuh"

namespace prad {

template <typename T> struct Vec16;
template <> struct Vec16<float> { using type = float4; static constexpr int N = 4; };
template <> struct Vec16<double> { using type = double2; static constexpr int N = 2; };

template <int N> struct PtrsIn { const void* p[N > 0 ? N : 1]; };
template <int N> struct PtrsOut { void* p[N > 0 ? N : 1]; };

// out[0..NOUT) = f(in[0..NIN)) per element.  UNROLL vectors per thread per trip keep
// several 128-bit loads in flight per thread.
template <typename T, int NIN, int NOUT, typename F, int UNROLL>
__global__ void __launch_bounds__(256)
map_kernel(PtrsIn<NIN> in, PtrsOut<NOUT> out, int64_t n, bool vec, F f) {
  constexpr int VEC = Vec16<T>::N;
  using V = typename Vec16<T>::type;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t nvec = n / VEC;
    for (int64_t base = tid; base < nvec; base += nthreads * UNROLL) {
      V vin[UNROLL][NIN > 0 ? NIN : 1];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        int64_t i = base + (int64_t)u * nthreads;
        if (i < nvec) {
#pragma unroll
          for (int k = 0; k < NIN; ++k) vin[u][k] = __ldcs(reinterpret_cast<const V*>(in.p[k]) + i);
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        int64_t i = base + (int64_t)u * nthreads;
        if (i < nvec) {
          V vout[NOUT];
#pragma unroll
          for (int q = 0; q < VEC; ++q) {
            T a[NIN > 0 ? NIN : 1], r[NOUT];
#pragma unroll
            for (int k = 0; k < NIN; ++k) a[k] = reinterpret_cast<const T*>(&vin[u][k])[q];
            f(a, r);
#pragma unroll
            for (int k = 0; k < NOUT; ++k) reinterpret_cast<T*>(&vout[k])[q] = r[k];
          }
#pragma unroll
          for (int k = 0; k < NOUT; ++k) __stcs(reinterpret_cast<V*>(out.p[k]) + i, vout[k]);
        }
      }
    }
    // tail
    for (int64_t i = nvec * VEC + tid; i < n; i += nthreads) {
      T a[NIN > 0 ? NIN : 1], r[NOUT];
#pragma unroll
      for (int k = 0; k < NIN; ++k) a[k] = reinterpret_cast<const T*>(in.p[k])[i];
      f(a, r);
#pragma unroll
      for (int k = 0; k < NOUT; ++k) reinterpret_cast<T*>(out.p[k])[i] = r[k];
    }
  } else {
    for (int64_t i = tid; i < n; i += nthreads) {
      T a[NIN > 0 ? NIN : 1], r[NOUT];
#pragma unroll
      for (int k = 0; k < NIN; ++k) a[k] = reinterpret_cast<const T*>(in.p[k])[i];
      f(a, r);
#pragma unroll
      for (int k = 0; k < NOUT; ++k) reinterpret_cast<T*>(out.p[k])[i] = r[k];
    }
  }
}

template <typename T, int NIN, int NOUT, typename F>
static prad_status launch_map(prad_ctx* ctx, const void* const (&in)[NIN], void* const (&out)[NOUT],
                              int64_t n, F f) {
  if (n <= 0) return PRAD_OK;
  PtrsIn<NIN> pi;
  PtrsOut<NOUT> po;
  bool vec = true;
  for (int k = 0; k < NIN; ++k) { pi.p[k] = in[k]; vec = vec && (((uintptr_t)in[k] & 15) == 0); }
  for (int k = 0; k < NOUT; ++k) { po.p[k] = out[k]; vec = vec && (((uintptr_t)out[k] & 15) == 0); }
  constexpr int UNROLL = 4;
  constexpr int VEC = Vec16<T>::N;
  int grid = stream_grid(ctx, ceil_div(n, VEC * UNROLL), 256, 8);
  map_kernel<T, NIN, NOUT, F, UNROLL><<<grid, 256, 0, ctx->stream>>>(pi, po, n, vec, f);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

// ---------------------------------------------------------------- functors
template <typename T> struct ActFwd {
  prad_act act; T alpha;
  __device__ void operator()(const T* a, T* r) const { r[0] = act_value<T>(act, a[0], alpha); }
};
template <typename T> struct ActBwd {  // a[0] = saved, a[1] = dy
  prad_act act; T alpha;
  __device__ void operator()(const T* a, T* r) const {
    r[0] = mul_rn(a[1], act_derivative<T>(act, a[0], alpha));
  }
};
template <typename T> struct HadFwd {
  __device__ void operator()(const T* a, T* r) const { r[0] = mul_rn(a[0], a[1]); }
};
template <typename T> struct HadBwd {  // a, b, dy -> da = dy*b, db = dy*a (HadamardProductOperation.cs:98,110)
  __device__ void operator()(const T* a, T* r) const {
    r[0] = mul_rn(a[2], a[1]);
    r[1] = mul_rn(a[2], a[0]);
  }
};
template <typename T> struct Add2 {
  __device__ void operator()(const T* a, T* r) const { r[0] = add_rn(a[0], a[1]); }
};
template <typename T> struct Add3 {
  __device__ void operator()(const T* a, T* r) const { r[0] = add_rn(add_rn(a[0], a[1]), a[2]); }
};
template <typename T> struct Scale {
  T s;
  __device__ void operator()(const T* a, T* r) const { r[0] = mul_rn(a[0], s); }
};
template <typename T> struct Accum {  // dest += src  (OperationBase.cs:299)
  __device__ void operator()(const T* a, T* r) const { r[0] = add_rn(a[0], a[1]); }
};

template <typename T>
static prad_status act_forward_t(prad_ctx* ctx, prad_act act, const void* x, void* y, int64_t n,
                                 double alpha) {
  const void* in[1] = {x};
  void* out[1] = {y};
  return launch_map<T, 1, 1>(ctx, in, out, n, ActFwd<T>{act, (T)alpha});
}
template <typename T>
static prad_status act_backward_t(prad_ctx* ctx, prad_act act, const void* saved, const void* dy,
                                  void* dx, int64_t n, double alpha) {
  const void* in[2] = {saved, dy};
  void* out[1] = {dx};
  return launch_map<T, 2, 1>(ctx, in, out, n, ActBwd<T>{act, (T)alpha});
}

// ---------------------------------------------------------------- add-broadcast
// (x and y may be the same buffer: no __restrict__ on them)
template <typename T>
__global__ void add_broadcast_kernel(const T* x, const T* __restrict__ bias, T* y, int64_t n, int cols) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = add_rn(x[i], bias[i % cols]);
}

// Column sums  dBias[j] = sum_i dOut[i][j]  (MatrixAddBroadcastingOperation.cs:60-63).
// Two deterministic stages: each CTA sums a band of rows for a 32-column strip into
// partial[band][col] (coalesced 128-byte row segments), then one pass adds the bands in
// band order.  Accumulation is in double for float data (LINQ Sum accumulates in double).
template <typename T>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const T* __restrict__ x, double* __restrict__ partial, int64_t rows,
                      int cols, int rows_per_band, T* __restrict__ direct_out, int accumulate) {
  // direct_out: there is one band only (a short matrix) and the sums go straight to the result: one launch
  __shared__ double sm[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_band;
  int64_t r1 = r0 + rows_per_band;
  if (r1 > rows) r1 = rows;
  double acc = 0.0;
  if (col < cols)
    for (int64_t r = r0 + w; r < r1; r += 8) acc += (double)x[r * cols + col];
  sm[w][lane] = acc;
  __syncthreads();
  if (w == 0) {
    double s = 0.0;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += sm[k][lane];
    if (col < cols) {
      if (direct_out) {
        const T v = (T)s;
        direct_out[col] = accumulate ? add_rn(direct_out[col], v) : v;
      } else {
        partial[(int64_t)blockIdx.y * cols + col] = s;
      }
    }
  }
}
template <typename T>
__global__ void colsum_final_kernel(const double* __restrict__ partial, T* __restrict__ out,
                                    int cols, int bands, int accumulate) {
  int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  double s = 0.0;
  for (int b = 0; b < bands; ++b) s += partial[(int64_t)b * cols + col];
  T v = (T)s;
  out[col] = accumulate ? add_rn(out[col], v) : v;
}

// Streaming form of the same column sums for matrices whose rows are a whole number of
// 128-bit vectors: the matrix is read like a copy (thread t takes vectors t, t+S, t+2S, ...
// with S a multiple of the vectors per row, so a thread always sees the same column group),
// every CTA adds the sums of its threads that share a group (in thread order) and writes one
// partial per group, and one CTA per column group adds the partials in CTA order.  Fully
// coalesced, deterministic.
// CTA_SUM: the sums of the threads of a CTA that share a column group are added in shared memory (in thread order) and
// the CTA writes one partial per group; otherwise (more than 256 groups: wide rows) every thread writes its own.
template <typename T, bool CTA_SUM>
__global__ void __launch_bounds__(256)
colsum_flat_partial_kernel(const T* __restrict__ x, double* __restrict__ partial, int64_t nvec,
                           int64_t stride_threads, int vec_per_row) {
  constexpr int VEC = Vec16<T>::N;
  using V = typename Vec16<T>::type;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (!CTA_SUM && t >= stride_threads) return;
  if (CTA_SUM && t >= stride_threads) nvec = 0;      // the last CTA's surplus threads add nothing
  double acc[VEC];
#pragma unroll
  for (int q = 0; q < VEC; ++q) acc[q] = 0.0;
  const V* xv = reinterpret_cast<const V*>(x);
  int64_t i = t;
  for (; i + 3 * stride_threads < nvec; i += 4 * stride_threads) {   // four loads in flight
    V v0 = __ldcs(xv + i), v1 = __ldcs(xv + i + stride_threads);
    V v2 = __ldcs(xv + i + 2 * stride_threads), v3 = __ldcs(xv + i + 3 * stride_threads);
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
      acc[q] += (double)reinterpret_cast<const T*>(&v0)[q];
      acc[q] += (double)reinterpret_cast<const T*>(&v1)[q];
      acc[q] += (double)reinterpret_cast<const T*>(&v2)[q];
      acc[q] += (double)reinterpret_cast<const T*>(&v3)[q];
    }
  }
  for (; i < nvec; i += stride_threads) {
    V v = __ldcs(xv + i);
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[q] += (double)reinterpret_cast<const T*>(&v)[q];
  }
  if constexpr (!CTA_SUM) {
#pragma unroll
    for (int q = 0; q < VEC; ++q) partial[t * VEC + q] = acc[q];
  } else {
    __shared__ double sm[256][VEC];
#pragma unroll
    for (int q = 0; q < VEC; ++q) sm[threadIdx.x][q] = acc[q];
    __syncthreads();
    if ((int)threadIdx.x < vec_per_row) {
      const int group = (int)(t % vec_per_row);
#pragma unroll
      for (int q = 0; q < VEC; ++q) acc[q] = 0.0;
      for (int j = threadIdx.x; j < 256; j += vec_per_row)
#pragma unroll
        for (int q = 0; q < VEC; ++q) acc[q] += sm[j][q];
#pragma unroll
      for (int q = 0; q < VEC; ++q) partial[((int64_t)blockIdx.x * vec_per_row + group) * VEC + q] = acc[q];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
colsum_flat_final_kernel(const double* __restrict__ partial, T* __restrict__ out, int vec_per_row,
                         int64_t stride_threads, int accumulate) {
  constexpr int VEC = Vec16<T>::N;
  __shared__ double sm[4][VEC];
  const int group = blockIdx.x;            // column group = VEC consecutive columns
  double acc[VEC];
#pragma unroll
  for (int q = 0; q < VEC; ++q) acc[q] = 0.0;
  for (int64_t t = group + (int64_t)threadIdx.x * vec_per_row; t < stride_threads; t += (int64_t)128 * vec_per_row)
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[q] += partial[t * VEC + q];
#pragma unroll
  for (int q = 0; q < VEC; ++q)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[q] += __shfl_xor_sync(0xffffffffu, acc[q], o);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0)
#pragma unroll
    for (int q = 0; q < VEC; ++q) sm[w][q] = acc[q];
  __syncthreads();
  if (threadIdx.x < VEC) {
    const int q = threadIdx.x;
    const T v = (T)(((sm[0][q] + sm[1][q]) + sm[2][q]) + sm[3][q]);
    T* o = out + group * VEC + q;
    *o = accumulate ? add_rn(*o, v) : v;
  }
}

template <typename T>
static prad_status add_broadcast_backward_t(prad_ctx* ctx, const void* dy, void* dbias,
                                            int64_t rows, int cols, int accumulate) {
  constexpr int VEC = Vec16<T>::N;
  if (cols % VEC == 0 && ((uintptr_t)dy & 15) == 0 && rows * (int64_t)cols >= (1 << 20)) {
    const int vec_per_row = cols / VEC;
    int64_t threads = (int64_t)ctx->sm_count * 8 * 256;
    const int64_t nvec = rows * vec_per_row;
    if (threads > nvec) threads = nvec;
    threads -= threads % vec_per_row;
    if (threads >= vec_per_row) {
      prad_status s = ensure_workspace(ctx, (size_t)threads * VEC * sizeof(double));
      if (s) return s;
      const int64_t ctas = ceil_div(threads, 256);
      if (vec_per_row <= 256)
        colsum_flat_partial_kernel<T, true><<<(unsigned)ctas, 256, 0, ctx->stream>>>((const T*)dy, (double*)ctx->ws, nvec,
                                                                                   threads, vec_per_row);
      else
        colsum_flat_partial_kernel<T, false><<<(unsigned)ctas, 256, 0, ctx->stream>>>((const T*)dy, (double*)ctx->ws, nvec,
                                                                                    threads, vec_per_row);
      PRAD_LAUNCHED(ctx);
      // entries the final pass adds per column group: one per CTA, or one per thread for very wide rows
      const int64_t entries = vec_per_row <= 256 ? ctas * vec_per_row : threads;
      colsum_flat_final_kernel<T><<<vec_per_row, 128, 0, ctx->stream>>>((const double*)ctx->ws, (T*)dbias,
                                                                      vec_per_row, entries, accumulate);
      PRAD_LAUNCHED(ctx);
      return PRAD_OK;
    }
  }
  int strips = (int)ceil_div(cols, 32);
  int64_t want_bands = ceil_div((int64_t)ctx->sm_count * 8, strips);
  int64_t max_bands = ceil_div(rows, 64);
  int bands = (int)(want_bands < max_bands ? want_bands : max_bands);
  if (bands < 1) bands = 1;
  if (bands > 65535) bands = 65535;
  if (rows <= 512) bands = 1;      // a short matrix (the bias gradient of a small batch): one launch, no second pass
  int rows_per_band = (int)ceil_div(rows, bands);
  bands = (int)ceil_div(rows, rows_per_band);
  if (bands == 1) {
    colsum_partial_kernel<T><<<dim3(strips, 1), 256, 0, ctx->stream>>>((const T*)dy, nullptr, rows, cols, rows_per_band,
                                                                      (T*)dbias, accumulate);
    PRAD_LAUNCHED(ctx);
    return PRAD_OK;
  }
  prad_status s = ensure_workspace(ctx, (size_t)bands * cols * sizeof(double));
  if (s) return s;
  colsum_partial_kernel<T><<<dim3(strips, bands), 256, 0, ctx->stream>>>(
      (const T*)dy, (double*)ctx->ws, rows, cols, rows_per_band, nullptr, 0);
  PRAD_LAUNCHED(ctx);
  colsum_final_kernel<T><<<(unsigned)ceil_div(cols, 128), 128, 0, ctx->stream>>>(
      (const double*)ctx->ws, (T*)dbias, cols, bands, accumulate);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

// ---------------------------------------------------------------- transpose (per slice)
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols) {
  __shared__ T tile[32][33];
  const int64_t slice = blockIdx.z;
  x += slice * (int64_t)rows * cols;
  y += slice * (int64_t)rows * cols;
  int c = blockIdx.x * 32 + threadIdx.x;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = blockIdx.y * 32 + j;
    if (r < rows && c < cols) tile[j][threadIdx.x] = x[(int64_t)r * cols + c];
  }
  __syncthreads();
  int r2 = blockIdx.y * 32 + threadIdx.x;  // becomes the fast index of y
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int c2 = blockIdx.x * 32 + j;
    if (c2 < cols && r2 < rows) y[(int64_t)c2 * rows + r2] = tile[threadIdx.x][j];
  }
}

// ---------------------------------------------------------------- n-ary sums
#define PRAD_MAX_SRCS 8
struct SrcTable { const void* p[PRAD_MAX_SRCS]; int count; };

// out[i] = sum_g src_g[i] in list order (GradientUtils.cs:33-39).  LINQ's Sum over float
// accumulates in double and casts once; for double it is a plain left fold.
template <typename T>
__device__ __forceinline__ T nary_combine(const T (&v)[PRAD_MAX_SRCS], int count, int mode, T inv_count) {
  if (mode == 0) {  // segmented sum, double accumulator
    double acc = 0.0;
#pragma unroll
    for (int g = 0; g < PRAD_MAX_SRCS; ++g)
      if (g < count) acc += (double)v[g];
    return (T)acc;
  }
  T acc = v[0];     // batch mean: left fold in T, then * (1/count)
#pragma unroll
  for (int g = 1; g < PRAD_MAX_SRCS; ++g)
    if (g < count) acc = add_rn(acc, v[g]);
  return mul_rn(acc, inv_count);
}

template <typename T, int U, int S>
__global__ void __launch_bounds__(256)
nary_sum_kernel(SrcTable t, T* out, int64_t n, int mode, T inv_count, bool vec) {
  // `out` is not restrict-qualified: with more than PRAD_MAX_SRCS sources the running sum is read back
  // through the source table (every thread loads its element before it stores it).
  // U vectors per thread and trip and at most S sources (few sources: more trips' loads in flight).
  constexpr int VEC = Vec16<T>::N;
  using V = typename Vec16<T>::type;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t done = 0;
  if (vec) {      // 128-bit loads of every source, all issued before the first use
    const int64_t nvec = n / VEC;
    for (int64_t i0 = tid; i0 < nvec; i0 += stride * U) {
      V in[U][S];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + u * stride;
        if (i < nvec) {
#pragma unroll
          for (int g = 0; g < S; ++g)
            if (g < t.count) in[u][g] = __ldcs(reinterpret_cast<const V*>(t.p[g]) + i);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + u * stride;
        if (i >= nvec) break;
        V o;
#pragma unroll
        for (int q = 0; q < VEC; ++q) {
          T v[PRAD_MAX_SRCS];
#pragma unroll
          for (int g = 0; g < S; ++g)
            if (g < t.count) v[g] = reinterpret_cast<const T*>(&in[u][g])[q];
          reinterpret_cast<T*>(&o)[q] = nary_combine<T>(v, t.count, mode, inv_count);
        }
        __stcs(reinterpret_cast<V*>(out) + i, o);
      }
    }
    done = nvec * VEC;
  }
  for (int64_t i = done + tid; i < n; i += stride) {
    T v[PRAD_MAX_SRCS];
#pragma unroll
    for (int g = 0; g < PRAD_MAX_SRCS; ++g)
      if (g < t.count) v[g] = reinterpret_cast<const T*>(t.p[g])[i];
    out[i] = nary_combine<T>(v, t.count, mode, inv_count);
  }
}

template <typename T>
static prad_status nary_t(prad_ctx* ctx, const void* const* srcs, int count, void* out, int64_t n,
                          int mode) {
  if (n <= 0) return PRAD_OK;
  // more than PRAD_MAX_SRCS sources: fold in groups, keeping list order.  The running value
  // is carried in `out`, which is exact for mode 1 (left fold) and for double mode 0; for
  // float mode 0 the carry rounds to float between groups of 7.
  T inv = (T)1 / (T)count;
  int done = 0;
  bool first = true;
  while (done < count) {
    SrcTable t;
    int k = 0;
    if (!first) t.p[k++] = out;
    while (k < PRAD_MAX_SRCS && done < count) t.p[k++] = srcs[done++];
    t.count = k;
    bool last = done == count;
    int grid = stream_grid(ctx, ceil_div(n, Vec16<T>::N), 256, 8);
    int m = mode == 0 ? 0 : 1;
    bool vec = ((uintptr_t)out & 15) == 0;
    for (int g = 0; g < t.count; ++g) vec = vec && (((uintptr_t)t.p[g] & 15) == 0);
    const T scale = (mode == 1 && last) ? inv : (T)1;
    if (t.count <= 2) nary_sum_kernel<T, 4, 2><<<grid, 256, 0, ctx->stream>>>(t, (T*)out, n, m, scale, vec);
    else if (t.count <= 4) nary_sum_kernel<T, 2, 4><<<grid, 256, 0, ctx->stream>>>(t, (T*)out, n, m, scale, vec);
    else nary_sum_kernel<T, 1, PRAD_MAX_SRCS><<<grid, 256, 0, ctx->stream>>>(t, (T*)out, n, m, scale, vec);
    PRAD_LAUNCHED(ctx);
    first = false;
  }
  return PRAD_OK;
}

}  // namespace prad

using namespace prad;

#define DISPATCH_DT(dt, CALL_F32, CALL_F64) ((dt) == PRAD_F32 ? (CALL_F32) : (CALL_F64))

extern "C" {

prad_status prad_act_forward(prad_ctx* ctx, prad_dtype dt, prad_act act, const void* x, void* y,
                             int64_t n, double act_alpha) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && act >= PRAD_ACT_NONE && act <= PRAD_ACT_AMPLIFIED_SIGMOID, PRAD_ERR_INVALID,
               "prad_act_forward: bad dtype or activation");
  PRAD_REQUIRE(n >= 0 && (n == 0 || (x && y)), PRAD_ERR_INVALID, "prad_act_forward: null pointer or negative size");
  return DISPATCH_DT(dt, act_forward_t<float>(ctx, act, x, y, n, act_alpha),
                     act_forward_t<double>(ctx, act, x, y, n, act_alpha));
}

prad_status prad_act_backward(prad_ctx* ctx, prad_dtype dt, prad_act act, const void* saved,
                              const void* dy, void* dx, int64_t n, double act_alpha) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && act >= PRAD_ACT_NONE && act <= PRAD_ACT_AMPLIFIED_SIGMOID, PRAD_ERR_INVALID,
               "prad_act_backward: bad dtype or activation");
  PRAD_REQUIRE(n >= 0 && (n == 0 || (saved && dy && dx)), PRAD_ERR_INVALID,
               "prad_act_backward: null pointer or negative size");
  return DISPATCH_DT(dt, act_backward_t<float>(ctx, act, saved, dy, dx, n, act_alpha),
                     act_backward_t<double>(ctx, act, saved, dy, dx, n, act_alpha));
}

prad_status prad_hadamard_forward(prad_ctx* ctx, prad_dtype dt, const void* a, const void* b,
                                  void* y, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && (n == 0 || (a && b && y)), PRAD_ERR_INVALID,
               "prad_hadamard_forward: bad argument");
  const void* in[2] = {a, b};
  void* out[1] = {y};
  return DISPATCH_DT(dt, (launch_map<float, 2, 1>(ctx, in, out, n, HadFwd<float>{})),
                     (launch_map<double, 2, 1>(ctx, in, out, n, HadFwd<double>{})));
}

prad_status prad_hadamard_backward(prad_ctx* ctx, prad_dtype dt, const void* a, const void* b,
                                   const void* dy, void* da, void* db, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && (n == 0 || (a && b && dy && da && db)), PRAD_ERR_INVALID,
               "prad_hadamard_backward: bad argument");
  const void* in[3] = {a, b, dy};
  void* out[2] = {da, db};
  return DISPATCH_DT(dt, (launch_map<float, 3, 2>(ctx, in, out, n, HadBwd<float>{})),
                     (launch_map<double, 3, 2>(ctx, in, out, n, HadBwd<double>{})));
}

prad_status prad_add_forward(prad_ctx* ctx, prad_dtype dt, const void* a, const void* b,
                             const void* c, void* y, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && (n == 0 || (a && b && y)), PRAD_ERR_INVALID,
               "prad_add_forward: bad argument");
  void* out[1] = {y};
  if (c) {
    const void* in[3] = {a, b, c};
    return DISPATCH_DT(dt, (launch_map<float, 3, 1>(ctx, in, out, n, Add3<float>{})),
                       (launch_map<double, 3, 1>(ctx, in, out, n, Add3<double>{})));
  }
  const void* in[2] = {a, b};
  return DISPATCH_DT(dt, (launch_map<float, 2, 1>(ctx, in, out, n, Add2<float>{})),
                     (launch_map<double, 2, 1>(ctx, in, out, n, Add2<double>{})));
}

prad_status prad_add_broadcast_forward(prad_ctx* ctx, prad_dtype dt, const void* x,
                                       const void* bias, void* y, int rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID,
               "prad_add_broadcast_forward: bad argument");
  int64_t n = (int64_t)rows * cols;
  if (n == 0) return PRAD_OK;
  PRAD_REQUIRE(x && bias && y, PRAD_ERR_INVALID, "prad_add_broadcast_forward: null pointer");
  int grid = stream_grid(ctx, n, 256, 8);
  if (dt == PRAD_F32)
    add_broadcast_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)x, (const float*)bias, (float*)y, n, cols);
  else
    add_broadcast_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)x, (const double*)bias, (double*)y, n, cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_add_broadcast_backward(prad_ctx* ctx, prad_dtype dt, const void* dy,
                                        void* dbias, int rows, int cols, int accumulate) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID,
               "prad_add_broadcast_backward: bad argument");
  if (cols == 0) return PRAD_OK;
  PRAD_REQUIRE(dbias && (dy || rows == 0), PRAD_ERR_INVALID, "prad_add_broadcast_backward: null pointer");
  if (rows == 0) {
    if (!accumulate) return prad_zero(ctx, dbias, (size_t)cols * dtype_size(dt));
    return PRAD_OK;
  }
  return DISPATCH_DT(dt, add_broadcast_backward_t<float>(ctx, dy, dbias, rows, cols, accumulate),
                     add_broadcast_backward_t<double>(ctx, dy, dbias, rows, cols, accumulate));
}

prad_status prad_scale(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, int64_t n,
                       double s) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && (n == 0 || (x && y)), PRAD_ERR_INVALID,
               "prad_scale: bad argument");
  const void* in[1] = {x};
  void* out[1] = {y};
  return DISPATCH_DT(dt, (launch_map<float, 1, 1>(ctx, in, out, n, Scale<float>{(float)s})),
                     (launch_map<double, 1, 1>(ctx, in, out, n, Scale<double>{s})));
}

prad_status prad_transpose(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, int rows,
                           int cols, int depth) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0 && depth >= 0, PRAD_ERR_INVALID,
               "prad_transpose: bad argument");
  if ((int64_t)rows * cols * depth == 0) return PRAD_OK;
  PRAD_REQUIRE(x && y && x != y, PRAD_ERR_INVALID, "prad_transpose: null or aliased pointers");
  PRAD_REQUIRE(depth <= 65535 && ceil_div(rows, 32) <= 65535, PRAD_ERR_UNSUPPORTED,
               "prad_transpose: too many slices or rows for one launch");
  dim3 grid((unsigned)ceil_div(cols, 32), (unsigned)ceil_div(rows, 32), (unsigned)depth), blk(32, 8);
  if (dt == PRAD_F32) transpose_kernel<float><<<grid, blk, 0, ctx->stream>>>((const float*)x, (float*)y, rows, cols);
  else transpose_kernel<double><<<grid, blk, 0, ctx->stream>>>((const double*)x, (double*)y, rows, cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_segmented_sum(prad_ctx* ctx, prad_dtype dt, const void* const* srcs_host,
                               int count, void* out, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && count >= 1 && n >= 0 && srcs_host && (out || n == 0),
               PRAD_ERR_INVALID, "prad_segmented_sum: bad argument");
  for (int i = 0; i < count; ++i)
    PRAD_REQUIRE(srcs_host[i] || n == 0, PRAD_ERR_INVALID, "prad_segmented_sum: source %d is null", i);
  return DISPATCH_DT(dt, nary_t<float>(ctx, srcs_host, count, out, n, 0),
                     nary_t<double>(ctx, srcs_host, count, out, n, 0));
}

prad_status prad_batch_mean(prad_ctx* ctx, prad_dtype dt, const void* const* srcs_host,
                            int count, void* out, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && count >= 1 && n >= 0 && srcs_host && (out || n == 0),
               PRAD_ERR_INVALID, "prad_batch_mean: bad argument");
  for (int i = 0; i < count; ++i)
    PRAD_REQUIRE(srcs_host[i] || n == 0, PRAD_ERR_INVALID, "prad_batch_mean: source %d is null", i);
  return DISPATCH_DT(dt, nary_t<float>(ctx, srcs_host, count, out, n, 1),
                     nary_t<double>(ctx, srcs_host, count, out, n, 1));
}

prad_status prad_accumulate(prad_ctx* ctx, prad_dtype dt, void* dest, const void* src,
                            int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && (n == 0 || (dest && src)), PRAD_ERR_INVALID,
               "prad_accumulate: bad argument");
  const void* in[2] = {dest, src};
  void* out[1] = {dest};
  return DISPATCH_DT(dt, (launch_map<float, 2, 1>(ctx, in, out, n, Accum<float>{})),
                     (launch_map<double, 2, 1>(ctx, in, out, n, Accum<double>{})));
}

}  // extern "C"

// ---------------------------------------------------------------- allocation-free column sums
// Variant of prad_add_broadcast_backward for callers that may not allocate device memory
// while they run: a plug-in that shares a device whose memory the host application has
// already budgeted to the last byte, a component that is forbidden to call an allocator
// after start-up, or a real-time loop in which a cudaMalloc stall (it synchronises the
// device) is not tolerable.
// The partial sums live in a fixed array that is part of the loaded module, so every device
// that loads this library keeps these 4 MiB until the process exits.
namespace prad {

constexpr int64_t STATIC_SCRATCH_DOUBLES = 512 * 1024;  // 4 MiB
static __device__ __align__(256) double g_static_colsum_scratch[STATIC_SCRATCH_DOUBLES];

constexpr int STATIC_MAX_DEVICES = 64;
static std::mutex g_static_mu;
static double* g_static_ptr[STATIC_MAX_DEVICES] = {nullptr};
static int g_static_sms[STATIC_MAX_DEVICES] = {0};

// Resolves the device address of the array on the current device, once per device.  In host
// code the array's name is only a handle for the runtime, never a device pointer.
static prad_status static_scratch_for_current_device(double** out_ptr, int* out_sms) {
  int dev = -1;
  PRAD_CUDA(cudaGetDevice(&dev));
  PRAD_REQUIRE(dev >= 0 && dev < STATIC_MAX_DEVICES, PRAD_ERR_UNSUPPORTED,
               "static scratch: device index %d is beyond the %d supported", dev, STATIC_MAX_DEVICES);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    double* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_colsum_scratch);
    if (e != cudaSuccess || !p) {
      (void)cudaGetLastError();
      set_error("static scratch: cudaGetSymbolAddress failed on device %d: %s", dev,
                cudaGetErrorString(e));
      return PRAD_ERR_CUDA;
    }
    int sms = 0;
    PRAD_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    g_static_sms[dev] = sms;
    g_static_ptr[dev] = p;
  }
  *out_ptr = g_static_ptr[dev];
  *out_sms = g_static_sms[dev];
  return PRAD_OK;
}

template <typename T>
static prad_status colsum_static_t(cudaStream_t st, double* scratch, int sms, const void* dy,
                                   void* dbias, int64_t rows, int cols, int accumulate) {
  int strips = (int)ceil_div(cols, 32);
  int64_t want_bands = ceil_div((int64_t)sms * 8, strips);
  int64_t max_bands = ceil_div(rows, 64);
  int64_t fit_bands = STATIC_SCRATCH_DOUBLES / cols;
  int64_t bands = want_bands < max_bands ? want_bands : max_bands;
  if (bands > fit_bands) bands = fit_bands;
  if (bands > 65535) bands = 65535;
  if (bands < 1) bands = 1;
  int rows_per_band = (int)ceil_div(rows, bands);
  bands = ceil_div(rows, rows_per_band);
  // every partial that the second kernel reads is written by the first one in this call, so
  // nothing left in the array by an earlier call can leak into the result
  colsum_partial_kernel<T><<<dim3(strips, (unsigned)bands), 256, 0, st>>>(
      (const T*)dy, scratch, rows, cols, rows_per_band, nullptr, 0);
  cudaError_t e = cudaPeekAtLastError();
  if (e == cudaSuccess) {
    colsum_final_kernel<T><<<(unsigned)ceil_div(cols, 128), 128, 0, st>>>(
        scratch, (T*)dbias, cols, (int)bands, accumulate);
    e = cudaPeekAtLastError();
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_error("prad_add_broadcast_backward_static: kernel launch failed: %s", cudaGetErrorString(e));
    return PRAD_ERR_CUDA;
  }
  return PRAD_OK;
}

}  // namespace prad

extern "C" prad_status prad_add_broadcast_backward_static(void* stream, prad_dtype dt,
                                                          const void* dy, void* dbias, int rows,
                                                          int cols, int accumulate) {
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_add_broadcast_backward_static: bad dtype");
  PRAD_REQUIRE(rows >= 1 && cols >= 1, PRAD_ERR_SHAPE,
               "prad_add_broadcast_backward_static: rows and cols must be at least 1");
  PRAD_REQUIRE(cols <= PRAD_STATIC_COLSUM_MAX_COLS, PRAD_ERR_UNSUPPORTED,
               "prad_add_broadcast_backward_static: %d columns exceed the fixed scratch (limit %d); "
               "use prad_add_broadcast_backward, which allocates",
               cols, PRAD_STATIC_COLSUM_MAX_COLS);
  PRAD_REQUIRE(dy && dbias, PRAD_ERR_INVALID, "prad_add_broadcast_backward_static: null pointer");
  double* scratch = nullptr;
  int sms = 0;
  prad_status s = static_scratch_for_current_device(&scratch, &sms);
  if (s) return s;
  cudaStream_t st = (cudaStream_t)stream;
  return dt == PRAD_F32 ? colsum_static_t<float>(st, scratch, sms, dy, dbias, rows, cols, accumulate)
                        : colsum_static_t<double>(st, scratch, sms, dy, dbias, rows, cols, accumulate);
}
