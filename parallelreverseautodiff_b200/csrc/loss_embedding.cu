// Loss values and loss gradients (MSE, categorical cross-entropy) and the embedding
// gather / ordered scatter-add.  (Compiled with -fmad=false.)
#include "act_math.cuh"
#include "common.cuh"
#include "reduce.cuh"

namespace prad {

template <typename T> struct Eps15;
template <> struct Eps15<float> { __device__ static float v() { return 1e-15f; } };   // lite PradTools.Epsilon
template <> struct Eps15<double> { __device__ static double v() { return 1e-15; } };  // PradTools.Epsilon

constexpr int LOSS_THREADS = 256;

// kind 0: MSE term (o-t)^2 (MeanSquaredErrorLossOperation.cs:50-55)
// kind 1: CCE term -t*log(o+eps) (CategoricalCrossEntropyLossOperation.cs:53-59)
template <typename T>
__global__ void __launch_bounds__(LOSS_THREADS)
loss_partial_kernel(const T* __restrict__ o, const T* __restrict__ t, double* __restrict__ partial,
                    int64_t n, int kind) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  double acc = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    T term;
    if (kind == 0) {
      T d = sub_rn(o[i], t[i]);
      term = mul_rn(d, d);
    } else {
      term = mul_rn(-t[i], t_log(add_rn(o[i], Eps15<T>::v())));
    }
    acc += (double)term;
  }
  double s = block_sum_d<LOSS_THREADS>(acc);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
template <typename T>
__global__ void loss_final_kernel(const double* __restrict__ partial, int nblocks, T* loss,
                                  T divisor) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double s = 0.0;
    for (int b = 0; b < nblocks; ++b) s += partial[b];
    loss[0] = div_rn((T)s, divisor);
  }
}

// MeanSquaredErrorLossOperation.cs:71-78: grad = (2/(R*C)) * (o - t)
template <typename T>
__global__ void __launch_bounds__(256)
mse_backward_kernel(const T* __restrict__ o, const T* __restrict__ t, T* __restrict__ g, int64_t n,
                    T scale) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    g[i] = mul_rn(scale, sub_rn(o[i], t[i]));
}
// CategoricalCrossEntropyLossOperation.cs:72-83: grad = -scale*y / (yHat + eps)
template <typename T>
__global__ void __launch_bounds__(256)
cce_backward_kernel(const T* __restrict__ o, const T* __restrict__ t, T* __restrict__ g, int64_t n,
                    T scale) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    g[i] = div_rn(mul_rn(-scale, t[i]), add_rn(o[i], Eps15<T>::v()));
}

template <typename T>
static prad_status loss_forward_t(prad_ctx* ctx, const void* o, const void* t, void* loss,
                                  int64_t rows, int cols, int kind) {
  int64_t n = rows * cols;
  int grid = stream_grid(ctx, n, LOSS_THREADS * 4, 4);
  prad_status s = ensure_workspace(ctx, (size_t)grid * sizeof(double));
  if (s) return s;
  loss_partial_kernel<T><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const T*)o, (const T*)t,
                                                                  (double*)ctx->ws, n, kind);
  PRAD_LAUNCHED(ctx);
  T divisor = kind == 0 ? (T)(rows * cols) : (T)rows;
  loss_final_kernel<T><<<1, 32, 0, ctx->stream>>>((const double*)ctx->ws, grid, (T*)loss, divisor);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

// ---------------------------------------------------------------- Swish
// SwishOperation.cs:41-107: y = x * sigmoid(beta x) with beta a [1 x 1] weight; the managed code
// computes in double whatever the storage type and stores back.  The backward is the one written
// there: dx = dy * sigmoid * ((1 + beta x) * (1 - sigmoid)); dBeta = sum dy * (x s (1 - s) - x^2 s^2).
template <typename T>
__global__ void __launch_bounds__(LOSS_THREADS)
swish_forward_kernel(const T* __restrict__ x, const T* __restrict__ beta, T* __restrict__ y, int64_t n) {
  const double b = (double)beta[0];
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const double xv = (double)x[i];
    const double sig = __ddiv_rn(1.0, __dadd_rn(1.0, exp(__dmul_rn(-b, xv))));
    y[i] = (T)__dmul_rn(xv, sig);
  }
}
template <typename T>
__global__ void __launch_bounds__(LOSS_THREADS)
swish_backward_kernel(const T* __restrict__ x, const T* __restrict__ beta, const T* __restrict__ dy,
                      T* __restrict__ dx, double* __restrict__ partial, int64_t n) {
  const double b = (double)beta[0];
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  double acc = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const double xv = (double)x[i], d = (double)dy[i];
    const double sig = __ddiv_rn(1.0, __dadd_rn(1.0, exp(__dmul_rn(-b, xv))));
    const double om = __dsub_rn(1.0, sig);
    dx[i] = (T)__dmul_rn(d, __dmul_rn(sig, __dmul_rn(__dadd_rn(1.0, __dmul_rn(b, xv)), om)));
    const double wrt = __dsub_rn(__dmul_rn(xv, __dmul_rn(sig, om)), __dmul_rn(__dmul_rn(xv, xv), __dmul_rn(sig, sig)));
    acc += (double)(T)__dmul_rn(d, wrt);      // each term is rounded to T before it is added, as there
  }
  double s = block_sum_d<LOSS_THREADS>(acc);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
template <typename T>
__global__ void swish_final_kernel(const double* __restrict__ partial, int nblocks, T* dbeta, int accumulate) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double s = 0.0;
    for (int b = 0; b < nblocks; ++b) s += partial[b];
    dbeta[0] = accumulate ? add_rn(dbeta[0], (T)s) : (T)s;
  }
}

template <typename T>
static prad_status swish_backward_t(prad_ctx* ctx, const void* x, const void* beta, const void* dy, void* dx,
                                    void* dbeta, int64_t n, int accumulate) {
  int grid = stream_grid(ctx, n, LOSS_THREADS * 4, 4);
  prad_status s = ensure_workspace(ctx, (size_t)grid * sizeof(double));
  if (s) return s;
  swish_backward_kernel<T><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const T*)x, (const T*)beta, (const T*)dy,
                                                                    (T*)dx, (double*)ctx->ws, n);
  PRAD_LAUNCHED(ctx);
  swish_final_kernel<T><<<1, 32, 0, ctx->stream>>>((const double*)ctx->ws, grid, (T*)dbeta, accumulate);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

// ---------------------------------------------------------------- SwigLU
// SwigLUOperation.cs:59-145: y = swish(x w_j + b_j) * (x v_j + c_j) with per-column w, v, b, c and
// the constructor's scalar beta; double arithmetic throughout, as there.  Backward as written:
// der = swish + beta * sigmoid * (1 - swish); the four per-column sums run over the rows.
// One thread per column and band of rows (consecutive threads = consecutive columns, so a row
// segment is read contiguously); bands are added in band order by the second kernel.
struct SwigLUParams { const void *w, *v, *b, *c; double beta; };

template <typename T>
__global__ void __launch_bounds__(128)
swiglu_forward_kernel(const T* __restrict__ x, SwigLUParams p, T* __restrict__ y, int64_t rows, int cols,
                      int64_t rows_per_band) {
  const int j = blockIdx.x * 128 + threadIdx.x;
  if (j >= cols) return;
  const double w = (double)((const T*)p.w)[j], v = (double)((const T*)p.v)[j];
  const double b = (double)((const T*)p.b)[j], c = (double)((const T*)p.c)[j];
  const int64_t r1 = min(rows, (int64_t)(blockIdx.y + 1) * rows_per_band);
  for (int64_t i = (int64_t)blockIdx.y * rows_per_band; i < r1; ++i) {
    const double xv = (double)x[i * cols + j];
    const double f = __dadd_rn(__dmul_rn(xv, w), b);
    const double swish = __dmul_rn(f, __ddiv_rn(1.0, __dadd_rn(1.0, exp(__dmul_rn(-p.beta, f)))));
    y[i * cols + j] = (T)__dmul_rn(swish, __dadd_rn(__dmul_rn(xv, v), c));
  }
}
template <typename T>
__global__ void __launch_bounds__(128)
swiglu_backward_kernel(const T* __restrict__ x, SwigLUParams p, const T* __restrict__ dy, T* __restrict__ dx,
                       double* __restrict__ partial, int64_t rows, int cols, int64_t rows_per_band) {
  const int j = blockIdx.x * 128 + threadIdx.x;
  if (j >= cols) return;
  const double w = (double)((const T*)p.w)[j], v = (double)((const T*)p.v)[j];
  const double b = (double)((const T*)p.b)[j], c = (double)((const T*)p.c)[j];
  const int64_t r1 = min(rows, (int64_t)(blockIdx.y + 1) * rows_per_band);
  double s_w = 0.0, s_v = 0.0, s_b = 0.0, s_c = 0.0;
  for (int64_t i = (int64_t)blockIdx.y * rows_per_band; i < r1; ++i) {
    const double xv = (double)x[i * cols + j], d = (double)dy[i * cols + j];
    const double f = __dadd_rn(__dmul_rn(xv, w), b);
    const double sig = __ddiv_rn(1.0, __dadd_rn(1.0, exp(__dmul_rn(-p.beta, f))));
    const double swish = __dmul_rn(f, sig);
    const double der = __dadd_rn(swish, __dmul_rn(__dmul_rn(p.beta, sig), __dsub_rn(1.0, swish)));
    const double lin = __dadd_rn(__dmul_rn(xv, v), c);
    dx[i * cols + j] = (T)__dmul_rn(d, __dmul_rn(v, der));
    s_w = __dadd_rn(s_w, __dmul_rn(d, __dmul_rn(__dmul_rn(xv, der), lin)));
    s_v = __dadd_rn(s_v, __dmul_rn(d, __dmul_rn(swish, xv)));
    s_b = __dadd_rn(s_b, __dmul_rn(d, __dmul_rn(der, lin)));
    s_c = __dadd_rn(s_c, __dmul_rn(d, swish));
  }
  double* out = partial + ((int64_t)blockIdx.y * 4) * cols + j;
  out[0] = s_w; out[cols] = s_v; out[2 * (int64_t)cols] = s_b; out[3 * (int64_t)cols] = s_c;
}
template <typename T>
__global__ void __launch_bounds__(128)
swiglu_final_kernel(const double* __restrict__ partial, int bands, int cols, T* dw, T* dv, T* db, T* dc) {
  const int j = blockIdx.x * 128 + threadIdx.x;
  if (j >= cols) return;
  double s[4] = {0.0, 0.0, 0.0, 0.0};
  for (int band = 0; band < bands; ++band)
#pragma unroll
    for (int q = 0; q < 4; ++q) s[q] = __dadd_rn(s[q], partial[((int64_t)band * 4 + q) * cols + j]);
  dw[j] = (T)s[0]; dv[j] = (T)s[1]; db[j] = (T)s[2]; dc[j] = (T)s[3];
}

static int swiglu_bands(const prad_ctx* ctx, int64_t rows, int cols) {
  const int64_t col_blocks = ceil_div(cols, 128);
  int64_t bands = ceil_div((int64_t)ctx->sm_count * 8, col_blocks);
  if (bands > ceil_div(rows, 16)) bands = ceil_div(rows, 16);   // at least 16 rows per band
  return (int)(bands < 1 ? 1 : bands);
}

// ---------------------------------------------------------------- BatchNormalization
// BatchNormalizationOperation.cs:52-158, as written: one population over the whole matrix; the
// variance loop and the normalisation use the SUM S of the elements and the sum V of squared
// deviations from S (the local variables at that point), while the fields read by the backward
// are S / n and V / n.  Everything in double.  stats (device, 4 doubles) = { S/n, V/n, S, V }.
template <typename T>
__global__ void __launch_bounds__(LOSS_THREADS)
bn_partial_kernel(const T* __restrict__ x, const double* __restrict__ stats, double* __restrict__ partial,
                  int64_t n, int second) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const double S = second ? stats[2] : 0.0;
  double acc = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const double v = (double)x[i];
    if (second) { const double d = __dsub_rn(v, S); acc += __dmul_rn(d, d); }
    else acc += v;
  }
  double s = block_sum_d<LOSS_THREADS>(acc);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void bn_final_kernel(const double* __restrict__ partial, int nblocks, double* stats, double n, int second) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double s = 0.0;
    for (int b = 0; b < nblocks; ++b) s += partial[b];
    stats[second ? 3 : 2] = s;
    stats[second ? 1 : 0] = s / n;
  }
}
template <typename T>
__global__ void __launch_bounds__(LOSS_THREADS)
bn_forward_kernel(const T* __restrict__ x, const double* __restrict__ stats, T* __restrict__ y, int64_t n) {
  const double S = stats[2], den = sqrt(__dadd_rn(stats[3], 1E-6));
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = (T)__ddiv_rn(__dsub_rn((double)x[i], S), den);
}
template <typename T>
__global__ void __launch_bounds__(LOSS_THREADS)
bn_backward_kernel(const T* __restrict__ x, const double* __restrict__ stats, const T* __restrict__ dy,
                   T* __restrict__ dx, int64_t n) {
  const double mean = stats[0], nn = (double)n;
  const double inv = __ddiv_rn(1.0, sqrt(__dadd_rn(stats[1], 1E-6)));
  const double inv3 = __dmul_rn(__dmul_rn(inv, inv), inv);
  const double dy_dmean = __ddiv_rn(-inv, nn);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const double xm = __dsub_rn((double)x[i], mean);
    const double dy_dvar = __dmul_rn(__dmul_rn(-0.5, xm), inv3);
    const double dvar_dx = __ddiv_rn(__dmul_rn(2.0, xm), nn);
    dx[i] = (T)__dmul_rn(__dadd_rn(__dadd_rn(inv, __dmul_rn(dy_dvar, dvar_dx)), dy_dmean), (double)dy[i]);
  }
}

// ---------------------------------------------------------------- embedding
// EmbeddingOperation.cs:56-60: out[i] = W[(int)input[i,0]]
template <typename T>
__global__ void __launch_bounds__(256)
embedding_gather_kernel(const T* __restrict__ index_col, const T* __restrict__ W,
                        T* __restrict__ out, int n, int vocab, int dim, int* __restrict__ bad) {
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    int idx = (int)index_col[i];
    if (idx < 0 || idx >= vocab) {  // the managed code would throw IndexOutOfRange
      if (threadIdx.x == 0) atomicExch(bad, i + 1);
      continue;
    }
    for (int j = threadIdx.x; j < dim; j += blockDim.x)
      out[(int64_t)i * dim + j] = W[(int64_t)idx * dim + j];
  }
}

// EmbeddingOperation.cs:69-76: dW[idx[i]][j] += dOut[i][j] for i = 0..n-1 IN THAT ORDER.
// Vocabulary rows are dealt to CTAs round-robin.  A CTA scans the index column in tiles,
// compacts (stably) the positions whose row it owns, and adds those rows of dOut one after
// the other; column j is always handled by the same thread, so every dW element sees its
// contributions in input-row order and the sum is bit-identical to the sequential loop.
// No floating-point atomics anywhere.
template <typename T> struct EmbVec;
template <> struct EmbVec<float> { using type = float4; static constexpr int N = 4; };
template <> struct EmbVec<double> { using type = double2; static constexpr int N = 2; };

constexpr int EMB_THREADS = 256;
constexpr int EMB_ITEMS = 4;
constexpr int EMB_TILE = EMB_THREADS * EMB_ITEMS;
constexpr int EMB_CAP = 2048;       // positions a CTA keeps in shared memory before it falls back to adding in place

// One tile of the index list: the positions whose vocabulary row this CTA owns (row % B == b), appended to
// `list` in input order (thread order == element order).  Returns how many; all threads get the same count.
template <typename T>
__device__ __forceinline__ int emb_compact_tile(const T* __restrict__ index_col, int tile, int n, int vocab, int B, int b,
                                                int* list, int cap_left, int* warp_cnt, int* tile_cnt, int* bad) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int mine[EMB_ITEMS];
  int c = 0;
#pragma unroll
  for (int q = 0; q < EMB_ITEMS; ++q) {
    const int i = tile + threadIdx.x * EMB_ITEMS + q;
    mine[q] = -1;
    if (i < n) {
      const int idx = (int)index_col[i];
      if (idx < 0 || idx >= vocab) {
        if (b == 0) atomicExch(bad, i + 1);
      } else if (idx % B == b) {
        mine[q] = i;
        ++c;
      }
    }
  }
  int incl = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += u;
  }
  if (lane == 31) warp_cnt[w] = incl;
  __syncthreads();
  int base = 0;
  for (int k = 0; k < w; ++k) base += warp_cnt[k];
  if (threadIdx.x == EMB_THREADS - 1) *tile_cnt = base + incl;
  int pos = base + incl - c;
#pragma unroll
  for (int q = 0; q < EMB_ITEMS; ++q)
    if (mine[q] >= 0) {
      if (pos < cap_left) list[pos] = mine[q];
      ++pos;
    }
  __syncthreads();
  return *tile_cnt;
}

// dW[idx[i]] += dOut[i] for i ascending (EmbeddingOperation.cs:70-86), without float atomics: vocabulary rows are
// dealt to the CTAs round-robin and a CTA adds the rows of dOut that hit one of its rows in input order.
// Usual case: all positions a CTA owns fit in shared memory; then every owned row is summed in registers and
// written exactly once (rows nobody hit are written as zeros), so dOut is read once and the table written once.
// Otherwise (more than EMB_CAP hits on one CTA's rows) the CTA zeroes its rows and adds tile by tile in place.
template <typename T>
__global__ void __launch_bounds__(EMB_THREADS)
embedding_scatter_ordered_kernel(const T* __restrict__ index_col, const T* __restrict__ dOut,
                                 T* __restrict__ dW, int n, int vocab, int dim,
                                 int* __restrict__ bad) {
  __shared__ int list[EMB_CAP];
  __shared__ int match[EMB_CAP];
  __shared__ int warp_cnt[EMB_THREADS / 32];
  __shared__ int tile_cnt, match_cnt;
  const int B = gridDim.x, b = blockIdx.x;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;

  // ---- collect the owned positions
  int total = 0;
  bool fits = true;
  for (int tile = 0; tile < n && fits; tile += EMB_TILE) {
    const int cnt = emb_compact_tile<T>(index_col, tile, n, vocab, B, b, list + total, EMB_CAP - total, warp_cnt, &tile_cnt, bad);
    if (total + cnt > EMB_CAP) fits = false;
    else total += cnt;
    __syncthreads();
  }

  if (fits) {
    using V = typename EmbVec<T>::type;
    constexpr int VEC = EmbVec<T>::N;
    const bool vec = dim % VEC == 0 && (((uintptr_t)dOut | (uintptr_t)dW) & 15) == 0;
    for (int v = b; v < vocab; v += B) {
      // positions that hit row v, in input order (warp 0: ordered compaction of 32 list entries per trip)
      if (w == 0) {
        int mc = 0;
        for (int e0 = 0; e0 < total; e0 += 32) {
          const int e = e0 + lane;
          const int i = e < total ? list[e] : -1;
          const bool hit = i >= 0 && (int)index_col[i] == v;
          const unsigned m = __ballot_sync(0xffffffffu, hit);
          if (hit) match[mc + __popc(m & ((1u << lane) - 1u))] = i;
          mc += __popc(m);
        }
        if (lane == 0) match_cnt = mc;
      }
      __syncthreads();
      const int mc = match_cnt;
      T* row = dW + (int64_t)v * dim;
      if (vec) {
        for (int j = threadIdx.x; j < dim / VEC; j += EMB_THREADS) {
          T acc[VEC];
#pragma unroll
          for (int q = 0; q < VEC; ++q) acc[q] = (T)0;
          for (int k = 0; k < mc; ++k) {
            const V x = __ldcs(reinterpret_cast<const V*>(dOut + (int64_t)match[k] * dim) + j);
#pragma unroll
            for (int q = 0; q < VEC; ++q) acc[q] = add_rn(acc[q], reinterpret_cast<const T*>(&x)[q]);
          }
          __stcs(reinterpret_cast<V*>(row) + j, *reinterpret_cast<const V*>(acc));
        }
      } else {
        for (int j = threadIdx.x; j < dim; j += EMB_THREADS) {
          T acc = (T)0;
          for (int k = 0; k < mc; ++k) acc = add_rn(acc, dOut[(int64_t)match[k] * dim + j]);
          row[j] = acc;
        }
      }
      __syncthreads();
    }
    return;
  }

  // ---- more hits than the list holds: zero the owned rows, then add tile by tile in place
  for (int v = b; v < vocab; v += B)
    for (int j = threadIdx.x; j < dim; j += EMB_THREADS) dW[(int64_t)v * dim + j] = (T)0;
  __syncthreads();
  for (int tile = 0; tile < n; tile += EMB_TILE) {
    const int cnt = emb_compact_tile<T>(index_col, tile, n, vocab, B, b, list, EMB_CAP, warp_cnt, &tile_cnt, bad);
    for (int e = 0; e < cnt; ++e) {
      const int i = list[e];
      const int idx = (int)index_col[i];
      for (int j = threadIdx.x; j < dim; j += EMB_THREADS) {
        const int64_t o = (int64_t)idx * dim + j;
        dW[o] = add_rn(dW[o], dOut[(int64_t)i * dim + j]);
      }
    }
    __syncthreads();
  }
}

static prad_status check_bad_index(prad_ctx* ctx, int* d_bad, const char* who) {
  PRAD_NOT_CAPTURING(ctx, who);   // the index check reads a flag back
  int h = 0;
  PRAD_CUDA(cudaMemcpyAsync(&h, d_bad, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  PRAD_REQUIRE(h == 0, PRAD_ERR_INVALID, "%s: index at input row %d is outside [0, vocab)", who, h - 1);
  return PRAD_OK;
}

// Ordered scatter-add for other translation units (the PRAD Tensor gather reverse): dW[idx[i]] += dOut[i]
// for i ascending; `bad` is a device int that receives 1 + the first offending position.
prad_status embedding_scatter_ordered(prad_ctx* ctx, prad_dtype dt, const void* index_col, const void* dOut,
                                      void* dW, int n, int vocab, int dim, int* bad) {
  int grid = vocab < ctx->sm_count * 8 ? vocab : ctx->sm_count * 8;
  if (dt == PRAD_F32) embedding_scatter_ordered_kernel<float><<<grid, EMB_THREADS, 0, ctx->stream>>>((const float*)index_col, (const float*)dOut, (float*)dW, n, vocab, dim, bad);
  else embedding_scatter_ordered_kernel<double><<<grid, EMB_THREADS, 0, ctx->stream>>>((const double*)index_col, (const double*)dOut, (double*)dW, n, vocab, dim, bad);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

}  // namespace prad

using namespace prad;

extern "C" {

prad_status prad_mse_forward(prad_ctx* ctx, prad_dtype dt, const void* out, const void* target,
                             void* loss_out, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows > 0 && cols > 0 && out && target && loss_out, PRAD_ERR_INVALID,
               "prad_mse_forward: bad argument");
  return dt == PRAD_F32 ? loss_forward_t<float>(ctx, out, target, loss_out, rows, cols, 0)
                        : loss_forward_t<double>(ctx, out, target, loss_out, rows, cols, 0);
}

prad_status prad_cce_forward(prad_ctx* ctx, prad_dtype dt, const void* out, const void* target,
                             void* loss_out, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows > 0 && cols > 0 && out && target && loss_out, PRAD_ERR_INVALID,
               "prad_cce_forward: bad argument");
  return dt == PRAD_F32 ? loss_forward_t<float>(ctx, out, target, loss_out, rows, cols, 1)
                        : loss_forward_t<double>(ctx, out, target, loss_out, rows, cols, 1);
}

prad_status prad_mse_backward(prad_ctx* ctx, prad_dtype dt, const void* out, const void* target,
                              void* grad, int64_t rows, int cols, int64_t rows_total) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0 && rows_total >= 1, PRAD_ERR_INVALID,
               "prad_mse_backward: bad argument");
  int64_t n = rows * cols;
  if (n == 0) return PRAD_OK;
  PRAD_REQUIRE(out && target && grad, PRAD_ERR_INVALID, "prad_mse_backward: null pointer");
  int grid = stream_grid(ctx, n, 256 * 4, 8);
  if (dt == PRAD_F32)
    mse_backward_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)out, (const float*)target, (float*)grad, n, 2.0f / (float)(rows_total * cols));
  else
    mse_backward_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)out, (const double*)target, (double*)grad, n, 2.0 / (double)(rows_total * cols));
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_cce_backward(prad_ctx* ctx, prad_dtype dt, const void* out, const void* target,
                              void* grad, int64_t rows, int cols, int64_t rows_total) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0 && rows_total >= 1, PRAD_ERR_INVALID,
               "prad_cce_backward: bad argument");
  int64_t n = rows * cols;
  if (n == 0) return PRAD_OK;
  PRAD_REQUIRE(out && target && grad, PRAD_ERR_INVALID, "prad_cce_backward: null pointer");
  int grid = stream_grid(ctx, n, 256 * 4, 8);
  if (dt == PRAD_F32)
    cce_backward_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)out, (const float*)target, (float*)grad, n, 1.0f / (float)rows_total);
  else
    cce_backward_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)out, (const double*)target, (double*)grad, n, 1.0 / (double)rows_total);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_embedding_forward(prad_ctx* ctx, prad_dtype dt, const void* index_col,
                                   const void* W, void* out, int n, int vocab, int dim) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && vocab >= 0 && dim >= 0, PRAD_ERR_INVALID,
               "prad_embedding_forward: bad argument");
  if (n == 0 || dim == 0) return PRAD_OK;
  PRAD_REQUIRE(index_col && W && out, PRAD_ERR_INVALID, "prad_embedding_forward: null pointer");
  prad_status s = ensure_workspace(ctx, 256);
  if (s) return s;
  int* bad = (int*)ctx->ws;
  PRAD_CUDA(cudaMemsetAsync(bad, 0, sizeof(int), ctx->stream));
  int grid = stream_grid(ctx, n, 1, 8);
  if (dt == PRAD_F32) embedding_gather_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)index_col, (const float*)W, (float*)out, n, vocab, dim, bad);
  else embedding_gather_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)index_col, (const double*)W, (double*)out, n, vocab, dim, bad);
  PRAD_LAUNCHED(ctx);
  return check_bad_index(ctx, bad, "prad_embedding_forward");
}

prad_status prad_embedding_backward(prad_ctx* ctx, prad_dtype dt, const void* index_col,
                                    const void* dOut, void* dW, int n, int vocab, int dim) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && vocab >= 0 && dim >= 0, PRAD_ERR_INVALID,
               "prad_embedding_backward: bad argument");
  if (vocab == 0 || dim == 0) return PRAD_OK;
  PRAD_REQUIRE(dW && (n == 0 || (index_col && dOut)), PRAD_ERR_INVALID,
               "prad_embedding_backward: null pointer");
  prad_status s = ensure_workspace(ctx, 256);
  if (s) return s;
  int* bad = (int*)ctx->ws;
  PRAD_CUDA(cudaMemsetAsync(bad, 0, sizeof(int), ctx->stream));
  int grid = vocab < ctx->sm_count * 8 ? vocab : ctx->sm_count * 8;
  if (dt == PRAD_F32) embedding_scatter_ordered_kernel<float><<<grid, EMB_THREADS, 0, ctx->stream>>>((const float*)index_col, (const float*)dOut, (float*)dW, n, vocab, dim, bad);
  else embedding_scatter_ordered_kernel<double><<<grid, EMB_THREADS, 0, ctx->stream>>>((const double*)index_col, (const double*)dOut, (double*)dW, n, vocab, dim, bad);
  PRAD_LAUNCHED(ctx);
  return check_bad_index(ctx, bad, "prad_embedding_backward");
}

prad_status prad_swish_forward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* beta, void* y, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && (n == 0 || (x && beta && y)), PRAD_ERR_INVALID,
               "prad_swish_forward: bad dtype, null pointer or negative size");
  if (n == 0) return PRAD_OK;
  const int grid = stream_grid(ctx, n, LOSS_THREADS * 4, 4);
  if (dt == PRAD_F32) swish_forward_kernel<float><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const float*)x, (const float*)beta, (float*)y, n);
  else swish_forward_kernel<double><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const double*)x, (const double*)beta, (double*)y, n);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_swish_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* beta, const void* dy,
                                void* dx, void* dbeta, int64_t n, int accumulate) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && beta && dbeta && (n == 0 || (x && dy && dx)), PRAD_ERR_INVALID,
               "prad_swish_backward: bad dtype, null pointer or negative size");
  return dt == PRAD_F32 ? swish_backward_t<float>(ctx, x, beta, dy, dx, dbeta, n, accumulate)
                        : swish_backward_t<double>(ctx, x, beta, dy, dx, dbeta, n, accumulate);
}

prad_status prad_swiglu_forward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* w, const void* v,
                                const void* b, const void* c, double beta, void* y, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_swiglu_forward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && w && v && b && c && y, PRAD_ERR_INVALID, "prad_swiglu_forward: null pointer");
  int bands = swiglu_bands(ctx, rows, cols);
  const int64_t rpb = ceil_div(rows, bands);
  bands = (int)ceil_div(rows, rpb);
  const dim3 grid((unsigned)ceil_div(cols, 128), (unsigned)bands);
  SwigLUParams p{w, v, b, c, beta};
  if (dt == PRAD_F32) swiglu_forward_kernel<float><<<grid, 128, 0, ctx->stream>>>((const float*)x, p, (float*)y, rows, cols, rpb);
  else swiglu_forward_kernel<double><<<grid, 128, 0, ctx->stream>>>((const double*)x, p, (double*)y, rows, cols, rpb);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_swiglu_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* w, const void* v,
                                 const void* b, const void* c, double beta, const void* dy, void* dx, void* dw,
                                 void* dv, void* db, void* dc, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_swiglu_backward: bad argument");
  if (cols == 0) return PRAD_OK;
  PRAD_REQUIRE(w && v && b && c && dw && dv && db && dc && (rows == 0 || (x && dy && dx)), PRAD_ERR_INVALID,
               "prad_swiglu_backward: null pointer");
  int bands = rows == 0 ? 0 : swiglu_bands(ctx, rows, cols);
  const int64_t rpb = bands ? ceil_div(rows, bands) : 1;
  bands = (int)ceil_div(rows, rpb);
  prad_status st = ensure_workspace(ctx, (size_t)(bands ? bands : 1) * 4 * cols * sizeof(double));
  if (st) return st;
  SwigLUParams p{w, v, b, c, beta};
  const unsigned cb = (unsigned)ceil_div(cols, 128);
  if (bands) {
    const dim3 grid(cb, (unsigned)bands);
    if (dt == PRAD_F32) swiglu_backward_kernel<float><<<grid, 128, 0, ctx->stream>>>((const float*)x, p, (const float*)dy, (float*)dx, (double*)ctx->ws, rows, cols, rpb);
    else swiglu_backward_kernel<double><<<grid, 128, 0, ctx->stream>>>((const double*)x, p, (const double*)dy, (double*)dx, (double*)ctx->ws, rows, cols, rpb);
    PRAD_LAUNCHED(ctx);
  }
  if (dt == PRAD_F32) swiglu_final_kernel<float><<<cb, 128, 0, ctx->stream>>>((const double*)ctx->ws, bands, cols, (float*)dw, (float*)dv, (float*)db, (float*)dc);
  else swiglu_final_kernel<double><<<cb, 128, 0, ctx->stream>>>((const double*)ctx->ws, bands, cols, (double*)dw, (double*)dv, (double*)db, (double*)dc);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_batchnorm_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, void* stats, int64_t rows,
                                   int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_batchnorm_forward: bad argument");
  const int64_t n = rows * cols;
  if (n == 0) return PRAD_OK;
  PRAD_REQUIRE(x && y && stats, PRAD_ERR_INVALID, "prad_batchnorm_forward: null pointer");
  const int grid = stream_grid(ctx, n, LOSS_THREADS * 4, 4);
  prad_status st = ensure_workspace(ctx, (size_t)grid * sizeof(double));
  if (st) return st;
  double* part = (double*)ctx->ws;
  double* sd = (double*)stats;
  for (int second = 0; second < 2; ++second) {
    if (dt == PRAD_F32) bn_partial_kernel<float><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const float*)x, sd, part, n, second);
    else bn_partial_kernel<double><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const double*)x, sd, part, n, second);
    PRAD_LAUNCHED(ctx);
    bn_final_kernel<<<1, 32, 0, ctx->stream>>>(part, grid, sd, (double)n, second);
    PRAD_LAUNCHED(ctx);
  }
  if (dt == PRAD_F32) bn_forward_kernel<float><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const float*)x, sd, (float*)y, n);
  else bn_forward_kernel<double><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const double*)x, sd, (double*)y, n);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_batchnorm_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* stats, const void* dy,
                                    void* dx, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_batchnorm_backward: bad argument");
  const int64_t n = rows * cols;
  if (n == 0) return PRAD_OK;
  PRAD_REQUIRE(x && stats && dy && dx, PRAD_ERR_INVALID, "prad_batchnorm_backward: null pointer");
  const int grid = stream_grid(ctx, n, LOSS_THREADS * 4, 4);
  if (dt == PRAD_F32) bn_backward_kernel<float><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const float*)x, (const double*)stats, (const float*)dy, (float*)dx, n);
  else bn_backward_kernel<double><<<grid, LOSS_THREADS, 0, ctx->stream>>>((const double*)x, (const double*)stats, (const double*)dy, (double*)dx, n);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

}  // extern "C"
