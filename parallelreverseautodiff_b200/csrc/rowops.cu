// Row-wise kernels: softmax and the reference form of layer normalisation, forward and
// backward.  One warp owns one row (lanes stride over the columns, so a warp's loads are
// contiguous 128-byte segments); row reductions are warp shuffles in a fixed order, which
// makes every result bit-reproducible from run to run.
// (Compiled with -fmad=false.)
#include "act_math.cuh"
#include "common.cuh"

namespace prad {

template <typename A> __device__ __forceinline__ A warp_sum(A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename A> __device__ __forceinline__ A warp_max(A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    A u = __shfl_xor_sync(0xffffffffu, v, o);
    v = u > v ? u : v;
  }
  return v;
}

constexpr int ROW_WARPS = 8;

// SoftmaxOperation.cs:85-109: subtract the row maximum, exponentiate, divide by the sum.
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
softmax_forward_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T* xr = x + r * cols;
    T* yr = y + r * cols;
    T mx = -INFINITY;
    for (int j = lane; j < cols; j += 32) { T v = xr[j]; mx = v > mx ? v : mx; }
    mx = warp_max(mx);
    T sum = 0;
    for (int j = lane; j < cols; j += 32) {
      T e = t_exp(sub_rn(xr[j], mx));
      yr[j] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    for (int j = lane; j < cols; j += 32) yr[j] = div_rn(yr[j], sum);
  }
}

// SineSoftmaxOperation.cs:47-77,155-176: e = exp(sin x), M = sum of e over the row, y_j = e_j / (M + e_j);
// Backward as written there: dx_j = dy_j * (M * e_j * cos x_j) / (M + e_j)^2.  One warp per row; the
// float overloads of PradMath go through double, so do these.
template <typename T> __device__ __forceinline__ T sine_exp(T x) { return (T)exp((double)(T)sin((double)x)); }
template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(ROW_WARPS * 32)
sine_softmax_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T* xr = x + r * cols;
    T m = 0;
    for (int j = lane; j < cols; j += 32) m += sine_exp<T>(xr[j]);
    m = warp_sum(m);
    for (int j = lane; j < cols; j += 32) {
      const T e = sine_exp<T>(xr[j]);
      if (!BACKWARD) {
        out[r * cols + j] = div_rn(e, add_rn(m, e));
      } else {
        const T num = mul_rn(mul_rn(m, e), (T)cos((double)xr[j]));
        const T s = add_rn(m, e);
        out[r * cols + j] = mul_rn(dy[r * cols + j], div_rn(num, mul_rn(s, s)));
      }
    }
  }
}

// SoftmaxOperation.cs:53-83.  The reference walks the explicit Jacobian; algebraically
//   dx_j = dy_j*y_j*(1-y_j) - y_j*sum_{k!=j} dy_k*y_k = y_j*(dy_j - sum_k dy_k*y_k).
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
softmax_backward_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                        int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T* yr = y + r * cols;
    const T* dr = dy + r * cols;
    T dot = 0;
    for (int j = lane; j < cols; j += 32) dot += mul_rn(dr[j], yr[j]);
    dot = warp_sum(dot);
    for (int j = lane; j < cols; j += 32) dx[r * cols + j] = mul_rn(yr[j], sub_rn(dr[j], dot));
  }
}

template <typename T> struct LnEps;
template <> struct LnEps<float> { __device__ static float v() { return 1e-9f; } };
template <> struct LnEps<double> { __device__ static double v() { return 1e-9; } };

// LayerNormalizationOperation.cs:56-85: mean = Average(), sigma = Sqrt(Sum((x-mean)^2)/n),
// y = (x-mean)/(sigma+eps).  Sums accumulate in double (LINQ), results are cast to T.
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
layernorm_forward_kernel(const T* __restrict__ x, T* __restrict__ y, T* __restrict__ mean,
                         T* __restrict__ stdv, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T* xr = x + r * cols;
    double s = 0.0;
    for (int j = lane; j < cols; j += 32) s += (double)xr[j];
    s = warp_sum(s);
    const T mu = (T)(s / (double)cols);
    double v = 0.0;
    for (int j = lane; j < cols; j += 32) {
      T d = sub_rn(xr[j], mu);
      v += (double)mul_rn(d, d);
    }
    v = warp_sum(v);
    const T sd = sqrt_rn(div_rn((T)v, (T)cols));
    if (lane == 0) { mean[r] = mu; stdv[r] = sd; }
    const T den = add_rn(sd, LnEps<T>::v());
    for (int j = lane; j < cols; j += 32) y[r * cols + j] = div_rn(sub_rn(xr[j], mu), den);
  }
}

// LayerNormalizationOperation.cs:88-112 -- the reference's diagonal-only backward:
//   dx = dy * ( (1-1/n)/(sigma+eps) - (x-mean)^2 / (n*(sigma+eps)^3) )
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
layernorm_backward_kernel(const T* __restrict__ x, const T* __restrict__ mean,
                          const T* __restrict__ stdv, const T* __restrict__ dy,
                          T* __restrict__ dx, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T mu = mean[r];
    const T se = add_rn(stdv[r], LnEps<T>::v());
    const T inv = div_rn((T)1, se);
    const T exp1 = mul_rn(sub_rn((T)1, div_rn((T)1, (T)cols)), inv);
    const T den = mul_rn((T)cols, mul_rn(mul_rn(se, se), se));
    for (int j = lane; j < cols; j += 32) {
      T d = sub_rn(x[r * cols + j], mu);
      T exp2 = div_rn(mul_rn(d, d), den);
      dx[r * cols + j] = mul_rn(dy[r * cols + j], sub_rn(exp1, exp2));
    }
  }
}

// ScaleAndShiftOperation.cs:60-73 / :84-98.  One warp per row; the two row sums accumulate in
// double and are cast back (the managed loop adds in T, left to right).
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
scale_shift_forward_kernel(const T* __restrict__ x, const T* __restrict__ beta, const T* __restrict__ gamma,
                           T* __restrict__ y, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T b = beta[r], g = gamma[r];
    for (int j = lane; j < cols; j += 32) y[r * cols + j] = add_rn(mul_rn(x[r * cols + j], b), g);
  }
}
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
scale_shift_backward_kernel(const T* __restrict__ x, const T* __restrict__ beta, const T* __restrict__ dy,
                            T* __restrict__ dx, T* __restrict__ dbeta, T* __restrict__ dgamma, int64_t rows,
                            int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T b = beta[r];
    double sb = 0.0, sg = 0.0;
    for (int j = lane; j < cols; j += 32) {
      const T d = dy[r * cols + j];
      dx[r * cols + j] = mul_rn(d, b);
      sb += (double)mul_rn(d, x[r * cols + j]);
      sg += (double)d;
    }
    sb = warp_sum(sb);
    sg = warp_sum(sg);
    if (lane == 0) { dbeta[r] = (T)sb; dgamma[r] = (T)sg; }
  }
}

// RMSNormOperation.cs:56-72 / :85-106 (Pow(x, 2) and Pow(rms, 3) as products)
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
rmsnorm_forward_kernel(const T* __restrict__ x, const T* __restrict__ g, T* __restrict__ y, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    double ss = 0.0;
    for (int j = lane; j < cols; j += 32) { const T v = x[r * cols + j]; ss += (double)mul_rn(v, v); }
    ss = warp_sum(ss);
    const T rms = sqrt_rn(div_rn((T)ss, (T)cols));
    for (int j = lane; j < cols; j += 32)
      y[r * cols + j] = mul_rn(div_rn(x[r * cols + j], rms), g[r * cols + j]);
  }
}
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
rmsnorm_backward_kernel(const T* __restrict__ x, const T* __restrict__ g, const T* __restrict__ dy,
                        T* __restrict__ dx, T* __restrict__ dg, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    double ss = 0.0;
    for (int j = lane; j < cols; j += 32) { const T v = x[r * cols + j]; ss += (double)mul_rn(v, v); }
    ss = warp_sum(ss);
    const T rms = sqrt_rn(div_rn((T)ss, (T)cols));
    const T den = mul_rn((T)cols, mul_rn(mul_rn(rms, rms), rms));
    for (int j = lane; j < cols; j += 32) {
      const T xv = x[r * cols + j], gv = g[r * cols + j], d = dy[r * cols + j];
      const T a = sub_rn(div_rn(gv, rms), div_rn(mul_rn(mul_rn(xv, gv), xv), den));
      dx[r * cols + j] = mul_rn(a, d);
      dg[r * cols + j] = mul_rn(div_rn(xv, rms), d);
    }
  }
}

// MatrixSumOperation.cs:45-50 / MatrixAverageOperation.cs:45-50: LINQ Sum / Average of a row
// (double accumulator); backward :57-65 copies dOutput[i][0] (divided by cols for the average).
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
row_sum_forward_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int cols, int average) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r = warp; r < rows; r += nwarps) {
    double s = 0.0;
    for (int j = lane; j < cols; j += 32) s += (double)x[r * cols + j];
    s = warp_sum(s);
    if (lane == 0) y[r] = average ? (T)(s / (double)cols) : (T)s;
  }
}
template <typename T>
__global__ void __launch_bounds__(256)
row_sum_backward_kernel(const T* __restrict__ dy, T* __restrict__ dx, int64_t n, int cols, int average) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const T d = dy[i / cols];
    dx[i] = average ? div_rn(d, (T)cols) : d;
  }
}

// MatrixBroadcastOperation.cs:55-62: y[i][j] = x[i % r][j % c]; backward :70-83 adds the tiles
// into each input element k outer, l inner, in T -- one thread per input element, same order.
template <typename T>
__global__ void __launch_bounds__(256)
broadcast_forward_kernel(const T* __restrict__ x, int r, int c, T* __restrict__ y, int64_t n, int C) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = x[(int64_t)((i / C) % r) * c + (int)((i % C) % c)];
}
template <typename T>
__global__ void __launch_bounds__(256)
broadcast_backward_kernel(const T* __restrict__ dy, int R, int C, T* __restrict__ dx, int r, int c) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < (int64_t)r * c; e += stride) {
    const int i = (int)(e / c), j = (int)(e % c);
    T acc = 0;
    for (int k = i; k < R; k += r)
      for (int l = j; l < C; l += c) acc = add_rn(acc, dy[(int64_t)k * C + l]);
    dx[e] = acc;
  }
}

// ---- short rows (cols <= 256): register-cached, several rows per warp -----------------------
// A lane keeps E = ceil(cols/32) elements of each of R rows in registers, so every input is
// read exactly once and R*E independent loads are in flight per lane; the R row reductions
// are independent shuffle chains.  Same arithmetic as the streaming kernels above.
constexpr int SR = 4;   // rows per warp pass

template <typename T, int E>
__global__ void __launch_bounds__(ROW_WARPS * 32)
softmax_forward_short(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r0 = warp * SR; r0 < rows; r0 += nwarps * SR) {
    T v[SR][E];
#pragma unroll
    for (int i = 0; i < SR; ++i)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int j = lane + 32 * e;
        v[i][e] = (r0 + i < rows && j < cols) ? x[(r0 + i) * cols + j] : (T)-INFINITY;
      }
    T mx[SR], sum[SR];
#pragma unroll
    for (int i = 0; i < SR; ++i) {
      mx[i] = v[i][0];
#pragma unroll
      for (int e = 1; e < E; ++e) mx[i] = v[i][e] > mx[i] ? v[i][e] : mx[i];
      mx[i] = warp_max(mx[i]);
    }
#pragma unroll
    for (int i = 0; i < SR; ++i) {
      sum[i] = 0;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int j = lane + 32 * e;
        v[i][e] = (r0 + i < rows && j < cols) ? t_exp(sub_rn(v[i][e], mx[i])) : (T)0;
        sum[i] += v[i][e];
      }
      sum[i] = warp_sum(sum[i]);
    }
#pragma unroll
    for (int i = 0; i < SR; ++i)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int j = lane + 32 * e;
        if (r0 + i < rows && j < cols) y[(r0 + i) * cols + j] = div_rn(v[i][e], sum[i]);
      }
  }
}

template <typename T, int E>
__global__ void __launch_bounds__(ROW_WARPS * 32)
softmax_backward_short(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                       int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r0 = warp * SR; r0 < rows; r0 += nwarps * SR) {
    T yv[SR][E], dv[SR][E];
#pragma unroll
    for (int i = 0; i < SR; ++i)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int j = lane + 32 * e;
        const bool ok = r0 + i < rows && j < cols;
        yv[i][e] = ok ? y[(r0 + i) * cols + j] : (T)0;
        dv[i][e] = ok ? dy[(r0 + i) * cols + j] : (T)0;
      }
    T dot[SR];
#pragma unroll
    for (int i = 0; i < SR; ++i) {
      dot[i] = 0;
#pragma unroll
      for (int e = 0; e < E; ++e) dot[i] += mul_rn(dv[i][e], yv[i][e]);
      dot[i] = warp_sum(dot[i]);
    }
#pragma unroll
    for (int i = 0; i < SR; ++i)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int j = lane + 32 * e;
        if (r0 + i < rows && j < cols) dx[(r0 + i) * cols + j] = mul_rn(yv[i][e], sub_rn(dv[i][e], dot[i]));
      }
  }
}

template <typename T, int E>
__global__ void __launch_bounds__(ROW_WARPS * 32)
layernorm_forward_short(const T* __restrict__ x, T* __restrict__ y, T* __restrict__ mean,
                        T* __restrict__ stdv, int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r0 = warp * SR; r0 < rows; r0 += nwarps * SR) {
    T v[SR][E];
#pragma unroll
    for (int i = 0; i < SR; ++i)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int j = lane + 32 * e;
        v[i][e] = (r0 + i < rows && j < cols) ? x[(r0 + i) * cols + j] : (T)0;
      }
#pragma unroll
    for (int i = 0; i < SR; ++i) {
      double s = 0.0;
#pragma unroll
      for (int e = 0; e < E; ++e) s += (double)v[i][e];   // padding lanes hold 0
      s = warp_sum(s);
      const T mu = (T)(s / (double)cols);
      double q = 0.0;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int j = lane + 32 * e;
        if (j < cols) { T d = sub_rn(v[i][e], mu); q += (double)mul_rn(d, d); }
      }
      q = warp_sum(q);
      const T sd = sqrt_rn(div_rn((T)q, (T)cols));
      if (r0 + i < rows) {
        if (lane == 0) { mean[r0 + i] = mu; stdv[r0 + i] = sd; }
        const T den = add_rn(sd, LnEps<T>::v());
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int j = lane + 32 * e;
          if (j < cols) y[(r0 + i) * cols + j] = div_rn(sub_rn(v[i][e], mu), den);
        }
      }
    }
  }
}

template <typename T, int E>
__global__ void __launch_bounds__(ROW_WARPS * 32)
layernorm_backward_short(const T* __restrict__ x, const T* __restrict__ mean,
                         const T* __restrict__ stdv, const T* __restrict__ dy, T* __restrict__ dx,
                         int64_t rows, int cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * ROW_WARPS;
  for (int64_t r0 = warp * SR; r0 < rows; r0 += nwarps * SR) {
    T xv[SR][E], dv[SR][E], mu[SR], sd[SR];
#pragma unroll
    for (int i = 0; i < SR; ++i) {
      const bool rok = r0 + i < rows;
      mu[i] = rok ? mean[r0 + i] : (T)0;
      sd[i] = rok ? stdv[r0 + i] : (T)1;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int j = lane + 32 * e;
        const bool ok = rok && j < cols;
        xv[i][e] = ok ? x[(r0 + i) * cols + j] : (T)0;
        dv[i][e] = ok ? dy[(r0 + i) * cols + j] : (T)0;
      }
    }
#pragma unroll
    for (int i = 0; i < SR; ++i) {
      const T se = add_rn(sd[i], LnEps<T>::v());
      const T inv = div_rn((T)1, se);
      const T exp1 = mul_rn(sub_rn((T)1, div_rn((T)1, (T)cols)), inv);
      const T den = mul_rn((T)cols, mul_rn(mul_rn(se, se), se));
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int j = lane + 32 * e;
        if (r0 + i < rows && j < cols) {
          T d = sub_rn(xv[i][e], mu[i]);
          dx[(r0 + i) * cols + j] = mul_rn(dv[i][e], sub_rn(exp1, div_rn(mul_rn(d, d), den)));
        }
      }
    }
  }
}

// LayerNorm backward is elementwise once the row statistics are known: for rows that are a
// whole number of 128-bit vectors it streams like a copy (row index = vector index / vectors
// per row; mean and sigma come from L1/L2).  Same arithmetic as layernorm_backward_kernel.
template <typename T> struct RowVec;
template <> struct RowVec<float> { using type = float4; static constexpr int N = 4; };
template <> struct RowVec<double> { using type = double2; static constexpr int N = 2; };

template <typename T>
__global__ void __launch_bounds__(256)
layernorm_backward_flat(const T* __restrict__ x, const T* __restrict__ mean, const T* __restrict__ stdv,
                        const T* __restrict__ dy, T* __restrict__ dx, int64_t nvec, int vec_per_row, int cols) {
  constexpr int VEC = RowVec<T>::N;
  using V = typename RowVec<T>::type;
  constexpr int U = 4;   // vectors in flight per thread
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const T one_minus = sub_rn((T)1, div_rn((T)1, (T)cols));
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < nvec; base += stride * U) {
    V xv[U], dv[U];
    T mu[U], sg[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + u * stride;
      if (i < nvec) {
        xv[u] = __ldcs(reinterpret_cast<const V*>(x) + i);
        dv[u] = __ldcs(reinterpret_cast<const V*>(dy) + i);
        const int64_t r = i / vec_per_row;
        mu[u] = mean[r];
        sg[u] = stdv[r];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + u * stride;
      if (i < nvec) {
        const T se = add_rn(sg[u], LnEps<T>::v());
        const T exp1 = mul_rn(one_minus, div_rn((T)1, se));
        // one IEEE division per vector: (x-mean)^2 / den is formed as (x-mean)^2 * (1/den), at most
        // one unit in the last place away from the reference's division (an IEEE divide per element
        // makes this kernel instruction-bound at two thirds of the HBM rate)
        const T rden = div_rn((T)1, mul_rn((T)cols, mul_rn(mul_rn(se, se), se)));
        V o;
#pragma unroll
        for (int q = 0; q < VEC; ++q) {
          T d = sub_rn(reinterpret_cast<const T*>(&xv[u])[q], mu[u]);
          reinterpret_cast<T*>(&o)[q] =
              mul_rn(reinterpret_cast<const T*>(&dv[u])[q], sub_rn(exp1, mul_rn(mul_rn(d, d), rden)));
        }
        __stcs(reinterpret_cast<V*>(dx) + i, o);
      }
    }
  }
}

static inline int short_e(int cols) { return cols <= 32 ? 1 : cols <= 64 ? 2 : cols <= 128 ? 4 : cols <= 256 ? 8 : 0; }
static inline int short_grid(const prad_ctx* ctx, int64_t rows) {
  return stream_grid(ctx, ceil_div(rows, SR), ROW_WARPS, 8);
}
// runs KERNEL<T, E> for the E that fits `cols`
#define PRAD_SHORT_ROWS(KERNEL, T, ...)                                                          \
  do {                                                                                           \
    const int g_ = short_grid(ctx, rows);                                                        \
    switch (short_e(cols)) {                                                                     \
      case 1: KERNEL<T, 1><<<g_, ROW_WARPS * 32, 0, ctx->stream>>>(__VA_ARGS__); break;          \
      case 2: KERNEL<T, 2><<<g_, ROW_WARPS * 32, 0, ctx->stream>>>(__VA_ARGS__); break;          \
      case 4: KERNEL<T, 4><<<g_, ROW_WARPS * 32, 0, ctx->stream>>>(__VA_ARGS__); break;          \
      default: KERNEL<T, 8><<<g_, ROW_WARPS * 32, 0, ctx->stream>>>(__VA_ARGS__); break;         \
    }                                                                                            \
  } while (0)

static inline int row_grid(const prad_ctx* ctx, int64_t rows) {
  return stream_grid(ctx, rows, ROW_WARPS, 8);
}

}  // namespace prad

using namespace prad;

extern "C" {

prad_status prad_sine_softmax_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_sine_softmax_forward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && y, PRAD_ERR_INVALID, "prad_sine_softmax_forward: null pointer");
  if (dt == PRAD_F32) sine_softmax_kernel<float, false><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)x, nullptr, (float*)y, rows, cols);
  else sine_softmax_kernel<double, false><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const double*)x, nullptr, (double*)y, rows, cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_sine_softmax_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* dy, void* dx, int64_t rows,
                                       int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_sine_softmax_backward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && dy && dx, PRAD_ERR_INVALID, "prad_sine_softmax_backward: null pointer");
  if (dt == PRAD_F32) sine_softmax_kernel<float, true><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)x, (const float*)dy, (float*)dx, rows, cols);
  else sine_softmax_kernel<double, true><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const double*)x, (const double*)dy, (double*)dx, rows, cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_softmax_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y,
                                 int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_softmax_forward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && y, PRAD_ERR_INVALID, "prad_softmax_forward: null pointer");
  if (short_e(cols)) {
    if (dt == PRAD_F32) PRAD_SHORT_ROWS(softmax_forward_short, float, (const float*)x, (float*)y, rows, cols);
    else PRAD_SHORT_ROWS(softmax_forward_short, double, (const double*)x, (double*)y, rows, cols);
  } else if (dt == PRAD_F32) softmax_forward_kernel<float><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)x, (float*)y, rows, cols);
  else softmax_forward_kernel<double><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const double*)x, (double*)y, rows, cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_softmax_backward(prad_ctx* ctx, prad_dtype dt, const void* y, const void* dy,
                                  void* dx, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_softmax_backward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(y && dy && dx, PRAD_ERR_INVALID, "prad_softmax_backward: null pointer");
  if (short_e(cols)) {
    if (dt == PRAD_F32) PRAD_SHORT_ROWS(softmax_backward_short, float, (const float*)y, (const float*)dy, (float*)dx, rows, cols);
    else PRAD_SHORT_ROWS(softmax_backward_short, double, (const double*)y, (const double*)dy, (double*)dx, rows, cols);
  } else if (dt == PRAD_F32) softmax_backward_kernel<float><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)y, (const float*)dy, (float*)dx, rows, cols);
  else softmax_backward_kernel<double><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const double*)y, (const double*)dy, (double*)dx, rows, cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_layernorm_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y,
                                   void* mean, void* stdv, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_layernorm_forward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && y && mean && stdv, PRAD_ERR_INVALID, "prad_layernorm_forward: null pointer");
  if (short_e(cols)) {
    if (dt == PRAD_F32) PRAD_SHORT_ROWS(layernorm_forward_short, float, (const float*)x, (float*)y, (float*)mean, (float*)stdv, rows, cols);
    else PRAD_SHORT_ROWS(layernorm_forward_short, double, (const double*)x, (double*)y, (double*)mean, (double*)stdv, rows, cols);
  } else if (dt == PRAD_F32) layernorm_forward_kernel<float><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)x, (float*)y, (float*)mean, (float*)stdv, rows, cols);
  else layernorm_forward_kernel<double><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const double*)x, (double*)y, (double*)mean, (double*)stdv, rows, cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_layernorm_backward(prad_ctx* ctx, prad_dtype dt, const void* x,
                                    const void* mean, const void* stdv, const void* dy, void* dx,
                                    int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_layernorm_backward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && mean && stdv && dy && dx, PRAD_ERR_INVALID, "prad_layernorm_backward: null pointer");
  const int vecn = dt == PRAD_F32 ? 4 : 2;
  if (cols % vecn == 0 && (((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dx) & 15) == 0) {
    const int64_t nvec = rows * (cols / vecn);
    const int grid = stream_grid(ctx, ceil_div(nvec, 4), 256, 8);
    if (dt == PRAD_F32) layernorm_backward_flat<float><<<grid, 256, 0, ctx->stream>>>((const float*)x, (const float*)mean, (const float*)stdv, (const float*)dy, (float*)dx, nvec, cols / vecn, cols);
    else layernorm_backward_flat<double><<<grid, 256, 0, ctx->stream>>>((const double*)x, (const double*)mean, (const double*)stdv, (const double*)dy, (double*)dx, nvec, cols / vecn, cols);
  } else if (short_e(cols)) {
    if (dt == PRAD_F32) PRAD_SHORT_ROWS(layernorm_backward_short, float, (const float*)x, (const float*)mean, (const float*)stdv, (const float*)dy, (float*)dx, rows, cols);
    else PRAD_SHORT_ROWS(layernorm_backward_short, double, (const double*)x, (const double*)mean, (const double*)stdv, (const double*)dy, (double*)dx, rows, cols);
  } else if (dt == PRAD_F32) layernorm_backward_kernel<float><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)x, (const float*)mean, (const float*)stdv, (const float*)dy, (float*)dx, rows, cols);
  else layernorm_backward_kernel<double><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const double*)x, (const double*)mean, (const double*)stdv, (const double*)dy, (double*)dx, rows, cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

#define PRAD_ROW_LAUNCH(KERNEL, ...)                                                                     \
  do {                                                                                                   \
    if (dt == PRAD_F32) KERNEL<float><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>(__VA_ARGS__(float)); \
    else KERNEL<double><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>(__VA_ARGS__(double));   \
    PRAD_LAUNCHED(ctx);                                                                                  \
  } while (0)

prad_status prad_scale_shift_forward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* beta,
                                     const void* gamma, void* y, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_scale_shift_forward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && beta && gamma && y, PRAD_ERR_INVALID, "prad_scale_shift_forward: null pointer");
#define ARGS(T) (const T*)x, (const T*)beta, (const T*)gamma, (T*)y, rows, cols
  PRAD_ROW_LAUNCH(scale_shift_forward_kernel, ARGS);
#undef ARGS
  return PRAD_OK;
}

prad_status prad_scale_shift_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* beta,
                                      const void* dy, void* dx, void* dbeta, void* dgamma,
                                      int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_scale_shift_backward: bad argument");
  if (rows == 0) return PRAD_OK;
  PRAD_REQUIRE(beta && dbeta && dgamma && (cols == 0 || (x && dy && dx)), PRAD_ERR_INVALID,
               "prad_scale_shift_backward: null pointer");
#define ARGS(T) (const T*)x, (const T*)beta, (const T*)dy, (T*)dx, (T*)dbeta, (T*)dgamma, rows, cols
  PRAD_ROW_LAUNCH(scale_shift_backward_kernel, ARGS);
#undef ARGS
  return PRAD_OK;
}

prad_status prad_rmsnorm_forward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* g, void* y,
                                 int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_rmsnorm_forward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && g && y, PRAD_ERR_INVALID, "prad_rmsnorm_forward: null pointer");
#define ARGS(T) (const T*)x, (const T*)g, (T*)y, rows, cols
  PRAD_ROW_LAUNCH(rmsnorm_forward_kernel, ARGS);
#undef ARGS
  return PRAD_OK;
}

prad_status prad_rmsnorm_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* g,
                                  const void* dy, void* dx, void* dg, int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_rmsnorm_backward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && g && dy && dx && dg, PRAD_ERR_INVALID, "prad_rmsnorm_backward: null pointer");
#define ARGS(T) (const T*)x, (const T*)g, (const T*)dy, (T*)dx, (T*)dg, rows, cols
  PRAD_ROW_LAUNCH(rmsnorm_backward_kernel, ARGS);
#undef ARGS
  return PRAD_OK;
}

prad_status prad_row_sum_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, int64_t rows, int cols,
                                 int average) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_row_sum_forward: bad argument");
  if (rows == 0) return PRAD_OK;
  PRAD_REQUIRE(y && (cols == 0 || x), PRAD_ERR_INVALID, "prad_row_sum_forward: null pointer");
  PRAD_REQUIRE(!(average && cols == 0), PRAD_ERR_INVALID, "prad_row_sum_forward: average of an empty row");
#define ARGS(T) (const T*)x, (T*)y, rows, cols, average
  PRAD_ROW_LAUNCH(row_sum_forward_kernel, ARGS);
#undef ARGS
  return PRAD_OK;
}

prad_status prad_row_sum_backward(prad_ctx* ctx, prad_dtype dt, const void* dy, void* dx, int64_t rows, int cols,
                                  int average) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_row_sum_backward: bad argument");
  const int64_t n = rows * cols;
  if (n == 0) return PRAD_OK;
  PRAD_REQUIRE(dy && dx, PRAD_ERR_INVALID, "prad_row_sum_backward: null pointer");
  const int grid = stream_grid(ctx, n, 256, 8);
  if (dt == PRAD_F32) row_sum_backward_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)dy, (float*)dx, n, cols, average);
  else row_sum_backward_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)dy, (double*)dx, n, cols, average);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_broadcast_forward(prad_ctx* ctx, prad_dtype dt, const void* x, int in_rows, int in_cols, void* y,
                                   int out_rows, int out_cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && in_rows >= 0 && in_cols >= 0 && out_rows >= 0 && out_cols >= 0, PRAD_ERR_INVALID,
               "prad_broadcast_forward: bad argument");
  const int64_t n = (int64_t)out_rows * out_cols;
  if (n == 0) return PRAD_OK;
  PRAD_REQUIRE(in_rows > 0 && in_cols > 0, PRAD_ERR_SHAPE, "prad_broadcast_forward: empty input for a non-empty target");
  PRAD_REQUIRE(x && y, PRAD_ERR_INVALID, "prad_broadcast_forward: null pointer");
  const int grid = stream_grid(ctx, n, 256, 8);
  if (dt == PRAD_F32) broadcast_forward_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)x, in_rows, in_cols, (float*)y, n, out_cols);
  else broadcast_forward_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)x, in_rows, in_cols, (double*)y, n, out_cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_broadcast_backward(prad_ctx* ctx, prad_dtype dt, const void* dy, int out_rows, int out_cols,
                                    void* dx, int in_rows, int in_cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && in_rows >= 0 && in_cols >= 0 && out_rows >= 0 && out_cols >= 0, PRAD_ERR_INVALID,
               "prad_broadcast_backward: bad argument");
  const int64_t n = (int64_t)in_rows * in_cols;
  if (n == 0) return PRAD_OK;
  PRAD_REQUIRE(dx && ((int64_t)out_rows * out_cols == 0 || dy), PRAD_ERR_INVALID, "prad_broadcast_backward: null pointer");
  const int grid = stream_grid(ctx, n, 256, 8);
  if (dt == PRAD_F32) broadcast_backward_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)dy, out_rows, out_cols, (float*)dx, in_rows, in_cols);
  else broadcast_backward_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)dy, out_rows, out_cols, (double*)dx, in_rows, in_cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

}  // extern "C"
