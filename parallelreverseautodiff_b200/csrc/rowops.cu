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

static inline int row_grid(const prad_ctx* ctx, int64_t rows) {
  return stream_grid(ctx, rows, ROW_WARPS, 8);
}

}  // namespace prad

using namespace prad;

extern "C" {

prad_status prad_softmax_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y,
                                 int64_t rows, int cols) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_softmax_forward: bad argument");
  if (rows == 0 || cols == 0) return PRAD_OK;
  PRAD_REQUIRE(x && y, PRAD_ERR_INVALID, "prad_softmax_forward: null pointer");
  if (dt == PRAD_F32) softmax_forward_kernel<float><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)x, (float*)y, rows, cols);
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
  if (dt == PRAD_F32) softmax_backward_kernel<float><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)y, (const float*)dy, (float*)dx, rows, cols);
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
  if (dt == PRAD_F32) layernorm_forward_kernel<float><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)x, (float*)y, (float*)mean, (float*)stdv, rows, cols);
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
  if (dt == PRAD_F32) layernorm_backward_kernel<float><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const float*)x, (const float*)mean, (const float*)stdv, (const float*)dy, (float*)dx, rows, cols);
  else layernorm_backward_kernel<double><<<row_grid(ctx, rows), ROW_WARPS * 32, 0, ctx->stream>>>((const double*)x, (const double*)mean, (const double*)stdv, (const double*)dy, (double*)dx, rows, cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

}  // extern "C"
