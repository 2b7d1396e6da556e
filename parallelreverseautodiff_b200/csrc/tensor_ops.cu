// Elementwise operations of the reference's second public API (PRAD `Tensor` / `TensorReverse`,
// src/PRAD/Tensor.Common.cs and TensorReverse.Common.cs), which evaluates them with MKL VML
// calls over flat arrays: one rounding per VML call, in the storage type.  The kernels below
// follow the same sequence of roundings (compiled with -fmad=false); the transcendental
// functions are CUDA's, which agree with VML's high-accuracy mode to about an ulp.
#include "act_math.cuh"
#include "common.cuh"

namespace prad {

template <typename T> struct TensorEps;
template <> struct TensorEps<float> { __device__ static float v() { return 1e-10f; } };    // PradTools.Epsilon10
template <> struct TensorEps<double> { __device__ static double v() { return 1e-10; } };

__device__ __forceinline__ float t_sin(float x) { return sinf(x); }
__device__ __forceinline__ double t_sin(double x) { return sin(x); }
__device__ __forceinline__ float t_cos(float x) { return cosf(x); }
__device__ __forceinline__ double t_cos(double x) { return cos(x); }
__device__ __forceinline__ float t_log10(float x) { return log10f(x); }
__device__ __forceinline__ double t_log10(double x) { return log10(x); }

// Tensor.Common.cs: Exp :814, Ln :825, Log (Vml.Log10) :836, Abs :788, ElementwiseSquare :1705,
// ElementwiseSquareRoot :1716, ElementwiseSin :1727, ElementwiseCos :1738, Reciprocal :737,
// ElementwiseNegate :2672
template <typename T> __device__ __forceinline__ T tensor_unary(int op, T x) {
  switch (op) {
    case PRAD_TENSOR_EXP: return t_exp(x);
    case PRAD_TENSOR_LN: return t_log(x);
    case PRAD_TENSOR_LOG10: return t_log10(x);
    case PRAD_TENSOR_ABS: return x < (T)0 ? -x : x;
    case PRAD_TENSOR_SQUARE: return mul_rn(x, x);
    case PRAD_TENSOR_SQRT: return sqrt_rn(x);
    case PRAD_TENSOR_SIN: return t_sin(x);
    case PRAD_TENSOR_COS: return t_cos(x);
    case PRAD_TENSOR_RECIPROCAL: return div_rn((T)1, x);
    default: return mul_rn(x, (T)-1);   // PRAD_TENSOR_NEGATE
  }
}

// TensorReverse.Common.cs: ExpReverse :657, LnReverse :637, LogReverse :548 (1/x, as written, also
// for the base-10 logarithm), AbsReverse :127, ElementwiseSquareReverse :1232,
// ElementwiseSquareRootReverse :1505 (0.5 * dy / maxmag(sqrt x, 1e-10)), ElementwiseSinReverse :1799,
// ElementwiseCosReverse :1823, ReciprocalReverse :2128 (reads the RESULT 1/x);
// `s` is the input x, except for the reciprocal where it is the forward result.
template <typename T> __device__ __forceinline__ T tensor_unary_reverse(int op, T s, T dy) {
  switch (op) {
    case PRAD_TENSOR_EXP: return mul_rn(t_exp(s), dy);
    case PRAD_TENSOR_LN:
    case PRAD_TENSOR_LOG10: return mul_rn(div_rn((T)1, s), dy);
    case PRAD_TENSOR_ABS: return s >= (T)0 ? dy : -dy;
    case PRAD_TENSOR_SQUARE: return mul_rn((T)2, mul_rn(dy, s));
    case PRAD_TENSOR_SQRT: {
      const T r = sqrt_rn(s), e = TensorEps<T>::v();
      const T m = fabs((double)r) >= fabs((double)e) ? r : e;     // Vml.MaxMag
      return mul_rn((T)0.5, div_rn(dy, m));
    }
    case PRAD_TENSOR_SIN: return mul_rn(dy, t_cos(s));
    case PRAD_TENSOR_COS: return mul_rn((T)-1, mul_rn(dy, t_sin(s)));
    case PRAD_TENSOR_RECIPROCAL: return mul_rn(mul_rn(dy, mul_rn(s, s)), (T)-1);
    default: return mul_rn(dy, (T)-1);   // negate
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
tensor_unary_kernel(int op, const T* x, T* y, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = tensor_unary<T>(op, x[i]);
}
template <typename T>
__global__ void __launch_bounds__(256)
tensor_unary_reverse_kernel(int op, const T* s, const T* dy, T* dx, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dx[i] = tensor_unary_reverse<T>(op, s[i], dy[i]);
}
// ElementwiseAdd :1391, ElementwiseSub :1583, ElementwiseMultiply :1596, ElementwiseDivide :1693
template <typename T>
__global__ void __launch_bounds__(256)
tensor_binary_kernel(int op, const T* a, const T* b, T* y, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const T u = a[i], v = b[i];
    y[i] = op == PRAD_TENSOR_ADD ? add_rn(u, v) : op == PRAD_TENSOR_SUB ? sub_rn(u, v)
           : op == PRAD_TENSOR_MUL ? mul_rn(u, v) : div_rn(u, v);
  }
}
// ElementwiseAddReverse :102, ElementwiseSubReverse :2433, ElementwiseMultiplyReverse :844,
// ElementwiseDivideReverse :2543 (dB = -((dy * a) / (b * b)))
template <typename T>
__global__ void __launch_bounds__(256)
tensor_binary_reverse_kernel(int op, const T* a, const T* b, const T* dy, T* da, T* db, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const T d = dy[i];
    T ga, gb;
    if (op == PRAD_TENSOR_ADD) { ga = d; gb = d; }
    else if (op == PRAD_TENSOR_SUB) { ga = d; gb = mul_rn((T)-1, d); }
    else if (op == PRAD_TENSOR_MUL) { ga = mul_rn(d, b[i]); gb = mul_rn(d, a[i]); }
    else { const T v = b[i]; ga = div_rn(d, v); gb = mul_rn((T)-1, div_rn(mul_rn(d, a[i]), mul_rn(v, v))); }
    if (da) da[i] = ga;
    if (db) db[i] = gb;
  }
}

}  // namespace prad

using namespace prad;

extern "C" {

prad_status prad_tensor_unary(prad_ctx* ctx, prad_dtype dt, prad_tensor_op op, const void* x, void* y, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && op >= PRAD_TENSOR_EXP && op <= PRAD_TENSOR_NEGATE && n >= 0 && (n == 0 || (x && y)),
               PRAD_ERR_INVALID, "prad_tensor_unary: bad dtype, operation, pointer or size");
  if (n == 0) return PRAD_OK;
  const int grid = stream_grid(ctx, n, 256, 8);
  if (dt == PRAD_F32) tensor_unary_kernel<float><<<grid, 256, 0, ctx->stream>>>((int)op, (const float*)x, (float*)y, n);
  else tensor_unary_kernel<double><<<grid, 256, 0, ctx->stream>>>((int)op, (const double*)x, (double*)y, n);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_tensor_unary_reverse(prad_ctx* ctx, prad_dtype dt, prad_tensor_op op, const void* saved,
                                      const void* dy, void* dx, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && op >= PRAD_TENSOR_EXP && op <= PRAD_TENSOR_NEGATE && n >= 0 &&
                   (n == 0 || (saved && dy && dx)),
               PRAD_ERR_INVALID, "prad_tensor_unary_reverse: bad dtype, operation, pointer or size");
  if (n == 0) return PRAD_OK;
  const int grid = stream_grid(ctx, n, 256, 8);
  if (dt == PRAD_F32) tensor_unary_reverse_kernel<float><<<grid, 256, 0, ctx->stream>>>((int)op, (const float*)saved, (const float*)dy, (float*)dx, n);
  else tensor_unary_reverse_kernel<double><<<grid, 256, 0, ctx->stream>>>((int)op, (const double*)saved, (const double*)dy, (double*)dx, n);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_tensor_binary(prad_ctx* ctx, prad_dtype dt, prad_tensor_op op, const void* a, const void* b, void* y,
                               int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && op >= PRAD_TENSOR_ADD && op <= PRAD_TENSOR_DIV && n >= 0 && (n == 0 || (a && b && y)),
               PRAD_ERR_INVALID, "prad_tensor_binary: bad dtype, operation, pointer or size");
  if (n == 0) return PRAD_OK;
  const int grid = stream_grid(ctx, n, 256, 8);
  if (dt == PRAD_F32) tensor_binary_kernel<float><<<grid, 256, 0, ctx->stream>>>((int)op, (const float*)a, (const float*)b, (float*)y, n);
  else tensor_binary_kernel<double><<<grid, 256, 0, ctx->stream>>>((int)op, (const double*)a, (const double*)b, (double*)y, n);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_tensor_binary_reverse(prad_ctx* ctx, prad_dtype dt, prad_tensor_op op, const void* a, const void* b,
                                       const void* dy, void* da, void* db, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && op >= PRAD_TENSOR_ADD && op <= PRAD_TENSOR_DIV && n >= 0, PRAD_ERR_INVALID,
               "prad_tensor_binary_reverse: bad dtype, operation or size");
  if (n == 0) return PRAD_OK;
  const bool needs_inputs = op == PRAD_TENSOR_MUL || op == PRAD_TENSOR_DIV;
  PRAD_REQUIRE(dy && (da || db) && (!needs_inputs || (a && b)), PRAD_ERR_INVALID, "prad_tensor_binary_reverse: null pointer");
  const int grid = stream_grid(ctx, n, 256, 8);
  if (dt == PRAD_F32) tensor_binary_reverse_kernel<float><<<grid, 256, 0, ctx->stream>>>((int)op, (const float*)a, (const float*)b, (const float*)dy, (float*)da, (float*)db, n);
  else tensor_binary_reverse_kernel<double><<<grid, 256, 0, ctx->stream>>>((int)op, (const double*)a, (const double*)b, (const double*)dy, (double*)da, (double*)db, n);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

}  // extern "C"
