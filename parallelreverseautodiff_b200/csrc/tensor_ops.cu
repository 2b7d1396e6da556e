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

// ---- Tensor.Gather (Tensor.Common.cs:959-1090) / TensorReverse.GatherReverse (TensorReverse.Common.cs:
// 2358-2426).  The tensor is viewed as x[outer][axis_len][inner] (outer = product of the dimensions
// before the axis, inner = product of those after it); the `count` indices are values of the storage
// type, negative ones count from the end (i < 0 ? shape[axis] + (int)i : (int)i); the result is
// y[outer][count][inner].
template <typename T>
__device__ __forceinline__ int wrapped_index(T raw, int axis_len) {
  return raw < (T)0 ? axis_len + (int)raw : (int)raw;
}
template <typename T>
__global__ void __launch_bounds__(256)
tensor_gather_kernel(const T* __restrict__ x, const T* __restrict__ idx, T* __restrict__ y, int64_t outer,
                     int axis_len, int count, int64_t inner, int* __restrict__ bad) {
  const int64_t total = outer * count * inner, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t in = e % inner, oc = e / inner;
    const int c = (int)(oc % count);
    const int64_t o = oc / count;
    const int v = wrapped_index<T>(idx[c], axis_len);
    if (v < 0 || v >= axis_len) { atomicExch(bad, c + 1); continue; }   // the managed code throws ArgumentException
    y[e] = x[(o * axis_len + v) * inner + in];
  }
}
// wrapped indices as values of the storage type (input of the ordered scatter-add); out-of-range ones
// are reported and replaced by -1 - which the scatter kernel reports as well and skips
template <typename T>
__global__ void __launch_bounds__(256)
tensor_wrap_indices_kernel(const T* __restrict__ idx, T* __restrict__ out, int count, int axis_len) {
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < count; c += gridDim.x * blockDim.x) {
    const int v = wrapped_index<T>(idx[c], axis_len);
    out[c] = (v < 0 || v >= axis_len) ? (T)-1 : (T)v;
  }
}
// General form: one thread per element of the input gradient walks the index list in order, so every
// element receives its contributions in the order of the upstream gradient's flat index -- the order
// of a sequential loop (the managed Parallel.For + lock adds them in a thread-dependent order).
template <typename T>
__global__ void __launch_bounds__(256)
tensor_gather_reverse_kernel(const T* __restrict__ up, const T* __restrict__ idx, T* __restrict__ dx, int64_t outer,
                             int axis_len, int count, int64_t inner, int* __restrict__ bad) {
  const int64_t total = outer * axis_len * inner, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t in = e % inner, ov = e / inner;
    const int v = (int)(ov % axis_len);
    const int64_t o = ov / axis_len;
    T acc = (T)0;
    for (int c = 0; c < count; ++c) {
      const int w = wrapped_index<T>(idx[c], axis_len);
      if (w < 0 || w >= axis_len) { if (e == 0) atomicExch(bad, c + 1); continue; }
      if (w == v) acc = add_rn(acc, up[(o * count + c) * inner + in]);
    }
    dx[e] = acc;
  }
}

// ---- Tensor.Tile (Tensor.Common.cs:1096-1230) / TensorReverse.TileReverse (TensorReverse.Common.cs:
// 2713-2785 and the specialised cases :3278-3370) for 2-D tensors.
template <typename T>
__global__ void __launch_bounds__(256)
tensor_tile_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols, int mr, int mc) {
  const int64_t oc = (int64_t)cols * mc, total = (int64_t)rows * mr * oc, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t r = e / oc, c = e % oc;
    y[e] = x[(r % rows) * cols + (c % cols)];
  }
}
// dx[i][j] collects its copies in the order of the upstream gradient's flat index, starting from zero.
// mode 0: general rule grad[i % rows][j % cols] += up[i][j];
// mode 1: multiples = {m, 1}: the specialised routine reads rows i*m .. i*m + m - 1 of the upstream
//         gradient for row i (as written there; it equals the general rule only for a one-row tensor).
template <typename T>
__global__ void __launch_bounds__(256)
tensor_tile_reverse_kernel(const T* __restrict__ up, T* __restrict__ dx, int rows, int cols, int mr, int mc, int mode) {
  const int64_t total = (int64_t)rows * cols, stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t oc = (int64_t)cols * mc;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t i = e / cols, j = e % cols;
    T acc = (T)0;
    if (mode == 1) {
      for (int m = 0; m < mr; ++m) acc = add_rn(acc, up[(i * mr + m) * cols + j]);
    } else {
      for (int tr = 0; tr < mr; ++tr)
        for (int tc = 0; tc < mc; ++tc) acc = add_rn(acc, up[((int64_t)tr * rows + i) * oc + (int64_t)tc * cols + j]);
    }
    dx[e] = acc;
  }
}

static prad_status read_bad_index(prad_ctx* ctx, int* d_bad, const char* who, int axis_len) {
  PRAD_NOT_CAPTURING(ctx, who);   // the index check reads a flag back
  int h = 0;
  PRAD_CUDA(cudaMemcpyAsync(&h, d_bad, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  PRAD_REQUIRE(h == 0, PRAD_ERR_INVALID, "%s: index at position %d is out of bounds for an axis of size %d", who, h - 1,
               axis_len);
  return PRAD_OK;
}

}  // namespace prad

using namespace prad;

extern "C" {

prad_status prad_tensor_matmul(prad_ctx* ctx, prad_dtype dt, const void* A, int a_rows, int a_cols, const void* B,
                               int b_rows, int b_cols, double alpha, double beta, void* C) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_tensor_matmul: bad dtype");
  PRAD_REQUIRE(a_rows >= 0 && a_cols >= 0 && b_rows >= 0 && b_cols >= 0, PRAD_ERR_SHAPE, "prad_tensor_matmul: negative dimension");
  PRAD_REQUIRE(a_cols == b_rows, PRAD_ERR_SHAPE, "Incompatible shapes for matrix multiplication.");
  if (a_rows == 0 || b_cols == 0) return PRAD_OK;
  PRAD_REQUIRE(C && (a_cols == 0 || (A && B)), PRAD_ERR_INVALID, "prad_tensor_matmul: null pointer");
  GemmEpilogue e;
  return gemm_dispatch(ctx, dt, false, false, a_rows, b_cols, a_cols, alpha, A, a_cols, B, b_cols, beta, C, b_cols, 1, 0, 0,
                       0, e);
}

prad_status prad_tensor_matmul_reverse(prad_ctx* ctx, prad_dtype dt, const void* A, int a_rows, int a_cols,
                                       const void* B, int b_rows, int b_cols, const void* dC, void* dA, void* dB) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_tensor_matmul_reverse: bad dtype");
  PRAD_REQUIRE(a_rows >= 0 && a_cols >= 0 && b_rows >= 0 && b_cols >= 0, PRAD_ERR_SHAPE,
               "prad_tensor_matmul_reverse: negative dimension");
  PRAD_REQUIRE(a_cols == b_rows, PRAD_ERR_SHAPE, "Incompatible shapes for matrix multiplication.");
  const int m = a_rows, k = a_cols, n = b_cols;
  PRAD_REQUIRE(dC || m == 0 || n == 0, PRAD_ERR_INVALID, "prad_tensor_matmul_reverse: the upstream gradient is null");
  PRAD_REQUIRE((!dA || B || k == 0 || n == 0) && (!dB || A || k == 0 || m == 0), PRAD_ERR_INVALID,
               "prad_tensor_matmul_reverse: null operand");
  GemmEpilogue e;
  prad_status s = PRAD_OK;
  // dL/dA = dL/dC * B^T (gemm NoTrans, Trans) ; dL/dB = A^T * dL/dC (gemm Trans, NoTrans)
  if (dA && m && k) s = gemm_dispatch(ctx, dt, false, true, m, k, n, 1.0, dC, n, B, n, 0.0, dA, k, 1, 0, 0, 0, e);
  if (s) return s;
  if (dB && k && n) s = gemm_dispatch(ctx, dt, true, false, k, n, m, 1.0, A, k, dC, n, 0.0, dB, n, 1, 0, 0, 0, e);
  return s;
}

prad_status prad_tensor_gather(prad_ctx* ctx, prad_dtype dt, const void* x, int64_t outer, int axis_len, int64_t inner,
                               const void* indices, int count, void* y) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && outer >= 0 && axis_len >= 0 && inner >= 0 && count >= 0, PRAD_ERR_INVALID,
               "prad_tensor_gather: bad dtype or negative size");
  if (outer * count * inner == 0) return PRAD_OK;
  PRAD_REQUIRE(x && indices && y, PRAD_ERR_INVALID, "prad_tensor_gather: null pointer");
  prad_status s = ensure_workspace(ctx, 256);
  if (s) return s;
  int* bad = (int*)ctx->ws;
  PRAD_CUDA(cudaMemsetAsync(bad, 0, sizeof(int), ctx->stream));
  const int grid = stream_grid(ctx, outer * count * inner, 256, 8);
  if (dt == PRAD_F32) tensor_gather_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)x, (const float*)indices, (float*)y, outer, axis_len, count, inner, bad);
  else tensor_gather_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)x, (const double*)indices, (double*)y, outer, axis_len, count, inner, bad);
  PRAD_LAUNCHED(ctx);
  return read_bad_index(ctx, bad, "prad_tensor_gather", axis_len);
}

prad_status prad_tensor_gather_reverse(prad_ctx* ctx, prad_dtype dt, const void* upstream, int64_t outer, int axis_len,
                                       int64_t inner, const void* indices, int count, void* dx) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && outer >= 0 && axis_len >= 0 && inner >= 0 && count >= 0, PRAD_ERR_INVALID,
               "prad_tensor_gather_reverse: bad dtype or negative size");
  if (outer * axis_len * inner == 0) return PRAD_OK;
  PRAD_REQUIRE(dx && (count == 0 || (upstream && indices)), PRAD_ERR_INVALID, "prad_tensor_gather_reverse: null pointer");
  const size_t es = dtype_size(dt);
  prad_status s = ensure_workspace(ctx, 256 + (size_t)count * es);
  if (s) return s;
  int* bad = (int*)ctx->ws;
  PRAD_CUDA(cudaMemsetAsync(bad, 0, sizeof(int), ctx->stream));
  const bool rows_form = outer <= 64 && inner <= INT32_MAX && (int64_t)count * axis_len > 4096;
  if (rows_form) {
    // large tables: wrap the indices once, then the ordered row scatter-add per outer slice
    void* wrapped = (char*)ctx->ws + 256;
    const int g = stream_grid(ctx, count, 256, 8);
    if (dt == PRAD_F32) tensor_wrap_indices_kernel<float><<<g, 256, 0, ctx->stream>>>((const float*)indices, (float*)wrapped, count, axis_len);
    else tensor_wrap_indices_kernel<double><<<g, 256, 0, ctx->stream>>>((const double*)indices, (double*)wrapped, count, axis_len);
    PRAD_LAUNCHED(ctx);
    for (int64_t o = 0; o < outer; ++o) {
      s = embedding_scatter_ordered(ctx, dt, wrapped, (const char*)upstream + (size_t)o * count * inner * es,
                                    (char*)dx + (size_t)o * axis_len * inner * es, count, axis_len, (int)inner, bad);
      if (s) return s;
    }
  } else {
    const int grid = stream_grid(ctx, outer * axis_len * inner, 256, 8);
    if (dt == PRAD_F32) tensor_gather_reverse_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)upstream, (const float*)indices, (float*)dx, outer, axis_len, count, inner, bad);
    else tensor_gather_reverse_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)upstream, (const double*)indices, (double*)dx, outer, axis_len, count, inner, bad);
    PRAD_LAUNCHED(ctx);
  }
  return read_bad_index(ctx, bad, "prad_tensor_gather_reverse", axis_len);
}

prad_status prad_tensor_tile(prad_ctx* ctx, prad_dtype dt, const void* x, int rows, int cols, int mult_rows, int mult_cols,
                             void* y) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_tensor_tile: bad dtype or negative size");
  PRAD_REQUIRE(mult_rows > 0 && mult_cols > 0, PRAD_ERR_INVALID,
               "Invalid multiples: Must match tensor dimensions and all values must be positive.");
  const int64_t total = (int64_t)rows * mult_rows * cols * mult_cols;
  if (total == 0) return PRAD_OK;
  PRAD_REQUIRE(x && y, PRAD_ERR_INVALID, "prad_tensor_tile: null pointer");
  const int grid = stream_grid(ctx, total, 256, 8);
  if (dt == PRAD_F32) tensor_tile_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)x, (float*)y, rows, cols, mult_rows, mult_cols);
  else tensor_tile_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)x, (double*)y, rows, cols, mult_rows, mult_cols);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

prad_status prad_tensor_tile_reverse(prad_ctx* ctx, prad_dtype dt, const void* upstream, int rows, int cols, int mult_rows,
                                     int mult_cols, void* dx) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && rows >= 0 && cols >= 0, PRAD_ERR_INVALID, "prad_tensor_tile_reverse: bad dtype or negative size");
  PRAD_REQUIRE(mult_rows > 0 && mult_cols > 0, PRAD_ERR_INVALID, "prad_tensor_tile_reverse: multiples must be positive");
  const int64_t total = (int64_t)rows * cols;
  if (total == 0) return PRAD_OK;
  PRAD_REQUIRE(upstream && dx, PRAD_ERR_INVALID, "prad_tensor_tile_reverse: null pointer");
  const int mode = mult_cols == 1 ? 1 : 0;   // {m, 1} takes the specialised routine first (TensorReverse.Common.cs:2736-2739)
  const int grid = stream_grid(ctx, total, 256, 8);
  if (dt == PRAD_F32) tensor_tile_reverse_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)upstream, (float*)dx, rows, cols, mult_rows, mult_cols, mode);
  else tensor_tile_reverse_kernel<double><<<grid, 256, 0, ctx->stream>>>((const double*)upstream, (double*)dx, rows, cols, mult_rows, mult_cols, mode);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

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
