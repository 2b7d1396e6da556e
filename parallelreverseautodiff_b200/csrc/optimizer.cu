// Gradient clip and Adam update as multi-tensor kernels: one launch walks every model
// element (weight / gradient / first moment / second moment quadruple) through a table
// passed by value.  HBM-bound streams; all reductions are two-stage and order-fixed, so
// results are bit-reproducible.  (Compiled with -fmad=false.)
#include <cmath>

#include "act_math.cuh"
#include "common.cuh"
#include "reduce.cuh"

namespace prad {

constexpr int MT_MAX = 48;          // tensors per launch (table is a kernel argument)
constexpr int MT_THREADS = 256;
constexpr int MT_CHUNK = 256 * 32;  // elements a CTA covers

template <typename T> struct MtVec;
template <> struct MtVec<float> { using type = float4; };
template <> struct MtVec<double> { using type = double2; };

struct MultiTensor {
  bool vec;   // every pointer of every tensor is 16-byte aligned
  void* w[MT_MAX];
  void* g[MT_MAX];
  void* m[MT_MAX];
  void* v[MT_MAX];
  int64_t size[MT_MAX];
  int blk_start[MT_MAX + 1];
  int count;
};

__device__ __forceinline__ int find_tensor(const MultiTensor& t, int blk) {
  int lo = 0, hi = t.count - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (t.blk_start[mid] <= blk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// stats layout in the workspace (doubles): [0,MT_MAX) mean, [MT_MAX,2*MT_MAX) std,
// [2*MT_MAX] global sum of squares, then the per-CTA partials.
constexpr int ST_MEAN = 0, ST_STD = MT_MAX, ST_SS = 2 * MT_MAX, ST_PART = 2 * MT_MAX + 8;

// pass kinds: 0 = sum g ; 1 = sum (g-mean)^2 (T arithmetic for the square, as Pow(v-mean,2)
// rounds to T in the float build) ; 2 = sum g^2 in double (global norm)
template <typename T>
__global__ void __launch_bounds__(MT_THREADS)
mt_partial_kernel(MultiTensor t, double* __restrict__ stats, int kind) {
  const int ti = find_tensor(t, blockIdx.x);
  const int64_t start = (int64_t)(blockIdx.x - t.blk_start[ti]) * MT_CHUNK;
  int64_t end = start + MT_CHUNK;
  if (end > t.size[ti]) end = t.size[ti];
  const T* g = (const T*)t.g[ti];
  const T mean = kind == 1 ? (T)stats[ST_MEAN + ti] : (T)0;
  double acc = 0.0;
  auto term = [&](T x) {
    if (kind == 0) acc += (double)x;
    else if (kind == 1) { T d = sub_rn(x, mean); acc += (double)mul_rn(d, d); }
    else acc += (double)x * (double)x;
  };
  int64_t i0 = start;
  if (t.vec) {    // 128-bit loads; chunk starts are multiples of the vector width
    constexpr int VEC = 16 / sizeof(T);
    using V = typename MtVec<T>::type;
    const int64_t vend = end - ((end - start) % VEC);
    for (int64_t i = start + (int64_t)threadIdx.x * VEC; i < vend; i += MT_THREADS * VEC) {
      V v = *reinterpret_cast<const V*>(g + i);
#pragma unroll
      for (int q = 0; q < VEC; ++q) term(reinterpret_cast<const T*>(&v)[q]);
    }
    i0 = vend;
  }
  for (int64_t i = i0 + threadIdx.x; i < end; i += MT_THREADS) term(g[i]);
  double s = block_sum_d<MT_THREADS>(acc);
  if (threadIdx.x == 0) stats[ST_PART + blockIdx.x] = s;
}

// one CTA per tensor adds that tensor's partials in CTA order (fixed tree)
template <typename T>
__global__ void __launch_bounds__(MT_THREADS)
mt_finalize_kernel(MultiTensor t, double* __restrict__ stats, int kind) {
  const int ti = blockIdx.x;
  double acc = 0.0;
  for (int b = t.blk_start[ti] + threadIdx.x; b < t.blk_start[ti + 1]; b += MT_THREADS)
    acc += stats[ST_PART + b];
  double s = block_sum_d<MT_THREADS>(acc);
  if (threadIdx.x == 0) {
    const T n = (T)t.size[ti];
    if (kind == 0) stats[ST_MEAN + ti] = (double)div_rn((T)s, n);           // mean = sum / count
    else stats[ST_STD + ti] = (double)sqrt_rn(div_rn((T)s, n));             // Sqrt(varianceSum / count)
  }
}
// global norm: every partial of every tensor, one CTA
__global__ void __launch_bounds__(MT_THREADS)
mt_finalize_ss_kernel(int nblocks, double* __restrict__ stats, int add_to_existing) {
  double acc = 0.0;
  for (int b = threadIdx.x; b < nblocks; b += MT_THREADS) acc += stats[ST_PART + b];
  double s = block_sum_d<MT_THREADS>(acc);
  if (threadIdx.x == 0) stats[ST_SS] = (add_to_existing ? stats[ST_SS] : 0.0) + s;
}

// .NET Math.Min propagates NaN (a zero-variance tensor gives z = 0/0)
template <typename T> __device__ __forceinline__ T net_min(T a, T b) {
  if (isnan(a) || isnan(b)) return (T)NAN;
  return a < b ? a : b;
}

// GradientClipper.cs:129-153 on one value
template <typename T>
__device__ __forceinline__ T clip_reference_value(T gi, T mean, T sd, T clip, T minv) {
  T z = div_rn(sub_rn(gi, mean), sd);
  T lim = net_min<T>(clip, add_rn((T)1, fabs(z)));
  T v = gi;
  if (v > lim) v = lim;
  else if (v < -lim) v = -lim;
  if (v > (T)0 && v < minv) v = minv;
  else if (v < (T)0 && v > -minv) v = -minv;
  return v;
}

template <typename T> struct AdamScalars {
  T lr, b1, b2, eps, omb1, omb2, c1, c2;  // c1/c2: reciprocal (RMAD) or divisor (PRAD) bias terms
  int form;
};

// AdamOptimizer.cs:195-239 (RMAD) / src/PRAD/AdamOptimizer.cs:79-103 (PRAD) on one element
template <typename T>
__device__ __forceinline__ void adam_value(const AdamScalars<T>& a, T g, T& w, T& m, T& v) {
  if (a.form == PRAD_ADAM_RMAD) {
    T fm = add_rn(mul_rn(a.b1, m), mul_rn(a.omb1, g));
    T sm = add_rn(mul_rn(a.b2, v), mul_rn(a.omb2, mul_rn(g, g)));
    T mh = mul_rn(a.c1, fm);
    T vh = mul_rn(a.c2, sm);
    T upd = div_rn(mul_rn(a.lr, mh), add_rn(sqrt_rn(vh), a.eps));
    w = sub_rn(w, upd);
    m = fm;
    v = sm;
  } else {
    T fm = add_rn(mul_rn(m, a.b1), mul_rn(g, a.omb1));
    T sm = add_rn(mul_rn(v, a.b2), mul_rn(mul_rn(g, g), a.omb2));
    T mh = div_rn(fm, a.c1);
    T vh = div_rn(sm, a.c2);
    T upd = div_rn(mul_rn(mh, a.lr), add_rn(sqrt_rn(vh), a.eps));
    w = sub_rn(w, upd);
    m = fm;
    v = sm;
  }
}

// The streaming pass.  clip_mode 0 none / 1 reference / 2 global norm (scale from stats);
// do_adam 0 = clip only (writes g), 1 = also update w, m, v; zero_grad clears g afterwards.
template <typename T>
__global__ void __launch_bounds__(MT_THREADS)
mt_apply_kernel(MultiTensor t, const double* __restrict__ stats, int clip_mode, T clip, T minv,
                double max_norm, int do_adam, AdamScalars<T> a, int zero_grad, const int* __restrict__ gemm_gave_up) {
  // A tensor-core product on this context ran out of a bounded wait: the gradients on the stream are
  // not valid, so weights, moments and gradients are left exactly as they are (one load per CTA; the
  // host learns of it at its next prad_sync / prad_download, which returns PRAD_ERR_TIMEOUT).
  if (gemm_gave_up && *gemm_gave_up != 0) return;
  const int ti = find_tensor(t, blockIdx.x);
  const int64_t start = (int64_t)(blockIdx.x - t.blk_start[ti]) * MT_CHUNK;
  int64_t end = start + MT_CHUNK;
  if (end > t.size[ti]) end = t.size[ti];
  T* g = (T*)t.g[ti];
  T* w = (T*)t.w[ti];
  T* m = (T*)t.m[ti];
  T* v = (T*)t.v[ti];
  T mean = 0, sd = 1, gscale = 1;
  bool scale_on = false;
  if (clip_mode == 1) { mean = (T)stats[ST_MEAN + ti]; sd = (T)stats[ST_STD + ti]; }
  if (clip_mode == 2) {
    double norm = sqrt(stats[ST_SS]);
    if (norm > max_norm) { gscale = (T)(max_norm / norm); scale_on = true; }
  }
  auto clip_one = [&](T gi) {
    if (clip_mode == 1) return clip_reference_value<T>(gi, mean, sd, clip, minv);
    if (scale_on) return mul_rn(gi, gscale);
    return gi;
  };
  int64_t i0 = start;
  if (t.vec) {
    constexpr int VEC = 16 / sizeof(T);
    using V = typename MtVec<T>::type;
    const int64_t vend = end - ((end - start) % VEC);
    for (int64_t i = start + (int64_t)threadIdx.x * VEC; i < vend; i += MT_THREADS * VEC) {
      V gv = *reinterpret_cast<const V*>(g + i);
      V wv, mv, vv;
      if (do_adam) {
        wv = *reinterpret_cast<const V*>(w + i);
        mv = *reinterpret_cast<const V*>(m + i);
        vv = *reinterpret_cast<const V*>(v + i);
      }
#pragma unroll
      for (int q = 0; q < VEC; ++q) {
        T gi = clip_one(reinterpret_cast<T*>(&gv)[q]);
        if (do_adam)
          adam_value<T>(a, gi, reinterpret_cast<T*>(&wv)[q], reinterpret_cast<T*>(&mv)[q], reinterpret_cast<T*>(&vv)[q]);
        reinterpret_cast<T*>(&gv)[q] = zero_grad ? (T)0 : gi;
      }
      if (do_adam) {
        *reinterpret_cast<V*>(w + i) = wv;
        *reinterpret_cast<V*>(m + i) = mv;
        *reinterpret_cast<V*>(v + i) = vv;
      }
      if (zero_grad || clip_mode != 0) *reinterpret_cast<V*>(g + i) = gv;
    }
    i0 = vend;
  }
  for (int64_t i = i0 + threadIdx.x; i < end; i += MT_THREADS) {
    T gi = clip_one(g[i]);
    if (do_adam) {
      T wi = w[i], mi = m[i], vi = v[i];
      adam_value<T>(a, gi, wi, mi, vi);
      w[i] = wi; m[i] = mi; v[i] = vi;
    }
    if (zero_grad) g[i] = (T)0;
    else if (clip_mode != 0) g[i] = gi;
  }
}

template <typename T>
static AdamScalars<T> adam_scalars(double lr, double b1, double b2, double eps, double iteration,
                                   prad_adam_form form) {
  AdamScalars<T> a;
  a.lr = (T)lr; a.b1 = (T)b1; a.b2 = (T)b2; a.eps = (T)eps;
  a.omb1 = (T)1 - a.b1;
  a.omb2 = (T)1 - a.b2;
  // PradMath.Pow(beta, iteration): computed in double, cast to T
  T p1 = (T)std::pow((double)a.b1, (double)(T)iteration);
  T p2 = (T)std::pow((double)a.b2, (double)(T)iteration);
  if (form == PRAD_ADAM_RMAD) {
    a.c1 = (T)1 / ((T)1 - p1);
    a.c2 = (T)1 / ((T)1 - p2);
  } else {
    a.c1 = (T)1 - p1;
    a.c2 = (T)1 - p2;
  }
  a.form = (int)form;
  return a;
}

// builds the table for tensors [first, first+cnt) ; returns the CTA count
static int build_table(MultiTensor& t, void* const* w, void* const* g, void* const* m,
                       void* const* v, const int64_t* sizes, int first, int cnt) {
  int blk = 0;
  t.count = cnt;
  t.vec = true;
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  for (int k = 0; k < cnt; ++k) {
    t.vec = t.vec && al(w ? w[first + k] : nullptr) && al(g ? g[first + k] : nullptr) &&
            al(m ? m[first + k] : nullptr) && al(v ? v[first + k] : nullptr);
    t.w[k] = w ? w[first + k] : nullptr;
    t.g[k] = g ? g[first + k] : nullptr;
    t.m[k] = m ? m[first + k] : nullptr;
    t.v[k] = v ? v[first + k] : nullptr;
    t.size[k] = sizes[first + k];
    t.blk_start[k] = blk;
    int64_t nb = ceil_div(sizes[first + k], MT_CHUNK);
    blk += (int)(nb < 1 ? 1 : nb);
  }
  t.blk_start[cnt] = blk;
  return blk;
}

template <typename T>
static prad_status clip_adam_t(prad_ctx* ctx, void* const* w, void* const* g, void* const* m,
                               void* const* v, const int64_t* sizes, int count, int clip_mode,
                               double clip_value, double min_value, int do_adam, double lr,
                               double b1, double b2, double eps, double iteration,
                               prad_adam_form form, int zero_grad, double* norm_out) {
  AdamScalars<T> a = adam_scalars<T>(lr, b1, b2, eps, iteration, form);
  // workspace: stats header + partials of the largest group
  int max_blocks = 0;
  MultiTensor t;
  for (int first = 0; first < count; first += MT_MAX) {
    int cnt = count - first < MT_MAX ? count - first : MT_MAX;
    int nb = build_table(t, w, g, m, v, sizes, first, cnt);
    if (nb > max_blocks) max_blocks = nb;
  }
  prad_status s = ensure_workspace(ctx, (size_t)(ST_PART + max_blocks) * sizeof(double));
  if (s) return s;
  double* stats = (double*)ctx->ws;

  if (clip_mode == 2) {  // the norm spans every tensor: first all partial sums, then apply
    for (int first = 0; first < count; first += MT_MAX) {
      int cnt = count - first < MT_MAX ? count - first : MT_MAX;
      int nb = build_table(t, w, g, m, v, sizes, first, cnt);
      mt_partial_kernel<T><<<nb, MT_THREADS, 0, ctx->stream>>>(t, stats, 2);
      PRAD_LAUNCHED(ctx);
      mt_finalize_ss_kernel<<<1, MT_THREADS, 0, ctx->stream>>>(nb, stats, first > 0);
      PRAD_LAUNCHED(ctx);
    }
  }
  for (int first = 0; first < count; first += MT_MAX) {
    int cnt = count - first < MT_MAX ? count - first : MT_MAX;
    int nb = build_table(t, w, g, m, v, sizes, first, cnt);
    if (clip_mode == 1) {
      mt_partial_kernel<T><<<nb, MT_THREADS, 0, ctx->stream>>>(t, stats, 0);
      PRAD_LAUNCHED(ctx);
      mt_finalize_kernel<T><<<cnt, MT_THREADS, 0, ctx->stream>>>(t, stats, 0);
      PRAD_LAUNCHED(ctx);
      mt_partial_kernel<T><<<nb, MT_THREADS, 0, ctx->stream>>>(t, stats, 1);
      PRAD_LAUNCHED(ctx);
      mt_finalize_kernel<T><<<cnt, MT_THREADS, 0, ctx->stream>>>(t, stats, 1);
      PRAD_LAUNCHED(ctx);
    }
    mt_apply_kernel<T><<<nb, MT_THREADS, 0, ctx->stream>>>(t, stats, clip_mode, (T)clip_value,
                                                           (T)min_value, clip_value, do_adam, a,
                                                           zero_grad, ctx->tc_err);
    PRAD_LAUNCHED(ctx);
  }
  if (norm_out) {
    PRAD_NOT_CAPTURING(ctx, "a clip call that returns the norm to the host");
    double ss = 0.0;
    PRAD_CUDA(cudaMemcpyAsync(&ss, stats + ST_SS, sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
    PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
    *norm_out = std::sqrt(ss);
  }
  return PRAD_OK;
}

static prad_status check_lists(const char* who, void* const* const* lists, int nlists,
                               const int64_t* sizes, int count) {
  PRAD_REQUIRE(count >= 0 && (count == 0 || sizes), PRAD_ERR_INVALID, "%s: bad tensor count or null sizes", who);
  for (int l = 0; l < nlists; ++l) {
    PRAD_REQUIRE(count == 0 || lists[l], PRAD_ERR_INVALID, "%s: null pointer list", who);
    for (int i = 0; i < count; ++i) {
      PRAD_REQUIRE(sizes[i] >= 0, PRAD_ERR_INVALID, "%s: tensor %d has a negative size", who, i);
      PRAD_REQUIRE(lists[l][i] || sizes[i] == 0, PRAD_ERR_INVALID, "%s: tensor %d is null", who, i);
    }
  }
  return PRAD_OK;
}

}  // namespace prad

using namespace prad;

extern "C" {

prad_status prad_clip_reference(prad_ctx* ctx, prad_dtype dt, void* const* grads_host,
                                const int64_t* sizes_host, int count, double clip_value,
                                double min_value) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt), PRAD_ERR_INVALID, "prad_clip_reference: bad dtype");
  void* const* lists[1] = {grads_host};
  prad_status s = check_lists("prad_clip_reference", lists, 1, sizes_host, count);
  if (s || count == 0) return s;
  return dt == PRAD_F32
             ? clip_adam_t<float>(ctx, nullptr, grads_host, nullptr, nullptr, sizes_host, count, 1, clip_value, min_value, 0, 0, 0, 0, 0, 1, PRAD_ADAM_RMAD, 0, nullptr)
             : clip_adam_t<double>(ctx, nullptr, grads_host, nullptr, nullptr, sizes_host, count, 1, clip_value, min_value, 0, 0, 0, 0, 0, 1, PRAD_ADAM_RMAD, 0, nullptr);
}

prad_status prad_clip_global_norm(prad_ctx* ctx, prad_dtype dt, void* const* grads_host,
                                  const int64_t* sizes_host, int count, double max_norm,
                                  double* norm_out) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && max_norm > 0, PRAD_ERR_INVALID, "prad_clip_global_norm: bad dtype or max_norm");
  void* const* lists[1] = {grads_host};
  prad_status s = check_lists("prad_clip_global_norm", lists, 1, sizes_host, count);
  if (s) return s;
  if (count == 0) { if (norm_out) *norm_out = 0.0; return PRAD_OK; }
  return dt == PRAD_F32
             ? clip_adam_t<float>(ctx, nullptr, grads_host, nullptr, nullptr, sizes_host, count, 2, max_norm, 0, 0, 0, 0, 0, 0, 1, PRAD_ADAM_RMAD, 0, norm_out)
             : clip_adam_t<double>(ctx, nullptr, grads_host, nullptr, nullptr, sizes_host, count, 2, max_norm, 0, 0, 0, 0, 0, 0, 1, PRAD_ADAM_RMAD, 0, norm_out);
}

prad_status prad_clip_adam(prad_ctx* ctx, prad_dtype dt, void* const* w_host,
                           void* const* g_host, void* const* m_host, void* const* v_host,
                           const int64_t* sizes_host, int count, int clip_mode,
                           double clip_value, double min_value, double lr, double beta1,
                           double beta2, double eps, double iteration, prad_adam_form form,
                           int zero_grad) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && clip_mode >= 0 && clip_mode <= 2 &&
                   (form == PRAD_ADAM_RMAD || form == PRAD_ADAM_PRAD),
               PRAD_ERR_INVALID, "prad_clip_adam: bad dtype, clip mode or Adam form");
  PRAD_REQUIRE(clip_mode != 2 || clip_value > 0, PRAD_ERR_INVALID, "prad_clip_adam: max norm must be positive");
  void* const* lists[4] = {w_host, g_host, m_host, v_host};
  prad_status s = check_lists("prad_clip_adam", lists, 4, sizes_host, count);
  if (s || count == 0) return s;
  return dt == PRAD_F32
             ? clip_adam_t<float>(ctx, w_host, g_host, m_host, v_host, sizes_host, count, clip_mode, clip_value, min_value, 1, lr, beta1, beta2, eps, iteration, form, zero_grad, nullptr)
             : clip_adam_t<double>(ctx, w_host, g_host, m_host, v_host, sizes_host, count, clip_mode, clip_value, min_value, 1, lr, beta1, beta2, eps, iteration, form, zero_grad, nullptr);
}

prad_status prad_adam(prad_ctx* ctx, prad_dtype dt, void* const* w_host, void* const* g_host,
                      void* const* m_host, void* const* v_host, const int64_t* sizes_host,
                      int count, double lr, double beta1, double beta2, double eps,
                      double iteration, prad_adam_form form, int zero_grad) {
  return prad_clip_adam(ctx, dt, w_host, g_host, m_host, v_host, sizes_host, count, 0, 0, 0, lr,
                        beta1, beta2, eps, iteration, form, zero_grad);
}

}  // extern "C"
