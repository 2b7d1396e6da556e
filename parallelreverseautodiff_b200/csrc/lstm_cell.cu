// One LSTM cell's Backward as a single kernel: what the managed graph runs as eleven operations per time
// step -- the loss gradient of that step, the fan-in sum at h_t (GradientUtils.AccumulateGradients,
// src/RMAD/GradientUtils.cs:22-42), HadamardProductOperation.Backward for o (.) tanh(c), i (.) g and
// f (.) c_prev (src/RMAD/HadamardProductOperation.cs:84-118), TanhOperation.Backward
// (src/RMAD/TanhOperation.cs:60-78), the fan-in sum at c_t, and the four gate derivatives
// (SigmoidOperation.cs:65-84, TanhOperation.cs:60-78).  Every element is independent of every other, so
// the chain is evaluated per element in registers with exactly the roundings of the separate kernels
// (one rounding per managed arithmetic operation, sums in list order): the results are bit-identical
// to running the operations one by one, with 1 launch instead of 11 and none of the intermediate
// tensors written.
#include "act_math.cuh"
#include "common.cuh"

namespace prad {

constexpr int LSTM_MAX_CONTRIB = 8;

template <typename T> struct LstmCellArgs {
  const T* h;          // h_t (for the loss gradient), may be null with y
  const T* y;          // target of step t, null = no loss at this step
  T loss_scale;        // 2 / (rows_total * cols) of MeanSquaredErrorLossOperation.Backward
  const T* contrib[LSTM_MAX_CONTRIB];   // further gradients w.r.t. h_t, added after the loss gradient in this order
  int n_contrib;
  const T* dc_next;    // gradient w.r.t. c_t from step t+1 (dc_{t+1} (.) f_{t+1}), null at the last step
  const T *i, *f, *g, *o, *tanh_c, *c_prev;   // gate outputs, tanh(c_t), c_{t-1} (null at t = 0)
  T *dpre_i, *dpre_f, *dpre_g, *dpre_o;       // gradients w.r.t. the gate pre-activations
  T* dc_prev;          // dc_t (.) f_t, the next dc_next (null when c_prev is null)
};

template <typename T>
__global__ void __launch_bounds__(256)
lstm_cell_backward_kernel(LstmCellArgs<T> a, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    // dh = loss gradient + contributions, left to right (a single source is passed through unchanged)
    T dh = (T)0;
    bool have = false;
    if (a.y) { dh = mul_rn(a.loss_scale, sub_rn(a.h[e], a.y[e])); have = true; }
    for (int k = 0; k < a.n_contrib; ++k) {
      const T v = a.contrib[k][e];
      dh = have ? add_rn(dh, v) : v;
      have = true;
    }
    const T o = a.o[e], tc = a.tanh_c[e];
    const T d_o = mul_rn(dh, tc), d_tc = mul_rn(dh, o);                 // h = o (.) tanh c
    const T dc_a = mul_rn(d_tc, sub_rn((T)1, mul_rn(tc, tc)));         // tanh backward reads its output
    const T dc = a.dc_next ? add_rn(dc_a, a.dc_next[e]) : dc_a;         // fan-in at c_t: (tanh path, next step)
    const T gi = a.i[e], gg = a.g[e], gf = a.f[e];
    const T d_i = mul_rn(dc, gg), d_g = mul_rn(dc, gi);                 // c = f (.) c_prev + i (.) g
    T d_f = (T)0;
    if (a.c_prev) {
      d_f = mul_rn(dc, a.c_prev[e]);
      a.dc_prev[e] = mul_rn(dc, gf);
    }
    a.dpre_i[e] = mul_rn(d_i, mul_rn(gi, sub_rn((T)1, gi)));            // sigmoid backward reads its output
    a.dpre_f[e] = mul_rn(d_f, mul_rn(gf, sub_rn((T)1, gf)));
    a.dpre_g[e] = mul_rn(d_g, sub_rn((T)1, mul_rn(gg, gg)));
    a.dpre_o[e] = mul_rn(d_o, mul_rn(o, sub_rn((T)1, o)));
  }
}

template <typename T>
static prad_status lstm_cell_backward_t(prad_ctx* ctx, int64_t n, const void* h, const void* y, double loss_scale,
                                        const void* const* contrib, int n_contrib, const void* dc_next,
                                        const void* const* gates, const void* tanh_c, const void* c_prev,
                                        void* const* dpre, void* dc_prev) {
  LstmCellArgs<T> a;
  a.h = (const T*)h;
  a.y = (const T*)y;
  a.loss_scale = (T)loss_scale;
  for (int k = 0; k < LSTM_MAX_CONTRIB; ++k) a.contrib[k] = k < n_contrib ? (const T*)contrib[k] : nullptr;
  a.n_contrib = n_contrib;
  a.dc_next = (const T*)dc_next;
  a.i = (const T*)gates[0];
  a.f = (const T*)gates[1];
  a.g = (const T*)gates[2];
  a.o = (const T*)gates[3];
  a.tanh_c = (const T*)tanh_c;
  a.c_prev = (const T*)c_prev;
  a.dpre_i = (T*)dpre[0];
  a.dpre_f = (T*)dpre[1];
  a.dpre_g = (T*)dpre[2];
  a.dpre_o = (T*)dpre[3];
  a.dc_prev = (T*)dc_prev;
  const int grid = stream_grid(ctx, n, 256, 8);
  lstm_cell_backward_kernel<T><<<grid, 256, 0, ctx->stream>>>(a, n);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

}  // namespace prad

using namespace prad;

extern "C" prad_status prad_lstm_cell_backward(prad_ctx* ctx, prad_dtype dt, int64_t n, const void* h, const void* target,
                                               double loss_scale, const void* const* dh_contrib_host, int n_contrib,
                                               const void* dc_next, const void* const* gates_ifgo_host, const void* tanh_c,
                                               const void* c_prev, void* const* dpre_ifgo_host, void* dc_prev) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && n_contrib >= 0 && n_contrib <= LSTM_MAX_CONTRIB, PRAD_ERR_INVALID,
               "prad_lstm_cell_backward: bad dtype, size, or more than %d contributions", LSTM_MAX_CONTRIB);
  if (n == 0) return PRAD_OK;
  PRAD_REQUIRE(gates_ifgo_host && dpre_ifgo_host && tanh_c && (n_contrib == 0 || dh_contrib_host), PRAD_ERR_INVALID,
               "prad_lstm_cell_backward: null pointer list");
  PRAD_REQUIRE((target != nullptr) == (target != nullptr && h != nullptr), PRAD_ERR_INVALID,
               "prad_lstm_cell_backward: a target needs h");
  PRAD_REQUIRE(target || n_contrib > 0, PRAD_ERR_INVALID, "prad_lstm_cell_backward: no gradient reaches h (no target, no contribution)");
  PRAD_REQUIRE((c_prev == nullptr) == (dc_prev == nullptr), PRAD_ERR_INVALID,
               "prad_lstm_cell_backward: c_prev and dc_prev go together (both null at the first time step)");
  for (int k = 0; k < 4; ++k)
    PRAD_REQUIRE(gates_ifgo_host[k] && dpre_ifgo_host[k], PRAD_ERR_INVALID, "prad_lstm_cell_backward: gate %d is null", k);
  for (int k = 0; k < n_contrib; ++k)
    PRAD_REQUIRE(dh_contrib_host[k], PRAD_ERR_INVALID, "prad_lstm_cell_backward: contribution %d is null", k);
  return dt == PRAD_F32
             ? lstm_cell_backward_t<float>(ctx, n, h, target, loss_scale, dh_contrib_host, n_contrib, dc_next, gates_ifgo_host,
                                           tanh_c, c_prev, dpre_ifgo_host, dc_prev)
             : lstm_cell_backward_t<double>(ctx, n, h, target, loss_scale, dh_contrib_host, n_contrib, dc_next, gates_ifgo_host,
                                            tanh_c, c_prev, dpre_ifgo_host, dc_prev);
}
