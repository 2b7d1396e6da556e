// Device-side scalar math of the activations, written once and used by the stand-alone
// elementwise kernels and by the GEMM epilogues.  Each function states the reference lines
// it reproduces.  Explicit __fmul_rn/__fadd_rn (and the double twins) keep the compiler from
// fusing a multiply with an add where the managed code rounds twice.
#pragma once

#include <cuda_runtime.h>

#include "../../include/prad_cuda.h"

namespace prad {

__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ double sub_rn(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ float div_rn(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ double div_rn(double a, double b) { return __ddiv_rn(a, b); }
__device__ __forceinline__ float sqrt_rn(float a) { return __fsqrt_rn(a); }
__device__ __forceinline__ double sqrt_rn(double a) { return __dsqrt_rn(a); }

__device__ __forceinline__ float t_exp(float x) { return expf(x); }
__device__ __forceinline__ double t_exp(double x) { return exp(x); }
__device__ __forceinline__ float t_tanh(float x) { return tanhf(x); }
__device__ __forceinline__ double t_tanh(double x) { return tanh(x); }
__device__ __forceinline__ float t_log(float x) { return logf(x); }
__device__ __forceinline__ double t_log(double x) { return log(x); }

template <typename T> struct GeluConst;
template <> struct GeluConst<double> {
  // PradMath.Sqrt(2 / Math.PI)
  __device__ static double s2pi() { return 0.7978845608028654; }
  __device__ static double k() { return 0.044715; }
  __device__ static double k3() { return 0.044715 * 3; }
};
template <> struct GeluConst<float> {
  // (float)Math.Sqrt(2 / (float)Math.PI) ; 0.044715f ; 0.044715f * 3 rounded to float
  __device__ static float s2pi() { return 0.7978845f; }
  __device__ static float k() { return 0.044715f; }
  __device__ static float k3() { return 0.044715f * 3.0f; }
};

// GELUOperation.cs:86-92
template <typename T> __device__ __forceinline__ T gelu_value(T x) {
  T x3 = mul_rn(mul_rn(x, x), x);
  T inner = mul_rn(GeluConst<T>::s2pi(), add_rn(x, mul_rn(GeluConst<T>::k(), x3)));
  T a = mul_rn((T)0.5, add_rn((T)1, t_tanh(inner)));
  return mul_rn(a, x);
}
// GELUOperation.cs:94-101, as written: c = (1-b^2)^2 and the 0.5*x*b term
template <typename T> __device__ __forceinline__ T gelu_derivative(T x) {
  T x2 = mul_rn(x, x);
  T x3 = mul_rn(x2, x);
  T b = t_tanh(mul_rn(GeluConst<T>::s2pi(), add_rn(x, mul_rn(GeluConst<T>::k(), x3))));
  T omb2 = sub_rn((T)1, mul_rn(b, b));
  T c = mul_rn(omb2, omb2);
  T d = mul_rn(GeluConst<T>::s2pi(), add_rn(mul_rn(GeluConst<T>::k3(), x2), (T)1));
  T t0 = mul_rn((T)0.5, x);
  T t1 = add_rn(mul_rn(c, d), b);
  T t2 = mul_rn((T)0.5, add_rn((T)1, b));
  return add_rn(mul_rn(t0, t1), t2);
}

__device__ __forceinline__ float t_pow(float x, float y) { return (float)pow((double)x, (double)y); }
__device__ __forceinline__ double t_pow(double x, double y) { return pow(x, y); }

// AmplifiedSigmoidOperation.cs:45-83.  PradMath.PI is (float)Math.PI in both precisions, so the
// base PI - 2 is 1.1415927410125732 either way; Pow goes through double and is cast back.
template <typename T> __device__ __forceinline__ T amp_base() { return (T)1.1415927410125732; }
template <typename T> __device__ __forceinline__ T amplified_sigmoid_value(T x) {
  return div_rn((T)1, add_rn((T)1, t_pow(amp_base<T>(), -x)));
}
// as written there: b^-x / (1 + b^-x)^2 (no ln b factor)
template <typename T> __device__ __forceinline__ T amplified_sigmoid_derivative(T x) {
  const T p = t_pow(amp_base<T>(), -x);
  return div_rn(p, t_pow(add_rn((T)1, p), (T)2));
}

// forward value of an activation
template <typename T> __device__ __forceinline__ T act_value(prad_act act, T x, T alpha) {
  switch (act) {
    case PRAD_ACT_LEAKY_RELU: return x > (T)0 ? x : mul_rn(alpha, x);        // LeakyReLUOperation.cs:66-67
    case PRAD_ACT_SIGMOID: return div_rn((T)1, add_rn((T)1, t_exp(-x)));     // SigmoidOperation.cs:57
    case PRAD_ACT_TANH: return t_tanh(x);                                    // TanhOperation.cs:52
    case PRAD_ACT_GELU: return gelu_value<T>(x);
    case PRAD_ACT_RELU: return x > (T)0 ? x : (T)0;                          // ReLUOperation.cs:50-51
    case PRAD_ACT_AMPLIFIED_SIGMOID: return amplified_sigmoid_value<T>(x);
    default: return x;
  }
}

// derivative factor from the tensor the managed op keeps (input x or output y)
template <typename T> __device__ __forceinline__ T act_derivative(prad_act act, T s, T alpha) {
  switch (act) {
    case PRAD_ACT_LEAKY_RELU: return s > (T)0 ? (T)1 : alpha;                // LeakyReLUOperation.cs:85-86
    case PRAD_ACT_SIGMOID: return mul_rn(s, sub_rn((T)1, s));                // SigmoidOperation.cs:75
    case PRAD_ACT_TANH: return sub_rn((T)1, mul_rn(s, s));                   // TanhOperation.cs:70
    case PRAD_ACT_GELU: return gelu_derivative<T>(s);
    case PRAD_ACT_RELU: return s > (T)0 ? (T)1 : (T)0;                       // ReLUOperation.cs:69-70
    case PRAD_ACT_AMPLIFIED_SIGMOID: return amplified_sigmoid_derivative<T>(s);
    default: return (T)1;
  }
}

}  // namespace prad
