/* Scalar expressions of the elementwise Ops (cgt/core.py:1160-1378) and the vector pack used to move
 * them, shared by the prebuilt kernels and by fused-chain kernels generated at run time: both call the
 * same templates with the same operand types, which is what makes a fused chain agree bit for bit
 * with the Op-by-Op sequence. Device code only (included from .cu files). */
#ifndef CGT_ELWISE_H
#define CGT_ELWISE_H
#include <stdint.h>
#include <math.h>
#include <type_traits>

#include "cgt_b200_ops.h"

template <typename TI, typename TO>
__device__ __forceinline__ TO unary_apply(int op, TI x) {
  // integer inputs promote to double for the math functions, as C++ overload resolution does
  typedef typename std::conditional<std::is_floating_point<TI>::value, TI, double>::type TM;
  switch (op) {
    case CGTB_U_ABS: return (TO)(fabs((TM)x));
    case CGTB_U_CEIL: return (TO)(ceil((TM)x));
    case CGTB_U_COS: return (TO)(cos((TM)x));
    case CGTB_U_EXP: return (TO)(exp((TM)x));
    case CGTB_U_ICEIL: return (TO)((int)ceil((TM)x));
    case CGTB_U_IFLOOR: return (TO)((int)floor((TM)x));
    case CGTB_U_LOG: return (TO)(log((TM)x));
    case CGTB_U_NEG: return (TO)(-x);
    case CGTB_U_SIGN: return (TO)(2 * (x > 0) - 1);
    case CGTB_U_SIN: return (TO)(sin((TM)x));
    case CGTB_U_SQUARE: return (TO)(x * x);
    case CGTB_U_SQRT: return (TO)(sqrt((TM)x));
    case CGTB_U_TANH: return (TO)(tanh((TM)x));
    case CGTB_U_SIGMOID: return (TO)(1.0 / (1.0 + exp((TM)(-x))));
    case CGTB_U_SOFTPLUS: return (TO)((x > 0) ? (x + log(exp((TM)(-x)) + 1)) : log(1 + exp((TM)x)));
    case CGTB_U_CAST: return (TO)(x);
  }
  return TO(0);
}

template <typename TX, typename TY> struct pow_type { typedef double type; };
template <> struct pow_type<float, float> { typedef float type; };

template <typename TX, typename TY, typename TO>
__device__ __forceinline__ TO binary_apply(int op, TX x, TY y) {
  switch (op) {
    case CGTB_B_MUL: return (TO)(x * y);
    case CGTB_B_ADD: return (TO)(x + y);
    case CGTB_B_SUB: return (TO)(x - y);
    case CGTB_B_DIV: return (TO)((x + 0.0) / y);
    case CGTB_B_LT: return (TO)(x < y);
    case CGTB_B_GT: return (TO)(x > y);
    case CGTB_B_LE: return (TO)(x <= y);
    case CGTB_B_GE: return (TO)(x >= y);
    case CGTB_B_POW: {
      typedef typename pow_type<TX, TY>::type TP;
      return (TO)(pow((TP)x, (TP)y));
    }
    case CGTB_B_EQ: return (TO)(x == y);
    case CGTB_B_NE: return (TO)(x != y);
  }
  return TO(0);
}

// ------------------------------------------------------------------------------------------------
// vector pack: N consecutive elements moved with the widest aligned access that fits
// ------------------------------------------------------------------------------------------------
template <typename T, int N>
struct alignas(sizeof(T) * N <= 16 ? sizeof(T) * N : 16) Pack {
  T v[N];
};

template <typename T, int N>
__device__ __forceinline__ Pack<T, N> load_pack(const T* p) {
  return *reinterpret_cast<const Pack<T, N>*>(p);
}
template <typename T, int N>
__device__ __forceinline__ void store_pack(T* p, const Pack<T, N>& v) {
  *reinterpret_cast<Pack<T, N>*>(p) = v;
}


#endif
