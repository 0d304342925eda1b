/* Opcode and dtype numbering shared by the CUDA library, its Python host side and the test oracle.
 *
 * dtype codes are numpy type numbers, as in the reference's cgtDtype enum (include/cgt_common.h:21-34).
 * Unary opcodes follow the reference's UNARY_INFO table (cgt/core.py:1118-1134) plus the two custom
 * UnaryInfo entries the configs use: softplus (cgt/nn.py:51-53) and cast (cgt/api.py:131-143).
 * Binary opcodes follow BINARY_INFO (cgt/core.py:1139-1152).
 */
#ifndef CGT_B200_OPS_H
#define CGT_B200_OPS_H

#ifdef __cplusplus
extern "C" {
#endif

typedef enum cgtbDtype {
  cgtb_i1 = 1,
  cgtb_i2 = 3,
  cgtb_i4 = 5,
  cgtb_i8 = 7,
  cgtb_f4 = 11,
  cgtb_f8 = 12
} cgtbDtype;

typedef enum cgtbDevtype { cgtbCPU = 0, cgtbGPU = 1 } cgtbDevtype;

typedef enum cgtbUnaryOp {
  CGTB_U_ABS = 0,      /* fabs(x) */
  CGTB_U_CEIL = 1,     /* ceil(x) */
  CGTB_U_COS = 2,      /* cos(x) */
  CGTB_U_EXP = 3,      /* exp(x) */
  CGTB_U_ICEIL = 4,    /* (int)ceil(x) */
  CGTB_U_IFLOOR = 5,   /* (int)floor(x) */
  CGTB_U_LOG = 6,      /* log(x) */
  CGTB_U_NEG = 7,      /* (-x) */
  CGTB_U_SIGN = 8,     /* 2*(x>0)-1  (so sign(0) == -1) */
  CGTB_U_SIN = 9,      /* sin(x) */
  CGTB_U_SQUARE = 10,  /* x*x */
  CGTB_U_SQRT = 11,    /* sqrt(x) */
  CGTB_U_TANH = 12,    /* tanh(x) */
  CGTB_U_SIGMOID = 13, /* 1.0/(1.0+exp(-x)) : exp in the input type, the rest in double */
  CGTB_U_SOFTPLUS = 14,/* (x > 0) ? (x + log(exp(-x) + 1)) : log(1+exp(x)) */
  CGTB_U_CAST = 15,    /* x, converted to the output type */
  CGTB_U_COUNT = 16
} cgtbUnaryOp;

typedef enum cgtbBinaryOp {
  CGTB_B_MUL = 0, /* x*y */
  CGTB_B_ADD = 1, /* x+y */
  CGTB_B_SUB = 2, /* x-y */
  CGTB_B_DIV = 3, /* (x+0.0)/y : always a double division */
  CGTB_B_LT = 4,
  CGTB_B_GT = 5,
  CGTB_B_LE = 6,
  CGTB_B_GE = 7,
  CGTB_B_POW = 8, /* pow(x,y) */
  CGTB_B_EQ = 9,
  CGTB_B_NE = 10,
  CGTB_B_COUNT = 11
} cgtbBinaryOp;

typedef enum cgtbReduceOp { CGTB_R_SUM = 0, CGTB_R_MAX = 1 } cgtbReduceOp;

#define CGTB_MAX_NDIM 8

#ifdef __cplusplus
}
#endif
#endif
