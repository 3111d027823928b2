// Element-type dispatch shared by the kernel launchers.
#pragma once

// dtype codes follow flagcxDataType_t
#define FCX_DISPATCH_SAME(DT, CALL)                                         \
  switch (DT) {                                                             \
    case 0: return CALL(int8_t, int8_t);                                    \
    case 1: return CALL(uint8_t, uint8_t);                                  \
    case 2: return CALL(int32_t, int32_t);                                  \
    case 3: return CALL(uint32_t, uint32_t);                                \
    case 4: return CALL(long long, long long);                              \
    case 5: return CALL(unsigned long long, unsigned long long);            \
    case 6: return CALL(__half, __half);                                    \
    case 7: return CALL(float, float);                                      \
    case 8: return CALL(double, double);                                    \
    case 9: return CALL(__nv_bfloat16, __nv_bfloat16);                      \
    case 10: return CALL(F8E4, F8E4);                                       \
    case 11: return CALL(F8E5, F8E5);                                       \
    default: return cudaErrorInvalidValue;                                  \
  }


#define FCX_DISPATCH_ALL(A, CALL)                                                        \
  do {                                                                                   \
    if ((A)->outDtype == (A)->dtype) { FCX_DISPATCH_SAME((A)->dtype, CALL) }             \
    /* fused cast: the reduction runs in fp32, the result is rounded once */             \
    if ((A)->dtype == 7 && (A)->outDtype == 9) return CALL(float, __nv_bfloat16);        \
    if ((A)->dtype == 7 && (A)->outDtype == 6) return CALL(float, __half);               \
    if ((A)->dtype == 7 && (A)->outDtype == 10) return CALL(float, F8E4);                \
    if ((A)->dtype == 9 && (A)->outDtype == 10) return CALL(__nv_bfloat16, F8E4);        \
    if ((A)->dtype == 9 && (A)->outDtype == 11) return CALL(__nv_bfloat16, F8E5);        \
    if ((A)->dtype == 9 && (A)->outDtype == 7) return CALL(__nv_bfloat16, float);        \
    if ((A)->dtype == 10 && (A)->outDtype == 9) return CALL(F8E4, __nv_bfloat16);        \
    return cudaErrorInvalidValue;                                                        \
  } while (0)

