// Host-side element arithmetic for every flagcxDataType_t, used by the CPU
// collective path and as the oracle of the perf tools.  16- and 8-bit floats
// are widened to fp32, combined pairwise and rounded back (nearest-even, fp8
// saturating to the largest finite value) with the same conversion rule as
// the GPU kernels; the GPU kernels keep the fp32 accumulator across all
// ranks and round only once, so low-precision sums can differ by an ulp.
// The reference's host reduce has no fp16/bf16 support
// (flagcx/service/utils.h:648-709); this one covers all twelve types.
#pragma once
#include "flagcx.h"
#include <cmath>
#include <cstdint>
#include <cstring>

namespace fcx {

inline float bf16ToFloat(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t floatToBf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
  uint32_t lsb = (u >> 16) & 1;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

inline float halfToFloat(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {
      int e = -1;
      do { e++; man <<= 1; } while (!(man & 0x400));
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

// Round an fp32 to a small float format with `eb` exponent and `mb` mantissa
// bits.  ieeeInf: the top exponent encodes inf/NaN (fp16, e5m2); otherwise
// only the all-ones pattern is NaN (e4m3).  saturate: overflow gives the
// largest finite value instead of inf/NaN.
inline uint32_t floatToSmall(float f, int eb, int mb, bool ieeeInf, bool saturate) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t sign = (u >> 31) << (eb + mb);
  uint32_t absu = u & 0x7fffffffu;
  int bias = (1 << (eb - 1)) - 1;
  uint32_t expMaxField = (1u << eb) - 1;
  uint32_t maxFinite = ieeeInf ? (((expMaxField - 1) << mb) | ((1u << mb) - 1))
                               : ((expMaxField << mb) | ((1u << mb) - 2));
  uint32_t nanPat = ieeeInf ? ((expMaxField << mb) | (1u << (mb - 1))) : ((expMaxField << mb) | ((1u << mb) - 1));
  uint32_t infPat = ieeeInf ? (expMaxField << mb) : nanPat;
  if (absu > 0x7f800000u) return sign | nanPat;
  if (absu == 0x7f800000u) return sign | (saturate ? maxFinite : infPat);
  int e = (int)(absu >> 23) - 127;
  uint32_t man = absu & 0x7fffffu;
  uint32_t out;
  if (e < 1 - bias) {
    // subnormal in the target: value = man' * 2^(1-bias-mb)
    int shift = (1 - bias) - e;  // how far below the smallest normal exponent
    if (shift > mb + 1) return sign;  // rounds to zero
    uint32_t full = man | 0x800000u;  // 24-bit significand
    int rs = 23 - mb + shift;
    uint32_t q = full >> rs, rem = full & ((1u << rs) - 1), half = 1u << (rs - 1);
    if (rem > half || (rem == half && (q & 1))) q++;
    out = q;  // may carry into the normal range, which is the right encoding
  } else {
    int rs = 23 - mb;
    uint32_t q = man >> rs, rem = man & ((1u << rs) - 1), half = 1u << (rs - 1);
    uint32_t ef = (uint32_t)(e + bias);
    out = (ef << mb) | q;
    if (rem > half || (rem == half && (q & 1))) out++;
  }
  if (out > maxFinite) return sign | (saturate ? maxFinite : infPat);
  return sign | out;
}

inline float smallToFloat(uint32_t v, int eb, int mb, bool ieeeInf) {
  int bias = (1 << (eb - 1)) - 1;
  uint32_t sign = (v >> (eb + mb)) & 1;
  uint32_t ef = (v >> mb) & ((1u << eb) - 1), man = v & ((1u << mb) - 1);
  float r;
  if (ef == (1u << eb) - 1 && (ieeeInf || man == (1u << mb) - 1)) {
    r = (ieeeInf && man == 0) ? INFINITY : NAN;
  } else if (ef == 0) {
    r = ldexpf((float)man, 1 - bias - mb);
  } else {
    r = ldexpf((float)(man | (1u << mb)), (int)ef - bias - mb);
  }
  return sign ? -r : r;
}

inline uint16_t floatToHalf(float f) { return (uint16_t)floatToSmall(f, 5, 10, true, false); }
inline uint8_t floatToE4m3(float f) { return (uint8_t)floatToSmall(f, 4, 3, false, true); }
inline uint8_t floatToE5m2(float f) { return (uint8_t)floatToSmall(f, 5, 2, true, true); }
inline float e4m3ToFloat(uint8_t v) { return smallToFloat(v, 4, 3, false); }
inline float e5m2ToFloat(uint8_t v) { return smallToFloat(v, 5, 2, true); }

inline size_t dtypeSize(flagcxDataType_t t) {
  switch (t) {
    case flagcxInt8: case flagcxUint8: case flagcxFloat8e4m3: case flagcxFloat8e5m2: return 1;
    case flagcxFloat16: case flagcxBfloat16: return 2;
    case flagcxInt32: case flagcxUint32: case flagcxFloat32: return 4;
    case flagcxInt64: case flagcxUint64: case flagcxFloat64: return 8;
    default: return 0;
  }
}

template <typename T>
inline T combine(T a, T b, flagcxRedOp_t op) {
  switch (op) {
    case flagcxProd: return a * b;
    case flagcxMax: return a > b ? a : b;
    case flagcxMin: return a < b ? a : b;
    default: return a + b;  // sum and avg
  }
}

// acc[i] = acc[i] (op) in[i]
inline void hostReduceInto(void *acc, const void *in, size_t n, flagcxDataType_t t, flagcxRedOp_t op) {
#define FCX_PLAIN(T)                                                     \
  { T *a = (T *)acc; const T *b = (const T *)in;                         \
    for (size_t i = 0; i < n; i++) a[i] = combine<T>(a[i], b[i], op); }  \
  break
#define FCX_VIA_FLOAT(S, TOF, FROMF)                                                   \
  { S *a = (S *)acc; const S *b = (const S *)in;                                       \
    for (size_t i = 0; i < n; i++) a[i] = FROMF(combine<float>(TOF(a[i]), TOF(b[i]), op)); } \
  break
  switch (t) {
    case flagcxInt8: FCX_PLAIN(int8_t);
    case flagcxUint8: FCX_PLAIN(uint8_t);
    case flagcxInt32: FCX_PLAIN(int32_t);
    case flagcxUint32: FCX_PLAIN(uint32_t);
    case flagcxInt64: FCX_PLAIN(int64_t);
    case flagcxUint64: FCX_PLAIN(uint64_t);
    case flagcxFloat32: FCX_PLAIN(float);
    case flagcxFloat64: FCX_PLAIN(double);
    case flagcxFloat16: FCX_VIA_FLOAT(uint16_t, halfToFloat, floatToHalf);
    case flagcxBfloat16: FCX_VIA_FLOAT(uint16_t, bf16ToFloat, floatToBf16);
    case flagcxFloat8e4m3: FCX_VIA_FLOAT(uint8_t, e4m3ToFloat, floatToE4m3);
    case flagcxFloat8e5m2: FCX_VIA_FLOAT(uint8_t, e5m2ToFloat, floatToE5m2);
    default: break;
  }
#undef FCX_PLAIN
#undef FCX_VIA_FLOAT
}

// a[i] /= n  (the second half of flagcxAvg)
inline void hostDivide(void *acc, size_t n, flagcxDataType_t t, int div) {
#define FCX_PLAIN(T) { T *a = (T *)acc; for (size_t i = 0; i < n; i++) a[i] = (T)(a[i] / (T)div); } break
#define FCX_VIA_FLOAT(S, TOF, FROMF) { S *a = (S *)acc; for (size_t i = 0; i < n; i++) a[i] = FROMF(TOF(a[i]) / (float)div); } break
  switch (t) {
    case flagcxInt8: FCX_PLAIN(int8_t);
    case flagcxUint8: FCX_PLAIN(uint8_t);
    case flagcxInt32: FCX_PLAIN(int32_t);
    case flagcxUint32: FCX_PLAIN(uint32_t);
    case flagcxInt64: FCX_PLAIN(int64_t);
    case flagcxUint64: FCX_PLAIN(uint64_t);
    case flagcxFloat32: FCX_PLAIN(float);
    case flagcxFloat64: FCX_PLAIN(double);
    case flagcxFloat16: FCX_VIA_FLOAT(uint16_t, halfToFloat, floatToHalf);
    case flagcxBfloat16: FCX_VIA_FLOAT(uint16_t, bf16ToFloat, floatToBf16);
    case flagcxFloat8e4m3: FCX_VIA_FLOAT(uint8_t, e4m3ToFloat, floatToE4m3);
    case flagcxFloat8e5m2: FCX_VIA_FLOAT(uint8_t, e5m2ToFloat, floatToE5m2);
    default: break;
  }
#undef FCX_PLAIN
#undef FCX_VIA_FLOAT
}

}  // namespace fcx
