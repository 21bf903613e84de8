// Software conversions and element-wise reductions for every ncclDataType_t on the host.
// Used by the host-memory data plane and as the CPU oracle of the GPU kernels: 16- and 8-bit
// floats are widened to fp32, reduced, and rounded back once (round-to-nearest-even), which is
// the rounding model of the device kernels (reference: src/device/symmetric/primitives.cuh:234-324).
#pragma once
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "nccl.h"

namespace b200 {

static inline float bitsToFloat(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t floatToBits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16ToFloat(uint16_t h) { return bitsToFloat((uint32_t)h << 16); }
static inline uint16_t floatToBf16(float f) {
  uint32_t u = floatToBits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1);
  return (uint16_t)(u >> 16);
}

static inline float halfToFloat(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  int exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ff;
  if (exp == 0) {
    if (man == 0) return bitsToFloat(sign);
    float v = ldexpf((float)man, -24);
    return sign ? -v : v;
  }
  if (exp == 31) return bitsToFloat(sign | 0x7f800000u | (man << 13));
  return bitsToFloat(sign | ((uint32_t)(exp + 112) << 23) | (man << 13));
}

// Generic IEEE-like narrowing with round-to-nearest-even: expBits/manBits of the target,
// `bias`, whether the target has infinities, and its largest finite magnitude.
static inline uint32_t narrowFloat(float f, int expBits, int manBits, int bias, bool hasInf, float maxFinite,
                                   uint32_t nanCode, uint32_t infCode) {
  uint32_t u = floatToBits(f);
  uint32_t sign = (u >> 31) << (expBits + manBits);
  float a = fabsf(f);
  if (a != a) return sign | nanCode;
  if (a > maxFinite) {
    // values past the largest finite number round to it unless they reach the next binade midpoint
    float ulpTop = ldexpf(1.0f, (int)floorf(log2f(maxFinite)) - manBits);
    if (hasInf && (isinf(a) || a >= maxFinite + ulpTop / 2)) return sign | infCode;
    a = maxFinite;
  }
  if (a == 0) return sign;
  int e;
  float m = frexpf(a, &e);  // a = m * 2^e, m in [0.5,1)
  int unbiased = e - 1;
  int minExp = 1 - bias;
  uint32_t out;
  if (unbiased < minExp) {
    // subnormal: quantum 2^(minExp - manBits)
    float q = ldexpf(a, -(minExp - manBits));
    float r = nearbyintf(q);
    out = (uint32_t)r;  // may carry into the first normal, which is the right encoding
  } else {
    float q = ldexpf(m * 2.0f - 1.0f, manBits);  // fraction scaled
    float r = nearbyintf(q);
    uint32_t man = (uint32_t)r;
    uint32_t ex = (uint32_t)(unbiased + bias);
    if (man == (1u << manBits)) { man = 0; ++ex; }
    out = (ex << manBits) | man;
  }
  return sign | out;
}

static inline uint16_t floatToHalf(float f) {
  return (uint16_t)narrowFloat(f, 5, 10, 15, true, 65504.0f, 0x7e00, 0x7c00);
}

// fp8 e4m3 (finite-only variant: no infinity, S.1111.111 is NaN, max 448) and e5m2 (IEEE-like).
static inline float e4m3ToFloat(uint8_t v) {
  int sign = v >> 7, exp = (v >> 3) & 0xf, man = v & 7;
  float r;
  if (exp == 0xf && man == 7) return bitsToFloat(0x7fc00000u);
  if (exp == 0) r = ldexpf((float)man, -9);
  else r = ldexpf(1.0f + man / 8.0f, exp - 7);
  return sign ? -r : r;
}
static inline uint8_t floatToE4m3(float f) {
  // saturating conversion (the device uses __NV_SATFINITE): overflow and inf clamp to +-448
  uint32_t sign = f < 0 || (f == 0 && signbit(f)) ? 0x80 : 0;
  float a = fabsf(f);
  if (a != a) return (uint8_t)(sign | 0x7f);
  if (a > 448.0f) a = 448.0f;
  return (uint8_t)(narrowFloat(a, 4, 3, 7, false, 448.0f, 0x7f, 0x7e) | sign);
}
static inline float e5m2ToFloat(uint8_t v) { return halfToFloat((uint16_t)v << 8); }
static inline uint8_t floatToE5m2(float f) {
  uint32_t sign = f < 0 || (f == 0 && signbit(f)) ? 0x80 : 0;
  float a = fabsf(f);
  if (a != a) return (uint8_t)(sign | 0x7f);
  if (a > 57344.0f) a = 57344.0f;
  return (uint8_t)(narrowFloat(a, 5, 2, 15, true, 57344.0f, 0x7f, 0x7c) | sign);
}

enum HostOp { HOP_SUM = 0, HOP_PROD = 1, HOP_MAX = 2, HOP_MIN = 3 };

template <typename A> static inline A applyOp(int op, A a, A b) {
  switch (op) {
    case HOP_SUM: return a + b;
    case HOP_PROD: return a * b;
    case HOP_MAX: return a > b ? a : b;
    default: return a < b ? a : b;
  }
}

// acc[i] = op(acc[i], in[i]) over `n` elements of `type`; narrow floats go through fp32.
static inline void hostReduceInto(void* acc, const void* in, size_t n, ncclDataType_t type, int op) {
#define LOOP_NATIVE(T)                                                              \
  { T* a = (T*)acc; const T* b = (const T*)in;                                      \
    for (size_t i = 0; i < n; ++i) a[i] = applyOp<T>(op, a[i], b[i]); } break
#define LOOP_WIDE(S, LOAD, STORE)                                                   \
  { S* a = (S*)acc; const S* b = (const S*)in;                                      \
    for (size_t i = 0; i < n; ++i) a[i] = STORE(applyOp<float>(op, LOAD(a[i]), LOAD(b[i]))); } break
  switch (type) {
    case ncclInt8: LOOP_NATIVE(int8_t);
    case ncclUint8: LOOP_NATIVE(uint8_t);
    case ncclInt32: LOOP_NATIVE(int32_t);
    case ncclUint32: LOOP_NATIVE(uint32_t);
    case ncclInt64: LOOP_NATIVE(int64_t);
    case ncclUint64: LOOP_NATIVE(uint64_t);
    case ncclFloat32: LOOP_NATIVE(float);
    case ncclFloat64: LOOP_NATIVE(double);
    case ncclFloat16: LOOP_WIDE(uint16_t, halfToFloat, floatToHalf);
    case ncclBfloat16: LOOP_WIDE(uint16_t, bf16ToFloat, floatToBf16);
    case ncclFloat8e4m3: LOOP_WIDE(uint8_t, e4m3ToFloat, floatToE4m3);
    case ncclFloat8e5m2: LOOP_WIDE(uint8_t, e5m2ToFloat, floatToE5m2);
    default: break;
  }
#undef LOOP_NATIVE
#undef LOOP_WIDE
}

// buf[i] = buf[i] * scale (floats) or buf[i] / div (integers): ncclAvg and PreMulSum post/pre steps.
static inline void hostScale(void* buf, size_t n, ncclDataType_t type, double scale, int64_t intDiv) {
#define LOOP_INT(T) { T* a = (T*)buf; if (intDiv > 1) for (size_t i = 0; i < n; ++i) a[i] = (T)(a[i] / (T)intDiv); } break
#define LOOP_F(S, LOAD, STORE) { S* a = (S*)buf; for (size_t i = 0; i < n; ++i) a[i] = STORE((float)(LOAD(a[i]) * (float)scale)); } break
  switch (type) {
    case ncclInt8: LOOP_INT(int8_t);
    case ncclUint8: LOOP_INT(uint8_t);
    case ncclInt32: LOOP_INT(int32_t);
    case ncclUint32: LOOP_INT(uint32_t);
    case ncclInt64: LOOP_INT(int64_t);
    case ncclUint64: LOOP_INT(uint64_t);
    case ncclFloat32: { float* a = (float*)buf; for (size_t i = 0; i < n; ++i) a[i] *= (float)scale; } break;
    case ncclFloat64: { double* a = (double*)buf; for (size_t i = 0; i < n; ++i) a[i] *= scale; } break;
    case ncclFloat16: LOOP_F(uint16_t, halfToFloat, floatToHalf);
    case ncclBfloat16: LOOP_F(uint16_t, bf16ToFloat, floatToBf16);
    case ncclFloat8e4m3: LOOP_F(uint8_t, e4m3ToFloat, floatToE4m3);
    case ncclFloat8e5m2: LOOP_F(uint8_t, e5m2ToFloat, floatToE5m2);
    default: break;
  }
#undef LOOP_INT
#undef LOOP_F
}

}  // namespace b200
