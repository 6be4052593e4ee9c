// Shared macros and small helpers for the TACE sm_100a kernels.
//
// The arithmetic helpers are plain C++ templates marked TACE_HD so the same
// code runs inside the CUDA kernels and, compiled by g++, inside the CPU unit
// tests of the generated contraction code.
#pragma once
#include <cmath>
#include <cstdint>

#if defined(__CUDACC__)
#define TACE_HD __host__ __device__
#define TACE_D __device__
#define TACE_INLINE __forceinline__
#define TACE_CONST static __device__ const
#else
#define TACE_HD
#define TACE_D
#define TACE_INLINE inline
#define TACE_CONST static const
#ifndef __restrict__
#define __restrict__
#endif
#endif

namespace tace {

// Four consecutive table entries; under nvcc one (fp32) or two (fp64) 16-byte loads, p 16-byte aligned.
#if defined(__CUDACC__)
TACE_HD TACE_INLINE void ld4(const float* p, float& a, float& b, float& c, float& d) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  a = v.x; b = v.y; c = v.z; d = v.w;
}
TACE_HD TACE_INLINE void ld4(const double* p, double& a, double& b, double& c, double& d) {
  const double2 u = *reinterpret_cast<const double2*>(p), v = *reinterpret_cast<const double2*>(p + 2);
  a = u.x; b = u.y; c = v.x; d = v.y;
}
#else
template <typename T>
inline void ld4(const T* p, T& a, T& b, T& c, T& d) { a = p[0]; b = p[1]; c = p[2]; d = p[3]; }
#endif

// Path weights of a generated backward pass held in arrays: get<p>() reads w[p], put<p>(v) stores dE/dw_p.
template <typename T>
struct TpArrayWeights {
  const T* w;
  T* dw;
  template <int P> TACE_HD TACE_INLINE T get() const { return w[P]; }
  template <int P> TACE_HD TACE_INLINE void put(T v) { dw[P] = v; }
};

template <typename T>
TACE_HD TACE_INLINE T sigmoid_(T x) { return T(1) / (T(1) + exp(-x)); }
template <>
TACE_HD TACE_INLINE float sigmoid_<float>(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T>
TACE_HD TACE_INLINE T silu_(T x) { return x * sigmoid_(x); }

// d/dx [x * sigmoid(x)] = s * (1 + x * (1 - s))
template <typename T>
TACE_HD TACE_INLINE T silu_grad_(T x) {
  const T s = sigmoid_(x);
  return s * (T(1) + x * (T(1) - s));
}

}  // namespace tace
