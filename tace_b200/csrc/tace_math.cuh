// Per-edge arithmetic of the TACE path: real spherical harmonics and their
// gradient, Bessel radial basis with polynomial envelope, the radial MLP.
//
// Conventions follow the reference model (paths relative to its project root):
//  * angular basis: e3nn real spherical harmonics, polar axis y, m = -l..l,
//    "component" normalisation, evaluated on edge_vector / edge_length
//    (tace/models/angular.py:288-315, tace/models/_e3nn/representation.py:321-324);
//  * radial basis: sqrt(2/rc) sin(n pi d / rc) / d times the C2 polynomial
//    envelope (tace/models/radial.py:74-78, 458-469, 990-991);
//  * radial MLP: 8 -> 64 -> 64 -> 64 with plain SiLU, no bias
//    (tace/models/mlp.py:136-191); the last (64 -> paths*channels) layer is a
//    separate GEMM.
// All functions are TACE_HD so the CPU unit tests run the same code.
#pragma once
#include "tace_common.cuh"

namespace tace {

constexpr int kNumBessel = 8;
constexpr int kHidden = 64;

// ---- spherical harmonics, component normalisation ---------------------------
template <typename T, int L>
TACE_HD TACE_INLINE void sh_eval(const T x, const T y, const T z, T (&Y)[(L + 1) * (L + 1)]) {
  Y[0] = T(1);
  if (L >= 1) {
    const T c1 = T(1.7320508075688772);
    Y[1] = c1 * x; Y[2] = c1 * y; Y[3] = c1 * z;
  }
  if (L >= 2) {
    const T c2 = T(2.23606797749979);  // sqrt(5)
    const T s3 = T(1.7320508075688772);
    const T x2z2 = x * x + z * z;
    Y[4] = c2 * s3 * x * z;
    Y[5] = c2 * s3 * x * y;
    Y[6] = c2 * (y * y - T(0.5) * x2z2);
    Y[7] = c2 * s3 * y * z;
    Y[8] = c2 * T(0.8660254037844386) * (z * z - x * x);
  }
  if (L >= 3) {
    const T c3 = T(2.6457513110645907);  // sqrt(7)
    const T a = T(0.7905694150420949);   // sqrt(10)/4
    const T b = T(3.872983346207417);    // sqrt(15)
    const T c = T(0.6123724356957945);   // sqrt(6)/4
    const T x2 = x * x, y2 = y * y, z2 = z * z;
    Y[9] = c3 * a * (T(3) * x * z2 - x * x2);
    Y[10] = c3 * b * x * y * z;
    Y[11] = c3 * c * (T(4) * y2 - x2 - z2) * x;
    Y[12] = c3 * T(0.5) * y * (T(2) * y2 - T(3) * (x2 + z2));
    Y[13] = c3 * c * z * (T(4) * y2 - x2 - z2);
    Y[14] = c3 * T(0.5) * b * y * (z2 - x2);
    Y[15] = c3 * a * (z * z2 - T(3) * x2 * z);
  }
}

// dn[a] = sum_i dY[i] * dY_i/dn_a  (dY[0] does not contribute)
template <typename T, int L>
TACE_HD TACE_INLINE void sh_grad(const T x, const T y, const T z, const T (&dY)[(L + 1) * (L + 1)], T (&dn)[3]) {
  T gx = T(0), gy = T(0), gz = T(0);
  if (L >= 1) {
    const T c1 = T(1.7320508075688772);
    gx += c1 * dY[1]; gy += c1 * dY[2]; gz += c1 * dY[3];
  }
  if (L >= 2) {
    const T c2 = T(2.23606797749979);
    const T s3 = T(1.7320508075688772);
    gx += c2 * (s3 * z * dY[4] + s3 * y * dY[5] - x * dY[6] - s3 * x * dY[8]);
    gy += c2 * (s3 * x * dY[5] + T(2) * y * dY[6] + s3 * z * dY[7]);
    gz += c2 * (s3 * x * dY[4] - z * dY[6] + s3 * y * dY[7] + s3 * z * dY[8]);
  }
  if (L >= 3) {
    const T c3 = T(2.6457513110645907);
    const T a = T(0.7905694150420949);
    const T b = T(3.872983346207417);
    const T c = T(0.6123724356957945);
    const T x2 = x * x, y2 = y * y, z2 = z * z;
    gx += c3 * (a * (T(3) * z2 - T(3) * x2) * dY[9] + b * y * z * dY[10] + c * (T(4) * y2 - T(3) * x2 - z2) * dY[11] -
                T(3) * x * y * dY[12] - c * T(2) * x * z * dY[13] - b * x * y * dY[14] - a * T(6) * x * z * dY[15]);
    gy += c3 * (b * x * z * dY[10] + c * T(8) * x * y * dY[11] + T(0.5) * (T(6) * y2 - T(3) * (x2 + z2)) * dY[12] +
                c * T(8) * y * z * dY[13] + T(0.5) * b * (z2 - x2) * dY[14]);
    gz += c3 * (a * T(6) * x * z * dY[9] + b * x * y * dY[10] - c * T(2) * x * z * dY[11] - T(3) * y * z * dY[12] +
                c * (T(4) * y2 - x2 - T(3) * z2) * dY[13] + b * y * z * dY[14] + a * (T(3) * z2 - T(3) * x2) * dY[15]);
  }
  dn[0] = gx; dn[1] = gy; dn[2] = gz;
}

// ---- radial basis -------------------------------------------------------------
template <typename T> TACE_HD TACE_INLINE T sin_(T x) { return sin(x); }
template <> TACE_HD TACE_INLINE float sin_<float>(float x) { return sinf(x); }
template <typename T> TACE_HD TACE_INLINE T cos_(T x) { return cos(x); }
template <> TACE_HD TACE_INLINE float cos_<float>(float x) { return cosf(x); }

template <typename T>
TACE_HD TACE_INLINE T ipow_(T x, int p) {
  T r = T(1);
  for (int i = 0; i < p; ++i) r *= x;
  return r;
}

// Frequencies n*pi/rc and the prefactor sqrt(2/rc) are taken from the model's buffers
// (they are stored in the checkpoint and may be trained), not recomputed.
template <typename T>
struct RadialParams {
  T w[kNumBessel];
  T pref;
  T rc;
  int p;  // envelope exponent
  int env_after_mlp;  // radial_basis.apply_cutoff = False: the basis carries no envelope, the MLP output is multiplied by it
};

// polynomial envelope u(d / rc) and du/dd (tace/models/radial.py:437-472)
template <typename T>
TACE_HD TACE_INLINE void envelope_eval(const T d, const RadialParams<T>& rp, T& u, T& du) {
  const T rc = rp.rc;
  const int p = rp.p;
  const T xr = d / rc;
  u = T(0); du = T(0);
  if (d < rc) {
    const T pp = T(p);
    const T xp = ipow_(xr, p - 1);  // x^(p-1)
    u = T(1) - (pp + T(1)) * (pp + T(2)) / T(2) * xp * xr + pp * (pp + T(2)) * xp * xr * xr -
        pp * (pp + T(1)) / T(2) * xp * xr * xr * xr;
    du = -(pp * (pp + T(1)) * (pp + T(2)) / T(2)) * xp * (T(1) - xr) * (T(1) - xr) / rc;
  }
}

// b[n] = pref sin(w_n d) / d * u(d/rc), n = 0..7 (u = 1 with env_after_mlp); if db != nullptr also d b[n] / d d.
template <typename T>
TACE_HD TACE_INLINE void radial_eval(const T d, const RadialParams<T>& rp, T (&b)[kNumBessel], T* db) {
  T u = T(1), du = T(0);
  if (!rp.env_after_mlp) envelope_eval<T>(d, rp, u, du);
  const T inv_d = T(1) / d;
  for (int n = 0; n < kNumBessel; ++n) {
    const T wn = rp.w[n];
    const T s = sin_(wn * d), c = cos_(wn * d);
    const T j = rp.pref * s * inv_d;
    b[n] = j * u;
    if (db) db[n] = rp.pref * (wn * c * d - s) * inv_d * inv_d * u + j * du;
  }
}

// ---- radial MLP hidden layers ---------------------------------------------------
// Weights are stored [in][out] with the 1/sqrt(fan_in) and sqrt(2) gains folded in.  Everything is
// kept in registers: y = x @ A is evaluated as a sum of outer-product rows, so the 64 outputs are
// statically indexed accumulators and each weight row is read with 16-byte loads (every thread of a
// warp reads the same address, i.e. one broadcast transaction per load).
template <typename T, int K>
TACE_HD TACE_INLINE void matvec64(const T (&x)[K], const T* __restrict__ A, T (&y)[kHidden]) {
#pragma unroll
  for (int j = 0; j < kHidden; ++j) y[j] = T(0);
#pragma unroll 4
  for (int k = 0; k < K; ++k) {  // partly unrolled so the weight loads of the next rows overlap the FMAs; y stays in registers
    const T xk = x[k];
#pragma unroll
    for (int j4 = 0; j4 < kHidden / 4; ++j4) {
      T a0, a1, a2, a3;
      ld4(A + k * kHidden + 4 * j4, a0, a1, a2, a3);
      y[4 * j4] += xk * a0; y[4 * j4 + 1] += xk * a1; y[4 * j4 + 2] += xk * a2; y[4 * j4 + 3] += xk * a3;
    }
  }
}

// Forward: h3 = silu(z3) feeds the last-layer GEMM; the pre-activations z1 | z2 | z3 (192 values) are
// written for the backward pass to zsave[k * zstride], k = 0..191.
template <typename T>
TACE_HD TACE_INLINE void mlp_hidden_fwd(const T (&b)[kNumBessel], const T* __restrict__ A0, const T* __restrict__ A1,
                                   const T* __restrict__ A2, T (&h3)[kHidden], T* __restrict__ zsave, long long zstride) {
  T z[kHidden], h[kHidden];
  matvec64<T, kNumBessel>(b, A0, z);
#pragma unroll
  for (int j = 0; j < kHidden; ++j) { zsave[j * zstride] = z[j]; h[j] = silu_(z[j]); }
  matvec64<T, kHidden>(h, A1, z);
#pragma unroll
  for (int j = 0; j < kHidden; ++j) { zsave[(kHidden + j) * zstride] = z[j]; h[j] = silu_(z[j]); }
  matvec64<T, kHidden>(h, A2, z);
#pragma unroll
  for (int j = 0; j < kHidden; ++j) { zsave[(2 * kHidden + j) * zstride] = z[j]; h3[j] = silu_(z[j]); }
}

// Backward: given dE/dh3 and the saved pre-activations, returns dE/db.
// A1t / A2t are the transposed ([out][in]) copies of A1 / A2; A0 is used as stored.
template <typename T>
TACE_HD TACE_INLINE void mlp_hidden_bwd(const T* __restrict__ zsave, long long zstride, const T* __restrict__ A0, const T* __restrict__ A1t,
                                   const T* __restrict__ A2t, const T (&dh3)[kHidden], T (&db)[kNumBessel]) {
  T dz[kHidden], dh[kHidden];
#pragma unroll
  for (int j = 0; j < kHidden; ++j) dz[j] = dh3[j] * silu_grad_(zsave[(2 * kHidden + j) * zstride]);
  matvec64<T, kHidden>(dz, A2t, dh);
#pragma unroll
  for (int j = 0; j < kHidden; ++j) dz[j] = dh[j] * silu_grad_(zsave[(kHidden + j) * zstride]);
  matvec64<T, kHidden>(dz, A1t, dh);
#pragma unroll
  for (int j = 0; j < kHidden; ++j) dz[j] = dh[j] * silu_grad_(zsave[j * zstride]);
#pragma unroll
  for (int k = 0; k < kNumBessel; ++k) {
    T s = T(0);
#pragma unroll
    for (int j4 = 0; j4 < kHidden / 4; ++j4) {
      T a0, a1, a2, a3;
      ld4(A0 + k * kHidden + 4 * j4, a0, a1, a2, a3);
      s += dz[4 * j4] * a0 + dz[4 * j4 + 1] * a1 + dz[4 * j4 + 2] * a2 + dz[4 * j4 + 3] * a3;
    }
    db[k] = s;
  }
}

// ---- edge geometry ----------------------------------------------------------------
// d = |v| + 1e-9 and n = v / d (tace/models/adapter.py:347, representation.py:321-324).
// Given dE/dd (through the radial basis) and dE/dn (through the angular basis):
//   dE/dv = dd * v/|v| + dn/d - v (v.dn) / (d^2 |v|).
template <typename T>
TACE_HD TACE_INLINE void edge_vector_grad(const T (&v)[3], const T d0, const T d, const T dd, const T (&dn)[3], T (&g)[3]) {
  const T vdn = v[0] * dn[0] + v[1] * dn[1] + v[2] * dn[2];
  const T a = dd / d0 - vdn / (d * d * d0);
  const T inv_d = T(1) / d;
  g[0] = a * v[0] + dn[0] * inv_d;
  g[1] = a * v[1] + dn[1] * inv_d;
  g[2] = a * v[2] + dn[2] * inv_d;
}

}  // namespace tace
