// The TECE edge block (atomic_basis.type = uv_so2): kernels around the SO(2) linears.
//
// Reference: tace/models/_e3nn/archive/oam_2026_07_05.py:547-823 (OAM20260705Convolution), the edge frame of
// tace/models/o2/rotation_matrix.py:74-88, the recursive Wigner matrices of tace/models/o2/wigner.py:231-357 and the
// graph softmax of tace/models/softmax.py:80-114.  Per edge: rotate the features of both ends into the frame whose polar
// (y) axis is the edge, keep the orders |m| <= mmax, weight them with the radial MLP output, run SO(2) linears (GEMMs,
// launched by the engine), gate + edge cluster expansion, attention-weighted inverse rotation and sum per target atom.
//
// Layouts (channel fastest): node features x [N][D][C], D = (L+1)^2; Wigner rows Wg [E][NR][D], NR rows in order-major
// layout (m = 0: l = 0..L | +1: l = 1..L | -1 | +2 | -2); Ks / Qt / Kp / Qp / down [E][NR][C]; Mw [E][NR][2C];
// radial weights W [E][NC][2C]; up [E][G + NF][Ca]; glu, U [E][NF][Ca] with NF = n + 2 n mmax, n = L + 1 (every order
// carries n rows there); coef [E][paths][n][Ca]; logit / alpha [E][H].  Edges are sorted by target (CSR rowptr).
//
// The derivative of the Wigner rows with respect to the edge vector is taken in forward mode (three directional
// derivatives carried through the frame and the recursion), so no hand-derived adjoint of the quaternion blend exists.
#include <cuda_runtime.h>

#include "kernels.h"
#include "tace_common.cuh"
#include "tace_math.cuh"
#include "tp_gen.cuh"

namespace tace {

namespace {

// ---- forward-mode scalar: value and three partial derivatives ------------------------------------
template <typename T>
struct Dual3 {
  T v, d[3];
};
template <typename T> TACE_D TACE_INLINE Dual3<T> mk(T v) { return {v, {T(0), T(0), T(0)}}; }
template <typename T> TACE_D TACE_INLINE Dual3<T> operator+(Dual3<T> a, Dual3<T> b) { return {a.v + b.v, {a.d[0] + b.d[0], a.d[1] + b.d[1], a.d[2] + b.d[2]}}; }
template <typename T> TACE_D TACE_INLINE Dual3<T> operator-(Dual3<T> a, Dual3<T> b) { return {a.v - b.v, {a.d[0] - b.d[0], a.d[1] - b.d[1], a.d[2] - b.d[2]}}; }
template <typename T> TACE_D TACE_INLINE Dual3<T> operator-(Dual3<T> a) { return {-a.v, {-a.d[0], -a.d[1], -a.d[2]}}; }
template <typename T> TACE_D TACE_INLINE Dual3<T> operator*(Dual3<T> a, Dual3<T> b) {
  return {a.v * b.v, {a.d[0] * b.v + a.v * b.d[0], a.d[1] * b.v + a.v * b.d[1], a.d[2] * b.v + a.v * b.d[2]}};
}
template <typename T> TACE_D TACE_INLINE Dual3<T> operator*(T a, Dual3<T> b) { return {a * b.v, {a * b.d[0], a * b.d[1], a * b.d[2]}}; }
template <typename T> TACE_D TACE_INLINE Dual3<T> operator/(Dual3<T> a, Dual3<T> b) {
  const T inv = T(1) / b.v, q = a.v * inv;
  return {q, {(a.d[0] - q * b.d[0]) * inv, (a.d[1] - q * b.d[1]) * inv, (a.d[2] - q * b.d[2]) * inv}};
}
template <typename T> TACE_D TACE_INLINE Dual3<T> dsqrt(Dual3<T> a) {
  const T r = sqrt(a.v), h = T(0.5) / r;
  return {r, {a.d[0] * h, a.d[1] * h, a.d[2] * h}};
}
template <typename T> TACE_D TACE_INLINE Dual3<T> dexp(Dual3<T> a) {
  const T e = exp(a.v);
  return {e, {a.d[0] * e, a.d[1] * e, a.d[2] * e}};
}
// plain scalars take the same code path
template <typename T> TACE_D TACE_INLINE T mkS(T, T v) { return v; }
template <typename T> TACE_D TACE_INLINE Dual3<T> mkS(Dual3<T>, T v) { return mk<T>(v); }
template <typename T> TACE_D TACE_INLINE T val(T a) { return a; }
template <typename T> TACE_D TACE_INLINE T val(Dual3<T> a) { return a.v; }
TACE_D TACE_INLINE float dsqrt(float a) { return sqrtf(a); }
TACE_D TACE_INLINE double dsqrt(double a) { return sqrt(a); }
TACE_D TACE_INLINE float dexp(float a) { return expf(a); }
TACE_D TACE_INLINE double dexp(double a) { return exp(a); }

template <typename T> struct Eps;
template <> struct Eps<float> { static constexpr float v = 1.1920928955078125e-07f; };
template <> struct Eps<double> { static constexpr double v = 2.220446049250313e-16; };

// tace/models/o2/rotation_matrix.py:74-88: rotation R (row-major [9]) that puts the edge on the y axis.  S = T or Dual3<T>.
template <typename T, typename S>
TACE_D void edge_frame(S vx, S vy, S vz, S (&R)[9]) {
  const T e2 = T(1e-7) * T(1e-7);
  const S zero = mkS(vx, T(0)), one = mkS(vx, T(1)), eps2 = mkS(vx, e2);
  const S nv = dsqrt(vx * vx + vy * vy + vz * vz + eps2);
  const S x = vx / nv, y = vy / nv, z = vz / nv;
  S qp[4] = {one + y, -z, zero, x};
  S qn[4] = {-z, one - y, x, zero};
  const S np_ = dsqrt(qp[0] * qp[0] + qp[1] * qp[1] + qp[2] * qp[2] + qp[3] * qp[3] + eps2);
  const S nn = dsqrt(qn[0] * qn[0] + qn[1] * qn[1] + qn[2] * qn[2] + qn[3] * qn[3] + eps2);
  for (int k = 0; k < 4; ++k) { qp[k] = qp[k] / np_; qn[k] = qn[k] / nn; }
  // C-infinity step in t = (y + 1) / 2 (rotation_matrix.py:25-36); outside (0, 1) it is constant
  const S t = T(0.5) * (y + one);
  S blend;
  if (val(t) <= T(0)) blend = zero;
  else if (val(t) >= T(1)) blend = one;
  else {
    const T eps = Eps<T>::v;
    const S tl = val(t) < eps ? mkS(vx, eps) : t;
    const S tr = val(one - t) < eps ? mkS(vx, eps) : one - t;
    const S left = dexp(-(one / tl)), right = dexp(-(one / tr));
    blend = left / (left + right);
  }
  S dot = qn[0] * qp[0] + qn[1] * qp[1] + qn[2] * qp[2] + qn[3] * qp[3];
  const bool flip = val(dot) < T(0);
  S q[4];
  for (int k = 0; k < 4; ++k) q[k] = (one - blend) * qn[k] + blend * (flip ? -qp[k] : qp[k]);
  const S nq = dsqrt(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3] + eps2);
  for (int k = 0; k < 4; ++k) q[k] = q[k] / nq;
  const S w = q[0], a = q[1], b = q[2], c = q[3];
  const S two = mkS(vx, T(2));
  R[0] = one - two * (b * b + c * c); R[1] = two * (a * b - w * c); R[2] = two * (a * c + w * b);
  R[3] = two * (a * b + w * c); R[4] = one - two * (a * a + c * c); R[5] = two * (b * c - w * a);
  R[6] = two * (a * c - w * b); R[7] = two * (b * c + w * a); R[8] = one - two * (a * a + b * b);
}

// blocks D^0..D^L of the rotation (wigner.py:316-357), D^l stored row-major at offset sum_{k<l} (2k+1)^2 of `blocks`
// (1 + 9 + 25 + 49 = 84 entries for L = 3)
template <typename T, typename S>
TACE_D void wigner_blocks(const S (&R)[9], int L, S* blocks) {
  blocks[0] = mkS(R[0], T(1));
  if (L >= 1) for (int k = 0; k < 9; ++k) blocks[1 + k] = R[k];
  int off_prev = 1, off = 10;
  for (int l = 2; l <= L; ++l) {
    const double* cg = (l == 2) ? w3j_1_1_2 : w3j_1_2_3;  // [3][2l-1][2l+1]
    const int dp = 2 * l - 1, dl = 2 * l + 1;
    // left[b][m][c] = sum_a cg[a][b][m] R[a][c]; then tmp[m][c][d] = sum_b left[b][m][c] Dprev[b][d]; D[m][n] = sum_cd tmp cg[c][d][n]
    for (int m = 0; m < dl; ++m)
      for (int n = 0; n < dl; ++n) {
        S acc = mkS(R[0], T(0));
        for (int c = 0; c < 3; ++c)
          for (int d = 0; d < dp; ++d) {
            const T cr = T(cg[(c * dp + d) * dl + n]);
            if (cr == T(0)) continue;
            S t = mkS(R[0], T(0));
            for (int a = 0; a < 3; ++a)
              for (int b = 0; b < dp; ++b) {
                const T cl = T(cg[(a * dp + b) * dl + m]);
                if (cl == T(0)) continue;
                t = t + cl * (R[a * 3 + c] * blocks[off_prev + b * dp + d]);
              }
            acc = acc + cr * t;
          }
        blocks[off + m * dl + n] = T(dl) * acc;
      }
    off_prev = off;
    off += dl * dl;
  }
}

TACE_D TACE_INLINE int block_offset(int l) { return l == 0 ? 0 : l == 1 ? 1 : l == 2 ? 10 : 35; }

template <typename T>
TACE_D TACE_INLINE T act_eval(int kind, T x) { return kind == 0 ? T(1.8467055342154763) * sigmoid_(x) : T(1.6791767923989418) * silu_(x); }
template <typename T>
TACE_D TACE_INLINE T act_grad(int kind, T x) {
  if (kind == 0) { const T s = sigmoid_(x); return T(1.8467055342154763) * s * (T(1) - s); }
  return T(1.6791767923989418) * silu_grad_(x);
}

// ---- K0: Wigner rows of every edge ---------------------------------------------------------------
template <typename T>
__global__ void tece_wigner_kernel(const TeceArgs<T> a) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  T R[9], blocks[84];
  edge_frame<T, T>(a.vec[3 * e], a.vec[3 * e + 1], a.vec[3 * e + 2], R);
  wigner_blocks<T, T>(R, a.L, blocks);
  const int D = (a.L + 1) * (a.L + 1);
  T* out = a.Wg + e * a.NR * D;
  for (int r = 0; r < a.NR; ++r) {
    const int l = a.row_l[r], m = a.row_m[r], dl = 2 * l + 1;
    for (int j = 0; j < D; ++j) out[r * D + j] = T(0);
    for (int j = 0; j < dl; ++j) out[r * D + l * l + j] = blocks[block_offset(l) + (l + m) * dl + j];
  }
}
// gvec[e][k] (+)= sum_{r, j} gWg[e][r][j] dWg[e][r][j] / dv_k
template <typename T>
__global__ void tece_wigner_bwd_kernel(const TeceArgs<T> a, int accumulate) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  typedef Dual3<T> S;
  S R[9], blocks[84];
  S vx = {a.vec[3 * e], {T(1), T(0), T(0)}}, vy = {a.vec[3 * e + 1], {T(0), T(1), T(0)}}, vz = {a.vec[3 * e + 2], {T(0), T(0), T(1)}};
  edge_frame<T, S>(vx, vy, vz, R);
  wigner_blocks<T, S>(R, a.L, blocks);
  const int D = (a.L + 1) * (a.L + 1);
  const T* g = a.gWg + e * a.NR * D;
  T acc[3] = {T(0), T(0), T(0)};
  for (int r = 0; r < a.NR; ++r) {
    const int l = a.row_l[r], m = a.row_m[r], dl = 2 * l + 1;
    for (int j = 0; j < dl; ++j) {
      const S& d = blocks[block_offset(l) + (l + m) * dl + j];
      const T gv = g[r * D + l * l + j];
      acc[0] += gv * d.d[0]; acc[1] += gv * d.d[1]; acc[2] += gv * d.d[2];
    }
  }
  for (int k = 0; k < 3; ++k) a.gvec[3 * e + k] = accumulate ? a.gvec[3 * e + k] + acc[k] : acc[k];
}

// ---- K1: rotate both ends into the edge frame, radial weighting ------------------------------------
template <typename T>
__global__ void tece_rotate_in_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.C) return;
  const long long e = idx / a.C;
  const int c = (int)(idx - e * a.C), C = a.C, D = (a.L + 1) * (a.L + 1);
  const T* xs = a.x + (long long)a.e_src[e] * D * C + c;
  const T* xt = a.x + (long long)a.e_dst[e] * D * C + c;
  const T* Wg = a.Wg + e * a.NR * D;
  const T* W = a.W + e * a.NC * 2 * C;
  for (int r = 0; r < a.NR; ++r) {
    const int l = a.row_l[r], dl = 2 * l + 1;
    T ks = T(0), qt = T(0);
    for (int j = 0; j < dl; ++j) {
      const T wv = Wg[r * D + l * l + j];
      ks += wv * xs[(long long)(l * l + j) * C];
      qt += wv * xt[(long long)(l * l + j) * C];
    }
    a.Ks[(e * a.NR + r) * C + c] = ks;
    a.Qt[(e * a.NR + r) * C + c] = qt;
    const int comp = a.row_comp[r];
    a.Mw[(e * a.NR + r) * 2 * C + c] = W[comp * 2 * C + c] * ks;
    a.Mw[(e * a.NR + r) * 2 * C + C + c] = W[comp * 2 * C + C + c] * qt;
  }
}
// backward of K1: gKs / gQt hold the gradients that came through the key / query projections; gMw the one through the
// weighted features.  Writes dW (radial-weight gradient, over W), the per-edge source rows dxe [E][D][C] and the per-edge
// target rows dxt [E][D][C] (summed per atom afterwards).
template <typename T>
__global__ void tece_rotate_in_bwd_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.C) return;
  const long long e = idx / a.C;
  const int c = (int)(idx - e * a.C), C = a.C, D = (a.L + 1) * (a.L + 1);
  const T* Wg = a.Wg + e * a.NR * D;
  T* W = a.W + e * a.NC * 2 * C;
  T gs[16], gt[16], dws[9], dwt[9], ws[9], wt[9];
  for (int j = 0; j < D; ++j) { gs[j] = T(0); gt[j] = T(0); }
  for (int k = 0; k < a.NC; ++k) { dws[k] = T(0); dwt[k] = T(0); ws[k] = W[k * 2 * C + c]; wt[k] = W[k * 2 * C + C + c]; }
  for (int r = 0; r < a.NR; ++r) {
    const int l = a.row_l[r], dl = 2 * l + 1, comp = a.row_comp[r];
    const long long at = (e * a.NR + r);
    const T gms = a.gMw[at * 2 * C + c], gmt = a.gMw[at * 2 * C + C + c];
    dws[comp] += gms * a.Ks[at * C + c];
    dwt[comp] += gmt * a.Qt[at * C + c];
    const T gks = a.gKs[at * C + c] + ws[comp] * gms;
    const T gqt = a.gQt[at * C + c] + wt[comp] * gmt;
    a.gKs[at * C + c] = gks;  // totals, read again by the Wigner-gradient kernel
    a.gQt[at * C + c] = gqt;
    for (int j = 0; j < dl; ++j) {
      const T wv = Wg[r * D + l * l + j];
      gs[l * l + j] += wv * gks;
      gt[l * l + j] += wv * gqt;
    }
  }
  for (int k = 0; k < a.NC; ++k) { W[k * 2 * C + c] = dws[k]; W[k * 2 * C + C + c] = dwt[k]; }
  for (int j = 0; j < D; ++j) { a.dxe[(e * D + j) * C + c] = gs[j]; a.dxt[(e * D + j) * C + c] = gt[j]; }
}
// gx[i][j][c] += sum over the edges into i of dxt[e][j][c]
template <typename T>
__global__ void tece_target_sum_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int D = (a.L + 1) * (a.L + 1);
  if (idx >= (long long)a.n_local * D * a.C) return;
  const long long i = idx / ((long long)D * a.C);
  const long long jc = idx - i * D * a.C;
  T acc = T(0);
  for (int e = a.rowptr[i]; e < a.rowptr[i + 1]; ++e) acc += a.dxt[(long long)e * D * a.C + jc];
  a.gx[idx] += acc;
}

// ---- the rotation kernels with rank and order limits known at compile time -------------------------------------
// for_rows visits the order-major rows with constant (row, rank, weight component) after unrolling, so the per-thread
// arrays of the kernels below are indexed statically and stay in registers.
template <int L, int MM, typename F>
TACE_D TACE_INLINE void for_rows(F&& f) {
  int r = 0, comp0 = 0;
#pragma unroll
  for (int m = 0; m <= MM; ++m) {
#pragma unroll
    for (int part = 0; part < (m ? 2 : 1); ++part)
#pragma unroll
      for (int l = m; l <= L; ++l) { f(r, l, comp0 + l - m); ++r; }
    comp0 += L + 1 - m;
  }
}
template <int L, int MM> struct RowCount { static constexpr int NR = (L + 1) + (MM >= 1 ? 2 * L : 0) + (MM >= 2 ? 2 * (L - 1) : 0); };

template <typename T, int L, int MM>
__global__ void __launch_bounds__(128) tece_rotate_in_t_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.C) return;
  const long long e = idx / a.C;
  constexpr int D = (L + 1) * (L + 1), NR = RowCount<L, MM>::NR;
  const int c = (int)(idx - e * a.C), C = a.C;
  const T* xs = a.x + (long long)a.e_src[e] * D * C + c;
  const T* xt = a.x + (long long)a.e_dst[e] * D * C + c;
  const T* __restrict__ Wg = a.Wg + e * NR * D;
  const T* __restrict__ W = a.W + e * a.NC * 2 * C;
  T vs[D], vt[D];
#pragma unroll
  for (int j = 0; j < D; ++j) { vs[j] = xs[(long long)j * C]; vt[j] = xt[(long long)j * C]; }
  for_rows<L, MM>([&](int r, int l, int comp) {
    T ks = T(0), qt = T(0);
#pragma unroll
    for (int j = 0; j < 2 * l + 1; ++j) {
      const T wv = Wg[r * D + l * l + j];
      ks += wv * vs[l * l + j];
      qt += wv * vt[l * l + j];
    }
    a.Ks[(e * NR + r) * C + c] = ks;
    a.Qt[(e * NR + r) * C + c] = qt;
    a.Mw[(e * NR + r) * 2 * C + c] = W[comp * 2 * C + c] * ks;
    a.Mw[(e * NR + r) * 2 * C + C + c] = W[comp * 2 * C + C + c] * qt;
  });
}
template <typename T, int L, int MM>
__global__ void __launch_bounds__(128) tece_rotate_in_bwd_t_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.C) return;
  const long long e = idx / a.C;
  constexpr int D = (L + 1) * (L + 1), NR = RowCount<L, MM>::NR, NC = (L + 1) + (MM >= 1 ? L : 0) + (MM >= 2 ? L - 1 : 0);
  const int c = (int)(idx - e * a.C), C = a.C;
  const T* __restrict__ Wg = a.Wg + e * NR * D;
  T* W = a.W + e * NC * 2 * C;
  T gs[D], gt[D], dws[NC], dwt[NC], ws[NC], wt[NC];
#pragma unroll
  for (int j = 0; j < D; ++j) { gs[j] = T(0); gt[j] = T(0); }
#pragma unroll
  for (int k = 0; k < NC; ++k) { dws[k] = T(0); dwt[k] = T(0); ws[k] = W[k * 2 * C + c]; wt[k] = W[k * 2 * C + C + c]; }
  // read-only inputs through restrict pointers: the stores of the totals below must not hold back the next rows' loads
  const T* __restrict__ gMw = a.gMw;
  const T* __restrict__ Ksp = a.Ks;
  const T* __restrict__ Qtp = a.Qt;
  for_rows<L, MM>([&](int r, int l, int comp) {
    const long long at = (e * NR + r);
    const T gms = gMw[at * 2 * C + c], gmt = gMw[at * 2 * C + C + c];
    dws[comp] += gms * Ksp[at * C + c];
    dwt[comp] += gmt * Qtp[at * C + c];
    const T gks = a.gKs[at * C + c] + ws[comp] * gms;
    const T gqt = a.gQt[at * C + c] + wt[comp] * gmt;
    a.gKs[at * C + c] = gks;
    a.gQt[at * C + c] = gqt;
#pragma unroll
    for (int j = 0; j < 2 * l + 1; ++j) {
      const T wv = Wg[r * D + l * l + j];
      gs[l * l + j] += wv * gks;
      gt[l * l + j] += wv * gqt;
    }
  });
#pragma unroll
  for (int k = 0; k < NC; ++k) { W[k * 2 * C + c] = dws[k]; W[k * 2 * C + C + c] = dwt[k]; }
#pragma unroll
  for (int j = 0; j < D; ++j) { a.dxe[(e * D + j) * C + c] = gs[j]; a.dxt[(e * D + j) * C + c] = gt[j]; }
}
template <typename T, int L, int MM>
__global__ void __launch_bounds__(128) tece_rotate_out_t_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)a.n_local * a.C) return;
  const long long i = idx / a.C;
  constexpr int D = (L + 1) * (L + 1), NR = RowCount<L, MM>::NR;
  const int c = (int)(idx - i * a.C), C = a.C, h = c / (C / a.H);
  T acc[D];
#pragma unroll
  for (int j = 0; j < D; ++j) acc[j] = T(0);
  for (int e = a.rowptr[i]; e < a.rowptr[i + 1]; ++e) {
    const T al = a.alpha[(long long)e * a.H + h];
    const T* Wg = a.Wg + (long long)e * NR * D;
    const T* dn = a.down + (long long)e * NR * C + c;
    for_rows<L, MM>([&](int r, int l, int) {
      const T v = al * a.row_scale[r] * dn[(long long)r * C];
#pragma unroll
      for (int j = 0; j < 2 * l + 1; ++j) acc[l * l + j] += Wg[r * D + l * l + j] * v;
    });
  }
#pragma unroll
  for (int j = 0; j < D; ++j) a.M[(i * D + j) * C + c] = acc[j];
}
// Wigner-row gradient, one warp per edge (see tece_wigner_grad_kernel below), with static shapes
template <typename T, int L, int MM>
__global__ void __launch_bounds__(128) tece_wigner_grad_t_kernel(const TeceArgs<T> a) {
  const int lane = threadIdx.x & 31;
  const long long e = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (e >= a.E) return;
  constexpr int D = (L + 1) * (L + 1), NR = RowCount<L, MM>::NR;
  constexpr int NE = D + (MM >= 1 ? 2 * (D - 1) : 0) + (MM >= 2 ? 2 * (D - 4) : 0);  // block entries of all rows
  const int C = a.C, Ch = C / a.H;
  T acc[NE];
#pragma unroll
  for (int k = 0; k < NE; ++k) acc[k] = T(0);
  const T* xs = a.x + (long long)a.e_src[e] * D * C;
  const T* xt = a.x + (long long)a.e_dst[e] * D * C;
  const T* gM = a.gM + (long long)a.e_dst[e] * D * C;
  for (int c = lane; c < C; c += 32) {
    const T al = a.alpha[e * a.H + c / Ch];
    T vs[D], vt[D], vg[D];
#pragma unroll
    for (int j = 0; j < D; ++j) { vs[j] = xs[(long long)j * C + c]; vt[j] = xt[(long long)j * C + c]; vg[j] = al * gM[(long long)j * C + c]; }
    int k = 0;
    for_rows<L, MM>([&](int r, int l, int) {
      const long long at = (e * NR + r) * C + c;
      const T gk = a.gKs[at], gq = a.gQt[at], dn = a.row_scale[r] * a.down[at];
#pragma unroll
      for (int j = 0; j < 2 * l + 1; ++j, ++k) acc[k] += gk * vs[l * l + j] + gq * vt[l * l + j] + dn * vg[l * l + j];
    });
  }
  T* out = a.gWg + e * NR * D;
  int k = 0;
  for_rows<L, MM>([&](int r, int l, int) {
#pragma unroll
    for (int j = 0; j < 2 * l + 1; ++j, ++k) {
      T v = acc[k];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) out[r * D + l * l + j] = v;
    }
  });
}
#define TECE_LM_DISPATCH(KERNEL, GRID, BLOCK)                                              \
  (a.L == 2 && a.mmax == 1   ? (KERNEL<T, 2, 1><<<GRID, BLOCK, 0, s>>>(a), true)          \
   : a.L == 2 && a.mmax == 2 ? (KERNEL<T, 2, 2><<<GRID, BLOCK, 0, s>>>(a), true)          \
   : a.L == 3 && a.mmax == 1 ? (KERNEL<T, 3, 1><<<GRID, BLOCK, 0, s>>>(a), true)          \
   : a.L == 3 && a.mmax == 2 ? (KERNEL<T, 3, 2><<<GRID, BLOCK, 0, s>>>(a), true)          \
                             : false)

// ---- K3: attention logits ---------------------------------------------------------------------------
template <typename T>
TACE_D void radial_projection(const TeceArgs<T>& a, T d, T* proj, T* dproj) {  // proj[2H], dproj = d proj / d d (or nullptr)
  T b[kNumBessel], db[kNumBessel];
  radial_eval<T>(d, a.rp, b, db);
  for (int j = 0; j < 2 * a.H; ++j) {
    T v = a.rproj_b[j], dv = T(0);
    for (int k = 0; k < kNumBessel; ++k) { v += b[k] * a.rproj_w[k * 2 * a.H + j]; dv += db[k] * a.rproj_w[k * 2 * a.H + j]; }
    proj[j] = v;
    if (dproj) dproj[j] = dv;
  }
}
template <typename T>
__global__ void tece_logit_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.H) return;
  const long long e = idx / a.H;
  const int h = (int)(idx - e * a.H), C = a.C, Ch = C / a.H, n0 = a.L + 1;
  T proj[32];
  radial_projection(a, a.dlen[e], proj, (T*)nullptr);
  const T phase = T(3.141592653589793) * tanh(proj[a.H + h]);
  const T* q = a.Qp + e * a.NR * C + h * Ch;
  const T* k = a.Kp + e * a.NR * C + h * Ch;
  T score = T(0);
  for (int r = 0; r < n0; ++r)
    for (int u = 0; u < Ch; ++u) score += q[r * C + u] * k[r * C + u];
  int off = n0;
  for (int m = 1; m <= a.mmax; ++m) {
    const int n = a.L + 1 - m;
    const T cs = cos(T(m) * phase), sn = sin(T(m) * phase);
    for (int r = 0; r < n; ++r)
      for (int u = 0; u < Ch; ++u) {
        const T kr = k[(off + r) * C + u], ki = k[(off + n + r) * C + u];
        score += q[(off + r) * C + u] * (cs * kr - sn * ki) + q[(off + n + r) * C + u] * (sn * kr + cs * ki);
      }
    off += 2 * n;
  }
  a.logit[idx] = score * a.temp[h] + proj[h];
}
// gQp / gKp from glogit; gproj[e][2H] = d E / d (radial projection)
template <typename T>
__global__ void tece_logit_bwd_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.H) return;
  const long long e = idx / a.H;
  const int h = (int)(idx - e * a.H), C = a.C, Ch = C / a.H, n0 = a.L + 1;
  T proj[32];
  radial_projection(a, a.dlen[e], proj, (T*)nullptr);
  const T th = tanh(proj[a.H + h]);
  const T phase = T(3.141592653589793) * th;
  const T gl = a.glogit[idx], gs = gl * a.temp[h];
  const T* q = a.Qp + e * a.NR * C + h * Ch;
  const T* k = a.Kp + e * a.NR * C + h * Ch;
  T* gq = a.gQp + e * a.NR * C + h * Ch;
  T* gk = a.gKp + e * a.NR * C + h * Ch;
  for (int r = 0; r < n0; ++r)
    for (int u = 0; u < Ch; ++u) { gq[r * C + u] = gs * k[r * C + u]; gk[r * C + u] = gs * q[r * C + u]; }
  int off = n0;
  T gphase = T(0);
  for (int m = 1; m <= a.mmax; ++m) {
    const int n = a.L + 1 - m;
    const T cs = cos(T(m) * phase), sn = sin(T(m) * phase);
    for (int r = 0; r < n; ++r)
      for (int u = 0; u < Ch; ++u) {
        const int ir = (off + r) * C + u, ii = (off + n + r) * C + u;
        const T kr = k[ir], ki = k[ii], qr = q[ir], qi = q[ii];
        gq[ir] = gs * (cs * kr - sn * ki);
        gq[ii] = gs * (sn * kr + cs * ki);
        gk[ir] = gs * (cs * qr + sn * qi);
        gk[ii] = gs * (-sn * qr + cs * qi);
        // d score / d (m phase) = qr (-sn kr - cs ki) + qi (cs kr - sn ki)
        gphase += gs * T(m) * (qr * (-sn * kr - cs * ki) + qi * (cs * kr - sn * ki));
      }
    off += 2 * n;
  }
  a.gproj[e * 2 * a.H + h] = gl;
  a.gproj[e * 2 * a.H + a.H + h] = gphase * T(3.141592653589793) * (T(1) - th * th);
}
// Lane-per-channel forms of the two kernels above, for head widths that are a power of two <= 32: thread (e, c) handles the
// channel's share of the dot products (contiguous loads), the head's lanes reduce with shuffles, the radial projection is
// read from proj [E][2H] (tece_proj_kernel).
template <typename T>
__global__ void tece_proj_kernel(const TeceArgs<T> a) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  T proj[32];
  radial_projection(a, a.dlen[e], proj, (T*)nullptr);
  for (int j = 0; j < 2 * a.H; ++j) a.proj[e * 2 * a.H + j] = proj[j];
}
template <typename T, bool BWD>
__global__ void tece_logit_lane_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.C) return;
  const long long e = idx / a.C;
  const int c = (int)(idx - e * a.C), C = a.C, Ch = C / a.H, h = c / Ch, n0 = a.L + 1;
  const T th = tanh(a.proj[e * 2 * a.H + a.H + h]);
  const T phase = T(3.141592653589793) * th;
  const T* __restrict__ q = a.Qp + e * a.NR * C + c;
  const T* __restrict__ k = a.Kp + e * a.NR * C + c;
  T gs = T(0);
  T* gq = nullptr; T* gk = nullptr;
  if (BWD) { gs = a.glogit[e * a.H + h] * a.temp[h]; gq = a.gQp + e * a.NR * C + c; gk = a.gKp + e * a.NR * C + c; }
  T part = T(0);  // forward: the channel's share of the score; backward: of d score / d phase
  for (int r = 0; r < n0; ++r) {
    if (!BWD) part += q[r * C] * k[r * C];
    else { gq[r * C] = gs * k[r * C]; gk[r * C] = gs * q[r * C]; }
  }
  int off = n0;
  for (int m = 1; m <= a.mmax; ++m) {
    const int n = a.L + 1 - m;
    const T cs = cos(T(m) * phase), sn = sin(T(m) * phase);
    for (int r = 0; r < n; ++r) {
      const int ir = (off + r) * C, ii = (off + n + r) * C;
      const T kr = k[ir], ki = k[ii], qr = q[ir], qi = q[ii];
      if (!BWD) part += qr * (cs * kr - sn * ki) + qi * (sn * kr + cs * ki);
      else {
        gq[ir] = gs * (cs * kr - sn * ki);
        gq[ii] = gs * (sn * kr + cs * ki);
        gk[ir] = gs * (cs * qr + sn * qi);
        gk[ii] = gs * (-sn * qr + cs * qi);
        part += gs * T(m) * (qr * (-sn * kr - cs * ki) + qi * (cs * kr - sn * ki));
      }
    }
    off += 2 * n;
  }
  for (int o = Ch >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (c % Ch == 0) {
    if (!BWD) a.logit[e * a.H + h] = part * a.temp[h] + a.proj[e * 2 * a.H + h];
    else {
      a.gproj[e * 2 * a.H + h] = a.glogit[e * a.H + h];
      a.gproj[e * 2 * a.H + a.H + h] = part * T(3.141592653589793) * (T(1) - th * th);
    }
  }
}
// ddlen_extra[e] = sum_j gproj[e][j] d proj_j / d d + gcut[e] d envelope / d d
template <typename T>
__global__ void tece_edge_scalar_bwd_kernel(const TeceArgs<T> a) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  T proj[32], dproj[32];
  radial_projection(a, a.dlen[e], proj, dproj);
  T acc = T(0);
  for (int j = 0; j < 2 * a.H; ++j) acc += a.gproj[e * 2 * a.H + j] * dproj[j];
  if (a.env) {
    T gc = T(0);
    for (int h = 0; h < a.H; ++h) gc += a.gcut[e * a.H + h];
    T u, du;
    envelope_eval<T>(a.dlen[e], a.rp, u, du);
    acc += gc * du;
  }
  a.ddlen_extra[e] = acc;
}

// ---- K4: softmax over the edges into one atom, per head (softmax.py:97-112) --------------------------
template <typename T>
__global__ void tece_softmax_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)a.n_local * a.H) return;
  const long long i = idx / a.H;
  const int h = (int)(idx - i * a.H);
  const int e0 = a.rowptr[i], e1 = a.rowptr[i + 1];
  if (e0 == e1) return;
  T mx = a.logit[(long long)e0 * a.H + h];
  for (int e = e0 + 1; e < e1; ++e) mx = fmax(mx, a.logit[(long long)e * a.H + h]);
  T sum = T(0);
  for (int e = e0; e < e1; ++e) sum += exp(a.logit[(long long)e * a.H + h] - mx) * (a.env ? a.env[e] : T(1));
  const T inv = T(1) / (sum + T(1e-16));
  for (int e = e0; e < e1; ++e) {
    const T cut = a.env ? a.env[e] : T(1);
    a.alpha[(long long)e * a.H + h] = exp(a.logit[(long long)e * a.H + h] - mx) * cut * inv * cut;
  }
}
// galpha -> glogit, gcut.  alpha = s cut, s = p / (S + eps), p = exp(l - max) cut
template <typename T>
__global__ void tece_softmax_bwd_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)a.n_local * a.H) return;
  const long long i = idx / a.H;
  const int h = (int)(idx - i * a.H);
  const int e0 = a.rowptr[i], e1 = a.rowptr[i + 1];
  if (e0 == e1) return;
  T mx = a.logit[(long long)e0 * a.H + h];
  for (int e = e0 + 1; e < e1; ++e) mx = fmax(mx, a.logit[(long long)e * a.H + h]);
  T sum = T(0);
  for (int e = e0; e < e1; ++e) sum += exp(a.logit[(long long)e * a.H + h] - mx) * (a.env ? a.env[e] : T(1));
  const T inv = T(1) / (sum + T(1e-16));
  T dot = T(0);  // sum_k s_k g_k with g_k = galpha_k cut_k
  for (int e = e0; e < e1; ++e) {
    const T cut = a.env ? a.env[e] : T(1);
    const T s = exp(a.logit[(long long)e * a.H + h] - mx) * cut * inv;
    dot += s * a.galpha[(long long)e * a.H + h] * cut;
  }
  for (int e = e0; e < e1; ++e) {
    const T cut = a.env ? a.env[e] : T(1);
    const T ex = exp(a.logit[(long long)e * a.H + h] - mx) * inv;  // s / cut
    const T s = ex * cut;
    const T g = a.galpha[(long long)e * a.H + h] * cut;
    a.glogit[(long long)e * a.H + h] = s * (g - dot);
    if (a.env) a.gcut[(long long)e * a.H + h] = a.galpha[(long long)e * a.H + h] * s + ex * (g - dot);
  }
}

// ---- K5: gate + edge cluster expansion on the SO(2) features ------------------------------------------
// rows of the full layout: order 0 rows [0, n); order m >= 1 real rows [n + (m-1) 2n, +n), imaginary rows the next n
template <typename T>
TACE_D TACE_INLINE int full_re(int n, int m) { return m == 0 ? 0 : n + (m - 1) * 2 * n; }

template <typename T, bool BWD>
__global__ void tece_mix_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.Ca) return;
  const long long e = idx / a.Ca;
  const int ca = (int)(idx - e * a.Ca), Ca = a.Ca, n = a.L + 1, NF = n + 2 * n * a.mmax, G = a.G;
  constexpr int MAXF = 20, MAXG = 12, MAXW = 28;  // L <= 3, mmax <= 2
  T x[MAXF], y[MAXF], gz[MAXG], cz[MAXW], out[MAXF];
  const T* up = a.up + e * (long long)(G + NF) * Ca + ca;
  const T* glu = a.glu + e * (long long)NF * Ca + ca;
  const T* cf = a.coefZ + e * (long long)a.n_paths * n * Ca + ca;
  for (int r = 0; r < G; ++r) gz[r] = up[(long long)r * Ca];
  for (int r = 0; r < NF; ++r) { x[r] = up[(long long)(G + r) * Ca]; y[r] = glu[(long long)r * Ca]; out[r] = x[r]; }
  for (int k = 0; k < a.n_paths * n; ++k) cz[k] = cf[(long long)k * Ca];
  T gx[MAXF], gy[MAXF], gg[MAXG], gc[MAXW], go[MAXF];
  if (BWD) {
    const T* gU = a.gU + e * (long long)NF * Ca + ca;
    for (int r = 0; r < NF; ++r) { go[r] = gU[(long long)r * Ca]; gx[r] = go[r]; gy[r] = T(0); }
    for (int r = 0; r < G; ++r) gg[r] = T(0);
    for (int k = 0; k < a.n_paths * n; ++k) gc[k] = T(0);
  }
  // gate (oam_2026_07_05.py:301-309, channel-wise layout): order m row i is scaled by act(gate[(m - start) n + i])
  const int start = a.gate_m0 ? 0 : 1;
  for (int m = 0; m <= a.mmax; ++m) {
    for (int part = 0; part < (m == 0 ? 1 : 2); ++part)
      for (int i = 0; i < n; ++i) {
        const int r = full_re<T>(n, m) + part * n + i;
        if (m == 0 && !a.gate_m0) {
          out[r] += act_eval<T>(a.act, x[r]);
          if (BWD) gx[r] += go[r] * act_grad<T>(a.act, x[r]);
        } else {
          const int g = (m - start) * n + i;
          out[r] += act_eval<T>(a.act, gz[g]) * x[r];
          if (BWD) { gx[r] += go[r] * act_eval<T>(a.act, gz[g]); gg[g] += go[r] * x[r] * act_grad<T>(a.act, gz[g]); }
        }
      }
  }
  // cluster expansion (oam_2026_07_05.py:417-488): channel-wise products of the complex order components
  for (int p = 0; p < a.n_paths; ++p) {
    const int m1 = a.p_m1[p], m2 = a.p_m2[p], m3 = a.p_m3[p], sum_mode = a.p_sum[p];
    const T sc = a.p_scale[p];
    const int x_re = full_re<T>(n, m1), y_re = full_re<T>(n, m2), o_re = full_re<T>(n, m3);
    for (int i = 0; i < n; ++i) {
      const T w = act_eval<T>(a.act, cz[p * n + i]) * sc;
      const T xr = x[x_re + i], xi = m1 ? x[x_re + n + i] : T(0);
      const T yr = y[y_re + i], yi = m2 ? y[y_re + n + i] : T(0);
      T zr, zi;
      if (sum_mode) { zr = xr * yr - xi * yi; zi = xr * yi + xi * yr; }
      else { zr = xr * yr + xi * yi; zi = xi * yr - xr * yi; }
      out[o_re + i] += w * zr;
      if (m3) out[o_re + n + i] += w * zi;
      if (BWD) {
        const T gr = go[o_re + i], gi = m3 ? go[o_re + n + i] : T(0);
        gc[p * n + i] += (gr * zr + gi * zi) * sc * act_grad<T>(a.act, cz[p * n + i]);
        const T ar = w * gr, ai = w * gi;  // gradient of (zr, zi)
        if (sum_mode) {
          gx[x_re + i] += ar * yr + ai * yi;
          if (m1) gx[x_re + n + i] += -ar * yi + ai * yr;
          gy[y_re + i] += ar * xr + ai * xi;
          if (m2) gy[y_re + n + i] += -ar * xi + ai * xr;
        } else {
          gx[x_re + i] += ar * yr - ai * yi;
          if (m1) gx[x_re + n + i] += ar * yi + ai * yr;
          gy[y_re + i] += ar * xr + ai * xi;
          if (m2) gy[y_re + n + i] += ar * xi - ai * xr;
        }
      }
    }
  }
  if (!BWD) {
    T* U = a.U + e * (long long)NF * Ca + ca;
    for (int r = 0; r < NF; ++r) U[(long long)r * Ca] = out[r];
  } else {
    T* gup = a.gup + e * (long long)(G + NF) * Ca + ca;
    T* gglu = a.gglu + e * (long long)NF * Ca + ca;
    T* gcf = a.gcoefZ + e * (long long)a.n_paths * n * Ca + ca;
    for (int r = 0; r < G; ++r) gup[(long long)r * Ca] = gg[r];
    for (int r = 0; r < NF; ++r) { gup[(long long)(G + r) * Ca] = gx[r]; gglu[(long long)r * Ca] = gy[r]; }
    for (int k = 0; k < a.n_paths * n; ++k) gcf[(long long)k * Ca] = gc[k];
  }
}

// The same kernel with rows per order, orders and gate layout known at compile time: every array index below is a constant
// after unrolling, so the ~150 per-thread values live in registers instead of local memory.
TACE_HD constexpr int mix_path_id(int mm, int m3, int m1, int m2) {  // position of path (m1, m2) -> m3 in the output-order-major list
  int p = 0;
  for (int q3 = 0; q3 <= mm; ++q3)
    for (int q1 = 0; q1 <= mm; ++q1)
      for (int q2 = 0; q2 <= q1; ++q2) {
        if (!(q1 + q2 == q3 || q1 - q2 == q3)) continue;
        if (q3 == m3 && q1 == m1 && q2 == m2) return p;
        ++p;
      }
  return -1;
}
TACE_HD constexpr int mix_path_count(int mm) {
  int p = 0;
  for (int q3 = 0; q3 <= mm; ++q3)
    for (int q1 = 0; q1 <= mm; ++q1)
      for (int q2 = 0; q2 <= q1; ++q2)
        if (q1 + q2 == q3 || q1 - q2 == q3) ++p;
  return p;
}
template <typename T, int N, int MM, bool GATE_M0, bool BWD>
__global__ void __launch_bounds__(64) tece_mix_t_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.Ca) return;
  const long long e = idx / a.Ca;
  const int ca = (int)(idx - e * a.Ca), Ca = a.Ca;
  constexpr int NF = N + 2 * N * MM, G = N * (MM + (GATE_M0 ? 1 : 0));
  constexpr int START = GATE_M0 ? 0 : 1;
  T x[NF], y[NF], gz[G > 0 ? G : 1], out[NF];
  const T* up = a.up + e * (long long)(G + NF) * Ca + ca;
  const T* glu = a.glu + e * (long long)NF * Ca + ca;
  const T* cf = a.coefZ + e * (long long)a.n_paths * N * Ca + ca;
#pragma unroll
  for (int r = 0; r < G; ++r) gz[r] = up[(long long)r * Ca];
#pragma unroll
  for (int r = 0; r < NF; ++r) { x[r] = up[(long long)(G + r) * Ca]; y[r] = glu[(long long)r * Ca]; out[r] = x[r]; }
  // every input is in registers before the first store: the gradients overwrite their forward buffers, so a load issued
  // after a store would have to wait for it
  constexpr int NW = mix_path_count(MM) * N;
  T cz[NW];
#pragma unroll
  for (int k = 0; k < NW; ++k) cz[k] = cf[(long long)k * Ca];
  T gx[NF], gy[NF], gg[G > 0 ? G : 1], go[NF];
  T* gcf = nullptr;
  if (BWD) {
    const T* gU = a.gU + e * (long long)NF * Ca + ca;
#pragma unroll
    for (int r = 0; r < NF; ++r) { go[r] = gU[(long long)r * Ca]; gx[r] = go[r]; gy[r] = T(0); }
#pragma unroll
    for (int r = 0; r < G; ++r) gg[r] = T(0);
    gcf = a.gcoefZ + e * (long long)a.n_paths * N * Ca + ca;
  }
#pragma unroll
  for (int m = 0; m <= MM; ++m) {
#pragma unroll
    for (int part = 0; part < (m == 0 ? 1 : 2); ++part)
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const int r = (m == 0 ? 0 : N + (m - 1) * 2 * N) + part * N + i;
        if (m == 0 && !GATE_M0) {
          out[r] += act_eval<T>(a.act, x[r]);
          if (BWD) gx[r] += go[r] * act_grad<T>(a.act, x[r]);
        } else {
          const int g = (m - START) * N + i;
          const T ag = act_eval<T>(a.act, gz[g]);
          out[r] += ag * x[r];
          if (BWD) { gx[r] += go[r] * ag; gg[g] += go[r] * x[r] * act_grad<T>(a.act, gz[g]); }
        }
      }
  }
#pragma unroll
  for (int m3 = 0; m3 <= MM; ++m3)
#pragma unroll
    for (int m1 = 0; m1 <= MM; ++m1)
#pragma unroll
      for (int m2 = 0; m2 <= m1; ++m2) {
        const bool sum_mode = (m1 + m2 == m3);
        if (!(sum_mode || m1 - m2 == m3)) continue;
        const int p = mix_path_id(MM, m3, m1, m2);
        const T sc = a.p_scale[p];
        const int x_re = (m1 == 0 ? 0 : N + (m1 - 1) * 2 * N), y_re = (m2 == 0 ? 0 : N + (m2 - 1) * 2 * N),
                  o_re = (m3 == 0 ? 0 : N + (m3 - 1) * 2 * N);
#pragma unroll
        for (int i = 0; i < N; ++i) {
          const T czv = cz[p * N + i];
          const T w = act_eval<T>(a.act, czv) * sc;
          const T xr = x[x_re + i], xi = m1 ? x[x_re + (m1 ? N : 0) + i] : T(0);
          const T yr = y[y_re + i], yi = m2 ? y[y_re + (m2 ? N : 0) + i] : T(0);
          T zr, zi;
          if (sum_mode) { zr = xr * yr - xi * yi; zi = xr * yi + xi * yr; }
          else { zr = xr * yr + xi * yi; zi = xi * yr - xr * yi; }
          out[o_re + i] += w * zr;
          if (m3) out[o_re + (m3 ? N : 0) + i] += w * zi;
          if (BWD) {
            const T gr = go[o_re + i], gi = m3 ? go[o_re + (m3 ? N : 0) + i] : T(0);
            gcf[(long long)(p * N + i) * Ca] = (gr * zr + gi * zi) * sc * act_grad<T>(a.act, czv);
            const T ar = w * gr, ai = w * gi;
            if (sum_mode) {
              gx[x_re + i] += ar * yr + ai * yi;
              if (m1) gx[x_re + (m1 ? N : 0) + i] += -ar * yi + ai * yr;
              gy[y_re + i] += ar * xr + ai * xi;
              if (m2) gy[y_re + (m2 ? N : 0) + i] += -ar * xi + ai * xr;
            } else {
              gx[x_re + i] += ar * yr - ai * yi;
              if (m1) gx[x_re + (m1 ? N : 0) + i] += ar * yi + ai * yr;
              gy[y_re + i] += ar * xr + ai * xi;
              if (m2) gy[y_re + (m2 ? N : 0) + i] += ar * xi - ai * xr;
            }
          }
        }
      }
  if (!BWD) {
    T* U = a.U + e * (long long)NF * Ca + ca;
#pragma unroll
    for (int r = 0; r < NF; ++r) U[(long long)r * Ca] = out[r];
  } else {
    T* gup = a.gup + e * (long long)(G + NF) * Ca + ca;
    T* gglu = a.gglu + e * (long long)NF * Ca + ca;
#pragma unroll
    for (int r = 0; r < G; ++r) gup[(long long)r * Ca] = gg[r];
#pragma unroll
    for (int r = 0; r < NF; ++r) { gup[(long long)(G + r) * Ca] = gx[r]; gglu[(long long)r * Ca] = gy[r]; }
  }
}
template <typename T, bool BWD>
bool launch_mix_static(const TeceArgs<T>& a, cudaStream_t s) {
  const unsigned grid = (unsigned)((a.E * a.Ca + 63) / 64);
#define MIXCASE(N_, MM_)                                                                                        \
  if (a.L + 1 == N_ && a.mmax == MM_) {                                                                         \
    if (a.gate_m0) tece_mix_t_kernel<T, N_, MM_, true, BWD><<<grid, 64, 0, s>>>(a);                              \
    else tece_mix_t_kernel<T, N_, MM_, false, BWD><<<grid, 64, 0, s>>>(a);                                       \
    return true;                                                                                                \
  }
  MIXCASE(3, 1) MIXCASE(3, 2) MIXCASE(4, 1) MIXCASE(4, 2)
#undef MIXCASE
  return false;
}

// ---- K6: attention-weighted inverse rotation and sum per target atom --------------------------------------
template <typename T>
__global__ void tece_rotate_out_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)a.n_local * a.C) return;
  const long long i = idx / a.C;
  const int c = (int)(idx - i * a.C), C = a.C, D = (a.L + 1) * (a.L + 1), h = c / (C / a.H);
  T acc[16];
  for (int j = 0; j < D; ++j) acc[j] = T(0);
  for (int e = a.rowptr[i]; e < a.rowptr[i + 1]; ++e) {
    const T al = a.alpha[(long long)e * a.H + h];
    const T* Wg = a.Wg + (long long)e * a.NR * D;
    for (int r = 0; r < a.NR; ++r) {
      const int l = a.row_l[r], dl = 2 * l + 1;
      const T v = al * a.row_scale[r] * a.down[((long long)e * a.NR + r) * C + c];
      for (int j = 0; j < dl; ++j) acc[l * l + j] += Wg[r * D + l * l + j] * v;
    }
  }
  for (int j = 0; j < D; ++j) a.M[(i * D + j) * C + c] = acc[j];
}
// gdown[e][r][c] = alpha scale_r sum_j Wg[e][r][j] gM[target][j][c].  FUSE (channels per head a power of two <= 32, so one
// head is a group of neighbouring lanes): also galpha[e][h] = sum over the head's channels and the rows of down * scale_r * t,
// reduced with shuffles, which saves the separate pass of tece_alpha_bwd_kernel over the same data.
template <typename T, bool FUSE>
__global__ void tece_rotate_out_bwd_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.C) return;
  const long long e = idx / a.C;
  const int c = (int)(idx - e * a.C), C = a.C, D = (a.L + 1) * (a.L + 1), h = c / (C / a.H);
  const T al = a.alpha[e * a.H + h];
  const T* __restrict__ Wg = a.Wg + e * a.NR * D;
  const T* __restrict__ gM = a.gM + (long long)a.e_dst[e] * D * C + c;
  const T* __restrict__ down = a.down;
  T part = T(0);
  for (int r = 0; r < a.NR; ++r) {
    const int l = a.row_l[r], dl = 2 * l + 1;
    T t = T(0);
    for (int j = 0; j < dl; ++j) t += Wg[r * D + l * l + j] * gM[(long long)(l * l + j) * C];
    t *= a.row_scale[r];
    a.gdown[(e * a.NR + r) * C + c] = al * t;
    if (FUSE) part += down[(e * a.NR + r) * C + c] * t;
  }
  if (FUSE) {
    const int Ch = C / a.H;
    for (int o = Ch >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (c % Ch == 0) a.galpha[e * a.H + h] = part;
  }
}
// galpha[e][h] = sum_{c in head} sum_r down[e][r][c] scale_r sum_j Wg[e][r][j] gM[target][j][c]
template <typename T>
__global__ void tece_alpha_bwd_kernel(const TeceArgs<T> a) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= a.E * a.H) return;
  const long long e = idx / a.H;
  const int h = (int)(idx - e * a.H), C = a.C, Ch = C / a.H, D = (a.L + 1) * (a.L + 1);
  const T* Wg = a.Wg + e * a.NR * D;
  T acc = T(0);
  for (int u = 0; u < Ch; ++u) {
    const int c = h * Ch + u;
    const T* gM = a.gM + (long long)a.e_dst[e] * D * C + c;
    for (int r = 0; r < a.NR; ++r) {
      const int l = a.row_l[r], dl = 2 * l + 1;
      T t = T(0);
      for (int j = 0; j < dl; ++j) t += Wg[r * D + l * l + j] * gM[(long long)(l * l + j) * C];
      acc += a.down[(e * a.NR + r) * C + c] * a.row_scale[r] * t;
    }
  }
  a.galpha[idx] = acc;
}
// gWg[e][r][j] = sum_c ( gKs_total x[source][j] + gQt_total x[target][j] + alpha scale_r gM[target][j] down[e][r] )
// One warp per edge: lane k owns the channels k, k + 32, ...; every lane accumulates all block entries of the edge (at most
// 70 for L = 3, mmax = 2), then the warp reduces them.  All loads are contiguous in the channel index.
template <typename T>
__global__ void __launch_bounds__(128) tece_wigner_grad_kernel(const TeceArgs<T> a) {
  const int lane = threadIdx.x & 31;
  const long long e = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (e >= a.E) return;
  const int D = (a.L + 1) * (a.L + 1), C = a.C, Ch = C / a.H;
  constexpr int MAXE = 70;
  T acc[MAXE];
#pragma unroll
  for (int k = 0; k < MAXE; ++k) acc[k] = T(0);
  const T* xs = a.x + (long long)a.e_src[e] * D * C;
  const T* xt = a.x + (long long)a.e_dst[e] * D * C;
  const T* gM = a.gM + (long long)a.e_dst[e] * D * C;
  for (int c = lane; c < C; c += 32) {
    const T al = a.alpha[e * a.H + c / Ch];
    T vs[16], vt[16], vg[16];
    for (int j = 0; j < D; ++j) { vs[j] = xs[(long long)j * C + c]; vt[j] = xt[(long long)j * C + c]; vg[j] = al * gM[(long long)j * C + c]; }
    int k = 0;
    for (int r = 0; r < a.NR; ++r) {
      const int l = a.row_l[r], dl = 2 * l + 1;
      const long long at = (e * a.NR + r) * C + c;
      const T gk = a.gKs[at], gq = a.gQt[at], dn = a.row_scale[r] * a.down[at];
      for (int j = 0; j < dl; ++j, ++k) acc[k] += gk * vs[l * l + j] + gq * vt[l * l + j] + dn * vg[l * l + j];
    }
  }
  T* out = a.gWg + e * a.NR * D;
  int k = 0;
  for (int r = 0; r < a.NR; ++r) {
    const int l = a.row_l[r], dl = 2 * l + 1;
    for (int j = 0; j < dl; ++j, ++k) {
      T v = acc[k];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) out[r * D + l * l + j] = v;
    }
  }
}

}  // namespace

#define TECE_LAUNCH(KERNEL, COUNT, ...)                                                   \
  do {                                                                                    \
    const long long cnt__ = (COUNT);                                                      \
    if (cnt__ > 0) KERNEL<<<(unsigned)((cnt__ + 127) / 128), 128, 0, s>>>(__VA_ARGS__);    \
    if (cudaGetLastError() != cudaSuccess) return cudaGetLastError();                      \
  } while (0)

template <typename T>
cudaError_t launch_tece(const TeceArgs<T>& a, int stage, cudaStream_t s) {
  const int D = (a.L + 1) * (a.L + 1);
  if (a.L > 3 || a.mmax > 2 || a.NR > 16 || a.NC > 9 || a.H > 16 || a.G > 12 || a.n_paths * (a.L + 1) > 28 || a.C % a.H != 0)
    return cudaErrorInvalidValue;
  cudaError_t err = cudaSuccess;
  // nothing to launch: stages over atoms need local atoms, every other stage needs edges (an atom without edges still gets
  // its zero message from TECE_ROTATE_OUT)
  const bool per_atom = stage == TECE_SOFTMAX || stage == TECE_ROTATE_OUT || stage == TECE_SOFTMAX_BWD || stage == TECE_TARGET_SUM;
  if (per_atom ? a.n_local <= 0 : a.E <= 0) return cudaSuccess;
  const int ch = a.C / a.H;
  const bool fuse_alpha = a.C % 32 == 0 && ch <= 32 && (ch & (ch - 1)) == 0;
  switch (stage) {
    case TECE_WIGNER: tece_wigner_kernel<T><<<(unsigned)((a.E + 63) / 64), 64, 0, s>>>(a); break;
    case TECE_ROTATE_IN:
      if (!TECE_LM_DISPATCH(tece_rotate_in_t_kernel, (unsigned)((a.E * a.C + 127) / 128), 128))
        tece_rotate_in_kernel<T><<<(unsigned)((a.E * a.C + 127) / 128), 128, 0, s>>>(a);
      break;
    case TECE_LOGIT:
      if (fuse_alpha) {
        tece_proj_kernel<T><<<(unsigned)((a.E + 127) / 128), 128, 0, s>>>(a);
        tece_logit_lane_kernel<T, false><<<(unsigned)((a.E * a.C + 127) / 128), 128, 0, s>>>(a);
      } else {
        tece_logit_kernel<T><<<(unsigned)((a.E * a.H + 127) / 128), 128, 0, s>>>(a);
      }
      break;
    case TECE_SOFTMAX: tece_softmax_kernel<T><<<(unsigned)(((long long)a.n_local * a.H + 127) / 128), 128, 0, s>>>(a); break;
    case TECE_MIX:
      if (!launch_mix_static<T, false>(a, s)) tece_mix_kernel<T, false><<<(unsigned)((a.E * a.Ca + 63) / 64), 64, 0, s>>>(a);
      break;
    case TECE_ROTATE_OUT:
      if (!TECE_LM_DISPATCH(tece_rotate_out_t_kernel, (unsigned)(((long long)a.n_local * a.C + 127) / 128), 128))
        tece_rotate_out_kernel<T><<<(unsigned)(((long long)a.n_local * a.C + 127) / 128), 128, 0, s>>>(a);
      break;
    case TECE_ROTATE_OUT_BWD:
      if (fuse_alpha) tece_rotate_out_bwd_kernel<T, true><<<(unsigned)((a.E * a.C + 127) / 128), 128, 0, s>>>(a);
      else tece_rotate_out_bwd_kernel<T, false><<<(unsigned)((a.E * a.C + 127) / 128), 128, 0, s>>>(a);
      break;
    case TECE_ALPHA_BWD:  // already done by the fused kernel above when the head width allows it
      if (!fuse_alpha) tece_alpha_bwd_kernel<T><<<(unsigned)((a.E * a.H + 127) / 128), 128, 0, s>>>(a);
      break;
    case TECE_SOFTMAX_BWD: tece_softmax_bwd_kernel<T><<<(unsigned)(((long long)a.n_local * a.H + 127) / 128), 128, 0, s>>>(a); break;
    case TECE_LOGIT_BWD:
      if (fuse_alpha) tece_logit_lane_kernel<T, true><<<(unsigned)((a.E * a.C + 127) / 128), 128, 0, s>>>(a);
      else tece_logit_bwd_kernel<T><<<(unsigned)((a.E * a.H + 127) / 128), 128, 0, s>>>(a);
      break;
    case TECE_EDGE_SCALAR_BWD: tece_edge_scalar_bwd_kernel<T><<<(unsigned)((a.E + 127) / 128), 128, 0, s>>>(a); break;
    case TECE_MIX_BWD:
      if (!launch_mix_static<T, true>(a, s)) tece_mix_kernel<T, true><<<(unsigned)((a.E * a.Ca + 63) / 64), 64, 0, s>>>(a);
      break;
    case TECE_ROTATE_IN_BWD:
      if (!TECE_LM_DISPATCH(tece_rotate_in_bwd_t_kernel, (unsigned)((a.E * a.C + 127) / 128), 128))
        tece_rotate_in_bwd_kernel<T><<<(unsigned)((a.E * a.C + 127) / 128), 128, 0, s>>>(a);
      break;
    case TECE_TARGET_SUM: tece_target_sum_kernel<T><<<(unsigned)(((long long)a.n_local * D * a.C + 127) / 128), 128, 0, s>>>(a); break;
    case TECE_WIGNER_GRAD:
      if (!TECE_LM_DISPATCH(tece_wigner_grad_t_kernel, (unsigned)((a.E + 3) / 4), 128))
        tece_wigner_grad_kernel<T><<<(unsigned)((a.E + 3) / 4), 128, 0, s>>>(a);
      break;
    case TECE_WIGNER_BWD: tece_wigner_bwd_kernel<T><<<(unsigned)((a.E + 63) / 64), 64, 0, s>>>(a, a.accumulate_gvec); break;
    default: err = cudaErrorInvalidValue;
  }
  return err != cudaSuccess ? err : cudaGetLastError();
}

template cudaError_t launch_tece<float>(const TeceArgs<float>&, int, cudaStream_t);
template cudaError_t launch_tece<double>(const TeceArgs<double>&, int, cudaStream_t);

}  // namespace tace
